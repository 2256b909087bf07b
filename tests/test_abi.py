"""CPU: the C-ABI library loads, exports every symbol the header declares, and its host-only
entry points agree with the oracle.  No kernel is launched here."""
import ctypes as C
import os
import re
import subprocess

import numpy as np
import pytest

from conftest import ROOT

HEADER = os.path.join(ROOT, "include", "comp_inference_b200.h")


def declared_symbols():
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(ci_[a-z0-9_]+)\s*\(", src)))


@pytest.fixture(scope="module")
def lib():
    from comp_inference_b200.csrc import build
    build.build()
    from comp_inference_b200 import _lib
    return _lib.load()


def test_header_symbols_are_exported_and_bound(lib):
    from comp_inference_b200 import _lib
    names = declared_symbols()
    assert len(names) >= 20
    out = subprocess.run(["nm", "-D", "--defined-only", _lib.LIB_PATH], capture_output=True, text=True, check=True).stdout
    exported = set(re.findall(r"\sT\s+(ci_[a-z0-9_]+)", out))
    for n in names:
        assert n in exported, f"{n} declared in the header but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"
    assert set(_lib.SIGNATURES) <= set(names)
    assert lib.ci_abi_version() == 1


def test_host_tables_match_oracle(lib, oracle, golden):
    for i in range(int(golden["n_lut"][0])):
        f, c = golden[f"lut{i}_freqs"], golden[f"lut{i}_cdf"]
        t = np.empty(256, np.uint32)
        s = np.empty(4096, np.uint8)
        assert lib.ci_build_tables(f.ctypes.data, c.ctypes.data, t.ctypes.data, s.ctypes.data) == 0
        to, so = oracle.build_tables(f, c)
        assert np.array_equal(t, to) and np.array_equal(s, so)


def test_normalize_freqs_matches_reference_vectors(lib, golden):
    for i in range(int(golden["n_lut"][0])):
        hist = np.bincount(golden[f"lut{i}_plane"], minlength=256).astype(np.uint64)
        f = np.empty(256, np.uint16)
        c = np.empty(256, np.uint16)
        assert lib.ci_normalize_freqs(hist.ctypes.data, f.ctypes.data, c.ctypes.data) == 0
        assert np.array_equal(f, golden[f"lut{i}_freqs"]) and np.array_equal(c, golden[f"lut{i}_cdf"])


def test_errors_are_reported_not_swallowed(lib):
    f = np.ones(256, np.uint16)                       # sums to 256, not 4096
    c = np.arange(256, dtype=np.uint16)
    t = np.empty(256, np.uint32)
    s = np.empty(4096, np.uint8)
    assert lib.ci_build_tables(f.ctypes.data, c.ctypes.data, t.ctypes.data, s.ctypes.data) == -1
    assert b"4096" in lib.ci_last_error()
    hist = np.zeros(256, np.uint64)
    assert lib.ci_normalize_freqs(hist.ctypes.data, f.ctypes.data, c.ctypes.data) == -1
    assert lib.ci_decode_plane(None, None, None) == -1


def test_product_package_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "comp_inference_b200")
    for dp, _, files in os.walk(pkg):
        for fn in files:
            if fn.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dp, fn)).read()
                assert "oracle" not in text, f"{fn} mentions the oracle"


def test_missing_library_fails_loudly(monkeypatch):
    from comp_inference_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", "/nonexistent/libci_b200.so")
    with pytest.raises(RuntimeError, match="no other backend"):
        _lib.load()
