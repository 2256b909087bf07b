import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden", "reference_vectors.npz")
GOLDEN_LEGACY = os.path.join(ROOT, "tests", "golden", "reference_vectors_legacy.npz")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def golden():
    return np.load(GOLDEN)


@pytest.fixture(scope="session")
def golden_legacy():
    """Legacy flat layout, streams the reference's rans_decomp_triton returned to the stored plane."""
    return np.load(GOLDEN_LEGACY)


@pytest.fixture(scope="session")
def oracle():
    from oracle import build, oracle as O
    build.build_oracle()
    return O


def make_weight(K, N, seed, std=0.02):
    """Seeded bf16 weight generated on the CPU so every machine sees the same bits."""
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(K, N, generator=g) * std).to(torch.bfloat16)


def bits(t):
    return t.contiguous().view(torch.uint16).cpu().numpy()


def golden_case(golden, i):
    p = f"t{i}_"
    K, N, th, tw, seed = (int(v) for v in golden[p + "geom"])
    d = {k[len(p):]: golden[k] for k in golden.files if k.startswith(p)}
    d.update(K=K, N=N, th=th, tw=tw, seed=seed)
    return d
