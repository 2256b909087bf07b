"""Builds the CPU oracle (and, where the reference sources are present, the
reference's own extension) -- test infrastructure, never part of the product.

    python oracle/build.py            # librans_oracle.so (+ _ref/ccore*.so if possible)
    python oracle/build.py --no-ref   # oracle only

``librans_oracle.so`` is the plain-C restatement in rans_oracle.c.

``_ref/ccore*.so`` is the reference's unmodified extension, compiled straight
from its two translation units where they lie (src/python_bindings.cpp,
src/cuda/rans_ops.cu) with a direct nvcc command; nothing is copied into this
repository.  It needs a GPU to run (its encoder is CUDA only), so it is used on
a GPU machine to cross-check compressed bytes against this repository's
encoders.  The output directory is not tracked by git.
"""
import argparse
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "librans_oracle.so")
REF_DIR = os.path.join(HERE, "_ref")


def _stale(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def build_oracle(force=False):
    src = os.path.join(HERE, "rans_oracle.c")
    if force or _stale(ORACLE_SO, [src]):
        cmd = ["gcc", "-O3", "-march=x86-64-v2", "-fPIC", "-shared", "-pthread", "-std=c11",
               "-fno-fast-math", "-ffp-contract=off", src, "-o", ORACLE_SO, "-lm"]
        subprocess.check_call(cmd)
    return ORACLE_SO


def default_ref_root():
    """The reference checkout is looked for beside this repository (override: CI_REFERENCE_ROOT)."""
    repo = os.path.dirname(HERE)
    return os.environ.get("CI_REFERENCE_ROOT", os.path.join(os.path.dirname(repo), "reference"))


def ref_so_path():
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    return os.path.join(REF_DIR, "ccore" + suffix)


def build_reference(ref_root, force=False):
    """Compiles the reference extension if its sources exist; returns the path or None."""
    binding = os.path.join(ref_root, "src", "python_bindings.cpp")
    ops = os.path.join(ref_root, "src", "cuda", "rans_ops.cu")
    if not (os.path.exists(binding) and os.path.exists(ops)):
        return None
    out = ref_so_path()
    if not force and not _stale(out, [binding, ops]):
        return out
    import torch
    from torch.utils import cpp_extension as ce
    os.makedirs(REF_DIR, exist_ok=True)
    inc = []
    for p in ce.include_paths("cuda"):
        inc += ["-I", p]
    inc += ["-I", sysconfig.get_paths()["include"], "-I", os.path.join(ref_root, "src"),
            "-I", os.path.join(ref_root, "src", "cpp"), "-I", os.path.join(ref_root, "src", "cuda")]
    try:
        import pybind11
        inc += ["-I", pybind11.get_include()]
    except ImportError:
        pass
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    common = ["-O2", "-std=c++17", "--use_fast_math", "-Xcompiler", "-fPIC",
              "-gencode", "arch=compute_100,code=sm_100",
              "-DTORCH_EXTENSION_NAME=ccore", "-DTORCH_API_INCLUDE_EXTENSION_H",
              f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
              "-D__CUDA_NO_HALF_OPERATORS__", "-D__CUDA_NO_HALF_CONVERSIONS__",
              "-D__CUDA_NO_BFLOAT16_CONVERSIONS__", "-D__CUDA_NO_HALF2_OPERATORS__",
              "--expt-relaxed-constexpr", "-w"]
    objs = []
    for i, src in enumerate([binding, ops]):
        obj = os.path.join(REF_DIR, f"ref_{i}.o")
        extra = ["-x", "cu"] if src.endswith(".cpp") else []
        if _stale(obj, [src]):
            subprocess.check_call(["nvcc", *common, *inc, *extra, "-c", src, "-o", obj])
        objs.append(obj)
    subprocess.check_call(["nvcc", "-shared", *objs, "-o", out, "-L", torch_lib,
                           "-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python", "-lc10_cuda", "-ltorch_cuda",
                           "-Xlinker", f"-rpath={torch_lib}"])
    for o in objs:
        os.remove(o)
    return out


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--no-ref", action="store_true")
    ap.add_argument("--ref-root", default=default_ref_root())
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    print(build_oracle(a.force))
    if not a.no_ref:
        try:
            print(build_reference(a.ref_root, a.force))
        except subprocess.CalledProcessError as e:
            print("reference extension did not build:", e, file=sys.stderr)
