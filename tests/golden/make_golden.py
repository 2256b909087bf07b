"""Generates the committed golden fixtures by running the REFERENCE's own code.

Run once, in a container that has the reference checkout (it is not needed, and
not read, when the tests run):

    TRITON_INTERPRET=1 python tests/golden/make_golden.py --ref-root <reference checkout>

What comes from the reference itself (imported by file path, unmodified):
  * get_rans_lut, extract_exp_and_mantissa, interleave_mantissas,
    uninterleave_mantissas       (comp_inference/comp_inference.py)
  * rans_decomp_triton_tiled     (comp_inference/rans_triton.py), Triton interpreter, CPU tensors
  * fused_rans_embedding_triton  (comp_inference/embedding_triton.py), same
  * rans_decomp_triton           (comp_inference/rans_triton.py), the legacy flat layout in the stream order
                                 of the reference's legacy encoder; written to reference_vectors_legacy.npz
                                 (``--part legacy``)

The reference's encoder is CUDA only and cannot run without a GPU, so the
compressed streams stored here are produced by the CPU oracle; what pins them is
that the reference's decoder and embedding kernel, fed those bytes, return the
original exponent plane / the original rows bit for bit (asserted below before
anything is written).
"""
import argparse
import importlib.util
import os
import sys
import types

os.environ.setdefault("TRITON_INTERPRET", "1")

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import oracle as O  # noqa: E402


def load_reference(ref_root):
    pkg_dir = os.path.join(ref_root, "comp_inference")
    pkg = types.ModuleType("comp_inference")
    pkg.__path__ = [pkg_dir]
    sys.modules["comp_inference"] = pkg
    sys.modules["comp_inference.ccore"] = types.ModuleType("comp_inference.ccore")  # CUDA-only extension: stubbed
    pkg.ccore = sys.modules["comp_inference.ccore"]
    mods = {}
    for name in ("rans_triton", "embedding_triton", "comp_inference"):
        spec = importlib.util.spec_from_file_location(f"comp_inference.{name}", os.path.join(pkg_dir, name + ".py"))
        m = importlib.util.module_from_spec(spec)
        sys.modules[f"comp_inference.{name}"] = m
        spec.loader.exec_module(m)
        mods[name] = m
    return mods


CASES = [
    # K, N, tile_h, tile_w, seed, std        what it exercises
    (96, 64, 64, 32, 11, 0.02),             # partial last K tile with an empty bottom-half stream
    (64, 32, 32, 32, 12, 0.02),             # exact tiles
    (80, 48, 32, 16, 13, 0.02),             # tile width 16, partial K tile (16 of 32 rows)
    (128, 64, 128, 64, 14, 1.0),            # tile width 64, wide exponent spread
    (48, 40, 16, 32, 15, 0.02),             # partial last N tile (columns beyond N)
    (40, 32, 16, 32, 16, 0.0),              # all-zero weights: a single exponent symbol
]

LUT_CASES = 8

LEGACY_CASES = [
    # rows, cols, seed, std                  what it exercises
    (1100, 24, 21, 0.02),                   # three segments, the last of 76 rows
    (512, 40, 22, 0.02),                    # exactly one segment
    (37, 130, 23, 1.0),                     # one short segment, more streams than one program of 128
    (600, 8, 24, 0.0),                      # a single symbol: streams without bytes
]


def legacy_part(ref):
    """The legacy flat layout: oracle-encoded streams that the reference's rans_decomp_triton returns to the
    original plane bit for bit."""
    rt, ci = ref["rans_triton"], ref["comp_inference"]
    out = {}
    for i, (rows, cols, seed, std) in enumerate(LEGACY_CASES):
        g = torch.Generator().manual_seed(seed)
        W = (torch.randn(rows, cols, generator=g) * std).to(torch.bfloat16)
        e_ref, _ = ci.extract_exp_and_mantissa(W)
        f_ref, c_ref = ci.get_rans_lut(e_ref)
        stream, states, sizes = O.encode_legacy_segments(e_ref.numpy(), f_ref.numpy(), c_ref.numpy())
        tables, slot_map = O.build_tables(f_ref.numpy().astype(np.uint16), c_ref.numpy().astype(np.uint16))
        st = torch.from_numpy(stream if stream.size else np.zeros(1, np.uint8))
        plane_ref = rt.rans_decomp_triton(
            st, torch.from_numpy(states.view(np.int32).copy()),
            torch.from_numpy(tables.view(np.int32).copy()), torch.from_numpy(slot_map.copy()),
            torch.from_numpy(sizes.view(np.int32).copy()), (rows, cols))
        assert torch.equal(plane_ref, e_ref), f"reference legacy decoder disagrees with the input plane, case {i}"
        p = f"l{i}_"
        out[p + "geom"] = np.array([rows, cols, seed], np.int64)
        out[p + "exp"] = e_ref.numpy()
        out[p + "freqs"] = f_ref.numpy().astype(np.uint16)
        out[p + "cdf"] = c_ref.numpy().astype(np.uint16)
        out[p + "stream"] = stream
        out[p + "states"] = states
        out[p + "sizes"] = sizes
        out[p + "tables"] = tables
        out[p + "slot_map"] = slot_map
        print(f"legacy case {i}: {rows}x{cols} streams={len(states)} bytes={stream.size} ok")
    out["n_cases"] = np.array([len(LEGACY_CASES)], np.int64)
    np.savez_compressed(os.path.join(HERE, "reference_vectors_legacy.npz"), **out)
    print("wrote", os.path.join(HERE, "reference_vectors_legacy.npz"))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref-root", required=True)
    ap.add_argument("--part", choices=("tiled", "legacy", "all"), default="all")
    a = ap.parse_args()
    ref = load_reference(a.ref_root)
    if a.part in ("legacy", "all"):
        legacy_part(ref)
    if a.part == "legacy":
        return
    rt, et, ci = ref["rans_triton"], ref["embedding_triton"], ref["comp_inference"]

    out = {}
    # ---- frequency tables from the reference's get_rans_lut -----------------
    rng = np.random.default_rng(7)
    for i in range(LUT_CASES):
        n = int(rng.integers(200, 60000))
        kind = i % 4
        if kind == 0:
            plane = np.clip(np.round(rng.normal(118, 1.6, n)), 0, 255).astype(np.uint8)
        elif kind == 1:
            plane = rng.integers(0, 256, n).astype(np.uint8)
        elif kind == 2:
            plane = np.full(n, 121, np.uint8)
            plane[: n // 50] = rng.integers(100, 130, n // 50)
        else:
            plane = (rng.zipf(1.3, n) % 256).astype(np.uint8)
        f, c = ci.get_rans_lut(torch.from_numpy(plane))
        out[f"lut{i}_plane"] = plane
        out[f"lut{i}_freqs"] = f.numpy().astype(np.uint16)
        out[f"lut{i}_cdf"] = c.numpy().astype(np.uint16)
        fo, co = O.rans_lut(plane)
        assert (fo == out[f"lut{i}_freqs"]).all() and (co == out[f"lut{i}_cdf"]).all(), f"LUT case {i}"

    # ---- tiled cases -----------------------------------------------------------
    for i, (K, N, th, tw, seed, std) in enumerate(CASES):
        g = torch.Generator().manual_seed(seed)
        W = (torch.randn(K, N, generator=g) * std).to(torch.bfloat16)
        raw = W.view(torch.uint16).numpy().copy()
        e_ref, m_ref = ci.extract_exp_and_mantissa(W)
        f_ref, c_ref = ci.get_rans_lut(e_ref)
        man_tiled_ref = ci.interleave_mantissas(m_ref.contiguous(), TILE_K=th, TILE_N=tw)
        r = O.encode_tiled(e_ref.numpy(), f_ref.numpy(), c_ref.numpy(), th, tw)
        assert (r.tile_height, r.tile_width) == (th, tw)

        def T(x, dt):
            return torch.from_numpy(np.ascontiguousarray(x).astype(dt))

        plane_ref = rt.rans_decomp_triton_tiled(
            T(r.stream, np.uint8), T(r.states, np.int32), T(r.tables, np.uint32).view(torch.int32),
            T(r.slot_map, np.uint8), (K, N), T(r.tile_offsets, np.int32), T(r.tile_max_lens, np.int32),
            tile_k=th, tile_n=tw)
        assert torch.equal(plane_ref, e_ref), f"reference decoder disagrees with the input plane, case {i}"
        ids = torch.tensor([0, K - 1, K // 2, K // 2 + 1, 1, K, -1, th // 2, max(th // 2 - 1, 0)], dtype=torch.int64)
        emb_ref = et.fused_rans_embedding_triton(
            ids, T(r.stream, np.uint8), T(r.states, np.int32), T(r.tables, np.uint32).view(torch.int32),
            T(r.slot_map, np.uint8), (K, N), T(r.tile_offsets, np.int32), T(r.tile_max_lens, np.int32),
            th, tw, man_tiled_ref)
        want = torch.zeros(len(ids), N, dtype=torch.bfloat16)
        for j, t in enumerate(ids.tolist()):
            if 0 <= t < K:
                want[j] = W[t]
        assert torch.equal(emb_ref.view(torch.uint16), want.view(torch.uint16)), f"reference embedding, case {i}"
        un_ref = ci.uninterleave_mantissas(man_tiled_ref.clone(), K, N, TILE_K=th, TILE_N=tw)
        assert torch.equal(un_ref, m_ref)
        rec_bits = ((m_ref.to(torch.int32) & 0x80) << 8) | (e_ref.to(torch.int32) << 7) | (m_ref.to(torch.int32) & 0x7F)
        assert torch.equal(rec_bits.to(torch.uint16), W.view(torch.uint16))

        p = f"t{i}_"
        out[p + "geom"] = np.array([K, N, th, tw, seed], np.int64)
        out[p + "raw"] = raw
        out[p + "exp"] = e_ref.numpy()
        out[p + "man"] = m_ref.numpy()
        out[p + "freqs"] = f_ref.numpy().astype(np.uint16)
        out[p + "cdf"] = c_ref.numpy().astype(np.uint16)
        out[p + "man_tiled"] = man_tiled_ref.numpy()
        out[p + "stream"] = r.stream
        out[p + "states"] = r.states
        out[p + "sizes"] = r.output_sizes
        out[p + "tables"] = r.tables
        out[p + "slot_map"] = r.slot_map
        out[p + "tile_offsets"] = r.tile_offsets
        out[p + "tile_max_lens"] = r.tile_max_lens
        out[p + "ref_plane"] = plane_ref.numpy()
        out[p + "emb_ids"] = ids.numpy()
        out[p + "ref_emb"] = emb_ref.view(torch.uint16).numpy()
        print(f"case {i}: K={K} N={N} tile={th}x{tw} stream={r.stream_len}B ok")

    out["n_cases"] = np.array([len(CASES)], np.int64)
    out["n_lut"] = np.array([LUT_CASES], np.int64)
    np.savez_compressed(os.path.join(HERE, "reference_vectors.npz"), **out)
    print("wrote", os.path.join(HERE, "reference_vectors.npz"))


if __name__ == "__main__":
    main()
