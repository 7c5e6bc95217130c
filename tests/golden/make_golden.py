#!/usr/bin/env python3
"""Generates the golden fixtures in this directory.

Three sources:
  * ref_primitives.npz -- outputs of the REFERENCE's own code: its host-compilable header
    src/cache/cuda/kernels/tq_common.h, compiled by `make -C oracle ref` into
    oracle/_ref/libtqref.so (bit packing for 2/3/4 bits, the parity sign pattern, the
    SplitMix Rademacher hash).  Needs the reference checkout, so it only runs where that
    is mounted; the fixture is what travels.
  * oracle_cases.npz -- outputs of the CPU oracle (oracle/liboracle.so) on small seeded
    inputs, so the CUDA path can be compared against committed numbers and so that an
    accidental change of the oracle shows up as a diff.
  * ref_cuda_block.npz -- outputs of the REFERENCE's own block-32 CUDA kernels
    (tq_quant_maxnorm_kernel, tq_dequant_kernel; compiled from the reference checkout by
    `make -C oracle refcuda`, see tests/ref_cuda.py) on small seeded inputs.  Needs a GPU and the
    compiled kernels: `python tests/golden/make_golden.py --ref-cuda <output.npz>`; the file is then
    copied here.  It pins the oracle's Format-B quantize / dequantize on machines without a GPU.

Usage: python tests/golden/make_golden.py [--ref-cuda <output.npz>]
"""
import ctypes
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import oracle_lib as o  # noqa: E402

P = o.P


def ref_primitives():
    so = os.path.join(o.ORACLE_DIR, "_ref", "libtqref.so")
    r = ctypes.CDLL(so)
    r.ref_sign.restype = ctypes.c_float
    r.ref_rademacher_sign.restype = ctypes.c_float
    r.ref_mix_seed.restype = ctypes.c_uint64
    rng = np.random.default_rng(20251125)
    out = {}
    for bits in (2, 3, 4):
        codes = rng.integers(0, 1 << bits, size=(8, 128), dtype=np.uint8)
        nbytes = 128 * bits // 8
        packed = np.zeros((8, nbytes), np.uint8)
        for i in range(8):
            r.ref_pack(bits, P(codes[i]), 128, P(packed[i]), nbytes)
            for t in range(128):
                assert r.ref_unpack(bits, P(packed[i]), t) == codes[i, t]
        out[f"codes_{bits}"] = codes
        out[f"packed_{bits}"] = packed
    for seed in (0, 1, 42, 12345):
        out[f"sign_{seed}"] = np.array([r.ref_sign(ctypes.c_uint64(seed), i) for i in range(256)], np.float32)
    for seed in (42, 12345):
        m = np.zeros((128, 128), np.int8)
        for row in range(128):
            for col in range(128):
                m[row, col] = int(r.ref_rademacher_sign(ctypes.c_uint64(seed), row, col))
        out[f"rademacher_{seed}"] = m
        out[f"mix_seed_{seed}"] = np.array([r.ref_mix_seed(ctypes.c_uint64(seed), row) for row in range(8)], np.uint64)
    np.savez_compressed(os.path.join(HERE, "ref_primitives.npz"), **out)


def oracle_cases():
    out = {}
    rng = np.random.default_rng(42)
    x = rng.standard_normal((64, 128)).astype(np.float32)
    x[5] = 0.0            # zero vector: scale 0, all codes at the zero-boundary bin
    x[6] *= 1e-12         # below MIN_NORM
    x[7] *= 300.0
    out["whole_x"] = x
    for bits in (2, 3, 4):
        p, s = o.quantize_batch(bits, 128, 42, x)
        out[f"whole_packed_{bits}"], out[f"whole_scales_{bits}"] = p, s
        out[f"whole_deq_{bits}"] = o.dequantize_batch(bits, 128, 42, p, s)
    for dim in (32, 64, 256):
        xd = rng.standard_normal((8, dim)).astype(np.float32)
        p, s = o.quantize_batch(3, dim, 7, xd)
        out[f"whole_x_d{dim}"], out[f"whole_packed_d{dim}"], out[f"whole_scales_d{dim}"] = xd, p, s
    for bits in (3, 4):
        p, s, sg, rn = o.qjl_quantize_batch(bits, 128, 42, 42, x[:16])
        out[f"qjl_packed_{bits}"], out[f"qjl_scales_{bits}"], out[f"qjl_signs_{bits}"], out[f"qjl_rnorms_{bits}"] = p, s, sg, rn
    q = (rng.standard_normal(128) / np.sqrt(128)).astype(np.float32)
    out["q"] = q
    out["rq_42"] = o.query_projections(q, 128, 42)
    p, s, sg, rn = o.qjl_quantize_batch(3, 128, 42, 42, x[:16])
    out["scores_3"] = o.attention_scores(3, 128, 42, 42, q, p, s, sg, rn)
    w = rng.random(16).astype(np.float32)
    out["w"] = w
    out["weighted_3"] = o.weighted_values(3, 128, 42, w, p, s)
    # block-32 format
    xb = rng.standard_normal((32, 128)).astype(np.float32)
    xb[:, [3, 40, 77]] *= 8.0
    xb[9] = 0.0
    out["block_x"] = xb
    for bits, nm, ob, tag in ((3, 0, -1, "pqo3"), (4, 0, -1, "pqo4"), (3, 1, -1, "pqo3_l2"), (3, 0, 0, "pq3"), (4, 0, 2, "mix4")):
        p, s = o.block_quantize(bits, 128, nm, ob, xb)
        out[f"block_packed_{tag}"], out[f"block_scales_{tag}"] = p, s
        out[f"block_deq_{tag}"] = o.block_dequantize(bits, 128, nm, ob, p, s)
    # decode attention: 4 query heads on 2 KV heads, 37 tokens, PQO3 and PQO4
    hq, hkv, L = 4, 2, 37
    k = rng.standard_normal((hkv * L, 128)).astype(np.float32)
    v = rng.standard_normal((hkv * L, 128)).astype(np.float32)
    qa = (rng.standard_normal((hq, 128)) / np.sqrt(128)).astype(np.float32)
    out["att_k"], out["att_v"], out["att_q"] = k, v, qa
    for bits, tag in ((3, "pqo3"), (4, "pqo4")):
        kp, ks = o.block_quantize(bits, 128, 0, -1, k)
        vp, vs = o.block_quantize(bits, 128, 0, -1, v)
        res = o.block_attention(bits, 128, 0, -1, qa, kp.reshape(hkv, L, -1), ks.reshape(hkv, L, -1), vp.reshape(hkv, L, -1),
                                vs.reshape(hkv, L, -1), L, 1.0 / np.sqrt(128))
        out[f"att_out_{tag}"] = res
    np.savez_compressed(os.path.join(HERE, "oracle_cases.npz"), **out)


def ref_cuda_block(path):
    """Runs the reference's quantize and dequantize kernels (IEEE build and the --use_fast_math build the
    reference ships) on 128 vectors of each synthetic K/V style; the rotated input is the oracle's."""
    import ref_cuda
    out = {}
    for style in ref_cuda_styles():
        x = ref_cuda.synthetic_kv(style, 128, 31)
        rot = o.block_rotate(x)
        out[f"x_{style}"] = x
        out[f"rot_{style}"] = rot
        for bits in (3, 4):
            for variant in ("ieee", "fastmath"):
                p, s = ref_cuda.quant_maxnorm(rot, bits, variant)
                out[f"packed_{style}_{bits}_{variant}"], out[f"scales_{style}_{bits}_{variant}"] = p, s
            p, s = out[f"packed_{style}_{bits}_ieee"], out[f"scales_{style}_{bits}_ieee"]
            for variant in ("ieee", "fastmath"):
                out[f"deq_{style}_{bits}_{variant}"] = ref_cuda.dequant(p, s, bits, variant)
    np.savez_compressed(path, **out)


def ref_cuda_styles():
    return ("outlier", "lognormal")


if __name__ == "__main__":
    if len(sys.argv) == 3 and sys.argv[1] == "--ref-cuda":
        ref_cuda_block(sys.argv[2])
        sys.exit(0)
    if os.path.exists(os.path.join(o.ORACLE_DIR, "_ref", "libtqref.so")):
        ref_primitives()
    else:
        print("oracle/_ref/libtqref.so missing (no reference checkout): ref_primitives.npz left as committed")
    oracle_cases()
