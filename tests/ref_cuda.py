"""ctypes access to the REFERENCE's own block-32 CUDA kernels (test infrastructure).

`make -C oracle refcuda` compiles the reference's tq_quant_kernel.cu and tq_dequant_kernel.cu for
sm_100a from the reference checkout, where they lie, into oracle/_ref/libtqrefcuda.so (IEEE arithmetic)
and oracle/_ref/libtqrefcuda_fastmath.so (the --use_fast_math of the reference's build.rs:21), with
their extern "C" launchers renamed tqref_*.  Only the quantize and dequantize launchers are ever called:
tq_quant_maxnorm_batch (tq_quant_kernel.cu:416-439) and tq_dequant_batch (tq_dequant_kernel.cu:104-125).
The reference's attention kernel is not built.

Used by the GPU parity tests and by tests/golden/make_golden.py; never by the library.
"""
import ctypes
import os

import numpy as np

import oracle_lib as o

REF_DIR = os.path.join(o.ORACLE_DIR, "_ref")
VARIANTS = {"ieee": "libtqrefcuda.so", "fastmath": "libtqrefcuda_fastmath.so"}


def available():
    return all(os.path.exists(os.path.join(REF_DIR, f)) for f in VARIANTS.values())


_libs = {}


def _lib(variant):
    if variant not in _libs:
        r = ctypes.CDLL(os.path.join(REF_DIR, VARIANTS[variant]))
        vp, i32, f32 = ctypes.c_void_p, ctypes.c_int32, ctypes.c_float
        r.tqref_quant_maxnorm_batch.argtypes = [vp, vp, vp, vp, i32, i32, i32, i32, i32, f32, f32, vp]
        r.tqref_quant_maxnorm_batch.restype = None
        r.tqref_dequant_batch.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32, i32, vp]
        r.tqref_dequant_batch.restype = None
        _libs[variant] = r
    return _libs[variant]


def quant_maxnorm(rotated, bits, variant="ieee", scale_sign=-1.0):
    """The reference's MaxNorm quantize-and-pack kernel on already rotated 32-blocks [n_blocks, 32] f32.
    Arguments as src/cache/cuda/quantize.rs:114-127 passes them for an all-outlier (PQO) cache: the
    `bits`-wide codebook's boundaries, its outermost centroid, scale sign -1.  Returns (packed
    [n_blocks, 4 * bits] u8, scales [n_blocks] u16)."""
    import torch
    c, b = o.block_codebook(bits, 0)
    rot = torch.from_numpy(np.ascontiguousarray(rotated, np.float32).reshape(-1, 32)).cuda()
    bd = torch.from_numpy(b).cuda()
    n = rot.shape[0]
    bpb = 4 * bits
    packed = torch.zeros((n, bpb), dtype=torch.uint8, device="cuda")
    scales = torch.zeros(n, dtype=torch.int16, device="cuda")
    torch.cuda.synchronize()
    _lib(variant).tqref_quant_maxnorm_batch(rot.data_ptr(), bd.data_ptr(), packed.data_ptr(), scales.data_ptr(), n, 32, bits,
                                            len(b), bpb, float(c[-1]), float(scale_sign), None)
    torch.cuda.synchronize()
    return packed.cpu().numpy(), scales.cpu().numpy().view(np.uint16)


def dequant(packed, scales, bits, variant="ieee"):
    """The reference's dequantize kernel with the `bits`-wide MaxNorm codebook and the sign pattern the crate
    uploads: row 0 of rotation_fwd times sqrt(32) (src/cache/pqo.rs:133-137), i.e. the +-1 pattern of
    src/cache/precomputed/rotation.rs:16-20 times (1/sqrt(32)) * sqrt(32) = 0.99999994 in f32.
    Returns [n_blocks, 32] f32."""
    import torch
    c, _ = o.block_codebook(bits, 0)
    pk = torch.from_numpy(np.ascontiguousarray(packed, np.uint8).reshape(-1, 4 * bits)).cuda()
    sc = torch.from_numpy(np.ascontiguousarray(scales, np.uint16).reshape(-1).view(np.int16)).cuda()
    cd = torch.from_numpy(c).cuda()
    sg = torch.from_numpy(uploaded_sign_pattern()).cuda()
    n = pk.shape[0]
    out = torch.zeros((n, 32), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    _lib(variant).tqref_dequant_batch(pk.data_ptr(), sc.data_ptr(), cd.data_ptr(), sg.data_ptr(), out.data_ptr(), n, 32, bits,
                                      4 * bits, None)
    torch.cuda.synchronize()
    return out.cpu().numpy()


def uploaded_sign_pattern():
    return ((o.block_signs() * (np.float32(1) / np.sqrt(np.float32(32)))) * np.sqrt(np.float32(32))).astype(np.float32)


def synthetic_kv(style, n, seed, head_dim=128):
    """Stand-ins for the K/V statistics the benchmark configurations name: "outlier" = N(0,1) with 2 % of the
    channels (3 of 128, fixed per seed) multiplied by 8; "lognormal" = N(0,1) times per-channel exp(N(0, 0.5)).
    Values are rounded through bf16, the dtype the configurations store K/V in."""
    import torch
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((n, head_dim)).astype(np.float32)
    if style == "outlier":
        x[:, rng.choice(head_dim, 3, replace=False)] *= 8.0
    elif style == "lognormal":
        x *= np.exp(rng.normal(0.0, 0.5, head_dim)).astype(np.float32)
    else:
        raise ValueError(style)
    return torch.from_numpy(x).to(torch.bfloat16).float().numpy()
