"""Block-32 quantize / dequantize against the REFERENCE's own CUDA kernels, run here.

The reference's tq_quant_maxnorm_kernel (tq_quant_kernel.cu:204-262) and tq_dequant_kernel
(tq_dequant_kernel.cu:38-98) are compiled from the reference checkout (see tests/ref_cuda.py) and fed the
oracle's butterfly-rotated blocks, exactly what the crate hands them (src/cache/cuda/quantize.rs:111-127).
Three parties are compared on the same inputs: the reference's kernels, the CPU oracle, and this library
(both its fused tqb_block_quantize / tqb_block_dequantize and its drop-in tq_quant_maxnorm_batch /
tq_dequant_batch symbols).

Bars: codes and f16 scales bit-exact against the IEEE build of the reference's kernels; against the
--use_fast_math build the reference ships (build.rs:21: approximate division) differing coordinates are
counted and must lie within 1e-6 (relative to the boundary spacing scale of 1) of a decision boundary;
dequantized values within 1e-5 relative.
"""
import ctypes

import numpy as np
import pytest
import torch

import oracle_lib as o
import ref_cuda
import turboquant_b200 as tq
from turboquant_b200._lib import lib

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not ref_cuda.available(), reason="oracle/_ref/libtqrefcuda*.so not built (no reference checkout)")]

N_VEC = 1 << 16          # 262,144 blocks per case
STYLES = ["outlier", "lognormal"]


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def u16(t):
    return t.cpu().numpy().view(np.uint16)


def unpack_codes(bits, packed):
    return o.unpack_indices(bits, packed.reshape(-1), packed.size * 8 // bits)


@pytest.mark.parametrize("style", STYLES)
@pytest.mark.parametrize("bits", [3, 4])
def test_quantize_equals_reference_kernel_ieee(bits, style):
    x = ref_cuda.synthetic_kv(style, N_VEC, 100 + bits)
    rot = o.block_rotate(x)
    ref_packed, ref_scales = ref_cuda.quant_maxnorm(rot, bits, "ieee")
    op, os_ = o.block_quantize(bits, 128, 0, -1, x, nthreads=8)
    assert np.array_equal(ref_packed.reshape(N_VEC, -1), op), "oracle codes differ from the reference's kernel"
    assert np.array_equal(ref_scales.reshape(N_VEC, 4), os_), "oracle scales differ from the reference's kernel"
    # this library, fused rotation + quantize on the un-rotated input
    idx, sc = tq.block_quantize(dev(x), bits)
    assert np.array_equal(idx.cpu().numpy(), ref_packed.reshape(N_VEC, -1))
    assert np.array_equal(u16(sc), ref_scales.reshape(N_VEC, 4))
    # this library's drop-in for the same launcher, same arguments as the reference's
    c, b = o.block_codebook(bits, 0)
    rot_d, b_d = dev(rot), dev(b)
    packed = torch.zeros(rot.shape[0] * 4 * bits, dtype=torch.uint8, device="cuda")
    scales = torch.zeros(rot.shape[0], dtype=torch.int16, device="cuda")
    lib.tq_quant_maxnorm_batch(ctypes.c_void_p(rot_d.data_ptr()), ctypes.c_void_p(b_d.data_ptr()),
                               ctypes.c_void_p(packed.data_ptr()), ctypes.c_void_p(scales.data_ptr()), rot.shape[0], 32, bits,
                               len(b), 4 * bits, float(c[-1]), -1.0, None)
    assert np.array_equal(packed.cpu().numpy(), ref_packed.reshape(-1))
    assert np.array_equal(u16(scales), ref_scales)


@pytest.mark.parametrize("style", STYLES)
@pytest.mark.parametrize("bits", [3, 4])
def test_quantize_vs_reference_kernel_fast_math(bits, style):
    # The build the reference ships divides approximately (amax / outer_centroid and rotated / scale become
    # __fdividef).  Every coordinate whose code differs must sit on a decision boundary to within 1e-6.
    x = ref_cuda.synthetic_kv(style, N_VEC, 100 + bits)
    rot = o.block_rotate(x)
    fm_packed, fm_scales = ref_cuda.quant_maxnorm(rot, bits, "fastmath")
    op, os_ = o.block_quantize(bits, 128, 0, -1, x, nthreads=8)
    ref_codes = unpack_codes(bits, fm_packed).reshape(-1, 32)
    my_codes = unpack_codes(bits, op).reshape(-1, 32)
    diff = ref_codes != my_codes
    n_diff = int(diff.sum())
    scale_diff = int((fm_scales.reshape(-1) != os_.reshape(-1)).sum())
    _, b = o.block_codebook(bits, 0)
    worst = 0.0
    if n_diff:
        blk, pos = np.nonzero(diff)
        assert np.abs(ref_codes[blk, pos].astype(int) - my_codes[blk, pos].astype(int)).max() == 1
        # the scale divided by is the f32 value before its f16 rounding; recompute it as the oracle does
        amax = np.abs(rot[blk]).max(axis=1).astype(np.float32)
        c, _ = o.block_codebook(bits, 0)
        s32 = np.maximum(amax / np.float32(c[-1]), np.float32(1e-10)).astype(np.float32)
        scaled = rot[blk, pos].astype(np.float64) / s32.astype(np.float64)
        worst = float(np.abs(scaled[:, None] - b[None, :].astype(np.float64)).min(axis=1).max())
        assert worst <= 1e-6, f"a differing code lies {worst} from the nearest boundary"
    print(f"\n[fast-math reference, {bits}-bit, {style}] differing codes {n_diff} of {ref_codes.size} "
          f"({n_diff / ref_codes.size:.2e}), worst distance to a boundary {worst:.2e}; differing f16 scales {scale_diff} of {os_.size}")
    assert n_diff <= ref_codes.size * 1e-4
    # a scale can differ by one f16 ulp where the approximate quotient crosses an f16 rounding point
    if scale_diff:
        a = np.array([o.f16_bits_to_f32(int(s)) for s in fm_scales.reshape(-1)[fm_scales.reshape(-1) != os_.reshape(-1)]])
        bb = np.array([o.f16_bits_to_f32(int(s)) for s in os_.reshape(-1)[fm_scales.reshape(-1) != os_.reshape(-1)]])
        assert np.abs(a - bb).max() <= np.abs(bb).max() * 2.0 ** -10
    assert scale_diff <= os_.size * 1e-3


@pytest.mark.parametrize("variant", ["ieee", "fastmath"])
@pytest.mark.parametrize("style", STYLES)
@pytest.mark.parametrize("bits", [3, 4])
def test_dequantize_vs_reference_kernel(bits, style, variant):
    x = ref_cuda.synthetic_kv(style, N_VEC, 200 + bits)
    op, os_ = o.block_quantize(bits, 128, 0, -1, x, nthreads=8)
    ref_out = ref_cuda.dequant(op.reshape(-1, 4 * bits), os_.reshape(-1), bits, variant).reshape(N_VEC, 128)
    want = o.block_dequantize(bits, 128, 0, -1, op, os_, nthreads=8)
    mine = tq.block_dequantize(dev(op), dev(os_.view(np.int16)), bits, 128).cpu().numpy()
    assert np.array_equal(mine, want)     # library == oracle, bit for bit
    denom = np.maximum(np.abs(want), 1e-30)
    rel = float((np.abs(ref_out - want) / denom).max())
    same = float((ref_out == want).mean())
    print(f"\n[{variant} reference dequantize, {bits}-bit, {style}] max relative difference to the oracle {rel:.2e}, "
          f"bit-identical values {same:.4%}")
    assert rel <= 1e-5
    # the drop-in symbol with the reference's own argument list
    c, _ = o.block_codebook(bits, 0)
    pk, sc, cd, sg = dev(op.reshape(-1)), dev(os_.reshape(-1).view(np.int16)), dev(c), dev(ref_cuda.uploaded_sign_pattern())
    out = torch.zeros(N_VEC * 128, device="cuda")
    lib.tq_dequant_batch(ctypes.c_void_p(pk.data_ptr()), ctypes.c_void_p(sc.data_ptr()), ctypes.c_void_p(cd.data_ptr()),
                         ctypes.c_void_p(sg.data_ptr()), ctypes.c_void_p(out.data_ptr()), N_VEC * 4, 32, bits, 4 * bits, None)
    got = out.cpu().numpy().reshape(N_VEC, 128)
    assert float((np.abs(got - ref_out) / np.maximum(np.abs(ref_out), 1e-30)).max()) <= 1e-5


def test_round_trip_through_both_implementations():
    # reference quantize -> library dequantize and library quantize -> reference dequantize agree with the
    # oracle's round trip: the two code paths are interchangeable on stored bytes
    bits = 3
    x = ref_cuda.synthetic_kv("outlier", 4096, 7)
    rot = o.block_rotate(x)
    rp, rs = ref_cuda.quant_maxnorm(rot, bits, "ieee")
    mine = tq.block_dequantize(dev(rp.reshape(4096, -1)), dev(rs.reshape(4096, 4).view(np.int16)), bits, 128).cpu().numpy()
    idx, sc = tq.block_quantize(dev(x), bits)
    theirs = ref_cuda.dequant(idx.cpu().numpy().reshape(-1, 12), u16(sc).reshape(-1), bits, "ieee").reshape(4096, 128)
    assert float((np.abs(mine - theirs) / np.maximum(np.abs(mine), 1e-30)).max()) <= 1e-5
    cos = float((x * mine).sum() / np.sqrt((x * x).sum() * (mine * mine).sum()))
    assert cos > 0.9
