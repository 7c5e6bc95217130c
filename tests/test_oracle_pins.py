"""Pins the CPU oracle against the reference's own known answers (no GPU).

Sources of truth, in order of strength:
  * tests/golden/ref_primitives.npz -- produced by the reference's own header
    src/cache/cuda/kernels/tq_common.h (see tests/golden/make_golden.py);
  * tests/golden/ref_cuda_block.npz -- produced on a B200 by the reference's own block-32 quantize
    and dequantize CUDA kernels, compiled from the reference checkout (tests/ref_cuda.py);
  * facts asserted by the reference's test-suite, cited per test;
  * tests/golden/oracle_cases.npz -- the oracle's own committed outputs (regression guard).
"""
import itertools
import os

import numpy as np
import pytest

import oracle_lib as o

GOLD = os.path.join(os.path.dirname(__file__), "golden")
REF = np.load(os.path.join(GOLD, "ref_primitives.npz"))
CASES = np.load(os.path.join(GOLD, "oracle_cases.npz"))


# ---- against the reference's own code ---------------------------------------------------
@pytest.mark.parametrize("bits", [2, 3, 4])
def test_pack_matches_reference_header(bits):
    for codes, packed in zip(REF[f"codes_{bits}"], REF[f"packed_{bits}"]):
        assert np.array_equal(o.pack_indices(bits, codes), packed)
        assert np.array_equal(o.unpack_indices(bits, packed, 128), codes)


@pytest.mark.parametrize("seed", [0, 1, 42, 12345])
def test_sign_pattern_matches_reference_header(seed):
    assert np.array_equal(o.sign_pattern(256, seed), REF[f"sign_{seed}"])


@pytest.mark.parametrize("seed", [42, 12345])
def test_rademacher_matches_reference_header(seed):
    m = REF[f"rademacher_{seed}"]
    for row in range(0, 128, 5):
        got = np.array([o.rademacher_sign(seed, row, c) for c in range(128)])
        assert np.array_equal(got, m[row].astype(np.float32))


# ---- against the reference's own block-32 CUDA kernels (outputs frozen on a B200) ---------
REFCUDA = np.load(os.path.join(GOLD, "ref_cuda_block.npz"))


@pytest.mark.parametrize("style", ["outlier", "lognormal"])
@pytest.mark.parametrize("bits", [3, 4])
def test_block_quantize_matches_reference_cuda_kernel(bits, style):
    # tq_quant_maxnorm_kernel (tq_quant_kernel.cu:204-262) on the oracle's rotated blocks, IEEE build:
    # packed codes and f16 scales bit for bit
    x = REFCUDA[f"x_{style}"]
    assert np.array_equal(o.block_rotate(x), REFCUDA[f"rot_{style}"])
    packed, scales = o.block_quantize(bits, 128, 0, -1, x)
    assert np.array_equal(packed.reshape(-1, 4 * bits), REFCUDA[f"packed_{style}_{bits}_ieee"])
    assert np.array_equal(scales.reshape(-1), REFCUDA[f"scales_{style}_{bits}_ieee"])
    # the --use_fast_math build the reference ships divides approximately: codes may differ only where a
    # coordinate sits on a decision boundary (none does in this slice), scales by one f16 ulp
    fm_codes = o.unpack_indices(bits, REFCUDA[f"packed_{style}_{bits}_fastmath"].reshape(-1), x.size)
    assert int((fm_codes != o.unpack_indices(bits, packed.reshape(-1), x.size)).sum()) <= 2
    fm_sc = REFCUDA[f"scales_{style}_{bits}_fastmath"].astype(np.int32)
    assert np.abs(fm_sc - scales.reshape(-1).astype(np.int32)).max() <= 1


@pytest.mark.parametrize("variant", ["ieee", "fastmath"])
@pytest.mark.parametrize("style", ["outlier", "lognormal"])
@pytest.mark.parametrize("bits", [3, 4])
def test_block_dequantize_matches_reference_cuda_kernel(bits, style, variant):
    # tq_dequant_kernel (tq_dequant_kernel.cu:38-98) multiplies by rsqrtf(32) where the CPU path
    # (src/cache/wht_tensor.rs:38) multiplies by 1/sqrt(32): equal to 1e-5 relative, not bit for bit
    packed, scales = REFCUDA[f"packed_{style}_{bits}_ieee"], REFCUDA[f"scales_{style}_{bits}_ieee"]
    got = o.block_dequantize(bits, 128, 0, -1, packed.reshape(128, -1), scales.reshape(128, 4)).reshape(-1, 32)
    want = REFCUDA[f"deq_{style}_{bits}_{variant}"]
    assert float((np.abs(got - want) / np.maximum(np.abs(want), 1e-30)).max()) <= 1e-5


# ---- facts asserted by the reference's tests ---------------------------------------------
def test_wht_known_vector_and_self_inverse():
    # src/rotation.rs:236-256
    assert np.allclose(o.wht(np.ones(4, np.float32)), [2, 0, 0, 0], atol=1e-6)
    x = np.array([1, 2, 3, 4], np.float32)
    assert np.allclose(o.wht(o.wht(x)), x, atol=1e-5)


def test_sign_pattern_is_parity_of_seed_plus_index():
    # src/rotation.rs:47-70: odd multiplier => low bit of the hash is the parity of seed + i
    s = o.sign_pattern(128, 42)
    assert set(np.unique(s)) == {-1.0, 1.0}
    assert np.array_equal(s, np.where((42 + np.arange(128)) % 2 == 0, 1.0, -1.0).astype(np.float32))


@pytest.mark.parametrize("bits,group", [(2, 4), (3, 8), (4, 2)])
def test_pack_roundtrip_exhaustive_groups(bits, group):
    # tests/roundtrip_tests.rs:305-347,485-498: every value combination of one group (sampled for 3-bit)
    vals = range(1 << bits)
    combos = itertools.product(vals, repeat=group) if bits != 3 else (
        np.random.default_rng(0).integers(0, 8, size=(4096, 8)).tolist())
    for combo in combos:
        c = np.array(combo, np.uint8)
        assert np.array_equal(o.unpack_indices(bits, o.pack_indices(bits, c), group), c)


def test_pack_3bit_byte_layout_and_tail_padding():
    # src/packed/mod.rs:268-281: b0 = v0 | v1<<3 | (v2&3)<<6 ; b1 = v2>>2 | v3<<1 | v4<<4 | (v5&1)<<7 ; b2 = v5>>1 | v6<<2 | v7<<5
    v = np.array([1, 3, 5, 7, 0, 2, 4, 6], np.uint8)
    assert o.pack_indices(3, v).tolist() == [0x59, 0x0F, 0xD1]
    # src/packed/indices.rs: a partial group is zero-padded to a whole group
    assert o.packed_len(3, 5) == 3 and o.packed_len(2, 5) == 2 and o.packed_len(4, 5) == 3
    p = o.pack_indices(3, v[:5])
    assert np.array_equal(o.unpack_indices(3, p, 5), v[:5]) and len(p) == 3


def test_block_sizes():
    # src/quantize.rs:648-658 (34/50/66 B) and src/qjl.rs:1174-1180 (52/68 B) at d = 128
    for bits, size in ((2, 34), (3, 50), (4, 66)):
        assert 2 + o.packed_len(bits, 128) == size
    for bits, size in ((3, 52), (4, 68)):
        assert 2 + o.packed_len(bits - 1, 128) + 16 + 2 == size


@pytest.mark.parametrize("bits,dim", [(b, d) for b in (2, 3, 4) for d in (32, 64, 128, 256)])
def test_codebook_shape_and_boundary_semantics(bits, dim):
    c, b = o.codebook(bits, dim)
    assert len(c) == 1 << bits and len(b) == (1 << bits) - 1
    assert np.all(np.diff(c) > 0) and np.all(np.diff(b) > 0)
    assert b[len(b) // 2] == 0.0                                   # symmetric, middle boundary exactly 0
    for i, ci in enumerate(c):                                      # tests/codebook_tests.rs:225-230
        assert o.nearest_centroid(bits, dim, ci) == i
    for i, bi in enumerate(b):                                      # tests/codebook_tests.rs:233-250
        assert o.nearest_centroid(bits, dim, bi - 1e-10) == i
        assert o.nearest_centroid(bits, dim, bi + 1e-10) == i + 1
        assert o.nearest_centroid(bits, dim, bi) == i               # a value on the boundary goes to the lower bin


@pytest.mark.parametrize("bits,lo,hi", [(3, 0.030, 0.038), (4, 0.007, 0.011)])
def test_normalized_mse_windows_on_the_reference_stream(bits, lo, hi):
    # tests/mse_validation.rs:83-142: 10,000 vectors from Lcg::new(12345) + Box-Muller, seed 42
    x = o.lcg_normal_vectors(12345, 10000, 128)
    p, s = o.quantize_batch(bits, 128, 42, x, nthreads=8)
    y = o.dequantize_batch(bits, 128, 42, p, s, nthreads=8)
    xd, yd = x.astype(np.float64), y.astype(np.float64)
    nmse = (((xd - yd) ** 2).sum(1) / (xd ** 2).sum(1)).mean()
    assert lo <= nmse <= hi, nmse


def test_config1_nmse_on_numpy_stream():
    # the CPU-runnable configuration: 10,000 x 128 N(0,1), bits 3 and 4, seed 42
    x = np.random.default_rng(42).standard_normal((10000, 128)).astype(np.float32)
    for bits, want in ((3, 0.0340), (4, 0.00935)):
        p, s = o.quantize_batch(bits, 128, 42, x, nthreads=8)
        y = o.dequantize_batch(bits, 128, 42, p, s, nthreads=8)
        nmse = (((x - y) ** 2).sum(1) / (x ** 2).sum(1)).mean()
        assert abs(nmse - want) < 0.0005, nmse


def test_zero_vector_quantizes_to_zero_scale():
    # src/quantize.rs:60-72,123-126
    p, s = o.quantize_batch(3, 128, 42, np.zeros((1, 128), np.float32))
    assert s[0] == 0
    assert np.all(o.dequantize_batch(3, 128, 42, p, s) == 0.0)


def test_qjl_uses_bits_minus_one_and_algorithm2_identity():
    # src/qjl.rs:1134-1162 (TQ3 => 2-bit polar) and tests/paper_verification_tests.rs:412-470
    rng = np.random.default_rng(3)
    x = rng.standard_normal((4, 128)).astype(np.float32)
    q = rng.standard_normal(128).astype(np.float32)
    p, s, sg, rn = o.qjl_quantize_batch(3, 128, 42, 42, x)
    assert p.shape[1] == 32 and sg.shape[1] == 16
    scores = o.attention_scores(3, 128, 42, 42, q, p, s, sg, rn)
    rec = o.dequantize_batch(2, 128, 42, p, s)
    R = o.rademacher_matrix(128, 42) / np.sqrt(np.float32(128))
    for i in range(4):
        z = np.array([1.0 if (sg[i][j >> 3] >> (j & 7)) & 1 else -1.0 for j in range(128)])
        closed = float(q @ rec[i]) + o.f16_bits_to_f32(rn[i]) * np.sqrt(np.pi / 2) / np.sqrt(128) * float((R @ q) @ z)
        assert abs(closed - scores[i]) < 1e-4
        # stored residual norm within f16 rounding of the true one (paper_verification_tests.rs:536-575)
        true = np.linalg.norm(x[i] - rec[i])
        assert abs(o.f16_bits_to_f32(rn[i]) - true) / true < 0.02


def test_qjl_estimator_is_nearly_unbiased():
    # tests/paper_verification_tests.rs:143-175 (mean bias < 0.03), scaled down to 300 pairs
    rng = np.random.default_rng(11)
    x = rng.standard_normal((300, 128)).astype(np.float32)
    x /= np.linalg.norm(x, axis=1, keepdims=True)
    q = rng.standard_normal(128).astype(np.float32)
    q /= np.linalg.norm(q)
    p, s, sg, rn = o.qjl_quantize_batch(3, 128, 42, 12345, x, nthreads=8)
    est = o.attention_scores(3, 128, 42, 12345, q, p, s, sg, rn, nthreads=8)
    assert abs(np.mean(est - x @ q)) < 0.03


def _sincos(shape, seed, fn, freq, amp, off=0):
    n = int(np.prod(shape))
    i = np.arange(n, dtype=np.float64)
    return (fn((i + seed + off) * freq) * amp).astype(np.float32).reshape(shape)


@pytest.mark.parametrize("bits,norm_mode,thr", [(3, 0, 0.85), (3, 1, 0.83), (4, 0, 0.92)])
def test_block_format_cosine_thresholds(bits, norm_mode, thr):
    # tests/cache_pqo_tests.rs:31-43,152-244: sin/cos tensors of shape [1, 8, S, 128]
    for x in (_sincos((8 * 16, 128), 0, np.sin, 0.0137, 2.0), _sincos((8 * 16, 128), 0, np.cos, 0.0213, 1.5, 1000)):
        p, s = o.block_quantize(bits, 128, norm_mode, -1, x)
        y = o.block_dequantize(bits, 128, norm_mode, -1, p, s)
        cos = float((x * y).sum() / np.sqrt((x * x).sum() * (y * y).sum()))
        assert cos > thr, cos


def test_block_format_geometry_and_outlier_marker():
    # tests/cache_storage_tests.rs:81-87 (packed_dim 48, 4 blocks); src/cache/storage.rs:122-125 (negative scale)
    x = np.random.default_rng(0).standard_normal((3, 128)).astype(np.float32)
    p, s = o.block_quantize(3, 128, 0, -1, x)
    assert p.shape == (3, 48) and s.shape == (3, 4)
    assert np.all(s.view(np.int16) < 0)                    # PQO: every block marked
    p0, s0 = o.block_quantize(3, 128, 0, 0, x)
    assert np.all(s0.view(np.int16) > 0)                   # PQ/TQ: none marked
    # bits-1 codebook packed at `bits` width: the top code bit is never used (src/cache/config.rs:82-84)
    assert o.unpack_indices(3, p0.reshape(-1), 3 * 128).max() <= 3


def test_block_codebooks():
    # src/cache/precomputed/codebooks.rs:51-88
    c3, b3 = o.block_codebook(3, 0)
    assert np.allclose(c3, [-2.1573, -1.3336, -0.7434, -0.2428, 0.2428, 0.7434, 1.3336, 2.1573])
    assert np.allclose(b3, [-1.7455, -1.0385, -0.4931, 0.0, 0.4931, 1.0385, 1.7455])
    c2, _ = o.block_codebook(2, 0)
    assert np.allclose(c2, c3[[0, 2, 5, 7]])
    c4, b4 = o.block_codebook(4, 0)
    assert np.allclose(np.diff(c4), 2 * 2.1573 / 15, atol=1e-6) and np.isclose(c4[0], -2.1573) and np.isclose(c4[-1], 2.1573)
    assert np.allclose(b4, (c4[:-1] + c4[1:]) / 2, atol=1e-6)


def test_block_attention_equals_dequantize_then_sdpa():
    rng = np.random.default_rng(5)
    hq, hkv, L = 4, 2, 19
    k = rng.standard_normal((hkv * L, 128)).astype(np.float32)
    v = rng.standard_normal((hkv * L, 128)).astype(np.float32)
    q = (rng.standard_normal((hq, 128)) / np.sqrt(128)).astype(np.float32)
    kp, ks = o.block_quantize(3, 128, 0, -1, k)
    vp, vs = o.block_quantize(3, 128, 0, -1, v)
    out = o.block_attention(3, 128, 0, -1, q, kp.reshape(hkv, L, -1), ks.reshape(hkv, L, -1), vp.reshape(hkv, L, -1),
                            vs.reshape(hkv, L, -1), L, 0.0884)
    kd = o.block_dequantize(3, 128, 0, -1, kp, ks).reshape(hkv, L, 128)
    vd = o.block_dequantize(3, 128, 0, -1, vp, vs).reshape(hkv, L, 128)
    assert np.allclose(out, o.sdpa(q, kd, vd, 0.0884), atol=1e-5)


# ---- regression guard on the oracle itself -------------------------------------------------
def test_oracle_reproduces_committed_cases():
    x = CASES["whole_x"]
    for bits in (2, 3, 4):
        p, s = o.quantize_batch(bits, 128, 42, x)
        assert np.array_equal(p, CASES[f"whole_packed_{bits}"]) and np.array_equal(s, CASES[f"whole_scales_{bits}"])
        assert np.array_equal(o.dequantize_batch(bits, 128, 42, p, s), CASES[f"whole_deq_{bits}"])
    for bits in (3, 4):
        p, s, sg, rn = o.qjl_quantize_batch(bits, 128, 42, 42, x[:16])
        assert np.array_equal(sg, CASES[f"qjl_signs_{bits}"]) and np.array_equal(rn, CASES[f"qjl_rnorms_{bits}"])
    xb = CASES["block_x"]
    for bits, nm, ob, tag in ((3, 0, -1, "pqo3"), (4, 0, -1, "pqo4"), (3, 1, -1, "pqo3_l2"), (3, 0, 0, "pq3"), (4, 0, 2, "mix4")):
        p, s = o.block_quantize(bits, 128, nm, ob, xb)
        assert np.array_equal(p, CASES[f"block_packed_{tag}"]) and np.array_equal(s, CASES[f"block_scales_{tag}"])
        assert np.array_equal(o.block_dequantize(bits, 128, nm, ob, p, s), CASES[f"block_deq_{tag}"])
