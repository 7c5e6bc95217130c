"""GPU parity of fused decode attention over the packed block-32 cache (tolerance 2e-3 max-abs
against the CPU oracle over the IDENTICAL packed bytes), of the split/shard merge, and of
PqoCache."""
import ctypes
import os

import numpy as np
import pytest
import torch

import oracle_lib as o
import turboquant_b200 as tq
from turboquant_b200._lib import lib

pytestmark = pytest.mark.gpu
CASES = np.load(os.path.join(os.path.dirname(__file__), "golden", "oracle_cases.npz"))
TOL = 2e-3   # attention outputs: max-abs error allowed by the parity contract


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def u16(t):
    return t.cpu().numpy().view(np.uint16)


def ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def make_cache(rng, hkv, L, stride, bits, head_dim=128, outliers=True, nm=0, ob=-1):
    k = rng.standard_normal((hkv, L, head_dim)).astype(np.float32)
    v = rng.standard_normal((hkv, L, head_dim)).astype(np.float32)
    if outliers:
        ch = rng.choice(head_dim, max(1, head_dim * 2 // 100 + 1), replace=False)
        k[:, :, ch] *= 8
        v[:, :, ch] *= 8
    pd, nb = head_dim * bits // 8, head_dim // 32
    ki = np.zeros((hkv, stride, pd), np.uint8); ks = np.zeros((hkv, stride, nb), np.uint16)
    vi = np.zeros((hkv, stride, pd), np.uint8); vs = np.zeros((hkv, stride, nb), np.uint16)
    if L:
        p, s = o.block_quantize(bits, head_dim, nm, ob, k.reshape(-1, head_dim), nthreads=8)
        ki[:, :L], ks[:, :L] = p.reshape(hkv, L, pd), s.reshape(hkv, L, nb)
        p, s = o.block_quantize(bits, head_dim, nm, ob, v.reshape(-1, head_dim), nthreads=8)
        vi[:, :L], vs[:, :L] = p.reshape(hkv, L, pd), s.reshape(hkv, L, nb)
    return ki, ks, vi, vs


def gpu_attend(q, ki, ks, vi, vs, L, bits, scale, **kw):
    return tq.decode_attention(dev(q), dev(ki), dev(ks.view(np.int16)), dev(vi), dev(vs.view(np.int16)), L, bits, scale, **kw)


@pytest.mark.parametrize("tag,bits", [("pqo3", 3), ("pqo4", 4)])
def test_golden_fixture(tag, bits):
    hq, hkv, L = 4, 2, 37
    kp, ks = o.block_quantize(bits, 128, 0, -1, CASES["att_k"])
    vp, vs = o.block_quantize(bits, 128, 0, -1, CASES["att_v"])
    out = gpu_attend(CASES["att_q"], kp.reshape(hkv, L, -1), ks.reshape(hkv, L, -1), vp.reshape(hkv, L, -1),
                     vs.reshape(hkv, L, -1), L, bits, 1.0 / np.sqrt(128)).cpu().numpy()
    assert np.abs(out - CASES[f"att_out_{tag}"]).max() < TOL


@pytest.mark.parametrize("bits", [3, 4])
@pytest.mark.parametrize("L", [1, 2, 31, 32, 33, 511, 512, 513])
def test_ragged_lengths(bits, L):
    rng = np.random.default_rng(L * 10 + bits)
    hq, hkv = 4, 2
    ki, ks, vi, vs = make_cache(rng, hkv, L, L + 3, bits)
    q = (rng.standard_normal((hq, 128)) / np.sqrt(128)).astype(np.float32)
    want = o.block_attention(bits, 128, 0, -1, q, ki, ks, vi, vs, L, 0.0884, nthreads=8)
    for parts in (0, 1, 3):
        got = gpu_attend(q, ki, ks, vi, vs, L, bits, 0.0884, num_partitions=parts).cpu().numpy()
        assert np.abs(got - want).max() < TOL


@pytest.mark.parametrize("bits,hq,hkv,head_dim", [(3, 16, 8, 128), (4, 32, 8, 128), (3, 64, 8, 128), (3, 8, 8, 128),
                                                  (4, 24, 2, 128), (3, 4, 2, 64), (4, 4, 2, 256), (3, 3, 1, 96)])
def test_gqa_groups_and_head_dims(bits, hq, hkv, head_dim):
    rng = np.random.default_rng(hq * 7 + head_dim)
    L = 300
    ki, ks, vi, vs = make_cache(rng, hkv, L, L, bits, head_dim)
    q = (rng.standard_normal((hq, head_dim)) / np.sqrt(head_dim)).astype(np.float32)
    scale = 1.0 / np.sqrt(head_dim)
    want = o.block_attention(bits, head_dim, 0, -1, q, ki, ks, vi, vs, L, scale, nthreads=8)
    got = gpu_attend(q, ki, ks, vi, vs, L, bits, scale).cpu().numpy()
    assert np.abs(got - want).max() < TOL


@pytest.mark.parametrize("bits", [3, 4])
@pytest.mark.parametrize("g", [1, 2, 4, 8])
@pytest.mark.parametrize("L", [17, 1000, 4133])
def test_tensor_core_kernel_against_oracle_and_general_kernel(bits, g, L):
    rng = np.random.default_rng(g * 100 + L)
    hkv = 3
    hq = hkv * g
    ki, ks, vi, vs = make_cache(rng, hkv, L, L + 5, bits)
    q = (rng.standard_normal((hq, 128)) / np.sqrt(128)).astype(np.float32)
    want = o.block_attention(bits, 128, 0, -1, q, ki, ks, vi, vs, L, 0.0884, nthreads=8)
    fast = gpu_attend(q, ki, ks, vi, vs, L, bits, 0.0884).cpu().numpy()
    slow = gpu_attend(q, ki, ks, vi, vs, L, bits, 0.0884, force_general=True).cpu().numpy()
    # 4-bit: exact-integer codes + hi/lo splits give f32-level agreement; 3-bit: the f16 table holds
    # centroid / kappa with a relative error below 1e-4
    tol = 2e-5 if bits == 4 else 3e-4
    assert np.abs(fast - want).max() < tol
    assert np.abs(slow - want).max() < 2e-5
    for parts in (1, 2, 7):
        got = gpu_attend(q, ki, ks, vi, vs, L, bits, 0.0884, num_partitions=parts).cpu().numpy()
        assert np.abs(got - want).max() < tol


@pytest.mark.parametrize("bits", [3, 4])
@pytest.mark.parametrize("g", [4, 8])
@pytest.mark.parametrize("L,stride", [(5, 16), (100, 128), (1000, 1024), (4133, 4200), (700, 701)])
def test_tensor_copy_staging_equals_cp_async_staging(bits, g, L, stride):
    # With the TMA flag even strides take the TMA-staged kernel, odd ones (701) fall back by themselves; both
    # must give the bits of the cp.async-staged kernel.  The slots behind the last token hold NaN/Inf scale patterns and
    # random codes: nothing of them may reach the result.
    rng = np.random.default_rng(bits * 1000 + g * 10 + L)
    hkv = 3
    ki, ks, vi, vs = make_cache(rng, hkv, L, stride, bits)
    for arr, fill in ((ks, 0x7E00), (vs, 0xFC00)):
        arr[:, L:] = fill
    ki[:, L:] = 0xA5
    vi[:, L:] = 0x5A
    q = (rng.standard_normal((hkv * g, 128)) / np.sqrt(128)).astype(np.float32)
    want = o.block_attention(bits, 128, 0, -1, q, ki, ks, vi, vs, L, 0.0884, nthreads=8)
    for parts in (0, 1, 3):
        a = gpu_attend(q, ki, ks, vi, vs, L, bits, 0.0884, num_partitions=parts, tma=True)
        b = gpu_attend(q, ki, ks, vi, vs, L, bits, 0.0884, num_partitions=parts)
        assert torch.equal(a, b)
        assert np.abs(a.cpu().numpy() - want).max() < (2e-5 if bits == 4 else 3e-4)
    assert lib.tqb_decode_stage_timeouts() == 0


@pytest.mark.parametrize("bits,nm,ob", [(4, 0, -1), (3, 0, -1), (3, 1, -1), (4, 0, 2)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("L", [1, 64, 65, 1000, 4097])
def test_fused_append_equals_append_then_attend(bits, nm, ob, dtype, L):
    # The new token's K/V rows quantized inside the attention call (in the kernel for the all-outlier MaxNorm
    # format, by a launch of its own otherwise) against quantize-then-attend: same cache bytes, same output.
    rng = np.random.default_rng(bits * 100 + nm * 10 + L)
    hkv, g, stride = 3, 4, L + 6
    mode = tq.QuantNormMode(nm)
    ki, ks, vi, vs = (dev(x) for x in make_cache(rng, hkv, L - 1, stride, bits, nm=nm, ob=ob))
    ks, vs = ks.view(torch.int16), vs.view(torch.int16)
    newk = torch.from_numpy(rng.standard_normal((hkv, 128)).astype(np.float32)).to(dtype).cuda()
    newv = torch.from_numpy(rng.standard_normal((hkv, 128)).astype(np.float32)).to(dtype).cuda()
    q = torch.from_numpy((rng.standard_normal((hkv * g, 128)) / np.sqrt(128)).astype(np.float32)).to(dtype).cuda()
    # reference: separate append, then attention
    ref = [t.clone() for t in (ki, ks, vi, vs)]
    tq.block_quantize(newk, bits, mode, ob, out=(ref[0], ref[1]), rows_per_group=1, group_stride=stride, row_offset=L - 1)
    tq.block_quantize(newv, bits, mode, ob, out=(ref[2], ref[3]), rows_per_group=1, group_stride=stride, row_offset=L - 1)
    want = tq.decode_attention(q, *ref, L, bits, 0.0884, norm_mode=mode, outlier_blocks=ob)
    for parts in (0, 1, 3):
        got_cache = [t.clone() for t in (ki, ks, vi, vs)]
        got = tq.decode_attention(q, *got_cache, L, bits, 0.0884, norm_mode=mode, outlier_blocks=ob, num_partitions=parts,
                                  append=(newk, newv))
        for a, b in zip(got_cache, ref):
            assert torch.equal(a, b)
        if parts == 0:
            assert torch.equal(got, want)
        else:
            assert (got.float() - want.float()).abs().max() < (1e-2 if dtype == torch.bfloat16 else 1e-5)


@pytest.mark.parametrize("bits,nm,ob", [(3, 0, -1), (3, 1, -1), (3, 0, 0), (4, 0, -1)])
def test_tensor_core_kernel_sharp_softmax(bits, nm, ob):
    # large logits: a handful of tokens carry all the weight, so element errors are not averaged away.
    # 4-bit is exact at any sharpness (|logit| ~ 60 here).  The 3-bit table carries a 2.3e-5 relative
    # centroid error, which a logit of magnitude x turns into ~2.3e-5 * x: inside the bound up to
    # |logit| ~ 30 (measured 1.6e-3 at 30, 2.9e-3 at 100), so the 3-bit cases run at |logit| ~ 30.
    scale = 1.0 if bits == 4 else 0.3
    rng = np.random.default_rng(bits * 7 + nm + ob)
    hq, hkv, L = 8, 2, 1500
    ki, ks, vi, vs = make_cache(rng, hkv, L, L, bits, nm=nm, ob=ob)
    q = rng.standard_normal((hq, 128)).astype(np.float32)
    want = o.block_attention(bits, 128, nm, ob, q, ki, ks, vi, vs, L, scale, nthreads=8)
    got = gpu_attend(q, ki, ks, vi, vs, L, bits, scale, norm_mode=tq.QuantNormMode(nm), outlier_blocks=ob).cpu().numpy()
    assert np.abs(got - want).max() < TOL, np.abs(got - want).max()


def test_sharp_softmax_and_query_dtypes():
    # large logits: one token dominates; also bf16 / f16 queries and outputs
    rng = np.random.default_rng(77)
    hq, hkv, L = 8, 2, 700
    ki, ks, vi, vs = make_cache(rng, hkv, L, L, 4)
    q = rng.standard_normal((hq, 128)).astype(np.float32)
    want = o.block_attention(4, 128, 0, -1, q, ki, ks, vi, vs, L, 1.0, nthreads=8)
    got = gpu_attend(q, ki, ks, vi, vs, L, 4, 1.0).cpu().numpy()
    assert np.abs(got - want).max() < TOL * max(1.0, np.abs(want).max())
    for dt in (torch.bfloat16, torch.float16):
        qh = torch.from_numpy(q / np.sqrt(128)).to(dt)
        want = o.block_attention(4, 128, 0, -1, qh.float().numpy(), ki, ks, vi, vs, L, 0.0884, nthreads=8)
        got = tq.decode_attention(qh.cuda(), dev(ki), dev(ks.view(np.int16)), dev(vi), dev(vs.view(np.int16)), L, 4, 0.0884)
        assert got.dtype == dt
        assert np.abs(got.float().cpu().numpy() - want).max() < 2e-2 * max(1.0, np.abs(want).max())  # output rounding of the half type


@pytest.mark.parametrize("nm,ob", [(1, -1), (0, 0), (0, 2)])
def test_other_cache_modes(nm, ob):
    rng = np.random.default_rng(nm * 10 + ob + 5)
    hq, hkv, L = 4, 2, 129
    ki, ks, vi, vs = make_cache(rng, hkv, L, L, 3, nm=nm, ob=ob)
    q = (rng.standard_normal((hq, 128)) / np.sqrt(128)).astype(np.float32)
    want = o.block_attention(3, 128, nm, ob, q, ki, ks, vi, vs, L, 0.0884)
    got = gpu_attend(q, ki, ks, vi, vs, L, 3, 0.0884, norm_mode=tq.QuantNormMode(nm), outlier_blocks=ob).cpu().numpy()
    assert np.abs(got - want).max() < TOL


@pytest.mark.parametrize("g", [1, 2, 4, 8])
@pytest.mark.parametrize("L", [200, 4133])
def test_qjl_correction_branch(g, L):
    # tq_attention_kernel.cu:197-231: per-key residual sign sketch over the whole head_dim.  The 3-bit tensor-core
    # kernel applies it on the integer tensor-core path; the general kernel (forced) is the cross-check.
    rng = np.random.default_rng(9 + g + L)
    hkv, D = 2, 128
    hq = hkv * g
    k = rng.standard_normal((hkv, L, D)).astype(np.float32)
    ki, ks, vi, vs = make_cache(rng, hkv, L, L + 3, 3, outliers=False, ob=0)
    kp, ksc = o.block_quantize(3, D, 0, 0, k.reshape(-1, D), nthreads=8)
    ki[:, :L], ks[:, :L] = kp.reshape(hkv, L, -1), ksc.reshape(hkv, L, -1)
    res = k.reshape(-1, D) - o.block_dequantize(3, D, 0, 0, kp, ksc, nthreads=8)
    signs = np.zeros((hkv, L + 3, D // 8), np.uint8)
    norms = np.zeros((hkv, L + 3), np.uint16)
    signs[:, :L] = np.stack([o.qjl_signs(r, D, 12345) for r in res]).reshape(hkv, L, D // 8)
    norms[:, :L] = np.array([o.f32_to_f16_bits(float(np.linalg.norm(r))) for r in res], np.uint16).reshape(hkv, L)
    signs[:, L:], norms[:, L:] = 0xFF, 0x7E00     # slots behind the last token: nothing of them may reach the result
    q = (rng.standard_normal((hq, D)) / np.sqrt(D)).astype(np.float32)
    rq = np.stack([o.query_projections(qh, D, 12345) for qh in q])
    want = o.block_attention(3, D, 0, 0, q, ki, ks, vi, vs, L, 0.0884, qjl=(signs, norms, rq), nthreads=8)
    args = dict(outlier_blocks=0, qjl=(dev(signs), dev(norms.view(np.int16)), dev(rq)))
    for parts in (0, 1, 3):
        got = gpu_attend(q, ki, ks, vi, vs, L, 3, 0.0884, num_partitions=parts, **args).cpu().numpy()
        assert np.abs(got - want).max() < 3e-4, np.abs(got - want).max()
    slow = gpu_attend(q, ki, ks, vi, vs, L, 3, 0.0884, force_general=True, **args).cpu().numpy()
    assert np.abs(slow - want).max() < 2e-5
    plain = o.block_attention(3, D, 0, 0, q, ki, ks, vi, vs, L, 0.0884, nthreads=8)
    assert np.abs(plain - want).max() > 1e-4      # the correction is not a no-op


def test_empty_cache_gives_zero_output():
    q = torch.randn((4, 128), device="cuda")
    z8 = torch.zeros((2, 4, 48), dtype=torch.uint8, device="cuda")
    z16 = torch.zeros((2, 4, 4), dtype=torch.int16, device="cuda")
    out = tq.decode_attention(q, z8, z16, z8, z16, 0, 3, 1.0)
    assert torch.all(out == 0)
    with pytest.raises(tq.RangeOutOfBounds):
        tq.decode_attention(q, z8, z16, z8, z16, 5, 3, 1.0)


def test_reference_fused_attention_symbol():
    # tq_fused_attention with the reference's argument list (src/cache/cuda/ffi.rs:50-78),
    # partition count = ceil(kv_len / 512) and caller-owned, pre-zeroed partial buffers
    rng = np.random.default_rng(21)
    hq, hkv, L, stride = 8, 2, 1100, 1300
    for bits in (3, 4):
        ki, ks, vi, vs = make_cache(rng, hkv, L, stride, bits)
        q = (rng.standard_normal((hq, 128)) / np.sqrt(128)).astype(np.float32)
        c, _ = o.block_codebook(bits, 0)
        sign = (o.block_signs() * (np.float32(1) / np.sqrt(np.float32(32))) * np.sqrt(np.float32(32))).astype(np.float32)
        parts = (L + 511) // 512
        out = torch.zeros((hq, 128), device="cuda")
        po = torch.zeros((hq * parts, 128), device="cuda")
        pm = torch.zeros(hq * parts, device="cuda"); ps = torch.zeros(hq * parts, device="cuda")
        t = [dev(q), dev(ki), dev(ks.view(np.int16)), dev(vi), dev(vs.view(np.int16)), dev(c), dev(sign)]
        lib.tq_fused_attention(*[ptr(x) for x in t], ptr(out), ptr(po), ptr(pm), ptr(ps), None, None, None, 0, hq, hkv, 128,
                               L, stride, 128 * bits // 8, 4, bits, 0.0884, parts, None)
        want = o.block_attention(bits, 128, 0, -1, q, ki, ks, vi, vs, L, 0.0884, nthreads=8)
        # the crate's own tables: a device-side gate routes the call to the tensor-core kernel
        assert np.abs(out.cpu().numpy() - want).max() < (2e-5 if bits == 4 else 3e-4)
        # any other table (here: the codebook scaled by 1.5) must take the general kernel and decode with it
        out2 = torch.zeros((hq, 128), device="cuda")
        for x in (po, pm, ps):
            x.zero_()
        t[5] = dev((c * np.float32(1.5)).astype(np.float32))
        lib.tq_fused_attention(*[ptr(x) for x in t], ptr(out2), ptr(po), ptr(pm), ptr(ps), None, None, None, 0, hq, hkv, 128,
                               L, stride, 128 * bits // 8, 4, bits, 0.0884, parts, None)
        # K and V both grow by 1.5: logits x 1.5 (= softmax scale x 1.5 on the original tables), values x 1.5
        want2 = 1.5 * o.block_attention(bits, 128, 0, -1, q, ki, ks, vi, vs, L, 0.0884 * 1.5, nthreads=8)
        assert np.abs(out2.cpu().numpy() - want2).max() < TOL


def test_sequence_shards_merge_to_the_unsharded_result():
    # split the sequence into 3 ragged shards, attend per shard, merge (max, sum, out) partials
    rng = np.random.default_rng(33)
    hq, hkv, L = 16, 2, 1000
    ki, ks, vi, vs = make_cache(rng, hkv, L, L, 3)
    q = (rng.standard_normal((hq, 128)) / np.sqrt(128)).astype(np.float32)
    want = o.block_attention(3, 128, 0, -1, q, ki, ks, vi, vs, L, 0.0884, nthreads=8)
    outs, lses = [], []
    for lo, hi in ((0, 400), (400, 401), (401, 1000)):
        out, lse = gpu_attend(q, ki[:, lo:hi], ks[:, lo:hi], vi[:, lo:hi], vs[:, lo:hi], hi - lo, 3, 0.0884, return_lse=True)
        outs.append(out); lses.append(lse)
    got = tq.lse_combine(torch.stack(outs), torch.stack(lses)).cpu().numpy()
    assert np.abs(got - want).max() < TOL
    # an empty shard contributes nothing
    e_out, e_lse = gpu_attend(q, ki[:, :4], ks[:, :4], vi[:, :4], vs[:, :4], 0, 3, 0.0884, return_lse=True)
    got2 = tq.lse_combine(torch.stack(outs + [e_out]), torch.stack(lses + [e_lse])).cpu().numpy()
    assert np.abs(got2 - want).max() < TOL


def _sincos(shape, seed, fn, freq, amp, off=0):
    i = np.arange(int(np.prod(shape)), dtype=np.float64)
    return torch.from_numpy((fn((i + seed + off) * freq) * amp).astype(np.float32).reshape(shape))


@pytest.mark.parametrize("bits,nm,thr", [(3, 0, 0.85), (3, 1, 0.83), (4, 0, 0.92)])
def test_pqo_cache_follows_the_reference_tests(bits, nm, thr):
    # tests/cache_pqo_tests.rs: first prefill returns the originals (:86-104), later calls return the
    # whole dequantized cache (:119-149), cosine thresholds (:152-244), reset / memory / layers (:251-304)
    cfg = tq.CacheConfig(bits=bits, head_dim=128, num_kv_heads=8, num_layers=2, norm_mode=tq.QuantNormMode(nm))
    cache = tq.PqoCache(cfg)
    k = _sincos((1, 8, 16, 128), 0, np.sin, 0.0137, 2.0).cuda()
    v = _sincos((1, 8, 16, 128), 0, np.cos, 0.0213, 1.5, 1000).cuda()
    r = cache.prefill(0, k, v)
    assert r.k is k and r.v is v and r.logit_bias is None
    assert cache.seq_len(0) == 16 and cache.seq_len(1) == 0
    assert cache.capacity(0) == 16 + 128                      # src/cache/storage.rs:114-116
    assert cache.memory_usage() == 2 * 8 * 16 * (128 * bits // 8) + 2 * 8 * 16 * 4 * 2
    k2 = _sincos((1, 8, 4, 128), 50, np.sin, 0.0137, 2.0).cuda()
    v2 = _sincos((1, 8, 4, 128), 50, np.cos, 0.0213, 1.5, 1000).cuda()
    r2 = cache.prefill(0, k2, v2)
    assert r2.k.shape == (1, 8, 20, 128)
    full_k = torch.cat([k, k2], dim=2)
    cos = torch.nn.functional.cosine_similarity(full_k.flatten(), r2.k.flatten(), dim=0).item()
    assert cos > thr
    want_k = o.block_dequantize(bits, 128, nm, -1, *o.block_quantize(bits, 128, nm, -1, full_k.cpu().numpy().reshape(-1, 128)))
    assert np.array_equal(r2.k.cpu().numpy().reshape(-1, 128), want_k)
    # decode: Fused output of shape [1, Hq, 1, D], equal to oracle attention over the same packed cache
    q = (torch.randn((1, 16, 1, 128), generator=torch.Generator().manual_seed(1)) / 128 ** 0.5).cuda()
    k3, v3 = torch.randn((1, 8, 1, 128)).cuda(), torch.randn((1, 8, 1, 128)).cuda()
    dec = cache.decode(0, k3, v3, q, tq.AttendConfig(softmax_scale=0.0884, n_kv_groups=2))
    assert dec.is_fused() and dec.fused.shape == (1, 16, 1, 128)
    assert dec.fused.abs().sum().item() > 0.01                # tests/cache_pqo_tests.rs:387-406
    allk = torch.cat([k, k2, k3], dim=2).cpu().numpy().reshape(8, 21, 128)
    allv = torch.cat([v, v2, v3], dim=2).cpu().numpy().reshape(8, 21, 128)
    kp, ks = o.block_quantize(bits, 128, nm, -1, allk.reshape(-1, 128))
    vp, vs = o.block_quantize(bits, 128, nm, -1, allv.reshape(-1, 128))
    want = o.block_attention(bits, 128, nm, -1, q.cpu().numpy().reshape(16, 128), kp.reshape(8, 21, -1), ks.reshape(8, 21, -1),
                             vp.reshape(8, 21, -1), vs.reshape(8, 21, -1), 21, 0.0884)
    assert np.abs(dec.fused.cpu().numpy().reshape(16, 128) - want).max() < TOL
    cache.reset()
    assert cache.seq_len(0) == 0 and cache.memory_usage() == 0
    with pytest.raises(tq.LayerOutOfRange):
        cache.seq_len(2)
    with pytest.raises(tq.InvalidDimension):
        tq.PqoCache(tq.CacheConfig(bits=3, head_dim=100, num_kv_heads=1, num_layers=1))   # src/cache/pqo.rs:32-39
    with pytest.raises(tq.UnsupportedBits):
        tq.PqoCache(tq.CacheConfig(bits=2, head_dim=128, num_kv_heads=1, num_layers=1))


def test_pqo_cache_growth_batch_and_host_buffers():
    # growth policy needed + max(needed/4, 128) with copy-on-grow; batch folds into heads;
    # host-buffer mode copies k, v, q in and the output back
    cfg = tq.CacheConfig(bits=4, head_dim=128, num_kv_heads=2, num_layers=1, batch=3)
    cache = tq.PqoCache(cfg)
    g = torch.Generator().manual_seed(5)
    ks_, vs_ = [], []
    for step, n in enumerate((100, 50, 200)):
        k, v = torch.randn((3, 2, n, 128), generator=g).bfloat16(), torch.randn((3, 2, n, 128), generator=g).bfloat16()
        cache.prefill(0, k.cuda(), v.cuda())
        ks_.append(k); vs_.append(v)
    assert cache.seq_len(0) == 350
    assert cache.capacity(0) == 350 + 128      # 100 -> 228; 150 fits; 350 -> 350 + max(87, 128)
    allk, allv = torch.cat(ks_, dim=2), torch.cat(vs_, dim=2)
    dk, dv = cache.dequantize_full(0)
    want = o.block_dequantize(4, 128, 0, -1, *o.block_quantize(4, 128, 0, -1, allk.float().numpy().reshape(-1, 128), nthreads=8))
    assert np.array_equal(dk.cpu().numpy().reshape(-1, 128), want)      # old rows survived both regrowths
    k1, v1 = torch.randn((3, 2, 1, 128), generator=g).bfloat16(), torch.randn((3, 2, 1, 128), generator=g).bfloat16()
    q = (torch.randn((3, 8, 1, 128), generator=g) / 128 ** 0.5).bfloat16()
    out_host = torch.empty_like(q).pin_memory()
    cache.decode(0, k1.pin_memory(), v1.pin_memory(), q.pin_memory(), tq.AttendConfig(0.0884, 4), out=out_host)
    cache.host_sync()
    allk, allv = torch.cat([allk, k1], dim=2), torch.cat([allv, v1], dim=2)
    kp, ksc = o.block_quantize(4, 128, 0, -1, allk.float().numpy().reshape(-1, 128), nthreads=8)
    vp, vsc = o.block_quantize(4, 128, 0, -1, allv.float().numpy().reshape(-1, 128), nthreads=8)
    want = o.block_attention(4, 128, 0, -1, q.float().numpy().reshape(24, 128), kp.reshape(6, 351, -1), ksc.reshape(6, 351, -1),
                             vp.reshape(6, 351, -1), vsc.reshape(6, 351, -1), 351, 0.0884, nthreads=8)
    assert np.abs(out_host.float().numpy().reshape(24, 128) - want).max() < 1e-2   # bf16 output rounding


@pytest.mark.parametrize("overlap", [False, True])
def test_host_buffer_modes_give_the_same_bits(overlap):
    """tqb_pqo_cache_decode with host buffers: pinned (mapped) buffers are read and written by the kernel itself,
    pageable ones are staged through copy streams; both must give the bits of the device-buffer call, over several
    layers and steps, with and without overlapping launches."""
    layers, batch, hkv, hq, d, ctx, steps = 3, 4, 2, 8, 128, 700, 3
    g = torch.Generator().manual_seed(9)
    k = torch.randn((batch, hkv, ctx, d), generator=g).bfloat16()
    v = torch.randn((batch, hkv, ctx, d), generator=g).bfloat16()
    nk = torch.randn((steps, layers, batch, hkv, 1, d), generator=g).bfloat16()
    nv = torch.randn((steps, layers, batch, hkv, 1, d), generator=g).bfloat16()
    q = (torch.randn((steps, layers, batch, hq, 1, d), generator=g) / d ** 0.5).bfloat16()
    att = tq.AttendConfig(1.0 / d ** 0.5, hq // hkv)
    outs = {}
    for mode in ("device", "pinned", "pageable"):
        cache = tq.PqoCache(tq.CacheConfig(bits=4, head_dim=d, num_kv_heads=hkv, num_layers=layers, batch=batch))
        cache.set_overlap(overlap)
        for layer in range(layers):
            cache.prefill(layer, k.cuda(), v.cuda())
        conv = {"device": lambda t: t.cuda(), "pinned": lambda t: t.clone().pin_memory(), "pageable": lambda t: t.clone()}[mode]
        res = torch.zeros((steps, layers, batch, hq, 1, d), dtype=torch.bfloat16)
        res = conv(res)
        held = []
        for s_ in range(steps):
            for layer in range(layers):
                args = [conv(nk[s_, layer]), conv(nv[s_, layer]), conv(q[s_, layer])]
                held.append(args)          # host buffers stay alive (and untouched) until host_sync
                cache.decode(layer, *args, att, out=res[s_, layer])
            cache.host_sync()
        torch.cuda.synchronize()
        outs[mode] = res.cpu().clone()
    assert torch.equal(outs["device"], outs["pinned"])
    assert torch.equal(outs["device"], outs["pageable"])
    assert float(outs["device"].float().abs().max()) > 0.0


def test_packed_shard_merge_equals_plain_shard_merge():
    # tqb_lse_combine_packed reads [out | (max, sum)] records, one per shard: the layout of a single all-gather
    g = torch.Generator(device="cuda").manual_seed(5)
    S, hq, D = 3, 16, 128
    outs = torch.randn((S, hq, D), generator=g, device="cuda")
    lses = torch.stack([torch.randn((S, hq), generator=g, device="cuda") * 3, torch.rand((S, hq), generator=g, device="cuda") + 0.5], dim=2)
    want = tq.lse_combine(outs, lses)
    packed = torch.cat([outs.reshape(S, -1), lses.reshape(S, -1)], dim=1).contiguous()
    got = torch.empty((hq, D), dtype=torch.float32, device="cuda")
    assert lib.tqb_lse_combine_packed(packed.data_ptr(), S, hq, D, got.data_ptr(), 0, None) == 0
    torch.cuda.synchronize()
    assert torch.equal(got, want)


@pytest.mark.parametrize("fold", [False, True])
@pytest.mark.parametrize("bits,hq,hkv,past,q_len,dtype,general", [
    (4, 8, 2, 300, 17, torch.bfloat16, False),     # g = 4
    (3, 4, 2, 0, 33, torch.float32, False),        # no past: the first query sees one token
    (4, 16, 2, 1000, 5, torch.float16, False),     # g = 8
    (4, 4, 4, 64, 9, torch.float32, True),         # general kernel
    (3, 6, 2, 129, 12, torch.bfloat16, False),     # g = 3: folded into decode launches whatever `fold` says
    (4, 32, 8, 700, 150, torch.bfloat16, False),   # several row tiles and cache tiles per CTA, ragged ends
    (3, 16, 8, 65, 130, torch.float32, False),     # g = 2, 3-bit
    (4, 2, 2, 40, 200, torch.float32, False),      # g = 1
    (4, 32, 8, 0, 300, torch.bfloat16, False),     # first row tile sees 32 tokens: the second softmax group's tile is all masked
    (3, 32, 8, 4000, 96, torch.float32, False),    # many steps: the stage and buffer rings wrap often
])
def test_chunk_attention_is_causal_decode_per_query_token(bits, hq, hkv, past, q_len, dtype, general, fold):
    # prefill chunk over the packed cache: query token i must equal a decode step that sees past + i + 1 tokens.
    # fold = False: the dedicated tcgen05 kernel where it applies (128 query rows per CTA; P and the dequantized V go
    # through f16, so it agrees with the oracle to a few 1e-4, inside the 2e-3 contract); fold = True: the chunk as
    # one decode grid head per query token (same kernels as decode: a few 1e-5).
    rng = np.random.default_rng(bits * 100 + hq + past + q_len)
    kv_len, stride, d = past + q_len, past + q_len + 7, 128
    k = rng.standard_normal((hkv * stride, d)).astype(np.float32)
    v = rng.standard_normal((hkv * stride, d)).astype(np.float32)
    ki, ks = tq.block_quantize(dev(k), bits)
    vi, vs = tq.block_quantize(dev(v), bits)
    ki, ks, vi, vs = (t.view(hkv, stride, -1) for t in (ki, ks, vi, vs))
    q = torch.from_numpy((rng.standard_normal((q_len, hq, d)) / np.sqrt(d)).astype(np.float32)).to(dtype)
    scale = 1.0 / np.sqrt(d)
    got = tq.chunk_attention(q.cuda(), ki, ks, vi, vs, kv_len, bits, scale, out_dtype=torch.float32,
                             force_general=general, fold=fold).cpu().numpy()
    assert got.shape == (q_len, hq, d)
    kin, ksn, vin, vsn = ki.cpu().numpy(), u16(ks), vi.cpu().numpy(), u16(vs)
    qf = q.float().numpy()
    folded = fold or general or (hq // hkv) not in (1, 2, 4, 8)
    worst = 0.0
    for i in sorted(set(range(0, q_len, max(1, q_len // 24))) | {q_len - 1}):
        want = o.block_attention(bits, d, 0, -1, qf[i], kin, ksn, vin, vsn, past + i + 1, scale, nthreads=4)
        err = float(np.abs(got[i] - want).max())
        worst = max(worst, err)
        assert err < 2e-3, (i, err)
        if folded:
            assert err < 1e-4     # measured: a few 1e-5
    print(f"\n[chunk {q_len} on {past} past tokens, {bits}-bit, g = {hq // hkv}, {'folded' if folded else 'tcgen05 kernel'}] max-abs error {worst:.2e}")
    assert lib.tqb_chunk_umma_timeouts() == 0
    if folded:
        # a chunk of one token is a decode step
        one = tq.chunk_attention(q[-1:].cuda(), ki, ks, vi, vs, kv_len, bits, scale, out_dtype=torch.float32, fold=True).cpu().numpy()
        dec = tq.decode_attention(q[-1].cuda(), ki, ks, vi, vs, kv_len, bits, scale, out_dtype=torch.float32).cpu().numpy()
        assert np.array_equal(one[0], dec)


def test_chunk_attention_argument_errors():
    ki = torch.zeros((2, 16, 64), dtype=torch.uint8, device="cuda")
    ks = torch.zeros((2, 16, 4), dtype=torch.int16, device="cuda")
    q = torch.zeros((9, 4, 128), device="cuda")
    with pytest.raises(tq.RangeOutOfBounds):
        tq.chunk_attention(q, ki, ks, ki, ks, 8, 4, 0.1)     # fewer tokens stored than the chunk holds


@pytest.mark.parametrize("bits", [3, 4])
def test_pqo_cache_prefill_attend_two_chunks_then_decode(bits):
    # batch 2, two prefill chunks with attention inside the cache, then a decode step: every query token equals
    # oracle attention over the oracle-quantized cache truncated at that token (causal)
    b, hkv, hq, d, scale = 2, 2, 8, 128, 0.0884
    cfg = tq.CacheConfig(bits=bits, head_dim=d, num_kv_heads=hkv, num_layers=1, batch=b)
    cache = tq.PqoCache(cfg)
    g = torch.Generator().manual_seed(bits)
    ks_all, vs_all = [], []
    for t in (37, 20):
        k = torch.randn((b, hkv, t, d), generator=g).bfloat16()
        v = torch.randn((b, hkv, t, d), generator=g).bfloat16()
        q = (torch.randn((b, hq, t, d), generator=g) / d ** 0.5).bfloat16()
        past = cache.seq_len(0)
        out = cache.prefill_attend(0, k.cuda(), v.cuda(), q.cuda(), tq.AttendConfig(softmax_scale=scale, n_kv_groups=hq // hkv))
        assert out.shape == (b, hq, t, d) and cache.seq_len(0) == past + t
        ks_all.append(k)
        vs_all.append(v)
        allk = torch.cat(ks_all, dim=2).float().numpy()
        allv = torch.cat(vs_all, dim=2).float().numpy()
        n = allk.shape[2]
        kp, ksc = o.block_quantize(bits, d, 0, -1, allk.reshape(-1, d))
        vp, vsc = o.block_quantize(bits, d, 0, -1, allv.reshape(-1, d))
        kp, ksc, vp, vsc = (a.reshape(b * hkv, n, -1) for a in (kp, ksc, vp, vsc))
        got = out.float().cpu().numpy()
        for i in (0, t // 2, t - 1):
            want = o.block_attention(bits, d, 0, -1, q[:, :, i].float().numpy().reshape(b * hq, d), kp, ksc, vp, vsc,
                                     past + i + 1, scale)
            assert np.abs(got[:, :, i].reshape(b * hq, d) - want).max() < 1e-2   # bf16 output
    k1 = torch.randn((b, hkv, 1, d), generator=g).bfloat16().cuda()
    q1 = (torch.randn((b, hq, 1, d), generator=g) / d ** 0.5).bfloat16().cuda()
    dec = cache.decode(0, k1, k1, q1, tq.AttendConfig(softmax_scale=scale, n_kv_groups=hq // hkv))
    assert dec.is_fused() and cache.seq_len(0) == 58 and torch.isfinite(dec.fused.float()).all()
