"""GPU parity of TqCache (block-32 polar codes + head_dim-wide QJL sketch of the key residual,
src/cache/tq.rs) against a composition of the CPU oracle's pieces."""
import numpy as np
import pytest
import torch

import oracle_lib as o
import turboquant_b200 as tq

pytestmark = pytest.mark.gpu
QJL_SEED = 12345   # src/cache/config.rs:18


def seq_norm_f16(r):
    s = np.float32(0)
    for x in r.astype(np.float32):
        s = np.float32(s + np.float32(x * x))
    return o.f32_to_f16_bits(float(np.sqrt(s)))


def oracle_tq(k, bits, D):
    """packed, scales, dequantized, signs, norms of keys [n, D] (outlier_blocks = 0)."""
    kp, ks = o.block_quantize(bits, D, 0, 0, k)
    kd = o.block_dequantize(bits, D, 0, 0, kp, ks)
    res = k - kd
    signs = np.stack([o.qjl_signs(r, D, QJL_SEED) for r in res])
    norms = np.array([seq_norm_f16(r) for r in res], np.uint16)
    return kp, ks, kd, signs, norms


def oracle_bias(q, signs, norms, D):
    """q [Hq, q_len, D]; signs [Hkv, L, D/8]; norms [Hkv, L] -> [Hq, q_len, L]."""
    hq, q_len = q.shape[:2]
    hkv, L = norms.shape
    g = hq // hkv
    pm = np.where(np.unpackbits(signs, axis=-1, bitorder="little") == 1, 1.0, -1.0).astype(np.float32)   # [Hkv, L, D]
    c = np.array([[o.f16_bits_to_f32(n) for n in row] for row in norms], np.float32) * (
        np.float32(np.sqrt(np.pi / 2)) / np.sqrt(np.float32(D)))
    out = np.zeros((hq, q_len, L), np.float32)
    for h in range(hq):
        for i in range(q_len):
            rq = o.query_projections(q[h, i], D, QJL_SEED)
            out[h, i] = (pm[h // g] @ rq) * c[h // g]
    return out


@pytest.mark.parametrize("bits", [3, 4])
def test_tq_cache_prefill_decode_and_bias(bits):
    D, hkv, hq = 128, 2, 4
    cfg = tq.CacheConfig(bits=bits, head_dim=D, num_kv_heads=hkv, num_layers=2, outlier_blocks=0)
    assert cfg.qjl_enabled()
    cache = tq.TqCache(cfg)
    g = torch.Generator().manual_seed(bits)
    k1, v1 = torch.randn((1, hkv, 21, D), generator=g), torch.randn((1, hkv, 21, D), generator=g)
    q1 = torch.randn((1, hq, 3, D), generator=g) / D ** 0.5
    r = cache.prefill(0, k1.cuda(), v1.cuda(), q1.cuda())
    assert r.logit_bias is not None and r.logit_bias.shape == (1, hq, 3, 21)     # tests/cache_type_correctness.rs:68-199
    assert torch.equal(r.k.cpu(), k1)                                            # first prefill returns the originals
    kp, ks, kd, signs, norms = oracle_tq(k1.numpy().reshape(-1, D), bits, D)
    want = oracle_bias(q1.numpy()[0], signs.reshape(hkv, 21, -1), norms.reshape(hkv, 21), D)
    assert np.abs(r.logit_bias.cpu().numpy()[0] - want).max() < 1e-5
    # decode: one more token, Dequantized result over all 22 tokens
    k2, v2 = torch.randn((1, hkv, 1, D), generator=g), torch.randn((1, hkv, 1, D), generator=g)
    q2 = torch.randn((1, hq, 1, D), generator=g) / D ** 0.5
    d = cache.decode(0, k2.cuda(), v2.cuda(), q2.cuda())
    assert not d.is_fused() and d.dequantized.k.shape == (1, hkv, 22, D) and d.dequantized.logit_bias.shape == (1, hq, 1, 22)
    allk = torch.cat([k1, k2], dim=2).numpy().reshape(-1, D)
    allv = torch.cat([v1, v2], dim=2).numpy().reshape(-1, D)
    kp, ks, kd, signs, norms = oracle_tq(allk, bits, D)
    assert np.array_equal(d.dequantized.k.cpu().numpy().reshape(-1, D), kd)
    vp, vs = o.block_quantize(bits, D, 0, 0, allv)
    assert np.array_equal(d.dequantized.v.cpu().numpy().reshape(-1, D), o.block_dequantize(bits, D, 0, 0, vp, vs))
    want = oracle_bias(q2.numpy()[0], signs.reshape(hkv, 22, -1), norms.reshape(hkv, 22), D)
    assert np.abs(d.dequantized.logit_bias.cpu().numpy()[0] - want).max() < 1e-5
    # the stored sketch is bit-identical to the oracle's
    import ctypes
    from turboquant_b200._lib import lib
    sp, npn, cap = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_int64()
    assert lib.tqb_tq_cache_qjl_ptrs(cache._h, 0, ctypes.byref(sp), ctypes.byref(npn), ctypes.byref(cap)) == 0
    assert cap.value == 21 + 128                                               # src/cache/tq.rs:75-77
    # fused alternative: third token, attention with the in-kernel correction
    k3, v3 = torch.randn((1, hkv, 1, D), generator=g), torch.randn((1, hkv, 1, D), generator=g)
    q3 = torch.randn((1, hq, 1, D), generator=g) / D ** 0.5
    f = cache.decode_fused(0, k3.cuda(), v3.cuda(), q3.cuda(), tq.AttendConfig(0.0884))
    assert f.is_fused() and f.fused.shape == (1, hq, 1, D)
    allk = np.concatenate([allk.reshape(hkv, 22, D), k3.numpy()[0]], axis=1).reshape(-1, D)
    allv = np.concatenate([allv.reshape(hkv, 22, D), v3.numpy()[0]], axis=1).reshape(-1, D)
    kp, ks, kd, signs, norms = oracle_tq(allk, bits, D)
    vp, vs = o.block_quantize(bits, D, 0, 0, allv)
    qn = q3.numpy()[0, :, 0]
    rq = np.stack([o.query_projections(x, D, QJL_SEED) for x in qn])
    want = o.block_attention(bits, D, 0, 0, qn, kp.reshape(hkv, 23, -1), ks.reshape(hkv, 23, -1), vp.reshape(hkv, 23, -1),
                             vs.reshape(hkv, 23, -1), 23, 0.0884, qjl=(signs.reshape(hkv, 23, -1), norms.reshape(hkv, 23), rq))
    assert np.abs(f.fused.cpu().numpy()[0, :, 0] - want).max() < 2e-3
    assert cache.seq_len(0) == 23 and cache.seq_len(1) == 0
    pd = D * bits // 8
    assert cache.memory_usage() == 2 * hkv * 23 * pd + 2 * hkv * 23 * 4 * 2 + hkv * (21 + 128) * (D // 8 + 2)
    cache.reset()
    assert cache.seq_len(0) == 0 and cache.memory_usage() == 0


def test_pqo_has_no_bias_and_tq_rejects_odd_head_dims():
    pqo = tq.PqoCache(tq.CacheConfig(bits=3, head_dim=128, num_kv_heads=1, num_layers=1))
    k = torch.randn((1, 1, 4, 128)).cuda()
    assert pqo.prefill(0, k, k).logit_bias is None
    with pytest.raises(tq.TqbRuntimeError):
        tq.TqCache(tq.CacheConfig(bits=3, head_dim=96, num_kv_heads=1, num_layers=1, outlier_blocks=0))


def test_residual_sketch_batch_and_growth():
    # batch folds into heads; the sketch arrays regrow with the reference's rule and keep old rows
    D = 64
    cfg = tq.CacheConfig(bits=4, head_dim=D, num_kv_heads=2, num_layers=1, outlier_blocks=0, batch=2)
    cache = tq.TqCache(cfg)
    g = torch.Generator().manual_seed(9)
    ks_ = []
    for n in (130, 40, 300):
        k = torch.randn((2, 2, n, D), generator=g)
        q = torch.randn((2, 4, 1, D), generator=g)
        r = cache.prefill(0, k.cuda(), k.cuda(), q.cuda())
        ks_.append(k)
    allk = torch.cat(ks_, dim=2).numpy()               # [2, 2, 470, D]
    kp, ks, kd, signs, norms = oracle_tq(allk.reshape(-1, D), 4, D)
    want = oracle_bias(q.numpy().reshape(8, 1, D), signs.reshape(4, 470, -1), norms.reshape(4, 470), D)
    assert np.abs(r.logit_bias.cpu().numpy().reshape(8, 1, 470) - want).max() < 1e-5
    assert np.array_equal(r.k.cpu().numpy().reshape(-1, D), kd)
