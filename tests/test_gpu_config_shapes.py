"""Parity at the shapes and context lengths the benchmark configurations name, through PqoCache.

Each case fills a cache layer with the batched quantize kernel on synthetic K/V of the configuration's
distribution, runs one decode step (append + fused attention), and compares with the CPU oracle's decode
attention over the IDENTICAL packed bytes copied down from the cache (tolerance 2e-3 max-abs, the parity
contract; the observed maximum is printed).  A strided sample of the stored rows is also compared bit for
bit with the oracle's own quantization of the same vectors.
"""
import numpy as np
import pytest
import torch

import oracle_lib as o
import turboquant_b200 as tq
import workloads as w

pytestmark = pytest.mark.gpu
TOL = 2e-3
OUT_TOL = 1e-2   # with bf16 outputs: rounding of the output type on values of magnitude ~1


def _fill_and_decode(shape, layer, ctx, batch=None):
    cfg = w.SHAPES[shape]
    b = cfg["batch"] if batch is None else batch
    dev = torch.device("cuda")
    cache = tq.PqoCache(tq.CacheConfig(bits=cfg["bits"], head_dim=cfg["head_dim"], num_kv_heads=cfg["hkv"], num_layers=1, batch=b))
    k, v = w.synth_kv(shape, layer, ctx, dev, batch=b)
    cache.prefill(0, k[:, :, :ctx - 1].contiguous(), v[:, :, :ctx - 1].contiguous())
    q = w.synth_q(shape, layer, dev, batch=b)[0].float()    # f32 queries and outputs: no output rounding in the way
    scale = 1.0 / cfg["head_dim"] ** 0.5
    out = cache.decode(0, k[:, :, ctx - 1:].float().contiguous(), v[:, :, ctx - 1:].float().contiguous(), q,
                       tq.AttendConfig(scale, cfg["hq"] // cfg["hkv"])).fused
    return cache, k, v, q, out, scale


def _check_rows(cache, cfg, k, v, stride_rows):
    """A strided sample of the stored K and V rows equals the oracle's quantization of the same vectors."""
    ki, ks, vi, vs = (t.numpy() for t in cache.export_layer(0))
    heads, n = ki.shape[0], ki.shape[1]
    rows = np.arange(0, heads * n, stride_rows)
    for src, idx, sc in ((k, ki, ks), (v, vi, vs)):
        x = src.float().reshape(heads * n, -1)[torch.as_tensor(rows, device=src.device)].cpu().numpy()
        op, os_ = o.block_quantize(cfg["bits"], cfg["head_dim"], 0, -1, x, nthreads=16)
        assert np.array_equal(idx.reshape(heads * n, -1)[rows], op)
        assert np.array_equal(sc.reshape(heads * n, -1)[rows].view(np.uint16), os_)


@pytest.mark.parametrize("ctx", [1024, 4096, 32768])
@pytest.mark.parametrize("layer", [0, 1])
def test_qwen3_shape_pqo3(ctx, layer):
    cfg = w.SHAPES["qwen3"]
    cache, k, v, q, out, scale = _fill_and_decode("qwen3", layer, ctx)
    assert cache.seq_len(0) == ctx
    want = w.oracle_decode_of_layer(cache, 0, q, scale)
    err = float(np.abs(out.cpu().numpy().reshape(-1, 128) - want).max())
    print(f"\n[qwen3 shape, PQO3, ctx {ctx}, layer {layer}] max-abs error vs oracle {err:.2e}")
    assert err < TOL
    _check_rows(cache, cfg, k, v, 97)


def test_llama8b_shape_pqo4_batch64_ctx8192():
    cfg = w.SHAPES["llama8b"]
    cache, k, v, q, out, scale = _fill_and_decode("llama8b", 0, 8192)
    want = w.oracle_decode_of_layer(cache, 0, q, scale)
    err = float(np.abs(out.cpu().numpy().reshape(-1, 128) - want).max())
    print(f"\n[llama-3-8b shape, PQO4, batch 64 x ctx 8192] max-abs error vs oracle {err:.2e}")
    assert err < TOL
    _check_rows(cache, cfg, k, v, 4099)
    # bf16 queries and outputs, the dtype the benchmark runs in
    qb = q.to(torch.bfloat16)
    k1, v1 = w.synth_kv("llama8b", 7, 1, torch.device("cuda"))
    outb = cache.decode(0, k1, v1, qb, tq.AttendConfig(scale, 4)).fused
    wantb = w.oracle_decode_of_layer(cache, 0, qb, scale)
    assert float(np.abs(outb.float().cpu().numpy().reshape(-1, 128) - wantb).max()) < OUT_TOL


def test_llama70b_shape_pqo3_ctx131072_unsharded_and_sharded():
    cfg = w.SHAPES["llama70b"]
    ctx = 131072
    cache, k, v, q, out, scale = _fill_and_decode("llama70b", 0, ctx)
    want = w.oracle_decode_of_layer(cache, 0, q, scale)
    err = float(np.abs(out.cpu().numpy().reshape(-1, 128) - want).max())
    print(f"\n[llama-3-70b shape, PQO3, ctx 131072, unsharded] max-abs error vs oracle {err:.2e}")
    assert err < TOL
    _check_rows(cache, cfg, k, v, 9973)
    # the same sequence as 8 token shards: shard-local (out, max, sum), then the log-sum-exp merge
    shards = 8
    outs, lses = [], []
    for r in range(shards):
        lo, hi = r * ctx // shards, (r + 1) * ctx // shards
        c = tq.PqoCache(tq.CacheConfig(bits=3, head_dim=128, num_kv_heads=8, num_layers=1))
        c.prefill(0, k[:, :, lo:hi].contiguous(), v[:, :, lo:hi].contiguous())
        po, pl = c.attend_partial(0, q, scale)
        outs.append(po)
        lses.append(pl)
    merged = tq.lse_combine(torch.stack(outs), torch.stack(lses)).cpu().numpy()
    err = float(np.abs(merged - want).max())
    print(f"[llama-3-70b shape, PQO3, ctx 131072, 8 sequence shards merged] max-abs error vs oracle {err:.2e}")
    assert err < TOL


@pytest.mark.parametrize("bits,layers", [(4, 6), (3, 2), (4, 1)])
def test_overlapped_layer_launches_through_the_cache(bits, layers):
    """PqoCache.set_overlap: the decode launches of successive layers start before their predecessor has finished
    (programmatic dependent launch) and take fewer, longer partitions.  Over several steps (every step appends a row
    that the same layer's next step reads; with one layer two launches in a row hit the same layer and stay ordered)
    the stored bytes must equal those of the ordered run bit for bit, the outputs up to the different split-K
    partitioning (one bf16 rounding step), and the last step must agree with the oracle."""
    hkv, hq, d, batch, ctx = 8, 32, 128, 12, 1500
    g = torch.Generator(device="cuda").manual_seed(7)
    k = torch.randn((batch, hkv, ctx, d), generator=g, device="cuda").to(torch.bfloat16)
    v = torch.randn((batch, hkv, ctx, d), generator=g, device="cuda").to(torch.bfloat16)
    steps = 5
    nk = torch.randn((steps, layers, batch, hkv, 1, d), generator=g, device="cuda").to(torch.bfloat16)
    nv = torch.randn((steps, layers, batch, hkv, 1, d), generator=g, device="cuda").to(torch.bfloat16)
    q = (torch.randn((steps, layers, batch, hq, 1, d), generator=g, device="cuda") / d ** 0.5).to(torch.bfloat16)
    att = tq.AttendConfig(softmax_scale=1.0 / d ** 0.5, n_kv_groups=hq // hkv)
    results = []
    for overlap in (False, True):
        cache = tq.PqoCache(tq.CacheConfig(bits=bits, head_dim=d, num_kv_heads=hkv, num_layers=layers, batch=batch))
        cache.set_overlap(overlap)
        for layer in range(layers):
            cache.prefill(layer, k, v)
        outs = torch.zeros((steps, layers, batch, hq, 1, d), dtype=torch.bfloat16, device="cuda")
        for s in range(steps):
            for layer in range(layers):
                cache.decode(layer, nk[s, layer], nv[s, layer], q[s, layer], att, out=outs[s, layer])
        torch.cuda.synchronize()
        packed = [cache.export_layer(layer) for layer in range(layers)]
        results.append((outs.cpu(), packed))
    for a, b in zip(results[0][1], results[1][1]):
        for x, y in zip(a, b):
            assert np.array_equal(np.asarray(x), np.asarray(y))
    assert float((results[0][0].float() - results[1][0].float()).abs().max()) <= 2.0 ** -7    # one bf16 step at |x| < 2
    want = w.oracle_decode_of_layer(cache, layers - 1, q[steps - 1, layers - 1], 1.0 / d ** 0.5)
    got = results[1][0][steps - 1, layers - 1].float().numpy().reshape(-1, d)
    assert float(np.abs(got - want).max()) < 1e-2     # bf16 outputs


@pytest.mark.parametrize("bits,parts", [(4, 3), (3, 5), (4, 1)])
def test_overlapped_launches_equal_ordered_launches_bit_for_bit(bits, parts):
    """TQB_DECODE_OVERLAP through the plain C entry point: a chain of launches over different caches that share one
    scratch buffer and one output-per-launch, same partition count, once ordered and once overlapped: identical bits
    (the early-started launch must not touch the shared scratch before its predecessor is done with it)."""
    hkv, hq, d, ctx, n = 40, 160, 128, 3000, 6
    g = torch.Generator(device="cuda").manual_seed(11)
    caches = []
    for _ in range(n):
        kv = torch.randn((hkv * ctx, d), generator=g, device="cuda").to(torch.bfloat16)
        ki, ks = tq.block_quantize(kv, bits)
        vi, vs = tq.block_quantize(kv.flip(0).contiguous(), bits)
        caches.append(tuple(t.view(hkv, ctx, -1) for t in (ki, ks, vi, vs)))
    q = (torch.randn((n, hq, d), generator=g, device="cuda") / d ** 0.5).float()
    from turboquant_b200._lib import lib
    scratch = torch.zeros(int(lib.tqb_decode_scratch_bytes(hq, d, parts)), dtype=torch.uint8, device="cuda")
    outs = {}
    for overlap in (False, True):
        o_ = torch.zeros((3, n, hq, d), device="cuda")
        for rep in range(3):
            for i in range(n):
                tq.decode_attention(q[i], *caches[i], ctx, bits, 1.0 / d ** 0.5, num_partitions=parts, scratch=scratch,
                                    out=o_[rep, i], overlap=overlap)
        torch.cuda.synchronize()
        outs[overlap] = o_.cpu()
    assert torch.equal(outs[False], outs[True])
    assert torch.equal(outs[True][0], outs[True][2])


def test_overlapped_launch_after_a_foreign_kernel_sees_its_output():
    """The contract of TQB_DECODE_OVERLAP in a model: q of a layer is written by another kernel (here a torch
    elementwise op on the same stream) launched just before the attention call.  That kernel does not let its
    successor start early, so the overlapped launch is ordered behind it like any other launch and reads the new q."""
    hkv, hq, d, batch, ctx, layers = 8, 32, 128, 4, 900, 5
    g = torch.Generator(device="cuda").manual_seed(3)
    k = torch.randn((batch, hkv, ctx, d), generator=g, device="cuda").to(torch.bfloat16)
    nk = torch.randn((batch, hkv, 1, d), generator=g, device="cuda").to(torch.bfloat16)
    q0 = (torch.randn((batch, hq, 1, d), generator=g, device="cuda") / d ** 0.5).float()
    att = tq.AttendConfig(softmax_scale=1.0 / d ** 0.5, n_kv_groups=hq // hkv)
    res = []
    for overlap in (False, True):
        cache = tq.PqoCache(tq.CacheConfig(bits=4, head_dim=d, num_kv_heads=hkv, num_layers=layers, batch=batch))
        cache.set_overlap(overlap)
        for layer in range(layers):
            cache.prefill(layer, k, k)
        outs = []
        x = q0.clone()
        for step in range(3):
            for layer in range(layers):
                x = x * 0.999 + 0.001 * (layer + 1)            # the "projection": a kernel that writes this layer's q
                outs.append(cache.decode(layer, nk, nk, x, att).fused.clone())
        torch.cuda.synchronize()
        res.append(torch.stack(outs).cpu())
    assert float((res[0] - res[1]).abs().max()) < 1e-5          # same inputs; only the split-K partitioning differs
