"""Synthetic stand-ins for the benchmark configurations (shapes, sizes and value distributions only; no
dataset items): shared by bench.py and the parity tests at those shapes.

  qwen3   PQO3, 28 layers, 16 query / 8 KV heads, head_dim 128, batch 1, context 1K .. 32K;
          K/V bf16 N(0,1) with 2 % of the channels (3 of 128, fixed per layer) scaled by 8.
  llama8b PQO4, 32 layers, 32 / 8 heads, batch 64, context 8,192; K/V bf16 N(0,1) times a per-channel
          log-normal(0, 0.5) scale (one scale vector per layer and per K / V).
  llama70b PQO3, 80 layers, 64 / 8 heads, batch 1, context 131,072; outlier channels as qwen3.
Queries are N(0,1) / sqrt(128) and softmax_scale = 1 / sqrt(128) everywhere.
"""
import numpy as np
import torch

SHAPES = {
    "qwen3": dict(bits=3, layers=28, hq=16, hkv=8, head_dim=128, batch=1, style="outlier"),
    "llama8b": dict(bits=4, layers=32, hq=32, hkv=8, head_dim=128, batch=64, style="lognormal"),
    "llama70b": dict(bits=3, layers=80, hq=64, hkv=8, head_dim=128, batch=1, style="outlier"),
}


def synth_kv(shape, layer, tokens, device, batch=None):
    """K, V bf16 [batch, hkv, tokens, D] of one layer, seeded by the layer index."""
    cfg = SHAPES[shape]
    b = cfg["batch"] if batch is None else batch
    d = cfg["head_dim"]
    g = torch.Generator(device=device).manual_seed(42 + layer)
    dims = (b, cfg["hkv"], tokens, d)
    if cfg["style"] == "lognormal":
        ks = torch.exp(torch.randn(d, generator=g, device=device) * 0.5)
        vs = torch.exp(torch.randn(d, generator=g, device=device) * 0.5)
    else:
        ch = np.random.default_rng(42 + layer).choice(d, 3, replace=False)
        ks = torch.ones(d, device=device)
        ks[torch.as_tensor(ch, device=device)] = 8.0
        vs = ks
    k = (torch.randn(dims, generator=g, device=device) * ks).to(torch.bfloat16)
    v = (torch.randn(dims, generator=g, device=device) * vs).to(torch.bfloat16)
    return k, v


def synth_q(shape, seed, device, batch=None, count=1):
    cfg = SHAPES[shape]
    b = cfg["batch"] if batch is None else batch
    g = torch.Generator(device=device).manual_seed(1234 + seed)
    q = torch.randn((count, b, cfg["hq"], 1, cfg["head_dim"]), generator=g, device=device) / cfg["head_dim"] ** 0.5
    return q.to(torch.bfloat16)


def oracle_decode_of_layer(cache, layer, q, softmax_scale, nthreads=16):
    """The CPU oracle's decode attention over the IDENTICAL packed bytes of one cache layer.
    q: [batch, Hq, 1, D] tensor; returns [batch * Hq, D] f32."""
    import oracle_lib as o
    cfg = cache.config
    ki, ks, vi, vs = (t.numpy() for t in cache.export_layer(layer, host=True))
    n = cache.seq_len(layer)
    qf = q.float().cpu().numpy().reshape(-1, cfg.head_dim)
    return o.block_attention(cfg.bits, cfg.head_dim, int(cfg.norm_mode), cfg.outlier_blocks, qf, ki, ks.view(np.uint16), vi,
                             vs.view(np.uint16), n, softmax_scale, nthreads=nthreads)
