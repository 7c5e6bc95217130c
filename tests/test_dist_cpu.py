"""Host-side logic of the multi-GPU paths on CPU ranks (gloo, world size 2): unit sharding and the
gather + log-sum-exp merge of sequence shards.  The shard-local partials are produced with numpy
from the oracle's dequantized K/V; the exchange itself is the code the GPU path uses."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle_lib as o


def _load_dist_module():
    # loaded by path: the package import needs the CUDA library, this module does not
    import importlib.util
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("tqb_dist", os.path.join(root, "turboquant_b200", "dist.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_shard_range_covers_everything_once():
    d = _load_dist_module()
    for n in (0, 1, 7, 8, 512, 513):
        for world in (1, 2, 3, 8):
            spans = [d.shard_range(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        d.shard_range(4, 2, 2)


def _partial(q, k, v, scale):
    """Un-normalised attention of one shard: (out [Hq, D], lse [Hq, 2]) with GQA head mapping."""
    hq, hkv = q.shape[0], k.shape[0]
    g = hq // hkv
    out = np.zeros((hq, q.shape[1]), np.float32)
    lse = np.zeros((hq, 2), np.float32)
    for h in range(hq):
        kk, vv = k[h // g], v[h // g]
        if len(kk) == 0:
            lse[h] = (-3.4e38, 0.0)
            continue
        s = (kk @ q[h]) * scale
        m = s.max()
        p = np.exp(s - m)
        out[h], lse[h] = p @ vv, (m, p.sum())
    return out, lse


def _combine(outs, lses):
    m = lses[:, :, 0].max(0)
    w = np.exp(lses[:, :, 0] - m)
    den = (lses[:, :, 1] * w).sum(0)
    return (outs * w[:, :, None]).sum(0) / den[:, None]


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    d = _load_dist_module()
    rng = np.random.default_rng(0)                      # same data on every rank
    hq, hkv, L, D = 8, 2, 301, 128
    k = rng.standard_normal((hkv * L, D)).astype(np.float32)
    v = rng.standard_normal((hkv * L, D)).astype(np.float32)
    q = (rng.standard_normal((hq, D)) / np.sqrt(D)).astype(np.float32)
    kd = o.block_dequantize(3, D, 0, -1, *o.block_quantize(3, D, 0, -1, k)).reshape(hkv, L, D)
    vd = o.block_dequantize(3, D, 0, -1, *o.block_quantize(3, D, 0, -1, v)).reshape(hkv, L, D)
    lo, hi = d.shard_range(L, world, rank)
    out, lse = _partial(q, kd[:, lo:hi], vd[:, lo:hi], 0.0884)
    outs, lses = d.gather_partials(torch.from_numpy(out), torch.from_numpy(lse))
    merged = _combine(outs.numpy(), lses.numpy())
    want = o.sdpa(q, kd, vd, 0.0884)
    err = float(np.abs(merged - want).max())
    # the packed form used by SequenceParallelDecoder: one flat record per rank, ONE all-gather
    rec = torch.from_numpy(np.concatenate([out.ravel(), lse.ravel()]))
    gathered = torch.empty((world * rec.numel(),), dtype=torch.float32)
    dist.all_gather_into_tensor(gathered, rec)
    g = gathered.numpy().reshape(world, -1)
    merged2 = _combine(g[:, :hq * D].reshape(world, hq, D), g[:, hq * D:].reshape(world, hq, 2))
    ret[rank] = max(err, float(np.abs(merged2 - want).max()))
    dist.barrier()
    dist.destroy_process_group()


def test_sequence_shards_gather_and_merge_on_two_gloo_ranks():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ret = mp.get_context("spawn").Manager().dict()
    mp.spawn(_worker, args=(2, port, ret), nprocs=2, join=True)
    assert len(ret) == 2 and all(err < 1e-5 for err in ret.values()), dict(ret)
