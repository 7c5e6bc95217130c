"""Sequence-parallel decode with the exchange fused into the attention kernel (tqb_peer_exchange_*).

On one GPU the ranks are emulated by ONE process, one after the other on one stream: every rank's attention kernel
(with its pushes) is enqueued before any combine kernel, so a combine kernel finds its flags set and never waits for
a kernel that has not run.  The bounded wait is made to run out by a rank that never pushes: the combine kernel
gives up after a short limit, counts the time-out and returns; the context stays usable.  With two or more GPUs the
same path runs as one process per GPU, the IPC handles exchanged through a gloo group.
"""
import ctypes
import os
import socket

import numpy as np
import pytest
import torch

import turboquant_b200 as tq
import workloads as w
from turboquant_b200._lib import lib

pytestmark = pytest.mark.gpu


def _shards(world, ctx, bits, hq, hkv, seed):
    """A cache per emulated rank holding its token shard, the unsharded cache, and a query."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    k = torch.randn((1, hkv, ctx, 128), generator=g, device="cuda").to(torch.bfloat16)
    v = torch.randn((1, hkv, ctx, 128), generator=g, device="cuda").to(torch.bfloat16)
    q = (torch.randn((1, hq, 1, 128), generator=g, device="cuda") / 128 ** 0.5).float()
    cfg = dict(bits=bits, head_dim=128, num_kv_heads=hkv, num_layers=1)
    full = tq.PqoCache(tq.CacheConfig(**cfg))
    full.prefill(0, k, v)
    caches = []
    for r in range(world):
        lo, hi = r * ctx // world, (r + 1) * ctx // world
        c = tq.PqoCache(tq.CacheConfig(**cfg))
        c.prefill(0, k[:, :, lo:hi].contiguous(), v[:, :, lo:hi].contiguous())
        caches.append(c)
    return full, caches, q


def _exchanges(world, hq):
    xs = [ctypes.c_void_p() for _ in range(world)]
    for r in range(world):
        assert lib.tqb_peer_exchange_create(world, r, hq, 128, ctypes.byref(xs[r])) == 0
    arr = (ctypes.c_void_p * world)(*[x.value for x in xs])
    for r in range(world):
        assert lib.tqb_peer_exchange_connect_local(xs[r], arr) == 0
    return xs


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("bits,hq,hkv,world,ctx", [(3, 64, 8, 4, 8192), (4, 32, 8, 2, 3001), (3, 16, 8, 8, 4096), (3, 8, 8, 3, 1000)])
def test_emulated_ranks_push_and_combine(bits, hq, hkv, world, ctx):
    full, caches, q = _shards(world, ctx, bits, hq, hkv, seed=bits * 100 + world)
    scale = 1.0 / 128 ** 0.5
    want = w.oracle_decode_of_layer(full, 0, q, scale)
    xs = _exchanges(world, hq)
    outs = [torch.full((hq, 128), float("nan"), device="cuda") for _ in range(world)]
    for step in range(3):     # several steps: the record slots rotate, the flags count up
        for r in range(world):
            assert lib.tqb_pqo_cache_attend_push(caches[r]._h, 0, q.data_ptr(), 0, hq, scale, xs[r], _stream()) == 0
        for r in range(world):
            assert lib.tqb_peer_exchange_combine(xs[r], hkv, outs[r].data_ptr(), 0, 1 << 24, _stream()) == 0
        torch.cuda.synchronize()
        for r in range(world):
            err = float(np.abs(outs[r].cpu().numpy() - want).max())
            assert err < 2e-3, (step, r, err)
            assert torch.equal(outs[r], outs[0])          # every rank merges the same records in the same order
    for x in xs:
        assert lib.tqb_peer_exchange_timeouts(x) == 0 and lib.tqb_peer_exchange_check(x) == 0
        lib.tqb_peer_exchange_destroy(x)


def test_bounded_wait_runs_out_when_a_rank_never_pushes():
    world, hq, hkv = 2, 16, 8
    full, caches, q = _shards(world, 2048, 3, hq, hkv, seed=5)
    xs = _exchanges(world, hq)
    out = torch.full((hq, 128), float("nan"), device="cuda")
    # only rank 0 pushes; rank 1's flags stay behind
    assert lib.tqb_pqo_cache_attend_push(caches[0]._h, 0, q.data_ptr(), 0, hq, 0.0884, xs[0], _stream()) == 0
    t0 = torch.cuda.Event(True); t1 = torch.cuda.Event(True)
    t0.record()
    assert lib.tqb_peer_exchange_combine(xs[0], hkv, out.data_ptr(), 0, 1 << 21, _stream()) == 0   # ~1 ms limit
    t1.record()
    torch.cuda.synchronize()                                   # returns: the kernel did not hang
    assert t0.elapsed_time(t1) < 500.0
    assert torch.all(out == 0)
    assert lib.tqb_peer_exchange_timeouts(xs[0]) == hq         # one per combine CTA
    assert lib.tqb_peer_exchange_check(xs[0]) == 13            # TQB_ERR_PEER_TIMEOUT
    from turboquant_b200.api import PeerTimeout, check
    with pytest.raises(PeerTimeout):
        check(13)
    # the context is still usable, and a complete step afterwards is correct
    want = w.oracle_decode_of_layer(full, 0, q, 0.0884)
    assert lib.tqb_pqo_cache_attend_push(caches[1]._h, 0, q.data_ptr(), 0, hq, 0.0884, xs[1], _stream()) == 0
    assert lib.tqb_peer_exchange_combine(xs[0], hkv, out.data_ptr(), 0, 1 << 24, _stream()) == 0
    torch.cuda.synchronize()
    assert float(np.abs(out.cpu().numpy() - want).max()) < 2e-3
    for x in xs:
        lib.tqb_peer_exchange_destroy(x)


def test_argument_checks():
    x = ctypes.c_void_p()
    assert lib.tqb_peer_exchange_create(9, 0, 8, 128, ctypes.byref(x)) == 7      # more than 8 ranks
    assert lib.tqb_peer_exchange_create(2, 2, 8, 128, ctypes.byref(x)) == 7      # rank outside the world
    assert lib.tqb_peer_exchange_create(2, 0, 8, 64, ctypes.byref(x)) == 9       # head_dim the pushing kernels do not cover
    assert lib.tqb_peer_exchange_create(2, 0, 8, 128, ctypes.byref(x)) == 0
    out = torch.zeros((8, 128), device="cuda")
    assert lib.tqb_peer_exchange_combine(x, 8, out.data_ptr(), 0, 1 << 20, None) == 7   # not connected, no step begun
    lib.tqb_peer_exchange_destroy(x)


def _rank_main(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch.distributed as dist
    from turboquant_b200.dist import FusedSequenceParallelDecoder, shard_range
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)     # host-side plumbing only: the IPC handles
    hq, hkv, ctx, bits = 64, 8, 16384, 3
    g = torch.Generator(device="cuda").manual_seed(11)
    k = torch.randn((1, hkv, ctx, 128), generator=g, device="cuda").to(torch.bfloat16)
    v = torch.randn((1, hkv, ctx, 128), generator=g, device="cuda").to(torch.bfloat16)
    q = (torch.randn((1, hq, 1, 128), generator=g, device="cuda") / 128 ** 0.5).float()
    lo, hi = shard_range(ctx, world, rank)
    cache = tq.PqoCache(tq.CacheConfig(bits=bits, head_dim=128, num_kv_heads=hkv, num_layers=1))
    cache.prefill(0, k[:, :, lo:hi].contiguous(), v[:, :, lo:hi].contiguous())
    dec = FusedSequenceParallelDecoder(cache, hq)
    out = None
    for _ in range(5):          # several layers' worth of steps: slots rotate, ranks may run one step apart
        out = dec.attend(0, q, 0.0884)
    torch.cuda.synchronize()
    dec.check()
    ret[rank] = out.cpu().numpy()
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_processes_two_gpus():
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ret = mp.get_context("spawn").Manager().dict()
    mp.spawn(_rank_main, args=(2, port, ret), nprocs=2, join=True)
    assert len(ret) == 2
    assert np.array_equal(ret[0], ret[1])
    # the same data, unsharded, through the oracle
    hq, hkv, ctx = 64, 8, 16384
    g = torch.Generator(device="cuda").manual_seed(11)
    k = torch.randn((1, hkv, ctx, 128), generator=g, device="cuda").to(torch.bfloat16)
    v = torch.randn((1, hkv, ctx, 128), generator=g, device="cuda").to(torch.bfloat16)
    q = (torch.randn((1, hq, 1, 128), generator=g, device="cuda") / 128 ** 0.5).float()
    full = tq.PqoCache(tq.CacheConfig(bits=3, head_dim=128, num_kv_heads=hkv, num_layers=1))
    full.prefill(0, k, v)
    want = w.oracle_decode_of_layer(full, 0, q, 0.0884)
    assert float(np.abs(ret[0] - want).max()) < 2e-3
