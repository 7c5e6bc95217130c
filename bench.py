#!/usr/bin/env python3
"""Benchmark of the hot path: batched decode attention over the packed block-32 KV cache.

Workload (the largest single-GPU configuration of the baseline): Llama-3-8B-shaped PQO4
batched decode -- 32 layers, 32 query heads, 8 KV heads (GQA 4), head_dim 128, batch 64,
context 8,192; K/V bf16 N(0,1) with per-channel log-normal(0, 0.5) scales (synthetic; seeds
42 + layer); the cache is filled by the batched quantize kernel, then decode steps run.
A step = one new token for each of the 64 sequences through all 32 layers
(append-quantize + fused attention per layer).  Scaling is weak: every rank holds its own
batch-64 cache, sharded by (batch, KV head) with no collective on the data path.

metric  = effective HBM GB/s: algorithmic compressed bytes read (2 * (64 + 8) = 144 B per
          token per KV head per layer) / time, whole job.
value   = steps with all inputs resident in HBM, CUDA-event timed.
e2e     = the same steps through PqoCache.decode with HOST (pinned) k, v, q buffers and
          the output read back to the host, copies inside the timed region.
roofline= the decode kernel alone: algorithmic bytes per launch / mean launch duration,
          measured with CUDA events around single launches.
--impl reference: the CPU restatement of the reference (the oracle) on the host cores.
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import numpy as np  # noqa: E402
import torch  # noqa: E402

CFG = dict(layers=32, hq=32, hkv=8, head_dim=128, batch=64, ctx=8192, bits=4)
WORKLOAD = "llama3-8b-shaped PQO4 batched decode: 32 layers, 32 q heads, 8 kv heads, head_dim 128, batch 64, ctx 8192"
METRIC = "decode_attn_effective_hbm_gbps"
def bytes_per_token_head():
    """Algorithmic bytes of one (token, KV head): packed K and V codes plus their four f16 scales each (144 B for PQO4)."""
    return 2 * (CFG["head_dim"] * CFG["bits"] // 8 + (CFG["head_dim"] // 32) * 2)


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return float(json.load(open(path))["hbm_gbs"]), "measured (MEASURED_PEAKS.json, copy bandwidth)"
    return 6650.0, "fallback (earlier measurement on this pool)"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.rows, self.proc, self.gpu = [], None, gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        sm = [float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        reasons = set()
        for r in self.rows:
            if len(r) >= 9:
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def synth_layer(layer, tokens, device):
    """K, V bf16 [batch, hkv, tokens, D]: N(0,1) times a per-channel log-normal(0, 0.5) scale."""
    g = torch.Generator(device=device).manual_seed(42 + layer)
    shape = (CFG["batch"], CFG["hkv"], tokens, CFG["head_dim"])
    ks = torch.exp(torch.randn(CFG["head_dim"], generator=g, device=device) * 0.5)
    vs = torch.exp(torch.randn(CFG["head_dim"], generator=g, device=device) * 0.5)
    k = (torch.randn(shape, generator=g, device=device) * ks).to(torch.bfloat16)
    v = (torch.randn(shape, generator=g, device=device) * vs).to(torch.bfloat16)
    return k, v


def run_ours(args):
    import turboquant_b200 as tq
    from turboquant_b200._lib import lib

    rank = int(os.environ.get("RANK", 0))
    local = int(os.environ.get("LOCAL_RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    L, B, HQ, HKV, D, CTX, BITS = (CFG[k] for k in ("layers", "batch", "hq", "hkv", "head_dim", "ctx", "bits"))
    scale = 1.0 / np.sqrt(D)
    cache = tq.PqoCache(tq.CacheConfig(bits=BITS, head_dim=D, num_kv_heads=HKV, num_layers=L, batch=B))
    att = tq.AttendConfig(softmax_scale=scale, n_kv_groups=HQ // HKV)

    # ---- fill the cache with the batched quantize kernel ----
    # The bulk-quantize figure is taken on the last layer's K/V into buffers allocated beforehand (a cache
    # fill also allocates and clears the layer's storage, which is not the kernel's time).
    nvec = 2 * B * HKV * CTX
    quant_bytes = nvec * (D * 2 + D * BITS // 8 + (D // 32) * 2)
    qt = []
    for layer in range(L):
        k, v = synth_layer(layer, CTX, dev)
        cache.prefill(layer, k, v)
        if layer == L - 1:
            rows = B * HKV * CTX
            qi = torch.empty((2, rows, D * BITS // 8), dtype=torch.uint8, device=dev)
            qs_ = torch.empty((2, rows, D // 32), dtype=torch.int16, device=dev)
            for rep in range(4):
                e0, e1 = torch.cuda.Event(True), torch.cuda.Event(True)
                e0.record()
                rc = lib.tqb_block_quantize_pair(BITS, D, 0, -1, k.data_ptr(), v.data_ptr(), 2, rows, 0, qi[0].data_ptr(),
                                                 qs_[0].data_ptr(), qi[1].data_ptr(), qs_[1].data_ptr(), 0, 0, 0,
                                                 ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
                e1.record()
                assert rc == 0, rc
                e1.synchronize()
                if rep:
                    qt.append(e0.elapsed_time(e1))
            del qi, qs_
        del k, v
    quant_ms = float(np.median(qt))

    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    n_tok = args.warmup + args.steps + 2 * (args.warmup + args.steps) + 4
    newk = torch.randn((4, B, HKV, 1, D), generator=g, device=dev).to(torch.bfloat16)
    newv = torch.randn((4, B, HKV, 1, D), generator=g, device=dev).to(torch.bfloat16)
    qs = (torch.randn((4, B, HQ, 1, D), generator=g, device=dev) * scale).to(torch.bfloat16)
    outs = torch.empty((L, B, HQ, 1, D), dtype=torch.bfloat16, device=dev)
    assert cache.capacity(0) >= CTX + n_tok, "decode steps would force a cache re-allocation inside the timed region"

    def step_device(i):
        for layer in range(L):
            cache.decode(layer, newk[i % 4], newv[i % 4], qs[(i + layer) % 4], att, out=outs[layer])

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def bytes_of_steps(first_len, nsteps):
        # each step attends over the cache after its own append
        return sum(L * B * HKV * (first_len + 1 + s) * bytes_per_token_head() for s in range(nsteps))

    # ---- value: device-resident steps ----
    for i in range(args.warmup):
        step_device(i)
    barrier()
    len0 = cache.seq_len(0)
    sampler = ClockSampler(local)
    sampler.start()
    e0, e1 = torch.cuda.Event(True), torch.cuda.Event(True)
    e0.record()
    for i in range(args.steps):
        step_device(i)
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop()
    step_bytes = bytes_of_steps(len0, args.steps)

    # ---- e2e: host buffers through PqoCache.decode ----
    hk = [newk[i].cpu().pin_memory() for i in range(4)]
    hv = [newv[i].cpu().pin_memory() for i in range(4)]
    hq_ = [qs[i].cpu().pin_memory() for i in range(4)]
    hout = torch.empty((L, B, HQ, 1, D), dtype=torch.bfloat16).pin_memory()

    def step_host(i):
        for layer in range(L):
            cache.decode(layer, hk[i % 4], hv[i % 4], hq_[(i + layer) % 4], att, out=hout[layer])
        cache.host_sync()   # the step's results are on the host

    for i in range(args.warmup):
        step_host(i)
    barrier()
    len1 = cache.seq_len(0)
    f0, f1 = torch.cuda.Event(True), torch.cuda.Event(True)
    f0.record()
    for i in range(args.steps):
        step_host(i)
    f1.record()
    barrier()
    e2e_ms = f0.elapsed_time(f1)
    e2e_bytes = bytes_of_steps(len1, args.steps)
    h2d = world * L * (2 * B * HKV * D + B * HQ * D) * 2    # whole job, like the value
    d2h = world * L * B * HQ * D * 2

    # ---- roofline: the decode kernel alone, one event pair per launch ----
    kv_len = cache.seq_len(0)
    nheads = B * HKV
    parts = int(lib.tqb_decode_num_partitions(nheads, kv_len))
    scratch = torch.empty(int(lib.tqb_decode_scratch_bytes(B * HQ, D, parts)), dtype=torch.uint8, device=dev)
    q2 = qs[0].reshape(B * HQ, D)
    dummy = torch.empty((B * HQ, D), dtype=torch.bfloat16, device=dev)
    stride = cache.capacity(0)
    from turboquant_b200._lib import TqbDecodeParams
    durs = []
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for rep in range(2):
        for layer in range(L):
            p = TqbDecodeParams()
            p.k_indices, p.k_scales, p.v_indices, p.v_scales = cache.layer_ptrs(layer)
            p.q, p.out, p.scratch, p.scratch_bytes = q2.data_ptr(), dummy.data_ptr(), scratch.data_ptr(), scratch.numel()
            p.q_dtype = p.out_dtype = 2
            p.bits, p.head_dim, p.norm_mode, p.outlier_blocks = BITS, D, 0, -1
            p.num_q_heads, p.num_kv_heads, p.kv_len, p.kv_stride = B * HQ, nheads, kv_len, stride
            p.num_partitions, p.softmax_scale, p.flags = parts, scale, 1     # split-K pass only
            s0, s1 = torch.cuda.Event(True), torch.cuda.Event(True)
            s0.record()
            rc = lib.tqb_decode_attention(ctypes.byref(p), stream)
            s1.record()
            assert rc == 0, rc
            s1.synchronize()
            if rep == 1:
                durs.append(s0.elapsed_time(s1))
    launch_ms = float(np.mean(durs))
    launch_bytes = nheads * kv_len * bytes_per_token_head()
    peak, peak_src = peaks()

    # ---- max over ranks ----
    if dist is not None:
        t = torch.tensor([ms, e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = t.tolist()
    total_bytes = step_bytes * world
    value = total_bytes / (ms * 1e-3) / 1e9
    e2e_value = e2e_bytes * world / (e2e_ms * 1e-3) / 1e9

    line = None
    if rank == 0:
        achieved = launch_bytes / (launch_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": round(value, 2), "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms / args.steps, 4), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "format": "PQO4 block-32 MaxNorm", "kv_dtype": "bf16",
                       "l2": "inputs larger than L2 (19.3 GB packed cache per GPU)", "sharding": "(batch, kv head), no collective"},
            "tokens_per_s": round(B * world * args.steps / (ms * 1e-3), 1),
            "pct_of_hbm_peak": round(100 * value / (peak * world), 2),
            "e2e": {"value": round(e2e_value, 2), "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "tokens_per_s": round(B * world * args.steps / (e2e_ms * 1e-3), 1)},
            "gpu_launches": args.steps * L,   # per layer: one kernel (append of the new token, attention, split-K merge)
            "roofline": {"bound": "hbm", "kernel": "decode attention (split-K pass)", "achieved": round(achieved, 1),
                         "peak": peak, "unit": "GB/s", "frac": round(achieved / peak, 4), "traffic": None,
                         "peak_source": peak_src, "launch_us": round(launch_ms * 1e3, 1),
                         "algorithmic_bytes_per_launch": launch_bytes},
            "quantize": {"mvec_per_s": round(nvec / (quant_ms * 1e-3) / 1e6, 1), "gbps": round(quant_bytes / (quant_ms * 1e-3) / 1e9, 1),
                         "frac_of_hbm_peak": round(quant_bytes / (quant_ms * 1e-3) / 1e9 / peak, 4),
                         "what": "bulk quantize of one layer: K and V, 2 x 64 x 8 x 8192 bf16 vectors -> PQO4 in one launch (328 B per vector in+out)"},
            "clocks": clocks,
        }
        if not args.no_cpu and world == 1:   # the CPU leg runs at N = 1 only
            line["cpu_baseline"] = cpu_baseline(max_seconds=20.0)
        tr = os.path.join(ROOT, "profiles", "decode_traffic.json")
        if os.path.exists(tr):
            line["roofline"]["traffic"] = json.load(open(tr)).get("bytes_per_launch_scaled")
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    return line


class CpuSample:
    """The oracle's decode attention on `seqs` sequences x 8 KV heads of one layer at context
    `ctx` (PQO4) over a packed cache built once, outside the timed passes."""

    def __init__(self, seqs, ctx, nthreads):
        import oracle_lib as o
        self.o, self.ctx, self.nthreads = o, ctx, nthreads
        rng = np.random.default_rng(0)
        hkv, hq, D, bits = CFG["hkv"] * seqs, CFG["hq"] * seqs, CFG["head_dim"], CFG["bits"]
        base = rng.standard_normal((CFG["hkv"] * ctx, D)).astype(np.float32)
        kp, ks = o.block_quantize(bits, D, 0, -1, base, nthreads=nthreads)
        self.kp = np.ascontiguousarray(np.tile(kp.reshape(CFG["hkv"], ctx, -1), (seqs, 1, 1)))
        self.ks = np.ascontiguousarray(np.tile(ks.reshape(CFG["hkv"], ctx, -1), (seqs, 1, 1)))
        self.q = (rng.standard_normal((hq, D)) / np.sqrt(D)).astype(np.float32)
        self.bytes = hkv * ctx * bytes_per_token_head()

    def run(self):
        t0 = time.perf_counter()
        self.o.block_attention(CFG["bits"], CFG["head_dim"], 0, -1, self.q, self.kp, self.ks, self.kp, self.ks, self.ctx,
                               1.0 / np.sqrt(CFG["head_dim"]), nthreads=self.nthreads)
        return time.perf_counter() - t0


def sized_sample(seconds_per_pass, cores):
    """Picks how many of the 64 sequences one CPU pass covers so that it lasts about `seconds_per_pass`."""
    dt = CpuSample(1, 1024, cores).run()
    per_seq = dt * (CFG["ctx"] / 1024)
    seqs = int(max(1, min(CFG["batch"], seconds_per_pass / max(per_seq, 1e-6))))
    return CpuSample(seqs, CFG["ctx"], cores), seqs


def cpu_baseline(max_seconds=20.0):
    cores = os.cpu_count() or 1
    sample, seqs = sized_sample(max_seconds / 3, cores)
    dt = min(sample.run() for _ in range(2))
    return {"value": round(sample.bytes / dt / 1e9, 4), "unit": "GB/s", "cores": cores, "kind": "port",
            "sample": f"one layer, {seqs} of 64 sequences x 8 kv heads x ctx 8192, PQO4, oracle decode attention on {cores} threads",
            "seconds": round(dt, 2)}


def run_reference(args):
    """The reference's CPU implementation of the path (its C++ restatement: no Rust toolchain
    exists on this machine), all host threads, same metric; each step is a bounded sample."""
    rank = int(os.environ.get("RANK", 0))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    budget = 120.0 / max(args.steps + args.warmup, 1)
    sample, seqs = sized_sample(min(budget, 10.0), cores)
    for _ in range(args.warmup):
        sample.run()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        sample.run()
    el = time.perf_counter() - t0
    value = sample.bytes * args.steps / el / 1e9
    desc = f"per step: one layer, {seqs} of 64 sequences x 8 kv heads x ctx 8192 (PQO4), oracle decode attention"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": round(value, 4), "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(el / args.steps * 1e3, 2), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "format": "PQO4 block-32 MaxNorm", "sample": desc},
        "cpu_baseline": {"value": round(value, 4), "unit": "GB/s", "cores": cores, "kind": "port", "sample": desc},
        "e2e": {"value": round(value, 4), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def run_whole_vector(args):
    """Secondary report (not the contract line): the whole-vector (core crate) kernels on synthetic N(0,1) data,
    CUDA-event times against the measured HBM peak.  Also the small case for profiler captures of these kernels."""
    import numpy as np
    import torch
    import turboquant_b200 as tq
    peak = peaks()[0]
    dev = "cuda"
    n, m, keys, dim = 1 << 19, 1 << 16, 1 << 21, 128

    def timed(fn):
        ts = []
        for _ in range(args.warmup + args.steps):
            e0, e1 = torch.cuda.Event(True), torch.cuda.Event(True)
            e0.record()
            fn()
            e1.record()
            e1.synchronize()
            ts.append(e0.elapsed_time(e1))
        return float(np.median(ts[args.warmup:]))

    x = torch.randn((n, dim), device=dev)
    rows = []

    def row(name, units, bytes_per_unit, ms):
        gbs = units * bytes_per_unit / ms / 1e6
        rows.append({"kernel": name, "units": units, "bytes_per_unit": bytes_per_unit, "ms": round(ms, 4),
                     "GB/s": round(gbs, 1), "frac_of_measured_peak": round(gbs / peak, 3)})

    for bits in (3, 4):
        cfg = tq.TurboQuantConfig(bits, dim).with_seed(42)
        pb = tq.packed_bytes(bits, dim)
        row(f"quantize_batch TQ{bits}", n, 4 * dim + pb + 2, timed(lambda: tq.quantize_batch(cfg, x)))
        p, s = tq.quantize_batch(cfg, x)
        row(f"dequantize_batch TQ{bits}", n, 4 * dim + pb + 2, timed(lambda: tq.dequantize_batch(cfg, p, s)))
        qpb = tq.packed_bytes(bits - 1, dim)
        row(f"qjl_quantize_batch TQ{bits}", m, 4 * dim + qpb + 2 + dim // 8 + 2,
            timed(lambda: tq.qjl_quantize_batch(cfg, x[:m], 42)))
        pk, sc, sg, rn = [t.repeat((keys // m,) + (1,) * (t.dim() - 1)) for t in tq.qjl_quantize_batch(cfg, x[:m], 42)]
        q = torch.randn(dim, device=dev) / dim ** 0.5
        rq = tq.query_projections(q, dim, 42).reshape(-1)
        row(f"qjl_attention_scores TQ{bits}", keys, qpb + 2 + dim // 8 + 2,
            timed(lambda: tq.qjl_attention_scores(cfg, q, rq, pk, sc, sg, rn)))
        w = torch.rand(keys, device=dev)
        row(f"weighted_values TQ{bits}", keys, qpb + 2 + 4, timed(lambda: tq.weighted_values(cfg, w, pk, sc)))
    print(json.dumps({"report": "whole-vector kernels", "dim": dim, "peak_GB/s": peak, "peak_source": peaks()[1],
                      "timing": "CUDA events, median of %d after %d warm-up calls (python call included)" % (args.steps, args.warmup),
                      "rows": rows}))


def run_chunk(args):
    """Secondary report (not the contract line): causal prefill-chunk attention over the packed cache
    (tqb_chunk_attention), Llama-3-8B head geometry, PQO4, bf16 queries; CUDA-event times."""
    import numpy as np
    import torch
    import turboquant_b200 as tq
    peak = peaks()[0]
    dev, hkv, hq, d, bits = "cuda", 8, 32, 128, 4
    rows = []
    for past, q_len in ((8192 - 128, 128), (8192 - 512, 512), (32768 - 256, 256), (0, 512)):
        n = past + q_len
        k = torch.randn((hkv * n, d), device=dev, dtype=torch.bfloat16)
        v = torch.randn_like(k)
        ki, ks = tq.block_quantize(k, bits)
        vi, vs = tq.block_quantize(v, bits)
        ki, ks, vi, vs = (t.view(hkv, n, -1) for t in (ki, ks, vi, vs))
        q = (torch.randn((q_len, hq, d), device=dev) / d ** 0.5).bfloat16()
        ts = []
        for _ in range(args.warmup + args.steps):
            e0, e1 = torch.cuda.Event(True), torch.cuda.Event(True)
            e0.record()
            tq.chunk_attention(q, ki, ks, vi, vs, n, bits, 1.0 / d ** 0.5)
            e1.record()
            e1.synchronize()
            ts.append(e0.elapsed_time(e1))
        ms = float(np.median(ts[args.warmup:]))
        attended = sum(past + i + 1 for i in range(q_len))          # (query token, key token) pairs per KV head group
        rows.append({"past_tokens": past, "q_len": q_len, "ms": round(ms, 4),
                     "cache_MB": round(n * hkv * bytes_per_token_head() / 1e6, 1),
                     "attended_GB/s": round(attended * hkv * bytes_per_token_head() / ms / 1e6, 1),
                     "attended_frac_of_measured_hbm_peak": round(attended * hkv * bytes_per_token_head() / ms / 1e6 / peak, 3),
                     "attention_TFLOP/s": round(attended * hq * d * 4 / ms / 1e9, 1)})
    print(json.dumps({"report": "prefill-chunk attention over the packed cache", "heads": [hq, hkv], "format": "PQO4",
                      "note": "the cache is re-read once per query token, mostly from L2; attended bytes = what one decode "
                              "step per query token would stream", "rows": rows}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--profile-case", action="store_true",
                    help="small case for profiler captures: 2 layers, batch 16 (151 MB of packed cache per launch, "
                         "above the L2 size, 0.4 GB on the device); its numbers are not bench values")
    ap.add_argument("--profile-bits", type=int, default=4, choices=[3, 4],
                    help="with --profile-case: code width of the small case (3 = PQO3, 4 = PQO4)")
    ap.add_argument("--whole-vector", action="store_true",
                    help="secondary report: the whole-vector (core crate) kernels, 2^19 vectors / 2^21 keys of d = 128 "
                         "(0.3 GB on the device); also the small case for profiler captures of those kernels")
    ap.add_argument("--chunk", action="store_true",
                    help="secondary report: causal prefill-chunk attention over the packed cache (tqb_chunk_attention)")
    args = ap.parse_args()
    if args.chunk:
        run_chunk(args)
        return
    if args.whole_vector:
        run_whole_vector(args)
        return
    if args.profile_case:
        CFG.update(layers=2, batch=16, bits=args.profile_bits)
        args.no_cpu = True
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
