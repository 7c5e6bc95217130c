#!/usr/bin/env python3
"""Benchmark of the hot path: batched decode attention over the packed block-32 KV cache.

Workload (the largest single-GPU configuration of the baseline): Llama-3-8B-shaped PQO4
batched decode -- 32 layers, 32 query heads, 8 KV heads (GQA 4), head_dim 128, batch 64,
context 8,192; K/V bf16 N(0,1) with per-channel log-normal(0, 0.5) scales (synthetic; seeds
42 + layer); the cache is filled by the batched quantize kernel, then decode steps run.
A step = one new token for each of the 64 sequences through all 32 layers
(append-quantize + fused attention per layer).  With N GPUs the ONE batch-64 problem is
sharded by (batch, KV head) units over the ranks, no collective on the data path: strong scaling.

metric  = effective HBM GB/s: algorithmic compressed bytes read (2 * (64 + 8) = 144 B per
          token per KV head per layer) / time, whole job.
value   = steps with all inputs resident in HBM, CUDA-event timed, max over ranks.
e2e     = the same steps through PqoCache.decode with HOST (pinned) k, v, q buffers and
          the output read back to the host, copies inside the timed region.
roofline= the decode kernel alone: algorithmic bytes per launch / mean launch duration,
          measured with CUDA events around single launches.
parity_max_abs = max-abs difference between one layer's decode output of the cache under test and the
          CPU oracle's attention over the identical packed bytes copied down from that cache.
Extra records (headline unchanged): `pqo3` (the same batch-64 x 8,192 shape stored as PQO3), `tq3_fused` (the same
shape in a TqCache with the QJL correction inside the attention kernel), `config3`
(Qwen3-0.6B shape, batch 1, context 1K .. 32K, per layer and per 28-layer step against the HBM roofline),
`seq_parallel` (Llama-3-70B shape, one 131,072-token sequence split along the tokens over the ranks,
partials exchanged and merged per layer).
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


def bytes_per_token_head(bits=None, head_dim=None):
    """Algorithmic bytes of one (token, KV head): packed K and V codes plus their four f16 scales each
    (144 B for PQO4, 112 B for PQO3 at head_dim 128)."""
    bits = CFG["bits"] if bits is None else bits
    head_dim = CFG["head_dim"] if head_dim is None else head_dim
    return 2 * (head_dim * bits // 8 + (head_dim // 32) * 2)


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
                                          "-lms", "100", "-i", str(self.gpu)], stdout=subprocess.PIPE, text=True)
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


EXTRA_DECODE_FLAGS = 0   # --profile-general: TQB_DECODE_FORCE_GENERAL on the per-launch timing of the small case


def stream_ptr():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def kernel_launch_ms(lib, cache, layers, q2, hq_total, bits, scale, reps=2):
    """The decode kernel alone (split-K pass, TQB_DECODE_PARTIALS_ONLY), one CUDA-event pair per launch, mean over
    the layers of the last repetition."""
    from turboquant_b200._lib import TqbDecodeParams
    dev = q2.device
    d = q2.shape[-1]
    kv_len = cache.seq_len(layers[0])
    nheads = cache.config.batch * cache.config.num_kv_heads
    parts = int(lib.tqb_decode_num_partitions(nheads, kv_len))
    scratch = torch.empty(int(lib.tqb_decode_scratch_bytes(hq_total, d, parts)), dtype=torch.uint8, device=dev)
    dummy = torch.empty((hq_total, d), dtype=q2.dtype, device=dev)
    code = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}[q2.dtype]
    durs = []
    for rep in range(reps):
        for layer in layers:
            p = TqbDecodeParams()
            p.k_indices, p.k_scales, p.v_indices, p.v_scales = cache.layer_ptrs(layer)
            p.q, p.out, p.scratch, p.scratch_bytes = q2.data_ptr(), dummy.data_ptr(), scratch.data_ptr(), scratch.numel()
            p.q_dtype = p.out_dtype = code
            p.bits, p.head_dim, p.norm_mode, p.outlier_blocks = bits, d, 0, -1
            p.num_q_heads, p.num_kv_heads, p.kv_len, p.kv_stride = hq_total, nheads, kv_len, cache.capacity(layer)
            p.num_partitions, p.softmax_scale, p.flags = parts, scale, 1 | EXTRA_DECODE_FLAGS     # split-K pass only
            s0, s1 = torch.cuda.Event(True), torch.cuda.Event(True)
            s0.record()
            rc = lib.tqb_decode_attention(ctypes.byref(p), stream_ptr())
            s1.record()
            assert rc == 0, rc
            s1.synchronize()
            if rep == reps - 1:
                durs.append(s0.elapsed_time(s1))
    return float(np.mean(durs)), nheads * kv_len


def run_ours(args):
    import turboquant_b200 as tq
    import workloads as w
    from turboquant_b200._lib import lib
    from turboquant_b200.dist import shard_range

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
    # strong scaling: the (batch, KV head) units of the one problem are dealt out in contiguous runs of whole sequences
    b_lo, b_hi = shard_range(B, world, rank)
    BL = b_hi - b_lo
    scale = 1.0 / np.sqrt(D)
    peak, peak_src = peaks()
    cache = tq.PqoCache(tq.CacheConfig(bits=BITS, head_dim=D, num_kv_heads=HKV, num_layers=L, batch=BL))
    att = tq.AttendConfig(softmax_scale=scale, n_kv_groups=HQ // HKV)
    # the launches of successive layers overlap head to tail (programmatic dependent launch): a step's inputs are not
    # outputs of the launch before them
    cache.set_overlap(not args.no_overlap)

    # ---- fill the cache with the batched quantize kernel ----
    # The bulk-quantize figure is taken on the last layer's K/V into buffers allocated beforehand (a cache
    # fill also allocates and clears the layer's storage, which is not the kernel's time).
    nvec = 2 * BL * HKV * CTX
    quant_bytes = nvec * (D * 2 + D * BITS // 8 + (D // 32) * 2)
    qt = []
    for layer in range(L):
        k, v = w.synth_kv("llama8b", layer, CTX, dev, batch=B)
        k, v = k[b_lo:b_hi].contiguous(), v[b_lo:b_hi].contiguous()
        cache.prefill(layer, k, v)
        if layer == L - 1:
            rows = BL * HKV * CTX
            qi = torch.empty((2, rows, D * BITS // 8), dtype=torch.uint8, device=dev)
            qs_ = torch.empty((2, rows, D // 32), dtype=torch.int16, device=dev)
            for rep in range(4):
                e0, e1 = torch.cuda.Event(True), torch.cuda.Event(True)
                e0.record()
                rc = lib.tqb_block_quantize_pair(BITS, D, 0, -1, k.data_ptr(), v.data_ptr(), 2, rows, 0, qi[0].data_ptr(),
                                                 qs_[0].data_ptr(), qi[1].data_ptr(), qs_[1].data_ptr(), 0, 0, 0, stream_ptr())
                e1.record()
                assert rc == 0, rc
                e1.synchronize()
                if rep:
                    qt.append(e0.elapsed_time(e1))
            del qi, qs_
        del k, v
    quant_ms = float(np.median(qt))

    g = torch.Generator(device=dev).manual_seed(1234)
    n_tok = 4 * (args.warmup + args.steps) + 8
    newk = torch.randn((4, B, HKV, 1, D), generator=g, device=dev).to(torch.bfloat16)[:, b_lo:b_hi].contiguous()
    newv = torch.randn((4, B, HKV, 1, D), generator=g, device=dev).to(torch.bfloat16)[:, b_lo:b_hi].contiguous()
    qs = (torch.randn((4, B, HQ, 1, D), generator=g, device=dev) * scale).to(torch.bfloat16)[:, b_lo:b_hi].contiguous()
    outs = torch.empty((L, BL, HQ, 1, D), dtype=torch.bfloat16, device=dev)
    assert cache.capacity(0) >= CTX + n_tok, "decode steps would force a cache re-allocation inside the timed region"

    def make_step(ks, vs, qs_, outs_, host):
        """One decode step = L calls of the C entry point tqb_pqo_cache_decode (what PqoCache.decode forwards to), with the
        argument objects built once: at 8 GPUs a layer takes ~16 us, and tensor indexing plus the Python wrapper
        cost about as much per call."""
        fn, h = lib.tqb_pqo_cache_decode, cache._h
        kp = [ctypes.c_void_p(t.data_ptr()) for t in ks]
        vp = [ctypes.c_void_p(t.data_ptr()) for t in vs]
        qp = [ctypes.c_void_p(t.data_ptr()) for t in qs_]
        op = [ctypes.c_void_p(outs_[layer].data_ptr()) for layer in range(L)]
        code, nq, sc, hb = ctypes.c_int32(2), ctypes.c_int32(HQ), ctypes.c_float(scale), ctypes.c_int32(1 if host else 0)

        def step(i):
            st = stream_ptr()
            k, v = kp[i % 4], vp[i % 4]
            for layer in range(L):
                rc = fn(h, layer, k, v, qp[(i + layer) % 4], code, nq, sc, op[layer], hb, st)
                if rc != 0:
                    raise RuntimeError("tqb_pqo_cache_decode failed with status %d" % rc)
        return step

    step_device = make_step([newk[j] for j in range(4)], [newv[j] for j in range(4)], [qs[j] for j in range(4)], outs, False)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def cool_down():
        barrier()
        time.sleep(1.0)

    def bytes_of_steps(first_len, nsteps):
        # each step attends over the cache after its own append
        return sum(L * BL * HKV * (first_len + 1 + s) * bytes_per_token_head() for s in range(nsteps))

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
    step_bytes = bytes_of_steps(len0, args.steps)
    # the same steps with the launches strictly ordered (no programmatic dependent launch).  Every block starts after a
    # second of idling and its own warm-up, so that the power state one block leaves behind does not colour the next.
    ordered = None
    if not args.no_overlap:
        cache.set_overlap(False)
        cool_down()
        for i in range(args.warmup):
            step_device(i)
        barrier()
        len_o = cache.seq_len(0)
        o0, o1 = torch.cuda.Event(True), torch.cuda.Event(True)
        o0.record()
        for i in range(args.steps):
            step_device(i)
        o1.record()
        barrier()
        ordered = (o0.elapsed_time(o1), bytes_of_steps(len_o, args.steps))
        cache.set_overlap(True)
    # ---- e2e: host buffers through PqoCache.decode ----
    hk = [newk[i].cpu().pin_memory() for i in range(4)]
    hv = [newv[i].cpu().pin_memory() for i in range(4)]
    hq_ = [qs[i].cpu().pin_memory() for i in range(4)]
    hout = torch.empty((L, BL, HQ, 1, D), dtype=torch.bfloat16).pin_memory()

    step_host_calls = make_step(hk, hv, hq_, hout, True)

    def step_host(i):
        step_host_calls(i)
        cache.host_sync()   # the step's results are on the host

    cool_down()
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
    clocks = sampler.stop()
    e2e_bytes = bytes_of_steps(len1, args.steps)
    h2d = L * (2 * B * HKV * D + B * HQ * D) * 2    # whole job, like the value
    d2h = L * B * HQ * D * 2

    # ---- roofline: the decode kernel alone, one event pair per launch ----
    launch_ms, launch_units = kernel_launch_ms(lib, cache, list(range(L)), qs[0].reshape(BL * HQ, D), BL * HQ, BITS, scale)
    launch_bytes = launch_units * bytes_per_token_head()

    # ---- parity of the cache under test: layer 0's decode output against the oracle over the identical bytes ----
    parity = None
    if rank == 0 and not args.no_cpu:
        got = cache.decode(0, newk[0], newv[0], qs[1], att).fused.float().cpu().numpy().reshape(-1, D)
        want = w.oracle_decode_of_layer(cache, 0, qs[1], scale, nthreads=os.cpu_count() or 1)
        parity = float(np.abs(got - want).max())

    # ---- max over ranks ----
    if dist is not None:
        t = torch.tensor([ms, e2e_ms, ordered[0] if ordered else 0.0], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms, ord_ms = t.tolist()
        tb = torch.tensor([float(step_bytes), float(e2e_bytes), float(ordered[1] if ordered else 0)], device=dev, dtype=torch.float64)
        dist.all_reduce(tb)
        total_bytes, total_e2e_bytes, ord_bytes = tb.tolist()
    else:
        total_bytes, total_e2e_bytes = step_bytes, e2e_bytes
        ord_ms, ord_bytes = ordered if ordered else (0.0, 0)
    value = total_bytes / (ms * 1e-3) / 1e9
    e2e_value = total_e2e_bytes / (e2e_ms * 1e-3) / 1e9

    line = None
    if rank == 0:
        achieved = launch_bytes / (launch_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": round(value, 2), "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms / args.steps, 4), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "format": "PQO4 block-32 MaxNorm", "kv_dtype": "bf16", "q_dtype": "bf16",
                       "accumulate_dtype": "scores: s8 x s8 integer tensor-core MMAs on 20-bit query digits, s32 accumulate, exact; P V: f16 tensor-core operands split hi + lo, f32 accumulate",
                       "l2": "inputs larger than L2 (%.1f GB packed cache per GPU)" % (L * BL * HKV * CTX * bytes_per_token_head() / 1e9),
                       "launches": "one per layer; %s" % ("strictly ordered" if args.no_overlap else "successive layers overlap head to tail (programmatic dependent launch)"),
                       "sharding": "one batch-64 problem dealt out by (batch, kv head) units, %d sequences per GPU, no collective" % BL},
            "tokens_per_s": round(B * args.steps / (ms * 1e-3), 1),
            "pct_of_hbm_peak": round(100 * value / (peak * world), 2),
            "e2e": {"value": round(e2e_value, 2), "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "tokens_per_s": round(B * args.steps / (e2e_ms * 1e-3), 1),
                    "how": "tqb_pqo_cache_decode (C ABI) on pinned host k / v / q / out, host_sync once per step: the attention kernel reads the "
                           "inputs and the merging CTAs write the result over PCIe themselves (no staging copy)"},
            "ordered_launches": ({"value": round(ord_bytes / (ord_ms * 1e-3) / 1e9, 2), "unit": "GB/s", "ms_per_step": round(ord_ms / args.steps, 4),
                                  "what": "the same steps with every launch waiting for the one before it (no programmatic dependent launch)"}
                                 if ordered else None),
            "gpu_launches": args.steps * L * world,   # per layer and rank: one kernel (append of the new token, attention, split-K merge)
            "roofline": {"bound": "hbm", "kernel": "decode attention (split-K pass)", "achieved": round(achieved, 1),
                         "peak": peak, "unit": "GB/s", "frac": round(achieved / peak, 4), "traffic": None,
                         "peak_source": peak_src, "launch_us": round(launch_ms * 1e3, 1),
                         "algorithmic_bytes_per_launch": launch_bytes, "measured_on": "rank 0",
                         "how": "isolated launches of the split-K pass, one CUDA-event pair per launch",
                         # the same kernel inside the timed steps, where successive launches overlap: whole-job bytes / time
                         "in_step": {"us_per_launch": round(ms / args.steps / L * 1e3, 1),
                                     "achieved": round(value / world, 1), "frac": round(value / world / peak, 4)}},
            "quantize": {"mvec_per_s": round(nvec / (quant_ms * 1e-3) / 1e6, 1), "gbps": round(quant_bytes / (quant_ms * 1e-3) / 1e9, 1),
                         "frac_of_hbm_peak": round(quant_bytes / (quant_ms * 1e-3) / 1e9 / peak, 4),
                         "what": "bulk quantize of one layer on rank 0: K and V, 2 x %d x 8 x 8192 bf16 vectors -> PQO4 in one launch "
                                 "(328 B per vector in+out)" % BL},
            "parity_max_abs": parity,
            "parity_what": "layer 0 decode output (bf16) vs CPU oracle attention over the identical packed bytes of the cache under "
                           "test; tolerance 1e-2 for bf16 outputs (2e-3 in the f32 tests)",
            "clocks": clocks,
        }
        tr = os.path.join(ROOT, "profiles", "decode_traffic.json")
        if os.path.exists(tr) and world == 1:
            # dram bytes of an ncu capture of the small case (--profile-case), scaled to this launch by the units processed
            line["roofline"]["traffic"] = json.load(open(tr)).get("bytes_per_launch_scaled")
    if rank == 0 and world == 1 and not args.no_cpu:
        line["cpu_baseline"] = cpu_baseline(cache, qs[1], scale, w)
    del cache, outs, hout
    torch.cuda.empty_cache()

    if not args.no_extras:
        if world == 1:
            extras = {}
            for name, fn in (("pqo3", lambda: extra_pqo3(tq, w, lib, dev, args, peak)),
                             ("tq3_fused", lambda: extra_tq3(tq, w, lib, dev, args, peak)),
                             ("config3", lambda: extra_config3(tq, w, lib, dev, args, peak)),
                             ("seq_parallel", lambda: extra_seq_parallel(tq, w, lib, dev, args, peak, None, 0, 1))):
                try:
                    extras[name] = fn()
                except Exception as exc:   # an extra record never takes the headline down
                    extras[name] = {"error": repr(exc)[:300]}
                torch.cuda.empty_cache()
            line.update(extras)
        else:
            try:
                sp = extra_seq_parallel(tq, w, lib, dev, args, peak, dist, rank, world)
            except Exception as exc:
                sp = {"error": repr(exc)[:300]}
            if rank == 0:
                line["seq_parallel"] = sp
    if rank == 0:
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    return line


def timed_chain(fn, warmup, iters):
    """CUDA-event time of `iters` back-to-back calls of fn (a dependent chain on one stream), in ms per call."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(True), torch.cuda.Event(True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    e1.synchronize()
    return e0.elapsed_time(e1) / iters


def extra_pqo3(tq, w, lib, dev, args, peak):
    """The headline shape stored as PQO3 (112 B per token and KV head): 8 of the 32 layers (3.8 GB, rotated so that
    every launch reads from HBM), device-resident decode steps and the decode kernel alone."""
    L, B, HQ, HKV, D, CTX = 8, CFG["batch"], CFG["hq"], CFG["hkv"], CFG["head_dim"], CFG["ctx"]
    scale = 1.0 / np.sqrt(D)
    cache = tq.PqoCache(tq.CacheConfig(bits=3, head_dim=D, num_kv_heads=HKV, num_layers=L, batch=B))
    for layer in range(L):
        k, v = w.synth_kv("llama8b", layer, CTX, dev)
        cache.prefill(layer, k, v)
        del k, v
    g = torch.Generator(device=dev).manual_seed(99)
    nk = torch.randn((B, HKV, 1, D), generator=g, device=dev).to(torch.bfloat16)
    q = (torch.randn((B, HQ, 1, D), generator=g, device=dev) * scale).to(torch.bfloat16)
    out = torch.empty_like(q)
    att = tq.AttendConfig(scale, HQ // HKV)
    bpt = bytes_per_token_head(3)

    def step():
        for layer in range(L):
            cache.decode(layer, nk, nk, q, att, out=out)
    ms_ordered = timed_chain(step, 2, max(3, args.steps))
    cache.set_overlap(True)     # successive layers' launches overlap head to tail, as in the headline
    ms = timed_chain(step, 2, max(3, args.steps))
    cache.set_overlap(False)
    step_bytes = L * B * HKV * cache.seq_len(0) * bpt
    launch_ms, units = kernel_launch_ms(lib, cache, list(range(L)), q.reshape(B * HQ, D), B * HQ, 3, scale)
    ach = units * bpt / (launch_ms * 1e-3) / 1e9
    got = cache.decode(0, nk, nk, q, att).fused.float().cpu().numpy().reshape(-1, D)
    par = float(np.abs(got - w.oracle_decode_of_layer(cache, 0, q, scale, nthreads=os.cpu_count() or 1)).max()) if not args.no_cpu else None
    return {"workload": "the headline shape stored as PQO3: 8 layers x 64 sequences x 8 kv heads x ctx 8192",
            "value": round(step_bytes / (ms * 1e-3) / 1e9, 1), "unit": "GB/s", "ms_per_8_layers": round(ms, 4),
            "value_ordered_launches": round(step_bytes / (ms_ordered * 1e-3) / 1e9, 1),
            "tokens_per_s_at_32_layers": round(B / (ms * 4e-3), 1),
            "roofline": {"bound": "hbm", "kernel": "decode attention (split-K pass), PQO3", "achieved": round(ach, 1), "peak": peak,
                         "unit": "GB/s", "frac": round(ach / peak, 4), "launch_us": round(launch_ms * 1e3, 1),
                         "algorithmic_bytes_per_launch": units * bpt, "algorithmic_bytes_per_token_head": bpt},
            "parity_max_abs": par}


def extra_tq3(tq, w, lib, dev, args, peak):
    """TqCache (TQ3: 2-bit codebook stored at 3 bits + a 128-bit QJL sign sketch and a residual norm per key) at the
    headline shape: 4 layers x 64 sequences x 8 kv heads x ctx 8192; a step = per layer, append (quantize, dequantize,
    residual sketch), query projection and fused attention with the in-kernel QJL correction.  Algorithmic bytes per
    (token, KV head): 56 (K) + 56 (V) + 16 (sketch) + 2 (norm) = 130."""
    L, B, HQ, HKV, D, CTX = 4, CFG["batch"], CFG["hq"], CFG["hkv"], CFG["head_dim"], CFG["ctx"]
    scale = 1.0 / np.sqrt(D)
    cache = tq.TqCache(tq.CacheConfig(bits=3, head_dim=D, num_kv_heads=HKV, num_layers=L, batch=B, outlier_blocks=0))
    g = torch.Generator(device=dev).manual_seed(7)
    q = (torch.randn((B, HQ, 1, D), generator=g, device=dev) * scale).to(torch.bfloat16)
    for layer in range(L):
        k, v = w.synth_kv("llama8b", layer, CTX, dev)
        cache.prefill(layer, k, v, q)
        del k, v
    nk = torch.randn((B, HKV, 1, D), generator=g, device=dev).to(torch.bfloat16)
    att = tq.AttendConfig(scale, HQ // HKV)

    def step():
        for layer in range(L):
            cache.decode_fused(layer, nk, nk, q, att)
    ms = timed_chain(step, 2, max(3, args.steps))
    bpt = 130
    step_bytes = L * B * HKV * cache.seq_len(0) * bpt
    return {"workload": "TqCache TQ3 fused decode (in-kernel QJL correction): 4 layers x 64 sequences x 8 kv heads x ctx 8192",
            "value": round(step_bytes / (ms * 1e-3) / 1e9, 1), "unit": "GB/s", "frac_of_hbm_peak": round(step_bytes / (ms * 1e-3) / 1e9 / peak, 4),
            "us_per_layer": round(ms * 1e3 / L, 1), "algorithmic_bytes_per_token_head": bpt,
            "note": "per layer: block quantize K and V, dequantize K, residual sketch, query projection, then one attention launch"}


def extra_config3(tq, w, lib, dev, args, peak):
    """Qwen3-0.6B shape (28 layers, 16 / 8 heads, PQO3, batch 1) at context 1K .. 32K: one decode step per layer, as a
    dependent chain.  Working sets under 0.5 GB are rotated through several copies of the cache so that no launch
    reads from L2.  `graph` replays the 28 launches of a step from a CUDA graph (what an engine that captures its
    decode step sees); `calls` issues them through PqoCache.decode one by one."""
    cfg = w.SHAPES["qwen3"]
    L, HQ, HKV, D = cfg["layers"], cfg["hq"], cfg["hkv"], cfg["head_dim"]
    scale = 1.0 / np.sqrt(D)
    bpt = bytes_per_token_head(3)
    rows = []
    for ctx in (1024, 4096, 16384, 32768):
        step_bytes = L * HKV * ctx * bpt
        copies = max(4, int(np.ceil(0.5e9 / step_bytes))) if step_bytes < 0.5e9 else 1
        cache = tq.PqoCache(tq.CacheConfig(bits=3, head_dim=D, num_kv_heads=HKV, num_layers=L * copies))
        for layer in range(L):
            k, v = w.synth_kv("qwen3", layer, ctx, dev)
            for c in range(copies):
                cache.prefill(c * L + layer, k[:, :, :ctx - 1].contiguous(), v[:, :, :ctx - 1].contiguous())
        nk = k[:, :, ctx - 1:].contiguous()
        q = w.synth_q("qwen3", 0, dev)[0]
        out = torch.empty_like(q)
        att = tq.AttendConfig(scale, HQ // HKV)
        state = {"c": 0}

        def step():
            base = (state["c"] % copies) * L
            state["c"] += 1
            for layer in range(L):
                cache.decode(base + layer, nk, nk, q, att, out=out)
        # every layer of every copy gets its token once, so that the graph replays below rewrite an existing row
        for _ in range(copies):
            step()
        torch.cuda.synchronize()
        for layer in range(L * copies):
            cache_len = cache.seq_len(layer)
            assert cache_len == ctx, cache_len
        # (i) one call per layer from Python: rewinds nothing, the cache grows by one token per step
        calls_ms = timed_chain(step, 2, max(5, args.steps))
        # (ii) CUDA graph per copy: 28 launches, replayed round-robin
        graph_ms = graph_o_ms = None
        try:
            graphs = []
            side = torch.cuda.Stream()
            with torch.cuda.stream(side):
                for c in range(copies):
                    gph = torch.cuda.CUDAGraph()
                    state["c"] = c
                    with torch.cuda.graph(gph, stream=side, capture_error_mode="relaxed"):
                        step()
                    graphs.append(gph)
            torch.cuda.synchronize()
            it = {"i": 0}

            def replay():
                graphs[it["i"] % copies].replay()
                it["i"] += 1
            graph_ms = timed_chain(replay, 3, max(20, 2 * args.steps))
            # (iii) the same graphs captured with the layers' launches allowed to overlap head to tail: an upper bound for
            # an engine whose other kernels fill the gaps (here nothing sits between two attention launches)
            cache.set_overlap(True)
            graphs_o = []
            with torch.cuda.stream(side):
                for c in range(copies):
                    gph = torch.cuda.CUDAGraph()
                    state["c"] = c
                    with torch.cuda.graph(gph, stream=side, capture_error_mode="relaxed"):
                        step()
                    graphs_o.append(gph)
            cache.set_overlap(False)
            torch.cuda.synchronize()

            def replay_o():
                graphs_o[it["i"] % copies].replay()
                it["i"] += 1
            graph_o_ms = timed_chain(replay_o, 3, max(20, 2 * args.steps))
        except Exception as exc:
            graph_ms = None
            rows.append({"ctx": ctx, "graph_error": repr(exc)[:200]})
        roof_us = step_bytes / (peak * 1e9) * 1e6
        row = {"ctx": ctx, "cache_copies_rotated": copies, "step_bytes": step_bytes, "roofline_us_per_step": round(roof_us, 1),
               "calls_us_per_step": round(calls_ms * 1e3, 1), "calls_us_per_layer": round(calls_ms * 1e3 / L, 2),
               "calls_frac_of_hbm_peak": round(roof_us / (calls_ms * 1e3), 4)}
        if graph_ms is not None:
            row.update({"graph_us_per_step": round(graph_ms * 1e3, 1), "graph_us_per_layer": round(graph_ms * 1e3 / L, 2),
                        "graph_frac_of_hbm_peak": round(roof_us / (graph_ms * 1e3), 4),
                        "tokens_per_s_graph": round(1.0 / (graph_ms * 1e-3), 1)})
        if graph_o_ms is not None:
            row.update({"graph_overlapped_us_per_step": round(graph_o_ms * 1e3, 1),
                        "graph_overlapped_frac_of_hbm_peak": round(roof_us / (graph_o_ms * 1e3), 4)})
        rows.append(row)
        del cache
        torch.cuda.empty_cache()
    return {"workload": "qwen3-0.6b-shaped PQO3 decode: 28 layers, 16 q heads, 8 kv heads, head_dim 128, batch 1",
            "note": "one launch per layer (append + attention + split-K merge); at these sizes a launch is bound by launch and "
                    "dependency latency, not bandwidth: 8 kv heads x ctx 1024 is 0.9 MB per launch",
            "rows": rows}


def extra_seq_parallel(tq, w, lib, dev, args, peak, dist, rank, world):
    """Llama-3-70B shape (64 / 8 heads, PQO3), ONE sequence of 131,072 tokens split along the tokens over the ranks:
    per layer every rank attends over its shard (un-normalised output and (max, sum) per head), the records are
    exchanged and merged with the log-sum-exp algebra.  Dependent-chain timing over `layers` layers x 10 steps,
    max over ranks; the layer time is split by timing the chain with the later stages left out."""
    from turboquant_b200.dist import FusedSequenceParallelDecoder, SequenceParallelDecoder, shard_range
    cfg = w.SHAPES["llama70b"]
    HQ, HKV, D, CTX = cfg["hq"], cfg["hkv"], cfg["head_dim"], 131072
    layers = 8 if world <= 2 else 32        # per-rank working set stays above the L2 size
    scale = 1.0 / np.sqrt(D)
    bpt = bytes_per_token_head(3)
    lo, hi = shard_range(CTX, world, rank)
    cache = tq.PqoCache(tq.CacheConfig(bits=3, head_dim=D, num_kv_heads=HKV, num_layers=layers))
    for layer in range(layers):
        k, v = w.synth_kv("llama70b", layer % 8, CTX, dev)
        cache.prefill(layer, k[:, :, lo:hi].contiguous(), v[:, :, lo:hi].contiguous())
        del k, v
    q = w.synth_q("llama70b", 0, dev)[0]
    steps = 10
    rec = {"workload": "llama3-70b-shaped PQO3 long-context decode: 64 q heads, 8 kv heads, head_dim 128, batch 1, ctx 131072, "
                       "%d layers x %d steps (dependent chain)" % (layers, steps),
           "n_gpus": world, "tokens_per_rank": hi - lo, "layer_bytes": HKV * CTX * bpt}
    if world == 1:
        def chain_kernel():
            for layer in range(layers):
                cache.attend_partial(layer, q, scale)
        ms = timed_chain(chain_kernel, 2, steps) / layers
        rec.update({"us_per_layer": round(ms * 1e3, 1), "value": round(HKV * CTX * bpt / (ms * 1e-3) / 1e9, 1), "unit": "GB/s",
                    "frac_of_hbm_peak": round(HKV * CTX * bpt / (ms * 1e-3) / 1e9 / peak, 4),
                    "exchange": "none (one GPU holds the whole sequence)"})
        return rec
    def max_over_ranks(x):
        t = torch.tensor([x], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def measure(dec):
        def chain_full():
            for layer in range(layers):
                dec.attend(layer, q, scale)

        def chain_kernel():
            for layer in range(layers):
                dec.attend_local(layer, q, scale)

        def chain_exchange():
            for layer in range(layers):
                dec.attend_local(layer, q, scale)
                dec.exchange()
        res = {}
        for name, fn in (("kernel", chain_kernel), ("kernel_exchange", chain_exchange), ("full", chain_full)):
            dist.barrier()
            res[name] = max_over_ranks(timed_chain(fn, 2, steps) / layers)
        full = res["full"]
        return {"us_per_layer": round(full * 1e3, 1), "value": round(HKV * CTX * bpt / (full * 1e-3) / 1e9, 1), "unit": "GB/s",
                "frac_of_n_x_hbm_peak": round(HKV * CTX * bpt / (full * 1e-3) / 1e9 / (peak * world), 4),
                "split_us_per_layer": {"kernel": round(res["kernel"] * 1e3, 1),
                                       "exchange": round((res["kernel_exchange"] - res["kernel"]) * 1e3, 1),
                                       "combine": round((full - res["kernel_exchange"]) * 1e3, 1)},
                "exchange": dec.exchange_kind}
    nccl = measure(SequenceParallelDecoder(cache, HQ, device=dev))
    fused_dec = FusedSequenceParallelDecoder(cache, HQ, device=dev)
    fused = measure(fused_dec)
    # the two exchanges must agree on the result
    a = SequenceParallelDecoder(cache, HQ, device=dev).attend(0, q, scale).clone()
    b = fused_dec.attend(0, q, scale).clone()
    torch.cuda.synchronize()
    fused_dec.check()
    fused["max_abs_diff_to_nccl_path"] = float((a - b).abs().max().item())
    best = fused if fused["us_per_layer"] <= nccl["us_per_layer"] else nccl
    rec.update({"us_per_layer": best["us_per_layer"], "value": best["value"], "unit": "GB/s",
                "frac_of_n_x_hbm_peak": best["frac_of_n_x_hbm_peak"], "fused_peer_store": fused, "nccl_all_gather": nccl})
    return rec


def cpu_baseline(cache, q, scale, w):
    """The oracle's decode attention (all host threads) over one layer's packed bytes copied down from the cache under
    test: the same 64 sequences x 8 KV heads x ctx 8192 the GPU attends over, best of three passes."""
    import oracle_lib as o
    cores = os.cpu_count() or 1
    cfg = cache.config
    ki, ks, vi, vs = (t.numpy() for t in cache.export_layer(0, host=True))
    n = cache.seq_len(0)
    qf = q.float().cpu().numpy().reshape(-1, cfg.head_dim)
    best = None
    for _ in range(3):
        t0 = time.perf_counter()
        o.block_attention(cfg.bits, cfg.head_dim, 0, -1, qf, ki, ks.view(np.uint16), vi, vs.view(np.uint16), n, scale, nthreads=cores)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    nbytes = ki.shape[0] * n * bytes_per_token_head()
    return {"value": round(nbytes / best / 1e9, 4), "unit": "GB/s", "cores": cores, "kind": "port",
            "sample": f"one layer of the cache under test: {ki.shape[0] // CFG['hkv']} sequences x 8 kv heads x ctx {n}, PQO4, "
                      f"oracle decode attention on {cores} threads, best of 3 passes",
            "seconds": round(best, 2)}


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
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "format": "PQO4 block-32 MaxNorm", "sample": desc},
        "cpu_baseline": {"value": round(value, 4), "unit": "GB/s", "cores": cores, "kind": "port", "sample": desc},
        "e2e": {"value": round(value, 4), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def run_whole_vector(args):
    """Secondary report (not the contract line): the whole-vector (core crate) kernels on synthetic N(0,1) data,
    CUDA-event times against the measured HBM peak.  Also the small case for profiler captures of these kernels."""
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
        wt = torch.rand(keys, device=dev)
        row(f"weighted_values TQ{bits}", keys, qpb + 2 + 4, timed(lambda: tq.weighted_values(cfg, wt, pk, sc)))
    print(json.dumps({"report": "whole-vector kernels", "dim": dim, "peak_GB/s": peak, "peak_source": peaks()[1],
                      "timing": "CUDA events, median of %d after %d warm-up calls (python call included)" % (args.steps, args.warmup),
                      "rows": rows}))


def run_block_kernels(args):
    """Secondary report (not the contract line): the block-32 quantize / dequantize kernels and the TqCache sketch
    kernels on synthetic bf16 data (2^20 vectors of d = 128, 0.6 GB on the device), CUDA-event times against the
    measured HBM peak.  Also the small case for profiler captures of those kernels."""
    import turboquant_b200 as tq
    peak = peaks()[0]
    dev = "cuda"
    n, dim = 1 << 20, 128
    x = torch.randn((n, dim), device=dev).to(torch.bfloat16)
    rows = []

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

    def row(name, units, bytes_per_unit, ms):
        gbs = units * bytes_per_unit / ms / 1e6
        rows.append({"kernel": name, "units": units, "bytes_per_unit": bytes_per_unit, "ms": round(ms, 4),
                     "GB/s": round(gbs, 1), "Mvec/s": round(units / ms / 1e3, 1), "frac_of_measured_peak": round(gbs / peak, 3)})

    for bits in (3, 4):
        pd = dim * bits // 8
        idx = torch.empty((n, pd), dtype=torch.uint8, device=dev)
        sc = torch.empty((n, 4), dtype=torch.int16, device=dev)
        row(f"block_quantize PQO{bits} (bf16 in)", n, 2 * dim + pd + 8, timed(lambda: tq.block_quantize(x, bits, out=(idx, sc))))
        row(f"block_quantize PQ{bits} all-normal (bf16 in)", n, 2 * dim + pd + 8,
            timed(lambda: tq.block_quantize(x, bits, outlier_blocks=0, out=(idx, sc))))
        tq.block_quantize(x, bits, out=(idx, sc))
        row(f"block_dequantize PQO{bits} (f32 out)", n, 4 * dim + pd + 8, timed(lambda: tq.block_dequantize(idx, sc, bits, dim)))
    # TqCache insert: polar quantize + dequantize + residual sign sketch (64 K vectors: the sketch is d^2 sign-adds per vector)
    m = 1 << 16
    cache = tq.TqCache(tq.CacheConfig(bits=3, head_dim=dim, num_kv_heads=8, num_layers=1, outlier_blocks=0))
    kk = x[:m].reshape(1, 8, m // 8, dim).contiguous()
    qq = torch.randn((1, 16, 1, dim), device=dev).to(torch.bfloat16)

    def insert():
        cache.reset()
        cache.prefill(0, kk, kk, qq)
    row("TqCache.prefill of 65,536 vectors (quantize K and V, dequantize K, residual sketch, logit bias)", m, 2 * 2 * dim + 2 * 56 + 18,
        timed(insert))
    print(json.dumps({"report": "block-32 kernels", "dim": dim, "peak_GB/s": peak, "peak_source": peaks()[1],
                      "timing": "CUDA events, median of %d after %d warm-up calls (python call included)" % (args.steps, args.warmup),
                      "rows": rows}))


def run_chunk(args):
    """Secondary report (not the contract line): causal prefill-chunk attention over the packed cache
    (tqb_chunk_attention), Llama-3-8B head geometry, PQO4, bf16 queries; CUDA-event times."""
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
        def timed(fold):
            ts, out = [], None
            for _ in range(args.warmup + args.steps):
                e0, e1 = torch.cuda.Event(True), torch.cuda.Event(True)
                e0.record()
                out = tq.chunk_attention(q, ki, ks, vi, vs, n, bits, 1.0 / d ** 0.5, fold=fold)
                e1.record()
                e1.synchronize()
                ts.append(e0.elapsed_time(e1))
            return float(np.median(ts[args.warmup:])), out
        ms, out = timed(False)                  # the tcgen05 chunk kernel
        ms_fold, out_fold = timed(True)         # the chunk folded into decode launches (f32 / integer score path)
        attended = sum(past + i + 1 for i in range(q_len))          # (query token, key token) pairs per KV head group
        rows.append({"past_tokens": past, "q_len": q_len, "ms": round(ms, 4), "ms_folded_into_decode": round(ms_fold, 4),
                     "max_abs_diff_vs_folded": float((out.float() - out_fold.float()).abs().max()),
                     "cache_MB": round(n * hkv * bytes_per_token_head() / 1e6, 1),
                     "attended_GB/s": round(attended * hkv * bytes_per_token_head() / ms / 1e6, 1),
                     "attended_frac_of_measured_hbm_peak": round(attended * hkv * bytes_per_token_head() / ms / 1e6 / peak, 3),
                     "attention_TFLOP/s": round(attended * hq * d * 4 / ms / 1e9, 1)})
    print(json.dumps({"report": "prefill-chunk attention over the packed cache", "heads": [hq, hkv], "format": "PQO4",
                      "note": "attended bytes = what one decode step per query token would stream", "rows": rows}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU legs (baseline and parity against the oracle)")
    ap.add_argument("--no-overlap", action="store_true", help="headline: order the layers' launches strictly (no programmatic dependent launch)")
    ap.add_argument("--no-extras", action="store_true", help="headline only: skip the pqo3 / config3 / seq_parallel records")
    ap.add_argument("--profile-case", action="store_true",
                    help="small case for profiler captures: 2 layers, batch 16 (151 MB of packed cache per launch, "
                         "above the L2 size, 0.4 GB on the device); its numbers are not bench values")
    ap.add_argument("--profile-bits", type=int, default=4, choices=[3, 4],
                    help="with --profile-case: code width of the small case (3 = PQO3, 4 = PQO4)")
    ap.add_argument("--profile-general", action="store_true",
                    help="with --profile-case: the per-launch timing runs the general (any shape, SIMT) decode kernel")
    ap.add_argument("--whole-vector", action="store_true",
                    help="secondary report: the whole-vector (core crate) kernels, 2^19 vectors / 2^21 keys of d = 128 "
                         "(0.3 GB on the device); also the small case for profiler captures of those kernels")
    ap.add_argument("--block-kernels", action="store_true",
                    help="secondary report: block-32 quantize / dequantize and the TqCache insert; also the small case for "
                         "profiler captures of those kernels")
    ap.add_argument("--chunk", action="store_true",
                    help="secondary report: causal prefill-chunk attention over the packed cache (tqb_chunk_attention)")
    args = ap.parse_args()
    if args.chunk:
        run_chunk(args)
        return
    if args.whole_vector:
        run_whole_vector(args)
        return
    if args.block_kernels:
        run_block_kernels(args)
        return
    if args.profile_case:
        CFG.update(layers=2, batch=16, bits=args.profile_bits)
        if args.profile_general:
            global EXTRA_DECODE_FLAGS
            EXTRA_DECODE_FLAGS = 2
        args.no_cpu = True
        args.no_extras = True
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
