"""Multi-GPU plumbing for the decode path (one process per GPU, torch.distributed).

Two ways the path shards (both without any collective inside a kernel):
  * (batch, KV head) units are independent: `shard_range` gives each rank a contiguous slice and
    nothing is exchanged;
  * one long sequence is split along the tokens: every rank attends over its shard and produces the
    un-normalised output and the (max, sum) pair per query head; `gather_partials` all-gathers
    them (NCCL over NVLink on GPUs, gloo in CPU tests) and `tqb_lse_combine` merges them with
    the log-sum-exp algebra of tq_fused_attention_reduce (tq_attention_kernel.cu:299-332).
"""
import torch
import torch.distributed as dist


def shard_range(n, world, rank):
    """Contiguous [lo, hi) slice of n units for `rank`; the first n % world ranks get one more."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("bad world/rank")
    base, rem = divmod(n, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def gather_partials(out_unnorm, lse, group=None):
    """All-gather shard-local results: [Hq, D], [Hq, 2] -> [world, Hq, D], [world, Hq, 2]."""
    world = dist.get_world_size(group)
    outs = torch.empty((world,) + tuple(out_unnorm.shape), dtype=out_unnorm.dtype, device=out_unnorm.device)
    lses = torch.empty((world,) + tuple(lse.shape), dtype=lse.dtype, device=lse.device)
    # gathered along dim 0 of a flat view: the form both NCCL and gloo accept
    dist.all_gather_into_tensor(outs.view(-1, *out_unnorm.shape[1:]), out_unnorm.contiguous(), group=group)
    dist.all_gather_into_tensor(lses.view(-1, *lse.shape[1:]), lse.contiguous(), group=group)
    return outs, lses


def sequence_parallel_attend(cache, layer, q, softmax_scale, group=None, out_dtype=torch.float32):
    """Decode attention of one query over a cache whose tokens are sharded across the ranks of
    `group`: local split-K pass, all-gather of (out, max, sum), merge on every rank."""
    from .api import lse_combine
    out, lse = cache.attend_partial(layer, q, softmax_scale)
    outs, lses = gather_partials(out, lse, group)
    return lse_combine(outs, lses, out_dtype)
