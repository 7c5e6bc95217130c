"""Multi-GPU plumbing for the decode path (one process per GPU, torch.distributed).

Two ways the path shards:
  * (batch, KV head) units are independent: `shard_range` gives each rank a contiguous slice and
    nothing is exchanged;
  * one long sequence is split along the tokens: every rank attends over its shard and produces the
    un-normalised output and the (max, sum) pair per query head; `gather_partials` all-gathers
    them (NCCL over NVLink on GPUs, gloo in CPU tests) and `tqb_lse_combine` merges them with
    the log-sum-exp algebra of tq_fused_attention_reduce (tq_attention_kernel.cu:299-332).
    `FusedSequenceParallelDecoder` replaces the all-gather by stores from inside the attention kernel: the CTA that
    finishes a KV head writes the head group's record into every rank's receive buffer over NVLink (peer memory
    shared through CUDA IPC) and a combine kernel waits, with a bound, for the flags of all ranks.
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


class SequenceParallelDecoder:
    """sequence_parallel_attend with everything pre-allocated and ONE all-gather per layer: the shard-local
    (out, max, sum) of all heads live in one flat record, the records of all ranks are gathered into one
    buffer and merged by tqb_lse_combine_packed."""

    def __init__(self, cache, num_q_heads, group=None, out_dtype=torch.float32, device=None):
        from ._lib import lib
        self.cache, self.group, self.out_dtype, self._lib = cache, group, out_dtype, lib
        self.world = dist.get_world_size(group)
        self.hq = cache.config.batch * num_q_heads
        self.nq = num_q_heads
        d = cache.config.head_dim
        dev = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.rec = torch.empty((self.hq * (d + 2),), dtype=torch.float32, device=dev)
        self.gathered = torch.empty((self.world * self.hq * (d + 2),), dtype=torch.float32, device=dev)
        self.out = torch.empty((self.hq, d), dtype=out_dtype, device=dev)

    exchange_kind = "NCCL all-gather of one flat (out, max, sum) record per rank, then a merge kernel"

    def attend_local(self, layer, q, softmax_scale):
        """Shard-local split-K pass: fills this rank's record (un-normalised out, then (max, sum) pairs)."""
        from .api import check, _dtype_code, _stream
        lib, d = self._lib, self.cache.config.head_dim
        q = q.contiguous()
        check(lib.tqb_pqo_cache_attend_partial(self.cache._h, layer, q.data_ptr(), _dtype_code(q.dtype), self.nq, softmax_scale,
                                               self.rec.data_ptr(), self.rec.data_ptr() + 4 * self.hq * d, _stream()))

    def exchange(self):
        dist.all_gather_into_tensor(self.gathered, self.rec, group=self.group)

    def combine(self):
        from .api import check, _dtype_code, _stream
        check(self._lib.tqb_lse_combine_packed(self.gathered.data_ptr(), self.world, self.hq, self.cache.config.head_dim,
                                               self.out.data_ptr(), _dtype_code(self.out_dtype), _stream()))
        return self.out

    def attend(self, layer, q, softmax_scale):
        self.attend_local(layer, q, softmax_scale)
        self.exchange()
        return self.combine()


class FusedSequenceParallelDecoder:
    """Sequence-parallel decode with the exchange fused into the attention kernel (tqb_peer_exchange_* in the C ABI).

    The receive buffer of every rank is created by the library, its CUDA IPC handle travels through
    `dist.all_gather_object` once, at construction; after that a layer is two launches (attention with the push,
    combine) and no collective call.  `wait_cycles` bounds every device-side wait (GPU clock cycles, ~0.5 s by default);
    `check()` raises PeerTimeout if one ever ran out."""

    exchange_kind = "records pushed into every rank's buffer by the attention kernel's merging CTAs (plain NVLink stores), flags, combine kernel"

    def __init__(self, cache, num_q_heads, group=None, out_dtype=torch.float32, device=None, wait_cycles=1 << 30):
        import ctypes
        from ._lib import lib
        from .api import check
        self.cache, self.group, self.out_dtype, self._lib = cache, group, out_dtype, lib
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.nq = num_q_heads
        self.hq = cache.config.batch * num_q_heads
        self.hkv = cache.config.batch * cache.config.num_kv_heads
        self.wait_cycles = int(wait_cycles)
        d = cache.config.head_dim
        dev = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self._x = ctypes.c_void_p()
        check(lib.tqb_peer_exchange_create(self.world, self.rank, self.hq, d, ctypes.byref(self._x)))
        mine = ctypes.create_string_buffer(64)
        check(lib.tqb_peer_exchange_handle(self._x, mine))
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(mine.raw), group=group)
        status = int(lib.tqb_peer_exchange_connect(self._x, b"".join(handles)))
        # every rank learns whether every rank could map its peers' buffers, so that a failure on one rank raises on
        # all of them instead of leaving the others waiting in their next collective
        statuses = [None] * self.world
        dist.all_gather_object(statuses, status, group=group)
        for st in statuses:
            check(st)
        self.out = torch.empty((self.hq, d), dtype=out_dtype, device=dev)

    def __del__(self):
        x = getattr(self, "_x", None)
        if x:
            self._lib.tqb_peer_exchange_destroy(x)
            self._x = None

    def attend_local(self, layer, q, softmax_scale):
        from .api import check, _dtype_code, _stream
        q = q.contiguous()
        check(self._lib.tqb_pqo_cache_attend_push(self.cache._h, layer, q.data_ptr(), _dtype_code(q.dtype), self.nq,
                                                  softmax_scale, self._x, _stream()))

    def exchange(self):
        pass   # the attention kernel has already stored the records where they are needed

    def combine(self):
        from .api import check, _dtype_code, _stream
        check(self._lib.tqb_peer_exchange_combine(self._x, self.hkv, self.out.data_ptr(), _dtype_code(self.out_dtype),
                                                  self.wait_cycles, _stream()))
        return self.out

    def attend(self, layer, q, softmax_scale):
        self.attend_local(layer, q, softmax_scale)
        return self.combine()

    def check(self):
        from .api import check
        check(self._lib.tqb_peer_exchange_check(self._x))
