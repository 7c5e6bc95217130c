"""Host-side mirror of the reference crate's public interface for the
quantize -> pack -> (QJL sketch) -> attend path, above the C ABI of libtqb200.so.

Names, argument meaning and error behaviour follow the reference (turboquant-rs 0.3.1):
`TurboQuantConfig`, `PackedBlock`, `quantize_vec` / `dequantize_vec`, `QjlBlock`,
`quantize_with_qjl`, `precompute_query_projections`, `estimate_inner_product`,
`QuantizedKVCache`, `CacheConfig`, `QuantNormMode`, `PqoCache`.  All arithmetic runs in the
CUDA library; torch is used for device memory and streams only.
"""
import ctypes
from dataclasses import dataclass
from enum import IntEnum

import numpy as np
import torch

from ._lib import TqbCacheConfig, TqbConfig, TqbDecodeParams, lib

TQB_F32, TQB_F16, TQB_BF16 = 0, 1, 2
ALL_BLOCKS = -1  # usize::MAX in src/cache/config.rs:49-50
DEFAULT_ROTATION_SEED = 42   # src/cache/config.rs:15
DEFAULT_QJL_SEED = 12345     # src/cache/config.rs:18
QUANT_BLOCK_SIZE = 32        # src/cache/config.rs:9


# ---------------------------------------------------------------------------------------
# Errors (src/error.rs:4-29)
# ---------------------------------------------------------------------------------------
class TurboQuantError(Exception):
    status = None


class InvalidDimension(TurboQuantError):
    status = 1


class UnsupportedBits(TurboQuantError):
    status = 2


class DimensionMismatch(TurboQuantError):
    status = 3


class LayerOutOfRange(TurboQuantError):
    status = 4


class RangeOutOfBounds(TurboQuantError):
    status = 5


class TqbRuntimeError(TurboQuantError):
    """Status codes beyond the reference's five error variants (null, CUDA, ...)."""


class PeerTimeout(TqbRuntimeError):
    """A bounded device-side wait for another rank's data ran out (TQB_ERR_PEER_TIMEOUT)."""
    status = 13


_ERRORS = {c.status: c for c in (InvalidDimension, UnsupportedBits, DimensionMismatch, LayerOutOfRange, RangeOutOfBounds)}


def check(status):
    if status == 0:
        return
    msg = lib.tqb_status_string(status).decode()
    cls = _ERRORS.get(status)
    if cls is not None:
        raise cls(msg)
    if status == PeerTimeout.status:
        raise PeerTimeout(msg)
    err = TqbRuntimeError(f"{msg} (status {status}, cuda error {lib.tqb_last_cuda_error()})")
    err.status = status
    raise err


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _dtype_code(dt):
    if dt == torch.float32:
        return TQB_F32
    if dt == torch.float16:
        return TQB_F16
    if dt == torch.bfloat16:
        return TQB_BF16
    raise TypeError(f"unsupported dtype {dt}")


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _np_ptr(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def packed_bytes(bits, count):
    return int(lib.tqb_packed_bytes(bits, count))


# ---------------------------------------------------------------------------------------
# TurboQuantConfig / PackedBlock  (src/packed/mod.rs:93-233)
# ---------------------------------------------------------------------------------------
class TurboQuantConfig:
    def __init__(self, bits, dim):
        # src/packed/mod.rs:124-132: bits first, then dim
        if bits not in (2, 3, 4):
            raise UnsupportedBits(f"unsupported bit width {bits}, expected 2, 3, or 4")
        if dim <= 0 or dim & (dim - 1):
            raise InvalidDimension(f"dimension {dim} is not a power of two")
        self.bits, self.dim, self.rotation_seed = bits, dim, 0

    def with_seed(self, seed):
        c = TurboQuantConfig(self.bits, self.dim)
        c.rotation_seed = seed
        return c

    def _c(self, bits=None):
        return TqbConfig(self.bits if bits is None else bits, self.dim, self.rotation_seed)


def pack_indices(bits, indices):
    """pack_indices_{2,3,4}bit (src/packed/indices.rs:188-268): LSB-first bit stream, tail
    zero-padded to a whole group.  Host bookkeeping (bit twiddling on a few bytes)."""
    idx = np.asarray(indices, dtype=np.uint8) & ((1 << bits) - 1)
    group = {2: 4, 3: 8, 4: 2}[bits]
    pad = (-len(idx)) % group
    idx = np.concatenate([idx, np.zeros(pad, np.uint8)])
    bitsarr = ((idx[:, None] >> np.arange(bits)) & 1).astype(np.uint8).reshape(-1)
    return np.packbits(bitsarr, bitorder="little")


def unpack_indices(bits, packed, count):
    """unpack_indices_{2,3,4}bit (src/packed/indices.rs:200-281)."""
    bitsarr = np.unpackbits(np.asarray(packed, dtype=np.uint8), bitorder="little")
    n = len(bitsarr) // bits
    vals = (bitsarr[: n * bits].reshape(n, bits) << np.arange(bits)).sum(1).astype(np.uint8)
    return vals[:count]


@dataclass
class PackedBlock:
    """src/packed/mod.rs:149-233.  `scale` holds the IEEE f16 bits."""
    bits: int
    scale: int
    packed_indices: bytes

    @classmethod
    def new(cls, bits, scale_f16_bits, indices):
        return cls(bits, int(scale_f16_bits), pack_indices(bits, indices).tobytes())

    @classmethod
    def from_raw(cls, bits, scale_f16_bits, packed_indices):
        return cls(bits, int(scale_f16_bits), bytes(packed_indices))

    def size_bytes(self):
        return 2 + len(self.packed_indices)

    def unpack(self, count):
        return unpack_indices(self.bits, np.frombuffer(self.packed_indices, np.uint8), count)

    def scale_f32(self):
        return float(np.array([self.scale], np.uint16).view(np.float16)[0])


@dataclass
class QjlBlock:
    """src/qjl.rs:111-134."""
    polar_block: PackedBlock
    qjl_signs: bytes
    residual_norm: int  # f16 bits

    @classmethod
    def from_parts(cls, polar_block, qjl_signs, residual_norm):
        return cls(polar_block, bytes(qjl_signs), int(residual_norm))

    def size_bytes(self):
        return self.polar_block.size_bytes() + len(self.qjl_signs) + 2


# ---------------------------------------------------------------------------------------
# Batched device operations of the whole-vector format
# ---------------------------------------------------------------------------------------
def quantize_batch(config, x):
    """x: CUDA f32 [n, dim] -> (packed u8 [n, pb], scales u16-as-int16 [n])."""
    if x.shape[-1] != config.dim:
        raise DimensionMismatch(f"expected vector of length {config.dim}, got {x.shape[-1]}")
    x = x.contiguous().float()
    n = x.shape[0]
    pb = packed_bytes(config.bits, config.dim)
    packed = torch.empty((n, pb), dtype=torch.uint8, device=x.device)
    scales = torch.empty((n,), dtype=torch.int16, device=x.device)
    c = config._c()
    check(lib.tqb_quantize_batch(ctypes.byref(c), _ptr(x), n, _ptr(packed), _ptr(scales), _stream()))
    return packed, scales


def dequantize_batch(config, packed, scales, rotated=False):
    n = packed.shape[0]
    out = torch.empty((n, config.dim), dtype=torch.float32, device=packed.device)
    c = config._c()
    fn = lib.tqb_dequantize_rotated_batch if rotated else lib.tqb_dequantize_batch
    check(fn(ctypes.byref(c), _ptr(packed), _ptr(scales), n, _ptr(out), _stream()))
    return out


_RBITS = {}


def rademacher_bits(dim, qjl_seed, device):
    """Device copy of the hash Rademacher bit matrix (src/qjl.rs:143-171), cached per
    (dim, seed, device) the way GpuPrecomputed caches its constants."""
    key = (dim, qjl_seed, str(device))
    if key not in _RBITS:
        host = np.zeros((dim, dim // 32), np.uint32)
        check(lib.tqb_qjl_rademacher_bits(dim, qjl_seed, _np_ptr(host)))
        _RBITS[key] = torch.from_numpy(host.view(np.int32)).to(device)
    return _RBITS[key]


def qjl_quantize_batch(config, x, qjl_seed):
    """quantize_with_qjl over a batch -> (packed, scales, signs, rnorms) device tensors."""
    if x.shape[-1] != config.dim:
        raise DimensionMismatch(f"expected vector of length {config.dim}, got {x.shape[-1]}")
    if config.bits not in (3, 4):
        raise UnsupportedBits(f"unsupported bit width {config.bits}")
    x = x.contiguous().float()
    n = x.shape[0]
    pb = packed_bytes(config.bits - 1, config.dim)
    dev = x.device
    packed = torch.empty((n, pb), dtype=torch.uint8, device=dev)
    scales = torch.empty((n,), dtype=torch.int16, device=dev)
    signs = torch.empty((n, config.dim // 8), dtype=torch.uint8, device=dev)
    rnorms = torch.empty((n,), dtype=torch.int16, device=dev)
    rb = rademacher_bits(config.dim, qjl_seed, dev)
    c = config._c()
    check(lib.tqb_qjl_quantize_batch(ctypes.byref(c), _ptr(rb), _ptr(x), n, _ptr(packed), _ptr(scales), _ptr(signs),
                                     _ptr(rnorms), _stream()))
    return packed, scales, signs, rnorms


def query_projections(q, dim, qjl_seed):
    q = q.contiguous().float().reshape(-1, dim)
    rq = torch.empty_like(q)
    rb = rademacher_bits(dim, qjl_seed, q.device)
    check(lib.tqb_qjl_query_projections(dim, _ptr(rb), _ptr(q), q.shape[0], _ptr(rq), _stream()))
    return rq


def qjl_attention_scores(config, q, rq, packed, scales, signs, rnorms):
    n = packed.shape[0]
    scores = torch.empty((n,), dtype=torch.float32, device=packed.device)
    c = config._c()
    check(lib.tqb_qjl_attention_scores(ctypes.byref(c), _ptr(q), _ptr(rq), _ptr(packed), _ptr(scales), _ptr(signs),
                                       _ptr(rnorms), n, _ptr(scores), _stream()))
    return scores


def weighted_values(config, w, packed, scales):
    n = packed.shape[0]
    dev = packed.device
    out = torch.empty((config.dim,), dtype=torch.float32, device=dev)
    sb = int(lib.tqb_weighted_values_scratch_bytes(config.dim))
    scratch = torch.empty((sb,), dtype=torch.uint8, device=dev)
    c = config._c()
    check(lib.tqb_weighted_values(ctypes.byref(c), _ptr(w), _ptr(packed), _ptr(scales), n, _ptr(out), _ptr(scratch), sb,
                                  _stream()))
    return out


# ---------------------------------------------------------------------------------------
# Single-vector API of the core crate (src/quantize.rs, src/qjl.rs)
# ---------------------------------------------------------------------------------------
def _dev():
    return torch.device("cuda", torch.cuda.current_device())


def _u16(t):
    return t.cpu().numpy().view(np.uint16)


def quantize_vec(config, data):
    """src/quantize.rs:142-157."""
    data = np.asarray(data, dtype=np.float32)
    if data.shape != (config.dim,):
        raise DimensionMismatch(f"expected vector of length {config.dim}, got {data.size}")
    packed, scales = quantize_batch(config, torch.from_numpy(data).to(_dev())[None])
    return PackedBlock.from_raw(config.bits, _u16(scales)[0], packed.cpu().numpy()[0].tobytes())


def dequantize_vec(config, block):
    """src/quantize.rs:207-239."""
    packed = torch.from_numpy(np.frombuffer(block.packed_indices, np.uint8).copy()).to(_dev())[None]
    scales = torch.from_numpy(np.array([block.scale], np.uint16).view(np.int16)).to(_dev())
    return dequantize_batch(config, packed, scales).cpu().numpy()[0]


def dequantize_rotated(config, block):
    """src/quantize.rs:306-316."""
    packed = torch.from_numpy(np.frombuffer(block.packed_indices, np.uint8).copy()).to(_dev())[None]
    scales = torch.from_numpy(np.array([block.scale], np.uint16).view(np.int16)).to(_dev())
    return dequantize_batch(config, packed, scales, rotated=True).cpu().numpy()[0]


def quantize_with_qjl(config, data, qjl_seed):
    """src/qjl.rs:355-377."""
    if config.bits not in (3, 4):
        raise UnsupportedBits(f"unsupported bit width {config.bits}, expected 2, 3, or 4")
    data = np.asarray(data, dtype=np.float32)
    if data.shape != (config.dim,):
        raise DimensionMismatch(f"expected vector of length {config.dim}, got {data.size}")
    p, s, sg, rn = qjl_quantize_batch(config, torch.from_numpy(data).to(_dev())[None], qjl_seed)
    polar = PackedBlock.from_raw(config.bits - 1, _u16(s)[0], p.cpu().numpy()[0].tobytes())
    return QjlBlock(polar, sg.cpu().numpy()[0].tobytes(), int(_u16(rn)[0]))


def precompute_query_projections(query, dim, qjl_seed):
    """src/qjl.rs:488-492."""
    q = torch.from_numpy(np.asarray(query, dtype=np.float32)).to(_dev())
    return query_projections(q, dim, qjl_seed).cpu().numpy()[0]


def estimate_inner_product(query, r_query, qjl_block, config):
    """src/qjl.rs:533-552."""
    dev = _dev()
    q = torch.from_numpy(np.asarray(query, dtype=np.float32)).to(dev)
    rq = torch.from_numpy(np.asarray(r_query, dtype=np.float32)).to(dev)
    pb = qjl_block.polar_block
    cfg = TurboQuantConfig(pb.bits + 1, config.dim).with_seed(config.rotation_seed)
    packed = torch.from_numpy(np.frombuffer(pb.packed_indices, np.uint8).copy()).to(dev)[None]
    scales = torch.from_numpy(np.array([pb.scale], np.uint16).view(np.int16)).to(dev)
    signs = torch.from_numpy(np.frombuffer(qjl_block.qjl_signs, np.uint8).copy()).to(dev)[None]
    rn = torch.from_numpy(np.array([qjl_block.residual_norm], np.uint16).view(np.int16)).to(dev)
    return float(qjl_attention_scores(cfg, q, rq, packed, scales, signs, rn).cpu()[0])


# ---------------------------------------------------------------------------------------
# QuantizedKVCache  (src/attention.rs:45-694)
# ---------------------------------------------------------------------------------------
class QuantizedKVCache:
    def __init__(self, config, num_layers, qjl_seed):
        self._config, self._qjl_seed = config, qjl_seed
        self._h = ctypes.c_void_p()
        c = config._c()
        check(lib.tqb_kv_cache_create(ctypes.byref(c), num_layers, qjl_seed, ctypes.byref(self._h)))

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            lib.tqb_kv_cache_destroy(h)
            self._h = None

    def config(self):
        return self._config

    def qjl_seed(self):
        return self._qjl_seed

    def num_layers(self):
        return int(lib.tqb_kv_cache_num_layers(self._h))

    def entry_count(self, layer):
        return int(lib.tqb_kv_cache_entry_count(self._h, layer))

    def push(self, layer, key, value):
        key = np.ascontiguousarray(key, dtype=np.float32)
        value = np.ascontiguousarray(value, dtype=np.float32)
        self.push_batch(layer, key[None], value[None])

    def push_batch(self, layer, keys, values):
        keys = np.ascontiguousarray(keys, dtype=np.float32)
        values = np.ascontiguousarray(values, dtype=np.float32)
        if 0 <= layer < self.num_layers():
            if len(keys) != len(values):  # attention.rs:277
                raise DimensionMismatch(f"expected vector of length {len(values)}, got {len(keys)}")
            if keys.ndim == 2 and values.ndim == 2 and keys.shape[1] != values.shape[1]:
                raise DimensionMismatch("key and value dimensions differ")
        vec_dim = keys.shape[1] if keys.ndim == 2 else 0
        check(lib.tqb_kv_cache_push_batch(self._h, layer, _np_ptr(keys), _np_ptr(values), len(keys), vec_dim, _stream()))

    def attention_scores(self, layer, query):
        query = np.ascontiguousarray(query, dtype=np.float32)
        n = max(self.entry_count(layer), 0)
        scores = np.zeros(n, np.float32)
        check(lib.tqb_kv_cache_attention_scores(self._h, layer, _np_ptr(query), query.size, _np_ptr(scores), _stream()))
        return scores

    def weighted_values(self, layer, weights):
        weights = np.ascontiguousarray(weights, dtype=np.float32)
        out = np.zeros(self._config.dim, np.float32)
        check(lib.tqb_kv_cache_weighted_values(self._h, layer, _np_ptr(weights), weights.size, _np_ptr(out), _stream()))
        return out

    def _dequantize_range(self, layer, start, end, is_keys):
        n = max(end - start, 0)
        out = np.zeros((n, self._config.dim), np.float32)
        check(lib.tqb_kv_cache_dequantize_range(self._h, layer, start, end, int(is_keys), _np_ptr(out), _stream()))
        return out

    def dequantize_keys_range(self, layer, start, end):
        return self._dequantize_range(layer, start, end, True)

    def dequantize_values_range(self, layer, start, end):
        return self._dequantize_range(layer, start, end, False)

    def dequantize_all_keys(self, layer):
        check(0 if 0 <= layer < self.num_layers() else 4)
        return self._dequantize_range(layer, 0, self.entry_count(layer), True)

    def dequantize_all_values(self, layer):
        check(0 if 0 <= layer < self.num_layers() else 4)
        return self._dequantize_range(layer, 0, self.entry_count(layer), False)

    def export_packed_range(self, layer, start, end, is_keys, with_qjl=False):
        """(packed_bytes, scales) as in src/attention.rs:663-677; with_qjl adds (signs, residual_norms)."""
        n = max(end - start, 0)
        pb = packed_bytes(self._config.bits - 1, self._config.dim)
        sb = self._config.dim // 8
        packed = np.zeros(n * pb, np.uint8)
        scales = np.zeros(n, np.uint16)
        signs = np.zeros(n * sb, np.uint8) if with_qjl else None
        rn = np.zeros(n, np.uint16) if with_qjl else None
        check(lib.tqb_kv_cache_export_packed_range(self._h, layer, start, end, int(is_keys), _np_ptr(packed), _np_ptr(scales),
                                                   _np_ptr(signs) if with_qjl else None,
                                                   _np_ptr(rn) if with_qjl else None, _stream()))
        return (packed, scales, signs, rn) if with_qjl else (packed, scales)

    def import_packed_range(self, layer, polar_bits, packed_bytes_, scales, qjl_signs_flat, residual_norms,
                            bytes_per_block, signs_per_block, is_keys):
        """PackedImport (src/attention.rs:147-166, :679-693)."""
        packed_bytes_ = np.ascontiguousarray(packed_bytes_, dtype=np.uint8)
        scales = np.ascontiguousarray(scales, dtype=np.uint16)
        qjl_signs_flat = np.ascontiguousarray(qjl_signs_flat, dtype=np.uint8)
        residual_norms = np.ascontiguousarray(residual_norms, dtype=np.uint16)
        check(lib.tqb_kv_cache_import_packed_range(self._h, layer, polar_bits, _np_ptr(packed_bytes_), _np_ptr(scales),
                                                   _np_ptr(qjl_signs_flat), _np_ptr(residual_norms), len(scales),
                                                   bytes_per_block, signs_per_block, int(is_keys), _stream()))

    def memory_usage(self):
        return int(lib.tqb_kv_cache_memory_usage(self._h))

    def fp16_equivalent_memory(self):
        return int(lib.tqb_kv_cache_fp16_equivalent_memory(self._h))


# ---------------------------------------------------------------------------------------
# Block-32 cache format (src/cache/)
# ---------------------------------------------------------------------------------------
class QuantNormMode(IntEnum):
    """src/cache/config.rs:21-44."""
    MaxNorm = 0
    L2Norm = 1

    @classmethod
    def from_str(cls, s):
        if s == "maxnorm":
            return cls.MaxNorm
        if s == "l2norm":
            return cls.L2Norm
        raise ValueError(f"Unknown norm mode `{s}`. Options: maxnorm, l2norm")

    def __str__(self):
        return "maxnorm" if self == QuantNormMode.MaxNorm else "l2norm"


@dataclass
class CacheConfig:
    """src/cache/config.rs:52-85 (+ batch: equal-length sequences fold into heads)."""
    bits: int
    head_dim: int
    num_kv_heads: int
    num_layers: int
    norm_mode: QuantNormMode = QuantNormMode.MaxNorm
    outlier_blocks: int = ALL_BLOCKS
    batch: int = 1

    def qjl_enabled(self):
        return self.outlier_blocks == 0

    def num_blocks(self):
        return self.head_dim // QUANT_BLOCK_SIZE

    def packed_dim(self):
        return self.head_dim * self.bits // 8

    def _c(self):
        return TqbCacheConfig(self.bits, self.head_dim, self.num_kv_heads, self.num_layers, int(self.norm_mode),
                              self.outlier_blocks, self.batch, 0, DEFAULT_ROTATION_SEED, DEFAULT_QJL_SEED)


def block_quantize(x, bits, norm_mode=QuantNormMode.MaxNorm, outlier_blocks=ALL_BLOCKS, out=None, rows_per_group=0,
                   group_stride=0, row_offset=0):
    """polar_quantize (src/cache/quantize_tensor.rs:40-79) on a CUDA tensor [n, head_dim]."""
    n, hd = x.shape
    x = x.contiguous()
    if out is None:
        idx = torch.empty((n, hd * bits // 8), dtype=torch.uint8, device=x.device)
        sc = torch.empty((n, max(hd // 32, 1)), dtype=torch.int16, device=x.device)
    else:
        idx, sc = out
    check(lib.tqb_block_quantize(bits, hd, int(norm_mode), outlier_blocks, _ptr(x), _dtype_code(x.dtype), n, 0, _ptr(idx),
                                 _ptr(sc), rows_per_group, group_stride, row_offset, _stream()))
    return idx, sc


def block_dequantize(indices, scales, bits, head_dim, norm_mode=QuantNormMode.MaxNorm, outlier_blocks=ALL_BLOCKS,
                     dtype=torch.float32):
    """polar_dequantize (src/cache/quantize_tensor.rs:179-220)."""
    n = indices.shape[0]
    out = torch.empty((n, head_dim), dtype=dtype, device=indices.device)
    check(lib.tqb_block_dequantize(bits, head_dim, int(norm_mode), outlier_blocks, _ptr(indices), _ptr(scales), n, 0, 0, 0,
                                   _ptr(out), _dtype_code(dtype), _stream()))
    return out


def decode_attention(q, k_idx, k_sc, v_idx, v_sc, kv_len, bits, softmax_scale, norm_mode=QuantNormMode.MaxNorm,
                     outlier_blocks=ALL_BLOCKS, num_partitions=0, out_dtype=None, return_lse=False, qjl=None,
                     scratch=None, out=None, partials_only=False, force_general=False, tma=False, append=None,
                     overlap=False):
    """Fused decode attention over packed K/V.

    q [Hq, D]; k_idx/v_idx [Hkv, kv_stride, D*bits/8]; k_sc/v_sc [Hkv, kv_stride, D/32].
    qjl = (signs [Hkv, kv_stride, D/8], norms [Hkv, kv_stride], rq [Hq, D]) enables the
    correction of tq_attention_kernel.cu:197-231.
    overlap=True: TQB_DECODE_OVERLAP | TQB_DECODE_TICKETS_ZERO - the launch may start before the previous decode
    launch on the stream has finished; `scratch` must then be given, zero-filled once by the caller."""
    hq, d = q.shape
    hkv, stride = k_idx.shape[0], k_idx.shape[1]
    q = q.contiguous()
    out_dtype = out_dtype or (torch.float32 if return_lse else q.dtype)
    if out is None:
        out = torch.empty((hq, d), dtype=out_dtype, device=q.device)
    lse = torch.empty((hq, 2), dtype=torch.float32, device=q.device) if return_lse else None
    parts = num_partitions or int(lib.tqb_decode_num_partitions(hkv, kv_len))
    sbytes = int(lib.tqb_decode_scratch_bytes(hq, d, parts))
    if scratch is None:
        scratch = torch.empty((max(sbytes, 16),), dtype=torch.uint8, device=q.device)
    p = TqbDecodeParams()
    p.q, p.k_indices, p.k_scales, p.v_indices, p.v_scales = (q.data_ptr(), k_idx.data_ptr(), k_sc.data_ptr(),
                                                             v_idx.data_ptr(), v_sc.data_ptr())
    p.out, p.lse_out = out.data_ptr(), (lse.data_ptr() if return_lse else None)
    p.scratch, p.scratch_bytes = scratch.data_ptr(), scratch.numel()
    if qjl is not None:
        p.qjl_signs, p.qjl_norms, p.rq, p.qjl_enabled = qjl[0].data_ptr(), qjl[1].data_ptr(), qjl[2].data_ptr(), 1
    p.q_dtype, p.out_dtype = _dtype_code(q.dtype), _dtype_code(out_dtype)
    p.bits, p.head_dim, p.norm_mode, p.outlier_blocks = bits, d, int(norm_mode), outlier_blocks
    p.num_q_heads, p.num_kv_heads, p.kv_len, p.kv_stride = hq, hkv, kv_len, stride
    p.num_partitions, p.softmax_scale = parts, softmax_scale
    p.flags = (1 if partials_only else 0) | (2 if force_general else 0) | (8 if tma else 0)
    if overlap:
        assert scratch is not None, "overlap=True needs a caller-owned scratch whose ticket area is zero"
        p.flags |= 4 | 32
    if append is not None:   # (k, v): the new token's vectors [Hkv, D] in q's dtype, written to row kv_len - 1
        ak, av = (t.contiguous() for t in append)
        assert ak.dtype == q.dtype and av.dtype == q.dtype
        p.append_k, p.append_v = ak.data_ptr(), av.data_ptr()
    check(lib.tqb_decode_attention(ctypes.byref(p), _stream()))
    return (out, lse) if return_lse else out


def chunk_attention(q, k_idx, k_sc, v_idx, v_sc, kv_len, bits, softmax_scale, norm_mode=QuantNormMode.MaxNorm,
                    outlier_blocks=ALL_BLOCKS, num_partitions=0, out_dtype=None, qjl=None, force_general=False, fold=False):
    """Causal attention of a chunk of query tokens over the packed cache (tqb_chunk_attention).
    fold=True takes the path that folds the chunk into decode launches instead of the dedicated tcgen05 kernel.

    q [q_len, Hq, D]; the cache arrays as for decode_attention, with the chunk's own K/V rows already stored;
    query token i attends to the first kv_len - q_len + i + 1 tokens.  Returns [q_len, Hq, D]."""
    q_len, hq, d = q.shape
    hkv, stride = k_idx.shape[0], k_idx.shape[1]
    q = q.contiguous()
    out_dtype = out_dtype or q.dtype
    out = torch.empty((q_len, hq, d), dtype=out_dtype, device=q.device)
    parts = num_partitions or int(lib.tqb_decode_num_partitions(hkv * q_len, kv_len))
    sbytes = int(lib.tqb_decode_scratch_bytes(hq * q_len, d, parts))
    scratch = torch.empty((max(sbytes, 16),), dtype=torch.uint8, device=q.device)
    p = TqbDecodeParams()
    p.q, p.k_indices, p.k_scales, p.v_indices, p.v_scales = (q.data_ptr(), k_idx.data_ptr(), k_sc.data_ptr(),
                                                             v_idx.data_ptr(), v_sc.data_ptr())
    p.out, p.lse_out = out.data_ptr(), None
    p.scratch, p.scratch_bytes = scratch.data_ptr(), scratch.numel()
    if qjl is not None:
        p.qjl_signs, p.qjl_norms, p.rq, p.qjl_enabled = qjl[0].data_ptr(), qjl[1].data_ptr(), qjl[2].data_ptr(), 1
    p.q_dtype, p.out_dtype = _dtype_code(q.dtype), _dtype_code(out_dtype)
    p.bits, p.head_dim, p.norm_mode, p.outlier_blocks = bits, d, int(norm_mode), outlier_blocks
    p.num_q_heads, p.num_kv_heads, p.kv_len, p.kv_stride = hq, hkv, kv_len, stride
    p.num_partitions, p.softmax_scale = parts, softmax_scale
    p.flags = (2 if force_general else 0) | (16 if fold else 0)
    check(lib.tqb_chunk_attention(ctypes.byref(p), q_len, _stream()))
    return out


def lse_combine(partial_out, partial_lse, out_dtype=torch.float32):
    """Merge shard-local (un-normalised output, (max, sum)) pairs: [S, Hq, D], [S, Hq, 2]."""
    s, hq, d = partial_out.shape
    out = torch.empty((hq, d), dtype=out_dtype, device=partial_out.device)
    check(lib.tqb_lse_combine(_ptr(partial_out.contiguous()), _ptr(partial_lse.contiguous()), s, hq, d, _ptr(out),
                              _dtype_code(out_dtype), _stream()))
    return out


@dataclass
class DequantResult:
    """mistralrs-kv-cache DequantResult as used at src/cache/common.rs:114-121."""
    k: torch.Tensor
    v: torch.Tensor
    logit_bias: torch.Tensor = None


@dataclass
class AttendConfig:
    softmax_scale: float
    n_kv_groups: int = 1


class DecodeOutput:
    """Fused(tensor) or Dequantized(DequantResult) (src/cache/pqo.rs:169-173, :219-221)."""

    def __init__(self, fused=None, dequantized=None):
        self.fused, self.dequantized = fused, dequantized

    def is_fused(self):
        return self.fused is not None


class PqoCache:
    """src/cache/pqo.rs:21-236.  k, v: [batch, num_kv_heads, seq, head_dim]; q: [batch, Hq, 1, head_dim]."""

    def __init__(self, config):
        self.config = config
        self._h = ctypes.c_void_p()
        c = config._c()
        check(lib.tqb_pqo_cache_create(ctypes.byref(c), ctypes.byref(self._h)))

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            lib.tqb_pqo_cache_destroy(h)
            self._h = None

    def set_overlap(self, enabled=True):
        """Let the decode launches of successive layers overlap head to tail (tqb_pqo_cache_set_overlap): the caller
        vouches that a call's q / k / v are not written by the kernel launched just before it."""
        check(lib.tqb_pqo_cache_set_overlap(self._h, 1 if enabled else 0))

    def _host(self, t):
        return 0 if t.is_cuda else 1

    def prefill(self, layer, k, v, q=None):
        """pqo.rs:184-200: returns the originals on the first call, else the full dequantized cache."""
        k, v = k.contiguous(), v.contiguous()
        new_tokens = k.shape[2]
        old = self.seq_len(layer) if 0 <= layer < self.config.num_layers else 0
        k_out = v_out = None
        if old > 0:
            shape = (self.config.batch, self.config.num_kv_heads, old + new_tokens, self.config.head_dim)
            k_out = torch.empty(shape, dtype=k.dtype, device=k.device)
            v_out = torch.empty(shape, dtype=k.dtype, device=k.device)
        check(lib.tqb_pqo_cache_prefill(self._h, layer, _ptr(k), _ptr(v), _dtype_code(k.dtype), new_tokens, _ptr(k_out),
                                        _ptr(v_out), self._host(k), _stream()))
        if old == 0:
            return DequantResult(k, v)
        if not k.is_cuda:
            torch.cuda.current_stream().synchronize()
        return DequantResult(k_out, v_out)

    def decode(self, layer, k, v, q, config, out=None):
        """pqo.rs:202-222 on the CUDA path: DecodeOutput::Fused([batch, Hq, 1, head_dim])."""
        k, v, q = k.contiguous(), v.contiguous(), q.contiguous()
        hq = q.shape[1]
        if out is None:
            out = torch.empty_like(q)
        check(lib.tqb_pqo_cache_decode(self._h, layer, _ptr(k), _ptr(v), _ptr(q), _dtype_code(k.dtype), hq,
                                       config.softmax_scale, _ptr(out), self._host(k), _stream()))
        return DecodeOutput(fused=out)

    def prefill_attend(self, layer, k, v, q, config):
        """Prefill with the attention done over the packed cache (no counterpart in pqo.rs, whose prefill returns the
        dequantized cache): stores the chunk, then causal attention of its queries over everything stored.
        k, v [batch, Hkv, T, D]; q [batch, Hq, T, D] (device tensors); returns [batch, Hq, T, D]."""
        k, v = k.contiguous(), v.contiguous()
        b, hq, t, d = q.shape
        qt = q.permute(2, 0, 1, 3).contiguous()            # [T, batch * Hq, D]
        out = torch.empty_like(qt)
        check(lib.tqb_pqo_cache_prefill_attend(self._h, layer, _ptr(k), _ptr(v), _ptr(qt), _dtype_code(k.dtype), t, hq,
                                               config.softmax_scale, _ptr(out), _stream()))
        return out.view(t, b, hq, d).permute(1, 2, 0, 3).contiguous()

    def host_sync(self):
        """Blocks until the results of earlier decode() calls with host tensors have reached the host."""
        check(lib.tqb_pqo_cache_host_sync(self._h))

    def attend_partial(self, layer, q, softmax_scale):
        """Shard-local result for sequence-parallel decode: (un-normalised out [B*Hq, D] f32, lse [B*Hq, 2])."""
        q = q.contiguous()
        hq = q.shape[1]
        n = self.config.batch * hq
        out = torch.empty((n, self.config.head_dim), dtype=torch.float32, device=q.device)
        lse = torch.empty((n, 2), dtype=torch.float32, device=q.device)
        check(lib.tqb_pqo_cache_attend_partial(self._h, layer, _ptr(q), _dtype_code(q.dtype), hq, softmax_scale, _ptr(out),
                                               _ptr(lse), _stream()))
        return out, lse

    def dequantize_full(self, layer, dtype=torch.float32):
        n = self.seq_len(layer)
        shape = (self.config.batch, self.config.num_kv_heads, n, self.config.head_dim)
        k = torch.empty(shape, dtype=dtype, device=_dev())
        v = torch.empty(shape, dtype=dtype, device=_dev())
        check(lib.tqb_pqo_cache_dequantize_full(self._h, layer, _ptr(k), _ptr(v), _dtype_code(dtype), 0, _stream()))
        return k, v

    def seq_len(self, layer):
        n = int(lib.tqb_pqo_cache_seq_len(self._h, layer))
        if n < 0:
            raise LayerOutOfRange(f"layer index {layer} out of range (num_layers = {self.config.num_layers})")
        return n

    def capacity(self, layer):
        return int(lib.tqb_pqo_cache_capacity(self._h, layer))

    def reset(self):
        check(lib.tqb_pqo_cache_reset(self._h))

    def memory_usage(self):
        return int(lib.tqb_pqo_cache_memory_usage(self._h))

    def export_layer(self, layer, host=True):
        """The layer's stored rows without capacity padding: (k_indices, k_scales, v_indices, v_scales) with
        indices [batch * Hkv, seq_len, packed_dim] u8 and scales [batch * Hkv, seq_len, head_dim / 32] i16 (f16 bits)."""
        n, heads = self.seq_len(layer), self.config.batch * self.config.num_kv_heads
        dev = "cpu" if host else _dev()
        pd, nb = self.config.head_dim * self.config.bits // 8, self.config.head_dim // 32
        ki, vi = (torch.empty((heads, n, pd), dtype=torch.uint8, device=dev) for _ in range(2))
        ks, vs = (torch.empty((heads, n, nb), dtype=torch.int16, device=dev) for _ in range(2))
        check(lib.tqb_pqo_cache_export_layer(self._h, layer, _ptr(ki), _ptr(ks), _ptr(vi), _ptr(vs), 1 if host else 0, _stream()))
        return ki, ks, vi, vs

    def layer_ptrs(self, layer):
        ptrs = [ctypes.c_void_p() for _ in range(4)]
        check(lib.tqb_pqo_cache_layer_ptrs(self._h, layer, *[ctypes.byref(p) for p in ptrs]))
        return [p.value for p in ptrs]


class TqCache:
    """src/cache/tq.rs:21-412: polar codes (outlier_blocks = 0) plus a QJL sign sketch of the key
    residual.  CUDA tensors only.  k, v: [batch, Hkv, seq, head_dim]; q: [batch, Hq, q_len, head_dim]."""

    def __init__(self, config):
        self.config = config
        self._h = ctypes.c_void_p()
        c = config._c()
        check(lib.tqb_tq_cache_create(ctypes.byref(c), ctypes.byref(self._h)))

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            lib.tqb_tq_cache_destroy(h)
            self._h = None

    def seq_len(self, layer):
        n = int(lib.tqb_tq_cache_seq_len(self._h, layer))
        if n < 0:
            raise LayerOutOfRange(f"layer index {layer} out of range (num_layers = {self.config.num_layers})")
        return n

    def prefill(self, layer, k, v, q):
        """tq.rs:263-288: DequantResult with the originals (first call) or the dequantized cache, and logit_bias."""
        k, v, q = k.contiguous(), v.contiguous(), q.contiguous()
        new_tokens, hq, q_len = k.shape[2], q.shape[1], q.shape[2]
        old = self.seq_len(layer)
        total = old + new_tokens
        cfg = self.config
        k_out = v_out = None
        if old > 0:
            k_out = torch.empty((cfg.batch, cfg.num_kv_heads, total, cfg.head_dim), dtype=k.dtype, device=k.device)
            v_out = torch.empty_like(k_out)
        bias = torch.empty((cfg.batch, hq, q_len, total), dtype=q.dtype, device=q.device)
        check(lib.tqb_tq_cache_prefill(self._h, layer, _ptr(k), _ptr(v), _ptr(q), _dtype_code(k.dtype), new_tokens, hq, q_len,
                                       _ptr(k_out), _ptr(v_out), _ptr(bias), _stream()))
        return DequantResult(k if old == 0 else k_out, v if old == 0 else v_out, bias)

    def decode(self, layer, k, v, q, config=None):
        """tq.rs:290-311: DecodeOutput::Dequantized(k, v, logit_bias) over every stored token."""
        k, v, q = k.contiguous(), v.contiguous(), q.contiguous()
        hq = q.shape[1]
        total = self.seq_len(layer) + 1
        cfg = self.config
        k_out = torch.empty((cfg.batch, cfg.num_kv_heads, total, cfg.head_dim), dtype=k.dtype, device=k.device)
        v_out = torch.empty_like(k_out)
        bias = torch.empty((cfg.batch, hq, 1, total), dtype=q.dtype, device=q.device)
        check(lib.tqb_tq_cache_decode(self._h, layer, _ptr(k), _ptr(v), _ptr(q), _dtype_code(k.dtype), hq, _ptr(k_out),
                                      _ptr(v_out), _ptr(bias), _stream()))
        return DecodeOutput(dequantized=DequantResult(k_out, v_out, bias))

    def decode_fused(self, layer, k, v, q, config):
        """Append, then fused attention with the in-kernel QJL correction (tq_attention_kernel.cu:197-231)."""
        k, v, q = k.contiguous(), v.contiguous(), q.contiguous()
        out = torch.empty_like(q)
        check(lib.tqb_tq_cache_decode_fused(self._h, layer, _ptr(k), _ptr(v), _ptr(q), _dtype_code(k.dtype), q.shape[1],
                                            config.softmax_scale, _ptr(out), _stream()))
        return DecodeOutput(fused=out)

    def reset(self):
        check(lib.tqb_tq_cache_reset(self._h))

    def memory_usage(self):
        return int(lib.tqb_tq_cache_memory_usage(self._h))
