"""ctypes wrapper around oracle/liboracle.so, the CPU restatement of the reference.

Test infrastructure: imported only by tests, the smoke check and the benchmark's CPU
baseline.  Builds the oracle with `make` when the shared object is missing.
"""
import ctypes
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
SO = os.path.join(ORACLE_DIR, "liboracle.so")


def build():
    src = os.path.join(ORACLE_DIR, "tq_oracle.cpp")
    if not os.path.exists(SO) or os.path.getmtime(SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", ORACLE_DIR, "liboracle.so"], stdout=subprocess.DEVNULL)
    return SO


_o = ctypes.CDLL(build())
_o.tqo_packed_len.restype = ctypes.c_size_t
_o.tqo_sign.restype = ctypes.c_float
_o.tqo_rademacher_sign.restype = ctypes.c_float
_o.tqo_f16_to_f32.restype = ctypes.c_float
_o.tqo_f32_to_f16.restype = ctypes.c_uint16
u64, i64, sz = ctypes.c_uint64, ctypes.c_int64, ctypes.c_size_t


def P(a):
    return a.ctypes.data_as(ctypes.c_void_p) if a is not None else None


def _ok(rc):
    if rc != 0:
        raise ValueError(f"oracle error class {rc}")


def packed_len(bits, count):
    return int(_o.tqo_packed_len(bits, sz(count)))


def pack_indices(bits, idx):
    idx = np.ascontiguousarray(idx, np.uint8)
    out = np.zeros(packed_len(bits, idx.size), np.uint8)
    _o.tqo_pack_indices(bits, P(idx), sz(idx.size), P(out))
    return out


def unpack_indices(bits, packed, count):
    packed = np.ascontiguousarray(packed, np.uint8)
    out = np.zeros(count, np.uint8)
    _o.tqo_unpack_indices(bits, P(packed), sz(count), P(out))
    return out


def sign_pattern(dim, seed):
    out = np.zeros(dim, np.float32)
    _o.tqo_sign_pattern(dim, u64(seed), P(out))
    return out


def rademacher_sign(seed, row, col):
    return float(_o.tqo_rademacher_sign(u64(seed), row, col))


def rademacher_matrix(dim, seed):
    return np.array([[rademacher_sign(seed, r, c) for c in range(dim)] for r in range(dim)], np.float32)


def wht(data):
    d = np.ascontiguousarray(data, np.float32).copy()
    _o.tqo_wht_inplace(P(d), d.size)
    return d


def codebook(bits, dim):
    c = np.zeros(1 << bits, np.float64)
    b = np.zeros((1 << bits) - 1, np.float64)
    n = _o.tqo_codebook(bits, dim, P(c), P(b))
    if n < 0:
        raise ValueError("no static codebook")
    return c, b


def nearest_centroid(bits, dim, v):
    _o.tqo_nearest_centroid.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_double]
    return int(_o.tqo_nearest_centroid(bits, dim, float(v)))


def f32_to_f16_bits(x):
    return int(_o.tqo_f32_to_f16(ctypes.c_float(x)))


def f16_bits_to_f32(h):
    return float(_o.tqo_f16_to_f32(ctypes.c_uint16(h)))


def pseudo_random_vec(dim, seed):
    out = np.zeros(dim, np.float32)
    _o.tqo_pseudo_random_vec(dim, u64(seed), P(out))
    return out


def lcg_normal_vectors(seed, n, dim):
    out = np.zeros((n, dim), np.float32)
    _o.tqo_lcg_normal_vectors(u64(seed), n, dim, P(out))
    return out


def quantize_batch(bits, dim, seed, x, nthreads=1):
    x = np.ascontiguousarray(x, np.float32).reshape(-1, dim)
    n = len(x)
    packed = np.zeros((n, packed_len(bits, dim)), np.uint8)
    scales = np.zeros(n, np.uint16)
    _ok(_o.tqo_quantize_batch(bits, dim, u64(seed), P(x), i64(n), P(packed), P(scales), nthreads))
    return packed, scales


def dequantize_batch(bits, dim, seed, packed, scales, nthreads=1):
    packed = np.ascontiguousarray(packed, np.uint8)
    scales = np.ascontiguousarray(scales, np.uint16)
    n = len(scales)
    out = np.zeros((n, dim), np.float32)
    _ok(_o.tqo_dequantize_batch(bits, dim, u64(seed), P(packed), P(scales), i64(n), P(out), nthreads))
    return out


def dequantize_rotated_batch(bits, dim, packed, scales):
    packed = np.ascontiguousarray(packed, np.uint8)
    scales = np.ascontiguousarray(scales, np.uint16)
    n = len(scales)
    out = np.zeros((n, dim), np.float32)
    _ok(_o.tqo_dequantize_rotated_batch(bits, dim, P(packed), P(scales), i64(n), P(out)))
    return out


def qjl_quantize_batch(bits, dim, rot_seed, qjl_seed, x, nthreads=1):
    x = np.ascontiguousarray(x, np.float32).reshape(-1, dim)
    n = len(x)
    packed = np.zeros((n, packed_len(bits - 1, dim)), np.uint8)
    scales = np.zeros(n, np.uint16)
    signs = np.zeros((n, dim // 8), np.uint8)
    rnorms = np.zeros(n, np.uint16)
    _ok(_o.tqo_qjl_quantize_batch(bits, dim, u64(rot_seed), u64(qjl_seed), P(x), i64(n), P(packed), P(scales), P(signs),
                                  P(rnorms), nthreads))
    return packed, scales, signs, rnorms


def qjl_signs(residual, dim, qjl_seed):
    residual = np.ascontiguousarray(residual, np.float32)
    out = np.zeros(dim // 8, np.uint8)
    _o.tqo_qjl_signs(P(residual), dim, u64(qjl_seed), P(out))
    return out


def query_projections(q, dim, qjl_seed):
    q = np.ascontiguousarray(q, np.float32)
    rq = np.zeros(dim, np.float32)
    _o.tqo_query_projections(P(q), dim, u64(qjl_seed), P(rq))
    return rq


def attention_scores(bits, dim, rot_seed, qjl_seed, q, packed, scales, signs, rnorms, nthreads=1):
    q = np.ascontiguousarray(q, np.float32)
    n = len(scales)
    out = np.zeros(n, np.float32)
    _ok(_o.tqo_attention_scores(bits, dim, u64(rot_seed), u64(qjl_seed), P(q), P(np.ascontiguousarray(packed)),
                                P(np.ascontiguousarray(scales)), P(np.ascontiguousarray(signs)),
                                P(np.ascontiguousarray(rnorms)), i64(n), P(out), nthreads))
    return out


def weighted_values(bits, dim, rot_seed, w, packed, scales):
    w = np.ascontiguousarray(w, np.float32)
    out = np.zeros(dim, np.float32)
    _ok(_o.tqo_weighted_values(bits, dim, u64(rot_seed), P(w), P(np.ascontiguousarray(packed)),
                               P(np.ascontiguousarray(scales)), i64(len(w)), P(out)))
    return out


def block_codebook(cb_bits, norm_mode):
    c = np.zeros(1 << cb_bits, np.float32)
    b = np.zeros((1 << cb_bits) - 1, np.float32)
    n = _o.tqo_block_codebook(cb_bits, norm_mode, P(c), P(b))
    if n < 0:
        raise ValueError("bad codebook request")
    return c, b


def block_signs():
    out = np.zeros(32, np.float32)
    _o.tqo_block_signs(P(out))
    return out


def block_rotate(x):
    """Forward rotation of 32-blocks (the input the reference hands to tq_quant_maxnorm_batch)."""
    x = np.ascontiguousarray(x, np.float32).reshape(-1, 32)
    out = np.zeros_like(x)
    _o.tqo_block_rotate(P(x), i64(len(x)), P(out))
    return out


def _ob(outlier_blocks, head_dim):
    return head_dim // 32 if outlier_blocks < 0 else outlier_blocks


def block_quantize(bits, head_dim, norm_mode, outlier_blocks, x, nthreads=1):
    x = np.ascontiguousarray(x, np.float32).reshape(-1, head_dim)
    n = len(x)
    packed = np.zeros((n, head_dim * bits // 8), np.uint8)
    scales = np.zeros((n, head_dim // 32), np.uint16)
    _ok(_o.tqo_block_quantize(bits, head_dim, norm_mode, _ob(outlier_blocks, head_dim), P(x), i64(n), P(packed), P(scales),
                              nthreads))
    return packed, scales


def block_dequantize(bits, head_dim, norm_mode, outlier_blocks, packed, scales, nthreads=1):
    packed = np.ascontiguousarray(packed, np.uint8).reshape(-1, head_dim * bits // 8)
    scales = np.ascontiguousarray(scales, np.uint16).reshape(-1, head_dim // 32)
    n = len(packed)
    out = np.zeros((n, head_dim), np.float32)
    _ok(_o.tqo_block_dequantize(bits, head_dim, norm_mode, _ob(outlier_blocks, head_dim), P(packed), P(scales), i64(n),
                                P(out), nthreads))
    return out


def block_attention(bits, head_dim, norm_mode, outlier_blocks, q, k_idx, k_sc, v_idx, v_sc, kv_len, softmax_scale,
                    qjl=None, nthreads=1, return_scores=False):
    """q [Hq, D]; k_idx/v_idx [Hkv, stride, pd] u8; k_sc/v_sc [Hkv, stride, D/32] u16."""
    q = np.ascontiguousarray(q, np.float32)
    hq = q.shape[0]
    hkv, stride = k_idx.shape[0], k_idx.shape[1]
    out = np.zeros((hq, head_dim), np.float32)
    scores = np.zeros((hq, kv_len), np.float32) if return_scores else None
    signs = norms = rq = None
    if qjl is not None:
        signs, norms, rq = (np.ascontiguousarray(qjl[0], np.uint8), np.ascontiguousarray(qjl[1], np.uint16),
                            np.ascontiguousarray(qjl[2], np.float32))
    _o.tqo_block_attention.argtypes = [ctypes.c_int] * 4 + [ctypes.c_void_p] * 8 + [ctypes.c_int] * 5 + [
        ctypes.c_float, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int]
    _ok(_o.tqo_block_attention(bits, head_dim, norm_mode, _ob(outlier_blocks, head_dim), P(q),
                               P(np.ascontiguousarray(k_idx, np.uint8)), P(np.ascontiguousarray(k_sc, np.uint16)),
                               P(np.ascontiguousarray(v_idx, np.uint8)), P(np.ascontiguousarray(v_sc, np.uint16)),
                               P(signs), P(norms), P(rq), 1 if qjl is not None else 0, hq, hkv, kv_len, stride,
                               softmax_scale, P(out), P(scores), nthreads))
    return (out, scores) if return_scores else out


def sdpa(q, k, v, softmax_scale, bias=None):
    """q [Hq, D]; k, v [Hkv, L, D] f32."""
    q = np.ascontiguousarray(q, np.float32)
    k = np.ascontiguousarray(k, np.float32)
    v = np.ascontiguousarray(v, np.float32)
    hq, d = q.shape
    hkv, L = k.shape[0], k.shape[1]
    out = np.zeros((hq, d), np.float32)
    _o.tqo_sdpa.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int] * 4 + [ctypes.c_float, ctypes.c_void_p]
    _o.tqo_sdpa(P(q), P(k), P(v), P(np.ascontiguousarray(bias, np.float32)) if bias is not None else None, hq, hkv, L, d,
                softmax_scale, P(out))
    return out
