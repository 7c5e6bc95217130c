"""ctypes loader for libtqb200.so (the C ABI declared in include/tqb200.h).

The library is the product: if it has not been built the import fails loudly, and no
Python or CPU implementation stands in for it.
"""
import ctypes
import os
import re

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libtqb200.so")
HEADER_PATH = os.path.join(HERE, "..", "include", "tqb200.h")

c_void_p, c_int, c_int32, c_int64, c_uint64, c_size_t, c_float = (
    ctypes.c_void_p, ctypes.c_int, ctypes.c_int32, ctypes.c_int64, ctypes.c_uint64, ctypes.c_size_t, ctypes.c_float)


class TqbConfig(ctypes.Structure):
    """tqb_config (TurboQuantConfig, src/packed/mod.rs:93-139)."""
    _fields_ = [("bits", c_int32), ("dim", c_int32), ("rotation_seed", c_uint64)]


class TqbCacheConfig(ctypes.Structure):
    """tqb_cache_config (CacheConfig, src/cache/config.rs:52-66)."""
    _fields_ = [("bits", c_int32), ("head_dim", c_int32), ("num_kv_heads", c_int32), ("num_layers", c_int32),
                ("norm_mode", c_int32), ("outlier_blocks", c_int32), ("batch", c_int32), ("reserved", c_int32),
                ("rotation_seed", c_uint64), ("qjl_seed", c_uint64)]


class TqbDecodeParams(ctypes.Structure):
    """tqb_decode_params."""
    _fields_ = [("q", c_void_p), ("k_indices", c_void_p), ("k_scales", c_void_p), ("v_indices", c_void_p),
                ("v_scales", c_void_p), ("out", c_void_p), ("lse_out", c_void_p), ("scratch", c_void_p),
                ("scratch_bytes", c_size_t), ("qjl_signs", c_void_p), ("qjl_norms", c_void_p), ("rq", c_void_p),
                ("qjl_enabled", c_int32), ("q_dtype", c_int32), ("out_dtype", c_int32), ("bits", c_int32),
                ("head_dim", c_int32), ("norm_mode", c_int32), ("outlier_blocks", c_int32), ("num_q_heads", c_int32),
                ("num_kv_heads", c_int32), ("kv_len", c_int32), ("kv_stride", c_int32), ("num_partitions", c_int32),
                ("softmax_scale", c_float), ("flags", c_int32), ("append_k", c_void_p), ("append_v", c_void_p)]


def declared_symbols(header_path=HEADER_PATH):
    """Names of every function declared in the public header."""
    text = open(header_path).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"\b(tqb?_[a-z0-9_]+)\s*\(", text)
    seen, out = set(), []
    for n in names:
        if n not in seen and not n.endswith("_t"):
            seen.add(n)
            out.append(n)
    return out


def _declare(lib):
    P, I, L, U, S, F = c_void_p, c_int32, c_int64, c_uint64, c_size_t, c_float
    sig = {
        "tqb_status_string": (ctypes.c_char_p, [c_int]),
        "tqb_last_cuda_error": (c_int, []),
        "tqb_version": (c_int, []),
        "tq_dequant_batch": (None, [P, P, P, P, P, I, I, I, I, P]),
        "tq_quant_maxnorm_batch": (None, [P, P, P, P, I, I, I, I, I, F, F, P]),
        "tq_pack_indices": (None, [P, P, I, I, I, I, P]),
        "tq_fused_attention": (None, [P] * 14 + [I] * 9 + [F, I, P]),
        "tqb_dequant_batch": (c_int, [P, P, P, P, P, I, I, I, I, P]),
        "tqb_quant_maxnorm_batch": (c_int, [P, P, P, P, I, I, I, I, I, F, F, P]),
        "tqb_pack_indices": (c_int, [P, P, I, I, I, I, P]),
        "tqb_fused_attention": (c_int, [P] * 14 + [I] * 9 + [F, I, P]),
        "tqb_config_validate": (c_int, [P]),
        "tqb_packed_bytes": (S, [I, S]),
        "tqb_get_codebook": (c_int, [I, I, P, P]),
        "tqb_generate_sign_pattern": (c_int, [I, U, P]),
        "tqb_quantize_batch": (c_int, [P, P, L, P, P, P]),
        "tqb_dequantize_batch": (c_int, [P, P, P, L, P, P]),
        "tqb_dequantize_rotated_batch": (c_int, [P, P, P, L, P, P]),
        "tqb_qjl_rademacher_bits": (c_int, [I, U, P]),
        "tqb_qjl_quantize_batch": (c_int, [P, P, P, L, P, P, P, P, P]),
        "tqb_qjl_query_projections": (c_int, [I, P, P, L, P, P]),
        "tqb_qjl_attention_scores": (c_int, [P, P, P, P, P, P, P, L, P, P]),
        "tqb_weighted_values_scratch_bytes": (S, [I]),
        "tqb_weighted_values": (c_int, [P, P, P, P, L, P, P, S, P]),
        "tqb_block_codebook": (c_int, [I, I, P, P]),
        "tqb_block_sign_pattern": (None, [P]),
        "tqb_block_quantize": (c_int, [I, I, I, I, P, I, L, L, P, P, L, L, L, P]),
        "tqb_decode_stage_timeouts": (ctypes.c_longlong, []),
        "tqb_block_quantize_pair": (c_int, [I, I, I, I, P, P, I, L, L, P, P, P, P, L, L, L, P]),
        "tqb_block_dequantize": (c_int, [I, I, I, I, P, P, L, L, L, L, P, I, P]),
        "tqb_decode_num_partitions": (I, [I, I]),
        "tqb_decode_num_partitions_overlapped": (I, [I, I]),
        "tqb_decode_scratch_bytes": (S, [I, I, I]),
        "tqb_decode_attention": (c_int, [P, P]),
        "tqb_chunk_attention": (c_int, [P, ctypes.c_int32, P]),
        "tqb_chunk_umma_timeouts": (ctypes.c_longlong, []),
        "tqb_decode_attention_static": (c_int, [P, P]),
        "tqb_decode_static_scratch_capacity": (S, []),
        "tqb_lse_combine": (c_int, [P, P, I, I, I, P, I, P]),
        "tqb_lse_combine_packed": (c_int, [P, I, I, I, P, I, P]),
        "tqb_pqo_cache_create": (c_int, [P, P]),
        "tqb_pqo_cache_destroy": (None, [P]),
        "tqb_pqo_cache_prefill": (c_int, [P, I, P, P, I, I, P, P, I, P]),
        "tqb_pqo_cache_decode": (c_int, [P, I, P, P, P, I, I, F, P, I, P]),
        "tqb_pqo_cache_prefill_attend": (c_int, [P, I, P, P, P, I, I, I, F, P, P]),
        "tqb_pqo_cache_host_sync": (c_int, [P]),
        "tqb_pqo_cache_dequantize_full": (c_int, [P, I, P, P, I, I, P]),
        "tqb_pqo_cache_seq_len": (L, [P, I]),
        "tqb_pqo_cache_capacity": (L, [P, I]),
        "tqb_pqo_cache_reset": (c_int, [P]),
        "tqb_pqo_cache_set_overlap": (c_int, [P, I]),
        "tqb_pqo_cache_memory_usage": (S, [P]),
        "tqb_pqo_cache_layer_ptrs": (c_int, [P, I, P, P, P, P]),
        "tqb_pqo_cache_export_layer": (c_int, [P, I, P, P, P, P, I, P]),
        "tqb_pqo_cache_attend_partial": (c_int, [P, I, P, I, I, F, P, P, P]),
        "tqb_peer_exchange_create": (c_int, [I, I, I, I, P]),
        "tqb_peer_exchange_destroy": (None, [P]),
        "tqb_peer_exchange_handle": (c_int, [P, P]),
        "tqb_peer_exchange_connect": (c_int, [P, P]),
        "tqb_peer_exchange_connect_local": (c_int, [P, P]),
        "tqb_pqo_cache_attend_push": (c_int, [P, I, P, I, I, F, P, P]),
        "tqb_peer_exchange_combine": (c_int, [P, I, P, I, L, P]),
        "tqb_peer_exchange_timeouts": (ctypes.c_longlong, [P]),
        "tqb_peer_exchange_check": (c_int, [P]),
        "tqb_residual_sketch": (c_int, [I, P, P, I, P, L, P, P, L, L, L, P]),
        "tqb_qjl_logit_bias": (c_int, [I, P, P, P, P, I, I, I, I, I, I, P]),
        "tqb_tq_cache_create": (c_int, [P, P]),
        "tqb_tq_cache_destroy": (None, [P]),
        "tqb_tq_cache_prefill": (c_int, [P, I, P, P, P, I, I, I, I, P, P, P, P]),
        "tqb_tq_cache_decode": (c_int, [P, I, P, P, P, I, I, P, P, P, P]),
        "tqb_tq_cache_decode_fused": (c_int, [P, I, P, P, P, I, I, F, P, P]),
        "tqb_tq_cache_seq_len": (L, [P, I]),
        "tqb_tq_cache_reset": (c_int, [P]),
        "tqb_tq_cache_memory_usage": (S, [P]),
        "tqb_tq_cache_qjl_ptrs": (c_int, [P, I, P, P, P]),
        "tqb_kv_cache_create": (c_int, [P, I, U, P]),
        "tqb_kv_cache_destroy": (None, [P]),
        "tqb_kv_cache_push_batch": (c_int, [P, I, P, P, L, L, P]),
        "tqb_kv_cache_attention_scores": (c_int, [P, I, P, L, P, P]),
        "tqb_kv_cache_weighted_values": (c_int, [P, I, P, L, P, P]),
        "tqb_kv_cache_dequantize_range": (c_int, [P, I, L, L, I, P, P]),
        "tqb_kv_cache_export_packed_range": (c_int, [P, I, L, L, I, P, P, P, P, P]),
        "tqb_kv_cache_import_packed_range": (c_int, [P, I, I, P, P, P, P, L, L, L, I, P]),
        "tqb_kv_cache_entry_count": (L, [P, I]),
        "tqb_kv_cache_num_layers": (I, [P]),
        "tqb_kv_cache_memory_usage": (S, [P]),
        "tqb_kv_cache_fp16_equivalent_memory": (S, [P]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return sig


def load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python turboquant_b200/build.py` "
            "(nvcc, sm_100a). There is no CPU fallback.")
    lib = ctypes.CDLL(LIB_PATH)
    lib._signatures = _declare(lib)
    return lib


lib = load()
