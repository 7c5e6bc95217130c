"""turboquant_b200: B200-native engine for the TurboQuant quantize -> pack -> attend path.

The package is a thin host layer over libtqb200.so (hand-written CUDA for sm_100a, C ABI in
include/tqb200.h).  Importing it loads the library and fails if it has not been built.
"""
from ._lib import lib, declared_symbols  # noqa: F401
from .api import (  # noqa: F401
    ALL_BLOCKS, DEFAULT_QJL_SEED, DEFAULT_ROTATION_SEED, QUANT_BLOCK_SIZE, AttendConfig, CacheConfig, DecodeOutput,
    DequantResult, DimensionMismatch, InvalidDimension, LayerOutOfRange, PackedBlock, PeerTimeout, PqoCache, QjlBlock,
    QuantizedKVCache, QuantNormMode, RangeOutOfBounds, TqbRuntimeError, TqCache, TurboQuantConfig, TurboQuantError,
    UnsupportedBits, block_dequantize, block_quantize, chunk_attention, decode_attention, dequantize_batch, dequantize_rotated,
    dequantize_vec, estimate_inner_product, lse_combine, pack_indices, packed_bytes, precompute_query_projections,
    qjl_attention_scores, qjl_quantize_batch, quantize_batch, quantize_vec, quantize_with_qjl, query_projections,
    rademacher_bits, unpack_indices, weighted_values)
