"""The C-ABI library loads without a GPU, exports every symbol the header declares, and its
host-only entry points agree with the oracle.  No kernel is launched here."""
import ctypes
import os

import numpy as np
import pytest

import oracle_lib as o
import turboquant_b200 as tq
from turboquant_b200._lib import TqbConfig, declared_symbols, lib

P = o.P


def test_every_declared_symbol_is_exported():
    names = declared_symbols()
    assert len(names) >= 50
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing
    for n in ("tq_dequant_batch", "tq_quant_maxnorm_batch", "tq_pack_indices", "tq_fused_attention"):
        assert n in names  # the reference's four FFI symbols (src/cache/cuda/ffi.rs:10-79)


def test_no_product_file_touches_the_oracle():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    pkg = os.path.join(root, "turboquant_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.lower() or f == "build.py", f
    assert "oracle" not in open(os.path.join(root, "include", "tqb200.h")).read().lower()


def test_status_strings_and_version():
    assert lib.tqb_version() == 1
    assert lib.tqb_status_string(0) == b"ok"
    assert b"dimension" in lib.tqb_status_string(1)


def test_packed_bytes():
    for bits in (2, 3, 4):
        for n in (0, 1, 5, 8, 31, 32, 128, 256):
            assert lib.tqb_packed_bytes(bits, n) == o.packed_len(bits, n)
    assert lib.tqb_packed_bytes(5, 8) == 0


def test_config_validation_order_and_codes():
    # src/packed/mod.rs:124-132: bits is checked before dim
    assert lib.tqb_config_validate(ctypes.byref(TqbConfig(5, 100, 0))) == 2
    assert lib.tqb_config_validate(ctypes.byref(TqbConfig(3, 100, 0))) == 1
    assert lib.tqb_config_validate(ctypes.byref(TqbConfig(3, 128, 0))) == 0
    assert lib.tqb_config_validate(ctypes.byref(TqbConfig(3, 512, 0))) == 9   # valid, but no static table
    with pytest.raises(tq.UnsupportedBits):
        tq.TurboQuantConfig(1, 128)
    with pytest.raises(tq.InvalidDimension):
        tq.TurboQuantConfig(3, 96)
    assert tq.TurboQuantConfig(3, 128).with_seed(42).rotation_seed == 42
    assert tq.TurboQuantConfig(3, 128).rotation_seed == 0


@pytest.mark.parametrize("bits,dim", [(b, d) for b in (2, 3, 4) for d in (32, 64, 128, 256)])
def test_codebooks_equal_the_oracle_tables(bits, dim):
    c = np.zeros(1 << bits)
    b = np.zeros((1 << bits) - 1)
    assert lib.tqb_get_codebook(bits, dim, P(c), P(b)) == 0
    oc, ob = o.codebook(bits, dim)
    assert np.array_equal(c, oc) and np.array_equal(b, ob)


def test_sign_patterns_and_block_tables_equal_the_oracle():
    for seed in (0, 7, 42):
        s = np.zeros(128, np.float32)
        assert lib.tqb_generate_sign_pattern(128, seed, P(s)) == 0
        assert np.array_equal(s, o.sign_pattern(128, seed))
    s32 = np.zeros(32, np.float32)
    lib.tqb_block_sign_pattern(P(s32))
    assert np.array_equal(s32, o.block_signs())
    for cb_bits in (2, 3, 4):
        for nm in (0, 1):
            c = np.zeros(1 << cb_bits, np.float32)
            b = np.zeros((1 << cb_bits) - 1, np.float32)
            assert lib.tqb_block_codebook(cb_bits, nm, P(c), P(b)) == 1 << cb_bits
            oc, ob = o.block_codebook(cb_bits, nm)
            assert np.array_equal(c, oc) and np.array_equal(b, ob)


def test_rademacher_bits_equal_the_reference_hash():
    ref = np.load(os.path.join(os.path.dirname(__file__), "golden", "ref_primitives.npz"))
    for seed in (42, 12345):
        bits = np.zeros((128, 4), np.uint32)
        assert lib.tqb_qjl_rademacher_bits(128, seed, P(bits)) == 0
        neg = (bits[:, :, None] >> np.arange(32)[None, None, :]) & 1
        assert np.array_equal(np.where(neg.reshape(128, 128) == 1, -1, 1), ref[f"rademacher_{seed}"])


def test_python_pack_unpack_match_the_reference_layout():
    ref = np.load(os.path.join(os.path.dirname(__file__), "golden", "ref_primitives.npz"))
    for bits in (2, 3, 4):
        for codes, packed in zip(ref[f"codes_{bits}"], ref[f"packed_{bits}"]):
            assert np.array_equal(tq.pack_indices(bits, codes), packed)
            assert np.array_equal(tq.unpack_indices(bits, packed, 128), codes)
    blk = tq.PackedBlock.new(3, 0x3C00, np.arange(128) % 8)
    assert blk.size_bytes() == 50 and np.array_equal(blk.unpack(128), np.arange(128) % 8)   # src/quantize.rs:648-658
    assert blk.scale_f32() == 1.0


def test_argument_errors_are_reported_before_any_launch():
    cfg = TqbConfig(3, 128, 42)
    # null pointers / bad sizes are rejected on the host (no device is touched)
    assert lib.tqb_quantize_batch(ctypes.byref(cfg), None, 4, None, None, None) == 6
    assert lib.tqb_quantize_batch(ctypes.byref(cfg), None, -1, None, None, None) == 7
    assert lib.tqb_quantize_batch(ctypes.byref(cfg), None, 0, None, None, None) == 0       # empty input
    assert lib.tqb_block_quantize(5, 128, 0, -1, None, 0, 1, 0, None, None, 0, 0, 0, None) == 2
    assert lib.tqb_block_quantize(3, 100, 0, -1, None, 0, 1, 0, None, None, 0, 0, 0, None) == 1
    assert lib.tqb_block_quantize(3, 128, 0, -1, None, 0, 0, 0, None, None, 0, 0, 0, None) == 0
    assert lib.tqb_dequant_batch(None, None, None, None, None, 0, 32, 3, 12, None) == 0     # tq_dequant_kernel.cu:116
    assert lib.tqb_dequant_batch(None, None, None, None, None, 4, 32, 3, 13, None) == 3
    assert lib.tqb_fused_attention(*([None] * 14), 0, 4, 2, 128, 0, 0, 48, 4, 3, 1.0, 1, None) == 0  # kv_len == 0
    assert lib.tqb_decode_attention(None, None) == 6
    assert lib.tqb_decode_num_partitions(8, 1024) >= 1
    assert lib.tqb_decode_scratch_bytes(16, 128, 4) == 256 + 4 * 16 * 4 * 130   # merge tickets + partials


def test_partition_choosers_are_host_functions():
    """tqb_decode_num_partitions: one to two residencies' worth of CTAs (148 SMs x 4), the single residency rounded down;
    tqb_decode_num_partitions_overlapped: about one CTA per SM and launch, partitions of at least 768 tokens."""
    from turboquant_b200._lib import lib
    assert lib.tqb_decode_num_partitions(512, 8192) == 2        # 2 x 592 / 512 = 2, partitions of 4096 tokens
    assert lib.tqb_decode_num_partitions(64, 8192) == 9         # 592 / 64 rounded down: 576 CTAs, one wave
    assert lib.tqb_decode_num_partitions(8, 131072) == 74       # one residency: 148 partitions would need the two-level merge twice as long
    assert lib.tqb_decode_num_partitions(8, 100) == 2           # never below 64 tokens per partition
    assert lib.tqb_decode_num_partitions(1000, 8192) == 1
    assert lib.tqb_decode_num_partitions_overlapped(512, 8192) == 1
    assert lib.tqb_decode_num_partitions_overlapped(64, 8192) == 2
    assert lib.tqb_decode_num_partitions_overlapped(8, 131072) == 18
    assert lib.tqb_decode_num_partitions_overlapped(8, 1024) == 1
    assert lib.tqb_decode_num_partitions_overlapped(0, 5) == 1


def test_public_header_is_plain_c():
    """include/tqb200.h is what a foreign-function binding reads: it must compile as C99 on its own (no C++ or CUDA
    types in the signatures)."""
    import os
    import shutil
    import subprocess
    import tempfile
    cc = shutil.which("gcc") or shutil.which("cc")
    if cc is None:
        pytest.skip("no C compiler")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    with tempfile.TemporaryDirectory() as td:
        src = os.path.join(td, "hdr.c")
        with open(src, "w") as f:
            f.write('#include "tqb200.h"\nint main(void) { return 0; }\n')
        res = subprocess.run([cc, "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", "-fsyntax-only",
                              "-I", os.path.join(root, "include"), src], capture_output=True, text=True)
    assert res.returncode == 0, res.stderr


def test_argument_checks_that_need_no_gpu():
    """Entry points validate their arguments on the host before they touch the device."""
    from turboquant_b200._lib import lib
    x = ctypes.c_void_p()
    assert lib.tqb_peer_exchange_create(9, 0, 8, 128, ctypes.byref(x)) == 7       # more than 8 ranks
    assert lib.tqb_peer_exchange_create(2, 2, 8, 128, ctypes.byref(x)) == 7       # rank outside the world
    assert lib.tqb_peer_exchange_create(2, 0, 0, 128, ctypes.byref(x)) == 7       # no query heads
    assert lib.tqb_peer_exchange_create(2, 0, 8, 64, ctypes.byref(x)) == 9        # head_dim the pushing kernels do not cover
    assert lib.tqb_peer_exchange_create(2, 0, 8, 128, None) == 6                  # NULL out pointer
    assert lib.tqb_pqo_cache_set_overlap(None, 1) == 6
    assert lib.tqb_peer_exchange_check(None) in (10, 13) or lib.tqb_peer_exchange_timeouts(None) == -1
    assert lib.tqb_decode_scratch_bytes(0, 128, 4) == 0
    # tickets (1 + G words per query head, rounded to 256 bytes) + partials + group partials; G = ceil(P / 8) above 16
    assert lib.tqb_decode_scratch_bytes(64, 128, 4) == 256 + 4 * 64 * 4 * 130
    assert lib.tqb_decode_scratch_bytes(64, 128, 18) == 1024 + 4 * 64 * (18 + 3) * 130
