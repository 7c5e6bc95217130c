"""The allocation-free decode entry point, through the C ABI.

`tqb_decode_attention_static` serves hosts that cannot allocate device memory at call time (all
memory already given to their own pool, or no tolerance for the device-wide synchronisation an
allocation implies): the split-K partials live in a fixed array inside the library.  The test calls
it several times in a row on different shapes and compares each result with the regular entry point,
which uses a caller-allocated scratch buffer: both run the same kernels, so the outputs must be equal
bit for bit.  This file is collected last on purpose.
"""
import ctypes

import numpy as np
import pytest
import torch

from turboquant_b200._lib import TqbDecodeParams, lib

pytestmark = pytest.mark.gpu


def _case(seed, hq, hkv, kv_len, bits, parts, head_dim=128):
    g = torch.Generator().manual_seed(seed)
    pd = head_dim * bits // 8
    t = dict(
        q=(torch.randn((hq, head_dim), generator=g) / head_dim ** 0.5).cuda(),
        ki=torch.randint(0, 256, (hkv, kv_len, pd), generator=g, dtype=torch.uint8).cuda(),
        vi=torch.randint(0, 256, (hkv, kv_len, pd), generator=g, dtype=torch.uint8).cuda(),
        ks=(torch.rand((hkv, kv_len, head_dim // 32), generator=g) + 0.5).half().cuda(),
        vs=(torch.rand((hkv, kv_len, head_dim // 32), generator=g) + 0.5).half().cuda(),
    )
    p = TqbDecodeParams()
    p.q, p.k_indices, p.k_scales = t["q"].data_ptr(), t["ki"].data_ptr(), t["ks"].data_ptr()
    p.v_indices, p.v_scales = t["vi"].data_ptr(), t["vs"].data_ptr()
    p.q_dtype = p.out_dtype = 0
    p.bits, p.head_dim, p.norm_mode, p.outlier_blocks = bits, head_dim, 0, -1
    p.num_q_heads, p.num_kv_heads, p.kv_len, p.kv_stride = hq, hkv, kv_len, kv_len
    p.num_partitions, p.softmax_scale = parts, 0.0884
    return p, t


def _run(fn, p, scratch):
    out = torch.full((p.num_q_heads, p.head_dim), float("nan"), device="cuda")
    p.out = out.data_ptr()
    p.scratch, p.scratch_bytes = (scratch.data_ptr(), scratch.numel()) if scratch is not None else (None, 0)
    rc = fn(ctypes.byref(p), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, rc
    torch.cuda.synchronize()
    return out.cpu().numpy()


def test_static_scratch_matches_caller_scratch_on_two_calls_in_a_row():
    assert lib.tqb_decode_static_scratch_capacity() == 8 << 20
    # first a wide shape with many partitions, then a smaller one that leaves most of the shared
    # array holding the first call's partials, then a head_dim-64 shape, which the tensor-core kernels do
    # not cover: it runs the general split-K kernel and the stand-alone merge kernel
    for seed, hq, hkv, kv_len, bits, parts, hd in ((1, 64, 16, 3000, 4, 7, 128), (2, 8, 4, 517, 3, 2, 128),
                                                    (3, 12, 4, 700, 3, 3, 64)):
        p, keep = _case(seed, hq, hkv, kv_len, bits, parts, hd)
        scratch = torch.empty(int(lib.tqb_decode_scratch_bytes(hq, hd, parts)), dtype=torch.uint8, device="cuda")
        want = _run(lib.tqb_decode_attention, p, scratch)
        got = _run(lib.tqb_decode_attention_static, p, None)
        assert np.isfinite(got).all()
        assert np.array_equal(got, want)
        del keep


def test_partials_only_is_refused():
    # the partials would stay in the library's array, which the caller cannot address
    p, keep = _case(4, 8, 4, 64, 4, 1)
    p.flags = 1   # TQB_DECODE_PARTIALS_ONLY
    out = torch.zeros((8, 128), device="cuda")
    p.out = out.data_ptr()
    assert lib.tqb_decode_attention_static(ctypes.byref(p), None) == 7   # TQB_ERR_INVALID_ARGUMENT
    del keep


def test_shapes_beyond_the_fixed_array_are_refused():
    p, keep = _case(3, 8, 4, 64, 4, 1)
    p.num_q_heads, p.num_kv_heads, p.num_partitions = 4096, 4, 8      # 4096 x 8 x 130 x 4 B = 17 MB > 8 MiB
    rc = lib.tqb_decode_attention_static(ctypes.byref(p), None)
    assert rc == 12 and b"fixed capacity" in lib.tqb_status_string(rc)
    del keep
