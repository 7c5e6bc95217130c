"""Seeded random shapes: the tensor-core decode kernels against the general kernel (which the other tests
pin to the oracle), through every option that changes the code path: partitions, TMA staging, fused append,
query dtype, group size, ragged lengths and strides."""
import numpy as np
import pytest
import torch

import turboquant_b200 as tq

pytestmark = pytest.mark.gpu


def _case(seed):
    rng = np.random.default_rng(seed)
    bits = int(rng.choice([3, 4]))
    g = int(rng.choice([1, 2, 3, 4, 5, 8]))
    hkv = int(rng.integers(1, 5))
    L = int(rng.choice([1, 2, 15, 16, 17, 63, 64, 65, 127, 129, 500, 1023, 2049, 3000]))
    stride = L + int(rng.choice([0, 1, 2, 7, 64]))
    parts = int(rng.choice([0, 1, 2, 5]))
    dtype = [torch.float32, torch.bfloat16, torch.float16][int(rng.integers(0, 3))]
    return bits, g, hkv, L, stride, parts, dtype


@pytest.mark.parametrize("seed", range(40))
def test_random_shape_matches_general_kernel(seed):
    bits, g, hkv, L, stride, parts, dtype = _case(seed)
    gen = torch.Generator(device="cuda").manual_seed(seed)
    k = torch.randn((hkv * stride, 128), generator=gen, device="cuda")
    v = torch.randn((hkv * stride, 128), generator=gen, device="cuda")
    k[:, 5] *= 8
    ki, ks = tq.block_quantize(k, bits)
    vi, vs = tq.block_quantize(v, bits)
    ki, ks, vi, vs = (t.view(hkv, stride, -1) for t in (ki, ks, vi, vs))
    q = (torch.randn((hkv * g, 128), generator=gen, device="cuda") * 0.3).to(dtype)
    want = tq.decode_attention(q, ki, ks, vi, vs, L, bits, 0.0884, force_general=True, out_dtype=torch.float32)
    tol = 2e-5 if bits == 4 else 3e-4
    for tma in (False, True):
        got = tq.decode_attention(q, ki, ks, vi, vs, L, bits, 0.0884, num_partitions=parts, tma=tma, out_dtype=torch.float32)
        assert (got - want).abs().max().item() < tol, (bits, g, hkv, L, stride, parts, dtype, tma)
    # fused append of the last token: same cache bytes as a separate quantize, same output
    if L >= 1:
        newk = k.view(hkv, stride, 128)[:, L - 1].contiguous().to(dtype)
        newv = v.view(hkv, stride, 128)[:, L - 1].contiguous().to(dtype)
        c2 = [t.clone() for t in (ki, ks, vi, vs)]
        for t in c2:
            t[:, L - 1] = 0
        ref = [t.clone() for t in c2]
        tq.block_quantize(newk, bits, out=(ref[0], ref[1]), rows_per_group=1, group_stride=stride, row_offset=L - 1)
        tq.block_quantize(newv, bits, out=(ref[2], ref[3]), rows_per_group=1, group_stride=stride, row_offset=L - 1)
        want2 = tq.decode_attention(q, *ref, L, bits, 0.0884, force_general=True, out_dtype=torch.float32)
        got2 = tq.decode_attention(q, *c2, L, bits, 0.0884, num_partitions=parts, append=(newk, newv), out_dtype=torch.float32)
        for a, b in zip(c2, ref):
            assert torch.equal(a, b)
        assert (got2 - want2).abs().max().item() < tol
