"""GPU parity of the block-32 (cache module) quantize / dequantize kernels and of the
reference's own FFI symbols, against the CPU oracle."""
import ctypes
import os

import numpy as np
import pytest
import torch

import oracle_lib as o
import turboquant_b200 as tq
from turboquant_b200._lib import lib

pytestmark = pytest.mark.gpu
CASES = np.load(os.path.join(os.path.dirname(__file__), "golden", "oracle_cases.npz"))
MODES = [(3, 0, -1, "pqo3"), (4, 0, -1, "pqo4"), (3, 1, -1, "pqo3_l2"), (3, 0, 0, "pq3"), (4, 0, 2, "mix4")]


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def u16(t):
    return t.cpu().numpy().view(np.uint16)


def ptr(t):
    return ctypes.c_void_p(t.data_ptr())


@pytest.mark.parametrize("bits,nm,ob,tag", MODES)
def test_golden_fixture(bits, nm, ob, tag):
    x = CASES["block_x"]
    idx, sc = tq.block_quantize(dev(x), bits, tq.QuantNormMode(nm), ob)
    assert np.array_equal(idx.cpu().numpy(), CASES[f"block_packed_{tag}"])
    assert np.array_equal(u16(sc), CASES[f"block_scales_{tag}"])
    deq = tq.block_dequantize(idx, sc, bits, 128, tq.QuantNormMode(nm), ob).cpu().numpy()
    assert np.array_equal(deq, CASES[f"block_deq_{tag}"])


@pytest.mark.parametrize("bits,nm,ob,tag", MODES + [(4, 0, 0, "pq4")])
@pytest.mark.parametrize("head_dim,n", [(128, 4099), (64, 17), (256, 5), (32, 3)])
def test_random_vs_oracle_bit_exact(bits, nm, ob, tag, head_dim, n):
    rng = np.random.default_rng(n)
    x = rng.standard_normal((n, head_dim)).astype(np.float32) * np.exp(rng.normal(0, 0.5, head_dim)).astype(np.float32)
    ob_eff = min(ob, head_dim // 32) if ob >= 0 else ob
    idx, sc = tq.block_quantize(dev(x), bits, tq.QuantNormMode(nm), ob_eff)
    op, os_ = o.block_quantize(bits, head_dim, nm, ob_eff, x, nthreads=8)
    assert np.array_equal(idx.cpu().numpy(), op)
    assert np.array_equal(u16(sc), os_)
    deq = tq.block_dequantize(idx, sc, bits, head_dim, tq.QuantNormMode(nm), ob_eff).cpu().numpy()
    assert np.array_equal(deq, o.block_dequantize(bits, head_dim, nm, ob_eff, op, os_, nthreads=8))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_half_precision_inputs_match_their_f32_upcast(dtype):
    # the reference casts to f32 first (src/cache/common.rs:88-95); the cast is exact, so codes are unchanged
    x = (torch.randn((1000, 128), generator=torch.Generator().manual_seed(3)) * 3).to(dtype)
    for bits in (3, 4):
        idx, sc = tq.block_quantize(x.cuda(), bits)
        op, os_ = o.block_quantize(bits, 128, 0, -1, x.float().numpy(), nthreads=8)
        assert np.array_equal(idx.cpu().numpy(), op) and np.array_equal(u16(sc), os_)
        deq = tq.block_dequantize(idx, sc, bits, 128, dtype=dtype).float().cpu().numpy()
        want = torch.from_numpy(o.block_dequantize(bits, 128, 0, -1, op, os_)).to(dtype).float().numpy()
        assert np.array_equal(deq, want)


def test_append_row_mapping():
    # CompressedStorage::append (src/cache/storage.rs:145-172): rows land at [head, offset + t]
    heads, new, cap, off = 3, 5, 16, 7
    x = torch.randn((heads * new, 128), generator=torch.Generator().manual_seed(0))
    idx = torch.zeros((heads, cap, 48), dtype=torch.uint8, device="cuda")
    sc = torch.zeros((heads, cap, 4), dtype=torch.int16, device="cuda")
    tq.block_quantize(x.cuda(), 3, out=(idx, sc), rows_per_group=new, group_stride=cap, row_offset=off)
    op, os_ = o.block_quantize(3, 128, 0, -1, x.numpy())
    got = idx.cpu().numpy()
    assert np.array_equal(got[:, off:off + new].reshape(-1, 48), op)
    assert not got[:, :off].any() and not got[:, off + new:].any()
    assert np.array_equal(u16(sc)[:, off:off + new].reshape(-1, 4), os_)


@pytest.mark.parametrize("bits,nm,ob", [(4, 0, -1), (3, 0, -1), (3, 1, -1), (4, 0, 2), (3, 0, 0), (4, 0, 0)])
def test_pair_launch_equals_two_single_launches(bits, nm, ob):
    # K and V of one append in one launch, with the append row mapping
    heads, new, cap, off = 4, 3, 8, 2
    g = torch.Generator().manual_seed(bits * 10 + nm)
    k = torch.randn((heads * new, 128), generator=g).to(torch.bfloat16).cuda()
    v = torch.randn((heads * new, 128), generator=g).to(torch.bfloat16).cuda()
    pd = 16 * bits

    def buffers():
        return (torch.zeros((heads, cap, pd), dtype=torch.uint8, device="cuda"),
                torch.zeros((heads, cap, 4), dtype=torch.int16, device="cuda"))
    ki, ks = buffers(); vi, vs = buffers()
    rc = lib.tqb_block_quantize_pair(bits, 128, nm, ob, k.data_ptr(), v.data_ptr(), 2, heads * new, 0, ki.data_ptr(),
                                     ks.data_ptr(), vi.data_ptr(), vs.data_ptr(), new, cap, off, None)
    assert rc == 0
    ki1, ks1 = buffers(); vi1, vs1 = buffers()
    tq.block_quantize(k, bits, tq.QuantNormMode(nm), ob, out=(ki1, ks1), rows_per_group=new, group_stride=cap, row_offset=off)
    tq.block_quantize(v, bits, tq.QuantNormMode(nm), ob, out=(vi1, vs1), rows_per_group=new, group_stride=cap, row_offset=off)
    torch.cuda.synchronize()
    for a, b in ((ki, ki1), (ks, ks1), (vi, vi1), (vs, vs1)):
        assert torch.equal(a, b)
    assert lib.tqb_block_quantize_pair(bits, 128, nm, ob, k.data_ptr(), None, 2, 4, 0, ki.data_ptr(), ks.data_ptr(),
                                       vi.data_ptr(), vs.data_ptr(), 0, 0, 0, None) == 6   # null pointer


def test_reference_ffi_symbols():
    # the four launchers of src/cache/cuda/ffi.rs:10-79, called with the reference's own argument lists
    rng = np.random.default_rng(2)
    n_vec, hd = 50, 128
    x = rng.standard_normal((n_vec, hd)).astype(np.float32)
    signs = o.block_signs()
    for bits in (3, 4):
        c, b = o.block_codebook(bits, 0)
        # host-side rotation as cuda_quantize_fast does with a matmul (src/cache/cuda/quantize.rs:111-113),
        # here in the oracle's butterfly order
        rot = np.stack([o.wht(blk) * signs for blk in x.reshape(-1, 32)]).astype(np.float32)
        nblocks, bpb = rot.shape[0], 32 * bits // 8
        packed = torch.zeros(nblocks * bpb, dtype=torch.uint8, device="cuda")
        scales = torch.zeros(nblocks, dtype=torch.int16, device="cuda")
        rot_d, b_d, c_d = dev(rot), dev(b), dev(c)   # keep the device copies alive across the asynchronous launches
        lib.tq_quant_maxnorm_batch(ptr(rot_d), ptr(b_d), ptr(packed), ptr(scales), nblocks, 32, bits, len(b), bpb,
                                   float(c[-1]), -1.0, None)
        op, os_ = o.block_quantize(bits, hd, 0, -1, x)
        assert np.array_equal(packed.cpu().numpy(), op.reshape(-1)) and np.array_equal(u16(scales), os_.reshape(-1))
        out = torch.zeros(nblocks * 32, device="cuda")
        sign_dev = dev((signs * (np.float32(1) / np.sqrt(np.float32(32))) * np.sqrt(np.float32(32))).astype(np.float32))
        lib.tq_dequant_batch(ptr(packed), ptr(scales), ptr(c_d), ptr(sign_dev), ptr(out), nblocks, 32, bits, bpb, None)
        assert np.array_equal(out.cpu().numpy().reshape(n_vec, hd), o.block_dequantize(bits, hd, 0, -1, op, os_))
        codes = rng.integers(0, 1 << bits, size=(n_vec, hd), dtype=np.uint8)
        pk = torch.zeros(n_vec * hd * bits // 8, dtype=torch.uint8, device="cuda")
        codes_d = dev(codes)
        lib.tq_pack_indices(ptr(codes_d), ptr(pk), n_vec * 4, 32, bits, bpb, None)
        assert np.array_equal(pk.cpu().numpy(), o.pack_indices(bits, codes.reshape(-1)))
        assert lib.tqb_quant_maxnorm_batch(None, None, None, None, 0, 32, bits, len(b), bpb, 1.0, 1.0, None) == 0


def test_quantize_dequantize_idempotence_at_bulk_size():
    # size-independent property at a bulk-prefill-like size: re-quantizing the dequantized
    # tensor reproduces the same codes almost everywhere and the same reconstruction error
    n = 1 << 18
    x = torch.randn((n, 128), device="cuda", dtype=torch.bfloat16)
    x[:, [5, 70, 101]] *= 8
    for bits, lo, hi in ((3, 0.85, 1.0), (4, 0.92, 1.0)):
        idx, sc = tq.block_quantize(x, bits)
        deq = tq.block_dequantize(idx, sc, bits, 128)
        cos = torch.nn.functional.cosine_similarity(x.float().flatten(), deq.flatten(), dim=0).item()
        assert lo < cos <= hi
        idx2, sc2 = tq.block_quantize(deq, bits)
        same = (idx2 == idx).all(dim=1).float().mean().item()
        assert same > 0.99, same
        # checksum-of-rows equality against the oracle on a strided sample of the same tensor
        rows = torch.arange(0, n, 997, device="cuda")
        op, os_ = o.block_quantize(bits, 128, 0, -1, x[rows].float().cpu().numpy(), nthreads=8)
        assert np.array_equal(idx[rows].cpu().numpy(), op) and np.array_equal(u16(sc[rows]), os_)
