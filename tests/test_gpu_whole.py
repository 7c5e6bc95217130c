"""GPU parity of the whole-vector (core crate) path against the CPU oracle, through the C ABI."""
import os

import numpy as np
import pytest
import torch

import oracle_lib as o
import turboquant_b200 as tq

pytestmark = pytest.mark.gpu
CASES = np.load(os.path.join(os.path.dirname(__file__), "golden", "oracle_cases.npz"))


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def u16(t):
    return t.cpu().numpy().view(np.uint16)


def boundary_margin(bits, dim, seed, x):
    """Smallest relative distance of any rotated coordinate to a decision boundary."""
    _, b = o.codebook(bits, dim)
    n = np.sqrt((x.astype(np.float32) ** 2).sum(1, keepdims=True))
    rot = np.stack([o.wht((xi / ni) * o.sign_pattern(dim, seed)) if ni > 1e-10 else np.zeros(dim, np.float32)
                    for xi, ni in zip(x, n[:, 0])])
    return np.abs(rot[:, :, None].astype(np.float64) - b[None, None, :]).min(-1)


@pytest.mark.parametrize("bits", [2, 3, 4])
def test_config1_codes_bit_exact(bits):
    # 10,000 x 128 N(0,1), seed 42: packed codes and f16 scales identical to the oracle
    x = np.random.default_rng(42).standard_normal((10000, 128)).astype(np.float32)
    cfg = tq.TurboQuantConfig(bits, 128).with_seed(42)
    packed, scales = tq.quantize_batch(cfg, dev(x))
    op, os_ = o.quantize_batch(bits, 128, 42, x, nthreads=8)
    assert np.array_equal(u16(scales), os_)
    diff_rows = np.nonzero((packed.cpu().numpy() != op).any(1))[0]
    # the parity bar allows code differences only within 1e-6 of a boundary; none are expected
    assert len(diff_rows) == 0, f"{len(diff_rows)} vectors differ"
    deq = tq.dequantize_batch(cfg, packed, scales).cpu().numpy()
    od = o.dequantize_batch(bits, 128, 42, op, os_, nthreads=8)
    assert np.array_equal(deq, od)          # no reduction on this path: bit-identical, well inside 1e-5 relative
    nmse = (((x - deq) ** 2).sum(1) / (x ** 2).sum(1)).mean()
    assert abs(nmse - {2: 0.1161, 3: 0.0340, 4: 0.00935}[bits]) < 0.0005


@pytest.mark.parametrize("bits", [2, 3, 4])
def test_golden_fixture_edge_vectors(bits):
    # includes an all-zero vector, one below MIN_NORM and one with a large norm
    x = CASES["whole_x"]
    cfg = tq.TurboQuantConfig(bits, 128).with_seed(42)
    packed, scales = tq.quantize_batch(cfg, dev(x))
    assert np.array_equal(packed.cpu().numpy(), CASES[f"whole_packed_{bits}"])
    assert np.array_equal(u16(scales), CASES[f"whole_scales_{bits}"])
    assert np.array_equal(tq.dequantize_batch(cfg, packed, scales).cpu().numpy(), CASES[f"whole_deq_{bits}"])


@pytest.mark.parametrize("dim", [32, 64, 256])
@pytest.mark.parametrize("n", [1, 33, 70])
def test_other_dims_and_ragged_batches(dim, n):
    x = np.random.default_rng(dim + n).standard_normal((n, dim)).astype(np.float32)
    for bits in (2, 3, 4):
        cfg = tq.TurboQuantConfig(bits, dim).with_seed(7)
        packed, scales = tq.quantize_batch(cfg, dev(x))
        op, os_ = o.quantize_batch(bits, dim, 7, x)
        assert np.array_equal(packed.cpu().numpy(), op) and np.array_equal(u16(scales), os_)
        assert np.array_equal(tq.dequantize_batch(cfg, packed, scales).cpu().numpy(), o.dequantize_batch(bits, dim, 7, op, os_))
        rot = tq.dequantize_batch(cfg, packed, scales, rotated=True).cpu().numpy()
        assert np.array_equal(rot, o.dequantize_rotated_batch(bits, dim, op, os_))


def test_empty_batch_and_errors():
    cfg = tq.TurboQuantConfig(3, 128).with_seed(42)
    p, s = tq.quantize_batch(cfg, torch.empty((0, 128), device="cuda"))
    assert p.shape == (0, 48) and s.shape == (0,)
    with pytest.raises(tq.DimensionMismatch):
        tq.quantize_batch(cfg, torch.zeros((2, 64), device="cuda"))
    with pytest.raises(tq.DimensionMismatch):
        tq.quantize_vec(cfg, np.zeros(100, np.float32))
    with pytest.raises(tq.UnsupportedBits):
        tq.quantize_with_qjl(tq.TurboQuantConfig(2, 128), np.zeros(128, np.float32), 1)


def test_single_vector_api_round_trip():
    x = o.pseudo_random_vec(128, 99)     # src/test_utils.rs:4-22
    cfg = tq.TurboQuantConfig(3, 128).with_seed(42)
    blk = tq.quantize_vec(cfg, x)
    assert blk.bits == 3 and blk.size_bytes() == 50
    op, os_ = o.quantize_batch(3, 128, 42, x[None])
    assert blk.packed_indices == op[0].tobytes() and blk.scale == os_[0]
    assert np.array_equal(tq.dequantize_vec(cfg, blk), o.dequantize_batch(3, 128, 42, op, os_)[0])
    assert np.array_equal(tq.dequantize_rotated(cfg, blk), o.dequantize_rotated_batch(3, 128, op, os_)[0])


@pytest.mark.parametrize("bits", [3, 4])
@pytest.mark.parametrize("dim", [64, 128, 256])
def test_qjl_blocks_bit_exact(bits, dim):
    x = np.random.default_rng(bits * dim).standard_normal((67, dim)).astype(np.float32)
    cfg = tq.TurboQuantConfig(bits, dim).with_seed(42)
    p, s, sg, rn = tq.qjl_quantize_batch(cfg, dev(x), 12345)
    op, os_, osg, orn = o.qjl_quantize_batch(bits, dim, 42, 12345, x, nthreads=8)
    assert np.array_equal(p.cpu().numpy(), op) and np.array_equal(u16(s), os_)
    assert np.array_equal(u16(rn), orn)
    assert np.array_equal(sg.cpu().numpy(), osg)     # sequential row sums => identical sign bits


def test_qjl_golden_fixture():
    x = CASES["whole_x"][:16]
    for bits in (3, 4):
        cfg = tq.TurboQuantConfig(bits, 128).with_seed(42)
        p, s, sg, rn = tq.qjl_quantize_batch(cfg, dev(x), 42)
        assert np.array_equal(p.cpu().numpy(), CASES[f"qjl_packed_{bits}"])
        assert np.array_equal(sg.cpu().numpy(), CASES[f"qjl_signs_{bits}"])
        assert np.array_equal(u16(rn), CASES[f"qjl_rnorms_{bits}"])
    rq = tq.query_projections(dev(CASES["q"]), 128, 42).cpu().numpy()[0]
    assert np.array_equal(rq, CASES["rq_42"])


def test_config2_scores_and_weighted_output():
    # single head, d = 128, 1,024 keys and values N(0,1), one query N(0,1)/sqrt(128), bits = 3
    # (2-bit polar + 1-bit QJL), rotation seed 42, QJL seed 42
    rng = np.random.default_rng(42)
    keys = rng.standard_normal((1024, 128)).astype(np.float32)
    values = rng.standard_normal((1024, 128)).astype(np.float32)
    q = (rng.standard_normal(128) / np.sqrt(128)).astype(np.float32)
    cfg = tq.TurboQuantConfig(3, 128).with_seed(42)
    cache = tq.QuantizedKVCache(cfg, 1, 42)
    cache.push_batch(0, keys, values)
    assert cache.entry_count(0) == 1024
    assert cache.memory_usage() == 2 * 1024 * 52        # src/qjl.rs:1174-1180
    assert cache.fp16_equivalent_memory() == 1024 * 128 * 2 * 2
    scores = cache.attention_scores(0, q)
    kp, ks, ksg, krn = o.qjl_quantize_batch(3, 128, 42, 42, keys, nthreads=8)
    vp, vs, _, _ = o.qjl_quantize_batch(3, 128, 42, 42, values, nthreads=8)
    want = o.attention_scores(3, 128, 42, 42, q, kp, ks, ksg, krn, nthreads=8)
    assert np.abs(scores - want).max() < 1e-5
    w = np.exp(want - want.max())
    w = (w / w.sum()).astype(np.float32)
    out = cache.weighted_values(0, w)
    assert np.abs(out - o.weighted_values(3, 128, 42, w, vp, vs)).max() < 1e-5   # far inside 2e-3


@pytest.mark.parametrize("bits,dim,n", [(3, 128, 9001), (4, 128, 8195), (3, 64, 4100), (4, 256, 4097), (4, 64, 5003), (3, 256, 4096)])
def test_long_lists_scores_and_weighted_values(bits, dim, n):
    # lists of 4,096 entries and more run on the tabulated-query / lane-per-32-elements kernels
    rng = np.random.default_rng(bits * 1000 + dim + n)
    keys = rng.standard_normal((n, dim)).astype(np.float32)
    keys[:: 97] *= 30.0
    keys[5] = 0.0
    q = (rng.standard_normal(dim) / np.sqrt(dim)).astype(np.float32)
    cfg = tq.TurboQuantConfig(bits, dim).with_seed(11)
    p, s, sg, rn = tq.qjl_quantize_batch(cfg, dev(keys), 77)
    rq = tq.query_projections(dev(q), dim, 77)
    got = tq.qjl_attention_scores(cfg, dev(q), rq.reshape(-1), p, s, sg, rn).cpu().numpy()
    want = o.attention_scores(bits, dim, 11, 77, q, p.cpu().numpy(), u16(s), sg.cpu().numpy(), u16(rn), nthreads=8)
    scale = np.abs(want).max()
    assert np.abs(got - want).max() < 2e-6 * max(scale, 1.0) + 1e-5
    # the short-list kernel on a prefix agrees too
    short = tq.qjl_attention_scores(cfg, dev(q), rq.reshape(-1), p[:1000], s[:1000], sg[:1000], rn[:1000]).cpu().numpy()
    assert np.abs(short - want[:1000]).max() < 2e-6 * max(scale, 1.0) + 1e-5
    w = rng.random(n).astype(np.float32)
    w /= w.sum()
    out = tq.weighted_values(cfg, dev(w), p, s).cpu().numpy()
    ref = o.weighted_values(bits, dim, 11, w, p.cpu().numpy(), u16(s))
    assert np.abs(out - ref).max() < 1e-5 * max(np.abs(ref).max(), 1.0)


def test_kv_cache_push_batch_equals_push_and_ranges():
    # src/attention.rs:1375-1430 (push_batch == repeated push, bit for bit), :1221-1296 (ranges)
    rng = np.random.default_rng(1)
    keys = rng.standard_normal((9, 128)).astype(np.float32)
    values = rng.standard_normal((9, 128)).astype(np.float32)
    cfg = tq.TurboQuantConfig(4, 128).with_seed(42)
    a, b = tq.QuantizedKVCache(cfg, 2, 12345), tq.QuantizedKVCache(cfg, 2, 12345)
    a.push_batch(1, keys, values)
    for k, v in zip(keys, values):
        b.push(1, k, v)
    for is_keys in (True, False):
        ea, eb = a.export_packed_range(1, 0, 9, is_keys, with_qjl=True), b.export_packed_range(1, 0, 9, is_keys, with_qjl=True)
        assert all(np.array_equal(x, y) for x, y in zip(ea, eb))
    full = a.dequantize_all_keys(1)
    assert np.array_equal(a.dequantize_keys_range(1, 2, 7), full[2:7])
    assert a.dequantize_keys_range(1, 4, 4).shape == (0, 128)
    assert a.entry_count(0) == 0 and a.attention_scores(0, keys[0]).shape == (0,)
    assert np.all(a.weighted_values(0, np.zeros(0, np.float32)) == 0)
    with pytest.raises(tq.RangeOutOfBounds):
        a.dequantize_keys_range(1, 5, 10)
    with pytest.raises(tq.RangeOutOfBounds):
        a.dequantize_values_range(1, 6, 5)
    with pytest.raises(tq.LayerOutOfRange):
        a.push(2, keys[0], values[0])
    with pytest.raises(tq.DimensionMismatch):
        a.push(0, keys[0][:64], values[0][:64])
    with pytest.raises(tq.DimensionMismatch):
        a.weighted_values(1, np.ones(3, np.float32))
    with pytest.raises(tq.DimensionMismatch):
        a.attention_scores(1, np.ones(64, np.float32))
    # export -> import round trip (src/attention.rs:663-693)
    c = tq.QuantizedKVCache(cfg, 2, 12345)
    for is_keys in (True, False):
        p, s, sg, rn = a.export_packed_range(1, 0, 9, is_keys, with_qjl=True)
        c.import_packed_range(1, 3, p, s, sg, rn, 48, 16, is_keys)
    q = rng.standard_normal(128).astype(np.float32)
    assert np.array_equal(c.attention_scores(1, q), a.attention_scores(1, q))


def test_estimate_inner_product_single_block():
    rng = np.random.default_rng(8)
    x, q = rng.standard_normal(128).astype(np.float32), rng.standard_normal(128).astype(np.float32)
    cfg = tq.TurboQuantConfig(3, 128).with_seed(42)
    blk = tq.quantize_with_qjl(cfg, x, 777)
    assert blk.size_bytes() == 52 and blk.polar_block.bits == 2
    rq = tq.precompute_query_projections(q, 128, 777)
    assert np.array_equal(rq, o.query_projections(q, 128, 777))
    p, s, sg, rn = o.qjl_quantize_batch(3, 128, 42, 777, x[None])
    want = o.attention_scores(3, 128, 42, 777, q, p, s, sg, rn)[0]
    assert abs(tq.estimate_inner_product(q, rq, blk, cfg) - want) < 1e-4


def test_unaligned_input_takes_the_warp_tile_kernel_with_the_same_bits():
    # the lane-layout batch kernel wants 16-byte aligned rows; a 4-byte aligned view falls back to the
    # warp-per-tile kernel, and both must agree with the oracle
    n = 300
    x = np.random.default_rng(5).standard_normal((n, 128)).astype(np.float32)
    buf = torch.zeros(n * 128 + 1, device="cuda")
    buf[1:] = torch.from_numpy(x).reshape(-1).cuda()
    view = buf[1:].view(n, 128)
    assert view.data_ptr() % 16 == 4
    for bits in (2, 3, 4):
        cfg = tq.TurboQuantConfig(bits, 128).with_seed(42)
        op, os_ = o.quantize_batch(bits, 128, 42, x, nthreads=4)
        for inp in (view, dev(x)):
            p, s = tq.quantize_batch(cfg, inp)
            assert np.array_equal(p.cpu().numpy(), op) and np.array_equal(u16(s), os_)
