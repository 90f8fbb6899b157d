"""Parity of the CUDA cluster / reconstruct operators (through the C ABI) with the CPU
oracle, the golden vectors, and the closed-form expectations of the reference's
tests/test_transformation.py (same grids of widths, sizes and bit counts)."""
import numpy as np
import pytest
import torch

from conftest import assert_close_rel
from oracle import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rt():
    from compressgnn_b200 import runtime
    return runtime


def cu(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def assign(rt, x, w, bits):
    return rt.cluster_assign(x, w, bits, rt.cluster_workspace(x, bits))


@pytest.mark.parametrize("tag", ["a", "b", "c", "f"])
def test_golden_lsh_ids_are_bit_exact(rt, golden, tag):
    x, w = cu(golden[f"lsh_{tag}_x"]), cu(golden[f"lsh_{tag}_planes"])
    ids, counts, active = assign(rt, x, w, w.size(1))
    assert active == int(golden[f"lsh_{tag}_active"])
    assert ids.dtype == torch.int64 and counts.dtype == torch.int32
    np.testing.assert_array_equal(ids.cpu().numpy(), golden[f"lsh_{tag}_ids"].astype(np.int64))
    np.testing.assert_array_equal(counts.cpu().numpy(),
                                  np.bincount(golden[f"lsh_{tag}_ids"], minlength=active + 1))
    legacy_ids, legacy_active = rt.cluster_forward(x, w, w.size(1))
    assert legacy_ids.dtype == torch.int32 and legacy_active == active
    np.testing.assert_array_equal(legacy_ids.cpu().numpy(), golden[f"lsh_{tag}_ids"])


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("width", [0, 1, 31, 33, 128, 602])
@pytest.mark.parametrize("n,bits", [(0, 8), (1, 0), (67, 8), (257, 16), (1500, 24)])
def test_assign_mean_grid_is_bit_exact_against_the_oracle(rt, dtype, width, n, bits):
    """Grid of reference tests/test_transformation.py:21-29; N(0,1) inputs, so the ids depend
    on the documented fma order, which the oracle restates exactly."""
    rng = np.random.default_rng(1000 * width + n + bits)
    x = rng.standard_normal((n, width)).astype(dtype)
    w = rng.standard_normal((width, bits)).astype(dtype)
    ids, counts, active = assign(rt, cu(x), cu(w), bits)
    rids, rcounts, ractive = oracle.cluster_assign(x, w)
    assert active == ractive
    np.testing.assert_array_equal(ids.cpu().numpy(), rids)
    np.testing.assert_array_equal(counts.cpu().numpy(), rcounts)
    y = rt.cluster_mean(cu(x), ids, counts)
    assert y.shape == (active + 1, width)
    assert_close_rel(y.cpu().numpy(), oracle.cluster_mean(x, rids, rcounts), what="mean")
    grad = rng.standard_normal((active + 1, width)).astype(dtype)
    dx = rt.cluster_mean_backward(cu(grad), ids, counts)
    assert_close_rel(dx.cpu().numpy(), oracle.cluster_mean_backward(grad, rids, rcounts),
                     rel=1e-6, what="mean backward")


def test_projection_matches_the_oracle_bit_for_bit(rt):
    rng = np.random.default_rng(77)
    for n, width, bits in [(1000, 128, 16), (333, 130, 7), (129, 96, 30), (64, 5, 1)]:
        x = rng.standard_normal((n, width)).astype(np.float32)
        w = rng.standard_normal((width, bits)).astype(np.float32)
        got = rt.project(cu(x), cu(w)).cpu().numpy()
        np.testing.assert_array_equal(got, oracle.project(x, w))
        ids, counts, active = rt.cluster_assign_from_projection(cu(got), rt.cluster_workspace(cu(x), bits))
        rids, rcounts, ractive = oracle.cluster_assign(x, w)
        assert active == ractive
        np.testing.assert_array_equal(ids.cpu().numpy(), rids)


@pytest.mark.parametrize("bits", [4, 8, 12, 16, 20, 24, 28])
@pytest.mark.parametrize("width", [16, 48, 128, 256])
def test_tile_copy_projection_is_bit_exact(rt, bits, width):
    """fp32, a width that is a multiple of 16 and a multiple of four planes take the kernel whose row
    tiles arrive by TMA: every tile-boundary case against the oracle, and against the cp.async kernel
    (reached through a feature matrix that starts 4 bytes off a 16-byte boundary)."""
    rng = np.random.default_rng(31 * bits + width)
    w = rng.standard_normal((width, bits)).astype(np.float32)
    for n in (1, 255, 512, 513, 1024 + 77, 5000):
        x = rng.standard_normal((n, width)).astype(np.float32)
        want = oracle.project(x, w)
        got = rt.project(cu(x), cu(w))
        np.testing.assert_array_equal(got.cpu().numpy(), want)
        ids, counts, active = assign(rt, cu(x), cu(w), bits)
        rids, rcounts, ractive = oracle.cluster_assign(x, w)
        assert active == ractive
        np.testing.assert_array_equal(ids.cpu().numpy(), rids)
        np.testing.assert_array_equal(counts.cpu().numpy(), rcounts)
        shifted = torch.empty(n * width + 1, dtype=torch.float32, device="cuda")[1:].view(n, width)
        shifted.copy_(cu(x))
        assert shifted.data_ptr() % 16 == 4
        assert torch.equal(rt.project(shifted, cu(w)), got)
    rt.raise_on_device_status()


def test_non_default_stream(rt):
    x = torch.randn(67, 33, device="cuda")
    w = torch.randn(33, 8, device="cuda")
    ids, counts, active = assign(rt, x, w, 8)
    ref = rt.cluster_mean(x, ids, counts)
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        ii, cc, aa = assign(rt, x, w, 8)
        yy = rt.cluster_mean(x, ii, cc)
    stream.synchronize()
    assert aa == active and torch.equal(ii, ids) and torch.equal(yy, ref)


@pytest.mark.parametrize("bits", [0, 8, 24])
def test_all_rows_collide(rt, bits):
    x = torch.ones(513, 33, device="cuda")
    w = torch.ones(33, bits, device="cuda")
    ids, counts, active = assign(rt, x, w, bits)
    assert active == 1 and counts.tolist() == [0, 513] and bool((ids == 1).all())


def test_large_mean_is_deterministic_with_long_segments(rt):
    """Config-3 shape in small: Gaussian mixture, buckets collapse, segments far longer than
    the plan's split."""
    rng = np.random.default_rng(4)
    n, width, bits = 60000, 128, 16
    cent = rng.standard_normal((64, width)).astype(np.float32)
    x = (cent[rng.integers(0, 64, n)] + 0.1 * rng.standard_normal((n, width))).astype(np.float32)
    w = rng.standard_normal((width, bits)).astype(np.float32)
    dx = cu(x)
    ids, counts, active = assign(rt, dx, cu(w), bits)
    rids, rcounts, ractive = oracle.cluster_assign(x, w)
    assert active == ractive
    np.testing.assert_array_equal(ids.cpu().numpy(), rids)
    plan = rt.index_plan(ids, active + 1)
    assert plan.long_rows > 0
    reps = rng.standard_normal((active + 1, 64)).astype(np.float32)
    bias = rng.standard_normal(64).astype(np.float32)
    fwd = rt.cluster_reconstruct(cu(reps), ids, cu(bias), True)
    go = cu(rng.standard_normal((n, 64)).astype(np.float32))
    exact = rt.cluster_reconstruct_backward(go, ids, fwd, active + 1, True)
    fast = rt.cluster_reconstruct_backward(go, ids, fwd, active + 1, True, output_is_forward_result=True)
    assert torch.equal(exact, fast)
    assert_close_rel(exact.cpu().numpy(),
                     oracle.reconstruct_backward(go.cpu().numpy(), rids, fwd.cpu().numpy(), active + 1, True)[0],
                     what="long reconstruct backward")
    y1 = rt.cluster_mean(dx, ids, counts)
    y2 = rt.cluster_mean(dx, ids, counts)
    assert torch.equal(y1, y2)
    assert_close_rel(y1.cpu().numpy(), oracle.cluster_mean(x, rids, rcounts), what="long mean")
    # an index tensor the library has never seen: the plan is rebuilt from the index alone
    fresh = ids.clone()
    y3 = rt.cluster_mean(dx, fresh, counts)
    assert torch.equal(y1, y3)


def test_golden_mean_and_reconstruct(rt, golden):
    g = golden
    idx, cnt = cu(g["mean_index"]), cu(g["mean_counts"])
    assert_close_rel(rt.cluster_mean(cu(g["mean_x"]), idx, cnt).cpu().numpy(), g["mean_out"],
                     what="golden mean")
    assert_close_rel(rt.cluster_mean_backward(cu(g["mean_grad_out"]), idx, cnt).cpu().numpy(),
                     g["mean_grad_in"], rel=1e-6, what="golden mean backward")
    for tag, relu in (("lin", False), ("relu", True)):
        y = rt.cluster_reconstruct(cu(g["rec_reps"]), idx, cu(g["rec_bias"]), relu)
        np.testing.assert_array_equal(y.cpu().numpy(), g[f"rec_{tag}_out"])
        dr, db = rt.cluster_reconstruct_backward(cu(g["rec_grad_out"]), idx, y, cnt.numel(), relu,
                                                 return_bias_grad=True)
        assert_close_rel(dr.cpu().numpy(), g[f"rec_{tag}_dreps"], what="golden d_reps")
        assert_close_rel(db.cpu().numpy(), g[f"rec_{tag}_dbias"], what="golden d_bias")


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("width", [1, 31, 33, 128, 256, 520, 602])
@pytest.mark.parametrize("relu", [False, True])
def test_reconstruct_grid(rt, dtype, width, relu):
    """Grid of reference tests/test_transformation.py:44-54, including unused groups."""
    rng = np.random.default_rng(width)
    idx = np.array([1, 1, 3, 1, 3, 3] * 50, np.int64)
    reps = rng.standard_normal((5, width)).astype(dtype)
    bias = rng.standard_normal(width).astype(dtype)
    go = rng.standard_normal((idx.size, width)).astype(dtype)
    y = rt.cluster_reconstruct(cu(reps), cu(idx), cu(bias), relu)
    ref = oracle.reconstruct(reps, idx, bias, relu)
    np.testing.assert_array_equal(y.cpu().numpy(), ref)
    y_nobias = rt.cluster_reconstruct(cu(reps), cu(idx), None, relu)
    np.testing.assert_array_equal(y_nobias.cpu().numpy(), oracle.reconstruct(reps, idx, None, relu))
    dr, db = rt.cluster_reconstruct_backward(cu(go), cu(idx), y, 5, relu, return_bias_grad=True)
    rdr, rdb = oracle.reconstruct_backward(go, idx, ref, 5, relu)
    assert_close_rel(dr.cpu().numpy(), rdr, what="d_reps")
    assert_close_rel(db.cpu().numpy(), rdb, what="d_bias")
    assert not dr[0].any() and not dr[2].any() and not dr[4].any()
    # one mask row per group instead of the whole forward output: same bits
    dr2 = rt.cluster_reconstruct_backward(cu(go), cu(idx), y, 5, relu, output_is_forward_result=True)
    assert torch.equal(dr, dr2)


def test_argument_errors_raise_runtime_error(rt):
    x = torch.randn(10, 7, device="cuda")
    with pytest.raises(RuntimeError):  # bad plane shape (reference test :105-107)
        rt.cluster_assign(x, torch.randn(7, 3, device="cuda"), 4, rt.cluster_workspace(x, 4))
    with pytest.raises(RuntimeError):
        rt.cluster_workspace(x, 31)
    with pytest.raises(RuntimeError):  # workspace made for fewer rows
        small = rt.cluster_workspace(x[:2].contiguous(), 4)
        rt.cluster_assign(torch.randn(5000, 7, device="cuda"), torch.randn(7, 4, device="cuda"), 4, small)
    idx = torch.tensor([0, 1, 7], device="cuda")
    cnt = torch.tensor([1, 1], dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError, match="outside"):  # index beyond the groups: reported, not trapped
        rt.cluster_mean(torch.randn(3, 4, device="cuda"), idx, cnt)
    out = rt.cluster_reconstruct(torch.randn(2, 4, device="cuda"), idx, None, False)
    assert rt.device_status() & 1 and not out[2].any()
    assert rt.device_status() == 0
