"""Parity of the CUDA SpMM path (through the C ABI) with the CPU oracle and the golden
vectors of the reference's own spmm_func."""
import numpy as np
import pytest
import torch

from conftest import assert_close_rel, golden_blocks
from oracle import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rt():
    from compressgnn_b200 import runtime
    return runtime


def cu(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def random_csr(rng, rows, src_rows, max_deg, long_rows=(), empty_frac=0.2):
    deg = rng.integers(0, max_deg + 1, rows)
    deg[rng.random(rows) < empty_frac] = 0
    for r, d in long_rows:
        if r < rows:
            deg[r] = d
    rowptr = np.zeros(rows + 1, np.int64)
    rowptr[1:] = np.cumsum(deg)
    col = rng.integers(0, src_rows, rowptr[-1]).astype(np.int64)
    return rowptr, col


def test_golden_spmm(rt, golden):
    g = golden
    args = [cu(g[k]) for k in ("spmm_rowptr", "spmm_col", "spmm_val", "spmm_mat")]
    out = rt.spmm_func(*args, "rowbalance_rowcache", None)
    assert_close_rel(out.cpu().numpy(), g["spmm_out"], what="golden spmm")
    base = cu(g["spmm_base"].copy())
    ret = rt.spmm_func(*args, "nnzbalance_rowcache", base)
    assert ret.data_ptr() == base.data_ptr()  # accumulated in place and returned
    assert_close_rel(base.cpu().numpy(), g["spmm_out_acc"], what="golden spmm accumulate")


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("width", [1, 3, 4, 16, 31, 33, 64, 128, 256, 602, 1100])
def test_spmm_widths(rt, dtype, width):
    rng = np.random.default_rng(width)
    rows, src_rows = 300, 211
    rowptr, col = random_csr(rng, rows, src_rows, 12, long_rows=[(7, 500), (123, 131), (299, 70)])
    val = rng.standard_normal(col.size).astype(dtype)
    mat = rng.standard_normal((src_rows, width)).astype(dtype)
    ref = oracle.spmm(rowptr, col, val, mat)
    out = rt.spmm_func(cu(rowptr), cu(col), cu(val), cu(mat), "rowbalance_rowcache", None)
    assert_close_rel(out.cpu().numpy(), ref, what=f"spmm width {width}")
    base = rng.standard_normal((rows, width)).astype(dtype)
    ref_acc = oracle.spmm(rowptr, col, val, mat, out=base.copy())
    got = rt.spmm_func(cu(rowptr), cu(col), cu(val), cu(mat), "nnzbalance_parreduce", cu(base))
    assert_close_rel(got.cpu().numpy(), ref_acc, what=f"spmm accumulate width {width}")


def test_accuracy_against_fp64(rt):
    """The fp32 CUDA result is as close to the exact (fp64) product as the reference's own
    fp32 loop is: error no larger than twice the CPU oracle's, row by row in max norm."""
    rng = np.random.default_rng(12)
    rowptr, col = random_csr(rng, 400, 300, 30, long_rows=[(0, 9000), (50, 700), (51, 129)])
    val = rng.standard_normal(col.size).astype(np.float32)
    mat = rng.standard_normal((300, 64)).astype(np.float32)
    exact = oracle.spmm(rowptr, col, val.astype(np.float64), mat.astype(np.float64))
    cpu = oracle.spmm(rowptr, col, val, mat).astype(np.float64)
    gpu = rt.spmm_func(cu(rowptr), cu(col), cu(val), cu(mat), "rowbalance_rowcache", None)
    gpu = gpu.cpu().numpy().astype(np.float64)
    err_cpu = np.abs(cpu - exact).max(axis=1)
    err_gpu = np.abs(gpu - exact).max(axis=1)
    scale = np.abs(exact).max(axis=1) + 1e-30
    assert np.all(err_gpu <= 2 * err_cpu + 2e-7 * scale), (err_gpu / scale).max()


def test_spmm_is_deterministic_and_reuses_its_plan(rt):
    rng = np.random.default_rng(5)
    rowptr, col = random_csr(rng, 2000, 1500, 40, long_rows=[(1, 5000), (77, 999)])
    val = rng.standard_normal(col.size).astype(np.float32)
    mat = rng.standard_normal((1500, 128)).astype(np.float32)
    d = [cu(rowptr), cu(col), cu(val), cu(mat)]
    first = rt.spmm_func(*d, "rowbalance_rowcache", None)
    plan = rt.csr_plan(d[0], d[1])
    assert plan.long_rows >= 2 and plan.chunks > plan.long_rows
    for _ in range(3):
        again = rt.spmm_func(*d, "rowbalance_rowcache", None)
        assert torch.equal(first, again)  # no float atomics: bit-identical every time
    assert rt.csr_plan(d[0], d[1]) is plan
    assert_close_rel(first.cpu().numpy(), oracle.spmm(rowptr, col, val, mat), what="long rows")


def test_spmm_sparse_rows_use_the_compact_row_list(rt):
    """Rule-level blocks are [R x R] with few non-empty rows (topo_partition keeps full-length
    row pointers); fresh output must still be zero on the untouched rows."""
    rng = np.random.default_rng(9)
    rows = 5000
    deg = np.zeros(rows, np.int64)
    hot = rng.choice(rows, 300, replace=False)
    deg[hot] = rng.integers(1, 6, 300)
    deg[hot[0]] = 300
    rowptr = np.zeros(rows + 1, np.int64)
    rowptr[1:] = np.cumsum(deg)
    col = rng.integers(0, rows, rowptr[-1]).astype(np.int64)
    val = rng.standard_normal(col.size).astype(np.float32)
    mat = rng.standard_normal((rows, 64)).astype(np.float32)
    d = [cu(rowptr), cu(col), cu(val), cu(mat)]
    out = rt.spmm_func(*d, "nnzbalance_rowcache", None)
    assert rt.csr_plan(d[0], d[1]).compact_rows == 1
    assert_close_rel(out.cpu().numpy(), oracle.spmm(rowptr, col, val, mat), what="compact rows")
    # in-place level update: out aliases the source, written rows are never read
    src = mat.copy()
    lvl_rows = hot[:150]
    deg2 = np.zeros(rows, np.int64)
    deg2[lvl_rows] = 3
    rp2 = np.zeros(rows + 1, np.int64)
    rp2[1:] = np.cumsum(deg2)
    others = np.setdiff1d(np.arange(rows), lvl_rows)
    col2 = rng.choice(others, rp2[-1]).astype(np.int64)
    val2 = np.ones(col2.size, np.float32)
    ref = oracle.spmm(rp2, col2, val2, src, out=src)
    buf = cu(mat)
    got = rt.spmm_func(cu(rp2), cu(col2), cu(val2), buf, "nnzbalance_rowcache", buf)
    assert got.data_ptr() == buf.data_ptr()
    assert_close_rel(buf.cpu().numpy(), ref, what="in-place level")


def test_spmm_empty_and_errors(rt):
    mat = torch.randn(5, 8, device="cuda")
    rowptr = torch.zeros(4, dtype=torch.int64, device="cuda")
    empty = torch.zeros(0, dtype=torch.int64, device="cuda")
    out = rt.spmm_func(rowptr, empty, torch.zeros(0, device="cuda"), mat, "rowbalance_rowcache", None)
    assert out.shape == (3, 8) and not out.any()
    with pytest.raises(RuntimeError, match="Invalid SpMM method"):
        rt.spmm_func(rowptr, empty, torch.zeros(0, device="cuda"), mat, "rowbalance", None)
    with pytest.raises(RuntimeError):
        rt.spmm_func(rowptr, empty, torch.zeros(0, device="cuda"), mat.t(), "rowbalance_rowcache", None)
    bad = torch.tensor([0, 2, 1, 3], dtype=torch.int64, device="cuda")
    with pytest.raises(RuntimeError, match="monotone"):
        rt.spmm_func(bad, torch.zeros(3, dtype=torch.int64, device="cuda"),
                     torch.ones(3, device="cuda"), mat, "rowbalance_rowcache", None)
    assert rt.device_status() == 0


def test_sources_and_outputs_are_checked_on_the_host(rt):
    """A matrix with fewer rows than the index array names, and an output that could not be
    accumulated in place, are refused before anything is launched."""
    rowptr = cu(np.array([0, 2, 3], np.int64))
    col = cu(np.array([0, 6, 2], np.int64))
    val = torch.ones(3, device="cuda")
    plan = rt.SegmentPlan.from_csr(rowptr, col)
    assert plan.source_rows == (7, 0)
    ok = rt.spmm_func(rowptr, col, val, torch.ones(7, 4, device="cuda"), "rowbalance_rowcache", None)
    assert ok.cpu().tolist() == [[2.0] * 4, [1.0] * 4]
    with pytest.raises(RuntimeError, match="refers to row 6"):
        rt.spmm_func(rowptr, col, val, torch.ones(6, 4, device="cuda"), "rowbalance_rowcache", None)
    pair = rt.SegmentPlan.from_csr(rowptr, col, cu(np.array([0, 1, 1], np.int64)), cu(np.array([9], np.int64)))
    assert pair.source_rows == (7, 10)
    with pytest.raises(RuntimeError, match="block 1 refers to row 9"):
        rt.spmm_pair_with_plan(pair, val, torch.ones(7, 4, device="cuda"), torch.ones(1, device="cuda"),
                               torch.ones(9, 4, device="cuda"))
    strided = torch.zeros(2, 8, device="cuda")[:, ::2]
    with pytest.raises(RuntimeError, match="contiguous"):
        rt.spmm_func(rowptr, col, val, torch.ones(7, 4, device="cuda"), "rowbalance_rowcache", strided)
    assert rt.device_status() == 0


def test_plan_records_the_row_length_histogram(rt):
    """The chunk length follows the row-length histogram: short rows with a thin tail get chunks of 64,
    rows that are long as a rule (or a heavy tail) chunks of 128."""
    rng = np.random.default_rng(5)
    rp, col = random_csr(rng, 4000, 900, 6, long_rows=[(10, 700)])
    thin = rt.SegmentPlan.from_csr(cu(rp), cu(col))
    lengths = np.diff(rp)
    assert thin.degree_max == 700 and thin.degree_p50 == int(np.sort(lengths)[len(lengths) // 2 - 1 + len(lengths) % 2])
    assert thin.degree_p99 < 64 and thin.split == 64 and thin.long_rows == 1
    rp, col = random_csr(rng, 300, 900, 200, empty_frac=0.0)
    long_rows = rt.SegmentPlan.from_csr(cu(rp), cu(col))
    assert long_rows.degree_p50 > 64 and long_rows.split == 128
    rp, col = random_csr(rng, 2000, 5000, 4, long_rows=[(i, 600 + i) for i in range(0, 2000, 40)])
    heavy_tail = rt.SegmentPlan.from_csr(cu(rp), cu(col))
    assert heavy_tail.degree_p99 > 512 and heavy_tail.split == 128


def test_fused_pair_matches_two_calls(rt):
    rng = np.random.default_rng(21)
    rows, n0, n1, width = 700, 400, 650, 96
    rp0, c0 = random_csr(rng, rows, n0, 6, long_rows=[(3, 400)])
    rp1, c1 = random_csr(rng, rows, n1, 9, long_rows=[(3, 90), (500, 300)])
    v0 = rng.standard_normal(c0.size).astype(np.float32)
    v1 = rng.standard_normal(c1.size).astype(np.float32)
    m0 = rng.standard_normal((n0, width)).astype(np.float32)
    m1 = rng.standard_normal((n1, width)).astype(np.float32)
    ref = oracle.spmm(rp1, c1, v1, m1, out=oracle.spmm(rp0, c0, v0, m0))
    plan = rt.SegmentPlan.from_csr(cu(rp0), cu(c0), cu(rp1), cu(c1))
    assert plan.terms == 2
    out = rt.spmm_pair_with_plan(plan, cu(v0), cu(m0), cu(v1), cu(m1))
    assert_close_rel(out.cpu().numpy(), ref, what="fused pair")
    again = rt.spmm_pair_with_plan(plan, cu(v0), cu(m0), cu(v1), cu(m1))
    assert torch.equal(out, again)


def test_golden_propagation_through_spmm_func(rt, golden):
    """The reference's forward/backward call sequence (layer/CompressgnnSPMM.py:54-60,80-85)
    replayed on spmm_func reproduces the reference's own outputs."""
    blocks = golden_blocks(golden)
    n, r = int(golden["dag_n"]), int(golden["dag_r"])
    dev = {k: tuple(cu(a) for a in v) for k, v in blocks.items() if k != "r2r"}
    levels = [tuple(cu(a) for a in lvl) for lvl in blocks["r2r"]]
    x = cu(golden["dag_x"])
    rule_out = rt.spmm_func(*dev["r2v"], x, "rowbalance_rowcache", None)
    for lvl in levels:
        rule_out = rt.spmm_func(*lvl, rule_out, "nnzbalance_rowcache", rule_out)
    out = rt.spmm_func(*dev["v2r"], rule_out, "nnzbalance_rowcache", None)
    out = rt.spmm_func(*dev["v2v"], x, "rowbalance_rowcache", out)
    assert_close_rel(out.cpu().numpy(), golden["dag_forward"], what="golden forward")
    g = cu(golden["dag_grad"])
    tr = lambda blk, ncols: tuple(cu(a) for a in oracle.transpose_csr(*blk, ncols))
    rule_g = rt.spmm_func(*tr(blocks["v2r"], r), g, "nnzbalance_rowcache", None)
    for lvl in reversed(blocks["r2r"]):
        rule_g = rt.spmm_func(*tr(lvl, r), rule_g, "nnzbalance_rowcache", rule_g)
    gx = rt.spmm_func(*tr(blocks["v2v"], n), g, "rowbalance_rowcache", None)
    gx = rt.spmm_func(*tr(blocks["r2v"], n), rule_g, "rowbalance_rowcache", gx)
    assert_close_rel(gx.cpu().numpy(), golden["dag_backward"], what="golden backward")


def test_offsets_beyond_32_bits(rt):
    """Source matrices with more than 2^31 elements (the 18.5 M-node x 128 configuration): row
    offsets are 64-bit in every kernel (the reference's rowcache kernel multiplies in int32)."""
    free, _total = torch.cuda.mem_get_info()
    src_rows, width = 17_500_000, 128  # 2.24e9 elements, 8.96 GB
    if free < 12 * 2**30:
        pytest.skip("needs 12 GB of free device memory")
    x = torch.zeros(src_rows, width, device="cuda")
    rng = np.random.default_rng(31)
    picks = np.unique(np.concatenate([rng.integers(16_900_000, src_rows, 200), [src_rows - 1, 16_777_216]]))
    x[torch.from_numpy(picks).cuda()] = torch.randn(picks.size, width, device="cuda")
    rows = 64
    deg = rng.integers(1, 9, rows)
    deg[5] = 150  # a chunked row as well
    rowptr = np.zeros(rows + 1, np.int64)
    rowptr[1:] = np.cumsum(deg)
    col = rng.choice(picks, rowptr[-1]).astype(np.int64)
    val = rng.standard_normal(col.size).astype(np.float32)
    out = rt.spmm_func(cu(rowptr), cu(col), cu(val), x, "rowbalance_rowcache", None)
    sub = x[torch.from_numpy(col).cuda()].cpu().numpy().astype(np.float64) * val[:, None]
    ref = np.add.reduceat(sub, rowptr[:-1], axis=0)
    assert_close_rel(out.cpu().numpy(), ref, what="rows beyond 2^31 elements")
    idx = torch.from_numpy(rng.choice(picks, 1000)).cuda()
    y = rt.cluster_reconstruct(x, idx, None, False)
    assert torch.equal(y, x.index_select(0, idx))
    del x
    torch.cuda.empty_cache()
