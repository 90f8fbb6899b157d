"""Pin the CPU oracle (oracle/cgnn_oracle.c) to the reference: against the committed golden
vectors (outputs of the reference's own CPU operators) and, where the compiled reference is
present (oracle/_ref), against fresh calls of it."""
import numpy as np
import pytest

from conftest import assert_close_rel, golden_blocks
from oracle import oracle


def test_spmm_matches_reference_vectors(golden):
    g = golden
    out = oracle.spmm(g["spmm_rowptr"], g["spmm_col"], g["spmm_val"], g["spmm_mat"])
    np.testing.assert_array_equal(out, g["spmm_out"])  # same loop order -> same bits
    acc = oracle.spmm(g["spmm_rowptr"], g["spmm_col"], g["spmm_val"], g["spmm_mat"],
                      out=g["spmm_base"].copy())
    np.testing.assert_array_equal(acc, g["spmm_out_acc"])
    assert_close_rel(out, g["spmm_out_nnzbalance"], what="rowbalance vs nnzbalance")


def test_propagation_matches_reference_vectors(golden):
    blocks = golden_blocks(golden)
    n, r = int(golden["dag_n"]), int(golden["dag_r"])
    np.testing.assert_array_equal(oracle.propagate_forward(blocks, golden["dag_x"]),
                                  golden["dag_forward"])
    np.testing.assert_array_equal(oracle.propagate_backward(blocks, golden["dag_grad"], n, r),
                                  golden["dag_backward"])


@pytest.mark.parametrize("tag", ["a", "b", "c", "f"])
def test_lsh_ids_match_reference_vectors(golden, tag):
    x, planes = golden[f"lsh_{tag}_x"], golden[f"lsh_{tag}_planes"]
    ids, counts, active = oracle.cluster_assign(x, planes)
    assert active == int(golden[f"lsh_{tag}_active"])
    np.testing.assert_array_equal(ids, golden[f"lsh_{tag}_ids"].astype(np.int64))
    assert counts[0] == 0 and counts.sum() == x.shape[0]
    np.testing.assert_array_equal(counts, np.bincount(ids, minlength=active + 1))


def test_mean_and_reconstruct_match_reference_vectors(golden):
    g = golden
    idx, cnt = g["mean_index"], g["mean_counts"]
    assert_close_rel(oracle.cluster_mean(g["mean_x"], idx, cnt), g["mean_out"], what="mean")
    assert_close_rel(oracle.cluster_mean_backward(g["mean_grad_out"], idx, cnt),
                     g["mean_grad_in"], what="mean backward")
    for tag, relu in (("lin", False), ("relu", True)):
        y = oracle.reconstruct(g["rec_reps"], idx, g["rec_bias"], relu)
        np.testing.assert_array_equal(y, g[f"rec_{tag}_out"])
        dr, db = oracle.reconstruct_backward(g["rec_grad_out"], idx, y, cnt.size, relu)
        assert_close_rel(dr, g[f"rec_{tag}_dreps"], what="reconstruct d_reps")
        assert_close_rel(db, g[f"rec_{tag}_dbias"], rel=1e-5, what="reconstruct d_bias")


def test_sharded_projection_is_consistent():
    rng = np.random.default_rng(3)
    x = rng.integers(-3, 4, (50, 40)).astype(np.float32)
    w = rng.integers(-2, 3, (40, 9)).astype(np.float32)
    base = oracle.project(x, w)
    for shards in (2, 4, 8):
        np.testing.assert_array_equal(oracle.project(x, w, shards), base)  # exact in integers


def test_edge_cases():
    empty = np.zeros((0, 5), np.float32)
    ids, counts, active = oracle.cluster_assign(empty, np.zeros((5, 4), np.float32))
    assert ids.size == 0 and active == 0 and counts.tolist() == [0]
    ones = np.ones((513, 33), np.float32)
    for bits in (0, 8, 20):
        ids, counts, active = oracle.cluster_assign(ones, np.ones((33, bits), np.float32))
        assert active == 1 and counts.tolist() == [0, 513]
    rowptr = np.zeros(4, np.int64)
    out = oracle.spmm(rowptr, np.zeros(0, np.int64), np.zeros(0, np.float32),
                      np.ones((2, 3), np.float32))
    assert out.shape == (3, 3) and not out.any()


def test_against_compiled_reference_when_present():
    rt, _off = oracle.reference_modules()
    if rt is None:
        pytest.skip("oracle/_ref not built in this checkout")
    import torch
    rng = np.random.default_rng(11)
    for dtype in (np.float32, np.float64):
        x = rng.integers(-5, 6, (123, 17)).astype(dtype)
        w = rng.integers(-5, 6, (17, 10)).astype(dtype)
        ids, _counts, active = oracle.cluster_assign(x, w)
        rids, ractive = rt.cluster_forward(torch.from_numpy(x), torch.from_numpy(w), 10)
        assert active == ractive
        np.testing.assert_array_equal(ids, rids.numpy().astype(np.int64))
        deg = rng.integers(0, 7, 60)
        rowptr = np.zeros(61, np.int64)
        rowptr[1:] = np.cumsum(deg)
        col = rng.integers(0, 123, rowptr[-1])
        val = rng.standard_normal(rowptr[-1]).astype(dtype)
        mat = rng.standard_normal((123, 17)).astype(dtype)
        ref = rt.spmm_func(torch.from_numpy(rowptr), torch.from_numpy(col), torch.from_numpy(val),
                           torch.from_numpy(mat), "rowbalance", None).numpy()
        np.testing.assert_array_equal(oracle.spmm(rowptr, col, val, mat), ref)
