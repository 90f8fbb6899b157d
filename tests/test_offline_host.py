"""Host-side graph preparation (libcgnn_host.so): the compressor meets the contract the
reference's tests pin (tests/test_offline_compression.py:7-55, tests/test_batch_compression.py
:15-65), and filters / partitions / norms reproduce the reference's helpers bit for bit --
against the golden vectors always, against the compiled reference (oracle/_ref) when present."""
from collections import Counter

import numpy as np
import pytest

from compressgnn_b200 import offline as off
from compressgnn_b200.loader import CompressgnnData, compress_graph_csr, resolve_backend
from oracle import oracle


def expand(v, e, node, n):
    stack = list(reversed(e[v[node]:v[node + 1]].tolist()))
    out = []
    while stack:
        child = stack.pop()
        if child < n:
            out.append(child)
        else:
            children = e[v[child]:v[child + 1]]
            assert np.all(children < child), "rule graph must be acyclic with children < rule"
            stack.extend(reversed(children.tolist()))
    return out


def check(rows, packed, ordered=True):
    v, e, n, nr = packed
    assert n == len(rows) and len(v) == n + nr + 1
    assert v[0] == 0 and v[-1] == len(e) and np.all(np.diff(v) >= 0)
    for node, row in enumerate(rows):
        actual = expand(v, e, node, n)
        assert actual == row if ordered else Counter(actual) == Counter(row)


def csr_of(rows, dtype=np.int32):
    v = np.array([0] + list(np.cumsum([len(x) for x in rows])), dtype=dtype)
    e = np.array([j for row in rows for j in row], dtype=dtype)
    return v, e


@pytest.mark.parametrize("n", [1, 2, 17, 128, 512])
def test_compressor_and_filters_preserve_every_row(n):
    rng = np.random.default_rng(73 + n)
    fixtures = [
        [[] for _ in range(n)],
        [[i] for i in range(n)],
        [list(range(min(n, 16))) for _ in range(n)],
        [sorted(rng.choice(n, size=min(n, 20), replace=False).tolist()) for _ in range(n)],
        [sorted(rng.integers(n, size=8).tolist()) for _ in range(n)],
    ]
    for rows in fixtures:
        v, e = csr_of(rows)
        for freq in [3, 4, 8, 16, 32]:
            packed = off.compress_csr_batch(v, e, min_pair_frequency=freq)
            assert packed[0].dtype == np.int32 and packed[1].dtype == np.int32
            check(rows, packed, ordered=True)
            filtered = off.filter_csr(*packed, 16)
            check(rows, filtered, ordered=False)
            check(rows, off.depth_filter_csr(*filtered, 3, 100000), ordered=False)


def test_compressor_finds_shared_runs_and_is_deterministic():
    rows = [list(range(32)) for _ in range(64)]
    v, e = csr_of(rows, np.int64)
    a = off.compress_csr_batch(v, e, min_pair_frequency=3)
    b = compress_graph_csr(v, e, 3, backend='cpu')
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1]) and a[3] == b[3] > 0
    assert a[1].size < e.size / 8  # 64 identical rows collapse onto a few rules
    check(rows, a)


def test_argument_errors():
    for freq in [-1, 0, 1, 2]:
        with pytest.raises(ValueError):
            off.compress_csr_batch(np.array([0, 0], np.int32), np.array([], np.int32), min_pair_frequency=freq)
    with pytest.raises(ValueError):
        compress_graph_csr(np.array([0, 1], np.int64), np.array([2**32], np.uint64))
    with pytest.raises(ValueError):
        compress_graph_csr(np.array([0, 1]), np.array([0.5]))
    for bad in ['wrong', 'legacy', None]:
        with pytest.raises(ValueError):
            resolve_backend(bad)
    assert resolve_backend('cpu') == 'cpu'
    import torch
    if torch.cuda.is_available():  # the device compressor is taken whenever a GPU is usable
        assert resolve_backend('auto') == 'cuda' and resolve_backend('cuda') == 'cuda'
    else:
        assert resolve_backend('auto') == 'cpu'
        with pytest.raises(RuntimeError):
            resolve_backend('cuda')


def test_partition_matches_the_reference_vectors(golden):
    g = golden
    n, r = int(g["dag_n"]), int(g["dag_r"])
    nd = off.get_norm_degree(np.concatenate([np.sort(np.array(expand(g["dag_vlist"], g["dag_elist"], v, n)))
                                             for v in range(n)]), n)
    np.testing.assert_array_equal(nd, g["dag_norm_degree"])
    w = off.gcn_norm_csr_compress(g["dag_vlist"], g["dag_elist"], nd, n, r)
    np.testing.assert_array_equal(w, g["dag_weight"])
    t = off.transpose_csr(g["dag_vlist"], g["dag_elist"], w, n + r)
    for mine, ref in zip(t, oracle.transpose_csr(g["dag_vlist"], g["dag_elist"], w, n + r)):
        np.testing.assert_array_equal(mine, ref)
    blocks = off.hybird_partition(*t, n)
    for name, blk in zip(("v2v", "v2r", "r2v", "r2r"), blocks):
        for part, arr in zip(("rowptr", "col", "val"), blk):
            np.testing.assert_array_equal(arr, g[f"dag_{name}_{part}"])
    levels = off.topo_partition(*blocks[3])
    assert len(levels) == int(g["dag_step"])
    for i, blk in enumerate(levels):
        for part, arr in zip(("rowptr", "col", "val"), blk):
            np.testing.assert_array_equal(arr, g[f"dag_level{i}_{part}"])


def test_loader_builds_an_equivalent_graph():
    """CompressgnnData end to end: the oracle's propagation over the loader's blocks equals the
    dense normalised adjacency (A_hat^T x forward, A_hat g backward)."""
    n = 300
    v, e = off.generate_copy_graph(n, 2.1, 4.0, 100, 0.7, 32, 8, seed=5)
    rng = np.random.default_rng(0)
    x = rng.standard_normal((n, 6)).astype(np.float32)
    mask = np.ones(n, bool)
    data = CompressgnnData(x, (v, e), np.zeros(n, np.int64), mask, mask, mask, min_pair_frequency=3,
                           threshold=1, min_edge=10)
    graph = data.edge_index
    assert data.rule_cnt > 0 and graph.step >= 1 and data.edge_cnt < data.input_edge_cnt
    assert graph.v2v_graph.sparse_sizes() == (n, n) and graph.r2v_graph.sparse_sizes() == (data.rule_cnt, n)
    blocks = {k: tuple(t.numpy() for t in getattr(graph, f"{k}_graph").csr()) for k in ("v2v", "v2r", "r2v")}
    blocks["r2r"] = [tuple(t.numpy() for t in lvl.csr()) for lvl in graph.r2r_graph]
    sv, se = off.add_self_loop_csr(v, e)
    nd = off.get_norm_degree(se, n).astype(np.float64)
    dense = np.zeros((n, n))
    for a in range(n):
        for b in se[sv[a]:sv[a + 1]]:
            dense[a, b] += nd[a] * nd[b]
    fwd = oracle.propagate_forward(blocks, x)
    np.testing.assert_allclose(fwd, dense.T @ x, rtol=1e-4, atol=1e-5)
    bwd = oracle.propagate_backward(blocks, x, n, data.rule_cnt)
    np.testing.assert_allclose(bwd, dense @ x, rtol=1e-4, atol=1e-5)
    # csc() of a block is the stable transpose the oracle computes
    for name in ("v2v", "v2r", "r2v"):
        blk = getattr(graph, f"{name}_graph")
        for mine, ref in zip(blk.csc(), oracle.transpose_csr(*blocks[name], blk.sparse_sizes()[1])):
            np.testing.assert_array_equal(mine.numpy(), ref)
    vd, rd = graph.vertex_degree.numpy(), graph.rule_degree.numpy()
    assert vd.sum() == se.size  # every original entry (self loops included) is accounted for
    assert rd.min() >= 1


def test_helpers_match_the_compiled_reference_when_present():
    _rt, ref = oracle.reference_modules()
    if ref is None:
        pytest.skip("oracle/_ref not built in this checkout")
    for seed, cand in ((1, 1), (2, 8)):
        n = 4000
        v, e = off.generate_copy_graph(n, 2.1, 5.0, 300, 0.7, 64, cand, seed=seed)
        sv, se = off.add_self_loop_csr(v, e)
        rsv, rse = ref.add_self_loop_csr(v, e)
        np.testing.assert_array_equal(sv, rsv)
        np.testing.assert_array_equal(se, rse)
        nd = off.get_norm_degree(se, n)
        np.testing.assert_array_equal(nd, ref.get_norm_degree(se, n))
        packed = off.compress_csr_batch(sv, se, min_pair_frequency=3)
        cv, ce = packed[0].astype(np.int64), packed[1].astype(np.int64)
        for thr in (0, 3, 16):
            mine = off.filter_csr(cv, ce, packed[2], packed[3], thr)
            theirs = ref.filter_csr(cv, ce, packed[2], packed[3], thr)
            assert mine[2:] == tuple(theirs[2:])
            np.testing.assert_array_equal(mine[0], theirs[0])
            np.testing.assert_array_equal(mine[1], theirs[1])
            for max_depth, min_edge in ((3, 1000000), (2, 10), (1, 0), (3, 200)):
                dm = off.depth_filter_csr(*mine, max_depth, min_edge)
                dt = ref.depth_filter_csr(*theirs, max_depth, min_edge)
                assert dm[2:] == tuple(dt[2:])
                np.testing.assert_array_equal(dm[0], dt[0])
                np.testing.assert_array_equal(dm[1], dt[1])
        fv, fe, fn, fr = off.filter_csr(cv, ce, packed[2], packed[3], 1)
        w = off.gcn_norm_csr_compress(fv, fe, nd, fn, fr)
        np.testing.assert_array_equal(w, ref.gcn_norm_csr_compress(fv, fe, nd, fn, fr))
        assert off.phase_count(fv, fe, fn, fr) == ref.gen_mask_vertex(fv, fe, fn, fr, "csc")[1]
        t = off.transpose_csr(fv, fe, w, fn + fr)
        mine, theirs = off.hybird_partition(*t, fn), ref.hybird_partition(*t, fn)
        for a, b in zip(mine, theirs):
            for x, y in zip(a, b):
                np.testing.assert_array_equal(x, y)
        lm, lt = off.topo_partition(*mine[3]), ref.topo_partition(*theirs[3])
        assert len(lm) == len(lt) >= 1
        for a, b in zip(lm, lt):
            for x, y in zip(a, b):
                np.testing.assert_array_equal(x, y)
        dm = off.gen_degree(mine[0][0], mine[0][1], mine[1][0], mine[1][1], mine[2][0], mine[2][1],
                            [l[0] for l in lm], [l[1] for l in lm])
        dt = ref.gen_degree(theirs[0][0], theirs[0][1], theirs[1][0], theirs[1][1], theirs[2][0],
                            theirs[2][1], [l[0] for l in lt], [l[1] for l in lt])
        np.testing.assert_array_equal(dm[0], dt[0])
        np.testing.assert_array_equal(dm[1], dt[1])
