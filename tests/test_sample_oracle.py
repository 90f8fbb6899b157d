"""The CPU restatement of neighbour sampling on the compressed graph against vectors produced by the
reference's own host sampler (tests/golden/make_sample_golden.py), and against that sampler itself when
oracle/_ref holds it."""
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import oracle

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def vectors():
    with np.load(ROOT / "tests" / "golden" / "sample_vectors.npz") as data:
        return {k: data[k] for k in data.files}


def graph_of(vectors, tag):
    levels = [(vectors[f"{tag}_r2r{i}_ptr"], vectors[f"{tag}_r2r{i}_col"]) for i in range(int(vectors[f"{tag}_levels"]))]
    return dict(v2v=(vectors[f"{tag}_v2v_ptr"], vectors[f"{tag}_v2v_col"]),
                v2r=(vectors[f"{tag}_v2r_ptr"], vectors[f"{tag}_v2r_col"]),
                r2v=(vectors[f"{tag}_r2v_ptr"], vectors[f"{tag}_r2v_col"]), r2r_levels=levels,
                v_degree=vectors[f"{tag}_v_degree"], r_degree=vectors[f"{tag}_r_degree"])


@pytest.mark.parametrize("tag", ["a", "b"])
def test_oracle_replays_the_reference_sampler(vectors, tag):
    g = graph_of(vectors, tag)
    for k in range(int(vectors[f"{tag}_cases"])):
        draws = iter(vectors[f"{tag}_{k}_draws"].tolist())
        got = oracle.neighbor_sample(seeds=vectors[f"{tag}_seeds"], fanouts=vectors[f"{tag}_{k}_fanouts"].tolist(),
                                     draw=lambda j, *_: next(draws), **g)
        for name, mine in zip(("samples", "rows", "cols"), got):
            np.testing.assert_array_equal(mine, vectors[f"{tag}_{k}_{name}"])
        assert next(draws, None) is None  # every recorded draw was used


@pytest.mark.parametrize("tag", ["a", "b"])
def test_oracle_against_the_compiled_reference_sampler(vectors, tag):
    ref = oracle.reference_sample_module()
    if ref is None:
        pytest.skip("oracle/_ref/compressgnn_sample.so is not built here")
    g = graph_of(vectors, tag)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a))
    seeds = vectors[f"{tag}_seeds"]
    for trial, fanouts in enumerate(([2], [3, 3], [1000, 2], [1, 2, 3])):
        torch.manual_seed(trial)
        want = ref.neighbor_sample_cg_sim(t(g["v2v"][0]), t(g["v2v"][1]), t(g["v2r"][0]), t(g["v2r"][1]), t(g["r2v"][0]),
                                          t(g["r2v"][1]), [t(l[0]) for l in g["r2r_levels"]],
                                          [t(l[1]) for l in g["r2r_levels"]], t(g["v_degree"]), t(g["r_degree"]),
                                          t(seeds), list(fanouts))
        torch.manual_seed(trial)
        got = oracle.neighbor_sample(seeds=seeds, fanouts=fanouts, draw=lambda j, *_: int(torch.randint(0, j, (1,))), **g)
        for mine, theirs in zip(got, want):
            np.testing.assert_array_equal(mine, theirs.numpy())


def test_index_order_and_list_order_cover_the_same_neighbours(vectors):
    """On every node: the neighbours reached by index 0 .. degree-1 are the neighbour list as a multiset, and
    the list has ``vertex_degree`` entries -- also below nested rules, where the reference's level lookup
    does not follow (built here with rules three deep)."""
    from compressgnn_b200 import offline as off
    from compressgnn_b200.loader import CompressgnnData
    n = 500
    v, e = off.generate_copy_graph(n, alpha=2.1, x_min=5.3, max_degree=200, copy_prob=0.7, window=64, candidates=8, seed=5)
    mask = np.ones(n, bool)
    data = CompressgnnData(np.zeros((n, 1), np.float32), (v, e), np.zeros(n, np.int64), mask, mask, mask,
                           min_pair_frequency=3, threshold=1, min_edge=10, max_depth=6, compression_backend="cpu")
    g = data.edge_index
    assert g.step >= 2
    blk = lambda b: tuple(x.numpy() for x in b.csr()[:2])
    blocks = (blk(g.v2v_graph), blk(g.v2r_graph), blk(g.r2v_graph), [blk(l) for l in g.r2r_graph])
    v_degree, r_degree = oracle.exact_degrees(*blocks)
    # the reference's gen_degree (which CompressGraph.vertex_degree follows) walks the levels last to first
    # and comes out short below nested rules
    assert (v_degree >= g.vertex_degree.numpy()).all() and (v_degree > g.vertex_degree.numpy()).any()
    graph = oracle.CompressedNeighbors(*blocks, v_degree, r_degree)
    sv, se = off.add_self_loop_csr(v, e)
    incoming = [[] for _ in range(n)]  # the loader hands over the transposed graph: a node lists what flows into it
    for src in range(n):
        for dst in se[sv[src]:sv[src + 1]]:
            incoming[dst].append(src)
    for node in range(n):
        listed = graph.neighbor_list(node)
        assert len(listed) == int(v_degree[node])
        assert sorted(listed) == sorted(graph.neighbor_at(node, i) for i in range(len(listed)))
        assert sorted(listed) == sorted(incoming[node])


def test_plain_graph_form_against_the_compiled_reference(vectors):
    ref = oracle.reference_sample_module()
    if ref is None:
        pytest.skip("oracle/_ref/compressgnn_sample.so is not built here")
    colptr, row = vectors["a_v2v_ptr"], vectors["a_v2v_col"]   # any CSR serves as an uncompressed graph
    seeds = vectors["a_seeds"][:4]
    for trial, fanouts in enumerate(([2, 2], [1000], [1, 3])):
        torch.manual_seed(40 + trial)
        want = ref.neighbor_sample_ori_impl(torch.from_numpy(colptr), torch.from_numpy(row), torch.from_numpy(seeds),
                                            list(fanouts))
        torch.manual_seed(40 + trial)
        got = oracle.neighbor_sample_plain(colptr, row, seeds, fanouts, draw=lambda j, *_: int(torch.randint(0, j, (1,))))
        for mine, theirs in zip(got, want):
            np.testing.assert_array_equal(mine, theirs.numpy())


def test_host_side_of_the_device_sampler(vectors):
    """The two pieces of compressgnn_b200.sample that are plain tensor code: one rule -> rule CSR out of the
    level blocks, and the exact degrees (against the oracle's, and against the reference's gen_degree arrays
    on a graph of one level, where the two agree)."""
    from compressgnn_b200.sample import exact_degrees, merge_rule_levels
    g = graph_of(vectors, "a")
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a))
    rules = g["r_degree"].size
    ptr, col = merge_rule_levels([t(l[0]) for l in g["r2r_levels"]], [t(l[1]) for l in g["r2r_levels"]], rules,
                                 torch.device("cpu"))
    lists = oracle.CompressedNeighbors(**g)
    for rule in range(rules):
        assert col[ptr[rule]:ptr[rule + 1]].tolist() == lists.children(rule)
    v_degree, r_degree = exact_degrees(t(g["v2v"][0]), t(g["v2r"][0]), t(g["v2r"][1]), t(g["r2v"][0]),
                                       [t(l[0]) for l in g["r2r_levels"]], [t(l[1]) for l in g["r2r_levels"]])
    want_v, want_r = oracle.exact_degrees(g["v2v"], g["v2r"], g["r2v"], g["r2r_levels"])
    np.testing.assert_array_equal(v_degree.numpy(), want_v)
    np.testing.assert_array_equal(r_degree.numpy(), want_r)
    np.testing.assert_array_equal(want_v, g["v_degree"])   # one level: gen_degree's arrays are exact
    np.testing.assert_array_equal(want_r, g["r_degree"])

