"""Neighbour sampling on the compressed graph, CUDA against the CPU restatement (which is pinned to the
reference's own host sampler in test_sample_oracle.py): same seeds and fan-outs, the same counter-based
random indices on both sides, so samples, rows and cols must be equal element for element."""
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import oracle

pytestmark = pytest.mark.gpu
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


def cu(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def device_sample(g, seeds, fanouts, seed):
    from compressgnn_b200.sample import neighbor_sample_cg_sim
    return neighbor_sample_cg_sim(cu(g["v2v"][0]), cu(g["v2v"][1]), cu(g["v2r"][0]), cu(g["v2r"][1]), cu(g["r2v"][0]),
                                  cu(g["r2v"][1]), [cu(l[0]) for l in g["r2r_levels"]], [cu(l[1]) for l in g["r2r_levels"]],
                                  cu(g["v_degree"]), cu(g["r_degree"]), cu(seeds), list(fanouts), seed=seed)


@pytest.mark.parametrize("tag", ["a", "b"])
def test_reference_graphs(vectors, tag):
    from compressgnn_b200 import runtime as rt
    g = graph_of(vectors, tag)
    seeds = vectors[f"{tag}_seeds"]
    for k in range(int(vectors[f"{tag}_cases"])):
        fanouts = vectors[f"{tag}_{k}_fanouts"].tolist()
        for seed in (0, 12345678901234):
            got = device_sample(g, seeds, fanouts, seed)
            want = oracle.neighbor_sample(seeds=seeds, fanouts=fanouts, seed=seed, **g)
            for mine, theirs in zip(got, want):
                np.testing.assert_array_equal(mine.cpu().numpy(), theirs)
        if max(fanouts) >= 1000 and len(fanouts) == 1:  # nothing random: the reference's own output
            for name, mine in zip(("samples", "rows", "cols"), got):
                np.testing.assert_array_equal(mine.cpu().numpy(), vectors[f"{tag}_{k}_{name}"])
    rt.raise_on_device_status()


def nested_graph(n=3000, seed=5):
    from compressgnn_b200 import offline as off
    from compressgnn_b200.loader import CompressgnnData
    v, e = off.generate_copy_graph(n, alpha=2.1, x_min=5.3, max_degree=400, copy_prob=0.7, window=64, candidates=8, seed=seed)
    mask = np.ones(n, bool)
    data = CompressgnnData(np.zeros((n, 1), np.float32), (v, e), np.zeros(n, np.int64), mask, mask, mask,
                           min_pair_frequency=3, threshold=1, min_edge=10, max_depth=6)
    return data.edge_index


def test_nested_rules_and_the_sampler_object():
    """Rules three deep (where the degrees must come from exact_degrees), through CompressGraphSampler."""
    from compressgnn_b200 import runtime as rt
    from compressgnn_b200.sample import CompressGraphSampler
    graph = nested_graph()
    assert graph.step >= 2
    blk = lambda b: tuple(x.numpy() for x in b.csr()[:2])
    blocks = (blk(graph.v2v_graph), blk(graph.v2r_graph), blk(graph.r2v_graph), [blk(l) for l in graph.r2r_graph])
    v_degree, r_degree = oracle.exact_degrees(*blocks)
    graph.to("cuda")
    sampler = graph.neighbor_sampler()
    assert isinstance(sampler, CompressGraphSampler) and graph.neighbor_sampler() is sampler
    np.testing.assert_array_equal(sampler._arrays[8].cpu().numpy(), v_degree)
    np.testing.assert_array_equal(sampler._arrays[9].cpu().numpy(), r_degree)
    rng = np.random.default_rng(1)
    for trial, fanouts in enumerate(([5, 5], [1000], [25, 10], [1, 1, 1, 1], [3, 0, 3])):
        seeds = rng.choice(graph.vertex_cnt, size=64, replace=False)
        got = sampler(torch.from_numpy(seeds), fanouts, seed=trial)
        want = oracle.neighbor_sample(*blocks, v_degree, r_degree, seeds, fanouts, seed=trial)
        for mine, theirs in zip(got, want):
            np.testing.assert_array_equal(mine.cpu().numpy(), theirs)
        again = sampler(torch.from_numpy(seeds), fanouts, seed=trial)  # the per-vertex tables were handed back clean
        assert all(torch.equal(a, b) for a, b in zip(got, again))
    other = sampler(torch.from_numpy(seeds), [5, 5], seed=99)
    assert not torch.equal(other[0], sampler(torch.from_numpy(seeds), [5, 5], seed=98)[0])
    empty = sampler(torch.empty(0, dtype=torch.int64), [5])
    assert all(t.numel() == 0 for t in empty)
    rt.raise_on_device_status()


def test_batches_of_the_benchmark_graph():
    """1024 seeds, fan-outs 25 and 10 on the 325 k-node graph: counts, membership and numbering."""
    import bench
    from compressgnn_b200 import runtime as rt
    from compressgnn_b200.sample import CompressGraphSampler
    data, _ = bench.build_graph("propagation")
    graph = data.edge_index
    blk = lambda b: tuple(x.numpy().copy() for x in b.csr()[:2])
    blocks = (blk(graph.v2v_graph), blk(graph.v2r_graph), blk(graph.r2v_graph), [blk(l) for l in graph.r2r_graph])
    v_degree, r_degree = oracle.exact_degrees(*blocks)
    lists = oracle.CompressedNeighbors(*blocks, v_degree, r_degree)
    graph.to("cuda")
    sampler = CompressGraphSampler.from_graph(graph)
    seeds = np.random.default_rng(7).choice(graph.vertex_cnt, size=1024, replace=False)
    fanouts = [25, 10]
    samples, rows, cols = (t.cpu().numpy() for t in sampler(torch.from_numpy(seeds), fanouts, seed=3))
    np.testing.assert_array_equal(samples[:1024], seeds)
    assert np.unique(samples).size == samples.size                      # every node has one local id
    order = cols[np.sort(np.unique(cols, return_index=True)[1])]         # local ids in order of first use as a target
    fresh = order[order >= 1024]
    np.testing.assert_array_equal(fresh, np.arange(1024, 1024 + fresh.size))  # new nodes are numbered as first seen
    per_row = np.bincount(rows, minlength=samples.size)
    hop_of = np.zeros(samples.size, int)
    hop_of[1024:] = 1
    frontier_end = rows.max() + 1
    want = np.minimum(v_degree[samples[:frontier_end]], np.array(fanouts)[hop_of[:frontier_end]])
    np.testing.assert_array_equal(per_row[:frontier_end], want)
    for local in list(range(0, 1024, 97)) + list(range(1024, frontier_end, 1501)):   # membership, with multiplicity
        mine = sorted(samples[cols[rows == local]].tolist())
        allowed = sorted(lists.neighbor_list(int(samples[local])))
        it = iter(allowed)
        assert all(any(x == y for y in it) for x in mine), local
    rt.raise_on_device_status()


def test_a_seed_outside_the_graph_is_reported_not_followed(vectors):
    from compressgnn_b200 import runtime as rt
    g = graph_of(vectors, "b")
    device_sample(g, np.array([3, 10 ** 6], np.int64), [2], 0)
    with pytest.raises(RuntimeError):
        rt.raise_on_device_status()


def test_plain_graph_form(vectors):
    """neighbor_sample_ori_impl: an uncompressed CSC graph, i.e. no rules at all."""
    from compressgnn_b200 import runtime as rt
    from compressgnn_b200.sample import neighbor_sample_ori_impl
    colptr, row = vectors["b_v2v_ptr"], vectors["b_v2v_col"]
    seeds = vectors["b_seeds"]
    for trial, fanouts in enumerate(([3, 3], [1000, 1], [1, 1, 1])):
        got = neighbor_sample_ori_impl(cu(colptr), cu(row), cu(seeds), fanouts, seed=trial)
        want = oracle.neighbor_sample_plain(colptr, row, seeds, fanouts, seed=trial)
        for mine, theirs in zip(got, want):
            np.testing.assert_array_equal(mine.cpu().numpy(), theirs)
    rt.raise_on_device_status()

