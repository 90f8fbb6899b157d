"""Generate ``tests/golden/sample_vectors.npz`` from the reference's own host neighbour sampler.

    python oracle/build_ref.py && python tests/golden/make_sample_golden.py

``oracle/build_ref.py`` compiles ``src/sample/csrc`` of a CompressGNN checkout into
``oracle/_ref/compressgnn_sample.so``.  For each case the file holds the compressed graph (CSR blocks and
the two degree arrays, produced by this package's loader from a seeded synthetic graph), the seeds, the
fan-outs, the random indices the reference drew (``torch::randint(0, j, {1})`` per draw, replayed here by
the same calls under the same ``torch.manual_seed``), and the reference's ``(samples, rows, cols)``.
"""
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import oracle  # noqa: E402
from compressgnn_b200 import offline as off  # noqa: E402
from compressgnn_b200.loader import CompressgnnData  # noqa: E402

ref = oracle.reference_sample_module()
assert ref is not None, "build oracle/_ref first (python oracle/build_ref.py)"
out = {}
t = lambda a: torch.from_numpy(np.ascontiguousarray(a))


def graph_arrays(n, seed, max_depth):
    v, e = off.generate_copy_graph(n, alpha=2.1, x_min=5.3, max_degree=200, copy_prob=0.7, window=64, candidates=8,
                                   seed=seed)
    mask = np.ones(n, bool)
    data = CompressgnnData(np.zeros((n, 1), np.float32), (v, e), np.zeros(n, np.int64), mask, mask, mask,
                           min_pair_frequency=3, threshold=1, min_edge=10**9, max_depth=max_depth,
                           compression_backend="cpu")
    g = data.edge_index
    blk = lambda b: tuple(x.numpy() for x in b.csr()[:2])
    return dict(v2v=blk(g.v2v_graph), v2r=blk(g.v2r_graph), r2v=blk(g.r2v_graph),
                r2r_levels=[blk(l) for l in g.r2r_graph], v_degree=g.vertex_degree.numpy(),
                r_degree=g.rule_degree.numpy())


# Rule graphs of at most one level (the depth filter cuts deeper ones down): get_neighbor / get_neighbor_list look a rule's children up
# in the level block numbered by the descent depth (storage_api.h:35-52, :94-107), which is the block that
# lists them only for a rule whose own children have none; below a deeper rule the reference returns
# elements of the wrong list.
cases = [("a", 600, 3, 3, [5, 17, 300, 42, 5], [[1000], [3, 2], [1, 1, 1], [5, 1000]]),
         ("b", 400, 9, 2, list(range(0, 400, 37)), [[4, 4], [2, 1000, 1], [7]])]
for tag, n, seed, max_depth, seeds, fanout_lists in cases:
    g = graph_arrays(n, seed, max_depth)
    assert len(g["r2r_levels"]) <= 1 and g["r_degree"].size > 20
    seeds = np.array(seeds, np.int64)
    for name in ("v2v", "v2r", "r2v"):
        out[f"{tag}_{name}_ptr"], out[f"{tag}_{name}_col"] = g[name]
    out[f"{tag}_levels"] = np.int64(len(g["r2r_levels"]))
    for i, (p, c) in enumerate(g["r2r_levels"]):
        out[f"{tag}_r2r{i}_ptr"], out[f"{tag}_r2r{i}_col"] = p, c
    out[f"{tag}_v_degree"], out[f"{tag}_r_degree"], out[f"{tag}_seeds"] = g["v_degree"], g["r_degree"], seeds
    out[f"{tag}_cases"] = np.int64(len(fanout_lists))
    for k, fanouts in enumerate(fanout_lists):
        torch.manual_seed(100 + k)
        got = ref.neighbor_sample_cg_sim(t(g["v2v"][0]), t(g["v2v"][1]), t(g["v2r"][0]), t(g["v2r"][1]),
                                         t(g["r2v"][0]), t(g["r2v"][1]), [t(l[0]) for l in g["r2r_levels"]],
                                         [t(l[1]) for l in g["r2r_levels"]], t(g["v_degree"]), t(g["r_degree"]),
                                         t(seeds), list(fanouts))
        drawn = []

        def draw(j, *_):
            drawn.append(int(torch.randint(0, j, (1,))))
            return drawn[-1]

        torch.manual_seed(100 + k)
        mine = oracle.neighbor_sample(seeds=seeds, fanouts=fanouts, draw=draw, **g)
        assert all(np.array_equal(a.numpy(), b) for a, b in zip(got, mine)), (tag, fanouts)
        out[f"{tag}_{k}_fanouts"] = np.array(fanouts, np.int64)
        out[f"{tag}_{k}_draws"] = np.array(drawn, np.int64)
        for name, arr in zip(("samples", "rows", "cols"), got):
            out[f"{tag}_{k}_{name}"] = arr.numpy()
        print(tag, fanouts, "levels", len(g["r2r_levels"]), "samples", got[0].numel(), "edges", got[1].numel(),
              "draws", len(drawn))

path = Path(__file__).with_name("sample_vectors.npz")
np.savez_compressed(path, **out)
print("wrote", path, path.stat().st_size, "bytes")
