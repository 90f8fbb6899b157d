"""Generate ``tests/golden/reference_vectors.npz`` from the reference's own CPU operators.

Run in a container that holds a checkout of ZhengChenCS/CompressGNN (``oracle/build_ref.py``
compiles its CPU runtime and offline helpers into ``oracle/_ref``):

    python oracle/build_ref.py && python tests/golden/make_golden.py

Every array written here is an input drawn from a seeded generator or an output of the
reference's code (``compressgnn_runtime.spmm_func`` / ``cluster_forward``,
``compressgnn_offline.hybird_partition`` / ``topo_partition`` / ``gcn_norm_csr_compress`` /
``get_norm_degree``) or of torch autograd applied to the reference's CPU formulas
(``layer/CompressgnnCluster.py:16-25``, ``layer/CompressgnnReconstruct.py:39-42``).
The committed ``.npz`` lets the same checks run where the reference is absent.
"""
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import oracle  # noqa: E402

rt, off = oracle.reference_modules()
assert rt is not None and off is not None, "build oracle/_ref first (python oracle/build_ref.py)"
torch.set_num_threads(1)
rng = np.random.default_rng(20241125)
out = {}


def t(a):
    return torch.from_numpy(np.ascontiguousarray(a))


# --- 1. plain SpMM block, fresh and accumulating ------------------------------------------
rows, src_rows, width = 37, 53, 33
deg = rng.integers(0, 9, rows)
deg[5] = 0
deg[11] = 40  # one long row
rowptr = np.zeros(rows + 1, np.int64)
rowptr[1:] = np.cumsum(deg)
col = rng.integers(0, src_rows, rowptr[-1]).astype(np.int64)
val = rng.standard_normal(rowptr[-1]).astype(np.float32)
mat = rng.standard_normal((src_rows, width)).astype(np.float32)
base = rng.standard_normal((rows, width)).astype(np.float32)
out["spmm_rowptr"], out["spmm_col"], out["spmm_val"], out["spmm_mat"], out["spmm_base"] = \
    rowptr, col, val, mat, base
out["spmm_out"] = rt.spmm_func(t(rowptr), t(col), t(val), t(mat), "rowbalance", None).numpy()
acc = t(base.copy())
out["spmm_out_acc"] = rt.spmm_func(t(rowptr), t(col), t(val), t(mat), "rowbalance", acc).numpy()
out["spmm_out_nnzbalance"] = rt.spmm_func(t(rowptr), t(col), t(val), t(mat), "nnzbalance", None).numpy()

# --- 2. compressed propagation over a hand-built rule DAG --------------------------------
# Original graph: 8 vertices; rule ids >= 8; children of a rule are smaller than the rule.
n = 8
compressed_rows = [
    [9, 3],        # v0
    [9],           # v1
    [8, 10, 5],    # v2
    [10, 0, 11],   # v3
    [8, 7],        # v4
    [1, 2, 9],     # v5
    [11],          # v6
    [6, 11, 8],    # v7
    [0, 1],        # r8
    [8, 2],        # r9  (nested: contains r8)
    [3, 4],        # r10
    [9, 10, 5],    # r11 (two levels deep)
]
r = len(compressed_rows) - n
vlist = np.zeros(n + r + 1, np.int64)
vlist[1:] = np.cumsum([len(x) for x in compressed_rows])
elist = np.array([c for row in compressed_rows for c in row], np.int64)


def expand(node):
    res = []
    for c in compressed_rows[node]:
        res += [c] if c < n else expand(c)
    return res


orig_rows = [sorted(expand(v)) for v in range(n)]
orig_dst = np.array([c for row in orig_rows for c in row], np.int64)
norm_degree = off.get_norm_degree(orig_dst, n)
weight = off.gcn_norm_csr_compress(vlist, elist, norm_degree, n, r)
# The reference hands the *transposed* graph to CompressGraph (loader/CompressgnnData.py:180).
t_vlist, t_elist, t_val = oracle.transpose_csr(vlist, elist, weight, n + r)
v2v, v2r, r2v, r2r = off.hybird_partition(t_vlist, t_elist, t_val.astype(np.float32), n)
levels = off.topo_partition(r2r[0], r2r[1], r2r[2])
out["dag_vlist"], out["dag_elist"], out["dag_weight"] = vlist, elist, weight
out["dag_norm_degree"] = norm_degree
out["dag_n"], out["dag_r"], out["dag_step"] = np.int64(n), np.int64(r), np.int64(len(levels))
for name, blk in (("v2v", v2v), ("v2r", v2r), ("r2v", r2v), ("r2r", r2r)):
    for part, arr in zip(("rowptr", "col", "val"), blk):
        out[f"dag_{name}_{part}"] = np.asarray(arr)
for i, blk in enumerate(levels):
    for part, arr in zip(("rowptr", "col", "val"), blk):
        out[f"dag_level{i}_{part}"] = np.asarray(arr)
x = rng.standard_normal((n, 12)).astype(np.float32)
g = rng.standard_normal((n, 12)).astype(np.float32)
out["dag_x"], out["dag_grad"] = x, g


def ref_spmm(blk, m, o=None):
    return rt.spmm_func(t(blk[0]), t(blk[1]), t(blk[2]), m, "rowbalance", o)


# forward in the call order of layer/CompressgnnSPMM.py:47-53
rule_out = ref_spmm(r2v, t(x))
for blk in levels:
    rule_out = ref_spmm(blk, rule_out, rule_out)
fwd = ref_spmm(v2v, t(x), ref_spmm(v2r, rule_out))
out["dag_forward"] = fwd.numpy()
# backward in the call order of the reference's GPU branch (layer/CompressgnnSPMM.py:80-85)
tr = lambda blk, ncols: oracle.transpose_csr(np.asarray(blk[0]), np.asarray(blk[1]), np.asarray(blk[2]), ncols)
rule_g = ref_spmm(tr(v2r, r), t(g))
for blk in reversed(levels):
    rule_g = ref_spmm(tr(blk, r), rule_g, rule_g)
bwd = ref_spmm(tr(r2v, n), rule_g, ref_spmm(tr(v2v, n), t(g)))
out["dag_backward"] = bwd.numpy()
# dense cross-check: forward must equal A_hat^T x with A_hat the normalised original graph
dense = np.zeros((n, n))
for v, row in enumerate(orig_rows):
    for c in row:
        dense[v, c] += norm_degree[v] * norm_degree[c]
assert np.allclose(dense.T @ x, out["dag_forward"], atol=1e-5)
assert np.allclose(dense @ g, out["dag_backward"], atol=1e-5)

# --- 3. LSH assignment --------------------------------------------------------------------
# (a) integer-valued features/planes: every dot product is exact in fp32 whatever the
#     summation order, so ids must match the reference bit for bit.
for tag, (nn, width, bits) in {"a": (257, 33, 8), "b": (300, 128, 16), "c": (67, 31, 3)}.items():
    xi = rng.integers(-4, 5, (nn, width)).astype(np.float32)
    wi = rng.integers(-3, 4, (width, bits)).astype(np.float32)
    ids, active = rt.cluster_forward(t(xi), t(wi), bits)
    out[f"lsh_{tag}_x"], out[f"lsh_{tag}_planes"] = xi, wi
    out[f"lsh_{tag}_ids"], out[f"lsh_{tag}_active"] = ids.numpy(), np.int64(active)
# (b) N(0,1) inputs; rows whose smallest |projection| (fp64) is below 1e-4 are dropped so the
#     BLAS summation order of the reference cannot flip a sign.
nn, width, bits = 400, 64, 12
xf = rng.standard_normal((nn, width)).astype(np.float32)
wf = rng.standard_normal((width, bits)).astype(np.float32)
margin = np.abs(xf.astype(np.float64) @ wf.astype(np.float64)).min(axis=1)
xf = xf[margin > 1e-4]
ids, active = rt.cluster_forward(t(xf), t(wf), bits)
out["lsh_f_x"], out["lsh_f_planes"] = xf, wf
out["lsh_f_ids"], out["lsh_f_active"] = ids.numpy(), np.int64(active)

# --- 4. mean / reconstruct, forward and backward (reference CPU formulas + autograd) --------
index = t(out["lsh_a_ids"].astype(np.int64))
groups = int(out["lsh_a_active"]) + 1
counts = torch.bincount(index, minlength=groups).to(torch.int32)
feat = torch.from_numpy(rng.standard_normal((257, 33)).astype(np.float32)).requires_grad_()
sums = torch.zeros(groups, 33).index_add_(0, index, feat)
mean = sums / counts.clamp_min(1).to(torch.float32)[:, None]  # scatter_mean arithmetic
gm = torch.from_numpy(rng.standard_normal((groups, 33)).astype(np.float32))
out["mean_x"], out["mean_index"], out["mean_counts"] = feat.detach().numpy(), index.numpy(), counts.numpy()
out["mean_out"] = mean.detach().numpy()
out["mean_grad_out"] = gm.numpy()
out["mean_grad_in"] = (gm.index_select(0, index) /
                       counts.index_select(0, index).clamp_min(1).to(torch.float32)[:, None]).numpy()
reps = torch.from_numpy(rng.standard_normal((groups, 33)).astype(np.float32)).requires_grad_()
bias = torch.from_numpy(rng.standard_normal(33).astype(np.float32)).requires_grad_()
go = torch.from_numpy(rng.standard_normal((257, 33)).astype(np.float32))
out["rec_reps"], out["rec_bias"], out["rec_grad_out"] = reps.detach().numpy(), bias.detach().numpy(), go.numpy()
for tag, relu in (("lin", False), ("relu", True)):
    y = reps.index_select(0, index) + bias
    if relu:
        y = y.relu()
    dr, db = torch.autograd.grad(y, (reps, bias), go)
    out[f"rec_{tag}_out"], out[f"rec_{tag}_dreps"], out[f"rec_{tag}_dbias"] = \
        y.detach().numpy(), dr.numpy(), db.numpy()

path = Path(__file__).resolve().parent / "reference_vectors.npz"
np.savez_compressed(path, **out)
print("wrote", path, path.stat().st_size, "bytes,", len(out), "arrays")
