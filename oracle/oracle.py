"""TEST INFRASTRUCTURE -- numpy front end of the CPU oracle (``cgnn_oracle.c``).

Only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline legs import
this module; the product package never does.  The arithmetic lives in ``cgnn_oracle.c``
(each function cites the reference lines it follows); this file compiles it with gcc,
wraps it for numpy arrays, and composes the level-ordered compressed propagation exactly
in the call order of the reference's ``layer/CompressgnnSPMM.py``.

Parity pin: ``tests/test_oracle_pins.py`` checks every function here against the
reference's own CPU operators (``oracle/_ref``, built by ``build_ref.py`` from the
reference sources) and against the committed fixtures in ``tests/golden/``.
"""
import ctypes
import subprocess
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
_SRC = HERE / "cgnn_oracle.c"
_LIB = HERE / "libcgnn_oracle.so"
_lib = None


def build(force=False):
    """Compile the C restatement next to its source (gcc only, no other dependency)."""
    if force or not _LIB.is_file() or _LIB.stat().st_mtime < _SRC.stat().st_mtime:
        subprocess.run(["gcc", "-O2", "-ffp-contract=off", "-shared", "-fPIC", str(_SRC),
                        "-lm", "-o", str(_LIB)], check=True)
    return _LIB


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(str(build()))
    return _lib


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p) if a is not None else None


def _suf(dtype):
    dtype = np.dtype(dtype)
    if dtype == np.float32:
        return "f32"
    if dtype == np.float64:
        return "f64"
    raise TypeError("oracle supports float32/float64 only")


def _c(a, dtype):
    return np.ascontiguousarray(a, dtype=dtype)


def _check(rc, what):
    if rc:
        raise RuntimeError(f"oracle {what} failed with status {rc}")


# ---------------------------------------------------------------------------------------
# SpMM and compressed propagation
# ---------------------------------------------------------------------------------------
def spmm(rowptr, col, val, mat, out=None):
    """``spmm_func(vlist, elist, value, mat, "rowbalance", out)`` on the CPU.

    Accumulates into ``out`` in place when given (and returns it), else into zeros.
    """
    mat = np.ascontiguousarray(mat)
    suf = _suf(mat.dtype)
    rowptr, col = _c(rowptr, np.int64), _c(col, np.int64)
    val = _c(val, mat.dtype)
    rows, width = rowptr.size - 1, mat.shape[1]
    if out is None:
        out = np.zeros((rows, width), dtype=mat.dtype)
    assert out.flags.c_contiguous and out.shape == (rows, width) and out.dtype == mat.dtype
    fn = getattr(lib(), f"oracle_spmm_rowbalance_{suf}")
    _check(fn(_p(rowptr), _p(col), _p(val), _p(mat), ctypes.c_int64(rows),
              ctypes.c_int64(width), _p(out)), "spmm")
    return out


def transpose_csr(rowptr, col, val, ncols):
    """Stable CSR transpose (entries of a column keep ascending row order), the data
    movement ``torch_sparse.SparseTensor.csc()`` performs for the reference
    (layer/CompressgnnSPMM.py:68-70, loader/CompressgnnData.py:180)."""
    rowptr, col = _c(rowptr, np.int64), _c(col, np.int64)
    rows = np.repeat(np.arange(rowptr.size - 1, dtype=np.int64), np.diff(rowptr))
    order = np.argsort(col, kind="stable")
    tptr = np.zeros(ncols + 1, dtype=np.int64)
    np.cumsum(np.bincount(col, minlength=ncols), out=tptr[1:])
    return tptr, rows[order], np.asarray(val)[order]


def propagate_forward(blocks, x):
    """Forward of ``Compressgnn_SPMM_Function`` (layer/CompressgnnSPMM.py:47-53):
    r2v, the r2r levels in place, v2r, then v2v accumulated.  ``blocks`` maps
    ``"v2v" | "v2r" | "r2v"`` to ``(rowptr, col, val)`` and ``"r2r"`` to a list of them."""
    rule_out = spmm(*blocks["r2v"], x)
    for level in blocks["r2r"]:
        rule_out = spmm(*level, rule_out, out=rule_out)
    out = spmm(*blocks["v2r"], rule_out)
    return spmm(*blocks["v2v"], x, out=out)


def propagate_backward(blocks, grad, n, r):
    """Backward in the order of the reference's GPU branch
    (layer/CompressgnnSPMM.py:65-70,80-85): transposed blocks, levels reversed.  (The
    reference's CPU branch at :71-78 cannot run: empty range, undefined names.)"""
    v2v_t = transpose_csr(*blocks["v2v"], n)
    v2r_t = transpose_csr(*blocks["v2r"], r)   # [r, n]
    r2v_t = transpose_csr(*blocks["r2v"], n)   # [n, r]
    rule_out = spmm(*v2r_t, grad)
    for level in reversed(blocks["r2r"]):
        rule_out = spmm(*transpose_csr(*level, r), rule_out, out=rule_out)
    out = spmm(*v2v_t, grad)
    return spmm(*r2v_t, rule_out, out=out)


# ---------------------------------------------------------------------------------------
# Cluster / reconstruct
# ---------------------------------------------------------------------------------------
def project(x, planes, shards=1):
    x, planes = np.ascontiguousarray(x), np.ascontiguousarray(planes)
    suf = _suf(x.dtype)
    n, width = x.shape
    bits = planes.shape[1]
    proj = np.zeros((n, bits), dtype=x.dtype)
    if shards == 1:
        fn = getattr(lib(), f"oracle_project_{suf}")
        _check(fn(_p(x), _p(planes), ctypes.c_int64(n), ctypes.c_int64(width), bits, _p(proj)),
               "project")
    else:
        assert suf == "f32"
        _check(lib().oracle_project_sharded_f32(_p(x), _p(planes), ctypes.c_int64(n),
                                                ctypes.c_int64(width), bits, int(shards),
                                                _p(proj)), "project_sharded")
    return proj


def codes_from_projection(proj):
    proj = np.ascontiguousarray(proj)
    n, bits = proj.shape
    codes = np.zeros(n, dtype=np.int32)
    fn = getattr(lib(), f"oracle_codes_{_suf(proj.dtype)}")
    _check(fn(_p(proj), ctypes.c_int64(n), bits, _p(codes)), "codes")
    return codes


def assign_from_codes(codes, bits):
    codes = _c(codes, np.int32)
    n = codes.size
    ids = np.zeros(n, dtype=np.int64)
    counts = np.zeros(n + 1, dtype=np.int32)
    active = ctypes.c_int64(0)
    _check(lib().oracle_assign(_p(codes), ctypes.c_int64(n), int(bits), _p(ids), _p(counts),
                               ctypes.byref(active)), "assign")
    return ids, counts[:active.value + 1].copy(), int(active.value)


def cluster_assign(x, planes, shards=1):
    """``(ids int64[N] 1-based, counts int32[active+1], active)`` as
    ``layer/CompressgnnCluster.py:41-50`` returns them."""
    proj = project(x, planes, shards)
    return assign_from_codes(codes_from_projection(proj), planes.shape[1])


def _cluster_call(name, dtype, *args):
    fn = getattr(lib(), f"oracle_{name}_{_suf(dtype)}")
    _check(fn(*args), name)


def cluster_mean(x, index, counts):
    x = np.ascontiguousarray(x)
    index, counts = _c(index, np.int64), _c(counts, np.int32)
    out = np.zeros((counts.size, x.shape[1]), dtype=x.dtype)
    _cluster_call("mean", x.dtype, _p(x), _p(index), _p(counts), ctypes.c_int64(x.shape[0]),
                  ctypes.c_int64(x.shape[1]), ctypes.c_int64(counts.size), _p(out))
    return out


def cluster_mean_backward(grad, index, counts):
    grad = np.ascontiguousarray(grad)
    index, counts = _c(index, np.int64), _c(counts, np.int32)
    out = np.zeros((index.size, grad.shape[1]), dtype=grad.dtype)
    _cluster_call("mean_backward", grad.dtype, _p(grad), _p(index), _p(counts),
                  ctypes.c_int64(index.size), ctypes.c_int64(grad.shape[1]),
                  ctypes.c_int64(counts.size), _p(out))
    return out


def reconstruct(reps, index, bias=None, relu=False):
    reps = np.ascontiguousarray(reps)
    index = _c(index, np.int64)
    bias = None if bias is None else _c(bias, reps.dtype)
    out = np.zeros((index.size, reps.shape[1]), dtype=reps.dtype)
    _cluster_call("reconstruct", reps.dtype, _p(reps), _p(index), _p(bias), int(bool(relu)),
                  ctypes.c_int64(index.size), ctypes.c_int64(reps.shape[1]),
                  ctypes.c_int64(reps.shape[0]), _p(out))
    return out


def reconstruct_backward(grad, index, output, groups, relu=False):
    """Returns ``(d_reps [groups, F], d_bias [F])``."""
    grad, output = np.ascontiguousarray(grad), np.ascontiguousarray(output)
    index = _c(index, np.int64)
    out = np.zeros((groups, grad.shape[1]), dtype=grad.dtype)
    bias_grad = np.zeros(grad.shape[1], dtype=grad.dtype)
    _cluster_call("reconstruct_backward", grad.dtype, _p(grad), _p(output), _p(index),
                  int(bool(relu)), ctypes.c_int64(index.size), ctypes.c_int64(grad.shape[1]),
                  ctypes.c_int64(groups), _p(out), _p(bias_grad))
    return out, bias_grad


# ---------------------------------------------------------------------------------------
# The compiled reference (oracle/_ref), when present
# ---------------------------------------------------------------------------------------
def reference_modules():
    """Import ``compressgnn_runtime`` / ``compressgnn_offline`` built from the reference's
    own sources by ``build_ref.py``.  Returns ``(runtime, offline)``; either is ``None``
    when its shared object is absent."""
    ref_dir = HERE / "_ref"
    mods = []
    if str(ref_dir) not in sys.path:
        sys.path.insert(0, str(ref_dir))
    for name in ("compressgnn_runtime", "compressgnn_offline"):
        mod = None
        if (ref_dir / f"{name}.so").is_file():
            try:
                if name == "compressgnn_runtime":
                    import torch  # noqa: F401  (libtorch symbols must be loaded first)
                mod = __import__(name)
            except ImportError:
                mod = None
        mods.append(mod)
    return tuple(mods)


def reference_propagation(blocks, x, grad, n, r, threads=None):
    """One forward and one backward compressed propagation on the CPU by the strongest checker at
    hand: the reference's own compiled ``spmm_func(..., "rowbalance", ...)`` chained in the order
    of layer/CompressgnnSPMM.py:47-53 (forward) and :80-85 (backward) when ``oracle/_ref`` is
    present, else this module's C restatement.  ``blocks`` as for ``propagate_forward``.
    Returns ``(out, grad_in, kind)`` as numpy arrays with ``kind`` "reference" or "port"."""
    rt, _off = reference_modules()
    if rt is None:
        return propagate_forward(blocks, x), propagate_backward(blocks, grad, n, r), "port"
    import os
    import torch
    torch.set_num_threads(threads or os.cpu_count() or 1)
    t = lambda blk: tuple(torch.from_numpy(np.ascontiguousarray(a)) for a in blk)
    spmm_ref = lambda blk, m, out=None: rt.spmm_func(blk[0], blk[1], blk[2], m, "rowbalance", out)
    xt, gt = torch.from_numpy(np.ascontiguousarray(x)), torch.from_numpy(np.ascontiguousarray(grad))
    rule = spmm_ref(t(blocks["r2v"]), xt)
    for level in blocks["r2r"]:
        rule = spmm_ref(t(level), rule, rule)
    out = spmm_ref(t(blocks["v2v"]), xt, spmm_ref(t(blocks["v2r"]), rule))
    rule_g = spmm_ref(t(transpose_csr(*blocks["v2r"], r)), gt)
    for level in reversed(blocks["r2r"]):
        rule_g = spmm_ref(t(transpose_csr(*level, r)), rule_g, rule_g)
    gx = spmm_ref(t(transpose_csr(*blocks["r2v"], n)), rule_g, spmm_ref(t(transpose_csr(*blocks["v2v"], n)), gt))
    return out.numpy(), gx.numpy(), "reference"


def reference_cuda_module():
    """The reference's runtime built WITH its CUDA kernels (``oracle/_ref_cuda``, see
    ``build_ref.build_runtime_cuda``; module name ``compressgnn_runtime_cuda`` so that it can sit
    beside the CPU build), or ``None`` when it is absent."""
    ref_dir = HERE / "_ref_cuda"
    if not (ref_dir / "compressgnn_runtime_cuda.so").is_file():
        return None
    if str(ref_dir) not in sys.path:
        sys.path.insert(0, str(ref_dir))
    try:
        import torch  # noqa: F401  (libtorch symbols must be loaded first)
        return __import__("compressgnn_runtime_cuda")
    except ImportError:
        return None


def reference_cuda_step(rt, graph, x, grad):
    """One forward and one backward compressed propagation by the reference's own CUDA kernels, launched
    as its GPU branches launch them (layer/CompressgnnSPMM.py:14-19 method choice, :54-60 forward,
    :80-85 backward).  ``graph`` is a CompressGraph on the device, ``x`` / ``grad`` device matrices.

    The kernels form ``elist * col_num`` and ``row * col_num`` in 32-bit integers
    (sparse/cuda/row_balance.cuh:82-128, nnz_balance.cuh:145-200): callers stay below 2^31 elements."""
    rows = max(graph.vertex_cnt, graph.rule_cnt)
    if rows * x.size(1) >= 2 ** 31:
        raise ValueError("the reference's CUDA kernels index with 32-bit products: matrix too large")

    def gpu_spmm(blk, m, out, prefer_row=False):
        method = "rowbalance_rowcache" if (prefer_row and blk[1].numel() >= 1000000 and m.size(-1) >= 64) \
            else "nnzbalance_rowcache"
        return rt.spmm_func(blk[0], blk[1], blk[2], m, method, out)

    g = graph
    rule_out = gpu_spmm(g.r2v_graph.csr(), x, None, prefer_row=True)
    for level in g.r2r_graph:
        rule_out = gpu_spmm(level.csr(), rule_out, rule_out)
    out = gpu_spmm(g.v2r_graph.csr(), rule_out, None)
    out = gpu_spmm(g.v2v_graph.csr(), x, out, prefer_row=True)
    rule_g = gpu_spmm(g.v2r_graph.csc(), grad, None)
    for level in reversed(g.r2r_graph):
        rule_g = gpu_spmm(level.csc(), rule_g, rule_g)
    gx = gpu_spmm(g.v2v_graph.csc(), grad, None, prefer_row=True)
    gx = gpu_spmm(g.r2v_graph.csc(), rule_g, gx, prefer_row=True)
    return out, gx


# ---------------------------------------------------------------------------------------
# Neighbour sampling on the compressed graph
# ---------------------------------------------------------------------------------------
def reference_sample_module():
    """``compressgnn_sample`` built from the reference's own sources (``build_ref.py``), or ``None``."""
    ref_dir = HERE / "_ref"
    if not (ref_dir / "compressgnn_sample.so").is_file():
        return None
    if str(ref_dir) not in sys.path:
        sys.path.insert(0, str(ref_dir))
    try:
        import torch  # noqa: F401  (libtorch symbols must be loaded first)
        return __import__("compressgnn_sample")
    except ImportError:
        return None


def philox_first_word(c0, c1, c2, c3, seed):
    """First output word of Philox4x32 with 7 rounds (Salmon et al., SC 2011) for counter (c0..c3), key `seed`."""
    mask = 0xFFFFFFFF
    k0, k1 = seed & mask, (seed >> 32) & mask
    for _ in range(7):
        p0, p1 = 0xD2511F53 * c0, 0xCD9E8D57 * c2
        c0, c1, c2, c3 = ((p1 >> 32) ^ c1 ^ k0) & mask, p1 & mask, ((p0 >> 32) ^ c3 ^ k1) & mask, p0 & mask
        k0, k1 = (k0 + 0x9E3779B9) & mask, (k1 + 0xBB67AE85) & mask
    return c0


def exact_degrees(v2v, v2r, r2v, r2r_levels):
    """``(vertex_degree, rule_degree)``: the number of vertices a rule expands to and the number of
    neighbours of a vertex.  The level blocks are taken in the order topo_partition emits them (level 0:
    rules whose children have no children), so that a child's size is final before its parents add it.
    (gen_degree, src/offline/csrc/gen_degree.h:62-72, walks the levels from the last to the first and
    agrees with this up to one level.)"""
    r_degree = np.diff(r2v[0]).astype(np.int64)
    for ptr, col in r2r_levels:
        rows = np.repeat(np.arange(ptr.size - 1), np.diff(ptr))
        np.add.at(r_degree, rows, r_degree[col])
    v_degree = np.diff(v2v[0]).astype(np.int64)
    rows = np.repeat(np.arange(v2r[0].size - 1), np.diff(v2r[0]))
    np.add.at(v_degree, rows, r_degree[v2r[1]])
    return v_degree, r_degree


class CompressedNeighbors:
    """Neighbour lists of a compressed graph given as ``(rowptr, col)`` blocks: a node's neighbours are its
    v2v entries followed by the expansion of its v2r rules.  The children of a rule are taken from whichever
    level block lists them (the reference indexes the levels by descent depth, storage_api.h:35-52 and
    :94-107, which is the same block as long as the rule's children have no children themselves)."""

    def __init__(self, v2v, v2r, r2v, r2r_levels, v_degree, r_degree):
        (self.v2v_p, self.v2v_c), (self.v2r_p, self.v2r_c), (self.r2v_p, self.r2v_c) = v2v, v2r, r2v
        self.levels, self.v_degree, self.r_degree = list(r2r_levels), v_degree, r_degree

    def children(self, rule):
        out = []
        for ptr, col in self.levels:
            out.extend(col[ptr[rule]:ptr[rule + 1]].tolist())
        return out

    def neighbor_list(self, node):
        """All neighbours in list order (ref: get_neighbor_list, storage_api.h:72-118): v2v entries, then
        the rules below the node breadth first, then every listed rule's own vertices."""
        out = self.v2v_c[self.v2v_p[node]:self.v2v_p[node + 1]].tolist()
        queue = self.v2r_c[self.v2r_p[node]:self.v2r_p[node + 1]].tolist()
        head = 0
        while head < len(queue):
            queue.extend(self.children(queue[head]))
            head += 1
        for rule in queue:
            out.extend(self.r2v_c[self.r2v_p[rule]:self.r2v_p[rule + 1]].tolist())
        return out

    def neighbor_at(self, node, index):
        """The ``index``-th neighbour (ref: get_neighbor, storage_api.h:7-70): skip the v2v entries, then whole
        rules by ``rule_degree``; inside a rule its own vertices come first, then the child that holds the index."""
        count = self.v2v_p[node + 1] - self.v2v_p[node]
        if index < count:
            return int(self.v2v_c[self.v2v_p[node] + index])
        index -= count
        for rule in self.v2r_c[self.v2r_p[node]:self.v2r_p[node + 1]].tolist():
            if index >= self.r_degree[rule]:
                index -= int(self.r_degree[rule])
                continue
            while True:
                own = self.r2v_p[rule + 1] - self.r2v_p[rule]
                if index < own:
                    return int(self.r2v_c[self.r2v_p[rule] + index])
                index -= own
                for child in self.children(rule):
                    if index < self.r_degree[child]:
                        rule = child
                        break
                    index -= int(self.r_degree[child])
                else:
                    raise IndexError("neighbour index out of range")
        raise IndexError("neighbour index out of range")


def neighbor_sample(v2v, v2r, r2v, r2r_levels, v_degree, r_degree, seeds, fanouts, seed=0, draw=None):
    """``(samples, rows, cols)`` of neighbour sampling on a compressed graph, node by node as
    neighbor_sample_sim_impl does it (ref: src/sample/csrc/neighbor_sample.h:27-131): a frontier node whose
    degree does not exceed the fan-out contributes its whole neighbour list; any other node ``fanout``
    distinct neighbour indices by Floyd's scheme (:97-121), each resolved by ``neighbor_at``.  New nodes get
    local ids in the order they are first seen.  Random indices: ``draw(j, position, t, hop)`` uniform below
    ``j``; by default Philox words counted by (frontier position, draw, hop) under ``seed``, mapped by
    multiply-shift -- the generator of the device code; pass ``lambda j, *_: int(torch.randint(0, j, (1,)))``
    to follow the reference's own draws."""
    graph = CompressedNeighbors(v2v, v2r, r2v, r2r_levels, v_degree, r_degree)
    if draw is None:
        def draw(j, position, t, hop):
            word = philox_first_word(position & 0xFFFFFFFF, (position >> 32) & 0xFFFFFFFF, t, hop, seed)
            return (word * j) >> 32

    samples = [int(s) for s in seeds]
    local = {}
    for i, s in enumerate(samples):
        local.setdefault(s, i)
    rows, cols = [], []
    begin, end = 0, len(samples)
    for hop, fanout in enumerate(fanouts):
        for i in range(begin, end):
            node = samples[i]
            degree = int(v_degree[node])
            if degree == 0:
                continue
            if fanout >= degree:
                picks = graph.neighbor_list(node)
            else:
                drawn, picks = [], []
                for t, j in enumerate(range(degree - fanout, degree)):
                    index = draw(j, i, t, hop)
                    if index in drawn:
                        index = j
                    drawn.append(index)
                    picks.append(graph.neighbor_at(node, index))
            for v in picks:
                if v not in local:
                    local[v] = len(samples)
                    samples.append(v)
                rows.append(i)
                cols.append(local[v])
        begin, end = end, len(samples)
    return np.array(samples, np.int64), np.array(rows, np.int64), np.array(cols, np.int64)


def neighbor_sample_plain(colptr, row, seeds, fanouts, seed=0, draw=None):
    """The uncompressed form (ref: neighbor_sample_ori_impl, src/sample/csrc/neighbor_sample.h:134-212): the
    same loop on a graph without rules; returns ``(samples, neighbour local ids, frontier local ids)``."""
    nodes = colptr.size - 1
    zeros = np.zeros(nodes + 1, np.int64)
    none = np.zeros(0, np.int64)
    samples, frontier, neighbours = neighbor_sample((colptr, row), (zeros, none), (np.zeros(1, np.int64), none), [],
                                                    np.diff(colptr), none, seeds, fanouts, seed=seed, draw=draw)
    return samples, neighbours, frontier

