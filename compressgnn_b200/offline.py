"""Host-side graph preparation: numpy front end of ``libcgnn_host.so``.

Function names, argument order and return shapes follow the reference's pybind module
``compressgnn_offline`` (``src/offline/csrc/function.cpp:25-73`` of ZhengChenCS/CompressGNN)
for the functions its CSR loader path uses, so ``loader/`` code written against the
reference reads the same here.  Index arrays are int64, weights float32.
"""
import ctypes
import operator
from pathlib import Path

import numpy as np

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "libcgnn_host.so"
_lib = None

_i64p = ctypes.POINTER(ctypes.c_int64)
_f32p = ctypes.POINTER(ctypes.c_float)


def lib():
    global _lib
    if _lib is None:
        if not LIB_PATH.is_file():
            raise ImportError(f"{LIB_PATH} is missing: build it with `python -m compressgnn_b200.build`")
        h = ctypes.CDLL(str(LIB_PATH))
        h.cgnn_host_last_error.restype = ctypes.c_char_p
        h.cgnn_host_result_count.restype = ctypes.c_int64
        h.cgnn_host_result_size.restype = ctypes.c_int64
        h.cgnn_host_result_scalar.restype = ctypes.c_int64
        h.cgnn_host_phase_count.restype = ctypes.c_int64
        h.cgnn_host_result_count.argtypes = [ctypes.c_void_p, ctypes.c_int]
        h.cgnn_host_result_size.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int]
        h.cgnn_host_result_copy.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
        h.cgnn_host_result_scalar.argtypes = [ctypes.c_void_p, ctypes.c_int]
        h.cgnn_host_result_free.argtypes = [ctypes.c_void_p]
        _lib = h
    return _lib


def _check(rc):
    if rc:
        raise ValueError(lib().cgnn_host_last_error().decode())


def _i64(a):
    """Contiguous int64 view/copy of an integer array (rejects non-integers like the
    reference's batch bridge, src/offline/bindings/batch_bridge.hpp:8-27)."""
    a = np.asarray(a)
    if a.ndim != 1 or a.dtype.kind not in "iu":
        raise ValueError("CSR arrays must be one-dimensional integer arrays")
    if a.dtype == np.uint64 and a.size and a.max() > np.iinfo(np.int64).max:
        raise ValueError("CSR value exceeds int32 range")
    return np.ascontiguousarray(a, dtype=np.int64)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


class _Result:
    def __init__(self):
        self.handle = ctypes.c_void_p(0)

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        if self.handle:
            lib().cgnn_host_result_free(self.handle)

    def arrays(self, kind):
        h, out = self.handle, []
        dtype = np.int64 if kind == 0 else np.float32
        for i in range(lib().cgnn_host_result_count(h, kind)):
            a = np.empty(lib().cgnn_host_result_size(h, kind, i), dtype=dtype)
            if a.size:
                lib().cgnn_host_result_copy(h, kind, i, _p(a))
            out.append(a)
        return out

    def scalar(self, i):
        return int(lib().cgnn_host_result_scalar(self.handle, i))


def add_self_loop_csr(vlist, elist):
    vlist, elist = _i64(vlist), _i64(elist)
    with _Result() as res:
        _check(lib().cgnn_host_add_self_loop_csr(_p(vlist), _p(elist), ctypes.c_int64(vlist.size - 1),
                                                 ctypes.byref(res.handle)))
        v, e = res.arrays(0)
    return v, e


def get_norm_degree(dst, vertex_cnt):
    dst = _i64(dst)
    out = np.empty(int(vertex_cnt), dtype=np.float32)
    _check(lib().cgnn_host_get_norm_degree(_p(dst), ctypes.c_int64(dst.size), ctypes.c_int64(vertex_cnt), _p(out)))
    return out


def gcn_norm_csr_compress(vlist, elist, norm_degree, vertex_cnt, rule_cnt):
    vlist, elist, norm_degree = _i64(vlist), _i64(elist), _f32(norm_degree)
    w = np.empty(elist.size, dtype=np.float32)
    _check(lib().cgnn_host_gcn_norm_csr_compress(_p(vlist), _p(elist), _p(norm_degree),
                                                 ctypes.c_int64(vertex_cnt), ctypes.c_int64(rule_cnt), _p(w)))
    return w


def gcn_norm_csr(vlist, elist, norm_degree, vertex_cnt):
    vlist, elist, norm_degree = _i64(vlist), _i64(elist), _f32(norm_degree)
    w = np.empty(elist.size, dtype=np.float32)
    _check(lib().cgnn_host_gcn_norm_csr(_p(vlist), _p(elist), _p(norm_degree), ctypes.c_int64(vertex_cnt), _p(w)))
    return w


def transpose_csr(vlist, elist, value, ncols):
    """Stable transpose: ``(rowptr, col, value)`` of the matrix with ``ncols`` rows."""
    vlist, elist = _i64(vlist), _i64(elist)
    value = None if value is None else _f32(value)
    tv = np.empty(int(ncols) + 1, dtype=np.int64)
    te = np.empty(elist.size, dtype=np.int64)
    tw = None if value is None else np.empty(elist.size, dtype=np.float32)
    _check(lib().cgnn_host_transpose_csr(_p(vlist), _p(elist), _p(value) if value is not None else None,
                                         ctypes.c_int64(vlist.size - 1), ctypes.c_int64(ncols), _p(tv), _p(te),
                                         _p(tw) if tw is not None else None))
    return tv, te, tw


def compress_csr_batch(vlist, elist, threads=4, rounds=12, min_pair_frequency=16):
    """``(vlist int32, elist int32, vertices, rules)``: rows ``vertices..`` are rule bodies whose
    symbols are smaller than the rule id; unfolding a vertex row gives the input row in order."""
    vlist, elist = _i64(vlist), _i64(elist)
    if vlist.size < 1 or (elist.size and (elist.max() > np.iinfo(np.int32).max or elist.min() < 0)):
        raise ValueError("CSR value exceeds int32 range")
    frequency, threads, rounds = (operator.index(min_pair_frequency), operator.index(threads),
                                  operator.index(rounds))
    with _Result() as res:
        _check(lib().cgnn_host_compress_csr_batch(_p(vlist), _p(elist), ctypes.c_int64(vlist.size - 1), threads,
                                                  rounds, frequency, ctypes.byref(res.handle)))
        v, e = res.arrays(0)
        n, r = res.scalar(0), res.scalar(1)
    return v.astype(np.int32), e.astype(np.int32), n, r


def filter_csr(vlist, elist, vertex_cnt, rule_cnt, threshold=16):
    vlist, elist = _i64(vlist), _i64(elist)
    with _Result() as res:
        _check(lib().cgnn_host_filter_csr(_p(vlist), _p(elist), ctypes.c_int64(vertex_cnt),
                                          ctypes.c_int64(rule_cnt), int(threshold), ctypes.byref(res.handle)))
        v, e = res.arrays(0)
        return v, e, res.scalar(0), res.scalar(1)


def depth_filter_csr(vlist, elist, vertex_cnt, rule_cnt, max_depth, min_edge):
    vlist, elist = _i64(vlist), _i64(elist)
    with _Result() as res:
        _check(lib().cgnn_host_depth_filter_csr(_p(vlist), _p(elist), ctypes.c_int64(vertex_cnt),
                                                ctypes.c_int64(rule_cnt), int(max_depth), int(min_edge),
                                                ctypes.byref(res.handle)))
        v, e = res.arrays(0)
        return v, e, res.scalar(0), res.scalar(1)


def hybird_partition(vlist, elist, value, vertex_cnt):
    """Four ``(rowptr, col, value)`` blocks: v2v, v2r, r2v, r2r (the reference's spelling)."""
    vlist, elist, value = _i64(vlist), _i64(elist), _f32(value)
    with _Result() as res:
        _check(lib().cgnn_host_hybrid_partition(_p(vlist), _p(elist), _p(value), ctypes.c_int64(vlist.size - 1),
                                                ctypes.c_int64(vertex_cnt), ctypes.byref(res.handle)))
        ints, vals = res.arrays(0), res.arrays(1)
    return tuple((ints[2 * b], ints[2 * b + 1], vals[b]) for b in range(4))


def topo_partition(vlist, elist, value):
    """List of per-level ``(rowptr, col, value)`` CSR blocks, each with full-height rowptr."""
    vlist, elist, value = _i64(vlist), _i64(elist), _f32(value)
    with _Result() as res:
        _check(lib().cgnn_host_topo_partition(_p(vlist), _p(elist), _p(value), ctypes.c_int64(vlist.size - 1),
                                              ctypes.byref(res.handle)))
        ints, vals = res.arrays(0), res.arrays(1)
    return [(ints[2 * l], ints[2 * l + 1], vals[l]) for l in range(len(vals))]


def gen_degree(v2v_vlist, v2v_elist, v2r_vlist, v2r_elist, r2v_vlist, r2v_elist, r2r_vlists, r2r_elists):
    v2v_vlist, v2r_vlist, v2r_elist, r2v_vlist = map(_i64, (v2v_vlist, v2r_vlist, v2r_elist, r2v_vlist))
    lv = [_i64(a) for a in r2r_vlists]
    le = [_i64(a) for a in r2r_elists]
    n, r = v2v_vlist.size - 1, r2v_vlist.size - 1
    vd, rd = np.empty(n, dtype=np.int64), np.empty(r, dtype=np.int64)
    arr_t = ctypes.c_void_p * max(len(lv), 1)
    pv = arr_t(*[a.ctypes.data for a in lv])
    pe = arr_t(*[a.ctypes.data for a in le])
    _check(lib().cgnn_host_gen_degree(_p(v2v_vlist), _p(v2r_vlist), _p(v2r_elist), _p(r2v_vlist),
                                      ctypes.c_int64(n), ctypes.c_int64(r), len(lv), pv, pe, _p(vd), _p(rd)))
    return vd, rd


def phase_count(vlist, elist, vertex_cnt, rule_cnt):
    """The ``step`` the reference's CSR loader records (``gen_mask_vertex(..., "csc")[1]``)."""
    vlist, elist = _i64(vlist), _i64(elist)
    return int(lib().cgnn_host_phase_count(_p(vlist), _p(elist), ctypes.c_int64(vertex_cnt),
                                           ctypes.c_int64(rule_cnt)))


def generate_copy_graph(n, alpha=2.1, x_min=4.0, max_degree=10000, copy_prob=0.7, window=64, candidates=1,
                        seed=2):
    """Seeded directed copying-model web graph as CSR ``(vlist, elist)``."""
    with _Result() as res:
        _check(lib().cgnn_host_generate_copy_graph(ctypes.c_int64(n), ctypes.c_double(alpha), ctypes.c_double(x_min),
                                                   ctypes.c_int64(max_degree), ctypes.c_double(copy_prob),
                                                   ctypes.c_int64(window), int(candidates), ctypes.c_uint64(seed),
                                                   ctypes.byref(res.handle)))
        v, e = res.arrays(0)
    return v, e


def generate_pa_graph(n, undirected_edges, copy_frac=0.3, seed=1):
    """Seeded undirected preferential-attachment graph with list copying, symmetric CSR."""
    with _Result() as res:
        _check(lib().cgnn_host_generate_pa_graph(ctypes.c_int64(n), ctypes.c_int64(undirected_edges),
                                                 ctypes.c_double(copy_frac), ctypes.c_uint64(seed),
                                                 ctypes.byref(res.handle)))
        v, e = res.arrays(0)
    return v, e
