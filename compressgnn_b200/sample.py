"""Neighbour sampling on the compressed graph (ref: ``src/sample/csrc/neighbor_sample.h:27-131``, bound in
the reference as ``compressgnn_sample.neighbor_sample_cg_sim``; host code there, CUDA here).

``neighbor_sample_cg_sim`` keeps the reference's argument list and result: ``(samples, rows, cols)`` --
``samples`` holds the seeds followed by every newly reached node in the order it is first seen, and sampled
edge ``e`` joins the frontier node with local id ``rows[e]`` to its neighbour with local id ``cols[e]``.
Per hop, a node with at most ``num_neighbors[hop]`` neighbours contributes all of them in list order, any
other node that many distinct ones (Floyd's scheme, as in the reference).  The random neighbour indices
come from a counter-based generator on the device under ``seed`` (drawn from torch's host generator when
not given), not from ``torch::randint`` calls on the host, so equal seeds give equal samples.
"""
import ctypes

import torch

from ._lib import check, lib
from .runtime import _ptr, _require, _stream_ptr, on_device

_NONE = 2 ** 31 - 1


class _GraphStruct(ctypes.Structure):
    _fields_ = [(name, ctypes.c_void_p) for name in
                ("v2v_ptr", "v2v_col", "v2r_ptr", "v2r_col", "r2v_ptr", "r2v_col", "r2r_ptr", "r2r_col",
                 "vertex_degree", "rule_degree")] + [("vertices", ctypes.c_int64), ("rules", ctypes.c_int64)]


def merge_rule_levels(r2r_vlist, r2r_elist, rules, device):
    """One rule -> rule CSR out of the per-level blocks (each ``[rules + 1]`` row pointers): a rule's
    children sit in exactly one level, so the merged row is that level's row."""
    rowptr = torch.zeros(rules + 1, dtype=torch.int64, device=device)
    if not r2r_vlist:
        return rowptr, torch.empty(0, dtype=torch.int64, device=device)
    lengths = sum(torch.diff(v.to(device)) for v in r2r_vlist)
    torch.cumsum(lengths, 0, out=rowptr[1:])
    rows = torch.cat([torch.repeat_interleave(torch.arange(rules, device=device), torch.diff(v.to(device)))
                      for v in r2r_vlist])
    cols = torch.cat([e.to(device) for e in r2r_elist])
    order = torch.sort(rows, stable=True).indices
    return rowptr, cols[order].contiguous()


def exact_degrees(v2v_vlist, v2r_vlist, v2r_elist, r2v_vlist, r2r_vlist, r2r_elist):
    """``(vertex_degree, rule_degree)`` with the level blocks taken first to last, the order in which
    ``topo_partition`` emits them (a child's size is final before its parents add it).  The reference's
    ``gen_degree`` (``src/offline/csrc/gen_degree.h:62-72``), which ``CompressGraph.vertex_degree`` follows,
    walks them last to first and comes out short below rules nested more than one level deep."""
    device = v2v_vlist.device
    r_degree = torch.diff(r2v_vlist).to(torch.int64)
    rules = r_degree.numel()
    for ptr, col in zip(r2r_vlist, r2r_elist):
        ptr, col = ptr.to(device), col.to(device)
        rows = torch.repeat_interleave(torch.arange(rules, device=device), torch.diff(ptr))
        r_degree = r_degree.index_add(0, rows, r_degree[col])
    v_degree = torch.diff(v2v_vlist).to(torch.int64)
    rows = torch.repeat_interleave(torch.arange(v_degree.numel(), device=device), torch.diff(v2r_vlist))
    return v_degree.index_add(0, rows, r_degree[v2r_elist]), r_degree


class CompressGraphSampler:
    """Sampler bound to one compressed graph on one CUDA device; ``sampler(input_node, num_neighbors)``.

    The object owns two per-vertex tables that a call fills and clears again, so calls on one sampler must
    not overlap (one call at a time; use one sampler per stream or worker).  A fan-out of 0 or less samples
    nothing at that hop, as in the reference."""

    def __init__(self, v2v_vlist, v2v_elist, v2r_vlist, v2r_elist, r2v_vlist, r2v_elist, r2r_vlist, r2r_elist,
                 v_degree, r_degree):
        device = v2v_vlist.device
        _require(device.type == "cuda", "the sampler needs the graph on a CUDA device (no CPU path)")
        as_i64 = lambda t: t.to(device=device, dtype=torch.int64).contiguous()
        self.device = device
        self.vertices, self.rules = v2v_vlist.numel() - 1, r2v_vlist.numel() - 1
        merged = merge_rule_levels(list(r2r_vlist), list(r2r_elist), self.rules, device)
        self._arrays = [as_i64(t) for t in (v2v_vlist, v2v_elist, v2r_vlist, v2r_elist, r2v_vlist, r2v_elist,
                                            merged[0], merged[1], v_degree, r_degree)]
        _require(self._arrays[8].numel() == self.vertices and self._arrays[9].numel() == self.rules,
                 "degree arrays do not match the graph")
        self._graph = _GraphStruct(*[t.data_ptr() if t.numel() else None for t in self._arrays],
                                   self.vertices, self.rules)
        self._local_of = torch.full((self.vertices,), _NONE, dtype=torch.int32, device=device)
        self._first = torch.full((self.vertices,), _NONE, dtype=torch.int32, device=device)

    @classmethod
    def from_graph(cls, graph):
        """From a ``CompressGraph`` that has been moved to the GPU."""
        blocks = [graph.v2v_graph, graph.v2r_graph, graph.r2v_graph]
        flat = [t for b in blocks for t in b.csr()[:2]]
        level_ptr = [lvl.csr()[0] for lvl in graph.r2r_graph]
        level_col = [lvl.csr()[1] for lvl in graph.r2r_graph]
        degrees = exact_degrees(flat[0], flat[2], flat[3], flat[4], level_ptr, level_col)
        return cls(*flat, level_ptr, level_col, *degrees)

    def __call__(self, input_node, num_neighbors, seed=None):
        device = self.device
        seeds = torch.as_tensor(input_node, dtype=torch.int64).to(device).contiguous()
        _require(seeds.dim() == 1, "input_node must be one-dimensional")
        if seed is None:
            seed = int(torch.randint(0, 2 ** 63 - 1, (1,), dtype=torch.int64).item())
        g = ctypes.byref(self._graph)
        rows, cols = [], []
        samples = seeds.clone()
        begin, end = 0, seeds.numel()
        with on_device(device):
            stream = _stream_ptr(device)
            local_of, first = self._local_of, self._first
            try:
                check(lib().cgnn_sample_seed(_ptr(samples), end, self.vertices, _ptr(local_of), stream))
                for hop, fanout in enumerate(num_neighbors):
                    frontier = end - begin
                    if frontier == 0:
                        break
                    count = torch.empty(frontier, dtype=torch.int64, device=device)
                    check(lib().cgnn_sample_count(g, _ptr(samples), begin, frontier, int(fanout), _ptr(count), stream))
                    inclusive = torch.cumsum(count, 0)
                    total = int(inclusive[-1].item())
                    if total == 0:
                        begin = end
                        continue
                    offset = inclusive - count
                    picked = torch.empty(total, dtype=torch.int64, device=device)
                    source = torch.empty(total, dtype=torch.int64, device=device)
                    scratch = torch.empty(total, dtype=torch.int64, device=device)
                    check(lib().cgnn_sample_pick(g, _ptr(samples), begin, frontier, int(fanout), _ptr(count), _ptr(offset),
                                                 hop, ctypes.c_uint64(seed), _ptr(picked), _ptr(source), _ptr(scratch),
                                                 stream))
                    is_new = scratch  # the scratch of the picks is free again
                    check(lib().cgnn_sample_claim(_ptr(picked), total, self.vertices, _ptr(local_of), _ptr(first),
                                                  _ptr(is_new), stream))
                    inclusive = torch.cumsum(is_new, 0)
                    fresh = int(inclusive[-1].item())
                    rank = inclusive - is_new
                    grown = torch.empty(end + fresh, dtype=torch.int64, device=device)
                    grown[:end] = samples
                    target = torch.empty(total, dtype=torch.int64, device=device)
                    check(lib().cgnn_sample_relabel(_ptr(picked), total, self.vertices, _ptr(is_new), _ptr(rank), end,
                                                    _ptr(local_of), _ptr(first), _ptr(target), _ptr(grown), stream))
                    samples = grown
                    rows.append(source)
                    cols.append(target)
                    begin, end = end, end + fresh
            except BaseException:
                local_of.fill_(_NONE)  # a hop that stopped half way may have left claims behind
                first.fill_(_NONE)
                raise
            # the table goes back to "nothing seen" for the next call: only the entries this call set
            inside = samples[(samples >= 0) & (samples < self.vertices)]
            local_of[inside] = _NONE
        empty = torch.empty(0, dtype=torch.int64, device=device)
        return samples, (torch.cat(rows) if rows else empty), (torch.cat(cols) if cols else empty)


def neighbor_sample_cg_sim(v2v_vlist, v2v_elist, v2r_vlist, v2r_elist, r2v_vlist, r2v_elist, r2r_vlist, r2r_elist,
                           v_degree, r_degree, input_node, num_neighbors, seed=None):
    """The reference's entry point (same positional arguments, CUDA tensors): ``(output_node, row, col)``."""
    sampler = CompressGraphSampler(v2v_vlist, v2v_elist, v2r_vlist, v2r_elist, r2v_vlist, r2v_elist, r2r_vlist,
                                   r2r_elist, v_degree, r_degree)
    return sampler(input_node, num_neighbors, seed=seed)


def neighbor_sample_ori_impl(colptr, row, input_node, num_neighbors, seed=None):
    """The reference's sampler for an uncompressed graph in CSC form (``neighbor_sample_ori_impl``,
    ``src/sample/csrc/neighbor_sample.h:134-212``): the same hops on a graph without rules.  As there,
    the second result holds the local ids of the sampled neighbours and the third those of the frontier nodes."""
    device = colptr.device
    nodes = colptr.numel() - 1
    none = torch.zeros(1, dtype=torch.int64, device=device)
    empty = torch.empty(0, dtype=torch.int64, device=device)
    degree = torch.diff(colptr.to(torch.int64))
    sampler = CompressGraphSampler(colptr, row, torch.zeros(nodes + 1, dtype=torch.int64, device=device), empty,
                                   none, empty, [], [], degree, empty)
    samples, frontier, neighbours = sampler(input_node, num_neighbors, seed=seed)
    return samples, neighbours, frontier

