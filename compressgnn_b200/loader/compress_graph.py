"""``CompressGraph``: the on-device compressed graph the propagation operator consumes.

Same attributes as the reference's ``loader/compress_graph.py:6-57``: ``v2v_graph [N x N]``,
``v2r_graph [N x R]``, ``r2v_graph [R x N]``, ``r2r_graph`` (a list of ``step`` level blocks,
each ``[R x R]`` with full-height row pointers), ``step``, ``vertex_degree``, ``rule_degree``
and ``.to(device)``.  The blocks are ``SparseBlock`` objects (``.csr()`` / ``.csc()``).

On a CUDA device the graph also owns the launch plans of the fused propagation (built on
first use): one plan per block of the forward and of the transposed backward, with the last
two blocks of each direction fused into one pass.
"""
import numpy as np
import torch

from .. import offline
from .sparse_block import SparseBlock


class PropagationPlan:
    """Plans for forward (A_hat^T x) and backward (A_hat g) on one device."""

    def __init__(self, graph):
        from ..runtime import SegmentPlan
        g = graph
        self.device = g.v2v_graph.device
        # forward: rules <- vertices, rule levels, vertices <- rules + vertices
        self.r2v = SegmentPlan.from_csr(*g.r2v_graph.csr()[:2])
        self.levels = [SegmentPlan.from_csr(*lvl.csr()[:2]) for lvl in g.r2r_graph]
        self.out = SegmentPlan.from_csr(*g.v2r_graph.csr()[:2], *g.v2v_graph.csr()[:2])
        # backward: the transposed blocks, levels last to first
        self.v2r_t = SegmentPlan.from_csr(*g.v2r_graph.csc()[:2])
        self.levels_t = [SegmentPlan.from_csr(*lvl.csc()[:2]) for lvl in g.r2r_graph]
        self.out_t = SegmentPlan.from_csr(*g.v2v_graph.csc()[:2], *g.r2v_graph.csc()[:2])
        self._graph = g
        self._passes = {}

    def whole_pass(self, backward, width, dtype):
        """The launch table of one direction as ``cgnn_propagate`` takes it (plans, values in plan
        order, scratch), built once per (direction, width, dtype, stream) and then reused: a pass is
        one native call."""
        import ctypes
        from ..runtime import _dtype_code_of, _stream_ptr
        stream = _stream_ptr(self.device)
        key = (bool(backward), int(width), dtype, stream)
        table = self._passes.get(key)
        if table is None:
            g = self._graph
            if backward:
                plans = [self.v2r_t] + list(reversed(self.levels_t)) + [self.out_t]
                values = [g.v2r_graph.value_as(dtype, True)] + \
                         [lvl.value_as(dtype, True) for lvl in reversed(g.r2r_graph)]
                last = (g.v2v_graph.value_as(dtype, True), g.r2v_graph.value_as(dtype, True))
            else:
                plans = [self.r2v] + list(self.levels) + [self.out]
                values = [g.r2v_graph.value_as(dtype)] + [lvl.value_as(dtype) for lvl in g.r2r_graph]
                last = (g.v2r_graph.value_as(dtype), g.v2v_graph.value_as(dtype))
            code = _dtype_code_of(dtype)
            ordered = [p.values(v) for p, v in zip(plans[:-1], values)] + [plans[-1].values(*last)]
            scratch = [p.scratch(width, code) for p in plans]
            n = len(plans)
            table = dict(
                n=n, code=code, keep=(plans, ordered),  # the tensors behind the raw pointers stay alive here
                plans=(ctypes.c_void_p * n)(*[p.handle.value for p in plans]),
                vals=(ctypes.c_void_p * n)(*[t.data_ptr() if t.numel() else None for t in ordered]),
                scratch=(ctypes.c_void_p * n)(*[s[0].value for s in scratch]),
                scratch_bytes=(ctypes.c_size_t * n)(*[s[1] for s in scratch]),
                rule_term=1 if backward else 0, stream=stream,
                source_rows=(plans[0].source_rows[0], plans[-1].source_rows))
            self._passes[key] = table
        return table


class CompressGraph:
    def __init__(self, vlist, elist, value, vertex_cnt):
        """``(vlist, elist, value)`` is the *transposed* weighted compressed graph in CSR (rows
        and columns ``>= vertex_cnt`` are rules), as ``CompressgnnData`` hands it over
        (ref: loader/CompressgnnData.py:169-182)."""
        vlist, elist, value = (np.asarray(torch.as_tensor(a).cpu()) for a in (vlist, elist, value))
        v2v, v2r, r2v, r2r = offline.hybird_partition(vlist, elist, value, vertex_cnt)
        levels = offline.topo_partition(*r2r)
        rule_cnt = r2v[0].size - 1
        mk = lambda blk, sizes: SparseBlock(torch.from_numpy(blk[0]), torch.from_numpy(blk[1]),
                                            torch.from_numpy(blk[2]), sparse_sizes=sizes)
        self.v2v_graph = mk(v2v, (vertex_cnt, vertex_cnt))
        self.v2r_graph = mk(v2r, (vertex_cnt, rule_cnt))
        self.r2v_graph = mk(r2v, (rule_cnt, vertex_cnt))
        self.step = len(levels)
        self.r2r_graph = [mk(lvl, (rule_cnt, rule_cnt)) for lvl in levels]
        vdeg, rdeg = offline.gen_degree(v2v[0], v2v[1], v2r[0], v2r[1], r2v[0], r2v[1],
                                        [lvl[0] for lvl in levels], [lvl[1] for lvl in levels])
        self.vertex_degree = torch.from_numpy(vdeg)
        self.rule_degree = torch.from_numpy(rdeg)
        self.vertex_cnt, self.rule_cnt = int(vertex_cnt), int(rule_cnt)
        self._plan = None

    def __repr__(self):
        return "CompressGraph"

    def to(self, device):
        self.v2v_graph = self.v2v_graph.to(device)
        self.v2r_graph = self.v2r_graph.to(device)
        self.r2v_graph = self.r2v_graph.to(device)
        self.r2r_graph = [lvl.to(device) for lvl in self.r2r_graph]
        self.vertex_degree = self.vertex_degree.to(device)
        self.rule_degree = self.rule_degree.to(device)
        self._plan = None
        self._sampler = None
        return self

    def blocks(self):
        return [self.v2v_graph, self.v2r_graph, self.r2v_graph] + list(self.r2r_graph)

    def edge_count(self):
        return sum(b.nnz() for b in self.blocks())

    def neighbor_sampler(self):
        """The neighbour sampler of this graph on its CUDA device (``compressgnn_b200.sample``), built on
        first use: merged rule table, exact degrees, per-vertex tables."""
        if getattr(self, "_sampler", None) is None or self._sampler.device != self.v2v_graph.device:
            from ..sample import CompressGraphSampler
            self._sampler = CompressGraphSampler.from_graph(self)
        return self._sampler

    def propagation_plan(self):
        if self._plan is None:
            if not self.v2v_graph.device.type == "cuda":
                raise RuntimeError("CompressGraph: move the graph to a CUDA device first; "
                                   "compressgnn_b200 has no CPU propagation path")
            self._plan = PropagationPlan(self)
        return self._plan
