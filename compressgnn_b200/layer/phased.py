"""Propagation over the per-phase edge-list form of the compressed graph.

``CompressgnnData(graph_type="coo")`` hands out ``edge_index`` as a list of ``step`` tensors
``[2, E_i]`` (source row, destination row over the ``vertex_cnt + rule_cnt`` nodes) with a
matching list ``edge_weight``; the reference walks the phases with an index_select, a multiply
and a scatter-add each (``layer/CompressgnnPropagation.py:68-83``): phase 0 moves vertex features
along every edge that leaves a vertex, each later phase moves finished rule rows on.

Here every phase is grouped by destination once (a stable sort on the device, kept for as long
as the caller's edge tensor lives) and then runs through the segment-reduce kernels like any
other CSR block: no atomics, the same bits on every run.  The backward pass runs the phases in
reverse over the edges grouped by source.
"""
import torch
from torch.autograd.function import once_differentiable

from .. import runtime as _native

_phase_cache = _native._TensorKeyedCache(limit=64)


class _Phase:
    """One phase's edges as two plans: grouped by destination (forward) and by source (backward)."""

    def __init__(self, edges, weight, nodes):
        src, dst = edges[0].contiguous(), edges[1].contiguous()
        self.edges = int(src.numel())
        if self.edges == 0:
            return
        self.by_dst, self.w_by_dst = self._group(dst, src, weight, nodes)
        self.by_src, self.w_by_src = self._group(src, dst, weight, nodes)

    @staticmethod
    def _group(rows, cols, weight, nodes):
        order = torch.sort(rows, stable=True)[1]
        rowptr = torch.zeros(nodes + 1, dtype=torch.int64, device=rows.device)
        torch.cumsum(torch.bincount(rows, minlength=nodes), 0, out=rowptr[1:])
        plan = _native.SegmentPlan.from_csr(rowptr, cols[order].contiguous())
        return plan, (None if weight is None else weight[order].contiguous())


def _phases(edge_index, edge_weight, nodes):
    phases = []
    for i, edges in enumerate(edge_index):
        weight = None if edge_weight is None else edge_weight[i]
        key = (edges,) if weight is None else (edges, weight)
        phase = _phase_cache.get(key, (nodes,))
        if phase is None:
            if not (edges.is_cuda and edges.dim() == 2 and edges.size(0) == 2 and edges.dtype == torch.int64):
                raise RuntimeError("edge_index phases must be int64 CUDA tensors of shape [2, E]")
            if edges.numel() and (int(edges.min()) < 0 or int(edges.max()) >= nodes):
                raise RuntimeError("edge_index refers to a node outside vertex_cnt + rule_cnt")
            phase = _Phase(edges, weight, nodes)
            _phase_cache.put(key, phase, (nodes,))
        phases.append(phase)
    return phases


def _value(phase_weight, dtype):
    return None if phase_weight is None else phase_weight.to(dtype)


class PhasedPropagation(torch.autograd.Function):
    """``out = (sum over phases) scatter_add(weight * rows[src], dst)``, vertex rows returned."""

    @staticmethod
    def forward(ctx, x, vertex_cnt, rule_cnt, edge_index, edge_weight):
        if not x.is_cuda:
            raise RuntimeError("compressgnn_b200 runs on CUDA tensors only (no CPU propagation path)")
        nodes = int(vertex_cnt) + int(rule_cnt)
        phases = _phases(edge_index, edge_weight, nodes)
        ctx.phases, ctx.vertex_cnt, ctx.nodes = phases, int(vertex_cnt), nodes
        x = x.contiguous()
        if x.size(0) != vertex_cnt:
            raise RuntimeError("x must have one row per vertex")
        # phase 0 reads vertex rows only, so it can write the node matrix afresh
        out = torch.empty(nodes, x.size(1), dtype=x.dtype, device=x.device)
        first = phases[0] if phases else None
        if first is None or first.edges == 0:
            out.zero_()
        else:
            _native.spmm_with_plan(first.by_dst, _value(first.w_by_dst, x.dtype), x, out=out)
        for phase in phases[1:]:
            if phase.edges:  # sources are finished rule rows, destinations are rows of later phases
                _native.spmm_with_plan(phase.by_dst, _value(phase.w_by_dst, x.dtype), out, out=out, accumulate=True)
        return out[:vertex_cnt]

    @staticmethod
    @once_differentiable
    def backward(ctx, grad):
        phases, n, nodes = ctx.phases, ctx.vertex_cnt, ctx.nodes
        g = torch.zeros(nodes, grad.size(1), dtype=grad.dtype, device=grad.device)
        g[:n] = grad
        for phase in reversed(phases[1:]):
            if phase.edges:
                _native.spmm_with_plan(phase.by_src, _value(phase.w_by_src, grad.dtype), g, out=g, accumulate=True)
        first = phases[0] if phases else None
        if first is None or first.edges == 0:
            return torch.zeros(n, grad.size(1), dtype=grad.dtype, device=grad.device), None, None, None, None
        full = _native.spmm_with_plan(first.by_src, _value(first.w_by_src, grad.dtype), g)
        return full[:n], None, None, None, None


def phased_propagate(x, edge_index, edge_weight, vertex_cnt, rule_cnt):
    return PhasedPropagation.apply(x, vertex_cnt, rule_cnt, list(edge_index),
                                   None if edge_weight is None else list(edge_weight))
