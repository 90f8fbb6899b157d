"""Compressed propagation for feature matrices that live in host memory.

The reference runs ``Compressgnn_SPMM`` on the CPU when it is handed CPU tensors
(``layer/CompressgnnSPMM.py:41-53``).  Here a host matrix is propagated on the GPU instead, and
because one pass over a resident matrix takes far less time than moving the matrix over PCIe,
the cost of such a call is the two copies.  ``HostPropagation`` therefore queues passes on three
streams -- upload, propagate, download -- over a small ring of device buffers, so that the
download of one pass and the upload of the next share the link in both directions.  A call
returns as soon as its work is queued; the event it returns (or ``synchronize()``) tells when
the host result is complete.
"""
import torch

from .. import runtime as _native
from . import spmm as _spmm


class HostPropagation:
    """Queue forward / backward propagation passes whose operands are pinned host tensors.

    ``graph``: a ``CompressGraph`` already moved to the GPU; ``width``: feature columns;
    ``depth``: device buffer sets in the ring (2 keeps both copy directions busy).
    Device memory held: ``depth * (2 * vertices + rules) * width`` elements.
    """

    def __init__(self, graph, width, dtype=torch.float32, depth=2):
        device = torch.device(graph.v2v_graph.device)
        if device.type != "cuda":
            raise RuntimeError("HostPropagation needs the graph on a CUDA device (graph.to(device))")
        if depth < 1:
            raise RuntimeError("depth must be at least 1")
        self.graph, self.width, self.dtype, self.device, self.depth = graph, int(width), dtype, device, int(depth)
        rows = graph.vertex_cnt
        self._in = [torch.empty(rows, self.width, dtype=dtype, device=device) for _ in range(depth)]
        self._rule = [_native.empty_row_aligned(graph.rule_cnt, buf) for buf in self._in]
        self._out = [torch.empty(rows, self.width, dtype=dtype, device=device) for _ in range(depth)]
        self._up, self._run, self._down = (torch.cuda.Stream(device) for _ in range(3))
        self._consumed = [None] * depth  # propagate stream is done reading _in[slot] / _rule[slot]
        self._drained = [None] * depth   # download stream is done reading _out[slot]
        self._queued = 0
        graph.propagation_plan()
        # whatever prepared the graph on the caller's stream is ordered before the first pass
        self._run.wait_stream(torch.cuda.current_stream(device))

    def _check(self, host, what):
        if host.is_cuda or host.shape != (self.graph.vertex_cnt, self.width) or host.dtype != self.dtype:
            raise RuntimeError(f"{what} must be a host [{self.graph.vertex_cnt}, {self.width}] {self.dtype} tensor")
        if not host.is_contiguous():
            raise RuntimeError(f"{what} must be contiguous")

    def _submit(self, one_pass, source, result):
        self._check(source, "source")
        self._check(result, "result")
        slot = self._queued % self.depth
        self._queued += 1
        with torch.cuda.stream(self._up):
            if self._consumed[slot] is not None:
                self._up.wait_event(self._consumed[slot])
            self._in[slot].copy_(source, non_blocking=True)
            uploaded = torch.cuda.Event()
            uploaded.record(self._up)
        with torch.cuda.stream(self._run):
            self._run.wait_event(uploaded)
            if self._drained[slot] is not None:
                self._run.wait_event(self._drained[slot])
            one_pass(self.graph, self._in[slot], out=self._out[slot], rule_out=self._rule[slot])
            self._consumed[slot] = torch.cuda.Event()
            self._consumed[slot].record(self._run)
        with torch.cuda.stream(self._down):
            self._down.wait_event(self._consumed[slot])
            result.copy_(self._out[slot], non_blocking=True)
            self._drained[slot] = torch.cuda.Event()
            self._drained[slot].record(self._down)
        return self._drained[slot]

    def forward(self, x_host, out_host):
        """Queue ``out_host = propagate(x_host)``; returns the event that marks ``out_host`` complete.
        ``x_host`` must stay unmodified until then."""
        return self._submit(_spmm._forward, x_host, out_host)

    def backward(self, grad_host, grad_in_host):
        """Queue the transposed pass ``grad_in_host = propagate^T(grad_host)``."""
        return self._submit(_spmm._backward, grad_host, grad_in_host)

    def synchronize(self):
        """Block until every queued pass has delivered its host result; raises if a kernel
        recorded a problem (bad index, a staged copy that never arrived) along the way."""
        self._down.synchronize()
        _native.raise_on_device_status()
