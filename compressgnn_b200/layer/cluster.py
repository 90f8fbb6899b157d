"""LSH bucket representatives with an assignment that is reused across epochs.

Public surface of the reference's ``layer/CompressgnnCluster.py`` (``_Mean`` :28-38,
``Compressgnn_Cluster_Function`` :53-66, ``Compressgnn_Cluster`` :69-187): the constructor
``Compressgnn_Cluster(in_feature, param_H, training=True, device=None, dtype=None, cache=True,
index_cache=False, refresh_interval=1, refresh_policy='fixed', q_min=1, q_max=10,
tau_loss=None)``, ``set_epoch``, ``reset_cache``, ``forward(input, epoch=None, cache_key=None,
force_refresh=False)`` and the attributes ``vertex_index``, ``active_bucket``,
``last_refreshed``, ``refresh_count``, ``current_interval``.

The module is put together from three parts:

``RefreshSchedule``   how many epochs an assignment may be kept (a fixed interval, or one
                      that follows the change of the training loss);
``AssignmentCache``   the kept assignments, one per (train/eval mode, device, stream), each
                      tagged with what it was computed for;
``Compressgnn_Cluster``  wires the two to the native assignment and to ``_Mean``.

Only the assignment (index, counts) is ever kept.  The representatives are recomputed from the
current features on every call, so gradients always reach the current upstream model.

One argument the reference does not have: ``process_group``.  With feature columns sharded
across GPUs every rank holds ``[N, F/G]`` features and its ``[F/G, H]`` slice of the hyperplanes;
the partial projections are summed with one all-reduce before sign packing, so all ranks derive
the same assignment.
"""
import math
import operator
from dataclasses import dataclass
from typing import Any, Optional, Tuple

import torch
from torch.autograd.function import once_differentiable

from .. import runtime as _native


def _require_cuda(x):
    if not x.is_cuda:
        raise RuntimeError("compressgnn_b200 runs on CUDA tensors only (no CPU cluster path)")


# ---------------------------------------------------------------------------------------------
# autograd functions
# ---------------------------------------------------------------------------------------------
class _Mean(torch.autograd.Function):
    """``reps[g] = mean of the rows of x whose index is g``; first-order gradient only."""

    @staticmethod
    def forward(ctx, x, index, counts):
        _require_cuda(x)
        ctx.save_for_backward(index, counts)
        return _native.cluster_mean(x.contiguous(), index, counts)

    @staticmethod
    @once_differentiable
    def backward(ctx, grad):
        index, counts = ctx.saved_tensors
        return _native.cluster_mean_backward(grad.contiguous(), index, counts), None, None


def _assign(input, planes, bits, workspace=None, process_group=None):
    """``(index int64[N], counts int32[active+1], active)`` for the current features."""
    _require_cuda(input)
    with torch.no_grad():
        input, planes = input.contiguous(), planes.contiguous()
        if workspace is None:
            workspace = _native.cluster_workspace(input, bits)
        if process_group is None:
            return _native.cluster_assign(input, planes, bits, workspace)
        from ..dist import allreduce_projection
        partial = allreduce_projection(_native.project(input, planes), process_group)
        return _native.cluster_assign_from_projection(partial, workspace)


class Compressgnn_Cluster_Function(torch.autograd.Function):
    """Assignment and mean in one uncached call (the reference's older entry point)."""

    @staticmethod
    def forward(ctx, input, random_vectors, param_H, is_training):
        index, counts, active = _assign(input, random_vectors, param_H)
        ctx.save_for_backward(index, counts)
        ctx.mark_non_differentiable(index)
        return _native.cluster_mean(input.contiguous(), index, counts), index, active

    @staticmethod
    @once_differentiable
    def backward(ctx, grad, _index_grad, _active_grad):
        index, counts = ctx.saved_tensors
        return _native.cluster_mean_backward(grad.contiguous(), index, counts), None, None, None


# ---------------------------------------------------------------------------------------------
# refresh schedule
# ---------------------------------------------------------------------------------------------
class RefreshSchedule:
    """Epoch clock plus the number of epochs an assignment stays valid.

    ``policy='fixed'``: always ``interval`` epochs.  ``policy='loss'``: after every reported
    loss the interval becomes ``q_min + (q_max - q_min) * exp(-|loss - previous| / tau)``
    rounded half up and clamped to ``[q_min, q_max]`` -- a loss that has stopped moving keeps
    the assignment for ``q_max`` epochs, a jumping loss recomputes it every ``q_min`` epochs.
    """

    def __init__(self, policy, interval, q_min, q_max, tau):
        if policy not in ('fixed', 'loss'):
            raise ValueError("refresh_policy: expected 'fixed' or 'loss', got {!r}".format(policy))
        if interval < 1:
            raise ValueError("refresh_interval counts epochs and must be at least 1")
        if not 1 <= q_min <= q_max:
            raise ValueError("the adaptive interval needs 1 <= q_min <= q_max")
        if policy == 'loss' and not (tau is not None and math.isfinite(tau) and tau > 0):
            raise ValueError("refresh_policy='loss' needs tau_loss > 0 (finite)")
        self.policy, self.fixed_interval = policy, interval
        self.q_min, self.q_max, self.tau = q_min, q_max, tau
        self.restart()

    @property
    def needs_epoch(self):
        """True when reuse across epochs is possible, i.e. the caller has to say which epoch it is."""
        return self.policy == 'loss' or self.fixed_interval > 1

    def restart(self):
        """Forget the clock and the loss history (a new run, or freshly loaded weights)."""
        self.epoch = None
        self.interval = self.fixed_interval if self.policy == 'fixed' else self.q_min
        self._loss_before = None
        self._loss_epoch = None

    def advance(self, epoch, loss=None):
        """Move the clock to ``epoch``.  Returns True when the clock went backwards, which starts
        a new run.  ``loss`` (a host number: the last finished training loss) feeds the adaptive
        interval once per epoch."""
        epoch = operator.index(epoch)
        if epoch < 0:
            raise ValueError("epochs are counted from zero")
        rewound = self.epoch is not None and epoch < self.epoch
        if rewound:
            self.restart()
        self.epoch = epoch
        if loss is None or self.policy != 'loss' or epoch == self._loss_epoch:
            return rewound
        if torch.is_tensor(loss):
            raise TypeError("set_epoch takes the loss as a Python number; reading a device tensor "
                            "here would stall the stream once per epoch")
        loss = float(loss)
        if not math.isfinite(loss):
            raise ValueError("the reported loss is not finite")
        if self._loss_before is not None:
            decay = math.exp(-abs(loss - self._loss_before) / self.tau)
            wanted = math.floor(self.q_min + (self.q_max - self.q_min) * decay + 0.5)
            self.interval = int(min(self.q_max, max(self.q_min, wanted)))
        self._loss_before, self._loss_epoch = loss, epoch
        return rewound

    def expired(self, computed_at):
        """Has an assignment computed at epoch ``computed_at`` outlived the current interval?"""
        return self.epoch - computed_at >= self.interval


# ---------------------------------------------------------------------------------------------
# assignment cache
# ---------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class AssignmentSignature:
    """Everything an assignment depends on besides the feature values themselves."""
    shape: Tuple[int, ...]
    dtype: torch.dtype
    cache_key: Any              # the caller's name for the node order (e.g. which graph / batch)
    planes_ptr: int             # the hyperplane buffer ...
    planes_version: int         # ... and its in-place modification counter


@dataclass
class Assignment:
    index: torch.Tensor         # int64[N], 1-based compact bucket ids
    counts: torch.Tensor        # int32[active + 1], counts[0] == 0
    active: int
    signature: AssignmentSignature
    epoch: Optional[int]


class AssignmentCache:
    """One kept ``Assignment`` per (train/eval mode, device, stream)."""

    def __init__(self):
        self._slots = {}

    def clear(self):
        self._slots.clear()

    def lookup(self, slot, signature):
        kept = self._slots.get(slot)
        return kept if kept is not None and kept.signature == signature else None

    def keep(self, slot, assignment):
        self._slots[slot] = assignment


# ---------------------------------------------------------------------------------------------
# the module
# ---------------------------------------------------------------------------------------------
class Compressgnn_Cluster(torch.nn.Module):
    """Mean representatives over LSH buckets.

    ``refresh_interval`` counts epochs, never calls: with an interval above one (or the loss
    policy) the zero-based epoch has to come in through ``set_epoch`` or ``forward(epoch=...)``.
    Constructed with ``training=False`` the module returns the representatives alone (the older
    contract); otherwise ``forward`` returns ``(reps, index)`` in ``train()`` and in ``eval()``,
    which keep separate assignments.
    """

    def __init__(self, in_feature, param_H, training=True, device=None, dtype=None, cache=True,
                 index_cache=False, refresh_interval=1, refresh_policy='fixed', q_min=1, q_max=10,
                 tau_loss=None, process_group=None):
        super().__init__()
        self.in_feature = operator.index(in_feature)
        self.param_H = operator.index(param_H)
        if self.in_feature < 0:
            raise ValueError("in_feature must not be negative")
        if not 0 <= self.param_H <= 30:
            raise ValueError("param_H (hyperplanes, one bit each) must lie in 0..30")
        self._schedule = RefreshSchedule(refresh_policy, operator.index(refresh_interval),
                                         operator.index(q_min), operator.index(q_max), tau_loss)
        self.cache, self.index_cache = bool(cache), bool(index_cache)
        self.is_training = bool(training)   # selects the return contract, not the cache slot
        self.process_group = process_group
        self.register_buffer('random_vectors',
                             torch.randn(self.in_feature, self.param_H, device=device, dtype=dtype))
        self._kept = AssignmentCache()
        self._workspaces = {}
        self.vertex_index = self.active_bucket = None
        self.last_refreshed = False
        self.refresh_count = 0
        self.train(training)

    # -- configuration, readable under the reference's attribute names -------------------------
    refresh_policy = property(lambda self: self._schedule.policy)
    refresh_interval = property(lambda self: self._schedule.fixed_interval)
    q_min = property(lambda self: self._schedule.q_min)
    q_max = property(lambda self: self._schedule.q_max)
    tau_loss = property(lambda self: self._schedule.tau)
    current_interval = property(lambda self: self._schedule.interval)

    # -- epoch clock and invalidation ---------------------------------------------------------
    def set_epoch(self, epoch, loss=None):
        """Zero-based epoch; ``loss`` is the previous finished training loss as a host number."""
        if self._schedule.advance(epoch, loss):
            self.reset_cache()
        return self

    def reset_cache(self):
        self._kept.clear()
        self.vertex_index = self.active_bucket = None
        self.last_refreshed = False

    def _apply(self, fn, *args, **kwargs):
        # .to() / .cuda() / .double(): buffers move, so kept assignments and workspaces are stale
        self.reset_cache()
        self._workspaces.clear()
        return super()._apply(fn, *args, **kwargs)

    def _load_from_state_dict(self, *args, **kwargs):
        self.reset_cache()
        self._schedule.restart()
        return super()._load_from_state_dict(*args, **kwargs)

    # -- forward -----------------------------------------------------------------------------
    def _check_input(self, input):
        if input.dim() != 2 or input.size(1) != self.in_feature:
            raise ValueError("input must be [nodes, {}], got {}".format(self.in_feature, tuple(input.shape)))
        planes = self.random_vectors
        if input.device != planes.device or input.dtype != planes.dtype:
            raise ValueError("input is {} on {} but the module holds {} on {}; move the module first".format(
                input.dtype, input.device, planes.dtype, planes.device))
        if input.dtype not in (torch.float32, torch.float64):
            raise ValueError("float32 and float64 are the supported feature types")

    def _workspace(self, input, stream):
        key = (input.device, stream, self.param_H)
        ws = self._workspaces.get(key)
        need = _native.lib().cgnn_cluster_workspace_bytes(int(input.size(0)), self.param_H)
        if ws is None or ws[2].numel() < need:  # sized by rows: grow when a larger input arrives
            ws = self._workspaces[key] = _native.cluster_workspace(input, self.param_H)
        return ws

    def _compute(self, input, stream, signature):
        if input.size(0) == 0:
            index = torch.empty(0, device=input.device, dtype=torch.int64)
            counts = torch.zeros(1, device=input.device, dtype=torch.int32)
            active = 0
        else:
            index, counts, active = _assign(input, self.random_vectors, self.param_H,
                                            self._workspace(input.contiguous(), stream), self.process_group)
        return Assignment(index, counts, active, signature, self._schedule.epoch)

    def forward(self, input, epoch=None, cache_key=None, force_refresh=False):
        kept = self.assignment(input, epoch=epoch, cache_key=cache_key, force_refresh=force_refresh)
        reps = _Mean.apply(input, kept.index, kept.counts)
        return (reps, kept.index) if self.is_training else reps

    def assignment(self, input, epoch=None, cache_key=None, force_refresh=False):
        """The bucket assignment ``forward`` would use for ``input`` now (kept or recomputed, by the same
        rules), without the means: ``.index`` int64[N], ``.counts`` int32[active + 1], ``.active``."""
        self._check_input(input)
        if epoch is not None:
            self.set_epoch(epoch)
        clock = self._schedule
        if self.cache and clock.epoch is None and clock.needs_epoch:
            raise ValueError("reuse across epochs needs the epoch: call set_epoch(epoch) or pass epoch=")
        _require_cuda(input)
        stream = torch.cuda.current_stream(input.device).cuda_stream
        slot = (self.training, input.device, stream)
        signature = AssignmentSignature(tuple(input.shape), input.dtype, cache_key,
                                        self.random_vectors.data_ptr(), self.random_vectors._version)
        kept = None
        if self.cache and not force_refresh and clock.epoch is not None:
            kept = self._kept.lookup(slot, signature)
            if kept is not None and clock.expired(kept.epoch):
                kept = None
        self.last_refreshed = kept is None
        if kept is None:
            kept = self._compute(input, stream, signature)
            self.refresh_count += 1
            if self.cache and clock.epoch is not None:
                self._kept.keep(slot, kept)
        self.vertex_index, self.active_bucket = kept.index, kept.active
        return kept
