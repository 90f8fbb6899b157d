"""LSH clustering with epoch-level reuse of the assignment.

Drop-in for the reference's ``layer/CompressgnnCluster.py``: ``Compressgnn_Cluster(in_feature,
param_H, training=True, device=None, dtype=None, cache=True, index_cache=False,
refresh_interval=1, refresh_policy='fixed', q_min=1, q_max=10, tau_loss=None)`` with
``set_epoch``, ``reset_cache``, ``forward(input, epoch=None, cache_key=None,
force_refresh=False)`` and the attributes ``vertex_index``, ``active_bucket``,
``last_refreshed``, ``refresh_count``, ``current_interval``; plus ``_Mean`` and the legacy
``Compressgnn_Cluster_Function``.  Only the assignment (index, counts, bucket permutation) is
cached; the mean representatives are recomputed from the current features on every call so
that gradients reach the current upstream model.

One addition: ``process_group``.  When features are sharded by column across GPUs, each rank
holds ``[N, F/G]`` features and its own ``[F/G, H]`` slice of the hyperplanes; the partial
projections are summed with one all-reduce before sign packing, so every rank derives the
same assignment.
"""
import math
import operator

import torch
from torch.autograd.function import once_differentiable

from .. import runtime as _native


def _require_cuda(x):
    if not x.is_cuda:
        raise RuntimeError("compressgnn_b200 runs on CUDA tensors only (no CPU cluster path)")


class _Mean(torch.autograd.Function):
    """``reps[g] = mean of x rows with index == g``; first-order gradient only."""

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
    """Compatibility entry point: assignment + mean in one call, no cache."""

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


class Compressgnn_Cluster(torch.nn.Module):
    """Mean representatives over LSH buckets; ``refresh_interval`` counts epochs, never calls.

    With ``refresh_interval > 1`` (or the loss policy) the caller must provide the zero-based
    epoch through ``set_epoch`` or ``forward(epoch=...)``.  ``training=False`` at construction
    keeps the old tensor-only return; otherwise ``forward`` returns ``(reps, index)`` in both
    ``train()`` and ``eval()``, which keep separate assignment caches.
    """

    def __init__(self, in_feature, param_H, training=True, device=None, dtype=None, cache=True,
                 index_cache=False, refresh_interval=1, refresh_policy='fixed', q_min=1, q_max=10,
                 tau_loss=None, process_group=None):
        super().__init__()
        self.in_feature = operator.index(in_feature)
        self.param_H = operator.index(param_H)
        if self.in_feature < 0 or not 0 <= self.param_H <= 30:
            raise ValueError('Expected nonnegative feature width and 0 <= param_H <= 30')
        self.refresh_interval = operator.index(refresh_interval)
        self.q_min, self.q_max = operator.index(q_min), operator.index(q_max)
        if self.refresh_interval < 1 or not 1 <= self.q_min <= self.q_max:
            raise ValueError('Refresh intervals must be positive integers, q_min <= q_max')
        if refresh_policy not in ('fixed', 'loss'):
            raise ValueError('refresh_policy must be fixed or loss')
        if refresh_policy == 'loss' and (tau_loss is None or not math.isfinite(tau_loss) or tau_loss <= 0):
            raise ValueError('Loss policy requires a finite positive tau_loss')
        self.refresh_policy, self.tau_loss = refresh_policy, tau_loss
        self.cache, self.index_cache = bool(cache), bool(index_cache)
        self.is_training = bool(training)  # return contract, not the cache namespace
        self.process_group = process_group
        self.register_buffer('random_vectors',
                             torch.randn(self.in_feature, self.param_H, device=device, dtype=dtype))
        self._epoch = self._previous_loss = self._last_loss_epoch = None
        self.current_interval = self._initial_interval()
        self._states, self._workspaces = {}, {}
        self.vertex_index = self.active_bucket = None
        self.last_refreshed = False
        self.refresh_count = 0
        self.train(training)

    def _initial_interval(self):
        return self.refresh_interval if self.refresh_policy == 'fixed' else self.q_min

    def set_epoch(self, epoch, loss=None):
        """Zero-based epoch; ``loss`` is the previous completed training loss as a host number."""
        epoch = operator.index(epoch)
        if epoch < 0:
            raise ValueError('epoch must be nonnegative')
        if self._epoch is not None and epoch < self._epoch:  # a new run: forget everything
            self.reset_cache()
            self._previous_loss = self._last_loss_epoch = None
            self.current_interval = self._initial_interval()
        self._epoch = epoch
        if loss is not None and self.refresh_policy == 'loss' and epoch != self._last_loss_epoch:
            if torch.is_tensor(loss):
                raise TypeError('Pass a host loss value; do not hide a GPU synchronization in set_epoch')
            loss = float(loss)
            if not math.isfinite(loss):
                raise ValueError('loss must be finite')
            if self._previous_loss is not None:
                raw = self.q_min + (self.q_max - self.q_min) * math.exp(
                    -abs(loss - self._previous_loss) / self.tau_loss)
                self.current_interval = min(self.q_max, max(self.q_min, int(math.floor(raw + .5))))
            self._previous_loss, self._last_loss_epoch = loss, epoch
        return self

    def reset_cache(self):
        self._states.clear()
        self.vertex_index = self.active_bucket = None
        self.last_refreshed = False

    def _apply(self, fn, *args, **kwargs):
        self.reset_cache()
        self._workspaces.clear()
        return super()._apply(fn, *args, **kwargs)

    def _load_from_state_dict(self, *args, **kwargs):
        self.reset_cache()
        self._previous_loss = self._last_loss_epoch = self._epoch = None
        self.current_interval = self._initial_interval()
        return super()._load_from_state_dict(*args, **kwargs)

    def _workspace(self, input, stream):
        key = (input.device, stream, self.param_H)
        ws = self._workspaces.get(key)
        need = _native.lib().cgnn_cluster_workspace_bytes(int(input.size(0)), self.param_H)
        if ws is None or ws[2].numel() < need:  # sized by rows: grow when a larger input arrives
            ws = _native.cluster_workspace(input, self.param_H)
            self._workspaces[key] = ws
        return ws

    def forward(self, input, epoch=None, cache_key=None, force_refresh=False):
        if input.dim() != 2 or input.size(1) != self.in_feature:
            raise ValueError('Expected [nodes, in_feature] input')
        if input.device != self.random_vectors.device or input.dtype != self.random_vectors.dtype:
            raise ValueError('Move the module to the input device and dtype before use')
        if input.dtype not in (torch.float32, torch.float64):
            raise ValueError('Only float32 and float64 are supported')
        if epoch is not None:
            self.set_epoch(epoch)
        if self.cache and self._epoch is None and (self.refresh_interval > 1 or self.refresh_policy == 'loss'):
            raise ValueError('Cross-epoch reuse requires set_epoch(epoch) or forward(epoch=epoch)')
        _require_cuda(input)
        stream = torch.cuda.current_stream(input.device).cuda_stream
        slot = (self.training, input.device, stream)
        signature = (tuple(input.shape), input.dtype, cache_key, self.random_vectors.data_ptr(),
                     self.random_vectors._version)
        state = self._states.get(slot)
        refresh = (not self.cache or force_refresh or self._epoch is None or state is None or
                   state['signature'] != signature or
                   self._epoch - state['epoch'] >= self.current_interval)
        if refresh:
            if input.size(0):
                index, counts, active = _assign(input, self.random_vectors, self.param_H,
                                                self._workspace(input.contiguous(), stream),
                                                self.process_group)
            else:
                index = torch.empty(0, device=input.device, dtype=torch.int64)
                counts = torch.zeros(1, device=input.device, dtype=torch.int32)
                active = 0
            state = dict(index=index, counts=counts, active=active, signature=signature, epoch=self._epoch)
            if self.cache and self._epoch is not None:
                self._states[slot] = state
            self.refresh_count += 1
        self.last_refreshed = refresh
        self.vertex_index, self.active_bucket = state['index'], state['active']
        output = _Mean.apply(input, state['index'], state['counts'])
        return (output, state['index']) if self.is_training else output
