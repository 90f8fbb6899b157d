"""Reconstruct node features from bucket representatives, fusing the shared bias and ReLU.

Drop-in for the reference's ``layer/CompressgnnReconstruct.py:11-42``:
``Compressgnn_Reconstruct(node_dim=-2).forward(src, index, bias=None, activation=None)``.
Unlike the reference, every CUDA call goes through the native gather (also without bias or
activation), and the bias gradient comes out of the same native call as the representative
gradient.
"""
import torch
from torch.autograd.function import once_differentiable

from .. import runtime as _native


class _Reconstruct(torch.autograd.Function):
    @staticmethod
    def forward(ctx, src, index, bias, relu, dropout_p=0.0):
        index = index.contiguous()
        seed = 0
        if dropout_p > 0.0:
            # a fresh 63-bit key per call from torch's host generator (follows torch.manual_seed; no device sync)
            seed = int(torch.randint(0, 2**63 - 1, (1,), dtype=torch.int64).item())
        output = _native.cluster_reconstruct(src.contiguous(), index,
                                             None if bias is None else bias.contiguous(), relu, dropout_p, seed)
        ctx.save_for_backward(index, output)
        ctx.groups, ctx.relu, ctx.has_bias, ctx.dropout_p = src.size(0), relu, bias is not None, dropout_p
        return output

    @staticmethod
    @once_differentiable
    def backward(ctx, grad):
        index, output = ctx.saved_tensors
        # `output` is this Function's own forward result.  Without dropout the rows of a group are identical
        # and one mask row per group suffices; with dropout every row has its own zeros (dropped or clamped
        # elements alike), so the gradient rows are masked one by one and the sums rescaled.
        dropped = ctx.dropout_p > 0.0
        result = _native.cluster_reconstruct_backward(grad.contiguous(), index, output, ctx.groups,
                                                      ctx.relu, return_bias_grad=ctx.has_bias,
                                                      output_is_forward_result=not dropped)
        if dropped:
            scale = 1.0 / (1.0 - ctx.dropout_p)
            result = tuple(t.mul_(scale) for t in result) if ctx.has_bias else result.mul_(scale)
        if ctx.has_bias:
            return result[0], None, result[1], None, None
        return result, None, None, None, None


class Compressgnn_Reconstruct(torch.nn.Module):
    def __init__(self, node_dim=-2):
        super().__init__()
        self.node_dim = node_dim

    def forward(self, src, index, bias=None, activation=None, dropout=0.0):
        """``dropout`` (not in the reference's signature): probability of the dropout that follows a ReLU
        activation, applied in the same pass; the caller passes 0 outside of training."""
        if activation not in (None, 'relu'):
            raise ValueError('Supported activations: None, relu')
        if dropout and activation != 'relu':
            raise ValueError('the fused dropout needs activation="relu"')
        if src.is_cuda and src.dim() == 2 and self.node_dim in (0, -2):
            return _Reconstruct.apply(src, index, bias, activation == 'relu', float(dropout))
        if src.is_cuda:
            output = src.index_select(self.node_dim, index)
            if bias is not None:
                output = output + bias
            output = output.relu() if activation == 'relu' else output
            return torch.nn.functional.dropout(output, dropout) if dropout else output
        raise RuntimeError("compressgnn_b200 runs on CUDA tensors only (no CPU reconstruct path)")
