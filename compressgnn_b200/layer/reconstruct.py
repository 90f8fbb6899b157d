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
    def forward(ctx, src, index, bias, relu):
        index = index.contiguous()
        output = _native.cluster_reconstruct(src.contiguous(), index,
                                             None if bias is None else bias.contiguous(), relu)
        ctx.save_for_backward(index, output)
        ctx.groups, ctx.relu, ctx.has_bias = src.size(0), relu, bias is not None
        return output

    @staticmethod
    @once_differentiable
    def backward(ctx, grad):
        index, output = ctx.saved_tensors
        # `output` is this Function's own forward result, so one mask row per group suffices.
        result = _native.cluster_reconstruct_backward(grad.contiguous(), index, output, ctx.groups,
                                                      ctx.relu, return_bias_grad=ctx.has_bias,
                                                      output_is_forward_result=True)
        if ctx.has_bias:
            return result[0], None, result[1], None
        return result, None, None, None


class Compressgnn_Reconstruct(torch.nn.Module):
    def __init__(self, node_dim=-2):
        super().__init__()
        self.node_dim = node_dim

    def forward(self, src, index, bias=None, activation=None):
        if activation not in (None, 'relu'):
            raise ValueError('Supported activations: None, relu')
        if src.is_cuda and src.dim() == 2 and self.node_dim in (0, -2):
            return _Reconstruct.apply(src, index, bias, activation == 'relu')
        if src.is_cuda:
            output = src.index_select(self.node_dim, index)
            if bias is not None:
                output = output + bias
            return output.relu() if activation == 'relu' else output
        raise RuntimeError("compressgnn_b200 runs on CUDA tensors only (no CPU reconstruct path)")
