"""The caller of the hot path: ``GNNLayer`` (propagate, then either a Linear on all nodes or
cluster -> Linear on representatives -> fused reconstruct) and a GCN stack of them
(ref: ``model/compressgnn/gcn.py:12-71``; the reference hard-wires three layers, here the
depth is a parameter so the two-layer benchmark configurations can be built, and the ReLU
after a hidden layer is handed to the layer so that it runs inside the reconstruct kernel)."""
import torch
import torch.nn.functional as F
from torch import Tensor

from torch.autograd.function import once_differentiable

from . import runtime as _native
from .layer import Compressgnn_Cluster, Compressgnn_Reconstruct, KPropagate


class _TransformedLinear(torch.autograd.Function):
    """``act(dropout)(Linear(bucket means of x))`` spread back over the nodes -- cluster mean, the Linear on
    the representatives and the fused reconstruction as ONE autograd node (ref: the three modules chained
    in model/compressgnn/gcn.py:27-34).  Same native calls and the same arithmetic as the modules one by
    one; what goes away is four autograd nodes per layer and direction, which is host time an epoch of
    ~1.5 ms is bound by."""

    @staticmethod
    def forward(ctx, x, index, counts, weight, bias, relu, dropout_p):
        x = x.contiguous()
        reps = _native.cluster_mean(x, index, counts)
        lin = reps @ weight.t()
        seed = 0
        if dropout_p > 0.0:
            seed = int(torch.randint(0, 2**63 - 1, (1,), dtype=torch.int64).item())
        out = _native.cluster_reconstruct(lin, index, bias, relu, dropout_p, seed)
        ctx.save_for_backward(index, counts, reps, weight, out)
        ctx.relu, ctx.dropout_p = relu, dropout_p
        return out

    @staticmethod
    @once_differentiable
    def backward(ctx, grad):
        index, counts, reps, weight, out = ctx.saved_tensors
        dropped = ctx.dropout_p > 0.0
        # without dropout the rows of a group are identical and one mask row per group suffices; with it
        # every row has its own zeros (dropped or clamped alike): exact mask, sums rescaled
        d_lin, d_bias = _native.cluster_reconstruct_backward(grad.contiguous(), index, out, reps.size(0), ctx.relu,
                                                             return_bias_grad=True,
                                                             output_is_forward_result=not dropped)
        if dropped:
            scale = 1.0 / (1.0 - ctx.dropout_p)
            d_lin.mul_(scale)
            d_bias.mul_(scale)
        d_weight = d_lin.t() @ reps if ctx.needs_input_grad[3] else None
        d_x = None
        if ctx.needs_input_grad[0]:
            d_x = _native.cluster_mean_backward(d_lin @ weight, index, counts)
        return d_x, None, None, d_weight, d_bias if ctx.needs_input_grad[4] else None, None, None


class GNNLayer(torch.nn.Module):
    def __init__(self, in_features, out_features, param_H=1, use_transformation=False, refresh_interval=1,
                 process_group=None, activation=None):
        super().__init__()
        if activation not in (None, "relu"):
            raise ValueError("activation must be None or 'relu'")
        self.activation = activation  # applied to the layer's output (fused into the reconstruction)
        self.lin = torch.nn.Linear(in_features=in_features, out_features=out_features, bias=True)
        self.P = KPropagate()
        self.use_transformation = use_transformation
        self.cluster = Compressgnn_Cluster(in_feature=in_features, param_H=param_H, training=True, cache=True,
                                           index_cache=False, refresh_interval=refresh_interval,
                                           process_group=process_group)
        self.reconstruct = Compressgnn_Reconstruct()

    def set_epoch(self, epoch, loss=None):
        self.cluster.set_epoch(epoch, loss=loss)

    def reset_cache(self):
        self.cluster.reset_cache()

    def forward(self, x: Tensor, edge_index, edge_weight=None, vertex_cnt: int = 0, rule_cnt: int = 0,
                dropout: float = 0.0) -> Tensor:
        """``dropout``: probability of the dropout the model applies to this layer's (ReLU) output; with the
        transformation path it runs inside the reconstruct kernel."""
        x = self.P(x=x, edge_index=edge_index, edge_weight=edge_weight, vertex_cnt=vertex_cnt, rule_cnt=rule_cnt)
        if self.use_transformation and x.is_cuda and x.dim() == 2 and self.cluster.is_training and \
                (self.activation == "relu" or not dropout):
            kept = self.cluster.assignment(x)
            return _TransformedLinear.apply(x, kept.index, kept.counts, self.lin.weight, self.lin.bias,
                                            self.activation == "relu", float(dropout))
        if self.use_transformation:
            reps, index = self.cluster(x)
            fused = dropout if self.activation == "relu" else 0.0
            x = self.reconstruct(F.linear(reps, self.lin.weight, None), index, bias=self.lin.bias,
                                 activation=self.activation, dropout=fused)
            return F.dropout(x, p=dropout) if dropout and not fused else x
        x = self.lin(x)
        x = x.relu() if self.activation == "relu" else x
        return F.dropout(x, p=dropout) if dropout else x


class GCN(torch.nn.Module):
    def __init__(self, in_features, out_features, hidden_features=128, param_H=1, dropout=0.3,
                 use_transformation=False, refresh_interval=1, num_layers=3):
        super().__init__()
        dims = [in_features] + [hidden_features] * (num_layers - 1) + [out_features]
        self.layers = torch.nn.ModuleList(
            GNNLayer(dims[i], dims[i + 1], param_H=param_H, use_transformation=use_transformation,
                     refresh_interval=refresh_interval, activation="relu" if i + 1 < num_layers else None)
            for i in range(num_layers))
        self.dropout = dropout

    def set_epoch(self, epoch, loss=None):
        for layer in self.layers:
            layer.set_epoch(epoch, loss=loss)

    def reset_cache(self):
        for layer in self.layers:
            layer.reset_cache()

    def _stack(self, x, edge_index, edge_weight, vertex_cnt, rule_cnt, dropout):
        last = len(self.layers) - 1
        for i, layer in enumerate(self.layers):
            # the hidden layers' ReLU and dropout are part of the layer (fused into the reconstruct kernel)
            p = self.dropout if (i != last and dropout and self.training) else 0.0
            x = layer(x=x, edge_index=edge_index, edge_weight=edge_weight, vertex_cnt=vertex_cnt, rule_cnt=rule_cnt,
                      dropout=p)
        return F.log_softmax(x, dim=1)

    def forward(self, x: Tensor, edge_index, edge_weight=None, vertex_cnt: int = 0, rule_cnt: int = 0) -> Tensor:
        return self._stack(x, edge_index, edge_weight, vertex_cnt, rule_cnt, True)

    def inference(self, x: Tensor, edge_index, edge_weight=None, vertex_cnt: int = 0, rule_cnt: int = 0) -> Tensor:
        return self._stack(x, edge_index, edge_weight, vertex_cnt, rule_cnt, False)
