"""Column sharding of the hot path across the GPUs of one node.

The dense feature matrix ``X [N, F]`` is cut into ``G`` contiguous column blocks, one per
rank; the compressed graph is replicated.  Propagation, mean, mean-backward and reconstruct
act on every column independently, so they run on the local block with no communication.
Only the LSH assignment needs whole rows: each rank projects its block onto its slice of the
hyperplanes and the partial projections are summed with ONE all-reduce (NCCL over NVLink on
GPUs, gloo in the CPU tests) before sign packing, after which every rank derives the same
bucket ids, counts and permutation.

A whole layer (``ShardedGNNLayer``, ``ShardedGCN``) needs two more, small exchanges because its
Linear contracts over all feature columns: the ``[B, F/G]`` blocks of the bucket representatives
are gathered in front of it (their gradients summed on the way back), and the gradients of
weight rows owned by different ranks are summed before the optimiser step.
"""
import torch
import torch.distributed as dist


def column_range(width, rank, world):
    """``(begin, end)`` of rank's block; blocks are ``ceil(width / world)`` wide, the last one
    takes what is left (the convention the CPU oracle's sharded projection uses)."""
    per = -(-int(width) // int(world))
    begin = min(rank * per, width)
    return begin, min(begin + per, width)


def shard_columns(x, rank, world):
    """This rank's contiguous column block of ``x`` as its own contiguous tensor."""
    begin, end = column_range(x.size(-1), rank, world)
    return x[..., begin:end].contiguous()


def shard_planes(planes, rank, world):
    """Rows of the ``[F, H]`` hyperplane matrix that belong to this rank's feature columns."""
    begin, end = column_range(planes.size(0), rank, world)
    return planes[begin:end].contiguous()


def allreduce_projection(partial, group=None):
    """Sum the ``[N, H]`` partial projections of all ranks in place (the path's one collective)."""
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=group)
    return partial


def gather_columns(local, group=None):
    """Concatenate every rank's column block (test / export helper, not on the hot path)."""
    world = dist.get_world_size(group)
    parts = [torch.empty_like(local) for _ in range(world)]
    dist.all_gather(parts, local, group=group)
    return torch.cat(parts, dim=-1)


class _GatherColumns(torch.autograd.Function):
    """``[B, F/G]`` column blocks of all ranks -> ``[B, F]`` on every rank: ONE all-gather.

    Backward: with ``replicated_consumer`` every rank computes the same thing from the gathered
    matrix, so the incoming gradient is already the full one and the local block is cut out of
    it (no communication); otherwise each rank consumed the matrix for its own slice of the
    outputs, and ONE reduce-scatter sums the gradients over the ranks and leaves every rank with
    the block it owns (half the bytes of an all-reduce, and no copy of the full gradient).
    """

    @staticmethod
    def forward(ctx, local, group, replicated_consumer):
        ctx.group, ctx.replicated = group, replicated_consumer
        ctx.rank, ctx.world = dist.get_rank(group), dist.get_world_size(group)
        local = local.contiguous()
        rows, width = local.shape
        stacked = torch.empty(ctx.world * rows, width, dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(stacked, local, group=group)   # rank g's block = rows [g*B, (g+1)*B)
        return stacked.view(ctx.world, rows, width).permute(1, 0, 2).reshape(rows, ctx.world * width)

    @staticmethod
    def backward(ctx, grad):
        rows, width = grad.size(0), grad.size(1) // ctx.world
        if ctx.replicated:
            begin = ctx.rank * width
            return grad[:, begin:begin + width].contiguous(), None, None
        stacked = grad.view(rows, ctx.world, width).permute(1, 0, 2).contiguous().view(ctx.world * rows, width)
        mine = torch.empty(rows, width, dtype=grad.dtype, device=grad.device)
        dist.reduce_scatter_tensor(mine, stacked, op=dist.ReduceOp.SUM, group=ctx.group)
        return mine, None, None


def gather_columns_autograd(local, group=None, replicated_consumer=False):
    """Differentiable ``gather_columns`` (equal block widths on all ranks)."""
    return _GatherColumns.apply(local, group, replicated_consumer)


class ShardedGNNLayer(torch.nn.Module):
    """A ``GNNLayer`` with transformation compression, run on one column block per rank.

    Built from a full layer (same weights on every rank).  Propagation, the bucket means and
    the reconstruction act on the local ``[N, F/G]`` block; the assignment sums the partial
    projections (inside ``Compressgnn_Cluster``); the Linear contracts over all feature
    columns, so the small ``[B, F/G]`` representative blocks are gathered first.  With
    ``shard_output`` the rank then produces only its block of the output columns (its rows of
    the weight); without it (class scores, whose width need not divide) every rank produces
    all output columns.
    """

    def __init__(self, layer, group=None, shard_output=True):
        super().__init__()
        from .layer import Compressgnn_Cluster, Compressgnn_Reconstruct, KPropagate
        if not layer.use_transformation:
            raise ValueError("ShardedGNNLayer needs a layer built with use_transformation=True")
        self.group, self.shard_output = group, shard_output
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        full = layer.cluster
        if full.in_feature % self.world or (shard_output and layer.lin.out_features % self.world):
            raise ValueError("feature widths must divide by the number of ranks")
        self.lin = layer.lin
        self.activation = layer.activation
        self.P = KPropagate()
        self.cluster = Compressgnn_Cluster(
            in_feature=full.in_feature // self.world, param_H=full.param_H, training=True, cache=True,
            index_cache=False, refresh_interval=full.refresh_interval, process_group=group,
            device=full.random_vectors.device, dtype=full.random_vectors.dtype)
        with torch.no_grad():
            self.cluster.random_vectors.copy_(shard_planes(full.random_vectors, self.rank, self.world))
        self.reconstruct = Compressgnn_Reconstruct()

    def set_epoch(self, epoch, loss=None):
        self.cluster.set_epoch(epoch, loss=loss)

    def reset_cache(self):
        self.cluster.reset_cache()

    def forward(self, x_local, edge_index, edge_weight=None, vertex_cnt=0, rule_cnt=0, dropout=0.0):
        p = self.P(x=x_local, edge_index=edge_index, edge_weight=edge_weight, vertex_cnt=vertex_cnt,
                   rule_cnt=rule_cnt)
        reps_local, index = self.cluster(p)
        reps = gather_columns_autograd(reps_local, self.group, replicated_consumer=not self.shard_output)
        weight, bias = self.lin.weight, self.lin.bias
        if self.shard_output:
            begin, end = column_range(self.lin.out_features, self.rank, self.world)
            weight, bias = weight[begin:end], bias[begin:end]
        fused = dropout if self.activation == "relu" else 0.0
        out = self.reconstruct(torch.nn.functional.linear(reps, weight, None), index, bias=bias,
                               activation=self.activation, dropout=fused)
        return torch.nn.functional.dropout(out, p=dropout) if dropout and not fused else out


class ShardedGCN(torch.nn.Module):
    """A ``GCN`` (all layers with transformation compression) on column-sharded features.

    ``forward`` takes this rank's ``[N, F/G]`` block of the input features and returns the full
    ``[N, classes]`` log-probabilities on every rank.  Hidden layers keep their outputs sharded;
    the last layer's output is replicated.  After ``backward`` call ``sync_gradients()``: a
    hidden layer's weight rows are owned by one rank each, so their gradients are summed over
    the ranks; the last layer's gradients are already identical everywhere.
    """

    def __init__(self, model, group=None):
        super().__init__()
        last = len(model.layers) - 1
        self.group = group
        self.dropout = model.dropout
        self.layers = torch.nn.ModuleList(
            ShardedGNNLayer(layer, group, shard_output=i != last) for i, layer in enumerate(model.layers))

    def set_epoch(self, epoch, loss=None):
        for layer in self.layers:
            layer.set_epoch(epoch, loss=loss)

    def reset_cache(self):
        for layer in self.layers:
            layer.reset_cache()

    def forward(self, x_local, edge_index, edge_weight=None, vertex_cnt=0, rule_cnt=0, dropout=True):
        last = len(self.layers) - 1
        x = x_local
        for i, layer in enumerate(self.layers):
            p = self.dropout if (i != last and dropout and self.training) else 0.0
            x = layer(x, edge_index, edge_weight, vertex_cnt, rule_cnt, dropout=p)
        return torch.nn.functional.log_softmax(x, dim=1)

    def consolidate_parameters(self):
        """Make every rank's copy of the model whole again after training WITHOUT ``sync_gradients``.

        A hidden layer's weight rows (and bias entries) ``[begin, end)`` are used by one rank only, and
        that rank sees their full gradient; the other ranks see zeros for them.  With an optimiser that
        leaves a parameter alone while its gradient is zero (Adam or SGD without weight decay) each
        rank can therefore step on its own and skip the per-epoch gradient all-reduce; the owners'
        blocks are gathered here once, when the whole model is needed (evaluation, checkpoint)."""
        world = dist.get_world_size(self.group)
        if world == 1:
            return
        rank = dist.get_rank(self.group)
        with torch.no_grad():
            for layer in self.layers:
                if not layer.shard_output:
                    continue  # computed identically on every rank
                for p in layer.lin.parameters():
                    begin, end = column_range(p.size(0), rank, world)
                    whole = torch.empty_like(p)
                    dist.all_gather_into_tensor(whole, p[begin:end].contiguous(), group=self.group)
                    p.copy_(whole)

    def sync_gradients(self):
        """Sum the hidden layers' parameter gradients over the ranks (one flat all-reduce)."""
        grads = [p.grad for layer in self.layers if layer.shard_output for p in layer.lin.parameters()
                 if p.grad is not None]
        if not grads or dist.get_world_size(self.group) == 1:
            return
        flat = torch.cat([g.reshape(-1) for g in grads])
        dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=self.group)
        offset = 0
        for g in grads:
            g.copy_(flat[offset:offset + g.numel()].view_as(g))
            offset += g.numel()


# Input width from which sharding a model's feature columns pays on one node.  Every epoch of a sharded
# model issues two collectives per hidden layer and a dozen more small launches; measured on B200s that
# is 0.3-0.5 ms per epoch, which the shard-local operators only win back when the first layer's work
# (proportional to the input width) is several times that: 1024 input columns gain at 2, 4 and 8 GPUs,
# 256 and fewer lose at every GPU count.
MIN_SHARDED_FEATURES = 512


def place_model(model, in_features, group=None, min_features=MIN_SHARDED_FEATURES):
    """``(module, sharded)``: a ``ShardedGCN`` over ``model`` when the input is wide enough for column
    sharding to pay, else ``model`` itself, to be run as a replica on every rank (the full feature matrix,
    the same parameters and the same random stream everywhere, no collective).  A sharded module takes
    ``shard_columns(x, rank, world)``, a replica takes ``x``."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world > 1 and in_features >= min_features and in_features % world == 0:
        return ShardedGCN(model, group), True
    return model, False

