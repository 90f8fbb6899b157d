"""Column-sharded hot path on 2 GPUs (NCCL): shard-local propagation equals the columns of the
single-GPU result; the cluster module with a process group gives every rank the assignment the
oracle's sharded projection order predicts; a column-sharded two-layer GCN step (forward,
gradients after ``sync_gradients``) equals plain torch on the full features.  Skipped on a box
with fewer than 2 GPUs."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port):
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from compressgnn_b200 import dist as cdist
        from compressgnn_b200 import offline as off
        from compressgnn_b200.layer import Compressgnn_Cluster, Compressgnn_Reconstruct, KPropagate
        from compressgnn_b200.loader import CompressgnnData
        from conftest import assert_close_rel
        from oracle import oracle
        n, width, bits = 3000, 64, 12
        v, e = off.generate_copy_graph(n, 2.1, 4.0, 200, 0.7, 32, 8, seed=11)
        rng = np.random.default_rng(11)
        x = rng.standard_normal((n, width)).astype(np.float32)
        mask = np.ones(n, bool)
        data = CompressgnnData(x, (v, e), np.zeros(n, np.int64), mask, mask, mask, min_pair_frequency=3,
                               threshold=1, min_edge=10)
        g = data.edge_index
        blocks = {k: tuple(t.numpy() for t in getattr(g, f"{k}_graph").csr()) for k in ("v2v", "v2r", "r2v")}
        blocks["r2r"] = [tuple(t.numpy() for t in lvl.csr()) for lvl in g.r2r_graph]
        full = oracle.propagate_forward(blocks, x)
        begin, end = cdist.column_range(width, rank, world)
        data.to(torch.device("cuda", rank))
        xs = cdist.shard_columns(data.x, rank, world).requires_grad_()
        out = KPropagate()(xs, data.edge_index, None, data.vertex_cnt, data.rule_cnt)
        assert_close_rel(out.detach().cpu().numpy(), full[:, begin:end], what=f"rank {rank} forward shard")
        go = torch.from_numpy(rng.standard_normal((n, width)).astype(np.float32)).cuda()
        (gx,) = torch.autograd.grad(out, xs, cdist.shard_columns(go, rank, world))
        ref_bwd = oracle.propagate_backward(blocks, go.cpu().numpy(), n, data.rule_cnt)
        assert_close_rel(gx.cpu().numpy(), ref_bwd[:, begin:end], what=f"rank {rank} backward shard")
        # cluster on the propagated shard: one all-reduce, identical ids on every rank
        planes = rng.standard_normal((width, bits)).astype(np.float32)
        cluster = Compressgnn_Cluster(end - begin, bits, device="cuda", process_group=dist.group.WORLD)
        with torch.no_grad():
            cluster.random_vectors.copy_(cdist.shard_planes(torch.from_numpy(planes), rank, world))
        feats = torch.from_numpy(full).cuda()
        reps, index = cluster(cdist.shard_columns(feats, rank, world))
        rids, rcounts, ractive = oracle.cluster_assign(full, planes, shards=world)
        margin = np.abs(full.astype(np.float64) @ planes.astype(np.float64)).min(axis=1)
        safe = margin > 1e-4  # NCCL's reduction order is its own; ties within rounding are exempt
        mine = index.cpu().numpy()[safe]
        # same partition of the safe rows into buckets, in the same (ascending code) order
        pairs = np.unique(np.stack([mine, rids[safe]]), axis=1)
        assert np.unique(pairs[0]).size == pairs.shape[1] == np.unique(pairs[1]).size
        assert np.all(np.diff(pairs[1][np.argsort(pairs[0])]) > 0)
        gathered = [torch.empty_like(index) for _ in range(world)]
        dist.all_gather(gathered, index)
        assert all(torch.equal(gathered[0], t) for t in gathered)  # bit-identical across ranks
        ref_reps = oracle.cluster_mean(full[:, begin:end], index.cpu().numpy(),
                                       np.bincount(index.cpu().numpy(), minlength=reps.size(0)).astype(np.int32))
        assert_close_rel(reps.cpu().numpy(), ref_reps, what="sharded mean")
        y = Compressgnn_Reconstruct()(reps, index, activation="relu")
        assert torch.equal(y, reps.index_select(0, index).relu())

        # a whole column-sharded GCN step against plain torch on the full features, using the
        # assignment the sharded layers chose
        from compressgnn_b200.model import GCN
        classes = 5
        torch.manual_seed(3)  # same weights and hyperplanes on every rank
        model = GCN(width, classes, hidden_features=32, param_H=10, dropout=0.0, use_transformation=True,
                    refresh_interval=5, num_layers=2).cuda()
        sharded = cdist.ShardedGCN(model, dist.group.WORLD)
        sharded.set_epoch(0)
        labels = torch.from_numpy(rng.integers(0, classes, n)).cuda()
        out = sharded(cdist.shard_columns(data.x, rank, world), data.edge_index, dropout=False)
        assert out.shape == (n, classes)

        def scatter_mean(t, index, groups):
            sums = torch.zeros(groups, t.size(1), device=t.device).index_add_(0, index, t)
            return sums / torch.bincount(index, minlength=groups).clamp_min(1).to(t.dtype)[:, None]

        def layer_ref(layer, feats):
            p = KPropagate()(feats, data.edge_index, None, data.vertex_cnt, data.rule_cnt)
            index = layer.cluster.vertex_index
            reps_ = scatter_mean(p, index, layer.cluster.active_bucket + 1)
            return (reps_ @ layer.lin.weight.t()).index_select(0, index) + layer.lin.bias

        ref = torch.log_softmax(layer_ref(sharded.layers[1], layer_ref(sharded.layers[0], data.x).relu()), 1)
        torch.testing.assert_close(out, ref, atol=2e-4, rtol=1e-3)
        torch.nn.functional.nll_loss(out, labels).backward()
        sharded.sync_gradients()
        params = list(model.parameters())
        for p_, gr in zip(params, torch.autograd.grad(torch.nn.functional.nll_loss(ref, labels), params)):
            torch.testing.assert_close(p_.grad, gr, atol=2e-4, rtol=1e-3)
        outs = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(outs, out.detach())
        assert all(torch.equal(outs[0], t) for t in outs)  # replicated result, bit for bit
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(600)
def test_two_gpus_shard_columns():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(2, _free_port()), nprocs=2, join=True)
