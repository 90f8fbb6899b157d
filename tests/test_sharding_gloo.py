"""World-size-2 run of the column-sharded path's host logic on CPU (gloo): shard ranges,
the one all-reduce of partial projections, and identical assignments on every rank.  The
arithmetic on each rank is the CPU oracle (no GPU here); the GPU twin of this test is
tests/test_multi_gpu.py."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, str(ROOT))
    from compressgnn_b200 import dist as cdist
    from oracle import oracle
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(7)  # same stream on every rank: the full problem
        n, width, bits = 500, 50, 12
        x = rng.standard_normal((n, width)).astype(np.float32)
        planes = rng.standard_normal((width, bits)).astype(np.float32)
        xs = cdist.shard_columns(torch.from_numpy(x), rank, world)
        ps = cdist.shard_planes(torch.from_numpy(planes), rank, world)
        begin, end = cdist.column_range(width, rank, world)
        assert xs.shape == (n, end - begin) and ps.shape == (end - begin, bits) and xs.is_contiguous()
        partial = torch.from_numpy(oracle.project(xs.numpy(), ps.numpy()))
        total = cdist.allreduce_projection(partial)
        ids, counts, active = oracle.assign_from_codes(oracle.codes_from_projection(total.numpy()), bits)
        # every rank must hold the same assignment, equal to the oracle's sharded order
        ref = oracle.cluster_assign(x, planes, shards=world)
        assert active == ref[2] and np.array_equal(ids, ref[0]) and np.array_equal(counts, ref[1])
        # column-independent operators: the local block of the full result
        mean_local = oracle.cluster_mean(xs.numpy(), ids, counts)
        mean_full = oracle.cluster_mean(x, ids, counts)
        assert np.array_equal(mean_local, mean_full[:, begin:end])
        gathered = cdist.gather_columns(torch.from_numpy(mean_local))
        assert np.array_equal(gathered.numpy(), mean_full)
        np.save(os.path.join(out_dir, f"ids_{rank}.npy"), ids)
    finally:
        dist.destroy_process_group()


def test_column_ranges_cover_the_width():
    from compressgnn_b200.dist import column_range
    for width in (1, 7, 16, 50, 256):
        for world in (1, 2, 4, 8):
            ranges = [column_range(width, r, world) for r in range(world)]
            assert ranges[0][0] == 0 and ranges[-1][1] == width
            assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))


@pytest.mark.timeout(300)
def test_two_ranks_agree_on_the_assignment(tmp_path):
    world, port = 2, _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    a, b = (np.load(tmp_path / f"ids_{r}.npy") for r in range(world))
    assert np.array_equal(a, b)


def _gather_worker(rank, world, port):
    sys.path.insert(0, str(ROOT))
    from compressgnn_b200 import dist as cdist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        gen = torch.Generator().manual_seed(3)  # the full problem on every rank
        full = torch.randn(6, 8, generator=gen, dtype=torch.float64)
        weight = torch.randn(10, 8, generator=gen, dtype=torch.float64)
        target = torch.randn(6, 10, generator=gen, dtype=torch.float64)
        ref_in = full.clone().requires_grad_()
        ((ref_in @ weight.t() - target) ** 2).sum().backward()
        begin, end = cdist.column_range(8, rank, world)
        # (a) every rank consumes the gathered matrix for its own slice of the outputs
        local = full[:, begin:end].clone().requires_grad_()
        gathered = cdist.gather_columns_autograd(local, None, replicated_consumer=False)
        assert torch.equal(gathered, full)
        ob, oe = cdist.column_range(10, rank, world)
        ((gathered @ weight[ob:oe].t() - target[:, ob:oe]) ** 2).sum().backward()
        torch.testing.assert_close(local.grad, ref_in.grad[:, begin:end])
        # (b) every rank computes all outputs: the gradient arrives whole, no reduction
        local = full[:, begin:end].clone().requires_grad_()
        gathered = cdist.gather_columns_autograd(local, None, replicated_consumer=True)
        ((gathered @ weight.t() - target) ** 2).sum().backward()
        torch.testing.assert_close(local.grad, ref_in.grad[:, begin:end])
        # (c) a model is sharded only from 512 input columns up (and only when the columns divide)
        from compressgnn_b200.model import GCN
        for width, want in ((1024, True), (512, True), (256, False), (16, False), (513, False)):
            model = GCN(width, 5, hidden_features=16, param_H=4, use_transformation=True, num_layers=2)
            net, sharded = cdist.place_model(model, width)
            assert sharded == want and isinstance(net, cdist.ShardedGCN) == want and (sharded or net is model)
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_differentiable_column_gather_on_two_ranks():
    """The gather in front of the Linear of a column-sharded layer: forward is the concatenation,
    backward sums over ranks when the consumers differ and only slices when they are replicas."""
    world, port = 2, _free_port()
    mp.spawn(_gather_worker, args=(world, port), nprocs=world, join=True)
