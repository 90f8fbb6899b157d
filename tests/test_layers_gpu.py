"""The layer/ modules on the GPU: compressed propagation through autograd against the oracle,
the Compressgnn_Cluster state machine and the fused reconstruct against closed forms -- the
checks of the reference's tests/test_transformation.py:41-107 and the propagation smoke of
tests/test_batch_compression.py:89-120, on CUDA only (this package has no CPU path)."""
import numpy as np
import pytest
import torch

from conftest import assert_close_rel
from oracle import oracle

pytestmark = pytest.mark.gpu


def scatter_mean(x, index, dim_size):
    """sum / max(count, 1): the arithmetic of torch_scatter.scatter_mean the reference's tests
    compare with."""
    sums = torch.zeros(dim_size, x.size(1), dtype=x.dtype, device=x.device).index_add_(0, index, x)
    cnt = torch.bincount(index, minlength=dim_size).clamp_min(1).to(x.dtype)
    return sums / cnt[:, None]


def close(a, b):
    torch.testing.assert_close(a, b, atol=1e-5, rtol=1e-4)


def make_data(n=600, width=24, seed=3, **kw):
    from compressgnn_b200 import offline as off
    from compressgnn_b200.loader import CompressgnnData
    v, e = off.generate_copy_graph(n, 2.1, 4.0, 200, 0.7, 32, 8, seed=seed)
    x = np.random.default_rng(seed).standard_normal((n, width)).astype(np.float32)
    mask = np.ones(n, bool)
    opts = dict(min_pair_frequency=3, threshold=1, min_edge=10)
    opts.update(kw)
    return CompressgnnData(x, (v, e), np.zeros(n, np.int64), mask, mask, mask, **opts)


def oracle_blocks(graph):
    blocks = {k: tuple(t.cpu().numpy() for t in getattr(graph, f"{k}_graph").csr()) for k in ("v2v", "v2r", "r2v")}
    blocks["r2r"] = [tuple(t.cpu().numpy() for t in lvl.csr()) for lvl in graph.r2r_graph]
    return blocks


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("width", [1, 8, 24, 130, 256])
def test_propagation_forward_backward(dtype, width):
    from compressgnn_b200.layer import KPropagate, compress_spmm
    data = make_data(width=width)
    blocks = oracle_blocks(data.edge_index)
    n, r = data.vertex_cnt, data.rule_cnt
    assert r > 0 and data.edge_index.step >= 1
    data.to("cuda")
    x = data.x.to(dtype).detach().clone().requires_grad_()
    out = KPropagate()(x, data.edge_index, None, data.vertex_cnt, data.rule_cnt)
    xn = x.detach().cpu().numpy()
    assert_close_rel(out.detach().cpu().numpy(), oracle.propagate_forward(blocks, xn), what="forward")
    assert torch.equal(compress_spmm(data.edge_index, x.detach()), out.detach())
    go = torch.randn_like(out)
    (gx,) = torch.autograd.grad(out, x, go)
    assert_close_rel(gx.cpu().numpy(), oracle.propagate_backward(blocks, go.cpu().numpy(), n, r), what="backward")
    assert torch.isfinite(out).all() and torch.isfinite(gx).all()


def test_propagation_smoke_graph_of_the_reference_tests():
    """64 rows x identical 32-neighbour lists, F=8 (ref tests/test_batch_compression.py:89-120)."""
    from compressgnn_b200.layer import KPropagate
    from compressgnn_b200.loader import CompressgnnData
    n = 64
    v = np.arange(n + 1, dtype=np.int32) * 32
    e = np.tile(np.arange(32, dtype=np.int32), n)
    x = np.random.default_rng(17).standard_normal((n, 8)).astype(np.float32)
    mask = np.ones(n, bool)
    for normalize in (False, True):
        data = CompressgnnData(x, (v, e), np.zeros(n, np.int64), mask, mask, mask, add_self_loop=False,
                               normalize=normalize, graph_type="csr")
        blocks = oracle_blocks(data.edge_index)
        data.to("cuda")
        feats = data.x.detach().clone().requires_grad_()
        out = KPropagate()(feats, data.edge_index, None, data.vertex_cnt, data.rule_cnt)
        grad = torch.autograd.grad(out.square().sum(), feats)[0]
        ref = oracle.propagate_forward(blocks, x)
        assert_close_rel(out.detach().cpu().numpy(), ref, what="smoke forward")
        assert_close_rel(grad.cpu().numpy(),
                         oracle.propagate_backward(blocks, 2 * ref, n, data.rule_cnt), what="smoke backward")


def test_mean_and_reconstruct_gradcheck():
    from compressgnn_b200.layer import Compressgnn_Reconstruct, _Mean
    idx = torch.tensor([1, 1, 3, 1, 3, 3], device="cuda")
    count = torch.bincount(idx, minlength=5).int()
    x = torch.randn(6, 5, device="cuda", dtype=torch.double, requires_grad=True)
    assert torch.autograd.gradcheck(lambda a: _Mean.apply(a, idx, count), (x,), eps=1e-6, atol=1e-5, rtol=1e-3)
    reconstruct = Compressgnn_Reconstruct()
    reps = torch.randn(5, 3, device="cuda", dtype=torch.double, requires_grad=True)
    bias = torch.full((3,), 2., device="cuda", dtype=torch.double, requires_grad=True)
    assert torch.autograd.gradcheck(lambda a, b: reconstruct(a, idx, b, "relu"), (reps, bias), eps=1e-6,
                                    atol=1e-5, rtol=1e-3)
    for dtype in (torch.float32, torch.float64):
        for width in (1, 31, 33, 128, 602):
            for relu in (None, "relu"):
                reps = torch.randn(5, width, device="cuda", dtype=dtype, requires_grad=True)
                bias = torch.randn(width, device="cuda", dtype=dtype, requires_grad=True)
                out = reconstruct(reps, idx, bias=bias, activation=relu)
                ref = reps.index_select(0, idx) + bias
                if relu:
                    ref = ref.relu()
                close(out, ref)
                go = torch.randn_like(out)
                a = torch.autograd.grad(out, (reps, bias), go)
                b = torch.autograd.grad(ref, (reps, bias), go)
                close(a[0], b[0])
                close(a[1], b[1])
    with pytest.raises(ValueError):
        reconstruct(reps, idx, activation="gelu")


def test_cluster_epoch_reuse_and_cache_rules():
    from compressgnn_b200.layer import Compressgnn_Cluster, Compressgnn_Reconstruct
    device = "cuda"
    torch.manual_seed(26)
    c = Compressgnn_Cluster(7, 4, device=device, refresh_interval=5)
    ptr = None
    for epoch in range(12):
        x = torch.randn(19, 7, device=device, requires_grad=True)
        out, index = c(x, epoch=epoch, cache_key="graph-A")
        assert c.last_refreshed == (epoch % 5 == 0)
        if epoch % 5:
            assert index.data_ptr() == ptr
        ptr = index.data_ptr()
        ref = scatter_mean(x, index, out.size(0))
        close(out, ref)  # means follow the current features even when the assignment is reused
        close(torch.autograd.grad(out.square().sum(), x)[0], torch.autograd.grad(ref.square().sum(), x)[0])
    assert c.refresh_count == 3
    c.reset_cache()
    c.set_epoch(0)
    x = torch.randn(19, 7, device=device, requires_grad=True)
    _train_out, train_index = c(x)
    train_ptr = train_index.data_ptr()
    c.eval()
    _eval_out, eval_index = c(-x)
    assert eval_index.data_ptr() != train_ptr
    c.train()
    _out, index = c(x, epoch=1)
    assert not c.last_refreshed and index.data_ptr() == train_ptr  # separate train / eval caches
    c(x, epoch=1, cache_key="different-order")
    assert c.last_refreshed
    c(torch.randn(20, 7, device=device), epoch=1)
    assert c.last_refreshed
    c.random_vectors.add_(.01)
    c(x, epoch=1)
    assert c.last_refreshed
    c.load_state_dict(c.state_dict())
    c(x, epoch=1)
    assert c.last_refreshed
    c.double()
    c(x.double(), epoch=1)
    assert c.last_refreshed
    # an assignment saved for backward must survive a later refresh
    c = c.float()
    a = torch.randn(19, 7, device=device, requires_grad=True)
    b = torch.randn(19, 7, device=device, requires_grad=True)
    ya, ia = c(a, epoch=5)
    yb, ib = c(b, epoch=10)
    ra, rb = scatter_mean(a, ia, ya.size(0)), scatter_mean(b, ib, yb.size(0))
    ga = torch.autograd.grad(ya.square().sum() + yb.square().sum(), (a, b))
    gb = torch.autograd.grad(ra.square().sum() + rb.square().sum(), (a, b))
    close(ga[0], gb[0])
    close(ga[1], gb[1])
    # two shared transforms on the representatives, one reconstruction, all parameter gradients
    reconstruct = Compressgnn_Reconstruct()
    layers = torch.nn.Sequential(torch.nn.Linear(7, 9), torch.nn.ReLU(), torch.nn.Linear(9, 3)).to(device)
    x = torch.randn(19, 7, device=device, requires_grad=True)
    rep, ii = c(x, epoch=15)
    out = reconstruct(layers(rep), ii)
    ref = layers(scatter_mean(x, ii, rep.size(0))).index_select(0, ii)
    close(out, ref)
    params = [x] + list(layers.parameters())
    for p, q in zip(torch.autograd.grad(out.square().sum(), params), torch.autograd.grad(ref.square().sum(), params)):
        close(p, q)


def test_cluster_argument_rules():
    from compressgnn_b200.layer import Compressgnn_Cluster, Compressgnn_Cluster_Function
    c = Compressgnn_Cluster(7, 4, device="cuda", refresh_interval=5)
    with pytest.raises(ValueError):  # the call count is never used as the epoch
        c(torch.zeros(10, 7, device="cuda"))
    with pytest.raises(ValueError):
        c(torch.zeros(10, 8, device="cuda"), epoch=0)
    a = Compressgnn_Cluster(7, 4, device="cuda", refresh_policy="loss", q_min=1, q_max=10, tau_loss=.1)
    a.set_epoch(0, loss=1.)
    a.set_epoch(1, loss=1.)
    assert a.current_interval == 10
    a.set_epoch(2, loss=2.)
    assert a.current_interval == 1
    with pytest.raises(TypeError):
        a.set_epoch(3, loss=torch.tensor(1.))
    x = torch.randn(10, 7, device="cuda", requires_grad=True)
    y, ii, active = Compressgnn_Cluster_Function.apply(x, a.random_vectors, 4, True)
    ref = scatter_mean(x, ii, active + 1)
    close(y, ref)
    close(torch.autograd.grad(y.sum(), x)[0], torch.autograd.grad(ref.sum(), x)[0])
    for invalid in (-1, 31):
        with pytest.raises(ValueError):
            Compressgnn_Cluster(7, invalid)
    empty, idx = Compressgnn_Cluster(7, 4, device="cuda")(torch.zeros(0, 7, device="cuda"))
    assert empty.shape == (1, 7) and idx.numel() == 0
    legacy = Compressgnn_Cluster(7, 4, training=False, device="cuda")
    assert torch.is_tensor(legacy(torch.randn(5, 7, device="cuda")))
    with pytest.raises(RuntimeError):
        Compressgnn_Cluster(7, 4)(torch.randn(5, 7))  # CPU tensors: no fallback


def test_gcn_with_both_compressions_trains_one_step():
    """Config-1 shape: 2-layer GCN, hidden 64, 7 classes, propagation + transformation
    compression; the model equals the same weights applied in plain torch with a dense
    adjacency and the bucket assignment the modules chose, and one optimiser step runs."""
    from compressgnn_b200 import offline as off
    from compressgnn_b200.loader import CompressgnnData
    from compressgnn_b200.model import GCN
    n, width, classes = 2708, 128, 7
    v, e = off.generate_pa_graph(n, 5278, 0.3, seed=1)
    assert e.size == 10556
    rng = np.random.default_rng(1)
    x = rng.standard_normal((n, width)).astype(np.float32)
    y = rng.integers(0, classes, n)
    mask = np.ones(n, bool)
    data = CompressgnnData(x, (v, e), y, mask, mask, mask, min_pair_frequency=3, threshold=1, min_edge=10)
    assert data.rule_cnt > 0
    sv, se = off.add_self_loop_csr(v, e)
    nd = off.get_norm_degree(se, n)
    dense = torch.zeros(n, n, dtype=torch.float64)
    rows = np.repeat(np.arange(n), np.diff(sv))
    dense[torch.from_numpy(rows), torch.from_numpy(se)] = torch.from_numpy((nd[rows] * nd[se]).astype(np.float64))
    dense_t = dense.t().float().cuda()
    data.to("cuda")
    torch.manual_seed(0)
    model = GCN(width, classes, hidden_features=64, param_H=16, dropout=0.0, use_transformation=True,
                refresh_interval=5, num_layers=2).cuda()
    model.set_epoch(0)
    out = model(data.x, data.edge_index)

    def layer_ref(layer, feats):
        # the same arithmetic in plain torch, on the assignment the module chose
        p = dense_t @ feats
        index = layer.cluster.vertex_index
        reps = scatter_mean(p, index, layer.cluster.active_bucket + 1)
        return (reps @ layer.lin.weight.t()).index_select(0, index) + layer.lin.bias

    ref = torch.log_softmax(layer_ref(model.layers[1], layer_ref(model.layers[0], data.x).relu()), 1)
    torch.testing.assert_close(out, ref, atol=2e-4, rtol=1e-3)
    opt = torch.optim.Adam(model.parameters(), lr=1e-3)
    loss = torch.nn.functional.nll_loss(out[data.train_mask], data.y[data.train_mask])
    loss.backward()
    grads = [p.grad.clone() for p in model.parameters()]
    loss_ref = torch.nn.functional.nll_loss(ref, data.y)
    for g, gr in zip(grads, torch.autograd.grad(loss_ref, list(model.parameters()))):
        torch.testing.assert_close(g, gr, atol=2e-4, rtol=1e-3)
    opt.step()
    model.set_epoch(1)
    assert torch.isfinite(model(data.x, data.edge_index)).all()
    assert model.layers[0].cluster.refresh_count == 1  # reused at epoch 1


@pytest.mark.parametrize("width", [128, 256, 24, 6])
def test_reconstruct_with_fused_dropout(width):
    """The hidden-layer epilogue in one pass: dropout_p(relu(reps[index] + bias)).  Every output element is
    either 0 or the plain result divided by (1 - p); the mask depends on the seed only; the backward equals
    autograd through the same mask written out in plain torch."""
    from compressgnn_b200 import runtime as rt
    from compressgnn_b200.layer import Compressgnn_Reconstruct
    gen = torch.Generator(device="cuda").manual_seed(width)
    n, groups, p = 20000, 300, 0.3
    reps = torch.randn(groups, width, device="cuda", generator=gen)
    bias = torch.randn(width, device="cuda", generator=gen)
    index = torch.randint(1, groups, (n,), device="cuda", generator=gen)
    plain = rt.cluster_reconstruct(reps, index, bias, True)
    fused = rt.cluster_reconstruct(reps, index, bias, True, dropout_p=p, seed=1234)
    kept = fused != 0
    torch.testing.assert_close(fused[kept], plain[kept] / (1 - p), rtol=1e-6, atol=0)
    positive = plain > 0
    rate = 1.0 - (kept & positive).sum().item() / positive.sum().item()
    assert abs(rate - p) < 0.01, rate
    assert torch.equal(fused, rt.cluster_reconstruct(reps, index, bias, True, dropout_p=p, seed=1234))
    other = rt.cluster_reconstruct(reps, index, bias, True, dropout_p=p, seed=1235)
    assert (other != fused).float().mean().item() > 0.1
    # neighbouring elements are dropped independently: the drop rate of each column is close to p as well
    # (columns whose bias leaves fewer than 2000 positive elements say little and are left out)
    enough = positive.sum(0) >= 2000
    col_rate = 1.0 - (kept & positive).sum(0).float() / positive.sum(0).float().clamp_min(1)
    assert enough.sum().item() >= width // 2
    assert (col_rate - p).abs()[enough].max().item() < 0.05
    with pytest.raises(RuntimeError):
        rt.cluster_reconstruct(reps, index, bias, False, dropout_p=p)
    with pytest.raises(ValueError):
        Compressgnn_Reconstruct()(reps, index, bias=bias, activation=None, dropout=p)
    # autograd: the module against plain torch with the realised mask
    torch.manual_seed(7)
    src = reps.clone().requires_grad_()
    b = bias.clone().requires_grad_()
    out = Compressgnn_Reconstruct()(src, index, bias=b, activation="relu", dropout=p)
    go = torch.randn(n, width, device="cuda", generator=gen)
    g_src, g_b = torch.autograd.grad(out, (src, b), go)
    src2, b2 = reps.clone().requires_grad_(), bias.clone().requires_grad_()
    ref = (src2.index_select(0, index) + b2).relu() * (out != 0) / (1 - p)
    torch.testing.assert_close(out, ref, rtol=1e-6, atol=1e-6)
    r_src, r_b = torch.autograd.grad(ref, (src2, b2), go)
    torch.testing.assert_close(g_src, r_src, rtol=1e-4, atol=1e-4)
    # 20000 terms of magnitude ~1 per column, summed in two different orders in fp32; one wrongly masked
    # element would move a column by ~1
    torch.testing.assert_close(g_b, r_b, rtol=1e-4, atol=1e-2)


@pytest.mark.parametrize("width", [6, 64, 130])
def test_fused_dropout_in_double_precision(width):
    """The same epilogue on fp64 rows (two values per 16-byte vector, and the scalar path at odd widths)."""
    from compressgnn_b200 import runtime as rt
    gen = torch.Generator(device="cuda").manual_seed(width)
    n, groups, p = 5000, 40, 0.25
    reps = torch.randn(groups, width, device="cuda", dtype=torch.float64, generator=gen)
    bias = torch.randn(width, device="cuda", dtype=torch.float64, generator=gen)
    index = torch.randint(0, groups, (n,), device="cuda", generator=gen)
    plain = rt.cluster_reconstruct(reps, index, bias, True)
    fused = rt.cluster_reconstruct(reps, index, bias, True, dropout_p=p, seed=77)
    kept = fused != 0
    torch.testing.assert_close(fused[kept], plain[kept] / (1 - p), rtol=1e-14, atol=0)
    positive = plain > 0
    rate = 1.0 - (kept & positive).sum().item() / positive.sum().item()
    assert abs(rate - p) < 0.02, rate
    # the mask depends on (seed, element position) only, not on the element type
    single = rt.cluster_reconstruct(reps.float(), index, bias.float(), True, dropout_p=p, seed=77)
    agree = ((single != 0) == kept) | (plain.abs() < 1e-6)
    assert agree.all()


def test_gcn_training_mode_uses_the_fused_dropout():
    from compressgnn_b200.model import GCN
    data = make_data(n=3000, width=32)
    data.to("cuda")
    torch.manual_seed(0)
    model = GCN(32, 5, hidden_features=128, param_H=8, dropout=0.5, use_transformation=True, num_layers=2).cuda()
    model.set_epoch(0)
    hidden = []
    hook = model.layers[0].register_forward_hook(lambda m, i, o: hidden.append(o.detach()))
    out = model(data.x, data.edge_index)
    out.logsumexp(1).sum().backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in model.parameters())
    model.eval()
    model.inference(data.x, data.edge_index)
    hook.remove()
    train_zero, eval_zero = [(h == 0).float().mean().item() for h in hidden]
    assert train_zero > eval_zero + 0.15   # half of the surviving (positive) activations are dropped in training


def test_k_fold_propagation_with_cache():
    """KPUPropagate (ref: layer/KPUPropagate.py:25-37): K propagations in a row, and with
    cached=True the first result is kept and handed back detached whatever comes in later."""
    from compressgnn_b200.layer import KPUPropagate
    data = make_data(width=24)
    blocks = oracle_blocks(data.edge_index)
    data.to("cuda")
    x = data.x.clone().requires_grad_()
    twice = KPUPropagate(K=2)
    out = twice(x, data.edge_index, None, data.vertex_cnt, data.rule_cnt)
    ref = oracle.propagate_forward(blocks, oracle.propagate_forward(blocks, data.x.cpu().numpy()))
    assert_close_rel(out.detach().cpu().numpy(), ref, what="two propagations")
    (gx,) = torch.autograd.grad(out, x, torch.ones_like(out))
    ones = np.ones_like(ref)
    n, r = data.vertex_cnt, data.rule_cnt
    assert_close_rel(gx.cpu().numpy(), oracle.propagate_backward(blocks, oracle.propagate_backward(blocks, ones, n, r), n, r),
                     what="gradient through two propagations")
    assert twice(2 * x, data.edge_index, None, n, r).data_ptr() != out.data_ptr()  # no cache unless asked for
    cached = KPUPropagate(K=2, cached=True)
    first = cached(x, data.edge_index, None, n, r)
    second = cached(torch.zeros_like(x), data.edge_index, None, n, r)
    assert torch.equal(first, second) and not second.requires_grad
    cached.reset_cache()
    assert not cached(torch.zeros_like(x), data.edge_index, None, n, r).any()
    assert repr(cached) == "KPUPropagate(K=2)"


@pytest.mark.parametrize("depth", [1, 2, 3])
def test_host_propagation_queue_matches_resident_passes(depth):
    """Passes queued on host matrices (upload / propagate / download streams over a ring of
    device buffers) deliver the bits of the resident passes, whatever the ring depth, and the
    resident result matches the oracle."""
    from compressgnn_b200.layer import HostPropagation
    from compressgnn_b200.layer import spmm as spmm_layer
    data = make_data(n=3000, width=40)
    blocks = oracle_blocks(data.edge_index)
    data.to("cuda")
    graph = data.edge_index
    n = data.vertex_cnt
    pipe = HostPropagation(graph, 40, depth=depth)
    gen = torch.Generator().manual_seed(depth)
    sources = [torch.randn(n, 40, generator=gen).pin_memory() for _ in range(7)]
    results = [torch.full((n, 40), float("nan")).pin_memory() for _ in range(7)]
    events = []
    for i, (src, dst) in enumerate(zip(sources, results)):
        events.append(pipe.forward(src, dst) if i % 2 == 0 else pipe.backward(src, dst))
    events[2].synchronize()
    assert torch.equal(results[0], spmm_layer._forward(graph, sources[0].cuda()).cpu())
    pipe.synchronize()
    for i, (src, dst) in enumerate(zip(sources, results)):
        one_pass = spmm_layer._forward if i % 2 == 0 else spmm_layer._backward
        assert torch.equal(dst, one_pass(graph, src.cuda()).cpu()), f"pass {i}"
    assert_close_rel(results[0].numpy(), oracle.propagate_forward(blocks, sources[0].numpy()), what="forward")
    assert_close_rel(results[1].numpy(), oracle.propagate_backward(blocks, sources[1].numpy(), n, data.rule_cnt),
                     what="backward")
    with pytest.raises(RuntimeError):
        pipe.forward(sources[0][:, :8].contiguous(), results[0])
    with pytest.raises(RuntimeError):
        pipe.forward(sources[0].cuda(), results[0])
