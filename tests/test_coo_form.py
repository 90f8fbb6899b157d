"""The edge-list ("coo") form of the compressed graph: the phase schedule against the reference's
own gen_mask_edge (compiled into oracle/_ref when its sources are at hand) and a hand-worked case,
and -- on the GPU -- the phased propagation against the oracle's level-ordered SpMM on the same
compressed graph (ref: loader/CompressgnnData.py:86-139, layer/CompressgnnPropagation.py:68-83)."""
import numpy as np
import pytest
import torch

from compressgnn_b200 import offline as off
from compressgnn_b200.loader import CompressgnnData
from compressgnn_b200.loader.data import edge_phases
from conftest import assert_close_rel
from oracle import oracle


def small_graph(n=600, seed=3):
    v, e = off.generate_copy_graph(n, 2.1, 4.0, 200, 0.7, 32, 8, seed=seed)
    src = np.repeat(np.arange(n, dtype=np.int64), np.diff(v))
    return v, e, src


def test_phase_schedule_by_hand():
    # vertices 0..2, rules 3..5:  0,1 -> 3;  3,2 -> 4;  4 -> 5 and 4 -> 0;  5 -> 1;  a lone rule edge 3 -> 2
    src = np.array([0, 1, 3, 2, 4, 4, 5, 3])
    dst = np.array([3, 3, 4, 4, 5, 0, 1, 2])
    order, steps = edge_phases(src, dst, 3, 3)
    assert order.tolist() == [0, 0, 1, 0, 2, 2, 3, 1] and steps == 4
    order, steps = edge_phases(np.array([0, 1]), np.array([1, 0]), 2, 0)
    assert order.tolist() == [0, 0] and steps == 1


def test_phase_schedule_matches_the_compiled_reference():
    _rt, ref = oracle.reference_modules()
    if ref is None:
        pytest.skip("oracle/_ref is not built here")
    v, e, _src = small_graph()
    data = CompressgnnData(np.zeros((600, 1), np.float32), (v, e), np.zeros(600), *[np.ones(600, bool)] * 3,
                           min_pair_frequency=3, threshold=1, min_edge=10, max_depth=6)
    assert data.step >= 2
    # the compressed graph in edge-list form, as the reference's csr2coo emits it
    from compressgnn_b200.loader.data import compress
    sv, se = off.add_self_loop_csr(v, e)
    cv, ce, n, r = compress(sv, se, 1, 6, 10, 3)
    cv, ce = cv.astype(np.int32), ce.astype(np.int32)
    csrc = np.repeat(np.arange(n + r, dtype=np.int32), np.diff(cv))
    mask, steps = ref.gen_mask_edge(csrc, ce, int(n), int(r))
    order, mine = edge_phases(csrc, ce, int(n), int(r))
    assert mine == steps
    for phase in range(steps):
        np.testing.assert_array_equal(np.asarray(mask)[phase], order == phase)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_phased_propagation_matches_the_oracle(dtype):
    from compressgnn_b200.layer import KPropagate
    n, width = 600, 24
    v, e, src = small_graph(n)
    x = np.random.default_rng(3).standard_normal((n, width)).astype(np.float32)
    masks = [np.ones(n, bool)] * 3
    opts = dict(min_pair_frequency=3, threshold=1, min_edge=10, max_depth=6)
    coo = CompressgnnData(x, (src, e), np.zeros(n, np.int64), *masks, graph_type="coo", **opts)
    csr = CompressgnnData(x, (v, e), np.zeros(n, np.int64), *masks, graph_type="csr", **opts)
    assert coo.rule_cnt == csr.rule_cnt > 0 and coo.edge_cnt == csr.edge_cnt and coo.step >= 2
    assert len(coo.edge_index) == coo.step == len(coo.edge_weight)
    assert sum(p.size(1) for p in coo.edge_index) == coo.edge_cnt
    g = csr.edge_index
    blocks = {k: tuple(t.numpy() for t in getattr(g, f"{k}_graph").csr()) for k in ("v2v", "v2r", "r2v")}
    blocks["r2r"] = [tuple(t.numpy() for t in lvl.csr()) for lvl in g.r2r_graph]
    coo.to("cuda")
    xd = coo.x.to(dtype).requires_grad_()
    out = KPropagate()(xd, coo.edge_index, coo.edge_weight, coo.vertex_cnt, coo.rule_cnt)
    assert out.shape == (n, width)
    xn = xd.detach().cpu().numpy()
    assert_close_rel(out.detach().cpu().numpy(), oracle.propagate_forward(blocks, xn), what="phased forward")
    go = torch.randn_like(out)
    (gx,) = torch.autograd.grad(out, xd, go)
    assert_close_rel(gx.cpu().numpy(), oracle.propagate_backward(blocks, go.cpu().numpy(), n, coo.rule_cnt),
                     what="phased backward")
    # the same call again reuses the grouped phases and returns the same bits
    again = KPropagate()(xd, coo.edge_index, coo.edge_weight, coo.vertex_cnt, coo.rule_cnt)
    assert torch.equal(again, out)
    with pytest.raises(RuntimeError):
        KPropagate()(xd.cpu(), coo.edge_index, coo.edge_weight, coo.vertex_cnt, coo.rule_cnt)
