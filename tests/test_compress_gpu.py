"""The device grammar compressor against the host compressor of this package: the two must return the
same arrays (the reference's tests/test_batch_compression.py:36-48 asks exactly that of its CPU and
CUDA back ends), and every vertex row must expand to its input row in order."""
import numpy as np
import pytest
import torch

from compressgnn_b200 import offline as off
from compressgnn_b200.loader import CompressgnnData, compress_graph_csr, resolve_backend

pytestmark = pytest.mark.gpu


def expand(v, e, node, n):
    stack = list(reversed(e[v[node]:v[node + 1]].tolist()))
    out = []
    while stack:
        child = stack.pop()
        if child < n:
            out.append(child)
        else:
            children = e[v[child]:v[child + 1]]
            assert np.all(children < child)
            stack.extend(reversed(children.tolist()))
    return out


def csr_of(rows):
    v = np.array([0] + list(np.cumsum([len(x) for x in rows])), dtype=np.int64)
    e = np.array([j for row in rows for j in row], dtype=np.int64)
    return v, e


def same(a, b):
    assert a[0].dtype == np.int32 and a[1].dtype == np.int32
    assert a[2] == b[2] and a[3] == b[3]
    np.testing.assert_array_equal(a[0], b[0])
    np.testing.assert_array_equal(a[1], b[1])


def test_backend_resolution_on_a_gpu():
    assert resolve_backend('auto') == 'cuda' and resolve_backend('cuda') == 'cuda' and resolve_backend('cpu') == 'cpu'


def test_fixtures_of_the_reference_test():
    rng = np.random.default_rng(17)
    fixtures = [[], [[]], [[0] * 50], [list(range(32)) for _ in range(64)]]
    fixtures += [[rng.integers(32, size=20).tolist() for _ in range(32)] for _ in range(4)]
    fixtures += [[[] for _ in range(5)], [[i] for i in range(7)], [[0, 1], [], [0, 1], [0, 1], [], [0, 1, 0, 1, 0, 1]]]
    for rows in fixtures:
        v, e = csr_of(rows)
        for frequency in [3, 16, 256]:
            host = compress_graph_csr(v, e, frequency, backend='cpu')
            device = compress_graph_csr(v, e, frequency, backend='cuda')
            same(device, host)
            dv, de, n, _ = device
            for node, row in enumerate(rows):
                assert expand(dv, de, node, n) == row


@pytest.mark.parametrize("rounds", [1, 2, 12])
@pytest.mark.parametrize("frequency", [3, 4, 16])
def test_web_graph_rows(rounds, frequency):
    """Rows with long shared runs and a few hubs (the copying-model generator of the benchmark), so that
    several rounds nest rules inside rules and the parse meets overlapping candidates."""
    v, e = off.generate_copy_graph(6000, alpha=2.1, x_min=5.3, max_degree=2000, copy_prob=0.7, window=64,
                                   candidates=8, seed=rounds + frequency)
    v, e = off.add_self_loop_csr(v, e)
    host = compress_graph_csr(v, e, frequency, backend='cpu', rounds=rounds)
    device = compress_graph_csr(v, e, frequency, backend='cuda', rounds=rounds)
    same(device, host)
    assert host[3] > 0
    dv, de, n, _ = device
    for node in range(0, n, 97):
        assert expand(dv, de, node, n) == e[v[node]:v[node + 1]].tolist()


def test_argument_errors():
    v, e = csr_of([[0, 1], [1, 5]])
    with pytest.raises(RuntimeError):
        compress_graph_csr(v, e, 3, backend='cuda')          # a value outside [0, n)
    with pytest.raises(ValueError):
        compress_graph_csr(*csr_of([[0]]), 2, backend='cuda')
    with pytest.raises(ValueError):
        compress_graph_csr(np.array([0, 1], np.int64), np.array([2**32], np.uint64), backend='cuda')
    with pytest.raises(ValueError):
        compress_graph_csr(np.array([0, 1]), np.array([0.5]), backend='cuda')
    from compressgnn_b200 import runtime as rt
    with pytest.raises(RuntimeError):
        rt.compress_csr_batch(torch.tensor([0, 2, 1], device="cuda"), torch.tensor([0, 0], device="cuda"))


def test_loader_builds_the_same_graph_with_either_back_end():
    n = 64
    v = np.arange(n + 1, dtype=np.int32) * 32
    e = np.tile(np.arange(32, dtype=np.int32), n)
    coo = np.vstack([np.repeat(np.arange(n, dtype=np.int32), 32), e])
    x = np.random.default_rng(3).standard_normal((n, 8)).astype(np.float32)
    mask = np.ones(n, dtype=bool)
    for graph_type, edge in [('coo', coo), ('csr', (v, e))]:
        for normalize in [False, True]:
            pieces = {}
            for backend in ['cpu', 'cuda']:
                data = CompressgnnData(x, edge, np.zeros(n, np.int64), mask, mask, mask, add_self_loop=False,
                                       normalize=normalize, graph_type=graph_type, compression_backend=backend)
                assert data.compression_backend == backend
                if graph_type == 'coo':
                    pieces[backend] = list(data.edge_index) + list(data.edge_weight)
                else:
                    g = data.edge_index
                    pieces[backend] = [part for blk in g.blocks() for part in blk.csr()]
            assert len(pieces['cpu']) == len(pieces['cuda'])
            assert all(torch.equal(a, b) for a, b in zip(pieces['cpu'], pieces['cuda']))
