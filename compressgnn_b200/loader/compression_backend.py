"""Backend choice for the grammar compressor (mirror of the reference's
``loader/compression_backend.py:6-40``).  Two compressors produce the same arrays: the host one in
``libcgnn_host.so`` (``'cpu'``) and the device one in ``libcgnn_b200.so`` (``'cuda'``,
``cgnn_compress_csr_batch``).  ``'auto'`` takes the device when one is usable, as the reference does
when its CUDA extension is installed."""
import operator

import numpy as np

from .. import offline


def _cuda_usable():
    try:
        import torch
        from .._lib import lib
        if not torch.cuda.is_available():
            return False
        lib()
        return True
    except (ImportError, OSError):
        return False


def resolve_backend(backend):
    if backend not in ('auto', 'cpu', 'cuda'):
        raise ValueError("compression_backend must be 'auto', 'cpu', or 'cuda'")
    if backend == 'cpu':
        return 'cpu'
    if _cuda_usable():
        return 'cuda'
    if backend == 'cuda':
        raise RuntimeError('CUDA compression requested but no usable CUDA device (or libcgnn_b200.so) is available')
    return 'cpu'


def _compress_on_device(vlist, elist, rounds, frequency):
    import torch
    from .. import runtime
    vlist, elist = offline._i64(vlist), offline._i64(elist)
    if vlist.size < 1 or (elist.size and (elist.max() > np.iinfo(np.int32).max or elist.min() < 0)):
        raise ValueError("CSR value exceeds int32 range")
    # Runtime failures (out of memory included) propagate; nothing falls back to the host.
    v, e, n, r = runtime.compress_csr_batch(torch.from_numpy(vlist).cuda(), torch.from_numpy(elist).cuda(),
                                            rounds=rounds, min_pair_frequency=frequency)
    return v.cpu().numpy(), e.cpu().numpy(), n, r


def compress_graph_csr(vlist, elist, min_pair_frequency=16, backend='auto', threads=4, rounds=12):
    frequency = operator.index(min_pair_frequency)
    threads = operator.index(threads)
    rounds = operator.index(rounds)
    if threads < 1 or rounds < 1:
        raise ValueError('compression_threads and compression_rounds must be positive')
    selected = resolve_backend(backend)
    if frequency < 3:
        raise ValueError('Batch compression needs min_pair_frequency >= 3')
    if selected == 'cuda':
        return _compress_on_device(vlist, elist, rounds, frequency)
    return offline.compress_csr_batch(vlist, elist, threads=threads, rounds=rounds,
                                      min_pair_frequency=frequency)
