"""Backend choice for the grammar compressor (mirror of the reference's
``loader/compression_backend.py:6-40``).  This package ships one compressor, a host (CPU)
implementation in ``libcgnn_host.so``; ``'auto'`` resolves to it and ``'cuda'`` is reported as
not installed, the way the reference reports a build without its CUDA compressor."""
import operator

from .. import offline


def resolve_backend(backend):
    if backend not in ('auto', 'cpu', 'cuda'):
        raise ValueError("compression_backend must be 'auto', 'cpu', or 'cuda'")
    if backend == 'cuda':
        raise RuntimeError('CUDA compression extension is not installed; this build compresses on the host')
    return 'cpu'


def compress_graph_csr(vlist, elist, min_pair_frequency=16, backend='auto', threads=4, rounds=12):
    frequency = operator.index(min_pair_frequency)
    threads = operator.index(threads)
    rounds = operator.index(rounds)
    if threads < 1 or rounds < 1:
        raise ValueError('compression_threads and compression_rounds must be positive')
    resolve_backend(backend)
    if frequency < 3:
        raise ValueError('Batch compression needs min_pair_frequency >= 3')
    return offline.compress_csr_batch(vlist, elist, threads=threads, rounds=rounds,
                                      min_pair_frequency=frequency)
