"""The allocation-free SpMM entry point, called through the C ABI.

``cgnn_spmm_static_scratch`` is for hosts that cannot create a scratch buffer at call time (a
process whose own pool already owns the whole GPU, or a loop that must avoid the device-wide
synchronisation of cudaMalloc/cudaFree): it uses a buffer built into the library.  It must give
exactly what ``cgnn_spmm`` gives with caller scratch -- on back-to-back calls whose scratch
layouts differ, since the built-in buffer keeps the previous call's contents -- and must turn
down work that does not fit.  Collected last so that a failure here cannot hide another test's.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(seed, rows, src_rows, width, long_rows):
    rng = np.random.default_rng(seed)
    deg = rng.integers(0, 10, rows)
    for r, d in long_rows:
        deg[r] = d
    rowptr = np.zeros(rows + 1, np.int64)
    rowptr[1:] = np.cumsum(deg)
    col = rng.integers(0, src_rows, rowptr[-1]).astype(np.int64)
    val = rng.standard_normal(col.size).astype(np.float32)
    mat = rng.standard_normal((src_rows, width)).astype(np.float32)
    return [torch.from_numpy(a).cuda() for a in (rowptr, col, val, mat)]


def _both(rt, lib, rowptr, col, val, mat):
    plan = rt.SegmentPlan.from_csr(rowptr, col)
    assert plan.chunks > 0, "the case must exercise the scratch path"
    values = plan.values(val)
    width = mat.size(1)
    stream = torch.cuda.current_stream().cuda_stream
    scratch_ptr, scratch_bytes = plan.scratch(width, 0)
    expected = torch.empty(plan.rows, width, device="cuda")
    rt.check(lib.cgnn_spmm(plan.handle, 0, width, values.data_ptr(), mat.data_ptr(), expected.data_ptr(), 0,
                           scratch_ptr, scratch_bytes, stream))
    got = torch.full((plan.rows, width), float("nan"), device="cuda")
    rt.check(lib.cgnn_spmm_static_scratch(plan.handle, 0, width, values.data_ptr(), mat.data_ptr(),
                                          got.data_ptr(), 0, stream))
    torch.cuda.synchronize()
    return expected, got, plan


def test_static_scratch_matches_caller_scratch_on_consecutive_calls():
    from compressgnn_b200 import runtime as rt
    lib = rt.lib()
    # two calls in a row with different numbers of long rows and widths: the second call's
    # ticket words land where the first call left partial sums
    first = _both(rt, lib, *_case(1, 400, 300, 64, [(3, 900), (77, 300), (200, 129)]))
    second = _both(rt, lib, *_case(2, 900, 500, 128, [(r, 200 + r) for r in range(0, 900, 30)]))
    third = _both(rt, lib, *_case(1, 400, 300, 64, [(3, 900), (77, 300), (200, 129)]))
    for expected, got, _plan in (first, second, third):
        assert torch.equal(expected, got)  # same kernel, same order of partial sums: same bits
    # accumulate into an existing output as well
    rowptr, col, val, mat = _case(5, 300, 200, 32, [(0, 700)])
    plan = rt.SegmentPlan.from_csr(rowptr, col)
    base = torch.randn(plan.rows, 32, device="cuda")
    a, b = base.clone(), base.clone()
    sp, sb = plan.scratch(32, 0)
    stream = torch.cuda.current_stream().cuda_stream
    values = plan.values(val)
    rt.check(lib.cgnn_spmm(plan.handle, 0, 32, values.data_ptr(), mat.data_ptr(), a.data_ptr(), 1, sp, sb, stream))
    rt.check(lib.cgnn_spmm_static_scratch(plan.handle, 0, 32, values.data_ptr(), mat.data_ptr(), b.data_ptr(), 1,
                                          stream))
    assert torch.equal(a, b)
    assert rt.device_status() == 0


def test_static_scratch_rejects_what_does_not_fit():
    from compressgnn_b200 import runtime as rt
    lib = rt.lib()
    rows = 64
    rowptr = torch.arange(0, (rows + 1) * 4096, 4096, dtype=torch.int64, device="cuda")
    col = torch.zeros(rows * 4096, dtype=torch.int64, device="cuda")
    plan = rt.SegmentPlan.from_csr(rowptr, col)
    width = 1024  # 64 rows x 32 chunks x 4 KB of partial sums = 8 MiB, plus tickets: over the built-in 8 MiB
    mat = torch.ones(1, width, device="cuda")
    out = torch.zeros(rows, width, device="cuda")
    rc = lib.cgnn_spmm_static_scratch(plan.handle, 0, width, None, mat.data_ptr(), out.data_ptr(), 0,
                                      torch.cuda.current_stream().cuda_stream)
    assert rc == 1
    message = lib.cgnn_last_error().decode()
    assert "bytes of scratch" in message and "cgnn_spmm" in message
    torch.cuda.synchronize()
    assert not out.any()  # nothing ran
