"""The C-ABI library loads without a GPU and exports every symbol include/cgnn_b200.h
declares; the ctypes signature table covers exactly those symbols."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def declared_symbols():
    text = (ROOT / "include" / "cgnn_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(cgnn_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_symbols()
    for required in ("cgnn_spmm", "cgnn_spmm_pair", "cgnn_plan_create", "cgnn_cluster_codes",
                     "cgnn_cluster_assign", "cgnn_cluster_mean", "cgnn_cluster_mean_backward",
                     "cgnn_cluster_reconstruct", "cgnn_cluster_reconstruct_backward",
                     "cgnn_cluster_project", "cgnn_last_error"):
        assert required in names


def test_library_exports_every_declared_symbol():
    from compressgnn_b200 import _lib
    if not _lib.LIB_PATH.is_file():
        from compressgnn_b200 import build
        build.build_cuda()
    handle = ctypes.CDLL(str(_lib.LIB_PATH))
    for name in declared_symbols():
        assert hasattr(handle, name), f"{name} declared in the header but not exported"
    assert sorted(_lib.SIGNATURES) == declared_symbols()
    lib = _lib.lib()
    assert lib.cgnn_version() >= 100
    assert lib.cgnn_cluster_workspace_bytes(1000, 16) > 6 * 4 * 1000


def test_argument_errors_need_no_gpu():
    """Validation happens on the host before any CUDA call."""
    from compressgnn_b200 import _lib
    lib = _lib.lib()
    plan = ctypes.c_void_p(0)
    rc = lib.cgnn_plan_create(ctypes.byref(plan), 4, 3, None, None, 0, None, None, 0, 0, None)
    assert rc == 1 and b"index_bytes" in lib.cgnn_last_error()
    rc = lib.cgnn_spmm(None, 0, 8, None, None, None, 0, None, 0, None)
    assert rc == 1
    rc = lib.cgnn_cluster_codes(0, None, None, 10, 4, 31, None, None)
    assert rc == 1
    with pytest.raises(RuntimeError):
        _lib.check(rc)
