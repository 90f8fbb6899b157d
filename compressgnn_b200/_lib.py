"""ctypes binding of ``libcgnn_b200.so`` (the C ABI declared in ``include/cgnn_b200.h``).

The library is the only compute path of this package: if it is missing the import fails
loudly -- there is no CPU or eager-PyTorch fallback.
"""
import ctypes
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "libcgnn_b200.so"

_c_i64 = ctypes.c_int64
_c_int = ctypes.c_int
_c_ptr = ctypes.c_void_p
_c_size = ctypes.c_size_t

# name -> (restype, argtypes); must list every symbol include/cgnn_b200.h declares.
SIGNATURES = {
    "cgnn_version": (_c_int, []),
    "cgnn_last_error": (ctypes.c_char_p, []),
    "cgnn_device_status": (_c_int, [ctypes.POINTER(_c_int)]),
    "cgnn_plan_create": (_c_int, [ctypes.POINTER(_c_ptr), _c_i64, _c_int, _c_ptr, _c_ptr, _c_i64,
                                  _c_ptr, _c_ptr, _c_i64, _c_int, _c_ptr]),
    "cgnn_plan_create_from_index": (_c_int, [ctypes.POINTER(_c_ptr), _c_ptr, _c_i64, _c_i64,
                                             _c_int, _c_ptr]),
    "cgnn_plan_destroy": (None, [_c_ptr]),
    "cgnn_plan_info": (_c_int, [_c_ptr, ctypes.POINTER(_c_i64)]),
    "cgnn_plan_source_rows": (_c_int, [_c_ptr, ctypes.POINTER(_c_i64)]),
    "cgnn_plan_degrees": (_c_int, [_c_ptr, ctypes.POINTER(_c_i64)]),
    "cgnn_plan_scratch_bytes": (_c_size, [_c_ptr, _c_i64, _c_int]),
    "cgnn_plan_ticket_bytes": (_c_size, [_c_ptr, _c_i64, _c_int]),
    "cgnn_spmm": (_c_int, [_c_ptr, _c_int, _c_i64, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr,
                           _c_size, _c_ptr]),
    "cgnn_spmm_static_scratch": (_c_int, [_c_ptr, _c_int, _c_i64, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr]),
    "cgnn_spmm_pair": (_c_int, [_c_ptr, _c_int, _c_i64, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int,
                                _c_ptr, _c_size, _c_ptr]),
    "cgnn_propagate": (_c_int, [_c_int, ctypes.POINTER(_c_ptr), ctypes.POINTER(_c_ptr), ctypes.POINTER(_c_ptr),
                                ctypes.POINTER(_c_size), _c_int, _c_i64, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int,
                                _c_int, _c_ptr]),
    "cgnn_plan_permute_values": (_c_int, [_c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr]),
    "cgnn_cluster_project": (_c_int, [_c_int, _c_ptr, _c_ptr, _c_i64, _c_i64, _c_int, _c_ptr,
                                      _c_ptr]),
    "cgnn_cluster_codes_from_projection": (_c_int, [_c_int, _c_ptr, _c_i64, _c_int, _c_ptr,
                                                    _c_ptr]),
    "cgnn_cluster_codes": (_c_int, [_c_int, _c_ptr, _c_ptr, _c_i64, _c_i64, _c_int, _c_ptr,
                                    _c_ptr]),
    "cgnn_cluster_workspace_bytes": (_c_size, [_c_i64, _c_int]),
    "cgnn_cluster_assign": (_c_int, [_c_ptr, _c_i64, _c_int, _c_ptr, _c_size, _c_ptr,
                                     ctypes.POINTER(_c_i64), _c_ptr]),
    "cgnn_cluster_assign_export": (_c_int, [_c_ptr, _c_i64, _c_i64, _c_ptr,
                                            ctypes.POINTER(_c_ptr), _c_int, _c_ptr]),
    "cgnn_cluster_mean": (_c_int, [_c_ptr, _c_int, _c_i64, _c_ptr, _c_ptr, _c_ptr, _c_ptr,
                                   _c_size, _c_ptr]),
    "cgnn_cluster_mean_backward": (_c_int, [_c_int, _c_i64, _c_i64, _c_i64, _c_ptr, _c_ptr,
                                            _c_ptr, _c_ptr, _c_ptr, _c_ptr]),
    "cgnn_cluster_reconstruct": (_c_int, [_c_int, _c_i64, _c_i64, _c_i64, _c_ptr, _c_ptr, _c_ptr,
                                          _c_int, _c_ptr, _c_ptr]),
    "cgnn_cluster_reconstruct_dropout": (_c_int, [_c_int, _c_i64, _c_i64, _c_i64, _c_ptr, _c_ptr, _c_ptr,
                                                  ctypes.c_double, ctypes.c_uint64, _c_ptr, _c_ptr]),
    "cgnn_cluster_reconstruct_backward": (_c_int, [_c_ptr, _c_int, _c_i64, _c_ptr, _c_ptr, _c_int,
                                                   _c_ptr, _c_ptr, _c_ptr, _c_size, _c_ptr]),
    "cgnn_sample_seed": (_c_int, [_c_ptr, _c_i64, _c_i64, _c_ptr, _c_ptr]),
    "cgnn_sample_count": (_c_int, [_c_ptr, _c_ptr, _c_i64, _c_i64, _c_i64, _c_ptr, _c_ptr]),
    "cgnn_sample_pick": (_c_int, [_c_ptr, _c_ptr, _c_i64, _c_i64, _c_i64, _c_ptr, _c_ptr, ctypes.c_uint32,
                                  ctypes.c_uint64, _c_ptr, _c_ptr, _c_ptr, _c_ptr]),
    "cgnn_sample_claim": (_c_int, [_c_ptr, _c_i64, _c_i64, _c_ptr, _c_ptr, _c_ptr, _c_ptr]),
    "cgnn_sample_relabel": (_c_int, [_c_ptr, _c_i64, _c_i64, _c_ptr, _c_ptr, _c_i64, _c_ptr, _c_ptr, _c_ptr,
                                     _c_ptr, _c_ptr]),
    "cgnn_compress_csr_batch": (_c_int, [_c_ptr, _c_ptr, _c_i64, _c_int, _c_int, _c_ptr, _c_ptr]),
    "cgnn_compressed_info": (_c_int, [_c_ptr, _c_ptr]),
    "cgnn_compressed_copy": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_ptr]),
    "cgnn_compressed_destroy": (None, [_c_ptr]),
}

_lib = None


def lib():
    """The loaded library; raises ImportError with build instructions when it is absent."""
    global _lib
    if _lib is None:
        if not LIB_PATH.is_file():
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m compressgnn_b200.build` "
                "(nvcc, sm_100a). compressgnn_b200 has no CPU or PyTorch fallback.")
        handle = ctypes.CDLL(str(LIB_PATH))
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError if the symbol is not exported
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib


def check(rc):
    """Turn a non-zero status into RuntimeError carrying the library's message (the
    reference's native argument errors are RuntimeError too: TORCH_CHECK)."""
    if rc != 0:
        msg = lib().cgnn_last_error()
        raise RuntimeError("cgnn_b200: " + (msg.decode() if msg else f"status {rc}"))
