"""Drop-in for the reference's pybind module ``compressgnn_runtime``.

Same eight function names, argument meaning, return contracts and error classes as
``src/runtime/csrc/function.cpp:9-21`` of ZhengChenCS/CompressGNN, implemented by passing
raw device pointers to the C ABI in ``include/cgnn_b200.h``.  CUDA tensors only: there is
no CPU path.

Two things the reference does not have are kept out of the callers' sight:

* **Segment plans.**  The kernels want 32-bit indices and a work decomposition by row
  degree.  ``spmm_func`` builds that once per ``(vlist, elist)`` tensor pair and caches it
  for as long as both tensors live and stay unmodified; ``cluster_assign`` keeps the bucket
  permutation it produced next to the returned index tensor, so ``cluster_mean`` and
  ``cluster_reconstruct_backward`` (which receive only ``index``) find it again.
* **Scratch.**  Rows longer than the plan's split leave partial sums in a zero-initialised
  torch buffer owned by the plan, one per (width, dtype, stream).  Launches on one plan
  from two streams at the same time would race on it.
"""
import ctypes
import weakref
from collections import OrderedDict

import torch

from ._lib import check, lib  # noqa: F401  (lib is re-exported for the layer modules)

_METHODS = ("rowbalance_parreduce", "rowbalance_seqreduce", "rowbalance_rowcache",
            "nnzbalance_parreduce", "nnzbalance_seqreduce", "nnzbalance_rowcache")
INT_MAX = 2**31 - 1


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None and t.numel() else ctypes.c_void_p(0)


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream_ptr(device):
    """The current CUDA stream of ``device`` as the integer the C ABI takes."""
    if _raw_stream is not None:  # no Stream object per call: a training epoch asks a hundred times
        device = torch.device(device)
        return _raw_stream(device.index if device.index is not None else torch.cuda.current_device())
    return torch.cuda.current_stream(device).cuda_stream


class on_device:
    """``with on_device(d):`` makes ``d`` the current CUDA device for the native calls inside, like
    ``torch.cuda.device(d)``, but does nothing at all when it already is (the usual case)."""
    __slots__ = ("index", "previous")

    def __init__(self, device):
        device = torch.device(device)
        self.index = device.index if device.index is not None else torch.cuda.current_device()
        self.previous = -1

    def __enter__(self):
        current = torch.cuda.current_device()
        if current != self.index:
            self.previous = current
            torch.cuda.set_device(self.index)
        return self

    def __exit__(self, *exc):
        if self.previous >= 0:
            torch.cuda.set_device(self.previous)
            self.previous = -1
        return False


def _dtype_code(t, what="tensor"):
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.float64:
        return 1
    raise RuntimeError(f"{what}: only float32 and float64 are supported")


def _dtype_code_of(dtype):
    if dtype == torch.float32:
        return 0
    if dtype == torch.float64:
        return 1
    raise RuntimeError("only float32 and float64 are supported")


def _require(cond, msg):
    if not cond:
        raise RuntimeError(msg)


class SegmentPlan:
    """Owner of a native ``cgnn_plan`` and of its scratch buffers."""

    def __init__(self, handle, device):
        self._handle = handle
        self.device = device
        self._scratch = {}
        self._values = _TensorKeyedCache(limit=8)
        info = (ctypes.c_int64 * 8)()
        check(lib().cgnn_plan_info(handle, info))
        (self.rows, self.nnz, self.split, self.long_rows, self.chunks, self.direct_units,
         self.terms, self.compact_rows) = [int(v) for v in info]
        need = (ctypes.c_int64 * 2)()
        check(lib().cgnn_plan_source_rows(handle, need))
        self.source_rows = (int(need[0]), int(need[1]))  # rows each source matrix must have
        hist = (ctypes.c_int64 * 4)()
        check(lib().cgnn_plan_degrees(handle, hist))
        self.degree_p50, self.degree_p99, self.degree_max = int(hist[0]), int(hist[1]), int(hist[2])

    @property
    def handle(self):
        return ctypes.c_void_p(self._handle)

    @classmethod
    def from_csr(cls, rowptr, col, rowptr1=None, col1=None, split=0):
        """Plan over one CSR block, or over two blocks that share their rows."""
        device = rowptr.device
        _require(rowptr.is_cuda and col.device == device, "plan: CSR arrays must be on one CUDA device")
        _require(rowptr.dtype == col.dtype and rowptr.dtype in (torch.int32, torch.int64),
                 "plan: CSR arrays must be int32 or int64")
        rowptr, col = rowptr.contiguous(), col.contiguous()
        if rowptr1 is not None:
            _require(rowptr1.dtype == rowptr.dtype and col1.dtype == rowptr.dtype and
                     rowptr1.numel() == rowptr.numel() and rowptr1.device == device and
                     col1.device == device, "plan: the two blocks must share rows, dtype and device")
            rowptr1, col1 = rowptr1.contiguous(), col1.contiguous()
        handle = ctypes.c_void_p(0)
        with on_device(device):
            check(lib().cgnn_plan_create(
                ctypes.byref(handle), rowptr.numel() - 1, rowptr.element_size(),
                ctypes.c_void_p(rowptr.data_ptr()), _ptr(col), col.numel(),
                ctypes.c_void_p(rowptr1.data_ptr()) if rowptr1 is not None else None,
                _ptr(col1) if col1 is not None else None,
                col1.numel() if col1 is not None else 0, int(split), _stream_ptr(device)))
        return cls(handle.value, device)

    built_from_index = 0  # plans built by a sort of the index (the path an assignment refresh does not take)

    @classmethod
    def from_index(cls, index, groups, split=0):
        """Plan that groups the positions of ``index`` by value (``groups`` segments)."""
        _require(index.is_cuda and index.dtype == torch.int64 and index.dim() == 1 and
                 index.is_contiguous(), "Expected contiguous int64 index on input device")
        SegmentPlan.built_from_index += 1
        handle = ctypes.c_void_p(0)
        with on_device(index.device):
            check(lib().cgnn_plan_create_from_index(ctypes.byref(handle), _ptr(index), index.numel(),
                                                    int(groups), int(split),
                                                    _stream_ptr(index.device)))
        return cls(handle.value, index.device)

    def values(self, val0, val1=None):
        """``val0`` (and ``val1`` of the second block) brought into the plan's entry order; the
        result is cached for as long as the given tensors live and stay unmodified."""
        tensors = (val0,) if val1 is None else (val0, val1)
        cached = self._values.get(tensors)
        if cached is None:
            _require(sum(t.numel() for t in tensors) == self.nnz, "values do not match the plan's entries")
            cached = torch.empty(self.nnz, dtype=val0.dtype, device=self.device)
            if self.nnz:
                with on_device(self.device):
                    check(lib().cgnn_plan_permute_values(
                        self.handle, _dtype_code(val0, "values"), _ptr(val0.contiguous()),
                        _ptr(val1.contiguous()) if val1 is not None else None, _ptr(cached),
                        _stream_ptr(self.device)))
            self._values.put(tensors, cached)
        return cached

    def scratch(self, width, dtype_code):
        """(pointer, bytes) of this plan's scratch for launches ``width`` columns wide on the
        current stream; allocated zeroed on first use (the ticket words must start at 0)."""
        key = (int(width), dtype_code, _stream_ptr(self.device))
        buf = self._scratch.get(key)
        if buf is None:
            nbytes = lib().cgnn_plan_scratch_bytes(self.handle, int(width), dtype_code)
            buf = torch.zeros(max(int(nbytes), 16), dtype=torch.uint8, device=self.device)
            self._scratch[key] = buf
        return ctypes.c_void_p(buf.data_ptr()), buf.numel()

    def __del__(self):
        handle, self._handle = getattr(self, "_handle", None), None
        if handle:
            try:
                lib().cgnn_plan_destroy(ctypes.c_void_p(handle))
            except Exception:  # interpreter shutdown
                pass


class _TensorKeyedCache:
    """Values attached to a tuple of live, unmodified tensors (identity + ``_version``)."""

    def __init__(self, limit=256):
        self._items = OrderedDict()
        self._limit = limit

    def get(self, tensors, extra=()):
        key = tuple(id(t) for t in tensors) + tuple(extra)
        hit = self._items.get(key)
        if hit is None:
            return None
        refs, versions, value = hit
        if all(r() is t for r, t in zip(refs, tensors)) and \
                versions == tuple(t._version for t in tensors):
            self._items.move_to_end(key)
            return value
        del self._items[key]
        return None

    def put(self, tensors, value, extra=()):
        key = tuple(id(t) for t in tensors) + tuple(extra)
        items = self._items

        def _drop(_ref, key=key):
            items.pop(key, None)

        self._items[key] = (tuple(weakref.ref(t, _drop) for t in tensors),
                            tuple(t._version for t in tensors), value)
        while len(self._items) > self._limit:
            self._items.popitem(last=False)

    def clear(self):
        self._items.clear()


_csr_plans = _TensorKeyedCache()
_index_plans = _TensorKeyedCache()


def clear_plan_caches():
    """Drop every cached plan (frees their device memory once unreferenced)."""
    _csr_plans.clear()
    _index_plans.clear()


def csr_plan(vlist, elist):
    plan = _csr_plans.get((vlist, elist))
    if plan is None:
        plan = SegmentPlan.from_csr(vlist, elist)
        _csr_plans.put((vlist, elist), plan)
    return plan


def index_plan(index, groups):
    plan = _index_plans.get((index,), (int(groups),))
    if plan is None:
        plan = SegmentPlan.from_index(index, groups)
        _index_plans.put((index,), plan, (int(groups),))
    return plan


# -----------------------------------------------------------------------------------------
# spmm_func  (ref: src/runtime/csrc/sparse/spmm.cpp:11-23, cuda/spmm_gpu.cu:8-107)
# -----------------------------------------------------------------------------------------
def spmm_with_plan(plan, value, mat, out=None, accumulate=False):
    """``out (+)= A @ mat`` for the CSR block behind ``plan``; ``value`` is the block's value
    array in its original CSR order, or None (ones)."""
    code = _dtype_code(mat, "spmm")
    width = mat.size(-1)
    if out is None:
        out = torch.empty((plan.rows, width), dtype=mat.dtype, device=mat.device)
        accumulate = False
    if out.numel() == 0:
        return out
    if plan.nnz == 0:
        return out if accumulate else out.zero_()
    _require(mat.size(0) >= plan.source_rows[0],
             f"spmm: the index array refers to row {plan.source_rows[0] - 1} but mat has {mat.size(0)} rows")
    sp, sb = plan.scratch(width, code)
    if value is not None:
        value = plan.values(value)
    with on_device(mat.device):
        check(lib().cgnn_spmm(plan.handle, code, width, _ptr(value), _ptr(mat), _ptr(out),
                              1 if accumulate else 0, sp, sb, _stream_ptr(mat.device)))
    return out


def empty_row_aligned(rows, like):
    """A ``[rows, like.size(1)]`` tensor whose first row starts a whole number of rows away from
    ``like``'s first row, so that the fused two-block pass can address both with one base
    pointer and a row index (see ``cgnn_spmm_pair``)."""
    width = like.size(1)
    buf = torch.empty(rows * width + width, dtype=like.dtype, device=like.device)
    row_bytes = width * like.element_size()
    shift = ((like.data_ptr() - buf.data_ptr()) % row_bytes) // like.element_size() if row_bytes else 0
    return buf[shift:shift + rows * width].view(rows, width)


def spmm_pair_with_plan(plan, value0, mat0, value1, mat1, out=None, accumulate=False):
    """``out (+)= A0 @ mat0 + A1 @ mat1`` in one pass (plan built over both blocks)."""
    code = _dtype_code(mat0, "spmm")
    width = mat0.size(-1)
    _require(mat1.size(-1) == width and mat1.dtype == mat0.dtype, "spmm_pair: operand mismatch")
    if out is None:
        out = torch.empty((plan.rows, width), dtype=mat0.dtype, device=mat0.device)
        accumulate = False
    if out.numel() == 0:
        return out
    for which, mat in enumerate((mat0, mat1)):
        _require(mat.size(0) >= plan.source_rows[which],
                 f"spmm_pair: block {which} refers to row {plan.source_rows[which] - 1} but its matrix has "
                 f"{mat.size(0)} rows")
    sp, sb = plan.scratch(width, code)
    value = plan.values(value0, value1)
    with on_device(mat0.device):
        check(lib().cgnn_spmm_pair(plan.handle, code, width, _ptr(value), _ptr(mat0), _ptr(mat1),
                                   _ptr(out), 1 if accumulate else 0, sp, sb,
                                   _stream_ptr(mat0.device)))
    return out


def propagate_pass(table, x, rule_out, out, first=0, last=None):
    """Issue the launches ``first .. last`` of one propagation direction (``table`` from
    ``PropagationPlan.whole_pass``) in one native call: rules gather from ``x`` into ``rule_out``, the
    rule levels run in place, the fused vertex pass writes ``out``."""
    n_rules, (need0, need1) = table["source_rows"]
    rule_side, x_side = (need0, need1) if table["rule_term"] == 0 else (need1, need0)
    _require(x.size(0) >= max(n_rules, x_side) and rule_out.size(0) >= rule_side,
             "propagate: the graph refers to rows beyond the feature or rule matrix")
    check(lib().cgnn_propagate(table["n"], table["plans"], table["vals"], table["scratch"], table["scratch_bytes"],
                               table["code"], x.size(1), x.data_ptr(), rule_out.data_ptr() if rule_out.numel() else None,
                               out.data_ptr(), table["rule_term"], first, table["n"] - 1 if last is None else last,
                               table["stream"]))
    return out


def spmm_func(vlist, elist, value, mat, method, optional_out=None):
    """``out = A @ mat`` with A given as CSR ``(vlist, elist, value)``.

    If ``optional_out`` is given it is accumulated into in place and returned, else a new
    ``[rows, F]`` tensor is returned.  ``method`` must be one of the reference's six CUDA
    kernel names; all of them run the same degree-aware kernel here (the name is a hint the
    plan does not need).
    """
    for name, t in (("vlist", vlist), ("elist", elist), ("value", value), ("mat", mat)):
        _require(t.is_cuda, f"{name} must be GPU tensor")
    _require(mat.is_contiguous(), "mat must be contiguous")
    if optional_out is not None:
        _require(optional_out.is_cuda, "optional_out must be GPU tensor")
        # accumulated in place and returned: a silent contiguous copy would break that contract
        _require(optional_out.is_contiguous(), "optional_out must be contiguous")
        out = optional_out
    else:
        sizes = list(mat.shape)
        sizes[0] = vlist.size(-1) - 1
        out = None
    _require(method in _METHODS, f"Invalid SpMM method for CUDA: {method}")
    _require(mat.dim() == 2, "mat must be a matrix")
    _require(value.dtype == mat.dtype, "value and mat must have the same dtype")
    if elist.numel() == 0 or (out is not None and out.numel() == 0):
        return out if out is not None else torch.zeros(sizes, dtype=mat.dtype, device=mat.device)
    plan = csr_plan(vlist, elist)
    if out is not None:
        _require(out.shape == (plan.rows, mat.size(1)) and out.dtype == mat.dtype,
                 "optional_out has the wrong shape or dtype")
    return spmm_with_plan(plan, value.contiguous(), mat, out, accumulate=out is not None)


# -----------------------------------------------------------------------------------------
# cluster_*  (ref: src/runtime/csrc/cluster/cuda/cluster_kernel.cu:111-208)
# -----------------------------------------------------------------------------------------
def _check_float(x, what="Expected contiguous CUDA matrix"):
    _require(x.is_cuda and x.dim() == 2 and x.is_contiguous(), what)
    _require(x.dtype in (torch.float32, torch.float64), "Only float32 and float64 are supported")


def _check_index(index, device):
    _require(index.device == device and index.dim() == 1 and index.is_contiguous() and
             index.dtype == torch.int64, "Expected contiguous int64 index on input device")


def _check_count(count, device):
    _require(count.device == device and count.dim() == 1 and count.is_contiguous() and
             count.dtype == torch.int32 and count.numel() >= 1,
             "Expected nonempty int32 counts on input device")


def _bits(bits):
    bits = int(bits)
    _require(0 <= bits <= 30, "Hash bits must be in [0,30]")
    return bits


def cluster_workspace(input, bits):
    """Workspace for ``cluster_assign`` on ``input``'s device: a list of three tensors
    ``[int32, int32, uint8]`` like the reference's.  The byte buffer is sized for
    ``input.size(0)`` rows (sort buffers, not a 2^bits histogram)."""
    _check_float(input)
    bits = _bits(bits)
    nbytes = lib().cgnn_cluster_workspace_bytes(int(input.size(0)), bits)
    ints = dict(dtype=torch.int32, device=input.device)
    return [torch.tensor([input.size(0), bits], **ints), torch.empty(0, **ints),
            torch.empty(int(nbytes), dtype=torch.uint8, device=input.device)]


def project(input, planes):
    """``input @ planes`` in the kernel's fixed accumulation order (column-sharded path)."""
    _check_float(input)
    _check_float(planes)
    bits = _bits(planes.size(1))
    _require(planes.device == input.device and planes.dtype == input.dtype and
             planes.size(0) == input.size(1), "Hash plane shape/device/dtype mismatch")
    proj = torch.empty((input.size(0), bits), dtype=input.dtype, device=input.device)
    with on_device(input.device):
        check(lib().cgnn_cluster_project(_dtype_code(input), _ptr(input), _ptr(planes),
                                         input.size(0), input.size(1), bits, _ptr(proj),
                                         _stream_ptr(input.device)))
    return proj


def _assign_from_codes(codes, n, bits, workspace, device):
    ws = workspace[2]
    need = lib().cgnn_cluster_workspace_bytes(n, bits)
    _require(ws.device == device and ws.dtype == torch.uint8 and ws.dim() == 1 and
             ws.is_contiguous() and ws.numel() >= need, "Workspace dtype/capacity mismatch")
    ids = torch.empty(n, dtype=torch.int64, device=device)
    active = ctypes.c_int64(0)
    stream = _stream_ptr(device)
    check(lib().cgnn_cluster_assign(_ptr(codes), n, bits, _ptr(ws), ws.numel(), _ptr(ids),
                                    ctypes.byref(active), stream))
    active = int(active.value)
    counts = torch.empty(active + 1, dtype=torch.int32, device=device)
    handle = ctypes.c_void_p(0)
    check(lib().cgnn_cluster_assign_export(_ptr(ws), n, active, _ptr(counts), ctypes.byref(handle),
                                           0, stream))
    plan = SegmentPlan(handle.value, device)
    _index_plans.put((ids,), plan, (active + 1,))
    return ids, counts, active


def _check_assign_args(input, planes, bits, workspace):
    _check_float(input)
    _check_float(planes)
    bits = _bits(bits)
    _require(planes.device == input.device and planes.dtype == input.dtype and
             planes.size(0) == input.size(1) and planes.size(1) == bits,
             "Hash plane shape/device/dtype mismatch")
    _require(input.size(0) <= INT_MAX, "Node count exceeds int32 bucket count capacity")
    _require(isinstance(workspace, (list, tuple)) and len(workspace) == 3,
             "Expected bucket, prefix and scan workspaces")
    for w in workspace:
        _require(torch.is_tensor(w) and w.device == input.device and w.dim() == 1 and
                 w.is_contiguous(), "Workspace device/shape mismatch")
    return bits


def cluster_assign(input, planes, bits, workspace):
    """``(ids int64[N], counts int32[active+1], active)``: 1-based dense bucket ids that
    ascend with the raw sign code, ``counts[0] == 0``."""
    bits = _check_assign_args(input, planes, bits, workspace)
    n, device = input.size(0), input.device
    if n == 0:
        return (torch.empty(0, dtype=torch.int64, device=device),
                torch.zeros(1, dtype=torch.int32, device=device), 0)
    with on_device(device):
        codes = torch.empty(n, dtype=torch.int32, device=device)
        check(lib().cgnn_cluster_codes(_dtype_code(input), _ptr(input), _ptr(planes), n,
                                       input.size(1), bits, _ptr(codes), _stream_ptr(device)))
        return _assign_from_codes(codes, n, bits, workspace, device)


def cluster_assign_from_projection(proj, workspace):
    """Same as ``cluster_assign`` but starting from an already reduced ``[N, bits]``
    projection (the column-sharded path sums partial projections across GPUs first)."""
    _check_float(proj)
    n, bits, device = proj.size(0), _bits(proj.size(1)), proj.device
    if n == 0:
        return (torch.empty(0, dtype=torch.int64, device=device),
                torch.zeros(1, dtype=torch.int32, device=device), 0)
    with on_device(device):
        codes = torch.empty(n, dtype=torch.int32, device=device)
        check(lib().cgnn_cluster_codes_from_projection(_dtype_code(proj), _ptr(proj), n, bits,
                                                       _ptr(codes), _stream_ptr(device)))
        return _assign_from_codes(codes, n, bits, workspace, device)


def cluster_forward(input, random_vectors, param_h):
    """Legacy entry: ``(int32 ids[N], active)`` (ref: cluster/cluster.cpp:12-30)."""
    _require(input.dim() == 2 and random_vectors.dim() == 2 and input.is_contiguous() and
             random_vectors.is_contiguous(), "Expected contiguous matrices")
    _require(0 <= int(param_h) <= 30 and random_vectors.size(0) == input.size(1) and
             random_vectors.size(1) == param_h, "Invalid hash plane shape/bits")
    _require(input.device == random_vectors.device and input.dtype == random_vectors.dtype,
             "Hash device/dtype mismatch")
    _require(input.dtype in (torch.float32, torch.float64), "Expected float32/float64 features")
    _require(input.is_cuda, "compressgnn_b200 has no CPU path")
    ids, _counts, active = cluster_assign(input, random_vectors, param_h,
                                          cluster_workspace(input, param_h))
    return ids.to(torch.int32), active


def cluster_mean(input, index, count, plan=None):
    """``out[g] = mean of input rows with index == g`` (zero for empty groups)."""
    _check_float(input)
    _check_index(index, input.device)
    _check_count(count, input.device)
    _require(index.numel() == input.size(0), "Input/index length mismatch")
    groups, width = count.numel(), input.size(1)
    out = torch.empty((groups, width), dtype=input.dtype, device=input.device)
    if input.numel() == 0:
        return out.zero_()
    if plan is None:
        plan = index_plan(index, groups)
    _require(plan.rows == groups and plan.nnz == index.numel(), "cluster_mean: plan does not match index/count")
    code = _dtype_code(input)
    sp, sb = plan.scratch(width, code)
    with on_device(input.device):
        check(lib().cgnn_cluster_mean(plan.handle, code, width, _ptr(input), _ptr(count), _ptr(out),
                                      sp, sb, _stream_ptr(input.device)))
    return out


def cluster_mean_backward(grad, index, count):
    """``out[r] = grad[index[r]] / max(count[index[r]], 1)``."""
    _check_float(grad)
    _check_index(index, grad.device)
    _check_count(count, grad.device)
    _require(grad.size(0) == count.numel(), "Gradient/count shape mismatch")
    out = torch.empty((index.numel(), grad.size(1)), dtype=grad.dtype, device=grad.device)
    if out.numel() == 0:
        return out
    with on_device(grad.device):
        scaled = torch.empty_like(grad)  # grad / count, divided once per group row
        check(lib().cgnn_cluster_mean_backward(_dtype_code(grad), index.numel(), grad.size(1),
                                               grad.size(0), _ptr(grad), _ptr(index), _ptr(count),
                                               _ptr(out), _ptr(scaled), _stream_ptr(grad.device)))
    return out


def cluster_reconstruct(reps, index, bias, relu, dropout_p=0.0, seed=0):
    """``out[r] = act(reps[index[r]] + bias)``; ``bias`` may be None.  With ``dropout_p > 0`` (ReLU only)
    the same pass also drops elements with that probability and scales the survivors by
    ``1 / (1 - dropout_p)``; the mask is a function of ``(seed, element position)``."""
    _check_float(reps)
    _check_index(index, reps.device)
    if bias is not None:
        _require(bias.device == reps.device and bias.dtype == reps.dtype and bias.dim() == 1 and
                 bias.numel() == reps.size(1) and bias.is_contiguous(),
                 "Invalid reconstruction bias")
    out = torch.empty((index.numel(), reps.size(1)), dtype=reps.dtype, device=reps.device)
    if out.numel() == 0:
        return out
    dropout_p = float(dropout_p)
    _require(0.0 <= dropout_p < 1.0, "dropout probability must lie in [0, 1)")
    _require(dropout_p == 0.0 or relu, "the fused dropout follows a ReLU (the backward reads its mask off the zeros)")
    with on_device(reps.device):
        if dropout_p > 0.0:
            check(lib().cgnn_cluster_reconstruct_dropout(
                _dtype_code(reps), index.numel(), reps.size(1), reps.size(0), _ptr(reps), _ptr(index), _ptr(bias),
                dropout_p, int(seed) & (2**64 - 1), _ptr(out), _stream_ptr(reps.device)))
        else:
            check(lib().cgnn_cluster_reconstruct(_dtype_code(reps), index.numel(), reps.size(1),
                                                 reps.size(0), _ptr(reps), _ptr(index), _ptr(bias),
                                                 1 if relu else 0, _ptr(out),
                                                 _stream_ptr(reps.device)))
    return out


def cluster_reconstruct_backward(grad, index, output, groups, relu, plan=None,
                                 return_bias_grad=False, output_is_forward_result=False):
    """``d_reps[g] = sum over rows r with index[r] == g of (relu and output[r] <= 0 ? 0 :
    grad[r])``.  With ``return_bias_grad`` also returns the column sums of ``d_reps`` (the
    bias gradient), computed in the same call.  ``output_is_forward_result`` promises that
    ``output`` is what ``cluster_reconstruct`` returned for this ``index`` (rows of a group are
    then identical), which lets the kernel read one mask row per group instead of all of
    ``output``."""
    _check_float(grad)
    _check_index(index, grad.device)
    _check_float(output)
    groups = int(groups)
    _require(groups >= 0 and output.shape == grad.shape and output.device == grad.device and
             output.dtype == grad.dtype and index.numel() == grad.size(0),
             "Invalid reconstruction gradient")
    width = grad.size(1)
    out = torch.empty((groups, width), dtype=grad.dtype, device=grad.device)
    bias_grad = torch.empty(width, dtype=grad.dtype, device=grad.device) if return_bias_grad else None
    if grad.numel() == 0:
        out.zero_()
        return (out, bias_grad.zero_()) if return_bias_grad else out
    if plan is None:
        plan = index_plan(index, groups)
    _require(plan.rows == groups and plan.nnz == index.numel(),
             "cluster_reconstruct_backward: plan does not match index/groups")
    code = _dtype_code(grad)
    sp, sb = plan.scratch(width, code)
    with on_device(grad.device):
        check(lib().cgnn_cluster_reconstruct_backward(
            plan.handle, code, width, _ptr(grad), _ptr(output),
            (2 if output_is_forward_result else 1) if relu else 0, _ptr(out),
            _ptr(bias_grad) if return_bias_grad else None, sp, sb, _stream_ptr(grad.device)))
    return (out, bias_grad) if return_bias_grad else out


def device_status():
    """Read and clear the kernels' status word (synchronises the device)."""
    status = ctypes.c_int(0)
    check(lib().cgnn_device_status(ctypes.byref(status)))
    return int(status.value)


_STATUS_BITS = ((1, "an index outside its table was skipped"),
                (2, "a bounded wait on a staged copy ran out: that launch's output is not to be used"),
                (4, "a CSR array held a negative or over-wide index"))


def compress_csr_batch(vlist, elist, rounds=12, min_pair_frequency=16):
    """Grammar compression of a CSR graph on the GPU (``cgnn_compress_csr_batch``): ``vlist`` /
    ``elist`` are int64 CUDA tensors; returns ``(vlist int32, elist int32, vertices, rules)`` as CUDA
    tensors with the arrays the host compressor of this package produces for the same input."""
    _require(vlist.is_cuda and elist.is_cuda and vlist.device == elist.device, "compress_csr_batch needs CUDA tensors")
    _require(vlist.dtype == torch.int64 and elist.dtype == torch.int64 and vlist.dim() == 1 and elist.dim() == 1 and
             vlist.numel() >= 1, "compress_csr_batch needs one-dimensional int64 arrays")
    vlist, elist = vlist.contiguous(), elist.contiguous()
    device = vlist.device
    handle = ctypes.c_void_p(0)
    with on_device(device):
        stream = _stream_ptr(device)
        check(lib().cgnn_compress_csr_batch(_ptr(vlist), _ptr(elist), vlist.numel() - 1, int(rounds),
                                            int(min_pair_frequency), ctypes.byref(handle), stream))
        try:
            info = (ctypes.c_int64 * 3)()
            check(lib().cgnn_compressed_info(handle, info))
            n, rules, entries = int(info[0]), int(info[1]), int(info[2])
            out_v = torch.empty(n + rules + 1, dtype=torch.int32, device=device)
            out_e = torch.empty(entries, dtype=torch.int32, device=device)
            check(lib().cgnn_compressed_copy(handle, _ptr(out_v), _ptr(out_e), stream))
        finally:
            lib().cgnn_compressed_destroy(handle)
    return out_v, out_e, n, rules


def raise_on_device_status():
    """``device_status()`` turned into an exception: raises RuntimeError naming the bits that were set."""
    status = device_status()
    if status:
        what = "; ".join(text for bit, text in _STATUS_BITS if status & bit)
        raise RuntimeError(f"compressgnn_b200 device status {status}: {what}")
