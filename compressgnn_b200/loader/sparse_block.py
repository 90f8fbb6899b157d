"""``SparseBlock``: the slice of ``torch_sparse.SparseTensor`` the CompressGNN loader and
layers use -- construction from ``rowptr/col/value``, ``.csr()``, ``.csc()``, ``.to()``,
``.sparse_sizes()`` -- without depending on torch_sparse.

``csc()`` returns the transposed block as ``(colptr, row, value)`` with the entries of a
column in ascending row order, which is what ``SparseTensor.csc()`` yields for the reference
(loader/compress_graph.py:21-35, layer/CompressgnnSPMM.py:68-70).
"""
import torch


class SparseBlock:
    def __init__(self, rowptr, col, value=None, sparse_sizes=None):
        self.rowptr = torch.as_tensor(rowptr).to(torch.int64).contiguous()
        self.col = torch.as_tensor(col).to(torch.int64).contiguous()
        if value is None:
            value = torch.ones(self.col.numel(), dtype=torch.float32, device=self.col.device)
        self.value = torch.as_tensor(value).contiguous()
        rows = self.rowptr.numel() - 1
        if sparse_sizes is None:
            cols = int(self.col.max()) + 1 if self.col.numel() else 0
            sparse_sizes = (rows, cols)
        if sparse_sizes[0] != rows:
            raise ValueError("rowptr length does not match sparse_sizes[0]")
        self._sizes = (int(sparse_sizes[0]), int(sparse_sizes[1]))
        self._csc = None
        self._typed = {}

    def sparse_sizes(self):
        return self._sizes

    def size(self, dim):
        return self._sizes[dim]

    def nnz(self):
        return self.col.numel()

    @property
    def device(self):
        return self.col.device

    def csr(self):
        return self.rowptr, self.col, self.value

    def csc(self):
        if self._csc is None:
            rows, cols = self._sizes
            counts = torch.bincount(self.col, minlength=cols) if self.col.numel() else \
                torch.zeros(cols, dtype=torch.int64, device=self.device)
            colptr = torch.zeros(cols + 1, dtype=torch.int64, device=self.device)
            torch.cumsum(counts, 0, out=colptr[1:])
            perm = torch.argsort(self.col, stable=True)
            row_of_entry = torch.repeat_interleave(
                torch.arange(rows, dtype=torch.int64, device=self.device), self.rowptr[1:] - self.rowptr[:-1])
            self._csc = (colptr, row_of_entry[perm].contiguous(), self.value[perm].contiguous())
        return self._csc

    def value_as(self, dtype, transposed=False):
        """The value array (of ``csr()`` or ``csc()``) in ``dtype``, converted once."""
        key = (dtype, transposed)
        if key not in self._typed:
            base = self.csc()[2] if transposed else self.value
            self._typed[key] = base if base.dtype == dtype else base.to(dtype)
        return self._typed[key]

    def to(self, device):
        out = SparseBlock.__new__(SparseBlock)
        out.rowptr, out.col, out.value = (t.to(device) for t in (self.rowptr, self.col, self.value))
        out._sizes = self._sizes
        out._csc = None if self._csc is None else tuple(t.to(device) for t in self._csc)
        out._typed = {}
        return out

    def __repr__(self):
        return f"SparseBlock(sizes={self._sizes}, nnz={self.nnz()}, device={self.device})"
