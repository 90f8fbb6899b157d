from .sparse_block import SparseBlock
from .compress_graph import CompressGraph
from .data import CompressgnnData, compress
from .compression_backend import compress_graph_csr, resolve_backend

__all__ = ["SparseBlock", "CompressGraph", "CompressgnnData", "compress", "compress_graph_csr",
           "resolve_backend"]
