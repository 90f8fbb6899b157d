from .spmm import Compressgnn_SPMM, Compressgnn_SPMM_Function, compress_spmm
from .propagation import Propagate, KPropagate, KPUPropagate
from .cluster import Compressgnn_Cluster, Compressgnn_Cluster_Function, _Mean
from .reconstruct import Compressgnn_Reconstruct, _Reconstruct
from .host_io import HostPropagation

__all__ = ["Compressgnn_SPMM", "Compressgnn_SPMM_Function", "compress_spmm", "Propagate", "KPropagate",
           "KPUPropagate", "Compressgnn_Cluster", "Compressgnn_Cluster_Function", "Compressgnn_Reconstruct", "HostPropagation"]
