"""Module wrappers around the compressed propagation (ref: ``layer/CompressgnnPropagation.py``
:62-85, ``layer/KPropagate.py:12-27``, ``layer/KPUPropagate.py:9-37``).  ``edge_index`` is either
a ``CompressGraph`` (the CSR / SpMM form) or the list of per-phase edge tensors of the COO form;
both end in the same segment-reduce kernels."""
from typing import Optional

import torch
from torch import Tensor

from ..loader.compress_graph import CompressGraph
from .phased import phased_propagate
from .spmm import Compressgnn_SPMM

AGGRS = {'add', 'sum', 'mean', 'min', 'max', 'mul'}


class Propagate(torch.nn.Module):
    def __init__(self, aggr: Optional[str] = 'add', node_dim: int = -2):
        super().__init__()
        if aggr is not None and not isinstance(aggr, str):
            raise ValueError(f"Only strings are vaild aggregation schemes(got '{type(aggr)}'")
        assert aggr is None or aggr in AGGRS
        self.aggr = aggr
        self.node_dim = node_dim
        self.SPMM = Compressgnn_SPMM()

    def compressgnn_propagate(self, x: Tensor, edge_index, edge_weight=None, size=None,
                              vertex_cnt: int = None, rule_cnt: int = None):
        if isinstance(edge_index, CompressGraph):
            return self.update(self.SPMM(edge_index=edge_index, x_j=x))
        if isinstance(edge_index, (list, tuple)) and (len(edge_index) == 0 or torch.is_tensor(edge_index[0])):
            # the per-phase edge lists of CompressgnnData(graph_type="coo") (ref :68-83)
            if self.aggr not in ('add', 'sum'):
                raise ValueError("the phased edge-list propagation sums its messages (aggr='add')")
            return self.update(phased_propagate(x, edge_index, edge_weight, vertex_cnt, rule_cnt))
        raise TypeError("edge_index must be a CompressGraph or the list of per-phase [2, E] edge tensors")

    def update(self, out: Tensor) -> Tensor:
        return out


class KPropagate(Propagate):
    def __init__(self, spmm_impl: str = "inplace", **kwargs):
        kwargs.setdefault('aggr', 'add')
        super().__init__(**kwargs)

    def forward(self, x: Tensor, edge_index, edge_weight=None, vertex_cnt=None, rule_cnt=None) -> Tensor:
        return self.compressgnn_propagate(edge_index=edge_index, x=x, edge_weight=edge_weight,
                                          vertex_cnt=vertex_cnt, rule_cnt=rule_cnt, size=None)


class KPUPropagate(Propagate):
    """K propagation steps with an optional cache of the result (SGC-style precompute)."""

    def __init__(self, K: int = 1, cached: bool = False, **kwargs):
        kwargs.setdefault('aggr', 'add')
        super().__init__(**kwargs)
        self.K = K
        self.cached = cached
        self._cached_x = None

    def reset_cache(self):
        self._cached_x = None

    def forward(self, x: Tensor, edge_index, edge_weight=None, vertex_cnt=None, rule_cnt=None) -> Tensor:
        if self._cached_x is not None:
            return self._cached_x.detach()
        for _ in range(self.K):
            x = self.compressgnn_propagate(x=x, edge_index=edge_index, edge_weight=edge_weight,
                                           vertex_cnt=vertex_cnt, rule_cnt=rule_cnt, size=None)
        if self.cached:
            self._cached_x = x
        return x

    def __repr__(self) -> str:
        return f'{self.__class__.__name__}(K={self.K})'
