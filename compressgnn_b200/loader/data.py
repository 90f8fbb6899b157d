"""``CompressgnnData``: the loader object of the compressed-propagation path (CSR branch of
the reference's ``loader/CompressgnnData.py:60-85,140-201``): self loops, symmetric
normalisation, grammar compression with the two rule filters, weights of the compressed
graph, transposition and the block partition into a ``CompressGraph``."""
import numpy as np
import torch

from .. import offline
from .compress_graph import CompressGraph
from .compression_backend import compress_graph_csr, resolve_backend


def compress(vlist, elist, threshold, max_depth, min_edge, min_pair_frequency=16,
             compression_backend='auto', compression_threads=4, compression_rounds=12, verbose=False):
    """Compressor followed by ``filter_csr`` and ``depth_filter_csr``
    (ref: loader/CompressgnnData.py:26-55).  Returns ``(vlist, elist, vertex_cnt, rule_cnt)``."""
    selected = resolve_backend(compression_backend)
    result = compress_graph_csr(vlist, elist, min_pair_frequency, selected, compression_threads,
                                compression_rounds)
    before = len(vlist) + len(elist)
    report = lambda tag, r: verbose and print("{} compression ratio: {} / {} = {:.4f}".format(
        tag, before, len(r[0]) + len(r[1]), before / (len(r[0]) + len(r[1]))))
    report("raw", result)
    result = offline.filter_csr(*result, threshold)
    report("after filter", result)
    result = offline.depth_filter_csr(*result, max_depth, min_edge)
    report("after depth filter", result)
    return result


class CompressgnnData:
    def __init__(self, x, edge_index, y, train_mask, vaild_mask, test_mask,
                 add_self_loop: bool = True, normalize: bool = True, graph_type: str = "csr",
                 max_depth: int = 3, min_edge: int = 1000000, threshold: int = 16, homo: bool = False,
                 min_pair_frequency: int = 16, compression_backend: str = "auto",
                 compression_threads: int = 4, compression_rounds: int = 12, verbose: bool = False):
        if graph_type != "csr":
            raise NotImplementedError("compressgnn_b200 builds the CSR (SpMM) form of the compressed graph; "
                                      "the COO scatter form is not part of this package")
        x = np.asarray(x).astype(np.float32)
        self.x = torch.as_tensor(x)
        self.y = torch.as_tensor(np.array(y))
        self.train_mask = torch.as_tensor(train_mask)
        self.vaild_mask = torch.as_tensor(vaild_mask)
        self.test_mask = torch.as_tensor(test_mask)
        self.vertex_cnt = self.x.size(0)
        self.feature_dim = self.x.size(1)
        self.graph_type = graph_type
        self.min_pair_frequency = min_pair_frequency
        self.compression_backend = resolve_backend(compression_backend)
        self.compression_threads = compression_threads
        self.compression_rounds = compression_rounds
        vlist, elist = np.asarray(edge_index[0]), np.asarray(edge_index[1])
        self.orig_edge_cnt = int(elist.shape[0])
        if add_self_loop:
            vlist, elist = offline.add_self_loop_csr(vlist, elist)
        if normalize:
            norm_degree = offline.get_norm_degree(elist, self.vertex_cnt)
        self.input_edge_cnt = int(elist.shape[0])
        new_vlist, new_elist, vertex_cnt, rule_cnt = compress(
            vlist, elist, threshold, max_depth, min_edge, min_pair_frequency,
            self.compression_backend, compression_threads, compression_rounds, verbose)
        self.vertex_cnt, self.rule_cnt = int(vertex_cnt), int(rule_cnt)
        self.edge_cnt = int(new_elist.shape[0])
        new_vlist, new_elist = new_vlist.astype(np.int64), new_elist.astype(np.int64)
        if normalize:
            weight = offline.gcn_norm_csr_compress(new_vlist, new_elist, norm_degree, vertex_cnt, rule_cnt)
        else:
            weight = np.ones(self.edge_cnt, dtype=np.float32)
        self.step = offline.phase_count(new_vlist, new_elist, vertex_cnt, rule_cnt)
        total = vertex_cnt + rule_cnt
        # The propagation consumes the transposed graph: row j lists what flows into j.
        t_vlist, t_elist, t_weight = offline.transpose_csr(new_vlist, new_elist, weight, total)
        self.edge_index = CompressGraph(t_vlist, t_elist, t_weight, self.vertex_cnt)

    def __repr__(self):
        return 'CompressgnnData(vertex_cnt:"%s", rule_cnt:"%s", edge_cnt:"%s", step:"%s", graph_type:"%s")' % (
            self.vertex_cnt, self.rule_cnt, self.edge_cnt, self.step, self.graph_type)

    def to(self, device):
        self.x = self.x.to(device)
        self.y = self.y.to(device)
        self.train_mask = self.train_mask.to(device)
        self.vaild_mask = self.vaild_mask.to(device)
        self.test_mask = self.test_mask.to(device)
        self.edge_index = self.edge_index.to(device)
        return self
