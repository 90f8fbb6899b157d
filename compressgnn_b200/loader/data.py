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


def edge_phases(src, dst, vertex_cnt, rule_cnt):
    """Phase of every edge of a compressed graph and the number of phases.

    An edge that leaves a vertex is phase 0.  An edge that leaves a rule is phase ``k`` when the last
    of the rule's incoming edges is phase ``k - 1``: a rule fed by vertices only sends in phase 1, a
    rule fed by phase-1 rules in phase 2, and so on -- the schedule gen_edge_order derives by peeling
    in-degrees (ref: src/offline/csrc/gen_mask.h:9-83).  At least one phase is always reported."""
    src, dst = np.asarray(src, dtype=np.int64), np.asarray(dst, dtype=np.int64)
    order = np.zeros(src.size, dtype=np.int32)
    from_rule = src >= vertex_cnt
    if not from_rule.any():
        return order, 1
    send = np.ones(rule_cnt, dtype=np.int32)          # phase in which a rule's outgoing edges run
    rs, rd = src[from_rule] - vertex_cnt, dst[from_rule]
    into_rule = rd >= vertex_cnt
    rs, rd = rs[into_rule], rd[into_rule] - vertex_cnt  # rule -> rule edges
    for _ in range(rule_cnt + 1):
        nxt = send.copy()
        np.maximum.at(nxt, rd, send[rs] + 1)
        if np.array_equal(nxt, send):
            break
        send = nxt
    else:
        raise ValueError("the rule graph has a cycle")
    order[from_rule] = send[src[from_rule] - vertex_cnt]
    return order, int(order.max()) + 1


class CompressgnnData:
    def __init__(self, x, edge_index, y, train_mask, vaild_mask, test_mask,
                 add_self_loop: bool = True, normalize: bool = True, graph_type: str = "csr",
                 max_depth: int = 3, min_edge: int = 1000000, threshold: int = 16, homo: bool = False,
                 min_pair_frequency: int = 16, compression_backend: str = "auto",
                 compression_threads: int = 4, compression_rounds: int = 12, verbose: bool = False):
        if graph_type not in ("csr", "coo"):
            raise ValueError("graph_type must be 'csr' or 'coo'")
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
        if graph_type == "coo":
            self._init_coo(edge_index, add_self_loop, normalize, threshold, max_depth, min_edge, verbose)
            return
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

    def _init_coo(self, edge_index, add_self_loop, normalize, threshold, max_depth, min_edge, verbose):
        """The edge-list form (ref: loader/CompressgnnData.py:86-139): ``edge_index`` arrives as
        ``(src, dst)`` sorted by source then destination; after compression the edges of the
        compressed graph are handed out as one ``[2, E_i]`` tensor per phase with their weights,
        phase 0 holding every edge that leaves a vertex and phase k the edges that leave the rules
        whose inputs are complete after phase k-1 (ref: gen_edge_order, src/offline/csrc/gen_mask.h:9-83)."""
        src, dst = np.asarray(edge_index[0], dtype=np.int64), np.asarray(edge_index[1], dtype=np.int64)
        if src.size and np.any(np.diff(src) < 0):
            raise ValueError("graph_type='coo' expects edges sorted by source")
        n = self.vertex_cnt
        self.orig_edge_cnt = int(src.size)
        vlist = np.zeros(n + 1, dtype=np.int64)
        np.cumsum(np.bincount(src, minlength=n), out=vlist[1:])
        elist = dst
        if add_self_loop:
            vlist, elist = offline.add_self_loop_csr(vlist, elist)
        if normalize:
            norm_degree = offline.get_norm_degree(elist, n)
        self.input_edge_cnt = int(elist.shape[0])
        new_vlist, new_elist, vertex_cnt, rule_cnt = compress(
            vlist, elist, threshold, max_depth, min_edge, self.min_pair_frequency,
            self.compression_backend, self.compression_threads, self.compression_rounds, verbose)
        self.vertex_cnt, self.rule_cnt = int(vertex_cnt), int(rule_cnt)
        new_vlist, new_elist = new_vlist.astype(np.int64), new_elist.astype(np.int64)
        self.edge_cnt = int(new_elist.shape[0])
        total = self.vertex_cnt + self.rule_cnt
        c_src = np.repeat(np.arange(total, dtype=np.int64), np.diff(new_vlist))
        c_dst = new_elist
        if normalize:  # the same four cases as the CSR form, edge by edge (ref: gcn_norm_coo_compress, norm.h:129-166)
            weight = offline.gcn_norm_csr_compress(new_vlist, new_elist, norm_degree, vertex_cnt, rule_cnt)
        else:
            weight = np.ones(self.edge_cnt, dtype=np.float32)
        order, self.step = edge_phases(c_src, c_dst, self.vertex_cnt, self.rule_cnt)
        self.edge_index, self.edge_weight = [], []
        for phase in range(self.step):
            pick = order == phase
            self.edge_index.append(torch.from_numpy(np.stack([c_src[pick], c_dst[pick]])))
            self.edge_weight.append(torch.from_numpy(weight[pick]))

    def __repr__(self):
        return 'CompressgnnData(vertex_cnt:"%s", rule_cnt:"%s", edge_cnt:"%s", step:"%s", graph_type:"%s")' % (
            self.vertex_cnt, self.rule_cnt, self.edge_cnt, self.step, self.graph_type)

    def to(self, device):
        self.x = self.x.to(device)
        self.y = self.y.to(device)
        self.train_mask = self.train_mask.to(device)
        self.vaild_mask = self.vaild_mask.to(device)
        self.test_mask = self.test_mask.to(device)
        if self.graph_type == "coo":
            self.edge_index = [e.to(device) for e in self.edge_index]
            self.edge_weight = [w.to(device) for w in self.edge_weight]
        else:
            self.edge_index = self.edge_index.to(device)
        return self
