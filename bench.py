"""Benchmark of the compressed-propagation hot path (and, on request, of the cluster /
reconstruct operators) on synthetic inputs.

    python bench.py --gpus N --steps K --warmup W            # this package, N GPUs (torchrun for N>1)
    python bench.py --impl reference --steps K --warmup W    # the reference's own CPU operators

Default workload ("propagation"): compressed propagation SpMM, forward + transposed backward,
on a seeded copying-model web graph with 325,557 nodes and ~3.2 M edges, features N x 256 fp32.
One step = one forward and one backward pass over the whole graph.  The metric is
original-edge x feature products per second: 2 * E_orig * F / t_step.

With N GPUs the feature columns are sharded and the graph replicated (no data-path collective).
The default is weak scaling -- each GPU keeps a 256-column block, so the job's matrix is
N x 256*gpus; `--scaling strong` divides the 256 columns instead.

Prints ONE JSON line (rank 0).  `value` is device-resident throughput (CUDA events, max over
ranks); `e2e` goes through the public host-buffer front end with pinned host matrices, copies included;
`roofline` is for the dominant kernel (the fused vertex pass of the forward); `cpu_baseline`
is the reference's CPU spmm_func chain on this host's cores.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

METRIC = "compressed_spmm_orig_edge_feat_per_s"
UNIT = "Gedge*feat/s"


# ---------------------------------------------------------------------------------------------
# Workload construction (host side, untimed)
# ---------------------------------------------------------------------------------------------
WORKLOADS = {
    # name: nodes, pareto x_min (sets E), feature width
    "propagation": dict(n=325557, x_min=5.3, width=256, seed=2),
    "propagation-small": dict(n=40000, x_min=5.3, width=256, seed=2),
    "propagation-xl": dict(n=18500000, x_min=8.6, width=128, seed=4),
}
COMPRESS = dict(min_pair_frequency=4, threshold=4, max_depth=3, min_edge=1000000)
# dram__bytes_read.sum + dram__bytes_write.sum of one forward fused vertex pass at N=1, from the
# ncu capture summarised in profiles/seg_bulk_kernel_fused_vertex_pass_config2.md (same workload).
NCU_TRAFFIC_BYTES = {("propagation", 1): 1.461e9}


def build_graph(name):
    """Seeded copying-model graph -> CompressgnnData (self loops, symmetric normalisation,
    grammar compression, block partition).  Stands in for the public web graphs the reference's
    scripts load; nothing of those datasets is used."""
    from compressgnn_b200 import offline as off
    from compressgnn_b200.loader import CompressgnnData
    w = WORKLOADS[name]
    n = w["n"]
    vlist, elist = off.generate_copy_graph(n, alpha=2.1, x_min=w["x_min"], max_degree=10000, copy_prob=0.7,
                                           window=64, candidates=8, seed=w["seed"])
    mask = np.ones(n, dtype=bool)
    data = CompressgnnData(np.zeros((n, 1), np.float32), (vlist, elist), np.zeros(n, np.int64), mask, mask, mask,
                           add_self_loop=True, normalize=True, graph_type="csr", **COMPRESS)
    return data, int(elist.size)


def block_bytes(block, width, rows_written, rows_accumulated, transposed=False):
    """Algorithmic bytes of one SpMM block: every distinct source row read once, every output
    row written once (and pre-read when accumulating), 4-byte column + 4-byte value per entry,
    4-byte row pointers."""
    rowptr, col, _val = block.csc() if transposed else block.csr()
    distinct = int(np.unique(col.cpu().numpy()).size) if col.numel() else 0
    return 4 * width * (rows_written + rows_accumulated + distinct) + 8 * col.numel() + 4 * rowptr.numel()


def propagation_bytes(graph, width):
    """Per-launch algorithmic bytes of the forward and backward passes."""
    g = graph
    n, r = g.vertex_cnt, g.rule_cnt
    nonempty = lambda b, t=False: int(((b.csc() if t else b.csr())[0].diff() > 0).sum())
    fwd = [("fwd_r2v", block_bytes(g.r2v_graph, width, r, 0))]
    for i, lvl in enumerate(g.r2r_graph):
        k = nonempty(lvl)
        fwd.append((f"fwd_level{i}", block_bytes(lvl, width, k, k)))
    fwd.append(("fwd_out", block_bytes(g.v2r_graph, width, n, 0) + block_bytes(g.v2v_graph, width, 0, 0)))
    bwd = [("bwd_v2r_t", block_bytes(g.v2r_graph, width, r, 0, True))]
    for i, lvl in reversed(list(enumerate(g.r2r_graph))):
        k = nonempty(lvl, True)
        bwd.append((f"bwd_level{i}", block_bytes(lvl, width, k, k, True)))
    bwd.append(("bwd_out", block_bytes(g.v2v_graph, width, n, 0, True) + block_bytes(g.r2v_graph, width, 0, 0, True)))
    return fwd, bwd


# ---------------------------------------------------------------------------------------------
# Clock sampling during the timed region
# ---------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.samples, self.proc, self.index = [], None, index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6 and parts[0].isdigit():
                self.samples.append(parts)

    def __exit__(self, *exc):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm = sorted(int(s[0]) for s in self.samples)
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = [n for i, n in enumerate(names) if any(s[2 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": int(self.samples[0][1]), "reasons": reasons,
                "samples": len(sm)}


# ---------------------------------------------------------------------------------------------
# Reference CPU arm / CPU baseline
# ---------------------------------------------------------------------------------------------
def cpu_propagation(data, width, steps, warmup, seed=0):
    """The reference's CPU path: spmm_func(..., "rowbalance", ...) chained in the order of
    layer/CompressgnnSPMM.py:47-53 (forward) and :80-85 (backward), all host threads.
    Returns (seconds per step, kind, cores, sample description)."""
    import torch
    from oracle import oracle
    rt, _off = oracle.reference_modules()
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    g = data.edge_index
    n, r = g.vertex_cnt, g.rule_cnt
    gen = torch.Generator().manual_seed(seed)
    if rt is not None:
        kind, sample_width = "reference", width
    else:
        kind, sample_width, cores = "port", min(width, 8), 1  # scalar single-thread C port: a column slice
    x = torch.randn(n, sample_width, generator=gen)
    grad = torch.randn(n, sample_width, generator=gen)
    fwd_blocks = dict(r2v=g.r2v_graph.csr(), v2r=g.v2r_graph.csr(), v2v=g.v2v_graph.csr(),
                      levels=[lvl.csr() for lvl in g.r2r_graph])
    bwd_blocks = dict(v2r_t=g.v2r_graph.csc(), v2v_t=g.v2v_graph.csc(), r2v_t=g.r2v_graph.csc(),
                      levels_t=[lvl.csc() for lvl in g.r2r_graph])

    if rt is not None:
        def spmm(blk, m, out=None):
            return rt.spmm_func(blk[0], blk[1], blk[2], m, "rowbalance", out)
    else:
        def spmm(blk, m, out=None):
            res = oracle.spmm(blk[0].numpy(), blk[1].numpy(), blk[2].numpy(), m.numpy(),
                              None if out is None else out.numpy())
            return torch.from_numpy(res)

    def step():
        rule_out = spmm(fwd_blocks["r2v"], x)
        for lvl in fwd_blocks["levels"]:
            rule_out = spmm(lvl, rule_out, rule_out)
        out = spmm(fwd_blocks["v2v"], x, spmm(fwd_blocks["v2r"], rule_out))
        rule_g = spmm(bwd_blocks["v2r_t"], grad)
        for lvl in reversed(bwd_blocks["levels_t"]):
            rule_g = spmm(lvl, rule_g, rule_g)
        gx = spmm(bwd_blocks["r2v_t"], rule_g, spmm(bwd_blocks["v2v_t"], grad))
        return out, gx

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / max(steps, 1)
    scale = width / sample_width  # a column slice scales linearly in the width
    sample = (f"full workload, {steps} steps" if sample_width == width else
              f"{sample_width} of {width} feature columns, {steps} steps, time scaled by {scale:g}")
    return dt * scale, kind, cores, sample


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------
def run_gpu(args):
    import torch
    import torch.distributed as dist
    from compressgnn_b200.layer import Compressgnn_SPMM, spmm as spmm_layer
    from compressgnn_b200 import runtime as rt

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")  # keep NCCL's banner off stdout (one JSON line)
        dist.init_process_group("nccl", device_id=device)

    wl = dict(WORKLOADS[args.workload])
    if args.width:
        wl["width"] = args.width
    if args.scaling == "weak":
        # every rank holds a full-width column block: the job's feature matrix is N x (F * world)
        width = wl["width"]
        width_total = width * world
    else:
        width_total = wl["width"]
        assert width_total % world == 0, "feature width must divide by the number of GPUs"
        width = width_total // world  # column shard of this rank; the graph is replicated
    data, e_orig = build_graph(args.workload)
    cpu_graph_for_baseline = data if rank == 0 else None
    graph = data.edge_index
    n = graph.vertex_cnt

    # CPU baseline first (rank 0, N=1 only), while the graph blocks are still host tensors.
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        sec, kind, cores, sample = cpu_propagation(cpu_graph_for_baseline, width_total, args.cpu_steps, 1)
        cpu = {"value": 2 * e_orig * width_total / sec / 1e9, "unit": UNIT, "cores": cores, "kind": kind,
               "sample": sample, "ms_per_step": sec * 1e3}

    fwd_bytes, bwd_bytes = propagation_bytes(graph, width)
    graph.to(device)
    gen = torch.Generator(device=device).manual_seed(1234 + rank)
    x = torch.randn(n, width, device=device, generator=gen)
    grad = torch.randn(n, width, device=device, generator=gen)
    plan = graph.propagation_plan()
    launches_per_step = 2 * (2 + graph.step)

    def step(record=None):
        out = spmm_layer._forward(graph, x, record)
        gx = spmm_layer._backward(graph, grad, record)
        return out, gx

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()

    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    records = []
    with ClockSampler(local_rank) as clocks:
        start.record()
        for _ in range(args.steps):
            rec = []
            step(rec)
            records.append(rec)
        stop.record()
        torch.cuda.synchronize()
        # keep the GPU busy a little longer if the region was too short for one clock sample
        t_end = time.time() + max(0.0, 0.6 - start.elapsed_time(stop) / 1e3)
        while time.time() < t_end:
            step()
            torch.cuda.synchronize()
    ms = start.elapsed_time(stop)
    if world > 1:
        t = torch.tensor([ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_per_step = ms / args.steps

    # per-launch durations (events recorded inside the timed region)
    per_launch = {}
    for rec in records:
        for name, e0, e1 in rec:
            per_launch.setdefault(name, []).append(e0.elapsed_time(e1))
    launch_ms = {k: float(np.mean(v)) for k, v in per_launch.items()}
    bytes_by_name = dict(fwd_bytes + bwd_bytes)

    # end to end through the public host-buffer front end: pinned host operands, every upload
    # and download inside the timed region, passes queued so that the two copy directions overlap
    e2e_sec = e2e_sync_sec = None
    if not args.no_e2e and 4 * n * width <= 4 * 2**30:  # four pinned copies of X: skipped for very large shards
        from compressgnn_b200.layer import HostPropagation
        pipe = HostPropagation(graph, width)
        x_host = x.cpu().pin_memory()
        g_host = grad.cpu().pin_memory()
        out_host = torch.empty_like(x_host).pin_memory()
        gx_host = torch.empty_like(x_host).pin_memory()

        def e2e_steps(count, wait_each):
            if world > 1:
                dist.barrier()
            t0 = time.perf_counter()
            for _ in range(count):
                pipe.forward(x_host, out_host)
                pipe.backward(g_host, gx_host)
                if wait_each:
                    pipe.synchronize()
            pipe.synchronize()
            sec = (time.perf_counter() - t0) / count
            if world > 1:
                t = torch.tensor([sec], device=device)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                sec = float(t.item())
            return sec

        e2e_steps(2, False)
        e2e_sync_sec = e2e_steps(args.steps, True)   # each step waited for before the next is queued
        e2e_sec = e2e_steps(args.steps, False)       # steps queued back to back, one wait at the end
        assert torch.equal(out_host, step()[0].cpu()), "host front end and resident path disagree"
        del pipe

    status = rt.device_status()
    assert status == 0, f"device status word {status}"
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks_path = ROOT / "MEASURED_PEAKS.json"
    if peaks_path.is_file():
        peak, peak_src = json.loads(peaks_path.read_text())["hbm_gbs"], "measured (MEASURED_PEAKS.json)"
    else:
        peak, peak_src = 6650.0, "fallback"
    dom = "fwd_out"
    achieved = bytes_by_name[dom] / (launch_ms[dom] * 1e-3) / 1e9
    work = 2 * e_orig * width_total
    line = {
        "metric": METRIC, "value": work / (ms_per_step * 1e-3) / 1e9, "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{args.workload}: compressed propagation SpMM fwd+bwd, copying-model web graph",
                   "nodes": n, "orig_edges": e_orig, "compressed_edges": graph.edge_count(),
                   "rules": graph.rule_cnt, "levels": graph.step, "feature_width": width_total,
                   "columns_per_gpu": width, "compressor": COMPRESS,
                   "l2": "inputs larger than L2 (X is %.0f MB per GPU)" % (4e-6 * n * width),
                   "parallelism": f"feature columns sharded over {world} GPU(s), graph replicated, no collective"},
        "e2e": ({"value": work / e2e_sec / 1e9, "unit": UNIT, "h2d_bytes_per_step": 2 * 4 * n * width,
                 "d2h_bytes_per_step": 2 * 4 * n * width, "ms_per_step": e2e_sec * 1e3,
                 "ms_per_step_waiting_each_step": e2e_sync_sec * 1e3,
                 "api": "HostPropagation.forward/backward on pinned host matrices"} if e2e_sec else None),
        "gpu_launches": launches_per_step * args.steps,
        "roofline": {"bound": "hbm", "kernel": "seg_bulk_kernel (fused v2r+v2v vertex pass, forward)",
                     "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_source": peak_src, "traffic": NCU_TRAFFIC_BYTES.get((args.workload, world)),
                     "algorithmic_bytes_per_launch": bytes_by_name[dom], "ms_per_launch": launch_ms[dom],
                     "launches": {k: {"ms": launch_ms[k], "algorithmic_GBps": bytes_by_name[k] / launch_ms[k] / 1e6}
                                  for k in launch_ms}},
        "clocks": clocks.summary(),
    }
    if cpu is not None:
        line["cpu_baseline"] = cpu
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def cpu_cluster(n, width, out_width, bits, fraction=8):
    """The reference's CPU path of the same epoch on 1/`fraction` of the nodes (all host threads):
    cluster_forward (src/runtime/csrc/cluster/cpu/cluster_cpu.cpp:27-70) + bincount, the mean and its
    backward as layer/CompressgnnCluster.py:16-25 computes them, Linear, and the CPU reconstruct of
    layer/CompressgnnReconstruct.py:39-42 with autograd for its backward."""
    import torch
    from oracle import oracle
    rt, _off = oracle.reference_modules()
    if rt is None:
        return {"value": None, "unit": "Mnode/s", "cores": 0, "kind": "reference",
                "sample": "unavailable: oracle/_ref is not built on this box"}
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    m = n // fraction
    gen = torch.Generator().manual_seed(3)
    cent = torch.randn(4096, width, generator=gen)
    x = (cent[torch.randint(0, 4096, (m,), generator=gen)] + 0.1 * torch.randn(m, width, generator=gen)).requires_grad_()
    planes = torch.randn(width, bits, generator=gen)
    lin = torch.nn.Linear(width, out_width)
    grad_out = torch.randn(m, out_width, generator=gen)

    def epoch(refresh, state):
        if refresh:
            ids, active = rt.cluster_forward(x.detach(), planes, bits)
            index = ids.long()
            state["index"], state["counts"] = index, torch.bincount(index, minlength=active + 1)
        index, counts = state["index"], state["counts"]
        sums = torch.zeros(counts.numel(), width).index_add_(0, index, x)
        reps = sums / counts.clamp_min(1).to(torch.float32)[:, None]
        y = (torch.nn.functional.linear(reps, lin.weight, None).index_select(0, index) + lin.bias).relu()
        y.backward(grad_out)
        x.grad = None

    state = {}
    epoch(True, state)
    t0 = time.perf_counter()
    epochs = 5
    for e in range(epochs):
        epoch(e % 5 == 0, state)
    sec = (time.perf_counter() - t0) / epochs * fraction
    return {"value": n / sec / 1e6, "unit": "Mnode/s", "cores": cores, "kind": "reference",
            "ms_per_step": sec * 1e3,
            "sample": f"{m} of {n} nodes, {epochs} epochs with one refresh, time scaled by {fraction}"}


def run_cluster(args):
    """Config 3: Compressgnn_Cluster -> Linear(128->256) on representatives -> fused reconstruct
    (bias + ReLU), forward + backward, 2.45 M nodes drawn from 4096 Gaussian centroids, H=16,
    refresh_interval=5.  A step = one epoch.  Per-operator CUDA-event times and algorithmic GB/s
    are reported next to the epoch time; the CPU leg runs the reference's cluster_forward
    plus the torch CPU formulas its layers use."""
    import torch
    from compressgnn_b200 import runtime as rt
    from compressgnn_b200.layer import Compressgnn_Cluster, Compressgnn_Reconstruct
    torch.cuda.set_device(0)
    n, width, out_width, bits = args.cluster_nodes, 128, 256, 16
    gen = torch.Generator(device="cuda").manual_seed(3)
    cent = torch.randn(4096, width, device="cuda", generator=gen)
    which = torch.randint(0, 4096, (n,), device="cuda", generator=gen)
    x = (cent[which] + 0.1 * torch.randn(n, width, device="cuda", generator=gen)).requires_grad_()
    del which
    torch.manual_seed(3)
    cluster = Compressgnn_Cluster(width, bits, device="cuda", refresh_interval=5)
    lin = torch.nn.Linear(width, out_width).cuda()
    reconstruct = Compressgnn_Reconstruct()
    grad_out = torch.randn(n, out_width, device="cuda", generator=gen)

    def epoch(e):
        cluster.set_epoch(e)
        reps, index = cluster(x)
        y = reconstruct(torch.nn.functional.linear(reps, lin.weight, None), index, bias=lin.bias, activation="relu")
        y.backward(grad_out)
        x.grad = None
        return y

    for e in range(max(args.warmup, 3)):
        epoch(e)
    cluster.reset_cache()
    cluster.refresh_count = 0
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(0) as clocks:
        start.record()
        for e in range(args.steps):
            epoch(e)
        stop.record()
        torch.cuda.synchronize()
    ms_epoch = start.elapsed_time(stop) / args.steps

    # per-operator timings on the same tensors (CUDA events, median of 20)
    def timed(fn, reps_=20):
        for _ in range(3):
            fn()
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(reps_)]
        for a, b in ev:
            a.record()
            fn()
            b.record()
        torch.cuda.synchronize()
        return sorted(a.elapsed_time(b) for a, b in ev)[reps_ // 2]

    xd = x.detach()
    ws = rt.cluster_workspace(xd, bits)
    ids, counts, active = rt.cluster_assign(xd, cluster.random_vectors, bits, ws)
    groups = active + 1
    reps = rt.cluster_mean(xd, ids, counts)
    table = torch.randn(groups, out_width, device="cuda", generator=gen)
    bias = torch.randn(out_width, device="cuda", generator=gen)
    y = rt.cluster_reconstruct(table, ids, bias, True)
    g_small = torch.randn(groups, width, device="cuda", generator=gen)
    ops = {
        "cluster_assign (projection+codes+compaction)": (lambda: rt.cluster_assign(xd, cluster.random_vectors, bits, ws),
                                                          4 * n * width + 4 * width * bits + 8 * n + 40 * n),
        "cluster_mean": (lambda: rt.cluster_mean(xd, ids, counts), 4 * n * width + 8 * n + 4 * groups * width),
        "cluster_mean_backward": (lambda: rt.cluster_mean_backward(g_small, ids, counts),
                                  4 * groups * width + 8 * n + 4 * n * width),
        "cluster_reconstruct (bias+relu)": (lambda: rt.cluster_reconstruct(table, ids, bias, True),
                                            4 * groups * out_width + 8 * n + 4 * out_width + 4 * n * out_width),
        "cluster_reconstruct_backward (relu, exact mask)": (
            lambda: rt.cluster_reconstruct_backward(grad_out, ids, y, groups, True),
            8 * n * out_width + 8 * n + 4 * groups * out_width),
        "cluster_reconstruct_backward (relu, one mask row per group)": (
            lambda: rt.cluster_reconstruct_backward(grad_out, ids, y, groups, True, output_is_forward_result=True),
            4 * n * out_width + 8 * n + 8 * groups * out_width),
    }
    peaks_path = ROOT / "MEASURED_PEAKS.json"
    peak = json.loads(peaks_path.read_text())["hbm_gbs"] if peaks_path.is_file() else 6650.0
    op_report = {}
    for name, (fn, nbytes) in ops.items():
        ms = timed(fn)
        op_report[name] = {"ms": ms, "algorithmic_GBps": nbytes / ms / 1e6, "frac_of_peak": nbytes / ms / 1e6 / peak}
    assert rt.device_status() == 0
    cpu = None if args.no_cpu_baseline else cpu_cluster(n, width, out_width, bits)
    line = {"metric": "cluster_linear_reconstruct_nodes_per_s", "value": n / (ms_epoch * 1e-3) / 1e6, "unit": "Mnode/s",
            "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_epoch,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "cluster: Compressgnn_Cluster + Linear 128->256 + Compressgnn_Reconstruct(relu), fwd+bwd",
                       "nodes": n, "feature_width": width, "out_width": out_width, "bits": bits, "centroids": 4096,
                       "active_buckets": active, "refresh_interval": 5, "refreshes": cluster.refresh_count,
                       "l2": "inputs larger than L2 (X is %.0f MB)" % (4e-6 * n * width)},
            "operators": op_report, "peak_GBps": peak, "clocks": clocks.summary(),
            "gpu_launches": None}
    if cpu is not None:
        line["cpu_baseline"] = cpu
    print(json.dumps(line))


def run_gcn(args):
    """Config 5: end-to-end 2-layer GCN with propagation and transformation compression
    (use_transformation=True, H=16, refresh_interval=5) on the config-2 graph, 47 uniform classes,
    input feature width swept over 16/64/256/1024.  A step = one training epoch (forward, NLL loss
    on all nodes, backward, Adam step), timed after warm-up epochs as the reference's
    benchmark/end2end/compressgnn_gcn.py does.  With N GPUs the feature columns of every layer are
    sharded (strong scaling: the same model and matrix on more GPUs) and the graph is replicated."""
    import torch
    import torch.distributed as dist
    from compressgnn_b200.model import GCN
    from compressgnn_b200 import dist as cdist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")  # keep NCCL's banner off stdout (one JSON line)
        dist.init_process_group("nccl", device_id=device)
    data, e_orig = build_graph("propagation")
    graph = data.edge_index
    n = graph.vertex_cnt
    graph.to(device)
    gen = torch.Generator(device=device).manual_seed(5)  # the same labels and features on every rank
    y = torch.randint(0, 47, (n,), device=device, generator=gen)
    y_col = y.unsqueeze(1)
    report = {}
    for width in (16, 64, 256, 1024):
        x = torch.randn(n, width, device=device, generator=gen)
        torch.manual_seed(5)
        model = GCN(width, 47, hidden_features=128, param_H=16, dropout=0.3, use_transformation=True,
                    refresh_interval=5, num_layers=2).to(device)
        opt = torch.optim.Adam(model.parameters(), lr=1e-3)
        if world > 1:
            x = cdist.shard_columns(x, rank, world)
            net = cdist.ShardedGCN(model, dist.group.WORLD)  # shares the parameters of `model`
        else:
            net = model

        def epoch(e):
            net.set_epoch(e)
            opt.zero_grad(set_to_none=True)
            # mean negative log-likelihood of the labels, written as a gather: the same number as
            # F.nll_loss, whose CUDA kernels take 0.5 ms per epoch at this size
            loss = -net(x, graph).gather(1, y_col).mean()
            loss.backward()
            if world > 1:
                net.sync_gradients()
            opt.step()
            return loss

        for e in range(max(args.warmup, 3)):
            epoch(e)
        net.reset_cache()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for e in range(args.steps):
            loss = epoch(e)
        stop.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(stop) / args.steps
        if world > 1:
            t = torch.tensor([ms], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        report[str(width)] = {"epoch_ms": ms, "final_loss": float(loss.detach())}
        del model, net, opt, x
    from compressgnn_b200 import runtime as rt
    assert rt.device_status() == 0
    if world > 1:
        dist.destroy_process_group()
    if rank != 0:
        return
    line = {"metric": "gcn_epoch_ms", "value": report["256"]["epoch_ms"], "unit": "ms", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": report["256"]["epoch_ms"],
            "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "gcn: 2-layer GCN, propagation + transformation compression, config-2 graph",
                       "nodes": n, "orig_edges": e_orig, "rules": graph.rule_cnt, "levels": graph.step, "classes": 47,
                       "hidden": 128, "bits": 16, "refresh_interval": 5, "compressor": COMPRESS,
                       "parallelism": f"feature columns of every layer sharded over {world} GPU(s), graph replicated; "
                                      "collectives: projection all-reduce on refresh epochs, representative "
                                      "all-gather and gradient all-reduces every epoch"},
            "epoch_ms_by_feature_width": report, "gpu_launches": None}
    print(json.dumps(line))


def run_reference(args):
    """The reference's CPU implementation of the same workload, on this box's host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    wl = dict(WORKLOADS[args.workload])
    if args.width:
        wl["width"] = args.width
    world = int(os.environ.get("WORLD_SIZE", "1"))
    data, e_orig = build_graph(args.workload)
    # The CPU has no GPUs to scale over: it runs one 256-column block per step whatever N is; in the
    # weak-scaling configuration (N blocks) the time per step is N times that, the throughput the same.
    sec, kind, cores, sample = cpu_propagation(data, wl["width"], args.steps, min(args.warmup, 2))
    blocks = world if args.scaling == "weak" else 1
    if blocks > 1:
        sample += f"; one of {blocks} column blocks timed, step time scaled by {blocks}"
    total_width = wl["width"] * blocks
    sec *= blocks
    value = 2 * e_orig * total_width / sec / 1e9
    g = data.edge_index
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": int(os.environ.get("WORLD_SIZE", "1")),
        "steps": args.steps, "warmup": min(args.warmup, 2), "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{args.workload}: compressed propagation SpMM fwd+bwd, copying-model web graph",
                   "nodes": g.vertex_cnt, "orig_edges": e_orig, "compressed_edges": g.edge_count(),
                   "rules": g.rule_cnt, "levels": g.step, "feature_width": total_width, "compressor": COMPRESS},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["cgnn", "reference"], default="cgnn")
    ap.add_argument("--workload", choices=sorted(WORKLOADS) + ["cluster", "gcn"], default="propagation")
    ap.add_argument("--cluster-nodes", type=int, default=2450000)
    ap.add_argument("--width", type=int, default=0,
                    help="feature columns per GPU of a propagation workload (default: the workload's own)")
    ap.add_argument("--scaling", choices=["weak", "strong"], default="weak",
                    help="weak: every GPU holds a full-width (256-column) block of a feature matrix that is "
                         "N x 256*gpus; strong: the 256 columns are divided among the GPUs")
    ap.add_argument("--cpu-steps", type=int, default=3, help="steps of the CPU baseline leg")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg")
    args = ap.parse_args()
    if args.workload == "cluster":
        run_cluster(args)
    elif args.workload == "gcn":
        run_gcn(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
