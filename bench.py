"""Benchmark of the compressed-propagation hot path (and of the cluster / reconstruct operators
and the GCN epoch around it) on synthetic inputs.

    python bench.py --gpus N --steps K --warmup W            # this package, N GPUs (torchrun for N>1)
    python bench.py --impl reference --steps K --warmup W    # the reference's own CPU operators

Default workload ("propagation"): compressed propagation SpMM, forward + transposed backward,
on a seeded copying-model web graph with 325,557 nodes and ~3.2 M edges, features N x 256 fp32.
One step = one forward and one backward pass over the whole graph.  The metric is
original-edge x feature products per second: 2 * E_orig * F / t_step.

With N GPUs the feature columns are sharded and the graph replicated (no data-path collective).
The default is strong scaling -- the workload's 256 columns are divided among the GPUs, the job is
the same at every N; `--scaling weak` gives every GPU a full 256-column block instead.

Prints ONE JSON line (rank 0).  `value` is device-resident throughput (CUDA events, max over
ranks); `e2e` goes through the public host-buffer front end with pinned host matrices, copies included;
`roofline` is for the dominant kernel (the fused vertex pass of the forward); `cpu_baseline`
is the reference's CPU spmm_func chain on this host's cores, and `parity_checked` compares the
GPU's forward and backward results with that chain's on the same inputs.  `extra` carries short
legs of the other operator groups: the cluster / reconstruct operators at 2.45 M nodes, the
2-layer GCN epoch over four feature widths (sharded over the GPUs when N > 1), the grammar
compression of the workload's graph on the device beside the host compressor, and neighbour sampling
on the compressed graph beside the reference's host sampler.
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
TRAFFIC_RECORD = ROOT / "profiles" / "ncu_traffic.json"
KERNEL_SOURCES = ("compressgnn_b200/csrc/cgnn_segreduce.cu", "compressgnn_b200/csrc/cgnn_common.cuh",
                  "compressgnn_b200/csrc/cgnn_plan.h")


def kernel_source_hash():
    """sha256 over the sources the segment kernels are built from (ties a recorded ncu figure to
    the code it was captured from)."""
    import hashlib
    h = hashlib.sha256()
    for rel in KERNEL_SOURCES:
        h.update((ROOT / rel).read_bytes())
    return h.hexdigest()


def recorded_traffic(workload, width, world):
    """DRAM bytes (read + write) of one launch of the dominant kernel from the committed ncu
    capture, or (None, why) when no capture matches this workload and the current kernel sources."""
    if world != 1:
        return None, "captured on one GPU only"
    if not TRAFFIC_RECORD.is_file():
        return None, "no ncu capture recorded"
    for rec in json.loads(TRAFFIC_RECORD.read_text())["captures"]:
        if rec["workload"] == workload and rec["feature_width"] == width:
            if rec["kernel_source_sha256"] != kernel_source_hash():
                return None, "the kernel sources changed since the ncu capture of " + rec["captured"]
            return rec["dram_bytes_per_launch"], "ncu capture of " + rec["captured"]
    return None, "no ncu capture of this workload"


def build_graph(name, compression_backend="auto"):
    """Seeded copying-model graph -> CompressgnnData (self loops, symmetric normalisation,
    grammar compression, block partition).  Stands in for the public web graphs the reference's
    scripts load; nothing of those datasets is used.  The host and the device compressor return the
    same arrays, so the workload does not depend on `compression_backend`."""
    from compressgnn_b200 import offline as off
    from compressgnn_b200.loader import CompressgnnData
    w = WORKLOADS[name]
    n = w["n"]
    vlist, elist = off.generate_copy_graph(n, alpha=2.1, x_min=w["x_min"], max_degree=10000, copy_prob=0.7,
                                           window=64, candidates=8, seed=w["seed"])
    mask = np.ones(n, dtype=bool)
    data = CompressgnnData(np.zeros((n, 1), np.float32), (vlist, elist), np.zeros(n, np.int64), mask, mask, mask,
                           add_self_loop=True, normalize=True, graph_type="csr",
                           compression_backend=compression_backend, **COMPRESS)
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
# Shared pieces of the two arms
# ---------------------------------------------------------------------------------------------
def measured_peak():
    peaks_path = ROOT / "MEASURED_PEAKS.json"
    if peaks_path.is_file():
        return json.loads(peaks_path.read_text())["hbm_gbs"], "measured (MEASURED_PEAKS.json)"
    return 6650.0, "fallback"


def workload_config(name, data, e_orig, width_total, width, world, scaling):
    """The `config` object of the JSON line: the same dict from both arms."""
    g = data.edge_index
    return {"workload": f"{name}: compressed propagation SpMM fwd+bwd, copying-model web graph",
            "nodes": g.vertex_cnt, "orig_edges": e_orig, "compressed_edges": g.edge_count(),
            "rules": g.rule_cnt, "levels": g.step, "feature_width": width_total,
            "columns_per_gpu": width, "compressor": COMPRESS,
            "l2": "inputs larger than L2 (X is %.0f MB per GPU)" % (4e-6 * g.vertex_cnt * width),
            "parallelism": f"feature columns sharded over {world} GPU(s) ({scaling} scaling), graph replicated, "
                           "no collective"}


def widths_for(args, world):
    """(columns of the whole job, columns of one GPU)."""
    base = args.width or WORKLOADS[args.workload]["width"]
    if args.scaling == "weak":
        return base * world, base
    assert base % world == 0, "feature width must divide by the number of GPUs"
    return base, base // world


def host_inputs(n, width, seed):
    """Features and upstream gradient, drawn on the host so that the CPU and the GPU legs of one
    run can be given the same numbers."""
    import torch
    gen = torch.Generator().manual_seed(seed)
    return torch.randn(n, width, generator=gen), torch.randn(n, width, generator=gen)


def scaled_error(actual, expected):
    """max |a - b| / max(|b|, rms(row of b), rms(b)): the parity tests' bar for this is 1e-5 in fp32."""
    import torch
    a, b = actual.double(), expected.double()
    scale = torch.maximum(torch.maximum(b.abs(), b.pow(2).mean(dim=1, keepdim=True).sqrt()), b.pow(2).mean().sqrt())
    return float(((a - b).abs() / (scale + 1e-30)).max())


# ---------------------------------------------------------------------------------------------
# Reference CPU arm / CPU baseline
# ---------------------------------------------------------------------------------------------
def cpu_propagation(data, x, grad, steps, warmup):
    """The reference's CPU path: spmm_func(..., "rowbalance", ...) chained in the order of
    layer/CompressgnnSPMM.py:47-53 (forward) and :80-85 (backward), all host threads, on the host
    tensors `x` and `grad`.  Without the compiled reference the single-thread C restatement runs
    on the first 8 columns and the time is scaled.
    Returns (seconds per step, kind, cores, sample description, (out, grad_in) of the last step)."""
    import torch
    from oracle import oracle
    rt, _off = oracle.reference_modules()
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    g = data.edge_index
    width = x.size(1)
    if rt is not None:
        kind, sample_width = "reference", width
    else:
        kind, sample_width, cores = "port", min(width, 8), 1
        x, grad = x[:, :sample_width].contiguous(), grad[:, :sample_width].contiguous()
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
        result = step()
    dt = (time.perf_counter() - t0) / max(steps, 1)
    scale = width / sample_width  # a column slice scales linearly in the width
    sample = (f"full workload, {steps} steps" if sample_width == width else
              f"{sample_width} of {width} feature columns, {steps} steps, time scaled by {scale:g}")
    return dt * scale, kind, cores, sample, result


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------
def init_ranks():
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")  # keep NCCL's banner off stdout (one JSON line)
        dist.init_process_group("nccl", device_id=device)
    return world, rank, local_rank, device


def build_graph_once(name, world, rank):
    """Every rank needs the host graph.  The large workload takes minutes of host time to generate
    and compress, so with several ranks rank 0 builds it and hands it over through a file in shared
    memory instead of every rank repeating the work on the same cores."""
    import torch
    import torch.distributed as dist
    if world == 1 or WORKLOADS[name]["n"] < 2_000_000:
        return build_graph(name)
    path = Path("/dev/shm") / f"cgnn_bench_{os.environ.get('MASTER_PORT', '0')}_{name}.pt"
    if rank == 0:
        built = build_graph(name)
        torch.save(built, path)
    dist.barrier()
    if rank != 0:
        built = torch.load(path, weights_only=False)
    dist.barrier()
    if rank == 0:
        path.unlink()
    return built


def reference_cuda_leg(graph, x, grad, our_step, steps, e_orig, width_total):
    """Time the reference's CUDA kernels (oracle/_ref_cuda) on the resident inputs and compare their
    results with ours.  Returns the fields of the informational `reference_cuda` block, or None when the
    module is absent or the matrix is too large for the 32-bit index products of those kernels."""
    import torch
    from oracle import oracle
    module = oracle.reference_cuda_module()
    if module is None or max(graph.vertex_cnt, graph.rule_cnt) * x.size(1) >= 2 ** 31:
        return None
    for _ in range(3):
        ref_out, ref_gx = oracle.reference_cuda_step(module, graph, x, grad)
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        ref_out, ref_gx = oracle.reference_cuda_step(module, graph, x, grad)
    stop.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(stop) / steps
    out, gx = our_step()
    return {"ms_per_step": ms, "value": 2 * e_orig * width_total / (ms * 1e-3) / 1e9, "unit": UNIT,
            "what": "the reference's own CUDA kernels (src/runtime/csrc/sparse/cuda) compiled for sm_100, launched "
                    "in the order and with the method choice of layer/CompressgnnSPMM.py:14-19,54-60,80-85; "
                    "informational, not the reference arm",
            "max_scaled_error_forward_vs_ours": scaled_error(out.cpu(), ref_out.cpu()),
            "max_scaled_error_backward_vs_ours": scaled_error(gx.cpu(), ref_gx.cpu())}


def run_gpu(args):
    import torch
    import torch.distributed as dist
    from compressgnn_b200.layer import spmm as spmm_layer
    from compressgnn_b200 import runtime as rt

    world, rank, local_rank, device = init_ranks()
    width_total, width = widths_for(args, world)
    data, e_orig = build_graph_once(args.workload, world, rank)
    graph = data.edge_index
    n = graph.vertex_cnt
    warmup = max(args.warmup, 3)
    config = workload_config(args.workload, data, e_orig, width_total, width, world, args.scaling)

    # Inputs come from the host at sizes a host matrix is reasonable for (the same numbers then go to
    # the CPU leg); the 18.5 M-node workload draws them on the device.
    from_host = 4 * n * width <= 2**30
    if from_host:
        x_host, grad_host = host_inputs(n, width, 1234 + rank)
        x, grad = x_host.to(device), grad_host.to(device)
    else:
        gen = torch.Generator(device=device).manual_seed(1234 + rank)
        x = torch.randn(n, width, device=device, generator=gen)
        grad = torch.randn(n, width, device=device, generator=gen)

    # CPU baseline first (rank 0, N=1 only), while the graph blocks are still host tensors.
    cpu = cpu_result = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline and from_host:
        sec, kind, cores, sample, cpu_result = cpu_propagation(data, x_host, grad_host, args.cpu_steps, 1)
        cpu = {"value": 2 * e_orig * width_total / sec / 1e9, "unit": UNIT, "cores": cores, "kind": kind,
               "sample": sample, "ms_per_step": sec * 1e3}

    fwd_bytes, bwd_bytes = propagation_bytes(graph, width)
    graph.to(device)
    graph.propagation_plan()
    launches_per_step = 2 * (2 + graph.step)

    def step(record=None):
        out = spmm_layer._forward(graph, x, record)
        gx = spmm_layer._backward(graph, grad, record)
        return out, gx

    for _ in range(warmup):
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

    # Durations of the two fused vertex passes: events recorded inside the timed region (a pass is one
    # native call, split in two around its last launch so that the events can sit between them).
    def mean_ms(recs):
        per_launch = {}
        for rec in recs:
            for name, e0, e1 in rec:
                per_launch.setdefault(name, []).append(e0.elapsed_time(e1))
        return {k: float(np.mean(v)) for k, v in per_launch.items()}

    launch_ms = mean_ms(records)
    bytes_by_name = dict(fwd_bytes + bwd_bytes)
    # The six-launch table comes from a second pass of the same steps in which every block is issued
    # by a call of its own with events around it (slower on the host, same kernels).
    detail = []
    for _ in range(args.steps):
        rec = []
        spmm_layer._forward(graph, x, rec, per_block=True)
        spmm_layer._backward(graph, grad, rec, per_block=True)
        detail.append(rec)
    torch.cuda.synchronize()
    detail_ms = mean_ms(detail)

    # the GPU's results against the CPU leg's, same inputs (N=1)
    parity = None
    if cpu_result is not None:
        out, gx = step()
        cols = cpu_result[0].size(1)
        err_f = scaled_error(out[:, :cols].cpu(), cpu_result[0])
        err_b = scaled_error(gx[:, :cols].cpu(), cpu_result[1])
        parity = {"against": f"cpu_baseline ({cpu['kind']}), same inputs, {cols} of {width} columns",
                  "max_scaled_error_forward": err_f, "max_scaled_error_backward": err_b, "tolerance": 1e-5,
                  "ok": bool(err_f <= 1e-5 and err_b <= 1e-5)}
        del out, gx
        assert parity["ok"], f"GPU and CPU results differ: {parity}"

    # end to end through the public host-buffer front end: pinned host operands, every upload
    # and download inside the timed region, passes queued so that the two copy directions overlap
    e2e_sec = e2e_sync_sec = None
    if not args.no_e2e and from_host:
        from compressgnn_b200.layer import HostPropagation
        pipe = HostPropagation(graph, width)
        x_pin = x_host.pin_memory()
        g_pin = grad_host.pin_memory()
        out_host = torch.empty_like(x_pin).pin_memory()
        gx_host = torch.empty_like(x_pin).pin_memory()

        def e2e_steps(count, wait_each):
            if world > 1:
                dist.barrier()
            t0 = time.perf_counter()
            for _ in range(count):
                pipe.forward(x_pin, out_host)
                pipe.backward(g_pin, gx_host)
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
        del pipe, x_pin, g_pin, out_host, gx_host

    # For context only (never a ratio's denominator): the reference's own CUDA kernels, compiled for
    # sm_100, on the same graph and inputs, launched as the reference's GPU branches launch them.
    ref_cuda = None
    if rank == 0 and world == 1 and not args.no_reference_cuda:
        ref_cuda = reference_cuda_leg(graph, x, grad, step, args.steps, e_orig, width_total)

    rt.raise_on_device_status()
    del x, grad

    # short legs of the other operator groups, after the timed region of the headline workload
    extra = {}
    if not args.no_extra and WORKLOADS[args.workload]["n"] < 2_000_000:
        if world == 1:
            extra["compress"] = measure_compress(args.workload, 3, with_cpu=not args.no_cpu_baseline)
            extra["sample"] = measure_sample(args.workload, 20, with_cpu=not args.no_cpu_baseline)
            extra["cluster"] = measure_cluster(args.cluster_nodes, max(3, min(args.steps, 10)), 3,
                                               with_cpu=not args.no_cpu_baseline)
        extra["gcn"] = measure_gcn(graph, e_orig, max(5, min(args.steps, 20)), 5, world, rank, device)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return

    peak, peak_src = measured_peak()
    dom = "fwd_out"
    achieved = bytes_by_name[dom] / (launch_ms[dom] * 1e-3) / 1e9
    traffic, traffic_src = recorded_traffic(args.workload, width, world)
    work = 2 * e_orig * width_total
    line = {
        "metric": METRIC, "value": work / (ms_per_step * 1e-3) / 1e9, "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config,
        "e2e": ({"value": work / e2e_sec / 1e9, "unit": UNIT, "h2d_bytes_per_step": 2 * 4 * n * width,
                 "d2h_bytes_per_step": 2 * 4 * n * width, "ms_per_step": e2e_sec * 1e3,
                 "ms_per_step_waiting_each_step": e2e_sync_sec * 1e3,
                 "host_GBps_all_ranks": 4 * 4 * n * width * world / e2e_sec / 1e9,
                 "limit": "host memory / PCIe: every step moves the feature matrix and the result both ways",
                 "api": "HostPropagation.forward/backward on pinned host matrices"} if e2e_sec else None),
        "gpu_launches": launches_per_step * args.steps,
        "roofline": {"bound": "hbm", "kernel": "fused v2r+v2v vertex pass of the forward (segment-reduce kernel)",
                     "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_source": peak_src, "traffic": traffic, "traffic_source": traffic_src,
                     "algorithmic_bytes_per_launch": bytes_by_name[dom], "ms_per_launch": launch_ms[dom],
                     "launches": {k: {"ms": detail_ms[k], "algorithmic_GBps": bytes_by_name[k] / detail_ms[k] / 1e6}
                                  for k in detail_ms},
                     "launches_source": "second pass of the same steps, one call and one event pair per block"},
        "clocks": clocks.summary(),
    }
    if world > 1 and args.scaling == "strong":
        # what column sharding can give at best: feature bytes divide by N, the index stream does not
        full = dict(fwd_bytes + bwd_bytes)
        shard_bytes = sum(full.values())
        index_bytes = 8 * graph.edge_count() * 2
        one_gpu = (shard_bytes - index_bytes) * world + index_bytes
        line["strong_scaling_ceiling_by_bytes"] = one_gpu / (world * shard_bytes)
    if cpu is not None:
        line["cpu_baseline"] = cpu
    if ref_cuda is not None:
        line["reference_cuda"] = ref_cuda
    if parity is not None:
        line["parity_checked"] = parity
    if extra:
        line["extra"] = extra
    print(json.dumps(line))


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


def measure_cluster(n, steps, warmup, with_cpu=True):
    """Config 3: Compressgnn_Cluster -> Linear(128->256) on representatives -> fused reconstruct
    (bias + ReLU), forward + backward, `n` nodes drawn from 4096 Gaussian centroids, H=16,
    refresh_interval=5.  A step = one epoch.  Per-operator CUDA-event times and algorithmic GB/s
    are reported next to the epoch time; the CPU leg runs the reference's cluster_forward
    plus the torch CPU formulas its layers use.  Returns the fields of a JSON line."""
    import torch
    from compressgnn_b200 import runtime as rt
    from compressgnn_b200.layer import Compressgnn_Cluster, Compressgnn_Reconstruct
    width, out_width, bits = 128, 256, 16
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

    # warm-up runs past a second assignment refresh (epoch 5): that is where the previous assignment and the new
    # one are alive together, and torch's caching allocator should have met that peak before the timed region
    # (an epoch that sends it back to cudaMalloc takes 10-40 ms)
    warm_epochs = max(warmup, 7)
    for e in range(warm_epochs):
        epoch(e)
    cluster.reset_cache()
    cluster.refresh_count = 0
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    plans_before = rt.SegmentPlan.built_from_index
    mallocs_before = torch.cuda.memory_stats().get("num_device_alloc", 0)
    with ClockSampler(torch.cuda.current_device()) as clocks:
        start.record()
        marks[0].record()
        for e in range(steps):
            epoch(e)
            marks[e + 1].record()
        stop.record()
        torch.cuda.synchronize()
    plans_sorted = rt.SegmentPlan.built_from_index - plans_before  # 0: every refresh handed its plan over
    device_mallocs = torch.cuda.memory_stats().get("num_device_alloc", 0) - mallocs_before
    ms_epoch = start.elapsed_time(stop) / steps
    each = sorted(a.elapsed_time(b) for a, b in zip(marks, marks[1:]))  # a stalled epoch shows as max >> median

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
                                                          4 * n * width + 4 * width * bits + 8 * n + 4 * 2**bits),
        "cluster_mean": (lambda: rt.cluster_mean(xd, ids, counts), 4 * n * width + 8 * n + 4 * groups * width),
        "cluster_mean_backward": (lambda: rt.cluster_mean_backward(g_small, ids, counts),
                                  4 * groups * width + 8 * n + 4 * n * width),
        "cluster_reconstruct (bias+relu)": (lambda: rt.cluster_reconstruct(table, ids, bias, True),
                                            4 * groups * out_width + 8 * n + 4 * out_width + 4 * n * out_width),
        "cluster_reconstruct (bias+relu+dropout 0.3)": (
            lambda: rt.cluster_reconstruct(table, ids, bias, True, dropout_p=0.3, seed=5),
            4 * groups * out_width + 8 * n + 4 * out_width + 4 * n * out_width),
        "cluster_reconstruct_backward (relu, exact mask)": (
            lambda: rt.cluster_reconstruct_backward(grad_out, ids, y, groups, True),
            8 * n * out_width + 8 * n + 4 * groups * out_width),
        "cluster_reconstruct_backward (relu, one mask row per group)": (
            lambda: rt.cluster_reconstruct_backward(grad_out, ids, y, groups, True, output_is_forward_result=True),
            4 * n * out_width + 8 * n + 8 * groups * out_width),
    }
    peak, peak_src = measured_peak()
    op_report = {}
    for name, (fn, nbytes) in ops.items():
        ms = timed(fn)
        op_report[name] = {"ms": ms, "algorithmic_bytes": nbytes, "algorithmic_GBps": nbytes / ms / 1e6,
                           "frac_of_peak": nbytes / ms / 1e6 / peak}
    # For context: the same operators by the reference's own CUDA kernels (oracle/_ref_cuda) on the same
    # tensors -- its assignment through a library GEMM and a 2^bits histogram, its means and the
    # reconstruct backward through float atomics, its gather/scatter kernels one element per thread.
    from oracle import oracle
    ref = oracle.reference_cuda_module()
    if ref is not None and n * out_width < 2 ** 31:
        rws = ref.cluster_workspace(xd, bits)
        ref_ops = {
            "cluster_assign (projection+codes+compaction)": lambda: ref.cluster_assign(xd, cluster.random_vectors, bits, rws),
            "cluster_mean": lambda: ref.cluster_mean(xd, ids, counts),
            "cluster_mean_backward": lambda: ref.cluster_mean_backward(g_small, ids, counts),
            "cluster_reconstruct (bias+relu)": lambda: ref.cluster_reconstruct(table, ids, bias, True),
            "cluster_reconstruct_backward (relu, exact mask)": lambda: ref.cluster_reconstruct_backward(grad_out, ids, y, groups, True),
        }
        for name, fn in ref_ops.items():
            op_report[name]["reference_cuda_ms"] = timed(fn, 10)
    rt.raise_on_device_status()
    # the operator that moves the most bytes per epoch is the roofline's subject
    dom = "cluster_reconstruct (bias+relu)"
    report = {"metric": "cluster_linear_reconstruct_nodes_per_s", "value": n / (ms_epoch * 1e-3) / 1e6, "unit": "Mnode/s",
              "steps": steps, "warmup": warm_epochs, "ms_per_step": ms_epoch, "ms_per_step_median": each[len(each) // 2],
              "ms_per_step_max": each[-1], "index_plans_rebuilt_in_timed_region": plans_sorted,
              "allocator_cudamallocs_in_timed_region": device_mallocs, "higher_is_better": True,
              "dtype": "f32", "data": "synthetic",
              "config": {"workload": "cluster: Compressgnn_Cluster + Linear 128->256 + Compressgnn_Reconstruct(relu), fwd+bwd",
                         "nodes": n, "feature_width": width, "out_width": out_width, "bits": bits, "centroids": 4096,
                         "active_buckets": active, "refresh_interval": 5, "refreshes": cluster.refresh_count,
                         "l2": "inputs larger than L2 (X is %.0f MB)" % (4e-6 * n * width)},
              "operators": op_report,
              "roofline": {"bound": "hbm", "kernel": dom, "achieved": op_report[dom]["algorithmic_GBps"], "peak": peak,
                           "unit": "GB/s", "frac": op_report[dom]["frac_of_peak"], "peak_source": peak_src,
                           "traffic": None, "traffic_source": "see the ncu summary of the cluster kernels (600 k nodes)",
                           "algorithmic_bytes_per_launch": op_report[dom]["algorithmic_bytes"],
                           "ms_per_launch": op_report[dom]["ms"]},
              "clocks": clocks.summary()}
    del x, grad_out, y, reps, table, xd
    if with_cpu:
        report["cpu_baseline"] = cpu_cluster(n, width, out_width, bits)
    return report


def measure_compress(name, steps, with_cpu=True):
    """Grammar compression of a workload's graph (self loops added) on the device, the two host arrays in
    and the two host arrays out: host time around `compress_graph_csr(..., backend='cuda')`, the median of
    `steps` calls after one warm-up call; the host compressor on the box's cores beside it, and whether the
    two returned the same arrays."""
    from compressgnn_b200 import offline as off
    from compressgnn_b200.loader import compress_graph_csr
    w = WORKLOADS[name]
    vlist, elist = off.generate_copy_graph(w["n"], alpha=2.1, x_min=w["x_min"], max_degree=10000, copy_prob=0.7,
                                           window=64, candidates=8, seed=w["seed"])
    vlist, elist = off.add_self_loop_csr(vlist, elist)
    frequency = COMPRESS["min_pair_frequency"]
    device = compress_graph_csr(vlist, elist, frequency, backend="cuda")
    times = []
    for _ in range(max(steps, 1)):
        t0 = time.perf_counter()
        device = compress_graph_csr(vlist, elist, frequency, backend="cuda")
        times.append(time.perf_counter() - t0)
    sec = sorted(times)[len(times) // 2]
    edges = int(elist.size)
    report = {"metric": "compress_edges_per_s", "value": edges / sec / 1e6, "unit": "Medge/s", "ms_per_step": sec * 1e3,
              "steps": len(times), "warmup": 1, "higher_is_better": True, "dtype": "int32", "data": "synthetic",
              "config": {"workload": f"compress: digram-substitution grammar compression of the {name} graph, "
                                     "host arrays in and out", "nodes": w["n"], "edges": edges,
                         "entries_out": int(device[1].size), "rules": int(device[3]), "rounds": 12,
                         "min_pair_frequency": frequency}}
    if with_cpu:
        cores = os.cpu_count() or 1
        t0 = time.perf_counter()
        host = compress_graph_csr(vlist, elist, frequency, backend="cpu", threads=cores)
        host_sec = time.perf_counter() - t0
        report["cpu_baseline"] = {"value": edges / host_sec / 1e6, "unit": "Medge/s", "cores": cores, "kind": "port",
                                  "ms_per_step": host_sec * 1e3,
                                  "sample": "the whole graph once, this package's host compressor (the reference's "
                                            "compressor is an external project that its tree does not contain)"}
        report["parity_checked"] = {"against": "host compressor", "arrays_equal": bool(
            np.array_equal(device[0], host[0]) and np.array_equal(device[1], host[1]) and device[3] == host[3])}
    return report


def measure_sample(name, batches, batch_size=1024, fanouts=(25, 10), with_cpu=True):
    """Neighbour sampling on the compressed graph of a workload: mini-batches of `batch_size` seed nodes drawn
    without replacement, two hops with the fan-outs GraphSAGE-style loaders use; CUDA events around `batches`
    batches after three warm-up batches (host time around them as well: a batch ends with the host knowing
    the sizes).  CPU baseline: the reference's own host sampler compiled from its sources (oracle/_ref) on
    the same graph arrays and seeds, one thread (it has no parallel form), on a bounded number of batches."""
    import torch
    from compressgnn_b200.sample import CompressGraphSampler
    from oracle import oracle
    data, e_orig = build_graph(name)
    graph = data.edge_index
    host = None
    if with_cpu:
        host = [t.clone() for b in (graph.v2v_graph, graph.v2r_graph, graph.r2v_graph) for t in b.csr()[:2]]
        host_levels = ([l.csr()[0].clone() for l in graph.r2r_graph], [l.csr()[1].clone() for l in graph.r2r_graph])
        host_degrees = (graph.vertex_degree.clone(), graph.rule_degree.clone())
    levels = graph.step
    graph.to("cuda")
    sampler = CompressGraphSampler.from_graph(graph)
    gen = torch.Generator().manual_seed(11)
    seeds = [torch.randperm(graph.vertex_cnt, generator=gen)[:batch_size] for _ in range(batches + 3)]
    device_seeds = [s.cuda() for s in seeds]
    edges = 0
    for s in device_seeds[:3]:
        sampler(s, fanouts, seed=1)
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    start.record()
    for i, s in enumerate(device_seeds[3:]):
        edges += sampler(s, fanouts, seed=i)[1].numel()
    stop.record()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    ms = start.elapsed_time(stop) / batches
    report = {"metric": "sampled_edges_per_s", "value": edges / batches / ms / 1e3, "unit": "Medge/s", "ms_per_step": ms,
              "host_ms_per_step": wall * 1e3 / batches, "steps": batches, "warmup": 3, "higher_is_better": True,
              "dtype": "int64", "data": "synthetic",
              "config": {"workload": f"sample: neighbour sampling on the compressed {name} graph", "nodes": graph.vertex_cnt,
                         "orig_edges": e_orig, "rules": graph.rule_cnt, "levels": levels, "batch": batch_size,
                         "fanouts": list(fanouts), "sampled_edges_per_batch": edges / batches}}
    ref = oracle.reference_sample_module() if with_cpu else None
    if with_cpu and ref is None:
        report["cpu_baseline"] = {"value": None, "unit": "Medge/s", "cores": 0, "kind": "reference",
                                  "sample": "unavailable: oracle/_ref/compressgnn_sample.so is not built on this box"}
    elif with_cpu and levels > 1:
        report["cpu_baseline"] = {"value": None, "unit": "Medge/s", "cores": 0, "kind": "reference",
                                  "sample": "not run: the reference's sampler indexes the rule levels by descent depth and "
                                            "does not follow rules nested more than one level deep"}
    elif with_cpu:
        n_cpu = min(batches, 8)
        cpu_edges = 0
        t0 = time.perf_counter()
        for s in seeds[3:3 + n_cpu]:
            cpu_edges += ref.neighbor_sample_cg_sim(*host, host_levels[0], host_levels[1], *host_degrees, s,
                                                    list(fanouts))[1].numel()
        cpu_sec = time.perf_counter() - t0
        report["cpu_baseline"] = {"value": cpu_edges / cpu_sec / 1e6, "unit": "Medge/s", "cores": 1, "kind": "reference",
                                  "ms_per_step": cpu_sec * 1e3 / n_cpu,
                                  "sample": f"{n_cpu} of the {batches} batches, the reference's host sampler (one thread)"}
    return report


def run_sample(args):
    import torch
    torch.cuda.set_device(0)
    report = measure_sample(args.graph, args.steps, with_cpu=not args.no_cpu_baseline)
    print(json.dumps(dict(report, n_gpus=1, scaling="strong", vs_baseline=None, gpu_launches=None)))


def run_compress(args):
    import torch
    torch.cuda.set_device(0)
    report = measure_compress(args.graph, min(args.steps, 5), with_cpu=not args.no_cpu_baseline)
    print(json.dumps(dict(report, n_gpus=1, scaling="strong", vs_baseline=None, gpu_launches=None)))


def run_cluster(args):
    import torch
    torch.cuda.set_device(0)
    report = measure_cluster(args.cluster_nodes, args.steps, args.warmup, with_cpu=not args.no_cpu_baseline)
    line = dict(report, n_gpus=1, scaling="strong", vs_baseline=None, gpu_launches=None)
    print(json.dumps(line))


def cpu_gcn_epoch(data, width, classes=47, hidden=128, bits=16, epochs=3):
    """One training epoch of the same 2-layer model on the host cores (all threads): propagation by the
    reference's CPU spmm_func chain (forward and, through a small autograd wrapper, backward), bucket
    assignment by its cluster_forward, means / Linear / reconstruct by the torch CPU formulas of its
    layers (layer/CompressgnnCluster.py:16-25, layer/CompressgnnReconstruct.py:39-42)."""
    import torch
    from oracle import oracle
    rt, _off = oracle.reference_modules()
    if rt is None:
        return {"value": None, "unit": "ms", "cores": 0, "kind": "reference",
                "sample": "unavailable: oracle/_ref is not built on this box"}
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    g = data.edge_index
    n = g.vertex_cnt
    fwd = dict(r2v=g.r2v_graph.csr(), v2r=g.v2r_graph.csr(), v2v=g.v2v_graph.csr(), levels=[l.csr() for l in g.r2r_graph])
    bwd = dict(v2r_t=g.v2r_graph.csc(), v2v_t=g.v2v_graph.csc(), r2v_t=g.r2v_graph.csc(),
               levels_t=[l.csc() for l in g.r2r_graph])
    spmm = lambda blk, m, out=None: rt.spmm_func(blk[0], blk[1], blk[2], m, "rowbalance", out)

    class Propagate(torch.autograd.Function):
        @staticmethod
        def forward(ctx, x):
            rule = spmm(fwd["r2v"], x)
            for lvl in fwd["levels"]:
                rule = spmm(lvl, rule, rule)
            return spmm(fwd["v2v"], x, spmm(fwd["v2r"], rule))

        @staticmethod
        def backward(ctx, grad):
            grad = grad.contiguous()
            rule = spmm(bwd["v2r_t"], grad)
            for lvl in reversed(bwd["levels_t"]):
                rule = spmm(lvl, rule, rule)
            return spmm(bwd["r2v_t"], rule, spmm(bwd["v2v_t"], grad))

    gen = torch.Generator().manual_seed(5)
    x = torch.randn(n, width, generator=gen)
    y = torch.randint(0, classes, (n, 1), generator=gen)
    lins = [torch.nn.Linear(width, hidden), torch.nn.Linear(hidden, classes)]
    planes = [torch.randn(width, bits, generator=gen), torch.randn(hidden, bits, generator=gen)]
    opt = torch.optim.Adam([p for l in lins for p in l.parameters()], lr=1e-3)
    state = [None, None]

    def layer(i, h, refresh):
        p = Propagate.apply(h)
        if refresh or state[i] is None:
            ids, active = rt.cluster_forward(p.detach().contiguous(), planes[i], bits)
            index = ids.long()
            state[i] = (index, torch.bincount(index, minlength=active + 1).clamp_min(1).to(torch.float32))
        index, counts = state[i]
        reps = torch.zeros(counts.numel(), p.size(1)).index_add_(0, index, p) / counts[:, None]
        return torch.nn.functional.linear(reps, lins[i].weight, None).index_select(0, index) + lins[i].bias

    def epoch(e):
        opt.zero_grad(set_to_none=True)
        h = torch.nn.functional.dropout(layer(0, x, e % 5 == 0).relu(), 0.3)
        loss = -torch.log_softmax(layer(1, h, e % 5 == 0), 1).gather(1, y).mean()
        loss.backward()
        opt.step()

    epoch(0)
    t0 = time.perf_counter()
    for e in range(1, epochs + 1):
        epoch(e)
    ms = (time.perf_counter() - t0) / epochs * 1e3
    return {"value": ms, "unit": "ms", "cores": cores, "kind": "reference", "feature_width": width,
            "sample": f"whole graph, {epochs} epochs after one warm-up epoch (none of them a refresh epoch)"}


def measure_gcn(graph, e_orig, steps, warmup, world, rank, device, widths=(16, 64, 256, 1024)):
    """Config 5: end-to-end 2-layer GCN with propagation and transformation compression
    (use_transformation=True, H=16, refresh_interval=5) on the config-2 graph (already on `device`),
    47 uniform classes, input feature width swept over 16/64/256/1024.  A step = one training epoch
    (forward, NLL loss on all nodes, backward, Adam step), timed after warm-up epochs as the reference's
    benchmark/end2end/compressgnn_gcn.py does.  With N GPUs the same model and matrix run with the feature
    columns of every layer sharded when the input has 512 columns or more, else as one replica per GPU
    (`dist.place_model`); the graph is replicated either way."""
    import torch
    import torch.distributed as dist
    from compressgnn_b200.model import GCN
    from compressgnn_b200 import dist as cdist
    from compressgnn_b200 import runtime as rt
    n = graph.vertex_cnt
    gen = torch.Generator(device=device).manual_seed(5)  # the same labels and features on every rank
    y = torch.randint(0, 47, (n,), device=device, generator=gen)
    y_col = y.unsqueeze(1)
    report = {}
    for width in widths:
        x = torch.randn(n, width, device=device, generator=gen)
        torch.manual_seed(5)
        model = GCN(width, 47, hidden_features=128, param_H=16, dropout=0.3, use_transformation=True,
                    refresh_interval=5, num_layers=2).to(device)
        opt = torch.optim.Adam(model.parameters(), lr=1e-3, fused=True)  # one kernel for all parameters
        # N > 1: column-sharded from 512 input columns up (shares the parameters of `model`), a replica on
        # every rank below that, where the collectives of a sharded epoch cost more than the shards save
        net, sharded = cdist.place_model(model, width, dist.group.WORLD if world > 1 else None)
        if sharded:
            x = cdist.shard_columns(x, rank, world)

        def epoch(e):
            net.set_epoch(e)
            opt.zero_grad(set_to_none=True)
            # mean negative log-likelihood of the labels, written as a gather: the same number as
            # F.nll_loss, whose CUDA kernels take 0.5 ms per epoch at this size
            loss = -net(x, graph).gather(1, y_col).mean()
            loss.backward()
            opt.step()  # N > 1: every rank steps on the weight rows it owns (see ShardedGCN.consolidate_parameters)
            return loss

        for e in range(max(warmup, 7)):  # past the second refresh, as in the cluster leg
            epoch(e)
        net.reset_cache()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
        start.record()
        marks[0].record()
        for e in range(steps):
            loss = epoch(e)
            marks[e + 1].record()
        stop.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(stop) / steps
        each = sorted(a.elapsed_time(b) for a, b in zip(marks, marks[1:]))
        if world > 1:
            t = torch.tensor([ms], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        if sharded:
            net.consolidate_parameters()
        report[str(width)] = {"epoch_ms": ms, "epoch_ms_median": each[len(each) // 2], "epoch_ms_max": each[-1],
                              "final_loss": float(loss.detach()),
                              "placement": "columns sharded" if sharded else ("replica per GPU" if world > 1 else "one GPU")}
        del model, net, opt, x
    rt.raise_on_device_status()
    return {"metric": "gcn_epoch_ms", "unit": "ms", "steps": steps, "warmup": max(warmup, 7), "n_gpus": world,
            "scaling": "strong", "higher_is_better": False, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "gcn: 2-layer GCN, propagation + transformation compression, config-2 graph",
                       "nodes": n, "orig_edges": e_orig, "rules": graph.rule_cnt, "levels": graph.step, "classes": 47,
                       "hidden": 128, "bits": 16, "refresh_interval": 5, "optimizer": "torch.optim.Adam(lr=1e-3, fused=True)",
                       "compressor": COMPRESS,
                       "parallelism": f"{world} GPU(s), graph replicated; inputs of 512 columns and more: feature "
                                      "columns of every layer sharded; narrower inputs: one replica per GPU, no "
                                      "collective (`placement` per width); collectives of a sharded epoch: "
                                      "projection all-reduce on refresh epochs; per hidden layer and "
                                      "epoch one all-gather of the representatives and one reduce-scatter of "
                                      "their gradient; no weight-gradient exchange (each rank steps on the "
                                      "weight rows it owns)"},
            "epoch_ms_by_feature_width": report}


def run_gcn(args):
    import torch.distributed as dist
    world, rank, _local_rank, device = init_ranks()
    data, e_orig = build_graph("propagation")
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu = cpu_gcn_epoch(data, 256)
    graph = data.edge_index
    graph.to(device)
    report = measure_gcn(graph, e_orig, args.steps, args.warmup, world, rank, device)
    if world > 1:
        dist.destroy_process_group()
    if rank != 0:
        return
    ms = report["epoch_ms_by_feature_width"]["256"]["epoch_ms"]
    line = dict(report, value=ms, ms_per_step=ms, vs_baseline=None, gpu_launches=None)
    if cpu is not None:
        line["cpu_baseline"] = cpu
    print(json.dumps(line))


def run_reference(args):
    """The reference's CPU implementation of the same workload, on this box's host cores: the same
    graph, inputs, `config`, steps and warm-up as the GPU arm."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    width_total, width = widths_for(args, world)
    data, e_orig = build_graph(args.workload, compression_backend="cpu")  # nothing of this arm touches the GPU
    warmup = max(args.warmup, 3)
    # The CPU has no GPUs to scale over.  Strong scaling: it runs the whole job (all columns) whatever N
    # is.  Weak scaling (N blocks of columns): one block is timed and the step time multiplied by N.
    base = args.width or WORKLOADS[args.workload]["width"]
    x, grad = host_inputs(data.edge_index.vertex_cnt, base, 1234)
    sec, kind, cores, sample, _ = cpu_propagation(data, x, grad, args.steps, warmup)
    blocks = width_total // base
    if blocks > 1:
        sample += f"; one of {blocks} column blocks timed, step time scaled by {blocks}"
        sec *= blocks
    value = 2 * e_orig * width_total / sec / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.workload, data, e_orig, width_total, width, world, args.scaling),
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
    ap.add_argument("--workload", choices=sorted(WORKLOADS) + ["cluster", "gcn", "compress", "sample"],
                    default="propagation")
    ap.add_argument("--cluster-nodes", type=int, default=2450000)
    ap.add_argument("--graph", choices=sorted(WORKLOADS), default="propagation",
                    help="graph of the compress and sample workloads")
    ap.add_argument("--width", type=int, default=0,
                    help="feature columns of a propagation workload (default: the workload's own)")
    ap.add_argument("--scaling", choices=["strong", "weak"], default="strong",
                    help="strong: the workload's columns are divided among the GPUs (the same job at every N); "
                         "weak: every GPU holds a full-width block of a feature matrix that is N x width*gpus")
    ap.add_argument("--cpu-steps", type=int, default=3, help="steps of the CPU baseline leg")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg")
    ap.add_argument("--no-reference-cuda", action="store_true",
                    help="skip the informational leg that times the reference's own CUDA kernels")
    ap.add_argument("--no-extra", action="store_true", help="skip the cluster and GCN legs reported under `extra`")
    args = ap.parse_args()
    if args.workload == "compress":
        run_compress(args)
    elif args.workload == "sample":
        run_sample(args)
    elif args.workload == "cluster":
        run_cluster(args)
    elif args.workload == "gcn":
        run_gcn(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
