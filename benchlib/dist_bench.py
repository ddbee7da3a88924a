"""Sharded leg of bench.py: the row-partitioned AutoSAGEConv forward on the ogbn-products-sized graph.

Launched by ``torch.distributed.run`` with one rank per GPU.  Every rank builds the same seeded
graph on its own GPU, keeps its nnz-balanced row shard, and the timed step is: gather of X over
NVLink (copy-engine pulls from peer memory, or NCCL send/recv; overlapped, shard by shard, with the
column-block SpMMs) followed by the Linear F->256 on the local rows.  Time is the maximum over ranks of the CUDA-event time between two barriers; the
reported value is whole-job algorithmic bytes (SpMM: CSR + gathered X + output; Linear: read
aggregated rows + write outputs) divided by that time.  Strong scaling: total work is fixed.
"""
from __future__ import annotations

import os
import statistics
import time

import torch
import torch.distributed as dist


EXCHANGE_NAMES = {
    "peer": "copy-engine pulls from peer memory",
    "nccl": "NCCL send/recv steps",
    "allgather": "NCCL all_gather_into_tensor per chunk",
    "push": "SM-driven 128-bit stores into peer memory per chunk",
}


def conv_bytes(n_rows: int, nnz: int, f: int, out_f: int) -> int:
    spmm = 8 * (n_rows + 1) + 8 * nnz + 4 * nnz * f + 4 * n_rows * f
    linear = 4 * n_rows * f + 4 * n_rows * out_f
    return spmm + linear


def bind_to_gpu_numa_node(local_rank: int) -> dict:
    """Restrict this process to the CPUs of the NUMA node its GPU hangs off (read from sysfs), so that
    the pinned host buffers allocated afterwards land in that node's memory.  With one process per GPU
    started by torch.distributed.run nothing else decides where pinned pages go, and copies between a GPU
    and the other socket's memory cross the inter-socket link.  Returns what it found and did."""
    found = {"gpu_numa_node": None, "bound_cpus": None, "cpus_before": len(os.sched_getaffinity(0))}
    try:
        props = torch.cuda.get_device_properties(local_rank)
        if hasattr(props, "pci_bus_id"):
            address = f"{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        else:
            import pynvml

            pynvml.nvmlInit()
            raw = pynvml.nvmlDeviceGetPciInfo(pynvml.nvmlDeviceGetHandleByIndex(local_rank)).busId
            address = (raw.decode() if isinstance(raw, bytes) else raw).lower()[-12:]
        found["pci"] = address
        node = int(open(f"/sys/bus/pci/devices/{address}/numa_node").read().strip())
        found["gpu_numa_node"] = node
        if node >= 0:
            cpus = set()
            for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
                first, _, last = part.partition("-")
                cpus.update(range(int(first), int(last or first) + 1))
            allowed = cpus & os.sched_getaffinity(0)
            if allowed:
                os.sched_setaffinity(0, allowed)
                found["bound_cpus"] = len(allowed)
    except (OSError, ValueError, ImportError, AttributeError, RuntimeError) as exc:
        found["error"] = f"{type(exc).__name__}: {exc}"
    return found


def compare_with_single_gpu(single_rows, y_sharded, out_sharded, weight) -> tuple[float, float]:
    """Worst error/bound of this rank's aggregated rows and layer outputs against the single-GPU run.
    Both sides are float32 results that each lie within rtol 1e-5 / atol 1e-5*sqrt(degree) of the exact
    value, so their difference may reach twice that; the layer's bound is the aggregation's carried
    through |W| plus the projection's own rounding."""
    y_single, out_single, root_degree = single_rows
    bound_y = 2.0 * (1e-5 * y_single.double().abs() + 1e-5 * root_degree[:, None])
    ratio_y = float(((y_sharded.double() - y_single.double()).abs() / bound_y).max()) if y_single.numel() else 0.0
    carried = bound_y.float() @ weight.abs().t()
    bound_out = carried.double() + 2.0 * (1e-5 * out_single.double().abs() + 1e-5 * weight.size(1) ** 0.5)
    ratio_out = float(((out_sharded.double() - out_single.double()).abs() / bound_out).max()) if out_single.numel() else 0.0
    return ratio_y, ratio_out


def _single_gpu_extras(args, bench, shard, layer, algorithmic, n, nnz, f, out_f, device) -> dict:
    """N = 1 only: the library comparator (cuSPARSE + cuBLAS), the CPU baseline on a bounded sample,
    and short runs of the other single-GPU configurations."""
    import argparse

    extras = {}
    stream = torch.cuda.current_stream()
    with torch.no_grad():
        matrix = torch.sparse_csr_tensor(shard.crow, shard.col, torch.ones(nnz, device=device), size=(n, n))
        x = layer.spmm.x_full

        def library_step():
            return layer.linear(torch.sparse.mm(matrix, x))

        library_step()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(3):
            library_step()
        b.record(stream)
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / 3
        extras["gpu_comparator"] = {"name": "torch.sparse.mm (cuSPARSE) + nn.Linear (cuBLAS), the reference's GPU fallback",
                                    "ms_per_step": round(ms, 4),
                                    "value": round(algorithmic / (ms * 1e-3) / 1e9, 2), "unit": "GB/s"}
        del matrix
        extras["fused_layer_kernel"] = _fused_layer_case(shard, layer, x, f, out_f, device)
    if not args.no_cpu_baseline:
        sub = argparse.Namespace(**vars(args))
        sub.steps, sub.warmup = 2, 1
        ref = bench.run_reference(sub)
        extras["cpu_baseline"] = dict(ref["cpu_baseline"], ms_per_step_on_sample=ref["ms_per_step"],
                                      host_cpus=os.cpu_count(), edges_f_per_s=ref["edges_f_per_s"])
    if not getattr(args, "no_other_configs", False):
        others = {}
        cases = (("c2_spmm", "c2_spmm", 64, 128), ("c3_sddmm", "c3_sddmm", 64, 128), ("c4_attention", "c4_attention", 64, 128),
                 ("c2_spmm_f64", "c2_spmm", 64, 64), ("c2_spmm_f256", "c2_spmm", 64, 256), ("c3_sddmm_f64", "c3_sddmm", 64, 64),
                 ("c5_spmm_f256", "c5_spmm", 128, 256))
        for label, workload, tile, features in cases:
            sub = argparse.Namespace(**vars(args))
            sub.workload, sub.tile, sub.features = workload, tile, features
            # the CPU baselines of SDDMM and attention are timed once, on the F = 128 runs
            sub.no_cpu_baseline = args.no_cpu_baseline or not (label in ("c3_sddmm", "c4_attention"))
            sub.steps, sub.warmup = min(args.steps, 10), 3
            sub.warps, sub.hub_threshold = {"c3_sddmm": (8, 8192), "c4_attention": (4, 1024)}.get(workload, (4, 1024))
            torch.cuda.empty_cache()
            try:
                got = bench.run_ours_single(sub)
                others[label] = {"workload": got["config"]["workload"], "ms_per_step": got["ms_per_step"],
                                    "value": got["value"], "unit": got["unit"],
                                    "edges_f_per_s": got["edges_f_per_s"],
                                    "roofline_frac": got["roofline"]["frac"],
                                    "traffic": got["roofline"]["traffic"],
                                    "e2e_value": got["e2e"]["value"],
                                    "e2e_graph_resident_value": got["e2e_graph_resident"]["value"],
                                    "gpu_launches": got["gpu_launches"]}
                if "cpu_baseline" in got:
                    others[label]["cpu_baseline"] = got["cpu_baseline"]
                if "gpu_comparator" in got:
                    others[label]["gpu_comparator_cusparse_ms"] = got["gpu_comparator"]["ms_per_step"]
            except Exception as exc:  # noqa: BLE001 - the headline line must still be printed
                others[label] = {"error": f"{type(exc).__name__}: {exc}"}
        extras["other_configs"] = others
        try:
            extras["c1_cpu_case"] = bench.small_cpu_case()
        except Exception as exc:  # noqa: BLE001
            extras["c1_cpu_case"] = {"error": f"{type(exc).__name__}: {exc}"}
        # the reference's own CUDA kernels, rebuilt for sm_100a, in a process of their own
        from benchlib import reference_kernels

        torch.cuda.empty_cache()
        extras["gpu_comparator_reference"] = {
            label: reference_kernels.run_in_subprocess(workload, 128)
            for label, workload in (("c2_spmm", "c2_spmm"), ("c3_sddmm", "c3_sddmm"), ("c5_spmm", "c5_spmm"))}
        extras["probe_ms_uncached"] = _probe_costs(bench, args, device)
    return extras


def _fused_layer_case(shard, layer, x, f, out_f, device) -> dict:
    """The same layer forward as ONE kernel (aggregation + Linear fused, asg_conv_fused): median of five
    calls and the largest difference from the default two-kernel forward.  Reported beside the headline
    because it is the slower form on this graph, which is why the layer does not take it by default."""
    from autosage_b200 import _native

    if shard.val is not None or not _native.conv_fused_supported(f, out_f):
        return {"unavailable": "the fused kernel takes 64 or 128 input features and up to 256 output features"}
    try:
        weight = layer.linear.weight.detach().contiguous()
        bias = None if layer.linear.bias is None else layer.linear.bias.detach().contiguous()
        expected = layer.forward()     # the default forward of the single-GPU layer (x is already loaded)
        out = torch.empty(x.size(0), out_f, device=device)
        workspace = _native.conv_fused(shard.crow, shard.col, None, x, weight, bias, out)
        times = []
        for _ in range(5):
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            _native.conv_fused(shard.crow, shard.col, None, x, weight, bias, out, workspace=workspace)
            end.record()
            end.synchronize()
            times.append(begin.elapsed_time(end))
        found = {"entry_point": "asg_conv_fused", "hub_threshold": _native.CONV_FUSED_HUB_THRESHOLD,
                 "ms_per_step": round(sorted(times)[2], 4), "status": _native.workspace_status(workspace),
                 "gpu_launches_per_step": 3}
        found["max_abs_difference_from_default"] = float((out - expected).abs().max())
        return found
    except Exception as exc:  # noqa: BLE001 - the headline line must still be printed
        return {"error": f"{type(exc).__name__}: {exc}"}


def _probe_costs(bench, args, device) -> dict:
    """Wall time of one scheduled call with an empty schedule cache (sample + probe + guardrail + the
    full-graph run it ends with) and of the same call replayed from the cache, per configuration."""
    import tempfile

    import autosage_b200

    found = {}
    saved = os.environ.get("AUTOSAGE_CACHE_DIR")
    for name, workload in (("c2", "c2_spmm"), ("c4", "c4_attention"), ("c5", "c5_spmm")):
        torch.cuda.empty_cache()
        try:
            w = bench.build_workload(workload, args.features, device)
            os.environ["AUTOSAGE_CACHE_DIR"] = tempfile.mkdtemp(prefix="autosage-bench-cache-")
            if workload == "c4_attention":
                def call():
                    return autosage_b200.csr_attention_forward(w["crow"], w["col"], w["q"], w["k"], w["v"],
                                                               scale=args.features ** -0.5)[1]["attention"]
            else:
                def call():
                    return autosage_b200.spmm_csr_auto(w["crow"], w["col"], w["val"], w["x"])[1]
            # one plain (unscheduled) call first: the process is then warm - kernels loaded, output-sized
            # blocks in torch's caching allocator - as it is when a model schedules its first layer
            if workload == "c4_attention":
                autosage_b200.csr_attention_forward(w["crow"], w["col"], w["q"], w["k"], w["v"], scale=args.features ** -0.5,
                                                    fused=False)
            else:
                autosage_b200.spmm_csr(w["crow"], w["col"], w["val"], w["x"])
            laps = []
            for _ in range(2):
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                info = call()
                torch.cuda.synchronize()
                laps.append((time.perf_counter() - t0) * 1e3)
                if not laps[1:]:
                    first = info
            found[name] = {"uncached_ms": round(laps[0], 2), "replay_ms": round(laps[1], 3), "choice": first["choice"],
                           "candidate": first["candidate"], "probe_rows": first.get("probe_rows"),
                           "probe_nonzeros": first.get("probe_nonzeros"), "replayed_from_cache": bool(info["from_cache"])}
            del w
        except Exception as exc:  # noqa: BLE001 - the headline line must still be printed
            found[name] = {"error": f"{type(exc).__name__}: {exc}"}
    if saved is None:
        os.environ.pop("AUTOSAGE_CACHE_DIR", None)
    else:
        os.environ["AUTOSAGE_CACHE_DIR"] = saved
    return found


def run(args):
    import bench  # the launcher script: clock sampler and peak lookup live there
    import autosage_b200
    from autosage_b200 import dist as asg_dist
    from benchlib import synthetic as syn

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise RuntimeError(f"--gpus {args.gpus} needs torch.distributed.run with {args.gpus} ranks (got {world})")
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    multi = world > 1
    if multi:
        dist.init_process_group("nccl", device_id=device)

    def barrier():
        if multi:
            dist.barrier()

    def reduce_max(t):
        if multi:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t
    if not autosage_b200.load_native():
        raise RuntimeError(f"libautosage_b200.so failed to load: {autosage_b200.ops.native_load_error()}")

    f, out_f = args.features, 256
    spec = syn.PRODUCTS_LIKE if args.workload.startswith("c5") else syn.REDDIT_LIKE
    crow, col, info = syn.powerlaw_csr(spec, seed=0, device=device)
    n, nnz = info["rows"], info["nnz"]
    bounds = asg_dist.partition_rows(crow, world)
    shard = asg_dist.shard_csr(crow, col, None, rank, world, bounds, groups=args.groups if args.groups else min(world, 4))

    torch.manual_seed(0)
    weight = torch.nn.init.xavier_uniform_(torch.empty(out_f, f, device=device))
    bias = torch.zeros(out_f, device=device)
    gen = torch.Generator(device=device).manual_seed(3)
    x_all = torch.randn(n, f, generator=gen, device=device)  # same stream of numbers on every rank

    def seeded(layer):
        with torch.no_grad():
            layer.linear.weight.copy_(weight)
            layer.linear.bias.copy_(bias)
        return layer

    # The same layer on ONE GPU (no sharding, no exchange), same X and weights, run inside this job so
    # that every multi-GPU line carries its own strong-scaling reference AND a result check: this rank's
    # rows of the single-GPU aggregation and output are kept and compared with the sharded step below.
    # Every rank times it on its own GPU at the same moment; the maximum over ranks is reported.
    single_ms = None
    single_rows = None
    if multi:
        whole = asg_dist.shard_csr(crow, col, None, 0, 1, asg_dist.partition_rows(crow, 1))
        solo = seeded(asg_dist.ShardedAutoSAGEConv(whole, f, out_f, bias=True, feature_tile=args.tile, warps=args.warps,
                                                   threshold=args.hub_threshold).to(device))
        solo.spmm.load_local(x_all)
        with torch.no_grad():
            for _ in range(3):
                solo()
            torch.cuda.synchronize()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps = max(3, min(args.steps, 5))
            t0.record()
            for _ in range(reps):
                solo()
            t1.record()
            torch.cuda.synchronize()
            lo, hi = shard.row_begin, shard.row_end
            single_rows = (solo.spmm.forward()[lo:hi].clone(), solo()[lo:hi].clone(),
                           (crow[lo + 1:hi + 1] - crow[lo:hi]).clamp_min(1).double().sqrt())
        single_ms = float(reduce_max(torch.tensor([t0.elapsed_time(t1) / reps], device=device)).item())
        del solo, whole
    del crow, col
    torch.cuda.empty_cache()

    layer = seeded(asg_dist.ShardedAutoSAGEConv(shard, f, out_f, bias=True, feature_tile=args.tile, warps=args.warps,
                                                threshold=args.hub_threshold, exchange=args.exchange,
                                                copy_streams=args.copy_streams, slabs=args.slabs, chunks=args.chunks,
                                                push_ctas=args.push_ctas).to(device))
    pinning = bind_to_gpu_numa_node(local_rank) if multi else None  # before any pinned buffer is allocated
    x_shard_host = x_all[shard.row_begin:shard.row_end].cpu().pin_memory()
    layer.spmm.load_local(x_all[shard.row_begin:shard.row_end])
    del x_all
    torch.cuda.empty_cache()

    stream = torch.cuda.current_stream()
    spmm_events: list[tuple] = []
    # multi-GPU: the whole step (pulls, barriers, column-block SpMMs, Linear) replayed as one CUDA graph
    replay = layer.capture() if multi and not args.no_graph else None

    def step():
        with torch.no_grad():
            if replay is not None:
                return replay()
            if multi:
                return layer()
            # one GPU: the layer's two stages written out, with events around the aggregation so that
            # the dominant kernel's launch time is measured inside the timed region
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            aggregated = layer.spmm.forward()
            b.record(stream)
            spmm_events.append((a, b))
            return asg_dist.apply_linear(layer.linear, aggregated)

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    spmm_events.clear()
    barrier()
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = bench.ClockSampler(local_rank)  # NVML set up and queried once before anything is timed
    torch.cuda.synchronize()
    barrier()
    torch.cuda.synchronize()
    step_marks = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    with sampler as clocks:
        host_begin = time.perf_counter()
        begin.record(stream)
        step_marks[0].record(stream)
        for i in range(args.steps):
            step()
            step_marks[i + 1].record(stream)
        end.record(stream)
        host_enqueue_ms = (time.perf_counter() - host_begin) * 1e3 / args.steps
        torch.cuda.synchronize()
        barrier()
        torch.cuda.synchronize()
    elapsed = reduce_max(torch.tensor([begin.elapsed_time(end)], device=device))
    ms_per_step = float(elapsed.item()) / args.steps
    # per step: the slowest rank's time; then median / min / max over the steps
    per_step = reduce_max(torch.tensor([step_marks[i].elapsed_time(step_marks[i + 1]) for i in range(args.steps)],
                                       device=device)).cpu().tolist()
    ms_median = statistics.median(per_step)
    spmm_launch_ms = [a.elapsed_time(b) for a, b in spmm_events]
    spmm_events.clear()

    # where the step goes (separate, untimed-for-the-metric runs): exchange alone, the column-block
    # SpMMs alone (no exchange), the Linear alone; maxima over ranks
    def timed(fn, reps=5):
        fn()
        torch.cuda.synchronize()
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(reps):
            fn()
        b.record(stream)
        torch.cuda.synchronize()
        barrier()
        return float(reduce_max(torch.tensor([a.elapsed_time(b) / reps], device=device)).item())

    def exchange_only():
        layer.spmm.exchange_only()

    def compute_only():
        if layer.spmm.slabs:
            layer.spmm._slab_products(aggregated_scratch, None)
            return
        kw = dict(feature_tile=args.tile, warps=args.warps, threshold=args.hub_threshold)
        blocks = layer.spmm._chunk_blocks if layer.spmm.layout is not None else shard.blocks
        for g, block in enumerate(blocks):
            asg_dist._block_spmm(block, layer.spmm.x_full, aggregated_scratch, g > 0, **kw)

    # timeline of a few more (untimed) steps: mean offsets of the exchange and compute marks from the
    # step's start on this rank, events recorded in the streams the work runs on
    timeline = None
    if multi:
        layer.spmm.trace = []
        with torch.no_grad():
            for _ in range(6):
                layer()  # eager on purpose: the marks are events recorded between the launches
        layer.spmm.trace = layer.spmm.trace[1:]  # the first traced step starts with the ranks out of step
        own = layer.spmm.timeline_ms()
        layer.spmm.trace = None
        names = sorted(own)
        mine = torch.tensor([own[name] for name in names], device=device)
        everyone = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(everyone, mine)
        stacked = torch.stack(everyone).cpu()
        order = sorted(range(len(names)), key=lambda i: float(stacked[:, i].max()))
        timeline = {names[i]: [round(float(stacked[:, i].min()), 3), round(float(stacked[:, i].max()), 3)] for i in order}

    # result check: this rank's rows of the sharded step against the single-GPU layer of the same job
    parity = None
    if multi and single_rows is not None:
        with torch.no_grad():
            ratios = compare_with_single_gpu(single_rows, layer.spmm.forward(), step(), weight)
        worst = reduce_max(torch.tensor(list(ratios), device=device)).cpu().tolist()
        parity = {"aggregated_rows_worst_error_over_bound": round(worst[0], 4),
                  "layer_output_worst_error_over_bound": round(worst[1], 4),
                  "rule": "|sharded - single| <= 2*(1e-5*|single| + 1e-5*sqrt(row degree)), carried through |W| for the output"}
        single_rows = None
        torch.cuda.empty_cache()

    aggregated_scratch = torch.empty(shard.n_local, f, device=device)
    with torch.no_grad():
        breakdown = {
            "exchange_ms": round(timed(exchange_only), 4),
            "block_spmm_ms": round(timed(compute_only), 4),
            "linear_ms": round(timed(lambda: asg_dist.apply_linear(layer.linear, aggregated_scratch)), 4),
        }
    del aggregated_scratch

    # end to end: X shard from pinned host memory in, output shard back to the host, every step.
    # Serial form: copy in, layer, copy out, one after the other on one stream.  Streamed form (the
    # one reported as e2e): the copy-out of step i runs on a second stream into one of two host buffers
    # while step i+1 copies in and computes - PCIe is full duplex - and the timed region ends when the
    # last output has reached the host.
    out_hosts = [torch.empty(shard.n_local, out_f).pin_memory() for _ in range(2)]
    out_host = out_hosts[0]
    drain = torch.cuda.Stream(device=device)

    def e2e_serial_step():
        layer.spmm.load_local(x_shard_host, non_blocking=True)
        out_host.copy_(step(), non_blocking=True)

    # a replayed graph writes the same output buffer every step: stage it in one of two device
    # buffers so that the copy-out of step i can still run under step i+1
    staged = [torch.empty(shard.n_local, out_f, device=device) for _ in range(2)] if replay is not None else None
    drained: list = [None, None]

    def e2e_streamed_step(i):
        layer.spmm.load_local(x_shard_host, non_blocking=True)
        out = step()
        if staged is not None:
            if drained[i % 2] is not None:
                stream.wait_event(drained[i % 2])
            staged[i % 2].copy_(out)
            out = staged[i % 2]
        drain.wait_stream(stream)
        with torch.cuda.stream(drain):
            out_hosts[i % 2].copy_(out, non_blocking=True)
            drained[i % 2] = torch.cuda.Event()
            drained[i % 2].record(drain)
        out.record_stream(drain)

    # enough steps for the streamed form to show its steady state: the first step's copy-in and compute are
    # not hidden behind a copy-out, and with five steps that start-up is a seventh of the figure
    e2e_steps = max(2, min(args.steps, 20))

    def time_e2e(run_steps):
        run_steps(1)
        stream.wait_stream(drain)
        torch.cuda.synchronize()
        barrier()
        begin.record(stream)
        run_steps(e2e_steps)
        stream.wait_stream(drain)
        end.record(stream)
        torch.cuda.synchronize()
        barrier()
        took = reduce_max(torch.tensor([begin.elapsed_time(end)], device=device))
        return float(took.item()) / e2e_steps

    e2e_serial_ms = time_e2e(lambda k: [e2e_serial_step() for _ in range(k)])
    e2e_ms = time_e2e(lambda k: [e2e_streamed_step(i) for i in range(k)])
    # the two PCIe directions alone, all ranks copying at once: per-rank GB/s, slowest and fastest rank
    def copy_rate(fn, nbytes):
        fn()
        torch.cuda.synchronize()
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(3):
            fn()
        b.record(stream)
        torch.cuda.synchronize()
        barrier()
        rate = torch.tensor([nbytes * 3 / (a.elapsed_time(b) * 1e-3) / 1e9], device=device)
        if not multi:
            return [round(float(rate.item()), 2)] * 2
        rates = [torch.zeros_like(rate) for _ in range(world)]
        dist.all_gather(rates, rate)
        flat = [float(r.item()) for r in rates]
        return [round(min(flat), 2), round(max(flat), 2)]

    last_out = step()
    pcie = {
        "h2d_GBps_per_rank_min_max": copy_rate(lambda: layer.spmm.load_local(x_shard_host, non_blocking=True),
                                               x_shard_host.numel() * 4),
        "d2h_GBps_per_rank_min_max": copy_rate(lambda: out_host.copy_(last_out, non_blocking=True), out_host.numel() * 4),
        "numa": pinning,
    }
    io_bytes = torch.tensor([x_shard_host.numel() * 4, out_host.numel() * 4], device=device, dtype=torch.long)
    local_nnz = torch.tensor([shard.col.numel()], device=device, dtype=torch.long)
    gathered = [torch.zeros_like(local_nnz) for _ in range(world)]
    if multi:
        dist.all_reduce(io_bytes)
        dist.all_gather(gathered, local_nnz)
    else:
        gathered = [local_nnz]

    n_blocks = len(layer.spmm._chunk_blocks) if layer.spmm.layout is not None else len(shard.blocks)
    algorithmic = conv_bytes(n, nnz, f, out_f)
    value = algorithmic / (ms_per_step * 1e-3) / 1e9
    peak, peak_kind = bench.measured_peak()
    if multi:
        roofline = {
            "bound": "hbm",
            "kernel": "whole step (SpMM kernels + Linear + exposed exchange), per-GPU share",
            "achieved": round(value / world, 2),
            "peak": peak,
            "peak_source": f"{peak_kind} HBM copy bandwidth (burst)",
            "unit": "GB/s",
            "frac": round(value / world / peak, 4),
            "traffic": None,
        }
    else:
        spmm_algorithmic = bench.spmm_bytes(n, nnz, f, False)
        launch_ms = statistics.fmean(spmm_launch_ms)
        achieved = spmm_algorithmic / (launch_ms * 1e-3) / 1e9
        traffic, traffic_source = bench.ncu_dram_traffic("c5_spmm", f, args.tile)
        roofline = {
            "bound": "hbm",
            "kernel": "spmm_kernel_deep + spmm_short_kernel (the aggregation; %.0f %% of the step)"
                      % (100.0 * launch_ms / ms_per_step),
            "achieved": round(achieved, 2),
            "peak": peak,
            "peak_source": f"{peak_kind} HBM copy bandwidth (burst)",
            "unit": "GB/s",
            "frac": round(achieved / peak, 4),
            "traffic": traffic,
            "traffic_source": traffic_source,
            "algorithmic_bytes_per_launch": spmm_algorithmic,
            "launch_ms": round(launch_ms, 4),
            "launch_ms_median_min_max": [round(statistics.median(spmm_launch_ms), 4), round(min(spmm_launch_ms), 4),
                                         round(max(spmm_launch_ms), 4)],
            "note": "X (1.25 GB) is ten times the 126 MB L2, so the byte model (CSR + gathered X rows + output) "
                    "is also the DRAM traffic to first order; hub-row reuse in L2 lets achieved pass the copy peak",
        }
    line = None
    if rank == 0:
        line = {
            "metric": "algorithmic_GBps",
            "value": round(value, 2),
            "unit": "GB/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": max(args.warmup, 3),
            "ms_per_step": round(ms_per_step, 4),
            "ms_per_step_median_min_max": [round(ms_median, 4), round(min(per_step), 4), round(max(per_step), 4)],
            "value_at_median": round(algorithmic / (ms_median * 1e-3) / 1e9, 2),
            "higher_is_better": True,
            "scaling": "strong",
            "vs_baseline": None,
            "dtype": "f32",
            "data": "synthetic",
            "config": {
                "workload": bench.conv_workload_label(n, nnz, f, out_f),
                "parallelism": f"rows sharded by nnz over {world} GPUs; X gathered over NVLink "
                               f"({EXCHANGE_NAMES.get(layer.spmm.exchange, layer.spmm.exchange)}), "
                               f"overlapped with {n_blocks} column-block SpMMs per GPU",
                "exchange": layer.spmm.exchange,
                "cuda_graph": replay is not None,  # N = 1 launches eagerly (host_enqueue_ms_per_step says what that costs)
                "feature_slabs": layer.spmm.slabs,
                "kernel_parameters": {"feature_tile": args.tile, "warps_per_block": args.warps,
                                      "hub_threshold": args.hub_threshold},
                "l2": "per-GPU inputs per step (CSR shard + gathered X) exceed the 126 MB L2; no explicit flush",
                "nnz_per_rank": [int(t.item()) for t in gathered],
            },
            "edges_f_per_s": round(nnz * f / (ms_per_step * 1e-3), 1),
            "algorithmic_bytes_per_step": algorithmic,
            "nvlink_receive_bytes_per_gpu": 4 * (n - shard.n_local) * f,
            "breakdown_ms": breakdown,
            "host_enqueue_ms_per_step": round(host_enqueue_ms, 4),
            # [earliest rank, latest rank] offset of each mark from its rank's step start
            "timeline_ms_min_max_over_ranks": timeline,
            "parity_vs_single_gpu": None if parity is None else (
                "ok" if max(parity["aggregated_rows_worst_error_over_bound"],
                            parity["layer_output_worst_error_over_bound"]) <= 1.0 else "FAILED"),
            "parity_detail": parity,
            "single_gpu_ms_per_step": None if single_ms is None else round(single_ms, 4),
            "speedup_vs_1gpu_same_workload": None if single_ms is None else round(single_ms / ms_per_step, 3),
            "roofline": roofline,
            "e2e": {
                "value": round(algorithmic / (e2e_ms * 1e-3) / 1e9, 2),
                "unit": "GB/s",
                "ms_per_step": round(e2e_ms, 3),
                "h2d_bytes_per_step": int(io_bytes[0].item()),
                "d2h_bytes_per_step": int(io_bytes[1].item()),
                "steps": e2e_steps,
                "inputs": "the CSR stays on the device (the layer's graph, as a model keeps its weights); this rank's X shard "
                          "comes in from pinned host memory and its output shard goes back, every step",
                "mode": "streamed: the copy-out of step i overlaps the copy-in and compute of step i+1 "
                        "(second stream, two pinned output buffers); every step's input and output cross PCIe "
                        "inside the timed region",
            },
            "e2e_pcie": pcie,
            "e2e_serial": {
                "value": round(algorithmic / (e2e_serial_ms * 1e-3) / 1e9, 2),
                "unit": "GB/s",
                "ms_per_step": round(e2e_serial_ms, 3),
                "mode": "copy in, layer, copy out, strictly one after the other on one stream",
            },
            # per step and GPU: two SpMM kernels (main + short-row queue) for every column block (or
            # feature band), and the Linear kernel
            "gpu_launches": args.steps * world * ((layer.spmm.slabs or n_blocks) * 2 + 1 + 1),  # + the weight split
            "clocks": clocks.summary(),
        }
        if not multi:
            line["scaling_note"] = "the same fixed workload runs at every N (strong scaling); N = 1 is this line"
            line.update(_single_gpu_extras(args, bench, shard, layer, algorithmic, n, nnz, f, out_f, device))
    if multi:
        dist.barrier()
        dist.destroy_process_group()
    return line
