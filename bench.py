"""Benchmark of the sparse hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload c2_spmm|c3_sddmm|c4_attention|c5_spmm|c5_conv] [--features F]

One "step" is one pass of the hot path (one SpMM / SDDMM / attention call) over the whole synthetic
graph.  Metric: algorithmic GB/s (bytes = CSR + gathered dense rows + output, the byte model of the
roofline) with edges*F/s alongside.  The default workload at every N is the AutoSAGEConv forward of
the ogbn-products-sized power-law graph (2,449,029 rows, ~123.7 M nnz, F = 128, Linear F->256), the configuration the
1/2/4/8-GPU series is quoted on: at N = 1 the whole graph on one GPU, at N > 1 rows sharded by nnz over
the ranks with X gathered over NVLink inside the timed region (peer-memory pulls, or NCCL send/recv
with --exchange nccl); strong scaling, and each multi-GPU line also carries the same layer timed on
one GPU in the same job (single_gpu_ms_per_step).  The N = 1 line adds short runs of configurations 2
(SpMM, 232,965 rows, ~114.6 M nnz, weighted), 3 (SDDMM) and 4 (fused attention) under other_configs;
--workload selects any of them as the headline instead.

The line printed by rank 0 carries, beside the contract keys:
  roofline      achieved algorithmic GB/s of the dominant kernel against the measured HBM copy peak
  cpu_baseline  the reference's CPU path (torch.sparse.mm over a CSR tensor, restated in oracle/)
                timed on this host on a bounded row sample of the same workload
  e2e           the same metric through the public API with HOST buffers (pinned), H2D and D2H
                copies inside the timed region
  clocks        SM clock and throttle reasons sampled during the timed region
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

FALLBACK_HBM_GBS = 6650.0

def ncu_dram_traffic(workload: str, f: int, tile: int) -> tuple:
    """(bytes, source) of dram__bytes_read.sum + dram__bytes_write.sum for one launch of the workload's
    dominant kernel, from profiles/dram_traffic.json (written from the ncu captures summarised beside
    it); (None, None) for a workload without a capture of the byte counters."""
    try:
        table = json.loads((ROOT / "profiles" / "dram_traffic.json").read_text())
        entry = table[f"{workload}/f{f}/tile{tile}"]
        return float(entry["dram_bytes_per_launch"]), entry["source"]
    except (OSError, ValueError, KeyError):
        return None, None


# ------------------------------------------------------------------------------------------------
def measured_peak() -> tuple[float, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    try:
        value = float(json.loads(path.read_text())["hbm_gbs"])
        return value, "measured"
    except (OSError, ValueError, KeyError):
        return FALLBACK_HBM_GBS, "fallback"


def spmm_bytes(n_rows: int, nnz: int, f: int, weighted: bool) -> int:
    """CSR + gathered X + output: 8(N+1) + 8 nnz [+ 4 nnz] + 4 nnz F + 4 N F."""
    return 8 * (n_rows + 1) + 8 * nnz + (4 * nnz if weighted else 0) + 4 * nnz * f + 4 * n_rows * f


def sddmm_bytes(n_rows: int, nnz: int, f: int) -> int:
    return 8 * (n_rows + 1) + 8 * nnz + 4 * n_rows * f + 4 * nnz * f + 4 * nnz


def attention_bytes(n_rows: int, nnz: int, f: int) -> int:
    return 8 * (n_rows + 1) + 8 * nnz + 4 * n_rows * f + 2 * 4 * nnz * f + 4 * n_rows * f


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index: int) -> None:
        self.samples: list[int] = []
        self.reasons: set[str] = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._handle = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM))
            # the first query of each kind is the slow one (milliseconds): make it here, outside any
            # timed region, so that the samples taken during a run cost microseconds
            pynvml.nvmlDeviceGetClockInfo(self._handle, pynvml.NVML_CLOCK_SM)
            getter = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or getattr(
                pynvml, "nvmlDeviceGetCurrentClocksThrottleReasons")
            getter(self._handle)
        except Exception:  # NVML missing: report nulls
            self._handle = None

    def _loop(self) -> None:
        nv = self._nvml
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self._handle, nv.NVML_CLOCK_SM)))
                getter = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or getattr(
                    nv, "nvmlDeviceGetCurrentClocksThrottleReasons")
                mask = int(getter(self._handle))
                for name, bit in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.05)

    def __enter__(self):
        if self._handle is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self) -> dict:
        return {
            "sm_mhz": statistics.median(self.samples) if self.samples else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
        }


# ------------------------------------------------------------------------------------------------
# CPU baseline (the reference's CPU path, restated in oracle/) on a bounded row sample
# ------------------------------------------------------------------------------------------------
def cpu_spmm_sample(crow_cpu, col_cpu, val_cpu, x_cpu, target_nnz: int, repeats: int):
    """Times torch.sparse.mm over the first rows holding ~target_nnz edges (all columns kept, so
    the gather pattern over X is the full workload's).  Returns (seconds per call, rows, nnz)."""
    from oracle import oracle

    rows = int(torch.searchsorted(crow_cpu, torch.tensor(target_nnz)).clamp(1, crow_cpu.numel() - 1))
    sub_crow = crow_cpu[: rows + 1].contiguous()
    nnz = int(sub_crow[-1])
    sub_col = col_cpu[:nnz].contiguous()
    sub_val = None if val_cpu is None else val_cpu[:nnz].contiguous()
    times = []
    for _ in range(repeats + 1):
        t0 = time.perf_counter()
        oracle.spmm_reference_cpu(sub_crow, sub_col, sub_val, x_cpu)
        times.append(time.perf_counter() - t0)
    return min(times[1:]) if len(times) > 1 else times[0], rows, nnz


# ------------------------------------------------------------------------------------------------
def build_workload(name: str, f: int, device):
    from benchlib import synthetic as syn

    spec = {"c2_spmm": syn.REDDIT_LIKE, "c3_sddmm": syn.REDDIT_LIKE, "c4_attention": syn.ARXIV_LIKE,
            "c5_spmm": syn.PRODUCTS_LIKE}[name]
    crow, col, info = syn.powerlaw_csr(spec, seed=0, device=device)
    n = info["rows"]
    w = {"name": name, "spec": spec, "info": info, "crow": crow, "col": col, "f": f, "n": n}
    if name == "c2_spmm":
        w["val"] = syn.edge_values(info["nnz"], seed=0, device=device)
        w["x"] = syn.dense(n, f, 3, device)
    elif name == "c5_spmm":
        w["val"] = None
        w["x"] = syn.dense(n, f, 3, device)
    elif name == "c3_sddmm":
        w["q"], w["k"] = syn.dense(n, f, 1, device), syn.dense(n, f, 2, device)
    else:
        w["q"], w["k"], w["v"] = syn.dense(n, f, 1, device), syn.dense(n, f, 2, device), syn.dense(n, f, 3, device)
    return w


def run_ours_single(args) -> dict:
    import autosage_b200
    from autosage_b200 import _native

    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device")
    if not autosage_b200.load_native():
        raise RuntimeError(f"libautosage_b200.so failed to load: {autosage_b200.ops.native_load_error()}")
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    w = build_workload(args.workload, args.features, device)
    n, nnz, f = w["n"], w["info"]["nnz"], w["f"]
    crow, col = w["crow"], w["col"]
    tile, warps, threshold = args.tile, args.warps, args.hub_threshold
    stream = torch.cuda.current_stream()

    if args.workload in ("c2_spmm", "c5_spmm"):
        val, x = w["val"], w["x"]
        y = torch.empty(n, f, device=device)
        ws, _ = _native.planned_workspace(crow, threshold)
        _native.plan_build(crow, threshold, ws)

        def step():
            _native.spmm(crow, col, val, x, y, feature_tile=tile, warps=warps, threshold=threshold,
                         flags=_native.FLAG_PLAN_READY, workspace=ws)

        algorithmic = spmm_bytes(n, nnz, f, val is not None)
        kernel_name = "spmm_kernel"
        host_inputs = [crow, col, x] + ([val] if val is not None else [])

        def e2e_step(dev_inputs):
            c, cc, xx = dev_inputs[0], dev_inputs[1], dev_inputs[2]
            vv = dev_inputs[3] if len(dev_inputs) > 3 else None
            return torch.ops.autosage.spmm_csr_split(c, cc, vv, xx, tile if tile in (64, 128) else 128,
                                                     warps if warps in (2, 4, 8) else 8, threshold)
    elif args.workload == "c3_sddmm":
        q, k = w["q"], w["k"]
        out = torch.empty(nnz, device=device)
        ws, _ = _native.planned_workspace(crow, threshold)
        _native.plan_build(crow, threshold, ws)

        def step():
            _native.sddmm(crow, col, q, k, out, warps=warps, threshold=threshold, flags=_native.FLAG_PLAN_READY,
                          workspace=ws)

        algorithmic = sddmm_bytes(n, nnz, f)
        kernel_name = "sddmm_kernel"
        host_inputs = [crow, col, q, k]

        def e2e_step(dev_inputs):
            return torch.ops.autosage.sddmm_csr_split(*dev_inputs, warps if warps in (2, 4, 8) else 8, threshold)
    else:
        q, k, v = w["q"], w["k"], w["v"]
        out = torch.empty(n, f, device=device)
        ws, _ = _native.planned_workspace(crow, threshold, _native.attention_extra_bytes(n))
        _native.plan_build(crow, threshold, ws)
        scale = f ** -0.5

        def step():
            _native.attention(crow, col, q, k, v, out, scale=scale, warps=warps, threshold=threshold,
                              flags=_native.FLAG_PLAN_READY, workspace=ws)

        algorithmic = attention_bytes(n, nnz, f)
        kernel_name = "attention_kernel"
        host_inputs = [crow, col, q, k, v]

        def e2e_step(dev_inputs):
            c, cc, qq, kk, vv = dev_inputs
            o = torch.empty_like(vv)
            w2, ready = _native.planned_workspace(c, threshold, _native.attention_extra_bytes(c.numel() - 1))
            _native.attention(c, cc, qq, kk, vv, o, scale=scale, warps=warps, threshold=threshold, flags=ready,
                              workspace=w2)
            return o

    # ---- device-resident timing -------------------------------------------------------------
    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    stops = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    with ClockSampler(0) as clocks:
        torch.cuda.synchronize()
        t_begin = torch.cuda.Event(enable_timing=True)
        t_end = torch.cuda.Event(enable_timing=True)
        t_begin.record(stream)
        for i in range(args.steps):
            starts[i].record(stream)
            step()
            stops[i].record(stream)
        t_end.record(stream)
        torch.cuda.synchronize()
    total_ms = t_begin.elapsed_time(t_end)
    per_launch = [s.elapsed_time(e) for s, e in zip(starts, stops)]
    ms_per_step = total_ms / args.steps
    status = _native.workspace_status(ws)
    if status != 0:
        raise RuntimeError(f"a kernel reported status {status}; the timing is invalid")
    value = algorithmic / (ms_per_step * 1e-3) / 1e9
    launch_ms = statistics.fmean(per_launch)
    peak, peak_kind = measured_peak()
    achieved = algorithmic / (launch_ms * 1e-3) / 1e9

    # ---- end to end through the public operators, host buffers ----------------------------------
    pinned = [t.cpu().pin_memory() for t in host_inputs]
    h2d_bytes = sum(t.numel() * t.element_size() for t in pinned)
    result_host = None
    e2e_steps = max(2, min(args.steps, 5))

    def e2e_once():
        nonlocal result_host
        dev_inputs = [t.to(device, non_blocking=True) for t in pinned]
        res = e2e_step(dev_inputs)
        if result_host is None:
            result_host = torch.empty(res.shape, dtype=res.dtype).pin_memory()
        result_host.copy_(res, non_blocking=True)

    del host_inputs
    e2e_once()
    torch.cuda.synchronize()
    e_begin, e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e_begin.record(stream)
    for _ in range(e2e_steps):
        e2e_once()
    e_end.record(stream)
    torch.cuda.synchronize()
    e2e_ms = e_begin.elapsed_time(e_end) / e2e_steps
    d2h_bytes = result_host.numel() * result_host.element_size()

    # The same call with the graph kept on the device (as a model keeps its weights) and only the dense
    # operands copied in every step - how a GNN layer is fed.  Reported beside e2e, not instead of it.
    graph_dev = [t.to(device) for t in pinned[:2]]
    dense_pinned = pinned[2:]

    def e2e_dense_only():
        dev_inputs = graph_dev + [t.to(device, non_blocking=True) for t in dense_pinned]
        result_host.copy_(e2e_step(dev_inputs), non_blocking=True)

    e2e_dense_only()
    torch.cuda.synchronize()
    e_begin.record(stream)
    for _ in range(e2e_steps):
        e2e_dense_only()
    e_end.record(stream)
    torch.cuda.synchronize()
    e2e_dense_ms = e_begin.elapsed_time(e_end) / e2e_steps
    dense_bytes = sum(t.numel() * t.element_size() for t in dense_pinned)

    line = {
        "metric": "algorithmic_GBps",
        "value": round(value, 2),
        "unit": "GB/s",
        "n_gpus": 1,
        "steps": args.steps,
        "warmup": max(args.warmup, 3),
        "ms_per_step": round(ms_per_step, 4),
        "higher_is_better": True,
        "scaling": "strong",
        "vs_baseline": None,
        "dtype": "f32",
        "data": "synthetic",
        "config": {
            "workload": f"{args.workload}: power-law CSR {n} rows, {nnz} nnz, F={f}"
                        + (", weighted" if args.workload == "c2_spmm" else ""),
            "kernel_parameters": {"feature_tile": tile, "warps_per_block": warps, "hub_threshold": threshold},
            "l2": "inputs per step (CSR + dense operand, %.2f GB) exceed the 126 MB L2; no explicit flush"
                  % ((8 * nnz + 4 * nnz + 4 * n * f) / 1e9),
            "plan": "degree-binned plan cached (replay path)",
        },
        "edges_f_per_s": round(nnz * f / (ms_per_step * 1e-3), 1),
        "algorithmic_bytes_per_step": algorithmic,
        "pct_of_8TBps": round(100.0 * value / 8000.0, 2),
        "roofline": {
            "bound": "hbm",
            "kernel": kernel_name,
            "achieved": round(achieved, 2),
            "peak": peak,
            "peak_source": f"{peak_kind} HBM copy bandwidth (burst)",
            "unit": "GB/s",
            "frac": round(achieved / peak, 4),
            "traffic": ncu_dram_traffic(args.workload, f, tile)[0],
            "traffic_source": ncu_dram_traffic(args.workload, f, tile)[1],
            "note": "achieved counts every gathered dense row (CSR + gathered rows + output); when the dense operand "
                    "fits the 126 MB L2 the gather is served by L2 and achieved exceeds the HBM peak",
            "launch_ms": round(launch_ms, 4),
            "launch_ms_median_min_max": [round(statistics.median(per_launch), 4), round(min(per_launch), 4),
                                         round(max(per_launch), 4)],
        },
        "e2e": {
            "value": round(algorithmic / (e2e_ms * 1e-3) / 1e9, 2),
            "unit": "GB/s",
            "ms_per_step": round(e2e_ms, 3),
            "h2d_bytes_per_step": h2d_bytes,
            "d2h_bytes_per_step": d2h_bytes,
            "steps": e2e_steps,
            "inputs": "CSR arrays and dense operands copied from pinned host memory every step",
        },
        "e2e_graph_resident": {
            "value": round(algorithmic / (e2e_dense_ms * 1e-3) / 1e9, 2),
            "unit": "GB/s",
            "ms_per_step": round(e2e_dense_ms, 3),
            "h2d_bytes_per_step": dense_bytes,
            "d2h_bytes_per_step": d2h_bytes,
            "inputs": "CSR arrays resident on the device; dense operands (and edge weights) copied every step",
        },
        # every operator launches two kernels per step: the main queues and the short-row queue
        # (SDDMM with a key matrix above 64 MB: one main launch per 64-feature pass)
        "gpu_launches": args.steps * (2 + (f // 64 - 1 if args.workload == "c3_sddmm" and f >= 128 and n * f * 4 > (64 << 20) else 0)),
        "clocks": clocks.summary(),
    }

    if args.workload in ("c2_spmm", "c5_spmm"):
        # the reference's own GPU baseline on this box: cuSPARSE through torch.sparse.mm (library call)
        weights = w["val"] if w.get("val") is not None else torch.ones(nnz, device=device)
        matrix = torch.sparse_csr_tensor(crow, col, weights, size=(n, n))
        torch.sparse.mm(matrix, w["x"])
        torch.cuda.synchronize()
        c_begin, c_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c_begin.record(stream)
        for _ in range(3):
            torch.sparse.mm(matrix, w["x"])
        c_end.record(stream)
        torch.cuda.synchronize()
        cusparse_ms = c_begin.elapsed_time(c_end) / 3
        line["gpu_comparator"] = {"name": "torch.sparse.mm (cuSPARSE), the reference scheduler's baseline",
                                  "ms_per_step": round(cusparse_ms, 4),
                                  "value": round(algorithmic / (cusparse_ms * 1e-3) / 1e9, 2), "unit": "GB/s"}
        del matrix, weights

    if not args.no_cpu_baseline and args.workload in ("c3_sddmm", "c4_attention"):
        # The reference's CPU path for these operators (gather-dot SDDMM; SDDMM -> row softmax ->
        # torch.sparse.mm for attention) on the first rows holding ~1 M edges: the gather-dot
        # materialises two [edges, F] operands, so the sample is kept small.
        from oracle import oracle

        torch.set_num_threads(max(1, os.cpu_count() or 1))
        crow_c = crow.cpu()
        target = min(1_000_000, nnz)
        rows = int(torch.searchsorted(crow_c, torch.tensor(target)).clamp(1, n))
        sub_crow = crow_c[: rows + 1].contiguous()
        sample_nnz = int(sub_crow[-1])
        sub_col = col[:sample_nnz].cpu()
        q_c, k_c = w["q"][:rows].cpu(), w["k"].cpu()
        if args.workload == "c3_sddmm":
            run_cpu = lambda: oracle.sddmm_reference_cpu(sub_crow, sub_col, q_c, k_c)  # noqa: E731
            sample_bytes, what = sddmm_bytes(rows, sample_nnz, f), "gather-dot SDDMM on CPU float32"
        else:
            v_c = w["v"].cpu()
            run_cpu = lambda: oracle.attention_reference_cpu(sub_crow, sub_col, q_c, k_c, v_c, f ** -0.5)  # noqa: E731
            sample_bytes, what = attention_bytes(rows, sample_nnz, f), "SDDMM -> row softmax -> torch.sparse.mm on CPU float32"
        laps = []
        for _ in range(3):
            t0 = time.perf_counter()
            run_cpu()
            laps.append(time.perf_counter() - t0)
        seconds = min(laps[1:])
        line["cpu_baseline"] = {
            "value": round(sample_bytes / seconds / 1e9, 3), "unit": "GB/s", "cores": torch.get_num_threads(),
            "host_cpus": os.cpu_count(), "kind": "port",
            "sample": f"first {rows} rows ({sample_nnz} nnz) of the same CSR against the full K"
                      + (" and V" if args.workload == "c4_attention" else "") + f"; {what} (the reference's CPU path), "
                      f"best of 2 after 1 warm-up, {seconds:.3f} s per call",
            "edges_f_per_s": round(sample_nnz * f / seconds, 1),
        }

    if not args.no_cpu_baseline and args.workload in ("c2_spmm", "c5_spmm"):
        from oracle import oracle

        crow_c, col_c = crow.cpu(), col.cpu()
        val_c = None if w.get("val") is None else w["val"].cpu()
        x_c = w["x"].cpu()
        seconds, rows, sample_nnz = cpu_spmm_sample(crow_c, col_c, val_c, x_c, args.cpu_sample_nnz, 2)
        sample_bytes = spmm_bytes(rows, sample_nnz, f, val_c is not None)
        line["cpu_baseline"] = {
            "value": round(sample_bytes / seconds / 1e9, 3),
            "unit": "GB/s",
            "cores": torch.get_num_threads(),
            "host_cpus": os.cpu_count(),
            "kind": "port",
            "sample": f"first {rows} rows ({sample_nnz} nnz) of the same CSR against the full X, "
                      f"torch.sparse.mm on CPU float32 (the reference's CPU path), best of 2 after 1 warm-up, "
                      f"{seconds:.3f} s per call",
            "edges_f_per_s": round(sample_nnz * f / seconds, 1),
            "oracle_threads": oracle.threads(),
        }
    return line


def small_cpu_case() -> dict:
    """The reference's CPU-runnable configuration: unweighted spmm_csr on a 4096-row CSR (degree uniform in
    [1, 32], distinct columns), X 4096 x 64, through the package's CPU path (torch.sparse.mm over a CSR
    tensor, rebuilt per call as in autosage/ops.py:124-143): 3 warm-ups, 20 timed calls, min and median;
    and the same call on the GPU, which at this size is launch-bound."""
    import autosage_b200
    from benchlib import synthetic as syn

    crow, col = syn.uniform_degree_csr(4096, 32, seed=0)
    x = syn.dense(4096, 64, 3)
    threads_before = torch.get_num_threads()
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    laps = []
    for i in range(23):
        t0 = time.perf_counter()
        y_cpu = autosage_b200.spmm_csr(crow, col, None, x)
        if i >= 3:
            laps.append((time.perf_counter() - t0) * 1e3)
    found = {"workload": f"c1: spmm_csr unweighted, 4096 rows, {col.numel()} nnz, F=64, CPU tensors",
             "cpu_ms_min": round(min(laps), 4), "cpu_ms_median": round(statistics.median(laps), 4),
             "cores": torch.get_num_threads(), "calls": 20}
    torch.set_num_threads(threads_before)
    if torch.cuda.is_available():
        dev = torch.device("cuda", 0)
        crow_d, col_d, x_d = crow.to(dev), col.to(dev), x.to(dev)
        for _ in range(3):
            y_gpu = autosage_b200.spmm_csr(crow_d, col_d, None, x_d)
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for _ in range(20):
            y_gpu = autosage_b200.spmm_csr(crow_d, col_d, None, x_d)
        end.record()
        torch.cuda.synchronize()
        found["gpu_ms_per_call"] = round(begin.elapsed_time(end) / 20, 4)
        found["gpu_matches_cpu"] = bool(torch.allclose(y_gpu.cpu(), y_cpu, rtol=1e-4, atol=1e-4))
    return found


def conv_workload_label(n: int, nnz: int, f: int, out_f: int = 256) -> str:
    """config.workload of the default benchmark; both arms print the same string."""
    return (f"c5_conv: row-partitioned AutoSAGEConv forward, power-law CSR {n} rows, {nnz} nnz, "
            f"F={f}, Linear {f}->{out_f}, unweighted")


def reference_graph(args):
    """The benchmark graph on the host.  With a GPU present it is generated there and copied back, which
    gives exactly the arrays the GPU arm multiplies (same device generator, same seed); without one the
    CPU generator draws the columns (same degrees, same distribution)."""
    from benchlib import synthetic as syn

    spec = syn.REDDIT_LIKE if not args.workload.startswith("c5") else syn.PRODUCTS_LIKE
    if args.cpu_sample_nnz > 0:
        # only the sampled rows are materialised: same degree sequence, columns iid uniform over all N
        # columns and sorted inside each row
        degree, _ = syn.powerlaw_degrees(spec.rows, spec.target_nnz, spec.alpha, spec.max_degree, 0)
        crow = torch.zeros(spec.rows + 1, dtype=torch.long)
        torch.cumsum(degree, 0, out=crow[1:])
        rows = int(torch.searchsorted(crow, torch.tensor(args.cpu_sample_nnz)).clamp(1, spec.rows))
        sub_crow, sub_col = syn.csr_from_degrees(degree[:rows], spec.rows, seed=0)
        return spec, sub_crow, sub_col, int(degree.sum()), rows
    device = torch.device("cuda", 0) if torch.cuda.is_available() else None
    crow, col, info = syn.powerlaw_csr(spec, seed=0, device=device)
    crow, col = crow.cpu(), col.cpu()
    if device is not None:
        torch.cuda.empty_cache()
    return spec, crow, col, info["nnz"], spec.rows


def run_reference(args) -> dict:
    """The reference's CPU implementation of the path (torch.sparse.mm over a CSR tensor, as restated
    in oracle/, then nn.Linear for the layer workload) on all of this host's cores.  By default every
    step is one call on the WHOLE graph of the GPU arm; --cpu-sample-nnz K (the in-line cpu_baseline leg
    of the GPU arm uses it) restricts a step to the first rows holding about K edges, gathering from the
    full X.  The reported time is the median of the timed steps."""
    from benchlib import synthetic as syn
    from oracle import oracle

    # torch.distributed.run exports OMP_NUM_THREADS=1; the CPU arm is meant to use every host core
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    spec, sub_crow, sub_col, total_nnz, rows = reference_graph(args)
    n, f = spec.rows, args.features
    nnz = int(sub_crow[-1])
    whole = rows == n
    weighted = not args.workload.startswith("c5")
    sub_val = syn.edge_values(nnz, seed=0) if weighted else None
    x = syn.dense(n, f, 3)
    conv = args.workload == "c5_conv"  # the layer forward: aggregation, then Linear F -> 256
    if conv:
        torch.manual_seed(0)
        linear = torch.nn.Linear(f, 256)
        torch.nn.init.xavier_uniform_(linear.weight)
        torch.nn.init.zeros_(linear.bias)

    def reference_step():
        aggregated = oracle.spmm_reference_cpu(sub_crow, sub_col, sub_val, x)
        return linear(aggregated) if conv else aggregated

    laps = []
    with torch.no_grad():
        for _ in range(max(1, min(args.warmup, 2))):
            reference_step()
        for _ in range(args.steps):
            t0 = time.perf_counter()
            reference_step()
            laps.append(time.perf_counter() - t0)
    seconds = statistics.median(laps)
    sample_bytes = spmm_bytes(rows, nnz, f, weighted) + (4 * rows * f + 4 * rows * 256 if conv else 0)
    value = round(sample_bytes / seconds / 1e9, 3)
    if whole:
        sample = (f"the whole graph ({rows} rows, {nnz} nnz) per step; torch.sparse.mm on CPU float32"
                  + (", then nn.Linear" if conv else "") + "; median of the timed steps")
    else:
        sample = (f"first {rows} rows ({nnz} nnz) of the {n}-row CSR against the full X; "
                  f"torch.sparse.mm on CPU float32" + (", then nn.Linear on those rows" if conv else "")
                  + "; median of the timed steps")
    workload = conv_workload_label(n, total_nnz, f) if conv else (
        f"{args.workload}: power-law CSR {n} rows, {total_nnz} nnz, F={f}" + (", weighted" if weighted else ""))
    return {
        "impl": "reference",
        "metric": "algorithmic_GBps",
        "value": value,
        "unit": "GB/s",
        "n_gpus": args.gpus,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": round(seconds * 1e3, 3),
        "ms_per_step_mean_min_max": [round(statistics.fmean(laps) * 1e3, 3), round(min(laps) * 1e3, 3),
                                     round(max(laps) * 1e3, 3)],
        "higher_is_better": True,
        "scaling": "strong",
        "vs_baseline": None,
        "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": workload, "sample": sample},
        "edges_f_per_s": round(nnz * f / seconds, 1),
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--workload", default=None)
    parser.add_argument("--features", type=int, default=128)
    parser.add_argument("--tile", type=int, default=None)
    parser.add_argument("--warps", type=int, default=4)
    parser.add_argument("--hub-threshold", type=int, default=1024)
    parser.add_argument("--cpu-sample-nnz", type=int, default=None,
                        help="CPU legs: edges of the row sample one call covers (default: 4,000,000 for the "
                             "in-line cpu_baseline of the GPU arm, 0 = the whole graph for --impl reference)")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-other-configs", action="store_true",
                        help="N = 1: skip the short runs of configurations 2, 3 and 4")
    parser.add_argument("--groups", default=None,
                        help="sharded path: number of column groups per GPU, or their sizes in arrival order "
                             "(e.g. 1,3,3,1 for 8 GPUs: own columns first, one owner last)")
    parser.add_argument("--slabs", type=int, default=0, help="feature bands of the slab exchange (sharded path; 0 = column blocks)")
    parser.add_argument("--copy-streams", type=int, default=1, help="streams used for the peer pulls (sharded path)")
    parser.add_argument("--no-graph", action="store_true",
                        help="sharded path: launch every step eagerly instead of replaying a CUDA graph")
    parser.add_argument("--exchange", default=None, choices=["peer", "nccl", "allgather", "push"],
                        help="how X is gathered (sharded path)")
    parser.add_argument("--chunks", type=int, default=2, help="chunks of the allgather / push exchange")
    parser.add_argument("--push-ctas", type=int, default=32, help="CTAs of the SM-driven push")
    args = parser.parse_args()
    if args.groups is not None:
        args.groups = [int(v) for v in args.groups.split(",")] if "," in args.groups else int(args.groups)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if args.workload is None:
        args.workload = "c5_conv"
    if args.tile is None:
        # X of configuration 2 is about the size of L2: 64-wide tiles keep the gathered slice
        # resident; configuration 5's X is ten times L2 and whole 128-float rows stream best.
        args.tile = 128 if args.workload.startswith("c5") else 64

    if args.cpu_sample_nnz is None:
        args.cpu_sample_nnz = 0 if args.impl == "reference" else 4_000_000
    if args.impl == "reference":
        if rank == 0:
            print(json.dumps(run_reference(args)), flush=True)
        return
    if world > 1 or args.gpus > 1 or args.workload == "c5_conv":
        from benchlib import dist_bench

        line = dist_bench.run(args)
        if line is not None:
            print(json.dumps(line), flush=True)
        return
    print(json.dumps(run_ours_single(args)), flush=True)


if __name__ == "__main__":
    main()
