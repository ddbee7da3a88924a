"""The scheduler: shortlist -> sampled probe -> guardrail -> run -> cached schedule.

Public behaviour follows the reference ``autosage/_auto.py`` (spmm_csr_auto :266-441,
calibrate_full :444-522, sddmm_csr_auto :544-741, _csr_row_softmax :744-759,
csr_attention_forward :762-780): same signatures, same result-dict keys, same cache records, the
0.95 guardrail against the vendor baseline, replay-only mode.  What changed is what is being
chosen: the candidates ``[feature_tile, warps_per_block, hub_threshold]`` now parameterise the
sm_100a kernels behind ``torch.ops.autosage`` (tile = features per pass, warps = CTA width shared
by a hub row, threshold = degree from which a row takes the CTA-per-hub path).

Deliberate departures, all invisible in the dict layout:
  * the probe runs on a seeded ROW sample that keeps every edge of a sampled row and gathers from
    the full dense operand, sized by WORK: the row fraction is raised from ``probe_fraction`` until
    the sample holds about AUTOSAGE_PROBE_EDGES edges (default 16 M, roughly half a millisecond of B200
    time; graphs below that are probed whole, without copying anything), and the candidates' time
    budget is the larger of ``probe_cap_ms`` and ``probe_iterations`` baseline runs.  The reference
    probes the sub-graph INDUCED by 3 % of the rows (``_auto.py:95-154``), which keeps ~0.1 % of the
    edges and ~3 % of every degree: on B200 every kernel then finishes in microseconds, the probe
    measures launch overhead and the latency of the one hub row it caught, and the guardrail picks the
    vendor baseline for graphs on which the kernels are 2-3x faster (measured).
    AUTOSAGE_PROBE_SAMPLE=induced restores the reference's sample and budget (same selected rows).
  * hub thresholds are ranked in full-graph degree units.  The reference derives them from the
    sampled sub-graph (``_auto.py:356``) and then applies them to the full graph (``:402``); here the
    shortlist comes from the full graph (with the induced sample each threshold is translated to the
    sample's matching degree quantile for the probe; the row sample needs no translation).
  * the library's default parameters are probed next to the analytical shortlist, so a schedule is
    never slower than the plain operator.
  * ``csr_attention_forward`` accepts ``scale`` and runs the fused one-pass kernel when it wins.
"""
from __future__ import annotations

import os
import statistics
import time
import weakref
from typing import Any, Callable, Optional

import torch

from . import _native
from ._cache import ScheduleCache, device_signature, graph_signature, log_probe, rounded_quantiles
from .config import SchedulerConfig
from .ops import (DEFAULT_HUB_THRESHOLD, DEFAULT_TILE, DEFAULT_WARPS, SDDMM_HUB_THRESHOLD, SDDMM_WARPS, _base_flags,
                  _normalize_csr, load_native, native_op, spmm_csr)

AUTOTUNE_SCHEMA_VERSION = 3
# (warps per CTA, hub threshold) the fused attention kernel is probed with first: the best of the B200 sweeps
ATTENTION_DEFAULT = (4, 1024)
_INF = float("inf")


# ------------------------------------------------------------------------------------------------
# timing
# ------------------------------------------------------------------------------------------------
@torch.no_grad()  # probes never need an autograd graph
def _time_cuda(function: Callable[[], torch.Tensor], *, warmup: int, iterations: int,
               cap_ms: Optional[float] = None) -> dict[str, Any]:
    """CUDA-event timing of ``function``: ``warmup`` untimed calls, then up to ``iterations`` timed
    ones, stopping early once their sum reaches ``cap_ms``."""
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(max(warmup, 0)):
        function()
    torch.cuda.synchronize()
    laps: list[float] = []
    spent = 0.0
    result = None
    budget = None if cap_ms is None else max(cap_ms, 0.0)
    for _ in range(max(iterations, 1)):
        begin, finish = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        result = function()
        finish.record()
        finish.synchronize()
        lap = float(begin.elapsed_time(finish))
        laps.append(lap)
        spent += lap
        if budget is not None and spent >= budget:
            break
    torch.cuda.synchronize()
    return {
        "best_ms": min(laps),
        "mean_ms": statistics.fmean(laps),
        "std_ms": statistics.pstdev(laps) if len(laps) > 1 else 0.0,
        "iterations": len(laps),
        "total_ms": spent,
        "wall_ms": (time.perf_counter() - t0) * 1000.0,
        "output": result,
    }


def _without_output(timing: dict[str, Any]) -> dict[str, Any]:
    return {k: v for k, v in timing.items() if k != "output"}


@torch.no_grad()
def _time_cuda_batch(functions: list[Callable[[], torch.Tensor]], *, warmup: int, iterations: int) -> list[dict[str, Any]]:
    """CUDA-event timing of several functions enqueued back to back: per function ``warmup`` untimed
    calls and ``iterations`` timed ones, every lap between its own pair of events, ONE host
    synchronisation after the last function.  (``_time_cuda`` synchronises after every lap, which the
    reference does per candidate, ``autosage/_auto.py:324-378``.)"""
    t0 = time.perf_counter()
    recorded: list[list[tuple]] = []
    for function in functions:
        for _ in range(max(warmup, 0)):
            function()
        pairs = []
        for _ in range(max(iterations, 1)):
            begin, finish = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            function()
            finish.record()
            pairs.append((begin, finish))
        recorded.append(pairs)
    torch.cuda.synchronize()
    wall_each = (time.perf_counter() - t0) * 1000.0 / max(len(functions), 1)
    timings = []
    for pairs in recorded:
        laps = [float(begin.elapsed_time(finish)) for begin, finish in pairs]
        timings.append({
            "best_ms": min(laps),
            "mean_ms": statistics.fmean(laps),
            "std_ms": statistics.pstdev(laps) if len(laps) > 1 else 0.0,
            "iterations": len(laps),
            "total_ms": sum(laps),
            "wall_ms": wall_each,
        })
    return timings


# ------------------------------------------------------------------------------------------------
# baselines (the guardrail's comparators; also what "baseline" schedules run)
# ------------------------------------------------------------------------------------------------
def _prepare_spmm_baseline(crow, col, val, x) -> tuple[Callable[[], torch.Tensor], str]:
    weights = torch.ones(col.numel(), device=x.device, dtype=x.dtype) if val is None else val.to(x.dtype)
    matrix = torch.sparse_csr_tensor(crow, col, weights, size=(crow.numel() - 1, x.size(0)),
                                     device=x.device, dtype=x.dtype)
    return (lambda: torch.sparse.mm(matrix, x)), "torch.sparse.mm(csr)"


def _row_ids(crow: torch.Tensor) -> torch.Tensor:
    degrees = (crow[1:] - crow[:-1]).to(torch.long)
    return torch.repeat_interleave(torch.arange(crow.numel() - 1, device=crow.device, dtype=torch.long), degrees)


def _prepare_sddmm_baseline(crow, col, query, key) -> tuple[Callable[[], torch.Tensor], str]:
    rows = _row_ids(crow)
    return (lambda: (query.index_select(0, rows) * key.index_select(0, col)).sum(dim=1)), "gather-dot"


# ------------------------------------------------------------------------------------------------
# induced sample (integer outputs are bit-exact with the reference, _auto.py:95-154)
# ------------------------------------------------------------------------------------------------
def _induced_sample_csr(crow, col, val, *, fraction: float, minimum_rows: int, seed: int):
    """Sub-graph induced by a seeded random row sample: keeps the edges whose row AND column are
    sampled and relabels both to sample positions.  Returns (crow, col, val, selected_rows)."""
    n = crow.numel() - 1
    k = min(max(int(n * fraction), minimum_rows, 1), n)
    device = crow.device
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    selected = torch.randperm(n, generator=gen, device=device)[:k].sort().values

    new_id = torch.full((n,), -1, dtype=torch.long, device=device)
    new_id[selected] = torch.arange(k, device=device)
    begin = crow.index_select(0, selected)
    degree = crow.index_select(0, selected + 1) - begin
    total = int(degree.sum().item())
    if total == 0:
        empty_val = None if val is None else torch.empty(0, dtype=val.dtype, device=val.device)
        return (torch.zeros(k + 1, dtype=torch.long, device=device),
                torch.empty(0, dtype=torch.long, device=col.device), empty_val, selected)

    owner = torch.repeat_interleave(torch.arange(k, device=device, dtype=torch.long), degree)
    first_slot = torch.cumsum(degree, 0) - degree  # position of each sampled row's first edge
    edge_pos = begin.index_select(0, owner) + (
        torch.arange(total, device=device, dtype=torch.long) - first_slot.index_select(0, owner))
    relabelled = new_id.index_select(0, col.index_select(0, edge_pos))
    keep = relabelled >= 0
    kept_per_row = torch.bincount(owner[keep], minlength=k)
    sampled_crow = torch.cat((torch.zeros(1, dtype=torch.long, device=device), kept_per_row.cumsum(0)))
    sampled_col = relabelled[keep].contiguous()
    sampled_val = None if val is None else val.index_select(0, edge_pos)[keep].contiguous()
    return sampled_crow, sampled_col, sampled_val, selected


def _row_sample_csr(crow, col, val, *, fraction: float, minimum_rows: int, seed: int):
    """The same seeded row selection as ``_induced_sample_csr``, but every edge of a selected row is
    kept and column ids stay global: a k x N slice of the matrix.  Returns (crow, col, val, selected)."""
    n = crow.numel() - 1
    k = min(max(int(n * fraction), minimum_rows, 1), n)
    device = crow.device
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    selected = torch.randperm(n, generator=gen, device=device)[:k].sort().values
    begin = crow.index_select(0, selected)
    degree = crow.index_select(0, selected + 1) - begin
    sampled_crow = torch.cat((torch.zeros(1, dtype=torch.long, device=device), degree.cumsum(0)))
    total = int(sampled_crow[-1].item())
    if total == 0:
        empty_val = None if val is None else torch.empty(0, dtype=val.dtype, device=val.device)
        return sampled_crow, torch.empty(0, dtype=torch.long, device=col.device), empty_val, selected
    owner = torch.repeat_interleave(torch.arange(k, device=device, dtype=torch.long), degree)
    edge_pos = begin.index_select(0, owner) + (
        torch.arange(total, device=device, dtype=torch.long) - sampled_crow[:-1].index_select(0, owner))
    sampled_col = col.index_select(0, edge_pos)
    sampled_val = None if val is None else val.index_select(0, edge_pos)
    return sampled_crow, sampled_col, sampled_val, selected


class _ProbeSample:
    """What a probe runs on.  ``row_side`` maps a dense operand indexed by ROW (Q) to the sample,
    ``column_side`` one indexed by COLUMN (X, K, V): gathered rows for the induced sub-graph, the
    operand itself for the row sample.  ``threshold`` maps a full-graph hub threshold to the sample."""

    def __init__(self, crow, col, val, selected, induced: bool, translation: Optional[dict[int, int]]) -> None:
        self.crow, self.col, self.val, self.selected, self.induced = crow, col, val, selected, induced
        self._translation = translation or {}

    def row_side(self, dense: torch.Tensor) -> torch.Tensor:
        return dense.index_select(0, self.selected).contiguous()

    def column_side(self, dense: torch.Tensor) -> torch.Tensor:
        return self.row_side(dense) if self.induced else dense

    def threshold(self, full: int) -> int:
        return max(1, int(self._translation.get(full, full)))

    @property
    def rows(self) -> int:
        return self.crow.numel() - 1

    # What the vendor baselines (which need exactly sized arrays) run on, and the numbers reported.
    def exact(self):
        return self.crow, self.col, self.val

    def exact_rows(self, row_operand: torch.Tensor) -> torch.Tensor:
        return row_operand

    def counts(self) -> tuple[int, int]:
        return self.rows, self.col.numel()


class _DeviceRowSample(_ProbeSample):
    """Row sample cut by the library (``asg_csr_row_sample``) without a host synchronisation.

    ``crow`` / ``col`` / ``val`` are the arrays as allocated: a valid CSR of all selected rows over a
    column array of ``capacity`` entries, of which the first ``kept[1]`` are meaningful (selected rows
    that did not fit the capacity are empty).  The library's kernels run on them as they are; whoever
    needs exactly sized arrays (cuSPARSE through torch, the reported counts) calls ``exact()``, which
    reads the two counters back - by then the candidates have been timed and the stream is idle."""

    def __init__(self, crow, col, val, selected, kept) -> None:
        super().__init__(crow, col, val, selected, False, None)
        self._kept = kept
        self._counts: Optional[tuple[int, int]] = None

    def counts(self) -> tuple[int, int]:
        if self._counts is None:
            rows_kept, edges_kept = (int(v) for v in self._kept.tolist())
            self._counts = (rows_kept, edges_kept)
        return self._counts

    def exact(self):
        rows_kept, edges_kept = self.counts()
        return (self.crow[: rows_kept + 1], self.col[:edges_kept],
                None if self.val is None else self.val[:edges_kept])

    def exact_rows(self, row_operand: torch.Tensor) -> torch.Tensor:
        return row_operand[: self.counts()[0]]


def _probe_sample_kind() -> str:
    return "induced" if os.getenv("AUTOSAGE_PROBE_SAMPLE", "rows").strip().lower() == "induced" else "rows"


# The probes call the library directly (not torch.ops.autosage): the operators keep the reference's
# square-matrix contract, the row sample is a k x N slice.
def _probe_spmm(crow, col, val, x, tile: int, warps: int, threshold: int) -> torch.Tensor:
    y = torch.empty(crow.numel() - 1, x.size(1), dtype=x.dtype, device=x.device)
    if y.numel() == 0:
        return y
    workspace, ready = _native.planned_workspace(crow, threshold)
    _native.spmm(crow, col, val, x, y, feature_tile=tile, warps=warps, threshold=threshold,
                 flags=_base_flags() | ready, workspace=workspace)
    return y


def _probe_sddmm(crow, col, query, key, warps: int, threshold: int) -> torch.Tensor:
    out = torch.empty(col.numel(), dtype=query.dtype, device=query.device)
    if out.numel() == 0:
        return out
    workspace, ready = _native.planned_workspace(crow, threshold)
    _native.sddmm(crow, col, query, key, out, warps=warps, threshold=threshold, flags=_base_flags() | ready,
                  workspace=workspace)
    return out


# ------------------------------------------------------------------------------------------------
# shortlist
# ------------------------------------------------------------------------------------------------
def _degree_quantiles(crow: torch.Tensor) -> tuple[int, int, int]:
    degrees = crow[1:] - crow[:-1]
    if degrees.numel() == 0:
        return 1, 1, 1
    q90, q95, q99 = (max(1, q) for q in rounded_quantiles(degrees, [0.9, 0.95, 0.99]))
    return q90, q95, q99


def _spmm_candidates(crow: torch.Tensor, feature_width: int, config: SchedulerConfig) -> list[tuple[int, int, int]]:
    """Up to ``candidate_count`` distinct (feature_tile, warps_per_block, hub_threshold) triples,
    nearest first to the analytical preference: tile 64 for F <= 64 else 128; 8/4/2 warps for a
    degree skew q99/q50 of >=4 / >=2 / less; threshold at the 95th degree percentile."""
    q90, q95, q99 = _degree_quantiles(crow)
    degrees = crow[1:] - crow[:-1]
    q50 = rounded_quantiles(degrees, [0.5])[0] if degrees.numel() else 1
    skew = q99 / max(q50, 1)
    want_warps = 8 if skew >= 4 else (4 if skew >= 2 else 2)
    want_tile = 64 if feature_width <= 64 else 128
    want_threshold = q95

    tile_options = [64, 128] if config.feature_tile is None else [config.feature_tile]
    warp_options = [2, 4, 8] if config.warps_per_block is None else [config.warps_per_block]
    if config.hub_threshold is None:
        threshold_options = list(dict.fromkeys((q95, q90, q99)))
    else:
        threshold_options = [config.hub_threshold]

    def distance(c: tuple[int, int, int]) -> tuple[float, tuple[int, int, int]]:
        tile, warps, threshold = c
        d = abs(tile - want_tile) / 64
        d += abs(warps - want_warps) / 6
        d += abs(threshold - want_threshold) / max(want_threshold, 1)
        return d, c

    pool = {(int(t), int(w), max(1, int(h))) for t in tile_options for w in warp_options for h in threshold_options}
    return sorted(pool, key=distance)[: max(1, config.candidate_count)]


def _threshold_translation(full_crow: torch.Tensor, sample_crow: torch.Tensor, config: SchedulerConfig) -> dict[int, int]:
    """Full-graph hub threshold -> the sample's threshold at the same degree quantile."""
    if config.hub_threshold is not None:
        return {int(config.hub_threshold): int(config.hub_threshold)}
    return {full: sample for full, sample in zip(_degree_quantiles(full_crow), _degree_quantiles(sample_crow))}


# ------------------------------------------------------------------------------------------------
# result helpers
# ------------------------------------------------------------------------------------------------
def _cache_hit_allowed(result: dict[str, Any], config: SchedulerConfig) -> bool:
    if result.get("schema_version") != AUTOTUNE_SCHEMA_VERSION:
        return False
    return True if config.replay_only else result.get("configuration") == config.tuning_signature()


def _cached_native_available(operation: str, choice: str, candidate: Optional[list[int]]) -> bool:
    if choice != "autosage":
        return True
    return native_op(operation + ("_split" if candidate is not None else "")) is not None


def _cpu_info(operation: str) -> dict[str, Any]:
    return {
        "operation": operation,
        "schema_version": AUTOTUNE_SCHEMA_VERSION,
        "choice": "baseline",
        "baseline": "torch CPU",
        "from_cache": False,
        "reason": "AutoSAGE scheduling is CUDA-only",
    }


def _replay_miss(operation: str, baseline_name: str) -> dict[str, Any]:
    return {
        "operation": operation,
        "schema_version": AUTOTUNE_SCHEMA_VERSION,
        "choice": "baseline",
        "baseline": baseline_name,
        "from_cache": False,
        "replay_only": True,
        "reason": "cache miss",
    }


def _run_spmm_choice(choice, candidate, crow, col, val, x) -> torch.Tensor:
    # torch's CSR SpMM cannot differentiate with respect to the values of a pattern that repeats a
    # column inside a row; a "baseline" schedule then runs the native operator, which can.
    needs_value_grad = val is not None and val.requires_grad and torch.is_grad_enabled()
    if choice == "autosage" or (needs_value_grad and x.is_cuda and native_op("spmm_csr") is not None):
        split, core = native_op("spmm_csr_split"), native_op("spmm_csr")
        if split is not None and candidate is not None:
            return split(crow, col, val, x, *(int(c) for c in candidate))
        if core is not None:
            return core(crow, col, val, x)
    return _prepare_spmm_baseline(crow, col, val, x)[0]()


def _run_sddmm_choice(choice, candidate, crow, col, query, key) -> torch.Tensor:
    if choice == "autosage":
        split, core = native_op("sddmm_csr_split"), native_op("sddmm_csr")
        if split is not None and candidate is not None:
            return split(crow, col, query, key, *(int(c) for c in candidate))
        if core is not None:
            return core(crow, col, query, key)
    return _prepare_sddmm_baseline(crow, col, query, key)[0]()


# ------------------------------------------------------------------------------------------------
# the probe engine shared by SpMM, SDDMM and fused attention
# ------------------------------------------------------------------------------------------------
class _Memo:
    """graph_signature memo: the signature sorts all degrees and copies 4096 indices to the host,
    which would otherwise happen on every replayed call.  Entries die with their tensors."""

    def __init__(self) -> None:
        self._entries: dict[tuple, tuple] = {}

    def signature(self, crow, col, width, operation, weighted, dtype) -> dict[str, Any]:
        key = (crow.data_ptr(), col.data_ptr(), crow.numel(), col.numel(), int(width), operation, bool(weighted), str(dtype))
        hit = self._entries.get(key)
        if hit is not None:
            crow_ref, col_ref, versions, value = hit
            if crow_ref() is crow and col_ref() is col and versions == (crow._version, col._version):
                return dict(value)
        value = graph_signature(crow, col, width, operation, weighted=weighted, dtype=dtype)
        if len(self._entries) > 64:
            self._entries.clear()
        self._entries[key] = (weakref.ref(crow), weakref.ref(col), (crow._version, col._version), dict(value))
        return value


_SIGNATURES = _Memo()


def _probe_and_choose(
    *,
    operation: str,
    label: str,
    config: SchedulerConfig,
    device: dict[str, Any],
    graph: dict[str, Any],
    cache: ScheduleCache,
    sample_ms: float,
    sample: _ProbeSample,
    make_baseline: Callable[[], tuple[Callable[[], torch.Tensor], str]],
    candidates: list[tuple[list[int], Callable[[], torch.Tensor]]],
    fallback: Optional[Callable[[], torch.Tensor]],
    verbose: bool,
    preferred: Optional[tuple] = None,
) -> dict[str, Any]:
    """Times the shortlisted candidates and the baseline on the sample and applies the guardrail.
    ``candidates`` pairs the full-graph parameter list stored in the schedule with a closure running it
    on the sample; ``fallback`` is the parameter-free native kernel used when hub splitting is disabled;
    ``make_baseline`` builds the vendor baseline on the sample's exactly sized arrays.

    Work-sized samples (the default): every candidate is enqueued back to back - one warm-up and two
    timed laps each, every lap between its own events - with a single synchronisation after the last
    one; only then are the sample's sizes read back, the baseline built and timed.  The induced sample
    (AUTOSAGE_PROBE_SAMPLE=induced) keeps the reference's procedure: baseline first, then candidate after
    candidate under ``probe_cap_ms``, synchronising after every lap."""
    work_sized = _probe_sample_kind() != "induced"
    timings: list[dict[str, Any]] = []
    best, best_params = _INF, None
    if work_sized:
        laps_each = max(1, min(2, config.probe_iterations))
        runs = list(candidates) if candidates else ([(None, fallback)] if fallback is not None else [])
        for (params, _), lap in zip(runs, _time_cuda_batch([run for _, run in runs], warmup=1, iterations=laps_each)):
            timings.append({"candidate": None if params is None else list(params), **lap})
            if lap["best_ms"] < best:
                best, best_params = lap["best_ms"], None if params is None else list(params)
        baseline, baseline_name = make_baseline()
        # a slow baseline (the gather-dot SDDMM takes tens of ms) is not timed three times
        base = _time_cuda(baseline, warmup=1, iterations=laps_each, cap_ms=25.0)
    else:
        baseline, baseline_name = make_baseline()
        base = _time_cuda(baseline, warmup=1, iterations=config.probe_iterations)
        remaining = config.probe_cap_ms
        if candidates:
            for index, (params, run) in enumerate(candidates):
                if index > 0 and remaining <= 0.0:
                    break
                lap = _time_cuda(run, warmup=1, iterations=config.probe_iterations, cap_ms=max(0.0, remaining))
                remaining = max(0.0, remaining - lap["total_ms"])
                timings.append({"candidate": list(params), **_without_output(lap)})
                if lap["best_ms"] < best:
                    best, best_params = lap["best_ms"], list(params)
        elif fallback is not None:
            lap = _time_cuda(fallback, warmup=1, iterations=config.probe_iterations, cap_ms=config.probe_cap_ms)
            best = lap["best_ms"]
            timings.append({"candidate": None, **_without_output(lap)})
    if candidates and preferred is not None:
        # a candidate within 5 % of the best is a tie on a sample: keep the library default then
        for entry in timings:
            if entry["candidate"] == list(preferred) and entry["best_ms"] <= 1.05 * best:
                best, best_params = entry["best_ms"], list(preferred)
    probe_rows, probe_nonzeros = sample.counts()

    enough = probe_rows >= config.minimum_probe_rows and probe_nonzeros >= config.minimum_probe_nonzeros
    wins = enough and best <= config.guardrail * base["best_ms"]
    result = {
        "operation": operation,
        "schema_version": AUTOTUNE_SCHEMA_VERSION,
        "choice": "autosage" if wins else "baseline",
        "candidate": best_params if wins else None,
        "baseline": baseline_name,
        "guardrail": config.guardrail,
        "configuration": config.tuning_signature(),
        "probe_rows": int(probe_rows),
        "probe_nonzeros": int(probe_nonzeros),
        "sampling_ms": sample_ms,
        "probe_ms": sample_ms + base["wall_ms"] + sum(t["wall_ms"] for t in timings),
        "baseline_probe_ms": base["best_ms"],
        "autosage_probe_ms": None if best == _INF else best,
        "sampled_speedup": (base["best_ms"] / best) if best not in (0.0, _INF) else None,
        "candidates": timings,
        "from_cache": False,
    }
    if config.cache:
        cache.store(device, graph, result)
    log_probe({"timestamp": time.time(), "device": device, "graph": graph, "result": result})
    if verbose or os.getenv("AUTOSAGE_VERBOSE") == "1":
        print(f"[autosage:{label}] rows={result['probe_rows']} nnz={result['probe_nonzeros']} "
              f"baseline={result['baseline_probe_ms']:.4f} ms auto={result['autosage_probe_ms']} "
              f"choice={result['choice']}")
    return result


def _lookup(cache: ScheduleCache, config: SchedulerConfig, device, graph, op_name: str) -> Optional[dict[str, Any]]:
    if not config.cache:
        return None
    record = cache.lookup(device, graph)
    if record is None:
        return None
    result = record.get("result", {})
    if not _cache_hit_allowed(result, config):
        return None
    if not _cached_native_available(op_name, result.get("choice", "baseline"), result.get("candidate")):
        return None
    return result


def _probe_target_edges() -> int:
    try:
        return max(1, int(os.getenv("AUTOSAGE_PROBE_EDGES", str(16 * 1024 * 1024))))
    except ValueError:
        return 16 * 1024 * 1024


class _WholeGraph(_ProbeSample):
    """The graph itself as its own probe sample (small graphs): nothing is copied."""

    def __init__(self, crow, col, val) -> None:
        super().__init__(crow, col, val, None, False, None)

    def row_side(self, dense: torch.Tensor) -> torch.Tensor:
        return dense


def _timed_sample(crow, col, val, config: SchedulerConfig, seed: int) -> tuple[_ProbeSample, float]:
    t0 = time.perf_counter()
    if _probe_sample_kind() == "induced":
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        s_crow, s_col, s_val, selected = _induced_sample_csr(crow, col, val, fraction=config.probe_fraction,
                                                             minimum_rows=config.probe_min_rows, seed=seed)
        return _ProbeSample(s_crow, s_col, s_val, selected, True, _threshold_translation(crow, s_crow, config)), t0
    nnz = col.numel()
    fraction = max(config.probe_fraction, min(1.0, _probe_target_edges() / max(nnz, 1)))
    rows = crow.numel() - 1
    if fraction >= 0.999 or max(int(rows * fraction), config.probe_min_rows) >= rows:
        return _WholeGraph(crow, col, val), t0
    if crow.is_cuda and load_native() and (val is None or val.dtype == torch.float32):
        # the library cuts the rows out: no ATen sequence, no host synchronisation
        k = min(max(int(rows * fraction), config.probe_min_rows, 1), rows)
        gen = torch.Generator(device=crow.device)
        gen.manual_seed(seed)
        selected = torch.randperm(rows, generator=gen, device=crow.device)[:k].sort().values
        capacity = min(nnz, int(1.25 * fraction * nnz) + (1 << 20))
        s_crow, s_col, s_val, kept = _native.csr_row_sample(crow, col, val, selected, capacity)
        return _DeviceRowSample(s_crow, s_col, s_val, selected, kept), t0
    s_crow, s_col, s_val, selected = _row_sample_csr(crow, col, val, fraction=fraction,
                                                     minimum_rows=config.probe_min_rows, seed=seed)
    return _ProbeSample(s_crow, s_col, s_val, selected, False, None), t0


def _with_library_default(shortlist: list, default: tuple, forced: bool) -> list:
    """The library's default parameters first (so a schedule never loses to the plain operator), then
    the analytical shortlist.  Nothing is added when the configuration pins a parameter."""
    if forced or default in shortlist:
        return list(shortlist)
    return [default] + list(shortlist)


# ------------------------------------------------------------------------------------------------
# SpMM
# ------------------------------------------------------------------------------------------------
def spmm_csr_auto(crow, col, val, x, *, guardrail: float = 0.95, k: int = 6, seed: int = 0,
                  verbose: bool = False) -> tuple[torch.Tensor, dict[str, Any]]:
    crow, col, val, x = _normalize_csr(crow, col, val, x)
    if not x.is_cuda:
        return spmm_csr(crow, col, val, x), _cpu_info("spmm")
    if x.dtype != torch.float32:
        run, name = _prepare_spmm_baseline(crow, col, val, x)
        return run(), {**_cpu_info("spmm"), "baseline": name,
                       "reason": "AutoSAGE CUDA kernels require float32 features"}

    load_native()
    config = SchedulerConfig.from_env(guardrail=guardrail, candidate_count=k)
    device = device_signature()
    graph = _SIGNATURES.signature(crow, col, x.size(1), "spmm", val is not None, x.dtype)
    cache = ScheduleCache()

    hit = _lookup(cache, config, device, graph, "spmm_csr")
    if hit is not None:
        output = _run_spmm_choice(hit.get("choice", "baseline"), hit.get("candidate"), crow, col, val, x)
        return output, {**hit, "from_cache": True}
    if config.replay_only:
        return _run_spmm_choice("baseline", None, crow, col, val, x), _replay_miss("spmm", "torch.sparse.mm(csr)")

    sample, t0 = _timed_sample(crow, col, val, config, seed)
    s_crow, s_col, s_val = sample.crow, sample.col, sample.val
    s_x = sample.column_side(x)
    if sample.induced:
        torch.cuda.synchronize()
    sample_ms = (time.perf_counter() - t0) * 1000.0

    def make_baseline():
        e_crow, e_col, e_val = sample.exact()
        return _prepare_spmm_baseline(e_crow, e_col, e_val, s_x)

    split = native_op("spmm_csr_split") if config.hub_split else None
    core = native_op("spmm_csr")
    runs: list[tuple[list[int], Callable[[], torch.Tensor]]] = []
    if split is not None:
        forced = any(v is not None for v in (config.feature_tile, config.warps_per_block, config.hub_threshold))
        shortlist = _with_library_default(_spmm_candidates(crow, x.size(1), config),
                                          (DEFAULT_TILE, DEFAULT_WARPS, DEFAULT_HUB_THRESHOLD), forced)
        for tile, warps, threshold in shortlist:
            runs.append(([tile, warps, threshold],
                         lambda t=tile, w=warps, h=sample.threshold(threshold): _probe_spmm(s_crow, s_col, s_val, s_x, t, w, h)))
    result = _probe_and_choose(
        operation="spmm", label="spmm", config=config, device=device, graph=graph, cache=cache,
        sample_ms=sample_ms, sample=sample, make_baseline=make_baseline, candidates=runs,
        fallback=(lambda: _probe_spmm(s_crow, s_col, s_val, s_x, DEFAULT_TILE, DEFAULT_WARPS, DEFAULT_HUB_THRESHOLD))
        if core is not None else None, verbose=verbose,
        preferred=(DEFAULT_TILE, DEFAULT_WARPS, DEFAULT_HUB_THRESHOLD))
    output = _run_spmm_choice(result["choice"], result["candidate"] if result["choice"] == "autosage" else None,
                              crow, col, val, x)
    return output, result


def calibrate_full(crow, col, val, x, guardrail: float = 0.95) -> tuple[str, dict[str, Any]]:
    """Times the baseline and every shortlisted candidate on the FULL graph and stores the winner."""
    crow, col, val, x = _normalize_csr(crow, col, val, x)
    if not x.is_cuda:
        return "baseline", _cpu_info("spmm")
    if x.dtype != torch.float32:
        return "baseline", {**_cpu_info("spmm"), "baseline": "torch.sparse.mm(csr)",
                            "reason": "AutoSAGE CUDA kernels require float32 features"}
    load_native()
    config = SchedulerConfig.from_env(guardrail=guardrail, candidate_count=6)
    baseline, baseline_name = _prepare_spmm_baseline(crow, col, val, x)
    base = _time_cuda(baseline, warmup=2, iterations=5)
    split = native_op("spmm_csr_split") if config.hub_split else None
    core = native_op("spmm_csr")
    best, winner = _INF, None
    laps: list[dict[str, Any]] = []
    if split is not None:
        for tile, warps, threshold in _spmm_candidates(crow, x.size(1), config):
            lap = _time_cuda(lambda t=tile, w=warps, h=threshold: split(crow, col, val, x, t, w, h),
                             warmup=2, iterations=5)
            laps.append({"candidate": [tile, warps, threshold], "best_ms": lap["best_ms"]})
            if lap["best_ms"] < best:
                best, winner = lap["best_ms"], [tile, warps, threshold]
    elif core is not None:
        best = _time_cuda(lambda: core(crow, col, val, x), warmup=2, iterations=5)["best_ms"]
        laps.append({"candidate": None, "best_ms": best})
    choice = "autosage" if best <= guardrail * base["best_ms"] else "baseline"
    result = {
        "operation": "spmm",
        "schema_version": AUTOTUNE_SCHEMA_VERSION,
        "choice": choice,
        "candidate": winner if choice == "autosage" else None,
        "baseline": baseline_name,
        "guardrail": guardrail,
        "configuration": config.tuning_signature(),
        "calibration": "full_graph",
        "baseline_ms": base["best_ms"],
        "autosage_ms": None if best == _INF else best,
        "speedup": (base["best_ms"] / best) if best not in (0.0, _INF) else None,
        "candidates": laps,
        "from_cache": False,
    }
    device = device_signature()
    graph = graph_signature(crow, col, x.size(1), "spmm", weighted=val is not None, dtype=x.dtype)
    if config.cache:
        ScheduleCache().store(device, graph, result)
    log_probe({"timestamp": time.time(), "device": device, "graph": graph, "result": result})
    return choice, result


# ------------------------------------------------------------------------------------------------
# SDDMM
# ------------------------------------------------------------------------------------------------
def _normalize_sddmm(crow, col, query, key):
    if crow.dtype not in (torch.int32, torch.int64) or col.dtype not in (torch.int32, torch.int64):
        raise TypeError("crow and col must use integer indices")
    crow, col = crow.to(torch.long).contiguous(), col.to(torch.long).contiguous()
    query, key = query.contiguous(), key.contiguous()
    if query.ndim != 2 or query.shape != key.shape:
        raise ValueError("query and key must have the same [N, F] shape")
    if not query.is_floating_point() or query.dtype != key.dtype:
        raise TypeError("query and key must use the same floating-point dtype")
    if crow.ndim != 1 or col.ndim != 1:
        raise ValueError("crow and col must be one-dimensional")
    if crow.numel() != query.size(0) + 1:
        raise ValueError("crow must contain N + 1 entries")
    if not (crow.device == col.device == query.device == key.device):
        raise ValueError("all SDDMM inputs must be on the same device")
    return crow, col, query, key


def _warp_threshold_pairs(crow, width, config) -> list[tuple[int, int]]:
    return list(dict.fromkeys((w, h) for _, w, h in _spmm_candidates(crow, width, config)))


def sddmm_csr_auto(crow, col, query, key, *, guardrail: float = 0.95, seed: int = 0,
                   verbose: bool = False) -> tuple[torch.Tensor, dict[str, Any]]:
    crow, col, query, key = _normalize_sddmm(crow, col, query, key)
    if not query.is_cuda:
        run, name = _prepare_sddmm_baseline(crow, col, query, key)
        return run(), {**_cpu_info("sddmm"), "baseline": name}
    if query.dtype != torch.float32:
        run, name = _prepare_sddmm_baseline(crow, col, query, key)
        return run(), {**_cpu_info("sddmm"), "baseline": name,
                       "reason": "AutoSAGE CUDA kernels require float32 features"}

    load_native()
    config = SchedulerConfig.from_env(guardrail=guardrail, candidate_count=6)
    device = device_signature()
    graph = _SIGNATURES.signature(crow, col, query.size(1), "sddmm", False, query.dtype)
    cache = ScheduleCache()

    hit = _lookup(cache, config, device, graph, "sddmm_csr")
    if hit is not None:
        output = _run_sddmm_choice(hit.get("choice", "baseline"), hit.get("candidate"), crow, col, query, key)
        return output, {**hit, "from_cache": True}
    if config.replay_only:
        return _run_sddmm_choice("baseline", None, crow, col, query, key), _replay_miss("sddmm", "gather-dot")

    sample, t0 = _timed_sample(crow, col, None, config, seed)
    s_crow, s_col = sample.crow, sample.col
    s_query, s_key = sample.row_side(query), sample.column_side(key)
    if sample.induced:
        torch.cuda.synchronize()
    sample_ms = (time.perf_counter() - t0) * 1000.0

    def make_baseline():
        e_crow, e_col, _ = sample.exact()
        return _prepare_sddmm_baseline(e_crow, e_col, sample.exact_rows(s_query), s_key)

    split = native_op("sddmm_csr_split") if config.hub_split else None
    core = native_op("sddmm_csr")
    runs: list[tuple[list[int], Callable[[], torch.Tensor]]] = []
    if split is not None:
        forced = config.warps_per_block is not None or config.hub_threshold is not None
        pairs = _with_library_default(_warp_threshold_pairs(crow, query.size(1), config),
                                      (SDDMM_WARPS, SDDMM_HUB_THRESHOLD), forced)
        for warps, threshold in pairs:
            runs.append(([warps, threshold],
                         lambda w=warps, h=sample.threshold(threshold): _probe_sddmm(s_crow, s_col, s_query, s_key, w, h)))
    result = _probe_and_choose(
        operation="sddmm", label="sddmm", config=config, device=device, graph=graph, cache=cache,
        sample_ms=sample_ms, sample=sample, make_baseline=make_baseline, candidates=runs,
        fallback=(lambda: _probe_sddmm(s_crow, s_col, s_query, s_key, SDDMM_WARPS, SDDMM_HUB_THRESHOLD))
        if core is not None else None, verbose=verbose, preferred=(SDDMM_WARPS, SDDMM_HUB_THRESHOLD))
    output = _run_sddmm_choice(result["choice"], result["candidate"] if result["choice"] == "autosage" else None,
                               crow, col, query, key)
    return output, result


# ------------------------------------------------------------------------------------------------
# softmax and attention
# ------------------------------------------------------------------------------------------------
def _csr_row_softmax(crow: torch.Tensor, scores: torch.Tensor) -> torch.Tensor:
    """Softmax over each CSR row segment of ``scores``.  float32 CUDA inputs run the segmented
    kernel; everything else runs the reference's scatter formulation (``_auto.py:744-759``)."""
    if scores.numel() == 0:
        return scores.clone()
    differentiating = torch.is_grad_enabled() and scores.requires_grad  # the kernel has no backward
    if (scores.is_cuda and scores.dtype == torch.float32 and crow.dtype == torch.long and not differentiating
            and load_native()):
        crow = crow.contiguous()
        scores = scores.contiguous()
        probs = torch.empty_like(scores)
        workspace, ready = _native.planned_workspace(crow, DEFAULT_HUB_THRESHOLD)
        _native.row_softmax(crow, scores, probs, warps=DEFAULT_WARPS, threshold=DEFAULT_HUB_THRESHOLD,
                            flags=ready, workspace=workspace)
        return probs
    rows = _row_ids(crow)
    peak = torch.full((crow.numel() - 1,), -torch.inf, dtype=scores.dtype, device=scores.device)
    peak.scatter_reduce_(0, rows, scores, reduce="amax", include_self=True)
    shifted = (scores - peak.index_select(0, rows)).exp()
    total = torch.zeros_like(peak).scatter_add_(0, rows, shifted)
    return shifted / total.index_select(0, rows)


def _fused_attention_enabled() -> bool:
    return os.getenv("AUTOSAGE_FUSED_ATTENTION", "1").strip().lower() not in {"0", "false", "no", "off"}


def _attention_unfused(crow, col, query, key, value, scale, guardrail, seed, verbose):
    scaled_query = query if scale is None else query * scale
    scores, sddmm_info = sddmm_csr_auto(crow, col, scaled_query, key, guardrail=guardrail, seed=seed, verbose=verbose)
    probabilities = _csr_row_softmax(crow.to(torch.long), scores.to(query.dtype))
    output, spmm_info = spmm_csr_auto(crow, col, probabilities, value, guardrail=guardrail, seed=seed, verbose=verbose)
    return output, {"sddmm": sddmm_info, "spmm": spmm_info}


def _fused_attention_kernel(crow, col, query, key, value, scale, warps, threshold) -> torch.Tensor:
    out = torch.empty_like(query)  # one output row per CSR row (the probe's row sample is k x N)
    if out.numel() == 0:
        return out
    workspace, ready = _native.planned_workspace(crow, threshold, _native.attention_extra_bytes(crow.numel() - 1))
    _native.attention(crow, col, query, key, value, out, scale=1.0 if scale is None else float(scale),
                      warps=warps, threshold=threshold, flags=_base_flags() | ready, workspace=workspace)
    return out


class _FusedAttention(torch.autograd.Function):
    """The fused kernel with a backward pass.  Forward: one pass, nothing per edge kept.  Backward
    recomputes the probabilities with the library's own kernels instead of storing them:
        S = scale * SDDMM(Q, K),  P = row_softmax(S),  DP = SDDMM(dOut, V),  D_r = <dOut_r, Out_r>
        dS = P * (DP - D[row]) * scale
        dQ = A(dS) K,   dK = A(dS)^T Q,   dV = A(P)^T dOut
    (A(w) = the CSR pattern with edge weights w; the transposed products run over the memoised transposed
    pattern, as the operators' own gradients do.)  The reference registers no gradient at all
    (csrc/spmm_binding.cpp:72-75); its Python pipeline is differentiable only through torch's ops."""

    @staticmethod
    def forward(ctx, crow, col, query, key, value, scale, warps, threshold):
        out = _fused_attention_kernel(crow, col, query, key, value, scale, warps, threshold)
        ctx.save_for_backward(crow, col, query, key, value, out)
        ctx.scale = 1.0 if scale is None else float(scale)
        return out

    @staticmethod
    @torch.no_grad()
    def backward(ctx, grad_out):
        from .ops import _transposed_pattern

        crow, col, query, key, value, out = ctx.saved_tensors
        grad_out = grad_out.contiguous()
        scale = ctx.scale
        ops = torch.ops.autosage
        scores = ops.sddmm_csr(crow, col, query * scale if scale != 1.0 else query, key)
        probs = _csr_row_softmax(crow, scores)
        rows = _row_ids(crow)
        row_dot = (grad_out * out).sum(dim=1)
        grad_scores = probs * (ops.sddmm_csr(crow, col, grad_out, value) - row_dot.index_select(0, rows)) * scale
        grad_q = grad_k = grad_v = None
        need_q, need_k, need_v = ctx.needs_input_grad[2:5]
        if need_q:
            grad_q = ops.spmm_csr(crow, col, grad_scores, key)
        if need_k or need_v:
            crow_t, col_t, perm = _transposed_pattern(crow, col)
            if need_k:
                grad_k = ops.spmm_csr(crow_t, col_t, grad_scores[perm].contiguous(), query)
            if need_v:
                grad_v = ops.spmm_csr(crow_t, col_t, probs[perm].contiguous(), grad_out)
        return None, None, grad_q, grad_k, grad_v, None, None, None


def _run_fused_attention(crow, col, query, key, value, scale, warps, threshold) -> torch.Tensor:
    if torch.is_grad_enabled() and (query.requires_grad or key.requires_grad or value.requires_grad):
        return _FusedAttention.apply(crow, col, query, key, value, scale, warps, threshold)
    return _fused_attention_kernel(crow, col, query, key, value, scale, warps, threshold)


def csr_attention_forward(crow, col, query, key, value, *, guardrail: float = 0.95, seed: int = 0,
                          verbose: bool = False, scale: Optional[float] = None,
                          fused: Optional[bool] = None) -> tuple[torch.Tensor, dict[str, Any]]:
    """softmax_row(scale * Q K^T on the CSR pattern) V.

    ``scale=None`` is the reference behaviour (no scaling, ``_auto.py:762-780``).  On float32 CUDA
    inputs with at most 512 features the one-pass fused kernel is scheduled like the other
    operators (probe on the sample against the three-pass pipeline, guardrail, cache under
    operation "attention"); ``fused=False`` or AUTOSAGE_FUSED_ATTENTION=0 forces the reference's
    three-pass composition.  The fused kernel is differentiable in query, key and value (its backward
    recomputes the probabilities, see ``_FusedAttention``).  The info dict keeps the reference's two
    keys and adds "attention".
    """
    use_fused = _fused_attention_enabled() if fused is None else bool(fused)
    eligible = (query.is_cuda and query.dtype == torch.float32 and key.dtype == torch.float32
                and value.dtype == torch.float32 and query.ndim == 2 and query.shape == key.shape == value.shape
                and query.size(1) <= 512)
    if not (use_fused and eligible):
        return _attention_unfused(crow, col, query, key, value, scale, guardrail, seed, verbose)

    crow, col, query, key = _normalize_sddmm(crow, col, query, key)
    value = value.contiguous()
    load_native()
    config = SchedulerConfig.from_env(guardrail=guardrail, candidate_count=6)
    device = device_signature()
    graph = _SIGNATURES.signature(crow, col, query.size(1), "attention", False, query.dtype)
    cache = ScheduleCache()

    def finish(result: dict[str, Any], from_cache: bool):
        if result.get("choice") == "autosage" and result.get("candidate") is not None:
            warps, threshold = (int(c) for c in result["candidate"])
            output = _run_fused_attention(crow, col, query, key, value, scale, warps, threshold)
            info = {**result, "from_cache": from_cache}
            stage = {"operation": None, "schema_version": AUTOTUNE_SCHEMA_VERSION, "choice": "autosage",
                     "candidate": result["candidate"], "fused": True, "from_cache": from_cache}
            return output, {"sddmm": {**stage, "operation": "sddmm"}, "spmm": {**stage, "operation": "spmm"},
                            "attention": info}
        output, infos = _attention_unfused(crow, col, query, key, value, scale, guardrail, seed, verbose)
        return output, {**infos, "attention": {**result, "from_cache": from_cache}}

    hit = None
    if config.cache:
        record = cache.lookup(device, graph)
        if record is not None and _cache_hit_allowed(record.get("result", {}), config):
            hit = record["result"]
    if hit is not None:
        return finish(hit, True)
    if config.replay_only:
        return finish(_replay_miss("attention", "sddmm+softmax+spmm"), False)

    sample, t0 = _timed_sample(crow, col, None, config, seed)
    s_crow, s_col = sample.crow, sample.col
    s_q, s_k, s_v = sample.row_side(query), sample.column_side(key), sample.column_side(value)
    if sample.induced:
        torch.cuda.synchronize()
    sample_ms = (time.perf_counter() - t0) * 1000.0

    def make_baseline():
        e_crow, e_col, _ = sample.exact()
        e_q = sample.exact_rows(s_q)

        def three_pass() -> torch.Tensor:
            q = e_q if scale is None else e_q * scale
            scores = _probe_sddmm(e_crow, e_col, q, s_k, SDDMM_WARPS, SDDMM_HUB_THRESHOLD)
            return _probe_spmm(e_crow, e_col, _csr_row_softmax(e_crow, scores), s_v, DEFAULT_TILE, DEFAULT_WARPS,
                               DEFAULT_HUB_THRESHOLD)

        return three_pass, "sddmm+softmax+spmm"

    forced = config.warps_per_block is not None or config.hub_threshold is not None
    pairs = _with_library_default(_warp_threshold_pairs(crow, query.size(1), config), ATTENTION_DEFAULT, forced)
    runs = []
    for warps, threshold in pairs:
        runs.append(([warps, threshold],
                     lambda w=warps, h=sample.threshold(threshold): _run_fused_attention(s_crow, s_col, s_q, s_k, s_v, scale, w, h)))
    result = _probe_and_choose(
        operation="attention", label="attention", config=config, device=device, graph=graph, cache=cache,
        sample_ms=sample_ms, sample=sample, make_baseline=make_baseline, candidates=runs, fallback=None, verbose=verbose,
        preferred=ATTENTION_DEFAULT)
    return finish(result, False)


__all__ = [
    "AUTOTUNE_SCHEMA_VERSION",
    "calibrate_full",
    "csr_attention_forward",
    "sddmm_csr_auto",
    "spmm_csr_auto",
]
