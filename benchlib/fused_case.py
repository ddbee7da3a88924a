"""The layer's two forms side by side: `python -m benchlib.fused_case [--scale S] [--hub-threshold T]`.

Builds the 2.45 M-row power-law benchmark graph (or a fraction `--scale` of it), runs the layer
forward (F = 128 -> 256, unweighted) as (a) the SpMM kernels followed by the tcgen05 Linear and (b) the
fused aggregation + Linear kernel, checks (b) against (a) and prints one JSON line with both times.
--only-fused leaves (a) out, which is what a profiler capture of the fused kernel wants."""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import torch  # noqa: E402


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--scale", type=float, default=1.0)
    parser.add_argument("--hub-threshold", type=int, nargs="+", default=[64])
    parser.add_argument("--hub-warps", type=int, default=4)
    parser.add_argument("--calls", type=int, default=5)
    parser.add_argument("--only-fused", action="store_true")
    args = parser.parse_args()
    import autosage_b200
    from autosage_b200 import _native
    from benchlib import synthetic as syn

    if not autosage_b200.load_native():
        raise RuntimeError(f"libautosage_b200.so failed to load: {autosage_b200.ops.native_load_error()}")
    device = torch.device("cuda", 0)
    crow, col, info = syn.powerlaw_csr(syn.PRODUCTS_LIKE, seed=0, device=device, scale=args.scale)
    n = info["rows"]
    x = syn.dense(n, 128, 3, device)
    torch.manual_seed(0)
    linear = torch.nn.Linear(128, 256).to(device)
    weight, bias = linear.weight.detach().contiguous(), linear.bias.detach().contiguous()

    def timed(function) -> float:
        for _ in range(2):
            function()
        torch.cuda.synchronize()
        times = []
        for _ in range(args.calls):
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            function()
            end.record()
            end.synchronize()
            times.append(begin.elapsed_time(end))
        return round(sorted(times)[len(times) // 2], 4)

    line = {"rows": n, "nnz": info["nnz"], "in_features": 128, "out_features": 256}
    reference = None
    if not args.only_fused:
        reference = torch.empty(n, 256, device=device)

        def two_kernels() -> None:
            aggregated = torch.ops.autosage.spmm_csr_split(crow, col, None, x, 128, 4, 1024)
            _native.linear_bias_umma(aggregated, weight, bias, reference)

        line["spmm_then_linear_ms"] = timed(two_kernels)
    out = torch.empty(n, 256, device=device)
    line["fused"] = []
    for threshold in args.hub_threshold:
        workspace = _native.conv_fused(crow, col, None, x, weight, bias, out, hub_threshold=threshold,
                                       hub_warps=args.hub_warps)
        entry = {"hub_threshold": threshold,
                 "ms": timed(lambda: _native.conv_fused(crow, col, None, x, weight, bias, out, hub_threshold=threshold,
                                                        hub_warps=args.hub_warps, workspace=workspace)),
                 "status": _native.workspace_status(workspace)}
        if reference is not None:
            entry["max_abs_difference"] = float((out - reference).abs().max())
        line["fused"].append(entry)
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
