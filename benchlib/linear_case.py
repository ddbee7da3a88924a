"""The layer's Linear alone: `python -m benchlib.linear_case [--rows R] [--in-features K] [--out-features N]`.

Builds x (R x K, N(0,1)), a weight (N x K) and a bias, runs the hand-written tcgen05 kernel a few
times, checks it against float64 and times it beside the CUTLASS instantiation and cuBLAS (unless
--only-umma, which is what a profiler capture of this kernel wants: nothing else on the GPU).  Prints
one JSON line."""
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
    parser.add_argument("--rows", type=int, default=600_000)
    parser.add_argument("--in-features", type=int, default=128)
    parser.add_argument("--out-features", type=int, default=256)
    parser.add_argument("--calls", type=int, default=5)
    parser.add_argument("--only-umma", action="store_true")
    args = parser.parse_args()
    import autosage_b200
    from autosage_b200 import _native

    if not autosage_b200.load_native():
        raise RuntimeError(f"libautosage_b200.so failed to load: {autosage_b200.ops.native_load_error()}")
    device = torch.device("cuda", 0)
    gen = torch.Generator().manual_seed(1)
    rows, k, n = args.rows, args.in_features, args.out_features
    x = torch.randn(rows, k, generator=gen).to(device)
    weight = (torch.randn(n, k, generator=gen) / k ** 0.5).to(device)
    bias = torch.randn(n, generator=gen).to(device)
    out = torch.empty(rows, n, device=device)
    workspace = _native.linear_bias_umma(x, weight, bias, out)

    def timed(function) -> float:
        for _ in range(2):
            function()
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for _ in range(args.calls):
            function()
        end.record()
        torch.cuda.synchronize()
        return round(begin.elapsed_time(end) / args.calls, 4)

    line = {"rows": rows, "in_features": k, "out_features": n,
            "umma_ms": timed(lambda: _native.linear_bias_umma(x, weight, bias, out, workspace)),
            "status": _native.workspace_status(workspace)}
    exact = x[:4096].double() @ weight.double().t() + bias.double()
    line["max_error_vs_float64_first_4096_rows"] = float((out[:4096].double() - exact).abs().max())
    if not args.only_umma:
        line["cutlass_ms"] = timed(lambda: _native.linear_bias(x, weight, bias, out))
        line["cublas_sgemm_plus_bias_ms"] = timed(lambda: torch.mm(x, weight.t(), out=out).add_(bias))
        wide = torch.empty(rows, 2 * k, device=device)
        line["stream_copy_same_read_volume_ms"] = timed(lambda: torch.cat([x, x], 1, out=wide))
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
