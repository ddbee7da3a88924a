"""SpMM on uniform-degree graphs: `python -m benchlib.uniform_case [--degrees 16 48 64 256]`.

Every row has the same number of edges and uniform random columns over a 2,449,029-row X (F = 128,
1.25 GB, ten times L2), so each run isolates one regime of the kernel - short rows, rows with a partly
filled last chunk, long light rows, hub rows - and shows what random 512-byte gathers reach on the memory
system at that row length.  Prints one JSON line per (degree, form) with the time and the model bytes per
second (gathered rows + column indices + output)."""
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
    parser.add_argument("--degrees", type=int, nargs="+", default=[4, 16, 48, 64, 256, 2048])
    parser.add_argument("--columns", type=int, default=2_449_029)
    parser.add_argument("--features", type=int, default=128)
    parser.add_argument("--edges", type=int, default=120_000_000, help="rows = edges / degree, at most --columns")
    args = parser.parse_args()
    import autosage_b200
    from autosage_b200 import _native

    if not autosage_b200.load_native():
        raise RuntimeError(f"libautosage_b200.so failed to load: {autosage_b200.ops.native_load_error()}")
    device = torch.device("cuda", 0)
    x = torch.randn(args.columns, args.features, device=device)

    def timed(function) -> float:
        for _ in range(2):
            function()
        torch.cuda.synchronize()
        times = []
        for _ in range(5):
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            function()
            end.record()
            end.synchronize()
            times.append(begin.elapsed_time(end))
        return sorted(times)[2]

    for degree in args.degrees:
        rows = min(args.columns, max(1, args.edges // degree))
        gen = torch.Generator(device=device)
        gen.manual_seed(degree)
        crow = torch.arange(0, (rows + 1) * degree, degree, device=device, dtype=torch.long)
        col = torch.randint(0, args.columns, (rows * degree,), device=device, generator=gen)
        y = torch.empty(rows, args.features, device=device)
        workspace = torch.empty(_native.workspace_bytes(rows), dtype=torch.uint8, device=device)
        forms = [("warp per row", 1 << 30)] + ([("CTA per row", 1024)] if degree >= 1024 else [])
        for name, threshold in forms:
            ms = timed(lambda: _native.spmm(crow, col, None, x, y, feature_tile=128, warps=4, threshold=threshold,
                                            flags=0, workspace=workspace))
            moved = rows * degree * (4 * args.features + 8) + rows * 4 * args.features
            print(json.dumps({"rows": rows, "degree": degree, "form": name, "ms": round(ms, 3),
                              "model_TBps": round(moved / ms / 1e9, 3)}), flush=True)
        del crow, col, y, workspace


if __name__ == "__main__":
    main()
