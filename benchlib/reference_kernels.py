"""The reference's own CUDA kernels as an on-box GPU comparator.

``build()`` compiles the six source files of the reference's extension (``csrc/*.cu``, ``csrc/*.cpp``,
headers under ``include/``) from where they lie in a reference checkout into
``baseline/_ref/libautosage_cuda.so`` with nvcc for sm_100a - the reference's ``CMakeLists.txt`` lists
exactly these files and nothing else, so a direct nvcc line replaces its CMake build.  Nothing of the
reference is copied into this repository; the output folder is git-ignored and travels with the
snapshot to the GPU box.

``python -m benchlib.reference_kernels --workload c2_spmm|c3_sddmm|c5_spmm --features F`` loads that
library (``torch.ops.load_library``, as ``autosage/ops.py:31-61`` does), runs the reference's operators
on the benchmark graph and prints one JSON line with their times.  It must run in a process of its
own: the library registers the same ``torch.ops.autosage`` names as this repository's package.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
OUTPUT = ROOT / "baseline" / "_ref" / "libautosage_cuda.so"
SOURCES = ("spmm_binding.cpp", "spmm_csr_vec4.cu", "launcher_spmm.cu", "spmm_hub.cu", "spmm_rows.cu", "sddmm_csr_op.cu")


def reference_checkout() -> Path:
    """Where the reference's sources are looked for: $AUTOSAGE_REFERENCE_DIR, else a `reference` folder
    beside this repository."""
    return Path(os.environ.get("AUTOSAGE_REFERENCE_DIR", str(ROOT.parent / "reference")))


def build(reference: Path | None = None, force: bool = False) -> Path | None:
    """Returns the library's path, or None when there is neither a reference checkout nor a prebuilt file."""
    reference = reference_checkout() if reference is None else reference
    csrc = reference / "csrc"
    if not csrc.is_dir():
        return OUTPUT if OUTPUT.is_file() else None
    sources = [csrc / name for name in SOURCES]
    if OUTPUT.is_file() and not force and all(OUTPUT.stat().st_mtime >= s.stat().st_mtime for s in sources):
        return OUTPUT
    import torch
    from torch.utils import cpp_extension

    OUTPUT.parent.mkdir(parents=True, exist_ok=True)
    torch_lib = Path(torch.__file__).resolve().parent / "lib"
    flags = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
             "--expt-relaxed-constexpr", "-x", "cu", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
             f"-I{reference / 'include'}"] + [f"-I{path}" for path in cpp_extension.include_paths("cuda")]
    objects, jobs = [], []
    for source in sources:  # one nvcc per file, all at once: the torch headers dominate the compile time
        obj = OUTPUT.parent / (source.stem + ".o")
        objects.append(obj)
        jobs.append((source, subprocess.Popen(["nvcc", *flags, "-c", str(source), "-o", str(obj)], stdout=subprocess.PIPE,
                                              stderr=subprocess.STDOUT, text=True)))
    for source, job in jobs:
        out, _ = job.communicate()
        if job.returncode != 0:
            raise RuntimeError(f"building the reference's CUDA extension failed on {source.name}:\n{out[-4000:]}")
    link = ["nvcc", "-shared", "-o", str(OUTPUT), *map(str, objects), f"-L{torch_lib}", "-lc10", "-lc10_cuda", "-ltorch_cpu",
            "-ltorch_cuda", "-ltorch", "-Xlinker", f"-rpath={torch_lib}"]
    done = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if done.returncode != 0:
        raise RuntimeError(f"linking the reference's CUDA extension failed:\n{done.stdout[-4000:]}")
    for obj in objects:
        obj.unlink(missing_ok=True)
    return OUTPUT


def _time(function, warmup: int = 2, laps: int = 5) -> float:
    import torch

    for _ in range(warmup):
        function()
    torch.cuda.synchronize()
    times = []
    for _ in range(laps):
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        function()
        end.record()
        end.synchronize()
        times.append(begin.elapsed_time(end))
    return min(times)


def run(workload: str, features: int) -> dict:
    import torch

    if "autosage_b200" in sys.modules:
        raise RuntimeError("run the reference's kernels in a process that has not loaded autosage_b200")
    if not OUTPUT.is_file():
        return {"unavailable": "baseline/_ref/libautosage_cuda.so was not built (no reference checkout at build time)"}
    torch.ops.load_library(str(OUTPUT))
    ops = torch.ops.autosage
    from benchlib import synthetic as syn

    device = torch.device("cuda", 0)
    spec = syn.PRODUCTS_LIKE if workload.startswith("c5") else syn.REDDIT_LIKE
    crow, col, info = syn.powerlaw_csr(spec, seed=0, device=device)
    n, nnz = info["rows"], info["nnz"]
    result = {"workload": workload, "rows": n, "nnz": nnz, "features": features,
              "library": "the reference's csrc/*.cu built for sm_100a with nvcc"}
    if workload in ("c2_spmm", "c5_spmm"):
        val = syn.edge_values(nnz, seed=0, device=device) if workload == "c2_spmm" else None
        x = syn.dense(n, features, 3, device)
        result["spmm_csr_ms"] = round(_time(lambda: ops.spmm_csr(crow, col, val, x)), 4)
        degree = (crow[1:] - crow[:-1]).float()
        q95 = max(1, int(torch.quantile(degree[: 1 << 24], 0.95).item()))
        best = None
        for tile, warps, threshold in ((128, 8, q95), (128, 4, q95), (64, 8, q95), (128, 8, 1024), (64, 4, 1024)):
            ms = _time(lambda: ops.spmm_csr_split(crow, col, val, x, tile, warps, threshold), warmup=1, laps=3)
            if best is None or ms < best[0]:
                best = (ms, [tile, warps, threshold])
        result["spmm_csr_split_best_ms"] = round(best[0], 4)
        result["spmm_csr_split_best_candidate"] = best[1]
        weights = val if val is not None else torch.ones(nnz, device=device)
        expected = torch.sparse.mm(torch.sparse_csr_tensor(crow, col, weights, size=(n, n)), x)
        result["max_abs_difference_from_cusparse"] = float((ops.spmm_csr(crow, col, val, x) - expected).abs().max())
    else:
        q, k = syn.dense(n, features, 1, device), syn.dense(n, features, 2, device)
        result["sddmm_csr_ms"] = round(_time(lambda: ops.sddmm_csr(crow, col, q, k)), 4)
        best = None
        for warps, threshold in ((8, 1566), (4, 1566), (8, 8192)):
            ms = _time(lambda: ops.sddmm_csr_split(crow, col, q, k, warps, threshold), warmup=1, laps=3)
            if best is None or ms < best[0]:
                best = (ms, [warps, threshold])
        result["sddmm_csr_split_best_ms"] = round(best[0], 4)
        result["sddmm_csr_split_best_candidate"] = best[1]
    return result


def run_in_subprocess(workload: str, features: int, timeout: float = 300.0) -> dict:
    """What bench.py calls: a child interpreter, so that the two operator libraries never meet."""
    if not OUTPUT.is_file():
        return {"unavailable": "baseline/_ref/libautosage_cuda.so was not built (no reference checkout at build time)"}
    env = dict(os.environ, PYTHONPATH=str(ROOT) + os.pathsep + os.environ.get("PYTHONPATH", ""))
    try:
        done = subprocess.run([sys.executable, "-m", "benchlib.reference_kernels", "--workload", workload, "--features",
                               str(features)], capture_output=True, text=True, timeout=timeout, cwd=str(ROOT), env=env)
    except subprocess.TimeoutExpired:
        return {"unavailable": f"the reference's kernels did not finish {workload} within {timeout:.0f} s"}
    for line in reversed(done.stdout.splitlines()):
        if line.startswith("{"):
            return json.loads(line)
    return {"unavailable": f"the reference's kernels failed on {workload}: {(done.stderr or done.stdout)[-300:]}"}


if __name__ == "__main__":
    parser = argparse.ArgumentParser()
    parser.add_argument("--build", action="store_true")
    parser.add_argument("--workload", default="c2_spmm", choices=["c2_spmm", "c3_sddmm", "c5_spmm"])
    parser.add_argument("--features", type=int, default=128)
    options = parser.parse_args()
    if options.build:
        print(build(force=True))
    else:
        try:
            print(json.dumps(run(options.workload, options.features)), flush=True)
        except Exception as exc:  # noqa: BLE001 - the caller reads one JSON line whatever happens
            print(json.dumps({"unavailable": f"{type(exc).__name__}: {exc}"}), flush=True)
