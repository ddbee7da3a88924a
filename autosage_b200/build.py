"""Build libautosage_b200.so (CUDA kernels + C ABI) for sm_100a with nvcc, in-tree.

Usage: python -m autosage_b200.build [--force] [--verbose]

The library links the CUDA runtime statically and has no dependency on libtorch, so it can be
loaded by any host program (ctypes, cgo, JNI, ...).  Objects are rebuilt only when a source or
header is newer than the library.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
CSRC = PACKAGE_DIR / "csrc"
INCLUDE = PACKAGE_DIR.parent / "include"
LIB_DIR = PACKAGE_DIR / "lib"
LIB_NAME = "libautosage_b200.so"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-O3",
    "-std=c++17",
    "-lineinfo",
    "-Xcompiler",
    "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    found = shutil.which("nvcc")
    if found:
        return found
    candidate = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda")) / "bin" / "nvcc"
    if candidate.is_file():
        return str(candidate)
    raise RuntimeError("nvcc was not found; it is required to build libautosage_b200.so")


def cutlass_include_dirs() -> list[Path]:
    """The CUTLASS/CuTe header tree (headers only) that asg_linear.cu instantiates its GEMM from.
    Looked up in CUTLASS_INCLUDE_DIR, then in the trees that Python packages of this environment
    vendor (flashinfer, tilelang).  Empty when none has the sm_100 collectives: the library is then
    built without that one kernel (asg_linear_bias reports it; the hand-written tcgen05 Linear and
    everything else do not need CUTLASS)."""
    import importlib.util

    candidates = []
    if os.environ.get("CUTLASS_INCLUDE_DIR"):
        candidates.append(Path(os.environ["CUTLASS_INCLUDE_DIR"]))
    for package, relative in (("flashinfer", "data/cutlass/include"), ("tilelang", "3rdparty/cutlass/include")):
        try:
            spec = importlib.util.find_spec(package)
        except (ImportError, ValueError):
            spec = None
        if spec is not None and spec.submodule_search_locations:
            candidates.append(Path(list(spec.submodule_search_locations)[0]) / relative)
    for candidate in candidates:
        if (candidate / "cutlass" / "gemm" / "collective" / "sm100_mma_warpspecialized_emulated.hpp").is_file():
            return [candidate]
    return []  # asg_linear.cu is then compiled without its CUTLASS kernel (ASG_NO_CUTLASS)


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def library_path() -> Path:
    return LIB_DIR / LIB_NAME


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    stamp = target.stat().st_mtime
    return any(dep.stat().st_mtime > stamp for dep in deps)


def build(force: bool = False, verbose: bool = False, extra_flags: list[str] | None = None,
          output: Path | None = None) -> Path:
    """Compile every .cu under csrc/ and link the shared library. Returns its path."""
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    target = output if output is not None else library_path()
    headers = sorted(CSRC.glob("*.cuh")) + sorted(INCLUDE.glob("*.h"))
    srcs = sources()
    if not force and not extra_flags and not _stale(target, srcs + headers + [Path(__file__)]):
        return target
    nvcc = _nvcc()
    flags = list(NVCC_FLAGS) + [f"-I{INCLUDE}", f"-I{CSRC}"] + list(extra_flags or [])
    cutlass = cutlass_include_dirs()
    flags += [f"-I{d}" for d in cutlass] + ["-diag-suppress", "20012"]
    if not cutlass:
        flags.append("-DASG_NO_CUTLASS")
    if verbose:
        flags += ["-Xptxas", "-v"]
    obj_dir = LIB_DIR / ("obj" if output is None else f"obj_{target.stem}")
    obj_dir.mkdir(parents=True, exist_ok=True)
    procs = []
    objects = []
    for src in srcs:
        obj = obj_dir / (src.stem + ".o")
        objects.append(obj)
        if not force and not extra_flags and not _stale(obj, [src] + headers + [Path(__file__)]):
            continue
        cmd = [nvcc, *flags, "-c", str(src), "-o", str(obj)]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, proc in procs:
        out, _ = proc.communicate()
        if proc.returncode != 0:
            failed = True
            sys.stderr.write(f"[autosage_b200.build] {src.name} failed:\n{out}\n")
        elif verbose and out:
            sys.stderr.write(f"[autosage_b200.build] {src.name}:\n{out}\n")
    if failed:
        raise RuntimeError("nvcc failed to compile libautosage_b200.so")
    link = [nvcc, "-shared", "-o", str(target), *map(str, objects), "-cudart", "static",
            "-Xcompiler", "-fPIC", "-Xlinker", "--exclude-libs,ALL"]
    done = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if done.returncode != 0:
        raise RuntimeError(f"linking {target.name} failed:\n{done.stdout}")
    return target


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
