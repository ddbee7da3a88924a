"""Seeded synthetic CSR graphs with the shapes of the graphs AutoSAGE was measured on.

The reference benchmarks on Reddit (PyG) and ogbn-products (OGB) plus two synthetic generators
(``scripts/benchmark.py:79-141``).  The datasets cannot be downloaded where this runs, so the
benchmark configurations are power-law stand-ins with the same row count, nnz and maximum degree:

    degrees   inverse-CDF samples of p(d) ~ d^-alpha truncated to [d_min, d_max]; d_min is found by
              bisection so that sum(degrees) lands within 0.5 % of the target nnz; the largest
              degree is forced to d_max
    columns   iid uniform in [0, N) (duplicates allowed), sorted inside each row
    values    1 - U[0, 1)  in (0, 1]
    dense     N(0, 1) float32 from a CPU generator (so CPU oracle and GPU see the same bits)

Rows are not sorted by degree: hubs are scattered over the row range.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


@dataclass(frozen=True)
class GraphSpec:
    name: str
    rows: int
    target_nnz: int
    alpha: float
    max_degree: int


# the benchmark graphs: stand-ins for Reddit, ogbn-arxiv and ogbn-products
REDDIT_LIKE = GraphSpec("powerlaw-232965", 232_965, 114_615_892, 2.1, 21_657)
ARXIV_LIKE = GraphSpec("powerlaw-169343", 169_343, 2_480_000, 2.2, 13_000)
PRODUCTS_LIKE = GraphSpec("powerlaw-2449029", 2_449_029, 123_718_280, 2.0, 17_500)


def _powerlaw_degrees(rows: int, alpha: float, d_min: float, d_max: int, uniform: torch.Tensor) -> torch.Tensor:
    a = 1.0 - alpha
    lo, hi = float(d_min) ** a, float(d_max) ** a
    degree = ((hi - lo) * uniform + lo).pow(1.0 / a).floor().clamp_(1, d_max).to(torch.long)
    degree[int(torch.argmax(degree))] = d_max
    return degree


def powerlaw_degrees(rows: int, target_nnz: int, alpha: float, max_degree: int, seed: int = 0) -> tuple[torch.Tensor, float]:
    """Row degrees (int64, CPU) and the d_min the bisection settled on."""
    gen = torch.Generator().manual_seed(seed)
    uniform = torch.rand(rows, generator=gen, dtype=torch.float64)
    lo, hi = 1.0, float(max_degree)
    degree = _powerlaw_degrees(rows, alpha, lo, max_degree, uniform)
    if int(degree.sum()) >= target_nnz:
        return degree, lo
    for _ in range(60):
        mid = 0.5 * (lo + hi)
        degree = _powerlaw_degrees(rows, alpha, mid, max_degree, uniform)
        total = int(degree.sum())
        if abs(total - target_nnz) <= 0.005 * target_nnz:
            return degree, mid
        if total < target_nnz:
            lo = mid
        else:
            hi = mid
    return degree, 0.5 * (lo + hi)


def csr_from_degrees(degree: torch.Tensor, num_cols: int, seed: int = 0, sort_columns: bool = True,
                     device: Optional[torch.device] = None) -> tuple[torch.Tensor, torch.Tensor]:
    """crow, col (int64) with iid uniform columns; generated on ``device`` when given (the column
    stream then comes from that device's generator), else on the CPU."""
    device = torch.device("cpu") if device is None else torch.device(device)
    degree = degree.to(device)
    crow = torch.zeros(degree.numel() + 1, dtype=torch.long, device=device)
    torch.cumsum(degree, 0, out=crow[1:])
    nnz = int(crow[-1])
    gen = torch.Generator(device=device).manual_seed(seed + 1)
    col = torch.randint(0, num_cols, (nnz,), generator=gen, device=device, dtype=torch.long)
    if sort_columns and nnz:
        # sort inside rows: one global sort of (row, col) packed into a single key
        rows = torch.repeat_interleave(torch.arange(degree.numel(), device=device), degree)
        key = rows * num_cols + col
        del rows
        col = key.sort().values % num_cols
    return crow, col


def powerlaw_csr(spec: GraphSpec, seed: int = 0, device: Optional[torch.device] = None, scale: float = 1.0):
    """CSR of ``spec`` (optionally shrunk: rows, nnz and max degree times ``scale``)."""
    rows = max(8, int(spec.rows * scale))
    target = max(rows, int(spec.target_nnz * scale))
    dmax = max(4, min(int(spec.max_degree * max(scale, 0.0) ** 0.5) if scale < 1.0 else spec.max_degree, rows))
    degree, d_min = powerlaw_degrees(rows, target, spec.alpha, dmax, seed)
    crow, col = csr_from_degrees(degree, rows, seed, device=device)
    return crow, col, {"rows": rows, "nnz": int(col.numel()), "d_min": d_min, "max_degree": int(degree.max())}


def uniform_degree_csr(rows: int, max_degree: int = 32, seed: int = 0) -> tuple[torch.Tensor, torch.Tensor]:
    """The small CPU-runnable benchmark graph: degree uniform in [1, max_degree], distinct uniform columns."""
    gen = torch.Generator().manual_seed(seed)
    degree = torch.randint(1, max_degree + 1, (rows,), generator=gen)
    crow = torch.zeros(rows + 1, dtype=torch.long)
    torch.cumsum(degree, 0, out=crow[1:])
    cols = [torch.randperm(rows, generator=gen)[: int(d)].sort().values for d in degree.tolist()]
    return crow, torch.cat(cols)


def edge_values(nnz: int, seed: int = 0, device: Optional[torch.device] = None) -> torch.Tensor:
    """float32 weights in (0, 1]."""
    device = torch.device("cpu") if device is None else torch.device(device)
    gen = torch.Generator(device=device).manual_seed(seed + 7)
    return 1.0 - torch.rand(nnz, generator=gen, device=device, dtype=torch.float32)


def dense(rows: int, features: int, seed: int, device: Optional[torch.device] = None) -> torch.Tensor:
    """N(0, 1) float32 matrix; generated on the CPU generator and copied when a device is given."""
    gen = torch.Generator().manual_seed(seed)
    matrix = torch.randn(rows, features, generator=gen, dtype=torch.float32)
    return matrix if device is None else matrix.to(device)
