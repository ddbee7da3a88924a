"""Shared builders for the parity tests (inputs are seeded, generated on the CPU)."""
from __future__ import annotations

import numpy as np
import torch


def csr_from_counts(counts, n_cols: int, seed: int):
    counts = torch.as_tensor(counts, dtype=torch.long)
    crow = torch.zeros(counts.numel() + 1, dtype=torch.long)
    torch.cumsum(counts, 0, out=crow[1:])
    gen = torch.Generator().manual_seed(seed)
    col = torch.randint(0, max(n_cols, 1), (int(crow[-1]),), generator=gen, dtype=torch.long)
    return crow, col


def random_csr(rows: int, mean_degree: int, seed: int, hubs: dict | None = None):
    """Degrees uniform in [0, 2*mean] (so empty rows and duplicate columns occur), optional hubs."""
    gen = torch.Generator().manual_seed(seed)
    counts = torch.randint(0, 2 * mean_degree + 1, (rows,), generator=gen)
    for row, degree in (hubs or {}).items():
        counts[row] = degree
    return csr_from_counts(counts, rows, seed + 1)


def dense(rows: int, features: int, seed: int) -> torch.Tensor:
    gen = torch.Generator().manual_seed(seed)
    return torch.randn(rows, features, generator=gen, dtype=torch.float32)


def weights(nnz: int, seed: int) -> torch.Tensor:
    gen = torch.Generator().manual_seed(seed)
    return 1.0 - torch.rand(nnz, generator=gen, dtype=torch.float32)


def misaligned_copy(t: torch.Tensor, offset_elements: int = 1) -> torch.Tensor:
    """A contiguous copy of ``t`` whose storage starts ``offset_elements`` items after an aligned
    allocation (4 bytes for float32), to exercise the unaligned kernels."""
    flat = torch.empty(t.numel() + offset_elements, dtype=t.dtype, device=t.device)
    view = flat[offset_elements:].view(t.shape)
    view.copy_(t)
    return view


def to_np(t):
    return None if t is None else t.detach().cpu().numpy()
