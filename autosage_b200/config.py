"""Scheduler configuration read from ``AUTOSAGE_*`` environment variables on every call.

Same fields, defaults, validation and ``tuning_signature()`` keys as the reference
``autosage/config.py:25-102`` (the signature is stored in each cached schedule and compared on
lookup, so its keys and value types are part of the on-disk format).
"""
from __future__ import annotations

import os
from dataclasses import dataclass, fields
from typing import Optional

_TRUE = frozenset({"1", "true", "yes", "on"})
_FALSE = frozenset({"0", "false", "no", "off"})

# fields that do not influence which kernel wins and therefore stay out of the tuning signature
_NOT_TUNING = frozenset({"cache", "replay_only"})


def _env_flag(name: str, default: bool) -> bool:
    raw = os.getenv(name)
    if raw is None:
        return default
    token = raw.strip().lower()
    if token in _TRUE:
        return True
    if token in _FALSE:
        return False
    raise ValueError(f"{name} must be a boolean value")


def _env_optional_int(name: str) -> Optional[int]:
    raw = os.getenv(name)
    if raw is None or raw == "":
        return None
    return int(raw)


@dataclass(frozen=True)
class SchedulerConfig:
    guardrail: float = 0.95
    probe_fraction: float = 0.03
    probe_min_rows: int = 512
    probe_iterations: int = 7
    probe_cap_ms: float = 1.0
    minimum_probe_rows: int = 64
    minimum_probe_nonzeros: int = 512
    candidate_count: int = 6
    hub_split: bool = True
    vec4: bool = True
    cache: bool = True
    replay_only: bool = False
    feature_tile: Optional[int] = None
    warps_per_block: Optional[int] = None
    hub_threshold: Optional[int] = None

    def __post_init__(self) -> None:
        if not (0 < self.guardrail <= 1):
            raise ValueError("guardrail must be in (0, 1]")
        if not (0 < self.probe_fraction <= 1):
            raise ValueError("probe_fraction must be in (0, 1]")
        if min(self.probe_min_rows, self.probe_iterations, self.candidate_count) < 1:
            raise ValueError("probe row, iteration, and candidate counts must be positive")
        if self.probe_cap_ms < 0:
            raise ValueError("probe_cap_ms cannot be negative")
        if self.feature_tile is not None and self.feature_tile not in (64, 128):
            raise ValueError("feature_tile must be 64 or 128")
        if self.warps_per_block is not None and self.warps_per_block not in (2, 4, 8):
            raise ValueError("warps_per_block must be 2, 4, or 8")
        if self.hub_threshold is not None and self.hub_threshold < 1:
            raise ValueError("hub_threshold must be positive")

    def tuning_signature(self) -> dict[str, object]:
        return {f.name: getattr(self, f.name) for f in fields(self) if f.name not in _NOT_TUNING}

    @classmethod
    def from_env(cls, *, guardrail: float = 0.95, candidate_count: int = 6) -> "SchedulerConfig":
        env = os.getenv
        return cls(
            guardrail=float(guardrail),
            candidate_count=int(candidate_count),
            probe_fraction=float(env("AUTOSAGE_PROBE_FRAC", "0.03")),
            probe_min_rows=int(env("AUTOSAGE_PROBE_MIN_ROWS", "512")),
            probe_iterations=int(env("AUTOSAGE_PROBE_ITERS", "7")),
            probe_cap_ms=float(env("AUTOSAGE_PROBE_CAP_MS", "1.0")),
            minimum_probe_rows=int(env("AUTOSAGE_MIN_PROBE_ROWS", "64")),
            minimum_probe_nonzeros=int(env("AUTOSAGE_MIN_PROBE_NNZ", "512")),
            hub_split=_env_flag("AUTOSAGE_HUB_CTA", True),
            vec4=_env_flag("AUTOSAGE_VEC4", True),
            cache=_env_flag("AUTOSAGE_CACHE", True),
            replay_only=_env_flag("AUTOSAGE_REPLAY_ONLY", False),
            feature_tile=_env_optional_int("AUTOSAGE_FTILE"),
            warps_per_block=_env_optional_int("AUTOSAGE_WPB"),
            hub_threshold=_env_optional_int("AUTOSAGE_HUB_T"),
        )
