"""Schedule cache on disk, cache keys and the probe log.

File format, key construction and hashing are those of the reference ``autosage/_cache.py``
(cache_directory :17-21, device_signature :24-37, _sample_hash :40-54, graph_signature :57-93,
ScheduleCache :96-148, log_probe :151-157) so that a ``schedules.json`` written by either
implementation is readable by the other:

    {"schema_version": 1,
     "records": {<key>: {"timestamp": int, "device": {...}, "graph": {...}, "result": {...}}}}

with ``<key>`` the compact, key-sorted JSON of ``{"device": ..., "graph": ...}``.
"""
from __future__ import annotations

import hashlib
import json
import os
import tempfile
import time
from pathlib import Path
from typing import Any, Optional

import torch

CACHE_SCHEMA_VERSION = 1
_HASH_WINDOW = 2048  # entries of crow / col that enter the structure hash (head half + tail half)
_QUANTILE_LIMIT = 16_000_000  # torch.quantile refuses larger inputs


def cache_directory() -> Path:
    override = os.getenv("AUTOSAGE_CACHE_DIR")
    return Path(override).expanduser() if override else Path.home() / ".cache" / "autosage"


def device_signature(device: Optional[int] = None) -> dict[str, Any]:
    if not torch.cuda.is_available():
        return {"type": "cpu", "torch": torch.__version__}
    props = torch.cuda.get_device_properties(torch.cuda.current_device() if device is None else device)
    return {
        "type": "cuda",
        "name": props.name,
        "compute_capability": [props.major, props.minor],
        "multiprocessors": props.multi_processor_count,
        "total_memory": int(props.total_memory),
        "cuda": torch.version.cuda,
        "torch": torch.__version__,
    }


def _structure_hash(crow: torch.Tensor, col: torch.Tensor) -> str:
    """First 24 hex digits of SHA-256 over the raw bytes of the first and last 1024 entries of crow,
    then of col (the whole tensor when it has at most 2048 entries)."""
    digest = hashlib.sha256()
    half = _HASH_WINDOW // 2
    for tensor in (crow, col):
        n = tensor.numel()
        if n == 0:
            continue
        window = tensor if n <= _HASH_WINDOW else torch.cat((tensor[:half], tensor[n - half:]))
        digest.update(window.detach().contiguous().cpu().numpy().tobytes())
    return digest.hexdigest()[:24]


def rounded_quantiles(values: torch.Tensor, points: list[float]) -> list[int]:
    """round(quantile(values, p)) with linear interpolation, as torch.quantile computes it; inputs
    too large for torch.quantile are handled with an explicit sort."""
    data = values.to(torch.float64)
    if data.numel() <= _QUANTILE_LIMIT:
        q = torch.quantile(data, torch.tensor(points, dtype=torch.float64, device=data.device))
    else:
        ordered = data.sort().values
        position = torch.tensor(points, dtype=torch.float64, device=data.device) * (ordered.numel() - 1)
        below = position.floor().to(torch.long)
        above = position.ceil().to(torch.long)
        weight = position - below.to(torch.float64)
        q = torch.lerp(ordered[below], ordered[above], weight)
    return [int(v) for v in q.round().to(torch.long).cpu().tolist()]


def graph_signature(
    crow: torch.Tensor,
    col: torch.Tensor,
    feature_width: int,
    operation: str,
    *,
    weighted: bool = False,
    dtype: Optional[torch.dtype] = None,
) -> dict[str, Any]:
    degrees = crow[1:] - crow[:-1]
    q50, q90, q99 = rounded_quantiles(degrees, [0.5, 0.9, 0.99]) if degrees.numel() else (0, 0, 0)
    return {
        "operation": operation,
        "feature_width": int(feature_width),
        "dtype": str(dtype) if dtype is not None else None,
        "weighted": bool(weighted),
        "rows": int(crow.numel() - 1),
        "nonzeros": int(col.numel()),
        "degree_q50": q50,
        "degree_q90": q90,
        "degree_q99": q99,
        "structure_hash": _structure_hash(crow, col),
    }


# Parsed schedules.json per path, valid while the file's (mtime, size, inode) is unchanged: a replayed
# call then costs one stat() instead of reading and parsing the whole file.
_PARSED: dict[str, tuple[tuple[int, int, int], dict[str, dict[str, Any]]]] = {}


def _file_stamp(path: Path) -> Optional[tuple[int, int, int]]:
    try:
        st = os.stat(path)
    except OSError:
        return None
    return (st.st_mtime_ns, st.st_size, st.st_ino)


class ScheduleCache:
    """JSON file of schedules; every ``store`` rewrites the file through a temporary + rename."""

    def __init__(self, path: Optional[os.PathLike[str] | str] = None):
        self.path = Path(path) if path is not None else cache_directory() / "schedules.json"
        stamp = _file_stamp(self.path)
        memo = _PARSED.get(str(self.path))
        if stamp is not None and memo is not None and memo[0] == stamp:
            self._records = memo[1]
        else:
            self._records = self._read()
            if stamp is not None and stamp == _file_stamp(self.path):
                _PARSED[str(self.path)] = (stamp, self._records)
            else:
                _PARSED.pop(str(self.path), None)

    @staticmethod
    def _key(device: dict[str, Any], graph: dict[str, Any]) -> str:
        return json.dumps({"device": device, "graph": graph}, sort_keys=True, separators=(",", ":"))

    def _read(self) -> dict[str, dict[str, Any]]:
        try:
            payload = json.loads(self.path.read_text(encoding="utf-8"))
        except (OSError, ValueError):
            return {}
        if not isinstance(payload, dict) or payload.get("schema_version") != CACHE_SCHEMA_VERSION:
            return {}
        records = payload.get("records", {})
        return records if isinstance(records, dict) else {}

    def lookup(self, device: dict[str, Any], graph: dict[str, Any]) -> Optional[dict[str, Any]]:
        return self._records.get(self._key(device, graph))

    def store(self, device: dict[str, Any], graph: dict[str, Any], result: dict[str, Any]) -> None:
        self._records[self._key(device, graph)] = {
            "timestamp": int(time.time()),
            "device": device,
            "graph": graph,
            "result": result,
        }
        folder = self.path.parent
        folder.mkdir(parents=True, exist_ok=True)
        fd, scratch = tempfile.mkstemp(prefix="schedules-", suffix=".json", dir=folder)
        try:
            with os.fdopen(fd, "w", encoding="utf-8") as out:
                json.dump({"schema_version": CACHE_SCHEMA_VERSION, "records": self._records}, out,
                          indent=2, sort_keys=True)
                out.write("\n")
            os.replace(scratch, self.path)
            stamp = _file_stamp(self.path)
            if stamp is not None:
                _PARSED[str(self.path)] = (stamp, self._records)
        finally:
            if os.path.exists(scratch):
                os.unlink(scratch)


def log_probe(event: dict[str, Any]) -> None:
    """Append one scheduling decision to probe_logs.jsonl unless AUTOSAGE_LOG_PROBES is not "1"."""
    if os.getenv("AUTOSAGE_LOG_PROBES", "1") != "1":
        return
    target = cache_directory() / "probe_logs.jsonl"
    target.parent.mkdir(parents=True, exist_ok=True)
    with target.open("a", encoding="utf-8") as out:
        out.write(json.dumps(event, sort_keys=True) + "\n")


__all__ = [
    "CACHE_SCHEMA_VERSION",
    "ScheduleCache",
    "cache_directory",
    "device_signature",
    "graph_signature",
    "log_probe",
]
