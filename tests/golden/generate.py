"""Regenerates the golden fixtures in this directory by RUNNING THE REFERENCE (AutoSAGE's own
Python package) on small seeded inputs.  Needs the reference checkout; the tests only need the
files this script writes.

    python tests/golden/generate.py [/path/to/AutoSAGE]

Outputs
    reference_vectors.npz   inputs and float64 outputs of the reference's CPU SpMM / SDDMM /
                            row softmax / attention pipeline, and its integer outputs (CSR build,
                            induced sample, row partition inputs)
    reference_keys.json     degree quantiles, shortlists, graph signatures, cache keys, tuning
                            signature and a schedules.json written by the reference's ScheduleCache
"""
from __future__ import annotations

import importlib.util
import json
import os
import sys
import tempfile
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def load_reference(root: str):
    package = Path(root) / "autosage"
    spec = importlib.util.spec_from_file_location("autosage_ref", package / "__init__.py",
                                                  submodule_search_locations=[str(package)])
    module = importlib.util.module_from_spec(spec)
    sys.modules["autosage_ref"] = module
    spec.loader.exec_module(module)
    return module


def random_csr(rows: int, mean_degree: int, seed: int, hub: int = 0):
    gen = torch.Generator().manual_seed(seed)
    counts = torch.randint(0, 2 * mean_degree + 1, (rows,), generator=gen)
    if hub:
        counts[rows // 3] = hub
    crow = torch.cat((torch.zeros(1, dtype=torch.long), counts.cumsum(0)))
    col = torch.randint(0, rows, (int(crow[-1]),), generator=gen)
    return crow, col


def main() -> None:
    if len(sys.argv) < 2:
        raise SystemExit("usage: python tests/golden/generate.py <path of the reference checkout>")
    root = sys.argv[1]
    ref = load_reference(root)
    from autosage_ref import _auto, _cache, config, ops  # type: ignore
    from autosage_ref.utils.csr import edge_index_to_csr  # type: ignore

    arrays: dict[str, np.ndarray] = {}
    keys: dict[str, object] = {"torch": torch.__version__, "cases": {}}

    cases = {
        "tiny": dict(rows=7, mean_degree=2, seed=11, hub=0, features=5),
        "ragged": dict(rows=96, mean_degree=6, seed=12, hub=0, features=33),
        "hub": dict(rows=160, mean_degree=4, seed=13, hub=150, features=64),
        "wide": dict(rows=64, mean_degree=9, seed=14, hub=0, features=132),
    }
    for name, c in cases.items():
        crow, col = random_csr(c["rows"], c["mean_degree"], c["seed"], c["hub"])
        gen = torch.Generator().manual_seed(c["seed"] + 100)
        f = c["features"]
        x = torch.randn(c["rows"], f, generator=gen)
        q = torch.randn(c["rows"], f, generator=gen)
        k = torch.randn(c["rows"], f, generator=gen)
        val = torch.rand(col.numel(), generator=gen) + 0.01
        arrays[f"{name}.crow"], arrays[f"{name}.col"] = crow.numpy(), col.numpy()
        arrays[f"{name}.x"], arrays[f"{name}.q"], arrays[f"{name}.k"] = x.numpy(), q.numpy(), k.numpy()
        arrays[f"{name}.val"] = val.numpy()
        # reference CPU path in float64 (autosage.spmm_csr accepts any float dtype on CPU)
        arrays[f"{name}.spmm_weighted"] = ref.spmm_csr(crow, col, val.double(), x.double()).numpy()
        arrays[f"{name}.spmm_unweighted"] = ref.spmm_csr(crow, col, None, x.double()).numpy()
        arrays[f"{name}.spmm_weighted_f32"] = ref.spmm_csr(crow, col, val, x).numpy()
        scores, _ = ref.sddmm_csr_auto(crow, col, q.double(), k.double())
        arrays[f"{name}.sddmm"] = scores.numpy()
        arrays[f"{name}.softmax"] = _auto._csr_row_softmax(crow, scores).numpy()
        out, _ = ref.csr_attention_forward(crow, col, q.double(), k.double(), x.double())
        arrays[f"{name}.attention"] = out.numpy()
        # integer outputs
        s_crow, s_col, s_val, selected = _auto._induced_sample_csr(
            crow, col, val, fraction=0.5, minimum_rows=4, seed=3)
        arrays[f"{name}.sample_crow"], arrays[f"{name}.sample_col"] = s_crow.numpy(), s_col.numpy()
        arrays[f"{name}.sample_val"], arrays[f"{name}.sample_rows"] = s_val.numpy(), selected.numpy()
        cfg = config.SchedulerConfig(candidate_count=18)
        keys["cases"][name] = {
            "degree_quantiles": list(_auto._degree_quantiles(crow)),
            "candidates_k18": [list(t) for t in _auto._spmm_candidates(crow, f, cfg)],
            "candidates_default": [list(t) for t in _auto._spmm_candidates(crow, f, config.SchedulerConfig())],
            "graph_signature": _cache.graph_signature(crow, col, f, "spmm", weighted=True, dtype=torch.float32),
            "graph_signature_sddmm": _cache.graph_signature(crow, col, f, "sddmm", dtype=torch.float32),
        }

    # structure hash over more than 2048 entries (head + tail windows)
    crow, col = random_csr(3000, 3, 21)
    arrays["long.crow"], arrays["long.col"] = crow.numpy(), col.numpy()
    keys["cases"]["long"] = {
        "graph_signature": _cache.graph_signature(crow, col, 128, "spmm", weighted=False, dtype=torch.float32),
        "degree_quantiles": list(_auto._degree_quantiles(crow)),
        "candidates_default": [list(t) for t in _auto._spmm_candidates(crow, 128, config.SchedulerConfig())],
    }

    # COO -> CSR with repeated destinations and an isolated node
    gen = torch.Generator().manual_seed(5)
    edge_index = torch.randint(0, 40, (2, 300), generator=gen)
    edge_index[1][edge_index[1] == 17] = 18  # node 17 receives nothing
    crow, col = edge_index_to_csr(edge_index, 40)
    arrays["coo.edge_index"], arrays["coo.crow"], arrays["coo.col"] = edge_index.numpy(), crow.numpy(), col.numpy()
    crow_s, col_s = edge_index_to_csr(edge_index, 40, rows_by="src")
    arrays["coo.crow_src"], arrays["coo.col_src"] = crow_s.numpy(), col_s.numpy()
    arrays["coo.weight_order"] = edge_index[1].argsort(stable=True).numpy()

    # cache keys and a cache file written by the reference
    device = {"type": "cuda", "name": "NVIDIA B200", "compute_capability": [10, 0], "multiprocessors": 148,
              "total_memory": 191_000_000_000, "cuda": "12.8", "torch": "2.11.0+cu128"}
    graph = keys["cases"]["hub"]["graph_signature"]
    keys["cache_key"] = _cache.ScheduleCache._key(device, graph)
    keys["device"] = device
    keys["tuning_signature"] = config.SchedulerConfig.from_env().tuning_signature()
    result = {"operation": "spmm", "schema_version": 3, "choice": "autosage", "candidate": [128, 8, 37],
              "baseline": "torch.sparse.mm(csr)", "guardrail": 0.95,
              "configuration": keys["tuning_signature"], "from_cache": False}
    with tempfile.TemporaryDirectory() as folder:
        os.environ["AUTOSAGE_CACHE_DIR"] = folder
        _cache.ScheduleCache().store(device, graph, result)
        text = (Path(folder) / "schedules.json").read_text(encoding="utf-8")
    payload = json.loads(text)
    for record in payload["records"].values():
        record["timestamp"] = 0  # the only non-deterministic field
    keys["stored_result"] = result
    (HERE / "reference_schedules.json").write_text(json.dumps(payload, indent=2, sort_keys=True) + "\n",
                                                   encoding="utf-8")
    np.savez_compressed(HERE / "reference_vectors.npz", **arrays)
    (HERE / "reference_keys.json").write_text(json.dumps(keys, indent=2, sort_keys=True) + "\n", encoding="utf-8")
    print(f"wrote {len(arrays)} arrays")


if __name__ == "__main__":
    main()
