"""Drop-in alias: ``import autosage`` resolves to the B200 implementation in ``autosage_b200``.

Programs written against the reference package (``from autosage import spmm_csr_auto``,
``from autosage._auto import _spmm_candidates``, ``from autosage.utils.csr import
edge_index_to_csr`` ...) run unchanged; every submodule name maps to the module of the same name in
``autosage_b200``.
"""
import importlib
import sys

import autosage_b200 as _impl

for _name in ("_auto", "_cache", "_version", "config", "conv", "ops", "utils", "utils.csr"):
    sys.modules[f"{__name__}.{_name}"] = importlib.import_module(f"autosage_b200.{_name}")

from autosage_b200 import *  # noqa: E402,F401,F403
from autosage_b200 import __all__, __version__  # noqa: E402,F401

_auto = sys.modules[f"{__name__}._auto"]
_cache = sys.modules[f"{__name__}._cache"]
config = sys.modules[f"{__name__}.config"]
conv = sys.modules[f"{__name__}.conv"]
ops = sys.modules[f"{__name__}.ops"]
utils = sys.modules[f"{__name__}.utils"]
