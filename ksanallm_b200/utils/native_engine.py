"""Loader of the native host runtime (pybind11 module ``_ksana_engine`` built in-tree under ``lib/``)."""
import importlib.util
import sys
from pathlib import Path

_LIB = Path(__file__).resolve().parent.parent / "lib"


def _load():
    cands = sorted(_LIB.glob("_ksana_engine*.so"))
    if not cands:
        raise ImportError(f"native engine module not built under {_LIB}: run `python -m ksanallm_b200.build`")
    spec = importlib.util.spec_from_file_location("_ksana_engine", cands[0])
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    sys.modules["_ksana_engine"] = mod
    return mod


_m = sys.modules.get("_ksana_engine") or _load()
globals().update({k: getattr(_m, k) for k in dir(_m) if not k.startswith("__")})
