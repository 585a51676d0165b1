"""Load the reference's own `triturus` package (baseline/_ref, see install_reference.py) inside a process that
also uses this repository's drop-in package of the same name.

The reference's modules import each other by absolute name (`from triturus.utils import ...`,
triturus/lm2exp.py:5), so they are imported with baseline/_ref first on sys.path while any already imported
`triturus*` modules are set aside, and sys.modules is put back afterwards.  The returned module objects keep
working: their functions resolve globals through their own module dictionaries.

Only tests and bench.py use this; nothing in the product package does.
"""

from __future__ import annotations

import importlib
import sys
from pathlib import Path
from types import SimpleNamespace

REF_DIR = Path(__file__).resolve().parent / "_ref"
SUITE_DIR = REF_DIR / "suite"


def available() -> str | None:
    """None when the reference and Triton can be used here, else the reason as one line."""
    if not (REF_DIR / "triturus" / "lm2exp.py").exists():
        return "baseline/_ref holds no copy of the reference (run baseline/install_reference.py)"
    try:
        import triton  # noqa: F401
    except Exception as exc:  # noqa: BLE001
        return f"triton cannot be imported: {exc}"
    return None


_CACHE: SimpleNamespace | None = None


def load() -> SimpleNamespace:
    """Namespace with the reference's `lm2exp`, `lt2exp`, `set_tf32_enabled`, its torch baselines
    (`torch_lm2exp`, `torch_lt2exp`) and the module objects themselves."""
    global _CACHE
    if _CACHE is not None:
        return _CACHE
    why = available()
    if why is not None:
        raise RuntimeError(why)
    saved = {k: v for k, v in sys.modules.items() if k == "triturus" or k.startswith("triturus.")
             or k == "baselines" or k.startswith("baselines.")}  # fmt: skip
    for k in saved:
        del sys.modules[k]
    paths = [str(REF_DIR), str(SUITE_DIR)]
    sys.path[:0] = paths
    try:
        lm = importlib.import_module("triturus.lm2exp")
        lt = importlib.import_module("triturus.lt2exp")
        ut = importlib.import_module("triturus.utils")
        bl_lm = importlib.import_module("baselines.lm2exp") if (SUITE_DIR / "baselines").exists() else None
        bl_lt = importlib.import_module("baselines.lt2exp") if (SUITE_DIR / "baselines").exists() else None
        if not Path(lm.__file__).resolve().is_relative_to(REF_DIR):
            raise RuntimeError(f"imported {lm.__file__} instead of the reference under {REF_DIR}")
    finally:
        for p in paths:
            sys.path.remove(p)
        for k in [k for k in sys.modules if k == "triturus" or k.startswith("triturus.")
                  or k == "baselines" or k.startswith("baselines.")]:  # fmt: skip
            del sys.modules[k]
        sys.modules.update(saved)
    _CACHE = SimpleNamespace(
        lm2exp=lm.lm2exp, lt2exp=lt.lt2exp, set_tf32_enabled=ut.set_tf32_enabled, utils=ut, lm2exp_module=lm,
        lt2exp_module=lt, torch_lm2exp=getattr(bl_lm, "lm2exp", None), torch_lt2exp=getattr(bl_lt, "lt2exp", None),
    )  # fmt: skip
    return _CACHE
