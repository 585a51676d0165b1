"""`from triturus.lt2exp import lt2exp` -> triturus_b200.lt2exp.lt2exp (replaces triturus/lt2exp.py:519)."""

from triturus_b200.lt2exp import lt2exp

__all__ = ["lt2exp"]
