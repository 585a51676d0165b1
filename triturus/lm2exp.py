"""`from triturus.lm2exp import lm2exp` -> triturus_b200.lm2exp.lm2exp (replaces triturus/lm2exp.py:167)."""

from triturus_b200.lm2exp import lm2exp

__all__ = ["lm2exp"]
