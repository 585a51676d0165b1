"""Drop-in for triturus/mm.py: `from triturus.mm import mm`."""

from triturus_b200.mm import mm

__all__ = ["mm"]
