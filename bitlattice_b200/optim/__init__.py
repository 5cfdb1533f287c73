"""Optimizers updating lattice weights in their storage format."""
from .lattice import DEFAULTS, DIRECTIONS, ROUNDINGS, SCALE_RULES, Lattice, defer_fused_updates
from .presets import PRESETS

__all__ = ["DEFAULTS", "DIRECTIONS", "PRESETS", "ROUNDINGS", "SCALE_RULES", "Lattice", "defer_fused_updates"]
