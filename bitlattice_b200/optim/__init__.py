"""Optimizers updating lattice weights in their storage format."""
from . import directions
from .lattice import DEFAULTS, DIRECTIONS, ROUNDINGS, SCALE_RULES, Lattice, defer_fused_updates
from .presets import PRESETS, param_groups

__all__ = ["DEFAULTS", "DIRECTIONS", "PRESETS", "ROUNDINGS", "SCALE_RULES", "Lattice", "defer_fused_updates",
           "directions", "param_groups"]
