"""How layers with lattice weights compute (mirror of the reference's ``bitlattice/compute_policy.py``).

A lattice weight carries a :class:`Compute` (``weight.compute``); ``None`` means exact computation: the weight is
dequantized and the GEMMs run in the activations' dtype. ``Compute("nvfp4")`` runs forward (and, with ``backward``,
both gradient GEMMs) on FP4 tensor cores. A requirement that cannot be met raises instead of falling back.
"""
from __future__ import annotations

import contextlib
from dataclasses import dataclass, field

import torch

from .backend import FP4_RECIPES, Fp4Recipe, as_recipe, fp4_unfit

__all__ = ["PRESETS", "Compute", "as_compute", "compute", "route"]

GEMMS = ("exact", "nvfp4")


@dataclass(frozen=True)
class Compute:
    """gemm: 'exact' | 'nvfp4'; backward: gradient GEMMs on FP4 tensor cores too; nvfp4: the operand recipe."""

    gemm: str = "exact"
    backward: bool = True
    nvfp4: Fp4Recipe = field(default_factory=Fp4Recipe)
    kernels: object | None = None

    def __post_init__(self):
        if self.gemm not in GEMMS:
            raise ValueError(f"gemm must be one of {GEMMS} (the MXFP8 routes are not built)")
        if not isinstance(self.nvfp4, Fp4Recipe):
            object.__setattr__(self, "nvfp4", as_recipe(self.nvfp4))

    @property
    def route(self) -> str:
        """'exact', 'fp4' or 'fp4_all'."""
        if self.gemm == "exact":
            return "exact"
        return "fp4_all" if self.backward else "fp4"

    def describe(self) -> str:
        if self.gemm == "exact":
            return "exact"
        name = next((k for k, r in FP4_RECIPES.items() if r == self.nvfp4), None)
        return f"{self.gemm}{'' if self.backward else ' forward only'}, recipe {name}"


PRESETS: dict[str, Compute] = {
    "exact": Compute(),
    "fp4": Compute("nvfp4", backward=False),
    "fp4_all": Compute("nvfp4"),
    **{name: Compute("nvfp4", nvfp4=r) for name, r in FP4_RECIPES.items() if name != "nvidia"},
}


def as_compute(c) -> Compute | None:
    if c is None or c == "auto":
        return None
    if isinstance(c, Compute):
        return c
    if c not in PRESETS:
        raise ValueError(f"unknown compute {c!r}; presets: {sorted(PRESETS)}")
    return PRESETS[c]


# Process-wide, not thread-local: the backward pass runs on autograd worker threads and must see the forward's setting
# (reference: compute_policy.py:100-102).
_scope: list[Compute] = []


@contextlib.contextmanager
def compute(c):
    """Every lattice layer computes as ``c`` (a :class:`Compute` or preset name) inside the block."""
    _scope.append(as_compute(c) or Compute())
    try:
        yield
    finally:
        _scope.pop()


def route(x: torch.Tensor, w) -> tuple[str, Compute]:
    """(route, Compute) of a call of the lattice layer with weight ``w`` on input ``x``; RuntimeError when the
    requirement cannot be met (reference: compute_policy.py:127-137)."""
    c = _scope[-1] if _scope else getattr(w, "compute", None)
    if c is None or c.gemm == "exact":
        return "exact", c or Compute()
    index = x.device.index if (x.is_cuda and x.device == w.device) else None
    why = fp4_unfit(w, index, c.backward)
    if why is not None:
        name = getattr(w, "_bl_name", None) or f"weight {tuple(w.shape)}"
        raise RuntimeError(f"{name}: cannot compute as {c.describe()}: {why}")
    return c.route, c
