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
    """``c`` as a :class:`Compute`: itself, the preset of that name, or None for 'auto' / None (the weight's own)."""
    if isinstance(c, Compute):
        return c
    if c in (None, "auto"):
        return None
    try:
        return PRESETS[c]
    except KeyError:
        raise ValueError(f"unknown compute {c!r}; presets: {sorted(PRESETS)}") from None


# The innermost ``compute(...)`` block wins over the weights' own settings. One stack for the whole process: backward
# (and recomputation under checkpointing) runs on autograd's threads and has to see what the forward pass saw
# (reference: compute_policy.py:100-102).
_scope: list[Compute] = []


@contextlib.contextmanager
def compute(c):
    """Inside the block every lattice layer computes as ``c`` (a :class:`Compute` or the name of a preset)."""
    chosen = as_compute(c)
    _scope.append(chosen if chosen is not None else Compute())
    try:
        yield
    finally:
        _scope.pop()


def route(x: torch.Tensor, w) -> tuple[str, Compute]:
    """Which way the layer with weight ``w`` goes for input ``x``: ('exact' | 'fp4' | 'fp4_all', the Compute in
    force). A setting the weight or the device cannot honour raises RuntimeError with the reason; nothing falls back
    silently (reference: compute_policy.py:127-137)."""
    setting = _scope[-1] if _scope else getattr(w, "compute", None)
    if setting is None:
        return "exact", Compute()
    if setting.gemm == "exact":
        return "exact", setting
    same_gpu = x.is_cuda and x.device == w.device
    reason = fp4_unfit(w, x.device.index if same_gpu else None, setting.backward)
    if reason is None:
        return setting.route, setting
    label = getattr(w, "_bl_name", None) or f"weight {tuple(w.shape)}"
    raise RuntimeError(f"{label}: cannot compute as {setting.describe()}: {reason}")
