"""The NVFP4 storage format as an ordered lattice.

Mirrors the part of the reference's ``bitlattice/formats.py`` that the NVFP4 linear layer and optimizer update use
(``ScaleSpec`` :46-82, ``TableFormat`` :116-170, the registry entry :415): 4-bit E2M1 codes, one E4M3 scale per 16
consecutive elements of a row, an fp32 per-tensor scale. Other formats of the reference are out of this build's scope;
``get`` says so instead of guessing.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from functools import cache

import torch

__all__ = ["E4M3_MAX", "E4M3_MIN", "Format", "ScaleSpec", "TableFormat", "available", "get"]

E4M3_MAX = 448.0
E4M3_MIN = 2.0 ** -9

_E2M1 = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0)


@dataclass(frozen=True)
class ScaleSpec:
    """``group`` consecutive elements of a row share one scale stored as ``dtype``."""

    group: int = 16
    dtype: str = "e4m3"
    global_scale: bool = True
    strict: bool = True

    @property
    def bits(self) -> int:
        return 8

    @property
    def torch_dtype(self) -> torch.dtype:
        return torch.float8_e4m3fn

    def groups_per_row(self, cols: int) -> int:
        if cols % self.group:
            raise ValueError(f"last dimension {cols} is not a multiple of the scale group {self.group}")
        return cols // self.group

    def shape(self, rows: int, cols: int) -> tuple[int, int]:
        return rows, self.groups_per_row(cols)


class Format:
    name: str
    bits: int
    kind: str

    @property
    def container_bits(self) -> int:
        return 4 if self.bits <= 4 else 8

    def __repr__(self) -> str:
        return f"{type(self).__name__}({self.name})"


@dataclass(frozen=True, repr=False)
class TableFormat(Format):
    """Codes decoded through a table; ``values[code]`` is the level in units of the scale."""

    name: str
    bits: int
    values: tuple[float, ...]
    scale_spec: ScaleSpec = field(default_factory=ScaleSpec)
    init: str = "absmax"
    kind: str = "table"

    @property
    def scale(self) -> ScaleSpec:
        return self.scale_spec

    @property
    def levels(self) -> tuple[float, ...]:
        return tuple(sorted({v + 0.0 for v in self.values}))     # -0.0 and 0.0 are one level

    @property
    def max_abs(self) -> float:
        return max(abs(v) for v in self.levels)

    def storage_bits(self, rows: int, cols: int) -> int:
        r, g = self.scale.shape(rows, cols)
        return rows * cols * self.bits + r * g * self.scale.bits + 32

    @cache
    def tables(self, device: str = "cpu") -> dict[str, torch.Tensor]:
        """decode / rank-of-code / sorted levels / canonical code of each rank (+0 is the canonical zero)."""
        levels = self.levels
        rank_of = {v: i for i, v in enumerate(levels)}
        canon: dict[float, int] = {}
        for code, v in enumerate(self.values):
            if (v + 0.0) not in canon and not (v == 0.0 and math.copysign(1.0, v) < 0):
                canon[v + 0.0] = code
        dev = torch.device(device)
        return {
            "decode": torch.tensor(self.values, dtype=torch.float32, device=dev),
            "rank": torch.tensor([rank_of[v + 0.0] for v in self.values], dtype=torch.int32, device=dev),
            "sorted": torch.tensor(levels, dtype=torch.float32, device=dev),
            "sorted_code": torch.tensor([canon[v] for v in levels], dtype=torch.int32, device=dev),
        }


_NVFP4 = TableFormat("nvfp4", 4, _E2M1)
_REGISTRY = {"nvfp4": _NVFP4}


def available() -> list[str]:
    return sorted(_REGISTRY)


def get(spec) -> Format:
    """Resolve a format name (or pass a Format through). Only 'nvfp4' is built."""
    if isinstance(spec, Format):
        return spec
    key = str(spec).lower()
    if key not in _REGISTRY:
        raise KeyError(f"format {spec!r} is outside this build (the NVFP4 hot path); known: {', '.join(available())}")
    return _REGISTRY[key]
