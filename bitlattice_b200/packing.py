"""Little-endian bit packing of integer codes along the last dimension.

Same layout and function names as the reference's ``bitlattice/packing.py:13-58``: sub-byte containers (1, 2, 4 bits)
put element ``j`` of every group of ``8 // bits`` elements at bit offset ``j * bits`` of one byte; 8-bit codes are one
byte each. Wider containers are outside the NVFP4 path and are not provided.
"""
from __future__ import annotations

import torch

__all__ = ["pack", "packed_cols", "sign_extend", "unpack"]


def _check(container_bits: int) -> int:
    if container_bits not in (1, 2, 4, 8):
        raise ValueError(f"container of {container_bits} bits is not part of the NVFP4 path (1, 2, 4 or 8)")
    return 8 // container_bits


def packed_cols(cols: int, container_bits: int) -> int:
    """Bytes per row of ``cols`` codes."""
    per = _check(container_bits)
    if cols % per:
        raise ValueError(f"last dimension {cols} is not a multiple of {per} ({container_bits}-bit codes)")
    return cols // per


def pack(codes: torch.Tensor, container_bits: int) -> torch.Tensor:
    """Raw bit patterns (any integer dtype) -> uint8 bytes; only the low ``container_bits`` bits are kept."""
    per = _check(container_bits)
    n = packed_cols(codes.shape[-1], container_bits)
    v = codes.to(torch.int32) & ((1 << container_bits) - 1)
    if per == 1:
        return v.to(torch.uint8)
    v = v.reshape(*codes.shape[:-1], n, per)
    out = torch.zeros(*codes.shape[:-1], n, dtype=torch.int32, device=codes.device)
    for j in range(per):
        out |= v[..., j] << (j * container_bits)
    return out.to(torch.uint8)


def unpack(packed: torch.Tensor, container_bits: int, cols: int) -> torch.Tensor:
    """Inverse of :func:`pack`: unsigned bit patterns as int32, ``cols`` per row."""
    per = _check(container_bits)
    b = packed.to(torch.int32)
    if per == 1:
        return b & 0xFF
    mask = (1 << container_bits) - 1
    parts = [(b >> (j * container_bits)) & mask for j in range(per)]
    return torch.stack(parts, dim=-1).reshape(*packed.shape[:-1], packed.shape[-1] * per)[..., :cols]


def sign_extend(raw: torch.Tensor, bits: int) -> torch.Tensor:
    """The low ``bits`` bits of ``raw`` read as a two's complement integer (int64)."""
    v = raw.to(torch.int64) & ((1 << bits) - 1)
    return torch.where(v >= (1 << (bits - 1)), v - (1 << bits), v)
