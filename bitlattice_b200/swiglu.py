"""SwiGLU glue of an MLP block on the library's kernels: ``a = silu(g) * u`` with the roundings of autograd.

The reference runs this inside its fused decoder block (``bitlattice/nn/fused_block.py:364-373, 419-423``) through
``torch.ops.bitlattice.swiglu_fwd`` / ``swiglu_bwd``; here it is a free-standing autograd function so that a
gate/up -> SwiGLU -> down block runs without an elementwise PyTorch kernel between the FP4 GEMMs.
"""
from __future__ import annotations

import torch

from . import _ops

__all__ = ["swiglu"]


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, g, u):
        g, u = g.contiguous(), u.contiguous()
        ctx.save_for_backward(g, u)
        return _ops.swiglu_fwd(g, u)

    @staticmethod
    def backward(ctx, da):
        g, u = ctx.saved_tensors
        dg, du = _ops.swiglu_bwd(g, u, da.contiguous())
        return dg, du


def swiglu(g: torch.Tensor, u: torch.Tensor) -> torch.Tensor:
    """silu(g) * u for bf16 / fp16 CUDA tensors; bit-identical to ``F.silu(g) * u`` in the forward and in ``u.grad``."""
    return _SwiGLU.apply(g, u)
