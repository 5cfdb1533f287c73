"""Update directions beyond raw / sign / colnorm, and low-precision momentum, for the Lattice optimizer on the GPU.

The three directions on the benchmarked path are fused into the update kernel (``bl_nvfp4_lattice_update``). The ones
here produce an fp32 direction ``D`` [rows, cols] that the update kernel then takes as given
(``bl_nvfp4_step_quantized``), as the reference does for all of its directions
(``bitlattice/optim/lattice.py:487-518`` -> ``bitlattice/_ops.py:110-144``):

  muon / muon_block   orthogonalised direction: Newton-Schulz iterations on the whole matrix or on blocks of it,
                      as matrix products in ``ns_dtype`` (library GEMMs: torch.matmul), quintic 'muon' or
                      'polar_express' coefficients, standard or Gram-matrix iteration
                      (reference: bitlattice/reference.py:398-459, csrc/directions.cpp:41-115)
  factored            Adafactor-like second-moment estimate from row and column averages kept across steps
                      (reference: bitlattice/reference.py:462-479, csrc/factored.cu)
  sinkhorn            alternating row / column RMS normalisation (reference: bitlattice/reference.py:482-486)
  normalize='row'     neuron-wise normalisation of the direction with a running mean square per row
                      (reference: bitlattice/reference.py:493-499)

All of them end in the RMS clip ``D = U / max(1, rms(U) / clip)``, computed by the library's direction kernel in its
fixed reduction order. These run outside the fused kernel and write D to memory: they are the functional counterpart
of the reference's directions, not a tuned path.

Momentum kept in a low-precision format between steps (reference: bitlattice/optim/lattice.py:396-462): 'ternary'
(one trit per element and a scale per row, stochastic rounding with the counter-based hash), 'fp8' (E4M3 with a
scale per 256 elements, round to nearest), 'bf16' and 'int8' (stochastic rounding with torch's device generator, as
the reference draws them).
"""
from __future__ import annotations

import math

import torch

from .. import _ops

__all__ = ["direction", "load_momentum", "momentum", "newton_schulz", "ns_coefficients", "store_momentum"]

_POLAR_EXPRESS = ((8.28721201814563, -23.595886519098837, 17.300387312530933),
                  (4.107059111542203, -2.9478499167379106, 0.5448431082926601),
                  (3.9486908534822946, -2.908902115962949, 0.5518191394370137),
                  (3.3184196573706015, -2.488488024314874, 0.51004894012372),
                  (2.300652019954817, -1.6689039845747493, 0.4188073119525673))
_NS_DTYPE = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}
MOM_BLOCK = 256                    # elements per scale of int8 / fp8 momentum


def ns_coefficients(kind: str, i: int) -> tuple[float, float, float]:
    """(a, b, c) of iteration ``i`` of x <- a x + (b s + c s^2) x, s = x x^T: the fixed quintic of Muon, or the
    Polar Express schedule (Amsel et al. 2025) with its safety factor 1.05."""
    if kind == "muon":
        return 3.4445, -4.7750, 2.0315
    if kind != "polar_express":
        raise ValueError(f"ns_coeffs={kind!r}; expected 'muon' or 'polar_express'")
    a, b, c = _POLAR_EXPRESS[min(i, 4)]
    return a / 1.05, b / 1.05 ** 3, c / 1.05 ** 5


def newton_schulz(g: torch.Tensor, steps: int = 5, eps: float = 1e-7, coeffs: str = "muon",
                  algo: str = "standard") -> torch.Tensor:
    """Approximate polar factor of ``g`` ([..., m, n], batched over leading dimensions), iterated in ``g.dtype``.
    'gram' iterates on the m x m Gram matrix and multiplies x only twice (restart after two steps); 'auto' picks it
    for wide matrices outside bf16."""
    dtype = g.dtype
    x = g.float()
    x = (x / (x.norm(dim=(-2, -1), keepdim=True) + eps)).to(dtype)
    tall = x.shape[-2] > x.shape[-1]
    if tall:
        x = x.mT
    use_gram = algo == "gram" or (algo == "auto" and x.shape[-1] >= 2 * x.shape[-2] and dtype != torch.bfloat16)
    if not use_gram:
        for i in range(steps):
            a, b, c = ns_coefficients(coeffs, i)
            s = x @ x.mT
            x = a * x + (b * s + c * s @ s) @ x
        return x.mT if tall else x
    eye = torch.eye(x.shape[-2], device=x.device, dtype=x.dtype)
    gram = x @ x.mT
    acc = None
    for i in range(steps):
        a, b, c = ns_coefficients(coeffs, i)
        if i == 2:                                   # restart: apply the accumulated polynomial, rebuild the Gram matrix
            x = acc @ x
            gram = x @ x.mT
        poly = a * eye + b * gram + c * gram @ gram
        acc = poly if i in (0, 2) else acc @ poly
        if i + 1 not in (steps, 2):
            gram = poly @ gram @ poly
    x = acc @ x
    return x.mT if tall else x


def _block_shape(block) -> tuple[int, int]:
    if isinstance(block, int):
        return int(block), int(block)
    return int(block[0]), -1 if block[1] is None else int(block[1])


def _muon(G2: torch.Tensor, block, steps: int, dtype: torch.dtype, coeffs: str, algo: str) -> torch.Tensor:
    g = G2.to(dtype)
    m, n = g.shape
    br, bc = block
    bc = n if bc is None or bc < 0 else br if bc == 0 else bc
    if br <= 0 or (m <= br and n <= bc):
        return (newton_schulz(g, steps, coeffs=coeffs, algo=algo) * math.sqrt(max(m, n))).float()
    x = torch.nn.functional.pad(g, (0, (-n) % bc, 0, (-m) % br))
    M, N = x.shape
    x = x.view(M // br, br, N // bc, bc).permute(0, 2, 1, 3).reshape(-1, br, bc)
    y = newton_schulz(x, steps, coeffs=coeffs, algo=algo) * math.sqrt(max(br, bc))
    y = y.view(M // br, N // bc, br, bc).permute(0, 2, 1, 3).reshape(M, N)
    return y[:m, :n].float()


def _factored(G2: torch.Tensor, r: torch.Tensor, c: torch.Tensor, k: int, beta2: float, eps: float = 1e-12):
    """r, c: running averages of the row / column mean squares (updated in place); k: the step number (from 1)."""
    x = G2.float()
    peak = x.abs().amax()
    x = x / torch.where(peak > 0, peak, torch.ones_like(peak))
    r.mul_(beta2).add_(x.square().mean(1), alpha=1 - beta2)
    c.mul_(beta2).add_(x.square().mean(0), alpha=1 - beta2)
    corr = 1 - beta2 ** k
    rr, cc = r / corr, c / corr
    v = (rr / rr.mean().clamp_min(eps))[:, None] * cc[None, :]
    return x / (v.sqrt() + eps)


def _sinkhorn(G2: torch.Tensor, iters: int) -> torch.Tensor:
    u = G2.float()
    for _ in range(iters):
        u = u / (u.square().mean(1, keepdim=True).sqrt() + 1e-30)
        u = u / (u.square().mean(0, keepdim=True).sqrt() + 1e-30)
    return u


def direction(G: torch.Tensor, kind: str, r=None, c=None, k: int = 1, beta2: float = 0.95, block=0, ns_steps: int = 5,
              ns_dtype: str = "bf16", sinkhorn_iters: int = 2, clip: float = 1.0, ns_coeffs: str = "muon",
              ns_algo: str = "auto", row_state=None, row_k: int = 1, row_beta: float = 0.95,
              row_eps: float = 1e-8) -> torch.Tensor:
    """fp32 direction [rows, cols] of the gradient ``G`` for any of the reference's kinds, RMS-clipped to ``clip``
    (same arguments as the reference's ``_ops.direction``). raw / sign / colnorm without row normalisation go to the
    library kernel directly."""
    G2 = G.reshape(1, -1) if G.dim() == 1 else G.reshape(G.shape[0], -1)
    if kind in ("raw", "sign", "colnorm") and row_state is None:
        return _ops.direction(G2, kind, clip=clip)
    if kind in ("muon", "muon_block"):
        blk = _block_shape(block) if kind == "muon_block" else (0, 0)
        U = _muon(G2, blk, ns_steps, _NS_DTYPE[ns_dtype], ns_coeffs, ns_algo)
    elif kind == "factored":
        U = _factored(G2, r, c, k, beta2)
    elif kind == "sinkhorn":
        U = _sinkhorn(G2, sinkhorn_iters)
    elif kind in ("raw", "sign", "colnorm"):
        U = _ops.direction(G2, kind, clip=float("inf"))
    else:
        raise ValueError(f"unknown direction {kind!r}")
    if row_state is not None:                        # neuron-wise normalisation with a running mean square per row
        row_state.mul_(row_beta).add_(U.square().mean(1), alpha=1 - row_beta)
        rowf = 1.0 / ((row_state / (1 - row_beta ** max(row_k, 1))).sqrt() + row_eps)
        U = U * rowf[:, None]
    return _ops.direction(U.contiguous(), "raw", clip=clip)             # the RMS clip, in the library's fixed order


# ------------------------------------------------------------------------------------------------ momentum

def _hash_uniform(n: int, seed: int, step: int, device) -> torch.Tensor:
    """u in [0, 1) for element indices 0..n-1 (the reference's counter-based generator, bitlattice/reference.py:22-30),
    evaluated with 64-bit integer tensor arithmetic masked to 32 bits."""
    m = 0xFFFFFFFF
    key = ((seed & m) * 0x9E3779B1 + (step & m) * 0x85EBCA77) & m
    x = (torch.arange(n, device=device, dtype=torch.int64) * 0x27D4EB2F + key) & m
    x = ((x ^ (x >> 16)) * 0x7FEB352D) & m
    x = ((x ^ (x >> 15)) * 0x846CA68B) & m
    x = x ^ (x >> 16)
    return (x >> 8).float() * (1.0 / 16777216.0)


def load_momentum(st: dict, mode: str, X: torch.Tensor) -> torch.Tensor:
    rows, cols = X.shape
    if mode == "bf16":
        return st["mb"].float() if "mb" in st else torch.zeros_like(X)
    if mode == "nvfp4":
        if "m4p" not in st:
            return torch.zeros_like(X)
        return _ops.dequantize(st["m4p"], st["m4s"], st["m4g"], None, "nvfp4", rows, cols, torch.float32)
    if "m8" not in st:
        return torch.zeros_like(X)
    return (st["m8"].float() * st["m8s"][:, None]).reshape(-1)[:X.numel()].view(rows, cols)


def store_momentum(st: dict, mode: str, m: torch.Tensor, seed: int, gens: dict) -> None:
    if mode == "nvfp4":             # stochastic rounding with four-over-six block scales (the general quantizer)
        st["m4p"], st["m4s"], st["m4g"] = _ops.nvfp4_quantize_general(m.contiguous(), mode="sr", four_over_six=True,
                                                                      seed=seed)
        return
    gen = gens.get(m.device)
    if gen is None:
        gen = gens[m.device] = torch.Generator(device=m.device)
    gen.manual_seed(seed)
    if mode == "bf16":                               # stochastic rounding: add 16 random low bits, truncate
        bits = m.contiguous().view(torch.int32)
        noise = torch.randint(0, 1 << 16, bits.shape, device=m.device, dtype=torch.int32, generator=gen)
        st["mb"] = ((bits + noise) & -65536).view(torch.float32).to(torch.bfloat16)
        return
    flat = m.reshape(-1)
    blocks = torch.nn.functional.pad(flat, (0, (-flat.numel()) % MOM_BLOCK)).view(-1, MOM_BLOCK)
    top = 127.0 if mode == "int8" else 448.0
    # (a tensor divisor: dividing by a Python scalar multiplies by its reciprocal on the GPU, one ulp off the quotient)
    scale = (blocks.abs().amax(1) / torch.full((), top, device=m.device)).clamp_min(1e-30)
    q = blocks / scale[:, None]
    if mode == "int8":
        u = torch.rand(q.shape, device=m.device, generator=gen)
        st["m8"] = torch.floor(q + u).clamp_(-127, 127).to(torch.int8)
    else:
        st["m8"] = q.to(torch.float8_e4m3fn)
    st["m8s"] = scale


def momentum(G2: torch.Tensor, st: dict, mode: str, beta1: float, seed: int, pid: int, gens: dict) -> torch.Tensor:
    """Exponential average of the gradient kept in ``mode`` between steps; returns the fp32 average that takes the
    gradient's place in the direction (reference: bitlattice/optim/lattice.py:396-431). ``st["step"]`` is the step
    being applied."""
    X = G2.float()
    if mode == "fp32":
        if "m" not in st:
            st["m"] = torch.zeros_like(X)
        st["m"].mul_(beta1).add_(X, alpha=1 - beta1)
        return st["m"]
    if mode in ("bf16", "int8", "fp8", "nvfp4"):
        if mode == "nvfp4" and X.shape[1] % 16:
            mode = "int8"                            # rows not made of 16-element blocks keep int8 momentum
        m = load_momentum(st, mode, X)
        m.mul_(beta1).add_(X, alpha=1 - beta1)
        store_momentum(st, mode, m, (seed + 7919 * pid + 104729 * st["step"]) & 0x7FFFFFFF, gens)
        return m
    if mode != "ternary":
        raise NotImplementedError(f"momentum={mode!r} is outside this build")
    peak = X.abs().amax()
    X = X / torch.where(peak > 0, peak, torch.ones_like(peak))
    if "mq" not in st:
        st["mq"] = torch.zeros_like(X, dtype=torch.int8)
        st["ms"] = torch.zeros(X.shape[0], device=X.device)
    m = beta1 * st["mq"].float() * st["ms"][:, None] + (1 - beta1) * X
    s = m.abs().amax(1).clamp_min(1e-30)
    q = m / s[:, None]
    fl = torch.floor(q)
    u = _hash_uniform(q.numel(), seed + 7919 * pid + 1, st["step"], q.device).view_as(q)
    st["mq"] = (fl + (u < q - fl).float()).clamp(-1, 1).to(torch.int8)
    st["ms"] = s
    return m
