"""Named option sets of the Lattice optimizer and the default grouping of a model's parameters (the names and contents
of the reference's ``bitlattice/optim/presets.py``, which are part of its API)."""
from __future__ import annotations

from typing import Any

import torch

__all__ = ["PRESETS", "param_groups"]

# Row bands of 256 over the full width, Gram iteration in fp16 with the Polar Express coefficients: the cheap
# orthogonalisation of the "_fast" presets.
_BANDS = dict(block=(256, None), ns_dtype="fp16", ns_coeffs="polar_express")


def _orthogonal(phase_bits: int = 2, **extra) -> dict[str, Any]:
    """Newton-Schulz direction on blocks (512 x 512 unless ``extra`` says otherwise)."""
    return dict(direction="muon_block", phase_bits=phase_bits, **extra)


PRESETS: dict[str, dict[str, Any]] = {
    "muon": _orthogonal(),
    "muon_fast": _orthogonal(**_BANDS),
    "normuon": _orthogonal(normalize="row"),                  # one running mean square per row scales the direction
    "normuon_fast": _orthogonal(**_BANDS, normalize="row"),
    "muon_precise": _orthogonal(phase_bits=8),
    # factored second-moment direction, 1 / 2 / 8 bits of phase
    **{name: dict(direction="factored", phase_bits=bits) for name, bits in (("light", 1), ("balanced", 2), ("precise", 8))},
    # nothing kept between steps
    "stateless": dict(direction="sinkhorn", vector_direction="sinkhorn", phase_bits=0, rounding="sr"),
}

_HEADS = frozenset(("lm_head", "embed_out", "output", "classifier", "head"))


def _bucket(name: str, p: torch.Tensor, embeddings: set[int]) -> str:
    owner = name.rpartition(".")[0].rpartition(".")[2]
    if id(p) in embeddings or owner in _HEADS:
        return "heads"
    return "matrices" if p.dim() >= 2 else "vectors"


def param_groups(model: torch.nn.Module, head_direction: str = "factored", head_momentum: str = "none",
                 no_decay_vectors: bool = True, weight_decay: float = 0.0) -> list[dict]:
    """Parameter groups for ``Lattice``: matrices with the optimizer's defaults; embeddings and output heads with
    ``head_direction`` / ``head_momentum`` (orthogonalising a vocabulary-sized matrix costs far too much); vectors,
    which are spared weight decay unless ``no_decay_vectors`` is off. Frozen, shared and meta-device parameters are
    left out; empty groups are not returned."""
    embeddings = {id(m.weight) for m in model.modules() if isinstance(m, torch.nn.Embedding)}
    buckets: dict[str, list] = {"matrices": [], "heads": [], "vectors": []}
    taken: set[int] = set()
    for name, p in model.named_parameters():
        if p.requires_grad and id(p) not in taken and p.device.type != "meta":
            taken.add(id(p))
            buckets[_bucket(name, p, embeddings)].append(p)
    options = {"matrices": {"weight_decay": weight_decay},
               "heads": {"direction": head_direction, "momentum": head_momentum, "weight_decay": weight_decay},
               "vectors": {"weight_decay": 0.0 if no_decay_vectors else weight_decay}}
    return [{"params": ps, **options[kind]} for kind, ps in buckets.items() if ps]
