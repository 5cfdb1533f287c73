"""Named option sets of the Lattice optimizer and the default grouping of a model's parameters (the names and contents
of the reference's ``bitlattice/optim/presets.py``, which are part of its API)."""
from __future__ import annotations

from typing import Any

import torch

__all__ = ["PRESETS", "param_groups"]

PRESETS: dict[str, dict[str, Any]] = {
    # orthogonalised (Newton-Schulz) direction on 512 x 512 blocks, 2-bit phase
    "muon": dict(direction="muon_block", phase_bits=2),
    # bands of 256 rows over the full width, Gram iteration in fp16 with the Polar Express coefficients
    "muon_fast": dict(direction="muon_block", phase_bits=2, block=(256, None), ns_dtype="fp16",
                      ns_coeffs="polar_express"),
    # the same with neuron-wise normalisation of the direction (one running mean square per row)
    "normuon": dict(direction="muon_block", phase_bits=2, normalize="row"),
    "normuon_fast": dict(direction="muon_block", phase_bits=2, block=(256, None), ns_dtype="fp16",
                         ns_coeffs="polar_express", normalize="row"),
    "muon_precise": dict(direction="muon_block", phase_bits=8),
    # factored second-moment direction with a 1 / 2 / 8-bit phase
    "light": dict(direction="factored", phase_bits=1),
    "balanced": dict(direction="factored", phase_bits=2),
    "precise": dict(direction="factored", phase_bits=8),
    # no optimizer state at all
    "stateless": dict(direction="sinkhorn", vector_direction="sinkhorn", phase_bits=0, rounding="sr"),
}

_HEADS = ("lm_head", "embed_out", "output", "classifier", "head")


def param_groups(model: torch.nn.Module, head_direction: str = "factored", head_momentum: str = "none",
                 no_decay_vectors: bool = True, weight_decay: float = 0.0) -> list[dict]:
    """Three groups: embeddings and output heads (``head_direction``: orthogonalising a vocabulary-sized matrix is far
    too expensive), other matrices (the optimizer's defaults), vectors (no weight decay unless asked)."""
    embedding_ids = {id(m.weight) for m in model.modules() if isinstance(m, torch.nn.Embedding)}
    buckets: dict[str, list] = {"heads": [], "matrices": [], "vectors": []}
    seen: set[int] = set()
    for name, p in model.named_parameters():
        if not p.requires_grad or id(p) in seen or p.device.type == "meta":
            continue
        seen.add(id(p))
        owner = name.rsplit(".", 1)[0].rsplit(".", 1)[-1] if "." in name else ""
        kind = "heads" if id(p) in embedding_ids or owner in _HEADS else "matrices" if p.dim() >= 2 else "vectors"
        buckets[kind].append(p)
    groups = []
    if buckets["matrices"]:
        groups.append({"params": buckets["matrices"], "weight_decay": weight_decay})
    if buckets["heads"]:
        groups.append({"params": buckets["heads"], "direction": head_direction, "momentum": head_momentum,
                       "weight_decay": weight_decay})
    if buckets["vectors"]:
        groups.append({"params": buckets["vectors"], "weight_decay": 0.0 if no_decay_vectors else weight_decay})
    return groups
