"""Checkpoints in the reference's native on-disk layout (``bitlattice/io/hf.py:451-568``):

    model-XXXXX-of-YYYYY.safetensors   every tensor; a lattice parameter ``name`` is stored as its parts
                                       ``name.__packed`` (uint8 codes), ``name.__scales`` (float8_e4m3fn block scales),
                                       ``name.__global_scale`` (fp32 [1]) -- no re-encoding on the way in or out
    model.safetensors.index.json       {"metadata": {}, "weight_map": {tensor name: file}}
    bitlattice.json                    {"version": 1, "tensors": {name: {"format": spec, "shape", "dtype"}}, "tied": {}}

so a checkpoint written here loads in the reference and the other way round. Built for this path only: NVFP4 lattice
parameters plus ordinary tensors of a module; model skeletons, Hugging Face configs and third-party quantized layouts
(ModelOpt, compressed-tensors, GPTQ, AWQ) stay with the reference's loader.

Third-party NVFP4 layouts convert without touching a code or a scale byte (reference: ``bitlattice/io/convert.py:40-54,
155-160``): compressed-tensors 'nvfp4-pack-quantized' (``weight_packed``, ``weight_scale``, ``weight_global_scale``
stored as a divisor) and ModelOpt NVFP4 (``weight``, ``weight_scale``, ``weight_scale_2`` stored as a multiplier)
share the byte layout of ``packed`` / ``scales``; only the per-tensor scale changes its convention.

N-sharded weights (``parallel.shard_rows``): ``save`` called by every rank of ``group`` gathers the row shards of each
lattice parameter on rank 0, which writes the checkpoint of the unsharded model; ``load_into`` gives each rank its rows.
"""
from __future__ import annotations

import json
import os
from typing import Any

import torch
import torch.distributed as dist

from . import formats as F
from .tensor import LatticeTensor, wait_for_update

__all__ = ["format_from_spec", "format_spec", "from_ct_nvfp4", "from_mo_nvfp4", "load_into", "load_state", "save",
           "to_ct_nvfp4"]

_PARTS = ("packed", "scales", "global_scale")


def format_spec(fmt) -> dict:
    """JSON description of a format, field for field the reference's (io/hf.py:431-441)."""
    d: dict[str, Any] = {"kind": fmt.kind, "name": fmt.name, "bits": fmt.bits}
    if fmt.kind == "table":
        d["values"] = list(fmt.values)
        d["init"] = fmt.init
    if fmt.scale is not None:
        d["scale"] = dict(group=fmt.scale.group, dtype=fmt.scale.dtype, global_scale=fmt.scale.global_scale,
                          strict=fmt.scale.strict)
    return d


def format_from_spec(d: dict):
    if d.get("kind") != "table":
        raise NotImplementedError(f"format kind {d.get('kind')!r} is outside this build (table formats are built)")
    return F.TableFormat(d["name"], d["bits"], tuple(float(v) for v in d["values"]), F.ScaleSpec(**d["scale"]),
                         d.get("init", "absmax"))


def _world(group) -> tuple[int, int]:
    if not (dist.is_available() and dist.is_initialized()):
        return 0, 1
    return dist.get_rank(group), dist.get_world_size(group)


def _gather_rows(t: torch.Tensor, group, rank: int, size: int) -> torch.Tensor | None:
    """Row shards of equal shape -> the full tensor on rank 0 (None elsewhere)."""
    t = t.detach().contiguous()
    raw = t.view(torch.uint8) if t.dtype == torch.float8_e4m3fn else t       # collectives on plain bytes
    out = torch.empty(size * raw.shape[0], *raw.shape[1:], dtype=raw.dtype, device=raw.device)
    dist.all_gather_into_tensor(out, raw, group=group)
    if rank != 0:
        return None
    return out.view(t.dtype) if raw is not t else out


def _named_tensors(obj):
    """(name, tensor, is_buffer) of a module's parameters and buffers, or of a plain mapping."""
    if isinstance(obj, torch.nn.Module):
        seen: dict[int, str] = {}
        for name, p in obj.named_parameters(remove_duplicate=False):
            if id(p) in seen:
                yield name, seen[id(p)], "tied"
                continue
            seen[id(p)] = name
            yield name, p, "param"
        for name, b in obj.named_buffers():
            yield name, b, "buffer"
    else:
        for name, t in obj.items():
            yield name, t, "param"


def save(obj, path: str, max_shard_bytes: int = 4 << 30, group=None) -> None:
    """Write the parameters and buffers of ``obj`` (a module, or a mapping name -> tensor) to ``path``. With an
    initialised process group every rank calls it; rank 0 writes."""
    rank, size = _world(group)
    meta: dict[str, Any] = {"version": 1, "tensors": {}}
    flat: dict[str, torch.Tensor] = {}
    for name, t, kind in _named_tensors(obj):
        if kind == "tied":
            meta.setdefault("tied", {})[name] = t
            continue
        if isinstance(t, LatticeTensor):
            wait_for_update(t)                 # an optimizer update still running on another stream finishes first
            sharded = size > 1 and hasattr(t, "_bl_row_offset")
            shape = list(t.shape)
            parts = {}
            for k in _PARTS:
                v = getattr(t, k)
                if sharded and k != "global_scale":
                    v = _gather_rows(v, group, rank, size)
                parts[k] = v
            if sharded:
                shape[0] *= size
            if rank == 0:
                meta["tensors"][name] = {"format": format_spec(t.fmt), "shape": shape,
                                         "dtype": str(t.dtype).replace("torch.", "")}
                for k, v in parts.items():
                    flat[f"{name}.__{k}"] = v.detach().contiguous().cpu()
        elif rank == 0:
            flat.setdefault(name, t.detach().contiguous().cpu())
    if rank != 0:
        if size > 1:
            dist.barrier(group=group)
        return
    try:
        _write(path, flat, meta, max_shard_bytes)
    finally:
        if size > 1:                           # the other ranks wait here: reach it even when writing failed
            dist.barrier(group=group)


def _write(path: str, flat: dict, meta: dict, max_shard_bytes: int) -> None:
    from safetensors.torch import save_file
    os.makedirs(path, exist_ok=True)
    shards, cur, used = [], {}, 0
    for k, v in flat.items():
        n = v.numel() * v.element_size()
        if cur and used + n > max_shard_bytes:
            shards.append(cur)
            cur, used = {}, 0
        cur[k] = v
        used += n
    shards.append(cur)
    weight_map = {}
    for i, sh in enumerate(shards):
        fname = f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        save_file(sh, os.path.join(path, fname), metadata={"format": "pt"})
        weight_map.update({k: fname for k in sh})
    with open(os.path.join(path, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {}, "weight_map": weight_map}, f, indent=1)
    with open(os.path.join(path, "bitlattice.json"), "w") as f:
        json.dump(meta, f, indent=1)


def _shard_files(path: str) -> list[str]:
    idx = os.path.join(path, "model.safetensors.index.json")
    if os.path.exists(idx):
        with open(idx) as f:
            return sorted({os.path.join(path, v) for v in json.load(f)["weight_map"].values()})
    files = sorted(os.path.join(path, f) for f in os.listdir(path) if f.endswith(".safetensors"))
    if not files:
        raise FileNotFoundError(f"no safetensors files in {path}")
    return files


def load_state(path: str, device="cpu", rows: dict | None = None) -> dict[str, torch.Tensor]:
    """name -> tensor for every entry of the checkpoint; lattice parameters come back as LatticeTensor built from their
    stored parts. ``rows``: optional {name: (lo, hi)} to keep only a row range of a lattice parameter."""
    from safetensors import safe_open
    with open(os.path.join(path, "bitlattice.json")) as f:
        meta = json.load(f)
    parts: dict[str, dict[str, torch.Tensor]] = {}
    out: dict[str, torch.Tensor] = {}
    for shard in _shard_files(path):
        with safe_open(shard, framework="pt", device="cpu") as f:
            for k in f.keys():
                if ".__" in k:
                    name, part = k.split(".__", 1)
                    t = f.get_tensor(k)
                    if rows and name in rows and part != "global_scale":
                        t = t[rows[name][0]:rows[name][1]].contiguous()
                    parts.setdefault(name, {})[part] = t.to(device)
                else:
                    out[k] = f.get_tensor(k).to(device)
    for name, info in meta["tensors"].items():
        p = parts[name]
        extra = set(p) - set(_PARTS)
        if extra:
            raise NotImplementedError(f"{name}: parts {sorted(extra)} (zero points / high-precision columns) are "
                                      "outside this build")
        shape = list(info["shape"])
        if rows and name in rows:
            shape[0] = rows[name][1] - rows[name][0]
        out[name] = LatticeTensor(p["packed"], p["scales"], p["global_scale"], None, format_from_spec(info["format"]),
                                  shape, getattr(torch, info["dtype"]))
    for name, target in meta.get("tied", {}).items():
        out[name] = out[target]
    return out


def load_into(module: torch.nn.Module, path: str, device=None, group=None) -> None:
    """Assign the checkpoint's tensors to ``module``'s parameters and buffers. A lattice parameter of the module that
    is a row shard (``_bl_row_offset`` set by ``parallel.shard_rows``) receives its own rows of the stored weight."""
    from .parallel import shard_bounds
    rank, size = _world(group)
    with open(os.path.join(path, "bitlattice.json")) as f:
        meta = json.load(f)
    params = dict(module.named_parameters(remove_duplicate=False))
    rows = {}
    for name, info in meta["tensors"].items():
        p = params.get(name)
        if size > 1 and p is not None and hasattr(p, "_bl_row_offset"):
            rows[name] = shard_bounds(info["shape"][0], rank, size)
    if device is None:
        device = next((p.device for p in params.values()), torch.device("cpu"))
    state = load_state(path, device, rows)
    buffers = dict(module.named_buffers())
    for name, t in state.items():
        owner, _, leaf = name.rpartition(".")
        mod = module.get_submodule(owner) if owner else module
        if name in buffers:
            mod._buffers[leaf] = t
            continue
        if name not in params:
            raise KeyError(f"{name} of the checkpoint is not a parameter or buffer of the module")
        old = params[name]
        new = torch.nn.Parameter(t, requires_grad=old.requires_grad and t.is_floating_point())
        if name in rows:
            new._bl_row_offset = rows[name][0]
            new._bl_rows_total = int(meta["tensors"][name]["shape"][0])
        mod._parameters[leaf] = new


# ------------------------------------------------------------------------------------ third-party NVFP4 layouts

def _as_lattice(codes: torch.Tensor, scales: torch.Tensor, global_scale: torch.Tensor, dtype, device) -> LatticeTensor:
    rows, half = codes.shape
    if scales.shape != (rows, half // 8):
        raise ValueError(f"scales {tuple(scales.shape)} do not match codes {tuple(codes.shape)} (one per 16 values)")
    sc = scales.to(device).contiguous()
    sc = sc if sc.dtype == torch.float8_e4m3fn else sc.view(torch.float8_e4m3fn)
    return LatticeTensor(codes.to(device, torch.uint8).contiguous(), sc,
                         global_scale.to(device, torch.float32).reshape(1), None, F.get("nvfp4"), (rows, 2 * half),
                         dtype)


def from_ct_nvfp4(tensors: dict, dtype=torch.bfloat16, device="cuda") -> LatticeTensor:
    """compressed-tensors NVFP4 (value = e2m1 * weight_scale / weight_global_scale) as a lattice weight: the stored
    divisor becomes the per-tensor multiplier 1 / weight_global_scale (fp32 division)."""
    return _as_lattice(tensors["weight_packed"], tensors["weight_scale"],
                       1.0 / tensors["weight_global_scale"].float(), dtype, device)


def from_mo_nvfp4(tensors: dict, dtype=torch.bfloat16, device="cuda") -> LatticeTensor:
    """ModelOpt NVFP4 (value = e2m1 * weight_scale * weight_scale_2) as a lattice weight."""
    return _as_lattice(tensors["weight"], tensors["weight_scale"], tensors["weight_scale_2"].float(), dtype, device)


def to_ct_nvfp4(w: LatticeTensor) -> dict[str, torch.Tensor]:
    """The compressed-tensors NVFP4 tensors of a lattice weight (the inverse of ``from_ct_nvfp4`` up to the rounding of
    the reciprocal)."""
    if w.fmt.name != "nvfp4":
        raise ValueError("only nvfp4 tensors are exported to compressed-tensors")
    return {"weight_packed": w.packed.contiguous(), "weight_scale": w.scales.contiguous(),
            "weight_global_scale": (1.0 / w.global_scale.float()).reshape(1)}
