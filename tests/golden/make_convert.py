"""Writes tests/golden/convert.npz: third-party NVFP4 checkpoint layouts (compressed-tensors 'nvfp4-pack-quantized' and
ModelOpt NVFP4) of one seeded weight, and what the REFERENCE's bitlattice.io.convert makes of them (LatticeTensor
parts, dequantized values) and exports back. The converters of this repository are checked against these arrays.

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_convert.py /path/to/reference
"""
import os
import sys

import numpy as np
import torch

REF = sys.argv[1]
sys.dont_write_bytecode = True
sys.path.insert(0, REF)

import bitlattice as bl  # noqa: E402
from bitlattice.io import convert  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "convert.npz")


def u8(t):
    return t.contiguous().view(torch.uint8).numpy()


def main():
    g = torch.Generator().manual_seed(321)
    w = torch.randn(96, 128, generator=g) * 0.03
    lt = bl.LatticeTensor.from_float(w, "nvfp4", method="rtn", dtype=torch.bfloat16)
    out = {}
    # compressed-tensors: the global scale is stored as a divisor
    ct = convert.to_ct_nvfp4(lt)
    out["ct_weight_packed"], out["ct_weight_scale"] = u8(ct["weight_packed"]), u8(ct["weight_scale"])
    out["ct_weight_global_scale"] = ct["weight_global_scale"].numpy()
    back = convert.from_ct_nvfp4(ct, torch.bfloat16, "cpu")
    out["ct_packed"], out["ct_scales"], out["ct_global"] = u8(back.packed), u8(back.scales), back.global_scale.numpy()
    out["ct_dequant"] = back.dequantize(torch.float32).numpy()
    # ModelOpt: the global scale is stored as a multiplier
    mo = {"weight": lt.packed.clone(), "weight_scale": lt.scales.clone(),
          "weight_scale_2": (lt.global_scale.float() * 1.5).reshape(())}
    out["mo_weight"], out["mo_weight_scale"] = u8(mo["weight"]), u8(mo["weight_scale"])
    out["mo_weight_scale_2"] = mo["weight_scale_2"].numpy()
    m = convert.from_mo_nvfp4(mo, torch.bfloat16, "cpu")
    out["mo_packed"], out["mo_scales"], out["mo_global"] = u8(m.packed), u8(m.scales), m.global_scale.numpy()
    out["mo_dequant"] = m.dequantize(torch.float32).numpy()
    np.savez_compressed(OUT, **out)
    print({k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
