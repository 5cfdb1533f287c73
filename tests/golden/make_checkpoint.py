"""Writes tests/golden/ckpt/: a checkpoint saved by the REFERENCE's own bitlattice.io.hf.save (safetensors shards +
model.safetensors.index.json + bitlattice.json) for a two-layer module with one NVFP4 lattice weight, one dense
weight, biases and a buffer. The loader and writer of this repository are checked against these files.

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_checkpoint.py /path/to/reference
"""
import os
import shutil
import sys

import torch

REF = sys.argv[1]
sys.dont_write_bytecode = True
sys.path.insert(0, REF)

import bitlattice as bl  # noqa: E402
from bitlattice.io import hf  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ckpt")


class Tiny(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.up = torch.nn.Linear(64, 64)
        self.down = torch.nn.Linear(64, 32)
        self.register_buffer("steps", torch.arange(5, dtype=torch.int64))


def main():
    torch.manual_seed(7)
    m = Tiny().to(torch.bfloat16)
    w = (torch.randn(64, 64, generator=torch.Generator().manual_seed(70)) * 0.05)
    m.up.weight = torch.nn.Parameter(bl.LatticeTensor.from_float(w, "nvfp4", method="rtn", dtype=torch.bfloat16))
    if os.path.isdir(OUT):
        shutil.rmtree(OUT)
    hf.save(m, OUT)
    print(sorted(os.listdir(OUT)))


if __name__ == "__main__":
    main()
