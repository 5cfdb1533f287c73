"""bitlattice_b200: the NVFP4 LatticeTensor linear layer and the lattice optimizer update of NeuroMarshal/bitlattice,
rebuilt for B200 (sm_100a) behind the reference's Python API.

    import bitlattice_b200 as bl
    w = torch.nn.Parameter(bl.LatticeTensor.from_float(dense_cuda_weight, "nvfp4", method="rtn"))
    opt = bl.optim.Lattice([w], lr=3e-3, direction="sign", phase_bits=4, fused_backward=True)
    with bl.compute("fp4_all"):
        y = torch.nn.functional.linear(x, w)        # forward, dgrad and wgrad on tcgen05 FP4 tensor cores
    y.backward(gy)                                   # ... and the fused lattice update of w from the hook

All arithmetic runs in ``libbitlattice_b200.so`` (hand-written CUDA behind a C ABI, ``include/bitlattice_b200.h``);
importing the package loads it and fails if it has not been built (``python bitlattice_b200/csrc/build.py``).
"""
from . import _C

_C.lib()          # fail loudly here, not at the first kernel call, when the CUDA library is missing

from . import backend, formats, io, optim, packing, parallel  # noqa: E402
from ._ops import HAVE_EXT  # noqa: E402
from .compute_policy import PRESETS as COMPUTE_PRESETS  # noqa: E402
from .compute_policy import Compute, compute  # noqa: E402
from .formats import Format, TableFormat  # noqa: E402
from .optim import Lattice  # noqa: E402
from .swiglu import swiglu  # noqa: E402
from .tensor import LatticeTensor, is_lattice  # noqa: E402

__version__ = "0.1.0"

__all__ = ["COMPUTE_PRESETS", "HAVE_EXT", "Compute", "Format", "Lattice", "LatticeTensor", "TableFormat", "backend",
           "compute", "formats", "io", "is_lattice", "optim", "packing", "parallel", "swiglu"]
