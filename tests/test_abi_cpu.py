"""The C-ABI library loads without a GPU and exports every function the public header declares."""
import ctypes
import os
import re

from conftest import ROOT


def _declared():
    text = open(os.path.join(ROOT, "include", "bitlattice_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(bl_[a-z0-9_]+)\s*\(", text)))


def test_header_functions_are_exported():
    from bitlattice_b200 import _C
    names = _declared()
    assert len(names) >= 14
    lib = ctypes.CDLL(_C.LIB_PATH)
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/bitlattice_b200.h but not exported"
    assert names == _C.exported_symbols()


def test_host_side_helpers_run_without_a_device():
    from bitlattice_b200 import _C
    L = _C.lib()
    assert L.bl_version() >= 1
    assert L.bl_blocked_scale_bytes(200, 9) == 2 * 3 * 512
    from bitlattice_b200 import _ops
    for rows, cols16 in ((1, 1), (128, 4), (129, 5), (200, 9), (65536, 256), (12288, 768), (32, 2)):
        assert _ops.blocked_scale_bytes(rows, cols16) == L.bl_blocked_scale_bytes(rows, cols16)
    assert L.bl_update_scratch_bytes(4096, 4096, 1, 1.0) == 0            # sign with clip >= 1 needs no statistics
    assert L.bl_update_scratch_bytes(4096, 4096, 2, 1.0) >= 32 * 4096 * 4
    # argument validation happens before any CUDA call
    assert L.bl_nvfp4_gemm(None, None, None, None, None, None, 1, 1, 1, None, 1, 8, 0, None) != 0
    assert b"null buffer" in L.bl_last_error()


def test_product_never_touches_the_oracle():
    """The package must not import, load or name the CPU oracle: it is test infrastructure only."""
    pkg = os.path.join(ROOT, "bitlattice_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                src = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in src.lower(), os.path.join(dirpath, f)
