"""The fixed-scratch lattice update (bl_nvfp4_lattice_update_fixed_scratch) against the ordinary entry point.

Some hosts of this library cannot give it scratch memory: they run where nothing may be allocated (a frozen memory
plan, a thread that must stay clear of the allocator's locks and of the device synchronisation cudaMalloc can imply).
For them the update keeps its column statistics in an array inside the library. This test drives that entry point
through the C ABI, twice in a row on the same weights (the second call meets whatever the first left in the array),
and requires codes, phase and scale bytes identical to those of bl_nvfp4_lattice_update with a caller-owned buffer.
It is collected last on purpose, and it must pass on its own in a fresh process as well as after the whole suite.
"""
import ctypes

import pytest
import torch

from bitlattice_b200 import _C, _ops

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _state(rows, cols, seed):
    g = torch.Generator(device=DEV).manual_seed(seed)
    w = torch.randn(rows, cols, device=DEV, generator=g) * 0.02
    am = _ops.amax_global(w)
    gs = am[1:2].clone()
    packed, scales = _ops.quantize_nvfp4(w, gs)
    return packed, torch.zeros(rows, cols // 2, dtype=torch.uint8, device=DEV), scales.view(torch.uint8).clone(), gs


def _call(name, packed, phase, scales, gs, G, rows, cols, direction, clip, step, scratch=None):
    args = [_C.ptr(packed), _C.ptr(phase), _C.ptr(scales), _C.ptr(gs), _C.ptr(G), _C.DTYPE[G.dtype], rows, cols, 0,
            4, 4, 3e-3, 1.0, 0, 1234, step, 0, 1, 1, 0.1, direction, clip]
    if name == "bl_nvfp4_lattice_update":
        args += [_C.ptr(scratch), scratch.numel() if scratch is not None else 0]
    args += [_C.device_of(packed), _C.stream_of(packed)]
    _C.call(name, *args)


@pytest.mark.parametrize("direction,clip", [(2, 1.0), (0, 0.5), (1, 0.25)])      # colnorm, raw, sign with a clip
def test_fixed_scratch_update_equals_ordinary_update(direction, clip):
    rows, cols = 384, 1024
    need = _C.lib().bl_update_scratch_bytes(rows, cols, direction, ctypes.c_double(clip))
    assert 0 < need <= _C.lib().bl_update_fixed_scratch_capacity()
    ref, got = _state(rows, cols, 5), _state(rows, cols, 5)
    scratch = torch.empty(need, dtype=torch.uint8, device=DEV)
    g = torch.Generator(device=DEV).manual_seed(6)
    for step in (1, 2):                                   # two calls in a row share the built-in array
        G = (torch.randn(rows, cols, device=DEV, generator=g) * (3.0 if direction == 0 else 1e-3)).to(torch.bfloat16)
        _call("bl_nvfp4_lattice_update", *ref, G, rows, cols, direction, clip, step, scratch)
        _call("bl_nvfp4_lattice_update_fixed_scratch", *got, G, rows, cols, direction, clip, step)
        torch.cuda.synchronize()
        for a, b in zip(ref[:3], got[:3]):
            assert torch.equal(a, b)
    assert not torch.equal(ref[0], _state(rows, cols, 5)[0])          # the updates did change the weights


def test_fixed_scratch_update_refuses_what_does_not_fit():
    rows, cols = 16384, 16384                              # 128 panels x 16384 columns of fp32 partial sums: 8 MiB
    cap = _C.lib().bl_update_fixed_scratch_capacity()
    assert _C.lib().bl_update_scratch_bytes(rows, cols, 2, ctypes.c_double(1.0)) > cap
    one = torch.zeros(16, dtype=torch.uint8, device=DEV)
    gs = torch.ones(1, device=DEV)
    with pytest.raises(RuntimeError, match="built-in scratch holds"):
        _call("bl_nvfp4_lattice_update_fixed_scratch", one, one, one, gs, torch.zeros(8, device=DEV,
              dtype=torch.bfloat16), rows, cols, 2, 1.0, 1)


def test_fixed_scratch_update_allocates_no_device_memory():
    """What the entry point is for: after the first call on the device (which looks up the built-in array's address),
    further calls leave the device's free memory and torch's allocator exactly as they were -- nothing is allocated,
    cached or freed by the library."""
    rows, cols = 384, 1024
    st = _state(rows, cols, 7)
    G = (torch.randn(rows, cols, device=DEV, generator=torch.Generator(device=DEV).manual_seed(8)) * 1e-3
         ).to(torch.bfloat16)
    _call("bl_nvfp4_lattice_update_fixed_scratch", *st, G, rows, cols, 2, 1.0, 1)        # first call: set-up
    torch.cuda.synchronize()
    before = (torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated(), torch.cuda.memory_reserved())
    for step in (2, 3, 4):
        _call("bl_nvfp4_lattice_update_fixed_scratch", *st, G, rows, cols, 2, 1.0, step)
    torch.cuda.synchronize()
    after = (torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated(), torch.cuda.memory_reserved())
    assert after == before


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fixed_scratch_update_on_a_device_that_is_not_current():
    """The array's address is per device: a call for device 1 while device 0 is current uses device 1's copy."""
    rows, cols = 256, 512
    torch.cuda.set_device(0)
    with torch.cuda.device(0):
        ref = _state(rows, cols, 9)
        G = (torch.randn(rows, cols, device=DEV, generator=torch.Generator(device=DEV).manual_seed(10)) * 1e-3
             ).to(torch.bfloat16)
        _call("bl_nvfp4_lattice_update_fixed_scratch", *ref, G, rows, cols, 2, 1.0, 1)
    other = tuple(t.to("cuda:1") for t in _state(rows, cols, 9))
    G1 = G.to("cuda:1")
    torch.cuda.synchronize(1)
    assert torch.cuda.current_device() == 0
    _call("bl_nvfp4_lattice_update_fixed_scratch", *other, G1, rows, cols, 2, 1.0, 1)
    torch.cuda.synchronize(1)
    for a, b in zip(ref[:3], other[:3]):
        assert torch.equal(a.cpu(), b.cpu())
