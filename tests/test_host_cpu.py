"""Host-side logic that needs no GPU: formats, packing, the compute policy, optimizer option checks, and that the
product fails loudly (instead of falling back) when asked to compute without a CUDA device."""
import numpy as np
import pytest
import torch

from conftest import golden

import bitlattice_b200 as bl
from bitlattice_b200 import _ops, formats as F
from bitlattice_b200.packing import pack, packed_cols, sign_extend, unpack


def cpu_weight(rows=32, cols=64, requires_grad=True):
    import oracle
    w = (torch.randn(rows, cols, generator=torch.Generator().manual_seed(0)) * 0.02).numpy()
    codes, scales, g = oracle.quantize_rows(w, None, "rtn")
    t = bl.LatticeTensor(torch.from_numpy(codes), torch.from_numpy(scales).view(torch.float8_e4m3fn),
                         torch.tensor([g]), None, "nvfp4", (rows, cols), torch.bfloat16)
    return torch.nn.Parameter(t, requires_grad=requires_grad)


def test_nvfp4_tables_match_reference_format():
    fmt = F.get("nvfp4")
    t = fmt.tables()
    assert fmt.levels == (-6.0, -4.0, -3.0, -2.0, -1.5, -1.0, -0.5, 0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
    assert t["rank"].tolist() == [7, 8, 9, 10, 11, 12, 13, 14, 7, 6, 5, 4, 3, 2, 1, 0]
    assert t["sorted_code"].tolist() == [15, 14, 13, 12, 11, 10, 9, 0, 1, 2, 3, 4, 5, 6, 7]
    assert fmt.scale.shape(8, 64) == (8, 4) and fmt.container_bits == 4
    with pytest.raises(KeyError):
        F.get("int4")
    with pytest.raises(ValueError):
        fmt.scale.groups_per_row(24)


@pytest.mark.parametrize("bits", [1, 2, 4, 8])
def test_packing_round_trip_and_layout(bits):
    g = torch.Generator().manual_seed(bits)
    codes = torch.randint(0, 1 << bits, (5, 64), generator=g, dtype=torch.int32)
    p = pack(codes, bits)
    assert p.dtype == torch.uint8 and p.shape == (5, packed_cols(64, bits))
    assert torch.equal(unpack(p, bits, 64), codes)
    if bits == 4:                                   # element 2j in the low nibble of byte j
        assert int(p[0, 0]) == int(codes[0, 0]) | (int(codes[0, 1]) << 4)
    half = 1 << (bits - 1)
    signed = torch.arange(-half, half, dtype=torch.int32)
    assert torch.equal(sign_extend(signed & ((1 << bits) - 1), bits), signed.long())
    with pytest.raises(ValueError):
        packed_cols(7, 4) if bits == 4 else packed_cols(63, bits) if bits != 8 else pack(codes, 16)


def test_packing_matches_reference_golden_phase_bytes():
    """The golden phase inputs were packed by the reference's own pack(); unpack -> pack reproduces them."""
    g = golden("step")
    for bits in (1, 2, 3, 4, 8):
        cb = _ops.phase_container(bits)
        raw = torch.from_numpy(g[f"phase_in_b{bits}"])
        assert torch.equal(pack(unpack(raw, cb, 128), cb), raw)


def test_phase_containers_and_trust_region():
    assert [_ops.phase_container(b) for b in range(9)] == [0, 1, 2, 4, 4, 8, 8, 8, 8]
    assert _ops.kappa(0.1, 1.0, 3e-3) == 3e-3 and _ops.kappa(0.1, 0.0, 3e-3) == 0.1
    assert _ops.strat_args("strat", 5, 16) == (10, 16) and _ops.strat_args("sr", 5, 16) == (0, 1)


def test_compute_policy_routes_and_requirements():
    p = cpu_weight()
    x = torch.zeros(4, 64, dtype=torch.bfloat16)
    from bitlattice_b200.compute_policy import route
    assert route(x, p)[0] == "exact"
    with bl.compute("fp4_all"):
        with pytest.raises(RuntimeError, match="not on a CUDA device"):
            route(x, p)
    assert bl.COMPUTE_PRESETS["fp4"].route == "fp4" and bl.COMPUTE_PRESETS["fp4_all"].route == "fp4_all"
    with pytest.raises(ValueError):
        bl.Compute("mxfp8")
    with pytest.raises(ValueError, match="scale_source"):
        bl.backend.Fp4Recipe(scale_source="sometimes")
    assert bl.backend.as_recipe("quartet2_delayed").scale_source == "delayed"
    with pytest.raises(ValueError, match="rotation=128"):
        bl.backend.Fp4Recipe(gradients="eden")
    with pytest.raises(ValueError, match="bound"):
        bl.backend.Fp4Recipe(dgrad_scale="bound")
    assert bl.compute_policy.as_compute("quartet2_fast").nvfp4 == bl.backend.FP4_RECIPES["quartet2_fast"]
    assert bl.compute_policy.as_compute("quartet2_fast").route == "fp4_all"
    assert not bl.backend.FP4_RECIPES["quartet2_fast"].packed_exchange and bl.backend.FP4_RECIPES["4over6"].packed_exchange
    bad = cpu_weight(rows=24, cols=64)
    assert "multiple of 32" in bl.backend.fp4_unfit(bad, 0, True)
    assert "multiple of 16" in bl.backend.fp4_unfit(bad, 0, False)


def test_no_cpu_fallback_anywhere():
    p = cpu_weight()
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        p.dequantize()
    with pytest.raises(RuntimeError, match="CUDA"):
        torch.nn.functional.linear(torch.zeros(4, 64, dtype=torch.bfloat16), p)
    with pytest.raises(RuntimeError, match="CUDA"):
        bl.LatticeTensor.from_float(torch.zeros(32, 64), "nvfp4", method="rtn")
    with pytest.raises(NotImplementedError):
        bl.LatticeTensor.from_float(torch.zeros(32, 64), "nvfp4", method="mse")


def test_optimizer_options_validated_like_the_reference():
    p = cpu_weight()
    with pytest.raises(ValueError):
        bl.Lattice([p], direction="adam")
    with pytest.raises(TypeError):
        bl.Lattice([p], direction="sign", betas=(0.9, 0.99))
    with pytest.raises(ValueError):
        bl.Lattice([p], direction="sign", phase_bits=9)
    with pytest.raises(ValueError):
        bl.Lattice([p], direction="sign", state="disk")
    with pytest.raises(KeyError):
        bl.Lattice([p], "nonexistent")
    with pytest.raises(NotImplementedError):
        bl.Lattice([p], direction="sign", state="ram")
    with pytest.raises(ValueError):
        bl.Lattice([p], direction="muon", ns_dtype="fp64")
    with pytest.raises(ValueError):
        bl.Lattice([p], vector_direction="muon")
    assert set(bl.optim.PRESETS) == {"muon", "muon_fast", "normuon", "normuon_fast", "muon_precise", "light", "balanced",
                                     "precise", "stateless"}
    with pytest.raises(NotImplementedError):
        bl.Lattice([torch.nn.Parameter(torch.zeros(4, 16))], direction="sign")
    with pytest.raises(RuntimeError, match="CUDA device"):
        bl.Lattice([p], direction="sign")              # a CPU weight cannot be updated: no CPU path


def test_lattice_tensor_container_semantics():
    p = cpu_weight(requires_grad=False)
    assert p.shape == (32, 64) and p.dtype == torch.bfloat16 and p.rows == 32 and p.cols == 64
    assert p.storage_bytes() == 32 * 32 + 32 * 4 + 4
    c = p.detach().clone()
    assert bl.is_lattice(c) and torch.equal(c.packed, p.packed) and c.packed.data_ptr() != p.packed.data_ptr()
    q = cpu_weight(requires_grad=False)
    q.packed.zero_()
    q.copy_(p)
    assert torch.equal(q.packed, p.packed) and getattr(q, "_bl_version", 0) == 1
    names, ctx = p.__tensor_flatten__()
    assert names == ["packed", "scales", "global_scale"]
    r = bl.LatticeTensor.__tensor_unflatten__(p.parts(), ctx, None, None)
    assert torch.equal(r.scales.view(torch.uint8), p.scales.view(torch.uint8))


def test_side_attributes_travel_with_views_and_copies():
    """A row shard stays a row shard through Parameter / detach / clone / to (the optimizer's RNG offset and the
    checkpoint gather read ``_bl_row_offset``); storage-sharing results also keep the weight version."""
    from bitlattice_b200.parallel import shard_rows
    from bitlattice_b200.tensor import to_parameter
    w = cpu_weight(rows=64, requires_grad=False)
    for rank in range(2):
        sh = shard_rows(w, rank, 2)
        lo = rank * 32
        assert sh._bl_row_offset == lo and sh._bl_rows_total == 64
        sh._bl_version = 3
        p = to_parameter(sh)
        assert p._bl_row_offset == lo and p._bl_version == 3
        assert torch.nn.Parameter(sh)._bl_row_offset == lo
        assert p.detach()._bl_row_offset == lo and p.detach()._bl_version == 3
        c = p.detach().clone()
        assert c._bl_row_offset == lo and not hasattr(c, "_bl_version")       # fresh storage: fresh version
        assert c._bl_rows_total == 64 and torch.nn.Parameter(sh)._bl_rows_total == 64
        assert p.detach().to(torch.float16)._bl_row_offset == lo
    assert not hasattr(to_parameter(w), "_bl_row_offset")


def test_shard_group_selects_the_whole_weight_update_and_rejects_unequal_shards(monkeypatch):
    """``Lattice(shard_group=...)``: which parameters and directions take the exchanged statistics, and the refusal of
    shards that are not equal and in rank order (raised on the host, before any library call; the constructor's
    refusal of CPU weights is switched off for this test of the host logic)."""
    from bitlattice_b200 import _ops
    from bitlattice_b200.optim.lattice import Lattice
    from bitlattice_b200.parallel import shard_rows
    monkeypatch.setattr(_ops, "cuda_ok", lambda *a: True)
    w = cpu_weight(rows=256, requires_grad=False)
    sh = torch.nn.Parameter(shard_rows(w, 1, 2))
    whole = torch.nn.Parameter(cpu_weight(rows=64, requires_grad=False))
    assert Lattice._is_shard(sh) and not Lattice._is_shard(whole)
    plain = Lattice([sh], lr=1e-3, direction="colnorm")
    assert not plain._whole_weight(plain.param_groups[0], "colnorm")
    opt = Lattice([sh], lr=1e-3, direction="colnorm", shard_group=True)
    g = opt.param_groups[0]
    assert opt._whole_weight(g, "colnorm") and opt._whole_weight(g, "raw") and not opt._whole_weight(g, "sign")
    assert opt._whole_weight({**g, "clip": 0.5}, "sign")
    opt._shard_world = lambda: (4, 1, None)          # four ranks, but the shard is one half of its weight
    with pytest.raises(RuntimeError, match="equal row shards in rank order"):
        opt._check_shards([sh])
    opt._shard_world = lambda: (2, 1, None)
    assert opt._check_shards([sh]) == (2, 1)


def test_newton_schulz_orthogonalises_and_matches_its_coefficients():
    """The polar-factor iteration on CPU tensors (pure matrix products): singular values move toward 1, the Gram
    variant agrees with the standard one, and tall inputs are handled through the transpose."""
    from bitlattice_b200.optim.directions import newton_schulz, ns_coefficients
    g = torch.randn(48, 96, generator=torch.Generator().manual_seed(0))
    x = newton_schulz(g, steps=5)
    sv = torch.linalg.svdvals(x)
    assert 0.6 < sv.min() and sv.max() < 1.3
    y = newton_schulz(g, steps=5, algo="gram")
    assert torch.allclose(x, y, atol=2e-3)
    t = newton_schulz(g.t().contiguous(), steps=5)
    assert torch.allclose(t, x.t(), atol=1e-5)
    assert ns_coefficients("muon", 3) == (3.4445, -4.7750, 2.0315)
    a, b, c = ns_coefficients("polar_express", 9)
    assert abs(a - 2.300652019954817 / 1.05) < 1e-12 and b < 0 < c
    with pytest.raises(ValueError):
        ns_coefficients("cubic", 0)


def test_an_index_offset_of_the_counter_hash_is_a_value_of_its_step():
    """``parallel.MATCH_UNSHARDED`` hands a rank's gradient columns the unsharded tensor's rounding draws through the
    quantizer's ``step`` argument: with the oracle's statement of the reference's hash (bitlattice/reference.py:22-30),
    u(index + offset, seed, 0) == u(index, seed, offset * mul / 0x85EBCA77 mod 2^32), also across the 2^32 wrap."""
    from bitlattice_b200 import parallel
    from oracle import fp4_general as G
    rng = np.random.default_rng(5)
    idx = rng.integers(0, 1 << 32, size=4096, dtype=np.uint64)
    for offset in (0, 1, 256 * 384, 3 * 65536 * 4096, (1 << 32) - 7, 5 * (1 << 32) + 11):
        step = (offset * parallel._HASH_INDEX_MUL * parallel._HASH_STEP_INV) & 0xFFFFFFFF
        for seed in (0, 77, 0x7FFFFFFF):
            assert np.array_equal(G.hash_u(idx + np.uint64(offset), seed, 0), G.hash_u(idx, seed, step))
