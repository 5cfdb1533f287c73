"""CUDA kernels (through the C ABI) against the CPU oracle and the reference's golden vectors.

Bit-exact (torch.equal) for codes, scale bytes, phase bytes and fp32 directions; the GEMM is compared with the
oracle's double-precision contraction of the dequantized operands within bf16 rounding (tolerances in the test).
"""
import numpy as np
import pytest
import torch

from conftest import golden

import oracle
from bitlattice_b200 import _ops

pytestmark = pytest.mark.gpu
DEV = "cuda"


def gen(seed):
    return torch.Generator().manual_seed(seed)


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)) if isinstance(a, np.ndarray) else a
    if dtype is not None:
        t = t.to(dtype)
    return t.to(DEV).contiguous()


def host(t):
    return t.detach().cpu().contiguous().view(torch.uint8).numpy() if t.dtype == torch.float8_e4m3fn else \
        t.detach().cpu().contiguous().numpy()


def nvfp4_weights(rows, cols, seed):
    w = (torch.randn(rows, cols, generator=gen(seed)) * 0.02).numpy()
    codes, scales, g = oracle.quantize_rows(w, None, "rtn")
    return codes, scales, float(g)


# ------------------------------------------------------------------------------------------------ lattice update

def _golden_step_names():
    return [str(n) for n in golden("step")["names"]]


@pytest.mark.parametrize("name", _golden_step_names())
def test_step_quantized_matches_reference_golden(name):
    g = golden("step")
    bits = int(name.split("_")[0][1:])
    rule = "fit_latent" if "fit_latent" in name else name.split("_")[1]
    rounding = name.split("_")[-1]
    trust_lr = 1.0 if rounding == "sr" else 0.0
    packed = dev(g["codes"])
    phase = dev(g[f"phase_in_b{bits}"]) if bits else None
    fmt = "nvfp4"
    scales = _ops.step_quantized(packed, phase, dev(g["scales"]), dev(g["g"]), None, dev(g["D"]), fmt, 16, 128,
                                 lr=float(g["lr"][0]), weight_decay=0.01, phase_bits=bits,
                                 phase_cb=_ops.phase_container(bits), rounding=rounding, seed=7, step=3, strata=16,
                                 scale_rule=rule, trust=0.1 if trust_lr == 0.0 else 0.01, trust_lr=trust_lr)
    assert np.array_equal(host(scales), g[name + "_scales"])
    assert np.array_equal(host(packed), g[name + "_codes"])
    if bits:
        assert np.array_equal(host(phase), g[name + "_phase"])


@pytest.mark.parametrize("bits", [0, 1, 2, 3, 4, 5, 8])
@pytest.mark.parametrize("rule", ["fixed", "fit", "fit_latent"])
def test_step_quantized_matches_oracle(bits, rule):
    rows, cols = 96, 272                       # cols/8 = 34 chunks: ragged against the 32-wide thread rows
    codes, scales, g = nvfp4_weights(rows, cols, 1)
    cb = _ops.phase_container(bits)
    half = 1 << max(bits - 1, 0)
    ph = None
    if bits:
        from bitlattice_b200.packing import pack
        raw = torch.randint(-half, half, (rows, cols), generator=gen(2 + bits), dtype=torch.int32)
        ph = pack(raw & ((1 << bits) - 1), cb).numpy()
    D = torch.randn(rows, cols, generator=gen(3)).numpy()
    se = oracle.e4m3_decode(scales).mean() * g
    kw = dict(lr=0.3 * float(se), weight_decay=0.01, phase_bits=bits, rounding="sr", seed=7, step=3,
              scale_rule=rule, trust=0.1, trust_lr=0.0)
    rc, rp, rs = oracle.lattice_step(codes, ph, scales, g, D, offset=12345, **kw)
    packed, phase = dev(codes), (dev(ph) if bits else None)
    new_scales = _ops.step_quantized(packed, phase, dev(scales), dev(np.array([g], np.float32)), None, dev(D), "nvfp4",
                                     rows, cols, phase_cb=cb, strata=16, offset=12345, **kw)
    assert np.array_equal(host(new_scales), rs)
    assert np.array_equal(host(packed), rc)
    if bits:
        assert np.array_equal(host(phase), rp)
    if rule != "fixed":
        assert (rs != scales).mean() > 0.05          # the refit is exercised


@pytest.mark.parametrize("bits", [1, 2, 4, 8])
def test_update_at_exact_ties_matches_oracle(bits):
    """Phase codes of -half with a zero gradient put every target exactly half-way between two levels: the kernel
    finds the nearest level with the hardware conversion (ties to even), the reference with ties to the lower level;
    the projected (code, phase) must agree all the same. Mixed with +max phase codes and a few non-zero gradients."""
    from bitlattice_b200.packing import pack
    rows, cols = 64, 256
    codes, scales, g = nvfp4_weights(rows, cols, 13)
    half = 1 << (bits - 1)
    raw = torch.full((rows, cols), -half, dtype=torch.int32)
    raw[::3] = half - 1
    cb = _ops.phase_container(bits)
    ph = pack(raw & ((1 << bits) - 1), cb).numpy()
    D = torch.zeros(rows, cols)
    D[::5, ::7] = torch.randn(rows, cols, generator=gen(14))[::5, ::7]
    for rule in ("fixed", "fit"):
        kw = dict(lr=1e-3, weight_decay=0.0, phase_bits=bits, rounding="sr", seed=3, step=2, scale_rule=rule, trust=0.1,
                  trust_lr=0.0)
        rc, rp, rs = oracle.lattice_step(codes, ph, scales, g, D.numpy(), **kw)
        packed, phase = dev(codes), dev(ph)
        new_scales = _ops.step_quantized(packed, phase, dev(scales), dev(np.array([g], np.float32)), None, dev(D),
                                         "nvfp4", rows, cols, phase_cb=cb, strata=16, **kw)
        assert np.array_equal(host(new_scales), rs)
        assert np.array_equal(host(packed), rc)
        assert np.array_equal(host(phase), rp)


@pytest.mark.parametrize("direction", ["sign", "raw", "colnorm"])
@pytest.mark.parametrize("clip", [1.0, 0.25])
@pytest.mark.parametrize("gdtype", [torch.bfloat16, torch.float32])
def test_fused_update_matches_oracle(direction, clip, gdtype):
    rows, cols = 300, 512                       # three row panels of the column statistics, the last one short
    codes, scales, g = nvfp4_weights(rows, cols, 4)
    G = (torch.randn(rows, cols, generator=gen(5)) * (3.0 if direction == "raw" else 1e-3)).to(gdtype)
    G[3, 5] = 0.0
    D, (rho, div) = oracle.direction(G.float().numpy(), direction, clip)
    kw = dict(lr=3e-3, weight_decay=0.0, phase_bits=4, rounding="sr", seed=1234, step=1, scale_rule="fit", trust=0.1,
              trust_lr=0.0)
    ph0 = np.zeros((rows, cols // 2), np.uint8)
    rc, rp, rs = oracle.lattice_step(codes, ph0, scales, g, D, **kw)
    packed, phase, sc = dev(codes), dev(ph0), dev(scales)
    _ops.lattice_update(packed, phase, sc, dev(np.array([g], np.float32)), None, dev(G), "nvfp4", rows, cols,
                        phase_cb=4, strata=16, direction=direction, clip=clip, **kw)
    assert np.array_equal(host(sc), rs)
    assert np.array_equal(host(packed), rc)
    assert np.array_equal(host(phase), rp)
    # and the direction operator on its own, bit for bit
    Dg = _ops.direction(dev(G), direction, clip=clip)
    assert np.array_equal(host(Dg), D)


@pytest.mark.parametrize("direction", ["sign", "raw", "colnorm"])
@pytest.mark.parametrize("clip", [1.0, 0.25])
def test_fused_update_with_extreme_gradient_values(direction, clip):
    """Zeros (single, a whole row, a whole column), values next to and inside the subnormal range, and very large
    values: the groups that hold them leave the range in which the update's unchecked divisions are exact and take
    the general route; results stay bit-identical to the oracle's, for those groups and for their neighbours."""
    rows, cols = 200, 256
    codes, scales, g = nvfp4_weights(rows, cols, 44)
    G = torch.randn(rows, cols, generator=gen(45)) * 1e-3
    G[3, 5] = 0.0
    G[7] = 0.0
    G[:, 33] = 0.0
    G[11, 64:80] = torch.tensor([1e-30, -1e-38, 1e-42, -1e-45, 3e-39, 1e-20, -1e-25, 2e-33] * 2)
    G[13, 100] = 1e15
    G[17, 200] = -3e12
    G[19, 16:32] = 1e-12
    D, _ = oracle.direction(G.numpy(), direction, clip)
    kw = dict(lr=3e-3, weight_decay=0.0, phase_bits=4, rounding="sr", seed=77, step=5, scale_rule="fit", trust=0.1,
              trust_lr=0.0)
    ph0 = np.zeros((rows, cols // 2), np.uint8)
    rc, rp, rs = oracle.lattice_step(codes, ph0, scales, g, D, **kw)
    packed, phase, sc = dev(codes), dev(ph0), dev(scales)
    _ops.lattice_update(packed, phase, sc, dev(np.array([g], np.float32)), None, dev(G), "nvfp4", rows, cols,
                        phase_cb=4, strata=16, direction=direction, clip=clip, **kw)
    assert np.array_equal(host(sc), rs)
    assert np.array_equal(host(packed), rc)
    assert np.array_equal(host(phase), rp)


@pytest.mark.parametrize("lr,wd", [(1e-12, 0.0), (300.0, 0.0), (3e-3, 0.3)])
def test_fused_update_with_unusual_step_sizes(lr, wd):
    """Learning rates outside the fast route's window (every group takes the general route) and a weight decay."""
    rows, cols = 64, 128
    codes, scales, g = nvfp4_weights(rows, cols, 46)
    G = (torch.randn(rows, cols, generator=gen(47)) * 1e-3).to(torch.bfloat16)
    D, _ = oracle.direction(G.float().numpy(), "colnorm", 1.0)
    kw = dict(lr=lr, weight_decay=wd, phase_bits=4, rounding="sr", seed=5, step=1, scale_rule="fit", trust=0.1,
              trust_lr=0.0)
    ph0 = np.zeros((rows, cols // 2), np.uint8)
    rc, rp, rs = oracle.lattice_step(codes, ph0, scales, g, D, **kw)
    packed, phase, sc = dev(codes), dev(ph0), dev(scales)
    _ops.lattice_update(packed, phase, sc, dev(np.array([g], np.float32)), None, dev(G), "nvfp4", rows, cols,
                        phase_cb=4, strata=16, direction="colnorm", clip=1.0, **kw)
    assert np.array_equal(host(sc), rs) and np.array_equal(host(packed), rc) and np.array_equal(host(phase), rp)


@pytest.mark.parametrize("bits", [1, 2, 3, 4, 6, 7, 8])
@pytest.mark.parametrize("rule", ["fixed", "fit", "fit_latent"])
def test_fused_update_matches_oracle_for_every_phase_width(bits, rule):
    """Two steps from a random phase state: 1..7 bits run the packed fast route, 8 bits the general one."""
    from bitlattice_b200.packing import pack
    rows, cols = 96, 256
    codes, scales, g = nvfp4_weights(rows, cols, 50 + bits)
    cb = _ops.phase_container(bits)
    raw = torch.randint(0, 1 << bits, (rows, cols), generator=gen(60 + bits), dtype=torch.int32)
    phase = pack(raw, cb).numpy()
    packed, ph, sc = dev(codes), dev(phase), dev(scales)
    gs = dev(np.array([g], np.float32))
    for step in (1, 2):
        G = (torch.randn(rows, cols, generator=gen(70 + step)) * 1e-3).to(torch.bfloat16)
        D, _ = oracle.direction(G.float().numpy(), "colnorm", 1.0)
        kw = dict(lr=3e-2, weight_decay=0.01, phase_bits=bits, rounding="sr", seed=9, step=step, scale_rule=rule,
                  trust=0.1, trust_lr=0.0)
        codes, phase, scales = oracle.lattice_step(codes, phase, scales, g, D, **kw)
        _ops.lattice_update(packed, ph, sc, gs, None, dev(G), "nvfp4", rows, cols, phase_cb=cb, strata=16,
                            direction="colnorm", clip=1.0, **kw)
        assert np.array_equal(host(sc), scales) and np.array_equal(host(packed), codes)
        assert np.array_equal(host(ph), phase)


@pytest.mark.parametrize("direction,clip", [("colnorm", 1.0), ("sign", 1.0), ("raw", 0.5)])
def test_update_many_equals_one_call_per_tensor(direction, clip):
    """bl_nvfp4_lattice_update_many packs its tensors into batches that share every launch; with ample scratch (full
    batches of 40), with the minimum (a batch closes early) and tensor by tensor the results are identical."""
    shapes = [(32, 64), (128, 256), (300, 512), (16, 16), (257, 1024)] * 9 + [(64, 4096)]          # 46 tensors
    def fresh():
        items = []
        for i, (r, c) in enumerate(shapes):
            codes, scales, g = nvfp4_weights(r, c, 100 + (i % 5))
            G = (torch.randn(r, c, generator=gen(200 + i)) * (3.0 if direction == "raw" else 1e-3)).to(torch.bfloat16)
            items.append(dict(packed=dev(codes), phase=torch.zeros(r, c // 2, dtype=torch.uint8, device=DEV),
                              scales=dev(scales), global_scale=dev(np.array([g], np.float32)), grad=dev(G), rows=r,
                              cols=c, offset=i * 1000, seed=11 + i, step=1 + i % 3))
        return items
    kw = dict(lr=3e-3, weight_decay=0.0, phase_bits=4, phase_cb=4, rounding="sr", strata=16, scale_rule="fit", trust=0.1,
              trust_lr=0.0, direction=direction, clip=clip)
    one = fresh()
    for it in one:
        _ops.lattice_update(it["packed"], it["phase"], it["scales"], it["global_scale"], None, it["grad"], "nvfp4",
                            it["rows"], it["cols"], seed=it["seed"], step=it["step"], offset=it["offset"], **kw)
    full = fresh()
    _ops.lattice_update_many(full, "nvfp4", **kw)
    tight = fresh()
    need = max(_ops.update_scratch_bytes(r, c, direction, clip) for r, c in shapes)
    scratch = torch.empty(max(need, 16), dtype=torch.uint8, device=DEV) if need else None
    _ops.lattice_update_many(tight, "nvfp4", scratch=scratch, **kw)
    for a, b, c in zip(one, full, tight):
        for k in ("packed", "phase", "scales"):
            assert torch.equal(a[k], b[k]) and torch.equal(a[k], c[k]), (k, a["rows"], a["cols"])


@pytest.mark.parametrize("direction", ["colnorm", "sign", "raw"])
@pytest.mark.parametrize("bits,wd,lr", [(4, 0.0, 3e-3), (4, 0.01, 3e-2), (7, 0.01, 3e-2), (2, 0.1, 1e-1)])
def test_update_routes_agree_at_scale(direction, bits, wd, lr):
    """The fast route of the update kernel (packed pairs, one range check per element) against its general route on
    16.7 M weights with a random phase state: identical codes, phase and scale bytes. (With a weight decay and a large
    step every product feeds a sum with cancellation: a single contracted multiply-add would show here.)"""
    rows, cols = 4096, 4096
    dg = lambda s: torch.Generator(device=DEV).manual_seed(s)
    w = torch.randn(rows, cols, device=DEV, generator=dg(0)) * 0.02
    gs = _ops.amax_global(w)[1:2].clone()
    packed0, scales0 = _ops.quantize_nvfp4(w, gs)
    cb = _ops.phase_container(bits)
    per = 8 // cb
    vals = torch.randint(0, 1 << bits, (rows, cols // per, per), device=DEV, dtype=torch.int32, generator=dg(1))
    phase0 = sum(vals[..., j] << (cb * j) for j in range(per)).to(torch.uint8)
    G = (torch.randn(rows, cols, device=DEV, generator=dg(2)) * (3.0 if direction == "raw" else 1e-3)).to(torch.bfloat16)
    out = {}
    try:
        for route in ("general", "auto"):
            _ops.update_select(route)
            st = [packed0.clone(), phase0.clone(), scales0.view(torch.uint8).clone()]
            _ops.lattice_update(st[0], st[1], st[2], gs, None, G, "nvfp4", rows, cols, lr=lr, weight_decay=wd,
                                phase_bits=bits, phase_cb=cb, rounding="sr", seed=9, step=1, strata=16,
                                scale_rule="fit", trust=0.1, trust_lr=0.0, direction=direction, clip=1.0)
            out[route] = st
    finally:
        _ops.update_select("auto")
    for a, b in zip(out["general"], out["auto"]):
        assert torch.equal(a, b)
    assert not torch.equal(out["auto"][0], packed0)


def test_direction_close_to_reference_golden():
    g = golden("direction")
    for kind in ("raw", "sign", "colnorm"):
        for clip in (1.0, 0.25):
            D = host(_ops.direction(dev(g["G"], torch.bfloat16), kind, clip=clip))
            ref = g[f"{kind}_clip{clip}"]
            if kind == "sign" and clip >= 1.0:
                assert np.array_equal(D, ref)
            else:
                np.testing.assert_allclose(D, ref, rtol=4e-7, atol=0.0)


def test_row_shards_reproduce_the_whole_update():
    """A row shard updated with offset = first_row * cols equals the same rows of the unsharded update
    (the reference's row tiles, csrc/update.cpp:50; the N-sharded layers rely on it)."""
    rows, cols = 256, 1024
    codes, scales, g = nvfp4_weights(rows, cols, 6)
    G = (torch.randn(rows, cols, generator=gen(7)) * 1e-3).to(torch.bfloat16)
    gs = dev(np.array([g], np.float32))
    kw = dict(lr=3e-3, weight_decay=0.0, phase_bits=4, phase_cb=4, rounding="sr", seed=99, step=2, strata=16,
              scale_rule="fit", trust=0.1, trust_lr=0.0, direction="sign")
    whole = [dev(codes), dev(np.zeros((rows, cols // 2), np.uint8)), dev(scales)]
    _ops.lattice_update(whole[0], whole[1], whole[2], gs, None, dev(G), "nvfp4", rows, cols, **kw)
    for r0, r1 in ((0, 64), (64, 256)):
        part = [dev(codes[r0:r1]), dev(np.zeros((r1 - r0, cols // 2), np.uint8)), dev(scales[r0:r1])]
        _ops.lattice_update(part[0], part[1], part[2], gs, None, dev(G[r0:r1]), "nvfp4", r1 - r0, cols,
                            offset=r0 * cols, **kw)
        for a, b in zip(part, whole):
            assert torch.equal(a, b[r0:r1])


def test_update_rejects_bad_arguments():
    codes, scales, g = nvfp4_weights(16, 64, 8)
    gs = dev(np.array([g], np.float32))
    kw = dict(lr=1e-3, weight_decay=0.0, phase_bits=0, phase_cb=0, rounding="sr", seed=0, step=1, strata=16,
              scale_rule="fit", trust=0.1, trust_lr=0.0)
    with pytest.raises(RuntimeError, match="multiple of 16"):
        _ops.lattice_update(dev(codes)[:, :28].contiguous(), None, dev(scales), gs, None,
                            torch.zeros(16, 56, device=DEV, dtype=torch.bfloat16), "nvfp4", 16, 56,
                            direction="sign", **kw)
    with pytest.raises(RuntimeError, match="outside this build"):
        _ops.lattice_update(dev(codes), None, dev(scales), gs, None,
                            torch.zeros(16, 64, device=DEV, dtype=torch.bfloat16), "nvfp4", 16, 64,
                            direction="muon", **kw)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        _ops.lattice_update(torch.from_numpy(codes), None, dev(scales), gs, None,
                            torch.zeros(16, 64, device=DEV, dtype=torch.bfloat16), "nvfp4", 16, 64,
                            direction="sign", **kw)


# ------------------------------------------------------------------------------------------------ quantizers

def test_activation_quantizer_matches_reference_golden():
    g = golden("quantize")
    x = dev(g["rtn_x"])                 # fp32: the tie row is not representable in bf16
    am = _ops.amax_global(x)
    assert host(am)[1] == g["rtn_g"][0]
    packed, scales = _ops.quantize_nvfp4(x, am[1:2])
    assert np.array_equal(host(scales), g["rtn_scales"])
    assert np.array_equal(host(packed), g["rtn_codes"])
    deq = _ops.dequantize(packed, scales, am[1:2].clone(), None, "nvfp4", 32, 128, torch.float32)
    assert np.array_equal(host(deq), g["rtn_deq_f32"])
    deq16 = _ops.dequantize(packed, scales, am[1:2].clone(), None, "nvfp4", 32, 128, torch.bfloat16)
    assert np.array_equal(host(deq16.view(torch.int16)), g["rtn_deq_bf16"])
    for seed in (1, 77):
        gy = dev(g["sr_x"], torch.bfloat16)
        am = _ops.amax_global(gy)
        assert host(am)[1] == g[f"sr{seed}_g"][0]
        packed, scales = _ops.quantize_nvfp4(gy, am[1:2], seed=seed)
        assert np.array_equal(host(scales), g[f"sr{seed}_scales"])
        assert np.array_equal(host(packed), g[f"sr{seed}_codes"])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
@pytest.mark.parametrize("mode", ["rtn", "sr"])
def test_row_quantizer_matches_oracle(dtype, mode):
    rows, cols = 77, 1040
    x = (torch.randn(rows, cols, generator=gen(10)) * (1.0 if mode == "rtn" else 1e-2)).to(dtype)
    x[5, 32:48] = 0.0
    xf = x.float().numpy()
    rc, rs, g = oracle.quantize_rows(xf, None, mode, seed=31)
    am = _ops.amax_global(dev(x))
    assert host(am)[0] == np.abs(xf).max() and host(am)[1] == g
    packed, scales = _ops.quantize_nvfp4(dev(x), am[1:2], seed=31 if mode == "sr" else -1)
    assert np.array_equal(host(scales), rs)
    assert np.array_equal(host(packed), rc)
    packed_b, blocked = _ops.quantize_nvfp4(dev(x), am[1:2], seed=31 if mode == "sr" else -1, blocked=True)
    assert torch.equal(packed_b, packed)
    assert np.array_equal(host(blocked), oracle.to_blocked(rs))
    assert np.array_equal(host(_ops.to_blocked(scales.view(torch.uint8))), oracle.to_blocked(rs))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
@pytest.mark.parametrize("select", ["mse", "mae"])
def test_four_over_six_quantizer_matches_oracle(dtype, select):
    rows, cols = 77, 1040
    x = torch.randn(rows, cols, generator=gen(12)).to(dtype)
    x[5, 32:48] = 0.0
    xf = x.float().numpy()
    rc, rs, g = oracle.quantize_rows_fos(xf, None, select)
    am = _ops.amax_global(dev(x))
    assert host(am)[3] == g
    packed, scales = _ops.quantize_nvfp4_4over6(dev(x), am[3:4], select)
    assert np.array_equal(host(scales), rs)
    assert np.array_equal(host(packed), rc)
    packed_b, blocked = _ops.quantize_nvfp4_4over6(dev(x), am[3:4], select, blocked=True)
    assert torch.equal(packed_b, packed)
    assert np.array_equal(host(blocked), oracle.to_blocked(rs))


def test_four_over_six_quantizer_matches_reference_golden():
    g = golden("fos")
    for tag in ("bf", "f32"):
        for select in ("mse", "mae"):
            x = dev(g[f"{tag}_x"], torch.bfloat16 if tag == "bf" else torch.float32)
            packed, scales = _ops.quantize_nvfp4_4over6(x, dev(g[f"{tag}_{select}_g"]), select)
            assert np.array_equal(host(packed), g[f"{tag}_{select}_codes"])
            assert np.array_equal(host(scales), g[f"{tag}_{select}_scales"])


def test_blocked_layout_matches_reference_golden():
    g = golden("quantize")
    assert np.array_equal(host(_ops.to_blocked(dev(g["blk_in"]))), g["blk_out"])


@pytest.mark.parametrize("rot", ["rot", "plain"])
@pytest.mark.parametrize("mode", ["rtn", "sr"])
def test_transposed_quantizer_matches_reference_golden(rot, mode):
    g = golden("transposed")
    x = dev(g["t_x"], torch.bfloat16)
    H = dev(g["H16"]) if rot == "rot" else None
    packed, scales, gout = _ops.quantize_nvfp4_t(x, H, 9 if mode == "sr" else -1, 0, dev(g["t_bound"]))
    assert host(gout)[0] == np.float32(oracle.global_from_bound(float(g["t_bound"][0])))
    assert np.array_equal(host(scales), g[f"t_{rot}_{mode}_scales"])
    assert np.array_equal(host(packed), g[f"t_{rot}_{mode}_codes"])


@pytest.mark.parametrize("mode", ["rtn", "sr"])
def test_transposed_quantizer_matches_oracle_ragged(mode):
    M, K = 208, 200                                   # neither a multiple of the 128 x 64 staging tile
    x = (torch.randn(M, K, generator=gen(11)) * 1e-2).to(torch.bfloat16)
    x[::7, ::3] *= 1e-6                 # blocks with a wide exponent spread take the sequential rotation
    x[5, :] = 0.0
    H = oracle.hadamard16()
    bound = oracle.global_from_amax(float(x.float().abs().max())) * 4.0
    g = oracle.global_from_bound(bound)
    rc, rs = oracle.quantize_t(x.float().numpy(), H, g, mode, seed=5)
    packed, scales, gout = _ops.quantize_nvfp4_t(dev(x), dev(H), 5 if mode == "sr" else -1, 0,
                                                 dev(np.array([bound], np.float32)))
    assert host(gout)[0] == np.float32(g)
    assert np.array_equal(host(scales), rs)
    assert np.array_equal(host(packed), rc)
    _, blocked, _ = _ops.quantize_nvfp4_t(dev(x), dev(H), 5 if mode == "sr" else -1, 0,
                                          dev(np.array([bound], np.float32)), blocked=True)
    assert np.array_equal(host(blocked), oracle.to_blocked(rs))
    # without a bound the scale comes from an amax pass over the rotated tensor
    packed2, scales2, g2 = _ops.quantize_nvfp4_t(dev(x), dev(H), -1, 0, None)
    assert 0 < host(g2)[0] <= np.float32(g)


def test_weight_transpose_requantization():
    g = golden("transposed")
    packed, scales, gout = _ops.requantize_nvfp4_t(dev(g["w_codes"]), dev(g["w_scales"]), dev(g["w_g"]))
    assert host(gout)[0] == g["w_g"][0]
    assert np.array_equal(host(scales), g["wt_scales"])
    assert np.array_equal(host(packed), g["wt_codes"])
    codes, sc, gs = nvfp4_weights(208, 160, 12)
    rc, rs = oracle.requantize_t(codes, sc, gs)
    packed, scales, _ = _ops.requantize_nvfp4_t(dev(codes), dev(sc), dev(np.array([gs], np.float32)))
    assert np.array_equal(host(scales), rs) and np.array_equal(host(packed), rc)


def test_quantizers_index_beyond_2_31_elements():
    """Size-independent property at a tensor of 2^31 + 2^27 elements: round-to-nearest quantization is local to rows
    (row operand) and to 16-row blocks (transposed operand), so quantizing the two halves of the rows separately with
    the same per-tensor scale reproduces the whole, bit for bit -- which it would not if an index wrapped at 32
    bits."""
    M, K = 139264, 16384
    x = torch.empty(M, K, device=DEV, dtype=torch.bfloat16)
    gen = torch.Generator(device=DEV).manual_seed(9)
    for r0 in range(0, M, 8192):                                   # filled in slabs to bound temporary memory
        x[r0:r0 + 8192] = torch.randn(8192, K, device=DEV, generator=gen).to(torch.bfloat16)
    g = _ops.amax_global(x)[1:2]
    h = M // 2
    codes, sf = _ops.quantize_nvfp4(x, g)
    for lo in (0, h):
        c2, s2 = _ops.quantize_nvfp4(x[lo:lo + h], g)
        assert torch.equal(codes[lo:lo + h], c2) and torch.equal(sf.view(torch.uint8)[lo:lo + h], s2.view(torch.uint8))
    assert int(codes[-1].max()) > 0
    del codes, sf, c2, s2
    from bitlattice_b200.backend import _hadamard16
    H = _hadamard16(torch.device(DEV), torch.float32)
    tc, ts, _ = _ops.quantize_nvfp4_t(x, H, -1, 0, g * 4.0)
    for lo in (0, h):
        c2, s2, _ = _ops.quantize_nvfp4_t(x[lo:lo + h], H, -1, 0, g * 4.0)
        assert torch.equal(tc[:, lo // 2:(lo + h) // 2], c2)
        assert torch.equal(ts.view(torch.uint8)[:, lo // 16:(lo + h) // 16], s2.view(torch.uint8))


# ------------------------------------------------------------------------------------------------ GEMM

def _operand(rows, K, seed, scale):
    x = (torch.randn(rows, K, generator=gen(seed)) * scale).numpy()
    codes, sf, g = oracle.quantize_rows(x, None, "rtn")
    return codes, sf, float(g)


@pytest.fixture
def gemm_kernel(request):
    """Runs a test once per GEMM kernel (the library's own choice included) and restores the choice afterwards."""
    _ops.gemm_select(request.param)
    yield request.param
    _ops.gemm_select("auto")


ALL_GEMM_KERNELS = pytest.mark.parametrize("gemm_kernel", ["auto", "tile", "persistent", "pair"], indirect=True)


@ALL_GEMM_KERNELS
@pytest.mark.parametrize("M,N,K", [(128, 128, 256), (128, 128, 64), (256, 384, 1024), (100, 136, 96), (48, 64, 128),
                                   (1, 8, 32), (300, 520, 2048), (520, 264, 352)])
def test_gemm_matches_oracle(M, N, K, gemm_kernel):
    """Tolerance: the tensor core accumulates exact E2M1 x E2M1 x UE4M3 x UE4M3 products in fp32 and the result is
    rounded once to bf16 -> every element within 2^-8 relative (one bf16 ulp) of the double-precision contraction,
    plus an absolute term for cancellation inside the fp32 accumulation."""
    ac, asf, ga = _operand(M, K, 20, 1.0)
    bc, bsf, gb = _operand(N, K, 21, 0.02)
    ref = oracle.gemm_nt(ac, asf, ga, bc, bsf, gb)
    y = _ops.nvfp4_gemm(dev(ac), _ops.to_blocked(dev(asf)), dev(np.array([ga], np.float32)), dev(bc),
                        _ops.to_blocked(dev(bsf)), dev(np.array([gb], np.float32)))
    assert _ops.gemm_status(0) == 0
    got = y.float().cpu().numpy()
    scale = np.abs(ref).max()
    assert np.all(np.abs(got - ref) <= 2.0 ** -8 * np.abs(ref) + 2e-5 * scale), \
        float(np.abs(got - ref).max() / scale)
    yf = _ops.nvfp4_gemm(dev(ac), _ops.to_blocked(dev(asf)), dev(np.array([ga], np.float32)), dev(bc),
                         _ops.to_blocked(dev(bsf)), dev(np.array([gb], np.float32)), out_dtype=torch.float32)
    np.testing.assert_allclose(yf.cpu().numpy(), ref, rtol=2e-5, atol=2e-5 * scale)


def test_gemm_kernels_agree_bit_for_bit():
    """All kernels accumulate each output element over K in the same order on the same tensor-core path, so their
    outputs are identical, ragged edges and a K that is not a multiple of the 256-element stage included."""
    M, N, K = 2304 + 72, 2560 + 40, 1024 + 96
    g0 = torch.Generator(device=DEV).manual_seed(3)
    a = torch.randint(0, 256, (M, K // 2), device=DEV, dtype=torch.uint8, generator=g0)
    b = torch.randint(0, 256, (N, K // 2), device=DEV, dtype=torch.uint8, generator=g0)
    asf = _ops.to_blocked(torch.randint(40, 72, (M, K // 16), device=DEV, dtype=torch.uint8, generator=g0))
    bsf = _ops.to_blocked(torch.randint(40, 72, (N, K // 16), device=DEV, dtype=torch.uint8, generator=g0))
    one = torch.ones(1, device=DEV)
    outs = {}
    try:
        for name in ("tile", "persistent", "pair"):
            _ops.gemm_select(name)
            outs[name] = _ops.nvfp4_gemm(a, asf, one, b, bsf, one, out_dtype=torch.float32)
    finally:
        _ops.gemm_select("auto")
    assert _ops.gemm_status(0) == 0
    assert torch.equal(outs["tile"], outs["persistent"]) and torch.equal(outs["tile"], outs["pair"])
    assert torch.isfinite(outs["tile"]).all() and outs["tile"].abs().max() > 0


@ALL_GEMM_KERNELS
def test_gemm_on_reused_addresses_with_changing_shapes(gemm_kernel):
    """The library keeps encoded tensor maps per (address, shape, box). Operands of different shapes that start at
    the same addresses (slices of one allocation, as torch's caching allocator hands out) must each get their own map:
    every product equals the one computed from freshly allocated copies of the operands."""
    g0 = torch.Generator(device=DEV).manual_seed(9)
    pool_a = torch.randint(0, 256, (1 << 21,), device=DEV, dtype=torch.uint8, generator=g0)
    pool_b = torch.randint(0, 256, (1 << 21,), device=DEV, dtype=torch.uint8, generator=g0)
    pool_sa = torch.randint(40, 72, (1 << 19,), device=DEV, dtype=torch.uint8, generator=g0)
    pool_sb = torch.randint(40, 72, (1 << 19,), device=DEV, dtype=torch.uint8, generator=g0)
    one = torch.ones(1, device=DEV)
    _ops.gemm_select(gemm_kernel)
    try:
        for _ in range(2):                                                  # second round: every map comes from the cache
            for M, N, K in [(512, 768, 1024), (768, 512, 1024), (512, 768, 512), (1024, 384, 2048), (512, 768, 1024)]:
                a, b = pool_a[:M * K // 2].view(M, K // 2), pool_b[:N * K // 2].view(N, K // 2)
                sa = pool_sa[:_ops.blocked_scale_bytes(M, K // 16)]
                sb = pool_sb[:_ops.blocked_scale_bytes(N, K // 16)]
                got = _ops.nvfp4_gemm(a, sa, one, b, sb, one, out_dtype=torch.float32)
                want = _ops.nvfp4_gemm(a.clone(), sa.clone(), one, b.clone(), sb.clone(), one, out_dtype=torch.float32)
                assert torch.equal(got, want), (M, N, K)
    finally:
        _ops.gemm_select("auto")
    assert _ops.gemm_status(0) == 0


@ALL_GEMM_KERNELS
def test_gemm_is_linear_in_row_blocks_at_scale(gemm_kernel):
    """Size-independent property at a layer-sized problem: the product of stacked operands is the stack of products
    (bit for bit: tiles never mix rows), and equal inputs give equal outputs."""
    M, N, K = 2048, 3072, 4096
    g0 = torch.Generator(device=DEV).manual_seed(0)
    a = torch.randint(0, 256, (M, K // 2), device=DEV, dtype=torch.uint8, generator=g0)
    b = torch.randint(0, 256, (N, K // 2), device=DEV, dtype=torch.uint8, generator=g0)
    asf = torch.randint(40, 72, (M, K // 16), device=DEV, dtype=torch.uint8, generator=g0)
    bsf = torch.randint(40, 72, (N, K // 16), device=DEV, dtype=torch.uint8, generator=g0)
    one = torch.ones(1, device=DEV)
    full = _ops.nvfp4_gemm(a, _ops.to_blocked(asf), one, b, _ops.to_blocked(bsf), one)
    again = _ops.nvfp4_gemm(a, _ops.to_blocked(asf), one, b, _ops.to_blocked(bsf), one)
    assert torch.equal(full, again)
    top = _ops.nvfp4_gemm(a[:1024].contiguous(), _ops.to_blocked(asf[:1024].contiguous()), one, b,
                          _ops.to_blocked(bsf), one)
    assert torch.equal(top, full[:1024])
    right = _ops.nvfp4_gemm(a, _ops.to_blocked(asf), one, b[1024:].contiguous(),
                            _ops.to_blocked(bsf[1024:].contiguous()), one)
    assert torch.equal(right, full[:, 1024:])
    assert _ops.gemm_status(0) == 0
    assert torch.isfinite(full.float()).all() and full.float().abs().max() > 0


@ALL_GEMM_KERNELS
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_gemm_accumulate_equals_adding_the_tensors(gemm_kernel, dtype):
    """out += product in the epilogue gives the bits of torch's `out + product` (the product rounded to the output type
    first), on full tiles and on ragged edges (N not a multiple of 32, rows not a multiple of 128)."""
    for M, N, K in ((256, 512, 256), (300, 520, 320)):
        g0 = torch.Generator(device=DEV).manual_seed(5)
        a = torch.randint(0, 256, (M, K // 2), device=DEV, dtype=torch.uint8, generator=g0)
        b = torch.randint(0, 256, (N, K // 2), device=DEV, dtype=torch.uint8, generator=g0)
        asf = _ops.to_blocked(torch.randint(40, 72, (M, K // 16), device=DEV, dtype=torch.uint8, generator=g0))
        bsf = _ops.to_blocked(torch.randint(40, 72, (N, K // 16), device=DEV, dtype=torch.uint8, generator=g0))
        one = torch.full((1,), 1e-3, device=DEV)
        base = (torch.randn(M, N, device=DEV, generator=g0) * 50).to(dtype)
        prod = _ops.nvfp4_gemm(a, asf, one, b, bsf, one, out_dtype=dtype)
        out = base.clone()
        _ops.nvfp4_gemm(a, asf, one, b, bsf, one, out=out, accumulate=True)
        assert torch.equal(out, base + prod)
    assert _ops.gemm_status(0) == 0


def test_gemm_rejects_bad_shapes():
    one = torch.ones(1, device=DEV)
    a = torch.zeros(16, 24, device=DEV, dtype=torch.uint8)      # K = 48
    sf = torch.zeros(512, device=DEV, dtype=torch.uint8)
    with pytest.raises(RuntimeError, match="multiple of 32"):
        _ops.nvfp4_gemm(a, sf, one, a, sf, one)


def test_shared_reciprocal_division_is_exact():
    """The kernels' division routine (shared correctly-rounded reciprocal + two fused corrections) equals the plain
    fp32 division bit for bit on 2^30 pseudo-random operand pairs."""
    import ctypes
    from bitlattice_b200 import _C
    bad = ctypes.c_uint64(1)
    for seed in (1, 77777):
        _C.call("bl_selftest_division", 1 << 29, seed, ctypes.byref(bad), 0)
        assert bad.value == 0


@pytest.mark.parametrize("p,N,K", [(2, 512, 1024), (8, 1024, 4096), (4, 1024, 192), (1, 128, 64)])
def test_assembled_gathered_operands_equal_the_unsharded_weight(p, N, K):
    """p ranks' send buffers (codes, tiled scales, re-quantized W^T slice of each row shard) stacked as an all-gather
    stacks them: the assembly kernel must return exactly the operands of the unsharded weight (K = 192 leaves a
    partial 128-row tile in the W^T scales, whose padding must read as zero)."""
    import bitlattice_b200 as bl
    from bitlattice_b200 import backend
    from bitlattice_b200.parallel import shard_rows
    wd = (torch.randn(N, K, generator=gen(5)) * 0.02).to(DEV)
    w = bl.LatticeTensor.from_float(wd, "nvfp4", method="rtn", dtype=torch.bfloat16)
    ref_row, ref_t = backend.weight_operand(w), backend.weight_t_operand(w)
    n = N // p
    sends, offsets = [], None
    filler = torch.full((48,), 0xAB, dtype=torch.uint8, device=DEV)           # another weight's pieces come first
    for r in range(p):
        s = shard_rows(w, r, p)
        tp, ts, _ = _ops.requantize_nvfp4_t(s.packed, s.scales, s.global_scale, blocked=False)
        pieces = [filler, s.packed, _ops.to_blocked(s.scales.view(torch.uint8)), tp, ts.view(torch.uint8)]
        offsets, off = [], 0
        for t in pieces:
            offsets.append(off)
            off += t.numel()
        sends.append(torch.cat([t.reshape(-1) for t in pieces]))
    recv = torch.stack(sends).contiguous()
    (codes, sf), (tcodes, tsf) = _ops.assemble_gathered(recv, n, K, offsets[1:])
    assert torch.equal(codes, ref_row.packed)
    assert torch.equal(sf, ref_row.scales.view(torch.uint8).reshape(-1))
    assert torch.equal(tcodes, ref_t.packed)
    assert torch.equal(tsf, ref_t.scales.view(torch.uint8).reshape(-1))


def test_assemble_gathered_rejects_unaligned_pieces():
    recv = torch.zeros(2, 128 * 64 * 2, dtype=torch.uint8, device=DEV)
    with pytest.raises(RuntimeError, match="multiples of 16"):
        _ops.assemble_gathered(recv, 128, 64, [8, 4096, 8192, 12288])
    with pytest.raises(RuntimeError, match="rows % 128"):
        _ops.assemble_gathered(recv, 64, 64, [0, 4096, 8192, 12288])


# ------------------------------------------------------------------------------------------------ bounded waits

def test_bounded_wait_gives_up_records_its_code_and_returns():
    """The give-up path of the GEMM kernels' waits, run alone: a warp waits on a barrier nothing arrives on, the wait
    expires after its (short) limit, records its code in the device flag, and the kernel runs to its end. The flag
    reads back through the status call and is clear afterwards."""
    code, returned = _ops.selftest_bounded_wait(0)
    assert code == 9 and returned == 2
    assert _ops.gemm_status(0) == 0
    # the GEMM still works after the flag has been raised and cleared
    a = torch.randint(0, 256, (128, 64), dtype=torch.uint8, device=DEV)
    sf = torch.full((_ops.blocked_scale_bytes(128, 8),), 56, dtype=torch.uint8, device=DEV)
    one = torch.ones(1, device=DEV)
    _ops.nvfp4_gemm(a, sf, one, a, sf, one)
    assert _ops.gemm_status(0) == 0


def test_optimizer_raises_on_a_recorded_gemm_failure():
    """Lattice.step() copies the GEMM error flag to pinned memory behind each step and the next step (or
    synchronize / state_dict) raises when it was set, instead of training on partial outputs."""
    import bitlattice_b200 as bl
    w = bl.LatticeTensor.from_float((torch.randn(64, 64, generator=gen(3)) * 0.02).to(DEV), "nvfp4", method="rtn",
                                    dtype=torch.bfloat16)
    p = torch.nn.Parameter(w)
    opt = bl.Lattice([p], lr=3e-3, direction="sign", phase_bits=2)
    p.grad = torch.randn(64, 64, device=DEV).to(torch.bfloat16)
    opt.step()
    opt.synchronize()                                         # flag copied and read: clean
    flag, _ = opt._gemm_flags[p.device]
    assert int(flag.item()) == 0
    flag.fill_(2)                                             # what the copy would have delivered after a failure
    p.grad = torch.randn(64, 64, device=DEV).to(torch.bfloat16)
    before = p.packed.clone()
    with pytest.raises(RuntimeError, match="gave up on a bounded wait"):
        opt.step()
    assert torch.equal(p.packed, before)                      # raised before any update was applied
    p.grad = None
    opt.step()                                                # reported once, cleared
