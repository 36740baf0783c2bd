"""Pins the CPU oracle against fixtures produced by the REFERENCE's own device
code (tests/golden/*.npz, generated on a B200 by tests/golden/make_golden.py from
oracle/_ref/libssb_ref.so).  Each stage is compared stage-isolated: the oracle is
fed the reference's own upstream outputs.  Tolerances are the reference parity
tools' model, |d| <= atol + rtol*|ref| with a capped violation fraction
(src/backend/tests/projection_parity.cpp:347-364, render_parity.cpp:342-357,
raster_bwd_parity.cpp:360-368, proj_bwd_parity.cpp:324-339, optim_parity.cpp:9-13):
the reference is built with --use_fast_math, the oracle with IEEE arithmetic."""
import os
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))

from golden_cases import (DIST_CASES, FPBO_L1_RUNS, FPBO_RUNS, FPBO_SCENE, decode_splat_blocks, encode_splat_blocks, frac_beyond_quanta, joint_state_decode, q16_moments_mismatch, dist_case_inputs, fpbo_inputs, ACCUM_CASES, CASES, LOSS_MAP_WEIGHT, QUANT_CASES, QUANT_SCENE, WIDE_CASES, accum_weight_map, adam_inputs,  # noqa: E402
                          build_case, loss_inputs, loss_map_base, quant_sh_inputs, raster_cotangents)  # noqa: E402


ALL_CASES = list(CASES) + list(WIDE_CASES)


def model_of(name):
    """Camera model of a fixture: 0 pinhole, 1 equidistant fisheye, 3 equirectangular."""
    return WIDE_CASES[name]["model"] if name in WIDE_CASES else 0


def load(name):
    return dict(np.load(os.path.join(HERE, "golden", f"{name}.npz")))


def frac_bad(got, ref, atol, rtol):
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    return float((~(np.abs(got - ref) <= atol + rtol * np.abs(ref))).mean())


def ref_proj(gold):
    return {k: gold[k] for k in ("aabb", "depths", "xy", "depth", "conic", "opac", "rgb")}


@pytest.mark.parametrize("name", ALL_CASES)
def test_projection_forward_vs_reference(oracle, name):
    cfg, sp, vm, K = build_case(name)
    gold = load(name)
    got = oracle.project_fwd(sp, vm, K, cfg.width, cfg.height, model=model_of(name))
    keep_ref = gold["aabb"][:, 2] > gold["aabb"][:, 0]
    keep_got = got["aabb"][:, 2] > got["aabb"][:, 0]
    assert keep_ref.sum() > 0 and (keep_ref != keep_got).mean() <= 2e-3
    both = keep_ref & keep_got
    assert frac_bad(got["aabb"][both], gold["aabb"][both], 5e-3, 5e-4) <= 2e-3
    assert frac_bad(got["depths"][both], gold["depths"][both], 5e-3, 5e-4) == 0.0
    for k in ("xy", "depth", "conic", "opac", "rgb"):
        assert frac_bad(got[k][both], gold[k][both], 5e-3, 5e-4) <= 2e-3, k
    assert frac_bad(got["radii"], gold["radii"], 1e-4, 1e-3) <= 2e-3


@pytest.mark.parametrize("name", ALL_CASES)
def test_tile_stage_vs_reference(oracle, name):
    """Counts, sorted keys, flatten ids and offsets from the reference's own projected floats."""
    cfg, sp, vm, K = build_case(name)
    gold = load(name)
    proj = ref_proj(gold)
    n, W, H, I = cfg.n_splats, cfg.width, cfg.height, vm.shape[0]
    counts, cum, keys, vals = oracle.tile_keys(proj, n, W, H)
    # the reference derives its spans with __logf and fast-math division: a borderline
    # splat may gain or lose a tile; everything else is identical
    diff = counts != gold["tiles_per_splat"].astype(np.int64)
    assert diff.mean() <= 2e-3, diff.sum()
    tw, th = oracle.tile_grid(W, H)
    sk, sv = oracle.sort_pairs(keys, vals, 0, 32 + oracle.tile_n_bits(tw * th * I))
    # every fixture scene is free of borderline splats: counts, sorted keys, flatten ids and offsets are the reference's, bit for bit
    assert not diff.any(), (name, int(diff.sum()))
    assert np.array_equal(sk, gold["sorted_ids"]) and np.array_equal(sv, gold["sorted_flat"])
    assert np.array_equal(oracle.tile_offsets(sk, tw * th * I), gold["offsets"])
    # the sort and range stages on the reference's own keys: exact
    rng = np.random.default_rng(0)
    perm = rng.permutation(gold["sorted_ids"].size)
    # (a permutation that keeps equal keys in order: sort by (perm) is not stable-safe, so use unique keys only)
    uk, first = np.unique(gold["sorted_ids"], return_index=True)
    k2, v2 = oracle.sort_pairs(uk[::-1].copy(), gold["sorted_flat"][first][::-1].copy(), 0, 32 + oracle.tile_n_bits(tw * th * I))
    assert np.array_equal(k2, uk) and np.array_equal(v2, gold["sorted_flat"][first])
    assert np.array_equal(oracle.tile_offsets(gold["sorted_ids"], tw * th * I), gold["offsets"])


@pytest.mark.parametrize("name", ALL_CASES)
def test_raster_forward_vs_reference(oracle, name):
    cfg, sp, vm, K = build_case(name)
    gold = load(name)
    I = vm.shape[0]
    got = oracle.raster_fwd(ref_proj(gold), gold["offsets"], gold["sorted_flat"], I, cfg.n_splats, cfg.width, cfg.height)
    assert gold["render_T"].min() < 0.5
    d = np.abs(got["rgb"] - gold["render_rgb"])
    assert d.max() <= 5e-3 and (d.max(axis=1) > 1e-4).mean() <= 2e-3
    assert np.abs(got["T"] - gold["render_T"]).max() <= 5e-3
    assert frac_bad(got["depth"], gold["render_depth"], 5e-3, 1e-3) <= 2e-3
    assert (got["last_ids"] != gold["last_ids"]).mean() <= 2e-3


@pytest.mark.parametrize("name", ALL_CASES)
def test_raster_backward_vs_reference(oracle, name):
    cfg, sp, vm, K = build_case(name)
    gold = load(name)
    I, W, H = vm.shape[0], cfg.width, cfg.height
    v_rgb, v_depth, v_T = raster_cotangents(name, I * H * W)
    render = dict(depth=gold["render_depth"], T=gold["render_T"], last_ids=gold["last_ids"])
    got = oracle.raster_bwd(ref_proj(gold), gold["offsets"], gold["sorted_flat"], I, cfg.n_splats, W, H, render, v_rgb, v_depth, v_T)
    for k in ("v_xy", "v_depth", "v_conic", "v_opac", "v_rgb"):
        ref = gold[k].reshape(got[k].shape)
        scale = np.abs(ref).max()
        assert frac_bad(got[k], ref, 1e-4 * scale, 2e-3) <= 5e-3, k


@pytest.mark.parametrize("name", ALL_CASES)
def test_projection_backward_vs_reference(oracle, name):
    cfg, sp, vm, K = build_case(name)
    gold = load(name)
    v = {k: gold[k] for k in ("v_xy", "v_depth", "v_conic", "v_opac", "v_rgb")}
    got = oracle.project_bwd(sp, vm, K, cfg.width, cfg.height, gold["aabb"], v, model=model_of(name))
    for k in got:
        ref = gold["g_" + k].reshape(got[k].shape)
        scale = np.abs(ref).max()
        assert frac_bad(got[k], ref, 1e-4 * scale, 2e-3) <= 5e-3, k


def _shq(tag, n):
    codes, bounds, bits, stride_arg = quant_sh_inputs(tag, n)
    return dict(packed=codes, bounds=bounds, bits=bits, bounds_stride=stride_arg)


@pytest.mark.parametrize("tag", sorted(QUANT_CASES))
def test_quantised_sh_projection_vs_reference(oracle, tag):
    """Projection forward and backward reading 8/16-bit SH codes, both bound layouts, against the reference's kernels."""
    cfg, sp, vm, K = build_case(QUANT_SCENE)
    base, gold = load(QUANT_SCENE), load("quant_proj")
    shq = _shq(tag, cfg.n_splats)
    got = oracle.project_fwd(sp, vm, K, cfg.width, cfg.height, shq=shq)
    ref_aabb = gold[f"{tag}_aabb"]
    assert np.array_equal(ref_aabb, base["aabb"])                      # the SH storage does not move the geometry
    both = (ref_aabb[:, 2] > ref_aabb[:, 0]) & (got["aabb"][:, 2] > got["aabb"][:, 0])
    assert both.sum() > 100
    ref_rgb = gold[f"{tag}_rgb"]
    assert np.abs(ref_rgb[both] - base["rgb"][both]).max() > 0.05       # and does change the colours
    assert frac_bad(got["rgb"][both], ref_rgb[both], 5e-3, 5e-4) <= 2e-3
    assert frac_bad(got["conic"][both], gold[f"{tag}_conic"][both], 5e-3, 5e-4) <= 2e-3
    v = {k: base[k] for k in ("v_xy", "v_depth", "v_conic", "v_opac", "v_rgb")}
    g = oracle.project_bwd(sp, vm, K, cfg.width, cfg.height, ref_aabb, v, shq=shq)
    for k in g:
        ref = gold[f"{tag}_g_{k}"].reshape(g[k].shape)
        assert frac_bad(g[k], ref, 1e-4 * np.abs(ref).max(), 2e-3) <= 5e-3, k


@pytest.mark.parametrize("tag", sorted(FPBO_RUNS))
def test_fused_backward_optimiser_vs_reference(oracle, tag):
    """The reference's fused projection-backward + optimiser kernel equals its unfused chain: projection backward over all views,
    then the geometry / DC / SH Adam updates -- the oracle's statement of those, two consecutive passes."""
    run = FPBO_RUNS[tag]
    cfg, sp, vm, K = build_case(FPBO_SCENE)
    base, gold = load(FPBO_SCENE), load("fpbo")
    n = cfg.n_splats
    extra = fpbo_inputs(n)
    v = {k: base[k] for k in ("v_xy", "v_depth", "v_conic", "v_opac", "v_rgb")}
    p = {k: x.copy() for k, x in sp.items()}
    m1 = {k: np.zeros_like(x) for k, x in p.items()}
    m2 = {k: np.zeros_like(x) for k, x in p.items()}
    for step in (1, 2):
        if step == 2:           # from the reference's parameters of the first pass, so that the passes are compared one by one
            p = {k: gold[f"{tag}_p1_{k}"].reshape(sp[k].shape).copy() for k in p}
        g = oracle.project_bwd(p, vm, K, cfg.width, cfg.height, base["aabb"], v)
        steps = (extra["steps"] + (step - 1)).astype(np.int32) if run["steps"] else None
        oracle.adam_geometry_ex(p, g, m1, m2, step, cfg.lrs, reg=run["reg"], scale_agnostic=bool(run["agnostic"]), radii=extra["radii"], steps=steps)
        oracle.adam_plain(p["features_dc"], g["features_dc"], m1["features_dc"], m2["features_dc"], step, cfg.lrs["lr_features_dc"], run["sh_reg"],
                          0.5 / 0.28209479177387814, 1.0, steps=steps, stride=3)    # the DC dead zone of the SH regulariser (:355-358)
        oracle.adam_plain(p["features_sh"], g["features_sh"], m1["features_sh"], m2["features_sh"], step, cfg.lrs["lr_features_sh"], run["sh_reg"], 0.0, 1.0,
                          steps=steps, stride=45)
        for k in p:
            assert frac_bad(p[k].reshape(-1), gold[f"{tag}_p{step}_{k}"], 5e-6, 1e-4) <= 2e-3, (tag, k, step)
    for k in p:
        ref1, ref2 = gold[f"{tag}_g1_{k}"], gold[f"{tag}_g2_{k}"]
        assert frac_bad(m1[k].reshape(-1), ref1, 1e-4 * np.abs(ref1).max(), 2e-3) <= 5e-3, k
        assert frac_bad(m2[k].reshape(-1), ref2, 1e-4 * np.abs(ref2).max(), 4e-3) <= 5e-3, k


def splat_block_state_close(got_vc, got_vb, got_oc, got_ob, ref_vc, ref_vb, ref_oc, ref_ob, n):
    """SH value codes / bounds and SH state codes / bounds in the per-256-splats layout against the reference's, compared as the
    numbers they stand for: a block's bounds come from its extreme entries, so rounding moves codes without moving values."""
    assert np.allclose(got_vb, ref_vb, rtol=2e-3, atol=2e-5) and np.allclose(got_ob.reshape(-1, 4), ref_ob.reshape(-1, 4), rtol=2e-3, atol=2e-3)
    gv, rv = decode_splat_blocks(got_vc, got_vb), decode_splat_blocks(ref_vc, ref_vb)
    rb = np.repeat(ref_vb.reshape(-1, 2), 256, axis=0)[:n]
    assert frac_beyond_quanta(gv, rv, rb[:, :1], rb[:, 1:], 65535.0, 3.0) <= 5e-3
    (gu, gs), (ru, rs) = joint_state_decode(got_oc, got_ob, 256 * 45), joint_state_decode(ref_oc, ref_ob, 256 * 45)
    ob = np.repeat(ref_ob.reshape(-1, 4), 256 * 45, axis=0)[: n * 45]
    assert frac_beyond_quanta(gu, ru, ob[:, 0], ob[:, 1], 255.0, 1.6) <= 1e-2
    assert frac_beyond_quanta(gs, rs, ob[:, 2], ob[:, 3], 255.0, 1.6) <= 1e-2
    return gv, rv


@pytest.mark.parametrize("tag", ["l1", "l1_deg1"])
def test_fused_backward_optimiser_level1_vs_reference(oracle, tag):
    """The reference's fused kernel at quantisation level 1 (16-bit SH values and 8-bit SH optimiser state with one bound per 256
    splats) against the oracle's chain: projection backward reading the codes, geometry and DC Adam, and the SH update on the
    splat-block layout; degree 1 on the 15-coefficient buffers writes the idle bands as zero."""
    run = FPBO_L1_RUNS[tag]
    cfg, sp, vm, K = build_case(FPBO_SCENE)
    base, gold = load(FPBO_SCENE), load("fpbo_l1")
    n, deg = cfg.n_splats, run["degree"]
    extra = fpbo_inputs(n)
    v = {k: base[k] for k in ("v_xy", "v_depth", "v_conic", "v_opac", "v_rgb")}
    five = ("means", "quats", "scales", "opacities", "features_dc")
    p = {k: sp[k].copy() for k in five}
    p["features_sh"] = np.zeros_like(sp["features_sh"])
    m1 = {k: np.zeros_like(x) for k, x in p.items()}
    m2 = {k: np.zeros_like(x) for k, x in p.items()}
    vc, vb = encode_splat_blocks(sp["features_sh"].reshape(n, 45), 16)
    oc, ob = np.zeros(n * 45 * 2, np.uint8), np.zeros(((n + 255) // 256) * 4, np.float32)
    for step in (1, 2):
        if step == 2:       # each pass from the reference's state of the pass before
            for k in five:
                p[k] = gold[f"{tag}_p1_{k}"].reshape(sp[k].shape).copy()
            vc, vb = gold[f"{tag}_s1_value_codes"].copy(), gold[f"{tag}_s1_value_bounds"].copy()
            oc, ob = gold[f"{tag}_s1_optim_codes"].copy(), gold[f"{tag}_s1_optim_bounds"].copy()
        shq = dict(packed=vc, bounds=vb.reshape(-1), bits=16, bounds_stride=0)
        g = oracle.project_bwd(p, vm, K, cfg.width, cfg.height, base["aabb"], v, shq=shq, sh_degree=deg)
        steps = (extra["steps"] + (step - 1)).astype(np.int32) if run["steps"] else None
        oracle.adam_geometry_ex(p, g, m1, m2, step, cfg.lrs, reg=run["reg"], scale_agnostic=bool(run["agnostic"]), radii=extra["radii"], steps=steps)
        oracle.adam_plain(p["features_dc"], g["features_dc"], m1["features_dc"], m2["features_dc"], step, cfg.lrs["lr_features_dc"], run["sh_reg"],
                          0.5 / 0.28209479177387814, 1.0, steps=steps, stride=3)
        vb = vb.reshape(-1).copy()
        oracle.adam_sh_splat_blocks(g["features_sh"].reshape(-1), oc, ob, vc, vb, 16, n, step, cfg.lrs["lr_features_sh"], l2_reg=run["sh_reg"],
                                    sh_degree=deg, steps=steps)
        for k in five:
            assert frac_bad(p[k].reshape(-1), gold[f"{tag}_p{step}_{k}"], 5e-6, 1e-4) <= 2e-3, (tag, k, step)
        gv, rv = splat_block_state_close(vc, vb.reshape(-1, 2), oc, ob, gold[f"{tag}_s{step}_value_codes"], gold[f"{tag}_s{step}_value_bounds"].reshape(-1, 2),
                                         gold[f"{tag}_s{step}_optim_codes"], gold[f"{tag}_s{step}_optim_bounds"], n)
        if deg < 3:
            n_active = 3 * deg * (deg + 2)
            span = (gold[f"{tag}_s{step}_value_bounds"].reshape(-1, 2)[:, 1] - gold[f"{tag}_s{step}_value_bounds"].reshape(-1, 2)[:, 0]).max()
            assert np.abs(rv[:, n_active:]).max() <= span / 65535.0 and np.abs(gv[:, n_active:]).max() <= span / 65535.0     # idle bands: zero
            assert np.abs(rv[:, :n_active]).max() > 0.01
    for k in five:
        ref1, ref2 = gold[f"{tag}_g1_{k}"], gold[f"{tag}_g2_{k}"]
        assert frac_bad(m1[k].reshape(-1), ref1, 1e-4 * np.abs(ref1).max(), 2e-3) <= 5e-3, k
        assert frac_bad(m2[k].reshape(-1), ref2, 1e-4 * np.abs(ref2).max(), 4e-3) <= 5e-3, k


@pytest.mark.parametrize("deg", [0, 1, 2])
def test_active_sh_degree_vs_reference(oracle, deg):
    """Projection with the SH degree warmed up (bands above the active degree neither read nor given a gradient) against
    the reference's Vanilla3DGS<0>, <1>, <2> kernels on the 15-coefficient rows of the ring2 scene."""
    cfg, sp, vm, K = build_case(QUANT_SCENE)
    base, gold = load(QUANT_SCENE), load("sh_degree")
    got = oracle.project_fwd(sp, vm, K, cfg.width, cfg.height, sh_degree=deg)
    ref_aabb = gold[f"d{deg}_aabb"]
    assert np.array_equal(ref_aabb, base["aabb"])                      # the degree does not move the geometry
    both = (ref_aabb[:, 2] > ref_aabb[:, 0]) & (got["aabb"][:, 2] > got["aabb"][:, 0])
    ref_rgb = gold[f"d{deg}_rgb"]
    assert np.abs(ref_rgb[both] - base["rgb"][both]).max() > 0.02       # and does change the colours
    assert frac_bad(got["rgb"][both], ref_rgb[both], 5e-3, 5e-4) <= 2e-3
    v = {k: base[k] for k in ("v_xy", "v_depth", "v_conic", "v_opac", "v_rgb")}
    g = oracle.project_bwd(sp, vm, K, cfg.width, cfg.height, ref_aabb, v, sh_degree=deg)
    n_active = (deg + 1) ** 2 - 1
    assert not g["features_sh"][:, n_active:].any() and not gold[f"d{deg}_g_features_sh"].reshape(-1, 15, 3)[:, n_active:].any()
    assert deg == 0 or np.abs(g["features_sh"][:, :n_active]).max() > 0
    for k in g:
        ref = gold[f"d{deg}_g_{k}"].reshape(g[k].shape)
        assert frac_bad(g[k], ref, 1e-4 * max(np.abs(ref).max(), 1e-12), 2e-3) <= 5e-3, k


@pytest.mark.parametrize("name", sorted(DIST_CASES))
def test_lens_distortion_projection_vs_reference(oracle, name):
    """Projection forward and backward with a lens-distortion tier, every (camera model, tier) pair the reference
    instantiates, against its kernels: visible set, all forward outputs, the six gradient arrays."""
    cfg, sp, vm, K, model, tier, rows, v = dist_case_inputs(name)
    gold = load("dist_proj")
    base = load(DIST_CASES[name]["scene"])
    got = oracle.project_fwd(sp, vm, K, cfg.width, cfg.height, model=model, dist=tier, dist_coeffs=rows)
    ref_aabb = gold[f"{name}_aabb"]
    keep_ref, keep_got = ref_aabb[:, 2] > ref_aabb[:, 0], got["aabb"][:, 2] > got["aabb"][:, 0]
    keep_base = base["aabb"][:, 2] > base["aabb"][:, 0]
    assert keep_ref.sum() > 100
    if name != "pinhole_thinprism":                    # (a mild lens: every splat stays valid)
        assert (keep_ref != keep_base).sum() > 10      # the lens changes what is seen
    assert (keep_ref != keep_got).mean() <= 2e-3
    both = keep_ref & keep_got
    assert np.abs(gold[f"{name}_xy"][both & keep_base] - base["xy"][both & keep_base]).max() > 0.5      # and where
    for k in ("aabb", "depths", "xy", "depth", "conic", "opac", "rgb"):
        assert frac_bad(got[k][both], gold[f"{name}_{k}"][both], 5e-3, 5e-4) <= 2e-3, k
    assert frac_bad(got["radii"], gold[f"{name}_radii"], 1e-4, 1e-3) <= 2e-3
    g = oracle.project_bwd(sp, vm, K, cfg.width, cfg.height, ref_aabb, v, model=model, dist=tier, dist_coeffs=rows)
    for k in g:
        ref = gold[f"{name}_g_{k}"].reshape(g[k].shape)
        assert frac_bad(g[k], ref, 1e-4 * np.abs(ref).max(), 2e-3) <= 5e-3, k


@pytest.mark.parametrize("key", ["ring2", "dense1", "ring2_q16_cell"])
def test_packed_projection_vs_reference(oracle, key):
    """The reference's packed projection is the unpacked one with the culled pairs removed, view-major: ids and count
    exactly, values as for the unpacked kernels; its packed backward equals the unpacked backward on the kept pairs."""
    name = key.split("_")[0]
    cfg, sp, vm, K = build_case(name)
    base, gold = load(name), load("packed_proj")
    n = cfg.n_splats
    shq = _shq("q16_cell", n) if key.endswith("q16_cell") else None
    V = int(gold[f"{key}_nnz"][0])
    keep_ref = base["aabb"][:, 2] > base["aabb"][:, 0]
    where = np.nonzero(keep_ref)[0]
    assert V == where.size
    assert np.array_equal(gold[f"{key}_camera_ids"], where // n) and np.array_equal(gold[f"{key}_gaussian_ids"], where % n)
    got = oracle.project_fwd(sp, vm, K, cfg.width, cfg.height, shq=shq)
    keep_got = got["aabb"][:, 2] > got["aabb"][:, 0]
    assert np.array_equal(keep_got, keep_ref)                          # same visible set, so the same ids and count
    for k in ("aabb", "depths", "xy", "depth", "conic", "opac", "rgb"):
        assert frac_bad(got[k][keep_ref], gold[f"{key}_{k}"], 5e-3, 5e-4) <= 2e-3, k
    assert frac_bad(got["radii"], gold[f"{key}_radii"], 1e-4, 1e-3) <= 2e-3
    # backward: the reference's packed mode (one thread per packed pair) against the oracle on the same cotangents
    v = {k: base[k] for k in ("v_xy", "v_depth", "v_conic", "v_opac", "v_rgb")}
    g = oracle.project_bwd(sp, vm, K, cfg.width, cfg.height, base["aabb"], v, shq=shq)
    for k in g:
        ref = gold[f"{key}_g_{k}"].reshape(g[k].shape)
        assert frac_bad(g[k], ref, 1e-4 * np.abs(ref).max(), 2e-3) <= 5e-3, k


def test_ssim_vs_reference(oracle):
    gold = load("ssim")
    for tag, (B, H, W, render, gt) in loss_inputs().items():
        v, losses = oracle.loss_l1_ssim(render, gt, B, H, W, 0.0, 0.2)     # w_l1 = 0: the SSIM part alone
        ref = gold[f"{tag}_grad"]
        assert frac_bad(v, ref, 1e-4 * np.abs(ref).max(), 1e-3) == 0.0
        # the reference's scalar sums SSIM over tile-grid positions; its tile (24) divides neither
        # size here only approximately -- it documents that mismatch (docs/testing.md:44-50)
        assert abs(float(gold[f"{tag}_ssim"][0]) - float(losses[1])) <= 0.05


def test_adam_vs_reference(oracle):
    gold = load("adam")
    inp = adam_inputs()
    p = {k: v.copy() for k, v in inp["params"].items()}
    m1 = {k: np.zeros_like(v) for k, v in p.items()}
    m2 = {k: np.zeros_like(v) for k, v in p.items()}
    lr, gs = inp["lrs"], inp["grad_scale"]
    for step, grads in enumerate(inp["grads"], start=1):
        g = {k: v.copy() for k, v in grads.items()}
        oracle.adam_geometry(p, g, m1, m2, step, lr, grad_scale=gs)
        oracle.adam_plain(p["features_dc"], g["features_dc"], m1["features_dc"], m2["features_dc"], step, lr["lr_features_dc"], 0.0,
                          0.5 / 0.28209479177387814, gs)
        oracle.adam_plain(p["features_sh"], g["features_sh"], m1["features_sh"], m2["features_sh"], step, lr["lr_features_sh"], 0.0, 0.0, gs)
        for k in p:
            assert frac_bad(p[k].reshape(-1), gold[f"p{step}_{k}"], 5e-6, 1e-4) <= 1e-3, (k, step)
    for k in p:
        assert frac_bad(m1[k].reshape(-1), gold[f"m1_{k}"], 1e-9, 2e-3) <= 2e-3, k
        assert frac_bad(m2[k].reshape(-1), gold[f"m2_{k}"], 1e-12, 2e-3) <= 2e-3, k
    for bits in (16, 8):
        q = inp[f"qq{bits}"]
        view = np.uint16 if bits == 16 else np.uint8
        state = [q["value_packed"].copy(), q["value_bounds"].copy(), q["optim_packed"].copy(), q["optim_bounds"].copy()]
        for step, grad in enumerate(q["grads"], start=1):
            vp, vb, op, ob = (a.copy() for a in state)
            oracle.adam_qq(grad.copy(), op, ob, vp, vb, bits, step, lr["lr_features_sh"], grad_scale=gs)
            rv, rb, ro, rob = (gold[f"qq{bits}_s{step}_{s}"] for s in ("value_packed", "value_bounds", "optim_packed", "optim_bounds"))
            dv = np.abs(vp.view(view).astype(np.int64) - rv.view(view).astype(np.int64))
            do = np.abs(op.astype(np.int64) - ro.astype(np.int64))
            assert dv.max() <= 1 and do.max() <= 1, (bits, step)           # +-1 quantum
            assert (dv > 0).mean() <= 5e-2 and (do > 0).mean() <= 5e-2
            assert np.allclose(vb, rb, rtol=1e-4, atol=1e-7) and np.allclose(ob, rob, rtol=2e-3, atol=1e-5)
            state = [rv.copy(), rb.copy(), ro.copy(), rob.copy()]            # continue from the reference's state
    # fp32 values with the 8-bit state (value_bits = 32), each step continued from the reference's state
    q = inp["q8"]
    x, op, ob = q["x0"].copy(), np.zeros(q["numel"] * 2, np.uint8), np.zeros(((q["numel"] + 255) // 256) * 4, np.float32)
    for step, grad in enumerate(q["grads"], start=1):
        oracle.adam_qq(grad.copy(), op, ob, x.view(np.uint8), np.zeros(2, np.float32), 32, step, lr["lr_features_sh"], grad_scale=gs)
        rx, ro, rob = (gold[f"q8_s{step}_{s}"] for s in ("x", "optim_packed", "optim_bounds"))
        do = np.abs(op.astype(np.int64) - ro.astype(np.int64))
        assert do.max() <= 1 and (do > 0).mean() <= 5e-2, step
        assert np.allclose(ob, rob, rtol=2e-3, atol=1e-5)
        assert frac_bad(x, rx, 5e-6, 1e-4) <= 1e-3, step
        x, op, ob = rx.copy(), ro.copy(), rob.copy()


def test_adam_extras_vs_reference(oracle):
    """Regularisers, per-splat step counters and the scale-agnostic mean against the reference's kernels, three steps."""
    gold = load("adam")
    inp = adam_inputs()
    ex, lr, gs, n = inp["ex"], inp["lrs"], inp["grad_scale"], inp["n"]
    for tag, agnostic in (("exA", False), ("exB", True)):
        p = {k: v.copy() for k, v in inp["params"].items()}
        m1 = {k: np.zeros_like(v) for k, v in p.items()}
        m2 = {k: np.zeros_like(v) for k, v in p.items()}
        for step, grads in enumerate(inp["grads"], start=1):
            g = {k: v.copy() for k, v in grads.items()}
            score = np.zeros(n, np.float32)
            oracle.adam_geometry_ex(p, g, m1, m2, step, lr, grad_scale=gs, reg=ex["reg"], scale_agnostic=agnostic, radii=ex["radii"], steps=ex["steps"],
                                    densify_score=score)
            if not agnostic and step == 1:
                assert np.allclose(score, gold["exA_densify_score"], rtol=1e-4, atol=1e-9) and score.min() > 0
            keys = ["means"]
            if not agnostic:
                oracle.adam_plain(p["features_dc"], g["features_dc"], m1["features_dc"], m2["features_dc"], step, lr["lr_features_dc"], 0.0,
                                  0.5 / 0.28209479177387814, gs, steps=ex["steps"], stride=3)
                oracle.adam_plain(p["features_sh"], g["features_sh"], m1["features_sh"], m2["features_sh"], step, lr["lr_features_sh"], 0.0, 0.0, gs,
                                  steps=ex["steps"], stride=45)
                keys = list(p)
            for k in keys:
                assert frac_bad(p[k].reshape(-1), gold[f"{tag}_p{step}_{k}"], 5e-6, 1e-4) <= 1e-3, (tag, k, step)
    q = inp["qq16"]
    n_sp = (q["numel"] + 44) // 45
    steps_q = np.ascontiguousarray(np.resize(ex["steps"], n_sp))
    vp, vb, op, ob = (q[k].copy() for k in ("value_packed", "value_bounds", "optim_packed", "optim_bounds"))
    oracle.adam_qq(q["grads"][0].copy(), op, ob, vp, vb, 16, 1, lr["lr_features_sh"], grad_scale=gs, steps=steps_q, stride=45)
    dv = np.abs(vp.view(np.uint16).astype(np.int64) - gold["qqs_value_packed"].view(np.uint16).astype(np.int64))
    do = np.abs(op.astype(np.int64) - gold["qqs_optim_packed"].astype(np.int64))
    assert dv.max() <= 1 and do.max() <= 1 and (dv > 0).mean() <= 5e-2 and (do > 0).mean() <= 5e-2
    assert np.allclose(vb, gold["qqs_value_bounds"], rtol=1e-4, atol=1e-7) and np.allclose(ob, gold["qqs_optim_bounds"], rtol=2e-3, atol=1e-5)


Q16_ORDER = ("means", "quats", "scales", "opacities", "features_dc")


def q16_code_diff(have, want):
    """Largest difference and fraction of differing 16-bit codes of two packed moment arrays."""
    d = np.abs(np.asarray(have).view(np.uint16).astype(np.int64) - np.asarray(want).view(np.uint16).astype(np.int64))
    return d.max(), (d > 0).mean()


def test_fused_backward_optimiser_level1_q16_moments_vs_reference(oracle):
    """The reference's stock configuration of its fused kernel: level 1 with the moments of the five non-SH arrays in 16-bit codes.
    The DC regulariser is scaled like the SH one (2 w / (3 n)) in this kernel, not taken undivided as in the unfused one."""
    tag = "l1_nq"
    run = FPBO_L1_RUNS[tag]
    cfg, sp, vm, K = build_case(FPBO_SCENE)
    base, gold = load(FPBO_SCENE), load("fpbo_l1")
    n = cfg.n_splats
    blocks = (n + 255) // 256
    extra = fpbo_inputs(n)
    v = {k: base[k] for k in ("v_xy", "v_depth", "v_conic", "v_opac", "v_rgb")}
    widths = dict(oracle.Q16_ATTRS)
    p = {k: sp[k].copy() for k in Q16_ORDER}
    p["features_sh"] = np.zeros_like(sp["features_sh"])
    q = {k: (np.zeros(n * widths[k] * 4, np.uint8), np.zeros(blocks * 4, np.float32)) for k in Q16_ORDER}
    vc, vb = encode_splat_blocks(sp["features_sh"].reshape(n, 45), 16)
    oc, ob = np.zeros(n * 45 * 2, np.uint8), np.zeros(blocks * 4, np.float32)
    for step in (1, 2):
        if step == 2:
            for k in Q16_ORDER:
                p[k] = gold[f"{tag}_p1_{k}"].reshape(sp[k].shape).copy()
                q[k] = (gold[f"{tag}_s1_nq_{k}"].copy(), gold[f"{tag}_s1_nqb_{k}"].copy())
            vc, vb = gold[f"{tag}_s1_value_codes"].copy(), gold[f"{tag}_s1_value_bounds"].copy()
            oc, ob = gold[f"{tag}_s1_optim_codes"].copy(), gold[f"{tag}_s1_optim_bounds"].copy()
        shq = dict(packed=vc, bounds=vb.reshape(-1), bits=16, bounds_stride=0)
        g = oracle.project_bwd(p, vm, K, cfg.width, cfg.height, base["aabb"], v, shq=shq)
        steps = (extra["steps"] + (step - 1)).astype(np.int32)
        oracle.adam_geometry_q16(p, g, q, step, cfg.lrs, sh_reg_weight=2.0 * run["sh_reg"] / (3 * n), reg=run["reg"], scale_agnostic=True,
                                 radii=extra["radii"], steps=steps)
        vb = vb.reshape(-1).copy()
        oracle.adam_sh_splat_blocks(g["features_sh"].reshape(-1), oc, ob, vc, vb, 16, n, step, cfg.lrs["lr_features_sh"], l2_reg=run["sh_reg"], steps=steps)
        for k in Q16_ORDER:
            assert frac_bad(p[k].reshape(-1), gold[f"{tag}_p{step}_{k}"], 5e-6, 1e-4) <= 2e-3, (k, step)
            # the codes as the moments they stand for: the 16-bit grid is finer than the agreement of two gradient sums
            assert q16_moments_mismatch(q[k][0], q[k][1], gold[f"{tag}_s{step}_nq_{k}"], gold[f"{tag}_s{step}_nqb_{k}"], n, widths[k]) <= 5e-3, (k, step)
        splat_block_state_close(vc, vb.reshape(-1, 2), oc, ob, gold[f"{tag}_s{step}_value_codes"], gold[f"{tag}_s{step}_value_bounds"].reshape(-1, 2),
                                gold[f"{tag}_s{step}_optim_codes"], gold[f"{tag}_s{step}_optim_bounds"], n)


def test_adam_16bit_non_sh_moments_vs_reference(oracle):
    """The geometry + DC update on 16-bit moment codes against the reference's non_sh_quant kernel: every step starts from the
    reference's parameters and codes of the step before."""
    gold = load("adam")
    inp = adam_inputs()
    ex, lr, gs, n = inp["ex"], inp["lrs"], inp["grad_scale"], inp["n"]
    widths = dict(oracle.Q16_ATTRS)
    for tag, use_ex in (("nq", False), ("nqx", True)):
        for step, grads in enumerate(inp["grads"], start=1):
            if step == 1:
                p = {k: inp["params"][k].copy() for k in Q16_ORDER}
                q = {k: (np.zeros(n * widths[k] * 4, np.uint8), np.zeros(((n + 255) // 256) * 4, np.float32)) for k in Q16_ORDER}
            else:
                p = {k: gold[f"{tag}_p{step - 1}_{k}"].reshape(inp["params"][k].shape).copy() for k in Q16_ORDER}
                q = {k: (gold[f"{tag}_q{step - 1}_{k}"].copy(), gold[f"{tag}_b{step - 1}_{k}"].copy()) for k in Q16_ORDER}
            g = {k: grads[k].copy() for k in Q16_ORDER}
            oracle.adam_geometry_q16(p, g, q, step, lr, sh_reg_weight=inp["nq_sh_reg_weight"], grad_scale=gs,
                                     reg=ex["reg"] if use_ex else None, steps=ex["steps"] if use_ex else None)
            for k in Q16_ORDER:
                assert frac_bad(p[k].reshape(-1), gold[f"{tag}_p{step}_{k}"], 5e-6, 1e-4) <= 1e-3, (tag, k, step)
                assert np.allclose(q[k][1], gold[f"{tag}_b{step}_{k}"], rtol=1e-4, atol=1e-6), (tag, k, step)
                worst, frac = q16_code_diff(q[k][0], gold[f"{tag}_q{step}_{k}"])
                assert worst <= 2 and frac <= 0.15, (tag, k, step, worst, frac)
    # a round trip of the codec alone: decode(encode(g1, g2)) is within one quantum of each range
    rng = np.random.default_rng(5)
    g1 = (rng.normal(size=(600, 3)) * 1e-3).astype(np.float32)
    g2 = (rng.uniform(1e-9, 1e-5, size=(600, 3))).astype(np.float32)
    packed, bounds = oracle.q16_encode(g1, g2)
    d1, d2 = oracle.q16_decode(packed, bounds, 600, 3)
    assert np.allclose(d2, g2, rtol=2e-3) and np.allclose(d1, g1, rtol=2e-3, atol=2e-4 * np.abs(g1).max())


def _nibble_diff(a, b):
    a, b = a.astype(np.int64), b.astype(np.int64)
    return np.maximum(np.abs((a & 15) - (b & 15)), np.abs((a >> 4) - (b >> 4)))


def test_adam_4bit_state_vs_reference(oracle):
    """QuantizedAdamState<4,256>: fp32 values over three steps, 16-bit values over two, each step from the reference's state."""
    gold = load("adam")
    inp = adam_inputs()
    lr, gs = inp["lrs"], inp["grad_scale"]
    q = inp["q8"]
    x, op, ob = q["x0"].copy(), np.zeros(q["numel"], np.uint8), np.zeros(((q["numel"] + 255) // 256) * 4, np.float32)
    for step, grad in enumerate(q["grads"], start=1):
        oracle.adam_qq(grad.copy(), op, ob, x.view(np.uint8), np.zeros(2, np.float32), 32, step, lr["lr_features_sh"], grad_scale=gs, optim_bits=4)
        rx, ro, rob = (gold[f"q4_s{step}_{s}"] for s in ("x", "optim_packed", "optim_bounds"))
        do = _nibble_diff(op, ro)
        assert do.max() <= 1 and (do > 0).mean() <= 5e-2, step
        assert np.allclose(ob, rob, rtol=2e-3, atol=1e-5)
        assert frac_bad(x, rx, 5e-6, 1e-4) <= 1e-3, step
        x, op, ob = rx.copy(), ro.copy(), rob.copy()
    q = inp["qq16"]
    vp, vb = q["value_packed"].copy(), q["value_bounds"].copy()
    op, ob = np.zeros(q["numel"], np.uint8), np.zeros(((q["numel"] + 255) // 256) * 4, np.float32)
    for step, grad in enumerate(q["grads"][:2], start=1):
        oracle.adam_qq(grad.copy(), op, ob, vp, vb, 16, step, lr["lr_features_sh"], grad_scale=gs, optim_bits=4)
        rv, rb, ro, rob = (gold[f"qq16o4_s{step}_{s}"] for s in ("value_packed", "value_bounds", "optim_packed", "optim_bounds"))
        dv = np.abs(vp.view(np.uint16).astype(np.int64) - rv.view(np.uint16).astype(np.int64))
        do = _nibble_diff(op, ro)
        assert dv.max() <= 1 and do.max() <= 1 and (dv > 0).mean() <= 5e-2 and (do > 0).mean() <= 5e-2, step
        assert np.allclose(vb, rb, rtol=1e-4, atol=1e-7) and np.allclose(ob, rob, rtol=2e-3, atol=1e-5)
        vp, vb, op, ob = rv.copy(), rb.copy(), ro.copy(), rob.copy()


@pytest.mark.parametrize("name", ACCUM_CASES)
def test_raster_accum_weight_vs_reference(oracle, name):
    """Densification weights (max / sum / average) of the backward walk against the reference's kernel."""
    cfg, sp, vm, K = build_case(name)
    gold, acc_gold = load(name), load("accum")
    I, W, H, n = vm.shape[0], cfg.width, cfg.height, cfg.n_splats
    proj = {k: np.ascontiguousarray(gold[k]) for k in ("xy", "conic", "opac")}
    render = dict(T=np.ascontiguousarray(gold["render_T"]), last_ids=np.ascontiguousarray(gold["last_ids"]))
    wmap = accum_weight_map(name, I * H * W)
    offs, fl = np.ascontiguousarray(gold["offsets"]), np.ascontiguousarray(gold["sorted_flat"])
    for mode, tag in ((1, "max"), (2, "sum"), (3, "avg")):
        acc, den = oracle.raster_accum_weight(proj, offs, fl, I, n, W, H, render, wmap, mode)
        ref = acc_gold[f"{name}_{tag}"]
        assert (ref > 0).sum() > n // 10
        assert frac_bad(acc, ref, 1e-5 * ref.max(), 2e-3) <= 5e-3, tag
        if mode == 3:
            assert frac_bad(den, acc_gold[f"{name}_avg_den"], 1e-5 * acc_gold[f"{name}_avg_den"].max(), 2e-3) <= 5e-3


def test_ssim_loss_map_vs_reference(oracle):
    """The densification loss map (three SSIM variants, added in place) against the reference's kernel."""
    gold = load("ssim_map")
    for tag, (B, H, W, render, gt) in loss_inputs().items():
        for mode in (1, 2, 3):
            lm = loss_map_base(tag, B * H * W)
            v, losses = oracle.loss_l1_ssim_map(render, gt, B, H, W, mode, LOSS_MAP_WEIGHT, lm, 0.0, 0.2)
            ref = gold[f"{tag}_map{mode}"]
            assert np.abs(ref - loss_map_base(tag, B * H * W)).max() > 0.05
            assert frac_bad(lm, ref, 2e-5, 1e-4) <= 1e-3, (tag, mode)
            v0, _ = oracle.loss_l1_ssim(render, gt, B, H, W, 0.0, 0.2)
            assert np.array_equal(v, v0)                                     # the gradient does not depend on the map


def test_masked_ssim_vs_reference(oracle):
    """The masked SSIM launch (window coverage, dropped samples, masked centres and pixels) against the reference's kernel,
    for a mask of the image's size and a nearest-sampled one of another size."""
    from golden_cases import loss_masks
    gold = load("ssim_masked")
    for tag, (B, H, W, render, gt) in loss_inputs().items():
        for kind, mask in loss_masks(tag, B, H, W).items():
            v, losses = oracle.loss_l1_ssim_masked(render, gt, B, H, W, mask=mask, w_l1=0.0, w_ssim=0.2)
            ref = gold[f"{tag}_{kind}_grad"]
            assert np.abs(ref).max() > 0
            assert frac_bad(v, ref, 2e-6 * np.abs(ref).max(), 2e-4) <= 1e-3, (tag, kind)
            assert abs(losses[1] - gold[f"{tag}_{kind}_ssim"][0]) <= 2e-5
            if kind == "same":
                assert np.all(v.reshape(B, H, W, 3)[mask == 0] == 0) and np.all(ref.reshape(B, H, W, 3)[mask == 0] == 0)
            for mode in (1, 2, 3):
                lm = loss_map_base(tag, B * H * W)
                oracle.loss_l1_ssim_masked(render, gt, B, H, W, mask=mask, map_mode=mode, map_weight=LOSS_MAP_WEIGHT, loss_map=lm, w_l1=0.0, w_ssim=0.2)
                assert frac_bad(lm, gold[f"{tag}_{kind}_map{mode}"], 2e-5, 1e-4) <= 1e-3, (tag, kind, mode)


def test_live_tile_map_and_intersection_vs_reference(oracle):
    """The live-tile map of a mask (own size and another size) and the intersection that skips dead tiles: bit for bit."""
    from golden_cases import LIVE_TILE_CASE, tile_masks
    cfg, sp, vm, K = build_case(LIVE_TILE_CASE)
    gold, live_gold = load(LIVE_TILE_CASE), load("tiles_live")
    proj = ref_proj(gold)
    n, W, H, I = cfg.n_splats, cfg.width, cfg.height, vm.shape[0]
    tw, th = oracle.tile_grid(W, H)
    for kind, mask in tile_masks(I, H, W).items():
        live = oracle.tile_active(mask, W, H)
        ref_live = live_gold[f"{kind}_tile_active"].reshape(I, th, tw)
        assert 0 < ref_live.sum() < ref_live.size
        assert np.array_equal(live, ref_live), kind
        counts, cum, keys, vals = oracle.tile_keys(proj, n, W, H, tile_active=live)
        assert np.array_equal(counts, live_gold[f"{kind}_tiles_per_splat"].astype(np.int64)), kind
        assert counts.sum() < gold["tiles_per_splat"].sum()
        sk, sv = oracle.sort_pairs(keys, vals, 0, 32 + oracle.tile_n_bits(tw * th * I))
        assert np.array_equal(sk, live_gold[f"{kind}_sorted_ids"]) and np.array_equal(sv, live_gold[f"{kind}_sorted_flat"]), kind
        offs = oracle.tile_offsets(sk, tw * th * I)
        assert np.array_equal(offs, live_gold[f"{kind}_offsets"]), kind
        # dead tiles have empty ranges
        ends = np.append(offs[1:], sk.size)
        assert np.all((ends - offs)[ref_live.reshape(-1) == 0] == 0)


def test_multi_scale_loss_vs_reference(oracle):
    """The whole multi-scale driver of the reference (pyramid with masked pooling, per-pixel + SSIM pass per level, fold of
    the gradients and of the loss maps, masked pixels cleared) on its own kernels, against the restatement."""
    from golden_cases import MULTI_SCALE_RUNS, loss_masks
    gold = load("loss_multi")
    for tag, (B, H, W, render, gt) in loss_inputs().items():
        masks = dict(loss_masks(tag, B, H, W), none=None)
        for kind, scales in MULTI_SCALE_RUNS:
            key = f"{tag}_{kind}_{scales}"
            v, losses, _ = oracle.loss_multi_scale(render, gt, B, H, W, scales, mask=masks[kind])
            ref = gold[key + "_grad"]
            assert frac_bad(v, ref, 2e-6 * np.abs(ref).max(), 2e-4) <= 1e-3, key
            rgb_loss, ssim = gold[key + "_scalars"]
            assert abs(0.8 * losses[0] - rgb_loss) <= 1e-5 * abs(rgb_loss) + 1e-7, (key, losses, rgb_loss)
            assert abs(losses[1] - ssim) <= 2e-5, (key, losses, ssim)
            for mode in (1, 3):
                _, _, lm = oracle.loss_multi_scale(render, gt, B, H, W, scales, mask=masks[kind], loss_map_mode=mode)
                assert frac_bad(lm, gold[key + f"_map{mode}"], 2e-5, 1e-4) <= 1e-3, (key, mode)


def test_densify_per_step_vs_reference(oracle):
    """Scale clip, averaged-weight quotient, score update (every way the engine picks its buffers), quantile clip and sample
    score against the reference's kernels; both noises against the reference's in distribution (the hash that drives them
    amplifies rounding, so they are not equal number for number)."""
    from golden_cases import DENSIFY_SCORE_RUNS, densify_inputs
    from tests import densify_util as D
    gold = load("densify")
    inp = densify_inputs()
    n = inp["radii"].shape[0]
    for name, kw in DENSIFY_SCORE_RUNS:
        a = D.score_run_args(kw)
        scales = inp["log_scales"].copy()
        acc = inp["accum_buffer"].copy() if a["use_accum"] else None
        aw = inp["accum_weight"].copy() if a["use_weights"] else None
        sample = np.zeros((n, 2), np.float32) if a["want_sample"] else None
        oracle.densify_update_scores(inp["radii"], scales, acc, accum_weight=aw, accum_den=inp["accum_den"] if a["accum_mode"] == 3 else None,
                                     world_grad=inp["world_grad"] if a["use_world"] else None, logit_opacs=inp["logit_opacs"], sample_score=sample,
                                     max_screen_size=a["max_screen_size"], clip_hardness=a["clip_hardness"], max_world_size=a["max_world_size"],
                                     accum_mode=a["accum_mode"], score_mode=a["score_mode"], blend_w=a["blend_w"], score_power=a["score_power"],
                                     clip_quantile=a["clip_quantile"], final_power=a["final_power"])
        D.check_score_run(name, dict(log_scales=scales, accum_weight=aw, accum_buffer=acc, sample_score=sample), gold)
    # the quantile alone: the sort-based statement equals the clipped maximum of the reference's accumulator
    ref_acc = gold["clip_score_accum_buffer"]
    assert abs(ref_acc[:, 0].max() - oracle.quantile_positive(gold["mean_accum_buffer"], 0.9, stride=2)) <= 1e-6
    for revised, scaler in ((0, 2e3), (1, 5e5 * 1.6e-4)):
        moved = inp["means"].copy()
        z = oracle.densify_add_noise(moved, inp["log_scales"], inp["quats"], inp["logit_opacs"], scaler, revised, radii=inp["radii"])
        D.check_noise(inp, moved, scaler, revised, reference_moved=gold[f"noise{revised}_means"])


@pytest.mark.parametrize("quant", [False, True])
def test_densify_relocation_and_growth_vs_reference(oracle, quant):
    """Relocation of the dead splats and the growth step (long-axis split, weighted draw without replacement) against the state
    the reference's kernels leave: same dead set, draws that agree except at the cut, same treatment of every source and slot."""
    import copy
    from golden_cases import DENSIFY_SPLIT as D, densify_split_inputs
    from tests import densify_util as U
    gold = load("densify_split")
    tag = "q" if quant else "f"
    st = densify_split_inputs(quant)
    before = copy.deepcopy(st)
    dead = U.dead_mask(st, D["cur_n"], D["min_opacity"])
    assert 20 < dead.sum() < 120

    def ref_state(phase):
        out = {k[len(tag) + len(phase) + 2:]: gold[k] for k in gold if k.startswith(f"{tag}_{phase}_")}
        for k, v in out.items():
            if before.get(k) is not None and isinstance(before[k], np.ndarray):
                out[k] = v.reshape(before[k].shape)
        return out
    src, dst = oracle.densify_split(0, st, D["cur_n"], D["seed"], D["split_k"], D["min_opacity"])
    assert np.array_equal(dst, np.flatnonzero(dead))
    ref = ref_state("reloc")
    # the reference's dead set: the slots whose rotation changed
    assert set(np.flatnonzero(np.any(ref["quats"] != before["quats"], axis=1)).tolist()) <= set(dst.tolist())
    U.check_split_state(before, st, ref, D["cur_n"], 0, 0, dead, quant)
    mid = ref            # the growth step continues from the reference's state, so both sides start equal
    st2 = copy.deepcopy(mid)
    st2["weights"] = before["weights"]
    for k in ("sh_optim_bounds", "sh_value_bounds", "sh_optim_bits", "sh_value_bits"):
        if k in before:
            st2[k] = before[k]
    for k in U.SPLIT_ATTRS:
        for pre in ("", "m1_", "m2_"):
            st2.setdefault(pre + k, None)
    mid_copy = copy.deepcopy(st2)
    oracle.densify_split(1, st2, D["cur_n"], D["seed"] + 1, D["split_k"], num_new=D["num_new"])
    U.check_split_state(mid_copy, st2, ref_state("add"), D["cur_n"], D["cur_n"], D["num_new"], None, quant)


def test_weighted_draw_is_the_smallest_keys(oracle):
    """The draw: k smallest keys w / log(1 - u), zero weights last, masked splats never while enough others remain; and it is
    proportional to the weights (frequency of a heavy half against a light half over many seeds)."""
    rng = np.random.default_rng(3)
    n = 600
    w = np.stack([rng.random(n), np.ones(n)], axis=1).astype(np.float32)
    w[:50, 0] = 0.0
    alive = np.ones(n, np.uint8); alive[100:130] = 0
    got = oracle.weighted_sample(w, 42, 200, alive)
    assert len(set(got.tolist())) == 200 and not (set(got.tolist()) & set(range(50))) and not (set(got.tolist()) & set(range(100, 130)))
    w2 = np.ones((n, 2), np.float32); w2[: n // 2, 0] = 4.0
    heavy = sum((oracle.weighted_sample(w2, seed, 60) < n // 2).sum() for seed in range(200)) / (200 * 60)
    assert 0.72 < heavy < 0.84           # 4 : 1 weights, 10 % drawn: about 0.78
