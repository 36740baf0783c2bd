"""The CUDA library against fixtures produced by the REFERENCE's own device code
(tests/golden/*.npz; see tests/golden/make_golden.py), stage by stage on the
reference's own upstream outputs, through the C ABI."""
import ctypes as C
import os
import sys

import numpy as np
import pytest

torch = pytest.importorskip("torch")

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))

from golden_cases import (DIST_CASES, FPBO_L1_RUNS, FPBO_RUNS, FPBO_SCENE, decode_splat_blocks, encode_splat_blocks, frac_beyond_quanta, joint_state_decode, q16_moments_mismatch, dist_case_inputs, fpbo_inputs, ACCUM_CASES, CASES, LOSS_MAP_WEIGHT, QUANT_CASES, QUANT_SCENE, WIDE_CASES, accum_weight_map, adam_inputs,  # noqa: E402
                          build_case, loss_inputs, loss_map_base, quant_sh_inputs, raster_cotangents)  # noqa: E402
from spirula_studio_b200 import lib as L  # noqa: E402

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def lib():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return L.load()


@pytest.fixture(scope="module")
def U():
    from tests import gpu_util
    return gpu_util


ALL_CASES = list(CASES) + list(WIDE_CASES)


def model_of(name):
    """Camera model of a fixture: 0 pinhole, 1 equidistant fisheye, 3 equirectangular."""
    return WIDE_CASES[name]["model"] if name in WIDE_CASES else 0


def load(name):
    return dict(np.load(os.path.join(HERE, "golden", f"{name}.npz")))


def ref_proj(gold):
    return {k: gold[k] for k in ("aabb", "depths", "xy", "depth", "conic", "opac", "rgb")}


@pytest.mark.parametrize("name", ALL_CASES)
def test_projection_forward_vs_reference(lib, U, name):
    cfg, sp, vm, K = build_case(name)
    gold = load(name)
    got = U.project_fwd(lib, U.splats_dev(sp), vm, K, cfg.width, cfg.height, model=model_of(name))
    aabb = got["aabb"].cpu().numpy()
    keep_ref, keep_got = gold["aabb"][:, 2] > gold["aabb"][:, 0], aabb[:, 2] > aabb[:, 0]
    assert (keep_ref != keep_got).mean() <= 2e-3
    both = keep_ref & keep_got
    scr = U.unpack_screen(lib, got["rec"], vm.shape[0] * cfg.n_splats)
    assert U.close_frac(aabb[both], gold["aabb"][both], 5e-3, 5e-4) <= 2e-3
    for k in ("xy", "depth", "conic", "opac", "rgb"):
        assert U.close_frac(scr[k][both], gold[k][both], 5e-3, 5e-4) <= 2e-3, k


@pytest.mark.parametrize("name", ALL_CASES)
def test_tile_stage_vs_reference(lib, U, name):
    cfg, sp, vm, K = build_case(name)
    gold = load(name)
    n, W, H, I = cfg.n_splats, cfg.width, cfg.height, vm.shape[0]
    rec = U.pack_screen(lib, ref_proj(gold))
    cap = 64 * n
    st, M, counts, cum, keys, vals, n_dev = U.tile_keys(lib, U.dev(gold["aabb"]), U.dev(gold["depths"]), rec, I * n, n, W, H, cap)
    assert st == 0
    diff = counts.cpu().numpy() != gold["tiles_per_splat"]
    assert diff.mean() <= 2e-3
    tw, th = (W + 15) // 16, (H + 15) // 16
    end_bit = 32 + lib.ssb_tile_n_bits(tw * th * I)
    sk, sv = U.sort_pairs(lib, keys, vals, n_dev, cap, 0, end_bit)
    offs = U.tile_ranges(lib, sk, n_dev, cap, tw * th * I)
    # every fixture scene is free of borderline splats: the integer stages equal the reference's, bit for bit
    assert not diff.any(), (name, int(diff.sum()))
    assert M == gold["sorted_ids"].size
    assert np.array_equal(sk.cpu().numpy()[:M], gold["sorted_ids"]) and np.array_equal(sv.cpu().numpy()[:M], gold["sorted_flat"])
    assert np.array_equal(offs.cpu().numpy(), gold["offsets"])
    # the fused call (what the step runs) gives the same lists and ranges as the unfused trio
    f_keys, f_vals, f_offs, f_M = U.intersect_tiles(lib, U.dev(gold["aabb"]), U.dev(gold["depths"]), rec, I * n, n, W, H, cap, tw * th * I)
    assert f_M == M and np.array_equal(f_offs.cpu().numpy(), offs.cpu().numpy())
    assert np.array_equal(f_keys.cpu().numpy()[:M], sk.cpu().numpy()[:M]) and np.array_equal(f_vals.cpu().numpy()[:M], sv.cpu().numpy()[:M])
    # our range kernel on the reference's own sorted keys: exact
    n_ref = torch.tensor([gold["sorted_ids"].size], dtype=torch.int64, device=U.DEV)
    offs2 = U.tile_ranges(lib, U.dev(gold["sorted_ids"]), n_ref, gold["sorted_ids"].size, tw * th * I)
    assert np.array_equal(offs2.cpu().numpy(), gold["offsets"])


@pytest.mark.parametrize("name", ALL_CASES)
def test_raster_forward_vs_reference(lib, U, name):
    cfg, sp, vm, K = build_case(name)
    gold = load(name)
    I, W, H = vm.shape[0], cfg.width, cfg.height
    rec = U.pack_screen(lib, ref_proj(gold))
    n_dev = torch.tensor([gold["sorted_flat"].size], dtype=torch.int64, device=U.DEV)
    got = U.raster_fwd(lib, rec, U.dev(gold["offsets"]), U.dev(gold["sorted_flat"]), n_dev, I, W, H)
    d = np.abs(got["rgb"].cpu().numpy() - gold["render_rgb"])
    assert d.max() <= 5e-3 and (d.max(axis=1) > 1e-4).mean() <= 2e-3
    assert np.abs(got["T"].cpu().numpy() - gold["render_T"]).max() <= 5e-3
    assert (got["last_ids"].cpu().numpy() != gold["last_ids"]).mean() <= 2e-3


@pytest.mark.parametrize("name", ALL_CASES)
def test_raster_backward_vs_reference(lib, U, name):
    cfg, sp, vm, K = build_case(name)
    gold = load(name)
    I, W, H, n = vm.shape[0], cfg.width, cfg.height, cfg.n_splats
    v_rgb, v_depth, v_T = (U.dev(a) for a in raster_cotangents(name, I * H * W))
    rec = U.pack_screen(lib, ref_proj(gold))
    n_dev = torch.tensor([gold["sorted_flat"].size], dtype=torch.int64, device=U.DEV)
    render = dict(depth=U.dev(gold["render_depth"]), T=U.dev(gold["render_T"]), last_ids=U.dev(gold["last_ids"]))
    v_rec = U.raster_bwd(lib, rec, U.dev(gold["offsets"]), U.dev(gold["sorted_flat"]), n_dev, I, W, H, render, v_rgb, v_depth, v_T, pairs=I * n)
    got = U.vrec_to_arrays(v_rec, I * n)
    for k in ("v_xy", "v_depth", "v_conic", "v_opac", "v_rgb"):
        ref = gold[k].reshape(got[k].shape)
        assert U.close_frac(got[k], ref, 1e-4 * np.abs(ref).max(), 2e-3) <= 5e-3, k


@pytest.mark.parametrize("name", ALL_CASES)
def test_projection_backward_vs_reference(lib, U, name):
    cfg, sp, vm, K = build_case(name)
    gold = load(name)
    I, n = vm.shape[0], cfg.n_splats
    spd = U.splats_dev(sp)
    grads = {k: torch.zeros_like(t) for k, t in spd.items()}
    s, g = L.splats_struct(spd), L.splats_struct(grads)
    d_vm, d_K, d_aabb = U.dev(vm), U.dev(K), U.dev(gold["aabb"])
    cams = L.cameras_struct(d_vm, d_K, cfg.width, cfg.height, model=model_of(name))
    vrec = U.arrays_to_vrec({k: gold[k].reshape(I * n, -1) if gold[k].ndim > 1 else gold[k] for k in ("v_xy", "v_depth", "v_conic", "v_opac", "v_rgb")}, I * n)
    L.check(lib.ssb_project_bwd(C.byref(s), None, n, C.byref(cams), L.ptr(d_aabb), L.ptr(vrec), C.byref(g), 0, None))
    torch.cuda.synchronize()
    for k in grads:
        ref = gold["g_" + k]
        assert U.close_frac(grads[k].cpu().numpy().reshape(-1), ref.reshape(-1), 1e-4 * np.abs(ref).max(), 2e-3) <= 5e-3, k


def _shq_dev(U, tag, n):
    codes, bounds, bits, stride_arg = quant_sh_inputs(tag, n)
    d_codes, d_bounds = U.dev(codes.view(np.uint8)), U.dev(bounds)
    return L.shq_struct(d_codes, d_bounds, bits, stride_arg), (d_codes, d_bounds)


@pytest.mark.parametrize("tag", sorted(QUANT_CASES))
def test_quantised_sh_projection_vs_reference(lib, U, tag):
    """ssb_project_fwd / ssb_project_bwd reading 8/16-bit SH codes (both bound layouts) against the reference's kernels."""
    cfg, sp, vm, K = build_case(QUANT_SCENE)
    base, gold = load(QUANT_SCENE), load("quant_proj")
    I, n = vm.shape[0], cfg.n_splats
    spd = U.splats_dev(sp)
    shq, keep_alive = _shq_dev(U, tag, n)
    got = U.project_fwd(lib, spd, vm, K, cfg.width, cfg.height, shq=shq)
    aabb = got["aabb"].cpu().numpy()
    ref_aabb = gold[f"{tag}_aabb"]
    both = (ref_aabb[:, 2] > ref_aabb[:, 0]) & (aabb[:, 2] > aabb[:, 0])
    assert both.sum() > 100
    scr = U.unpack_screen(lib, got["rec"], I * n)
    assert U.close_frac(scr["rgb"][both], gold[f"{tag}_rgb"][both], 5e-3, 5e-4) <= 2e-3
    assert U.close_frac(scr["conic"][both], gold[f"{tag}_conic"][both], 5e-3, 5e-4) <= 2e-3
    grads = {k: torch.zeros_like(t) for k, t in spd.items()}
    s, g = L.splats_struct({**spd, "features_sh": None}), L.splats_struct(grads)
    d_vm, d_K, d_aabb = U.dev(vm), U.dev(K), U.dev(ref_aabb)
    cams = L.cameras_struct(d_vm, d_K, cfg.width, cfg.height)
    vrec = U.arrays_to_vrec({k: base[k].reshape(I * n, -1) if base[k].ndim > 1 else base[k] for k in ("v_xy", "v_depth", "v_conic", "v_opac", "v_rgb")}, I * n)
    L.check(lib.ssb_project_bwd(C.byref(s), C.byref(shq), n, C.byref(cams), L.ptr(d_aabb), L.ptr(vrec), C.byref(g), 0, None))
    torch.cuda.synchronize()
    for k in grads:
        ref = gold[f"{tag}_g_{k}"]
        assert U.close_frac(grads[k].cpu().numpy().reshape(-1), ref.reshape(-1), 1e-4 * np.abs(ref).max(), 2e-3) <= 5e-3, k
    del keep_alive


@pytest.mark.parametrize("tag", sorted(FPBO_RUNS))
def test_fused_backward_optimiser_vs_reference(lib, U, tag):
    """ssb_project_bwd_optimize (projection backward of all views fused with the optimiser, gradients through an L2-resident
    scratch) against the reference's fused kernel, two consecutive passes, each from the reference's state of the pass before."""
    run = FPBO_RUNS[tag]
    cfg, sp, vm, K = build_case(FPBO_SCENE)
    base, gold = load(FPBO_SCENE), load("fpbo")
    I, n, W, H = vm.shape[0], cfg.n_splats, cfg.width, cfg.height
    m = I * n
    extra = fpbo_inputs(n)
    order = ("means", "quats", "scales", "opacities", "features_dc", "features_sh")
    d_vm, d_K, d_aabb = U.dev(vm), U.dev(K), U.dev(base["aabb"])
    vrec = U.arrays_to_vrec({k: base[k].reshape(m, -1) if base[k].ndim > 1 else base[k] for k in ("v_xy", "v_depth", "v_conic", "v_opac", "v_rgb")}, m)
    d_radii = U.dev(extra["radii"])
    cams = L.cameras_struct(d_vm, d_K, W, H)
    ws = torch.zeros(int(lib.ssb_project_bwd_optimize_workspace_bytes(n)), dtype=torch.uint8, device=U.DEV)
    lr = cfg.lrs
    p = {k: U.dev(sp[k].reshape(-1)) for k in order}
    m1 = {k: torch.zeros_like(t) for k, t in p.items()}
    m2 = {k: torch.zeros_like(t) for k, t in p.items()}
    for step in (1, 2):
        if step == 2:
            p = {k: U.dev(gold[f"{tag}_p1_{k}"]) for k in order}
        d_steps = U.dev((extra["steps"] + (step - 1)).astype(np.int32)) if run["steps"] else None
        ex = L.SsbAdamExtras(*[float(x) for x in run["reg"]], run["agnostic"], d_radii.data_ptr(), d_steps.data_ptr() if d_steps is not None else None, n, None)
        acfg = L.SsbAdamConfig(lr["lr_means"], lr["lr_quats"], lr["lr_scales"], lr["lr_opacities"], lr["lr_features_dc"], lr["lr_features_sh"],
                               run["sh_reg"], 1.0, step, 0)
        s, a, b = L.splats_struct(p), L.splats_struct(m1), L.splats_struct(m2)
        L.check(lib.ssb_project_bwd_optimize(C.byref(s), None, n, C.byref(cams), L.ptr(d_aabb), L.ptr(vrec), C.byref(a), C.byref(b), None, C.byref(acfg),
                                             C.byref(ex), L.ptr(ws), ws.numel(), None))
        torch.cuda.synchronize()
        for k in order:
            assert U.close_frac(p[k].cpu().numpy(), gold[f"{tag}_p{step}_{k}"], 5e-6, 1e-4) <= 2e-3, (tag, k, step)
    for k in order:
        ref1, ref2 = gold[f"{tag}_g1_{k}"], gold[f"{tag}_g2_{k}"]
        assert U.close_frac(m1[k].cpu().numpy(), ref1, 1e-4 * np.abs(ref1).max(), 2e-3) <= 5e-3, (tag, k)
        assert U.close_frac(m2[k].cpu().numpy(), ref2, 1e-4 * np.abs(ref2).max(), 4e-3) <= 5e-3, (tag, k)
    # a workspace smaller than ssb_project_bwd_optimize_workspace_bytes is refused before anything is launched
    s2 = L.splats_struct(p)
    assert lib.ssb_project_bwd_optimize(C.byref(s2), None, n, C.byref(cams), L.ptr(d_aabb), L.ptr(vrec), C.byref(a), C.byref(b), None, C.byref(acfg),
                                        C.byref(ex), L.ptr(ws), 16, None) == L.SSB_ERR_INVALID_ARGUMENT


def _splat_block_state_close(got_vc, got_vb, got_oc, got_ob, ref_vc, ref_vb, ref_oc, ref_ob, n):
    """SH value and state codes in the per-256-splats layout, compared as the numbers they stand for (a block's bounds come from
    its extreme entries, so rounding moves codes without moving values)."""
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
def test_fused_backward_optimiser_level1_vs_reference(lib, U, tag):
    """ssb_project_bwd_optimize on the reference's level-1 layouts (16-bit SH values and 8-bit SH optimiser state with one bound per
    256 splats, SsbShAdamState::layout = SSB_SH_LAYOUT_SPLAT_BLOCKS) against the reference's fused kernel at that level, two
    passes, each from the reference's state of the pass before; SH degree 1 writes the idle bands as zero."""
    run = FPBO_L1_RUNS[tag]
    cfg, sp, vm, K = build_case(FPBO_SCENE)
    base, gold = load(FPBO_SCENE), load("fpbo_l1")
    I, n, W, H, deg = vm.shape[0], cfg.n_splats, cfg.width, cfg.height, run["degree"]
    m = I * n
    extra = fpbo_inputs(n)
    five = ("means", "quats", "scales", "opacities", "features_dc")
    d_vm, d_K, d_aabb = U.dev(vm), U.dev(K), U.dev(base["aabb"])
    vrec = U.arrays_to_vrec({k: base[k].reshape(m, -1) if base[k].ndim > 1 else base[k] for k in ("v_xy", "v_depth", "v_conic", "v_opac", "v_rgb")}, m)
    d_radii = U.dev(extra["radii"])
    cams = L.cameras_struct(d_vm, d_K, W, H, sh_degree=deg)
    ws = torch.zeros(int(lib.ssb_project_bwd_optimize_workspace_bytes(n)), dtype=torch.uint8, device=U.DEV)
    lr = cfg.lrs
    p = {k: U.dev(sp[k].reshape(-1)) for k in five}
    m1 = {k: torch.zeros_like(t) for k, t in p.items()}
    m2 = {k: torch.zeros_like(t) for k, t in p.items()}
    vc0, vb0 = encode_splat_blocks(sp["features_sh"].reshape(n, 45), 16)
    vc, vb = U.dev(vc0.view(np.uint8)), U.dev(vb0.reshape(-1))
    oc, ob = torch.zeros(n * 45 * 2, dtype=torch.uint8, device=U.DEV), torch.zeros(((n + 255) // 256) * 4, device=U.DEV)
    for step in (1, 2):
        if step == 2:
            p = {k: U.dev(gold[f"{tag}_p1_{k}"]) for k in five}
            vc, vb = U.dev(gold[f"{tag}_s1_value_codes"].view(np.uint8)), U.dev(gold[f"{tag}_s1_value_bounds"].reshape(-1))
            oc, ob = U.dev(gold[f"{tag}_s1_optim_codes"]), U.dev(gold[f"{tag}_s1_optim_bounds"].reshape(-1))
        d_steps = U.dev((extra["steps"] + (step - 1)).astype(np.int32)) if run["steps"] else None
        ex = L.SsbAdamExtras(*[float(x) for x in run["reg"]], run["agnostic"], d_radii.data_ptr(), d_steps.data_ptr() if d_steps is not None else None, n, None)
        acfg = L.SsbAdamConfig(lr["lr_means"], lr["lr_quats"], lr["lr_scales"], lr["lr_opacities"], lr["lr_features_dc"], lr["lr_features_sh"],
                               run["sh_reg"], 1.0, step, 0)
        pd, ad, bd = dict(p, features_sh=None), dict(m1, features_sh=None), dict(m2, features_sh=None)
        s, a, b = L.splats_struct(pd), L.splats_struct(ad), L.splats_struct(bd)
        shq = L.shq_struct(vc, vb, 16, 0)
        sh = L.SsbShAdamState(oc.data_ptr(), ob.data_ptr(), vc.data_ptr(), vb.data_ptr(), 16, 8, L.SH_LAYOUT_SPLAT_BLOCKS)
        L.check(lib.ssb_project_bwd_optimize(C.byref(s), C.byref(shq), n, C.byref(cams), L.ptr(d_aabb), L.ptr(vrec), C.byref(a), C.byref(b), C.byref(sh),
                                             C.byref(acfg), C.byref(ex), L.ptr(ws), ws.numel(), None))
        torch.cuda.synchronize()
        for k in five:
            assert U.close_frac(p[k].cpu().numpy(), gold[f"{tag}_p{step}_{k}"], 5e-6, 1e-4) <= 2e-3, (tag, k, step)
        gv, rv = _splat_block_state_close(vc.cpu().numpy().view(np.uint16), vb.cpu().numpy().reshape(-1, 2), oc.cpu().numpy(), ob.cpu().numpy(),
                                          gold[f"{tag}_s{step}_value_codes"], gold[f"{tag}_s{step}_value_bounds"].reshape(-1, 2),
                                          gold[f"{tag}_s{step}_optim_codes"], gold[f"{tag}_s{step}_optim_bounds"], n)
        if deg < 3:
            n_active = 3 * deg * (deg + 2)
            vbr = gold[f"{tag}_s{step}_value_bounds"].reshape(-1, 2)
            assert np.abs(gv[:, n_active:]).max() <= (vbr[:, 1] - vbr[:, 0]).max() / 65535.0
    for k in five:
        ref1, ref2 = gold[f"{tag}_g1_{k}"], gold[f"{tag}_g2_{k}"]
        assert U.close_frac(m1[k].cpu().numpy(), ref1, 1e-4 * np.abs(ref1).max(), 2e-3) <= 5e-3, (tag, k)
        assert U.close_frac(m2[k].cpu().numpy(), ref2, 1e-4 * np.abs(ref2).max(), 4e-3) <= 5e-3, (tag, k)
    # a range must start on a block of 256 splats (nothing is launched)
    assert lib.ssb_adam_step_sh_splat_blocks(L.ptr(ws), L.ptr(oc), L.ptr(ob), L.ptr(vc), L.ptr(vb), 16, 128, n - 128, n, 0, C.byref(acfg), None,
                                             None) == L.SSB_ERR_INVALID_ARGUMENT


def test_fused_backward_optimiser_level1_q16_moments_vs_reference(lib, U, oracle):
    """ssb_project_bwd_optimize_q16 on the reference's stock layouts (level 1 and the moments of the five non-SH arrays in 16-bit
    codes) against the reference's fused kernel in that configuration, two passes, each from the reference's state."""
    tag = "l1_nq"
    run = FPBO_L1_RUNS[tag]
    cfg, sp, vm, K = build_case(FPBO_SCENE)
    base, gold = load(FPBO_SCENE), load("fpbo_l1")
    I, n, W, H = vm.shape[0], cfg.n_splats, cfg.width, cfg.height
    m, blocks = I * n, (n + 255) // 256
    extra = fpbo_inputs(n)
    five = ("means", "quats", "scales", "opacities", "features_dc")
    widths = dict(oracle.Q16_ATTRS)
    d_vm, d_K, d_aabb = U.dev(vm), U.dev(K), U.dev(base["aabb"])
    vrec = U.arrays_to_vrec({k: base[k].reshape(m, -1) if base[k].ndim > 1 else base[k] for k in ("v_xy", "v_depth", "v_conic", "v_opac", "v_rgb")}, m)
    d_radii = U.dev(extra["radii"])
    cams = L.cameras_struct(d_vm, d_K, W, H)
    ws = torch.zeros(int(lib.ssb_project_bwd_optimize_workspace_bytes(n)), dtype=torch.uint8, device=U.DEV)
    lr = cfg.lrs
    p = {k: U.dev(sp[k].reshape(-1)) for k in five}
    nq_p = {k: torch.zeros(n * widths[k] * 4, dtype=torch.uint8, device=U.DEV) for k in five}
    nq_b = {k: torch.zeros(blocks * 4, device=U.DEV) for k in five}
    vc0, vb0 = encode_splat_blocks(sp["features_sh"].reshape(n, 45), 16)
    vc, vb = U.dev(vc0.view(np.uint8)), U.dev(vb0.reshape(-1))
    oc, ob = torch.zeros(n * 45 * 2, dtype=torch.uint8, device=U.DEV), torch.zeros(blocks * 4, device=U.DEV)
    for step in (1, 2):
        if step == 2:
            p = {k: U.dev(gold[f"{tag}_p1_{k}"]) for k in five}
            nq_p = {k: U.dev(gold[f"{tag}_s1_nq_{k}"]) for k in five}
            nq_b = {k: U.dev(gold[f"{tag}_s1_nqb_{k}"]) for k in five}
            vc, vb = U.dev(gold[f"{tag}_s1_value_codes"].view(np.uint8)), U.dev(gold[f"{tag}_s1_value_bounds"].reshape(-1))
            oc, ob = U.dev(gold[f"{tag}_s1_optim_codes"]), U.dev(gold[f"{tag}_s1_optim_bounds"].reshape(-1))
        d_steps = U.dev((extra["steps"] + (step - 1)).astype(np.int32))
        ex = L.SsbAdamExtras(*[float(x) for x in run["reg"]], 1, d_radii.data_ptr(), d_steps.data_ptr(), n, None)
        acfg = L.SsbAdamConfig(lr["lr_means"], lr["lr_quats"], lr["lr_scales"], lr["lr_opacities"], lr["lr_features_dc"], lr["lr_features_sh"],
                               run["sh_reg"], 1.0, step, 0)
        s = L.splats_struct(dict(p, features_sh=None))
        mom = L.SsbMomentsQ16()
        for t, k in enumerate(five):
            mom.d_packed[t], mom.d_bounds[t] = nq_p[k].data_ptr(), nq_b[k].data_ptr()
        shq = L.shq_struct(vc, vb, 16, 0)
        sh = L.SsbShAdamState(oc.data_ptr(), ob.data_ptr(), vc.data_ptr(), vb.data_ptr(), 16, 8, L.SH_LAYOUT_SPLAT_BLOCKS)
        L.check(lib.ssb_project_bwd_optimize_q16(C.byref(s), C.byref(shq), n, C.byref(cams), L.ptr(d_aabb), L.ptr(vrec), C.byref(mom), None, None,
                                                 C.byref(sh), C.byref(acfg), C.byref(ex), L.ptr(ws), ws.numel(), None))
        torch.cuda.synchronize()
        for k in five:
            assert U.close_frac(p[k].cpu().numpy(), gold[f"{tag}_p{step}_{k}"], 5e-6, 1e-4) <= 2e-3, (k, step)
            assert q16_moments_mismatch(nq_p[k].cpu().numpy(), nq_b[k].cpu().numpy(), gold[f"{tag}_s{step}_nq_{k}"], gold[f"{tag}_s{step}_nqb_{k}"], n,
                                        widths[k]) <= 5e-3, (k, step)
        _splat_block_state_close(vc.cpu().numpy().view(np.uint16), vb.cpu().numpy().reshape(-1, 2), oc.cpu().numpy(), ob.cpu().numpy(),
                                 gold[f"{tag}_s{step}_value_codes"], gold[f"{tag}_s{step}_value_bounds"].reshape(-1, 2),
                                 gold[f"{tag}_s{step}_optim_codes"], gold[f"{tag}_s{step}_optim_bounds"], n)


@pytest.mark.parametrize("bits,degree,n", [(16, 3, 700), (8, 3, 1200), (16, 2, 130), (8, 1, 513)])
def test_sh_splat_block_adam_vs_oracle(lib, U, oracle, bits, degree, n):
    """ssb_adam_step_sh_splat_blocks on its own against the oracle's restatement (pinned through fpbo_l1.npz at 16 bits): 8- and
    16-bit values, per-splat step counters, ragged last block, fewer splats than one block, active SH degrees below 3, three steps
    from a random state, in two ranges where the splat count allows."""
    rng = np.random.default_rng(17 + bits + n)
    cells, blocks = n * 45, (n + 255) // 256
    sh = (rng.normal(size=(n, 45)) * 0.2).astype(np.float32)
    vc, vb = encode_splat_blocks(sh, bits)
    oc = rng.integers(0, 256, size=cells * 2, dtype=np.uint8)
    ob = np.tile(np.array([-3.0, 3.0, 0.0, 24.0], np.float32), blocks)
    steps = rng.integers(1, 30, size=n).astype(np.int32)
    d_vc, d_vb, d_oc, d_ob = U.dev(vc.view(np.uint8)), U.dev(vb.reshape(-1)), U.dev(oc), U.dev(ob)
    h_vc, h_vb, h_oc, h_ob = vc.copy(), vb.reshape(-1).copy(), oc.copy(), ob.copy()
    lr, l2 = 2.5e-3, 0.03
    for step in (1, 2, 3):
        g = (rng.normal(size=cells) * 1e-3).astype(np.float32)
        g[rng.integers(0, cells, size=5)] = np.nan                      # non-finite gradients count as zero
        st = (steps + step).astype(np.int32) if step > 1 else None       # first a scalar step, then per-splat counters
        d_g, d_st = U.dev(g), (U.dev(st) if st is not None else None)
        acfg = L.SsbAdamConfig(0.0, 0.0, 0.0, 0.0, 0.0, lr, l2, 0.5, step, 1)
        first_ranges = [(0, n)] if n <= 256 else [(0, 256), (256, n - 256)]
        for f0, cnt in first_ranges:
            L.check(lib.ssb_adam_step_sh_splat_blocks(L.ptr(d_g), L.ptr(d_oc), L.ptr(d_ob), L.ptr(d_vc), L.ptr(d_vb), bits, f0, cnt, n, degree + 1, C.byref(acfg),
                                                      L.ptr(d_st) if d_st is not None else None, None))
        torch.cuda.synchronize()
        oracle.adam_sh_splat_blocks(np.nan_to_num(g, nan=0.0), h_oc, h_ob, h_vc, h_vb, bits, n, step, lr, l2_reg=l2, grad_scale=0.5, sh_degree=degree, steps=st)
        n_active = 3 * degree * (degree + 2)
        live = np.tile(np.arange(45) < n_active, n)
        assert not d_g.cpu().numpy()[live].any()            # cfg.zero_grad clears what was consumed
        got_vb, got_ob = d_vb.cpu().numpy(), d_ob.cpu().numpy()
        assert np.allclose(got_vb, h_vb, rtol=1e-4, atol=1e-6) and np.allclose(got_ob, h_ob, rtol=1e-4, atol=1e-5), step
        qv = float((1 << bits) - 1)
        got_codes = d_vc.cpu().numpy().view(np.uint16 if bits == 16 else np.uint8).astype(np.int64)
        dv = np.abs(got_codes - h_vc.astype(np.int64))
        assert dv.max() <= (2 if bits == 16 else 1) and (dv > 0).mean() <= 0.05, (step, dv.max(), (dv > 0).mean())
        do = np.abs(d_oc.cpu().numpy().astype(np.int64) - h_oc.astype(np.int64))
        assert do.max() <= 1 and (do > 0).mean() <= 0.02, (step, do.max(), (do > 0).mean())
        if degree < 3:        # idle cells: zero value, zero moments
            vals = decode_splat_blocks(got_codes.astype(np.uint16), got_vb.reshape(-1, 2), bits)
            assert np.abs(vals[:, n_active:]).max() <= (got_vb.reshape(-1, 2)[:, 1] - got_vb.reshape(-1, 2)[:, 0]).max() / qv
        # continue from the library's own state on both sides, so that the steps are compared one by one
        h_vc, h_vb = d_vc.cpu().numpy().view(np.uint16 if bits == 16 else np.uint8).copy(), got_vb.copy()
        h_oc, h_ob = d_oc.cpu().numpy().copy(), got_ob.copy()


@pytest.mark.parametrize("deg", [0, 1, 2])
def test_active_sh_degree_vs_reference(lib, U, deg):
    """ssb_project_fwd / ssb_project_bwd with SsbCameras::sh_degree_plus1 (the SH degree warm-up) against the reference's
    Vanilla3DGS<0>, <1>, <2> kernels; several-view and single-view backward kernels; NaNs in the unused bands are not read."""
    cfg, sp, vm, K = build_case(QUANT_SCENE)
    base, gold = load(QUANT_SCENE), load("sh_degree")
    I, n, W, H = vm.shape[0], cfg.n_splats, cfg.width, cfg.height
    m = I * n
    n_active = (deg + 1) ** 2 - 1
    sp_nan = {k: v.copy() for k, v in sp.items()}
    sp_nan["features_sh"][:, n_active:] = np.nan
    spd = U.splats_dev(sp_nan)
    d_vm, d_K = U.dev(vm), U.dev(K)
    cams = L.cameras_struct(d_vm, d_K, W, H, sh_degree=deg)
    aabb, depths, radii = torch.zeros(m, 4, device=U.DEV), torch.zeros(m, device=U.DEV), torch.zeros(n, device=U.DEV)
    rec = torch.zeros(m * L.SCREEN_REC_FLOATS, device=U.DEV)
    s = L.splats_struct(spd)
    L.check(lib.ssb_project_fwd(C.byref(s), None, n, C.byref(cams), L.ptr(aabb), L.ptr(depths), L.ptr(radii), L.ptr(rec), None))
    torch.cuda.synchronize()
    h_aabb, ref_aabb = aabb.cpu().numpy(), gold[f"d{deg}_aabb"]
    both = (ref_aabb[:, 2] > ref_aabb[:, 0]) & (h_aabb[:, 2] > h_aabb[:, 0])
    assert both.sum() > 100
    scr = U.unpack_screen(lib, rec, m)
    assert np.isfinite(scr["rgb"]).all()
    assert U.close_frac(scr["rgb"][both], gold[f"d{deg}_rgb"][both], 5e-3, 5e-4) <= 2e-3
    vrec = U.arrays_to_vrec({k: base[k].reshape(m, -1) if base[k].ndim > 1 else base[k] for k in ("v_xy", "v_depth", "v_conic", "v_opac", "v_rgb")}, m)
    d_ref_aabb = U.dev(ref_aabb)
    for views in (I, 1):
        grads = {k: torch.zeros_like(t) for k, t in spd.items()}
        g = L.splats_struct(grads)
        if views == I:
            L.check(lib.ssb_project_bwd(C.byref(s), None, n, C.byref(cams), L.ptr(d_ref_aabb), L.ptr(vrec), C.byref(g), 0, None))
        else:
            for view in range(I):
                cams1 = L.cameras_struct(d_vm[view:view + 1], d_K[view:view + 1], W, H, sh_degree=deg)
                L.check(lib.ssb_project_bwd(C.byref(s), None, n, C.byref(cams1), L.ptr(d_ref_aabb[view * n:(view + 1) * n]),
                                            L.ptr(vrec[view * n * L.SCREEN_REC_FLOATS:]), C.byref(g), 1 if view else 0, None))
        torch.cuda.synchronize()
        gsh = grads["features_sh"].cpu().numpy().reshape(n, 15, 3)
        assert np.isfinite(gsh).all() and not gsh[:, n_active:].any()
        for k in grads:
            ref = gold[f"d{deg}_g_{k}"]
            assert np.isfinite(grads[k].cpu().numpy()).all(), k
            assert U.close_frac(grads[k].cpu().numpy().reshape(-1), ref.reshape(-1), 1e-4 * max(np.abs(ref).max(), 1e-12), 2e-3) <= 5e-3, (k, views)
    bad = L.cameras_struct(d_vm, d_K, W, H, sh_degree=4)
    assert lib.ssb_project_fwd(C.byref(s), None, n, C.byref(bad), L.ptr(aabb), L.ptr(depths), L.ptr(radii), L.ptr(rec), None) == L.SSB_ERR_INVALID_ARGUMENT


@pytest.mark.parametrize("name", sorted(DIST_CASES))
def test_lens_distortion_projection_vs_reference(lib, U, name):
    """ssb_project_fwd / ssb_project_bwd with a lens-distortion tier (SsbCameras::distortion, d_dist_coeffs) against the
    reference's kernels for every (camera model, tier) pair it instantiates; the packed forward pass agrees with the
    unpacked one, and a pair outside the reference's table is refused."""
    cfg, sp, vm, K, model, tier, rows, v = dist_case_inputs(name)
    gold = load("dist_proj")
    I, n, W, H = vm.shape[0], cfg.n_splats, cfg.width, cfg.height
    m = I * n
    spd = U.splats_dev(sp)
    d_vm, d_K, d_rows = U.dev(vm), U.dev(K), U.dev(rows)
    cams = L.cameras_struct(d_vm, d_K, W, H, model=model, distortion=tier, dist_coeffs=d_rows)
    aabb, depths, radii = torch.zeros(m, 4, device=U.DEV), torch.zeros(m, device=U.DEV), torch.zeros(n, device=U.DEV)
    rec = torch.zeros(m * L.SCREEN_REC_FLOATS, device=U.DEV)
    s = L.splats_struct(spd)
    L.check(lib.ssb_project_fwd(C.byref(s), None, n, C.byref(cams), L.ptr(aabb), L.ptr(depths), L.ptr(radii), L.ptr(rec), None))
    torch.cuda.synchronize()
    h_aabb, ref_aabb = aabb.cpu().numpy(), gold[f"{name}_aabb"]
    keep_ref, keep_got = ref_aabb[:, 2] > ref_aabb[:, 0], h_aabb[:, 2] > h_aabb[:, 0]
    assert keep_ref.sum() > 100 and (keep_ref != keep_got).mean() <= 2e-3
    both = keep_ref & keep_got
    scr = U.unpack_screen(lib, rec, m)
    assert U.close_frac(h_aabb[both], ref_aabb[both], 5e-3, 5e-4) <= 2e-3
    assert U.close_frac(depths.cpu().numpy()[both], gold[f"{name}_depths"][both], 5e-3, 5e-4) <= 2e-3
    for k in ("xy", "depth", "conic", "opac", "rgb"):
        assert U.close_frac(scr[k][both], gold[f"{name}_{k}"][both], 5e-3, 5e-4) <= 2e-3, k
    assert U.close_frac(radii.cpu().numpy(), gold[f"{name}_radii"], 1e-4, 1e-3) <= 2e-3
    # backward on the reference's visible set
    grads = {k: torch.zeros_like(t) for k, t in spd.items()}
    g = L.splats_struct(grads)
    vrec = U.arrays_to_vrec(v, m)
    d_ref_aabb = U.dev(ref_aabb)
    L.check(lib.ssb_project_bwd(C.byref(s), None, n, C.byref(cams), L.ptr(d_ref_aabb), L.ptr(vrec), C.byref(g), 0, None))
    torch.cuda.synchronize()
    for k in grads:
        ref = gold[f"{name}_g_{k}"]
        assert U.close_frac(grads[k].cpu().numpy().reshape(-1), ref.reshape(-1), 1e-4 * np.abs(ref).max(), 2e-3) <= 5e-3, k
    # one view at a time (the single-view kernel variant) gives the same gradients
    if I > 1:
        grads1 = {k: torch.zeros_like(t) for k, t in spd.items()}
        g1 = L.splats_struct(grads1)
        for view in range(I):
            cams1 = L.cameras_struct(d_vm[view:view + 1], d_K[view:view + 1], W, H, model=model, distortion=tier, dist_coeffs=d_rows[view:view + 1])
            L.check(lib.ssb_project_bwd(C.byref(s), None, n, C.byref(cams1), L.ptr(d_ref_aabb[view * n:(view + 1) * n]),
                                        L.ptr(vrec[view * n * L.SCREEN_REC_FLOATS:]), C.byref(g1), 1, None))
        torch.cuda.synchronize()
        for k in grads:
            a, b = grads1[k].cpu().numpy().reshape(-1), grads[k].cpu().numpy().reshape(-1)
            assert U.close_frac(a, b, 1e-5 * np.abs(b).max(), 1e-4) <= 1e-3, k
    # the packed forward pass keeps exactly the unpacked pass's visible pairs and values
    cap = int(keep_got.sum()) + 5
    ws = torch.zeros(max(lib.ssb_project_fwd_packed_workspace_bytes(n, I), 16), dtype=torch.uint8, device=U.DEV)
    p_aabb, p_depths, p_radii = torch.zeros(cap, 4, device=U.DEV), torch.zeros(cap, device=U.DEV), torch.zeros(n, device=U.DEV)
    p_rec = torch.zeros(cap * L.SCREEN_REC_FLOATS, device=U.DEV)
    p_cam, p_gid = torch.zeros(cap, dtype=torch.int32, device=U.DEV), torch.zeros(cap, dtype=torch.int32, device=U.DEV)
    n_vis, h_n = torch.zeros(1, dtype=torch.int64, device=U.DEV), C.c_int64(-1)
    L.check(lib.ssb_project_fwd_packed(C.byref(s), None, n, C.byref(cams), L.ptr(ws), ws.numel(), L.ptr(p_aabb), L.ptr(p_depths), L.ptr(p_radii),
                                       L.ptr(p_rec), L.ptr(p_cam), L.ptr(p_gid), cap, L.ptr(n_vis), C.byref(h_n), None))
    torch.cuda.synchronize()
    assert h_n.value == keep_got.sum()
    where = np.nonzero(keep_got)[0]
    assert np.array_equal(p_cam.cpu().numpy()[:h_n.value], where // n) and np.array_equal(p_gid.cpu().numpy()[:h_n.value], where % n)
    assert torch.equal(p_aabb[:h_n.value], aabb[torch.from_numpy(where).to(U.DEV)])
    # outside the reference's table
    bad = L.cameras_struct(d_vm, d_K, W, H, model=L.CAMERA_EQUIRECT, distortion=tier, dist_coeffs=d_rows)
    assert lib.ssb_project_fwd(C.byref(s), None, n, C.byref(bad), L.ptr(aabb), L.ptr(depths), L.ptr(radii), L.ptr(rec), None) == L.SSB_ERR_UNSUPPORTED
    if model != 0:
        bad = L.cameras_struct(d_vm, d_K, W, H, model=model, distortion=L.DISTORTION_RATIONAL, dist_coeffs=d_rows)
        assert lib.ssb_project_bwd(C.byref(s), None, n, C.byref(bad), L.ptr(d_ref_aabb), L.ptr(vrec), C.byref(g), 0, None) == L.SSB_ERR_UNSUPPORTED


@pytest.mark.parametrize("key", ["ring2", "dense1", "ring2_q16_cell"])
def test_packed_projection_vs_reference(lib, U, key):
    """ssb_project_fwd_packed / ssb_project_bwd_packed against the reference's packed projection kernels: pair count and
    ids exactly, values and gradients within the projection tolerances."""
    name = key.split("_")[0]
    cfg, sp, vm, K = build_case(name)
    base, gold = load(name), load("packed_proj")
    I, n, W, H = vm.shape[0], cfg.n_splats, cfg.width, cfg.height
    spd = U.splats_dev(sp)
    shq = keep_alive = None
    if key.endswith("q16_cell"):
        shq, keep_alive = _shq_dev(U, "q16_cell", n)
    V = int(gold[f"{key}_nnz"][0])
    cap = V + 17
    ws_bytes = lib.ssb_project_fwd_packed_workspace_bytes(n, I)
    ws = torch.zeros(max(ws_bytes, 16), dtype=torch.uint8, device=U.DEV)
    p_aabb = torch.zeros(cap, 4, device=U.DEV); p_depths = torch.zeros(cap, device=U.DEV); p_radii = torch.zeros(n, device=U.DEV)
    p_rec = torch.zeros(cap * L.SCREEN_REC_FLOATS, device=U.DEV)
    p_cam = torch.full((cap,), -1, dtype=torch.int32, device=U.DEV); p_gid = torch.full((cap,), -1, dtype=torch.int32, device=U.DEV)
    n_vis = torch.zeros(1, dtype=torch.int64, device=U.DEV)
    h_n = C.c_int64(-1)
    s = L.splats_struct(spd if shq is None else {**spd, "features_sh": None})
    d_vm, d_K = U.dev(vm), U.dev(K)
    cams = L.cameras_struct(d_vm, d_K, W, H)
    L.check(lib.ssb_project_fwd_packed(C.byref(s), C.byref(shq) if shq is not None else None, n, C.byref(cams), L.ptr(ws), ws_bytes,
                                       L.ptr(p_aabb), L.ptr(p_depths), L.ptr(p_radii), L.ptr(p_rec), L.ptr(p_cam), L.ptr(p_gid), cap,
                                       L.ptr(n_vis), C.byref(h_n), None))
    assert h_n.value == V
    assert np.array_equal(p_cam.cpu().numpy()[:V], gold[f"{key}_camera_ids"]) and np.array_equal(p_gid.cpu().numpy()[:V], gold[f"{key}_gaussian_ids"])
    assert U.close_frac(p_aabb.cpu().numpy()[:V], gold[f"{key}_aabb"], 5e-3, 5e-4) <= 2e-3
    assert U.close_frac(p_depths.cpu().numpy()[:V], gold[f"{key}_depths"], 5e-3, 5e-4) <= 2e-3
    assert U.close_frac(p_radii.cpu().numpy(), gold[f"{key}_radii"], 1e-4, 1e-3) <= 2e-3
    scr = U.unpack_screen(lib, p_rec, cap)
    for k in ("xy", "depth", "conic", "opac", "rgb"):
        assert U.close_frac(scr[k][:V], gold[f"{key}_{k}"].reshape(scr[k][:V].shape), 5e-3, 5e-4) <= 2e-3, k
    # backward: the cotangents of the unpacked fixture gathered at the packed pairs
    pair = gold[f"{key}_camera_ids"].astype(np.int64) * n + gold[f"{key}_gaussian_ids"]
    v = {k: (base[k].reshape(I * n, -1) if base[k].ndim > 1 else base[k])[pair] for k in ("v_xy", "v_depth", "v_conic", "v_opac", "v_rgb")}
    vrec = torch.zeros(cap * L.SCREEN_REC_FLOATS, device=U.DEV)
    vrec[: V * L.SCREEN_REC_FLOATS] = U.arrays_to_vrec(v, V)
    grads = {k: torch.zeros_like(t) for k, t in spd.items()}
    g = L.splats_struct(grads)
    bws_bytes = lib.ssb_project_bwd_packed_workspace_bytes(n, I)
    bws = torch.zeros(max(bws_bytes, 16), dtype=torch.uint8, device=U.DEV)
    L.check(lib.ssb_project_bwd_packed(C.byref(s), C.byref(shq) if shq is not None else None, n, C.byref(cams), L.ptr(p_aabb), L.ptr(vrec),
                                       L.ptr(p_cam), L.ptr(p_gid), L.ptr(n_vis), cap, L.ptr(bws), bws_bytes, C.byref(g), 0, None))
    torch.cuda.synchronize()
    for k in grads:
        ref = gold[f"{key}_g_{k}"]
        assert U.close_frac(grads[k].cpu().numpy().reshape(-1), ref.reshape(-1), 1e-4 * np.abs(ref).max(), 2e-3) <= 5e-3, k
    del keep_alive


def test_ssim_vs_reference(lib, U):
    gold = load("ssim")
    for tag, (B, H, W, render, gt) in loss_inputs().items():
        d_render, d_gt = U.dev(render), U.dev(gt)
        d_v, d_l = torch.zeros(B * H * W, 3, device=U.DEV), torch.zeros(3, device=U.DEV)
        L.check(lib.ssb_loss_l1_ssim_fwdbwd(L.ptr(d_render), L.ptr(d_gt), B, H, W, 0.0, 0.2, L.ptr(d_v), L.ptr(d_l), None))
        torch.cuda.synchronize()
        ref = gold[f"{tag}_grad"]
        assert U.close_frac(d_v.cpu().numpy(), ref, 1e-4 * np.abs(ref).max(), 1e-3) == 0.0


def test_adam_vs_reference(lib, U):
    gold = load("adam")
    inp = adam_inputs()
    n, lr, gs = inp["n"], inp["lrs"], inp["grad_scale"]
    p = {k: U.dev(v.reshape(-1)) for k, v in inp["params"].items()}
    m1 = {k: torch.zeros_like(t) for k, t in p.items()}
    m2 = {k: torch.zeros_like(t) for k, t in p.items()}
    for step, grads in enumerate(inp["grads"], start=1):
        g = {k: U.dev(v.reshape(-1)) for k, v in grads.items()}
        cfg = L.SsbAdamConfig(lr["lr_means"], lr["lr_quats"], lr["lr_scales"], lr["lr_opacities"], lr["lr_features_dc"], lr["lr_features_sh"],
                              0.0, gs, step, 0)
        structs = [L.splats_struct(d) for d in (p, g, m1, m2)]
        L.check(lib.ssb_adam_step(*[C.byref(s) for s in structs], 0, n, C.byref(cfg), None))
        torch.cuda.synchronize()
        for k in p:
            assert U.close_frac(p[k].cpu().numpy(), gold[f"p{step}_{k}"], 5e-6, 1e-4) <= 1e-3, (k, step)
    for bits in (16, 8):
        q = inp[f"qq{bits}"]
        view = np.uint16 if bits == 16 else np.uint8
        state = [q["value_packed"], q["value_bounds"], q["optim_packed"], q["optim_bounds"]]
        for step, grad in enumerate(q["grads"], start=1):
            vp, vb, op, ob = (U.dev(a) for a in state)
            d_g = U.dev(grad)
            cfg = L.SsbAdamConfig(0, 0, 0, 0, 0, lr["lr_features_sh"], 0.0, gs, step, 0)
            L.check(lib.ssb_adam_step_sh_quantized(L.ptr(d_g), L.ptr(op), L.ptr(ob), L.ptr(vp), L.ptr(vb), bits, 0, q["numel"], q["numel"],
                                                   C.byref(cfg), None))
            torch.cuda.synchronize()
            rv, rb, ro, rob = (gold[f"qq{bits}_s{step}_{s}"] for s in ("value_packed", "value_bounds", "optim_packed", "optim_bounds"))
            dv = np.abs(vp.cpu().numpy().view(view).astype(np.int64) - rv.view(view).astype(np.int64))
            do = np.abs(op.cpu().numpy().astype(np.int64) - ro.astype(np.int64))
            assert dv.max() <= 1 and do.max() <= 1, (bits, step)
            assert (dv > 0).mean() <= 5e-2 and (do > 0).mean() <= 5e-2
            assert np.allclose(vb.cpu().numpy(), rb, rtol=1e-4, atol=1e-7)
            state = [rv, rb, ro, rob]
    q = inp["q8"]
    state = [q["x0"], np.zeros(q["numel"] * 2, np.uint8), np.zeros(((q["numel"] + 255) // 256) * 4, np.float32)]
    for step, grad in enumerate(q["grads"], start=1):
        x, op, ob = (U.dev(a) for a in state)
        d_g = U.dev(grad)
        cfg = L.SsbAdamConfig(0, 0, 0, 0, 0, lr["lr_features_sh"], 0.0, gs, step, 0)
        L.check(lib.ssb_adam_step_sh_quantized(L.ptr(d_g), L.ptr(op), L.ptr(ob), L.ptr(x), None, 32, 0, q["numel"], q["numel"], C.byref(cfg), None))
        torch.cuda.synchronize()
        rx, ro, rob = (gold[f"q8_s{step}_{s}"] for s in ("x", "optim_packed", "optim_bounds"))
        do = np.abs(op.cpu().numpy().astype(np.int64) - ro.astype(np.int64))
        assert do.max() <= 1 and (do > 0).mean() <= 5e-2, step
        assert U.close_frac(x.cpu().numpy(), rx, 5e-6, 1e-4) <= 1e-3, step
        state = [rx, ro, rob]


@pytest.mark.gpu
def test_adam_extras_vs_reference(lib, U):
    """ssb_adam_step_ex (regularisers, per-splat step counters, scale-agnostic mean) and the quantised SH step with
    counters against the reference's kernels."""
    gold = load("adam")
    inp = adam_inputs()
    ex, lr, gs, n = inp["ex"], inp["lrs"], inp["grad_scale"], inp["n"]
    d_radii, d_steps = U.dev(ex["radii"]), U.dev(ex["steps"])
    reg = [float(v) for v in ex["reg"]]
    for tag, agnostic in (("exA", 0), ("exB", 1)):
        p = {k: U.dev(v.reshape(-1)) for k, v in inp["params"].items()}
        m1 = {k: torch.zeros_like(t) for k, t in p.items()}
        m2 = {k: torch.zeros_like(t) for k, t in p.items()}
        d_score = torch.zeros(n, device=U.DEV)
        extras = L.SsbAdamExtras(*reg, agnostic, d_radii.data_ptr(), d_steps.data_ptr(), n, d_score.data_ptr())
        for step, grads in enumerate(inp["grads"], start=1):
            g = {k: U.dev(v.reshape(-1)) for k, v in grads.items()}
            cfg = L.SsbAdamConfig(lr["lr_means"], lr["lr_quats"], lr["lr_scales"], lr["lr_opacities"], lr["lr_features_dc"], lr["lr_features_sh"],
                                  0.0, gs, step, 0)
            structs = [L.splats_struct(d) for d in (p, g, m1, m2)]
            # two calls over half the splats each: the range offsets the counters and the radii
            half = n // 2
            L.check(lib.ssb_adam_step_ex(*[C.byref(s) for s in structs], 0, half, C.byref(cfg), C.byref(extras), None))
            L.check(lib.ssb_adam_step_ex(*[C.byref(s) for s in structs], half, n - half, C.byref(cfg), C.byref(extras), None))
            torch.cuda.synchronize()
            for k in (list(p) if not agnostic else ["means"]):
                assert U.close_frac(p[k].cpu().numpy(), gold[f"{tag}_p{step}_{k}"], 5e-6, 1e-4) <= 1e-3, (tag, k, step)
            if not agnostic and step == 1:
                assert np.allclose(d_score.cpu().numpy(), gold["exA_densify_score"], rtol=1e-4, atol=1e-9)
    q = inp["qq16"]
    n_sp = (q["numel"] + 44) // 45
    steps_q = U.dev(np.ascontiguousarray(np.resize(ex["steps"], n_sp)))
    vp, vb, op, ob = (U.dev(q[k]) for k in ("value_packed", "value_bounds", "optim_packed", "optim_bounds"))
    d_g = U.dev(q["grads"][0])
    cfg = L.SsbAdamConfig(0, 0, 0, 0, 0, lr["lr_features_sh"], 0.0, gs, 1, 0)
    L.check(lib.ssb_adam_step_sh_quantized_ex(L.ptr(d_g), L.ptr(op), L.ptr(ob), L.ptr(vp), L.ptr(vb), 16, 8, 0, q["numel"], q["numel"],
                                              C.byref(cfg), L.ptr(steps_q), 45, None))
    torch.cuda.synchronize()
    dv = np.abs(vp.cpu().numpy().view(np.uint16).astype(np.int64) - gold["qqs_value_packed"].view(np.uint16).astype(np.int64))
    do = np.abs(op.cpu().numpy().astype(np.int64) - gold["qqs_optim_packed"].astype(np.int64))
    assert dv.max() <= 1 and do.max() <= 1 and (dv > 0).mean() <= 5e-2 and (do > 0).mean() <= 5e-2
    assert np.allclose(vb.cpu().numpy(), gold["qqs_value_bounds"], rtol=1e-4, atol=1e-7)


@pytest.mark.gpu
def test_adam_16bit_non_sh_moments_vs_reference(lib, U):
    """ssb_adam_step_q16 against the reference's non_sh_quant kernel, every step from the reference's parameters and codes of the
    step before; then the same update in two calls over block-aligned ranges."""
    from test_golden_cpu import Q16_ORDER, q16_code_diff
    gold = load("adam")
    inp = adam_inputs()
    ex, lr, gs, n = inp["ex"], inp["lrs"], inp["grad_scale"], inp["n"]
    widths = dict(means=3, quats=4, scales=3, opacities=1, features_dc=3)
    nblk = (n + 255) // 256
    d_steps = U.dev(ex["steps"])
    reg = [float(v) for v in ex["reg"]]

    def run(tag, use_ex, step, grads, ranges):
        if step == 1:
            p = {k: U.dev(inp["params"][k].reshape(-1)) for k in Q16_ORDER}
            packed = {k: torch.zeros(n * widths[k] * 4, dtype=torch.uint8, device=U.DEV) for k in Q16_ORDER}
            bounds = {k: torch.zeros(nblk * 4, device=U.DEV) for k in Q16_ORDER}
        else:
            p = {k: U.dev(gold[f"{tag}_p{step - 1}_{k}"]) for k in Q16_ORDER}
            packed = {k: U.dev(gold[f"{tag}_q{step - 1}_{k}"]) for k in Q16_ORDER}
            bounds = {k: U.dev(gold[f"{tag}_b{step - 1}_{k}"]) for k in Q16_ORDER}
        g = {k: U.dev(grads[k].reshape(-1)) for k in Q16_ORDER}
        mom = L.SsbMomentsQ16()
        for t, k in enumerate(Q16_ORDER):
            mom.d_packed[t], mom.d_bounds[t] = packed[k].data_ptr(), bounds[k].data_ptr()
        cfg = L.SsbAdamConfig(lr["lr_means"], lr["lr_quats"], lr["lr_scales"], lr["lr_opacities"], lr["lr_features_dc"], 0.0,
                              inp["nq_sh_reg_weight"], gs, step, 0)
        extras = L.SsbAdamExtras(*reg, 0, None, d_steps.data_ptr(), n, None) if use_ex else None
        ps, gs_ = L.splats_struct({**p, "features_sh": None}), L.splats_struct({**g, "features_sh": None})
        for first, count in ranges:
            L.check(lib.ssb_adam_step_q16(C.byref(ps), C.byref(gs_), C.byref(mom), first, count, C.byref(cfg),
                                          C.byref(extras) if extras is not None else None, None))
        torch.cuda.synchronize()
        return p, packed, bounds

    for tag, use_ex in (("nq", False), ("nqx", True)):
        for step, grads in enumerate(inp["grads"], start=1):
            for ranges in ([(0, n)], [(0, 256), (256, n - 256)]):
                p, packed, bounds = run(tag, use_ex, step, grads, ranges)
                for k in Q16_ORDER:
                    assert U.close_frac(p[k].cpu().numpy(), gold[f"{tag}_p{step}_{k}"], 5e-6, 1e-4) <= 1e-3, (tag, k, step)
                    assert np.allclose(bounds[k].cpu().numpy(), gold[f"{tag}_b{step}_{k}"], rtol=1e-4, atol=1e-6), (tag, k, step)
                    worst, frac = q16_code_diff(packed[k].cpu().numpy(), gold[f"{tag}_q{step}_{k}"])
                    assert worst <= 2 and frac <= 0.15, (tag, k, step, worst, frac)
    # a range that does not start on a block of 256 splats is refused
    p, packed, bounds = run("nq", False, 1, inp["grads"][0], [])
    mom = L.SsbMomentsQ16()
    for t, k in enumerate(Q16_ORDER):
        mom.d_packed[t], mom.d_bounds[t] = packed[k].data_ptr(), bounds[k].data_ptr()
    cfg = L.SsbAdamConfig(0, 0, 0, 0, 0, 0, 0, 1.0, 1, 0)
    ps = L.splats_struct({**p, "features_sh": None})
    assert lib.ssb_adam_step_q16(C.byref(ps), C.byref(ps), C.byref(mom), 100, 10, C.byref(cfg), None, None) == L.SSB_ERR_INVALID_ARGUMENT


def test_adam_4bit_state_vs_reference(lib, U):
    """ssb_adam_step_sh_quantized_ex with optim_bits = 4 against the reference's kernels, each step from the reference's state."""
    gold = load("adam")
    inp = adam_inputs()
    lr, gs = inp["lrs"], inp["grad_scale"]

    def nibble_diff(a, b):
        a, b = a.astype(np.int64), b.astype(np.int64)
        return np.maximum(np.abs((a & 15) - (b & 15)), np.abs((a >> 4) - (b >> 4)))

    q = inp["q8"]
    state = [q["x0"], np.zeros(q["numel"], np.uint8), np.zeros(((q["numel"] + 255) // 256) * 4, np.float32)]
    for step, grad in enumerate(q["grads"], start=1):
        x, op, ob = (U.dev(a) for a in state)
        d_g = U.dev(grad)
        cfg = L.SsbAdamConfig(0, 0, 0, 0, 0, lr["lr_features_sh"], 0.0, gs, step, 0)
        L.check(lib.ssb_adam_step_sh_quantized_ex(L.ptr(d_g), L.ptr(op), L.ptr(ob), L.ptr(x), None, 32, 4, 0, q["numel"], q["numel"], C.byref(cfg),
                                                  None, 1, None))
        torch.cuda.synchronize()
        rx, ro, rob = (gold[f"q4_s{step}_{s}"] for s in ("x", "optim_packed", "optim_bounds"))
        do = nibble_diff(op.cpu().numpy(), ro)
        assert do.max() <= 1 and (do > 0).mean() <= 5e-2, step
        assert U.close_frac(x.cpu().numpy(), rx, 5e-6, 1e-4) <= 1e-3, step
        state = [rx, ro, rob]
    q = inp["qq16"]
    state = [q["value_packed"], q["value_bounds"], np.zeros(q["numel"], np.uint8), np.zeros(((q["numel"] + 255) // 256) * 4, np.float32)]
    for step, grad in enumerate(q["grads"][:2], start=1):
        vp, vb, op, ob = (U.dev(a) for a in state)
        d_g = U.dev(grad)
        cfg = L.SsbAdamConfig(0, 0, 0, 0, 0, lr["lr_features_sh"], 0.0, gs, step, 0)
        L.check(lib.ssb_adam_step_sh_quantized_ex(L.ptr(d_g), L.ptr(op), L.ptr(ob), L.ptr(vp), L.ptr(vb), 16, 4, 0, q["numel"], q["numel"],
                                                  C.byref(cfg), None, 1, None))
        torch.cuda.synchronize()
        rv, rb, ro, rob = (gold[f"qq16o4_s{step}_{s}"] for s in ("value_packed", "value_bounds", "optim_packed", "optim_bounds"))
        dv = np.abs(vp.cpu().numpy().view(np.uint16).astype(np.int64) - rv.view(np.uint16).astype(np.int64))
        do = nibble_diff(op.cpu().numpy(), ro)
        assert dv.max() <= 1 and do.max() <= 1 and (dv > 0).mean() <= 5e-2 and (do > 0).mean() <= 5e-2, step
        assert np.allclose(vb.cpu().numpy(), rb, rtol=1e-4, atol=1e-7)
        state = [rv, rb, ro, rob]


@pytest.mark.gpu
@pytest.mark.parametrize("name", ACCUM_CASES)
def test_raster_accum_weight_vs_reference(lib, U, name):
    """ssb_raster_bwd_accum: the densification weights against the reference's kernel, and the gradients unchanged by the mode."""
    cfg, sp, vm, K = build_case(name)
    gold, acc_gold = load(name), load("accum")
    I, W, H, n = vm.shape[0], cfg.width, cfg.height, cfg.n_splats
    v_rgb, v_depth, v_T = (U.dev(a) for a in raster_cotangents(name, I * H * W))
    rec = U.pack_screen(lib, ref_proj(gold))
    n_dev = torch.tensor([gold["sorted_flat"].size], dtype=torch.int64, device=U.DEV)
    render = dict(depth=U.dev(gold["render_depth"]), T=U.dev(gold["render_T"]), last_ids=U.dev(gold["last_ids"]))
    offs, fl = U.dev(gold["offsets"]), U.dev(gold["sorted_flat"])
    wmap = U.dev(accum_weight_map(name, I * H * W))
    base = U.vrec_to_arrays(U.raster_bwd(lib, rec, offs, fl, n_dev, I, W, H, render, v_rgb, v_depth, v_T, pairs=I * n), I * n)
    for mode, tag in ((L.SSB_ACCUM_MAX, "max"), (L.SSB_ACCUM_SUM, "sum"), (L.SSB_ACCUM_AVG, "avg")):
        for with_depth in (True, False):
            v_rec = torch.zeros(I * n * L.SCREEN_REC_FLOATS, device=U.DEV)
            acc, den = torch.zeros(n, device=U.DEV), torch.zeros(n, device=U.DEV)
            L.check(lib.ssb_raster_bwd_accum(L.ptr(rec), I * n, L.ptr(offs), L.ptr(fl), fl.numel(), L.ptr(n_dev), I, W, H, L.ptr(render["depth"]), L.ptr(render["T"]),
                                             L.ptr(render["last_ids"]), L.ptr(v_rgb), L.ptr(v_depth) if with_depth else None, L.ptr(v_T), L.ptr(v_rec),
                                             mode, L.ptr(wmap), n, None, L.ptr(acc), L.ptr(den), None))
            torch.cuda.synchronize()
            ref = acc_gold[f"{name}_{tag}"]
            assert U.close_frac(acc.cpu().numpy(), ref, 1e-5 * ref.max(), 2e-3) <= 5e-3, (tag, with_depth)
            if mode == L.SSB_ACCUM_AVG:
                ref_den = acc_gold[f"{name}_avg_den"]
                assert U.close_frac(den.cpu().numpy(), ref_den, 1e-5 * ref_den.max(), 2e-3) <= 5e-3
            if with_depth:
                got = U.vrec_to_arrays(v_rec, I * n)
                for k in base:
                    assert U.close_frac(got[k], base[k], 1e-5 * np.abs(base[k]).max(), 1e-4) <= 1e-3, (k, tag)


@pytest.mark.gpu
def test_ssim_loss_map_vs_reference(lib, U):
    """ssb_loss_l1_ssim_fwdbwd_map: the densification loss map against the reference's kernel; gradient and scalars as without a map."""
    gold = load("ssim_map")
    for tag, (B, H, W, render, gt) in loss_inputs().items():
        d_r, d_g = U.dev(render), U.dev(gt)
        v0 = torch.zeros(B * H * W, 3, device=U.DEV); l0 = torch.zeros(3, device=U.DEV)
        L.check(lib.ssb_loss_l1_ssim_fwdbwd(L.ptr(d_r), L.ptr(d_g), B, H, W, 0.8, 0.2, L.ptr(v0), L.ptr(l0), None))
        for mode in (1, 2, 3):
            v = torch.zeros(B * H * W, 3, device=U.DEV); losses = torch.zeros(3, device=U.DEV)
            lm = U.dev(loss_map_base(tag, B * H * W))
            L.check(lib.ssb_loss_l1_ssim_fwdbwd_map(L.ptr(d_r), L.ptr(d_g), B, H, W, 0.8, 0.2, L.ptr(v), L.ptr(losses), mode, LOSS_MAP_WEIGHT, L.ptr(lm), None))
            torch.cuda.synchronize()
            ref = gold[f"{tag}_map{mode}"]
            assert U.close_frac(lm.cpu().numpy(), ref, 2e-5, 1e-4) <= 1e-3, (tag, mode)
            assert torch.equal(v, v0) and torch.allclose(losses, l0, rtol=1e-5, atol=1e-7)


@pytest.mark.gpu
def test_masked_ssim_vs_reference(lib, U):
    """ssb_loss_multi_scale with one level and a mask: the SSIM gradient, its mean and the loss-map variants against the
    reference's masked kernel (mask of the image's size, and one of another size that is nearest-sampled)."""
    from golden_cases import loss_masks
    gold = load("ssim_masked")
    w_ssim = 0.2
    for tag, (B, H, W, render, gt) in loss_inputs().items():
        d_r, d_g = U.dev(render), U.dev(gt)
        for kind, mask in loss_masks(tag, B, H, W).items():
            d_m = torch.from_numpy(mask).to(U.DEV)
            for mode in (0, 2, 3, 4):
                cfg = L.SsbLossConfig(0.0, w_ssim, 1, mode, d_m.data_ptr(), mask.shape[1], mask.shape[2])
                need = lib.ssb_loss_workspace_bytes(B, H, W, C.byref(cfg))
                ws = torch.empty(need, dtype=torch.uint8, device=U.DEV)
                v = torch.zeros(B * H * W, 3, device=U.DEV); losses = torch.zeros(3, device=U.DEV); lm = torch.zeros(B * H * W, device=U.DEV)
                L.check(lib.ssb_loss_multi_scale(L.ptr(d_r), L.ptr(d_g), B, H, W, C.byref(cfg), L.ptr(v), L.ptr(losses), L.ptr(lm), L.ptr(ws), need, None))
                torch.cuda.synchronize()
                if mode == 0:
                    ref = gold[f"{tag}_{kind}_grad"]
                    assert U.close_frac(v.cpu().numpy(), ref, 2e-6 * np.abs(ref).max(), 2e-4) <= 1e-3, (tag, kind)
                    assert abs(losses[1].item() - gold[f"{tag}_{kind}_ssim"][0]) <= 2e-5
                else:
                    # the reference adds weight * (1 - v) onto a seeded map; the library overwrites with w_ssim * (1 - v)
                    ref = (gold[f"{tag}_{kind}_map{mode - 1}"] - loss_map_base(tag, B * H * W)) * (w_ssim / LOSS_MAP_WEIGHT)
                    assert U.close_frac(lm.cpu().numpy(), ref, 2e-5, 1e-4) <= 1e-3, (tag, kind, mode)


@pytest.mark.gpu
def test_live_tile_map_and_intersection_vs_reference(lib, U):
    """ssb_tile_active and the *_live intersection calls against the reference's tile_active_kernel and its intersection with
    a live-tile map: the map, the per-splat counts, the sorted lists and the ranges, bit for bit; fused call = unfused trio."""
    from golden_cases import LIVE_TILE_CASE, tile_masks
    cfg, sp, vm, K = build_case(LIVE_TILE_CASE)
    gold, live_gold = load(LIVE_TILE_CASE), load("tiles_live")
    n, W, H, I = cfg.n_splats, cfg.width, cfg.height, vm.shape[0]
    rec = U.pack_screen(lib, ref_proj(gold))
    tw, th = (W + 15) // 16, (H + 15) // 16
    cap = 64 * n
    end_bit = 32 + lib.ssb_tile_n_bits(tw * th * I)
    aabb, depths = U.dev(gold["aabb"]), U.dev(gold["depths"])
    for kind, mask in tile_masks(I, H, W).items():
        d_mask = torch.from_numpy(mask).to(U.DEV)
        live = torch.full((I * tw * th,), -1, dtype=torch.int32, device=U.DEV)
        L.check(lib.ssb_tile_active(L.ptr(d_mask), I, mask.shape[1], mask.shape[2], W, H, L.ptr(live), None))
        torch.cuda.synchronize()
        assert np.array_equal(live.cpu().numpy(), live_gold[f"{kind}_tile_active"]), kind
        st, M, counts, cum, keys, vals, n_dev = U.tile_keys(lib, aabb, depths, rec, I * n, n, W, H, cap, tile_active=live)
        assert st == 0 and M == live_gold[f"{kind}_sorted_ids"].size
        assert np.array_equal(counts.cpu().numpy(), live_gold[f"{kind}_tiles_per_splat"]), kind
        sk, sv = U.sort_pairs(lib, keys, vals, n_dev, cap, 0, end_bit)
        offs = U.tile_ranges(lib, sk, n_dev, cap, tw * th * I)
        assert np.array_equal(sk.cpu().numpy()[:M], live_gold[f"{kind}_sorted_ids"]) and np.array_equal(sv.cpu().numpy()[:M], live_gold[f"{kind}_sorted_flat"])
        assert np.array_equal(offs.cpu().numpy(), live_gold[f"{kind}_offsets"]), kind
        f_keys, f_vals, f_offs, f_M = U.intersect_tiles(lib, aabb, depths, rec, I * n, n, W, H, cap, tw * th * I, tile_active=live)
        assert f_M == M and np.array_equal(f_offs.cpu().numpy(), live_gold[f"{kind}_offsets"])
        assert np.array_equal(f_keys.cpu().numpy()[:M], live_gold[f"{kind}_sorted_ids"]) and np.array_equal(f_vals.cpu().numpy()[:M], live_gold[f"{kind}_sorted_flat"])


@pytest.mark.gpu
def test_multi_scale_loss_vs_reference(lib, U):
    """ssb_loss_multi_scale against the reference's own multi-scale driver: gradient, loss scalars and loss maps."""
    from golden_cases import MULTI_SCALE_RUNS, loss_masks
    gold = load("loss_multi")
    for tag, (B, H, W, render, gt) in loss_inputs().items():
        d_r, d_g = U.dev(render), U.dev(gt)
        masks = dict(loss_masks(tag, B, H, W), none=None)
        for kind, scales in MULTI_SCALE_RUNS:
            key = f"{tag}_{kind}_{scales}"
            mask = masks[kind]
            d_m = torch.from_numpy(mask).to(U.DEV) if mask is not None else None
            for mode in (0, 1, 3):
                cfg = L.SsbLossConfig(0.8, 0.2, scales, mode, d_m.data_ptr() if d_m is not None else None,
                                      mask.shape[1] if mask is not None else 0, mask.shape[2] if mask is not None else 0)
                need = lib.ssb_loss_workspace_bytes(B, H, W, C.byref(cfg))
                ws = torch.empty(need, dtype=torch.uint8, device=U.DEV)
                v = torch.zeros(B * H * W, 3, device=U.DEV); losses = torch.zeros(3, device=U.DEV); lm = torch.zeros(B * H * W, device=U.DEV)
                L.check(lib.ssb_loss_multi_scale(L.ptr(d_r), L.ptr(d_g), B, H, W, C.byref(cfg), L.ptr(v), L.ptr(losses), L.ptr(lm), L.ptr(ws), need, None))
                torch.cuda.synchronize()
                if mode == 0:
                    ref = gold[key + "_grad"]
                    assert U.close_frac(v.cpu().numpy(), ref, 2e-6 * np.abs(ref).max(), 2e-4) <= 1e-3, key
                    rgb_loss, ssim = gold[key + "_scalars"]
                    assert abs(0.8 * losses[0].item() - rgb_loss) <= 1e-5 * abs(rgb_loss) + 1e-7
                    assert abs(losses[1].item() - ssim) <= 2e-5
                else:
                    assert U.close_frac(lm.cpu().numpy(), gold[key + f"_map{mode}"], 2e-5, 1e-4) <= 1e-3, (key, mode)


@pytest.mark.gpu
def test_densify_per_step_vs_reference(lib, U):
    """ssb_densify_update_scores against the reference's scale-clip, quotient, score-update, quantile-clip kernels, and
    ssb_densify_add_noise against the reference's noise in distribution."""
    from golden_cases import DENSIFY_SCORE_RUNS, densify_inputs
    from tests import densify_util as D
    gold = load("densify")
    inp = densify_inputs()
    n = inp["radii"].shape[0]
    ws_bytes = lib.ssb_densify_workspace_bytes(n)
    ws = torch.zeros(ws_bytes, dtype=torch.uint8, device=U.DEV)
    for name, kw in DENSIFY_SCORE_RUNS:
        a = D.score_run_args(kw)
        radii, scales, opacs = U.dev(inp["radii"]), U.dev(inp["log_scales"]), U.dev(inp["logit_opacs"])
        acc = U.dev(inp["accum_buffer"]) if a["use_accum"] else None
        aw = U.dev(inp["accum_weight"]) if a["use_weights"] else None
        den = U.dev(inp["accum_den"]) if a["accum_mode"] == 3 else None
        wg = U.dev(inp["world_grad"]) if a["use_world"] else None
        sample = torch.zeros(n, 2, device=U.DEV) if a["want_sample"] else None
        cfg = L.SsbDensifyScoreConfig(a["max_screen_size"], a["clip_hardness"], a["max_world_size"], a["accum_mode"], a["score_mode"], a["blend_w"],
                                      a["score_power"], a["clip_quantile"], a["final_power"])
        L.check(lib.ssb_densify_update_scores(C.byref(cfg), n, L.ptr(radii), L.ptr(scales), L.ptr(opacs), L.ptr(aw), L.ptr(den), L.ptr(wg), L.ptr(acc),
                                              L.ptr(sample), L.ptr(ws), ws_bytes, None))
        torch.cuda.synchronize()
        host = lambda t: t.cpu().numpy() if t is not None else None
        D.check_score_run(name, dict(log_scales=host(scales), accum_weight=host(aw), accum_buffer=host(acc), sample_score=host(sample)), gold)
    for revised, scaler in ((0, 2e3), (1, 5e5 * 1.6e-4)):
        moved, radii, scales, quats, opacs = (U.dev(inp[k]) for k in ("means", "radii", "log_scales", "quats", "logit_opacs"))
        L.check(lib.ssb_densify_add_noise(n, scaler, revised, L.ptr(radii), L.ptr(moved), L.ptr(scales), L.ptr(quats), L.ptr(opacs), None))
        torch.cuda.synchronize()
        D.check_noise(inp, moved.cpu().numpy(), scaler, revised, reference_moved=gold[f"noise{revised}_means"])
        again = U.dev(inp["means"])
        L.check(lib.ssb_densify_add_noise(n, scaler, revised, L.ptr(radii), L.ptr(again), L.ptr(scales), L.ptr(quats), L.ptr(opacs), None))
        torch.cuda.synchronize()
        assert torch.equal(again, moved)                       # a function of its input


def _densify_state(lib, U, st):
    """Device copies of a densify_split_inputs() state and the SsbDensifyState over them."""
    d = {k: (U.dev(v) if isinstance(v, np.ndarray) else None) for k, v in st.items() if not isinstance(v, int)}
    sp = lambda pre: L.splats_struct({a: d.get(pre + a) for a in ("means", "quats", "scales", "opacities", "features_dc", "features_sh")})
    ds = L.SsbDensifyState()
    ds.params, ds.m1, ds.m2 = sp(""), sp("m1_"), sp("m2_")
    ds.sh = L.SsbShAdamState(d["sh_optim_packed"].data_ptr() if d.get("sh_optim_packed") is not None else None,
                             d["sh_optim_bounds"].data_ptr() if d.get("sh_optim_bounds") is not None else None,
                             d["sh_value_packed"].data_ptr() if d.get("sh_value_packed") is not None else None,
                             d["sh_value_bounds"].data_ptr() if d.get("sh_value_bounds") is not None else None,
                             st.get("sh_value_bits", 32), st.get("sh_optim_bits", 0))
    ds.d_accum_buffer, ds.d_sample_score, ds.d_steps = d["accum"].data_ptr(), d["weights"].data_ptr(), d["steps"].data_ptr()
    return d, ds


@pytest.mark.gpu
@pytest.mark.parametrize("quant", [False, True])
def test_densify_relocation_and_growth_vs_reference(lib, U, oracle, quant):
    """ssb_densify_relocate / ssb_densify_add: exactly the oracle's result (same draw, same slots), and the reference's kernels'
    state up to the draw's cut and the reference's own slot order."""
    import copy
    from golden_cases import DENSIFY_SPLIT as D, densify_split_inputs
    from tests import densify_util as DU
    gold = load("densify_split")
    tag = "q" if quant else "f"
    st = densify_split_inputs(quant)
    before = copy.deepcopy(st)
    dead = DU.dead_mask(st, D["cur_n"], D["min_opacity"])
    d, ds = _densify_state(lib, U, st)
    ws_bytes = lib.ssb_densify_relocate_workspace_bytes(D["cap"])
    ws = torch.zeros(ws_bytes, dtype=torch.uint8, device=U.DEV)
    n_dead = torch.full((1,), -1, dtype=torch.int32, device=U.DEV)

    def host_state():
        out = {k: (t.cpu().numpy().reshape(before[k].shape) if t is not None else None) for k, t in d.items()}
        out.update({k: v for k, v in st.items() if isinstance(v, int)})
        return out

    def ref_state(phase):
        out = {k[len(tag) + len(phase) + 2:]: gold[k] for k in gold if k.startswith(f"{tag}_{phase}_")}
        return {k: (v.reshape(before[k].shape) if isinstance(before.get(k), np.ndarray) else v) for k, v in out.items()}

    def same_as_oracle(ours, want):
        for k, v in want.items():
            if isinstance(v, np.ndarray) and k not in ("weights",):
                if v.dtype.kind == "f":
                    assert np.allclose(ours[k], v, rtol=2e-5, atol=2e-6, equal_nan=True), k
                elif k in ("sh_value_packed",):
                    assert np.abs(ours[k].view(np.uint16).astype(np.int64) - v.view(np.uint16).astype(np.int64)).max() <= 1, k
                else:
                    assert np.array_equal(ours[k], v), k

    L.check(lib.ssb_densify_relocate(C.byref(ds), D["cur_n"], D["min_opacity"], D["split_k"], D["seed"], L.ptr(ws), ws_bytes, L.ptr(n_dead), None))
    torch.cuda.synchronize()
    assert n_dead.item() == dead.sum()
    ours = host_state()
    want = copy.deepcopy(before)
    oracle.densify_split(0, want, D["cur_n"], D["seed"], D["split_k"], D["min_opacity"])
    same_as_oracle(ours, want)
    DU.check_split_state(before, ours, ref_state("reloc"), D["cur_n"], 0, 0, dead, quant)
    mid = copy.deepcopy(ours)
    L.check(lib.ssb_densify_add(C.byref(ds), D["cur_n"], D["num_new"], D["split_k"], D["seed"] + 1, L.ptr(ws), ws_bytes, None))
    torch.cuda.synchronize()
    ours2 = host_state()
    want2 = copy.deepcopy(want)
    oracle.densify_split(1, want2, D["cur_n"], D["seed"] + 1, D["split_k"], num_new=D["num_new"])
    same_as_oracle(ours2, want2)
    # against the reference: its growth step started from ITS relocated state, so compare structure slot by slot on its own terms
    ref_mid, ref_add = ref_state("reloc"), ref_state("add")
    for k in ("weights", "sh_optim_bounds", "sh_value_bounds"):
        if before.get(k) is not None:
            ref_mid[k] = before[k]
    st_ref = copy.deepcopy(ref_mid)
    for k in DU.SPLIT_ATTRS:
        for pre in ("", "m1_", "m2_"):
            st_ref.setdefault(pre + k, None)
    st_ref.update({k: v for k, v in st.items() if isinstance(v, int)})
    base = copy.deepcopy(st_ref)
    oracle.densify_split(1, st_ref, D["cur_n"], D["seed"] + 1, D["split_k"], num_new=D["num_new"])
    DU.check_split_state(base, st_ref, ref_add, D["cur_n"], D["cur_n"], D["num_new"], None, quant)
    DU.check_split_state(mid, ours2, ours2, D["cur_n"], D["cur_n"], D["num_new"], None, quant)
