"""GPU parity of the loss and optimiser kernels and of whole iterations driven
through ssb_step_views / Trainer, plus size-independent properties at the full
benchmark size (sortedness, permutation checksum, range monotonicity)."""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")

from spirula_studio_b200 import lib as L, scenes  # noqa: E402

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


@pytest.mark.parametrize("B,H,W", [(1, 240, 320), (2, 67, 101), (1, 16, 16), (1, 5, 7)])
def test_loss_l1_ssim(lib, U, oracle, B, H, W):
    rng = np.random.default_rng(B * 1000 + H)
    render = rng.random((B * H * W, 3), dtype=np.float32)
    gt = rng.random((B * H * W, 3), dtype=np.float32)
    ref_v, ref_l = oracle.loss_l1_ssim(render, gt, B, H, W, 0.8, 0.2)
    d_v = torch.full((B * H * W, 3), 3.0, device=U.DEV)
    d_l = torch.full((3,), 5.0, device=U.DEV)
    d_render, d_gt = U.dev(render), U.dev(gt)
    L.check(lib.ssb_loss_l1_ssim_fwdbwd(L.ptr(d_render), L.ptr(d_gt), B, H, W, 0.8, 0.2, L.ptr(d_v), L.ptr(d_l), None))
    torch.cuda.synchronize()
    assert np.allclose(d_l.cpu().numpy(), ref_l, rtol=2e-4, atol=2e-6)
    scale = np.abs(ref_v).max()
    assert U.close_frac(d_v.cpu().numpy(), ref_v, 1e-4 * scale, 1e-3) == 0.0


def _np_state(sp):
    p = {k: np.ascontiguousarray(v).copy() for k, v in sp.items()}
    z = lambda: {k: np.zeros_like(v) for k, v in p.items()}
    return p, z(), z()


def test_adam_fp32(lib, U, oracle):
    cfg = scenes.scaled(scenes.CONFIGS["plumbing_50k"], n_splats=5003)
    sp = scenes.make_splats(cfg)
    rng = np.random.default_rng(8)
    p, m1, m2 = _np_state(sp)
    dp = {k: U.dev(v.reshape(-1)) for k, v in p.items()}
    dm1 = {k: torch.zeros_like(t) for k, t in dp.items()}
    dm2 = {k: torch.zeros_like(t) for k, t in dp.items()}
    lrs = cfg.lrs
    for step in (1, 2, 3):
        g = {k: (rng.normal(size=v.shape) * 1e-3).astype(np.float32) for k, v in p.items()}
        if step == 2:   # non-finite appearance gradients are dropped (FusedAppearanceOptim.cu:39-40)
            g["features_sh"][::13] = np.inf
            g["features_dc"][::29] = np.nan
        dg = {k: U.dev(v.reshape(-1)) for k, v in g.items()}
        gs = 0.25
        oracle.adam_geometry(p, {k: v.copy() for k, v in g.items()}, m1, m2, step, lrs, grad_scale=gs)
        oracle.adam_plain(p["features_dc"], g["features_dc"].copy(), m1["features_dc"], m2["features_dc"], step, lrs["lr_features_dc"],
                          0.0, 0.5 / 0.28209479177387814, gs)
        oracle.adam_plain(p["features_sh"], g["features_sh"].copy(), m1["features_sh"], m2["features_sh"], step, lrs["lr_features_sh"], 0.0, 0.0, gs)
        cfg_a = L.SsbAdamConfig(lrs["lr_means"], lrs["lr_quats"], lrs["lr_scales"], lrs["lr_opacities"], lrs["lr_features_dc"],
                                lrs["lr_features_sh"], 0.0, gs, step, 1)
        structs = [L.splats_struct(d) for d in (dp, dg, dm1, dm2)]
        L.check(lib.ssb_adam_step(*[C.byref(s) for s in structs], 0, cfg.n_splats, C.byref(cfg_a), None))
        torch.cuda.synchronize()
        for k in p:
            assert U.close_frac(dp[k].cpu().numpy(), p[k].reshape(-1), 1e-7, 1e-5) <= 1e-4, (k, step)
            assert U.close_frac(dm1[k].cpu().numpy(), m1[k].reshape(-1), 1e-10, 1e-3) <= 1e-4, (k, step)
            assert float(dg[k].abs().sum()) == 0.0        # zero_grad
    # a sub-range only touches its own splats
    before = dp["means"].clone()
    g0 = {k: torch.ones_like(t) for k, t in dp.items()}
    structs = [L.splats_struct(d) for d in (dp, g0, dm1, dm2)]
    cfg_a = L.SsbAdamConfig(1e-3, 1e-3, 5e-3, 5e-2, 2.5e-3, 2.5e-3, 0.0, 1.0, 4, 0)
    L.check(lib.ssb_adam_step(*[C.byref(s) for s in structs], 100, 50, C.byref(cfg_a), None))
    torch.cuda.synchronize()
    changed = (dp["means"] != before).view(-1, 3).any(dim=1).nonzero().flatten().cpu().numpy()
    assert changed.min() == 100 and changed.max() == 149 and changed.size == 50


@pytest.mark.parametrize("bits", [16, 8])
def test_adam_quantized_sh(lib, U, oracle, bits):
    """Codes may differ by one quantum where log1pf/expm1f round differently
    (the reference's own tolerance, src/backend/tests/optim_parity.cpp:9-13)."""
    rng = np.random.default_rng(bits)
    n_cells = 45 * 1000 + 7
    x0 = rng.normal(0, 0.05, size=n_cells).astype(np.float32)
    vp, vb = oracle.quant_encode(x0, bits)
    nb = (n_cells + 255) // 256
    op, ob = np.zeros(n_cells * 2, np.uint8), np.zeros(nb * 4, np.float32)
    d_vp, d_vb, d_op, d_ob = U.dev(vp), U.dev(vb), U.dev(op), U.dev(ob)
    view = np.uint16 if bits == 16 else np.uint8
    for step in (1, 2, 3):
        g = (rng.normal(size=n_cells) * 1e-3).astype(np.float32)
        d_g = U.dev(g)
        oracle.adam_qq(g.copy(), op, ob, vp, vb, bits, step, 2.5e-3, grad_scale=0.5)
        cfg_a = L.SsbAdamConfig(0, 0, 0, 0, 0, 2.5e-3, 0.0, 0.5, step, 1)
        L.check(lib.ssb_adam_step_sh_quantized(L.ptr(d_g), L.ptr(d_op), L.ptr(d_ob), L.ptr(d_vp), L.ptr(d_vb), bits, 0, n_cells, n_cells,
                                               C.byref(cfg_a), None))
        torch.cuda.synchronize()
        assert float(d_g.abs().sum()) == 0.0
        dv = np.abs(d_vp.cpu().numpy().view(view).astype(np.int64) - vp.view(view).astype(np.int64))
        do = np.abs(d_op.cpu().numpy().astype(np.int64) - op.astype(np.int64))
        assert dv.max() <= 1 and do.max() <= 1
        assert (dv > 0).mean() <= 2e-2 and (do > 0).mean() <= 2e-2
        assert np.allclose(d_vb.cpu().numpy(), vb, rtol=1e-5, atol=1e-8)
        assert np.allclose(d_ob.cpu().numpy(), ob, rtol=1e-4, atol=1e-6)
        # continue both sides from the same state so differences do not compound
        d_vp.copy_(U.dev(vp)); d_vb.copy_(U.dev(vb)); d_op.copy_(U.dev(op)); d_ob.copy_(U.dev(ob))


def test_adam_quantized_state_fp32_values(lib, U, oracle):
    """value_bits = 32: fp32 values, 8-bit optimiser state (the reference's fused_adam_step_quantized)."""
    rng = np.random.default_rng(32)
    n_cells = 45 * 700 + 5
    x = rng.normal(0, 0.05, size=n_cells).astype(np.float32)
    nb = (n_cells + 255) // 256
    op, ob = np.zeros(n_cells * 2, np.uint8), np.zeros(nb * 4, np.float32)
    d_x, d_op, d_ob = U.dev(x), U.dev(op), U.dev(ob)
    for step in (1, 2, 3):
        g = (rng.normal(size=n_cells) * 1e-3).astype(np.float32)
        d_g = U.dev(g)
        oracle.adam_qq(g.copy(), op, ob, x.view(np.uint8), np.zeros(2, np.float32), 32, step, 2.5e-3, grad_scale=0.5)
        cfg_a = L.SsbAdamConfig(0, 0, 0, 0, 0, 2.5e-3, 0.0, 0.5, step, 1)
        L.check(lib.ssb_adam_step_sh_quantized(L.ptr(d_g), L.ptr(d_op), L.ptr(d_ob), L.ptr(d_x), None, 32, 0, n_cells, n_cells, C.byref(cfg_a), None))
        torch.cuda.synchronize()
        assert float(d_g.abs().sum()) == 0.0
        assert np.allclose(d_x.cpu().numpy(), x, rtol=1e-5, atol=1e-7)
        do = np.abs(d_op.cpu().numpy().astype(np.int64) - op.astype(np.int64))
        assert do.max() <= 1 and (do > 0).mean() <= 2e-2
        assert np.allclose(d_ob.cpu().numpy(), ob, rtol=1e-4, atol=1e-6)
        d_x.copy_(U.dev(x)); d_op.copy_(U.dev(op)); d_ob.copy_(U.dev(ob))


def _oracle_iteration(oracle, cfg, sp, vm, K, targets, shq=None, dist=0, rows=None, sh_degree=3):
    """Gradients of one multi-view iteration, one camera per sub-batch, summed (reference split-batch loop)."""
    W, H, n = cfg.width, cfg.height, cfg.n_splats
    tot = None
    losses = np.zeros(3)
    renders = []
    for v in range(vm.shape[0]):
        dr = None if rows is None else rows[v:v + 1]
        ch = oracle.forward_chain(sp, vm[v:v + 1], K[v:v + 1], W, H, shq=shq, dist=dist, dist_coeffs=dr, sh_degree=sh_degree)
        vr, l = oracle.loss_l1_ssim(ch["render"]["rgb"], targets[v].reshape(-1, 3), 1, H, W, 0.8, 0.2)
        losses += l
        gs = oracle.raster_bwd(ch["proj"], ch["offsets"], ch["sorted_vals"], 1, n, W, H, ch["render"], vr)
        g = oracle.project_bwd(sp, vm[v:v + 1], K[v:v + 1], W, H, ch["proj"]["aabb"], gs, shq=shq, dist=dist, dist_coeffs=dr, sh_degree=sh_degree)
        tot = g if tot is None else {k: tot[k] + g[k] for k in g}
        renders.append(ch)
    return tot, losses, renders


@pytest.mark.parametrize("quant", [False, True])
def test_whole_iteration_matches_oracle(lib, U, oracle, quant):
    from spirula_studio_b200.trainer import Trainer
    cfg = scenes.scaled(scenes.CONFIGS["plumbing_50k"], n_splats=12000, width=208, height=144, n_views=3)
    cfg.rig, cfg.rig_radius, cfg.log_scale_mu = "ring", 3.0, -3.0
    if quant:
        cfg.sh_value_bits, cfg.sh_optim_bits = 16, 8
    sp = scenes.make_splats(cfg)
    vm, K = scenes.make_cameras(cfg)
    targets = np.stack([scenes.make_target(cfg, v) for v in range(cfg.n_views)])
    shq = None
    if quant:
        packed, bounds = oracle.quant_encode(sp["features_sh"], 16)
        shq = dict(packed=packed, bounds=bounds, bits=16, bounds_stride=256)
    ref_g, ref_l, renders = _oracle_iteration(oracle, cfg, sp, vm, K, targets, shq)

    tr = Trainer(cfg, sp, device=U.DEV)
    h_vm, h_K, h_gt = (torch.from_numpy(a).pin_memory() for a in (vm, K, targets))
    tr.losses.zero_()
    d_vm, d_K, d_gt = h_vm.to(U.DEV), h_K.to(U.DEV), h_gt.to(U.DEV)
    tr.views_fwd_bwd(d_vm, d_K, d_gt, cfg.n_views)
    torch.cuda.synchronize()
    # last view's image
    rgb_p = C.c_void_p()
    L.check(lib.ssb_step_peek(tr.handle, C.byref(rgb_p), None, None, None, None, None))
    assert tr.last_isects() == renders[-1]["sorted_vals"].size or abs(tr.last_isects() - renders[-1]["sorted_vals"].size) <= 3
    img_t = U.tensor_from_device_ptr(rgb_p.value, (cfg.height * cfg.width, 3))
    d_img = np.abs(img_t.cpu().numpy() - renders[-1]["render"]["rgb"])
    assert d_img.max() <= 5e-3 and (d_img.max(axis=1) > 1e-4).mean() <= 2e-3
    assert np.allclose(tr.losses.cpu().numpy(), ref_l, rtol=1e-3, atol=1e-5)
    for k in ref_g:
        got = tr.grads[k].cpu().numpy().reshape(ref_g[k].shape)
        scale = np.abs(ref_g[k]).max()
        assert U.close_frac(got, ref_g[k], 2e-5 * scale, 1e-3) <= 5e-3, k
    # optimiser pass: post-Adam parameters within 1e-3 relative of the oracle's
    p, m1, m2 = _np_state(sp)
    gs = 1.0 / cfg.n_views
    oracle.adam_geometry(p, {k: v.copy() for k, v in ref_g.items()}, m1, m2, 1, cfg.lrs, grad_scale=gs)
    oracle.adam_plain(p["features_dc"], ref_g["features_dc"].copy(), m1["features_dc"], m2["features_dc"], 1, cfg.lrs["lr_features_dc"], 0.0,
                      0.5 / 0.28209479177387814, gs)
    tr.optimizer_step(cfg.n_views)
    torch.cuda.synchronize()
    for k in ("means", "quats", "scales", "opacities", "features_dc"):
        got = tr.params[k].cpu().numpy().reshape(p[k].shape)
        # a first Adam step moves every coordinate by lr*sign(g): where |g| is at rounding level the sign may differ
        assert U.close_frac(got, p[k], 1e-6, 1e-3) <= 2e-2, k
    if not quant:
        oracle.adam_plain(p["features_sh"], ref_g["features_sh"].copy(), m1["features_sh"], m2["features_sh"], 1, cfg.lrs["lr_features_sh"], 0.0, 0.0, gs)
        got = tr.params["features_sh"].cpu().numpy().reshape(p["features_sh"].shape)
        assert U.close_frac(got, p["features_sh"], 1e-6, 1e-3) <= 2e-2
    # the same iteration through the host-buffer entry point gives the same loss
    tr2 = Trainer(cfg, sp, device=U.DEV)
    l1, ssim, loss = tr2.train_step(h_vm, h_K, h_gt, cfg.n_views)
    assert abs(loss - ref_l[2] / cfg.n_views) <= 1e-3 * abs(ref_l[2] / cfg.n_views) + 1e-5
    tr.close(); tr2.close()


@pytest.mark.parametrize("quant", [False, True])
def test_iteration_with_sh_degree_warmup_matches_oracle(lib, U, oracle, quant):
    """Trainer.set_sh_degree -> ssb_step_set_sh_degree: an iteration at SH degree 1 against the oracle's; the bands above the
    degree take no gradient, and an optimiser step leaves them (and their Adam state) where they were."""
    from spirula_studio_b200.trainer import Trainer
    cfg = scenes.scaled(scenes.CONFIGS["plumbing_50k"], n_splats=9000, width=176, height=128, n_views=2)
    cfg.rig, cfg.rig_radius, cfg.log_scale_mu = "ring", 3.0, -3.0
    if quant:
        cfg.sh_value_bits, cfg.sh_optim_bits = 16, 8
    sp = scenes.make_splats(cfg)
    vm, K = scenes.make_cameras(cfg)
    targets = np.stack([scenes.make_target(cfg, v) for v in range(cfg.n_views)])
    shq = None
    if quant:
        packed, bounds = oracle.quant_encode(sp["features_sh"], 16)
        shq = dict(packed=packed, bounds=bounds, bits=16, bounds_stride=256)
    assert Trainer.sh_degree_for_step(0) == 0 and Trainer.sh_degree_for_step(1999) == 1 and Trainer.sh_degree_for_step(10 ** 6) == 3
    ref_g, ref_l, _ = _oracle_iteration(oracle, cfg, sp, vm, K, targets, shq, sh_degree=1)
    full_g, full_l, _ = _oracle_iteration(oracle, cfg, sp, vm, K, targets, shq)
    assert abs(full_l[2] - ref_l[2]) > 1e-4 * abs(ref_l[2])
    tr = Trainer(cfg, sp, device=U.DEV)
    tr.set_sh_degree(Trainer.sh_degree_for_step(1500))
    d_vm, d_K, d_gt = (torch.from_numpy(a).to(U.DEV) for a in (vm, K, targets))
    tr.losses.zero_()
    tr.views_fwd_bwd(d_vm, d_K, d_gt, cfg.n_views)
    torch.cuda.synchronize()
    assert np.allclose(tr.losses.cpu().numpy(), ref_l, rtol=1e-3, atol=1e-5)
    for k in ref_g:
        got = tr.grads[k].cpu().numpy().reshape(ref_g[k].shape)
        assert U.close_frac(got, ref_g[k], 2e-5 * np.abs(ref_g[k]).max(), 1e-3) <= 5e-3, k
    assert not tr.grads["features_sh"].view(-1, 15, 3)[:, 3:].any()
    if quant:
        before = tr.sh_packed.clone().view(torch.int16).view(-1, 15, 3)[:, 3:].clone()
        state_before = tr.sh_optim_packed.clone()
    else:
        before = tr.params["features_sh"].view(-1, 15, 3)[:, 3:].clone()
    tr.optimizer_step(cfg.n_views)
    torch.cuda.synchronize()
    if quant:
        # the value codes of a block are re-encoded against the block's new bounds, so the unused bands may move by a code;
        # their decoded values stay within one quantum
        dec0 = oracle.quant_decode(packed, bounds, sp["features_sh"].size, 16).reshape(-1, 15, 3)[:, 3:]
        dec1 = oracle.quant_decode(tr.sh_packed.cpu().numpy(), tr.sh_bounds.cpu().numpy(), sp["features_sh"].size, 16).reshape(-1, 15, 3)[:, 3:]
        assert np.abs(dec1 - dec0).max() <= 2.0 * (bounds.reshape(-1, 2)[:, 1] - bounds.reshape(-1, 2)[:, 0]).max() / 65535.0 + 1e-7
    else:
        assert torch.equal(tr.params["features_sh"].view(-1, 15, 3)[:, 3:], before)
        assert not tr.m1["features_sh"].view(-1, 15, 3)[:, 3:].any()
    tr.close()


@pytest.mark.parametrize("quant", [False, True])
def test_iteration_with_the_reference_optimiser_options_matches_oracle(lib, U, oracle, quant):
    """Trainer(optim=OptimOptions()): the stock optimiser flags of the reference -- per-splat regularisers, the scale-agnostic
    mean update fed by the iteration's view radii, per-splat bias-correction counters, the SH regulariser -- against the
    oracle's optimiser on the oracle's gradients, two iterations."""
    from spirula_studio_b200.trainer import OptimOptions, Trainer
    cfg = scenes.scaled(scenes.CONFIGS["plumbing_50k"], n_splats=9000, width=176, height=128, n_views=2)
    cfg.rig, cfg.rig_radius, cfg.log_scale_mu = "ring", 3.0, -3.0
    if quant:
        cfg.sh_value_bits, cfg.sh_optim_bits = 16, 8
    sp = scenes.make_splats(cfg)
    vm, K = scenes.make_cameras(cfg)
    targets = np.stack([scenes.make_target(cfg, v) for v in range(cfg.n_views)])
    opt = OptimOptions(sh_reg=0.05)
    n, W, H = cfg.n_splats, cfg.width, cfg.height
    shq = None
    if quant:
        packed, bounds = oracle.quant_encode(sp["features_sh"], 16)
        shq = dict(packed=packed, bounds=bounds, bits=16, bounds_stride=256)
    ref_g, ref_l, _ = _oracle_iteration(oracle, cfg, sp, vm, K, targets, shq)
    radii = oracle.project_fwd(sp, vm, K, W, H, shq=shq)["radii"]
    tr = Trainer(cfg, sp, device=U.DEV, optim=opt)
    d_vm, d_K, d_gt = (torch.from_numpy(a).to(U.DEV) for a in (vm, K, targets))
    tr.step_device(d_vm, d_K, d_gt, cfg.n_views, cfg.n_views)
    torch.cuda.synchronize()
    assert np.allclose(tr.radii.cpu().numpy(), radii, rtol=1e-3, atol=1e-6) and radii.max() > 0
    assert (tr.steps == 1).all()
    p, m1, m2 = _np_state(sp)
    gs = 1.0 / cfg.n_views
    steps = np.ones(n, np.int32)
    reg = [opt.max_gauss_ratio, opt.scale_regularization_weight, opt.opacity_reg, opt.scale_reg, opt.erank_reg, opt.erank_reg_s3, opt.quat_norm_reg]
    oracle.adam_geometry_ex(p, {k: v.copy() for k, v in ref_g.items()}, m1, m2, 1, cfg.lrs, grad_scale=gs, reg=reg, scale_agnostic=True, radii=radii, steps=steps)
    oracle.adam_plain(p["features_dc"], ref_g["features_dc"].copy(), m1["features_dc"], m2["features_dc"], 1, cfg.lrs["lr_features_dc"], opt.sh_reg,
                      0.5 / 0.28209479177387814, gs, steps=steps, stride=3)
    for k in ("means", "quats", "scales", "opacities", "features_dc"):
        got = tr.params[k].cpu().numpy().reshape(p[k].shape)
        assert U.close_frac(got, p[k], 1e-6, 1e-3) <= 2e-2, k
    plain = Trainer(cfg, sp, device=U.DEV)
    plain.step_device(d_vm, d_K, d_gt, cfg.n_views, cfg.n_views)
    torch.cuda.synchronize()
    assert (plain.params["scales"] - tr.params["scales"]).abs().max().item() > 0        # the options do change the step
    # a second iteration: the counters advance, the radii are those of this iteration only
    tr.step_device(d_vm, d_K, d_gt, cfg.n_views, cfg.n_views)
    torch.cuda.synchronize()
    assert (tr.steps == 2).all() and np.isfinite(tr.params["means"].cpu().numpy()).all()
    tr.close(); plain.close()


def test_forward_only_render_matches_oracle_and_leaves_training_alone(lib, U, oracle):
    """ssb_step_render (the viewer's forward-only path): colour, normalised ray depth and transmittance of an arbitrary camera
    against the oracle's forward chain, at full and at a lower SH degree; rendering between iterations changes nothing in them."""
    from spirula_studio_b200.trainer import Trainer
    cfg = scenes.scaled(scenes.CONFIGS["plumbing_50k"], n_splats=9000, width=176, height=128, n_views=2)
    cfg.rig, cfg.rig_radius, cfg.log_scale_mu = "ring", 3.0, -3.0
    sp = scenes.make_splats(cfg)
    vm, K = scenes.make_cameras(cfg)
    targets = np.stack([scenes.make_target(cfg, v) for v in range(cfg.n_views)])
    W, H, n = cfg.width, cfg.height, cfg.n_splats
    tr = Trainer(cfg, sp, device=U.DEV)
    for deg in (3, 1):
        tr.set_sh_degree(deg)
        ch = oracle.forward_chain(sp, vm[1:2], K[1:2], W, H, sh_degree=deg)
        rgb, T, dep = tr.render(vm[1], K[1], depth=True)
        torch.cuda.synchronize()
        d_img = np.abs(rgb.cpu().numpy().reshape(-1, 3) - ch["render"]["rgb"])
        assert d_img.max() <= 5e-3 and (d_img.max(axis=1) > 1e-4).mean() <= 2e-3, deg
        assert np.abs(T.cpu().numpy().reshape(-1) - ch["render"]["T"].reshape(-1)).max() <= 5e-3
        d_dep = np.abs(dep.cpu().numpy().reshape(-1) - ch["render"]["depth"].reshape(-1))
        assert (d_dep > 5e-3 + 1e-3 * np.abs(ch["render"]["depth"].reshape(-1))).mean() <= 2e-3
    tr.set_sh_degree(3)
    tr2 = Trainer(cfg, sp, device=U.DEV)
    h = tuple(torch.from_numpy(a).pin_memory() for a in (vm, K, targets))
    for it in range(3):
        la = tr.train_step(*h, cfg.n_views)
        tr.render(vm[it % 2], K[it % 2])                 # between iterations, on the training stream
        lb = tr2.train_step(*h, cfg.n_views)
        assert abs(la[2] - lb[2]) <= 1e-4 * abs(lb[2]), it
    tr.close(); tr2.close()


def test_iteration_with_lens_distortion_matches_oracle(lib, U, oracle):
    """The step object with a distortion tier (Trainer.set_distortion -> ssb_step_set_distortion): three pinhole views, each with
    its own thin-prism row, device-resident and host-buffer entry points, against the oracle's iteration."""
    from spirula_studio_b200.trainer import Trainer
    cfg = scenes.scaled(scenes.CONFIGS["plumbing_50k"], n_splats=9000, width=176, height=128, n_views=3)
    cfg.rig, cfg.rig_radius, cfg.log_scale_mu = "ring", 3.0, -3.0
    sp = scenes.make_splats(cfg)
    vm, K = scenes.make_cameras(cfg)
    targets = np.stack([scenes.make_target(cfg, v) for v in range(cfg.n_views)])
    rows = np.array([[0.3, -0.08, 0.01, -0.002, 0.004, -0.003, 0.005, -0.004],
                     [-0.4, 0.05, 0.0, 0.001, -0.002, 0.003, -0.004, 0.002],
                     [0.1, 0.0, 0.0, 0.0, 0.01, 0.01, 0.0, 0.0]], np.float32)
    ref_g, ref_l, renders = _oracle_iteration(oracle, cfg, sp, vm, K, targets, dist=L.DISTORTION_THIN_PRISM, rows=rows)
    plain_g, plain_l, _ = _oracle_iteration(oracle, cfg, sp, vm, K, targets)
    assert abs(plain_l[2] - ref_l[2]) > 1e-3 * abs(ref_l[2])                  # the lens matters in this scene
    tr = Trainer(cfg, sp, device=U.DEV)
    tr.set_distortion(L.DISTORTION_THIN_PRISM, rows)
    h_vm, h_K, h_gt = (torch.from_numpy(a).pin_memory() for a in (vm, K, targets))
    tr.losses.zero_()
    tr.views_fwd_bwd(h_vm.to(U.DEV), h_K.to(U.DEV), h_gt.to(U.DEV), cfg.n_views)
    torch.cuda.synchronize()
    assert np.allclose(tr.losses.cpu().numpy(), ref_l, rtol=1e-3, atol=1e-5)
    for k in ref_g:
        got = tr.grads[k].cpu().numpy().reshape(ref_g[k].shape)
        assert U.close_frac(got, ref_g[k], 2e-5 * np.abs(ref_g[k]).max(), 1e-3) <= 5e-3, k
    tr2 = Trainer(cfg, sp, device=U.DEV)
    tr2.set_distortion(L.DISTORTION_THIN_PRISM, rows)
    l1, ssim, loss = tr2.train_step(h_vm, h_K, h_gt, cfg.n_views)
    assert abs(loss - ref_l[2] / cfg.n_views) <= 1e-3 * abs(ref_l[2] / cfg.n_views) + 1e-5
    # back to no distortion: the plain iteration again
    tr.set_distortion(L.DISTORTION_NONE)          # (tr has not taken an optimiser step)
    tr.losses.zero_()
    tr.views_fwd_bwd(h_vm.to(U.DEV), h_K.to(U.DEV), h_gt.to(U.DEV), cfg.n_views)
    torch.cuda.synchronize()
    assert np.allclose(tr.losses.cpu().numpy(), plain_l, rtol=1e-3, atol=1e-5)
    # a pair the projection does not build is refused when it is set
    assert lib.ssb_step_set_distortion(tr.handle, 7, None) == L.SSB_ERR_UNSUPPORTED
    tr.close(); tr2.close()


@pytest.mark.parametrize("mode", [L.SSB_ACCUM_MAX, L.SSB_ACCUM_AVG])
def test_step_densification_outputs_match_oracle(lib, U, oracle, mode):
    """ssb_step_set_densify: the per-splat weights the step accumulates over three views (two lanes running side by side)
    against the oracle's loss map folded by the oracle's backward walk, and the gradients unchanged by the option."""
    from spirula_studio_b200.trainer import Trainer
    cfg = scenes.scaled(scenes.CONFIGS["plumbing_50k"], n_splats=8000, width=176, height=128, n_views=3)
    cfg.rig, cfg.rig_radius, cfg.log_scale_mu = "ring", 3.0, -3.0
    sp = scenes.make_splats(cfg)
    vm, K = scenes.make_cameras(cfg)
    targets = np.stack([scenes.make_target(cfg, v) for v in range(cfg.n_views)])
    W, H, n = cfg.width, cfg.height, cfg.n_splats
    want, want_den = np.zeros(n, np.float64), np.zeros(n, np.float64)
    for v in range(cfg.n_views):
        ch = oracle.forward_chain(sp, vm[v:v + 1], K[v:v + 1], W, H)
        lm = np.zeros(H * W, np.float32)
        oracle.loss_l1_ssim_map(ch["render"]["rgb"], targets[v].reshape(-1, 3), 1, H, W, 2, 0.5, lm)
        acc, den = oracle.raster_accum_weight(ch["proj"], ch["offsets"], ch["sorted_vals"], 1, n, W, H, ch["render"], lm, mode)
        want = np.maximum(want, acc) if mode == L.SSB_ACCUM_MAX else want + acc
        want_den += den
    tr = Trainer(cfg, sp, device=U.DEV)
    d_vm, d_K, d_gt = (torch.from_numpy(a).to(U.DEV) for a in (vm, K, targets))
    tr.losses.zero_()
    tr.views_fwd_bwd(d_vm, d_K, d_gt, cfg.n_views)
    torch.cuda.synchronize()
    base = {k: t.clone() for k, t in tr.grads.items()}
    acc, den = torch.zeros(n, device=U.DEV), torch.zeros(n, device=U.DEV)
    L.check(lib.ssb_step_set_densify(tr.handle, 2, 0.5, mode, L.ptr(acc), L.ptr(den)))
    tr.views_fwd_bwd(d_vm, d_K, d_gt, cfg.n_views)
    torch.cuda.synchronize()
    assert (want > 0).sum() > n // 20
    assert U.close_frac(acc.cpu().numpy(), want, 1e-5 * want.max(), 2e-3) <= 5e-3
    if mode == L.SSB_ACCUM_AVG:
        assert U.close_frac(den.cpu().numpy(), want_den, 1e-5 * want_den.max(), 2e-3) <= 5e-3
    for k in base:
        scale = float(base[k].abs().max())
        assert float((tr.grads[k] - base[k]).abs().max()) <= 1e-4 * scale, k
    L.check(lib.ssb_step_set_densify(tr.handle, 0, 0.0, L.SSB_ACCUM_NONE, None, None))     # and off again
    acc.zero_()
    tr.views_fwd_bwd(d_vm, d_K, d_gt, cfg.n_views)
    torch.cuda.synchronize()
    assert float(acc.abs().max()) == 0.0
    tr.close()


def test_wide_camera_iteration_matches_oracle(lib, U, oracle):
    """A batch that mixes equidistant-fisheye and equirectangular views of different sizes (the wide
    field-of-view configuration, scaled down): summed gradients and losses against the oracle."""
    from spirula_studio_b200.trainer import Trainer
    cfg = scenes.scaled(scenes.CONFIGS["wide_5m"], n_splats=9000, width=144, n_views=4)
    cfg.log_scale_mu, cfg.mean_extent = -2.4, 4.0
    sp = scenes.make_splats(cfg)
    vm, K = scenes.make_cameras(cfg)
    n = cfg.n_splats
    tot, ref_l = None, np.zeros(3)
    for v in range(cfg.n_views):
        _, model, W, H, _, _ = scenes.view_kind(cfg, v)
        ch = oracle.forward_chain(sp, vm[v:v + 1], K[v:v + 1], W, H, model=model)
        assert ch["sorted_vals"].size > 2000
        vr, l = oracle.loss_l1_ssim(ch["render"]["rgb"], scenes.make_target(cfg, v).reshape(-1, 3), 1, H, W, 0.8, 0.2)
        ref_l += l
        gs = oracle.raster_bwd(ch["proj"], ch["offsets"], ch["sorted_vals"], 1, n, W, H, ch["render"], vr)
        g = oracle.project_bwd(sp, vm[v:v + 1], K[v:v + 1], W, H, ch["proj"]["aabb"], gs, model=model)
        tot = g if tot is None else {k: tot[k] + g[k] for k in g}
    tr = Trainer(cfg, sp, device=U.DEV)
    assert len(tr.handles) == 2
    batches = []
    for kind in range(2):
        views = [v for v in range(cfg.n_views) if scenes.view_kind(cfg, v)[0] == kind]
        gt = np.stack([scenes.make_target(cfg, v) for v in views])
        batches.append((kind, torch.from_numpy(vm[views].copy()).pin_memory(), torch.from_numpy(K[views].copy()).pin_memory(),
                        torch.from_numpy(gt).pin_memory()))
    tr.losses.zero_()
    dev_batches = [(k, a.to(U.DEV), b.to(U.DEV), c.to(U.DEV)) for k, a, b, c in batches]
    for i, (k, d_vm, d_K, d_gt) in enumerate(dev_batches):
        tr.views_fwd_bwd(d_vm, d_K, d_gt, d_vm.shape[0], accumulate=i > 0, kind=k)
    torch.cuda.synchronize()
    assert np.allclose(tr.losses.cpu().numpy(), ref_l, rtol=1e-3, atol=1e-5)
    for k in tot:
        got = tr.grads[k].cpu().numpy().reshape(tot[k].shape)
        scale = np.abs(tot[k]).max()
        assert U.close_frac(got, tot[k], 2e-5 * scale, 1e-3) <= 5e-3, k
    # and through the host-buffer entry point
    tr2 = Trainer(cfg, sp, device=U.DEV)
    l1, ssim, loss = tr2.train_step_kinds(batches, cfg.n_views)
    assert abs(loss - ref_l[2] / cfg.n_views) <= 1e-3 * abs(ref_l[2] / cfg.n_views) + 1e-5
    tr.close(); tr2.close()


def test_peer_reduce_and_broadcast_with_virtual_ranks(lib, U):
    """The peer-memory kernels with three 'ranks' that are three buffers on this one GPU: each rank's
    segments end up holding the sum of all ranks' data (reduce), then every rank's copy of them equals
    the owner's (broadcast).  Segment lengths that are not multiples of 16 bytes exercise the tails."""
    world, n = 3, 40_000
    g = torch.Generator(device=U.DEV); g.manual_seed(7)
    grads = [torch.randn(n, device=U.DEV, generator=g) for _ in range(world)]
    orig = [t.clone() for t in grads]
    other = [torch.randint(0, 255, (9001,), device=U.DEV, generator=g, dtype=torch.uint8) for _ in range(world)]
    orig_other = [t.clone() for t in other]
    total = sum(orig)
    bounds = [0, 13_312, 26_624, n]                     # owner r holds floats [bounds[r], bounds[r+1]) and a second piece
    for r in range(world):
        segs = [(0, bounds[r] * 4, (bounds[r + 1] - bounds[r]) * 4 - (4 if r == 1 else 0)), (0, (n - 64 + 16 * r) * 4, 4 * 3)]
        if r != 2:
            segs = segs[:1]
        t = L.peer_table(world, r, [[x.data_ptr() for x in grads]], segs)
        L.check(lib.ssb_peer_reduce_f32(C.byref(t), None))
    torch.cuda.synchronize()
    for r in range(world):
        lo, hi = bounds[r], bounds[r + 1] - (1 if r == 1 else 0)
        if r == 2:
            hi = n - 64          # the tail of rank 2's range was also covered by its second segment; check the first part
        assert torch.allclose(grads[r][lo:hi], total[lo:hi], rtol=1e-6, atol=1e-6)
    assert torch.equal(grads[1][bounds[2] - 1:bounds[2]], orig[1][bounds[2] - 1:bounds[2]])    # the float left out stays
    assert torch.equal(grads[0][bounds[1]:], orig[0][bounds[1]:])                                # others' ranges untouched
    # broadcast: floats of buffer 0 and an odd byte range of buffer 1
    for r in range(world):
        segs = [(0, bounds[r] * 4, (bounds[r + 1] - bounds[r]) * 4), (1, 16 * (100 * r + 1), 2999)]
        t = L.peer_table(world, r, [[x.data_ptr() for x in grads], [x.data_ptr() for x in other]], segs)
        L.check(lib.ssb_peer_broadcast(C.byref(t), None))
        torch.cuda.synchronize()
        for q in range(world):
            assert torch.equal(grads[q][bounds[r]:bounds[r + 1]], grads[r][bounds[r]:bounds[r + 1]])
            o = 16 * (100 * r + 1)
            assert torch.equal(other[q][o:o + 2999], other[r][o:o + 2999])
    # arguments are checked
    t = L.peer_table(world, 0, [[x.data_ptr() for x in grads]], [(0, 8, 64)])
    assert lib.ssb_peer_reduce_f32(C.byref(t), None) == L.SSB_ERR_INVALID_ARGUMENT


@pytest.mark.parametrize("quant", [False, True])
def test_fused_exchange_with_virtual_ranks(lib, U, quant):
    """ssb_reduce_adam_broadcast with three 'ranks' that are three sets of buffers on this one GPU (no kernel waits on
    another, so the ranks' calls simply run one after the other): every replica must end up with the parameters a
    single optimiser pass over the summed gradients gives, bit for bit in the fp32 arrays, and ranges a rank does not
    own must not be touched by it."""
    world, n = 3, 1536 + 512 + 200            # ranges in multiples of 512 splats; the last one is short
    attrs = (("means", 3), ("quats", 4), ("scales", 3), ("opacities", 1), ("features_dc", 3), ("features_sh", 45))
    rng = np.random.default_rng(77)
    cfg_s = scenes.scaled(scenes.CONFIGS["plumbing_50k"], n_splats=n)
    sp = scenes.make_splats(cfg_s, seed=5)

    def flat(arrays):          # one allocation holding the six arrays, each on a 256-byte boundary (the Trainer's layout)
        offs, tot = {}, 0
        for k, w in attrs:
            offs[k] = tot
            tot += (n * w + 63) // 64 * 64
        buf = torch.zeros(tot, device=U.DEV)
        views = {k: buf[offs[k]: offs[k] + n * w] for k, w in attrs}
        for k, _ in attrs:
            if arrays is not None:
                views[k].copy_(U.dev(np.ascontiguousarray(arrays[k]).reshape(-1)))
        return buf, views

    part = [{k: (rng.normal(size=(n * w)) * 1e-3).astype(np.float32) for k, w in attrs} for _ in range(world)]
    total = {k: sum(torch.from_numpy(part[r][k]) for r in range(world)) for k, _ in attrs}      # fp32 sum in rank order
    params, grads, m1, m2 = [], [], [], []
    for r in range(world):
        params.append(flat(sp)); grads.append(flat(part[r])); m1.append(flat(None)); m2.append(flat(None))
    cells = n * 45
    nb = (cells + 255) // 256
    shq = None
    if quant:
        enc = torch.zeros(cells * 2, dtype=torch.uint8, device=U.DEV); bnd = torch.zeros(nb * 2, device=U.DEV)
        L.check(lib.ssb_quant_encode(L.ptr(params[0][1]["features_sh"]), cells, 16, L.ptr(enc), L.ptr(bnd), None))
        shq = [dict(packed=enc.clone(), bounds=bnd.clone(), opt=torch.zeros(cells * 2, dtype=torch.uint8, device=U.DEV),
                    optb=torch.zeros(nb * 4, device=U.DEV)) for _ in range(world)]
    cfg = L.SsbAdamConfig(1e-3, 1e-3, 5e-3, 5e-2, 2.5e-3, 2.5e-3, 0.0, 0.25, 1, 0)

    def structs(r, with_sh):
        def st(v):
            return L.splats_struct(v if with_sh else {**v, "features_sh": None})
        return st(params[r][1]), L.splats_struct(grads[r][1]), st(m1[r][1]), st(m2[r][1])

    # reference: one rank holding the summed gradients, plain optimiser pass over everything
    ref_p, ref_g, ref_m1, ref_m2 = flat(sp), flat({k: total[k].numpy() for k, _ in attrs}), flat(None), flat(None)
    rp = L.splats_struct(ref_p[1] if not quant else {**ref_p[1], "features_sh": None})
    rg = L.splats_struct(ref_g[1])
    rm1 = L.splats_struct(ref_m1[1] if not quant else {**ref_m1[1], "features_sh": None})
    rm2 = L.splats_struct(ref_m2[1] if not quant else {**ref_m2[1], "features_sh": None})
    L.check(lib.ssb_adam_step(C.byref(rp), C.byref(rg), C.byref(rm1), C.byref(rm2), 0, n, C.byref(cfg), None))
    if quant:
        r_enc, r_bnd = enc.clone(), bnd.clone()
        r_opt, r_optb = torch.zeros(cells * 2, dtype=torch.uint8, device=U.DEV), torch.zeros(nb * 4, device=U.DEV)
        L.check(lib.ssb_adam_step_sh_quantized(L.ptr(ref_g[1]["features_sh"]), L.ptr(r_opt), L.ptr(r_optb), L.ptr(r_enc), L.ptr(r_bnd), 16, 0, cells,
                                               cells, C.byref(cfg), None))
    torch.cuda.synchronize()
    before = params[2][0].clone()
    ranges = [(0, 1024), (1024, 1024), (2048, n - 2048)]
    for r, (f, c) in enumerate(ranges):
        rep = L.peer_replicas(world, r, [g_[0].data_ptr() for g_ in grads], [p_[0].data_ptr() for p_ in params],
                              [s_["packed"].data_ptr() for s_ in shq] if quant else None, [s_["bounds"].data_ptr() for s_ in shq] if quant else None)
        ps, gs, a, b = structs(r, not quant)
        sh = L.SsbShAdamState(shq[r]["opt"].data_ptr(), shq[r]["optb"].data_ptr(), shq[r]["packed"].data_ptr(), shq[r]["bounds"].data_ptr(), 16, 8) if quant else None
        L.check(lib.ssb_reduce_adam_broadcast(C.byref(rep), C.byref(ps), C.byref(gs), C.byref(a), C.byref(b), C.byref(sh) if quant else None,
                                              f, c, n, C.byref(cfg), None, None))
        torch.cuda.synchronize()
        if r == 0:        # rank 0 has written its range into every replica and nothing else
            for k, w in attrs[:5]:
                assert torch.equal(params[2][1][k][1024 * w:], flat_view(before, attrs, n, k)[1024 * w:]), k
    for r in range(world):
        for k, w in attrs:
            if quant and k == "features_sh":
                continue
            # peers are summed in rank order after the rank's own part: compare with the tolerance of a reordered fp32 sum
            assert torch.allclose(params[r][1][k], ref_p[1][k], rtol=2e-5, atol=1e-7), (r, k)
            assert torch.equal(params[r][1][k], params[0][1][k]), (r, k)                # replicas identical
        if quant:
            d = (shq[r]["packed"].view(torch.int16).int() - r_enc.view(torch.int16).int()).abs()
            assert int(d.max()) <= 2 and float((d > 0).float().mean()) < 2e-2
            assert torch.equal(shq[r]["packed"], shq[0]["packed"]) and torch.equal(shq[r]["bounds"], shq[0]["bounds"])
    # arguments are checked: a range that cuts a quantisation block, a gradient array outside the exchanged buffer
    rep = L.peer_replicas(world, 0, [g_[0].data_ptr() for g_ in grads], [p_[0].data_ptr() for p_ in params],
                          [s_["packed"].data_ptr() for s_ in shq] if quant else None, [s_["bounds"].data_ptr() for s_ in shq] if quant else None)
    ps, gs, a, b = structs(0, not quant)
    if quant:
        sh = L.SsbShAdamState(shq[0]["opt"].data_ptr(), shq[0]["optb"].data_ptr(), shq[0]["packed"].data_ptr(), shq[0]["bounds"].data_ptr(), 16, 8)
        assert lib.ssb_reduce_adam_broadcast(C.byref(rep), C.byref(ps), C.byref(gs), C.byref(a), C.byref(b), C.byref(sh), 0, 1000, n, C.byref(cfg),
                                             None, None) == L.SSB_ERR_INVALID_ARGUMENT
    stray = torch.zeros(n * 3, device=U.DEV)
    bad = L.splats_struct({**grads[0][1], "means": stray}) if stray.data_ptr() < grads[0][0].data_ptr() else None
    if bad is not None:
        assert lib.ssb_reduce_adam_broadcast(C.byref(rep), C.byref(ps), C.byref(bad), C.byref(a), C.byref(b), C.byref(sh) if quant else None,
                                             0, 1024, n, C.byref(cfg), None, None) == L.SSB_ERR_INVALID_ARGUMENT


def test_fused_exchange_with_16bit_moments_and_optimiser_options(lib, U):
    """ssb_reduce_adam_broadcast_q16 on three virtual ranks with the reference's stock optimiser state: 16-bit codes for the
    moments of the five non-SH arrays, quantised SH values and state, per-splat counters, regularisers and the scale-agnostic
    mean.  Every replica ends with the parameters of one ssb_adam_step_q16 + ssb_adam_step_sh_quantized_ex pass over the summed
    gradients, and each rank's codes in its own range are the reference pass's."""
    world, n = 3, 1536 + 512 + 200
    attrs = (("means", 3), ("quats", 4), ("scales", 3), ("opacities", 1), ("features_dc", 3), ("features_sh", 45))
    rng = np.random.default_rng(78)
    sp = scenes.make_splats(scenes.scaled(scenes.CONFIGS["plumbing_50k"], n_splats=n), seed=6)

    def flat(arrays):
        offs, tot = {}, 0
        for k, w in attrs:
            offs[k] = tot
            tot += (n * w + 63) // 64 * 64
        buf = torch.zeros(tot, device=U.DEV)
        views = {k: buf[offs[k]: offs[k] + n * w] for k, w in attrs}
        if arrays is not None:
            for k, _ in attrs:
                views[k].copy_(U.dev(np.ascontiguousarray(arrays[k]).reshape(-1)))
        return buf, views

    def moments():
        m = L.SsbMomentsQ16()
        keep = []
        for t, (k, w) in enumerate(attrs[:5]):
            pk, bd = torch.zeros(n * w * 4, dtype=torch.uint8, device=U.DEV), torch.zeros(((n + 255) // 256) * 4, device=U.DEV)
            m.d_packed[t], m.d_bounds[t] = pk.data_ptr(), bd.data_ptr()
            keep.append((pk, bd))
        return m, keep

    part = [{k: (rng.normal(size=(n * w)) * 1e-3).astype(np.float32) for k, w in attrs} for _ in range(world)]
    total = {k: sum(torch.from_numpy(part[r][k]) for r in range(world)) for k, _ in attrs}
    cells, nb = n * 45, (n * 45 + 255) // 256
    radii = U.dev(rng.uniform(0.5, 30.0, n).astype(np.float32))
    steps = U.dev(rng.integers(1, 40, n).astype(np.int32))
    extras = L.SsbAdamExtras(10.0, 0.0, 0.01, 0.01, 0.0, 0.0, 0.01, 1, radii.data_ptr(), steps.data_ptr(), n, None)
    cfg = L.SsbAdamConfig(1e-3, 1e-3, 5e-3, 5e-2, 2.5e-3, 2.5e-3, 0.05, 0.25, 1, 0)

    def sh_state():
        enc = torch.zeros(cells * 2, dtype=torch.uint8, device=U.DEV); bnd = torch.zeros(nb * 2, device=U.DEV)
        L.check(lib.ssb_quant_encode(L.ptr(U.dev(sp["features_sh"].reshape(-1))), cells, 16, L.ptr(enc), L.ptr(bnd), None))
        return dict(packed=enc, bounds=bnd, opt=torch.zeros(cells * 2, dtype=torch.uint8, device=U.DEV), optb=torch.zeros(nb * 4, device=U.DEV))

    # reference: one rank, the summed gradients
    ref_p, ref_g = flat(sp), flat({k: total[k].numpy() for k, _ in attrs})
    ref_m, ref_keep = moments()
    ref_sh = sh_state()
    rp, rg = L.splats_struct({**ref_p[1], "features_sh": None}), L.splats_struct(ref_g[1])
    L.check(lib.ssb_adam_step_q16(C.byref(rp), C.byref(rg), C.byref(ref_m), 0, n, C.byref(cfg), C.byref(extras), None))
    L.check(lib.ssb_adam_step_sh_quantized_ex(L.ptr(ref_g[1]["features_sh"]), L.ptr(ref_sh["opt"]), L.ptr(ref_sh["optb"]), L.ptr(ref_sh["packed"]),
                                              L.ptr(ref_sh["bounds"]), 16, 8, 0, cells, cells, C.byref(cfg), L.ptr(steps), 45, None))
    params = [flat(sp) for _ in range(world)]
    grads = [flat(part[r]) for r in range(world)]
    moms = [moments() for _ in range(world)]
    shq = [sh_state() for _ in range(world)]
    torch.cuda.synchronize()
    ranges = [(0, 1024), (1024, 1024), (2048, n - 2048)]
    for r, (f, c) in enumerate(ranges):
        rep = L.peer_replicas(world, r, [g_[0].data_ptr() for g_ in grads], [p_[0].data_ptr() for p_ in params],
                              [s_["packed"].data_ptr() for s_ in shq], [s_["bounds"].data_ptr() for s_ in shq])
        ps, gs = L.splats_struct({**params[r][1], "features_sh": None}), L.splats_struct(grads[r][1])
        sh = L.SsbShAdamState(shq[r]["opt"].data_ptr(), shq[r]["optb"].data_ptr(), shq[r]["packed"].data_ptr(), shq[r]["bounds"].data_ptr(), 16, 8)
        L.check(lib.ssb_reduce_adam_broadcast_q16(C.byref(rep), C.byref(ps), C.byref(gs), C.byref(moms[r][0]), None, None, C.byref(sh),
                                                  f, c, n, C.byref(cfg), C.byref(extras), None))
        torch.cuda.synchronize()
    for r in range(world):
        for k, w in attrs[:5]:
            assert torch.allclose(params[r][1][k], ref_p[1][k], rtol=2e-5, atol=2e-7), (r, k)
            assert torch.equal(params[r][1][k], params[0][1][k]), (r, k)
        assert torch.equal(shq[r]["packed"], shq[0]["packed"]) and torch.equal(shq[r]["bounds"], shq[0]["bounds"])
        d = (shq[r]["packed"].view(torch.int16).int() - ref_sh["packed"].view(torch.int16).int()).abs()
        assert int(d.max()) <= 2 and float((d > 0).float().mean()) < 2e-2
        # the rank's own range of moment codes: the reference pass's, up to the rounding of a reordered gradient sum
        f, c = ranges[r]
        for t, (k, w) in enumerate(attrs[:5]):
            mine = moms[r][1][t][0].view(torch.int16).int().view(-1, 2)[f * w:(f + c) * w]
            want = ref_keep[t][0].view(torch.int16).int().view(-1, 2)[f * w:(f + c) * w]
            dd = ((mine & 0xffff) - (want & 0xffff)).abs()
            assert int(dd.max()) <= 64 and float((dd > 2).float().mean()) < 0.02, (r, k, int(dd.max()))
            assert mine.any() and not moms[r][1][t][0].view(torch.int16).view(-1, 2)[:f * w].any()      # nothing outside the range
    # a range that does not start on a block of 256 splats is refused
    rep = L.peer_replicas(world, 0, [g_[0].data_ptr() for g_ in grads], [p_[0].data_ptr() for p_ in params],
                          [s_["packed"].data_ptr() for s_ in shq], [s_["bounds"].data_ptr() for s_ in shq])
    ps, gs = L.splats_struct({**params[0][1], "features_sh": None}), L.splats_struct(grads[0][1])
    sh = L.SsbShAdamState(shq[0]["opt"].data_ptr(), shq[0]["optb"].data_ptr(), shq[0]["packed"].data_ptr(), shq[0]["bounds"].data_ptr(), 16, 8)
    assert lib.ssb_reduce_adam_broadcast_q16(C.byref(rep), C.byref(ps), C.byref(gs), C.byref(moms[0][0]), None, None, C.byref(sh), 128, 128, n,
                                             C.byref(cfg), C.byref(extras), None) == L.SSB_ERR_INVALID_ARGUMENT


def flat_view(buf, attrs, n, name):
    off = 0
    for k, w in attrs:
        if k == name:
            return buf[off: off + n * w]
        off += (n * w + 63) // 64 * 64
    raise KeyError(name)


@pytest.mark.parametrize("bits", [16, 8])
def test_full_size_quant_roundtrip(lib, U, bits):
    """The SH codec at the benchmark's size (45M cells): decode(encode(x)) is within half a quantum of x in every
    256-cell block, the bounds are the block's min and max, and encoding the decoded values again is idempotent."""
    n_cells = 1_000_000 * 45
    g = torch.Generator(device=U.DEV); g.manual_seed(bits)
    x = torch.randn(n_cells, device=U.DEV, generator=g) * 0.05
    nb = (n_cells + 255) // 256
    packed = torch.zeros(n_cells * (bits // 8), dtype=torch.uint8, device=U.DEV)
    bounds = torch.zeros(nb * 2, device=U.DEV)
    y = torch.zeros_like(x)
    L.check(lib.ssb_quant_encode(L.ptr(x), n_cells, bits, L.ptr(packed), L.ptr(bounds), None))
    L.check(lib.ssb_quant_decode(L.ptr(packed), L.ptr(bounds), n_cells, bits, L.ptr(y), None))
    torch.cuda.synchronize()
    pad = nb * 256 - n_cells
    xb = torch.cat([x, x[-1:].expand(pad)]).view(nb, 256)
    lo, hi = bounds.view(nb, 2)[:, 0], bounds.view(nb, 2)[:, 1]
    assert torch.equal(lo, xb.min(dim=1).values) and torch.equal(hi, xb.max(dim=1).values)
    quantum = ((hi - lo) / float((1 << bits) - 1)).repeat_interleave(256)[:n_cells]
    # half a quantum plus the fp32 rounding of the code and of the decode (a few thousandths of a 16-bit quantum)
    assert bool(((y - x).abs() <= 0.5 * quantum * 1.02 + 2e-8).all())
    packed2 = torch.zeros_like(packed); bounds2 = torch.zeros_like(bounds)
    L.check(lib.ssb_quant_encode(L.ptr(y), n_cells, bits, L.ptr(packed2), L.ptr(bounds2), None))
    torch.cuda.synchronize()
    assert torch.equal(packed2, packed)


def test_full_size_raster_properties(lib, U):
    """The rasterisers at the benchmark's size (one 1080p view of 1M splats): transmittance within [0, 1], colour
    non-negative and bounded by the opacity-weighted sum, last indices inside their tile's range, the depth-free
    variant equal to the full one, and the backward pass linear in its cotangent (twice the colour cotangent
    gives twice every gradient, up to the order of the floating-point reductions)."""
    cfg = scenes.CONFIGS["mid_1m"]
    sp = scenes.make_splats(cfg)
    vm, K = scenes.make_cameras(cfg)
    n, W, H = cfg.n_splats, cfg.width, cfg.height
    pr = U.project_fwd(lib, U.splats_dev(sp), vm[3:4], K[3:4], W, H)
    tw, th = (W + 15) // 16, (H + 15) // 16
    cap = 8 * n
    _, flat, offs, M = U.intersect_tiles(lib, pr["aabb"], pr["depths"], pr["rec"], n, n, W, H, cap, tw * th, want_keys=False)
    n_dev = torch.tensor([M], dtype=torch.int64, device=U.DEV)
    out = U.raster_fwd(lib, pr["rec"], offs, flat, n_dev, 1, W, H)
    T, rgb, last = out["T"], out["rgb"], out["last_ids"].long()
    assert bool(((T >= 0) & (T <= 1)).all()) and bool((rgb >= 0).all()) and bool(torch.isfinite(rgb).all())
    ys, xs = torch.meshgrid(torch.arange(H, device=U.DEV), torch.arange(W, device=U.DEV), indexing="ij")
    tile = ((ys // 16) * tw + xs // 16).reshape(-1)
    ends = torch.cat([offs[1:].long(), torch.tensor([M], device=U.DEV)])
    blended = T < 1.0
    assert bool(((last >= offs.long()[tile]) & (last < ends[tile]))[blended].all())
    # depth-free variant
    rgb2 = torch.zeros_like(rgb); T2 = torch.zeros_like(T); last2 = torch.zeros_like(out["last_ids"])
    L.check(lib.ssb_raster_fwd(L.ptr(pr["rec"]), n, L.ptr(offs), L.ptr(flat), flat.numel(), L.ptr(n_dev), 1, W, H, L.ptr(rgb2), None, L.ptr(T2), L.ptr(last2), None))
    torch.cuda.synchronize()
    assert torch.equal(rgb2, rgb) and torch.equal(T2, T) and torch.equal(last2, out["last_ids"])
    # linearity of the backward pass
    g = torch.Generator(device=U.DEV); g.manual_seed(5)
    v = torch.randn(H * W, 3, device=U.DEV, generator=g)
    g1 = U.raster_bwd(lib, pr["rec"], offs, flat, n_dev, 1, W, H, out, v, pairs=n).view(n, 12)
    g2 = U.raster_bwd(lib, pr["rec"], offs, flat, n_dev, 1, W, H, out, 2.0 * v, pairs=n).view(n, 12)
    scale = g1.abs().max(dim=0).values.clamp_min(1e-20)
    assert float(((g2 - 2.0 * g1).abs() / scale).max()) < 1e-3
    assert float(g1.abs().sum()) > 0 and bool(torch.isfinite(g1).all())
    # densification weights: with a weight map of ones the per-splat sums of alpha * T add up to the opacity
    # 1 - T of all pixels (every fragment the forward pass blended is visited exactly once), the sum equals its
    # own denominator, the maximum is a fragment weight (<= 1) and never exceeds the sum
    ones = torch.ones(H * W, device=U.DEV)
    res = {}
    for mode in (L.SSB_ACCUM_MAX, L.SSB_ACCUM_AVG):
        v_rec = torch.zeros(n * L.SCREEN_REC_FLOATS, device=U.DEV)
        acc, den = torch.zeros(n, device=U.DEV), torch.zeros(n, device=U.DEV)
        L.check(lib.ssb_raster_bwd_accum(L.ptr(pr["rec"]), n, L.ptr(offs), L.ptr(flat), flat.numel(), L.ptr(n_dev), 1, W, H, None, L.ptr(out["T"]), L.ptr(out["last_ids"]),
                                         L.ptr(v), None, None, L.ptr(v_rec), mode, L.ptr(ones), n, None, L.ptr(acc), L.ptr(den), None))
        torch.cuda.synchronize()
        res[mode] = (acc, den)
        assert float((v_rec.view(n, 12) - g1).abs().max()) <= 1e-3 * float(g1.abs().max())     # gradients unchanged by the mode
    mx, (sm, den) = res[L.SSB_ACCUM_MAX][0], res[L.SSB_ACCUM_AVG]
    total, want = float(den.double().sum()), float((1.0 - T.double()).sum())
    assert abs(total - want) <= 1e-3 * want, (total, want)
    assert float((sm - den).abs().max()) <= 1e-4 * float(den.max())
    assert float(mx.max()) <= 1.0 and bool((mx <= sm * (1 + 1e-5) + 1e-7).all()) and bool(((mx > 0) == (sm > 0)).all())


def test_full_size_intersection_paths_agree(lib, U):
    """At the benchmark's size (1M splats, 1080p, about 4.4M pairs) the two independent device paths are held
    against each other: keys -> radix sort -> ranges, and the fused bin-by-tile intersection (the oracle
    comparison at this size is in test_gpu_fullsize.py).  Their sorted keys, sorted pair indices, ranges and counts must be identical, the
    keys ascending, and equal keys in ascending pair order."""
    cfg = scenes.CONFIGS["mid_1m"]
    sp = scenes.make_splats(cfg)
    vm, K = scenes.make_cameras(cfg)
    n, W, H = cfg.n_splats, cfg.width, cfg.height
    pr = U.project_fwd(lib, U.splats_dev(sp), vm[:1], K[:1], W, H)
    cap = 8 * n
    st, M, counts, cum, keys, vals, n_dev = U.tile_keys(lib, pr["aabb"], pr["depths"], pr["rec"], n, n, W, H, cap)
    assert st == 0 and 3_000_000 < M < cap
    tw, th = (W + 15) // 16, (H + 15) // 16
    sk, sv = U.sort_pairs(lib, keys, vals, n_dev, cap, 0, 32 + lib.ssb_tile_n_bits(tw * th))
    offs = U.tile_ranges(lib, sk, n_dev, cap, tw * th)
    f_keys, f_vals, f_offs, f_M = U.intersect_tiles(lib, pr["aabb"], pr["depths"], pr["rec"], n, n, W, H, cap, tw * th)
    assert f_M == M
    assert torch.equal(f_offs, offs) and torch.equal(f_keys[:M], sk[:M]) and torch.equal(f_vals[:M], sv[:M])
    k = f_keys[:M]
    assert bool((k[1:] >= k[:-1]).all())
    same = k[1:] == k[:-1]
    assert bool((f_vals[:M][1:][same] > f_vals[:M][:-1][same]).all())
    assert int(counts.sum()) == M


def test_full_size_sort_and_range_properties(lib, U):
    """At the benchmark's pair count (several million), what must hold at any size: the output is
    sorted on the bit range, is a permutation of the input (checksums of keys,
    values and key*value), equal keys keep their input order, and the ranges
    are monotone and bracket exactly the keys of each tile."""
    g = torch.Generator(device=U.DEV); g.manual_seed(1)
    n, n_tiles = 5_000_000, 8160
    tiles = torch.randint(0, n_tiles, (n,), device=U.DEV, generator=g, dtype=torch.int64)
    depth = torch.randint(0, 1 << 20, (n,), device=U.DEV, generator=g, dtype=torch.int64) | (1 << 31)
    keys = (tiles << 32) | depth
    vals = torch.arange(n, device=U.DEV, dtype=torch.int32)
    cap = n + 1000
    dk = torch.zeros(cap, dtype=torch.int64, device=U.DEV); dk[:n] = keys
    dv = torch.zeros(cap, dtype=torch.int32, device=U.DEV); dv[:n] = vals
    n_dev = torch.tensor([n], dtype=torch.int64, device=U.DEV)
    end_bit = 32 + lib.ssb_tile_n_bits(n_tiles)
    sk, sv = U.sort_pairs(lib, dk, dv, n_dev, cap, 0, end_bit)
    sk, sv = sk[:n], sv[:n]
    assert bool((sk[1:] >= sk[:-1]).all())
    assert int(sk.sum()) == int(keys.sum()) and int(sv.long().sum()) == int(vals.long().sum())
    assert bool((keys[sv.long()] == sk).all())                       # values still belong to their keys
    same = sk[1:] == sk[:-1]
    assert bool((sv[1:][same] > sv[:-1][same]).all())                # stability: ties keep input order
    offs = U.tile_ranges(lib, sk, n_dev, cap, n_tiles).long()
    assert bool((offs[1:] >= offs[:-1]).all()) and int(offs[0]) == 0
    counts = torch.bincount(tiles, minlength=n_tiles)
    ends = torch.cat([offs[1:], torch.tensor([n], device=U.DEV)])
    assert bool(((ends - offs) == counts).all())


@pytest.mark.parametrize("quant", [False, True])
def test_fused_backward_equals_per_view_backward(lib, U, quant):
    """ssb_step_set_fused_backward + ssb_step_backward_optimize (projection backward of all views together with the
    optimiser, a range of splats at a time, no world-gradient arrays) against the per-view backward followed by
    ssb_adam_step_*: same parameters and optimiser state after three iterations, up to the order of the sums over views."""
    from spirula_studio_b200.trainer import Trainer
    cfg = scenes.scaled(scenes.CONFIGS["plumbing_50k"], n_splats=140001, width=176, height=128, n_views=5)     # two ranges, the second ragged
    cfg.rig, cfg.rig_radius, cfg.log_scale_mu = "ring", 3.0, -3.0
    if quant:
        cfg.sh_value_bits, cfg.sh_optim_bits = 16, 8
    sp = scenes.make_splats(cfg)
    vm, K = scenes.make_cameras(cfg)
    gt = np.stack([scenes.make_target(cfg, v) for v in range(cfg.n_views)])
    host = tuple(torch.from_numpy(a).pin_memory() for a in (vm, K, gt))
    dev3 = tuple(t.to(U.DEV) for t in host)
    a, b = Trainer(cfg, sp, device=U.DEV), Trainer(cfg, sp, device=U.DEV, fused_backward=True)
    assert b.fused_backward and not a.fused_backward
    for it in range(3):
        if it == 1:
            # views handed over in two calls (3 + 2): the second call's views are appended to the kept ones
            for tr in (a, b):
                tr.losses.zero_()
                tr.views_fwd_bwd(dev3[0][:3], dev3[1][:3], dev3[2][:3], 3)
                tr.views_fwd_bwd(dev3[0][3:], dev3[1][3:], dev3[2][3:], 2, accumulate=True)
                tr.optimizer_step(cfg.n_views)
            la, lb = a.losses.cpu().numpy(), b.losses.cpu().numpy()
        else:
            la, lb = np.array(a.train_step(*host, cfg.n_views)), np.array(b.train_step(*host, cfg.n_views))
        assert np.allclose(la, lb, rtol=1e-4, atol=1e-6), (it, la, lb)
    torch.cuda.synchronize()
    for k in ("means", "quats", "scales", "opacities", "features_dc") + (() if quant else ("features_sh",)):
        x, y = a.params[k].cpu().numpy(), b.params[k].cpu().numpy()
        assert np.abs(x - np.asarray(sp[k]).reshape(-1)).max() > 0
        # Adam's first steps move a coordinate by about lr whatever the gradient's size, so a gradient at rounding level
        # can flip a step's sign; such coordinates are rare
        assert U.close_frac(y, x, 1e-6, 1e-3) <= 5e-3, k
        assert U.close_frac(b.m1[k].cpu().numpy(), a.m1[k].cpu().numpy(), 1e-9, 1e-3) <= 5e-3, k
    if quant:
        # compare the SH VALUES the codes stand for: a flipped first step moves a value by 2 lr, and a block's bounds with it
        def values(tr):
            out = torch.empty(cfg.n_splats * 45, device=U.DEV)
            L.check(lib.ssb_quant_decode(L.ptr(tr.sh_packed), L.ptr(tr.sh_bounds), cfg.n_splats * 45, 16, L.ptr(out), None))
            return out
        va, vb = values(a), values(b)
        lr = cfg.lrs["lr_features_sh"]
        assert (va - vb).abs().max().item() <= 3 * 3 * lr
        assert ((va - vb).abs() > 0.1 * lr).float().mean().item() <= 3e-2
    assert a.check_capacity() == b.check_capacity()
    a.close(); b.close()


def test_stock_configuration_on_the_fused_path_with_the_reference_layouts(lib, U, tmp_path):
    """The reference's stock trainer flags end to end on the fused backward + optimiser: 16-bit SH values and 8-bit SH optimiser
    state with one bound per 256 splats (fused_state_layout="reference"), 16-bit moments for the other arrays, regularisers,
    scale-agnostic mean, per-splat step counters.  Against the per-view path with the shared layouts: same losses, parameters
    that move together; the SH degree warm-up keeps the idle bands at zero; a checkpoint carries the reference's slot names
    for this layout and resumes."""
    import tarfile
    from spirula_studio_b200.trainer import OptimOptions, Trainer
    from spirula_studio_b200 import checkpoint as ckpt
    cfg = scenes.scaled(scenes.CONFIGS["plumbing_50k"], n_splats=140001, width=176, height=128, n_views=4)      # two ranges, ragged last block
    cfg.rig, cfg.rig_radius, cfg.log_scale_mu = "ring", 3.0, -3.0
    cfg.sh_value_bits, cfg.sh_optim_bits = 16, 8
    sp = scenes.make_splats(cfg)
    vm, K = scenes.make_cameras(cfg)
    gt = np.stack([scenes.make_target(cfg, v) for v in range(cfg.n_views)])
    host = tuple(torch.from_numpy(a).pin_memory() for a in (vm, K, gt))
    stock = dict(non_sh_optim_bits=16, optim=OptimOptions())
    a = Trainer(cfg, sp, device=U.DEV, **stock)
    b = Trainer(cfg, sp, device=U.DEV, fused_backward=True, fused_state_layout="reference", **stock)
    assert b.fused_backward and b.sh_bounds.numel() == 2 * ((cfg.n_splats + 255) // 256) and a.sh_bounds.numel() == 2 * ((cfg.n_splats * 45 + 255) // 256)
    with pytest.raises(ValueError):
        Trainer(cfg, sp, device=U.DEV, fused_state_layout="reference", **stock)        # the layout belongs to the fused path
    first = None
    for it in range(3):
        la, lb = np.array(a.train_step(*host, cfg.n_views)), np.array(b.train_step(*host, cfg.n_views))
        # the first iteration sees the same parameters (two quantisation grids of the same SH values); afterwards the paths differ
        # by the coordinates whose near-zero first steps took opposite signs
        assert np.allclose(la, lb, rtol=2e-3 if it == 0 else 2e-2, atol=1e-5), (it, la, lb)
        first = la if first is None else first
    assert lb[0] < first[0]
    torch.cuda.synchronize()
    lrs = dict(means=cfg.lrs["lr_means"], quats=cfg.lrs["lr_quats"], scales=cfg.lrs["lr_scales"], opacities=cfg.lrs["lr_opacities"],
               features_dc=cfg.lrs["lr_features_dc"])
    for k, lr in lrs.items():
        x, y, x0 = a.params[k].cpu().numpy(), b.params[k].cpu().numpy(), np.asarray(sp[k], np.float32).reshape(-1)
        assert np.isfinite(y).all() and np.abs(y - x0).max() > 0
        # early Adam steps are worth about lr each whatever the gradient's size: the two paths (different summation order, different
        # SH quantisation grids) may disagree on the sign of a near-zero step, rarely
        assert (np.abs(x - y) > 0.5 * lr).mean() <= 6e-2, k
    def sh_values(tr):
        n = cfg.n_splats
        codes = tr.sh_packed.cpu().numpy().view(np.uint16).reshape(n, 45).astype(np.float32) / 65535.0
        per = 256 if tr.fused_state_layout == "reference" else None
        bounds = tr.sh_bounds.cpu().numpy().reshape(-1, 2)
        if per:
            mm = np.repeat(bounds, 256, axis=0)[:n]
            return mm[:, :1] + (mm[:, 1:] - mm[:, :1]) * codes
        mm = np.repeat(bounds, 256, axis=0)[: n * 45]
        return (mm[:, 0] + (mm[:, 1] - mm[:, 0]) * codes.reshape(-1)).reshape(n, 45)
    va, vb = sh_values(a), sh_values(b)
    lr_sh = cfg.lrs["lr_features_sh"]
    assert (np.abs(va - vb) > 0.5 * lr_sh + 2e-4).mean() <= 3e-2          # a 16-bit step of a 256-splat block is about 1e-5 here
    # checkpoint: the reference's slot names and flag for this layout; a fresh trainer resumes from it
    out = tmp_path / "ck"
    out.mkdir()
    path = ckpt.save_checkpoint(b, str(out))
    with tarfile.open(path) as tf:
        names = set(tf.getnames())
        manifest = tf.extractfile("state.json").read().decode()
    assert {"eng.sh_quant_fpbo.q.npy", "eng.sh_quant_fpbo.qb.npy", "eng.world.sh_vq16_fpbo.q.npy", "eng.world.sh_vq16_fpbo.qb.npy",
            "eng.means_qfpbo.q.npy", "eng.bias_correction_steps.npy", "eng.radii.npy"} <= names
    assert '"use_fused_proj_bwd_optim": 1' in manifest and "eng.sh_quant.q.npy" not in names
    c = Trainer(cfg, scenes.make_splats(cfg, seed=99), device=U.DEV, fused_backward=True, fused_state_layout="reference", **stock)     # other splats: all of it is replaced
    assert ckpt.load_checkpoint(c, str(out)) == 3
    for t_b, t_c in ((b.sh_packed, c.sh_packed), (b.sh_bounds, c.sh_bounds), (b.sh_optim_packed, c.sh_optim_packed), (b.sh_optim_bounds, c.sh_optim_bounds),
                     (b.params["means"], c.params["means"]), (b.steps, c.steps), (b.nsq_packed["quats"], c.nsq_packed["quats"])):
        assert torch.equal(t_b, t_c)
    with pytest.raises(RuntimeError):
        ckpt.load_checkpoint(a, str(out))                  # a trainer with the shared layout refuses the archive
    lb2, lc2 = np.array(b.train_step(*host, cfg.n_views)), np.array(c.train_step(*host, cfg.n_views))
    assert np.allclose(lb2, lc2, rtol=1e-4, atol=1e-6)
    # SH degree warm-up on this layout: the bands above the active degree are written as zero
    b.set_sh_degree(1)
    b.train_step(*host, cfg.n_views)
    torch.cuda.synchronize()
    vb1 = sh_values(b)
    span = (b.sh_bounds.view(-1, 2)[:, 1] - b.sh_bounds.view(-1, 2)[:, 0]).max().item()
    assert np.abs(vb1[:, 9:]).max() <= span / 65535.0 and np.abs(vb1[:, :9]).max() > 0.01
    for tr in (a, b, c):
        tr.close()


@pytest.mark.parametrize("quant", [False, True])
def test_densification_strategy_runs_with_the_trainer(lib, U, quant):
    """The revised strategy around a Trainer (spirula_studio_b200/densify.py = the host logic of engine_densify_step): scores and
    noise every iteration, relocation + growth on schedule.  The count follows min(capacity, growth * count), dead splats are
    replaced, unused slots stay invisible, everything stays finite and the loss keeps falling."""
    from spirula_studio_b200.trainer import Trainer
    from spirula_studio_b200.densify import DensifyConfig, Densifier
    cfg = scenes.scaled(scenes.CONFIGS["plumbing_50k"], n_splats=12032, width=176, height=128, n_views=3)
    cfg.rig, cfg.rig_radius, cfg.log_scale_mu = "ring", 3.0, -3.0
    if quant:
        cfg.sh_value_bits, cfg.sh_optim_bits = 16, 8
    sp = scenes.make_splats(cfg)
    start = 8000
    sp["opacities"][:start:17] = -8.0                     # some dead splats among the ones in use
    vm, K = scenes.make_cameras(cfg)
    gt = np.stack([scenes.make_target(cfg, v) for v in range(cfg.n_views)])
    host = tuple(torch.from_numpy(a).pin_memory() for a in (vm, K, gt))
    tr = Trainer(cfg, sp, device=U.DEV)
    dc = DensifyConfig(refine_start_iter=4, refine_stop_iter=1000, refine_every=8, growth_factor=1.1, noise_lr=5e5 * 1.6e-4, noise_lr_final=5e5 * 1.6e-6)
    dn = Densifier(tr, dc, start)
    steps, losses, counts = 40, [], []
    for step in range(steps):
        dn.before_step()
        losses.append(tr.train_step(*host, cfg.n_views)[2])
        added = dn.after_step(step, steps)
        counts.append(dn.count)
        if step > dc.refine_start_iter and step % dc.refine_every == 0:
            assert added == min(cfg.n_splats, int(dc.growth_factor * (dn.count - added))) - (dn.count - added)
            assert dn.num_relocated.item() >= 0
            assert not dn.accum_buffer.any()
        else:
            assert added == 0
    torch.cuda.synchronize()
    assert counts[0] == start and counts[-1] == 11712 and counts[-1] <= cfg.n_splats          # 8000 * 1.1^4, floored each time
    op = tr.params["opacities"]
    assert (op[dn.count:] == -30.0).all()                                                       # unused slots untouched
    used = torch.sigmoid(op[:dn.count])
    assert (used <= dc.min_opacity).float().mean().item() < 0.01                                # the seeded dead splats were replaced
    for k, t in tr.params.items():
        if t is not None and not (quant and k == "features_sh"):
            assert torch.isfinite(t[: dn.count * (t.numel() // cfg.n_splats)]).all(), k
    assert np.isfinite(losses).all() and np.mean(losses[-5:]) < np.mean(losses[:5])
    assert dn.radii.max().item() > 0 and dn.accum_buffer[: dn.count, 1].max().item() >= 1
    tr.close()
