"""ssb_loss_multi_scale on the GPU against the oracle: masks of the image's size and of another size, one to four levels,
every loss-map mode, ragged image sizes; and the same loss inside the training step (ssb_step_set_loss).  The masked SSIM
part is pinned against the reference's own kernel in test_gpu_golden.py / test_golden_cpu.py (ssim_masked.npz)."""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")

from spirula_studio_b200 import lib as L, scenes  # noqa: E402

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def lib():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return L.load()


def run_loss(lib, render, gt, B, H, W, scales, mask=None, mode=0, w_l1=0.8, w_ssim=0.2):
    d_r, d_g = torch.from_numpy(render).to(DEV), torch.from_numpy(gt).to(DEV)
    d_m = torch.from_numpy(mask).to(DEV) if mask is not None else None
    cfg = L.SsbLossConfig(w_l1, w_ssim, scales, mode, d_m.data_ptr() if d_m is not None else None,
                          mask.shape[1] if mask is not None else 0, mask.shape[2] if mask is not None else 0)
    need = lib.ssb_loss_workspace_bytes(B, H, W, C.byref(cfg))
    assert need > 0
    ws = torch.empty(need, dtype=torch.uint8, device=DEV)
    v = torch.full((B * H * W, 3), 7.0, device=DEV)
    losses = torch.full((3,), 5.0, device=DEV)
    lm = torch.full((B * H * W,), 3.0, device=DEV) if mode else None
    L.check(lib.ssb_loss_multi_scale(L.ptr(d_r), L.ptr(d_g), B, H, W, C.byref(cfg), L.ptr(v), L.ptr(losses), L.ptr(lm), L.ptr(ws), need, None))
    torch.cuda.synchronize()
    return v.cpu().numpy(), losses.cpu().numpy(), lm.cpu().numpy() if lm is not None else None


def frac_bad(a, b, atol, rtol):
    return float((np.abs(a - b) > atol + rtol * np.abs(b)).mean())


def images(B, H, W, seed):
    rng = np.random.default_rng(seed)
    # smooth + noise, so that SSIM is neither ~0 nor ~1
    base = rng.random((B, H // 6 + 2, W // 6 + 2, 3), dtype=np.float32)
    up = np.kron(base, np.ones((1, 6, 6, 1), np.float32))[:, :H, :W]
    r = np.clip(up + 0.1 * rng.standard_normal((B, H, W, 3)).astype(np.float32), 0, 1)
    g = np.clip(up + 0.1 * rng.standard_normal((B, H, W, 3)).astype(np.float32), 0, 1)
    return r.reshape(-1, 3).copy(), g.reshape(-1, 3).copy()


def masks(B, H, W, seed):
    rng = np.random.default_rng(seed)
    same = (rng.random((B, H, W)) > 0.1).astype(np.uint8)
    same[:, H // 5: H // 2, W // 2:] = 0
    other = (rng.random((B, H // 3 + 1, W // 2 + 3)) > 0.2).astype(np.uint8)
    return dict(none=None, same=same, other=other)


@pytest.mark.parametrize("B,H,W", [(1, 96, 130), (2, 67, 45), (1, 33, 31)])
@pytest.mark.parametrize("scales", [1, 2, 4])
def test_multi_scale_loss_matches_oracle(lib, oracle, B, H, W, scales):
    r, g = images(B, H, W, 3 * H + scales)
    for kind, mk in masks(B, H, W, H + W).items():
        for mode in ((0, 1, 3) if kind != "same" else (0, 1, 2, 3, 4)):
            v, losses, lm = run_loss(lib, r, g, B, H, W, scales, mk, mode)
            v_ref, l_ref, lm_ref = oracle.loss_multi_scale(r, g, B, H, W, scales, mask=mk, loss_map_mode=mode)
            tag = (kind, mode)
            assert np.allclose(losses, l_ref, rtol=2e-4, atol=1e-6), (tag, losses, l_ref)
            scale = np.abs(v_ref).max()
            # a sign flip of the L1 term needs |render - target| at rounding level: none in these inputs
            assert frac_bad(v, v_ref, 2e-5 * scale, 1e-3) <= 2e-4, tag
            if mode:
                assert frac_bad(lm, lm_ref, 2e-5, 2e-4) <= 2e-4, tag
            if mk is not None and mk.shape[1:] == (H, W):
                assert np.all(v.reshape(B, H, W, 3)[mk == 0] == 0), tag        # masked pixels receive no gradient


def test_one_level_unmasked_is_the_plain_loss(lib):
    B, H, W = 2, 70, 90
    r, g = images(B, H, W, 9)
    v, losses, lm = run_loss(lib, r, g, B, H, W, 1, None, 2)
    d_r, d_g = torch.from_numpy(r).to(DEV), torch.from_numpy(g).to(DEV)
    v0 = torch.zeros(B * H * W, 3, device=DEV); l0 = torch.zeros(3, device=DEV); lm0 = torch.zeros(B * H * W, device=DEV)
    L.check(lib.ssb_loss_l1_ssim_fwdbwd_map(L.ptr(d_r), L.ptr(d_g), B, H, W, 0.8, 0.2, L.ptr(v0), L.ptr(l0), 1, 0.2, L.ptr(lm0), None))
    torch.cuda.synchronize()
    assert np.array_equal(v, v0.cpu().numpy()) and np.allclose(losses, l0.cpu().numpy(), rtol=1e-6)
    assert np.allclose(lm, lm0.cpu().numpy(), rtol=1e-6, atol=1e-7)
    # an all-ones mask changes nothing beyond the coverage's rounding
    v1, l1, _ = run_loss(lib, r, g, B, H, W, 1, np.ones((B, H, W), np.uint8), 0)
    assert np.abs(v1 - v).max() <= 1e-5 * np.abs(v).max() and np.allclose(l1, losses, rtol=1e-5)


def test_argument_checks(lib):
    cfg = L.SsbLossConfig(0.8, 0.2, 5, 0, None, 0, 0)
    assert lib.ssb_loss_workspace_bytes(1, 8, 8, C.byref(cfg)) == L.SSB_ERR_INVALID_ARGUMENT
    x = torch.zeros(8 * 8 * 3, device=DEV)
    for scales, mode, want in ((5, 0, L.SSB_ERR_INVALID_ARGUMENT), (1, 5, L.SSB_ERR_UNSUPPORTED), (1, 7, L.SSB_ERR_UNSUPPORTED),
                               (1, 11, L.SSB_ERR_INVALID_ARGUMENT)):
        cfg = L.SsbLossConfig(0.8, 0.2, scales, mode, None, 0, 0)
        assert lib.ssb_loss_multi_scale(L.ptr(x), L.ptr(x), 1, 8, 8, C.byref(cfg), L.ptr(x), None, L.ptr(x), L.ptr(x), 768, None) == want
    cfg = L.SsbLossConfig(0.8, 0.2, 3, 0, None, 0, 0)
    assert lib.ssb_loss_multi_scale(L.ptr(x), L.ptr(x), 1, 8, 8, C.byref(cfg), L.ptr(x), None, None, L.ptr(x), 64, None) == L.SSB_ERR_CAPACITY


def test_step_uses_the_general_loss(lib, oracle):
    """ssb_step_set_loss: the step's losses and image gradient with two levels and per-view masks equal the oracle's loss on the step's own render."""
    from spirula_studio_b200.trainer import Trainer
    from tests import gpu_util as U
    cfg = scenes.scaled(scenes.CONFIGS["plumbing_50k"], n_splats=8000, width=160, height=112, n_views=2)
    cfg.rig, cfg.rig_radius, cfg.log_scale_mu = "ring", 3.0, -3.0
    sp = scenes.make_splats(cfg)
    vm, K = scenes.make_cameras(cfg)
    gt = np.stack([scenes.make_target(cfg, v) for v in range(cfg.n_views)]).astype(np.float32)
    H, W = cfg.height, cfg.width
    mk = masks(cfg.n_views, H, W, 4)["same"]
    d_mask = torch.from_numpy(mk).to(DEV)
    tr = Trainer(cfg, sp, device=DEV)
    lc = L.SsbLossConfig(0.0, 0.0, 2, 0, d_mask.data_ptr(), H, W)
    L.check(lib.ssb_step_set_loss(tr.handle, C.byref(lc)))
    d_vm, d_K, d_gt = (torch.from_numpy(a).to(DEV) for a in (vm, K, gt))
    tr.losses.zero_()
    tr.views_fwd_bwd(d_vm, d_K, d_gt, cfg.n_views)
    torch.cuda.synchronize()
    got = tr.losses.cpu().numpy()
    pairs_masked = tr.last_isects()
    g_masked = {k: t.clone() for k, t in tr.grads.items()}
    # the last view's render, pushed through the oracle's loss
    rgb_p = C.c_void_p()
    L.check(lib.ssb_step_peek(tr.handle, C.byref(rgb_p), None, None, None, None, None))
    img = U.tensor_from_device_ptr(rgb_p.value, (H * W, 3)).cpu().numpy()
    _, l_last, _ = oracle.loss_multi_scale(img, gt[-1].reshape(-1, 3), 1, H, W, 2, mask=mk[-1:])
    # and the first view's, rendered again without the general loss
    L.check(lib.ssb_step_set_loss(tr.handle, None))
    tr.losses.zero_()
    tr.views_fwd_bwd(d_vm, d_K, d_gt, 1)
    torch.cuda.synchronize()
    L.check(lib.ssb_step_peek(tr.handle, C.byref(rgb_p), None, None, None, None, None))
    img0 = U.tensor_from_device_ptr(rgb_p.value, (H * W, 3)).cpu().numpy()
    _, l_first, _ = oracle.loss_multi_scale(img0, gt[0].reshape(-1, 3), 1, H, W, 2, mask=mk[:1])
    assert np.allclose(got, l_first + l_last, rtol=1e-3, atol=1e-5), (got, l_first + l_last)
    # with the mask the step left the dead tiles of the last view out of the intersection; the render in live tiles is unchanged
    tr.losses.zero_()
    tr.views_fwd_bwd(d_vm, d_K, d_gt, cfg.n_views)
    torch.cuda.synchronize()
    live = oracle.tile_active(mk[-1:], W, H)[0]
    assert 0 < live.sum() < live.size and pairs_masked < tr.last_isects()
    L.check(lib.ssb_step_peek(tr.handle, C.byref(rgb_p), None, None, None, None, None))
    full = U.tensor_from_device_ptr(rgb_p.value, (H, W, 3)).cpu().numpy()
    live_px = np.kron(live, np.ones((16, 16), np.int32))[:H, :W].astype(bool)
    assert np.array_equal(full[live_px], img.reshape(H, W, 3)[live_px])
    # the masked, two-level gradient differs from the plain one and is finite
    assert all(torch.isfinite(t).all() for t in g_masked.values())
    assert (g_masked["means"] - tr.grads["means"]).abs().max() > 0
    tr.close()
