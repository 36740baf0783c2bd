"""What happens when a view has more (splat, tile) pairs than the caller's buffers hold, or when a list
names a record that does not exist.  The reference cannot get there: it reads the pair count back to the
host and sizes its buffers exactly (src/kernels/tile/IntersectTile.cu:432-459).  This library keeps the
count on the device, so every consumer of the intersection clamps its ranges to the capacity, skips
entries that name no record, and reports through a status word; nothing here reads or writes outside
the buffers it was given (guard regions placed behind them stay untouched)."""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")

from spirula_studio_b200 import lib as L, scenes  # noqa: E402

pytestmark = pytest.mark.gpu

GUARD = 4096


@pytest.fixture(scope="module")
def lib():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return L.load()


@pytest.fixture(scope="module")
def U():
    from tests import gpu_util
    return gpu_util


def _scene(n=9000, w=208, h=144, views=1):
    cfg = scenes.scaled(scenes.CONFIGS["plumbing_50k"], n_splats=n, width=w, height=h, n_views=views)
    cfg.log_scale_mu = -3.0
    if views > 1:
        cfg.rig, cfg.rig_radius = "ring", 3.0
    return cfg, scenes.make_splats(cfg), *scenes.make_cameras(cfg)


def _raster_both(lib, U, rec, n, offs, flat_buf, cap, n_dev, W, H, v_rgb, vrec_buf):
    """Forward and backward with an explicit list capacity; flat_buf / vrec_buf carry a guard region behind them."""
    P = W * H
    out = dict(rgb=torch.zeros(P, 3, device=U.DEV), T=torch.zeros(P, device=U.DEV), last_ids=torch.zeros(P, dtype=torch.int32, device=U.DEV))
    L.check(lib.ssb_raster_fwd(L.ptr(rec), n, L.ptr(offs), L.ptr(flat_buf), cap, L.ptr(n_dev), 1, W, H,
                               L.ptr(out["rgb"]), None, L.ptr(out["T"]), L.ptr(out["last_ids"]), None))
    L.check(lib.ssb_raster_bwd(L.ptr(rec), n, L.ptr(offs), L.ptr(flat_buf), cap, L.ptr(n_dev), 1, W, H, None, L.ptr(out["T"]),
                               L.ptr(out["last_ids"]), L.ptr(v_rgb), None, None, L.ptr(vrec_buf), None))
    torch.cuda.synchronize()
    return out


def test_overflowing_intersection_is_clamped_for_its_consumers(lib, U):
    cfg, sp, vm, K = _scene()
    n, W, H = cfg.n_splats, cfg.width, cfg.height
    tw, th = (W + 15) // 16, (H + 15) // 16
    pr = U.project_fwd(lib, U.splats_dev(sp), vm, K, W, H)
    _, flat_full, offs_full, M = U.intersect_tiles(lib, pr["aabb"], pr["depths"], pr["rec"], n, n, W, H, 16 * n, tw * th, want_keys=False)
    assert M > 4 * tw * th
    n_dev = torch.tensor([M], dtype=torch.int64, device=U.DEV)
    g = torch.Generator(device=U.DEV); g.manual_seed(3)
    v_rgb = torch.randn(H * W, 3, device=U.DEV, generator=g)
    vrec_full = torch.zeros(n * 12, device=U.DEV)
    full = _raster_both(lib, U, pr["rec"], n, offs_full, flat_full, flat_full.numel(), n_dev, W, H, v_rgb, vrec_full)

    cap = M // 2
    lib.ssb_device_status(None, None)
    # list buffer of `cap` entries followed by a guard of entries that name no record; were a kernel to read
    # one, it would skip it and say so
    ws_bytes = lib.ssb_intersect_tiles_workspace_bytes(tw * th, cap)
    ws = torch.zeros(ws_bytes, dtype=torch.uint8, device=U.DEV)
    flat_buf = torch.full((cap + GUARD,), -1, dtype=torch.int32, device=U.DEV)
    offs = torch.full((tw * th,), -7, dtype=torch.int32, device=U.DEV)
    m_dev = torch.zeros(1, dtype=torch.int64, device=U.DEV)
    L.check(lib.ssb_intersect_tiles(L.ptr(pr["aabb"]), L.ptr(pr["depths"]), L.ptr(pr["rec"]), n, n, W, H, L.ptr(ws), ws_bytes, None,
                                    L.ptr(flat_buf), cap, L.ptr(offs), L.ptr(m_dev), None))
    torch.cuda.synchronize()
    assert int(m_dev.item()) == M                                   # the full count is reported
    assert int(offs.min()) >= 0 and int(offs.max()) <= cap          # no range leaves the list buffer
    assert bool((flat_buf[cap:] == -1).all())                       # nothing written behind it
    vrec_buf = torch.zeros((n + GUARD) * 12, device=U.DEV)
    vrec_buf[n * 12:] = 7.0
    got = _raster_both(lib, U, pr["rec"], n, offs, flat_buf, cap, m_dev, W, H, v_rgb, vrec_buf)
    assert bool((vrec_buf[n * 12:] == 7.0).all())                   # no gradient written behind the record array
    bits = C.c_int32(0)
    assert lib.ssb_device_status(C.byref(bits), None) == L.SSB_ERR_CAPACITY
    assert bits.value == L.STATUS_PAIRS_DROPPED                     # dropped pairs, and no entry outside a buffer was met
    # tiles whose lists lie wholly below the capacity are rendered, and back-propagated from, exactly as in the full run
    ends_full = torch.cat([offs_full[1:].long(), torch.tensor([M], device=U.DEV)])
    whole = ends_full <= cap
    assert int(whole.sum()) > 0 and int((~whole).sum()) > 0
    ys, xs = torch.meshgrid(torch.arange(H, device=U.DEV), torch.arange(W, device=U.DEV), indexing="ij")
    pix_whole = whole[((ys // 16) * tw + xs // 16).reshape(-1)]
    assert torch.equal(got["rgb"][pix_whole], full["rgb"][pix_whole])
    assert torch.equal(got["T"][pix_whole], full["T"][pix_whole])
    assert torch.equal(got["last_ids"][pix_whole], full["last_ids"][pix_whole])
    # tiles past the cut are empty
    cut = offs_full.long() >= cap
    pix_cut = cut[((ys // 16) * tw + xs // 16).reshape(-1)]
    assert bool((got["T"][pix_cut] == 1.0).all()) and bool((got["rgb"][pix_cut] == 0).all())


def test_list_entries_that_name_no_record_are_skipped_and_reported(lib, U):
    cfg, sp, vm, K = _scene(n=4000, w=96, h=64)
    n, W, H = cfg.n_splats, cfg.width, cfg.height
    tw, th = (W + 15) // 16, (H + 15) // 16
    pr = U.project_fwd(lib, U.splats_dev(sp), vm, K, W, H)
    _, flat, offs, M = U.intersect_tiles(lib, pr["aabb"], pr["depths"], pr["rec"], n, n, W, H, 16 * n, tw * th, want_keys=False)
    n_dev = torch.tensor([M], dtype=torch.int64, device=U.DEV)
    v_rgb = torch.ones(H * W, 3, device=U.DEV)
    lib.ssb_device_status(None, None)
    bad = flat.clone()
    bad[: M : 7] = n + 11                                          # beyond the record array
    bad[3: M : 13] = -5                                            # negative
    vrec = torch.zeros((n + GUARD) * 12, device=U.DEV)
    vrec[n * 12:] = 7.0
    out = _raster_both(lib, U, pr["rec"], n, offs, bad, bad.numel(), n_dev, W, H, v_rgb, vrec)
    bits = C.c_int32(0)
    assert lib.ssb_device_status(C.byref(bits), None) == L.SSB_ERR_INVALID_ARGUMENT and bits.value & L.STATUS_BAD_INDEX
    assert bool(torch.isfinite(out["rgb"]).all()) and bool((vrec[n * 12:] == 7.0).all())
    # the same list with those entries removed renders the same image
    keep = torch.ones(bad.numel(), dtype=torch.bool, device=U.DEV)
    keep[: M : 7] = False
    keep[3: M : 13] = False
    keep[M:] = False
    kept_before = torch.cumsum(keep.long(), 0) - keep.long()
    ends = torch.cat([offs[1:].long(), torch.tensor([M], device=U.DEV)])
    offs2 = kept_before[offs.long().clamp(max=M - 1)].int()
    offs2[offs.long() >= M] = int(keep.sum())
    flat2 = flat[keep].contiguous()
    m2 = torch.tensor([flat2.numel()], dtype=torch.int64, device=U.DEV)
    vrec2 = torch.zeros(n * 12, device=U.DEV)
    ref = _raster_both(lib, U, pr["rec"], n, offs2, flat2, flat2.numel(), m2, W, H, v_rgb, vrec2)
    assert lib.ssb_device_status(None, None) == L.SSB_OK
    assert torch.equal(out["rgb"], ref["rgb"]) and torch.equal(out["T"], ref["T"])
    assert float((vrec[: n * 12] - vrec2).abs().max()) <= 1e-4 * float(vrec2.abs().max())
    del ends


def test_step_reports_a_view_that_outgrew_its_capacity(lib, U):
    """Three views through the step object with room for about half of each view's pairs: the step completes,
    says so, and renders the tiles below the cut exactly as a step with enough room does."""
    from spirula_studio_b200.trainer import Trainer
    cfg, sp, vm, K = _scene(n=9000, views=3)
    W, H, n = cfg.width, cfg.height, cfg.n_splats
    tw, th = (W + 15) // 16, (H + 15) // 16
    targets = np.stack([scenes.make_target(cfg, v) for v in range(cfg.n_views)])
    d_vm, d_K, d_gt = (torch.from_numpy(a).to(U.DEV) for a in (vm, K, targets))

    def run(capacity):
        tr = Trainer(cfg, sp, device=U.DEV, isect_capacity=capacity)
        tr.losses.zero_()
        tr.views_fwd_bwd(d_vm, d_K, d_gt, cfg.n_views)
        torch.cuda.synchronize()
        rgb_p = C.c_void_p()
        L.check(lib.ssb_step_peek(tr.handle, C.byref(rgb_p), None, None, None, None, None))
        img = U.tensor_from_device_ptr(rgb_p.value, (H * W, 3))
        return tr, img

    tr_full, img_full = run(0)
    worst = tr_full.check_capacity()
    assert worst > 0
    m_last = tr_full.last_isects()
    cap = m_last // 2
    tr_small, img_small = run(cap)
    with pytest.raises(L.SsbError) as err:
        tr_small.check_capacity()
    assert err.value.status == L.SSB_ERR_CAPACITY
    assert tr_small.check_capacity() == 0                         # the check clears the count
    with pytest.raises(L.SsbError):
        tr_small.last_isects()                                    # the last view alone was too large as well
    assert bool(torch.isfinite(tr_small.grads_flat).all())
    # the same through the host-buffer entry point: the count arrives with the loss scalars
    h_vm, h_K, h_gt = (torch.from_numpy(a).pin_memory() for a in (vm, K, targets))
    with pytest.raises(L.SsbError) as err2:
        tr_small.train_step(h_vm, h_K, h_gt, cfg.n_views)
    assert err2.value.status == L.SSB_ERR_CAPACITY
    # last view: tiles whose lists end below the cut are identical in both runs
    pr = U.project_fwd(lib, U.splats_dev(sp), vm[-1:], K[-1:], W, H)
    _, _, offs_full, M = U.intersect_tiles(lib, pr["aabb"], pr["depths"], pr["rec"], n, n, W, H, 16 * n, tw * th, want_keys=False)
    assert M == m_last
    ends_full = torch.cat([offs_full[1:].long(), torch.tensor([M], device=U.DEV)])
    ys, xs = torch.meshgrid(torch.arange(H, device=U.DEV), torch.arange(W, device=U.DEV), indexing="ij")
    pix_whole = (ends_full <= cap)[((ys // 16) * tw + xs // 16).reshape(-1)]
    assert int(pix_whole.sum()) > 0
    assert torch.equal(img_small[pix_whole], img_full[pix_whole])
    lib.ssb_device_status(None, None)
    tr_full.close(); tr_small.close()
