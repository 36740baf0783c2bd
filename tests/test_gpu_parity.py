"""Parity of the CUDA path (through the C ABI) with the CPU oracle on the same
seeded inputs.  Integer stages are compared bit for bit given the oracle's
floating-point inputs; floating-point stages use the reference parity tools'
tolerance model |d| <= atol + rtol*|ref| with a capped violation fraction
(src/backend/tests/projection_parity.cpp:347-364, render_parity.cpp:342-357,
raster_bwd_parity.cpp:360-368), tightened where the north-star states a bound:
images 1e-4 max abs, gradients and post-Adam parameters 1e-3 relative."""
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


def scene(n=20000, w=320, h=240, views=2, seed=scenes.SPLAT_SEED, base="plumbing_50k", scale_mu=None, extent=None):
    cfg = scenes.scaled(scenes.CONFIGS[base], n_splats=n, width=w, height=h, n_views=views)
    if scale_mu is not None:
        cfg.log_scale_mu = scale_mu
    if extent is not None:
        cfg.mean_extent = extent
    if views > 1:
        cfg.rig, cfg.rig_radius = "ring", 3.0
    sp = scenes.make_splats(cfg, seed=seed)
    vm, K = scenes.make_cameras(cfg)
    return cfg, sp, vm, K


# ---------------------------------------------------------------- projection
@pytest.mark.parametrize("views", [1, 2])
def test_projection_forward(lib, U, oracle, views):
    cfg, sp, vm, K = scene(views=views, scale_mu=-3.5)
    W, H, n = cfg.width, cfg.height, cfg.n_splats
    ref = oracle.project_fwd(sp, vm, K, W, H)
    got = U.project_fwd(lib, U.splats_dev(sp), vm, K, W, H)
    aabb = got["aabb"].cpu().numpy()
    keep_ref = ref["aabb"][:, 2] > ref["aabb"][:, 0]
    keep_got = aabb[:, 2] > aabb[:, 0]
    assert keep_ref.sum() > 0.3 * keep_ref.size
    assert (keep_ref != keep_got).mean() <= 2e-4            # borderline culls may flip
    both = keep_ref & keep_got
    scr = U.unpack_screen(lib, got["rec"], views * n)
    assert U.close_frac(aabb[both], ref["aabb"][both], 5e-3, 5e-4) <= 2e-4
    assert U.close_frac(got["depths"].cpu().numpy()[both], ref["depths"][both], 1e-5, 1e-5) == 0.0
    for k, (atol, rtol) in dict(xy=(2e-3, 1e-5), depth=(1e-5, 1e-5), conic=(1e-5, 5e-4), opac=(1e-6, 1e-5), rgb=(2e-5, 1e-5)).items():
        assert U.close_frac(scr[k][both], ref[k][both], atol, rtol) <= 2e-4, k
    assert U.close_frac(got["radii"].cpu().numpy(), ref["radii"], 1e-6, 1e-4) <= 2e-4
    # visible counts
    assert abs(int(keep_got.sum()) - int(keep_ref.sum())) <= max(2, int(2e-4 * keep_ref.size))


def test_projection_forward_quantized_sh(lib, U, oracle):
    cfg, sp, vm, K = scene(n=8000, views=1, scale_mu=-3.5)
    W, H, n = cfg.width, cfg.height, cfg.n_splats
    for bits in (16, 8):
        packed, bounds = oracle.quant_encode(sp["features_sh"], bits)
        ref = oracle.project_fwd(sp, vm, K, W, H, shq=dict(packed=packed, bounds=bounds, bits=bits, bounds_stride=256))
        d_packed, d_bounds = U.dev(packed), U.dev(bounds)
        shq = L.shq_struct(d_packed, d_bounds, bits, 256)
        got = U.project_fwd(lib, U.splats_dev(sp), vm, K, W, H, shq=shq)
        keep = (ref["aabb"][:, 2] > ref["aabb"][:, 0]) & (got["aabb"].cpu().numpy()[:, 2] > got["aabb"].cpu().numpy()[:, 0])
        scr = U.unpack_screen(lib, got["rec"], n)
        assert U.close_frac(scr["rgb"][keep], ref["rgb"][keep], 2e-5, 1e-5) <= 2e-4
        # and the codec itself: GPU encode gives the same codes as the oracle (+-1 at rounding ties)
        gp = torch.zeros_like(d_packed)
        gb = torch.zeros_like(d_bounds)
        d_sh = U.dev(sp["features_sh"].reshape(-1))
        L.check(lib.ssb_quant_encode(L.ptr(d_sh), n * 45, bits, L.ptr(gp), L.ptr(gb), None))
        torch.cuda.synchronize()
        assert np.array_equal(gb.cpu().numpy(), bounds)
        view = np.uint16 if bits == 16 else np.uint8
        diff = np.abs(gp.cpu().numpy().view(view).astype(np.int64) - packed.view(view).astype(np.int64))
        assert diff.max() <= 1 and (diff > 0).mean() < 1e-3


def test_projection_backward(lib, U, oracle):
    cfg, sp, vm, K = scene(n=12000, views=2, scale_mu=-3.5)
    W, H, n = cfg.width, cfg.height, cfg.n_splats
    ref_f = oracle.project_fwd(sp, vm, K, W, H)
    rng = np.random.default_rng(3)
    m = 2 * n
    v = dict(v_xy=rng.normal(size=(m, 2)), v_depth=rng.normal(size=m), v_conic=rng.normal(size=(m, 3)) * 0.05, v_opac=rng.normal(size=m),
             v_rgb=rng.normal(size=(m, 3)))
    v = {k: x.astype(np.float32) for k, x in v.items()}
    ref = oracle.project_bwd(sp, vm, K, W, H, ref_f["aabb"], v)
    spd = U.splats_dev(sp)
    grads = {k: torch.full_like(t, 7.0) for k, t in spd.items()}      # overwritten when accumulate == 0
    s, g = L.splats_struct(spd), L.splats_struct(grads)
    d_vm, d_K, d_aabb = U.dev(vm), U.dev(K), U.dev(ref_f["aabb"])
    cams = L.cameras_struct(d_vm, d_K, W, H)
    vrec = U.arrays_to_vrec(v, m)
    L.check(lib.ssb_project_bwd(C.byref(s), None, n, C.byref(cams), L.ptr(d_aabb), L.ptr(vrec), C.byref(g), 0, None))
    torch.cuda.synchronize()
    for k in ref:
        got = grads[k].cpu().numpy().reshape(ref[k].shape)
        scale = np.abs(ref[k]).max()
        assert U.close_frac(got, ref[k], 1e-5 * scale, 1e-3) <= 2e-3, k
    # accumulate == 1 adds on top
    L.check(lib.ssb_project_bwd(C.byref(s), None, n, C.byref(cams), L.ptr(d_aabb), L.ptr(vrec), C.byref(g), 1, None))
    torch.cuda.synchronize()
    got = grads["means"].cpu().numpy().reshape(-1, 3)
    assert U.close_frac(got, 2 * ref["means"], 2e-5 * np.abs(ref["means"]).max(), 1e-3) <= 2e-3


def wide_scene(model, n=6000, seed=21):
    """Camera inside the cloud: an equidistant fisheye (model 1, ~190 degrees), an equisolid fisheye (model 2, ~167 degrees:
    2 f exceeds the half diagonal, so the singular direction straight behind the camera maps outside the image) or an
    equirectangular camera (model 3)."""
    W, H, f = (240, 240, 72.0 if model == 1 else 90.0) if model in (1, 2) else (320, 160, 320 / (2 * np.pi))
    cfg = scenes.scaled(scenes.CONFIGS["plumbing_50k"], n_splats=n, width=W, height=H)
    cfg.log_scale_mu, cfg.mean_extent = -2.6, 3.0
    sp = scenes.make_splats(cfg, seed=seed)
    vm = np.stack([scenes.look_at((0.2, -0.1, 0.15), (1.0, 0.3, 2.0)), scenes.look_at((-0.3, 0.2, 0.1), (-1.0, 0.5, -1.0))]).reshape(2, 16)
    K = np.tile(np.array([[f, f, W / 2.0, H / 2.0]], dtype=np.float32), (2, 1))
    return cfg, sp, vm.astype(np.float32), K


def away_from_back_axis(sp, vm, limit_deg=170.0):
    """[views, n] mask of splats whose direction is more than 10 degrees away from straight behind the camera.  Both fisheye
    projections are singular there (the whole image circle is one direction): a one-ulp change of a mean moves the conic and
    the gradients of such a splat by more than the tolerances below, in the oracle as much as in the library."""
    out = []
    for m in vm.reshape(-1, 4, 4).astype(np.float64):
        pc = sp["means"].astype(np.float64) @ m[:3, :3].T + m[:3, 3]
        out.append(np.degrees(np.arctan2(np.hypot(pc[:, 0], pc[:, 1]), pc[:, 2])) < limit_deg)
    return np.stack(out)


@pytest.mark.parametrize("model", [L.CAMERA_FISHEYE, L.CAMERA_EQUISOLID, L.CAMERA_EQUIRECT])
def test_projection_forward_wide_cameras(lib, U, oracle, model):
    cfg, sp, vm, K = wide_scene(model)
    W, H, n = cfg.width, cfg.height, cfg.n_splats
    ref = oracle.project_fwd(sp, vm, K, W, H, model=model)
    got = U.project_fwd(lib, U.splats_dev(sp), vm, K, W, H, model=model)
    aabb = got["aabb"].cpu().numpy()
    keep_ref, keep_got = ref["aabb"][:, 2] > ref["aabb"][:, 0], aabb[:, 2] > aabb[:, 0]
    assert keep_ref.sum() > 0.3 * keep_ref.size
    assert (keep_ref != keep_got).mean() <= 5e-4
    both = keep_ref & keep_got
    if model == L.CAMERA_EQUISOLID:
        both &= away_from_back_axis(sp, vm).reshape(-1)
    scr = U.unpack_screen(lib, got["rec"], 2 * n)
    assert U.close_frac(aabb[both], ref["aabb"][both], 5e-3, 5e-4) <= 5e-4
    assert U.close_frac(got["depths"].cpu().numpy()[both], ref["depths"][both], 1e-5, 1e-5) == 0.0
    for k, (atol, rtol) in dict(xy=(2e-3, 1e-5), depth=(1e-5, 1e-5), conic=(1e-5, 1e-3), opac=(1e-6, 1e-5), rgb=(2e-5, 1e-5)).items():
        assert U.close_frac(scr[k][both], ref[k][both], atol, rtol) <= 5e-4, k


@pytest.mark.parametrize("model", [L.CAMERA_FISHEYE, L.CAMERA_EQUISOLID, L.CAMERA_EQUIRECT])
def test_projection_backward_wide_cameras(lib, U, oracle, model):
    cfg, sp, vm, K = wide_scene(model)
    W, H, n = cfg.width, cfg.height, cfg.n_splats
    ref_f = oracle.project_fwd(sp, vm, K, W, H, model=model)
    rng = np.random.default_rng(4)
    m = 2 * n
    v = dict(v_xy=rng.normal(size=(m, 2)), v_depth=rng.normal(size=m), v_conic=rng.normal(size=(m, 3)) * 0.05, v_opac=rng.normal(size=m),
             v_rgb=rng.normal(size=(m, 3)))
    v = {k: x.astype(np.float32) for k, x in v.items()}
    ref = oracle.project_bwd(sp, vm, K, W, H, ref_f["aabb"], v, model=model)
    spd = U.splats_dev(sp)
    for views in (2, 1):      # the several-view and the single-view kernel
        grads = {k: torch.full_like(t, 7.0) for k, t in spd.items()}
        s, g = L.splats_struct(spd), L.splats_struct(grads)
        d_vm, d_K, d_aabb = U.dev(vm), U.dev(K), U.dev(ref_f["aabb"])
        cams = L.cameras_struct(d_vm, d_K, W, H, model=model, count=views)
        vrec = U.arrays_to_vrec(v, m)
        L.check(lib.ssb_project_bwd(C.byref(s), None, n, C.byref(cams), L.ptr(d_aabb), L.ptr(vrec), C.byref(g), 0, None))
        torch.cuda.synchronize()
        want = ref if views == 2 else oracle.project_bwd(sp, vm[:1], K[:1], W, H, ref_f["aabb"][:n], {k: x[:n] for k, x in v.items()}, model=model)
        rows = away_from_back_axis(sp, vm[:views]).all(0) if model == L.CAMERA_EQUISOLID else np.ones(n, bool)
        for k in want:
            got = grads[k].cpu().numpy().reshape(want[k].shape)
            scale = np.abs(want[k]).max()
            assert U.close_frac(got[rows], want[k][rows], 1e-5 * scale, 1e-3) <= 2e-3, (k, views)


def test_distorted_pinhole_with_the_jacobian_limit_active(lib, U, oracle):
    """Pinhole + OpenCV tier on a wide cloud of large splats: many centres lie outside the 1.3x frustum, so the third
    column of the Jacobian is limited (src/shaders/primitive_3dgs.slang:84-95) while d(mean2d)/d(mean) is not; forward and
    backward against the oracle, several-view and single-view kernels."""
    cfg, sp, vm, K = scene(n=6000, w=160, h=120, views=2, scale_mu=-1.2, extent=4.0)
    W, H, n = cfg.width, cfg.height, cfg.n_splats
    rows = np.array([[0.06, -0.01, 0.002, -0.001, 0, 0, 0, 0], [-0.05, 0.004, 0.001, 0.002, 0, 0, 0, 0]], np.float32)
    ref_f = oracle.project_fwd(sp, vm, K, W, H, dist=L.DISTORTION_OPENCV, dist_coeffs=rows)
    keep_ref = ref_f["aabb"][:, 2] > ref_f["aabb"][:, 0]
    # how many visible splats have the limit active: centre more than 15 % of the width outside the image on x
    out_x = (ref_f["xy"][:, 0] < -0.15 * W) | (ref_f["xy"][:, 0] > 1.15 * W)
    assert (keep_ref & out_x).sum() > 50
    spd = U.splats_dev(sp)
    d_vm, d_K, d_rows = U.dev(vm), U.dev(K), U.dev(rows)
    m = 2 * n
    cams = L.cameras_struct(d_vm, d_K, W, H, distortion=L.DISTORTION_OPENCV, dist_coeffs=d_rows)
    aabb, depths, radii = torch.zeros(m, 4, device=U.DEV), torch.zeros(m, device=U.DEV), torch.zeros(n, device=U.DEV)
    rec = torch.zeros(m * L.SCREEN_REC_FLOATS, device=U.DEV)
    s = L.splats_struct(spd)
    L.check(lib.ssb_project_fwd(C.byref(s), None, n, C.byref(cams), L.ptr(aabb), L.ptr(depths), L.ptr(radii), L.ptr(rec), None))
    torch.cuda.synchronize()
    h_aabb = aabb.cpu().numpy()
    keep_got = h_aabb[:, 2] > h_aabb[:, 0]
    assert (keep_ref != keep_got).mean() <= 5e-4
    both = keep_ref & keep_got
    scr = U.unpack_screen(lib, rec, m)
    assert U.close_frac(h_aabb[both], ref_f["aabb"][both], 5e-3, 5e-4) <= 5e-4
    for k, (atol, rtol) in dict(xy=(2e-3, 1e-5), conic=(1e-5, 1e-3), opac=(1e-6, 1e-5)).items():
        assert U.close_frac(scr[k][both], ref_f[k][both], atol, rtol) <= 5e-4, k
    rng = np.random.default_rng(11)
    v = dict(v_xy=rng.normal(size=(m, 2)), v_depth=rng.normal(size=m), v_conic=rng.normal(size=(m, 3)) * 0.05, v_opac=rng.normal(size=m),
             v_rgb=rng.normal(size=(m, 3)))
    v = {k: x.astype(np.float32) for k, x in v.items()}
    d_aabb, vrec = U.dev(ref_f["aabb"]), U.arrays_to_vrec(v, m)
    for views in (2, 1):
        grads = {k: torch.full_like(t, 7.0) for k, t in spd.items()}
        g = L.splats_struct(grads)
        cams_v = L.cameras_struct(d_vm, d_K, W, H, count=views, distortion=L.DISTORTION_OPENCV, dist_coeffs=d_rows)
        L.check(lib.ssb_project_bwd(C.byref(s), None, n, C.byref(cams_v), L.ptr(d_aabb), L.ptr(vrec), C.byref(g), 0, None))
        torch.cuda.synchronize()
        want = oracle.project_bwd(sp, vm[:views], K[:views], W, H, ref_f["aabb"][:views * n], {k: x[:views * n] for k, x in v.items()},
                                  dist=L.DISTORTION_OPENCV, dist_coeffs=rows[:views])
        for k in want:
            got = grads[k].cpu().numpy().reshape(want[k].shape)
            assert U.close_frac(got, want[k], 1e-5 * np.abs(want[k]).max(), 1e-3) <= 2e-3, (k, views)


# ------------------------------------------------------- keys / sort / ranges
@pytest.mark.parametrize("views,scale_mu", [(1, -3.5), (2, -3.0), (1, -2.0)])
def test_tile_keys_bit_exact(lib, U, oracle, views, scale_mu):
    cfg, sp, vm, K = scene(n=15000, views=views, scale_mu=scale_mu)
    W, H, n = cfg.width, cfg.height, cfg.n_splats
    proj = oracle.project_fwd(sp, vm, K, W, H)
    counts, cum, keys, vals = oracle.tile_keys(proj, n, W, H)
    rec = U.pack_screen(lib, proj)
    cap = int(keys.size) + 100
    st, M, g_counts, g_cum, g_keys, g_vals, n_dev = U.tile_keys(lib, U.dev(proj["aabb"]), U.dev(proj["depths"]), rec, views * n, n, W, H, cap)
    assert st == 0 and M == keys.size and int(n_dev.item()) == M
    assert np.array_equal(g_counts.cpu().numpy().astype(np.int64), counts)
    assert np.array_equal(g_cum.cpu().numpy().astype(np.int64), cum)
    assert np.array_equal(g_keys.cpu().numpy()[:M], keys)
    assert np.array_equal(g_vals.cpu().numpy()[:M], vals)
    # a capacity that is too small is reported, not overrun
    st2, M2, *_ = U.tile_keys(lib, U.dev(proj["aabb"]), U.dev(proj["depths"]), rec, views * n, n, W, H, max(M // 2, 1))
    assert st2 == L.SSB_ERR_CAPACITY and M2 == M


@pytest.mark.parametrize("views,scale_mu,n,w,h", [(1, -3.5, 15000, 320, 240), (2, -3.0, 15000, 320, 240), (1, -2.0, 15000, 320, 240),
                                                  (1, -1.2, 9000, 64, 48)])
def test_intersect_tiles_fused_bit_exact(lib, U, oracle, views, scale_mu, n, w, h):
    """ssb_intersect_tiles against keys -> stable sort -> ranges of the oracle: same sorted keys, same sorted
    flatten ids, same ranges, same count.  The last case has lists longer than the kernel sorts in shared
    memory (a few tiles, thousands of large splats each)."""
    cfg, sp, vm, K = scene(n=n, w=w, h=h, views=views, scale_mu=scale_mu)
    W, H = cfg.width, cfg.height
    proj = oracle.project_fwd(sp, vm, K, W, H)
    counts, cum, keys, vals = oracle.tile_keys(proj, n, W, H)
    tw, th = oracle.tile_grid(W, H)
    n_tiles = tw * th * views
    sk, sv = oracle.sort_pairs(keys, vals, 0, 32 + oracle.tile_n_bits(n_tiles))
    offs = oracle.tile_offsets(sk, n_tiles)
    M = int(keys.size)
    if scale_mu > -1.5:
        assert np.diff(np.append(offs, M)).max() > 4096
    rec = U.pack_screen(lib, proj)
    d_aabb, d_depths = U.dev(proj["aabb"]), U.dev(proj["depths"])
    g_keys, g_vals, g_offs, g_M = U.intersect_tiles(lib, d_aabb, d_depths, rec, views * n, n, W, H, M + 64, n_tiles)
    assert g_M == M
    assert np.array_equal(g_offs.cpu().numpy().astype(np.int64), offs.astype(np.int64))
    assert np.array_equal(g_vals.cpu().numpy()[:M], sv)
    assert np.array_equal(g_keys.cpu().numpy()[:M], sk)
    assert int(g_vals[M:].max()) == -1                      # nothing written past the count
    # the keys are optional
    _, g_vals2, _, _ = U.intersect_tiles(lib, d_aabb, d_depths, rec, views * n, n, W, H, M + 64, n_tiles, want_keys=False)
    assert np.array_equal(g_vals2.cpu().numpy()[:M], sv)
    # too small a capacity: the full count is still reported, every range handed on is clamped to the capacity,
    # what fits is a prefix of the sorted order, and the device status word says that pairs were dropped
    cap = max(M // 2, 1)
    lib.ssb_device_status(None, None)                      # clear what earlier calls may have left
    _, g_vals3, g_offs3, g_M3 = U.intersect_tiles(lib, d_aabb, d_depths, rec, views * n, n, W, H, cap, n_tiles, want_keys=False)
    assert g_M3 == M and np.array_equal(g_offs3.cpu().numpy().astype(np.int64), np.minimum(offs.astype(np.int64), cap))
    bits = C.c_int32(0)
    assert lib.ssb_device_status(C.byref(bits), None) == L.SSB_ERR_CAPACITY and bits.value & L.STATUS_PAIRS_DROPPED
    assert lib.ssb_device_status(C.byref(bits), None) == L.SSB_OK and bits.value == 0        # reading clears it
    whole = offs[np.append(offs[1:], M) <= cap]            # tiles that lie wholly below the capacity
    if whole.size:
        end = int(np.append(offs[1:], M)[np.append(offs[1:], M) <= cap].max())
        assert np.array_equal(g_vals3.cpu().numpy()[:end], sv[:end])


def test_packed_projection_and_intersection(lib, U, oracle):
    """Packed projection = the visible pairs of the unpacked one, compacted view-major with their ids; the packed
    intersection gives the lists of the unpacked one with packed indices in place of pair indices."""
    cfg, sp, vm, K = scene(n=9000, views=2, scale_mu=-3.0, extent=3.5)     # part of the cloud is outside each view
    W, H, n = cfg.width, cfg.height, cfg.n_splats
    spd = U.splats_dev(sp)
    un = U.project_fwd(lib, spd, vm, K, W, H)
    aabb = un["aabb"].cpu().numpy()
    keep = aabb[:, 2] > aabb[:, 0]
    V = int(keep.sum())
    assert 0.2 * keep.size < V < keep.size
    cap = V + 50
    ws_bytes = lib.ssb_project_fwd_packed_workspace_bytes(n, 2)
    ws = torch.zeros(ws_bytes, dtype=torch.uint8, device=U.DEV)
    p_aabb = torch.zeros(cap, 4, device=U.DEV); p_depths = torch.zeros(cap, device=U.DEV); p_radii = torch.zeros(n, device=U.DEV)
    p_rec = torch.zeros(cap * L.SCREEN_REC_FLOATS, device=U.DEV)
    p_cam = torch.full((cap,), -1, dtype=torch.int32, device=U.DEV); p_gid = torch.full((cap,), -1, dtype=torch.int32, device=U.DEV)
    n_vis = torch.zeros(1, dtype=torch.int64, device=U.DEV)
    h_n = C.c_int64(-1)
    s = L.splats_struct(spd)
    cams = L.cameras_struct(un["vm"], un["K"], W, H)
    L.check(lib.ssb_project_fwd_packed(C.byref(s), None, n, C.byref(cams), L.ptr(ws), ws_bytes, L.ptr(p_aabb), L.ptr(p_depths), L.ptr(p_radii),
                                       L.ptr(p_rec), L.ptr(p_cam), L.ptr(p_gid), cap, L.ptr(n_vis), C.byref(h_n), None))
    assert h_n.value == V and int(n_vis.item()) == V
    where = np.nonzero(keep)[0]
    assert np.array_equal(p_cam.cpu().numpy()[:V], where // n) and np.array_equal(p_gid.cpu().numpy()[:V], where % n)
    assert int(p_cam[V:].max()) == -1
    assert np.array_equal(p_aabb.cpu().numpy()[:V], aabb[keep])
    assert np.array_equal(p_depths.cpu().numpy()[:V], un["depths"].cpu().numpy()[keep])
    assert np.array_equal(p_rec.cpu().numpy().reshape(cap, -1)[:V], un["rec"].cpu().numpy().reshape(2 * n, -1)[keep])
    assert np.array_equal(p_radii.cpu().numpy(), un["radii"].cpu().numpy())
    # a capacity that is too small is reported
    st = lib.ssb_project_fwd_packed(C.byref(s), None, n, C.byref(cams), L.ptr(ws), ws_bytes, L.ptr(p_aabb), L.ptr(p_depths), None,
                                    L.ptr(p_rec), L.ptr(p_cam), L.ptr(p_gid), V // 2, L.ptr(n_vis), C.byref(h_n), None)
    assert st == L.SSB_ERR_CAPACITY and h_n.value == V
    L.check(lib.ssb_project_fwd_packed(C.byref(s), None, n, C.byref(cams), L.ptr(ws), ws_bytes, L.ptr(p_aabb), L.ptr(p_depths), None,
                                       L.ptr(p_rec), L.ptr(p_cam), L.ptr(p_gid), cap, L.ptr(n_vis), None, None))
    # intersection: unpacked (pair index = view * n + splat) against packed (pair index = packed position)
    tw, th = oracle.tile_grid(W, H)
    n_tiles = tw * th * 2
    u_keys, u_vals, u_offs, M = U.intersect_tiles(lib, un["aabb"], un["depths"], un["rec"], 2 * n, n, W, H, 40 * n, n_tiles)
    icap = M + 10
    iws_bytes = lib.ssb_intersect_tiles_workspace_bytes(n_tiles, icap)
    iws = torch.zeros(iws_bytes, dtype=torch.uint8, device=U.DEV)
    keys = torch.full((icap,), -1, dtype=torch.int64, device=U.DEV); vals = torch.full((icap,), -1, dtype=torch.int32, device=U.DEV)
    offs = torch.full((n_tiles,), -7, dtype=torch.int32, device=U.DEV); n_is = torch.zeros(1, dtype=torch.int64, device=U.DEV)
    L.check(lib.ssb_intersect_tiles_packed(L.ptr(p_aabb), L.ptr(p_depths), L.ptr(p_rec), L.ptr(p_cam), L.ptr(n_vis), cap, 2, W, H,
                                           L.ptr(iws), iws_bytes, L.ptr(keys), L.ptr(vals), icap, L.ptr(offs), L.ptr(n_is), None))
    torch.cuda.synchronize()
    assert int(n_is.item()) == M
    assert np.array_equal(offs.cpu().numpy(), u_offs.cpu().numpy())
    assert np.array_equal(keys.cpu().numpy()[:M], u_keys.cpu().numpy()[:M])
    assert np.array_equal(where[vals.cpu().numpy()[:M]], u_vals.cpu().numpy()[:M])
    # backward: packed cotangents give the gradients of the unpacked call
    rng = np.random.default_rng(9)
    v_un = (rng.normal(size=(2 * n, L.SCREEN_REC_FLOATS)) * 0.1).astype(np.float32)
    d_v_un = U.dev(v_un.reshape(-1))
    d_v_pk = torch.zeros(cap * L.SCREEN_REC_FLOATS, device=U.DEV)
    d_v_pk.view(cap, -1)[:V] = U.dev(v_un[keep])
    g_un = {k: torch.zeros_like(t) for k, t in spd.items()}
    g_pk = {k: torch.full_like(t, 3.0) for k, t in spd.items()}
    gs_un, gs_pk = L.splats_struct(g_un), L.splats_struct(g_pk)
    L.check(lib.ssb_project_bwd(C.byref(s), None, n, C.byref(cams), L.ptr(un["aabb"]), L.ptr(d_v_un), C.byref(gs_un), 0, None))
    bws_bytes = lib.ssb_project_bwd_packed_workspace_bytes(n, 2)
    bws = torch.zeros(bws_bytes, dtype=torch.uint8, device=U.DEV)
    L.check(lib.ssb_project_bwd_packed(C.byref(s), None, n, C.byref(cams), L.ptr(p_aabb), L.ptr(d_v_pk), L.ptr(p_cam), L.ptr(p_gid), L.ptr(n_vis), cap,
                                       L.ptr(bws), bws_bytes, C.byref(gs_pk), 0, None))
    torch.cuda.synchronize()
    for k in g_un:
        assert torch.equal(g_un[k], g_pk[k]), k
    assert float(g_un["means"].abs().sum()) > 0


def test_intersect_tiles_empty(lib, U, oracle):
    cfg, sp, vm, K = scene(n=256, views=1)
    sp["means"][:, 2] = 50.0
    proj = oracle.project_fwd(sp, vm, K, cfg.width, cfg.height)
    rec = U.pack_screen(lib, proj)
    tw, th = oracle.tile_grid(cfg.width, cfg.height)
    _, vals, offs, M = U.intersect_tiles(lib, U.dev(proj["aabb"]), U.dev(proj["depths"]), rec, 256, 256, cfg.width, cfg.height, 16, tw * th)
    assert M == 0 and int(offs.abs().sum()) == 0 and int(vals.max()) == -1


def test_tile_keys_empty_and_all_culled(lib, U, oracle):
    cfg, sp, vm, K = scene(n=256, views=1)
    sp["means"][:, 2] = 50.0    # behind the camera at (0,0,3) looking down -z
    proj = oracle.project_fwd(sp, vm, K, cfg.width, cfg.height)
    assert not np.any(proj["aabb"])
    rec = U.pack_screen(lib, proj)
    st, M, counts, cum, keys, vals, n_dev = U.tile_keys(lib, U.dev(proj["aabb"]), U.dev(proj["depths"]), rec, 256, 256, cfg.width, cfg.height, 16)
    assert st == 0 and M == 0 and int(counts.sum()) == 0
    tw, th = oracle.tile_grid(cfg.width, cfg.height)
    offs = U.tile_ranges(lib, keys, n_dev, 16, tw * th)
    assert int(offs.abs().sum()) == 0


@pytest.mark.parametrize("n", [0, 1, 31, 4096, 4097, 100003])
def test_sort_pairs_bit_exact(lib, U, oracle, n):
    rng = np.random.default_rng(n)
    keys = rng.integers(0, 1 << 46, size=n, dtype=np.int64)
    if n > 10:
        keys[::5] = keys[3]                       # ties exercise stability
        keys[1::11] |= np.int64(1) << 60          # bits outside the sorted range must be ignored
    vals = np.arange(n, dtype=np.int32)
    cap = n + 13
    for b0, b1 in ((0, 45), (0, 33), (0, 64), (32, 45)):
        dk = torch.zeros(cap, dtype=torch.int64, device=U.DEV); dk[:n] = U.dev(keys)
        dv = torch.zeros(cap, dtype=torch.int32, device=U.DEV); dv[:n] = U.dev(vals)
        n_dev = torch.tensor([n], dtype=torch.int64, device=U.DEV)
        sk, sv = U.sort_pairs(lib, dk, dv, n_dev, cap, b0, b1)
        rk, rv = oracle.sort_pairs(keys, vals, b0, b1)
        assert np.array_equal(sv.cpu().numpy()[:n], rv) and np.array_equal(sk.cpu().numpy()[:n], rk)


def test_tile_ranges_bit_exact(lib, U, oracle):
    rng = np.random.default_rng(9)
    n_tiles = 1200
    tiles = np.sort(rng.integers(5, 1100, size=30000)).astype(np.int64)
    keys = (tiles << 32) | rng.integers(0, 1 << 32, size=tiles.size, dtype=np.int64)
    ref = oracle.tile_offsets(keys, n_tiles)
    n_dev = torch.tensor([keys.size], dtype=torch.int64, device=U.DEV)
    got = U.tile_ranges(lib, U.dev(keys), n_dev, keys.size, n_tiles)
    assert np.array_equal(got.cpu().numpy(), ref)


# ------------------------------------------------------------------ raster
def _chain(oracle, cfg, sp, vm, K):
    return oracle.forward_chain(sp, vm, K, cfg.width, cfg.height)


@pytest.mark.parametrize("views,scale_mu,w,h", [(1, -3.2, 320, 240), (2, -2.6, 200, 136), (1, -1.5, 100, 70)])
def test_raster_forward(lib, U, oracle, views, scale_mu, w, h):
    cfg, sp, vm, K = scene(n=15000, w=w, h=h, views=views, scale_mu=scale_mu)
    ch = _chain(oracle, cfg, sp, vm, K)
    W, H = cfg.width, cfg.height
    rec = U.pack_screen(lib, ch["proj"])
    M = ch["sorted_vals"].size
    n_dev = torch.tensor([M], dtype=torch.int64, device=U.DEV)
    got = U.raster_fwd(lib, rec, U.dev(ch["offsets"]), U.dev(ch["sorted_vals"]), n_dev, views, W, H)
    ref = ch["render"]
    assert ref["T"].min() < 0.5   # the scene is not trivially empty
    # 1e-4 max abs, except where a fragment sits on the alpha = 1/255 or T = 1e-4 decision
    # (exp here is ex2.approx like the reference's __expf, the oracle's is libm): such a
    # pixel moves by at most one fragment's weight, ~1/255, and there are few of them
    d_rgb = np.abs(got["rgb"].cpu().numpy() - ref["rgb"])
    d_T = np.abs(got["T"].cpu().numpy() - ref["T"])
    assert d_rgb.max() <= 5e-3 and (d_rgb.max(axis=1) > 1e-4).mean() <= 1e-3
    assert d_T.max() <= 5e-3 and (d_T > 1e-4).mean() <= 1e-3
    assert U.close_frac(got["depth"].cpu().numpy(), ref["depth"], 1e-3, 1e-4) <= 1e-3
    assert (got["last_ids"].cpu().numpy() != ref["last_ids"]).mean() <= 1e-3


@pytest.mark.parametrize("views,scale_mu,w,h", [(1, -3.2, 320, 240), (2, -2.6, 200, 136), (1, -1.5, 100, 70)])
def test_raster_backward(lib, U, oracle, views, scale_mu, w, h):
    cfg, sp, vm, K = scene(n=15000, w=w, h=h, views=views, scale_mu=scale_mu)
    ch = _chain(oracle, cfg, sp, vm, K)
    W, H, n = cfg.width, cfg.height, cfg.n_splats
    rng = np.random.default_rng(5)
    P = views * H * W
    v_rgb = rng.normal(size=(P, 3)).astype(np.float32)
    v_depth = (0.1 * rng.normal(size=P)).astype(np.float32)
    v_T = (0.1 * rng.normal(size=P)).astype(np.float32)
    ref = oracle.raster_bwd(ch["proj"], ch["offsets"], ch["sorted_vals"], views, n, W, H, ch["render"], v_rgb, v_depth, v_T)
    rec = U.pack_screen(lib, ch["proj"])
    M = ch["sorted_vals"].size
    n_dev = torch.tensor([M], dtype=torch.int64, device=U.DEV)
    render = {k: U.dev(v) for k, v in ch["render"].items()}
    v_rec = U.raster_bwd(lib, rec, U.dev(ch["offsets"]), U.dev(ch["sorted_vals"]), n_dev, views, W, H, render, U.dev(v_rgb), U.dev(v_depth),
                         U.dev(v_T), pairs=views * n)
    got = U.vrec_to_arrays(v_rec, views * n)
    for k in ref:
        scale = np.abs(ref[k]).max()
        assert U.close_frac(got[k], ref[k], 2e-5 * scale, 1e-3) <= 2e-3, k
