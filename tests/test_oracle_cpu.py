"""CPU checks of the oracle itself: its backward passes against central finite
differences of its forward passes, and its integer stages against brute-force
definitions (numpy stable argsort, searchsorted)."""
import numpy as np
import pytest

from spirula_studio_b200 import scenes


def small_scene(n=400, w=96, h=64, seed=1, scale_mu=-2.6):
    cfg = scenes.scaled(scenes.CONFIGS["plumbing_50k"], n_splats=n, width=w, height=h)
    cfg.log_scale_mu = scale_mu
    cfg.mean_extent = 0.6
    sp = scenes.make_splats(cfg, seed=seed)
    vm, K = scenes.make_cameras(cfg)
    return cfg, sp, vm, K


def test_det_logf_matches_log(oracle):
    lib = oracle.load()
    xs = np.concatenate([np.linspace(1.0, 300.0, 4000), np.logspace(-3, 6, 2000)]).astype(np.float32)
    got = np.array([lib.oracle_det_logf(float(x)) for x in xs], dtype=np.float64)
    ref = np.log(xs.astype(np.float64))
    assert np.max(np.abs(got - ref) / np.maximum(1.0, np.abs(ref))) < 3e-7


def test_sort_is_stable_on_bit_range(oracle):
    rng = np.random.default_rng(0)
    n = 5000
    keys = rng.integers(0, 1 << 45, size=n, dtype=np.int64)
    keys[::7] = keys[0]  # many ties
    vals = np.arange(n, dtype=np.int32)
    for b0, b1 in ((0, 45), (0, 32), (8, 40), (32, 45), (0, 64)):
        ko, vo = oracle.sort_pairs(keys, vals, b0, b1)
        mask = (~np.uint64(0)) if b1 - b0 >= 64 else np.uint64(((1 << (b1 - b0)) - 1) << b0)
        order = np.argsort(keys.astype(np.uint64) & mask, kind="stable")
        assert np.array_equal(vo, vals[order]) and np.array_equal(ko, keys[order])


def test_tile_offsets_definition(oracle):
    rng = np.random.default_rng(1)
    n_tiles = 97
    tiles = np.sort(rng.integers(3, 90, size=2000)).astype(np.int64)
    keys = (tiles << 32) | rng.integers(0, 1 << 32, size=tiles.size, dtype=np.int64)
    offs = oracle.tile_offsets(keys, n_tiles)
    assert np.array_equal(offs, np.searchsorted(tiles, np.arange(n_tiles), side="left").astype(np.int32))
    assert np.array_equal(oracle.tile_offsets(keys[:0], n_tiles), np.zeros(n_tiles, np.int32))


def test_tile_keys_cover_footprint(oracle):
    """Every pixel where a splat's alpha exceeds 1/255 lies in a tile the splat was binned to."""
    cfg, sp, vm, K = small_scene(n=200)
    W, H = cfg.width, cfg.height
    proj = oracle.project_fwd(sp, vm, K, W, H)
    counts, cum, keys, vals = oracle.tile_keys(proj, cfg.n_splats, W, H)
    assert cum[-1] == keys.size == counts.sum() and np.all(np.diff(cum) == counts[1:])
    tw, th = oracle.tile_grid(W, H)
    binned = set(zip(vals.tolist(), (keys >> 32).tolist()))
    ys, xs = np.mgrid[0:H, 0:W]
    px, py = xs + 0.5, ys + 0.5
    for g in range(cfg.n_splats):
        if counts[g] == 0:
            continue
        dx, dy = proj["xy"][g, 0] - px, proj["xy"][g, 1] - py
        a, b, c = proj["conic"][g]
        sigma = 0.5 * (a * dx * dx + c * dy * dy) + b * dx * dy
        alpha = np.minimum(0.999, proj["opac"][g] * np.exp(-sigma))
        hit = (alpha > 1.0 / 255.0 + 1e-6) & (sigma >= 0)
        for t in np.unique((ys[hit] // 16) * tw + xs[hit] // 16):
            assert (g, int(t)) in binned


def _proj_scalar(oracle, sp, vm, K, W, H, v, model=0):
    o = oracle.project_fwd(sp, vm, K, W, H, model=model)
    keep = o["aabb"][:, 2] > o["aabb"][:, 0]
    tot = 0.0
    for name, key in (("xy", "v_xy"), ("depth", "v_depth"), ("conic", "v_conic"), ("opac", "v_opac"), ("rgb", "v_rgb")):
        a = o[name].astype(np.float64).reshape(len(keep), -1)[keep]
        tot += float((a * v[key].astype(np.float64).reshape(len(keep), -1)[keep]).sum())
    return tot, keep


@pytest.mark.parametrize("attr", ["means", "quats", "scales", "opacities", "features_dc", "features_sh"])
def test_projection_backward_matches_finite_differences(oracle, attr):
    cfg, sp, vm, K = small_scene(n=64, w=200, h=160, seed=3)
    sp["means"] *= 0.5
    W, H = cfg.width, cfg.height
    rng = np.random.default_rng(5)
    n = cfg.n_splats
    v = dict(v_xy=rng.normal(size=(n, 2)), v_depth=rng.normal(size=n), v_conic=rng.normal(size=(n, 3)) * 0.1,
             v_opac=rng.normal(size=n), v_rgb=rng.normal(size=(n, 3)))
    v = {k: x.astype(np.float32) for k, x in v.items()}
    base = oracle.project_fwd(sp, vm, K, W, H)
    g = oracle.project_bwd(sp, vm, K, W, H, base["aabb"], v)
    d = rng.normal(size=sp[attr].shape).astype(np.float32)
    eps = 2e-3
    plus = {k: x.copy() for k, x in sp.items()}
    minus = {k: x.copy() for k, x in sp.items()}
    plus[attr] = sp[attr] + eps * d
    minus[attr] = sp[attr] - eps * d
    lp, kp = _proj_scalar(oracle, plus, vm, K, W, H, v)
    lm, km = _proj_scalar(oracle, minus, vm, K, W, H, v)
    assert np.array_equal(kp, km)
    fd = (lp - lm) / (2 * eps)
    an = float((g[attr].astype(np.float64) * d).sum())
    assert abs(fd - an) <= 2e-2 * max(1.0, abs(fd)), (fd, an)


def wide_scene(model, n=96, seed=11):
    """Camera inside the cloud: an equidistant (model 1) or equisolid (model 2) fisheye, or an equirectangular one (model 3)."""
    W, H, f = (120, 120, 36.0 if model == 1 else 40.0) if model in (1, 2) else (160, 80, 160 / (2 * np.pi))
    cfg = scenes.scaled(scenes.CONFIGS["plumbing_50k"], n_splats=n, width=W, height=H)
    cfg.log_scale_mu, cfg.mean_extent = -2.2, 2.5
    sp = scenes.make_splats(cfg, seed=seed)
    vm = scenes.look_at((0.2, -0.1, 0.15), (1.0, 0.3, 2.0)).reshape(1, 16).astype(np.float32)
    K = np.array([[f, f, W / 2.0, H / 2.0]], dtype=np.float32)
    return cfg, sp, vm, K


@pytest.mark.parametrize("model", [1, 2, 3])
@pytest.mark.parametrize("attr", ["means", "quats", "scales", "opacities"])
def test_wide_projection_backward_matches_finite_differences(oracle, model, attr):
    """Fisheye, equisolid and equirectangular cameras: the vjp against central differences of the forward pass."""
    cfg, sp, vm, K = wide_scene(model)
    W, H, n = cfg.width, cfg.height, cfg.n_splats
    rng = np.random.default_rng(6)
    v = dict(v_xy=rng.normal(size=(n, 2)), v_depth=rng.normal(size=n), v_conic=rng.normal(size=(n, 3)) * 0.1,
             v_opac=rng.normal(size=n), v_rgb=rng.normal(size=(n, 3)))
    v = {k: x.astype(np.float32) for k, x in v.items()}
    base = oracle.project_fwd(sp, vm, K, W, H, model=model)
    keep = base["aabb"][:, 2] > base["aabb"][:, 0]
    assert keep.sum() > n // 4
    g = oracle.project_bwd(sp, vm, K, W, H, base["aabb"], v, model=model)
    d = rng.normal(size=sp[attr].shape).astype(np.float32)
    eps = 1e-3
    plus = {k: x.copy() for k, x in sp.items()}
    minus = {k: x.copy() for k, x in sp.items()}
    plus[attr] = sp[attr] + eps * d
    minus[attr] = sp[attr] - eps * d
    lp, kp = _proj_scalar(oracle, plus, vm, K, W, H, v, model)
    lm, km = _proj_scalar(oracle, minus, vm, K, W, H, v, model)
    assert np.array_equal(kp, km)
    fd = (lp - lm) / (2 * eps)
    an = float((g[attr].astype(np.float64) * d).sum())
    assert abs(fd - an) <= 3e-2 * max(1.0, abs(fd)), (fd, an)


def test_wide_sorting_depth(oracle):
    """Sorting depth: squared distance (equirectangular), z^4 + (x^2+y^2)^2/512 (both fisheyes)."""
    for model in (1, 2, 3):
        cfg, sp, vm, K = wide_scene(model)
        o = oracle.project_fwd(sp, vm, K, cfg.width, cfg.height, model=model)
        keep = o["aabb"][:, 2] > o["aabb"][:, 0]
        m = vm.reshape(4, 4).astype(np.float64)
        pc = sp["means"].astype(np.float64) @ m[:3, :3].T + m[:3, 3]
        if model == 3:
            want = (pc ** 2).sum(1)
        else:
            want = pc[:, 2] ** 4 + ((pc[:, 0] ** 2 + pc[:, 1] ** 2) ** 2) / 512.0
        assert np.allclose(o["depths"][keep], want[keep], rtol=1e-4)
        assert np.allclose(o["depth"][keep], np.sqrt((pc ** 2).sum(1))[keep], rtol=1e-5)
        if model == 3:
            assert (pc[keep, 2] < 0).any()      # splats behind the camera are seen


def _frozen_blend(proj64, order, mask, W, H, v_rgb, v_depth):
    """float64 blend of one 16x16 tile with the contributing (splat, pixel) set held fixed."""
    ys, xs = np.mgrid[0:H, 0:W]
    px, py = (xs + 0.5).reshape(-1), (ys + 0.5).reshape(-1)
    T = np.ones(px.size)
    C = np.zeros((px.size, 3))
    D = np.zeros(px.size)
    for k, g in enumerate(order):
        dx, dy = proj64["xy"][g, 0] - px, proj64["xy"][g, 1] - py
        a, b, c = proj64["conic"][g]
        sigma = 0.5 * (a * dx * dx + c * dy * dy) + b * dx * dy
        alpha = np.minimum(0.999, proj64["opac"][g] * np.exp(-sigma)) * mask[k]
        w = alpha * T
        C += w[:, None] * proj64["rgb"][g][None, :]
        D += w * proj64["depth"][g]
        T = T * (1.0 - alpha)
    depth = D / np.maximum(1.0 - T, 1e-10)
    return float((C * v_rgb).sum() + (depth * v_depth).sum())


@pytest.mark.parametrize("field", ["xy", "conic", "opac", "rgb", "depth"])
def test_raster_backward_matches_finite_differences(oracle, field):
    """The render is only piecewise smooth (alpha threshold, early stop), so the set of
    contributing (splat, pixel) pairs is frozen at the base point and the smooth function
    that remains is differentiated numerically in float64."""
    cfg, sp, vm, K = small_scene(n=60, w=16, h=16, seed=7, scale_mu=-2.0)
    cfg.fx = cfg.fy = 40.0
    K[:, 0] = K[:, 1] = 40.0
    W, H = cfg.width, cfg.height
    ch = oracle.forward_chain(sp, vm, K, W, H)
    proj, offs, vals, render = ch["proj"], ch["offsets"], ch["sorted_vals"], ch["render"]
    assert vals.size > 20
    rng = np.random.default_rng(11)
    v_rgb = rng.normal(size=(H * W, 3)).astype(np.float32)
    v_depth = (rng.normal(size=H * W) * 0.1).astype(np.float32)
    g = oracle.raster_bwd(proj, offs, vals, 1, cfg.n_splats, W, H, render, v_rgb, v_depth=v_depth)
    # contributing set at the base point
    ys, xs = np.mgrid[0:H, 0:W]
    px, py = (xs + 0.5).reshape(-1), (ys + 0.5).reshape(-1)
    mask = np.zeros((vals.size, H * W))
    for k, s_id in enumerate(vals):
        dx, dy = proj["xy"][s_id, 0] - px, proj["xy"][s_id, 1] - py
        a, b, c = proj["conic"][s_id]
        sigma = 0.5 * (a * dx * dx + c * dy * dy) + b * dx * dy
        alpha = np.minimum(0.999, proj["opac"][s_id] * np.exp(-sigma))
        mask[k] = (alpha > 1.0 / 255.0) & (sigma >= 0) & (k <= render["last_ids"]) & (alpha < 0.998)
    p64 = {k: x.astype(np.float64) for k, x in proj.items() if x is not None}
    d = rng.normal(size=proj[field].shape)
    if field == "conic":
        d *= 0.01
    eps = 1e-5
    hi = dict(p64); lo = dict(p64)
    hi[field] = p64[field] + eps * d
    lo[field] = p64[field] - eps * d
    fd = (_frozen_blend(hi, vals, mask, W, H, v_rgb, v_depth) - _frozen_blend(lo, vals, mask, W, H, v_rgb, v_depth)) / (2 * eps)
    an = float((g["v_" + field].astype(np.float64) * d).sum())
    assert abs(fd - an) <= 2e-3 * max(1.0, abs(fd)), (fd, an)


def test_loss_gradient_matches_finite_differences(oracle):
    rng = np.random.default_rng(2)
    H, W = 40, 56
    render = rng.random((H * W, 3), dtype=np.float32)
    gt = rng.random((H * W, 3), dtype=np.float32)
    v, losses = oracle.loss_l1_ssim(render, gt, 1, H, W, 0.8, 0.2)
    assert 0.0 < losses[1] < 1.0 and abs(losses[2] - (0.8 * losses[0] + 0.2 * (1 - losses[1]))) < 1e-6
    # along the gradient itself, so the L1 kinks (|r-g| < eps) stay a small part of the total
    d = (v / np.abs(v).max()).astype(np.float32)
    eps = 1e-3
    lp = oracle.loss_l1_ssim(render + eps * d, gt, 1, H, W)[1][2]
    lm = oracle.loss_l1_ssim(render - eps * d, gt, 1, H, W)[1][2]
    fd = (float(lp) - float(lm)) / (2 * eps)
    an = float((v.astype(np.float64) * d).sum())
    assert abs(fd - an) <= 1e-2 * max(abs(fd), 1e-3), (fd, an)


def test_ssim_of_identical_images_is_one(oracle):
    rng = np.random.default_rng(3)
    H, W = 33, 47
    img = rng.random((H * W, 3), dtype=np.float32)
    v, losses = oracle.loss_l1_ssim(img, img.copy(), 1, H, W)
    assert abs(losses[1] - 1.0) < 1e-5 and losses[0] == 0.0
    assert np.max(np.abs(v)) < 1e-6


def test_quant_codec_roundtrip(oracle):
    rng = np.random.default_rng(4)
    x = rng.normal(0, 0.05, size=45 * 300).astype(np.float32)
    for bits in (8, 16):
        packed, bounds = oracle.quant_encode(x, bits)
        y = oracle.quant_decode(packed, bounds, x.size, bits)
        b = bounds.reshape(-1, 2)
        step = np.repeat((b[:, 1] - b[:, 0]) / ((1 << bits) - 1), 256)[: x.size]
        assert np.all(np.abs(x - y) <= 0.5 * step + 1e-7)


def test_adam_quantized_state_with_fp32_values(oracle):
    """Only the optimiser state quantised (value_bits = 32): the first step from a zero state uses this step's
    unquantised moments, so it must equal the plain fp32 Adam step; later steps differ only by the state's 8-bit error."""
    rng = np.random.default_rng(12)
    n = 256 * 7 + 19
    x0 = rng.normal(0, 0.05, size=n).astype(np.float32)
    g = (rng.normal(size=n) * 1e-3).astype(np.float32)
    xq = x0.copy()
    op, ob = np.zeros(n * 2, np.uint8), np.zeros(((n + 255) // 256) * 4, np.float32)
    oracle.adam_qq(g.copy(), op, ob, xq.view(np.uint8), np.zeros(2, np.float32), 32, 1, 2.5e-3, grad_scale=0.5)
    xp, m1, m2 = x0.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32)
    oracle.adam_plain(xp, g.copy(), m1, m2, 1, 2.5e-3, 0.0, 0.0, 0.5)
    assert np.allclose(xq, xp, rtol=0, atol=1e-7)
    g2 = (rng.normal(size=n) * 1e-3).astype(np.float32)
    oracle.adam_qq(g2.copy(), op, ob, xq.view(np.uint8), np.zeros(2, np.float32), 32, 2, 2.5e-3, grad_scale=0.5)
    oracle.adam_plain(xp, g2.copy(), m1, m2, 2, 2.5e-3, 0.0, 0.0, 0.5)
    assert np.abs(xq - xp).max() < 0.2 * 2.5e-3          # a step is at most lr; the state error moves it by a fraction


def test_adam_first_step_moves_by_lr(oracle):
    """With zero moments the first bias-corrected Adam step is lr * sign(g)."""
    rng = np.random.default_rng(6)
    n = 1000
    p = rng.normal(size=n).astype(np.float32)
    g = rng.normal(size=n).astype(np.float32)
    p0 = p.copy()
    m1, m2 = np.zeros(n, np.float32), np.zeros(n, np.float32)
    oracle.adam_plain(p, g, m1, m2, 1, 2.5e-3)
    assert np.allclose(p0 - p, 2.5e-3 * np.sign(g), rtol=1e-4, atol=1e-9)
    assert np.allclose(m1, 0.1 * g, rtol=1e-6) and np.allclose(m2, 0.001 * g * g, rtol=1e-4)


def _per_splat_losses64(s, o, q, reg):
    """Sum of the five per-splat regularisers in float64 (src/shaders/per_splat_losses.slang:5-107)."""
    max_ratio, w_ratio, w_op, w_ms, w_er, w_er3, w_qn = reg
    e = np.exp(s)
    E = np.exp(2 * s)
    p = E / E.sum()
    p1, p3 = p.max(), p.min()
    p2 = 1.0 - p1 - p3
    r = np.exp(-(p1 * np.log(p1) + p2 * np.log(p2) + p3 * np.log(p3)))
    n = np.linalg.norm(q)
    return (w_op / (1 + np.exp(-o)) + w_ms * 1e-2 * s.sum() / 3 + w_ratio * (max(e.max() / e.min(), max_ratio) - max_ratio)
            + w_er * max(-np.log(r - 0.99999), 0.0) + w_er3 * p3 + w_qn * (n - 1 - np.log(n)))


def test_adam_regulariser_gradients_match_finite_differences(oracle):
    """With zero data gradients and a zero state, the first moment after one step is 0.1 * (regulariser gradient / N)."""
    rng = np.random.default_rng(77)
    n = 64
    p = dict(means=rng.normal(size=(n, 3)).astype(np.float32), quats=rng.normal(size=(n, 4)).astype(np.float32),
             scales=rng.normal(-2.0, 0.6, size=(n, 3)).astype(np.float32), opacities=rng.normal(size=n).astype(np.float32))
    p["quats"] /= np.linalg.norm(p["quats"], axis=1, keepdims=True)
    p0 = {k: v.copy() for k, v in p.items()}
    g = {k: np.zeros_like(v) for k, v in p.items()}
    m1 = {k: np.zeros_like(v) for k, v in p.items()}
    m2 = {k: np.zeros_like(v) for k, v in p.items()}
    reg = np.array([3.0, 0.7, 0.9, 1.1, 0.5, 0.3, 0.0], np.float32)
    lrs = dict(lr_means=1e-3, lr_quats=1e-3, lr_scales=5e-3, lr_opacities=5e-2)
    oracle.adam_geometry_ex(p, g, m1, m2, 1, lrs, reg=reg)
    gs, go = m1["scales"] * 10 * n, m1["opacities"] * 10 * n
    h = 1e-5
    for i in range(n):
        s, o, q = p0["scales"][i].astype(np.float64), float(p0["opacities"][i]), p0["quats"][i].astype(np.float64)
        for k in range(3):
            d = np.zeros(3); d[k] = h
            fd = (_per_splat_losses64(s + d, o, q, reg) - _per_splat_losses64(s - d, o, q, reg)) / (2 * h)
            assert abs(gs[i, k] - fd) <= 2e-3 * max(1.0, abs(fd)), (i, k, gs[i, k], fd)
        fd = (_per_splat_losses64(s, o + h, q, reg) - _per_splat_losses64(s, o - h, q, reg)) / (2 * h)
        assert abs(go[i] - fd) <= 2e-3 * max(1.0, abs(fd))
    assert np.abs(m1["means"]).max() == 0 and np.abs(m1["quats"]).max() < 1e-7


def test_adam_extras_default_to_the_plain_step(oracle):
    """No regularisers, no scale-agnostic mean and per-splat counters all equal to the scalar step: identical updates."""
    rng = np.random.default_rng(78)
    n = 300
    mk = lambda: dict(means=rng.normal(size=(n, 3)).astype(np.float32), quats=rng.normal(size=(n, 4)).astype(np.float32),
                      scales=rng.normal(size=(n, 3)).astype(np.float32), opacities=rng.normal(size=n).astype(np.float32))
    p, g, m1, m2 = mk(), mk(), mk(), mk()
    for k in m2:
        m2[k] = np.abs(m2[k])
    a = [{k: v.copy() for k, v in d.items()} for d in (p, g, m1, m2)]
    b = [{k: v.copy() for k, v in d.items()} for d in (p, g, m1, m2)]
    lrs = dict(lr_means=1e-3, lr_quats=1e-3, lr_scales=5e-3, lr_opacities=5e-2)
    oracle.adam_geometry(*a, 7, lrs, grad_scale=0.5)
    oracle.adam_geometry_ex(*b, 3, lrs, grad_scale=0.5, steps=np.full(n, 7, np.int32))
    for da, db in zip(a, b):
        for k in da:
            assert np.array_equal(da[k], db[k]), k
    # the scale-agnostic update changes only the means and their moments
    c = [{k: v.copy() for k, v in d.items()} for d in (p, g, m1, m2)]
    oracle.adam_geometry_ex(*c, 7, lrs, grad_scale=0.5, scale_agnostic=True, radii=rng.uniform(1, 30, size=n).astype(np.float32))
    for k in ("quats", "scales", "opacities"):
        assert np.array_equal(a[0][k], c[0][k])
    assert not np.array_equal(a[0]["means"], c[0]["means"])
    # plain and quantised element-wise kernels: counters equal to the scalar step reproduce it
    x = rng.normal(size=45 * 40).astype(np.float32); gr = rng.normal(size=x.size).astype(np.float32)
    xa, xb = x.copy(), x.copy()
    ma, va, mb, vb = (np.zeros_like(x) for _ in range(4))
    oracle.adam_plain(xa, gr.copy(), ma, va, 5, 2.5e-3)
    oracle.adam_plain(xb, gr.copy(), mb, vb, 1, 2.5e-3, steps=np.full(40, 5, np.int32), stride=45)
    assert np.array_equal(xa, xb)
