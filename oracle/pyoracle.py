"""numpy/ctypes front end of the CPU oracle (oracle/ssb_oracle.cpp).

TEST INFRASTRUCTURE: imported only by tests/, __graft_entry__.smoke() and the
CPU-baseline legs of bench.py.  The shipped library never loads it.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libssb_oracle.so")
_lib = None

f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")


def build():
    subprocess.check_call(["make", "-C", _HERE, "-s"])


def load():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        _lib = C.CDLL(_SO)
        _lib.oracle_tile_count.restype = C.c_int64
        _lib.oracle_tile_count_live.restype = C.c_int64
        _lib.oracle_num_threads.restype = C.c_int
        _lib.oracle_tile_n_bits.restype = C.c_int
        _lib.oracle_det_logf.restype = C.c_float
        _lib.oracle_det_logf.argtypes = [C.c_float]
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _f(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float32)


def num_threads():
    return load().oracle_num_threads()


def set_num_threads(n):
    load().oracle_set_num_threads(C.c_int(n))


def tile_grid(W, H):
    return (W + 15) // 16, (H + 15) // 16


def _sh_args(splats, shq):
    if shq is None:
        return _p(splats["features_sh"]), None, None, C.c_int(32), C.c_int64(256)
    return None, _p(shq["packed"]), _p(shq["bounds"]), C.c_int(shq["bits"]), C.c_int64(shq.get("bounds_stride", 256))


def _dist_args(dist, dist_coeffs, n_views):
    """(tier, pointer to [C][8] float32 rows or NULL); the array is returned too so that it outlives the call."""
    if not dist:
        return 0, None, None
    rows = np.zeros((n_views, 8), np.float32)
    if dist_coeffs is not None:
        rows[:] = np.asarray(dist_coeffs, np.float32).reshape(-1, 8)
    return int(dist), _p(rows), rows


def project_fwd(splats, viewmats, intrins, W, H, model=0, antialiased=0, shq=None, with_radii=True, dist=0, dist_coeffs=None, sh_degree=3):
    """dist: lens distortion tier (0 none, 1 OpenCV, 2 thin prism, 3 rational) with dist_coeffs [C][8]."""
    lib = load()
    s = {k: _f(v) for k, v in splats.items() if v is not None}
    N, Cn = s["means"].shape[0], viewmats.shape[0]
    viewmats, intrins = _f(viewmats), _f(intrins)
    out = dict(aabb=np.zeros((Cn * N, 4), np.float32), depths=np.zeros(Cn * N, np.float32),
               radii=np.zeros(N, np.float32) if with_radii else None,
               xy=np.zeros((Cn * N, 2), np.float32), depth=np.zeros(Cn * N, np.float32),
               conic=np.zeros((Cn * N, 3), np.float32), opac=np.zeros(Cn * N, np.float32), rgb=np.zeros((Cn * N, 3), np.float32))
    sh = _sh_args(s, shq)
    tier, d_ptr, _keep = _dist_args(dist, dist_coeffs, Cn)
    lib.oracle_project_fwd_dist(C.c_int64(N), C.c_int(Cn), C.c_int(W), C.c_int(H), C.c_int(model), C.c_int(tier), d_ptr, C.c_int(sh_degree), C.c_int(antialiased),
                           _p(s["means"]), _p(s["quats"]), _p(s["scales"]), _p(s["opacities"]), _p(s["features_dc"]), *sh,
                           _p(viewmats), _p(intrins), _p(out["aabb"]), _p(out["depths"]), _p(out["radii"]),
                           _p(out["xy"]), _p(out["depth"]), _p(out["conic"]), _p(out["opac"]), _p(out["rgb"]))
    return out


def project_bwd(splats, viewmats, intrins, W, H, aabb, v, model=0, antialiased=0, shq=None, dist=0, dist_coeffs=None, sh_degree=3):
    """v: dict of v_xy, v_depth, v_conic, v_opac, v_rgb. Returns dict of world gradients."""
    lib = load()
    s = {k: _f(val) for k, val in splats.items() if val is not None}
    N, Cn = s["means"].shape[0], viewmats.shape[0]
    viewmats, intrins = _f(viewmats), _f(intrins)
    g = dict(means=np.zeros((N, 3), np.float32), quats=np.zeros((N, 4), np.float32), scales=np.zeros((N, 3), np.float32),
             opacities=np.zeros(N, np.float32), features_dc=np.zeros((N, 3), np.float32), features_sh=np.zeros((N, 15, 3), np.float32))
    vv = {k: _f(x) for k, x in v.items()}
    sh = _sh_args(s, shq)
    tier, d_ptr, _keep = _dist_args(dist, dist_coeffs, Cn)
    lib.oracle_project_bwd_dist(C.c_int64(N), C.c_int(Cn), C.c_int(W), C.c_int(H), C.c_int(model), C.c_int(tier), d_ptr, C.c_int(sh_degree), C.c_int(antialiased),
                           _p(s["means"]), _p(s["quats"]), _p(s["scales"]), _p(s["opacities"]), _p(s["features_dc"]), *sh,
                           _p(viewmats), _p(intrins), _p(_f(aabb)),
                           _p(vv["v_xy"]), _p(vv["v_depth"]), _p(vv["v_conic"]), _p(vv["v_opac"]), _p(vv["v_rgb"]),
                           _p(g["means"]), _p(g["quats"]), _p(g["scales"]), _p(g["opacities"]), _p(g["features_dc"]), _p(g["features_sh"]))
    return g


def tile_keys(proj, N, W, H, tile_active=None):
    """proj: output of project_fwd. Returns counts, cum, keys, flatten ids (unsorted).  tile_active: int32 [I, th, tw] live-tile map."""
    lib = load()
    total = proj["depths"].shape[0]
    counts = np.zeros(total, np.int64)
    cum = np.zeros(total, np.int64)
    live = None if tile_active is None else np.ascontiguousarray(tile_active, dtype=np.int32)
    M = lib.oracle_tile_count_live(C.c_int64(total), C.c_int64(N), C.c_int(W), C.c_int(H), _p(proj["aabb"]), _p(proj["xy"]), _p(proj["conic"]),
                                   _p(proj["opac"]), _p(live), _p(counts), _p(cum))
    keys = np.zeros(M, np.int64)
    vals = np.zeros(M, np.int32)
    lib.oracle_tile_emit_live(C.c_int64(total), C.c_int64(N), C.c_int(W), C.c_int(H), _p(proj["aabb"]), _p(proj["depths"]),
                              _p(proj["xy"]), _p(proj["conic"]), _p(proj["opac"]), _p(live), _p(cum), _p(keys), _p(vals))
    return counts, cum, keys, vals


def tile_active(mask, W, H):
    """Live-tile map int32 [I, th, tw] of a mask uint8 [I, Hm, Wm] (nonzero = the pixel takes part) for W x H images."""
    lib = load()
    mask = np.ascontiguousarray(mask, dtype=np.uint8)
    I, Hm, Wm = mask.shape
    out = np.zeros((I, (H + 15) // 16, (W + 15) // 16), np.int32)
    lib.oracle_tile_active(_p(mask), C.c_int(I), C.c_int(Hm), C.c_int(Wm), C.c_int(W), C.c_int(H), _p(out))
    return out


def sort_pairs(keys, vals, begin_bit, end_bit):
    lib = load()
    n = keys.shape[0]
    ko, vo = np.zeros(n, np.int64), np.zeros(n, np.int32)
    lib.oracle_sort_pairs(C.c_int64(n), C.c_int(begin_bit), C.c_int(end_bit), _p(np.ascontiguousarray(keys)),
                          _p(np.ascontiguousarray(vals)), _p(ko), _p(vo))
    return ko, vo


def tile_n_bits(n_tiles):
    return load().oracle_tile_n_bits(C.c_int(n_tiles))


def tile_offsets(sorted_keys, n_tiles_total):
    lib = load()
    offs = np.zeros(n_tiles_total, np.int32)
    lib.oracle_tile_offsets(C.c_int64(sorted_keys.shape[0]), _p(np.ascontiguousarray(sorted_keys)), C.c_int64(n_tiles_total), _p(offs))
    return offs


def raster_fwd(proj, offsets, flatten_ids, I, N, W, H):
    lib = load()
    P = I * H * W
    out = dict(rgb=np.zeros((P, 3), np.float32), depth=np.zeros(P, np.float32), T=np.zeros(P, np.float32), last_ids=np.zeros(P, np.int32))
    lib.oracle_raster_fwd(C.c_int(I), C.c_int64(N), C.c_int(W), C.c_int(H), C.c_int64(flatten_ids.shape[0]),
                          _p(proj["xy"]), _p(proj["depth"]), _p(proj["conic"]), _p(proj["opac"]), _p(proj["rgb"]),
                          _p(offsets), _p(flatten_ids), _p(out["rgb"]), _p(out["depth"]), _p(out["T"]), _p(out["last_ids"]))
    return out


def raster_bwd(proj, offsets, flatten_ids, I, N, W, H, render, v_rgb, v_depth=None, v_T=None):
    lib = load()
    total = proj["depths"].shape[0]
    g = dict(v_xy=np.zeros((total, 2), np.float32), v_depth=np.zeros(total, np.float32), v_conic=np.zeros((total, 3), np.float32),
             v_opac=np.zeros(total, np.float32), v_rgb=np.zeros((total, 3), np.float32))
    lib.oracle_raster_bwd(C.c_int(I), C.c_int64(N), C.c_int(W), C.c_int(H), C.c_int64(flatten_ids.shape[0]),
                          _p(proj["xy"]), _p(proj["depth"]), _p(proj["conic"]), _p(proj["opac"]), _p(proj["rgb"]),
                          _p(offsets), _p(flatten_ids), _p(render["depth"]), _p(render["T"]), _p(render["last_ids"]),
                          _p(_f(v_rgb)), _p(_f(v_depth)), _p(_f(v_T)),
                          _p(g["v_xy"]), _p(g["v_depth"]), _p(g["v_conic"]), _p(g["v_opac"]), _p(g["v_rgb"]))
    return g


def raster_accum_weight(proj, offsets, flatten_ids, I, N, W, H, render, weight_map, mode):
    """Per-splat densification weight of the backward walk: mode 1 max, 2 sum, 3 average (returns sum and denominator)."""
    acc, den = np.zeros(N, np.float32), np.zeros(N, np.float32)
    load().oracle_raster_accum_weight(C.c_int(I), C.c_int64(N), C.c_int(W), C.c_int(H), C.c_int64(flatten_ids.shape[0]), C.c_int(mode),
                                      _p(proj["xy"]), _p(proj["conic"]), _p(proj["opac"]), _p(offsets), _p(flatten_ids),
                                      _p(render["T"]), _p(render["last_ids"]), _p(_f(weight_map)), _p(acc), _p(den))
    return acc, den


def loss_l1_ssim(render, gt, B, H, W, w_l1=0.8, w_ssim=0.2):
    lib = load()
    v = np.zeros((B * H * W, 3), np.float32)
    losses = np.zeros(3, np.float32)
    lib.oracle_loss_l1_ssim(C.c_int(B), C.c_int(H), C.c_int(W), C.c_float(w_l1), C.c_float(w_ssim), _p(_f(render)), _p(_f(gt)), _p(v), _p(losses))
    return v, losses


def loss_l1_ssim_map(render, gt, B, H, W, mode, weight, loss_map, w_l1=0.8, w_ssim=0.2):
    """loss_l1_ssim that also adds weight * (1 - mean SSIM variant) into loss_map [B*H*W] (float32, in place)."""
    lib = load()
    v = np.zeros((B * H * W, 3), np.float32)
    losses = np.zeros(3, np.float32)
    lib.oracle_loss_l1_ssim_map(C.c_int(B), C.c_int(H), C.c_int(W), C.c_float(w_l1), C.c_float(w_ssim), _p(_f(render)), _p(_f(gt)), _p(v), _p(losses),
                                C.c_int(mode), C.c_float(weight), _p(loss_map))
    return v, losses


def loss_l1_ssim_masked(render, gt, B, H, W, mask=None, map_mode=0, map_weight=0.0, map_l1=False, loss_map=None, w_l1=0.8, w_ssim=0.2):
    """One level with a mask (uint8 [Bm, Hm, Wm], nonzero = takes part) and the loss-map variants; loss_map is added to in place."""
    lib = load()
    v = np.zeros((B * H * W, 3), np.float32)
    losses = np.zeros(3, np.float32)
    if mask is not None:
        mask = np.ascontiguousarray(mask, dtype=np.uint8)
        Bm, Hm, Wm = mask.shape
    else:
        Bm = Hm = Wm = 0
    lib.oracle_loss_l1_ssim_masked(C.c_int(B), C.c_int(H), C.c_int(W), C.c_float(w_l1), C.c_float(w_ssim), _p(_f(render)), _p(_f(gt)),
                                   _p(mask) if mask is not None else None, C.c_int(Bm), C.c_int(Hm), C.c_int(Wm), _p(v), _p(losses),
                                   C.c_int(map_mode), C.c_float(map_weight), C.c_int(int(map_l1)), _p(loss_map) if loss_map is not None else None)
    return v, losses


def loss_multi_scale(render, gt, B, H, W, num_scales, mask=None, loss_map_mode=0, w_l1=0.8, w_ssim=0.2):
    """The multi-scale loss; returns (v_render [B*H*W, 3], losses[3], loss_map [B*H*W] or None)."""
    lib = load()
    v = np.zeros((B * H * W, 3), np.float32)
    losses = np.zeros(3, np.float32)
    loss_map = np.zeros(B * H * W, np.float32) if loss_map_mode else None
    Hm = Wm = 0
    if mask is not None:
        mask = np.ascontiguousarray(mask, dtype=np.uint8)
        assert mask.shape[0] == B
        Hm, Wm = mask.shape[1:]
    lib.oracle_loss_multi_scale(C.c_int(B), C.c_int(H), C.c_int(W), C.c_int(num_scales), C.c_float(w_l1), C.c_float(w_ssim), _p(_f(render)),
                                _p(_f(gt)), _p(mask) if mask is not None else None, C.c_int(Hm), C.c_int(Wm), _p(v), _p(losses),
                                C.c_int(loss_map_mode), _p(loss_map) if loss_map is not None else None)
    return v, losses, loss_map


def quantile_positive(x, q, stride=1):
    lib = load()
    lib.oracle_quantile_positive.restype = C.c_float
    x = np.ascontiguousarray(x, dtype=np.float32)
    return float(lib.oracle_quantile_positive(_p(x), C.c_int64(x.size // stride), C.c_int64(stride), C.c_float(q)))


def densify_update_scores(radii, log_scales, accum_buffer, accum_weight=None, accum_den=None, world_grad=None, logit_opacs=None, sample_score=None,
                          max_screen_size=np.inf, clip_hardness=np.inf, max_world_size=np.inf, accum_mode=1, score_mode=0, blend_w=0.0,
                          score_power=1.0, clip_quantile=1.0, final_power=1.0):
    """In place on log_scales [n, 3], accum_weight [n], accum_buffer [n, 2] (may be None) and sample_score [n, 2] (may be None)."""
    lib = load()
    n = radii.shape[0]
    lib.oracle_densify_update_scores(C.c_int64(n), C.c_float(max_screen_size), C.c_float(clip_hardness), C.c_float(max_world_size), C.c_int(accum_mode),
                                     C.c_int(score_mode), C.c_float(blend_w), C.c_float(score_power), C.c_float(clip_quantile), C.c_float(final_power),
                                     _p(radii), _p(log_scales), _p(logit_opacs), _p(accum_weight), _p(accum_den), _p(world_grad), _p(accum_buffer),
                                     _p(sample_score))


def densify_add_noise(means, log_scales, quats, logit_opacs, scaler, revised, radii=None):
    """In place on means [n, 3]; returns the unit normals [n, 3] that were drawn."""
    lib = load()
    n = means.shape[0]
    z = np.zeros((n, 3), np.float32)
    lib.oracle_densify_add_noise(C.c_int64(n), C.c_float(scaler), C.c_int(int(revised)), _p(radii), _p(means), _p(log_scales), _p(quats), _p(logit_opacs),
                                 _p(z))
    return z


def weighted_sample(weights, seed, k, alive=None):
    """Indices of the k smallest Efraimidis-Spirakis keys; weights [n, 2] float32 (score in lane 0)."""
    lib = load()
    n = weights.shape[0]
    out = np.zeros(k, np.int32)
    lib.oracle_weighted_sample(C.c_int64(n), C.c_uint32(seed), _p(_f(weights)), _p(alive), C.c_int64(k), _p(out))
    return out


def densify_split(mode, st, cur_n, seed, split_k, min_opacity=0.005, num_new=0):
    """mode 0: relocate the dead splats of st (dict of numpy arrays, changed in place); mode 1: add num_new splats.
    st: means, quats, scales, opacities, features_dc, features_sh (or None), m1_*/m2_* (or None), accum [cap, 2], weights [cap, 2],
    optional steps, sh_optim_packed/bounds/bits, sh_value_packed/bounds/bits.  Returns (src indices, dst indices)."""
    lib = load()
    lib.oracle_densify_split.restype = C.c_int64
    cap = st["means"].shape[0]
    src = np.zeros(cap, np.int32); dst = np.zeros(cap, np.int32)
    attrs = ("means", "quats", "scales", "opacities", "features_dc", "features_sh")
    args = [C.c_int(mode), C.c_int64(cur_n), C.c_int64(num_new), C.c_float(min_opacity), C.c_float(split_k), C.c_uint32(seed), _p(st["weights"])]
    args += [_p(st.get(a)) for a in attrs]
    args += [_p(st.get("m1_" + a)) for a in attrs] + [_p(st.get("m2_" + a)) for a in attrs]
    args += [_p(st.get("sh_optim_packed")), _p(st.get("sh_optim_bounds")), C.c_int(st.get("sh_optim_bits", 0)),
             _p(st.get("sh_value_packed")), _p(st.get("sh_value_bounds")), C.c_int(st.get("sh_value_bits", 32)),
             _p(st.get("accum")), _p(st.get("steps")), _p(src), _p(dst)]
    k = lib.oracle_densify_split(*args)
    return src[:k].copy(), dst[:k].copy()


def adam_geometry(p, g, m1, m2, step, lrs, grad_scale=1.0, zero_grad=0):
    """In place on the numpy arrays of p, g, m1, m2 (dicts with means, quats, scales, opacities)."""
    lib = load()
    N = p["means"].shape[0]
    lib.oracle_adam_geometry(C.c_int64(N), C.c_int(step), C.c_float(grad_scale), C.c_int(zero_grad),
                             C.c_float(lrs["lr_means"]), C.c_float(lrs["lr_quats"]), C.c_float(lrs["lr_scales"]), C.c_float(lrs["lr_opacities"]),
                             _p(p["means"]), _p(g["means"]), _p(m1["means"]), _p(m2["means"]),
                             _p(p["quats"]), _p(g["quats"]), _p(m1["quats"]), _p(m2["quats"]),
                             _p(p["scales"]), _p(g["scales"]), _p(m1["scales"]), _p(m2["scales"]),
                             _p(p["opacities"]), _p(g["opacities"]), _p(m1["opacities"]), _p(m2["opacities"]))


def adam_geometry_ex(p, g, m1, m2, step, lrs, grad_scale=1.0, zero_grad=0, reg=None, scale_agnostic=False, radii=None, steps=None,
                     densify_score=None):
    """adam_geometry with the optional parts: reg = the seven regulariser numbers (max_gauss_ratio, scale_regularization,
    mcmc_opacity, mcmc_scale, erank, erank_s3, quat_norm; undivided weights), the scale-agnostic mean update (needs radii)
    and per-splat int32 step counters."""
    lib = load()
    N = p["means"].shape[0]
    reg_a = None if reg is None else np.ascontiguousarray(reg, np.float32)
    lib.oracle_adam_geometry_ex(C.c_int64(N), C.c_int(step), C.c_float(grad_scale), C.c_int(zero_grad),
                                C.c_float(lrs["lr_means"]), C.c_float(lrs["lr_quats"]), C.c_float(lrs["lr_scales"]), C.c_float(lrs["lr_opacities"]),
                                _p(p["means"]), _p(g["means"]), _p(m1["means"]), _p(m2["means"]),
                                _p(p["quats"]), _p(g["quats"]), _p(m1["quats"]), _p(m2["quats"]),
                                _p(p["scales"]), _p(g["scales"]), _p(m1["scales"]), _p(m2["scales"]),
                                _p(p["opacities"]), _p(g["opacities"]), _p(m1["opacities"]), _p(m2["opacities"]),
                                _p(reg_a) if reg_a is not None else None, C.c_int(1 if scale_agnostic else 0),
                                _p(radii) if radii is not None else None, _p(steps) if steps is not None else None,
                                _p(densify_score) if densify_score is not None else None)


def adam_plain(param, grad, m1, m2, step, lr, l2_reg=0.0, l2_reg_offset=0.0, grad_scale=1.0, zero_grad=0, steps=None, stride=1):
    load().oracle_adam_plain_steps(C.c_int64(param.size), C.c_int(step), C.c_float(lr), C.c_float(l2_reg), C.c_float(l2_reg_offset),
                                   C.c_float(grad_scale), C.c_int(zero_grad), _p(param), _p(grad), _p(m1), _p(m2),
                                   _p(steps) if steps is not None else None, C.c_int(stride))


Q16_ATTRS = (("means", 3), ("quats", 4), ("scales", 3), ("opacities", 1), ("features_dc", 3))
_EPS = np.float32(1e-15)


def q16_decode(packed, bounds, n, width):
    """Moments (g1, g2) [n, width] from the 16-bit joint codes of QuantizedAdamState<16, 256> with one float4 of bounds per 256
    splats (src/core/Tensor.h:1034-1068): packed uint16 [n * width, 2] = (u, log-s) codes."""
    codes = packed.view(np.uint16).reshape(n * width, 2).astype(np.float32)
    mm = np.repeat(bounds.reshape(-1, 4), 256 * width, axis=0)[: n * width].astype(np.float32)
    inv = np.float32(1.0 / 65535.0)
    u = mm[:, 0] + (mm[:, 1] - mm[:, 0]) * (codes[:, 0] * inv)
    ls = mm[:, 2] + (mm[:, 3] - mm[:, 2]) * (codes[:, 1] * inv)
    sq = _EPS * np.expm1(ls)
    return (u * (sq + _EPS)).reshape(n, width).astype(np.float32), (sq * sq).reshape(n, width).astype(np.float32)


def q16_encode(g1, g2):
    """Codes and bounds of moments [n, width]: bounds = per block of 256 splats the min / max of u and of log-s (:1070-1135)."""
    n, width = g1.shape
    sq = np.sqrt(np.maximum(g2.reshape(-1), 0)).astype(np.float32)
    u = (g1.reshape(-1) / (sq + _EPS)).astype(np.float32)
    ls = np.log1p(sq * np.float32(1e15)).astype(np.float32)
    blocks = (n + 255) // 256
    bounds = np.zeros((blocks, 4), np.float32)
    codes = np.zeros((n * width, 2), np.uint16)
    for b in range(blocks):
        sl = slice(b * 256 * width, min(n, (b + 1) * 256) * width)
        bounds[b] = (u[sl].min(), u[sl].max(), ls[sl].min(), ls[sl].max())
        ur, sr = max(bounds[b, 1] - bounds[b, 0], _EPS), max(bounds[b, 3] - bounds[b, 2], _EPS)
        codes[sl, 0] = np.clip(np.round(np.float32(65535.0) * (u[sl] - bounds[b, 0]) / ur), 0, 65535)
        codes[sl, 1] = np.clip(np.round(np.float32(65535.0) * (ls[sl] - bounds[b, 2]) / sr), 0, 65535)
    return codes.view(np.uint8).reshape(-1).copy(), bounds.reshape(-1)


def adam_geometry_q16(p, g, q, step, lrs, sh_reg_weight=0.0, grad_scale=1.0, zero_grad=0, reg=None, scale_agnostic=False, radii=None, steps=None):
    """The geometry + DC update with 16-bit moments: q = {attr: (packed, bounds)} is decoded, the fp32 update runs, q is re-encoded
    (non_sh_quant path, src/kernels/optim/FusedGeometryOptim.cu:144-380; DC regulariser = sh_reg_weight undivided, :343-345)."""
    n = p["means"].shape[0]
    m1, m2 = {}, {}
    for a, w in Q16_ATTRS:
        m1[a], m2[a] = q16_decode(q[a][0], q[a][1], n, w)
        if w == 1:
            m1[a], m2[a] = m1[a].reshape(-1), m2[a].reshape(-1)
    if reg is not None or scale_agnostic or steps is not None:
        adam_geometry_ex(p, g, m1, m2, step, lrs, grad_scale, zero_grad, reg=reg, scale_agnostic=scale_agnostic, radii=radii, steps=steps)
    else:
        adam_geometry(p, g, m1, m2, step, lrs, grad_scale, zero_grad)
    numel = n * 3
    adam_plain(p["features_dc"], g["features_dc"], m1["features_dc"], m2["features_dc"], step, lrs["lr_features_dc"],
               l2_reg=sh_reg_weight * numel / 2.0, l2_reg_offset=0.5 / 0.28209479177387814, grad_scale=grad_scale, zero_grad=zero_grad,
               steps=steps, stride=3)
    for a, w in Q16_ATTRS:
        q[a] = q16_encode(m1[a].reshape(n, w), m2[a].reshape(n, w))


def quant_encode(values, bits):
    values = _f(values).reshape(-1)
    n = values.size
    packed = np.zeros(n * (2 if bits == 16 else 1), np.uint8)
    bounds = np.zeros(((n + 255) // 256) * 2, np.float32)
    load().oracle_quant_encode(C.c_int64(n), C.c_int(bits), _p(values), _p(packed), _p(bounds))
    return packed, bounds


def quant_decode(packed, bounds, n, bits):
    out = np.zeros(n, np.float32)
    load().oracle_quant_decode(C.c_int64(n), C.c_int(bits), _p(packed), _p(bounds), _p(out))
    return out


def adam_qq(grad, optim_packed, optim_bounds, value_packed, value_bounds, value_bits, step, lr, l2_reg=0.0, grad_scale=1.0, zero_grad=0,
            steps=None, stride=1, optim_bits=8):
    """optim_bits = 4: optim_packed holds one byte per cell instead of two."""
    load().oracle_adam_qq_ex(C.c_int64(grad.size), C.c_int(step), C.c_float(lr), C.c_float(l2_reg), C.c_float(0.0), C.c_float(grad_scale),
                                C.c_int(zero_grad), C.c_int(value_bits), _p(grad), _p(optim_packed), _p(optim_bounds), _p(value_packed),
                                _p(value_bounds), _p(steps) if steps is not None else None, C.c_int(stride), C.c_int(optim_bits))


def adam_sh_splat_blocks(grad, optim_packed, optim_bounds, value_packed, value_bounds, value_bits, n_splats, step, lr, l2_reg=0.0,
                         grad_scale=1.0, sh_degree=3, steps=None):
    """SH Adam on the layouts of the reference's fused backward + optimiser at quantisation level 1: bounds per 256 splats."""
    load().oracle_adam_sh_splat_blocks(C.c_int64(n_splats), C.c_int(3 * sh_degree * (sh_degree + 2)), C.c_int(step), C.c_float(lr), C.c_float(l2_reg),
                                       C.c_float(grad_scale), C.c_int(value_bits), _p(grad), _p(optim_packed), _p(optim_bounds), _p(value_packed),
                                       _p(value_bounds), _p(steps) if steps is not None else None)


def forward_chain(splats, viewmats, intrins, W, H, shq=None, model=0, dist=0, dist_coeffs=None, sh_degree=3):
    """projection -> keys -> sort -> ranges -> raster for all views in one batch (as the reference's batched launch)."""
    N, I = splats["means"].shape[0], viewmats.shape[0]
    proj = project_fwd(splats, viewmats, intrins, W, H, shq=shq, model=model, dist=dist, dist_coeffs=dist_coeffs, sh_degree=sh_degree)
    counts, cum, keys, vals = tile_keys(proj, N, W, H)
    tw, th = tile_grid(W, H)
    nb = tile_n_bits(tw * th * I)
    sk, sv = sort_pairs(keys, vals, 0, 32 + nb)
    offs = tile_offsets(sk, tw * th * I)
    render = raster_fwd(proj, offs, sv, I, N, W, H)
    return dict(proj=proj, counts=counts, cum=cum, keys=keys, vals=vals, sorted_keys=sk, sorted_vals=sv, offsets=offs, render=render)
