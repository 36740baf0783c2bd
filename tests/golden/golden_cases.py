"""Seeded inputs of the golden fixtures.  Imported both by make_golden.py (which
feeds them to the reference's device code on a GPU) and by the tests (which feed
them to the oracle and to the CUDA library), so the fixtures only store outputs.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from spirula_studio_b200 import scenes  # noqa: E402

CASES = {
    # two ring cameras, splats a few pixels wide, moderately deep tile lists
    "ring2": dict(seed=101, n=1200, w=96, h=64, views=2, scale_mu=-2.6, extent=1.0),
    # one camera, large overlapping splats: long lists, saturated pixels, early termination
    "dense1": dict(seed=202, n=600, w=64, h=48, views=1, scale_mu=-1.6, extent=0.7),
}


# wide field-of-view cameras: the same splat cloud seen by one equidistant fisheye camera
# (model 1, about 190 degrees across the image), one equisolid fisheye camera (model 2, r = 2 f sin(theta/2):
# about 167 degrees across the image, the direction straight behind the camera maps outside it) and one
# equirectangular camera (model 3),
# all near the middle of the cloud so splats lie in every direction, behind the camera included
WIDE_CASES = {
    "wide_fisheye": dict(seed=404, n=1500, model=1, w=96, h=96, f=29.0, scale_mu=-2.4, extent=3.0),
    "wide_equisolid": dict(seed=404, n=1500, model=2, w=96, h=96, f=36.0, scale_mu=-2.4, extent=3.0),
    "wide_equirect": dict(seed=404, n=1500, model=3, w=128, h=64, f=128 / (2 * np.pi), scale_mu=-2.4, extent=3.0),
}


def build_wide_case(name):
    """Returns (cfg, splats, viewmats[1,16], intrins[1,4], camera model)."""
    c = WIDE_CASES[name]
    cfg = scenes.scaled(scenes.CONFIGS["plumbing_50k"], n_splats=c["n"], width=c["w"], height=c["h"], n_views=1, name=name)
    cfg.log_scale_mu = c["scale_mu"]
    cfg.mean_extent = c["extent"]
    cfg.fx = cfg.fy = float(c["f"])
    sp = scenes.make_splats(cfg, seed=c["seed"])
    rng = np.random.default_rng(c["seed"] + 7)
    eye = rng.uniform(-0.4, 0.4, size=3)
    target = eye + rng.normal(size=3)
    vm = scenes.look_at(eye, target).reshape(1, 16)
    K = np.array([[cfg.fx, cfg.fy, c["w"] / 2.0, c["h"] / 2.0]], dtype=np.float32)
    return cfg, sp, vm.astype(np.float32), K, c["model"]


def build_case(name):
    if name in WIDE_CASES:
        return build_wide_case(name)[:4]
    c = CASES[name]
    cfg = scenes.scaled(scenes.CONFIGS["plumbing_50k"], n_splats=c["n"], width=c["w"], height=c["h"], n_views=c["views"], name=name)
    cfg.log_scale_mu = c["scale_mu"]
    cfg.mean_extent = c["extent"]
    if c["views"] > 1:
        cfg.rig, cfg.rig_radius = "ring", 3.0
    sp = scenes.make_splats(cfg, seed=c["seed"])
    vm, K = scenes.make_cameras(cfg, seed=c["seed"] + 7)
    return cfg, sp, vm, K


def raster_cotangents(name, n_pixels):
    rng = np.random.default_rng((CASES.get(name) or WIDE_CASES[name])["seed"] + 1)
    v_rgb = rng.normal(size=(n_pixels, 3)).astype(np.float32)
    v_depth = (0.1 * rng.normal(size=n_pixels)).astype(np.float32)
    v_T = (0.1 * rng.normal(size=n_pixels)).astype(np.float32)
    return v_rgb, v_depth, v_T


def accum_weight_map(name, n_pixels):
    """Per-pixel densification weight map (non-negative, a fifth of the pixels zero) for the raster backward accumulation."""
    rng = np.random.default_rng((CASES.get(name) or WIDE_CASES[name])["seed"] + 2)
    w = rng.random(n_pixels, dtype=np.float32)
    w[rng.random(n_pixels) < 0.2] = 0.0
    return w


# Lens distortion tiers: the (camera model, tier) pairs the reference instantiates, each on the scene of the undistorted
# fixture of the same model.  tier: 1 OpenCV (k1 k2 p1 p2), 2 thin prism (k1 k2 k3 k4 p1 p2 sx1 sy1), 3 rational
# (k1 k2 k3 k4 k5 k6 p1 p2).  Coefficients are strong enough that part of the image fails the reference's validity test
# of the distortion map, and each view gets its own row.
DIST_CASES = {
    "pinhole_opencv": dict(scene="ring2", model=0, tier=1, coeffs=[-1.5, 0.3, 0.004, -0.003, 0, 0, 0, 0]),     # strong barrel: folds at the edges
    "pinhole_thinprism": dict(scene="ring2", model=0, tier=2, coeffs=[0.12, -0.03, 0.01, -0.002, 0.003, -0.002, 0.004, -0.003]),
    "pinhole_rational": dict(scene="ring2", model=0, tier=3, coeffs=[2.5, 0.5, 0.006, 0.3, 0.01, -0.002, 0.003, -0.002]),
    "fisheye_opencv": dict(scene="wide_fisheye", model=1, tier=1, coeffs=[0.04, -0.006, 0.003, -0.002, 0, 0, 0, 0]),
    "fisheye_thinprism": dict(scene="wide_fisheye", model=1, tier=2, coeffs=[0.03, -0.004, 0.0006, -0.00005, 0.002, -0.003, 0.004, 0.002]),
    "equisolid_opencv": dict(scene="wide_equisolid", model=2, tier=1, coeffs=[0.05, 0.01, -0.003, 0.002, 0, 0, 0, 0]),
    "equisolid_thinprism": dict(scene="wide_equisolid", model=2, tier=2, coeffs=[-0.04, 0.01, 0.002, 0.0003, 0.003, 0.002, -0.004, 0.003]),
}


def dist_case_inputs(name):
    """(cfg, splats, viewmats, intrins, model, tier, coeffs [views][8], screen-space cotangents) of a DIST_CASES entry."""
    c = DIST_CASES[name]
    cfg, sp, vm, K = build_case(c["scene"])
    views = vm.shape[0]
    rows = np.array([c["coeffs"]] * views, np.float32)
    rows *= (1.0 - 0.25 * np.arange(views, dtype=np.float32))[:, None]      # later views: weaker lenses
    rng = np.random.default_rng(900 + sorted(DIST_CASES).index(name))
    m = views * cfg.n_splats
    v = dict(v_xy=rng.normal(size=(m, 2)).astype(np.float32), v_depth=(0.1 * rng.normal(size=m)).astype(np.float32),
             v_conic=(0.05 * rng.normal(size=(m, 3))).astype(np.float32), v_opac=rng.normal(size=m).astype(np.float32),
             v_rgb=rng.normal(size=(m, 3)).astype(np.float32))
    return cfg, sp, vm, K, c["model"], c["tier"], rows, v


# The reference's fused projection-backward + optimiser kernel (its production default), two consecutive passes on the ring2
# scene with the screen-space cotangents of that fixture: "plain" = no regulariser, a scalar step; "ex" = per-splat
# regularisers, SH regulariser, the scale-agnostic mean update and per-splat step counters.
FPBO_SCENE = "ring2"
FPBO_RUNS = {"plain": dict(reg=[10.0, 0, 0, 0, 0, 0, 0], sh_reg=0.0, agnostic=0, steps=False),
             "ex": dict(reg=[3.0, 0.7, 0.9, 1.1, 0.5, 0.3, 0.2], sh_reg=0.05, agnostic=1, steps=True)}


def fpbo_inputs(n):
    rng = np.random.default_rng(811)
    return dict(radii=rng.uniform(0.5, 40.0, size=n).astype(np.float32), steps=rng.integers(1, 50, size=n).astype(np.int32))


# The same kernel at quantisation level 1 (16-bit SH values and 8-bit SH optimiser state, one bound per 256 splats): "l1" = every
# optimiser option on, fp32 moments for the other arrays; "l1_deg1" = SH degree 1 on the 15-coefficient buffers (the warm-up:
# idle bands are written as zero); "l1_nq" = the moments of the other arrays in 16-bit codes as well (the stock configuration).
FPBO_L1_RUNS = {"l1": dict(reg=[3.0, 0.7, 0.9, 1.1, 0.5, 0.3, 0.2], sh_reg=0.05, agnostic=1, steps=True, degree=3, nq=False),
                "l1_deg1": dict(reg=[10.0, 0, 0, 0, 0, 0, 0], sh_reg=0.05, agnostic=0, steps=False, degree=1, nq=False),
                "l1_nq": dict(reg=[3.0, 0.7, 0.9, 1.1, 0.5, 0.3, 0.2], sh_reg=0.05, agnostic=1, steps=True, degree=3, nq=True)}


def encode_splat_blocks(values, bits=16):
    """values [n, 45] -> (codes uint16/uint8 [n * 45], bounds float32 [blocks, 2]): the linear min/max codec of the reference
    (QuantizedTensor<BITS>::encode_v, src/core/Tensor.h:1379-1392) with one bound per 256 splats."""
    n = values.shape[0]
    flat = values.reshape(n, -1).astype(np.float32)
    qmax = np.float32((1 << bits) - 1)
    blocks = (n + 255) // 256
    codes = np.zeros(flat.shape, np.uint16 if bits == 16 else np.uint8)
    bounds = np.zeros((blocks, 2), np.float32)
    for b in range(blocks):
        blk = flat[b * 256:(b + 1) * 256]
        lo, hi = np.float32(blk.min()), np.float32(blk.max())
        rng_ = np.maximum(hi - lo, np.float32(1e-30))
        codes[b * 256:(b + 1) * 256] = np.clip(np.round(qmax * (blk - lo) / rng_), 0, qmax).astype(codes.dtype)
        bounds[b] = (lo, hi)
    return codes.reshape(-1), bounds


def decode_splat_blocks(codes, bounds, bits=16):
    """The inverse: codes [n * 45] and bounds [blocks, 2] -> float32 [n, 45]."""
    n = codes.size // 45
    mm = np.repeat(bounds.reshape(-1, 2), 256, axis=0)[:n]
    q = codes.reshape(n, 45).astype(np.float32) * np.float32(1.0 / ((1 << bits) - 1))
    return (mm[:, :1] + (mm[:, 1:] - mm[:, :1]) * q).astype(np.float32)


def joint_state_decode(codes, bounds, cells_per_block):
    """8-bit joint optimiser-state codes (two bytes per cell: u, log-s) and float4 bounds per block of cells_per_block cells ->
    (u, log-s) float32 arrays (QuantizedAdamState<8>::decode_us, src/core/Tensor.h:1044-1066)."""
    c = codes.reshape(-1, 2).astype(np.float32) * np.float32(1.0 / 255.0)
    mm = np.repeat(bounds.reshape(-1, 4), cells_per_block, axis=0)[: c.shape[0]]
    return mm[:, 0] + (mm[:, 1] - mm[:, 0]) * c[:, 0], mm[:, 2] + (mm[:, 3] - mm[:, 2]) * c[:, 1]


def frac_beyond_quanta(a, b, ref_lo, ref_hi, levels, quanta):
    """Fraction of entries of two decoded arrays that differ by more than `quanta` steps of the reference's code grid."""
    step = np.maximum(ref_hi - ref_lo, 1e-30) / levels
    return float((np.abs(a.astype(np.float64) - b.astype(np.float64)) > quanta * step + 1e-12).mean())


def q16_moments_mismatch(have_packed, have_bounds, ref_packed, ref_bounds, n, width):
    """Fraction of cells of two 16-bit joint moment arrays (QuantizedAdamState<16, 256> with one float4 of bounds per 256 splats)
    that agree neither as moments (|d| <= 1e-4 max + 2e-3 |ref| for g1, 4e-3 for g2) nor as codes (u and log-s within three steps
    of the reference's grid).  Two implementations sum a splat's gradient in different orders: where the grid is fine (u = +-3.16
    on the first step) that moves a code by a few steps but not the moment; where it is coarse (a wide u range) it moves the
    moment by a whole step but the code by at most one."""
    def coords(packed, bounds):
        c = np.asarray(packed).view(np.uint16).reshape(n * width, 2).astype(np.float64) / 65535.0
        mm = np.repeat(np.asarray(bounds, np.float64).reshape(-1, 4), 256 * width, axis=0)[: n * width]
        return mm[:, 0] + (mm[:, 1] - mm[:, 0]) * c[:, 0], mm[:, 2] + (mm[:, 3] - mm[:, 2]) * c[:, 1], mm
    hu, hs, _ = coords(have_packed, have_bounds)
    ru, rs, mm = coords(ref_packed, ref_bounds)
    eps = 1e-15
    hq, rq = eps * np.expm1(hs), eps * np.expm1(rs)
    h1, r1, h2, r2 = hu * (hq + eps), ru * (rq + eps), hq * hq, rq * rq
    as_moments = (np.abs(h1 - r1) <= 1e-4 * np.abs(r1).max() + 2e-3 * np.abs(r1)) & (np.abs(h2 - r2) <= 1e-4 * np.abs(r2).max() + 4e-3 * np.abs(r2))
    as_codes = (np.abs(hu - ru) <= 3.0 * (mm[:, 1] - mm[:, 0]) / 65535.0 + 1e-12) & (np.abs(hs - rs) <= 3.0 * (mm[:, 3] - mm[:, 2]) / 65535.0 + 1e-12)
    return float((~(as_moments | as_codes)).mean())


ACCUM_CASES = ("ring2", "dense1")

# Quantised SH storage read by the projection (forward and backward): 8- or 16-bit codes with (min, max) bounds
# per 256 cells ("cell" layout, bounds stride 256) or per 256 splats ("splat" layout, the stride argument 0 of the
# reference = 256 * 45 cells), on the ring2 scene.  As in the reference's own projection test
# (src/backend/tests/projection_parity.cpp:160-197) codes and bounds are drawn at random: any pair is a valid input.
QUANT_SCENE = "ring2"
QUANT_CASES = {"q16_cell": (16, 256), "q16_splat": (16, 0), "q8_cell": (8, 256), "q8_splat": (8, 0)}
FPBO_STRIDE = 256 * 45


def quant_sh_inputs(tag, n_splats):
    """(codes uint8/uint16 [n*45], bounds float32 [blocks*2], bits, stride argument) of a QUANT_CASES entry."""
    bits, stride_arg = QUANT_CASES[tag]
    cells = n_splats * 45
    stride = stride_arg if stride_arg > 0 else FPBO_STRIDE
    rng = np.random.default_rng(700 + sorted(QUANT_CASES).index(tag))
    codes = rng.integers(0, 1 << bits, size=cells, dtype=np.uint16 if bits == 16 else np.uint8)
    nb = (cells + stride - 1) // stride
    lo = rng.uniform(-0.25, 0.05, size=nb).astype(np.float32)
    hi = (lo + rng.uniform(0.02, 0.4, size=nb)).astype(np.float32)
    bounds = np.stack([lo, hi], axis=1).reshape(-1).astype(np.float32)
    return codes, bounds, bits, stride_arg


def loss_inputs():
    out = {}
    for tag, (B, H, W, seed) in dict(a=(1, 48, 64, 5), b=(2, 37, 53, 6)).items():
        rng = np.random.default_rng(seed)
        out[tag] = (B, H, W, rng.random((B * H * W, 3), dtype=np.float32), rng.random((B * H * W, 3), dtype=np.float32))
    return out


LOSS_MAP_WEIGHT = 0.7


def loss_map_base(tag, n_pixels):
    """What the densification loss map holds before the SSIM term is added in place (the per-pixel loss pass writes it)."""
    return np.random.default_rng(50 + ord(tag)).random(n_pixels, dtype=np.float32)


def loss_masks(tag, B, H, W):
    """Masks for the loss fixtures (uint8, 1 = the pixel takes part): "same" has the image's size, a masked rectangle that
    reaches the border, a masked stripe and 10 % masked speckle; "half" is stored at another resolution (nearest-sampled)."""
    rng = np.random.default_rng(70 + ord(tag))
    same = (rng.random((B, H, W)) > 0.10).astype(np.uint8)
    same[:, H // 4: H // 2, W // 3:] = 0
    same[:, :, 5:8] = 0
    Hh, Wh = H // 2 + 1, W // 2
    half = (rng.random((B, Hh, Wh)) > 0.15).astype(np.uint8)
    half[:, : Hh // 3, : Wh // 2] = 0
    return dict(same=same, half=half)


LIVE_TILE_CASE = "ring2"


def tile_masks(I, H, W):
    """Masks for the live-tile fixtures (uint8, 1 = the pixel takes part): "same" masks the right half but one pixel, the top
    rows and a block whose border pixel ring stays live; "other" is a coarse mask at another resolution."""
    same = np.ones((I, H, W), np.uint8)
    same[:, :, W // 2:] = 0
    same[:, H // 2 + 3, W - 5] = 1                 # one unmasked pixel keeps its tile alive
    same[0, : H // 4, :] = 0
    same[-1, 32:64, 32:48] = 0                     # whole tiles masked, but their neighbours' pixels touch the one-pixel pad
    other = np.ones((I, 9, 13), np.uint8)
    other[:, 2:6, 3:9] = 0
    other[0, 7:, :] = 0
    return dict(same=same, other=other)


MULTI_SCALE_RUNS = (("none", 2), ("none", 3), ("same", 3), ("half", 2))     # (mask kind, levels) of loss_multi.npz


def densify_inputs(n=3000, seed=909):
    """Per-splat inputs of the densification fixtures: screen radii (a fifth unseen), log-scales, logit opacities, this
    step's raster weights (numerator and denominator), a world-gradient score and an accumulator with a few steps in it."""
    rng = np.random.default_rng(seed)
    radii = (rng.random(n) * 0.6).astype(np.float32)
    radii[rng.random(n) < 0.2] = 0.0
    out = dict(
        radii=radii,
        log_scales=(rng.standard_normal((n, 3)) * 0.6 - 3.0).astype(np.float32),
        logit_opacs=(rng.standard_normal(n) * 2.0 - 1.0).astype(np.float32),
        means=(rng.standard_normal((n, 3)) * 2.0).astype(np.float32),
        quats=rng.standard_normal((n, 4)).astype(np.float32),
        accum_weight=(rng.random(n) ** 3 * 2.0).astype(np.float32),
        accum_den=(rng.random(n) * 3.0).astype(np.float32),
        world_grad=(rng.random(n) ** 2 * 1e-3).astype(np.float32),
        accum_buffer=np.stack([rng.random(n) ** 2, rng.integers(0, 6, n)], axis=1).astype(np.float32),
    )
    out["accum_weight"][rng.random(n) < 0.1] = 0.0
    out["accum_weight"][::17] *= -1.0
    out["accum_den"][rng.random(n) < 0.1] = 0.0
    out["accum_buffer"][out["accum_buffer"][:, 1] == 0, 0] = 0.0
    return out


# (name, keyword arguments of the score update) of densify.npz
DENSIFY_SCORE_RUNS = (
    ("clip_screen", dict(max_screen_size=0.3, clip_hardness=1.5, accum=False)),
    ("clip_world", dict(max_screen_size=0.3, clip_hardness=float("inf"), max_world_size=0.06, accum=False)),
    ("mean", dict(score_mode=0, score_power=0.4)),
    ("max", dict(score_mode=1, score_power=1.0)),
    ("geom", dict(score_mode=3, score_power=0.4)),
    ("blend", dict(score_mode=0, score_power=0.4, blend_w=0.3, world=True)),
    ("world_only", dict(score_mode=0, score_power=0.4, blend_w=1.0, world=True)),
    ("by_opacity", dict(score_mode=0, score_power=0.4, weights=False)),
    ("avg", dict(score_mode=0, score_power=0.4, accum_mode=3)),
    ("clip_score", dict(score_mode=0, score_power=0.4, clip_quantile=0.9, final_power=0.5, sample=True)),
    ("sample_only", dict(score_mode=1, score_power=1.0, final_power=2.0, sample=True)),
)


DENSIFY_SPLIT = dict(cur_n=800, cap=920, num_new=40, split_k=0.6, min_opacity=0.005, seed=2 * 700)


def densify_split_inputs(quant, seed=911):
    """State of DENSIFY_SPLIT['cap'] splats for the relocation fixtures: about 6 % dead (low opacity, two with a non-finite
    parameter), scores with a tenth zero, moments that are nowhere zero, per-splat step counters; quant: q16 SH values and
    the 8-bit joint SH optimiser state (bounds per 256 cells) instead of the fp32 arrays."""
    from oracle import pyoracle as O
    cap, cur = DENSIFY_SPLIT["cap"], DENSIFY_SPLIT["cur_n"]
    rng = np.random.default_rng(seed)
    st = dict(
        means=(rng.standard_normal((cap, 3)) * 2.0).astype(np.float32), quats=rng.standard_normal((cap, 4)).astype(np.float32),
        scales=(rng.standard_normal((cap, 3)) * 0.6 - 3.0).astype(np.float32), opacities=(rng.standard_normal(cap) * 2.0 - 1.0).astype(np.float32),
        features_dc=rng.standard_normal((cap, 3)).astype(np.float32), features_sh=(rng.standard_normal((cap, 45)) * 0.1).astype(np.float32),
        accum=np.stack([rng.random(cap) ** 2, rng.integers(1, 6, cap)], axis=1).astype(np.float32),
        steps=rng.integers(1, 500, cap).astype(np.int32))
    st["opacities"][rng.random(cap) < 0.05] = -7.0
    st["means"][17, 1] = np.inf
    st["scales"][123, 0] = np.nan
    st["accum"][rng.random(cap) < 0.1, 0] = 0.0
    st["weights"] = st["accum"].copy()
    st["weights"][:, 0] = st["weights"][:, 0] ** 0.5
    for a, w in (("means", 3), ("quats", 4), ("scales", 3), ("opacities", 1), ("features_dc", 3), ("features_sh", 45)):
        shape = (cap, w) if w > 1 else (cap,)
        st["m1_" + a] = (rng.standard_normal(shape) * 1e-3 + 2e-3).astype(np.float32)
        st["m2_" + a] = (rng.random(shape) * 1e-5 + 1e-7).astype(np.float32)
    for a in ("means", "quats", "scales", "opacities", "features_dc", "features_sh", "accum", "steps", "weights"):
        st[a][cur:] = 0                                  # slots past the current count are empty
    if quant:
        packed, bounds = O.quant_encode(st["features_sh"], 16)
        st.update(sh_value_packed=packed.copy(), sh_value_bounds=bounds.copy(), sh_value_bits=16)
        blocks = (cap * 45 + 255) // 256
        ob = np.stack([-rng.random(blocks) * 3 - 0.1, rng.random(blocks) * 3 + 0.1, rng.random(blocks) * 2, rng.random(blocks) * 5 + 20], axis=1)
        ob[::5, 0] = 0.2                                 # blocks whose u range does not contain zero: the zero code saturates
        ob[::7, 2] = 0.0
        st.update(sh_optim_packed=rng.integers(0, 256, cap * 45 * 2, dtype=np.uint8), sh_optim_bounds=ob.astype(np.float32), sh_optim_bits=8)
        st["features_sh"] = st["m1_features_sh"] = st["m2_features_sh"] = None
    return st


def adam_inputs():
    n = 700
    cfg = scenes.scaled(scenes.CONFIGS["plumbing_50k"], n_splats=n)
    params = scenes.make_splats(cfg, seed=303)
    rng = np.random.default_rng(304)
    grads = [{k: (rng.normal(size=v.shape) * 1e-3).astype(np.float32) for k, v in params.items()} for _ in range(3)]
    out = dict(n=n, params=params, grads=grads, lrs=cfg.lrs, grad_scale=0.25)
    from oracle import pyoracle as O
    for bits in (16, 8):
        numel = 45 * 300 + 11
        x0 = rng.normal(0, 0.05, size=numel).astype(np.float32)
        vp, vb = O.quant_encode(x0, bits)
        nb = (numel + 255) // 256
        out[f"qq{bits}"] = dict(numel=numel, value_packed=vp, value_bounds=vb, optim_packed=np.zeros(numel * 2, np.uint8),
                                optim_bounds=np.zeros(nb * 4, np.float32),
                                grads=[(rng.normal(size=numel) * 1e-3).astype(np.float32) for _ in range(3)])
    # optimiser state quantised, values fp32 (three steps from a zero state)
    numel = 45 * 200 + 7
    out["q8"] = dict(numel=numel, x0=rng.normal(0, 0.05, size=numel).astype(np.float32),
                     grads=[(rng.normal(size=numel) * 1e-3).astype(np.float32) for _ in range(3)])
    # optional parts of the optimiser: regularisers, per-splat step counters, scale-agnostic mean
    out["ex"] = dict(reg=np.array([3.0, 0.7, 0.9, 1.1, 0.5, 0.3, 0.2], np.float32),   # max ratio, then six undivided weights
                     radii=rng.uniform(0.5, 40.0, size=n).astype(np.float32),
                     steps=rng.integers(1, 50, size=n).astype(np.int32))
    out["nq_sh_reg_weight"] = 0.05       # the DC regulariser of the run with 16-bit non-SH moments
    return out
