"""Seeded synthetic scenes with the shapes, sizes and value distributions of the
benchmark configurations.  They stand in for the public capture datasets the
reference's own benchmark driver targets (reference/python/benchmark.py:36-55),
which cannot be shipped: only their scale is reproduced.

Everything is numpy (PCG64); callers move the arrays wherever they need them.
Camera convention: OpenCV (x right, y down, z forward), world "down" is +y,
viewmat = [R | t] row-major world-to-camera with t = -R c
(the reference reads rows 0..2 as R|t, src/kernels/projection/ProjectionFwd_kernel.cuh:52-59).
"""
from dataclasses import dataclass, field

import numpy as np

SPLAT_SEED = 20260718
TARGET_SEED = 20260719


@dataclass
class SceneConfig:
    name: str
    n_splats: int
    width: int
    height: int
    fx: float
    fy: float
    n_views: int
    mean_extent: float          # means uniform in [-extent, extent]^3
    log_scale_mu: float = -4.0
    log_scale_sigma: float = 0.5
    opacity_mu: float = 0.0
    opacity_sigma: float = 1.0
    rig: str = "ring"           # "single" | "ring" | "sphere" | "inside" (centres within rig_radius of the origin)
    mean_ball: bool = False     # means uniform in the ball of radius mean_extent instead of the cube
    camera_model: int = 0       # 0 pinhole, 1 equidistant fisheye, 3 equirectangular (src/core/Common.cuh:94-99)
    # several camera kinds in one batch: tuples (camera_model, width, height, fx, fy); view i uses
    # entry i % len(view_kinds).  Empty: every view is (camera_model, width, height, fx, fy).
    view_kinds: tuple = ()
    rig_radius: float = 8.0
    sh_value_bits: int = 32     # 16 = the reference's quantised SH storage
    sh_optim_bits: int = 32
    lrs: dict = field(default_factory=lambda: dict(
        lr_means=1e-3, lr_scales=5e-3, lr_quats=1e-3, lr_opacities=5e-2, lr_features_dc=2.5e-3, lr_features_sh=2.5e-3))


CONFIGS = {
    # small plumbing scene, one camera at (0,0,3) looking at the origin
    "plumbing_50k": SceneConfig("plumbing_50k", 50_000, 640, 480, 500.0, 500.0, 1, 1.0, rig="single", rig_radius=3.0),
    # mid scene: 1M splats, 16 views of 1920x1080 on a radius-8 ring, quantised SH
    "mid_1m": SceneConfig("mid_1m", 1_000_000, 1920, 1080, 1400.0, 1400.0, 16, 4.0, rig="ring", rig_radius=8.0,
                          sh_value_bits=16, sh_optim_bits=8),
    # dense scene: 3M small, mostly transparent splats, 32 views of 2560x1440 on a radius-6 sphere
    "dense_3m": SceneConfig("dense_3m", 3_000_000, 2560, 1440, 1866.6666, 1866.6666, 32, 4.0, log_scale_mu=-5.0,
                            log_scale_sigma=0.6, opacity_mu=-1.0, opacity_sigma=1.5, rig="sphere", rig_radius=6.0),
    # VRAM-scale scene: 10M splats, 64 views of 3840x2160 on a radius-25 ring, quantised SH
    "vram_10m": SceneConfig("vram_10m", 10_000_000, 3840, 2160, 2800.0, 2800.0, 64, 20.0, log_scale_mu=-4.5,
                            log_scale_sigma=0.7, rig="ring", rig_radius=25.0, sh_value_bits=16, sh_optim_bits=8),
    # wide field of view: 5M splats in a radius-15 ball, 16 views from within radius 2 of the origin, alternating
    # equidistant fisheye (1920x1920, f = 600, ~190 degrees) and equirectangular 360-degree (4096x2048)
    "wide_5m": SceneConfig("wide_5m", 5_000_000, 1920, 1920, 600.0, 600.0, 16, 15.0, log_scale_mu=-4.5, log_scale_sigma=0.6,
                           rig="inside", rig_radius=2.0, mean_ball=True,
                           view_kinds=((1, 1920, 1920, 600.0, 600.0), (3, 4096, 2048, 4096 / (2 * np.pi), 4096 / (2 * np.pi)))),
}


def view_kind(cfg: "SceneConfig", view: int):
    """(kind index, camera_model, width, height, fx, fy) of a view of the batch."""
    if not cfg.view_kinds:
        return 0, cfg.camera_model, cfg.width, cfg.height, cfg.fx, cfg.fy
    k = view % len(cfg.view_kinds)
    return (k,) + tuple(cfg.view_kinds[k])


def n_view_kinds(cfg: "SceneConfig"):
    return max(1, len(cfg.view_kinds))


def scaled(cfg: SceneConfig, n_splats=None, width=None, height=None, n_views=None, name=None) -> SceneConfig:
    """Same distributions at a smaller size (parity tests). Focal lengths follow the width."""
    import copy
    c = copy.deepcopy(cfg)
    if width is not None:
        s = width / cfg.width
        c.fx, c.fy, c.width = cfg.fx * s, cfg.fy * s, width
        c.height = height if height is not None else int(round(cfg.height * s))
        # every camera kind shrinks by the same factor (sizes kept even)
        c.view_kinds = tuple((m, max(2, int(round(w * s / 2)) * 2), max(2, int(round(h * s / 2)) * 2), fx * s, fy * s)
                             for m, w, h, fx, fy in cfg.view_kinds)
    elif height is not None:
        c.height = height
    if n_splats is not None:
        c.n_splats = n_splats
    if n_views is not None:
        c.n_views = n_views
    c.name = name or f"{cfg.name}_scaled"
    return c


def make_splats(cfg: SceneConfig, seed: int = SPLAT_SEED):
    rng = np.random.Generator(np.random.PCG64(seed))
    n = cfg.n_splats
    f32 = np.float32
    if cfg.mean_ball:
        d = rng.normal(size=(n, 3))
        d /= np.linalg.norm(d, axis=1, keepdims=True)
        means = (d * (cfg.mean_extent * rng.uniform(size=(n, 1)) ** (1.0 / 3.0))).astype(f32)
    else:
        means = rng.uniform(-cfg.mean_extent, cfg.mean_extent, size=(n, 3)).astype(f32)
    scales = rng.normal(cfg.log_scale_mu, cfg.log_scale_sigma, size=(n, 3)).astype(f32)
    q = rng.normal(0.0, 1.0, size=(n, 4))
    quats = (q / np.linalg.norm(q, axis=1, keepdims=True)).astype(f32)
    opacities = rng.normal(cfg.opacity_mu, cfg.opacity_sigma, size=(n,)).astype(f32)
    features_dc = rng.normal(0.0, 0.3, size=(n, 3)).astype(f32)
    features_sh = rng.normal(0.0, 0.05, size=(n, 15, 3)).astype(f32)
    return dict(means=means, quats=quats, scales=scales, opacities=opacities, features_dc=features_dc,
                features_sh=features_sh)


def look_at(eye, target=(0.0, 0.0, 0.0), down=(0.0, 1.0, 0.0)):
    eye = np.asarray(eye, dtype=np.float64)
    z = np.asarray(target, dtype=np.float64) - eye
    z /= np.linalg.norm(z)
    x = np.cross(np.asarray(down, dtype=np.float64), z)
    if np.linalg.norm(x) < 1e-8:  # looking straight along "down"
        x = np.cross(np.array([0.0, 0.0, 1.0]), z)
    x /= np.linalg.norm(x)
    y = np.cross(z, x)
    R = np.stack([x, y, z], axis=0)
    t = -R @ eye
    m = np.eye(4)
    m[:3, :3] = R
    m[:3, 3] = t
    return m.astype(np.float32)


def make_cameras(cfg: SceneConfig, seed: int = SPLAT_SEED + 7):
    rng = np.random.Generator(np.random.PCG64(seed))
    eyes = []
    if cfg.rig == "single":
        eyes = [(0.0, 0.0, cfg.rig_radius)]
    elif cfg.rig == "ring":
        hs = rng.uniform(-1.0, 1.0, size=cfg.n_views)
        for k in range(cfg.n_views):
            a = 2.0 * np.pi * k / cfg.n_views
            eyes.append((cfg.rig_radius * np.cos(a), hs[k], cfg.rig_radius * np.sin(a)))
    elif cfg.rig == "sphere":  # Fibonacci directions
        ga = np.pi * (3.0 - np.sqrt(5.0))
        for k in range(cfg.n_views):
            yy = 1.0 - 2.0 * (k + 0.5) / cfg.n_views
            r = np.sqrt(max(0.0, 1.0 - yy * yy))
            eyes.append((cfg.rig_radius * r * np.cos(ga * k), cfg.rig_radius * yy, cfg.rig_radius * r * np.sin(ga * k)))
    elif cfg.rig == "inside":  # centres uniform within rig_radius of the origin, random viewing directions
        d = rng.normal(size=(cfg.n_views, 3))
        d /= np.linalg.norm(d, axis=1, keepdims=True)
        c = d * (cfg.rig_radius * rng.uniform(size=(cfg.n_views, 1)) ** (1.0 / 3.0))
        look = rng.normal(size=(cfg.n_views, 3))
        viewmats = np.stack([look_at(c[k], c[k] + look[k]) for k in range(cfg.n_views)], axis=0).reshape(-1, 16)
    else:
        raise ValueError(cfg.rig)
    if cfg.rig != "inside":
        viewmats = np.stack([look_at(e) for e in eyes[: cfg.n_views]], axis=0).reshape(-1, 16)
    intrins = np.zeros((len(viewmats), 4), dtype=np.float32)
    for v in range(len(viewmats)):
        _, _, w, h, fx, fy = view_kind(cfg, v)
        intrins[v] = (fx, fy, w / 2.0, h / 2.0)
    return viewmats.astype(np.float32), intrins


def make_target(cfg: SceneConfig, view: int, seed: int = TARGET_SEED):
    """i.i.d. uniform [0,1] RGB target of one view, [H, W, 3] fp32."""
    rng = np.random.Generator(np.random.PCG64(seed + 1000 * view))
    _, _, w, h, _, _ = view_kind(cfg, view)
    return rng.random(size=(h, w, 3), dtype=np.float32)
