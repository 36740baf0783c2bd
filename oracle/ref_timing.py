"""TEST INFRASTRUCTURE.  Times the REFERENCE's own CUDA kernels (oracle/_ref/libssb_ref.so: the
reference's device code compiled from its sources with its own nvcc flags, behind the launch shims of
oracle/ref_tool/) stage by stage on a GPU, on the views of a benchmark scene, with this library's kernels
timed on the same inputs beside them.  It is the denominator of "how much faster than the reference's
CUDA backend": per stage, CUDA events around the launch, warm-up first, averaged over views.

    python oracle/ref_timing.py [--workload mid_1m] [--views 16] [--repeats 3] [--out file.json]

What is and is not inside a reference time:
  * projection, tile intersection (count, cub scan, keys, cub radix sort, offsets, INCLUDING the host
    read of the pair count that do_intersect_tile_generic performs; cub temp storage pre-allocated as the
    reference's grow-only scratch is), rasteriser forward and backward WITH the depth channel (the
    reference always renders and back-propagates depth), fused SSIM, projection backward, and the three
    optimiser kernels (geometry, DC, doubly quantised SH).
  * NOT inside: the reference's per-pixel loss kernel (the L1 part of the loss is formed here with a torch
    expression and not timed), its gradient zeroing between steps, and all host-side engine work.  The sum
    therefore flatters the reference.
This library's side is timed through its C ABI on the same tensors, both with the depth channel (like for
like) and without it (what its training step runs, because that loss has no depth term).
"""
import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

REF_SO = os.path.join(HERE, "_ref", "libssb_ref.so")


def available():
    return os.path.exists(REF_SO)


def _P(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


class _Timer:
    """Accumulates CUDA-event times per stage name."""

    def __init__(self, torch):
        self.torch, self.ms, self.count = torch, {}, {}

    def run(self, name, fn, record=True):
        e0, e1 = self.torch.cuda.Event(enable_timing=True), self.torch.cuda.Event(enable_timing=True)
        e0.record()
        rc = fn()
        e1.record()
        e1.synchronize()
        if rc not in (0, None):
            raise RuntimeError(f"{name} returned {rc}")
        if record:
            self.ms[name] = self.ms.get(name, 0.0) + e0.elapsed_time(e1)
            self.count[name] = self.count.get(name, 0) + 1

    def mean(self):
        return {k: self.ms[k] / self.count[k] for k in self.ms}


def _sample_clocks(gpu_index):
    path = tempfile.mktemp(prefix="ref_clocks_", suffix=".csv")
    try:
        proc = subprocess.Popen(["nvidia-smi", "-i", str(gpu_index), "--query-gpu=clocks.sm,clocks.max.sm,clocks_event_reasons.active",
                                 "--format=csv,noheader,nounits", "-lms", "100"], stdout=open(path, "w"), stderr=subprocess.DEVNULL)
    except OSError:
        return None, path
    return proc, path


def _read_clocks(proc, path):
    if proc is None:
        return None
    proc.terminate()
    try:
        proc.wait(timeout=5)
    except subprocess.TimeoutExpired:
        proc.kill()
    sm, mx = [], []
    try:
        for line in open(path):
            f = [x.strip() for x in line.split(",")]
            try:
                sm.append(float(f[0])); mx.append(float(f[1]))
            except (ValueError, IndexError):
                continue
        os.unlink(path)
    except OSError:
        pass
    return {"sm_mhz_median": float(np.median(sm)), "sm_max_mhz": float(np.max(mx)), "samples": len(sm)} if sm else None


def time_kernels(cfg, n_views=None, repeats=3, device="cuda:0", with_ours=True):
    """Per-stage mean milliseconds per view (and per optimiser pass) of the reference's kernels, and of this
    library's on the same inputs.  Returns a dict ready for JSON."""
    import torch

    from oracle import pyoracle as O
    from spirula_studio_b200 import scenes

    ref = C.CDLL(REF_SO)
    ref.ref_set_sync(0)
    torch.cuda.set_device(device)
    dev = torch.device(device)
    n, W, H = cfg.n_splats, cfg.width, cfg.height
    n_views = min(n_views or cfg.n_views, cfg.n_views)
    tw, th = (W + 15) // 16, (H + 15) // 16
    Pn = W * H
    sp = scenes.make_splats(cfg)
    vm, K = scenes.make_cameras(cfg)
    to = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    z = lambda *s, dt=torch.float32: torch.zeros(*s, dtype=dt, device=dev)
    d = {k: to(v.reshape(-1)) for k, v in sp.items()}
    bits = cfg.sh_value_bits if cfg.sh_value_bits in (8, 16) else 32
    sh_packed = sh_bounds = None
    if bits != 32:
        packed, bounds = O.quant_encode(sp["features_sh"], bits)
        sh_packed, sh_bounds = to(packed.view(np.uint8)), to(bounds)
    d_vm, d_K = to(vm), to(K)
    aabb, depths, radii = z(n, 4), z(n), z(n)
    xy, depth, conic, opac, rgb = z(n, 2), z(n), z(n, 3), z(n), z(n, 3)
    cap = 16 * n
    tps, cum = z(n, dt=torch.int64), z(n, dt=torch.int64)
    ids_a, ids_b = z(cap, dt=torch.int64), z(cap, dt=torch.int64)
    fl_a, fl_b = z(cap, dt=torch.int32), z(cap, dt=torch.int32)
    offs = z(tw * th, dt=torch.int32)
    tmp = z(256 << 20, dt=torch.uint8)
    r_rgb, r_depth, r_T, r_last = z(Pn, 3), z(Pn), z(Pn), z(Pn, dt=torch.int32)
    g_xy, g_depth, g_conic, g_opac, g_rgb = z(n, 2), z(n), z(n, 3), z(n), z(n, 3)
    grads = {k: torch.zeros_like(t) for k, t in d.items()}
    v_depth, v_T, ssim_out = z(Pn), z(Pn), z(1)
    sh_arg = (None if bits != 32 else _P(d["features_sh"]))
    pk = (_P(sh_packed), _P(sh_bounds), bits, C.c_int64(256)) if bits != 32 else (None, None, 32, C.c_int64(256))

    ours = None
    if with_ours:
        from spirula_studio_b200 import lib as L
        lib = L.load()
        shq = L.shq_struct(sh_packed, sh_bounds, bits, 256) if bits != 32 else None
        s_struct = L.splats_struct({k: (None if (k == "features_sh" and bits != 32) else v) for k, v in d.items()})
        g_struct = L.splats_struct(grads)
        o_aabb, o_depths, o_rec, o_vrec = z(n, 4), z(n), z(n * 12), z(n * 12)
        ws_bytes = lib.ssb_intersect_tiles_workspace_bytes(tw * th, cap)
        o_ws = z(ws_bytes, dt=torch.uint8)
        o_flat, o_offs, o_m = z(cap, dt=torch.int32), z(tw * th, dt=torch.int32), z(1, dt=torch.int64)
        o_rgb, o_dep, o_T, o_last, o_vrgb, o_loss = z(Pn, 3), z(Pn), z(Pn), z(Pn, dt=torch.int32), z(Pn, 3), z(3)
        ours = _Timer(torch)

    t = _Timer(torch)
    pairs = []
    clock_proc, clock_path = _sample_clocks(dev.index or 0)
    for v in range(n_views):
        gt = to(scenes.make_target(cfg, v).reshape(-1, 3))
        cam_vm, cam_K = d_vm[v:v + 1].contiguous(), d_K[v:v + 1].contiguous()
        for rep in range(repeats + 1):
            rec = rep > 0                      # the first pass over a view warms up
            for a in (aabb, depths, xy, depth, conic, opac, rgb):
                a.zero_()
            t.run("project_fwd", lambda: ref.ref_project_fwd(
                1, n, W, H, _P(d["means"]), _P(d["quats"]), _P(d["scales"]), _P(d["opacities"]), _P(d["features_dc"]), sh_arg, *pk,
                _P(cam_vm), _P(cam_K), _P(aabb), _P(depths), _P(radii), _P(xy), _P(depth), _P(conic), _P(opac), _P(rgb)), rec)
            M, sel = C.c_int64(0), C.c_int32(0)
            t.run("intersect", lambda: ref.ref_intersect_tile_prealloc(
                1, n, W, H, _P(aabb), _P(depths), _P(xy), _P(conic), _P(opac), _P(tps), _P(cum), C.c_int64(cap),
                _P(ids_a), _P(ids_b), _P(fl_a), _P(fl_b), _P(offs), _P(tmp), C.c_int64(tmp.numel()), C.byref(M), C.byref(sel)), rec)
            fl = fl_b if sel.value else fl_a
            m = M.value
            t.run("raster_fwd", lambda: ref.ref_raster_fwd(
                1, n, m, W, H, _P(xy), _P(depth), _P(conic), _P(opac), _P(rgb), _P(offs), _P(fl), _P(r_rgb), _P(r_depth), _P(r_T), _P(r_last)), rec)
            # L1 part of the loss gradient (the reference's per-pixel loss kernel, not timed), then its SSIM kernel in place
            v_rgb = (0.8 / (3.0 * Pn)) * torch.sign(r_rgb - gt)
            t.run("loss_ssim", lambda: ref.ref_ssim_inplace(1, H, W, _P(r_rgb), _P(gt), C.c_float(-0.2), _P(v_rgb), _P(ssim_out)), rec)
            for a in (g_xy, g_depth, g_conic, g_opac, g_rgb):
                a.zero_()
            t.run("raster_bwd", lambda: ref.ref_raster_bwd(
                1, n, m, W, H, _P(xy), _P(depth), _P(conic), _P(opac), _P(rgb), _P(offs), _P(fl), _P(r_rgb), _P(r_depth), _P(r_T), _P(r_last),
                _P(v_rgb), _P(v_depth), _P(v_T), _P(g_xy), _P(g_depth), _P(g_conic), _P(g_opac), _P(g_rgb)), rec)
            t.run("project_bwd", lambda: ref.ref_project_bwd(
                1, n, W, H, _P(d["means"]), _P(d["quats"]), _P(d["scales"]), _P(d["opacities"]), _P(d["features_dc"]), sh_arg, *pk,
                _P(cam_vm), _P(cam_K), _P(aabb), _P(g_xy), _P(g_depth), _P(g_conic), _P(g_opac), _P(g_rgb),
                _P(grads["means"]), _P(grads["quats"]), _P(grads["scales"]), _P(grads["opacities"]), _P(grads["features_dc"]),
                _P(grads["features_sh"])), rec)
            if rec and rep == 1:
                pairs.append(m)
            if ours is not None:
                cams = L.cameras_struct(cam_vm, cam_K, W, H)
                ours.run("project_fwd", lambda: lib.ssb_project_fwd(C.byref(s_struct), C.byref(shq) if shq else None, n, C.byref(cams),
                                                                     _P(o_aabb), _P(o_depths), None, _P(o_rec), None), rec)
                ours.run("intersect", lambda: lib.ssb_intersect_tiles(_P(o_aabb), _P(o_depths), _P(o_rec), n, n, W, H, _P(o_ws), ws_bytes, None,
                                                                       _P(o_flat), cap, _P(o_offs), _P(o_m), None), rec)
                ours.run("raster_fwd", lambda: lib.ssb_raster_fwd(_P(o_rec), n, _P(o_offs), _P(o_flat), cap, _P(o_m), 1, W, H, _P(o_rgb), None,
                                                                   _P(o_T), _P(o_last), None), rec)
                ours.run("raster_fwd_depth", lambda: lib.ssb_raster_fwd(_P(o_rec), n, _P(o_offs), _P(o_flat), cap, _P(o_m), 1, W, H, _P(o_rgb),
                                                                         _P(o_dep), _P(o_T), _P(o_last), None), rec)
                ours.run("loss_l1_ssim", lambda: lib.ssb_loss_l1_ssim_fwdbwd(_P(o_rgb), _P(gt), 1, H, W, C.c_float(0.8), C.c_float(0.2), _P(o_vrgb),
                                                                              _P(o_loss), None), rec)
                o_vrec.zero_()
                ours.run("raster_bwd", lambda: lib.ssb_raster_bwd(_P(o_rec), n, _P(o_offs), _P(o_flat), cap, _P(o_m), 1, W, H, None, _P(o_T),
                                                                   _P(o_last), _P(o_vrgb), None, None, _P(o_vrec), None), rec)
                o_vrec.zero_()
                ours.run("raster_bwd_depth", lambda: lib.ssb_raster_bwd(_P(o_rec), n, _P(o_offs), _P(o_flat), cap, _P(o_m), 1, W, H, _P(o_dep),
                                                                         _P(o_T), _P(o_last), _P(o_vrgb), _P(v_depth), _P(v_T), _P(o_vrec), None), rec)
                ours.run("project_bwd", lambda: lib.ssb_project_bwd(C.byref(s_struct), C.byref(shq) if shq else None, n, C.byref(cams), _P(o_aabb),
                                                                     _P(o_vrec), C.byref(g_struct), 1, None), rec)
    # ---- optimiser: geometry, DC, SH (doubly quantised when the scene stores SH that way)
    lr = cfg.lrs
    m1 = {k: torch.zeros_like(t_) for k, t_ in d.items()}
    m2 = {k: torch.zeros_like(t_) for k, t_ in d.items()}
    cells = n * 45
    gs = 1.0 / cfg.n_views
    if bits != 32:
        opt_packed, opt_bounds = z(cells * 2, dt=torch.uint8), z(((cells + 255) // 256) * 4)
        val_packed = sh_packed.clone()
        val_bounds = sh_bounds.clone()
    for i in range(3 + max(repeats, 5)):
        rec = i >= 3
        step = i + 1
        t.run("adam_geometry", lambda: ref.ref_adam_geometry(
            C.c_int64(n), step, C.c_float(gs), 0, C.c_float(lr["lr_means"]), C.c_float(lr["lr_quats"]), C.c_float(lr["lr_scales"]),
            C.c_float(lr["lr_opacities"]),
            _P(d["means"]), _P(grads["means"]), _P(m1["means"]), _P(m2["means"]), _P(d["quats"]), _P(grads["quats"]), _P(m1["quats"]), _P(m2["quats"]),
            _P(d["scales"]), _P(grads["scales"]), _P(m1["scales"]), _P(m2["scales"]),
            _P(d["opacities"]), _P(grads["opacities"]), _P(m1["opacities"]), _P(m2["opacities"])), rec)
        t.run("adam_dc", lambda: ref.ref_adam_plain(C.c_int64(3 * n), step, C.c_float(lr["lr_features_dc"]), C.c_float(0.0),
                                                    C.c_float(0.5 / 0.28209479177387814), C.c_float(gs), 0, _P(d["features_dc"]),
                                                    _P(grads["features_dc"]), _P(m1["features_dc"]), _P(m2["features_dc"])), rec)
        if bits != 32:
            t.run("adam_sh", lambda: ref.ref_adam_qq(C.c_int64(cells), step, C.c_float(lr["lr_features_sh"]), C.c_float(0.0), C.c_float(gs), 0, bits,
                                                     _P(grads["features_sh"]), _P(opt_packed), _P(opt_bounds), _P(val_packed), _P(val_bounds)), rec)
        else:
            t.run("adam_sh", lambda: ref.ref_adam_plain(C.c_int64(cells), step, C.c_float(lr["lr_features_sh"]), C.c_float(0.0), C.c_float(0.0),
                                                        C.c_float(gs), 0, _P(d["features_sh"]), _P(grads["features_sh"]), _P(m1["features_sh"]),
                                                        _P(m2["features_sh"])), rec)
        if ours is not None:
            cfg_a = L.SsbAdamConfig(lr["lr_means"], lr["lr_quats"], lr["lr_scales"], lr["lr_opacities"], lr["lr_features_dc"], lr["lr_features_sh"],
                                    0.0, gs, step, 0)
            p_struct = s_struct
            m1s, m2s = (L.splats_struct({k: (None if (k == "features_sh" and bits != 32) else v) for k, v in m.items()}) for m in (m1, m2))

            def adam_ours():
                st = lib.ssb_adam_step(C.byref(p_struct), C.byref(g_struct), C.byref(m1s), C.byref(m2s), 0, n, C.byref(cfg_a), None)
                if st == 0 and bits != 32:
                    st = lib.ssb_adam_step_sh_quantized(_P(grads["features_sh"]), _P(opt_packed), _P(opt_bounds), _P(val_packed), _P(val_bounds),
                                                        bits, 0, cells, cells, C.byref(cfg_a), None)
                return st
            ours.run("adam", adam_ours, rec)
    ref.ref_set_sync(1)
    clocks = _read_clocks(clock_proc, clock_path)
    rm = t.mean()
    view_stages = ("project_fwd", "intersect", "raster_fwd", "loss_ssim", "raster_bwd", "project_bwd")
    ref_view = sum(rm[k] for k in view_stages)
    ref_adam = rm["adam_geometry"] + rm["adam_dc"] + rm["adam_sh"]
    out = {
        "workload": cfg.name, "n_splats": n, "resolution": [W, H], "views_timed": n_views, "repeats_per_view": repeats,
        "pairs_per_view_mean": float(np.mean(pairs)) if pairs else 0.0,
        "reference_ms": {k: round(v, 4) for k, v in rm.items()},
        "reference_ms_per_view": round(ref_view, 4), "reference_ms_adam": round(ref_adam, 4),
        "reference_ms_per_iteration": round(cfg.n_views * ref_view + ref_adam, 3),
        "reference_iters_per_s_kernels_only": round(1e3 / (cfg.n_views * ref_view + ref_adam), 3),
        "clocks": clocks,
        "not_in_reference_time": "per-pixel L1 loss kernel, gradient zeroing, host-side engine work",
    }
    if ours is not None:
        om = ours.mean()
        our_view = om["project_fwd"] + om["intersect"] + om["raster_fwd"] + om["loss_l1_ssim"] + om["raster_bwd"] + om["project_bwd"]
        our_view_depth = our_view - om["raster_fwd"] - om["raster_bwd"] + om["raster_fwd_depth"] + om["raster_bwd_depth"]
        out.update({
            "ours_ms": {k: round(v, 4) for k, v in om.items()},
            "ours_ms_per_view": round(our_view, 4), "ours_ms_per_view_with_depth": round(our_view_depth, 4),
            "ours_ms_per_iteration_serial": round(cfg.n_views * our_view + om["adam"], 3),
            "ratio_per_stage": {
                "project_fwd": round(rm["project_fwd"] / om["project_fwd"], 2), "intersect": round(rm["intersect"] / om["intersect"], 2),
                "raster_fwd_like_for_like": round(rm["raster_fwd"] / om["raster_fwd_depth"], 2), "raster_fwd": round(rm["raster_fwd"] / om["raster_fwd"], 2),
                "loss (ssim only vs l1+ssim)": round(rm["loss_ssim"] / om["loss_l1_ssim"], 2),
                "raster_bwd_like_for_like": round(rm["raster_bwd"] / om["raster_bwd_depth"], 2), "raster_bwd": round(rm["raster_bwd"] / om["raster_bwd"], 2),
                "project_bwd": round(rm["project_bwd"] / om["project_bwd"], 2), "adam": round(ref_adam / om["adam"], 2)},
            "ratio_iteration_kernels_only": round((cfg.n_views * ref_view + ref_adam) / (cfg.n_views * our_view + om["adam"]), 3),
        })
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="mid_1m")
    ap.add_argument("--views", type=int, default=0)
    ap.add_argument("--splats", type=int, default=0)
    ap.add_argument("--repeats", type=int, default=3)
    ap.add_argument("--out", default="")
    a = ap.parse_args()
    if not available():
        print(json.dumps({"unavailable": f"{REF_SO} has not been built (make -C oracle -f Makefile.ref REF=<reference root>)"}))
        return
    from spirula_studio_b200 import scenes
    cfg = scenes.CONFIGS[a.workload]
    if a.splats:
        cfg = scenes.scaled(cfg, n_splats=a.splats, name=cfg.name)
    res = time_kernels(cfg, n_views=a.views or None, repeats=a.repeats)
    text = json.dumps(res, indent=1)
    print(text)
    if a.out:
        with open(a.out, "w") as f:
            f.write(text + "\n")


if __name__ == "__main__":
    main()
