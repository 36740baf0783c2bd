"""Generates the golden fixtures in this directory by running the REFERENCE's own
device code (oracle/_ref/libssb_ref.so, built from the reference sources by
oracle/Makefile.ref) on a GPU, on small seeded scenes.

    python tests/golden/make_golden.py [out_dir [fixture ...]]

With fixture names (ring2, dense1, wide_fisheye, wide_equisolid, wide_equirect, ssim, ssim_map, adam, accum, quant_proj,
packed_proj, dist_proj, ...) only those are written; accum, quant_proj and packed_proj read the committed ring2.npz / dense1.npz.

Inputs are not stored: they are regenerated from `golden_cases.py` (same seeds).
Every stage is run stage-isolated on the reference's own upstream outputs, so a
fixture holds exactly what that stage of the reference produced for the inputs
the previous fixture records.
"""
import ctypes as C
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, HERE)

from golden_cases import (ACCUM_CASES, CASES, DENSIFY_SCORE_RUNS, DIST_CASES, FPBO_L1_RUNS, FPBO_RUNS, FPBO_SCENE, encode_splat_blocks, dist_case_inputs, fpbo_inputs, DENSIFY_SPLIT, LIVE_TILE_CASE, LOSS_MAP_WEIGHT, MULTI_SCALE_RUNS, QUANT_CASES, QUANT_SCENE, WIDE_CASES, accum_weight_map, adam_inputs,  # noqa: E402
                          build_case, densify_inputs, densify_split_inputs, loss_inputs, loss_map_base, loss_masks, quant_sh_inputs, raster_cotangents, tile_masks)  # noqa: E402

DEV = "cuda:0"


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def P(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def check(rc, what):
    if rc != 0:
        raise RuntimeError(f"{what} failed with {rc}")


def run_case(ref, name, out_dir):
    cfg, sp, vm, K = build_case(name)
    model = WIDE_CASES[name]["model"] if name in WIDE_CASES else 0
    n, W, H, I = cfg.n_splats, cfg.width, cfg.height, vm.shape[0]
    d = {k: dev(v.reshape(-1)) for k, v in sp.items()}
    d_vm, d_K = dev(vm), dev(K)
    m = I * n
    z = lambda *s, dt=torch.float32: torch.zeros(*s, dtype=dt, device=DEV)
    aabb, depths, radii = z(m, 4), z(m), z(n)
    xy, depth, conic, opac, rgb = z(m, 2), z(m), z(m, 3), z(m), z(m, 3)
    fwd = ref.ref_project_fwd if model == 0 else (lambda *a: ref.ref_project_fwd_model(model, *a))
    bwd = ref.ref_project_bwd if model == 0 else (lambda *a: ref.ref_project_bwd_model(model, *a))
    check(fwd(I, n, W, H, P(d["means"]), P(d["quats"]), P(d["scales"]), P(d["opacities"]), P(d["features_dc"]),
                              P(d["features_sh"]), None, None, 32, C.c_int64(256), P(d_vm), P(d_K), P(aabb), P(depths), P(radii),
                              P(xy), P(depth), P(conic), P(opac), P(rgb)), "ref_project_fwd")
    # culled pairs: the reference leaves their screen entries unwritten (zeros here)
    out = dict(aabb=aabb, depths=depths, radii=radii, xy=xy, depth=depth, conic=conic, opac=opac, rgb=rgb)

    cap = 64 * n
    tps, cum = z(m, dt=torch.int64), z(m, dt=torch.int64)
    ids_a, ids_b = z(cap, dt=torch.int64), z(cap, dt=torch.int64)
    fl_a, fl_b = z(cap, dt=torch.int32), z(cap, dt=torch.int32)
    tw, th = (W + 15) // 16, (H + 15) // 16
    offs = z(I * tw * th, dt=torch.int32)
    M, sel = C.c_int64(0), C.c_int32(0)
    check(ref.ref_intersect_tile(I, n, W, H, P(aabb), P(depths), P(xy), P(conic), P(opac), P(tps), P(cum), C.c_int64(cap),
                                 P(ids_a), P(ids_b), P(fl_a), P(fl_b), P(offs), C.byref(M), C.byref(sel)), "ref_intersect_tile")
    M = M.value
    ids, fl = (ids_b, fl_b) if sel.value else (ids_a, fl_a)
    out.update(tiles_per_splat=tps.to(torch.int32), sorted_ids=ids[:M], sorted_flat=fl[:M], offsets=offs)

    P_ = I * H * W
    r_rgb, r_depth, r_T, r_last = z(P_, 3), z(P_), z(P_), z(P_, dt=torch.int32)
    check(ref.ref_raster_fwd(I, n, M, W, H, P(xy), P(depth), P(conic), P(opac), P(rgb), P(offs), P(fl), P(r_rgb), P(r_depth), P(r_T), P(r_last)),
          "ref_raster_fwd")
    out.update(render_rgb=r_rgb, render_depth=r_depth, render_T=r_T, last_ids=r_last)

    v_rgb, v_depth, v_T = (dev(a) for a in raster_cotangents(name, P_))
    g_xy, g_depth, g_conic, g_opac, g_rgb = z(m, 2), z(m), z(m, 3), z(m), z(m, 3)
    check(ref.ref_raster_bwd(I, n, M, W, H, P(xy), P(depth), P(conic), P(opac), P(rgb), P(offs), P(fl), P(r_rgb), P(r_depth), P(r_T), P(r_last),
                             P(v_rgb), P(v_depth), P(v_T), P(g_xy), P(g_depth), P(g_conic), P(g_opac), P(g_rgb)), "ref_raster_bwd")
    out.update(v_xy=g_xy, v_depth=g_depth, v_conic=g_conic, v_opac=g_opac, v_rgb=g_rgb)

    g = {k: torch.zeros_like(t) for k, t in d.items()}
    check(bwd(I, n, W, H, P(d["means"]), P(d["quats"]), P(d["scales"]), P(d["opacities"]), P(d["features_dc"]),
                              P(d["features_sh"]), None, None, 32, C.c_int64(256), P(d_vm), P(d_K), P(aabb),
                              P(g_xy), P(g_depth), P(g_conic), P(g_opac), P(g_rgb),
                              P(g["means"]), P(g["quats"]), P(g["scales"]), P(g["opacities"]), P(g["features_dc"]), P(g["features_sh"])), "ref_project_bwd")
    out.update({"g_" + k: t for k, t in g.items()})
    np.savez_compressed(os.path.join(out_dir, f"{name}.npz"), **{k: t.cpu().numpy() for k, t in out.items()})
    print(name, "pairs", M, "visible", int((aabb[:, 2] > aabb[:, 0]).sum()))


def run_loss(ref, out_dir):
    out = {}
    for tag, (B, H, W, render, gt) in loss_inputs().items():
        v = torch.zeros(B * H * W, 3, device=DEV)
        s = torch.zeros(1, device=DEV)
        d_render, d_gt = dev(render), dev(gt)      # named: a temporary's memory would be reused by the next one
        check(ref.ref_ssim_inplace(B, H, W, P(d_render), P(d_gt), C.c_float(-0.2), P(v), P(s)), "ref_ssim_inplace")
        out[f"{tag}_grad"] = v.cpu().numpy()
        out[f"{tag}_ssim"] = s.cpu().numpy()
    np.savez_compressed(os.path.join(out_dir, "ssim.npz"), **out)


def run_loss_map(ref, out_dir):
    """The densification loss map of the SSIM kernel, added in place onto a seeded map, for the three SsimLossMapMode values."""
    out = {}
    for tag, (B, H, W, render, gt) in loss_inputs().items():
        d_render, d_gt = dev(render), dev(gt)
        for mode in (1, 2, 3):
            v = torch.zeros(B * H * W, 3, device=DEV)
            s = torch.zeros(1, device=DEV)
            lm = dev(loss_map_base(tag, B * H * W))
            check(ref.ref_ssim_inplace_map(B, H, W, P(d_render), P(d_gt), C.c_float(-0.2), P(v), P(s), C.c_float(LOSS_MAP_WEIGHT), P(lm), mode),
                  "ref_ssim_inplace_map")
            out[f"{tag}_map{mode}"] = lm.cpu().numpy()
    np.savez_compressed(os.path.join(out_dir, "ssim_map.npz"), **out)


def run_loss_masked(ref, out_dir):
    """The masked SSIM launch (coverage pass + kernel) for a mask of the image's size and one of another size: gradient, mean
    SSIM and the three loss-map variants added onto a seeded map."""
    out = {}
    for tag, (B, H, W, render, gt) in loss_inputs().items():
        d_render, d_gt = dev(render), dev(gt)
        for kind, mask in loss_masks(tag, B, H, W).items():
            d_mask = torch.from_numpy(mask.astype(np.bool_)).to(DEV)
            Bm, Hm, Wm = mask.shape
            for mode in (0, 1, 2, 3):
                v = torch.zeros(B * H * W, 3, device=DEV)
                s = torch.zeros(1, device=DEV)
                lm = dev(loss_map_base(tag, B * H * W))
                check(ref.ref_ssim_inplace_masked(B, H, W, P(d_render), P(d_gt), P(d_mask), Bm, Hm, Wm, C.c_float(-0.2), P(v), P(s),
                                                  C.c_float(LOSS_MAP_WEIGHT), P(lm), mode), "ref_ssim_inplace_masked")
                if mode == 0:
                    out[f"{tag}_{kind}_grad"] = v.cpu().numpy()
                    out[f"{tag}_{kind}_ssim"] = s.cpu().numpy()
                else:
                    out[f"{tag}_{kind}_map{mode}"] = lm.cpu().numpy()
    np.savez_compressed(os.path.join(out_dir, "ssim_masked.npz"), **out)


def run_tiles_live(ref, out_dir):
    """The live-tile map of a mask and the intersection that skips dead tiles, on the committed projection of one case."""
    case = np.load(os.path.join(HERE, LIVE_TILE_CASE + ".npz"))
    cfg, sp, vm, K = build_case(LIVE_TILE_CASE)
    n, W, H, I = cfg.n_splats, cfg.width, cfg.height, vm.shape[0]
    m = I * n
    aabb, depths, xy, conic, opac = (dev(case[k]) for k in ("aabb", "depths", "xy", "conic", "opac"))
    z = lambda *s, dt=torch.float32: torch.zeros(*s, dtype=dt, device=DEV)
    tw, th = (W + 15) // 16, (H + 15) // 16
    out = {}
    for kind, mask in tile_masks(I, H, W).items():
        d_mask = torch.from_numpy(mask.astype(np.bool_)).to(DEV)
        live = z(I * tw * th, dt=torch.int32)
        check(ref.ref_tile_active(P(d_mask), I, mask.shape[1], mask.shape[2], W, H, P(live)), "ref_tile_active")
        cap = 64 * n
        tps, cum = z(m, dt=torch.int64), z(m, dt=torch.int64)
        ids_a, ids_b = z(cap, dt=torch.int64), z(cap, dt=torch.int64)
        fl_a, fl_b = z(cap, dt=torch.int32), z(cap, dt=torch.int32)
        offs = z(I * tw * th, dt=torch.int32)
        M, sel = C.c_int64(0), C.c_int32(0)
        check(ref.ref_intersect_tile_live(I, n, W, H, P(aabb), P(depths), P(xy), P(conic), P(opac), P(live), P(tps), P(cum), C.c_int64(cap),
                                          P(ids_a), P(ids_b), P(fl_a), P(fl_b), P(offs), C.byref(M), C.byref(sel)), "ref_intersect_tile_live")
        ids, fl = (ids_b, fl_b) if sel.value else (ids_a, fl_a)
        out.update({f"{kind}_tile_active": live.cpu().numpy(), f"{kind}_tiles_per_splat": tps.to(torch.int32).cpu().numpy(),
                    f"{kind}_sorted_ids": ids[:M.value].cpu().numpy(), f"{kind}_sorted_flat": fl[:M.value].cpu().numpy(),
                    f"{kind}_offsets": offs.cpu().numpy()})
        print("tiles_live", kind, "live tiles", int(live.sum()), "of", live.numel(), "pairs", M.value)
    np.savez_compressed(os.path.join(out_dir, "tiles_live.npz"), **out)


def run_loss_multi(ref, out_dir):
    """The reference's whole multi-scale loss driver (pyramid, per-pixel pass, SSIM pass, fold of the levels, loss map)
    on the colour modalities: gradient, loss scalars and the loss map of modes 1 (loss_full) and 3 (SSIM contrast-structure)."""
    out = {}
    for tag, (B, H, W, render, gt) in loss_inputs().items():
        d_render, d_gt = dev(render), dev(gt)
        masks = dict(loss_masks(tag, B, H, W), none=None)
        for kind, scales in MULTI_SCALE_RUNS:
            mask = masks[kind]
            d_mask = torch.from_numpy(mask.astype(np.bool_)).to(DEV) if mask is not None else None
            Hm, Wm = (mask.shape[1], mask.shape[2]) if mask is not None else (0, 0)
            for mode in (0, 1, 3):
                v = torch.zeros(B * H * W, 3, device=DEV)
                lm = torch.zeros(B * H * W, device=DEV) if mode else None
                rgb_loss, ssim = C.c_float(0), C.c_float(0)
                check(ref.ref_multi_scale_loss(scales, B, H, W, P(d_render), P(d_gt), P(d_mask) if d_mask is not None else None, Hm, Wm,
                                               C.c_float(0.8), C.c_float(0.2), mode, P(v), P(lm) if lm is not None else None,
                                               C.byref(rgb_loss), C.byref(ssim)), "ref_multi_scale_loss")
                key = f"{tag}_{kind}_{scales}"
                if mode == 0:
                    out[key + "_grad"] = v.cpu().numpy()
                    out[key + "_scalars"] = np.array([rgb_loss.value, ssim.value], np.float32)
                else:
                    out[key + f"_map{mode}"] = lm.cpu().numpy()
    np.savez_compressed(os.path.join(out_dir, "loss_multi.npz"), **out)


def run_densify(ref, out_dir):
    """The reference's per-step densification kernels: scale clip, averaged-weight quotient, score update (mean, max, geometric
    mean; blended, world-gradient-only and opacity-weighted scores), quantile clip with the powered sample score, and both noises."""
    inp = densify_inputs()
    n = inp["radii"].shape[0]
    out = {}
    inf = float("inf")
    for name, kw in DENSIFY_SCORE_RUNS:
        radii, scales, opacs = dev(inp["radii"]), dev(inp["log_scales"]), dev(inp["logit_opacs"])
        aw, den, wg, acc = dev(inp["accum_weight"]), dev(inp["accum_den"]), dev(inp["world_grad"]), dev(inp["accum_buffer"])
        if kw.get("max_screen_size") is not None or kw.get("max_world_size") is not None:
            check(ref.ref_densify_clip_scale(C.c_int64(n), P(radii), P(scales), None, C.c_float(kw.get("max_screen_size", inf)),
                                             C.c_float(kw.get("clip_hardness", inf)), C.c_float(kw.get("max_world_size", inf))), "clip_scale")
            out[f"{name}_log_scales"] = scales.cpu().numpy()
        if kw.get("accum", True):
            blend = kw.get("blend_w", 0.0)
            if kw.get("accum_mode", 1) == 3:
                both = torch.cat([aw, den])
                check(ref.ref_densify_accum_finalize(C.c_int64(n), P(both)), "accum_finalize")
                aw = both[:n].clone()
                out[f"{name}_accum_weight"] = aw.cpu().numpy()
            # buffers as engine_densify_step picks them (src/engine/EngineDensify.cpp:222-243)
            has_w, has_wg = kw.get("weights", True), kw.get("world", False)
            if blend >= 1.0 and has_wg:
                score, score2, op = wg, None, None
            elif has_w:
                score, score2, op = aw, (wg if blend > 0 and has_wg else None), None
            else:
                score, score2, op = opacs, None, opacs
            check(ref.ref_densify_update_weight(C.c_int64(n), P(radii), P(op), P(score), P(score2), C.c_float(blend), C.c_float(kw["score_power"]),
                                                P(acc), kw["score_mode"]), "update_weight")
            sample = torch.zeros(n, 2, device=DEV) if kw.get("sample") else None
            if kw.get("sample") or kw.get("clip_quantile", 1.0) < 1.0:
                check(ref.ref_densify_clip_score(C.c_int64(n), P(acc), C.c_float(kw.get("clip_quantile", 1.0)), C.c_float(kw.get("final_power", 1.0)),
                                                 P(sample)), "clip_score")
            out[f"{name}_accum_buffer"] = acc.cpu().numpy()
            if sample is not None:
                out[f"{name}_sample_score"] = sample.cpu().numpy()
    for revised in (0, 1):
        means, radii, scales, quats, opacs = (dev(inp[k]) for k in ("means", "radii", "log_scales", "quats", "logit_opacs"))   # named: see run_loss
        check(ref.ref_densify_add_noise(C.c_int64(n), C.c_float(5e5 * 1.6e-4 if revised else 2e3), revised, P(radii), P(means), P(scales), P(quats),
                                        P(opacs)), "add_noise")
        out[f"noise{revised}_means"] = means.cpu().numpy()
    np.savez_compressed(os.path.join(out_dir, "densify.npz"), **out)


SPLIT_ATTRS = ("means", "quats", "scales", "opacities", "features_dc", "features_sh")
SPLIT_KEYS = (SPLIT_ATTRS + tuple("m1_" + a for a in SPLIT_ATTRS) + tuple("m2_" + a for a in SPLIT_ATTRS) +
              ("accum", "steps", "sh_optim_packed", "sh_value_packed"))


def run_densify_split(ref, out_dir):
    """The reference's relocation of dead splats and its growth step (long-axis split, weighted draw without replacement), fp32
    SH and quantised SH (q16 values + 8-bit joint state): the whole state after the relocation and after the growth."""
    out = {}
    D = DENSIFY_SPLIT
    for quant in (False, True):
        st = densify_split_inputs(quant)
        d = {k: (dev(v) if isinstance(v, np.ndarray) else None) for k, v in st.items() if not isinstance(v, int)}
        ptr = lambda k: P(d.get(k))
        def call(mode, seed):
            args = [mode, C.c_int64(D["cur_n"] if mode == 0 else D["cur_n"]), C.c_int64(D["num_new"]), C.c_int64(D["cap"]), C.c_float(D["min_opacity"]),
                    C.c_float(D["split_k"]), C.c_uint32(seed), ptr("weights")]
            args += [ptr(a) for a in SPLIT_ATTRS] + [ptr("m1_" + a) for a in SPLIT_ATTRS] + [ptr("m2_" + a) for a in SPLIT_ATTRS]
            args += [ptr("sh_optim_packed"), ptr("sh_optim_bounds"), st.get("sh_optim_bits", 32), ptr("sh_value_packed"), ptr("sh_value_bounds"),
                     st.get("sh_value_bits", 32), ptr("accum"), ptr("steps")]
            check(ref.ref_densify_split(*args), "ref_densify_split")
        tag = "q" if quant else "f"
        call(0, D["seed"])
        for k in SPLIT_KEYS:
            if d.get(k) is not None:
                out[f"{tag}_reloc_{k}"] = d[k].cpu().numpy()
        call(1, D["seed"] + 1)
        for k in SPLIT_KEYS:
            if d.get(k) is not None:
                out[f"{tag}_add_{k}"] = d[k].cpu().numpy()
    np.savez_compressed(os.path.join(out_dir, "densify_split.npz"), **out)


def run_adam(ref, out_dir):
    inp = adam_inputs()
    out = {}
    # geometry + plain Adam, three steps with fresh gradients each
    p = {k: dev(v.reshape(-1)) for k, v in inp["params"].items()}
    m1 = {k: torch.zeros_like(t) for k, t in p.items()}
    m2 = {k: torch.zeros_like(t) for k, t in p.items()}
    n = inp["n"]
    lr = inp["lrs"]
    for step, grads in enumerate(inp["grads"], start=1):
        g = {k: dev(v.reshape(-1)) for k, v in grads.items()}
        check(ref.ref_adam_geometry(C.c_int64(n), step, C.c_float(inp["grad_scale"]), 0, C.c_float(lr["lr_means"]), C.c_float(lr["lr_quats"]),
                                    C.c_float(lr["lr_scales"]), C.c_float(lr["lr_opacities"]),
                                    P(p["means"]), P(g["means"]), P(m1["means"]), P(m2["means"]),
                                    P(p["quats"]), P(g["quats"]), P(m1["quats"]), P(m2["quats"]),
                                    P(p["scales"]), P(g["scales"]), P(m1["scales"]), P(m2["scales"]),
                                    P(p["opacities"]), P(g["opacities"]), P(m1["opacities"]), P(m2["opacities"])), "ref_adam_geometry")
        check(ref.ref_adam_plain(C.c_int64(3 * n), step, C.c_float(lr["lr_features_dc"]), C.c_float(0.0), C.c_float(0.5 / 0.28209479177387814),
                                 C.c_float(inp["grad_scale"]), 0, P(p["features_dc"]), P(g["features_dc"]), P(m1["features_dc"]), P(m2["features_dc"])),
              "ref_adam_plain dc")
        check(ref.ref_adam_plain(C.c_int64(45 * n), step, C.c_float(lr["lr_features_sh"]), C.c_float(0.0), C.c_float(0.0),
                                 C.c_float(inp["grad_scale"]), 0, P(p["features_sh"]), P(g["features_sh"]), P(m1["features_sh"]), P(m2["features_sh"])),
              "ref_adam_plain sh")
        for k in p:
            out[f"p{step}_{k}"] = p[k].cpu().numpy()
        if step == 3:
            for k in p:
                out[f"m1_{k}"] = m1[k].cpu().numpy()
                out[f"m2_{k}"] = m2[k].cpu().numpy()
    # doubly quantised SH Adam: one step from a given encoded state, for 16- and 8-bit values
    for bits in (16, 8):
        q = inp[f"qq{bits}"]
        vp, vb, op, ob = dev(q["value_packed"]), dev(q["value_bounds"]), dev(q["optim_packed"]), dev(q["optim_bounds"])
        for step, grad in enumerate(q["grads"], start=1):
            d_grad = dev(grad)
            check(ref.ref_adam_qq(C.c_int64(q["numel"]), step, C.c_float(lr["lr_features_sh"]), C.c_float(0.0), C.c_float(inp["grad_scale"]), 0, bits,
                                  P(d_grad), P(op), P(ob), P(vp), P(vb)), "ref_adam_qq")
            out[f"qq{bits}_s{step}_value_packed"] = vp.cpu().numpy()
            out[f"qq{bits}_s{step}_value_bounds"] = vb.cpu().numpy()
            out[f"qq{bits}_s{step}_optim_packed"] = op.cpu().numpy()
            out[f"qq{bits}_s{step}_optim_bounds"] = ob.cpu().numpy()
    # 8-bit optimiser state with fp32 values: three steps from a zero state
    q = inp["q8"]
    # The reference kernel stores param[idx] for every thread of its last 256-thread block, also past numel
    # (FusedAppearanceOptim.cu:190), so the value buffer is padded to whole blocks here.
    nb = (q["numel"] + 255) // 256
    x_buf = torch.zeros(nb * 256, dtype=torch.float32, device=DEV)
    x = x_buf[:q["numel"]]
    x.copy_(dev(q["x0"]))
    op = torch.zeros(q["numel"] * 2, dtype=torch.uint8, device=DEV)
    ob = torch.zeros(nb * 4, dtype=torch.float32, device=DEV)
    for step, grad in enumerate(q["grads"], start=1):
        d_grad = dev(grad)
        check(ref.ref_adam_q8(C.c_int64(q["numel"]), step, C.c_float(lr["lr_features_sh"]), C.c_float(0.0), C.c_float(inp["grad_scale"]), 0,
                              P(x), P(d_grad), P(op), P(ob)), "ref_adam_q8")
        out[f"q8_s{step}_x"] = x.cpu().numpy()
        out[f"q8_s{step}_optim_packed"] = op.cpu().numpy()
        out[f"q8_s{step}_optim_bounds"] = ob.cpu().numpy()
    # optional parts: "exA" = regularisers + per-splat step counters (geometry, DC with stride 3, SH with stride 45),
    # "exB" = the same with the scale-agnostic mean update; three steps each from the seeded parameters
    ex = inp["ex"]
    d_reg_host = np.ascontiguousarray(ex["reg"])
    d_radii, d_steps = dev(ex["radii"]), dev(ex["steps"])
    d_score = torch.zeros(n, dtype=torch.float32, device=DEV)
    for tag, agnostic in (("exA", 0), ("exB", 1)):
        p = {k: dev(v.reshape(-1)) for k, v in inp["params"].items()}
        m1 = {k: torch.zeros_like(t) for k, t in p.items()}
        m2 = {k: torch.zeros_like(t) for k, t in p.items()}
        for step, grads in enumerate(inp["grads"], start=1):
            g = {k: dev(v.reshape(-1)) for k, v in grads.items()}
            check(ref.ref_adam_geometry_ex(C.c_int64(n), step, C.c_float(inp["grad_scale"]), 0, C.c_float(lr["lr_means"]), C.c_float(lr["lr_quats"]),
                                           C.c_float(lr["lr_scales"]), C.c_float(lr["lr_opacities"]),
                                           P(p["means"]), P(g["means"]), P(m1["means"]), P(m2["means"]),
                                           P(p["quats"]), P(g["quats"]), P(m1["quats"]), P(m2["quats"]),
                                           P(p["scales"]), P(g["scales"]), P(m1["scales"]), P(m2["scales"]),
                                           P(p["opacities"]), P(g["opacities"]), P(m1["opacities"]), P(m2["opacities"]),
                                           d_reg_host.ctypes.data_as(C.c_void_p), agnostic, P(d_radii), P(d_steps), P(d_score)), "ref_adam_geometry_ex")
            if not agnostic and step == 1:
                out["exA_densify_score"] = d_score.cpu().numpy()
            if not agnostic:
                check(ref.ref_adam_plain_steps(C.c_int64(3 * n), P(d_steps), 3, C.c_float(lr["lr_features_dc"]), C.c_float(0.0),
                                               C.c_float(0.5 / 0.28209479177387814), C.c_float(inp["grad_scale"]), 0,
                                               P(p["features_dc"]), P(g["features_dc"]), P(m1["features_dc"]), P(m2["features_dc"])), "plain_steps dc")
                check(ref.ref_adam_plain_steps(C.c_int64(45 * n), P(d_steps), 45, C.c_float(lr["lr_features_sh"]), C.c_float(0.0), C.c_float(0.0),
                                               C.c_float(inp["grad_scale"]), 0,
                                               P(p["features_sh"]), P(g["features_sh"]), P(m1["features_sh"]), P(m2["features_sh"])), "plain_steps sh")
            keys = list(p) if not agnostic else ["means"]
            for k in keys:
                out[f"{tag}_p{step}_{k}"] = p[k].cpu().numpy()
    # 16-bit moments of the five non-SH arrays (the non_sh_quant kernel), three steps from a zero state:
    # "nq" = DC regulariser only, "nqx" = all regularisers + per-splat step counters
    for tag, use_ex in (("nq", False), ("nqx", True)):
        p = {k: dev(v.reshape(-1)) for k, v in inp["params"].items() if k != "features_sh"}
        widths = dict(means=3, quats=4, scales=3, opacities=1, features_dc=3)
        order = ("means", "quats", "scales", "opacities", "features_dc")
        nblk = (n + 255) // 256
        packed = {k: torch.zeros(n * widths[k] * 4, dtype=torch.uint8, device=DEV) for k in order}
        bounds = {k: torch.zeros(nblk * 4, dtype=torch.float32, device=DEV) for k in order}
        pk = (C.c_void_p * 5)(*[packed[k].data_ptr() for k in order])
        bd = (C.c_void_p * 5)(*[bounds[k].data_ptr() for k in order])
        for step, grads in enumerate(inp["grads"], start=1):
            g = {k: dev(v.reshape(-1)) for k, v in grads.items() if k != "features_sh"}
            check(ref.ref_adam_geometry_q16(C.c_int64(n), step, C.c_float(inp["grad_scale"]), 0, C.c_float(lr["lr_means"]), C.c_float(lr["lr_quats"]),
                                            C.c_float(lr["lr_scales"]), C.c_float(lr["lr_opacities"]), C.c_float(lr["lr_features_dc"]),
                                            C.c_float(inp["nq_sh_reg_weight"]),
                                            P(p["means"]), P(g["means"]), P(p["quats"]), P(g["quats"]), P(p["scales"]), P(g["scales"]),
                                            P(p["opacities"]), P(g["opacities"]), P(p["features_dc"]), P(g["features_dc"]), pk, bd,
                                            d_reg_host.ctypes.data_as(C.c_void_p) if use_ex else None, P(d_steps) if use_ex else None),
                  "ref_adam_geometry_q16")
            for k in order:
                out[f"{tag}_p{step}_{k}"] = p[k].cpu().numpy()
                out[f"{tag}_q{step}_{k}"] = packed[k].cpu().numpy()
                out[f"{tag}_b{step}_{k}"] = bounds[k].cpu().numpy()
    # doubly quantised SH step with per-splat counters (16-bit values), one step from the seeded state;
    # the counters are padded because the kernel reads steps[idx / stride] in every thread of its last block
    q = inp["qq16"]
    n_sp = (q["numel"] + 44) // 45
    steps_q = torch.ones(n_sp + 8, dtype=torch.int32, device=DEV)
    steps_q[:n_sp] = dev(np.resize(ex["steps"], n_sp))
    vp, vb, op, ob = dev(q["value_packed"]), dev(q["value_bounds"]), dev(q["optim_packed"]), dev(q["optim_bounds"])
    d_grad = dev(q["grads"][0])
    check(ref.ref_adam_qq_steps(C.c_int64(q["numel"]), P(steps_q), 45, C.c_float(lr["lr_features_sh"]), C.c_float(0.0), C.c_float(inp["grad_scale"]), 0, 16,
                                P(d_grad), P(op), P(ob), P(vp), P(vb)), "ref_adam_qq_steps")
    out["qqs_value_packed"], out["qqs_value_bounds"] = vp.cpu().numpy(), vb.cpu().numpy()
    out["qqs_optim_packed"], out["qqs_optim_bounds"] = op.cpu().numpy(), ob.cpu().numpy()
    # 4-bit optimiser state (one byte per cell): fp32 values for three steps from a zero state (the q8 inputs),
    # and 16-bit values for one step from the seeded state (the qq16 inputs)
    q = inp["q8"]
    nb = (q["numel"] + 255) // 256
    x_buf = torch.zeros(nb * 256, dtype=torch.float32, device=DEV)      # whole blocks: see the note above
    x = x_buf[:q["numel"]]
    x.copy_(dev(q["x0"]))
    op = torch.zeros(nb * 256, dtype=torch.uint8, device=DEV)
    ob = torch.zeros(nb * 4, dtype=torch.float32, device=DEV)
    for step, grad in enumerate(q["grads"], start=1):
        d_grad = dev(grad)
        check(ref.ref_adam_q4(C.c_int64(q["numel"]), step, C.c_float(lr["lr_features_sh"]), C.c_float(0.0), C.c_float(inp["grad_scale"]), 0,
                              P(x), P(d_grad), P(op), P(ob)), "ref_adam_q4")
        out[f"q4_s{step}_x"] = x.cpu().numpy()
        out[f"q4_s{step}_optim_packed"] = op[:q["numel"]].cpu().numpy()
        out[f"q4_s{step}_optim_bounds"] = ob.cpu().numpy()
    q = inp["qq16"]
    vp, vb = dev(q["value_packed"]), dev(q["value_bounds"])
    op = torch.zeros(q["numel"], dtype=torch.uint8, device=DEV)
    ob = torch.zeros(((q["numel"] + 255) // 256) * 4, dtype=torch.float32, device=DEV)
    for step, grad in enumerate(q["grads"][:2], start=1):
        d_grad = dev(grad)
        check(ref.ref_adam_qq_o4(C.c_int64(q["numel"]), step, C.c_float(lr["lr_features_sh"]), C.c_float(0.0), C.c_float(inp["grad_scale"]), 0, 16,
                                 P(d_grad), P(op), P(ob), P(vp), P(vb)), "ref_adam_qq_o4")
        out[f"qq16o4_s{step}_value_packed"], out[f"qq16o4_s{step}_value_bounds"] = vp.cpu().numpy(), vb.cpu().numpy()
        out[f"qq16o4_s{step}_optim_packed"], out[f"qq16o4_s{step}_optim_bounds"] = op.cpu().numpy(), ob.cpu().numpy()
    np.savez_compressed(os.path.join(out_dir, "adam.npz"), **out)


def run_accum(ref, out_dir):
    """Per-splat densification weights of the raster backward pass (max, sum, average) on the committed intermediate
    arrays of two fixture scenes: accum.npz."""
    out = {}
    for name in ACCUM_CASES:
        cfg, sp, vm, K = build_case(name)
        gold = np.load(os.path.join(HERE, f"{name}.npz"))
        I, W, H, n = vm.shape[0], cfg.width, cfg.height, cfg.n_splats
        m, M, P_ = I * n, gold["sorted_flat"].size, I * H * W
        xy, depth, conic, opac, rgb = (dev(gold[k]) for k in ("xy", "depth", "conic", "opac", "rgb"))
        offs, fl = dev(gold["offsets"]), dev(gold["sorted_flat"])
        r_rgb, r_depth, r_T, r_last = (dev(gold[k]) for k in ("render_rgb", "render_depth", "render_T", "last_ids"))
        v_rgb, v_depth, v_T = (dev(a) for a in raster_cotangents(name, P_))
        wmap = dev(accum_weight_map(name, P_))
        for mode, tag in ((1, "max"), (2, "sum"), (3, "avg")):
            z = lambda *shape: torch.zeros(*shape, dtype=torch.float32, device=DEV)
            g_xy, g_depth, g_conic, g_opac, g_rgb = z(m, 2), z(m), z(m, 3), z(m), z(m, 3)
            acc, den = z(n), z(n)
            check(ref.ref_raster_bwd_accum(mode, I, n, M, W, H, P(xy), P(depth), P(conic), P(opac), P(rgb), P(offs), P(fl), P(r_rgb), P(r_depth),
                                           P(r_T), P(r_last), P(v_rgb), P(v_depth), P(v_T), P(g_xy), P(g_depth), P(g_conic), P(g_opac), P(g_rgb),
                                           P(wmap), P(acc), P(den)), "ref_raster_bwd_accum")
            out[f"{name}_{tag}"] = acc.cpu().numpy()
            if mode == 3:
                out[f"{name}_avg_den"] = den.cpu().numpy()
    np.savez_compressed(os.path.join(out_dir, "accum.npz"), **out)


def run_quant_proj(ref, out_dir):
    """Projection forward and backward of the reference's kernels reading quantised SH (8/16-bit codes, both bound
    layouts).  Only what the SH storage changes is stored: the colours, the validity boxes, and the six gradient arrays
    for the screen-space cotangents the fp32 fixture of the same scene holds."""
    name = QUANT_SCENE
    cfg, sp, vm, K = build_case(name)
    gold = np.load(os.path.join(HERE, f"{name}.npz"))
    n, W, H, I = cfg.n_splats, cfg.width, cfg.height, vm.shape[0]
    m = I * n
    d = {k: dev(v.reshape(-1)) for k, v in sp.items()}
    d_vm, d_K = dev(vm), dev(K)
    z = lambda *s, dt=torch.float32: torch.zeros(*s, dtype=dt, device=DEV)
    v = {k: dev(gold[k]) for k in ("v_xy", "v_depth", "v_conic", "v_opac", "v_rgb")}
    out = {}
    for tag in QUANT_CASES:
        codes, bounds, bits, stride_arg = quant_sh_inputs(tag, n)
        d_codes, d_bounds = dev(codes.view(np.uint8)), dev(bounds)
        aabb, depths, radii = z(m, 4), z(m), z(n)
        xy, depth, conic, opac, rgb = z(m, 2), z(m), z(m, 3), z(m), z(m, 3)
        check(ref.ref_project_fwd(I, n, W, H, P(d["means"]), P(d["quats"]), P(d["scales"]), P(d["opacities"]), P(d["features_dc"]), None,
                                  P(d_codes), P(d_bounds), bits, C.c_int64(stride_arg), P(d_vm), P(d_K), P(aabb), P(depths), P(radii),
                                  P(xy), P(depth), P(conic), P(opac), P(rgb)), "ref_project_fwd (quantised SH)")
        out[f"{tag}_aabb"], out[f"{tag}_rgb"], out[f"{tag}_conic"] = aabb.cpu().numpy(), rgb.cpu().numpy(), conic.cpu().numpy()
        g = {k: torch.zeros_like(t) for k, t in d.items()}
        check(ref.ref_project_bwd(I, n, W, H, P(d["means"]), P(d["quats"]), P(d["scales"]), P(d["opacities"]), P(d["features_dc"]), None,
                                  P(d_codes), P(d_bounds), bits, C.c_int64(stride_arg), P(d_vm), P(d_K), P(aabb),
                                  P(v["v_xy"]), P(v["v_depth"]), P(v["v_conic"]), P(v["v_opac"]), P(v["v_rgb"]),
                                  P(g["means"]), P(g["quats"]), P(g["scales"]), P(g["opacities"]), P(g["features_dc"]), P(g["features_sh"])),
              "ref_project_bwd (quantised SH)")
        for k, t in g.items():
            out[f"{tag}_g_{k}"] = t.cpu().numpy()
    np.savez_compressed(os.path.join(out_dir, "quant_proj.npz"), **out)


def run_dist_proj(ref, out_dir):
    """Projection forward and backward of the reference's kernels with a lens-distortion tier, for every (camera model,
    tier) pair it instantiates: all forward outputs, and the six gradient arrays for seeded screen-space cotangents."""
    out = {}
    for name in DIST_CASES:
        cfg, sp, vm, K, model, tier, rows, v = dist_case_inputs(name)
        n, W, H, I = cfg.n_splats, cfg.width, cfg.height, vm.shape[0]
        m = I * n
        d = {k: dev(val.reshape(-1)) for k, val in sp.items()}
        d_vm, d_K, d_rows = dev(vm), dev(K), dev(rows)
        z = lambda *s, dt=torch.float32: torch.zeros(*s, dtype=dt, device=DEV)
        aabb, depths, radii = z(m, 4), z(m), z(n)
        xy, depth, conic, opac, rgb = z(m, 2), z(m), z(m, 3), z(m), z(m, 3)
        check(ref.ref_project_fwd_dist(model, tier, I, n, W, H, P(d["means"]), P(d["quats"]), P(d["scales"]), P(d["opacities"]), P(d["features_dc"]),
                                       P(d["features_sh"]), P(d_vm), P(d_K), P(d_rows), P(aabb), P(depths), P(radii),
                                       P(xy), P(depth), P(conic), P(opac), P(rgb)), "ref_project_fwd_dist " + name)
        for k, t in dict(aabb=aabb, depths=depths, radii=radii, xy=xy, depth=depth, conic=conic, opac=opac, rgb=rgb).items():
            out[f"{name}_{k}"] = t.cpu().numpy()
        dv = {k: dev(val) for k, val in v.items()}
        g = {k: torch.zeros_like(t) for k, t in d.items()}
        check(ref.ref_project_bwd_dist(model, tier, I, n, W, H, P(d["means"]), P(d["quats"]), P(d["scales"]), P(d["opacities"]), P(d["features_dc"]),
                                       P(d["features_sh"]), P(d_vm), P(d_K), P(d_rows), P(aabb),
                                       P(dv["v_xy"]), P(dv["v_depth"]), P(dv["v_conic"]), P(dv["v_opac"]), P(dv["v_rgb"]),
                                       P(g["means"]), P(g["quats"]), P(g["scales"]), P(g["opacities"]), P(g["features_dc"]), P(g["features_sh"])),
              "ref_project_bwd_dist " + name)
        for k, t in g.items():
            out[f"{name}_g_{k}"] = t.cpu().numpy()
        print(name, "visible", int((aabb[:, 2] > aabb[:, 0]).sum().item()), "of", m)
    np.savez_compressed(os.path.join(out_dir, "dist_proj.npz"), **out)


def run_fpbo(ref, out_dir):
    """The reference's fused projection-backward + optimiser kernel (level 0, unpacked), two passes per run from zero moments:
    parameters after each pass, moments after the second."""
    cfg, sp, vm, K = build_case(FPBO_SCENE)
    gold = np.load(os.path.join(HERE, f"{FPBO_SCENE}.npz"))
    n, W, H, I = cfg.n_splats, cfg.width, cfg.height, vm.shape[0]
    lr = cfg.lrs
    lrs = np.array([lr["lr_means"], lr["lr_quats"], lr["lr_scales"], lr["lr_opacities"], lr["lr_features_dc"], lr["lr_features_sh"]], np.float32)
    d_vm, d_K, d_aabb = dev(vm), dev(K), dev(gold["aabb"])
    v = {k: dev(gold[k]) for k in ("v_xy", "v_depth", "v_conic", "v_opac", "v_rgb")}
    extra = fpbo_inputs(n)
    d_radii, d_steps = dev(extra["radii"]), dev(extra["steps"])
    order = ("means", "quats", "scales", "opacities", "features_dc", "features_sh")
    out = {}
    for tag, run in FPBO_RUNS.items():
        p = {k: dev(sp[k].reshape(-1)) for k in order}
        g1 = {k: torch.zeros_like(t) for k, t in p.items()}
        g2 = {k: torch.zeros_like(t) for k, t in p.items()}
        reg = np.array(run["reg"], np.float32)
        for step in (1, 2):
            zero = {k: torch.zeros_like(t) for k, t in p.items()}
            steps_t = None
            if run["steps"]:
                steps_t = (d_steps + (step - 1)).contiguous()
            check(ref.ref_fpbo(I, n, W, H, *[P(p[k]) for k in order], P(d_vm), P(d_K), P(d_aabb),
                               P(v["v_xy"]), P(v["v_depth"]), P(v["v_conic"]), P(v["v_opac"]), P(v["v_rgb"]),
                               *[P(zero[k]) for k in order], *[P(g1[k]) for k in order], *[P(g2[k]) for k in order],
                               P(d_radii), lrs.ctypes.data_as(C.c_void_p), reg.ctypes.data_as(C.c_void_p), C.c_float(run["sh_reg"]),
                               run["agnostic"], step, P(steps_t) if steps_t is not None else None), "ref_fpbo " + tag)
            for k in order:
                out[f"{tag}_p{step}_{k}"] = p[k].cpu().numpy()
        for k in order:
            out[f"{tag}_g1_{k}"], out[f"{tag}_g2_{k}"] = g1[k].cpu().numpy(), g2[k].cpu().numpy()
    np.savez_compressed(os.path.join(out_dir, "fpbo.npz"), **out)


def run_fpbo_l1(ref, out_dir):
    """The reference's fused projection-backward + optimiser kernel at quantisation level 1 (16-bit SH values, 8-bit SH optimiser
    state, one bound per 256 splats; in one run the other moments as 16-bit codes too), two passes per run from the zero state:
    after each pass the five fp32 parameter arrays, the SH value codes and bounds, the SH state codes and bounds; after the
    second the other moments (fp32 arrays or codes and bounds)."""
    cfg, sp, vm, K = build_case(FPBO_SCENE)
    gold = np.load(os.path.join(HERE, f"{FPBO_SCENE}.npz"))
    n, W, H, I = cfg.n_splats, cfg.width, cfg.height, vm.shape[0]
    blocks = (n + 255) // 256
    lr = cfg.lrs
    lrs = np.array([lr["lr_means"], lr["lr_quats"], lr["lr_scales"], lr["lr_opacities"], lr["lr_features_dc"], lr["lr_features_sh"]], np.float32)
    d_vm, d_K, d_aabb = dev(vm), dev(K), dev(gold["aabb"])
    v = [dev(gold[k]) for k in ("v_xy", "v_depth", "v_conic", "v_opac", "v_rgb")]
    extra = fpbo_inputs(n)
    d_radii, d_steps = dev(extra["radii"]), dev(extra["steps"])
    five = ("means", "quats", "scales", "opacities", "features_dc")
    widths = dict(means=3, quats=4, scales=3, opacities=1, features_dc=3)
    codes0, bounds0 = encode_splat_blocks(sp["features_sh"].reshape(n, 45), 16)
    ptrs = lambda ts: (C.c_void_p * len(ts))(*[t.data_ptr() if t is not None else 0 for t in ts])
    out = {}
    for tag, run in FPBO_L1_RUNS.items():
        p = {k: dev(sp[k].reshape(-1)) for k in five}
        sh_fp32 = torch.zeros(n * 45, device=DEV)
        vcodes, vbounds = dev(codes0.view(np.uint8)), dev(bounds0)
        ocodes, obounds = torch.zeros(n * 45 * 2, dtype=torch.uint8, device=DEV), torch.zeros(blocks * 4, device=DEV)
        g1 = {k: torch.zeros_like(t) for k, t in p.items()}
        g2 = {k: torch.zeros_like(t) for k, t in p.items()}
        nq_p = {k: torch.zeros(n * widths[k] * 4, dtype=torch.uint8, device=DEV) for k in five}
        nq_b = {k: torch.zeros(blocks * 4, device=DEV) for k in five}
        reg = np.array(run["reg"], np.float32)
        for step in (1, 2):
            zero = [torch.zeros_like(p[k]) for k in five] + [torch.zeros(n * 45, device=DEV)]
            steps_t = (d_steps + (step - 1)).contiguous() if run["steps"] else None
            check(ref.ref_fpbo_l1(I, n, W, H, run["degree"], ptrs([p[k] for k in five] + [sh_fp32]), P(d_vm), P(d_K), P(d_aabb), ptrs(v), ptrs(zero),
                                  ptrs([g1[k] for k in five]), ptrs([g2[k] for k in five]), P(ocodes), P(obounds), P(vcodes), P(vbounds),
                                  ptrs([nq_p[k] for k in five]) if run["nq"] else None, ptrs([nq_b[k] for k in five]) if run["nq"] else None,
                                  P(d_radii), lrs.ctypes.data_as(C.c_void_p), reg.ctypes.data_as(C.c_void_p), C.c_float(run["sh_reg"]),
                                  run["agnostic"], step, P(steps_t) if steps_t is not None else None), "ref_fpbo_l1 " + tag)
            for k in five:
                out[f"{tag}_p{step}_{k}"] = p[k].cpu().numpy()
            out[f"{tag}_s{step}_value_codes"], out[f"{tag}_s{step}_value_bounds"] = vcodes.cpu().numpy().view(np.uint16), vbounds.cpu().numpy()
            out[f"{tag}_s{step}_optim_codes"], out[f"{tag}_s{step}_optim_bounds"] = ocodes.cpu().numpy(), obounds.cpu().numpy()
            if run["nq"]:
                for k in five:
                    out[f"{tag}_s{step}_nq_{k}"], out[f"{tag}_s{step}_nqb_{k}"] = nq_p[k].cpu().numpy(), nq_b[k].cpu().numpy()
        if not run["nq"]:
            for k in five:
                out[f"{tag}_g1_{k}"], out[f"{tag}_g2_{k}"] = g1[k].cpu().numpy(), g2[k].cpu().numpy()
        assert not sh_fp32.any().item()          # the fp32 SH array is not this level's storage
    np.savez_compressed(os.path.join(out_dir, "fpbo_l1.npz"), **out)


def run_sh_degree(ref, out_dir):
    """Projection forward and backward of the reference's Vanilla3DGS<0>, <1> and <2> kernels (the SH degree warm-up) on the
    ring2 scene with its 15-coefficient SH rows: the colours, the validity boxes and the six gradient arrays for the
    screen-space cotangents of the degree-3 fixture."""
    name = QUANT_SCENE
    cfg, sp, vm, K = build_case(name)
    gold = np.load(os.path.join(HERE, f"{name}.npz"))
    n, W, H, I = cfg.n_splats, cfg.width, cfg.height, vm.shape[0]
    m = I * n
    d = {k: dev(v.reshape(-1)) for k, v in sp.items()}
    d_vm, d_K = dev(vm), dev(K)
    z = lambda *s, dt=torch.float32: torch.zeros(*s, dtype=dt, device=DEV)
    v = {k: dev(gold[k]) for k in ("v_xy", "v_depth", "v_conic", "v_opac", "v_rgb")}
    out = {}
    for deg in (0, 1, 2):
        aabb, depths, radii = z(m, 4), z(m), z(n)
        xy, depth, conic, opac, rgb = z(m, 2), z(m), z(m, 3), z(m), z(m, 3)
        check(ref.ref_project_fwd_deg(deg, I, n, W, H, P(d["means"]), P(d["quats"]), P(d["scales"]), P(d["opacities"]), P(d["features_dc"]),
                                      P(d["features_sh"]), P(d_vm), P(d_K), P(aabb), P(depths), P(radii),
                                      P(xy), P(depth), P(conic), P(opac), P(rgb)), "ref_project_fwd_deg")
        out[f"d{deg}_aabb"], out[f"d{deg}_rgb"] = aabb.cpu().numpy(), rgb.cpu().numpy()
        g = {k: torch.zeros_like(t) for k, t in d.items()}
        check(ref.ref_project_bwd_deg(deg, I, n, W, H, P(d["means"]), P(d["quats"]), P(d["scales"]), P(d["opacities"]), P(d["features_dc"]),
                                      P(d["features_sh"]), P(d_vm), P(d_K), P(aabb),
                                      P(v["v_xy"]), P(v["v_depth"]), P(v["v_conic"]), P(v["v_opac"]), P(v["v_rgb"]),
                                      P(g["means"]), P(g["quats"]), P(g["scales"]), P(g["opacities"]), P(g["features_dc"]), P(g["features_sh"])),
              "ref_project_bwd_deg")
        for k, t in g.items():
            out[f"d{deg}_g_{k}"] = t.cpu().numpy()
    np.savez_compressed(os.path.join(out_dir, "sh_degree.npz"), **out)


def run_packed_proj(ref, out_dir):
    """The reference's packed projection (mask, scan, compacting kernel) and the packed mode of its projection backward
    kernel on two scenes, fp32 SH and one quantised layout: ids, count and the packed outputs; the backward pass takes the
    fp32 fixture's screen-space cotangents gathered at the packed pairs."""
    out = {}
    for name, tag in (("ring2", None), ("dense1", None), ("ring2", "q16_cell")):
        cfg, sp, vm, K = build_case(name)
        gold = np.load(os.path.join(HERE, f"{name}.npz"))
        n, W, H, I = cfg.n_splats, cfg.width, cfg.height, vm.shape[0]
        m = I * n
        d = {k: dev(v.reshape(-1)) for k, v in sp.items()}
        d_vm, d_K = dev(vm), dev(K)
        z = lambda *s, dt=torch.float32: torch.zeros(*s, dtype=dt, device=DEV)
        sh_args = (P(d["features_sh"]), None, None, 32, C.c_int64(256))
        if tag:
            codes, bounds, bits, stride_arg = quant_sh_inputs(tag, n)
            d_codes, d_bounds = dev(codes.view(np.uint8)), dev(bounds)
            sh_args = (None, P(d_codes), P(d_bounds), bits, C.c_int64(stride_arg))
        mask, scan = z(m, dt=torch.bool), z(m, dt=torch.int64)
        cam_ids, g_ids = z(m, dt=torch.int32), z(m, dt=torch.int32)
        aabb, depths, radii = z(m, 4), z(m), z(n)
        xy, depth, conic, opac, rgb = z(m, 2), z(m), z(m, 3), z(m), z(m, 3)
        nnz = C.c_int64(0)
        check(ref.ref_project_fwd_packed(I, n, W, H, P(d["means"]), P(d["quats"]), P(d["scales"]), P(d["opacities"]), P(d["features_dc"]), *sh_args,
                                         P(d_vm), P(d_K), P(mask), P(scan), C.c_int64(m), P(cam_ids), P(g_ids), P(aabb), P(depths), P(radii),
                                         P(xy), P(depth), P(conic), P(opac), P(rgb), C.byref(nnz)), "ref_project_fwd_packed")
        V = nnz.value
        key = f"{name}_{tag}" if tag else name
        out[f"{key}_nnz"] = np.array([V], np.int64)
        for k, t in dict(camera_ids=cam_ids, gaussian_ids=g_ids, aabb=aabb, depths=depths, xy=xy, depth=depth, conic=conic, opac=opac, rgb=rgb).items():
            out[f"{key}_{k}"] = t[:V].cpu().numpy()
        out[f"{key}_radii"] = radii.cpu().numpy()
        # backward, packed mode: cotangents of the unpacked fixture gathered at the packed pairs
        pair = (cam_ids[:V].long() * n + g_ids[:V].long())
        pv = {k: dev(gold[k])[pair].contiguous() for k in ("v_xy", "v_depth", "v_conic", "v_opac", "v_rgb")}
        g = {k: torch.zeros_like(t) for k, t in d.items()}
        check(ref.ref_project_bwd_packed(I, n, V, W, H, P(d["means"]), P(d["quats"]), P(d["scales"]), P(d["opacities"]), P(d["features_dc"]), *sh_args,
                                         P(d_vm), P(d_K), P(cam_ids), P(g_ids), P(aabb),
                                         P(pv["v_xy"]), P(pv["v_depth"]), P(pv["v_conic"]), P(pv["v_opac"]), P(pv["v_rgb"]),
                                         P(g["means"]), P(g["quats"]), P(g["scales"]), P(g["opacities"]), P(g["features_dc"]), P(g["features_sh"])),
              "ref_project_bwd_packed")
        for k, t in g.items():
            out[f"{key}_g_{k}"] = t.cpu().numpy()
    np.savez_compressed(os.path.join(out_dir, "packed_proj.npz"), **out)


def main():
    out_dir = sys.argv[1] if len(sys.argv) > 1 else HERE
    os.makedirs(out_dir, exist_ok=True)
    ref = C.CDLL(os.path.join(ROOT, "oracle", "_ref", "libssb_ref.so"))
    only = set(sys.argv[2:])
    for name in list(CASES) + list(WIDE_CASES):
        if not only or name in only:
            run_case(ref, name, out_dir)
    if not only or "ssim" in only:
        run_loss(ref, out_dir)
    if not only or "adam" in only:
        run_adam(ref, out_dir)
    if not only or "dist_proj" in only:
        run_dist_proj(ref, out_dir)
    if not only or "sh_degree" in only:
        run_sh_degree(ref, out_dir)
    if not only or "fpbo" in only:
        run_fpbo(ref, out_dir)
    if not only or "fpbo_l1" in only:
        run_fpbo_l1(ref, out_dir)
    if not only or "ssim_map" in only:
        run_loss_map(ref, out_dir)
    if not only or "ssim_masked" in only:
        run_loss_masked(ref, out_dir)
    if not only or "loss_multi" in only:
        run_loss_multi(ref, out_dir)
    if not only or "densify_split" in only:
        run_densify_split(ref, out_dir)
    if not only or "densify" in only:
        run_densify(ref, out_dir)
    if not only or "tiles_live" in only:
        run_tiles_live(ref, out_dir)
    if not only or "accum" in only:
        run_accum(ref, out_dir)
    if not only or "quant_proj" in only:
        run_quant_proj(ref, out_dir)
    if not only or "packed_proj" in only:
        run_packed_proj(ref, out_dir)
    print("wrote fixtures to", out_dir)


if __name__ == "__main__":
    main()
