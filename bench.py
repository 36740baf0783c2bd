#!/usr/bin/env python
"""Benchmark of the training hot path: train iterations per second on the
"mid" scene (1,000,000 SH-degree-3 Gaussians with 16-bit quantised SH values and
8-bit quantised SH optimiser state, a batch of sixteen 1920x1080 pinhole views).

One iteration = forward + L1/SSIM loss + backward of every view of the batch
(one camera per sub-batch, gradients summed), a sum all-reduce of the gradients
when several GPUs share the batch, and one Adam pass over all parameters.

    python bench.py --gpus N --steps K --warmup W            # this library
    python bench.py --impl reference --steps K --warmup W     # CPU restatement, host cores

Prints ONE JSON line (rank 0).  Inputs are seeded synthetic data of the
configuration's shapes and distributions.
"""
import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

_JSON_FD = None


def claim_stdout():
    """Keeps stdout to the one JSON line: libraries (NCCL's version banner among them) write to file
    descriptor 1, so that descriptor is pointed at stderr and the JSON line goes to a saved copy."""
    global _JSON_FD
    sys.stdout.flush()
    _JSON_FD = os.dup(1)
    os.dup2(2, 1)


def emit(line):
    data = (json.dumps(line) + "\n").encode()
    os.write(_JSON_FD if _JSON_FD is not None else 1, data)

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "train iters/sec (fwd+bwd+SSIM+Adam), 1M SH3 Gaussians @1080p"
UNIT = "iters/s"
WORKLOAD = "mid_1m"


# DRAM bytes one launch moves (dram__bytes_read.sum + dram__bytes_write.sum): RECORDED CONSTANTS from one ncu
# pass over this file's own command on the mid_1m workload, one view per launch (a stage of several kernels:
# their sum).  They are not measured by the run that prints them (a profiler cannot run inside a timed
# benchmark); the JSON line says so in `traffic_source`.
NCU_TRAFFIC_MID1M = {"project_fwd": 184.1e6, "tile_keys": 190.5e6, "sort": 35.6e6, "raster_fwd": 68.3e6,
                     "loss": 51.5e6, "raster_bwd": 111.2e6, "project_bwd": 426.4e6, "adam": 846.8e6}
# FP32 operations one launch (one view) executes, thread level, FMA counted as two: 2 * ffma + fadd + fmul of
# smsp__sass_thread_inst_executed_op_{ffma,fadd,fmul}_pred_on.sum from the same kind of capture.  RECORDED CONSTANTS like
# the traffic above.  The rasterisers and the loss kernel are arithmetic kernels whose working set sits in L2: their
# roofline is the FP32 pipe, not HBM.
NCU_FLOP_MID1M = {"raster_fwd": 3.975e9, "loss": 4.308e9, "raster_bwd": 10.110e9}
# FP32 peak: 148 SMs x 128 lanes x 2 (FMA) x the maximum SM clock; there is no measured FP32 figure for this pool.
FP32_LANES = 148 * 128


def shard(total, world, rank):
    """Contiguous block of views owned by `rank`."""
    base, rem = divmod(total, world)
    start = rank * base + min(rank, rem)
    return start, base + (1 if rank < rem else 0)


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.path = tempfile.mktemp(prefix="ssb_clocks_", suffix=".csv")
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(gpu_index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "50"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1])); mx.append(float(f[2]))
                except ValueError:
                    continue
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except OSError:
            pass
        if sm:
            out = {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(np.max(mx)), "reasons": sorted(reasons), "samples": len(sm)}
        return out


def stage_bytes(stage, n, visible, pairs, pixels, tiles, quant_bits, sort_passes):
    """Algorithmic bytes one launch (one view) of a stage moves."""
    sh_b = 45 * (4 if quant_bits == 32 else quant_bits // 8)
    if stage == "project_fwd":
        return visible * (56 + sh_b + 60) + (n - visible) * 56
    # the step bins pairs by tile and sorts each tile's list (ssb_intersect_tiles): the key stage reads 44 B per
    # (view, splat) and writes one 8-byte (depth, pair) word per pair plus the tile table; the sort stage reads
    # that word and writes the 4-byte sorted pair index; the ranges come out of the key stage's scan
    if stage == "tile_keys":
        return n * 44 + pairs * 8 + tiles * 8
    if stage == "sort":
        return pairs * 12
    if stage == "tile_ranges":
        return 0
    if stage == "raster_fwd":
        return pairs * 40 + pixels * 24
    if stage == "loss":
        return pixels * 36
    if stage == "raster_bwd":
        return pixels * 44 + pairs * 40
    if stage == "project_bwd":
        return visible * (56 + sh_b + 40 + 16 + 236) + (n - visible) * 16
    raise KeyError(stage)


def adam_bytes(n, quant_bits):
    if quant_bits == 32:
        return n * 59 * 28
    value_b = quant_bits // 8
    return n * (14 * 28 + 45 * (4 + 2 * value_b + 2 * 2))


# --------------------------------------------------------------------------
def oracle_view_seconds(cfg, splats, vm, K, view, shq):
    from oracle import pyoracle as O
    from spirula_studio_b200 import scenes
    t0 = time.perf_counter()
    _, model, W, H, _, _ = scenes.view_kind(cfg, view)
    n = cfg.n_splats
    ch = O.forward_chain(splats, vm[view:view + 1], K[view:view + 1], W, H, shq=shq, model=model)
    gt = scenes.make_target(cfg, view)
    t_gen = time.perf_counter()
    v, _ = O.loss_l1_ssim(ch["render"]["rgb"], gt.reshape(-1, 3), 1, H, W, 0.8, 0.2)
    gs = O.raster_bwd(ch["proj"], ch["offsets"], ch["sorted_vals"], 1, n, W, H, ch["render"], v)
    g = O.project_bwd(splats, vm[view:view + 1], K[view:view + 1], W, H, ch["proj"]["aabb"], gs, shq=shq, model=model)
    return time.perf_counter() - t0, g, t_gen


def oracle_adam_seconds(cfg, splats, grads, state, step, shq):
    from oracle import pyoracle as O
    t0 = time.perf_counter()
    p, m1, m2 = state
    lr = cfg.lrs
    O.adam_geometry(p, grads, m1, m2, step, lr, grad_scale=1.0 / cfg.n_views)
    O.adam_plain(p["features_dc"], grads["features_dc"], m1["features_dc"], m2["features_dc"], step, lr["lr_features_dc"], 0.0,
                 0.5 / 0.28209479177387814, 1.0 / cfg.n_views)
    if shq is None:
        O.adam_plain(p["features_sh"], grads["features_sh"], m1["features_sh"], m2["features_sh"], step, lr["lr_features_sh"], 0.0, 0.0,
                     1.0 / cfg.n_views)
    else:
        O.adam_qq(grads["features_sh"].reshape(-1), shq["optim_packed"], shq["optim_bounds"], shq["packed"], shq["bounds"], shq["bits"], step,
                  lr["lr_features_sh"], grad_scale=1.0 / cfg.n_views)
    return time.perf_counter() - t0


def cpu_port_run(cfg, steps, warmup):
    """Times the CPU restatement: each step = one view of the batch (all stages) + one Adam pass.
    Uses every host core whatever OMP_NUM_THREADS says (launchers such as torchrun set it to 1)."""
    from oracle import pyoracle as O
    from spirula_studio_b200 import scenes
    O.set_num_threads(len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1))
    splats = scenes.make_splats(cfg)
    vm, K = scenes.make_cameras(cfg)
    shq = None
    if cfg.sh_value_bits in (8, 16):
        packed, bounds = O.quant_encode(splats["features_sh"], cfg.sh_value_bits)
        cells = cfg.n_splats * 45
        shq = dict(packed=packed, bounds=bounds, bits=cfg.sh_value_bits, bounds_stride=256,
                   optim_packed=np.zeros(cells * 2, np.uint8), optim_bounds=np.zeros(((cells + 255) // 256) * 4, np.float32))
    state = ({k: v.copy() for k, v in splats.items()}, {k: np.zeros_like(v) for k, v in splats.items()},
             {k: np.zeros_like(v) for k, v in splats.items()})
    tv, ta = [], []
    for i in range(warmup + steps):
        t, g, _ = oracle_view_seconds(cfg, splats, vm, K, i % cfg.n_views, shq)
        a = oracle_adam_seconds(cfg, splats, g, state, i + 1, shq)
        if i >= warmup:
            tv.append(t); ta.append(a)
    t_view, t_adam = float(np.mean(tv)), float(np.mean(ta))
    t_iter = cfg.n_views * t_view + t_adam
    return 1.0 / t_iter, t_iter, t_view, t_adam, O.num_threads()


def run_reference(args, cfg, rank):
    if rank != 0:
        return
    value, t_iter, t_view, t_adam, cores = cpu_port_run(cfg, args.steps, args.warmup)
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "impl": "reference", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * t_iter, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": cfg.name, "n_splats": cfg.n_splats, "views_per_iteration": cfg.n_views, "resolution": [cfg.width, cfg.height],
                   "sh_value_bits": cfg.sh_value_bits, "sh_optim_bits": cfg.sh_optim_bits},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"each step = 1 of {cfg.n_views} views at full size through every stage ({t_view:.2f} s) plus one Adam pass "
                                   f"({t_adam:.2f} s); iteration time = {cfg.n_views} x view + Adam"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference has no CPU implementation of this path and its Vulkan backend cannot run here (no graphics stack); "
                "this arm times the CPU restatement under oracle/ on the host cores",
    }
    emit(line)


# --------------------------------------------------------------------------
def run_ours(args, cfg, rank, world, local_rank):
    import torch
    import torch.distributed as dist

    from spirula_studio_b200 import lib as L, scenes
    from spirula_studio_b200.trainer import Trainer

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the library has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = f"cuda:{local_rank}"
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device(dev))
    lib = L.load()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    total_views = cfg.n_views
    v0, nv = shard(total_views, world, rank)
    splats = scenes.make_splats(cfg)
    vm, K = scenes.make_cameras(cfg)
    # "multimem" (own fused kernels through the NVSwitch multicast address; falls back to "peer" where symmetric memory
    # cannot be set up), "peer" (the same kernels with per-peer loads and stores) or "nccl" (all-reduce + full Adam)
    grad_sync = os.environ.get("SSB_GRAD_SYNC", "multimem")
    # SSB_FUSED_BACKWARD=1 (one GPU): the projection backward of all views runs together with the optimiser, so the world
    # gradients never travel through HBM.  Off by default: at mid_1m it measured 37.5 iterations/s against 39.5, because the
    # projection backward is bound by instruction issue, not by the gradient traffic the fusion removes, and the per-view
    # kernels hide behind the next view's forward pass on the second stream while the fused pass runs exposed at the end.
    fused = os.environ.get("SSB_FUSED_BACKWARD", "0") != "0"
    # SSB_STOCK_FLAGS=1: the reference trainer's stock optimiser flags (regularisers, scale-agnostic mean, per-splat step counters,
    # 16-bit moments for the non-SH arrays) instead of the plain Adam step the headline is quoted on; with SSB_FUSED_BACKWARD=1
    # and SSB_FUSED_LAYOUT=reference the quantised SH buffers take the reference's per-256-splat layout of its fused path.
    stock = os.environ.get("SSB_STOCK_FLAGS", "0") != "0"
    layout = os.environ.get("SSB_FUSED_LAYOUT", "shared")
    extra = {}
    if stock:
        from spirula_studio_b200.trainer import OptimOptions
        extra = dict(non_sh_optim_bits=16, optim=OptimOptions())
    tr = Trainer(cfg, splats, device=dev, world_size=world, rank=rank, grad_sync=grad_sync, fused_backward=fused, fused_state_layout=layout, **extra)
    del splats
    # this rank's views, grouped by camera kind (one kind for every workload but the wide-camera one)
    n_kinds = scenes.n_view_kinds(cfg)
    host, resident, kind_dims = [], [], []
    h2d_bytes = 0
    for kind in range(n_kinds):
        _, model, kw, kh, _, _ = scenes.view_kind(cfg, kind)
        kind_dims.append((kw, kh))
        views = [v for v in range(v0, v0 + nv) if scenes.view_kind(cfg, v)[0] == kind]
        h_vm = torch.from_numpy(vm[views].copy().reshape(len(views), 16)).pin_memory()
        h_K = torch.from_numpy(K[views].copy().reshape(len(views), 4)).pin_memory()
        h_gt = torch.empty((len(views), kh, kw, 3), dtype=torch.float32).pin_memory()
        for i, v in enumerate(views):
            h_gt[i].copy_(torch.from_numpy(scenes.make_target(cfg, v)))
        host.append((kind, h_vm, h_K, h_gt))
        resident.append((kind, h_vm.to(dev), h_K.to(dev), h_gt.to(dev), len(views)))
        h2d_bytes += len(views) * (kw * kh * 12 + 64 + 16)
    P = cfg.width * cfg.height

    # ---- device-resident timing -------------------------------------------
    for _ in range(args.warmup):
        tr.step_device_kinds(resident, total_views)
    pairs = tr.last_isects() if resident[0][4] > 0 else 0
    tr.check_capacity()                                            # raises if any view outgrew the pair capacity
    sampler = ClockSampler(local_rank) if rank == 0 else None
    barrier()
    launches0 = lib.ssb_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        tr.step_device_kinds(resident, total_views)
    e1.record()
    barrier()
    launches = lib.ssb_launch_count() - launches0
    ms_total = max_over_ranks(e0.elapsed_time(e1))
    ms_step = ms_total / args.steps

    # ---- end to end: host buffers in, loss scalars out --------------------
    # every step copies its inputs from pinned host memory and reads its loss scalars back; the scalars are
    # handed to the caller one step late (as the reference reports them), so the host never stalls the device
    for _ in range(min(args.warmup, 2)):
        tr.train_step_kinds(host, total_views, stale_loss=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        tr.train_step_kinds(host, total_views, stale_loss=True)
    losses = tr.last_losses()          # waits for the last step's device -> host read
    e1.record()
    barrier()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1)) / args.steps
    clocks = sampler.stop() if sampler else None

    # ---- where the gradient exchange spends its time (own pass, normal overlapped step)
    exchange = None
    if world > 1 and tr.grad_sync in ("peer", "multimem"):
        tr.trace = []
        n_tr = max(2, min(args.steps, 5))
        for _ in range(n_tr):
            tr.step_device_kinds(resident, total_views)
        exchange = {k: round(v / n_tr, 4) for k, v in tr.exchange_breakdown().items()}
        tr.trace = None

    # ---- per-stage device times (separate pass, CUDA events inside the library)
    stage_ms = [np.zeros(len(L.STAGES), np.float32) for _ in range(n_kinds)]
    n_prof = [0] * n_kinds
    adam_ms = comm_ms = 0.0
    prof_steps = max(1, min(args.steps, 4))
    for h in tr.handles:
        L.check(lib.ssb_step_set_profiling(h, 1))
    ea, eb, ec = (torch.cuda.Event(enable_timing=True) for _ in range(3))
    for _ in range(prof_steps):
        tr.losses.zero_()
        first = True
        for kind, d_vm, d_K, d_gt, knv in resident:
            if knv == 0:
                continue
            tr.views_fwd_bwd(d_vm, d_K, d_gt, knv, accumulate=not first, kind=kind)
            first = False
            views_done = C.c_int32(0)
            L.check(lib.ssb_step_get_profile(tr.handles[kind], stage_ms[kind].ctypes.data_as(C.c_void_p), C.byref(views_done)))
            n_prof[kind] += views_done.value
        ea.record(); tr.allreduce_grads(); eb.record(); tr.optimizer_step(total_views); ec.record()
        torch.cuda.synchronize()
        comm_ms += ea.elapsed_time(eb); adam_ms += eb.elapsed_time(ec)
    for h in tr.handles:
        L.check(lib.ssb_step_set_profiling(h, 0))
    per_view_ms = stage_ms[0] / max(n_prof[0], 1)
    adam_ms /= prof_steps; comm_ms /= prof_steps

    # visible pairs of the last view of the first kind, for the byte counts
    visible = 0
    if resident[0][4] > 0:
        aabb_p = C.c_void_p()
        L.check(lib.ssb_step_peek(tr.handle, None, None, None, None, None, C.byref(aabb_p)))
        aabb = L.device_bytes_tensor(aabb_p.value, cfg.n_splats * 16, dev).view(torch.float32).view(-1, 4)
        visible = int((aabb[:, 2] > aabb[:, 0]).sum().item())

    if rank == 0:
        peak, peak_kind = peaks()
        tiles = ((cfg.width + 15) // 16) * ((cfg.height + 15) // 16)
        sort_passes = (32 + lib.ssb_tile_n_bits(tiles) + 7) // 8
        kernels = {}
        for i, name in enumerate(L.STAGES):
            b = stage_bytes(name, cfg.n_splats, visible, pairs, P, tiles, cfg.sh_value_bits, sort_passes)
            ms = float(per_view_ms[i])
            gbs = b / (ms * 1e-3) / 1e9 if ms > 0 else 0.0
            kernels[name] = {"ms": round(ms, 4), "launches_per_iteration": resident[0][4], "algorithmic_bytes": int(b), "gbs": round(gbs, 1), "frac_of_hbm": round(gbs / peak, 4)}
        ab = adam_bytes(cfg.n_splats, cfg.sh_value_bits)
        kernels["adam"] = {"ms": round(adam_ms, 4), "launches_per_iteration": 1, "algorithmic_bytes": int(ab),
                           "gbs": round(ab / (adam_ms * 1e-3) / 1e9, 1) if adam_ms > 0 else 0.0,
                           "frac_of_hbm": round(ab / (adam_ms * 1e-3) / 1e9 / peak, 4) if adam_ms > 0 else 0.0}
        if tr.fused_backward:
            # the projection backward of ALL views runs inside this pass (ssb_step_backward_optimize), range by range
            nv = resident[0][4]
            pb = stage_bytes("project_bwd", cfg.n_splats, visible, pairs, P, tiles, cfg.sh_value_bits, sort_passes)
            fb = nv * (visible * 48 + cfg.n_splats * 16) + ab          # every view's records and aabb once, parameters and state once
            kernels["adam"].update({"includes": "projection backward of all views, fused with the optimiser (no world-gradient arrays)",
                                    "algorithmic_bytes": int(fb), "unfused_algorithmic_bytes": int(nv * pb + ab),
                                    "gbs": round(fb / (adam_ms * 1e-3) / 1e9, 1) if adam_ms > 0 else 0.0,
                                    "frac_of_hbm": round(fb / (adam_ms * 1e-3) / 1e9 / peak, 4) if adam_ms > 0 else 0.0})
            kernels["project_bwd"]["note"] = "runs inside the optimiser pass (see adam)"
        kernels["allreduce"] = {"ms": round(comm_ms, 4), "bytes": int(tr.grads_flat.numel() * 4), "mode": tr.grad_sync,
                                "note": "peer / multimem: nothing here, the sum over the ranks happens inside the optimiser kernels (adam time, with "
                                        "both barriers); nccl: all-reduce of the whole gradient buffer"}
        for kind in range(1, n_kinds):       # further camera kinds: per-view stage times only
            kw, kh = kind_dims[kind]
            kernels[f"kind{kind}_{kw}x{kh}"] = {name: round(float(stage_ms[kind][i] / max(n_prof[kind], 1)), 4) for i, name in enumerate(L.STAGES)}
            kernels[f"kind{kind}_{kw}x{kh}"]["pairs_per_view"] = tr.last_isects(kind) if resident[kind][4] > 0 else 0
        share = {k: v["ms"] * v.get("launches_per_iteration", 1) for k, v in kernels.items() if k != "allreduce" and "ms" in v}
        dom = max(share, key=share.get)
        full_size = cfg.name == "mid_1m" and not args.splats
        if full_size:
            for k, t in NCU_TRAFFIC_MID1M.items():
                kernels[k]["dram_traffic"] = int(t)
        sm_max = (clocks or {}).get("sm_max_mhz") or 1965.0
        fp32_peak = FP32_LANES * 2 * sm_max * 1e6 / 1e12            # TFLOP/s
        if full_size:
            for k, f in NCU_FLOP_MID1M.items():
                tf = f / (kernels[k]["ms"] * 1e-3) / 1e12 if kernels[k]["ms"] > 0 else 0.0
                kernels[k].update({"flop": int(f), "tflops_fp32": round(tf, 2), "frac_of_fp32": round(tf / fp32_peak, 4)})
        recorded = "recorded constant from an earlier ncu capture of this command, not measured by this run"
        if full_size and dom in NCU_FLOP_MID1M:
            # the dominant kernel is an arithmetic kernel: its roofline is the FP32 pipe (achieved = recorded flop count of one
            # launch / this run's measured launch time); its HBM figures stay in `kernels`
            roof = {"kernel": dom, "bound": "fp32", "achieved": kernels[dom]["tflops_fp32"], "peak": round(fp32_peak, 2), "unit": "TFLOP/s",
                    "frac": kernels[dom]["frac_of_fp32"], "traffic": int(NCU_TRAFFIC_MID1M[dom]), "traffic_source": recorded,
                    "flop_source": recorded, "peak_source": f"148 SMs x 128 FP32 lanes x 2 x {sm_max:.0f} MHz (nominal: no measured FP32 peak for this pool)",
                    "hbm": {"achieved": kernels[dom]["gbs"], "peak": peak, "unit": "GB/s", "frac": kernels[dom]["frac_of_hbm"],
                            "peak_source": f"{peak_kind} copy bandwidth"},
                    "note": "the rasterisers and the loss kernel work out of L2 (DRAM at 1-3 % of peak, traffic below the algorithmic bytes); "
                            "they are bound by instruction issue and shared-memory bandwidth, so the FP32 pipe is the roofline that means "
                            "something; the HBM-bound stages (projection, Adam) carry their own fractions in `kernels`"}
        else:
            roof = {"kernel": dom, "bound": "hbm", "achieved": kernels[dom]["gbs"], "peak": peak, "unit": "GB/s", "frac": kernels[dom]["frac_of_hbm"],
                    "traffic": int(NCU_TRAFFIC_MID1M[dom]) if full_size and dom in NCU_TRAFFIC_MID1M else None,
                    "traffic_source": recorded if full_size else None, "peak_source": f"{peak_kind} copy bandwidth"}
        value = 1e3 / ms_step
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": cfg.name, "n_splats": cfg.n_splats, "views_per_iteration": total_views, "views_per_gpu": nv,
                       "resolution": [cfg.width, cfg.height], "sh_value_bits": cfg.sh_value_bits, "sh_optim_bits": cfg.sh_optim_bits,
                       "parallelism": f"views sharded over {world} GPU(s), replicated parameters, gradients combined by " +
                                      ("this library's fused reduce + sharded Adam + broadcast kernels over peer memory" if tr.grad_sync == "peer" else
                                       "this library's fused reduce + sharded Adam + broadcast kernels through the NVSwitch multicast address"
                                       if tr.grad_sync == "multimem" else "an NCCL all-reduce" if tr.grad_sync == "nccl" else "nothing (one GPU)"),
                       "optimiser": ("stock flags of the reference trainer" if stock else "plain Adam") +
                                    (", projection backward fused with the optimiser" if tr.fused_backward else "") +
                                    (", reference fused-path layouts" if tr.fused_state_layout == "reference" else ""),
                       "pairs_per_view": int(pairs), "visible_per_view": visible,
                       "l2": "inputs (parameters, gradients, moments, targets: > 1 GB) exceed the 126 MB L2; no flush between iterations"},
            "e2e": {"value": 1e3 / e2e_ms, "unit": UNIT, "ms_per_step": e2e_ms, "h2d_bytes_per_step": int(h2d_bytes), "d2h_bytes_per_step": 12},
            "gpu_launches": int(launches), "clocks": clocks, "roofline": roof, "kernels": kernels,
            "losses_last": {"l1": losses[0], "ssim": losses[1], "loss": losses[2]},
            "device_bytes": tr.device_bytes(),
        }
        if exchange is not None:
            line["exchange_ms_rank0"] = exchange
        if world == 1 and not args.no_cpu_baseline:
            cfg_cpu = cfg
            v, t_iter, t_view, t_adam, cores = cpu_port_run(cfg_cpu, 2, 0)
            line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": cores, "kind": "port",
                                    "sample": f"2 of {cfg.n_views} views at full size through every stage ({t_view:.2f} s each) and 2 Adam passes "
                                              f"({t_adam:.2f} s each); iteration time = {cfg.n_views} x view + Adam"}
        if world == 1 and not args.no_ref_cuda:
            # the reference's own CUDA kernels on this GPU, same scene, per stage (test-side leg, after the timed region)
            from oracle import ref_timing
            if ref_timing.available():
                tr.close()
                torch.cuda.empty_cache()
                rt = ref_timing.time_kernels(cfg, n_views=min(cfg.n_views, 4), repeats=2, device=dev, with_ours=False)
                line["reference_cuda_kernels"] = rt
                rm = rt["reference_ms"]
                for ours_name, ref_name in (("project_fwd", "project_fwd"), ("raster_fwd", "raster_fwd"), ("loss", "loss_ssim"),
                                            ("raster_bwd", "raster_bwd"), ("project_bwd", "project_bwd")):
                    kernels[ours_name]["ref_ms"] = rm[ref_name]
                kernels["tile_keys"]["ref_ms"] = rm["intersect"]       # the reference's whole intersection, against tile_keys + sort here
                kernels["sort"]["ref_ms"] = 0.0
                kernels["adam"]["ref_ms"] = rt["reference_ms_adam"]
                line["vs_reference_cuda_kernels"] = {
                    "reference_ms_per_iteration": rt["reference_ms_per_iteration"], "ours_ms_per_iteration": ms_step,
                    "ratio": rt["reference_ms_per_iteration"] / ms_step,
                    "note": "sum of the reference's kernel times (its L1 loss kernel, gradient zeroing and host work excluded) over this "
                            "library's measured iteration time"}
            else:
                line["reference_cuda_kernels"] = {"unavailable": "oracle/_ref/libssb_ref.so is not built on this machine"}
        emit(line)
    tr.close()
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=WORKLOAD)
    ap.add_argument("--splats", type=int, default=0, help="override the splat count (smaller cases for profiling)")
    ap.add_argument("--views", type=int, default=0, help="override the views per iteration")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-ref-cuda", action="store_true", help="skip timing the reference's CUDA kernels after the run")
    args = ap.parse_args()
    claim_stdout()
    from spirula_studio_b200 import scenes
    cfg = scenes.CONFIGS[args.workload]
    if args.splats or args.views:
        cfg = scenes.scaled(cfg, n_splats=args.splats or None, n_views=args.views or None, name=cfg.name)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, cfg, rank)
    else:
        run_ours(args, cfg, rank, world, local_rank)


if __name__ == "__main__":
    main()
