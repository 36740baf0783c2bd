"""The revised densification strategy around a Trainer: the host logic of engine_densify_step
(src/engine/EngineDensify.cpp:36-371) on top of the library's kernels.

Every iteration (call `after_step` once the optimiser has run):
    scale clip + score update (+ quantile clip)     ssb_densify_update_scores
    position noise                                  ssb_densify_add_noise
and every `refine_every` iterations while densification is ongoing, before the noise:
    relocation of the dead splats                   ssb_densify_relocate      seed 2 * step
    growth to min(capacity, growth_factor * count)  ssb_densify_add           seed 2 * step + 1
    the score accumulator is cleared

The Trainer's arrays have room for `cfg.n_splats` splats (the capacity); `count` of them are in use.  Unused slots hold an
opacity logit of -30, so every kernel of the iteration culls them, and they are outside the relocation's range.

Several ranks (views sharded over GPUs): what the iteration's views accumulate -- the per-splat weights, their denominators
and the view radii -- is combined over the ranks first (sum or maximum, three all-reduces of n floats), after which every
rank holds the same inputs and runs the same kernels: the draw is a function of the seed and the scores, the compaction is
ordered and the sort is stable, so every replica relocates and adds the same splats and no parameter has to be exchanged.
Moments that a rank does not own under the sharded optimiser are cleared with everyone else's and never read.
"""
import ctypes as C
import math
from dataclasses import dataclass

import torch

from . import lib as L


@dataclass
class DensifyConfig:
    """Defaults of the reference's training flags (src/config/TrainConfig.h:155-186)."""
    refine_start_iter: int = 500
    refine_stop_iter: int = 15000
    refine_stop_num_iter: int = 0
    refine_every: int = 100
    growth_factor: float = 1.05
    min_opacity: float = 0.005
    noise_lr: float = 80.0
    noise_lr_final: float = 0.8
    max_screen_size: float = 0.3
    max_screen_size_clip_hardness: float = 1.5
    max_world_size: float = math.inf
    score_mode: int = L.SCORE_MEAN
    score_power: float = 0.4
    score_blend_world_grad: float = 0.0
    score_clip_quantile: float = 1.0
    final_score_power: float = 1.0
    las_split_opacity_k_init: float = 0.6
    las_split_opacity_k_final: float = 0.6
    las_split_opacity_k_warmup: int = 0
    accum_mode: int = L.SSB_ACCUM_MAX
    loss_map_mode: int = 2              # SsimLossMapMode of the per-view loss map the weights are gathered from
    loss_map_weight: float = 0.2


class Densifier:
    def __init__(self, trainer, cfg: DensifyConfig, count: int):
        if len(trainer.handles) != 1:
            raise NotImplementedError("the densification strategy runs with one camera kind")
        if trainer.non_sh_optim_bits != 32:
            raise NotImplementedError("relocation and growth clear fp32 moments; 16-bit non-SH moment codes are not handled")
        if trainer.fused_backward:
            raise NotImplementedError("the per-splat weights are gathered by the per-view raster backward")
        self.tr, self.cfg, self.count = trainer, cfg, int(count)
        n, dev, lib = trainer.n, trainer.device, trainer.lib
        assert 0 < self.count <= n
        z = lambda *shape, dt=torch.float32: torch.zeros(*shape, dtype=dt, device=dev)
        # the view radii are shared with the trainer's scale-agnostic mean update when that is on
        self.radii = trainer.radii if getattr(trainer, "radii", None) is not None else z(n)
        trainer._radii_external = True
        self.accum_weight, self.accum_den = z(n), z(n)
        self.accum_buffer, self.sample_score = z(n, 2), z(n, 2)
        self.ws = z(int(lib.ssb_densify_relocate_workspace_bytes(n)) + int(lib.ssb_densify_workspace_bytes(n)), dt=torch.uint8)
        self.num_relocated = z(1, dt=torch.int32)
        trainer.params["opacities"][self.count:] = -30.0
        L.check(lib.ssb_step_set_radii(trainer.handle, L.ptr(self.radii)))
        L.check(lib.ssb_step_set_densify(trainer.handle, cfg.loss_map_mode, cfg.loss_map_weight, cfg.accum_mode, L.ptr(self.accum_weight),
                                         L.ptr(self.accum_den)))
        tr = trainer
        st = L.SsbDensifyState()
        st.params = L.splats_struct(tr.params if not tr.quant else {**tr.params, "features_sh": None})
        st.m1, st.m2 = L.splats_struct(tr.m1), L.splats_struct(tr.m2)
        if tr.quant:
            st.sh = L.SsbShAdamState(tr.sh_optim_packed.data_ptr(), tr.sh_optim_bounds.data_ptr(), tr.sh_packed.data_ptr(), tr.sh_bounds.data_ptr(),
                                     tr.cfg.sh_value_bits, 8)
        else:
            st.sh = L.SsbShAdamState(None, None, None, None, 32, 0)
        st.d_accum_buffer = self.accum_buffer.data_ptr()
        st.d_sample_score = None
        st.d_steps = trainer.steps.data_ptr() if getattr(trainer, "steps", None) is not None else None
        self.state = st

    def before_step(self):
        """Clears what the iteration's views accumulate into."""
        self.radii.zero_(); self.accum_weight.zero_(); self.accum_den.zero_()

    def after_step(self, step: int, max_steps: int) -> int:
        """The strategy's work after iteration `step`'s optimiser pass; returns the number of splats added."""
        c, tr, lib = self.cfg, self.tr, self.tr.lib
        if tr.world_size > 1:
            import torch.distributed as dist
            if tr.radii is None:                 # (the trainer's optimiser step has combined shared radii already)
                dist.all_reduce(self.radii, op=dist.ReduceOp.MAX, group=tr.pg)
            dist.all_reduce(self.accum_weight, op=dist.ReduceOp.MAX if c.accum_mode == L.SSB_ACCUM_MAX else dist.ReduceOp.SUM, group=tr.pg)
            if c.accum_mode == L.SSB_ACCUM_AVG:
                dist.all_reduce(self.accum_den, op=dist.ReduceOp.SUM, group=tr.pg)
        ongoing = step < max(c.refine_stop_iter, max_steps - c.refine_stop_num_iter)
        do_densify = ongoing and step > c.refine_start_iter and step % c.refine_every == 0
        progress = (step + 0.5) / max_steps
        n = self.count
        use_power = c.final_score_power != 1.0
        sc = L.SsbDensifyScoreConfig(c.max_screen_size, c.max_screen_size_clip_hardness, c.max_world_size, c.accum_mode, c.score_mode,
                                     c.score_blend_world_grad, c.score_power, c.score_clip_quantile, c.final_score_power)
        L.check(lib.ssb_densify_update_scores(C.byref(sc), n, L.ptr(self.radii), L.ptr(tr.params["scales"]), L.ptr(tr.params["opacities"]),
                                              L.ptr(self.accum_weight), L.ptr(self.accum_den), None, L.ptr(self.accum_buffer) if ongoing else None,
                                              L.ptr(self.sample_score) if (use_power and ongoing) else None, L.ptr(self.ws), self.ws.numel(), None))
        self.state.d_sample_score = self.sample_score.data_ptr() if use_power else None
        added = 0
        k = c.las_split_opacity_k_final
        if c.las_split_opacity_k_warmup > 0:
            t = min(1.0, max(0.0, step / c.las_split_opacity_k_warmup))
            k = c.las_split_opacity_k_init + t * (c.las_split_opacity_k_final - c.las_split_opacity_k_init)
        if do_densify:
            L.check(lib.ssb_densify_relocate(C.byref(self.state), n, c.min_opacity, k, 2 * step, L.ptr(self.ws), self.ws.numel(),
                                             L.ptr(self.num_relocated), None))
            target = min(tr.n, int(c.growth_factor * n))
            added = max(0, target - n)
            if added:
                L.check(lib.ssb_densify_add(C.byref(self.state), n, added, k, 2 * step + 1, L.ptr(self.ws), self.ws.numel(), None))
            self.accum_buffer.zero_()
        if c.noise_lr > 0.0 and c.noise_lr_final > 0.0:
            scalar = c.noise_lr * (c.noise_lr_final / c.noise_lr) ** progress
            L.check(lib.ssb_densify_add_noise(n + added, scalar, 1, L.ptr(self.radii), L.ptr(tr.params["means"]), L.ptr(tr.params["scales"]),
                                              L.ptr(tr.params["quats"]), L.ptr(tr.params["opacities"]), None))
        self.count = n + added
        return added
