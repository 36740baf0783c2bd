"""Host-side driver of one training iteration on one GPU (one process per GPU).

Mirrors the reference's multi-view step (src/engine/EngineTrainStep.cpp:287-437):
each view is rendered and back-propagated on its own, per-splat gradients are
summed over the views, and ONE optimiser pass runs with grad_scale = 1 / views.
With several processes (one per GPU) the views of a batch are split between
ranks and every rank keeps a replica of the parameters.  Gradients are combined
in one of two ways:
  "peer" (default): each rank owns a contiguous range of splats and runs ONE
      fused pass over it (ssb_exchange_step): the optimiser kernels read the
      peers' partial gradients of the range straight from their memory over
      NVLink, sum them in registers, update, and store the new parameters into
      every replica.  Two stream-ordered barriers per iteration keep the ranks
      in step; a barrier that fails (a rank is gone) ends the step with
      SSB_ERR_PEER before any kernel that depends on that rank is launched.
  "multimem": the same fused pass, but the exchanged buffers live in torch
      symmetric memory and the kernels address them through their NVSwitch
      multicast address: the switch adds the ranks' gradients on a load and
      replicates a parameter store, so each rank receives its range once and
      sends each update once instead of once per peer.  Falls back to "peer"
      where that cannot be set up.
  "nccl": one NCCL all-reduce of the whole gradient buffer, then every rank
      applies the same Adam update to all parameters.

torch supplies device memory, streams and torch.distributed; all arithmetic is
done by libssb_b200 through its C ABI.
"""
import ctypes as C
from dataclasses import dataclass

import numpy as np
import torch

from . import lib as L
from .scenes import SceneConfig, n_view_kinds, view_kind

_ATTRS = (("means", 3), ("quats", 4), ("scales", 3), ("opacities", 1), ("features_dc", 3), ("features_sh", 45))
FLOATS_PER_SPLAT = sum(w for _, w in _ATTRS)  # 59


def _pad(x, a=64):
    return (x + a - 1) // a * a


def _flat_len(n, attrs=_ATTRS):
    return sum(_pad(n * w) for _, w in attrs)


def _flat_views(flat, n, attrs=_ATTRS):
    """Per-attribute views into one fp32 buffer (attribute-major, each attribute
    starting on a 256-byte boundary so 16-byte vector accesses stay aligned)."""
    out, off = {}, 0
    for name, w in attrs:
        out[name] = flat[off: off + n * w]
        off += _pad(n * w)
    return out


@dataclass
class OptimOptions:
    """The reference's optimiser flags next to the learning rates (OptimConfig, src/engine/EngineConfig.h; stock values of
    src/config/TrainConfig.h:258-304): per-splat regularisers, the scale-agnostic mean update, per-splat bias-correction
    counters.  Passed to Trainer(optim=...); without it the trainer runs the plain Adam step the benchmark times."""
    max_gauss_ratio: float = 10.0
    scale_regularization_weight: float = 0.0
    opacity_reg: float = 0.01            # mcmc_opacity_reg_weight
    scale_reg: float = 0.01              # mcmc_scale_reg_weight
    erank_reg: float = 0.0
    erank_reg_s3: float = 0.0
    quat_norm_reg: float = 0.01
    sh_reg: float = 0.001
    use_scale_agnostic_mean: bool = True
    use_per_splat_bias_correction: bool = True


class Trainer:
    def __init__(self, cfg: SceneConfig, splats: dict, device="cuda:0", isect_capacity=0, w_l1=0.8, w_ssim=0.2,
                 process_group=None, world_size=1, rank=0, grad_sync="peer", fused_backward=False, non_sh_optim_bits=32, optim=None,
                 fused_state_layout="shared"):
        self.lib = L.load()
        self.cfg = cfg
        self.device = torch.device(device)
        self.n = int(cfg.n_splats)
        self.world_size, self.rank, self.pg = world_size, rank, process_group
        if grad_sync not in ("peer", "multimem", "nccl"):
            raise ValueError(f"grad_sync must be 'peer', 'multimem' or 'nccl', not {grad_sync!r}")
        self.grad_sync = grad_sync if world_size > 1 else "none"
        if self.grad_sync == "multimem" and not self._symmetric_memory_usable():
            self.grad_sync = "peer"
        self._symm_tensors = []
        if self.grad_sync in ("peer", "multimem") and world_size > L.MAX_PEERS:
            raise ValueError(f"peer gradient exchange supports at most {L.MAX_PEERS} ranks")
        self._peer_allocs, self._peer_maps = [], []
        n = self.n
        dev = self.device
        self.params_flat = self._shared_zeros(_flat_len(n) * 4).view(torch.float32)
        self.params = _flat_views(self.params_flat, n)
        for name, _ in _ATTRS:
            self.params[name].copy_(torch.from_numpy(np.ascontiguousarray(splats[name]).reshape(-1)))
        self.grads_flat = self._shared_zeros(_flat_len(n) * 4).view(torch.float32)
        self.grads = _flat_views(self.grads_flat, n)
        self.quant = cfg.sh_value_bits in (8, 16)
        n_mom = _flat_len(n) if not self.quant else _flat_len(n, _ATTRS[:5])
        self.m1_flat = torch.zeros(n_mom, dtype=torch.float32, device=dev)
        self.m2_flat = torch.zeros(n_mom, dtype=torch.float32, device=dev)
        self.m1 = _flat_views(self.m1_flat, n) if not self.quant else self._geo_views(self.m1_flat)
        self.m2 = _flat_views(self.m2_flat, n) if not self.quant else self._geo_views(self.m2_flat)
        # Moments of means, rotations, scales, opacities and DC in 16-bit codes (the reference's non_sh_optim_bits = 16,
        # src/engine/EngineOptim.cpp:136-146): 4 bytes per cell and one float4 of bounds per 256 splats and array replace the
        # fp32 pairs (8 bytes per cell).  Every rank then updates every splat, so the gradients must already be summed
        # (one rank, or the NCCL all-reduce).
        if non_sh_optim_bits not in (16, 32):
            raise ValueError(f"non_sh_optim_bits must be 32 (off) or 16; got {non_sh_optim_bits}")
        self.non_sh_optim_bits = non_sh_optim_bits
        self.nsq_packed, self.nsq_bounds, self._nsq = {}, {}, None
        if non_sh_optim_bits == 16:
            self._nsq = L.SsbMomentsQ16()
            for t, (name, width) in enumerate(_ATTRS[:5]):
                self.nsq_packed[name] = torch.zeros(n * width * 4, dtype=torch.uint8, device=dev)
                self.nsq_bounds[name] = torch.zeros(((n + 255) // 256) * 4, dtype=torch.float32, device=dev)
                self._nsq.d_packed[t], self._nsq.d_bounds[t] = self.nsq_packed[name].data_ptr(), self.nsq_bounds[name].data_ptr()
        # Where the quantised SH buffers keep their bounds.  "shared": one per 256 cells, the layout of the unfused optimiser calls
        # (the fused backward + optimiser then shares it with them).  "reference": one per 256 splats, the layout the reference
        # keeps for its fused path (pool slots eng.sh_quant_fpbo, eng.world.sh_vq16_fpbo; state.json use_fused_proj_bwd_optim = 1),
        # so that its stock checkpoints load and resume; only the fused backward + optimiser updates it.
        if fused_state_layout not in ("shared", "reference"):
            raise ValueError(f"fused_state_layout must be 'shared' or 'reference', not {fused_state_layout!r}")
        self.fused_state_layout = fused_state_layout
        if fused_state_layout == "reference" and not (self.quant and fused_backward and world_size == 1 and n_view_kinds(cfg) == 1):
            raise ValueError("fused_state_layout='reference' needs quantised SH and the fused backward + optimiser (one GPU, one camera kind)")
        self.shq = None
        if self.quant and fused_state_layout == "reference":
            cells, blocks = n * 45, (n + 255) // 256
            bytes_per = 2 if cfg.sh_value_bits == 16 else 1
            self.sh_packed = torch.zeros(cells * bytes_per, dtype=torch.uint8, device=dev)
            self.sh_bounds = torch.zeros(blocks * 2, dtype=torch.float32, device=dev)
            self.sh_optim_packed = torch.zeros(cells * 2, dtype=torch.uint8, device=dev)
            self.sh_optim_bounds = torch.zeros(blocks * 4, dtype=torch.float32, device=dev)
            self._encode_splat_blocks(self.params["features_sh"], cfg.sh_value_bits)
            self.shq = L.shq_struct(self.sh_packed, self.sh_bounds, cfg.sh_value_bits, 0)
        elif self.quant:
            cells = n * 45
            blocks = (cells + 255) // 256
            bytes_per = 2 if cfg.sh_value_bits == 16 else 1
            self.sh_packed = self._shared_zeros(cells * bytes_per)
            self.sh_bounds = self._shared_zeros(blocks * 2 * 4).view(torch.float32)
            self.sh_optim_packed = torch.zeros(cells * 2, dtype=torch.uint8, device=dev)
            self.sh_optim_bounds = torch.zeros(blocks * 4, dtype=torch.float32, device=dev)
            L.check(self.lib.ssb_quant_encode(L.ptr(self.params["features_sh"]), cells, cfg.sh_value_bits,
                                              L.ptr(self.sh_packed), L.ptr(self.sh_bounds), None))
            self.shq = L.shq_struct(self.sh_packed, self.sh_bounds, cfg.sh_value_bits, 256)
        # one set of per-view buffers per camera kind of the batch (model and image size are fixed per set)
        self.handles = []
        for k in range(n_view_kinds(cfg)):
            _, model, width, height, _, _ = view_kind(cfg, k)
            step_cfg = L.SsbStepConfig(n, width, height, model, 0, isect_capacity, w_l1, w_ssim)
            handle = C.c_void_p()
            L.check(self.lib.ssb_step_create(C.byref(step_cfg), C.byref(handle)))
            self.handles.append(handle)
        self.handle = self.handles[0]
        self.losses = torch.zeros(3, dtype=torch.float32, device=dev)
        self.iteration = 0
        self._p_struct = L.splats_struct(self.params if not self.quant else {**self.params, "features_sh": None})
        self._g_struct = L.splats_struct(self.grads)
        self._m1_struct = L.splats_struct(self.m1)
        self._m2_struct = L.splats_struct(self.m2)
        # device staging for one rank's share of a batch, per camera kind (filled by train_step)
        self._staging = {}
        self._copy_stream = None
        # One GPU, one camera kind: the projection backward of all views can run together with the optimiser
        # (ssb_step_backward_optimize), so the world gradients never travel through HBM.  With several ranks the
        # gradients have to be summed over the ranks first, so the per-view backward stays.
        self.fused_backward = bool(fused_backward) and world_size == 1 and len(self.handles) == 1
        self._kept_cams = []
        if self.fused_backward:
            L.check(self.lib.ssb_step_set_fused_backward(self.handle, max(int(cfg.n_views), 1)))
            self._fused_room = max(int(cfg.n_views), 1)
        # the reference's optimiser options: regularisers, scale-agnostic mean (needs the view radii), per-splat counters
        self.optim = optim
        self.radii = self.steps = None
        self._extras = None
        self._radii_external = False         # a Densifier clears the radii itself (before_step)
        if optim is not None:
            if optim.use_scale_agnostic_mean:
                self.radii = torch.zeros(n, dtype=torch.float32, device=dev)
                for h in self.handles:
                    L.check(self.lib.ssb_step_set_radii(h, L.ptr(self.radii)))
            if optim.use_per_splat_bias_correction:
                self.steps = torch.zeros(n, dtype=torch.int32, device=dev)
            self._extras = L.SsbAdamExtras(optim.max_gauss_ratio, optim.scale_regularization_weight, optim.opacity_reg, optim.scale_reg,
                                           optim.erank_reg, optim.erank_reg_s3, optim.quat_norm_reg, 1 if optim.use_scale_agnostic_mean else 0,
                                           self.radii.data_ptr() if self.radii is not None else None,
                                           self.steps.data_ptr() if self.steps is not None else None, n, None)
        # the range of splats whose optimiser step this rank performs
        self.first, self.count = 0, n
        if self.grad_sync in ("peer", "multimem"):
            self._setup_peers()

    def _encode_splat_blocks(self, values, bits):
        """Initial SH values -> codes with one (min, max) bound per 256 splats (QuantizedTensor<bits>::encode_v of the reference,
        src/core/Tensor.h:1379-1392, on its per-splat-block layout); runs once, at construction."""
        n, blocks = self.n, (self.n + 255) // 256
        v = values.view(n, 45)
        block_of = torch.arange(n, device=v.device) // 256
        lo = torch.full((blocks,), float("inf"), device=v.device).scatter_reduce_(0, block_of, v.amin(dim=1), "amin")
        hi = torch.full((blocks,), float("-inf"), device=v.device).scatter_reduce_(0, block_of, v.amax(dim=1), "amax")
        qmax = float((1 << bits) - 1)
        span = (hi - lo).clamp_min(1e-30)
        codes = torch.round(qmax * (v - lo[block_of, None]) / span[block_of, None]).clamp_(0, qmax).to(torch.int32).reshape(-1)
        if bits == 16:
            self.sh_packed.view(-1, 2)[:, 0] = (codes & 255).to(torch.uint8)
            self.sh_packed.view(-1, 2)[:, 1] = (codes >> 8).to(torch.uint8)
        else:
            self.sh_packed.copy_(codes.to(torch.uint8))
        self.sh_bounds.view(blocks, 2)[:, 0] = lo
        self.sh_bounds.view(blocks, 2)[:, 1] = hi

    # -- peer-memory gradient exchange -------------------------------------
    def _symmetric_memory_usable(self):
        """Every rank must take the same decision, so the ranks vote."""
        ok = 1.0
        try:
            import torch.distributed._symmetric_memory as symm
            probe = symm.empty(1024, dtype=torch.uint8, device=self.device)
            group = self.pg if self.pg is not None else torch.distributed.group.WORLD
            h = symm.rendezvous(probe, group)
            if not h.multicast_ptr:
                ok = 0.0
        except Exception:
            ok = 0.0
        vote = torch.tensor([ok], dtype=torch.float32, device=self.device)
        torch.distributed.all_reduce(vote, op=torch.distributed.ReduceOp.MIN, group=self.pg)
        return bool(vote.item() > 0.5)

    def _shared_zeros(self, nbytes):
        """Zeroed device bytes; an exportable allocation when peers will access it."""
        if self.grad_sync == "multimem":
            import torch.distributed._symmetric_memory as symm
            t = symm.empty(max(int(nbytes), 16), dtype=torch.uint8, device=self.device)
            t.zero_()
            self._symm_tensors.append(t)
            return t[:int(nbytes)]
        if self.grad_sync != "peer":
            return torch.zeros(nbytes, dtype=torch.uint8, device=self.device)
        ptr = C.c_void_p()
        L.check(self.lib.ssb_peer_alloc(max(int(nbytes), 16), C.byref(ptr)))
        self._peer_allocs.append(ptr)
        return L.device_bytes_tensor(ptr.value, int(nbytes), self.device)

    def _setup_peers(self):
        import torch.distributed as dist
        W, r, n = self.world_size, self.rank, self.n
        # ranges are multiples of 512 splats so that every array's slice starts on a 16-byte boundary
        per = ((n + W - 1) // W + 511) // 512 * 512
        self.first = min(n, r * per)
        self.count = min(n, self.first + per) - self.first
        bufs = [self.grads_flat, self.params_flat] + ([self.sh_packed, self.sh_bounds] if self.quant else [])
        bases = [[0] * W for _ in bufs]
        mcast = [0] * len(bufs)
        if self.grad_sync == "multimem":
            import torch.distributed._symmetric_memory as symm
            group = self.pg if self.pg is not None else dist.group.WORLD
            torch.cuda.synchronize(self.device)          # the buffers' initial contents are in place
            by_address = {t.data_ptr(): t for t in self._symm_tensors}
            for b, view in enumerate(bufs):
                t = by_address[view.data_ptr()]           # the symmetric allocation this buffer is a view of
                h = symm.rendezvous(t, group)
                for p in range(W):
                    bases[b][p] = int(h.buffer_ptrs[p])
                bases[b][r] = t.data_ptr()
                mcast[b] = int(h.multicast_ptr)
        else:
            mine = []
            for t in bufs:
                h = (C.c_ubyte * L.PEER_HANDLE_BYTES)()
                L.check(self.lib.ssb_peer_export(C.c_void_p(t.data_ptr()), h))
                mine.append(bytes(h))
            everyone = [None] * W
            dist.all_gather_object(everyone, mine, group=self.pg)
            for p in range(W):
                for b, t in enumerate(bufs):
                    if p == r:
                        bases[b][p] = t.data_ptr()
                    else:
                        ptr = C.c_void_p()
                        h = (C.c_ubyte * L.PEER_HANDLE_BYTES).from_buffer_copy(everyone[p][b])
                        L.check(self.lib.ssb_peer_open(h, C.byref(ptr)))
                        self._peer_maps.append(ptr)
                        bases[b][p] = ptr.value
        f, c = self.first, self.count
        grad_segs, param_segs, off = [], [], 0
        for name, w in _ATTRS:
            grad_segs.append((0, (off + f * w) * 4, c * w * 4))
            if not (self.quant and name == "features_sh"):
                param_segs.append((0, (off + f * w) * 4, c * w * 4))
            off += _pad(n * w)
        tables_bases, tables_mcast = [bases[1]], [mcast[1]]
        if self.quant:
            bytes_per = 2 if self.cfg.sh_value_bits == 16 else 1
            b0, b1 = f * 45 // 256, ((f + c) * 45 + 255) // 256
            param_segs.append((1, f * 45 * bytes_per, c * 45 * bytes_per))
            param_segs.append((2, b0 * 8, (b1 - b0) * 8))
            tables_bases += [bases[2], bases[3]]
            tables_mcast += [mcast[2], mcast[3]]
        self._reduce_table = L.peer_table(W, r, [bases[0]], grad_segs, [mcast[0]])
        self._bcast_table = L.peer_table(W, r, tables_bases, param_segs, tables_mcast)
        self._replicas = L.peer_replicas(W, r, bases[0], bases[1], bases[2] if self.quant else None, bases[3] if self.quant else None,
                                         multicast=mcast if self.grad_sync == "multimem" else None)
        self._barrier_cb = L.BARRIER_FN(self._barrier_status)       # kept alive: the library calls it
        self._token = torch.zeros(1, dtype=torch.float32, device=self.device)
        self._barrier()          # every rank has mapped every buffer before anyone touches them

    def _barrier(self):
        """Orders the ranks on the current stream: work enqueued after it on any rank starts only after
        the work enqueued before it on every rank has finished."""
        torch.distributed.all_reduce(self._token, group=self.pg)

    def _barrier_status(self, ctx, stream):
        """The barrier as the library's callback: 0 when every rank arrived, 1 when the collective failed or timed out."""
        try:
            self._barrier()
            return 0
        except Exception as e:          # a rank that is gone shows up here as a process-group error or timeout
            self._barrier_error = e
            return 1

    def _geo_views(self, flat):
        out = _flat_views(flat, self.n, _ATTRS[:5])
        out["features_sh"] = None
        return out

    def close(self):
        for h in getattr(self, "handles", []):
            if h:
                self.lib.ssb_step_destroy(h)
        self.handles = []
        self.handle = C.c_void_p()
        if getattr(self, "_peer_maps", None) or getattr(self, "_peer_allocs", None) or getattr(self, "_symm_tensors", None):
            torch.cuda.synchronize(self.device)
            if self.world_size > 1 and torch.distributed.is_initialized():
                self._barrier()                      # nobody unmaps while a peer may still be writing
                torch.cuda.synchronize(self.device)
            for ptr in self._peer_maps:
                self.lib.ssb_peer_close(ptr)
            self._peer_maps = []
            # tensors viewing these allocations must not be used after this point
            for ptr in self._peer_allocs:
                self.lib.ssb_peer_free(ptr)
            self._peer_allocs = []
            self._symm_tensors = []

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def device_bytes(self):
        own = sum(t.numel() * t.element_size() for t in (self.params_flat, self.grads_flat, self.m1_flat, self.m2_flat))
        if self.quant:
            own += sum(t.numel() * t.element_size() for t in (self.sh_packed, self.sh_bounds, self.sh_optim_packed, self.sh_optim_bounds))
        return own + sum(int(self.lib.ssb_step_device_bytes(h)) for h in self.handles)

    # -- pieces ------------------------------------------------------------
    def _keep_cams(self, d_viewmats, d_intrins, n_views, fresh):
        """Fused backward: remembers the cameras of the views the step object keeps, and makes room for them."""
        if fresh:
            self._kept_cams = []
        self._kept_cams.append((d_viewmats[:n_views], d_intrins[:n_views]))
        total = sum(int(c[0].shape[0]) for c in self._kept_cams)
        if total > self._fused_room:
            if len(self._kept_cams) > 1:
                raise RuntimeError("fused backward: the view count of an iteration grew while views were being kept")
            L.check(self.lib.ssb_step_set_fused_backward(self.handle, total))
            self._fused_room = total

    def render(self, viewmat, intrin, kind=0, depth=False):
        """One image of the current splats, forward only (the viewer's path): viewmat [16] / intrin [4] as numpy or tensors.
        Returns (rgb [H][W][3], transmittance [H][W]) and, with depth=True, the ray-depth image as a third tensor."""
        _, _, width, height, _, _ = view_kind(self.cfg, kind)
        as_dev = lambda a, n: torch.as_tensor(np.asarray(a, np.float32) if not torch.is_tensor(a) else a, dtype=torch.float32).reshape(n).to(self.device)
        d_vm, d_K = as_dev(viewmat, 16), as_dev(intrin, 4)
        rgb = torch.empty(height, width, 3, device=self.device)
        T = torch.empty(height, width, device=self.device)
        dep = torch.empty(height, width, device=self.device) if depth else None
        stream = C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        L.check(self.lib.ssb_step_render(self.handles[kind], C.byref(self._p_struct), C.byref(self.shq) if self.shq else None, L.ptr(d_vm), L.ptr(d_K),
                                         L.ptr(rgb), L.ptr(dep) if depth else None, L.ptr(T), stream))
        return (rgb, T, dep) if depth else (rgb, T)

    def set_sh_degree(self, degree):
        """Active SH degree (0..3) of every following iteration: the reference's warm-up raises it with the step count
        (`sh_degree_for_step`)."""
        for h in self.handles:
            L.check(self.lib.ssb_step_set_sh_degree(h, int(degree)))

    @staticmethod
    def sh_degree_for_step(step, warmup_every=1000, max_degree=3):
        """sh_degree_to_use of the reference's trainer (src/app/TrainerCore.cpp:948)."""
        return min(max_degree, step // max(warmup_every, 1))

    def set_distortion(self, tier, coeffs=None, kind=0):
        """Lens-distortion tier (lib.DISTORTION_*) of the cameras of `kind` with one row of eight coefficients per view, in the
        order of the views handed to each following train_step / views_fwd_bwd call (call again before handing other views).
        coeffs: numpy or tensor [views][8] in the tier's own order, or None for zeros."""
        if self.fused_backward and tier != L.DISTORTION_NONE:
            raise NotImplementedError("lens distortion runs with the per-view backward")
        rows = None
        if tier != L.DISTORTION_NONE and coeffs is not None:
            rows = torch.as_tensor(np.ascontiguousarray(coeffs, dtype=np.float32) if not torch.is_tensor(coeffs) else coeffs,
                                   dtype=torch.float32).reshape(-1, 8).to(self.device).contiguous()
        if not hasattr(self, "_dist_rows"):
            self._dist_rows = {}
        self._dist_rows[kind] = rows                     # keeps the device rows alive
        L.check(self.lib.ssb_step_set_distortion(self.handles[kind], int(tier), L.ptr(rows) if rows is not None else None))

    def views_fwd_bwd(self, d_viewmats, d_intrins, d_gt, n_views, accumulate=False, stream=None, kind=0):
        """Forward + loss + backward of n_views views (all of camera kind `kind`) already resident on the device."""
        if self.fused_backward:
            self._keep_cams(d_viewmats, d_intrins, n_views, not accumulate)
        L.check(self.lib.ssb_step_views(self.handles[kind], C.byref(self._p_struct), C.byref(self.shq) if self.shq else None,
                                        L.ptr(d_viewmats), L.ptr(d_intrins), L.ptr(d_gt), n_views,
                                        C.byref(self._g_struct), 1 if accumulate else 0, L.ptr(self.losses), stream))

    def allreduce_grads(self):
        """Makes the summed gradients available where the optimiser will read them: everywhere ("nccl"),
        or, for this rank's range of splats, in this rank's buffer ("peer")."""
        if self.grad_sync == "nccl":
            torch.distributed.all_reduce(self.grads_flat, op=torch.distributed.ReduceOp.SUM, group=self.pg)
        elif self.grad_sync in ("peer", "multimem"):
            self._mark("views_done")                              # the sum happens inside the optimiser pass

    def _mark(self, name):
        """With self.trace set (a list), records a CUDA event under `name`; see exchange_breakdown()."""
        if getattr(self, "trace", None) is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self.trace.append((name, ev))

    def exchange_breakdown(self):
        """Milliseconds between consecutive marks of the traced iterations, summed by the later mark's name."""
        torch.cuda.synchronize(self.device)
        out = {}
        for (n0, e0), (n1, e1) in zip(self.trace[:-1], self.trace[1:]):
            if n1 != "views_done":
                out[n1] = out.get(n1, 0.0) + e0.elapsed_time(e1)
        return out

    def optimizer_step(self, total_views, stream=None):
        lr = self.cfg.lrs
        self.iteration += 1
        cfg = L.SsbAdamConfig(lr["lr_means"], lr["lr_quats"], lr["lr_scales"], lr["lr_opacities"], lr["lr_features_dc"],
                              lr["lr_features_sh"], self.optim.sh_reg if self.optim is not None else 0.0, 1.0 / float(total_views), self.iteration, 0)
        f, c = self.first, self.count
        ex = C.byref(self._extras) if self._extras is not None else None
        if self.steps is not None:
            self.steps += 1                        # every slot, before use (src/engine/EngineOptim.cpp:367-375)
        if self.radii is not None and self.world_size > 1:
            torch.distributed.all_reduce(self.radii, op=torch.distributed.ReduceOp.MAX, group=self.pg)    # every rank saw other views
        if self.fused_backward:
            cams = self._kept_cams
            if not cams:
                return
            d_vm = cams[0][0] if len(cams) == 1 else torch.cat([x[0] for x in cams])
            d_K = cams[0][1] if len(cams) == 1 else torch.cat([x[1] for x in cams])
            sh = None
            if self.quant:
                layout = L.SH_LAYOUT_SPLAT_BLOCKS if self.fused_state_layout == "reference" else L.SH_LAYOUT_CELL_BLOCKS
                sh = L.SsbShAdamState(self.sh_optim_packed.data_ptr(), self.sh_optim_bounds.data_ptr(), self.sh_packed.data_ptr(),
                                      self.sh_bounds.data_ptr(), self.cfg.sh_value_bits, 8, layout)
            head = (self.handle, C.byref(self._p_struct), C.byref(self.shq) if self.shq else None, L.ptr(d_vm), L.ptr(d_K), int(d_vm.shape[0]))
            tail = (C.byref(self._m1_struct), C.byref(self._m2_struct), C.byref(sh) if sh is not None else None, C.byref(cfg), ex, stream)
            if self._nsq is not None:
                L.check(self.lib.ssb_step_backward_optimize_q16(*head, C.byref(self._nsq), *tail))
            else:
                L.check(self.lib.ssb_step_backward_optimize(*head, *tail))
            self._kept_cams = []
            return
        if self.grad_sync in ("peer", "multimem"):
            sh = None
            if self.quant:
                sh = L.SsbShAdamState(self.sh_optim_packed.data_ptr(), self.sh_optim_bounds.data_ptr(), self.sh_packed.data_ptr(),
                                      self.sh_bounds.data_ptr(), self.cfg.sh_value_bits, 8)
            head = (C.byref(self._replicas), C.byref(self._p_struct), C.byref(self._g_struct))
            tail = (C.byref(self._m1_struct), C.byref(self._m2_struct), C.byref(sh) if sh is not None else None, f, c, self.n, C.byref(cfg), ex)
            if self._nsq is not None:            # 16-bit moments of the non-SH arrays: the q16 entry points, per-peer loads and stores
                args, reduce, exchange = head + (C.byref(self._nsq),) + tail, self.lib.ssb_reduce_adam_broadcast_q16, self.lib.ssb_exchange_step_q16
            else:
                args, reduce, exchange = head + tail, self.lib.ssb_reduce_adam_broadcast, self.lib.ssb_exchange_step
            if getattr(self, "trace", None) is not None:          # the same three steps with a time mark after each
                self._barrier(); self._mark("barrier1")
                L.check(reduce(*args, stream)); self._mark("reduce_adam_broadcast")
                self._barrier(); self._mark("barrier2")
            else:
                L.check(exchange(*args, self._barrier_cb, None, stream))
            return
        d_steps = L.ptr(self.steps) if self.steps is not None else None
        if self._nsq is not None:
            L.check(self.lib.ssb_adam_step_q16(C.byref(self._p_struct), C.byref(self._g_struct), C.byref(self._nsq), f, c, C.byref(cfg), ex, stream))
            if not self.quant:
                L.check(self.lib.ssb_adam_plain(L.ptr(self.params["features_sh"]), L.ptr(self.grads["features_sh"]), L.ptr(self.m1["features_sh"]),
                                                L.ptr(self.m2["features_sh"]), self.n * 45, 45, lr["lr_features_sh"], self.iteration, d_steps,
                                                cfg.sh_reg_weight, 0.0, 1.0 / float(total_views), 0, stream))
        elif ex is not None:
            L.check(self.lib.ssb_adam_step_ex(C.byref(self._p_struct), C.byref(self._g_struct), C.byref(self._m1_struct),
                                              C.byref(self._m2_struct), f, c, C.byref(cfg), ex, stream))
        else:
            L.check(self.lib.ssb_adam_step(C.byref(self._p_struct), C.byref(self._g_struct), C.byref(self._m1_struct),
                                           C.byref(self._m2_struct), f, c, C.byref(cfg), stream))
        if self.quant:
            cells = self.n * 45
            if d_steps is not None:
                L.check(self.lib.ssb_adam_step_sh_quantized_ex(L.ptr(self.grads["features_sh"]), L.ptr(self.sh_optim_packed),
                                                               L.ptr(self.sh_optim_bounds), L.ptr(self.sh_packed), L.ptr(self.sh_bounds),
                                                               self.cfg.sh_value_bits, 8, f * 45, c * 45, cells, C.byref(cfg), d_steps, 45, stream))
            else:
                L.check(self.lib.ssb_adam_step_sh_quantized(L.ptr(self.grads["features_sh"]), L.ptr(self.sh_optim_packed),
                                                            L.ptr(self.sh_optim_bounds), L.ptr(self.sh_packed), L.ptr(self.sh_bounds),
                                                            self.cfg.sh_value_bits, f * 45, c * 45, cells, C.byref(cfg), stream))

    # -- whole iteration ---------------------------------------------------
    def step_device(self, d_viewmats, d_intrins, d_gt, n_local_views, total_views):
        """One iteration with this rank's views (one camera kind) already in HBM; losses stay on the device."""
        self.step_device_kinds([(0, d_viewmats, d_intrins, d_gt, n_local_views)], total_views)

    def step_device_kinds(self, batches, total_views):
        """One iteration; `batches` = [(kind, d_viewmats, d_intrins, d_gt, n_views), ...], this rank's views by camera kind."""
        self.losses.zero_()
        if self.radii is not None and not self._radii_external:
            self.radii.zero_()
        first = True
        for kind, d_viewmats, d_intrins, d_gt, nv in batches:
            if nv > 0:
                self.views_fwd_bwd(d_viewmats, d_intrins, d_gt, nv, accumulate=not first, kind=kind)
                first = False
        if first:
            self.grads_flat.zero_()
        self.allreduce_grads()
        self.optimizer_step(total_views)

    def train_step(self, h_viewmats, h_intrins, h_gt, total_views, chunk=2, stale_loss=False):
        """One iteration from HOST buffers of one camera kind; see train_step_kinds."""
        return self.train_step_kinds([(0, h_viewmats, h_intrins, h_gt)], total_views, chunk, stale_loss)

    def train_step_kinds(self, batches, total_views, chunk=2, stale_loss=False):
        """One iteration from HOST buffers (pinned torch tensors holding this rank's views, one entry
        (kind, viewmats, intrins, targets) per camera kind): host->device copies of cameras and targets,
        the iteration, and a device->host read of the loss scalars. Returns (l1, ssim, loss) averaged
        over this rank's views.

        The targets are copied `chunk` views at a time on a side stream while the whole batch is enqueued
        in one call per camera kind; on the device, only a view's loss stage waits for that view's target
        (ssb_step_views_gated), so the PCIe transfer hides behind projection, intersection and rasterisation.

        stale_loss=True returns the scalars of the PREVIOUS call instead (zeros on the first call), which
        is how the reference reports its loss (one step late, src/kernels/loss/PerPixelLoss.cu:1374-1400):
        the host then never waits for the iteration it has just enqueued, and the next call's copies
        start while this one still computes (two sets of staging buffers alternate).  `last_losses()`
        waits for and returns the newest values."""
        if self._copy_stream is None:
            self._copy_stream = torch.cuda.Stream(device=self.device)
            self._loss_host = [torch.zeros(3, dtype=torch.float32).pin_memory() for _ in range(2)]
            # the largest per-view pair count of every step object, read back with the loss scalars
            self._pairs_dev = [L.device_bytes_tensor(int(self.lib.ssb_step_max_pairs_device(h)), 8, self.device).view(torch.int64)
                               for h in self.handles]
            self._pairs_host = [torch.zeros(len(self.handles), dtype=torch.int64).pin_memory() for _ in range(2)]
            self._loss_ready = [torch.cuda.Event(), torch.cuda.Event()]
            self._set_free = [None, None]          # event after which staging set k may be overwritten
            self._loss_views = [1, 1]
            self._calls = 0
        main = torch.cuda.current_stream(self.device)
        k = self._calls & 1
        self.losses.zero_()
        if self.radii is not None and not self._radii_external:
            self.radii.zero_()
        # staging set k was last read by the iteration before the previous one
        if self._set_free[k] is not None:
            self._copy_stream.wait_event(self._set_free[k])
        calls = []          # (kind, views, per-view event handles, keep-alive list)
        nv_total = 0
        with torch.cuda.stream(self._copy_stream):
            # cameras of every kind first (a few hundred bytes), then the targets view by view
            for kind, h_viewmats, h_intrins, h_gt in batches:
                st = self._staging.get((kind, k))
                if st is None or st[2].shape != h_gt.shape:
                    st = (torch.empty_like(h_viewmats, device=self.device), torch.empty_like(h_intrins, device=self.device),
                          torch.empty_like(h_gt, device=self.device))
                    self._staging[(kind, k)] = st
                st[0].copy_(h_viewmats, non_blocking=True)
                st[1].copy_(h_intrins, non_blocking=True)
            cams_ready = torch.cuda.Event()
            cams_ready.record(self._copy_stream)
            for kind, h_viewmats, h_intrins, h_gt in batches:
                nv = int(h_viewmats.shape[0])
                nv_total += nv
                st = self._staging[(kind, k)]
                handles = (C.c_void_p * max(nv, 1))()
                keep = []
                c0 = 0
                while c0 < nv:
                    # the first copies are single views so that their loss stage can start as early as possible
                    c1 = min(nv, c0 + (1 if c0 < 2 else chunk))
                    st[2][c0:c1].copy_(h_gt[c0:c1], non_blocking=True)
                    ev = torch.cuda.Event()
                    ev.record(self._copy_stream)
                    keep.append(ev)
                    for v in range(c0, c1):
                        handles[v] = ev.cuda_event
                    c0 = c1
                calls.append((kind, nv, handles, keep))
        if nv_total == 0:
            self.grads_flat.zero_()
        main.wait_event(cams_ready)
        first = True
        for kind, nv, handles, keep in calls:
            if nv == 0:
                continue
            d_view, d_intr, d_gt = self._staging[(kind, k)]
            if self.fused_backward:
                self._keep_cams(d_view, d_intr, nv, first)
            # one call per camera kind: each view's loss stage waits on the device for its own target
            L.check(self.lib.ssb_step_views_gated(self.handles[kind], C.byref(self._p_struct), C.byref(self.shq) if self.shq else None,
                                                  L.ptr(d_view), L.ptr(d_intr), L.ptr(d_gt), nv, handles,
                                                  C.byref(self._g_struct), 0 if first else 1, L.ptr(self.losses), None))
            first = False
        self._keep_events = [c[3] for c in calls]      # the events must outlive the work that waits on them
        self.allreduce_grads()
        self.optimizer_step(total_views)
        # device -> host read of this step's scalars (asynchronous: pinned destination)
        self._loss_host[k].copy_(self.losses, non_blocking=True)
        for i, t in enumerate(self._pairs_dev):
            self._pairs_host[k][i:i + 1].copy_(t, non_blocking=True)
        self._loss_ready[k].record(main)
        self._loss_views[k] = max(nv_total, 1)
        done = torch.cuda.Event()
        done.record(main)
        self._set_free[k] = done
        self._calls += 1
        if not stale_loss:
            return self.last_losses()
        if self._calls == 1:
            return (0.0, 0.0, 0.0)
        p = 1 - k
        self._loss_ready[p].synchronize()
        self._raise_if_pairs_dropped(p)
        return tuple((self._loss_host[p] / self._loss_views[p]).tolist())

    def last_losses(self):
        """(l1, ssim, loss) of the newest host-buffer step, averaged over this rank's views; waits for it."""
        k = (self._calls - 1) & 1
        self._loss_ready[k].synchronize()
        self._raise_if_pairs_dropped(k)
        return tuple((self._loss_host[k] / self._loss_views[k]).tolist())

    def _raise_if_pairs_dropped(self, k):
        """The pair counts travel to the host with the loss scalars, so an iteration needs no extra
        synchronisation to notice that a view outgrew isect_capacity (it was then rendered from clamped lists)."""
        for i, h in enumerate(self.handles):
            cap = int(self.lib.ssb_step_isect_capacity(h))
            m = int(self._pairs_host[k][i])
            if m > cap:
                raise L.SsbError(L.SSB_ERR_CAPACITY, f"a view had {m} (splat, tile) pairs, more than isect_capacity = {cap}; "
                                                     "the pairs beyond it were dropped: create the Trainer with a larger isect_capacity")

    def check_capacity(self):
        """Synchronises and raises SsbError(SSB_ERR_CAPACITY) if any view since the last check had more
        (splat, tile) pairs than isect_capacity; returns the largest pair count seen."""
        worst = 0
        for h in self.handles:
            m = C.c_int64(0)
            L.check(self.lib.ssb_step_status(h, C.byref(m), 1, None))
            worst = max(worst, m.value)
        return worst

    def last_isects(self, kind=0):
        m = C.c_int64(0)
        L.check(self.lib.ssb_step_last_isects(self.handles[kind], C.byref(m), None))
        return m.value
