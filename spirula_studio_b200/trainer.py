"""Host-side driver of one training iteration on one GPU (one process per GPU).

Mirrors the reference's multi-view step (src/engine/EngineTrainStep.cpp:287-437):
each view is rendered and back-propagated on its own, per-splat gradients are
summed over the views, and ONE optimiser pass runs with grad_scale = 1 / views.
With several processes the views of a batch are split between ranks, the
gradient buffer is summed with an NCCL all-reduce, and every rank applies the
same update to its replica of the parameters.

torch supplies device memory, streams and torch.distributed; all arithmetic is
done by libssb_b200 through its C ABI.
"""
import ctypes as C

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


class Trainer:
    def __init__(self, cfg: SceneConfig, splats: dict, device="cuda:0", isect_capacity=0, w_l1=0.8, w_ssim=0.2,
                 process_group=None, world_size=1, rank=0):
        self.lib = L.load()
        self.cfg = cfg
        self.device = torch.device(device)
        self.n = int(cfg.n_splats)
        self.world_size, self.rank, self.pg = world_size, rank, process_group
        n = self.n
        dev = self.device
        self.params_flat = torch.zeros(_flat_len(n), dtype=torch.float32, device=dev)
        self.params = _flat_views(self.params_flat, n)
        for name, _ in _ATTRS:
            self.params[name].copy_(torch.from_numpy(np.ascontiguousarray(splats[name]).reshape(-1)))
        self.grads_flat = torch.zeros(_flat_len(n), dtype=torch.float32, device=dev)
        self.grads = _flat_views(self.grads_flat, n)
        self.quant = cfg.sh_value_bits in (8, 16)
        n_mom = _flat_len(n) if not self.quant else _flat_len(n, _ATTRS[:5])
        self.m1_flat = torch.zeros(n_mom, dtype=torch.float32, device=dev)
        self.m2_flat = torch.zeros(n_mom, dtype=torch.float32, device=dev)
        self.m1 = _flat_views(self.m1_flat, n) if not self.quant else self._geo_views(self.m1_flat)
        self.m2 = _flat_views(self.m2_flat, n) if not self.quant else self._geo_views(self.m2_flat)
        self.shq = None
        if self.quant:
            cells = n * 45
            blocks = (cells + 255) // 256
            bytes_per = 2 if cfg.sh_value_bits == 16 else 1
            self.sh_packed = torch.zeros(cells * bytes_per, dtype=torch.uint8, device=dev)
            self.sh_bounds = torch.zeros(blocks * 2, dtype=torch.float32, device=dev)
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
    def views_fwd_bwd(self, d_viewmats, d_intrins, d_gt, n_views, accumulate=False, stream=None, kind=0):
        """Forward + loss + backward of n_views views (all of camera kind `kind`) already resident on the device."""
        L.check(self.lib.ssb_step_views(self.handles[kind], C.byref(self._p_struct), C.byref(self.shq) if self.shq else None,
                                        L.ptr(d_viewmats), L.ptr(d_intrins), L.ptr(d_gt), n_views,
                                        C.byref(self._g_struct), 1 if accumulate else 0, L.ptr(self.losses), stream))

    def allreduce_grads(self):
        if self.world_size > 1:
            torch.distributed.all_reduce(self.grads_flat, op=torch.distributed.ReduceOp.SUM, group=self.pg)

    def optimizer_step(self, total_views, stream=None):
        lr = self.cfg.lrs
        self.iteration += 1
        cfg = L.SsbAdamConfig(lr["lr_means"], lr["lr_quats"], lr["lr_scales"], lr["lr_opacities"], lr["lr_features_dc"],
                              lr["lr_features_sh"], 0.0, 1.0 / float(total_views), self.iteration, 0)
        L.check(self.lib.ssb_adam_step(C.byref(self._p_struct), C.byref(self._g_struct), C.byref(self._m1_struct),
                                       C.byref(self._m2_struct), 0, self.n, C.byref(cfg), stream))
        if self.quant:
            cells = self.n * 45
            L.check(self.lib.ssb_adam_step_sh_quantized(L.ptr(self.grads["features_sh"]), L.ptr(self.sh_optim_packed),
                                                        L.ptr(self.sh_optim_bounds), L.ptr(self.sh_packed), L.ptr(self.sh_bounds),
                                                        self.cfg.sh_value_bits, 0, cells, cells, C.byref(cfg), stream))

    # -- whole iteration ---------------------------------------------------
    def step_device(self, d_viewmats, d_intrins, d_gt, n_local_views, total_views):
        """One iteration with this rank's views (one camera kind) already in HBM; losses stay on the device."""
        self.step_device_kinds([(0, d_viewmats, d_intrins, d_gt, n_local_views)], total_views)

    def step_device_kinds(self, batches, total_views):
        """One iteration; `batches` = [(kind, d_viewmats, d_intrins, d_gt, n_views), ...], this rank's views by camera kind."""
        self.losses.zero_()
        first = True
        for kind, d_viewmats, d_intrins, d_gt, nv in batches:
            if nv > 0:
                self.views_fwd_bwd(d_viewmats, d_intrins, d_gt, nv, accumulate=not first, kind=kind)
                first = False
        if first:
            self.grads_flat.zero_()
        self.allreduce_grads()
        self.optimizer_step(total_views)

    def train_step(self, h_viewmats, h_intrins, h_gt, total_views, chunk=2):
        """One iteration from HOST buffers of one camera kind; see train_step_kinds."""
        return self.train_step_kinds([(0, h_viewmats, h_intrins, h_gt)], total_views, chunk)

    def train_step_kinds(self, batches, total_views, chunk=2):
        """One iteration from HOST buffers (pinned torch tensors holding this rank's views, one entry
        (kind, viewmats, intrins, targets) per camera kind): host->device copies of cameras and targets,
        the iteration, and a device->host read of the loss scalars. Returns (l1, ssim, loss) averaged
        over this rank's views.

        The targets are copied `chunk` views at a time on a side stream and each chunk is
        rendered as soon as it has landed, so the PCIe transfer of later views hides behind
        the computation of earlier ones."""
        if self._copy_stream is None:
            self._copy_stream = torch.cuda.Stream(device=self.device)
        main = torch.cuda.current_stream(self.device)
        self.losses.zero_()
        # the previous iteration may still be reading the staging buffers
        self._copy_stream.wait_stream(main)
        events = []
        nv_total = 0
        with torch.cuda.stream(self._copy_stream):
            for kind, h_viewmats, h_intrins, h_gt in batches:
                nv = int(h_viewmats.shape[0])
                nv_total += nv
                st = self._staging.get(kind)
                if st is None or st[2].shape != h_gt.shape:
                    st = (torch.empty_like(h_viewmats, device=self.device), torch.empty_like(h_intrins, device=self.device),
                          torch.empty_like(h_gt, device=self.device))
                    self._staging[kind] = st
                st[0].copy_(h_viewmats, non_blocking=True)
                st[1].copy_(h_intrins, non_blocking=True)
                for c0 in range(0, nv, chunk):
                    c1 = min(nv, c0 + chunk)
                    st[2][c0:c1].copy_(h_gt[c0:c1], non_blocking=True)
                    ev = torch.cuda.Event()
                    ev.record(self._copy_stream)
                    events.append((kind, c0, c1, ev))
        if nv_total == 0:
            self.grads_flat.zero_()
        for i, (kind, c0, c1, ev) in enumerate(events):
            main.wait_event(ev)
            d_view, d_intr, d_gt = self._staging[kind]
            L.check(self.lib.ssb_step_views(self.handles[kind], C.byref(self._p_struct), C.byref(self.shq) if self.shq else None,
                                            L.ptr(d_view[c0:]), L.ptr(d_intr[c0:]), L.ptr(d_gt[c0:]), c1 - c0,
                                            C.byref(self._g_struct), 1 if i > 0 else 0, L.ptr(self.losses), None))
        self.allreduce_grads()
        self.optimizer_step(total_views)
        out = self.losses.cpu()
        return tuple((out / max(nv_total, 1)).tolist())

    def last_isects(self, kind=0):
        m = C.c_int64(0)
        L.check(self.lib.ssb_step_last_isects(self.handles[kind], C.byref(m), None))
        return m.value
