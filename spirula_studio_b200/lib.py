"""ctypes binding of libssb_b200.so (the C ABI declared in include/ssb.h).

Only plain pointers and sizes cross the boundary.  torch is used by callers for
device memory and streams; nothing here imports it.  Loading fails loudly when
the shared library has not been built: there is no CPU fallback.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libssb_b200.so")

SSB_OK = 0
SSB_ERR_INVALID_ARGUMENT = -1
SSB_ERR_CUDA = -2
SSB_ERR_CAPACITY = -3
SSB_ERR_OUT_OF_MEMORY = -4
SSB_ERR_UNSUPPORTED = -5
SSB_ERR_PEER = -6
SSB_ERR_IO = -7

DISTORTION_NONE, DISTORTION_OPENCV, DISTORTION_THIN_PRISM, DISTORTION_RATIONAL = 0, 1, 2, 3
CAMERA_PINHOLE, CAMERA_FISHEYE, CAMERA_EQUISOLID, CAMERA_EQUIRECT = 0, 1, 2, 3
SSB_ACCUM_NONE, SSB_ACCUM_MAX, SSB_ACCUM_SUM, SSB_ACCUM_AVG = 0, 1, 2, 3
STATUS_BAD_INDEX, STATUS_PAIRS_DROPPED = 1, 2
NUM_SH = 15
TILE = 16
SCREEN_REC_FLOATS = 12
STAGES = ("project_fwd", "tile_keys", "sort", "tile_ranges", "raster_fwd", "loss", "raster_bwd", "project_bwd")


class SsbError(RuntimeError):
    def __init__(self, status, message):
        super().__init__(f"ssb status {status}: {message}")
        self.status = status


class SsbSplats(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("means", "quats", "scales", "opacities", "features_dc", "features_sh")]


class SsbShQuant(C.Structure):
    _fields_ = [("packed", C.c_void_p), ("bounds", C.c_void_p), ("bits", C.c_int32), ("reserved", C.c_int32),
                ("bounds_stride", C.c_int64)]


class SsbCameras(C.Structure):
    _fields_ = [("d_viewmats", C.c_void_p), ("d_intrins", C.c_void_p), ("count", C.c_int32), ("width", C.c_int32),
                ("height", C.c_int32), ("model", C.c_int32), ("antialiased", C.c_int32), ("distortion", C.c_int32),
                ("sh_degree_plus1", C.c_int32), ("d_dist_coeffs", C.c_void_p)]


class SsbLossConfig(C.Structure):
    _fields_ = [("w_l1", C.c_float), ("w_ssim", C.c_float), ("num_scales", C.c_int32), ("loss_map_mode", C.c_int32),
                ("d_mask", C.c_void_p), ("mask_h", C.c_int32), ("mask_w", C.c_int32)]


LOSS_MAP_NONE, LOSS_MAP_LOSS_FULL, LOSS_MAP_SSIM_FULL, LOSS_MAP_SSIM_CS, LOSS_MAP_SSIM_STRUCTURE = range(5)


class SsbDensifyScoreConfig(C.Structure):
    _fields_ = [("max_screen_size", C.c_float), ("max_screen_size_clip_hardness", C.c_float), ("max_world_size", C.c_float),
                ("accum_mode", C.c_int32), ("score_mode", C.c_int32), ("score_blend_world_grad", C.c_float), ("score_power", C.c_float),
                ("score_clip_quantile", C.c_float), ("final_score_power", C.c_float)]


SCORE_MEAN, SCORE_MAX, SCORE_MEDIAN, SCORE_GEOM = range(4)


class SsbAdamConfig(C.Structure):
    _fields_ = [("lr_means", C.c_float), ("lr_quats", C.c_float), ("lr_scales", C.c_float), ("lr_opacities", C.c_float),
                ("lr_features_dc", C.c_float), ("lr_features_sh", C.c_float), ("sh_reg_weight", C.c_float),
                ("grad_scale", C.c_float), ("step", C.c_int32), ("zero_grad", C.c_int32)]


class SsbAdamExtras(C.Structure):
    _fields_ = [("max_gauss_ratio", C.c_float), ("scale_regularization_weight", C.c_float), ("mcmc_opacity_reg_weight", C.c_float),
                ("mcmc_scale_reg_weight", C.c_float), ("erank_reg_weight", C.c_float), ("erank_reg_weight_s3", C.c_float),
                ("quat_norm_reg_weight", C.c_float), ("use_scale_agnostic_mean", C.c_int32), ("d_radii", C.c_void_p),
                ("d_steps", C.c_void_p), ("n_total", C.c_int64), ("d_densify_score", C.c_void_p)]


class SsbStepConfig(C.Structure):
    _fields_ = [("n_splats", C.c_int64), ("width", C.c_int32), ("height", C.c_int32), ("camera_model", C.c_int32),
                ("antialiased", C.c_int32), ("isect_capacity", C.c_int64), ("w_l1", C.c_float), ("w_ssim", C.c_float)]


_P = C.c_void_p
_I32, _I64, _F = C.c_int32, C.c_int64, C.c_float

# name -> (restype, argtypes); every symbol include/ssb.h declares
SIGNATURES = {
    "ssb_last_error_string": (C.c_char_p, []),
    "ssb_version_string": (C.c_char_p, []),
    "ssb_project_fwd": (C.c_int, [_P, _P, _I64, _P, _P, _P, _P, _P, _P]),
    "ssb_project_bwd": (C.c_int, [_P, _P, _I64, _P, _P, _P, _P, C.c_int, _P]),
    "ssb_screen_unpack": (C.c_int, [_P, _I64, _P, _P, _P, _P, _P, _P]),
    "ssb_screen_pack": (C.c_int, [_P, _P, _P, _P, _P, _I64, _P, _P]),
    "ssb_screen_unpack_add": (C.c_int, [_P, _I64, _P, _P, _P, _P, _P, _P]),
    "ssb_tile_keys_workspace_bytes": (_I64, [_I64]),
    "ssb_tile_keys": (C.c_int, [_P, _P, _P, _I64, _I64, _I32, _I32, _P, _I64, _P, _P, _P, _P, _I64, _P, _P, _P]),
    "ssb_sort_workspace_bytes": (_I64, [_I64]),
    "ssb_sort_pairs_u64": (C.c_int, [_P, _P, _P, _P, _P, _I64, _I32, _I32, _P, _I64, _P, _P]),
    "ssb_sort_check": (C.c_int, [_P, _P]),
    "ssb_sort_pairs_u64_noalloc": (C.c_int, [_P, _P, _P, _P, _P, _I64, _I32, _I32, _P, _P]),
    "ssb_intersect_tiles_workspace_bytes": (_I64, [_I64, _I64]),
    "ssb_intersect_tiles": (C.c_int, [_P, _P, _P, _I64, _I64, _I32, _I32, _P, _I64, _P, _P, _I64, _P, _P, _P]),
    "ssb_intersect_tiles_live": (C.c_int, [_P, _P, _P, _I64, _I64, _I32, _I32, _P, _I64, _P, _P, _I64, _P, _P, _P, _P]),
    "ssb_tile_active": (C.c_int, [_P, _I32, _I32, _I32, _I32, _I32, _P, _P]),
    "ssb_tile_keys_live": (C.c_int, [_P, _P, _P, _I64, _I64, _I32, _I32, _P, _I64, _P, _P, _P, _P, _I64, _P, _P, _P, _P]),
    "ssb_project_fwd_packed_workspace_bytes": (_I64, [_I64, _I32]),
    "ssb_project_fwd_packed": (C.c_int, [_P, _P, _I64, _P, _P, _I64, _P, _P, _P, _P, _P, _P, _I64, _P, _P, _P]),
    "ssb_project_bwd_packed_workspace_bytes": (_I64, [_I64, _I32]),
    "ssb_project_bwd_packed": (C.c_int, [_P, _P, _I64, _P, _P, _P, _P, _P, _P, _I64, _P, _I64, _P, C.c_int, _P]),
    "ssb_intersect_tiles_packed": (C.c_int, [_P, _P, _P, _P, _P, _I64, _I32, _I32, _I32, _P, _I64, _P, _P, _I64, _P, _P, _P]),
    "ssb_intersect_tiles_packed_live": (C.c_int, [_P, _P, _P, _P, _P, _I64, _I32, _I32, _I32, _P, _I64, _P, _P, _I64, _P, _P, _P, _P]),
    "ssb_tile_n_bits": (_I32, [_I64]),
    "ssb_peer_alloc": (C.c_int, [_I64, _P]),
    "ssb_peer_free": (C.c_int, [_P]),
    "ssb_peer_export": (C.c_int, [_P, _P]),
    "ssb_peer_open": (C.c_int, [_P, _P]),
    "ssb_peer_close": (C.c_int, [_P]),
    "ssb_peer_reduce_f32": (C.c_int, [_P, _P]),
    "ssb_peer_broadcast": (C.c_int, [_P, _P]),
    "ssb_reduce_adam_broadcast": (C.c_int, [_P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _P, _P, _P]),
    "ssb_reduce_adam_broadcast_q16": (C.c_int, [_P, _P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _P, _P, _P]),
    "ssb_exchange_step": (C.c_int, [_P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _P, _P, _P, _P, _P]),
    "ssb_exchange_step_q16": (C.c_int, [_P, _P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _P, _P, _P, _P, _P]),
    "ssb_tile_ranges": (C.c_int, [_P, _P, _I64, _I64, _P, _P]),
    "ssb_raster_fwd": (C.c_int, [_P, _I64, _P, _P, _I64, _P, _I32, _I32, _I32, _P, _P, _P, _P, _P]),
    "ssb_raster_bwd": (C.c_int, [_P, _I64, _P, _P, _I64, _P, _I32, _I32, _I32, _P, _P, _P, _P, _P, _P, _P, _P]),
    "ssb_raster_bwd_accum": (C.c_int, [_P, _I64, _P, _P, _I64, _P, _I32, _I32, _I32, _P, _P, _P, _P, _P, _P, _P, _I32, _P, _I64, _P, _P, _P, _P]),
    "ssb_device_status": (C.c_int, [_P, _P]),
    "ssb_step_max_pairs_device": (_P, [_P]),
    "ssb_step_isect_capacity": (_I64, [_P]),
    "ssb_step_status": (C.c_int, [_P, _P, C.c_int, _P]),
    "ssb_loss_l1_ssim_fwdbwd": (C.c_int, [_P, _P, _I32, _I32, _I32, _F, _F, _P, _P, _P]),
    "ssb_step_set_densify": (C.c_int, [_P, _I32, _F, _I32, _P, _P]),
    "ssb_loss_l1_ssim_fwdbwd_map": (C.c_int, [_P, _P, _I32, _I32, _I32, _F, _F, _P, _P, _I32, _F, _P, _P]),
    "ssb_loss_workspace_bytes": (_I64, [_I32, _I32, _I32, _P]),
    "ssb_loss_multi_scale": (C.c_int, [_P, _P, _I32, _I32, _I32, _P, _P, _P, _P, _P, _I64, _P]),
    "ssb_step_set_loss": (C.c_int, [_P, _P]),
    "ssb_step_set_radii": (C.c_int, [_P, _P]),
    "ssb_step_set_distortion": (C.c_int, [_P, _I32, _P]),
    "ssb_step_set_sh_degree": (C.c_int, [_P, _I32]),
    "ssb_step_render": (C.c_int, [_P, _P, _P, _P, _P, _P, _P, _P, _P]),
    "ssb_project_bwd_optimize_workspace_bytes": (C.c_int64, [_I64]),
    "ssb_project_bwd_optimize": (C.c_int, [_P, _P, _I64, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I64, _P]),
    "ssb_project_bwd_optimize_q16": (C.c_int, [_P, _P, _I64, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I64, _P]),
    "ssb_ply_write": (C.c_int, [C.c_char_p, _P, _P, _I64, _P, _P]),
    "ssb_ply_info": (C.c_int, [C.c_char_p, _P, _P]),
    "ssb_ply_read": (C.c_int, [C.c_char_p, _I64, _I32, _P, _P, _P, _P, _P, _P]),
    "ssb_step_set_fused_backward": (C.c_int, [_P, _I32]),
    "ssb_step_backward_optimize": (C.c_int, [_P, _P, _P, _P, _P, _I32, _P, _P, _P, _P, _P, _P]),
    "ssb_step_backward_optimize_q16": (C.c_int, [_P, _P, _P, _P, _P, _I32, _P, _P, _P, _P, _P, _P, _P]),
    "ssb_adam_step_q16": (C.c_int, [_P, _P, _P, _I64, _I64, _P, _P, _P]),
    "ssb_adam_plain": (C.c_int, [_P, _P, _P, _P, _I64, _I32, _F, _I32, _P, _F, _F, _F, _I32, _P]),
    "ssb_adam_step": (C.c_int, [_P, _P, _P, _P, _I64, _I64, _P, _P]),
    "ssb_adam_step_sh_quantized": (C.c_int, [_P, _P, _P, _P, _P, _I32, _I64, _I64, _I64, _P, _P]),
    "ssb_adam_step_ex": (C.c_int, [_P, _P, _P, _P, _I64, _I64, _P, _P, _P]),
    "ssb_adam_step_sh_quantized_ex": (C.c_int, [_P, _P, _P, _P, _P, _I32, _I32, _I64, _I64, _I64, _P, _P, _I32, _P]),
    "ssb_adam_step_sh_splat_blocks": (C.c_int, [_P, _P, _P, _P, _P, _I32, _I64, _I64, _I64, _I32, _P, _P, _P]),
    "ssb_quant_encode": (C.c_int, [_P, _I64, _I32, _P, _P, _P]),
    "ssb_quant_decode": (C.c_int, [_P, _P, _I64, _I32, _P, _P]),
    "ssb_step_create": (C.c_int, [_P, _P]),
    "ssb_step_destroy": (None, [_P]),
    "ssb_step_device_bytes": (_I64, [_P]),
    "ssb_step_views": (C.c_int, [_P, _P, _P, _P, _P, _P, _I32, _P, C.c_int, _P, _P]),
    "ssb_step_views_gated": (C.c_int, [_P, _P, _P, _P, _P, _P, _I32, _P, _P, C.c_int, _P, _P]),
    "ssb_step_last_isects": (C.c_int, [_P, _P, _P]),
    "ssb_step_peek": (C.c_int, [_P, _P, _P, _P, _P, _P, _P]),
    "ssb_step_set_profiling": (C.c_int, [_P, C.c_int]),
    "ssb_step_get_profile": (C.c_int, [_P, _P, _P]),
    "ssb_launch_count": (_I64, []),
    "ssb_densify_workspace_bytes": (_I64, [_I64]),
    "ssb_densify_relocate_workspace_bytes": (_I64, [_I64]),
    "ssb_densify_relocate": (C.c_int, [_P, _I64, _F, _F, C.c_uint32, _P, _I64, _P, _P]),
    "ssb_densify_add": (C.c_int, [_P, _I64, _I64, _F, C.c_uint32, _P, _I64, _P]),
    "ssb_densify_update_scores": (C.c_int, [_P, _I64, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I64, _P]),
    "ssb_densify_add_noise": (C.c_int, [_I64, _F, _I32, _P, _P, _P, _P, _P, _P]),
    "ssb_ckpt_array_header": (C.c_int, [C.c_int, C.c_uint64, _P, C.c_int]),
    "ssb_ckpt_member_header": (C.c_int, [C.c_char_p, C.c_uint64, _P]),
    "ssb_ckpt_writer_open": (C.c_int, [C.c_char_p, _P]),
    "ssb_ckpt_write_bytes": (C.c_int, [_P, C.c_char_p, _P, C.c_uint64]),
    "ssb_ckpt_write_host": (C.c_int, [_P, C.c_char_p, _P, C.c_uint64, C.c_int]),
    "ssb_ckpt_write_device": (C.c_int, [_P, C.c_char_p, _P, C.c_uint64, C.c_int, _P]),
    "ssb_ckpt_writer_close": (C.c_int, [_P]),
    "ssb_ckpt_reader_open": (C.c_int, [C.c_char_p, _P]),
    "ssb_ckpt_member_count": (C.c_int, [_P]),
    "ssb_ckpt_member_info": (C.c_int, [_P, C.c_int, _P, C.c_int, _P]),
    "ssb_ckpt_read_bytes": (C.c_int, [_P, C.c_char_p, _P, C.c_uint64, _P]),
    "ssb_ckpt_array_info": (C.c_int, [_P, C.c_char_p, _P, C.c_int, _P]),
    "ssb_ckpt_read_host": (C.c_int, [_P, C.c_char_p, _P, C.c_uint64]),
    "ssb_ckpt_read_device": (C.c_int, [_P, C.c_char_p, _P, C.c_uint64, _P]),
    "ssb_ckpt_reader_close": (C.c_int, [_P]),
}

_lib = None


def load():
    """Returns the loaded library; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `make -C {os.path.join(_HERE, 'csrc')}` "
            "(or __graft_entry__.build()). There is no CPU fallback.")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError = a declared symbol is not exported
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(status):
    if status != SSB_OK:
        raise SsbError(status, load().ssb_last_error_string().decode("utf-8", "replace"))


def ptr(t):
    """Device (or host) address of a tensor-like object, or None."""
    if t is None:
        return None
    return C.c_void_p(t.data_ptr())


def splats_struct(d):
    """d: mapping with the six arrays (tensors or None)."""
    s = SsbSplats()
    for n, _ in SsbSplats._fields_:
        t = d.get(n)
        setattr(s, n, t.data_ptr() if t is not None else None)
    return s


def shq_struct(packed=None, bounds=None, bits=32, bounds_stride=256):
    q = SsbShQuant()
    q.packed = packed.data_ptr() if packed is not None else None
    q.bounds = bounds.data_ptr() if bounds is not None else None
    q.bits = bits
    q.reserved = 0
    q.bounds_stride = bounds_stride
    return q


MAX_PEERS, MAX_PEER_BUFFERS, MAX_PEER_SEGMENTS, PEER_HANDLE_BYTES = 8, 4, 12, 64


class SsbPeerSegment(C.Structure):
    _fields_ = [("buffer", C.c_int32), ("pad", C.c_int32), ("offset_bytes", C.c_int64), ("bytes", C.c_int64)]


class SsbPeerTable(C.Structure):
    _fields_ = [("world", C.c_int32), ("self", C.c_int32), ("n_segments", C.c_int32), ("pad", C.c_int32),
                ("base", (C.c_void_p * MAX_PEERS) * MAX_PEER_BUFFERS), ("seg", SsbPeerSegment * MAX_PEER_SEGMENTS),
                ("multicast", C.c_void_p * MAX_PEER_BUFFERS)]


def peer_table(world, rank, bases, segments, multicast=None):
    """bases[b][r] = device address of rank r's copy of buffer b; segments = [(buffer, offset_bytes, bytes), ...];
    multicast[b] = NVSwitch multicast address of buffer b (optional)."""
    t = SsbPeerTable()
    for b, addr in enumerate(multicast or []):
        t.multicast[b] = addr or None
    t.world, t.self, t.n_segments = world, rank, len(segments)
    for b, per_rank in enumerate(bases):
        for r, addr in enumerate(per_rank):
            t.base[b][r] = addr
    for i, (b, off, nbytes) in enumerate(segments):
        t.seg[i].buffer, t.seg[i].offset_bytes, t.seg[i].bytes = b, off, nbytes
    return t


class SsbPeerReplicas(C.Structure):
    _fields_ = [("world", C.c_int32), ("self", C.c_int32), ("grads", C.c_void_p * MAX_PEERS), ("params", C.c_void_p * MAX_PEERS),
                ("sh_packed", C.c_void_p * MAX_PEERS), ("sh_bounds", C.c_void_p * MAX_PEERS),
                ("mc_grads", C.c_void_p), ("mc_params", C.c_void_p), ("mc_sh_packed", C.c_void_p), ("mc_sh_bounds", C.c_void_p)]


class SsbShAdamState(C.Structure):
    _fields_ = [("d_optim_packed", C.c_void_p), ("d_optim_bounds", C.c_void_p), ("d_value_packed", C.c_void_p),
                ("d_value_bounds", C.c_void_p), ("value_bits", C.c_int32), ("optim_bits", C.c_int32), ("layout", C.c_int32)]


SH_LAYOUT_CELL_BLOCKS, SH_LAYOUT_SPLAT_BLOCKS = 0, 1


class SsbMomentsQ16(C.Structure):
    _fields_ = [("d_packed", C.c_void_p * 5), ("d_bounds", C.c_void_p * 5)]


class SsbDensifyState(C.Structure):
    _fields_ = [("params", SsbSplats), ("m1", SsbSplats), ("m2", SsbSplats), ("sh", SsbShAdamState), ("d_accum_buffer", C.c_void_p),
                ("d_sample_score", C.c_void_p), ("d_steps", C.c_void_p)]


# int barrier(void* ctx, void* stream): 0 once every rank has arrived (ordered on the stream), non-zero on failure
BARRIER_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_void_p)


def peer_replicas(world, rank, grads, params, sh_packed=None, sh_bounds=None, multicast=None):
    """Each argument: the device address of every rank's copy of that allocation, as mapped in this process;
    multicast = (grads, params, sh_packed, sh_bounds) NVSwitch multicast addresses, or None."""
    r = SsbPeerReplicas()
    r.world, r.self = world, rank
    if multicast:
        r.mc_grads, r.mc_params, r.mc_sh_packed, r.mc_sh_bounds = [a or None for a in (list(multicast) + [None] * 4)[:4]]
    for name, addrs in (("grads", grads), ("params", params), ("sh_packed", sh_packed), ("sh_bounds", sh_bounds)):
        arr = getattr(r, name)
        for p_, a in enumerate(addrs or []):
            arr[p_] = a or None
    return r


class _DevicePtr:
    """Wraps a raw device address so torch can view it (the allocation stays owned by the caller)."""
    def __init__(self, address, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (address, False), "version": 3}


def device_bytes_tensor(address, nbytes, device):
    """uint8 torch tensor over `nbytes` of device memory at `address`."""
    import torch
    return torch.as_tensor(_DevicePtr(address, nbytes), device=device)


def cameras_struct(viewmats, intrins, width, height, model=CAMERA_PINHOLE, antialiased=0, count=None, distortion=0, dist_coeffs=None, sh_degree=None):
    """dist_coeffs: device float32 [count][8] rows of the distortion tier (DISTORTION_*), or None for zeros.
    sh_degree: active SH degree 0..3 (None = all bands)."""
    c = SsbCameras()
    c.d_viewmats = viewmats.data_ptr()
    c.d_intrins = intrins.data_ptr()
    c.count = int(viewmats.shape[0]) if count is None else count
    c.width, c.height, c.model, c.antialiased = width, height, model, antialiased
    c.distortion = distortion
    c.d_dist_coeffs = dist_coeffs.data_ptr() if dist_coeffs is not None else None
    c.sh_degree_plus1 = 0 if sh_degree is None else int(sh_degree) + 1
    return c
