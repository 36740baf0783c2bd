"""The C ABI without a GPU: the library loads, exports every symbol the header
declares, and validates arguments before touching the device."""
import ctypes as C
import os
import re

from spirula_studio_b200 import lib as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "ssb.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ssb_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    lib = L.load()
    names = declared_symbols()
    assert len(names) >= 25
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in ssb.h but not exported"
        assert n in L.SIGNATURES, f"{n} has no ctypes signature in lib.py"
    assert sorted(L.SIGNATURES) == names


def test_version_and_pure_host_helpers():
    lib = L.load()
    assert b"sm_100a" in lib.ssb_version_string()
    # smallest b with 2^b > n_tiles (src/kernels/tile/IntersectTile.cu:489-490)
    for n, want in ((1, 1), (2, 2), (3, 2), (4, 3), (8160, 13), (8191, 13), (8192, 14)):
        assert lib.ssb_tile_n_bits(n) == want
    assert lib.ssb_tile_keys_workspace_bytes(1_000_000) >= 8_000_000
    assert lib.ssb_sort_workspace_bytes(12_000_000) > 0


def test_argument_errors_are_statuses_not_crashes():
    lib = L.load()
    assert lib.ssb_project_fwd(None, None, 10, None, None, None, None, None, None) == L.SSB_ERR_INVALID_ARGUMENT
    assert b"NULL" in lib.ssb_last_error_string()
    assert lib.ssb_step_create(None, None) == L.SSB_ERR_INVALID_ARGUMENT
    cfg = L.SsbAdamConfig(1e-3, 1e-3, 1e-3, 1e-3, 1e-3, 1e-3, 0.0, 1.0, 0, 0)   # step 0 is invalid
    s = L.SsbSplats()
    assert lib.ssb_adam_step(C.byref(s), C.byref(s), C.byref(s), C.byref(s), 0, 4, C.byref(cfg), None) == L.SSB_ERR_INVALID_ARGUMENT
    sel = C.c_int32(0)
    one = C.c_void_p(8)
    assert lib.ssb_sort_pairs_u64(one, one, one, one, one, 10, 40, 30, one, 1 << 30, C.byref(sel), None) == L.SSB_ERR_INVALID_ARGUMENT
    assert lib.ssb_quant_encode(one, 10, 12, one, one, None) == L.SSB_ERR_INVALID_ARGUMENT
    # the optional entry points reject what their reference counterparts throw on
    assert lib.ssb_raster_bwd_accum(one, 4, one, one, 4, one, 1, 16, 16, None, one, one, one, None, None, one, 9, None, 4, None, one, None,
                                    None) == L.SSB_ERR_INVALID_ARGUMENT                       # not a DensifyAccumMode
    assert lib.ssb_raster_bwd_accum(one, 4, one, one, 4, one, 1, 16, 16, None, one, one, one, None, None, one, L.SSB_ACCUM_AVG, None, 4, None, one,
                                    None, None) == L.SSB_ERR_INVALID_ARGUMENT                 # average without a denominator array
    assert lib.ssb_loss_l1_ssim_fwdbwd_map(one, one, 1, 16, 16, 0.8, 0.2, one, None, 2, 1.0, None, None) == L.SSB_ERR_INVALID_ARGUMENT
    assert lib.ssb_adam_step_sh_quantized_ex(one, one, one, one, one, 16, 5, 0, 256, 256, C.byref(L.SsbAdamConfig(0, 0, 0, 0, 0, 1e-3, 0, 1, 1, 0)),
                                             None, 1, None) == L.SSB_ERR_INVALID_ARGUMENT     # optim_bits must be 4 or 8
    ex = L.SsbAdamExtras(0, 0, 0, 0, 0, 0, 0, 1, None, None, 4, None)                        # scale-agnostic mean without radii
    ok_cfg = L.SsbAdamConfig(1e-3, 1e-3, 1e-3, 1e-3, 1e-3, 1e-3, 0.0, 1.0, 1, 0)
    assert lib.ssb_adam_step_ex(C.byref(s), C.byref(s), C.byref(s), C.byref(s), 0, 4, C.byref(ok_cfg), C.byref(ex), None) == L.SSB_ERR_INVALID_ARGUMENT
    assert lib.ssb_step_set_densify(None, 1, 1.0, 1, one, None) == L.SSB_ERR_INVALID_ARGUMENT
    cams = L.SsbCameras()
    cams.count, cams.width, cams.height, cams.model = 1, 64, 64, 7    # not a camera model
    sp = L.SsbSplats()
    sp.features_sh = 8
    assert lib.ssb_project_fwd(C.byref(sp), None, 0, C.byref(cams), one, one, None, one, None) == L.SSB_ERR_UNSUPPORTED
    # (camera model, lens-distortion tier) pairs outside the reference's instantiation table are refused, as it refuses them
    for model, tier, want in ((L.CAMERA_PINHOLE, L.DISTORTION_RATIONAL, L.SSB_OK), (L.CAMERA_FISHEYE, L.DISTORTION_THIN_PRISM, L.SSB_OK),
                              (L.CAMERA_FISHEYE, L.DISTORTION_RATIONAL, L.SSB_ERR_UNSUPPORTED), (L.CAMERA_EQUIRECT, L.DISTORTION_OPENCV, L.SSB_ERR_UNSUPPORTED),
                              (L.CAMERA_PINHOLE, 4, L.SSB_ERR_UNSUPPORTED)):
        cams.model, cams.distortion = model, tier
        assert lib.ssb_project_fwd(C.byref(sp), None, 0, C.byref(cams), one, one, None, one, None) == want, (model, tier)
    assert b"distortion" in lib.ssb_last_error_string()
    # loss configuration
    bad = L.SsbLossConfig(0.8, 0.2, 0, 0, None, 0, 0)
    assert lib.ssb_loss_workspace_bytes(1, 16, 16, C.byref(bad)) == L.SSB_ERR_INVALID_ARGUMENT
    ok = L.SsbLossConfig(0.8, 0.2, 3, 1, None, 0, 0)
    assert lib.ssb_loss_workspace_bytes(1, 1080, 1920, C.byref(ok)) < 1080 * 1920 * (12 * 3 + 4) // 2
    assert lib.ssb_tile_active(None, 1, 4, 4, 64, 64, one, None) == L.SSB_ERR_INVALID_ARGUMENT


def test_packed_projection_workspaces_are_a_few_bytes_per_pair():
    """The packed projection keeps memory proportional to the visible pairs: its scratch is one 4-byte flag (forward) or
    one 4-byte slot index (backward) per (view, splat) pair, not a copy of every pair's outputs."""
    lib = L.load()
    for n, views in ((1_000_000, 16), (10_000_000, 8), (1000, 1)):
        pairs = n * views
        assert lib.ssb_project_fwd_packed_workspace_bytes(n, views) <= 8 * pairs + 1024
        assert lib.ssb_project_bwd_packed_workspace_bytes(n, views) <= 8 * pairs + 1024
