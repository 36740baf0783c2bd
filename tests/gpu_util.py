"""Helpers for the GPU parity tests: move numpy arrays to the device and call
the C ABI of libssb_b200 with raw pointers."""
import ctypes as C

import numpy as np
import torch

from spirula_studio_b200 import lib as L

DEV = "cuda:0"


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.to(DEV)


def splats_dev(sp):
    return {k: dev(v) for k, v in sp.items() if v is not None}


def pack_screen(lib, proj):
    """Oracle projection outputs (reference ScreenBuffer arrays) -> device records."""
    m = proj["depths"].shape[0]
    rec = torch.zeros(m * L.SCREEN_REC_FLOATS, dtype=torch.float32, device=DEV)
    xy, depth, conic, opac, rgb = (dev(proj[k]) for k in ("xy", "depth", "conic", "opac", "rgb"))
    L.check(lib.ssb_screen_pack(L.ptr(xy), L.ptr(depth), L.ptr(conic), L.ptr(opac), L.ptr(rgb), m, L.ptr(rec), None))
    torch.cuda.synchronize()
    return rec


def unpack_screen(lib, rec, m):
    out = dict(xy=torch.zeros(m, 2, device=DEV), depth=torch.zeros(m, device=DEV), conic=torch.zeros(m, 3, device=DEV),
               opac=torch.zeros(m, device=DEV), rgb=torch.zeros(m, 3, device=DEV))
    L.check(lib.ssb_screen_unpack(L.ptr(rec), m, L.ptr(out["xy"]), L.ptr(out["depth"]), L.ptr(out["conic"]), L.ptr(out["opac"]),
                                  L.ptr(out["rgb"]), None))
    torch.cuda.synchronize()
    return {k: v.cpu().numpy() for k, v in out.items()}


def project_fwd(lib, sp_dev, viewmats, intrins, W, H, shq=None, n=None, model=0):
    n = n or sp_dev["means"].shape[0]
    vm, K = dev(viewmats), dev(intrins)
    Cn = vm.shape[0]
    aabb = torch.zeros(Cn * n, 4, device=DEV)
    depths = torch.zeros(Cn * n, device=DEV)
    radii = torch.zeros(n, device=DEV)
    rec = torch.zeros(Cn * n * L.SCREEN_REC_FLOATS, device=DEV)
    s = L.splats_struct(sp_dev if shq is None else {**sp_dev, "features_sh": None})
    cams = L.cameras_struct(vm, K, W, H, model=model)
    L.check(lib.ssb_project_fwd(C.byref(s), C.byref(shq) if shq is not None else None, n, C.byref(cams), L.ptr(aabb), L.ptr(depths),
                                L.ptr(radii), L.ptr(rec), None))
    torch.cuda.synchronize()
    return dict(aabb=aabb, depths=depths, radii=radii, rec=rec, vm=vm, K=K)


def tile_keys(lib, aabb, depths, rec, total, n_per_image, W, H, capacity, tile_active=None):
    ws_bytes = lib.ssb_tile_keys_workspace_bytes(total)
    ws = torch.zeros(ws_bytes, dtype=torch.uint8, device=DEV)
    counts = torch.zeros(max(total, 1), dtype=torch.int32, device=DEV)
    cum = torch.zeros(max(total, 1), dtype=torch.int32, device=DEV)
    keys = torch.zeros(max(capacity, 1), dtype=torch.int64, device=DEV)
    vals = torch.zeros(max(capacity, 1), dtype=torch.int32, device=DEV)
    n_dev = torch.zeros(1, dtype=torch.int64, device=DEV)
    m = C.c_int64(-1)
    if tile_active is not None:
        st = lib.ssb_tile_keys_live(L.ptr(aabb), L.ptr(depths), L.ptr(rec), total, n_per_image, W, H, L.ptr(ws), ws_bytes, L.ptr(counts), L.ptr(cum),
                                    L.ptr(keys), L.ptr(vals), capacity, L.ptr(n_dev), C.byref(m), L.ptr(tile_active), None)
    else:
        st = lib.ssb_tile_keys(L.ptr(aabb), L.ptr(depths), L.ptr(rec), total, n_per_image, W, H, L.ptr(ws), ws_bytes, L.ptr(counts), L.ptr(cum),
                               L.ptr(keys), L.ptr(vals), capacity, L.ptr(n_dev), C.byref(m), None)
    return st, m.value, counts, cum, keys, vals, n_dev


def intersect_tiles(lib, aabb, depths, rec, total, n_per_image, W, H, capacity, n_tiles_total, want_keys=True, tile_active=None):
    """The fused call: sorted keys (optional), sorted flatten ids, per-tile ranges, pair count."""
    ws_bytes = lib.ssb_intersect_tiles_workspace_bytes(n_tiles_total, capacity)
    ws = torch.zeros(ws_bytes, dtype=torch.uint8, device=DEV)
    keys = torch.full((max(capacity, 1),), -1, dtype=torch.int64, device=DEV) if want_keys else None
    vals = torch.full((max(capacity, 1),), -1, dtype=torch.int32, device=DEV)
    offs = torch.full((max(n_tiles_total, 1),), -7, dtype=torch.int32, device=DEV)
    n_dev = torch.full((1,), -1, dtype=torch.int64, device=DEV)
    if tile_active is not None:
        L.check(lib.ssb_intersect_tiles_live(L.ptr(aabb), L.ptr(depths), L.ptr(rec), total, n_per_image, W, H, L.ptr(ws), ws_bytes,
                                             L.ptr(keys) if want_keys else None, L.ptr(vals), capacity, L.ptr(offs), L.ptr(n_dev), L.ptr(tile_active), None))
    else:
        L.check(lib.ssb_intersect_tiles(L.ptr(aabb), L.ptr(depths), L.ptr(rec), total, n_per_image, W, H, L.ptr(ws), ws_bytes,
                                        L.ptr(keys) if want_keys else None, L.ptr(vals), capacity, L.ptr(offs), L.ptr(n_dev), None))
    torch.cuda.synchronize()
    return keys, vals, offs, int(n_dev.item())


def sort_pairs(lib, keys, vals, n_dev, capacity, begin_bit, end_bit):
    kb, vb = torch.zeros_like(keys), torch.zeros_like(vals)
    ws_bytes = lib.ssb_sort_workspace_bytes(capacity)
    ws = torch.zeros(ws_bytes, dtype=torch.uint8, device=DEV)
    sel = C.c_int32(-1)
    L.check(lib.ssb_sort_pairs_u64(L.ptr(keys), L.ptr(vals), L.ptr(kb), L.ptr(vb), L.ptr(n_dev), capacity, begin_bit, end_bit, L.ptr(ws),
                                   ws_bytes, C.byref(sel), None))
    L.check(lib.ssb_sort_check(L.ptr(ws), None))
    return (kb, vb) if sel.value == 1 else (keys, vals)


def tile_ranges(lib, sorted_keys, n_dev, capacity, n_tiles):
    offs = torch.full((n_tiles,), -7, dtype=torch.int32, device=DEV)
    L.check(lib.ssb_tile_ranges(L.ptr(sorted_keys), L.ptr(n_dev), capacity, n_tiles, L.ptr(offs), None))
    torch.cuda.synchronize()
    return offs


def raster_fwd(lib, rec, offs, flat, n_dev, I, W, H):
    P = I * H * W
    out = dict(rgb=torch.zeros(P, 3, device=DEV), depth=torch.zeros(P, device=DEV), T=torch.zeros(P, device=DEV),
               last_ids=torch.zeros(P, dtype=torch.int32, device=DEV))
    L.check(lib.ssb_raster_fwd(L.ptr(rec), rec.numel() // L.SCREEN_REC_FLOATS, L.ptr(offs), L.ptr(flat), flat.numel(), L.ptr(n_dev), I, W, H, L.ptr(out["rgb"]), L.ptr(out["depth"]),
                               L.ptr(out["T"]), L.ptr(out["last_ids"]), None))
    torch.cuda.synchronize()
    return out


def raster_bwd(lib, rec, offs, flat, n_dev, I, W, H, render, v_rgb, v_depth=None, v_T=None, pairs=None):
    v_rec = torch.zeros(pairs * L.SCREEN_REC_FLOATS, device=DEV)
    L.check(lib.ssb_raster_bwd(L.ptr(rec), min(pairs, rec.numel() // L.SCREEN_REC_FLOATS), L.ptr(offs), L.ptr(flat), flat.numel(), L.ptr(n_dev), I, W, H, L.ptr(render["depth"]), L.ptr(render["T"]),
                               L.ptr(render["last_ids"]), L.ptr(v_rgb), L.ptr(v_depth), L.ptr(v_T), L.ptr(v_rec), None))
    torch.cuda.synchronize()
    return v_rec


def vrec_to_arrays(v_rec, m):
    """Gradient records -> the reference's five gradient arrays (numpy)."""
    r = v_rec.view(m, 12).cpu().numpy()
    return dict(v_xy=r[:, 0:2].copy(), v_conic=r[:, 4:7].copy(), v_opac=r[:, 7].copy(), v_rgb=r[:, 8:11].copy(), v_depth=r[:, 11].copy())


def arrays_to_vrec(v, m):
    r = np.zeros((m, 12), np.float32)
    r[:, 0:2] = v["v_xy"]; r[:, 4:7] = v["v_conic"]; r[:, 7] = v["v_opac"]; r[:, 8:11] = v["v_rgb"]; r[:, 11] = v["v_depth"]
    return dev(r.reshape(-1))


def close_frac(got, ref, atol, rtol):
    """Fraction of elements violating |got-ref| <= atol + rtol*|ref| (the reference tools' tolerance model)."""
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    bad = ~(np.abs(got - ref) <= atol + rtol * np.abs(ref))
    return float(bad.mean()) if bad.size else 0.0


def tensor_from_device_ptr(address, shape, dtype=torch.float32):
    """Copies a raw device buffer owned by the library into a fresh torch tensor."""
    out = torch.empty(shape, dtype=dtype, device=DEV)
    rt = C.CDLL("libcudart.so.12")
    rt.cudaMemcpy.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int]
    torch.cuda.synchronize()
    err = rt.cudaMemcpy(C.c_void_p(out.data_ptr()), C.c_void_p(address), out.numel() * out.element_size(), 3)
    assert err == 0, f"cudaMemcpy failed with {err}"
    return out
