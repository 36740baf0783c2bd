"""The allocation-free sort entry point (ssb_sort_pairs_u64_noalloc) against the
regular one (ssb_sort_pairs_u64), through the C ABI.

The variant exists for callers that are not allowed to create device memory at
the point where they sort (a plug-in whose host forbids cudaMalloc, a loop where
an allocation's device-wide synchronisation would stall other streams): its
scratch is a fixed array inside the library.  Two calls in a row are checked,
because the second one meets whatever the first left in that shared array.
This file sorts last in the suite on purpose: a run that stops at the first
failure has then already run every other test."""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")

from spirula_studio_b200 import lib as L  # noqa: E402

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _sort(lib, fn_noalloc, keys, vals, n, cap, b0, b1):
    ka = torch.zeros(cap, dtype=torch.int64, device=DEV); ka[:n] = keys
    va = torch.zeros(cap, dtype=torch.int32, device=DEV); va[:n] = vals
    kb, vb = torch.zeros_like(ka), torch.zeros_like(va)
    n_dev = torch.tensor([n], dtype=torch.int64, device=DEV)
    sel = C.c_int32(-1)
    if fn_noalloc:
        st = lib.ssb_sort_pairs_u64_noalloc(L.ptr(ka), L.ptr(va), L.ptr(kb), L.ptr(vb), L.ptr(n_dev), cap, b0, b1, C.byref(sel), None)
    else:
        ws_bytes = lib.ssb_sort_workspace_bytes(cap)
        ws = torch.zeros(ws_bytes, dtype=torch.uint8, device=DEV)
        st = lib.ssb_sort_pairs_u64(L.ptr(ka), L.ptr(va), L.ptr(kb), L.ptr(vb), L.ptr(n_dev), cap, b0, b1, L.ptr(ws), ws_bytes, C.byref(sel), None)
    torch.cuda.synchronize()
    assert st == 0, lib.ssb_last_error_string()
    # did any bounded wait inside the sort give up?  NULL names the built-in scratch of the current device
    assert lib.ssb_sort_check(None if fn_noalloc else L.ptr(ws), None) == L.SSB_OK, lib.ssb_last_error_string()
    out_k, out_v = (kb, vb) if sel.value == 1 else (ka, va)
    return out_k[:n].cpu().numpy(), out_v[:n].cpu().numpy()


def test_noalloc_sort_matches_regular_sort_twice_in_a_row():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    lib = L.load()
    g = torch.Generator(device=DEV); g.manual_seed(7)
    cases = [(700_001, 1 << 20, 0, 45), (123_457, 200_000, 0, 45)]      # the second call is smaller than the first
    for n, cap, b0, b1 in cases:
        tiles = torch.randint(0, 8160, (n,), device=DEV, generator=g, dtype=torch.int64)
        depth = torch.randint(0, 1 << 12, (n,), device=DEV, generator=g, dtype=torch.int64) | (1 << 31)   # many ties
        keys = (tiles << 32) | depth
        vals = torch.arange(n, device=DEV, dtype=torch.int32)
        k1, v1 = _sort(lib, True, keys, vals, n, cap, b0, b1)
        k0, v0 = _sort(lib, False, keys, vals, n, cap, b0, b1)
        assert np.array_equal(k1, k0) and np.array_equal(v1, v0)         # integer work: bit for bit
        assert np.all(np.diff(k1) >= 0)
    # beyond the built-in scratch: a clear error, nothing touched
    one = torch.zeros(8, dtype=torch.int64, device=DEV)
    sel = C.c_int32(5)
    st = lib.ssb_sort_pairs_u64_noalloc(L.ptr(one), L.ptr(one), L.ptr(one), L.ptr(one), L.ptr(one), (1 << 20) + 1, 0, 45, C.byref(sel), None)
    assert st == L.SSB_ERR_CAPACITY and b"1048576" in lib.ssb_last_error_string() and sel.value == 5
    # a negative capacity is refused by this entry point itself
    st = lib.ssb_sort_pairs_u64_noalloc(L.ptr(one), L.ptr(one), L.ptr(one), L.ptr(one), L.ptr(one), -1, 0, 45, C.byref(sel), None)
    assert st == L.SSB_ERR_INVALID_ARGUMENT and b"negative" in lib.ssb_last_error_string() and sel.value == 5
