"""splat.ply on the CPU: the library's reader against what the reference's reader returned for the same files
(tests/golden/ply_read.npz, made by tests/golden/make_ply_golden.py), and its refusals."""
import ctypes as C
import os
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import ply_cases as P  # noqa: E402

from spirula_studio_b200 import lib as L  # noqa: E402


def read(lib, path):
    num, deg = C.c_int64(-1), C.c_int32(-1)
    rc = lib.ssb_ply_info(path.encode(), C.byref(num), C.byref(deg))
    if rc != L.SSB_OK:
        return rc, None
    n, k = num.value, (deg.value + 1) ** 2 - 1
    a = dict(means=np.zeros((n, 3), np.float32), quats=np.zeros((n, 4), np.float32), scales=np.zeros((n, 3), np.float32),
             opacities=np.zeros(n, np.float32), features_dc=np.zeros((n, 3), np.float32), features_sh=np.zeros((n, k, 3), np.float32))
    p = lambda x: x.ctypes.data_as(C.c_void_p)
    rc = lib.ssb_ply_read(path.encode(), n, deg.value, p(a["means"]), p(a["quats"]), p(a["scales"]), p(a["opacities"]), p(a["features_dc"]),
                          p(a["features_sh"]) if k else None)
    a["sh_degree"] = np.array([deg.value])
    return rc, a


@pytest.fixture(scope="module")
def gold():
    return dict(np.load(os.path.join(HERE, "golden", "ply_read.npz")))


def test_reader_returns_what_the_reference_reader_returns(tmp_path, gold):
    lib = L.load()
    files = {"writer": P.file_bytes(P.splats())}
    files.update({k: v[0] for k, v in P.dialects().items()})
    for name, data in files.items():
        path = str(tmp_path / (name + ".ply"))
        open(path, "wb").write(data)
        rc, a = read(lib, path)
        assert rc == L.SSB_OK, name
        for k, v in a.items():
            assert np.array_equal(v, gold[f"{name}_{k}"], equal_nan=True), (name, k)
    # and both return what was put in
    sp = P.splats()
    keep = P.keep_mask(sp)
    assert keep[600] and not keep[[5, 17, 101, 300, 401, 555, 601]].any() and 0.8 * len(keep) < keep.sum() < len(keep) - 7
    for k in ("means", "quats", "scales", "opacities", "features_dc", "features_sh"):
        assert np.array_equal(gold[f"writer_{k}"], sp[k][keep]), k
    for name, (_, want) in P.dialects().items():
        for k, v in want.items():
            assert np.allclose(gold[f"{name}_{k}"].reshape(np.shape(v)), v, rtol=0, atol=1e-6), (name, k)
    # without the SH columns (the mesher's use): same geometry
    path = str(tmp_path / "writer.ply")
    n = int(keep.sum())
    m, q, s, o, d = (np.zeros((n, w), np.float32) for w in (3, 4, 3, 1, 3))
    p = lambda x: x.ctypes.data_as(C.c_void_p)
    assert lib.ssb_ply_read(path.encode(), n, 3, p(m), p(q), p(s), p(o), p(d), None) == L.SSB_OK
    assert np.array_equal(m, sp["means"][keep]) and np.array_equal(o.reshape(-1), sp["opacities"][keep])


def test_files_the_reference_reader_refuses_are_refused(tmp_path, gold):
    lib = L.load()
    for name, data in P.NOT_SPLATS.items():
        path = str(tmp_path / (name + ".ply"))
        open(path, "wb").write(data)
        rc, _ = read(lib, path)
        assert gold[f"status_{name}"][0] != 0 and rc == L.SSB_ERR_UNSUPPORTED, name
    assert lib.ssb_ply_info(str(tmp_path / "missing.ply").encode(), None, None) == L.SSB_ERR_IO
    # the caller's sizes must be the file's
    path = str(tmp_path / "w.ply")
    open(path, "wb").write(P.file_bytes(P.splats()))
    one = np.zeros(8, np.float32).ctypes.data_as(C.c_void_p)
    assert lib.ssb_ply_read(path.encode(), 5, 3, one, one, one, one, one, None) == L.SSB_ERR_INVALID_ARGUMENT
    # a truncated body is an I/O error, not a crash
    open(path, "wb").write(P.file_bytes(P.splats())[:-100])
    rc, _ = read(lib, path)
    assert rc == L.SSB_ERR_IO
