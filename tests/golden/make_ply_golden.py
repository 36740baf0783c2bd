"""Generates tests/golden/ply_read.npz: what the REFERENCE's splat.ply reader (src/checkpoint/SplatPly.cpp, reached through
oracle/_ref/libssb_ref.so: oracle/ref_tool/ref_ply.cu) returns for the files of ply_cases.py.  Host only:

    make -C oracle -f Makefile.ref REF=<reference checkout>
    python tests/golden/make_ply_golden.py
"""
import ctypes as C
import os
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, HERE)
import ply_cases as P  # noqa: E402


def ref_read(ref, path):
    """(status, arrays) of the reference's reader."""
    num, deg = C.c_int64(0), C.c_int(0)
    rc = ref.ref_ply_info(path.encode(), C.byref(num), C.byref(deg))
    if rc != 0:
        return rc, None
    n, k = num.value, (deg.value + 1) ** 2 - 1
    a = dict(means=np.zeros((n, 3), np.float32), quats=np.zeros((n, 4), np.float32), scales=np.zeros((n, 3), np.float32),
             opacities=np.zeros(n, np.float32), features_dc=np.zeros((n, 3), np.float32), features_sh=np.zeros((n, k, 3), np.float32))
    p = lambda x: x.ctypes.data_as(C.c_void_p)
    rc = ref.ref_ply_read(path.encode(), p(a["means"]), p(a["quats"]), p(a["scales"]), p(a["opacities"]), p(a["features_dc"]),
                          p(a["features_sh"]) if k else None)
    a["sh_degree"] = np.array([deg.value])
    return rc, a


def main():
    out_dir = sys.argv[1] if len(sys.argv) > 1 else HERE
    ref = C.CDLL(os.path.join(ROOT, "oracle", "_ref", "libssb_ref.so"))
    out = {}
    files = {"writer": P.file_bytes(P.splats())}
    files.update({k: v[0] for k, v in P.dialects().items()})
    with tempfile.TemporaryDirectory() as tmp:
        for name, data in files.items():
            path = os.path.join(tmp, name + ".ply")
            open(path, "wb").write(data)
            rc, a = ref_read(ref, path)
            assert rc == 0, (name, rc)
            for k, v in a.items():
                out[f"{name}_{k}"] = v
        for name, data in P.NOT_SPLATS.items():
            path = os.path.join(tmp, name + ".ply")
            open(path, "wb").write(data)
            rc, _ = ref_read(ref, path)
            out[f"status_{name}"] = np.array([rc])
            print(name, "->", rc)
    np.savez_compressed(os.path.join(out_dir, "ply_read.npz"), **out)
    print("wrote ply_read.npz with", len(out), "arrays")


if __name__ == "__main__":
    main()
