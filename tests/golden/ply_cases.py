"""Inputs of the splat.ply fixtures (shared by the generator and the tests): a numpy restatement of the reference's PLY
writer (src/engine/EngineCheckpoint.cpp:275-330) and a few files in other dialects its reader accepts."""
import numpy as np

OPA_MIN = np.float32(-5.5373)
K = 15


def splats(n=700, seed=31):
    """Raw splat arrays with non-finite entries and low opacities sprinkled in."""
    rng = np.random.default_rng(seed)
    sp = dict(means=rng.normal(size=(n, 3)), quats=rng.normal(size=(n, 4)), scales=rng.normal(-3, 1, size=(n, 3)),
              opacities=rng.normal(0, 4, size=n), features_dc=rng.normal(0, 0.5, size=(n, 3)),
              features_sh=rng.normal(0, 0.1, size=(n, K, 3)))
    sp = {k: v.astype(np.float32) for k, v in sp.items()}
    sp["means"][5, 1] = np.nan
    sp["quats"][17, 3] = np.inf
    sp["scales"][101, 0] = -np.inf
    sp["opacities"][300] = np.nan
    sp["features_dc"][401, 2] = np.nan
    sp["features_sh"][555, 7, 1] = np.inf
    sp["opacities"][600] = OPA_MIN                 # exactly the threshold: kept
    sp["opacities"][601] = np.nextafter(OPA_MIN, np.float32(-10))      # just below: dropped
    return sp


def keep_mask(sp, sh_is_quantised=False):
    ok = np.isfinite(sp["means"]).all(1) & np.isfinite(sp["quats"]).all(1) & np.isfinite(sp["scales"]).all(1)
    ok &= np.isfinite(sp["opacities"]) & np.isfinite(sp["features_dc"]).all(1)
    if not sh_is_quantised:
        ok &= np.isfinite(sp["features_sh"]).reshape(len(ok), -1).all(1)
    with np.errstate(invalid="ignore"):
        ok &= ~(sp["opacities"] < OPA_MIN)
    return ok


def header(kept):
    lines = ["ply", "format binary_little_endian 1.0", f"element vertex {kept}"]
    lines += [f"property float {a}" for a in ("x", "y", "z", "nx", "ny", "nz", "f_dc_0", "f_dc_1", "f_dc_2")]
    lines += [f"property float f_rest_{j}" for j in range(3 * K)]
    lines += [f"property float {a}" for a in ("opacity", "scale_0", "scale_1", "scale_2", "rot_0", "rot_1", "rot_2", "rot_3")]
    return ("\n".join(lines) + "\nend_header\n").encode()


def rows(sp, keep, sh_values=None):
    """[kept][62] float32: the vertex rows in the writer's column order; sh_values [n][K][3] replaces features_sh."""
    sh = sp["features_sh"] if sh_values is None else sh_values
    n = keep.sum()
    r = np.zeros((n, 62), np.float32)
    r[:, 0:3] = sp["means"][keep]
    r[:, 6:9] = sp["features_dc"][keep]
    r[:, 9:54] = sh[keep].transpose(0, 2, 1).reshape(n, 45)           # channel-major
    r[:, 54] = sp["opacities"][keep]
    r[:, 55:58] = sp["scales"][keep]
    r[:, 58:62] = sp["quats"][keep]
    return r


def file_bytes(sp, sh_values=None, sh_is_quantised=False):
    keep = keep_mask(sp, sh_is_quantised)
    return header(int(keep.sum())) + rows(sp, keep, sh_values).tobytes()


def dialects(seed=32):
    """{name: (file bytes, expected arrays)}: files the reference's reader accepts that its writer never makes."""
    rng = np.random.default_rng(seed)
    n = 9
    cols = ["x", "y", "z", "opacity", "scale_0", "scale_1", "scale_2", "rot_0", "rot_1", "rot_2", "rot_3", "f_dc_0", "f_dc_1", "f_dc_2"]
    vals = {c: rng.normal(size=n).astype(np.float32) for c in cols}
    want = dict(means=np.stack([vals["x"], vals["y"], vals["z"]], 1), opacities=vals["opacity"],
                scales=np.stack([vals[f"scale_{k}"] for k in range(3)], 1), quats=np.stack([vals[f"rot_{k}"] for k in range(4)], 1),
                features_dc=np.stack([vals[f"f_dc_{k}"] for k in range(3)], 1))
    out = {}
    # ASCII, no f_rest (degree 0), properties in another order, a comment and a second element after the vertices
    order = list(reversed(cols))
    text = "ply\nformat ascii 1.0\ncomment made by hand\nelement vertex %d\n" % n
    text += "".join(f"property float {c}\n" for c in order) + "element face 1\nproperty list uchar int vertex_indices\nend_header\n"
    text += "".join(" ".join(repr(float(vals[c][i])) for c in order) + "\n" for i in range(n)) + "3 0 1 2\n"
    out["ascii_deg0"] = (text.encode(), dict(want, sh_degree=0))
    # binary, degree 1 (9 f_rest columns), doubles for the positions, a uchar column in between, CRLF header lines
    rest = rng.normal(size=(n, 3, 3)).astype(np.float32)            # [n][coefficient][channel]
    props = [("double", "x"), ("double", "y"), ("double", "z"), ("uchar", "flag")] + [("float", c) for c in cols[3:]]
    props += [("float", f"f_rest_{j}") for j in range(9)]
    hdr = "ply\r\nformat binary_little_endian 1.0\r\nelement vertex %d\r\n" % n + "".join(f"property {t} {c}\r\n" for t, c in props) + "end_header\r\n"
    body = b""
    for i in range(n):
        body += np.array([vals["x"][i], vals["y"][i], vals["z"][i]], np.float64).tobytes() + bytes([i])
        body += np.array([vals[c][i] for c in cols[3:]], np.float32).tobytes()
        body += rest[i].T.reshape(-1).astype(np.float32).tobytes()          # channel-major
    out["binary_deg1"] = (hdr.encode() + body, dict(want, sh_degree=1, features_sh=rest))
    return out


NOT_SPLATS = {
    "points_only": b"ply\nformat ascii 1.0\nelement vertex 1\nproperty float x\nproperty float y\nproperty float z\nend_header\n0 0 0\n",
    "not_ply": b"hello\n",
    "vertex_list": (b"ply\nformat ascii 1.0\nelement vertex 1\nproperty list uchar int idx\nproperty float x\nend_header\n"),
    "rest_not_whole": None,      # filled below: 4 f_rest columns
}
_c = ["x", "y", "z", "opacity", "scale_0", "scale_1", "scale_2", "rot_0", "rot_1", "rot_2", "rot_3", "f_dc_0", "f_dc_1", "f_dc_2"] + [f"f_rest_{j}" for j in range(4)]
NOT_SPLATS["rest_not_whole"] = ("ply\nformat ascii 1.0\nelement vertex 1\n" + "".join(f"property float {c}\n" for c in _c) + "end_header\n" +
                                " ".join("0" for _ in _c) + "\n").encode()
