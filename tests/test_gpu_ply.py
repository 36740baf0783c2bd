"""splat.ply on the GPU: ssb_ply_write against a numpy restatement of the reference's writer (byte for byte with fp32 SH,
dequantised values within an ulp with 8/16-bit SH), read back by the library's reader and -- where the reference-side
library is present -- by the reference's reader; a trainer's checkpoint directory holds both files."""
import ctypes as C
import os
import sys

import numpy as np
import pytest

torch = pytest.importorskip("torch")

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import ply_cases as P  # noqa: E402

from spirula_studio_b200 import checkpoint as ck, lib as L, scenes  # noqa: E402
from tests.test_ply_cpu import read  # noqa: E402

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
REF_SO = os.path.join(os.path.dirname(HERE), "oracle", "_ref", "libssb_ref.so")


@pytest.fixture(scope="module")
def lib():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return L.load()


def write(lib, path, spd, shq=None):
    kept = C.c_int64(-1)
    s = L.splats_struct(spd if shq is None else {**spd, "features_sh": None})
    L.check(lib.ssb_ply_write(path.encode(), C.byref(s), C.byref(shq) if shq is not None else None, spd["means"].shape[0] // 3, C.byref(kept), None))
    return kept.value


@pytest.mark.parametrize("n", [700, 300_000])
def test_writer_is_the_reference_writers_file(lib, tmp_path, n):
    sp = P.splats(n=n)
    spd = {k: torch.from_numpy(v.reshape(-1)).to(DEV) for k, v in sp.items()}
    path = str(tmp_path / "splat.ply")
    kept = write(lib, path, spd)
    keep = P.keep_mask(sp)
    assert kept == keep.sum() < n
    data = open(path, "rb").read()
    assert data == P.file_bytes(sp)                 # header text, order of the kept splats, every value
    rc, a = read(lib, path)
    assert rc == L.SSB_OK
    for k in ("means", "quats", "scales", "opacities", "features_dc", "features_sh"):
        assert np.array_equal(a[k], sp[k][keep]), k
    if os.path.exists(REF_SO):
        ref = C.CDLL(REF_SO)
        num, deg = C.c_int64(0), C.c_int(0)
        assert ref.ref_ply_info(path.encode(), C.byref(num), C.byref(deg)) == 0 and (num.value, deg.value) == (kept, 3)
        b = {k: np.zeros_like(v) for k, v in a.items() if k != "sh_degree"}
        p = lambda x: x.ctypes.data_as(C.c_void_p)
        assert ref.ref_ply_read(path.encode(), p(b["means"]), p(b["quats"]), p(b["scales"]), p(b["opacities"]), p(b["features_dc"]), p(b["features_sh"])) == 0
        for k in b:
            assert np.array_equal(a[k], b[k]), k


@pytest.mark.parametrize("bits,stride", [(16, 256), (8, 256), (16, 0)])
def test_writer_dequantises_sh_values(lib, tmp_path, bits, stride):
    sp = P.splats(n=1000)
    n = 1000
    cells = n * 45
    rng = np.random.default_rng(3)
    codes = rng.integers(0, 1 << bits, size=cells, dtype=np.uint16 if bits == 16 else np.uint8)
    cell_stride = stride if stride > 0 else 256 * 45
    nb = (cells + cell_stride - 1) // cell_stride
    lo = rng.uniform(-0.3, 0.0, nb).astype(np.float32)
    hi = (lo + rng.uniform(0.05, 0.5, nb)).astype(np.float32)
    blk = np.arange(cells) // cell_stride
    qmax = np.float32(1.0 / (65535.0 if bits == 16 else 255.0))
    values = (lo[blk] + (hi[blk] - lo[blk]) * (codes.astype(np.float32) * qmax)).astype(np.float32).reshape(n, 15, 3)
    spd = {k: torch.from_numpy(v.reshape(-1)).to(DEV) for k, v in sp.items()}
    d_codes = torch.from_numpy(codes.view(np.uint8)).to(DEV)
    d_bounds = torch.from_numpy(np.stack([lo, hi], 1).reshape(-1)).to(DEV)
    shq = L.shq_struct(d_codes, d_bounds, bits, stride)
    path = str(tmp_path / "q.ply")
    kept = write(lib, path, spd, shq)
    keep = P.keep_mask(sp, sh_is_quantised=True)            # quantised values are finite by construction: SH is not looked at
    assert kept == keep.sum() and keep[555] and not keep[[5, 17, 101, 300, 401, 601]].any()
    data = open(path, "rb").read()
    want = P.file_bytes(sp, sh_values=values, sh_is_quantised=True)
    hdr = P.header(kept)
    assert data[:len(hdr)] == hdr and len(data) == len(want)
    got_rows = np.frombuffer(data[len(hdr):], np.float32).reshape(kept, 62)
    want_rows = np.frombuffer(want[len(hdr):], np.float32).reshape(kept, 62)
    assert np.array_equal(got_rows[:, :9], want_rows[:, :9]) and np.array_equal(got_rows[:, 54:], want_rows[:, 54:])
    assert np.allclose(got_rows[:, 9:54], want_rows[:, 9:54], rtol=0, atol=1e-7)           # a fused multiply-add may round once less


def test_checkpoint_directory_holds_the_ply_and_the_state(lib, tmp_path):
    from spirula_studio_b200.trainer import Trainer
    cfg = scenes.scaled(scenes.CONFIGS["plumbing_50k"], n_splats=5000, width=96, height=64, n_views=1)
    cfg.sh_value_bits, cfg.sh_optim_bits = 16, 8
    sp = scenes.make_splats(cfg)
    sp["opacities"][:50] = -9.0
    tr = Trainer(cfg, sp, device=DEV)
    ck.save_checkpoint(tr, str(tmp_path))
    assert os.path.exists(tmp_path / "state.tar") and os.path.exists(tmp_path / "splat.ply")
    rc, a = read(lib, str(tmp_path / "splat.ply"))
    assert rc == L.SSB_OK and a["means"].shape[0] == 5000 - 50 and a["sh_degree"][0] == 3
    assert np.array_equal(a["means"], sp["means"][50:])
    from oracle import pyoracle as O
    packed, bounds = O.quant_encode(sp["features_sh"], 16)
    dec = O.quant_decode(packed, bounds, sp["features_sh"].size, 16).reshape(5000, 15, 3)
    assert np.allclose(a["features_sh"], dec[50:], rtol=0, atol=1e-6)
    tr.close()
