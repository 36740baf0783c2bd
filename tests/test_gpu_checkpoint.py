"""Checkpoints on the GPU: a Trainer saved and restored through state.tar, device arrays larger than the
staging buffers, and -- where the reference-side library (oracle/_ref/libssb_ref.so) is present -- the
library's file compared byte for byte with the one the reference's tar_write_npy_device writes for the
same device buffers, and handed to the reference's reader."""
import ctypes as C
import io
import os
import tarfile

import numpy as np
import pytest

torch = pytest.importorskip("torch")

from spirula_studio_b200 import checkpoint as ck, lib as L, scenes  # noqa: E402

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_SO = os.path.join(ROOT, "oracle", "_ref", "libssb_ref.so")
DEV = "cuda:0"


@pytest.fixture(scope="module")
def lib():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return L.load()


def small_scene(quant):
    cfg = scenes.scaled(scenes.CONFIGS["plumbing_50k"], n_splats=9000, width=176, height=128, n_views=2)
    cfg.rig, cfg.rig_radius, cfg.log_scale_mu = "ring", 3.0, -3.0
    if quant:
        cfg.sh_value_bits, cfg.sh_optim_bits = 16, 8
    sp = scenes.make_splats(cfg)
    vm, K = scenes.make_cameras(cfg)
    gt = np.stack([scenes.make_target(cfg, v) for v in range(cfg.n_views)])
    return cfg, sp, tuple(torch.from_numpy(a).pin_memory() for a in (vm, K, gt))


@pytest.mark.parametrize("quant", [False, True])
def test_trainer_resumes_from_state_tar(lib, tmp_path, quant):
    from spirula_studio_b200.trainer import Trainer
    cfg, sp, host = small_scene(quant)
    tr = Trainer(cfg, sp, device=DEV)
    for _ in range(3):
        tr.train_step(*host, cfg.n_views)
    path = ck.save_checkpoint(tr, str(tmp_path))
    saved = {n: t.clone() for n, t, _ in ck.saved_buffers(tr)}

    # the file, read by tarfile + numpy: the reference's member names in slot order, flat arrays, same bytes
    with tarfile.open(path) as t:
        infos = t.getmembers()
        assert [m.name for m in infos] == ["state.json"] + [n + ".npy" for n in saved]
        assert t.extractfile(infos[0]).read().decode() == ck.state_json(tr, 3)
        for info, (name, want) in zip(infos[1:], saved.items()):
            a = np.load(io.BytesIO(t.extractfile(info).read()))
            assert a.ndim == 1 and a.dtype == (np.uint8 if want.dtype == torch.uint8 else np.float32)
            assert a.tobytes() == want.cpu().numpy().tobytes(), name

    # a fresh trainer restored from it holds exactly the saved state and goes on from the saved step
    sp0 = {k: np.zeros_like(v) for k, v in sp.items()}
    sp0["quats"][:, 0] = 1.0
    tr2 = Trainer(cfg, sp0, device=DEV)
    assert ck.load_checkpoint(tr2, str(tmp_path)) == 3 and tr2.iteration == 3
    for (name, got, _), want in zip(ck.saved_buffers(tr2), saved.values()):
        assert torch.equal(got, want), name
    la, lb = tr.train_step(*host, cfg.n_views), tr2.train_step(*host, cfg.n_views)
    assert abs(la[2] - lb[2]) <= 1e-4 * abs(la[2])
    assert tr.iteration == tr2.iteration == 4
    for k in ("means", "scales", "opacities"):
        a, b = tr.params[k], tr2.params[k]
        assert (a - b).abs().max().item() <= 1e-3 * cfg.lrs["lr_" + k] + 1e-7 * a.abs().max().item() or \
            ((a - b).abs() > 1e-6).float().mean().item() < 1e-2, k

    # a trainer of another capacity or another storage layout is refused, as the reference refuses it
    cfg3, sp3, _ = small_scene(quant)
    cfg3 = scenes.scaled(cfg3, n_splats=cfg.n_splats - 512)
    tr3 = Trainer(cfg3, {k: v[: cfg3.n_splats] for k, v in sp3.items()}, device=DEV)
    with pytest.raises(RuntimeError, match="max_num_splats mismatch"):
        ck.load_checkpoint(tr3, str(tmp_path))
    cfg4, sp4, _ = small_scene(not quant)
    tr4 = Trainer(cfg4, sp4, device=DEV)
    with pytest.raises(RuntimeError, match="layout"):
        ck.load_checkpoint(tr4, str(tmp_path))
    for t_ in (tr, tr2, tr3, tr4):
        t_.close()


@pytest.mark.parametrize("quant", [False, True])
def test_trainer_with_16bit_non_sh_moments_tracks_fp32_and_resumes(lib, tmp_path, quant):
    """non_sh_optim_bits = 16: the moments of the five non-SH arrays live in 16-bit codes.  The parameters follow the trainer
    with fp32 moments closely (a code is 1/65535 of its block's range), the checkpoint carries the reference's
    eng.<attr>_qfpbo slots instead of the fp32 pairs, and a restored trainer goes on identically."""
    from spirula_studio_b200.trainer import Trainer
    cfg, sp, host = small_scene(quant)
    tr32, tr16 = Trainer(cfg, sp, device=DEV), Trainer(cfg, sp, device=DEV, non_sh_optim_bits=16)
    for _ in range(4):
        la, lb = tr32.train_step(*host, cfg.n_views), tr16.train_step(*host, cfg.n_views)
    assert abs(la[2] - lb[2]) <= 2e-3 * abs(la[2])
    for k in ("means", "quats", "scales", "opacities", "features_dc"):
        a, b = tr32.params[k], tr16.params[k]
        # An early Adam step is about +-lr whatever the gradient's size, so a cell whose gradient is near zero may take
        # the other sign after the smallest perturbation: bounded by the four steps, and rare.  Everywhere else the
        # quantised moments change a step by a small fraction of lr.
        d = (a - b).abs()
        assert d.max().item() <= 8.0 * cfg.lrs["lr_" + k], k
        assert (d > 0.02 * cfg.lrs["lr_" + k]).float().mean().item() < 0.02, k
    assert tr16.nsq_packed["means"].any() and tr16.nsq_bounds["features_dc"].any()
    path = ck.save_checkpoint(tr16, str(tmp_path))
    with tarfile.open(path) as t:
        names = [m.name for m in t.getmembers()]
        text = t.extractfile("state.json").read().decode()
    assert '"non_sh_optim_bits": 16' in text
    assert "eng.means_qfpbo.q.npy" in names and "eng.features_dc_qfpbo.qb.npy" in names and "eng.g1_means.npy" not in names
    if quant:       # the reference's slot order: fp32 moments, the qfpbo states, the SH state, the SH values
        assert names.index("eng.features_dc_qfpbo.qb.npy") < names.index("eng.sh_quant.q.npy")
    else:
        assert names.index("eng.g2_features_sh.npy") < names.index("eng.means_qfpbo.q.npy")
    tr2 = Trainer(cfg, sp, device=DEV, non_sh_optim_bits=16)
    assert ck.load_checkpoint(tr2, str(tmp_path)) == 4
    for (name, got, _), (_, want, _) in zip(ck.saved_buffers(tr2), ck.saved_buffers(tr16)):
        assert torch.equal(got, want), name
    with pytest.raises(RuntimeError, match="layout"):
        ck.load_checkpoint(tr32, str(tmp_path))
    for t_ in (tr32, tr16, tr2):
        t_.close()


def test_densifying_run_resumes_with_its_strategy_state(lib, tmp_path):
    """A checkpoint taken in the middle of a densifying run carries the number of splats in use (state.json, and the PLY holds
    only those), the view radii and the score accumulator under the reference's slot names; a fresh trainer + strategy
    restored from it grows exactly as the original does."""
    from spirula_studio_b200.densify import DensifyConfig, Densifier
    from spirula_studio_b200.trainer import Trainer
    cfg = scenes.scaled(scenes.CONFIGS["plumbing_50k"], n_splats=12032, width=176, height=128, n_views=2)
    cfg.rig, cfg.rig_radius, cfg.log_scale_mu = "ring", 3.0, -3.0
    cfg.sh_value_bits, cfg.sh_optim_bits = 16, 8
    sp = scenes.make_splats(cfg)
    vm, K = scenes.make_cameras(cfg)
    gt = np.stack([scenes.make_target(cfg, v) for v in range(cfg.n_views)])
    host = tuple(torch.from_numpy(a).pin_memory() for a in (vm, K, gt))
    dc = DensifyConfig(refine_start_iter=2, refine_stop_iter=1000, refine_every=4, growth_factor=1.1, noise_lr=80.0 * 1.6e-4, noise_lr_final=0.8 * 1.6e-4)
    steps = 20

    def run(tr, dn, first, last):
        counts = []
        for step in range(first, last):
            dn.before_step()
            tr.train_step(*host, cfg.n_views)
            dn.after_step(step, steps)
            counts.append(dn.count)
        return counts

    from spirula_studio_b200.trainer import OptimOptions
    tr = Trainer(cfg, sp, device=DEV, optim=OptimOptions())        # the reference's stock optimiser flags: radii and counters are state too
    dn = Densifier(tr, dc, 8000)
    assert dn.radii is tr.radii
    run(tr, dn, 0, 10)
    assert 8000 < dn.count < cfg.n_splats and dn.accum_buffer.any()
    path = ck.save_checkpoint(tr, str(tmp_path), step=10, densifier=dn)
    with tarfile.open(path) as t:
        names = [m.name for m in t.getmembers()]
        text = t.extractfile("state.json").read().decode()
    assert names[-3:] == ["eng.radii.npy", "eng.accum_buffer.npy", "eng.bias_correction_steps.npy"] and f'"cur_num_splats": {dn.count}' in text
    assert '"use_per_splat_bias_correction": 1' in text
    assert f'"max_num_splats": {cfg.n_splats}' in text
    num = C.c_int64(0)
    deg = C.c_int32(0)
    L.check(lib.ssb_ply_info(str(tmp_path / "splat.ply").encode(), C.byref(num), C.byref(deg)))
    assert 0 < num.value <= dn.count                      # unused slots (opacity logit -30) never reach the PLY
    tr2 = Trainer(cfg, {k: np.zeros_like(v) + (1.0 if k == "quats" else 0.0) for k, v in sp.items()}, device=DEV, optim=OptimOptions())
    dn2 = Densifier(tr2, dc, 1)
    assert ck.load_checkpoint(tr2, str(tmp_path), densifier=dn2) == 10
    assert dn2.count == dn.count and torch.equal(dn2.accum_buffer, dn.accum_buffer) and torch.equal(dn2.radii, dn.radii)
    assert torch.equal(tr2.steps, tr.steps) and tr.steps.max().item() == 10 and tr.steps.min().item() < 10       # relocated splats restart their counters
    plain = Trainer(cfg, sp, device=DEV)
    with pytest.raises(RuntimeError, match="layout"):
        ck.load_checkpoint(plain, str(tmp_path))
    plain.close()
    a, b = run(tr, dn, 10, steps), run(tr2, dn2, 10, steps)
    assert a == b and a[-1] > a[0]
    for k in ("means", "scales", "opacities"):
        x, y = tr.params[k][: dn.count * (tr.params[k].numel() // cfg.n_splats)], tr2.params[k][: dn.count * (tr2.params[k].numel() // cfg.n_splats)]
        assert ((x - y).abs() > 1e-3 * (1.0 + y.abs())).float().mean().item() < 0.02, k
    tr.close(); tr2.close()


def test_device_arrays_larger_than_the_staging_buffers(lib, tmp_path):
    # 80 MiB + 20 bytes: three staging chunks, the last one ragged; both staging buffers get reused
    n = (80 << 20) // 4 + 5
    g = torch.Generator(device=DEV).manual_seed(5)
    a = torch.randint(-2**31, 2**31 - 1, (n,), dtype=torch.int32, device=DEV, generator=g)
    small = torch.arange(7, dtype=torch.float32, device=DEV)
    path = str(tmp_path / "big.tar")
    w, r = C.c_void_p(), C.c_void_p()
    L.check(lib.ssb_ckpt_writer_open(path.encode(), C.byref(w)))
    L.check(lib.ssb_ckpt_write_device(w, b"big.npy", L.ptr(a), n * 4, ck.DTYPE_I4, None))
    L.check(lib.ssb_ckpt_write_device(w, b"small.npy", L.ptr(small), 28, ck.DTYPE_F4, None))
    L.check(lib.ssb_ckpt_write_device(w, b"empty.npy", None, 0, ck.DTYPE_F4, None))
    L.check(lib.ssb_ckpt_writer_close(w))
    with tarfile.open(path) as t:
        got = np.load(io.BytesIO(t.extractfile("big.npy").read()))
        assert got.dtype == np.int32 and np.array_equal(got, a.cpu().numpy())
        assert np.load(io.BytesIO(t.extractfile("empty.npy").read())).shape == (0,)
    b = torch.zeros_like(a)
    s2 = torch.zeros_like(small)
    L.check(lib.ssb_ckpt_reader_open(path.encode(), C.byref(r)))
    L.check(lib.ssb_ckpt_read_device(r, b"big.npy", L.ptr(b), n * 4, None))
    L.check(lib.ssb_ckpt_read_device(r, b"small.npy", L.ptr(s2), 28, None))
    assert lib.ssb_ckpt_read_device(r, b"small.npy", L.ptr(s2), 24, None) == L.SSB_ERR_CAPACITY
    L.check(lib.ssb_ckpt_reader_close(r))
    assert torch.equal(a, b) and torch.equal(small, s2)


def test_file_is_the_reference_writers_and_its_reader_takes_it(lib, tmp_path):
    if not os.path.exists(REF_SO):
        pytest.skip("the reference-side library has not been built on this machine")
    ref = C.CDLL(REF_SO)
    ref.ref_ckpt_write.argtypes = [C.c_char_p, C.c_char_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]
    ref.ref_ckpt_read_device.argtypes = [C.c_char_p, C.c_char_p, C.c_void_p, C.c_uint64, C.c_char_p]
    ref.ref_ckpt_read_json.argtypes = [C.c_char_p, C.c_char_p, C.c_int]
    from spirula_studio_b200.trainer import Trainer
    cfg, sp, host = small_scene(True)
    tr = Trainer(cfg, sp, device=DEV)
    tr.train_step(*host, cfg.n_views)
    torch.cuda.synchronize()
    ours = ck.save_checkpoint(tr, str(tmp_path / "ours"))
    bufs = ck.saved_buffers(tr)
    # one more array past the reference's 32 MiB host chunk
    big = torch.randint(0, 255, ((40 << 20) + 3,), dtype=torch.uint8, device=DEV)
    w = C.c_void_p()
    ours_big = str(tmp_path / "ours_big.tar")
    L.check(lib.ssb_ckpt_writer_open(ours_big.encode(), C.byref(w)))
    text = ck.state_json(tr, tr.iteration).encode()
    L.check(lib.ssb_ckpt_write_bytes(w, b"state.json", text, len(text)))
    L.check(lib.ssb_ckpt_write_device(w, b"eng.radii.npy", L.ptr(big), big.numel(), ck.DTYPE_U1, None))
    L.check(lib.ssb_ckpt_writer_close(w))

    def ref_write(path, entries):
        n = len(entries)
        names = (C.c_char_p * n)(*[e[0].encode() for e in entries])
        ptrs = (C.c_void_p * n)(*[e[1].data_ptr() for e in entries])
        sizes = (C.c_uint64 * n)(*[e[1].numel() * e[1].element_size() for e in entries])
        tags = (C.c_uint8 * n)(*[e[2] for e in entries])
        assert ref.ref_ckpt_write(path.encode(), text, n, names, ptrs, sizes, tags, 1) == 0

    theirs, theirs_big = str(tmp_path / "theirs.tar"), str(tmp_path / "theirs_big.tar")
    ref_write(theirs, bufs)
    ref_write(theirs_big, [("eng.radii", big, ck.DTYPE_U1)])
    assert open(ours, "rb").read() == open(theirs, "rb").read()
    assert open(ours_big, "rb").read() == open(theirs_big, "rb").read()

    # the reference's reader on the library's file
    out = C.create_string_buffer(4096)
    assert ref.ref_ckpt_read_json(ours.encode(), out, 4096) == len(text) and out.value == text
    descr = C.create_string_buffer(8)
    for name, t, tag in bufs:
        back = torch.zeros_like(t)
        nbytes = t.numel() * t.element_size()
        assert ref.ref_ckpt_read_device(ours.encode(), name.encode(), back.data_ptr(), nbytes, descr) == 0, name
        assert descr.value.decode() == ("|u1" if tag == ck.DTYPE_U1 else "<f4")
        assert torch.equal(back, t), name
        assert ref.ref_ckpt_read_device(ours.encode(), name.encode(), back.data_ptr(), nbytes + 4, None) == -3
    back = torch.zeros_like(big)
    assert ref.ref_ckpt_read_device(ours_big.encode(), b"eng.radii", back.data_ptr(), big.numel(), None) == 0
    assert torch.equal(back, big)
    # and the library's reader on the reference's file
    tr2 = Trainer(cfg, sp, device=DEV)
    os.makedirs(tmp_path / "theirs")
    os.replace(theirs, tmp_path / "theirs" / "state.tar")
    assert ck.load_checkpoint(tr2, str(tmp_path / "theirs")) == 1
    for (name, got, _), (_, want, _) in zip(ck.saved_buffers(tr2), bufs):
        assert torch.equal(got, want), name
    tr.close(); tr2.close()
