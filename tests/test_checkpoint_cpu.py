"""The checkpoint container without a GPU: the library's state.tar bytes against the fixture the
reference's own helpers wrote (tests/golden/make_ckpt_golden.py), and against numpy / tarfile as
independent readers and writers of the two formats."""
import ctypes as C
import io
import os
import sys
import tarfile

import numpy as np
import pytest

from spirula_studio_b200 import lib as L

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import ckpt_cases as K  # noqa: E402

GOLDEN_TAR = os.path.join(HERE, "golden", "ckpt_state.tar")


def write_archive(lib, path, members, json_text=K.STATE_JSON):
    w = C.c_void_p()
    L.check(lib.ssb_ckpt_writer_open(path.encode(), C.byref(w)))
    text = json_text.encode()
    L.check(lib.ssb_ckpt_write_bytes(w, b"state.json", text, len(text)))
    for name, tag, a in members:
        L.check(lib.ssb_ckpt_write_host(w, (name + ".npy").encode(), a.ctypes.data, a.nbytes, tag))
    L.check(lib.ssb_ckpt_writer_close(w))


def test_headers_match_the_reference_byte_for_byte():
    lib = L.load()
    gold = np.load(os.path.join(HERE, "golden", "ckpt_headers.npz"))
    buf = C.create_string_buffer(1024)
    for tag in range(len(K.DESCR)):
        for n in K.HEADER_NUMELS:
            ln = lib.ssb_ckpt_array_header(tag, n, buf, 1024)
            want = gold[f"npy_{tag}_{n}"].tobytes()
            assert ln == len(want) and ln % 64 == 0
            assert buf.raw[:ln] == want, (tag, n)
    for i, name in enumerate(K.HEADER_NAMES):
        for size in K.HEADER_SIZES:
            L.check(lib.ssb_ckpt_member_header(name.encode(), size, buf))
            assert buf.raw[:512] == gold[f"tar_{i}_{size}"].tobytes(), (name, size)
    assert lib.ssb_ckpt_array_header(10, 1, buf, 1024) == L.SSB_ERR_INVALID_ARGUMENT
    assert lib.ssb_ckpt_array_header(7, 1, buf, 8) == L.SSB_ERR_CAPACITY
    assert lib.ssb_ckpt_member_header(b"y" * 100, 1, buf) == L.SSB_ERR_INVALID_ARGUMENT


def test_archive_matches_the_reference_byte_for_byte(tmp_path):
    lib = L.load()
    path = str(tmp_path / "state.tar")
    write_archive(lib, path, K.members())
    assert open(path, "rb").read() == open(GOLDEN_TAR, "rb").read()


def test_numpy_and_tarfile_read_what_the_library_writes(tmp_path):
    lib = L.load()
    path = str(tmp_path / "state.tar")
    members = K.members(seed=11)
    write_archive(lib, path, members)
    with tarfile.open(path) as t:
        infos = t.getmembers()
        assert [m.name for m in infos] == ["state.json"] + [m[0] + ".npy" for m in members]
        assert t.extractfile(infos[0]).read().decode() == K.STATE_JSON
        for info, (name, tag, a) in zip(infos[1:], members):
            assert (info.mode, info.uid, info.gid, info.mtime, info.type) == (0o644, 0, 0, 0, tarfile.REGTYPE)
            got = np.load(io.BytesIO(t.extractfile(info).read()))
            assert got.dtype == a.dtype and got.shape == a.shape
            assert got.tobytes() == a.tobytes()
            assert info.offset_data % 512 == 0


@pytest.mark.parametrize("source", ["reference", "tarfile"])
def test_reader_takes_reference_and_foreign_archives(tmp_path, source):
    lib = L.load()
    members = K.members()
    if source == "reference":
        path = GOLDEN_TAR
    else:
        # GNU tar written by Python, arrays saved by numpy (NPY v1 headers of another length, v2 for one member)
        path = str(tmp_path / "foreign.tar")
        with tarfile.open(path, "w", format=tarfile.GNU_FORMAT) as t:
            def add(name, data):
                info = tarfile.TarInfo(name)
                info.size = len(data)
                t.addfile(info, io.BytesIO(data))
            add("state.json", K.STATE_JSON.encode())
            for i, (name, tag, a) in enumerate(members):
                b = io.BytesIO()
                if i == 1:
                    np.lib.format.write_array(b, a, version=(2, 0))
                else:
                    np.save(b, a)
                add(name + ".npy", b.getvalue())
    r = C.c_void_p()
    L.check(lib.ssb_ckpt_reader_open(path.encode(), C.byref(r)))
    assert lib.ssb_ckpt_member_count(r) == 1 + len(members)
    name_buf, size = C.create_string_buffer(128), C.c_uint64()
    L.check(lib.ssb_ckpt_member_info(r, 0, name_buf, 128, C.byref(size)))
    assert name_buf.value == b"state.json" and size.value == len(K.STATE_JSON)
    assert lib.ssb_ckpt_member_info(r, 1, name_buf, 4, None) == L.SSB_ERR_CAPACITY
    text = C.create_string_buffer(size.value)
    L.check(lib.ssb_ckpt_read_bytes(r, b"state.json", text, size.value, None))
    assert text.raw.decode() == K.STATE_JSON
    descr = C.create_string_buffer(8)
    for name, tag, a in members:
        member = (name + ".npy").encode()
        L.check(lib.ssb_ckpt_array_info(r, member, descr, 8, C.byref(size)))
        assert size.value == a.nbytes
        assert descr.value.decode().lstrip("<|") == K.DESCR[tag].lstrip("<|")
        got = np.empty_like(a)
        L.check(lib.ssb_ckpt_read_host(r, member, got.ctypes.data, got.nbytes))
        assert got.tobytes() == a.tobytes()
        # a buffer of another size is refused, as the reference refuses a slot whose byte size differs
        assert lib.ssb_ckpt_read_host(r, member, got.ctypes.data, got.nbytes + a.itemsize) == L.SSB_ERR_CAPACITY
    assert lib.ssb_ckpt_read_host(r, b"world.nothing.npy", None, 0) == L.SSB_ERR_INVALID_ARGUMENT
    L.check(lib.ssb_ckpt_reader_close(r))


def test_file_errors_are_statuses(tmp_path):
    lib = L.load()
    r, w = C.c_void_p(), C.c_void_p()
    assert lib.ssb_ckpt_reader_open(str(tmp_path / "missing.tar").encode(), C.byref(r)) == L.SSB_ERR_IO
    assert lib.ssb_ckpt_writer_open(str(tmp_path / "no_such_dir" / "state.tar").encode(), C.byref(w)) == L.SSB_ERR_IO
    assert lib.ssb_ckpt_writer_open(None, C.byref(w)) == L.SSB_ERR_INVALID_ARGUMENT
    # an empty archive: only the end-of-archive blocks
    path = str(tmp_path / "empty.tar")
    L.check(lib.ssb_ckpt_writer_open(path.encode(), C.byref(w)))
    assert lib.ssb_ckpt_write_host(w, b"a.npy", None, 6, 7) == L.SSB_ERR_INVALID_ARGUMENT      # 6 bytes are not whole floats
    L.check(lib.ssb_ckpt_writer_close(w))
    assert open(path, "rb").read() == bytes(1024)
    L.check(lib.ssb_ckpt_reader_open(path.encode(), C.byref(r)))
    assert lib.ssb_ckpt_member_count(r) == 0
    L.check(lib.ssb_ckpt_reader_close(r))


def test_manifest_text_and_slot_list_follow_the_reference():
    """state.json key order and formatting (src/engine/EngineCheckpoint.cpp:73-127) and the slot order of
    src/core/PoolSlots.h:88-125, on a stand-in for a trainer (no device needed)."""
    from types import SimpleNamespace
    from spirula_studio_b200 import checkpoint as ck
    from spirula_studio_b200.scenes import CONFIGS
    tr = SimpleNamespace(cfg=CONFIGS["mid_1m"], n=1000, quant=True, non_sh_optim_bits=32, steps=None, radii=None)
    text = ck.state_json(tr, 42)
    keys = [ln.split('"')[1] for ln in text.splitlines() if ln.startswith('  "')]
    assert keys == ["format_version", "full_resume", "quant_codec", "quant_block_size", "quant_eps", "step", "primitive",
                    "cur_num_splats", "max_num_splats", "num_sh", "sh_degree", "packed", "sh_optim_bits", "sh_value_bits",
                    "non_sh_optim_bits", "use_fused_proj_bwd_optim", "use_per_splat_bias_correction", "camera", "bilagrid_rgb",
                    "bilagrid_depth", "bilagrid_normal", "ppisp"]
    import json
    d = json.loads(text)
    assert (d["step"], d["max_num_splats"], d["sh_optim_bits"], d["sh_value_bits"], d["num_sh"]) == (42, 1000, 8, 16, 15)
    assert d["camera"] == {"num": 16, "width": 1920, "height": 1080, "model": "PINHOLE"}
    assert ck._json_value(text, "step") == 42 and ck._json_value(text, "primitive") == "3dgs"
    none = dict.fromkeys(("means", "quats", "scales", "opacities", "features_dc", "features_sh"))
    tr.params = tr.m1 = tr.m2 = none
    tr.sh_optim_packed = tr.sh_optim_bounds = tr.sh_packed = tr.sh_bounds = None
    names = [n for n, _, _ in ck.saved_buffers(tr)]
    geo = ["means", "quats", "scales", "opacities", "features_dc"]
    assert names == [f"world.{a}" for a in geo] + [f"eng.g1_{a}" for a in geo] + [f"eng.g2_{a}" for a in geo] + \
        ["eng.sh_quant.q", "eng.sh_quant.qb", "eng.world.sh_vq16.q", "eng.world.sh_vq16.qb"]
    tr.quant = False
    names = [n for n, _, _ in ck.saved_buffers(tr)]
    assert names == [f"world.{a}" for a in geo + ["features_sh"]] + [f"eng.g1_{a}" for a in geo + ["features_sh"]] + \
        [f"eng.g2_{a}" for a in geo + ["features_sh"]]
    # 16-bit non-SH moments: the qfpbo slots replace the fp32 pairs and sit before the SH state
    tr.quant, tr.non_sh_optim_bits = True, 16
    tr.nsq_packed = tr.nsq_bounds = none
    assert '"non_sh_optim_bits": 16' in ck.state_json(tr, 1)
    names = [n for n, _, _ in ck.saved_buffers(tr)]
    assert names == [f"world.{a}" for a in geo] + [f"eng.{a}_qfpbo.{x}" for a in geo for x in ("q", "qb")] + \
        ["eng.sh_quant.q", "eng.sh_quant.qb", "eng.world.sh_vq16.q", "eng.world.sh_vq16.qb"]
    # optimiser options: the radii of the scale-agnostic mean and the per-splat counters follow, in the slot table's order
    tr.steps = tr.radii = object()
    assert '"use_per_splat_bias_correction": 1' in ck.state_json(tr, 1)
    dens = SimpleNamespace(radii=object(), accum_buffer=None, count=900)
    assert [n for n, _, _ in ck.saved_buffers(tr, dens)][-3:] == ["eng.radii", "eng.accum_buffer", "eng.bias_correction_steps"]
    assert [n for n, _, _ in ck.saved_buffers(tr)][-2:] == ["eng.radii", "eng.bias_correction_steps"]
    assert '"cur_num_splats": 900' in ck.state_json(tr, 1, cur_num_splats=900)
