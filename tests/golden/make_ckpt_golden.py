"""Generates tests/golden/ckpt_state.tar and ckpt_headers.npz with the REFERENCE's checkpoint helpers
(src/core/CheckpointIO.h, reached through oracle/_ref/libssb_ref.so: oracle/ref_tool/ref_ckpt.cu).
Host data only, so it runs without a GPU:

    make -C oracle -f Makefile.ref REF=<reference checkout>
    python tests/golden/make_ckpt_golden.py
"""
import ctypes as C
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, HERE)
import ckpt_cases as K  # noqa: E402


def main():
    out_dir = sys.argv[1] if len(sys.argv) > 1 else HERE
    ref = C.CDLL(os.path.join(ROOT, "oracle", "_ref", "libssb_ref.so"))
    ref.ref_ckpt_npy_header.argtypes = [C.c_char_p, C.c_uint64, C.c_char_p, C.c_int]
    ref.ref_ckpt_tar_header.argtypes = [C.c_char_p, C.c_uint64, C.c_char_p]
    out = {}
    buf = C.create_string_buffer(1024)
    for tag, descr in enumerate(K.DESCR):
        for n in K.HEADER_NUMELS:
            ln = ref.ref_ckpt_npy_header(descr.encode(), n, buf, 1024)
            assert ln > 0
            out[f"npy_{tag}_{n}"] = np.frombuffer(buf.raw[:ln], dtype=np.uint8).copy()
    for i, name in enumerate(K.HEADER_NAMES):
        for size in K.HEADER_SIZES:
            assert ref.ref_ckpt_tar_header(name.encode(), size, buf) == 0
            out[f"tar_{i}_{size}"] = np.frombuffer(buf.raw[:512], dtype=np.uint8).copy()
    np.savez_compressed(os.path.join(out_dir, "ckpt_headers.npz"), **out)

    mem = K.members()
    n = len(mem)
    names = (C.c_char_p * n)(*[m[0].encode() for m in mem])
    ptrs = (C.c_void_p * n)(*[m[2].ctypes.data for m in mem])
    sizes = (C.c_uint64 * n)(*[m[2].nbytes for m in mem])
    tags = (C.c_uint8 * n)(*[m[1] for m in mem])
    path = os.path.join(out_dir, "ckpt_state.tar")
    ref.ref_ckpt_write.argtypes = [C.c_char_p, C.c_char_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]
    assert ref.ref_ckpt_write(path.encode(), K.STATE_JSON.encode(), n, names, ptrs, sizes, tags, 0) == 0
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
