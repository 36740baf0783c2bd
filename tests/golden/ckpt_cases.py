"""Inputs of the checkpoint-container fixture (shared by the generator and the tests)."""
import numpy as np

# NpyScalar tags of the reference (src/core/Tensor.h:26): u1 u2 u4 u8 i4 i8 f2 f4 f8 b1
DESCR = ("|u1", "<u2", "<u4", "<u8", "<i4", "<i8", "<f2", "<f4", "<f8", "|b1")
NP_DTYPES = (np.uint8, np.uint16, np.uint32, np.uint64, np.int32, np.int64, np.float16, np.float32, np.float64, np.bool_)

STATE_JSON = '{\n  "format_version": 1,\n  "step": 1234,\n  "max_num_splats": 77\n}\n'

# element counts chosen so that the dict text crosses a 64-byte boundary between neighbours and the
# members end both on and off a 512-byte boundary
HEADER_NUMELS = (0, 1, 9, 10, 99, 100, 12345, 999999, 1000000, 45 * 10_000_000, 2**31, 2**40 + 7)
# member sizes around the switch from an octal to a base-256 size field (8 GiB)
HEADER_SIZES = (0, 1, 511, 512, 513, 0o77777777777 - 1, 0o77777777777, 0o77777777777 + 1, 2**40 + 12345)
HEADER_NAMES = ("state.json", "world.means.npy", "eng.world.sh_vq16.qb.npy", "x" * 99)


def members(seed=7):
    """[(slot name, tag, array)]: one array per element type, ragged sizes."""
    rng = np.random.default_rng(seed)
    out = []
    sizes = (3 * 77, 384, 45 * 77 * 2, 5, 77, 2, 33, 4 * 77, 3, 448)
    names = ("world.means", "eng.g1_quats", "eng.sh_quant.q", "eng.accum_buffer", "eng.radii", "eng.bias_correction_steps",
             "half.values", "eng.sh_quant.qb", "double.values", "flags")
    order = (7, 7, 0, 3, 4, 5, 6, 7, 8, 9)          # tags, in the order the members are written
    for name, tag, n in zip(names, order, sizes):
        dt = NP_DTYPES[tag]
        if np.issubdtype(dt, np.floating):
            a = rng.standard_normal(n).astype(dt)
        elif dt is np.bool_:
            a = rng.integers(0, 2, n).astype(dt)
        else:
            a = rng.integers(0, np.iinfo(dt).max, n, dtype=dt, endpoint=True)
        out.append((name, tag, a))
    return out
