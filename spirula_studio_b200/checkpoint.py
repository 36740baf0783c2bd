"""Full-resume checkpoints of a Trainer in the reference's wire format.

Mirrors engine_save_checkpoint / engine_load_checkpoint (src/engine/EngineCheckpoint.cpp:350-474):
`<dir>/splat.ply` is the inference artefact (ssb_ply_write) and `<dir>/state.tar` a ustar archive whose first member is state.json (the manifest built by
_build_state_json, src/engine/EngineCheckpoint.cpp:73-127) followed by one flat NPY array per live
buffer, named after the reference's pool slots (src/core/PoolSlots.h:88-125) and written in the slot
table's order:

    world.means .quats .scales .opacities .features_dc   float32, always
    world.features_sh                                    float32, only when SH values are not quantised
    eng.g1_<attr>, eng.g2_<attr>                         Adam moments; the features_sh pair only when the
                                                         SH optimiser state is not quantised; the other five
                                                         only when non_sh_optim_bits is 32
    eng.<attr>_qfpbo.q / .qb                             16-bit joint moments of the five non-SH arrays
    eng.sh_quant.q / .qb                                 8-bit joint SH optimiser state: packed bytes / float bounds
    eng.world.sh_vq8|16.q / .qb                          quantised SH values: packed bytes / float bounds
    eng.sh_quant_fpbo.*, eng.world.sh_vq8|16_fpbo.*      the same two with one bound per 256 splats: the layout of the reference's
                                                         fused backward + optimiser (Trainer fused_state_layout="reference";
                                                         state.json use_fused_proj_bwd_optim = 1)
    eng.radii, eng.accum_buffer                          with a Densifier: the view radii and the strategy's score
                                                         accumulator; state.json's cur_num_splats is then the number
                                                         of splats in use, and splat.ply holds those
    eng.bias_correction_steps                            int32 per-splat Adam step counters (OptimOptions)

The archive is produced by libssb_b200 (ssb_ckpt_*), which streams device buffers through pinned
staging memory.  With several ranks every rank holds the same parameters but only its own range of
optimiser state, so save() first completes the moments on rank 0 (one broadcast per owner of a range)
and rank 0 alone writes; load() is called on every rank and each reads the whole file.
"""
import ctypes as C
import os

import torch

from . import lib as L

DTYPE_U1, DTYPE_U2, DTYPE_U4, DTYPE_U8, DTYPE_I4, DTYPE_I8, DTYPE_F2, DTYPE_F4, DTYPE_F8, DTYPE_B1 = range(10)
_MODEL_NAMES = {0: "PINHOLE", 1: "FISHEYE", 2: "EQUISOLID", 3: "EQUIRECTANGULAR"}
_GEO = ("means", "quats", "scales", "opacities", "features_dc")


def state_json(trainer, step, full=True, cur_num_splats=None):
    """The manifest text, key for key and byte for byte as the reference formats it."""
    cfg = trainer.cfg
    cur = trainer.n if cur_num_splats is None else int(cur_num_splats)
    sh_optim_bits = 8 if trainer.quant else 32
    lines = [
        '  "format_version": 1',
        f'  "full_resume": {1 if full else 0}',
        '  "quant_codec": "joint_u_log_sqrt_g2_v1"',
        '  "quant_block_size": 256',
        '  "quant_eps": 1e-15',
        f'  "step": {int(step)}',
        '  "primitive": "3dgs"',
        f'  "cur_num_splats": {cur}',
        f'  "max_num_splats": {trainer.n}',
        f'  "num_sh": {L.NUM_SH}',
        '  "sh_degree": 3',
        '  "packed": 0',
        f'  "sh_optim_bits": {sh_optim_bits}',
        f'  "sh_value_bits": {cfg.sh_value_bits if trainer.quant else 32}',
        f'  "non_sh_optim_bits": {trainer.non_sh_optim_bits}',
        f'  "use_fused_proj_bwd_optim": {1 if getattr(trainer, "fused_state_layout", "shared") == "reference" else 0}',
        f'  "use_per_splat_bias_correction": {1 if getattr(trainer, "steps", None) is not None else 0}',
        f'  "camera": {{"num": {cfg.n_views}, "width": {cfg.width}, "height": {cfg.height}, '
        f'"model": "{_MODEL_NAMES.get(cfg.camera_model, "PINHOLE")}"}}',
        '  "bilagrid_rgb": {"enabled": 0}',
        '  "bilagrid_depth": {"enabled": 0}',
        '  "bilagrid_normal": {"enabled": 0}',
        '  "ppisp": {"enabled": 0}',
    ]
    return "{\n" + ",\n".join(lines) + "\n}\n"


def saved_buffers(trainer, densifier=None):
    """[(slot name, tensor, dtype tag)] of the trainer's live state, in the reference's slot order; with a Densifier also
    the strategy's resumable state (eng.radii, eng.accum_buffer)."""
    out = [(f"world.{a}", trainer.params[a], DTYPE_F4) for a in _GEO]
    if not trainer.quant:
        out.append(("world.features_sh", trainer.params["features_sh"], DTYPE_F4))
    nsq = trainer.non_sh_optim_bits == 16
    for g, mom in (("g1", trainer.m1), ("g2", trainer.m2)):
        if not nsq:
            out += [(f"eng.{g}_{a}", mom[a], DTYPE_F4) for a in _GEO]
        if not trainer.quant:
            out.append((f"eng.{g}_features_sh", mom["features_sh"], DTYPE_F4))
    if nsq:
        for a in _GEO:
            out += [(f"eng.{a}_qfpbo.q", trainer.nsq_packed[a], DTYPE_U1), (f"eng.{a}_qfpbo.qb", trainer.nsq_bounds[a], DTYPE_F4)]
    if trainer.quant:
        # the reference keeps the per-256-splats layout of its fused path under slots of its own (src/core/PoolSlots.h:114-120)
        fpbo = "_fpbo" if getattr(trainer, "fused_state_layout", "shared") == "reference" else ""
        vq = f"eng.world.sh_vq{trainer.cfg.sh_value_bits}{fpbo}"
        out += [(f"eng.sh_quant{fpbo}.q", trainer.sh_optim_packed, DTYPE_U1), (f"eng.sh_quant{fpbo}.qb", trainer.sh_optim_bounds, DTYPE_F4),
                (vq + ".q", trainer.sh_packed, DTYPE_U1), (vq + ".qb", trainer.sh_bounds, DTYPE_F4)]
    radii = densifier.radii if densifier is not None else getattr(trainer, "radii", None)
    if radii is not None:
        out.append(("eng.radii", radii, DTYPE_F4))
    if densifier is not None:
        out.append(("eng.accum_buffer", densifier.accum_buffer, DTYPE_F4))
    if getattr(trainer, "steps", None) is not None:
        out.append(("eng.bias_correction_steps", trainer.steps, DTYPE_I4))
    return out


def _owned_slices(trainer, first, count):
    """Views of the optimiser state that the owner of splats [first, first + count) has updated."""
    widths = dict(means=3, quats=4, scales=3, opacities=1, features_dc=3, features_sh=45)
    out = []
    for mom in (trainer.m1, trainer.m2):
        out += [mom[a][first * widths[a]: (first + count) * widths[a]] for a in widths if mom.get(a) is not None]
    if trainer.quant:
        c0, c1 = first * 45, (first + count) * 45          # ranges start on multiples of 512 splats: whole 256-cell blocks
        b0, b1 = c0 // 256, (c1 + 255) // 256
        out += [trainer.sh_optim_packed[c0 * 2: c1 * 2], trainer.sh_optim_bounds[b0 * 4: b1 * 4]]
    return out


def gather_optimizer_state(trainer):
    """Completes every rank's copy of the optimiser state: the owner of each range broadcasts its part."""
    if trainer.world_size == 1 or trainer.grad_sync == "nccl":
        return
    import torch.distributed as dist
    ranges = [None] * trainer.world_size
    dist.all_gather_object(ranges, (trainer.first, trainer.count), group=trainer.pg)
    for owner, (first, count) in enumerate(ranges):
        if count == 0:
            continue
        for piece in _owned_slices(trainer, first, count):
            dist.broadcast(piece, src=dist.get_global_rank(trainer.pg, owner) if trainer.pg is not None else owner, group=trainer.pg)


def export_ply(trainer, path, count=None):
    """Writes the trainer's splats (the first `count`: the ones in use) as a 3D Gaussian Splatting PLY (the reference's
    splat.ply: non-finite and low-opacity splats dropped, quantised SH dequantised); returns the number of vertices written."""
    kept = C.c_int64(-1)
    stream = C.c_void_p(torch.cuda.current_stream(trainer.device).cuda_stream)
    L.check(trainer.lib.ssb_ply_write(path.encode(), C.byref(trainer._p_struct), C.byref(trainer.shq) if trainer.shq else None,
                                      trainer.n if count is None else int(count), C.byref(kept), stream))
    return kept.value


def save_checkpoint(trainer, output_dir, step=None, full=True, densifier=None):
    """Writes <output_dir>/splat.ply and <output_dir>/state.tar, as engine_save_checkpoint does; returns the path of
    state.tar (on every rank; rank 0 writes)."""
    step = trainer.iteration if step is None else step
    path = os.path.join(output_dir, "state.tar")
    if full:
        gather_optimizer_state(trainer)
    if trainer.rank != 0:
        return path
    os.makedirs(output_dir, exist_ok=True)
    lib = trainer.lib
    torch.cuda.synchronize(trainer.device)
    count = None if densifier is None else densifier.count
    export_ply(trainer, os.path.join(output_dir, "splat.ply"), count)
    stream = C.c_void_p(torch.cuda.current_stream(trainer.device).cuda_stream)
    w = C.c_void_p()
    L.check(lib.ssb_ckpt_writer_open(path.encode(), C.byref(w)))
    try:
        text = state_json(trainer, step, full, count).encode()
        L.check(lib.ssb_ckpt_write_bytes(w, b"state.json", text, len(text)))
        for name, t, tag in (saved_buffers(trainer, densifier) if full else []):
            L.check(lib.ssb_ckpt_write_device(w, (name + ".npy").encode(), L.ptr(t), t.numel() * t.element_size(), tag, stream))
    finally:
        rc = lib.ssb_ckpt_writer_close(w)
    L.check(rc)
    return path


def _json_value(text, key, default=None):
    """Top-level value of our flat manifest (the reference's _json_find: first match of the quoted key)."""
    k = text.find(f'"{key}"')
    if k < 0:
        return default
    v = text[text.index(":", k) + 1:].lstrip()
    if v.startswith('"'):
        return v[1: v.index('"', 1)]
    end = 0
    while end < len(v) and v[end] not in ",\n}":
        end += 1
    return int(float(v[:end]))


def load_checkpoint(trainer, input_dir, densifier=None):
    """Restores a trainer (built for the same scene) from <input_dir>/state.tar; returns the saved step.

    As in the reference, every array member must name a live buffer of exactly its byte size; the
    capacity and the quantisation layout recorded in state.json must match the trainer's."""
    lib = trainer.lib
    path = os.path.join(input_dir, "state.tar")
    r = C.c_void_p()
    L.check(lib.ssb_ckpt_reader_open(path.encode(), C.byref(r)))
    try:
        size = C.c_uint64()
        rc = lib.ssb_ckpt_read_bytes(r, b"state.json", None, 0, C.byref(size))
        if rc != L.SSB_OK:
            raise RuntimeError(f"load_checkpoint: state.json missing in {path}")
        buf = C.create_string_buffer(size.value)
        L.check(lib.ssb_ckpt_read_bytes(r, b"state.json", buf, size.value, None))
        text = buf.raw.decode()
        step = _json_value(text, "step", 0)
        if _json_value(text, "max_num_splats", 0) != trainer.n:
            raise RuntimeError(f"load_checkpoint: max_num_splats mismatch (trainer {trainer.n} vs checkpoint "
                               f"{_json_value(text, 'max_num_splats', 0)})")
        want = (8 if trainer.quant else 32, trainer.cfg.sh_value_bits if trainer.quant else 32, trainer.non_sh_optim_bits,
                1 if getattr(trainer, "steps", None) is not None else 0, 1 if getattr(trainer, "fused_state_layout", "shared") == "reference" else 0)
        have = tuple(_json_value(text, k, d) for k, d in (("sh_optim_bits", 32), ("sh_value_bits", 32), ("non_sh_optim_bits", 32),
                                                          ("use_per_splat_bias_correction", 0), ("use_fused_proj_bwd_optim", 0)))
        if want != have:
            raise RuntimeError(f"load_checkpoint: optimiser-state layout {have} of the checkpoint is not the trainer's {want}")
        targets = {name: t for name, t, _ in saved_buffers(trainer, densifier)}
        if densifier is not None:
            densifier.count = _json_value(text, "cur_num_splats", trainer.n)
        stream = C.c_void_p(torch.cuda.current_stream(trainer.device).cuda_stream)
        name_buf = C.create_string_buffer(128)
        for i in range(lib.ssb_ckpt_member_count(r)):
            L.check(lib.ssb_ckpt_member_info(r, i, name_buf, 128, None))
            member = name_buf.value.decode()
            if not member.endswith(".npy"):
                continue
            t = targets.get(member[:-4])
            if t is None:
                raise RuntimeError(f"load_checkpoint: unknown slot '{member[:-4]}'")
            L.check(lib.ssb_ckpt_read_device(r, member.encode(), L.ptr(t), t.numel() * t.element_size(), stream))
    finally:
        lib.ssb_ckpt_reader_close(r)
    trainer.iteration = step
    torch.cuda.synchronize(trainer.device)
    if trainer.world_size > 1:            # nobody starts an iteration before every replica is restored
        import torch.distributed as dist
        dist.barrier(group=trainer.pg)
    return step
