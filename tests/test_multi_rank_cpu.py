"""The multi-GPU iteration's host logic on two CPU ranks (gloo): views are
split into contiguous blocks, each rank back-propagates its own views, the
gradient buffers are summed with an all-reduce, and both ranks then apply the
same Adam update with grad_scale = 1 / total views -- which must equal the
single-process multi-view iteration (src/engine/EngineTrainStep.cpp:287-437)."""
import os
import sys

import numpy as np
import pytest

torch = pytest.importorskip("torch")
import torch.distributed as dist  # noqa: E402
import torch.multiprocessing as mp  # noqa: E402

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from bench import shard  # noqa: E402


def test_shard_covers_every_view_once():
    for total in (1, 2, 15, 16, 17, 64):
        for world in (1, 2, 3, 4, 8):
            seen = []
            for r in range(world):
                s, n = shard(total, world, r)
                seen += list(range(s, s + n))
            assert seen == list(range(total))
            sizes = [shard(total, world, r)[1] for r in range(world)]
            assert max(sizes) - min(sizes) <= 1


def _scene():
    from spirula_studio_b200 import scenes
    cfg = scenes.scaled(scenes.CONFIGS["plumbing_50k"], n_splats=1500, width=96, height=64, n_views=3)
    cfg.rig, cfg.rig_radius, cfg.log_scale_mu = "ring", 3.0, -2.8
    return cfg, scenes.make_splats(cfg), *scenes.make_cameras(cfg)


def _view_grads(cfg, sp, vm, K, views):
    from oracle import pyoracle as O
    from spirula_studio_b200 import scenes
    names = ("means", "quats", "scales", "opacities", "features_dc", "features_sh")
    tot = {k: np.zeros_like(sp[k]) for k in names}
    for v in views:
        ch = O.forward_chain(sp, vm[v:v + 1], K[v:v + 1], cfg.width, cfg.height)
        vr, _ = O.loss_l1_ssim(ch["render"]["rgb"], scenes.make_target(cfg, v).reshape(-1, 3), 1, cfg.height, cfg.width)
        gs = O.raster_bwd(ch["proj"], ch["offsets"], ch["sorted_vals"], 1, cfg.n_splats, cfg.width, cfg.height, ch["render"], vr)
        g = O.project_bwd(sp, vm[v:v + 1], K[v:v + 1], cfg.width, cfg.height, ch["proj"]["aabb"], gs)
        for k in names:
            tot[k] += g[k].reshape(tot[k].shape)
    return tot


def _flat(d):
    return np.concatenate([d[k].reshape(-1) for k in ("means", "quats", "scales", "opacities", "features_dc", "features_sh")])


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import pyoracle as O
    O.set_num_threads(2)
    cfg, sp, vm, K = _scene()
    s, n = shard(cfg.n_views, world, rank)
    g = _view_grads(cfg, sp, vm, K, range(s, s + n))
    flat = torch.from_numpy(_flat(g))
    dist.all_reduce(flat, op=dist.ReduceOp.SUM)
    # every rank applies the same update to its replica
    p = {k: v.copy() for k, v in sp.items()}
    off, gsum = 0, {}
    for k in ("means", "quats", "scales", "opacities", "features_dc", "features_sh"):
        gsum[k] = flat[off: off + p[k].size].numpy().reshape(p[k].shape).copy()
        off += p[k].size
    m1 = {k: np.zeros_like(v) for k, v in p.items()}
    m2 = {k: np.zeros_like(v) for k, v in p.items()}
    O.adam_geometry(p, gsum, m1, m2, 1, cfg.lrs, grad_scale=1.0 / cfg.n_views)
    np.save(os.path.join(out_dir, f"grads_{rank}.npy"), flat.numpy())
    np.save(os.path.join(out_dir, f"means_{rank}.npy"), p["means"])
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_iteration_equals_single_process(tmp_path):
    world, port = 2, 29000 + os.getpid() % 2000
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    cfg, sp, vm, K = _scene()
    ref = _flat(_view_grads(cfg, sp, vm, K, range(cfg.n_views)))
    g0, g1 = (np.load(tmp_path / f"grads_{r}.npy") for r in range(2))
    assert np.array_equal(g0, g1)                                   # both ranks hold the same sum
    assert np.allclose(g0, ref, rtol=1e-5, atol=1e-9)               # = the one-process sum (fp32 order only)
    m0, m1 = (np.load(tmp_path / f"means_{r}.npy") for r in range(2))
    assert np.array_equal(m0, m1)                                   # replicas stay identical
    assert np.abs(m0 - sp["means"]).max() > 0


# ---- what a rank sees when another rank is gone ---------------------------------------------------------------
# No GPU is involved: the failure is made on the host (a rank that raises before the exchange), the barrier of the
# multi-GPU step is a gloo all-reduce with a short timeout, and ssb_exchange_step must come back with SSB_ERR_PEER
# before it launches anything.

def test_exchange_step_returns_peer_error_when_the_barrier_fails():
    import ctypes as C
    from spirula_studio_b200 import lib as L
    lib = L.load()
    calls = []

    def failing_barrier(ctx, stream):
        calls.append(1)
        return 1

    cb = L.BARRIER_FN(failing_barrier)
    rep = L.SsbPeerReplicas()
    rep.world, rep.self = 2, 0
    s = L.SsbSplats()
    cfg = L.SsbAdamConfig(1e-3, 1e-3, 1e-3, 1e-3, 1e-3, 1e-3, 0.0, 1.0, 1, 0)
    st = lib.ssb_exchange_step(C.byref(rep), C.byref(s), C.byref(s), C.byref(s), C.byref(s), None, 0, 16, 16, C.byref(cfg), None, cb, None, None)
    assert st == L.SSB_ERR_PEER and calls == [1]                    # the first barrier failed: nothing else was attempted
    assert b"did not arrive" in lib.ssb_last_error_string()
    assert lib.ssb_exchange_step(C.byref(rep), C.byref(s), C.byref(s), C.byref(s), C.byref(s), None, 0, 16, 16, C.byref(cfg), None,
                                 L.BARRIER_FN(), None, None) == L.SSB_ERR_INVALID_ARGUMENT      # no barrier given


def _failing_worker(rank, world, port, out_dir):
    import ctypes as C
    import datetime
    import time
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
    from spirula_studio_b200 import lib as L
    lib = L.load()
    token = torch.zeros(1)
    dist.all_reduce(token)                       # both ranks are up
    if rank == 1:
        # this rank fails between two iterations, with nothing of its own in flight, and leaves
        with open(os.path.join(out_dir, "rank1.txt"), "w") as f:
            f.write("raised before the exchange")
        os._exit(0)

    def barrier(ctx, stream):
        try:
            dist.all_reduce(token)
            return 0
        except Exception:
            return 1

    cb = L.BARRIER_FN(barrier)
    rep = L.SsbPeerReplicas()
    rep.world, rep.self = 2, 0
    s = L.SsbSplats()
    cfg = L.SsbAdamConfig(1e-3, 1e-3, 1e-3, 1e-3, 1e-3, 1e-3, 0.0, 1.0, 1, 0)
    t0 = time.time()
    st = lib.ssb_exchange_step(C.byref(rep), C.byref(s), C.byref(s), C.byref(s), C.byref(s), None, 0, 16, 16, C.byref(cfg), None, cb, None, None)
    with open(os.path.join(out_dir, "rank0.txt"), "w") as f:
        f.write(f"{st} {time.time() - t0:.2f}")
    os._exit(0)                                  # the process group cannot be torn down cleanly without its peer


def test_a_rank_that_left_is_reported_within_the_timeout(tmp_path):
    world, port = 2, 31000 + os.getpid() % 2000
    mp.spawn(_failing_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    from spirula_studio_b200 import lib as L
    status, seconds = (tmp_path / "rank0.txt").read_text().split()
    assert int(status) == L.SSB_ERR_PEER
    assert float(seconds) < 30.0                 # the process-group timeout is 3 s; the step never waits for ever
    assert (tmp_path / "rank1.txt").exists()


# ---- checkpoint of a sharded optimiser state -------------------------------------------------------------------
# Each rank has updated only its own range of the Adam moments; before rank 0 writes state.tar the owners
# broadcast their ranges.  Run on CPU tensors over gloo with a stand-in for the trainer.
def _gather_worker(rank, world, port, out_dir):
    from types import SimpleNamespace
    from spirula_studio_b200 import checkpoint as ck
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    n, per = 1300, 1024                                   # ranges of 512-splat multiples: [0, 1024) and [1024, 1300)
    first = min(n, rank * per)
    count = min(n, first + per) - first
    widths = dict(means=3, quats=4, scales=3, opacities=1, features_dc=3)

    def moments(tag):
        out = {}
        for i, (a, w) in enumerate(widths.items()):
            t = torch.zeros(n * w)
            t[first * w: (first + count) * w] = torch.arange(first * w, (first + count) * w, dtype=torch.float32) + 1000 * i + tag
            out[a] = t
        out["features_sh"] = None
        return out

    cells, blocks = n * 45, (n * 45 + 255) // 256
    packed = torch.zeros(cells * 2, dtype=torch.uint8)
    packed[first * 90: (first + count) * 90] = (torch.arange(first * 90, (first + count) * 90) % 251).to(torch.uint8) + 1
    bounds = torch.zeros(blocks * 4)
    b0, b1 = first * 45 // 256, ((first + count) * 45 + 255) // 256
    bounds[b0 * 4: b1 * 4] = torch.arange(b0 * 4, b1 * 4, dtype=torch.float32) + 0.5
    tr = SimpleNamespace(world_size=world, rank=rank, pg=None, grad_sync="peer", first=first, count=count, quant=True,
                         m1=moments(0.25), m2=moments(0.75), sh_optim_packed=packed, sh_optim_bounds=bounds)
    ck.gather_optimizer_state(tr)
    torch.save(dict(m1=tr.m1, m2=tr.m2, packed=packed, bounds=bounds), os.path.join(out_dir, f"gathered_{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_sharded_optimizer_state_is_completed_before_a_save(tmp_path):
    world, port = 2, 31000 + os.getpid() % 2000
    mp.spawn(_gather_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    a, b = (torch.load(tmp_path / f"gathered_{r}.pt") for r in range(2))
    n = 1300
    for i, (k, w) in enumerate(dict(means=3, quats=4, scales=3, opacities=1, features_dc=3).items()):
        for mom, tag in (("m1", 0.25), ("m2", 0.75)):
            want = torch.arange(n * w, dtype=torch.float32) + 1000 * i + tag
            assert torch.equal(a[mom][k], want) and torch.equal(b[mom][k], want), (mom, k)
    want_p = (torch.arange(n * 90) % 251).to(torch.uint8) + 1
    assert torch.equal(a["packed"], want_p) and torch.equal(b["packed"], want_p)
    want_b = torch.arange(((n * 45 + 255) // 256) * 4, dtype=torch.float32) + 0.5
    assert torch.equal(a["bounds"], want_b) and torch.equal(b["bounds"], want_b)
