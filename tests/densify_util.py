"""Shared by the CPU (oracle) and GPU (library) densification tests: the runs of the fixture and the checks on the noise."""
import numpy as np

INF = float("inf")


def score_run_args(kw):
    """Keyword arguments of a DENSIFY_SCORE_RUNS entry -> the full parameter set of the score update."""
    return dict(max_screen_size=kw.get("max_screen_size", INF), clip_hardness=kw.get("clip_hardness", INF), max_world_size=kw.get("max_world_size", INF),
                accum_mode=kw.get("accum_mode", 1), score_mode=kw.get("score_mode", 0), blend_w=kw.get("blend_w", 0.0),
                score_power=kw.get("score_power", 1.0), clip_quantile=kw.get("clip_quantile", 1.0), final_power=kw.get("final_power", 1.0),
                use_accum=kw.get("accum", True), use_weights=kw.get("weights", True), use_world=kw.get("world", False), want_sample=kw.get("sample", False))


def close_frac(a, b, atol, rtol):
    return float((np.abs(a - b) > atol + rtol * np.abs(b)).mean())


def check_score_run(name, got, gold):
    """got: dict with log_scales, accum_weight, accum_buffer, sample_score (None where not produced)."""
    for key, atol, rtol in (("log_scales", 2e-6, 1e-6), ("accum_weight", 1e-7, 1e-6), ("accum_buffer", 1e-7, 2e-5), ("sample_score", 1e-7, 5e-5)):
        g = gold.get(f"{name}_{key}")
        if g is None:
            continue
        assert got[key] is not None, (name, key)
        assert close_frac(got[key].reshape(g.shape), g, atol, rtol) <= 1e-3, (name, key)


def shaping(inp, scaler, revised):
    """Per-splat matrix A with displacement = A z (z unit normal), from the noise formulas in float64."""
    l = inp["log_scales"].astype(np.float64)
    q = inp["quats"].astype(np.float64)
    q = q / np.linalg.norm(q, axis=1, keepdims=True)
    w, x, y, z = q.T
    R = np.stack([np.stack([1 - 2 * (y * y + z * z), 2 * (x * y - w * z), 2 * (x * z + w * y)], 1),
                  np.stack([2 * (x * y + w * z), 1 - 2 * (x * x + z * z), 2 * (y * z - w * x)], 1),
                  np.stack([2 * (x * z - w * y), 2 * (y * z + w * x), 1 - 2 * (x * x + y * y)], 1)], 1)
    opac = 1.0 / (1.0 + np.exp(-inp["logit_opacs"].astype(np.float64)))
    if revised:
        s = np.exp(l)
        amp = np.minimum(0.05 * scaler * np.sqrt(2 * np.log(np.maximum(255 * opac, 1.0))) * (1 - opac) ** 150, 1.0)
        amp = np.where(inp["radii"] > 0, amp, 0.0)
    else:
        s = np.exp(2 * l)
        amp = scaler / (1.0 + np.exp(-100.0 * ((1 - opac) - 0.995)))
    A = np.einsum("nij,nj,nkj->nik", R, s, R) * amp[:, None, None]
    return A, amp


def check_noise(inp, moved, scaler, revised, reference_moved=None):
    """The displacement is A z with z a unit normal draw per splat: whiten it and test the first two moments; unseen splats
    (revised) do not move; where given, the reference's displacement passes the same test and has the same scale."""
    A, amp = shaping(inp, scaler, revised)
    d = moved.astype(np.float64) - inp["means"].astype(np.float64)
    still = amp == 0.0
    assert np.all(d[still] == 0.0)
    # whiten only where the smallest axis of A is well above the float32 rounding of the mean it was added to
    smallest = np.linalg.svd(A, compute_uv=False)[:, -1]
    live = smallest > 1e-3 * np.maximum(np.abs(inp["means"]).max(axis=1), np.abs(moved).max(axis=1))
    assert live.sum() > 200, live.sum()
    z = np.linalg.solve(A[live], d[live][..., None])[..., 0]
    n = z.shape[0]
    assert np.all(np.abs(z.mean(0)) < 5.0 / np.sqrt(n)), z.mean(0)
    assert np.all(np.abs(z.var(0) - 1.0) < 0.15), z.var(0)
    assert abs(np.corrcoef(z.T)[0, 1]) < 0.15 and abs(np.corrcoef(z.T)[0, 2]) < 0.15
    if reference_moved is not None:
        dr = reference_moved.astype(np.float64) - inp["means"].astype(np.float64)
        assert np.all(dr[still] == 0.0)
        zr = np.linalg.solve(A[live], dr[live][..., None])[..., 0]
        assert np.all(np.abs(zr.mean(0)) < 5.0 / np.sqrt(n)) and np.all(np.abs(zr.var(0) - 1.0) < 0.15)
        ratio = np.median(np.linalg.norm(d[live], axis=1)) / np.median(np.linalg.norm(dr[live], axis=1))
        assert 0.85 < ratio < 1.15, ratio


# ---- relocation / growth -----------------------------------------------------------------------------------------------
SPLIT_ATTRS = ("means", "quats", "scales", "opacities", "features_dc", "features_sh")
WIDTH = dict(means=3, quats=4, scales=3, opacities=1, features_dc=3, features_sh=45)


def dead_mask(st, cur_n, min_opacity):
    """The dead splats among the first cur_n, by the reference's rule in float64 (borderline opacities do not occur in the fixtures)."""
    o = st["opacities"][:cur_n].astype(np.float64)
    m, q, s, c = (st[k][:cur_n].astype(np.float64) for k in ("means", "quats", "scales", "features_dc"))
    with np.errstate(all="ignore"):
        low = 1.0 / (1.0 + np.exp(-o)) <= min_opacity
        fin = np.isfinite((m * m).sum(1) / (q * q).sum(1) + (s * c).sum(1) * o)
    return low | ~fin


def check_split_state(before, after, ref_after, cur_n, first_new, n_new, dead, quant):
    """`after` (ours) and `ref_after` (the reference's) come from the same `before`.  new slots: `dead` indices (relocation) or
    first_new .. first_new + n_new - 1 (growth).  The two draws agree except near the cut of the sampling order (the keys use
    different logarithms), and the reference fills dead slots in an order of its own, so slots are matched through the rotation
    they inherit from their source, which no other splat shares."""
    slots = np.flatnonzero(dead) if dead is not None else np.arange(first_new, first_new + n_new)
    assert slots.size > 0
    def sources(state):
        # a source is a splat outside the new slots whose scale or opacity changed
        cand = np.setdiff1d(np.arange(cur_n), slots)
        changed = cand[np.any(state["scales"][cand] != before["scales"][cand], axis=1)]
        return changed
    ours_src, ref_src = sources(after), sources(ref_after)
    assert ours_src.size == slots.size and ref_src.size == slots.size
    common = np.intersect1d(ours_src, ref_src)
    assert common.size >= 0.95 * slots.size, (common.size, slots.size)
    # sources drawn by both: identical treatment
    for k in ("means", "scales", "opacities"):
        a, b = after[k][common], ref_after[k][common]
        assert np.allclose(a, b, rtol=2e-5, atol=2e-6), k
    # every new slot of ours: find its source through the rotation, check the split
    key = {}
    for s in range(cur_n):
        key.setdefault(tuple(before["quats"][s]), []).append(s)

    def source_of(state, d):
        # splats that were split before share their rotation with their twin: take the one whose split this slot continues
        cands = [s for s in key[tuple(state["quats"][d])]
                 if s != d and np.array_equal(state["scales"][s], state["scales"][d]) and
                 np.allclose(0.5 * (state["means"][d].astype(np.float64) + state["means"][s]), before["means"][s], rtol=1e-5, atol=1e-5)]
        assert len(cands) == 1, (d, cands)
        return cands[0]

    for state in (after, ref_after):
        seen = set()
        for d in slots:
            s = source_of(state, d)
            assert s not in seen and not (dead is not None and dead[s])
            seen.add(s)
            assert np.allclose(state["scales"][d], state["scales"][s]) and state["opacities"][d] == state["opacities"][s]
            mid = 0.5 * (state["means"][d].astype(np.float64) + state["means"][s])
            assert np.allclose(mid, before["means"][s], rtol=1e-5, atol=1e-5)
            assert np.array_equal(state["features_dc"][d], before["features_dc"][s])
            assert np.array_equal(state["accum"][d], before["accum"][s]) and state["steps"][d] == 0
            for a in SPLIT_ATTRS:
                if state.get("m1_" + a) is not None:
                    assert not np.any(state["m1_" + a][d]) and not np.any(state["m2_" + a][d]), a
            if not quant:
                assert np.array_equal(state["features_sh"][d], before["features_sh"][s])
            else:
                # values: the source's, decoded with its bounds, clipped to the slot's blocks and re-encoded (within a quantum);
                # state: the codes nearest to (0, 0) under the slot's bounds
                vb = before["sh_value_bounds"].reshape(-1, 2).astype(np.float64)
                cs, cd = 45 * s + np.arange(45), 45 * d + np.arange(45)
                codes = lambda st_, c: st_["sh_value_packed"].view(np.uint16)[c].astype(np.float64)
                lo_s, hi_s, lo_d, hi_d = vb[cs >> 8, 0], vb[cs >> 8, 1], vb[cd >> 8, 0], vb[cd >> 8, 1]
                v_src = lo_s + (hi_s - lo_s) * codes(before, cs) / 65535.0
                v_dst = lo_d + (hi_d - lo_d) * codes(state, cd) / 65535.0
                quantum = np.maximum(hi_d - lo_d, 1e-30) / 65535.0
                assert np.all(np.abs(v_dst - np.clip(v_src, lo_d, hi_d)) <= 1.01 * quantum + 1e-7)
                ob = before["sh_optim_bounds"].reshape(-1, 4).astype(np.float64)[cd >> 8]
                zero = lambda lo, hi: np.clip(np.round(255.0 * (0.0 - lo) / np.maximum(hi - lo, 1e-30)), 0, 255)
                got = state["sh_optim_packed"].reshape(-1, 2)[cd].astype(np.float64)
                assert np.abs(got[:, 0] - zero(ob[:, 0], ob[:, 1])).max() <= 1 and np.abs(got[:, 1] - zero(ob[:, 2], ob[:, 3])).max() <= 1
        assert seen == set(sources(state).tolist())
    # slots both sides fill from the same source hold the same bytes (quantised copies and zero codes included)
    ours_of = {source_of(after, d): d for d in slots}
    ref_of = {source_of(ref_after, d): d for d in slots}
    same = 0
    for s in common:
        do, dr = ours_of[s], ref_of[s]
        if quant and (45 * do // 256 != 45 * dr // 256 or (45 * do + 44) // 256 != (45 * dr + 44) // 256):
            continue                                     # other quantisation blocks, other bounds: the codes legitimately differ
        same += 1
        if quant:
            a = after["sh_value_packed"].view(np.uint16)[45 * do: 45 * do + 45].astype(np.int64)
            b = ref_after["sh_value_packed"].view(np.uint16)[45 * dr: 45 * dr + 45].astype(np.int64)
            assert np.abs(a - b).max() <= 1
            assert np.array_equal(after["sh_optim_packed"][90 * do: 90 * do + 90], ref_after["sh_optim_packed"][90 * dr: 90 * dr + 90])
    # nothing else moved
    untouched = np.setdiff1d(np.arange(before["means"].shape[0]), np.concatenate([slots, ours_src]))
    for k in ("means", "quats", "scales", "opacities", "features_dc", "accum", "steps"):
        assert np.array_equal(after[k][untouched], before[k][untouched], equal_nan=True), k
