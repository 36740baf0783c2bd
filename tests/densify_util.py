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
