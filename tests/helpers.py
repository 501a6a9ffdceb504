"""Shared input generators and comparison helpers for the parity tests."""
import numpy as np

MAX_ABS_TOL = 1e-2    # tolerance on attention outputs stated for this path
MEAN_ABS_TOL = 1e-3


def f16_round(a):
    return a.astype(np.float16).astype(np.float32)


def make_qkv(seed, n_head, n_kv, hd, n_rows, n_ctx=None, batch=1):
    """q [batch][n_head][hd] fp32 holding fp16-representable values, K,V [n_kv][n_ctx][hd] fp16 with the
    first n_rows rows i.i.d. N(0,1) and the rest zero."""
    rng = np.random.default_rng(seed)
    n_ctx = n_ctx or n_rows
    q = f16_round(rng.standard_normal((batch, n_head, hd), dtype=np.float32))
    K = np.zeros((n_kv, n_ctx, hd), np.float16)
    V = np.zeros((n_kv, n_ctx, hd), np.float16)
    K[:, :n_rows] = rng.standard_normal((n_kv, n_rows, hd), dtype=np.float32).astype(np.float16)
    V[:, :n_rows] = rng.standard_normal((n_kv, n_rows, hd), dtype=np.float32).astype(np.float16)
    return q, K, V


def assert_close(got, want, what=""):
    got = np.asarray(got, np.float32)
    want = np.asarray(want, np.float32)
    assert got.shape == want.shape, (got.shape, want.shape)
    assert np.isfinite(got).all(), "non-finite values in " + what
    err = np.abs(got - want)
    mx, mean = float(err.max()), float(err.mean())
    assert mx <= MAX_ABS_TOL and mean <= MEAN_ABS_TOL, "%s: max-abs %.3e (tol %.0e) mean-abs %.3e (tol %.0e)" % (
        what, mx, MAX_ABS_TOL, mean, MEAN_ABS_TOL)
    return mx, mean


def lse_merge(parts):
    """Reference merge of (m, l, O) partials in float64: parts = list of (m [H], l [H], O [H][D])."""
    m = np.stack([p[0] for p in parts]).astype(np.float64)
    l = np.stack([p[1] for p in parts]).astype(np.float64)
    O = np.stack([p[2] for p in parts]).astype(np.float64)
    M = m.max(axis=0)
    w = np.where(np.isneginf(m), 0.0, np.exp(m - M))
    L = (w * l).sum(axis=0)
    return ((w[..., None] * O).sum(axis=0) / L[..., None]).astype(np.float32)


def assert_f16_rows_match(got, want32, what="", max_mismatch=0.02):
    """got: fp16 rows from the device cache; want32: the oracle's fp32 rows.  Far into a context the
    rotation angle is thousands of radians, so device and host libm may differ by an ulp or two of fp32
    before the fp16 rounding: allow a small fraction of elements to land on the neighbouring fp16 value."""
    want = want32.astype(np.float16)
    g, w = got.astype(np.float32), want.astype(np.float32)
    neq = got.view(np.uint16) != want.view(np.uint16)
    assert neq.mean() <= max_mismatch, "%s: %.2f%% of fp16 elements differ" % (what, 100 * neq.mean())
    assert np.abs(g - w).max() <= 2.0 ** -9 * max(1.0, float(np.abs(w).max())), what
