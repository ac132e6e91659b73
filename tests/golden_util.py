"""Compact storage of reference outputs: small arrays whole, large ones as a
strided sample plus their sum and L2 norm (float64)."""
import numpy as np

MAX_KEEP = 4096


def pack(arr):
    a = np.asarray(arr)
    flat = a.reshape(-1)
    stride = max(1, -(-flat.size // MAX_KEEP))
    stats = np.array([flat.astype(np.float64).sum(), np.linalg.norm(flat.astype(np.float64)), flat.size, stride], np.float64)
    return flat[::stride].copy(), stats


def check(name, got, sample, stats, tol, exact=False):
    g = np.asarray(got).reshape(-1)
    assert g.size == int(stats[2]), "%s: size %d != %d" % (name, g.size, int(stats[2]))
    gs = g[::int(stats[3])]
    if exact:
        assert np.array_equal(gs, sample), "%s: not bit-exact against the reference" % name
        return 0.0
    den = np.linalg.norm(sample.astype(np.float64))
    err = np.linalg.norm(gs.astype(np.float64) - sample.astype(np.float64)) / (den if den > 0 else 1.0)
    assert err <= tol, "%s: relative L2 error %.3g vs reference > %.1g" % (name, err, tol)
    norm = np.linalg.norm(g.astype(np.float64))
    assert abs(norm - stats[1]) <= max(tol * 10 * stats[1], 1e-5), "%s: L2 norm %.8g vs reference %.8g" % (name, norm, stats[1])
    return err
