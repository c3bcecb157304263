"""CPU checks of the oracle's RMSNorm / SwiGLU restatements (the checkers of tests/test_gpu_producers.py)."""
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden", "rms_norm_fused_add_seed24.npz")


def test_oracle_rms_norm_fused_add_matches_reference_golden(oracle):
    """The reference's own case (tests/test_rms_norm_fused_add.py:31-53) at its own tolerance."""
    g = np.load(GOLDEN)
    H, T = int(g["hidden"]), int(g["tokens"])
    np.random.seed(int(g["seed"]))
    x = np.asfortranarray(np.random.randn(H, T, 1, 1).astype(np.float32))
    r = np.asfortranarray(np.random.randn(H, T, 1, 1).astype(np.float32))
    w = np.random.randn(H).astype(np.float32)
    xt, rt = np.ascontiguousarray(x.reshape(H, T).T), np.ascontiguousarray(r.reshape(H, T).T)
    normed, res = oracle.rms_norm(xt, w, float(g["eps"]), rt)
    np.testing.assert_allclose(normed, g["normed"], atol=1e-5, rtol=1e-5)
    np.testing.assert_allclose(res, g["residual"], atol=1e-5, rtol=1e-5)
    assert np.array_equal(rt, np.ascontiguousarray(r.reshape(H, T).T)), "the caller's residual must not be modified"


def test_oracle_rms_norm_plain_and_large_rows(oracle):
    rng = np.random.default_rng(0)
    for T, H in ((1, 4096), (3, 11008), (2, 100)):
        x = rng.standard_normal((T, H)).astype(np.float32)
        w = rng.standard_normal(H).astype(np.float32)
        normed, res = oracle.rms_norm(x, w, 1e-6)
        assert res is None
        x64 = x.astype(np.float64)
        want = x64 / np.sqrt((x64 * x64).mean(axis=1, keepdims=True) + 1e-6) * w
        np.testing.assert_allclose(normed, want, rtol=2e-6, atol=1e-7)


def test_oracle_swiglu(oracle):
    rng = np.random.default_rng(1)
    g = (rng.standard_normal(5000) * 4).astype(np.float32)
    u = rng.standard_normal(5000).astype(np.float32)
    g[:4] = [0.0, 100.0, -100.0, -0.0]
    got = oracle.swiglu(g, u)
    g64 = g.astype(np.float64)
    want = g64 / (1 + np.exp(-g64)) * u
    np.testing.assert_allclose(got, want, rtol=1e-6, atol=1e-30)
    assert got[1] == np.float32(100.0) * u[1] and got[2] == 0.0
