"""The oracle's restatement of the operations either side of the projections (reference.rs:59-80, 447-455, 466-490)
against an independent float64 computation."""
import numpy as np

from oracle import oracle as O


def test_sigmoid_gate_and_norm_tail_against_float64():
    rng = np.random.default_rng(3)
    x, g = rng.standard_normal((4, 512)).astype(np.float32), (4.0 * rng.standard_normal((4, 512))).astype(np.float32)
    want = x.astype(np.float64) / (1.0 + np.exp(-g.astype(np.float64)))
    assert np.allclose(O.sigmoid_gate(x, g), want, rtol=2e-6, atol=1e-7)
    hidden, src = rng.standard_normal((3, 640)).astype(np.float32), (0.05 * rng.standard_normal((3, 640))).astype(np.float32)
    w1, w2 = (1 + 0.1 * rng.standard_normal(640)).astype(np.float32), (1 + 0.1 * rng.standard_normal(640)).astype(np.float32)
    h, out = O.norm_residual_norm(hidden, src, w1, 1e-8, w2, 1e-5)
    s64 = src.astype(np.float64)
    h64 = hidden + s64 / np.sqrt((s64 ** 2).mean(-1, keepdims=True) + 1e-8) * w1
    o64 = h64 / np.sqrt((h64 ** 2).mean(-1, keepdims=True) + 1e-5) * w2
    assert np.allclose(h, h64, rtol=3e-6, atol=1e-6) and np.allclose(out, o64, rtol=3e-6, atol=1e-6)
    h_only, none = O.norm_residual_norm(hidden, src, w1, 1e-8)
    assert none is None and np.array_equal(h_only, h)
