"""CPU checks of the numpy restatement of the node-level bf16 operators against closed forms."""
import numpy as np

from oracle import oracle_ffi as orc


def test_unary_known_points():
    x = np.array([0.0, 1.0, -1.0, 4.0], dtype=np.float32)
    assert np.array_equal(orc.node_unary("relu", x), np.array([0, 1, 0, 4], dtype=np.float32))
    silu = orc.node_unary("silu", x)
    assert silu[0] == 0 and abs(silu[1] - 0.7310586) < 4e-3 and abs(silu[2] + 0.2689414) < 2e-3
    g_t, g_e = orc.node_unary("gelu", x), orc.node_unary("gelu_erf", x)
    assert abs(g_e[1] - 0.8413447) < 4e-3 and abs(g_t[1] - 0.8411920) < 4e-3
    assert np.abs(g_t - g_e).max() < 8e-3


def test_norm_properties():
    rng = np.random.default_rng(0)
    x = orc.bf16_round(rng.standard_normal((5, 256)).astype(np.float32) * 3 + 1)
    r = orc.node_norm(x, 1e-6, True)
    assert np.allclose((r.astype(np.float64) ** 2).mean(-1), 1.0, atol=1e-2)
    n = orc.node_norm(x, 1e-6, False)
    assert np.allclose(n.mean(-1), 0.0, atol=1e-2) and np.allclose(n.std(-1), 1.0, atol=1e-2)


def test_bin_scale_mul_mat():
    rng = np.random.default_rng(1)
    a = orc.bf16_round(rng.standard_normal((2, 3, 8)).astype(np.float32))
    b = orc.bf16_round(rng.standard_normal((8,)).astype(np.float32))
    assert np.array_equal(orc.node_bin("add", a, b), orc.bf16_round(a + b))
    assert np.array_equal(orc.node_scale(a, 2.0, 0.0), 2 * a)
    w = orc.bf16_round(rng.standard_normal((4, 8)).astype(np.float32))
    out = orc.node_mul_mat(w, a)
    assert out.shape == (2, 3, 4)
    assert np.allclose(out, a @ w.T, rtol=2e-2, atol=2e-2)
