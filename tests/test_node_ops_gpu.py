"""Node-level bf16 operators (per-node hook surface, src/cuda/vla_cuda_bf16.cu:698-720) against the
numpy restatement.  Tolerances: add / mul are single float32 operations -> bit-exact; scale, unary and
norm go through libm-vs-device transcendentals or a fused multiply-add -> at most one bf16 ulp on a
small fraction of elements; mul_mat rel-L2 <= 2e-3 (float32 accumulation order + bf16 rounding)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def _orc():
    from oracle import oracle_ffi as orc

    return orc


def _bf(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(torch.bfloat16).cuda()


def _np(t):
    return t.float().cpu().numpy()


def _ulp_check(got, want, max_frac, abs_tol=1e-6):
    """At most one bf16 ulp apart (or abs_tol, where 1 + tanh / 1 + erf cancel near zero output)."""
    orc = _orc()
    gb = orc.f32_to_bf16_bits(got).astype(np.int32)
    wb = orc.f32_to_bf16_bits(want).astype(np.int32)
    # sign-magnitude -> monotone integer
    gm = np.where(gb & 0x8000, -(gb & 0x7FFF), gb & 0x7FFF)
    wm = np.where(wb & 0x8000, -(wb & 0x7FFF), wb & 0x7FFF)
    d = np.abs(gm - wm)
    bad = (d > 1) & (np.abs(got - want) > abs_tol)
    assert not bad.any(), f"{bad.sum()} elements off by more than one ulp, max distance {d[bad].max()}"
    diff = (d > 0) & (np.abs(got - want) > abs_tol)
    assert diff.mean() <= max_frac, f"{diff.mean():.4f} of elements differ"


@pytest.mark.parametrize("op", ["silu", "relu", "gelu", "gelu_erf"])
@pytest.mark.parametrize("n", [1, 7, 8, 4099, 300 * 2048])
def test_unary(op, n):
    import vla_cpp_b200 as vb

    orc = _orc()
    rng = np.random.default_rng(n)
    x = orc.bf16_round((rng.standard_normal(n) * 3).astype(np.float32))
    got = _np(vb.node_unary(op, _bf(x)))
    want = orc.node_unary(op, x)
    if op == "relu":
        assert np.array_equal(got, want)
    else:
        _ulp_check(got, want, 0.02)


@pytest.mark.parametrize("n", [5, 4096, 51 * 720 + 3])
def test_scale(n):
    import vla_cpp_b200 as vb

    orc = _orc()
    rng = np.random.default_rng(n)
    x = orc.bf16_round(rng.standard_normal(n).astype(np.float32))
    got = _np(vb.node_scale(_bf(x), 0.125, 0.0))
    assert np.array_equal(got, orc.node_scale(x, 0.125, 0.0))
    got = _np(vb.node_scale(_bf(x), 1.7, -0.3))
    _ulp_check(got, orc.node_scale(x, 1.7, -0.3), 0.01)


@pytest.mark.parametrize("op", ["add", "mul"])
@pytest.mark.parametrize("f32", [False, True])
@pytest.mark.parametrize("shape,bshape", [((51, 720), (51, 720)), ((4, 51, 720), (720,)), ((3, 7, 33), (7, 33))])
def test_bin(op, f32, shape, bshape):
    import vla_cpp_b200 as vb

    orc = _orc()
    rng = np.random.default_rng(len(shape) * 100 + len(bshape))
    a = orc.bf16_round(rng.standard_normal(shape).astype(np.float32))
    b = rng.standard_normal(bshape).astype(np.float32)
    if not f32:
        b = orc.bf16_round(b)
    bt = torch.from_numpy(b).cuda() if f32 else _bf(b)
    got = _np(vb.node_bin(op, _bf(a), bt))
    assert np.array_equal(got, orc.node_bin(op, a, b))


@pytest.mark.parametrize("rms", [True, False])
@pytest.mark.parametrize("rows,cols", [(1, 720), (51, 1024), (300, 2560), (17, 33)])
def test_norm(rms, rows, cols):
    import vla_cpp_b200 as vb

    orc = _orc()
    rng = np.random.default_rng(rows * cols)
    x = orc.bf16_round((rng.standard_normal((rows, cols)) * 2 + 0.5).astype(np.float32))
    got = _np(vb.node_norm(_bf(x), 1e-6, rms))
    _ulp_check(got, orc.node_norm(x, 1e-6, rms), 0.02)


@pytest.mark.parametrize("m,n,k,nb,wb", [(51, 2160, 720, 1, False), (1, 1024, 1024, 1, False),
                                         (300, 960, 2048, 1, False), (51, 64, 64, 4, True),
                                         (128, 256, 512, 3, False)])
@pytest.mark.parametrize("tiling", [0, 3])
def test_mul_mat(m, n, k, nb, wb, tiling):
    import vla_cpp_b200 as vb

    orc = _orc()
    rng = np.random.default_rng(m + n + k)
    x = orc.bf16_round(rng.standard_normal((nb, m, k) if nb > 1 else (m, k)).astype(np.float32))
    w = orc.bf16_round((rng.standard_normal((nb, n, k) if wb else (n, k)) / np.sqrt(k)).astype(np.float32))
    vb.set_gemm_tiling(tiling)
    try:
        got = _np(vb.node_mul_mat(_bf(w), _bf(x)))
    finally:
        vb.set_gemm_tiling(0)
    want = orc.node_mul_mat(w, x)
    rel = np.linalg.norm(got - want) / np.linalg.norm(want)
    assert rel <= 2e-3, rel


def test_bad_args():
    import vla_cpp_b200 as vb
    from vla_cpp_b200 import api

    x = torch.zeros(64, dtype=torch.bfloat16, device="cuda")
    L = vb.lib()
    import ctypes as C

    assert L.vlab200_node_unary_bf16(9, api._ptr(x), api._ptr(x), C.c_int64(64), None) != 0
    assert L.vlab200_node_bin_bf16(0, api._ptr(x), api._ptr(x), 0, api._ptr(x), C.c_int64(64), C.c_int64(5), None) != 0
    assert L.vlab200_node_norm_bf16(api._ptr(x), api._ptr(x), C.c_int64(1), C.c_int64(0), C.c_float(1e-6), 1, None) != 0
    assert L.vlab200_node_mul_mat_bf16(None, api._ptr(x), api._ptr(x), 8, 8, 8, 1, 0, None) != 0
