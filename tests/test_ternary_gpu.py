"""GPU parity of the BitVLA ternary path, through the C ABI.

Bar: int32 accumulators and int8 quantised activations bit-exact against the CPU oracle;
bf16 outputs bit-equal to the oracle's IEEE epilogue; within 1 bf16 ulp of the reference's
own CUDA kernels (those divide with --use_fast_math)."""
import ctypes as C

import numpy as np
import pytest

from tests.gpu_util import bf16_bits, bits_to_bf16_tensor, reference_bitnet_lib, require_cuda, to_dev

pytestmark = pytest.mark.gpu

LM_SHAPES = [(2560, 2560, 1), (640, 2560, 1), (13824, 2560, 2), (2560, 6912, 1)]  # (N, K, ws_num)
# the vision tower's projections, which the reference's kernels also serve (src/kernels/bitvla/bitnet_kernels.cu:68-70,
# 85-87): hidden 1152, MLP 4304 (N not a multiple of 32: the last 256-column tile is cut after 208 columns), and the
# MLP width padded to 4352 on the K side
VIT_SHAPES = [(1152, 1152, 1), (4304, 1152, 1), (1152, 4352, 1)]


def make_case(rng, m, n, k, ws_num, raw_bytes=False):
    a = rng.integers(-127, 128, (m, k)).astype(np.int8)
    if raw_bytes:  # tests/bitvla_gemm_check.cu:84 feeds uniform bytes (code 0 -> -2 included)
        packed = rng.integers(0, 256, n * k // 4).astype(np.uint8)
    else:
        packed = None
    s = (40.0 + rng.integers(0, 100, m)).astype(np.float32)
    ws = (0.01 + 0.001 * rng.integers(0, 50, ws_num)).astype(np.float32)
    return a, packed, s, ws


def assert_bf16_close(got_bits, ref_bits):
    """The tensor-core epilogue evaluates acc / s * ws as acc * (ws / s): the float result may differ
    from the two-step form in the last bit, which survives the bf16 rounding only on near-ties.
    At most 1 bf16 ulp, on at most 0.1 % of the elements."""
    d = np.abs(got_bits.astype(np.int32) - ref_bits.astype(np.int32))
    assert d.max() <= 1, f"max bf16 ulp distance {d.max()}"
    assert (d != 0).mean() <= 1e-3, f"{(d != 0).mean():.2e} of the elements differ"


def run_gpu(api, a, packed, s, ws, n, path):
    import torch

    m = a.shape[0]
    acc = torch.full((m, n), -7, dtype=torch.int32, device="cuda")
    out = api.ternary_linear(to_dev(a), to_dev(packed), to_dev(s), to_dev(ws), n, acc_out=acc, path=path)
    assert api.device_status() == 0
    return acc.cpu().numpy(), bf16_bits(out)


@pytest.mark.parametrize("m", [1, 2, 3, 5, 8])
@pytest.mark.parametrize("shape", LM_SHAPES)
def test_gemv_bit_exact(oracle, m, shape):
    require_cuda()
    from vla_cpp_b200 import api

    n, k, ws_num = shape
    rng = np.random.default_rng(1000 + m + n + k)
    tern = rng.integers(-1, 2, (n, k)).astype(np.int8)
    packed = oracle.pack_ladder_int2(tern)
    a, _, s, ws = make_case(rng, m, n, k, ws_num)
    acc, out = run_gpu(api, a, packed, s, ws, n, path=1)
    ref_acc = oracle.gemm_i8_i32(a, tern)
    assert np.array_equal(acc, ref_acc)
    assert np.array_equal(out, oracle.ternary_epilogue(ref_acc, s, ws))


@pytest.mark.parametrize("path", [2, 3])  # 2: one CTA per tile, 3: CTA pairs (cta_group::2)
@pytest.mark.parametrize("m", [9, 17, 128, 300, 517])
@pytest.mark.parametrize("shape", [LM_SHAPES[0], LM_SHAPES[1]])
def test_gemm_tensor_core_bit_exact_full(oracle, m, shape, path):
    require_cuda()
    from vla_cpp_b200 import api

    n, k, ws_num = shape
    rng = np.random.default_rng(2000 + m + n)
    a, packed, s, ws = make_case(rng, m, n, k, ws_num, raw_bytes=True)
    acc, out = run_gpu(api, a, packed, s, ws, n, path=path)
    ref_acc = oracle.ternary_gemm_i32(a, packed, n)
    assert np.array_equal(acc, ref_acc)
    assert_bf16_close(out, oracle.ternary_epilogue(ref_acc, s, ws))


@pytest.mark.parametrize("m", [300, 4800])
@pytest.mark.parametrize("shape", LM_SHAPES)
def test_gemm_tensor_core_sampled_rows_at_full_size(oracle, m, shape):
    """BASELINE sizes (M = 300, 4800): every column of 48 sampled rows (first, last, tile edges)."""
    require_cuda()
    from vla_cpp_b200 import api

    n, k, ws_num = shape
    rng = np.random.default_rng(3000 + m + n + k)
    tern = rng.integers(-1, 2, (n, k)).astype(np.int8)
    packed = oracle.pack_ladder_int2(tern)
    a, _, s, ws = make_case(rng, m, n, k, ws_num)
    acc, out = run_gpu(api, a, packed, s, ws, n, path=0)
    rows = np.unique(np.concatenate([[0, 1, 127, 128, 129, m - 1, m - 2], rng.integers(0, m, 41)])).astype(np.int32)
    rows = rows[rows < m]
    ref_acc = oracle.gemm_i8_i32_rows(a, tern, rows)
    assert np.array_equal(acc[rows], ref_acc)
    assert_bf16_close(out[rows], oracle.ternary_epilogue(ref_acc, s[rows], ws))
    # linearity in A as a whole-matrix property: acc(A) + acc(-A) == 0
    acc_neg, _ = run_gpu(api, (-a).astype(np.int8), packed, s, ws, n, path=0)
    assert not np.any(acc + acc_neg)


@pytest.mark.parametrize("m", [1, 7, 256, 300, 768])
@pytest.mark.parametrize("shape", VIT_SHAPES)
def test_vision_tower_shapes_whole_matrix(oracle, m, shape):
    """Every accumulator and every bf16 output of the three vision-tower shapes (256 patches per view; 1 and 7 rows run
    the GEMV), against the CPU integer GEMM and, where it was built, the reference's own bitlinear_int8xint2_m."""
    torch = require_cuda()
    from vla_cpp_b200 import api

    n, k, ws_num = shape
    rng = np.random.default_rng(7000 + m + n + k)
    tern = rng.integers(-1, 2, (n, k)).astype(np.int8)
    packed = oracle.pack_ladder_int2(tern)
    a, _, s, ws = make_case(rng, m, n, k, ws_num)
    ref_acc = oracle.gemm_i8_i32(a, tern)
    ref_out = oracle.ternary_epilogue(ref_acc, s, ws)
    outs = {}
    for path in ([0] if m <= 8 else [0, 2, 3]):
        acc, out = run_gpu(api, a, packed, s, ws, n, path=path)
        assert np.array_equal(acc, ref_acc), path
        if m <= 8:
            assert np.array_equal(out, ref_out)
        else:
            assert_bf16_close(out, ref_out)
        outs[path] = out
    if m > 8:
        assert np.array_equal(outs[2], outs[3])
    ref = reference_bitnet_lib()
    if ref is not None and m > 1:
        ad, pd, sd, wd = to_dev(a), to_dev(packed), to_dev(s), to_dev(ws)
        theirs = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
        ref.bitlinear_int8xint2_m(C.c_void_p(ad.data_ptr()), C.c_void_p(pd.data_ptr()), C.c_void_p(theirs.data_ptr()),
                                  C.c_void_p(sd.data_ptr()), C.c_void_p(wd.data_ptr()), m, n, k, C.c_void_p(0))
        torch.cuda.synchronize()
        diff = np.abs(outs[0].astype(np.int32) - bf16_bits(theirs).astype(np.int32))
        assert diff.max() <= 1, f"max ulp distance {diff.max()}"
        assert (diff == 0).mean() > 0.95


def test_gemv_and_tensor_core_paths_agree(oracle):
    require_cuda()
    from vla_cpp_b200 import api

    n, k, ws_num = 2560, 2560, 1
    rng = np.random.default_rng(5)
    a, packed, s, ws = make_case(rng, 8, n, k, ws_num, raw_bytes=True)
    acc1, out1 = run_gpu(api, a, packed, s, ws, n, path=1)
    for path in (2, 3):
        acc2, out2 = run_gpu(api, a, packed, s, ws, n, path=path)
        assert np.array_equal(acc1, acc2)
        assert_bf16_close(out2, out1)


@pytest.mark.parametrize("m,n,k,ws_num", [(257, 1536, 384, 2), (1000, 3840, 2560, 6), (4800, 13824, 2560, 2)])
def test_pair_and_single_cta_kernels_bit_identical(m, n, k, ws_num):
    """The CTA-pair kernel and the one-CTA kernel run the same arithmetic: equal accumulators and equal
    bf16 bits on every element, at sizes where the oracle would take minutes."""
    require_cuda()
    from vla_cpp_b200 import api

    rng = np.random.default_rng(m + n)
    a, packed, s, ws = make_case(rng, m, n, k, ws_num, raw_bytes=True)
    acc2, out2 = run_gpu(api, a, packed, s, ws, n, path=2)
    acc3, out3 = run_gpu(api, a, packed, s, ws, n, path=3)
    assert np.array_equal(acc2, acc3)
    assert np.array_equal(out2, out3)


@pytest.mark.parametrize("m,k", [(1, 2560), (17, 2560), (300, 6912), (5, 1024), (3, 72)])
def test_act_quant_bit_exact(oracle, m, k):
    require_cuda()
    from vla_cpp_b200 import api

    rng = np.random.default_rng(m * 7 + k)
    x = oracle.bf16_round(rng.standard_normal((m, k)).astype(np.float32))
    if m > 2:
        x[1] = 0.0  # all-zero token: amax floor
        x[2, 0] = 300.0
    xd = bits_to_bf16_tensor(oracle.f32_to_bf16_bits(x))
    q, s = api.act_quant(xd)
    assert api.device_status() == 0
    rq, rs = oracle.act_quant(x)
    assert np.array_equal(s.cpu().numpy().view(np.uint32), rs.view(np.uint32))
    assert np.array_equal(q.cpu().numpy(), rq)


@pytest.mark.parametrize("m", [600, 256, 517])
@pytest.mark.parametrize("shape", LM_SHAPES)
def test_against_reference_cuda_kernels(oracle, m, shape):
    """Same seeded inputs as tests/bitvla_gemm_check.cu:81-88 style, through the reference's
    own bitlinear_int8xint2_m compiled from its sources: outputs within 1 bf16 ulp."""
    torch = require_cuda()
    from vla_cpp_b200 import api

    ref = reference_bitnet_lib()
    if ref is None:
        pytest.skip("oracle/_ref/libbitnet_ref.so not built")
    n, k, ws_num = shape
    rng = np.random.default_rng(1234 + n + m)
    a, packed, s, ws = make_case(rng, m, n, k, ws_num, raw_bytes=True)
    ad, pd, sd, wd = to_dev(a), to_dev(packed), to_dev(s), to_dev(ws)
    mine = api.ternary_linear(ad, pd, sd, wd, n)
    theirs = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
    ref.bitlinear_int8xint2_m(C.c_void_p(ad.data_ptr()), C.c_void_p(pd.data_ptr()), C.c_void_p(theirs.data_ptr()),
                              C.c_void_p(sd.data_ptr()), C.c_void_p(wd.data_ptr()), m, n, k, C.c_void_p(0))
    torch.cuda.synchronize()
    assert api.device_status() == 0
    x, y = bf16_bits(mine).astype(np.int32), bf16_bits(theirs).astype(np.int32)
    # bf16 bit patterns of the same sign are ordered like integers
    diff = np.abs(x - y)
    assert diff.max() <= 1, f"max ulp distance {diff.max()}"
    assert (diff == 0).mean() > 0.95


def test_reference_act_quant_agrees(oracle):
    torch = require_cuda()
    from vla_cpp_b200 import api

    ref = reference_bitnet_lib()
    if ref is None:
        pytest.skip("oracle/_ref/libbitnet_ref.so not built")
    rng = np.random.default_rng(77)
    x = torch.from_numpy(rng.standard_normal((300, 2560)).astype(np.float32)).cuda().to(torch.bfloat16)
    q, s = api.act_quant(x)
    rq = torch.empty_like(q)
    rs = torch.empty_like(s)
    ref.bitvla_act_quant_cuda(C.c_void_p(x.data_ptr()), C.c_void_p(rq.data_ptr()), C.c_void_p(rs.data_ptr()), 300,
                              2560, C.c_void_p(0))
    torch.cuda.synchronize()
    # the reference divides with --use_fast_math: scales may differ in the last bits,
    # quantised values by at most one step on rounding ties
    np.testing.assert_allclose(s.cpu().numpy(), rs.cpu().numpy(), rtol=1e-6)
    d = (q.cpu().numpy().astype(np.int32) - rq.cpu().numpy().astype(np.int32))
    assert np.abs(d).max() <= 1 and (d != 0).mean() < 1e-3


def test_drop_in_symbols_compute(oracle):
    """bitlinear_int8xint2_m / bitvla_act_quant_cuda by their reference names and signatures."""
    torch = require_cuda()
    from vla_cpp_b200 import api

    L = api.lib()
    n, k, m = 13824, 2560, 40
    rng = np.random.default_rng(9)
    tern = rng.integers(-1, 2, (n, k)).astype(np.int8)
    packed = oracle.pack_ladder_int2(tern)
    x = oracle.bf16_round(rng.standard_normal((m, k)).astype(np.float32))
    xd = bits_to_bf16_tensor(oracle.f32_to_bf16_bits(x))
    q = torch.empty((m, k), dtype=torch.int8, device="cuda")
    s = torch.empty((m,), dtype=torch.float32, device="cuda")
    out = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    ws = np.array([0.021, 0.034], np.float32)
    wd, pd = to_dev(ws), to_dev(packed)
    L.bitvla_act_quant_cuda(C.c_void_p(xd.data_ptr()), C.c_void_p(q.data_ptr()), C.c_void_p(s.data_ptr()), m, k,
                            C.c_void_p(0))
    L.bitlinear_int8xint2_m(C.c_void_p(q.data_ptr()), C.c_void_p(pd.data_ptr()), C.c_void_p(out.data_ptr()),
                            C.c_void_p(s.data_ptr()), C.c_void_p(wd.data_ptr()), m, n, k, C.c_void_p(0))
    assert api.device_status() == 0
    rq, rs = oracle.act_quant(x)
    ref = oracle.ternary_epilogue(oracle.gemm_i8_i32(rq, tern), rs, ws)
    assert_bf16_close(bf16_bits(out), ref)


@pytest.mark.parametrize("shape", LM_SHAPES)
def test_whole_matrix_at_4800_rows_against_oracle_and_reference(oracle, shape):
    """M = 4800 (16 sequences of 300 tokens), every element: all int32 accumulators against the CPU
    integer GEMM, all bf16 outputs against the oracle's epilogue and, where the reference's CUDA kernels
    were built, against bitlinear_int8xint2_m itself (<= 1 bf16 ulp: it divides with --use_fast_math)."""
    torch = require_cuda()
    from vla_cpp_b200 import api

    n, k, ws_num = shape
    m = 4800
    rng = np.random.default_rng(4800 + n + k)
    tern = rng.integers(-1, 2, (n, k)).astype(np.int8)
    packed = oracle.pack_ladder_int2(tern)
    a, _, s, ws = make_case(rng, m, n, k, ws_num)
    ad, pd, sd, wd = to_dev(a), to_dev(packed), to_dev(s), to_dev(ws)
    acc = torch.full((m, n), -7, dtype=torch.int32, device="cuda")
    mine = api.ternary_linear(ad, pd, sd, wd, n, acc_out=acc)
    assert api.device_status() == 0
    ref_acc = oracle.gemm_i8_i32(a, tern)
    assert np.array_equal(acc.cpu().numpy(), ref_acc)
    assert_bf16_close(bf16_bits(mine), oracle.ternary_epilogue(ref_acc, s, ws))
    ref = reference_bitnet_lib()
    if ref is not None:
        theirs = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
        ref.bitlinear_int8xint2_m(C.c_void_p(ad.data_ptr()), C.c_void_p(pd.data_ptr()), C.c_void_p(theirs.data_ptr()),
                                  C.c_void_p(sd.data_ptr()), C.c_void_p(wd.data_ptr()), m, n, k, C.c_void_p(0))
        torch.cuda.synchronize()
        diff = np.abs(bf16_bits(mine).astype(np.int32) - bf16_bits(theirs).astype(np.int32))
        assert diff.max() <= 1, f"max ulp distance {diff.max()}"
        assert (diff == 0).mean() > 0.95


@pytest.mark.parametrize("n,k,scale", [(640, 2560, 0.02), (2560, 6912, 1.0), (16, 128, 1e-7), (13824, 2560, 0.05)])
def test_ternarize_pack_on_device_matches_oracle(oracle, n, k, scale):
    """Float weights -> absmean scale, ternary values and ladder bytes on the GPU, bit for bit what the
    oracle's restatement of the reference's load-time code produces (and therefore what the reference's
    Python packer produces: tests/golden/ladder_pack.npz pins the oracle)."""
    require_cuda()
    from vla_cpp_b200 import api

    rng = np.random.default_rng(n + k)
    w = (rng.standard_normal((n, k)) * scale).astype(np.float32)
    w[0, :16] = [0.5 * scale * 0.7978845, -0.5 * scale * 0.7978845] * 8  # values near the rounding boundary
    tern, absmean = oracle.ternarize(w)
    want = oracle.pack_ladder_int2(tern)
    packed, sc = api.ternarize_pack(to_dev(w))
    assert api.device_status() == 0
    assert sc.cpu().numpy()[0] == np.float32(absmean)
    assert np.array_equal(packed.cpu().numpy(), want)
