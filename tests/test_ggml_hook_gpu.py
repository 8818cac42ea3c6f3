"""The ggml CUDA extension hook (vla_cuda_bf16_forward / vla_cuda_bf16_fused_binbcast) built from
vla_cpp_b200/csrc/ggml_hook_adapter.cpp and driven the way the patched ggml-cuda would drive it: one graph node
at a time, everything read from the tensor's public fields (src/cuda/vla_cuda_bf16.cu:686-720 is the reference's
implementation of the same two symbols).  llama.cpp's ggml.h is not available here, so the adapter is compiled
against tests/c/ggml_stub/ggml.h, which declares the same public names; the tensors below are instances of that
stand-in struct pointing at device memory.

Bars: add / mul / relu bit-exact against the oracle's float-math-one-rounding restatement, silu / gelu / scale /
norm within 1 bf16 ulp, mul_mat rel-L2 <= 2e-3; nodes the hook cannot take are declined (return false)."""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest

from tests.gpu_util import ROOT, bf16_bits, bits_to_bf16_tensor, rel_l2, require_cuda, to_dev

pytestmark = pytest.mark.gpu

F32, BF16 = 0, 30
OP = dict(ADD=1, MUL=2, SCALE=3, NORM=4, RMS_NORM=5, MUL_MAT=6, UNARY=7, SOFT_MAX=8)
UNARY = dict(silu=1, relu=2, gelu=3, gelu_erf=4, tanh=5)


class Tensor(C.Structure):
    pass


Tensor._fields_ = [("type", C.c_int), ("ne", C.c_int64 * 4), ("nb", C.c_size_t * 4), ("op", C.c_int),
                   ("op_params", C.c_int32 * 16), ("src", C.POINTER(Tensor) * 10), ("data", C.c_void_p)]


@pytest.fixture(scope="module")
def hook(tmp_path_factory):
    require_cuda()
    out = str(tmp_path_factory.mktemp("hook") / "libvla_ggml_hook.so")
    libdir = os.path.join(ROOT, "vla_cpp_b200")
    subprocess.run(["g++", "-std=c++17", "-Wall", "-Werror", "-fPIC", "-shared", "-DVLA_HOOK_NO_GGML_GLOBALS",
                    "-I", os.path.join(ROOT, "tests", "c", "ggml_stub"), "-I", os.path.join(ROOT, "include"),
                    os.path.join(libdir, "csrc", "ggml_hook_adapter.cpp"), "-o", out, "-L", libdir, "-lvla_b200",
                    "-Wl,-rpath," + libdir], check=True, capture_output=True, text=True)
    lib = C.CDLL(out)
    lib.vla_cuda_bf16_forward.restype = C.c_bool
    lib.vla_cuda_bf16_forward.argtypes = [C.POINTER(Tensor), C.c_void_p]
    lib.vla_cuda_bf16_fused_binbcast.restype = C.c_bool
    lib.vla_cuda_bf16_fused_binbcast.argtypes = [C.POINTER(Tensor), C.c_int, C.c_void_p]
    return lib


def tensor(t, ne=None, nb=None):
    """A stand-in ggml_tensor over a torch cuda tensor; ne fastest-first (ggml order), nb in bytes."""
    import torch

    g = Tensor()
    g.type = F32 if t.dtype == torch.float32 else BF16
    es = t.element_size()
    shape = list(t.shape)[::-1] + [1] * (4 - t.dim()) if ne is None else list(ne)
    strides = ([s * es for s in t.stride()][::-1] + [0] * (4 - t.dim())) if nb is None else list(nb)
    for i in range(4):
        g.ne[i] = shape[i]
        if nb is None and i >= t.dim():
            strides[i] = strides[i - 1] * shape[i - 1] if i else es
        g.nb[i] = strides[i]
    g.data = t.data_ptr()
    return g


def node(op, dst, *srcs, params=()):
    dst.op = op
    for i, s in enumerate(srcs):
        dst.src[i] = C.pointer(s)
    for i, p in enumerate(params):
        dst.op_params[i] = p
    return dst


def f32_bits(x):
    return int(np.float32(x).view(np.int32))


def bf(oracle, a):
    return bits_to_bf16_tensor(oracle.f32_to_bf16_bits(a))


def back(oracle, t):
    return oracle.bf16_bits_to_f32(bf16_bits(t))


def stream():
    import torch

    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def test_add_with_a_float_bias_row_and_mul_with_a_per_row_scalar(oracle, hook):
    import torch

    rng = np.random.default_rng(1)
    x = oracle.bf16_round(rng.standard_normal((3, 37, 200)).astype(np.float32))
    bias = rng.standard_normal(200).astype(np.float32)
    xd, out = bf(oracle, x), torch.empty((3, 37, 200), dtype=torch.bfloat16, device="cuda")
    n = node(OP["ADD"], tensor(out), tensor(xd), tensor(to_dev(bias)))
    assert hook.vla_cuda_bf16_forward(C.byref(n), stream())
    torch.cuda.synchronize()
    assert np.array_equal(back(oracle, out), oracle.bf16_round(x + bias))
    # src1 = one bf16 value per row: ggml shape [1, 37, 3] against [200, 37, 3]
    sc = oracle.bf16_round(rng.standard_normal((3, 37, 1)).astype(np.float32))
    n = node(OP["MUL"], tensor(out), tensor(xd), tensor(bf(oracle, sc)))
    assert hook.vla_cuda_bf16_forward(C.byref(n), stream())
    torch.cuda.synchronize()
    assert np.array_equal(back(oracle, out), oracle.bf16_round(x * sc))


def test_strided_view_operand(oracle, hook):
    """src0 is a column slice of a wider matrix (row stride larger than the row): handled by the strided operator."""
    import torch

    rng = np.random.default_rng(2)
    wide = oracle.bf16_round(rng.standard_normal((50, 96)).astype(np.float32))
    wd = bf(oracle, wide)
    view = wd[:, 16:80]
    b = oracle.bf16_round(rng.standard_normal((50, 64)).astype(np.float32))
    out = torch.empty((50, 64), dtype=torch.bfloat16, device="cuda")
    n = node(OP["ADD"], tensor(out), tensor(view), tensor(bf(oracle, b)))
    assert hook.vla_cuda_bf16_forward(C.byref(n), stream())
    torch.cuda.synchronize()
    assert np.array_equal(back(oracle, out), oracle.bf16_round(wide[:, 16:80] + b))


@pytest.mark.parametrize("op", ["ADD", "MUL"])
@pytest.mark.parametrize("f32_addends", [False, True])
def test_fused_run_of_adds_or_muls_matches_float_accumulation(oracle, hook, op, f32_addends):
    """ggml hands a run of up to 8 ADD / MUL nodes over as one node: src[0] the base, src[1..n] the addends; the
    result is accumulated in float and rounded once (src/cuda/vla_cuda_bf16.cu:330-389)."""
    import torch

    rng = np.random.default_rng(3)
    x = oracle.bf16_round(rng.standard_normal((40, 136)).astype(np.float32))
    adds = [rng.standard_normal(136).astype(np.float32) * 0.5 + (1.0 if op == "MUL" else 0.0) for _ in range(5)]
    if not f32_addends:
        adds = [oracle.bf16_round(a) for a in adds]
    out = torch.empty((40, 136), dtype=torch.bfloat16, device="cuda")
    dev = [to_dev(a) if f32_addends else bf(oracle, a) for a in adds]
    n = node(OP[op], tensor(out), tensor(bf(oracle, x)), *[tensor(d) for d in dev])
    assert hook.vla_cuda_bf16_fused_binbcast(C.byref(n), len(adds), stream())
    torch.cuda.synchronize()
    acc = x.copy()
    for a in adds:
        acc = (acc * a if op == "MUL" else acc + a).astype(np.float32)
    assert np.array_equal(back(oracle, out), oracle.bf16_round(acc))
    # an addend whose layout differs from src[1]'s is refused, as is a run of one
    odd = node(OP[op], tensor(out), tensor(bf(oracle, x)), tensor(dev[0]), tensor(bf(oracle, x)))
    assert not hook.vla_cuda_bf16_fused_binbcast(C.byref(odd), 2, stream())
    assert not hook.vla_cuda_bf16_fused_binbcast(C.byref(n), 1, stream())


def test_mul_mat_scale_norm_unary_nodes(oracle, hook):
    import torch

    rng = np.random.default_rng(4)
    w = oracle.bf16_round((rng.standard_normal((96, 256)) / 16).astype(np.float32))
    x = oracle.bf16_round(rng.standard_normal((2, 70, 256)).astype(np.float32))
    wd, xd = bf(oracle, w), bf(oracle, x)
    out = torch.empty((2, 70, 96), dtype=torch.bfloat16, device="cuda")
    n = node(OP["MUL_MAT"], tensor(out), tensor(wd), tensor(xd))
    assert hook.vla_cuda_bf16_forward(C.byref(n), stream())
    torch.cuda.synchronize()
    assert rel_l2(back(oracle, out), oracle.node_mul_mat(w, x)) <= 2e-3

    y = torch.empty_like(xd)
    n = node(OP["SCALE"], tensor(y), tensor(xd), params=(f32_bits(0.37), f32_bits(-1.25)))
    assert hook.vla_cuda_bf16_forward(C.byref(n), stream())
    torch.cuda.synchronize()
    d = np.abs(bf16_bits(y).astype(np.int32) - oracle.f32_to_bf16_bits(oracle.node_scale(x, 0.37, -1.25)).astype(np.int32))
    assert d.max() <= 1
    z = torch.empty_like(xd)
    for rms, opname in ((True, "RMS_NORM"), (False, "NORM")):
        n = node(OP[opname], tensor(z), tensor(xd), params=(f32_bits(1e-5),))
        assert hook.vla_cuda_bf16_forward(C.byref(n), stream())
        torch.cuda.synchronize()
        d = np.abs(bf16_bits(z).astype(np.int32) - oracle.f32_to_bf16_bits(oracle.node_norm(x, 1e-5, rms)).astype(np.int32))
        assert d.max() <= 1 and (d != 0).mean() < 2e-2
    for name in ("silu", "relu", "gelu", "gelu_erf"):
        n = node(OP["UNARY"], tensor(z), tensor(xd), params=(UNARY[name],))
        assert hook.vla_cuda_bf16_forward(C.byref(n), stream())
        torch.cuda.synchronize()
        d = np.abs(bf16_bits(z).astype(np.int32) - oracle.f32_to_bf16_bits(oracle.node_unary(name, x)).astype(np.int32))
        assert d.max() <= (0 if name == "relu" else 1)


def test_nodes_outside_the_contract_are_declined(oracle, hook):
    import torch

    x = torch.zeros((8, 64), dtype=torch.bfloat16, device="cuda")
    f = torch.zeros((8, 64), dtype=torch.float32, device="cuda")
    assert not hook.vla_cuda_bf16_forward(None, stream())
    assert not hook.vla_cuda_bf16_forward(C.byref(node(OP["SOFT_MAX"], tensor(x), tensor(x))), stream())
    assert not hook.vla_cuda_bf16_forward(C.byref(node(OP["ADD"], tensor(f), tensor(f), tensor(f))), stream())  # float32 node
    assert not hook.vla_cuda_bf16_forward(C.byref(node(OP["UNARY"], tensor(x), tensor(x), params=(UNARY["tanh"],))), stream())
    assert not hook.vla_cuda_bf16_forward(C.byref(node(OP["UNARY"], tensor(x), tensor(x[:, ::2]), params=(UNARY["silu"],))),
                                         stream())  # non-contiguous source of a dense-only operator
    wide = torch.zeros((8, 100), dtype=torch.bfloat16, device="cuda")
    assert not hook.vla_cuda_bf16_forward(C.byref(node(OP["MUL_MAT"], tensor(x), tensor(wide), tensor(wide))), stream())  # K % 8
