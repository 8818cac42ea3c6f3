"""Helpers shared by the GPU parity tests."""
import ctypes as C
import os

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def require_cuda():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from vla_cpp_b200 import api

    api.lib()  # a missing library is an error on a GPU box, not a skip
    return torch


def to_dev(a):
    import torch

    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def bf16_bits(t):
    """cuda bf16 tensor -> numpy uint16 bit patterns."""
    import torch

    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def bits_to_bf16_tensor(bits):
    import torch

    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).cuda().view(torch.bfloat16)


def rel_l2(a, b):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def reference_bitnet_lib():
    """The reference's own CUDA kernels (oracle/_ref/libbitnet_ref.so), or None."""
    p = os.path.join(ROOT, "oracle", "_ref", "libbitnet_ref.so")
    if not os.path.exists(p):
        return None
    return C.CDLL(p)
