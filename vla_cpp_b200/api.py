"""ctypes binding of libvla_b200.so plus thin torch-tensor front ends.

torch is used for device memory and streams only; all arithmetic happens inside the
library's kernels.  Argument meaning and error behaviour follow the reference entry
points named in include/vla_b200.h.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libvla_b200.so")
_LIB = None

OK, ERR_ARG, ERR_CUDA, ERR_DEVICE, ERR_UNSUPPORTED = 0, -1, -2, -3, -4


class VlaB200Error(RuntimeError):
    def __init__(self, code, what):
        self.code = code
        super().__init__(f"{what}: status {code}" + (f" ({lib().vlab200_last_error().decode()})" if code == ERR_CUDA else ""))


def lib():
    """Loads the CUDA library; raises if it has not been built (no fallback path exists)."""
    global _LIB
    if _LIB is None:
        if not os.path.exists(LIB_PATH):
            raise FileNotFoundError(
                f"{LIB_PATH} is missing: build it with `python -m vla_cpp_b200.build` (needs nvcc)")
        L = C.CDLL(LIB_PATH)
        L.vlab200_last_error.restype = C.c_char_p
        L.vlab200_abi_version.restype = C.c_int32
        for name in EXPORTS:
            fn = getattr(L, name)
            if name.startswith("vlab200_") and name not in ("vlab200_last_error",):
                fn.restype = C.c_int32
        _LIB = L
    return _LIB


# every symbol include/vla_b200.h declares
EXPORTS = [
    "vlab200_abi_version", "vlab200_last_error", "vlab200_device_status",
    "vlab200_act_quant", "vlab200_ternary_linear",
    "bitlinear_int8xint2", "bitlinear_int8xint2_m", "bitvla_act_quant_cuda",
]


def _check(rc, what):
    if rc != OK:
        raise VlaB200Error(rc, what)


def _ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else C.c_void_p(0)


def _stream():
    import torch

    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def device_status(reset=True):
    out = C.c_int32(0)
    _check(lib().vlab200_device_status(C.byref(out), int(reset)), "vlab200_device_status")
    return out.value


def act_quant(x, q=None, scales=None):
    """x: cuda bf16 [M, K] -> (int8 [M, K], float32 [M])."""
    import torch

    assert x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous()
    m, k = x.shape
    q = torch.empty((m, k), dtype=torch.int8, device=x.device) if q is None else q
    scales = torch.empty((m,), dtype=torch.float32, device=x.device) if scales is None else scales
    _check(lib().vlab200_act_quant(_ptr(x), _ptr(q), _ptr(scales), m, k, _stream()), "vlab200_act_quant")
    return q, scales


def ternary_linear(a, w_ladder, s, ws, n, out=None, acc_out=None, path=0):
    """a: int8 [M, K]; w_ladder: uint8 [N*K/4]; s: f32 [M]; ws: f32 [ws_num] -> bf16 [M, N]."""
    import torch

    assert a.is_cuda and a.dtype == torch.int8 and a.is_contiguous()
    m, k = a.shape
    out = torch.empty((m, n), dtype=torch.bfloat16, device=a.device) if out is None else out
    _check(lib().vlab200_ternary_linear(_ptr(a), _ptr(w_ladder), _ptr(out), _ptr(acc_out), _ptr(s), _ptr(ws),
                                        int(ws.numel()), m, n, k, int(path), _stream()), "vlab200_ternary_linear")
    return out
