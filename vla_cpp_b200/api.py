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
        detail = lib().vlab200_last_error().decode() if code in (ERR_CUDA, ERR_UNSUPPORTED) else ""
        super().__init__(f"{what}: status {code}" + (f" ({detail})" if detail else ""))


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
        L.vlab200_kv_store_bytes.restype = C.c_int64
        L.vlab200_engine_create.restype = C.c_void_p
        L.vlab200_engine_free.restype = None
        L.vlab200_prefill_create.restype = C.c_void_p
        L.vlab200_prefill_free.restype = None
        L.vlab200_vision_create.restype = C.c_void_p
        L.vlab200_vision_free.restype = None
        L.vlab200_vision_tokens_per_view.argtypes = [C.c_void_p]
        L.vlab200_bitvla_lm_init.restype = C.c_void_p
        L.vlab200_bitvla_lm_init.argtypes = [C.c_int32] * 6 + [C.c_float, C.c_float, C.c_int32, C.c_int32]
        L.vlab200_bitvla_lm_free.restype = None
        L.vlab200_gguf_open.restype = C.c_void_p
        L.vlab200_gguf_open.argtypes = [C.c_char_p]
        L.vlab200_gguf_close.restype = None
        L.vlab200_gguf_close.argtypes = [C.c_void_p]
        L.vlab200_gguf_n_tensors.restype = C.c_int64
        L.vlab200_gguf_n_tensors.argtypes = [C.c_void_p]
        L.vlab200_gguf_tensor_name.restype = C.c_char_p
        L.vlab200_gguf_tensor_name.argtypes = [C.c_void_p, C.c_int64]
        L.vlab200_gguf_tensor_data.restype = C.c_void_p
        L.vlab200_gguf_tensor_data.argtypes = [C.c_void_p, C.c_char_p]
        L.vlab200_gguf_tensor_info.argtypes = [C.c_void_p, C.c_char_p, C.POINTER(C.c_int32), C.POINTER(C.c_int32),
                                               C.POINTER(C.c_int64), C.POINTER(C.c_uint64)]
        L.vlab200_gguf_read_f32.argtypes = [C.c_void_p, C.c_char_p, C.c_void_p, C.c_int64, C.c_int32]
        L.vlab200_gguf_meta_u32.argtypes = [C.c_void_p, C.c_char_p, C.POINTER(C.c_uint32)]
        L.vlab200_gguf_meta_f64.argtypes = [C.c_void_p, C.c_char_p, C.POINTER(C.c_double)]
        L.vlab200_gguf_meta_str.argtypes = [C.c_void_p, C.c_char_p, C.c_char_p, C.c_int32]
        L.vlab200_bitvla_lm_create_from_gguf.restype = C.c_void_p
        L.vlab200_bitvla_lm_create_from_gguf.argtypes = [C.c_void_p, C.c_int32, C.c_int32]
        L.vlab200_engine_create_from_gguf.restype = C.c_void_p
        L.vlab200_engine_create_from_gguf.argtypes = [C.c_void_p, C.c_int32, C.c_int32]
        _LIB = L
    return _LIB


# every symbol include/vla_b200.h declares
EXPORTS = [
    "vlab200_abi_version", "vlab200_last_error", "vlab200_device_status", "vlab200_selftest_bounded_wait",
    "vlab200_kv_store_bytes", "vlab200_kv_store_write", "vlab200_rope_table", "vlab200_fold_norm_weight",
    "vlab200_qkv_rope_append",
    "vlab200_attention", "vlab200_denoise_attn_loop", "vlab200_denoise_attn_loop_host",
    "vlab200_denoise_attn_loop_static",
    "vlab200_engine_create", "vlab200_engine_free", "vlab200_engine_set_prefix", "vlab200_engine_denoise",
    "vlab200_engine_denoise_host", "vlab200_engine_run_stage", "vlab200_engine_set_prefix_len",
    "vlab200_engine_get_prefix", "vlab200_shard_range", "vlab200_engines_denoise_host",
    "vlab200_prefill_create", "vlab200_prefill_free", "vlab200_prefill_run", "vlab200_set_gemm_tiling",
    "vlab200_vision_create", "vlab200_vision_free", "vlab200_vision_tokens_per_view", "vlab200_vision_run",
    "vlab200_act_quant", "vlab200_ternary_linear", "vlab200_ternarize_pack",
    "vlab200_bitvla_lm_init", "vlab200_bitvla_lm_free", "vlab200_bitvla_lm_set_layer",
    "vlab200_bitvla_lm_set_output_norm", "vlab200_bitvla_lm_forward", "vlab200_bitvla_norm_quant",
    "vlab200_gguf_open", "vlab200_gguf_close", "vlab200_gguf_n_tensors", "vlab200_gguf_tensor_name",
    "vlab200_gguf_tensor_info", "vlab200_gguf_tensor_data", "vlab200_gguf_read_f32", "vlab200_gguf_meta_u32",
    "vlab200_gguf_meta_f64", "vlab200_gguf_meta_str", "vlab200_engine_create_from_gguf",
    "vlab200_bitvla_lm_create_from_gguf",
    "vlab200_node_mul_mat_bf16", "vlab200_node_bin_bf16", "vlab200_node_bin_nd_bf16", "vlab200_node_scale_bf16", "vlab200_node_unary_bf16",
    "vlab200_node_norm_bf16",
    "bitlinear_int8xint2", "bitlinear_int8xint2_m", "bitvla_act_quant_cuda",
    "bitvla_lm_cuda_init", "bitvla_lm_cuda_free", "bitvla_lm_cuda_set_layer", "bitvla_lm_cuda_set_output_norm",
    "bitvla_lm_cuda_forward",
    "bitvla_vit_cuda_init", "bitvla_vit_cuda_free", "bitvla_vit_cuda_set_layer", "bitvla_vit_cuda_set_embed",
    "bitvla_vit_cuda_set_mmproj", "bitvla_vit_cuda_forward",
    "bitvla_fp32head_cuda_init", "bitvla_fp32head_proprio_forward", "bitvla_fp32head_action_forward",
    "bitvla_fp32head_cuda_free",
]


def _check(rc, what):
    if rc != OK:
        raise VlaB200Error(rc, what)


def _ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else C.c_void_p(0)


def _stream():
    import torch

    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def set_gemm_tiling(tiling):
    """0 = automatic, 1 = 128x256 tiles, 2 = 128x128, 3 = CTA pairs, 4 = 128x64 (testing / measurement knob)."""
    _check(lib().vlab200_set_gemm_tiling(int(tiling)), "vlab200_set_gemm_tiling")


def device_status(reset=True):
    out = C.c_int32(0)
    _check(lib().vlab200_device_status(C.byref(out), int(reset)), "vlab200_device_status")
    return out.value


def selftest_bounded_wait(budget_cycles=100000):
    """Runs the kernel whose waits can never be satisfied; True when they gave up within the budget."""
    out = C.c_int32(0)
    _check(lib().vlab200_selftest_bounded_wait(C.c_int64(budget_cycles), C.byref(out), _stream()),
           "vlab200_selftest_bounded_wait")
    return bool(out.value)


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


def ternarize_pack(w):
    """w: cuda float32 [N, K] -> (uint8 [N*K/4] ladder pack, float32 [1] absmean scale), computed on the device."""
    import torch

    assert w.is_cuda and w.dtype == torch.float32 and w.is_contiguous() and w.dim() == 2
    n, k = w.shape
    packed = torch.empty((n * k // 4,), dtype=torch.uint8, device=w.device)
    scale = torch.empty((1,), dtype=torch.float32, device=w.device)
    scratch = torch.empty((1,), dtype=torch.float64, device=w.device)
    _check(lib().vlab200_ternarize_pack(_ptr(w), C.c_int64(n), C.c_int64(k), _ptr(packed), _ptr(scale), _ptr(scratch),
                                        _stream()), "vlab200_ternarize_pack")
    return packed, scale


MASK_NONE, MASK_PI0, MASK_CAUSAL, MASK_LAST_PRIVATE = 0, 1, 2, 3


class _KvStoreC(C.Structure):
    _fields_ = [("k_pages", C.c_void_p), ("v_pages", C.c_void_p), ("n_layers", C.c_int32), ("n_obs", C.c_int32),
                ("n_kv", C.c_int32), ("head_dim", C.c_int32), ("cap", C.c_int32), ("prefix_len", C.c_int32)]


class KvStore:
    """bf16 prefix+suffix K/V pages [n_layers][n_obs][n_kv][cap][head_dim] in device memory."""

    def __init__(self, n_layers, n_obs, n_kv, head_dim, prefix_len, suffix_len, device="cuda"):
        import torch

        self.cap = prefix_len + suffix_len
        nbytes = lib().vlab200_kv_store_bytes(n_layers, n_obs, n_kv, head_dim, self.cap)
        if nbytes < 0:
            raise VlaB200Error(ERR_ARG, "vlab200_kv_store_bytes")
        shape = (n_layers, n_obs, n_kv, self.cap, head_dim)
        self.k = torch.zeros(shape, dtype=torch.bfloat16, device=device)
        self.v = torch.zeros(shape, dtype=torch.bfloat16, device=device)
        assert self.k.numel() * 2 == nbytes
        self.n_layers, self.n_obs, self.n_kv, self.head_dim = n_layers, n_obs, n_kv, head_dim
        self.prefix_len, self.suffix_len = prefix_len, suffix_len
        self.c = _KvStoreC(self.k.data_ptr(), self.v.data_ptr(), n_layers, n_obs, n_kv, head_dim, self.cap,
                           prefix_len)

    def write_prefix(self, layer, k_f32, v_f32, obs0=0):
        """k_f32, v_f32: cuda float32 [n, prefix_len, n_kv, head_dim] (K already rotated)."""
        assert k_f32.is_contiguous() and v_f32.is_contiguous()
        n = k_f32.shape[0]
        assert tuple(k_f32.shape) == (n, self.prefix_len, self.n_kv, self.head_dim) == tuple(v_f32.shape)
        _check(lib().vlab200_kv_store_write(C.byref(self.c), layer, obs0, n, _ptr(k_f32), _ptr(v_f32), _stream()),
               "vlab200_kv_store_write")


def rope_table(pos0, S, head_dim, base=10000.0, device="cuda"):
    import torch

    cos_t = torch.empty((S, head_dim // 2), dtype=torch.float32, device=device)
    sin_t = torch.empty_like(cos_t)
    _check(lib().vlab200_rope_table(_ptr(cos_t), _ptr(sin_t), pos0, S, head_dim, C.c_float(base), _stream()),
           "vlab200_rope_table")
    return cos_t, sin_t


def fold_norm_weight(w, ln_w):
    """bf16 [..., rows, H] weight times an RMSNorm weight [H] (float32) -> new bf16 tensor."""
    import torch

    assert w.dtype == torch.bfloat16 and w.is_contiguous() and ln_w.dtype == torch.float32
    out = torch.empty_like(w)
    H = w.shape[-1]
    _check(lib().vlab200_fold_norm_weight(_ptr(w), _ptr(ln_w), _ptr(out), C.c_int64(w.numel() // H), H, _stream()),
           "vlab200_fold_norm_weight")
    return out


def qkv_rope_append(store, layer, x, ln_w, wqkv, rope, eps, S, n_q, q_out=None, project_kv=True):
    """x: [n_obs*S, H] bf16 or f32; wqkv: bf16 [(n_q + 2 n_kv) hd, H]; rope = (cos, sin) tables.
    Returns q: bf16 [n_obs, n_q, S, hd]; suffix K/V land in the store."""
    import torch

    assert x.is_contiguous() and wqkv.is_contiguous() and wqkv.dtype == torch.bfloat16
    H = x.shape[-1]
    if q_out is None:
        q_out = torch.empty((store.n_obs, n_q, S, store.head_dim), dtype=torch.bfloat16, device=x.device)
    _check(lib().vlab200_qkv_rope_append(C.byref(store.c), layer, _ptr(x), int(x.dtype == torch.float32), _ptr(ln_w),
                                         _ptr(wqkv), _ptr(rope[0]), _ptr(rope[1]), C.c_float(eps), S, H, n_q,
                                         int(project_kv), _ptr(q_out), _stream()), "vlab200_qkv_rope_append")
    return q_out


def attention(store, layer, q, S, n_q, kv_len, mask_mode, pad_ranges=None, out=None):
    """q: bf16 [n_obs, n_q, S, hd] -> bf16 [n_obs, S, n_q*hd]."""
    import torch

    if out is None:
        out = torch.empty((store.n_obs, S, n_q * store.head_dim), dtype=torch.bfloat16, device=q.device)
    _check(lib().vlab200_attention(C.byref(store.c), layer, _ptr(q), _ptr(out), S, n_q, kv_len, mask_mode,
                                   _ptr(pad_ranges), _stream()), "vlab200_attention")
    return out


class _DenoiseAttnArgs(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("n_layers", "steps", "S", "H", "n_q", "mask_mode", "x_is_f32")] + [
        ("eps", C.c_float)] + [(n, C.c_void_p) for n in (
            "x", "ln_w", "wqkv", "rope_cos", "rope_sin", "q_scratch", "out", "pad_ranges")]


class DenoiseAttn:
    """The isolated denoise-attention op over a KvStore: steps x layers of fused
    QKV+RoPE+append and attention, driven by the library's C++ loop."""

    def __init__(self, store, H, n_q, S, ln_w, wqkv, eps, mask_mode, pos0=None, rope_base=10000.0, fold=True):
        """ln_w: f32 [n_layers, H]; wqkv: bf16 [n_layers, (n_q+2n_kv)hd, H].  fold=True multiplies the
        RMSNorm weights into wqkv once (load-time step), which lets bf16 hidden states go straight
        to the tensor cores by TMA; fold=False keeps them separate (needed for float32 hidden states)."""
        import torch

        self.store, self.H, self.n_q, self.S, self.eps, self.mask_mode = store, H, n_q, S, eps, mask_mode
        self.n_layers = wqkv.shape[0]
        if fold:
            self.wqkv = torch.stack([fold_norm_weight(wqkv[l].contiguous(), ln_w[l].contiguous())
                                     for l in range(self.n_layers)])
            self.ln_w = None
        else:
            self.ln_w, self.wqkv = ln_w.contiguous(), wqkv.contiguous()
        self.rope = rope_table(store.prefix_len if pos0 is None else pos0, S, store.head_dim, rope_base)
        dev = wqkv.device
        self.q = torch.empty((store.n_obs, n_q, S, store.head_dim), dtype=torch.bfloat16, device=dev)
        self.out = torch.empty((self.n_layers, store.n_obs, S, n_q * store.head_dim), dtype=torch.bfloat16,
                               device=dev)
        self._stage = None

    def _args(self, x_ptr, steps, x_is_f32):
        return _DenoiseAttnArgs(self.n_layers, steps, self.S, self.H, self.n_q, self.mask_mode, int(x_is_f32),
                                self.eps, x_ptr, self.ln_w.data_ptr() if self.ln_w is not None else None, self.wqkv.data_ptr(),
                                self.rope[0].data_ptr(), self.rope[1].data_ptr(), self.q.data_ptr(),
                                self.out.data_ptr(), None)

    def run(self, x):
        """x: cuda [steps, n_layers, n_obs*S, H] bf16/f32.  Returns the last step's outputs (device)."""
        import torch

        assert x.is_cuda and x.is_contiguous() and x.shape[1] == self.n_layers
        a = self._args(x.data_ptr(), x.shape[0], x.dtype == torch.float32)
        _check(lib().vlab200_denoise_attn_loop(C.byref(self.store.c), C.byref(a), _stream()),
               "vlab200_denoise_attn_loop")
        return self.out

    def run_static(self, x):
        """Like run(), but the query buffer comes from the library's built-in scratch array (no
        device allocation on this path; limited to 16 MiB of queries)."""
        import torch

        assert x.is_cuda and x.is_contiguous() and x.shape[1] == self.n_layers
        a = self._args(x.data_ptr(), x.shape[0], x.dtype == torch.float32)
        a.q_scratch = None
        _check(lib().vlab200_denoise_attn_loop_static(C.byref(self.store.c), C.byref(a), _stream()),
               "vlab200_denoise_attn_loop_static")
        return self.out

    def run_host(self, x_host, out_host):
        """x_host: pinned host tensor [steps, n_layers, n_obs*S, H]; out_host: pinned host bf16 like self.out."""
        import torch

        assert not x_host.is_cuda and x_host.is_contiguous()
        step_elems = x_host[0].numel()
        if self._stage is None or self._stage.numel() != 2 * step_elems or self._stage.dtype != x_host.dtype:
            self._stage = torch.empty(2 * step_elems, dtype=x_host.dtype, device=self.out.device)
        a = self._args(x_host.data_ptr(), x_host.shape[0], x_host.dtype == torch.float32)
        _check(lib().vlab200_denoise_attn_loop_host(C.byref(self.store.c), C.byref(a), _ptr(self._stage),
                                                    C.c_void_p(out_host.data_ptr()), _stream()),
               "vlab200_denoise_attn_loop_host")
        return out_host


class Gguf:
    """A GGUF checkpoint opened through the library's reader (host only; no GPU needed)."""

    def __init__(self, path):
        self.h = lib().vlab200_gguf_open(str(path).encode())
        if not self.h:
            raise VlaB200Error(ERR_ARG, "vlab200_gguf_open: " + lib().vlab200_last_error().decode())

    def close(self):
        if getattr(self, "h", None):
            lib().vlab200_gguf_close(self.h)
            self.h = None

    __del__ = close

    def names(self):
        n = lib().vlab200_gguf_n_tensors(self.h)
        return [lib().vlab200_gguf_tensor_name(self.h, i).decode() for i in range(n)]

    def info(self, name):
        """-> (ggml type id, dims fastest-first, bytes) or None."""
        t, nd, nb = C.c_int32(), C.c_int32(), C.c_uint64()
        dims = (C.c_int64 * 4)()
        if lib().vlab200_gguf_tensor_info(self.h, name.encode(), C.byref(t), C.byref(nd), dims, C.byref(nb)) != OK:
            return None
        return t.value, [dims[i] for i in range(nd.value)], nb.value

    def raw(self, name):
        """The tensor's bytes as a numpy uint8 array (a copy)."""
        import numpy as np

        inf = self.info(name)
        ptr = lib().vlab200_gguf_tensor_data(self.h, name.encode())
        if inf is None or not ptr:
            raise KeyError(name)
        return np.ctypeslib.as_array(C.cast(ptr, C.POINTER(C.c_uint8)), shape=(inf[2],)).copy()

    def f32(self, name, gemma_norm=False):
        import numpy as np

        inf = self.info(name)
        if inf is None:
            raise KeyError(name)
        out = np.empty(inf[1][::-1], dtype=np.float32)
        _check(lib().vlab200_gguf_read_f32(self.h, name.encode(), out.ctypes.data_as(C.c_void_p), out.size,
                                           int(gemma_norm)), "vlab200_gguf_read_f32")
        return out

    def meta(self, key):
        u, d = C.c_uint32(), C.c_double()
        buf = C.create_string_buffer(256)
        if lib().vlab200_gguf_meta_u32(self.h, key.encode(), C.byref(u)) == OK:
            return u.value
        if lib().vlab200_gguf_meta_f64(self.h, key.encode(), C.byref(d)) == OK:
            return d.value
        if lib().vlab200_gguf_meta_str(self.h, key.encode(), buf, 256) == OK:
            return buf.value.decode()
        return None


class _PolicyConfig(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("model", "n_layers", "H", "n_q", "n_kv", "head_dim", "inter", "chunk",
                                          "action_dim", "state_dim", "steps", "self_every")] + [
        ("rms_eps", C.c_float), ("rope_base", C.c_float), ("min_period", C.c_double), ("max_period", C.c_double),
        ("cond_dim", C.c_int32)]


_PER_LAYER = ("wq", "wk", "wv", "wo", "wgate", "wup", "wdown", "ln_in", "ln_post")
_GLOBAL = ("w_sp", "b_sp", "w_ain", "b_ain", "w_at1", "b_at1", "w_at2", "b_at2", "out_norm", "w_aout", "b_aout")
# pi0.5 (model 2): adaptive-norm dense maps per layer and the time MLP, all float32
_ADA_PER_LAYER = ("ada_in_w", "ada_in_b", "ada_post_w", "ada_post_b")
_ADA_GLOBAL = ("ada_final_w", "ada_final_b", "w_tin", "b_tin", "w_tout", "b_tout")


class _PolicyWeights(C.Structure):
    _fields_ = ([(n, C.POINTER(C.c_void_p)) for n in _PER_LAYER] + [(n, C.c_void_p) for n in _GLOBAL] +
                [(n, C.POINTER(C.c_void_p)) for n in _ADA_PER_LAYER] + [(n, C.c_void_p) for n in _ADA_GLOBAL])


class PolicyEngine:
    """Batched flow-matching denoise loop of a pi0- or SmolVLA-shaped action expert.

    cfg: dict with the vlab200_policy_config fields.  weights: dict of cuda tensors -- per-layer
    lists for wq, wk, wv, wo, wgate, wup, wdown (bf16 [out, in]) and ln_in, ln_post (f32), plus
    w_sp/b_sp (pi0), w_ain/b_ain, w_at1/b_at1, w_at2/b_at2, out_norm, w_aout/b_aout."""

    def __init__(self, cfg, weights, max_obs, prefix_len):
        import torch

        self.cfg = dict(cfg)
        c = _PolicyConfig(**{k: cfg.get(k, 0) if k == "cond_dim" else cfg[k] for k, _ in _PolicyConfig._fields_})
        w = _PolicyWeights()
        keep = []
        ada = cfg["model"] == 2
        for name in _ADA_PER_LAYER + _ADA_GLOBAL if ada else ():
            if name in _ADA_PER_LAYER:
                ts = [t.contiguous() for t in weights[name]]
                assert all(t.is_cuda and t.dtype == torch.float32 for t in ts), name
                arr = (C.c_void_p * len(ts))(*[t.data_ptr() for t in ts])
                keep += [ts, arr]
                setattr(w, name, C.cast(arr, C.POINTER(C.c_void_p)))
            else:
                t = weights[name].contiguous()
                assert t.is_cuda and t.dtype == torch.float32, name
                keep.append(t)
                setattr(w, name, t.data_ptr())
        for name in _PER_LAYER:
            if ada and name.startswith("ln"):
                continue
            ts = [t.contiguous() for t in weights[name]]
            want = torch.float32 if name.startswith("ln") else torch.bfloat16
            assert all(t.is_cuda and t.dtype == want for t in ts), name
            arr = (C.c_void_p * len(ts))(*[t.data_ptr() for t in ts])
            keep += [ts, arr]
            setattr(w, name, C.cast(arr, C.POINTER(C.c_void_p)))
        for name in _GLOBAL:
            t = weights.get(name)
            if t is None:
                setattr(w, name, None)
                continue
            t = t.contiguous()
            want = torch.bfloat16 if name.startswith("w_") else torch.float32
            assert t.is_cuda and t.dtype == want, name
            keep.append(t)
            setattr(w, name, t.data_ptr())
        self.max_obs, self.prefix_len = max_obs, prefix_len
        self.chunk, self.A, self.sd = cfg["chunk"], cfg["action_dim"], cfg["state_dim"]
        self.h = lib().vlab200_engine_create(C.byref(c), C.byref(w), max_obs, prefix_len)
        torch.cuda.synchronize()
        del keep
        if not self.h:
            raise VlaB200Error(ERR_CUDA, "vlab200_engine_create")

    @classmethod
    def from_gguf(cls, gguf, max_obs, prefix_len):
        """The engine of a pi0 or SmolVLA checkpoint (reference tensor names and metadata keys)."""
        import torch

        self = cls.__new__(cls)
        self.h = lib().vlab200_engine_create_from_gguf(gguf.h, max_obs, prefix_len)
        torch.cuda.synchronize()
        if not self.h:
            raise VlaB200Error(ERR_ARG, "vlab200_engine_create_from_gguf: " + lib().vlab200_last_error().decode())
        self.max_obs, self.prefix_len = max_obs, prefix_len
        arch = gguf.meta("general.architecture")
        self.chunk, self.A, self.sd = (gguf.meta(arch + ".chunk_size"), gguf.meta(arch + ".max_action_dim"),
                                       gguf.meta(arch + ".max_state_dim"))
        self.cfg = None
        return self

    def __del__(self):
        if getattr(self, "h", None):
            lib().vlab200_engine_free(C.c_void_p(self.h))
            self.h = None

    def set_prefix(self, layer, k_f32, v_f32, obs0=0):
        """k_f32, v_f32: cuda float32 [n, prefix_len, n_kv, hd] (K rotated)."""
        assert k_f32.is_contiguous() and v_f32.is_contiguous()
        _check(lib().vlab200_engine_set_prefix(C.c_void_p(self.h), layer, obs0, k_f32.shape[0], _ptr(k_f32),
                                               _ptr(v_f32), _stream()), "vlab200_engine_set_prefix")

    def denoise(self, x0, state=None, pos_base=-1, pad_ranges=None):
        """x0: cuda f32 [n_obs, chunk, A]; state: cuda f32 [n_obs, state_dim] -> x_T like x0."""
        import torch

        assert x0.is_cuda and x0.dtype == torch.float32 and x0.is_contiguous()
        out = torch.empty_like(x0)
        _check(lib().vlab200_engine_denoise(C.c_void_p(self.h), x0.shape[0], _ptr(state), _ptr(x0), _ptr(out),
                                            pos_base, _ptr(pad_ranges), _stream()), "vlab200_engine_denoise")
        return out

    def denoise_host(self, x0_host, state_host, out_host, pos_base=-1, pad_ranges_host=None):
        """Pinned host float32 buffers in and out (pad_ranges_host: host int32 [n_obs, 2]); copies are enqueued
        on the current stream."""
        _check(lib().vlab200_engine_denoise_host(
            C.c_void_p(self.h), x0_host.shape[0],
            C.c_void_p(state_host.data_ptr()) if state_host is not None else None,
            C.c_void_p(x0_host.data_ptr()), C.c_void_p(out_host.data_ptr()), pos_base,
            C.c_void_p(pad_ranges_host.data_ptr()) if pad_ranges_host is not None else None, _stream()),
            "vlab200_engine_denoise_host")
        return out_host


    def get_prefix(self, layer, n_kv, head_dim, n_obs=1, obs0=0):
        """-> (K, V) cuda float32 [n_obs, prefix_len, n_kv, head_dim] read back from the pages."""
        import torch

        k = torch.empty((n_obs, self.prefix_len, n_kv, head_dim), dtype=torch.float32, device="cuda")
        v = torch.empty_like(k)
        _check(lib().vlab200_engine_get_prefix(C.c_void_p(self.h), layer, obs0, n_obs, _ptr(k), _ptr(v), _stream()),
               "vlab200_engine_get_prefix")
        return k, v

    def set_prefix_len(self, prefix_len):
        """Prefix rows in use from now on (<= the length the engine was created with)."""
        _check(lib().vlab200_engine_set_prefix_len(C.c_void_p(self.h), int(prefix_len)), "vlab200_engine_set_prefix_len")
        self.prefix_len = int(prefix_len)

    STAGES = {"qkv": 0, "attention": 1, "o_proj": 2, "gate_up": 3, "down": 4}

    def run_stage(self, layer, stage, n_obs, reps=1):
        """Measurement hook: `reps` launches of one stage of one expert layer (after a denoise call)."""
        _check(lib().vlab200_engine_run_stage(C.c_void_p(self.h), layer, self.STAGES[stage], n_obs, reps, _stream()),
               "vlab200_engine_run_stage")


class _PrefillConfig(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("n_layers", "hidden", "n_q", "n_kv", "head_dim", "inter", "act")] + [
        ("rms_eps", C.c_float), ("rope_base", C.c_float)]


class _PrefillWeights(C.Structure):
    _fields_ = [(n, C.POINTER(C.c_void_p)) for n in _PER_LAYER]


class Prefill:
    """The backbone's layers over the prefix embeddings, writing K/V straight into a PolicyEngine's pages.

    cfg: dict with the vlab200_prefill_config fields (act: 1 SiLU, 2 tanh-GELU); weights: per-layer lists wq, wk,
    wv, wo, wgate, wup, wdown (cuda bf16 [out, in]) and ln_in, ln_post (cuda float32)."""

    def __init__(self, cfg, weights, max_obs, max_prefix):
        import torch

        c = _PrefillConfig(**{k: cfg[k] for k, _ in _PrefillConfig._fields_})
        w = _PrefillWeights()
        keep = []
        for name in _PER_LAYER:
            ts = [t.contiguous() for t in weights[name]]
            want = torch.float32 if name.startswith("ln") else torch.bfloat16
            assert all(t.is_cuda and t.dtype == want for t in ts), name
            arr = (C.c_void_p * len(ts))(*[t.data_ptr() for t in ts])
            keep += [ts, arr]
            setattr(w, name, C.cast(arr, C.POINTER(C.c_void_p)))
        self.h = lib().vlab200_prefill_create(C.byref(c), C.byref(w), max_obs, max_prefix)
        torch.cuda.synchronize()
        del keep
        if not self.h:
            raise VlaB200Error(ERR_CUDA, "vlab200_prefill_create: " + lib().vlab200_last_error().decode())

    def __del__(self):
        if getattr(self, "h", None):
            lib().vlab200_prefill_free(C.c_void_p(self.h))
            self.h = None

    def run(self, engine, x_emb, positions=None, mask_mode=MASK_NONE, pad_ranges=None, obs0=0):
        """x_emb: cuda float32 [n_obs, P, hidden]; positions: host int32 array [P] or None (0..P-1)."""
        import numpy as np
        import torch

        assert x_emb.is_cuda and x_emb.dtype == torch.float32 and x_emb.is_contiguous()
        n_obs, P = x_emb.shape[0], x_emb.shape[1]
        pos = None
        if positions is not None:
            pos = np.ascontiguousarray(positions, dtype=np.int32)
            assert pos.size == P
        _check(lib().vlab200_prefill_run(C.c_void_p(self.h), C.c_void_p(engine.h), obs0, n_obs, _ptr(x_emb), P,
                                         pos.ctypes.data_as(C.c_void_p) if pos is not None else None, mask_mode,
                                         _ptr(pad_ranges), _stream()), "vlab200_prefill_run")
        torch.cuda.synchronize()  # pos (host memory) must outlive the copy enqueued on the stream


class VlaImage(C.Structure):
    _fields_ = [("data", C.c_void_p), ("w", C.c_int32), ("h", C.c_int32), ("format", C.c_int32)]


class VlaInputs(C.Structure):
    _fields_ = [("images", C.POINTER(VlaImage)), ("n_images", C.c_int32), ("precomputed_img_emb", C.POINTER(C.c_float)),
                ("n_img_views", C.c_int32), ("lang_tokens", C.POINTER(C.c_int32)), ("n_lang", C.c_int32),
                ("state", C.POINTER(C.c_float)), ("noise", C.POINTER(C.c_float)), ("attention_mask", C.POINTER(C.c_int32)),
                ("attention_mask_n", C.c_int32), ("timing_detail", C.c_int32)]


class VlaStats(C.Structure):
    _fields_ = [(n, C.c_float) for n in ("ms_total", "ms_vision", "ms_inference", "ms_prefill", "ms_denoise")]


class VlaModel:
    """include/vla.h from Python: vla_model_load / vla_predict / vla_last_stats on a pi0 or SmolVLA GGUF checkpoint.

    predict(): images = list of numpy arrays [side, side, 3] (uint8 0..255 or float32 0..1) for the checkpoint's own
    vision tower, or img_emb = float32 [n_views * n_img, hidden] with n_views; lang_tokens int32; state float32
    [max_state_dim]; noise float32 [n_suffix, max_action_dim] or None (sampled inside).  Returns float32
    [n_suffix, max_action_dim]; self.stats holds the phase times of the last call."""

    def __init__(self, path):
        L = lib()
        L.vla_model_load.restype = C.c_void_p
        L.vla_model_load.argtypes = [C.c_char_p, C.c_char_p, C.c_char_p]
        L.vla_model_free.argtypes = [C.c_void_p]
        L.vla_predict.argtypes = [C.c_void_p, C.POINTER(VlaInputs), C.POINTER(C.POINTER(C.c_float)), C.POINTER(C.c_int64)]
        L.vla_free_actions.argtypes = [C.POINTER(C.c_float)]
        L.vla_last_stats.argtypes = [C.c_void_p, C.POINTER(VlaStats)]
        self.h = L.vla_model_load(None, str(path).encode(), None)
        if not self.h:
            raise VlaB200Error(ERR_ARG, "vla_model_load: " + L.vlab200_last_error().decode())
        self.stats = VlaStats()

    def close(self):
        if getattr(self, "h", None):
            lib().vla_model_free(self.h)
            self.h = None

    __del__ = close

    def predict(self, lang_tokens, state, images=None, img_emb=None, n_views=0, noise=None, timing=True):
        import numpy as np

        f32 = lambda a: None if a is None else np.ascontiguousarray(a, np.float32)
        fp = lambda a: None if a is None else a.ctypes.data_as(C.POINTER(C.c_float))
        lang = np.ascontiguousarray(lang_tokens, np.int32)
        state, noise, img_emb = f32(state), f32(noise), f32(img_emb)
        inp = VlaInputs()
        keep = []
        if images is not None:
            arr = (VlaImage * len(images))()
            for v, a in enumerate(images):
                a = np.ascontiguousarray(a)
                assert a.dtype in (np.uint8, np.float32) and a.ndim == 3 and a.shape[2] == 3
                keep.append(a)
                arr[v].data, arr[v].w, arr[v].h, arr[v].format = a.ctypes.data, a.shape[1], a.shape[0], int(a.dtype == np.float32)
            inp.images, inp.n_images = arr, len(images)
        else:
            inp.precomputed_img_emb, inp.n_img_views = fp(img_emb), n_views
        inp.lang_tokens, inp.n_lang = lang.ctypes.data_as(C.POINTER(C.c_int32)), lang.size
        inp.state, inp.noise, inp.timing_detail = fp(state), fp(noise), 1 if timing else 0
        act, n = C.POINTER(C.c_float)(), C.c_int64(0)
        rc = lib().vla_predict(self.h, C.byref(inp), C.byref(act), C.byref(n))
        if rc != 0:
            raise VlaB200Error(rc, "vla_predict: " + lib().vlab200_last_error().decode())
        out = np.ctypeslib.as_array(act, shape=(n.value,)).copy()
        lib().vla_free_actions(act)
        lib().vla_last_stats(self.h, C.byref(self.stats))
        rows = noise.shape[0] if noise is not None and noise.ndim == 2 else None
        return out.reshape(rows, -1) if rows else out


class _VisionConfig(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("image", "patch", "hidden", "n_layers", "n_heads", "inter", "shuffle",
                                         "out_dim")] + [("ln_eps", C.c_float), ("out_scale", C.c_float)]


_VISION_LAYER_VECS = ("ln1_w", "ln1_b", "ln2_w", "ln2_b")
_VISION_LAYER_MATS = ("wq", "wk", "wv", "wo", "fc1", "fc2")
_VISION_LAYER_BIAS = ("bq", "bk", "bv", "bo", "b1", "b2")


class _VisionWeights(C.Structure):
    _fields_ = ([("patch_w", C.c_void_p), ("patch_b", C.c_void_p), ("pos", C.c_void_p)] +
                [(n, C.POINTER(C.c_void_p)) for n in _VISION_LAYER_VECS + _VISION_LAYER_MATS + _VISION_LAYER_BIAS] +
                [("post_w", C.c_void_p), ("post_b", C.c_void_p), ("connector", C.c_void_p), ("connector_b", C.c_void_p)])


class VisionTower:
    """SigLIP encoder + connector: camera views -> the image-token embeddings of the prefix.

    cfg: dict with the vlab200_vision_config fields; weights: patch_w (cuda bf16 [hidden, 3 * patch * patch]),
    patch_b, pos, post_w, post_b (cuda float32), connector (cuda bf16 [out_dim, hidden * shuffle^2]), optional
    connector_b, and per-layer lists ln1_w, ln1_b, ln2_w, ln2_b, bq, bk, bv, bo, b1, b2 (float32), wq, wk, wv, wo,
    fc1, fc2 (bf16 [out, in])."""

    def __init__(self, cfg, weights, max_views=4):
        import torch

        c = _VisionConfig(**{k: cfg[k] for k, _ in _VisionConfig._fields_})
        w = _VisionWeights()
        keep = []
        for name in ("patch_w", "patch_b", "pos", "post_w", "post_b", "connector", "connector_b"):
            t = weights.get(name)
            if t is None:
                continue
            t = t.contiguous()
            assert t.is_cuda and t.dtype == (torch.bfloat16 if name in ("patch_w", "connector") else torch.float32), name
            keep.append(t)
            setattr(w, name, t.data_ptr())
        for name in _VISION_LAYER_VECS + _VISION_LAYER_MATS + _VISION_LAYER_BIAS:
            ts = [t.contiguous() for t in weights[name]]
            want = torch.bfloat16 if name in _VISION_LAYER_MATS else torch.float32
            assert len(ts) == cfg["n_layers"] and all(t.is_cuda and t.dtype == want for t in ts), name
            arr = (C.c_void_p * len(ts))(*[t.data_ptr() for t in ts])
            keep += [ts, arr]
            setattr(w, name, C.cast(arr, C.POINTER(C.c_void_p)))
        self.cfg = dict(cfg)
        self.h = lib().vlab200_vision_create(C.byref(c), C.byref(w), max_views)
        torch.cuda.synchronize()
        del keep
        if not self.h:
            raise VlaB200Error(ERR_CUDA, "vlab200_vision_create: " + lib().vlab200_last_error().decode())
        self.tokens_per_view = lib().vlab200_vision_tokens_per_view(C.c_void_p(self.h))

    def __del__(self):
        if getattr(self, "h", None):
            lib().vlab200_vision_free(C.c_void_p(self.h))
            self.h = None

    def run(self, pixels):
        """pixels: cuda uint8 (0..255) or float32 (0..1) [n_views, image, image, 3] -> float32 [n_views * tokens, out_dim]."""
        import torch

        assert pixels.is_cuda and pixels.is_contiguous() and pixels.dtype in (torch.uint8, torch.float32)
        side = self.cfg["image"]
        assert tuple(pixels.shape[1:]) == (side, side, 3), pixels.shape
        n_views = pixels.shape[0]
        out = torch.empty((n_views * self.tokens_per_view, self.cfg["out_dim"]), dtype=torch.float32, device=pixels.device)
        _check(lib().vlab200_vision_run(C.c_void_p(self.h), _ptr(pixels), 1 if pixels.dtype == torch.float32 else 0, n_views,
                                        _ptr(out), _stream()), "vlab200_vision_run")
        return out


NQ_PLAIN, NQ_ADD, NQ_GATE_UP = 0, 1, 2


def bitvla_norm_quant(x, w, eps, mode=NQ_PLAIN, add=None, quantise=True):
    """x: cuda bf16 [M, K] (mode 2: [M, 2K]) -> (int8 [M, K], float32 [M]) or, with quantise=False, bf16 [M, K].
    mode 1 also replaces x by x + add."""
    import torch

    assert x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous() and w.dtype == torch.bfloat16
    m, k = x.shape[0], w.shape[0]
    assert x.shape[1] == (2 * k if mode == NQ_GATE_UP else k)
    if quantise:
        q = torch.empty((m, k), dtype=torch.int8, device=x.device)
        s = torch.empty((m,), dtype=torch.float32, device=x.device)
        y = None
    else:
        q = s = None
        y = torch.empty((m, k), dtype=torch.bfloat16, device=x.device)
    _check(lib().vlab200_bitvla_norm_quant(_ptr(x), _ptr(add), _ptr(w), C.c_float(eps), m, k, mode, _ptr(q), _ptr(s),
                                           _ptr(y), _stream()), "vlab200_bitvla_norm_quant")
    return (q, s) if quantise else y


NODE_UNARY = {"silu": 0, "relu": 1, "gelu": 2, "gelu_erf": 3}


def _bf16_cuda(*ts):
    import torch

    for t in ts:
        assert t.is_cuda and t.dtype == torch.bfloat16 and t.is_contiguous()


def node_mul_mat(w, x):
    """w: cuda bf16 [N, K] or [B, N, K]; x: [M, K] or [B, M, K] -> bf16 [.., M, N] = x @ w^T."""
    import torch

    _bf16_cuda(w, x)
    nb = x.shape[0] if x.dim() == 3 else 1
    m, k = x.shape[-2], x.shape[-1]
    n = w.shape[-2]
    assert w.shape[-1] == k and (w.dim() == 2 or w.shape[0] == nb)
    out = torch.empty((*x.shape[:-1], n), dtype=torch.bfloat16, device=x.device)
    _check(lib().vlab200_node_mul_mat_bf16(_ptr(w), _ptr(x), _ptr(out), n, m, k, nb, int(w.dim() == 3), _stream()),
           "vlab200_node_mul_mat_bf16")
    return out


def node_bin(op, a, b):
    """a: cuda bf16; b: bf16 or float32 whose shape matches the trailing dims of a -> a + b or a * b."""
    import torch

    _bf16_cuda(a)
    assert b.is_cuda and b.is_contiguous() and b.dtype in (torch.bfloat16, torch.float32)
    out = torch.empty_like(a)
    _check(lib().vlab200_node_bin_bf16({"add": 0, "mul": 1}[op], _ptr(a), _ptr(b), int(b.dtype == torch.float32),
                                       _ptr(out), C.c_int64(a.numel()), C.c_int64(b.numel()), _stream()),
           "vlab200_node_bin_bf16")
    return out


def node_scale(x, scale, bias=0.0):
    import torch

    _bf16_cuda(x)
    out = torch.empty_like(x)
    _check(lib().vlab200_node_scale_bf16(_ptr(x), _ptr(out), C.c_int64(x.numel()), C.c_float(scale), C.c_float(bias),
                                         _stream()), "vlab200_node_scale_bf16")
    return out


def node_unary(op, x):
    import torch

    _bf16_cuda(x)
    out = torch.empty_like(x)
    _check(lib().vlab200_node_unary_bf16(NODE_UNARY[op], _ptr(x), _ptr(out), C.c_int64(x.numel()), _stream()),
           "vlab200_node_unary_bf16")
    return out


def node_norm(x, eps, rms=True):
    import torch

    _bf16_cuda(x)
    out = torch.empty_like(x)
    cols = x.shape[-1]
    _check(lib().vlab200_node_norm_bf16(_ptr(x), _ptr(out), C.c_int64(x.numel() // cols), C.c_int64(cols),
                                        C.c_float(eps), int(rms), _stream()), "vlab200_node_norm_bf16")
    return out


_LM_FIELDS = ["attn_norm_w", "attn_sub_norm_w", "ffn_norm_w", "ffn_sub_norm_w", "q_packed", "q_ws", "k_packed",
              "k_ws", "v_packed", "v_ws", "o_packed", "o_ws", "gate_up_packed", "gate_up_ws", "down_packed",
              "down_ws"]


class _BitvlaLmLayer(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in _LM_FIELDS]


class BitvlaLM:
    """BitVLA language-model stack (BitNet layers on the ternary kernels).

    Mirrors bitvla_lm_cuda_init / set_layer / set_output_norm / forward of the reference
    (src/kernels/bitvla/bitvla_lm_cuda.cu:314-393,668-725).  layers: list of dicts of cuda tensors with
    the vlab200_bitvla_lm_layer field names (norm weights bf16, packs uint8, scales float32)."""

    def __init__(self, hidden, n_q, n_kv, head_dim, ffn, layers, output_norm, rope_base=10000.0, rms_eps=1e-5,
                 max_seq=512, max_batch=1):
        import torch

        self.hidden = hidden
        self.h = lib().vlab200_bitvla_lm_init(hidden, n_q, n_kv, head_dim, ffn, len(layers), rope_base, rms_eps,
                                              max_seq, max_batch)
        if not self.h:
            raise VlaB200Error(ERR_CUDA, "vlab200_bitvla_lm_init")
        self._keep = [layers, output_norm]
        for i, lw in enumerate(layers):
            st = _BitvlaLmLayer()
            for n in _LM_FIELDS:
                t = lw[n]
                want = torch.float32 if n.endswith("_ws") else (torch.uint8 if n.endswith("_packed") else torch.bfloat16)
                assert t.is_cuda and t.is_contiguous() and t.dtype == want, n
                setattr(st, n, t.data_ptr())
            _check(lib().vlab200_bitvla_lm_set_layer(C.c_void_p(self.h), i, C.byref(st)), "vlab200_bitvla_lm_set_layer")
        assert output_norm.is_cuda and output_norm.dtype == torch.bfloat16
        _check(lib().vlab200_bitvla_lm_set_output_norm(C.c_void_p(self.h), _ptr(output_norm)),
               "vlab200_bitvla_lm_set_output_norm")

    def __del__(self):
        if getattr(self, "h", None):
            lib().vlab200_bitvla_lm_free(C.c_void_p(self.h))
            self.h = None

    @classmethod
    def from_gguf(cls, gguf, max_seq=512, max_batch=1):
        """The LM stack of a BitVLA checkpoint (ladder-int2 tensors with .scale sidecars); the context owns the weights."""
        self = cls.__new__(cls)
        self.h = lib().vlab200_bitvla_lm_create_from_gguf(gguf.h, max_seq, max_batch)
        if not self.h:
            raise VlaB200Error(ERR_ARG, "vlab200_bitvla_lm_create_from_gguf: " + lib().vlab200_last_error().decode())
        self.hidden = gguf.meta("bitvla.lm.hidden")
        self._keep = []
        return self

    def forward(self, x, out=None):
        """x: cuda bf16 [n_seq, seq, hidden] (or [seq, hidden]) -> same shape."""
        import torch

        assert x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous() and x.shape[-1] == self.hidden
        n_seq, seq = (1, x.shape[0]) if x.dim() == 2 else (x.shape[0], x.shape[1])
        out = torch.empty_like(x) if out is None else out
        _check(lib().vlab200_bitvla_lm_forward(C.c_void_p(self.h), _ptr(x), _ptr(out), seq, n_seq, _stream()),
               "vlab200_bitvla_lm_forward")
        return out
