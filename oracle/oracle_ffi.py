"""ctypes/numpy front end of the CPU oracle (oracle/liboracle.so).

Test infrastructure: imported by tests/, by the smoke check and by the benchmark's
CPU-baseline leg only.  The product package never imports this module.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def build(force=False):
    so = os.path.join(_HERE, "liboracle.so")
    src = os.path.join(_HERE, "vla_oracle.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "liboracle.so"], check=True, capture_output=True)
    return so


def lib():
    global _LIB
    if _LIB is None:
        _LIB = C.CDLL(build())
        _LIB.orc_num_threads.restype = C.c_int
    return _LIB


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


def num_threads():
    return int(lib().orc_num_threads())


def set_num_threads(n):
    lib().orc_set_num_threads(int(n))


def f32_to_bf16_bits(x):
    x = _c(x, np.float32)
    out = np.empty(x.shape, np.uint16)
    lib().orc_f32_to_bf16(_p(x), C.c_int64(x.size), _p(out))
    return out


def bf16_bits_to_f32(x):
    x = _c(x, np.uint16)
    out = np.empty(x.shape, np.float32)
    lib().orc_bf16_to_f32(_p(x), C.c_int64(x.size), _p(out))
    return out


def bf16_round(x):
    return bf16_bits_to_f32(f32_to_bf16_bits(x))


def ternarize(w):
    w = _c(w, np.float32)
    t = np.empty(w.shape, np.int8)
    am = C.c_float()
    lib().orc_ternarize(_p(w), C.c_int64(w.size), _p(t), C.byref(am))
    return t, np.float32(am.value)


def pack_ladder_int2(t):
    t = _c(t, np.int8)
    n, k = t.shape
    out = np.empty(n * k // 4, np.uint8)
    rc = lib().orc_pack_ladder_int2(_p(t), C.c_int64(n), C.c_int64(k), _p(out))
    if rc:
        raise ValueError("N must be a multiple of 16 and K of 128")
    return out


def unpack_ladder_int2(packed, n, k):
    packed = _c(packed, np.uint8)
    out = np.empty((n, k), np.int8)
    rc = lib().orc_unpack_ladder_int2(_p(packed), C.c_int64(n), C.c_int64(k), _p(out))
    if rc:
        raise ValueError("N must be a multiple of 16 and K of 128")
    return out


def act_quant(x):
    x = _c(x, np.float32)
    m, k = x.shape
    q = np.empty((m, k), np.int8)
    s = np.empty(m, np.float32)
    lib().orc_act_quant(_p(x), m, k, _p(q), _p(s))
    return q, s


def gemm_i8_i32(a, w):
    a, w = _c(a, np.int8), _c(w, np.int8)
    m, k = a.shape
    n = w.shape[0]
    acc = np.empty((m, n), np.int32)
    lib().orc_gemm_i8_i32(_p(a), _p(w), m, n, k, _p(acc))
    return acc


def gemm_i8_i32_rows(a, w, rows):
    a, w = _c(a, np.int8), _c(w, np.int8)
    rows = _c(rows, np.int32)
    k = a.shape[1]
    n = w.shape[0]
    acc = np.empty((rows.size, n), np.int32)
    lib().orc_gemm_i8_i32_rows(_p(a), _p(w), _p(rows), int(rows.size), n, k, _p(acc))
    return acc


def ternary_gemm_i32(a, packed, n):
    a = _c(a, np.int8)
    packed = _c(packed, np.uint8)
    m, k = a.shape
    acc = np.empty((m, n), np.int32)
    rc = lib().orc_ternary_gemm_i32(_p(a), _p(packed), m, n, k, _p(acc))
    if rc:
        raise ValueError("bad ternary gemm shape")
    return acc


def ternary_epilogue(acc, s, ws):
    acc = _c(acc, np.int32)
    s, ws = _c(s, np.float32), _c(ws, np.float32)
    m, n = acc.shape
    out = np.empty((m, n), np.uint16)
    lib().orc_ternary_epilogue(_p(acc), _p(s), _p(ws), int(ws.size), m, n, _p(out))
    return out


def linear(x, w, b=None):
    x, w = _c(x, np.float32), _c(w, np.float32)
    t, i = x.shape
    o = w.shape[0]
    y = np.empty((t, o), np.float32)
    bb = _c(b, np.float32) if b is not None else None
    lib().orc_linear(_p(x), _p(w), _p(bb) if bb is not None else None, t, i, o, _p(y))
    return y


def rmsnorm(x, w, eps):
    x = _c(x, np.float32)
    t, h = x.shape
    y = np.empty_like(x)
    ww = _c(w, np.float32) if w is not None else None
    lib().orc_rmsnorm(_p(x), _p(ww) if ww is not None else None, t, h, C.c_float(eps), _p(y))
    return y


def rope_neox(x, pos, base=10000.0):
    """x: [T][heads][hd]; returns a rotated copy."""
    x = _c(x, np.float32).copy()
    pos = _c(pos, np.int32)
    t, heads, hd = x.shape
    lib().orc_rope_neox(_p(x), _p(pos), t, heads, hd, C.c_float(base))
    return x


def rope_table(pos, hd, base=10000.0):
    pos = _c(pos, np.int32)
    cos_t = np.empty((pos.size, hd // 2), np.float32)
    sin_t = np.empty((pos.size, hd // 2), np.float32)
    lib().orc_rope_table(_p(pos), int(pos.size), hd, C.c_float(base), _p(cos_t), _p(sin_t))
    return cos_t, sin_t


def time_emb(t, dim, min_p, max_p):
    out = np.empty(dim, np.float32)
    lib().orc_time_emb(C.c_double(t), dim, C.c_double(min_p), C.c_double(max_p), _p(out))
    return out


MASK_NONE, MASK_PI0, MASK_SMOLVLA, MASK_PREFILL_STATE = 0, 1, 2, 3


def attention(q, k, v, p, mode, pad_start=0, pad_end=0):
    """q: [S][n_q][hd]; k, v: [Tkv][n_kv][hd] -> [S][n_q*hd]."""
    q, k, v = _c(q, np.float32), _c(k, np.float32), _c(v, np.float32)
    s, n_q, hd = q.shape
    tkv, n_kv, _ = k.shape
    out = np.empty((s, n_q * hd), np.float32)
    lib().orc_attention(_p(q), _p(k), _p(v), s, tkv, n_q, n_kv, hd, p, mode, pad_start, pad_end, _p(out))
    return out


def qkv_rope(x, ln_w, wqkv, pos, n_q, n_kv, hd, eps, rope_base=10000.0, act_bf16=False):
    x, ln_w, wqkv = _c(x, np.float32), _c(ln_w, np.float32), _c(wqkv, np.float32)
    pos = _c(pos, np.int32)
    s, h = x.shape
    q = np.empty((s, n_q, hd), np.float32)
    k = np.empty((s, n_kv, hd), np.float32)
    v = np.empty((s, n_kv, hd), np.float32)
    lib().orc_qkv_rope(_p(x), _p(ln_w), _p(wqkv), _p(pos), s, h, n_q, n_kv, hd, C.c_float(eps),
                       C.c_float(rope_base), int(act_bf16), _p(q), _p(k), _p(v))
    return q, k, v


def vlm_prefill(x, layers, cfg, pos=None, mask_mode=MASK_NONE, pad=(0, 0)):
    """The backbone's layers over the prefix embeddings x [P][hidden] (float32); returns per layer the rotated K and
    the V, each [P][n_kv][hd], that the denoise loop caches.  Layer body: src/models/smolvla.cpp:778-813
    (build_vlm_layer, SiLU) and src/models/pi0.cpp:159-233 (build_gemma_layer, tanh-GELU); loops
    smolvla.cpp:1374-1379, pi0.cpp:557-566.  layers: list of dicts ln_in, wqkv [(n_q+2n_kv)hd][H] (q, k, v rows),
    wo, ln_post, wgate, wup, wdown.  cfg: n_q, n_kv, hd, rms_eps, rope_base, act ("silu" | "gelu")."""
    h = _c(x, np.float32).copy()
    P = h.shape[0]
    pos = np.arange(P, dtype=np.int32) if pos is None else _c(pos, np.int32)
    ks, vs = [], []
    for li, lw in enumerate(layers):
        q, k, v = qkv_rope(h, lw["ln_in"], lw["wqkv"], pos, cfg["n_q"], cfg["n_kv"], cfg["hd"], cfg["rms_eps"],
                           cfg["rope_base"])
        ks.append(k)
        vs.append(v)
        if li + 1 == len(layers):
            break
        att = attention(q, k, v, 0, mask_mode, pad[0], pad[1])
        h = h + linear(att, lw["wo"])
        xm = rmsnorm(h, lw["ln_post"], cfg["rms_eps"])
        gate, up = linear(xm, lw["wgate"]), linear(xm, lw["wup"])
        if cfg["act"] == "silu":
            act = gate / (np.float32(1) + np.exp(-gate, dtype=np.float32))
        else:
            c0 = np.float32(0.79788456080286535588)
            act = np.float32(0.5) * gate * (np.float32(1) + np.tanh(c0 * (gate + np.float32(0.044715) * gate * gate * gate),
                                                                     dtype=np.float32))
        h = h + linear((act * up).astype(np.float32), lw["wdown"])
    return ks, vs


# ---- vision tower (numpy float32): SigLIP encoder + connector ----

def pi05_denoise(kp, vp, x0, w, cfg):
    """The pi0.5 Euler loop for one observation (src/models/pi05.cpp:604-631; layer build_expert_layer :226-292;
    build_adarms :208-224): time enters through adaptive RMSNorm, residuals are gated, the action tokens see the prefix
    and one another without a mask.  kp, vp: per layer the prefix's rotated K and its V [P][n_kv][hd]; x0 [chunk][A].
    w: w_ain, b_ain, w_tin, b_tin, w_tout, b_tout, ada_final_w, ada_final_b, w_aout, b_aout and layers = dicts wq, wk, wv,
    wo, wgate, wup, wdown, ada_in_w, ada_in_b, ada_post_w, ada_post_b.  cfg: H, n_q, n_kv, hd, steps, rms_eps, rope_base,
    min_period, max_period."""
    H, n_q, n_kv, hd, T = cfg["H"], cfg["n_q"], cfg["n_kv"], cfg["hd"], cfg["steps"]
    silu = lambda a: a / (np.float32(1) + np.exp(-a, dtype=np.float32))
    x = _c(x0, np.float32).copy()
    S, P = x.shape[0], kp[0].shape[0]
    pos = np.arange(P, P + S, dtype=np.int32)
    dt = np.float32(-1.0) / np.float32(T)

    def adarms(h, dense_w, dense_b, cond):
        mod = linear(cond, dense_w, dense_b)[0]
        n = rmsnorm(h, None, cfg["rms_eps"])
        return (n + n * mod[None, :H] + mod[None, H:2 * H]).astype(np.float32), mod[2 * H:]

    for s in range(T):
        t = np.float32(1.0) + np.float32(s) * dt
        tau = time_emb(float(t), H, cfg["min_period"], cfg["max_period"])[None, :]
        cond = silu(linear(silu(linear(tau, w["w_tin"], w["b_tin"])), w["w_tout"], w["b_tout"]))
        h = linear(x, w["w_ain"], w["b_ain"])
        for l, lw in enumerate(w["layers"]):
            xn, gate = adarms(h, lw["ada_in_w"], lw["ada_in_b"], cond)
            q = rope_neox(linear(xn, lw["wq"]).reshape(S, n_q, hd), pos, cfg["rope_base"])
            k = rope_neox(linear(xn, lw["wk"]).reshape(S, n_kv, hd), pos, cfg["rope_base"])
            v = linear(xn, lw["wv"]).reshape(S, n_kv, hd)
            att = attention(q, np.concatenate([kp[l], k]), np.concatenate([vp[l], v]), P, MASK_NONE)
            h = h + linear(att, lw["wo"]) * gate[None, :]
            xn, gate = adarms(h, lw["ada_post_w"], lw["ada_post_b"], cond)
            inter = gelu_tanh(linear(xn, lw["wgate"])) * linear(xn, lw["wup"])
            h = h + linear(inter.astype(np.float32), lw["wdown"]) * gate[None, :]
        xf, _ = adarms(h, w["ada_final_w"], w["ada_final_b"], cond)
        x = x + dt * linear(xf, w["w_aout"], w["b_aout"])
    return x


def preprocess_image_chw(img):
    """img: [side][side][3] uint8 (0..255) or float32 (0..1), H W C -> float32 [3][side][side] in [-1, 1]
    (src/modules/preprocess.h:56-75: px = u8 / 255.0f, out = px * 2 - 1)."""
    img = np.asarray(img)
    px = img.astype(np.float32) / np.float32(255.0) if img.dtype == np.uint8 else img.astype(np.float32)
    return np.ascontiguousarray((px * np.float32(2.0) - np.float32(1.0)).transpose(2, 0, 1))


def pixel_shuffle_hf(src, grid, s):
    """src: [grid * grid][embed] -> [(grid / s)^2][embed * s * s], channel innermost
    (src/modules/preprocess.h:37-52): token (h2, w2) column block hs * s + ws <- patch (h2 s + hs, w2 s + ws)."""
    src = np.asarray(src, np.float32)
    embed = src.shape[1]
    g2 = grid // s
    x = src.reshape(g2, s, g2, s, embed).transpose(0, 2, 1, 3, 4)  # [h2][w2][hs][ws][e]
    return np.ascontiguousarray(x.reshape(g2 * g2, s * s * embed))


def layer_norm(x, w, b, eps):
    """ggml_norm followed by weight and bias (src/models/smolvla.cpp:397): mean, variance of the centred values."""
    x = np.asarray(x, np.float32)
    mean = x.mean(axis=1, dtype=np.float32, keepdims=True)
    d = x - mean
    var = (d * d).mean(axis=1, dtype=np.float32, keepdims=True)
    return (d * (np.float32(1) / np.sqrt(var + np.float32(eps))) * w + b).astype(np.float32)


def gelu_tanh(x):
    c0 = np.float32(0.79788456080286535588)
    return np.float32(0.5) * x * (np.float32(1) + np.tanh(c0 * (x + np.float32(0.044715) * x * x * x), dtype=np.float32))


def siglip_tower(img, w, cfg):
    """One camera view -> its image-token embeddings [n_tokens][out_dim].

    Patch embedding (a stride-P convolution = a linear map over flattened patches), position embedding, encoder
    blocks, post-LayerNorm: src/models/smolvla.cpp:1511-1524 with the block of :394-426; pixel shuffle and the
    bias-free connector :1533-1563; pi0's variant (src/models/pi0.cpp:479-499) has no shuffle, an optional
    connector bias and scales the result by 1/sqrt(out_dim).
    w: patch_w [hidden][3][P][P], patch_b, pos [n_patches][hidden], layers (list of dicts ln1_w, ln1_b, wq, bq, wk,
    bk, wv, bv, wo, bo, ln2_w, ln2_b, fc1, b1, fc2, b2), post_w, post_b, connector, connector_b (or None).
    cfg: image, patch, hidden, n_heads, shuffle, ln_eps, out_scale."""
    P, side, H, heads = cfg["patch"], cfg["image"], cfg["hidden"], cfg["n_heads"]
    g = side // P
    hd = H // heads
    chw = preprocess_image_chw(img)
    patches = chw.reshape(3, g, P, g, P).transpose(1, 3, 0, 2, 4).reshape(g * g, 3 * P * P)
    h = linear(patches, np.asarray(w["patch_w"], np.float32).reshape(H, -1), w["patch_b"]) + w["pos"]
    n = g * g
    for lw in w["layers"]:
        n1 = layer_norm(h, lw["ln1_w"], lw["ln1_b"], cfg["ln_eps"])
        q = linear(n1, lw["wq"], lw["bq"]).reshape(n, heads, hd)
        k = linear(n1, lw["wk"], lw["bk"]).reshape(n, heads, hd)
        v = linear(n1, lw["wv"], lw["bv"]).reshape(n, heads, hd)
        att = attention(q, k, v, 0, MASK_NONE)
        h = h + linear(att, lw["wo"], lw["bo"])
        n2 = layer_norm(h, lw["ln2_w"], lw["ln2_b"], cfg["ln_eps"])
        h = h + linear(gelu_tanh(linear(n2, lw["fc1"], lw["b1"])), lw["fc2"], lw["b2"])
    post = layer_norm(h, w["post_w"], w["post_b"], cfg["ln_eps"])
    s = cfg.get("shuffle", 1)
    if s > 1:
        post = pixel_shuffle_hf(post, g, s)
    out = linear(post, w["connector"], w.get("connector_b"))
    sc = cfg.get("out_scale", 0.0)
    return out * np.float32(sc) if sc not in (0.0, 1.0) else out


class DenoiseCfg(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "model", "n_layers", "H", "n_q", "n_kv", "hd", "inter", "P", "chunk", "A", "state_dim", "T",
        "pos_base", "pad_start", "pad_end", "self_every", "act_bf16")] + [
        ("rms_eps", C.c_float), ("rope_base", C.c_float), ("min_period", C.c_double), ("max_period", C.c_double)]


class DenoiseWeights(C.Structure):
    _fields_ = [(n, C.POINTER(C.c_void_p)) for n in (
        "ln_in", "Wqkv", "Wo", "ln_post", "Wgate", "Wup", "Wdown")] + [
        (n, C.c_void_p) for n in ("W_sp", "b_sp", "W_ain", "b_ain", "W_at1", "b_at1", "W_at2", "b_at2",
                                   "out_norm", "W_aout", "b_aout")]


def _ptr_array(arrs):
    keep = [_c(a, np.float32) for a in arrs]
    arr = (C.c_void_p * len(keep))(*[a.ctypes.data for a in keep])
    return arr, keep


class DenoiseModel:
    """Holds float32 weights (dict of numpy arrays / lists per layer) for orc_denoise_loop."""

    def __init__(self, cfg: dict, weights: dict):
        self.cfg = DenoiseCfg(**cfg)
        self._keep = []
        w = DenoiseWeights()
        for name in ("ln_in", "Wqkv", "Wo", "ln_post", "Wgate", "Wup", "Wdown"):
            arr, keep = _ptr_array(weights[name])
            self._keep += [arr, keep]
            setattr(w, name, C.cast(arr, C.POINTER(C.c_void_p)))
        for name in ("W_sp", "b_sp", "W_ain", "b_ain", "W_at1", "b_at1", "W_at2", "b_at2", "out_norm",
                     "W_aout", "b_aout"):
            a = weights.get(name)
            if a is None:
                setattr(w, name, None)
            else:
                a = _c(a, np.float32)
                self._keep.append(a)
                setattr(w, name, a.ctypes.data)
        self.w = w

    def denoise(self, kp, vp, state, x0):
        """kp, vp: lists (n_layers) of [P][n_kv][hd]; state [state_dim]; x0 [chunk][A]."""
        ka, kk = _ptr_array(kp)
        va, vk = _ptr_array(vp)
        x0 = _c(x0, np.float32)
        st = _c(state if state is not None else np.zeros(self.cfg.state_dim), np.float32)
        out = np.empty_like(x0)
        rc = lib().orc_denoise_loop(C.byref(self.cfg), C.byref(self.w), ka, va, _p(st), _p(x0), _p(out))
        assert rc == 0
        return out

    def expert_layer(self, l, h, kp, vp, is_self=True):
        h = _c(h, np.float32).copy()
        kp, vp = _c(kp, np.float32), _c(vp, np.float32)
        lib().orc_expert_layer(C.byref(self.cfg), C.byref(self.w), l, _p(h), h.shape[0], _p(kp), _p(vp),
                               int(is_self))
        return h


# --------------------------------------------------------------- BitVLA LM layer --
# Composite restatement of run_layer (src/kernels/bitvla/bitvla_lm_cuda.cu:395-525) and
# bitvla_lm_cuda_forward (:668-725) from the pinned pieces above (act-quant, ladder GEMM,
# epilogue) plus numpy for the bf16 element-wise kernels.  PARITY UNPINNED as a whole: the
# reference holds no golden vector for a layer and its CUDA build cannot run here.

def bitvla_rmsnorm_bf16(x, w, eps):
    """rmsnorm_bf16_kernel (bitvla_lm_cuda.cu:37-75): bf16(x * rsqrt(mean x^2 + eps) * w)."""
    x = _c(x, np.float32)
    ss = (x.astype(np.float64) ** 2).sum(-1)
    scale = (1.0 / np.sqrt(ss / x.shape[-1] + eps)).astype(np.float32)
    return bf16_round((x * scale[:, None]) * _c(w, np.float32)[None, :])


def bitvla_linear(xn, packed, ws, n):
    """act-quant -> ternary GEMM -> bf16 epilogue (bitvla_lm_cuda.cu:427-436)."""
    q, s = act_quant(xn)
    acc = ternary_gemm_i32(q, packed, n)
    return bf16_bits_to_f32(ternary_epilogue(acc, s, np.atleast_1d(ws)))


def bitvla_rope_table(seq, hd, base):
    """Host loop of bitvla_lm_cuda_init (bitvla_lm_cuda.cu:333-342), float arithmetic."""
    half = hd // 2
    k = np.arange(half, dtype=np.float32)
    freq = (np.float32(1.0) / np.power(np.float32(base), (2 * k) / np.float32(hd))).astype(np.float32)
    ang = (np.arange(seq, dtype=np.float32)[:, None] * freq[None, :]).astype(np.float32)
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)


def bitvla_lm_layer(h, lw, cfg, cos, sin):
    """h: [seq, hidden] bf16-valued float32 -> same.  lw: dict with the reference's
    bitvla_lm_layer_cuda fields (norms bf16-valued float32, packs uint8, scales float32)."""
    n_q, n_kv, hd, ffn, eps = cfg["n_q"], cfg["n_kv"], cfg["head_dim"], cfg["ffn"], cfg["rms_eps"]
    seq, hidden = h.shape
    hq, hkv, half = n_q * hd, n_kv * hd, hd // 2
    hn = bitvla_rmsnorm_bf16(h, lw["attn_norm_w"], eps)
    q = bitvla_linear(hn, lw["q_packed"], lw["q_ws"], hq).reshape(seq, n_q, hd).transpose(1, 0, 2)
    k = bitvla_linear(hn, lw["k_packed"], lw["k_ws"], hkv).reshape(seq, n_kv, hd).transpose(1, 0, 2)
    v = bitvla_linear(hn, lw["v_packed"], lw["v_ws"], hkv).reshape(seq, n_kv, hd).transpose(1, 0, 2)

    def rope(t):  # rope_neox_bf16_kernel (bitvla_lm_cuda.cu:77-99)
        a, b = t[..., :half], t[..., half:]
        c, s = cos[None, :seq], sin[None, :seq]
        return bf16_round(np.concatenate([a * c - b * s, b * c + a * s], -1).astype(np.float32))

    q, k = rope(q), rope(k)
    att = np.empty((seq, n_q, hd), np.float32)
    scl = np.float32(1.0 / np.sqrt(np.float32(hd)))
    for qh in range(n_q):
        kvh = qh * n_kv // n_q  # repeat_kv_bf16_kernel (bitvla_lm_cuda.cu:181-190)
        sc = bf16_round((q[qh] @ k[kvh].T).astype(np.float32))  # scores stored bf16 (:452-463)
        x = sc * scl  # softmax_scaled_bf16_kernel (:101-157)
        p = np.exp(x - x.max(-1, keepdims=True)).astype(np.float32)
        p = bf16_round(p * (np.float32(1.0) / p.sum(-1, keepdims=True, dtype=np.float32)))
        att[:, qh] = bf16_round((p @ v[kvh]).astype(np.float32))
    an = bitvla_rmsnorm_bf16(att.reshape(seq, hq), lw["attn_sub_norm_w"], eps)
    h = bf16_round(h + bitvla_linear(an, lw["o_packed"], lw["o_ws"], hidden))
    hn = bitvla_rmsnorm_bf16(h, lw["ffn_norm_w"], eps)
    gu = bitvla_linear(hn, lw["gate_up_packed"], lw["gate_up_ws"], 2 * ffn)
    g, u = np.maximum(gu[:, :ffn], 0), gu[:, ffn:]
    t = bf16_round((g * g * u).astype(np.float32))  # gate_up_fused_sqrelu_mul_bf16_kernel (:527-542)
    tn = bitvla_rmsnorm_bf16(t, lw["ffn_sub_norm_w"], eps)
    return bf16_round(h + bitvla_linear(tn, lw["down_packed"], lw["down_ws"], hidden))


def bitvla_lm_forward(x, layers, output_norm, cfg):
    """bitvla_lm_cuda_forward (bitvla_lm_cuda.cu:668-725) for one sequence x [seq, hidden]."""
    cos, sin = bitvla_rope_table(x.shape[0], cfg["head_dim"], cfg["rope_base"])
    h = bf16_round(x)
    for lw in layers:
        h = bitvla_lm_layer(h, lw, cfg, cos, sin)
    return bitvla_rmsnorm_bf16(h, output_norm, cfg["rms_eps"])


def bitvla_layernorm_bf16(x, w, b, eps):
    """layernorm_bias_bf16_kernel (bitvla_lm_cuda.cu:552-607): mean and centred variance of the bf16 row in float,
    bf16((x - mean) * rsqrt(var + eps) * w + b)."""
    x = _c(x, np.float32)
    mean = (x.astype(np.float64).sum(-1) / x.shape[-1]).astype(np.float32)
    d = x - mean[:, None]
    var = ((d.astype(np.float64) ** 2).sum(-1) / x.shape[-1]).astype(np.float32)
    inv = (np.float32(1.0) / np.sqrt(var + np.float32(eps))).astype(np.float32)
    return bf16_round((d * inv[:, None]) * _c(w, np.float32)[None, :] + _c(b, np.float32)[None, :])


def bitvla_vit_forward(patches, w, cfg):
    """bitvla_vit_cuda_forward (src/kernels/bitvla/bitvla_vit_cuda.cu:261-330, layer body :161-259) for one image.
    patches [n_patches, patch_flat]; w: patch_w [hidden, patch_flat], patch_b, pos [n_patches, hidden], mm_w1, mm_b1, mm_w2,
    mm_b2 and layers = dicts ln1_w, ln1_b, ln2_w, ln2_b, {q,k,v,o,fc1,fc2}_packed / _ws / _b (fc2 packed over the MLP
    width padded to a multiple of 128); every array bf16-valued float32 but the packs (uint8) and scales.
    cfg: hidden, n_heads, ffn, ln_eps.  Every value the reference stores as bf16 is rounded here."""
    import math

    H, heads, ffn, eps = cfg["hidden"], cfg["n_heads"], cfg["ffn"], cfg["ln_eps"]
    hd, ffn_pad = H // heads, (ffn + 127) // 128 * 128
    r = bf16_round
    x = r(_c(patches, np.float32))
    h = r(linear(x, w["patch_w"]))
    h = r(r(h + w["patch_b"][None, :]) + w["pos"])
    seq = h.shape[0]
    scl = np.float32(1.0 / np.sqrt(np.float32(hd)))
    for lw in w["layers"]:
        n1 = bitvla_layernorm_bf16(h, lw["ln1_w"], lw["ln1_b"], eps)
        a, s = act_quant(n1)

        def proj(name, q=a, sc=s, n=H):
            acc = ternary_gemm_i32(q, lw[name + "_packed"], n)
            y = bf16_bits_to_f32(ternary_epilogue(acc, sc, np.atleast_1d(lw[name + "_ws"])))
            return r(y + lw[name + "_b"][None, :])

        q = proj("q").reshape(seq, heads, hd).transpose(1, 0, 2)
        k = proj("k").reshape(seq, heads, hd).transpose(1, 0, 2)
        v = proj("v").reshape(seq, heads, hd).transpose(1, 0, 2)
        att = np.empty((seq, heads, hd), np.float32)
        for hh in range(heads):
            sc = r((q[hh] @ k[hh].T).astype(np.float32))  # scores stored bf16 (:198-209)
            xs = sc * scl
            p = np.exp(xs - xs.max(-1, keepdims=True)).astype(np.float32)
            p = r(p * (np.float32(1.0) / p.sum(-1, keepdims=True, dtype=np.float32)))
            att[:, hh] = r((p @ v[hh]).astype(np.float32))
        a2, s2 = act_quant(att.reshape(seq, H))
        h = r(h + proj("o", a2, s2))
        n2 = bitvla_layernorm_bf16(h, lw["ln2_w"], lw["ln2_b"], eps)
        a3, s3 = act_quant(n2)
        f1 = proj("fc1", a3, s3, ffn)
        c0 = np.float32(0.7978845608028654)
        g = r(np.float32(0.5) * f1 * (np.float32(1) + np.tanh(c0 * (f1 + np.float32(0.044715) * f1 * f1 * f1), dtype=np.float32)))
        gp = np.zeros((seq, ffn_pad), np.float32)
        gp[:, :ffn] = g
        a4, s4 = act_quant(gp)
        h = r(h + proj("fc2", a4, s4))
    erf = np.vectorize(math.erf, otypes=[np.float64])
    m1 = r(r(linear(h, w["mm_w1"])) + w["mm_b1"][None, :])
    m1 = r(np.float32(0.5) * m1 * (np.float32(1) + erf(m1 * np.float32(0.7071067811865475)).astype(np.float32)))
    return r(r(linear(m1, w["mm_w2"])) + w["mm_b2"][None, :])


def bitvla_fp32head(w, cfg, state=None, ah_in=None):
    """The float32 proprioception projector and action head (src/kernels/bitvla/bitvla_fp32head_cuda.cu:258-358) in
    float64 numpy: proprio = W2 gelu_erf(W1 state + b1) + b2; action = fc2(LN2(h)), h = relu(fc1(LN1(in))) followed by
    two blocks h += relu(W LN(h) + b).  w: dict with the names of bitvla_fp32head_cuda_init's arguments."""
    import math

    f = lambda k: np.asarray(w[k], np.float64)
    erf = np.vectorize(math.erf, otypes=[np.float64])

    def ln(x, wk, bk):
        m = x.mean(-1, keepdims=True)
        d = x - m
        return d / np.sqrt((d * d).mean(-1, keepdims=True) + cfg["ah_ln_eps"]) * f(wk) + f(bk)

    out = {}
    if state is not None:
        h1 = f("pp_fc1_w") @ np.asarray(state, np.float64) + f("pp_fc1_b")
        h1 = 0.5 * h1 * (1.0 + erf(h1 * 0.70710678118654752440))
        out["proprio"] = f("pp_fc2_w") @ h1 + f("pp_fc2_b")
    if ah_in is not None:
        x = ln(np.asarray(ah_in, np.float64), "ah_ln1_w", "ah_ln1_b")
        h = np.maximum(x @ f("ah_fc1_w").T + f("ah_fc1_b"), 0)
        for blk in ("b0", "b1"):
            h = h + np.maximum(ln(h, f"ah_{blk}_lnw", f"ah_{blk}_lnb") @ f(f"ah_{blk}_w").T + f(f"ah_{blk}_b"), 0)
        out["action"] = ln(h, "ah_ln2_w", "ah_ln2_b") @ f("ah_fc2_w").T + f("ah_fc2_b")
    return out


# ---- node-level bf16 operators (the reference's per-node CUDA hook, src/cuda/vla_cuda_bf16.cu) ----
# Inputs are float32 arrays holding bf16 values; float32 math; one bf16 rounding of the result.

def node_unary(op, x):
    """op: "silu" | "relu" | "gelu" (tanh form) | "gelu_erf" (src/cuda/vla_cuda_bf16.cu:463-474)."""
    import math

    x = np.asarray(x, dtype=np.float32)
    if op == "silu":
        y = x / (np.float32(1) + np.exp(-x, dtype=np.float32))
    elif op == "relu":
        y = np.maximum(x, np.float32(0))
    elif op == "gelu_erf":
        erf = np.vectorize(math.erf, otypes=[np.float64])
        y = np.float32(0.5) * x * (np.float32(1) + erf(x * np.float32(0.70710678118654752440)).astype(np.float32))
    else:
        c = np.float32(0.79788456080286535588)
        y = np.float32(0.5) * x * (np.float32(1) + np.tanh(c * (x + np.float32(0.044715) * x * x * x), dtype=np.float32))
    return bf16_round(y.astype(np.float32))


def node_scale(x, scale, bias):
    """scale * x + bias (src/cuda/vla_cuda_bf16.cu:501-527); the product and the sum round separately in
    float32 unless the compiler contracts them, so the test allows one bf16 ulp."""
    x = np.asarray(x, dtype=np.float32)
    return bf16_round((np.float32(scale) * x + np.float32(bias)).astype(np.float32))


def node_bin(op, a, b):
    """a (+|*) b with b broadcast along the leading dimensions (src/cuda/vla_cuda_bf16.cu:396-452)."""
    a = np.asarray(a, dtype=np.float32)
    b = np.asarray(b, dtype=np.float32)
    return bf16_round((a * b if op == "mul" else a + b).astype(np.float32))


def node_norm(x, eps, rms):
    """Row norm without weight: x * rsqrt(mean x^2 + eps), or (x - mean) * rsqrt(var + eps)
    (src/cuda/vla_cuda_bf16.cu:548-579)."""
    x = np.asarray(x, dtype=np.float32)
    x64 = x.astype(np.float64)
    if rms:
        inv = 1.0 / np.sqrt((x64 * x64).mean(-1, keepdims=True) + eps)
        return bf16_round((x64 * inv).astype(np.float32))
    mean = x64.mean(-1, keepdims=True)
    var = (x64 * x64).mean(-1, keepdims=True) - mean * mean
    return bf16_round(((x64 - mean) / np.sqrt(var + eps)).astype(np.float32))


def node_mul_mat(w, x):
    """out[b][m][n] = sum_k x[b][m][k] * w[(b)][n][k], bf16 operands, float32 accumulation, bf16 result
    (src/cuda/vla_cuda_bf16.cu:624-678).  w: [N, K] shared by all batches or [B, N, K]."""
    x = np.asarray(x, dtype=np.float32)
    w = np.asarray(w, dtype=np.float32)
    if x.ndim == 2:
        return bf16_round(linear(x, w))
    return np.stack([bf16_round(linear(x[b], w[b] if w.ndim == 3 else w)) for b in range(x.shape[0])])
