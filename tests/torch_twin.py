"""Independent float32 torch restatement of the dense part of the denoise step,
written from the mathematics (not from the C oracle) so the two can check each
other.  CPU only; used by tests."""
import math

import torch


def rmsnorm(x, w, eps):
    return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * w


def rope_neox(x, pos, base=10000.0):
    # x: [T, heads, hd]
    hd = x.shape[-1]
    half = hd // 2
    inv = base ** (-2.0 * torch.arange(half, dtype=torch.float32) / hd)
    ang = pos.to(torch.float32)[:, None] * inv[None, :]
    c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
    a, b = x[..., :half], x[..., half:]
    return torch.cat([a * c - b * s, b * c + a * s], -1)


def mask(mode, P, S, Tkv, pad_start=0, pad_end=0):
    m = torch.zeros(S, Tkv)
    cols = torch.arange(Tkv)
    m[:, (cols < P) & (cols >= pad_start) & (cols < pad_end)] = -math.inf
    for r in range(S):
        for c in range(P, Tkv):
            sc = c - P
            vis = True
            if mode == 1:
                vis = (sc == 0) if r == 0 else True
            elif mode == 2:
                vis = sc <= r
            if not vis:
                m[r, c] = -math.inf
    return m


def attention(q, k, v, m):
    # q [S, n_q, hd], k/v [Tkv, n_kv, hd]
    S, n_q, hd = q.shape
    n_kv = k.shape[1]
    g = n_q // n_kv
    kk = k.repeat_interleave(g, dim=1)
    vv = v.repeat_interleave(g, dim=1)
    sc = torch.einsum("shd,thd->hst", q, kk) / math.sqrt(hd) + m[None]
    p = torch.softmax(sc, -1)
    return torch.einsum("hst,thd->shd", p, vv).reshape(S, n_q * hd)


def gelu_tanh(x):
    return torch.nn.functional.gelu(x, approximate="tanh")


def expert_layer_self(h, W, kp, vp, cfg, pos, m):
    n_q, n_kv, hd = cfg["n_q"], cfg["n_kv"], cfg["hd"]
    S = h.shape[0]
    xn = rmsnorm(h, W["ln_in"], cfg["rms_eps"])
    qkv = xn @ W["Wqkv"].T
    q = qkv[:, : n_q * hd].reshape(S, n_q, hd)
    k = qkv[:, n_q * hd : (n_q + n_kv) * hd].reshape(S, n_kv, hd)
    v = qkv[:, (n_q + n_kv) * hd :].reshape(S, n_kv, hd)
    q, k = rope_neox(q, pos), rope_neox(k, pos)
    att = attention(q, torch.cat([kp, k]), torch.cat([vp, v]), m)
    h1 = h + att @ W["Wo"].T
    xm = rmsnorm(h1, W["ln_post"], cfg["rms_eps"])
    act = gelu_tanh if cfg["model"] == 0 else torch.nn.functional.silu
    return h1 + (act(xm @ W["Wgate"].T) * (xm @ W["Wup"].T)) @ W["Wdown"].T


def time_emb(t, dim, mn, mx):
    half = dim // 2
    frac = torch.arange(half, dtype=torch.float64) / max(half - 1, 1)
    period = mn * (mx / mn) ** frac
    s = 2.0 * math.pi / period * t
    return torch.cat([s.sin(), s.cos()]).to(torch.float32)


def denoise_pi0(cfg, W, layers, kp, vp, state, x0):
    P, chunk, T, H = cfg["P"], cfg["chunk"], cfg["T"], cfg["H"]
    S = chunk + 1
    pos = torch.arange(P, P + S)
    m = mask(1, P, S, P + S)
    x = x0.clone()
    dt = torch.tensor(-1.0 / T, dtype=torch.float32)
    for step in range(T):
        t = float(torch.tensor(1.0, dtype=torch.float32) + torch.tensor(float(step)) * dt)
        te = time_emb(t, H, cfg["min_period"], cfg["max_period"])
        a = x @ W["W_ain"].T + W["b_ain"]
        a = torch.cat([a, te[None].expand(chunk, H)], -1)
        u = torch.nn.functional.silu(a @ W["W_at1"].T + W["b_at1"]) @ W["W_at2"].T + W["b_at2"]
        s = (state @ W["W_sp"].T + W["b_sp"])[None]
        h = torch.cat([s, u])
        for l, Wl in enumerate(layers):
            h = expert_layer_self(h, Wl, kp[l], vp[l], cfg, pos, m)
        hn = rmsnorm(h, W["out_norm"], cfg["rms_eps"])
        v = hn[1:] @ W["W_aout"].T + W["b_aout"]
        x = x + dt * v
    return x
