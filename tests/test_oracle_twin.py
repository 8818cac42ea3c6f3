"""The dense part of the oracle has no stored reference outputs (the reference
runs it through ggml, absent here), so it is cross-checked against an independent
torch-fp32 restatement of the same mathematics."""
import numpy as np
import torch

from tests import torch_twin as tw


def _rand(rng, *shape, scale=1.0):
    return (rng.standard_normal(shape) * scale).astype(np.float32)


def test_attention_all_mask_modes(oracle):
    rng = np.random.default_rng(1)
    S, P, n_q, n_kv, hd = 7, 11, 6, 2, 16
    q, k, v = _rand(rng, S, n_q, hd), _rand(rng, P + S, n_kv, hd), _rand(rng, P + S, n_kv, hd)
    for mode, ps, pe in [(0, 0, 0), (1, 0, 0), (2, 0, 0), (2, 4, 9)]:
        got = oracle.attention(q, k, v, P, mode, ps, pe)
        ref = tw.attention(torch.from_numpy(q), torch.from_numpy(k), torch.from_numpy(v),
                           tw.mask(mode, P, S, P + S, ps, pe)).numpy()
        np.testing.assert_allclose(got, ref, rtol=1e-4, atol=1e-5)


def test_qkv_rope(oracle):
    rng = np.random.default_rng(2)
    S, H, n_q, n_kv, hd = 5, 48, 6, 2, 16
    x, ln = _rand(rng, S, H), 1 + _rand(rng, H, scale=0.1)
    w = _rand(rng, (n_q + 2 * n_kv) * hd, H, scale=0.05)
    pos = np.arange(100, 100 + S).astype(np.int32)
    q, k, v = oracle.qkv_rope(x, ln, w, pos, n_q, n_kv, hd, 1e-6)
    xn = tw.rmsnorm(torch.from_numpy(x), torch.from_numpy(ln), 1e-6)
    qkv = xn @ torch.from_numpy(w).T
    tq = tw.rope_neox(qkv[:, : n_q * hd].reshape(S, n_q, hd), torch.from_numpy(pos))
    tk = tw.rope_neox(qkv[:, n_q * hd:(n_q + n_kv) * hd].reshape(S, n_kv, hd), torch.from_numpy(pos))
    np.testing.assert_allclose(q, tq.numpy(), rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(k, tk.numpy(), rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(v.reshape(S, -1), qkv[:, (n_q + n_kv) * hd:].numpy(), rtol=1e-4, atol=1e-5)


def small_pi0(rng, L=2):
    cfg = dict(model=0, n_layers=L, H=32, n_q=4, n_kv=1, hd=16, inter=64, P=9, chunk=5, A=8, state_dim=8, T=3,
               pos_base=9, pad_start=0, pad_end=0, self_every=1, act_bf16=0, rms_eps=1e-6, rope_base=10000.0,
               min_period=4e-3, max_period=4.0)
    H, A, I = cfg["H"], cfg["A"], cfg["inter"]
    qf, kvf = cfg["n_q"] * cfg["hd"], cfg["n_kv"] * cfg["hd"]
    per = dict(ln_in=[], Wqkv=[], Wo=[], ln_post=[], Wgate=[], Wup=[], Wdown=[])
    for _ in range(L):
        per["ln_in"].append(1 + _rand(rng, H, scale=0.1))
        per["Wqkv"].append(_rand(rng, qf + 2 * kvf, H, scale=0.2))
        per["Wo"].append(_rand(rng, H, qf, scale=0.2))
        per["ln_post"].append(1 + _rand(rng, H, scale=0.1))
        per["Wgate"].append(_rand(rng, I, H, scale=0.2))
        per["Wup"].append(_rand(rng, I, H, scale=0.2))
        per["Wdown"].append(_rand(rng, H, I, scale=0.2))
    glob = dict(W_sp=_rand(rng, H, 8, scale=0.2), b_sp=_rand(rng, H, scale=0.1),
                W_ain=_rand(rng, H, A, scale=0.2), b_ain=_rand(rng, H, scale=0.1),
                W_at1=_rand(rng, H, 2 * H, scale=0.2), b_at1=_rand(rng, H, scale=0.1),
                W_at2=_rand(rng, H, H, scale=0.2), b_at2=_rand(rng, H, scale=0.1),
                out_norm=1 + _rand(rng, H, scale=0.1), W_aout=_rand(rng, A, H, scale=0.2),
                b_aout=_rand(rng, A, scale=0.1))
    return cfg, per, glob


def test_pi0_denoise_loop(oracle):
    rng = np.random.default_rng(3)
    cfg, per, glob = small_pi0(rng)
    L, P = cfg["n_layers"], cfg["P"]
    kp = [_rand(rng, P, cfg["n_kv"], cfg["hd"]) for _ in range(L)]
    vp = [_rand(rng, P, cfg["n_kv"], cfg["hd"]) for _ in range(L)]
    state, x0 = _rand(rng, 8), _rand(rng, cfg["chunk"], cfg["A"])
    model = oracle.DenoiseModel(cfg, {**per, **glob})
    got = model.denoise(kp, vp, state, x0)
    t = lambda a: torch.from_numpy(a)
    layers = [{k: t(per[k][l]) for k in per} for l in range(L)]
    ref = tw.denoise_pi0(cfg, {k: t(v) for k, v in glob.items()}, layers, [t(a) for a in kp], [t(a) for a in vp],
                         t(state), t(x0)).numpy()
    np.testing.assert_allclose(got, ref, rtol=2e-4, atol=2e-5)
    assert np.abs(got - x0).max() > 1e-3  # the loop actually moved the sample
