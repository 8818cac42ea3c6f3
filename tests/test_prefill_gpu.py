"""The prefix producer (vlab200_prefill_*): the backbone's layers over the prefix embeddings, writing every
layer's rotated K and V into the denoise engine's bf16 pages, against the CPU oracle's restatement of
build_vlm_layer / build_gemma_layer (src/models/smolvla.cpp:778-813, src/models/pi0.cpp:159-233).

Bars: rel-L2 <= 2e-2 on each layer's K and V pages (bf16 activations on the GPU, float32 oracle on the same
bf16-representable weights); SmolVLA cross-attention layers are compared after expert_cross_kv
(smolvla.cpp:853-860); the action chunk of a denoise loop fed by those pages stays within 1e-2 of the oracle's
loop fed by the oracle's prefill."""
import numpy as np
import pytest

from tests.gpu_util import bits_to_bf16_tensor, rel_l2, require_cuda, to_dev
from tests.test_engine_gpu import make_policy, oracle_model

pytestmark = pytest.mark.gpu


def make_vlm(oracle, rng, L, hidden, n_q, n_kv, hd, inter, sigma=None):
    qf, kvf = n_q * hd, n_kv * hd
    r = lambda *s, sc: oracle.bf16_round((rng.standard_normal(s) * (sigma or sc)).astype(np.float32))
    layers = []
    for _ in range(L):
        lw = dict(wq=r(qf, hidden, sc=hidden ** -0.5), wk=r(kvf, hidden, sc=hidden ** -0.5),
                  wv=r(kvf, hidden, sc=hidden ** -0.5), wo=r(hidden, qf, sc=qf ** -0.5),
                  wgate=r(inter, hidden, sc=hidden ** -0.5), wup=r(inter, hidden, sc=hidden ** -0.5),
                  wdown=r(hidden, inter, sc=inter ** -0.5),
                  ln_in=(1 + 0.1 * rng.standard_normal(hidden)).astype(np.float32),
                  ln_post=(1 + 0.1 * rng.standard_normal(hidden)).astype(np.float32))
        lw["wqkv"] = np.concatenate([lw["wq"], lw["wk"], lw["wv"]])
        layers.append(lw)
    return layers


def run_prefill_case(oracle, seed, model, n_obs, P, pos, mask_mode, pad, vlm_dims, expert_kw, act, check_denoise=True):
    torch = require_cuda()
    import vla_cpp_b200 as vb

    rng = np.random.default_rng(seed)
    L, hidden, n_q, n_kv, hd, inter = vlm_dims
    layers = make_vlm(oracle, rng, L, hidden, n_q, n_kv, hd, inter)
    cfg, per, glob, wqkv = make_policy(oracle, rng, P=P, model=model, L=L, n_q=expert_kw.pop("n_q_e", n_q), n_kv=n_kv, hd=hd,
                                       **expert_kw)
    bf = lambda a: bits_to_bf16_tensor(oracle.f32_to_bf16_bits(a))
    weights = {k: [bf(a) if k.startswith("w") else to_dev(a) for a in v] for k, v in per.items()}
    weights.update({k: (bf(a) if k.startswith("w_") else to_dev(a)) for k, v in glob.items() for a in [v]})
    eng = vb.PolicyEngine(cfg, weights, max_obs=n_obs + 1, prefix_len=P + 3)  # pages sized for a longer prefix
    eng.set_prefix_len(P)
    pcfg = dict(n_layers=L, hidden=hidden, n_q=n_q, n_kv=n_kv, head_dim=hd, inter=inter, act=act,
                rms_eps=cfg["rms_eps"], rope_base=cfg["rope_base"])
    pw = {k: [bf(lw[k]) if k.startswith("w") else to_dev(lw[k]) for lw in layers]
          for k in ("wq", "wk", "wv", "wo", "wgate", "wup", "wdown", "ln_in", "ln_post")}
    pre = vb.Prefill(pcfg, pw, max_obs=n_obs, max_prefix=P + 3)
    x = rng.standard_normal((n_obs, P, hidden)).astype(np.float32)
    pads = None if pad is None else to_dev(np.tile(np.asarray(pad, np.int32), (n_obs, 1)))
    pre.run(eng, to_dev(x), positions=pos, mask_mode=mask_mode, pad_ranges=pads)
    assert vb.device_status() == 0
    ocfg = dict(n_q=n_q, n_kv=n_kv, hd=hd, rms_eps=cfg["rms_eps"], rope_base=cfg["rope_base"],
                act="silu" if act == 1 else "gelu")
    worst = 0.0
    ref_kv = []
    for b in range(n_obs):
        ks, vs = oracle.vlm_prefill(x[b], layers, ocfg, pos=pos, mask_mode=mask_mode, pad=pad or (0, 0))
        ref_kv.append((ks, vs))
    for l in range(L):
        k_dev, v_dev = eng.get_prefix(l, n_kv, hd, n_obs=n_obs)
        k_dev, v_dev = k_dev.cpu().numpy(), v_dev.cpu().numpy()
        cross = model == 1 and cfg["self_every"] > 1 and l % cfg["self_every"] != 0
        for b in range(n_obs):
            rk, rv = ref_kv[b][0][l], ref_kv[b][1][l]
            if cross:  # expert_cross_kv on the flattened kv axis
                rk = oracle.linear(rk.reshape(P, -1), per["wk"][l]).reshape(P, n_kv, hd)
                rv = oracle.linear(rv.reshape(P, -1), per["wv"][l]).reshape(P, n_kv, hd)
            ek, ev = rel_l2(k_dev[b], rk), rel_l2(v_dev[b], rv)
            worst = max(worst, ek, ev)
            assert ek <= 2e-2 and ev <= 2e-2, (l, b, ek, ev)
    out_err = None
    if check_denoise:
        state = rng.standard_normal((n_obs, cfg["state_dim"])).astype(np.float32)
        x0 = rng.standard_normal((n_obs, cfg["chunk"], cfg["action_dim"])).astype(np.float32)
        pos_base = -1 if model == 0 else int(pos[-1]) + 1
        out = eng.denoise(to_dev(x0), to_dev(state), pos_base=pos_base, pad_ranges=pads).cpu().numpy()
        om = oracle_model(oracle, cfg, per, glob, wqkv, P, P if pos_base < 0 else pos_base, pad or (0, 0))
        out_err = 0.0
        for b in range(n_obs):
            ref = om.denoise(ref_kv[b][0], ref_kv[b][1], state[b], x0[b])
            out_err = max(out_err, rel_l2(out[b], ref))
        assert out_err <= 1e-2, out_err
    assert vb.device_status() == 0
    return worst, out_err


def test_smolvla_shaped_prefill_small_with_cross_layers_pads_and_state_token(oracle):
    P, n_img, n_lang_max, n_lang = 30, 20, 9, 5
    pos = np.arange(P, dtype=np.int32)
    pos[-1] = n_img + n_lang  # the state token sits right after the real language tokens
    pad = (n_img + n_lang, n_img + n_lang_max)
    w, o = run_prefill_case(oracle, 1, model=1, n_obs=2, P=P, pos=pos, mask_mode=3, pad=pad,
                            vlm_dims=(4, 256, 6, 2, 64, 384),
                            expert_kw=dict(H=192, inter=256, chunk=10, A=32, sd=32, T=3, self_every=2), act=1)
    print(f"smolvla-shaped prefill: worst K/V rel_l2 {w:.3e}, chunk rel_l2 {o:.3e}")


def test_pi0_shaped_prefill_small(oracle):
    w, o = run_prefill_case(oracle, 2, model=0, n_obs=3, P=70, pos=None, mask_mode=0, pad=None,
                            vlm_dims=(3, 256, 4, 1, 128, 512),
                            expert_kw=dict(H=128, inter=256, chunk=10, A=32, sd=32, T=3), act=2)
    print(f"pi0-shaped prefill: worst K/V rel_l2 {w:.3e}, chunk rel_l2 {o:.3e}")


def test_smolvla_backbone_at_full_width_and_depth(oracle):
    """SmolVLA's own VLM dimensions: 16 layers, hidden 960, 15 q / 5 kv heads of 64, MLP 2560, prefix 177."""
    P, n_img, n_lang_max, n_lang = 177, 128, 48, 31
    pos = np.arange(P, dtype=np.int32)
    pos[-1] = n_img + n_lang
    pad = (n_img + n_lang, n_img + n_lang_max)
    w, o = run_prefill_case(oracle, 3, model=1, n_obs=1, P=P, pos=pos, mask_mode=3, pad=pad,
                            vlm_dims=(16, 960, 15, 5, 64, 2560),
                            expert_kw=dict(H=720, inter=2048, chunk=50, A=32, sd=32, T=2, self_every=2), act=1)
    print(f"smolvla full-size prefill: worst K/V rel_l2 {w:.3e}, chunk rel_l2 {o:.3e}")


def test_pi0_backbone_at_full_width(oracle):
    """Gemma-2B-shaped layers (hidden 2048, 8 q / 1 kv heads of 256, MLP 16384) over the 816-token prefix; four
    layers (the last one only produces K/V) keep the oracle within seconds."""
    w, o = run_prefill_case(oracle, 4, model=0, n_obs=1, P=816, pos=None, mask_mode=0, pad=None,
                            vlm_dims=(4, 2048, 8, 1, 256, 16384),
                            expert_kw=dict(H=1024, inter=4096, chunk=50, A=32, sd=32, T=2), act=2)
    print(f"pi0 full-width prefill: worst K/V rel_l2 {w:.3e}, chunk rel_l2 {o:.3e}")
