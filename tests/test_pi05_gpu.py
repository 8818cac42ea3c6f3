"""The pi0.5-shaped denoise loop (engine model 2: adaptive RMSNorm conditioned on the time step, gated residuals, no
state token, no mask among the action tokens; src/models/pi05.cpp:208-292,604-631) against the CPU oracle's
restatement (oracle_ffi.pi05_denoise).

Bar: rel-L2 <= 1e-2 on the final action chunk (north-star tolerance), at small sizes and at the expert's full size
(18 layers, hidden 1024, 8 q / 1 kv heads of 256, MLP 4096, prefix 816, chunk 50, 10 Euler steps)."""
import numpy as np
import pytest

from tests.gpu_util import bits_to_bf16_tensor, rel_l2, require_cuda, to_dev

pytestmark = pytest.mark.gpu


def make_pi05(oracle, rng, L, H, n_q, n_kv, hd, inter, chunk, A, T, cond_dim=None, sigma=None):
    Hc = cond_dim or H
    qf, kvf = n_q * hd, n_kv * hd
    r = lambda *s, sc=1.0: oracle.bf16_round((rng.standard_normal(s) * (sigma or sc)).astype(np.float32))
    f = lambda *s, sc=1.0: (rng.standard_normal(s) * sc).astype(np.float32)
    layers = []
    for _ in range(L):
        layers.append(dict(wq=r(qf, H, sc=H ** -0.5), wk=r(kvf, H, sc=H ** -0.5), wv=r(kvf, H, sc=H ** -0.5), wo=r(H, qf, sc=qf ** -0.5),
                           wgate=r(inter, H, sc=H ** -0.5), wup=r(inter, H, sc=H ** -0.5), wdown=r(H, inter, sc=inter ** -0.5),
                           # scale and shift modulations of moderate size, gates around one
                           ada_in_w=f(3 * H, Hc, sc=0.3 * Hc ** -0.5), ada_in_b=np.concatenate([f(2 * H, sc=0.1), 1 + f(H, sc=0.1)]),
                           ada_post_w=f(3 * H, Hc, sc=0.3 * Hc ** -0.5), ada_post_b=np.concatenate([f(2 * H, sc=0.1), 1 + f(H, sc=0.1)])))
    w = dict(layers=layers, w_ain=r(H, A, sc=A ** -0.5), b_ain=f(H, sc=0.1), w_tin=f(Hc, H, sc=H ** -0.5), b_tin=f(Hc, sc=0.1),
             w_tout=f(Hc, Hc, sc=Hc ** -0.5), b_tout=f(Hc, sc=0.1), ada_final_w=f(3 * H, Hc, sc=0.3 * Hc ** -0.5),
             ada_final_b=f(3 * H, sc=0.1), w_aout=r(A, H, sc=H ** -0.5), b_aout=f(A, sc=0.1))
    cfg = dict(model=2, n_layers=L, H=H, n_q=n_q, n_kv=n_kv, head_dim=hd, inter=inter, chunk=chunk, action_dim=A, state_dim=0,
               steps=T, self_every=1, rms_eps=1e-6, rope_base=10000.0, min_period=4e-3, max_period=4.0, cond_dim=Hc)
    return cfg, w


def run_pi05(oracle, seed, n_obs, P, check_obs=None, **kw):
    require_cuda()
    import vla_cpp_b200 as vb

    rng = np.random.default_rng(seed)
    cfg, w = make_pi05(oracle, rng, **kw)
    L, n_kv, hd, chunk, A = cfg["n_layers"], cfg["n_kv"], cfg["head_dim"], cfg["chunk"], cfg["action_dim"]
    bf = lambda a: bits_to_bf16_tensor(oracle.f32_to_bf16_bits(a))
    weights = {k: [bf(lw[k]) for lw in w["layers"]] for k in ("wq", "wk", "wv", "wo", "wgate", "wup", "wdown")}
    weights.update({k: [to_dev(lw[k]) for lw in w["layers"]] for k in ("ada_in_w", "ada_in_b", "ada_post_w", "ada_post_b")})
    weights.update(w_ain=bf(w["w_ain"]), b_ain=to_dev(w["b_ain"]), w_aout=bf(w["w_aout"]), b_aout=to_dev(w["b_aout"]))
    weights.update({k: to_dev(w[k]) for k in ("ada_final_w", "ada_final_b", "w_tin", "b_tin", "w_tout", "b_tout")})
    eng = vb.PolicyEngine(cfg, weights, max_obs=n_obs + 1, prefix_len=P)
    kp = oracle.bf16_round(rng.standard_normal((L, n_obs, P, n_kv, hd)).astype(np.float32))
    vp = oracle.bf16_round(rng.standard_normal((L, n_obs, P, n_kv, hd)).astype(np.float32))
    for l in range(L):
        eng.set_prefix(l, to_dev(kp[l]), to_dev(vp[l]))
    x0 = rng.standard_normal((n_obs, chunk, A)).astype(np.float32)
    out = eng.denoise(to_dev(x0), None).cpu().numpy()
    assert vb.device_status() == 0
    again = eng.denoise(to_dev(x0), None).cpu().numpy()
    assert np.array_equal(out, again)
    ocfg = dict(H=cfg["H"], n_q=cfg["n_q"], n_kv=n_kv, hd=hd, steps=cfg["steps"], rms_eps=cfg["rms_eps"], rope_base=cfg["rope_base"],
                min_period=cfg["min_period"], max_period=cfg["max_period"])
    worst = 0.0
    for b in (range(n_obs) if check_obs is None else check_obs):
        ref = oracle.pi05_denoise([kp[l][b] for l in range(L)], [vp[l][b] for l in range(L)], x0[b], w, ocfg)
        worst = max(worst, rel_l2(out[b], ref))
    return worst


@pytest.mark.parametrize("n_obs,P,kw", [
    (1, 40, dict(L=2, H=128, n_q=4, n_kv=1, hd=64, inter=512, chunk=10, A=32, T=3)),
    (3, 70, dict(L=3, H=256, n_q=4, n_kv=2, hd=64, inter=768, chunk=12, A=32, T=4, cond_dim=192)),
    (7, 33, dict(L=2, H=128, n_q=2, n_kv=1, hd=128, inter=512, chunk=50, A=32, T=2)),
])
def test_pi05_loop_small(oracle, n_obs, P, kw):
    err = run_pi05(oracle, 5 + n_obs, n_obs, P, **kw)
    print(f"pi0.5 loop n_obs={n_obs} P={P}: rel_l2 {err:.3e}")
    assert err <= 1e-2, err


@pytest.mark.parametrize("n_obs,sigma", [(1, None), (6, 0.02)])
def test_pi05_loop_full_size(oracle, n_obs, sigma):
    """The expert at its real size, every layer and every Euler step; unit-scale weights and the N(0, 0.02) of the
    benchmark configurations."""
    err = run_pi05(oracle, 90 + n_obs, n_obs, 816, check_obs=[0, n_obs - 1], L=18, H=1024, n_q=8, n_kv=1, hd=256, inter=4096,
                   chunk=50, A=32, T=10, sigma=sigma)
    print(f"pi0.5 full-size loop n_obs={n_obs} sigma={sigma}: rel_l2 {err:.3e}")
    assert err <= 1e-2, err
