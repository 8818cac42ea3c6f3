"""The whole flow-matching denoise loop (vlab200_engine_*) against the CPU oracle.

Bar: rel-L2 <= 1e-2 on the final action chunk (bf16 activations on the GPU, float32 oracle on
the same bf16-representable weights); the displacement x_T - x_0 is checked as well so that the
noise x_0 cannot hide an error in the predicted velocities."""
import os

import numpy as np
import pytest

from tests.gpu_util import bits_to_bf16_tensor, rel_l2, require_cuda, to_dev

pytestmark = pytest.mark.gpu


def make_policy(oracle, rng, model, L, H, n_q, n_kv, hd, inter, P, chunk, A, sd, T, self_every=1, wscale=None,
                sigma=None):
    """sigma: every matrix drawn N(0, sigma) (the benchmark configurations say N(0, 0.02)); otherwise each matrix
    gets 1/sqrt(fan_in) so that activations keep unit scale at any width."""
    qf, kvf = n_q * hd, n_kv * hd
    r = lambda *s, sc=1.0: oracle.bf16_round((rng.standard_normal(s) * (sigma or sc)).astype(np.float32))
    f = lambda *s, sc=1.0: (rng.standard_normal(s) * sc).astype(np.float32)
    ws = wscale or (1.0 / np.sqrt(H))
    per = {k: [] for k in ("wq", "wk", "wv", "wo", "wgate", "wup", "wdown", "ln_in", "ln_post")}
    wqkv = []
    for l in range(L):
        is_self = model == 0 or self_every <= 1 or l % self_every == 0
        per["wq"].append(r(qf, H, sc=ws))
        if is_self:
            per["wk"].append(r(kvf, H, sc=ws))
            per["wv"].append(r(kvf, H, sc=ws))
        else:
            per["wk"].append(r(kvf, kvf, sc=1.0 / np.sqrt(kvf)))
            per["wv"].append(r(kvf, kvf, sc=1.0 / np.sqrt(kvf)))
        per["wo"].append(r(H, qf, sc=1.0 / np.sqrt(qf)))
        per["wgate"].append(r(inter, H, sc=ws))
        per["wup"].append(r(inter, H, sc=ws))
        per["wdown"].append(r(H, inter, sc=1.0 / np.sqrt(inter)))
        per["ln_in"].append(1 + f(H, sc=0.1))
        per["ln_post"].append(1 + f(H, sc=0.1))
        wqkv.append(np.concatenate([per["wq"][l].ravel(), per["wk"][l].ravel(), per["wv"][l].ravel()]))
    glob = dict(w_ain=r(H, A, sc=1.0 / np.sqrt(A)), b_ain=f(H, sc=0.1), w_at1=r(H, 2 * H, sc=1.0 / np.sqrt(2 * H)),
                b_at1=f(H, sc=0.1), w_at2=r(H, H, sc=ws), b_at2=f(H, sc=0.1), out_norm=1 + f(H, sc=0.1),
                w_aout=r(A, H, sc=ws), b_aout=f(A, sc=0.1))
    if model == 0:
        glob.update(w_sp=r(H, sd, sc=1.0 / np.sqrt(sd)), b_sp=f(H, sc=0.1))
    cfg = dict(model=model, n_layers=L, H=H, n_q=n_q, n_kv=n_kv, head_dim=hd, inter=inter, chunk=chunk, action_dim=A,
               state_dim=sd, steps=T, self_every=self_every, rms_eps=1e-6 if model == 0 else 1e-5, rope_base=10000.0,
               min_period=4e-3, max_period=4.0)
    return cfg, per, glob, wqkv


def oracle_model(oracle, cfg, per, glob, wqkv, P, pos_base, pad):
    ocfg = dict(model=cfg["model"], n_layers=cfg["n_layers"], H=cfg["H"], n_q=cfg["n_q"], n_kv=cfg["n_kv"],
                hd=cfg["head_dim"], inter=cfg["inter"], P=P, chunk=cfg["chunk"], A=cfg["action_dim"],
                state_dim=cfg["state_dim"], T=cfg["steps"], pos_base=pos_base, pad_start=pad[0], pad_end=pad[1],
                self_every=max(cfg["self_every"], 1), act_bf16=0, rms_eps=cfg["rms_eps"], rope_base=cfg["rope_base"],
                min_period=cfg["min_period"], max_period=cfg["max_period"])
    ow = dict(ln_in=per["ln_in"], Wqkv=wqkv, Wo=per["wo"], ln_post=per["ln_post"], Wgate=per["wgate"],
              Wup=per["wup"], Wdown=per["wdown"], W_sp=glob.get("w_sp"), b_sp=glob.get("b_sp"), W_ain=glob["w_ain"],
              b_ain=glob["b_ain"], W_at1=glob["w_at1"], b_at1=glob["b_at1"], W_at2=glob["w_at2"], b_at2=glob["b_at2"],
              out_norm=glob["out_norm"], W_aout=glob["w_aout"], b_aout=glob["b_aout"])
    return oracle.DenoiseModel(ocfg, ow)


def run_case(oracle, seed, n_obs, P, pos_base=-1, pad=None, tiling=0, check_obs=None, **kw):
    """check_obs: the observations compared with the oracle (default: all; the full-depth cases check a few,
    the oracle needs seconds per observation there)."""
    torch = require_cuda()
    import vla_cpp_b200 as vb

    vb.set_gemm_tiling(tiling)

    rng = np.random.default_rng(seed)
    cfg, per, glob, wqkv = make_policy(oracle, rng, P=P, **kw)
    L, n_kv, hd, chunk, A, sd = cfg["n_layers"], cfg["n_kv"], cfg["head_dim"], cfg["chunk"], cfg["action_dim"], cfg["state_dim"]
    bf = lambda a: bits_to_bf16_tensor(oracle.f32_to_bf16_bits(a))
    weights = {k: [bf(a) if k.startswith("w") else to_dev(a) for a in v] for k, v in per.items()}
    weights.update({k: (bf(a) if k.startswith("w_") else to_dev(a)) for k, v in glob.items() for a in [v]})
    eng = vb.PolicyEngine(cfg, weights, max_obs=n_obs + 1, prefix_len=P)  # one spare slot: views must keep strides
    kp = oracle.bf16_round(rng.standard_normal((L, n_obs, P, n_kv, hd)).astype(np.float32))
    vp = oracle.bf16_round(rng.standard_normal((L, n_obs, P, n_kv, hd)).astype(np.float32))
    for l in range(L):
        eng.set_prefix(l, to_dev(kp[l]), to_dev(vp[l]))
    state = rng.standard_normal((n_obs, sd)).astype(np.float32)
    x0 = rng.standard_normal((n_obs, chunk, A)).astype(np.float32)
    pads = None
    if pad is not None:
        pads = to_dev(np.tile(np.asarray(pad, np.int32), (n_obs, 1)))
    out = eng.denoise(to_dev(x0), to_dev(state), pos_base=pos_base, pad_ranges=pads).cpu().numpy()
    assert vb.device_status() == 0
    assert np.isfinite(out).all()
    om = oracle_model(oracle, cfg, per, glob, wqkv, P, P if pos_base < 0 else pos_base, pad or (0, 0))
    worst, worst_d = 0.0, 0.0
    for b in (range(n_obs) if check_obs is None else check_obs):
        ref = om.denoise([kp[l, b] for l in range(L)], [vp[l, b] for l in range(L)], state[b], x0[b])
        worst = max(worst, rel_l2(out[b], ref))
        worst_d = max(worst_d, rel_l2(out[b] - x0[b], ref - x0[b]))
        assert np.linalg.norm(ref - x0[b]) > 0.05 * np.linalg.norm(x0[b])  # the loop moved the sample
    # host-buffer entry point gives the same result
    x0h, sth = torch.from_numpy(x0).pin_memory(), torch.from_numpy(state).pin_memory()
    outh = torch.empty_like(x0h).pin_memory()
    padh = None if pad is None else torch.from_numpy(np.tile(np.asarray(pad, np.int32), (n_obs, 1))).pin_memory()
    eng.denoise_host(x0h, sth, outh, pos_base=pos_base, pad_ranges_host=padh)
    torch.cuda.synchronize()
    assert np.array_equal(outh.numpy(), out)
    vb.set_gemm_tiling(0)
    return worst, worst_d


def test_pi0_small(oracle):
    w, d = run_case(oracle, 1, n_obs=3, P=40, model=0, L=2, H=128, n_q=4, n_kv=1, hd=64, inter=256, chunk=10, A=32,
                    sd=32, T=3)
    assert w < 1e-2 and d < 3e-2, (w, d)


def test_pi0_full_width_two_layers(oracle):
    w, d = run_case(oracle, 2, n_obs=2, P=816, model=0, L=2, H=1024, n_q=8, n_kv=1, hd=256, inter=4096, chunk=50,
                    A=32, sd=32, T=2)
    assert w < 1e-2 and d < 3e-2, (w, d)


def test_smolvla_small_with_cross_layers_pads_and_position_base(oracle):
    w, d = run_case(oracle, 3, n_obs=3, P=30, pos_base=27, pad=(20, 29), model=1, L=4, H=192, n_q=6, n_kv=2, hd=64,
                    inter=256, chunk=10, A=32, sd=32, T=3, self_every=2)
    assert w < 1e-2 and d < 3e-2, (w, d)


def test_smolvla_full_width_two_layers(oracle):
    w, d = run_case(oracle, 4, n_obs=2, P=177, pos_base=170, model=1, L=2, H=720, n_q=15, n_kv=5, hd=64, inter=2048,
                    chunk=50, A=32, sd=32, T=2, self_every=2)
    assert w < 1e-2 and d < 3e-2, (w, d)


@pytest.mark.parametrize("tiling", [1, 2, 3, 4])
def test_pi0_every_gemm_tiling_matches_oracle(oracle, tiling):
    """The four tilings of the bf16 GEMMs (one CTA per 128x256 / 128x128 / 128x64 tile, CTA pairs on 256x256)
    forced in turn on a case with several row tiles (7 observations x 51 rows = 357 rows)."""
    w, d = run_case(oracle, 5, n_obs=7, P=64, tiling=tiling, model=0, L=2, H=512, n_q=8, n_kv=1, hd=64, inter=1024,
                    chunk=50, A=32, sd=32, T=2)
    assert w < 1e-2 and d < 3e-2, (w, d)


def test_gemm_tilings_are_bit_identical(oracle):
    torch = require_cuda()
    import vla_cpp_b200 as vb

    rng = np.random.default_rng(11)
    kw = dict(model=0, L=2, H=512, n_q=8, n_kv=1, hd=64, inter=1024, chunk=50, A=32, sd=32, T=2)
    n_obs, P = 12, 64  # 612 suffix rows: above the few-row path of the QKV projection, so every tiling runs the same kernels
    cfg, per, glob, _ = make_policy(oracle, rng, P=P, **kw)
    bf = lambda a: bits_to_bf16_tensor(oracle.f32_to_bf16_bits(a))
    weights = {k: [bf(a) if k.startswith("w") else to_dev(a) for a in v] for k, v in per.items()}
    weights.update({k: (bf(a) if k.startswith("w_") else to_dev(a)) for k, v in glob.items() for a in [v]})
    eng = vb.PolicyEngine(cfg, weights, max_obs=n_obs, prefix_len=P)
    for l in range(cfg["n_layers"]):
        kp = torch.randn((n_obs, P, cfg["n_kv"], cfg["head_dim"]), device="cuda")
        eng.set_prefix(l, kp, torch.randn_like(kp))
    x0 = torch.randn((n_obs, cfg["chunk"], cfg["action_dim"]), device="cuda")
    state = torch.randn((n_obs, cfg["state_dim"]), device="cuda")
    outs = []
    for tiling in (1, 2, 3, 4, 0):
        vb.set_gemm_tiling(tiling)
        outs.append(eng.denoise(x0, state).cpu().numpy())
        assert vb.device_status() == 0
    vb.set_gemm_tiling(0)
    for o in outs[1:]:
        assert np.array_equal(o, outs[0])


# ---- the benchmark configurations at their full depth: every layer, all ten Euler steps ----------------------
PI0_FULL = dict(model=0, L=18, H=1024, n_q=8, n_kv=1, hd=256, inter=4096, chunk=50, A=32, sd=32, T=10)
SMOLVLA_FULL = dict(model=1, L=16, H=720, n_q=15, n_kv=5, hd=64, inter=2048, chunk=50, A=32, sd=32, T=10,
                    self_every=2)


@pytest.mark.parametrize("n_obs,check,sigma", [(1, [0], 0.02), (6, [0, 5], 0.02), (6, [3], None)])
def test_pi0_full_depth_18_layers_10_steps(oracle, n_obs, check, sigma):
    """pi0-shaped expert exactly as benchmarked: 18 layers x 10 steps, prefix 816, 180 layer-steps of bf16
    activations against the float32 oracle.  One observation takes the few-row path, six the fused path."""
    w, d = run_case(oracle, 21 + n_obs, n_obs=n_obs, P=816, check_obs=check, sigma=sigma, **PI0_FULL)
    print(f"pi0 full depth n_obs={n_obs} sigma={sigma}: rel_l2={w:.3e} displacement rel_l2={d:.3e}")
    assert w < 1e-2 and d < 3e-2, (w, d)


@pytest.mark.parametrize("n_obs,check,sigma", [(1, [0], 0.02), (6, [0, 5], 0.02), (6, [2], None)])
def test_smolvla_full_depth_16_layers_10_steps(oracle, n_obs, check, sigma):
    """SmolVLA-shaped expert as benchmarked: 16 layers alternating self / cross attention x 10 steps, prefix 177
    with padded language slots and the rebased suffix positions."""
    w, d = run_case(oracle, 41 + n_obs, n_obs=n_obs, P=177, pos_base=170, pad=(160, 176), check_obs=check, sigma=sigma,
                    **SMOLVLA_FULL)
    print(f"smolvla full depth n_obs={n_obs} sigma={sigma}: rel_l2={w:.3e} displacement rel_l2={d:.3e}")
    assert w < 1e-2 and d < 3e-2, (w, d)


def test_several_engines_one_host_thread_each(oracle):
    """vlab200_engines_denoise_host: 11 observations cut over 3 engines (3 replicas; on a one-GPU box they all live
    on that GPU, each with its own stream and host thread), blocks of at most max_obs = 2 observations at a time.
    Every observation's chunk is bit-identical to what one engine computes for it alone."""
    import ctypes as C

    torch = require_cuda()
    import vla_cpp_b200 as vb

    rng = np.random.default_rng(23)
    kw = dict(model=0, L=2, H=128, n_q=4, n_kv=1, hd=64, inter=256, chunk=10, A=32, sd=32, T=2)
    n_total, n_eng, P, max_obs = 11, 3, 24, 2
    cfg, per, glob, _ = make_policy(oracle, rng, P=P, **kw)
    bf = lambda a: bits_to_bf16_tensor(oracle.f32_to_bf16_bits(a))
    weights = {k: [bf(a) if k.startswith("w") else to_dev(a) for a in v] for k, v in per.items()}
    weights.update({k: (bf(a) if k.startswith("w_") else to_dev(a)) for k, v in glob.items() for a in [v]})
    kp = torch.randn((cfg["n_layers"], 1, P, cfg["n_kv"], cfg["head_dim"]), device="cuda")
    vp = torch.randn_like(kp)
    engines = [vb.PolicyEngine(cfg, weights, max_obs=max_obs, prefix_len=P) for _ in range(n_eng)]
    for e in engines:  # the same prefix in every slot: what an observation computes then depends on its inputs only
        for l in range(cfg["n_layers"]):
            e.set_prefix(l, kp[l].expand(max_obs, -1, -1, -1).contiguous(), vp[l].expand(max_obs, -1, -1, -1).contiguous())
    x0 = torch.randn((n_total, cfg["chunk"], cfg["action_dim"])).pin_memory()
    state = torch.randn((n_total, cfg["state_dim"])).pin_memory()
    out = torch.zeros_like(x0).pin_memory()
    torch.cuda.synchronize()
    arr = (C.c_void_p * n_eng)(*[e.h for e in engines])

    def run_all():
        rc = vb.lib().vlab200_engines_denoise_host(arr, n_eng, C.c_int64(n_total), C.c_void_p(state.data_ptr()),
                                                   C.c_void_p(x0.data_ptr()), C.c_void_p(out.data_ptr()), -1, None)
        assert rc == 0, vb.lib().vlab200_last_error()
        assert vb.device_status() == 0

    # Blocks of one observation take the persistent loop kernel, blocks of two the launch-per-operator path: the two
    # agree to rounding, not to the bit.  With the loop kernel off every block takes the same kernels.
    old_env = os.environ.get("VLAB200_CHUNK_LOOP")
    os.environ["VLAB200_CHUNK_LOOP"] = "0"
    try:
        run_all()
        for o in range(n_total):
            alone = engines[0].denoise(x0[o:o + 1].cuda(), state[o:o + 1].cuda()).cpu()
            assert torch.equal(alone[0], out[o]), o
    finally:
        if old_env is None:
            del os.environ["VLAB200_CHUNK_LOOP"]
        else:
            os.environ["VLAB200_CHUNK_LOOP"] = old_env
    exact = out.clone()
    run_all()  # default: three host threads launch the cooperative loop kernel and the operator path side by side
    assert ((out - exact).norm() / exact.norm()).item() <= 1e-2
    # sharding arithmetic of the native helper
    seen = []
    for r in range(n_eng):
        s, c = C.c_int64(), C.c_int64()
        assert vb.lib().vlab200_shard_range(C.c_int64(n_total), n_eng, r, C.byref(s), C.byref(c)) == 0
        seen += list(range(s.value, s.value + c.value))
    assert seen == list(range(n_total))
