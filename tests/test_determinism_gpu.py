"""Run-to-run determinism of the kernels whose statistics warps read TMA-filled shared memory with
ordinary loads (fused QKV projection, bf16 GEMM with the RMS factor in its epilogue).

Every output element is produced by exactly one CTA from fixed inputs, so two runs must agree bit for
bit.  They did not while the stage was handed back to TMA without a proxy fence after the loads: row
sums came out one k-slice off on CTAs that work on more than one tile.  The cases below give every CTA
several tiles, on both tilings (one CTA per tile, CTA pairs)."""
import numpy as np
import pytest

from tests.gpu_util import require_cuda

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("tiling", [1, 3])
@pytest.mark.parametrize("shape", [dict(H=1024, n_q=8, n_kv=1, hd=256, S=51, P=64, B=64),
                                   dict(H=720, n_q=15, n_kv=5, hd=64, S=51, P=177, B=256),
                                   dict(H=1024, n_q=16, n_kv=2, hd=128, S=20, P=32, B=160)])
def test_qkv_projection_is_deterministic(tiling, shape):
    torch = require_cuda()
    import vla_cpp_b200 as vb

    H, n_q, n_kv, hd, S, P, B = (shape[k] for k in ("H", "n_q", "n_kv", "hd", "S", "P", "B"))
    g = torch.Generator(device="cuda")
    g.manual_seed(1)
    st = vb.KvStore(1, B, n_kv, hd, P, S)
    rope = vb.rope_table(P, S, hd)
    x = torch.randn((B * S, H), device="cuda", generator=g).to(torch.bfloat16)
    w = (torch.randn(((n_q + 2 * n_kv) * hd, H), device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    q = torch.empty((B, n_q, S, hd), dtype=torch.bfloat16, device="cuda")
    vb.set_gemm_tiling(tiling)
    try:
        first = None
        for _ in range(6):
            st.k.zero_(); st.v.zero_(); q.zero_()
            vb.qkv_rope_append(st, 0, x, None, w, rope, 1e-6, S, n_q, q_out=q)
            torch.cuda.synchronize()
            cur = (q.clone(), st.k.clone(), st.v.clone())
            if first is None:
                first = cur
            else:
                assert all(torch.equal(a, b) for a, b in zip(first, cur))
        assert vb.device_status() == 0
        # and the row statistics are the right ones: V rows = rmsnorm(x) @ Wv^T
        xf = x.float()
        xn = xf * torch.rsqrt((xf * xf).mean(-1, keepdim=True) + 1e-6)
        v_ref = (xn @ w[(n_q + n_kv) * hd:].float().T).view(B, S, n_kv, hd).permute(0, 2, 1, 3)
        v = first[2][0, :, :, P:P + S].float()
        assert float((v - v_ref).abs().max()) <= 2.0 ** -7 * float(v_ref.abs().max()) + 1e-3
    finally:
        vb.set_gemm_tiling(0)


@pytest.mark.parametrize("tiling", [1, 3])
def test_engine_loop_is_deterministic(oracle, tiling):
    torch = require_cuda()
    import vla_cpp_b200 as vb
    from tests.gpu_util import bits_to_bf16_tensor, to_dev
    from tests.test_engine_gpu import make_policy

    rng = np.random.default_rng(21)
    kw = dict(model=0, L=2, H=512, n_q=8, n_kv=1, hd=64, inter=2048, chunk=50, A=32, sd=32, T=2)
    n_obs, P = 160, 48  # 8160 rows: 64 row tiles x 16 column tiles of the gate/up GEMM on 148 SMs
    cfg, per, glob, _ = make_policy(oracle, rng, P=P, **kw)
    bf = lambda a: bits_to_bf16_tensor(oracle.f32_to_bf16_bits(a))
    weights = {k: [bf(a) if k.startswith("w") else to_dev(a) for a in v] for k, v in per.items()}
    weights.update({k: (bf(a) if k.startswith("w_") else to_dev(a)) for k, v in glob.items() for a in [v]})
    eng = vb.PolicyEngine(cfg, weights, max_obs=n_obs, prefix_len=P)
    g = torch.Generator(device="cuda")
    g.manual_seed(2)
    for l in range(cfg["n_layers"]):
        kp = torch.randn((n_obs, P, cfg["n_kv"], cfg["head_dim"]), device="cuda", generator=g)
        eng.set_prefix(l, kp, torch.randn(kp.shape, device="cuda", generator=g))
    x0 = torch.randn((n_obs, cfg["chunk"], cfg["action_dim"]), device="cuda", generator=g)
    state = torch.randn((n_obs, cfg["state_dim"]), device="cuda", generator=g)
    vb.set_gemm_tiling(tiling)
    try:
        outs = [eng.denoise(x0, state).cpu().numpy() for _ in range(4)]
        assert vb.device_status() == 0
    finally:
        vb.set_gemm_tiling(0)
    for o in outs[1:]:
        assert np.array_equal(o, outs[0])


def test_a_wait_that_runs_out_reports_and_leaves_the_context_usable(oracle):
    """Every mbarrier wait in the library has a cycle budget.  The self-test kernel waits (with a budget of 1e5
    cycles, ~50 us) on a barrier that nothing signals: the wait must give up, the kernel must return through its
    common exit, the status word must read 104 (DEV_TIMEOUT_MISC) until reset, and the next ordinary kernel must
    run and be correct.  Nothing hangs or faults by construction: the wait is bounded."""
    torch = require_cuda()
    import vla_cpp_b200 as vb

    assert vb.device_status() == 0
    assert vb.selftest_bounded_wait(100000) is True
    assert vb.device_status(reset=False) == 104
    assert vb.device_status(reset=True) == 104
    assert vb.device_status() == 0
    x = torch.randn((4, 256), device="cuda").to(torch.bfloat16)
    q, s = vb.act_quant(x)
    rq, rs = oracle.act_quant(x.float().cpu().numpy())
    assert np.array_equal(q.cpu().numpy(), rq) and np.array_equal(s.cpu().numpy(), rs)
    assert vb.device_status() == 0
