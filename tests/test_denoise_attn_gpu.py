"""GPU parity of the prefix-KV store, fused QKV+RoPE+append and attention kernels, through
the C ABI.  Tolerance (from the build's contract): rel-L2 <= 2e-2 per attention / QKV output
in bf16 against the float32 oracle; the KV page writer is bit-exact (a bf16 rounding)."""
import numpy as np
import pytest

from tests.gpu_util import bf16_bits, bits_to_bf16_tensor, rel_l2, require_cuda, to_dev

pytestmark = pytest.mark.gpu
TOL = 2e-2

SMOL = dict(H=720, n_q=15, n_kv=5, hd=64, S=51, P=177, eps=1e-5)   # isolated-op config (bf16)
PI0 = dict(H=1024, n_q=8, n_kv=1, hd=256, S=51, P=816, eps=1e-6)


def bf16_tensor(oracle, a):
    return bits_to_bf16_tensor(oracle.f32_to_bf16_bits(a))


def from_bf16(oracle, t):
    return oracle.bf16_bits_to_f32(bf16_bits(t))


def test_kv_store_write_is_a_bf16_rounding(oracle):
    torch = require_cuda()
    import vla_cpp_b200 as vb

    rng = np.random.default_rng(0)
    L, B, n_kv, hd, P, S = 3, 4, 5, 64, 37, 6
    st = vb.KvStore(L, B, n_kv, hd, P, S)
    k = rng.standard_normal((B, P, n_kv, hd)).astype(np.float32)
    v = rng.standard_normal((B, P, n_kv, hd)).astype(np.float32)
    st.write_prefix(1, to_dev(k), to_dev(v))
    st.write_prefix(2, to_dev(k[1:3]), to_dev(v[1:3]), obs0=2)
    assert vb.device_status() == 0
    kp = bf16_bits(st.k)  # [L][B][n_kv][cap][hd]
    vp = bf16_bits(st.v)
    assert np.array_equal(kp[1, :, :, :P], oracle.f32_to_bf16_bits(k).transpose(0, 2, 1, 3))
    assert np.array_equal(vp[1, :, :, :P], oracle.f32_to_bf16_bits(v).transpose(0, 2, 1, 3))
    assert np.array_equal(kp[2, 2:4, :, :P], oracle.f32_to_bf16_bits(k[1:3]).transpose(0, 2, 1, 3))
    assert not kp[0].any() and not kp[1, :, :, P:].any() and not kp[2, :2].any()


def test_rope_table(oracle):
    require_cuda()
    import vla_cpp_b200 as vb

    for hd, pos0, S in [(64, 177, 51), (256, 816, 51), (64, 0, 50)]:
        c, s = vb.rope_table(pos0, S, hd)
        rc, rs = oracle.rope_table(np.arange(pos0, pos0 + S), hd)
        np.testing.assert_allclose(c.cpu().numpy(), rc, atol=3e-4)  # float32 angle ulp at pos ~870 is 6e-5
        np.testing.assert_allclose(s.cpu().numpy(), rs, atol=3e-4)


def qkv_case(oracle, cfg, n_obs, seed, x_f32=False, project_kv=True, ln_rand=True, fold=False):
    import torch
    import vla_cpp_b200 as vb

    rng = np.random.default_rng(seed)
    H, n_q, n_kv, hd, S, P = (cfg[k] for k in ("H", "n_q", "n_kv", "hd", "S", "P"))
    n_rows = (n_q + (2 * n_kv if project_kv else 0)) * hd
    x = rng.standard_normal((n_obs * S, H)).astype(np.float32)
    if not x_f32:
        x = oracle.bf16_round(x)
    w = oracle.bf16_round((rng.standard_normal((n_rows, H)) * 0.02).astype(np.float32))
    ln = (1 + 0.1 * rng.standard_normal(H)).astype(np.float32) if ln_rand else np.ones(H, np.float32)
    st = vb.KvStore(2, n_obs, n_kv, hd, P, S)
    rope = vb.rope_table(P, S, hd)
    xd = to_dev(x) if x_f32 else bf16_tensor(oracle, x)
    wd, lnd = bf16_tensor(oracle, w), to_dev(ln)
    if fold:  # RMSNorm weight multiplied into the projection once; x then goes to the MMA by TMA
        wd, lnd = vb.fold_norm_weight(wd, lnd), None
    q = vb.qkv_rope_append(st, 1, xd, lnd, wd, rope, cfg["eps"], S, n_q, project_kv=project_kv)
    assert vb.device_status() == 0
    pos = np.arange(P, P + S).astype(np.int32)
    q_gpu = from_bf16(oracle, q)            # [n_obs][n_q][S][hd]
    k_gpu = from_bf16(oracle, st.k[1])      # [n_obs][n_kv][cap][hd]
    v_gpu = from_bf16(oracle, st.v[1])
    errs = []
    for b in range(n_obs):
        xb = x[b * S:(b + 1) * S]
        if project_kv:
            rq, rk, rv = oracle.qkv_rope(xb, ln, w, pos, n_q, n_kv, hd, cfg["eps"])
            errs.append(rel_l2(k_gpu[b, :, P:P + S].transpose(1, 0, 2), rk))
            errs.append(rel_l2(v_gpu[b, :, P:P + S].transpose(1, 0, 2), rv))
        else:
            rq = oracle.rope_neox(oracle.linear(oracle.rmsnorm(xb, ln, cfg["eps"]), w).reshape(S, n_q, hd), pos)
        errs.append(rel_l2(q_gpu[b].transpose(1, 0, 2), rq))
    assert not k_gpu[:, :, :P].any() and not from_bf16(oracle, st.k[0]).any()  # only suffix rows of layer 1 touched
    if not project_kv:
        assert not k_gpu.any() and not v_gpu.any()
    return max(errs)


@pytest.mark.parametrize("n_obs", [1, 3, 16])
def test_qkv_rope_append_smolvla_shape(oracle, n_obs):
    require_cuda()
    assert qkv_case(oracle, SMOL, n_obs, seed=10 + n_obs) < TOL


@pytest.mark.parametrize("n_obs", [1, 3, 16, 40])
def test_qkv_rope_append_folded_weights_tma_path(oracle, n_obs):
    require_cuda()
    assert qkv_case(oracle, SMOL, n_obs, seed=100 + n_obs, fold=True) < TOL


def test_qkv_rope_append_folded_pi0_shape_and_q_only(oracle):
    require_cuda()
    assert qkv_case(oracle, PI0, 5, seed=110, fold=True) < TOL
    assert qkv_case(oracle, SMOL, 3, seed=111, fold=True, project_kv=False) < TOL


def test_fold_norm_weight_is_exact_product(oracle):
    require_cuda()
    import vla_cpp_b200 as vb

    rng = np.random.default_rng(5)
    w = oracle.bf16_round(rng.standard_normal((96, 720)).astype(np.float32))
    ln = (1 + 0.1 * rng.standard_normal(720)).astype(np.float32)
    got = bf16_bits(vb.fold_norm_weight(bf16_tensor(oracle, w), to_dev(ln)))
    assert np.array_equal(got, oracle.f32_to_bf16_bits(w * ln[None, :]))


def test_qkv_rope_append_f32_input_and_unit_norm(oracle):
    require_cuda()
    assert qkv_case(oracle, SMOL, 2, seed=21, x_f32=True) < TOL
    assert qkv_case(oracle, SMOL, 2, seed=22, ln_rand=False) < TOL


def test_qkv_rope_append_pi0_shape(oracle):
    require_cuda()
    assert qkv_case(oracle, PI0, 3, seed=30) < TOL
    assert qkv_case(oracle, PI0, 1, seed=31, x_f32=True) < TOL


def test_q_only_projection_for_cross_attention_layers(oracle):
    require_cuda()
    assert qkv_case(oracle, SMOL, 2, seed=40, project_kv=False) < TOL


def attn_case(oracle, n_obs, n_q, n_kv, S, P, mask_mode, seed, cross=False, pads=None, poison=False, hd=64, tiling=0):
    import torch
    import vla_cpp_b200 as vb

    vb.set_gemm_tiling(tiling)  # 1 / 3 also force the one-CTA / CTA-pair form of the streaming attention kernel

    rng = np.random.default_rng(seed)
    st = vb.KvStore(2, n_obs, n_kv, hd, P, S)
    kv_len = P if cross else P + S
    k = oracle.bf16_round(rng.standard_normal((n_obs, n_kv, st.cap, hd)).astype(np.float32))
    v = oracle.bf16_round(rng.standard_normal((n_obs, n_kv, st.cap, hd)).astype(np.float32))
    q = oracle.bf16_round(rng.standard_normal((n_obs, n_q, S, hd)).astype(np.float32))
    kd, vd = k.copy(), v.copy()
    if poison:  # rows past kv_len hold NaN patterns: they must not reach the output
        kd[:, :, kv_len:] = np.nan
        vd[:, :, kv_len:] = np.nan
    st.k[1].copy_(bf16_tensor(oracle, kd))
    st.v[1].copy_(bf16_tensor(oracle, vd))
    pad_t = to_dev(np.asarray(pads, np.int32)) if pads is not None else None
    out = vb.attention(st, 1, bf16_tensor(oracle, q), S, n_q, kv_len, mask_mode, pad_ranges=pad_t)
    vb.set_gemm_tiling(0)
    assert vb.device_status() == 0
    got = from_bf16(oracle, out)  # [n_obs][S][n_q*hd]
    assert np.isfinite(got).all()
    worst = 0.0
    for b in range(n_obs):
        ps, pe = (pads[b] if pads is not None else (0, 0))
        ref = oracle.attention(q[b].transpose(1, 0, 2), k[b, :, :kv_len].transpose(1, 0, 2),
                               v[b, :, :kv_len].transpose(1, 0, 2), P, mask_mode, int(ps), int(pe))
        worst = max(worst, rel_l2(got[b], ref))
    return worst


@pytest.mark.parametrize("mask_mode", [0, 1, 2])
def test_attention_smolvla_shape_all_masks(oracle, mask_mode):
    require_cuda()
    assert attn_case(oracle, 3, 15, 5, 51, 177, mask_mode, seed=50 + mask_mode) < TOL


def test_attention_batch_and_pad_ranges(oracle):
    require_cuda()
    pads = [(130 + b, 176) if b % 2 else (0, 0) for b in range(16)]
    assert attn_case(oracle, 16, 15, 5, 50, 177, 2, seed=60, pads=pads) < TOL


def test_attention_edge_shapes(oracle):
    require_cuda()
    assert attn_case(oracle, 2, 4, 4, 5, 3, 2, seed=70) < TOL            # tiny, MHA
    assert attn_case(oracle, 2, 8, 1, 32, 224, 1, seed=71) < TOL          # MQA, kv_len = 256 (max), R = 256
    assert attn_case(oracle, 2, 6, 2, 40, 1, 2, seed=72) < TOL            # one prefix token
    assert attn_case(oracle, 1, 15, 5, 51, 177, 2, seed=73) < TOL         # single observation


def test_cross_attention_ignores_rows_past_kv_len(oracle):
    require_cuda()
    assert attn_case(oracle, 2, 15, 5, 50, 177, 0, seed=80, cross=True, poison=True) < TOL
    assert attn_case(oracle, 2, 15, 5, 50, 170, 0, seed=81, cross=True, poison=True,
                     pads=[(150, 169), (0, 0)]) < TOL


def test_attention_rejects_unsupported(oracle):
    require_cuda()
    import vla_cpp_b200 as vb

    st = vb.KvStore(1, 1, 1, 64, 20, 5)
    st.c.head_dim = 96  # no kernel for this head size
    q = np.zeros((1, 8, 5, 96), np.float32)
    with pytest.raises(vb.VlaB200Error) as e:
        vb.attention(st, 0, bf16_tensor(oracle, q), 5, 8, 25, 1)
    assert e.value.code == -4
    st.c.head_dim = 64
    with pytest.raises(vb.VlaB200Error) as e:  # kv_len beyond the page capacity
        vb.attention(st, 0, bf16_tensor(oracle, q), 5, 8, 26, 1)
    assert e.value.code == -1


@pytest.mark.parametrize("tiling", [1, 3])  # one CTA per row tile / CTA pairs (two row tiles of an item per MMA)
@pytest.mark.parametrize("mask_mode", [0, 1, 2])
def test_attention_pi0_shape_streaming_kernel(oracle, mask_mode, tiling):
    """8 q heads on 1 kv head, head_dim 256, 816 + 51 keys: 4 row tiles x 14 key blocks."""
    require_cuda()
    assert attn_case(oracle, 2, 8, 1, 51, 816, mask_mode, seed=200 + mask_mode, hd=256, tiling=tiling) < TOL


@pytest.mark.parametrize("tiling", [1, 3])
def test_attention_streaming_kernel_other_shapes(oracle, tiling):
    require_cuda()
    # BitVLA-LM-like heads (20q / 5kv, head_dim 128), bidirectional; 160 rows per item = two row tiles
    assert attn_case(oracle, 2, 20, 5, 40, 300, 0, seed=210, hd=128, tiling=tiling) < TOL
    # an odd number of row tiles (3 x 128 >= 8 x 40 rows): the pair's second CTA has no rows in the last unit
    assert attn_case(oracle, 2, 8, 1, 40, 200, 2, seed=216, hd=128, tiling=tiling) < TOL
    # five observations x 4 row tiles: units wrap around the CTA pairs
    assert attn_case(oracle, 5, 8, 1, 51, 130, 1, seed=217, hd=256, tiling=tiling) < TOL
    # head_dim 64 beyond the on-chip kernel's limits: 400 keys; and g*S = 408 rows
    assert attn_case(oracle, 2, 6, 2, 30, 370, 2, seed=211, hd=64) < TOL
    assert attn_case(oracle, 1, 8, 1, 51, 100, 1, seed=212, hd=64) < TOL
    # pad ranges, ragged key tail (kv_len % 64 != 0), cross-attention over a poisoned suffix
    assert attn_case(oracle, 3, 8, 1, 51, 816, 1, seed=213, hd=256, pads=[(700, 816), (0, 0), (64, 128)], tiling=tiling) < TOL
    assert attn_case(oracle, 2, 8, 1, 51, 777, 0, seed=214, hd=256, cross=True, poison=True, tiling=tiling) < TOL
    assert attn_case(oracle, 1, 8, 1, 5, 3, 2, seed=215, hd=256, tiling=tiling) < TOL


def test_attention_pair_kernel_several_units_per_cta_pair(oracle):
    """More work units than CTA pairs: a pair drains a unit's O after the first key block of its next unit, reads that
    unit's hidden key range one unit ahead and keeps its block counters running across units.  Every observation is
    compared with the oracle; hidden ranges differ between neighbours."""
    require_cuda()
    n_obs = 100  # x 2 tile pairs = 200 units on 74 CTA pairs
    pads = [((7 * b) % 90, (7 * b) % 90 + (b % 3) * 20) for b in range(n_obs)]
    # two key blocks (130 + 51 keys), pi0 mask, hidden ranges
    assert attn_case(oracle, n_obs, 8, 1, 51, 130, 1, seed=230, hd=256, pads=pads, tiling=3) < TOL
    # one key block per unit (60 + 51 keys <= 128): the drain follows directly
    assert attn_case(oracle, n_obs, 8, 1, 51, 60, 2, seed=231, hd=256, tiling=3) < TOL
    # head_dim 128 (three S buffers), five key blocks, bidirectional
    assert attn_case(oracle, 90, 8, 2, 50, 500, 0, seed=232, hd=128, tiling=3) < TOL


@pytest.mark.parametrize("tiling", [1, 3])
def test_attention_streaming_kernel_large_score_spread(oracle, tiling):
    """Keys whose scores grow along the sequence force the lazy running-maximum update (and the
    rescale of O through TMEM) to trigger."""
    torch = require_cuda()
    import vla_cpp_b200 as vb

    vb.set_gemm_tiling(tiling)

    hd, n_q, n_kv, S, P, n_obs = 256, 8, 1, 51, 816, 1
    rng = np.random.default_rng(300)
    st = vb.KvStore(1, n_obs, n_kv, hd, P, S)
    q = oracle.bf16_round(rng.standard_normal((n_obs, n_q, S, hd)).astype(np.float32))
    ramp = np.linspace(0.2, 3.0, st.cap).astype(np.float32)[None, None, :, None]
    k = oracle.bf16_round((rng.standard_normal((n_obs, n_kv, st.cap, hd)) * ramp).astype(np.float32))
    v = oracle.bf16_round(rng.standard_normal((n_obs, n_kv, st.cap, hd)).astype(np.float32))
    st.k[0].copy_(bf16_tensor(oracle, k))
    st.v[0].copy_(bf16_tensor(oracle, v))
    out = vb.attention(st, 0, bf16_tensor(oracle, q), S, n_q, P + S, vb.MASK_PI0)
    vb.set_gemm_tiling(0)
    assert vb.device_status() == 0
    ref = oracle.attention(q[0].transpose(1, 0, 2), k[0].transpose(1, 0, 2), v[0].transpose(1, 0, 2), P, 1)
    assert rel_l2(from_bf16(oracle, out)[0], ref) < TOL


@pytest.mark.parametrize("mask_mode", [2, 0])
def test_attention_hd64_score_spread_within_a_column_half(oracle, mask_mode):
    """head_dim 64, 228 keys: key norms grow along the sequence (and jump in the middle of each half of the key range), so
    later 32-key chunks beat the first chunk of their half by far more than 2^8: the single-pass kernel has to raise its
    reference and rescale the P chunks it has already written."""
    torch = require_cuda()
    import vla_cpp_b200 as vb

    hd, n_q, n_kv, S, P, n_obs = 64, 15, 5, 51, 177, 3
    rng = np.random.default_rng(310 + mask_mode)
    st = vb.KvStore(1, n_obs, n_kv, hd, P, S)
    q = oracle.bf16_round(rng.standard_normal((n_obs, n_q, S, hd)).astype(np.float32))
    ramp = np.linspace(0.3, 2.5, st.cap).astype(np.float32)
    ramp[70:] *= 2.0   # inside the first half of the key range (keys 0..127)
    ramp[200:] *= 1.6  # inside the second half
    k = oracle.bf16_round((rng.standard_normal((n_obs, n_kv, st.cap, hd)) * ramp[None, None, :, None]).astype(np.float32))
    v = oracle.bf16_round(rng.standard_normal((n_obs, n_kv, st.cap, hd)).astype(np.float32))
    st.k[0].copy_(bf16_tensor(oracle, k))
    st.v[0].copy_(bf16_tensor(oracle, v))
    out = vb.attention(st, 0, bf16_tensor(oracle, q), S, n_q, P + S, mask_mode)
    assert vb.device_status() == 0
    got = from_bf16(oracle, out)
    assert np.isfinite(got).all()
    for b in range(n_obs):
        ref = oracle.attention(q[b].transpose(1, 0, 2), k[b].transpose(1, 0, 2), v[b].transpose(1, 0, 2), P, mask_mode)
        assert rel_l2(got[b], ref) < TOL


def test_isolated_denoise_attention_two_layers_chain(oracle):
    """QKV+RoPE+append feeding attention, two layers, as the isolated-op config runs them."""
    require_cuda()
    import vla_cpp_b200 as vb

    cfg, n_obs = SMOL, 4
    H, n_q, n_kv, hd, S, P = (cfg[k] for k in ("H", "n_q", "n_kv", "hd", "S", "P"))
    rng = np.random.default_rng(90)
    st = vb.KvStore(2, n_obs, n_kv, hd, P, S)
    rope = vb.rope_table(P, S, hd)
    pos = np.arange(P, P + S).astype(np.int32)
    for layer in range(2):
        kp = rng.standard_normal((n_obs, P, n_kv, hd)).astype(np.float32)
        vp = rng.standard_normal((n_obs, P, n_kv, hd)).astype(np.float32)
        st.write_prefix(layer, to_dev(kp), to_dev(vp))
        x = oracle.bf16_round(rng.standard_normal((n_obs * S, H)).astype(np.float32))
        w = oracle.bf16_round((rng.standard_normal(((n_q + 2 * n_kv) * hd, H)) * 0.02).astype(np.float32))
        ln = np.ones(H, np.float32)
        q = vb.qkv_rope_append(st, layer, bf16_tensor(oracle, x), to_dev(ln), bf16_tensor(oracle, w), rope,
                               cfg["eps"], S, n_q)
        out = vb.attention(st, layer, q, S, n_q, P + S, vb.MASK_CAUSAL)
        assert vb.device_status() == 0
        got = from_bf16(oracle, out)
        for b in range(n_obs):
            rq, rk, rv = oracle.qkv_rope(x[b * S:(b + 1) * S], ln, w, pos, n_q, n_kv, hd, cfg["eps"])
            K = np.concatenate([oracle.bf16_round(kp[b]), rk])
            V = np.concatenate([oracle.bf16_round(vp[b]), rv])
            ref = oracle.attention(rq, K, V, P, 2)
            assert rel_l2(got[b], ref) < TOL


def test_loop_driver_matches_stepwise_calls(oracle):
    """vlab200_denoise_attn_loop (C++ driver, folded weights) against per-call composition, and the
    host-buffer variant against the device-resident one."""
    torch = require_cuda()
    import vla_cpp_b200 as vb

    cfg, n_obs, L, T = SMOL, 3, 2, 2
    H, n_q, n_kv, hd, S, P = (cfg[k] for k in ("H", "n_q", "n_kv", "hd", "S", "P"))
    g = torch.Generator(device="cuda").manual_seed(3)
    st = vb.KvStore(L, n_obs, n_kv, hd, P, S)
    for l in range(L):
        st.write_prefix(l, torch.randn((n_obs, P, n_kv, hd), device="cuda", generator=g),
                        torch.randn((n_obs, P, n_kv, hd), device="cuda", generator=g))
    w = (torch.randn((L, (n_q + 2 * n_kv) * hd, H), device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    ln = 1 + 0.1 * torch.randn((L, H), device="cuda", generator=g)
    x = torch.randn((T, L, n_obs * S, H), device="cuda", generator=g).to(torch.bfloat16)
    op = vb.DenoiseAttn(st, H, n_q, S, ln, w, cfg["eps"], vb.MASK_CAUSAL)
    out = op.run(x).clone()
    assert vb.device_status() == 0
    rope = vb.rope_table(P, S, hd)
    for l in range(L):  # the last step decides the result
        q = vb.qkv_rope_append(st, l, x[T - 1, l], ln[l].contiguous(), w[l].contiguous(), rope, cfg["eps"], S, n_q)
        ref = vb.attention(st, l, q, S, n_q, P + S, vb.MASK_CAUSAL)
        a, b = from_bf16(oracle, out[l]), from_bf16(oracle, ref)
        assert rel_l2(a, b) < 1e-2  # folded vs unfolded weights differ by bf16 roundings only
    x_host = x.cpu().pin_memory()
    out_host = torch.empty(op.out.shape, dtype=torch.bfloat16).pin_memory()
    op.run_host(x_host, out_host)
    torch.cuda.synchronize()
    assert vb.device_status() == 0
    assert torch.equal(out_host, out.cpu())


def test_attention_output_aligned_to_16_bytes_only(oracle):
    """The head_dim-64 kernel writes 32-byte sectors when `out` allows it and falls back to 16-byte stores when the
    buffer is only 16-byte aligned: same bits either way."""
    torch = require_cuda()
    import vla_cpp_b200 as vb

    rng = np.random.default_rng(77)
    n_obs, n_q, n_kv, S, P, hd = 3, 15, 5, 51, 177, 64
    st = vb.KvStore(1, n_obs, n_kv, hd, P, S)
    st.k.copy_(bf16_tensor(oracle, oracle.bf16_round(rng.standard_normal(tuple(st.k.shape)).astype(np.float32))))
    st.v.copy_(bf16_tensor(oracle, oracle.bf16_round(rng.standard_normal(tuple(st.v.shape)).astype(np.float32))))
    q = bf16_tensor(oracle, oracle.bf16_round(rng.standard_normal((n_obs, n_q, S, hd)).astype(np.float32)))
    want = vb.attention(st, 0, q, S, n_q, P + S, 2)
    assert want.data_ptr() % 32 == 0
    n = want.numel()
    buf = torch.zeros(n + 16, dtype=torch.bfloat16, device="cuda")
    out = buf[8:8 + n].view(want.shape)  # 16 bytes past a 32-byte boundary
    assert out.data_ptr() % 32 == 16
    vb.attention(st, 0, q, S, n_q, P + S, 2, out=out)
    assert vb.device_status() == 0
    assert torch.equal(out, want) and float(buf[:8].abs().sum()) == 0 and float(buf[8 + n:].abs().sum()) == 0
