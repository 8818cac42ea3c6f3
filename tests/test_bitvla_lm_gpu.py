"""GPU parity of the BitVLA language-model block (BitNet layers on the ternary kernels), through
the C ABI, against the CPU oracle's restatement of the reference layer.

Bars:
  * fused norm/quant stage: the bf16 normalised row within 1 bf16 ulp of the oracle on <= 0.1 % of the
    elements (rsqrt and summation order), and the int8 row + scale bit-identical to the oracle's
    act-quant of that very row;
  * whole stack: relative L2 <= 5e-2 on the bf16 output against the CPU oracle.  The bar is derived from the
    comparison with the reference's own CUDA forward (tests/test_bitvla_lm_ref_gpu.py, measured on B200 at the LM's
    real width): reference vs this library 1.99e-2 (1 layer x 300 tokens) and 3.43e-2 (2 layers x 37 tokens),
    reference vs the oracle 1.81e-2 / 3.26e-2, this library vs the oracle 1.97e-2 / 3.39e-2 -- three implementations
    of the same arithmetic sit 2-3.5e-2 from one another on 1-2 layers, because every layer re-quantises to int8 four
    times and squares the gate, which turns last-bit differences into flipped int8 codes.  5e-2 is that distance with
    head-room of 1.5x; the per-stage tests below are bit-exact, and the stage-by-stage comparison with the reference's
    layer-0 dump shows where the distance enters (attention: 4.4e-3, growing to 2e-2 at the layer output)."""
import numpy as np
import pytest

from tests.gpu_util import bf16_bits, bits_to_bf16_tensor, require_cuda, to_dev

pytestmark = pytest.mark.gpu

REL_L2_TOL = 5e-2

SMALL = dict(hidden=256, n_q=4, n_kv=2, head_dim=64, ffn=384, rms_eps=1e-5, rope_base=10000.0)
LM = dict(hidden=2560, n_q=20, n_kv=5, head_dim=128, ffn=6912, rms_eps=1e-5, rope_base=500000.0)


def make_layer(oracle, rng, cfg):
    hidden, ffn = cfg["hidden"], cfg["ffn"]
    hq, hkv = cfg["n_q"] * cfg["head_dim"], cfg["n_kv"] * cfg["head_dim"]
    lw = {}

    def tern(name, n, k, ws_num=1):
        t = rng.integers(-1, 2, (n, k)).astype(np.int8)
        lw[name + "_packed"] = oracle.pack_ladder_int2(t)
        lw[name + "_ws"] = (rng.uniform(0.8, 1.2, ws_num) / np.sqrt(2.0 * k / 3.0)).astype(np.float32)

    tern("q", hq, hidden)
    tern("k", hkv, hidden)
    tern("v", hkv, hidden)
    tern("o", hidden, hq)
    tern("gate_up", 2 * ffn, hidden, 2)
    tern("down", hidden, ffn)
    for name, k in (("attn_norm_w", hidden), ("attn_sub_norm_w", hq), ("ffn_norm_w", hidden), ("ffn_sub_norm_w", ffn)):
        lw[name] = oracle.bf16_round(rng.uniform(0.8, 1.2, k).astype(np.float32))
    return lw


def to_dev_layer(oracle, lw):
    out = {}
    for k, v in lw.items():
        if k.endswith("_packed") or k.endswith("_ws"):
            out[k] = to_dev(v)
        else:
            out[k] = bits_to_bf16_tensor(oracle.f32_to_bf16_bits(v))
    return out


def rel_l2(got, ref):
    return float(np.linalg.norm(got - ref) / max(np.linalg.norm(ref), 1e-30))


@pytest.mark.parametrize("cfg,n_layers,seq,n_seq", [(SMALL, 2, 40, 1), (SMALL, 2, 150, 3), (SMALL, 1, 5, 2),
                                                     (LM, 1, 70, 1), (LM, 2, 6, 1)])
def test_lm_stack_matches_oracle(oracle, cfg, n_layers, seq, n_seq):
    require_cuda()
    from vla_cpp_b200 import api

    rng = np.random.default_rng(7 + seq + 13 * n_layers + cfg["hidden"])
    layers = [make_layer(oracle, rng, cfg) for _ in range(n_layers)]
    out_norm = oracle.bf16_round(rng.uniform(0.8, 1.2, cfg["hidden"]).astype(np.float32))
    x = oracle.bf16_round(rng.standard_normal((n_seq, seq, cfg["hidden"])).astype(np.float32))

    dev_layers = [to_dev_layer(oracle, lw) for lw in layers]
    lm = api.BitvlaLM(cfg["hidden"], cfg["n_q"], cfg["n_kv"], cfg["head_dim"], cfg["ffn"], dev_layers,
                      bits_to_bf16_tensor(oracle.f32_to_bf16_bits(out_norm)), rope_base=cfg["rope_base"],
                      rms_eps=cfg["rms_eps"], max_seq=max(seq, 64), max_batch=n_seq)
    xd = bits_to_bf16_tensor(oracle.f32_to_bf16_bits(x))
    got = oracle.bf16_bits_to_f32(bf16_bits(lm.forward(xd)))
    assert api.device_status() == 0
    got2 = oracle.bf16_bits_to_f32(bf16_bits(lm.forward(xd)))  # second call: no state carried over
    assert np.array_equal(got, got2)
    for i in range(n_seq):
        ref = oracle.bitvla_lm_forward(x[i], layers, out_norm, cfg)
        err = rel_l2(got[i], ref)
        assert err <= REL_L2_TOL, f"sequence {i}: rel L2 {err:.3e}"


def test_lm_rejects_bad_arguments(oracle):
    require_cuda()
    from vla_cpp_b200 import api

    rng = np.random.default_rng(3)
    layers = [to_dev_layer(oracle, make_layer(oracle, rng, SMALL))]
    out_norm = bits_to_bf16_tensor(oracle.f32_to_bf16_bits(np.ones(SMALL["hidden"], np.float32)))
    lm = api.BitvlaLM(SMALL["hidden"], SMALL["n_q"], SMALL["n_kv"], SMALL["head_dim"], SMALL["ffn"], layers, out_norm,
                      max_seq=16, max_batch=1)
    import torch

    x = torch.zeros((32, SMALL["hidden"]), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(api.VlaB200Error):
        lm.forward(x)  # seq > max_seq
    with pytest.raises(api.VlaB200Error):
        api.BitvlaLM(100, 4, 2, 64, 384, layers, out_norm)  # hidden not a multiple of 128


@pytest.mark.parametrize("mode", [0, 1, 2])
@pytest.mark.parametrize("m,k", [(1, 256), (37, 2560), (5, 6912), (3, 250), (2, 8200), (4, 4096), (3, 8192),
                                 (70, 2560), (100, 1024), (65, 4096), (64, 2048)])  # 250, 8200: scalar kernel
def test_norm_quant_stage(oracle, mode, m, k):
    require_cuda()
    from vla_cpp_b200 import api

    rng = np.random.default_rng(100 * mode + m + k)
    cols = 2 * k if mode == 2 else k
    x = oracle.bf16_round(rng.standard_normal((m, cols)).astype(np.float32) * 1.7)
    add = oracle.bf16_round(rng.standard_normal((m, k)).astype(np.float32))
    w = oracle.bf16_round(rng.uniform(0.5, 1.5, k).astype(np.float32))
    eps = 1e-5

    def dev(a):
        return bits_to_bf16_tensor(oracle.f32_to_bf16_bits(a))

    if mode == 0:
        pre = x
    elif mode == 1:
        pre = oracle.bf16_round(x + add)
    else:
        g = np.maximum(x[:, :k], 0)
        pre = oracle.bf16_round((g * g * x[:, k:]).astype(np.float32))
    ref_y = oracle.bitvla_rmsnorm_bf16(pre, w, eps)

    xd = dev(x)
    y = api.bitvla_norm_quant(xd, dev(w), eps, mode, add=dev(add) if mode == 1 else None, quantise=False)
    y_bits = bf16_bits(y)
    if mode == 1:  # the residual stream is updated in place
        assert np.array_equal(bf16_bits(xd), oracle.f32_to_bf16_bits(pre))
    d = np.abs(y_bits.astype(np.int32) - oracle.f32_to_bf16_bits(ref_y).astype(np.int32))
    assert d.max() <= 1 and (d != 0).mean() <= 1e-3, (d.max(), (d != 0).mean())

    q, s = api.bitvla_norm_quant(dev(x), dev(w), eps, mode, add=dev(add) if mode == 1 else None)
    ref_q, ref_s = oracle.act_quant(oracle.bf16_bits_to_f32(y_bits))
    assert api.device_status() == 0
    assert np.array_equal(s.cpu().numpy(), ref_s)
    assert np.array_equal(q.cpu().numpy(), ref_q)
