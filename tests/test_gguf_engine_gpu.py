"""Engine built from a pi0- or SmolVLA-shaped GGUF (the reference converters' tensor names, metadata keys and dtypes,
scripts/convert_pi0_to_gguf.py:234-244, scripts/gguf_blocks.py:104-142,196-211) against the engine built from
the same weights handed over directly: bit-identical action chunks."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

gguf = pytest.importorskip("gguf")

from tests.gpu_util import bits_to_bf16_tensor, require_cuda, to_dev
from tests.test_engine_gpu import make_policy


@pytest.fixture(scope="module")
def oracle():
    from oracle import oracle_ffi

    oracle_ffi.build()
    return oracle_ffi


def _golden_names(arch):
    """Tensor suffixes and metadata keys as the reference's converters write them (tests/golden/gguf_names.json,
    recorded from scripts/gguf_blocks.py and scripts/convert_*_to_gguf.py by tests/golden/make_golden.py)."""
    import json
    import os

    g = json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "gguf_names.json")))[arch]
    suffixes = [n.split(".", 3)[3] for n, _, _ in g["decoder_blocks"] if n.startswith("aex.blk.0.")]
    return suffixes, {k for k, _ in g["kv"]}, g["projections"], g["output_norm"]


def _write_policy(path, oracle, cfg, per, glob, bf16_matrices, arch="pi0", extra=None, hidden=2048):
    F32, BF16 = gguf.GGMLQuantizationType.F32, gguf.GGMLQuantizationType.BF16
    w = gguf.GGUFWriter(str(path), arch)
    suffixes, golden_keys, golden_proj, golden_out_norm = _golden_names(arch)

    def kv(k):
        assert arch + "." + k in golden_keys, k  # only keys the reference converter writes
        return arch + "." + k
    for key, val in (("n_layers", cfg["n_layers"]), ("expert_h", cfg["H"]), ("n_q_heads", cfg["n_q"]),
                     ("n_kv_heads", cfg["n_kv"]), ("head_dim", cfg["head_dim"]), ("expert_inter", cfg["inter"]),
                     ("chunk_size", cfg["chunk"]), ("num_steps", cfg["steps"]), ("max_state_dim", cfg["state_dim"]),
                     ("max_action_dim", cfg["action_dim"]), ("hidden", hidden)):
        w.add_uint32(kv(key), val)
    w.add_float64(kv("min_period"), cfg["min_period"])
    w.add_float64(kv("max_period"), cfg["max_period"])
    if arch == "pi0":
        w.add_float64(kv("rope_theta"), cfg["rope_base"])
        w.add_float32(kv("rms_norm_eps"), cfg["rms_eps"])
    else:
        w.add_uint32(kv("self_attn_every_n_layers"), cfg["self_every"])

    def mat(name, a):
        if bf16_matrices:
            w.add_tensor(name, oracle.f32_to_bf16_bits(a).astype(np.uint16), raw_shape=list(a.shape), raw_dtype=BF16)
        else:
            w.add_tensor(name, np.ascontiguousarray(a, dtype=np.float32), raw_dtype=F32)

    vec = lambda name, a: w.add_tensor(name, np.ascontiguousarray(a, dtype=np.float32), raw_dtype=F32)
    ours = {"attn_norm.weight": "ln_raw_in", "attn_q.weight": "wq", "attn_k.weight": "wk", "attn_v.weight": "wv",
            "attn_o.weight": "wo", "ffn_norm.weight": "ln_raw_post", "ffn_gate.weight": "wgate", "ffn_up.weight": "wup",
            "ffn_down.weight": "wdown"}
    assert sorted(ours) == sorted(suffixes)
    for l in range(cfg["n_layers"]):
        for suffix in suffixes:  # the converter's order
            (vec if "norm" in suffix else mat)(f"aex.blk.{l}.{suffix}", per[ours[suffix]][l])
    vec(golden_out_norm, glob["out_norm_raw"])
    heads = (("w_sp", "state_proj"),) if arch == "pi0" else ()
    for k, n in heads + (("w_ain", "action_in_proj"), ("w_at1", "action_time_mlp_in"),
                         ("w_at2", "action_time_mlp_out"), ("w_aout", "action_out_proj")):
        assert n + ".weight" in golden_proj and n + ".bias" in golden_proj
        mat(n + ".weight", glob[k])
        vec(n + ".bias", glob["b_" + k[2:]])
    if extra is not None:
        extra(w, kv, mat, vec)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()


@pytest.mark.parametrize("arch,bf16_matrices", [("pi0", True), ("pi0", False), ("smolvla", True)])
def test_engine_from_gguf_matches_direct_engine(oracle, tmp_path, arch, bf16_matrices):
    torch = require_cuda()
    import vla_cpp_b200 as vb

    rng = np.random.default_rng(11)
    P, n_obs = 40, 3
    if arch == "pi0":
        cfg, per, glob, _ = make_policy(oracle, rng, model=0, L=2, H=128, n_q=2, n_kv=1, hd=64, inter=256, P=P,
                                        chunk=10, A=32, sd=32, T=3)
        # Gemma norms are stored without their +1
        off = np.float32(1)
    else:
        cfg, per, glob, _ = make_policy(oracle, rng, model=1, L=4, H=128, n_q=4, n_kv=2, hd=64, inter=256, P=P,
                                        chunk=10, A=32, sd=32, T=3, self_every=2)
        off = np.float32(0)
    per["ln_raw_in"] = [(a - off).astype(np.float32) for a in per["ln_in"]]
    per["ln_raw_post"] = [(a - off).astype(np.float32) for a in per["ln_post"]]
    per["ln_in"] = [a + off for a in per["ln_raw_in"]]
    per["ln_post"] = [a + off for a in per["ln_raw_post"]]
    glob["out_norm_raw"] = (glob["out_norm"] - off).astype(np.float32)
    glob["out_norm"] = glob["out_norm_raw"] + off
    path = tmp_path / "policy.gguf"
    _write_policy(path, oracle, cfg, per, glob, bf16_matrices, arch)

    g = vb.Gguf(path)
    eng_g = vb.PolicyEngine.from_gguf(g, max_obs=n_obs, prefix_len=P)
    g.close()  # the engine holds its own copies
    bf = lambda a: bits_to_bf16_tensor(oracle.f32_to_bf16_bits(a))
    keys = ("wq", "wk", "wv", "wo", "wgate", "wup", "wdown", "ln_in", "ln_post")
    weights = {k: [bf(a) if k.startswith("w") else to_dev(a) for a in per[k]] for k in keys}
    weights.update({k: (bf(v) if k.startswith("w_") else to_dev(v)) for k, v in glob.items() if not k.endswith("_raw")})
    eng_d = vb.PolicyEngine(cfg, weights, max_obs=n_obs, prefix_len=P)

    L, n_kv, hd = cfg["n_layers"], cfg["n_kv"], cfg["head_dim"]
    kp = rng.standard_normal((L, n_obs, P, n_kv, hd)).astype(np.float32)
    vp = rng.standard_normal((L, n_obs, P, n_kv, hd)).astype(np.float32)
    for e in (eng_g, eng_d):
        for l in range(L):
            e.set_prefix(l, to_dev(kp[l]), to_dev(vp[l]))
    state = to_dev(rng.standard_normal((n_obs, cfg["state_dim"])).astype(np.float32))
    x0 = to_dev(rng.standard_normal((n_obs, cfg["chunk"], cfg["action_dim"])).astype(np.float32))
    out_g = eng_g.denoise(x0, state).cpu().numpy()
    out_d = eng_d.denoise(x0, state).cpu().numpy()
    assert vb.device_status() == 0
    assert np.isfinite(out_g).all() and np.array_equal(out_g, out_d)


def test_engine_from_gguf_reports_what_is_wrong(oracle, tmp_path):
    require_cuda()
    import vla_cpp_b200 as vb

    rng = np.random.default_rng(12)
    cfg, per, glob, _ = make_policy(oracle, rng, model=0, L=1, H=128, n_q=2, n_kv=1, hd=64, inter=256, P=8, chunk=10,
                                    A=32, sd=32, T=2)
    per["ln_raw_in"], per["ln_raw_post"], glob["out_norm_raw"] = per["ln_in"], per["ln_post"], glob["out_norm"]
    per["wo"][0] = per["wo"][0][:, :64]  # wrong shape
    path = tmp_path / "bad.gguf"
    _write_policy(path, oracle, cfg, per, glob, True)
    g = vb.Gguf(path)
    with pytest.raises(vb.VlaB200Error, match="attn_o"):
        vb.PolicyEngine.from_gguf(g, max_obs=1, prefix_len=8)


def _write_bitvla_lm(path, cfg, layers, out_norm, drop=None):
    """The LM part of scripts/convert_bitvla_to_gguf.py:165-178,215-236,366-386: ladder packs as 1-D I8 tensors with
    float32 .scale sidecars, norm vectors float32, "bitvla.lm.*" metadata."""
    I8, F32 = gguf.GGMLQuantizationType.I8, gguf.GGMLQuantizationType.F32
    w = gguf.GGUFWriter(str(path), "bitvla")
    for k, v in (("hidden", cfg["hidden"]), ("layers", len(layers)), ("q_heads", cfg["n_q"]), ("kv_heads", cfg["n_kv"]),
                 ("head_dim", cfg["head_dim"]), ("inter", cfg["ffn"])):
        w.add_uint32("bitvla.lm." + k, v)
    w.add_float32("bitvla.lm.rope_theta", cfg["rope_base"])
    w.add_float32("bitvla.lm.rms_eps", cfg["rms_eps"])
    w.add_uint32("bitvla.quant.int2_packed", 1)  # scripts/convert_bitvla_to_gguf.py:263
    names = dict(q="attn_q", k="attn_k", v="attn_v", o="attn_o", gate_up="ffn_gate_up", down="ffn_down")
    for l, lw in enumerate(layers):
        for k in ("attn_norm", "attn_sub_norm", "ffn_norm", "ffn_sub_norm"):
            w.add_tensor(f"lm.blk.{l}.{k}.weight", np.ascontiguousarray(lw[k + "_w"], dtype=np.float32), raw_dtype=F32)
        for k, n in names.items():
            packed = np.ascontiguousarray(lw[k + "_packed"], dtype=np.uint8)
            w.add_tensor(f"lm.blk.{l}.{n}.weight", packed, raw_shape=[int(packed.size)], raw_dtype=I8)
            if drop != f"lm.blk.{l}.{n}.scale":
                w.add_tensor(f"lm.blk.{l}.{n}.scale", np.ascontiguousarray(lw[k + "_ws"], dtype=np.float32), raw_dtype=F32)
    w.add_tensor("lm.output_norm.weight", np.ascontiguousarray(out_norm, dtype=np.float32), raw_dtype=F32)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()


def test_bitvla_lm_from_gguf_matches_direct_context(oracle, tmp_path):
    require_cuda()
    import vla_cpp_b200 as vb
    from tests.gpu_util import bf16_bits
    from tests.test_bitvla_lm_gpu import SMALL, make_layer, to_dev_layer

    rng = np.random.default_rng(21)
    layers = [make_layer(oracle, rng, SMALL) for _ in range(2)]
    out_norm = oracle.bf16_round(rng.uniform(0.8, 1.2, SMALL["hidden"]).astype(np.float32))
    path = tmp_path / "bitvla.gguf"
    _write_bitvla_lm(path, SMALL, layers, out_norm)
    g = vb.Gguf(path)
    assert g.info("lm.blk.0.ffn_gate_up.weight") == (24, [2 * SMALL["ffn"] * SMALL["hidden"] // 4],
                                                     2 * SMALL["ffn"] * SMALL["hidden"] // 4)
    lm_g = vb.BitvlaLM.from_gguf(g, max_seq=64, max_batch=2)
    g.close()
    lm_d = vb.BitvlaLM(SMALL["hidden"], SMALL["n_q"], SMALL["n_kv"], SMALL["head_dim"], SMALL["ffn"],
                       [to_dev_layer(oracle, lw) for lw in layers], bits_to_bf16_tensor(oracle.f32_to_bf16_bits(out_norm)),
                       rope_base=SMALL["rope_base"], rms_eps=SMALL["rms_eps"], max_seq=64, max_batch=2)
    x = bits_to_bf16_tensor(oracle.f32_to_bf16_bits(
        oracle.bf16_round(rng.standard_normal((2, 37, SMALL["hidden"])).astype(np.float32))))
    a, b = bf16_bits(lm_g.forward(x)), bf16_bits(lm_d.forward(x))
    assert vb.device_status() == 0
    assert np.array_equal(a, b)

    _write_bitvla_lm(tmp_path / "nosidecar.gguf", SMALL, layers, out_norm, drop="lm.blk.1.attn_o.scale")
    g = vb.Gguf(tmp_path / "nosidecar.gguf")
    with pytest.raises(vb.VlaB200Error, match="sidecar"):
        vb.BitvlaLM.from_gguf(g)


def test_bitvla_lm_from_float_checkpoint_is_ternarised_and_packed_at_load(oracle, tmp_path):
    """A checkpoint without "bitvla.quant.int2_packed" carries float matrices (ffn_gate and ffn_up separate); the
    loader ternarises and ladder-packs them on the device, as the reference's load_bit does on the host
    (src/models/bitvla.cpp:515-543,755-757,808-815).  Result: bit-identical to a context built from the oracle's
    ternarisation + packing of the same matrices."""
    require_cuda()
    import vla_cpp_b200 as vb
    from tests.gpu_util import bf16_bits
    from tests.test_bitvla_lm_gpu import SMALL

    cfg = SMALL
    rng = np.random.default_rng(33)
    hidden, ffn = cfg["hidden"], cfg["ffn"]
    hq, hkv = cfg["n_q"] * cfg["head_dim"], cfg["n_kv"] * cfg["head_dim"]
    F32 = gguf.GGMLQuantizationType.F32
    w = gguf.GGUFWriter(str(tmp_path / "float.gguf"), "bitvla")
    for k, v in (("hidden", hidden), ("layers", 2), ("q_heads", cfg["n_q"]), ("kv_heads", cfg["n_kv"]),
                 ("head_dim", cfg["head_dim"]), ("inter", ffn)):
        w.add_uint32("bitvla.lm." + k, v)
    w.add_float32("bitvla.lm.rope_theta", cfg["rope_base"])
    w.add_float32("bitvla.lm.rms_eps", cfg["rms_eps"])
    layers = []
    shapes = dict(attn_q=(hq, hidden), attn_k=(hkv, hidden), attn_v=(hkv, hidden), attn_o=(hidden, hq),
                  ffn_gate=(ffn, hidden), ffn_up=(ffn, hidden), ffn_down=(hidden, ffn))
    for l in range(2):
        lw, mats = {}, {}
        for k, n in (("attn_norm", hidden), ("attn_sub_norm", hq), ("ffn_norm", hidden), ("ffn_sub_norm", ffn)):
            lw[k + "_w"] = oracle.bf16_round(rng.uniform(0.8, 1.2, n).astype(np.float32))
            w.add_tensor(f"lm.blk.{l}.{k}.weight", lw[k + "_w"], raw_dtype=F32)
        for name, shp in shapes.items():
            mats[name] = (rng.standard_normal(shp) * rng.uniform(0.01, 0.05)).astype(np.float32)
            w.add_tensor(f"lm.blk.{l}.{name}.weight", mats[name], raw_dtype=F32)
        for short, name in (("q", "attn_q"), ("k", "attn_k"), ("v", "attn_v"), ("o", "attn_o"), ("down", "ffn_down")):
            t, am = oracle.ternarize(mats[name])
            lw[short + "_packed"], lw[short + "_ws"] = oracle.pack_ladder_int2(t), np.array([am], np.float32)
        tg, ag = oracle.ternarize(mats["ffn_gate"])
        tu, au = oracle.ternarize(mats["ffn_up"])
        lw["gate_up_packed"] = oracle.pack_ladder_int2(np.concatenate([tg, tu]))
        lw["gate_up_ws"] = np.array([ag, au], np.float32)
        layers.append(lw)
    out_norm = oracle.bf16_round(rng.uniform(0.8, 1.2, hidden).astype(np.float32))
    w.add_tensor("lm.output_norm.weight", out_norm, raw_dtype=F32)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    from tests.test_bitvla_lm_gpu import to_dev_layer

    g = vb.Gguf(tmp_path / "float.gguf")
    lm_g = vb.BitvlaLM.from_gguf(g, max_seq=64, max_batch=1)
    g.close()
    lm_d = vb.BitvlaLM(hidden, cfg["n_q"], cfg["n_kv"], cfg["head_dim"], ffn, [to_dev_layer(oracle, lw) for lw in layers],
                       bits_to_bf16_tensor(oracle.f32_to_bf16_bits(out_norm)), rope_base=cfg["rope_base"],
                       rms_eps=cfg["rms_eps"], max_seq=64, max_batch=1)
    x = bits_to_bf16_tensor(oracle.f32_to_bf16_bits(oracle.bf16_round(rng.standard_normal((29, hidden)).astype(np.float32))))
    a, b = bf16_bits(lm_g.forward(x)), bf16_bits(lm_d.forward(x))
    assert vb.device_status() == 0
    assert np.array_equal(a, b)
