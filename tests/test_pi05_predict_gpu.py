"""vla_predict on a pi0.5-shaped checkpoint (GGUF in the naming of scripts/convert_pi05_to_gguf.py, pinned by
tests/golden/gguf_names.json "pi05"): load -> config -> predict from image embeddings and from camera views ->
actions un-normalised by quantiles, against the CPU oracle run the way src/models/pi05.cpp:505-705 runs a request
(prefix = [image embeddings ; E[lang] * sqrt(hidden)], Gemma prefill without mask, adaptive-norm expert loop).

Bar: rel-L2 <= 1e-2 on the final action chunk."""
import json
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

gguf = pytest.importorskip("gguf")

from tests.gpu_util import rel_l2, require_cuda
from tests.test_pi05_gpu import make_pi05
from tests.test_predict_gpu import tower_geometry, write_tower
from tests.test_prefill_gpu import make_vlm
from tests.test_vision_gpu import make_tower

GOLDEN = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "gguf_names.json")))["pi05"]


def write_pi05(path, oracle, rng, tower):
    hidden, n_q, n_kv, hd, inter, L = 256, 4, 1, 64, 512, 3
    cfg, w = make_pi05(oracle, rng, L=L, H=128, n_q=n_q, n_kv=n_kv, hd=hd, inter=384, chunk=10, A=32, T=3)
    vlm = make_vlm(oracle, rng, L, hidden, n_q, n_kv, hd, inter)
    vocab, n_lang_max = 300, 12
    emb = oracle.bf16_round((rng.standard_normal((vocab, hidden)) * 0.05).astype(np.float32))
    q01, q99 = rng.uniform(-2, -1, 7).astype(np.float32), rng.uniform(1, 2, 7).astype(np.float32)
    tcfg = tower_geometry("pi0", hidden, 256) if tower else None
    if tcfg:
        tcfg["out_scale"] = 0.0  # pi0.5 takes the projector's raw output (src/models/pi05.cpp:572-577)
    tw = make_tower(oracle, rng, tcfg, connector_bias=True) if tower else None
    F32, BF16 = gguf.GGMLQuantizationType.F32, gguf.GGMLQuantizationType.BF16
    wr = gguf.GGUFWriter(str(path), "pi05")
    keys = {k for k, _ in GOLDEN["kv"]}

    def kv(k):
        assert "pi05." + k in keys, k
        return "pi05." + k
    for key, val in (("hidden", hidden), ("intermediate", inter), ("n_q_heads", n_q), ("n_kv_heads", n_kv), ("head_dim", hd),
                     ("n_layers", L), ("expert_h", cfg["H"]), ("expert_inter", cfg["inter"]), ("chunk_size", cfg["chunk"]),
                     ("num_steps", cfg["steps"]), ("max_state_dim", 32), ("max_action_dim", 32), ("real_state_dim", 8),
                     ("real_action_dim", 7), ("tokenizer_max_length", n_lang_max), ("adarms_cond_dim", cfg["H"])):
        wr.add_uint32(kv(key), val)
    wr.add_bool(kv("use_adarms_expert"), True)
    wr.add_string(kv("norm_mode"), "quantiles")
    wr.add_float64(kv("min_period"), cfg["min_period"])
    wr.add_float64(kv("max_period"), cfg["max_period"])
    wr.add_float64(kv("rope_theta"), cfg["rope_base"])
    wr.add_float32(kv("rms_norm_eps"), cfg["rms_eps"])
    names = {n.replace(".blk.1.", ".blk.0.") for n, _, _ in GOLDEN["decoder_blocks"]} | set(GOLDEN["projections"]) | set(GOLDEN["output_norm"])

    def mat(name, a):
        wr.add_tensor(name, oracle.f32_to_bf16_bits(a).astype(np.uint16), raw_shape=list(a.shape), raw_dtype=BF16)

    def vec(name, a):
        wr.add_tensor(name, np.ascontiguousarray(a, dtype=np.float32), raw_dtype=F32)

    def put(fn, name, a):
        base = name.split(".")
        probe = ".".join(["aex", "blk", "0"] + base[3:]) if name.startswith("aex.blk.") else name
        assert probe in names, name
        fn(name, a)
    for l, lw in enumerate(w["layers"]):
        b = f"aex.blk.{l}."
        for ours, theirs, fn in (("ada_in_w", "attn_norm.weight", vec), ("ada_in_b", "attn_norm.bias", vec),
                                 ("ada_post_w", "ffn_norm.weight", vec), ("ada_post_b", "ffn_norm.bias", vec),
                                 ("wq", "attn_q.weight", mat), ("wk", "attn_k.weight", mat), ("wv", "attn_v.weight", mat),
                                 ("wo", "attn_o.weight", mat), ("wgate", "ffn_gate.weight", mat), ("wup", "ffn_up.weight", mat),
                                 ("wdown", "ffn_down.weight", mat)):
            put(fn, b + theirs, lw[ours])
    put(vec, "aex.output_norm.weight", w["ada_final_w"])
    put(vec, "aex.output_norm.bias", w["ada_final_b"])
    for ours, theirs in (("w_ain", "action_in_proj"), ("w_tin", "time_mlp_in"), ("w_tout", "time_mlp_out"), ("w_aout", "action_out_proj")):
        put(vec if ours in ("w_tin", "w_tout") else mat, theirs + ".weight", w[ours])
        put(vec, theirs + ".bias", w["b_" + ours[2:]])
    for l, lw in enumerate(vlm):
        for suffix, key in (("attn_norm.weight", "ln_in"), ("attn_q.weight", "wq"), ("attn_k.weight", "wk"), ("attn_v.weight", "wv"),
                            ("attn_o.weight", "wo"), ("ffn_norm.weight", "ln_post"), ("ffn_gate.weight", "wgate"),
                            ("ffn_up.weight", "wup"), ("ffn_down.weight", "wdown")):
            a = lw[key]
            (vec if "norm" in suffix else mat)(f"vlm.blk.{l}.{suffix}", (a - np.float32(1)).astype(np.float32) if "norm" in suffix else a)
    mat("token_embd.weight", emb)
    vec("action_q01", q01)
    vec("action_q99", q99)
    if tower:
        write_tower(wr, kv, mat, vec, "pi0", tcfg, tw)
    wr.write_header_to_file()
    wr.write_kv_data_to_file()
    wr.write_tensors_to_file()
    wr.close()
    return cfg, w, vlm, emb, (q01, q99), dict(hidden=hidden, n_q=n_q, n_kv=n_kv, hd=hd, tower_cfg=tcfg, tower=tw)


@pytest.mark.parametrize("n_views,n_lang,pixels", [(1, 7, False), (2, 12, False), (2, 9, True)])
def test_pi05_predict_against_the_oracle(oracle, tmp_path, n_views, n_lang, pixels):
    require_cuda()
    import vla_cpp_b200 as vb

    rng = np.random.default_rng(23 + n_views + n_lang)
    path = tmp_path / "pi05.gguf"
    cfg, w, vlm, emb, (q01, q99), d = write_pi05(path, oracle, rng, tower=pixels)
    model = vb.VlaModel(path)
    hidden = d["hidden"]
    lang = rng.integers(0, emb.shape[0], n_lang).astype(np.int32)
    noise = rng.standard_normal((cfg["chunk"], 32)).astype(np.float32)
    state = np.zeros(32, np.float32)
    if pixels:
        side = d["tower_cfg"]["image"]
        views = [rng.integers(0, 256, (side, side, 3), dtype=np.uint8) for _ in range(n_views)]
        img = np.concatenate([oracle.siglip_tower(a, d["tower"], d["tower_cfg"]) for a in views]).astype(np.float32)
        got = model.predict(lang, state, images=views, noise=noise)
        assert model.stats.ms_vision > 0
    else:
        img = (rng.standard_normal((256 * n_views, hidden)) * 0.5).astype(np.float32)
        got = model.predict(lang, state, img_emb=img, n_views=n_views, noise=noise)
    again = model.predict(lang, state, images=views, noise=noise) if pixels else model.predict(lang, state, img_emb=img, n_views=n_views, noise=noise)
    assert np.array_equal(got, again)
    # ---- the same request through the oracle ----
    x = np.concatenate([img, emb[lang] * np.float32(np.sqrt(np.float32(hidden)))]).astype(np.float32)
    ocfg = dict(n_q=d["n_q"], n_kv=d["n_kv"], hd=d["hd"], rms_eps=cfg["rms_eps"], rope_base=cfg["rope_base"], act="gelu")
    ks, vs = oracle.vlm_prefill(x, vlm, ocfg)
    pcfg = dict(H=cfg["H"], n_q=cfg["n_q"], n_kv=cfg["n_kv"], hd=cfg["head_dim"], steps=cfg["steps"], rms_eps=cfg["rms_eps"],
                rope_base=cfg["rope_base"], min_period=cfg["min_period"], max_period=cfg["max_period"])
    ref = oracle.pi05_denoise(ks, vs, noise, w, pcfg)
    want = np.zeros_like(ref)
    want[:, :7] = (ref[:, :7] + np.float32(1)) * (q99 - q01) * np.float32(0.5) + q01
    assert np.all(got[:, 7:] == 0)
    err = rel_l2(got, want)
    print(f"vla_predict pi05 views={n_views} n_lang={n_lang} pixels={pixels}: rel_l2 {err:.3e}; vision {model.stats.ms_vision:.2f} ms, "
          f"prefill {model.stats.ms_prefill:.2f} ms, denoise {model.stats.ms_denoise:.2f} ms")
    assert err <= 1e-2, err
