"""vla_predict end to end through include/vla.h (ABI v1) on a synthetic checkpoint: GGUF file -> vla_model_load ->
vla_model_config -> vla_predict (image embeddings given, as vla_inputs.precomputed_img_emb allows) ->
vla_free_actions, against the CPU oracle run the way the reference's predict runs it
(src/models/pi0.cpp:451-681, src/models/smolvla.cpp:1476-1710): state normalisation, prefix embeddings and their
scales, prefill masks / positions, the denoise loop, action un-normalisation, zeroed padding columns.

Bar: rel-L2 <= 1e-2 on the final action chunk (north-star tolerance)."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

gguf = pytest.importorskip("gguf")

from tests.gpu_util import rel_l2, require_cuda
from tests.test_engine_gpu import make_policy, oracle_model
from tests.test_gguf_engine_gpu import _write_policy
from tests.test_prefill_gpu import make_vlm
from tests.test_vision_gpu import make_tower


class VlaImage(C.Structure):
    _fields_ = [("data", C.c_void_p), ("w", C.c_int32), ("h", C.c_int32), ("format", C.c_int32)]


class VlaInputs(C.Structure):
    _fields_ = [("images", C.POINTER(VlaImage)), ("n_images", C.c_int32), ("precomputed_img_emb", C.POINTER(C.c_float)),
                ("n_img_views", C.c_int32), ("lang_tokens", C.POINTER(C.c_int32)), ("n_lang", C.c_int32),
                ("state", C.POINTER(C.c_float)), ("noise", C.POINTER(C.c_float)), ("attention_mask", C.POINTER(C.c_int32)),
                ("attention_mask_n", C.c_int32), ("timing_detail", C.c_int32)]


class VlaStats(C.Structure):
    _fields_ = [(n, C.c_float) for n in ("ms_total", "ms_vision", "ms_inference", "ms_prefill", "ms_denoise")]


def fptr(a):
    return a.ctypes.data_as(C.POINTER(C.c_float))


def tower_geometry(arch, hidden, n_img):
    """A narrow SigLIP tower whose token count matches the checkpoint: pi0 needs 256 tokens per view and gets head_dim 72
    (the So400m value, padded inside the library); SmolVLA gets a pixel shuffle of 2."""
    if arch == "pi0":
        return dict(image=64, patch=4, hidden=144, n_layers=2, n_heads=2, inter=256, shuffle=1, out_dim=hidden, ln_eps=1e-6,
                    out_scale=float(np.float32(1) / np.sqrt(np.float32(hidden))))
    side = int(round(n_img ** 0.5)) * 2 * 16
    return dict(image=side, patch=16, hidden=128, n_layers=2, n_heads=2, inter=256, shuffle=2, out_dim=hidden, ln_eps=1e-6,
                out_scale=0.0)


def write_tower(w, kv, mat, vec, arch, tcfg, tw):
    """Tensor names and metadata keys of the converters (tests/golden/gguf_names.json "vision")."""
    import json
    import os

    golden = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "gguf_names.json")))["vision"]
    names = {n for n, _, _ in golden["tower"]} | set(golden["connector_smolvla"]) | set(golden["connector_pi0"])
    w.add_uint32(kv("vit_hidden"), tcfg["hidden"])
    w.add_uint32(kv("vit_layers"), tcfg["n_layers"])
    w.add_uint32(kv("vit_heads"), tcfg["n_heads"])
    w.add_uint32(kv("image_size"), tcfg["image"])
    w.add_uint32(kv("patch_size"), tcfg["patch"])
    w.add_float32(kv("vit_ln_eps"), tcfg["ln_eps"])
    if arch == "smolvla":
        w.add_uint32(kv("vit_inter"), tcfg["inter"])
        w.add_uint32(kv("vit_pixel_shuffle"), tcfg["shuffle"])
    else:
        w.add_uint32(kv("n_img_tokens"), (tcfg["image"] // tcfg["patch"]) ** 2)

    def put(fn, name, a):
        assert name.replace(".blk.1.", ".blk.0.") in names, name
        fn(name, a)
    put(vec, "vit.patch_embd.weight", tw["patch_w"])
    put(vec, "vit.patch_embd.bias", tw["patch_b"])
    put(vec, "vit.pos_embd", tw["pos"])
    put(vec, "vit.post_ln.weight", tw["post_w"])
    put(vec, "vit.post_ln.bias", tw["post_b"])
    for l, lw in enumerate(tw["layers"]):
        b = f"vit.blk.{l}."
        for ours, theirs in (("ln1_w", "ln1.weight"), ("ln1_b", "ln1.bias"), ("ln2_w", "ln2.weight"), ("ln2_b", "ln2.bias"),
                             ("bq", "attn_q.bias"), ("bk", "attn_k.bias"), ("bv", "attn_v.bias"), ("bo", "attn_o.bias"),
                             ("b1", "fc1.bias"), ("b2", "fc2.bias")):
            put(vec, b + theirs, lw[ours])
        for ours, theirs in (("wq", "attn_q"), ("wk", "attn_k"), ("wv", "attn_v"), ("wo", "attn_o"), ("fc1", "fc1"), ("fc2", "fc2")):
            put(mat, b + theirs + ".weight", lw[ours])
    if arch == "smolvla":
        put(mat, "mm.fc.weight", tw["connector"])
    else:
        put(mat, "mm.proj.weight", tw["connector"])
        put(vec, "mm.proj.bias", tw["connector_b"])


def build_checkpoint(oracle, tmp_path, arch, rng, tower=False):
    """A small but complete checkpoint in the reference's naming: backbone layers, expert, embeddings, statistics and,
    with tower=True, the SigLIP tower and its connector."""
    if arch == "pi0":
        hidden, n_q, n_kv, hd, inter, L = 256, 4, 1, 64, 512, 3
        cfg, per, glob, wqkv = make_policy(oracle, rng, model=0, L=L, H=128, n_q=n_q, n_kv=n_kv, hd=hd, inter=256, P=1,
                                           chunk=10, A=32, sd=32, T=3)
        off, n_lang_max, n_img = np.float32(1), 12, 256
    else:
        hidden, n_q, n_kv, hd, inter, L = 192, 6, 2, 64, 256, 4
        cfg, per, glob, wqkv = make_policy(oracle, rng, model=1, L=L, H=128, n_q=n_q, n_kv=n_kv, hd=hd, inter=256, P=1,
                                           chunk=10, A=32, sd=32, T=3, self_every=2)
        off, n_lang_max, n_img = np.float32(0), 9, 16
    per["ln_raw_in"] = [(a - off).astype(np.float32) for a in per["ln_in"]]
    per["ln_raw_post"] = [(a - off).astype(np.float32) for a in per["ln_post"]]
    per["ln_in"] = [a + off for a in per["ln_raw_in"]]
    per["ln_post"] = [a + off for a in per["ln_raw_post"]]
    glob["out_norm_raw"] = (glob["out_norm"] - off).astype(np.float32)
    glob["out_norm"] = glob["out_norm_raw"] + off
    vlm = make_vlm(oracle, rng, L, hidden, n_q, n_kv, hd, inter)
    vocab = 300
    emb = oracle.bf16_round((rng.standard_normal((vocab, hidden)) * 0.05).astype(np.float32))
    stats = dict(state_mean=rng.standard_normal(8).astype(np.float32), state_std=rng.uniform(0.5, 2, 8).astype(np.float32),
                 action_mean=rng.standard_normal(7).astype(np.float32), action_std=rng.uniform(0.5, 2, 7).astype(np.float32))
    w_state = (rng.standard_normal((hidden, 32)) * 0.1).astype(np.float32)
    b_state = (rng.standard_normal(hidden) * 0.1).astype(np.float32)
    tcfg = tower_geometry(arch, hidden, n_img) if tower else None
    tw = make_tower(oracle, rng, tcfg, connector_bias=arch == "pi0") if tower else None

    def extra(w, kv, mat, vec):
        if tower:
            write_tower(w, kv, mat, vec, arch, tcfg, tw)
        w.add_uint32(kv("intermediate"), inter)
        w.add_uint32(kv("real_state_dim"), 8)
        w.add_uint32(kv("real_action_dim"), 7)
        w.add_uint32(kv("tokenizer_max_length"), n_lang_max)
        if arch == "smolvla":
            w.add_uint32(kv("n_img_tokens"), n_img)
        for l, lw in enumerate(vlm):
            for suffix, key in (("attn_norm.weight", "ln_in"), ("attn_q.weight", "wq"), ("attn_k.weight", "wk"),
                                ("attn_v.weight", "wv"), ("attn_o.weight", "wo"), ("ffn_norm.weight", "ln_post"),
                                ("ffn_gate.weight", "wgate"), ("ffn_up.weight", "wup"), ("ffn_down.weight", "wdown")):
                a = lw[key]
                (vec if "norm" in suffix else mat)(f"vlm.blk.{l}.{suffix}", (a - off).astype(np.float32) if "norm" in suffix else a)
        mat("token_embd.weight", emb)
        if arch == "smolvla":
            vec("state_proj.weight", w_state)
            vec("state_proj.bias", b_state)
        for k, v in stats.items():
            vec(k, v)

    path = tmp_path / (arch + "_full.gguf")
    _write_policy(path, oracle, cfg, per, glob, True, arch, extra=extra, hidden=hidden)
    dims = dict(hidden=hidden, n_q=n_q, n_kv=n_kv, hd=hd, n_lang_max=n_lang_max, n_img=n_img, tower_cfg=tcfg, tower=tw)
    return path, cfg, per, glob, wqkv, vlm, emb, stats, (w_state, b_state), dims


@pytest.mark.parametrize("arch,n_views,n_lang", [("pi0", 1, 7), ("pi0", 2, 12), ("smolvla", 2, 5), ("smolvla", 1, 9)])
def test_vla_predict_against_the_oracle(oracle, tmp_path, arch, n_views, n_lang):
    run_predict_case(oracle, tmp_path, arch, n_views, n_lang, pixels=None)


@pytest.mark.parametrize("arch,n_views,n_lang,pixels", [("pi0", 1, 7, "u8"), ("pi0", 2, 9, "mixed"), ("smolvla", 2, 5, "f32"),
                                                        ("smolvla", 2, 6, "mixed")])
def test_vla_predict_from_camera_views(oracle, tmp_path, arch, n_views, n_lang, pixels):
    """vla_inputs.images through the library's own vision tower (checkpoint with vit.* / mm.* tensors); the oracle runs
    its SigLIP restatement on the same pixels and then the same prefill and denoise loop."""
    run_predict_case(oracle, tmp_path, arch, n_views, n_lang, pixels=pixels)


def run_predict_case(oracle, tmp_path, arch, n_views, n_lang, pixels):
    require_cuda()
    import vla_cpp_b200 as vb

    L = vb.lib()
    L.vla_model_load.restype = C.c_void_p
    L.vla_model_load.argtypes = [C.c_char_p, C.c_char_p, C.c_char_p]
    L.vla_model_free.argtypes = [C.c_void_p]
    L.vla_predict.argtypes = [C.c_void_p, C.POINTER(VlaInputs), C.POINTER(C.POINTER(C.c_float)), C.POINTER(C.c_int64)]
    L.vla_free_actions.argtypes = [C.POINTER(C.c_float)]
    L.vla_last_stats.argtypes = [C.c_void_p, C.POINTER(VlaStats)]

    rng = np.random.default_rng(17 + n_views + n_lang)
    path, cfg, per, glob, wqkv, vlm, emb, stats, (w_state, b_state), d = build_checkpoint(oracle, tmp_path, arch, rng,
                                                                                           tower=pixels is not None)
    m = L.vla_model_load(None, str(path).encode(), None)
    assert m, L.vlab200_last_error()
    hidden, n_img = d["hidden"], d["n_img"] * n_views
    views, keep = [], []
    if pixels is None:
        img = (rng.standard_normal((n_img, hidden)) * 0.5).astype(np.float32)
    else:
        side = d["tower_cfg"]["image"]
        for v in range(n_views):
            as_f32 = pixels == "f32" or (pixels == "mixed" and v % 2 == 1)
            u8 = rng.integers(0, 256, (side, side, 3), dtype=np.uint8)
            views.append(np.ascontiguousarray(u8.astype(np.float32) / np.float32(255)) if as_f32 else u8)
        img = np.concatenate([oracle.siglip_tower(a, d["tower"], d["tower_cfg"]) for a in views]).astype(np.float32)
        assert img.shape == (n_img, hidden)
    lang = rng.integers(0, emb.shape[0], n_lang).astype(np.int32)
    state = np.zeros(32, np.float32)
    state[:8] = rng.standard_normal(8)
    noise = rng.standard_normal((cfg["chunk"], 32)).astype(np.float32)
    inp = VlaInputs()
    if pixels is None:
        inp.precomputed_img_emb, inp.n_img_views = fptr(img), n_views
    else:
        arr = (VlaImage * n_views)()
        for v, a in enumerate(views):
            arr[v].data, arr[v].w, arr[v].h, arr[v].format = a.ctypes.data, a.shape[1], a.shape[0], int(a.dtype == np.float32)
        keep.append(arr)
        inp.images, inp.n_images = arr, n_views
    inp.lang_tokens, inp.n_lang = lang.ctypes.data_as(C.POINTER(C.c_int32)), n_lang
    inp.state, inp.noise, inp.timing_detail = fptr(state), fptr(noise), 1
    act, n = C.POINTER(C.c_float)(), C.c_int64(0)
    rc = L.vla_predict(m, C.byref(inp), C.byref(act), C.byref(n))
    assert rc == 0, (rc, L.vlab200_last_error())
    assert n.value == cfg["chunk"] * 32
    got = np.ctypeslib.as_array(act, shape=(n.value,)).reshape(cfg["chunk"], 32).copy()
    L.vla_free_actions(act)
    st = VlaStats()
    assert L.vla_last_stats(m, C.byref(st)) == 0
    assert st.ms_total > 0 and st.ms_prefill > 0 and st.ms_denoise > 0
    assert (st.ms_vision > 0) == (pixels is not None)

    # a second call with the same noise reproduces the result bit for bit; without noise it is sampled internally
    rc = L.vla_predict(m, C.byref(inp), C.byref(act), C.byref(n))
    assert rc == 0
    again = np.ctypeslib.as_array(act, shape=(n.value,)).reshape(cfg["chunk"], 32).copy()
    L.vla_free_actions(act)
    assert np.array_equal(got, again)
    inp.noise = None
    assert L.vla_predict(m, C.byref(inp), C.byref(act), C.byref(n)) == 0
    sampled = np.ctypeslib.as_array(act, shape=(n.value,)).reshape(cfg["chunk"], 32).copy()
    L.vla_free_actions(act)
    assert np.isfinite(sampled).all() and not np.array_equal(sampled, got)
    # out-of-vocabulary token ids are refused before any gather
    bad = lang.copy()
    bad[0] = emb.shape[0]
    inp.lang_tokens = bad.ctypes.data_as(C.POINTER(C.c_int32))
    assert L.vla_predict(m, C.byref(inp), C.byref(act), C.byref(n)) == -2
    L.vla_model_free(m)

    # ---- the same request through the oracle, as the reference's predict assembles it ----
    sn = state.copy()
    sn[:8] = (sn[:8] - stats["state_mean"]) / (stats["state_std"] + np.float32(1e-8))
    scale = np.float32(np.sqrt(np.float32(hidden)))
    ocfg = dict(n_q=d["n_q"], n_kv=d["n_kv"], hd=d["hd"], rms_eps=cfg["rms_eps"], rope_base=cfg["rope_base"],
                act="gelu" if arch == "pi0" else "silu")
    if arch == "pi0":
        x = np.concatenate([img, emb[lang] * scale])
        P = x.shape[0]
        ks, vs = oracle.vlm_prefill(x, vlm, ocfg)
        om = oracle_model(oracle, cfg, per, glob, wqkv, P, P, (0, 0))
    else:
        ids = np.zeros(d["n_lang_max"], np.int64)
        ids[:n_lang] = lang
        state_tok = (w_state @ sn + b_state).astype(np.float32)
        x = np.concatenate([img * scale, emb[ids] * scale, state_tok[None]]).astype(np.float32)
        P = x.shape[0]
        pos = np.arange(P, dtype=np.int32)
        pos[-1] = n_img + n_lang
        pad = (n_img + n_lang, n_img + d["n_lang_max"])
        ks, vs = oracle.vlm_prefill(x, vlm, ocfg, pos=pos, mask_mode=3, pad=pad)
        for l in range(cfg["n_layers"]):
            if l % cfg["self_every"] != 0:  # the oracle's loop applies expert_cross_kv itself from the raw prefix K/V
                pass
        om = oracle_model(oracle, cfg, per, glob, wqkv, P, n_img + n_lang + 1, pad)
    ref = om.denoise(ks, vs, sn, noise)
    want = np.zeros_like(ref)
    want[:, :7] = ref[:, :7] * (stats["action_std"] + np.float32(1e-8)) + stats["action_mean"]
    assert np.all(got[:, 7:] == 0)
    err = rel_l2(got, want)
    print(f"vla_predict {arch} views={n_views} n_lang={n_lang} pixels={pixels}: rel_l2 {err:.3e}; vision {st.ms_vision:.2f} ms, "
          f"prefill {st.ms_prefill:.2f} ms, denoise {st.ms_denoise:.2f} ms")
    assert err <= 1e-2, err
