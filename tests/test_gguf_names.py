"""Checkpoint naming pinned to the reference's converters.  tests/golden/gguf_names.json was recorded by calling
the converters' own functions (scripts/gguf_blocks.py, scripts/convert_{pi0,smolvla,bitvla}_to_gguf.py) with a
recording writer (tests/golden/make_golden.py); here a file carrying exactly those metadata keys, with the types the
converters use, must load through vla_model_load, and the loader must resolve its values.  Host only."""
import ctypes as C
import json
import os

import numpy as np
import pytest

gguf = pytest.importorskip("gguf")
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = json.load(open(os.path.join(ROOT, "tests", "golden", "gguf_names.json")))

VALUES = dict(hidden=2048, intermediate=16384, n_q_heads=8, n_kv_heads=1, head_dim=256, n_layers=18, expert_h=1024,
              expert_inter=4096, chunk_size=50, num_steps=10, max_state_dim=32, max_action_dim=32, real_state_dim=8,
              real_action_dim=7, tokenizer_max_length=48, self_attn_every_n_layers=2, n_img_tokens=64,
              min_period=4e-3, max_period=4.0, rope_theta=10000.0, rms_norm_eps=1e-6, norm_eps=1e-8)


def write_metadata_only(path, arch):
    """Every key of the reference converter, written with the converter's type; values where the loader reads them."""
    g = GOLDEN[arch]
    w = gguf.GGUFWriter(str(path), g["arch"])
    for key, kind in g["kv"]:
        short = key.split(".", 1)[1]
        if kind == "string":
            w.add_string(key, "x")
        elif kind == "bool":
            w.add_bool(key, True)
        else:
            getattr(w, "add_" + kind)(key, VALUES.get(short, 1))
    w.add_tensor("dummy", np.zeros(4, np.float32))
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()


@pytest.mark.parametrize("arch", ["pi0", "smolvla", "pi05"])
def test_a_file_with_the_converters_metadata_keys_loads(tmp_path, arch):
    import vla_cpp_b200

    L = vla_cpp_b200.lib()
    L.vla_model_load.restype = C.c_void_p
    L.vla_model_load.argtypes = [C.c_char_p, C.c_char_p, C.c_char_p]
    L.vla_model_free.argtypes = [C.c_void_p]
    path = tmp_path / (arch + ".gguf")
    write_metadata_only(path, arch)
    m = L.vla_model_load(None, str(path).encode(), None)
    assert m, L.vlab200_last_error()
    L.vla_model_free(m)


def test_expert_tensor_names_are_the_converters():
    """The names the engine loader asks for are the ones write_decoder_blocks(..., "aex", n) and PROJ_SUFFIXES give."""
    src = open(os.path.join(ROOT, "vla_cpp_b200", "csrc", "gguf.cu")).read()
    for arch in ("pi0", "smolvla"):
        g = GOLDEN[arch]
        for name, _, _ in g["decoder_blocks"]:
            suffix = name.split(".", 3)[3]  # aex.blk.N.<suffix>
            assert name.startswith("aex.blk.") and '"' + suffix + '"' in src, name
        for name in g["projections"] + [g["output_norm"]]:
            if arch == "smolvla" and name.startswith("state_proj"):
                continue  # SmolVLA's state token belongs to the prefix, not to the denoise loop
            assert '"' + name + '"' in src, name


def test_bitvla_pack_naming_is_the_converters():
    src = open(os.path.join(ROOT, "vla_cpp_b200", "csrc", "bitvla_lm.cu")).read()
    names = {n: (t, shape) for n, t, shape in GOLDEN["bitvla"]["packed"]}
    assert names["lm.blk.0.attn_q.weight"] == ("I8", [16 * 128 // 4]) and names["lm.blk.0.attn_q.scale"] == ("F32", [1])
    assert names["lm.blk.0.ffn_gate_up.weight"] == ("I8", [2 * 16 * 128 // 4])
    assert names["lm.blk.0.ffn_gate_up.scale"] == ("F32", [2])
    assert '"' + GOLDEN["bitvla"]["packed_flag_key"] + '"' in src
    for piece in ('"attn_q"', '"ffn_gate_up"', '".weight"', '".scale"', '"lm.blk."'):
        assert piece in src, piece


TINY = dict(hidden=64, intermediate=128, n_q_heads=2, n_kv_heads=1, head_dim=64, n_layers=2, vocab_size=32, expert_h=64,
            expert_inter=128, chunk_size=4, num_steps=2, vit_hidden=64, vit_layers=1, vit_heads=1, vit_inter=128,
            image_size=32, patch_size=16, vit_pixel_shuffle=1)


@pytest.mark.parametrize("arch", ["pi0", "smolvla", "pi05"])
def test_the_random_init_writer_uses_the_converters_names(tmp_path, arch):
    """vla_cpp_b200.synth_gguf writes only metadata keys and tensor names that the reference's converters write, and
    the file resolves through vla_model_load / vla_model_config.  Host only."""
    import vla_cpp_b200
    from vla_cpp_b200 import synth_gguf

    path = tmp_path / (arch + "_tiny.gguf")
    dims = dict(TINY)
    if arch != "smolvla":
        dims.update(image_size=224, patch_size=14)  # pi0 / pi0.5 fix 256 image tokens per view (src/models/pi0.cpp:286)
    d = synth_gguf.write_checkpoint(path, arch, dims=dims)
    g = GOLDEN[arch]
    kv_names = {k for k, _ in g["kv"]}
    block = {n.split(".", 3)[3] for n, _, _ in g["decoder_blocks"]}
    vision = {n.replace("vit.blk.0.", "") for n, _, _ in GOLDEN["vision"]["tower"]}
    conn = set(GOLDEN["vision"]["connector_" + ("smolvla" if arch == "smolvla" else "pi0")])
    r = gguf.GGUFReader(str(path))
    for k in r.fields:
        if k.startswith(arch + "."):
            assert k in kv_names, k
    for t in r.tensors:
        n = t.name
        if n.startswith(("vlm.blk.", "aex.blk.")):
            assert n.split(".", 3)[3] in block, n
        elif n.startswith("vit.blk."):
            assert n.split(".", 3)[3] in vision, n
        elif n.startswith("vit."):
            assert n in vision, n
        elif n.startswith("mm."):
            assert n in conn, n
        elif n in g["projections"]:
            pass
        else:
            out_norm = g["output_norm"] if isinstance(g["output_norm"], list) else [g["output_norm"]]
            assert n in ["token_embd.weight", "vlm.output_norm.weight", "state_mean", "state_std", "action_mean", "action_std",
                         "action_q01", "action_q99"] + out_norm, n
    L = vla_cpp_b200.lib()
    L.vla_model_load.restype = C.c_void_p
    L.vla_model_load.argtypes = [C.c_char_p, C.c_char_p, C.c_char_p]
    L.vla_model_free.argtypes = [C.c_void_p]
    m = L.vla_model_load(None, str(path).encode(), None)
    assert m, L.vlab200_last_error()
    L.vla_model_free(m)
    assert d["n_img_tokens"] == (4 if arch == "smolvla" else 256)
