"""Regenerates the golden fixtures in this directory from the reference itself.

Runs only where the reference tree is mounted (it is never needed at test time):
  python tests/golden/make_golden.py [/path/to/reference]

* ladder_pack.npz  -- scripts/convert_bitvla_to_gguf.py (imported as a module):
                      weight_quant_to_ternary() and pack_ladder_int2() applied to
                      seeded random matrices.
* time_emb.npz     -- src/layers/embed.h sinusoidal_time_emb(), through the driver
                      oracle/_ref/time_emb_ref (built by oracle/Makefile).
"""
import os
import subprocess
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def ladder(ref):
    import torch

    sys.path.insert(0, os.path.join(ref, "scripts"))
    import convert_bitvla_to_gguf as conv

    out = {}
    rng = np.random.default_rng(20240521)
    for i, (n, k) in enumerate([(16, 128), (32, 256), (48, 384), (64, 128)]):
        w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
        if i == 3:
            w[:] = 1e-7  # exercises the absmean floor of 1e-5
        tern, absmean = conv.weight_quant_to_ternary(torch.from_numpy(w))
        packed = conv.pack_ladder_int2(tern)
        out[f"w{i}"] = w
        out[f"tern{i}"] = tern.astype(np.int8)
        out[f"absmean{i}"] = np.float32(absmean)
        out[f"packed{i}"] = packed.astype(np.uint8)
    # fused projection: per-part scales, rows concatenated
    parts = [torch.from_numpy((rng.standard_normal((16, 128)) * s).astype(np.float32)) for s in (0.02, 0.05)]
    packed, scales = conv.pack_fused_projection(parts)
    out["fused_w0"], out["fused_w1"] = parts[0].numpy(), parts[1].numpy()
    out["fused_packed"], out["fused_scales"] = packed.astype(np.uint8), scales.astype(np.float32)
    np.savez_compressed(os.path.join(HERE, "ladder_pack.npz"), **out)


def time_emb():
    exe = os.path.join(ROOT, "oracle", "_ref", "time_emb_ref")
    out = {}
    cases = []
    for dim in (720, 1024, 2, 8):
        for step in range(10):
            # pi0 evaluates the timestep in float32, SmolVLA in double
            dt = np.float32(-1.0) / np.float32(10)
            cases.append((float(np.float32(1.0) + np.float32(step) * dt), dim, 4e-3, 4.0))
            cases.append((1.0 + float(step) * float(dt), dim, 4e-3, 4.0))
    args, vals = [], []
    for t, dim, mn, mx in cases:
        txt = subprocess.run([exe, repr(t), str(dim), repr(mn), repr(mx)], check=True, capture_output=True, text=True).stdout
        bits = np.array([int(x, 16) for x in txt.split()], dtype=np.uint32)
        assert bits.size == dim
        args.append((t, dim, mn, mx))
        vals.append(bits.view(np.float32))
    out["args"] = np.array(args, dtype=np.float64)
    out["offsets"] = np.cumsum([0] + [v.size for v in vals]).astype(np.int64)
    out["values"] = np.concatenate(vals)
    np.savez_compressed(os.path.join(HERE, "time_emb.npz"), **out)


class _Recorder:
    """Stands in for gguf.GGUFWriter: records what the reference's converter functions would write."""

    def __init__(self):
        self.kv, self.tensors = [], []

    def add_tensor(self, name, data, raw_shape=None, raw_dtype=None):
        self.tensors.append([name, getattr(raw_dtype, "name", str(raw_dtype)),
                             [int(x) for x in (raw_shape if raw_shape is not None else data.shape)]])

    def __getattr__(self, attr):  # add_uint32 / add_float32 / add_float64 / add_string / add_bool
        if not attr.startswith("add_"):
            raise AttributeError(attr)
        return lambda key, value: self.kv.append([key, attr[4:]])


def gguf_names(ref):
    """Tensor names, dtypes and metadata keys as the reference's converters write them, recorded by calling the
    converters' own functions (scripts/gguf_blocks.py write_pi_kv / write_decoder_blocks, scripts/convert_pi0_to_gguf.py
    and convert_smolvla_to_gguf.py PROJ_SUFFIXES / _add_kv, scripts/convert_bitvla_to_gguf.py _add_bit /
    _add_bit_fused) on tiny tensors with a recording writer."""
    import json

    import torch

    sys.path.insert(0, os.path.join(ref, "scripts"))
    import convert_bitvla_to_gguf as cb
    import convert_pi0_to_gguf as cp
    import convert_pi05_to_gguf as cp5
    import convert_smolvla_to_gguf as cs
    import gguf_blocks as gb

    vit = dict(vit_hidden=8, vit_layers=1, vit_heads=1, vit_inter=8, image_size=32, patch_size=16, n_img_tokens=4,
               vit_ln_eps=1e-6, vit_pixel_shuffle=1)
    base = dict(hidden=8, intermediate=8, n_q_heads=1, n_kv_heads=1, head_dim=8, n_layers=2, vocab_size=16, expert_h=8,
                expert_inter=8, chunk_size=2, num_steps=2, n_action_steps=2, max_state_dim=8, max_action_dim=8,
                real_state_dim=8, real_action_dim=8, tokenizer_max_length=4, min_period=4e-3, max_period=4.0,
                rope_theta=10000.0, rms_norm_eps=1e-6, norm_eps=1e-8, paligemma_variant="gemma_2b",
                action_expert_variant="gemma_300m", self_attn_every_n_layers=2, expert_width_multiplier=0.75, vit=vit)
    tiny = lambda name: torch.zeros((2, 2), dtype=torch.bfloat16)
    out = {}
    r = _Recorder()
    gb.write_pi_kv(r, cp.KV, base)
    gb.write_decoder_blocks(r, tiny, "root", "aex", 2)
    out["pi0"] = {"arch": cp.ARCH, "kv": r.kv, "decoder_blocks": r.tensors, "projections": list(cp.PROJ_SUFFIXES),
                  "output_norm": "aex.output_norm.weight"}
    r = _Recorder()
    cs._add_kv(r, base)
    gb.write_decoder_blocks(r, tiny, "root", "aex", 2)
    out["smolvla"] = {"arch": cs.ARCH, "kv": r.kv, "decoder_blocks": r.tensors, "projections": list(cs.PROJ_SUFFIXES),
                      "output_norm": "aex.output_norm.weight"}
    r = _Recorder()
    w = torch.randn(16, 128)
    cb._add_bit(r, "lm.blk.0.attn_q", w)
    cb._add_bit_fused(r, "lm.blk.0.ffn_gate_up", [w, w])
    out["bitvla"] = {"packed": r.tensors, "packed_flag_key": "bitvla.quant.int2_packed"}
    # pi0.5: write_pi_kv(adarms=True) and the adaptive-norm expert blocks (scripts/convert_pi05_to_gguf.py:81-96,250-262)
    r = _Recorder()
    gb.write_pi_kv(r, cp5.KV, base, adarms=True)

    class _Sf:
        get_tensor = staticmethod(tiny)

    cp5._write_adarms_blocks(r, _Sf, 2)
    out["pi05"] = {"arch": cp5.ARCH, "kv": r.kv, "decoder_blocks": r.tensors, "projections": list(cp5.PROJ_SUFFIXES),
                   "output_norm": ["aex.output_norm.weight", "aex.output_norm.bias"]}
    # the SigLIP tower as both converters write it (scripts/gguf_blocks.py write_siglip_tower / write_paligemma_vision,
    # scripts/convert_smolvla_to_gguf.py:213-214), one layer
    r = _Recorder()
    gb.write_siglip_tower(r, tiny, "root", 1, f32_norms=True)
    out["vision"] = {"tower": r.tensors, "connector_smolvla": ["mm.fc.weight"],
                     "connector_pi0": ["mm.proj.weight", "mm.proj.bias"]}
    json.dump(out, open(os.path.join(HERE, "gguf_names.json"), "w"), indent=1)


def vla_h_layout(ref):
    """sizeof / offsetof of the reference's public C structs (its include/vla.h), as printed by tests/c/vla_h_layout.c."""
    import tempfile

    src = os.path.join(os.path.dirname(HERE), "c", "vla_h_layout.c")
    with tempfile.TemporaryDirectory() as d:
        exe = os.path.join(d, "layout")
        subprocess.run(["gcc", "-std=c99", "-I", os.path.join(ref, "include"), src, "-o", exe], check=True)
        txt = subprocess.run([exe], check=True, capture_output=True, text=True).stdout
    open(os.path.join(HERE, "vla_h_layout.txt"), "w").write(txt)


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <path of the vla.cpp source tree>")
    ref = sys.argv[1]
    ladder(ref)
    time_emb()
    vla_h_layout(ref)
    gguf_names(ref)
    print("golden fixtures written to", HERE)
