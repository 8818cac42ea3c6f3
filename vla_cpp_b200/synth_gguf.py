"""Random-init checkpoints in the reference's GGUF naming, for benchmarks and smoke runs without real weights.

Metadata keys and tensor names are the ones the reference's converters write and its loaders read
(scripts/convert_smolvla_to_gguf.py:103-136,199-217, scripts/gguf_blocks.py:60-86,104-142; name map
src/models/smolvla.cpp:648-756, shapes smolvla.cpp:1097-1236; pi0: src/models/pi0.cpp:258-293,424-437,
src/modules/gemma_expert.h:46-62, src/modules/siglip_vit.cpp:23-34, src/modules/encoder.cpp:26-48).
Matrices are N(0, sigma) in PyTorch order [out, in]; norm weights are 1 (stored as 0 for Gemma norms, whose
loader adds 1); biases N(0, sigma); dataset statistics mean 0 / std 1; `token_embd.weight` is always BF16
(smolvla.cpp:1097-1099).

    python -m vla_cpp_b200.synth_gguf smolvla /tmp/smolvla_random.gguf
"""
import sys

import numpy as np

SMOLVLA_DIMS = dict(
    hidden=960, intermediate=2560, n_q_heads=15, n_kv_heads=5, head_dim=64, n_layers=16, vocab_size=49280,
    expert_h=720, expert_inter=2048, chunk_size=50, num_steps=10, max_state_dim=32, max_action_dim=32,
    real_state_dim=32, real_action_dim=32, self_attn_every_n_layers=2, tokenizer_max_length=48,
    min_period=4e-3, max_period=4.0, norm_eps=1e-8,
    vit_hidden=768, vit_layers=12, vit_heads=12, vit_inter=3072, image_size=512, patch_size=16, vit_pixel_shuffle=4,
    vit_ln_eps=1e-6)

PI0_DIMS = dict(
    hidden=2048, intermediate=16384, n_q_heads=8, n_kv_heads=1, head_dim=256, n_layers=18, vocab_size=257152,
    expert_h=1024, expert_inter=4096, chunk_size=50, num_steps=10, max_state_dim=32, max_action_dim=32,
    real_state_dim=32, real_action_dim=32, tokenizer_max_length=48, min_period=4e-3, max_period=4.0, norm_eps=1e-8,
    rope_theta=10000.0, rms_norm_eps=1e-6,
    vit_hidden=1152, vit_layers=27, vit_heads=16, vit_inter=4304, image_size=224, patch_size=14, vit_pixel_shuffle=1,
    vit_ln_eps=1e-6)


def _bf16_bits(a):
    """float32 -> bfloat16 bit patterns, round to nearest even."""
    u = np.ascontiguousarray(a, np.float32).view(np.uint32)
    return ((u + (((u >> 16) & 1) + np.uint32(0x7FFF))) >> 16).astype(np.uint16)


def write_checkpoint(path, arch, dims=None, seed=0, sigma=0.02, matrix_dtype="f32"):
    """Writes a random-init `arch` ("smolvla" | "pi0") checkpoint to `path`; returns the dims used.

    matrix_dtype "f32" or "bf16" for the matrices other than the embedding table (both are accepted by the loader
    and held as bf16 on the device)."""
    import gguf

    assert arch in ("smolvla", "pi0", "pi05") and matrix_dtype in ("f32", "bf16")  # pi05: pi0's sizes
    d = dict(SMOLVLA_DIMS if arch == "smolvla" else PI0_DIMS)
    d.update(dims or {})
    rng = np.random.default_rng(seed)
    F32, BF16 = gguf.GGMLQuantizationType.F32, gguf.GGMLQuantizationType.BF16
    w = gguf.GGUFWriter(str(path), arch)
    kv = lambda k: arch + "." + k
    u32 = ["hidden", "intermediate", "n_q_heads", "n_kv_heads", "head_dim", "n_layers", "vocab_size", "expert_h",
           "expert_inter", "chunk_size", "num_steps", "max_state_dim", "max_action_dim", "real_state_dim",
           "real_action_dim", "tokenizer_max_length", "vit_hidden", "vit_layers", "vit_heads", "image_size", "patch_size"]
    grid = d["image_size"] // d["patch_size"]
    n_img_tokens = (grid // d["vit_pixel_shuffle"]) ** 2
    for k in u32:
        w.add_uint32(kv(k), int(d[k]))
    w.add_uint32(kv("n_img_tokens"), n_img_tokens)
    w.add_float64(kv("min_period"), d["min_period"])
    w.add_float64(kv("max_period"), d["max_period"])
    w.add_float32(kv("norm_eps"), d["norm_eps"])
    w.add_float32(kv("vit_ln_eps"), d["vit_ln_eps"])
    if arch == "smolvla":
        w.add_uint32(kv("self_attn_every_n_layers"), int(d["self_attn_every_n_layers"]))
        w.add_uint32(kv("vit_inter"), int(d["vit_inter"]))
        w.add_uint32(kv("vit_pixel_shuffle"), int(d["vit_pixel_shuffle"]))
    else:
        w.add_float64(kv("rope_theta"), d["rope_theta"])
        w.add_float32(kv("rms_norm_eps"), d["rms_norm_eps"])
    if arch == "pi05":  # scripts/gguf_blocks.py write_pi_kv(adarms=True)
        w.add_bool(kv("use_adarms_expert"), True)
        w.add_uint32(kv("adarms_cond_dim"), int(d["expert_h"]))
        w.add_string(kv("norm_mode"), "quantiles")

    def bf16(name, shape):
        a = rng.standard_normal(shape, dtype=np.float32) * np.float32(sigma)
        w.add_tensor(name, _bf16_bits(a), raw_shape=list(shape), raw_dtype=BF16)

    def mat(name, out, inp):
        if matrix_dtype == "bf16":
            bf16(name, (out, inp))
        else:
            w.add_tensor(name, rng.standard_normal((out, inp), dtype=np.float32) * np.float32(sigma), raw_dtype=F32)

    def vec(name, n, value=None):
        a = np.full(n, value, np.float32) if value is not None else rng.standard_normal(n, dtype=np.float32) * np.float32(sigma)
        w.add_tensor(name, a, raw_dtype=F32)

    norm_one = 1.0 if arch == "smolvla" else 0.0  # Gemma norms are stored without their +1
    H, I, hd = d["hidden"], d["intermediate"], d["head_dim"]
    qf, kvf = d["n_q_heads"] * hd, d["n_kv_heads"] * hd
    E, EI = d["expert_h"], d["expert_inter"]
    bf16("token_embd.weight", (d["vocab_size"], H))

    def ada_norm(name, width):
        # pi0.5: the norm is a dense map of the time conditioning, rows scale | shift | gate; biases give gate 1
        w.add_tensor(name + ".weight", rng.standard_normal((3 * width, width), dtype=np.float32) * np.float32(sigma), raw_dtype=F32)
        w.add_tensor(name + ".bias", np.concatenate([np.zeros(2 * width, np.float32), np.ones(width, np.float32)]), raw_dtype=F32)

    def decoder_block(prefix, width, inter, k_in, ada=False):
        if ada:
            ada_norm(prefix + "attn_norm", width)
            for q, rows, cols in (("attn_q", qf, width), ("attn_k", kvf, k_in), ("attn_v", kvf, k_in), ("attn_o", width, qf)):
                mat(prefix + q + ".weight", rows, cols)
            ada_norm(prefix + "ffn_norm", width)
            mat(prefix + "ffn_gate.weight", inter, width)
            mat(prefix + "ffn_up.weight", inter, width)
            mat(prefix + "ffn_down.weight", width, inter)
            return
        vec(prefix + "attn_norm.weight", width, norm_one)
        mat(prefix + "attn_q.weight", qf, width)
        mat(prefix + "attn_k.weight", kvf, k_in)
        mat(prefix + "attn_v.weight", kvf, k_in)
        mat(prefix + "attn_o.weight", width, qf)
        vec(prefix + "ffn_norm.weight", width, norm_one)
        mat(prefix + "ffn_gate.weight", inter, width)
        mat(prefix + "ffn_up.weight", inter, width)
        mat(prefix + "ffn_down.weight", width, inter)

    every = d.get("self_attn_every_n_layers", 0) if arch == "smolvla" else 0
    for i in range(d["n_layers"]):
        decoder_block(f"vlm.blk.{i}.", H, I, H)
        cross = every > 1 and i % every != 0  # cross-attention layers project the prefix K/V: [kvf, kvf]
        decoder_block(f"aex.blk.{i}.", E, EI, kvf if cross else E, ada=arch == "pi05")
    vec("vlm.output_norm.weight", H, norm_one)
    sd, ad = d["max_state_dim"], d["max_action_dim"]
    if arch == "pi05":
        ada_norm("aex.output_norm", E)
        heads = (("action_in_proj", E, ad), ("time_mlp_in", E, E), ("time_mlp_out", E, E), ("action_out_proj", ad, E))
    else:
        vec("aex.output_norm.weight", E, norm_one)
        heads = (("state_proj", H if arch == "smolvla" else E, sd), ("action_in_proj", E, ad),
                 ("action_time_mlp_in", E, 2 * E), ("action_time_mlp_out", E, E), ("action_out_proj", ad, E))
    for name, out, inp in heads:
        # the projection heads stay float32 in the reference
        w.add_tensor(name + ".weight", rng.standard_normal((out, inp), dtype=np.float32) * np.float32(sigma), raw_dtype=F32)
        vec(name + ".bias", out)
    # SigLIP tower and connector
    VH, VI, P = d["vit_hidden"], d["vit_inter"], d["patch_size"]
    w.add_tensor("vit.patch_embd.weight", rng.standard_normal((VH, 3, P, P), dtype=np.float32) * np.float32(sigma), raw_dtype=F32)
    vec("vit.patch_embd.bias", VH)
    w.add_tensor("vit.pos_embd", rng.standard_normal((grid * grid, VH), dtype=np.float32) * np.float32(sigma), raw_dtype=F32)
    for i in range(d["vit_layers"]):
        b = f"vit.blk.{i}."
        vec(b + "ln1.weight", VH, 1.0)
        vec(b + "ln1.bias", VH, 0.0)
        vec(b + "ln2.weight", VH, 1.0)
        vec(b + "ln2.bias", VH, 0.0)
        for q in ("q", "k", "v", "o"):
            mat(b + f"attn_{q}.weight", VH, VH)
            vec(b + f"attn_{q}.bias", VH)
        mat(b + "fc1.weight", VI, VH)
        vec(b + "fc1.bias", VI)
        mat(b + "fc2.weight", VH, VI)
        vec(b + "fc2.bias", VH)
    vec("vit.post_ln.weight", VH, 1.0)
    vec("vit.post_ln.bias", VH, 0.0)
    if arch == "smolvla":
        mat("mm.fc.weight", H, VH * d["vit_pixel_shuffle"] ** 2)
    else:
        mat("mm.proj.weight", H, VH)
        vec("mm.proj.bias", H)
    vec("state_mean", d["real_state_dim"], 0.0)
    vec("state_std", d["real_state_dim"], 1.0)
    vec("action_mean", d["real_action_dim"], 0.0)
    vec("action_std", d["real_action_dim"], 1.0)
    if arch == "pi05":
        vec("action_q01", d["real_action_dim"], -1.0)
        vec("action_q99", d["real_action_dim"], 1.0)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    d["n_img_tokens"] = n_img_tokens
    return d


if __name__ == "__main__":
    if len(sys.argv) < 3:
        raise SystemExit("usage: python -m vla_cpp_b200.synth_gguf <smolvla|pi0|pi05> <out.gguf> [f32|bf16]")
    print(write_checkpoint(sys.argv[2], sys.argv[1], matrix_dtype=sys.argv[3] if len(sys.argv) > 3 else "f32"))
