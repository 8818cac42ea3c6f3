// Device side of vla_predict for pi0- and SmolVLA-shaped checkpoints: prefix embeddings -> prefix producer
// (the backbone's layers, K/V straight into the engine's pages) -> denoise engine -> un-normalised actions.
//
// Follows the reference's predict paths: src/models/pi0.cpp:451-681 and src/models/smolvla.cpp:1476-1710.
//   pi0      prefix = [image embeddings ; E[lang] * sqrt(hidden)], positions 0..P-1, no mask; the state goes
//            into the suffix (normalised with the dataset statistics); P changes with the number of language tokens
//   pi0.5    (src/models/pi05.cpp:505-705) as pi0 without a state token (the state is part of the prompt); the tower's
//            embeddings are the raw projector output; actions are un-normalised by mean / std or by quantiles
//   SmolVLA  prefix = [image embeddings * sqrt(hidden) ; E[lang padded to n_lang_max] * sqrt(hidden) ; state_proj(state)],
//            padded language slots masked, the state token visible to itself only and rotated at position
//            n_img + n_lang; suffix positions start one past it
// Image embeddings come from vla_inputs.precomputed_img_emb or, when the checkpoint carries the SigLIP tower
// ("vit.*" and "mm.*" tensors), from vla_inputs.images through the vision tower (vision.cu).
#include "predict.h"

#include <cuda_bf16.h>

#include <cmath>
#include <cstring>
#include <random>
#include <string>

namespace vb {

struct Predictor {
    int arch = 0;  // 0 pi0, 1 SmolVLA, 2 pi0.5
    bool quantile_norm = false;
    std::vector<float> action_q01, action_q99;
    vla_config cfg{};
    vlab200_engine *eng = nullptr;
    vlab200_prefill *pre = nullptr;
    DevBuf token_embd, w_state, b_state;  // bf16 [vocab][hidden]; SmolVLA state projection float32 [hidden][sd], [hidden]
    int64_t vocab = 0;
    int max_prefix = 0, max_views = 4;
    std::vector<float> state_mean, state_std, action_mean, action_std;
    DevBuf x_emb, ids, img_stage, state_dev, pads, pixels;
    vlab200_vision *vis = nullptr;
    int vit_image = 0;
    std::mt19937 rng{std::random_device{}()};
    cudaEvent_t ev[4] = {nullptr, nullptr, nullptr, nullptr};
    ~Predictor() {
        vlab200_vision_free(vis);
        vlab200_prefill_free(pre);
        vlab200_engine_free(eng);
        for (cudaEvent_t e : ev)
            if (e) cudaEventDestroy(e);
    }
};

// rows [row0, row0 + n) of x_emb = scale * table[ids[i]]
__global__ void embed_rows_kernel(const __nv_bfloat16 *__restrict__ table, const int32_t *__restrict__ ids, float scale,
                                  float *__restrict__ out, int n, int hidden) {
    const int i = blockIdx.x;
    if (i >= n) return;
    const __nv_bfloat16 *src = table + (size_t)ids[i] * hidden;
    for (int k = threadIdx.x; k < hidden; k += blockDim.x) out[(size_t)i * hidden + k] = scale * __bfloat162float(src[k]);
}

__global__ void scale_copy_kernel(const float *__restrict__ in, float scale, float *__restrict__ out, size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = scale * in[i];
}

// out[o] = b[o] + sum_k W[o][k] x[k]   (float32; the SmolVLA state token, src/models/smolvla.cpp:1365-1366)
__global__ void state_embed_kernel(const float *__restrict__ W, const float *__restrict__ b, const float *__restrict__ x,
                                   float *__restrict__ out, int hidden, int sd) {
    const int o = blockIdx.x * blockDim.x + threadIdx.x;
    if (o >= hidden) return;
    float acc = b ? b[o] : 0.0f;
    for (int k = 0; k < sd; ++k) acc = fmaf(W[(size_t)o * sd + k], x[k], acc);
    out[o] = acc;
}

static void read_stats(const vlab200_gguf *g, const char *name, std::vector<float> &dst) {
    // missing or mis-sized statistics mean identity, as in load_stats (src/models/pi0.cpp:300-329)
    std::vector<float> tmp(dst.size());
    if (!tmp.empty() && vlab200_gguf_read_f32(g, name, tmp.data(), (int64_t)tmp.size(), 0) == VLAB200_OK) dst = tmp;
}

// The SigLIP tower and its connector from the checkpoint: geometry keys and defaults of src/models/smolvla.cpp:320-322,
// 985-1004 and src/models/pi0.cpp:93-95,402-414; tensor names of smolvla.cpp:705-747 (hf_to_gguf) and
// src/modules/siglip_vit.cpp:23-34, src/modules/encoder.cpp:25-48; connector "mm.fc.weight" (SmolVLA, after the
// pixel shuffle) or "mm.proj.weight" / "mm.proj.bias" (pi0, scaled by 1/sqrt(hidden), pi0.cpp:494-498).
static bool load_tower(Predictor *p, const vlab200_gguf *g) {
    const bool smol = p->arch == 1;
    const vla_config &c = p->cfg;
    const std::string pfx = smol ? "smolvla." : (p->arch == 2 ? "pi05." : "pi0.");
    int64_t vh = smol ? 768 : 1152, vl = smol ? 12 : 27, heads = smol ? 12 : 16, patch = smol ? 16 : 14,
            image = smol ? 512 : 224, shuffle = smol ? 4 : 1, inter = smol ? 3072 : 0, n_tok = smol ? 64 : 256;
    auto vu = [&](const char *k, int64_t &d) {
        uint32_t u = 0;
        if (vlab200_gguf_meta_u32(g, (pfx + k).c_str(), &u) == VLAB200_OK) d = u;
    };
    vu("vit_hidden", vh); vu("vit_layers", vl); vu("vit_heads", heads); vu("patch_size", patch); vu("image_size", image);
    vu("n_img_tokens", n_tok);
    if (smol) { vu("vit_pixel_shuffle", shuffle); vu("vit_inter", inter); }
    double dv = 0;
    const float eps = vlab200_gguf_meta_f64(g, (pfx + "vit_ln_eps").c_str(), &dv) == VLAB200_OK ? (float)dv : 1e-6f;
    if (!smol) {  // the MLP width is the checkpoint's: rows of fc1
        int32_t type = 0, nd = 0;
        int64_t dims[4] = {0, 0, 0, 0};
        uint64_t nb = 0;
        if (vlab200_gguf_tensor_info(g, "vit.blk.0.fc1.weight", &type, &nd, dims, &nb) != VLAB200_OK) return false;
        inter = dims[1];
    }
    if (vh <= 0 || vl <= 0 || vl > 256 || heads <= 0 || patch <= 0 || image <= 0 || shuffle <= 0 || inter <= 0 || image % patch) {
        set_last_error("vla_predict: bad vision geometry in the checkpoint");
        return false;
    }
    const int64_t grid = image / patch, np = grid * grid;
    if (grid % shuffle || (grid / shuffle) * (grid / shuffle) != n_tok || n_tok != c.n_img) {
        set_last_error("vla_predict: vit geometry mismatch (grid %lld, shuffle %lld, n_img_tokens %lld, n_img %lld)", (long long)grid,
                       (long long)shuffle, (long long)n_tok, (long long)c.n_img);
        return false;
    }
    const int L = (int)vl;
    const int64_t c4 = vh * shuffle * shuffle;
    std::vector<DevBuf> bufs((size_t)L * 16 + 8);
    bool ok = true;
    auto up = [&](size_t slot, const std::string &name, int64_t d0, int64_t d1, bool bf) -> const void * {
        if (ok && gguf_upload(g, name.c_str(), d0, d1, bf, false, &bufs[slot]) != VLAB200_OK) ok = false;
        return bufs[slot].p;
    };
    vlab200_vision_weights w{};
    const size_t G = (size_t)L * 16;
    w.patch_w = up(G + 0, "vit.patch_embd.weight", vh * 3 * patch * patch, -1, true);
    w.patch_b = static_cast<const float *>(up(G + 1, "vit.patch_embd.bias", vh, 1, false));
    w.pos = static_cast<const float *>(up(G + 2, "vit.pos_embd", vh, np, false));
    w.post_w = static_cast<const float *>(up(G + 3, "vit.post_ln.weight", vh, 1, false));
    w.post_b = static_cast<const float *>(up(G + 4, "vit.post_ln.bias", vh, 1, false));
    if (smol) {
        w.connector = up(G + 5, "mm.fc.weight", c4, c.hidden, true);
    } else {
        w.connector = up(G + 5, "mm.proj.weight", c4, c.hidden, true);
        int32_t type = 0, nd = 0;
        int64_t dims[4] = {0, 0, 0, 0};
        uint64_t nb = 0;
        if (vlab200_gguf_tensor_info(g, "mm.proj.bias", &type, &nd, dims, &nb) == VLAB200_OK)
            w.connector_b = static_cast<const float *>(up(G + 6, "mm.proj.bias", c.hidden, 1, false));
    }
    std::vector<const void *> mats[6];
    std::vector<const float *> vecs[10];
    for (auto &m : mats) m.resize((size_t)L);
    for (auto &v : vecs) v.resize((size_t)L);
    static const char *mat_names[6] = {"attn_q", "attn_k", "attn_v", "attn_o", "fc1", "fc2"};
    static const char *vec_names[10] = {"ln1.weight", "ln1.bias", "ln2.weight", "ln2.bias", "attn_q.bias", "attn_k.bias",
                                        "attn_v.bias", "attn_o.bias", "fc1.bias", "fc2.bias"};
    for (int l = 0; l < L && ok; ++l) {
        const std::string b = "vit.blk." + std::to_string(l) + ".";
        for (int j = 0; j < 6; ++j) {
            const int64_t d0 = j == 5 ? inter : vh, d1 = j == 4 ? inter : vh;
            mats[j][(size_t)l] = up((size_t)l * 16 + j, b + mat_names[j] + ".weight", d0, d1, true);
        }
        for (int j = 0; j < 10; ++j)
            vecs[j][(size_t)l] = static_cast<const float *>(up((size_t)l * 16 + 6 + j, b + vec_names[j], j == 8 ? inter : vh, 1, false));
    }
    if (!ok) return false;
    w.wq = mats[0].data(); w.wk = mats[1].data(); w.wv = mats[2].data(); w.wo = mats[3].data();
    w.fc1 = mats[4].data(); w.fc2 = mats[5].data();
    w.ln1_w = vecs[0].data(); w.ln1_b = vecs[1].data(); w.ln2_w = vecs[2].data(); w.ln2_b = vecs[3].data();
    w.bq = vecs[4].data(); w.bk = vecs[5].data(); w.bv = vecs[6].data(); w.bo = vecs[7].data();
    w.b1 = vecs[8].data(); w.b2 = vecs[9].data();
    vlab200_vision_config vc{};
    vc.image = (int)image; vc.patch = (int)patch; vc.hidden = (int)vh; vc.n_layers = L; vc.n_heads = (int)heads;
    vc.inter = (int)inter; vc.shuffle = (int)shuffle; vc.out_dim = (int)c.hidden; vc.ln_eps = eps;
    // pi0 scales the projector by 1/sqrt(hidden) (pi0.cpp:498); pi0.5 undoes that scale (pi05.cpp:572-577): raw output
    vc.out_scale = p->arch == 0 ? 1.0f / std::sqrt((float)c.hidden) : 0.0f;
    p->vis = vlab200_vision_create(&vc, &w, p->max_views);
    p->vit_image = (int)image;
    return p->vis != nullptr && p->pixels.alloc((size_t)p->max_views * image * image * 3 * 4) == VLAB200_OK;
}

Predictor *predictor_create(const vlab200_gguf *g, const char *arch, const vla_config *cfg) {
    auto *p = new (std::nothrow) Predictor();
    if (!p) return nullptr;
    p->arch = std::strcmp(arch, "pi0") == 0 ? 0 : (std::strcmp(arch, "pi05") == 0 ? 2 : 1);
    p->cfg = *cfg;
    const vla_config &c = p->cfg;
    const int64_t n_img_max = c.n_img * p->max_views;
    p->max_prefix = (int)(n_img_max + c.n_lang + (p->arch == 1 ? 1 : 0));
    bool ok = true;
    // ---- the backbone's layers: "vlm.blk.N.*" with the decoder-block suffixes the converters write ----
    const int L = (int)c.n_layers;
    const int64_t H = c.hidden, I = c.intermediate, qf = c.q_full_dim, kvf = c.kv_full_dim;
    std::vector<DevBuf> bufs((size_t)L * 9);
    std::vector<const void *> wq(L), wk(L), wv(L), wo(L), wg(L), wu(L), wd(L);
    std::vector<const float *> ln_in(L), ln_post(L);
    const bool gemma = p->arch != 1;
    for (int l = 0; l < L && ok; ++l) {
        const std::string b = "vlm.blk." + std::to_string(l) + ".";
        DevBuf *d = &bufs[(size_t)l * 9];
        auto up = [&](int slot, const char *suffix, int64_t d0, int64_t d1, bool bf, bool gm) -> const void * {
            if (ok && gguf_upload(g, (b + suffix).c_str(), d0, d1, bf, gm, &d[slot]) != VLAB200_OK) ok = false;
            return d[slot].p;
        };
        ln_in[l] = static_cast<const float *>(up(0, "attn_norm.weight", H, 1, false, gemma));
        wq[l] = up(1, "attn_q.weight", H, qf, true, false);
        wk[l] = up(2, "attn_k.weight", H, kvf, true, false);
        wv[l] = up(3, "attn_v.weight", H, kvf, true, false);
        wo[l] = up(4, "attn_o.weight", qf, H, true, false);
        ln_post[l] = static_cast<const float *>(up(5, "ffn_norm.weight", H, 1, false, gemma));
        wg[l] = up(6, "ffn_gate.weight", H, I, true, false);
        wu[l] = up(7, "ffn_up.weight", H, I, true, false);
        wd[l] = up(8, "ffn_down.weight", I, H, true, false);
    }
    if (ok) {
        vlab200_prefill_config pc{};
        pc.n_layers = L; pc.hidden = (int)H; pc.n_q = (int)c.n_q_heads; pc.n_kv = (int)c.n_kv_heads;
        pc.head_dim = (int)c.head_dim; pc.inter = (int)I; pc.act = gemma ? 2 : 1;
        pc.rms_eps = c.rms_eps; pc.rope_base = c.rope_freq_base;
        vlab200_prefill_weights pw{wq.data(), wk.data(), wv.data(), wo.data(), wg.data(), wu.data(), wd.data(),
                                   ln_in.data(), ln_post.data()};
        p->pre = vlab200_prefill_create(&pc, &pw, 1, p->max_prefix);
        ok = p->pre != nullptr;
    }
    bufs.clear();  // the prefill keeps prepared copies
    if (ok) {
        p->eng = vlab200_engine_create_from_gguf(g, 1, p->max_prefix);
        ok = p->eng != nullptr;
    }
    // ---- token embeddings (bf16 table), SmolVLA state projection, dataset statistics ----
    if (ok) {
        int32_t type = 0, nd = 0;
        int64_t dims[4] = {0, 0, 0, 0};
        uint64_t nb = 0;
        if (vlab200_gguf_tensor_info(g, "token_embd.weight", &type, &nd, dims, &nb) != VLAB200_OK || dims[0] != H) {
            set_last_error("vla_predict: token_embd.weight is missing or is not [vocab][%lld]", (long long)H);
            ok = false;
        } else {
            p->vocab = dims[1];
            ok = gguf_upload(g, "token_embd.weight", H, p->vocab, true, false, &p->token_embd) == VLAB200_OK;
        }
    }
    if (ok && p->arch == 1)
        ok = gguf_upload(g, "state_proj.weight", c.max_state_dim, H, false, false, &p->w_state) == VLAB200_OK &&
             gguf_upload(g, "state_proj.bias", H, 1, false, false, &p->b_state) == VLAB200_OK;
    p->state_mean.assign((size_t)c.real_state_dim, 0.0f);
    p->state_std.assign((size_t)c.real_state_dim, 1.0f);
    p->action_mean.assign((size_t)c.real_action_dim, 0.0f);
    p->action_std.assign((size_t)c.real_action_dim, 1.0f);
    read_stats(g, "state_mean", p->state_mean);
    read_stats(g, "state_std", p->state_std);
    read_stats(g, "action_mean", p->action_mean);
    read_stats(g, "action_std", p->action_std);
    if (p->arch == 2) {  // src/models/pi05.cpp:411,361-366
        char mode[32] = "";
        p->quantile_norm = vlab200_gguf_meta_str(g, "pi05.norm_mode", mode, sizeof mode) == VLAB200_OK && std::strcmp(mode, "quantiles") == 0;
        if (p->quantile_norm) {
            p->action_q01.assign((size_t)c.real_action_dim, -1.0f);
            p->action_q99.assign((size_t)c.real_action_dim, 1.0f);
            read_stats(g, "action_q01", p->action_q01);
            read_stats(g, "action_q99", p->action_q99);
        }
    }
    if (ok)
        ok = p->x_emb.alloc((size_t)p->max_prefix * H * 4) == VLAB200_OK && p->ids.alloc((size_t)c.n_lang * 4) == VLAB200_OK &&
             p->img_stage.alloc((size_t)n_img_max * H * 4) == VLAB200_OK &&
             p->state_dev.alloc((size_t)c.max_state_dim * 4) == VLAB200_OK && p->pads.alloc(8) == VLAB200_OK;
    for (int i = 0; ok && i < 4; ++i) ok = cudaEventCreate(&p->ev[i]) == cudaSuccess;
    if (ok) {  // the tower is optional: a checkpoint without it serves precomputed image embeddings only
        int32_t type = 0, nd = 0;
        int64_t dims[4] = {0, 0, 0, 0};
        uint64_t nb = 0;
        if (vlab200_gguf_tensor_info(g, "vit.patch_embd.weight", &type, &nd, dims, &nb) == VLAB200_OK) ok = load_tower(p, g);
    }
    if (!ok) {
        delete p;
        return nullptr;
    }
    return p;
}

void predictor_free(Predictor *p) { delete p; }

int predictor_run(Predictor *p, const vla_inputs *in, std::vector<float> *actions, vla_stats *stats) {
    const vla_config &c = p->cfg;
    const int H = (int)c.hidden, sd = (int)c.max_state_dim, ad = (int)c.max_action_dim, chunk = (int)c.n_suffix;
    const bool from_pixels = !in->precomputed_img_emb;
    const int n_views = from_pixels ? in->n_images : in->n_img_views;
    if (from_pixels && !p->vis) {
        set_last_error("vla_predict: the checkpoint has no vision tower (vit.* tensors); pass vla_inputs.precomputed_img_emb");
        return VLAB200_ERR_UNSUPPORTED;
    }
    if (n_views < 1 || n_views > p->max_views) {
        set_last_error("vla_predict: %d camera views outside [1, %d]", n_views, p->max_views);
        return VLAB200_ERR_ARG;
    }
    if (from_pixels) {
        if (!in->images) return VLAB200_ERR_ARG;
        for (int v = 0; v < n_views; ++v) {
            const vla_image &im = in->images[v];
            // a view of another size would be read past its end (src/modules/preprocess.h:30-32,58-62)
            if (!im.data || im.w != p->vit_image || im.h != p->vit_image || (im.format != VLA_PIXEL_U8 && im.format != VLA_PIXEL_F32_RGB_01)) {
                set_last_error("vla_predict: image view %d is %dx%d, expected %dx%d", v, im.w, im.h, p->vit_image, p->vit_image);
                return VLAB200_ERR_ARG;
            }
        }
    }
    // language tokens index the embedding table: reject ids outside it (src/models/smolvla.cpp:1579-1589)
    const int n_lang = in->n_lang;
    if (n_lang < 1 || n_lang > (int)c.n_lang) {
        set_last_error("vla_predict: lang_tokens length %d out of range [1, %lld]", n_lang, (long long)c.n_lang);
        return VLAB200_ERR_ARG;
    }
    for (int i = 0; i < n_lang; ++i)
        if (in->lang_tokens[i] < 0 || in->lang_tokens[i] >= p->vocab) {
            set_last_error("vla_predict: lang_tokens[%d] = %d out of vocab range [0, %lld)", i, in->lang_tokens[i],
                           (long long)p->vocab);
            return VLAB200_ERR_ARG;
        }
    cudaStream_t cs = nullptr;
    const int n_img = (int)c.n_img * n_views;
    const int n_lang_rows = p->arch == 1 ? (int)c.n_lang : n_lang;  // SmolVLA pads the language block
    const int P = n_img + n_lang_rows + (p->arch == 1 ? 1 : 0);
    const float lang_scale = p->arch == 1 ? std::sqrt((float)H) : (float)std::sqrt((double)H);
    // ---- inputs ----
    std::vector<float> state((size_t)sd, 0.0f);
    if (in->state) std::memcpy(state.data(), in->state, (size_t)sd * sizeof(float));
    for (int64_t i = 0; i < c.real_state_dim && i < sd; ++i)
        state[(size_t)i] = (state[(size_t)i] - p->state_mean[(size_t)i]) / (p->state_std[(size_t)i] + c.norm_eps);
    std::vector<float> x0((size_t)chunk * ad);
    if (in->noise) {
        std::memcpy(x0.data(), in->noise, x0.size() * sizeof(float));
    } else {
        std::normal_distribution<float> nd(0.0f, 1.0f);
        for (float &v : x0) v = nd(p->rng);
    }
    std::vector<int32_t> ids((size_t)n_lang_rows, 0);
    std::memcpy(ids.data(), in->lang_tokens, (size_t)n_lang * sizeof(int32_t));
    const bool timed = in->timing_detail == VLA_TIMING_PHASE;
    int rc;
    if (from_pixels) {
        // views of one pixel format go through the tower together, mixed formats one view at a time
        if (timed) VB_CUDA(cudaEventRecord(p->ev[3], cs));
        bool same = true;
        for (int v = 1; v < n_views; ++v) same = same && in->images[v].format == in->images[0].format;
        const size_t px = (size_t)p->vit_image * p->vit_image * 3;
        if (same) {
            const size_t bytes = px * (in->images[0].format == VLA_PIXEL_U8 ? 1 : 4);
            for (int v = 0; v < n_views; ++v)
                VB_CUDA(cudaMemcpyAsync(static_cast<char *>(p->pixels.p) + (size_t)v * bytes, in->images[v].data, bytes,
                                        cudaMemcpyHostToDevice, cs));
            if ((rc = vlab200_vision_run(p->vis, p->pixels.p, in->images[0].format == VLA_PIXEL_F32_RGB_01, n_views,
                                         p->img_stage.as<float>(), cs)))
                return rc;
        } else {
            for (int v = 0; v < n_views; ++v) {
                const bool f32 = in->images[v].format == VLA_PIXEL_F32_RGB_01;
                char *dst = static_cast<char *>(p->pixels.p) + (size_t)v * px * 4;
                VB_CUDA(cudaMemcpyAsync(dst, in->images[v].data, px * (f32 ? 4 : 1), cudaMemcpyHostToDevice, cs));
                if ((rc = vlab200_vision_run(p->vis, dst, f32, 1, p->img_stage.as<float>() + (size_t)v * c.n_img * H, cs))) return rc;
            }
        }
    } else {
        VB_CUDA(cudaMemcpyAsync(p->img_stage.p, in->precomputed_img_emb, (size_t)n_img * H * 4, cudaMemcpyHostToDevice, cs));
    }
    VB_CUDA(cudaMemcpyAsync(p->ids.p, ids.data(), ids.size() * 4, cudaMemcpyHostToDevice, cs));
    VB_CUDA(cudaMemcpyAsync(p->state_dev.p, state.data(), (size_t)sd * 4, cudaMemcpyHostToDevice, cs));
    if (timed) VB_CUDA(cudaEventRecord(p->ev[0], cs));
    // ---- prefix embeddings ----
    float *x = p->x_emb.as<float>();
    scale_copy_kernel<<<148, 256, 0, cs>>>(p->img_stage.as<float>(), p->arch == 1 ? lang_scale : 1.0f, x, (size_t)n_img * H);
    embed_rows_kernel<<<n_lang_rows, 256, 0, cs>>>(p->token_embd.as<__nv_bfloat16>(), p->ids.as<int32_t>(), lang_scale,
                                                   x + (size_t)n_img * H, n_lang_rows, H);
    int32_t pad[2] = {0, 0};
    std::vector<int32_t> pos;
    int pos_base = -1;
    if (p->arch == 1) {
        state_embed_kernel<<<(H + 127) / 128, 128, 0, cs>>>(p->w_state.as<float>(), p->b_state.as<float>(),
                                                           p->state_dev.as<float>(), x + (size_t)(P - 1) * H, H, sd);
        pad[0] = n_img + n_lang;
        pad[1] = n_img + (int)c.n_lang;
        pos.resize((size_t)P);
        for (int i = 0; i < P; ++i) pos[(size_t)i] = i;
        pos[(size_t)P - 1] = n_img + n_lang;  // the state token's position
        pos_base = n_img + n_lang + 1;
        VB_CUDA(cudaMemcpyAsync(p->pads.p, pad, 8, cudaMemcpyHostToDevice, cs));
    }
    VB_CUDA(cudaGetLastError());
    const int32_t *pads_dev = (p->arch == 1 && pad[1] > pad[0]) ? p->pads.as<int32_t>() : nullptr;
    if ((rc = vlab200_engine_set_prefix_len(p->eng, P))) return rc;
    if ((rc = vlab200_prefill_run(p->pre, p->eng, 0, 1, x, P, p->arch == 1 ? pos.data() : nullptr, p->arch == 1 ? 3 : 0,
                                  pads_dev, cs)))
        return rc;
    if (timed) VB_CUDA(cudaEventRecord(p->ev[1], cs));
    // ---- denoise loop, actions back ----
    actions->assign((size_t)chunk * ad, 0.0f);
    if ((rc = vlab200_engine_denoise_host(p->eng, 1, p->arch == 0 ? state.data() : nullptr, x0.data(), actions->data(),
                                          pos_base, (p->arch == 1 && pads_dev) ? pad : nullptr, cs)))
        return rc;
    if (timed) VB_CUDA(cudaEventRecord(p->ev[2], cs));
    VB_CUDA(cudaStreamSynchronize(cs));
    int status = 0;
    if (vlab200_device_status(&status, 1) != VLAB200_OK || status != 0) {
        set_last_error("vla_predict: a kernel reported device status %d", status);
        return VLAB200_ERR_DEVICE;
    }
    // un-normalise the real action columns, zero the padding (src/models/smolvla.cpp:1698-1705, pi0.cpp:673-677)
    for (int t = 0; t < chunk; ++t)
        for (int j = 0; j < ad; ++j) {
            float &v = (*actions)[(size_t)t * ad + j];
            if (j >= c.real_action_dim) v = 0.0f;
            else if (p->quantile_norm) v = (v + 1.0f) * (p->action_q99[(size_t)j] - p->action_q01[(size_t)j]) * 0.5f + p->action_q01[(size_t)j];
            else v = v * (p->action_std[(size_t)j] + c.norm_eps) + p->action_mean[(size_t)j];
        }
    if (timed) {
        cudaEventElapsedTime(&stats->ms_prefill, p->ev[0], p->ev[1]);
        cudaEventElapsedTime(&stats->ms_denoise, p->ev[1], p->ev[2]);
        stats->ms_inference = stats->ms_prefill + stats->ms_denoise;
        if (from_pixels) cudaEventElapsedTime(&stats->ms_vision, p->ev[3], p->ev[0]);
    }
    return VLAB200_OK;
}

}  // namespace vb
