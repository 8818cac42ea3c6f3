// The model-level C ABI (include/vla.h, ABI v1) on top of the denoise engine.
//
// Mirrors the boundary rules of the reference's src/vla_c_api.cpp:44-190: NULL handles and NULL
// output pointers give VLA_ERR_ARG, vla_model_load gives NULL on any failure, an empty result
// gives VLA_ERR_PREDICT, no exception leaves the library, the action buffer is malloc'd and
// released by vla_free_actions.  Loading parses the checkpoint's metadata on the host (the
// same required keys as src/models/pi0.cpp:258-293 and src/models/smolvla.cpp:590-632) and needs
// no GPU; device objects are created by the first vla_predict.
#include <chrono>
#include <cstdlib>
#include <cstring>
#include <new>
#include <string>
#include <vector>

#include "../../include/vla.h"
#include "host_common.h"
#include "predict.h"

struct vla_model {
    vlab200_gguf *gguf = nullptr;
    vla_config cfg{};
    vla_stats stats{};
    std::string arch;
    vb::Predictor *predictor = nullptr;  // device side, created on first use
};

namespace {

bool meta_u32(const vlab200_gguf *g, const std::string &key, int64_t *dst) {
    uint32_t v = 0;
    if (vlab200_gguf_meta_u32(g, key.c_str(), &v) != VLAB200_OK) {
        vb::set_last_error("vla_model_load: required metadata key %s is missing", key.c_str());
        return false;
    }
    *dst = (int64_t)v;
    return true;
}

// vla::Config as the two supported architectures resolve it at load time.
bool resolve_config(const vlab200_gguf *g, const std::string &arch, vla_config *c) {
    const std::string p = arch + ".";
    std::memset(c, 0, sizeof(*c));
    int64_t steps = 0, every = 0;
    if (!meta_u32(g, p + "hidden", &c->hidden) || !meta_u32(g, p + "intermediate", &c->intermediate) ||
        !meta_u32(g, p + "n_q_heads", &c->n_q_heads) || !meta_u32(g, p + "n_kv_heads", &c->n_kv_heads) ||
        !meta_u32(g, p + "head_dim", &c->head_dim) || !meta_u32(g, p + "n_layers", &c->n_layers) ||
        !meta_u32(g, p + "expert_h", &c->expert_h) || !meta_u32(g, p + "expert_inter", &c->expert_inter) ||
        !meta_u32(g, p + "chunk_size", &c->n_suffix) || !meta_u32(g, p + "num_steps", &steps) ||
        !meta_u32(g, p + "max_state_dim", &c->max_state_dim) || !meta_u32(g, p + "max_action_dim", &c->max_action_dim) ||
        !meta_u32(g, p + "real_state_dim", &c->real_state_dim) ||
        !meta_u32(g, p + "real_action_dim", &c->real_action_dim) ||
        !meta_u32(g, p + "tokenizer_max_length", &c->n_lang))
        return false;
    if (vlab200_gguf_meta_f64(g, (p + "min_period").c_str(), &c->min_period) != VLAB200_OK ||
        vlab200_gguf_meta_f64(g, (p + "max_period").c_str(), &c->max_period) != VLAB200_OK) {
        vb::set_last_error("vla_model_load: %smin_period / %smax_period missing", p.c_str(), p.c_str());
        return false;
    }
    c->num_steps = (int32_t)steps;
    c->n_state = 1;
    c->q_full_dim = c->n_q_heads * c->head_dim;
    c->kv_full_dim = c->n_kv_heads * c->head_dim;
    c->rope_n_dims = (int32_t)c->head_dim;
    c->rope_mode = 2;  // GGML_ROPE_TYPE_NEOX
    double v = 0;
    c->norm_eps = vlab200_gguf_meta_f64(g, (p + "norm_eps").c_str(), &v) == VLAB200_OK ? (float)v : 1e-8f;
    c->denormalized = 1;
    if (arch == "pi0" || arch == "pi05") {  // src/models/pi0.cpp:267-300, src/models/pi05.cpp:300-326
        c->n_img = 256;
        c->self_attn_every_n = 0;
        c->rms_eps = vlab200_gguf_meta_f64(g, (p + "rms_norm_eps").c_str(), &v) == VLAB200_OK ? (float)v : 1e-6f;
        c->rope_freq_base = vlab200_gguf_meta_f64(g, (p + "rope_theta").c_str(), &v) == VLAB200_OK ? (float)v : 10000.0f;
        if (arch == "pi05") c->n_state = 0;  // the state is part of the prompt, not a token of its own
    } else {              // src/models/smolvla.cpp:604-632
        if (!meta_u32(g, "smolvla.self_attn_every_n_layers", &every)) return false;
        int64_t n_img = 64;
        uint32_t u = 0;
        if (vlab200_gguf_meta_u32(g, "smolvla.n_img_tokens", &u) == VLAB200_OK) n_img = u;
        c->n_img = n_img;
        c->self_attn_every_n = (int32_t)every;
        c->rms_eps = 1e-5f;
        c->rope_freq_base = 10000.0f;
        c->n_prefix = c->n_img + c->n_lang + c->n_state;  // per view; predict rescales n_img by the view count
        c->n_full = c->n_prefix + c->n_suffix;
    }
    return true;
}

}  // namespace

extern "C" {

int32_t vla_abi_version(void) { return VLA_ABI_VERSION; }

vla_model *vla_model_load(const char *mmproj_path, const char *ckpt_path, const char *config_path) {
    (void)mmproj_path;  // both supported architectures carry their vision tower inside the checkpoint
    (void)config_path;
    if (!ckpt_path) return nullptr;
    try {
        vlab200_gguf *g = vlab200_gguf_open(ckpt_path);
        if (!g) return nullptr;
        char arch[32] = "";
        vlab200_gguf_meta_str(g, "general.architecture", arch, sizeof arch);
        vla_model *m = new (std::nothrow) vla_model();
        if (!m || (std::strcmp(arch, "pi0") != 0 && std::strcmp(arch, "pi05") != 0 && std::strcmp(arch, "smolvla") != 0)) {
            if (m) vb::set_last_error("vla_model_load: architecture '%s' is not served by this library (pi0, pi05, smolvla)", arch);
            delete m;
            vlab200_gguf_close(g);
            return nullptr;
        }
        m->gguf = g;
        m->arch = arch;
        if (!resolve_config(g, m->arch, &m->cfg)) {
            vla_model_free(m);
            return nullptr;
        }
        // predict sizes its buffers from the max_* dims and loops to the real_* dims (src/model.cpp:131-149)
        if (m->cfg.real_state_dim > m->cfg.max_state_dim || m->cfg.real_action_dim > m->cfg.max_action_dim) {
            vb::set_last_error("vla_model_load: real_state_dim / real_action_dim exceed their max_* dims");
            vla_model_free(m);
            return nullptr;
        }
        return m;
    } catch (...) {
        return nullptr;
    }
}

void vla_model_free(vla_model *m) {
    if (!m) return;
    vb::predictor_free(m->predictor);
    if (m->gguf) vlab200_gguf_close(m->gguf);
    delete m;
}

int32_t vla_model_config(const vla_model *m, vla_config *out) {
    if (!m || !out) return VLA_ERR_ARG;
    *out = m->cfg;
    return VLA_OK;
}

int32_t vla_predict(vla_model *m, const vla_inputs *in, float **out_actions, int64_t *out_n) {
    if (!m || !in || !out_actions || !out_n) return VLA_ERR_ARG;
    *out_actions = nullptr;
    *out_n = 0;
    if (in->n_images < 0 || in->n_lang < 0 || in->n_img_views < 0) return VLA_ERR_ARG;
    if (in->n_images > 0 && !in->images) return VLA_ERR_ARG;
    if (in->n_lang > 0 && !in->lang_tokens) return VLA_ERR_ARG;
    try {
        const auto t0 = std::chrono::steady_clock::now();
        if (!m->predictor) m->predictor = vb::predictor_create(m->gguf, m->arch.c_str(), &m->cfg);
        if (!m->predictor) return VLA_ERR_PREDICT;
        std::vector<float> act;
        m->stats = vla_stats{};
        if (vb::predictor_run(m->predictor, in, &act, &m->stats) != VLAB200_OK || act.empty()) return VLA_ERR_PREDICT;
        float *buf = static_cast<float *>(std::malloc(act.size() * sizeof(float)));
        if (!buf) return VLA_ERR_EXCEPTION;
        std::memcpy(buf, act.data(), act.size() * sizeof(float));
        *out_actions = buf;
        *out_n = (int64_t)act.size();
        m->stats.ms_total = std::chrono::duration<float, std::milli>(std::chrono::steady_clock::now() - t0).count();
        return VLA_OK;
    } catch (...) {
        return VLA_ERR_EXCEPTION;
    }
}

void vla_free_actions(float *actions) { std::free(actions); }

int32_t vla_last_stats(const vla_model *m, vla_stats *out) {
    if (!m || !out) return VLA_ERR_ARG;
    *out = m->stats;
    return VLA_OK;
}

}  // extern "C"
