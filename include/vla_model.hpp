// vla_model.hpp -- the C++ face of the model-level API, for programs written against the reference's
// src/model.h (vla-cli, vla-server and vla-bench link that interface: vla::model_load / model_free /
// model_config / predict / last_stats / config_is_sane, src/model.h:48-233).  Header-only: every call
// forwards to the C ABI of include/vla.h, so a program needs this header and libvla_b200.so, nothing else.
//
// Differences from the reference: vla::Options is not offered (the library has one device path, bf16
// activations), and vla::Config is the C struct vla_config (same field names as the reference's Config).
#pragma once
#include <cstdio>
#include <string>
#include <vector>

#include "vla.h"

namespace vla {

using Config = ::vla_config;

enum class TimingDetail { NONE, PHASE };
enum class PixelFormat { U8, F32_RGB_01 };

struct ImageView {
    const void *data;
    int w, h;
    PixelFormat format = PixelFormat::U8;
};

// Everything is borrowed for the duration of predict().  Give either images or precomputed_img_emb.
struct Inputs {
    const ImageView *images = nullptr;
    int n_images = 0;
    const float *precomputed_img_emb = nullptr;  // [n_img_views * n_img][hidden], in the scale the LM expects
    int n_img_views = 0;
    const int32_t *lang_tokens = nullptr;
    int n_lang = 0;
    const float *state = nullptr;  // max_state_dim floats
    const float *noise = nullptr;  // n_suffix * max_action_dim floats, or nullptr to sample
    const int32_t *attention_mask = nullptr;
    int attention_mask_n = 0;
    TimingDetail timing_detail = TimingDetail::NONE;
};

struct Stats {
    float ms_total = 0.f, ms_vision = 0.f, ms_inference = 0.f, ms_prefill = 0.f, ms_denoise = 0.f;
};

struct Model {
    ::vla_model *handle = nullptr;
    Config cfg{};
    Stats stats{};
};

// real_* dims beyond max_* dims would make predict() write out of bounds (src/model.cpp:131-149).
inline bool config_is_sane(const Config &c) {
    const struct { const char *name; int64_t real, max; } pairs[] = {{"state", c.real_state_dim, c.max_state_dim},
                                                                     {"action", c.real_action_dim, c.max_action_dim}};
    for (const auto &p : pairs) {
        if (p.real < 0 || p.max < 0) {
            std::fprintf(stderr, "vla: negative %s dim (real=%lld max=%lld)\n", p.name, (long long)p.real, (long long)p.max);
            return false;
        }
        if (p.max > 0 && p.real > p.max) {
            std::fprintf(stderr, "vla: real_%s_dim %lld exceeds max_%s_dim %lld\n", p.name, (long long)p.real, p.name,
                         (long long)p.max);
            return false;
        }
    }
    return true;
}

inline Model *model_load(const std::string &mmproj_path, const std::string &ckpt_path, const std::string &config_path = "") {
    ::vla_model *h = ::vla_model_load(mmproj_path.empty() ? nullptr : mmproj_path.c_str(), ckpt_path.c_str(),
                                      config_path.empty() ? nullptr : config_path.c_str());
    if (!h) return nullptr;
    Model *m = new Model();
    m->handle = h;
    if (::vla_model_config(h, &m->cfg) != VLA_OK || !config_is_sane(m->cfg)) {
        ::vla_model_free(h);
        delete m;
        return nullptr;
    }
    return m;
}

inline void model_free(Model *m) {
    if (!m) return;
    ::vla_model_free(m->handle);
    delete m;
}

inline const Config &model_config(const Model *m) { return m->cfg; }

// Empty vector on failure, like the reference (src/model.cpp:293-296).
inline std::vector<float> predict(Model *m, const Inputs &in) {
    if (!m || !m->handle) return {};
    std::vector<::vla_image> views((size_t)(in.n_images > 0 ? in.n_images : 0));
    for (size_t i = 0; i < views.size(); ++i)
        views[i] = ::vla_image{in.images[i].data, in.images[i].w, in.images[i].h,
                               in.images[i].format == PixelFormat::F32_RGB_01 ? VLA_PIXEL_F32_RGB_01 : VLA_PIXEL_U8};
    ::vla_inputs ci{};
    ci.images = views.empty() ? nullptr : views.data();
    ci.n_images = (int32_t)views.size();
    ci.precomputed_img_emb = in.precomputed_img_emb;
    ci.n_img_views = in.n_img_views;
    ci.lang_tokens = in.lang_tokens;
    ci.n_lang = in.n_lang;
    ci.state = in.state;
    ci.noise = in.noise;
    ci.attention_mask = in.attention_mask;
    ci.attention_mask_n = in.attention_mask_n;
    ci.timing_detail = in.timing_detail == TimingDetail::PHASE ? VLA_TIMING_PHASE : VLA_TIMING_NONE;
    float *buf = nullptr;
    int64_t n = 0;
    std::vector<float> out;
    if (::vla_predict(m->handle, &ci, &buf, &n) == VLA_OK && buf && n > 0) out.assign(buf, buf + n);
    ::vla_free_actions(buf);
    ::vla_stats s{};
    if (::vla_last_stats(m->handle, &s) == VLA_OK)
        m->stats = Stats{s.ms_total, s.ms_vision, s.ms_inference, s.ms_prefill, s.ms_denoise};
    return out;
}

inline const Stats &last_stats(const Model *m) { return m->stats; }

}  // namespace vla
