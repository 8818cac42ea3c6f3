/*
 * vla.h -- the model-level C ABI of vla.cpp (ABI version 1), as exported by libvla_b200.so.
 *
 * Declaration-compatible with the reference's public header (include/vla.h:37-161 there): same
 * type names, field order and widths, enumerator values and function signatures, so a program
 * or binding written against the reference header (bindings/python/vla_cpp/_ffi.py:124-163,
 * tests/test_c_api.c) compiles and links against this library unchanged.  Plain C.
 *
 * Ownership and error rules (reference: src/vla_c_api.cpp:44-190):
 *   - everything reachable from vla_inputs is borrowed for the duration of the call;
 *   - vla_predict returns a malloc'd buffer that the caller hands back to vla_free_actions;
 *   - a NULL handle or output pointer is VLA_ERR_ARG, never a crash; vla_model_free(NULL) and
 *     vla_free_actions(NULL) are no-ops; vla_model_load returns NULL on any failure;
 *   - no C++ exception crosses the boundary (VLA_ERR_EXCEPTION);
 *   - a handle is not thread-safe.
 */
#ifndef VLA_H
#define VLA_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define VLA_API __attribute__((visibility("default")))
#define VLA_ABI_VERSION 1

typedef struct vla_model vla_model;

typedef enum { VLA_OK = 0, VLA_ERR_ARG = -1, VLA_ERR_PREDICT = -2, VLA_ERR_EXCEPTION = -3 } vla_status;
typedef enum { VLA_PIXEL_U8 = 0, VLA_PIXEL_F32_RGB_01 = 1 } vla_pixel_format;
typedef enum { VLA_TIMING_NONE = 0, VLA_TIMING_PHASE = 1 } vla_timing_detail;

/* Resolved model configuration (30 fields; layout of the reference's vla_config). */
typedef struct {
    int64_t n_img, n_lang, n_state, n_prefix, n_suffix, n_full;            /* token counts */
    int64_t hidden, expert_h, intermediate, expert_inter;                  /* widths */
    int64_t n_q_heads, n_kv_heads, head_dim, q_full_dim, kv_full_dim, n_layers;
    int32_t self_attn_every_n;                                             /* SmolVLA: self-attention every n-th layer */
    int64_t max_state_dim, max_action_dim, real_state_dim, real_action_dim;
    float norm_eps;
    double min_period, max_period;                                         /* time-embedding periods */
    int32_t num_steps;                                                     /* Euler steps */
    float rms_eps;
    int32_t rope_n_dims, rope_mode;
    float rope_freq_base;
    int32_t denormalized;                                                  /* != 0: dataset statistics already applied */
} vla_config;

typedef struct {
    const void *data; /* first pixel, interleaved RGB */
    int32_t w, h;
    int32_t format;   /* vla_pixel_format */
} vla_image;

typedef struct {
    const vla_image *images;
    int32_t n_images;
    const float *precomputed_img_emb; /* optional [n_img_views * n_img][hidden]: replaces the vision tower */
    int32_t n_img_views;
    const int32_t *lang_tokens;
    int32_t n_lang;
    const float *state;               /* max_state_dim floats */
    const float *noise;               /* n_suffix * max_action_dim floats, or NULL: sampled internally */
    const int32_t *attention_mask;    /* Evo-1 only */
    int32_t attention_mask_n;
    int32_t timing_detail;            /* vla_timing_detail */
} vla_inputs;

typedef struct { float ms_total, ms_vision, ms_inference, ms_prefill, ms_denoise; } vla_stats;

VLA_API int32_t vla_abi_version(void);
VLA_API vla_model *vla_model_load(const char *mmproj_path, const char *ckpt_path, const char *config_path);
VLA_API void vla_model_free(vla_model *m);
VLA_API int32_t vla_model_config(const vla_model *m, vla_config *out);
/* On VLA_OK *out_actions holds *out_n floats, row-major [n_suffix][max_action_dim], columns past
 * real_action_dim zero. */
VLA_API int32_t vla_predict(vla_model *m, const vla_inputs *in, float **out_actions, int64_t *out_n);
VLA_API void vla_free_actions(float *actions);
VLA_API int32_t vla_last_stats(const vla_model *m, vla_stats *out);

#ifdef __cplusplus
}
#endif
#endif /* VLA_H */
