/* Prints sizeof / offsetof of every public struct field of a vla.h (whichever one -I selects), one
 * "name value" pair per line.  Compiled once against the reference's header (tests/golden/make_golden.py,
 * output stored as tests/golden/vla_h_layout.txt) and once against this repository's include/vla.h. */
#include <stddef.h>
#include <stdio.h>

#include "vla.h"

#define F(T, f) printf(#T "." #f " %zu\n", offsetof(T, f))

int main(void) {
    printf("VLA_ABI_VERSION %d\n", VLA_ABI_VERSION);
    printf("status %d %d %d %d\n", VLA_OK, VLA_ERR_ARG, VLA_ERR_PREDICT, VLA_ERR_EXCEPTION);
    printf("pixel %d %d timing %d %d\n", VLA_PIXEL_U8, VLA_PIXEL_F32_RGB_01, VLA_TIMING_NONE, VLA_TIMING_PHASE);
    printf("sizeof.vla_config %zu\n", sizeof(vla_config));
    F(vla_config, n_img); F(vla_config, n_lang); F(vla_config, n_state); F(vla_config, n_prefix);
    F(vla_config, n_suffix); F(vla_config, n_full); F(vla_config, hidden); F(vla_config, expert_h);
    F(vla_config, intermediate); F(vla_config, expert_inter); F(vla_config, n_q_heads); F(vla_config, n_kv_heads);
    F(vla_config, head_dim); F(vla_config, q_full_dim); F(vla_config, kv_full_dim); F(vla_config, n_layers);
    F(vla_config, self_attn_every_n); F(vla_config, max_state_dim); F(vla_config, max_action_dim);
    F(vla_config, real_state_dim); F(vla_config, real_action_dim); F(vla_config, norm_eps);
    F(vla_config, min_period); F(vla_config, max_period); F(vla_config, num_steps); F(vla_config, rms_eps);
    F(vla_config, rope_n_dims); F(vla_config, rope_mode); F(vla_config, rope_freq_base); F(vla_config, denormalized);
    printf("sizeof.vla_image %zu\n", sizeof(vla_image));
    F(vla_image, data); F(vla_image, w); F(vla_image, h); F(vla_image, format);
    printf("sizeof.vla_inputs %zu\n", sizeof(vla_inputs));
    F(vla_inputs, images); F(vla_inputs, n_images); F(vla_inputs, precomputed_img_emb); F(vla_inputs, n_img_views);
    F(vla_inputs, lang_tokens); F(vla_inputs, n_lang); F(vla_inputs, state); F(vla_inputs, noise);
    F(vla_inputs, attention_mask); F(vla_inputs, attention_mask_n); F(vla_inputs, timing_detail);
    printf("sizeof.vla_stats %zu\n", sizeof(vla_stats));
    F(vla_stats, ms_total); F(vla_stats, ms_vision); F(vla_stats, ms_inference); F(vla_stats, ms_prefill);
    F(vla_stats, ms_denoise);
    return 0;
}
