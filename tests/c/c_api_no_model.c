/* The part of the C ABI contract that needs no checkpoint: version, NULL handles, status codes.
 * Compiled as C so that include/vla.h stays C-clean.  Same contract as the reference's
 * tests/test_c_api.c:33-49 checks on its own library.  argv[1], when given, is a GGUF file whose
 * metadata must load and resolve (no GPU involved). */
#include <stdio.h>
#include <string.h>

#include "vla.h"

static int bad = 0;
#define EXPECT(cond)                                        \
    do {                                                    \
        if (!(cond)) {                                      \
            printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); \
            ++bad;                                          \
        }                                                   \
    } while (0)

int main(int argc, char **argv) {
    vla_config cfg;
    vla_stats st;
    vla_inputs in;
    float *actions = (float *)&bad; /* must be reset to NULL by a failing predict only after the handle check */
    int64_t n = 7;
    memset(&in, 0, sizeof in);

    EXPECT(vla_abi_version() == VLA_ABI_VERSION);
    vla_model_free(NULL);
    vla_free_actions(NULL);
    EXPECT(vla_model_load(NULL, NULL, NULL) == NULL);
    EXPECT(vla_model_load("", "/nonexistent/file.gguf", NULL) == NULL);
    EXPECT(vla_model_config(NULL, &cfg) == VLA_ERR_ARG);
    EXPECT(vla_last_stats(NULL, &st) == VLA_ERR_ARG);
    EXPECT(vla_predict(NULL, &in, &actions, &n) == VLA_ERR_ARG);

    if (argc > 1) {
        vla_model *m = vla_model_load(NULL, argv[1], NULL);
        EXPECT(m != NULL);
        if (m) {
            EXPECT(vla_model_config(m, NULL) == VLA_ERR_ARG);
            EXPECT(vla_model_config(m, &cfg) == VLA_OK);
            EXPECT(vla_predict(m, NULL, &actions, &n) == VLA_ERR_ARG);
            EXPECT(vla_predict(m, &in, NULL, &n) == VLA_ERR_ARG);
            in.n_lang = -1;
            EXPECT(vla_predict(m, &in, &actions, &n) == VLA_ERR_ARG);
            EXPECT(actions == NULL && n == 0); /* outputs are cleared before the inputs are validated */
            in.n_lang = 3;                     /* tokens announced but not given */
            EXPECT(vla_predict(m, &in, &actions, &n) == VLA_ERR_ARG);
            EXPECT(vla_last_stats(m, &st) == VLA_OK);
            printf("config hidden=%lld expert_h=%lld n_layers=%lld n_suffix=%lld n_lang=%lld n_img=%lld q_full=%lld "
                   "kv_full=%lld steps=%d every=%d rms_eps=%g rope=%g min=%g max=%g denorm=%d\n",
                   (long long)cfg.hidden, (long long)cfg.expert_h, (long long)cfg.n_layers, (long long)cfg.n_suffix,
                   (long long)cfg.n_lang, (long long)cfg.n_img, (long long)cfg.q_full_dim, (long long)cfg.kv_full_dim,
                   cfg.num_steps, cfg.self_attn_every_n, (double)cfg.rms_eps, (double)cfg.rope_freq_base,
                   cfg.min_period, cfg.max_period, cfg.denormalized);
            vla_model_free(m);
        }
    }
    printf(bad ? "c api: %d check(s) failed\n" : "c api: ok\n", bad);
    return bad ? 1 : 0;
}
