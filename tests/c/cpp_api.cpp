// Compiles against include/vla_model.hpp the way a program written for the reference's src/model.h would:
// no model, then (argv[1]) a metadata-only checkpoint.
#include <cstdio>

#include "vla_model.hpp"

int main(int argc, char **argv) {
    int bad = 0;
    vla::model_free(nullptr);
    if (vla::model_load("", "/nonexistent.gguf") != nullptr) ++bad;
    vla::Inputs in;
    if (!vla::predict(nullptr, in).empty()) ++bad;
    vla::Config c{};
    c.real_action_dim = 9;
    c.max_action_dim = 8;
    if (vla::config_is_sane(c)) ++bad;
    c.real_action_dim = 7;
    if (!vla::config_is_sane(c)) ++bad;
    if (argc > 1) {
        vla::Model *m = vla::model_load("", argv[1]);
        if (!m) {
            ++bad;
        } else {
            const vla::Config &cfg = vla::model_config(m);
            std::printf("cpp api: expert_h=%lld n_suffix=%lld steps=%d\n", (long long)cfg.expert_h, (long long)cfg.n_suffix,
                        cfg.num_steps);
            if (vla::last_stats(m).ms_total != 0.f) ++bad;
            vla::model_free(m);
        }
    }
    std::printf(bad ? "cpp api: %d check(s) failed\n" : "cpp api: ok\n", bad);
    return bad ? 1 : 0;
}
