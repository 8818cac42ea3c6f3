// Device side of vla_predict.
#include "predict.h"

namespace vb {

struct Predictor {};

Predictor *predictor_create(const vlab200_gguf *, const char *, const vla_config *) {
    set_last_error("vla_predict: the prefix producer (VLM prefill) is not part of this build");
    return nullptr;
}

void predictor_free(Predictor *p) { delete p; }

int predictor_run(Predictor *, const vla_inputs *, std::vector<float> *, vla_stats *) { return VLAB200_ERR_UNSUPPORTED; }

}  // namespace vb
