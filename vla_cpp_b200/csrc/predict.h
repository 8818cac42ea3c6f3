// One observation end to end on the device: prefix producer (language / image / state embeddings through
// the VLM layers into the K/V pages) followed by the denoise engine.  Used by the vla.h C ABI.
#pragma once
#include <vector>

#include "../../include/vla.h"
#include "host_common.h"

namespace vb {

struct Predictor;

// Builds the device-side objects of a loaded checkpoint (needs a GPU); nullptr on failure (last error set).
Predictor *predictor_create(const vlab200_gguf *g, const char *arch, const vla_config *cfg);
void predictor_free(Predictor *p);
// Runs one observation; fills `actions` ([n_suffix][max_action_dim], un-normalised) and the phase timings.
int predictor_run(Predictor *p, const vla_inputs *in, std::vector<float> *actions, vla_stats *stats);

}  // namespace vb
