// The whole Euler loop of one observation as ONE persistent kernel (chunk_loop.cu); built and owned by the engine.
#pragma once
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

namespace vb {

// What the loop kernel needs from an engine: sizes and device pointers (prepared weights, pages of observation 0, the
// float32 residual stream and x).  Arrays indexed by layer are host arrays of device pointers.  The loop keeps its own
// bf16 activations, q and K/V pages in the padded layout its tiles are copied from, and a padded copy of every weight.
struct ChunkLoopDesc {
    int model;  // 0 pi0 (state token, row 0 private), 1 SmolVLA (causal suffix, cross layers), 2 pi0.5 (adaptive norms, no mask)
    int L, H, I, n_q, n_kv, hd, S, chunk, A, sd, steps, cap, P, act;
    float rms_eps;
    const int *is_self;
    const void *const *wqkv, *const *wo, *const *wgu, *const *wdown;
    const void *w_ain, *w_sp, *w_at1l, *w_at2, *w_aout;
    const float *b_ain, *b_sp, *tvec, *b_at2, *b_aout;
    void *k_pages, *v_pages;    // bf16 [L][max_obs][n_kv][cap][hd]; the loop uses observation 0
    size_t layer_stride;        // elements between two layers' pages
    float *h, *x;               // f32 [S][H], [chunk][A]
    const float *rope_self, *rope_cross;  // [2][S][hd/2] (cos | sin)
    // pi0.5: float32 [L][2][steps][3H] (scale | shift | gate of the layer's two norms for every step), then [steps][3H] final
    const float *mods;
};

struct ChunkLoop;

// Builds the phase table for `d` on the current device.  VLAB200_ERR_UNSUPPORTED when the shapes do not fit the
// kernel's shared-memory plan (the caller then keeps the launch-per-operator path).
int chunk_loop_create(const ChunkLoopDesc &d, ChunkLoop **out);
void chunk_loop_free(ChunkLoop *cl);
// One chunk: x (in place, [chunk][A] float32) through `steps` Euler steps.  state: [sd] float32 (pi0), pad: two int32
// (key range hidden from every row) or nullptr.  Both are device pointers read by the kernel.  VLAB200_ERR_UNSUPPORTED (nothing
// launched, x untouched) when the grid cannot be co-resident because part of the device is not available to this process.
int chunk_loop_run(ChunkLoop *cl, const float *state, const int32_t *pad, cudaStream_t stream);
int chunk_loop_phases(const ChunkLoop *cl);  // phases (= grid-wide barriers) per Euler step

}  // namespace vb
