// Host-side drivers (C++) of the denoise hot path: the layer x step loop of the isolated
// denoise-attention op, with device-resident or host-resident hidden states.
//
// The reference unrolls steps x layers into one ggml graph (src/models/smolvla.cpp:1393-1419,
// src/models/pi0.cpp:570-588) and walks it node by node; here each layer-step is two kernel
// launches (fused QKV+RoPE+append, attention) on one stream.
#include <cuda_bf16.h>

#include <cstdint>
#include <mutex>
#include <vector>

#include "host_common.h"

namespace vb {

static int check_loop_args(const vlab200_kv_store *st, const vlab200_denoise_attn_args *a) {
    if (!st || !a) return VLAB200_ERR_ARG;
    if (a->n_layers <= 0 || a->n_layers > st->n_layers || a->steps <= 0 || a->S <= 0 || a->H <= 0 || a->n_q <= 0)
        return VLAB200_ERR_ARG;
    if (!a->x || !a->wqkv || !a->rope_cos || !a->rope_sin || !a->q_scratch || !a->out)
        return VLAB200_ERR_ARG;
    return VLAB200_OK;
}

static int run_layer_step(const vlab200_kv_store *st, const vlab200_denoise_attn_args *a, int layer,
                          const void *x_layer, void *out_layer, cudaStream_t cs) {
    const size_t w_elems = (size_t)(a->n_q + 2 * st->n_kv) * st->head_dim * a->H;
    const void *w = static_cast<const __nv_bfloat16 *>(a->wqkv) + (size_t)layer * w_elems;
    int rc = vlab200_qkv_rope_append(st, layer, x_layer, a->x_is_f32, a->ln_w ? a->ln_w + (size_t)layer * a->H : nullptr, w, a->rope_cos,
                                     a->rope_sin, a->eps, a->S, a->H, a->n_q, 1, a->q_scratch, cs);
    if (rc) return rc;
    return vlab200_attention(st, layer, a->q_scratch, out_layer, a->S, a->n_q, st->prefix_len + a->S, a->mask_mode,
                             a->pad_ranges, cs);
}

// Scratch for vlab200_denoise_attn_loop_static: lives in the library image, so every device
// that loads the library carries these bytes until the process exits.
constexpr size_t kStaticQBytes = (size_t)16 << 20;
static __device__ __align__(256) unsigned char g_static_q_scratch[kStaticQBytes];

// The array name is only a host-side handle; kernels need its device address.  Looked up once
// per device, with that device current.
static int static_q_scratch_ptr(void **out) {
    static void *ptrs[64] = {nullptr};
    static std::mutex mu;
    int dev = 0;
    VB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return VLAB200_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lk(mu);
    if (!ptrs[dev]) {
        void *p = nullptr;
        VB_CUDA(cudaGetSymbolAddress(&p, g_static_q_scratch));
        ptrs[dev] = p;
    }
    *out = ptrs[dev];
    return VLAB200_OK;
}

}  // namespace vb

extern "C" {

int32_t vlab200_denoise_attn_loop(const vlab200_kv_store *st, const vlab200_denoise_attn_args *a, void *stream) {
    int rc = vb::check_loop_args(st, a);
    if (rc) return rc;
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    const size_t x_elem = a->x_is_f32 ? 4 : 2;
    const size_t x_layer_bytes = (size_t)st->n_obs * a->S * a->H * x_elem;
    const size_t out_layer_elems = (size_t)st->n_obs * a->S * a->n_q * st->head_dim;
    for (int step = 0; step < a->steps; ++step)
        for (int l = 0; l < a->n_layers; ++l) {
            const char *x = static_cast<const char *>(a->x) + ((size_t)step * a->n_layers + l) * x_layer_bytes;
            void *out = static_cast<__nv_bfloat16 *>(a->out) + (size_t)l * out_layer_elems;
            rc = vb::run_layer_step(st, a, l, x, out, cs);
            if (rc) return rc;
        }
    return VLAB200_OK;
}

int32_t vlab200_denoise_attn_loop_static(const vlab200_kv_store *st, const vlab200_denoise_attn_args *a,
                                         void *stream) {
    if (!st || !a) return VLAB200_ERR_ARG;
    if (st->n_obs <= 0 || a->n_q <= 0 || a->S <= 0 || st->head_dim <= 0) return VLAB200_ERR_ARG;
    // every factor is bounded before the product is formed, so the size cannot wrap
    constexpr int32_t kMaxFactor = 1 << 20;
    const bool absurd = st->n_obs > kMaxFactor || a->n_q > kMaxFactor || a->S > kMaxFactor || st->head_dim > 1024;
    const size_t need = absurd ? SIZE_MAX : (size_t)st->n_obs * a->n_q * ((size_t)a->S * st->head_dim * 2);
    if (absurd || (size_t)st->n_obs * a->n_q > ((size_t)1 << 40) || need > vb::kStaticQBytes) {
        vb::set_last_error("vlab200_denoise_attn_loop_static: the query buffer needs %zu bytes, the built-in scratch "
                           "holds %zu; use vlab200_denoise_attn_loop with a caller-provided q_scratch",
                           need, vb::kStaticQBytes);
        return VLAB200_ERR_UNSUPPORTED;
    }
    void *q = nullptr;
    int rc = vb::static_q_scratch_ptr(&q);
    if (rc) return rc;
    vlab200_denoise_attn_args b = *a;
    b.q_scratch = q;
    return vlab200_denoise_attn_loop(st, &b, stream);
}

int32_t vlab200_denoise_attn_loop_host(const vlab200_kv_store *st, const vlab200_denoise_attn_args *a,
                                       void *x_stage, void *out_host, void *stream) {
    int rc = vb::check_loop_args(st, a);
    if (rc) return rc;
    if (!x_stage || !out_host) return VLAB200_ERR_ARG;
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    const size_t x_elem = a->x_is_f32 ? 4 : 2;
    const size_t x_layer_bytes = (size_t)st->n_obs * a->S * a->H * x_elem;
    const size_t x_step_bytes = x_layer_bytes * a->n_layers;
    const size_t out_layer_elems = (size_t)st->n_obs * a->S * a->n_q * st->head_dim;
    // copy stream + events: step s+1's hidden states travel while step s computes
    // one set per (calling thread, device): streams and events belong to the device that was current
    // when they were created; they live until the thread exits
    struct CopyLane {
        cudaStream_t stream = nullptr;
        cudaEvent_t copied[2] = {nullptr, nullptr}, consumed[2] = {nullptr, nullptr};
    };
    static thread_local CopyLane lanes[64];
    int dev = 0;
    VB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return VLAB200_ERR_UNSUPPORTED;
    cudaStream_t &copy_stream = lanes[dev].stream;
    cudaEvent_t *ev_copied = lanes[dev].copied, *ev_consumed = lanes[dev].consumed;
    if (!copy_stream) {
        VB_CUDA(cudaStreamCreateWithFlags(&copy_stream, cudaStreamNonBlocking));
        for (int i = 0; i < 2; ++i) {
            VB_CUDA(cudaEventCreateWithFlags(&ev_copied[i], cudaEventDisableTiming));
            VB_CUDA(cudaEventCreateWithFlags(&ev_consumed[i], cudaEventDisableTiming));
        }
    }
    // order the first copy after whatever the caller queued on `stream`
    VB_CUDA(cudaEventRecord(ev_consumed[0], cs));
    VB_CUDA(cudaEventRecord(ev_consumed[1], cs));
    for (int step = 0; step < a->steps; ++step) {
        const int buf = step & 1;
        char *stage = static_cast<char *>(x_stage) + (size_t)buf * x_step_bytes;
        VB_CUDA(cudaStreamWaitEvent(copy_stream, ev_consumed[buf], 0));
        VB_CUDA(cudaMemcpyAsync(stage, static_cast<const char *>(a->x) + (size_t)step * x_step_bytes, x_step_bytes,
                                cudaMemcpyHostToDevice, copy_stream));
        VB_CUDA(cudaEventRecord(ev_copied[buf], copy_stream));
        VB_CUDA(cudaStreamWaitEvent(cs, ev_copied[buf], 0));
        for (int l = 0; l < a->n_layers; ++l) {
            void *out = static_cast<__nv_bfloat16 *>(a->out) + (size_t)l * out_layer_elems;
            rc = vb::run_layer_step(st, a, l, stage + (size_t)l * x_layer_bytes, out, cs);
            if (rc) return rc;
        }
        VB_CUDA(cudaEventRecord(ev_consumed[buf], cs));
    }
    VB_CUDA(cudaMemcpyAsync(out_host, a->out, out_layer_elems * a->n_layers * 2, cudaMemcpyDeviceToHost, cs));
    return VLAB200_OK;
}

}  // extern "C"
