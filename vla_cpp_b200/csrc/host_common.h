// Host-side helpers shared by the translation units of libvla_b200.so.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>

#include "../../include/vla_b200.h"

namespace vb {

// Pointer to the per-device status word (device memory) for the current device,
// or nullptr when no CUDA device can be used.
int *device_status_ptr();

// Number of SMs of the current device (looked up once per device); 0 when no device can be used.
int sm_count();

// Opts kernel `func` into `bytes` of dynamic shared memory on the current device.  The attribute is
// per device, so the call is remembered per (device, function) and repeated only when a larger
// size is asked for.  Thread-safe.
int ensure_dyn_smem(const void *func, int bytes);
template <typename F>
int ensure_dyn_smem(F *func, int bytes) {
    return ensure_dyn_smem(reinterpret_cast<const void *>(func), bytes);
}

// printf-style text for vlab200_last_error() on the calling thread.
void set_last_error(const char *fmt, ...);

// Records and returns a CUDA failure as VLAB200_ERR_CUDA.
int cuda_fail(cudaError_t e, const char *what);

#define VB_CUDA(expr)                                        \
    do {                                                     \
        cudaError_t _e = (expr);                             \
        if (_e != cudaSuccess) return vb::cuda_fail(_e, #expr); \
    } while (0)

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link-time libcuda).
// dims/strides innermost first; strides_bytes has rank-1 entries (dim 1 .. rank-1).
int make_tensor_map(CUtensorMap *map, CUtensorMapDataType dt, int rank, const void *base, const uint64_t *dims,
                    const uint64_t *strides_bytes, const uint32_t *box, CUtensorMapSwizzle swz);

// Launches `kernel` so that it may overlap the tail of the preceding kernel in `stream` (programmatic
// dependent launch).  Only for kernels that call pdl_wait() before their first access to global memory.
template <typename... KArgs, typename... Args>
int launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args &&...args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
    return e == cudaSuccess ? VLAB200_OK : cuda_fail(e, "cudaLaunchKernelEx");
}

// Owning device allocation (move-only).
struct DevBuf {
    void *p = nullptr;
    DevBuf() = default;
    DevBuf(const DevBuf &) = delete;
    DevBuf &operator=(const DevBuf &) = delete;
    DevBuf(DevBuf &&o) noexcept : p(o.p) { o.p = nullptr; }
    DevBuf &operator=(DevBuf &&o) noexcept {
        if (this != &o) {
            if (p) cudaFree(p);
            p = o.p;
            o.p = nullptr;
        }
        return *this;
    }
    int alloc(size_t bytes) {
        cudaError_t e = cudaMalloc(&p, bytes ? bytes : 16);
        return e == cudaSuccess ? VLAB200_OK : cuda_fail(e, "cudaMalloc");
    }
    ~DevBuf() {
        if (p) cudaFree(p);
    }
    template <typename T>
    T *as() const {
        return static_cast<T *>(p);
    }
};

// A checkpoint tensor ([d1][d0], d1 == 1 for vectors, d1 < 0: d0 elements of any shape; f32 / f16 / bf16 in the file) uploaded as bf16 or float32,
// optionally with the Gemma-norm "+1" (gguf.cu).  VLAB200_OK or an error with the last-error text set.
int gguf_upload(const vlab200_gguf *g, const char *name, int64_t d0, int64_t d1, bool as_bf16, bool gemma, DevBuf *out);

// vlab200_attention with an optional float workspace for the key-split path of calls with few work units (attn.cu).
int attention_ws(const vlab200_kv_store *st, int layer, const void *q, void *out, int S, int n_q, int kv_len, int mask_mode,
                 const int32_t *pad_ranges, cudaStream_t stream, float *ws, size_t ws_bytes);

// Float32 linear for a few rows (bitvla_fp32head.cu): out[m][n] = (residual ? residual[m][n] : 0) +
// act(bias[n] + sum_k x[m][k] W[n][k]), W float32 [N][K] streamed once; act 0 none, 1 ReLU, 2 erf-GELU, 3 SiLU.
int skinny_linear(const float *W, const float *bias, const float *x, const float *residual, float *out, int M, int N, int K,
                  int act, cudaStream_t cs);

}  // namespace vb
