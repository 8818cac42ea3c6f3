// BitVLA's float32 proprioception projector and action head under the reference's own context API:
// bitvla_fp32head_cuda_init / bitvla_fp32head_proprio_forward / bitvla_fp32head_action_forward /
// bitvla_fp32head_cuda_free (src/kernels/bitvla/bitvla_fp32head_cuda.h:66-129; bodies
// src/kernels/bitvla/bitvla_fp32head_cuda.cu:186-358).
//
//   proprio:  out = W2 . gelu_erf(W1 . state + b1) + b2                                   (one row)
//   action:   x = LayerNorm1(in)  [chunk rows of action_dim * hidden]
//             h = relu(W_fc1 x + b);  h += relu(W_b0 LayerNorm(h) + b);  h += relu(W_b1 LayerNorm(h) + b)
//             out = W_fc2 LayerNorm2(h) + b                                                [chunk][action_dim]
//
// Everything stays float32, as in the reference (it keeps these small layers out of the ternary path to preserve the
// regression accuracy of the continuous outputs).  With at most `chunk` (8) rows every product is a skinny
// matrix-vector problem bound by streaming the float32 weights from HBM once (fc1 of the head: 2560 x 17920 x 4 B =
// 183 MB): f32_skinny_linear_kernel gives each warp two weight rows, read with 16-byte loads and multiplied against an
// activation tile staged in shared memory; bias, ReLU / erf-GELU and the residual add ride in its epilogue.  The
// reference issues a cuBLAS SGEMM plus separate bias, activation and add kernels (19 launches per action forward;
// 9 here).
#include <cuda_runtime.h>

#include <cstdio>
#include <new>

#include "host_common.h"
#include "tc5.cuh"

namespace vb {

constexpr int SK_ROWS = 8;      // activation rows per pass
constexpr int SK_KT = 1024;     // activation tile (floats per row) in shared memory
constexpr int SK_COLS = 16;     // weight rows (output columns) per CTA: 8 warps x 2
enum { SK_ACT_NONE = 0, SK_ACT_RELU = 1, SK_ACT_GELU_ERF = 2, SK_ACT_SILU = 3 };

// out[m][n] = (residual ? residual[m][n] : 0) + act(bias[n] + sum_k x[m][k] W[n][k]),  m in [m0, m0 + rows)
__global__ void __launch_bounds__(256) f32_skinny_linear_kernel(const float *__restrict__ W, const float *__restrict__ bias,
                                                                const float *__restrict__ x, const float *residual, float *out,
                                                                int m0, int rows, int N, int K, int act) {
    __shared__ __align__(16) float xs[SK_ROWS][SK_KT];
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_base = blockIdx.x * SK_COLS + warp * 2;
    float acc[2][SK_ROWS];
#pragma unroll
    for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int m = 0; m < SK_ROWS; ++m) acc[c][m] = 0.0f;
    const bool vec = (K & 3) == 0;
    constexpr int NJ = SK_KT / 128;  // float4 loads per lane, weight row and tile
    // both weight rows of the warp against one read of the activation tile; a row past N re-reads the last valid one
    // (its sums are dropped at the end)
    const bool active = n_base < N;
    const float *wa = W + (size_t)(active ? n_base : 0) * K;
    const float *wb = W + (size_t)(active ? min(n_base + 1, N - 1) : 0) * K;
    for (int k0 = 0; k0 < K; k0 += SK_KT) {
        const int kt = min(SK_KT, K - k0);
        // the tile's weights go into registers first (16 x 16 B in flight per lane): their HBM latency overlaps the
        // staging of the activation tile below
        float4 a4[NJ], b4[NJ];
        if (vec && active) {
#pragma unroll
            for (int j = 0; j < NJ; ++j) {
                const int k = lane * 4 + 128 * j;
                a4[j] = k < kt ? __ldg(reinterpret_cast<const float4 *>(wa + k0 + k)) : make_float4(0.f, 0.f, 0.f, 0.f);
                b4[j] = k < kt ? __ldg(reinterpret_cast<const float4 *>(wb + k0 + k)) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
        __syncthreads();  // the previous tile has been consumed
        for (int m = 0; m < SK_ROWS; ++m) {
            const float *xr = x + (size_t)(m0 + m) * K + k0;
            for (int k = threadIdx.x; k < SK_KT; k += 256) xs[m][k] = (m < rows && k < kt) ? xr[k] : 0.0f;
        }
        __syncthreads();
        if (!active) continue;
        if (vec) {
#pragma unroll
            for (int j = 0; j < NJ; ++j) {
                const int k = lane * 4 + 128 * j;
#pragma unroll
                for (int m = 0; m < SK_ROWS; ++m) {
                    const float4 x4 = *reinterpret_cast<const float4 *>(&xs[m][k]);
                    acc[0][m] = fmaf(a4[j].x, x4.x, fmaf(a4[j].y, x4.y, fmaf(a4[j].z, x4.z, fmaf(a4[j].w, x4.w, acc[0][m]))));
                    acc[1][m] = fmaf(b4[j].x, x4.x, fmaf(b4[j].y, x4.y, fmaf(b4[j].z, x4.z, fmaf(b4[j].w, x4.w, acc[1][m]))));
                }
            }
        } else {
            for (int k = lane; k < kt; k += 32) {
                const float a1 = __ldg(wa + k0 + k), b1 = __ldg(wb + k0 + k);
#pragma unroll
                for (int m = 0; m < SK_ROWS; ++m) {
                    acc[0][m] = fmaf(a1, xs[m][k], acc[0][m]);
                    acc[1][m] = fmaf(b1, xs[m][k], acc[1][m]);
                }
            }
        }
    }
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        const int n = n_base + c;
#pragma unroll
        for (int m = 0; m < SK_ROWS; ++m) {
            float v = acc[c][m];
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
            if (lane == 0 && n < N && m < rows) {
                v += bias ? bias[n] : 0.0f;
                if (act == SK_ACT_RELU) v = fmaxf(v, 0.0f);
                else if (act == SK_ACT_GELU_ERF) v = 0.5f * v * (1.0f + erff(v * 0.70710678118654752440f));
                else if (act == SK_ACT_SILU) v = v / (1.0f + expf(-v));
                const size_t o = (size_t)(m0 + m) * N + n;
                out[o] = residual ? residual[o] + v : v;
            }
        }
    }
}

// (x - mean) * rsqrt(var + eps) * w + b over rows of K floats: the mean, then the variance of the centred values
// (layernorm_fp32_kernel, bitvla_fp32head_cuda.cu:71-117)
__global__ void __launch_bounds__(256) f32_layernorm_kernel(const float *__restrict__ x, const float *__restrict__ w,
                                                            const float *__restrict__ b, float *__restrict__ out, float eps, int K) {
    __shared__ float red[8];
    pdl_launch_dependents();
    pdl_wait();
    const float *row = x + (size_t)blockIdx.x * K;
    float *o = out + (size_t)blockIdx.x * K;
    auto block_sum = [&](float v) {
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
        __syncthreads();
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
        __syncthreads();
        float t = red[0];
#pragma unroll
        for (int i = 1; i < 8; ++i) t += red[i];
        return t;
    };
    // rows of up to 256 x LN_CACHE floats are read from memory once and kept in registers
    constexpr int LN_CACHE = 72;
    float c[LN_CACHE];
    const bool cached = K <= 256 * LN_CACHE;
    float s = 0.0f;
    if (cached) {
#pragma unroll
        for (int j = 0; j < LN_CACHE; ++j) {
            const int k = threadIdx.x + 256 * j;
            c[j] = k < K ? row[k] : 0.0f;
            s += c[j];
        }
    } else {
        for (int k = threadIdx.x; k < K; k += 256) s += row[k];
    }
    const float mean = block_sum(s) / (float)K;
    float vs = 0.0f;
    if (cached) {
#pragma unroll
        for (int j = 0; j < LN_CACHE; ++j) {
            const float d = threadIdx.x + 256 * j < K ? c[j] - mean : 0.0f;
            vs = fmaf(d, d, vs);
        }
    } else {
        for (int k = threadIdx.x; k < K; k += 256) {
            const float d = row[k] - mean;
            vs = fmaf(d, d, vs);
        }
    }
    const float inv_std = rsqrtf(block_sum(vs) / (float)K + eps);
    if (cached) {
#pragma unroll
        for (int j = 0; j < LN_CACHE; ++j) {
            const int k = threadIdx.x + 256 * j;
            if (k < K) o[k] = fmaf((c[j] - mean) * inv_std, w[k], b[k]);
        }
    } else {
        for (int k = threadIdx.x; k < K; k += 256) o[k] = fmaf((row[k] - mean) * inv_std, w[k], b[k]);
    }
}

int skinny_linear(const float *W, const float *bias, const float *x, const float *residual, float *out, int M, int N, int K,
                  int act, cudaStream_t cs) {
    for (int m0 = 0; m0 < M; m0 += SK_ROWS) {
        const int rows = M - m0 < SK_ROWS ? M - m0 : SK_ROWS;
        int rc = launch_pdl(f32_skinny_linear_kernel, dim3((N + SK_COLS - 1) / SK_COLS), dim3(256), 0, cs, W, bias, x, residual, out, m0,
                            rows, N, K, act);
        if (rc) return rc;
    }
    return VLAB200_OK;
}

}  // namespace vb

struct bitvla_fp32head_cuda_ctx {
    int proprio_dim, hidden, chunk, action_dim, in_dim;
    float eps;
    vb::DevBuf w[20];  // in the order of the init arguments
    vb::DevBuf state, pp_h1, pp_out, ah_in, ah_norm, ah_h, ah_tmp, ah_out;
};

extern "C" {

bitvla_fp32head_cuda_ctx *bitvla_fp32head_cuda_init(int proprio_dim, int lm_hidden, int chunk, int action_dim, float ah_ln_eps,
                                                    const float *pp_fc1_w, const float *pp_fc1_b, const float *pp_fc2_w,
                                                    const float *pp_fc2_b, const float *ah_ln1_w, const float *ah_ln1_b,
                                                    const float *ah_fc1_w, const float *ah_fc1_b, const float *ah_b0_lnw,
                                                    const float *ah_b0_lnb, const float *ah_b0_w, const float *ah_b0_b,
                                                    const float *ah_b1_lnw, const float *ah_b1_lnb, const float *ah_b1_w,
                                                    const float *ah_b1_b, const float *ah_ln2_w, const float *ah_ln2_b,
                                                    const float *ah_fc2_w, const float *ah_fc2_b) {
    if (proprio_dim <= 0 || lm_hidden <= 0 || chunk <= 0 || action_dim <= 0) {
        std::fprintf(stderr, "vla_b200(bitvla_fp32head): bad dimensions\n");
        return nullptr;
    }
    auto *c = new (std::nothrow) bitvla_fp32head_cuda_ctx();
    if (!c) return nullptr;
    c->proprio_dim = proprio_dim; c->hidden = lm_hidden; c->chunk = chunk; c->action_dim = action_dim;
    c->in_dim = action_dim * lm_hidden;
    c->eps = ah_ln_eps;
    const size_t H = (size_t)lm_hidden, D = (size_t)c->in_dim;
    const float *host[20] = {pp_fc1_w, pp_fc1_b, pp_fc2_w, pp_fc2_b, ah_ln1_w, ah_ln1_b, ah_fc1_w, ah_fc1_b, ah_b0_lnw, ah_b0_lnb,
                             ah_b0_w, ah_b0_b, ah_b1_lnw, ah_b1_lnb, ah_b1_w, ah_b1_b, ah_ln2_w, ah_ln2_b, ah_fc2_w, ah_fc2_b};
    const size_t count[20] = {H * proprio_dim, H, H * H, H, D, D, H * D, H, H, H, H * H, H, H, H, H * H, H, H, H, (size_t)action_dim * H,
                              (size_t)action_dim};
    bool ok = true;
    for (int i = 0; i < 20 && ok; ++i) {
        ok = host[i] != nullptr && c->w[i].alloc(count[i] * 4) == VLAB200_OK &&
             cudaMemcpy(c->w[i].p, host[i], count[i] * 4, cudaMemcpyHostToDevice) == cudaSuccess;
    }
    const size_t M = (size_t)chunk;
    ok = ok && c->state.alloc((size_t)proprio_dim * 4) == VLAB200_OK && c->pp_h1.alloc(H * 4) == VLAB200_OK &&
         c->pp_out.alloc(H * 4) == VLAB200_OK && c->ah_in.alloc(M * D * 4) == VLAB200_OK && c->ah_norm.alloc(M * D * 4) == VLAB200_OK &&
         c->ah_h.alloc(M * H * 4) == VLAB200_OK && c->ah_tmp.alloc(M * H * 4) == VLAB200_OK &&
         c->ah_out.alloc(M * (size_t)action_dim * 4) == VLAB200_OK;
    if (!ok) {
        std::fprintf(stderr, "vla_b200(bitvla_fp32head): a weight pointer is null or a device allocation / upload failed\n");
        delete c;
        return nullptr;
    }
    return c;
}

void bitvla_fp32head_cuda_free(bitvla_fp32head_cuda_ctx *ctx) { delete ctx; }

int bitvla_fp32head_proprio_forward(bitvla_fp32head_cuda_ctx *ctx, const float *host_state, float *host_out, void *stream) {
    if (!ctx || !host_state || !host_out) return -1;
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    const int H = ctx->hidden;
    auto f = [&](int i) { return ctx->w[i].as<float>(); };
    bool ok = cudaMemcpyAsync(ctx->state.p, host_state, (size_t)ctx->proprio_dim * 4, cudaMemcpyHostToDevice, cs) == cudaSuccess;
    ok = ok && vb::skinny_linear(f(0), f(1), ctx->state.as<float>(), nullptr, ctx->pp_h1.as<float>(), 1, H, ctx->proprio_dim,
                                 vb::SK_ACT_GELU_ERF, cs) == VLAB200_OK;
    ok = ok && vb::skinny_linear(f(2), f(3), ctx->pp_h1.as<float>(), nullptr, ctx->pp_out.as<float>(), 1, H, H, vb::SK_ACT_NONE, cs) ==
                   VLAB200_OK;
    ok = ok && cudaMemcpyAsync(host_out, ctx->pp_out.p, (size_t)H * 4, cudaMemcpyDeviceToHost, cs) == cudaSuccess;
    ok = ok && cudaStreamSynchronize(cs) == cudaSuccess;
    if (!ok) {
        std::fprintf(stderr, "vla_b200(bitvla_fp32head): proprio forward failed: %s\n", cudaGetErrorString(cudaGetLastError()));
        return -1;
    }
    return 0;
}

int bitvla_fp32head_action_forward(bitvla_fp32head_cuda_ctx *ctx, const float *host_ah_input, float *host_norm_actions, void *stream) {
    if (!ctx || !host_ah_input || !host_norm_actions) return -1;
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    const int M = ctx->chunk, D = ctx->in_dim, H = ctx->hidden, A = ctx->action_dim;
    auto f = [&](int i) { return ctx->w[i].as<float>(); };
    float *in = ctx->ah_in.as<float>(), *big = ctx->ah_norm.as<float>(), *h = ctx->ah_h.as<float>(), *tmp = ctx->ah_tmp.as<float>(),
          *out = ctx->ah_out.as<float>();
    auto ln = [&](const float *x, int wi, float *y, int K) {
        return vb::launch_pdl(vb::f32_layernorm_kernel, dim3(M), dim3(256), 0, cs, x, static_cast<const float *>(f(wi)),
                              static_cast<const float *>(f(wi + 1)), y, ctx->eps, K) == VLAB200_OK;
    };
    bool ok = cudaMemcpyAsync(in, host_ah_input, (size_t)M * D * 4, cudaMemcpyHostToDevice, cs) == cudaSuccess;
    ok = ok && ln(in, 4, big, D);
    ok = ok && vb::skinny_linear(f(6), f(7), big, nullptr, h, M, H, D, vb::SK_ACT_RELU, cs) == VLAB200_OK;
    ok = ok && ln(h, 8, tmp, H);
    ok = ok && vb::skinny_linear(f(10), f(11), tmp, h, h, M, H, H, vb::SK_ACT_RELU, cs) == VLAB200_OK;  // h += relu(...)
    ok = ok && ln(h, 12, tmp, H);
    ok = ok && vb::skinny_linear(f(14), f(15), tmp, h, h, M, H, H, vb::SK_ACT_RELU, cs) == VLAB200_OK;
    ok = ok && ln(h, 16, tmp, H);
    ok = ok && vb::skinny_linear(f(18), f(19), tmp, nullptr, out, M, A, H, vb::SK_ACT_NONE, cs) == VLAB200_OK;
    ok = ok && cudaMemcpyAsync(host_norm_actions, out, (size_t)M * A * 4, cudaMemcpyDeviceToHost, cs) == cudaSuccess;
    ok = ok && cudaStreamSynchronize(cs) == cudaSuccess;
    if (!ok) {
        std::fprintf(stderr, "vla_b200(bitvla_fp32head): action forward failed: %s %s\n", cudaGetErrorString(cudaGetLastError()),
                     vlab200_last_error());
        return -1;
    }
    return 0;
}

}  // extern "C"
