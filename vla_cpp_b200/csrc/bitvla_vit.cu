// BitVLA vision tower (ternary SigLIP ViT + 2-layer projector) on this library's kernels, under the reference's own
// context API: bitvla_vit_cuda_init / _free / _set_layer / _set_embed / _set_mmproj / _forward
// (src/kernels/bitvla/bitvla_vit_cuda.h:86-144; forward and layer body src/kernels/bitvla/bitvla_vit_cuda.cu:161-330).
//
// The reference runs one layer as ~30 launches (LayerNorm, act-quant, three ternary GEMMs, three bias adds, three
// head transposes, cuBLAS QK^T with bf16 scores in HBM, softmax, cuBLAS PV, merge transpose, act-quant, GEMM, bias,
// add, LayerNorm, act-quant, GEMM, bias, GELU, padded copy, act-quant, GEMM, bias, add).  Here it is 10:
//
//   vit_ln_quant_kernel      [h += bf16(proj + bias) ->] LayerNorm -> bf16 -> per-token absmax int8
//   ternary GEMM             q | k | v as one matrix (packs concatenated at set_layer, three weight scales)
//   vit_split_heads_kernel   + bias, head split, head_dim zero-padded to the attention kernel's width
//   attention                streaming tcgen05 kernel (float scores on chip), softmax scale 1 / sqrt(real head_dim)
//   vit_merge_quant_kernel   heads back to [seq][hidden] -> act-quant
//   ternary GEMM             o
//   vit_ln_quant_kernel      h += bf16(o + bias); LayerNorm 2 -> int8
//   ternary GEMM             fc1
//   vit_gelu_quant_kernel    + bias -> tanh-GELU -> bf16, zero-padded to a multiple of 128 -> act-quant
//   ternary GEMM             fc2   (its bias and residual add are fused into the next vit_ln_quant_kernel)
//
// Every value the reference stores as bf16 is rounded to bf16 here too, in the same order; the patch embedding and the
// projector run on the bf16 tcgen05 GEMM with the bias (and erf-GELU) in the epilogue.
#include <cuda_bf16.h>

#include <cmath>
#include <cstdio>
#include <new>
#include <vector>

#include "gemm.h"
#include "host_common.h"
#include "tc5.cuh"

namespace vb {

int attention_flash(const vlab200_kv_store *st, int layer, const void *q, void *out, int S, int n_q, int kv_len,
                    int mask_mode, const int32_t *pad_ranges, cudaStream_t stream, float softmax_scale, float *ws, size_t ws_bytes);

__device__ __forceinline__ float vit_block_sum(float v, float *red) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = red[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) t += red[i];
    return t;
}

__device__ __forceinline__ float vit_block_max(float v, float *red) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = red[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) t = fmaxf(t, red[i]);
    return t;
}

// the tail shared by the three row kernels: row[] holds K_q bf16-representable floats (zeros past the real width);
// scale = 127 / max(amax, 1e-5), q = clamp(rne(y * scale), -128, 127)  (src/kernels/bitvla/bitnet_kernels.h:465-521)
__device__ __forceinline__ void vit_quant_row(const float *row, float amax, int K_q, int8_t *q_out, float *s_out, float *red) {
    amax = vit_block_max(amax, red);
    amax = amax < 1e-5f ? 1e-5f : amax;
    const float qs = __fdiv_rn(127.0f, amax);
    if (threadIdx.x == 0) *s_out = qs;
    for (int k = threadIdx.x; k < K_q; k += 256)
        q_out[k] = (signed char)(int)fminf(fmaxf(rintf(row[k] * qs), -128.f), 127.f);
}

// One CTA per token.  add != nullptr: h[m][k] = bf16(h + bf16(add[m][k] + add_bias[k])) first (bitvla_add_bias_bf16 +
// bitvla_add_bf16, bitvla_vit_cuda.cu:226-227,246-247).  ln_w == nullptr: only that update.  Otherwise
// y = bf16((h - mean) * rsqrt(var + eps) * w + b) with the mean and the centred variance of the bf16 row in float
// (layernorm_bias_bf16_kernel, bitvla_lm_cuda.cu:552-607), then the act-quant of y.
__global__ void __launch_bounds__(256) vit_ln_quant_kernel(__nv_bfloat16 *__restrict__ h, const __nv_bfloat16 *__restrict__ add,
                                                           const __nv_bfloat16 *__restrict__ add_bias,
                                                           const __nv_bfloat16 *__restrict__ ln_w,
                                                           const __nv_bfloat16 *__restrict__ ln_b, float eps, int K,
                                                           int8_t *__restrict__ q_out, float *__restrict__ s_out) {
    extern __shared__ float row[];
    __shared__ float red[8];
    pdl_launch_dependents();
    pdl_wait();
    const int m = blockIdx.x, tid = threadIdx.x;
    __nv_bfloat16 *hr = h + (size_t)m * K;
    float sum = 0.f;
    for (int k = tid; k < K; k += 256) {
        float x = __bfloat162float(hr[k]);
        if (add) {
            const float o = __bfloat162float(__float2bfloat16(__bfloat162float(add[(size_t)m * K + k]) + __bfloat162float(add_bias[k])));
            const __nv_bfloat16 r = __float2bfloat16(x + o);
            hr[k] = r;
            x = __bfloat162float(r);
        }
        row[k] = x;
        sum += x;
    }
    if (!ln_w) return;
    const float mean = vit_block_sum(sum, red) / (float)K;
    float vs = 0.f;
    for (int k = tid; k < K; k += 256) {
        const float d = row[k] - mean;
        vs += d * d;
    }
    const float inv_std = rsqrtf(vit_block_sum(vs, red) / (float)K + eps);
    float amax = 0.f;
    for (int k = tid; k < K; k += 256) {
        const float y = __bfloat162float(__float2bfloat16(fmaf((row[k] - mean) * inv_std, __bfloat162float(ln_w[k]), __bfloat162float(ln_b[k]))));
        row[k] = y;
        amax = fmaxf(amax, fabsf(y));
    }
    vit_quant_row(row, amax, K, q_out + (size_t)m * K, s_out + m, red);
}

// qkv [seq][3 H] (q | k | v) + bias -> q [heads][seq][hd_pad], K / V pages [heads][seq][hd_pad], zero past hd.
// (bitvla_add_bias_bf16 + bitvla_transpose_sNhd_to_NshHd_bf16, bitvla_vit_cuda.cu:185-195)
// One CTA per token; a thread moves 8 consecutive head-dim elements (16 bytes) at a time when hd % 8 == 0.
__global__ void __launch_bounds__(256) vit_split_heads_kernel(const __nv_bfloat16 *__restrict__ qkv, const __nv_bfloat16 *__restrict__ bq,
                                                              const __nv_bfloat16 *__restrict__ bk, const __nv_bfloat16 *__restrict__ bv,
                                                              __nv_bfloat16 *__restrict__ q, __nv_bfloat16 *__restrict__ kp,
                                                              __nv_bfloat16 *__restrict__ vp, int seq, int heads, int hd, int hd_pad) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, H = heads * hd;
    const __nv_bfloat16 *src = qkv + (size_t)t * 3 * H;
    const bool al16 = ((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(bq) | reinterpret_cast<uintptr_t>(bk) |
                        reinterpret_cast<uintptr_t>(bv)) & 15) == 0;
    if ((hd & 7) == 0 && al16) {
        const int cpr = hd_pad >> 3;  // 16-byte chunks per padded head row
        for (int i = threadIdx.x; i < 3 * heads * cpr; i += blockDim.x) {
            const int which = i / (heads * cpr), r = i % (heads * cpr), hh = r / cpr, d = (r % cpr) * 8;
            uint4 out = make_uint4(0u, 0u, 0u, 0u);
            if (d < hd) {
                const __nv_bfloat16 *b = which == 0 ? bq : (which == 1 ? bk : bv);
                const uint4 xv = *reinterpret_cast<const uint4 *>(src + which * H + hh * hd + d);
                const uint4 bvv = *reinterpret_cast<const uint4 *>(b + hh * hd + d);
                const __nv_bfloat162 *x2 = reinterpret_cast<const __nv_bfloat162 *>(&xv);
                const __nv_bfloat162 *b2 = reinterpret_cast<const __nv_bfloat162 *>(&bvv);
                __nv_bfloat162 *o2 = reinterpret_cast<__nv_bfloat162 *>(&out);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 xf = __bfloat1622float2(x2[e]), bf = __bfloat1622float2(b2[e]);
                    o2[e] = __floats2bfloat162_rn(xf.x + bf.x, xf.y + bf.y);
                }
            }
            __nv_bfloat16 *dst = which == 0 ? q : (which == 1 ? kp : vp);
            *reinterpret_cast<uint4 *>(dst + ((size_t)hh * seq + t) * hd_pad + d) = out;
        }
        return;
    }
    for (int i = threadIdx.x; i < 3 * heads * hd_pad; i += blockDim.x) {
        const int which = i / (heads * hd_pad), r = i % (heads * hd_pad), hh = r / hd_pad, d = r % hd_pad;
        __nv_bfloat16 val = __float2bfloat16(0.0f);
        if (d < hd) {
            const __nv_bfloat16 *b = which == 0 ? bq : (which == 1 ? bk : bv);
            val = __float2bfloat16(__bfloat162float(src[which * H + hh * hd + d]) + __bfloat162float(b[hh * hd + d]));
        }
        __nv_bfloat16 *dst = which == 0 ? q : (which == 1 ? kp : vp);
        dst[((size_t)hh * seq + t) * hd_pad + d] = val;
    }
}

// attention output [seq][heads * hd_pad] -> the real head_dim columns [seq][H] -> act-quant
// (bitvla_transpose_NshHd_to_sNhd_bf16 + bitvla_act_quant_cuda, bitvla_vit_cuda.cu:222-223)
__global__ void __launch_bounds__(256) vit_merge_quant_kernel(const __nv_bfloat16 *__restrict__ att, int heads, int hd, int hd_pad,
                                                              int8_t *__restrict__ q_out, float *__restrict__ s_out) {
    extern __shared__ float row[];
    __shared__ float red[8];
    pdl_launch_dependents();
    pdl_wait();
    const int m = blockIdx.x, K = heads * hd;
    float amax = 0.f;
    for (int k = threadIdx.x; k < K; k += 256) {
        const float y = __bfloat162float(att[((size_t)m * heads + k / hd) * hd_pad + k % hd]);
        row[k] = y;
        amax = fmaxf(amax, fabsf(y));
    }
    vit_quant_row(row, amax, K, q_out + (size_t)m * K, s_out + m, red);
}

// y = bf16(gelu_tanh(bf16(x + bias))) over the real F columns, zero up to F_pad, then act-quant over F_pad
// (bitvla_add_bias_bf16, gelu_tanh_bf16_kernel bitvla_lm_cuda.cu:610-621, padded copy, bitvla_vit_cuda.cu:233-243)
__global__ void __launch_bounds__(256) vit_gelu_quant_kernel(const __nv_bfloat16 *__restrict__ x, const __nv_bfloat16 *__restrict__ bias,
                                                             int F, int F_pad, int8_t *__restrict__ q_out, float *__restrict__ s_out) {
    extern __shared__ float row[];
    __shared__ float red[8];
    pdl_launch_dependents();
    pdl_wait();
    const int m = blockIdx.x;
    float amax = 0.f;
    for (int k = threadIdx.x; k < F_pad; k += 256) {
        float y = 0.f;
        if (k < F) {
            const float v = __bfloat162float(__float2bfloat16(__bfloat162float(x[(size_t)m * F + k]) + __bfloat162float(bias[k])));
            // tanh.approx: what the reference's tanhf becomes under its --use_fast_math build
            const float u = 0.7978845608028654f * (v + 0.044715f * v * v * v);
            float th;
            asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(u));
            y = __bfloat162float(__float2bfloat16(0.5f * v * (1.0f + th)));
        }
        row[k] = y;
        amax = fmaxf(amax, fabsf(y));
    }
    vit_quant_row(row, amax, F_pad, q_out + (size_t)m * F_pad, s_out + m, red);
}

// h = bf16(bf16(h + patch_b[k]) + pos[m][k])  (bitvla_vit_cuda.cu:283-284)
__global__ void vit_embed_finish_kernel(__nv_bfloat16 *__restrict__ h, const __nv_bfloat16 *__restrict__ patch_b,
                                        const __nv_bfloat16 *__restrict__ pos, int H, size_t total) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const float a = __bfloat162float(__float2bfloat16(__bfloat162float(h[i]) + __bfloat162float(patch_b[i % H])));
        h[i] = __float2bfloat16(a + __bfloat162float(pos[i]));
    }
}

// rows of `cols` bf16 -> rows of `cols_pad` bf16, zero filled (a row stride TMA accepts)
__global__ void vit_pad_rows_kernel(const __nv_bfloat16 *__restrict__ src, __nv_bfloat16 *__restrict__ dst, int cols, int cols_pad,
                                    size_t total) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int c = (int)(i % cols_pad);
        dst[i] = c < cols ? src[(i / cols_pad) * cols + c] : __float2bfloat16(0.0f);
    }
}

__global__ void vit_bf16_to_f32_kernel(const __nv_bfloat16 *__restrict__ src, float *__restrict__ dst, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = __bfloat162float(src[i]);
}

struct VitLayer {
    bitvla_vit_layer_cuda w{};
    DevBuf qkv_packed, qkv_ws;
    bool set = false;
};

}  // namespace vb

struct bitvla_vit_cuda_ctx {
    int n_layers, hidden, n_heads, hd, hd_pad, ffn, ffn_pad, n_patches, patch_flat, patch_pad, mm_out;
    float ln_eps;
    std::vector<vb::VitLayer> layers;
    const __nv_bfloat16 *patch_b = nullptr, *pos = nullptr, *mm_w1 = nullptr, *mm_w2 = nullptr;
    vb::DevBuf patch_w, mm_b1, mm_b2;                    // K-padded bf16 copy; float32 copies of the biases
    vb::DevBuf patches, h, a8, a8f, s, qkv, q, kp, vp, att, proj, fc1, mm_h1;
    bool embed_set = false, mm_set = false;
};

using vb::DevBuf;

extern "C" {

bitvla_vit_cuda_ctx *bitvla_vit_cuda_init(int n_layers, int hidden, int n_heads, int ffn, int n_patches, int patch_flat,
                                          float ln_eps, int mm_out) {
    auto fail = [](const char *why) {
        std::fprintf(stderr, "vla_b200(bitvla_vit_cuda): %s\n", why);
        vb::set_last_error("bitvla_vit_cuda_init: %s", why);
        return static_cast<bitvla_vit_cuda_ctx *>(nullptr);
    };
    if (n_layers <= 0 || hidden <= 0 || n_heads <= 0 || hidden % n_heads || ffn <= 0 || n_patches <= 0 || patch_flat <= 0 || mm_out <= 0)
        return fail("bad dimensions");
    const int hd = hidden / n_heads;
    if (hidden % 128 || ffn % 16 || mm_out % 8 || hd % 2 || hd > 256) return fail("needs hidden % 128 == 0, ffn % 16 == 0, mm_out % 8 == 0, head_dim <= 256");
    auto *c = new (std::nothrow) bitvla_vit_cuda_ctx();
    if (!c) return nullptr;
    c->n_layers = n_layers; c->hidden = hidden; c->n_heads = n_heads; c->hd = hd;
    c->hd_pad = hd <= 64 ? 64 : (hd <= 128 ? 128 : 256);
    c->ffn = ffn; c->ffn_pad = (ffn + 127) / 128 * 128;  // the K side of fc2, as the reference pads it
    c->n_patches = n_patches; c->patch_flat = patch_flat; c->patch_pad = (patch_flat + 7) / 8 * 8; c->mm_out = mm_out;
    c->ln_eps = ln_eps;
    c->layers.resize((size_t)n_layers);
    const size_t S = (size_t)n_patches, H = (size_t)hidden, QF = (size_t)n_heads * c->hd_pad;
    int rc = VLAB200_OK;
    if (!rc) rc = c->patches.alloc(S * c->patch_pad * 2);
    if (!rc) rc = c->patch_w.alloc(H * c->patch_pad * 2);
    if (!rc) rc = c->mm_b1.alloc((size_t)mm_out * 4);
    if (!rc) rc = c->mm_b2.alloc((size_t)mm_out * 4);
    if (!rc) rc = c->h.alloc(S * H * 2);
    if (!rc) rc = c->a8.alloc(S * H);
    if (!rc) rc = c->a8f.alloc(S * c->ffn_pad);
    if (!rc) rc = c->s.alloc(S * 4);
    if (!rc) rc = c->qkv.alloc(S * 3 * H * 2);
    if (!rc) rc = c->q.alloc(S * QF * 2);
    if (!rc) rc = c->kp.alloc(S * QF * 2);
    if (!rc) rc = c->vp.alloc(S * QF * 2);
    if (!rc) rc = c->att.alloc(S * QF * 2);
    if (!rc) rc = c->proj.alloc(S * H * 2);
    if (!rc) rc = c->fc1.alloc(S * (size_t)ffn * 2);
    if (!rc) rc = c->mm_h1.alloc(S * (size_t)mm_out * 2);
    for (int l = 0; l < n_layers && !rc; ++l) {
        rc = c->layers[(size_t)l].qkv_packed.alloc(3 * H * H / 4);
        if (!rc) rc = c->layers[(size_t)l].qkv_ws.alloc(3 * sizeof(float));
    }
    if (rc) {
        delete c;
        return fail("device allocation failed");
    }
    return c;
}

void bitvla_vit_cuda_free(bitvla_vit_cuda_ctx *ctx) { delete ctx; }

void bitvla_vit_cuda_set_layer(bitvla_vit_cuda_ctx *ctx, int L, const bitvla_vit_layer_cuda *layer) {
    if (!ctx || !layer || L < 0 || L >= ctx->n_layers) {
        std::fprintf(stderr, "vla_b200(bitvla_vit_cuda): set_layer: bad arguments\n");
        return;
    }
    vb::VitLayer &dst = ctx->layers[(size_t)L];
    dst.w = *layer;
    // q | k | v as one ternary matrix: a ladder pack is a sequence of independent 16-row runs, so the three packs
    // concatenate; one weight scale per projection
    const size_t bytes = (size_t)ctx->hidden * ctx->hidden / 4;
    const int8_t *packs[3] = {layer->q_packed, layer->k_packed, layer->v_packed};
    const float *wss[3] = {layer->q_ws, layer->k_ws, layer->v_ws};
    bool ok = true;
    for (int j = 0; j < 3; ++j) {
        ok = ok && cudaMemcpy(static_cast<char *>(dst.qkv_packed.p) + j * bytes, packs[j], bytes, cudaMemcpyDeviceToDevice) == cudaSuccess;
        ok = ok && cudaMemcpy(dst.qkv_ws.as<float>() + j, wss[j], sizeof(float), cudaMemcpyDeviceToDevice) == cudaSuccess;
    }
    if (!ok) {
        vb::cuda_fail(cudaGetLastError(), "bitvla_vit_cuda_set_layer");
        std::fprintf(stderr, "vla_b200(bitvla_vit_cuda): set_layer %d: %s\n", L, vlab200_last_error());
        return;
    }
    dst.set = true;
}

void bitvla_vit_cuda_set_embed(bitvla_vit_cuda_ctx *ctx, const void *patch_w, const void *patch_b, const void *pos_emb) {
    if (!ctx || !patch_w || !patch_b || !pos_emb) return;
    const size_t total = (size_t)ctx->hidden * ctx->patch_pad;
    vb::vit_pad_rows_kernel<<<(unsigned)((total + 255) / 256), 256>>>(static_cast<const __nv_bfloat16 *>(patch_w),
                                                                      ctx->patch_w.as<__nv_bfloat16>(), ctx->patch_flat, ctx->patch_pad, total);
    ctx->patch_b = static_cast<const __nv_bfloat16 *>(patch_b);
    ctx->pos = static_cast<const __nv_bfloat16 *>(pos_emb);
    ctx->embed_set = cudaDeviceSynchronize() == cudaSuccess;
}

void bitvla_vit_cuda_set_mmproj(bitvla_vit_cuda_ctx *ctx, const void *W1, const void *b1, const void *W2, const void *b2) {
    if (!ctx || !W1 || !b1 || !W2 || !b2) return;
    ctx->mm_w1 = static_cast<const __nv_bfloat16 *>(W1);
    ctx->mm_w2 = static_cast<const __nv_bfloat16 *>(W2);
    const int n = ctx->mm_out;
    vb::vit_bf16_to_f32_kernel<<<(n + 255) / 256, 256>>>(static_cast<const __nv_bfloat16 *>(b1), ctx->mm_b1.as<float>(), n);
    vb::vit_bf16_to_f32_kernel<<<(n + 255) / 256, 256>>>(static_cast<const __nv_bfloat16 *>(b2), ctx->mm_b2.as<float>(), n);
    ctx->mm_set = cudaDeviceSynchronize() == cudaSuccess;
}

int bitvla_vit_cuda_forward(bitvla_vit_cuda_ctx *ctx, const void *d_patches, void *d_out, void *stream) {
    auto fail = [](const char *why, int rc) {
        std::fprintf(stderr, "vla_b200(bitvla_vit_cuda): forward: %s (%d) %s\n", why, rc, vlab200_last_error());
        return -1;
    };
    if (!ctx || !d_patches || !d_out) return fail("null argument", VLAB200_ERR_ARG);
    if (!ctx->embed_set || !ctx->mm_set) return fail("set_embed / set_mmproj have not been called", VLAB200_ERR_ARG);
    for (const vb::VitLayer &l : ctx->layers)
        if (!l.set) return fail("a layer has not been set", VLAB200_ERR_ARG);
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    const int S = ctx->n_patches, H = ctx->hidden, heads = ctx->n_heads, hd = ctx->hd, hp = ctx->hd_pad, F = ctx->ffn,
              FP = ctx->ffn_pad, PP = ctx->patch_pad, MM = ctx->mm_out;
    __nv_bfloat16 *h = ctx->h.as<__nv_bfloat16>(), *proj = ctx->proj.as<__nv_bfloat16>();
    int8_t *a8 = ctx->a8.as<int8_t>(), *a8f = ctx->a8f.as<int8_t>();
    float *s = ctx->s.as<float>();
    int rc;
    // ---- patch embedding: patches . Wp^T (float accumulation, bf16 out), + bias, + position ----
    const void *A = d_patches;
    if (PP != ctx->patch_flat) {  // a 16-byte row stride for TMA
        const size_t total = (size_t)S * PP;
        vb::vit_pad_rows_kernel<<<(unsigned)((total + 255) / 256), 256, 0, cs>>>(static_cast<const __nv_bfloat16 *>(d_patches),
                                                                                 ctx->patches.as<__nv_bfloat16>(), ctx->patch_flat, PP, total);
        A = ctx->patches.p;
    }
    {
        vb::GemmParams g{};
        g.M = S; g.N = H; g.K = PP; g.epi = vb::EPI_BIAS_ACT; g.act = vb::ACT_NONE; g.out_bf = h; g.ld_out = H;
        if ((rc = vb::dense_gemm(A, PP, ctx->patch_w.p, g, cs))) return fail("patch embedding", rc);
        const size_t total = (size_t)S * H;
        vb::vit_embed_finish_kernel<<<148 * 2, 256, 0, cs>>>(h, ctx->patch_b, ctx->pos, H, total);
    }
    const float scale = 1.0f / std::sqrt((float)hd);
    const size_t row_smem = (size_t)(FP > H ? FP : H) * sizeof(float);
    if (row_smem > 48 * 1024) {
        if ((rc = vb::ensure_dyn_smem(vb::vit_ln_quant_kernel, (int)row_smem))) return fail("shared memory", rc);
        if ((rc = vb::ensure_dyn_smem(vb::vit_gelu_quant_kernel, (int)row_smem))) return fail("shared memory", rc);
        if ((rc = vb::ensure_dyn_smem(vb::vit_merge_quant_kernel, (int)row_smem))) return fail("shared memory", rc);
    }
    const __nv_bfloat16 *pend = nullptr, *pend_bias = nullptr;  // a projection whose bias + residual add is still due
    for (int L = 0; L < ctx->n_layers; ++L) {
        const vb::VitLayer &lr = ctx->layers[(size_t)L];
        const bitvla_vit_layer_cuda &w = lr.w;
        const auto bf = [](const void *p) { return static_cast<const __nv_bfloat16 *>(p); };
        if ((rc = vb::launch_pdl(vb::vit_ln_quant_kernel, dim3(S), dim3(256), (size_t)H * 4, cs, h, pend, pend_bias, bf(w.ln1_w),
                                 bf(w.ln1_b), ctx->ln_eps, H, a8, s)))
            return fail("ln1", rc);
        if ((rc = vlab200_ternary_linear(a8, lr.qkv_packed.as<uint8_t>(), ctx->qkv.p, nullptr, s, lr.qkv_ws.as<float>(), 3, S, 3 * H, H, 0, cs)))
            return fail("qkv projection", rc);
        if ((rc = vb::launch_pdl(vb::vit_split_heads_kernel, dim3(S), dim3(256), 0, cs, ctx->qkv.as<__nv_bfloat16>(), bf(w.q_b), bf(w.k_b),
                                 bf(w.v_b), ctx->q.as<__nv_bfloat16>(), ctx->kp.as<__nv_bfloat16>(), ctx->vp.as<__nv_bfloat16>(), S, heads, hd, hp)))
            return fail("head split", rc);
        vlab200_kv_store view{ctx->kp.p, ctx->vp.p, 1, 1, heads, hp, S, 0};
        if ((rc = vb::attention_flash(&view, 0, ctx->q.p, ctx->att.p, S, heads, S, 0, nullptr, cs, scale, nullptr, 0))) return fail("attention", rc);
        if ((rc = vb::launch_pdl(vb::vit_merge_quant_kernel, dim3(S), dim3(256), (size_t)H * 4, cs, ctx->att.as<__nv_bfloat16>(), heads, hd,
                                 hp, a8, s)))
            return fail("merge", rc);
        if ((rc = vlab200_ternary_linear(a8, reinterpret_cast<const uint8_t *>(w.o_packed), proj, nullptr, s, w.o_ws, 1, S, H, H, 0, cs)))
            return fail("o projection", rc);
        if ((rc = vb::launch_pdl(vb::vit_ln_quant_kernel, dim3(S), dim3(256), (size_t)H * 4, cs, h, static_cast<const __nv_bfloat16 *>(proj),
                                 bf(w.o_b), bf(w.ln2_w), bf(w.ln2_b), ctx->ln_eps, H, a8, s)))
            return fail("ln2", rc);
        if ((rc = vlab200_ternary_linear(a8, reinterpret_cast<const uint8_t *>(w.fc1_packed), ctx->fc1.p, nullptr, s, w.fc1_ws, 1, S, F, H, 0, cs)))
            return fail("fc1", rc);
        if ((rc = vb::launch_pdl(vb::vit_gelu_quant_kernel, dim3(S), dim3(256), (size_t)FP * 4, cs, ctx->fc1.as<__nv_bfloat16>(), bf(w.fc1_b), F,
                                 FP, a8f, s)))
            return fail("gelu", rc);
        if ((rc = vlab200_ternary_linear(a8f, reinterpret_cast<const uint8_t *>(w.fc2_packed), proj, nullptr, s, w.fc2_ws, 1, S, H, FP, 0, cs)))
            return fail("fc2", rc);
        pend = proj;
        pend_bias = bf(w.fc2_b);
    }
    // the last fc2's bias and residual add, without a norm
    if ((rc = vb::launch_pdl(vb::vit_ln_quant_kernel, dim3(S), dim3(256), (size_t)H * 4, cs, h, pend, pend_bias,
                             static_cast<const __nv_bfloat16 *>(nullptr), static_cast<const __nv_bfloat16 *>(nullptr), ctx->ln_eps, H,
                             static_cast<int8_t *>(nullptr), static_cast<float *>(nullptr))))
        return fail("final residual", rc);
    // ---- projector: erf-GELU(h W1^T + b1) W2^T + b2 (bitvla_vit_cuda.cu:292-327) ----
    vb::GemmParams g{};
    g.M = S; g.N = MM; g.K = H; g.epi = vb::EPI_BIAS_ACT; g.act = vb::ACT_GELU_ERF; g.bias = ctx->mm_b1.as<float>();
    g.out_bf = ctx->mm_h1.as<__nv_bfloat16>(); g.ld_out = MM;
    if ((rc = vb::dense_gemm(h, H, ctx->mm_w1, g, cs))) return fail("projector fc1", rc);
    g = vb::GemmParams{};
    g.M = S; g.N = MM; g.K = MM; g.epi = vb::EPI_BIAS_ACT; g.act = vb::ACT_NONE; g.bias = ctx->mm_b2.as<float>();
    g.out_bf = static_cast<__nv_bfloat16 *>(d_out); g.ld_out = MM;
    if ((rc = vb::dense_gemm(ctx->mm_h1.p, MM, ctx->mm_w2, g, cs))) return fail("projector fc2", rc);
    return 0;
}

}  // extern "C"
