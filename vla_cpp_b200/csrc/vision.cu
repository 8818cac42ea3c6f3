// SigLIP vision tower + connector on the device: camera views in, image-token embeddings of the prefix out.
//
// Follows the reference's towers: src/models/smolvla.cpp:394-426 (encoder block), :1511-1563 (patch embedding,
// layers, post-LayerNorm, pixel shuffle, connector) and src/models/pi0.cpp:130-155,479-517 (same block, linear
// projector with optional bias and a 1/sqrt(out) scale); preprocessing and the pixel-shuffle order are those of
// src/modules/preprocess.h:37-75.
//
//   pixels (u8 or float32, HWC)  --patchify-->  bf16 [views * n_patches][3 P P]      (x / 255) * 2 - 1
//   residual stream h (float32)  = pos + bias, then += patches . Wpatch^T            (tcgen05 GEMM, residual epilogue)
//   per layer: LayerNorm -> q|k|v (+bias) -> head-major pages -> attention (no mask) -> Wo (+bias, residual)
//              -> LayerNorm -> fc1 (+bias, tanh-GELU) -> fc2 (+bias, residual)
//   post-LayerNorm written straight into pixel-shuffled rows, connector GEMM -> float32 [views * n_tokens][out]
//
// All matrix products run on the library's tcgen05 GEMM, attention on its flash kernel.  A head_dim that the
// attention kernels do not have (SigLIP-So400m: 72) is zero-padded to the next one (128) in prepared copies of
// Wq/Wk/Wv/Wo, with sqrt(padded / real) folded into Wq and bq so that the kernel's 1/sqrt(padded) is the model's
// 1/sqrt(real).
#include <cuda_bf16.h>

#include <cmath>
#include <new>
#include <vector>

#include "gemm.h"
#include "host_common.h"

struct vlab200_vision {
    vlab200_vision_config c;
    int max_views, np, grid, hd, hd_pad, kp, qf, n_tok, c4;
    vb::DevBuf patch_w, posb, post_w, post_b, connector, connector_b;
    std::vector<vb::DevBuf> wqkv, bqkv, wo, bo, w1, b1, w2, b2, ln1w, ln1b, ln2w, ln2b;
    vb::DevBuf a_patch, h, hb, nb, qkv, q, kpg, vpg, att, f, shuf, ident;
};

namespace vb {

// A[t][c P P + ph P + pw] = pixel(row P + ph, col P + pw, c) * 2 - 1, the column order of the conv weight
// [hidden][3][P][P]; columns >= 3 P P (padding of K to a multiple of 8) are zero.
__global__ void patchify_kernel(const void *__restrict__ pixels, int is_f32, __nv_bfloat16 *__restrict__ A, int n_views,
                                int side, int P, int kp) {
    const int grid = side / P, np = grid * grid, pp = P * P;
    const size_t total = (size_t)n_views * np * kp;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int k = (int)(i % kp);
        const size_t r = i / kp;
        const int t = (int)(r % np), v = (int)(r / np);
        float val = 0.0f;
        if (k < 3 * pp) {
            const int c = k / pp, ph = (k % pp) / P, pw = k % P;
            const int y = (t / grid) * P + ph, x = (t % grid) * P + pw;
            const size_t src = (((size_t)v * side + y) * side + x) * 3 + c;
            const float px = is_f32 ? static_cast<const float *>(pixels)[src]
                                    : (float)static_cast<const unsigned char *>(pixels)[src] / 255.0f;
            val = px * 2.0f - 1.0f;
        }
        A[i] = __float2bfloat16(val);
    }
}

// h[v][t][e] = posb[t][e]  (position embedding + patch bias), the value the patch GEMM accumulates onto
__global__ void init_stream_kernel(const float *__restrict__ posb, float *__restrict__ h, size_t per_view, size_t total) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
        h[i] = posb[i % per_view];
}

__global__ void add_vec_kernel(const float *__restrict__ a, const float *__restrict__ b, float *__restrict__ out, int n_rows,
                               int H) {
    const size_t total = (size_t)n_rows * H;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
        out[i] = a[i] + b[i % H];
}

// LayerNorm with weight and bias, one warp per row, float32 in, bf16 out: mean, then the variance of the centred
// values (ggml_norm's order).  shuffle > 1 writes row p of view v into its pixel-shuffled place: token
// (p_y / s) * (grid / s) + p_x / s, columns ((p_y % s) * s + p_x % s) * H ... + H  (pixel_shuffle_hf).
__global__ void layernorm_kernel(const float *__restrict__ x, const float *__restrict__ w, const float *__restrict__ b,
                                 __nv_bfloat16 *__restrict__ out, int M, int H, float eps, int np, int grid, int shuffle) {
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= M) return;
    const float *xr = x + (size_t)row * H;
    float s = 0.0f;
    for (int k = lane; k < H; k += 32) s += xr[k];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    const float mean = s / (float)H;
    float s2 = 0.0f;
    for (int k = lane; k < H; k += 32) {
        const float d = xr[k] - mean;
        s2 = fmaf(d, d, s2);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s2 += __shfl_xor_sync(0xffffffffu, s2, o);
    const float rstd = 1.0f / sqrtf(s2 / (float)H + eps);
    __nv_bfloat16 *orow;
    if (shuffle > 1) {
        const int v = row / np, p = row % np, py = p / grid, px = p % grid, g2 = grid / shuffle;
        const size_t tok = (size_t)v * g2 * g2 + (size_t)(py / shuffle) * g2 + px / shuffle;
        orow = out + (tok * shuffle * shuffle + (size_t)(py % shuffle) * shuffle + px % shuffle) * H;
    } else {
        orow = out + (size_t)row * H;
    }
    for (int k = lane; k < H; k += 32) orow[k] = __float2bfloat16((xr[k] - mean) * rstd * w[k] + b[k]);
}

// dst [heads * hd_pad][K] <- src [heads * hd][K] * scale, rows d >= hd of every head zero
__global__ void pad_head_rows_kernel(const __nv_bfloat16 *__restrict__ src, __nv_bfloat16 *__restrict__ dst, int heads, int hd,
                                     int hd_pad, int K, float scale) {
    const size_t total = (size_t)heads * hd_pad * K;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int k = (int)(i % K);
        const size_t r = i / K;
        const int d = (int)(r % hd_pad), h = (int)(r / hd_pad);
        float v = 0.0f;
        if (d < hd) {
            const __nv_bfloat16 s = src[((size_t)h * hd + d) * K + k];
            if (scale == 1.0f) {
                dst[i] = s;
                continue;
            }
            v = __bfloat162float(s) * scale;
        }
        dst[i] = __float2bfloat16(v);
    }
}

__global__ void pad_head_vec_kernel(const float *__restrict__ src, float *__restrict__ dst, int heads, int hd, int hd_pad,
                                    float scale) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= heads * hd_pad) return;
    const int d = i % hd_pad, h = i / hd_pad;
    dst[i] = d < hd ? src[h * hd + d] * scale : 0.0f;
}

// dst [N][heads * hd_pad] <- src [N][heads * hd], columns d >= hd of every head zero; also pads plain rows
// (heads = 1: dst [N][hd_pad] <- src [N][hd])
__global__ void pad_head_cols_kernel(const __nv_bfloat16 *__restrict__ src, __nv_bfloat16 *__restrict__ dst, int N, int heads,
                                     int hd, int hd_pad) {
    const size_t total = (size_t)N * heads * hd_pad;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int d = (int)(i % hd_pad);
        const size_t r = i / hd_pad;
        const int h = (int)(r % heads);
        const size_t n = r / heads;
        dst[i] = d < hd ? src[(n * heads + h) * hd + d] : __float2bfloat16(0.0f);
    }
}

__global__ void fill_identity_rotation_kernel(float *cos_t, float *sin_t, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        cos_t[i] = 1.0f;
        sin_t[i] = 0.0f;
    }
}

__global__ void scale_inplace_kernel(float *x, float s, size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) x[i] *= s;
}

static int dev_copy(DevBuf &dst, const void *src, size_t bytes) {
    int rc = dst.alloc(bytes);
    if (rc) return rc;
    VB_CUDA(cudaMemcpy(dst.p, src, bytes, cudaMemcpyDeviceToDevice));
    return VLAB200_OK;
}

}  // namespace vb

extern "C" {

vlab200_vision *vlab200_vision_create(const vlab200_vision_config *cfg, const vlab200_vision_weights *w, int32_t max_views) {
    if (!cfg || !w || max_views <= 0) {
        vb::set_last_error("vlab200_vision_create: null configuration / weights, or max_views <= 0");
        return nullptr;
    }
    const vlab200_vision_config &c = *cfg;
    if (c.image <= 0 || c.patch <= 0 || c.image % c.patch || c.hidden <= 0 || c.hidden % 8 || c.n_layers <= 0 || c.n_heads <= 0 ||
        c.hidden % c.n_heads || c.inter <= 0 || c.inter % 8 || c.shuffle < 1 || (c.image / c.patch) % c.shuffle || c.out_dim <= 0 ||
        c.out_dim % 8) {
        vb::set_last_error("vlab200_vision_create: bad configuration");
        return nullptr;
    }
    const int hd = c.hidden / c.n_heads;
    const int hd_pad = hd <= 64 ? 64 : (hd <= 128 ? 128 : 256);
    if (hd > 256 || hd % 2) {
        vb::set_last_error("vlab200_vision_create: head_dim %d is not supported", hd);
        return nullptr;
    }
    if (!w->patch_w || !w->patch_b || !w->pos || !w->post_w || !w->post_b || !w->connector || !w->ln1_w || !w->ln1_b || !w->ln2_w ||
        !w->ln2_b || !w->wq || !w->wk || !w->wv || !w->wo || !w->fc1 || !w->fc2 || !w->bq || !w->bk || !w->bv || !w->bo || !w->b1 ||
        !w->b2) {
        vb::set_last_error("vlab200_vision_create: a weight pointer is null");
        return nullptr;
    }
    auto *v = new (std::nothrow) vlab200_vision();
    if (!v) return nullptr;
    v->c = c;
    v->max_views = max_views;
    v->grid = c.image / c.patch;
    v->np = v->grid * v->grid;
    v->hd = hd;
    v->hd_pad = hd_pad;
    v->kp = (3 * c.patch * c.patch + 7) / 8 * 8;
    v->qf = c.n_heads * hd_pad;
    v->n_tok = v->np / (c.shuffle * c.shuffle);
    v->c4 = c.hidden * c.shuffle * c.shuffle;
    const int L = c.n_layers, H = c.hidden, I = c.inter, qf = v->qf, heads = c.n_heads;
    const float qscale = hd == hd_pad ? 1.0f : std::sqrt((float)hd_pad / (float)hd);
    int rc = VLAB200_OK;
    auto grid_for = [](size_t n) { return (int)((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8); };
    do {
        // patch embedding [H][3 P P] -> [H][kp]; position embedding + bias
        if ((rc = v->patch_w.alloc((size_t)H * v->kp * 2))) break;
        vb::pad_head_cols_kernel<<<grid_for((size_t)H * v->kp), 256>>>(static_cast<const __nv_bfloat16 *>(w->patch_w),
                                                                        v->patch_w.as<__nv_bfloat16>(), H, 1, 3 * c.patch * c.patch, v->kp);
        if ((rc = v->posb.alloc((size_t)v->np * H * 4))) break;
        vb::add_vec_kernel<<<grid_for((size_t)v->np * H), 256>>>(w->pos, w->patch_b, v->posb.as<float>(), v->np, H);
        if ((rc = vb::dev_copy(v->post_w, w->post_w, (size_t)H * 4))) break;
        if ((rc = vb::dev_copy(v->post_b, w->post_b, (size_t)H * 4))) break;
        if ((rc = vb::dev_copy(v->connector, w->connector, (size_t)c.out_dim * v->c4 * 2))) break;
        if (w->connector_b && (rc = vb::dev_copy(v->connector_b, w->connector_b, (size_t)c.out_dim * 4))) break;
        for (auto *vec : {&v->wqkv, &v->bqkv, &v->wo, &v->bo, &v->w1, &v->b1, &v->w2, &v->b2, &v->ln1w, &v->ln1b, &v->ln2w, &v->ln2b})
            vec->resize((size_t)L);
        for (int l = 0; l < L && !rc; ++l) {
            if ((rc = v->wqkv[l].alloc((size_t)3 * qf * H * 2))) break;
            if ((rc = v->bqkv[l].alloc((size_t)3 * qf * 4))) break;
            const void *ws[3] = {w->wq[l], w->wk[l], w->wv[l]};
            const float *bs[3] = {w->bq[l], w->bk[l], w->bv[l]};
            for (int j = 0; j < 3; ++j) {
                vb::pad_head_rows_kernel<<<grid_for((size_t)qf * H), 256>>>(static_cast<const __nv_bfloat16 *>(ws[j]),
                                                                           v->wqkv[l].as<__nv_bfloat16>() + (size_t)j * qf * H, heads, hd,
                                                                           hd_pad, H, j == 0 ? qscale : 1.0f);
                vb::pad_head_vec_kernel<<<(qf + 127) / 128, 128>>>(bs[j], v->bqkv[l].as<float>() + (size_t)j * qf, heads, hd, hd_pad,
                                                                  j == 0 ? qscale : 1.0f);
            }
            if ((rc = v->wo[l].alloc((size_t)H * qf * 2))) break;
            vb::pad_head_cols_kernel<<<grid_for((size_t)H * qf), 256>>>(static_cast<const __nv_bfloat16 *>(w->wo[l]),
                                                                       v->wo[l].as<__nv_bfloat16>(), H, heads, hd, hd_pad);
            if ((rc = vb::dev_copy(v->bo[l], w->bo[l], (size_t)H * 4))) break;
            if ((rc = vb::dev_copy(v->w1[l], w->fc1[l], (size_t)I * H * 2))) break;
            if ((rc = vb::dev_copy(v->b1[l], w->b1[l], (size_t)I * 4))) break;
            if ((rc = vb::dev_copy(v->w2[l], w->fc2[l], (size_t)H * I * 2))) break;
            if ((rc = vb::dev_copy(v->b2[l], w->b2[l], (size_t)H * 4))) break;
            if ((rc = vb::dev_copy(v->ln1w[l], w->ln1_w[l], (size_t)H * 4))) break;
            if ((rc = vb::dev_copy(v->ln1b[l], w->ln1_b[l], (size_t)H * 4))) break;
            if ((rc = vb::dev_copy(v->ln2w[l], w->ln2_w[l], (size_t)H * 4))) break;
            if ((rc = vb::dev_copy(v->ln2b[l], w->ln2_b[l], (size_t)H * 4))) break;
        }
        if (rc) break;
        const size_t M = (size_t)max_views * v->np;
        if ((rc = v->a_patch.alloc(M * v->kp * 2))) break;
        if ((rc = v->h.alloc(M * H * 4))) break;
        if ((rc = v->hb.alloc(M * H * 2))) break;
        if ((rc = v->nb.alloc(M * H * 2))) break;
        if ((rc = v->qkv.alloc(M * (size_t)3 * qf * 2))) break;
        if ((rc = v->q.alloc(M * qf * 2))) break;
        if ((rc = v->kpg.alloc(M * qf * 2))) break;
        if ((rc = v->vpg.alloc(M * qf * 2))) break;
        if ((rc = v->att.alloc(M * qf * 2))) break;
        if ((rc = v->f.alloc(M * I * 2))) break;
        if ((rc = v->shuf.alloc(M * H * 2))) break;
        const int nrot = v->np * (hd_pad / 2);
        if ((rc = v->ident.alloc((size_t)2 * nrot * 4))) break;
        vb::fill_identity_rotation_kernel<<<(nrot + 127) / 128, 128>>>(v->ident.as<float>(), v->ident.as<float>() + nrot, nrot);
        if (cudaDeviceSynchronize() != cudaSuccess) rc = vb::cuda_fail(cudaGetLastError(), "vlab200_vision_create");
    } while (false);
    if (rc) {
        if (rc != VLAB200_ERR_CUDA) vb::set_last_error("vlab200_vision_create: failed with status %d", rc);
        delete v;
        return nullptr;
    }
    return v;
}

void vlab200_vision_free(vlab200_vision *v) { delete v; }

int32_t vlab200_vision_tokens_per_view(const vlab200_vision *v) { return v ? v->n_tok : 0; }

int32_t vlab200_vision_run(vlab200_vision *v, const void *pixels, int32_t pixels_f32, int32_t n_views, float *img_emb,
                           void *stream) {
    if (!v || !pixels || !img_emb || n_views <= 0 || n_views > v->max_views) return VLAB200_ERR_ARG;
    const vlab200_vision_config &c = v->c;
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    const int H = c.hidden, I = c.inter, qf = v->qf, np = v->np, M = n_views * np;
    auto grid_for = [](size_t n) { return (int)((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8); };
    int rc;
    vb::patchify_kernel<<<grid_for((size_t)M * v->kp), 256, 0, cs>>>(pixels, pixels_f32 ? 1 : 0, v->a_patch.as<__nv_bfloat16>(),
                                                                    n_views, c.image, c.patch, v->kp);
    vb::init_stream_kernel<<<grid_for((size_t)M * H), 256, 0, cs>>>(v->posb.as<float>(), v->h.as<float>(), (size_t)np * H,
                                                                   (size_t)M * H);
    VB_CUDA(cudaGetLastError());
    auto residual = [&](const void *A, int K, const void *W, const float *bias) {
        vb::GemmParams g{};
        g.M = M; g.N = H; g.K = K; g.epi = vb::EPI_RESIDUAL; g.bias = bias;
        g.h = v->h.as<float>(); g.out_bf = v->hb.as<__nv_bfloat16>(); g.ld_out = H;
        return vb::dense_gemm(A, K, W, g, cs);
    };
    auto layernorm = [&](const float *w, const float *b, __nv_bfloat16 *out, int shuffle) {
        vb::layernorm_kernel<<<(M + 7) / 8, 256, 0, cs>>>(v->h.as<float>(), w, b, out, M, H, c.ln_eps, np, v->grid, shuffle);
        return cudaGetLastError() == cudaSuccess ? VLAB200_OK : vb::cuda_fail(cudaGetLastError(), "layernorm_kernel");
    };
    if ((rc = residual(v->a_patch.p, v->kp, v->patch_w.p, nullptr))) return rc;
    const float *cos_t = v->ident.as<float>(), *sin_t = cos_t + (size_t)np * (v->hd_pad / 2);
    for (int l = 0; l < c.n_layers; ++l) {
        if ((rc = layernorm(v->ln1w[l].as<float>(), v->ln1b[l].as<float>(), v->nb.as<__nv_bfloat16>(), 1))) return rc;
        vb::GemmParams g{};
        g.M = M; g.N = 3 * qf; g.K = H; g.epi = vb::EPI_BIAS_ACT; g.act = vb::ACT_NONE; g.bias = v->bqkv[l].as<float>();
        g.out_bf = v->qkv.as<__nv_bfloat16>(); g.ld_out = 3 * qf;
        if ((rc = vb::dense_gemm(v->nb.p, H, v->wqkv[l].p, g, cs))) return rc;
        if ((rc = vb::rope_split(v->qkv.p, cos_t, sin_t, v->q.p, v->kpg.p, v->vpg.p, M, np, c.n_heads, c.n_heads, c.n_heads, v->hd_pad,
                                 np, 0, cs)))
            return rc;
        vlab200_kv_store view{v->kpg.p, v->vpg.p, 1, n_views, c.n_heads, v->hd_pad, np, 0};
        if ((rc = vlab200_attention(&view, 0, v->q.p, v->att.p, np, c.n_heads, np, 0, nullptr, cs))) return rc;
        if ((rc = residual(v->att.p, qf, v->wo[l].p, v->bo[l].as<float>()))) return rc;
        if ((rc = layernorm(v->ln2w[l].as<float>(), v->ln2b[l].as<float>(), v->nb.as<__nv_bfloat16>(), 1))) return rc;
        g = vb::GemmParams{};
        g.M = M; g.N = I; g.K = H; g.epi = vb::EPI_BIAS_ACT; g.act = vb::ACT_GELU_TANH; g.bias = v->b1[l].as<float>();
        g.out_bf = v->f.as<__nv_bfloat16>(); g.ld_out = I;
        if ((rc = vb::dense_gemm(v->nb.p, H, v->w1[l].p, g, cs))) return rc;
        if ((rc = residual(v->f.p, I, v->w2[l].p, v->b2[l].as<float>()))) return rc;
    }
    if ((rc = layernorm(v->post_w.as<float>(), v->post_b.as<float>(), v->shuf.as<__nv_bfloat16>(), c.shuffle))) return rc;
    vb::GemmParams g{};
    g.M = n_views * v->n_tok; g.N = c.out_dim; g.K = v->c4; g.epi = vb::EPI_BIAS_ACT; g.act = vb::ACT_NONE;
    g.bias = v->connector_b.as<float>(); g.out_f32 = img_emb; g.ld_out = c.out_dim;
    if ((rc = vb::dense_gemm(v->shuf.p, v->c4, v->connector.p, g, cs))) return rc;
    if (c.out_scale != 0.0f && c.out_scale != 1.0f) {
        const size_t n = (size_t)g.M * c.out_dim;
        vb::scale_inplace_kernel<<<grid_for(n), 256, 0, cs>>>(img_emb, c.out_scale, n);
        VB_CUDA(cudaGetLastError());
    }
    return VLAB200_OK;
}

}  // extern "C"
