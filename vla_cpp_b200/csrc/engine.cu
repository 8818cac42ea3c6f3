// The flow-matching denoise loop of a pi0- or SmolVLA-shaped policy, batched over observations:
// host-side C++ driver + the small kernels around the GEMM / attention kernels.
//
// Per Euler step (src/models/pi0.cpp:570-588, src/models/smolvla.cpp:1393-1418):
//   suffix embedding   a = W_ain x + b;  u = W_at2 silu(W_at1 [a ; tau_k] + b) + b   (pi0: + state token)
//   L expert layers    fused RMSNorm+QKV+RoPE(+KV append) -> attention -> Wo + residual ->
//                      fused RMSNorm + gate/up + activation -> Wdown + residual
//   head               v = W_aout (rms(h) * w_out) + b on the action rows;  x += dt * v   (x stays f32)
// pi0.5 (model 2; src/models/pi05.cpp:208-292,604-631): no state token, the suffix embedding is W_ain x + b alone, and
// time enters through adaptive RMSNorm: cond_k = silu(W_tout silu(W_tin tau_k + b) + b), per layer
// (scale | shift | gate) = W_ada cond_k + b, x_norm = rms(x) (1 + scale) + shift, residual += gate * projection.  All
// of these vectors depend on the step schedule only, so they are computed once, in float32, when the engine is built;
// a layer is adarms_norm -> q|k|v GEMM -> rotation/split/append -> attention (no mask) -> Wo with the gate in its
// residual epilogue -> adarms_norm -> gate/up -> Wdown with the gate.
// W_at1 [a ; tau_k] is split: the tau_k half is a per-step constant vector computed once at
// engine creation, so the GEMM runs over K = H only.  RMSNorm weights are folded into the
// projections that consume the normalised activations (load-time step).
#include <cuda_bf16.h>

#include <cmath>
#include <cstdlib>
#include <new>
#include <string>
#include <thread>
#include <vector>

#include "chunk_loop.h"
#include "gemm.h"
#include "host_common.h"
#include "tc5.cuh"

namespace vb {

// ------------------------------------------------------------------ small kernels --

// W'[r][k] = bf16(W[r][k] * ln[k]) written at out row (r * row_mul + row_add): concatenation and
// gate/up interleaving are both expressed through the row map.
__global__ void fold_rows_kernel(const __nv_bfloat16 *__restrict__ w, const float *__restrict__ ln,
                                 __nv_bfloat16 *__restrict__ out, int rows, int K, int row_mul, int row_add) {
    const size_t total = (size_t)rows * K;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / K, k = i % K;
        const float v = __bfloat162float(w[i]) * (ln ? ln[k] : 1.0f);
        out[(r * row_mul + row_add) * K + k] = __float2bfloat16(v);
    }
}

__global__ void f32_to_bf16_kernel(const float *__restrict__ in, __nv_bfloat16 *__restrict__ out, size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = __float2bfloat16(in[i]);
}

// tvec[s][o] = b_at1[o] + sum_k W_at1[o][H + k] * tau[s][k]   (one warp per output)
__global__ void time_vector_kernel(const __nv_bfloat16 *__restrict__ w_at1, const float *__restrict__ b_at1,
                                   const float *__restrict__ tau, float *__restrict__ tvec, int H, int T) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= T * H) return;
    const int s = warp / H, o = warp % H;
    const __nv_bfloat16 *wr = w_at1 + (size_t)o * 2 * H + H;
    float acc = 0.0f;
    for (int k = lane; k < H; k += 32) acc = fmaf(__bfloat162float(wr[k]), tau[s * H + k], acc);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (lane == 0) tvec[warp] = acc + (b_at1 ? b_at1[o] : 0.0f);
}

// a[row][o] = bf16(b_ain[o] + sum_k W_ain[o][k] x[row][k]) for the n_rows = n_obs*chunk action
// tokens.  One CTA takes AIN_ROWS tokens (their x rows, A <= 64 floats each, sit in shared memory) and one
// thread one output column: its weight row is read once (16-byte loads) and kept in registers for all the
// tokens of the CTA, so W_ain crosses L2 -> SM once per AIN_ROWS tokens instead of once per token.
constexpr int AIN_ROWS = 16;
__global__ void __launch_bounds__(256) action_in_kernel(const float *__restrict__ x,
                                                        const __nv_bfloat16 *__restrict__ w_ain,
                                                        const float *__restrict__ b_ain, __nv_bfloat16 *__restrict__ a,
                                                        float *__restrict__ a_f32, int n_rows, int H, int A) {
    __shared__ float sx[AIN_ROWS][64];
    pdl_launch_dependents();
    pdl_wait();
    const int row0 = blockIdx.x * AIN_ROWS;
    const int rows = min(AIN_ROWS, n_rows - row0);
    for (int i = threadIdx.x; i < rows * A; i += blockDim.x) sx[i / A][i % A] = x[(size_t)row0 * A + i];
    __syncthreads();
    const int o = blockIdx.y * blockDim.x + threadIdx.x;
    if (o >= H) return;
    uint4 wv[8];  // A % 8 == 0, A <= 64
    const uint4 *wr = reinterpret_cast<const uint4 *>(w_ain + (size_t)o * A);
#pragma unroll
    for (int k8 = 0; k8 < 8; ++k8)
        if (k8 * 8 < A) wv[k8] = __ldg(wr + k8);
    const float bias = b_ain ? b_ain[o] : 0.0f;
    for (int r = 0; r < rows; ++r) {
        float acc = bias;
#pragma unroll
        for (int k8 = 0; k8 < 8; ++k8) {
            if (k8 * 8 >= A) break;
            const __nv_bfloat162 *h2 = reinterpret_cast<const __nv_bfloat162 *>(&wv[k8]);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __bfloat1622float2(h2[e]);
                acc = fmaf(f.x, sx[r][k8 * 8 + 2 * e], acc);
                acc = fmaf(f.y, sx[r][k8 * 8 + 2 * e + 1], acc);
            }
        }
        a[(size_t)(row0 + r) * H + o] = __float2bfloat16(acc);
        if (a_f32) a_f32[(size_t)(row0 + r) * H + o] = acc;  // pi0.5: the embedding is the residual stream itself
    }
}

// Adaptive RMSNorm (build_adarms, src/models/pi05.cpp:208-224): n = x * rsqrt(mean x^2 + eps);
// y = bf16(n + n * scale[k] + shift[k]); mod = scale | shift | gate, H floats each.  One warp per row.
__global__ void __launch_bounds__(256) adarms_norm_kernel(const float *__restrict__ x, const float *__restrict__ mod,
                                                          __nv_bfloat16 *__restrict__ y, int M, int H, float eps) {
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= M) return;
    const float *xr = x + (size_t)row * H;
    float ss = 0.0f;
    for (int k = lane; k < H; k += 32) ss = fmaf(xr[k], xr[k], ss);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    const float r = rsqrtf(ss / (float)H + eps);
    for (int k = lane; k < H; k += 32) {
        const float n = xr[k] * r;
        y[(size_t)row * H + k] = __float2bfloat16(n + n * mod[k] + mod[H + k]);
    }
}

// pi0: the state token (row 0 of each observation) of h / hb = W_sp state + b_sp.
__global__ void __launch_bounds__(256) state_token_kernel(const float *__restrict__ state,
                                                          const __nv_bfloat16 *__restrict__ w_sp,
                                                          const float *__restrict__ b_sp, float *__restrict__ h,
                                                          __nv_bfloat16 *__restrict__ hb, int H, int sd, int S) {
    __shared__ float ss[64];
    pdl_launch_dependents();
    pdl_wait();
    const int obs = blockIdx.x;
    if (threadIdx.x < sd) ss[threadIdx.x] = state[(size_t)obs * sd + threadIdx.x];
    __syncthreads();
    for (int o = threadIdx.x; o < H; o += blockDim.x) {
        const __nv_bfloat16 *wr = w_sp + (size_t)o * sd;
        float acc = b_sp ? b_sp[o] : 0.0f;
        for (int k = 0; k < sd; ++k) acc = fmaf(__bfloat162float(wr[k]), ss[k], acc);
        h[(size_t)obs * S * H + o] = acc;
        hb[(size_t)obs * S * H + o] = __float2bfloat16(acc);
    }
}

// x[obs][t][a] += dt * v[obs*S + (S - chunk) + t][a]   (v from the head GEMM, row stride A)
__global__ void euler_kernel(float *__restrict__ x, const float *__restrict__ v, int n, int A, int chunk, int S,
                             float dt) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int a = i % A, row = i / A;
    const int obs = row / chunk, t = row % chunk;
    x[i] += dt * v[((size_t)obs * S + (S - chunk) + t) * A + a];
}

}  // namespace vb

namespace vb {

// pages [n_obs][n_kv][cap][hd] rows [0, P) -> float32 [n_obs][P][n_kv][hd]
__global__ void pages_to_f32_kernel(const __nv_bfloat16 *__restrict__ pages, float *__restrict__ out, int n_kv, int cap,
                                    int hd, int P, size_t total) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int d = (int)(i % hd);
        size_t r = i / hd;
        const int kvh = (int)(r % n_kv);
        r /= n_kv;
        const int tok = (int)(r % P);
        const size_t obs = r / P;
        out[i] = __bfloat162float(pages[((obs * n_kv + kvh) * cap + tok) * hd + d]);
    }
}

constexpr int kFewRows = 256;  // suffix rows (n_obs * S) up to which the QKV projection takes the narrow-tile path
constexpr int kSplitSlices = 8;  // most K slices of a residual GEMM with few rows
// key-split attention: at most one (unit, slice) per SM, 128 rows of head_dim + 2 floats each
static size_t kAttnWsBytes(int hd) { return (size_t)160 * 128 * (hd + 2) * sizeof(float); }
}

// ------------------------------------------------------------------------ engine --
struct vlab200_engine {
    vlab200_policy_config c;
    int device = 0;  // the device that was current at creation: all of the engine's memory lives there
    int max_obs, P, P_max, S, cap, qf, kvf;  // P: rows of the prefix in use (<= P_max, the rows the pages were sized for)
    std::vector<int> is_self;
    // prepared weights
    std::vector<vb::DevBuf> wqkv, wo, wgu, wdown, wkx, wvx;
    vb::DevBuf w_ain, b_ain, w_sp, b_sp, w_at1l, tvec, w_at2, b_at2, out_norm, w_aout, b_aout;
    vb::DevBuf attn_ws;  // float32 workspace of the key-split attention path (calls with one or two observations)
    vb::DevBuf splitk;  // float32 [kSplitSlices][kFewRows][H]: K slices of Wo / Wdown when a call has few suffix rows
    vb::DevBuf mods;  // pi0.5: float32 [n_layers][2][steps][3H] (scale | shift | gate of the two norms), then [steps][3H] final
    // workspace
    vb::DevBuf k_pages, v_pages, h, hb, q, att, g, a, m1, x, rope_self, rope_cross, tmp_bf, x_stage, state_stage, pad_stage, vbuf;
    int rope_pos0 = -1;
    // one observation: the whole loop as one persistent kernel (chunk_loop.cu), built on first use for the prefix length in use
    vb::ChunkLoop *loop = nullptr;
    int loop_P = -1;
    ~vlab200_engine() { vb::chunk_loop_free(loop); }
};

namespace vb {

static int copy_dev(DevBuf &dst, const void *src, size_t bytes) {
    int rc = dst.alloc(bytes);
    if (rc) return rc;
    if (src) VB_CUDA(cudaMemcpy(dst.p, src, bytes, cudaMemcpyDeviceToDevice));
    return VLAB200_OK;
}

static int fold_rows(const void *w, const float *ln, void *out, int rows, int K, int row_mul, int row_add) {
    fold_rows_kernel<<<148 * 4, 256>>>(static_cast<const __nv_bfloat16 *>(w), ln, static_cast<__nv_bfloat16 *>(out),
                                       rows, K, row_mul, row_add);
    VB_CUDA(cudaGetLastError());
    return VLAB200_OK;
}

static int engine_build(vlab200_engine *e, const vlab200_policy_weights *w) {
    const vlab200_policy_config &c = e->c;
    const int L = c.n_layers, H = c.H, hd = c.head_dim, I = c.inter;
    const int qf = e->qf, kvf = e->kvf;
    const bool ada = c.model == 2;  // adaptive norms: nothing to fold, the norm is its own kernel
    e->wqkv.resize(L); e->wo.resize(L); e->wgu.resize(L); e->wdown.resize(L); e->wkx.resize(L); e->wvx.resize(L);
    int rc;
    for (int l = 0; l < L; ++l) {
        const bool self = e->is_self[l];
        const int rows = self ? qf + 2 * kvf : qf;
        const float *ln_in = ada ? nullptr : w->ln_in[l], *ln_post = ada ? nullptr : w->ln_post[l];
        if ((rc = e->wqkv[l].alloc((size_t)rows * H * 2))) return rc;
        auto *dst = e->wqkv[l].as<__nv_bfloat16>();
        if ((rc = fold_rows(w->wq[l], ln_in, dst, qf, H, 1, 0))) return rc;
        if (self) {
            if ((rc = fold_rows(w->wk[l], ln_in, dst + (size_t)qf * H, kvf, H, 1, 0))) return rc;
            if ((rc = fold_rows(w->wv[l], ln_in, dst + (size_t)(qf + kvf) * H, kvf, H, 1, 0))) return rc;
        } else {
            if ((rc = copy_dev(e->wkx[l], w->wk[l], (size_t)kvf * kvf * 2))) return rc;
            if ((rc = copy_dev(e->wvx[l], w->wv[l], (size_t)kvf * kvf * 2))) return rc;
        }
        if ((rc = copy_dev(e->wo[l], w->wo[l], (size_t)H * qf * 2))) return rc;
        if ((rc = e->wgu[l].alloc((size_t)2 * I * H * 2))) return rc;
        if ((rc = fold_rows(w->wgate[l], ln_post, e->wgu[l].p, I, H, 2, 0))) return rc;
        if ((rc = fold_rows(w->wup[l], ln_post, e->wgu[l].p, I, H, 2, 1))) return rc;
        if ((rc = copy_dev(e->wdown[l], w->wdown[l], (size_t)H * I * 2))) return rc;
    }
    const int A = c.action_dim, sd = c.state_dim, T = c.steps;
    if ((rc = copy_dev(e->w_ain, w->w_ain, (size_t)H * A * 2))) return rc;
    if ((rc = copy_dev(e->b_ain, w->b_ain, (size_t)H * 4))) return rc;
    if (c.model == 0) {
        if ((rc = copy_dev(e->w_sp, w->w_sp, (size_t)H * sd * 2))) return rc;
        if ((rc = copy_dev(e->b_sp, w->b_sp, (size_t)H * 4))) return rc;
    }
    if (!ada) {
        if ((rc = e->w_at1l.alloc((size_t)H * H * 2))) return rc;
        VB_CUDA(cudaMemcpy2D(e->w_at1l.p, (size_t)H * 2, w->w_at1, (size_t)2 * H * 2, (size_t)H * 2, H,
                             cudaMemcpyDeviceToDevice));
    }
    // time embeddings tau_k on the host in double, as the reference computes them
    // (src/layers/embed.h:61-73; pi0 forms the timestep in float, SmolVLA in double)
    std::vector<float> tau((size_t)T * H);
    const float dtf = -1.0f / (float)T;
    for (int s = 0; s < T; ++s) {
        const double t = c.model != 1 ? (double)(1.0f + (float)s * dtf) : 1.0 + (double)s * (double)dtf;
        const int half = H / 2;
        for (int i = 0; i < half; ++i) {
            const double frac = half == 1 ? 0.0 : (double)i / (double)(half - 1);
            const double period = c.min_period * std::pow(c.max_period / c.min_period, frac);
            const double ang = (2.0 * M_PI / period) * t;
            tau[(size_t)s * H + i] = (float)std::sin(ang);
            tau[(size_t)s * H + half + i] = (float)std::cos(ang);
        }
    }
    DevBuf tau_d;
    if ((rc = tau_d.alloc(tau.size() * 4))) return rc;
    VB_CUDA(cudaMemcpy(tau_d.p, tau.data(), tau.size() * 4, cudaMemcpyHostToDevice));
    if (!ada) {
        if ((rc = e->tvec.alloc((size_t)T * H * 4))) return rc;
        time_vector_kernel<<<(T * H * 32 + 255) / 256, 256>>>(static_cast<const __nv_bfloat16 *>(w->w_at1), w->b_at1,
                                                             tau_d.as<float>(), e->tvec.as<float>(), H, T);
        VB_CUDA(cudaGetLastError());
        if ((rc = copy_dev(e->w_at2, w->w_at2, (size_t)H * H * 2))) return rc;
        if ((rc = copy_dev(e->b_at2, w->b_at2, (size_t)H * 4))) return rc;
    } else {
        // cond_k for every step, then every layer's (scale | shift | gate) for every step: float32 throughout
        // (the reference keeps these weights float32, src/models/pi05.cpp:467-484)
        const int Hc = c.cond_dim > 0 ? c.cond_dim : H;
        DevBuf c1, cond;
        if ((rc = c1.alloc((size_t)T * Hc * 4)) || (rc = cond.alloc((size_t)T * Hc * 4))) return rc;
        if ((rc = skinny_linear(w->w_tin, w->b_tin, tau_d.as<float>(), nullptr, c1.as<float>(), T, Hc, H, 3, nullptr))) return rc;
        if ((rc = skinny_linear(w->w_tout, w->b_tout, c1.as<float>(), nullptr, cond.as<float>(), T, Hc, Hc, 3, nullptr))) return rc;
        const size_t per = (size_t)T * 3 * H;
        if ((rc = e->mods.alloc(((size_t)L * 2 + 1) * per * 4))) return rc;
        float *mods = e->mods.as<float>();
        for (int l = 0; l < L; ++l) {
            if ((rc = skinny_linear(w->ada_in_w[l], w->ada_in_b[l], cond.as<float>(), nullptr, mods + ((size_t)l * 2) * per, T, 3 * H, Hc, 0, nullptr)))
                return rc;
            if ((rc = skinny_linear(w->ada_post_w[l], w->ada_post_b[l], cond.as<float>(), nullptr, mods + ((size_t)l * 2 + 1) * per, T, 3 * H, Hc, 0,
                                    nullptr)))
                return rc;
        }
        if ((rc = skinny_linear(w->ada_final_w, w->ada_final_b, cond.as<float>(), nullptr, mods + (size_t)L * 2 * per, T, 3 * H, Hc, 0, nullptr)))
            return rc;
        VB_CUDA(cudaDeviceSynchronize());  // c1 / cond are released on return
    }
    // the output norm weight is folded into the action head like the layer norms into their projections
    if ((rc = e->w_aout.alloc((size_t)A * H * 2))) return rc;
    if ((rc = fold_rows(w->w_aout, ada ? nullptr : w->out_norm, e->w_aout.p, A, H, 1, 0))) return rc;
    if ((rc = copy_dev(e->b_aout, w->b_aout, (size_t)A * 4))) return rc;
    // workspace
    const size_t B = e->max_obs, M = B * e->S, Mc = B * c.chunk;
    const size_t page_bytes = (size_t)L * B * c.n_kv * e->cap * hd * 2;
    if ((rc = e->k_pages.alloc(page_bytes)) || (rc = e->v_pages.alloc(page_bytes))) return rc;
    VB_CUDA(cudaMemset(e->k_pages.p, 0, page_bytes));
    VB_CUDA(cudaMemset(e->v_pages.p, 0, page_bytes));
    if ((rc = e->h.alloc(M * H * 4)) || (rc = e->hb.alloc(M * H * 2)) || (rc = e->q.alloc(M * qf * 2)) ||
        (rc = e->att.alloc(M * qf * 2)) || (rc = e->g.alloc(M * I * 2)) || (rc = e->a.alloc(Mc * H * 2)) ||
        (rc = e->m1.alloc(Mc * H * 2)) || (rc = e->x.alloc(Mc * A * 4)) ||
        (rc = e->rope_self.alloc((size_t)2 * e->S * (hd / 2) * 4)) ||
        (rc = e->rope_cross.alloc((size_t)2 * e->S * (hd / 2) * 4)) ||
        (rc = e->tmp_bf.alloc((size_t)2 * B * e->P * kvf * 2)) || (rc = e->x_stage.alloc(Mc * A * 4)) ||
        (rc = e->state_stage.alloc(B * (size_t)(c.state_dim > 0 ? c.state_dim : 1) * 4)) ||
        (rc = e->pad_stage.alloc(B * 2 * 4)) || (rc = e->vbuf.alloc(M * A * 4)) ||
        (rc = e->splitk.alloc((size_t)kSplitSlices * kFewRows * H * 4)) || (rc = e->attn_ws.alloc(kAttnWsBytes(hd))))
        return rc;
    VB_CUDA(cudaMemset(e->h.p, 0, M * H * 4));
    VB_CUDA(cudaMemset(e->hb.p, 0, M * H * 2));
    VB_CUDA(cudaDeviceSynchronize());
    return VLAB200_OK;
}

static vlab200_kv_store engine_store(const vlab200_engine *e, int n_obs_view) {
    vlab200_kv_store st;
    st.k_pages = e->k_pages.p;
    st.v_pages = e->v_pages.p;
    st.n_layers = e->c.n_layers;
    st.n_obs = n_obs_view;
    st.n_kv = e->c.n_kv;
    st.head_dim = e->c.head_dim;
    st.cap = e->cap;
    st.prefix_len = e->P;
    return st;
}


// One expert layer = five launches (six on the few-row path).  Stages, in order:
//   0 fused RMSNorm + Q/K/V projection + RoPE + KV append   1 attention   2 O-projection + residual
//   3 fused RMSNorm + gate/up + activation                   4 down projection + residual
constexpr int kLayerStages = 5;

static int layer_stage(vlab200_engine *e, int l, int stage, int n_obs, const float *rs, const float *rx,
                       const int32_t *pad_ranges, cudaStream_t cs) {
    const vlab200_policy_config &c = e->c;
    const int H = c.H, S = e->S, hd = c.head_dim, I = c.inter, half = hd / 2;
    const int M = n_obs * S;
    const bool self = e->is_self[l];
    int rc;
    // pages are laid out for max_obs observations per layer; the kernels walk st.n_obs
    // observations from the store base, so hand them a one-layer view of the live ones
    vlab200_kv_store live = engine_store(e, e->max_obs);
    live.n_obs = n_obs;
    const size_t layer_off = (size_t)l * e->max_obs * c.n_kv * e->cap * hd;
    live.k_pages = e->k_pages.as<__nv_bfloat16>() + layer_off;
    live.v_pages = e->v_pages.as<__nv_bfloat16>() + layer_off;
    live.n_layers = 1;
    switch (stage) {
    case 0: {
        const float *rope = self ? rs : rx;
        const int qkv_n = (c.n_q + (self ? 2 * c.n_kv : 0)) * hd;
        if (M <= kFewRows && qkv_n <= I) {
            // Few rows: the fused kernel's 128 x 256 tiles leave most SMs idle (10 CTAs for one
            // observation).  Project with the narrow-tile GEMM (RMS factor in its epilogue) into the
            // MLP scratch buffer, which is free here, then rotate / split / append in one small kernel.
            GemmParams p{};
            p.M = M; p.N = qkv_n; p.K = H; p.epi = EPI_BIAS_ACT; p.act = ACT_NONE; p.use_rms = 1;
            p.eps = c.rms_eps; p.out_bf = e->g.as<__nv_bfloat16>(); p.ld_out = qkv_n;
            if ((rc = dense_gemm(e->hb.p, H, e->wqkv[l].p, p, cs))) return rc;
            return rope_split(e->g.p, rope, rope + (size_t)S * half, e->q.p, live.k_pages, live.v_pages, M, S, c.n_q,
                              self ? c.n_kv : 0, c.n_kv, hd, e->cap, e->P, cs);
        }
        return vlab200_qkv_rope_append(&live, 0, e->hb.p, 0, nullptr, e->wqkv[l].p, rope, rope + (size_t)S * half,
                                       c.rms_eps, S, H, c.n_q, self ? 1 : 0, e->q.p, cs);
    }
    case 1: {
        const int kv_len = self ? e->P + S : e->P;
        const int mode = self ? (c.model == 0 ? 1 : 2) : 0;
        return attention_ws(&live, 0, e->q.p, e->att.p, S, c.n_q, kv_len, mode, pad_ranges, cs, e->attn_ws.as<float>(),
                            kAttnWsBytes(hd));
    }
    case 2: {
        GemmParams p{};
        p.M = M; p.N = H; p.K = e->qf; p.epi = EPI_RESIDUAL;
        p.h = e->h.as<float>(); p.out_bf = e->hb.as<__nv_bfloat16>(); p.ld_out = H;
        p.partial = e->splitk.as<float>(); p.partial_slices = kSplitSlices; p.partial_rows = kFewRows;
        return dense_gemm(e->att.p, e->qf, e->wo[l].p, p, cs);
    }
    case 3: {
        GemmParams p{};
        p.M = M; p.N = 2 * I; p.K = H; p.epi = EPI_GATED; p.use_rms = 1; p.eps = c.rms_eps;
        p.act = c.model == 0 ? ACT_GELU_TANH : ACT_SILU;
        p.out_bf = e->g.as<__nv_bfloat16>(); p.ld_out = I;
        return dense_gemm(e->hb.p, H, e->wgu[l].p, p, cs);
    }
    case 4: {
        GemmParams p{};
        p.M = M; p.N = H; p.K = I; p.epi = EPI_RESIDUAL;
        p.h = e->h.as<float>(); p.out_bf = e->hb.as<__nv_bfloat16>(); p.ld_out = H;
        p.partial = e->splitk.as<float>(); p.partial_slices = kSplitSlices; p.partial_rows = kFewRows;
        return dense_gemm(e->g.p, I, e->wdown[l].p, p, cs);
    }
    default:
        return VLAB200_ERR_ARG;
    }
}

// One pi0.5 expert layer at Euler step `step` (build_expert_layer, src/models/pi05.cpp:226-292): seven launches.
static int ada_layer(vlab200_engine *e, int l, int step, int n_obs, const float *rope, cudaStream_t cs) {
    const vlab200_policy_config &c = e->c;
    const int H = c.H, S = e->S, hd = c.head_dim, I = c.inter, half = hd / 2, T = c.steps;
    const int M = n_obs * S, qkv_n = e->qf + 2 * e->kvf;
    const size_t per = (size_t)T * 3 * H;
    const float *mod_in = e->mods.as<float>() + ((size_t)l * 2) * per + (size_t)step * 3 * H;
    const float *mod_post = e->mods.as<float>() + ((size_t)l * 2 + 1) * per + (size_t)step * 3 * H;
    vlab200_kv_store live = engine_store(e, e->max_obs);
    live.n_obs = n_obs;
    const size_t layer_off = (size_t)l * e->max_obs * c.n_kv * e->cap * hd;
    live.k_pages = e->k_pages.as<__nv_bfloat16>() + layer_off;
    live.v_pages = e->v_pages.as<__nv_bfloat16>() + layer_off;
    live.n_layers = 1;
    int rc;
    float *h = e->h.as<float>();
    __nv_bfloat16 *hb = e->hb.as<__nv_bfloat16>();
    if ((rc = launch_pdl(adarms_norm_kernel, dim3((M + 7) / 8), dim3(256), 0, cs, static_cast<const float *>(h), mod_in, hb, M, H, c.rms_eps)))
        return rc;
    GemmParams p{};
    if (M <= kFewRows) {  // few rows: narrow-tile GEMM, then rotation / split / append (as in layer_stage)
        p.M = M; p.N = qkv_n; p.K = H; p.epi = EPI_BIAS_ACT; p.act = ACT_NONE; p.out_bf = e->g.as<__nv_bfloat16>(); p.ld_out = qkv_n;
        if ((rc = dense_gemm(hb, H, e->wqkv[l].p, p, cs))) return rc;
        if ((rc = rope_split(e->g.p, rope, rope + (size_t)S * half, e->q.p, live.k_pages, live.v_pages, M, S, c.n_q, c.n_kv, c.n_kv,
                             hd, e->cap, e->P, cs)))
            return rc;
    } else if ((rc = vlab200_qkv_rope_append(&live, 0, hb, 0, nullptr, e->wqkv[l].p, rope, rope + (size_t)S * half, -1.0f, S, H, c.n_q,
                                             1, e->q.p, cs))) {  // the fused kernel without its RMS factor
        return rc;
    }
    // no mask: every action token sees the prefix and every action token (soft_max_ext without a mask, pi05.cpp:264)
    if ((rc = attention_ws(&live, 0, e->q.p, e->att.p, S, c.n_q, e->P + S, 0, nullptr, cs, e->attn_ws.as<float>(), kAttnWsBytes(hd))))
        return rc;
    p = GemmParams{};
    p.M = M; p.N = H; p.K = e->qf; p.epi = EPI_RESIDUAL; p.colscale = mod_in + 2 * H;
    p.h = h; p.out_bf = hb; p.ld_out = H; p.partial = e->splitk.as<float>(); p.partial_slices = kSplitSlices; p.partial_rows = kFewRows;
    if ((rc = dense_gemm(e->att.p, e->qf, e->wo[l].p, p, cs))) return rc;
    if ((rc = launch_pdl(adarms_norm_kernel, dim3((M + 7) / 8), dim3(256), 0, cs, static_cast<const float *>(h), mod_post, hb, M, H, c.rms_eps)))
        return rc;
    p = GemmParams{};
    p.M = M; p.N = 2 * I; p.K = H; p.epi = EPI_GATED; p.act = ACT_GELU_TANH; p.out_bf = e->g.as<__nv_bfloat16>(); p.ld_out = I;
    if ((rc = dense_gemm(hb, H, e->wgu[l].p, p, cs))) return rc;
    p = GemmParams{};
    p.M = M; p.N = H; p.K = I; p.epi = EPI_RESIDUAL; p.colscale = mod_post + 2 * H;
    p.h = h; p.out_bf = hb; p.ld_out = H; p.partial = e->splitk.as<float>(); p.partial_slices = kSplitSlices; p.partial_rows = kFewRows;
    return dense_gemm(e->g.p, I, e->wdown[l].p, p, cs);
}

// The persistent loop kernel for calls with one observation, on the engine's own buffers.
static int engine_chunk_loop(vlab200_engine *e) {
    const vlab200_policy_config &c = e->c;
    ChunkLoopDesc d{};
    d.model = c.model; d.L = c.n_layers; d.H = c.H; d.I = c.inter; d.n_q = c.n_q; d.n_kv = c.n_kv; d.hd = c.head_dim; d.S = e->S;
    d.chunk = c.chunk; d.A = c.action_dim; d.sd = c.state_dim; d.steps = c.steps; d.cap = e->cap; d.P = e->P;
    d.act = c.model == 1 ? ACT_SILU : ACT_GELU_TANH; d.rms_eps = c.rms_eps;
    d.is_self = e->is_self.data();
    std::vector<const void *> wqkv(c.n_layers), wo(c.n_layers), wgu(c.n_layers), wdown(c.n_layers);
    for (int l = 0; l < c.n_layers; ++l) {
        wqkv[l] = e->wqkv[l].p; wo[l] = e->wo[l].p; wgu[l] = e->wgu[l].p; wdown[l] = e->wdown[l].p;
    }
    d.wqkv = wqkv.data(); d.wo = wo.data(); d.wgu = wgu.data(); d.wdown = wdown.data();
    d.w_ain = e->w_ain.p; d.w_sp = e->w_sp.p; d.w_at1l = e->w_at1l.p; d.w_at2 = e->w_at2.p; d.w_aout = e->w_aout.p;
    d.b_ain = e->b_ain.as<float>(); d.b_sp = e->b_sp.as<float>(); d.tvec = e->tvec.as<float>(); d.b_at2 = e->b_at2.as<float>();
    d.b_aout = e->b_aout.as<float>();
    d.k_pages = e->k_pages.p; d.v_pages = e->v_pages.p;
    d.layer_stride = (size_t)e->max_obs * c.n_kv * e->cap * c.head_dim;
    d.h = e->h.as<float>(); d.x = e->x.as<float>();
    d.rope_self = e->rope_self.as<float>(); d.rope_cross = e->rope_cross.as<float>();
    d.mods = c.model == 2 ? e->mods.as<float>() : nullptr;
    return chunk_loop_create(d, &e->loop);
}

}  // namespace vb

extern "C" {

vlab200_engine *vlab200_engine_create(const vlab200_policy_config *cfg, const vlab200_policy_weights *w,
                                      int32_t max_obs, int32_t prefix_len) {
    if (!cfg || !w || max_obs <= 0 || prefix_len <= 0) {
        vb::set_last_error("vlab200_engine_create: null configuration / weights, or max_obs / prefix_len <= 0");
        return nullptr;
    }
    const vlab200_policy_config &c = *cfg;
    if (c.n_layers <= 0 || c.H <= 0 || c.n_q <= 0 || c.n_kv <= 0 || c.n_q % c.n_kv || c.inter <= 0 || c.chunk <= 0 ||
        c.action_dim <= 0 || c.action_dim > 64 || c.action_dim % 8 || c.state_dim > 64 || c.steps <= 0 || c.model < 0 || c.model > 2) {
        vb::set_last_error("vlab200_engine_create: bad configuration");
        return nullptr;
    }
    if (c.H % 8) {
        vb::set_last_error("vlab200_engine_create: hidden size %d is not a multiple of 8", c.H);
        return nullptr;
    }
    if (c.model == 2 && (!w->ada_in_w || !w->ada_in_b || !w->ada_post_w || !w->ada_post_b || !w->ada_final_w || !w->ada_final_b ||
                         !w->w_tin || !w->b_tin || !w->w_tout || !w->b_tout || (c.n_q + 2 * c.n_kv) * c.head_dim > c.inter)) {
        vb::set_last_error("vlab200_engine_create: pi0.5 needs the adaptive-norm and time-MLP weights and (n_q + 2 n_kv) head_dim <= inter");
        return nullptr;
    }
    vlab200_engine *e = new (std::nothrow) vlab200_engine();
    if (!e) {
        vb::set_last_error("vlab200_engine_create: out of host memory");
        return nullptr;
    }
    e->c = c;
    if (cudaGetDevice(&e->device) != cudaSuccess) e->device = 0;
    e->max_obs = max_obs;
    e->P = prefix_len;
    e->P_max = prefix_len;
    e->S = c.chunk + (c.model == 0 ? 1 : 0);  // pi0 alone carries the state as a suffix token
    e->cap = e->P + e->S;
    e->qf = c.n_q * c.head_dim;
    e->kvf = c.n_kv * c.head_dim;
    e->is_self.resize(c.n_layers);
    for (int l = 0; l < c.n_layers; ++l)
        e->is_self[l] = (c.model != 1) || (c.self_every <= 1) || (l % c.self_every == 0);
    const int brc = vb::engine_build(e, w);
    if (brc != VLAB200_OK) {
        if (brc != VLAB200_ERR_CUDA) vb::set_last_error("vlab200_engine_create: building the engine failed with status %d", brc);
        delete e;
        return nullptr;
    }
    return e;
}

void vlab200_engine_free(vlab200_engine *e) { delete e; }

int32_t vlab200_engine_set_prefix(vlab200_engine *e, int32_t layer, int32_t obs0, int32_t n_obs, const float *K,
                                  const float *V, void *stream) {
    if (!e || !K || !V || layer < 0 || layer >= e->c.n_layers || obs0 < 0 || n_obs <= 0 || obs0 + n_obs > e->max_obs)
        return VLAB200_ERR_ARG;
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    vlab200_kv_store st = vb::engine_store(e, e->max_obs);
    if (e->is_self[layer]) return vlab200_kv_store_write(&st, layer, obs0, n_obs, K, V, cs);
    // SmolVLA cross-attention layer: K' = Wk K_flat, V' = Wv V_flat once per observation
    // (src/models/smolvla.cpp:853-860), written head-major into the pages of this layer
    const size_t n = (size_t)n_obs * e->P * e->kvf;
    __nv_bfloat16 *kb = e->tmp_bf.as<__nv_bfloat16>(), *vbuf = kb + (size_t)e->max_obs * e->P_max * e->kvf;
    vb::f32_to_bf16_kernel<<<148 * 4, 256, 0, cs>>>(K, kb, n);
    vb::f32_to_bf16_kernel<<<148 * 4, 256, 0, cs>>>(V, vbuf, n);
    VB_CUDA(cudaGetLastError());
    const size_t page_off = ((size_t)layer * e->max_obs + obs0) * e->c.n_kv * e->cap * e->c.head_dim;
    for (int which = 0; which < 2; ++which) {
        vb::GemmParams p{};
        p.M = n_obs * e->P; p.N = e->kvf; p.K = e->kvf;
        p.epi = vb::EPI_BIAS_ACT; p.act = vb::ACT_NONE; p.use_rms = 0; p.eps = 0.f;
        p.out_bf = (which ? e->v_pages.as<__nv_bfloat16>() : e->k_pages.as<__nv_bfloat16>()) + page_off;
        p.ld_out = e->c.head_dim;
        p.rows_in = e->P; p.rows_out = 0; p.row_off = 0;
        p.scatter_hd = e->c.head_dim; p.scatter_cap = e->cap;
        int rc = vb::dense_gemm(which ? vbuf : kb, e->kvf, which ? e->wvx[layer].p : e->wkx[layer].p, p, cs);
        if (rc) return rc;
    }
    return VLAB200_OK;
}

int32_t vlab200_engine_denoise(vlab200_engine *e, int32_t n_obs, const float *state, const float *x0, float *x_out,
                               int32_t pos_base, const int32_t *pad_ranges, void *stream) {
    if (!e || !x0 || !x_out || n_obs <= 0 || n_obs > e->max_obs) return VLAB200_ERR_ARG;
    if (e->c.model == 0 && !state) return VLAB200_ERR_ARG;
    const vlab200_policy_config &c = e->c;
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    const int H = c.H, S = e->S, chunk = c.chunk, A = c.action_dim, hd = c.head_dim;
    const int M = n_obs * S, Mc = n_obs * chunk;
    int rc;
    if (pos_base < 0) pos_base = e->P;
    float *rs = e->rope_self.as<float>(), *rx = e->rope_cross.as<float>();
    const int half = hd / 2;
    if ((rc = vlab200_rope_table(rs, rs + (size_t)S * half, pos_base, S, hd, c.rope_base, cs))) return rc;
    if ((rc = vlab200_rope_table(rx, rx + (size_t)S * half, 0, S, hd, c.rope_base, cs))) return rc;
    VB_CUDA(cudaMemcpyAsync(e->x.p, x0, (size_t)Mc * A * 4, cudaMemcpyDeviceToDevice, cs));
    // One observation: the whole loop as one persistent kernel (10.4 vs 11.4 ms per chunk for a pi0-shaped expert, 5.9 vs
    // 7.6 ms SmolVLA-shaped); VLAB200_CHUNK_LOOP=0 keeps the launch-per-operator path.
    const char *loop_env = std::getenv("VLAB200_CHUNK_LOOP");
    const bool want_loop = !loop_env || loop_env[0] != '0';
    if (n_obs == 1 && want_loop) {
        if (e->loop_P != e->P) {
            vb::chunk_loop_free(e->loop);
            e->loop = nullptr;
            e->loop_P = e->P;
            if ((rc = vb::engine_chunk_loop(e)) && rc != VLAB200_ERR_UNSUPPORTED) return rc;
        }
        if (e->loop) {
            rc = vb::chunk_loop_run(e->loop, state, pad_ranges, cs);
            if (rc == VLAB200_OK) {
                VB_CUDA(cudaMemcpyAsync(x_out, e->x.p, (size_t)Mc * A * 4, cudaMemcpyDeviceToDevice, cs));
                return VLAB200_OK;
            }
            if (rc != VLAB200_ERR_UNSUPPORTED) return rc;
            vb::chunk_loop_free(e->loop);  // the grid does not fit this process's share of the device: a launch per operator from now on
            e->loop = nullptr;
        }
    }
    const float dt = -1.0f / (float)c.steps;
    for (int step = 0; step < c.steps; ++step) {
        if ((rc = vb::launch_pdl(vb::action_in_kernel, dim3((Mc + vb::AIN_ROWS - 1) / vb::AIN_ROWS, (H + 255) / 256), dim3(256), 0, cs,
                                 e->x.as<float>(), e->w_ain.as<__nv_bfloat16>(), e->b_ain.as<float>(), e->a.as<__nv_bfloat16>(),
                                 c.model == 2 ? e->h.as<float>() : static_cast<float *>(nullptr), Mc, H, A)))
            return rc;
        if (c.model == 2) {
            for (int l = 0; l < c.n_layers; ++l)
                if ((rc = vb::ada_layer(e, l, step, n_obs, rs, cs))) return rc;
            const float *mod_f = e->mods.as<float>() + (size_t)c.n_layers * 2 * c.steps * 3 * H + (size_t)step * 3 * H;
            if ((rc = vb::launch_pdl(vb::adarms_norm_kernel, dim3((M + 7) / 8), dim3(256), 0, cs, static_cast<const float *>(e->h.as<float>()),
                                     mod_f, e->hb.as<__nv_bfloat16>(), M, H, c.rms_eps)))
                return rc;
            vb::GemmParams p{};
            p.M = M; p.N = A; p.K = H; p.epi = vb::EPI_BIAS_ACT; p.act = vb::ACT_NONE;
            p.out_f32 = e->vbuf.as<float>(); p.bias = e->b_aout.as<float>(); p.ld_out = A;
            if ((rc = vb::dense_gemm(e->hb.p, H, e->w_aout.p, p, cs))) return rc;
            if ((rc = vb::launch_pdl(vb::euler_kernel, dim3((Mc * A + 255) / 256), dim3(256), 0, cs, e->x.as<float>(),
                                     e->vbuf.as<float>(), Mc * A, A, chunk, S, dt)))
                return rc;
            continue;
        }
        if (c.model == 0 &&
            (rc = vb::launch_pdl(vb::state_token_kernel, dim3(n_obs), dim3(256), 0, cs, state, e->w_sp.as<__nv_bfloat16>(),
                                 e->b_sp.as<float>(), e->h.as<float>(), e->hb.as<__nv_bfloat16>(), H, c.state_dim, S)))
            return rc;
        {
            vb::GemmParams p{};
            p.M = Mc; p.N = H; p.K = H; p.epi = vb::EPI_BIAS_ACT; p.act = vb::ACT_SILU;
            p.out_bf = e->m1.as<__nv_bfloat16>(); p.bias = e->tvec.as<float>() + (size_t)step * H; p.ld_out = H;
            if ((rc = vb::dense_gemm(e->a.p, H, e->w_at1l.p, p, cs))) return rc;
        }
        {
            vb::GemmParams p{};
            p.M = Mc; p.N = H; p.K = H; p.epi = vb::EPI_BIAS_ACT; p.act = vb::ACT_NONE;
            p.out_bf = e->hb.as<__nv_bfloat16>(); p.out_f32 = e->h.as<float>(); p.bias = e->b_at2.as<float>();
            p.ld_out = H; p.rows_in = chunk; p.rows_out = S; p.row_off = S - chunk;
            if ((rc = vb::dense_gemm(e->m1.p, H, e->w_at2.p, p, cs))) return rc;
        }
        for (int l = 0; l < c.n_layers; ++l)
            for (int stage = 0; stage < vb::kLayerStages; ++stage)
                if ((rc = vb::layer_stage(e, l, stage, n_obs, rs, rx, pad_ranges, cs))) return rc;
        {   // v = W_aout (rms(h) * w_out) + b_aout over every suffix row, then the Euler update on the action rows
            vb::GemmParams p{};
            p.M = M; p.N = A; p.K = H; p.epi = vb::EPI_BIAS_ACT; p.act = vb::ACT_NONE; p.use_rms = 1; p.eps = c.rms_eps;
            p.out_f32 = e->vbuf.as<float>(); p.bias = e->b_aout.as<float>(); p.ld_out = A;
            if ((rc = vb::dense_gemm(e->hb.p, H, e->w_aout.p, p, cs))) return rc;
            if ((rc = vb::launch_pdl(vb::euler_kernel, dim3((Mc * A + 255) / 256), dim3(256), 0, cs, e->x.as<float>(),
                                     e->vbuf.as<float>(), Mc * A, A, chunk, S, dt)))
                return rc;
        }
    }
    VB_CUDA(cudaMemcpyAsync(x_out, e->x.p, (size_t)Mc * A * 4, cudaMemcpyDeviceToDevice, cs));
    return VLAB200_OK;
}

int32_t vlab200_engine_denoise_host(vlab200_engine *e, int32_t n_obs, const float *state_host, const float *x0_host,
                                    float *x_out_host, int32_t pos_base, const int32_t *pad_ranges_host,
                                    void *stream) {
    if (!e || !x0_host || !x_out_host || n_obs <= 0 || n_obs > e->max_obs) return VLAB200_ERR_ARG;
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    const size_t xb = (size_t)n_obs * e->c.chunk * e->c.action_dim * 4, sb = (size_t)n_obs * e->c.state_dim * 4;
    float *x_dev = e->x_stage.as<float>();
    float *s_dev = e->state_stage.as<float>();
    VB_CUDA(cudaMemcpyAsync(x_dev, x0_host, xb, cudaMemcpyHostToDevice, cs));
    if (state_host) VB_CUDA(cudaMemcpyAsync(s_dev, state_host, sb, cudaMemcpyHostToDevice, cs));
    int32_t *pad_dev = nullptr;
    if (pad_ranges_host) {
        pad_dev = e->pad_stage.as<int32_t>();
        VB_CUDA(cudaMemcpyAsync(pad_dev, pad_ranges_host, (size_t)n_obs * 2 * 4, cudaMemcpyHostToDevice, cs));
    }
    int rc = vlab200_engine_denoise(e, n_obs, state_host ? s_dev : nullptr, x_dev, x_dev, pos_base, pad_dev, cs);
    if (rc) return rc;
    VB_CUDA(cudaMemcpyAsync(x_out_host, x_dev, xb, cudaMemcpyDeviceToHost, cs));
    return VLAB200_OK;
}

int32_t vlab200_engine_run_stage(vlab200_engine *e, int32_t layer, int32_t stage, int32_t n_obs, int32_t reps,
                                 void *stream) {
    if (!e || layer < 0 || layer >= e->c.n_layers || stage < 0 || stage >= vb::kLayerStages || n_obs <= 0 ||
        n_obs > e->max_obs || reps <= 0)
        return VLAB200_ERR_ARG;
    if (e->c.model == 2) return VLAB200_ERR_UNSUPPORTED;  // the pi0.5 layer has its own seven stages
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    const float *rs = e->rope_self.as<float>(), *rx = e->rope_cross.as<float>();
    for (int i = 0; i < reps; ++i) {
        int rc = vb::layer_stage(e, layer, stage, n_obs, rs, rx, nullptr, cs);
        if (rc) return rc;
    }
    return VLAB200_OK;
}

int32_t vlab200_engine_get_prefix(vlab200_engine *e, int32_t layer, int32_t obs0, int32_t n_obs, float *K, float *V,
                                  void *stream) {
    if (!e || !K || !V || layer < 0 || layer >= e->c.n_layers || obs0 < 0 || n_obs <= 0 || obs0 + n_obs > e->max_obs)
        return VLAB200_ERR_ARG;
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    const size_t page_off = ((size_t)layer * e->max_obs + obs0) * e->c.n_kv * e->cap * e->c.head_dim;
    const size_t total = (size_t)n_obs * e->P * e->kvf;
    vb::pages_to_f32_kernel<<<148 * 4, 256, 0, cs>>>(e->k_pages.as<__nv_bfloat16>() + page_off, K, e->c.n_kv, e->cap,
                                                     e->c.head_dim, e->P, total);
    vb::pages_to_f32_kernel<<<148 * 4, 256, 0, cs>>>(e->v_pages.as<__nv_bfloat16>() + page_off, V, e->c.n_kv, e->cap,
                                                     e->c.head_dim, e->P, total);
    VB_CUDA(cudaGetLastError());
    return VLAB200_OK;
}

int32_t vlab200_engine_set_prefix_len(vlab200_engine *e, int32_t prefix_len) {
    if (!e || prefix_len <= 0 || prefix_len > e->P_max) return VLAB200_ERR_ARG;
    e->P = prefix_len;
    return VLAB200_OK;
}

}  // extern "C"

// ------------------------------------------------------------- several GPUs, one process --
// Observations are independent (one predict = one observation, src/model.h:204-225): a list of them is cut into
// contiguous blocks, one per engine (= per GPU, each with its weight replica and its own K/V pages); one host thread
// and one stream per engine; nothing is exchanged between GPUs on the way.
extern "C" {

int32_t vlab200_shard_range(int64_t n_items, int32_t n_ranks, int32_t rank, int64_t *start, int64_t *count) {
    if (!start || !count || n_items < 0 || n_ranks <= 0 || rank < 0 || rank >= n_ranks) return VLAB200_ERR_ARG;
    const int64_t base = n_items / n_ranks, rem = n_items % n_ranks;
    *count = base + (rank < rem ? 1 : 0);
    *start = (int64_t)rank * base + (rank < rem ? rank : rem);
    return VLAB200_OK;
}

int32_t vlab200_engines_denoise_host(vlab200_engine *const *engines, int32_t n_engines, int64_t n_obs,
                                     const float *state_host, const float *x0_host, float *x_out_host, int32_t pos_base,
                                     const int32_t *pad_ranges_host) {
    if (!engines || n_engines <= 0 || n_obs < 0 || !x0_host || !x_out_host) return VLAB200_ERR_ARG;
    for (int i = 0; i < n_engines; ++i)
        if (!engines[i]) return VLAB200_ERR_ARG;
    std::vector<int> rcs((size_t)n_engines, VLAB200_OK);
    std::vector<std::string> errs((size_t)n_engines);
    std::vector<std::thread> workers;
    for (int r = 0; r < n_engines; ++r)
        workers.emplace_back([&, r] {
            vlab200_engine *e = engines[r];
            int64_t start = 0, count = 0;
            vlab200_shard_range(n_obs, n_engines, r, &start, &count);
            auto fail = [&](int rc) {
                rcs[(size_t)r] = rc;
                errs[(size_t)r] = vlab200_last_error();
            };
            if (cudaSetDevice(e->device) != cudaSuccess) return fail(vb::cuda_fail(cudaGetLastError(), "cudaSetDevice"));
            cudaStream_t st = nullptr;
            if (cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking) != cudaSuccess)
                return fail(vb::cuda_fail(cudaGetLastError(), "cudaStreamCreate"));
            const size_t xrow = (size_t)e->c.chunk * e->c.action_dim, srow = (size_t)e->c.state_dim;
            int rc = VLAB200_OK;
            // blocks of at most max_obs observations, one after the other on this engine's stream
            for (int64_t done = 0; done < count && rc == VLAB200_OK; done += e->max_obs) {
                const int64_t o = start + done;
                const int32_t n = (int32_t)(count - done < e->max_obs ? count - done : e->max_obs);
                rc = vlab200_engine_denoise_host(e, n, state_host ? state_host + (size_t)o * srow : nullptr, x0_host + (size_t)o * xrow,
                                                 x_out_host + (size_t)o * xrow, pos_base,
                                                 pad_ranges_host ? pad_ranges_host + (size_t)o * 2 : nullptr, st);
                // the staging buffers are reused by the next block
                if (rc == VLAB200_OK && cudaStreamSynchronize(st) != cudaSuccess) rc = vb::cuda_fail(cudaGetLastError(), "cudaStreamSynchronize");
            }
            cudaStreamDestroy(st);
            if (rc != VLAB200_OK) fail(rc);
        });
    for (std::thread &t : workers) t.join();
    for (int r = 0; r < n_engines; ++r)
        if (rcs[(size_t)r] != VLAB200_OK) {
            vb::set_last_error("engine %d: %s", r, errs[(size_t)r].c_str());
            return rcs[(size_t)r];
        }
    return VLAB200_OK;
}

}  // extern "C"

// ------------------------------------------------------------------ prefix producer --
// The VLM layers over the prefix tokens of an observation (image, language and, for SmolVLA, state
// embeddings), written straight into the denoise engine's bf16 K/V pages: layer l's rotated K and its V
// are what expert layer l reads for the whole denoise loop (src/models/smolvla.cpp:778-813,1374-1391;
// src/models/pi0.cpp:159-233,557-566).  Same five stages as an expert layer with the prefix as the
// "suffix" of an empty cache; SmolVLA's cross-attention layers get Wk K / Wv V (expert_cross_kv) in place.
struct vlab200_prefill {
    vlab200_prefill_config c;
    int max_obs, max_prefix, qf, kvf;
    std::vector<vb::DevBuf> wqkv, wo, wgu, wdown;
    vb::DevBuf h, hb, qkv, q, att, g, rope, pos;
};

namespace vb {

__global__ void embed_to_stream_kernel(const float *__restrict__ x, float *__restrict__ h, __nv_bfloat16 *__restrict__ hb,
                                       size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float v = x[i];
        h[i] = v;
        hb[i] = __float2bfloat16(v);
    }
}

// cos / sin rows for explicit positions (the SmolVLA state token does not sit at its row index)
__global__ void rope_table_pos_kernel(float *cos_t, float *sin_t, const int32_t *__restrict__ pos, int S, int hd, float base) {
    const int half = hd >> 1;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= S * half) return;
    const int t = i / half, d = i % half;
    const float freq = powf(base, -2.0f * (float)d / (float)hd);
    const float ang = (float)pos[t] * freq;
    cos_t[i] = cosf(ang);
    sin_t[i] = sinf(ang);
}

// pages [n_obs][n_kv][cap][hd] rows [0, P) -> token-major [n_obs * P][n_kv * hd]
__global__ void pages_to_rows_kernel(const __nv_bfloat16 *__restrict__ pages, __nv_bfloat16 *__restrict__ rows, int n_kv,
                                     int cap, int hd, int P, size_t total_vec) {
    const int hv = hd / 8;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total_vec; i += (size_t)gridDim.x * blockDim.x) {
        const int v8 = (int)(i % hv);
        size_t r = i / hv;
        const int kvh = (int)(r % n_kv);
        r /= n_kv;
        const int tok = (int)(r % P);
        const size_t obs = r / P;
        const uint4 val = *reinterpret_cast<const uint4 *>(pages + ((obs * n_kv + kvh) * cap + tok) * hd + (size_t)v8 * 8);
        *reinterpret_cast<uint4 *>(rows + ((obs * P + tok) * n_kv + kvh) * hd + (size_t)v8 * 8) = val;
    }
}

}  // namespace vb

extern "C" {

vlab200_prefill *vlab200_prefill_create(const vlab200_prefill_config *cfg, const vlab200_prefill_weights *w,
                                        int32_t max_obs, int32_t max_prefix) {
    if (!cfg || !w || max_obs <= 0 || max_prefix <= 0) {
        vb::set_last_error("vlab200_prefill_create: null configuration / weights, or max_obs / max_prefix <= 0");
        return nullptr;
    }
    const vlab200_prefill_config &c = *cfg;
    if (c.n_layers <= 0 || c.hidden <= 0 || c.hidden % 8 || c.n_q <= 0 || c.n_kv <= 0 || c.n_q % c.n_kv || c.inter <= 0 ||
        (c.head_dim != 64 && c.head_dim != 128 && c.head_dim != 256) || (c.act != vb::ACT_SILU && c.act != vb::ACT_GELU_TANH)) {
        vb::set_last_error("vlab200_prefill_create: bad configuration");
        return nullptr;
    }
    auto *p = new (std::nothrow) vlab200_prefill();
    if (!p) return nullptr;
    p->c = c;
    p->max_obs = max_obs;
    p->max_prefix = max_prefix;
    p->qf = c.n_q * c.head_dim;
    p->kvf = c.n_kv * c.head_dim;
    const int L = c.n_layers, H = c.hidden, I = c.inter, qf = p->qf, kvf = p->kvf;
    p->wqkv.resize(L); p->wo.resize(L); p->wgu.resize(L); p->wdown.resize(L);
    int rc = VLAB200_OK;
    for (int l = 0; l < L && !rc; ++l) {
        // same prepared forms as the engine: norm weights folded in, q/k/v concatenated, gate/up interleaved
        if ((rc = p->wqkv[l].alloc((size_t)(qf + 2 * kvf) * H * 2))) break;
        auto *dst = p->wqkv[l].as<__nv_bfloat16>();
        if ((rc = vb::fold_rows(w->wq[l], w->ln_in[l], dst, qf, H, 1, 0))) break;
        if ((rc = vb::fold_rows(w->wk[l], w->ln_in[l], dst + (size_t)qf * H, kvf, H, 1, 0))) break;
        if ((rc = vb::fold_rows(w->wv[l], w->ln_in[l], dst + (size_t)(qf + kvf) * H, kvf, H, 1, 0))) break;
        if (l + 1 == L) break;  // the last layer only has to produce K and V
        if ((rc = vb::copy_dev(p->wo[l], w->wo[l], (size_t)H * qf * 2))) break;
        if ((rc = p->wgu[l].alloc((size_t)2 * I * H * 2))) break;
        if ((rc = vb::fold_rows(w->wgate[l], w->ln_post[l], p->wgu[l].p, I, H, 2, 0))) break;
        if ((rc = vb::fold_rows(w->wup[l], w->ln_post[l], p->wgu[l].p, I, H, 2, 1))) break;
        if ((rc = vb::copy_dev(p->wdown[l], w->wdown[l], (size_t)H * I * 2))) break;
    }
    const size_t M = (size_t)max_obs * max_prefix;
    if (!rc) rc = p->h.alloc(M * H * 4);
    if (!rc) rc = p->hb.alloc(M * H * 2);
    if (!rc) rc = p->qkv.alloc(M * (size_t)(qf + 2 * kvf) * 2);
    if (!rc) rc = p->q.alloc(M * qf * 2);
    if (!rc) rc = p->att.alloc(M * qf * 2);
    if (!rc) rc = p->g.alloc(M * I * 2);
    if (!rc) rc = p->rope.alloc((size_t)2 * max_prefix * (c.head_dim / 2) * 4);
    if (!rc) rc = p->pos.alloc((size_t)max_prefix * 4);
    if (!rc && cudaDeviceSynchronize() != cudaSuccess) rc = vb::cuda_fail(cudaGetLastError(), "vlab200_prefill_create");
    if (rc) {
        if (rc != VLAB200_ERR_CUDA) vb::set_last_error("vlab200_prefill_create: failed with status %d", rc);
        delete p;
        return nullptr;
    }
    return p;
}

void vlab200_prefill_free(vlab200_prefill *p) { delete p; }

int32_t vlab200_prefill_run(vlab200_prefill *p, vlab200_engine *e, int32_t obs0, int32_t n_obs, const float *x_emb,
                            int32_t P, const int32_t *pos_host, int32_t mask_mode, const int32_t *pad_ranges,
                            void *stream) {
    if (!p || !e || !x_emb || obs0 < 0 || n_obs <= 0 || n_obs > p->max_obs || obs0 + n_obs > e->max_obs || P <= 0 ||
        P > p->max_prefix || P != e->P)
        return VLAB200_ERR_ARG;
    const vlab200_prefill_config &c = p->c;
    if (c.n_layers != e->c.n_layers || c.n_kv != e->c.n_kv || c.head_dim != e->c.head_dim) {
        vb::set_last_error("vlab200_prefill_run: the prefill and the engine disagree on layers / kv heads / head_dim");
        return VLAB200_ERR_ARG;
    }
    if (mask_mode != 0 && mask_mode != 3) return VLAB200_ERR_ARG;
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    const int H = c.hidden, I = c.inter, hd = c.head_dim, qf = p->qf, kvf = p->kvf, half = hd / 2;
    const int M = n_obs * P, qkv_n = qf + 2 * kvf;
    int rc;
    float *cos_t = p->rope.as<float>(), *sin_t = cos_t + (size_t)P * half;
    if (pos_host) {
        VB_CUDA(cudaMemcpyAsync(p->pos.p, pos_host, (size_t)P * 4, cudaMemcpyHostToDevice, cs));
        vb::rope_table_pos_kernel<<<(P * half + 127) / 128, 128, 0, cs>>>(cos_t, sin_t, p->pos.as<int32_t>(), P, hd, c.rope_base);
        VB_CUDA(cudaGetLastError());
    } else if ((rc = vlab200_rope_table(cos_t, sin_t, 0, P, hd, c.rope_base, cs))) {
        return rc;
    }
    vb::embed_to_stream_kernel<<<148 * 4, 256, 0, cs>>>(x_emb, p->h.as<float>(), p->hb.as<__nv_bfloat16>(), (size_t)M * H);
    VB_CUDA(cudaGetLastError());
    for (int l = 0; l < c.n_layers; ++l) {
        const size_t page_off = ((size_t)l * e->max_obs + obs0) * c.n_kv * e->cap * hd;
        __nv_bfloat16 *kp = e->k_pages.as<__nv_bfloat16>() + page_off, *vp = e->v_pages.as<__nv_bfloat16>() + page_off;
        {   // RMSNorm (factor in the epilogue, weight folded) + q | k | v, then rotation and the page write
            vb::GemmParams g{};
            g.M = M; g.N = qkv_n; g.K = H; g.epi = vb::EPI_BIAS_ACT; g.act = vb::ACT_NONE; g.use_rms = 1; g.eps = c.rms_eps;
            g.out_bf = p->qkv.as<__nv_bfloat16>(); g.ld_out = qkv_n;
            if ((rc = vb::dense_gemm(p->hb.p, H, p->wqkv[l].p, g, cs))) return rc;
            if ((rc = vb::rope_split(p->qkv.p, cos_t, sin_t, p->q.p, kp, vp, M, P, c.n_q, c.n_kv, c.n_kv, hd, e->cap, 0, cs)))
                return rc;
        }
        if (l + 1 < c.n_layers) {
            vlab200_kv_store view{kp, vp, 1, n_obs, c.n_kv, hd, e->cap, 0};
            if ((rc = vlab200_attention(&view, 0, p->q.p, p->att.p, P, c.n_q, P, mask_mode, pad_ranges, cs))) return rc;
            vb::GemmParams g{};
            g.M = M; g.N = H; g.K = qf; g.epi = vb::EPI_RESIDUAL;
            g.h = p->h.as<float>(); g.out_bf = p->hb.as<__nv_bfloat16>(); g.ld_out = H;
            if ((rc = vb::dense_gemm(p->att.p, qf, p->wo[l].p, g, cs))) return rc;
            g = vb::GemmParams{};
            g.M = M; g.N = 2 * I; g.K = H; g.epi = vb::EPI_GATED; g.use_rms = 1; g.eps = c.rms_eps; g.act = c.act;
            g.out_bf = p->g.as<__nv_bfloat16>(); g.ld_out = I;
            if ((rc = vb::dense_gemm(p->hb.p, H, p->wgu[l].p, g, cs))) return rc;
            g = vb::GemmParams{};
            g.M = M; g.N = H; g.K = I; g.epi = vb::EPI_RESIDUAL;
            g.h = p->h.as<float>(); g.out_bf = p->hb.as<__nv_bfloat16>(); g.ld_out = H;
            if ((rc = vb::dense_gemm(p->g.p, I, p->wdown[l].p, g, cs))) return rc;
        }
        if (!e->is_self[l]) {
            // expert_cross_kv (src/models/smolvla.cpp:853-860): K' = Wk K, V' = Wv V on the flattened kv axis of the
            // rotated prefix K / V, once per observation; the layer's own attention above has already read the raw pages
            __nv_bfloat16 *kb = e->tmp_bf.as<__nv_bfloat16>(), *vbuf = kb + (size_t)e->max_obs * e->P_max * kvf;
            const size_t total_vec = (size_t)n_obs * P * c.n_kv * (hd / 8);
            vb::pages_to_rows_kernel<<<148 * 4, 256, 0, cs>>>(kp, kb, c.n_kv, e->cap, hd, P, total_vec);
            vb::pages_to_rows_kernel<<<148 * 4, 256, 0, cs>>>(vp, vbuf, c.n_kv, e->cap, hd, P, total_vec);
            VB_CUDA(cudaGetLastError());
            for (int which = 0; which < 2; ++which) {
                vb::GemmParams g{};
                g.M = M; g.N = kvf; g.K = kvf; g.epi = vb::EPI_BIAS_ACT; g.act = vb::ACT_NONE;
                g.out_bf = which ? vp : kp; g.ld_out = hd;
                g.rows_in = P; g.rows_out = 0; g.row_off = 0; g.scatter_hd = hd; g.scatter_cap = e->cap;
                if ((rc = vb::dense_gemm(which ? vbuf : kb, kvf, which ? e->wvx[l].p : e->wkx[l].p, g, cs))) return rc;
            }
        }
    }
    return VLAB200_OK;
}

}  // extern "C"
