// BitVLA language-model block on the ternary kernels: the callers either side of
// vlab200_ternary_linear, so that a whole BitNet transformer layer runs on this library.
//
// One layer of the reference (run_layer, src/kernels/bitvla/bitvla_lm_cuda.cu:395-525) is 25
// launches: rmsnorm, act-quant, three ternary GEMMs, three head-split transposes, two RoPE
// passes, two GQA repeats, cuBLAS QK^T with the score matrix in HBM, softmax, cuBLAS PV,
// merge transpose, rmsnorm, act-quant, GEMM, add, rmsnorm, act-quant, GEMM, gate*up,
// rmsnorm, act-quant, GEMM, add.  Here it is 9:
//
//   norm_quant_kernel   [residual add ->] RMSNorm (bf16 rounding as the reference) -> per-token
//                       absmax int8; one pass over the row, nothing but int8 + scale written
//   ternary GEMM        q, k, v as ONE matrix (rows concatenated at set_layer, one weight scale
//                       per 'group' rows through ws_num)
//   rope_split_kernel   NeoX RoPE on q and k, head split, K / V rows into the attention pages
//   attention           streaming tcgen05 kernel, no score matrix, no repeated K/V
//   norm_quant_kernel   attn sub-norm -> int8
//   ternary GEMM        o
//   norm_quant_kernel   h += o; ffn norm -> int8
//   ternary GEMM        gate_up
//   norm_quant_kernel   relu(gate)^2 * up -> ffn sub-norm -> int8
//   ternary GEMM        down   (its residual add is fused into the next norm_quant_kernel)
//
// Sequences of equal length can be batched (n_seq); the reference runs one per call.
#include <cuda_bf16.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <string>
#include <vector>

#include "gemm.h"
#include "host_common.h"
#include "tc5.cuh"

namespace vb {

enum { NQ_PLAIN = 0, NQ_ADD = 1, NQ_GATE_UP = 2 };

__device__ __forceinline__ float block_sum_256(float v, float *red) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    __syncthreads();  // red may still be read from the previous reduction
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = red[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) t += red[i];
    return t;
}

__device__ __forceinline__ float block_max_256(float v, float *red) {
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

// One CTA per token row.  MODE selects where the row comes from:
//   NQ_PLAIN    x = in[m][k]
//   NQ_ADD      x = bf16(in[m][k] + add[m][k]), written back to in (bitvla_add_bf16, reference
//               bitvla_lm_cuda.cu:497,522)
//   NQ_GATE_UP  x = bf16(relu(g)^2 * u), g = in[m][k], u = in[m][K + k] (row stride 2K;
//               gate_up_fused_sqrelu_mul_bf16_kernel, bitvla_lm_cuda.cu:527-542)
// then y = bf16(x * rsqrt(mean x^2 + eps) * w[k]) (rmsnorm_bf16_kernel, bitvla_lm_cuda.cu:37-75) and
// either y is stored (out_bf != nullptr) or quantised: s = 127 / max(max|y|, 1e-5),
// q = clamp(rne(y * s), -128, 127) (act_quant_kernel, src/kernels/bitvla/bitnet_kernels.h:465-521).
// The row lives in shared memory as float between the passes (K * 4 bytes).
template <int MODE>
__global__ void __launch_bounds__(256) norm_quant_kernel(__nv_bfloat16 *__restrict__ in,
                                                         const __nv_bfloat16 *__restrict__ add,
                                                         const __nv_bfloat16 *__restrict__ w, float eps, int K,
                                                         int8_t *__restrict__ q_out, float *__restrict__ s_out,
                                                         __nv_bfloat16 *__restrict__ out_bf) {
    extern __shared__ float row[];
    __shared__ float red[8];
    pdl_launch_dependents();
    pdl_wait();
    const int m = blockIdx.x, tid = threadIdx.x;
    const int K2 = K >> 1;
    const size_t ld = MODE == NQ_GATE_UP ? 2 * (size_t)K : (size_t)K;
    __nv_bfloat162 *src = reinterpret_cast<__nv_bfloat162 *>(in + m * ld);
    float ss = 0.f;
    for (int i = tid; i < K2; i += 256) {
        float2 x = __bfloat1622float2(src[i]);
        if (MODE == NQ_ADD) {
            const float2 a = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162 *>(add + m * ld)[i]);
            const __nv_bfloat162 r = __floats2bfloat162_rn(x.x + a.x, x.y + a.y);
            src[i] = r;
            x = __bfloat1622float2(r);
        } else if (MODE == NQ_GATE_UP) {
            const float2 u = __bfloat1622float2(src[K2 + i]);
            const float g0 = fmaxf(x.x, 0.f), g1 = fmaxf(x.y, 0.f);
            x = __bfloat1622float2(__floats2bfloat162_rn(g0 * g0 * u.x, g1 * g1 * u.y));
        }
        row[2 * i] = x.x;
        row[2 * i + 1] = x.y;
        ss += x.x * x.x + x.y * x.y;
    }
    ss = block_sum_256(ss, red);
    const float scale = rsqrtf(ss / (float)K + eps);
    const __nv_bfloat162 *w2 = reinterpret_cast<const __nv_bfloat162 *>(w);
    float amax = 0.f;
    for (int i = tid; i < K2; i += 256) {
        const float2 wv = __bfloat1622float2(w2[i]);
        const __nv_bfloat162 y = __floats2bfloat162_rn(row[2 * i] * scale * wv.x, row[2 * i + 1] * scale * wv.y);
        if (out_bf) reinterpret_cast<__nv_bfloat162 *>(out_bf + (size_t)m * K)[i] = y;
        const float2 yf = __bfloat1622float2(y);
        row[2 * i] = yf.x;
        row[2 * i + 1] = yf.y;
        amax = fmaxf(amax, fmaxf(fabsf(yf.x), fabsf(yf.y)));
    }
    if (out_bf) return;
    amax = block_max_256(amax, red);
    amax = amax < 1e-5f ? 1e-5f : amax;
    const float qs = __fdiv_rn(127.0f, amax);
    if (tid == 0) s_out[m] = qs;
    char2 *dst = reinterpret_cast<char2 *>(q_out + (size_t)m * K);
    for (int i = tid; i < K2; i += 256) {  // each thread re-reads the elements it wrote itself
        const float a = fminf(fmaxf(rintf(row[2 * i] * qs), -128.f), 127.f);
        const float b = fminf(fmaxf(rintf(row[2 * i + 1] * qs), -128.f), 127.f);
        dst[i] = make_char2((signed char)(int)a, (signed char)(int)b);
    }
}

// The same stage with 16-byte accesses and the row held in registers (packed bf16) between the passes: thread t
// owns the 8-element groups t, t + 256, ... (at most NV of them), so K <= 2048 * NV and K % 8 == 0.  Per element the
// arithmetic is the one of norm_quant_kernel; only the order of the float sum of squares differs.
template <int MODE, int NV>
__global__ void __launch_bounds__(256) norm_quant_vec_kernel(__nv_bfloat16 *__restrict__ in,
                                                             const __nv_bfloat16 *__restrict__ add,
                                                             const __nv_bfloat16 *__restrict__ w, float eps, int K,
                                                             int8_t *__restrict__ q_out, float *__restrict__ s_out,
                                                             __nv_bfloat16 *__restrict__ out_bf) {
    __shared__ float red[8];
    pdl_launch_dependents();
    pdl_wait();
    const int m = blockIdx.x, tid = threadIdx.x;
    const int K8 = K >> 3;
    const size_t ld = MODE == NQ_GATE_UP ? 2 * (size_t)K : (size_t)K;
    uint4 *src = reinterpret_cast<uint4 *>(in + m * ld);
    uint4 x[NV];
    float ss = 0.f;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
        const int i = tid + v * 256;
        if (i >= K8) break;
        uint4 xv = src[i];
        uint32_t *xw = reinterpret_cast<uint32_t *>(&xv);
        if (MODE == NQ_ADD) {
            const uint4 av = reinterpret_cast<const uint4 *>(add + m * ld)[i];
            const uint32_t *aw = reinterpret_cast<const uint32_t *>(&av);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&xw[e]));
                const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&aw[e]));
                const __nv_bfloat162 r = __floats2bfloat162_rn(a.x + b.x, a.y + b.y);
                xw[e] = *reinterpret_cast<const uint32_t *>(&r);
            }
            src[i] = xv;
        } else if (MODE == NQ_GATE_UP) {
            const uint4 uv = src[K8 + i];
            const uint32_t *uw = reinterpret_cast<const uint32_t *>(&uv);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&xw[e]));
                const float2 u = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&uw[e]));
                const float g0 = fmaxf(g.x, 0.f), g1 = fmaxf(g.y, 0.f);
                const __nv_bfloat162 r = __floats2bfloat162_rn(g0 * g0 * u.x, g1 * g1 * u.y);
                xw[e] = *reinterpret_cast<const uint32_t *>(&r);
            }
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&xw[e]));
            ss += f.x * f.x + f.y * f.y;
        }
        x[v] = xv;
    }
    ss = block_sum_256(ss, red);
    const float scale = rsqrtf(ss / (float)K + eps);
    float amax = 0.f;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
        const int i = tid + v * 256;
        if (i >= K8) break;
        const uint4 wv = __ldg(reinterpret_cast<const uint4 *>(w) + i);
        const uint32_t *ww = reinterpret_cast<const uint32_t *>(&wv);
        uint32_t *xw = reinterpret_cast<uint32_t *>(&x[v]);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&xw[e]));
            const float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&ww[e]));
            const __nv_bfloat162 y = __floats2bfloat162_rn(f.x * scale * g.x, f.y * scale * g.y);
            xw[e] = *reinterpret_cast<const uint32_t *>(&y);
            const float2 yf = __bfloat1622float2(y);
            amax = fmaxf(amax, fmaxf(fabsf(yf.x), fabsf(yf.y)));
        }
        if (out_bf) reinterpret_cast<uint4 *>(out_bf + (size_t)m * K)[i] = x[v];
    }
    if (out_bf) return;
    amax = block_max_256(amax, red);
    amax = amax < 1e-5f ? 1e-5f : amax;
    const float qs = __fdiv_rn(127.0f, amax);
    if (tid == 0) s_out[m] = qs;
    uint2 *dst = reinterpret_cast<uint2 *>(q_out + (size_t)m * K);
#pragma unroll
    for (int v = 0; v < NV; ++v) {
        const int i = tid + v * 256;
        if (i >= K8) break;
        const uint32_t *xw = reinterpret_cast<const uint32_t *>(&x[v]);
        uint32_t o[2] = {0u, 0u};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 yf = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&xw[e]));
            const int a = (int)fminf(fmaxf(rintf(yf.x * qs), -128.f), 127.f);
            const int b = (int)fminf(fmaxf(rintf(yf.y * qs), -128.f), 127.f);
            o[e >> 1] |= ((uint32_t)(a & 0xff) | ((uint32_t)(b & 0xff) << 8)) << (16 * (e & 1));
        }
        dst[i] = make_uint2(o[0], o[1]);
    }
}

// qkv: bf16 [M][(n_q + 2 n_kv_proj) hd] (q heads, k heads, v heads) -> q_out [n_seq][n_q][seq][hd]
// rotated, K page rows rotated, V page rows copied.  Pages: [n_seq][n_kv_store][cap][hd], token s of a
// sequence goes to page row row0 + s.  n_kv_proj == 0: only q heads are present (cross-attention).
// The rotation is computed in float on bf16 inputs and rounded once, as rope_neox_bf16_kernel
// (bitvla_lm_cuda.cu:77-99) does after the head split (bitvla_lm_cuda.cu:441-446).
__global__ void __launch_bounds__(128) rope_split_kernel(const __nv_bfloat16 *__restrict__ qkv,
                                                         const float *__restrict__ cos_t,
                                                         const float *__restrict__ sin_t,
                                                         __nv_bfloat16 *__restrict__ q_out,
                                                         __nv_bfloat16 *__restrict__ k_pages,
                                                         __nv_bfloat16 *__restrict__ v_pages, int seq, int n_q,
                                                         int n_kv_proj, int n_kv_store, int hd, int cap, int row0) {
    pdl_launch_dependents();
    pdl_wait();
    const int m = blockIdx.x;
    const int sq = m / seq, s = m % seq;
    const int half = hd >> 1;
    const int n_heads = n_q + 2 * n_kv_proj;
    const __nv_bfloat16 *src = qkv + (size_t)m * n_heads * hd;
    for (int i = threadIdx.x; i < n_heads * half; i += blockDim.x) {
        const int head = i / half, k = i % half;
        const __nv_bfloat16 *hp = src + (size_t)head * hd;
        const float a = __bfloat162float(hp[k]), b = __bfloat162float(hp[k + half]);
        __nv_bfloat16 *dst;
        float lo = a, hi = b;
        if (head < n_q + n_kv_proj) {
            const float c = cos_t[(size_t)s * half + k], sn = sin_t[(size_t)s * half + k];
            lo = a * c - b * sn;
            hi = b * c + a * sn;
            dst = head < n_q ? q_out + (((size_t)sq * n_q + head) * seq + s) * hd
                             : k_pages + (((size_t)sq * n_kv_store + (head - n_q)) * cap + row0 + s) * hd;
        } else {
            dst = v_pages + (((size_t)sq * n_kv_store + (head - n_q - n_kv_proj)) * cap + row0 + s) * hd;
        }
        dst[k] = __float2bfloat16(lo);
        dst[k + half] = __float2bfloat16(hi);
    }
}

// The same with 16-byte accesses: one work item = 8 consecutive elements of a head's first half and the matching
// 8 of its second half (hd % 16 == 0, 16-byte aligned buffers).
__global__ void __launch_bounds__(128) rope_split_vec_kernel(const __nv_bfloat16 *__restrict__ qkv,
                                                             const float *__restrict__ cos_t,
                                                             const float *__restrict__ sin_t,
                                                             __nv_bfloat16 *__restrict__ q_out,
                                                             __nv_bfloat16 *__restrict__ k_pages,
                                                             __nv_bfloat16 *__restrict__ v_pages, int seq, int n_q,
                                                             int n_kv_proj, int n_kv_store, int hd, int cap, int row0) {
    pdl_launch_dependents();
    pdl_wait();
    const int m = blockIdx.x;
    const int sq = m / seq, s = m % seq;
    const int half = hd >> 1, h8 = half >> 3;
    const int n_heads = n_q + 2 * n_kv_proj;
    const __nv_bfloat16 *src = qkv + (size_t)m * n_heads * hd;
    for (int i = threadIdx.x; i < n_heads * h8; i += blockDim.x) {
        const int head = i / h8, k = (i % h8) * 8;
        const __nv_bfloat16 *hp = src + (size_t)head * hd;
        uint4 lo = *reinterpret_cast<const uint4 *>(hp + k), hi = *reinterpret_cast<const uint4 *>(hp + k + half);
        __nv_bfloat16 *dst;
        if (head < n_q + n_kv_proj) {
            const float4 *cp = reinterpret_cast<const float4 *>(cos_t + (size_t)s * half + k);
            const float4 *sp = reinterpret_cast<const float4 *>(sin_t + (size_t)s * half + k);
            const float4 c0 = __ldg(cp), c1 = __ldg(cp + 1), s0 = __ldg(sp), s1 = __ldg(sp + 1);
            const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
            const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
            uint32_t *lw = reinterpret_cast<uint32_t *>(&lo), *hw = reinterpret_cast<uint32_t *>(&hi);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&lw[e]));
                const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&hw[e]));
                const __nv_bfloat162 l2 = __floats2bfloat162_rn(a.x * c[2 * e] - b.x * sn[2 * e],
                                                                a.y * c[2 * e + 1] - b.y * sn[2 * e + 1]);
                const __nv_bfloat162 h2 = __floats2bfloat162_rn(b.x * c[2 * e] + a.x * sn[2 * e],
                                                                b.y * c[2 * e + 1] + a.y * sn[2 * e + 1]);
                lw[e] = *reinterpret_cast<const uint32_t *>(&l2);
                hw[e] = *reinterpret_cast<const uint32_t *>(&h2);
            }
            dst = head < n_q ? q_out + (((size_t)sq * n_q + head) * seq + s) * hd
                             : k_pages + (((size_t)sq * n_kv_store + (head - n_q)) * cap + row0 + s) * hd;
        } else {
            dst = v_pages + (((size_t)sq * n_kv_store + (head - n_q - n_kv_proj)) * cap + row0 + s) * hd;
        }
        *reinterpret_cast<uint4 *>(dst + k) = lo;
        *reinterpret_cast<uint4 *>(dst + k + half) = hi;
    }
}

// Host entry for other translation units (the engine's few-row path).
int rope_split(const void *qkv, const float *cos_t, const float *sin_t, void *q_out, void *k_pages, void *v_pages,
               int M, int seq, int n_q, int n_kv_proj, int n_kv_store, int hd, int cap, int row0, cudaStream_t st) {
    auto al16 = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    if (hd % 16 == 0 && al16(qkv) && al16(cos_t) && al16(sin_t) && al16(q_out) && al16(k_pages) && al16(v_pages)) {
        return launch_pdl(rope_split_vec_kernel, dim3(M), dim3(128), 0, st, static_cast<const __nv_bfloat16 *>(qkv), cos_t, sin_t,
                          static_cast<__nv_bfloat16 *>(q_out), static_cast<__nv_bfloat16 *>(k_pages),
                          static_cast<__nv_bfloat16 *>(v_pages), seq, n_q, n_kv_proj, n_kv_store, hd, cap, row0);
    }
    return launch_pdl(rope_split_kernel, dim3(M), dim3(128), 0, st, static_cast<const __nv_bfloat16 *>(qkv), cos_t, sin_t,
                      static_cast<__nv_bfloat16 *>(q_out), static_cast<__nv_bfloat16 *>(k_pages),
                      static_cast<__nv_bfloat16 *>(v_pages), seq, n_q, n_kv_proj, n_kv_store, hd, cap, row0);
}

static int gcd_int(int a, int b) {
    while (b) {
        const int t = a % b;
        a = b;
        b = t;
    }
    return a;
}

struct LmLayer {
    vlab200_bitvla_lm_layer w{};
    DevBuf qkv_packed, qkv_ws;
    bool set = false;
};

}  // namespace vb

struct vlab200_bitvla_lm {
    int hidden, n_q, n_kv, hd, ffn, n_layers, max_seq, max_batch, hq, hkv, qkv_group, qkv_ws_num;
    float rope_base, eps;
    const void *output_norm = nullptr;
    std::vector<vb::LmLayer> layers;
    vb::DevBuf cos_t, sin_t, h, a8, s, qkv, q, k_pages, v_pages, att, proj, gate_up;
    std::vector<vb::DevBuf> owned;  // weights uploaded by vlab200_bitvla_lm_create_from_gguf
};

using vb::DevBuf;

extern "C" {

vlab200_bitvla_lm *vlab200_bitvla_lm_init(int32_t hidden, int32_t n_q, int32_t n_kv, int32_t head_dim, int32_t ffn,
                                          int32_t n_layers, float rope_base, float rms_eps, int32_t max_seq,
                                          int32_t max_batch) {
    if (hidden <= 0 || n_q <= 0 || n_kv <= 0 || n_q % n_kv || ffn <= 0 || n_layers <= 0 || max_seq <= 0 ||
        max_batch <= 0 || (head_dim != 64 && head_dim != 128 && head_dim != 256)) {
        vb::set_last_error("vlab200_bitvla_lm_init: bad dimensions");
        return nullptr;
    }
    const int hq = n_q * head_dim, hkv = n_kv * head_dim;
    if (hidden % 128 || hq % 128 || ffn % 128 || hkv % 32) {
        vb::set_last_error("vlab200_bitvla_lm_init: hidden, n_q*head_dim and ffn must be multiples of 128 (K of the "
                           "ladder pack), n_kv*head_dim of 32");
        return nullptr;
    }
    auto *c = new (std::nothrow) vlab200_bitvla_lm();
    if (!c) return nullptr;
    c->hidden = hidden; c->n_q = n_q; c->n_kv = n_kv; c->hd = head_dim; c->ffn = ffn; c->n_layers = n_layers;
    c->max_seq = max_seq; c->max_batch = max_batch; c->hq = hq; c->hkv = hkv;
    c->rope_base = rope_base; c->eps = rms_eps;
    c->qkv_group = vb::gcd_int(hq, hkv);
    c->qkv_ws_num = (hq + 2 * hkv) / c->qkv_group;
    c->layers.resize(n_layers);
    const size_t rows = (size_t)max_seq * max_batch;
    size_t kmax = (size_t)hidden;
    if ((size_t)ffn > kmax) kmax = ffn;
    if ((size_t)hq > kmax) kmax = hq;
    const int64_t page_bytes = vlab200_kv_store_bytes(1, max_batch, n_kv, head_dim, max_seq);
    int rc = c->cos_t.alloc((size_t)max_seq * head_dim / 2 * 4);
    if (!rc) rc = c->sin_t.alloc((size_t)max_seq * head_dim / 2 * 4);
    if (!rc) rc = c->h.alloc(rows * hidden * 2);
    if (!rc) rc = c->a8.alloc(rows * kmax);
    if (!rc) rc = c->s.alloc(rows * 4);
    if (!rc) rc = c->qkv.alloc(rows * (hq + 2 * hkv) * 2);
    if (!rc) rc = c->q.alloc(rows * hq * 2);
    if (!rc) rc = c->k_pages.alloc((size_t)page_bytes);
    if (!rc) rc = c->v_pages.alloc((size_t)page_bytes);
    if (!rc) rc = c->att.alloc(rows * hq * 2);
    if (!rc) rc = c->proj.alloc(rows * hidden * 2);
    if (!rc) rc = c->gate_up.alloc(rows * 2 * ffn * 2);
    // same table as the reference's host loop (bitvla_lm_cuda.cu:333-342), positions 0 .. max_seq-1
    if (!rc) rc = vlab200_rope_table(c->cos_t.as<float>(), c->sin_t.as<float>(), 0, max_seq, head_dim, rope_base, nullptr);
    if (!rc && cudaStreamSynchronize(nullptr) != cudaSuccess) rc = VLAB200_ERR_CUDA;
    if (rc) {
        delete c;
        return nullptr;
    }
    return c;
}

void vlab200_bitvla_lm_free(vlab200_bitvla_lm *ctx) { delete ctx; }

int32_t vlab200_bitvla_lm_set_layer(vlab200_bitvla_lm *ctx, int32_t L, const vlab200_bitvla_lm_layer *layer) {
    if (!ctx || !layer || L < 0 || L >= ctx->n_layers) return VLAB200_ERR_ARG;
    const vlab200_bitvla_lm_layer &w = *layer;
    if (!w.attn_norm_w || !w.attn_sub_norm_w || !w.ffn_norm_w || !w.ffn_sub_norm_w || !w.q_packed || !w.q_ws ||
        !w.k_packed || !w.k_ws || !w.v_packed || !w.v_ws || !w.o_packed || !w.o_ws || !w.gate_up_packed ||
        !w.gate_up_ws || !w.down_packed || !w.down_ws) {
        vb::set_last_error("vlab200_bitvla_lm_set_layer: null weight pointer");
        return VLAB200_ERR_ARG;
    }
    vb::LmLayer &l = ctx->layers[L];
    l.w = w;
    // q, k, v rows back to back: a ladder pack is a sequence of independent 16-row runs, so the
    // packed matrices concatenate byte-wise; their scales are repeated once per 'group' rows.
    const size_t qb = (size_t)ctx->hq * ctx->hidden / 4, kb = (size_t)ctx->hkv * ctx->hidden / 4;
    if (!l.qkv_packed.p) {
        int rc = l.qkv_packed.alloc(qb + 2 * kb);
        if (!rc) rc = l.qkv_ws.alloc((size_t)ctx->qkv_ws_num * 4);
        if (rc) return rc;
    }
    uint8_t *dst = l.qkv_packed.as<uint8_t>();
    VB_CUDA(cudaMemcpy(dst, w.q_packed, qb, cudaMemcpyDeviceToDevice));
    VB_CUDA(cudaMemcpy(dst + qb, w.k_packed, kb, cudaMemcpyDeviceToDevice));
    VB_CUDA(cudaMemcpy(dst + qb + kb, w.v_packed, kb, cudaMemcpyDeviceToDevice));
    float sc[3];
    VB_CUDA(cudaMemcpy(&sc[0], w.q_ws, 4, cudaMemcpyDeviceToHost));
    VB_CUDA(cudaMemcpy(&sc[1], w.k_ws, 4, cudaMemcpyDeviceToHost));
    VB_CUDA(cudaMemcpy(&sc[2], w.v_ws, 4, cudaMemcpyDeviceToHost));
    std::vector<float> ws(ctx->qkv_ws_num);
    const int nq_groups = ctx->hq / ctx->qkv_group, nk_groups = ctx->hkv / ctx->qkv_group;
    for (int i = 0; i < ctx->qkv_ws_num; ++i) ws[i] = i < nq_groups ? sc[0] : (i < nq_groups + nk_groups ? sc[1] : sc[2]);
    VB_CUDA(cudaMemcpy(l.qkv_ws.p, ws.data(), ws.size() * 4, cudaMemcpyHostToDevice));
    l.set = true;
    return VLAB200_OK;
}

int32_t vlab200_bitvla_lm_set_output_norm(vlab200_bitvla_lm *ctx, const void *w_bf16) {
    if (!ctx || !w_bf16) return VLAB200_ERR_ARG;
    ctx->output_norm = w_bf16;
    return VLAB200_OK;
}

}  // extern "C"

namespace vb {

template <int MODE>
static int launch_norm_quant(void *in, const void *add, const void *w, float eps, int M, int K, int8_t *q, float *s,
                             void *out_bf, cudaStream_t st) {
    auto al16 = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    __nv_bfloat16 *in_b = static_cast<__nv_bfloat16 *>(in);
    const __nv_bfloat16 *add_b = static_cast<const __nv_bfloat16 *>(add), *w_b = static_cast<const __nv_bfloat16 *>(w);
    __nv_bfloat16 *out_b = static_cast<__nv_bfloat16 *>(out_bf);
    if (K % 8 == 0 && K <= 8192 && al16(in) && al16(add) && al16(w) && al16(out_bf) && (reinterpret_cast<uintptr_t>(q) & 7) == 0) {
        if (K <= 4096) return launch_pdl(norm_quant_vec_kernel<MODE, 2>, dim3(M), dim3(256), 0, st, in_b, add_b, w_b, eps, K, q, s, out_b);
        return launch_pdl(norm_quant_vec_kernel<MODE, 4>, dim3(M), dim3(256), 0, st, in_b, add_b, w_b, eps, K, q, s, out_b);
    }
    const size_t smem = (size_t)K * 4;
    if (smem > 48 * 1024)
        if (int rc = ensure_dyn_smem(norm_quant_kernel<MODE>, 200 * 1024)) return rc;
    return launch_pdl(norm_quant_kernel<MODE>, dim3(M), dim3(256), smem, st, in_b, add_b, w_b, eps, K, q, s, out_b);
}

}  // namespace vb

extern "C" int32_t vlab200_bitvla_norm_quant(void *x_bf16, const void *add_bf16, const void *w_bf16, float eps,
                                             int32_t M, int32_t K, int32_t mode, int8_t *q, float *scales,
                                             void *y_bf16, void *stream) {
    if (!x_bf16 || !w_bf16 || M < 0 || K <= 0 || K % 2 || (mode == vb::NQ_ADD && !add_bf16) ||
        (!y_bf16 && (!q || !scales)))
        return VLAB200_ERR_ARG;
    if ((size_t)K * 4 > 200 * 1024) {
        vb::set_last_error("vlab200_bitvla_norm_quant: K=%d exceeds the %d floats a row may hold in shared memory", K,
                           200 * 1024 / 4);
        return VLAB200_ERR_UNSUPPORTED;
    }
    if (M == 0) return VLAB200_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (mode) {
        case vb::NQ_PLAIN: return vb::launch_norm_quant<vb::NQ_PLAIN>(x_bf16, nullptr, w_bf16, eps, M, K, q, scales, y_bf16, st);
        case vb::NQ_ADD: return vb::launch_norm_quant<vb::NQ_ADD>(x_bf16, add_bf16, w_bf16, eps, M, K, q, scales, y_bf16, st);
        case vb::NQ_GATE_UP: return vb::launch_norm_quant<vb::NQ_GATE_UP>(x_bf16, nullptr, w_bf16, eps, M, K, q, scales, y_bf16, st);
        default: return VLAB200_ERR_ARG;
    }
}

namespace vb {

// Writes device bf16 tensors as float32 files <dir>/<name>.bin (layer-0 stage dump, debugging only).
struct L0Dump {
    const char *dir;
    cudaStream_t st;
    DevBuf tmp;
    L0Dump(const char *d, cudaStream_t s, size_t tmp_elems) : dir(d && *d ? d : nullptr), st(s) {
        if (dir && tmp.alloc(tmp_elems * 2) != VLAB200_OK) dir = nullptr;
    }
    bool on() const { return dir != nullptr; }
    std::vector<float> fetch(const void *dev, size_t n) {
        std::vector<uint16_t> raw(n);
        std::vector<float> f(n);
        cudaStreamSynchronize(st);
        cudaMemcpy(raw.data(), dev, n * 2, cudaMemcpyDeviceToHost);
        for (size_t i = 0; i < n; ++i) {
            const uint32_t b = (uint32_t)raw[i] << 16;
            std::memcpy(&f[i], &b, 4);
        }
        return f;
    }
    void put(const char *name, const std::vector<float> &f) {
        const std::string path = std::string(dir) + "/" + name + ".bin";
        if (FILE *fp = std::fopen(path.c_str(), "wb")) {
            std::fwrite(f.data(), sizeof(float), f.size(), fp);
            std::fclose(fp);
        }
    }
    void write(const char *name, const void *dev, size_t n) { put(name, fetch(dev, n)); }
    // the fused projection holds q | k | v per token; the reference's file holds the q, k and v matrices one after another
    void write_qkv(const char *name, const void *dev, int M, int hq, int hkv) {
        const int row = hq + 2 * hkv;
        const std::vector<float> f = fetch(dev, (size_t)M * row);
        std::vector<float> out(f.size());
        float *q = out.data(), *k = q + (size_t)M * hq, *v = k + (size_t)M * hkv;
        for (int m = 0; m < M; ++m) {
            std::memcpy(q + (size_t)m * hq, &f[(size_t)m * row], (size_t)hq * 4);
            std::memcpy(k + (size_t)m * hkv, &f[(size_t)m * row + hq], (size_t)hkv * 4);
            std::memcpy(v + (size_t)m * hkv, &f[(size_t)m * row + hq + hkv], (size_t)hkv * 4);
        }
        put(name, out);
    }
    void write_sum(const char *name, const void *a, const void *b, size_t n) {
        std::vector<float> x = fetch(a, n);
        const std::vector<float> y = fetch(b, n);
        for (size_t i = 0; i < n; ++i) x[i] = __bfloat162float(__float2bfloat16_rn(x[i] + y[i]));
        put(name, x);
    }
};

}  // namespace vb

extern "C" int32_t vlab200_bitvla_lm_forward(vlab200_bitvla_lm *ctx, const void *d_in, void *d_out, int32_t seq,
                                             int32_t n_seq, void *stream) {
    if (!ctx || !d_in || !d_out) return VLAB200_ERR_ARG;
    if (seq <= 0 || n_seq <= 0 || seq > ctx->max_seq || n_seq > ctx->max_batch) {
        vb::set_last_error("vlab200_bitvla_lm_forward: seq=%d n_seq=%d outside max_seq=%d max_batch=%d", seq, n_seq,
                           ctx->max_seq, ctx->max_batch);
        return VLAB200_ERR_ARG;
    }
    if (!ctx->output_norm) {
        vb::set_last_error("vlab200_bitvla_lm_forward: output norm not set");
        return VLAB200_ERR_ARG;
    }
    for (const vb::LmLayer &l : ctx->layers)
        if (!l.set) {
            vb::set_last_error("vlab200_bitvla_lm_forward: a layer was not set");
            return VLAB200_ERR_ARG;
        }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int M = seq * n_seq, H = ctx->hidden, hq = ctx->hq, hkv = ctx->hkv, F = ctx->ffn;
    int8_t *a8 = ctx->a8.as<int8_t>();
    float *s = ctx->s.as<float>();
    VB_CUDA(cudaMemcpyAsync(ctx->h.p, d_in, (size_t)M * H * 2, cudaMemcpyDeviceToDevice, st));
    const vlab200_kv_store store = {ctx->k_pages.p, ctx->v_pages.p, 1, n_seq, ctx->n_kv, ctx->hd, ctx->max_seq, 0};
    int rc = VLAB200_OK;
    // Stage dump of layer 0, switched on like the reference's (VLA_BITVLA_DUMP_L0=<dir>, one sequence): the same ten
    // float32 files under the same names (src/kernels/bitvla/bitvla_lm_cuda.cu:400-420 and the l0_dump calls up to
    // :523), so the two stacks can be compared stage by stage.  A debugging path: it synchronises, allocates and
    // runs the normalisations a second time without their fused quantisation.
    vb::L0Dump dump(n_seq == 1 ? std::getenv("VLA_BITVLA_DUMP_L0") : nullptr, st, (size_t)M * (size_t)(F > hq ? (F > H ? F : H) : (hq > H ? hq : H)));
    for (int L = 0; L < ctx->n_layers && !rc; ++L) {
        const vb::LmLayer &l = ctx->layers[L];
        const bool dl = dump.on() && L == 0;
        if (dl) {
            vb::launch_norm_quant<vb::NQ_PLAIN>(ctx->h.p, nullptr, l.w.attn_norm_w, ctx->eps, M, H, nullptr, nullptr, dump.tmp.p, st);
            dump.write("L0_01_attn_norm", dump.tmp.p, (size_t)M * H);
        }
        if (L == 0) rc = vb::launch_norm_quant<vb::NQ_PLAIN>(ctx->h.p, nullptr, l.w.attn_norm_w, ctx->eps, M, H, a8, s, nullptr, st);
        else rc = vb::launch_norm_quant<vb::NQ_ADD>(ctx->h.p, ctx->proj.p, l.w.attn_norm_w, ctx->eps, M, H, a8, s, nullptr, st);
        if (rc) break;
        rc = vlab200_ternary_linear(a8, l.qkv_packed.as<uint8_t>(), ctx->qkv.p, nullptr, s, l.qkv_ws.as<float>(),
                                    ctx->qkv_ws_num, M, hq + 2 * hkv, H, 0, st);
        if (rc) break;
        if (dl) dump.write_qkv("L0_02_qkv_proj", ctx->qkv.p, M, hq, hkv);
        rc = vb::rope_split(ctx->qkv.p, ctx->cos_t.as<float>(), ctx->sin_t.as<float>(), ctx->q.p, ctx->k_pages.p,
                            ctx->v_pages.p, M, seq, ctx->n_q, ctx->n_kv, ctx->n_kv, ctx->hd, ctx->max_seq, 0, st);
        if (rc) break;
        rc = vlab200_attention(&store, 0, ctx->q.p, ctx->att.p, seq, ctx->n_q, seq, /*mask_mode=*/0, nullptr, st);
        if (rc) break;
        if (dl) {
            dump.write("L0_03_attn_merged_pre_subnorm", ctx->att.p, (size_t)M * hq);
            vb::launch_norm_quant<vb::NQ_PLAIN>(ctx->att.p, nullptr, l.w.attn_sub_norm_w, ctx->eps, M, hq, nullptr, nullptr, dump.tmp.p, st);
            dump.write("L0_04_attn_sub_norm", dump.tmp.p, (size_t)M * hq);
        }
        rc = vb::launch_norm_quant<vb::NQ_PLAIN>(ctx->att.p, nullptr, l.w.attn_sub_norm_w, ctx->eps, M, hq, a8, s, nullptr, st);
        if (rc) break;
        rc = vlab200_ternary_linear(a8, static_cast<const uint8_t *>(l.w.o_packed), ctx->proj.p, nullptr, s,
                                    static_cast<const float *>(l.w.o_ws), 1, M, H, hq, 0, st);
        if (rc) break;
        if (dl) dump.write("L0_05_o_proj_out", ctx->proj.p, (size_t)M * H);
        rc = vb::launch_norm_quant<vb::NQ_ADD>(ctx->h.p, ctx->proj.p, l.w.ffn_norm_w, ctx->eps, M, H, a8, s, nullptr, st);
        if (rc) break;
        if (dl) {
            dump.write("L0_06_after_attn_residual", ctx->h.p, (size_t)M * H);
            vb::launch_norm_quant<vb::NQ_PLAIN>(ctx->h.p, nullptr, l.w.ffn_norm_w, ctx->eps, M, H, nullptr, nullptr, dump.tmp.p, st);
            dump.write("L0_07_ffn_norm", dump.tmp.p, (size_t)M * H);
        }
        rc = vlab200_ternary_linear(a8, static_cast<const uint8_t *>(l.w.gate_up_packed), ctx->gate_up.p, nullptr, s,
                                    static_cast<const float *>(l.w.gate_up_ws), 2, M, 2 * F, H, 0, st);
        if (rc) break;
        if (dl) {
            vb::launch_norm_quant<vb::NQ_GATE_UP>(ctx->gate_up.p, nullptr, l.w.ffn_sub_norm_w, ctx->eps, M, F, nullptr, nullptr, dump.tmp.p, st);
            dump.write("L0_08_ffn_sub_norm", dump.tmp.p, (size_t)M * F);
        }
        rc = vb::launch_norm_quant<vb::NQ_GATE_UP>(ctx->gate_up.p, nullptr, l.w.ffn_sub_norm_w, ctx->eps, M, F, a8, s, nullptr, st);
        if (rc) break;
        rc = vlab200_ternary_linear(a8, static_cast<const uint8_t *>(l.w.down_packed), ctx->proj.p, nullptr, s,
                                    static_cast<const float *>(l.w.down_ws), 1, M, H, F, 0, st);
        if (dl && !rc) {
            dump.write("L0_09_down_out", ctx->proj.p, (size_t)M * H);
            dump.write_sum("L0_10_final", ctx->h.p, ctx->proj.p, (size_t)M * H);  // the residual add is fused into the next stage
        }
    }
    if (rc) return rc;
    // h += down of the last layer, then the output norm (bitvla_lm_cuda.cu:718)
    return vb::launch_norm_quant<vb::NQ_ADD>(ctx->h.p, ctx->proj.p, ctx->output_norm, ctx->eps, M, H, nullptr, nullptr,
                                             d_out, st);
}

// The reference's own names and signatures for the context API (src/kernels/bitvla/bitvla_lm_cuda.h:247-286),
// so that src/models/bitvla.cpp (call sites :760-821,1326-1334) links against this library unchanged.
// One sequence per call (max_batch = n_seq = 1), as the reference runs it; bitvla_lm_layer_cuda has the
// field order of vlab200_bitvla_lm_layer, so the struct pointer passes through.
extern "C" {

bitvla_lm_cuda_ctx *bitvla_lm_cuda_init(int hidden, int n_q, int n_kv, int head_dim, int ffn, int n_layers,
                                        float rope_base, float rms_eps, int max_seq) {
    vlab200_bitvla_lm *c = vlab200_bitvla_lm_init(hidden, n_q, n_kv, head_dim, ffn, n_layers, rope_base, rms_eps,
                                                  max_seq, 1);
    if (!c) std::fprintf(stderr, "vla(bitvla_lm_cuda): %s\n", vlab200_last_error());
    return reinterpret_cast<bitvla_lm_cuda_ctx *>(c);
}

void bitvla_lm_cuda_free(bitvla_lm_cuda_ctx *ctx) { vlab200_bitvla_lm_free(reinterpret_cast<vlab200_bitvla_lm *>(ctx)); }

void bitvla_lm_cuda_set_layer(bitvla_lm_cuda_ctx *ctx, int L, const bitvla_lm_layer_cuda *layer) {
    if (vlab200_bitvla_lm_set_layer(reinterpret_cast<vlab200_bitvla_lm *>(ctx), L, layer) != VLAB200_OK)
        std::fprintf(stderr, "vla(bitvla_lm_cuda): set_layer %d failed: %s\n", L, vlab200_last_error());
}

void bitvla_lm_cuda_set_output_norm(bitvla_lm_cuda_ctx *ctx, const void *w) {
    vlab200_bitvla_lm_set_output_norm(reinterpret_cast<vlab200_bitvla_lm *>(ctx), w);
}

int bitvla_lm_cuda_forward(bitvla_lm_cuda_ctx *ctx, const void *d_in, void *d_out, int seq, void *stream) {
    const int rc = vlab200_bitvla_lm_forward(reinterpret_cast<vlab200_bitvla_lm *>(ctx), d_in, d_out, seq, 1, stream);
    if (rc != VLAB200_OK) std::fprintf(stderr, "vla(bitvla_lm_cuda): forward failed (%d): %s\n", rc, vlab200_last_error());
    return rc == VLAB200_OK ? 0 : -1;
}

}  // extern "C"

// The LM stack of a BitVLA checkpoint: metadata "bitvla.lm.*" (src/models/bitvla.cpp:360-364), per layer four
// float32 norm vectors (uploaded as bf16, bitvla.cpp:768-771) and six ladder-int2 tensors "<base>.weight" (I8,
// N*K/4 bytes) with their "<base>.scale" float32 sidecars (scripts/convert_bitvla_to_gguf.py:165-178;
// bitvla.cpp:739-753 fails the load when a sidecar is missing, and so does this).
extern "C" vlab200_bitvla_lm *vlab200_bitvla_lm_create_from_gguf(const vlab200_gguf *g, int32_t max_seq,
                                                                 int32_t max_batch) {
    if (!g) return vb::set_last_error("gguf: null handle"), nullptr;
    uint32_t hidden, n_layers, n_q, n_kv, hd, ffn;
    const struct { const char *key; uint32_t *dst; } u32s[] = {
        {"bitvla.lm.hidden", &hidden}, {"bitvla.lm.layers", &n_layers}, {"bitvla.lm.q_heads", &n_q},
        {"bitvla.lm.kv_heads", &n_kv}, {"bitvla.lm.head_dim", &hd}, {"bitvla.lm.inter", &ffn}};
    for (const auto &e : u32s)
        if (vlab200_gguf_meta_u32(g, e.key, e.dst) != VLAB200_OK)
            return vb::set_last_error("gguf: missing u32 metadata %s", e.key), nullptr;
    double rope = 500000.0, eps = 1e-5;
    if (vlab200_gguf_meta_f64(g, "bitvla.lm.rope_theta", &rope) != VLAB200_OK ||
        vlab200_gguf_meta_f64(g, "bitvla.lm.rms_eps", &eps) != VLAB200_OK)
        return vb::set_last_error("gguf: missing bitvla.lm.rope_theta / bitvla.lm.rms_eps"), nullptr;
    vlab200_bitvla_lm *c = vlab200_bitvla_lm_init((int)hidden, (int)n_q, (int)n_kv, (int)hd, (int)ffn, (int)n_layers,
                                                  (float)rope, (float)eps, max_seq, max_batch);
    if (!c) return nullptr;
    bool ok = true;
    std::vector<float> tmp;
    std::vector<uint16_t> tmp16;
    auto upload = [&](const void *src, size_t bytes) -> const void * {
        c->owned.emplace_back();
        vb::DevBuf &b = c->owned.back();
        if (b.alloc(bytes) != VLAB200_OK) return ok = false, nullptr;
        if (cudaMemcpy(b.p, src, bytes, cudaMemcpyHostToDevice) != cudaSuccess)
            return vb::cuda_fail(cudaGetLastError(), "cudaMemcpy (gguf upload)"), ok = false, nullptr;
        return b.p;
    };
    auto norm = [&](const std::string &name, int64_t n) -> const void * {  // float32 vector -> bf16 on the device
        if (!ok) return nullptr;
        tmp.resize((size_t)n);
        if (vlab200_gguf_read_f32(g, name.c_str(), tmp.data(), n, 0) != VLAB200_OK) return ok = false, nullptr;
        tmp16.resize((size_t)n);
        for (int64_t i = 0; i < n; ++i) {
            const __nv_bfloat16 h = __float2bfloat16_rn(tmp[(size_t)i]);
            std::memcpy(&tmp16[(size_t)i], &h, 2);
        }
        return upload(tmp16.data(), (size_t)n * 2);
    };
    // ladder pack of an [N][K] matrix and its n_scales sidecar entries
    auto bit = [&](const std::string &base, int64_t N, int64_t K, int n_scales, const void **packed, const float **ws) {
        if (!ok) return;
        const std::string wn = base + ".weight", sn = base + ".scale";
        int32_t type = 0, nd = 0;
        int64_t dims[4];
        uint64_t nb = 0;
        if (vlab200_gguf_tensor_info(g, wn.c_str(), &type, &nd, dims, &nb) != VLAB200_OK) {
            vb::set_last_error("gguf: missing tensor %s", wn.c_str());
            ok = false;
            return;
        }
        if (type != 24 || nb != (uint64_t)(N * K / 4)) {
            vb::set_last_error("gguf: %s is type %d with %llu bytes, expected I8 with %lld (ladder int2 of %lld x %lld)",
                               wn.c_str(), type, (unsigned long long)nb, (long long)(N * K / 4), (long long)N, (long long)K);
            ok = false;
            return;
        }
        tmp.resize((size_t)n_scales);
        if (vlab200_gguf_read_f32(g, sn.c_str(), tmp.data(), n_scales, 0) != VLAB200_OK) {
            vb::set_last_error("gguf: int2 tensor %s has no %s sidecar with %d entries", wn.c_str(), sn.c_str(), n_scales);
            ok = false;
            return;
        }
        *ws = static_cast<const float *>(upload(tmp.data(), (size_t)n_scales * 4));
        if (ok) *packed = upload(vlab200_gguf_tensor_data(g, wn.c_str()), (size_t)nb);
    };
    // A checkpoint written without "bitvla.quant.int2_packed" holds float matrices: they are ternarised and
    // ladder-packed here, on the device, as the reference's load_bit / pack_and_upload_fused do on the host
    // (src/models/bitvla.cpp:515-543,755-757,808-815).  `parts` are the row blocks of a fused projection.
    uint32_t packed_flag = 0;
    const bool packed_file = vlab200_gguf_meta_u32(g, "bitvla.quant.int2_packed", &packed_flag) == VLAB200_OK && packed_flag != 0;
    vb::DevBuf stage_w, stage_acc;
    auto bit_float = [&](const std::vector<std::string> &parts, int64_t N_each, int64_t K, const void **packed,
                         const float **ws) {
        if (!ok) return;
        const size_t n_parts = parts.size();
        c->owned.emplace_back();
        vb::DevBuf &pk = c->owned.back();
        c->owned.emplace_back();
        vb::DevBuf &sc = c->owned.back();
        if (pk.alloc((size_t)(N_each * K / 4) * n_parts) != VLAB200_OK || sc.alloc(n_parts * 4) != VLAB200_OK ||
            (!stage_acc.p && stage_acc.alloc(8) != VLAB200_OK)) {
            ok = false;
            return;
        }
        for (size_t i = 0; ok && i < n_parts; ++i) {
            const std::string wn = parts[i] + ".weight";
            tmp.resize((size_t)(N_each * K));
            if (vlab200_gguf_read_f32(g, wn.c_str(), tmp.data(), N_each * K, 0) != VLAB200_OK) {
                vb::set_last_error("gguf: %s is missing or is not a %lld x %lld float tensor", wn.c_str(), (long long)N_each,
                                   (long long)K);
                ok = false;
                return;
            }
            vb::DevBuf w_dev;
            if (w_dev.alloc(tmp.size() * 4) != VLAB200_OK ||
                cudaMemcpy(w_dev.p, tmp.data(), tmp.size() * 4, cudaMemcpyHostToDevice) != cudaSuccess ||
                vlab200_ternarize_pack(w_dev.as<float>(), N_each, K, pk.as<uint8_t>() + (size_t)i * (size_t)(N_each * K / 4),
                                       sc.as<float>() + i, stage_acc.as<double>(), nullptr) != VLAB200_OK ||
                cudaStreamSynchronize(nullptr) != cudaSuccess) {
                vb::cuda_fail(cudaGetLastError(), "ternarise + pack at load");
                ok = false;
                return;
            }
        }
        *packed = pk.p;
        *ws = sc.as<float>();
    };
    const int64_t hq = (int64_t)n_q * hd, hkv = (int64_t)n_kv * hd;
    for (uint32_t l = 0; ok && l < n_layers; ++l) {
        const std::string b = "lm.blk." + std::to_string(l) + ".";
        vlab200_bitvla_lm_layer ly{};
        ly.attn_norm_w = norm(b + "attn_norm.weight", hidden);
        ly.attn_sub_norm_w = norm(b + "attn_sub_norm.weight", hidden);
        ly.ffn_norm_w = norm(b + "ffn_norm.weight", hidden);
        ly.ffn_sub_norm_w = norm(b + "ffn_sub_norm.weight", ffn);
        if (packed_file) {
            bit(b + "attn_q", hq, hidden, 1, &ly.q_packed, &ly.q_ws);
            bit(b + "attn_k", hkv, hidden, 1, &ly.k_packed, &ly.k_ws);
            bit(b + "attn_v", hkv, hidden, 1, &ly.v_packed, &ly.v_ws);
            bit(b + "attn_o", hidden, hq, 1, &ly.o_packed, &ly.o_ws);
            bit(b + "ffn_gate_up", 2 * (int64_t)ffn, hidden, 2, &ly.gate_up_packed, &ly.gate_up_ws);
            bit(b + "ffn_down", hidden, ffn, 1, &ly.down_packed, &ly.down_ws);
        } else {
            bit_float({b + "attn_q"}, hq, hidden, &ly.q_packed, &ly.q_ws);
            bit_float({b + "attn_k"}, hkv, hidden, &ly.k_packed, &ly.k_ws);
            bit_float({b + "attn_v"}, hkv, hidden, &ly.v_packed, &ly.v_ws);
            bit_float({b + "attn_o"}, hidden, hq, &ly.o_packed, &ly.o_ws);
            bit_float({b + "ffn_gate", b + "ffn_up"}, ffn, hidden, &ly.gate_up_packed, &ly.gate_up_ws);
            bit_float({b + "ffn_down"}, hidden, ffn, &ly.down_packed, &ly.down_ws);
        }
        if (ok && vlab200_bitvla_lm_set_layer(c, (int)l, &ly) != VLAB200_OK) ok = false;
    }
    if (ok) {
        const void *on = norm("lm.output_norm.weight", hidden);
        if (ok) vlab200_bitvla_lm_set_output_norm(c, on);
    }
    if (!ok || cudaDeviceSynchronize() != cudaSuccess) {
        vlab200_bitvla_lm_free(c);
        return nullptr;
    }
    return c;
}
