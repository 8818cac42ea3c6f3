// Persistent tcgen05 GEMM with fused prologue statistics and epilogues for the rest of the
// expert layer (O-projection + residual, gated MLP, suffix-embedding MLPs):
//
//   C[m][n] = sum_k A[m][k] * W[n][k]      A: bf16 [M][K], W: bf16 [N][K] (PyTorch [out][in])
//
// Structure (same as the QKV kernel): one CTA per SM walks 128 x 256 output tiles; warp 0 loads
// both operands by TMA (SWIZZLE_128B) into a 4-stage ring, warp 1 issues tcgen05.mma kind::f16
// into a double-buffered f32 accumulator in TMEM, warps 6-9 optionally accumulate sum(a^2) per
// row from the A tiles in shared memory (RMSNorm whose weight was folded into W), and eight
// epilogue warps (two per TMEM lane quarter) drain the accumulator.
//
// Epilogues
//   RESIDUAL  h[m][n] += C (* colscale[n]) (+ bias[n])   (f32 master copy) and hb = bf16(h)   -- Wo, Wdown
//   GATED     g[m][i] = act(r C[m][2i]) * (r C[m][2i+1]),  r = rsqrt(mean a^2 + eps) -- Wgate/Wup
//             (gate and up rows interleaved in W; act = SiLU or tanh-GELU)
//   BIAS_ACT  y[m'][n] = act(C + bias[n]); bf16 and/or f32 output; rows may be re-mapped
//             (m -> (m / rows_in) * rows_out + row_off + m % rows_in) so that the action-token
//             rows land behind the state token of each observation                   -- W_at1, W_at2
//
// Reference: src/models/pi0.cpp:224-248, src/models/smolvla.cpp:843-848,1397-1403 (one mul_mat /
// add / mul / unary ggml node each; src/cuda/vla_cuda_bf16.cu:624-678 for the cuBLAS GEMM node).
#include <cuda_bf16.h>

#include <cstdlib>

#include <atomic>

#include "gemm.h"
#include "host_common.h"
#include "tc5.cuh"

namespace vb {

constexpr int G_BM = 128, G_BK = 64, G_THREADS = 448;
constexpr int G_A_BYTES = G_BM * 128;
// BN = 256 minimises operand traffic per flop; BN = 128 doubles the number of tiles when the
// problem has too few of them to occupy the SMs.
// PAIR: two CTAs (a cluster) share one 256 x 256 tile through tcgen05 cta_group::2 -- each loads its
// own 128 activation rows and only HALF of the weight tile, which halves the shared-memory bytes
// written and read per flop (a lone CTA moves 96 KB through shared memory per 512 tensor cycles,
// more than the 128 B/clk the SM has).
template <int BN, bool PAIR>
struct GemmCfg {
    static constexpr int STAGES = PAIR ? 6 : (BN == 256 ? 4 : (BN == 128 ? 6 : 8));
    static constexpr int B_ROWS = PAIR ? BN / 2 : BN;  // weight rows this CTA stages
    static constexpr int B_BYTES = B_ROWS * 128;
    static constexpr int STAGE_BYTES = G_A_BYTES + B_BYTES;
    static constexpr int SMEM = STAGES * STAGE_BYTES + 256 + 1024 + 1024;  // + barriers, statistics, alignment
};

// Both activations are x * sigmoid(.): SiLU(x) = x / (1 + e^-x) and, since 1 + tanh(u) = 2 / (1 + e^-2u),
// tanh-GELU(x) = 0.5 x (1 + tanh(u)) = x / (1 + e^-2u) with u = k0 x (1 + k1 x^2) (constants of
// src/cuda/vla_cuda_bf16.cu:470-474).  One ex2 and one reciprocal each (relative error ~1e-6) keep the
// epilogue off the critical path; tanhf and an IEEE division cost several times the issue slots.
template <int ACT>
__device__ __forceinline__ float act_t(float x) {
    if (ACT == ACT_SILU) return __fdividef(x, 1.0f + __expf(-x));
    if (ACT == ACT_GELU_TANH) {
        const float k0 = 0.79788456080286535587989211986876f, k1 = 0.044715f;
        const float u = k0 * x * (1.0f + k1 * x * x);
        return __fdividef(x, 1.0f + __expf(-2.0f * u));
    }
    if (ACT == ACT_GELU_ERF) return 0.5f * x * (1.0f + erff(x * 0.70710678118654752440f));
    return x;
}

// The activation is uniform over a launch: the epilogues branch on it ONCE per 32-column chunk and run a loop compiled
// for that activation.  (With the activation as a run-time argument of the element function the compiler evaluated
// every variant for every element and selected: the epilogue of a plain projection paid for SiLU, tanh-GELU and erf.)
template <int ACT>
__device__ __forceinline__ void gated_chunk(const uint32_t (&v)[32], float rms, uint32_t (&w)[8]) {
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        const float g0 = act_t<ACT>(__uint_as_float(v[4 * e]) * rms) * (__uint_as_float(v[4 * e + 1]) * rms);
        const float g1 = act_t<ACT>(__uint_as_float(v[4 * e + 2]) * rms) * (__uint_as_float(v[4 * e + 3]) * rms);
        const __nv_bfloat162 h2 = __floats2bfloat162_rn(g0, g1);
        w[e] = *reinterpret_cast<const uint32_t *>(&h2);
    }
}

template <int ACT>
__device__ __forceinline__ void act_chunk(float (&f)[32]) {
#pragma unroll
    for (int e = 0; e < 32; ++e) f[e] = act_t<ACT>(f[e]);
}

// SPLIT: the K loop of every output tile is cut into p.ksplit slices that run as separate work items; a slice stores its
// float accumulator to p.partial[slice][m][n] and splitk_reduce_kernel adds the slices in a fixed order (few rows and a
// narrow N would otherwise leave most SMs without work while a handful stream all of K).
template <int G_BN, bool PAIR, bool SPLIT = false>
__device__ __forceinline__ void dense_gemm_body(const CUtensorMap &a_map, const CUtensorMap &w_map, const GemmParams &p,
                                                int tiles_m, int tiles_n) {
    using Cfg = GemmCfg<G_BN, PAIR>;
    constexpr int G_STAGES = Cfg::STAGES, G_STAGE_BYTES = Cfg::STAGE_BYTES;
    constexpr int TILE_M = PAIR ? 2 * G_BM : G_BM;  // rows of one work unit
    const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
    // Every CTA (pair) walks a contiguous range of tiles; column tiles vary fastest, so consecutive tiles mostly
    // share their rows of A and the row statistics are computed once per row tile instead of once per tile.
    const int unit = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
    const int n_units = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
    extern __shared__ uint8_t g_smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(g_smem_raw) + 1023) &
                                                ~static_cast<uintptr_t>(1023));
    uint8_t *aux = smem + G_STAGES * G_STAGE_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(aux);
    uint64_t *full = bars, *empty = bars + 8;
    uint64_t *accum_full = bars + 16, *accum_empty = bars + 18, *stats_full = bars + 20, *stats_empty = bars + 22;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 24);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    float *stats = reinterpret_cast<float *>(aux + 256);  // [2][128]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ksteps = (p.K + G_BK - 1) / G_BK;
    const int ks_n = SPLIT ? p.ksplit : 1;
    const int n_tiles = tiles_m * tiles_n * ks_n;
    const int t_begin = (int)((long long)n_tiles * unit / n_units), t_end = (int)((long long)n_tiles * (unit + 1) / n_units);
    const WaitCtx wc{abort_flag, p.status};
    const uint32_t empty_count = p.use_rms ? 5u : 1u;

    if (threadIdx.x == 0) {
        for (int i = 0; i < G_STAGES; ++i) {
            mbar_init(&full[i], (PAIR && rank == 0) ? 2 : 1);  // even CTA of a pair: + the odd CTA's "stage landed"
            mbar_init(&empty[i], empty_count);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&accum_full[i], 1);
            mbar_init(&accum_empty[i], PAIR ? 16 : 256);  // pairs: one arrival per epilogue warp of both CTAs
            mbar_init(&stats_full[i], 128);
            mbar_init(&stats_empty[i], 256);
        }
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (PAIR) {
        __syncthreads();
        cluster_sync_all();  // both CTAs' barriers exist before anything arrives on them remotely
    }
    if (warp == 1) {
        if (PAIR) {
            tmem_alloc_pair(tmem_slot, 2 * G_BN);
            tmem_relinquish_pair();
        } else {
            tmem_alloc(tmem_slot, 2 * G_BN);
            tmem_relinquish();
        }
    }
    tc_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync_all();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (threadIdx.x == 0) {  // the descriptors are kernel parameters: fetching them does not depend on the previous kernel
        tma_prefetch_desc(&a_map);
        tma_prefetch_desc(&w_map);
    }
    pdl_launch_dependents();
    pdl_wait();  // everything above overlapped the previous kernel's tail; global memory is touched below

    if (warp == 0) {
        if (lane == 0) {
            uint32_t st = 0, ph = 0;
            bool ok = true;
            for (int tile = t_begin; ok && tile < t_end; ++tile) {
                const int sp = SPLIT ? tile / ks_n : tile, ks = SPLIT ? tile % ks_n : 0;
                const int kbeg = SPLIT ? ks * ksteps / ks_n : 0, kend = SPLIT ? (ks + 1) * ksteps / ks_n : ksteps;
                const int m0 = (sp / tiles_n) * TILE_M + (int)rank * G_BM;
                const int n0 = (sp % tiles_n) * G_BN + (int)rank * Cfg::B_ROWS * (PAIR ? 1 : 0);
                for (int kt = kbeg; kt < kend; ++kt) {
                    ok = mbar_wait(&empty[st], ph ^ 1u, wc, DEV_TIMEOUT_EMPTY);
                    if (!ok) break;
                    mbar_expect_tx(&full[st], G_STAGE_BYTES);
                    uint8_t *sa = smem + st * G_STAGE_BYTES;
                    tma_load_2d(sa, &a_map, &full[st], kt * G_BK, m0);
                    tma_load_2d(sa + G_A_BYTES, &w_map, &full[st], kt * G_BK, n0);
                    if (++st == G_STAGES) { st = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = make_idesc(1, 1, 1, 0, 0, TILE_M, G_BN);
            // descriptors differ between stages and k sub-steps only in the 14-bit start address
            const uint64_t a_desc0 = smem_desc_sw128(smem_u32(smem), 16, 1024);
            const uint64_t b_desc0 = smem_desc_sw128(smem_u32(smem + G_A_BYTES), 16, 1024);
            uint32_t st = 0, ph = 0, j = 0;
            bool ok = true;
            for (int tile = t_begin; ok && tile < t_end; ++tile, ++j) {
                const uint32_t buf = j & 1u;
                ok = mbar_wait(&accum_empty[buf], ((j >> 1) & 1u) ^ 1u, wc, DEV_TIMEOUT_EMPTY);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * G_BN;
                const int ks = SPLIT ? tile % ks_n : 0;
                const int kbeg = SPLIT ? ks * ksteps / ks_n : 0, kend = SPLIT ? (ks + 1) * ksteps / ks_n : ksteps;
                for (int kt = kbeg; kt < kend; ++kt) {
                    ok = mbar_wait(&full[st], ph, wc, DEV_TIMEOUT_FULL);
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t off = (uint64_t)(st * (G_STAGE_BYTES >> 4));
#pragma unroll
                    for (int k = 0; k < G_BK / 16; ++k) {
                        const uint32_t acc = (kt != kbeg || k != 0) ? 1u : 0u;  // the first MMA of a tile overwrites the accumulator
                        if (PAIR) mma_f16_pair(d_tmem, a_desc0 + off + 2 * k, b_desc0 + off + 2 * k, idesc, acc);
                        else mma_f16(d_tmem, a_desc0 + off + 2 * k, b_desc0 + off + 2 * k, idesc, acc);
                    }
                    if (PAIR) tc_commit_pair(&empty[st], 3);
                    else tc_commit(&empty[st]);
                    if (++st == G_STAGES) { st = 0; ph ^= 1u; }
                }
                if (!ok) break;
                if (PAIR) tc_commit_pair(&accum_full[buf], 3);
                else tc_commit(&accum_full[buf]);
            }
        } else if (PAIR && lane == 0) {
            // odd CTA of a pair: tell the even CTA when this CTA's stage has landed
            uint32_t st = 0, ph = 0;
            bool ok = true;
            for (int tile = t_begin; ok && tile < t_end; ++tile) {
                for (int kt = 0; kt < ksteps; ++kt) {
                    ok = mbar_wait(&full[st], ph, wc, DEV_TIMEOUT_FULL);
                    if (!ok) break;
                    mbar_arrive_cluster(&full[st], 0);
                    if (++st == G_STAGES) { st = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp >= 6 && warp < 10) {
        if (p.use_rms) {
            const int row = (warp - 6) * 32 + lane;
            const uint32_t row_base = (row >> 3) * 1024 + (row & 7) * 128;
            const uint32_t sw = row & 7;
            uint32_t st = 0, ph = 0, j = 0;
            bool ok = true;
            int prev_mt = -1;
            float row_sum = 0.0f;
            for (int tile = t_begin; ok && tile < t_end; ++tile, ++j) {
                const uint32_t buf = j & 1u;
                const int mt = tile / tiles_n;
                const bool fresh = mt != prev_mt;  // same rows of A as the previous tile: keep their sums
                prev_mt = mt;
                float s0 = 0.0f, s1 = 0.0f;
                for (int kt = 0; kt < ksteps; ++kt) {
                    ok = mbar_wait(&full[st], ph, wc, DEV_TIMEOUT_FULL);
                    if (!ok) break;
                    if (fresh) {
                        const uint8_t *at = smem + st * G_STAGE_BYTES + row_base;
#pragma unroll
                        for (int c = 0; c < 8; ++c) {
                            const uint4 v = *reinterpret_cast<const uint4 *>(at + ((c ^ sw) << 4));
                            const __nv_bfloat162 *h2 = reinterpret_cast<const __nv_bfloat162 *>(&v);
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const float2 f = __bfloat1622float2(h2[e]);
                                s0 = fmaf(f.x, f.x, s0);
                                s1 = fmaf(f.y, f.y, s1);
                            }
                        }
                    }
                    stage_release(&empty[st], s0 + s1, lane);
                    if (++st == G_STAGES) { st = 0; ph ^= 1u; }
                }
                if (!ok) break;
                if (fresh) row_sum = s0 + s1;
                ok = mbar_wait(&stats_empty[buf], ((j >> 1) & 1u) ^ 1u, wc, DEV_TIMEOUT_EMPTY);
                if (!ok) break;
                stats[buf * 128 + row] = row_sum;
                mbar_arrive(&stats_full[buf]);
            }
        }
    } else {
        // ---- epilogue warps 2..5 (group 0: first half of the tile's columns) and 10..13 (group 1: second half) ----
        const int qtr = warp & 3;
        const int grp = warp >= 10 ? 1 : 0;
        const int row = qtr * 32 + lane;
        uint32_t j = 0;
        bool ok = true;
        for (int tile = t_begin; ok && tile < t_end; ++tile, ++j) {
            const uint32_t buf = j & 1u;
            const int sp = SPLIT ? tile / ks_n : tile;
            const int m0 = (sp / tiles_n) * TILE_M + (int)rank * G_BM, n0 = (sp % tiles_n) * G_BN;
            const int m = m0 + row;
            const bool row_ok = m < p.M;
            ok = mbar_wait(&accum_full[buf], (j >> 1) & 1u, wc, DEV_TIMEOUT_ACCUM);
            if (ok && p.use_rms) ok = mbar_wait(&stats_full[buf], (j >> 1) & 1u, wc, DEV_TIMEOUT_ACCUM);
            if (!ok) break;
            tc_fence_after();
            const float rms = p.use_rms ? rsqrtf(stats[buf * 128 + row] / (float)p.K + p.eps) : 1.0f;
            const uint32_t lane_addr = tmem_base + buf * G_BN + ((uint32_t)(qtr * 32) << 16);
            size_t mo = (size_t)m;
            if (p.rows_in > 0 && p.scatter_hd == 0) mo = (size_t)(m / p.rows_in) * p.rows_out + p.row_off + (m % p.rows_in);
            for (int c = grp * (G_BN / 2); c < (grp + 1) * (G_BN / 2); c += 32) {
                const int n = n0 + c;
                if (n >= p.N) break;  // N % 8 == 0: a chunk may be cut after a multiple of 8 columns
                uint32_t v[32];
                tmem_ld32(lane_addr + (uint32_t)c, v);
                tmem_ld_wait();
                if (!row_ok) continue;
                if constexpr (SPLIT) {  // this slice's float sums, row-major [slice][M][N]
                    float4 *dst = reinterpret_cast<float4 *>(p.partial + ((size_t)(tile % ks_n) * p.M + m) * p.N + n);
#pragma unroll
                    for (int e = 0; e < 8; ++e)
                        if (n + 4 * e < p.N)
                            dst[e] = make_float4(__uint_as_float(v[4 * e]), __uint_as_float(v[4 * e + 1]), __uint_as_float(v[4 * e + 2]),
                                                 __uint_as_float(v[4 * e + 3]));
                    continue;
                }
                if (p.epi == EPI_RESIDUAL) {
                    if (p.colscale) {  // gated residual: the projection's column n is multiplied by colscale[n] first
#pragma unroll
                        for (int e = 0; e < 32; ++e)
                            if (n + e < p.N) v[e] = __float_as_uint(__uint_as_float(v[e]) * __ldg(p.colscale + n + e));
                    }
                    if (p.bias) {
#pragma unroll
                        for (int e = 0; e < 32; ++e)
                            if (n + e < p.N) v[e] = __float_as_uint(__uint_as_float(v[e]) + __ldg(p.bias + n + e));
                    }
                    float *hrow = p.h + mo * p.ld_out + n;
                    __nv_bfloat16 *brow = p.out_bf + mo * p.ld_out + n;
                    if (p.al32) {
                        // 8 float32 columns = one 32-byte sector per load / store and thread
#pragma unroll
                        for (int q8 = 0; q8 < 2; ++q8) {
                            if (n + 16 * q8 >= p.N) break;
                            const bool two = n + 16 * q8 + 8 < p.N;
                            uint32_t w[8];
#pragma unroll
                            for (int hlf = 0; hlf < 2; ++hlf) {
                                if (hlf && !two) break;
                                const int c0 = 16 * q8 + 8 * hlf;
                                uint32_t a[8];
                                ld_global_v8(hrow + c0, a);
#pragma unroll
                                for (int e = 0; e < 8; ++e) a[e] = __float_as_uint(__uint_as_float(a[e]) + __uint_as_float(v[c0 + e]));
                                st_global_v8(hrow + c0, a);
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    const __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(a[2 * e]), __uint_as_float(a[2 * e + 1]));
                                    w[4 * hlf + e] = *reinterpret_cast<const uint32_t *>(&h2);
                                }
                            }
                            if (two) st_global_v8(brow + 16 * q8, w);
                            else *reinterpret_cast<uint4 *>(brow + 16 * q8) = make_uint4(w[0], w[1], w[2], w[3]);
                        }
                    } else {
                    float4 *hp = reinterpret_cast<float4 *>(hrow);
                    uint4 *bp = reinterpret_cast<uint4 *>(brow);
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        if (n + 8 * q4 >= p.N) break;
                        float4 a = hp[2 * q4], b = hp[2 * q4 + 1];
                        a.x += __uint_as_float(v[8 * q4]); a.y += __uint_as_float(v[8 * q4 + 1]);
                        a.z += __uint_as_float(v[8 * q4 + 2]); a.w += __uint_as_float(v[8 * q4 + 3]);
                        b.x += __uint_as_float(v[8 * q4 + 4]); b.y += __uint_as_float(v[8 * q4 + 5]);
                        b.z += __uint_as_float(v[8 * q4 + 6]); b.w += __uint_as_float(v[8 * q4 + 7]);
                        hp[2 * q4] = a;
                        hp[2 * q4 + 1] = b;
                        const __nv_bfloat162 h0 = __floats2bfloat162_rn(a.x, a.y), h1 = __floats2bfloat162_rn(a.z, a.w);
                        const __nv_bfloat162 h2 = __floats2bfloat162_rn(b.x, b.y), h3 = __floats2bfloat162_rn(b.z, b.w);
                        bp[q4] = make_uint4(*reinterpret_cast<const uint32_t *>(&h0), *reinterpret_cast<const uint32_t *>(&h1),
                                            *reinterpret_cast<const uint32_t *>(&h2), *reinterpret_cast<const uint32_t *>(&h3));
                    }
                    }
                } else if (p.epi == EPI_GATED) {
                    uint32_t w[8];
                    if (p.act == ACT_SILU) gated_chunk<ACT_SILU>(v, rms, w);
                    else gated_chunk<ACT_GELU_TANH>(v, rms, w);
                    __nv_bfloat16 *brow = p.out_bf + mo * p.ld_out + (n >> 1);
                    if (p.al32 && n + 16 < p.N) {
                        st_global_v8(brow, w);
                    } else {
                        uint4 *bp = reinterpret_cast<uint4 *>(brow);
                        bp[0] = make_uint4(w[0], w[1], w[2], w[3]);
                        if (n + 16 < p.N) bp[1] = make_uint4(w[4], w[5], w[6], w[7]);
                    }
                } else {
                    float f[32];
#pragma unroll
                    for (int e = 0; e < 32; ++e)
                        f[e] = __uint_as_float(v[e]) * rms + ((p.bias && n + e < p.N) ? __ldg(p.bias + n + e) : 0.0f);
                    if (p.act == ACT_SILU) act_chunk<ACT_SILU>(f);
                    else if (p.act == ACT_GELU_TANH) act_chunk<ACT_GELU_TANH>(f);
                    else if (p.act == ACT_GELU_ERF) act_chunk<ACT_GELU_ERF>(f);
                    if (p.out_f32) {
                        float4 *fp = reinterpret_cast<float4 *>(p.out_f32 + mo * p.ld_out + n);
#pragma unroll
                        for (int e = 0; e < 8; ++e)
                            if (n + 4 * e < p.N) fp[e] = make_float4(f[4 * e], f[4 * e + 1], f[4 * e + 2], f[4 * e + 3]);
                    }
                    if (p.out_bf) {
                        size_t off = mo * p.ld_out + n;
                        if (p.scatter_hd > 0)  // head-major pages: [obs][head][cap][hd]
                            off = ((size_t)(m / p.rows_in) * (p.N / p.scatter_hd) + (size_t)(n / p.scatter_hd)) *
                                      ((size_t)p.scatter_cap * p.scatter_hd) +
                                  (size_t)(m % p.rows_in) * p.scatter_hd + (n % p.scatter_hd);
                        uint4 *bp = reinterpret_cast<uint4 *>(p.out_bf + off);
#pragma unroll
                        for (int q4 = 0; q4 < 4; ++q4) {
                            if (n + 8 * q4 >= p.N) break;
                            uint32_t w[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const __nv_bfloat162 h2 = __floats2bfloat162_rn(f[8 * q4 + 2 * e], f[8 * q4 + 2 * e + 1]);
                                w[e] = *reinterpret_cast<const uint32_t *>(&h2);
                            }
                            bp[q4] = make_uint4(w[0], w[1], w[2], w[3]);
                        }
                    }
                }
            }
            tc_fence_before();
            if (PAIR) {
                __syncwarp();
                if (lane == 0) {
                    if (rank == 0) mbar_arrive(&accum_empty[buf]);
                    else mbar_arrive_cluster(&accum_empty[buf], 0);
                }
            } else {
                mbar_arrive(&accum_empty[buf]);
            }
            if (p.use_rms) mbar_arrive(&stats_empty[buf]);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync_all();  // neither CTA may exit while the other can still signal its barriers
    if (warp == 1) {
        tc_fence_after();
        if (PAIR) tmem_dealloc_pair(tmem_base, 2 * G_BN);
        else tmem_dealloc(tmem_base, 2 * G_BN);
    }
}

template <int G_BN>
__global__ void __launch_bounds__(G_THREADS, 1)
dense_gemm_kernel(const __grid_constant__ CUtensorMap a_map, const __grid_constant__ CUtensorMap w_map,
                  const GemmParams p, int tiles_m, int tiles_n) {
    dense_gemm_body<G_BN, false>(a_map, w_map, p, tiles_m, tiles_n);
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(G_THREADS, 1)
dense_gemm_pair_kernel(const __grid_constant__ CUtensorMap a_map, const __grid_constant__ CUtensorMap w_map,
                       const GemmParams p, int tiles_m, int tiles_n) {
    dense_gemm_body<256, true>(a_map, w_map, p, tiles_m, tiles_n);
}

__global__ void __launch_bounds__(G_THREADS, 1)
dense_gemm_splitk_kernel(const __grid_constant__ CUtensorMap a_map, const __grid_constant__ CUtensorMap w_map,
                         const GemmParams p, int tiles_m, int tiles_n) {
    dense_gemm_body<64, false, true>(a_map, w_map, p, tiles_m, tiles_n);
}

// h[m][n] += (sum over the K slices, in slice order) (* colscale[n]) (+ bias[n]); hb = bf16(h).  Four columns per thread.
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float *__restrict__ partial, int ksplit, int M, int N,
                                                            const float *__restrict__ colscale, const float *__restrict__ bias,
                                                            float *__restrict__ h, __nv_bfloat16 *__restrict__ hb, int ld) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t total4 = (size_t)M * N / 4;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total4; i += (size_t)gridDim.x * blockDim.x) {
        const int m = (int)(i / (N / 4)), n = (int)(i % (N / 4)) * 4;
        float4 a = *reinterpret_cast<const float4 *>(partial + (size_t)m * N + n);
        for (int s = 1; s < ksplit; ++s) {
            const float4 b = *reinterpret_cast<const float4 *>(partial + ((size_t)s * M + m) * N + n);
            a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
        }
        if (colscale) {
            const float4 c = *reinterpret_cast<const float4 *>(colscale + n);
            a.x *= c.x; a.y *= c.y; a.z *= c.z; a.w *= c.w;
        }
        if (bias) {
            const float4 c = *reinterpret_cast<const float4 *>(bias + n);
            a.x += c.x; a.y += c.y; a.z += c.z; a.w += c.w;
        }
        float4 *hp = reinterpret_cast<float4 *>(h + (size_t)m * ld + n);
        float4 r = *hp;
        r.x += a.x; r.y += a.y; r.z += a.z; r.w += a.w;
        *hp = r;
        const __nv_bfloat162 lo = __floats2bfloat162_rn(r.x, r.y), hi = __floats2bfloat162_rn(r.z, r.w);
        *reinterpret_cast<uint2 *>(hb + (size_t)m * ld + n) =
            make_uint2(*reinterpret_cast<const uint32_t *>(&lo), *reinterpret_cast<const uint32_t *>(&hi));
    }
}

// 0 = choose by cost; 1 / 2 / 3 / 4 force the 128 x 256, 128 x 128, CTA-pair and 128 x 64 tilings (testing knob).
static std::atomic<int> g_gemm_variant{0};
constexpr float kPairTileFactor = 0.95f;  // time of a pair's 256 x 256 tile relative to a lone CTA's 128 x 256 tile

void dense_gemm_set_variant(int v) { g_gemm_variant.store((v >= 0 && v <= 4) ? v : 0, std::memory_order_relaxed); }
int dense_gemm_variant() { return g_gemm_variant.load(std::memory_order_relaxed); }

// Four tilings: one CTA per 128 x 256 tile, per 128 x 128 or 128 x 64 tile (more CTAs streaming the weights when the
// problem has few rows), a CTA pair per 256 x 256 tile (half the shared-memory traffic per flop).  Cost of the cheapest
// one in units of one 128 x 256 tile on one SM; the per-tile factors are measured ratios.
static float tiling_cost(int M, int N, int n_sm, int *variant_out) {
    const int tiles_m = (M + G_BM - 1) / G_BM, tiles_mp = (M + 2 * G_BM - 1) / (2 * G_BM);
    const int tn256 = (N + 255) / 256, tn128 = (N + 127) / 128, tn64 = (N + 63) / 64, pairs = n_sm / 2;
    auto waves = [](int tiles, int units) { return (tiles + units - 1) / units; };
    const float cost256 = (float)waves(tiles_m * tn256, n_sm);
    const float cost128 = N > 128 ? 0.60f * waves(tiles_m * tn128, n_sm) : 1e30f;
    const float cost64 = N > 64 ? 0.33f * waves(tiles_m * tn64, n_sm) : 1e30f;  // few rows: as many CTAs as possible stream W
    const float cost_pair = pairs > 0 ? kPairTileFactor * waves(tiles_mp * tn256, pairs) : 1e30f;
    int variant = (cost_pair <= cost256 && cost_pair <= cost128) ? 3 : (cost128 < cost256 ? 2 : 1);
    float best = variant == 3 ? cost_pair : (variant == 2 ? cost128 : cost256);
    if (cost64 < best) {
        variant = 4;
        best = cost64;
    }
    if (variant_out) *variant_out = variant;
    return best;
}

static int dense_gemm_one(const void *A, int lda, const void *W, GemmParams p, cudaStream_t stream, int forced_variant);

// Launches the GEMM.  A: bf16 [M][K] (row stride lda elements), W: bf16 [N][K].
//
// Rows are independent, so a problem whose tiles fill the machine unevenly is cut in two along M: the first rows as
// CTA-pair tiles in a whole number of waves, the remaining rows with whichever tiling is cheapest for them (for
// 6528 x 1024: 72 pair tiles on 74 pairs, then 128 tiles of 128 x 128 on 148 SMs, instead of 408 tiles in three waves).
// Every output element is computed by the same arithmetic in either part, so results do not depend on the cut.
int dense_gemm(const void *A, int lda, const void *W, GemmParams p, cudaStream_t stream) {
    if (!A || !W || p.M <= 0 || p.N <= 0 || p.K <= 0) return VLAB200_ERR_ARG;
    const int n_sm = sm_count();
    // Few rows, narrow N, long K (Wo / Wdown of one to five observations: 16 or 32 tiles of 128 x 64 for N = 1024, each
    // streaming all of K through one SM): cut K so that the slices fill the machine, then add the slices in a fixed order.
    if (p.partial && p.epi == EPI_RESIDUAL && dense_gemm_variant() == 0 && p.M <= p.partial_rows && p.rows_in == 0 &&
        p.scatter_hd == 0 && !p.use_rms && p.N % 4 == 0 && n_sm > 0) {
        const int tiles = ((p.M + G_BM - 1) / G_BM) * ((p.N + 63) / 64), ksteps = (p.K + G_BK - 1) / G_BK;
        int ksplit = n_sm / tiles;
        if (ksplit > ksteps / 4) ksplit = ksteps / 4;  // at least four 64-wide k-steps per slice
        if (ksplit > p.partial_slices) ksplit = p.partial_slices;
        if (ksplit >= 2) {
            GemmParams ps = p;
            ps.ksplit = ksplit;
            int rc = dense_gemm_one(A, lda, W, ps, stream, 5);
            if (rc) return rc;
            const size_t total4 = (size_t)p.M * p.N / 4;
            const int blocks = (int)((total4 + 255) / 256 < (size_t)n_sm * 4 ? (total4 + 255) / 256 : (size_t)n_sm * 4);
            return launch_pdl(splitk_reduce_kernel, dim3(blocks), dim3(256), 0, stream, static_cast<const float *>(p.partial), ksplit,
                              p.M, p.N, p.colscale, p.bias, p.h, p.out_bf, p.ld_out);
        }
    }
    static const bool split_off = std::getenv("VLAB200_NO_GEMM_SPLIT") != nullptr;  // measurement knob
    if (!split_off && dense_gemm_variant() == 0 && n_sm >= 2 && p.rows_in == 0 && p.scatter_hd == 0 && p.M > 2 * G_BM) {
        const int pairs = n_sm / 2, tn256 = (p.N + 255) / 256, tiles_mp = (p.M + 2 * G_BM - 1) / (2 * G_BM);
        int v_all = 0;
        const float whole = tiling_cost(p.M, p.N, n_sm, &v_all);
        // a second launch costs about 6 us; a 128 x 256 tile takes about K / 64 x 0.5 us
        const float launch_pen = 6.0f / (0.5f * (float)((p.K + G_BK - 1) / G_BK));
        float best = whole;
        int best_rows = 0;
        for (int w = 1; w * pairs < tiles_mp * tn256; ++w) {
            const int a = w * pairs / tn256;  // pair row-tiles that fit into w waves
            if (a <= 0 || a >= tiles_mp) continue;
            const float c = kPairTileFactor * (float)w + tiling_cost(p.M - a * 2 * G_BM, p.N, n_sm, nullptr) + launch_pen;
            if (c < best) {
                best = c;
                best_rows = a * 2 * G_BM;
            }
        }
        if (best_rows > 0 && best < 0.97f * whole) {
            GemmParams pa = p, pb = p;
            pa.M = best_rows;
            pb.M = p.M - best_rows;
            const size_t off = (size_t)best_rows * p.ld_out;
            if (pb.h) pb.h += off;
            if (pb.out_bf) pb.out_bf += off;
            if (pb.out_f32) pb.out_f32 += off;
            int rc = dense_gemm_one(A, lda, W, pa, stream, 3);
            if (rc) return rc;
            return dense_gemm_one(static_cast<const __nv_bfloat16 *>(A) + (size_t)best_rows * lda, lda, W, pb, stream, 0);
        }
    }
    return dense_gemm_one(A, lda, W, p, stream, 0);
}

static int dense_gemm_one(const void *A, int lda, const void *W, GemmParams p, cudaStream_t stream, int forced_variant) {
    if (!A || !W || p.M <= 0 || p.N <= 0 || p.K <= 0) return VLAB200_ERR_ARG;
    if (p.N % 8 || (p.epi == EPI_GATED && p.N % 16) || p.K % 8 || lda % 8 || p.ld_out % 8) return VLAB200_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(W) & 15)) return VLAB200_ERR_ARG;
    {
        // 256-bit epilogue accesses need every touched row segment on a 32-byte boundary
        const bool f32_ok = !p.h || ((reinterpret_cast<uintptr_t>(p.h) & 31) == 0 && p.ld_out % 8 == 0);
        const bool bf_ok = !p.out_bf || ((reinterpret_cast<uintptr_t>(p.out_bf) & 31) == 0 && p.ld_out % 16 == 0);
        p.al32 = (p.rows_in == 0 && f32_ok && bf_ok) ? 1 : 0;
    }
    p.status = device_status_ptr();
    if (!p.status) return cuda_fail(cudaGetLastError(), "device_status_ptr");
    CUtensorMap amap, wmap;
    {
        const uint64_t dims[2] = {(uint64_t)p.K, (uint64_t)p.M};
        const uint64_t strides[1] = {(uint64_t)lda * 2};
        const uint32_t box[2] = {G_BK, G_BM};
        int rc = make_tensor_map(&amap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, A, dims, strides, box,
                                 CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc) return rc;
    }
    {
        const uint64_t dims[2] = {(uint64_t)p.K, (uint64_t)p.N};
        const uint64_t strides[1] = {(uint64_t)p.K * 2};
        const uint32_t box[2] = {G_BK, 256};
        int rc = make_tensor_map(&wmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, W, dims, strides, box,
                                 CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc) return rc;
    }
    const int n_sm = sm_count();
    if (n_sm <= 0) return cuda_fail(cudaGetLastError(), "sm_count");
    int variant = forced_variant > 0 ? forced_variant : dense_gemm_variant();
    if (variant == 0) tiling_cost(p.M, p.N, n_sm, &variant);
    const int tiles_m = (p.M + G_BM - 1) / G_BM, tiles_mp = (p.M + 2 * G_BM - 1) / (2 * G_BM);
    const int tn256 = (p.N + 255) / 256, tn128 = (p.N + 127) / 128, tn64 = (p.N + 63) / 64, pairs = n_sm / 2;
    if (variant == 2 && p.N <= 128) variant = 1;
    if (variant == 4 && p.N <= 64) variant = 1;
    const uint64_t wdims[2] = {(uint64_t)p.K, (uint64_t)p.N};
    const uint64_t wstrides[1] = {(uint64_t)p.K * 2};
    if (variant == 5) {  // split-K slices on 128 x 64 tiles
        const uint32_t box[2] = {G_BK, 64};
        int rc = make_tensor_map(&wmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, W, wdims, wstrides, box,
                                 CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc) return rc;
        if (int rc = ensure_dyn_smem(dense_gemm_splitk_kernel, GemmCfg<64, false>::SMEM)) return rc;
        const int nt = tiles_m * tn64 * p.ksplit;
        return launch_pdl(dense_gemm_splitk_kernel, dim3(nt < n_sm ? nt : n_sm), dim3(G_THREADS), GemmCfg<64, false>::SMEM, stream,
                          amap, wmap, p, tiles_m, tn64);
    }
    if (variant == 3) {
        const uint32_t box[2] = {G_BK, 128};  // each CTA of a pair stages half of the 256 weight rows
        int rc = make_tensor_map(&wmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, W, wdims, wstrides, box,
                                 CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc) return rc;
        if (int rc = ensure_dyn_smem(dense_gemm_pair_kernel, GemmCfg<256, true>::SMEM)) return rc;
        const int nt = tiles_mp * tn256;
        return launch_pdl(dense_gemm_pair_kernel, dim3(2 * (nt < pairs ? nt : pairs)), dim3(G_THREADS), GemmCfg<256, true>::SMEM,
                          stream, amap, wmap, p, tiles_mp, tn256);
    } else if (variant == 4) {
        const uint32_t box[2] = {G_BK, 64};
        int rc = make_tensor_map(&wmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, W, wdims, wstrides, box,
                                 CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc) return rc;
        if (int rc = ensure_dyn_smem(dense_gemm_kernel<64>, GemmCfg<64, false>::SMEM)) return rc;
        const int nt = tiles_m * tn64;
        return launch_pdl(dense_gemm_kernel<64>, dim3(nt < n_sm ? nt : n_sm), dim3(G_THREADS), GemmCfg<64, false>::SMEM, stream,
                          amap, wmap, p, tiles_m, tn64);
    } else if (variant == 2) {
        const uint32_t box[2] = {G_BK, 128};
        int rc = make_tensor_map(&wmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, W, wdims, wstrides, box,
                                 CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc) return rc;
        if (int rc = ensure_dyn_smem(dense_gemm_kernel<128>, GemmCfg<128, false>::SMEM)) return rc;
        const int nt = tiles_m * tn128;
        return launch_pdl(dense_gemm_kernel<128>, dim3(nt < n_sm ? nt : n_sm), dim3(G_THREADS), GemmCfg<128, false>::SMEM, stream,
                          amap, wmap, p, tiles_m, tn128);
    } else {
        if (int rc = ensure_dyn_smem(dense_gemm_kernel<256>, GemmCfg<256, false>::SMEM)) return rc;
        const int nt = tiles_m * tn256;
        return launch_pdl(dense_gemm_kernel<256>, dim3(nt < n_sm ? nt : n_sm), dim3(G_THREADS), GemmCfg<256, false>::SMEM, stream,
                          amap, wmap, p, tiles_m, tn256);
    }
    VB_CUDA(cudaGetLastError());
    return VLAB200_OK;
}

}  // namespace vb

extern "C" int32_t vlab200_set_gemm_tiling(int32_t tiling) {
    if (tiling < 0 || tiling > 4) return VLAB200_ERR_ARG;
    vb::dense_gemm_set_variant(tiling);
    return VLAB200_OK;
}
