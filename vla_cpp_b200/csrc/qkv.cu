// Fused RMSNorm -> QKV projection -> NeoX RoPE -> KV append for the action-suffix tokens,
// plus the prefix-KV page writer.  One tcgen05 GEMM per layer-step:
//
//   x [M = n_obs*S][H] (bf16 or f32)  --(x * ln_w, bf16, swizzled smem)-->  A operand
//   Wqkv [(n_q + 2 n_kv) hd][H] bf16  --(TMA, SWIZZLE_128B)-->              B operand
//   accumulator f32 in TMEM; epilogue multiplies row m by rsqrt(mean(x_m^2)+eps)
//   (the per-row RMSNorm factor commutes with the projection), rotates q/k, and writes
//   q to [obs][head][tok][hd], k/v into rows prefix_len+tok of the (layer, obs, kv head) pages.
//
// Reference: src/models/pi0.cpp:170-201, src/models/smolvla.cpp:820-833 (three mul_mat,
// two rope, two concat that copy the whole prefix KV each layer-step).
#include <cuda_bf16.h>

#include "gemm.h"
#include "host_common.h"
#include "tc5.cuh"

namespace vb {

constexpr int QKV_BM = 128, QKV_BN = 256, QKV_BK = 64;  // BK in elements (128 bytes of bf16)
constexpr int QKV_STAGES = 4;
constexpr int QKV_THREADS = 192;
constexpr int QKV_A_BYTES = QKV_BM * 128, QKV_B_BYTES = QKV_BN * 128;
constexpr int QKV_STAGE_BYTES = QKV_A_BYTES + QKV_B_BYTES;

struct QkvParams {
    const void *x;          // [M][H]
    const float *ln_w;      // [H]
    const float *rope_cos;  // [S][hd/2]
    const float *rope_sin;
    __nv_bfloat16 *q_out;   // [n_obs][n_q][S][hd]
    __nv_bfloat16 *k_pages; // layer base: [n_obs][n_kv][cap][hd]
    __nv_bfloat16 *v_pages;
    int M, H, S, hd, n_q, n_kv_proj, n_kv, cap, prefix_len;
    float eps;
    int *status;
};

template <bool X_F32>
__global__ void __launch_bounds__(QKV_THREADS, 1)
qkv_rope_kernel(const __grid_constant__ CUtensorMap w_map, const QkvParams p) {
    extern __shared__ uint8_t qkv_smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(qkv_smem_raw) + 1023) &
                                                ~static_cast<uintptr_t>(1023));
    uint64_t *full_a = reinterpret_cast<uint64_t *>(smem + QKV_STAGES * QKV_STAGE_BYTES);
    uint64_t *full_b = full_a + QKV_STAGES;
    uint64_t *empty = full_b + QKV_STAGES;
    uint64_t *accum_bar = empty + QKV_STAGES;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(accum_bar + 1);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    float *ln_s = reinterpret_cast<float *>(smem + QKV_STAGES * QKV_STAGE_BYTES + 256);  // [ksteps*64]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.x * QKV_BM, n0 = blockIdx.y * QKV_BN;
    const int ksteps = (p.H + QKV_BK - 1) / QKV_BK;
    const WaitCtx wc{abort_flag, p.status};

    if (threadIdx.x == 0) {
        for (int i = 0; i < QKV_STAGES; ++i) {
            mbar_init(&full_a[i], 128);
            mbar_init(&full_b[i], 1);
            mbar_init(&empty[i], 1);
        }
        mbar_init(accum_bar, 1);
        *abort_flag = 0;
        fence_barrier_init();
    }
    for (int i = threadIdx.x; i < ksteps * QKV_BK; i += QKV_THREADS) ln_s[i] = i < p.H ? p.ln_w[i] : 0.0f;
    if (warp == 1) {
        tmem_alloc(tmem_slot, QKV_BN);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            tma_prefetch_desc(&w_map);
            for (int kt = 0; kt < ksteps; ++kt) {
                const int st = kt % QKV_STAGES;
                const uint32_t ph = (uint32_t)(kt / QKV_STAGES) & 1u;
                if (!mbar_wait(&empty[st], ph ^ 1u, wc, DEV_TIMEOUT_EMPTY)) break;
                mbar_expect_tx(&full_b[st], QKV_B_BYTES);
                tma_load_2d(smem + st * QKV_STAGE_BYTES + QKV_A_BYTES, &w_map, &full_b[st], kt * QKV_BK, n0);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(1, 1, 1, 0, 0, QKV_BM, QKV_BN);
            for (int kt = 0; kt < ksteps; ++kt) {
                const int st = kt % QKV_STAGES;
                const uint32_t ph = (uint32_t)(kt / QKV_STAGES) & 1u;
                if (!mbar_wait(&full_a[st], ph, wc, DEV_TIMEOUT_FULL)) break;
                if (!mbar_wait(&full_b[st], ph, wc, DEV_TIMEOUT_FULL)) break;
                tc_fence_after();
                const uint32_t a_addr = smem_u32(smem + st * QKV_STAGE_BYTES);
                const uint32_t b_addr = a_addr + QKV_A_BYTES;
#pragma unroll
                for (int k = 0; k < QKV_BK / 16; ++k) {
                    mma_f16(tmem_base, smem_desc_sw128(a_addr + k * 32, 16, 1024),
                            smem_desc_sw128(b_addr + k * 32, 16, 1024), idesc, (kt | k) != 0 ? 1u : 0u);
                }
                tc_commit(&empty[st]);
            }
            tc_commit(accum_bar);
        }
    } else {
        // ---- A producer: thread owns row (quarter*32 + lane), the row it later reads from TMEM ----
        const int qtr = warp & 3;
        const int row = qtr * 32 + lane;
        const int m = m0 + row;
        const bool row_ok = m < p.M;
        float sumsq = 0.0f;
        const uint32_t row_base = (row >> 3) * 1024 + (row & 7) * 128;
        const uint32_t sw = row & 7;
        // register prefetch of the next 64 elements of this row
        uint4 raw[X_F32 ? 16 : 8];
        auto load_raw = [&](int kt) {
            const int k0 = kt * QKV_BK;
            if constexpr (X_F32) {
                const float *xr = static_cast<const float *>(p.x) + (size_t)m * p.H + k0;
#pragma unroll
                for (int i = 0; i < 16; ++i)
                    raw[i] = (row_ok && k0 + 4 * i < p.H) ? __ldg(reinterpret_cast<const uint4 *>(xr) + i)
                                                           : make_uint4(0, 0, 0, 0);
            } else {
                const __nv_bfloat16 *xr = static_cast<const __nv_bfloat16 *>(p.x) + (size_t)m * p.H + k0;
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    raw[i] = (row_ok && k0 + 8 * i < p.H) ? __ldg(reinterpret_cast<const uint4 *>(xr) + i)
                                                           : make_uint4(0, 0, 0, 0);
            }
        };
        load_raw(0);
        for (int kt = 0; kt < ksteps; ++kt) {
            const int st = kt % QKV_STAGES;
            const uint32_t ph = (uint32_t)(kt / QKV_STAGES) & 1u;
            // convert the prefetched chunk: y = bf16(x * ln_w), sumsq += x^2
            uint4 packed[8];
            const float *lw = ln_s + kt * QKV_BK;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                float f[8];
                if constexpr (X_F32) {
                    const float4 a = *reinterpret_cast<const float4 *>(&raw[2 * c]);
                    const float4 b = *reinterpret_cast<const float4 *>(&raw[2 * c + 1]);
                    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
                    f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
                } else {
                    const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&raw[c]);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float2 t = __bfloat1622float2(h[j]);
                        f[2 * j] = t.x;
                        f[2 * j + 1] = t.y;
                    }
                }
                uint32_t w[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    sumsq = fmaf(f[2 * j], f[2 * j], sumsq);
                    sumsq = fmaf(f[2 * j + 1], f[2 * j + 1], sumsq);
                    const __nv_bfloat162 h2 =
                        __floats2bfloat162_rn(f[2 * j] * lw[8 * c + 2 * j], f[2 * j + 1] * lw[8 * c + 2 * j + 1]);
                    w[j] = *reinterpret_cast<const uint32_t *>(&h2);
                }
                packed[c] = make_uint4(w[0], w[1], w[2], w[3]);
            }
            if (kt + 1 < ksteps) load_raw(kt + 1);
            if (!mbar_wait(&empty[st], ph ^ 1u, wc, DEV_TIMEOUT_EMPTY)) break;
            uint8_t *at = smem + st * QKV_STAGE_BYTES + row_base;
#pragma unroll
            for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4 *>(at + ((c ^ sw) << 4)) = packed[c];
            fence_proxy_async_smem();
            mbar_arrive(&full_a[st]);
        }
        // ---- epilogue ----
        // (tcgen05.ld is warp-collective: every lane runs the loads, only stores are predicated)
        if (mbar_wait(accum_bar, 0, wc, DEV_TIMEOUT_ACCUM)) {
            tc_fence_after();
            const float rms = p.eps < 0.0f ? 1.0f : rsqrtf(sumsq / (float)p.H + p.eps);  // eps < 0: x is already normalised
            const int obs = m / p.S, tok = m % p.S;
            const int hd = p.hd, half = hd >> 1;
            const int n_total = (p.n_q + 2 * p.n_kv_proj) * hd;
            const float *cs = p.rope_cos + (size_t)tok * half;
            const float *sn = p.rope_sin + (size_t)tok * half;
            const uint32_t lane_addr = tmem_base + ((uint32_t)(qtr * 32) << 16);
            for (int hc = 0; hc < QKV_BN; hc += hd) {  // one head per iteration
                const int n = n0 + hc;
                if (n >= n_total) break;
                const int head = n / hd;
                __nv_bfloat16 *dst;
                bool rotate = true;
                if (head < p.n_q) {
                    dst = p.q_out + (((size_t)obs * p.n_q + head) * p.S + tok) * hd;
                } else if (head < p.n_q + p.n_kv_proj) {
                    const int kvh = head - p.n_q;
                    dst = p.k_pages + (((size_t)obs * p.n_kv + kvh) * p.cap + p.prefix_len + tok) * hd;
                } else {
                    const int kvh = head - p.n_q - p.n_kv_proj;
                    dst = p.v_pages + (((size_t)obs * p.n_kv + kvh) * p.cap + p.prefix_len + tok) * hd;
                    rotate = false;
                }
                for (int c = 0; c < half; c += 32) {
                    uint32_t lo[32], hi[32];
                    tmem_ld32(lane_addr + (uint32_t)(hc + c), lo);
                    tmem_ld32(lane_addr + (uint32_t)(hc + half + c), hi);
                    tmem_ld_wait();
                    uint32_t olo[16], ohi[16];
#pragma unroll
                    for (int j = 0; j < 32; j += 2) {
                        float a0 = __uint_as_float(lo[j]) * rms, a1 = __uint_as_float(lo[j + 1]) * rms;
                        float b0 = __uint_as_float(hi[j]) * rms, b1 = __uint_as_float(hi[j + 1]) * rms;
                        if (rotate) {
                            const float c0 = cs[c + j], c1 = cs[c + j + 1], s0 = sn[c + j], s1 = sn[c + j + 1];
                            const float r0 = a0 * c0 - b0 * s0, r1 = a1 * c1 - b1 * s1;
                            b0 = b0 * c0 + a0 * s0;
                            b1 = b1 * c1 + a1 * s1;
                            a0 = r0;
                            a1 = r1;
                        }
                        const __nv_bfloat162 l2 = __floats2bfloat162_rn(a0, a1), h2 = __floats2bfloat162_rn(b0, b1);
                        olo[j >> 1] = *reinterpret_cast<const uint32_t *>(&l2);
                        ohi[j >> 1] = *reinterpret_cast<const uint32_t *>(&h2);
                    }
                    if (!row_ok) continue;
                    uint4 *dl = reinterpret_cast<uint4 *>(dst + c), *dh = reinterpret_cast<uint4 *>(dst + half + c);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        dl[j] = make_uint4(olo[4 * j], olo[4 * j + 1], olo[4 * j + 2], olo[4 * j + 3]);
                        dh[j] = make_uint4(ohi[4 * j], ohi[4 * j + 1], ohi[4 * j + 2], ohi[4 * j + 3]);
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, QKV_BN);
    }
}


// ---------------------------------------------------------------------------------------
// Fast path: bf16 x and weights with ln_w already folded in (W'[n][k] = W[n][k] * ln_w[k]).
// Persistent CTAs (one per SM) walk the 128 x 256 output tiles; both operands arrive by TMA
// through a 4-stage ring; the f32 accumulator is double-buffered in TMEM (2 x 256 columns) so
// the epilogue of tile j overlaps the main loop of tile j+1.
//   warp 0      TMA loader (x tile 128 x 64, weight tile 256 x 64 per stage)
//   warp 1      tcgen05.mma issuer
//   warps 2-5, 10-13  epilogue (two warps per TMEM lane quarter, alternating heads):
//               TMEM -> RMSNorm factor -> RoPE -> transpose in shared memory -> q buffer / KV pages
//   warps 6-9   row statistics: read the x tile from shared memory, accumulate sum(x^2) per row
constexpr int QKVF_THREADS = 448;
constexpr int QKVF_STAGING = 8 * 4096;  // per epilogue warp: 2 pieces x 32 rows x 64 bytes

// PAIR: a cluster of two CTAs shares one 256 x 256 tile through tcgen05 cta_group::2; each CTA loads
// its own 128 rows of x and only half of the weight tile (half the shared-memory bytes per flop).
template <bool PAIR>
__device__ __forceinline__ void qkv_rope_tma_body(const CUtensorMap &x_map, const CUtensorMap &w_map, const QkvParams &p,
                                                  int tiles_m, int tiles_n, int nst) {
    constexpr int STAGE_BYTES = QKV_A_BYTES + (PAIR ? QKV_B_BYTES / 2 : QKV_B_BYTES);
    constexpr int TILE_M = PAIR ? 2 * QKV_BM : QKV_BM;
    const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
    // Every CTA (pair) walks a contiguous range of tiles; column tiles vary fastest, so consecutive tiles mostly
    // share their rows of x and the row statistics are computed once per row tile instead of once per tile.
    const int unit = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
    const int n_units = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
    extern __shared__ uint8_t qkvf_smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(qkvf_smem_raw) + 1023) &
                                                ~static_cast<uintptr_t>(1023));
    uint8_t *aux = smem + nst * STAGE_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(aux);
    uint64_t *full = bars, *empty = bars + 6;
    uint64_t *accum_full = bars + 12, *accum_empty = accum_full + 2;
    uint64_t *stats_full = accum_empty + 2, *stats_empty = stats_full + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(stats_empty + 2);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    float *stats = reinterpret_cast<float *>(aux + 256);   // [2][128]
    uint8_t *staging = aux + 256 + 1024;                   // [4 warps][2][32][64 B]
    float *rope_s = reinterpret_cast<float *>(staging + QKVF_STAGING);  // cos [half][S], sin [half][S]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ksteps = (p.H + QKV_BK - 1) / QKV_BK;
    const int n_tiles = tiles_m * tiles_n;
    const int t_begin = (int)((long long)n_tiles * unit / n_units), t_end = (int)((long long)n_tiles * (unit + 1) / n_units);
    const int half = p.hd >> 1;
    const WaitCtx wc{abort_flag, p.status};

    if (threadIdx.x == 0) {
        for (int i = 0; i < nst; ++i) {
            mbar_init(&full[i], (PAIR && rank == 0) ? 2 : 1);  // even CTA of a pair: + the odd CTA's "stage landed"
            mbar_init(&empty[i], 5);  // MMA commit + one arrive per statistics warp
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
    if (threadIdx.x == 0) {  // kernel parameters: independent of the previous kernel
        tma_prefetch_desc(&x_map);
        tma_prefetch_desc(&w_map);
    }
    pdl_launch_dependents();
    pdl_wait();  // the barrier set-up above overlapped the previous kernel's tail; global memory is read from here on
    // RoPE table, transposed so that lanes (consecutive tokens) read consecutive words
    for (int i = threadIdx.x; i < p.S * half; i += QKVF_THREADS) {
        const int t = i / half, d = i % half;
        rope_s[d * p.S + t] = p.rope_cos[i];
        rope_s[(half + d) * p.S + t] = p.rope_sin[i];
    }
    if (PAIR) {
        __syncthreads();
        cluster_sync_all();  // both CTAs' barriers exist before anything arrives on them remotely
    }
    if (warp == 1) {
        if (PAIR) {
            tmem_alloc_pair(tmem_slot, 512);
            tmem_relinquish_pair();
        } else {
            tmem_alloc(tmem_slot, 512);
            tmem_relinquish();
        }
    }
    tc_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync_all();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t st = 0, ph = 0;
            bool ok = true;
            for (int tile = t_begin; ok && tile < t_end; ++tile) {
                const int m0 = (tile / tiles_n) * TILE_M + (int)rank * QKV_BM;
                const int n0 = (tile % tiles_n) * QKV_BN + (int)rank * (QKV_BN / 2);
                for (int kt = 0; kt < ksteps; ++kt) {
                    ok = mbar_wait(&empty[st], ph ^ 1u, wc, DEV_TIMEOUT_EMPTY);
                    if (!ok) break;
                    mbar_expect_tx(&full[st], STAGE_BYTES);
                    uint8_t *sa = smem + st * STAGE_BYTES;
                    tma_load_2d(sa, &x_map, &full[st], kt * QKV_BK, m0);
                    tma_load_2d(sa + QKV_A_BYTES, &w_map, &full[st], kt * QKV_BK, n0);
                    if (++st == (uint32_t)nst) { st = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = make_idesc(1, 1, 1, 0, 0, TILE_M, QKV_BN);
            // descriptors differ between stages and k sub-steps only in the 14-bit start address
            const uint64_t a_desc0 = smem_desc_sw128(smem_u32(smem), 16, 1024);
            const uint64_t b_desc0 = smem_desc_sw128(smem_u32(smem + QKV_A_BYTES), 16, 1024);
            uint32_t st = 0, ph = 0, j = 0;
            bool ok = true;
            for (int tile = t_begin; ok && tile < t_end; ++tile, ++j) {
                const uint32_t buf = j & 1u;
                ok = mbar_wait(&accum_empty[buf], ((j >> 1) & 1u) ^ 1u, wc, DEV_TIMEOUT_EMPTY);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * QKV_BN;
                for (int kt = 0; kt < ksteps; ++kt) {
                    ok = mbar_wait(&full[st], ph, wc, DEV_TIMEOUT_FULL);
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t off = (uint64_t)(st * (STAGE_BYTES >> 4));
#pragma unroll
                    for (int k = 0; k < QKV_BK / 16; ++k) {
                        if (PAIR) mma_f16_pair(d_tmem, a_desc0 + off + 2 * k, b_desc0 + off + 2 * k, idesc, (kt | k) != 0 ? 1u : 0u);
                        else mma_f16(d_tmem, a_desc0 + off + 2 * k, b_desc0 + off + 2 * k, idesc, (kt | k) != 0 ? 1u : 0u);
                    }
                    if (PAIR) tc_commit_pair(&empty[st], 3);
                    else tc_commit(&empty[st]);
                    if (++st == (uint32_t)nst) { st = 0; ph ^= 1u; }
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
                    if (++st == (uint32_t)nst) { st = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp >= 6 && warp < 10) {
        // ---- row statistics: thread <-> row of the tile ----
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
            const bool fresh = mt != prev_mt;  // same rows of x as the previous tile: keep their sums
            prev_mt = mt;
            float s0 = 0.0f, s1 = 0.0f;
            for (int kt = 0; kt < ksteps; ++kt) {
                ok = mbar_wait(&full[st], ph, wc, DEV_TIMEOUT_FULL);
                if (!ok) break;
                if (fresh) {
                    const uint8_t *at = smem + st * STAGE_BYTES + row_base;
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        const uint4 v = *reinterpret_cast<const uint4 *>(at + ((c ^ sw) << 4));
                        const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&v);
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float2 f = __bfloat1622float2(h[e]);
                            s0 = fmaf(f.x, f.x, s0);
                            s1 = fmaf(f.y, f.y, s1);
                        }
                    }
                }
                stage_release(&empty[st], s0 + s1, lane);
                if (++st == (uint32_t)nst) { st = 0; ph ^= 1u; }
            }
            if (!ok) break;
            if (fresh) row_sum = s0 + s1;
            ok = mbar_wait(&stats_empty[buf], ((j >> 1) & 1u) ^ 1u, wc, DEV_TIMEOUT_EMPTY);
            if (!ok) break;
            stats[buf * 128 + row] = row_sum;
            mbar_arrive(&stats_full[buf]);
        }
    } else {
        // ---- epilogue warps 2..5 (group 0) and 10..13 (group 1) ----
        const int qtr = warp & 3;
        const int grp = warp >= 10 ? 1 : 0;
        const int row = qtr * 32 + lane;
        const int hd = p.hd;
        const int n_total = (p.n_q + 2 * p.n_kv_proj) * hd;
        uint8_t *stg = staging + (grp * 4 + qtr) * 4096;
        const uint32_t my_sw = (uint32_t)((lane >> 1) & 3);
        uint32_t j = 0;
        bool ok = true;
        for (int tile = t_begin; ok && tile < t_end; ++tile, ++j) {
            const uint32_t buf = j & 1u;
            const int m0 = (tile / tiles_n) * TILE_M + (int)rank * QKV_BM, n0 = (tile % tiles_n) * QKV_BN;
            const int m = m0 + row;
            const int tok = m % p.S;
            // the four rows this lane writes out after the transpose through shared memory
            int w_obs[4], w_tok[4];
            bool w_ok[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int mr = m0 + qtr * 32 + (lane >> 2) + 8 * i;
                w_ok[i] = mr < p.M;
                w_obs[i] = mr / p.S;
                w_tok[i] = mr % p.S;
            }
            ok = mbar_wait(&accum_full[buf], (j >> 1) & 1u, wc, DEV_TIMEOUT_ACCUM);
            if (ok) ok = mbar_wait(&stats_full[buf], (j >> 1) & 1u, wc, DEV_TIMEOUT_ACCUM);
            if (!ok) break;
            tc_fence_after();
            const float rms = p.eps < 0.0f ? 1.0f : rsqrtf(stats[buf * 128 + row] / (float)p.H + p.eps);
            const float *cs = rope_s + tok, *sn = rope_s + (size_t)half * p.S + tok;
            const uint32_t lane_addr = tmem_base + buf * QKV_BN + ((uint32_t)(qtr * 32) << 16);
            // heads of the tile alternate between the two groups; a single wide head is split by columns
            const int heads_in_tile = QKV_BN / hd;
            for (int hc = (heads_in_tile > 1 ? grp * hd : 0); hc < QKV_BN; hc += (heads_in_tile > 1 ? 2 * hd : hd)) {
                const int n = n0 + hc;
                if (n >= n_total) break;
                const int head = n / hd;
                bool rotate = true;
                __nv_bfloat16 *base;
                size_t obs_stride, tok0;  // element offsets: base + obs*obs_stride + (tok0 + tok)*hd
                if (head < p.n_q) {
                    base = p.q_out + (size_t)head * p.S * hd;
                    obs_stride = (size_t)p.n_q * p.S * hd;
                    tok0 = 0;
                } else {
                    const bool is_v = head >= p.n_q + p.n_kv_proj;
                    const int kvh = head - p.n_q - (is_v ? p.n_kv_proj : 0);
                    base = (is_v ? p.v_pages : p.k_pages) + (size_t)kvh * p.cap * hd;
                    obs_stride = (size_t)p.n_kv * p.cap * hd;
                    tok0 = (size_t)p.prefix_len;
                    rotate = !is_v;
                }
                for (int c = (heads_in_tile > 1 ? 0 : grp * 32); c < half; c += (heads_in_tile > 1 ? 32 : 64)) {
                    // 16 columns of each half per round: lo / hi / packed output stay within 48 registers
                    // (the kernel is capped at 128 and spilled with 32-column rounds)
                    uint8_t *mine = stg + lane * 64;
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        uint32_t lo[16], hi[16];
                        tmem_ld16(lane_addr + (uint32_t)(hc + c + hh * 16), lo);
                        tmem_ld16(lane_addr + (uint32_t)(hc + half + c + hh * 16), hi);
                        tmem_ld_wait();
                        uint32_t olo[8], ohi[8];
#pragma unroll
                        for (int e = 0; e < 16; e += 2) {
                            float a0 = __uint_as_float(lo[e]) * rms, a1 = __uint_as_float(lo[e + 1]) * rms;
                            float b0 = __uint_as_float(hi[e]) * rms, b1 = __uint_as_float(hi[e + 1]) * rms;
                            if (rotate) {
                                const int ce = c + hh * 16 + e;
                                const float c0 = cs[ce * p.S], c1 = cs[(ce + 1) * p.S];
                                const float s0 = sn[ce * p.S], s1 = sn[(ce + 1) * p.S];
                                const float r0 = a0 * c0 - b0 * s0, r1 = a1 * c1 - b1 * s1;
                                b0 = b0 * c0 + a0 * s0;
                                b1 = b1 * c1 + a1 * s1;
                                a0 = r0;
                                a1 = r1;
                            }
                            const __nv_bfloat162 l2 = __floats2bfloat162_rn(a0, a1), h2 = __floats2bfloat162_rn(b0, b1);
                            olo[e >> 1] = *reinterpret_cast<const uint32_t *>(&l2);
                            ohi[e >> 1] = *reinterpret_cast<const uint32_t *>(&h2);
                        }
                        // transpose through shared memory: thread-per-row -> 64 contiguous bytes per 4 lanes
#pragma unroll
                        for (int q2 = 0; q2 < 2; ++q2) {
                            const uint32_t q4 = (uint32_t)(hh * 2 + q2);
                            *reinterpret_cast<uint4 *>(mine + ((q4 ^ my_sw) << 4)) =
                                make_uint4(olo[4 * q2], olo[4 * q2 + 1], olo[4 * q2 + 2], olo[4 * q2 + 3]);
                            *reinterpret_cast<uint4 *>(mine + 2048 + ((q4 ^ my_sw) << 4)) =
                                make_uint4(ohi[4 * q2], ohi[4 * q2 + 1], ohi[4 * q2 + 2], ohi[4 * q2 + 3]);
                        }
                    }
                    __syncwarp();
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int rr = (lane >> 2) + 8 * i;
                        const uint32_t off = (uint32_t)rr * 64 + ((((uint32_t)lane & 3u) ^ (uint32_t)((rr >> 1) & 3)) << 4);
                        const uint4 vlo = *reinterpret_cast<const uint4 *>(stg + off);
                        const uint4 vhi = *reinterpret_cast<const uint4 *>(stg + 2048 + off);
                        if (w_ok[i]) {
                            __nv_bfloat16 *d = base + (size_t)w_obs[i] * obs_stride + (tok0 + w_tok[i]) * hd + (lane & 3) * 8;
                            *reinterpret_cast<uint4 *>(d + c) = vlo;
                            *reinterpret_cast<uint4 *>(d + half + c) = vhi;
                        }
                    }
                    __syncwarp();
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
            mbar_arrive(&stats_empty[buf]);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync_all();  // neither CTA may exit while the other can still signal its barriers
    if (warp == 1) {
        tc_fence_after();
        if (PAIR) tmem_dealloc_pair(tmem_base, 512);
        else tmem_dealloc(tmem_base, 512);
    }
}

__global__ void __launch_bounds__(QKVF_THREADS, 1)
qkv_rope_tma_kernel(const __grid_constant__ CUtensorMap x_map, const __grid_constant__ CUtensorMap w_map,
                    const QkvParams p, int tiles_m, int tiles_n, int nst) {
    qkv_rope_tma_body<false>(x_map, w_map, p, tiles_m, tiles_n, nst);
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(QKVF_THREADS, 1)
qkv_rope_tma_pair_kernel(const __grid_constant__ CUtensorMap x_map, const __grid_constant__ CUtensorMap w_map,
                         const QkvParams p, int tiles_m, int tiles_n, int nst) {
    qkv_rope_tma_body<true>(x_map, w_map, p, tiles_m, tiles_n, nst);
}


// W'[n][k] = bf16(W[n][k] * ln_w[k])
__global__ void fold_norm_weight_kernel(const __nv_bfloat16 *__restrict__ w, const float *__restrict__ ln_w,
                                        __nv_bfloat16 *__restrict__ out, size_t rows, int H) {
    const size_t total = rows * (size_t)H;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
        out[i] = __float2bfloat16(__bfloat162float(w[i]) * ln_w[i % H]);
}

// ---- prefix KV page writer: f32 [n_obs][P][n_kv][hd] -> bf16 pages [n_obs][n_kv][cap][hd] ----
// (the reference keeps the prefill's K/V as F32 graph tensors: src/models/pi0.cpp:172-194,
//  src/models/smolvla.cpp:793-794)
__global__ void __launch_bounds__(256) kv_store_write_kernel(const float *__restrict__ K, const float *__restrict__ V,
                                                             __nv_bfloat16 *__restrict__ kp,
                                                             __nv_bfloat16 *__restrict__ vp, int P, int n_kv, int hd,
                                                             int cap, size_t total_vec) {
    const int vec_per_row = hd >> 3;  // 8 elements per thread
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total_vec;
         i += (size_t)gridDim.x * blockDim.x) {
        const int v8 = (int)(i % vec_per_row);
        size_t r = i / vec_per_row;
        const int kvh = (int)(r % n_kv);
        r /= n_kv;
        const int tok = (int)(r % P);
        const size_t obs = r / P;
        const size_t src = ((obs * P + tok) * n_kv + kvh) * hd + (size_t)v8 * 8;
        const size_t dst = ((obs * n_kv + kvh) * cap + tok) * hd + (size_t)v8 * 8;
        auto conv = [](const float *s) {
            const float4 a = __ldg(reinterpret_cast<const float4 *>(s));
            const float4 b = __ldg(reinterpret_cast<const float4 *>(s) + 1);
            const __nv_bfloat162 h0 = __floats2bfloat162_rn(a.x, a.y), h1 = __floats2bfloat162_rn(a.z, a.w);
            const __nv_bfloat162 h2 = __floats2bfloat162_rn(b.x, b.y), h3 = __floats2bfloat162_rn(b.z, b.w);
            return make_uint4(*reinterpret_cast<const uint32_t *>(&h0), *reinterpret_cast<const uint32_t *>(&h1),
                              *reinterpret_cast<const uint32_t *>(&h2), *reinterpret_cast<const uint32_t *>(&h3));
        };
        *reinterpret_cast<uint4 *>(kp + dst) = conv(K + src);
        *reinterpret_cast<uint4 *>(vp + dst) = conv(V + src);
    }
}

__global__ void rope_table_kernel(float *cos_t, float *sin_t, int pos0, int S, int hd, float base) {
    const int half = hd >> 1;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= S * half) return;
    const int t = i / half, d = i % half;
    const float freq = powf(base, -2.0f * (float)d / (float)hd);
    const float ang = (float)(pos0 + t) * freq;
    cos_t[i] = cosf(ang);
    sin_t[i] = sinf(ang);
}

static size_t layer_stride_elems(const vlab200_kv_store *st) {
    return (size_t)st->n_obs * st->n_kv * st->cap * st->head_dim;
}

static int check_store(const vlab200_kv_store *st, int layer) {
    if (!st || !st->k_pages || !st->v_pages) return VLAB200_ERR_ARG;
    if (st->n_layers <= 0 || st->n_obs <= 0 || st->n_kv <= 0 || st->cap <= 0 || st->prefix_len < 0 ||
        st->prefix_len > st->cap)
        return VLAB200_ERR_ARG;
    if (layer < 0 || layer >= st->n_layers) return VLAB200_ERR_ARG;
    if (st->head_dim % 64 || st->head_dim > 256) return VLAB200_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(st->k_pages) & 15) || (reinterpret_cast<uintptr_t>(st->v_pages) & 15))
        return VLAB200_ERR_ARG;
    return VLAB200_OK;
}

}  // namespace vb

extern "C" {

int64_t vlab200_kv_store_bytes(int32_t n_layers, int32_t n_obs, int32_t n_kv, int32_t head_dim, int32_t cap) {
    if (n_layers <= 0 || n_obs <= 0 || n_kv <= 0 || head_dim <= 0 || cap <= 0) return -1;
    return (int64_t)n_layers * n_obs * n_kv * cap * head_dim * 2;
}

int32_t vlab200_kv_store_write(const vlab200_kv_store *st, int32_t layer, int32_t obs0, int32_t n_obs,
                               const float *K, const float *V, void *stream) {
    int rc = vb::check_store(st, layer);
    if (rc) return rc;
    if (!K || !V || obs0 < 0 || n_obs < 0 || obs0 + n_obs > st->n_obs) return VLAB200_ERR_ARG;
    if ((reinterpret_cast<uintptr_t>(K) & 15) || (reinterpret_cast<uintptr_t>(V) & 15)) return VLAB200_ERR_ARG;
    if (n_obs == 0 || st->prefix_len == 0) return VLAB200_OK;
    const size_t off = (size_t)layer * vb::layer_stride_elems(st) + (size_t)obs0 * st->n_kv * st->cap * st->head_dim;
    const size_t total_vec = (size_t)n_obs * st->prefix_len * st->n_kv * (st->head_dim / 8);
    const int blocks = (int)((total_vec + 255) / 256 < 148 * 16 ? (total_vec + 255) / 256 : 148 * 16);
    vb::kv_store_write_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        K, V, static_cast<__nv_bfloat16 *>(st->k_pages) + off, static_cast<__nv_bfloat16 *>(st->v_pages) + off,
        st->prefix_len, st->n_kv, st->head_dim, st->cap, total_vec);
    VB_CUDA(cudaGetLastError());
    return VLAB200_OK;
}

int32_t vlab200_rope_table(float *cos_out, float *sin_out, int32_t pos0, int32_t S, int32_t head_dim, float base,
                           void *stream) {
    if (!cos_out || !sin_out || S <= 0 || head_dim <= 0 || (head_dim & 1)) return VLAB200_ERR_ARG;
    const int n = S * (head_dim / 2);
    vb::rope_table_kernel<<<(n + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(cos_out, sin_out, pos0, S,
                                                                                         head_dim, base);
    VB_CUDA(cudaGetLastError());
    return VLAB200_OK;
}

int32_t vlab200_fold_norm_weight(const void *w_bf16, const float *ln_w, void *out_bf16, int64_t rows, int32_t H,
                                 void *stream) {
    if (!w_bf16 || !ln_w || !out_bf16 || rows <= 0 || H <= 0) return VLAB200_ERR_ARG;
    vb::fold_norm_weight_kernel<<<148 * 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16 *>(w_bf16), ln_w, static_cast<__nv_bfloat16 *>(out_bf16), (size_t)rows, H);
    VB_CUDA(cudaGetLastError());
    return VLAB200_OK;
}

int32_t vlab200_qkv_rope_append(const vlab200_kv_store *st, int32_t layer, const void *x, int32_t x_is_f32,
                                const float *ln_w, const void *wqkv_bf16, const float *rope_cos,
                                const float *rope_sin, float eps, int32_t S, int32_t H, int32_t n_q,
                                int32_t project_kv, void *q_out, void *stream) {
    int rc = vb::check_store(st, layer);
    if (rc) return rc;
    if (!x || !wqkv_bf16 || !rope_cos || !rope_sin || !q_out) return VLAB200_ERR_ARG;
    if (!ln_w && x_is_f32) return VLAB200_ERR_UNSUPPORTED;  // folded weights go with the bf16 TMA path
    if (S <= 0 || H <= 0 || n_q <= 0) return VLAB200_ERR_ARG;
    if (project_kv && st->prefix_len + S > st->cap) return VLAB200_ERR_ARG;
    if (H % 8 || H > 4096) return VLAB200_ERR_UNSUPPORTED;  // 16-byte rows; ln_w staged in shared memory
    if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(wqkv_bf16) & 15) ||
        (reinterpret_cast<uintptr_t>(q_out) & 15))
        return VLAB200_ERR_ARG;
    int *status = vb::device_status_ptr();
    if (!status) return vb::cuda_fail(cudaGetLastError(), "device_status_ptr");
    const int hd = st->head_dim;
    const int n_kv_proj = project_kv ? st->n_kv : 0;
    const int n_total = (n_q + 2 * n_kv_proj) * hd;
    const int M = st->n_obs * S;
    CUtensorMap wmap;
    const uint64_t dims[2] = {(uint64_t)H, (uint64_t)n_total};
    const uint64_t strides[1] = {(uint64_t)H * 2};
    const uint32_t box[2] = {vb::QKV_BK, vb::QKV_BN};
    rc = vb::make_tensor_map(&wmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, wqkv_bf16, dims, strides, box,
                             CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    vb::QkvParams p;
    p.x = x;
    p.ln_w = ln_w;
    p.rope_cos = rope_cos;
    p.rope_sin = rope_sin;
    p.q_out = static_cast<__nv_bfloat16 *>(q_out);
    const size_t off = (size_t)layer * vb::layer_stride_elems(st);
    p.k_pages = static_cast<__nv_bfloat16 *>(st->k_pages) + off;
    p.v_pages = static_cast<__nv_bfloat16 *>(st->v_pages) + off;
    p.M = M; p.H = H; p.S = S; p.hd = hd; p.n_q = n_q; p.n_kv_proj = n_kv_proj; p.n_kv = st->n_kv;
    p.cap = st->cap; p.prefix_len = st->prefix_len; p.eps = eps; p.status = status;
    const int ksteps = (H + vb::QKV_BK - 1) / vb::QKV_BK;
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    if (!ln_w) {
        // folded weights + bf16 x: persistent all-TMA kernel
        CUtensorMap xmap;
        const uint64_t xdims[2] = {(uint64_t)H, (uint64_t)M};
        const uint64_t xstrides[1] = {(uint64_t)H * 2};
        const uint32_t xbox[2] = {vb::QKV_BK, vb::QKV_BM};
        rc = vb::make_tensor_map(&xmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x, xdims, xstrides, xbox,
                                 CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc) return rc;
        // shared memory: stages + barriers/stats + store staging + transposed RoPE table
        const int aux = 256 + 1024 + vb::QKVF_STAGING + 2 * (hd / 2) * S * 4;
        if ((rc = vb::ensure_dyn_smem(vb::qkv_rope_tma_kernel, 227 * 1024))) return rc;
        if ((rc = vb::ensure_dyn_smem(vb::qkv_rope_tma_pair_kernel, 227 * 1024))) return rc;
        const int n_sm = vb::sm_count();
        if (n_sm <= 0) return vb::cuda_fail(cudaGetLastError(), "sm_count");
        const int tiles_m = (M + vb::QKV_BM - 1) / vb::QKV_BM, tiles_n = (n_total + vb::QKV_BN - 1) / vb::QKV_BN;
        const int tiles_mp = (M + 2 * vb::QKV_BM - 1) / (2 * vb::QKV_BM), pairs = n_sm / 2;
        // CTA pairs (256-row tiles) once they fill the machine at least as well as single CTAs do
        const int waves1 = (tiles_m * tiles_n + n_sm - 1) / n_sm;
        const int waves2 = pairs > 0 ? (tiles_mp * tiles_n + pairs - 1) / pairs : 1 << 30;
        const int variant = vb::dense_gemm_variant();
        const bool pair = variant == 3 || (variant == 0 && waves2 <= waves1 && tiles_mp * tiles_n >= pairs);
        if (pair) {
            const uint32_t wbox[2] = {vb::QKV_BK, vb::QKV_BN / 2};  // each CTA stages half of the weight tile
            const uint64_t wdims[2] = {(uint64_t)H, (uint64_t)n_total};
            const uint64_t wstrides[1] = {(uint64_t)H * 2};
            rc = vb::make_tensor_map(&wmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, wqkv_bf16, wdims, wstrides, wbox,
                                     CU_TENSOR_MAP_SWIZZLE_128B);
            if (rc) return rc;
            const int stage = vb::QKV_A_BYTES + vb::QKV_B_BYTES / 2;
            int nst = 6;
            while (nst > 2 && nst * stage + aux + 1024 > 227 * 1024) --nst;
            const int fsmem = nst * stage + aux + 1024;
            if (fsmem > 227 * 1024) return VLAB200_ERR_UNSUPPORTED;
            const int nt = tiles_mp * tiles_n;
            return vb::launch_pdl(vb::qkv_rope_tma_pair_kernel, dim3(2 * (nt < pairs ? nt : pairs)), dim3(vb::QKVF_THREADS), fsmem, cs,
                                  xmap, wmap, p, tiles_mp, tiles_n, nst);
        } else {
            int nst = 4;
            while (nst > 2 && nst * vb::QKV_STAGE_BYTES + aux + 1024 > 227 * 1024) --nst;
            const int fsmem = nst * vb::QKV_STAGE_BYTES + aux + 1024;
            if (fsmem > 227 * 1024) return VLAB200_ERR_UNSUPPORTED;
            const int nt = tiles_m * tiles_n;
            return vb::launch_pdl(vb::qkv_rope_tma_kernel, dim3(nt < n_sm ? nt : n_sm), dim3(vb::QKVF_THREADS), fsmem, cs, xmap, wmap,
                                  p, tiles_m, tiles_n, nst);
        }
        VB_CUDA(cudaGetLastError());
        return VLAB200_OK;
    }
    const int smem = vb::QKV_STAGES * vb::QKV_STAGE_BYTES + 256 + ksteps * vb::QKV_BK * 4 + 1024;
    dim3 grid((M + vb::QKV_BM - 1) / vb::QKV_BM, (n_total + vb::QKV_BN - 1) / vb::QKV_BN);
    if (x_is_f32) {
        if ((rc = vb::ensure_dyn_smem(vb::qkv_rope_kernel<true>, smem))) return rc;
        vb::qkv_rope_kernel<true><<<grid, vb::QKV_THREADS, smem, cs>>>(wmap, p);
    } else {
        if ((rc = vb::ensure_dyn_smem(vb::qkv_rope_kernel<false>, smem))) return rc;
        vb::qkv_rope_kernel<false><<<grid, vb::QKV_THREADS, smem, cs>>>(wmap, p);
    }
    VB_CUDA(cudaGetLastError());
    return VLAB200_OK;
}

}  // extern "C"

