// Action-query attention for wide heads / long prefixes (head_dim 128 or 256, any number of
// keys): the pi0-shaped case (8 q heads on 1 kv head, head_dim 256, 816 + 51 keys).
//
// Work unit = (kv head, observation, 128-row tile of the g*S stacked query rows).  Persistent
// CTAs walk the units; K and V pages stream through shared memory in 64-key blocks:
//
//   loader warp   TMA (SWIZZLE_128B): the Q tile once per unit, K / V blocks through 2-stage rings
//   MMA warp      S_j = Q K_j^T (kind::f16, f32 in TMEM, double-buffered), O += P_j V_j with
//                 A = P_j read from TMEM and V_j as an MN-major operand; S_{j+1} is issued
//                 before P_j V_j so the tensor pipe works while block j is in the softmax
//   4 softmax warps  one thread per row: block maximum, exp2 with the scale folded in, running
//                 row sum; P_j (bf16) overwrites S_j in TMEM.  The running maximum is only raised
//                 (and O rescaled through TMEM) when a block exceeds it by more than 2^8, which
//                 keeps P within bf16 range without touching O in the common case.
//
// Reference: src/models/pi0.cpp:204-223 (explicit K^T Q -> soft_max_ext -> V P with the score
// matrix and two permuted copies of K/V in HBM every layer-step), mask src/models/pi0.cpp:640-651.
#include <cuda_bf16.h>

#include "gemm.h"
#include "host_common.h"
#include "tc5.cuh"

namespace vb {

constexpr int FA_THREADS = 192;  // warps 0-3 softmax/epilogue, 4 loader, 5 MMA
constexpr int FA_BKV = 64;       // keys per block

struct FlashParams {
    __nv_bfloat16 *out;  // [n_obs][S][n_q*hd]
    const int32_t *pad;
    int S, n_q, n_kv, g, kv_len, prefix_len, mask_mode, R, n_mt, n_units, n_blocks, page0;
    float scale_log2;
    int out_al32;  // out is 32-byte aligned: 256-bit stores
    int *status;
    // key-split mode (few work units): a unit's key blocks are cut into n_split slices that run as separate work items;
    // a slice leaves its un-normalised O rows, running maximum and row sum in the workspace for attn_split_combine_kernel
    int n_split;
    float *ws_o;   // [n_units * n_split][128][HD]
    float *ws_ml;  // [n_units * n_split][128][2]: maximum (log2 units), row sum
};

__device__ __forceinline__ float fa_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]),
        "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]),
        "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

template <int HD>
struct FlashSmem {
    static constexpr int CB = HD / 64;                   // 64-element column blocks
    static constexpr int Q_BYTES = CB * 128 * 128;       // [CB][128 rows][128 B]
    static constexpr int KV_BYTES = CB * FA_BKV * 128;   // [CB][64 keys][128 B]
    static constexpr int K_OFF = Q_BYTES, V_OFF = Q_BYTES + 2 * KV_BYTES;
    static constexpr int BAR_OFF = Q_BYTES + 4 * KV_BYTES;
    static constexpr int TOTAL = BAR_OFF + 256 + 1024;
    static constexpr int O_COLS = HD;                    // O [0, HD), S buffers at HD, HD + 64
    static constexpr int TMEM_COLS = (HD + 128 <= 256) ? 256 : 512;
};

template <int HD, bool SPLIT = false>
__global__ void __launch_bounds__(FA_THREADS, HD == 64 ? 2 : 1)
attn_flash_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
                  const __grid_constant__ CUtensorMap v_map, const FlashParams p) {
    using L = FlashSmem<HD>;
    extern __shared__ uint8_t fa_smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(fa_smem_raw) + 1023) &
                                                ~static_cast<uintptr_t>(1023));
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + L::BAR_OFF);
    uint64_t *q_full = bars, *q_free = bars + 1, *o_done = bars + 2, *o_free = bars + 3;
    uint64_t *k_full = bars + 4, *k_free = bars + 6, *v_full = bars + 8, *v_free = bars + 10;
    uint64_t *s_full = bars + 12, *p_full = bars + 14, *pv_done = bars + 16;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 18);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const WaitCtx wc{abort_flag, p.status};
    const int nb = p.n_blocks;
    const int ns = SPLIT ? p.n_split : 1;  // key slices per unit
    const int n_work = p.n_units * ns;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        mbar_init(q_free, 1);
        mbar_init(o_done, 1);
        mbar_init(o_free, 128);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&k_full[i], 1);
            mbar_init(&k_free[i], 1);
            mbar_init(&v_full[i], 1);
            mbar_init(&v_free[i], 1);
            mbar_init(&s_full[i], 1);
            mbar_init(&p_full[i], 128);
            mbar_init(&pv_done[i], 1);
        }
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 5) {
        tmem_alloc(tmem_slot, L::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (threadIdx.x == 0) {  // kernel parameters: independent of the previous kernel
        tma_prefetch_desc(&q_map);
        tma_prefetch_desc(&k_map);
        tma_prefetch_desc(&v_map);
    }
    pdl_launch_dependents();
    pdl_wait();  // everything above overlapped the previous kernel's tail; global memory is touched below

    if (warp == 4) {
        // ----------------------------------------------------------------- loader
        if (lane == 0) {
            uint32_t ui = 0, jb = 0;  // units and key blocks processed so far by this CTA
            bool ok = true;
            for (int wu = blockIdx.x; ok && wu < n_work; wu += gridDim.x, ++ui) {
                const int unit = SPLIT ? wu / ns : wu, sp = SPLIT ? wu % ns : 0;
                const int j0 = SPLIT ? sp * nb / ns : 0, j1 = SPLIT ? (sp + 1) * nb / ns : nb;
                const int item = unit / p.n_mt, mt = unit % p.n_mt;
                const int obs = item / p.n_kv, kvh = item % p.n_kv;
                const int page = p.page0 + item;
                const int qrow0 = (obs * p.n_q + kvh * p.g) * p.S + mt * 128;
                ok = mbar_wait(q_free, (ui & 1u) ^ 1u, wc, DEV_TIMEOUT_EMPTY);
                if (!ok) break;
                mbar_expect_tx(q_full, L::Q_BYTES);
                for (int cb = 0; cb < L::CB; ++cb) tma_load_2d(smem + cb * 16384, &q_map, q_full, cb * 64, qrow0);
                for (int j = j0; j < j1; ++j, ++jb) {
                    const int st = jb & 1;
                    const uint32_t ph = (jb >> 1) & 1u;
                    ok = mbar_wait(&k_free[st], ph ^ 1u, wc, DEV_TIMEOUT_EMPTY);
                    if (!ok) break;
                    mbar_expect_tx(&k_full[st], L::KV_BYTES);
                    for (int cb = 0; cb < L::CB; ++cb)
                        tma_load_3d(smem + L::K_OFF + st * L::KV_BYTES + cb * 8192, &k_map, &k_full[st], cb * 64,
                                    j * FA_BKV, page);
                    ok = mbar_wait(&v_free[st], ph ^ 1u, wc, DEV_TIMEOUT_EMPTY);
                    if (!ok) break;
                    mbar_expect_tx(&v_full[st], L::KV_BYTES);
                    for (int cb = 0; cb < L::CB; ++cb)
                        tma_load_3d(smem + L::V_OFF + st * L::KV_BYTES + cb * 8192, &v_map, &v_full[st], cb * 64,
                                    j * FA_BKV, page);
                }
            }
        }
    } else if (warp == 5) {
        // ----------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_s = make_idesc(1, 1, 1, 0, 0, 128, FA_BKV);
            constexpr uint32_t idesc_o = make_idesc(1, 1, 1, 0, 1, 128, HD);
            const uint32_t q_addr = smem_u32(smem);
            const uint32_t k_base = q_addr + L::K_OFF, v_base = q_addr + L::V_OFF;
            uint32_t ui = 0, jb = 0;
            bool ok = true;
            auto issue_s = [&](uint32_t jbx) {  // S block with global block counter jbx
                const uint32_t st = jbx & 1u;
                const uint32_t k_addr = k_base + st * L::KV_BYTES;
                const uint32_t d = tmem_base + L::O_COLS + st * 64;
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk)
                    mma_f16(d, smem_desc_sw128(q_addr + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024),
                            smem_desc_sw128(k_addr + (kk >> 2) * 8192 + (kk & 3) * 32, 16, 1024), idesc_s,
                            kk != 0 ? 1u : 0u);
                tc_commit(&s_full[st]);
                tc_commit(&k_free[st]);
            };
            for (int wu = blockIdx.x; ok && wu < n_work; wu += gridDim.x, ++ui) {
                const int sp = SPLIT ? wu % ns : 0;
                const int j0 = SPLIT ? sp * nb / ns : 0, j1 = SPLIT ? (sp + 1) * nb / ns : nb;
                ok = mbar_wait(q_full, ui & 1u, wc, DEV_TIMEOUT_FULL);
                if (!ok) break;
                // first S block of the unit: its TMEM buffer was last read by the P V of block jb-2, which this thread
                // issued earlier -- the tensor pipe runs a thread's MMAs in issue order, so there is nothing to wait for
                ok = mbar_wait(&k_full[jb & 1u], (jb >> 1) & 1u, wc, DEV_TIMEOUT_FULL);
                if (!ok) break;
                tc_fence_after();
                issue_s(jb);
                if (j1 - j0 == 1) tc_commit(q_free);
                for (int j = j0; j < j1; ++j, ++jb) {
                    const uint32_t st = jb & 1u, ph = (jb >> 1) & 1u;
                    if (j + 1 < j1) {
                        const uint32_t jn = jb + 1;
                        ok = mbar_wait(&k_full[jn & 1u], (jn >> 1) & 1u, wc, DEV_TIMEOUT_FULL);
                        if (!ok) break;
                        tc_fence_after();
                        issue_s(jn);
                        if (j + 2 == j1) tc_commit(q_free);  // the unit's last S block has been issued
                    }
                    ok = mbar_wait(&p_full[st], ph, wc, DEV_TIMEOUT_FULL);
                    if (ok) ok = mbar_wait(&v_full[st], ph, wc, DEV_TIMEOUT_FULL);
                    if (ok && j == j0) ok = mbar_wait(o_free, (ui & 1u) ^ 1u, wc, DEV_TIMEOUT_EMPTY);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t v_addr = v_base + st * L::KV_BYTES;
                    const uint32_t p_tmem = tmem_base + L::O_COLS + st * 64;
#pragma unroll
                    for (int k16 = 0; k16 < FA_BKV / 16; ++k16)
                        mma_f16_tmem_a(tmem_base, p_tmem + (uint32_t)(k16 * 8),
                                       smem_desc_sw128(v_addr + k16 * 2048, 8192, 1024), idesc_o,
                                       (j != j0 || k16 != 0) ? 1u : 0u);
                    tc_commit(&pv_done[st]);
                    tc_commit(&v_free[st]);
                }
                if (!ok) break;
                tc_commit(o_done);
            }
        }
    } else {
        // ----------------------------------------------------------------- softmax / epilogue
        const int qtr = warp;
        const uint32_t lane_sel = (uint32_t)(qtr * 32) << 16;
        const int n_suffix_cols = p.kv_len - p.prefix_len;
        uint32_t ui = 0, jb = 0;
        bool ok = true;
        for (int wu = blockIdx.x; ok && wu < n_work; wu += gridDim.x, ++ui) {
            const int unit = SPLIT ? wu / ns : wu, sp = SPLIT ? wu % ns : 0;
            const int j0 = SPLIT ? sp * nb / ns : 0, j1 = SPLIT ? (sp + 1) * nb / ns : nb;
            const int item = unit / p.n_mt, mt = unit % p.n_mt;
            const int obs = item / p.n_kv, kvh = item % p.n_kv;
            const int row = mt * 128 + qtr * 32 + lane;
            const bool row_ok = row < p.R;
            const int head_l = row_ok ? row / p.S : 0, tok = row_ok ? row % p.S : 0;
            int pad_lo = 0, pad_hi = 0;
            if (p.pad) {
                pad_lo = p.pad[2 * obs];
                pad_hi = p.pad[2 * obs + 1];
            }
            int limit = n_suffix_cols;
            if (p.mask_mode == 2) limit = min(tok + 1, n_suffix_cols);
            else if (p.mask_mode == 1) limit = tok == 0 ? min(1, n_suffix_cols) : n_suffix_cols;
            else if (p.mask_mode == 3) limit = tok == p.S - 1 ? n_suffix_cols : n_suffix_cols - 1;
            const int jmax = p.prefix_len + limit;
            int clean_end = p.prefix_len;
            if (pad_hi > pad_lo) clean_end = min(clean_end, pad_lo);
            const int pad_w = pad_hi - pad_lo;
            float m_used = -INFINITY;  // running maximum in log2 units (lazy)
            float l_sum = 0.0f;
            for (int j = j0; j < j1; ++j, ++jb) {
                const uint32_t st = jb & 1u, ph = (jb >> 1) & 1u;
                const uint32_t s_addr = tmem_base + L::O_COLS + st * 64 + lane_sel;
                ok = mbar_wait(&s_full[st], ph, wc, DEV_TIMEOUT_FULL);
                if (!ok) break;
                tc_fence_after();
                uint32_t sa[32], sb[32];
                tmem_ld32(s_addr, sa);
                tmem_ld32(s_addr + 32, sb);
                tmem_ld_wait();
                const int c0 = j * FA_BKV;
                const bool clean = c0 + FA_BKV <= clean_end;
                if (!clean) {
                    const int rel_jmax = jmax - c0, rel_pad = pad_lo - c0;
                    if (pad_w <= 0) {  // the usual case (no hidden range in this unit): one comparison per column
#pragma unroll
                        for (int e = 0; e < 32; ++e) {
                            sa[e] = e < rel_jmax ? sa[e] : 0xff800000u;
                            sb[e] = e + 32 < rel_jmax ? sb[e] : 0xff800000u;
                        }
                    } else {
#pragma unroll
                        for (int e = 0; e < 32; ++e) {
                            const bool v0 = e < rel_jmax && !((unsigned)(e - rel_pad) < (unsigned)pad_w);
                            const bool v1 = e + 32 < rel_jmax && !((unsigned)(e + 32 - rel_pad) < (unsigned)pad_w);
                            sa[e] = v0 ? sa[e] : 0xff800000u;
                            sb[e] = v1 ? sb[e] : 0xff800000u;
                        }
                    }
                }
                float t[8];
#pragma unroll
                for (int e = 0; e < 8; ++e)
                    t[e] = fmaxf(fmaxf(fmaxf(__uint_as_float(sa[4 * e]), __uint_as_float(sa[4 * e + 1])),
                                       fmaxf(__uint_as_float(sa[4 * e + 2]), __uint_as_float(sa[4 * e + 3]))),
                                 fmaxf(fmaxf(__uint_as_float(sb[4 * e]), __uint_as_float(sb[4 * e + 1])),
                                       fmaxf(__uint_as_float(sb[4 * e + 2]), __uint_as_float(sb[4 * e + 3]))));
                const float bm = fmaxf(fmaxf(fmaxf(t[0], t[1]), fmaxf(t[2], t[3])),
                                       fmaxf(fmaxf(t[4], t[5]), fmaxf(t[6], t[7]))) * p.scale_log2;
                // raise the running maximum only when a block exceeds it by more than 2^8
                float factor = 1.0f;
                const bool raise = bm > m_used + 8.0f;
                if (raise) {
                    factor = (m_used == -INFINITY) ? 0.0f : fa_ex2(m_used - bm);
                    m_used = bm;
                    l_sum *= factor;
                }
                if (j > j0 && __any_sync(0xffffffffu, raise)) {
                    // O holds contributions scaled with the old maximum: rescale it in TMEM once the
                    // previous block's P V has landed
                    const uint32_t jp = jb - 1;
                    ok = mbar_wait(&pv_done[jp & 1u], (jp >> 1) & 1u, wc, DEV_TIMEOUT_ACCUM);
                    if (!ok) break;
                    tc_fence_after();
                    for (int c = 0; c < HD; c += 32) {
                        uint32_t ov[32];
                        tmem_ld32(tmem_base + lane_sel + (uint32_t)c, ov);
                        tmem_ld_wait();
#pragma unroll
                        for (int e = 0; e < 32; ++e) ov[e] = __float_as_uint(__uint_as_float(ov[e]) * factor);
                        tmem_st32(tmem_base + lane_sel + (uint32_t)c, ov);
                    }
                    tmem_st_wait();
                }
                const float mref = (m_used == -INFINITY) ? 0.0f : m_used;
                uint32_t pk[32];
                float s0 = 0.0f, s1 = 0.0f;
#pragma unroll
                for (int e = 0; e < 32; e += 2) {
                    const float p0 = fa_ex2(fmaf(__uint_as_float(sa[e]), p.scale_log2, -mref));
                    const float p1 = fa_ex2(fmaf(__uint_as_float(sa[e + 1]), p.scale_log2, -mref));
                    const float p2 = fa_ex2(fmaf(__uint_as_float(sb[e]), p.scale_log2, -mref));
                    const float p3 = fa_ex2(fmaf(__uint_as_float(sb[e + 1]), p.scale_log2, -mref));
                    s0 += p0 + p2;
                    s1 += p1 + p3;
                    pk[e >> 1] = __byte_perm(__float_as_uint(p0) + 0x8000u, __float_as_uint(p1) + 0x8000u, 0x7632);
                    pk[16 + (e >> 1)] = __byte_perm(__float_as_uint(p2) + 0x8000u, __float_as_uint(p3) + 0x8000u, 0x7632);
                }
                l_sum += s0 + s1;
                tmem_st32(s_addr, pk);  // P_j (64 keys, bf16) over the first 32 columns of S_j
                tmem_st_wait();
                tc_fence_before();
                mbar_arrive(&p_full[st]);
            }
            if (!ok) break;
            // ---- epilogue: O / l -> bf16 -> out ----
            ok = mbar_wait(o_done, ui & 1u, wc, DEV_TIMEOUT_ACCUM);
            if (!ok) break;
            tc_fence_after();
            if constexpr (SPLIT) {
                // this slice's un-normalised rows and their (maximum, sum): attn_split_combine_kernel merges the slices
                const size_t wrow = (size_t)wu * 128 + qtr * 32 + lane;
                float4 *wo = reinterpret_cast<float4 *>(p.ws_o + wrow * HD);
                for (int c = 0; c < HD; c += 32) {
                    uint32_t ov[32];
                    tmem_ld32(tmem_base + lane_sel + (uint32_t)c, ov);
                    tmem_ld_wait();
                    if (row_ok) {
#pragma unroll
                        for (int e = 0; e < 8; ++e)
                            wo[(c >> 2) + e] = make_float4(__uint_as_float(ov[4 * e]), __uint_as_float(ov[4 * e + 1]),
                                                           __uint_as_float(ov[4 * e + 2]), __uint_as_float(ov[4 * e + 3]));
                    }
                }
                if (row_ok) *reinterpret_cast<float2 *>(p.ws_ml + wrow * 2) = make_float2(m_used, l_sum);
                tc_fence_before();
                mbar_arrive(o_free);
                continue;
            }
            const float inv = 1.0f / l_sum;
            __nv_bfloat16 *dst = p.out + ((size_t)obs * p.S + tok) * ((size_t)p.n_q * HD) + (size_t)(kvh * p.g + head_l) * HD;
            for (int c = 0; c < HD; c += 32) {
                uint32_t ov[32];
                tmem_ld32(tmem_base + lane_sel + (uint32_t)c, ov);
                tmem_ld_wait();
                if (row_ok) {
#pragma unroll
                    for (int q8 = 0; q8 < 2; ++q8) {
                        uint32_t w[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(ov[16 * q8 + 2 * e]) * inv,
                                                                           __uint_as_float(ov[16 * q8 + 2 * e + 1]) * inv);
                            w[e] = *reinterpret_cast<const uint32_t *>(&h);
                        }
                        if (p.out_al32) {  // one full 32-byte sector per store instruction and thread
                            st_global_v8(dst + c + 16 * q8, w);
                        } else {
                            uint4 *d4 = reinterpret_cast<uint4 *>(dst + c + 16 * q8);
                            d4[0] = make_uint4(w[0], w[1], w[2], w[3]);
                            d4[1] = make_uint4(w[4], w[5], w[6], w[7]);
                        }
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(o_free);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 5) {
        tc_fence_after();
        tmem_dealloc(tmem_base, L::TMEM_COLS);
    }
}

// ------------------------------------------------------------------ CTA pairs --
// The same algorithm on clusters of two CTAs (tcgen05 cta_group::2, M = 256): the pair works on two
// 128-row tiles of ONE item, so a K / V block is fetched once per pair -- each CTA stages half of it
// (K: 32 of the block's 64 keys, V: half of the head dimension) -- and one MMA instruction serves both
// row tiles.  That halves the L2 -> SM traffic per row (the single-CTA kernel re-streams K / V for every
// row tile and was at the L2 bandwidth the GEMMs also meet) and the MMA instructions per row (a thread
// issues at most one tcgen05.mma every ~64 cycles, twice the duration of an N = 64 MMA).  Rings are 4
// deep.  The even CTA issues; commits are multicast to both CTAs; the odd CTA's MMA warp forwards "my
// Q tile / K half / V half has landed", its softmax warps arrive on the even CTA's p_full / o_free.
constexpr int FP_BKV = 128;   // keys per block: 16 Q K^T MMAs (N = 128) serve twice the keys of the one-CTA kernel's N = 64
constexpr int FP_THREADS = 352;  // warps 0-7 softmax (quarter = warp & 3, column half = warp >> 2), 8 loader, 9 Q K^T issuer, 10 P V issuer
constexpr int FP_LOADER_WARP = 8, FP_MMA_WARP = 9, FP_PV_WARP = 10;

template <int HD>
struct FlashPairSmem {
    static constexpr int STAGES = HD == 256 ? 2 : 4;   // K / V ring depth (what fits beside the Q tile)
    static constexpr int NS = (512 - HD) / FP_BKV;     // S / P buffers of 128 TMEM columns behind O: Q K^T runs NS - 1 blocks ahead
    static constexpr int CB = HD / 64;                 // 64-element column blocks of the head dimension
    static constexpr int CBH = HD / 128;               // column blocks of V this CTA stages
    static constexpr int Q_BYTES = CB * 128 * 128;     // [CB][128 rows][128 B]
    static constexpr int K_BYTES = CB * (FP_BKV / 2) * 128;  // [CB][64 keys][128 B]: this CTA's half of the block's keys
    static constexpr int V_BYTES = CBH * FP_BKV * 128;       // [CBH][128 keys][128 B]: this CTA's half of the head dimension
    static constexpr int K_OFF = Q_BYTES, V_OFF = K_OFF + STAGES * K_BYTES;
    static constexpr int BAR_OFF = V_OFF + STAGES * V_BYTES;
    static constexpr int XCH_OFF = BAR_OFF + 512;      // float [2 halves][128 rows] block maxima, then row sums, then the maxima of odd blocks
    static constexpr int TOTAL = XCH_OFF + 3072 + 1024;
    static constexpr int O_COLS = HD;
    static constexpr int TMEM_COLS = 512;              // O [0, HD), then NS S buffers of 128 columns
    static_assert(HD + NS * FP_BKV <= 512 && NS >= 2, "TMEM");
};

__device__ __forceinline__ void mma_f16_tmem_a_pair(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc,
                                                    uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

template <int HD>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(FP_THREADS, 1)
attn_flash_pair_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
                       const __grid_constant__ CUtensorMap v_map, const FlashParams p) {
    using L = FlashPairSmem<HD>;
    constexpr int FP_STAGES = L::STAGES, FP_NS = L::NS;
    extern __shared__ uint8_t fa_smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(fa_smem_raw) + 1023) &
                                                ~static_cast<uintptr_t>(1023));
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + L::BAR_OFF);
    uint64_t *q_full = bars, *q_free = bars + 1, *o_done = bars + 2, *o_free = bars + 3;
    uint64_t *k_full = bars + 4, *k_free = bars + 8, *v_full = bars + 12, *v_free = bars + 16;  // [FP_STAGES]
    uint64_t *s_full = bars + 20, *p_full = bars + 24, *pv_done = bars + 28;                    // [FP_NS]
    uint64_t *pair_bar = bars + 32;  // [4] the two softmax warps of a lane quarter meet here (64 arrivals)
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 36);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    volatile uint32_t *pv_issued = reinterpret_cast<volatile uint32_t *>(tmem_slot + 2);  // P V blocks issued so far (even CTA)

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int cid = blockIdx.x >> 1, ncl = gridDim.x >> 1;
    const WaitCtx wc{abort_flag, p.status};
    const int nb = (p.kv_len + FP_BKV - 1) / FP_BKV;
    const int n_mt2 = (p.n_mt + 1) >> 1;                 // pairs of row tiles per item
    const int n_units = (p.n_units / p.n_mt) * n_mt2;    // (item, tile pair)
    const uint32_t both = rank == 0 ? 2u : 1u;           // even CTA: own TMA + the odd CTA's forward

    if (threadIdx.x == 0) {
        mbar_init(q_full, both);
        mbar_init(q_free, 1);
        mbar_init(o_done, 1);
        mbar_init(o_free, 16);  // one arrival per softmax warp of both CTAs (used in the even CTA)
        for (int i = 0; i < 4; ++i) mbar_init(&pair_bar[i], 64);
        for (int i = 0; i < FP_STAGES; ++i) {
            mbar_init(&k_full[i], both);
            mbar_init(&k_free[i], 1);
            mbar_init(&v_full[i], both);
            mbar_init(&v_free[i], 1);
        }
        for (int i = 0; i < FP_NS; ++i) {
            mbar_init(&s_full[i], 1);
            mbar_init(&p_full[i], 16);
            mbar_init(&pv_done[i], 1);
        }
        *abort_flag = 0;
        *pv_issued = 0;
        fence_barrier_init();
    }
    __syncthreads();
    cluster_sync_all();  // both CTAs' barriers exist before anything arrives on them remotely
    if (warp == FP_MMA_WARP) {
        tmem_alloc_pair(tmem_slot, L::TMEM_COLS);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (threadIdx.x == 0) {  // kernel parameters: independent of the previous kernel
        tma_prefetch_desc(&q_map);
        tma_prefetch_desc(&k_map);
        tma_prefetch_desc(&v_map);
    }
    pdl_launch_dependents();
    pdl_wait();  // everything above overlapped the previous kernel's tail; global memory is touched below

    if (warp == FP_LOADER_WARP) {
        // ----------------------------------------------------------------- loader (each CTA its own halves)
        if (lane == 0) {
            uint32_t ui = 0, jb = 0;
            bool ok = true;
            for (int unit = cid; ok && unit < n_units; unit += ncl, ++ui) {
                const int item = unit / n_mt2, mt = (unit % n_mt2) * 2 + (int)rank;
                const int obs = item / p.n_kv, kvh = item % p.n_kv;
                const int page = p.page0 + item;
                const int qrow0 = (obs * p.n_q + kvh * p.g) * p.S + mt * 128;
                ok = mbar_wait(q_free, (ui & 1u) ^ 1u, wc, DEV_TIMEOUT_EMPTY);
                if (!ok) break;
                mbar_expect_tx(q_full, L::Q_BYTES);
                for (int cb = 0; cb < L::CB; ++cb) tma_load_2d(smem + cb * 16384, &q_map, q_full, cb * 64, qrow0);
                for (int j = 0; j < nb; ++j, ++jb) {
                    const int st = jb % FP_STAGES;
                    const uint32_t ph = (jb / FP_STAGES) & 1u;
                    ok = mbar_wait(&k_free[st], ph ^ 1u, wc, DEV_TIMEOUT_EMPTY);
                    if (!ok) break;
                    mbar_expect_tx(&k_full[st], L::K_BYTES);
                    for (int cb = 0; cb < L::CB; ++cb)
                        tma_load_3d(smem + L::K_OFF + st * L::K_BYTES + cb * 8192, &k_map, &k_full[st], cb * 64,
                                    j * FP_BKV + (int)rank * (FP_BKV / 2), page);
                    ok = mbar_wait(&v_free[st], ph ^ 1u, wc, DEV_TIMEOUT_EMPTY);
                    if (!ok) break;
                    mbar_expect_tx(&v_full[st], L::V_BYTES);
                    for (int cb = 0; cb < L::CBH; ++cb)
                        tma_load_3d(smem + L::V_OFF + st * L::V_BYTES + cb * (FP_BKV * 128), &v_map, &v_full[st],
                                    ((int)rank * L::CBH + cb) * 64, j * FP_BKV, page);
                }
            }
        }
    } else if (warp == FP_MMA_WARP) {
        if (lane == 0 && rank == 0) {
            // ------------------------------------------------------------- MMA issuer (even CTA)
            constexpr uint32_t idesc_s = make_idesc(1, 1, 1, 0, 0, 256, FP_BKV);
            const uint32_t q_addr = smem_u32(smem);
            const uint64_t q_desc0 = smem_desc_sw128(q_addr, 16, 1024);
            const uint64_t k_desc0 = smem_desc_sw128(q_addr + L::K_OFF, 16, 1024);
            uint32_t ui = 0, jb = 0;
            bool ok = true;
            auto issue_s = [&](uint32_t jbx) {  // S block with global block counter jbx
                const uint32_t st = jbx % FP_STAGES;
                const uint64_t k_desc = k_desc0 + (uint64_t)(st * (L::K_BYTES >> 4));
                const uint32_t d = tmem_base + L::O_COLS + (jbx % FP_NS) * FP_BKV;
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk)
                    mma_f16_pair(d, q_desc0 + (uint64_t)((kk >> 2) * 1024 + (kk & 3) * 2),
                                 k_desc + (uint64_t)((kk >> 2) * 512 + (kk & 3) * 2), idesc_s, kk != 0 ? 1u : 0u);
                tc_commit_pair(&s_full[jbx % FP_NS], 3);
                tc_commit_pair(&k_free[st], 3);
            };
            // S block jbx may be issued once its K half-blocks have landed and the P V of the block that
            // used the same TMEM buffer (jbx - FP_NS) has finished.  This thread issues only the Q K^T MMAs
            // (16 per block, the longer stream); the P V MMAs come from a thread of their own (warp
            // FP_PV_WARP): one thread issuing both spent ~2500 cycles per block, twice the tensor time.
            // It does not wait for that P V block to COMPLETE: the tensor pipe takes the MMAs of a CTA pair in the order
            // they were issued, so it is enough that the P V thread has issued them (a counter in shared memory that
            // it bumps after its last MMA of a block).  Waiting for the commit instead kept the pipe idle for the
            // ~500 cycles between the block's last MMA and the moment this thread saw the barrier flip.
            auto ready_s = [&](uint32_t jbx) -> bool {
                bool r = mbar_wait(&k_full[jbx % FP_STAGES], (jbx / FP_STAGES) & 1u, wc, DEV_TIMEOUT_FULL);
                if (r && jbx >= FP_NS && *pv_issued < jbx - FP_NS + 1u) {
                    const long long t0 = clock64();
                    for (uint32_t it = 1; *pv_issued < jbx - FP_NS + 1u; ++it) {
                        if ((it & 63u) == 0) {
                            if (*abort_flag) return false;
                            if (clock64() - t0 > wc.budget) {
                                *abort_flag = 1;
                                atomicCAS(p.status, 0, (int)DEV_TIMEOUT_FULL);
                                return false;
                            }
                        }
                    }
                }
                return r;
            };
            for (int unit = cid; ok && unit < n_units; unit += ncl, ++ui) {
                ok = mbar_wait(q_full, ui & 1u, wc, DEV_TIMEOUT_FULL);
                if (!ok) break;
                for (int j = 0; j < nb; ++j, ++jb) {
                    ok = ready_s(jb);
                    if (!ok) break;
                    tc_fence_after();
                    issue_s(jb);
                }
                if (!ok) break;
                tc_commit_pair(q_free, 3);  // the unit's last S block has been issued
            }
        } else if (lane == 0) {
            // ------------------------------------------------------------- odd CTA: forward "landed" to the even CTA
            uint32_t ui = 0, jb = 0;
            bool ok = true;
            for (int unit = cid; ok && unit < n_units; unit += ncl, ++ui) {
                ok = mbar_wait(q_full, ui & 1u, wc, DEV_TIMEOUT_FULL);
                if (!ok) break;
                mbar_arrive_cluster(q_full, 0);
                for (int j = 0; j < nb; ++j, ++jb) {
                    const uint32_t st = jb % FP_STAGES, ph = (jb / FP_STAGES) & 1u;
                    ok = mbar_wait(&k_full[st], ph, wc, DEV_TIMEOUT_FULL);
                    if (!ok) break;
                    mbar_arrive_cluster(&k_full[st], 0);
                    ok = mbar_wait(&v_full[st], ph, wc, DEV_TIMEOUT_FULL);
                    if (!ok) break;
                    mbar_arrive_cluster(&v_full[st], 0);
                }
            }
        }
    } else if (warp == FP_PV_WARP) {
        if (lane == 0 && rank == 0) {
            // ------------------------------------------------------------- P V issuer (even CTA)
            constexpr uint32_t idesc_o = make_idesc(1, 1, 1, 0, 1, 256, HD);
            const uint64_t v_desc0 = smem_desc_sw128(smem_u32(smem) + L::V_OFF, FP_BKV * 128, 1024);
            uint32_t ui = 0, jb = 0;
            bool ok = true;
            for (int unit = cid; ok && unit < n_units; unit += ncl, ++ui) {
                for (int j = 0; j < nb; ++j, ++jb) {
                    const uint32_t sb = jb % FP_NS, sph = (jb / FP_NS) & 1u;         // S / P buffer and its phase
                    const uint32_t st = jb % FP_STAGES, ph = (jb / FP_STAGES) & 1u;  // K / V stage and its phase
                    ok = mbar_wait(&p_full[sb], sph, wc, DEV_TIMEOUT_FULL);
                    if (ok) ok = mbar_wait(&v_full[st], ph, wc, DEV_TIMEOUT_FULL);
                    if (ok && j == 0) ok = mbar_wait(o_free, (ui & 1u) ^ 1u, wc, DEV_TIMEOUT_EMPTY);
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t v_desc = v_desc0 + (uint64_t)(st * (L::V_BYTES >> 4));
                    const uint32_t p_tmem = tmem_base + L::O_COLS + sb * FP_BKV;
#pragma unroll
                    for (int k16 = 0; k16 < FP_BKV / 16; ++k16)
                        mma_f16_tmem_a_pair(tmem_base, p_tmem + (uint32_t)(k16 * 8), v_desc + (uint64_t)(k16 * 128), idesc_o,
                                            (j | k16) != 0 ? 1u : 0u);
                    *pv_issued = jb + 1u;
                    tc_commit_pair(&pv_done[sb], 3);
                    tc_commit_pair(&v_free[st], 3);
                }
                if (!ok) break;
                tc_commit_pair(o_done, 3);
            }
        }
    } else {
        // ----------------------------------------------------------------- softmax / epilogue (own row tile)
        // Two warps per TMEM lane quarter: warp `half` takes 32 of a block's 64 key columns of its rows (one
        // row per lane), half of the O columns when O is rescaled and half of them in the epilogue.  The two
        // exchange block maxima and row sums through shared memory; their meeting (an mbarrier, so that the
        // wait is bounded) also orders half 1's P store over columns that half 0 has just read.
        const int qtr = warp & 3, half = warp >> 2;
        const uint32_t lane_sel = (uint32_t)(qtr * 32) << 16;
        float *xch = reinterpret_cast<float *>(smem + L::XCH_OFF);
        const int my_slot = qtr * 32 + lane;
        uint32_t pair_n = 0;
        auto pair_sync = [&]() -> bool {
            mbar_arrive(&pair_bar[qtr]);
            return mbar_wait(&pair_bar[qtr], (pair_n++) & 1u, wc, DEV_TIMEOUT_MISC);
        };
        const int n_suffix_cols = p.kv_len - p.prefix_len;
        auto arrive_even = [&](uint64_t *bar) {  // one arrival per warp on the even CTA's barrier
            __syncwarp();
            if (lane == 0) {
                if (rank == 0) mbar_arrive(bar);
                else mbar_arrive_cluster(bar, 0);
            }
        };
        // The O drain of a unit runs AFTER the first S block of the next unit: that block only needs its S buffer, and the
        // ~2000 cycles between a unit's last P and "O complete" (its last P V) are spent on it instead of on waiting.
        auto drain = [&](uint32_t u, float l_mine, __nv_bfloat16 *dst, bool row_ok) -> bool {
            xch[256 + half * 128 + my_slot] = l_mine;
            if (!mbar_wait(o_done, u & 1u, wc, DEV_TIMEOUT_ACCUM)) return false;
            tc_fence_after();
            if (!pair_sync()) return false;
            const float inv = 1.0f / (l_mine + xch[256 + (half ^ 1) * 128 + my_slot]);
            for (int c = half * (HD / 2); c < (half + 1) * (HD / 2); c += 32) {
                uint32_t ov[32];
                tmem_ld32(tmem_base + lane_sel + (uint32_t)c, ov);
                tmem_ld_wait();
                if (c + 32 >= (half + 1) * (HD / 2)) {  // O is out of TMEM: the next unit's P V may start while the last stores go out
                    tc_fence_before();
                    arrive_even(o_free);
                }
                if (row_ok) {
#pragma unroll
                    for (int q8 = 0; q8 < 2; ++q8) {
                        uint32_t w[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(ov[16 * q8 + 2 * e]) * inv,
                                                                           __uint_as_float(ov[16 * q8 + 2 * e + 1]) * inv);
                            w[e] = *reinterpret_cast<const uint32_t *>(&h);
                        }
                        if (p.out_al32) {  // one full 32-byte sector per store instruction and thread
                            st_global_v8(dst + c + 16 * q8, w);
                        } else {
                            uint4 *d4 = reinterpret_cast<uint4 *>(dst + c + 16 * q8);
                            d4[0] = make_uint4(w[0], w[1], w[2], w[3]);
                            d4[1] = make_uint4(w[4], w[5], w[6], w[7]);
                        }
                    }
                }
            }
            // (the row-sum slots are next written after at least two more meetings of the pair)
            return true;
        };
        uint32_t ui = 0, jb = 0;
        bool ok = true;
        float prev_l = 0.0f;  // the unit whose O is still to be drained
        __nv_bfloat16 *prev_dst = nullptr;
        bool prev_row_ok = false;
        int pad_lo = 0, pad_hi = 0;  // of the unit about to start (read one unit ahead: a global-memory round trip)
        if (p.pad && cid < n_units) {
            const int obs0 = (cid / n_mt2) / p.n_kv;
            pad_lo = p.pad[2 * obs0];
            pad_hi = p.pad[2 * obs0 + 1];
        }
        for (int unit = cid; ok && unit < n_units; unit += ncl, ++ui) {
            const int item = unit / n_mt2, mt = (unit % n_mt2) * 2 + (int)rank;
            const int obs = item / p.n_kv, kvh = item % p.n_kv;
            const int row = mt * 128 + qtr * 32 + lane;
            const bool row_ok = row < p.R;
            const int head_l = row_ok ? row / p.S : 0, tok = row_ok ? row % p.S : 0;
            int pad_lo_n = 0, pad_hi_n = 0;
            if (p.pad && unit + ncl < n_units) {
                const int obs_n = ((unit + ncl) / n_mt2) / p.n_kv;
                pad_lo_n = p.pad[2 * obs_n];
                pad_hi_n = p.pad[2 * obs_n + 1];
            }
            int limit = n_suffix_cols;
            if (p.mask_mode == 2) limit = min(tok + 1, n_suffix_cols);
            else if (p.mask_mode == 1) limit = tok == 0 ? min(1, n_suffix_cols) : n_suffix_cols;
            else if (p.mask_mode == 3) limit = tok == p.S - 1 ? n_suffix_cols : n_suffix_cols - 1;
            const int jmax = p.prefix_len + limit;
            int clean_end = p.prefix_len;
            if (pad_hi > pad_lo) clean_end = min(clean_end, pad_lo);
            const int pad_w = pad_hi - pad_lo;
            float m_used = -INFINITY;  // running maximum in log2 units (lazy), identical in both halves
            float l_sum = 0.0f;        // this half's part of the row sum
            for (int j = 0; j < nb; ++j, ++jb) {
                const uint32_t sb = jb % FP_NS, sph = (jb / FP_NS) & 1u;
                const uint32_t s_addr = tmem_base + L::O_COLS + sb * FP_BKV + lane_sel;
                ok = mbar_wait(&s_full[sb], sph, wc, DEV_TIMEOUT_FULL);
                if (!ok) break;
                tc_fence_after();
                uint32_t sa[32], sc[32];  // this half's 64 of the block's 128 key columns
                tmem_ld32(s_addr + (uint32_t)(half * 64), sa);
                tmem_ld32(s_addr + (uint32_t)(half * 64 + 32), sc);
                tmem_ld_wait();
                const int c0 = j * FP_BKV + half * 64;
                const bool clean = j * FP_BKV + FP_BKV <= clean_end;
                if (!clean) {
                    const int rel_jmax = jmax - c0, rel_pad = pad_lo - c0;
                    if (pad_w <= 0) {  // the usual case (no hidden range in this unit): one comparison per column
#pragma unroll
                        for (int e = 0; e < 32; ++e) {
                            sa[e] = e < rel_jmax ? sa[e] : 0xff800000u;
                            sc[e] = e + 32 < rel_jmax ? sc[e] : 0xff800000u;
                        }
                    } else {
#pragma unroll
                        for (int e = 0; e < 32; ++e) {
                            const bool v0 = e < rel_jmax && !((unsigned)(e - rel_pad) < (unsigned)pad_w);
                            const bool v1 = e + 32 < rel_jmax && !((unsigned)(e + 32 - rel_pad) < (unsigned)pad_w);
                            sa[e] = v0 ? sa[e] : 0xff800000u;
                            sc[e] = v1 ? sc[e] : 0xff800000u;
                        }
                    }
                }
                float t[8];
#pragma unroll
                for (int e = 0; e < 8; ++e)
                    t[e] = fmaxf(fmaxf(fmaxf(__uint_as_float(sa[4 * e]), __uint_as_float(sa[4 * e + 1])),
                                       fmaxf(__uint_as_float(sa[4 * e + 2]), __uint_as_float(sa[4 * e + 3]))),
                                 fmaxf(fmaxf(__uint_as_float(sc[4 * e]), __uint_as_float(sc[4 * e + 1])),
                                       fmaxf(__uint_as_float(sc[4 * e + 2]), __uint_as_float(sc[4 * e + 3]))));
                float bm = fmaxf(fmaxf(fmaxf(t[0], t[1]), fmaxf(t[2], t[3])), fmaxf(fmaxf(t[4], t[5]), fmaxf(t[6], t[7])));
                float *xm = xch + (jb & 1u) * 512;  // two sets of slots, used in turn: one meeting per block is enough
                xm[half * 128 + my_slot] = bm;
                ok = pair_sync();
                if (!ok) break;
                bm = fmaxf(bm, xm[(half ^ 1) * 128 + my_slot]) * p.scale_log2;
                float factor = 1.0f;
                const bool raise = bm > m_used + 8.0f;
                if (raise) {
                    factor = (m_used == -INFINITY) ? 0.0f : fa_ex2(m_used - bm);
                    m_used = bm;
                    l_sum *= factor;
                }
                if (j > 0 && __any_sync(0xffffffffu, raise)) {
                    const uint32_t jp = jb - 1;
                    ok = mbar_wait(&pv_done[jp % FP_NS], (jp / FP_NS) & 1u, wc, DEV_TIMEOUT_ACCUM);
                    if (!ok) break;
                    tc_fence_after();
                    // not unrolled: unrolling this loop pushed the kernel over its 168-register cap (spills)
#pragma unroll 1
            for (int c = half * (HD / 2); c < (half + 1) * (HD / 2); c += 32) {
                        uint32_t ov[32];
                        tmem_ld32(tmem_base + lane_sel + (uint32_t)c, ov);
                        tmem_ld_wait();
#pragma unroll
                        for (int e = 0; e < 32; ++e) ov[e] = __float_as_uint(__uint_as_float(ov[e]) * factor);
                        tmem_st32(tmem_base + lane_sel + (uint32_t)c, ov);
                    }
                    tmem_st_wait();
                }
                const float mref = (m_used == -INFINITY) ? 0.0f : m_used;
                uint32_t pk[32];
                float s0 = 0.0f, s1 = 0.0f;
#pragma unroll
                for (int e = 0; e < 32; e += 2) {
                    const float p0 = fa_ex2(fmaf(__uint_as_float(sa[e]), p.scale_log2, -mref));
                    const float p1 = fa_ex2(fmaf(__uint_as_float(sa[e + 1]), p.scale_log2, -mref));
                    const float p2 = fa_ex2(fmaf(__uint_as_float(sc[e]), p.scale_log2, -mref));
                    const float p3 = fa_ex2(fmaf(__uint_as_float(sc[e + 1]), p.scale_log2, -mref));
                    s0 += p0 + p2;
                    s1 += p1 + p3;
                    pk[e >> 1] = __byte_perm(__float_as_uint(p0) + 0x8000u, __float_as_uint(p1) + 0x8000u, 0x7632);
                    pk[16 + (e >> 1)] = __byte_perm(__float_as_uint(p2) + 0x8000u, __float_as_uint(p3) + 0x8000u, 0x7632);
                }
                l_sum += s0 + s1;
                tmem_st32(s_addr + (uint32_t)(half * 32), pk);  // P_j (128 keys, bf16) over the first 64 columns of S_j
                tmem_st_wait();
                tc_fence_before();
                arrive_even(&p_full[sb]);
                if (j == 0 && ui > 0) {
                    ok = drain(ui - 1, prev_l, prev_dst, prev_row_ok);
                    if (!ok) {
                        ++jb;
                        break;
                    }
                }
            }
            if (!ok) break;
            // ---- O / l -> bf16 -> out (each half stores half of the head dimension): after the next unit's first block ----
            prev_l = l_sum;
            prev_dst = p.out + ((size_t)obs * p.S + tok) * ((size_t)p.n_q * HD) + (size_t)(kvh * p.g + head_l) * HD;
            prev_row_ok = row_ok;
            pad_lo = pad_lo_n;
            pad_hi = pad_hi_n;
        }
        if (ok && ui > 0) ok = drain(ui - 1, prev_l, prev_dst, prev_row_ok);
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // neither CTA may exit while the other can still signal its barriers
    if (warp == FP_MMA_WARP) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, L::TMEM_COLS);
    }
}

// Merges the key slices of every (unit, row): M = max_s m_s; O = sum_s O_s 2^(m_s - M); l = sum_s l_s 2^(m_s - M);
// out = bf16(O / l), slices in order.  One warp per row, HD / 32 columns per lane.
template <int HD>
__global__ void __launch_bounds__(256) attn_split_combine_kernel(const FlashParams p) {
    pdl_launch_dependents();
    pdl_wait();
    const int warp_g = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (warp_g >= p.n_units * 128) return;
    const int unit = warp_g >> 7, r = warp_g & 127;
    const int item = unit / p.n_mt, mt = unit % p.n_mt;
    const int obs = item / p.n_kv, kvh = item % p.n_kv;
    const int row = mt * 128 + r;
    if (row >= p.R) return;
    const int head_l = row / p.S, tok = row % p.S;
    float M = -INFINITY;
    for (int s = 0; s < p.n_split; ++s) M = fmaxf(M, p.ws_ml[(((size_t)unit * p.n_split + s) * 128 + r) * 2]);
    float acc[HD / 32];
#pragma unroll
    for (int i = 0; i < HD / 32; ++i) acc[i] = 0.0f;
    float l = 0.0f;
    for (int s = 0; s < p.n_split; ++s) {
        const size_t wrow = ((size_t)unit * p.n_split + s) * 128 + r;
        const float2 ml = *reinterpret_cast<const float2 *>(p.ws_ml + wrow * 2);
        const float w = ml.x == -INFINITY ? 0.0f : fa_ex2(ml.x - M);
        l = fmaf(ml.y, w, l);
#pragma unroll
        for (int i = 0; i < HD / 32; ++i) acc[i] = fmaf(p.ws_o[wrow * HD + i * 32 + lane], w, acc[i]);
    }
    const float inv = 1.0f / l;
    __nv_bfloat16 *dst = p.out + ((size_t)obs * p.S + tok) * ((size_t)p.n_q * HD) + (size_t)(kvh * p.g + head_l) * HD;
#pragma unroll
    for (int i = 0; i < HD / 32; ++i) dst[i * 32 + lane] = __float2bfloat16(acc[i] * inv);
}

template <int HD>
static int launch_flash(const vlab200_kv_store *st, int layer, const void *q, void *out, int S, int n_q, int kv_len,
                        int mask_mode, const int32_t *pad_ranges, cudaStream_t stream, float softmax_scale, float *ws,
                        size_t ws_bytes) {
    using L = FlashSmem<HD>;
    int *status = device_status_ptr();
    if (!status) return cuda_fail(cudaGetLastError(), "device_status_ptr");
    CUtensorMap qmap, kmap, vmap;
    {
        const uint64_t dims[2] = {(uint64_t)HD, (uint64_t)st->n_obs * n_q * S};
        const uint64_t strides[1] = {(uint64_t)HD * 2};
        const uint32_t box[2] = {64, 128};
        int rc = make_tensor_map(&qmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, q, dims, strides, box,
                                 CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc) return rc;
    }
    {
        // rows >= kv_len are outside the map: TMA zero-fills them
        const uint64_t dims[3] = {(uint64_t)HD, (uint64_t)kv_len, (uint64_t)st->n_layers * st->n_obs * st->n_kv};
        const uint64_t strides[2] = {(uint64_t)HD * 2, (uint64_t)st->cap * HD * 2};
        const uint32_t box[3] = {64, FA_BKV, 1};
        int rc = make_tensor_map(&kmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, st->k_pages, dims, strides, box,
                                 CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc) return rc;
        rc = make_tensor_map(&vmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, st->v_pages, dims, strides, box,
                             CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc) return rc;
    }
    FlashParams p;
    p.out = static_cast<__nv_bfloat16 *>(out);
    p.pad = pad_ranges;
    p.S = S; p.n_q = n_q; p.n_kv = st->n_kv; p.g = n_q / st->n_kv; p.kv_len = kv_len; p.prefix_len = st->prefix_len;
    p.mask_mode = mask_mode;
    p.R = p.g * S;
    p.n_mt = (p.R + 127) / 128;
    p.n_units = st->n_obs * st->n_kv * p.n_mt;
    p.n_blocks = (kv_len + FA_BKV - 1) / FA_BKV;
    p.page0 = layer * st->n_obs * st->n_kv;
    // softmax_scale > 0 replaces 1 / sqrt(HD): heads narrower than HD that were zero-padded to it
    p.scale_log2 = 1.4426950408889634f * (softmax_scale > 0.0f ? softmax_scale : 1.0f / sqrtf((float)HD));
    p.out_al32 = (reinterpret_cast<uintptr_t>(out) & 31) == 0 ? 1 : 0;
    p.status = status;
    const int n_sm = sm_count();
    if constexpr (HD >= 128) {
        // CTA pairs once an item has two row tiles and the pairs fill the machine (or when forced for tests)
        const int n_pair_units = st->n_obs * st->n_kv * ((p.n_mt + 1) / 2), pairs = n_sm / 2;
        const int forced = dense_gemm_variant();
        if (p.n_mt >= 2 && forced != 1 && (forced == 3 || n_pair_units >= pairs)) {
            using LP = FlashPairSmem<HD>;
            // each CTA stages 64 of a block's 128 keys (the one-CTA kernel's K map has that box) and, for V, all
            // 128 keys of half of the head dimension
            CUtensorMap vmap128;
            const uint64_t dims[3] = {(uint64_t)HD, (uint64_t)kv_len, (uint64_t)st->n_layers * st->n_obs * st->n_kv};
            const uint64_t strides[2] = {(uint64_t)HD * 2, (uint64_t)st->cap * HD * 2};
            const uint32_t box[3] = {64, FP_BKV, 1};
            int rc = make_tensor_map(&vmap128, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, st->v_pages, dims, strides, box,
                                     CU_TENSOR_MAP_SWIZZLE_128B);
            if (rc) return rc;
            if ((rc = ensure_dyn_smem(attn_flash_pair_kernel<HD>, LP::TOTAL))) return rc;
            const int ncl = n_pair_units < pairs ? n_pair_units : pairs;
            return launch_pdl(attn_flash_pair_kernel<HD>, dim3(2 * ncl), dim3(FP_THREADS), LP::TOTAL, stream, qmap, kmap, vmap128, p);
        }
    }
    p.n_split = 1;
    if (ws && p.n_units * 2 <= n_sm && p.n_blocks >= 4) {
        // few units (one observation): cut every unit's keys into slices of at least two 64-key blocks so that the slices fill
        // the machine, then merge them (flash-decoding)
        int n_split = n_sm / p.n_units;
        if (n_split > p.n_blocks / 2) n_split = p.n_blocks / 2;  // two to four blocks per slice measured alike, one slower
        const size_t need = (size_t)p.n_units * n_split * 128 * (HD + 2) * sizeof(float);
        if (n_split >= 2 && need <= ws_bytes) {
            p.n_split = n_split;
            p.ws_o = ws;
            p.ws_ml = ws + (size_t)p.n_units * n_split * 128 * HD;
            if (int rc = ensure_dyn_smem(attn_flash_kernel<HD, true>, L::TOTAL)) return rc;
            if (int rc = launch_pdl(attn_flash_kernel<HD, true>, dim3(p.n_units * n_split), dim3(FA_THREADS), L::TOTAL, stream, qmap, kmap,
                                    vmap, p))
                return rc;
            return launch_pdl(attn_split_combine_kernel<HD>, dim3((p.n_units * 128 + 7) / 8), dim3(256), 0, stream, p);
        }
    }
    if (int rc = ensure_dyn_smem(attn_flash_kernel<HD>, L::TOTAL)) return rc;
    const int slots = (HD == 64 ? 2 : 1) * n_sm;  // head_dim 64: two CTAs share an SM (256 TMEM columns, 50 KB each)
    const int grid = p.n_units < slots ? p.n_units : slots;
    return launch_pdl(attn_flash_kernel<HD>, dim3(grid), dim3(FA_THREADS), L::TOTAL, stream, qmap, kmap, vmap, p);
}

int attention_flash(const vlab200_kv_store *st, int layer, const void *q, void *out, int S, int n_q, int kv_len,
                    int mask_mode, const int32_t *pad_ranges, cudaStream_t stream, float softmax_scale, float *ws,
                    size_t ws_bytes) {
    if (st->head_dim == 256)
        return launch_flash<256>(st, layer, q, out, S, n_q, kv_len, mask_mode, pad_ranges, stream, softmax_scale, ws, ws_bytes);
    if (st->head_dim == 128)
        return launch_flash<128>(st, layer, q, out, S, n_q, kv_len, mask_mode, pad_ranges, stream, softmax_scale, ws, ws_bytes);
    if (st->head_dim == 64)
        return launch_flash<64>(st, layer, q, out, S, n_q, kv_len, mask_mode, pad_ranges, stream, softmax_scale, ws, ws_bytes);
    return VLAB200_ERR_UNSUPPORTED;
}

}  // namespace vb
