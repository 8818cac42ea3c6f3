// Action-query attention over the prefix + suffix KV pages (head_dim 64, up to 256 keys).
//
// Persistent kernel, one CTA per SM, looping over work items (kv head, observation) of one
// layer.  The g = n_q / n_kv query heads that share a kv head are stacked into one block of
// R = g*S rows (GQA/MQA head sharing: K and V are fetched once for all of them) and processed
// as 128-row tcgen05 tiles.
//
//   loader warp   TMA (SWIZZLE_128B): Q rows, K page, V page of the next items into 2-deep rings
//                 while the current ones compute (pages are read from HBM exactly once)
//   2 MMA warps   one per TMEM region (items alternate between the two regions):
//                 S = Q K^T (kind::f16, f32 accumulator, all keys at once), then O = P V with
//                 A = P read from TMEM and V as an MN-major operand
//   2 x 8 softmax warps (per region two warps per TMEM lane quarter, one per half of the key
//                 columns): one thread per (row, column half), straight out of TMEM, exp2 with the
//                 scale folded in, masks applied as selects; P (bf16) overwrites consumed S columns.
//                 More than 128 keys: ONE pass per half with a lazily raised reference, an O
//                 accumulator per half, the halves merged in the epilogue.  Fewer keys: two passes
//                 (maximum, then exp2), the halves exchange row maximum and row sum through shared
//                 memory.  Epilogue O / rowsum -> bf16
//
// TMEM region (256 columns): S [0, nk16) in nchunks chunks of 32 columns, the first n_a of them
// owned by column half A.  P (bf16, 16 columns per chunk) overwrites columns its own half has
// already consumed: half A at [0, 16 n_a), half B at [32 n_a, 32 n_a + 16 (nchunks - n_a)); O (64
// columns) follows the P of half A (n_a >= 4) or of half B.
//
// Reference: src/layers/attn.h:38-46, src/models/pi0.cpp:204-223 (mul_mat -> soft_max -> mul_mat
// with the score matrix in HBM), src/models/smolvla.cpp:835-842,874-881 (ggml_flash_attn_ext);
// masks src/models/pi0.cpp:640-651, smolvla.cpp:1655-1664.
#include <cuda_bf16.h>

#include <cstdlib>

#include "host_common.h"
#include "tc5.cuh"

namespace vb {

// streaming kernel for wide heads / long key ranges (attn_flash.cu)
int attention_flash(const vlab200_kv_store *st, int layer, const void *q, void *out, int S, int n_q, int kv_len,
                    int mask_mode, const int32_t *pad_ranges, cudaStream_t stream, float softmax_scale = 0.0f,
                    float *ws = nullptr, size_t ws_bytes = 0);

constexpr int ATT_SOFTMAX_WARPS = 16;
constexpr int ATT_THREADS = (ATT_SOFTMAX_WARPS + 3) * 32;  // + loader + 2 MMA issuers
constexpr int ATT_MAX_KEYS = 256;
constexpr int ATT_Q_TILE_BYTES = 128 * 128;
constexpr int ATT_KV_BYTES = ATT_MAX_KEYS * 128;
constexpr int ATT_QK_BYTES = 2 * ATT_Q_TILE_BYTES + ATT_KV_BYTES;  // Q0, Q1, K of one item
constexpr int ATT_SMEM_DATA = 2 * ATT_QK_BYTES + 2 * ATT_KV_BYTES;  // two Q/K buffers, two V buffers
constexpr int ATT_REGION_COLS = 256;

struct AttnParams {
    __nv_bfloat16 *out;  // [n_obs][S][n_q*hd]
    const int32_t *pad;  // [n_obs][2] masked prefix columns, or null
    int S, n_q, n_kv, g, kv_len, prefix_len, mask_mode, nk16, R, n_items, page0;
    int t1_rows;   // rows of the second 128-row tile (0: none)
    int out_al32;  // 1: out is 32-byte aligned (256-bit stores)
    int t1_rot;    // 1: t1_rows <= 32, its rows are placed in TMEM quarter (item ordinal % 4)
    float scale_log2;
    int *status;
};


__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ void region_sync(int r) {  // the 256 softmax threads of region r
    asm volatile("bar.sync %0, 256;" ::"r"(r + 1) : "memory");
}

// Per-row mask description: columns [0, jmax) minus [pad_lo, pad_hi) are visible; columns below
// clean_end need no test in any lane of the warp.
struct RowMask {
    int jmax, pad_lo, pad_hi, clean_end;
};

__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// Visibility of the 32 columns of chunk c as a bit mask (bit j = column c*32 + j is visible).
__device__ __forceinline__ uint32_t low_bits(int n) {  // bits [0, n), n clamped to [0, 32]
    return n >= 32 ? 0xffffffffu : (n <= 0 ? 0u : ((1u << n) - 1u));
}
__device__ __forceinline__ uint32_t att_vis_bits(int c, const RowMask &rm) {
    const uint32_t below_jmax = low_bits(rm.jmax - c * 32);
    const uint32_t pad = low_bits(rm.pad_hi - c * 32) & ~low_bits(rm.pad_lo - c * 32);
    return below_jmax & ~pad;
}
// Visibility is applied to the INPUT of max / exp2 (a select to -inf), never as a branch around
// them, so lanes with different row limits stay converged.
__device__ __forceinline__ float att_masked(uint32_t bits, int j, uint32_t vis) {
    return (vis & (1u << j)) ? __uint_as_float(bits) : -INFINITY;
}

__device__ __forceinline__ void att_max_chunk(const uint32_t (&sv)[32], int c, const RowMask &rm, float (&mx)[4]) {
    if (c * 32 + 32 <= rm.clean_end) {
        float t[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
            t[j] = max3(__uint_as_float(sv[4 * j]), __uint_as_float(sv[4 * j + 1]),
                        fmaxf(__uint_as_float(sv[4 * j + 2]), __uint_as_float(sv[4 * j + 3])));
        mx[0] = max3(mx[0], t[0], t[1]);
        mx[1] = max3(mx[1], t[2], t[3]);
        mx[2] = max3(mx[2], t[4], t[5]);
        mx[3] = max3(mx[3], t[6], t[7]);
    } else {
        const uint32_t vis = att_vis_bits(c, rm);
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
            mx[0] = max3(mx[0], att_masked(sv[j], j, vis),
                         att_masked(sv[j + 1], j + 1, vis));
            mx[1] = max3(mx[1], att_masked(sv[j + 2], j + 2, vis),
                         att_masked(sv[j + 3], j + 3, vis));
            mx[2] = max3(mx[2], att_masked(sv[j + 4], j + 4, vis),
                         att_masked(sv[j + 5], j + 5, vis));
            mx[3] = max3(mx[3], att_masked(sv[j + 6], j + 6, vis),
                         att_masked(sv[j + 7], j + 7, vis));
        }
    }
}

// p = exp2(s*c - m*c) for one 32-column chunk; P (bf16) is stored over consumed S columns.  bf16
// rounding uses integer adds (round-half-up on the magnitude; p >= 0).
__device__ __forceinline__ void att_exp_chunk(const uint32_t (&sv)[32], int c, const RowMask &rm, float scale_log2,
                                              float m2, float &sum0, float &sum1, uint32_t p_addr) {
    uint32_t pk[16];
    if (c * 32 + 32 <= rm.clean_end) {
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
            const float p0 = ex2_approx(fmaf(__uint_as_float(sv[j]), scale_log2, -m2));
            const float p1 = ex2_approx(fmaf(__uint_as_float(sv[j + 1]), scale_log2, -m2));
            sum0 += p0;
            sum1 += p1;
            pk[j >> 1] = __byte_perm(__float_as_uint(p0) + 0x8000u, __float_as_uint(p1) + 0x8000u, 0x7632);
        }
    } else {
        const uint32_t vis = att_vis_bits(c, rm);
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
            // exp2(-inf) = 0 for the masked columns
            const float p0 = ex2_approx(fmaf(att_masked(sv[j], j, vis), scale_log2, -m2));
            const float p1 =
                ex2_approx(fmaf(att_masked(sv[j + 1], j + 1, vis), scale_log2, -m2));
            sum0 += p0;
            sum1 += p1;
            pk[j >> 1] = __byte_perm(__float_as_uint(p0) + 0x8000u, __float_as_uint(p1) + 0x8000u, 0x7632);
        }
    }
    tmem_st16(p_addr, pk);
}

// SP (single pass, key ranges of more than 128 keys): the two column halves of a row are independent softmax problems.
// Each walks its chunks ONCE with a lazily raised reference (the first chunk's maximum; raised, with the P chunks already
// written rescaled in TMEM, only when a later chunk exceeds it by more than 2^8), P V of each half accumulates into an O of
// its own (columns 64.. and 192.., both inside consumed S columns: n_a is 4), and the epilogue merges the two like two key
// slices.  This removes the maximum pass over S (a second round of TMEM loads) and the exchange in the middle of a unit.
template <bool SP>
__global__ void __launch_bounds__(ATT_THREADS, 1)
attn_hd64_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap q_map32,
                 const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                 const AttnParams p) {
    extern __shared__ uint8_t att_smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(att_smem_raw) + 1023) &
                                                ~static_cast<uintptr_t>(1023));
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + ATT_SMEM_DATA);
    uint64_t *full_qk = bars, *full_v = bars + 2, *free_qk = bars + 4, *free_v = bars + 6;    // per buffer
    uint64_t *bar_s = bars + 8, *bar_o = bars + 10, *bar_free = bars + 12;  // per region
    uint64_t *bar_p = bars + 14;                                            // per region and column half
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 18);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    float *xch = reinterpret_cast<float *>(smem + ATT_SMEM_DATA + 256);  // [2 regions][max|sum][2 halves][128 rows]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const WaitCtx wc{abort_flag, p.status};
    const int n_tiles = p.t1_rows > 0 ? 2 : 1;

    if (threadIdx.x == 0) {
        for (int i = 0; i < 2; ++i) {
            mbar_init(&full_qk[i], 1);
            mbar_init(&full_v[i], 1);
            mbar_init(&free_qk[i], 1);
            mbar_init(&free_v[i], 1);
            mbar_init(&bar_s[i], 1);
            mbar_init(&bar_p[2 * i], 128);
            mbar_init(&bar_p[2 * i + 1], 128);
            mbar_init(&bar_o[i], 1);
            mbar_init(&bar_free[i], 256);
        }
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == ATT_SOFTMAX_WARPS) {
        tmem_alloc(tmem_slot, 512);
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
    const int nchunks = (p.nk16 + 31) / 32;
    // Chunks of the first column half.  Chunks below the prefix end take the unmasked path in every row
    // (pad ranges aside); a masked chunk costs about 1.4 of those, so the first half gets more chunks when
    // the second one holds the masked ones.
    int n_a = (nchunks + 1) / 2;
    {
        const int n_clean = min(p.prefix_len / 32, nchunks);
        int best = 1 << 30;
        for (int a = (nchunks + 1) / 2; a <= max((nchunks + 1) / 2, nchunks - 1); ++a) {
            const int clean_a = min(a, n_clean), clean_b = n_clean - clean_a;
            const int cost_a = 10 * clean_a + 14 * (a - clean_a);
            const int cost_b = 10 * clean_b + 14 * (nchunks - a - clean_b);
            const int cost = max(cost_a, cost_b);
            if (cost < best) {
                best = cost;
                n_a = a;
            }
        }
    }
    if (SP) n_a = 4;
    const int pb_col = n_a * 32;  // P of the second half starts where its S columns start
    // O (64 columns) goes behind the P of the first half when that half's consumed S columns have room for it,
    // else behind the P of the second half.
    const int o_col = (n_a >= 4) ? n_a * 16 : pb_col + (nchunks - n_a) * 16;

    if (warp == ATT_SOFTMAX_WARPS) {
        // ------------------------------------------------------------- loader
        if (lane == 0) {
            int n = 0;
            for (int item = blockIdx.x; item < p.n_items; item += gridDim.x, ++n) {
                const int st = n & 1;
                const uint32_t m = (uint32_t)(n >> 1);
                // Q and K are released as soon as the item's last S MMA has read them, V after its last P V
                if (!mbar_wait(&free_qk[st], (m & 1u) ^ 1u, wc, DEV_TIMEOUT_EMPTY)) break;
                const int obs = item / p.n_kv, kvh = item % p.n_kv;
                const int page = p.page0 + item;
                const int qrow0 = (obs * p.n_q + kvh * p.g) * p.S;
                uint8_t *sQ = smem + st * ATT_QK_BYTES;
                uint8_t *sK = sQ + 2 * ATT_Q_TILE_BYTES, *sV = smem + 2 * ATT_QK_BYTES + st * ATT_KV_BYTES;
                uint32_t bytes = ATT_Q_TILE_BYTES + ATT_KV_BYTES;
                if (p.t1_rows > 0) bytes += p.t1_rot ? 32 * 128 : ATT_Q_TILE_BYTES;
                mbar_expect_tx(&full_qk[st], bytes);
                tma_load_2d(sQ, &q_map, &full_qk[st], 0, qrow0);
                if (p.t1_rows > 0) {
                    if (p.t1_rot)
                        tma_load_2d(sQ + ATT_Q_TILE_BYTES + (n & 3) * 32 * 128, &q_map32, &full_qk[st], 0, qrow0 + 128);
                    else
                        tma_load_2d(sQ + ATT_Q_TILE_BYTES, &q_map, &full_qk[st], 0, qrow0 + 128);
                }
                tma_load_3d(sK, &k_map, &full_qk[st], 0, 0, page);
                if (!mbar_wait(&free_v[st], (m & 1u) ^ 1u, wc, DEV_TIMEOUT_EMPTY)) break;
                mbar_expect_tx(&full_v[st], (uint32_t)ATT_KV_BYTES);
                tma_load_3d(sV, &v_map, &full_v[st], 0, 0, page);
            }
        }
    } else if (warp > ATT_SOFTMAX_WARPS) {
        // ------------------------------------------------------------- MMA issuer of region r
        const int r = warp - ATT_SOFTMAX_WARPS - 1;
        if (lane == 0) {
            const uint32_t idesc_s = make_idesc(1, 1, 1, 0, 0, 128, p.nk16);
            const uint32_t idesc_o = make_idesc(1, 1, 1, 0, 1, 128, 64);
            const uint32_t treg = tmem_base + (uint32_t)(r * ATT_REGION_COLS);
            const int k16_a = n_a * 2;  // 16-key steps whose P lives in the first column half
            int n = r;
            bool ok = true;
            for (int item = blockIdx.x + r * gridDim.x; ok && item < p.n_items; item += 2 * gridDim.x, n += 2) {
                const int st = n & 1;  // == r
                const uint32_t m = (uint32_t)(n >> 1);
                const uint32_t q_addr = smem_u32(smem + st * ATT_QK_BYTES);
                const uint32_t k_addr = q_addr + 2 * ATT_Q_TILE_BYTES;
                const uint32_t v_addr = smem_u32(smem + 2 * ATT_QK_BYTES + st * ATT_KV_BYTES);
                ok = mbar_wait(&full_qk[st], m & 1u, wc, DEV_TIMEOUT_FULL);
                for (int t = 0; ok && t < n_tiles; ++t) {
                    const uint32_t k_unit = m * (uint32_t)n_tiles + (uint32_t)t;  // units completed in this region
                    ok = mbar_wait(&bar_free[r], (k_unit & 1u) ^ 1u, wc, DEV_TIMEOUT_EMPTY);
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        mma_f16(treg, smem_desc_sw128(q_addr + t * ATT_Q_TILE_BYTES + k * 32, 16, 1024),
                                smem_desc_sw128(k_addr + k * 32, 16, 1024), idesc_s, k != 0 ? 1u : 0u);
                    tc_commit(&bar_s[r]);
                    if (t == n_tiles - 1) tc_commit(&free_qk[st]);  // Q, K of this item are dead once these MMAs ran
                    if (t == 0) ok = mbar_wait(&full_v[st], m & 1u, wc, DEV_TIMEOUT_FULL);
                    if (!ok) break;
                    // P V over the keys of the column half whose consumed S columns hold O (O may only be
                    // written once that half has finished reading S), then over the other half's keys
                    const int n_k16 = p.nk16 / 16;
                    const int first = (SP || n_a >= 4) ? 0 : 1;
                    uint32_t acc = 0u;
                    for (int part = 0; ok && part < 2; ++part) {
                        const int h = part ^ first;
                        const int k_lo = h ? k16_a : 0, k_hi = h ? n_k16 : min(k16_a, n_k16);
                        if (k_lo >= k_hi) continue;
                        ok = mbar_wait(&bar_p[2 * r + h], k_unit & 1u, wc, DEV_TIMEOUT_FULL);
                        if (!ok) break;
                        tc_fence_after();
                        if (SP) acc = 0u;  // an accumulator per half
                        const uint32_t o_dst = SP ? (h ? 192u : 64u) : (uint32_t)o_col;
                        for (int k16 = k_lo; k16 < k_hi; ++k16) {
                            const uint32_t p_col = h ? (uint32_t)(pb_col + (k16 - k16_a) * 8) : (uint32_t)(k16 * 8);
                            mma_f16_tmem_a(treg + o_dst, treg + p_col, smem_desc_sw128(v_addr + k16 * 2048, 16, 1024),
                                           idesc_o, acc);
                            acc = 1u;
                        }
                    }
                    if (!ok) break;
                    tc_commit(&bar_o[r]);
                }
                if (ok) tc_commit(&free_v[st]);  // every MMA that reads this V buffer has been issued
            }
        }
    } else {
        // ------------------------------------------------------------- softmax warps of region r
        const int r = warp >> 3, half = (warp >> 2) & 1, qtr = warp & 3;
        const uint32_t lane_addr = tmem_base + (uint32_t)(r * ATT_REGION_COLS) + ((uint32_t)(qtr * 32) << 16);
        const int n_suffix_cols = p.kv_len - p.prefix_len;
        const int c_begin = half ? n_a : 0, c_end = half ? nchunks : n_a;
        const uint32_t p_base = lane_addr + (half ? (uint32_t)pb_col : 0u);
        float *x_max = xch + r * 512, *x_sum = x_max + 256;  // [2 halves][128 rows] each
        const int my_row_slot = qtr * 32 + lane;
        int n = r;
        bool ok = true;
        for (int item = blockIdx.x + r * gridDim.x; ok && item < p.n_items; item += 2 * gridDim.x, n += 2) {
            const uint32_t m = (uint32_t)(n >> 1);
            const int obs = item / p.n_kv, kvh = item % p.n_kv;
            int pad_lo = 0, pad_hi = 0;
            if (p.pad) {
                pad_lo = p.pad[2 * obs];
                pad_hi = p.pad[2 * obs + 1];
            }
            for (int t = 0; ok && t < n_tiles; ++t) {
                const uint32_t k_unit = m * (uint32_t)n_tiles + (uint32_t)t;
                // row of this thread inside the R-row block, or -1
                int row;
                if (t == 0) row = qtr * 32 + lane;
                else if (p.t1_rot) row = (qtr == (n & 3)) ? 128 + lane : -1;
                else row = 128 + qtr * 32 + lane;
                const bool row_ok = row >= 0 && row < p.R;
                const bool warp_active = __any_sync(0xffffffffu, row_ok);
                const int head_l = row_ok ? row / p.S : 0, tok = row_ok ? row % p.S : 0;
                int limit = n_suffix_cols;
                if (p.mask_mode == 2) limit = min(tok + 1, n_suffix_cols);
                else if (p.mask_mode == 1) limit = tok == 0 ? min(1, n_suffix_cols) : n_suffix_cols;
                else if (p.mask_mode == 3) limit = tok == p.S - 1 ? n_suffix_cols : n_suffix_cols - 1;
                int clean_end = p.prefix_len;
                if (pad_hi > pad_lo) clean_end = min(clean_end, pad_lo);
                const RowMask rm{p.prefix_len + limit, pad_lo, pad_hi, clean_end};
                ok = mbar_wait(&bar_s[r], k_unit & 1u, wc, DEV_TIMEOUT_FULL);
                if (!ok) break;
                tc_fence_after();
                float sum_half;
                if (SP) {
                    // ---- one pass: reference = the first chunk's maximum, raised lazily ----
                    float sum0 = 0.0f, sum1 = 0.0f;
                    float m_ref = -INFINITY;  // log2 units
                    if (warp_active) {
                        for (int c = c_begin; c < c_end; ++c) {
                            uint32_t sa[32];
                            tmem_ld32(lane_addr + (uint32_t)(c * 32), sa);
                            tmem_ld_wait();
                            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
                            att_max_chunk(sa, c, rm, mx);
                            const float cm = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * p.scale_log2;
                            const bool raise = cm > m_ref + 8.0f;
                            if (c > c_begin && __any_sync(0xffffffffu, raise)) {
                                // rare: the P chunks written so far are relative to the old reference
                                const float f = raise ? (m_ref == -INFINITY ? 0.0f : ex2_approx(m_ref - cm)) : 1.0f;
                                tmem_st_wait();
                                for (int cc = c_begin; cc < c; ++cc) {
                                    uint32_t pk[16];
                                    tmem_ld16(p_base + (uint32_t)((cc - c_begin) * 16), pk);
                                    tmem_ld_wait();
#pragma unroll
                                    for (int j = 0; j < 16; ++j) {
                                        const float a = __uint_as_float(pk[j] << 16) * f, b = __uint_as_float(pk[j] & 0xffff0000u) * f;
                                        pk[j] = __byte_perm(__float_as_uint(a) + 0x8000u, __float_as_uint(b) + 0x8000u, 0x7632);
                                    }
                                    tmem_st16(p_base + (uint32_t)((cc - c_begin) * 16), pk);
                                }
                                sum0 *= f;
                                sum1 *= f;
                                tmem_ld32(lane_addr + (uint32_t)(c * 32), sa);  // (not kept in registers across the rescaling)
                                tmem_ld_wait();
                            }
                            if (raise) m_ref = cm;
                            att_exp_chunk(sa, c, rm, p.scale_log2, m_ref == -INFINITY ? 0.0f : m_ref, sum0, sum1,
                                          p_base + (uint32_t)((c - c_begin) * 16));
                        }
                        tmem_st_wait();
                    }
                    x_max[half * 128 + my_row_slot] = m_ref;
                    sum_half = sum0 + sum1;
                } else {
                // ---- pass 1: maximum over this thread's columns ----
                float mxx = -INFINITY;
                if (warp_active) {
                    float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
                    for (int c = c_begin; c < c_end; ++c) {
                        uint32_t sa[32];
                        tmem_ld32(lane_addr + (uint32_t)(c * 32), sa);
                        tmem_ld_wait();
                        att_max_chunk(sa, c, rm, mx);
                    }
                    mxx = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
                }
                x_max[half * 128 + my_row_slot] = mxx;
                region_sync(r);
                mxx = fmaxf(mxx, x_max[(half ^ 1) * 128 + my_row_slot]);
                const float m2 = (mxx == -INFINITY) ? 0.0f : mxx * p.scale_log2;
                // ---- pass 2: p = exp2(s*c - m*c), P (bf16) over this half's consumed S columns ----
                float sum0 = 0.0f, sum1 = 0.0f;
                if (warp_active) {
                    for (int c = c_begin; c < c_end; ++c) {
                        uint32_t sa[32];
                        tmem_ld32(lane_addr + (uint32_t)(c * 32), sa);
                        tmem_ld_wait();
                        att_exp_chunk(sa, c, rm, p.scale_log2, m2, sum0, sum1, p_base + (uint32_t)((c - c_begin) * 16));
                    }
                    tmem_st_wait();
                }
                sum_half = sum0 + sum1;
                }
                x_sum[half * 128 + my_row_slot] = sum_half;
                tc_fence_before();
                mbar_arrive(&bar_p[2 * r + half]);
                ok = mbar_wait(&bar_o[r], k_unit & 1u, wc, DEV_TIMEOUT_ACCUM);
                if (!ok) break;
                tc_fence_after();
                region_sync(r);  // both halves' partial sums are in shared memory
                float sum = x_sum[my_row_slot] + x_sum[128 + my_row_slot];
                uint32_t o[32];
                if (SP) {
                    // merge the two halves: O = (wA O_A + wB O_B) / (wA l_A + wB l_B)
                    const float mA = x_max[my_row_slot], mB = x_max[128 + my_row_slot], mm = fmaxf(mA, mB);
                    const float wA = mA == -INFINITY ? 0.0f : ex2_approx(mA - mm), wB = mB == -INFINITY ? 0.0f : ex2_approx(mB - mm);
                    sum = wA * x_sum[my_row_slot] + wB * x_sum[128 + my_row_slot];
                    if (warp_active) {
#pragma unroll
                        for (int j = 0; j < 2; ++j) {
                            uint32_t oa[16], ob[16];
                            tmem_ld16(lane_addr + (uint32_t)(64 + half * 32 + 16 * j), oa);
                            tmem_ld16(lane_addr + (uint32_t)(192 + half * 32 + 16 * j), ob);
                            tmem_ld_wait();
#pragma unroll
                            for (int e = 0; e < 16; ++e)
                                o[16 * j + e] = __float_as_uint(fmaf(wA, __uint_as_float(oa[e]), wB * __uint_as_float(ob[e])));
                        }
                    }
                } else if (warp_active) {
                    tmem_ld32(lane_addr + (uint32_t)(o_col + half * 32), o);
                    tmem_ld_wait();
                }
                tc_fence_before();
                mbar_arrive(&bar_free[r]);
                if (row_ok) {
                    const float inv = 1.0f / sum;
                    __nv_bfloat16 *dst = p.out + ((size_t)obs * p.S + tok) * ((size_t)p.n_q * 64) +
                                         (size_t)(kvh * p.g + head_l) * 64 + half * 32;
                    // one full 32-byte sector per store instruction and thread
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        uint32_t w[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(o[16 * j + 2 * e]) * inv,
                                                                           __uint_as_float(o[16 * j + 2 * e + 1]) * inv);
                            w[e] = *reinterpret_cast<const uint32_t *>(&h);
                        }
                        if (p.out_al32) {
                            asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst + 16 * j),
                                         "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
                                         : "memory");
                        } else {
                            uint4 *d4 = reinterpret_cast<uint4 *>(dst + 16 * j);
                            d4[0] = make_uint4(w[0], w[1], w[2], w[3]);
                            d4[1] = make_uint4(w[4], w[5], w[6], w[7]);
                        }
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == ATT_SOFTMAX_WARPS) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

}  // namespace vb


extern "C" int32_t vlab200_attention(const vlab200_kv_store *st, int32_t layer, const void *q, void *out,
                                     int32_t S, int32_t n_q, int32_t kv_len, int32_t mask_mode,
                                     const int32_t *pad_ranges, void *stream) {
    return vb::attention_ws(st, layer, q, out, S, n_q, kv_len, mask_mode, pad_ranges, static_cast<cudaStream_t>(stream), nullptr, 0);
}

// vlab200_attention with an optional float workspace: with it, calls that have few work units (one observation) run
// the streaming kernel over key slices on separate SMs and merge the slices (attn_flash.cu).
int vb::attention_ws(const vlab200_kv_store *st, int layer, const void *q, void *out, int S, int n_q, int kv_len, int mask_mode,
                     const int32_t *pad_ranges, cudaStream_t stream, float *ws, size_t ws_bytes) {
    if (!st || !st->k_pages || !st->v_pages || !q || !out) return VLAB200_ERR_ARG;
    if (layer < 0 || layer >= st->n_layers || S <= 0 || n_q <= 0 || st->n_kv <= 0 || n_q % st->n_kv)
        return VLAB200_ERR_ARG;
    if (kv_len <= 0 || kv_len > st->cap || st->prefix_len > kv_len || mask_mode < 0 || mask_mode > 3)
        return VLAB200_ERR_ARG;
    if ((reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(out) & 15) ||
        (reinterpret_cast<uintptr_t>(st->k_pages) & 15) || (reinterpret_cast<uintptr_t>(st->v_pages) & 15))
        return VLAB200_ERR_ARG;
    const int g = n_q / st->n_kv;
    const int R = g * S;
    if (st->head_dim != 64 && st->head_dim != 128 && st->head_dim != 256) return VLAB200_ERR_UNSUPPORTED;
    // the whole-range kernel gives one CTA per (observation, kv head): with a workspace and few of those, the key-split
    // streaming kernel spreads them over more SMs
    const bool few = ws && st->n_obs * st->n_kv * 4 <= vb::sm_count() && kv_len > 3 * 64;
    if (st->head_dim != 64 || kv_len > vb::ATT_MAX_KEYS || R > 256 || few)
        return vb::attention_flash(st, layer, q, out, S, n_q, kv_len, mask_mode, pad_ranges, stream, 0.0f, ws, ws_bytes);
    int *status = vb::device_status_ptr();
    if (!status) return vb::cuda_fail(cudaGetLastError(), "device_status_ptr");

    CUtensorMap qmap, qmap32, kmap, vmap;
    {
        const uint64_t dims[2] = {64, (uint64_t)st->n_obs * n_q * S};
        const uint64_t strides[1] = {128};
        const uint32_t box[2] = {64, 128}, box32[2] = {64, 32};
        int rc = vb::make_tensor_map(&qmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, q, dims, strides, box,
                                     CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc) return rc;
        rc = vb::make_tensor_map(&qmap32, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, q, dims, strides, box32,
                                 CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc) return rc;
    }
    {
        // rows >= kv_len are outside the map, so TMA zero-fills them (they enter P V with p = 0)
        const uint64_t dims[3] = {64, (uint64_t)kv_len, (uint64_t)st->n_layers * st->n_obs * st->n_kv};
        const uint64_t strides[2] = {128, (uint64_t)st->cap * 128};
        const uint32_t box[3] = {64, vb::ATT_MAX_KEYS, 1};
        int rc = vb::make_tensor_map(&kmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, st->k_pages, dims, strides, box,
                                     CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc) return rc;
        rc = vb::make_tensor_map(&vmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, st->v_pages, dims, strides, box,
                                 CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc) return rc;
    }
    vb::AttnParams p;
    p.out = static_cast<__nv_bfloat16 *>(out);
    p.pad = pad_ranges;
    p.S = S; p.n_q = n_q; p.n_kv = st->n_kv; p.g = g; p.kv_len = kv_len; p.prefix_len = st->prefix_len;
    p.mask_mode = mask_mode;
    p.nk16 = (kv_len + 15) / 16 * 16;
    p.R = R;
    p.n_items = st->n_obs * st->n_kv;
    p.page0 = layer * st->n_obs * st->n_kv;
    p.t1_rows = R > 128 ? R - 128 : 0;
    p.t1_rot = (p.t1_rows > 0 && p.t1_rows <= 32) ? 1 : 0;
    p.scale_log2 = 1.4426950408889634f / sqrtf(64.0f);
    p.out_al32 = (reinterpret_cast<uintptr_t>(out) & 31) == 0 ? 1 : 0;
    p.status = status;
    const int smem = vb::ATT_SMEM_DATA + 256 + 2 * 512 * 4 + 1024;
    // more than 128 keys (5 to 8 chunks of 32): the single-pass variant; VLAB200_ATTN_TWO_PASS=1 keeps the two-pass one
    static const bool two_pass_env = std::getenv("VLAB200_ATTN_TWO_PASS") != nullptr;
    const bool single_pass = (p.nk16 + 31) / 32 >= 5 && !two_pass_env;
    auto kernel = single_pass ? vb::attn_hd64_kernel<true> : vb::attn_hd64_kernel<false>;
    int rc_attr = vb::ensure_dyn_smem(kernel, smem);
    if (rc_attr) return rc_attr;
    const int n_sm = vb::sm_count();
    const int grid = p.n_items < n_sm ? p.n_items : n_sm;
    return vb::launch_pdl(kernel, dim3(grid), dim3(vb::ATT_THREADS), smem, static_cast<cudaStream_t>(stream), qmap, qmap32, kmap, vmap,
                          p);
}
