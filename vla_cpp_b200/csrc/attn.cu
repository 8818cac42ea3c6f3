// Action-query attention over the prefix + suffix KV pages (head_dim 64, up to 256 keys).
//
// One CTA per (kv head, observation).  The g = n_q / n_kv query heads that share the kv head
// are stacked into one row block of g*S rows (GQA/MQA head sharing: K and V are fetched once
// for all of them), processed as 128-row tcgen05 tiles:
//
//   TMA (SWIZZLE_128B): Q rows, the K page, the V page -> shared memory (pages are read once)
//   S = Q K^T           tcgen05.mma kind::f16, f32 accumulator in TMEM (whole key range at once)
//   softmax             one thread per row (TMEM lane): two passes over its row, exp2 with
//                       the scale folded in, masked columns skipped; P written back to TMEM
//                       as bf16 over the consumed S columns
//   O = P V             tcgen05.mma with A = P from TMEM, B = V page as an MN-major operand
//   epilogue            O / rowsum -> bf16 -> out[obs][tok][head*hd ..]
//
// Reference: src/layers/attn.h:38-46, src/models/pi0.cpp:204-223 (explicit mul_mat -> soft_max
// -> mul_mat with the score matrix in HBM), src/models/smolvla.cpp:835-842,874-881
// (ggml_flash_attn_ext); masks src/models/pi0.cpp:640-651, smolvla.cpp:1655-1664.
#include <cuda_bf16.h>

#include "host_common.h"
#include "tc5.cuh"

namespace vb {

constexpr int ATT_THREADS = 160;      // warps 0-3: softmax / epilogue (TMEM quarters), warp 4: TMA + MMA
constexpr int ATT_MAX_KEYS = 256;
constexpr int ATT_Q_TILE_BYTES = 128 * 128;
constexpr int ATT_KV_BYTES = ATT_MAX_KEYS * 128;
constexpr int ATT_TMEM_COLS = 256;    // S [0,256) / P [0,128) aliased, O [128,192)
constexpr int ATT_O_COL = 128;

struct AttnParams {
    __nv_bfloat16 *out;  // [n_obs][S][n_q*hd]
    const int32_t *pad;  // [n_obs][2] masked prefix columns, or null
    int S, n_q, n_kv, g, kv_len, prefix_len, mask_mode, nk16, R, n_mt, page0;
    float scale_log2;
    int *status;
};

__global__ void __launch_bounds__(ATT_THREADS, 2)
attn_hd64_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
                 const __grid_constant__ CUtensorMap v_map, const AttnParams p) {
    extern __shared__ uint8_t att_smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(att_smem_raw) + 1023) &
                                                ~static_cast<uintptr_t>(1023));
    uint8_t *sQ = smem;
    uint8_t *sK = smem + 2 * ATT_Q_TILE_BYTES;
    uint8_t *sV = sK + ATT_KV_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(sV + ATT_KV_BYTES);
    uint64_t *bar_qk = bars, *bar_v = bars + 1, *bar_s = bars + 2, *bar_p = bars + 3, *bar_o = bars + 4,
             *bar_free = bars + 5;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 6);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kvh = blockIdx.x, obs = blockIdx.y;
    const WaitCtx wc{abort_flag, p.status};

    if (threadIdx.x == 0) {
        mbar_init(bar_qk, 1);
        mbar_init(bar_v, 1);
        mbar_init(bar_s, 1);
        mbar_init(bar_p, 128);
        mbar_init(bar_o, 1);
        mbar_init(bar_free, 128);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 4) {
        tmem_alloc(tmem_slot, ATT_TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 4) {
        if (lane == 0) {
            const int page = p.page0 + obs * p.n_kv + kvh;
            const int qrow0 = (obs * p.n_q + kvh * p.g) * p.S;
            mbar_expect_tx(bar_qk, (uint32_t)(p.n_mt * ATT_Q_TILE_BYTES + ATT_KV_BYTES));
            for (int mt = 0; mt < p.n_mt; ++mt) tma_load_2d(sQ + mt * ATT_Q_TILE_BYTES, &q_map, bar_qk, 0, qrow0 + mt * 128);
            tma_load_3d(sK, &k_map, bar_qk, 0, 0, page);
            mbar_expect_tx(bar_v, (uint32_t)ATT_KV_BYTES);
            tma_load_3d(sV, &v_map, bar_v, 0, 0, page);

            const uint32_t idesc_s = make_idesc(1, 1, 1, 0, 0, 128, p.nk16);
            const uint32_t idesc_o = make_idesc(1, 1, 1, 0, 1, 128, 64);
            const uint32_t q_addr = smem_u32(sQ), k_addr = smem_u32(sK), v_addr = smem_u32(sV);
            bool ok = mbar_wait(bar_qk, 0, wc, DEV_TIMEOUT_FULL);
            for (int mt = 0; ok && mt < p.n_mt; ++mt) {
                if (mt > 0) ok = mbar_wait(bar_free, (uint32_t)(mt - 1) & 1u, wc, DEV_TIMEOUT_EMPTY);
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    mma_f16(tmem_base, smem_desc_sw128(q_addr + mt * ATT_Q_TILE_BYTES + k * 32, 16, 1024),
                            smem_desc_sw128(k_addr + k * 32, 16, 1024), idesc_s, k != 0 ? 1u : 0u);
                tc_commit(bar_s);
                ok = mbar_wait(bar_p, (uint32_t)mt & 1u, wc, DEV_TIMEOUT_FULL);
                if (ok && mt == 0) ok = mbar_wait(bar_v, 0, wc, DEV_TIMEOUT_FULL);
                if (!ok) break;
                tc_fence_after();
                for (int k16 = 0; k16 < p.nk16 / 16; ++k16)
                    mma_f16_tmem_a(tmem_base + ATT_O_COL, tmem_base + (uint32_t)(k16 * 8),
                                   smem_desc_sw128(v_addr + k16 * 2048, 16, 1024), idesc_o, k16 != 0 ? 1u : 0u);
                tc_commit(bar_o);
            }
        }
    } else {
        const int qtr = warp;  // warps 0..3 <-> TMEM lane quarters 0..3
        const uint32_t lane_addr = tmem_base + ((uint32_t)(qtr * 32) << 16);
        int pad_lo = 0, pad_hi = 0;
        if (p.pad) {
            pad_lo = p.pad[2 * obs];
            pad_hi = p.pad[2 * obs + 1];
        }
        const int n_suffix_cols = p.kv_len - p.prefix_len;
        const int nchunks = (p.nk16 + 31) / 32;
        for (int mt = 0; mt < p.n_mt; ++mt) {
            const int r = mt * 128 + qtr * 32 + lane;
            const bool row_ok = r < p.R;
            const int head_l = r / p.S, tok = r % p.S;
            int limit = n_suffix_cols;
            if (p.mask_mode == 2) limit = min(tok + 1, n_suffix_cols);
            else if (p.mask_mode == 1) limit = tok == 0 ? min(1, n_suffix_cols) : n_suffix_cols;
            const int jmax = p.prefix_len + limit;
            if (!mbar_wait(bar_s, (uint32_t)mt & 1u, wc, DEV_TIMEOUT_FULL)) break;
            tc_fence_after();
            // pass 1: row maximum over the visible columns
            float mx = -INFINITY;
            for (int c = 0; c < nchunks; ++c) {
                uint32_t sv[32];
                tmem_ld32(lane_addr + (uint32_t)(c * 32), sv);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const int col = c * 32 + j;
                    const bool vis = col < jmax && !(col >= pad_lo && col < pad_hi);
                    if (vis) mx = fmaxf(mx, __uint_as_float(sv[j]));
                }
            }
            const float m2 = (mx == -INFINITY) ? 0.0f : mx * p.scale_log2;
            // pass 2: p = exp2(s*c - m*c), P (bf16) over the consumed S columns
            float sum = 0.0f;
            for (int c = 0; c < nchunks; ++c) {
                uint32_t sv[32];
                tmem_ld32(lane_addr + (uint32_t)(c * 32), sv);
                tmem_ld_wait();
                uint32_t pk[16];
#pragma unroll
                for (int j = 0; j < 32; j += 2) {
                    const int col = c * 32 + j;
                    const bool v0 = col < jmax && !(col >= pad_lo && col < pad_hi);
                    const bool v1 = col + 1 < jmax && !(col + 1 >= pad_lo && col + 1 < pad_hi);
                    const float p0 = v0 ? exp2f(fmaf(__uint_as_float(sv[j]), p.scale_log2, -m2)) : 0.0f;
                    const float p1 = v1 ? exp2f(fmaf(__uint_as_float(sv[j + 1]), p.scale_log2, -m2)) : 0.0f;
                    sum += p0 + p1;
                    const __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
                    pk[j >> 1] = *reinterpret_cast<const uint32_t *>(&h);
                }
                tmem_st16(lane_addr + (uint32_t)(c * 16), pk);
            }
            if (mt == 0) {
                // keys kv_len .. nk16-1 enter the P V product with p = 0: make their V rows finite
                if (!mbar_wait(bar_v, 0, wc, DEV_TIMEOUT_FULL)) break;
                const int tail_rows = p.nk16 - p.kv_len;
                for (int i = threadIdx.x; i < tail_rows * 8; i += 128) {
                    const int row = p.kv_len + (i >> 3);
                    *reinterpret_cast<uint4 *>(sV + (row >> 3) * 1024 + (row & 7) * 128 + ((i & 7) << 4)) =
                        make_uint4(0, 0, 0, 0);
                }
                fence_proxy_async_smem();
            }
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(bar_p);
            if (!mbar_wait(bar_o, (uint32_t)mt & 1u, wc, DEV_TIMEOUT_ACCUM)) break;
            tc_fence_after();
            uint32_t o0[32], o1[32];
            tmem_ld32(lane_addr + ATT_O_COL, o0);
            tmem_ld32(lane_addr + ATT_O_COL + 32, o1);
            tmem_ld_wait();
            tc_fence_before();
            mbar_arrive(bar_free);
            if (row_ok) {
                const float inv = 1.0f / sum;
                __nv_bfloat16 *dst = p.out + ((size_t)obs * p.S + tok) * ((size_t)p.n_q * 64) +
                                     (size_t)(kvh * p.g + head_l) * 64;
                uint4 *d4 = reinterpret_cast<uint4 *>(dst);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    uint32_t w[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(o0[8 * j + 2 * e]) * inv,
                                                                       __uint_as_float(o0[8 * j + 2 * e + 1]) * inv);
                        w[e] = *reinterpret_cast<const uint32_t *>(&h);
                    }
                    d4[j] = make_uint4(w[0], w[1], w[2], w[3]);
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    uint32_t w[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(o1[8 * j + 2 * e]) * inv,
                                                                       __uint_as_float(o1[8 * j + 2 * e + 1]) * inv);
                        w[e] = *reinterpret_cast<const uint32_t *>(&h);
                    }
                    d4[4 + j] = make_uint4(w[0], w[1], w[2], w[3]);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 4) {
        tc_fence_after();
        tmem_dealloc(tmem_base, ATT_TMEM_COLS);
    }
}

}  // namespace vb

extern "C" int32_t vlab200_attention(const vlab200_kv_store *st, int32_t layer, const void *q, void *out,
                                     int32_t S, int32_t n_q, int32_t kv_len, int32_t mask_mode,
                                     const int32_t *pad_ranges, void *stream) {
    if (!st || !st->k_pages || !st->v_pages || !q || !out) return VLAB200_ERR_ARG;
    if (layer < 0 || layer >= st->n_layers || S <= 0 || n_q <= 0 || st->n_kv <= 0 || n_q % st->n_kv)
        return VLAB200_ERR_ARG;
    if (kv_len <= 0 || kv_len > st->cap || st->prefix_len > kv_len || mask_mode < 0 || mask_mode > 2)
        return VLAB200_ERR_ARG;
    if ((reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(out) & 15) ||
        (reinterpret_cast<uintptr_t>(st->k_pages) & 15) || (reinterpret_cast<uintptr_t>(st->v_pages) & 15))
        return VLAB200_ERR_ARG;
    const int g = n_q / st->n_kv;
    const int R = g * S;
    if (st->head_dim != 64 || kv_len > vb::ATT_MAX_KEYS || R > 256) return VLAB200_ERR_UNSUPPORTED;
    int *status = vb::device_status_ptr();
    if (!status) return vb::cuda_fail(cudaGetLastError(), "device_status_ptr");

    CUtensorMap qmap, kmap, vmap;
    {
        const uint64_t dims[2] = {64, (uint64_t)st->n_obs * n_q * S};
        const uint64_t strides[1] = {128};
        const uint32_t box[2] = {64, 128};
        int rc = vb::make_tensor_map(&qmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, q, dims, strides, box,
                                     CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc) return rc;
    }
    {
        const uint64_t dims[3] = {64, (uint64_t)st->cap, (uint64_t)st->n_layers * st->n_obs * st->n_kv};
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
    p.n_mt = (R + 127) / 128;
    p.page0 = layer * st->n_obs * st->n_kv;
    p.scale_log2 = 1.4426950408889634f / sqrtf(64.0f);
    p.status = status;
    const int smem = 2 * vb::ATT_Q_TILE_BYTES + 2 * vb::ATT_KV_BYTES + 128 + 1024;
    static bool attr_done = false;
    if (!attr_done) {
        VB_CUDA(cudaFuncSetAttribute(vb::attn_hd64_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        attr_done = true;
    }
    dim3 grid(st->n_kv, st->n_obs);
    vb::attn_hd64_kernel<<<grid, vb::ATT_THREADS, smem, static_cast<cudaStream_t>(stream)>>>(qmap, kmap, vmap, p);
    VB_CUDA(cudaGetLastError());
    return VLAB200_OK;
}
