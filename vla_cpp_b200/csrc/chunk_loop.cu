// One observation, the whole Euler loop, ONE kernel.
//
// With a single observation the suffix is 50 / 51 rows: every product of the loop streams its weights once and does
// almost no arithmetic, and a launch per operator spends most of its time between kernels (about 1,600 launches per
// chunk for a pi0-shaped expert).  Here one persistent cooperative kernel (one CTA of 256 threads per SM) walks a
// table of PHASES -- the operators of one Euler step, src/models/pi0.cpp:570-588, src/models/smolvla.cpp:1393-1418 --
// and separates them with a grid-wide barrier (one atomic arrival + a bounded acquire spin per CTA).  Per layer:
// q|k|v, attention, key-slice merge, Wo + residual, gate/up, Wdown + residual = six phases.
//
// Phase kinds
//   GEMM     C[M <= 64][N] = A[M][K] W[N][K]^T.  A unit is NG (2 or 4) groups of 8 output columns; units are dealt to
//            the CTAs in contiguous ranges.  A unit's weights arrive as K chunks of 2048 / NG columns, one
//            cp.async.bulk per chunk, in a 3-stage ring that is fed by one thread from a cursor that runs AHEAD of the
//            computation, across phase boundaries and barriers (weights do not depend on anything the loop computes),
//            so HBM streams while the CTAs wait for each other.  A is brought in K slices of at most 1024 columns (all
//            M rows, one bulk copy); a product with a longer K (Wo, Wdown) walks its slices one after the other and
//            keeps accumulating in registers, so its residual update needs no second pass over partial sums.  The 8
//            warps are 2 row halves x 4 K quarters of mma.sync m16n8k16 with ldmatrix operands; the quarters are added
//            through shared memory in a fixed order by all threads (one row, 4 adjacent columns each).  Epilogues:
//            residual += projection with the bf16 mirror and per-unit sums of squares (the consumer's RMS factor),
//            act(gate) * up, RMS factor + NeoX rotation + append of q|k|v, bias + activation, and the Euler update.
//            A bulk copy costs the issuing thread 40-60 ns whatever its size (measured: 51 row copies of 2 KB took
//            3 us, 192 of 512 B 7.8 us), so every operand tile has to be ONE contiguous range: all bf16 matrices the
//            loop reads (weights, activations, q, K/V pages) live in PADDED images -- [K slice][row][slice columns + 8]
//            -- whose rows are 16 bytes apart modulo 128, which is also what makes the ldmatrix reads conflict-free.
//   ATT      (kv head, 32 stacked query rows, key slice) units: S = Q K^T and P V by mma.sync on tiles staged by three
//            bulk copies; un-normalised O rows, maximum and row sum per unit.      COMBINE merges the key slices.
//   EMBED    action-in projection (+ pi0's state token) on CUDA cores.
// Everything one CTA writes for another goes through L2 (st / ld .cg, bulk copies), never through L1.  Phase
// descriptors are fetched one phase ahead into shared memory (cp.async), the weight cursor's table sits there too.
// Results do not depend on the run: every sum has a fixed order.
// The tensor-core path of the large-batch kernels (tcgen05 + TMEM) costs an allocation, a commit and a TMEM read per
// tile, which is what a 51-row problem cannot amortise; mma.sync with register accumulators has no such fixed cost.
// What bounds a phase here is a chain of L2 round trips (barrier arrival + poll, A tile, rms partials, residual
// read-modify-write, store drain), about 0.7 us each, not the tensor pipe and not HBM.
#include <cuda_bf16.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <new>
#include <vector>

#include "chunk_loop.h"
#include "gemm.h"
#include "host_common.h"
#include "tc5.cuh"

namespace vb {
namespace {

enum { PH_GEMM = 0, PH_ATT = 2, PH_COMBINE = 3, PH_EMBED = 4 };
enum { OUT_RESID = 0, OUT_GATED = 1, OUT_QKV = 2, OUT_BIAS_ACT = 3, OUT_EULER = 4 };
enum { RMS_NONE = 0, RMS_PARTS = 1, RMS_LOCAL = 2 };  // use_rms: row sums of squares from the producer's per-sub-unit partials, or from the A tile

constexpr int CL_THREADS = 256;   // the eight computing warps
constexpr int CL_BLOCK = 288;     // + one warp whose lane 0 feeds the weight ring
constexpr int CL_STAGES = 3;
constexpr int CL_MAX_KSLICE = 1024;                               // columns of one K slice
constexpr int CL_STAGE_BYTES = 16 * (CL_MAX_KSLICE * 2 + 16);     // 16 padded weight rows of at most 1024 columns
constexpr int CL_DESC_BYTES = 352;                                // one phase descriptor slot (two of them: this phase, the next)
constexpr int CL_DESC_OFF = 1536;
constexpr int CL_WTAB_OFF = 2304;                                 // weight cursor table: one 32-byte entry per GEMM phase of a step
constexpr int CL_WTAB_MAX = 104;
constexpr int CL_HEADER = 5632;                                   // barriers, abort flag, small float arrays, descriptors, cursor table
constexpr int CL_RING_OFF = CL_HEADER;
constexpr int CL_ARENA_OFF = CL_RING_OFF + CL_STAGES * CL_STAGE_BYTES;
constexpr int CL_SMEM = 232448;
constexpr int CL_ARENA = CL_SMEM - CL_ARENA_OFF;
constexpr int CL_SC_LD = 20;                                      // floats per scratch row (16 columns + 4: conflict-free float2 writes)
constexpr int CL_SC_ROW = CL_SC_LD * 4;                           // bytes; the scratch tile holds the four K quarters of M x 16 sums
constexpr int CL_EMBED_ROWS = 10;
constexpr int CL_DEV_TIMEOUT = 105;

// A bf16 matrix [rows][cols] as a padded image: K slices of `kslice` columns, each a block of `rows` rows of
// kslice * 2 + 16 bytes.  Element (row, col) sits at this byte offset.
__host__ __device__ __forceinline__ size_t pad_off(int rows, int kslice, int row, int col) {
    const int s = col / kslice, c = col - s * kslice;
    return ((size_t)s * rows + row) * ((size_t)kslice * 2 + 16) + (size_t)c * 2;
}

struct alignas(16) LoopPhase {
    int type, out_mode, act, use_rms;
    int M, N, K, kslices, n_sub, half;  // half > 0: q|k|v pairing distance (head_dim / 2)
    int row_off, hd, out_rows, out_kslice;
    int ng, kchunk;                     // GEMM: 8-column groups per unit (2 / 4 / 8; n_sub counts units), columns per weight chunk
    float eps, scale_log2, dt;
    int bias_step_stride;
    const uint8_t *Ap, *Wp;             // padded images of A ([M][K]) and W ([N][K]), both cut into `kslices` slices
    float *out_f32, *h, *x;
    float *ssq_out;                     // [n_sub][64]: sum of squares of the bf16 values this phase writes, per sub-unit and row (optional)
    const float *ssq_in;                // RMS_PARTS: the producer's partials, ssq_n of them per row
    long long ssq_n;
    // pi0.5 (adaptive RMSNorm, gated residuals): per-step vectors, element stride mod_stride between steps
    const float *colscale;              // OUT_RESID: gate on the projection before it is added
    const float *scale_next;            // OUT_RESID / EMBED: the mirror is written as bf16(h * (1 + scale_next[col])) for the norm that reads it
    long long mod_stride;
    uint8_t *outp;                      // padded image the phase writes (out_rows rows, slices of out_kslice columns)
    uint8_t *hbp, *qp, *kpp, *vpp;      // padded: residual mirror [S][H], q [n_q S][hd], this layer's K / V pages [n_kv cap][hd]
    const float *bias, *rope;
    int n_q, n_kvp, n_kv, g, S, R, n_rt, ns, ks, kv_len, P, mask_mode, cap, chunk, A_dim, sd, H;
    float *ws_o, *ws_ml;
    const __nv_bfloat16 *w_dense, *w2;  // EMBED: W_ain [H][A], W_sp [H][sd] (plain row-major)
    const float *b2;                    // EMBED: b_sp
};

struct LoopParams {
    const LoopPhase *phases;
    const void *wtab;  // WEntry per GEMM phase of a step, in phase order
    int n_phases, steps, n_wtab;
    unsigned *counter;
    int *status;
    const float *state;
    const int32_t *pad;
    unsigned long long *trace;  // developer aid: global-timer stamp of CTA 0 after every barrier (nullptr: off)
    // prefix rows of the engine's pages -> padded pages, once per call
    const __nv_bfloat16 *k_src, *v_src;
    uint8_t *kpp, *vpp;
    size_t src_layer_stride;  // elements
    int L, n_kv, cap, P, hd;
};

// ------------------------------------------------------------------------------------------ device helpers
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm4_t(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm2_t(uint32_t (&r)[2], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float ex2f(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
template <int ACT>
__device__ __forceinline__ float act_f(float x) {
    if (ACT == ACT_SILU) return __fdividef(x, 1.0f + __expf(-x));
    if (ACT == ACT_GELU_TANH) {
        const float k0 = 0.79788456080286535587989211986876f, k1 = 0.044715f;
        const float u = k0 * x * (1.0f + k1 * x * x);
        return __fdividef(x, 1.0f + __expf(-2.0f * u));
    }
    return x;
}
__device__ __forceinline__ float act_rt(float x, int act) {
    return act == ACT_SILU ? act_f<ACT_SILU>(x) : act == ACT_GELU_TANH ? act_f<ACT_GELU_TANH>(x) : x;
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t *>(&v);
}


struct WEntry {  // what the weight cursor needs to know about one GEMM phase
    const uint8_t *Wp;   // padded image cut into chunks of kchunk columns
    int n_units, n_chunks, N, half;
    uint32_t stride;     // kchunk * 2 + 16
    int ng;
};
static_assert(sizeof(LoopPhase) <= CL_DESC_BYTES && sizeof(LoopPhase) % 16 == 0, "descriptor slot");
static_assert(sizeof(WEntry) == 32, "cursor table entry");

// barrier of the computing warps (the feeder warp is not part of it)
__device__ __forceinline__ void cons_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

struct Smem {
    uint64_t *full, *a_full, *empty, *done;
    const WEntry *wtab;
    int n_wtab;
    volatile int *abort_flag;
    float *rms, *red_max, *red_sum;
    uint8_t *ring, *arena;
};

// The carve-up of the dynamic shared memory; every phase function rebuilds it from the base (a few constant offsets) instead
// of taking it by reference, which would put it into local memory.
__device__ __forceinline__ Smem get_smem() {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    Smem sm;
    sm.full = reinterpret_cast<uint64_t *>(smem_raw);          // [CL_STAGES]
    sm.a_full = sm.full + CL_STAGES;                          // [2]
    sm.empty = sm.a_full + 2;                                 // [CL_STAGES]
    sm.done = sm.empty + CL_STAGES;
    sm.abort_flag = reinterpret_cast<volatile int *>(smem_raw + 120);
    sm.n_wtab = *reinterpret_cast<const int *>(smem_raw + 124);
    sm.rms = reinterpret_cast<float *>(smem_raw + 128);
    sm.red_max = reinterpret_cast<float *>(smem_raw + 512);
    sm.red_sum = reinterpret_cast<float *>(smem_raw + 1024);
    sm.wtab = reinterpret_cast<const WEntry *>(smem_raw + CL_WTAB_OFF);
    sm.ring = smem_raw + CL_RING_OFF;
    sm.arena = smem_raw + CL_ARENA_OFF;
    return sm;
}

// Sub-units of a phase dealt to this CTA: ids [b, e) with id = unit * chunks + chunk: the range is cut between units.
__device__ __forceinline__ void sub_range(int n_chunks, int n_units, int &b, int &e) {
    b = (int)((unsigned)n_units * blockIdx.x / gridDim.x) * n_chunks;
    e = (int)((unsigned)n_units * (blockIdx.x + 1) / gridDim.x) * n_chunks;
}

// weight rows of the 16-column block `sub16`: two groups of 8 rows
__device__ __forceinline__ void sub_rows(int half, int sub16, int &r0, int &r1) {
    if (half > 0) {
        const int per = half >> 3, hh = sub16 / per, j = sub16 - hh * per;
        r0 = hh * 2 * half + 8 * j;
        r1 = r0 + half;
    } else {
        r0 = 16 * sub16;
        r1 = r0 + 8;
    }
}

// The feeder: one thread walks the GEMM phases of every step in order and copies each (unit, chunk) of this CTA into the
// next ring stage as soon as the eight computing warps have released it.  It runs ahead of the computation by the depth
// of the ring, across phase boundaries and grid barriers.
__device__ __noinline__ void feeder_loop(const LoopParams &lp) {
    const Smem sm = get_smem();
    const WaitCtx wc{sm.abort_flag, lp.status};
    unsigned issued = 0;
    bool ok = true;
    for (int step = 0; ok && step < lp.steps; ++step)
        for (int gi = 0; ok && gi < sm.n_wtab; ++gi) {
            const WEntry w = sm.wtab[gi];
            int id0, id1;
            sub_range(w.n_chunks, w.n_units, id0, id1);
            for (int id = id0; id < id1; ++id, ++issued) {
                const int u = id / w.n_chunks, c = id - u * w.n_chunks;
                const unsigned stage = issued % CL_STAGES;
                if (issued >= CL_STAGES && !mbar_wait_backoff(&sm.empty[stage], ((issued / CL_STAGES) - 1u) & 1u, wc, CL_DEV_TIMEOUT, 20)) {
                    ok = false;
                    break;
                }
                uint64_t *bar = &sm.full[stage];
                uint8_t *dst = sm.ring + (size_t)stage * CL_STAGE_BYTES;
                const uint8_t *src = w.Wp + (size_t)c * w.N * w.stride;
                mbar_expect_tx(bar, 16u * w.stride);
                if (w.half > 0) {
                    int r0, r1;
                    sub_rows(w.half, u, r0, r1);
                    bulk_g2s(dst, src + (size_t)r0 * w.stride, 8u * w.stride, bar);
                    bulk_g2s(dst + 8u * w.stride, src + (size_t)r1 * w.stride, 8u * w.stride, bar);
                } else {
                    bulk_g2s(dst, src + (size_t)u * 16u * w.stride, 16u * w.stride, bar);
                }
            }
        }
    *reinterpret_cast<volatile unsigned *>(reinterpret_cast<uint8_t *>(sm.full) + 384) = issued;
    mbar_arrive(sm.done);
}

// Grid-wide barrier: every CTA arrives once; `target` counts arrivals since the launch.
__device__ __forceinline__ bool grid_barrier(const LoopParams &lp, unsigned target, const Smem &sm, const WaitCtx &wc) {
    cons_sync();
    if (threadIdx.x == 0 && !*sm.abort_flag) {
        __threadfence();
        atomicAdd(lp.counter, 1u);
        const long long t0 = clock64();
        for (uint32_t it = 0;; ++it) {
            unsigned v;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(lp.counter) : "memory");
            if (v >= target) break;
            if ((it & 255u) == 255u) {
                int st;
                asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(st) : "l"(lp.status) : "memory");
                if (st != 0 || clock64() - t0 > wc.budget) {
                    atomicCAS(lp.status, 0, CL_DEV_TIMEOUT);
                    *sm.abort_flag = 1;
                    break;
                }
            }
        }
    }
    cons_sync();
    return *sm.abort_flag == 0;
}

// ------------------------------------------------------------------------------------------------ GEMM
// The epilogue of one 16-column block (two 8-column groups) of a unit: every thread owns one row and four adjacent columns
// of the block; the four K quarters are added from the scratch tile in a fixed order.
__device__ __forceinline__ void gemm_epilogue(const LoopPhase &pg, const Smem &sm, const float *sc, int sub16, int step, int M, int N,
                                              int half, int out_mode, int use_rms, int act, int erow, int ec4) {
    const int tid = threadIdx.x;
    float ssq = 0.0f;
    if (erow < M && (out_mode != OUT_QKV || ec4 < 8)) {
        int r0, r1;
        sub_rows(half, sub16, r0, r1);
        const float *src = sc + (size_t)erow * CL_SC_LD + ec4;
        float4 v = *reinterpret_cast<const float4 *>(src);
#pragma unroll
        for (int k = 1; k < 4; ++k) {
            const float4 t = *reinterpret_cast<const float4 *>(src + (size_t)k * M * CL_SC_LD);
            v.x += t.x; v.y += t.y; v.z += t.z; v.w += t.w;
        }
        const float rms = use_rms ? sm.rms[erow] : 1.0f;
        v.x *= rms; v.y *= rms; v.z *= rms; v.w *= rms;
        const int wrow = ec4 < 8 ? r0 + ec4 : r1 + ec4 - 8;  // first of the four output columns
        if (out_mode == OUT_RESID) {  // residual stream += projection; bf16 mirror; sums of squares of the mirror
            float4 *hp = reinterpret_cast<float4 *>(pg.h + (size_t)erow * N + wrow);
            float4 hv = __ldcg(hp);
            if (pg.colscale) {
                const float4 gt = *reinterpret_cast<const float4 *>(pg.colscale + (size_t)step * pg.mod_stride + wrow);
                v.x *= gt.x; v.y *= gt.y; v.z *= gt.z; v.w *= gt.w;
            }
            hv.x += v.x; hv.y += v.y; hv.z += v.z; hv.w += v.w;
            __stcg(hp, hv);
            if (pg.scale_next) {  // the adaptive norm's (1 + scale) goes into the mirror, its sums of squares come from h itself
                const float4 sn = *reinterpret_cast<const float4 *>(pg.scale_next + (size_t)step * pg.mod_stride + wrow);
                __stcg(reinterpret_cast<uint2 *>(pg.hbp + pad_off(M, N, erow, wrow)),
                       make_uint2(pack_bf16(hv.x + hv.x * sn.x, hv.y + hv.y * sn.y), pack_bf16(hv.z + hv.z * sn.z, hv.w + hv.w * sn.w)));
                ssq = fmaf(hv.x, hv.x, fmaf(hv.y, hv.y, fmaf(hv.z, hv.z, hv.w * hv.w)));
            } else {
                const uint2 pk = make_uint2(pack_bf16(hv.x, hv.y), pack_bf16(hv.z, hv.w));
                __stcg(reinterpret_cast<uint2 *>(pg.hbp + pad_off(M, N, erow, wrow)), pk);
                const float2 f0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&pk.x));
                const float2 f1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&pk.y));
                ssq = fmaf(f0.x, f0.x, fmaf(f0.y, f0.y, fmaf(f1.x, f1.x, f1.y * f1.y)));
            }
        } else if (out_mode == OUT_GATED) {
            // interleaved weight rows: even = gate, odd = up
            if (pg.bias) {
                const float4 b = *reinterpret_cast<const float4 *>(pg.bias + (size_t)step * pg.bias_step_stride + wrow);
                v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
            }
            const float o0 = act_rt(v.x, act) * v.y, o1 = act_rt(v.z, act) * v.w;
            __stcg(reinterpret_cast<unsigned *>(pg.outp + pad_off(pg.out_rows, pg.out_kslice, erow, wrow >> 1)), pack_bf16(o0, o1));
        } else if (out_mode == OUT_QKV) {
            float4 w = *reinterpret_cast<const float4 *>(src + 8);  // the partner columns (k + half)
#pragma unroll
            for (int k = 1; k < 4; ++k) {
                const float4 t = *reinterpret_cast<const float4 *>(src + 8 + (size_t)k * M * CL_SC_LD);
                w.x += t.x; w.y += t.y; w.z += t.z; w.w += t.w;
            }
            w.x *= rms; w.y *= rms; w.z *= rms; w.w *= rms;
            if (pg.bias) {
                const float *bp = pg.bias + (size_t)step * pg.bias_step_stride;
                const float4 b0 = *reinterpret_cast<const float4 *>(bp + r0 + ec4), b1 = *reinterpret_cast<const float4 *>(bp + r1 + ec4);
                v.x += b0.x; v.y += b0.y; v.z += b0.z; v.w += b0.w;
                w.x += b1.x; w.y += b1.y; w.z += b1.z; w.w += b1.w;
            }
            const int hd = 2 * half, head = r0 / hd, k = r0 - head * hd + ec4;
            const int n_q = pg.n_q, n_kvp = pg.n_kvp, S = pg.S;
            const uint32_t sq = (uint32_t)hd * 2u + 16u;
            uint8_t *dst;
            float4 lo = v, hi = w;
            if (head < n_q + n_kvp) {
                const float4 c = *reinterpret_cast<const float4 *>(pg.rope + (size_t)erow * half + k);
                const float4 sn = *reinterpret_cast<const float4 *>(pg.rope + (size_t)(S + erow) * half + k);
                lo = make_float4(v.x * c.x - w.x * sn.x, v.y * c.y - w.y * sn.y, v.z * c.z - w.z * sn.z, v.w * c.w - w.w * sn.w);
                hi = make_float4(w.x * c.x + v.x * sn.x, w.y * c.y + v.y * sn.y, w.z * c.z + v.z * sn.z, w.w * c.w + v.w * sn.w);
                dst = head < n_q ? pg.qp + ((size_t)head * S + erow) * sq : pg.kpp + ((size_t)(head - n_q) * pg.cap + pg.P + erow) * sq;
            } else {
                dst = pg.vpp + ((size_t)(head - n_q - n_kvp) * pg.cap + pg.P + erow) * sq;
            }
            __stcg(reinterpret_cast<uint2 *>(dst + k * 2), make_uint2(pack_bf16(lo.x, lo.y), pack_bf16(lo.z, lo.w)));
            __stcg(reinterpret_cast<uint2 *>(dst + (k + half) * 2), make_uint2(pack_bf16(hi.x, hi.y), pack_bf16(hi.z, hi.w)));
        } else {
            if (pg.bias) {
                const float4 b = *reinterpret_cast<const float4 *>(pg.bias + (size_t)step * pg.bias_step_stride + wrow);
                v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
            }
            if (out_mode == OUT_EULER) {
                const int t = erow - (pg.S - pg.chunk);
                if (t >= 0) {
                    float4 *xp = reinterpret_cast<float4 *>(pg.x + (size_t)t * N + wrow);
                    float4 xv = __ldcg(xp);
                    const float dt = pg.dt;
                    xv.x += dt * v.x; xv.y += dt * v.y; xv.z += dt * v.z; xv.w += dt * v.w;
                    __stcg(xp, xv);
                }
            } else {
                v.x = act_rt(v.x, act); v.y = act_rt(v.y, act); v.z = act_rt(v.z, act); v.w = act_rt(v.w, act);
                const int orow = erow + pg.row_off;
                __stcg(reinterpret_cast<uint2 *>(pg.outp + pad_off(pg.out_rows, pg.out_kslice, orow, wrow)),
                       make_uint2(pack_bf16(v.x, v.y), pack_bf16(v.z, v.w)));
                if (pg.out_f32) __stcg(reinterpret_cast<float4 *>(pg.out_f32 + (size_t)orow * N + wrow), v);
            }
        }
    }
    if (pg.ssq_out) {  // the four threads of a row hold its 16 columns
        ssq += __shfl_xor_sync(0xffffffffu, ssq, 1);
        ssq += __shfl_xor_sync(0xffffffffu, ssq, 2);
        if ((tid & 3) == 0 && erow < M) __stcg(pg.ssq_out + (size_t)sub16 * 64 + erow, ssq);
    }
}

// A unit = NG groups of 8 output columns; its weights arrive as K chunks of 2048 / NG columns (one ring stage each), A as
// K slices of at most 1024 columns; the accumulators live in registers across all chunks and slices of the unit.
template <int NG>
__device__ __noinline__ void gemm_phase(const LoopPhase &pg, const LoopParams &lp, int step, unsigned &cons, unsigned &a_cnt_ref) {
    const Smem sm = get_smem();
    const WaitCtx wc{sm.abort_flag, lp.status};
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int mh = warp & 1, kq = warp >> 1;
    const int M = pg.M, N = pg.N, K = pg.K, kslices = pg.kslices, n_units = pg.n_sub, half = pg.half;
    const int out_mode = pg.out_mode, use_rms = pg.use_rms, act = pg.act;
    const int kchunk = pg.kchunk, n_chunks = K / kchunk;
    int id0, id1;
    sub_range(n_chunks, n_units, id0, id1);
    if (id0 >= id1) return;
    const uint8_t *Ap = pg.Ap;
    const float eps = pg.eps;
    const int kslice = K / kslices, cps = kslice / kchunk;  // chunks per A slice
    const uint32_t astride = (uint32_t)kslice * 2u + 16u, wstride = (uint32_t)kchunk * 2u + 16u;
    const uint32_t slot_bytes = kslices > 1 ? (uint32_t)M * astride : 0u;  // two A buffers when A comes in slices
    float *sc = reinterpret_cast<float *>(sm.arena + (size_t)(kslices > 1 ? 2 : 1) * M * astride);  // [4 K quarters][M][CL_SC_LD]
    const uint32_t as_addr = smem_u32(sm.arena);
    unsigned a_cnt = a_cnt_ref, a_iss = a_cnt_ref;  // A tiles consumed / issued since the launch: barrier and buffer alternate with them
    const int nk = kchunk >> 4, ks0 = kq * nk / 4, ks1 = (kq + 1) * nk / 4;
    // ldmatrix lane addressing
    const int mi = lane >> 3, lr = lane & 7;
    uint32_t a_off[2];
#pragma unroll
    for (int mtl = 0; mtl < 2; ++mtl) {
        int row = (2 * mh + mtl) * 16 + lr + (mi & 1) * 8;
        row = min(row, M - 1);
        a_off[mtl] = as_addr + (uint32_t)row * astride + (uint32_t)(mi >> 1) * 16u;
    }
    const uint32_t b_lane = (uint32_t)(lr + (mi >> 1) * 8) * wstride + (uint32_t)(mi & 1) * 16u;
    const bool mt_ok[2] = {(2 * mh) * 16 < M, (2 * mh + 1) * 16 < M};
    const int g = lane >> 2, q2 = (lane & 3) * 2;
    const int erow = tid >> 2, ec4 = (tid & 3) * 4;
    float acc[2][NG][4];
    uint32_t a_slot = 0;  // byte offset of the A buffer in use
    for (int id = id0; id < id1; ++id) {
        const int u = id / n_chunks, c = id - u * n_chunks, slice = c / cps, cs = c - slice * cps;
        if (cs == 0 && (kslices > 1 || id == id0)) {  // an unsliced A serves every unit of the phase
            cons_sync();  // every warp is done with the slice before: the buffer that is filled next is free
            if (tid == 0) {
                if (slice == 0) {
                    mbar_expect_tx(&sm.a_full[a_iss & 1u], (uint32_t)M * astride);
                    bulk_g2s(sm.arena + (a_iss & 1u) * slot_bytes, Ap, (uint32_t)M * astride, &sm.a_full[a_iss & 1u]);
                }
                if (slice + 1 < kslices) {  // the next slice loads while this one is multiplied
                    const unsigned nx = a_iss + (slice == 0 ? 1u : 0u);
                    mbar_expect_tx(&sm.a_full[nx & 1u], (uint32_t)M * astride);
                    bulk_g2s(sm.arena + (nx & 1u) * slot_bytes, Ap + (size_t)(slice + 1) * M * astride, (uint32_t)M * astride, &sm.a_full[nx & 1u]);
                }
            }
            a_iss += (slice == 0 ? 1u : 0u) + (slice + 1 < kslices ? 1u : 0u);
            if (use_rms == RMS_PARTS && id == id0) {  // rms factors from the producer's partial sums, fixed order
                const int r = tid >> 2, q = tid & 3, n = (int)pg.ssq_n;
                float part[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) part[j] = (r < M && q + 4 * j < n) ? __ldcg(pg.ssq_in + (size_t)(q + 4 * j) * 64 + r) : 0.0f;
                float ss = 0.0f;
#pragma unroll
                for (int j = 0; j < 16; ++j) ss += part[j];
                ss += __shfl_xor_sync(0xffffffffu, ss, 1);
                ss += __shfl_xor_sync(0xffffffffu, ss, 2);
                if (q == 0 && r < M) sm.rms[r] = rsqrtf(ss / (float)K + eps);
            }
            mbar_wait(&sm.a_full[a_cnt & 1u], (a_cnt >> 1) & 1u, wc, CL_DEV_TIMEOUT);
            a_slot = (a_cnt & 1u) * slot_bytes;
            ++a_cnt;
            const uint8_t *As = sm.arena + a_slot;
            if (use_rms == RMS_LOCAL) {  // four threads per row, interleaved 16-byte chunks
                const int r = tid >> 2, q = tid & 3;
                float s0 = 0.0f, s1 = 0.0f;
                if (r < M) {
                    const uint4 *rowp = reinterpret_cast<const uint4 *>(As + (size_t)r * astride);
                    for (int cc = q; cc < (kslice >> 3); cc += 8) {
                        const uint4 v0 = rowp[cc], v1 = cc + 4 < (kslice >> 3) ? rowp[cc + 4] : make_uint4(0, 0, 0, 0);
                        const __nv_bfloat162 *h0 = reinterpret_cast<const __nv_bfloat162 *>(&v0), *h1 = reinterpret_cast<const __nv_bfloat162 *>(&v1);
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float2 f0 = __bfloat1622float2(h0[e]), f1 = __bfloat1622float2(h1[e]);
                            s0 = fmaf(f0.x, f0.x, s0); s0 = fmaf(f0.y, f0.y, s0);
                            s1 = fmaf(f1.x, f1.x, s1); s1 = fmaf(f1.y, f1.y, s1);
                        }
                    }
                }
                float ss = s0 + s1;
                ss += __shfl_xor_sync(0xffffffffu, ss, 1);
                ss += __shfl_xor_sync(0xffffffffu, ss, 2);
                if (q == 0 && r < M) sm.rms[r] = rsqrtf(ss / (float)K + eps);
            }
        }
        const unsigned stage = cons % CL_STAGES;
        mbar_wait(&sm.full[stage], (cons / CL_STAGES) & 1u, wc, CL_DEV_TIMEOUT);
        const uint32_t w_addr = smem_u32(sm.ring + (size_t)stage * CL_STAGE_BYTES) + b_lane;
        if (c == 0) {
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < NG; ++j)
#pragma unroll
                    for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.0f;
        }
        const uint32_t a_k = a_slot + (uint32_t)cs * (uint32_t)kchunk * 2u;
#pragma unroll 2
        for (int ks = ks0; ks < ks1; ++ks) {
            uint32_t a[2][4];
#pragma unroll
            for (int mtl = 0; mtl < 2; ++mtl) ldsm4(a[mtl], a_off[mtl] + a_k + (uint32_t)ks * 32u);
#pragma unroll
            for (int gp = 0; gp < NG / 2; ++gp) {
                uint32_t b[4];
                ldsm4(b, w_addr + (uint32_t)gp * 16u * wstride + (uint32_t)ks * 32u);
#pragma unroll
                for (int mtl = 0; mtl < 2; ++mtl) {
                    if (!mt_ok[mtl]) continue;
                    mma_bf16(acc[mtl][2 * gp], a[mtl], b[0], b[1]);
                    mma_bf16(acc[mtl][2 * gp + 1], a[mtl], b[2], b[3]);
                }
            }
        }
        __syncwarp();  // every lane's fragments of this stage have been consumed by its products
        if (lane == 0) mbar_arrive(&sm.empty[stage]);
        ++cons;
        if (c + 1 < n_chunks) continue;  // more of this unit's K follows: keep accumulating
        cons_sync();  // the previous unit's epilogue has read the scratch tile
        // ---- epilogue: NG / 2 blocks of 16 columns through the scratch tile
#pragma unroll
        for (int blk = 0; blk < NG / 2; ++blk) {
            if (blk > 0) cons_sync();  // the previous block's sums have been read
            float *dst = sc + (size_t)kq * M * CL_SC_LD;
#pragma unroll
            for (int mtl = 0; mtl < 2; ++mtl)
#pragma unroll
                for (int hr = 0; hr < 2; ++hr) {
                    const int row = (2 * mh + mtl) * 16 + g + hr * 8;
                    if (row >= M) continue;
                    float *rp = dst + (size_t)row * CL_SC_LD + q2;
                    *reinterpret_cast<float2 *>(rp) = make_float2(acc[mtl][2 * blk][2 * hr], acc[mtl][2 * blk][2 * hr + 1]);
                    *reinterpret_cast<float2 *>(rp + 8) = make_float2(acc[mtl][2 * blk + 1][2 * hr], acc[mtl][2 * blk + 1][2 * hr + 1]);
                }
            cons_sync();
            gemm_epilogue(pg, sm, sc, u * (NG / 2) + blk, step, M, N, half, out_mode, use_rms, act, erow, ec4);
        }
    }
    a_cnt_ref = a_cnt;
}

// ----------------------------------------------------------------------------------------------- EMBED
__device__ __noinline__ void embed_phase(const LoopPhase &p, const LoopParams &lp, int step) {
    const Smem sm = get_smem();
    float *xs = reinterpret_cast<float *>(sm.arena);
    const int A = p.A_dim, H = p.H, chunk = p.chunk, sd = p.sd;
    cons_sync();
    for (int i = threadIdx.x; i < chunk * A; i += CL_THREADS) xs[i] = __ldcg(p.x + i);
    float *ss = xs + chunk * A;
    for (int i = threadIdx.x; i < sd; i += CL_THREADS) ss[i] = lp.state[i];
    cons_sync();
    const int nrb = (chunk + CL_EMBED_ROWS - 1) / CL_EMBED_ROWS;
    const int gt = blockIdx.x * CL_THREADS + threadIdx.x, gn = gridDim.x * CL_THREADS;
    for (int item = gt; item < nrb * H; item += gn) {
        const int o = item % H, rb = item / H;
        uint4 wv[8];
        const uint4 *wr = reinterpret_cast<const uint4 *>(p.w_dense + (size_t)o * A);
#pragma unroll
        for (int k8 = 0; k8 < 8; ++k8)
            if (k8 * 8 < A) wv[k8] = __ldg(wr + k8);
        const float bias = p.bias ? p.bias[o] : 0.0f;
        const int rend = min(chunk, (rb + 1) * CL_EMBED_ROWS);
        for (int r = rb * CL_EMBED_ROWS; r < rend; ++r) {
            float acc = bias;
#pragma unroll
            for (int k8 = 0; k8 < 8; ++k8) {
                if (k8 * 8 >= A) break;
                const __nv_bfloat162 *h2 = reinterpret_cast<const __nv_bfloat162 *>(&wv[k8]);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 f = __bfloat1622float2(h2[e]);
                    acc = fmaf(f.x, xs[r * A + k8 * 8 + 2 * e], acc);
                    acc = fmaf(f.y, xs[r * A + k8 * 8 + 2 * e + 1], acc);
                }
            }
            if (!p.scale_next) {
                *reinterpret_cast<__nv_bfloat16 *>(p.outp + pad_off(chunk, H, r, o)) = __float2bfloat16(acc);
            } else {
                // pi0.5: the embedding IS the residual stream (rows = action tokens); mirror with the first norm's (1 + scale),
                // sums of squares per 32 columns (a warp holds 32 consecutive columns of one row block)
                __stcg(p.h + (size_t)r * H + o, acc);
                const float sn = p.scale_next[(size_t)step * p.mod_stride + o];
                *reinterpret_cast<__nv_bfloat16 *>(p.hbp + pad_off(p.S, H, r, o)) = __float2bfloat16(acc + acc * sn);
                float sq = acc * acc;
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, off);
                if ((threadIdx.x & 31) == 0) __stcg(p.ssq_out + (size_t)(o >> 5) * 64 + r, sq);
            }
        }
    }
    if (sd > 0)  // pi0: the state token is row 0 of the residual stream
        for (int o = gt; o < H; o += gn) {
            const __nv_bfloat16 *wr = p.w2 + (size_t)o * sd;
            float acc = p.b2 ? p.b2[o] : 0.0f;
            for (int k = 0; k < sd; ++k) acc = fmaf(__bfloat162float(wr[k]), ss[k], acc);
            __stcg(p.h + o, acc);
            *reinterpret_cast<__nv_bfloat16 *>(p.hbp + pad_off(p.S, H, 0, o)) = __float2bfloat16(acc);
        }
}

// ------------------------------------------------------------------------------------------- ATTENTION
template <int HD>
__device__ __noinline__ void att_phase(const LoopPhase &pg, const LoopParams &lp, unsigned &a_cnt) {
    const Smem sm = get_smem();
    const WaitCtx wc{sm.abort_flag, lp.status};
    constexpr int SQ = HD * 2 + 16;   // bytes per staged row
    constexpr int NGV = HD / 64;      // 8-column groups of the output per warp
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int mt = warp & 1, kp = warp >> 1;
    const int mi = lane >> 3, lr = lane & 7, g = lane >> 2, q2 = (lane & 3) * 2;
    const int ks = pg.ks, ns = pg.ns, n_rt = pg.n_rt, kv_len = pg.kv_len, R = pg.R, S = pg.S, P = pg.P, cap = pg.cap, mask_mode = pg.mask_mode;
    const int gq = pg.g;
    const float scale_log2 = pg.scale_log2;
    uint8_t *Qs = sm.arena, *Ks = Qs + 32 * SQ, *Vs = Ks + (size_t)ks * SQ, *Ps = Vs + (size_t)ks * SQ;
    const int SP = (ks + 8) * 2;
    const int n_units = pg.n_kv * n_rt * ns;
    int pad_lo = 0, pad_hi = 0;
    if (lp.pad) {
        pad_lo = lp.pad[0];
        pad_hi = lp.pad[1];
    }
    for (int u = blockIdx.x; u < n_units; u += gridDim.x) {
        const int kvh = u / (n_rt * ns), rem = u - kvh * (n_rt * ns), rt = rem / ns, s = rem - rt * ns;
        const int key0 = s * ks, nkeys = min(ks, kv_len - key0), ks16 = (nkeys + 15) & ~15;
        const int row0 = rt * 32, nrows = min(32, R - row0);
        cons_sync();  // the arena is free
        if (tid == 0) {
            uint64_t *bar = &sm.a_full[a_cnt & 1u];
            mbar_expect_tx(bar, (uint32_t)(nrows + 2 * nkeys) * SQ);
            bulk_g2s(Qs, pg.qp + ((size_t)kvh * gq * S + row0) * SQ, (uint32_t)nrows * SQ, bar);
            bulk_g2s(Ks, pg.kpp + ((size_t)kvh * cap + key0) * SQ, (uint32_t)nkeys * SQ, bar);
            bulk_g2s(Vs, pg.vpp + ((size_t)kvh * cap + key0) * SQ, (uint32_t)nkeys * SQ, bar);
        }
        for (int i = tid; i < (ks16 - nkeys) * (HD / 8); i += CL_THREADS) {
            const int r = nkeys + i / (HD / 8), c = i % (HD / 8);
            *reinterpret_cast<uint4 *>(Vs + (size_t)r * SQ + c * 16) = make_uint4(0, 0, 0, 0);
        }
        mbar_wait(&sm.a_full[a_cnt & 1u], (a_cnt >> 1) & 1u, wc, CL_DEV_TIMEOUT);
        ++a_cnt;
        cons_sync();
        // ---- S = Q K^T for this warp's 16 rows and its share of the 8-key groups
        const int ng = ks16 >> 3, g0 = kp * ng / 4, g1 = (kp + 1) * ng / 4, n_g = g1 - g0;  // n_g <= 3
        float sacc[3][4];
#pragma unroll
        for (int i = 0; i < 3; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) sacc[i][e] = 0.0f;
        {
            const int qrow = min(mt * 16 + lr + (mi & 1) * 8, nrows - 1);
            const uint32_t q_addr = smem_u32(Qs) + (uint32_t)qrow * SQ + (uint32_t)(mi >> 1) * 16u;
            const uint32_t k_addr = smem_u32(Ks) + (uint32_t)(g0 * 8 + lr) * SQ + (uint32_t)mi * 16u;
#pragma unroll 2
            for (int kk = 0; kk < HD / 32; ++kk) {
                uint32_t a0[4], a1[4];
                ldsm4(a0, q_addr + kk * 64);
                ldsm4(a1, q_addr + kk * 64 + 32);
#pragma unroll
                for (int gi = 0; gi < 3; ++gi) {
                    if (gi >= n_g) break;
                    uint32_t b[4];
                    ldsm4(b, k_addr + (uint32_t)gi * 8u * SQ + kk * 64);
                    mma_bf16(sacc[gi], a0, b[0], b[1]);
                    mma_bf16(sacc[gi], a1, b[2], b[3]);
                }
            }
        }
        // ---- mask, row maximum over the unit's keys
        const int rl[2] = {mt * 16 + g, mt * 16 + g + 8};
        int jmax[2];
#pragma unroll
        for (int hr = 0; hr < 2; ++hr) {
            const int tok = (row0 + rl[hr]) % S;
            const int n_suf = kv_len - P;
            int limit = n_suf;
            if (mask_mode == 2) limit = min(tok + 1, n_suf);
            else if (mask_mode == 1) limit = tok == 0 ? min(1, n_suf) : n_suf;
            jmax[hr] = min(P + limit, key0 + nkeys);
        }
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int gi = 0; gi < 3; ++gi) {
            if (gi >= n_g) break;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int j = key0 + (g0 + gi) * 8 + q2 + (e & 1), hr = e >> 1;
                const bool vis = j < jmax[hr] && !(j >= pad_lo && j < pad_hi);
                sacc[gi][e] = vis ? sacc[gi][e] * scale_log2 : -INFINITY;
                mx[hr] = fmaxf(mx[hr], sacc[gi][e]);
            }
        }
#pragma unroll
        for (int hr = 0; hr < 2; ++hr) {
            mx[hr] = fmaxf(mx[hr], __shfl_xor_sync(0xffffffffu, mx[hr], 1));
            mx[hr] = fmaxf(mx[hr], __shfl_xor_sync(0xffffffffu, mx[hr], 2));
            if ((lane & 3) == 0) sm.red_max[rl[hr] * 4 + kp] = mx[hr];
        }
        cons_sync();
        float sum[2] = {0.0f, 0.0f};
#pragma unroll
        for (int hr = 0; hr < 2; ++hr) {
            const float *rm = sm.red_max + rl[hr] * 4;
            const float m = fmaxf(fmaxf(rm[0], rm[1]), fmaxf(rm[2], rm[3]));
            mx[hr] = m == -INFINITY ? 0.0f : m;
        }
#pragma unroll
        for (int gi = 0; gi < 3; ++gi) {
            if (gi >= n_g) break;
            float pv[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                pv[e] = ex2f(sacc[gi][e] - mx[e >> 1]);
                sum[e >> 1] += pv[e];
            }
            const int col = (g0 + gi) * 8 + q2;
            *reinterpret_cast<uint32_t *>(Ps + (size_t)rl[0] * SP + col * 2) = pack_bf16(pv[0], pv[1]);
            *reinterpret_cast<uint32_t *>(Ps + (size_t)rl[1] * SP + col * 2) = pack_bf16(pv[2], pv[3]);
        }
#pragma unroll
        for (int hr = 0; hr < 2; ++hr) {
            sum[hr] += __shfl_xor_sync(0xffffffffu, sum[hr], 1);
            sum[hr] += __shfl_xor_sync(0xffffffffu, sum[hr], 2);
            if ((lane & 3) == 0) sm.red_sum[rl[hr] * 4 + kp] = sum[hr];
        }
        cons_sync();
        // ---- O = P V: this warp's HD / 8 output columns, all 32 rows
        float oacc[2][NGV][4];
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int j = 0; j < NGV; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) oacc[i][j][e] = 0.0f;
        const int c0 = warp * (HD / 8);
        {
            const uint32_t p_addr = smem_u32(Ps) + (uint32_t)(lr + (mi & 1) * 8) * SP + (uint32_t)(mi >> 1) * 16u;
            const uint32_t v_addr = smem_u32(Vs) + (uint32_t)(lr + (mi & 1) * 8) * SQ + (uint32_t)(c0 + (NGV > 1 ? (mi >> 1) * 8 : 0)) * 2u;
            for (int kk = 0; kk < (ks16 >> 4); ++kk) {
                uint32_t a[2][4];
                ldsm4(a[0], p_addr + kk * 32);
                ldsm4(a[1], p_addr + 16 * SP + kk * 32);
                if (NGV == 1) {
                    uint32_t b[2];
                    ldsm2_t(b, v_addr + (uint32_t)kk * 16u * SQ);
                    mma_bf16(oacc[0][0], a[0], b[0], b[1]);
                    mma_bf16(oacc[1][0], a[1], b[0], b[1]);
                } else {
#pragma unroll
                    for (int gp = 0; gp < NGV / 2; ++gp) {
                        uint32_t b[4];
                        ldsm4_t(b, v_addr + (uint32_t)kk * 16u * SQ + gp * 32);
                        mma_bf16(oacc[0][2 * gp], a[0], b[0], b[1]);
                        mma_bf16(oacc[1][2 * gp], a[1], b[0], b[1]);
                        mma_bf16(oacc[0][2 * gp + 1], a[0], b[2], b[3]);
                        mma_bf16(oacc[1][2 * gp + 1], a[1], b[2], b[3]);
                    }
                }
            }
        }
        float *wo = pg.ws_o + (size_t)u * 32 * HD;
#pragma unroll
        for (int m2 = 0; m2 < 2; ++m2)
#pragma unroll
            for (int hr = 0; hr < 2; ++hr) {
                const int row = m2 * 16 + g + hr * 8;
                if (row >= nrows) continue;
#pragma unroll
                for (int j = 0; j < NGV; ++j)
                    __stcg(reinterpret_cast<float2 *>(wo + (size_t)row * HD + c0 + j * 8 + q2), make_float2(oacc[m2][j][2 * hr], oacc[m2][j][2 * hr + 1]));
            }
        if (tid < 32 && tid < nrows) {
            const float *rm = sm.red_max + tid * 4, *rs = sm.red_sum + tid * 4;
            const float m = fmaxf(fmaxf(rm[0], rm[1]), fmaxf(rm[2], rm[3]));
            const float l = ((rs[0] + rs[1]) + rs[2]) + rs[3];
            __stcg(reinterpret_cast<float2 *>(pg.ws_ml + ((size_t)u * 32 + tid) * 2), make_float2(m, l));
        }
    }
}

template <int HD>
__device__ __forceinline__ void combine_phase(const LoopPhase &p) {
    const int R = p.R, S = p.S, ns = p.ns, n_rt = p.n_rt, gq = p.g, out_rows = p.out_rows, out_kslice = p.out_kslice;
    const int items = p.n_kv * R * (HD / 4);
    const float2 *ml = reinterpret_cast<const float2 *>(p.ws_ml);
    for (int it = blockIdx.x * CL_THREADS + threadIdx.x; it < items; it += gridDim.x * CL_THREADS) {
        const int c4 = it % (HD / 4), rr = it / (HD / 4);
        const int kvh = rr / R, r = rr - kvh * R, rt = r >> 5, rl = r & 31;
        const int u0 = (kvh * n_rt + rt) * ns;
        float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
        float L = 0.0f, mmax = -INFINITY;
        for (int s0 = 0; s0 < ns; s0 += 8) {
            float2 m[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) m[j] = s0 + j < ns ? __ldcg(ml + (size_t)(u0 + s0 + j) * 32 + rl) : make_float2(-INFINITY, 0.0f);
#pragma unroll
            for (int j = 0; j < 8; ++j) mmax = fmaxf(mmax, m[j].x);
        }
        for (int s0 = 0; s0 < ns; s0 += 8) {
            float2 m[8];
            float4 v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (s0 + j < ns) {
                    m[j] = __ldcg(ml + (size_t)(u0 + s0 + j) * 32 + rl);
                    v[j] = __ldcg(reinterpret_cast<const float4 *>(p.ws_o + ((size_t)(u0 + s0 + j) * 32 + rl) * HD) + c4);
                }
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (s0 + j < ns && m[j].x != -INFINITY) {
                    const float w = ex2f(m[j].x - mmax);
                    o.x = fmaf(w, v[j].x, o.x); o.y = fmaf(w, v[j].y, o.y); o.z = fmaf(w, v[j].z, o.z); o.w = fmaf(w, v[j].w, o.w);
                    L = fmaf(w, m[j].y, L);
                }
        }
        const float inv = L > 0.0f ? 1.0f / L : 0.0f;
        const int head_l = r / S, tok = r - head_l * S;
        const int col = (kvh * gq + head_l) * HD + c4 * 4;
        __stcg(reinterpret_cast<uint2 *>(p.outp + pad_off(out_rows, out_kslice, tok, col)),
               make_uint2(pack_bf16(o.x * inv, o.y * inv), pack_bf16(o.z * inv, o.w * inv)));
    }
}

// prefix rows of the engine's K / V pages (observation 0) -> the padded pages the attention tiles are copied from
__device__ __noinline__ void pages_prologue(const LoopParams &lp) {
    const int c16 = lp.hd / 8;  // 16-byte chunks per row
    const size_t per_layer = (size_t)lp.n_kv * lp.P * c16, total = per_layer * lp.L;
    const uint32_t sq = (uint32_t)lp.hd * 2u + 16u;
    for (size_t i = (size_t)blockIdx.x * CL_THREADS + threadIdx.x; i < total; i += (size_t)gridDim.x * CL_THREADS) {
        const int l = (int)(i / per_layer);
        size_t r = i - (size_t)l * per_layer;
        const int c = (int)(r % c16);
        r /= c16;
        const int tok = (int)(r % lp.P), kvh = (int)(r / lp.P);
        const size_t so = (size_t)l * lp.src_layer_stride + ((size_t)kvh * lp.cap + tok) * lp.hd + (size_t)c * 8;
        const size_t dof = ((size_t)l * lp.n_kv * lp.cap + (size_t)kvh * lp.cap + tok) * sq + (size_t)c * 16;
        __stcg(reinterpret_cast<uint4 *>(lp.kpp + dof), __ldg(reinterpret_cast<const uint4 *>(lp.k_src + so)));
        __stcg(reinterpret_cast<uint4 *>(lp.vpp + dof), __ldg(reinterpret_cast<const uint4 *>(lp.v_src + so)));
    }
}

// ---------------------------------------------------------------------------------------------- kernel
// One instantiation per head_dim: the kernel's code has to stay small (each phase runs its code once every few microseconds
// and what does not fit the SM's instruction cache is fetched from L2 every time).
template <int HD>
__global__ void __launch_bounds__(CL_BLOCK, 1) chunk_loop_kernel(const __grid_constant__ LoopParams lp) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    if (threadIdx.x == 0) *reinterpret_cast<int *>(smem_raw + 124) = lp.n_wtab;
    __syncthreads();
    const Smem sm = get_smem();
    WEntry *wtab = reinterpret_cast<WEntry *>(smem_raw + CL_WTAB_OFF);
    if (threadIdx.x == 0) {
        for (int i = 0; i < CL_STAGES; ++i) {
            mbar_init(&sm.full[i], 1);
            mbar_init(&sm.empty[i], CL_THREADS / 32);
        }
        mbar_init(&sm.a_full[0], 1);
        mbar_init(&sm.a_full[1], 1);
        mbar_init(sm.done, 1);
        *sm.abort_flag = 0;
        fence_barrier_init();
    }
    for (int i = threadIdx.x; i < lp.n_wtab * 8; i += CL_BLOCK)
        reinterpret_cast<uint32_t *>(wtab)[i] = reinterpret_cast<const uint32_t *>(lp.wtab)[i];
    // descriptor of phase 0 into slot 0; from then on every phase fetches its successor's while it works
    for (int i = threadIdx.x; i < (int)(sizeof(LoopPhase) / 4); i += CL_BLOCK)
        reinterpret_cast<uint32_t *>(smem_raw + CL_DESC_OFF)[i] = reinterpret_cast<const uint32_t *>(lp.phases)[i];
    __syncthreads();
    if (threadIdx.x >= CL_THREADS) {  // the feeder warp: lane 0 works, the warp takes no part in any later barrier
        if (threadIdx.x == CL_THREADS) feeder_loop(lp);
        return;
    }
    const WaitCtx wc{sm.abort_flag, lp.status};
    unsigned cons = 0, a_cnt = 0, barriers = 0, seq = 0;
    pages_prologue(lp);
    ++barriers;
    bool ok = grid_barrier(lp, barriers * gridDim.x, sm, wc);
    for (int step = 0; ok && step < lp.steps; ++step) {
        for (int ph = 0; ok && ph < lp.n_phases; ++ph, ++seq) {
            const LoopPhase &p = *reinterpret_cast<const LoopPhase *>(smem_raw + CL_DESC_OFF + (seq & 1u) * CL_DESC_BYTES);
            if (threadIdx.x < (int)(sizeof(LoopPhase) / 16)) {  // the next phase's descriptor: asynchronous 16-byte copies
                const int nx = ph + 1 == lp.n_phases ? 0 : ph + 1;
                const uint32_t dst = smem_u32(smem_raw + CL_DESC_OFF + ((seq + 1) & 1u) * CL_DESC_BYTES) + threadIdx.x * 16u;
                const uint8_t *src = reinterpret_cast<const uint8_t *>(lp.phases + nx) + threadIdx.x * 16u;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
                asm volatile("cp.async.commit_group;" ::: "memory");
            }
            switch (p.type) {
            case PH_GEMM:
                gemm_phase<2>(p, lp, step, cons, a_cnt);
                break;
            case PH_EMBED: embed_phase(p, lp, step); break;
            case PH_ATT:
                att_phase<HD>(p, lp, a_cnt);
                break;
            default:
                combine_phase<HD>(p);
                break;
            }
            asm volatile("cp.async.wait_all;" ::: "memory");
            ++barriers;
            ok = grid_barrier(lp, barriers * gridDim.x, sm, wc);
            if (lp.trace && blockIdx.x == 0 && threadIdx.x == 0) {
                unsigned long long t;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
                lp.trace[barriers - 2] = t;
            }
        }
    }
    // Weight chunks still on their way must land before the CTA gives its shared memory back (only after a failure are
    // there any: the feeder stops with the computation).
    if (threadIdx.x == 0 && mbar_wait(sm.done, 0u, wc, CL_DEV_TIMEOUT)) {
        const unsigned issued = *reinterpret_cast<volatile unsigned *>(smem_raw + 384);
        for (unsigned i = cons; i < issued; ++i) mbar_wait(&sm.full[i % CL_STAGES], (i / CL_STAGES) & 1u, wc, CL_DEV_TIMEOUT);
    }
    cons_sync();
}

// dense [rows][K] bf16 -> padded image with K slices of `kslice` columns (the pad bytes stay zero)
__global__ void pad_image_kernel(const __nv_bfloat16 *__restrict__ src, uint8_t *__restrict__ dst, int rows, int K, int kslice) {
    const size_t total = (size_t)rows * (K / 8);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int row = (int)(i / (K / 8)), col = (int)(i % (K / 8)) * 8;
        *reinterpret_cast<uint4 *>(dst + pad_off(rows, kslice, row, col)) = *reinterpret_cast<const uint4 *>(src + (size_t)row * K + col);
    }
}

// pi0.5: the adaptive norm's shift passes through the projection as a per-column constant,
// out[s][n] = (add ? add[n] : 0) + sum_k W[n][k] shift_s[k]   (shift_s = shift + s * stride; one warp per (s, n))
__global__ void shift_bias_kernel(const __nv_bfloat16 *__restrict__ W, const float *__restrict__ shift, size_t stride, const float *__restrict__ add,
                                  float *__restrict__ out, int steps, int N, int K) {
    const size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= (size_t)steps * N) return;
    const int s = (int)(warp / N), n = (int)(warp % N);
    const __nv_bfloat16 *wr = W + (size_t)n * K;
    const float *sh = shift + (size_t)s * stride;
    float acc = 0.0f;
    for (int k = lane; k < K; k += 32) acc = fmaf(__bfloat162float(wr[k]), sh[k], acc);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (lane == 0) out[warp] = acc + (add ? add[n] : 0.0f);
}

}  // namespace

// ------------------------------------------------------------------------------------------------ host
struct ChunkLoop {
    const void *kernel = nullptr;
    DevBuf phases, wtab, counter, ws_o, ws_ml, trace;
    DevBuf hbp, ap, m1p, attp, gp, qp, kpp, vpp;  // padded activations and pages
    DevBuf ssq;                                    // [H / 16][64] partial sums of squares of the residual mirror
    std::vector<DevBuf> cvec;                      // pi0.5: the shift terms of every norm, [steps][N] each
    std::vector<DevBuf> wp;                        // padded weights
    int n_phases = 0, steps = 0, n_cta = 0;
    LoopParams lp{};
};

namespace {

// K slices of a projection's A operand: one when all of K (<= 1024 columns) fits the arena beside the scratch tile, else the
// fewest of at most 512 columns such that TWO of them fit (they alternate: the next slice loads while this one is
// multiplied).  The slices of a unit run back to back on one CTA and accumulate in registers.
int choose_kslices(int K, int M) {
    if (K <= CL_MAX_KSLICE && K % 16 == 0 && (size_t)M * (K * 2 + 16) + (size_t)4 * M * CL_SC_ROW <= (size_t)CL_ARENA) return 1;
    for (int ks = 2; ks <= 64; ++ks) {
        if (K % ks) continue;
        const int kslice = K / ks;
        if (kslice % 16 || kslice > 512) continue;
        if ((size_t)2 * M * (kslice * 2 + 16) + (size_t)4 * M * CL_SC_ROW > (size_t)CL_ARENA) continue;
        return ks;
    }
    return 0;
}

// columns per weight chunk of a unit of `ng` groups: the largest divisor of the A slice that is a multiple of 16 and fits a ring stage
int pick_kchunk(int kslice, int ng) {
    for (int kc = std::min(kslice, CL_MAX_KSLICE); kc >= 16; --kc)
        if (kslice % kc == 0 && kc % 16 == 0 && (size_t)ng * 8 * (kc * 2 + 16) <= (size_t)CL_STAGE_BYTES) return kc;
    return 0;
}

size_t image_bytes(int rows, int K, int kslices) { return (size_t)kslices * rows * ((size_t)(K / kslices) * 2 + 16); }

}  // namespace

int chunk_loop_create(const ChunkLoopDesc &d, ChunkLoop **out) {
    *out = nullptr;
    const int n_sm = sm_count();
    if (n_sm <= 0) return VLAB200_ERR_CUDA;
    const int hd = d.hd, half = hd / 2, qf = d.n_q * hd, H = d.H, S = d.S;
    if (d.model < 0 || d.model > 2 || (d.model == 2 && (!d.mods || H % 32))) return VLAB200_ERR_UNSUPPORTED;
    if (hd != 64 && hd != 128 && hd != 256) return VLAB200_ERR_UNSUPPORTED;
    if (S > 64 || H % 16 || H > CL_MAX_KSLICE || d.A % 16 || (2 * d.I) % 16 || qf % 16 || d.I % 16) return VLAB200_ERR_UNSUPPORTED;
    if ((size_t)S * (H * 2 + 16) + (size_t)4 * S * CL_SC_ROW > (size_t)CL_ARENA) return VLAB200_ERR_UNSUPPORTED;
    if ((size_t)(d.chunk * d.A + 64) * 4 > (size_t)CL_ARENA || d.A > 64) return VLAB200_ERR_UNSUPPORTED;
    int occ = 0;
    const void *kernel = hd == 64    ? reinterpret_cast<const void *>(chunk_loop_kernel<64>)
                         : hd == 128 ? reinterpret_cast<const void *>(chunk_loop_kernel<128>)
                                     : reinterpret_cast<const void *>(chunk_loop_kernel<256>);
    if (ensure_dyn_smem(kernel, CL_SMEM)) return VLAB200_ERR_CUDA;
    VB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kernel, CL_BLOCK, CL_SMEM));
    int coop = 0, dev = 0;
    VB_CUDA(cudaGetDevice(&dev));
    VB_CUDA(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev));
    if (occ < 1 || !coop) return VLAB200_ERR_UNSUPPORTED;
    const int n_cta = n_sm;
    const int g = d.n_q / d.n_kv, R = g * S, n_rt = (R + 31) / 32;
    const int ks_o = choose_kslices(qf, S), ks_d = choose_kslices(d.I, S);
    if (!ks_o || !ks_d) return VLAB200_ERR_UNSUPPORTED;

    ChunkLoop *cl = new (std::nothrow) ChunkLoop();
    if (!cl) return VLAB200_ERR_CUDA;
    int rc = VLAB200_OK;
    auto fail = [&](int code) {
        delete cl;
        return code;
    };
    const uint32_t sq = (uint32_t)hd * 2u + 16u;
    const size_t page_layer = (size_t)d.n_kv * d.cap * sq;
    if ((rc = cl->hbp.alloc(image_bytes(S, H, 1))) || (rc = cl->ap.alloc(image_bytes(d.chunk, H, 1))) ||
        (rc = cl->m1p.alloc(image_bytes(d.chunk, H, 1))) || (rc = cl->attp.alloc(image_bytes(S, qf, ks_o))) ||
        (rc = cl->gp.alloc(image_bytes(S, d.I, ks_d))) || (rc = cl->qp.alloc((size_t)d.n_q * S * sq)) ||
        (rc = cl->kpp.alloc(page_layer * d.L)) || (rc = cl->vpp.alloc(page_layer * d.L)) || (rc = cl->ssq.alloc((size_t)(H / 16) * 64 * 4)))
        return fail(rc);
    for (DevBuf *b : {&cl->hbp, &cl->ap, &cl->m1p, &cl->attp, &cl->gp, &cl->qp})
        if (cudaMemset(b->p, 0, 16) != cudaSuccess) return fail(VLAB200_ERR_CUDA);
    if (cudaMemset(cl->hbp.p, 0, image_bytes(S, H, 1)) != cudaSuccess || cudaMemset(cl->ap.p, 0, image_bytes(d.chunk, H, 1)) != cudaSuccess ||
        cudaMemset(cl->m1p.p, 0, image_bytes(d.chunk, H, 1)) != cudaSuccess || cudaMemset(cl->attp.p, 0, image_bytes(S, qf, ks_o)) != cudaSuccess ||
        cudaMemset(cl->gp.p, 0, image_bytes(S, d.I, ks_d)) != cudaSuccess || cudaMemset(cl->qp.p, 0, (size_t)d.n_q * S * sq) != cudaSuccess ||
        cudaMemset(cl->kpp.p, 0, page_layer * d.L) != cudaSuccess || cudaMemset(cl->vpp.p, 0, page_layer * d.L) != cudaSuccess)
        return fail(VLAB200_ERR_CUDA);
    // padded weight images
    auto pad_weight = [&](const void *w, int rows, int K, int kslices, const uint8_t **image) -> int {
        cl->wp.emplace_back();
        DevBuf &b = cl->wp.back();
        const size_t bytes = image_bytes(rows, K, kslices);
        int r = b.alloc(bytes);
        if (r) return r;
        VB_CUDA(cudaMemset(b.p, 0, bytes));
        pad_image_kernel<<<n_sm * 4, 256>>>(static_cast<const __nv_bfloat16 *>(w), b.as<uint8_t>(), rows, K, K / kslices);
        VB_CUDA(cudaGetLastError());
        *image = b.as<uint8_t>();
        return VLAB200_OK;
    };
    cl->wp.reserve((size_t)d.L * 4 + 8);

    std::vector<LoopPhase> ph;
    bool bad = false;
    auto gemm = [&](const uint8_t *Ap, int M, const void *w_dense, int N, int K, int kslices, int out_mode) {
        LoopPhase p{};
        p.type = PH_GEMM; p.out_mode = out_mode; p.Ap = Ap; p.M = M; p.N = N; p.K = K; p.kslices = kslices;
        p.ng = 2;  // units of 4 groups (half as many, twice the weight bytes each) measured 2-5 % slower, and their code costs instruction cache
        p.kchunk = pick_kchunk(K / kslices, p.ng);
        p.n_sub = N / (8 * p.ng);
        p.eps = d.rms_eps; p.S = S; p.chunk = d.chunk;
        if (!p.kchunk || pad_weight(w_dense, N, K, K / p.kchunk, &p.Wp)) bad = true;
        return p;
    };
    size_t ws_units = 0;
    const bool ada = d.model == 2;
    const size_t mod_step = (size_t)3 * H, mod_block = (size_t)d.steps * mod_step;  // one norm's vectors for every step
    auto mod_in = [&](int l) { return d.mods + (size_t)(2 * l) * mod_block; };
    auto mod_post = [&](int l) { return d.mods + (size_t)(2 * l + 1) * mod_block; };
    const float *mod_final = ada ? d.mods + (size_t)(2 * d.L) * mod_block : nullptr;
    // W shift (+ bias) of a norm whose output feeds `w_dense` [N][H]
    auto shift_bias = [&](const void *w_dense, int N, const float *mod, const float *add, const float **out_vec) -> int {
        cl->cvec.emplace_back();
        DevBuf &b = cl->cvec.back();
        int r = b.alloc((size_t)d.steps * N * 4);
        if (r) return r;
        const size_t warps = (size_t)d.steps * N;
        shift_bias_kernel<<<(unsigned)((warps * 32 + 255) / 256), 256>>>(static_cast<const __nv_bfloat16 *>(w_dense), mod + H, mod_step, add,
                                                                          b.as<float>(), d.steps, N, H);
        VB_CUDA(cudaGetLastError());
        *out_vec = b.as<float>();
        return VLAB200_OK;
    };
    cl->cvec.reserve((size_t)d.L * 2 + 2);
    // ---- suffix embedding
    {
        LoopPhase p{};
        p.type = PH_EMBED; p.w_dense = static_cast<const __nv_bfloat16 *>(d.w_ain); p.bias = d.b_ain; p.x = d.x;
        p.outp = cl->ap.as<uint8_t>(); p.chunk = d.chunk; p.A_dim = d.A; p.H = H; p.S = S;
        p.sd = d.model == 0 ? d.sd : 0; p.w2 = static_cast<const __nv_bfloat16 *>(d.w_sp); p.b2 = d.b_sp; p.h = d.h;
        p.hbp = cl->hbp.as<uint8_t>();
        if (ada) {  // the embedding is the residual stream; its mirror carries the first norm's (1 + scale)
            p.scale_next = mod_in(0); p.mod_stride = (long long)mod_step; p.ssq_out = cl->ssq.as<float>();
        }
        ph.push_back(p);
        if (!ada) {
            LoopPhase m1 = gemm(cl->ap.as<uint8_t>(), d.chunk, d.w_at1l, H, H, 1, OUT_BIAS_ACT);
            m1.act = ACT_SILU; m1.bias = d.tvec; m1.bias_step_stride = H; m1.outp = cl->m1p.as<uint8_t>(); m1.out_rows = d.chunk; m1.out_kslice = H;
            ph.push_back(m1);
            LoopPhase m2 = gemm(cl->m1p.as<uint8_t>(), d.chunk, d.w_at2, H, H, 1, OUT_BIAS_ACT);
            m2.act = ACT_NONE; m2.bias = d.b_at2; m2.outp = cl->hbp.as<uint8_t>(); m2.out_rows = S; m2.out_kslice = H; m2.out_f32 = d.h;
            m2.row_off = S - d.chunk;
            ph.push_back(m2);
        }
    }
    for (int l = 0; l < d.L; ++l) {
        const bool self = d.is_self[l];
        uint8_t *kp = cl->kpp.as<uint8_t>() + (size_t)l * page_layer, *vp = cl->vpp.as<uint8_t>() + (size_t)l * page_layer;
        const int n_heads = d.n_q + (self ? 2 * d.n_kv : 0);
        LoopPhase qkv = gemm(cl->hbp.as<uint8_t>(), S, d.wqkv[l], n_heads * hd, H, 1, OUT_QKV);
        qkv.use_rms = (l == 0 && !ada) ? RMS_LOCAL : RMS_PARTS; qkv.ssq_in = cl->ssq.as<float>(); qkv.ssq_n = (l == 0 && ada) ? H / 32 : H / 16;
        qkv.half = half; qkv.qp = cl->qp.as<uint8_t>();
        if (ada) {
            if ((rc = shift_bias(d.wqkv[l], n_heads * hd, mod_in(l), nullptr, &qkv.bias))) return fail(rc);
            qkv.bias_step_stride = n_heads * hd;
        }
        qkv.kpp = kp; qkv.vpp = vp; qkv.rope = self ? d.rope_self : d.rope_cross; qkv.n_q = d.n_q; qkv.n_kvp = self ? d.n_kv : 0;
        qkv.cap = d.cap; qkv.P = d.P;
        ph.push_back(qkv);
        LoopPhase at{};
        at.type = PH_ATT; at.hd = hd; at.qp = cl->qp.as<uint8_t>(); at.kpp = kp; at.vpp = vp; at.n_kv = d.n_kv; at.g = g;
        at.S = S; at.R = R; at.n_rt = n_rt; at.kv_len = self ? d.P + S : d.P; at.P = d.P; at.cap = d.cap; at.n_q = d.n_q;
        at.mask_mode = (self && !ada) ? (d.model == 0 ? 1 : 2) : 0;  // pi0.5: every action token sees the prefix and every action token
        at.scale_log2 = 1.4426950408889634f / std::sqrt((float)hd);
        {   // keys per slice: the fewest rounds over the CTAs, then the cheapest unit
            int best = 0;
            double best_cost = 0;
            for (int ks = 16; ks <= 96; ks += 16) {
                if ((size_t)32 * sq + (size_t)2 * ks * sq + (size_t)32 * (ks + 8) * 2 > (size_t)CL_ARENA) continue;
                const int ns = (at.kv_len + ks - 1) / ks;
                if (ns > 64) continue;
                const int units = d.n_kv * n_rt * ns;
                const double cost = (double)((units + n_cta - 1) / n_cta) * (600.0 + (double)ks * hd * 0.07) + 10.0 * ns;
                if (!best || cost < best_cost) {
                    best = ks;
                    best_cost = cost;
                }
            }
            if (!best) bad = true;
            at.ks = best ? best : 16;
            at.ns = (at.kv_len + at.ks - 1) / at.ks;
        }
        ws_units = std::max(ws_units, (size_t)d.n_kv * n_rt * at.ns);
        ph.push_back(at);
        LoopPhase cb = at;
        cb.type = PH_COMBINE; cb.outp = cl->attp.as<uint8_t>(); cb.out_rows = S; cb.out_kslice = qf / ks_o;
        ph.push_back(cb);
        LoopPhase o = gemm(cl->attp.as<uint8_t>(), S, d.wo[l], H, qf, ks_o, OUT_RESID);
        o.h = d.h; o.hbp = cl->hbp.as<uint8_t>(); o.ssq_out = cl->ssq.as<float>();
        if (ada) {
            o.colscale = mod_in(l) + 2 * H; o.scale_next = mod_post(l); o.mod_stride = (long long)mod_step;
        }
        ph.push_back(o);
        LoopPhase gu = gemm(cl->hbp.as<uint8_t>(), S, d.wgu[l], 2 * d.I, H, 1, OUT_GATED);
        gu.use_rms = RMS_PARTS; gu.ssq_in = cl->ssq.as<float>(); gu.ssq_n = H / 16;
        gu.act = d.act; gu.outp = cl->gp.as<uint8_t>(); gu.out_rows = S; gu.out_kslice = d.I / ks_d;
        if (ada) {
            if ((rc = shift_bias(d.wgu[l], 2 * d.I, mod_post(l), nullptr, &gu.bias))) return fail(rc);
            gu.bias_step_stride = 2 * d.I;
        }
        ph.push_back(gu);
        LoopPhase dn = gemm(cl->gp.as<uint8_t>(), S, d.wdown[l], H, d.I, ks_d, OUT_RESID);
        dn.h = d.h; dn.hbp = cl->hbp.as<uint8_t>(); dn.ssq_out = cl->ssq.as<float>();
        if (ada) {
            dn.colscale = mod_post(l) + 2 * H; dn.scale_next = l + 1 < d.L ? mod_in(l + 1) : mod_final; dn.mod_stride = (long long)mod_step;
        }
        ph.push_back(dn);
    }
    {
        LoopPhase hdp = gemm(cl->hbp.as<uint8_t>(), S, d.w_aout, d.A, H, 1, OUT_EULER);
        hdp.use_rms = RMS_PARTS; hdp.ssq_in = cl->ssq.as<float>(); hdp.ssq_n = H / 16; hdp.bias = d.b_aout; hdp.x = d.x; hdp.dt = -1.0f / (float)d.steps;
        if (ada) {
            if ((rc = shift_bias(d.w_aout, d.A, mod_final, d.b_aout, &hdp.bias))) return fail(rc);
            hdp.bias_step_stride = d.A;
        }
        ph.push_back(hdp);
    }
    if (bad) return fail(VLAB200_ERR_UNSUPPORTED);
    if ((rc = cl->ws_o.alloc(ws_units * 32 * hd * 4)) || (rc = cl->ws_ml.alloc(ws_units * 32 * 2 * 4)) ||
        (rc = cl->phases.alloc(ph.size() * sizeof(LoopPhase))) || (rc = cl->counter.alloc(64)))
        return fail(rc);
    for (LoopPhase &p : ph)
        if (p.type == PH_ATT || p.type == PH_COMBINE) {
            p.ws_o = cl->ws_o.as<float>();
            p.ws_ml = cl->ws_ml.as<float>();
        }
    std::vector<WEntry> wt;
    for (const LoopPhase &p : ph)
        if (p.type == PH_GEMM) {
            WEntry w{};
            w.Wp = p.Wp; w.n_units = p.n_sub; w.n_chunks = p.K / p.kchunk; w.N = p.N; w.half = p.half; w.ng = p.ng;
            w.stride = (uint32_t)p.kchunk * 2u + 16u;
            wt.push_back(w);
        }
    if ((int)wt.size() > CL_WTAB_MAX) return fail(VLAB200_ERR_UNSUPPORTED);
    if ((rc = cl->wtab.alloc(wt.size() * sizeof(WEntry)))) return fail(rc);
    cudaError_t ce = cudaMemcpy(cl->wtab.p, wt.data(), wt.size() * sizeof(WEntry), cudaMemcpyHostToDevice);
    if (ce == cudaSuccess) ce = cudaMemcpy(cl->phases.p, ph.data(), ph.size() * sizeof(LoopPhase), cudaMemcpyHostToDevice);
    if (ce == cudaSuccess) ce = cudaDeviceSynchronize();  // the padded weight images are complete
    if (ce != cudaSuccess) {
        delete cl;
        return cuda_fail(ce, "chunk loop: phase table / weight images");
    }
    cl->n_phases = (int)ph.size();
    cl->steps = d.steps;
    cl->n_cta = n_cta;
    cl->kernel = kernel;
    LoopParams &lp = cl->lp;
    lp.phases = cl->phases.as<LoopPhase>();
    lp.n_phases = cl->n_phases;
    lp.wtab = cl->wtab.p;
    lp.n_wtab = (int)wt.size();
    lp.steps = d.steps;
    lp.counter = cl->counter.as<unsigned>();
    lp.status = device_status_ptr();
    lp.k_src = static_cast<const __nv_bfloat16 *>(d.k_pages);
    lp.v_src = static_cast<const __nv_bfloat16 *>(d.v_pages);
    lp.kpp = cl->kpp.as<uint8_t>();
    lp.vpp = cl->vpp.as<uint8_t>();
    lp.src_layer_stride = d.layer_stride;
    lp.L = d.L; lp.n_kv = d.n_kv; lp.cap = d.cap; lp.P = d.P; lp.hd = hd;
    *out = cl;
    return VLAB200_OK;
}

void chunk_loop_free(ChunkLoop *cl) { delete cl; }

int chunk_loop_phases(const ChunkLoop *cl) { return cl ? cl->n_phases : 0; }

int chunk_loop_run(ChunkLoop *cl, const float *state, const int32_t *pad, cudaStream_t stream) {
    if (!cl) return VLAB200_ERR_ARG;
    VB_CUDA(cudaMemsetAsync(cl->counter.p, 0, 4, stream));
    LoopParams lp = cl->lp;
    lp.state = state;
    lp.pad = pad;
    const char *trace_path = std::getenv("VLAB200_CHUNK_LOOP_TRACE");  // developer aid: per-phase durations into a text file
    if (trace_path) {
        if (!cl->trace.p && cl->trace.alloc((size_t)(cl->n_phases * cl->steps + 1) * 8)) return VLAB200_ERR_CUDA;
        lp.trace = cl->trace.as<unsigned long long>();
    }
    void *args[] = {&lp};
    const cudaError_t le = cudaLaunchCooperativeKernel(cl->kernel, dim3(cl->n_cta), dim3(CL_BLOCK), args, CL_SMEM, stream);
    if (le == cudaErrorCooperativeLaunchTooLarge) {  // fewer SMs than the device reports are ours (a partitioned GPU): not an error of the call
        cudaGetLastError();
        return VLAB200_ERR_UNSUPPORTED;
    }
    if (le != cudaSuccess) return cuda_fail(le, "cudaLaunchCooperativeKernel");
    if (lp.trace) {
        const size_t n = (size_t)cl->n_phases * cl->steps;
        std::vector<unsigned long long> t(n);
        VB_CUDA(cudaStreamSynchronize(stream));
        VB_CUDA(cudaMemcpy(t.data(), lp.trace, n * 8, cudaMemcpyDeviceToHost));
        if (FILE *f = std::fopen(trace_path, "w")) {
            for (size_t i = 1; i < n; ++i) std::fprintf(f, "%d %llu\n", (int)(i % cl->n_phases), t[i] - t[i - 1]);  // phase index, ns
            std::fclose(f);
        }
    }
    return VLAB200_OK;
}

}  // namespace vb
