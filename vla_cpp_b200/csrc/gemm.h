// Interface of the persistent tcgen05 GEMM (gemm.cu) used by the denoise engine.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace vb {

enum { EPI_RESIDUAL = 0, EPI_GATED = 1, EPI_BIAS_ACT = 2 };
enum { ACT_NONE = 0, ACT_SILU = 1, ACT_GELU_TANH = 2, ACT_GELU_ERF = 3 };

struct GemmParams {
    int M, N, K;
    int epi, act, use_rms;
    float eps;
    float *h;               // RESIDUAL: f32 [M][N] read-modify-write
    __nv_bfloat16 *out_bf;  // RESIDUAL: bf16 mirror [M][N]; GATED: [M][N/2]; BIAS_ACT: bf16 output (optional)
    float *out_f32;         // BIAS_ACT: f32 output (optional)
    const float *bias;      // BIAS_ACT, RESIDUAL: [N] (optional)
    const float *colscale;  // RESIDUAL: [N] factor on the projection before it is added (optional; adaRMS gates)
    int ld_out;             // row stride (elements) of out_bf / out_f32 / h
    int rows_in, rows_out, row_off;  // BIAS_ACT row re-mapping (rows_in == 0: identity)
    int scatter_hd, scatter_cap;     // BIAS_ACT into head-major pages: [m / rows_in][n / hd][cap][hd] (0: off)
    int al32;  // set by dense_gemm: h / out_bf rows start on 32-byte boundaries (256-bit epilogue accesses)
    // split-K workspace (optional): float32 [partial_slices][M][N], M <= partial_rows; with it a RESIDUAL problem may run as
    // K slices on separate SMs followed by a fixed-order reduction (ksplit is chosen by dense_gemm)
    float *partial;
    int partial_slices, partial_rows, ksplit;
    int *status;
};

// A: bf16 [M][K] (row stride lda elements), W: bf16 [N][K].
int dense_gemm(const void *A, int lda, const void *W, GemmParams p, cudaStream_t stream);

// NeoX rotation + head split of a fused [M][(n_q + 2 n_kv_proj) hd] bf16 projection into the q buffer
// [M / seq][n_q][seq][hd] and K / V page rows row0 + s (pages [.][n_kv_store][cap][hd]); bitvla_lm.cu.
int rope_split(const void *qkv, const float *cos_t, const float *sin_t, void *q_out, void *k_pages, void *v_pages,
               int M, int seq, int n_q, int n_kv_proj, int n_kv_store, int hd, int cap, int row0, cudaStream_t st);

// 0 = choose the tiling by cost (default); 1 / 2 / 3 / 4 force 128 x 256, 128 x 128, CTA pairs, 128 x 64.
void dense_gemm_set_variant(int v);
int dense_gemm_variant();

}  // namespace vb
