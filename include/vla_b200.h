/*
 * vla_b200.h -- C ABI of libvla_b200.so: the flow-matching denoise step of vla.cpp
 * policies as hand-written sm_100a CUDA kernels.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless the name ends in _host;
 *   - `stream` is a cudaStream_t passed as void* (NULL = default stream);
 *   - functions only enqueue work (no synchronisation, no allocation unless stated)
 *     and return a vlab200_status; kernels that wait on hardware barriers do so with
 *     a cycle budget and report a timeout through vlab200_device_status();
 *   - matrices are row-major; a linear weight is W[out][in]; bf16 is the raw 16-bit
 *     pattern (__nv_bfloat16).
 *
 * Each entry point names the reference interface it replaces (path:line inside the
 * vla.cpp source tree).
 */
#ifndef VLA_B200_H
#define VLA_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define VLAB200_API __attribute__((visibility("default")))
#define VLAB200_ABI_VERSION 1

typedef enum {
    VLAB200_OK = 0,
    VLAB200_ERR_ARG = -1,         /* null pointer, negative size, misaligned buffer */
    VLAB200_ERR_CUDA = -2,        /* a CUDA call failed; see vlab200_last_error() */
    VLAB200_ERR_DEVICE = -3,      /* a kernel reported a failure in the device status word */
    VLAB200_ERR_UNSUPPORTED = -4  /* shape outside what the kernels implement */
} vlab200_status;

VLAB200_API int32_t vlab200_abi_version(void);

/* Text of the last failure on the calling thread ("" if none). */
VLAB200_API const char *vlab200_last_error(void);

/* Synchronises the current device and reads its status word (0 = no kernel reported a
 * failure; 101..104 = a bounded wait inside a kernel ran out).  reset != 0 clears it. */
VLAB200_API int32_t vlab200_device_status(int32_t *out, int32_t reset);

/* ---------------------------------------------------------------- BitVLA ternary path */

/* Per-token absmax int8 quantisation: scales[m] = 127 / max(max_k |x[m][k]|, 1e-5),
 * q = clamp(round_half_even(x * scale), -128, 127).  x: bf16 [M][K], K % 8 == 0.
 * Replaces bitvla_act_quant_cuda (src/kernels/bitvla/bitnet_kernels.cu:118-124, kernel
 * src/kernels/bitvla/bitnet_kernels.h:465-521). */
VLAB200_API int32_t vlab200_act_quant(const void *x_bf16, int8_t *q, float *scales, int32_t M, int32_t K,
                                      void *stream);

/* out[m][n] = bf16( float(acc[m][n]) / s[m] * ws[n / (N / ws_num)] ),
 * acc[m][n] = sum_k A[m][k] * W[n][k] exactly in int32, W in {-2..1} decoded from the
 * reference's 2-bit "ladder" pack (N*K/4 bytes; N % 16 == 0, K % 128 == 0).
 * acc_out (optional, int32 [M][N]) receives the raw accumulators.
 * path: 0 = automatic (M <= 8: HBM-bound GEMV on the packed weights; larger M: tcgen05
 * int8 MMA), 1 = force GEMV, 2 = force tensor-core kernel (needs N % 32 == 0).
 * Replaces bitlinear_int8xint2 / bitlinear_int8xint2_m
 * (src/kernels/bitvla/bitnet_kernels.cu:31-116, kernels bitnet_kernels.h:108-409). */
VLAB200_API int32_t vlab200_ternary_linear(const int8_t *A, const uint8_t *W_ladder, void *out_bf16,
                                           int32_t *acc_out, const float *s, const float *ws, int32_t ws_num,
                                           int32_t M, int32_t N, int32_t K, int32_t path, void *stream);

/* The reference's own symbol names and signatures for the three calls above
 * (src/kernels/bitvla/bitnet_kernels.cu:31,76,118), so src/models/bitvla.cpp and
 * src/kernels/bitvla/bitvla_lm_cuda.cu link against this library unchanged.  The bf16
 * pointers are __nv_bfloat16*, `stream` a cudaStream_t.  Unlike the reference they accept
 * any N % 16 == 0, K % 128 == 0 and report an unsupported shape on stderr instead of
 * aborting the process.  ws_num is inferred from (N, K) exactly as the reference's
 * dispatch table does (gate_up 13824x2560 -> 2, head qkv 3840x2560 -> 3, otherwise 1). */
VLAB200_API void bitlinear_int8xint2(int8_t *input0, int8_t *input1, void *output0, float *s, float *ws, int M,
                                     int N, int K, void *stream);
VLAB200_API void bitlinear_int8xint2_m(int8_t *input0, int8_t *input1, void *output0, float *s, float *ws, int M,
                                       int N, int K, void *stream);
VLAB200_API void bitvla_act_quant_cuda(const void *in, int8_t *out, float *scales, int M, int K, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* VLA_B200_H */
