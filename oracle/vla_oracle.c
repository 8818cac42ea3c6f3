/*
 * vla_oracle.c -- CPU restatement of the vla.cpp flow-matching denoise step.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA path is compared
 * against (and the timed CPU baseline of the benchmark).  Nothing in the product
 * library links, loads or calls it.
 *
 * Pinning status (which parts are tied to the reference by something stronger
 * than reading its source):
 *   - ladder int2 packing / ternarisation: pinned against vectors produced by the
 *     reference's own Python packer (scripts/convert_bitvla_to_gguf.py:95-152),
 *     stored under tests/golden/.
 *   - ternary GEMM bf16 outputs and act-quant: pinned on a GPU against the
 *     reference's own CUDA kernels compiled unmodified from
 *     src/kernels/bitvla/bitnet_kernels.{h,cu}.
 *   - sinusoidal time embedding: pinned against the reference's
 *     src/layers/embed.h:61-73 compiled with g++ (vectors under tests/golden/).
 *   - RMSNorm / RoPE / attention / expert layer / Euler loop: PARITY UNPINNED.
 *     The reference runs these through ggml (third party, llama.cpp tag b10331,
 *     fetched at configure time, absent here) and stores no golden outputs, so
 *     this is a restatement from the reference's call sites, cross-checked only
 *     by an independent torch-fp32 twin in tests/.
 *
 * All dense math is float32 (the reference's default: F32 activations, weights
 * whose values are bf16-representable).  `act_bf16` rounds activations to bf16
 * at the points where the CUDA path stores bf16.
 *
 * Layout convention: row-major, token-major.  ggml's [hd, heads, T] is
 * x[t][head][d] here.  A linear weight is W[out][in] (PyTorch order), i.e.
 * y[t][o] = sum_i W[o][i] * x[t][i]            (src/layers/linear.h:24-27).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------ bf16 -- */

static inline float bf16_bits_to_f32(uint16_t h) {
    uint32_t u = ((uint32_t)h) << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* round-to-nearest-even, the conversion __float2bfloat16 performs */
static inline uint16_t f32_to_bf16_bits(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u); /* NaN */
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;
    return (uint16_t)(u >> 16);
}

static inline float bf16_round(float f) { return bf16_bits_to_f32(f32_to_bf16_bits(f)); }

ORC_API void orc_f32_to_bf16(const float *x, int64_t n, uint16_t *out) {
    for (int64_t i = 0; i < n; ++i) out[i] = f32_to_bf16_bits(x[i]);
}
ORC_API void orc_bf16_to_f32(const uint16_t *x, int64_t n, float *out) {
    for (int64_t i = 0; i < n; ++i) out[i] = bf16_bits_to_f32(x[i]);
}
ORC_API int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
/* Launchers such as torchrun export OMP_NUM_THREADS=1; the timed baseline asks for its threads itself. */
ORC_API void orc_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* ------------------------------------------------------- ternary / BitVLA -- */

/* Per-tensor absmean ternarisation.  src/models/bitvla.cpp:430-451,
 * scripts/convert_bitvla_to_gguf.py:95-101. */
ORC_API void orc_ternarize(const float *W, int64_t n, int8_t *t, float *absmean) {
    double s = 0.0;
    for (int64_t i = 0; i < n; ++i) s += fabs((double)W[i]);
    float mean = n > 0 ? (float)(s / (double)n) : 0.0f;
    if (mean < 1e-5f) mean = 1e-5f;
    *absmean = mean;
    const float inv = 1.0f / mean;
    for (int64_t i = 0; i < n; ++i) {
        float q = nearbyintf(W[i] * inv);
        if (q > 1.0f) q = 1.0f;
        if (q < -1.0f) q = -1.0f;
        t[i] = (int8_t)q;
    }
}

/* Slot s of the ladder layout -> (row n, first k of its 16 consecutive k).
 * src/models/bitvla.cpp:453-483, scripts/convert_bitvla_to_gguf.py:103-152. */
static inline void ladder_slot(int64_t s, int64_t K, int64_t *n, int64_t *k) {
    const int64_t slots_per_block = K;            /* 16 rows * K / 16 */
    const int64_t n_block = s / slots_per_block;
    int64_t r = s % slots_per_block;
    const int64_t k0 = r / 128;   r %= 128;
    const int64_t major = r / 32; r %= 32;
    const int64_t y_half = r / 16; r %= 16;
    const int64_t sub_k = r / 8;
    const int64_t y = r % 8;
    *n = n_block * 16 + y_half * 8 + y;
    *k = k0 * 128 + major * 32 + sub_k * 16;
}

/* W: [N][K] values in {-1,0,1}; out: N*K/4 bytes. */
ORC_API int orc_pack_ladder_int2(const int8_t *W, int64_t N, int64_t K, uint8_t *out) {
    if (N % 16 || K % 128) return -1;
    const int64_t n_slots = N * K / 16;
    for (int64_t s = 0; s < n_slots; ++s) {
        int64_t n, k;
        ladder_slot(s, K, &n, &k);
        for (int b = 0; b < 4; ++b) {
            uint8_t v = 0;
            for (int j = 0; j < 4; ++j) {
                const int t = W[n * K + k + b + 4 * j];
                v |= (uint8_t)(((uint8_t)(t + 2) & 3u) << (2 * j));
            }
            out[s * 4 + b] = v;
        }
    }
    return 0;
}

/* Inverse, with the decode arithmetic of the CUDA kernels: code c -> c - 2, so
 * the unused code 0 decodes to -2 (src/kernels/bitvla/bitnet_kernels.h:70-90). */
ORC_API int orc_unpack_ladder_int2(const uint8_t *packed, int64_t N, int64_t K, int8_t *W) {
    if (N % 16 || K % 128) return -1;
    const int64_t n_slots = N * K / 16;
    for (int64_t s = 0; s < n_slots; ++s) {
        int64_t n, k;
        ladder_slot(s, K, &n, &k);
        for (int b = 0; b < 4; ++b)
            for (int j = 0; j < 4; ++j)
                W[n * K + k + b + 4 * j] = (int8_t)(((packed[s * 4 + b] >> (2 * j)) & 3) - 2);
    }
    return 0;
}

/* Per-token absmax int8 quantisation.  src/kernels/bitvla/bitnet_kernels.h:465-521,
 * CPU form src/models/bitvla.cpp:69-96.  x is float (bf16-representable when it
 * mirrors the CUDA kernel's bf16 input). */
ORC_API void orc_act_quant(const float *x, int M, int K, int8_t *q, float *scales) {
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; ++m) {
        const float *row = x + (int64_t)m * K;
        float amax = 0.0f;
        for (int k = 0; k < K; ++k) {
            const float v = fabsf(row[k]);
            if (v > amax) amax = v;
        }
        if (amax < 1e-5f) amax = 1e-5f;
        const float s = 127.0f / amax;
        scales[m] = s;
        for (int k = 0; k < K; ++k) {
            float v = nearbyintf(row[k] * s);
            if (v > 127.0f) v = 127.0f;
            if (v < -128.0f) v = -128.0f;
            q[(int64_t)m * K + k] = (int8_t)v;
        }
    }
}

/* acc[m][n] = sum_k A[m][k] * W[n][k], exact int32, W given unpacked [N][K]. */
ORC_API void orc_gemm_i8_i32(const int8_t *A, const int8_t *W, int M, int N, int K, int32_t *acc) {
#pragma omp parallel for schedule(static) collapse(2)
    for (int m = 0; m < M; ++m)
        for (int n = 0; n < N; ++n) {
            const int8_t *a = A + (int64_t)m * K;
            const int8_t *w = W + (int64_t)n * K;
            int32_t s = 0;
            for (int k = 0; k < K; ++k) s += (int32_t)a[k] * (int32_t)w[k];
            acc[(int64_t)m * N + n] = s;
        }
}

/* Same, but only for the listed rows (rows[i] indexes A); acc is [n_rows][N]. */
ORC_API void orc_gemm_i8_i32_rows(const int8_t *A, const int8_t *W, const int32_t *rows, int n_rows,
                                  int N, int K, int32_t *acc) {
#pragma omp parallel for schedule(static) collapse(2)
    for (int i = 0; i < n_rows; ++i)
        for (int n = 0; n < N; ++n) {
            const int8_t *a = A + (int64_t)rows[i] * K;
            const int8_t *w = W + (int64_t)n * K;
            int32_t s = 0;
            for (int k = 0; k < K; ++k) s += (int32_t)a[k] * (int32_t)w[k];
            acc[(int64_t)i * N + n] = s;
        }
}

/* Ternary GEMM on the packed weights: unpack, then exact int32 GEMM.
 * src/kernels/bitvla/bitnet_kernels.h:108-145 (M=1), :165-247 (M>1). */
ORC_API int orc_ternary_gemm_i32(const int8_t *A, const uint8_t *Wp, int M, int N, int K, int32_t *acc) {
    int8_t *W = (int8_t *)malloc((size_t)N * K);
    if (!W) return -2;
    int rc = orc_unpack_ladder_int2(Wp, N, K, W);
    if (rc == 0) orc_gemm_i8_i32(A, W, M, N, K, acc);
    free(W);
    return rc;
}

/* out = bf16(float(acc) / s[m] * ws[n / (N / ws_num)]), IEEE division.
 * src/kernels/bitvla/bitnet_kernels.h:245,404-405 (the reference compiles this
 * with --use_fast_math, so its division may differ in the last bit). */
ORC_API void orc_ternary_epilogue(const int32_t *acc, const float *s, const float *ws, int ws_num, int M,
                                  int N, uint16_t *out) {
    const int group = N / ws_num;
    for (int m = 0; m < M; ++m)
        for (int n = 0; n < N; ++n) {
            const float v = ((float)acc[(int64_t)m * N + n]) / s[m] * ws[n / group];
            out[(int64_t)m * N + n] = f32_to_bf16_bits(v);
        }
}

/* ------------------------------------------------------------ dense ops -- */

/* y[t][o] = sum_i W[o][i] x[t][i] (+ b[o]).  src/layers/linear.h:24-27. */
ORC_API void orc_linear(const float *x, const float *W, const float *b, int T, int in, int out, float *y) {
    /* one weight row stays in cache for all T tokens; the dot product is a SIMD reduction (float32,
     * summation order differs from a left-to-right loop by rounding only) */
#pragma omp parallel for schedule(static)
    for (int o = 0; o < out; ++o) {
        const float *wr = W + (int64_t)o * in;
        for (int t = 0; t < T; ++t) {
            const float *xr = x + (int64_t)t * in;
            float acc = 0.0f;
#pragma omp simd reduction(+ : acc)
            for (int i = 0; i < in; ++i) acc += wr[i] * xr[i];
            y[(int64_t)t * out + o] = acc + (b ? b[o] : 0.0f);
        }
    }
}

/* y = x * rsqrt(mean(x^2) + eps) * w.  src/cuda/vla_cuda_bf16.cu:549-579,
 * src/kernels/bitvla/bitvla_lm_cuda.cu:37-75. */
ORC_API void orc_rmsnorm(const float *x, const float *w, int T, int H, float eps, float *y) {
    for (int t = 0; t < T; ++t) {
        const float *xr = x + (int64_t)t * H;
        float ss = 0.0f;
        for (int i = 0; i < H; ++i) ss += xr[i] * xr[i];
        const float r = 1.0f / sqrtf(ss / (float)H + eps);
        for (int i = 0; i < H; ++i) y[(int64_t)t * H + i] = xr[i] * r * (w ? w[i] : 1.0f);
    }
}

/* NeoX rotary embedding in place on x[t][head][hd]; pairs (i, i+hd/2),
 * theta_i = pos * base^(-2i/hd).  src/kernels/bitvla/bitvla_lm_cuda.cu:77-98,333-346;
 * the half-split pairing is the one tests/test_rope_conventions.cpp:41-50 pins. */
ORC_API void orc_rope_neox(float *x, const int32_t *pos, int T, int heads, int hd, float base) {
    const int half = hd / 2;
    for (int t = 0; t < T; ++t)
        for (int i = 0; i < half; ++i) {
            const float freq = powf(base, -2.0f * (float)i / (float)hd);
            const float ang = (float)pos[t] * freq;
            const float c = cosf(ang), s = sinf(ang);
            for (int h = 0; h < heads; ++h) {
                float *v = x + ((int64_t)t * heads + h) * hd;
                const float a = v[i], b = v[i + half];
                v[i] = a * c - b * s;
                v[i + half] = b * c + a * s;
            }
        }
}

/* cos/sin table [T][hd/2] the CUDA path is handed (same arithmetic as above). */
ORC_API void orc_rope_table(const int32_t *pos, int T, int hd, float base, float *cos_t, float *sin_t) {
    const int half = hd / 2;
    for (int t = 0; t < T; ++t)
        for (int i = 0; i < half; ++i) {
            const float freq = powf(base, -2.0f * (float)i / (float)hd);
            const float ang = (float)pos[t] * freq;
            cos_t[t * half + i] = cosf(ang);
            sin_t[t * half + i] = sinf(ang);
        }
}

/* Openpi-style time embedding, [sin ; cos] over log-spaced periods.
 * src/layers/embed.h:61-73. */
ORC_API void orc_time_emb(double t, int dim, double min_p, double max_p, float *out) {
    const int half = dim / 2;
    for (int i = 0; i < half; ++i) {
        const double frac = (half == 1) ? 0.0 : (double)i / (double)(half - 1);
        const double period = min_p * pow(max_p / min_p, frac);
        const double s = (2.0 * M_PI / period) * t;
        out[i] = (float)sin(s);
        out[half + i] = (float)cos(s);
    }
}

static inline float silu_f(float x) { return x / (1.0f + expf(-x)); }
/* tanh-GELU, constants as src/cuda/vla_cuda_bf16.cu:470-474 */
static inline float gelu_tanh_f(float x) {
    const float k0 = 0.79788456080286535587989211986876f, k1 = 0.044715f;
    return 0.5f * x * (1.0f + tanhf(k0 * x * (1.0f + k1 * x * x)));
}

/* Mask rules.  mode 0: every column visible (cross-attention / no suffix rule).
 * mode 1 (pi0, src/models/pi0.cpp:640-651): prefix visible; suffix row 0 sees only
 *   suffix column 0, rows >= 1 see all suffix columns.
 * mode 2 (SmolVLA, src/models/smolvla.cpp:1655-1664): prefix visible except
 *   [pad_start, pad_end); suffix causal. */
/* mode 0: everything visible; 1: pi0 suffix rule (src/models/pi0.cpp:640-651); 2: causal suffix
 * (src/models/smolvla.cpp:1655-1664); 3: SmolVLA prefill rule with P = 0 (smolvla.cpp:1637-1645): the last column
 * (state token) is visible to the last row only, padded columns to nobody. */
static inline int mask_visible(int mode, int P, int row, int col, int pad_start, int pad_end, int S, int Tkv) {
    if (mode == 3) {
        if (col >= pad_start && col < pad_end) return 0;
        return col < Tkv - 1 || row == S - 1;
    }
    if (col < P) return !(col >= pad_start && col < pad_end);
    const int sc = col - P;
    if (mode == 1) return row == 0 ? (sc == 0) : 1;
    if (mode == 2) return sc <= row;
    return 1;
}

/* O = softmax(Q K^T * scale + mask) V with GQA head sharing (q head h reads kv
 * head h / (n_q / n_kv)).  q: [S][n_q][hd]; K, V: [Tkv][n_kv][hd]; out: [S][n_q*hd].
 * src/layers/attn.h:38-46, src/models/pi0.cpp:204-223, smolvla.cpp:835-842;
 * head mapping src/kernels/bitvla/bitvla_lm_cuda.cu:181-190. */
ORC_API void orc_attention(const float *q, const float *K, const float *V, int S, int Tkv, int n_q, int n_kv,
                           int hd, int P, int mode, int pad_start, int pad_end, float *out) {
    const float scale = 1.0f / sqrtf((float)hd);
    const int g = n_q / n_kv;
#pragma omp parallel for schedule(static) collapse(2)
    for (int j = 0; j < S; ++j)
        for (int h = 0; h < n_q; ++h) {
            const int kvh = h / g;
            const float *qv = q + ((int64_t)j * n_q + h) * hd;
            float *sc = (float *)malloc(sizeof(float) * (size_t)Tkv);
            float mx = -INFINITY;
            for (int i = 0; i < Tkv; ++i) {
                if (!mask_visible(mode, P, j, i, pad_start, pad_end, S, Tkv)) {
                    sc[i] = -INFINITY;
                    continue;
                }
                const float *kv = K + ((int64_t)i * n_kv + kvh) * hd;
                float d = 0.0f;
                for (int e = 0; e < hd; ++e) d += qv[e] * kv[e];
                sc[i] = d * scale;
                if (sc[i] > mx) mx = sc[i];
            }
            float den = 0.0f;
            for (int i = 0; i < Tkv; ++i) {
                sc[i] = (sc[i] == -INFINITY) ? 0.0f : expf(sc[i] - mx);
                den += sc[i];
            }
            float *o = out + ((int64_t)j * n_q + h) * hd;
            for (int e = 0; e < hd; ++e) o[e] = 0.0f;
            for (int i = 0; i < Tkv; ++i) {
                if (sc[i] == 0.0f) continue;
                const float p = sc[i] / den;
                const float *vv = V + ((int64_t)i * n_kv + kvh) * hd;
                for (int e = 0; e < hd; ++e) o[e] += p * vv[e];
            }
            free(sc);
        }
}

static void round_bf16_inplace(float *x, int64_t n) {
    for (int64_t i = 0; i < n; ++i) x[i] = bf16_round(x[i]);
}

/* RMSNorm -> Q,K,V projections -> NeoX RoPE on q,k.  Wqkv: [(n_q+2 n_kv) hd][H]
 * (rows: q heads, then k heads, then v heads).  Outputs q [S][n_q][hd],
 * k, v [S][n_kv][hd].  src/models/pi0.cpp:170-201, smolvla.cpp:820-833. */
ORC_API void orc_qkv_rope(const float *x, const float *ln_w, const float *Wqkv, const int32_t *pos, int S,
                          int H, int n_q, int n_kv, int hd, float eps, float rope_base, int act_bf16,
                          float *q, float *k, float *v) {
    float *xn = (float *)malloc(sizeof(float) * (size_t)S * H);
    orc_rmsnorm(x, ln_w, S, H, eps, xn);
    if (act_bf16) round_bf16_inplace(xn, (int64_t)S * H);
    orc_linear(xn, Wqkv, NULL, S, H, n_q * hd, q);
    orc_linear(xn, Wqkv + (int64_t)n_q * hd * H, NULL, S, H, n_kv * hd, k);
    orc_linear(xn, Wqkv + (int64_t)(n_q + n_kv) * hd * H, NULL, S, H, n_kv * hd, v);
    orc_rope_neox(q, pos, S, n_q, hd, rope_base);
    orc_rope_neox(k, pos, S, n_kv, hd, rope_base);
    if (act_bf16) {
        round_bf16_inplace(q, (int64_t)S * n_q * hd);
        round_bf16_inplace(k, (int64_t)S * n_kv * hd);
        round_bf16_inplace(v, (int64_t)S * n_kv * hd);
    }
    free(xn);
}

/* ------------------------------------------------- the denoise loop itself -- */

typedef struct {
    int32_t model;      /* 0 = pi0 (src/models/pi0.cpp), 1 = SmolVLA (src/models/smolvla.cpp) */
    int32_t n_layers;
    int32_t H;          /* expert hidden */
    int32_t n_q, n_kv, hd;
    int32_t inter;      /* expert MLP width */
    int32_t P;          /* prefix length (KV rows cached per layer) */
    int32_t chunk;      /* action tokens (50) */
    int32_t A;          /* max_action_dim (32) */
    int32_t state_dim;  /* max_state_dim (32), pi0 only inside the loop */
    int32_t T;          /* Euler steps */
    int32_t pos_base;   /* RoPE position of suffix token 0 on self-attention layers */
    int32_t pad_start, pad_end; /* masked prefix columns (SmolVLA); equal => none */
    int32_t self_every; /* SmolVLA: layer l is self-attention iff l % self_every == 0; pi0: 1 */
    int32_t act_bf16;   /* round activations to bf16 where the CUDA path stores bf16 */
    float rms_eps, rope_base;
    double min_period, max_period;
} orc_denoise_cfg;

typedef struct {
    /* per layer, arrays of n_layers pointers */
    const float *const *ln_in;   /* [H] */
    const float *const *Wqkv;    /* self layers: [(n_q+2n_kv)hd][H]; SmolVLA cross layers: q rows [n_q hd][H]
                                    followed by Wk, Wv [n_kv hd][n_kv hd] acting on the flattened prefix K/V */
    const float *const *Wo;      /* [H][n_q hd] */
    const float *const *ln_post; /* [H] */
    const float *const *Wgate;   /* [inter][H] */
    const float *const *Wup;     /* [inter][H] */
    const float *const *Wdown;   /* [H][inter] */
    /* suffix embedding / head */
    const float *W_sp, *b_sp;    /* pi0: [H][state_dim] */
    const float *W_ain, *b_ain;  /* [H][A] */
    const float *W_at1, *b_at1;  /* [H][2H] */
    const float *W_at2, *b_at2;  /* [H][H] */
    const float *out_norm;       /* [H] */
    const float *W_aout, *b_aout;/* [A][H] */
} orc_denoise_weights;

/* One expert layer on the suffix (self-attention over prefix+suffix KV, or
 * SmolVLA cross-attention over re-projected prefix KV).
 * src/models/pi0.cpp:159-233, smolvla.cpp:815-888. */
static void expert_layer(const orc_denoise_cfg *c, const orc_denoise_weights *w, int l, float *h, int S,
                         const float *Kp, const float *Vp /* [P][n_kv][hd], cross: re-projected */,
                         int is_self) {
    const int H = c->H, nq = c->n_q, nkv = c->n_kv, hd = c->hd, P = c->P;
    const int qf = nq * hd, kvf = nkv * hd;
    float *q = (float *)malloc(sizeof(float) * (size_t)S * qf);
    float *att = (float *)malloc(sizeof(float) * (size_t)S * qf);
    int32_t *pos = (int32_t *)malloc(sizeof(int32_t) * (size_t)S);
    if (is_self) {
        const int Tkv = P + S;
        float *K = (float *)malloc(sizeof(float) * (size_t)Tkv * kvf);
        float *V = (float *)malloc(sizeof(float) * (size_t)Tkv * kvf);
        memcpy(K, Kp, sizeof(float) * (size_t)P * kvf);
        memcpy(V, Vp, sizeof(float) * (size_t)P * kvf);
        for (int j = 0; j < S; ++j) pos[j] = c->pos_base + j;
        orc_qkv_rope(h, w->ln_in[l], w->Wqkv[l], pos, S, H, nq, nkv, hd, c->rms_eps, c->rope_base,
                     c->act_bf16, q, K + (size_t)P * kvf, V + (size_t)P * kvf);
        orc_attention(q, K, V, S, Tkv, nq, nkv, hd, P, c->model == 0 ? 1 : 2, c->pad_start, c->pad_end, att);
        free(K);
        free(V);
    } else {
        /* q only, rebased positions 0..S-1, attention over the prefix columns */
        float *xn = (float *)malloc(sizeof(float) * (size_t)S * H);
        orc_rmsnorm(h, w->ln_in[l], S, H, c->rms_eps, xn);
        if (c->act_bf16) round_bf16_inplace(xn, (int64_t)S * H);
        orc_linear(xn, w->Wqkv[l], NULL, S, H, qf, q);
        for (int j = 0; j < S; ++j) pos[j] = j;
        orc_rope_neox(q, pos, S, nq, hd, c->rope_base);
        if (c->act_bf16) round_bf16_inplace(q, (int64_t)S * qf);
        orc_attention(q, Kp, Vp, S, P, nq, nkv, hd, P, 0, c->pad_start, c->pad_end, att);
        free(xn);
    }
    if (c->act_bf16) round_bf16_inplace(att, (int64_t)S * qf);
    /* h1 = h + Wo att */
    float *o = (float *)malloc(sizeof(float) * (size_t)S * H);
    orc_linear(att, w->Wo[l], NULL, S, qf, H, o);
    for (int64_t i = 0; i < (int64_t)S * H; ++i) h[i] += o[i];
    /* gated MLP */
    float *xm = (float *)malloc(sizeof(float) * (size_t)S * H);
    orc_rmsnorm(h, w->ln_post[l], S, H, c->rms_eps, xm);
    if (c->act_bf16) round_bf16_inplace(xm, (int64_t)S * H);
    const int I = c->inter;
    float *g = (float *)malloc(sizeof(float) * (size_t)S * I);
    float *u = (float *)malloc(sizeof(float) * (size_t)S * I);
    orc_linear(xm, w->Wgate[l], NULL, S, H, I, g);
    orc_linear(xm, w->Wup[l], NULL, S, H, I, u);
    for (int64_t i = 0; i < (int64_t)S * I; ++i)
        g[i] = (c->model == 0 ? gelu_tanh_f(g[i]) : silu_f(g[i])) * u[i];
    if (c->act_bf16) round_bf16_inplace(g, (int64_t)S * I);
    orc_linear(g, w->Wdown[l], NULL, S, I, H, o);
    for (int64_t i = 0; i < (int64_t)S * H; ++i) h[i] += o[i];
    free(q); free(att); free(pos); free(o); free(xm); free(g); free(u);
}

/* SmolVLA cross layers: K' = Wk Kp_flat, V' = Wv Vp_flat once per observation.
 * src/models/smolvla.cpp:853-860. */
ORC_API void orc_cross_kv(const float *Kp, const float *Vp, const float *Wk, const float *Wv, int P, int kvf,
                          float *Kx, float *Vx) {
    orc_linear(Kp, Wk, NULL, P, kvf, kvf, Kx);
    orc_linear(Vp, Wv, NULL, P, kvf, kvf, Vx);
}

/* Full flow-matching loop for one observation: x0 [chunk][A] -> x_T [chunk][A].
 * Kp/Vp: n_layers pointers to [P][n_kv][hd] (K already rotated with prefix
 * positions).  state: [state_dim] (normalised), used by pi0 only.
 * src/models/pi0.cpp:568-588, smolvla.cpp:1393-1418. */
ORC_API int orc_denoise_loop(const orc_denoise_cfg *c, const orc_denoise_weights *w, const float *const *Kp,
                             const float *const *Vp, const float *state, const float *x0, float *x_out) {
    const int H = c->H, A = c->A, chunk = c->chunk;
    const int S = chunk + (c->model == 0 ? 1 : 0);
    const int kvf = c->n_kv * c->hd, qf = c->n_q * c->hd;
    const float dt = -1.0f / (float)c->T;
    float *x = (float *)malloc(sizeof(float) * (size_t)chunk * A);
    memcpy(x, x0, sizeof(float) * (size_t)chunk * A);
    float *h = (float *)malloc(sizeof(float) * (size_t)S * H);
    float *a = (float *)malloc(sizeof(float) * (size_t)chunk * 2 * H);
    float *m1 = (float *)malloc(sizeof(float) * (size_t)chunk * H);
    float *temb = (float *)malloc(sizeof(float) * (size_t)H);
    float *hn = (float *)malloc(sizeof(float) * (size_t)S * H);
    float *v = (float *)malloc(sizeof(float) * (size_t)chunk * A);
    float *tmp = (float *)malloc(sizeof(float) * (size_t)chunk * H);
    /* cross-attention K/V, once per observation */
    float **Kx = (float **)calloc((size_t)c->n_layers, sizeof(float *));
    float **Vx = (float **)calloc((size_t)c->n_layers, sizeof(float *));
    for (int l = 0; l < c->n_layers; ++l) {
        const int is_self = (c->model == 0) || (l % c->self_every == 0);
        if (is_self) continue;
        Kx[l] = (float *)malloc(sizeof(float) * (size_t)c->P * kvf);
        Vx[l] = (float *)malloc(sizeof(float) * (size_t)c->P * kvf);
        const float *Wk = w->Wqkv[l] + (size_t)qf * H;
        const float *Wv = Wk + (size_t)kvf * kvf;
        orc_cross_kv(Kp[l], Vp[l], Wk, Wv, c->P, kvf, Kx[l], Vx[l]);
        if (c->act_bf16) {
            round_bf16_inplace(Kx[l], (int64_t)c->P * kvf);
            round_bf16_inplace(Vx[l], (int64_t)c->P * kvf);
        }
    }
    for (int step = 0; step < c->T; ++step) {
        const double tk = 1.0 + (double)step * (double)dt;
        /* the reference evaluates the timestep in float for pi0, double for SmolVLA */
        orc_time_emb(c->model == 0 ? (double)(1.0f + (float)step * dt) : tk, H, c->min_period,
                     c->max_period, temb);
        /* a = [W_ain x + b ; time] */
        orc_linear(x, w->W_ain, w->b_ain, chunk, A, H, tmp);
        for (int t = 0; t < chunk; ++t) {
            memcpy(a + (size_t)t * 2 * H, tmp + (size_t)t * H, sizeof(float) * (size_t)H);
            memcpy(a + (size_t)t * 2 * H + H, temb, sizeof(float) * (size_t)H);
        }
        orc_linear(a, w->W_at1, w->b_at1, chunk, 2 * H, H, m1);
        for (int64_t i = 0; i < (int64_t)chunk * H; ++i) m1[i] = silu_f(m1[i]);
        float *h_act = h + (c->model == 0 ? H : 0);
        orc_linear(m1, w->W_at2, w->b_at2, chunk, H, H, h_act);
        if (c->model == 0) orc_linear(state, w->W_sp, w->b_sp, 1, c->state_dim, H, h);
        for (int l = 0; l < c->n_layers; ++l) {
            const int is_self = (c->model == 0) || (l % c->self_every == 0);
            expert_layer(c, w, l, h, S, is_self ? Kp[l] : Kx[l], is_self ? Vp[l] : Vx[l], is_self);
        }
        orc_rmsnorm(h, w->out_norm, S, H, c->rms_eps, hn);
        orc_linear(hn + (c->model == 0 ? H : 0), w->W_aout, w->b_aout, chunk, H, A, v);
        for (int64_t i = 0; i < (int64_t)chunk * A; ++i) x[i] += dt * v[i];
    }
    memcpy(x_out, x, sizeof(float) * (size_t)chunk * A);
    for (int l = 0; l < c->n_layers; ++l) { free(Kx[l]); free(Vx[l]); }
    free(Kx); free(Vx);
    free(x); free(h); free(a); free(m1); free(temb); free(hn); free(v); free(tmp);
    return 0;
}

/* One expert layer exposed for per-layer parity tests (h updated in place). */
ORC_API void orc_expert_layer(const orc_denoise_cfg *c, const orc_denoise_weights *w, int l, float *h, int S,
                              const float *Kp, const float *Vp, int is_self) {
    expert_layer(c, w, l, h, S, Kp, Vp, is_self);
}
