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

/* Self-test of the kernels' failure path: one small kernel whose warps wait, with a budget of
 * `budget_cycles` GPU clock cycles (at most 1e8, i.e. well under a second), on a hardware barrier that
 * nothing ever signals.  The wait gives up, the kernel returns normally, *gave_up is 1 and the device
 * status word reads 104 until it is reset; the context stays usable.  Synchronises `stream`.
 * No counterpart in the reference. */
VLAB200_API int32_t vlab200_selftest_bounded_wait(int64_t budget_cycles, int32_t *gave_up, void *stream);

/* ------------------------------------------------- prefix-KV store, QKV+RoPE, attention */

/* bf16 K/V pages, written once per observation for the prefix and appended per denoise
 * step for the suffix.  Layout of k_pages / v_pages (caller-allocated device memory,
 * zero-initialised, 16-byte aligned, vlab200_kv_store_bytes() each):
 *     [n_layers][n_obs][n_kv][cap][head_dim]      (one contiguous page per layer, observation
 *                                                  and kv head; rows are tokens)
 * Rows [0, prefix_len) hold the prefix (K already rotated with prefix positions), rows
 * [prefix_len, prefix_len + S) the current step's suffix.  The reference keeps the same data
 * as F32 graph tensors [hd, n_kv, P] per layer and concatenates the suffix onto a copy of it
 * every layer-step (src/models/pi0.cpp:191-201, src/models/smolvla.cpp:793-794,832-833). */
typedef struct {
    void *k_pages;
    void *v_pages;
    int32_t n_layers;
    int32_t n_obs;
    int32_t n_kv;       /* kv heads */
    int32_t head_dim;   /* 64, 128 or 256 */
    int32_t cap;        /* token rows per page, >= prefix_len + suffix length */
    int32_t prefix_len; /* P */
} vlab200_kv_store;

/* Bytes of ONE of the two page arrays; -1 on a non-positive dimension. */
VLAB200_API int64_t vlab200_kv_store_bytes(int32_t n_layers, int32_t n_obs, int32_t n_kv, int32_t head_dim,
                                           int32_t cap);

/* Writes the prefix rows of `layer` for observations [obs0, obs0 + n_obs) from the prefill's
 * K, V: float32 [n_obs][prefix_len][n_kv][head_dim] (ggml [hd, n_kv, P] per observation), K
 * already rotated.  Replaces the k_out / v_out hand-off of build_gemma_layer / build_vlm_layer
 * (src/models/pi0.cpp:191-194, src/models/smolvla.cpp:793-794). */
VLAB200_API int32_t vlab200_kv_store_write(const vlab200_kv_store *st, int32_t layer, int32_t obs0, int32_t n_obs,
                                           const float *K, const float *V, void *stream);

/* cos/sin tables [S][head_dim/2] (float32) for positions pos0 .. pos0+S-1 of a plain NeoX
 * RoPE with frequency base `base` (ggml_rope_ext call of src/models/smolvla.cpp:759-766). */
VLAB200_API int32_t vlab200_rope_table(float *cos_out, float *sin_out, int32_t pos0, int32_t S, int32_t head_dim,
                                       float base, void *stream);

/* out[n][k] = bf16(w[n][k] * ln_w[k]) for a bf16 [rows][H] weight: folds an RMSNorm weight
 * (Gemma-style norms already carry their +1, src/gguf_reader.h:169) into the projection that
 * consumes the normalised activations.  Run once at load time; `out` may alias `w`. */
VLAB200_API int32_t vlab200_fold_norm_weight(const void *w_bf16, const float *ln_w, void *out_bf16, int64_t rows,
                                             int32_t H, void *stream);

/* Fused RMSNorm -> Q/K/V projection -> NeoX RoPE -> KV append for the suffix tokens of ALL
 * observations of the store (M = n_obs * S rows):
 *   xn = x * rsqrt(mean(x^2) + eps) * ln_w;  [q | k | v] = Wqkv xn;  q, k rotated;
 *   q_out bf16 [n_obs][n_q][S][head_dim];  k, v -> page rows prefix_len + tok.
 * x: [n_obs*S][H], bf16 or (x_is_f32) float32.  Wqkv: bf16 [(n_q + 2 n_kv) head_dim][H], rows
 * ordered q heads, k heads, v heads.  project_kv == 0 projects q only (SmolVLA cross-attention
 * layers, src/models/smolvla.cpp:870-873; Wqkv then holds the q rows only).  H % 8 == 0.
 * ln_w == NULL means Wqkv was already multiplied by ln_w (vlab200_fold_norm_weight); with bf16 x
 * this selects the fastest kernel (both operands by TMA, persistent CTAs).  eps < 0: x is taken as already
 * normalised (no RMS factor; the pi0.5 expert normalises adaptively before the projection, src/models/pi05.cpp:237-241).
 * Replaces the rms_norm/mul, three mul_mat, two rope and two concat nodes of
 * src/models/pi0.cpp:170-201 and src/models/smolvla.cpp:820-833. */
VLAB200_API int32_t vlab200_qkv_rope_append(const vlab200_kv_store *st, int32_t layer, const void *x,
                                            int32_t x_is_f32, const float *ln_w, const void *wqkv_bf16,
                                            const float *rope_cos, const float *rope_sin, float eps, int32_t S,
                                            int32_t H, int32_t n_q, int32_t project_kv, void *q_out,
                                            void *stream);

/* out[obs][tok][h*hd ..] = softmax(q K^T / sqrt(hd) + mask) V over page rows [0, kv_len) of
 * `layer`, query head h reading kv head h / (n_q / n_kv).  q: bf16 [n_obs][n_q][S][hd];
 * out: bf16 [n_obs][S][n_q*hd].  mask_mode: 0 = all rows < kv_len visible; 1 = pi0 rule
 * (suffix row 0 sees only suffix column 0, other rows every column; src/models/pi0.cpp:640-651);
 * 2 = causal over the suffix (src/models/smolvla.cpp:1655-1664); 3 = the last column is visible to the last
 * query token only (SmolVLA prefill: the state token sees the prefix, nothing else sees the state token,
 * src/models/smolvla.cpp:1637-1645).  pad_ranges (optional, int32
 * [n_obs][2]) masks prefix columns [lo, hi) per observation (padded language slots).
 * head_dim 64 with kv_len <= 256 and (n_q / n_kv) * S <= 256 runs a kernel that holds the whole
 * key range on chip; head_dim 64 / 128 / 256 of any length stream K and V in 64-key blocks with
 * an online softmax.
 * Replaces ggml_flash_attn_ext / mul_mat+soft_max_ext+mul_mat at src/models/pi0.cpp:204-223,
 * src/models/smolvla.cpp:835-842,874-881 (src/layers/attn.h:38-57). */
VLAB200_API int32_t vlab200_attention(const vlab200_kv_store *st, int32_t layer, const void *q, void *out,
                                      int32_t S, int32_t n_q, int32_t kv_len, int32_t mask_mode,
                                      const int32_t *pad_ranges, void *stream);

/* The isolated denoise-attention op: for step in [0, steps), layer in [0, n_layers):
 * vlab200_qkv_rope_append(layer) then vlab200_attention(layer) over every observation of
 * the store, on one stream.  It is the layer x step loop the reference unrolls into its graph
 * (src/models/smolvla.cpp:1405-1415, src/models/pi0.cpp:572-577) restricted to the QKV and
 * attention nodes, with the hidden states given as inputs. */
typedef struct {
    int32_t n_layers, steps, S, H, n_q, mask_mode, x_is_f32;
    float eps;
    const void *x;          /* [steps][n_layers][n_obs*S][H] hidden states, bf16 or float32 */
    const float *ln_w;      /* [n_layers][H], or NULL when wqkv already has it folded in */
    const void *wqkv;       /* bf16 [n_layers][(n_q + 2 n_kv) hd][H] */
    const float *rope_cos;  /* [S][hd/2] */
    const float *rope_sin;
    void *q_scratch;        /* bf16 [n_obs][n_q][S][hd] */
    void *out;              /* bf16 [n_layers][n_obs][S][n_q*hd]: the last step's attention output */
    const int32_t *pad_ranges; /* optional, see vlab200_attention */
} vlab200_denoise_attn_args;

VLAB200_API int32_t vlab200_denoise_attn_loop(const vlab200_kv_store *st, const vlab200_denoise_attn_args *a,
                                              void *stream);

/* vlab200_denoise_attn_loop for callers that have no way to obtain device scratch memory: a
 * plugin running inside a host that owns the allocator and hands out only input and output
 * buffers, or code running while cudaMalloc is off limits (inside a latency-critical control
 * loop, or when the device is fully committed to other tenants).  It has no counterpart in the
 * reference.  The query buffer (a->q_scratch, which is ignored here) comes from a 16 MiB array
 * built into the library image, so n_obs * n_q * S * head_dim * 2 bytes must not exceed 16 MiB
 * (VLAB200_ERR_UNSUPPORTED with an explanatory vlab200_last_error() otherwise).  The call
 * allocates nothing on host or device.  The first call on each device looks up the array's
 * device address; make that first call outside any stream capture.  All calls on a device share
 * the one array and it keeps whatever the previous call left in it (every row that is read is
 * written first, so nothing needs clearing); two calls whose kernels overlap on the GPU (different
 * streams, or threads) race on it. */
VLAB200_API int32_t vlab200_denoise_attn_loop_static(const vlab200_kv_store *st,
                                                     const vlab200_denoise_attn_args *a, void *stream);

/* Same loop with the hidden states and the result in (pinned) HOST memory: a->x is a host
 * pointer; each step's hidden states [n_layers][n_obs*S][H] are copied into the device
 * staging buffer x_stage (2 x that size, double-buffered on an internal copy stream) while
 * the previous step computes; after the last step a->out (device) is copied to out_host.
 * Creates one stream and four events per calling thread on first use. */
VLAB200_API int32_t vlab200_denoise_attn_loop_host(const vlab200_kv_store *st, const vlab200_denoise_attn_args *a,
                                                   void *x_stage, void *out_host, void *stream);

/* ------------------------------------------------------------- whole denoise loop (engine) */

/* Shape of a flow-matching policy's action expert (fields follow vla_config of include/vla.h:59-96
 * in the reference: expert_h, n_q_heads, n_kv_heads, head_dim, expert_inter, n_suffix / chunk,
 * max_action_dim, max_state_dim, num_steps, self_attn_every_n, rms_eps, rope_freq_base, periods). */
typedef struct {
    int32_t model;       /* 0 = pi0 (state token in the suffix, tanh-GELU MLP; src/models/pi0.cpp),
                            1 = SmolVLA (SiLU MLP, alternating self / cross layers; src/models/smolvla.cpp),
                            2 = pi0.5 (adaptive RMSNorm conditioned on the time step, gated residuals, no state token,
                                no mask among the action tokens; src/models/pi05.cpp:208-292,604-631) */
    int32_t n_layers, H, n_q, n_kv, head_dim, inter, chunk, action_dim, state_dim, steps;
    int32_t self_every;  /* SmolVLA: layer l self-attends iff l % self_every == 0; <= 1: every layer */
    float rms_eps, rope_base;
    double min_period, max_period;
    int32_t cond_dim;    /* pi0.5: width of the time-conditioning vector (pi05.adarms_cond_dim); 0 = H */
} vlab200_policy_config;

/* Device pointers to the expert's weights, in the reference's tensor shapes (GGUF names of
 * src/modules/gemma_expert.h:46-62 / src/models/smolvla.cpp:648-756): matrices bf16 [out][in],
 * vectors float32.  Per-layer entries are HOST arrays of n_layers device pointers.
 * SmolVLA cross layers: wk, wv are [n_kv*hd][n_kv*hd].  The engine keeps its own prepared copies
 * (norm weights folded in, q/k/v concatenated, gate/up interleaved); the caller's buffers may be
 * released after vlab200_engine_create returns. */
typedef struct {
    const void *const *wq, *const *wk, *const *wv, *const *wo, *const *wgate, *const *wup, *const *wdown;
    const float *const *ln_in, *const *ln_post;
    const void *w_sp;   const float *b_sp;    /* pi0: [H][state_dim] */
    const void *w_ain;  const float *b_ain;   /* [H][action_dim] */
    const void *w_at1;  const float *b_at1;   /* [H][2H] */
    const void *w_at2;  const float *b_at2;   /* [H][H] */
    const float *out_norm;                    /* [H] (Gemma norms with their +1 applied) */
    const void *w_aout; const float *b_aout;  /* [action_dim][H] */
    /* pi0.5 only (ln_in, ln_post, out_norm, w_sp, w_at1, w_at2 are not read then); all float32, as the reference keeps
     * them: per layer the adaptive-norm dense maps [3H][cond_dim] + [3H] (rows scale | shift | gate; GGUF
     * "aex.blk.N.attn_norm.{weight,bias}" / "ffn_norm"), the final one ("aex.output_norm"), and the time MLP
     * [cond_dim][H], [cond_dim][cond_dim] ("time_mlp_in" / "time_mlp_out") */
    const float *const *ada_in_w, *const *ada_in_b, *const *ada_post_w, *const *ada_post_b;
    const float *ada_final_w, *ada_final_b;
    const float *w_tin, *b_tin, *w_tout, *b_tout;
} vlab200_policy_weights;

typedef struct vlab200_engine vlab200_engine;

/* Allocates (cudaMalloc) the prepared weights, the KV pages for max_obs observations with
 * prefix_len prefix rows, and the activation workspace.  NULL on failure (vlab200_last_error). */
VLAB200_API vlab200_engine *vlab200_engine_create(const vlab200_policy_config *cfg,
                                                  const vlab200_policy_weights *w, int32_t max_obs,
                                                  int32_t prefix_len);
VLAB200_API void vlab200_engine_free(vlab200_engine *e);

/* Prefix K/V of `layer` for observations [obs0, obs0+n_obs): float32 [n_obs][prefix_len][n_kv][hd],
 * K rotated (what build_gemma_layer / build_vlm_layer hand over, src/models/pi0.cpp:191-194,
 * src/models/smolvla.cpp:793-794).  Self-attention layers store it as bf16 pages; SmolVLA
 * cross-attention layers store Wk K / Wv V instead (expert_cross_kv, smolvla.cpp:853-860). */
VLAB200_API int32_t vlab200_engine_set_prefix(vlab200_engine *e, int32_t layer, int32_t obs0, int32_t n_obs,
                                              const float *K, const float *V, void *stream);

/* The Euler loop for n_obs observations: x0, x_out float32 [n_obs][chunk][action_dim] (device),
 * state float32 [n_obs][state_dim] (pi0; normalised), pos_base = RoPE position of suffix token 0
 * on self-attention layers (< 0: prefix_len), pad_ranges optional [n_obs][2] masked prefix columns.
 * Replaces the unrolled suffix sub-graph of src/models/pi0.cpp:568-588 / smolvla.cpp:1393-1418.
 * A call with ONE observation runs the whole loop as one persistent cooperative kernel (the reference's
 * answer to per-operator cost is one cached graph per predict, src/scratch_ctx.h:34-141); its first use builds a padded copy
 * of the expert's weights on the engine's device.  Environment VLAB200_CHUNK_LOOP=0 keeps a launch per operator.  The two
 * paths round activations to bf16 at different points: results agree to ~3e-3 rel-L2, each is reproducible bit for bit. */
VLAB200_API int32_t vlab200_engine_denoise(vlab200_engine *e, int32_t n_obs, const float *state, const float *x0,
                                           float *x_out, int32_t pos_base, const int32_t *pad_ranges,
                                           void *stream);

/* Same with state, x0, x_out and the optional pad_ranges ([n_obs][2]) in (pinned) host memory: the copies
 * are enqueued on `stream`. */
VLAB200_API int32_t vlab200_engine_denoise_host(vlab200_engine *e, int32_t n_obs, const float *state_host,
                                                const float *x0_host, float *x_out_host, int32_t pos_base,
                                                const int32_t *pad_ranges_host, void *stream);

/* Reads the prefix rows of `layer` back as float32 [n_obs][prefix_len][n_kv][hd] (the layout
 * vlab200_engine_set_prefix takes; cross-attention layers return the projected K' / V' they store). */
VLAB200_API int32_t vlab200_engine_get_prefix(vlab200_engine *e, int32_t layer, int32_t obs0, int32_t n_obs,
                                              float *K, float *V, void *stream);

/* Rows of the prefix in use for the following set_prefix / prefill / denoise calls: 0 < prefix_len <= the
 * prefix_len the engine was created with (which sized the pages).  pi0 requests differ in their number of
 * language tokens, so the prefix length changes from call to call (src/models/pi0.cpp:527-528). */
VLAB200_API int32_t vlab200_engine_set_prefix_len(vlab200_engine *e, int32_t prefix_len);

/* ---- prefix producer: the VLM layers that fill the K/V pages -----------------------------------------
 * Runs the backbone's transformer layers over the prefix embeddings of n_obs observations and writes every
 * layer's rotated K and its V as bf16 rows [0, P) of the engine's pages for observations [obs0, obs0+n_obs)
 * -- no float32 hand-off, no second copy.  SmolVLA cross-attention layers receive Wk K / Wv V
 * (expert_cross_kv) in place.  The last layer stops after its K/V (its attention and MLP feed nothing).
 * Layer = RMSNorm -> q,k,v -> NeoX RoPE -> masked GQA attention -> Wo + residual -> RMSNorm ->
 * act(gate) * up -> Wdown + residual, act 1 = SiLU (SmolVLA, src/models/smolvla.cpp:778-813), 2 = tanh-GELU
 * (Gemma, src/models/pi0.cpp:159-233).  Weights as for vlab200_engine_create: matrices bf16 [out][in], norm
 * vectors float32 (Gemma norms with their +1), host arrays of n_layers device pointers; prepared copies are
 * kept.  x_emb: float32 [n_obs][P][hidden] (device), already scaled as the model expects
 * (smolvla.cpp:1362-1369, pi0.cpp:553-555).  pos_host: int32 [P] RoPE positions (HOST; NULL = 0..P-1).
 * mask_mode 0 = every prefix token sees every other (pi0), 3 = the last token (state) is seen only by itself
 * (smolvla.cpp:1637-1645); pad_ranges as in vlab200_attention.  P must equal the engine's prefix length in
 * use.  Replaces the prefill loops of smolvla.cpp:1374-1391 and pi0.cpp:557-566. */
typedef struct {
    int32_t n_layers, hidden, n_q, n_kv, head_dim, inter, act;
    float rms_eps, rope_base;
} vlab200_prefill_config;
typedef struct {
    const void *const *wq, *const *wk, *const *wv, *const *wo, *const *wgate, *const *wup, *const *wdown;
    const float *const *ln_in, *const *ln_post;
} vlab200_prefill_weights;
typedef struct vlab200_prefill vlab200_prefill;
VLAB200_API vlab200_prefill *vlab200_prefill_create(const vlab200_prefill_config *cfg,
                                                    const vlab200_prefill_weights *w, int32_t max_obs,
                                                    int32_t max_prefix);
VLAB200_API void vlab200_prefill_free(vlab200_prefill *p);
VLAB200_API int32_t vlab200_prefill_run(vlab200_prefill *p, vlab200_engine *e, int32_t obs0, int32_t n_obs,
                                        const float *x_emb, int32_t P, const int32_t *pos_host, int32_t mask_mode,
                                        const int32_t *pad_ranges, void *stream);

/* ---- vision tower: camera views -> image-token embeddings of the prefix ------------------------------
 * SigLIP encoder + connector of the reference's towers (src/models/smolvla.cpp:394-426 block, :1511-1563
 * patch embedding / layers / post-LayerNorm / pixel shuffle / connector; src/models/pi0.cpp:130-155,479-517 the
 * same block with a biased linear projector and a 1/sqrt(out) scale; preprocessing and pixel-shuffle order of
 * src/modules/preprocess.h:37-75).  Block = LayerNorm -> q,k,v (+bias) -> unmasked attention -> Wo (+bias) +
 * residual -> LayerNorm -> fc1 (+bias) -> tanh-GELU -> fc2 (+bias) + residual.  All weights are device pointers:
 * matrices bf16 [out][in] (patch_w = the conv kernel [hidden][3][patch][patch] flattened), vectors float32;
 * per-layer entries are host arrays of n_layers device pointers; prepared copies are kept.
 * shuffle: pixel-shuffle factor of the connector (1 = none; the connector then is [out_dim][hidden]); with
 * shuffle = s it is [out_dim][hidden * s * s] in the channel-innermost order of pixel_shuffle_hf.
 * connector_b optional.  out_scale: factor on the connector's output (pi0: 1 / sqrt(out_dim); 0 or 1 = none).
 * head_dim = hidden / n_heads; 64 / 128 / 256 run as they are, any other even value <= 256 is zero-padded to the
 * next of them in the prepared weights.
 * vlab200_vision_run: pixels = DEVICE buffer [n_views][image][image][3], uint8 (0..255) or float32 (0..1) in
 * H, W, C order (vla_image's layout); x -> x / 255 (uint8 only) -> 2 x - 1.  img_emb: float32 device
 * [n_views * tokens_per_view][out_dim], the tensor vla_inputs.precomputed_img_emb would carry. */
typedef struct {
    int32_t image, patch, hidden, n_layers, n_heads, inter, shuffle, out_dim;
    float ln_eps, out_scale;
} vlab200_vision_config;
typedef struct {
    const void *patch_w;
    const float *patch_b, *pos; /* [hidden], [n_patches][hidden] */
    const float *const *ln1_w, *const *ln1_b, *const *ln2_w, *const *ln2_b;
    const void *const *wq, *const *wk, *const *wv, *const *wo, *const *fc1, *const *fc2;
    const float *const *bq, *const *bk, *const *bv, *const *bo, *const *b1, *const *b2;
    const float *post_w, *post_b;
    const void *connector;
    const float *connector_b;
} vlab200_vision_weights;
typedef struct vlab200_vision vlab200_vision;
VLAB200_API vlab200_vision *vlab200_vision_create(const vlab200_vision_config *cfg, const vlab200_vision_weights *w,
                                                  int32_t max_views);
VLAB200_API void vlab200_vision_free(vlab200_vision *v);
VLAB200_API int32_t vlab200_vision_tokens_per_view(const vlab200_vision *v);
VLAB200_API int32_t vlab200_vision_run(vlab200_vision *v, const void *pixels, int32_t pixels_f32, int32_t n_views,
                                       float *img_emb, void *stream);

/* Several GPUs in one process.  vlab200_shard_range: the contiguous block [start, start + count) of `rank` when
 * n_items independent observations are cut over n_ranks (the first n_items % n_ranks ranks get one more).
 * vlab200_engines_denoise_host: n_obs observations in (pinned) host memory through n_engines engines, each
 * created with its own device current (a weight replica and K/V pages per GPU, prefix K/V already set for the
 * engine's block, observation o of the block in slot o - start); one host thread and one stream per engine,
 * blocks of at most max_obs observations at a time, no exchange between GPUs; returns when every block is back in
 * x_out_host.  The reference runs one observation per predict on one device (src/model.h:204-225). */
VLAB200_API int32_t vlab200_shard_range(int64_t n_items, int32_t n_ranks, int32_t rank, int64_t *start, int64_t *count);
VLAB200_API int32_t vlab200_engines_denoise_host(vlab200_engine *const *engines, int32_t n_engines, int64_t n_obs,
                                                 const float *state_host, const float *x0_host, float *x_out_host,
                                                 int32_t pos_base, const int32_t *pad_ranges_host);

/* Measurement hook: launches ONE stage of expert layer `layer` `reps` times on the engine's own buffers, as
 * vlab200_engine_denoise would (0 = fused RMSNorm+QKV+RoPE+append, 1 = attention, 2 = O-projection + residual,
 * 3 = fused RMSNorm + gate/up + activation, 4 = down projection + residual), so that a caller can bracket one
 * kernel with CUDA events.  Call vlab200_engine_denoise once before (it fills the RoPE tables and activations);
 * the residual stream is left modified.  No counterpart in the reference. */
VLAB200_API int32_t vlab200_engine_run_stage(vlab200_engine *e, int32_t layer, int32_t stage, int32_t n_obs,
                                             int32_t reps, void *stream);

/* Tiling of the bf16 GEMMs (the fused QKV projection, and inside the engine the O-projection, MLP,
 * embedding MLPs and action head):
 * 0 = chosen per call from the problem size (default), 1 = one CTA per 128 x 256 tile,
 * 2 = one CTA per 128 x 128 tile (QKV: same as 1), 3 = CTA pairs (tcgen05 cta_group::2) on 256 x 256 tiles,
 * 4 = one CTA per 128 x 64 tile (QKV: same as 1).
 * All tilings give the same results bit for bit; the knob exists for tests and measurements.
 * Process-wide, not thread-safe against concurrent engine calls.  No counterpart in the reference. */
VLAB200_API int32_t vlab200_set_gemm_tiling(int32_t tiling);

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
 * int8 MMA, on CTA pairs when N >= 256), 1 = force GEMV, 2 = force the one-CTA-per-tile
 * tensor-core kernel, 3 = force the CTA-pair kernel (with ws_num > 1, 2 and 3 need (N / ws_num) % 32 == 0).
 * Replaces bitlinear_int8xint2 / bitlinear_int8xint2_m
 * (src/kernels/bitvla/bitnet_kernels.cu:31-116, kernels bitnet_kernels.h:108-409). */
VLAB200_API int32_t vlab200_ternary_linear(const int8_t *A, const uint8_t *W_ladder, void *out_bf16,
                                           int32_t *acc_out, const float *s, const float *ws, int32_t ws_num,
                                           int32_t M, int32_t N, int32_t K, int32_t path, void *stream);

/* Load-time ternarisation of a float weight matrix and packing into the ladder layout, on the device:
 *   absmean = max(mean |W|, 1e-5);  w = clamp(round_half_even(W / absmean), -1, 1);  *scale_out = absmean;
 *   packed_out = N*K/4 bytes in the layout vlab200_ternary_linear consumes.
 * W: float32 [N][K] (device, 16-byte aligned), N % 16 == 0, K % 128 == 0; scratch: one double (device).
 * A fused projection (gate|up, q|k|v) is packed one sub-matrix at a time: the pack is a sequence of
 * independent 16-row runs of 4K bytes, so sub-matrix i starts at packed_out + rows_before * K / 4 and gets its
 * own scale.  Replaces recover_ternary_and_scale + pack_ladder_int2 (src/models/bitvla.cpp:430-483; Python
 * form scripts/convert_bitvla_to_gguf.py:95-152), which run on the host at load time. */
VLAB200_API int32_t vlab200_ternarize_pack(const float *W, int64_t N, int64_t K, uint8_t *packed_out,
                                           float *scale_out, double *scratch, void *stream);

/* ---- BitVLA language-model block: the callers either side of the ternary linear ----------
 * One BitNet transformer layer = RMSNorm -> act-quant -> ternary q/k/v -> NeoX RoPE ->
 * bidirectional GQA attention -> sub-norm -> act-quant -> ternary o -> residual -> RMSNorm ->
 * act-quant -> ternary gate_up -> relu(gate)^2 * up -> sub-norm -> act-quant -> ternary down ->
 * residual, every intermediate rounded to bf16 where the reference stores bf16.
 * Same life cycle and argument meaning as bitvla_lm_cuda_init / _set_layer / _set_output_norm /
 * _forward / _free (src/kernels/bitvla/bitvla_lm_cuda.cu:314-393,668-725, layer body
 * bitvla_lm_cuda.cu:395-525); the layer struct has the field order of bitvla_lm_layer_cuda
 * (src/kernels/bitvla/bitvla_lm_cuda.h:211-229) so a pointer to one can be passed as is.
 * Differences: `max_batch` / `n_seq` run several sequences of equal length in one call (rows
 * [i*seq, (i+1)*seq) of d_in / d_out belong to sequence i, attention never crosses sequences);
 * set_layer copies the q, k, v packs into one fused matrix (device memory is allocated in init
 * and set_layer only, never in forward); attention keeps scores in float on chip instead of
 * rounding them to bf16 in HBM.  gate_up_ws holds two scales (gate rows, up rows), the other
 * *_ws one.  Needs hidden, n_q*head_dim, ffn multiples of 128 and head_dim in {64,128,256}. */
typedef struct {
    const void *attn_norm_w;     /* bf16 [hidden] */
    const void *attn_sub_norm_w; /* bf16 [n_q*head_dim] */
    const void *ffn_norm_w;      /* bf16 [hidden] */
    const void *ffn_sub_norm_w;  /* bf16 [ffn] */
    const void *q_packed;        /* ladder pack [n_q*head_dim][hidden] */
    const float *q_ws;
    const void *k_packed;        /* [n_kv*head_dim][hidden] */
    const float *k_ws;
    const void *v_packed;
    const float *v_ws;
    const void *o_packed;        /* [hidden][n_q*head_dim] */
    const float *o_ws;
    const void *gate_up_packed;  /* [2*ffn][hidden], gate rows then up rows */
    const float *gate_up_ws;     /* 2 floats */
    const void *down_packed;     /* [hidden][ffn] */
    const float *down_ws;
} vlab200_bitvla_lm_layer;

typedef struct vlab200_bitvla_lm vlab200_bitvla_lm;

/* The fused element-wise stage between two ternary linears, one pass over each token row:
 *   mode 0: x = x_bf16[m][k]
 *   mode 1: x = bf16(x_bf16[m][k] + add_bf16[m][k]), also written back to x_bf16 (residual add)
 *   mode 2: x = bf16(relu(g)^2 * u), g = x_bf16[m][k], u = x_bf16[m][K + k] (rows of 2K: gate | up)
 *   y = bf16(x * rsqrt(mean_k x^2 + eps) * w_bf16[k])
 *   y_bf16 != NULL: y is stored (bf16 [M][K]) and nothing is quantised; otherwise
 *   scales[m] = 127 / max(max_k |y|, 1e-5), q[m][k] = clamp(rne(y * scales[m]), -128, 127).
 * Replaces bitvla_add_bf16 / gate_up_fused_sqrelu_mul_bf16 + bitvla_rmsnorm_bf16 + bitvla_act_quant_cuda
 * (src/kernels/bitvla/bitvla_lm_cuda.cu:37-75,527-549; src/kernels/bitvla/bitnet_kernels.h:465-521).
 * K even, K <= 51200. */
VLAB200_API int32_t vlab200_bitvla_norm_quant(void *x_bf16, const void *add_bf16, const void *w_bf16, float eps,
                                              int32_t M, int32_t K, int32_t mode, int8_t *q, float *scales,
                                              void *y_bf16, void *stream);

/* NULL on failure (vlab200_last_error() says why). */
VLAB200_API vlab200_bitvla_lm *vlab200_bitvla_lm_init(int32_t hidden, int32_t n_q, int32_t n_kv, int32_t head_dim,
                                                      int32_t ffn, int32_t n_layers, float rope_base,
                                                      float rms_eps, int32_t max_seq, int32_t max_batch);
VLAB200_API void vlab200_bitvla_lm_free(vlab200_bitvla_lm *ctx);
/* Weight pointers stay owned by the caller and must outlive the context (q/k/v packs are copied). */
VLAB200_API int32_t vlab200_bitvla_lm_set_layer(vlab200_bitvla_lm *ctx, int32_t L,
                                                const vlab200_bitvla_lm_layer *layer);
VLAB200_API int32_t vlab200_bitvla_lm_set_output_norm(vlab200_bitvla_lm *ctx, const void *w_bf16);
/* d_in, d_out: bf16 [n_seq*seq][hidden] device pointers; d_out = output_norm(layers(d_in)). */
VLAB200_API int32_t vlab200_bitvla_lm_forward(vlab200_bitvla_lm *ctx, const void *d_in, void *d_out, int32_t seq,
                                              int32_t n_seq, void *stream);

/* ---- GGUF checkpoints ------------------------------------------------------------------
 * Reader for the reference's on-disk format (GGUF v2 / v3, written by scripts/convert_*_to_gguf.py
 * through gguf.GGUFWriter).  The reference goes through ggml's gguf_* API and its wrapper
 * src/gguf_reader.h:60-200 (typed metadata getters, read_raw, read_f32, read_convert with the
 * Gemma-norm "+1"); this library parses the container itself (the file is mmap'ed read-only). */
typedef struct vlab200_gguf vlab200_gguf;

/* NULL on failure (vlab200_last_error() says why: missing file, bad magic, truncated directory...). */
VLAB200_API vlab200_gguf *vlab200_gguf_open(const char *path);
VLAB200_API void vlab200_gguf_close(vlab200_gguf *g);
VLAB200_API int64_t vlab200_gguf_n_tensors(const vlab200_gguf *g);
VLAB200_API const char *vlab200_gguf_tensor_name(const vlab200_gguf *g, int64_t index); /* file order */
/* type: ggml type id (0 F32, 1 F16, 30 BF16, 24 I8, 8 Q8_0 ...); dims: ggml order, dims[0] fastest;
 * n_bytes 0 for a type whose size this reader does not know.  VLAB200_ERR_ARG: no such tensor. */
VLAB200_API int32_t vlab200_gguf_tensor_info(const vlab200_gguf *g, const char *name, int32_t *type,
                                             int32_t *n_dims, int64_t dims[4], uint64_t *n_bytes);
/* Pointer into the mapping (valid until close); the read_raw of src/gguf_reader.h:119-136 without a copy. */
VLAB200_API const void *vlab200_gguf_tensor_data(const vlab200_gguf *g, const char *name);
/* F32 / F16 / BF16 tensor as float32; gemma_norm != 0 adds 1.0 to every element
 * (read_f32 + read_convert, src/gguf_reader.h:138-176).  n_elems must match the tensor. */
VLAB200_API int32_t vlab200_gguf_read_f32(const vlab200_gguf *g, const char *name, float *dst, int64_t n_elems,
                                          int32_t gemma_norm);
/* Typed metadata getters (u32 / f32-or-f64 / string); VLAB200_ERR_ARG when the key is absent or has
 * another type (src/gguf_reader.h:80-104). */
VLAB200_API int32_t vlab200_gguf_meta_u32(const vlab200_gguf *g, const char *key, uint32_t *out);
VLAB200_API int32_t vlab200_gguf_meta_f64(const vlab200_gguf *g, const char *key, double *out);
VLAB200_API int32_t vlab200_gguf_meta_str(const vlab200_gguf *g, const char *key, char *buf, int32_t cap);

/* The denoise engine of a pi0 or SmolVLA checkpoint (general.architecture "pi0" / "smolvla"; SmolVLA:
 * "smolvla.*" keys of src/models/smolvla.cpp:604-632, same tensor names through hf_to_gguf :648-703, no norm +1,
 * no state_proj in the loop).  pi0: metadata keys "pi0.*" (src/models/pi0.cpp:267-293), expert
 * tensors "aex.blk.N.{attn_norm,attn_q,attn_k,attn_v,attn_o,ffn_norm,ffn_gate,ffn_up,ffn_down}.weight",
 * "aex.output_norm.weight" (Gemma norms get their +1) and the projection heads
 * (src/modules/gemma_expert.h:46-62, src/models/pi0.cpp:431-437).  Matrices are uploaded as bf16,
 * vectors as float32; shapes are checked against the metadata.  NULL on failure. */
VLAB200_API vlab200_engine *vlab200_engine_create_from_gguf(const vlab200_gguf *g, int32_t max_obs,
                                                            int32_t prefix_len);

/* The BitVLA LM stack of a checkpoint: "bitvla.lm.*" metadata (src/models/bitvla.cpp:360-364), per
 * layer the four norm vectors and the six ladder-int2 tensors "lm.blk.N.<proj>.weight" (I8) with their
 * "<proj>.scale" float32 sidecars (scripts/convert_bitvla_to_gguf.py:165-178; a missing sidecar fails the
 * load as in bitvla.cpp:739-753), and "lm.output_norm.weight".  The context owns the uploaded weights. */
VLAB200_API vlab200_bitvla_lm *vlab200_bitvla_lm_create_from_gguf(const vlab200_gguf *g, int32_t max_seq,
                                                                  int32_t max_batch);

/* ---- node-level bf16 operators ----------------------------------------------------------
 * What a per-node CUDA hook dispatches when it is handed one graph node at a time: the
 * reference's vla_cuda_bf16_forward (src/cuda/vla_cuda_bf16.cu:698-720) handles MUL_MAT, ADD,
 * MUL, SCALE, NORM, RMS_NORM and UNARY on bf16 tensors.  Same arithmetic here: bf16 storage,
 * float32 math, one rounding per element.  All tensors contiguous; `stream` a cudaStream_t. */

/* out[b][m][n] = sum_k x[b][m][k] * w[b or 0][n][k]  (mul_mat, vla_cuda_bf16.cu:624-678, which
 * calls cuBLAS; here the tcgen05 GEMM of this library).  w_batched != 0: w is [n_batch][N][K].
 * K % 8 == 0 and 16-byte aligned pointers (TMA). */
VLAB200_API int32_t vlab200_node_mul_mat_bf16(const void *w_bf16, const void *x_bf16, void *out_bf16, int32_t N,
                                              int32_t M, int32_t K, int32_t n_batch, int32_t w_batched,
                                              void *stream);
/* out[i] = a[i] + b[i % nb] (op 0) or a[i] * b[i % nb] (op 1); b bf16, or float32 when b_is_f32
 * (bin_bcast, vla_cuda_bf16.cu:396-452).  n % nb == 0: b is broadcast over the leading dims. */
VLAB200_API int32_t vlab200_node_bin_bf16(int32_t op, const void *a_bf16, const void *b, int32_t b_is_f32,
                                          void *out_bf16, int64_t n, int64_t nb, void *stream);
/* The general form of add / mul with ggml's broadcast rule and strided operands, and the fused run of up to 8
 * ADD or MUL nodes that ggml hands over as one node:
 *   dst[i] = ((src0[i] op b_0[j]) op b_1[j]) ... op b_{n-1}[j]
 * i = (i0, i1, i2, i3) with extents ne[4] (ne[0] fastest), j = i with every dimension whose addend extent ne1[d]
 * is 1 set to 0.  All addends share one shape (ne1), one stride set (s1) and one type (bf16, or float32 when
 * addends_f32).  s0 / s1 / d: strides of src0 / the addends / dst in ELEMENTS.  Float accumulation, one rounding,
 * exactly as the unfused sequence would give (vla_cuda_bf16.cu:99-171 row-broadcast kernels, :330-389 fused
 * kernel).  VLAB200_ERR_UNSUPPORTED when ne[1] or ne[2]*ne[3] exceeds 65535 (the reference declines those too). */
VLAB200_API int32_t vlab200_node_bin_nd_bf16(int32_t op, const void *src0_bf16, const void *const *addends,
                                             int32_t n_addends, int32_t addends_f32, void *dst_bf16,
                                             const int64_t ne[4], const int64_t s0[4], const int64_t ne1[4],
                                             const int64_t s1[4], const int64_t d[4], void *stream);
/* out = scale * x + bias (vla_cuda_bf16.cu:501-527).  16-byte aligned pointers. */
VLAB200_API int32_t vlab200_node_scale_bf16(const void *x_bf16, void *out_bf16, int64_t n, float scale, float bias,
                                            void *stream);
/* op 0 SiLU, 1 ReLU, 2 GELU (tanh form), 3 GELU (erf form) (vla_cuda_bf16.cu:458-495).
 * 16-byte aligned pointers. */
VLAB200_API int32_t vlab200_node_unary_bf16(int32_t op, const void *x_bf16, void *out_bf16, int64_t n,
                                            void *stream);
/* Row norm without weight over [rows][cols]: rms != 0: x * rsqrt(mean x^2 + eps), else
 * (x - mean) * rsqrt(var + eps) (k_norm_bf16, vla_cuda_bf16.cu:546-605). */
VLAB200_API int32_t vlab200_node_norm_bf16(const void *x_bf16, void *out_bf16, int64_t rows, int64_t cols,
                                           float eps, int32_t rms, void *stream);

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

/* The reference's LM context API by its own names and signatures
 * (src/kernels/bitvla/bitvla_lm_cuda.h:247-286; callers src/models/bitvla.cpp:760-821,1326-1334): init
 * allocates the workspace for one sequence of up to max_seq tokens (NULL on failure), set_layer /
 * set_output_norm bind caller-owned device pointers, forward returns 0 or -1 and writes
 * d_out = output_norm(layers(d_in)) for seq x hidden bf16 rows.  Failures are reported on stderr as the
 * reference does.  They forward to vlab200_bitvla_lm_* with max_batch = n_seq = 1. */
typedef struct bitvla_lm_cuda_ctx bitvla_lm_cuda_ctx;
typedef vlab200_bitvla_lm_layer bitvla_lm_layer_cuda;
VLAB200_API bitvla_lm_cuda_ctx *bitvla_lm_cuda_init(int hidden, int n_q, int n_kv, int head_dim, int ffn,
                                                    int n_layers, float rope_base, float rms_eps, int max_seq);
VLAB200_API void bitvla_lm_cuda_free(bitvla_lm_cuda_ctx *ctx);
VLAB200_API void bitvla_lm_cuda_set_layer(bitvla_lm_cuda_ctx *ctx, int L, const bitvla_lm_layer_cuda *layer);
VLAB200_API void bitvla_lm_cuda_set_output_norm(bitvla_lm_cuda_ctx *ctx, const void *w);
VLAB200_API int bitvla_lm_cuda_forward(bitvla_lm_cuda_ctx *ctx, const void *d_in, void *d_out, int seq,
                                       void *stream);

/* The reference's vision-tower context API by its own names and signatures
 * (src/kernels/bitvla/bitvla_vit_cuda.h:44-144; forward src/kernels/bitvla/bitvla_vit_cuda.cu:161-330; callers
 * src/models/bitvla.cpp): a ternary SigLIP ViT (LayerNorm -> act-quant -> ternary q/k/v + bias -> unmasked attention ->
 * act-quant -> ternary o + bias -> residual -> LayerNorm -> act-quant -> ternary fc1 + bias -> tanh-GELU -> zero-pad
 * to a multiple of 128 -> act-quant -> ternary fc2 + bias -> residual, bf16 residual stream) between a bf16 patch
 * embedding (+ bias + position) and a two-layer projector (erf-GELU).  The layer struct has the reference's field
 * order; bf16 pointers are __nv_bfloat16*, `stream` a cudaStream_t.  init allocates every buffer (NULL on failure),
 * set_* bind caller-owned device pointers (q/k/v packs are copied into one fused matrix, the patch-embedding weight
 * into a copy with 16-byte rows, the projector biases into float32), forward returns 0 or -1 and writes
 * n_patches x mm_out bf16 rows for one image.  Needs hidden % 128 == 0, ffn % 16 == 0, mm_out % 8 == 0; head_dim
 * = hidden / n_heads is zero-padded to 64 / 128 / 256 for the attention kernel (softmax scale 1/sqrt(head_dim)). */
typedef struct {
    void *ln1_w, *ln1_b, *ln2_w, *ln2_b;   /* bf16 [hidden] */
    int8_t *q_packed; float *q_ws; void *q_b;       /* ladder pack [hidden][hidden], one scale, bf16 bias */
    int8_t *k_packed; float *k_ws; void *k_b;
    int8_t *v_packed; float *v_ws; void *v_b;
    int8_t *o_packed; float *o_ws; void *o_b;
    int8_t *fc1_packed; float *fc1_ws; void *fc1_b; /* [ffn][hidden] */
    int8_t *fc2_packed; float *fc2_ws; void *fc2_b; /* [hidden][ffn padded to a multiple of 128] */
} bitvla_vit_layer_cuda;
typedef struct bitvla_vit_cuda_ctx bitvla_vit_cuda_ctx;
VLAB200_API bitvla_vit_cuda_ctx *bitvla_vit_cuda_init(int n_layers, int hidden, int n_heads, int ffn, int n_patches,
                                                      int patch_flat, float ln_eps, int mm_out);
VLAB200_API void bitvla_vit_cuda_free(bitvla_vit_cuda_ctx *ctx);
VLAB200_API void bitvla_vit_cuda_set_layer(bitvla_vit_cuda_ctx *ctx, int L, const bitvla_vit_layer_cuda *layer);
VLAB200_API void bitvla_vit_cuda_set_embed(bitvla_vit_cuda_ctx *ctx, const void *patch_w, const void *patch_b,
                                           const void *pos_emb);
VLAB200_API void bitvla_vit_cuda_set_mmproj(bitvla_vit_cuda_ctx *ctx, const void *W1, const void *b1, const void *W2,
                                            const void *b2);
VLAB200_API int bitvla_vit_cuda_forward(bitvla_vit_cuda_ctx *ctx, const void *d_patches, void *d_out, void *stream);

/* The reference's float32 proprioception projector and action head by their own names and signatures
 * (src/kernels/bitvla/bitvla_fp32head_cuda.h:66-129; bodies src/kernels/bitvla/bitvla_fp32head_cuda.cu:186-358).
 * init copies the HOST weight arrays (PyTorch order [out][in]) to the device; proprio_forward maps a host state
 * vector [proprio_dim] to [lm_hidden] (fc1 -> erf-GELU -> fc2); action_forward maps host rows
 * [chunk][action_dim * lm_hidden] to normalised actions [chunk][action_dim] (LayerNorm -> fc1 -> ReLU -> two
 * residual blocks h += ReLU(W LayerNorm(h) + b) -> LayerNorm -> fc2); both synchronise `stream` (a cudaStream_t)
 * before they return 0 (or -1).  All arithmetic is float32. */
typedef struct bitvla_fp32head_cuda_ctx bitvla_fp32head_cuda_ctx;
VLAB200_API bitvla_fp32head_cuda_ctx *bitvla_fp32head_cuda_init(
    int proprio_dim, int lm_hidden, int chunk, int action_dim, float ah_ln_eps, const float *pp_fc1_w,
    const float *pp_fc1_b, const float *pp_fc2_w, const float *pp_fc2_b, const float *ah_ln1_w, const float *ah_ln1_b,
    const float *ah_fc1_w, const float *ah_fc1_b, const float *ah_b0_lnw, const float *ah_b0_lnb, const float *ah_b0_w,
    const float *ah_b0_b, const float *ah_b1_lnw, const float *ah_b1_lnb, const float *ah_b1_w, const float *ah_b1_b,
    const float *ah_ln2_w, const float *ah_ln2_b, const float *ah_fc2_w, const float *ah_fc2_b);
VLAB200_API int bitvla_fp32head_proprio_forward(bitvla_fp32head_cuda_ctx *ctx, const float *host_state, float *host_out,
                                                void *stream);
VLAB200_API int bitvla_fp32head_action_forward(bitvla_fp32head_cuda_ctx *ctx, const float *host_ah_input,
                                               float *host_norm_actions, void *stream);
VLAB200_API void bitvla_fp32head_cuda_free(bitvla_fp32head_cuda_ctx *ctx);

#ifdef __cplusplus
}
#endif
#endif /* VLA_B200_H */
