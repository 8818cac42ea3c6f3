/* Test stand-in for llama.cpp's public ggml.h: ONLY the names vla_cpp_b200/csrc/ggml_hook_adapter.cpp uses, with
 * the meaning the public API documents (ne[] extents with ne[0] fastest, nb[] byte strides, src[] operands,
 * op_params raw parameter words).  Field order and enumerator values are this file's own -- the adapter refers
 * to everything by name, so it compiles unchanged against the real header. */
#pragma once
#include <stddef.h>
#include <stdint.h>

#define GGML_MAX_DIMS 4
#define GGML_MAX_SRC 10

enum ggml_type { GGML_TYPE_F32 = 0, GGML_TYPE_F16 = 1, GGML_TYPE_BF16 = 30 };
enum ggml_op { GGML_OP_NONE = 0, GGML_OP_ADD, GGML_OP_MUL, GGML_OP_SCALE, GGML_OP_NORM, GGML_OP_RMS_NORM, GGML_OP_MUL_MAT,
               GGML_OP_UNARY, GGML_OP_SOFT_MAX };
enum ggml_unary_op { GGML_UNARY_OP_ABS = 0, GGML_UNARY_OP_SILU, GGML_UNARY_OP_RELU, GGML_UNARY_OP_GELU, GGML_UNARY_OP_GELU_ERF,
                     GGML_UNARY_OP_TANH };

struct ggml_tensor {
    enum ggml_type type;
    int64_t ne[GGML_MAX_DIMS];
    size_t nb[GGML_MAX_DIMS];
    enum ggml_op op;
    int32_t op_params[16];
    struct ggml_tensor *src[GGML_MAX_SRC];
    void *data;
};

static inline size_t ggml_type_size(enum ggml_type t) { return t == GGML_TYPE_F32 ? 4 : 2; }
static inline int64_t ggml_nelements(const struct ggml_tensor *t) { return t->ne[0] * t->ne[1] * t->ne[2] * t->ne[3]; }
static inline bool ggml_is_contiguous(const struct ggml_tensor *t) {
    size_t want = ggml_type_size(t->type);
    for (int i = 0; i < GGML_MAX_DIMS; ++i) {
        if (t->ne[i] != 1 && t->nb[i] != want) return false;
        want *= (size_t)t->ne[i];
    }
    return true;
}
static inline bool ggml_are_same_shape(const struct ggml_tensor *a, const struct ggml_tensor *b) {
    for (int i = 0; i < GGML_MAX_DIMS; ++i)
        if (a->ne[i] != b->ne[i]) return false;
    return true;
}
/* a can be repeated to b's shape: every extent of b is a multiple of a's */
static inline bool ggml_can_repeat(const struct ggml_tensor *a, const struct ggml_tensor *b) {
    for (int i = 0; i < GGML_MAX_DIMS; ++i)
        if (a->ne[i] <= 0 || b->ne[i] % a->ne[i]) return false;
    return true;
}
static inline enum ggml_unary_op ggml_get_unary_op(const struct ggml_tensor *t) { return (enum ggml_unary_op)t->op_params[0]; }
