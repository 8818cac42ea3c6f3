// ggml CUDA extension hook on top of libvla_b200.so: the two symbols the reference's hook patch consults
// (scripts/patch_ggml_cuda_ext_hook.py:58-111) --
//     bool vla_cuda_bf16_forward(ggml_tensor *dst, void *stream)
//     bool vla_cuda_bf16_fused_binbcast(ggml_tensor *dst, int n_fuse, void *stream)
// with the typedefs of src/cuda/vla_cuda_bf16.cu:48-55, plus vla::cuda_register_bf16_ops() (:725-735), which
// installs them.  Contract (same as the reference's file): return false = "not mine", ggml runs its own kernel;
// everything is read from the public ggml_tensor fields; runs on ggml's stream, never synchronises or
// allocates; anything the operators cannot address (views of the wrong kind, oversized grids) is declined.
//
// Needs ggml.h (llama.cpp, not part of this repository): build with
//     g++ -std=c++17 -fPIC -shared -I$VLA_GGML_DIR/include -Iinclude ggml_hook_adapter.cpp -L... -lvla_b200
// and link it into the program that owns the patched ggml-cuda.  The tests compile it against a minimal
// stand-in header that declares the same public names.
#include <cstdint>
#include <cstring>

#include "ggml.h"
#include "vla_b200.h"

extern "C" {
typedef bool (*ggml_cuda_ext_forward_t)(struct ggml_tensor *dst, void *stream);
typedef bool (*ggml_cuda_ext_fused_binbcast_t)(struct ggml_tensor *dst, int n_fuse, void *stream);
#ifndef VLA_HOOK_NO_GGML_GLOBALS
extern ggml_cuda_ext_forward_t ggml_cuda_ext_forward;
extern ggml_cuda_ext_fused_binbcast_t ggml_cuda_ext_fused_binbcast;
#endif
}

namespace {

inline int64_t elem_stride(const ggml_tensor *t, int i) { return (int64_t)(t->nb[i] / ggml_type_size(t->type)); }

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// ADD / MUL with ggml broadcast; n_fuse addends in dst->src[1 .. n_fuse], all with src[1]'s layout and type.
bool bin_bcast(ggml_tensor *dst, int op, int n_fuse, void *stream) {
    const ggml_tensor *src0 = dst->src[0], *src1 = dst->src[1];
    if (!src0 || !src1 || n_fuse < 1 || n_fuse > 8) return false;
    if (dst->type != GGML_TYPE_BF16 || src0->type != GGML_TYPE_BF16) return false;
    if (src1->type != GGML_TYPE_BF16 && src1->type != GGML_TYPE_F32) return false;
    if (!ggml_are_same_shape(src0, dst) || !ggml_can_repeat(src1, src0)) return false;
    const void *addends[8];
    addends[0] = src1->data;
    for (int k = 1; k < n_fuse; ++k) {  // re-checked rather than trusted: a mismatch would read out of bounds
        const ggml_tensor *s = dst->src[k + 1];
        if (!s || s->type != src1->type || !ggml_are_same_shape(s, src1)) return false;
        for (int d = 0; d < GGML_MAX_DIMS; ++d)
            if (s->nb[d] != src1->nb[d]) return false;
        addends[k] = s->data;
    }
    // the contiguous, trailing-dimension broadcast goes through the 16-byte vectorised operator
    if (n_fuse == 1 && ggml_is_contiguous(src0) && ggml_is_contiguous(dst) && ggml_is_contiguous(src1)) {
        bool trailing = true;  // src1 covers the fastest dims entirely and is 1 in the rest
        bool seen_one = false;
        for (int d = 0; d < GGML_MAX_DIMS; ++d) {
            if (src1->ne[d] == dst->ne[d] && !seen_one) continue;
            if (src1->ne[d] == 1) { seen_one = true; continue; }
            trailing = false;
        }
        if (trailing)
            return vlab200_node_bin_bf16(op, src0->data, src1->data, src1->type == GGML_TYPE_F32, dst->data,
                                         ggml_nelements(dst), ggml_nelements(src1), stream) == VLAB200_OK;
    }
    int64_t ne[4], s0[4], ne1[4], s1[4], d[4];
    for (int i = 0; i < 4; ++i) {
        ne[i] = dst->ne[i]; s0[i] = elem_stride(src0, i); ne1[i] = src1->ne[i];
        s1[i] = elem_stride(src1, i); d[i] = elem_stride(dst, i);
    }
    return vlab200_node_bin_nd_bf16(op, src0->data, addends, n_fuse, src1->type == GGML_TYPE_F32, dst->data, ne, s0, ne1,
                                    s1, d, stream) == VLAB200_OK;
}

bool mul_mat(ggml_tensor *dst, void *stream) {
    const ggml_tensor *w = dst->src[0], *x = dst->src[1];
    if (!w || !x) return false;
    if (dst->type != GGML_TYPE_BF16 || w->type != GGML_TYPE_BF16 || x->type != GGML_TYPE_BF16) return false;
    if (!ggml_is_contiguous(w) || !ggml_is_contiguous(x) || !ggml_is_contiguous(dst)) return false;
    const bool shared = w->ne[2] == 1 && w->ne[3] == 1;
    if (!shared && !(w->ne[2] == x->ne[2] && w->ne[3] == x->ne[3])) return false;
    if (w->ne[0] % 8 || !aligned16(w->data) || !aligned16(x->data) || !aligned16(dst->data)) return false;  // TMA operands
    return vlab200_node_mul_mat_bf16(w->data, x->data, dst->data, (int32_t)w->ne[1], (int32_t)x->ne[1], (int32_t)x->ne[0],
                                     (int32_t)(x->ne[2] * x->ne[3]), shared ? 0 : 1, stream) == VLAB200_OK;
}

bool dense_bf16_pair(const ggml_tensor *dst) {
    const ggml_tensor *x = dst->src[0];
    return x && dst->type == GGML_TYPE_BF16 && x->type == GGML_TYPE_BF16 && ggml_is_contiguous(x) && ggml_is_contiguous(dst) &&
           aligned16(x->data) && aligned16(dst->data);
}

bool scale(ggml_tensor *dst, void *stream) {
    if (!dense_bf16_pair(dst)) return false;
    float s = 1.0f, b = 0.0f;
    std::memcpy(&s, reinterpret_cast<const char *>(dst->op_params), sizeof(float));
    std::memcpy(&b, reinterpret_cast<const char *>(dst->op_params) + sizeof(float), sizeof(float));
    return vlab200_node_scale_bf16(dst->src[0]->data, dst->data, ggml_nelements(dst), s, b, stream) == VLAB200_OK;
}

bool norm(ggml_tensor *dst, bool rms, void *stream) {
    if (!dense_bf16_pair(dst)) return false;
    float eps = 0.0f;
    std::memcpy(&eps, dst->op_params, sizeof(float));
    const int64_t cols = dst->src[0]->ne[0];
    if (cols <= 0) return false;
    return vlab200_node_norm_bf16(dst->src[0]->data, dst->data, ggml_nelements(dst) / cols, cols, eps, rms ? 1 : 0, stream) ==
           VLAB200_OK;
}

bool unary(ggml_tensor *dst, void *stream) {
    if (!dense_bf16_pair(dst)) return false;
    int op;
    switch (ggml_get_unary_op(dst)) {
    case GGML_UNARY_OP_SILU: op = 0; break;
    case GGML_UNARY_OP_RELU: op = 1; break;
    case GGML_UNARY_OP_GELU: op = 2; break;
    case GGML_UNARY_OP_GELU_ERF: op = 3; break;
    default: return false;
    }
    return vlab200_node_unary_bf16(op, dst->src[0]->data, dst->data, ggml_nelements(dst), stream) == VLAB200_OK;
}

}  // namespace

extern "C" __attribute__((visibility("default"))) bool vla_cuda_bf16_fused_binbcast(ggml_tensor *dst, int n_fuse, void *stream) {
    if (!dst || n_fuse < 2) return false;
    if (dst->op == GGML_OP_ADD) return bin_bcast(dst, 0, n_fuse, stream);
    if (dst->op == GGML_OP_MUL) return bin_bcast(dst, 1, n_fuse, stream);
    return false;
}

extern "C" __attribute__((visibility("default"))) bool vla_cuda_bf16_forward(ggml_tensor *dst, void *stream) {
    if (!dst) return false;
    switch (dst->op) {
    case GGML_OP_MUL_MAT: return mul_mat(dst, stream);
    case GGML_OP_ADD: return bin_bcast(dst, 0, 1, stream);
    case GGML_OP_MUL: return bin_bcast(dst, 1, 1, stream);
    case GGML_OP_SCALE: return scale(dst, stream);
    case GGML_OP_NORM: return norm(dst, false, stream);
    case GGML_OP_RMS_NORM: return norm(dst, true, stream);
    case GGML_OP_UNARY: return unary(dst, stream);
    default: return false;
    }
}

#ifndef VLA_HOOK_NO_GGML_GLOBALS
namespace vla {
// Installs both hooks; call once after the CUDA backend is up (idempotent).
void cuda_register_bf16_ops() {
    ggml_cuda_ext_forward = vla_cuda_bf16_forward;
    ggml_cuda_ext_fused_binbcast = vla_cuda_bf16_fused_binbcast;
}
}  // namespace vla
#endif
