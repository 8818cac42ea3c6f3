// Node-level bf16 operators: what a per-node CUDA hook needs when it is handed ONE graph node at a
// time (the reference installs such a hook in ggml's CUDA backend: vla_cuda_bf16_forward dispatches
// MUL_MAT / ADD / MUL / SCALE / NORM / RMS_NORM / UNARY on bf16 tensors,
// src/cuda/vla_cuda_bf16.cu:698-720).  The fused kernels of this library make most of these nodes
// disappear from the denoise loop; the operators here cover the nodes that remain outside it, with the
// same arithmetic: bf16 storage, float math, one rounding per element.
//
//   mul_mat   persistent tcgen05 GEMM of gemm.cu (replaces the cuBLAS call, vla_cuda_bf16.cu:624-678)
//   others    HBM-bound streaming kernels, 16-byte accesses, grid = a few CTAs per SM
#include <cuda_bf16.h>

#include "gemm.h"
#include "host_common.h"

namespace vb {

__device__ __forceinline__ float2 unpack2(uint32_t u) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&u));
}
__device__ __forceinline__ uint32_t pack2(float a, float b) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t *>(&h);
}

enum { UN_SILU = 0, UN_RELU = 1, UN_GELU_TANH = 2, UN_GELU_ERF = 3 };

// src/cuda/vla_cuda_bf16.cu:463-474
template <int OP>
__device__ __forceinline__ float unary_f(float x) {
    if (OP == UN_SILU) return x / (1.0f + expf(-x));
    if (OP == UN_RELU) return x > 0.0f ? x : 0.0f;
    if (OP == UN_GELU_ERF) return 0.5f * x * (1.0f + erff(x * 0.70710678118654752440f));
    const float c = 0.79788456080286535588f;
    return 0.5f * x * (1.0f + tanhf(c * (x + 0.044715f * x * x * x)));
}

// out[i] = f(x[i]); MODE 0: unary OP, 1: scale * x + bias
template <int MODE, int OP>
__global__ void __launch_bounds__(256) map_kernel(const __nv_bfloat16 *__restrict__ x, __nv_bfloat16 *__restrict__ out,
                                                  int64_t n, float scale, float bias) {
    const int64_t nvec = n >> 3;
    const uint4 *xv = reinterpret_cast<const uint4 *>(x);
    uint4 *ov = reinterpret_cast<uint4 *>(out);
    auto f = [&](float v) { return MODE == 0 ? unary_f<OP>(v) : scale * v + bias; };
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
        const uint4 u = __ldg(xv + i);
        const float2 a = unpack2(u.x), b = unpack2(u.y), c = unpack2(u.z), d = unpack2(u.w);
        ov[i] = make_uint4(pack2(f(a.x), f(a.y)), pack2(f(b.x), f(b.y)), pack2(f(c.x), f(c.y)), pack2(f(d.x), f(d.y)));
    }
    for (int64_t i = (nvec << 3) + blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        out[i] = __float2bfloat16(f(__bfloat162float(x[i])));
}

// out[i] = a[i] (+|*) b[i % nb]; b bf16 or float32 (the reference's fused add takes a float32 src1)
template <bool MUL, typename TB>
__global__ void __launch_bounds__(256) bin_kernel(const __nv_bfloat16 *__restrict__ a, const TB *__restrict__ b,
                                                  __nv_bfloat16 *__restrict__ out, int64_t n, int64_t nb) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const float x = __bfloat162float(a[i]);
        const float y = static_cast<float>(b[nb == n ? i : i % nb]);
        out[i] = __float2bfloat16(MUL ? x * y : x + y);
    }
}

// 8 elements per thread and iteration (16-byte accesses); n % 8 == 0, nb % 8 == 0, 16-byte aligned pointers
template <bool MUL, typename TB>
__global__ void __launch_bounds__(256) bin_vec_kernel(const __nv_bfloat16 *__restrict__ a, const TB *__restrict__ b,
                                                      __nv_bfloat16 *__restrict__ out, int64_t n8, int64_t nb8) {
    const uint4 *av = reinterpret_cast<const uint4 *>(a);
    uint4 *ov = reinterpret_cast<uint4 *>(out);
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n8; i += (int64_t)gridDim.x * blockDim.x) {
        const uint4 x = __ldg(av + i);
        const int64_t j = nb8 == n8 ? i : i % nb8;
        float y[8];
        if (sizeof(TB) == 2) {
            const uint4 u = __ldg(reinterpret_cast<const uint4 *>(b) + j);
            const float2 p0 = unpack2(u.x), p1 = unpack2(u.y), p2 = unpack2(u.z), p3 = unpack2(u.w);
            y[0] = p0.x; y[1] = p0.y; y[2] = p1.x; y[3] = p1.y; y[4] = p2.x; y[5] = p2.y; y[6] = p3.x; y[7] = p3.y;
        } else {
            const float4 u0 = __ldg(reinterpret_cast<const float4 *>(b) + 2 * j), u1 = __ldg(reinterpret_cast<const float4 *>(b) + 2 * j + 1);
            y[0] = u0.x; y[1] = u0.y; y[2] = u0.z; y[3] = u0.w; y[4] = u1.x; y[5] = u1.y; y[6] = u1.z; y[7] = u1.w;
        }
        const float2 x0 = unpack2(x.x), x1 = unpack2(x.y), x2 = unpack2(x.z), x3 = unpack2(x.w);
        auto f = [](float p, float q) { return MUL ? p * q : p + q; };
        ov[i] = make_uint4(pack2(f(x0.x, y[0]), f(x0.y, y[1])), pack2(f(x1.x, y[2]), f(x1.y, y[3])),
                           pack2(f(x2.x, y[4]), f(x2.y, y[5])), pack2(f(x3.x, y[6]), f(x3.y, y[7])));
    }
}

// one CTA per row: (x - mean) * rsqrt(var + eps), or x * rsqrt(mean x^2 + eps) (src/cuda/vla_cuda_bf16.cu:548-579)
template <bool RMS>
__global__ void __launch_bounds__(256) norm_kernel(const __nv_bfloat16 *__restrict__ x, __nv_bfloat16 *__restrict__ out,
                                                   int64_t cols, float eps, bool vec) {
    __shared__ float red[2][8];
    const __nv_bfloat16 *xr = x + (size_t)blockIdx.x * cols;
    __nv_bfloat16 *orow = out + (size_t)blockIdx.x * cols;
    float s = 0.f, ss = 0.f;
    if (vec) {  // cols % 8 == 0 and 16-byte aligned rows
        const uint4 *xv = reinterpret_cast<const uint4 *>(xr);
        for (int64_t c = threadIdx.x; c < (cols >> 3); c += 256) {
            const uint4 u = __ldg(xv + c);
            const float2 a = unpack2(u.x), b = unpack2(u.y), d = unpack2(u.z), e = unpack2(u.w);
            s += ((a.x + a.y) + (b.x + b.y)) + ((d.x + d.y) + (e.x + e.y));
            ss += ((a.x * a.x + a.y * a.y) + (b.x * b.x + b.y * b.y)) + ((d.x * d.x + d.y * d.y) + (e.x * e.x + e.y * e.y));
        }
    } else {
        for (int64_t c = threadIdx.x; c < cols; c += 256) {
            const float v = __bfloat162float(xr[c]);
            s += v;
            ss += v * v;
        }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        s += __shfl_xor_sync(0xffffffffu, s, off);
        ss += __shfl_xor_sync(0xffffffffu, ss, off);
    }
    if ((threadIdx.x & 31) == 0) {
        red[0][threadIdx.x >> 5] = s;
        red[1][threadIdx.x >> 5] = ss;
    }
    __syncthreads();
    s = ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        s += red[0][i];
        ss += red[1][i];
    }
    const float mean = RMS ? 0.0f : s / (float)cols;
    const float inv = rsqrtf(ss / (float)cols - mean * mean + eps);
    if (vec) {
        const uint4 *xv = reinterpret_cast<const uint4 *>(xr);
        uint4 *ov = reinterpret_cast<uint4 *>(orow);
        for (int64_t c = threadIdx.x; c < (cols >> 3); c += 256) {
            const uint4 u = __ldg(xv + c);
            const float2 a = unpack2(u.x), b = unpack2(u.y), d = unpack2(u.z), e = unpack2(u.w);
            ov[c] = make_uint4(pack2((a.x - mean) * inv, (a.y - mean) * inv), pack2((b.x - mean) * inv, (b.y - mean) * inv),
                               pack2((d.x - mean) * inv, (d.y - mean) * inv), pack2((e.x - mean) * inv, (e.y - mean) * inv));
        }
    } else {
        for (int64_t c = threadIdx.x; c < cols; c += 256) orow[c] = __float2bfloat16((__bfloat162float(xr[c]) - mean) * inv);
    }
}

// dst[i0,i1,i2,i3] = ((src0[..] op b_0[j]) op b_1[j]) ... op b_{n-1}[j], j the ggml-broadcast index of (i0..i3) in the
// addends' shape (extent 1 or equal per dimension, every addend with the same shape and strides), float accumulation,
// one rounding.  Covers the reference's row-broadcast kernels and its fused run of up to 8 ADD / MUL nodes
// (src/cuda/vla_cuda_bf16.cu:99-171,358-389).  Grid: x over dim 0, y = dim 1, z = dims 2 and 3, so the index
// arithmetic is paid once per CTA.  Strides are in elements.
constexpr int kMaxFuse = 8;
template <typename TB>
struct AddendPtrs {
    const TB *p[kMaxFuse];
};
struct NdShape {
    int64_t ne[4], s0[4], ne1[4], s1[4], d[4];
};

template <bool MUL, typename TB>
__global__ void __launch_bounds__(256) bin_nd_kernel(const __nv_bfloat16 *__restrict__ src0, const AddendPtrs<TB> b, int n_b,
                                                     __nv_bfloat16 *__restrict__ dst, const NdShape sh) {
    const int64_t i1 = blockIdx.y, i2 = blockIdx.z % sh.ne[2], i3 = blockIdx.z / sh.ne[2];
    const int64_t row1 = (sh.ne1[1] == 1 ? 0 : i1) * sh.s1[1] + (sh.ne1[2] == 1 ? 0 : i2) * sh.s1[2] +
                         (sh.ne1[3] == 1 ? 0 : i3) * sh.s1[3];
    const __nv_bfloat16 *r0 = src0 + i1 * sh.s0[1] + i2 * sh.s0[2] + i3 * sh.s0[3];
    __nv_bfloat16 *rd = dst + i1 * sh.d[1] + i2 * sh.d[2] + i3 * sh.d[3];
    const bool bc0 = sh.ne1[0] == 1;
    for (int64_t i0 = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i0 < sh.ne[0]; i0 += (int64_t)gridDim.x * blockDim.x) {
        const int64_t j = row1 + (bc0 ? 0 : i0) * sh.s1[0];
        float acc = __bfloat162float(r0[i0 * sh.s0[0]]);
        for (int k = 0; k < n_b; ++k) {
            const float y = static_cast<float>(b.p[k][j]);
            acc = MUL ? acc * y : acc + y;
        }
        rd[i0 * sh.d[0]] = __float2bfloat16(acc);
    }
}

static int stream_grid(int64_t work_items) {
    int n_sm = sm_count();
    if (n_sm <= 0) n_sm = 148;
    const int64_t blocks = (work_items + 255) / 256;
    const int64_t cap = (int64_t)n_sm * 8;
    return (int)(blocks < 1 ? 1 : (blocks < cap ? blocks : cap));
}

}  // namespace vb

extern "C" {

int32_t vlab200_node_mul_mat_bf16(const void *w_bf16, const void *x_bf16, void *out_bf16, int32_t N, int32_t M, int32_t K,
                                  int32_t n_batch, int32_t w_batched, void *stream) {
    if (!w_bf16 || !x_bf16 || !out_bf16 || N <= 0 || M < 0 || K <= 0 || n_batch <= 0) return VLAB200_ERR_ARG;
    if (M == 0) return VLAB200_OK;
    for (int b = 0; b < n_batch; ++b) {
        vb::GemmParams p{};
        p.M = M; p.N = N; p.K = K; p.epi = vb::EPI_BIAS_ACT; p.act = vb::ACT_NONE;
        p.out_bf = static_cast<__nv_bfloat16 *>(out_bf16) + (size_t)b * M * N;
        p.ld_out = N;
        const __nv_bfloat16 *w = static_cast<const __nv_bfloat16 *>(w_bf16) + (w_batched ? (size_t)b * N * K : 0);
        const __nv_bfloat16 *x = static_cast<const __nv_bfloat16 *>(x_bf16) + (size_t)b * M * K;
        const int rc = vb::dense_gemm(x, K, w, p, static_cast<cudaStream_t>(stream));
        if (rc) return rc;
    }
    return VLAB200_OK;
}

int32_t vlab200_node_bin_bf16(int32_t op, const void *a_bf16, const void *b, int32_t b_is_f32, void *out_bf16, int64_t n,
                              int64_t nb, void *stream) {
    if (!a_bf16 || !b || !out_bf16 || n < 0 || nb <= 0 || (op != 0 && op != 1) || n % nb) return VLAB200_ERR_ARG;
    if (n == 0) return VLAB200_OK;
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    const int grid = vb::stream_grid(n);
    const __nv_bfloat16 *a = static_cast<const __nv_bfloat16 *>(a_bf16);
    __nv_bfloat16 *o = static_cast<__nv_bfloat16 *>(out_bf16);
    if (n % 8 == 0 && nb % 8 == 0 &&
        ((reinterpret_cast<uintptr_t>(a_bf16) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(out_bf16)) & 15) == 0) {
        const int vgrid = vb::stream_grid(n / 8);
        const int64_t n8 = n / 8, nb8 = nb / 8;
        if (b_is_f32) {
            if (op) vb::bin_vec_kernel<true, float><<<vgrid, 256, 0, cs>>>(a, static_cast<const float *>(b), o, n8, nb8);
            else vb::bin_vec_kernel<false, float><<<vgrid, 256, 0, cs>>>(a, static_cast<const float *>(b), o, n8, nb8);
        } else {
            if (op) vb::bin_vec_kernel<true, __nv_bfloat16><<<vgrid, 256, 0, cs>>>(a, static_cast<const __nv_bfloat16 *>(b), o, n8, nb8);
            else vb::bin_vec_kernel<false, __nv_bfloat16><<<vgrid, 256, 0, cs>>>(a, static_cast<const __nv_bfloat16 *>(b), o, n8, nb8);
        }
        VB_CUDA(cudaGetLastError());
        return VLAB200_OK;
    }
    if (b_is_f32) {
        if (op) vb::bin_kernel<true, float><<<grid, 256, 0, cs>>>(a, static_cast<const float *>(b), o, n, nb);
        else vb::bin_kernel<false, float><<<grid, 256, 0, cs>>>(a, static_cast<const float *>(b), o, n, nb);
    } else {
        if (op) vb::bin_kernel<true, __nv_bfloat16><<<grid, 256, 0, cs>>>(a, static_cast<const __nv_bfloat16 *>(b), o, n, nb);
        else vb::bin_kernel<false, __nv_bfloat16><<<grid, 256, 0, cs>>>(a, static_cast<const __nv_bfloat16 *>(b), o, n, nb);
    }
    VB_CUDA(cudaGetLastError());
    return VLAB200_OK;
}

int32_t vlab200_node_bin_nd_bf16(int32_t op, const void *src0_bf16, const void *const *addends, int32_t n_addends,
                                 int32_t addends_f32, void *dst_bf16, const int64_t ne[4], const int64_t s0[4],
                                 const int64_t ne1[4], const int64_t s1[4], const int64_t d[4], void *stream) {
    if (!src0_bf16 || !addends || !dst_bf16 || !ne || !s0 || !ne1 || !s1 || !d || (op != 0 && op != 1)) return VLAB200_ERR_ARG;
    if (n_addends < 1 || n_addends > vb::kMaxFuse) return VLAB200_ERR_UNSUPPORTED;
    vb::NdShape sh;
    for (int i = 0; i < 4; ++i) {
        if (ne[i] < 0 || ne1[i] < 1 || (ne1[i] != 1 && ne1[i] != ne[i])) return VLAB200_ERR_ARG;  // ggml broadcast: 1 or equal
        sh.ne[i] = ne[i]; sh.s0[i] = s0[i]; sh.ne1[i] = ne1[i]; sh.s1[i] = s1[i]; sh.d[i] = d[i];
    }
    if (ne[0] == 0 || ne[1] == 0 || ne[2] == 0 || ne[3] == 0) return VLAB200_OK;
    if (ne[1] > 65535 || ne[2] * ne[3] > 65535) return VLAB200_ERR_UNSUPPORTED;  // the caller declines such a node
    for (int k = 0; k < n_addends; ++k)
        if (!addends[k]) return VLAB200_ERR_ARG;
    unsigned bx = 32;
    while (bx < 256 && (int64_t)bx < ne[0]) bx *= 2;
    int64_t gx = (ne[0] + bx - 1) / bx;
    if (gx > 1024) gx = 1024;
    const dim3 grid((unsigned)gx, (unsigned)ne[1], (unsigned)(ne[2] * ne[3]));
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    const __nv_bfloat16 *a = static_cast<const __nv_bfloat16 *>(src0_bf16);
    __nv_bfloat16 *o = static_cast<__nv_bfloat16 *>(dst_bf16);
    if (addends_f32) {
        vb::AddendPtrs<float> b{};
        for (int k = 0; k < n_addends; ++k) b.p[k] = static_cast<const float *>(addends[k]);
        if (op) vb::bin_nd_kernel<true, float><<<grid, bx, 0, cs>>>(a, b, n_addends, o, sh);
        else vb::bin_nd_kernel<false, float><<<grid, bx, 0, cs>>>(a, b, n_addends, o, sh);
    } else {
        vb::AddendPtrs<__nv_bfloat16> b{};
        for (int k = 0; k < n_addends; ++k) b.p[k] = static_cast<const __nv_bfloat16 *>(addends[k]);
        if (op) vb::bin_nd_kernel<true, __nv_bfloat16><<<grid, bx, 0, cs>>>(a, b, n_addends, o, sh);
        else vb::bin_nd_kernel<false, __nv_bfloat16><<<grid, bx, 0, cs>>>(a, b, n_addends, o, sh);
    }
    VB_CUDA(cudaGetLastError());
    return VLAB200_OK;
}

int32_t vlab200_node_scale_bf16(const void *x_bf16, void *out_bf16, int64_t n, float scale, float bias, void *stream) {
    if (!x_bf16 || !out_bf16 || n < 0) return VLAB200_ERR_ARG;
    if ((reinterpret_cast<uintptr_t>(x_bf16) & 15) || (reinterpret_cast<uintptr_t>(out_bf16) & 15)) return VLAB200_ERR_ARG;
    if (n == 0) return VLAB200_OK;
    vb::map_kernel<1, 0><<<vb::stream_grid((n + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16 *>(x_bf16), static_cast<__nv_bfloat16 *>(out_bf16), n, scale, bias);
    VB_CUDA(cudaGetLastError());
    return VLAB200_OK;
}

int32_t vlab200_node_unary_bf16(int32_t op, const void *x_bf16, void *out_bf16, int64_t n, void *stream) {
    if (!x_bf16 || !out_bf16 || n < 0 || op < 0 || op > 3) return VLAB200_ERR_ARG;
    if ((reinterpret_cast<uintptr_t>(x_bf16) & 15) || (reinterpret_cast<uintptr_t>(out_bf16) & 15)) return VLAB200_ERR_ARG;
    if (n == 0) return VLAB200_OK;
    const int grid = vb::stream_grid((n + 7) / 8);
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    const __nv_bfloat16 *x = static_cast<const __nv_bfloat16 *>(x_bf16);
    __nv_bfloat16 *o = static_cast<__nv_bfloat16 *>(out_bf16);
    switch (op) {
        case vb::UN_SILU: vb::map_kernel<0, vb::UN_SILU><<<grid, 256, 0, cs>>>(x, o, n, 0.f, 0.f); break;
        case vb::UN_RELU: vb::map_kernel<0, vb::UN_RELU><<<grid, 256, 0, cs>>>(x, o, n, 0.f, 0.f); break;
        case vb::UN_GELU_TANH: vb::map_kernel<0, vb::UN_GELU_TANH><<<grid, 256, 0, cs>>>(x, o, n, 0.f, 0.f); break;
        default: vb::map_kernel<0, vb::UN_GELU_ERF><<<grid, 256, 0, cs>>>(x, o, n, 0.f, 0.f); break;
    }
    VB_CUDA(cudaGetLastError());
    return VLAB200_OK;
}

int32_t vlab200_node_norm_bf16(const void *x_bf16, void *out_bf16, int64_t rows, int64_t cols, float eps, int32_t rms,
                               void *stream) {
    if (!x_bf16 || !out_bf16 || rows < 0 || cols <= 0 || rows > 2147483647) return VLAB200_ERR_ARG;
    if (rows == 0) return VLAB200_OK;
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    const bool vec = cols % 8 == 0 && ((reinterpret_cast<uintptr_t>(x_bf16) | reinterpret_cast<uintptr_t>(out_bf16)) & 15) == 0;
    if (rms)
        vb::norm_kernel<true><<<(int)rows, 256, 0, cs>>>(static_cast<const __nv_bfloat16 *>(x_bf16),
                                                        static_cast<__nv_bfloat16 *>(out_bf16), cols, eps, vec);
    else
        vb::norm_kernel<false><<<(int)rows, 256, 0, cs>>>(static_cast<const __nv_bfloat16 *>(x_bf16),
                                                         static_cast<__nv_bfloat16 *>(out_bf16), cols, eps, vec);
    VB_CUDA(cudaGetLastError());
    return VLAB200_OK;
}

}  // extern "C"
