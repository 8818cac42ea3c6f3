#include "host_common.h"
#include "tc5.cuh"

#include <cstdarg>
#include <cstring>
#include <map>
#include <mutex>
#include <utility>

namespace vb {

__device__ int g_dev_status;

static thread_local char g_last_error[256] = "";

void set_last_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    std::vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
    va_end(ap);
}

int cuda_fail(cudaError_t e, const char *what) {
    std::snprintf(g_last_error, sizeof(g_last_error), "CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e),
                  what);
    return VLAB200_ERR_CUDA;
}

int *device_status_ptr() {
    static int *ptrs[64] = {nullptr};
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lk(mu);
    if (!ptrs[dev]) {
        void *p = nullptr;
        if (cudaGetSymbolAddress(&p, g_dev_status) != cudaSuccess) return nullptr;
        ptrs[dev] = static_cast<int *>(p);
    }
    return ptrs[dev];
}

int sm_count() {
    static int counts[64] = {0};
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    std::lock_guard<std::mutex> lk(mu);
    if (!counts[dev]) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
        counts[dev] = n;
    }
    return counts[dev];
}

int ensure_dyn_smem(const void *func, int bytes) {
    static std::map<std::pair<int, const void *>, int> opted;  // (device, kernel) -> bytes opted into
    static std::mutex mu;
    int dev = 0;
    VB_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lk(mu);
    int &have = opted[std::make_pair(dev, func)];
    if (bytes > have) {
        VB_CUDA(cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
        have = bytes;
    }
    return VLAB200_OK;
}

typedef CUresult (*encode_tiled_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                    const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                    CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                    CUtensorMapFloatOOBfill);

static encode_tiled_fn get_encode() {
    static encode_tiled_fn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<encode_tiled_fn>(p);
    });
    return fn;
}

int make_tensor_map(CUtensorMap *map, CUtensorMapDataType dt, int rank, const void *base, const uint64_t *dims,
                    const uint64_t *strides_bytes, const uint32_t *box, CUtensorMapSwizzle swz) {
    encode_tiled_fn fn = get_encode();
    if (!fn) {
        std::snprintf(g_last_error, sizeof(g_last_error), "cuTensorMapEncodeTiled entry point unavailable");
        return VLAB200_ERR_CUDA;
    }
    cuuint64_t gdim[5];
    cuuint64_t gstr[5];
    cuuint32_t bx[5], es[5];
    for (int i = 0; i < rank; ++i) {
        gdim[i] = dims[i];
        bx[i] = box[i];
        es[i] = 1;
        if (i + 1 < rank) gstr[i] = strides_bytes[i];
    }
    CUresult r = fn(map, dt, (cuuint32_t)rank, const_cast<void *>(base), gdim, gstr, bx, es,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        std::snprintf(g_last_error, sizeof(g_last_error), "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
        return VLAB200_ERR_CUDA;
    }
    return VLAB200_OK;
}

}  // namespace vb

namespace vb {

// Self-test of the bounded wait every kernel of this library relies on: two warps wait on an mbarrier that
// nobody arrives at.  The first to exhaust the budget raises the CTA's abort flag and records
// DEV_TIMEOUT_MISC; the other leaves through the flag; both reach the common exit.
__global__ void bounded_wait_selftest_kernel(int *status, long long budget, int *out) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        abort_flag = 0;
    }
    fence_barrier_init();
    __syncthreads();
    WaitCtx w{&abort_flag, status, budget};
    bool ok = true;
    if ((threadIdx.x & 31) == 0) ok = mbar_wait(&bar, 0, w, DEV_TIMEOUT_MISC);
    __syncthreads();  // the common exit of every role
    if ((threadIdx.x & 31) == 0) out[threadIdx.x >> 5] = ok ? 0 : 1;
    if (threadIdx.x == 0) out[2] = abort_flag;
}

}  // namespace vb

extern "C" {

int32_t vlab200_selftest_bounded_wait(int64_t budget_cycles, int32_t *gave_up, void *stream) {
    if (!gave_up || budget_cycles <= 0 || budget_cycles > 100000000) return VLAB200_ERR_ARG;
    int *status = vb::device_status_ptr();
    if (!status) return vb::cuda_fail(cudaGetLastError(), "device_status_ptr");
    vb::DevBuf out;
    int rc = out.alloc(3 * sizeof(int));
    if (rc) return rc;
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    VB_CUDA(cudaMemsetAsync(out.p, 0xff, 3 * sizeof(int), cs));
    vb::bounded_wait_selftest_kernel<<<1, 64, 0, cs>>>(status, (long long)budget_cycles, out.as<int>());
    VB_CUDA(cudaGetLastError());
    int h[3] = {-1, -1, -1};
    VB_CUDA(cudaMemcpyAsync(h, out.p, sizeof h, cudaMemcpyDeviceToHost, cs));
    VB_CUDA(cudaStreamSynchronize(cs));
    *gave_up = (h[0] == 1 && h[1] == 1 && h[2] == 1) ? 1 : 0;
    return VLAB200_OK;
}

const char *vlab200_last_error(void) { return vb::g_last_error; }

int32_t vlab200_abi_version(void) { return VLAB200_ABI_VERSION; }

int32_t vlab200_device_status(int32_t *out, int32_t reset) {
    if (!out) return VLAB200_ERR_ARG;
    int *p = vb::device_status_ptr();
    if (!p) return vb::cuda_fail(cudaGetLastError(), "device_status_ptr");
    VB_CUDA(cudaDeviceSynchronize());
    int v = 0;
    VB_CUDA(cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost));
    *out = v;
    if (reset && v != 0) VB_CUDA(cudaMemset(p, 0, sizeof(int)));
    return VLAB200_OK;
}

}  // extern "C"
