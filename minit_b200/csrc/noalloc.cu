// mt_qgemm_static: the streaming quantized GEMM for callers that cannot hand us a workspace.
//
// Who needs this: a host program that reserves all of the GPU's memory for its own pool at
// start-up (an inference server with a fixed memory plan, a plugin sandbox) leaves nothing
// for a later cudaMalloc, and a latency-critical decode loop cannot afford the implicit
// device synchronisation cudaMalloc/cudaFree bring with them.  Such a caller can still own
// x, the weights and out (they come from its pool) but has no way to size and allocate the
// split-K scratch mt_qgemm asks for.  Here that scratch is a fixed array inside this library:
// every GPU on which the module of this file is loaded carries MT_STATIC_SCRATCH_BYTES of it
// until the process exits.  The driver loads that module at library load under
// CUDA_MODULE_LOADING=EAGER and, with the default lazy loading, at the first call of this
// entry point on the device (the symbol look-up below): that first call is the one that
// reserves the bytes, so it belongs at start-up, before the host's pool takes what is left.
//
// How the array is addressed: in host code the name `g_static_scratch` is only the host-side
// handle of the device symbol, not a device address.  The device address is obtained once
// per device with cudaGetSymbolAddress (with that device current) and that pointer is what
// the kernels receive.
#include <mutex>
#include "common.cuh"

namespace mt {

static __device__ __align__(256) unsigned char g_static_scratch[MT_STATIC_SCRATCH_BYTES];

static std::mutex g_setup_mu;
static void* g_scratch_ptr[64] = {nullptr};   // device address of the array, per device ordinal

// Set-up, once per device, with that device current.  Returns the array's device address.
static int static_scratch(void** out) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); return MT_ERR_CUDA; }
    if (dev < 0 || dev >= 64) return MT_ERR_DEVICE;
    std::lock_guard<std::mutex> lk(g_setup_mu);
    if (g_scratch_ptr[dev] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || p == nullptr) {
            cudaGetLastError();
            return MT_ERR_CUDA;
        }
        g_scratch_ptr[dev] = p;
    }
    *out = g_scratch_ptr[dev];
    return MT_OK;
}

}  // namespace mt

using namespace mt;

extern "C" int mt_qgemm_static(void* stream, const void* x, const uint32_t* qweight, const int32_t* g_idx,
                               const uint32_t* qzeros, const void* scales, const void* bias, void* out,
                               int m, int n, int k, int nr_groups, int bits, int dtype, int flags) {
    if (bits != 4 && bits != 8) return MT_ERR_BITS;
    if (dtype != MT_F16 && dtype != MT_BF16) return MT_ERR_DTYPE;
    if (m < 0 || n < 0 || k <= 0 || nr_groups < 1) return MT_ERR_SHAPE;
    if (n % 8 != 0 || k % 32 != 0 || k % nr_groups != 0) return MT_ERR_SHAPE;
    if (!g_idx && (k / nr_groups) % (4 * (32 / bits)) != 0) return MT_ERR_SHAPE;
    if (m == 0 || n == 0) return MT_OK;
    // the fixed array is the limit: anything whose split-K scratch would not fit is refused, not degraded
    if (mt_workspace_bytes(m, n, k, bits) > (size_t)MT_STATIC_SCRATCH_BYTES) return MT_ERR_TOO_LARGE;
    if (!x || !qweight || !scales || !out) return MT_ERR_NULL;
    auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    if (!al(x) || !al(qweight) || !al(scales) || !al(out) || (qzeros && !al(qzeros)) || (bias && !al(bias))) return MT_ERR_ALIGN;
    int major = 0, dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) {
        cudaGetLastError();
        return MT_ERR_CUDA;
    }
    if (major != 10) return MT_ERR_DEVICE;
    void* scratch = nullptr;
    int rc = static_scratch(&scratch);
    if (rc != MT_OK) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // The array keeps whatever the previous call left in it.  The tile counters at its start are
    // the only part that has to begin at zero, so they are cleared here on the caller's stream.
    if (cudaMemsetAsync(scratch, 0, kCounterBytes, st) != cudaSuccess) { cudaGetLastError(); return MT_ERR_CUDA; }
    QGemmArgs a = {};
    a.x = x; a.qweight = qweight; a.g_idx = g_idx; a.qzeros = qzeros; a.scales = scales; a.bias = bias; a.out = out;
    a.m = m; a.n = n; a.k = k; a.groups = nr_groups; a.bits = bits; a.dtype = dtype;
    a.workspace = scratch; a.workspace_bytes = MT_STATIC_SCRATCH_BYTES;
    a.flags = (flags & ~(MT_FLAG_FORCE_TC | MT_FLAG_PDL)) | MT_FLAG_FORCE_SMALL;
    return launch_small(st, a);
}
