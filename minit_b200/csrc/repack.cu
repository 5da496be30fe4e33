// Load-time layout transforms (run once per checkpoint, not on the decode path):
//
//  * w8_pack: plain int8 weights [K,N] -> the 8-bit GPTQ word layout [K/4, N] (byte i of word
//    (kw, n) = w[4 kw + i][n] + 128), so that a per-channel int8 linear runs on the same kernels
//    as a GPTQ int8 linear with one group, stored zero 127 (minit/quantize/dispatch.py:14-20 with
//    G = 1) and scales [1,N].
//  * act-order: a GPTQ checkpoint quantized with desc_act stores g_idx[k] = group of row k in
//    arbitrary order (examples/qwen1_5_int8.py:97-138 indexes scales and zeros through it for
//    every element).  Sorting the rows by group once (stable) turns it into the contiguous-group
//    layout all fast kernels assume; the activations are then read through the same permutation:
//    x[:, perm] @ W[perm, :] == x @ W.
#include "common.cuh"

namespace mt {
namespace {

// one thread: 4 columns x 4 rows -> 4 words
__global__ void w8_pack_kernel(const int8_t* __restrict__ w, uint32_t* __restrict__ out, int n, int k) {
    const long long total = (long long)(k / 4) * (n / 4);
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int c4 = int(i % (n / 4)), kw = int(i / (n / 4));
        uint32_t r[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) r[j] = __ldg(reinterpret_cast<const uint32_t*>(w + (size_t)(4 * kw + j) * n + 4 * c4)) ^ 0x80808080u;
        uint4 o;   // column c: byte c of each row
        const uint32_t t01 = prmt(r[0], r[1], 0x5140), t23 = prmt(r[2], r[3], 0x5140);   // (r0.b0, r1.b0, r0.b1, r1.b1)
        const uint32_t u01 = prmt(r[0], r[1], 0x7362), u23 = prmt(r[2], r[3], 0x7362);   // (r0.b2, r1.b2, r0.b3, r1.b3)
        o.x = prmt(t01, t23, 0x5410); o.y = prmt(t01, t23, 0x7632);
        o.z = prmt(u01, u23, 0x5410); o.w = prmt(u01, u23, 0x7632);
        *reinterpret_cast<uint4*>(out + (size_t)kw * n + 4 * c4) = o;
    }
}

// Stable sort of the rows by group, one CTA: thread g collects the rows of group g in order.
// status: 0 ok, 1 a group does not hold exactly k / groups rows, 2 a g_idx value is out of range.
__global__ void act_order_perm_kernel(const int32_t* __restrict__ g_idx, int32_t* __restrict__ perm, int* __restrict__ status,
                                      int k, int groups) {
    const int gs = k / groups;
    __shared__ int bad;
    if (threadIdx.x == 0) bad = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < k; i += blockDim.x) {
        const int g = g_idx[i];
        if (g < 0 || g >= groups) bad = 2;
    }
    __syncthreads();
    if (bad == 0) {
        for (int g = threadIdx.x; g < groups; g += blockDim.x) {
            int cnt = 0;
            for (int i = 0; i < k; ++i) {
                if (g_idx[i] == g) {
                    if (cnt < gs) perm[(size_t)g * gs + cnt] = i;
                    ++cnt;
                }
            }
            if (cnt != gs) bad = 1;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0 && status) *status = bad;
}

// out row r = in row perm[r], element-wise inside the packed words; one thread: one output word
template <int BITS>
__global__ void repack_rows_kernel(const uint32_t* __restrict__ qw, const int32_t* __restrict__ perm,
                                   uint32_t* __restrict__ out, int n, int k) {
    constexpr int PACK = 32 / BITS;
    constexpr uint32_t MASK = (1u << BITS) - 1u;
    const long long total = (long long)(k / PACK) * n;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int col = int(i % n), kw = int(i / n);
        uint32_t word = 0;
#pragma unroll
        for (int j = 0; j < PACK; ++j) {
            int src = perm[kw * PACK + j];
            src = src < 0 ? 0 : (src >= k ? k - 1 : src);
            const uint32_t v = (__ldg(qw + (size_t)(src / PACK) * n + col) >> (BITS * (src % PACK))) & MASK;
            word |= v << (BITS * j);
        }
        out[i] = word;
    }
}

// x_out[m, j] = x[m, perm[j]], 16-bit elements
__global__ void gather_columns_kernel(const uint16_t* __restrict__ x, const int32_t* __restrict__ perm,
                                      uint16_t* __restrict__ out, int m, int k) {
    const long long total = (long long)m * k;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int j = int(i % k), row = int(i / k);
        int src = perm[j];
        src = src < 0 ? 0 : (src >= k ? k - 1 : src);
        out[i] = x[(size_t)row * k + src];
    }
}

inline unsigned blocks_for(long long total) {
    long long b = (total + 255) / 256;
    const long long cap = 148LL * 16;
    return (unsigned)(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace

int launch_w8_pack(cudaStream_t st, const int8_t* w, uint32_t* out, int n, int k) {
    w8_pack_kernel<<<blocks_for((long long)(k / 4) * (n / 4)), 256, 0, st>>>(w, out, n, k);
    return cudaGetLastError() == cudaSuccess ? MT_OK : MT_ERR_CUDA;
}

int launch_act_order_perm(cudaStream_t st, const int32_t* g_idx, int32_t* perm, int* status, int k, int groups) {
    act_order_perm_kernel<<<1, 1024, 0, st>>>(g_idx, perm, status, k, groups);
    return cudaGetLastError() == cudaSuccess ? MT_OK : MT_ERR_CUDA;
}

int launch_repack_rows(cudaStream_t st, const uint32_t* qw, const int32_t* perm, uint32_t* out, int n, int k, int bits) {
    const long long total = (long long)(k / (32 / bits)) * n;
    if (bits == 4) repack_rows_kernel<4><<<blocks_for(total), 256, 0, st>>>(qw, perm, out, n, k);
    else repack_rows_kernel<8><<<blocks_for(total), 256, 0, st>>>(qw, perm, out, n, k);
    return cudaGetLastError() == cudaSuccess ? MT_OK : MT_ERR_CUDA;
}

int launch_gather_columns(cudaStream_t st, const void* x, const int32_t* perm, void* out, int m, int k) {
    gather_columns_kernel<<<blocks_for((long long)m * k), 256, 0, st>>>(static_cast<const uint16_t*>(x), perm, static_cast<uint16_t*>(out), m, k);
    return cudaGetLastError() == cudaSuccess ? MT_OK : MT_ERR_CUDA;
}

}  // namespace mt
