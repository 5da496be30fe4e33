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
//  * gate / up interleave: the two input projections of a gated feed-forward
//    (examples/llama3_70b.py:118-130: down(silu(gate(x)) * up(x))) become one linear of 2 I columns in
//    which every block of eight columns holds four gate columns and the four up columns of the same
//    indices, so that the thread (or neighbouring lane) that finishes a gate value also holds its up
//    value and the activation runs in the GEMM epilogue.
// Also the two stand-alone elementwise kernels (activation on the interleaved layout, residual add)
// that serve the fused entry point on batch sizes whose GEMM kernels have no such epilogue.
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

// Gate / up interleave, columns: out[r, c] for c in [0, 2 * half) takes gate column 4 * (c / 8) + c % 8 when
// c % 8 < 4, else up column 4 * (c / 8) + c % 8 - 4: each block of eight output columns holds four gate
// columns followed by the four up columns of the same indices.
template <typename E>
__global__ void interleave_cols_kernel(const E* __restrict__ a, const E* __restrict__ b, E* __restrict__ out, int rows, int half) {
    const long long total = (long long)rows * half * 2;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int c = int(i % (2 * half)); const long long r = i / (2 * half);
        const int w = c & 7, src = (c >> 3) * 4 + (w & 3);
        out[i] = (w < 4 ? a : b)[r * half + src];
    }
}

// The same interleave for packed zero points [G, half / pack] -> [G, 2 * half / pack].
template <int BITS>
__global__ void interleave_zeros_kernel(const uint32_t* __restrict__ za, const uint32_t* __restrict__ zb, uint32_t* __restrict__ out,
                                        int groups, int half) {
    constexpr int PACK = 32 / BITS;
    const int wout = 2 * half / PACK, win = half / PACK;
    const long long total = (long long)groups * wout;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int wj = int(i % wout); const long long g = i / wout;
        uint32_t v;
        if constexpr (BITS == 4) {       // output word = 4 gate nibbles, 4 up nibbles: half of an input word each
            const int sh = 16 * (wj & 1);
            v = ((za[g * win + (wj >> 1)] >> sh) & 0xffffu) | (((zb[g * win + (wj >> 1)] >> sh) & 0xffffu) << 16);
        } else {                         // output words alternate: 4 gate bytes, 4 up bytes
            v = (wj & 1) ? zb[g * win + (wj >> 1)] : za[g * win + (wj >> 1)];
        }
        out[i] = v;
    }
}

// out[m, 4b + j] = silu(in[m, 8b + j]) * in[m, 8b + 4 + j]: the activation of a gated feed-forward on the
// interleaved gate / up layout, one rounding.
template <typename T>
__global__ void swiglu_interleaved_kernel(const uint4* __restrict__ in, uint2* __restrict__ out, long long blocks8) {
    using H = F16x2<T>;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < blocks8; i += (long long)gridDim.x * blockDim.x) {
        const uint4 v = in[i];
        uint2 o;
        o.x = H::pack(silu_mul(H::to_float(uint16_t(v.x & 0xffff)), H::to_float(uint16_t(v.z & 0xffff))),
                      silu_mul(H::to_float(uint16_t(v.x >> 16)), H::to_float(uint16_t(v.z >> 16))));
        o.y = H::pack(silu_mul(H::to_float(uint16_t(v.y & 0xffff)), H::to_float(uint16_t(v.w & 0xffff))),
                      silu_mul(H::to_float(uint16_t(v.y >> 16)), H::to_float(uint16_t(v.w >> 16))));
        out[i] = o;
    }
}

// io[i] = T(float(io[i]) + float(res[i])), eight elements per thread
template <typename T>
__global__ void add_residual_kernel(uint4* __restrict__ io, const uint4* __restrict__ res, long long vecs) {
    using H = F16x2<T>;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < vecs; i += (long long)gridDim.x * blockDim.x) {
        uint4 a = io[i]; const uint4 b = res[i];
        uint32_t* pa = reinterpret_cast<uint32_t*>(&a); const uint32_t* pb = reinterpret_cast<const uint32_t*>(&b);
#pragma unroll
        for (int q = 0; q < 4; ++q)
            pa[q] = H::pack(H::to_float(uint16_t(pa[q] & 0xffff)) + H::to_float(uint16_t(pb[q] & 0xffff)),
                            H::to_float(uint16_t(pa[q] >> 16)) + H::to_float(uint16_t(pb[q] >> 16)));
        io[i] = a;
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

int launch_interleave_gate_up(cudaStream_t st, const uint32_t* qw_g, const uint32_t* qw_u, const uint32_t* qz_g, const uint32_t* qz_u,
                              const void* s_g, const void* s_u, const void* b_g, const void* b_u,
                              uint32_t* qw_out, uint32_t* qz_out, void* s_out, void* b_out, int half, int k, int groups, int bits) {
    const int pack = 32 / bits;
    interleave_cols_kernel<uint32_t><<<blocks_for((long long)(k / pack) * half * 2), 256, 0, st>>>(qw_g, qw_u, qw_out, k / pack, half);
    interleave_cols_kernel<uint16_t><<<blocks_for((long long)groups * half * 2), 256, 0, st>>>(
        static_cast<const uint16_t*>(s_g), static_cast<const uint16_t*>(s_u), static_cast<uint16_t*>(s_out), groups, half);
    if (qz_out) {
        const long long total = (long long)groups * (2 * half / pack);
        if (bits == 4) interleave_zeros_kernel<4><<<blocks_for(total), 256, 0, st>>>(qz_g, qz_u, qz_out, groups, half);
        else interleave_zeros_kernel<8><<<blocks_for(total), 256, 0, st>>>(qz_g, qz_u, qz_out, groups, half);
    }
    if (b_out)
        interleave_cols_kernel<uint16_t><<<blocks_for((long long)half * 2), 256, 0, st>>>(
            static_cast<const uint16_t*>(b_g), static_cast<const uint16_t*>(b_u), static_cast<uint16_t*>(b_out), 1, half);
    return cudaGetLastError() == cudaSuccess ? MT_OK : MT_ERR_CUDA;
}

int launch_swiglu_interleaved(cudaStream_t st, const void* in, void* out, int m, int n, int dtype) {
    const long long blocks8 = (long long)m * n / 8;
    if (dtype == MT_F16) swiglu_interleaved_kernel<__half><<<blocks_for(blocks8), 256, 0, st>>>(static_cast<const uint4*>(in), static_cast<uint2*>(out), blocks8);
    else swiglu_interleaved_kernel<__nv_bfloat16><<<blocks_for(blocks8), 256, 0, st>>>(static_cast<const uint4*>(in), static_cast<uint2*>(out), blocks8);
    return cudaGetLastError() == cudaSuccess ? MT_OK : MT_ERR_CUDA;
}

int launch_add_residual(cudaStream_t st, void* io, const void* res, int m, int n, int dtype) {
    const long long vecs = (long long)m * n / 8;
    if (dtype == MT_F16) add_residual_kernel<__half><<<blocks_for(vecs), 256, 0, st>>>(static_cast<uint4*>(io), static_cast<const uint4*>(res), vecs);
    else add_residual_kernel<__nv_bfloat16><<<blocks_for(vecs), 256, 0, st>>>(static_cast<uint4*>(io), static_cast<const uint4*>(res), vecs);
    return cudaGetLastError() == cudaSuccess ? MT_OK : MT_ERR_CUDA;
}

}  // namespace mt
