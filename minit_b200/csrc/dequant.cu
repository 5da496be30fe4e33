// Standalone GPTQ dequantisation: packed int4/int8 -> W[K,N] in fp16/bf16, bit-exact with
// the reference formula (minit/quantize/dispatch.py:14-20):
//     W = (T(q) - (T(z) + 1)) * s        evaluated in T
// q, z+1 and their difference are small integers, exactly representable in T, so the only
// rounding is the final multiply.  (q - z - 1) * s is computed here in fp32, where the
// product of a <=9-bit integer and an 11-bit (8-bit for bf16) significand is exact, and is
// then rounded once to T with round-to-nearest-even -- the same value the T multiply gives.
//
// HBM-bound: 2 bytes written per weight.  One thread expands one 128-bit load (4 adjacent
// columns x `pack` k-values) and stores `pack` rows of 8 bytes; a warp writes 256 contiguous
// bytes per row.
#include "common.cuh"

namespace mt {

template <int BITS, typename T>
__global__ void __launch_bounds__(256)
dequant_kernel(const uint32_t* __restrict__ qweight, const int32_t* __restrict__ g_idx,
               const uint32_t* __restrict__ qzeros, const T* __restrict__ scales,
               T* __restrict__ w_out, int n, int k, int groups) {
    constexpr int PACK = 32 / BITS;
    constexpr uint32_t MASK = (1u << BITS) - 1u;
    const int n4 = n >> 2;                       // uint4 units per packed row
    const int kp = k / PACK;
    const int gs = k / groups;
    const long long total = (long long)kp * n4;
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const int pr = int(idx / n4);
        const int c = int(idx - (long long)pr * n4) << 2;   // first of 4 columns
        const uint4 wv = ldg_stream(qweight + (size_t)pr * n + c);
        const uint32_t w[4] = {wv.x, wv.y, wv.z, wv.w};
        int g_prev = -1;
        float s[4] = {0.f, 0.f, 0.f, 0.f};
        int zp1[4] = {0, 0, 0, 0};
#pragma unroll
        for (int j = 0; j < PACK; ++j) {
            const int kk = pr * PACK + j;
            const int g = g_idx ? min(max(__ldg(g_idx + kk), 0), groups - 1) : kk / gs;
            if (g != g_prev) {
                g_prev = g;
                const uint2 sv = __ldg(reinterpret_cast<const uint2*>(scales + (size_t)g * n + c));
                s[0] = F16x2<T>::to_float(uint16_t(sv.x & 0xffff));
                s[1] = F16x2<T>::to_float(uint16_t(sv.x >> 16));
                s[2] = F16x2<T>::to_float(uint16_t(sv.y & 0xffff));
                s[3] = F16x2<T>::to_float(uint16_t(sv.y >> 16));
                if (qzeros) {
                    const uint32_t zw = __ldg(qzeros + (size_t)g * (n / PACK) + c / PACK) >> ((c % PACK) * BITS);
#pragma unroll
                    for (int i = 0; i < 4; ++i) zp1[i] = int((zw >> (i * BITS)) & MASK) + 1;
                } else {
#pragma unroll
                    for (int i = 0; i < 4; ++i) zp1[i] = 1 << (BITS - 1);
                }
            }
            float v[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) v[i] = float(int((w[i] >> (j * BITS)) & MASK) - zp1[i]) * s[i];
            uint2 o;
            o.x = F16x2<T>::pack(v[0], v[1]);
            o.y = F16x2<T>::pack(v[2], v[3]);
            *reinterpret_cast<uint2*>(w_out + (size_t)kk * n + c) = o;
        }
    }
}

// One element per byte -> W.  Serves QuantizedTensor.dequantize() when the caller holds the
// unpacked tensors the reference's QuantizedTensor is built from (minit/quantize/tensor.py:9-30).
template <typename T>
__global__ void __launch_bounds__(256)
dequant_unpacked_kernel(const uint8_t* __restrict__ q, const int32_t* __restrict__ g_idx, const uint8_t* __restrict__ z,
                        const T* __restrict__ scales, T* __restrict__ w_out, int n, int k, int groups) {
    const int gs = k / groups;
    const long long total = (long long)k * (n >> 2);
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const int kk = int(idx / (n >> 2));
        const int c = int(idx - (long long)kk * (n >> 2)) << 2;
        const int g = g_idx ? min(max(__ldg(g_idx + kk), 0), groups - 1) : kk / gs;
        const uint32_t qv = __ldg(reinterpret_cast<const uint32_t*>(q + (size_t)kk * n + c));
        const uint32_t zv = __ldg(reinterpret_cast<const uint32_t*>(z + (size_t)g * n + c));
        const uint2 sv = __ldg(reinterpret_cast<const uint2*>(scales + (size_t)g * n + c));
        const uint16_t sh[4] = {uint16_t(sv.x & 0xffff), uint16_t(sv.x >> 16), uint16_t(sv.y & 0xffff), uint16_t(sv.y >> 16)};
        float v[4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
            v[i] = float(int((qv >> (8 * i)) & 0xffu) - int((zv >> (8 * i)) & 0xffu) - 1) * F16x2<T>::to_float(sh[i]);
        uint2 o; o.x = F16x2<T>::pack(v[0], v[1]); o.y = F16x2<T>::pack(v[2], v[3]);
        *reinterpret_cast<uint2*>(w_out + (size_t)kk * n + c) = o;
    }
}

// int32-packed -> one element per byte (the reference's unpack(), examples/qwen1_5_int8.py:40-50,
// generalised to 4-bit with the accessor formula of examples/qwen1_5_int8.py:97-138).
// axis 0: [R/pack, C] -> [R, C];  axis 1: [R, C/pack] -> [R, C].
template <int BITS>
__global__ void __launch_bounds__(256)
unpack_kernel(const uint32_t* __restrict__ packed, uint8_t* __restrict__ out, int rows, int cols, int axis) {
    constexpr int PACK = 32 / BITS;
    constexpr uint32_t MASK = (1u << BITS) - 1u;
    const long long total = (long long)rows * cols;
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const int r = int(idx / cols), c = int(idx - (long long)r * cols);
        uint32_t w; int j;
        if (axis == 0) { w = __ldg(packed + (size_t)(r / PACK) * cols + c); j = r % PACK; }
        else { w = __ldg(packed + (size_t)r * (cols / PACK) + c / PACK); j = c % PACK; }
        out[idx] = uint8_t((w >> (j * BITS)) & MASK);
    }
}

static unsigned grid_for(long long total) {
    long long blocks = (total + 255) / 256;
    const long long cap = 148LL * 32;
    return (unsigned)(blocks > cap ? cap : blocks);
}

int launch_dequant_unpacked(cudaStream_t st, const uint8_t* q, const int32_t* g_idx, const uint8_t* z, const void* scales,
                            void* w_out, int n, int k, int groups, int dtype) {
    const long long total = (long long)k * (n / 4);
    if (total == 0) return MT_OK;
    if (dtype == MT_F16)
        dequant_unpacked_kernel<__half><<<grid_for(total), 256, 0, st>>>(q, g_idx, z, reinterpret_cast<const __half*>(scales),
                                                                          reinterpret_cast<__half*>(w_out), n, k, groups);
    else
        dequant_unpacked_kernel<__nv_bfloat16><<<grid_for(total), 256, 0, st>>>(q, g_idx, z, reinterpret_cast<const __nv_bfloat16*>(scales),
                                                                                 reinterpret_cast<__nv_bfloat16*>(w_out), n, k, groups);
    return cudaGetLastError() == cudaSuccess ? MT_OK : MT_ERR_CUDA;
}

int launch_unpack(cudaStream_t st, const uint32_t* packed, uint8_t* out, int rows, int cols, int bits, int axis) {
    const long long total = (long long)rows * cols;
    if (total == 0) return MT_OK;
    if (bits == 4) unpack_kernel<4><<<grid_for(total), 256, 0, st>>>(packed, out, rows, cols, axis);
    else unpack_kernel<8><<<grid_for(total), 256, 0, st>>>(packed, out, rows, cols, axis);
    return cudaGetLastError() == cudaSuccess ? MT_OK : MT_ERR_CUDA;
}

int launch_dequant(cudaStream_t st, const uint32_t* qweight, const int32_t* g_idx, const uint32_t* qzeros,
                   const void* scales, void* w_out, int n, int k, int groups, int bits, int dtype) {
    const int pack = 32 / bits;
    const long long total = (long long)(k / pack) * (n / 4);
    if (total == 0) return MT_OK;
    long long blocks = (total + 255) / 256;
    const long long cap = 148LL * 32;
    if (blocks > cap) blocks = cap;
#define MT_DQ(B, TT) dequant_kernel<B, TT><<<(unsigned)blocks, 256, 0, st>>>(qweight, g_idx, qzeros, \
        reinterpret_cast<const TT*>(scales), reinterpret_cast<TT*>(w_out), n, k, groups)
    if (bits == 4) { if (dtype == MT_F16) MT_DQ(4, __half); else MT_DQ(4, __nv_bfloat16); }
    else           { if (dtype == MT_F16) MT_DQ(8, __half); else MT_DQ(8, __nv_bfloat16); }
#undef MT_DQ
    return cudaGetLastError() == cudaSuccess ? MT_OK : MT_ERR_CUDA;
}

}  // namespace mt
