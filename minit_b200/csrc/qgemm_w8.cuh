// Streaming int8 weight-only GEMM, one scale per output channel, weights as plain int8 [K,N]
// row-major (M <= 64 per launch).  Same structure as the GPTQ streaming kernel (HBM roofline,
// weights read once with 128-bit loads into a register ring, mma.sync m16n8k16 with the
// weights as the A operand, split-K with last-arriver reduction); what differs is the layout:
// one 128-bit load holds 16 adjacent columns of ONE k, so a thread loads four consecutive
// rows and pairs bytes of rows (k, k+1) and (k+2, k+3) with two PRMTs per column pair.
//
// Arithmetic: w is converted exactly (w + 128 via XOR 0x80, magic-number int->fp16, minus
// 1152), the dot products accumulate x*w in fp32, and the per-channel scale multiplies the
// fp32 sum once in the epilogue:  out = T(scale[n] * sum_k x[k] w[k,n] + bias[n]).
#pragma once
#include "common.cuh"

namespace mt {

struct W8Params {
    const void* x;
    const int8_t* w;
    const void* scales;
    const void* bias;
    void* out;
    float* partial;
    unsigned* counters;
    int m, n, k;
    int nchunks, chunks_per_split, splits;
    int pdl;
};

// CPT = columns per thread (16: uint4 loads, 8: uint2 loads).  A warp covers 8*CPT columns.
template <typename T, int MT, int WN, int CPT>
__global__ void __launch_bounds__(WN * 32)
qgemm_w8_kernel(const W8Params p) {
    using H = F16x2<T>;
    constexpr int U = 8;                 // steps (of 16 k) per staged x chunk
    constexpr int KC = U * 16;           // 128
    constexpr int PITCH = KC * 2 + 32;
    constexpr int R = 2;                 // register ring depth in steps
    constexpr int ROWS = MT * 8;
    constexpr int THREADS = WN * 32;
    constexpr int XUNITS = ROWS * KC / 8;
    constexpr int XPT = (XUNITS + THREADS - 1) / THREADS;
    constexpr int WPR = CPT / 4;         // 32-bit words per row per thread
    constexpr int NTILE = CPT / 2;       // mma tiles (2 columns each) per thread

    extern __shared__ __align__(16) unsigned char smem[];
    unsigned char* xs = smem;            // [2][ROWS][PITCH]
    __shared__ int s_last;

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int tile = blockIdx.x, split = blockIdx.y;
    const int col = tile * (WN * 8 * CPT) + warp * (8 * CPT) + CPT * g;
    const bool col_ok = col < p.n;
    const T* __restrict__ xg = reinterpret_cast<const T*>(p.x);

    const int c_begin = split * p.chunks_per_split;
    const int c_end = min(p.nchunks, c_begin + p.chunks_per_split);
    const int s_begin = c_begin * U, s_end = c_end * U;   // global step range

    float acc[MT][NTILE][4];
#pragma unroll
    for (int j = 0; j < MT; ++j)
#pragma unroll
        for (int i = 0; i < NTILE; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[j][i][e] = 0.f;

    uint32_t ring[R][4][WPR];
    uint4 xreg[XPT];

    auto load_step = [&](int step, int slot) {
        const int k0 = step * 16 + 4 * t;
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int kk = k0 + r;
            if (col_ok && step < s_end && kk < p.k) {
                const int8_t* src = p.w + (size_t)kk * p.n + col;
                if constexpr (CPT == 16) {
                    const uint4 v = ldg_stream(src);
                    ring[slot][r][0] = v.x; ring[slot][r][1] = v.y; ring[slot][r][2] = v.z; ring[slot][r][3] = v.w;
                } else {
                    const uint2 v = ldg_stream8(src);
                    ring[slot][r][0] = v.x; ring[slot][r][1] = v.y;
                }
            } else {
#pragma unroll
                for (int q = 0; q < WPR; ++q) ring[slot][r][q] = 0u;   // w = 0
            }
        }
    };
    auto load_x = [&](int chunk) {
#pragma unroll
        for (int i = 0; i < XPT; ++i) {
            const int unit = tid + i * THREADS;
            const int r = unit / (KC / 8), u8 = unit % (KC / 8);
            const int kk = chunk * KC + u8 * 8;
            if (unit < XUNITS && r < p.m && kk < p.k)
                xreg[i] = __ldg(reinterpret_cast<const uint4*>(xg + (size_t)r * p.k + kk));
            else xreg[i] = make_uint4(0, 0, 0, 0);
        }
    };
    auto store_x = [&](int buf) {
        unsigned char* dst = xs + buf * ROWS * PITCH;
#pragma unroll
        for (int i = 0; i < XPT; ++i) {
            const int unit = tid + i * THREADS;
            if (unit < XUNITS) {
                const int r = unit / (KC / 8), u8 = unit % (KC / 8);
                *reinterpret_cast<uint4*>(dst + r * PITCH + u8 * 16) = xreg[i];
            }
        }
    };

    // prologue (independent of the previous kernel): fill the weight ring
#pragma unroll
    for (int s = 0; s < R; ++s) load_step(s_begin + s, s);
    if (p.pdl) griddep_wait();
    if (c_begin < c_end) load_x(c_begin);

    for (int c = c_begin; c < c_end; ++c) {
        const int buf = (c - c_begin) & 1;
        store_x(buf);
        if (c + 1 < c_end) load_x(c + 1);
        __syncthreads();
        const unsigned char* xb = xs + buf * ROWS * PITCH;
#pragma unroll
        for (int u = 0; u < U; ++u) {
            constexpr uint32_t MAGIC = 0x64646464u;
            uint32_t rows[4][WPR];
#pragma unroll
            for (int r = 0; r < 4; ++r)
#pragma unroll
                for (int q = 0; q < WPR; ++q) rows[r][q] = ring[u % R][r][q] ^ 0x80808080u;   // w + 128, unsigned
            load_step(c * U + u + R, u % R);
            // a[i][0] = column i, (k0,k1);  a[i][1] = column i, (k2,k3)
            uint32_t a[CPT][2];
#pragma unroll
            for (int q = 0; q < WPR; ++q) {
                const uint32_t t01 = prmt(rows[0][q], rows[1][q], 0x5140u);   // (r0.b0, r1.b0, r0.b1, r1.b1)
                const uint32_t t23 = prmt(rows[2][q], rows[3][q], 0x5140u);
                const uint32_t u01 = prmt(rows[0][q], rows[1][q], 0x7362u);   // (r0.b2, r1.b2, r0.b3, r1.b3)
                const uint32_t u23 = prmt(rows[2][q], rows[3][q], 0x7362u);
                if constexpr (!H::kIsBf16) {
                    const uint32_t off = 0x64806480u;                          // 1024 + 128
                    a[4 * q + 0][0] = H::sub(prmt(t01, MAGIC, 0x4140u), off);
                    a[4 * q + 0][1] = H::sub(prmt(t23, MAGIC, 0x4140u), off);
                    a[4 * q + 1][0] = H::sub(prmt(t01, MAGIC, 0x4342u), off);
                    a[4 * q + 1][1] = H::sub(prmt(t23, MAGIC, 0x4342u), off);
                    a[4 * q + 2][0] = H::sub(prmt(u01, MAGIC, 0x4140u), off);
                    a[4 * q + 2][1] = H::sub(prmt(u23, MAGIC, 0x4140u), off);
                    a[4 * q + 3][0] = H::sub(prmt(u01, MAGIC, 0x4342u), off);
                    a[4 * q + 3][1] = H::sub(prmt(u23, MAGIC, 0x4342u), off);
                } else {
                    const float off = 8388608.f + 128.f;
                    auto cv = [&](uint32_t v, uint32_t sel_lo, uint32_t sel_hi) {
                        const float lo = __uint_as_float(prmt(v, 0x4B000000u, sel_lo)) - off;
                        const float hi = __uint_as_float(prmt(v, 0x4B000000u, sel_hi)) - off;
                        return H::pack(lo, hi);
                    };
                    a[4 * q + 0][0] = cv(t01, 0x7540u, 0x7541u); a[4 * q + 0][1] = cv(t23, 0x7540u, 0x7541u);
                    a[4 * q + 1][0] = cv(t01, 0x7542u, 0x7543u); a[4 * q + 1][1] = cv(t23, 0x7542u, 0x7543u);
                    a[4 * q + 2][0] = cv(u01, 0x7540u, 0x7541u); a[4 * q + 2][1] = cv(u23, 0x7540u, 0x7541u);
                    a[4 * q + 3][0] = cv(u01, 0x7542u, 0x7543u); a[4 * q + 3][1] = cv(u23, 0x7542u, 0x7543u);
                }
            }
#pragma unroll
            for (int j = 0; j < MT; ++j) {
                const uint2 b = *reinterpret_cast<const uint2*>(xb + (8 * j + g) * PITCH + (4 * u + t) * 8);
#pragma unroll
                for (int i = 0; i < NTILE; ++i)
                    mma16816<T>(acc[j][i], a[2 * i][0], a[2 * i + 1][0], a[2 * i][1], a[2 * i + 1][1], b.x, b.y);
            }
        }
    }
    if (p.pdl) griddep_launch_dependents();

    // epilogue.  acc[j][i][e]: batch row 8j + 2t + (e&1), column col + 2i + (e>>1)
    const T* __restrict__ sc = reinterpret_cast<const T*>(p.scales);
    const T* __restrict__ bias = reinterpret_cast<const T*>(p.bias);
    T* __restrict__ out = reinterpret_cast<T*>(p.out);
    auto finish = [&](int row, const float (&v)[CPT]) {
        uint32_t o[CPT / 2];
#pragma unroll
        for (int q = 0; q < CPT / 2; ++q) {
            const uint32_t sv = __ldg(reinterpret_cast<const uint32_t*>(sc + col) + q);
            float lo = v[2 * q] * H::to_float(uint16_t(sv & 0xffff));
            float hi = v[2 * q + 1] * H::to_float(uint16_t(sv >> 16));
            if (bias) {
                const uint32_t bv = __ldg(reinterpret_cast<const uint32_t*>(bias + col) + q);
                lo += H::to_float(uint16_t(bv & 0xffff)); hi += H::to_float(uint16_t(bv >> 16));
            }
            o[q] = H::pack(lo, hi);
        }
        uint32_t* dst = reinterpret_cast<uint32_t*>(out + (size_t)row * p.n + col);
#pragma unroll
        for (int q = 0; q < CPT / 8; ++q)
            *reinterpret_cast<uint4*>(dst + 4 * q) = make_uint4(o[4 * q], o[4 * q + 1], o[4 * q + 2], o[4 * q + 3]);
    };
    auto gather = [&](int j, int h, float (&v)[CPT]) {
#pragma unroll
        for (int i = 0; i < NTILE; ++i) { v[2 * i] = acc[j][i][h]; v[2 * i + 1] = acc[j][i][2 + h]; }
    };
    if (p.splits == 1) {
        if (col_ok) {
#pragma unroll
            for (int j = 0; j < MT; ++j)
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int row = 8 * j + 2 * t + h;
                    if (row < p.m) { float v[CPT]; gather(j, h, v); finish(row, v); }
                }
        }
        return;
    }
    if (col_ok) {
#pragma unroll
        for (int j = 0; j < MT; ++j)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int row = 8 * j + 2 * t + h;
                if (row < p.m) {
                    float v[CPT]; gather(j, h, v);
                    float4* dst = reinterpret_cast<float4*>(p.partial + ((size_t)split * p.m + row) * p.n + col);
#pragma unroll
                    for (int q = 0; q < CPT / 4; ++q) __stcg(dst + q, make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]));
                }
            }
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = (atomicAdd(p.counters + tile, 1u) == unsigned(p.splits - 1));
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (col_ok) {
#pragma unroll
        for (int j = 0; j < MT; ++j)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int row = 8 * j + 2 * t + h;
                if (row < p.m) {
                    float v[CPT];
#pragma unroll
                    for (int q = 0; q < CPT; ++q) v[q] = 0.f;
                    for (int s = 0; s < p.splits; ++s) {
                        const float* src = p.partial + ((size_t)s * p.m + row) * p.n + col;
#pragma unroll
                        for (int q = 0; q < CPT / 4; ++q) {
                            const float4 pv = ldcg_f4(src + 4 * q);
                            v[4 * q] += pv.x; v[4 * q + 1] += pv.y; v[4 * q + 2] += pv.z; v[4 * q + 3] += pv.w;
                        }
                    }
                    finish(row, v);
                }
            }
    }
    if (tid == 0) p.counters[tile] = 0;
}

}  // namespace mt
