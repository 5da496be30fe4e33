// Streaming fused unpack + dequant + GEMM for decode-sized batches (M <= 64 per launch).
//
// Roofline: HBM.  Every packed weight word is read exactly once with a 128-bit load and is
// consumed from registers; nothing but x (tiny) goes through shared memory.
//
// Work decomposition
//   grid  = (N tiles of 32*WN columns) x (split-K slices); one CTA streams its K slice in
//           chunks of KC = 8 steps, a step being 4 packed rows (32 k for int4, 16 k for int8).
//   warp  = 32 columns: lane (g = lane/4, t = lane%4) loads, per step, the uint4 at packed row
//           4*step + t, columns 4g..4g+3.  The 8 g-lanes of one t cover 128 contiguous bytes of a
//           row, so a warp load touches 4 full 128-byte lines and a CTA 4 x (128*WN) bytes.
//   math  = mma.sync m16n8k16 with the weights as the A operand (16 output columns x 16 k)
//           and x^T as B (16 k x 8 batch rows): the batch is padded to 8*MT rows, so M = 1
//           costs one tensor instruction per 256 weights and no CUDA-core FMAs at all.
//           The k-slot order inside one MMA is arbitrary as long as A and B agree; it is
//           chosen so that the cheap nibble pairing (j, j+4) produced by one LOP3 is a legal
//           fragment register: x is staged in shared memory already permuted to match.
//   dequant = exact: magic-number int->fp16/bf16, integer subtraction of (zero+1) in T
//           (exact), one multiply by the scale in T.  The A operand therefore holds exactly
//           the reference's W[k,n] (minit/quantize/dispatch.py:14-20); products accumulate
//           in fp32.
//   split-K = each slice writes an fp32 partial tile to the workspace; the last CTA to
//           arrive at a tile (atomic counter) sums the slices in slice order (deterministic),
//           adds the bias, rounds once to T and resets the counter.  No spin-waits.
#pragma once
#include "common.cuh"
#include "ar_mailbox.cuh"

namespace mt {

struct SmallParams {
    const void* x;
    const uint32_t* qw;
    const int32_t* g_idx;
    const uint32_t* qz;
    const void* scales;
    const void* bias;
    void* out;
    float* partial;        // [splits][M][N]
    unsigned* counters;    // [n_tiles]
    int m, n, k, groups, gs;
    int nchunks, chunks_per_split, splits;
    int zp1_const;         // zero+1 used when qz == nullptr
    int pdl;
    ArParams ar;           // fused one-shot all-reduce over peer memory (ar.world > 1): see ar_mailbox.cuh
};

// ---------------------------------------------------------------------------
// per-(group, 4 columns) constants
// ---------------------------------------------------------------------------
template <int BITS, typename T> struct GroupConst {
    uint32_t s[4];    // scale, duplicated in both halves   (int8+bf16: fp32 bits of the scale)
    uint32_t za[4];   // magic + (zero+1), duplicated       (int8+bf16: fp32 bits of 2^23 + zero + 1)
    uint32_t zb[4];   // int4+fp16 only: -(64 + zero + 1), duplicated
};

template <int BITS, typename T>
__device__ __forceinline__ void make_group_const(GroupConst<BITS, T>& gc, uint2 sraw, uint32_t zbits, bool has_z, int zp1_const) {
    constexpr uint32_t MASK = (1u << BITS) - 1u;
    const uint32_t sv[4] = {sraw.x & 0xffffu, sraw.x >> 16, sraw.y & 0xffffu, sraw.y >> 16};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t zp1 = has_z ? (((zbits >> (i * BITS)) & MASK) + 1u) : uint32_t(zp1_const);
        if constexpr (BITS == 8 && F16x2<T>::kIsBf16) {
            gc.s[i] = sv[i] << 16;                       // bf16 -> fp32 bits
            gc.za[i] = 0x4B000000u + zp1;                // 2^23 + zp1 as fp32 bits (zp1 < 2^23)
        } else {
            gc.s[i] = sv[i] * 0x00010001u;
            const uint32_t magic = F16x2<T>::kIsBf16 ? 0x43004300u : 0x64006400u;   // 128.0 / 1024.0
            gc.za[i] = magic | (zp1 * 0x00010001u);      // exact: zp1 fits below the magic's ulp range
            if constexpr (BITS == 4 && !F16x2<T>::kIsBf16) {
                // -(64 + zp1): 1024 - (1024 + 64 + zp1) in fp16, exact
                gc.zb[i] = F16x2<T>::sub(0x64006400u, 0x64006400u | ((64u + zp1) * 0x00010001u));
            }
        }
    }
}

// Dequantise one packed word (one column, PACK k-values) into MMA-ready registers.
//  int4: f[0]=(k0,k4) f[1]=(k1,k5) f[2]=(k2,k6) f[3]=(k3,k7)      int8: f[0]=(k0,k1) f[1]=(k2,k3)
template <int BITS, typename T>
__device__ __forceinline__ void dequant_word(uint32_t w, const GroupConst<BITS, T>& gc, int i, uint32_t (&f)[BITS == 4 ? 4 : 2]) {
    using H = F16x2<T>;
    if constexpr (BITS == 4) {
        if constexpr (!H::kIsBf16) {
            const uint32_t w8 = w >> 8;
            const uint32_t lo0 = and_or(w, 0x000f000fu, 0x64006400u);     // 1024 + (n0, n4)
            const uint32_t hi0 = and_or(w, 0x00f000f0u, 0x64006400u);     // 1024 + 16*(n1, n5)
            const uint32_t lo1 = and_or(w8, 0x000f000fu, 0x64006400u);    // 1024 + (n2, n6)
            const uint32_t hi1 = and_or(w8, 0x00f000f0u, 0x64006400u);    // 1024 + 16*(n3, n7)
            const uint32_t sixteenth = 0x2c002c00u;                        // 1/16
            f[0] = H::mul(H::sub(lo0, gc.za[i]), gc.s[i]);
            f[1] = H::mul(H::fma(hi0, sixteenth, gc.zb[i]), gc.s[i]);
            f[2] = H::mul(H::sub(lo1, gc.za[i]), gc.s[i]);
            f[3] = H::mul(H::fma(hi1, sixteenth, gc.zb[i]), gc.s[i]);
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t lo = and_or(w >> (4 * j), 0x000f000fu, 0x43004300u);   // 128 + (n_j, n_{j+4})
                f[j] = H::mul(H::sub(lo, gc.za[i]), gc.s[i]);
            }
        }
    } else {
        if constexpr (!H::kIsBf16) {
            const uint32_t p0 = prmt(w, 0x64646464u, 0x4140u);   // 1024 + (b0, b1)
            const uint32_t p1 = prmt(w, 0x64646464u, 0x4342u);   // 1024 + (b2, b3)
            f[0] = H::mul(H::sub(p0, gc.za[i]), gc.s[i]);
            f[1] = H::mul(H::sub(p1, gc.za[i]), gc.s[i]);
        } else {
            // bf16 cannot hold 128 + b exactly for b >= 128: go through fp32 (2^23 + b is exact)
            const float s = __uint_as_float(gc.s[i]);
            const float z = __uint_as_float(gc.za[i]);
            const float v0 = (__uint_as_float(prmt(w, 0x4B000000u, 0x7540u)) - z) * s;
            const float v1 = (__uint_as_float(prmt(w, 0x4B000000u, 0x7541u)) - z) * s;
            const float v2 = (__uint_as_float(prmt(w, 0x4B000000u, 0x7542u)) - z) * s;
            const float v3 = (__uint_as_float(prmt(w, 0x4B000000u, 0x7543u)) - z) * s;
            f[0] = H::pack(v0, v1);
            f[1] = H::pack(v2, v3);
        }
    }
}

// ---------------------------------------------------------------------------
// kernel
// ---------------------------------------------------------------------------
template <int BITS> struct SmallCfg {
    static constexpr int PACK = 32 / BITS;
    static constexpr int U = 8;                        // steps per chunk
    static constexpr int KSTEP = 4 * PACK;             // k per step: 32 / 16
    static constexpr int KC = U * KSTEP;               // k per chunk: 256 / 128
    // row pitch of the staged x chunk, chosen so the fragment loads are bank-conflict free
    static constexpr int PITCH = KC * 2 + (BITS == 4 ? 64 : 32);
};

// GPC = groups per chunk (1, 2, 4 or 8); group size * GPC == KC, or GPC == 1 and group size % KC == 0.
// ACT = per-k group lookup through g_idx (act-order); GPC is ignored then.
template <int BITS, typename T, int MT, int WN, int GPC, bool ACT>
__global__ void __launch_bounds__(WN * 32)
qgemm_small_kernel(const SmallParams p) {
    using Cfg = SmallCfg<BITS>;
    using H = F16x2<T>;
    constexpr int PACK = Cfg::PACK, U = Cfg::U, KSTEP = Cfg::KSTEP, KC = Cfg::KC, PITCH = Cfg::PITCH;
    constexpr int NF = BITS == 4 ? 4 : 2;
    constexpr int ROWS = MT * 8;
    constexpr int THREADS = WN * 32;
    constexpr int XUNITS = ROWS * KC / 8;                 // 16-byte units in one staged x chunk
    constexpr int XPT = (XUNITS + THREADS - 1) / THREADS; // units per thread
    constexpr int SPG = ACT ? 1 : U / GPC;                // steps per group inside a chunk
    constexpr int GPT = (KC + THREADS - 1) / THREADS;     // act-order: group ids each thread stages per chunk

    extern __shared__ __align__(16) unsigned char smem[];
    unsigned char* xs = smem;                              // [2][ROWS][PITCH]
    __shared__ int s_last;

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int tile = blockIdx.x, split = blockIdx.y;
    const int col = tile * (WN * 32) + warp * 32 + 4 * g;     // first of this thread's 4 columns
    const bool col_ok = col < p.n;
    const int kp_total = p.k / PACK;
    const T* __restrict__ xg = reinterpret_cast<const T*>(p.x);
    const T* __restrict__ sg = reinterpret_cast<const T*>(p.scales);

    const int c_begin = split * p.chunks_per_split;
    const int c_end = min(p.nchunks, c_begin + p.chunks_per_split);

    // act-order: (scale, zero+1) panel for this CTA's columns and ALL groups, in shared memory
    //   panel[g][c] = { half2/bf162 (magic + zp1, scale) } as one 32-bit word, 4 columns = 16 bytes
    uint32_t* panel = reinterpret_cast<uint32_t*>(smem + 2 * ROWS * PITCH);
    int* gsm = reinterpret_cast<int*>(panel + (ACT ? p.groups * (WN * 32) : 0));   // [2][KC] group ids of the chunk

    float acc[MT][2][4];
#pragma unroll
    for (int j = 0; j < MT; ++j)
#pragma unroll
        for (int s = 0; s < 2; ++s)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[j][s][e] = 0.f;

    uint4 w[U];              // register ring: w[u] is refilled with the next chunk's step u right after use
    // scales / zeros stream from HBM: fetched two chunks ahead (set A = this chunk, set B = the next)
    uint2 sraw[GPC], sraw_b[GPC];
    uint32_t zraw[GPC], zraw_b[GPC];
    uint4 xreg[XPT];
    int greg[GPT];

    auto load_weight = [&](int chunk, int u) {
        const int pr = chunk * (KC / PACK) + 4 * u + t;
        if (col_ok && pr < kp_total) w[u] = ldg_stream(p.qw + (size_t)pr * p.n + col);
        else w[u] = make_uint4(0, 0, 0, 0);
    };
    auto load_scale = [&](int chunk, int q, uint2 (&sraw)[GPC], uint32_t (&zraw)[GPC]) {
        const int kk = chunk * KC + q * (KC / GPC);
        const int gi = min(kk / p.gs, p.groups - 1);
        if (col_ok && chunk < c_end) {
            sraw[q] = __ldg(reinterpret_cast<const uint2*>(sg + (size_t)gi * p.n + col));
            // raw word: the shift happens when the value is consumed, so nothing waits on this load here
            zraw[q] = p.qz ? __ldg(p.qz + (size_t)gi * (p.n / PACK) + col / PACK) : 0u;
        } else { sraw[q] = make_uint2(0, 0); zraw[q] = 0; }
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
        if constexpr (ACT) {
#pragma unroll
            for (int i = 0; i < GPT; ++i) {   // out-of-range group ids are clamped, never dereferenced
                const int kk = chunk * KC + tid + i * THREADS;
                greg[i] = (tid + i * THREADS < KC && kk < p.k) ? min(max(__ldg(p.g_idx + kk), 0), p.groups - 1) : 0;
            }
        }
    };
    auto store_x = [&](int buf) {
        unsigned char* dst = xs + buf * ROWS * PITCH;
#pragma unroll
        for (int i = 0; i < XPT; ++i) {
            const int unit = tid + i * THREADS;
            if (unit < XUNITS) {
                const int r = unit / (KC / 8), u8 = unit % (KC / 8);
                uint4 v = xreg[i];
                if constexpr (BITS == 4) {   // (h0..h7) -> (h0,h4,h1,h5,h2,h6,h3,h7)
                    uint4 o;
                    o.x = prmt(v.x, v.z, 0x5410u); o.y = prmt(v.x, v.z, 0x7632u);
                    o.z = prmt(v.y, v.w, 0x5410u); o.w = prmt(v.y, v.w, 0x7632u);
                    v = o;
                }
                *reinterpret_cast<uint4*>(dst + r * PITCH + u8 * 16) = v;
            }
        }
        if constexpr (ACT) {
#pragma unroll
            for (int i = 0; i < GPT; ++i)
                if (tid + i * THREADS < KC) gsm[buf * KC + tid + i * THREADS] = greg[i];
        }
    };

    // ---- prologue: everything that does not depend on the previous kernel in the stream ----
    if (c_begin < c_end) {
#pragma unroll
        for (int u = 0; u < U; ++u) load_weight(c_begin, u);
        if constexpr (!ACT) {
#pragma unroll
            for (int q = 0; q < GPC; ++q) { load_scale(c_begin, q, sraw, zraw); load_scale(c_begin + 1, q, sraw_b, zraw_b); }
        }
    }
    if constexpr (ACT) {
        // build the panel: one thread per (group, 4-column unit)
        const int units = p.groups * (WN * 8);
        for (int i = tid; i < units; i += THREADS) {
            const int gi = i / (WN * 8), cu = i % (WN * 8);
            const int c = tile * (WN * 32) + cu * 4;
            uint4 e = make_uint4(0, 0, 0, 0);
            if (c < p.n) {
                const uint2 sv = __ldg(reinterpret_cast<const uint2*>(sg + (size_t)gi * p.n + c));
                const uint32_t zb = p.qz ? (__ldg(p.qz + (size_t)gi * (p.n / PACK) + c / PACK) >> ((c % PACK) * BITS)) : 0u;
                constexpr uint32_t MASK = (1u << BITS) - 1u;
                const uint32_t sv4[4] = {sv.x & 0xffffu, sv.x >> 16, sv.y & 0xffffu, sv.y >> 16};
                uint32_t ev[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const uint32_t zp1 = p.qz ? (((zb >> (q * BITS)) & MASK) + 1u) : uint32_t(p.zp1_const);
                    ev[q] = uint32_t(H::from_float(float(zp1))) | (sv4[q] << 16);   // (zero+1 as T, scale)
                }
                e = make_uint4(ev[0], ev[1], ev[2], ev[3]);
            }
            *reinterpret_cast<uint4*>(panel + (size_t)gi * (WN * 32) + cu * 4) = e;
        }
    }
    if (p.pdl) griddep_wait();
    if (c_begin < c_end) load_x(c_begin);

    // ---- main loop over chunks ----
    for (int c = c_begin; c < c_end; ++c) {
        const int buf = (c - c_begin) & 1;
        const bool more = c + 1 < c_end;
        store_x(buf);
        if (more) load_x(c + 1);
        __syncthreads();   // x(c) visible; every warp is past its reads of the other buffer
        const unsigned char* xb = xs + buf * ROWS * PITCH;
        GroupConst<BITS, T> gc;
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint32_t w4[4] = {w[u].x, w[u].y, w[u].z, w[u].w};
            if (more) load_weight(c + 1, u);
            uint32_t f[4][NF];
            if constexpr (!ACT) {
                if (u % SPG == 0) {
                    make_group_const<BITS, T>(gc, sraw[u / SPG], zraw[u / SPG] >> ((col % PACK) * BITS), p.qz != nullptr, p.zp1_const);
                    load_scale(c + 2, u / SPG, sraw, zraw);   // the slot just consumed takes the chunk after next
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) dequant_word<BITS, T>(w4[i], gc, i, f[i]);
            } else {
                // per-k (scale, zero) lookup: k = chunk*KC + (4u+t)*PACK + j
                const int* gk = gsm + buf * KC + (4 * u + t) * PACK;
                const uint32_t* prow = panel + warp * 32 + 4 * g;
                uint4 e[PACK];
#pragma unroll
                for (int j = 0; j < PACK; ++j) e[j] = *reinterpret_cast<const uint4*>(prow + (size_t)gk[j] * (WN * 32));
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint32_t wi = w4[i];
#pragma unroll
                    for (int q = 0; q < NF; ++q) {
                        // the two k-values sharing fragment register q
                        const int ja = BITS == 4 ? q : 2 * q, jb = BITS == 4 ? q + 4 : 2 * q + 1;
                        const uint32_t ea = (&e[ja].x)[i], eb = (&e[jb].x)[i];
                        const uint32_t zz = prmt(ea, eb, 0x5410u);   // (zp1_a, zp1_b)
                        const uint32_t ss = prmt(ea, eb, 0x7632u);   // (s_a, s_b)
                        uint32_t qv;                                 // (q_a, q_b) as T, exact
                        if constexpr (BITS == 4) {
                            const uint32_t magic = H::kIsBf16 ? 0x43004300u : 0x64006400u;
                            qv = H::sub(and_or(wi >> (4 * q), 0x000f000fu, magic), magic);
                        } else {
                            const uint32_t bl = (wi >> (8 * ja)) & 0xffu, bh = (wi >> (8 * jb)) & 0xffu;
                            qv = H::pack(float(bl), float(bh));
                        }
                        f[i][q] = H::mul(H::sub(qv, zz), ss);
                    }
                }
            }
            // B fragments: batch row 8j+g, k-unit (4u+t) of the chunk
#pragma unroll
            for (int j = 0; j < MT; ++j) {
                const unsigned char* xp = xb + (8 * j + g) * PITCH;
                if constexpr (BITS == 4) {
                    const uint4 b = *reinterpret_cast<const uint4*>(xp + (4 * u + t) * 16);
                    mma16816<T>(acc[j][0], f[0][0], f[1][0], f[0][1], f[1][1], b.x, b.y);
                    mma16816<T>(acc[j][0], f[0][2], f[1][2], f[0][3], f[1][3], b.z, b.w);
                    mma16816<T>(acc[j][1], f[2][0], f[3][0], f[2][1], f[3][1], b.x, b.y);
                    mma16816<T>(acc[j][1], f[2][2], f[3][2], f[2][3], f[3][3], b.z, b.w);
                } else {
                    const uint2 b = *reinterpret_cast<const uint2*>(xp + (4 * u + t) * 8);
                    mma16816<T>(acc[j][0], f[0][0], f[1][0], f[0][1], f[1][1], b.x, b.y);
                    mma16816<T>(acc[j][1], f[2][0], f[3][0], f[2][1], f[3][1], b.x, b.y);
                }
            }
        }
        if constexpr (!ACT) {   // rotate: set B (next chunk) becomes current, the refilled set A waits one more chunk
#pragma unroll
            for (int q = 0; q < GPC; ++q) {
                const uint2 ts = sraw[q]; sraw[q] = sraw_b[q]; sraw_b[q] = ts;
                const uint32_t tz = zraw[q]; zraw[q] = zraw_b[q]; zraw_b[q] = tz;
            }
        }
    }
    if (p.pdl) griddep_launch_dependents();

    // ---- epilogue ----
    // acc[j][s][e]: batch row 8j + 2t + (e&1), column col + 2s + (e>>1)
    //
    // Row-parallel use (p.ar.world > 1): the finished fp32 partials go through the mailbox
    // all-reduce of ar_mailbox.cuh before they are rounded and stored; the exchange of one tile
    // overlaps the other tiles' main loops.
    const T* __restrict__ bias = reinterpret_cast<const T*>(p.bias);
    T* __restrict__ out = reinterpret_cast<T*>(p.out);
    const bool fused_ar = ar_active(p.ar);
    const unsigned epoch = fused_ar ? ar_epoch(p.ar) : 0u;
    auto finish = [&](int row, float v0, float v1, float v2, float v3) {
        if (bias) {
            const uint2 bv = __ldg(reinterpret_cast<const uint2*>(bias + col));
            v0 += H::to_float(uint16_t(bv.x & 0xffff)); v1 += H::to_float(uint16_t(bv.x >> 16));
            v2 += H::to_float(uint16_t(bv.y & 0xffff)); v3 += H::to_float(uint16_t(bv.y >> 16));
        }
        if (fused_ar) {
            const float4 sum = ar_exchange(p.ar, epoch, (size_t)row * p.n + col, make_float4(v0, v1, v2, v3));
            v0 = sum.x; v1 = sum.y; v2 = sum.z; v3 = sum.w;
        }
        uint2 o; o.x = H::pack(v0, v1); o.y = H::pack(v2, v3);
        *reinterpret_cast<uint2*>(out + (size_t)row * p.n + col) = o;
    };
    // Grid-wide bookkeeping of the fused path: the last CTA to leave publishes the epoch for the next call.
    auto leave = [&]() {
        if (!fused_ar) return;
        __syncthreads();
        if (tid == 0) ar_leave(p.ar, epoch, gridDim.x * gridDim.y);
    };
    if (p.splits == 1) {
        if (col_ok) {
#pragma unroll
            for (int j = 0; j < MT; ++j)
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int row = 8 * j + 2 * t + h;
                    if (row < p.m) finish(row, acc[j][0][h], acc[j][0][2 + h], acc[j][1][h], acc[j][1][2 + h]);
                }
        }
        leave();
        return;
    }
    if (col_ok) {
#pragma unroll
        for (int j = 0; j < MT; ++j)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int row = 8 * j + 2 * t + h;
                if (row < p.m)
                    __stcg(reinterpret_cast<float4*>(p.partial + ((size_t)split * p.m + row) * p.n + col),
                           make_float4(acc[j][0][h], acc[j][0][2 + h], acc[j][1][h], acc[j][1][2 + h]));
            }
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = (atomicAdd(p.counters + tile, 1u) == unsigned(p.splits - 1));
    __syncthreads();
    if (!s_last) { leave(); return; }
    __threadfence();
    if (col_ok) {
#pragma unroll
        for (int j = 0; j < MT; ++j)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int row = 8 * j + 2 * t + h;
                if (row < p.m) {
                    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
                    for (int s = 0; s < p.splits; ++s) {
                        const float4 v = ldcg_f4(p.partial + ((size_t)s * p.m + row) * p.n + col);
                        sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
                    }
                    finish(row, sum.x, sum.y, sum.z, sum.w);
                }
            }
    }
    if (tid == 0) p.counters[tile] = 0;
    leave();
}

}  // namespace mt
