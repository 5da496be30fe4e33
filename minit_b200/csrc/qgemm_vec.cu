// Decode GEMV (M <= 2) on the CUDA cores: out[M,N] = x[M,K] @ dequant(W)[K,N] (+ bias).
//
// At M <= 2 the product is a pure stream of the packed weights (minit/quantize/tensor.py:29-30
// expands them to fp16 first; examples/qwen1_5_int8.py:95-149 fuses that with the product).  The
// legacy mma.sync pipe cannot convert-and-multiply a 7 TB/s stream of 4-bit weights, so this kernel
// spends as few issue slots per packed word as the arithmetic allows:
//
//   * a packed nibble (byte) masked in place IS an fp16 subnormal: (word & 0x000f000f) read as
//     f16x2 is (q_j, q_{j+4}) * 2^-24, (word & 0x00f000f0) is 16 * (q_{j+1}, q_{j+5}) * 2^-24.
//     One AND and one fma.rn.f16x2 per two weights: no integer-to-float conversion, no zero-point
//     subtraction, no scaling in the inner loop.
//   * the activations are staged once per warp in shared memory, block-scaled per chunk of 64 (32)
//     values to [2^14, 2^15) so that the products land in the fp16 normal range, permuted to the
//     nibble pairs above and with the odd positions pre-divided by 16.
//   * every chunk the four f16x2 accumulators of a column are folded in fp32:
//         out += s[g,n] * (2^(24-e) * sum(q x') - (z[g,n]+1) * sum(x))
//     which is the GPTQ formula (q - (z+1)) * s summed over the chunk.  Accumulators see at most
//     8 additions between folds.
//   * a lane owns 4 adjacent columns (one 16-byte load per packed row), a warp a contiguous run of
//     rows, a CTA 8 such runs of one 128-column block; split-K across CTAs ends in the same
//     last-arriver reduction as the streaming kernel.  The weight, scale and zero loads of the
//     prologue do not depend on the previous kernel and are issued before griddepcontrol.wait.
#include "common.cuh"

namespace mt {
namespace {

constexpr int VEC_THREADS = 256;
constexpr int VEC_WARPS = 8;
constexpr int VEC_COLS = 128;   // columns per CTA
constexpr int VEC_D = 8;        // packed rows in flight per thread

struct VecParams {
    const void* x; const uint32_t* qw; const uint32_t* qz; const void* scales; const void* bias; void* out;
    unsigned* counters; float* partial;
    int m, n, k, groups;
    int cpg;          // chunks per group
    int nchunks;      // K / CK
    int units;        // splits * VEC_WARPS warp slices
    int splits;
    int slice_ks;     // k-steps (8 values of k) of shared memory per warp and batch row
    int zp1_const;
    int pdl;
};

__device__ __forceinline__ uint32_t hfma2(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d; asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c)); return d; }
__device__ __forceinline__ uint32_t hmul2(uint32_t a, uint32_t b) {
    uint32_t d; asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d; }
__device__ __forceinline__ uint32_t hadd2(uint32_t a, uint32_t b) {
    uint32_t d; asm("add.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d; }
__device__ __forceinline__ float h2sum(uint32_t h) {
    const __half2 v = *reinterpret_cast<const __half2*>(&h);
    return __low2float(v) + __high2float(v);
}
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi); return *reinterpret_cast<const uint32_t*>(&h); }

// BITS 4 | 8; T the activation / scale type; MB batch rows; CK values of k per fold chunk (64 | 32)
template <int BITS, typename T, int MB, int CK>
__global__ void __launch_bounds__(VEC_THREADS, 2) qgemm_vec_kernel(const VecParams p) {
    using H = F16x2<T>;
    constexpr int PACK = 32 / BITS;
    constexpr int RPK = 8 / PACK;            // packed rows per k-step of 8 values: 1 (int4) or 2 (int8)
    constexpr int CKS = CK / 8;              // k-steps per chunk
    constexpr int KPR = VEC_D / RPK;         // k-steps per trip round the register ring
    constexpr int SRK = CKS > KPR ? CKS : KPR;   // k-steps per unrolled body
    constexpr uint32_t MASK_LO = BITS == 4 ? 0x000f000fu : 0x00ff00ffu;
    constexpr uint32_t MASK_HI = 0x00f000f0u;

    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ __align__(16) float red[VEC_WARPS * MB * VEC_COLS];
    __shared__ int s_last;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tile = blockIdx.x, split = blockIdx.y;
    const int col = tile * VEC_COLS + lane * 4;

    // this warp's run of chunks
    const int u = split * VEC_WARPS + warp;
    const int c_lo = int((long long)u * p.nchunks / p.units);
    const int c_hi = int((long long)(u + 1) * p.nchunks / p.units);
    const int nks = (c_hi - c_lo) * CKS;
    const int nrows = nks * RPK;
    const size_t rstride = size_t(p.n) / 4;     // uint4 per packed row
    const uint4* wp = reinterpret_cast<const uint4*>(p.qw + (size_t)c_lo * CKS * RPK * p.n + col);

    // ---- prologue: everything that does not depend on the previous kernel ----
    uint4 w[VEC_D];
#pragma unroll
    for (int i = 0; i < VEC_D; ++i) w[i] = i < nrows ? ldg_stream(wp + i * rstride) : make_uint4(0, 0, 0, 0);
    const uint4* wnext = wp + VEC_D * rstride;

    // scale / zero words of the current group and of the two after it, raw
    const T* sc = reinterpret_cast<const T*>(p.scales);
    int g = c_lo / p.cpg;
    int left = p.cpg - (c_lo - g * p.cpg);     // chunks left in the current group
    const int zshift = (lane & (PACK / 4 - 1)) * (4 * BITS);   // this lane's 4 zero points inside their packed word
    auto load_s = [&](int gi) -> uint2 {
        gi = gi < p.groups ? gi : p.groups - 1;
        return __ldg(reinterpret_cast<const uint2*>(sc + (size_t)gi * p.n + col));
    };
    auto load_z = [&](int gi) -> uint32_t {
        if (!p.qz) return 0u;
        gi = gi < p.groups ? gi : p.groups - 1;
        return __ldg(p.qz + (size_t)gi * (p.n / PACK) + col / PACK);
    };
    uint2 s0 = load_s(g), s1 = load_s(g + 1), s2 = load_s(g + 2);
    uint32_t z0 = load_z(g), z1 = load_z(g + 1), z2 = load_z(g + 2);

    if (p.pdl) { griddep_launch_dependents(); griddep_wait(); }

    // ---- stage the activations of this warp's run: block-scale, permute, fp16 ----
    unsigned char* xs_base = smem + (size_t)warp * MB * p.slice_ks * 16;
    float2* meta_base = reinterpret_cast<float2*>(smem + (size_t)VEC_WARPS * MB * p.slice_ks * 16) + (size_t)warp * MB * (p.slice_ks / CKS);
    const T* xg = reinterpret_cast<const T*>(p.x);
#pragma unroll
    for (int mb = 0; mb < MB; ++mb) {
        const bool row_ok = mb < p.m;
        for (int i = 0; i < p.slice_ks; i += 32) {
            const int ks = i + lane;
            uint4 raw = make_uint4(0, 0, 0, 0);
            if (row_ok && ks < nks) raw = __ldg(reinterpret_cast<const uint4*>(xg + (size_t)mb * p.k + ((size_t)c_lo * CKS + ks) * 8));
            float f[8];
            const uint32_t rw[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                f[2 * j] = H::to_float(uint16_t(rw[j] & 0xffff));
                f[2 * j + 1] = H::to_float(uint16_t(rw[j] >> 16));
            }
            float amax = 0.f, sum = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) { amax = fmaxf(amax, fabsf(f[j])); sum += f[j]; }
#pragma unroll
            for (int o = 1; o < CKS; o <<= 1) {
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
                sum += __shfl_xor_sync(0xffffffffu, sum, o);
            }
            int e = 0;                                            // x' = x * 2^e has its chunk maximum in [2^14, 2^15)
            if (amax > 0.f && amax < 3.0e38f) e = 14 - (int((__float_as_uint(amax) >> 23) & 0xff) - 127);
            e = e < -100 ? -100 : (e > 100 ? 100 : e);
            const float up = __uint_as_float(uint32_t(127 + e) << 23);
            const float post = __uint_as_float(uint32_t(127 + 24 - e) << 23);
            uint4 o4;
            if constexpr (BITS == 4) {
                const float dn = up * 0.0625f;
                o4.x = pack_h2(f[0] * up, f[4] * up); o4.y = pack_h2(f[1] * dn, f[5] * dn);
                o4.z = pack_h2(f[2] * up, f[6] * up); o4.w = pack_h2(f[3] * dn, f[7] * dn);
            } else {
                o4.x = pack_h2(f[0] * up, f[2] * up); o4.y = pack_h2(f[1] * up, f[3] * up);
                o4.z = pack_h2(f[4] * up, f[6] * up); o4.w = pack_h2(f[5] * up, f[7] * up);
            }
            if (ks < p.slice_ks) {
                *reinterpret_cast<uint4*>(xs_base + ((size_t)mb * p.slice_ks + ks) * 16) = o4;
                if ((ks % CKS) == 0) meta_base[(size_t)mb * (p.slice_ks / CKS) + ks / CKS] = make_float2(post, sum);
            }
        }
    }
    __syncwarp();

    // ---- main loop ----
    float sf[4], zf[4];
    auto convert = [&](uint2 s, uint32_t z) {
        sf[0] = H::to_float(uint16_t(s.x & 0xffff)); sf[1] = H::to_float(uint16_t(s.x >> 16));
        sf[2] = H::to_float(uint16_t(s.y & 0xffff)); sf[3] = H::to_float(uint16_t(s.y >> 16));
        if (p.qz) {
            const uint32_t zz = z >> zshift;
#pragma unroll
            for (int c = 0; c < 4; ++c) zf[c] = float(int((zz >> (BITS * c)) & ((1u << BITS) - 1u)) + 1);
        } else {
#pragma unroll
            for (int c = 0; c < 4; ++c) zf[c] = float(p.zp1_const);
        }
    };
    convert(s0, z0);

    float acc[MB][4];
#pragma unroll
    for (int mb = 0; mb < MB; ++mb)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[mb][c] = 0.f;
    uint32_t a[MB][4][4];

    int row = 0;   // packed rows consumed
    for (int ks0 = 0; ks0 < nks; ks0 += SRK) {
#pragma unroll
        for (int j = 0; j < SRK; ++j) {
            uint4 xv[MB];
#pragma unroll
            for (int mb = 0; mb < MB; ++mb)
                xv[mb] = *reinterpret_cast<const uint4*>(xs_base + ((size_t)mb * p.slice_ks + ks0 + j) * 16);
            const bool first = (j % CKS) == 0;
#pragma unroll
            for (int rr = 0; rr < RPK; ++rr) {
                constexpr int dummy = 0; (void)dummy;
                const int slot = (j * RPK + rr) % VEC_D;
                const uint4 wv = w[slot];
                w[slot] = (row + VEC_D < nrows) ? ldg_stream(wnext) : make_uint4(0, 0, 0, 0);
                wnext += rstride;
                ++row;
                const uint32_t q4[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const uint32_t q = q4[c], q8 = q >> 8;
#pragma unroll
                    for (int mb = 0; mb < MB; ++mb) {
                        if constexpr (BITS == 4) {
                            const uint32_t w0 = q & MASK_LO, w1 = q & MASK_HI, w2 = q8 & MASK_LO, w3 = q8 & MASK_HI;
                            if (first) {
                                a[mb][c][0] = hmul2(w0, xv[mb].x); a[mb][c][1] = hmul2(w1, xv[mb].y);
                                a[mb][c][2] = hmul2(w2, xv[mb].z); a[mb][c][3] = hmul2(w3, xv[mb].w);
                            } else {
                                a[mb][c][0] = hfma2(w0, xv[mb].x, a[mb][c][0]); a[mb][c][1] = hfma2(w1, xv[mb].y, a[mb][c][1]);
                                a[mb][c][2] = hfma2(w2, xv[mb].z, a[mb][c][2]); a[mb][c][3] = hfma2(w3, xv[mb].w, a[mb][c][3]);
                            }
                        } else {
                            const uint32_t w0 = q & MASK_LO, w1 = q8 & MASK_LO;
                            const uint32_t x0 = rr == 0 ? xv[mb].x : xv[mb].z, x1 = rr == 0 ? xv[mb].y : xv[mb].w;
                            if (first) {
                                a[mb][c][2 * rr] = hmul2(w0, x0); a[mb][c][2 * rr + 1] = hmul2(w1, x1);
                            } else {
                                a[mb][c][2 * rr] = hfma2(w0, x0, a[mb][c][2 * rr]); a[mb][c][2 * rr + 1] = hfma2(w1, x1, a[mb][c][2 * rr + 1]);
                            }
                        }
                    }
                }
            }
            if ((j + 1) % CKS == 0) {
                // fold the chunk that ends here
                const int ci = (ks0 + j) / CKS;
#pragma unroll
                for (int mb = 0; mb < MB; ++mb) {
                    const float2 mt2 = meta_base[(size_t)mb * (p.slice_ks / CKS) + ci];   // (2^(24-e), sum of x)
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const float f = h2sum(hadd2(hadd2(a[mb][c][0], a[mb][c][1]), hadd2(a[mb][c][2], a[mb][c][3])));
                        const float t = fmaf(f, mt2.x, -zf[c] * mt2.y);
                        acc[mb][c] = fmaf(sf[c], t, acc[mb][c]);
                    }
                }
                if (--left == 0) {          // next chunk opens a new group
                    left = p.cpg;
                    ++g;
                    convert(s1, z1);
                    s1 = s2; z1 = z2;
                    s2 = load_s(g + 2); z2 = load_z(g + 2);
                }
            }
        }
    }

    // ---- reduce the 8 warps of the CTA, then the splits ----
#pragma unroll
    for (int mb = 0; mb < MB; ++mb)
        *reinterpret_cast<float4*>(red + ((size_t)warp * MB + mb) * VEC_COLS + lane * 4) = make_float4(acc[mb][0], acc[mb][1], acc[mb][2], acc[mb][3]);
    __syncthreads();
    const int mb_r = tid / VEC_COLS, cc = tid % VEC_COLS;
    const bool active = mb_r < MB && mb_r < p.m;
    float v = 0.f;
    if (active) {
#pragma unroll
        for (int wi = 0; wi < VEC_WARPS; ++wi) v += red[((size_t)wi * MB + mb_r) * VEC_COLS + cc];
    }
    const int gc = tile * VEC_COLS + cc;
    const T* bias = reinterpret_cast<const T*>(p.bias);
    uint16_t* out = reinterpret_cast<uint16_t*>(p.out);
    if (p.splits == 1) {
        if (active) {
            if (bias) v += H::to_float(reinterpret_cast<const uint16_t*>(bias)[gc]);
            out[(size_t)mb_r * p.n + gc] = H::from_float(v);
        }
        return;
    }
    if (active) __stcg(p.partial + ((size_t)split * p.m + mb_r) * p.n + gc, v);
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = (atomicAdd(p.counters + tile, 1u) == unsigned(p.splits - 1));
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (active) {
        float sum = 0.f;
        for (int s = 0; s < p.splits; ++s) sum += __ldcg(p.partial + ((size_t)s * p.m + mb_r) * p.n + gc);
        if (bias) sum += H::to_float(reinterpret_cast<const uint16_t*>(bias)[gc]);
        out[(size_t)mb_r * p.n + gc] = H::from_float(sum);
    }
    if (tid == 0) p.counters[tile] = 0;
}

template <int BITS, typename T, int MB, int CK>
int launch_one(cudaStream_t st, const VecParams& p, dim3 grid, size_t smem) {
    auto kern = qgemm_vec_kernel<BITS, T, MB, CK>;
    if (smem > 48 * 1024) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) { cudaGetLastError(); return MT_ERR_CUDA; }
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = dim3(VEC_THREADS); cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = p.pdl ? 1 : 0;
    if (cudaLaunchKernelEx(&cfg, kern, p) != cudaSuccess) { cudaGetLastError(); return MT_ERR_CUDA; }
    return MT_OK;
}

template <int BITS, typename T>
int launch_mb(cudaStream_t st, const VecParams& p, int ck, dim3 grid, size_t smem) {
    if (p.m == 1) return ck == 64 ? launch_one<BITS, T, 1, 64>(st, p, grid, smem) : launch_one<BITS, T, 1, 32>(st, p, grid, smem);
    return ck == 64 ? launch_one<BITS, T, 2, 64>(st, p, grid, smem) : launch_one<BITS, T, 2, 32>(st, p, grid, smem);
}

}  // namespace

bool vec_supported(const QGemmArgs& a) {
    if (a.g_idx || a.m < 1 || a.m > 2 || a.groups < 1) return false;
    if (a.n % VEC_COLS != 0 || a.k % a.groups != 0) return false;
    const int gs = a.k / a.groups;
    if (gs % 32 != 0) return false;
    if (a.n / VEC_COLS >= kMaxTiles - 1) return false;
    return a.workspace != nullptr && a.workspace_bytes >= kCounterBytes;
}

int launch_vec(cudaStream_t st, const QGemmArgs& a) {
    if (!vec_supported(a)) return MT_ERR_UNSUPPORTED;
    const int gs = a.k / a.groups;
    const int ck = gs % 64 == 0 ? 64 : 32;
    const int cks = ck / 8;
    const int nchunks = a.k / ck;
    const int tiles = a.n / VEC_COLS;
    // split-K: every warp gets at least one chunk and at most 2048 values of k (its activations live
    // in shared memory) and the partial sums must fit the workspace.  Among the admissible factors
    // pick the one a small cost model likes best: 2 CTAs fit an SM; a CTA that shares its SM
    // streams ~23.6 GB/s, one that has the SM to itself ~32 GB/s (its own loads in flight are the
    // limit); a wave costs ~4 us of launch, prologue and reduction, later waves ~1.5 us.
    const int forced = (a.flags >> 16) & 0xff;
    int splits = forced;
    const int min_splits = (a.k + VEC_WARPS * 2048 - 1) / (VEC_WARPS * 2048);
    int max_splits = nchunks / VEC_WARPS;
    if (max_splits < 1) max_splits = 1;
    const size_t cap = (a.workspace_bytes - kCounterBytes) / ((size_t)a.m * a.n * 4);
    if ((size_t)max_splits > cap) max_splits = cap < 1 ? 1 : (int)cap;
    if (max_splits > 64) max_splits = 64;
    if (min_splits > max_splits) return min_splits > 1 && (size_t)min_splits > cap ? MT_ERR_WORKSPACE : MT_ERR_TOO_LARGE;
    if (forced) {
        splits = splits < min_splits ? min_splits : (splits > max_splits ? max_splits : splits);
    } else {
        const double slots = 296.0, sms = 148.0;
        const double total_kb = (double)a.k * VEC_COLS * a.bits / 8.0 / 1024.0;
        double best = 1e30;
        for (int s = min_splits; s <= max_splits; ++s) {
            const double kb = total_kb / s * 1.024;              // KB -> 1e3 bytes: GB/s == KB/us
            const long long ctas = (long long)tiles * s;
            const long long full = ctas / (long long)slots;
            const double rem = double(ctas - full * (long long)slots);
            double t = 0.0;
            if (full > 0) t += 4.0 + kb / 23.6 + double(full - 1) * (1.5 + kb / 23.6);
            if (rem > 0) t += (full > 0 ? 1.5 : 4.0) + kb / (rem <= sms ? 32.0 : 23.6);
            t += 0.02 * s;                                        // more partial sums to write and add
            if (t < best) { best = t; splits = s; }
        }
    }
    VecParams p;
    p.x = a.x; p.qw = a.qweight; p.qz = a.qzeros; p.scales = a.scales; p.bias = a.bias; p.out = a.out;
    p.counters = static_cast<unsigned*>(a.workspace);
    p.partial = reinterpret_cast<float*>(static_cast<char*>(a.workspace) + kCounterBytes);
    p.m = a.m; p.n = a.n; p.k = a.k; p.groups = a.groups;
    p.cpg = gs / ck; p.nchunks = nchunks; p.splits = splits; p.units = splits * VEC_WARPS;
    const int max_chunks = (nchunks + p.units - 1) / p.units;
    int slice_ks = max_chunks * cks;
    slice_ks = (slice_ks + 31) / 32 * 32;      // staging loop works in steps of 32 k-steps; the pad is zero
    p.slice_ks = slice_ks;
    p.zp1_const = 1 << (a.bits - 1);
    p.pdl = (a.flags & MT_FLAG_PDL) ? 1 : 0;
    const int mb = a.m == 1 ? 1 : 2;
    const size_t smem = (size_t)VEC_WARPS * mb * slice_ks * 16 + (size_t)VEC_WARPS * mb * (slice_ks / cks) * 8;
    if (smem > 160 * 1024) return MT_ERR_TOO_LARGE;
    const dim3 grid(tiles, splits);
    if (a.bits == 4) return a.dtype == MT_F16 ? launch_mb<4, __half>(st, p, ck, grid, smem) : launch_mb<4, __nv_bfloat16>(st, p, ck, grid, smem);
    return a.dtype == MT_F16 ? launch_mb<8, __half>(st, p, ck, grid, smem) : launch_mb<8, __nv_bfloat16>(st, p, ck, grid, smem);
}

}  // namespace mt
