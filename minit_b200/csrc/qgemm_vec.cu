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
#include "tma.cuh"

namespace mt {
namespace {

constexpr int VEC_THREADS = 256;
constexpr int VEC_WARPS = 8;
constexpr int VEC_COLS = 128;   // columns per CTA
constexpr int VEC_D = 8;        // packed rows in flight per thread

struct VecParams {
    const void* x; const uint32_t* qw; const uint32_t* qz; const void* scales; const void* bias; void* out;
    const int32_t* xperm;   // act-order: activations are read as x[perm[k]] (null: in order)
    unsigned* counters; float* partial;
    int m, n, k, groups;
    int cpg;          // chunks per group
    int nchunks;      // K / CK
    int units;        // splits * VEC_WARPS warp slices
    int splits;
    int slice_ks;     // k-steps (8 values of k) of shared memory per warp and batch row
    int zp1_const;
    int pdl;
    int cluster;      // the `splits` CTAs of a column block form a thread-block cluster: split-K sums meet in CTA 0's shared memory
    ArParams ar;      // row-parallel use: all-reduce of the finished sums over peer memory (ar_mailbox.cuh)
    const void* residual;   // [M,N] T or null, added to the finished (all-reduced) sum before the one rounding
    int swiglu;       // columns are gate / up interleaved in blocks of 4 + 4: out[M,N/2] = silu(gate) * up
    RopeArgs rope;    // rope.cosv != null: rotary embedding + cache append of a fused q/k/v row instead of the store
};

__device__ __forceinline__ float h2sum(uint32_t h) {
    const __half2 v = *reinterpret_cast<const __half2*>(&h);
    return __low2float(v) + __high2float(v);
}
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi); return *reinterpret_cast<const uint32_t*>(&h); }

// Eight consecutive activations of a row, optionally read through the act-order permutation
// (x[perm[k0 .. k0+7]]): the weights' rows were sorted by group once, the activations follow here.
template <typename T, bool COHERENT = false>
__device__ __forceinline__ uint4 load_x8(const T* __restrict__ xrow, const int32_t* __restrict__ perm, size_t k0, int kmax) {
    if constexpr (COHERENT) {
        // activations written earlier in the SAME launch by other SMs: read through L2, never through the read-only path
        if (!perm) return __ldcg(reinterpret_cast<const uint4*>(xrow + k0));
        int idx[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) idx[i] = min(max(__ldg(perm + k0 + i), 0), kmax);
        const unsigned short* xs = reinterpret_cast<const unsigned short*>(xrow);
        uint4 r;
        r.x = uint32_t(__ldcg(xs + idx[0])) | (uint32_t(__ldcg(xs + idx[1])) << 16);
        r.y = uint32_t(__ldcg(xs + idx[2])) | (uint32_t(__ldcg(xs + idx[3])) << 16);
        r.z = uint32_t(__ldcg(xs + idx[4])) | (uint32_t(__ldcg(xs + idx[5])) << 16);
        r.w = uint32_t(__ldcg(xs + idx[6])) | (uint32_t(__ldcg(xs + idx[7])) << 16);
        return r;
    }
    if (!perm) return __ldg(reinterpret_cast<const uint4*>(xrow + k0));
    int4 i0 = __ldg(reinterpret_cast<const int4*>(perm + k0)), i1 = __ldg(reinterpret_cast<const int4*>(perm + k0 + 4));
    // a permutation entry outside [0, K) is clamped, like every other index this library reads from the caller
    i0.x = min(max(i0.x, 0), kmax); i0.y = min(max(i0.y, 0), kmax); i0.z = min(max(i0.z, 0), kmax); i0.w = min(max(i0.w, 0), kmax);
    i1.x = min(max(i1.x, 0), kmax); i1.y = min(max(i1.y, 0), kmax); i1.z = min(max(i1.z, 0), kmax); i1.w = min(max(i1.w, 0), kmax);
    const unsigned short* xs = reinterpret_cast<const unsigned short*>(xrow);
    uint4 r;
    r.x = uint32_t(__ldg(xs + i0.x)) | (uint32_t(__ldg(xs + i0.y)) << 16);
    r.y = uint32_t(__ldg(xs + i0.z)) | (uint32_t(__ldg(xs + i0.w)) << 16);
    r.z = uint32_t(__ldg(xs + i1.x)) | (uint32_t(__ldg(xs + i1.y)) << 16);
    r.w = uint32_t(__ldg(xs + i1.z)) | (uint32_t(__ldg(xs + i1.w)) << 16);
    return r;
}

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
    __shared__ __align__(16) float xred[8 * MB * VEC_COLS];      // cluster mode: one row of sums per split, in CTA 0 of the cluster
    __shared__ int s_last;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tile = blockIdx.x, split = blockIdx.y;
    if (p.cluster) cluster_arrive_relaxed();                      // phase 0: "this CTA runs, its shared memory exists"
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
            if (row_ok && ks < nks) raw = load_x8(xg + (size_t)mb * p.k, p.xperm, ((size_t)c_lo * CKS + ks) * 8, p.k - 1);
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
    const bool fused_ar = ar_active(p.ar);
    const unsigned epoch = fused_ar ? ar_epoch(p.ar) : 0u;      // after griddepcontrol.wait: the previous call has published its epoch
    if (p.splits > 1 && p.cluster) {
        // split-K inside a cluster: every CTA stores its row into CTA 0's shared memory, one cluster
        // barrier, CTA 0 adds the rows in split order.  No global-memory round trip.
        cluster_wait_acquire();                                  // phase 0 complete: CTA 0 is resident
        if (active) st_cluster_f32(xred + ((size_t)split * MB + mb_r) * VEC_COLS + cc, 0u, v);
        cluster_arrive_release();
        cluster_wait_acquire();
        if (split != 0) {
            if (fused_ar && tid == 0) ar_leave(p.ar, epoch, gridDim.x * gridDim.y);
            return;
        }
        if (active) {
            v = 0.f;
            for (int s = 0; s < p.splits; ++s) v += xred[((size_t)s * MB + mb_r) * VEC_COLS + cc];
        }
    } else if (p.splits > 1) {
        if (active) __stcg(p.partial + ((size_t)split * p.m + mb_r) * p.n + gc, v);
        __threadfence();
        __syncthreads();
        if (tid == 0) s_last = (atomicAdd(p.counters + tile, 1u) == unsigned(p.splits - 1));
        __syncthreads();
        if (!s_last) {
            if (fused_ar && tid == 0) ar_leave(p.ar, epoch, gridDim.x * gridDim.y);
            return;
        }
        __threadfence();
        if (active) {
            v = 0.f;
            for (int s = 0; s < p.splits; ++s) v += __ldcg(p.partial + ((size_t)s * p.m + mb_r) * p.n + gc);
        }
        if (tid == 0) p.counters[tile] = 0;
    }
    if (active && bias) v += H::to_float(reinterpret_cast<const uint16_t*>(bias)[gc]);
    const uint16_t* resid = reinterpret_cast<const uint16_t*>(p.residual);
    if (p.rope.cosv) {
        // the pair (even column, odd column) sits in neighbouring lanes; the even one rotates and stores both
        const float im = __shfl_xor_sync(0xffffffffu, v, 1);
        if (active && !(cc & 1)) rope_store_pair<T>(p.rope, p.rope.offset_dev ? *p.rope.offset_dev : p.rope.offset, mb_r, gc, v, im);
    } else if (p.swiglu) {
        // gate column cc (cc % 8 < 4) and its up column cc + 4 sit four lanes apart in the same warp
        const float u = __shfl_xor_sync(0xffffffffu, v, 4);
        if (active && !(cc & 4)) out[(size_t)mb_r * (p.n >> 1) + ((gc >> 3) << 2) + (gc & 3)] = H::from_float(silu_mul(v, u));
    } else if (!fused_ar) {
        if (active && resid) v += H::to_float(resid[(size_t)mb_r * p.n + gc]);
        if (active) out[(size_t)mb_r * p.n + gc] = H::from_float(v);
    } else {
        // four adjacent columns per thread for the exchange: regroup through shared memory
        __syncthreads();                                     // every warp is done reading `red`
        if (active) red[mb_r * VEC_COLS + cc] = v;
        __syncthreads();
        if (tid < 32 * MB && tid / 32 < p.m) {
            const int mb = tid / 32, c4 = (tid % 32) * 4;
            const float4 mine4 = *reinterpret_cast<const float4*>(red + mb * VEC_COLS + c4);
            float4 sum = ar_exchange(p.ar, epoch, (size_t)mb * p.n + tile * VEC_COLS + c4, mine4);
            if (resid) {
                const uint2 rv = __ldg(reinterpret_cast<const uint2*>(resid + (size_t)mb * p.n + tile * VEC_COLS + c4));
                sum.x += H::to_float(uint16_t(rv.x & 0xffff)); sum.y += H::to_float(uint16_t(rv.x >> 16));
                sum.z += H::to_float(uint16_t(rv.y & 0xffff)); sum.w += H::to_float(uint16_t(rv.y >> 16));
            }
            uint2 o; o.x = H::pack(sum.x, sum.y); o.y = H::pack(sum.z, sum.w);
            *reinterpret_cast<uint2*>(out + (size_t)mb * p.n + tile * VEC_COLS + c4) = o;
        }
        __syncthreads();
        if (tid == 0) ar_leave(p.ar, epoch, gridDim.x * gridDim.y);
    }
}


// ----------------------------------------------------------------------------------------------
// Stream-K variant: the same arithmetic, a different schedule.
//
// The (column block, chunk) units of the whole problem are laid out in one line, column block
// major, and cut into equal runs, one per WARP; the grid is one CTA per SM whatever the shape, so
// there is no wave quantisation and no split-K factor to pick.  Warps never synchronise with one
// another: a lane copies its own 16 bytes of every packed row with cp.async into a shared-memory
// ring (D rows deep, so the bytes in flight do not cost registers) and reads them back itself.  A
// run that ends inside a column block leaves an fp32 partial row; the last warp to arrive at a
// column block adds the partials in warp order (deterministic) and writes the output.
// The activations are staged just in time: 32 k-steps (256 values of k) per warp, double
// buffered, the global load issued two blocks ahead.
// A CTA uses half of an SM (registers, shared memory), and the kernel releases its dependents
// at once: under programmatic dependent launch the next kernel's CTAs become resident beside this
// one's, fill their rings with weights and wait, so the stream does not stop between kernels.
// ----------------------------------------------------------------------------------------------
struct StreamParams {
    const void* x; const uint32_t* qw; const uint32_t* qz; const void* scales; const void* bias; void* out;
    const int32_t* xperm;   // act-order: activations are read as x[perm[k]] (null: in order)
    unsigned* counters; float* partial;
    int m, n, k, groups;
    int cpg, nchunks, tiles;
    int units;         // tiles * nchunks
    int warps;         // warps that get a run (<= units)
    int per, rem;      // units / warps, units % warps: the first `rem` warps get per + 1 units
    int zp1_const;
    int pdl;
    ArParams ar;       // row-parallel use: all-reduce of the finished sums over peer memory (ar_mailbox.cuh)
    const void* residual;   // [M,N] T or null, added to the finished (all-reduced) sum before the one rounding
    int swiglu;        // columns are gate / up interleaved in blocks of 4 + 4: out[M,N/2] = silu(gate) * up
    RopeArgs rope;     // rope.cosv != null: rotary embedding + cache append of a fused q/k/v row instead of the store
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
    const int sz = valid ? 16 : 0;   // 0: the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v; asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr)); return v;
}

// The cursor of a warp's weight copies: which packed row comes next, and where its column block ends.
struct RingIt {
    const uint4* ptr;       // next packed row (this lane's 16 bytes of it)
    const uint4* qbase;     // the lane's 16 bytes of row 0, column block 0
    uint32_t rstride_b;     // bytes between packed rows
    int rows;               // rows left in the current column block
    int tile;               // current column block
    int issued, total;      // rows requested so far / rows of the run
    int tile_rows;          // packed rows of a whole column block
};

// A list of linears walked inside one launch (qgemm_vchain_kernel): what an entry needs to know about its neighbours.
struct ChainCtx {
    unsigned* done;             // column blocks finished so far in this launch, all entries together (entries finish in order)
    volatile unsigned* seen;    // shared memory: the largest value of *done that this CTA's polling thread has read
    unsigned* err;              // error word (6: the wait for the previous entry ran out)
    unsigned need;              // column blocks that must be finished before this entry reads its activations
    unsigned epoch;             // epoch of this entry's all-reduce
    int spin_limit;
    const StreamParams* next;   // the entry after this one (null: last)
    bool late;                  // tuning: request the next entry's rows after the combine step, not before
    bool prefilled;             // `it` is this entry's cursor and its first D rows are already on their way
    RingIt it;
};

template <int BITS, typename T, int MB, int CK, int NW, int D, bool CHAIN>
__device__ __forceinline__ void vstream_body(const StreamParams& p, unsigned char* smem, float* seg, int* seg_tile, ChainCtx& cx) {
    using H = F16x2<T>;
    constexpr int PACK = 32 / BITS;
    constexpr int RPK = 8 / PACK;            // packed rows per k-step (8 values of k)
    constexpr int CKS = CK / 8;              // k-steps per chunk
    constexpr int CRW = CKS * RPK;           // packed rows per chunk
    constexpr int BODY = D > 16 ? D : 16;    // packed rows per unrolled body
    constexpr int RG = 4;                    // packed rows per cp.async group
    constexpr int NG = D / RG;               // groups in flight
    constexpr int XB = 32;                   // k-steps per activation block
    constexpr uint32_t MASK_LO = BITS == 4 ? 0x000f000fu : 0x00ff00ffu;
    constexpr uint32_t MASK_HI = 0x00f000f0u;
    static_assert(D % RG == 0 && BODY % D == 0, "ring depth");

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (!CHAIN && p.pdl) griddep_launch_dependents();
    const int j = blockIdx.x * NW + warp;
    const bool idle = j >= p.warps;

    // the run of warp jj in entry q: the first `rem` warps get per + 1 units
    auto run_of = [](const StreamParams& q, int jj, int& first, int& count) {
        if (jj >= q.warps) { first = 0; count = 0; return; }
        first = jj * q.per + (jj < q.rem ? jj : q.rem); count = q.per + (jj < q.rem ? 1 : 0);
    };
    int u0, nun;                      // chunks of this warp's run (0: no run, the warp only joins the CTA's combine step)
    run_of(p, j, u0, nun);
    int tile = u0 / p.nchunks;
    const int c_first = u0 - tile * p.nchunks;
    const int total_rows = nun * CRW;
    const int total_ks = nun * CKS;

    // ---- shared memory: weight ring | per-warp activation blocks | per-warp block meta ----
    const uint32_t ring_s = smem_u32(smem) + uint32_t(tid) * 16;                       // + slot * NW*32*16
    constexpr uint32_t SLOT_BYTES = NW * 32 * 16;
    unsigned char* xw = smem + (size_t)D * SLOT_BYTES + (size_t)warp * (2 * MB * XB * 16);
    float2* metaw = reinterpret_cast<float2*>(smem + (size_t)D * SLOT_BYTES + (size_t)NW * (2 * MB * XB * 16)) + (size_t)warp * (2 * MB * (XB / CKS));
    const uint32_t xw_s = smem_u32(xw);

    // ---- activations: block b covers k-steps [32b, 32b+32) of the run, lane = k-step ----
    const T* xg = reinterpret_cast<const T*>(p.x);
    auto load_x = [&](int b, uint4 (&xr)[MB]) {
        const int ks = b * XB + lane;
        const bool ok = ks < total_ks;
        const int cl = (c_first + ks / CKS) % p.nchunks;               // chunk inside K
        const size_t k = (size_t)cl * CK + (size_t)(ks % CKS) * 8;
#pragma unroll
        for (int mb = 0; mb < MB; ++mb)
            xr[mb] = (ok && mb < p.m) ? load_x8<T, CHAIN>(xg + (size_t)mb * p.k, p.xperm, k, p.k - 1) : make_uint4(0, 0, 0, 0);
    };
    auto stage_x = [&](int b, const uint4 (&xr)[MB]) {
        const int buf = b & 1;
#pragma unroll
        for (int mb = 0; mb < MB; ++mb) {
            float f[8];
            const uint32_t rw[4] = {xr[mb].x, xr[mb].y, xr[mb].z, xr[mb].w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                f[2 * q] = H::to_float(uint16_t(rw[q] & 0xffff));
                f[2 * q + 1] = H::to_float(uint16_t(rw[q] >> 16));
            }
            float amax = 0.f, sum = 0.f;
#pragma unroll
            for (int q = 0; q < 8; ++q) { amax = fmaxf(amax, fabsf(f[q])); sum += f[q]; }
#pragma unroll
            for (int o = 1; o < CKS; o <<= 1) {
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
                sum += __shfl_xor_sync(0xffffffffu, sum, o);
            }
            int e = 0;
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
            *reinterpret_cast<uint4*>(xw + ((size_t)(buf * MB + mb) * XB + lane) * 16) = o4;
            if ((lane % CKS) == 0) metaw[(buf * MB + mb) * (XB / CKS) + lane / CKS] = make_float2(post, sum);
        }
    };
    // The weight prefetch comes before the wait for the previous kernel: the activation loads then
    // queue behind 64 KB of weight requests per CTA, but a CTA that becomes resident early fills its
    // ring during the previous kernel's tail (measured: waiting first costs 1-2 us per launch).
    uint4 xr[MB], xr0[MB];

    // ---- weight copies: issue iterator runs D rows ahead of the consumer ----
    auto ring_begin = [&](const StreamParams& q) -> RingIt {
        int q_u0, q_nun;
        run_of(q, j, q_u0, q_nun);
        const int q_tile = q_u0 / q.nchunks, q_c = q_u0 - q_tile * q.nchunks;
        RingIt r;
        r.qbase = reinterpret_cast<const uint4*>(q.qw) + lane;
        r.rstride_b = uint32_t(q.n) * 4u;
        r.ptr = r.qbase + (size_t)q_tile * (VEC_COLS / 4) + (size_t)q_c * CRW * (size_t(q.n) / 4);
        r.rows = (q.nchunks - q_c) * CRW;
        r.tile = q_tile; r.issued = 0; r.total = q_nun * CRW; r.tile_rows = q.nchunks * CRW;
        return r;
    };
    auto issue = [&](RingIt& r, int slot) {
        const bool valid = r.issued < r.total;
        cp_async16(ring_s + uint32_t(slot) * SLOT_BYTES, valid ? r.ptr : r.qbase, valid);
        ++r.issued;
        r.ptr = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(r.ptr) + r.rstride_b);
        if (--r.rows == 0) { ++r.tile; r.ptr = r.qbase + (size_t)r.tile * (VEC_COLS / 4); r.rows = r.tile_rows; }
    };
    // RG consecutive rows at once: when they lie in one column block and are all valid (almost always) the
    // addresses are base + r * stride and the bookkeeping runs once per group instead of once per row
    auto issue_group = [&](RingIt& r, int slot0) {
        if (r.rows > RG && r.issued + RG <= r.total) {
            const char* base = reinterpret_cast<const char*>(r.ptr);
#pragma unroll
            for (int q = 0; q < RG; ++q)
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(ring_s + uint32_t(slot0 + q) * SLOT_BYTES),
                             "l"(base + (unsigned long long)(uint32_t(q) * r.rstride_b)) : "memory");
            r.issued += RG; r.rows -= RG;
            r.ptr = reinterpret_cast<const uint4*>(base + (unsigned long long)(uint32_t(RG) * r.rstride_b));
        } else {
#pragma unroll
            for (int q = 0; q < RG; ++q) issue(r, slot0 + q);
        }
    };
    auto fill_ring = [&](RingIt& r) {
#pragma unroll
        for (int gq = 0; gq < NG; ++gq) {
            issue_group(r, gq * RG);
            cp_async_commit();
        }
    };
    RingIt it;
    if (CHAIN && cx.prefilled) {
        it = cx.it;                       // requested while the previous entry's sums were being combined
    } else {
        it = ring_begin(p);
        fill_ring(it);
    }

    // ---- scales / zero points: current group converted, next two raw ----
    const T* sc = reinterpret_cast<const T*>(p.scales);
    int g = c_first / p.cpg;
    int left = p.cpg - (c_first - g * p.cpg);
    const int zshift = (lane & (PACK / 4 - 1)) * (4 * BITS);
    int pf_tile = tile, pf_g = g;
    auto pf_advance = [&]() { if (++pf_g == p.groups) { pf_g = 0; ++pf_tile; } };
    auto load_s = [&]() -> uint2 {
        const int tt = pf_tile < p.tiles ? pf_tile : p.tiles - 1;
        return __ldg(reinterpret_cast<const uint2*>(sc + (size_t)pf_g * p.n + tt * VEC_COLS + lane * 4));
    };
    auto load_z = [&]() -> uint32_t {
        if (!p.qz) return 0u;
        const int tt = pf_tile < p.tiles ? pf_tile : p.tiles - 1;
        return __ldg(p.qz + (size_t)pf_g * (p.n / PACK) + (tt * VEC_COLS + lane * 4) / PACK);
    };
    uint2 s0 = load_s(); uint32_t z0 = load_z(); pf_advance();
    uint2 s1 = load_s(); uint32_t z1 = load_z(); pf_advance();
    uint2 s2 = load_s(); uint32_t z2 = load_z();

    if constexpr (CHAIN) {
        // the activations may be the previous entry's output: wait, bounded, until all its column blocks are stored
        // One thread of the CTA polls the counter in global memory and relays what it saw through shared memory:
        // thousands of warps polling one word would queue at its L2 slice and hold up the weight stream behind them.
        // (Warps without a run in this entry do not wait; the CTA's warp 0 has a run whenever any of its warps has.)
        if (cx.need && !idle) {
            if (lane == 0) {
                int spins = 0;
                for (;;) {
                    if (*cx.seen >= cx.need) break;
                    if (warp == 0) {
                        unsigned v;
                        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(cx.done) : "memory");
                        if (v >= cx.need) { __threadfence(); *cx.seen = v; break; }
                    }
                    if (++spins > cx.spin_limit) { if (cx.err) atomicExch(cx.err, 6u); break; }   // give up and flag it: the host reads the word
                    __nanosleep(warp == 0 ? 100 : 40);
                }
                __threadfence();
            }
            __syncwarp();
        }
    } else {
        if (p.pdl) griddep_wait();
    }
    load_x(0, xr0);
    load_x(1, xr);

    stage_x(0, xr0);

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

    const T* bias = reinterpret_cast<const T*>(p.bias);
    uint16_t* out = reinterpret_cast<uint16_t*>(p.out);
    const bool fused_ar = ar_active(p.ar);
    const unsigned epoch = !fused_ar ? 0u : CHAIN ? cx.epoch : ar_epoch(p.ar);   // after griddepcontrol.wait: the previous call has published its epoch
    auto write_out = [&](int t, const float4 (&r)[MB]) {
        const int colb = t * VEC_COLS + lane * 4;
        float b0 = 0.f, b1 = 0.f, b2 = 0.f, b3 = 0.f;
        if (bias) {
            const uint2 bv = __ldg(reinterpret_cast<const uint2*>(bias + colb));
            b0 = H::to_float(uint16_t(bv.x & 0xffff)); b1 = H::to_float(uint16_t(bv.x >> 16));
            b2 = H::to_float(uint16_t(bv.y & 0xffff)); b3 = H::to_float(uint16_t(bv.y >> 16));
        }
#pragma unroll
        for (int mb = 0; mb < MB; ++mb)
            if (mb < p.m) {
                float4 v = make_float4(r[mb].x + b0, r[mb].y + b1, r[mb].z + b2, r[mb].w + b3);
                if (p.rope.cosv) {
                    const int off = p.rope.offset_dev ? *p.rope.offset_dev : p.rope.offset;
                    rope_store_pair<T>(p.rope, off, mb, colb, v.x, v.y);
                    rope_store_pair<T>(p.rope, off, mb, colb + 2, v.z, v.w);
                    continue;
                }
                if (p.swiglu) {
                    // an even lane holds four gate columns, the next lane their up columns (the whole warp is here)
                    const float4 u = make_float4(__shfl_xor_sync(0xffffffffu, v.x, 1), __shfl_xor_sync(0xffffffffu, v.y, 1),
                                                 __shfl_xor_sync(0xffffffffu, v.z, 1), __shfl_xor_sync(0xffffffffu, v.w, 1));
                    if (!(lane & 1)) {
                        uint2 o; o.x = H::pack(silu_mul(v.x, u.x), silu_mul(v.y, u.y)); o.y = H::pack(silu_mul(v.z, u.z), silu_mul(v.w, u.w));
                        *reinterpret_cast<uint2*>(out + (size_t)mb * (p.n >> 1) + (colb >> 1)) = o;
                    }
                    continue;
                }
                if (fused_ar) v = ar_exchange(p.ar, epoch, (size_t)mb * p.n + colb, v);
                if (p.residual) {
                    const uint2* rp = reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(p.residual) + (size_t)mb * p.n + colb);
                    const uint2 rv = CHAIN ? __ldcg(rp) : __ldg(rp);
                    v.x += H::to_float(uint16_t(rv.x & 0xffff)); v.y += H::to_float(uint16_t(rv.x >> 16));
                    v.z += H::to_float(uint16_t(rv.y & 0xffff)); v.w += H::to_float(uint16_t(rv.y >> 16));
                }
                uint2 o; o.x = H::pack(v.x, v.y); o.y = H::pack(v.z, v.w);
                *reinterpret_cast<uint2*>(out + (size_t)mb * p.n + colb) = o;
            }
        if constexpr (CHAIN) {
            // one more column block of this launch is in memory: release it to the entries that read it
            __syncwarp();
            if (lane == 0) { __threadfence(); atomicAdd(cx.done, 1u); }
        }
    };
    // first and last warp with a run in column block t
    auto owner = [&](int u) -> int {
        const int big = p.rem * (p.per + 1);              // units held by the warps with per + 1
        return u < big ? u / (p.per + 1) : p.rem + (u - big) / p.per;
    };
    auto owners = [&](int t, int& jf, int& jl) {
        jf = owner(t * p.nchunks);
        jl = owner(t * p.nchunks + p.nchunks - 1);
    };
    int nseg = 0;
    // the finished part of column block `tile`: written out if no other warp has a share in the
    // block, else parked in shared memory for the CTA's combine step
    auto flush = [&]() {
        int jf, jl;
        owners(tile, jf, jl);
        float4 r[MB];
#pragma unroll
        for (int mb = 0; mb < MB; ++mb) r[mb] = make_float4(acc[mb][0], acc[mb][1], acc[mb][2], acc[mb][3]);
        if (jf == jl) {
            write_out(tile, r);
        } else {
            const int slot = warp * 2 + (nseg < 1 ? nseg : 1);
#pragma unroll
            for (int mb = 0; mb < MB; ++mb)
                *reinterpret_cast<float4*>(seg + ((size_t)slot * MB + mb) * VEC_COLS + lane * 4) = r[mb];
            if (lane == 0) seg_tile[slot] = tile;
            ++nseg;
        }
#pragma unroll
        for (int mb = 0; mb < MB; ++mb)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[mb][c] = 0.f;
    };

    // ---- main loop: BODY packed rows per trip ----
    int chunks_todo = nun;
    bool dirty = false, done = idle;
    for (int body = 0; !done; ++body) {
        const int ks_body = body * (BODY / RPK);          // first k-step of this body
        if ((ks_body % XB) == 0) {
            // entering activation block b: stage block b+1 (loaded one block ago), start the load of b+2
            const int b = ks_body / XB;
            __syncwarp();                                 // every lane is done reading block b-1, whose buffer is rewritten
            stage_x(b + 1, xr);
            load_x(b + 2, xr);
            __syncwarp();
        }
        const int buf = (ks_body / XB) & 1;
        const uint32_t xs_s = xw_s + uint32_t(buf * MB * XB + (ks_body % XB)) * 16;
        const float2* meta = metaw + buf * MB * (XB / CKS) + (ks_body % XB) / CKS;
#pragma unroll
        for (int rb = 0; rb < BODY; ++rb) {
            if (rb % RG == 0) cp_async_wait<NG - 1>();
            const int slot = rb % D;
            const int kj = rb / RPK, rr = rb % RPK;          // k-step inside the body, row inside the k-step
            const uint4 wv = lds128(ring_s + uint32_t(slot) * SLOT_BYTES);
            uint4 xv[MB];
#pragma unroll
            for (int mb = 0; mb < MB; ++mb) xv[mb] = lds128(xs_s + uint32_t(mb * XB + kj) * 16);
            const bool first = (kj % CKS) == 0;
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
            if (rb % RG == RG - 1) {
                // the four rows of this group are in registers: refill their slots
                issue_group(it, (rb - (RG - 1)) % D);
                cp_async_commit();
            }
            if (rr == RPK - 1 && (kj + 1) % CKS == 0) {
                if (!done) {
                    // ---- fold the chunk that ends here ----
                    const int ci = kj / CKS;
#pragma unroll
                    for (int mb = 0; mb < MB; ++mb) {
                        const float2 mt2 = meta[mb * (XB / CKS) + ci];   // (2^(24-e), sum of x)
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            const float f = h2sum(hadd2(hadd2(a[mb][c][0], a[mb][c][1]), hadd2(a[mb][c][2], a[mb][c][3])));
                            const float t = fmaf(f, mt2.x, -zf[c] * mt2.y);
                            acc[mb][c] = fmaf(sf[c], t, acc[mb][c]);
                        }
                    }
                    dirty = true;
                    if (--left == 0) {
                        left = p.cpg;
                        if (++g == p.groups) { flush(); dirty = false; g = 0; ++tile; }
                        convert(s1, z1);
                        s1 = s2; z1 = z2;
                        pf_advance();
                        s2 = load_s(); z2 = load_z();
                    }
                    if (--chunks_todo == 0) {
                        if (dirty) flush();
                        done = true;
                    }
                }
            }
        }
    }
    cp_async_wait<0>();
    if constexpr (CHAIN) {
        // the ring is free: request the first rows of the next entry now, so that its weights stream while this
        // entry's partial sums are combined and while the next entry waits for them
        if (cx.next && !cx.late) { cx.it = ring_begin(*cx.next); fill_ring(cx.it); cx.prefilled = true; }
    }

    // ---- combine the shared partial rows: CTA first, then across CTAs ----
    if (lane == 0) {
        if (nseg < 1) seg_tile[warp * 2] = -1;
        if (nseg < 2) seg_tile[warp * 2 + 1] = -1;
    }
    __syncthreads();
    const int cta = blockIdx.x;
    for (int q = 0; q < 2; ++q) {
        const int slot = warp * 2 + q;
        const int t = seg_tile[slot];
        if (t < 0) continue;
        bool lead = true;                                   // the first slot of the CTA that holds this column block does the sum
        for (int s2i = 0; s2i < slot; ++s2i) lead = lead && seg_tile[s2i] != t;
        if (!lead) continue;
        float4 r[MB];
#pragma unroll
        for (int mb = 0; mb < MB; ++mb) r[mb] = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int s2i = slot; s2i < NW * 2; ++s2i) {
            if (seg_tile[s2i] != t) continue;
#pragma unroll
            for (int mb = 0; mb < MB; ++mb) {
                const float4 v = *reinterpret_cast<const float4*>(seg + ((size_t)s2i * MB + mb) * VEC_COLS + lane * 4);
                r[mb].x += v.x; r[mb].y += v.y; r[mb].z += v.z; r[mb].w += v.w;
            }
        }
        int jf, jl;
        owners(t, jf, jl);
        const int cf = jf / NW, cl = jl / NW;               // first and last CTA with a share in the block
        bool write = true;
        if (cf != cl) {
            // The LAST CTA with a share in the block finishes it.  The others store their partial row and count
            // themselves in with a release-add that nobody waits for (every lane releases its own 16 bytes); the owner
            // polls the count -- bounded -- and then adds the rows in CTA order, its own (still in registers) last.
            // It only ever waits for CTAs with a smaller index, which were dispatched before it.
            if (cta != cl) {
#pragma unroll
                for (int mb = 0; mb < MB; ++mb)
                    if (mb < p.m) __stcg(reinterpret_cast<float4*>(p.partial + ((size_t)(cta + t) * MB + mb) * VEC_COLS + lane * 4), r[mb]);
                asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(p.counters + t) : "memory");
                write = false;
            } else {
                const unsigned target = 32u * unsigned(cl - cf);
                for (int spins = 0;; ++spins) {
                    unsigned v;
                    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p.counters + t) : "memory");
                    if (v >= target) break;
                    if (spins > (1 << 21)) { if (p.ar.err) atomicExch(p.ar.err, 7u); break; }   // give up and flag it: the host reads the word
                    if (spins > 8) __nanosleep(40);
                }
                float4 own[MB];
#pragma unroll
                for (int mb = 0; mb < MB; ++mb) { own[mb] = r[mb]; r[mb] = make_float4(0.f, 0.f, 0.f, 0.f); }
                for (int cc = cf; cc < cl; cc += 8) {       // eight independent loads in flight, summed in CTA order
                    float4 v[8][MB];
#pragma unroll
                    for (int qq = 0; qq < 8; ++qq)
#pragma unroll
                        for (int mb = 0; mb < MB; ++mb)
                            v[qq][mb] = (cc + qq < cl && mb < p.m)
                                ? __ldcg(reinterpret_cast<const float4*>(p.partial + ((size_t)(cc + qq + t) * MB + mb) * VEC_COLS + lane * 4))
                                : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int qq = 0; qq < 8; ++qq)
#pragma unroll
                        for (int mb = 0; mb < MB; ++mb) { r[mb].x += v[qq][mb].x; r[mb].y += v[qq][mb].y; r[mb].z += v[qq][mb].z; r[mb].w += v[qq][mb].w; }
                }
#pragma unroll
                for (int mb = 0; mb < MB; ++mb) { r[mb].x += own[mb].x; r[mb].y += own[mb].y; r[mb].z += own[mb].z; r[mb].w += own[mb].w; }
                __syncwarp();
                if (lane == 0) p.counters[t] = 0;
            }
        }
        if (write) write_out(t, r);
    }
    if constexpr (CHAIN) {
        if (cx.next && cx.late) { cx.it = ring_begin(*cx.next); fill_ring(cx.it); cx.prefilled = true; }
        __syncthreads();                 // the next entry rewrites the partial rows in shared memory
    } else if (fused_ar) {
        __syncthreads();
        if (tid == 0) ar_leave(p.ar, epoch, gridDim.x);
    }
}

template <int BITS, typename T, int MB, int CK, int NW, int D, int MINB>
__global__ void __launch_bounds__(NW * 32, MINB) qgemm_vstream_kernel(const StreamParams p) {
    extern __shared__ __align__(16) unsigned char smem[];
    // partial rows of column blocks that a warp shares with others: at most two per warp (the
    // block its run starts in and the block it ends in), combined across the CTA before they leave it
    __shared__ __align__(16) float seg[NW * 2 * MB * VEC_COLS];
    __shared__ int seg_tile[NW * 2];
    ChainCtx cx;
    vstream_body<BITS, T, MB, CK, NW, D, false>(p, smem, seg, seg_tile, cx);
}

// ----------------------------------------------------------------------------------------------
// Several linears in ONE launch.  The grid is resident as a whole (cooperative launch, one CTA per
// half SM) and every CTA walks the list: entry e+1 may read what entry e wrote (a decoder layer's
// o-projection -> gate/up -> down), so a warp waits -- bounded -- until the launch-wide count of
// stored column blocks reaches the end of entry e before it reads entry e+1's activations.  Its
// weight ring is already filling by then: the copies of an entry's first rows are requested before
// the previous entry's partial sums are combined, so the weight stream never stops at a boundary.
// All-reduce entries use consecutive epochs; the last CTA to leave publishes the final one and
// returns the two control words to zero for the next launch (or graph replay).
// ----------------------------------------------------------------------------------------------
constexpr int kChainMax = MT_CHAIN_MAX;
struct ChainParams {
    StreamParams e[kChainMax];
    unsigned need[kChainMax];     // column blocks of all earlier entries
    int ar_index[kChainMax];      // this entry's exchange is the i-th of the launch (-1: none)
    int count, ar_count;
    unsigned* done; unsigned* leave; unsigned* err;
    int spin_limit;
    int late;
    ArParams ar;                  // shared by the entries that exchange
};

template <int BITS, typename T, int MB, int CK, int NW, int D, int MINB>
__global__ void __launch_bounds__(NW * 32, MINB) qgemm_vchain_kernel(const __grid_constant__ ChainParams cp) {
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ __align__(16) float seg[NW * 2 * MB * VEC_COLS];
    __shared__ int seg_tile[NW * 2];
    __shared__ unsigned seen;
    if (threadIdx.x == 0) seen = 0;
    __syncthreads();
    ChainCtx cx;
    cx.seen = &seen;
    cx.late = cp.late != 0;
    cx.done = cp.done; cx.err = cp.err; cx.spin_limit = cp.spin_limit; cx.prefilled = false;
    const unsigned epoch0 = cp.ar_count ? ar_epoch(cp.ar) : 0u;    // the previous launch has completed: the word is stable
    for (int e = 0; e < cp.count; ++e) {
        cx.need = cp.need[e];
        cx.epoch = epoch0 + unsigned(cp.ar_index[e] < 0 ? 0 : cp.ar_index[e]);
        cx.next = e + 1 < cp.count ? &cp.e[e + 1] : nullptr;
        vstream_body<BITS, T, MB, CK, NW, D, true>(cp.e[e], smem, seg, seg_tile, cx);
    }
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(cp.leave, 1u) == gridDim.x - 1) {
            *cp.done = 0; *cp.leave = 0;
            if (cp.ar_count) {
                __threadfence();
                *reinterpret_cast<volatile unsigned*>(cp.ar.peers[cp.ar.rank]) = epoch0 + unsigned(cp.ar_count - 1);
            }
        }
    }
}

template <int BITS, typename T, int MB, int CK>
int launch_one(cudaStream_t st, const VecParams& p, dim3 grid, size_t smem) {
    auto kern = qgemm_vec_kernel<BITS, T, MB, CK>;
    static bool configured[64] = {};                       // per device ordinal: opt in to large dynamic shared memory once
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { cudaGetLastError(); return MT_ERR_CUDA; }
    if (!configured[dev]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024) != cudaSuccess) { cudaGetLastError(); return MT_ERR_CUDA; }
        configured[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = dim3(VEC_THREADS); cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (p.pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    if (p.cluster) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = 1; attr[na].val.clusterDim.y = grid.y; attr[na].val.clusterDim.z = 1;
        ++na;
    }
    cfg.attrs = attr; cfg.numAttrs = na;
    if (cudaLaunchKernelEx(&cfg, kern, p) != cudaSuccess) { cudaGetLastError(); return MT_ERR_CUDA; }
    return MT_OK;
}

template <int BITS, typename T>
int launch_mb(cudaStream_t st, const VecParams& p, int ck, dim3 grid, size_t smem) {
    if (p.m == 1) return ck == 64 ? launch_one<BITS, T, 1, 64>(st, p, grid, smem) : launch_one<BITS, T, 1, 32>(st, p, grid, smem);
    return ck == 64 ? launch_one<BITS, T, 2, 64>(st, p, grid, smem) : launch_one<BITS, T, 2, 32>(st, p, grid, smem);
}

template <int BITS, typename T, int MB, int CK, int NW, int D, int MINB>
int launch_stream_one(cudaStream_t st, const StreamParams& p, int grid) {
    auto kern = qgemm_vstream_kernel<BITS, T, MB, CK, NW, D, MINB>;
    constexpr int CKS = CK / 8;
    const size_t smem = (size_t)D * NW * 32 * 16 + (size_t)NW * 2 * MB * 32 * 16 + (size_t)NW * 2 * MB * (32 / CKS) * 8;
    static bool configured[64] = {};                       // per device ordinal: the attribute is set once
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { cudaGetLastError(); return MT_ERR_CUDA; }
    if (!configured[dev]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) { cudaGetLastError(); return MT_ERR_CUDA; }
        configured[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(NW * 32); cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = p.pdl ? 1 : 0;
    if (cudaLaunchKernelEx(&cfg, kern, p) != cudaSuccess) { cudaGetLastError(); return MT_ERR_CUDA; }
    return MT_OK;
}

template <int BITS, typename T, int NW, int D, int MINB>
int launch_stream_mb(cudaStream_t st, const StreamParams& p, int ck, int grid) {
    if (p.m == 1) return ck == 64 ? launch_stream_one<BITS, T, 1, 64, NW, D, MINB>(st, p, grid) : launch_stream_one<BITS, T, 1, 32, NW, D, MINB>(st, p, grid);
    return ck == 64 ? launch_stream_one<BITS, T, 2, 64, NW, D, MINB>(st, p, grid) : launch_stream_one<BITS, T, 2, 32, NW, D, MINB>(st, p, grid);
}

// Parameters of the stream-K schedule for one linear on `ctas` CTAs of NW warps.
static int make_stream_params(const QGemmArgs& a, int ctas, int NW, StreamParams& p, int& ck) {
    const int gs = a.k / a.groups;
    ck = gs % 64 == 0 ? 64 : 32;
    p.x = a.x; p.qw = a.qweight; p.qz = a.qzeros; p.scales = a.scales; p.bias = a.bias; p.out = a.out;
    p.xperm = a.x_perm;
    p.counters = static_cast<unsigned*>(a.workspace);
    p.partial = reinterpret_cast<float*>(static_cast<char*>(a.workspace) + kCounterBytes);
    p.m = a.m; p.n = a.n; p.k = a.k; p.groups = a.groups;
    p.cpg = gs / ck; p.nchunks = a.k / ck; p.tiles = a.n / VEC_COLS;
    if ((long long)p.tiles * p.nchunks > (1LL << 30)) return MT_ERR_TOO_LARGE;
    p.units = p.tiles * p.nchunks;
    const int mb = a.m == 1 ? 1 : 2;
    long long warps = (long long)ctas * NW;
    if (warps > p.units) warps = p.units;
    const long long cap = (long long)((a.workspace_bytes - kCounterBytes) / ((size_t)mb * VEC_COLS * 4)) - p.tiles;
    if (warps > cap) warps = cap;
    if (warps < 1) return MT_ERR_WORKSPACE;
    p.warps = (int)warps;
    p.per = p.units / p.warps; p.rem = p.units % p.warps;
    p.ar = make_ar_params(a);
    if (p.ar.world > 1 && (size_t)a.m * a.n * 8 > p.ar.slot_bytes) return MT_ERR_TOO_LARGE;
    p.residual = a.residual; p.swiglu = a.epilogue == MT_EPILOGUE_SWIGLU ? 1 : 0;
    if (a.rope) p.rope = *a.rope; else p.rope.cosv = nullptr;
    p.zp1_const = 1 << (a.bits - 1);
    p.pdl = (a.flags & MT_FLAG_PDL) ? 1 : 0;
    return MT_OK;
}

template <int NW, int D, int MINB>
int launch_stream_cfg(cudaStream_t st, const QGemmArgs& a, int ctas) {
    StreamParams p;
    int ck = 0;
    const int rc = make_stream_params(a, ctas, NW, p, ck);
    if (rc != MT_OK) return rc;
    const int grid = (p.warps + NW - 1) / NW;
    if (a.bits == 4) return a.dtype == MT_F16 ? launch_stream_mb<4, __half, NW, D, MINB>(st, p, ck, grid) : launch_stream_mb<4, __nv_bfloat16, NW, D, MINB>(st, p, ck, grid);
    return a.dtype == MT_F16 ? launch_stream_mb<8, __half, NW, D, MINB>(st, p, ck, grid) : launch_stream_mb<8, __nv_bfloat16, NW, D, MINB>(st, p, ck, grid);
}

constexpr int CH_NW = 8, CH_D = 16, CH_MINB = 2;

template <int BITS, typename T, int MB, int CK>
int launch_chain_one(cudaStream_t st, const ChainParams& cp) {
    auto kern = qgemm_vchain_kernel<BITS, T, MB, CK, CH_NW, CH_D, CH_MINB>;
    constexpr int CKS = CK / 8;
    const size_t smem = (size_t)CH_D * CH_NW * 32 * 16 + (size_t)CH_NW * 2 * MB * 32 * 16 + (size_t)CH_NW * 2 * MB * (32 / CKS) * 8;
    static int resident[64] = {};                          // per device ordinal: CTAs that fit the GPU at once (0: not asked yet)
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { cudaGetLastError(); return MT_ERR_CUDA; }
    if (!resident[dev]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) { cudaGetLastError(); return MT_ERR_CUDA; }
        int per_sm = 0, sms = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, CH_NW * 32, smem) != cudaSuccess ||
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || per_sm < 1 || sms < 1) { cudaGetLastError(); return MT_ERR_CUDA; }
        resident[dev] = per_sm * sms;
    }
    int grid = 0;
    for (int e = 0; e < cp.count; ++e) grid = max(grid, (cp.e[e].warps + CH_NW - 1) / CH_NW);
    // the CTAs wait for one another, so all of them must be resident: a cooperative launch fails instead of hanging
    if (grid > resident[dev]) return MT_ERR_UNSUPPORTED;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(CH_NW * 32); cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, kern, cp) != cudaSuccess) { cudaGetLastError(); return MT_ERR_CUDA; }
    return MT_OK;
}

template <int BITS, typename T>
int launch_chain_mb(cudaStream_t st, const ChainParams& cp, int m, int ck) {
    if (m == 1) return ck == 64 ? launch_chain_one<BITS, T, 1, 64>(st, cp) : launch_chain_one<BITS, T, 1, 32>(st, cp);
    return ck == 64 ? launch_chain_one<BITS, T, 2, 64>(st, cp) : launch_chain_one<BITS, T, 2, 32>(st, cp);
}

}  // namespace

// CTAs of the split-K kernel that can be resident at once when launched as clusters of s (cached
// per device).  All instantiations share the launch bounds, so one of them stands for all.
static int cluster_slots(int s) {
    static int cache[64][9] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64 || s < 1 || s > 8) { cudaGetLastError(); return 256; }
    if (cache[dev][s] == 0) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(1, s * 64); cfg.blockDim = dim3(VEC_THREADS); cfg.dynamicSmemBytes = 20 * 1024;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = s; attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr; cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, qgemm_vec_kernel<4, __half, 1, 64>, &cfg) != cudaSuccess || n < 1) { cudaGetLastError(); n = 256 / s; }
        cache[dev][s] = n * s;
    }
    return cache[dev][s];
}

bool vec_supported(const QGemmArgs& a) {
    if (a.g_idx || a.m < 1 || a.m > 2 || a.groups < 1) return false;
    if (a.n % VEC_COLS != 0 || a.k % a.groups != 0) return false;
    const int gs = a.k / a.groups;
    if (gs % 32 != 0) return false;
    if (a.n / VEC_COLS >= kMaxTiles - 1) return false;
    return a.workspace != nullptr && a.workspace_bytes >= kCounterBytes;
}

// Schedule of the decode GEMV for a request: > 0 = split-K factor, 0 = stream-K, < 0 = MT_ERR_*.
int vec_plan(const QGemmArgs& a) {
    if (!vec_supported(a)) return MT_ERR_UNSUPPORTED;
    const int variant = (a.flags >> 24) & 0xf;
    if (variant == 2) return 0;
    const int gs = a.k / a.groups;
    const int ck = gs % 64 == 0 ? 64 : 32;
    const int nchunks = a.k / ck;
    const int tiles = a.n / VEC_COLS;
    // split-K: every warp gets at least one chunk and at most 2048 values of k (its activations live
    // in shared memory) and the partial sums must fit the workspace.  Among the admissible factors a
    // small cost model picks: CTA slots come from the occupancy of the cluster launch, capped at 256
    // (2 CTAs fit an SM, but clusters do not tile every GPC and the previous launch of a chain still
    // holds slots); a CTA that shares its SM streams ~23.6 GB/s, one that has the SM to itself ~30 GB/s
    // (its own loads in flight are the limit); a wave costs ~2.4 us of launch, prologue and reduction
    // (+0.3 us for the cluster hand-over, +1.8 us when the splits meet in global memory), every further
    // wave 3 us and 5 % for its ragged end.  When no factor fills the waves well the stream-K schedule
    // (~6.5 us fixed, then ~6 TB/s) takes over.
    const int forced = (a.flags >> 16) & 0xff;
    const bool no_cluster = ((a.flags >> 28) & 1) != 0;          // bit 28 of the flags: tuning, no clusters
    int splits = forced;
    const int min_splits = (a.k + VEC_WARPS * 2048 - 1) / (VEC_WARPS * 2048);
    int max_splits = nchunks / VEC_WARPS;
    if (max_splits < 1) max_splits = 1;
    const size_t cap = (a.workspace_bytes - kCounterBytes) / ((size_t)a.m * a.n * 4);
    if ((size_t)max_splits > cap) max_splits = cap < 1 ? 1 : (int)cap;
    if (max_splits > 64) max_splits = 64;
    if (min_splits > max_splits) return min_splits > 1 && (size_t)min_splits > cap ? MT_ERR_WORKSPACE : MT_ERR_TOO_LARGE;
    if (forced) return splits < min_splits ? min_splits : (splits > max_splits ? max_splits : splits);
    const double slow = a.m == 1 ? 1.0 : 0.65;                  // two batch rows: the FMA pipe, not HBM, sets the rate
    const double total_kb = (double)a.k * VEC_COLS * a.bits / 8.0 / 1024.0;
    double best = 1e30;
    for (int s = min_splits; s <= max_splits; ++s) {
        const bool cl = s >= 2 && s <= 8 && !no_cluster;
        int slots = 296;
        if (cl) { slots = cluster_slots(s); if (slots > 256) slots = 256 / s * s; }
        const double kb = total_kb / s * 1.024;                  // KB -> 1e3 bytes: GB/s == KB/us
        const long long ctas = (long long)tiles * s;
        const long long full = ctas / slots;
        const long long rem = ctas - full * slots;
        const double t0 = 2.4 + (s == 1 ? 0.0 : cl ? 0.3 : 1.8);
        double t = 0.0;
        if (full > 0) t += t0 + kb / (23.6 * slow) + double(full - 1) * (3.0 + kb / (23.6 * slow));
        if (rem > 0) t += (full > 0 ? 3.0 : t0) + kb / ((rem <= 160 ? 30.0 : 23.6) * slow);
        if (full + (rem > 0) > 1) t *= 1.05;
        t += 0.02 * s;                                            // more partial sums to write and add
        if (t < best) { best = t; splits = s; }
    }
    const double t_stream = 6.5 + total_kb * 1.024 * tiles / (6000.0 * slow);
    if (variant == 0 && t_stream < best) return 0;
    return splits;
}

// `count` linears (each one a request the stream-K GEMV accepts: M <= 2, no g_idx) in one launch, in list order, every
// entry free to read what an earlier one wrote.  All entries share M, the bit width, the dtype, the workspace and --
// where they exchange -- the peers.  Returns MT_ERR_UNSUPPORTED when the list does not fit the scheme (the caller
// then launches the linears one by one).
int launch_vec_chain(cudaStream_t st, const QGemmArgs* list, int count) {
    if (count < 1 || count > kChainMax) return MT_ERR_UNSUPPORTED;
    ChainParams cp;
    cp.count = count; cp.ar_count = 0;
    int ck0 = 0;
    unsigned tiles_before = 0;
    const QGemmArgs& a0 = list[0];
    for (int e = 0; e < count; ++e) {
        const QGemmArgs& a = list[e];
        if (!vec_supported(a) || a.m != a0.m || a.bits != a0.bits || a.dtype != a0.dtype || a.workspace != a0.workspace ||
            a.workspace_bytes != a0.workspace_bytes) return MT_ERR_UNSUPPORTED;
        if (a.n / VEC_COLS >= kMaxTiles - 4) return MT_ERR_UNSUPPORTED;      // the last words of the counter area are the chain's
        int ck = 0;
        const int rc = make_stream_params(a, 296, CH_NW, cp.e[e], ck);
        if (rc != MT_OK) return rc;
        if (e == 0) ck0 = ck; else if (ck != ck0) return MT_ERR_UNSUPPORTED;
        cp.need[e] = tiles_before;
        tiles_before += unsigned(cp.e[e].tiles);
        cp.ar_index[e] = -1;
        if (cp.e[e].ar.world > 1) {
            if (cp.ar_count && (cp.e[e].ar.peers != cp.ar.peers || cp.e[e].ar.slot_bytes != cp.ar.slot_bytes)) return MT_ERR_UNSUPPORTED;
            cp.ar = cp.e[e].ar;
            cp.ar_index[e] = cp.ar_count++;
        }
    }
    unsigned* words = static_cast<unsigned*>(a0.workspace);
    cp.done = words + (kMaxTiles - 3); cp.leave = words + (kMaxTiles - 2); cp.err = words + (kMaxTiles - 1);
    cp.spin_limit = (a0.flags & MT_FLAG_AR_SHORT_WAIT) ? (1 << 10) : (1 << 21);
    cp.late = ((a0.flags >> 24) & 0xf) == 3;
    if (a0.bits == 4) return a0.dtype == MT_F16 ? launch_chain_mb<4, __half>(st, cp, a0.m, ck0) : launch_chain_mb<4, __nv_bfloat16>(st, cp, a0.m, ck0);
    return a0.dtype == MT_F16 ? launch_chain_mb<8, __half>(st, cp, a0.m, ck0) : launch_chain_mb<8, __nv_bfloat16>(st, cp, a0.m, ck0);
}

int launch_vec(cudaStream_t st, const QGemmArgs& a) {
    const int plan = vec_plan(a);
    if (plan < 0) return plan;
    const int ctas_arg = (a.flags >> 16) & 0xff;
    if (plan == 0) return launch_stream_cfg<8, 16, 2>(st, a, ((a.flags >> 24) & 0xf) == 2 && ctas_arg ? ctas_arg * 37 : 296);
    const int splits = plan;
    const bool no_cluster = ((a.flags >> 28) & 1) != 0;
    const int gs = a.k / a.groups;
    const int ck = gs % 64 == 0 ? 64 : 32;
    const int cks = ck / 8;
    const int nchunks = a.k / ck;
    const int tiles = a.n / VEC_COLS;
    VecParams p;
    p.x = a.x; p.qw = a.qweight; p.qz = a.qzeros; p.scales = a.scales; p.bias = a.bias; p.out = a.out;
    p.xperm = a.x_perm;
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
    p.cluster = (splits >= 2 && splits <= 8 && !no_cluster) ? 1 : 0;
    p.ar = make_ar_params(a);
    if (p.ar.world > 1 && (size_t)a.m * a.n * 8 > p.ar.slot_bytes) return MT_ERR_TOO_LARGE;
    p.residual = a.residual; p.swiglu = a.epilogue == MT_EPILOGUE_SWIGLU ? 1 : 0;
    if (a.rope) p.rope = *a.rope; else p.rope.cosv = nullptr;
    const int mb = a.m == 1 ? 1 : 2;
    const size_t smem = (size_t)VEC_WARPS * mb * slice_ks * 16 + (size_t)VEC_WARPS * mb * (slice_ks / cks) * 8;
    if (smem > 160 * 1024) return MT_ERR_TOO_LARGE;
    const dim3 grid(tiles, splits);
    if (a.bits == 4) return a.dtype == MT_F16 ? launch_mb<4, __half>(st, p, ck, grid, smem) : launch_mb<4, __nv_bfloat16>(st, p, ck, grid, smem);
    return a.dtype == MT_F16 ? launch_mb<8, __half>(st, p, ck, grid, smem) : launch_mb<8, __nv_bfloat16>(st, p, ck, grid, smem);
}

}  // namespace mt
