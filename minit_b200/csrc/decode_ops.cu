// The steps either side of the quantized linears in a decoder layer, for decode-sized batches:
//
//  * rms_norm      out = T(float(x) / sqrt(mean(x^2) + eps) * float(w)) per row
//                  (minit/cuda/kernel/cuda/rms_norm.py:55-91: fp32 sum of squares, divide, multiply, one rounding).
//  * rope_append   rotary embedding of the q and k parts of a fused qkv row, (x[2i], x[2i+1]) rotated by
//                  (cos, sin)[position, i] in fp32 (minit/cuda/kernel/cuda/rope.py:58-73), q to its own tensor,
//                  k and v straight into the preallocated cache at row offset + token: the reference grows
//                  the cache by concatenation (examples/llama3_70b.py:99-102) and stores every kv head
//                  nr_groups times (:85-94); here the cache holds each kv head once.
//  * attention     softmax(q k^T / sqrt(d) + causal mask) v for the new tokens against the cache
//                  (examples/llama3_70b.py:103-115), one kernel: a CTA takes one kv head, one token and a
//                  range of cached positions for all query heads of the group (K and V are read once per
//                  group), keeps scores, online softmax and the weighted sum in fp32 (mma.sync m16n8k16 with
//                  the group's query heads as the rows: 64 tensor instructions per 32 positions instead of
//                  ~2300 FMAs), merges the ranges of a cluster through shared memory and the clusters through
//                  global memory, always in order.  The reference rounds the scores,
//                  the scaled scores, the probabilities and the output to the tensor dtype in separate
//                  kernels (softmax: minit/cuda/kernel/cuda/softmax.py:55-106).
//
// All three are bound by HBM (the cache) or by launch latency (16 KB rows), so: 16-byte loads, the
// cache streamed through shared memory once, grids of a few CTAs per SM.  The batch (8 query heads per
// kv head) is far too small for tcgen05's 128-row tiles; the warp-level tensor path is enough to keep
// the arithmetic well under the memory time.
#include "common.cuh"

namespace mt {
namespace {

constexpr int ATT_D = 128;                 // head size
constexpr int ATT_MAXG = 8;                // query heads per kv head
constexpr int ATT_TILE = 32;               // cached positions per warp tile: one per lane
constexpr int ATT_ROW = ATT_D * 2 + 16;    // bytes of a K / V row in shared memory (padded: 16-byte reads of 8 rows hit 32 banks)
constexpr int ATT_WARP_SMEM = 2 * ATT_TILE * ATT_ROW;   // K tile, V tile
constexpr int ATT_CLUSTER = 8;               // CTAs of one (token, kv head) that merge through shared memory
constexpr int ATT_PER_SINGLE = 6;            // tiles per warp up to which one cluster takes the whole sequence (no global stage)
constexpr int ATT_MAXCL = 10;                // clusters per (token, kv head) at most: merged through global memory
constexpr int ATT_PART = ATT_D + 4;        // floats of a partial result per query head: 128 weighted sums, max, sum (+ pad: rows stay 16-byte aligned)

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// One CTA per row; a thread keeps its (up to RMS_NV) 16-byte pieces of the row in registers between the two passes,
// so the row is read once, and the weight load overlaps the reduction.
constexpr int RMS_NV = 4;
template <typename T>
__global__ void __launch_bounds__(1024) rms_norm_kernel(const uint4* __restrict__ x, const uint4* __restrict__ w, uint4* __restrict__ out,
                                                        int h8, float inv_h, float eps) {
    using H = F16x2<T>;
    __shared__ float red[32];
    griddep_launch_dependents();                            // a following linear launched as a programmatic dependent may prefetch its weights now
    const uint4* xr = x + (size_t)blockIdx.x * h8;
    const int nt = blockDim.x;
    uint4 v[RMS_NV], g[RMS_NV];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < RMS_NV; ++j) {
        const int i = threadIdx.x + j * nt;
        v[j] = make_uint4(0u, 0u, 0u, 0u); g[j] = v[j];
        if (i < h8) { v[j] = xr[i]; g[j] = __ldg(w + i); }
    }
#pragma unroll
    for (int j = 0; j < RMS_NV; ++j) {
        const uint32_t* p = reinterpret_cast<const uint32_t*>(&v[j]);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float a = H::to_float(uint16_t(p[q] & 0xffff)), b = H::to_float(uint16_t(p[q] >> 16));
            ss = fmaf(a, a, ss); ss = fmaf(b, b, ss);
        }
    }
    for (int i = threadIdx.x + RMS_NV * nt; i < h8; i += nt) {          // rows longer than RMS_NV * 8 * threads values
        const uint4 t = xr[i];
        const uint32_t* p = reinterpret_cast<const uint32_t*>(&t);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float a = H::to_float(uint16_t(p[q] & 0xffff)), b = H::to_float(uint16_t(p[q] >> 16));
            ss = fmaf(a, a, ss); ss = fmaf(b, b, ss);
        }
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int q = 0; q < (nt >> 5); ++q) tot += red[q];
    const float rms = sqrtf(tot * inv_h + eps);
    auto scale_store = [&](const uint4& xv, const uint4& gv, int i) {
        const uint32_t* p = reinterpret_cast<const uint32_t*>(&xv);
        const uint32_t* pg = reinterpret_cast<const uint32_t*>(&gv);
        uint4 o; uint32_t* po = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
        for (int q = 0; q < 4; ++q)
            po[q] = H::pack(H::to_float(uint16_t(p[q] & 0xffff)) / rms * H::to_float(uint16_t(pg[q] & 0xffff)),
                            H::to_float(uint16_t(p[q] >> 16)) / rms * H::to_float(uint16_t(pg[q] >> 16)));
        out[(size_t)blockIdx.x * h8 + i] = o;
    };
#pragma unroll
    for (int j = 0; j < RMS_NV; ++j) {
        const int i = threadIdx.x + j * nt;
        if (i < h8) scale_store(v[j], g[j], i);
    }
    for (int i = threadIdx.x + RMS_NV * nt; i < h8; i += nt) scale_store(xr[i], __ldg(w + i), i);
}

// one thread per (token, head of q | k | v, pair of values)
template <typename T>
__global__ void rope_append_kernel(const uint32_t* __restrict__ qkv, const float* __restrict__ cosv, const float* __restrict__ sinv,
                                   uint32_t* __restrict__ q_out, uint32_t* __restrict__ k_cache, uint32_t* __restrict__ v_cache,
                                   int m, int hq, int hkv, int offset, const int* __restrict__ offset_dev, int capacity, int table_rows, int HALF) {
    using H = F16x2<T>;
    const int heads = hq + 2 * hkv;
    const long long total = (long long)m * heads * HALF;
    griddep_launch_dependents();
    const int off = offset_dev ? *offset_dev : offset;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int c = int(i % HALF); const int hd = int((i / HALF) % heads); const int tok = int(i / ((long long)HALF * heads));
        const int pos = off + tok;
        const uint32_t v = qkv[i];                                       // row layout [q heads | k heads | v heads] x [D]
        if (hd >= hq + hkv) {                                            // v: copy
            if (pos < capacity) v_cache[((size_t)pos * hkv + (hd - hq - hkv)) * HALF + c] = v;
            continue;
        }
        const int tp = pos < table_rows ? pos : table_rows - 1;
        const float re = H::to_float(uint16_t(v & 0xffff)), im = H::to_float(uint16_t(v >> 16));
        const float cs = cosv[(size_t)tp * HALF + c], sn = sinv[(size_t)tp * HALF + c];
        const uint32_t r = H::pack(re * cs - im * sn, im * cs + re * sn);
        if (hd < hq) q_out[((size_t)tok * hq + hd) * HALF + c] = r;
        else if (pos < capacity) k_cache[((size_t)pos * hkv + (hd - hq)) * HALF + c] = r;
    }
}

struct AttParams {
    const void* q; const void* k_cache; const void* v_cache; void* out;
    float* partial; unsigned* counters;
    const int* offset_dev;
    int m, hq, hkv, group;      // group = hq / hkv
    int offset;                 // cached positions before the first new token
    int splits, chunk;          // CTAs per (token, kv head); positions per CTA (a multiple of 32 x warps per CTA)
    int cluster;                // CTAs per thread-block cluster (divides splits)
    int max_len;                // the caller's bound on offset + m: no cache row at or beyond it is read
    float scale;
};

// NW warps per CTA: 8 (one CTA per SM, eight tiles in flight) while one cluster takes the whole sequence, 4 (two CTAs
// per SM, more and shorter ranges) beyond
template <typename T, int NW>
__global__ void __launch_bounds__(NW * 32) attention_decode_kernel(const AttParams p) {
    using H = F16x2<T>;
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ int s_last;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int split = blockIdx.x, kvh = blockIdx.y, tok = blockIdx.z;
    const int G = p.group;
    if (p.cluster > 1) cluster_arrive_relaxed();            // phase 0: "this CTA runs, its shared memory exists"
    griddep_launch_dependents();
    const int off = p.offset_dev ? *p.offset_dev : p.offset;
    const int len = min(off + tok + 1, p.max_len);          // causal: the token sees the cache and itself
    const int s0 = split * p.chunk, s1 = min(len, s0 + p.chunk);

    unsigned char* ks = smem + warp * ATT_WARP_SMEM;
    unsigned char* vs = ks + ATT_TILE * ATT_ROW;
    const uint32_t ks_a = (uint32_t)__cvta_generic_to_shared(ks), vs_a = (uint32_t)__cvta_generic_to_shared(vs);
    const unsigned char* kc = static_cast<const unsigned char*>(p.k_cache);
    const unsigned char* vc = static_cast<const unsigned char*>(p.v_cache);
    const size_t row_bytes = (size_t)p.hkv * ATT_D * 2;
    // a tile's K (or V) rows -> shared memory (16 lanes copy one 256-byte row; rows past the range: zeros); one
    // cp.async group per call, also when there is nothing to copy, so that the group count stays uniform
    auto issue = [&](int t0, const unsigned char* src, uint32_t dst) {
        if (t0 < s1) {
#pragma unroll
            for (int r = 0; r < ATT_TILE / 2; ++r) {
                const int row = 2 * r + (lane >> 4), pos = t0 + row;
                const bool live = pos < s1;
                const size_t go = (live ? (size_t)pos : 0) * row_bytes + (size_t)kvh * ATT_D * 2 + (lane & 15) * 16;
                const int sz = live ? 16 : 0;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst + row * ATT_ROW + (lane & 15) * 16), "l"(src + go), "r"(sz) : "memory");
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    int t0 = s0 + warp * ATT_TILE;
    issue(t0, kc, ks_a);
    issue(t0, vc, vs_a);

    // Tensor-core formulation (mma.sync m16n8k16, fp32 accumulate): rows = the group's query heads (8 of 16 rows
    // used), scores S = Q K^T with K rows as the col-major B operand, output O = P V with P re-used from the score
    // accumulators as the A operand and V read through ldmatrix.trans.  gq = lane / 4 is this lane's head,
    // tq = lane % 4 its column pair.
    const int gq = lane >> 2, tq = lane & 3;
    uint32_t qa[ATT_D / 16][2];                             // A fragments of Q: (head gq, d = 16 ks + 2 tq, +1) and (.., d + 8)
    {
        const uint32_t* q32 = reinterpret_cast<const uint32_t*>(p.q) + ((size_t)tok * p.hq + (size_t)kvh * G + gq) * (ATT_D / 2);
#pragma unroll
        for (int ks2 = 0; ks2 < ATT_D / 16; ++ks2) {
            qa[ks2][0] = gq < G ? __ldg(q32 + 8 * ks2 + tq) : 0u;
            qa[ks2][1] = gq < G ? __ldg(q32 + 8 * ks2 + 4 + tq) : 0u;
        }
    }
    float mx = -INFINITY, ls = 0.f;                         // running maximum and (this lane's share of) the sum of head gq
    float oc[ATT_D / 8][4];                                 // O accumulators: [jd][0..1] = (head gq, d = 8 jd + 2 tq, +1)
#pragma unroll
    for (int jd = 0; jd < ATT_D / 8; ++jd) oc[jd][0] = oc[jd][1] = oc[jd][2] = oc[jd][3] = 0.f;
    const int lm = lane >> 3, lr = lane & 7;                // ldmatrix: this lane supplies row lr of matrix lm

    for (; t0 < s1; t0 += NW * ATT_TILE) {
        // groups in flight: K of this tile, V of this tile.  K of the next tile is requested as soon as the scores are
        // done, V of the next after the weighted sum, so each copy overlaps the other half of the arithmetic.
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        __syncwarp();
        // ---- scores ----
        float sc[ATT_TILE / 8][4];
#pragma unroll
        for (int j = 0; j < ATT_TILE / 8; ++j) {
            sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f;
#pragma unroll
            for (int kk = 0; kk < ATT_D / 32; ++kk) {       // matrices: d 32 kk + (0, 8, 16, 24) of keys 8 j .. 8 j + 7
                uint32_t b0, b1, b2, b3;
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                             : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3) : "r"(ks_a + (8 * j + lr) * ATT_ROW + 64 * kk + 16 * lm));
                mma16816<T>(sc[j], qa[2 * kk][0], 0u, qa[2 * kk][1], 0u, b0, b1);
                mma16816<T>(sc[j], qa[2 * kk + 1][0], 0u, qa[2 * kk + 1][1], 0u, b2, b3);
            }
        }
        // ---- online softmax of head gq over the tile's 32 positions (8 in this lane, the rest in its quad) ----
        float mloc = -INFINITY;
#pragma unroll
        for (int j = 0; j < ATT_TILE / 8; ++j)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const bool live = t0 + 8 * j + 2 * tq + e < s1;
                sc[j][e] = live ? sc[j][e] * p.scale : -INFINITY;
                mloc = fmaxf(mloc, sc[j][e]);
            }
        mloc = fmaxf(mloc, __shfl_xor_sync(0xffffffffu, mloc, 1));
        mloc = fmaxf(mloc, __shfl_xor_sync(0xffffffffu, mloc, 2));
        const float mn = fmaxf(mx, mloc);                   // finite: position t0 is live
        const float resc = __expf(mx - mn);                 // 0 on the first tile (mx = -inf)
        mx = mn;
        float lsum = 0.f;
        uint32_t pa[ATT_TILE / 16][2];                      // A fragments of P for the two 16-position steps
#pragma unroll
        for (int j = 0; j < ATT_TILE / 8; ++j) {
            const float p0 = __expf(sc[j][0] - mn), p1 = __expf(sc[j][1] - mn);      // exp(-inf) = 0 for dead positions
            lsum += p0 + p1;
            pa[j >> 1][j & 1] = H::pack(p0, p1);
        }
        ls = ls * resc + lsum;
        __syncwarp();                                       // every lane has read its K fragments
        issue(t0 + NW * ATT_TILE, kc, ks_a);
#pragma unroll
        for (int jd = 0; jd < ATT_D / 8; ++jd) { oc[jd][0] *= resc; oc[jd][1] *= resc; }
        asm volatile("cp.async.wait_group 1;" ::: "memory"); // V of this tile (the next K may still be in flight)
        __syncwarp();
        // ---- O += P V ----
#pragma unroll
        for (int ks2 = 0; ks2 < ATT_TILE / 16; ++ks2) {
#pragma unroll
            for (int jp = 0; jp < ATT_D / 16; ++jp) {       // matrices: (keys 16 ks, d 16 jp), (keys + 8, d), (keys, d + 8), (keys + 8, d + 8)
                uint32_t b0, b1, b2, b3;
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                             : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3)
                             : "r"(vs_a + (16 * ks2 + 8 * (lm & 1) + lr) * ATT_ROW + 32 * jp + 16 * (lm >> 1)));
                mma16816<T>(oc[2 * jp], pa[ks2][0], 0u, pa[ks2][1], 0u, b0, b1);
                mma16816<T>(oc[2 * jp + 1], pa[ks2][0], 0u, pa[ks2][1], 0u, b2, b3);
            }
        }
        __syncwarp();                                       // every lane is done with the V tile before it is overwritten
        issue(t0 + NW * ATT_TILE, vc, vs_a);
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");

    // ---- the CTA's warps -> one partial per query head (merged in warp order); a warp parks its partial in its own
    //      (now idle) tile buffer ----
    auto part = [&](int w, int h) -> float* { return reinterpret_cast<float*>(smem + w * ATT_WARP_SMEM) + h * ATT_PART; };
    __syncwarp();
    ls += __shfl_xor_sync(0xffffffffu, ls, 1);
    ls += __shfl_xor_sync(0xffffffffu, ls, 2);
    if (gq < G) {
        if (tq == 0) { part(warp, gq)[ATT_D] = mx; part(warp, gq)[ATT_D + 1] = ls; }
#pragma unroll
        for (int jd = 0; jd < ATT_D / 8; ++jd)
            *reinterpret_cast<float2*>(&part(warp, gq)[8 * jd + 2 * tq]) = make_float2(oc[jd][0], oc[jd][1]);
    }
    __syncthreads();
    // thread -> dimension d of every ATT_HS-th query head: first the CTA's warps, then (through the cluster's shared
    // memory) the CTAs of the cluster, then (through global memory, last CTA to arrive) the clusters
    constexpr int ATT_HS = NW * 32 / ATT_D;          // threads per dimension: each takes the heads hh, hh + ATT_HS, ...
    constexpr int NH = ATT_MAXG / ATT_HS;
    const int d = tid & (ATT_D - 1), hh = tid / ATT_D;
    const int C = p.cluster;
    const int crank = C > 1 ? split % C : 0, cl = split / C, ncl = p.splits / C;
    float* xred = reinterpret_cast<float*>(smem + NW * ATT_WARP_SMEM);      // [C][G][ATT_PART], used in cluster rank 0
    auto merge_store = [&](int h, float l_all, float a_all) {
        reinterpret_cast<uint16_t*>(p.out)[((size_t)tok * p.hq + (size_t)kvh * G + h) * ATT_D + d] = H::from_float(l_all > 0.f ? a_all / l_all : 0.f);
    };
    float m_c[NH], l_c[NH], a_c[NH];
#pragma unroll
    for (int hi = 0; hi < NH; ++hi) {
        const int h = hi * ATT_HS + hh;
        m_c[hi] = -INFINITY; l_c[hi] = 0.f; a_c[hi] = 0.f;
        if (h < G) {
#pragma unroll
            for (int w = 0; w < NW; ++w) m_c[hi] = fmaxf(m_c[hi], part(w, h)[ATT_D]);
#pragma unroll
            for (int w = 0; w < NW; ++w) {
                const float f = part(w, h)[ATT_D] == -INFINITY ? 0.f : __expf(part(w, h)[ATT_D] - m_c[hi]);
                l_c[hi] = fmaf(part(w, h)[ATT_D + 1], f, l_c[hi]);
                a_c[hi] = fmaf(part(w, h)[d], f, a_c[hi]);
            }
        }
    }
    if (C > 1) {
        cluster_wait_acquire();                             // phase 0 complete: rank 0 of the cluster is resident
#pragma unroll
        for (int hi = 0; hi < NH; ++hi) {
            const int h = hi * ATT_HS + hh;
            if (h < G) {
                float* row = xred + ((size_t)crank * ATT_MAXG + h) * ATT_PART;
                st_cluster_f32(row + d, 0u, a_c[hi]);
                if (d == 0) { st_cluster_f32(row + ATT_D, 0u, m_c[hi]); st_cluster_f32(row + ATT_D + 1, 0u, l_c[hi]); }
            }
        }
        cluster_arrive_release();
        cluster_wait_acquire();
        if (crank != 0) return;
#pragma unroll
        for (int hi = 0; hi < NH; ++hi) {
            const int h = hi * ATT_HS + hh;
            if (h < G) {
                float mm = -INFINITY;
                for (int r = 0; r < C; ++r) mm = fmaxf(mm, xred[((size_t)r * ATT_MAXG + h) * ATT_PART + ATT_D]);
                float ll = 0.f, aa = 0.f;
                for (int r = 0; r < C; ++r) {               // in rank order: the result does not depend on arrival order
                    const float* row = xred + ((size_t)r * ATT_MAXG + h) * ATT_PART;
                    const float f = row[ATT_D] == -INFINITY ? 0.f : __expf(row[ATT_D] - mm);
                    ll = fmaf(row[ATT_D + 1], f, ll);
                    aa = fmaf(row[d], f, aa);
                }
                m_c[hi] = mm; l_c[hi] = ll; a_c[hi] = aa;
            }
        }
    }
    if (ncl == 1) {
#pragma unroll
        for (int hi = 0; hi < NH; ++hi)
            if (hi * ATT_HS + hh < G) merge_store(hi * ATT_HS + hh, l_c[hi], a_c[hi]);
        return;
    }
    const size_t slot = ((size_t)tok * p.hkv + kvh) * ncl;
#pragma unroll
    for (int hi = 0; hi < NH; ++hi) {
        const int h = hi * ATT_HS + hh;
        if (h < G) {
            float* dst = p.partial + ((slot + cl) * ATT_MAXG + h) * ATT_PART;
            if (d == 0) { __stcg(dst + ATT_D, m_c[hi]); __stcg(dst + ATT_D + 1, l_c[hi]); }
            __stcg(dst + d, a_c[hi]);
        }
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = (atomicAdd(p.counters + tok * p.hkv + kvh, 1u) == unsigned(ncl - 1));
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // warp w merges query head w (w + NW, ...), a lane four dimensions: every load of a head is in flight at once
#pragma unroll 1
    for (int h = warp; h < G; h += NW) {
        const float* src = p.partial + (slot * ATT_MAXG + h) * ATT_PART;
        float ms[ATT_MAXCL], lv[ATT_MAXCL]; float4 av[ATT_MAXCL];
#pragma unroll
        for (int c = 0; c < ATT_MAXCL; ++c) {
            const bool on = c < ncl;
            const float* s2 = src + (size_t)(on ? c : 0) * ATT_MAXG * ATT_PART;
            ms[c] = on ? __ldcg(s2 + ATT_D) : -INFINITY;
            lv[c] = on ? __ldcg(s2 + ATT_D + 1) : 0.f;
            av[c] = on ? __ldcg(reinterpret_cast<const float4*>(s2) + lane) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        float mm = -INFINITY;
#pragma unroll
        for (int c = 0; c < ATT_MAXCL; ++c) mm = fmaxf(mm, ms[c]);
        float ll = 0.f; float4 aa = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int c = 0; c < ATT_MAXCL; ++c) {               // in cluster order
            const float f = ms[c] == -INFINITY ? 0.f : __expf(ms[c] - mm);
            ll = fmaf(lv[c], f, ll);
            aa.x = fmaf(av[c].x, f, aa.x); aa.y = fmaf(av[c].y, f, aa.y); aa.z = fmaf(av[c].z, f, aa.z); aa.w = fmaf(av[c].w, f, aa.w);
        }
        const float inv = ll > 0.f ? 1.f / ll : 0.f;
        uint2 o; o.x = H::pack(aa.x * inv, aa.y * inv); o.y = H::pack(aa.z * inv, aa.w * inv);
        *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(p.out) + ((size_t)tok * p.hq + (size_t)kvh * G + h) * ATT_D + lane * 4) = o;
    }
    if (tid == 0) p.counters[tok * p.hkv + kvh] = 0;
}

// CTAs per (token, kv head) = clusters x cluster size; positions per CTA.  Up to ATT_CLUSTER * ATT_PER_SINGLE tiles
// one cluster takes the whole sequence, its CTAs a few tiles per warp, and everything merges through shared memory
// (the global stage costs ~7 us: partials, fence, counter, read back); longer sequences use up to ATT_MAXCL clusters.
void attention_plan(int max_len, int& splits, int& chunk, int& cluster, int& warps) {
    warps = 8;
    int tile = warps * ATT_TILE;
    int tiles = (max_len + tile - 1) / tile;
    if (tiles < 1) tiles = 1;
    if (tiles <= ATT_CLUSTER) { cluster = tiles; splits = tiles; chunk = tile; return; }
    cluster = ATT_CLUSTER;
    if (tiles <= ATT_CLUSTER * ATT_PER_SINGLE) { splits = ATT_CLUSTER; chunk = (tiles + splits - 1) / splits * tile; return; }
    warps = 4;
    tile = warps * ATT_TILE;
    tiles = (max_len + tile - 1) / tile;
    int ncl = (tiles + ATT_CLUSTER * ATT_PER_SINGLE - 1) / (ATT_CLUSTER * ATT_PER_SINGLE);
    if (ncl > ATT_MAXCL) ncl = ATT_MAXCL;
    splits = ncl * ATT_CLUSTER;
    const int per = (tiles + splits - 1) / splits;
    chunk = per * tile;
}

}  // namespace

// Plain stream-ordered launches of kernels that release their programmatic dependents at once: a linear that follows
// with MT_FLAG_PDL becomes resident and prefetches its weights while the small kernel runs (it waits for the
// kernel's completion before it touches the activations).  Launching THESE kernels as programmatic dependents as
// well was measured and lost: CTAs of the following linears then become resident two and three kernels ahead and
// a Llama-3-70B layer took 116 us instead of 109 (same GPU, alternating runs); without the early release 113.
template <typename... KArgs, typename... Args>
static int launch_plain(void (*kern)(KArgs...), dim3 grid, dim3 block, cudaStream_t st, Args... args) {
    kern<<<grid, block, 0, st>>>(static_cast<KArgs>(args)...);
    return cudaGetLastError() == cudaSuccess ? MT_OK : MT_ERR_CUDA;
}

int launch_rms_norm(cudaStream_t st, const void* x, const void* w, void* out, int rows, int h, float eps, int dtype) {
    const int h8 = h / 8;
    int threads = (h8 + 31) / 32 * 32;                      // one 16-byte piece per thread up to 8192 values
    if (threads > 1024) threads = 1024;
    if (dtype == MT_F16)
        return launch_plain(rms_norm_kernel<__half>, dim3(rows), dim3(threads), st, static_cast<const uint4*>(x), static_cast<const uint4*>(w),
                          static_cast<uint4*>(out), h8, 1.f / h, eps);
    return launch_plain(rms_norm_kernel<__nv_bfloat16>, dim3(rows), dim3(threads), st, static_cast<const uint4*>(x), static_cast<const uint4*>(w),
                      static_cast<uint4*>(out), h8, 1.f / h, eps);
}

int launch_rope_append(cudaStream_t st, const void* qkv, const float* cosv, const float* sinv, void* q_out, void* k_cache, void* v_cache,
                       int m, int hq, int hkv, int d, int offset, const int* offset_dev, int capacity, int table_rows, int dtype) {
    const long long total = (long long)m * (hq + 2 * hkv) * (d / 2);
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    if (dtype == MT_F16)
        return launch_plain(rope_append_kernel<__half>, dim3((unsigned)blocks), dim3(256), st, static_cast<const uint32_t*>(qkv), cosv, sinv,
                          static_cast<uint32_t*>(q_out), static_cast<uint32_t*>(k_cache), static_cast<uint32_t*>(v_cache), m, hq, hkv, offset,
                          offset_dev, capacity, table_rows, d / 2);
    return launch_plain(rope_append_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(256), st, static_cast<const uint32_t*>(qkv), cosv, sinv,
                      static_cast<uint32_t*>(q_out), static_cast<uint32_t*>(k_cache), static_cast<uint32_t*>(v_cache), m, hq, hkv, offset,
                      offset_dev, capacity, table_rows, d / 2);
}

size_t attention_workspace_bytes(int m, int hkv, int max_len) {
    int splits, chunk, cluster, warps;
    attention_plan(max_len, splits, chunk, cluster, warps);
    const size_t counters = (((size_t)m * hkv * 4) + 255) & ~(size_t)255;
    return counters + (size_t)m * hkv * (splits / cluster) * ATT_MAXG * ATT_PART * 4;
}

template <typename T, int NW>
static int launch_attention_inst(cudaStream_t st, const AttParams& p, dim3 grid) {
    auto kern = attention_decode_kernel<T, NW>;
    // the K / V tiles of the warps, then the cluster's merge rows (always ATT_CLUSTER of them: one attribute value)
    const size_t smem = (size_t)NW * ATT_WARP_SMEM + (size_t)ATT_CLUSTER * ATT_MAXG * ATT_PART * 4;
    static bool configured[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { cudaGetLastError(); return MT_ERR_CUDA; }
    if (!configured[dev]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) { cudaGetLastError(); return MT_ERR_CUDA; }
        configured[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = dim3(NW * 32); cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = p.cluster; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = p.cluster > 1 ? 1 : 0;
    if (cudaLaunchKernelEx(&cfg, kern, p) != cudaSuccess) { cudaGetLastError(); return MT_ERR_CUDA; }
    return MT_OK;
}

int launch_attention_decode(cudaStream_t st, const void* q, const void* k_cache, const void* v_cache, void* out,
                            int m, int hq, int hkv, int d, int offset, const int* offset_dev, int max_len, float scale,
                            void* workspace, size_t workspace_bytes, int dtype) {
    if (d != ATT_D || hkv < 1 || hq % hkv != 0 || hq / hkv > ATT_MAXG) return MT_ERR_UNSUPPORTED;
    AttParams p;
    p.q = q; p.k_cache = k_cache; p.v_cache = v_cache; p.out = out;
    p.m = m; p.hq = hq; p.hkv = hkv; p.group = hq / hkv; p.offset = offset; p.offset_dev = offset_dev; p.scale = scale;
    int warps;
    attention_plan(max_len, p.splits, p.chunk, p.cluster, warps);
    p.max_len = max_len;
    if (attention_workspace_bytes(m, hkv, max_len) > workspace_bytes) return MT_ERR_WORKSPACE;
    const size_t counters = (((size_t)m * hkv * 4) + 255) & ~(size_t)255;
    p.counters = static_cast<unsigned*>(workspace);
    p.partial = reinterpret_cast<float*>(static_cast<char*>(workspace) + counters);
    const dim3 grid(p.splits, hkv, m);
    if (dtype == MT_F16) return warps == 8 ? launch_attention_inst<__half, 8>(st, p, grid) : launch_attention_inst<__half, 4>(st, p, grid);
    return warps == 8 ? launch_attention_inst<__nv_bfloat16, 8>(st, p, grid) : launch_attention_inst<__nv_bfloat16, 4>(st, p, grid);
}

// ----------------------------------------------------------------------------------------------
// Attention for prefill-sized and multi-sequence batches, any head size that is a multiple of 32 up to 256:
//   out[b, i, n, :] = softmax_t(q[b, i, n, :] . k[b, t, n / group, :] * scale, t <= offset_b + i) @ v[b, :, n / group, :]
// (examples/llama3_70b.py:103-115: scores for every (query, key) pair, -inf above the diagonal shifted by the cached
// positions, softmax over the keys, weighted sum of the values).  One warp per (sequence, head, four query positions): a
// lane scores one key of a block of 32 against the four scaled query rows in shared memory (whole dot products), each
// row's block maximum and sum update its running softmax, then every lane adds its d / 32 output values of the 32
// weighted value rows to the four rows; a key or value row is read once for the four.  fp32
// throughout, one rounding at the end (the reference rounds scores, scaled scores, probabilities and output separately).
// ----------------------------------------------------------------------------------------------
struct AttRowsParams {
    const void* q; const void* k_cache; const void* v_cache; void* out;
    const int* offsets;         // [batch] cached positions before the first new token of each sequence, or null: `offset` for all
    int batch, m, hq, hkv, d, offset, capacity;
    float scale;
};

constexpr int ATR_WARPS = 4;
constexpr int ATR_ROWS = 4;     // consecutive query positions per warp: every key and value row is read once for the four
constexpr int ATR_MAXE = 8;     // d / 32 <= 8

template <typename T>
__global__ void __launch_bounds__(ATR_WARPS * 32) attention_rows_kernel(const AttRowsParams p) {
    using H = F16x2<T>;
    __shared__ float qs[ATR_WARPS][ATR_ROWS][256];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int i0 = (blockIdx.x * ATR_WARPS + warp) * ATR_ROWS;      // first query position of this warp
    const int n = blockIdx.y, b = blockIdx.z;
    if (i0 >= p.m) return;                                // whole warps leave together: no block-wide barrier below
    const int d = p.d, E = d >> 5;
    const int kvh = n / (p.hq / p.hkv);
    const int off = p.offsets ? p.offsets[b] : p.offset;
    const int rows = min(ATR_ROWS, p.m - i0);
    int nk[ATR_ROWS];                                     // the causal mask: row r sees keys 0 .. off + i0 + r
#pragma unroll
    for (int r = 0; r < ATR_ROWS; ++r) nk[r] = r < rows ? min(off + i0 + r + 1, p.capacity) : 0;
    const int nkeys = nk[rows - 1];
#pragma unroll
    for (int r = 0; r < ATR_ROWS; ++r) {
        const uint16_t* q = reinterpret_cast<const uint16_t*>(p.q) + (((size_t)b * p.m + min(i0 + r, p.m - 1)) * p.hq + n) * d;
        for (int e = lane; e < d; e += 32) qs[warp][r][e] = H::to_float(q[e]) * p.scale;
    }
    __syncwarp();
    const size_t row = (size_t)p.hkv * d;                 // elements between cache positions
    const uint16_t* kb = reinterpret_cast<const uint16_t*>(p.k_cache) + ((size_t)b * p.capacity * p.hkv + kvh) * d;
    const uint16_t* vb = reinterpret_cast<const uint16_t*>(p.v_cache) + ((size_t)b * p.capacity * p.hkv + kvh) * d;
    float acc[ATR_ROWS][ATR_MAXE];
    float mx[ATR_ROWS], l[ATR_ROWS];
#pragma unroll
    for (int r = 0; r < ATR_ROWS; ++r) {
        mx[r] = -INFINITY; l[r] = 0.f;
#pragma unroll
        for (int e = 0; e < ATR_MAXE; ++e) acc[r][e] = 0.f;
    }
    for (int t0 = 0; t0 < nkeys; t0 += 32) {
        const int t = t0 + lane;
        float dot[ATR_ROWS];
#pragma unroll
        for (int r = 0; r < ATR_ROWS; ++r) dot[r] = 0.f;
        if (t < nkeys) {
            const uint4* kr = reinterpret_cast<const uint4*>(kb + (size_t)t * row);
            for (int c = 0; c < d / 8; ++c) {
                const uint4 kv = __ldg(kr + c);
                const uint32_t w[4] = {kv.x, kv.y, kv.z, kv.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float k0 = H::to_float(uint16_t(w[j] & 0xffff)), k1 = H::to_float(uint16_t(w[j] >> 16));
#pragma unroll
                    for (int r = 0; r < ATR_ROWS; ++r) dot[r] = fmaf(qs[warp][r][c * 8 + 2 * j + 1], k1, fmaf(qs[warp][r][c * 8 + 2 * j], k0, dot[r]));
                }
            }
        }
        float pr[ATR_ROWS];
#pragma unroll
        for (int r = 0; r < ATR_ROWS; ++r) {
            const float sc = t < nk[r] ? dot[r] : -INFINITY;
            float bm = sc;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, o));
            const float mnew = fmaxf(mx[r], bm);
            // a row whose keys all lie before this block (or a padding row) keeps -inf here: no change, no NaN
            const float corr = mnew == -INFINITY ? 1.f : __expf(mx[r] - mnew);
            pr[r] = t < nk[r] ? __expf(sc - mnew) : 0.f;
            float ps = pr[r];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
            l[r] = l[r] * corr + ps;
#pragma unroll
            for (int e = 0; e < ATR_MAXE; ++e) acc[r][e] *= corr;
            mx[r] = mnew;
        }
        const int cnt = min(32, nkeys - t0);
        for (int j = 0; j < cnt; ++j) {
            const uint16_t* vr = vb + (size_t)(t0 + j) * row + lane * E;
            float vv[ATR_MAXE];
#pragma unroll
            for (int e = 0; e < ATR_MAXE; ++e) vv[e] = e < E ? H::to_float(vr[e]) : 0.f;
#pragma unroll
            for (int r = 0; r < ATR_ROWS; ++r) {
                const float pj = __shfl_sync(0xffffffffu, pr[r], j);
#pragma unroll
                for (int e = 0; e < ATR_MAXE; ++e) acc[r][e] = fmaf(pj, vv[e], acc[r][e]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < ATR_ROWS; ++r) {
        if (r < rows) {
            uint16_t* o = reinterpret_cast<uint16_t*>(p.out) + (((size_t)b * p.m + i0 + r) * p.hq + n) * d + lane * E;
            const float inv = 1.f / l[r];
#pragma unroll
            for (int e = 0; e < ATR_MAXE; ++e)
                if (e < E) o[e] = H::from_float(acc[r][e] * inv);
        }
    }
}

int launch_attention_rows(cudaStream_t st, const void* q, const void* k_cache, const void* v_cache, void* out, const int* offsets,
                          int batch, int m, int hq, int hkv, int d, int offset, int capacity, float scale, int dtype) {
    if (d % 32 != 0 || d < 32 || d > 256 || hkv < 1 || hq % hkv != 0) return MT_ERR_UNSUPPORTED;
    if (batch > 65535 || hq > 65535) return MT_ERR_TOO_LARGE;
    AttRowsParams p;
    p.q = q; p.k_cache = k_cache; p.v_cache = v_cache; p.out = out; p.offsets = offsets;
    p.batch = batch; p.m = m; p.hq = hq; p.hkv = hkv; p.d = d; p.offset = offset; p.capacity = capacity; p.scale = scale;
    const dim3 grid((m + ATR_WARPS * ATR_ROWS - 1) / (ATR_WARPS * ATR_ROWS), hq, batch);
    if (dtype == MT_F16) attention_rows_kernel<__half><<<grid, ATR_WARPS * 32, 0, st>>>(p);
    else attention_rows_kernel<__nv_bfloat16><<<grid, ATR_WARPS * 32, 0, st>>>(p);
    return cudaGetLastError() == cudaSuccess ? MT_OK : MT_ERR_CUDA;
}

}  // namespace mt
