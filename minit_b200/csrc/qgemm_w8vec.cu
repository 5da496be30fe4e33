// Decode GEMV (M <= 2) for int8 weights kept as plain int8 [K,N] with one scale per output channel:
// out[M,N] = (x[M,K] @ float(w[K,N])) * scales[N] (+ bias).  The G = 1, stored-zero = 127 special case of
// the GPTQ formula (minit/quantize/dispatch.py:14-20) on the layout a plain int8 checkpoint has.
//
// The same idea as the GPTQ-layout GEMV, turned by ninety degrees: a 32-bit word of a row holds four
// adjacent COLUMNS of one k, so (w ^ 0x80808080) & 0x00ff00ff read as f16x2 is (w_n + 128, w_{n+2} + 128)
// * 2^-24 (fp16 subnormals), one XOR-AND (a single LOP3) and one fma.rn.f16x2 per two weights against
// the block-scaled activation of that row broadcast into both halves.  Accumulators (one f16x2 per
// column pair, two alternating sets) see 8 additions per chunk of 16 rows and are then folded in fp32:
//     acc[n] += 2^(24-e) * sum_k (w + 128) x'  -  128 * sum_k x;      out[n] = scales[n] * acc[n] (+ bias)
// A lane owns 8 adjacent columns (8-byte loads, 256 contiguous bytes per warp and row, 16 rows in
// flight per thread), a warp a contiguous run of rows, a CTA 8 such runs of one 256-column block;
// split-K across the CTAs of a thread-block cluster (DSMEM) or, beyond 8 splits, through global memory.
#include "common.cuh"

namespace mt {
namespace {

constexpr int W8V_THREADS = 256;
constexpr int W8V_WARPS = 8;
constexpr int W8V_COLS = 256;     // columns per CTA
constexpr int W8V_D = 16;         // rows in flight per thread
constexpr int W8V_CK = 16;        // rows per fold chunk

struct W8VParams {
    const void* x; const int8_t* w; const void* scales; const void* bias; void* out;
    unsigned* counters; float* partial;
    int m, n, k;
    int nchunks;      // K / 16
    int units;        // splits * 8 warp runs
    int splits;
    int slice_chunks; // chunks of shared memory per warp and batch row (multiple of 2)
    int pdl, cluster;
};

// (a ^ b) & c
__device__ __forceinline__ uint32_t xor_and(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d; asm("lop3.b32 %0, %1, %2, %3, 0x28;" : "=r"(d) : "r"(a), "r"(b), "r"(c)); return d; }
template <typename T, int MB>
__global__ void __launch_bounds__(W8V_THREADS, 2) qgemm_w8vec_kernel(const W8VParams p) {
    using H = F16x2<T>;
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ __align__(16) float red[W8V_WARPS * MB * W8V_COLS];
    __shared__ __align__(16) float xred[8 * MB * W8V_COLS];
    __shared__ int s_last;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tile = blockIdx.x, split = blockIdx.y;
    const int col = tile * W8V_COLS + lane * 8;
    if (p.cluster) cluster_arrive_relaxed();

    const int u = split * W8V_WARPS + warp;
    const int c_lo = int((long long)u * p.nchunks / p.units);
    const int c_hi = int((long long)(u + 1) * p.nchunks / p.units);
    const int nrows = (c_hi - c_lo) * W8V_CK;
    const size_t rstride = size_t(p.n) / 8;     // uint2 per row
    const uint2* wp = reinterpret_cast<const uint2*>(p.w + (size_t)c_lo * W8V_CK * p.n + col);

    // ---- prologue: the weights do not depend on the previous kernel ----
    uint2 w[W8V_D];
#pragma unroll
    for (int i = 0; i < W8V_D; ++i) w[i] = i < nrows ? ldg_stream8(wp + i * rstride) : make_uint2(0x80808080u, 0x80808080u);
    const uint2* wnext = wp + W8V_D * rstride;

    if (p.pdl) { griddep_launch_dependents(); griddep_wait(); }

    // ---- stage the activations of this warp's run: block-scaled per chunk of 16, both halves equal ----
    // layout per (batch row, chunk): 16 x f16x2 (x', x') = 64 bytes, then meta (2^(24-e), sum of x)
    uint32_t* xs = reinterpret_cast<uint32_t*>(smem) + (size_t)warp * MB * p.slice_chunks * 16;
    float2* meta = reinterpret_cast<float2*>(smem + (size_t)W8V_WARPS * MB * p.slice_chunks * 64) + (size_t)warp * MB * p.slice_chunks;
    const T* xg = reinterpret_cast<const T*>(p.x);
#pragma unroll
    for (int mb = 0; mb < MB; ++mb) {
        for (int i = 0; i < p.slice_chunks; i += 2) {           // 32 lanes = 2 chunks of 16 values
            const int ch = i + (lane >> 4);
            const bool live = mb < p.m && ch < c_hi - c_lo;
            float f = 0.f;
            if (live) f = H::to_float(reinterpret_cast<const uint16_t*>(xg)[(size_t)mb * p.k + (size_t)(c_lo + ch) * W8V_CK + (lane & 15)]);
            float amax = fabsf(f), sum = f;
#pragma unroll
            for (int o = 1; o < 16; o <<= 1) {
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
                sum += __shfl_xor_sync(0xffffffffu, sum, o);
            }
            int e = 0;                                            // x' = x * 2^e has its chunk maximum in [2^14, 2^15)
            if (amax > 0.f && amax < 3.0e38f) e = 14 - (int((__float_as_uint(amax) >> 23) & 0xff) - 127);
            e = e < -100 ? -100 : (e > 100 ? 100 : e);
            const float up = __uint_as_float(uint32_t(127 + e) << 23);
            const float post = __uint_as_float(uint32_t(127 + 24 - e) << 23);
            const __half2 h = __float2half2_rn(f * up);
            if (ch < p.slice_chunks) {
                xs[((size_t)mb * p.slice_chunks + ch) * 16 + (lane & 15)] = *reinterpret_cast<const uint32_t*>(&h);
                if ((lane & 15) == 0) meta[(size_t)mb * p.slice_chunks + ch] = make_float2(post, sum);
            }
        }
    }
    __syncwarp();

    // ---- main loop: one chunk of 16 rows per trip, 8 columns per lane ----
    float acc[MB][8];
#pragma unroll
    for (int mb = 0; mb < MB; ++mb)
#pragma unroll
        for (int c = 0; c < 8; ++c) acc[mb][c] = 0.f;
    int row = 0;
    for (int ch = 0; ch < c_hi - c_lo; ++ch) {
        uint32_t a[MB][2][4];                                      // [set][column pair]: pairs (0,2) (1,3) (4,6) (5,7)
#pragma unroll
        for (int r = 0; r < W8V_CK; ++r) {
            const uint2 wv = w[r];
            w[r] = (row + W8V_D < nrows) ? ldg_stream8(wnext) : make_uint2(0x80808080u, 0x80808080u);
            wnext += rstride;
            ++row;
            const int set = r & 1;
            const uint32_t q0 = xor_and(wv.x, 0x80808080u, 0x00ff00ffu), q1 = xor_and(wv.x >> 8, 0x00808080u, 0x00ff00ffu);
            const uint32_t q2 = xor_and(wv.y, 0x80808080u, 0x00ff00ffu), q3 = xor_and(wv.y >> 8, 0x00808080u, 0x00ff00ffu);
#pragma unroll
            for (int mb = 0; mb < MB; ++mb) {
                const uint32_t x2 = xs[((size_t)mb * p.slice_chunks + ch) * 16 + r];
                if (r < 2) {
                    a[mb][set][0] = hmul2(q0, x2); a[mb][set][1] = hmul2(q1, x2);
                    a[mb][set][2] = hmul2(q2, x2); a[mb][set][3] = hmul2(q3, x2);
                } else {
                    a[mb][set][0] = hfma2(q0, x2, a[mb][set][0]); a[mb][set][1] = hfma2(q1, x2, a[mb][set][1]);
                    a[mb][set][2] = hfma2(q2, x2, a[mb][set][2]); a[mb][set][3] = hfma2(q3, x2, a[mb][set][3]);
                }
            }
        }
#pragma unroll
        for (int mb = 0; mb < MB; ++mb) {
            const float2 mt2 = meta[(size_t)mb * p.slice_chunks + ch];      // (2^(24-e), sum of x)
            const float zs = 128.f * mt2.y;
#pragma unroll
            for (int pr = 0; pr < 4; ++pr) {
                const uint32_t hsum = hadd2(a[mb][0][pr], a[mb][1][pr]);
                const __half2 hv = *reinterpret_cast<const __half2*>(&hsum);
                // pair pr of word (pr >> 1): columns (4 * (pr >> 1) + (pr & 1)) and the same + 2
                const int c0 = 4 * (pr >> 1) + (pr & 1);
                acc[mb][c0] += fmaf(__low2float(hv), mt2.x, -zs);
                acc[mb][c0 + 2] += fmaf(__high2float(hv), mt2.x, -zs);
            }
        }
    }

    // ---- reduce the 8 warps of the CTA, then the splits ----
#pragma unroll
    for (int mb = 0; mb < MB; ++mb) {
        float* dst = red + ((size_t)warp * MB + mb) * W8V_COLS + lane * 8;
        *reinterpret_cast<float4*>(dst) = make_float4(acc[mb][0], acc[mb][1], acc[mb][2], acc[mb][3]);
        *reinterpret_cast<float4*>(dst + 4) = make_float4(acc[mb][4], acc[mb][5], acc[mb][6], acc[mb][7]);
    }
    __syncthreads();
    const T* sc = reinterpret_cast<const T*>(p.scales);
    const T* bias = reinterpret_cast<const T*>(p.bias);
    uint16_t* out = reinterpret_cast<uint16_t*>(p.out);
    // thread tid owns column tid of the block, for every batch row
    const int gc = tile * W8V_COLS + tid;
    float v[MB];
#pragma unroll
    for (int mb = 0; mb < MB; ++mb) {
        v[mb] = 0.f;
#pragma unroll
        for (int wi = 0; wi < W8V_WARPS; ++wi) v[mb] += red[((size_t)wi * MB + mb) * W8V_COLS + tid];
    }
    if (p.splits > 1 && p.cluster) {
        cluster_wait_acquire();
#pragma unroll
        for (int mb = 0; mb < MB; ++mb) st_cluster_f32(xred + ((size_t)split * MB + mb) * W8V_COLS + tid, 0u, v[mb]);
        cluster_arrive_release();
        cluster_wait_acquire();
        if (split != 0) return;
#pragma unroll
        for (int mb = 0; mb < MB; ++mb) {
            v[mb] = 0.f;
            for (int s = 0; s < p.splits; ++s) v[mb] += xred[((size_t)s * MB + mb) * W8V_COLS + tid];
        }
    } else if (p.splits > 1) {
#pragma unroll
        for (int mb = 0; mb < MB; ++mb)
            if (mb < p.m) __stcg(p.partial + ((size_t)split * p.m + mb) * p.n + gc, v[mb]);
        __threadfence();
        __syncthreads();
        if (tid == 0) s_last = (atomicAdd(p.counters + tile, 1u) == unsigned(p.splits - 1));
        __syncthreads();
        if (!s_last) return;
        __threadfence();
#pragma unroll
        for (int mb = 0; mb < MB; ++mb) {
            v[mb] = 0.f;
            if (mb < p.m)
                for (int s = 0; s < p.splits; ++s) v[mb] += __ldcg(p.partial + ((size_t)s * p.m + mb) * p.n + gc);
        }
        if (tid == 0) p.counters[tile] = 0;
    }
    const float s = H::to_float(reinterpret_cast<const uint16_t*>(sc)[gc]);
    const float b = bias ? H::to_float(reinterpret_cast<const uint16_t*>(bias)[gc]) : 0.f;
#pragma unroll
    for (int mb = 0; mb < MB; ++mb)
        if (mb < p.m) out[(size_t)mb * p.n + gc] = H::from_float(fmaf(v[mb], s, b));
}

template <typename T, int MB>
int launch_one(cudaStream_t st, const W8VParams& p, dim3 grid, size_t smem) {
    auto kern = qgemm_w8vec_kernel<T, MB>;
    static bool configured[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { cudaGetLastError(); return MT_ERR_CUDA; }
    if (!configured[dev]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 1024) != cudaSuccess) { cudaGetLastError(); return MT_ERR_CUDA; }
        configured[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = dim3(W8V_THREADS); cfg.dynamicSmemBytes = smem; cfg.stream = st;
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

}  // namespace

bool w8vec_supported(const QGemmArgs& a) {
    if (a.m < 1 || a.m > 2 || a.n % W8V_COLS != 0 || a.k % W8V_CK != 0) return false;
    if (a.n / W8V_COLS >= kMaxTiles - 1) return false;
    return a.workspace != nullptr && a.workspace_bytes >= kCounterBytes;
}

int launch_w8vec(cudaStream_t st, const QGemmArgs& a) {
    if (!w8vec_supported(a)) return MT_ERR_UNSUPPORTED;
    const int nchunks = a.k / W8V_CK;
    const int tiles = a.n / W8V_COLS;
    // split-K: one wave of CTAs (2 per SM; clusters of up to 8 keep the hand-over in shared memory), every
    // warp at least 2 chunks and at most 2048 rows (its activations live in shared memory)
    int max_splits = nchunks / (W8V_WARPS * 2);
    if (max_splits < 1) max_splits = 1;
    const size_t cap = (a.workspace_bytes - kCounterBytes) / ((size_t)a.m * a.n * 4);
    const int min_splits = (a.k + W8V_WARPS * 2048 - 1) / (W8V_WARPS * 2048);
    int splits = 256 / tiles;
    if (splits > 8) splits = 8;
    if (splits > max_splits) splits = max_splits;
    if (splits < min_splits) splits = min_splits;
    if (splits < 1) splits = 1;
    if (splits > 8 && (size_t)splits > cap) return MT_ERR_WORKSPACE;
    W8VParams p;
    p.x = a.x; p.w = a.w8; p.scales = a.scales; p.bias = a.bias; p.out = a.out;
    p.counters = static_cast<unsigned*>(a.workspace);
    p.partial = reinterpret_cast<float*>(static_cast<char*>(a.workspace) + kCounterBytes);
    p.m = a.m; p.n = a.n; p.k = a.k;
    p.nchunks = nchunks; p.splits = splits; p.units = splits * W8V_WARPS;
    int slice = (nchunks + p.units - 1) / p.units;
    slice = (slice + 1) & ~1;
    p.slice_chunks = slice;
    p.pdl = (a.flags & MT_FLAG_PDL) ? 1 : 0;
    p.cluster = (splits >= 2 && splits <= 8) ? 1 : 0;
    const int mb = a.m == 1 ? 1 : 2;
    const size_t smem = (size_t)W8V_WARPS * mb * slice * 64 + (size_t)W8V_WARPS * mb * slice * 8;
    if (smem > 128 * 1024) return MT_ERR_TOO_LARGE;
    const dim3 grid(tiles, splits);
    if (a.dtype == MT_F16) return mb == 1 ? launch_one<__half, 1>(st, p, grid, smem) : launch_one<__half, 2>(st, p, grid, smem);
    return mb == 1 ? launch_one<__nv_bfloat16, 1>(st, p, grid, smem) : launch_one<__nv_bfloat16, 2>(st, p, grid, smem);
}

}  // namespace mt
