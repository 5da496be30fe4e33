// Prefill-sized fused dequant + GEMM on the 5th-generation tensor cores (tcgen05 + TMEM).
//
// Roofline: dense fp16/bf16 tensor throughput.
//
// out^T tile = W^T tile x x^T tile:  the 128 output columns of a tile are the MMA "M" rows
// (TMEM lanes), BM batch rows are the MMA "N" columns, so one dequantised 128 x 64 weight tile
// feeds BM = 256 batch rows per k-block and the CUDA-core dequant cost is amortised 256 ways.
//
// Per CTA (persistent, one per SM, 320 threads):
//   warp 0      TMA producer: per k-block (64 k) one 2-D bulk tensor load of the packed qweight
//               rows [64/pack, 128 columns] (plain layout) and one of the x tile [BM, 64]
//               (128-byte swizzle, K-major = the canonical UMMA operand layout).
//   warps 2-5   dequant: thread i owns output column i of the tile; it reads its packed words
//               from shared memory, rebuilds exactly the reference's W[k,n] (T arithmetic, see
//               qgemm_small.cuh) and writes 16-byte k-chunks into the A operand buffer in the
//               K-major 128-byte-swizzled layout (chunk index XOR row%8), then
//               fence.proxy.async + mbarrier arrive.
//   warp 1      MMA issuer: one elected thread issues 4 x tcgen05.mma (128 x BM x 16, fp32
//               accumulate in TMEM) per k-block and tcgen05.commit's the stage back to the
//               producer; two TMEM accumulators (2 x BM columns) alternate between tiles.
//   warps 6-9   epilogue: tcgen05.ld 32 lanes x 32 columns at a time, + bias, round to T,
//               store out[m, n]; overlaps the next tile's main loop.
// Every mbarrier wait is bounded; on expiry the kernel records a code in the error word
// (last counter slot of the workspace) and every role leaves its loop.
#include "tma.cuh"
#include "tcgen05.cuh"
#include "qgemm_small.cuh"   // GroupConst / dequant_word

namespace mt {

struct TcParams {
    const uint32_t* qz;
    const void* scales;
    const void* bias;
    void* out;
    unsigned* err;          // error word (may be null)
    int m, n, k, groups, gs;
    int n_tiles, m_tiles;
    int zp1_const;
    int band;               // row tiles per band of the tile order (qgemm_tcx_kernel)
    int bm;                 // batch rows per tile (qgemm_tcx_kernel)
    // qgemm_tcx_kernel: the tiles of the last, partly filled wave are cut along K into `split` parts each (items), so that
    // the wave's CTAs all have work; parts leave fp32 partial tiles, the last part to arrive adds them in part order
    int full_tiles, split, total_items;
    float* partial; unsigned* counters;
};

constexpr int TC_BN = 128;     // output columns per tile (MMA M)
constexpr int TC_BK = 64;      // k per stage
constexpr int TC_STAGES = 4;
constexpr int TC_THREADS = 320;

template <int BITS, int BM> struct TcSmem {
    static constexpr int PACK = 32 / BITS;
    static constexpr int QROWS = TC_BK / PACK;
    static constexpr int A_BYTES = TC_BN * 128;
    static constexpr int B_BYTES = BM * 128;
    static constexpr int Q_BYTES = QROWS * TC_BN * 4;
    static constexpr int OFF_A = 0;
    static constexpr int OFF_B = OFF_A + TC_STAGES * A_BYTES;
    static constexpr int OFF_Q = OFF_B + TC_STAGES * B_BYTES;
    static constexpr int OFF_BAR = OFF_Q + TC_STAGES * Q_BYTES;
    static constexpr int TOTAL = OFF_BAR + 256 + 1024;   // barriers + slack for manual 1024-byte alignment
};

template <int BITS, typename T, int BM>
__global__ void __launch_bounds__(TC_THREADS, 1)
qgemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_q, const TcParams p) {
    using S = TcSmem<BITS, BM>;
    using H = F16x2<T>;
    constexpr int PACK = S::PACK, QROWS = S::QROWS;
    constexpr uint32_t TMEM_COLS = 2 * BM < 32 ? 32 : 2 * BM;
    static_assert((TMEM_COLS & (TMEM_COLS - 1)) == 0 && TMEM_COLS <= 512, "TMEM columns must be a power of two <= 512");

    extern __shared__ unsigned char smem_raw[];
    // operand tiles need 1024-byte alignment in the shared address space (swizzle atoms)
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bar0 = sbase + S::OFF_BAR;
    auto bar_full = [&](int s) { return bar0 + 8u * s; };
    auto bar_aready = [&](int s) { return bar0 + 8u * (TC_STAGES + s); };
    auto bar_empty = [&](int s) { return bar0 + 8u * (2 * TC_STAGES + s); };
    auto bar_tfull = [&](int a) { return bar0 + 8u * (3 * TC_STAGES + a); };
    auto bar_tempty = [&](int a) { return bar0 + 8u * (3 * TC_STAGES + 2 + a); };
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + S::OFF_BAR + 8 * (3 * TC_STAGES + 4));
    __shared__ int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kblocks = (p.k + TC_BK - 1) / TC_BK;
    const int total_tiles = p.n_tiles * p.m_tiles;

    if (tid == 0) {
        abort_flag = 0;
        for (int s = 0; s < TC_STAGES; ++s) { mbar_init(bar_full(s), 1); mbar_init(bar_aready(s), 128); mbar_init(bar_empty(s), 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(bar_tfull(a), 1); mbar_init(bar_tempty(a), 128); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            int it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const int n0 = (tile / p.m_tiles) * TC_BN, m0 = (tile % p.m_tiles) * BM;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = it % TC_STAGES; const uint32_t ph = (it / TC_STAGES) & 1;
                    if (!mbar_wait_sleep<200>(bar_empty(s), ph ^ 1, &abort_flag)) { ok = false; break; }
                    mbar_expect_tx(bar_full(s), S::Q_BYTES + S::B_BYTES);
                    tma_load_2d(sbase + S::OFF_Q + s * S::Q_BYTES, &tmap_q, n0, kb * QROWS, bar_full(s));
                    tma_load_2d(sbase + S::OFF_B + s * S::B_BYTES, &tmap_x, kb * TC_BK, m0, bar_full(s));
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            // instruction descriptor: D=f32, A/B = f16|bf16, both K-major, N = BM, M = 128
            const uint32_t fmt = H::kIsBf16 ? 1u : 0u;
            const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(BM >> 3) << 17) | ((uint32_t)(TC_BN >> 4) << 24);
            int it = 0, lt = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++lt) {
                const int acc = lt & 1; const uint32_t aph = (lt >> 1) & 1;
                if (!mbar_wait_sleep<100>(bar_tempty(acc), aph ^ 1, &abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BM);
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = it % TC_STAGES; const uint32_t ph = (it / TC_STAGES) & 1;
                    if (!mbar_wait_sleep<20>(bar_full(s), ph, &abort_flag) || !mbar_wait_sleep<20>(bar_aready(s), ph, &abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint64_t adesc = tc_desc_sw128(sbase + S::OFF_A + s * S::A_BYTES);
                    const uint64_t bdesc = tc_desc_sw128(sbase + S::OFF_B + s * S::B_BYTES);
#pragma unroll
                    for (int k4 = 0; k4 < TC_BK / 16; ++k4)
                        tc_mma_ss(d_tmem, adesc + (uint64_t)(k4 * 2), bdesc + (uint64_t)(k4 * 2), idesc, (kb | k4) != 0 ? 1u : 0u);
                    tc_commit(bar_empty(s));
                }
                if (ok) tc_commit(bar_tfull(acc));
            }
        }
    } else if (warp < 6) {
        // ---------------- dequant warps: thread i <-> output column i of the tile ----------------
        const int i = tid - 64;
        const T* __restrict__ sg = reinterpret_cast<const T*>(p.scales);
        int it = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
            const int n0 = (tile / p.m_tiles) * TC_BN;
            const int n = n0 + i;
            const bool n_ok = n < p.n;
            int g_cur = -1;
            GroupConst<BITS, T> gc;
            // scale / zero of the next two groups are already in flight when a group starts: a load
            // that is waited for right away costs a DRAM round trip per group in every dequant thread
            uint32_t sraw0 = 0, zraw0 = 0, sraw1 = 0, zraw1 = 0;
            auto fetch = [&](int g, uint32_t& sr, uint32_t& zr) {
                sr = 0; zr = 0;
                if (n_ok && g < p.groups) {
                    sr = (uint32_t)__ldg(reinterpret_cast<const uint16_t*>(sg) + (size_t)g * p.n + n);
                    if (p.qz) zr = __ldg(p.qz + (size_t)g * (p.n / PACK) + n / PACK);
                }
            };
            fetch(0, sraw0, zraw0);
            fetch(1, sraw1, zraw1);
            for (int kb = 0; kb < kblocks; ++kb, ++it) {
                const int s = it % TC_STAGES; const uint32_t ph = (it / TC_STAGES) & 1;
                const int g = min((kb * TC_BK) / p.gs, p.groups - 1);
                if (g != g_cur) {
                    g_cur = g;
                    make_group_const<BITS, T>(gc, make_uint2(sraw0, 0u), zraw0 >> ((n % PACK) * BITS), p.qz != nullptr, p.zp1_const);
                    sraw0 = sraw1; zraw0 = zraw1;
                    fetch(g + 2, sraw1, zraw1);
                }
                if (!mbar_wait_sleep<40>(bar_full(s), ph, &abort_flag)) { ok = false; break; }
                const uint32_t* q = reinterpret_cast<const uint32_t*>(smem + S::OFF_Q + s * S::Q_BYTES) + i;
                unsigned char* arow = smem + S::OFF_A + s * S::A_BYTES + (i >> 3) * 1024 + (i & 7) * 128;
                if constexpr (BITS == 4) {
#pragma unroll
                    for (int r = 0; r < QROWS; ++r) {
                        uint32_t f[4];
                        dequant_word<4, T>(q[r * TC_BN], gc, 0, f);   // (k0,k4) (k1,k5) (k2,k6) (k3,k7)
                        uint4 v;
                        v.x = prmt(f[0], f[1], 0x5410u); v.y = prmt(f[2], f[3], 0x5410u);   // (k0,k1) (k2,k3)
                        v.z = prmt(f[0], f[1], 0x7632u); v.w = prmt(f[2], f[3], 0x7632u);   // (k4,k5) (k6,k7)
                        *reinterpret_cast<uint4*>(arow + ((r ^ (i & 7)) << 4)) = v;
                    }
                } else {
#pragma unroll
                    for (int r = 0; r < QROWS; r += 2) {
                        uint32_t f0[2], f1[2];
                        dequant_word<8, T>(q[r * TC_BN], gc, 0, f0);
                        dequant_word<8, T>(q[(r + 1) * TC_BN], gc, 0, f1);
                        *reinterpret_cast<uint4*>(arow + (((r >> 1) ^ (i & 7)) << 4)) = make_uint4(f0[0], f0[1], f1[0], f1[1]);
                    }
                }
                fence_proxy_async();
                mbar_arrive(bar_aready(s));
            }
        }
    } else {
        // ---------------- epilogue warps ----------------
        const int q4 = warp & 3;                  // TMEM lane quarter this warp may access
        const int nl = q4 * 32 + lane;            // output column inside the tile
        const T* __restrict__ bias = reinterpret_cast<const T*>(p.bias);
        T* __restrict__ out = reinterpret_cast<T*>(p.out);
        int lt = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++lt) {
            const int n0 = (tile / p.m_tiles) * TC_BN, m0 = (tile % p.m_tiles) * BM;
            const int acc = lt & 1; const uint32_t aph = (lt >> 1) & 1;
            const int n = n0 + nl;
            const float bv = (bias && n < p.n) ? H::to_float(reinterpret_cast<const uint16_t*>(bias)[n]) : 0.f;
            if (!mbar_wait_sleep<500>(bar_tfull(acc), aph, &abort_flag)) { ok = false; break; }
            tc_fence_after();
#pragma unroll 1
            for (int c0 = 0; c0 < BM; c0 += 32) {
                uint32_t r[32];
                tc_ld32(tmem_base + ((uint32_t)(q4 * 32) << 16) + (uint32_t)(acc * BM + c0), r);
                tc_wait_ld();
                if (n < p.n) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int mrow = m0 + c0 + j;
                        if (mrow < p.m)
                            reinterpret_cast<uint16_t*>(out)[(size_t)mrow * p.n + n] = H::from_float(__uint_as_float(r[j]) + bv);
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(bar_tempty(acc));
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
    if (tid == 0 && abort_flag && p.err) atomicExch(p.err, 1u);
}

// =============================================================================================
// Wide-tile variant for int4 prefill: one CTA computes a 256 (columns) x 256 (batch rows) tile
// as two 128-column MMA tiles that share the same x k-block.  Per k-block a CTA now fetches
// 32 KB of x + 8 KB of packed weights for 2 x (128 x 256 x 64) MACs: 1.8x fewer L2->SM bytes
// per MAC than the 128 x 256 tile above, which was running at the L2 bandwidth limit.  All 512
// TMEM columns hold the two accumulators, so the epilogue of a tile is not overlapped with the
// next tile's main loop (about 5 % of a tile at K = 4096).
//   warp 0 TMA, warps 1 and 14 MMA issue (one per 128-column half), warps 2-9 dequant (thread i <-> column i of 256),
//   warps 10-13 epilogue.
// =============================================================================================
constexpr int TCW_STAGES = 3;
constexpr int TCW_THREADS = 15 * 32;     // TMA, MMA (first half), 8 dequant warps, 4 epilogue warps, MMA (second half)
constexpr int TCW_BM = 256;

struct TcwSmem {
    static constexpr int QROWS = TC_BK / 8;
    static constexpr int A_BYTES = 2 * TC_BN * 128;     // two 128-row operand tiles
    static constexpr int B_BYTES = TCW_BM * 128;
    static constexpr int Q_BYTES = QROWS * 256 * 4;
    static constexpr int OFF_A = 0;
    static constexpr int OFF_B = OFF_A + TCW_STAGES * A_BYTES;
    static constexpr int OFF_Q = OFF_B + TCW_STAGES * B_BYTES;
    static constexpr int OFF_BAR = OFF_Q + TCW_STAGES * Q_BYTES;
    static constexpr int TOTAL = OFF_BAR + 256 + 1024;
};

template <typename T>
__global__ void __launch_bounds__(TCW_THREADS, 1)
qgemm_tcw_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_q, const TcParams p) {
    using S = TcwSmem;
    using H = F16x2<T>;
    constexpr int PACK = 8, QROWS = S::QROWS, BM = TCW_BM;

    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bar0 = sbase + S::OFF_BAR;
    auto bar_full = [&](int s) { return bar0 + 8u * s; };
    auto bar_aready = [&](int s) { return bar0 + 8u * (TCW_STAGES + s); };
    auto bar_empty = [&](int s) { return bar0 + 8u * (2 * TCW_STAGES + s); };
    const uint32_t bar_tfull = bar0 + 8u * (3 * TCW_STAGES), bar_tempty = bar0 + 8u * (3 * TCW_STAGES + 1);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + S::OFF_BAR + 8 * (3 * TCW_STAGES + 2));
    __shared__ int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kblocks = (p.k + TC_BK - 1) / TC_BK;
    const int total_tiles = p.n_tiles * p.m_tiles;      // n_tiles counts 256-column tiles here

    if (tid == 0) {
        abort_flag = 0;
        for (int s = 0; s < TCW_STAGES; ++s) { mbar_init(bar_full(s), 1); mbar_init(bar_aready(s), 256); mbar_init(bar_empty(s), 2); }
        mbar_init(bar_tfull, 2); mbar_init(bar_tempty, 128);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            int it = 0; bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const int n0 = (tile / p.m_tiles) * 256, m0 = (tile % p.m_tiles) * BM;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = it % TCW_STAGES; const uint32_t ph = (it / TCW_STAGES) & 1;
                    if (!mbar_wait_sleep<200>(bar_empty(s), ph ^ 1, &abort_flag)) { ok = false; break; }
                    mbar_expect_tx(bar_full(s), S::Q_BYTES + S::B_BYTES);
                    tma_load_2d(sbase + S::OFF_Q + s * S::Q_BYTES, &tmap_q, n0, kb * QROWS, bar_full(s));
                    tma_load_2d(sbase + S::OFF_B + s * S::B_BYTES, &tmap_x, kb * TC_BK, m0, bar_full(s));
                }
            }
        }
    } else if (warp == 1 || warp == 14) {
        // two issuing threads in separate warps, one per 128-column half: a stage is free after both have committed
        const int nt = warp == 1 ? 0 : 1;
        if (lane == 0) {
            const uint32_t fmt = H::kIsBf16 ? 1u : 0u;
            const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(BM >> 3) << 17) | ((uint32_t)(TC_BN >> 4) << 24);
            int it = 0, lt = 0; bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++lt) {
                if (!mbar_wait_sleep<100>(bar_tempty, (lt & 1) ^ 1, &abort_flag)) { ok = false; break; }
                tc_fence_after();
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = it % TCW_STAGES; const uint32_t ph = (it / TCW_STAGES) & 1;
                    if (!mbar_wait_sleep<20>(bar_full(s), ph, &abort_flag) || !mbar_wait_sleep<20>(bar_aready(s), ph, &abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint64_t bdesc = tc_desc_sw128(sbase + S::OFF_B + s * S::B_BYTES);
                    const uint64_t adesc = tc_desc_sw128(sbase + S::OFF_A + s * S::A_BYTES + nt * (TC_BN * 128));
#pragma unroll
                    for (int k4 = 0; k4 < TC_BK / 16; ++k4)
                        tc_mma_ss(tmem_base + (uint32_t)(nt * BM), adesc + (uint64_t)(k4 * 2), bdesc + (uint64_t)(k4 * 2), idesc, (kb | k4) != 0 ? 1u : 0u);
                    tc_commit(bar_empty(s));
                }
                if (ok) tc_commit(bar_tfull);
            }
        }
    } else if (warp >= 2 && warp < 10) {
        // dequant: thread i <-> column i of the 256-column tile
        const int i = tid - 64;
        const int nt = i >> 7, il = i & 127;
        const T* __restrict__ sg = reinterpret_cast<const T*>(p.scales);
        int it = 0; bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
            const int n = (tile / p.m_tiles) * 256 + i;
            const bool n_ok = n < p.n;
            int g_cur = -1;
            GroupConst<4, T> gc;
            uint32_t sraw0 = 0, zraw0 = 0, sraw1 = 0, zraw1 = 0;
            auto fetch = [&](int g, uint32_t& sr, uint32_t& zr) {
                sr = 0; zr = 0;
                if (n_ok && g < p.groups) {
                    sr = (uint32_t)__ldg(reinterpret_cast<const uint16_t*>(sg) + (size_t)g * p.n + n);
                    if (p.qz) zr = __ldg(p.qz + (size_t)g * (p.n / PACK) + n / PACK);
                }
            };
            fetch(0, sraw0, zraw0);
            fetch(1, sraw1, zraw1);
            for (int kb = 0; kb < kblocks; ++kb, ++it) {
                const int s = it % TCW_STAGES; const uint32_t ph = (it / TCW_STAGES) & 1;
                const int g = min((kb * TC_BK) / p.gs, p.groups - 1);
                if (g != g_cur) {
                    g_cur = g;
                    make_group_const<4, T>(gc, make_uint2(sraw0, 0u), zraw0 >> ((n % PACK) * 4), p.qz != nullptr, p.zp1_const);
                    sraw0 = sraw1; zraw0 = zraw1;
                    fetch(g + 2, sraw1, zraw1);
                }
                if (!mbar_wait_sleep<40>(bar_full(s), ph, &abort_flag)) { ok = false; break; }
                const uint32_t* q = reinterpret_cast<const uint32_t*>(smem + S::OFF_Q + s * S::Q_BYTES) + i;
                unsigned char* arow = smem + S::OFF_A + s * S::A_BYTES + nt * (TC_BN * 128) + (il >> 3) * 1024 + (il & 7) * 128;
#pragma unroll
                for (int r = 0; r < QROWS; ++r) {
                    uint32_t f[4];
                    dequant_word<4, T>(q[r * 256], gc, 0, f);   // (k0,k4) (k1,k5) (k2,k6) (k3,k7)
                    uint4 v;
                    v.x = prmt(f[0], f[1], 0x5410u); v.y = prmt(f[2], f[3], 0x5410u);
                    v.z = prmt(f[0], f[1], 0x7632u); v.w = prmt(f[2], f[3], 0x7632u);
                    *reinterpret_cast<uint4*>(arow + ((r ^ (il & 7)) << 4)) = v;
                }
                fence_proxy_async();
                mbar_arrive(bar_aready(s));
            }
        }
    } else if (warp >= 10 && warp < 14) {
        // epilogue: warp & 3 = TMEM lane quarter; each thread owns one column of each 128-column tile
        const int q4 = warp & 3;
        const int nl = q4 * 32 + lane;
        const T* __restrict__ bias = reinterpret_cast<const T*>(p.bias);
        T* __restrict__ out = reinterpret_cast<T*>(p.out);
        int lt = 0; bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++lt) {
            const int n0 = (tile / p.m_tiles) * 256, m0 = (tile % p.m_tiles) * BM;
            if (!mbar_wait_sleep<500>(bar_tfull, lt & 1, &abort_flag)) { ok = false; break; }
            tc_fence_after();
#pragma unroll 1
            for (int nt = 0; nt < 2; ++nt) {
                const int n = n0 + nt * 128 + nl;
                const float bv = (bias && n < p.n) ? H::to_float(reinterpret_cast<const uint16_t*>(bias)[n]) : 0.f;
#pragma unroll 1
                for (int c0 = 0; c0 < BM; c0 += 32) {
                    uint32_t r[32];
                    tc_ld32(tmem_base + ((uint32_t)(q4 * 32) << 16) + (uint32_t)(nt * BM + c0), r);
                    tc_wait_ld();
                    if (n < p.n) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const int mrow = m0 + c0 + j;
                            if (mrow < p.m)
                                reinterpret_cast<uint16_t*>(out)[(size_t)mrow * p.n + n] = H::from_float(__uint_as_float(r[j]) + bv);
                        }
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(bar_tempty);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
    if (tid == 0 && abort_flag && p.err) atomicExch(p.err, 1u);
}

// =============================================================================================
// Prefill variant with the dequantized weights in TENSOR MEMORY: 256 (columns) x 192 (batch rows) per CTA.
// The 256 x 256 tile above moves, per k-block of 1024 tensor-pipe cycles, 96 KB of MMA operand reads, 32 KB of
// dequantized-A writes and 40 KB of TMA writes through shared memory: 168 B/clk against the SM's 128, so the
// tensor pipe waits for shared memory half of the time.  Here the converter warps write W straight into tensor
// memory (one tcgen05.st per thread and k-block, as the mid-batch kernel does) and the MMA takes A from there:
// shared memory carries the x tile (read twice, once per 128-column half), the packed words and nothing else
// (117 B/clk at the full tensor rate), and a stage shrinks from 72 KB to 32 KB, so six stages cover the latency of
// the TMA loads.  Tensor memory: 2 x 192 accumulator columns + 2 slots x 2 halves x 32 columns of A = 512.
//   warp 0 TMA, warp 1 MMA issue, warps 2-17 converters in two groups that take alternate k-blocks (a group's
//   chain -- wait for the stage, convert, wait for its A slot, tcgen05.st -- is longer than the 768 cycles the MMAs
//   of a k-block take; thread <-> column, TMEM lane quarter = warp % 4), warps 18-25 epilogue (not overlapped with
//   the next tile: the accumulators are single-buffered; eight warps keep it short).
// =============================================================================================
constexpr int TCX_THREADS = 28 * 32;     // TMA (x), MMA (first half), 2 x 8 converter warps, 8 epilogue warps, MMA (second half), TMA (packed words)
constexpr int TCX_BM = 192;

template <int BM> struct TcxSmem {
    static constexpr int STAGES = BM > 64 ? 6 : 12;      // 192 KB in flight either way
    static constexpr int QROWS = TC_BK / 8;
    static constexpr int B_BYTES = BM * 128;
    static constexpr int Q_BYTES = QROWS * 256 * 4;
    static constexpr int OFF_B = 0;
    static constexpr int OFF_Q = OFF_B + STAGES * B_BYTES;
    static constexpr int OFF_SZ = OFF_Q + STAGES * Q_BYTES;          // per converter thread: 2 x (scale word, zero word)
    static constexpr int OFF_ET = OFF_SZ + 512 * 16;                  // epilogue: two tiles of 32 rows x 128 columns of T
    static constexpr int OFF_BAR = OFF_ET + 2 * 32 * 128 * 2;
    static constexpr int TOTAL = OFF_BAR + 512 + 1024;
    static_assert(B_BYTES % 1024 == 0, "x tiles need 1024-byte alignment");
};

// Tile order of the persistent grid: row tiles in bands, inside a band column tile major.  The ~148 tiles in flight
// then share one band of x tiles (1.5 MB each) and a few weight tiles instead of every x tile of the batch, which at
// 8192 rows (67 MB of x) no longer fits the L2 next to the output stream.
constexpr int TCX_BAND_MAX = 24;
__device__ __forceinline__ void tcx_tile_origin(int tile, const TcParams& p, int& n0, int& m0) {
    const int per_band = p.band * p.n_tiles;
    const int band = tile / per_band, r = tile - band * per_band;
    const int rows = min(p.band, p.m_tiles - band * p.band);          // row tiles of this band (the last one may be short)
    const int nt = r / rows, mt = band * p.band + (r - nt * rows);
    n0 = nt * 256; m0 = mt * p.bm;
}

// Work item -> tile, k-block range, and (for a part of a split tile) its part number and the split tile's index.
__device__ __forceinline__ void tcx_item(int item, const TcParams& p, int kblocks, int& tile, int& kb0, int& kb1, int& part, int& sidx) {
    if (item < p.full_tiles) { tile = item; kb0 = 0; kb1 = kblocks; part = -1; sidx = 0; return; }
    const int j = item - p.full_tiles;
    sidx = j / p.split; part = j - sidx * p.split; tile = p.full_tiles + sidx;
    const int per = (kblocks + p.split - 1) / p.split;
    kb0 = part * per; kb1 = min(kblocks, kb0 + per);
}

template <typename T, int BM>
__global__ void __launch_bounds__(TCX_THREADS, 1)
qgemm_tcx_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_q, const TcParams p) {
    using S = TcxSmem<BM>;
    using H = F16x2<T>;
    constexpr int PACK = 8, QROWS = S::QROWS;
    static_assert(BM % 32 == 0 && BM <= 192, "batch rows per tile: 2 * BM accumulator columns + at least 128 columns of A");
    // Slots of A in tensor memory (64 columns each: two halves x 32).  A slot is rewritten only after the MMAs that read it
    // have committed, the converters have seen that, stored and said so, and the issuing thread has seen THAT: about 2000
    // cycles, during which the tensor pipe lives on the other slots.  Two slots (192-row tiles) hold 1536 cycles of MMA
    // work, three (160 rows) 1920, four (128 rows and fewer) more than enough.
    constexpr int NSLOT = (512 - 2 * BM) / 64 > 4 ? 4 : (512 - 2 * BM) / 64;
    static_assert(NSLOT >= 2 && NSLOT < S::STAGES, "A slots");
    constexpr uint32_t A_COL0 = 2 * BM;                      // first tensor-memory column of the A slots

    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bar0 = sbase + S::OFF_BAR;
    // One barrier per stage for everything the MMAs of a k-block need: `full` counts the x tile's bytes AND the eight
    // converter warps that wrote this k-block's weights into tensor memory, so the issuing thread waits once per
    // k-block; its one commit (`empty`) frees the stage for the producer and tells the converters two k-blocks later
    // that their A slot has been read.  `qfull`: the packed words of the stage have landed (the converters' input).
    auto bar_full = [&](int s) { return bar0 + 8u * s; };
    auto bar_empty = [&](int s) { return bar0 + 8u * (S::STAGES + s); };
    auto bar_qfull = [&](int s) { return bar0 + 8u * (2 * S::STAGES + s); };
    const uint32_t bar_tfull = bar0 + 8u * (3 * S::STAGES), bar_tempty = bar0 + 8u * (3 * S::STAGES + 1);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + S::OFF_BAR + 8 * (3 * S::STAGES + 2));
    __shared__ int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kblocks = (p.k + TC_BK - 1) / TC_BK;
    const int kpg = p.gs / TC_BK;                        // k-blocks per scale group (the group size is a multiple of 64)
    const int total_items = p.total_items;              // tiles of 256 columns x 192 rows; the last wave's are cut along K

    if (tid == 0) {
        abort_flag = 0;
        for (int s = 0; s < S::STAGES; ++s) { mbar_init(bar_full(s), 1 + 8); mbar_init(bar_empty(s), 2); mbar_init(bar_qfull(s), 1); }
        mbar_init(bar_tfull, 2); mbar_init(bar_tempty, 256);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_a = tmem_base + A_COL0;

    if (warp == 0 || warp == 27) {
        // two producer threads in separate warps, one for the x tiles and one for the packed words: a thread issues about
        // four TMA copies per microsecond, and a k-block of the MMAs lasts 0.2-0.4 us
        const bool words = warp == 27;
        if (lane == 0) {
            int it = 0; bool ok = true;
            for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
                int tile, kb0, kb1, part, sidx; tcx_item(item, p, kblocks, tile, kb0, kb1, part, sidx);
                int n0, m0; tcx_tile_origin(tile, p, n0, m0);
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = it % S::STAGES; const uint32_t ph = (it / S::STAGES) & 1;
                    if (!mbar_wait_sleep<200>(bar_empty(s), ph ^ 1, &abort_flag)) { ok = false; break; }
                    if (words) {
                        mbar_expect_tx(bar_qfull(s), S::Q_BYTES);
                        tma_load_2d(sbase + S::OFF_Q + s * S::Q_BYTES, &tmap_q, n0, kb * QROWS, bar_qfull(s));
                    } else {
                        mbar_expect_tx(bar_full(s), S::B_BYTES);
                        tma_load_2d(sbase + S::OFF_B + s * S::B_BYTES, &tmap_x, kb * TC_BK, m0, bar_full(s));
                    }
                }
            }
        }
    } else if (warp == 1 || warp == 26) {
        // two issuing threads, one per 128-column half (separate warps, so that they really run side by side): each
        // waits for the stage, issues its four MMAs of the k-block and commits; a stage is free after both commits
        const int nt = warp == 1 ? 0 : 1;
        if (lane == 0) {
            const uint32_t fmt = H::kIsBf16 ? 1u : 0u;
            const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(BM >> 3) << 17) | ((uint32_t)(TC_BN >> 4) << 24);
            int it = 0, lt = 0; bool ok = true;
            uint32_t early = 0u;
            for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x, ++lt) {
                int tile, kb0, kb1, part, sidx; tcx_item(item, p, kblocks, tile, kb0, kb1, part, sidx);
                if (!mbar_wait_sleep<100>(bar_tempty, (lt & 1) ^ 1, &abort_flag)) { ok = false; break; }
                tc_fence_after();
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = it % S::STAGES; const uint32_t ph = (it / S::STAGES) & 1;
                    const int as = it % NSLOT;
                    if (!early && !mbar_wait_sleep<20>(bar_full(s), ph, &abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    // ask about the next k-block now; the answer is read at the top of the next turn, behind this turn's MMAs
                    {
                        const int nit = it + 1;
                        early = mbar_test(bar_full(nit % S::STAGES), (uint32_t)((nit / S::STAGES) & 1));
                    }
                    const uint64_t bdesc = tc_desc_sw128(sbase + S::OFF_B + s * S::B_BYTES);
#pragma unroll
                    for (int k4 = 0; k4 < TC_BK / 16; ++k4)
                        tc_mma_ts(tmem_base + (uint32_t)(nt * BM), tmem_a + (uint32_t)((as * 2 + nt) * 32 + k4 * 8), bdesc + (uint64_t)(k4 * 2), idesc,
                                  (kb != kb0 || k4 != 0) ? 1u : 0u);
                    tc_commit(bar_empty(s));       // the stage is free, and so is this slot of A in tensor memory
                }
                if (ok) tc_commit(bar_tfull);
            }
        }
    } else if (warp >= 2 && warp < 18) {
        // converters: group = which k-blocks (even | odd) and which A slot; TMEM lane quarter = warp % 4 (the
        // hardware's rule); 128-column half = second bit of the warp's index inside its group
        const int grp = (warp - 2) >> 3;
        const int q4 = warp & 3, nt = ((warp - 2) >> 2) & 1;
        const int i = nt * 128 + q4 * 32 + lane;          // column inside the 256-column tile
        const T* __restrict__ sg = reinterpret_cast<const T*>(p.scales);
        int it = 0; bool ok = true;
        uint32_t q_early = 0u;                              // answer of the early look at this turn's `qfull`
        volatile uint32_t* szbuf = reinterpret_cast<volatile uint32_t*>(smem + S::OFF_SZ) + (tid - 64) * 4;
        const uint32_t szbuf_s = sbase + S::OFF_SZ + (uint32_t)(tid - 64) * 16u;
        for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
            int tile, kb0, kb1, part, sidx; tcx_item(item, p, kblocks, tile, kb0, kb1, part, sidx);
            int n0c, m0c; tcx_tile_origin(tile, p, n0c, m0c);
            const int n = n0c + i;
            const bool n_ok = n < p.n;
            int g_cur = -1;
            GroupConst<4, T> gc;
            // Scale and zero word of the NEXT group travel through two private words of shared memory (cp.async): a load
            // into a register that the loop carries to the next turn makes the compiler's register moves at the loop edge
            // wait for it, and the turn then pays the whole global-load latency (measured: 1000 of 2600 cycles).
            auto prefetch = [&](int g, int buf) {
                if (n_ok && g < p.groups) {
                    const uint32_t dst = szbuf_s + (uint32_t)buf * 8u;
                    const uint16_t* sp = reinterpret_cast<const uint16_t*>(sg) + (((size_t)g * p.n + n) & ~(size_t)1);
                    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(sp) : "memory");
                    if (p.qz) asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst + 4u), "l"(p.qz + (size_t)g * (p.n / PACK) + n / PACK) : "memory");
                }
                asm volatile("cp.async.commit_group;" ::: "memory");
            };
            auto take = [&](int g, int buf, uint32_t& sr, uint32_t& zr) {
                asm volatile("cp.async.wait_group 0;" ::: "memory");
                sr = 0; zr = 0;
                if (n_ok && g < p.groups) {
                    sr = (szbuf[buf * 2] >> ((n & 1) * 16)) & 0xffffu;
                    if (p.qz) zr = szbuf[buf * 2 + 1];
                }
            };
            // this group's first k-block of the item, its scale group and its place inside the group: tracked by addition from
            // here on (a division per turn is a chain of forty dependent instructions in a warp that has no others to issue)
            const int kb_first = kb0 + (((it & 1) != grp) ? 1 : 0);
            int g = min(kb_first / kpg, p.groups - 1), kin = kb_first - (kb_first / kpg) * kpg;
            int g_next = g;                                         // group whose words are on their way into buffer `cur`
            int cur = 0;
            asm volatile("cp.async.wait_group 0;" ::: "memory");   // the last prefetch of the previous item must not land after this one
            prefetch(g_next, cur);
            int s = it % S::STAGES; uint32_t ph = (it / S::STAGES) & 1;          // stage and phase of k-block `it`, kept by addition too
            for (int kb = kb0; kb < kb1; ++kb, ++it, s = (s + 1 == S::STAGES ? 0 : s + 1), ph ^= (s == 0 ? 1u : 0u)) {
                if ((it & 1) != grp) continue;              // the other group's k-block
                const int as = it % NSLOT;
                if (g != g_cur) {
                    if (g != g_next) prefetch(g, cur);                       // the prefetch guessed another group
                    uint32_t sraw, zraw;
                    take(g, cur, sraw, zraw);
                    g_cur = g;
                    make_group_const<4, T>(gc, make_uint2(sraw, 0u), zraw >> ((n % PACK) * 4), p.qz != nullptr, p.zp1_const);
                    g_next = g + 1; cur ^= 1;
                    prefetch(g_next, cur);                                   // the next group's words, on their way until that group starts
                }
                if (!q_early && !mbar_wait_sleep<40>(bar_qfull(s), ph, &abort_flag)) { ok = false; break; }
                // two early looks, answered behind the conversion arithmetic: is this group's A slot free (the MMAs of its
                // previous turn have committed), and have the packed words of its next turn landed
                const int s_prev = s >= NSLOT ? s - NSLOT : s - NSLOT + S::STAGES; const uint32_t ph_prev = s >= NSLOT ? ph : ph ^ 1u;   // k-block it - NSLOT: the last user of this slot
                const int s_next = s + 2 < S::STAGES ? s + 2 : s + 2 - S::STAGES; const uint32_t ph_next = s + 2 < S::STAGES ? ph : ph ^ 1u;   // k-block it + 2
                uint32_t a_free = 1u;
                if (it >= NSLOT) a_free = mbar_test(bar_empty(s_prev), ph_prev);
                q_early = mbar_test(bar_qfull(s_next), ph_next);
                const uint32_t* q = reinterpret_cast<const uint32_t*>(smem + S::OFF_Q + s * S::Q_BYTES) + i;
                uint32_t a[32];
#pragma unroll
                for (int r = 0; r < QROWS; ++r) {
                    uint32_t f[4];
                    dequant_word<4, T>(q[r * 256], gc, 0, f);   // (k0,k4) (k1,k5) (k2,k6) (k3,k7)
                    a[4 * r + 0] = prmt(f[0], f[1], 0x5410u); a[4 * r + 1] = prmt(f[2], f[3], 0x5410u);   // k in order: two per column
                    a[4 * r + 2] = prmt(f[0], f[1], 0x7632u); a[4 * r + 3] = prmt(f[2], f[3], 0x7632u);
                }
                if (!a_free) {                                   // the MMAs NSLOT k-blocks back have read this slot
                    if (!mbar_wait_sleep<40>(bar_empty(s_prev), ph_prev, &abort_flag)) { ok = false; break; }
                }
                tc_fence_after();
                tc_st32(tmem_a + ((uint32_t)(q4 * 32) << 16) + (uint32_t)((as * 2 + nt) * 32), a);
                tc_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_full(s));
                kin += 2;                                        // this group's next k-block is two further
                while (kin >= kpg) { kin -= kpg; if (g < p.groups - 1) ++g; }
            }
        }
    } else if (warp >= 18 && warp < 26) {
        // epilogue, eight warps: warp & 3 = TMEM lane quarter, the other bit = 128-column half; a thread owns one column
        const int q4 = warp & 3;
        const int nt = (warp - 18) >> 2;
        const int nl = q4 * 32 + lane;
        const T* __restrict__ bias = reinterpret_cast<const T*>(p.bias);
        T* __restrict__ out = reinterpret_cast<T*>(p.out);
        int lt = 0; bool ok = true;
        for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x, ++lt) {
            int tile, kb0, kb1, part, sidx; tcx_item(item, p, kblocks, tile, kb0, kb1, part, sidx);
            int n0, m0; tcx_tile_origin(tile, p, n0, m0);
            // A warp whose wait gives up must still pass the named barriers below as often as the other three warps of its
            // half (which may have seen the tile complete just before the abort): it goes through the loop without touching
            // tensor memory or the output, then leaves.
            const bool got = mbar_wait_sleep<500>(bar_tfull, lt & 1, &abort_flag);
            if (!got) ok = false;
            tc_fence_after();
            if (part >= 0) {
                if (!got) break;
                // A part of a tile that was cut along K: leave the fp32 sums of this part in the workspace; the warp that
                // finds all other parts there adds them in part order (its own from tensor memory) and stores the tile.
                const size_t slice = (size_t)BM * 128;                     // one 128-column half of one part
                float* mine = p.partial + ((size_t)(sidx * p.split + part) * 2 + nt) * slice;
#pragma unroll 1
                for (int c0 = 0; c0 < BM; c0 += 32) {
                    uint32_t r[32];
                    tc_ld32(tmem_base + ((uint32_t)(q4 * 32) << 16) + (uint32_t)(nt * BM + c0), r);
                    tc_wait_ld();
#pragma unroll
                    for (int j = 0; j < 32; ++j) __stcg(mine + (size_t)(c0 + j) * 128 + nl, __uint_as_float(r[j]));
                }
                __threadfence();
                __syncwarp();
                unsigned old = 0;
                unsigned* ctr = p.counters + sidx * 8 + (warp - 18);
                if (lane == 0) old = atomicAdd(ctr, 1u);
                old = __shfl_sync(0xffffffffu, old, 0);
                if (old == unsigned(p.split - 1)) {
                    __threadfence();
                    const int n = n0 + nt * 128 + nl;
                    const float bv = (bias && n < p.n) ? H::to_float(reinterpret_cast<const uint16_t*>(bias)[n]) : 0.f;
#pragma unroll 1
                    for (int c0 = 0; c0 < BM; c0 += 16) {                   // 16 rows at a time: the sums and the own values fit the registers
                        uint32_t r[16];
                        tc_ld<16>(tmem_base + ((uint32_t)(q4 * 32) << 16) + (uint32_t)(nt * BM + c0), r);
                        tc_wait_ld();
                        float acc[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) acc[j] = 0.f;
                        for (int q = 0; q < p.split; ++q) {                     // part order, whoever arrives last
                            const float* src = p.partial + ((size_t)(sidx * p.split + q) * 2 + nt) * slice + (size_t)c0 * 128 + nl;
#pragma unroll
                            for (int j = 0; j < 16; ++j) acc[j] += (q == part) ? __uint_as_float(r[j]) : __ldcg(src + (size_t)j * 128);
                        }
                        if (n < p.n) {
#pragma unroll
                            for (int j = 0; j < 16; ++j) {
                                const int mrow = m0 + c0 + j;
                                if (mrow < p.m) reinterpret_cast<uint16_t*>(out)[(size_t)mrow * p.n + n] = H::from_float(acc[j] + bv);
                            }
                        }
                    }
                    if (lane == 0) *ctr = 0;
                }
            } else {
                // A thread holds one output COLUMN (its TMEM lane) and 32 rows of it; the output is row major.  Stored as it is,
                // a warp writes 64 contiguous bytes per instruction (measured: 15 000 cycles per tile, during which the MMAs
                // wait).  So the four warps of a 128-column half turn 32 rows x 128 columns through shared memory and store whole
                // 256-byte row segments, 16 bytes per lane.
                const int n = n0 + nt * 128 + nl;
                const float bv = (bias && n < p.n) ? H::to_float(reinterpret_cast<const uint16_t*>(bias)[n]) : 0.f;
                uint16_t* et = reinterpret_cast<uint16_t*>(smem + S::OFF_ET) + nt * (32 * 128);      // [32 rows][128 columns]
                const int ncol = n0 + nt * 128 + 8 * (lane & 15);                                       // first of this lane's 8 columns
#pragma unroll 1
                for (int c0 = 0; c0 < BM; c0 += 32) {
                    if (got) {
                        uint32_t r[32];
                        tc_ld32(tmem_base + ((uint32_t)(q4 * 32) << 16) + (uint32_t)(nt * BM + c0), r);
                        tc_wait_ld();
#pragma unroll
                        for (int j = 0; j < 32; ++j) et[j * 128 + nl] = H::from_float(__uint_as_float(r[j]) + bv);
                    }
                    if (nt == 0) asm volatile("bar.sync 2, 128;" ::: "memory"); else asm volatile("bar.sync 3, 128;" ::: "memory");
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const int rr = q4 * 8 + 2 * q + (lane >> 4);                                     // row of the 32: two rows per instruction
                        const int mrow = m0 + c0 + rr;
                        const uint4 v = *reinterpret_cast<const uint4*>(et + rr * 128 + 8 * (lane & 15));
                        if (got && mrow < p.m) {
                            uint16_t* dst = reinterpret_cast<uint16_t*>(out) + (size_t)mrow * p.n + ncol;
                            if (ncol + 8 <= p.n) {
                                *reinterpret_cast<uint4*>(dst) = v;
                            } else {
                                const uint16_t* h = reinterpret_cast<const uint16_t*>(&v);
                                for (int e = 0; e < 8; ++e) if (ncol + e < p.n) dst[e] = h[e];
                            }
                        }
                    }
                    if (nt == 0) asm volatile("bar.sync 2, 128;" ::: "memory"); else asm volatile("bar.sync 3, 128;" ::: "memory");   // the tile is rewritten by the next 32 rows
                }
            }
            if (!got) break;
            tc_fence_before();
            mbar_arrive(bar_tempty);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
    if (tid == 0 && abort_flag && p.err) atomicExch(p.err, 1u);
}

// ---- host side -------------------------------------------------------------------------
EncodeTiledFn get_tensor_map_encoder() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
        else
            cudaGetLastError();
    }
    return fn;
}

// 65 to 128 rows: the 256 x 192 tile with the weights in tensor memory is the kernel of choice when its one row of tiles
// gives at least ~100 CTAs work.
bool tc_tmem_a_preferred(int m, int n, int bits) {
    return bits == 4 && m > 64 && m <= 128 && (n + 255) / 256 >= 100;
}

// Parts per tile of the last, partly filled wave of 256 x 192 tiles (1: leave it alone).  A wave that is at most half
// full is cut so that its parts fill the GPU once: the wave then takes 1 / split of a tile's time.
int tcx_tail_split(int m, int n, int k, int sms, int bm) {
    const int tiles = ((n + 255) / 256) * ((m + bm - 1) / bm);
    const int rest = tiles % sms;
    if (tiles < sms || rest == 0) return 1;                  // less than one wave in all: one tile per CTA is all there is
    int split = sms / rest;
    if (split > 4) split = 4;
    const int kblocks = (k + TC_BK - 1) / TC_BK;
    while (split > 1 && kblocks < 16 * split) --split;       // a part keeps at least 16 k-blocks
    return split < 1 ? 1 : split;
}
size_t tcx_workspace_bytes(int m, int n, int k) {
    const int sms = 148;
    size_t need = 0;
    for (int bm : {192, 160}) {
        const int split = tcx_tail_split(m, n, k, sms, bm);
        if (split <= 1) continue;
        const int tiles = ((n + 255) / 256) * ((m + bm - 1) / bm);
        const size_t b = (size_t)(tiles % sms) * split * 2 * bm * 128 * 4;
        if (b > need) need = b;
    }
    return need;
}

bool tc_supported(const QGemmArgs& a) {
    if (a.g_idx != nullptr) return false;
    const int gs = a.k / a.groups;
    if (gs % TC_BK != 0) return false;
    if (a.n % 8 != 0 || a.k % 32 != 0) return false;
    return true;
}

template <int BITS, typename T, int BM>
static int launch_tc_inst(cudaStream_t st, const QGemmArgs& a, const CUtensorMap& mx, const CUtensorMap& mq, const TcParams& p) {
    using S = TcSmem<BITS, BM>;
    auto kern = qgemm_tc_kernel<BITS, T, BM>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL) != cudaSuccess) {
        cudaGetLastError();
        return MT_ERR_TOO_LARGE;
    }
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int tiles = p.n_tiles * p.m_tiles;
    const int grid = tiles < sms ? tiles : sms;
    kern<<<grid, TC_THREADS, S::TOTAL, st>>>(mx, mq, p);
    return cudaGetLastError() == cudaSuccess ? MT_OK : MT_ERR_CUDA;
}

// Launch of qgemm_tcx_kernel with tiles of 256 columns x bm rows.  split_all == 0: one item per tile, the tiles of a last
// wave that is at most half full cut along K (tcx_tail_split); split_all > 0: EVERY tile cut into that many parts (the
// schedule for few, deep tiles).  `mq` is the packed-weight map with the 256-column box; `p` holds the common fields.
static int launch_tcx(cudaStream_t st, const QGemmArgs& a, EncodeTiledFn enc, const CUtensorMap& mq, TcParams p, int bm, int split_all) {
    CUtensorMap mxb;
    {
        cuuint64_t dims[2] = {(cuuint64_t)a.k, (cuuint64_t)a.m};
        cuuint64_t strides[1] = {(cuuint64_t)a.k * 2};
        cuuint32_t box[2] = {(cuuint32_t)TC_BK, (cuuint32_t)bm};
        cuuint32_t es[2] = {1, 1};
        const CUtensorMapDataType dt = a.dtype == MT_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
        if (enc(&mxb, dt, 2, const_cast<void*>(a.x), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return MT_ERR_CUDA;
    }
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    p.bm = bm;
    p.n_tiles = (a.n + 255) / 256; p.m_tiles = (a.m + bm - 1) / bm;
    // bands of at most 24 row tiles, all of the same height (measured on 4096 x 28672: all 22 row tiles in one band at
    // 4096 rows 1124 TFLOP/s against 1081 with bands of 8; at 8192 rows one band of 43 gives 994, bands of 16 1065)
    const int nbands = (p.m_tiles + TCX_BAND_MAX - 1) / TCX_BAND_MAX;
    p.band = (p.m_tiles + nbands - 1) / nbands;
    if ((a.flags >> 24) & 0xf) p.band = ((a.flags >> 24) & 0xf) * 4;      // tuning: bits 24-27 of the flags = band / 4
    const int tiles = p.n_tiles * p.m_tiles;
    p.full_tiles = tiles; p.split = 1; p.partial = nullptr; p.counters = nullptr;
    const bool ws_ok = a.workspace && a.workspace_bytes >= kCounterBytes;
    if (split_all == 1) {
        // one part per tile: nothing to add
    } else if (split_all > 1) {
        const size_t need = (size_t)tiles * split_all * 2 * bm * 128 * 4;
        if (!ws_ok || a.workspace_bytes < kCounterBytes + need || tiles * 8 > kMaxTiles - 8) return MT_ERR_WORKSPACE;
        p.full_tiles = 0; p.split = split_all;
    } else {
        const int split = bm > 64 ? tcx_tail_split(a.m, a.n, a.k, sms, bm) : 1;
        const int rest = tiles % sms;
        const size_t need = (size_t)rest * split * 2 * bm * 128 * 4;
        if (split > 1 && ws_ok && a.workspace_bytes >= kCounterBytes + need && rest * 8 <= kMaxTiles - 8) {
            p.full_tiles = tiles - rest; p.split = split;
        }
    }
    if (p.split > 1) {
        p.counters = static_cast<unsigned*>(a.workspace);
        p.partial = reinterpret_cast<float*>(static_cast<char*>(a.workspace) + kCounterBytes);
    }
    p.total_items = p.full_tiles + (tiles - p.full_tiles) * p.split;
    const int grid = p.total_items < sms ? p.total_items : sms;
#define MT_TCX(T_, BM_) do { \
        auto kern = qgemm_tcx_kernel<T_, BM_>; \
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, TcxSmem<BM_>::TOTAL) != cudaSuccess) { cudaGetLastError(); return MT_ERR_TOO_LARGE; } \
        kern<<<grid, TCX_THREADS, TcxSmem<BM_>::TOTAL, st>>>(mxb, mq, p); } while (0)
    if (bm == 192)      { if (a.dtype == MT_F16) MT_TCX(__half, 192); else MT_TCX(__nv_bfloat16, 192); }
    else if (bm == 160) { if (a.dtype == MT_F16) MT_TCX(__half, 160); else MT_TCX(__nv_bfloat16, 160); }
    else if (bm == 64)  { if (a.dtype == MT_F16) MT_TCX(__half, 64); else MT_TCX(__nv_bfloat16, 64); }
    else return MT_ERR_UNSUPPORTED;
#undef MT_TCX
    return cudaGetLastError() == cudaSuccess ? MT_OK : MT_ERR_CUDA;
}

// Batches that fit ONE row of tiles of the tensor-memory-A kernel (up to 192 rows; tiles of 64, 160 or 192 rows): every
// tile is cut into `split` parts along K so that the parts fill the GPU's waves (few, deep tiles otherwise: 224 tiles of
// 128 k-blocks on 8192 x 57344, 32 tiles of 448 on 28672 x 8192).
static int tcx_rows_bm(int m) { return m <= 64 ? 64 : (m <= 160 ? 160 : 192); }
static int tcx_rows_split(int m, int n, int k, int sms) {
    const int tiles = (n + 255) / 256;
    const int kblocks = (k + TC_BK - 1) / TC_BK;
    // time in k-blocks: waves x (k-blocks of a part + the part's fp32 partial tile, written and read back: 2 x bm x 128 x 4
    // bytes per 128-column half, about bm / 16 k-blocks' worth at an SM's share of the memory bandwidth)
    const double partial = tcx_rows_bm(m) / 16.0;
    int best = 1; double best_cost = 1e30;
    for (int s : {1, 2, 3, 4, 6, 8}) {
        if (s > 1 && kblocks < 16 * s) break;
        const double waves = double((tiles * s + sms - 1) / sms);
        const double cost = waves * (double(kblocks) / s + (s > 1 ? partial : 0.0));
        if (cost < best_cost) { best_cost = cost; best = s; }
    }
    return best;
}
size_t tcx_rows_workspace_bytes(int m, int n, int k) {
    const int s = tcx_rows_split(m, n, k, 148);
    return s > 1 ? (size_t)((n + 255) / 256) * s * 2 * tcx_rows_bm(m) * 128 * 4 : 0;
}
bool tcx_rows_supported(const QGemmArgs& a) {
    if (!tc_supported(a) || a.bits != 4 || a.m < 1 || a.m > 192 || a.n < 256) return false;
    if (((a.n + 255) / 256) * 8 > kMaxTiles - 8) return false;
    return a.workspace != nullptr && a.workspace_bytes >= kCounterBytes + tcx_rows_workspace_bytes(a.m, a.n, a.k);
}
int launch_tcx_rows(cudaStream_t st, const QGemmArgs& a) {
    EncodeTiledFn enc = get_tensor_map_encoder();
    if (!enc || !tcx_rows_supported(a)) return MT_ERR_UNSUPPORTED;
    CUtensorMap mq;
    {
        cuuint64_t dims[2] = {(cuuint64_t)a.n, (cuuint64_t)(a.k / 8)};
        cuuint64_t strides[1] = {(cuuint64_t)a.n * 4};
        cuuint32_t box[2] = {256u, (cuuint32_t)(TC_BK / 8)};
        cuuint32_t es[2] = {1, 1};
        if (enc(&mq, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<uint32_t*>(a.qweight), dims, strides, box, es,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return MT_ERR_CUDA;
    }
    TcParams p;
    p.qz = a.qzeros; p.scales = a.scales; p.bias = a.bias; p.out = a.out;
    p.err = static_cast<unsigned*>(a.workspace) + (kMaxTiles - 1);
    p.m = a.m; p.n = a.n; p.k = a.k; p.groups = a.groups; p.gs = a.k / a.groups;
    p.zp1_const = 1 << (a.bits - 1);
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    int split = tcx_rows_split(a.m, a.n, a.k, sms);
    if (((a.flags >> 16) & 0xff) != 0) split = (a.flags >> 16) & 0xff;      // tuning: MT_FLAG_SPLITS forces the parts per tile
    return launch_tcx(st, a, enc, mq, p, tcx_rows_bm(a.m), split);
}

int launch_tc(cudaStream_t st, const QGemmArgs& a) {
    EncodeTiledFn enc = get_tensor_map_encoder();
    if (!enc) return MT_ERR_UNSUPPORTED;
    // one row of tiles of the tensor-memory-A kernel, cut along K: up to 64 rows by flag only (mt_qgemm sends 33..64 rows here
    // itself), from 65 to 192 rows whenever the request fits
    if (a.m <= 64 && (a.flags & MT_FLAG_TC_TMEM_A)) return launch_tcx_rows(st, a);
    if (a.m > 64 && a.m <= 192 && !(a.flags & MT_FLAG_TC_SMEM_A) && tcx_rows_supported(a)) return launch_tcx_rows(st, a);
    const int pack = 32 / a.bits;
    const int bm = a.m > 128 ? 256 : (a.m > 64 ? 128 : 64);
    CUtensorMap mx, mq;
    {
        cuuint64_t dims[2] = {(cuuint64_t)a.k, (cuuint64_t)a.m};
        cuuint64_t strides[1] = {(cuuint64_t)a.k * 2};
        cuuint32_t box[2] = {(cuuint32_t)TC_BK, (cuuint32_t)bm};
        cuuint32_t es[2] = {1, 1};
        const CUtensorMapDataType dt = a.dtype == MT_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
        if (enc(&mx, dt, 2, const_cast<void*>(a.x), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return MT_ERR_CUDA;
    }
    {
        cuuint64_t dims[2] = {(cuuint64_t)a.n, (cuuint64_t)(a.k / pack)};
        cuuint64_t strides[1] = {(cuuint64_t)a.n * 4};
        cuuint32_t box[2] = {(cuuint32_t)TC_BN, (cuuint32_t)(TC_BK / pack)};
        cuuint32_t es[2] = {1, 1};
        if (enc(&mq, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<uint32_t*>(a.qweight), dims, strides, box, es,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return MT_ERR_CUDA;
    }
    const bool wide = a.bits == 4 && a.m > 64 && a.n >= 256;       // the 256-column tiles (int4)
    TcParams p;
    p.qz = a.qzeros; p.scales = a.scales; p.bias = a.bias; p.out = a.out;
    p.err = (a.workspace && a.workspace_bytes >= kCounterBytes) ? static_cast<unsigned*>(a.workspace) + (kMaxTiles - 1) : nullptr;
    p.m = a.m; p.n = a.n; p.k = a.k; p.groups = a.groups; p.gs = a.k / a.groups;
    p.n_tiles = (a.n + TC_BN - 1) / TC_BN; p.m_tiles = (a.m + bm - 1) / bm;
    p.zp1_const = 1 << (a.bits - 1);
    // Two int4 prefill tiles: 256 x 192 with the dequantized weights in tensor memory (about 8 % faster per unit of work)
    // and 256 x 256 with them in shared memory.  Both run one tile per CTA at a time on a persistent grid, so the one
    // whose tile count fills the last wave better wins: compare waves x rows per tile.
    // From 65 to 128 rows only the first has a tile that fits (the 256 x 256 one would be half empty), and it pays when
    // its single row of tiles nearly fills the GPU (tc_tmem_a_preferred): 8192 x 57344 at 128 rows 196 us against 336 us
    // for the mid-batch kernel, but 28672 x 8192 (32 tiles) 309 us against 218 us.
    // row tile of the tensor-memory-A kernel: 192 rows (two A slots) measured 1099 / 1113 / 1099 TFLOP/s on the three 4096-row
    // shapes, 160 rows (three slots) 1044 / 1106 / 993 on the same GPU; bit 28 of the flags selects the latter (tuning)
    const int xbm = ((a.flags >> 28) & 1) ? 160 : 192;
    bool tmem_a = (a.flags & MT_FLAG_TC_TMEM_A) != 0 || (wide && a.m <= 128 && tc_tmem_a_preferred(a.m, a.n, a.bits));
    if (wide && a.m > 128 && !tmem_a && !(a.flags & MT_FLAG_TC_SMEM_A)) {
        int dev = 0, sms = 148;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        const long long nt256 = (a.n + 255) / 256;
        const long long tiles_x = nt256 * ((a.m + xbm - 1) / xbm);
        const long long waves_w = (nt256 * ((a.m + TCW_BM - 1) / TCW_BM) + sms - 1) / sms;
        // time of the 256 x 192 tiles in units of one row of a tile: full waves, plus the last wave cut along K
        const int split = tcx_tail_split(a.m, a.n, a.k, sms, xbm);
        const long long cost_x = (tiles_x / sms) * xbm * split + ((tiles_x % sms) ? xbm : 0);     // x split
        tmem_a = cost_x * 92 <= waves_w * TCW_BM * 100 * split;
    }
    if (wide && (tmem_a || a.m > 128)) {   // the packed-weight box covers 256 columns
        cuuint64_t dims[2] = {(cuuint64_t)a.n, (cuuint64_t)(a.k / pack)};
        cuuint64_t strides[1] = {(cuuint64_t)a.n * 4};
        cuuint32_t box[2] = {256u, (cuuint32_t)(TC_BK / pack)};
        cuuint32_t es[2] = {1, 1};
        if (enc(&mq, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<uint32_t*>(a.qweight), dims, strides, box, es,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return MT_ERR_CUDA;
    }
    if (wide && tmem_a) return launch_tcx(st, a, enc, mq, p, xbm, /*split_all=*/0);
    if (wide && a.m > 128) {
        p.n_tiles = (a.n + 255) / 256;
        int dev = 0, sms = 148;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        const int tiles = p.n_tiles * p.m_tiles;
        const int grid = tiles < sms ? tiles : sms;
        if (a.dtype == MT_F16) {
            auto kern = qgemm_tcw_kernel<__half>;
            if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, TcwSmem::TOTAL) != cudaSuccess) { cudaGetLastError(); return MT_ERR_TOO_LARGE; }
            kern<<<grid, TCW_THREADS, TcwSmem::TOTAL, st>>>(mx, mq, p);
        } else {
            auto kern = qgemm_tcw_kernel<__nv_bfloat16>;
            if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, TcwSmem::TOTAL) != cudaSuccess) { cudaGetLastError(); return MT_ERR_TOO_LARGE; }
            kern<<<grid, TCW_THREADS, TcwSmem::TOTAL, st>>>(mx, mq, p);
        }
        return cudaGetLastError() == cudaSuccess ? MT_OK : MT_ERR_CUDA;
    }
#define MT_TC(B_, T_) \
    (bm == 256 ? launch_tc_inst<B_, T_, 256>(st, a, mx, mq, p) : bm == 128 ? launch_tc_inst<B_, T_, 128>(st, a, mx, mq, p) \
                                                                          : launch_tc_inst<B_, T_, 64>(st, a, mx, mq, p))
    if (a.bits == 4) return a.dtype == MT_F16 ? MT_TC(4, __half) : MT_TC(4, __nv_bfloat16);
    return a.dtype == MT_F16 ? MT_TC(8, __half) : MT_TC(8, __nv_bfloat16);
#undef MT_TC
}

}  // namespace mt
