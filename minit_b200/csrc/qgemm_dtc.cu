// Decode GEMV/GEMM (M <= 32) for GPTQ weights with contiguous groups on tcgen05 + TMEM.
//
// Roofline: HBM.  On B200 the only FMA engine cheap enough to keep up with 6.5 TB/s of int4
// weights (~46 weights per clock per SM) is the tcgen05 tensor core: legacy mma.sync runs at
// about 1/16 of its rate and CUDA-core FMAs cost several instructions per weight.  So even the
// M = 1 product is issued as tcgen05.mma, and the CUDA cores do no per-weight arithmetic:
//
//   converter warps   read packed words from the TMA-staged tile and OR in the fp16 magic
//                     number: (w & 0x000f000f) | 0x64006400 = (1024 + q_j, 1024 + q_{j+4}), five
//                     integer instructions per eight weights (bits 4..7 give 1024 + 16 q; those
//                     k-slots of x are pre-divided by 16).  No zero point, no scale.  The 32
//                     registers of one k-block go to TMEM with ONE tcgen05.st: the A operand of
//                     the MMA lives in tensor memory and never touches shared memory.
//   x warp            stages x[m, k-block] as the B operand (K-major, 128-byte swizzle, k-slots in
//                     the same permuted order) and, per scale group, the sums
//                     X1 = sum of x as the tensor core sees it, X2 = sum of x as q sees it.
//   MMA warp          one thread issues tcgen05.mma.kind::f16 (M=128 columns of W, N=16|32
//                     batch rows, K=16), A from TMEM, B from shared memory, one fp32 accumulator
//                     per (column tile, scale group) in TMEM, double buffered.
//   fold warps        per scale group: tcgen05.ld the group's accumulator and apply, once per
//                     group instead of once per weight,
//                         out[n,m] += s[g,n] * (D_g[n,m] - 1024 X1_g[m] - (z[g,n]+1) X2_g[m]).
//                     They also own split-K (fp32 partials, last-arriver reduction) and the store.
//   TMA warp          2-D bulk tensor loads of [64 k / pack rows] x [256 columns] of qweight into
//                     an 8-stage ring (1 KB contiguous per row, 64 KB in flight per SM).
//
// All products entering the tensor core are exact in fp32; cancelling the 1024 X1 offset
// (|.| ~ 1e4) costs ~1e-3 absolute per group before the scale, four orders of magnitude below the
// acceptance bound.  Every mbarrier wait is bounded and reports through the workspace error word.
#include <stdlib.h>
#include "tma.cuh"
#include "tcgen05.cuh"

namespace mt {

struct DtcParams {
    const void* x;
    const uint32_t* qw;
    const uint32_t* qz;
    const void* scales;
    const void* bias;
    void* out;
    float* partial;
    unsigned* counters;
    unsigned* err;
    int m, n, k, groups, gs;
    int tiles, fpt, total_folds;   // fpt = folds per column tile (K / fold size); total_folds = tiles * fpt
    int zp1_const;
};

constexpr int DT_NTILES = 2;               // 128-column MMA tiles per CTA tile
constexpr int DT_NT = DT_NTILES * 128;     // 256 columns = 1 KB contiguous per packed row
constexpr int DT_ASTAGES = 3;              // A-operand (TMEM) ring (k-blocks)
constexpr int DT_DBUF = 2;                 // accumulator buffers per column tile
constexpr int DT_XSLOTS = 4;               // x ring, one slot per fold
// Two CTAs share an SM (each owns half of TMEM and < half of shared memory): every role exists
// twice per SM, which hides the hand-off latencies between the roles.
// warp roles
constexpr int DT_W_FOLD = 0;               // 4 warps (TMEM lane quarters)
constexpr int DT_W_CONV = 4;               // 8 warps: 2 tiles x 4 quarters
constexpr int DT_W_PROD = 12;              // bulk-copy producer
constexpr int DT_W_MMA = 13;               // MMA issuer
constexpr int DT_W_X = 14;                 // x staging
constexpr int DT_THREADS = 15 * 32;

template <int BITS, int MP, int KPB> struct DtcSmem {
    static constexpr int PACK = 32 / BITS;
    static constexpr int PROWS = 64 / PACK;                        // packed rows per k-block
    static constexpr int P_BYTES = PROWS * DT_NT * 4;              // 8 KB (int4) / 16 KB (int8)
    static constexpr int PSTAGES = BITS == 4 ? 8 : 5;              // packed-weight ring (k-blocks): 64 / 80 KB in flight per CTA
    static constexpr int XB_BYTES = MP * 128;                      // one B tile (MP rows x 64 k)
    static constexpr int XSLOT_BYTES = KPB * XB_BYTES + 2 * MP * 4;   // tiles of one fold + X1/X2
    static constexpr int OFF_P = 0;
    static constexpr int OFF_X = OFF_P + PSTAGES * P_BYTES;
    static constexpr int XSLOT_STRIDE = (XSLOT_BYTES + 1023) & ~1023;
    static constexpr int OFF_BAR = OFF_X + DT_XSLOTS * XSLOT_STRIDE;
    static constexpr int NBARS = 2 * PSTAGES + 2 * DT_ASTAGES + 2 * DT_XSLOTS + 2 * DT_DBUF;
    static constexpr int TOTAL = OFF_BAR + NBARS * 8 + 64 + 1024;
    static constexpr int D_COLS = DT_NTILES * DT_DBUF * MP;              // accumulators: (tile, buffer)
    static constexpr int A_COLS = DT_ASTAGES * DT_NTILES * 32;     // A ring: 32 columns per (stage, tile)
    static constexpr int TMEM_COLS = 256;                          // half of the SM's tensor memory
    static_assert(D_COLS + A_COLS <= TMEM_COLS, "TMEM budget");
};

__device__ __forceinline__ void fold_bar_sync(int set) { asm volatile("bar.sync %0, 128;" ::"r"(1 + set) : "memory"); }

// BITS: 4 | 8.  T: __half | __nv_bfloat16 (int8 needs __half).  MLD: batch rows the fold reads
// (1, 2, 4, 8 or 16, >= M; the MMA always runs N = 16).  KPB: k-blocks (64 k) per fold (1 | 2 | 4).
template <int BITS, typename T, int MLD, int KPB>
__global__ void __launch_bounds__(DT_THREADS, 2)
qgemm_dtc_kernel(const DtcParams p) {
    constexpr int MP = 16;
    using S = DtcSmem<BITS, MP, KPB>;
    using H = F16x2<T>;
    constexpr int PACK = S::PACK, PROWS = S::PROWS, DT_PSTAGES = S::PSTAGES;
    constexpr bool SCALE_ODD = BITS == 4 && !H::kIsBf16;
    constexpr float MAGIC = H::kIsBf16 ? 128.f : 1024.f;
    constexpr int FP = KPB * 64;                      // k per fold

#ifdef MT_DTC_TIMING
    const long long t_entry = clock64();
    unsigned long long g_entry; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(g_entry));
#endif
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bar0 = sbase + S::OFF_BAR;
    auto bar_pfull = [&](int s) { return bar0 + 8u * s; };
    auto bar_pempty = [&](int s) { return bar0 + 8u * (DT_PSTAGES + s); };
    auto bar_afull = [&](int s) { return bar0 + 8u * (2 * DT_PSTAGES + s); };
    auto bar_aempty = [&](int s) { return bar0 + 8u * (2 * DT_PSTAGES + DT_ASTAGES + s); };
    auto bar_xfull = [&](int s) { return bar0 + 8u * (2 * DT_PSTAGES + 2 * DT_ASTAGES + s); };
    auto bar_xempty = [&](int s) { return bar0 + 8u * (2 * DT_PSTAGES + 2 * DT_ASTAGES + DT_XSLOTS + s); };
    auto bar_dfull = [&](int b) { return bar0 + 8u * (2 * DT_PSTAGES + 2 * DT_ASTAGES + 2 * DT_XSLOTS + b); };
    auto bar_dempty = [&](int b) { return bar0 + 8u * (2 * DT_PSTAGES + 2 * DT_ASTAGES + 2 * DT_XSLOTS + DT_DBUF + b); };
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + S::OFF_BAR + S::NBARS * 8);
    int* s_last = reinterpret_cast<int*>(smem + S::OFF_BAR + S::NBARS * 8 + 16);
    __shared__ int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int folds_per_group = p.gs / FP;
    // stream-K: the tiles x folds iteration space is cut into gridDim.x equal runs, one per CTA; a run
    // walks down K inside a column tile and continues at the top of the next tile
    const long long TF = p.total_folds;
    const int x0 = (int)((TF * blockIdx.x) / gridDim.x), x1 = (int)((TF * (blockIdx.x + 1)) / gridDim.x);

    if (tid == 0) {
        abort_flag = 0;
        for (int s = 0; s < DT_PSTAGES; ++s) { mbar_init(bar_pfull(s), 1); mbar_init(bar_pempty(s), 8); }
        for (int s = 0; s < DT_ASTAGES; ++s) { mbar_init(bar_afull(s), 256); mbar_init(bar_aempty(s), 1); }
        for (int s = 0; s < DT_XSLOTS; ++s) { mbar_init(bar_xfull(s), 1); mbar_init(bar_xempty(s), 129); }
        for (int b = 0; b < DT_DBUF; ++b) { mbar_init(bar_dfull(b), 1); mbar_init(bar_dempty(b), 128); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == DT_W_MMA) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)S::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_a = tmem_base + S::D_COLS;

    // segment = the part of the CTA's run that lies in one column tile: folds [f0, f1) of `tile`
#define MT_FOR_SEGMENTS for (int x = x0, tile, f0, f1; x < x1 && ok && (tile = x / p.fpt, f0 = x - tile * p.fpt, f1 = min(p.fpt, f0 + x1 - x), true); x += f1 - f0)
#ifdef MT_DTC_TIMING
    long long tw[6] = {0, 0, 0, 0, 0, 0};
    const long long t_begin = clock64();
    int tslot = 0;
    auto wait = [&](uint32_t bar, uint32_t parity) {
        const long long t0 = clock64();
        const bool r = mbar_wait(bar, parity, &abort_flag);
        tw[tslot] += clock64() - t0;
        return r;
    };
#define MT_SLOT(n) tslot = n
#define MT_TIC long long _tic = clock64()
#define MT_TOC(n) do { const long long _now = clock64(); tw[n] += _now - _tic; _tic = _now; } while (0)
#else
    auto wait = [&](uint32_t bar, uint32_t parity) { return mbar_wait(bar, parity, &abort_flag); };
#define MT_SLOT(n)
#define MT_TIC
#define MT_TOC(n)
#endif

    if (warp == DT_W_PROD) {
        // ------------------------------ bulk-copy producer ------------------------------
        // One 1-D bulk copy per packed row (DT_NT * 4 contiguous bytes), one lane per row.
        const uint32_t* __restrict__ qw = p.qw;
        int it = 0; bool ok = true;
        MT_FOR_SEGMENTS {
            const int col0 = tile * DT_NT;
            const uint32_t row_bytes = (uint32_t)min(DT_NT, p.n - col0) * 4u;
            for (int kb = f0 * KPB; kb < f1 * KPB; ++kb, ++it) {
                const int s = it % DT_PSTAGES; const uint32_t ph = (it / DT_PSTAGES) & 1;
                if (!wait(bar_pempty(s), ph ^ 1)) { ok = false; break; }
                if (lane == 0) mbar_expect_tx(bar_pfull(s), row_bytes * PROWS);
                __syncwarp();
                if (lane < PROWS) {
                    const uint32_t dst = sbase + S::OFF_P + s * S::P_BYTES + lane * (DT_NT * 4);
                    const uint32_t* src = qw + (size_t)(kb * PROWS + lane) * p.n + col0;
                    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                 ::"r"(dst), "l"(src), "r"(row_bytes), "r"(bar_pfull(s)) : "memory");
                }
            }
        }
    } else if (warp == DT_W_MMA) {
        // ------------------------------ MMA issuer ------------------------------
        // One thread; the MMAs of the two column tiles are interleaved so that consecutive
        // instructions accumulate into different TMEM regions (independent chains).
        if (lane == 0) {
            const uint32_t fmt = H::kIsBf16 ? 1u : 0u;
            const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(MP >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
            int ait = 0, fit = 0; bool ok = true;
            MT_FOR_SEGMENTS {
                for (int f = f0; f < f1 && ok; ++f, ++fit) {
                    const int xs = fit % DT_XSLOTS; const uint32_t xph = (fit / DT_XSLOTS) & 1;
                    const int buf = fit % DT_DBUF; const uint32_t dph = (fit / DT_DBUF) & 1;
                    MT_SLOT(0); if (!wait(bar_xfull(xs), xph)) { ok = false; break; }
                    MT_SLOT(1); if (!wait(bar_dempty(buf), dph ^ 1)) { ok = false; break; }
                    for (int kb = 0; kb < KPB; ++kb, ++ait) {
                        const int as = ait % DT_ASTAGES; const uint32_t aph = (ait / DT_ASTAGES) & 1;
                        MT_SLOT(2); if (!wait(bar_afull(as), aph)) { ok = false; break; }
                        MT_TIC;
                        tc_fence_after();
                        const uint64_t bdesc = tc_desc_sw128(sbase + S::OFF_X + xs * S::XSLOT_STRIDE + kb * S::XB_BYTES);
#pragma unroll
                        for (int k4 = 0; k4 < 4; ++k4)
#pragma unroll
                            for (int nt = 0; nt < DT_NTILES; ++nt)
                                tc_mma_ts(tmem_base + (uint32_t)((nt * DT_DBUF + buf) * MP),
                                          tmem_a + (uint32_t)((as * DT_NTILES + nt) * 32 + k4 * 8),
                                          bdesc + (uint64_t)(k4 * 2), idesc, (kb | k4) != 0 ? 1u : 0u);
                        tc_commit(bar_aempty(as));
                        MT_TOC(3);
                    }
                    if (ok) { tc_commit(bar_dfull(buf)); tc_commit(bar_xempty(xs)); }
                }
            }
        }
    } else if (warp == DT_W_X) {
        // ------------------------------ x warp ------------------------------
        // Only rows < M are staged; the padding rows of every slot are zeroed once and stay zero.
        const T* __restrict__ xg = reinterpret_cast<const T*>(p.x);
        constexpr int UPR = 8 * KPB;                   // 16-byte units per batch row per fold
        for (int i = lane; i < DT_XSLOTS * S::XSLOT_STRIDE / 16; i += 32)
            reinterpret_cast<uint4*>(smem + S::OFF_X)[i] = make_uint4(0, 0, 0, 0);
        fence_proxy_async();
        __syncwarp();
        const int nu = p.m * UPR;                      // units per fold that carry data
        // the first 32 units of a fold are fetched one fold ahead (all of them when M * UPR <= 32)
        auto fetch0 = [&](int f) {
            uint4 v = make_uint4(0, 0, 0, 0);
            if (lane < nu) v = __ldg(reinterpret_cast<const uint4*>(xg + (size_t)(lane / UPR) * p.k + f * FP + (lane % UPR) * 8));
            return v;
        };
        uint4 v_next = make_uint4(0, 0, 0, 0);
        if (x0 < x1) v_next = fetch0(x0 % p.fpt);
        int fit = 0; bool ok = true;
        MT_FOR_SEGMENTS {
            for (int f = f0; f < f1; ++f, ++fit) {
                const int xs = fit % DT_XSLOTS; const uint32_t xph = (fit / DT_XSLOTS) & 1;
                const uint4 v_first = v_next;
                if (f + 1 < f1) v_next = fetch0(f + 1);
                else if (x + (f1 - f0) < x1) v_next = fetch0(0);   // the next segment starts at the top of the next tile
                if (!wait(bar_xempty(xs), xph ^ 1)) { ok = false; break; }
                unsigned char* slot = smem + S::OFF_X + xs * S::XSLOT_STRIDE;
                float* X1 = reinterpret_cast<float*>(slot + KPB * S::XB_BYTES);
                float* X2 = X1 + MP;
                for (int u0 = 0; u0 < nu; u0 += 32) {
                    const int u = u0 + lane;
                    const int row = u / UPR, c = u % UPR;
                    uint4 v = v_first;
                    if (u0 > 0) {
                        v = make_uint4(0, 0, 0, 0);
                        if (u < nu) v = __ldg(reinterpret_cast<const uint4*>(xg + (size_t)row * p.k + f * FP + c * 8));
                    }
                    if constexpr (SCALE_ODD) {
                        const uint32_t one_sixteenth = 0x2c003c00u;      // (1.0, 1/16)
                        v.x = H::mul(v.x, one_sixteenth); v.y = H::mul(v.y, one_sixteenth);
                        v.z = H::mul(v.z, one_sixteenth); v.w = H::mul(v.w, one_sixteenth);
                    }
                    float seen = 0.f, eff = 0.f;
                    const uint32_t vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const float lo = H::to_float(uint16_t(vv[q] & 0xffffu)), hi = H::to_float(uint16_t(vv[q] >> 16));
                        seen += lo + hi;
                        eff += lo + (SCALE_ODD ? 16.f * hi : hi);
                    }
#pragma unroll
                    for (int d = UPR / 2; d >= 1; d >>= 1) {
                        seen += __shfl_xor_sync(0xffffffffu, seen, d);
                        eff += __shfl_xor_sync(0xffffffffu, eff, d);
                    }
                    if (u < nu) {
                        if (c == 0) { X1[row] = MAGIC * seen; X2[row] = eff; }
                        if constexpr (BITS == 4) {   // (h0..h7) -> (h0,h4,h1,h5,h2,h6,h3,h7): the k-slot order of the A registers
                            uint4 o;
                            o.x = prmt(v.x, v.z, 0x5410u); o.y = prmt(v.x, v.z, 0x7632u);
                            o.z = prmt(v.y, v.w, 0x5410u); o.w = prmt(v.y, v.w, 0x7632u);
                            v = o;
                        }
                        const int kb = c >> 3, ch = c & 7;
                        *reinterpret_cast<uint4*>(slot + kb * S::XB_BYTES + (row >> 3) * 1024 + (row & 7) * 128 + ((ch ^ (row & 7)) << 4)) = v;
                    }
                }
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_xfull(xs));
            }
        }
    } else if (warp >= DT_W_CONV && warp < DT_W_CONV + 8) {
        // ------------------------------ converter warps ------------------------------
        const int j = warp - DT_W_CONV;                 // 0..7
        const int nt = j >> 2;                          // column tile of 128
        const int q4 = warp & 3;                        // TMEM lane quarter (== j & 3)
        const int ccol = nt * 128 + q4 * 32 + lane;     // column inside the CTA tile
        int it = 0; bool ok = true;
        MT_FOR_SEGMENTS {
            for (int kb = f0 * KPB; kb < f1 * KPB; ++kb, ++it) {
                const int s = it % DT_PSTAGES; const uint32_t ph = (it / DT_PSTAGES) & 1;
                const int as = it % DT_ASTAGES; const uint32_t aph = (it / DT_ASTAGES) & 1;
                MT_SLOT(0); if (!wait(bar_pfull(s), ph)) { ok = false; break; }
                MT_TIC;
                const uint32_t* pk = reinterpret_cast<const uint32_t*>(smem + S::OFF_P + s * S::P_BYTES) + ccol;
                uint32_t a[32];
#pragma unroll
                for (int r = 0; r < PROWS; ++r) {
                    const uint32_t w = pk[r * DT_NT];
                    if constexpr (BITS == 4) {
                        if constexpr (!H::kIsBf16) {
                            const uint32_t w8 = w >> 8;
                            a[4 * r + 0] = and_or(w, 0x000f000fu, 0x64006400u);    // 1024 + (q0, q4)
                            a[4 * r + 1] = and_or(w, 0x00f000f0u, 0x64006400u);    // 1024 + 16 (q1, q5)
                            a[4 * r + 2] = and_or(w8, 0x000f000fu, 0x64006400u);   // 1024 + (q2, q6)
                            a[4 * r + 3] = and_or(w8, 0x00f000f0u, 0x64006400u);   // 1024 + 16 (q3, q7)
                        } else {
#pragma unroll
                            for (int q = 0; q < 4; ++q) a[4 * r + q] = and_or(w >> (4 * q), 0x000f000fu, 0x43004300u);
                        }
                    } else {
                        a[2 * r + 0] = prmt(w, 0x64646464u, 0x4140u);              // 1024 + (b0, b1)
                        a[2 * r + 1] = prmt(w, 0x64646464u, 0x4342u);              // 1024 + (b2, b3)
                    }
                }
                // the packed stage has been read into registers: give it back to the producer
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_pempty(s));
                MT_TOC(2);
                MT_SLOT(1); if (!wait(bar_aempty(as), aph ^ 1)) { ok = false; break; }
#ifdef MT_DTC_TIMING
                _tic = clock64();
#endif
                tc_fence_after();
                tc_st32(tmem_a + ((uint32_t)(q4 * 32) << 16) + (uint32_t)((as * DT_NTILES + nt) * 32), a);
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                tc_fence_before();
                mbar_arrive(bar_afull(as));
                MT_TOC(3);
            }
        }
    } else if (warp < DT_W_CONV) {
        // ------------------------------ fold warps ------------------------------
        const int q4 = warp & 3;                        // TMEM lane quarter
        const int nl = q4 * 32 + lane;                  // column inside a 128-column tile
        const T* __restrict__ sg = reinterpret_cast<const T*>(p.scales);
        const T* __restrict__ bias = reinterpret_cast<const T*>(p.bias);
        T* __restrict__ out = reinterpret_cast<T*>(p.out);
        constexpr uint32_t ZMASK = (1u << BITS) - 1u;
        int fit0 = 0; bool ok = true;                   // fold counter at the start of the unit
        MT_FOR_SEGMENTS {
            // CTAs that contribute to this tile: those whose runs intersect [tile * fpt, (tile + 1) * fpt)
            const int c_first = (int)((((long long)tile * p.fpt + 1) * gridDim.x - 1) / TF);
            const int c_last = (int)((((long long)(tile + 1) * p.fpt) * gridDim.x - 1) / TF);
            const int nparts = c_last - c_first + 1, rank = (int)blockIdx.x - c_first;
            int ncol[DT_NTILES]; bool nok[DT_NTILES]; int zsh[DT_NTILES];
#pragma unroll
            for (int nt = 0; nt < DT_NTILES; ++nt) {
                ncol[nt] = tile * DT_NT + nt * 128 + nl; nok[nt] = ncol[nt] < p.n; zsh[nt] = (ncol[nt] % PACK) * BITS;
            }
            float oacc[DT_NTILES][MLD];
#pragma unroll
            for (int nt = 0; nt < DT_NTILES; ++nt)
#pragma unroll
                for (int m = 0; m < MLD; ++m) oacc[nt][m] = 0.f;
            // Scales and zeros stream from HBM (nothing else reads them), so their latency is a full
            // DRAM round trip under load: they are fetched PF folds ahead into a small register ring.
            constexpr int PF = 4;
            uint32_t sraw[PF][DT_NTILES], zraw[PF][DT_NTILES];
            auto load_raw = [&](int slot, int f) {   // nothing may depend on these loads until PF folds later
                const int g = f / folds_per_group;
#pragma unroll
                for (int nt = 0; nt < DT_NTILES; ++nt) {
                    sraw[slot][nt] = 0u; zraw[slot][nt] = 0u;
                    if (nok[nt] && f < f1) {
                        sraw[slot][nt] = (uint32_t)__ldg(reinterpret_cast<const uint16_t*>(sg) + (size_t)g * p.n + ncol[nt]);
                        if (p.qz) zraw[slot][nt] = __ldg(p.qz + (size_t)g * (p.n / PACK) + ncol[nt] / PACK);
                    }
                }
            };
#pragma unroll
            for (int i = 0; i < PF; ++i) load_raw(i, f0 + i);
            for (int f = f0; f < f1 && ok; ++f) {
                MT_TIC;
                const int fit = fit0 + (f - f0);
                const int xs = fit % DT_XSLOTS; const uint32_t xph = (fit / DT_XSLOTS) & 1;
                const int buf = fit % DT_DBUF; const uint32_t dph = (fit / DT_DBUF) & 1;
                float sc[DT_NTILES], zp[DT_NTILES];
#pragma unroll
                for (int nt = 0; nt < DT_NTILES; ++nt) {
                    sc[nt] = H::to_float(uint16_t(sraw[0][nt]));
                    zp[nt] = p.qz ? float(((zraw[0][nt] >> zsh[nt]) & ZMASK) + 1u) : float(p.zp1_const);
                }
#pragma unroll
                for (int i = 0; i + 1 < PF; ++i)
#pragma unroll
                    for (int nt = 0; nt < DT_NTILES; ++nt) { sraw[i][nt] = sraw[i + 1][nt]; zraw[i][nt] = zraw[i + 1][nt]; }
                load_raw(PF - 1, f + PF);
                MT_TOC(2);
                MT_SLOT(0); if (!wait(bar_xfull(xs), xph)) { ok = false; break; }
                MT_SLOT(1); if (!wait(bar_dfull(buf), dph)) { ok = false; break; }
#ifdef MT_DTC_TIMING
                _tic = clock64();
#endif
                tc_fence_after();
                const float* X1 = reinterpret_cast<const float*>(smem + S::OFF_X + xs * S::XSLOT_STRIDE + KPB * S::XB_BYTES);
                const float* X2 = X1 + MP;
                uint32_t r[DT_NTILES][MLD];
#pragma unroll
                for (int nt = 0; nt < DT_NTILES; ++nt)
                    tc_ld<MLD>(tmem_base + ((uint32_t)(q4 * 32) << 16) + (uint32_t)((nt * DT_DBUF + buf) * MP), r[nt]);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int m = 0; m < MLD; ++m) {
                    const float x1 = X1[m], x2 = X2[m];
#pragma unroll
                    for (int nt = 0; nt < DT_NTILES; ++nt) {
                        const float v = fmaf(-zp[nt], x2, __uint_as_float(r[nt][m]) - x1);
                        oacc[nt][m] = fmaf(sc[nt], v, oacc[nt][m]);
                    }
                }
                tc_fence_before();
                mbar_arrive(bar_dempty(buf));
                mbar_arrive(bar_xempty(xs));
                MT_TOC(3);
            }
            fit0 += f1 - f0;
            if (!ok) break;
            MT_TIC;
            // ---- unit epilogue: direct store, or an fp32 partial per split and last-arriver reduction ----
            if (nparts == 1) {
#pragma unroll
                for (int nt = 0; nt < DT_NTILES; ++nt)
                    if (nok[nt]) {
                        const float bv = bias ? H::to_float(reinterpret_cast<const uint16_t*>(bias)[ncol[nt]]) : 0.f;
#pragma unroll
                        for (int m = 0; m < MLD; ++m)
                            if (m < p.m) reinterpret_cast<uint16_t*>(out)[(size_t)m * p.n + ncol[nt]] = H::from_float(oacc[nt][m] + bv);
                    }
                continue;
            }
#pragma unroll
            for (int nt = 0; nt < DT_NTILES; ++nt)
                if (nok[nt]) {
#pragma unroll
                    for (int m = 0; m < MLD; ++m)
                        if (m < p.m) __stcg(p.partial + ((size_t)rank * p.m + m) * p.n + ncol[nt], oacc[nt][m]);
                }
            __threadfence();
            fold_bar_sync(0);
            if (q4 == 0 && lane == 0) s_last[0] = (atomicAdd(p.counters + tile, 1u) == unsigned(nparts - 1));
            fold_bar_sync(0);
            if (s_last[0]) {
                __threadfence();
#pragma unroll
                for (int nt = 0; nt < DT_NTILES; ++nt)
                    if (nok[nt]) {
                        const float bv = bias ? H::to_float(reinterpret_cast<const uint16_t*>(bias)[ncol[nt]]) : 0.f;
                        for (int m = 0; m < p.m; ++m) {
                            float sum = 0.f;
                            for (int s = 0; s < nparts; ++s) sum += __ldcg(p.partial + ((size_t)s * p.m + m) * p.n + ncol[nt]);
                            reinterpret_cast<uint16_t*>(out)[(size_t)m * p.n + ncol[nt]] = H::from_float(sum + bv);
                        }
                    }
                if (q4 == 0 && lane == 0) p.counters[tile] = 0;
            }
            fold_bar_sync(0);   // s_last[0] is reused by the next unit
            MT_TOC(4);
        }
    }

#ifdef MT_DTC_TIMING
    if (blockIdx.x == 0 && lane == 0) {
        long long* dst = reinterpret_cast<long long*>(p.counters + 2048) + warp * 6;
        dst[0] = clock64() - t_begin;
        for (int i = 0; i < 5; ++i) dst[1 + i] = tw[i];
        if (warp == DT_W_PROD) {   // whole-kernel phases: entry -> roles start, globaltimer at entry and at role end
            unsigned long long g_now; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(g_now));
            dst[3] = t_begin - t_entry; dst[4] = (long long)g_entry; dst[5] = (long long)g_now;
        }
    }
#endif
    tc_fence_before();
    __syncthreads();
    if (warp == DT_W_MMA) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)S::TMEM_COLS) : "memory");
    }
    if (tid == 0 && abort_flag && p.err) atomicExch(p.err, 3u);
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
static int fold_k(int gs) { return gs % 256 == 0 ? 256 : gs % 128 == 0 ? 128 : gs % 64 == 0 ? 64 : 0; }

static void dtc_plan(const QGemmArgs& a, int& grid, int& max_parts);

bool dtc_supported(const QGemmArgs& a) {
    if (a.g_idx != nullptr || a.m < 1 || a.m > 16) return false;
    if (a.bits == 8 && a.dtype == MT_BF16) return false;          // 128 + b is not exact in bf16 for b >= 128
    const int gs = a.k / a.groups;
    if (fold_k(gs) == 0) return false;
    if (a.workspace == nullptr || a.workspace_bytes < kCounterBytes) return false;
    if ((a.n + DT_NT - 1) / DT_NT >= kMaxTiles) return false;
    int grid, max_parts;
    dtc_plan(a, grid, max_parts);
    return (size_t)max_parts * a.m * a.n * 4 <= a.workspace_bytes - kCounterBytes;
}

template <int BITS, typename T, int MLD, int KPB>
static int launch_dtc_inst(cudaStream_t st, const DtcParams& p, int grid) {
    using S = DtcSmem<BITS, 16, KPB>;
    auto kern = qgemm_dtc_kernel<BITS, T, MLD, KPB>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL) != cudaSuccess) {
        cudaGetLastError();
        return MT_ERR_TOO_LARGE;
    }
    kern<<<grid, DT_THREADS, S::TOTAL, st>>>(p);
    return cudaGetLastError() == cudaSuccess ? MT_OK : MT_ERR_CUDA;
}

template <int BITS, typename T>
static int launch_dtc_t(cudaStream_t st, const DtcParams& p, int grid, int kpb) {
#define MT_K(MLD_) \
    (kpb == 4 ? launch_dtc_inst<BITS, T, MLD_, 4>(st, p, grid) : kpb == 2 ? launch_dtc_inst<BITS, T, MLD_, 2>(st, p, grid) \
                                                                        : launch_dtc_inst<BITS, T, MLD_, 1>(st, p, grid))
    if (p.m == 1) return MT_K(1);
    if (p.m == 2) return MT_K(2);
    if (p.m <= 4) return MT_K(4);
    if (p.m <= 8) return MT_K(8);
    return MT_K(16);
#undef MT_K
}

// grid size and the largest number of CTAs that can contribute to one column tile
static void dtc_plan(const QGemmArgs& a, int& grid, int& max_parts) {
    const int gs = a.k / a.groups;
    const int fp = fold_k(gs);
    const int tiles = (a.n + DT_NT - 1) / DT_NT;
    const int fpt = a.k / fp;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const long long total = (long long)tiles * fpt;
    grid = (int)(total < 2LL * sms ? total : 2LL * sms);
    const long long per = total / grid;                       // >= 1
    max_parts = (int)((fpt + per - 1) / per) + 1;
}

int launch_dtc(cudaStream_t st, const QGemmArgs& a) {
    const int gs = a.k / a.groups;
    const int fp = fold_k(gs);
    const int tiles = (a.n + DT_NT - 1) / DT_NT;
    int grid, max_parts;
    dtc_plan(a, grid, max_parts);
    DtcParams p;
    p.x = a.x; p.qw = a.qweight; p.qz = a.qzeros; p.scales = a.scales; p.bias = a.bias; p.out = a.out;
    p.counters = static_cast<unsigned*>(a.workspace);
    p.err = p.counters + (kMaxTiles - 1);
    p.partial = reinterpret_cast<float*>(static_cast<char*>(a.workspace) + kCounterBytes);
    p.m = a.m; p.n = a.n; p.k = a.k; p.groups = a.groups; p.gs = gs;
    p.tiles = tiles; p.fpt = a.k / fp; p.total_folds = tiles * p.fpt;
    p.zp1_const = 1 << (a.bits - 1);
    const int kpb = fp / 64;
    if (a.bits == 4) return a.dtype == MT_F16 ? launch_dtc_t<4, __half>(st, p, grid, kpb) : launch_dtc_t<4, __nv_bfloat16>(st, p, grid, kpb);
    return launch_dtc_t<8, __half>(st, p, grid, kpb);
}

}  // namespace mt
