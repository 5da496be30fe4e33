// Mid-size batches (2 < M <= 64 per pass) for GPTQ weights with contiguous groups: every warp
// dequantizes, the tensor core multiplies.
//
// Why another kernel: between the CUDA-core GEMV (M <= 2) and the prefill kernels (M >= 256) the
// other kernels are bound by how fast weights are CONVERTED, not by HBM or by the tensor pipe: the
// register-ring kernel by the legacy mma.sync rate (one m16n8k16 per 32 cycles per scheduler), the
// prefill kernels by their four dequantizing warps (minit/quantize/tensor.py:29-30 materialises the
// whole fp16 matrix instead; examples/qwen1_5_int8.py:156-200 converts per thread and per row).
// Here the roles are sized for the stream:
//
//   16 converter warps  four groups of four; a thread owns one TMEM lane = one column of each of the
//                       CTA's two 128-column tiles and converts every fourth k-block of the run: it
//                       reads the packed words of its columns from the bulk-copy ring, rebuilds W = (q - (z+1)) * s exactly as the
//                       dequantizer does (magic-number int->fp16, subtract, one multiply), and
//                       writes the 64 values of a k-block into TENSOR MEMORY with one tcgen05.st:
//                       the A operand never touches shared memory.
//   1 MMA warp          tcgen05.mma.kind::f16, M = 128 columns of W, N = BM batch rows, K = 16, A from
//                       TMEM, B from shared memory, fp32 accumulators in TMEM for the CTA's whole
//                       run of a column tile (scales are already in the weights: no per-group fold).
//                       One such MMA costs ~46 cycles whatever N <= 91: the HBM rate at N = 16 and 64 alike.
//   1 producer warp     one 2-D tensor copy (TMA) per k-block of the CTA tile into an 8-stage ring: 64 KB
//                       in flight per SM, tracked by the copy engine.
//   2 loader warps      x[m, k-block] -> the B operand tile (K-major, 128-byte swizzle), k-slots in the
//                       order the converter produces them.
//   epilogue            the converter warps drain the accumulators at the end of a run's part of a tile
//                       (group -> one 128-column tile and half of the batch rows).
// Stream-K: the (256-column tile, k-block) units are cut into equal runs, one per CTA (one CTA per
// SM); a tile shared by several CTAs is completed by the last one to arrive (fp32 partial tiles).
// Every mbarrier wait is bounded and reports through the workspace error word.
#include <stdlib.h>
#include "tma.cuh"
#include "tcgen05.cuh"

namespace mt {
namespace {

constexpr int UM_NT = 2;                    // 128-column MMA tiles per CTA tile
constexpr int UM_COLS = UM_NT * 128;        // 256 columns
constexpr int UM_CONV = 16;                 // converter warps: 4 groups x 4 TMEM lane quarters (a thread feeds both tiles)
constexpr int UM_GROUPS = UM_CONV / 4;
constexpr int UM_W_MMA = UM_CONV;           // warp 16
constexpr int UM_W_LOAD = UM_CONV + 1;      // warps 17, 18
constexpr int UM_LOADERS = 2;
constexpr int UM_W_PROD = UM_W_LOAD + UM_LOADERS;   // warp 19: bulk-copy producer of the packed weights
constexpr int UM_THREADS = (UM_CONV + 1 + UM_LOADERS + 1) * 32;   // 640
constexpr int UM_ASTAGES = 6;               // A ring in TMEM (k-blocks): 6 x 64 columns + 128 accumulator columns = all 512
constexpr int UM_NPAIR = UM_ASTAGES / 2;     // k-block pairs in the rings
constexpr int UM_BSTAGES = UM_ASTAGES;      // B ring in shared memory: slot i % 4 like the A ring, so one barrier frees both
constexpr int UM_XSTAGES = 6;               // raw activation tiles in flight per loader (k-blocks)

struct UmParams {
    const void* x; const uint32_t* qw; const uint32_t* qz; const void* scales; const void* bias; void* out;
    float* partial; unsigned* counters; unsigned* err;
    int m, n, k, groups, gs;
    int tiles, kbt;          // column tiles, k-blocks (64 values of k) per tile
    int units, per, rem;     // tiles * kbt units; CTA c gets per (+1 if c < rem) units
    int zp1_const;
};

// Bounded wait that does not poll: mbarrier.try_wait with a suspend-time hint parks the thread until the
// phase completes or the hint expires, so waiting warps leave the issue slots to the converters.
__device__ __forceinline__ bool um_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    for (int i = 0; i < (1 << 20); ++i) {                // ~1 us per turn: gives up after about a second
        uint32_t ok;
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\nselp.b32 %0, 1, 0, p;\n}"
                     : "=r"(ok) : "r"(bar), "r"(parity), "r"(1000u) : "memory");
        if (ok) return true;
        if ((i & 63) == 63 && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}

template <int BITS, int BM> struct UmSmem {
    static constexpr int PROWS = 64 / (32 / BITS);                    // packed rows per k-block: 8 | 16
    static constexpr int P_BYTES = PROWS * UM_COLS * 4;               // packed words of one k-block of the CTA tile: 8 | 16 KB
    static constexpr int PSTAGES = BITS == 4 ? 8 : 4;                 // 64 KB of packed weights in flight per SM
    static constexpr int B_BYTES = BM * 128;                          // one B tile: BM rows x 64 k
    static constexpr int OFF_P = 0;
    static constexpr int OFF_B = OFF_P + PSTAGES * P_BYTES;
    static constexpr int OFF_XS = OFF_B + UM_BSTAGES * B_BYTES;      // staging ring of raw activation tiles
    static constexpr int OFF_BAR = OFF_XS + UM_XSTAGES * B_BYTES;
    static constexpr int NBARS = 2 * UM_ASTAGES + 2 * UM_BSTAGES + 3 + 2 * PSTAGES;
    static constexpr int TOTAL = OFF_BAR + NBARS * 8 + 64 + 1024;
    static constexpr int D_COLS = UM_NT * BM;
    static constexpr int A_COLS = UM_ASTAGES * UM_NT * 32;
    static constexpr int TMEM_COLS = 512;
    static_assert(D_COLS + A_COLS <= TMEM_COLS, "TMEM budget");
};

// BITS 4 | 8; T __half | __nv_bfloat16 (8-bit needs __half: 128 + b is not exact in bf16); BM batch rows per pass (16 | 32 | 64)
template <int BITS, typename T, int BM>
__global__ void __launch_bounds__(UM_THREADS, 1) qgemm_umma_kernel(const __grid_constant__ CUtensorMap tmap_q, const UmParams p) {
    using S = UmSmem<BITS, BM>;
    using H = F16x2<T>;
    constexpr int PACK = 32 / BITS, PROWS = 64 / PACK;               // packed rows per k-block: 8 | 16

    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bar0 = sbase + S::OFF_BAR;
    auto bar_afull = [&](int s) { return bar0 + 8u * s; };
    auto bar_aempty = [&](int s) { return bar0 + 8u * (UM_ASTAGES + s); };
    auto bar_bfull = [&](int s) { return bar0 + 8u * (2 * UM_ASTAGES + s); };
    auto bar_bempty = [&](int s) { return bar0 + 8u * (2 * UM_ASTAGES + UM_BSTAGES + s); };
    const uint32_t bar_dfull = bar0 + 8u * (2 * UM_ASTAGES + 2 * UM_BSTAGES);
    const uint32_t bar_dempty = bar_dfull + 8u;
    const uint32_t bar_esync = bar_dfull + 16u;          // the 16 converter warps meet here around a shared tile's hand-over
    auto bar_pfull = [&](int s) { return bar_dfull + 24u + 8u * s; };
    auto bar_pempty = [&](int s) { return bar_dfull + 24u + 8u * (S::PSTAGES + s); };
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + S::OFF_BAR + S::NBARS * 8);
    int* s_last = reinterpret_cast<int*>(smem + S::OFF_BAR + S::NBARS * 8 + 16);
    __shared__ int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int cta = blockIdx.x;
    const int x0 = cta * p.per + (cta < p.rem ? cta : p.rem);
    const int nrun = p.per + (cta < p.rem ? 1 : 0);

    if (tid == 0) {
        abort_flag = 0;
        // one full / empty barrier per PAIR of k-blocks (slots 2p, 2p+1): both operands of both k-blocks meet there, so the
        // MMA thread waits and commits once per 16 MMAs (its per-hand-off cost, not the MMAs, paces the kernel)
        for (int s = 0; s < UM_NPAIR; ++s) { mbar_init(bar_afull(s), 2 * (4 + 1)); mbar_init(bar_aempty(s), 1); }
        for (int s = 0; s < UM_BSTAGES; ++s) { mbar_init(bar_bfull(s), UM_LOADERS); mbar_init(bar_bempty(s), 1); }
        mbar_init(bar_dfull, 1); mbar_init(bar_dempty, UM_CONV); mbar_init(bar_esync, UM_CONV);
        for (int s = 0; s < S::PSTAGES; ++s) { mbar_init(bar_pfull(s), 1); mbar_init(bar_pempty(s), 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == UM_W_MMA) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)S::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_a = tmem_base + S::D_COLS;
    auto wait = [&](uint32_t bar, uint32_t parity) { return um_wait(bar, parity, &abort_flag); };

    // first / last CTA with a unit in column tile t
    auto owner = [&](int u) -> int {
        const int big = p.rem * (p.per + 1);
        return u < big ? u / (p.per + 1) : p.rem + (u - big) / p.per;
    };

    if (warp == UM_W_MMA) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            const uint32_t fmt = H::kIsBf16 ? 1u : 0u;
            const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(BM >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
            int seg = 0; bool ok = true;
            int kb = x0 % p.kbt;
            uint32_t aph = 0;                            // parity of the ring pass
            for (int i0 = 0; i0 < nrun && ok; i0 += UM_ASTAGES, aph ^= 1u) {
#pragma unroll
                for (int pr = 0; pr < UM_NPAIR; ++pr) {          // slot indices are static: addresses and descriptors fold to constants
                    if (i0 + 2 * pr >= nrun || !ok) break;
                    if (!wait(bar_afull(pr), aph)) { ok = false; break; }
                    tc_fence_after();
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int as = 2 * pr + h;
                        const int i = i0 + as;
                        if (i >= nrun) break;
                        const bool first = (i == 0) || (kb == 0);
                        const bool last = (i == nrun - 1) || (kb == p.kbt - 1);
                        kb = (kb + 1 == p.kbt) ? 0 : kb + 1;
                        if (first) { if (!wait(bar_dempty, (seg & 1) ^ 1)) { ok = false; break; } tc_fence_after(); }
                        const uint64_t bdesc = tc_desc_sw128(sbase + S::OFF_B + as * S::B_BYTES);
#pragma unroll
                        for (int k4 = 0; k4 < 4; ++k4)
#pragma unroll
                            for (int nt = 0; nt < UM_NT; ++nt)
                                tc_mma_ts(tmem_base + (uint32_t)(nt * BM), tmem_a + (uint32_t)((as * UM_NT + nt) * 32 + k4 * 8),
                                          bdesc + (uint64_t)(k4 * 2), idesc, (first && k4 == 0) ? 0u : 1u);
                        if (last) { tc_commit(bar_dfull); ++seg; }
                    }
                    if (!ok) break;
                    tc_commit(bar_aempty(pr));           // frees the A and B slots of both k-blocks
                }
            }
        }
    } else if (warp == UM_W_PROD) {
        // ------------------------------ packed-weight producer ------------------------------
        // One 2-D tensor copy per k-block: the box is the CTA tile's 256 columns x the k-block's packed rows
        // (8 | 16 KB; columns beyond N are zero-filled).  The copy engine tracks the bytes in flight, not the
        // load/store unit: 4-byte loads per thread capped the SM near 1.4 TB/s, and one 1 KB bulk copy per
        // packed row is eight times the descriptors for the same bytes.
        int tile = x0 / p.kbt, kb = x0 - tile * p.kbt;
        bool ok = true;
        for (int i = 0; i < nrun && ok; ++i) {
            const int ps = i % S::PSTAGES; const uint32_t pph = (i / S::PSTAGES) & 1;
            if (!wait(bar_pempty(ps), pph ^ 1)) { ok = false; break; }
            if (lane == 0) {
                mbar_expect_tx(bar_pfull(ps), (uint32_t)S::P_BYTES);
                tma_load_2d(sbase + S::OFF_P + ps * S::P_BYTES, &tmap_q, tile * UM_COLS, kb * PROWS, bar_pfull(ps));
            }
            __syncwarp();
            if (++kb == p.kbt) { kb = 0; ++tile; }
        }
    } else if (warp >= UM_W_LOAD) {
        // ------------------------------ B loaders ------------------------------
        // Loader lw builds the operand tiles of k-blocks lw, lw + 2, ... (two independent chains hide each
        // other's latencies).  A tile is BM rows x 8 units of 16 bytes.  A lane copies its units raw into a
        // staging ring with cp.async, three of its k-blocks ahead (an L2 round trip per k-block would
        // otherwise pace the whole kernel), and later moves the ones it copied itself into the operand
        // tile, permuting the k-slots on the way.
        const int lw = warp - UM_W_LOAD;
        constexpr int UPL = BM * 8 / 32;                 // units per lane per k-block
        constexpr int AHEAD = UM_XSTAGES / UM_LOADERS;   // k-blocks of this loader in flight
        const T* __restrict__ xg = reinterpret_cast<const T*>(p.x);
        const uint32_t stage_s = sbase + S::OFF_XS;
        auto issue = [&](int i) {
            if (i < nrun) {
                const int kb = (x0 + i) % p.kbt;
#pragma unroll
                for (int t = 0; t < UPL; ++t) {
                    const int un = t * 32 + lane;
                    const int row = un >> 3, ch = un & 7;
                    const bool live = row < p.m;
                    const T* src = xg + (live ? (size_t)row * p.k + (size_t)kb * 64 + ch * 8 : 0);
                    const int sz = live ? 16 : 0;        // rows beyond M: zero fill
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;"
                                 ::"r"(stage_s + uint32_t((i % UM_XSTAGES) * S::B_BYTES + un * 16)), "l"(src), "r"(sz) : "memory");
                }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
#pragma unroll
        for (int d = 0; d < AHEAD - 1; ++d) issue(lw + UM_LOADERS * d);
        bool ok = true;
        const int nrun_pad = (nrun + 1) & ~1;            // the second k-block of the last pair may not exist: its owners still arrive
        for (int i = lw; i < nrun_pad && ok; i += UM_LOADERS) {
            issue(i + UM_LOADERS * (AHEAD - 1));
            asm volatile("cp.async.wait_group %0;" ::"n"(AHEAD - 1) : "memory");
            const int bs = i % UM_BSTAGES; const uint32_t bph = (i / UM_BSTAGES) & 1;
            const int pr = bs >> 1;
            if (!wait(bar_aempty(pr), bph ^ 1)) { ok = false; break; }
            if (i >= nrun) { __syncwarp(); if (lane == 0) mbar_arrive(bar_afull(pr)); continue; }
            unsigned char* tile_s = smem + S::OFF_B + bs * S::B_BYTES;
            const unsigned char* raw_s = smem + S::OFF_XS + (i % UM_XSTAGES) * S::B_BYTES;
#pragma unroll
            for (int t = 0; t < UPL; ++t) {
                const int un = t * 32 + lane;
                const int row = un >> 3, ch = un & 7;
                uint4 v = *reinterpret_cast<const uint4*>(raw_s + un * 16);
                if constexpr (BITS == 4) {               // (h0..h7) -> (h0,h4,h1,h5,h2,h6,h3,h7): the k-slot order of the A registers
                    uint4 o;
                    o.x = prmt(v.x, v.z, 0x5410u); o.y = prmt(v.x, v.z, 0x7632u);
                    o.z = prmt(v.y, v.w, 0x5410u); o.w = prmt(v.y, v.w, 0x7632u);
                    v = o;
                }
                *reinterpret_cast<uint4*>(tile_s + (row >> 3) * 1024 + (row & 7) * 128 + ((ch ^ (row & 7)) << 4)) = v;
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_afull(pr));
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
    } else {
        // ------------------------------ converter warps (+ epilogue) ------------------------------
        // warp = (group, TMEM lane quarter); a thread owns one lane = column cc of BOTH 128-column tiles, and
        // its group converts every UM_GROUPS-th k-block of the run.  All per-k-block bookkeeping (tile,
        // k-block, scale group, addresses) advances incrementally: a thread converts only 128 weights per
        // turn, so a division per turn would cost as much as the conversion.
        const int grp = warp >> 2;                       // 0..3
        const int q4 = warp & 3;                         // TMEM lane quarter
        const int cl = q4 * 32 + lane;                   // column inside a 128-column tile
        const T* __restrict__ sg = reinterpret_cast<const T*>(p.scales);
        const T* __restrict__ bias = reinterpret_cast<const T*>(p.bias);
        uint16_t* __restrict__ out = reinterpret_cast<uint16_t*>(p.out);
        constexpr uint32_t ZMASK = (1u << BITS) - 1u;
        const int kpg = p.gs / 64;                       // k-blocks per scale group
        const size_t row_words = (size_t)p.n;

        // scale / zero iterator: unit index, its tile / k-block / group, advancing by UM_GROUPS units per turn;
        // the words of the NEXT turn are loaded at the start of each turn
        int f_i = grp;
        int f_tile = (x0 + f_i) / p.kbt, f_kb = (x0 + f_i) - f_tile * p.kbt;
        int f_g = f_kb / kpg, f_kin = f_kb - f_g * kpg;
        constexpr int SZ = 3;                            // turns of scale / zero words in flight: they stream from HBM (nothing
                                                         // else reads them), so one turn ahead is less than their latency
        uint32_t sr[UM_NT], zr[UM_NT], sr_n[SZ][UM_NT], zr_n[SZ][UM_NT];
        auto fetch = [&](uint32_t (&s)[UM_NT], uint32_t (&z)[UM_NT]) {
            const bool live = f_i < nrun;
#pragma unroll
            for (int nt = 0; nt < UM_NT; ++nt) {
                const int col = f_tile * UM_COLS + nt * 128 + cl;
                s[nt] = 0u; z[nt] = 0u;
                if (live && col < p.n) {
                    s[nt] = (uint32_t)__ldg(reinterpret_cast<const uint16_t*>(sg) + (size_t)f_g * row_words + col);
                    if (p.qz) z[nt] = __ldg(p.qz + (size_t)f_g * (p.n / PACK) + col / PACK);
                }
            }
            f_i += UM_GROUPS; f_kb += UM_GROUPS; f_kin += UM_GROUPS;
            while (f_kin >= kpg) { f_kin -= kpg; ++f_g; }
            if (f_kb >= p.kbt) {                         // next column tile
                f_kb -= p.kbt; ++f_tile;
                if (f_kb >= p.kbt) { f_tile += f_kb / p.kbt; f_kb %= p.kbt; }
                f_g = f_kb / kpg; f_kin = f_kb - f_g * kpg;
            }
        };
#pragma unroll
        for (int d = 0; d < SZ; ++d) fetch(sr_n[d], zr_n[d]);

        int seg = 0, nsync = 0; bool ok = true;
        // bounded meeting of the converter warps (an mbarrier, not bar.sync: a warp that gave up must not hang the others)
        auto conv_sync = [&]() {
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_esync);
            if (!wait(bar_esync, nsync & 1)) ok = false;
            ++nsync;
        };
        // the finished part of a column tile: stored, or handed over as an fp32 partial tile.  The sixteen warps
        // split the accumulator: group -> (128-column tile, half of the batch rows).
        auto epilogue = [&](int tile) {
            if (!wait(bar_dfull, seg & 1)) { ok = false; return; }
            tc_fence_after();
            const int nt = grp & 1;
            const int cc = nt * 128 + cl;
            const int col = tile * UM_COLS + cc;
            const bool okc = col < p.n;
            const int cf = owner(tile * p.kbt), cla = owner(tile * p.kbt + p.kbt - 1);
            const int nparts = cla - cf + 1;
            constexpr int HALF = BM / 2;                 // batch rows this group drains
            const int j0 = (grp >> 1) * HALF;
            const float bv = (bias && okc) ? H::to_float(reinterpret_cast<const uint16_t*>(bias)[col]) : 0.f;
            float* part = p.partial + (size_t)(cta + tile) * BM * UM_COLS;
#pragma unroll
            for (int jb = 0; jb < HALF; jb += 8) {
                uint32_t r[8];
                tc_ld<8>(tmem_base + ((uint32_t)(q4 * 32) << 16) + (uint32_t)(nt * BM + j0 + jb), r);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const int row = j0 + jb + e;
                    if (row < p.m && okc) {
                        if (nparts == 1) out[(size_t)row * p.n + col] = H::from_float(__uint_as_float(r[e]) + bv);
                        else __stcg(part + (size_t)row * UM_COLS + cc, __uint_as_float(r[e]));
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_dempty);
            ++seg;
            if (nparts == 1) return;
            __threadfence();
            conv_sync();
            if (tid == 0) *reinterpret_cast<volatile int*>(s_last) = (atomicAdd(p.counters + tile, 1u) == unsigned(nparts - 1));
            conv_sync();
            if (ok && *reinterpret_cast<volatile int*>(s_last)) {
                __threadfence();
                if (okc) {
                    for (int row = j0; row < j0 + HALF && row < p.m; ++row) {
                        float sum = 0.f;
                        for (int c = cf; c <= cla; ++c) sum += __ldcg(p.partial + ((size_t)(c + tile) * BM + row) * UM_COLS + cc);
                        out[(size_t)row * p.n + col] = H::from_float(sum + bv);
                    }
                }
                if (tid == 0) p.counters[tile] = 0;
            }
            conv_sync();                                 // s_last is reused by the next shared tile
        };
        // epilogues of the run's column-tile segments that end before unit `limit`, oldest first
        int ep_i = 0, ep_tile = x0 / p.kbt;
        int ep_end = (ep_tile + 1) * p.kbt - 1 - x0;     // last unit of the oldest undrained segment
        if (ep_end > nrun - 1) ep_end = nrun - 1;
        auto drain_until = [&](int limit) {
            while (ep_i < nrun && ep_end < limit && ok) {
                epilogue(ep_tile);
                ep_i = ep_end + 1; ++ep_tile;
                ep_end += p.kbt;
                if (ep_end > nrun - 1) ep_end = nrun - 1;
            }
        };

        const int nrun_pad = (nrun + 1) & ~1;            // the second k-block of the last pair may not exist: its owners still arrive
        for (int i = grp; i < nrun_pad && ok; i += UM_GROUPS) {
            const int as = i % UM_ASTAGES; const uint32_t aph = (i / UM_ASTAGES) & 1;
            const int pr = as >> 1;
            if (i >= nrun) {
                if (!wait(bar_aempty(pr), aph ^ 1)) { ok = false; break; }
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_afull(pr));
                continue;
            }
#pragma unroll
            for (int nt = 0; nt < UM_NT; ++nt) { sr[nt] = sr_n[0][nt]; zr[nt] = zr_n[0][nt]; }
#pragma unroll
            for (int d = 0; d + 1 < SZ; ++d)
#pragma unroll
                for (int nt = 0; nt < UM_NT; ++nt) { sr_n[d][nt] = sr_n[d + 1][nt]; zr_n[d][nt] = zr_n[d + 1][nt]; }
            fetch(sr_n[SZ - 1], zr_n[SZ - 1]);
            const int ps = i % S::PSTAGES; const uint32_t pph = (i / S::PSTAGES) & 1;
            if (!wait(bar_pfull(ps), pph)) { ok = false; break; }
            const uint32_t* pk = reinterpret_cast<const uint32_t*>(smem + S::OFF_P + ps * S::P_BYTES) + cl;
            uint32_t wq[UM_NT][PROWS];
#pragma unroll
            for (int nt = 0; nt < UM_NT; ++nt)
#pragma unroll
                for (int r = 0; r < PROWS; ++r) wq[nt][r] = pk[r * UM_COLS + nt * 128];
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_pempty(ps));  // the stage is in registers: give it back to the producer
            bool waited = false;
#pragma unroll
            for (int nt = 0; nt < UM_NT; ++nt) {
                // ---- W = (q - (z+1)) * s for this column's 64 values of k ----
                uint32_t a[32];
                const uint32_t s16 = sr[nt] & 0xffffu;
                const uint32_t s2 = s16 | (s16 << 16);
                const int zp1 = p.qz ? int((zr[nt] >> ((cl % PACK) * BITS)) & ZMASK) + 1 : p.zp1_const;   // tiles start on multiples of PACK
                if constexpr (BITS == 4 && !H::kIsBf16) {
                    const uint32_t c_lo = H::pack(float(1024 + zp1), float(1024 + zp1));     // exact: integers <= 1040
                    const uint32_t c_hi = H::pack(-float(64 + zp1), -float(64 + zp1));
                    const uint32_t sixteenth = 0x2c002c00u;                                    // (1/16, 1/16)
#pragma unroll
                    for (int r = 0; r < PROWS; ++r) {
                        const uint32_t w = wq[nt][r], w8 = w >> 8;
                        a[4 * r + 0] = H::mul(H::sub(and_or(w, 0x000f000fu, 0x64006400u), c_lo), s2);            // (q0, q4)
                        a[4 * r + 1] = H::mul(H::fma(and_or(w, 0x00f000f0u, 0x64006400u), sixteenth, c_hi), s2); // (q1, q5): (1024 + 16 q) / 16 - 64 - zp1
                        a[4 * r + 2] = H::mul(H::sub(and_or(w8, 0x000f000fu, 0x64006400u), c_lo), s2);           // (q2, q6)
                        a[4 * r + 3] = H::mul(H::fma(and_or(w8, 0x00f000f0u, 0x64006400u), sixteenth, c_hi), s2); // (q3, q7)
                    }
                } else if constexpr (BITS == 4) {
                    const uint32_t c_lo = H::pack(float(128 + zp1), float(128 + zp1));        // exact in bf16: integers <= 144
#pragma unroll
                    for (int r = 0; r < PROWS; ++r)
#pragma unroll
                        for (int q = 0; q < 4; ++q)
                            a[4 * r + q] = H::mul(H::sub(and_or(wq[nt][r] >> (4 * q), 0x000f000fu, 0x43004300u), c_lo), s2);
                } else {
                    const uint32_t c_lo = H::pack(float(1024 + zp1), float(1024 + zp1));     // exact: integers <= 1280
#pragma unroll
                    for (int r = 0; r < PROWS; ++r) {
                        a[2 * r + 0] = H::mul(H::sub(prmt(wq[nt][r], 0x64646464u, 0x4140u), c_lo), s2);          // 1024 + (b0, b1)
                        a[2 * r + 1] = H::mul(H::sub(prmt(wq[nt][r], 0x64646464u, 0x4342u), c_lo), s2);          // 1024 + (b2, b3)
                    }
                }
                if (!waited) {
                    if (!wait(bar_aempty(pr), aph ^ 1)) { ok = false; break; }
                    tc_fence_after();
                    waited = true;
                }
                tc_st32(tmem_a + ((uint32_t)(q4 * 32) << 16) + (uint32_t)((as * UM_NT + nt) * 32), a);
            }
            if (!ok) break;
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_afull(pr));
            // Tiles that end before this group's next k-block (i + 4): the group has converted its share of them.  The
            // MMA thread starts a pair of k-blocks only when both are converted, and a pair may straddle two tiles: a
            // tile that ends on the even k-block just before an odd next k-block needs that k-block converted before
            // it can finish, so it is drained one turn later.
            drain_until((i & 1) ? i + UM_GROUPS - 1 : i + UM_GROUPS);
        }
        drain_until(nrun);
    }

    tc_fence_before();
    __syncthreads();
    if (warp == UM_W_MMA) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)S::TMEM_COLS) : "memory");
    }
    if (tid == 0 && abort_flag && p.err) atomicExch(p.err, 5u);
}

template <int BITS, typename T, int BM>
int launch_inst(cudaStream_t st, const CUtensorMap& mq, const UmParams& p, int grid) {
    using S = UmSmem<BITS, BM>;
    auto kern = qgemm_umma_kernel<BITS, T, BM>;
    static bool configured[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { cudaGetLastError(); return MT_ERR_CUDA; }
    if (!configured[dev]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL) != cudaSuccess) { cudaGetLastError(); return MT_ERR_CUDA; }
        configured[dev] = true;
    }
    kern<<<grid, UM_THREADS, S::TOTAL, st>>>(mq, p);
    return cudaGetLastError() == cudaSuccess ? MT_OK : MT_ERR_CUDA;
}

template <int BITS, typename T>
int launch_bm(cudaStream_t st, const CUtensorMap& mq, const UmParams& p, int grid, int bm) {
    if (bm == 16) return launch_inst<BITS, T, 16>(st, mq, p, grid);
    if (bm == 32) return launch_inst<BITS, T, 32>(st, mq, p, grid);
    return launch_inst<BITS, T, 64>(st, mq, p, grid);
}

int plan(const QGemmArgs& a, int m, int& grid, int& bm, size_t& need) {
    bm = m <= 16 ? 16 : m <= 32 ? 32 : 64;
    const int tiles = (a.n + UM_COLS - 1) / UM_COLS, kbt = a.k / 64;
    const long long units = (long long)tiles * kbt;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    long long g = units / 16;                           // at least 16 k-blocks per CTA: partial tiles stay a small share of the traffic
    if (g < 1) g = 1;
    if (g > sms) g = sms;
    if (g > units) g = units;
    grid = (int)g;
    need = (size_t)(grid + tiles) * bm * UM_COLS * 4;
    return tiles;
}

}  // namespace

bool umma_supported(const QGemmArgs& a) {
    if (a.g_idx != nullptr || a.m < 1 || a.groups < 1 || a.k % a.groups != 0) return false;
    if (a.bits == 8 && a.dtype == MT_BF16) return false;          // 128 + b is not exact in bf16 for b >= 128
    const int gs = a.k / a.groups;
    if (gs % 64 != 0 || a.k % 64 != 0 || a.n % 8 != 0) return false;
    if ((a.n + UM_COLS - 1) / UM_COLS >= kMaxTiles - 1) return false;
    if ((long long)((a.n + UM_COLS - 1) / UM_COLS) * (a.k / 64) > (1LL << 30)) return false;
    if (a.workspace == nullptr || a.workspace_bytes < kCounterBytes) return false;
    if (!get_tensor_map_encoder()) return false;
    int grid, bm; size_t need;
    plan(a, a.m < 64 ? a.m : 64, grid, bm, need);
    return need <= a.workspace_bytes - kCounterBytes;
}

size_t umma_workspace_bytes(int m, int n, int k) {
    QGemmArgs a = {};
    a.n = n; a.k = k;
    int grid, bm; size_t need;
    plan(a, m < 64 ? m : 64, grid, bm, need);
    return need;
}

int launch_umma(cudaStream_t st, const QGemmArgs& a) {
    if (!umma_supported(a)) return MT_ERR_UNSUPPORTED;
    CUtensorMap mq;
    {
        const int pack = 32 / a.bits;
        cuuint64_t dims[2] = {(cuuint64_t)a.n, (cuuint64_t)(a.k / pack)};
        cuuint64_t strides[1] = {(cuuint64_t)a.n * 4};
        cuuint32_t box[2] = {(cuuint32_t)UM_COLS, (cuuint32_t)(64 / pack)};
        cuuint32_t es[2] = {1, 1};
        if (get_tensor_map_encoder()(&mq, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<uint32_t*>(a.qweight), dims, strides, box, es,
                                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return MT_ERR_CUDA;
    }
    for (int r0 = 0; r0 < a.m; r0 += 64) {
        const int m = a.m - r0 < 64 ? a.m - r0 : 64;
        int grid, bm; size_t need;
        const int tiles = plan(a, m, grid, bm, need);
        UmParams p;
        p.x = static_cast<const char*>(a.x) + (size_t)r0 * a.k * 2;
        p.out = static_cast<char*>(a.out) + (size_t)r0 * a.n * 2;
        p.qw = a.qweight; p.qz = a.qzeros; p.scales = a.scales; p.bias = a.bias;
        p.counters = static_cast<unsigned*>(a.workspace);
        p.err = p.counters + (kMaxTiles - 1);
        p.partial = reinterpret_cast<float*>(static_cast<char*>(a.workspace) + kCounterBytes);
        p.m = m; p.n = a.n; p.k = a.k; p.groups = a.groups; p.gs = a.k / a.groups;
        p.tiles = tiles; p.kbt = a.k / 64; p.units = tiles * p.kbt;
        p.per = p.units / grid; p.rem = p.units % grid;
        p.zp1_const = 1 << (a.bits - 1);
        int rc;
        if (a.bits == 4) rc = a.dtype == MT_F16 ? launch_bm<4, __half>(st, mq, p, grid, bm) : launch_bm<4, __nv_bfloat16>(st, mq, p, grid, bm);
        else rc = launch_bm<8, __half>(st, mq, p, grid, bm);
        if (rc != MT_OK) return rc;
    }
    return MT_OK;
}

}  // namespace mt
