// Mid-size batches (2 < M <= 64 per pass) for GPTQ weights with contiguous groups of a multiple of 128:
// the packed integers go to the tensor core AS INTEGERS.
//
// Replaces the per-thread dequantize-and-multiply loop of examples/qwen1_5_int8.py:156-200 (and the
// dequantize-then-matmul of minit/quantize/dispatch.py:8-20) for the batch sizes where the product is
// still a stream of the packed weights.  Turning every weight into fp16 costs more issue slots than the
// stream leaves at 6.5 TB/s, so this kernel does not dequantize at all:
//
//   * tcgen05.mma.kind::i8 multiplies unsigned 8-bit by signed 8-bit with exact 32-bit sums.  A packed
//     nibble masked in place IS the unsigned byte q (word & 0x0f0f0f0f: the even nibbles of a word,
//     (word >> 4) & 0x0f0f0f0f: the odd ones): three integer instructions per eight weights, written
//     straight to tensor memory (tcgen05.st) as the A operand (M = 128 output columns per tile).  An
//     8-bit weight needs no instruction at all.
//   * the activations are split once per call by a small pre-pass (xprep_kernel): per row and per 128
//     values of k a power-of-two block scale 2^e brings the largest |x| into [2^13, 2^14), x' = rint(x 2^e)
//     is written as two signed bytes x' = 256 h + l, and sum(x') and 2^-e are kept.  The B operand of a
//     128-k block is the 2 BM x 128 byte tile [h rows | l rows], stored by the pre-pass in the
//     shared-memory image the tensor core reads (K-major, 128-byte swizzle, k-slots in the order the
//     nibble masks produce), so the main kernel fetches it with one bulk copy.
//   * per 128 values of k the integer sums V = 256 D_h + D_l = sum_k q x' leave tensor memory
//     (tcgen05.ld) and are folded in fp32 with the scale and zero point of that block's group:
//         out[m, n] += s[g, n] * 2^-e[m] * (V - (z[g, n] + 1) * sum_k x')
//     which is the GPTQ formula (q - (z + 1)) * s applied to x' 2^-e.  The only approximation is the
//     14-bit block-fixed-point x' (relative output error ~1e-4 of rms, far inside the 1e-2 bound).
//
// Roles (19 warps, one CTA per SM): two groups of 4 converter warps (a thread = one column of each 128-column tile: reads
// the packed words from the stage, masks, one tcgen05.st per tile); 8 fold warps = (tile, TMEM lane quarter)
// or (TMEM lane quarter, half of the batch rows): a thread owns one output column and folds the k-block the tensor core finished
// while it works on the next one (two accumulator buffers), scale and zero word read straight from global
// memory one k-block ahead; two producer warps of one lane each (TMA of the packed rows of a k-block, 16 KB per
// stage, 8 stages | one bulk copy of the B tile per k-block, scales and zero words in blocks of eight groups); one MMA
// lane per tile.  Stream-K over (column tile, k-block) units as in the other
// kernels; a tile shared by several CTAs is finished, slice by slice, by the last warp to arrive.
// Every wait is bounded and reports through the workspace error word.
#include "tma.cuh"
#include "tcgen05.cuh"

namespace mt {
namespace {

constexpr int MD_FOLD = 8;                         // fold warps: 0 .. MD_FOLD - 1
constexpr int MD_DBUF16 = 4;                       // accumulator buffers of the 16-row tile
constexpr int MD_ROWS_PER_LD = 8;                  // batch rows per tcgen05.ld in the fold
constexpr int MD_FAST_NS = 20;                     // sleep between polls of a barrier on the critical path
constexpr int MD_SLOW_NS = 400;                    // ... of a barrier that a role running ahead waits on
constexpr int MD_CGROUPS = 2;                      // converter groups of four warps, alternating k-blocks
constexpr int MD_W_CONV = MD_FOLD;                                  // the converter warps follow the fold warps
constexpr int MD_W_PROD = MD_FOLD + 4 * MD_CGROUPS;                 // two producer warps, one lane each: packed rows | activation tiles, scales and zero words
constexpr int MD_W_MMA = MD_W_PROD + 2;                             // two MMA warps (column tile 0 and 1)
constexpr int MD_THREADS = (MD_W_MMA + 2) * 32;
constexpr int MD_SZG = 8;                                           // scale groups per scale / zero block
constexpr int MD_SZST = 3;                                          // blocks in the ring
constexpr int MD_KB = 128;                         // values of k per unit

template <int BITS, int BM> struct MdCfg {
    static constexpr int PACK = 32 / BITS;
    static constexpr int PROWS = MD_KB / PACK;     // packed rows per k-block: 16 | 32
    static constexpr int NT = BM <= 32 ? 2 : 1;    // 128-column tiles per CTA tile
    static constexpr int COLS = NT * 128;
    static constexpr int RS = MD_FOLD / (4 * NT);  // fold warps that share a (tile, lane quarter) split the batch rows: 1 | 2
    static constexpr int RW = BM / RS;             // batch rows a fold warp handles: 16 | 32
    static constexpr int RC = MD_ROWS_PER_LD;      // rows per tcgen05.ld and per stage of the fold arithmetic
    static constexpr int NB = 2 * BM;              // MMA N: h rows then l rows
    static constexpr int DBUF = BM == 16 ? MD_DBUF16 : 2;   // accumulator buffers: the MMAs of a k-block wait for the fold of DBUF k-blocks earlier
    static constexpr int D_COLS = DBUF * NT * NB;
    static constexpr int A_STAGE = NT * 32;        // TMEM columns of one k-block of the A operand
    static constexpr int AST = BM == 64 ? 4 : (512 - D_COLS) / A_STAGE;   // slots of the A operand in tensor memory: 6 | 4 | 4
    static constexpr int W_BYTES = PROWS * COLS * 4;
    static constexpr int P_STAGE = W_BYTES;
    static constexpr int PST = ((BM == 64 ? 96 : 128) * 1024) / P_STAGE / 2 * 2;   // packed weights in flight per SM
    static constexpr int B_TILE = NB * 128;
    static constexpr int B_COPY = B_TILE + BM * 8;                    // tile + sum(x') [BM] int32 + 2^-e [BM] fp32
    static constexpr int B_STAGE = B_TILE + 1024;                     // the sums and block scales behind the tile
    static constexpr int S_BYTES = MD_SZG * COLS * 2;                 // scales of MD_SZG groups, this CTA tile's columns
    static constexpr int Z_BYTES = MD_SZG * (COLS / PACK) * 4;        // zero words of the same groups
    static constexpr int SZ_STAGE = S_BYTES + Z_BYTES;
    // An activation stage is busy from the request of its copies (three asynchronous copies issued by one lane: ~2500
    // cycles) to the end of the fold of its k-block, about four k-block periods: the ring is deeper than the A ring
    static constexpr int BST = BM == 64 ? 6 : 8;
    static constexpr int OFF_P = 0;
    static constexpr int OFF_B = OFF_P + PST * P_STAGE;
    static constexpr int OFF_SZ = OFF_B + BST * B_STAGE;
    static constexpr int OFF_BAR = OFF_SZ + MD_SZST * SZ_STAGE;
    static constexpr int NBARS = 2 * PST + 3 * BST + 2 * MD_SZST;
    static constexpr int TOTAL = OFF_BAR + NBARS * 8 + 64 + 1024;
    static_assert(BM * 8 <= 1024 && OFF_SZ % 128 == 0 && S_BYTES % 128 == 0, "activation stage and scale block layout");
    // A wait by phase parity is only right for a thread that has seen every earlier phase of that barrier: every
    // producer is ONE thread that walks its ring in order, and the two converter groups see every other phase of
    // barriers whose ring length is even.
    static_assert(PST >= 2 && BST % 2 == 0 && PST % 2 == 0, "ring lengths against the groups that wait on them");
    static_assert(D_COLS + AST * A_STAGE <= 512 && AST >= 3 && DBUF < BST, "TMEM budget");
    static_assert(OFF_B % 1024 == 0, "B tiles need 1024-byte alignment");
    static_assert(TOTAL <= 227 * 1024, "shared memory budget");
};

struct MdParams {
    const unsigned char* xl;      // pre-pass output: per k-block [B tile | sum(x') | 2^-e]
    const void* scales; const uint32_t* qz;   // [G, N] T; [G, N / pack] or null (symmetric midpoint)
    const void* bias; void* out;
    float* partial; unsigned* counters; unsigned* err;
    int m, n, k;
    int tiles, kbt;               // column tiles, k-blocks per tile
    int kpg;                      // k-blocks per scale group
    int units, per, rem;
    int zp1_const;
    int pdl;
    ArParams ar;                  // row-parallel use: all-reduce of the finished sums over peer memory
    const void* residual;         // [M,N] T or null: added to the finished (all-reduced) sum before the one rounding
};

// Bounded wait with an explicit poll rate.  Every poll of an mbarrier is an instruction for the unit that serves all of
// them and an issue slot taken from the warps that do arithmetic, so a role that runs ahead of the pipeline (producers,
// converters) sleeps long between polls and only the roles on the critical path (MMA lanes, fold warps) poll closely.
// Gives up after about a second and raises the CTA's abort flag.
template <int SLEEP_NS>
__device__ __forceinline__ bool md_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    constexpr int LIMIT = 1000000000 / (SLEEP_NS + 50);
    for (int i = 0; i < LIMIT; ++i) {
        uint32_t ok;
        asm volatile("{\n.reg .pred p;\nmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.b32 %0, 1, 0, p;\n}"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        if ((i & 255) == 255 && *abort_flag) return false;
        __nanosleep(SLEEP_NS);
    }
    *abort_flag = 1;
    return false;
}

// The peers' values of one column for the RW rows a fold thread holds, added to v[] (this rank's partials) in rank order.
// Kept out of line, working on an array in local memory: inlined, its address registers and loaded cells pushed the
// kernel's accumulators out of registers.
template <int RW>
__device__ __noinline__ void md_pull_all(ArParams ar, unsigned epoch, size_t cell0, size_t stride, int nrows, float* v) {
    for (int r = 0; r < RW && r < nrows; r += 8) {
        float v8[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v8[j] = v[r + j];
        ar_pull_rows<8>(ar, epoch, cell0 + (size_t)r * stride, stride, min(8, nrows - r), v8);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[r + j] = v8[j];
    }
}

__device__ __forceinline__ void md_mma_i8(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
                 "tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, p;\n}"
                 ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void md_bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
template <int NR>
__device__ __forceinline__ void md_st(uint32_t taddr, const uint32_t (&r)[NR]) {
    static_assert(NR == 8 || NR == 16, "tcgen05.st width");
    if constexpr (NR == 8) {
        asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                     ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]) : "memory");
    } else {
        asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                     ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                       "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
    }
}

// ----------------------------------------------------------------------------------------------
// pre-pass: activations -> two-limb block-fixed-point B tiles (one block per k-block of 128 values)
// ----------------------------------------------------------------------------------------------
// grid = K / 128 blocks of 256 threads; warp w handles batch rows w, w + 8, ...; lane = 4 consecutive k.
template <typename T, int BITS>
__global__ void __launch_bounds__(256) xprep_kernel(const T* __restrict__ x, unsigned char* __restrict__ xl, int m, int k, int bm, int pdl) {
    using H = F16x2<T>;
    const int kb = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nb = 2 * bm;
    unsigned char* tile = xl + (size_t)kb * (nb * 128 + bm * 8);
    int* sums = reinterpret_cast<int*>(tile + nb * 128);
    float* pes = reinterpret_cast<float*>(tile + nb * 128 + bm * 4);
    if (pdl) { griddep_launch_dependents(); griddep_wait(); }
    for (int r = warp; r < bm; r += 8) {
        float f[4] = {0.f, 0.f, 0.f, 0.f};
        if (r < m) {
            const uint2 raw = __ldg(reinterpret_cast<const uint2*>(x + (size_t)r * k + (size_t)kb * MD_KB) + lane);
            f[0] = H::to_float(uint16_t(raw.x & 0xffff)); f[1] = H::to_float(uint16_t(raw.x >> 16));
            f[2] = H::to_float(uint16_t(raw.y & 0xffff)); f[3] = H::to_float(uint16_t(raw.y >> 16));
        }
        float amax = fmaxf(fmaxf(fabsf(f[0]), fabsf(f[1])), fmaxf(fabsf(f[2]), fabsf(f[3])));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        int e = 0;                                           // x' = x * 2^e has its block maximum in [2^13, 2^14)
        if (amax > 0.f && amax < 3.0e38f) e = 13 - (int((__float_as_uint(amax) >> 23) & 0xff) - 127);
        e = e < -100 ? -100 : (e > 100 ? 100 : e);
        const float up = __uint_as_float(uint32_t(127 + e) << 23);
        int xi[4], sum = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float v = fminf(fmaxf(f[j] * up, -16384.f), 16384.f);   // NaN -> -16384: garbage in, bounded garbage out
            xi[j] = __float2int_rn(v);
            sum += xi[j];
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        int lo[4], hi[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) { lo[j] = ((xi[j] + 128) & 255) - 128; hi[j] = (xi[j] - lo[j]) >> 8; }
        const int rh = r, rl = bm + r;                        // tile rows of the two limbs
        auto row_base = [&](int R) { return tile + (R >> 3) * 1024 + (R & 7) * 128; };
        auto slot_addr = [&](unsigned char* base, int R, int p) { return base + ((((p >> 4) ^ (R & 7)) << 4) | (p & 15)); };
        if constexpr (BITS == 4) {
            // k = 4 lane + j sits in word rw = lane / 2 at nibble i = (lane % 2) * 4 + j; slot = 8 rw + i / 2 (+ 4 for odd i)
            const int rw = lane >> 1, i0 = (lane & 1) * 4;
            const int pe_ = 8 * rw + i0 / 2, po = pe_ + 4;
            *reinterpret_cast<uint16_t*>(slot_addr(row_base(rh), rh, pe_)) = uint16_t((hi[0] & 255) | ((hi[2] & 255) << 8));
            *reinterpret_cast<uint16_t*>(slot_addr(row_base(rh), rh, po)) = uint16_t((hi[1] & 255) | ((hi[3] & 255) << 8));
            *reinterpret_cast<uint16_t*>(slot_addr(row_base(rl), rl, pe_)) = uint16_t((lo[0] & 255) | ((lo[2] & 255) << 8));
            *reinterpret_cast<uint16_t*>(slot_addr(row_base(rl), rl, po)) = uint16_t((lo[1] & 255) | ((lo[3] & 255) << 8));
        } else {
            const int p = 4 * lane;                           // bytes of a word are consecutive k: slot = k
            *reinterpret_cast<uint32_t*>(slot_addr(row_base(rh), rh, p)) =
                uint32_t(hi[0] & 255) | (uint32_t(hi[1] & 255) << 8) | (uint32_t(hi[2] & 255) << 16) | (uint32_t(hi[3] & 255) << 24);
            *reinterpret_cast<uint32_t*>(slot_addr(row_base(rl), rl, p)) =
                uint32_t(lo[0] & 255) | (uint32_t(lo[1] & 255) << 8) | (uint32_t(lo[2] & 255) << 16) | (uint32_t(lo[3] & 255) << 24);
        }
        if (lane == 0) {
            sums[r] = sum;
            pes[r] = r < m ? __uint_as_float(uint32_t(127 - e) << 23) : 0.f;
        }
    }
}

// ----------------------------------------------------------------------------------------------
// main kernel
// ----------------------------------------------------------------------------------------------
// Barriers.  Every mbarrier operation costs its thread 200-350 cycles even when the phase is long complete, so the
// protocol is built to give the busiest roles ONE wait per k-block:
//   pfull[PST] / pempty[PST]   packed rows in the stage (copy engine)            / read by the converter group (4 warps)
//   full[BST]                  everything the MMAs of a k-block need: the A operand in tensor memory (4 converter warps),
//                              the activation tile with its scales / zero words (copy engine, one arrival of a producer
//                              lane) and a free accumulator buffer (the MD_FOLD fold warps, two k-blocks earlier)
//   done[BST]                  the MMAs of a k-block have completed (one commit per MMA lane): frees the A slot for the
//                              converters and hands the accumulators to the fold warps
//   bempty[BST]                the fold warps are done with the activation stage (sum(x'), 2^-e, scales, zero words)
// AR = false is the instantiation a single rank runs: the exchange code of the epilogue is compiled out of it (with that
// code present, unused, the same kernel took 19.7 instead of 18.0 ms per step on the 32-row batch of the 70B layers).
template <int BITS, typename T, int BM, bool AR>
__global__ void __launch_bounds__(MD_THREADS, 1) qgemm_mid_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_s,
                                                                  const __grid_constant__ CUtensorMap tmap_z, const MdParams p) {
    using C = MdCfg<BITS, BM>;
    using H = F16x2<T>;

    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bar0 = sbase + C::OFF_BAR;
    auto bar_pfull = [&](int s) { return bar0 + 8u * s; };
    auto bar_pempty = [&](int s) { return bar0 + 8u * (C::PST + s); };
    auto bar_full = [&](int s) { return bar0 + 8u * (2 * C::PST + s); };
    auto bar_done = [&](int s) { return bar0 + 8u * (2 * C::PST + C::BST + s); };
    auto bar_bempty = [&](int s) { return bar0 + 8u * (2 * C::PST + 2 * C::BST + s); };
    auto bar_szfull = [&](int s) { return bar0 + 8u * (2 * C::PST + 3 * C::BST + s); };
    auto bar_szempty = [&](int s) { return bar0 + 8u * (2 * C::PST + 3 * C::BST + MD_SZST + s); };
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + C::OFF_BAR + C::NBARS * 8);
    __shared__ int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int cta = blockIdx.x;
    const int x0 = cta * p.per + (cta < p.rem ? cta : p.rem);
    const int nrun = p.per + (cta < p.rem ? 1 : 0);

    if (tid == 0) {
        abort_flag = 0;
        for (int s = 0; s < C::PST; ++s) { mbar_init(bar_pfull(s), 1); mbar_init(bar_pempty(s), 4); }
        for (int s = 0; s < C::BST; ++s) { mbar_init(bar_full(s), 4 + 1 + MD_FOLD); mbar_init(bar_done(s), C::NT); mbar_init(bar_bempty(s), MD_FOLD); }
        for (int s = 0; s < MD_SZST; ++s) { mbar_init(bar_szfull(s), 1); mbar_init(bar_szempty(s), MD_FOLD); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        // the first DBUF k-blocks find their accumulator buffers free: stand in for the fold warps' arrivals
        for (int s = 0; s < C::DBUF; ++s)
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0], %1;" ::"r"(bar_full(s)), "r"((uint32_t)MD_FOLD) : "memory");
    }
    if (warp == MD_W_MMA) tc_alloc<512>(smem_u32(tmem_slot));
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_a = tmem_base + C::D_COLS;
    auto wait = [&](uint32_t bar, uint32_t parity) { return md_wait<MD_FAST_NS>(bar, parity, &abort_flag); };        // critical path
    auto lazy_wait = [&](uint32_t bar, uint32_t parity) { return md_wait<MD_SLOW_NS>(bar, parity, &abort_flag); };   // roles that run ahead

    // first / last CTA with a unit of column tile t
    auto owner = [&](int u) -> int {
        const int big = p.rem * (p.per + 1);
        return u < big ? u / (p.per + 1) : p.rem + (u - big) / p.per;
    };

    if (warp >= MD_W_PROD && warp < MD_W_MMA) {
        // ------------------------------ producers: two warps, one lane each ------------------------------
        // A thread completes only about four asynchronous copies per microsecond (each wait / expect / issue step is a
        // long-latency instruction and they depend on one another), and several lanes of ONE warp in such loops fall
        // into step with the slowest.  So: one thread for the packed rows (one copy per k-block) and one for the activation
        // tiles (one copy per k-block) plus the scales and zero words (two copies per MD_SZG scale groups).
        const int role = warp - MD_W_PROD;
        if (lane == 0 && role == 0) {
            // The packed weights do not depend on the previous kernel in the stream: the first ring of stages is requested
            // at once; every later stage waits for the converters to have read its previous content.
            int t = x0 / p.kbt, b = x0 - t * p.kbt;
            for (int i = 0; i < nrun; ++i) {
                const int ps = i % C::PST;
                if (i >= C::PST && !lazy_wait(bar_pempty(ps), ((i / C::PST) & 1) ^ 1)) break;
                mbar_expect_tx(bar_pfull(ps), (uint32_t)C::W_BYTES);
                tma_load_2d(sbase + C::OFF_P + ps * C::P_STAGE, &tmap_q, t * C::COLS, b * C::PROWS, bar_pfull(ps));
                if (++b == p.kbt) { b = 0; ++t; }
            }
        } else if (lane == 0 && role == 1) {
            if (p.pdl) { griddep_launch_dependents(); griddep_wait(); }   // the activation tiles are written by the pre-pass
            // one scale / zero block = the scales and zero words of MD_SZG consecutive groups of a column tile; a new block
            // starts with the run, with every column tile and every MD_SZG groups
            const uint32_t stx = (uint32_t)(C::S_BYTES + (p.qz ? C::Z_BYTES : 0));
            int t = x0 / p.kbt, kb = x0 - t * p.kbt, nblk = 0, cur = -1;
            for (int i = 0; i < nrun; ++i) {
                const int gb = (kb / p.kpg) / MD_SZG;
                if (gb != cur) {
                    cur = gb;
                    const int ss = nblk % MD_SZST;
                    if (nblk >= MD_SZST && !lazy_wait(bar_szempty(ss), ((nblk / MD_SZST) & 1) ^ 1)) break;
                    const uint32_t dst = sbase + C::OFF_SZ + ss * C::SZ_STAGE;
                    mbar_expect_tx(bar_szfull(ss), stx);
                    tma_load_2d(dst, &tmap_s, t * C::COLS, gb * MD_SZG, bar_szfull(ss));
                    if (p.qz) tma_load_2d(dst + C::S_BYTES, &tmap_z, t * C::COLS / C::PACK, gb * MD_SZG, bar_szfull(ss));
                    ++nblk;
                }
                const int bs = i % C::BST;
                if (i >= C::BST && !lazy_wait(bar_bempty(bs), ((i / C::BST) & 1) ^ 1)) break;
                mbar_expect_tx(bar_full(bs), (uint32_t)C::B_COPY);
                md_bulk_load(sbase + C::OFF_B + bs * C::B_STAGE, p.xl + (size_t)kb * C::B_COPY, (uint32_t)C::B_COPY, bar_full(bs));
                if (++kb == p.kbt) { kb = 0; ++t; cur = -1; }
            }
        }
    } else if (warp >= MD_W_MMA) {
        // ------------------------------ MMA issuers: one lane per column tile ------------------------------
        const int nt = warp - MD_W_MMA;
        if (lane == 0 && nt < C::NT) {
            // kind::i8: D s32 (2 << 4), A unsigned 8-bit (0 << 7), B signed 8-bit (1 << 10), K-major both, N = 2 BM, M = 128
            const uint32_t idesc = (2u << 4) | (1u << 10) | ((uint32_t)(C::NB >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
            uint32_t early_ok = 0u;
            for (int i = 0; i < nrun; ++i) {
                const int as = i % C::AST, bs = i % C::BST, db = i % C::DBUF;
                if (!early_ok && !wait(bar_full(bs), (i / C::BST) & 1)) break;
                tc_fence_after();
                const uint64_t bdesc = tc_desc_sw128(sbase + C::OFF_B + bs * C::B_STAGE);
                const uint32_t d = tmem_base + (uint32_t)((db * C::NT + nt) * C::NB), a = tmem_a + (uint32_t)((as * C::NT + nt) * 32);
#pragma unroll
                for (int k4 = 0; k4 < 4; ++k4) md_mma_i8(d, a + (uint32_t)(k4 * 8), bdesc + (uint64_t)(k4 * 2), idesc, k4 ? 1u : 0u);
                tc_commit(bar_done(bs));
                // ask about the next k-block now: the answer takes ~200 cycles either way and is read at the top of the next turn
                early_ok = 0u;
                if (i + 1 < nrun) {
                    const int in = i + 1;
                    asm volatile("{\n.reg .pred p;\nmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.b32 %0, 1, 0, p;\n}"
                                 : "=r"(early_ok) : "r"(bar_full(in % C::BST)), "r"((uint32_t)((in / C::BST) & 1)) : "memory");
                }
            }
        }
    } else if (warp >= MD_W_CONV) {
        // ------------------------------ converters: two groups of four warps, a thread = one column of every tile ------------------------------
        // Few, fat warps: what a warp pays per k-block for waits, barrier traffic and addresses is paid four times per
        // k-block.  Group g takes the k-blocks i = g, g + 2, ...  A thread reads the PROWS packed words of its column from
        // the stage, masks the nibbles into bytes and stores the 128 bytes of its TMEM lane with one tcgen05.st per tile.
        const int q4 = warp & 3;
        const int grp = (warp - MD_W_CONV) >> 2;
        const uint32_t lane_base = (uint32_t)(q4 * 32) << 16;
        const int cq = q4 * 32 + lane;                          // column inside a 128-column tile
        for (int i = grp; i < nrun; i += MD_CGROUPS) {
            const int ps = i % C::PST, as = i % C::AST, bs = i % C::BST;
            if (!lazy_wait(bar_pfull(ps), (i / C::PST) & 1)) break;
            const uint32_t* pk = reinterpret_cast<const uint32_t*>(smem + C::OFF_P + ps * C::P_STAGE) + cq;
            bool ok = true;
#pragma unroll
            for (int nt = 0; nt < C::NT; ++nt) {
                uint32_t a[32];
                if constexpr (BITS == 4) {
#pragma unroll
                    for (int r = 0; r < 16; ++r) {
                        const uint32_t w = pk[r * C::COLS + nt * 128];
                        a[2 * r] = w & 0x0f0f0f0fu;              // nibbles 0, 2, 4, 6 as bytes
                        a[2 * r + 1] = (w >> 4) & 0x0f0f0f0fu;   // nibbles 1, 3, 5, 7
                    }
                } else {
#pragma unroll
                    for (int r = 0; r < 32; ++r) a[r] = pk[r * C::COLS + nt * 128];
                }
                if (nt == C::NT - 1) {
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_pempty(ps));   // the stage is in registers
                }
                if (nt == 0) {
                    // the A slot is free when the MMAs of the k-block that used it last (AST k-blocks ago) have completed
                    if (i >= C::AST && !lazy_wait(bar_done((i - C::AST) % C::BST), ((i - C::AST) / C::BST) & 1)) { ok = false; break; }
                    tc_fence_after();
                }
                tc_st32(tmem_a + lane_base + (uint32_t)((as * C::NT + nt) * 32), a);
            }
            if (!ok) break;
            tc_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_full(bs));
        }
    } else {
        // ------------------------------ fold warps ------------------------------
        const int q4 = warp & 3;                              // TMEM lane quarter (= warp % 4)
        const int jj = warp >> 2;
        const int nt = C::NT == 2 ? (jj & 1) : 0;
        const int rs = C::NT == 2 ? (jj >> 1) : jj;           // which share of the batch rows
        const int cl = nt * 128 + q4 * 32 + lane;             // column inside the CTA tile
        const uint32_t lane_base = (uint32_t)(q4 * 32) << 16;
        const int r0 = rs * C::RW;
        constexpr uint32_t ZMASK = (1u << BITS) - 1u;
        const int zsh = (cl % C::PACK) * BITS;
        const T* __restrict__ bias = reinterpret_cast<const T*>(p.bias);
        uint16_t* __restrict__ out = reinterpret_cast<uint16_t*>(p.out);
        const uint16_t* __restrict__ resid = reinterpret_cast<const uint16_t*>(p.residual);
        const bool fused_ar = AR && ar_active(p.ar);
        unsigned epoch = 0u;
        bool epoch_read = false;

        float acc[C::RW];
#pragma unroll
        for (int r = 0; r < C::RW; ++r) acc[r] = 0.f;

        // the finished part of column tile `tile`: stored, or left as an fp32 partial slice that the last warp to arrive sums
        auto flush = [&](int tile) {
            const int col = tile * C::COLS + cl;
            const bool okc = col < p.n;
            const int cf = owner(tile * p.kbt), cla = owner(tile * p.kbt + p.kbt - 1);
            const int nparts = cla - cf + 1;
            bool write = true;
            if (nparts > 1) {
                float* part = p.partial + (size_t)(cta + tile) * BM * C::COLS;
#pragma unroll
                for (int r = 0; r < C::RW; ++r) __stcg(part + (size_t)(r0 + r) * C::COLS + cl, acc[r]);
                __threadfence();
                __syncwarp();
                const int cidx = tile * MD_FOLD + warp;        // one 16-bit counter per (tile, fold warp), two per word
                const int sh = (cidx & 1) * 16;
                unsigned old = 0;
                if (lane == 0) old = (atomicAdd(p.counters + (cidx >> 1), 1u << sh) >> sh) & 0xffffu;
                old = __shfl_sync(0xffffffffu, old, 0);
                write = old == unsigned(nparts - 1);
                if (write) {
                    __threadfence();
#pragma unroll
                    for (int r = 0; r < C::RW; ++r) acc[r] = 0.f;
                    for (int c = cf; c <= cla; ++c) {           // CTA order: the same sum whoever arrives last
                        const float* src = p.partial + (size_t)(c + tile) * BM * C::COLS + (size_t)r0 * C::COLS + cl;
#pragma unroll
                        for (int r = 0; r < C::RW; ++r) acc[r] += __ldcg(src + (size_t)r * C::COLS);
                    }
                    if (lane == 0) atomicSub(p.counters + (cidx >> 1), unsigned(nparts) << sh);
                }
            }
            if (write && okc) {
                const float bv = bias ? H::to_float(reinterpret_cast<const uint16_t*>(bias)[col]) : 0.f;
                if (fused_ar && !epoch_read) { epoch = ar_epoch(p.ar); epoch_read = true; }
                float bvf = bv;
                float xch[C::RW];                                // handed to md_pull_all by address: lives in local memory, acc stays in registers
                const bool two_shot = fused_ar && p.ar.two_shot;
                const int owner = two_shot ? ar_owner(p.ar, col) : 0;
                if (two_shot && owner == p.ar.rank) {
                    // this rank adds the column: wait for every rank's partial, add in rank order, send the sums to everyone
#pragma unroll
                    for (int r = 0; r < C::RW; ++r) xch[r] = acc[r] + bv;
                    md_pull_all<C::RW>(p.ar, epoch, (size_t)r0 * p.n + col, (size_t)p.n, p.m - r0, xch);
#pragma unroll
                    for (int r = 0; r < C::RW; ++r) acc[r] = xch[r];
#pragma unroll
                    for (int r = 0; r < C::RW; ++r)
                        if (r0 + r < p.m) ar_push1(p.ar, epoch, (size_t)(r0 + r) * p.n + col, acc[r]);
                    bvf = 0.f;                                   // the sums hold every rank's bias already
                } else if (two_shot) {
#pragma unroll
                    for (int r = 0; r < C::RW; ++r)
                        if (r0 + r < p.m) ar_push_to(p.ar, epoch, owner, (size_t)(r0 + r) * p.n + col, acc[r] + bv);
                } else if (fused_ar) {
#pragma unroll
                    for (int r = 0; r < C::RW; ++r)
                        if (r0 + r < p.m) ar_push1(p.ar, epoch, (size_t)(r0 + r) * p.n + col, acc[r] + bv);
                }
                if (fused_ar && !two_shot) {
                    // collect the peers' values eight rows at a time (one trip to memory per peer and group, not per value)
#pragma unroll
                    for (int r = 0; r < C::RW; ++r) xch[r] = acc[r] + bv;
                    md_pull_all<C::RW>(p.ar, epoch, (size_t)r0 * p.n + col, (size_t)p.n, p.m - r0, xch);
#pragma unroll
                    for (int r = 0; r < C::RW; ++r) acc[r] = xch[r];
                    bvf = 0.f;                                   // the sums hold every rank's bias already
                }
#pragma unroll
                for (int r = 0; r < C::RW; ++r) {
                    const int row = r0 + r;
                    if (row < p.m) {
                        float v = acc[r] + bvf;
                        if (two_shot && owner != p.ar.rank) v = ar_read_from(p.ar, epoch, owner, (size_t)row * p.n + col);
                        if (resid) v += H::to_float(resid[(size_t)row * p.n + col]);
                        out[(size_t)row * p.n + col] = H::from_float(v);
                    }
                }
            }
#pragma unroll
            for (int r = 0; r < C::RW; ++r) acc[r] = 0.f;
        };

        int tile = x0 / p.kbt, kb = x0 - tile * p.kbt;
        if (p.pdl) griddep_wait();                              // before anything an earlier kernel wrote is touched (out / partial)
        // one column tile's share of the run at a time: the store / partial-sum code sits between the tiles, outside the
        // loop over k-blocks, which stays small enough for the instruction cache next to the other roles' loops
        bool live = true;
        uint32_t early_ok = 0u;
        int sz_cur = -1, sz_n = 0;                                // scale / zero block in use (group block index) and blocks seen
        const unsigned char* sz_stage = smem;
        for (int j = 0; j < nrun && live;) {
            const int seg_end = (nrun - j < p.kbt - kb) ? nrun : j + (p.kbt - kb);
            int g0 = kb / p.kpg;                                   // once per column tile
            int kin = kb - g0 * p.kpg, gb = g0 / MD_SZG, gi = g0 - gb * MD_SZG;
        for (; j < seg_end; ++j) {
            const int bs = j % C::BST, db = j % C::DBUF;
            // The MMAs of this k-block have completed.  Their issuing lanes waited for the copy engine's bytes of this stage
            // (`full`) before they issued, so the stage's sums, scales and zero words are in shared memory long since.
            if (!early_ok && !wait(bar_done(bs), (j / C::BST) & 1)) { live = false; break; }
            tc_fence_after();
            const uint32_t dbase = tmem_base + lane_base + (uint32_t)((db * C::NT + nt) * C::NB + r0);
            // scale and zero word of this k-block's group, from the block of MD_SZG groups in shared memory
            if (gb != sz_cur) {                                   // a new block (once per MD_SZG groups): hand the old one back, wait for the new one
                if (sz_cur >= 0) { __syncwarp(); if (lane == 0) mbar_arrive(bar_szempty((sz_n - 1) % MD_SZST)); }
                sz_cur = gb;
                if (!wait(bar_szfull(sz_n % MD_SZST), (sz_n / MD_SZST) & 1)) { live = false; break; }
                sz_stage = smem + C::OFF_SZ + (sz_n % MD_SZST) * C::SZ_STAGE;
                ++sz_n;
            }
            const float sf = H::to_float(reinterpret_cast<const uint16_t*>(sz_stage)[gi * C::COLS + cl]);
            const int nzp1 = -(p.qz ? int((reinterpret_cast<const uint32_t*>(sz_stage + C::S_BYTES)[gi * (C::COLS / C::PACK) + cl / C::PACK] >> zsh) & ZMASK) + 1
                                   : p.zp1_const);
            const unsigned char* bst = smem + C::OFF_B + bs * C::B_STAGE + C::B_TILE;
            // An early poll for the NEXT k-block: the barrier unit answers after ~200 cycles whatever the answer, so the
            // question is asked now and the answer read at the top of the next turn, behind this turn's arithmetic.
            early_ok = 0u;
            if (j + 1 < nrun) {
                const int jn = j + 1;
                asm volatile("{\n.reg .pred p;\nmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.b32 %0, 1, 0, p;\n}"
                             : "=r"(early_ok) : "r"(bar_done(jn % C::BST)), "r"((uint32_t)((jn / C::BST) & 1)) : "memory");
            }
#pragma unroll
            for (int c0 = 0; c0 < C::RW; c0 += C::RC) {
                uint32_t dh[C::RC], dl[C::RC];
                tc_ld<C::RC>(dbase + c0, dh);
                tc_ld<C::RC>(dbase + BM + c0, dl);
                tc_wait_ld();
                if (c0 + C::RC == C::RW) {                       // the accumulator buffer is in registers: it is free for the k-block DBUF later
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_full((j + C::DBUF) % C::BST));
                }
                // stage by stage over the rows of the chunk, so that independent instructions sit next to one another
                // (issuing the next chunk's TMEM loads ahead of this arithmetic measured 3-8 % slower at every batch size)
                int sx[C::RC]; float pe[C::RC];
#pragma unroll
                for (int r = 0; r < C::RC; r += 4) {
                    const int4 sv = *reinterpret_cast<const int4*>(bst + (r0 + c0 + r) * 4);                  // sum_k x' of four batch rows
                    const float4 pv = *reinterpret_cast<const float4*>(bst + BM * 4 + (r0 + c0 + r) * 4);    // their 2^-e
                    sx[r] = sv.x; sx[r + 1] = sv.y; sx[r + 2] = sv.z; sx[r + 3] = sv.w;
                    pe[r] = pv.x; pe[r + 1] = pv.y; pe[r + 2] = pv.z; pe[r + 3] = pv.w;
                }
                int v[C::RC];
#pragma unroll
                for (int r = 0; r < C::RC; ++r) v[r] = (int(dh[r]) << 8) + int(dl[r]);
#pragma unroll
                for (int r = 0; r < C::RC; ++r) v[r] += nzp1 * sx[r];                                         // sum_k (q - (z + 1)) x'
                float f[C::RC];
#pragma unroll
                for (int r = 0; r < C::RC; ++r) f[r] = __int2float_rn(v[r]);
#pragma unroll
                for (int r = 0; r < C::RC; ++r) pe[r] *= sf;
#pragma unroll
                for (int r = 0; r < C::RC; ++r) acc[c0 + r] = fmaf(pe[r], f[r], acc[c0 + r]);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_bempty(bs));
            ++kb;
            if (++kin == p.kpg) { kin = 0; if (++gi == MD_SZG) { gi = 0; ++gb; } }   // next group / next block of groups, no division
        }
            if (!live) break;
            flush(tile);
            kb = 0; ++tile;
            if (sz_cur >= 0) { __syncwarp(); if (lane == 0) mbar_arrive(bar_szempty((sz_n - 1) % MD_SZST)); sz_cur = -1; }   // the next tile starts a new block
        }
        if (fused_ar) {
            // every CTA of the grid reports when its exchanges are done; the last one publishes the epoch for the next call
            asm volatile("bar.sync 1, %0;" ::"n"(MD_FOLD * 32) : "memory");
            if (tid == 0) ar_leave(p.ar, epoch_read ? epoch : ar_epoch(p.ar), gridDim.x);
        }
    }

    // A wait that expired has raised the abort flag and every role has left its loop.  Copies this CTA requested may
    // still be in flight towards its shared memory and MMAs may still be running: give them time to land (they complete
    // within microseconds) before the tensor memory is freed and the CTA exits.
    if (*reinterpret_cast<volatile int*>(&abort_flag)) {
        for (int i = 0; i < 100; ++i) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == MD_W_MMA) {
        tc_fence_after();
        tc_dealloc<512>(tmem_base);
    }
    if (tid == 0 && abort_flag && p.err) atomicExch(p.err, 5u);
}

template <int BITS, typename T, int BM, bool AR>
int launch_inst_ar(cudaStream_t st, const CUtensorMap& mq, const CUtensorMap& ms, const CUtensorMap& mz, const MdParams& p, int grid) {
    using C = MdCfg<BITS, BM>;
    auto kern = qgemm_mid_kernel<BITS, T, BM, AR>;
    static bool configured[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { cudaGetLastError(); return MT_ERR_CUDA; }
    if (!configured[dev]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::TOTAL) != cudaSuccess) { cudaGetLastError(); return MT_ERR_CUDA; }
        configured[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(MD_THREADS); cfg.dynamicSmemBytes = C::TOTAL; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = p.pdl ? 1 : 0;
    if (cudaLaunchKernelEx(&cfg, kern, mq, ms, mz, p) != cudaSuccess) { cudaGetLastError(); return MT_ERR_CUDA; }
    return MT_OK;
}

template <int BITS, typename T, int BM>
int launch_inst(cudaStream_t st, const CUtensorMap& mq, const CUtensorMap& ms, const CUtensorMap& mz, const MdParams& p, int grid) {
    return p.ar.world > 1 ? launch_inst_ar<BITS, T, BM, true>(st, mq, ms, mz, p, grid) : launch_inst_ar<BITS, T, BM, false>(st, mq, ms, mz, p, grid);
}

template <int BITS, typename T>
int launch_bm(cudaStream_t st, const CUtensorMap& mq, const CUtensorMap& ms, const CUtensorMap& mz, const MdParams& p, int grid, int bm) {
    if (bm == 16) return launch_inst<BITS, T, 16>(st, mq, ms, mz, p, grid);
    if (bm == 32) return launch_inst<BITS, T, 32>(st, mq, ms, mz, p, grid);
    return launch_inst<BITS, T, 64>(st, mq, ms, mz, p, grid);
}

template <typename T>
int launch_prep(cudaStream_t st, const void* x, unsigned char* xl, int m, int k, int bm, int bits, int pdl) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(k / MD_KB); cfg.blockDim = dim3(256); cfg.dynamicSmemBytes = 0; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = pdl ? 1 : 0;
    const T* xt = static_cast<const T*>(x);
    cudaError_t e = bits == 4 ? cudaLaunchKernelEx(&cfg, xprep_kernel<T, 4>, xt, xl, m, k, bm, pdl)
                              : cudaLaunchKernelEx(&cfg, xprep_kernel<T, 8>, xt, xl, m, k, bm, pdl);
    if (e != cudaSuccess) { cudaGetLastError(); return MT_ERR_CUDA; }
    return MT_OK;
}

struct MdPlan { int bm, cols, tiles, kbt, grid; size_t partial_bytes, xl_bytes; };

MdPlan plan(int m, int n, int k) {
    MdPlan pl;
    pl.bm = m <= 16 ? 16 : m <= 32 ? 32 : 64;
    pl.cols = pl.bm <= 32 ? 256 : 128;
    pl.tiles = (n + pl.cols - 1) / pl.cols;
    pl.kbt = k / MD_KB;
    const long long units = (long long)pl.tiles * pl.kbt;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    long long g = units / 4;                            // at least 4 k-blocks per CTA
    if (g < 1) g = 1;
    if (g > sms) g = sms;
    pl.grid = (int)g;
    pl.partial_bytes = (size_t)(pl.grid + pl.tiles) * pl.bm * pl.cols * 4;
    pl.xl_bytes = (size_t)pl.kbt * (2 * pl.bm * 128 + pl.bm * 8);
    return pl;
}

}  // namespace

bool mid_supported(const QGemmArgs& a) {
    if (a.g_idx != nullptr || a.m < 1 || a.groups < 1 || a.k % a.groups != 0) return false;
    const int gs = a.k / a.groups;
    if (gs % MD_KB != 0 || a.n % 32 != 0 || a.n < 32) return false;
    if (a.workspace == nullptr || a.workspace_bytes < kCounterBytes) return false;
    if (!get_tensor_map_encoder()) return false;
    const MdPlan pl = plan(a.m < 64 ? a.m : 64, a.n, a.k);
    if ((long long)(pl.tiles + 1) * MD_FOLD > 2LL * (kMaxTiles - 1)) return false;   // 16-bit counters, two per word, the last word is the error word
    if ((long long)pl.tiles * pl.kbt > (1LL << 30)) return false;
    return pl.partial_bytes + pl.xl_bytes <= a.workspace_bytes - kCounterBytes;
}

size_t mid_workspace_bytes(int m, int n, int k) {
    if (k % MD_KB != 0) return 0;
    const MdPlan pl = plan(m < 64 ? m : 64, n, k);
    return pl.partial_bytes + pl.xl_bytes + 256;
}

int launch_mid(cudaStream_t st, const QGemmArgs& a) {
    if (!mid_supported(a)) return MT_ERR_UNSUPPORTED;
    EncodeTiledFn enc = get_tensor_map_encoder();
    const int pack = 32 / a.bits;
    const int m0 = a.m < 64 ? a.m : 64;
    const MdPlan pl0 = plan(m0, a.n, a.k);
    CUtensorMap mq, ms, mz;
    {
        cuuint64_t dims[2] = {(cuuint64_t)a.n, (cuuint64_t)(a.k / pack)};
        cuuint64_t strides[1] = {(cuuint64_t)a.n * 4};
        cuuint32_t box[2] = {(cuuint32_t)pl0.cols, (cuuint32_t)(MD_KB / pack)};
        cuuint32_t es[2] = {1, 1};
        if (enc(&mq, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<uint32_t*>(a.qweight), dims, strides, box, es,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) return MT_ERR_CUDA;
    }
    {
        cuuint64_t dims[2] = {(cuuint64_t)a.n, (cuuint64_t)a.groups};
        cuuint64_t strides[1] = {(cuuint64_t)a.n * 2};
        cuuint32_t box[2] = {(cuuint32_t)pl0.cols, (cuuint32_t)MD_SZG};
        cuuint32_t es[2] = {1, 1};
        if (enc(&ms, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void*>(a.scales), dims, strides, box, es,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) return MT_ERR_CUDA;
    }
    mz = ms;
    if (a.qzeros) {
        cuuint64_t dims[2] = {(cuuint64_t)(a.n / pack), (cuuint64_t)a.groups};
        cuuint64_t strides[1] = {(cuuint64_t)(a.n / pack) * 4};
        cuuint32_t box[2] = {(cuuint32_t)(pl0.cols / pack), (cuuint32_t)MD_SZG};
        cuuint32_t es[2] = {1, 1};
        if (enc(&mz, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<uint32_t*>(a.qzeros), dims, strides, box, es,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) return MT_ERR_CUDA;
    }
    for (int r0 = 0; r0 < a.m; r0 += 64) {
        const int m = a.m - r0 < 64 ? a.m - r0 : 64;
        MdPlan pl = plan(m, a.n, a.k);
        if (pl.cols != pl0.cols) {                       // a last pass with fewer rows keeps the first pass's tile width (one set of tensor maps)
            pl.bm = pl0.cols == 128 ? 64 : pl.bm;
            pl.cols = pl0.cols; pl.tiles = pl0.tiles; pl.grid = pl0.grid;
            pl.partial_bytes = (size_t)(pl.grid + pl.tiles) * pl.bm * pl.cols * 4;
            pl.xl_bytes = (size_t)pl.kbt * (2 * pl.bm * 128 + pl.bm * 8);
        }
        MdParams p;
        unsigned char* base = static_cast<unsigned char*>(a.workspace) + kCounterBytes;
        p.partial = reinterpret_cast<float*>(base);
        unsigned char* xl = base + ((pl.partial_bytes + 255) & ~(size_t)255);
        p.xl = xl;
        p.bias = a.bias;
        p.out = static_cast<char*>(a.out) + (size_t)r0 * a.n * 2;
        p.residual = a.residual ? static_cast<const char*>(a.residual) + (size_t)r0 * a.n * 2 : nullptr;
        p.counters = static_cast<unsigned*>(a.workspace);
        p.err = p.counters + (kMaxTiles - 1);
        p.m = m; p.n = a.n; p.k = a.k;
        p.scales = a.scales; p.qz = a.qzeros;
        p.tiles = pl.tiles; p.kbt = pl.kbt; p.kpg = (a.k / a.groups) / MD_KB;
        p.units = pl.tiles * pl.kbt; p.per = p.units / pl.grid; p.rem = p.units % pl.grid;
        p.zp1_const = 1 << (a.bits - 1);
        p.pdl = (a.flags & MT_FLAG_PDL) ? 1 : 0;
        p.ar = make_ar_params(a);
        if (p.ar.world > 1 && (a.m > 64 || (size_t)a.m * a.n * 8 > p.ar.slot_bytes)) return MT_ERR_TOO_LARGE;
        const void* xrow = static_cast<const char*>(a.x) + (size_t)r0 * a.k * 2;
        int rc = a.dtype == MT_F16 ? launch_prep<__half>(st, xrow, xl, m, a.k, pl.bm, a.bits, p.pdl)
                                   : launch_prep<__nv_bfloat16>(st, xrow, xl, m, a.k, pl.bm, a.bits, p.pdl);
        if (rc != MT_OK) return rc;
        if (a.bits == 4) rc = a.dtype == MT_F16 ? launch_bm<4, __half>(st, mq, ms, mz, p, pl.grid, pl.bm) : launch_bm<4, __nv_bfloat16>(st, mq, ms, mz, p, pl.grid, pl.bm);
        else rc = a.dtype == MT_F16 ? launch_bm<8, __half>(st, mq, ms, mz, p, pl.grid, pl.bm) : launch_bm<8, __nv_bfloat16>(st, mq, ms, mz, p, pl.grid, pl.bm);
        if (rc != MT_OK) return rc;
    }
    return MT_OK;
}

}  // namespace mt
