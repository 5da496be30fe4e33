// C ABI of the quantized-linear path: argument validation, kernel selection, launch
// configuration.  No allocation, no synchronisation, no exceptions.
#include "common.cuh"
#include "qgemm_small.cuh"
#include "qgemm_w8.cuh"

namespace mt {

int launch_small_i4_f16(cudaStream_t, const SmallParams&, int, int, int, bool, dim3, size_t);
int launch_small_i4_bf16(cudaStream_t, const SmallParams&, int, int, int, bool, dim3, size_t);
int launch_small_i8_f16(cudaStream_t, const SmallParams&, int, int, int, bool, dim3, size_t);
int launch_small_i8_bf16(cudaStream_t, const SmallParams&, int, int, int, bool, dim3, size_t);
int launch_w8_inst(cudaStream_t, const W8Params&, int dtype, int mt, int wn, int cpt, dim3, size_t);

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Compute capability of the current device, cached per device ordinal.
static int check_device() {
    static int cached[64] = {0};   // 0 unknown, 1 ok, -1 not sm_100
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); return MT_ERR_CUDA; }
    if (dev < 0 || dev >= 64) return MT_ERR_DEVICE;
    if (cached[dev] == 0) {
        int major = 0;
        if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) {
            cudaGetLastError();
            return MT_ERR_CUDA;
        }
        cached[dev] = (major == 10) ? 1 : -1;
    }
    return cached[dev] == 1 ? MT_OK : MT_ERR_DEVICE;
}

static inline int batch_tiles(int m) { return m <= 8 ? 1 : m <= 16 ? 2 : m <= 32 ? 4 : 8; }

struct SplitPlan { int wn, tiles, splits, chunks_per_split; };

// Pick the CTA width and the split-K factor: enough CTAs to cover 148 SMs twice, as wide a
// column tile as that allows (longer contiguous row segments), and split-K partial traffic
// held to about a quarter of the weight bytes.
static SplitPlan plan_splits(int m, int n, int k, int bits, int nchunks, int cols_per_warp,
                             const int* wn_options, int n_options, size_t partial_capacity_bytes) {
    const int target = 148 * 2;
    long long smax = ((long long)k * bits) / (256LL * m);
    if (smax < 1) smax = 1;
    if (smax > nchunks) smax = nchunks;
    const long long cap = (long long)(partial_capacity_bytes / ((size_t)m * n * 4));
    if (smax > cap) smax = cap < 1 ? 1 : cap;
    SplitPlan best = {0, 0, 0, 0};
    for (int i = 0; i < n_options; ++i) {
        const int wn = wn_options[i];
        const int tile_cols = wn * cols_per_warp;
        const int tiles = (n + tile_cols - 1) / tile_cols;
        if (tiles > kMaxTiles) continue;
        long long s = (target + tiles - 1) / tiles;
        if (s > smax) s = smax;
        if (s < 1) s = 1;
        const int cps = (nchunks + (int)s - 1) / (int)s;
        const int splits = (nchunks + cps - 1) / cps;
        SplitPlan cand = {wn, tiles, splits, cps};
        if (best.wn == 0) best = cand;
        if ((long long)tiles * splits >= (target * 3) / 4) return cand;   // widest tile that fills the GPU
        if ((long long)tiles * splits > (long long)best.tiles * best.splits) best = cand;
    }
    return best;
}

int launch_small(cudaStream_t st, const QGemmArgs& a) {
    const int bits = a.bits, pack = 32 / bits;
    const int kc = bits == 4 ? 256 : 128, kstep = 4 * pack;
    const int nchunks = (a.k + kc - 1) / kc;
    const int gs = a.k / a.groups;
    const bool act = a.g_idx != nullptr;
    int gpc = 1;
    if (!act) {
        if (gs % kc == 0) gpc = 1;
        else if (gs % (kc / 2) == 0) gpc = 2;
        else if (gs % kstep == 0) gpc = 8;
        else return MT_ERR_SHAPE;
    }
    if (a.workspace == nullptr || a.workspace_bytes < kCounterBytes) return MT_ERR_WORKSPACE;
    const size_t partial_cap = a.workspace_bytes - kCounterBytes;
    auto fn = bits == 4 ? (a.dtype == MT_F16 ? launch_small_i4_f16 : launch_small_i4_bf16)
                        : (a.dtype == MT_F16 ? launch_small_i8_f16 : launch_small_i8_bf16);
    const size_t esz = 2;
    for (int r0 = 0; r0 < a.m; r0 += 64) {
        const int m = a.m - r0 < 64 ? a.m - r0 : 64;
        const int mt = batch_tiles(m);
        const int pitch = kc * 2 + (bits == 4 ? 64 : 32);
        int opts[3]; int nopts = 0;
        const int all[3] = {8, 4, 2};
        for (int i = 0; i < 3; ++i) {
            const int wn = all[i];
            if (mt == 8 && wn != 8) continue;
            if (mt == 4 && wn == 2) continue;
            const size_t smem = (size_t)2 * mt * 8 * pitch + (act ? (size_t)a.groups * wn * 32 * 4 + 2 * kc * 4 : 0);
            if (smem > 200 * 1024) continue;
            opts[nopts++] = wn;
        }
        if (nopts == 0) return MT_ERR_TOO_LARGE;
        const SplitPlan pl = plan_splits(m, a.n, a.k, bits, nchunks, 32, opts, nopts, partial_cap);
        if (pl.wn == 0) return MT_ERR_TOO_LARGE;
        if (pl.splits > 1 && (size_t)pl.splits * m * a.n * 4 > partial_cap) return MT_ERR_WORKSPACE;
        SmallParams p;
        p.x = static_cast<const char*>(a.x) + (size_t)r0 * a.k * esz;
        p.qw = a.qweight; p.g_idx = a.g_idx; p.qz = a.qzeros; p.scales = a.scales; p.bias = a.bias;
        p.out = static_cast<char*>(a.out) + (size_t)r0 * a.n * esz;
        p.counters = static_cast<unsigned*>(a.workspace);
        p.partial = reinterpret_cast<float*>(static_cast<char*>(a.workspace) + kCounterBytes);
        p.m = m; p.n = a.n; p.k = a.k; p.groups = a.groups; p.gs = gs;
        p.nchunks = nchunks; p.chunks_per_split = pl.chunks_per_split; p.splits = pl.splits;
        p.zp1_const = 1 << (bits - 1);
        p.pdl = (a.flags & MT_FLAG_PDL) ? 1 : 0;
        p.ar = make_ar_params(a);
        if (p.ar.world > 1 && (size_t)m * a.n * 8 > p.ar.slot_bytes) return MT_ERR_TOO_LARGE;
        const size_t smem = (size_t)2 * mt * 8 * pitch + (act ? (size_t)a.groups * pl.wn * 32 * 4 + 2 * kc * 4 : 0);
        const int rc = fn(st, p, mt, pl.wn, gpc, act, dim3(pl.tiles, pl.splits), smem);
        if (rc != MT_OK) return rc;
    }
    return MT_OK;
}

int launch_small_w8(cudaStream_t st, const QGemmArgs& a) {
    const int kc = 128;
    const int nchunks = (a.k + kc - 1) / kc;
    if (a.workspace == nullptr || a.workspace_bytes < kCounterBytes) return MT_ERR_WORKSPACE;
    const size_t partial_cap = a.workspace_bytes - kCounterBytes;
    for (int r0 = 0; r0 < a.m; r0 += 64) {
        const int m = a.m - r0 < 64 ? a.m - r0 : 64;
        const int mt = batch_tiles(m);
        const int cpt = mt <= 2 ? 16 : 8;
        int opts[2]; int nopts = 0;
        if (mt <= 2) { opts[nopts++] = 4; opts[nopts++] = 2; } else { opts[nopts++] = 4; }
        const SplitPlan pl = plan_splits(m, a.n, a.k, 8, nchunks, 8 * cpt, opts, nopts, partial_cap);
        if (pl.wn == 0) return MT_ERR_TOO_LARGE;
        if (pl.splits > 1 && (size_t)pl.splits * m * a.n * 4 > partial_cap) return MT_ERR_WORKSPACE;
        W8Params p;
        p.x = static_cast<const char*>(a.x) + (size_t)r0 * a.k * 2;
        p.w = a.w8; p.scales = a.scales; p.bias = a.bias;
        p.out = static_cast<char*>(a.out) + (size_t)r0 * a.n * 2;
        p.counters = static_cast<unsigned*>(a.workspace);
        p.partial = reinterpret_cast<float*>(static_cast<char*>(a.workspace) + kCounterBytes);
        p.m = m; p.n = a.n; p.k = a.k;
        p.nchunks = nchunks; p.chunks_per_split = pl.chunks_per_split; p.splits = pl.splits;
        p.pdl = (a.flags & MT_FLAG_PDL) ? 1 : 0;
        const size_t smem = (size_t)2 * mt * 8 * (kc * 2 + 32);
        const int rc = launch_w8_inst(st, p, a.dtype, mt, pl.wn, cpt, dim3(pl.tiles, pl.splits), smem);
        if (rc != MT_OK) return rc;
    }
    return MT_OK;
}

}  // namespace mt

using namespace mt;

extern "C" {

int mt_version(void) { return 100; }

const char* mt_strerror(int status) {
    switch (status) {
        case MT_OK: return "ok";
        case MT_ERR_NULL: return "a required pointer is NULL";
        case MT_ERR_ALIGN: return "a pointer is not 16-byte aligned";
        case MT_ERR_SHAPE: return "m/n/k/nr_groups violate the layout rules";
        case MT_ERR_DTYPE: return "dtype must be MT_F16 (0) or MT_BF16 (1)";
        case MT_ERR_BITS: return "bits must be 4 or 8";
        case MT_ERR_WORKSPACE: return "workspace is missing or smaller than mt_workspace_bytes()";
        case MT_ERR_CUDA: return "the CUDA runtime reported an error";
        case MT_ERR_UNSUPPORTED: return "no kernel in this build for the request";
        case MT_ERR_DEVICE: return "the current device is not compute capability 10.x (B200)";
        case MT_ERR_TOO_LARGE: return "the request exceeds a fixed built-in capacity";
        case MT_ERR_NCCL: return "NCCL reported an error or could not be loaded";
        case MT_ERR_PEER_TIMEOUT: return "a bounded wait inside a kernel expired (a peer rank was late or absent); the output is not valid";
    }
    return "unknown status";
}

size_t mt_workspace_bytes(int m, int n, int k, int bits) {
    if (m <= 0 || n <= 0 || k <= 0 || (bits != 4 && bits != 8)) return kCounterBytes;
    // split-K keeps splits * min(m,64) <= k*bits/256 + 64 rows of fp32 partials
    const size_t rows = (size_t)k * bits / 256 + 64;
    size_t bytes = rows * (size_t)n * 4;
    if (m > 2 && m <= 192 && k % 64 == 0) {                     // fp32 partial tiles of the mid-batch kernel
        const size_t mid = umma_workspace_bytes(m, n, k);
        if (mid > bytes) bytes = mid;
    }
    if (m > 2 && k % 128 == 0) {                                // partial tiles and the two-limb activation tiles of the integer kernel
        const size_t mid = mid_workspace_bytes(m, n, k);
        if (mid > bytes) bytes = mid;
    }
    if (m > 32 && m <= 192 && bits == 4) {                       // one row of tiles of the tensor-memory-A kernel, every tile cut along K
        const size_t parts = tcx_rows_workspace_bytes(m, n, k);
        if (parts > bytes) bytes = parts;
    }
    if (m > 128 && bits == 4) {                                  // prefill: the last wave of tiles cut along K
        const size_t tail = tcx_workspace_bytes(m, n, k);
        if (tail > bytes) bytes = tail;
    }
    return kCounterBytes + bytes;
}

static int validate_gptq(const uint32_t* qweight, const uint32_t* qzeros, const void* scales,
                         int n, int k, int nr_groups, int bits, int dtype) {
    if (bits != 4 && bits != 8) return MT_ERR_BITS;
    if (dtype != MT_F16 && dtype != MT_BF16) return MT_ERR_DTYPE;
    if (n < 0 || k < 0 || nr_groups < 1) return MT_ERR_SHAPE;
    if (n % 8 != 0 || k % 32 != 0 || k % nr_groups != 0) return MT_ERR_SHAPE;
    if (n == 0 || k == 0) return MT_OK;
    if (!qweight || !scales) return MT_ERR_NULL;
    if (!aligned16(qweight) || !aligned16(scales) || (qzeros && !aligned16(qzeros))) return MT_ERR_ALIGN;
    return MT_OK;
}

int mt_dequant(void* stream, const uint32_t* qweight, const int32_t* g_idx, const uint32_t* qzeros,
               const void* scales, void* w_out, int n, int k, int nr_groups, int bits, int dtype) {
    int rc = validate_gptq(qweight, qzeros, scales, n, k, nr_groups, bits, dtype);
    if (rc != MT_OK) return rc;
    if (n == 0 || k == 0) return MT_OK;
    if (!w_out) return MT_ERR_NULL;
    if (!aligned16(w_out)) return MT_ERR_ALIGN;
    if ((rc = check_device()) != MT_OK) return rc;
    return launch_dequant(static_cast<cudaStream_t>(stream), qweight, g_idx, qzeros, scales, w_out, n, k, nr_groups, bits, dtype);
}

int mt_dequant_unpacked(void* stream, const uint8_t* q, const int32_t* g_idx, const uint8_t* z, const void* scales,
                        void* w_out, int n, int k, int nr_groups, int dtype) {
    if (dtype != MT_F16 && dtype != MT_BF16) return MT_ERR_DTYPE;
    if (n < 0 || k < 0 || nr_groups < 1 || n % 4 != 0 || (!g_idx && k % nr_groups != 0)) return MT_ERR_SHAPE;
    if (n == 0 || k == 0) return MT_OK;
    if (!q || !z || !scales || !w_out) return MT_ERR_NULL;
    if (!aligned16(q) || !aligned16(z) || !aligned16(scales) || !aligned16(w_out)) return MT_ERR_ALIGN;
    int rc = check_device();
    if (rc != MT_OK) return rc;
    return launch_dequant_unpacked(static_cast<cudaStream_t>(stream), q, g_idx, z, scales, w_out, n, k, nr_groups, dtype);
}

int mt_unpack(void* stream, const uint32_t* packed, uint8_t* out, int rows, int cols, int bits, int axis) {
    if (bits != 4 && bits != 8) return MT_ERR_BITS;
    if (axis != 0 && axis != 1) return MT_ERR_SHAPE;
    const int pack = 32 / bits;
    if (rows < 0 || cols < 0 || (axis == 0 ? rows % pack : cols % pack) != 0) return MT_ERR_SHAPE;
    if (rows == 0 || cols == 0) return MT_OK;
    if (!packed || !out) return MT_ERR_NULL;
    int rc = check_device();
    if (rc != MT_OK) return rc;
    return launch_unpack(static_cast<cudaStream_t>(stream), packed, out, rows, cols, bits, axis);
}

// Where the integer tensor-core kernel beats the register-ring kernel, from timings of both on the linears of a
// 70B decoder layer split 1, 2, 4 and 8 ways (K or N from 1024 to 57344): the more rows, the smaller the weights at
// which its set-up is paid back; with few k-blocks (K < 3072) the ring kernel always wins.
static bool mid_preferred(int m, int n, int k) {
    if (m < 3 || m > 32 || k < 3072) return false;
    const long long weights = (long long)k * n;
    if (m <= 8) return weights >= 100LL * 1000 * 1000;
    if (m <= 16) return weights >= 40LL * 1000 * 1000;
    return weights >= 8LL * 1000 * 1000;
}

int mt_qgemm(void* stream, const void* x, const uint32_t* qweight, const int32_t* g_idx,
             const uint32_t* qzeros, const void* scales, const void* bias, void* out,
             int m, int n, int k, int nr_groups, int bits, int dtype,
             void* workspace, size_t workspace_bytes, int flags) {
    int rc = validate_gptq(qweight, qzeros, scales, n, k, nr_groups, bits, dtype);
    if (rc != MT_OK) return rc;
    if (m < 0) return MT_ERR_SHAPE;
    if (m == 0 || n == 0) return MT_OK;
    if (k == 0) return MT_ERR_SHAPE;
    if (!x || !out) return MT_ERR_NULL;
    if (!aligned16(x) || !aligned16(out) || (bias && !aligned16(bias))) return MT_ERR_ALIGN;
    if (!g_idx && (k / nr_groups) % (4 * (32 / bits)) != 0) return MT_ERR_SHAPE;
    if (workspace && !aligned16(workspace)) return MT_ERR_ALIGN;
    if ((rc = check_device()) != MT_OK) return rc;
    QGemmArgs a = {};
    a.x = x; a.qweight = qweight; a.g_idx = g_idx; a.qzeros = qzeros; a.scales = scales; a.bias = bias; a.out = out;
    a.m = m; a.n = n; a.k = k; a.groups = nr_groups; a.bits = bits; a.dtype = dtype;
    a.workspace = workspace; a.workspace_bytes = workspace_bytes; a.flags = flags;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (flags & MT_FLAG_FORCE_TC) return tc_supported(a) ? launch_tc(st, a) : MT_ERR_UNSUPPORTED;
    if (flags & MT_FLAG_FORCE_SMALL) return launch_small(st, a);
    if (flags & MT_FLAG_FORCE_VEC) return vec_supported(a) ? launch_vec(st, a) : MT_ERR_UNSUPPORTED;
    if (flags & MT_FLAG_FORCE_UMMA) return umma_supported(a) ? launch_umma(st, a) : MT_ERR_UNSUPPORTED;
    if (flags & MT_FLAG_FORCE_MID) return mid_supported(a) ? launch_mid(st, a) : MT_ERR_UNSUPPORTED;
    // Mid-size batches.  Up to 32 rows the integer tensor-core kernel (packed nibbles as unsigned bytes, two-limb
    // activations, scale and zero point folded per 128 values of k) holds 0.38-0.56 of HBM peak on large weights; it
    // pays ~10 us of set-up (a pre-pass launch, tensor maps, tensor-memory allocation), so smaller weights stay on the
    // register-ring kernel (mid_preferred).  From 33 to 64 rows its fold costs more than dequantizing, and the tcgen05
    // kernel whose sixteen warps rebuild fp16 weights takes over; between 64 and 128 rows two passes of that one beat
    // the prefill kernels when K is deep (their grid has no split along K).
    const long long weights = (long long)k * n;
    if (mid_preferred(m, n, k) && mid_supported(a)) return launch_mid(st, a);
    // 33 to 192 rows on int4 weights with contiguous groups: one row of tiles of the tensor-memory-A prefill kernel, every tile
    // cut along K (28672 x 8192 at 64 rows: 76 us against 109 us for the mid-batch kernel; 8192 x 57344: 172 against 170).
    // Up to 64 rows it wins where the weight has fewer 256-column tiles than the GPU has SMs (the cut along K then fills the
    // GPU: 28672 x 8192 76-83 us against 109, 4096 x 28672 40 against 60); with more tiles the mid-batch kernel's stream-K
    // partition is as good or better (8192 x 57344: 169 us against 172-212).
    if (m > 32 && m <= 192 && tcx_rows_supported(a) && (m > 64 || (n + 255) / 256 < 148 || !umma_supported(a))) return launch_tcx_rows(st, a);
    if (umma_supported(a)) {
        if (m > 32 && m <= 64) return launch_umma(st, a);
        if (m > 8 && m <= 32 && weights >= (128LL << 20)) return launch_umma(st, a);
        if (m > 64 && m <= 128 && k >= 8192 && !(tc_tmem_a_preferred(m, n, bits) && tc_supported(a))) return launch_umma(st, a);
    }
    if (m > 64 && tc_supported(a)) return launch_tc(st, a);
    // Decode at M <= 2: the CUDA-core GEMV (packed integers multiplied as fp16 subnormals) streams
    // 1.5-2x faster than either tensor-core decode kernel on every shape measured.
    if (m <= 2 && vec_supported(a)) return launch_vec(st, a);
    return launch_small(st, a);
}

static int qgemm_allreduce_impl(void* stream, const void* x, const uint32_t* qweight, const int32_t* g_idx,
                               const uint32_t* qzeros, const void* scales, const void* bias, const void* residual, void* out,
                               int m, int n, int k, int nr_groups, int bits, int dtype,
                               void* workspace, size_t workspace_bytes, int flags,
                               void* const* peer_buffers, int rank, int world, size_t buffer_bytes) {
    int rc = validate_gptq(qweight, qzeros, scales, n, k, nr_groups, bits, dtype);
    if (rc != MT_OK) return rc;
    if (m < 0 || m > 64 || k == 0) return MT_ERR_SHAPE;          // one launch: the exchange is per launch
    if (world < 1 || world > kArMaxWorld || rank < 0 || rank >= world) return MT_ERR_SHAPE;
    if (m == 0 || n == 0) return MT_OK;
    if (!x || !out || (world > 1 && !peer_buffers)) return MT_ERR_NULL;
    if (!aligned16(x) || !aligned16(out) || (bias && !aligned16(bias)) || (workspace && !aligned16(workspace))) return MT_ERR_ALIGN;
    if (residual && !aligned16(residual)) return MT_ERR_ALIGN;
    if (!g_idx && (k / nr_groups) % (4 * (32 / bits)) != 0) return MT_ERR_SHAPE;
    if (world > 1 && buffer_bytes < kArDataOffset + 2 * (size_t)world * 256) return MT_ERR_WORKSPACE;
    if ((rc = check_device()) != MT_OK) return rc;
    QGemmArgs a = {};
    a.x = x; a.qweight = qweight; a.g_idx = g_idx; a.qzeros = qzeros; a.scales = scales; a.bias = bias; a.out = out;
    a.m = m; a.n = n; a.k = k; a.groups = nr_groups; a.bits = bits; a.dtype = dtype;
    a.workspace = workspace; a.workspace_bytes = workspace_bytes; a.flags = flags;
    if (world > 1) {
        a.ar_peers = reinterpret_cast<unsigned char* const*>(peer_buffers);
        a.ar_rank = rank; a.ar_world = world; a.ar_bytes = buffer_bytes;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (!(flags & MT_FLAG_FORCE_SMALL) && m <= 2 && vec_supported(a)) {
        a.residual = residual;                                   // the GEMV adds it to the reduced sum before its one rounding
        return launch_vec(st, a);
    }
    if (!(flags & MT_FLAG_FORCE_SMALL) && (mid_preferred(m, n, k) || ((flags & MT_FLAG_FORCE_MID) && m > 2)) && mid_supported(a)) {
        a.residual = residual;                                   // the integer kernel exchanges and adds it in its epilogue too
        return launch_mid(st, a);
    }
    rc = launch_small(st, a);
    if (rc == MT_OK && residual) rc = launch_add_residual(st, out, residual, m, n, dtype);
    return rc;
}

int mt_qgemm_allreduce(void* stream, const void* x, const uint32_t* qweight, const int32_t* g_idx,
                       const uint32_t* qzeros, const void* scales, const void* bias, void* out,
                       int m, int n, int k, int nr_groups, int bits, int dtype,
                       void* workspace, size_t workspace_bytes, int flags,
                       void* const* peer_buffers, int rank, int world, size_t buffer_bytes) {
    return qgemm_allreduce_impl(stream, x, qweight, g_idx, qzeros, scales, bias, nullptr, out, m, n, k, nr_groups, bits, dtype,
                                workspace, workspace_bytes, flags, peer_buffers, rank, world, buffer_bytes);
}

int mt_qgemm_residual(void* stream, const void* x, const uint32_t* qweight, const int32_t* g_idx,
                      const uint32_t* qzeros, const void* scales, const void* bias, const void* residual, void* out,
                      int m, int n, int k, int nr_groups, int bits, int dtype,
                      void* workspace, size_t workspace_bytes, int flags,
                      void* const* peer_buffers, int rank, int world, size_t buffer_bytes) {
    if (world > 1)
        return qgemm_allreduce_impl(stream, x, qweight, g_idx, qzeros, scales, bias, residual, out, m, n, k, nr_groups, bits, dtype,
                                    workspace, workspace_bytes, flags, peer_buffers, rank, world, buffer_bytes);
    if (!residual) return mt_qgemm(stream, x, qweight, g_idx, qzeros, scales, bias, out, m, n, k, nr_groups, bits, dtype, workspace, workspace_bytes, flags);
    // one rank: any batch size.  The decode GEMV adds the residual in its epilogue; every other kernel is
    // followed by one elementwise launch.
    if (!aligned16(residual)) return MT_ERR_ALIGN;
    const bool forced_other = (flags & (MT_FLAG_FORCE_SMALL | MT_FLAG_FORCE_TC | MT_FLAG_FORCE_UMMA)) != 0;
    if (m >= 1 && m <= 2 && !forced_other && !g_idx)
        return qgemm_allreduce_impl(stream, x, qweight, g_idx, qzeros, scales, bias, residual, out, m, n, k, nr_groups, bits, dtype,
                                    workspace, workspace_bytes, flags, nullptr, 0, 1, 0);
    int rc = mt_qgemm(stream, x, qweight, g_idx, qzeros, scales, bias, out, m, n, k, nr_groups, bits, dtype, workspace, workspace_bytes, flags);
    if (rc == MT_OK && m > 0 && n > 0) rc = launch_add_residual(static_cast<cudaStream_t>(stream), out, residual, m, n, dtype);
    return rc;
}

int mt_qgemm_chain(void* stream, const mt_chain_linear* linears, int count, int m, int bits, int dtype,
                   void* workspace, size_t workspace_bytes, int flags,
                   void* const* peer_buffers, int rank, int world, size_t buffer_bytes) {
    if (count < 0) return MT_ERR_SHAPE;
    if (count == 0 || m == 0) return MT_OK;
    if (!linears) return MT_ERR_NULL;
    if (count > MT_CHAIN_MAX || m < 0 || m > 2) return MT_ERR_UNSUPPORTED;
    if (world < 1 || world > kArMaxWorld || rank < 0 || rank >= world) return MT_ERR_SHAPE;
    if (!workspace) return MT_ERR_NULL;
    if (!aligned16(workspace)) return MT_ERR_ALIGN;
    QGemmArgs list[MT_CHAIN_MAX];
    bool any_ar = false;
    for (int e = 0; e < count; ++e) {
        const mt_chain_linear& l = linears[e];
        int rc = validate_gptq(l.qweight, l.qzeros, l.scales, l.n, l.k, l.nr_groups, bits, dtype);
        if (rc != MT_OK) return rc;
        if (l.n == 0 || l.k == 0) return MT_ERR_SHAPE;
        if (l.epilogue != MT_EPILOGUE_NONE && l.epilogue != MT_EPILOGUE_SWIGLU) return MT_ERR_UNSUPPORTED;
        if (l.epilogue == MT_EPILOGUE_SWIGLU && (l.n % 16 != 0 || l.allreduce || l.residual)) return MT_ERR_UNSUPPORTED;
        if (!l.x || !l.out) return MT_ERR_NULL;
        if (!aligned16(l.x) || !aligned16(l.out) || (l.bias && !aligned16(l.bias)) || (l.residual && !aligned16(l.residual))) return MT_ERR_ALIGN;
        if ((l.k / l.nr_groups) % (4 * (32 / bits)) != 0) return MT_ERR_SHAPE;
        QGemmArgs a = {};
        a.x = l.x; a.qweight = l.qweight; a.qzeros = l.qzeros; a.scales = l.scales; a.bias = l.bias; a.out = l.out;
        a.residual = l.residual; a.epilogue = l.epilogue;
        a.m = m; a.n = l.n; a.k = l.k; a.groups = l.nr_groups; a.bits = bits; a.dtype = dtype;
        a.workspace = workspace; a.workspace_bytes = workspace_bytes; a.flags = flags;
        if (l.allreduce && world > 1) {
            if (!peer_buffers) return MT_ERR_NULL;
            if (buffer_bytes < kArDataOffset + 2 * (size_t)world * 256) return MT_ERR_WORKSPACE;
            a.ar_peers = reinterpret_cast<unsigned char* const*>(peer_buffers);
            a.ar_rank = rank; a.ar_world = world; a.ar_bytes = buffer_bytes;
            any_ar = true;
        }
        list[e] = a;
    }
    (void)any_ar;
    const int rc = check_device();
    if (rc != MT_OK) return rc;
    return launch_vec_chain(static_cast<cudaStream_t>(stream), list, count);
}

int mt_qgemm_swiglu(void* stream, const void* x, const uint32_t* qweight, const uint32_t* qzeros, const void* scales,
                    const void* bias, void* out, void* scratch, int m, int n, int k, int nr_groups, int bits, int dtype,
                    void* workspace, size_t workspace_bytes, int flags) {
    int rc = validate_gptq(qweight, qzeros, scales, n, k, nr_groups, bits, dtype);
    if (rc != MT_OK) return rc;
    if (m < 0 || n % 16 != 0) return MT_ERR_SHAPE;               // out rows of N/2 values keep the 16-byte alignment
    if (m == 0 || n == 0) return MT_OK;
    if (k == 0) return MT_ERR_SHAPE;
    if (!x || !out) return MT_ERR_NULL;
    if (!aligned16(x) || !aligned16(out) || (bias && !aligned16(bias)) || (workspace && !aligned16(workspace))) return MT_ERR_ALIGN;
    if ((k / nr_groups) % (4 * (32 / bits)) != 0) return MT_ERR_SHAPE;
    if ((rc = check_device()) != MT_OK) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    QGemmArgs a = {};
    a.x = x; a.qweight = qweight; a.qzeros = qzeros; a.scales = scales; a.bias = bias; a.out = out;
    a.m = m; a.n = n; a.k = k; a.groups = nr_groups; a.bits = bits; a.dtype = dtype;
    a.workspace = workspace; a.workspace_bytes = workspace_bytes; a.flags = flags;
    const bool forced_other = (flags & (MT_FLAG_FORCE_SMALL | MT_FLAG_FORCE_TC | MT_FLAG_FORCE_UMMA)) != 0;
    if (m <= 2 && !forced_other && vec_supported(a)) {
        a.epilogue = MT_EPILOGUE_SWIGLU;
        return launch_vec(st, a);
    }
    if (!scratch) return MT_ERR_NULL;
    if (!aligned16(scratch)) return MT_ERR_ALIGN;
    rc = mt_qgemm(stream, x, qweight, nullptr, qzeros, scales, bias, scratch, m, n, k, nr_groups, bits, dtype, workspace, workspace_bytes, flags);
    if (rc == MT_OK) rc = launch_swiglu_interleaved(st, scratch, out, m, n, dtype);
    return rc;
}

int mt_interleave_gate_up(void* stream, const uint32_t* gate_qweight, const uint32_t* up_qweight,
                          const uint32_t* gate_qzeros, const uint32_t* up_qzeros, const void* gate_scales, const void* up_scales,
                          const void* gate_bias, const void* up_bias,
                          uint32_t* qweight_out, uint32_t* qzeros_out, void* scales_out, void* bias_out,
                          int n_half, int k, int nr_groups, int bits) {
    if (bits != 4 && bits != 8) return MT_ERR_BITS;
    if (n_half < 0 || k < 0 || nr_groups < 1 || n_half % 8 != 0 || k % 32 != 0) return MT_ERR_SHAPE;
    if (n_half == 0 || k == 0) return MT_OK;
    if (!gate_qweight || !up_qweight || !gate_scales || !up_scales || !qweight_out || !scales_out) return MT_ERR_NULL;
    if ((gate_qzeros == nullptr) != (up_qzeros == nullptr) || (gate_qzeros == nullptr) != (qzeros_out == nullptr)) return MT_ERR_NULL;
    if ((gate_bias == nullptr) != (up_bias == nullptr) || (gate_bias == nullptr) != (bias_out == nullptr)) return MT_ERR_NULL;
    int rc = check_device();
    if (rc != MT_OK) return rc;
    return launch_interleave_gate_up(static_cast<cudaStream_t>(stream), gate_qweight, up_qweight, gate_qzeros, up_qzeros,
                                     gate_scales, up_scales, gate_bias, up_bias, qweight_out, qzeros_out, scales_out, bias_out,
                                     n_half, k, nr_groups, bits);
}

int mt_swiglu(void* stream, const void* gate_up, void* out, int m, int n, int dtype) {
    if (dtype != MT_F16 && dtype != MT_BF16) return MT_ERR_DTYPE;
    if (m < 0 || n < 0 || n % 16 != 0) return MT_ERR_SHAPE;
    if (m == 0 || n == 0) return MT_OK;
    if (!gate_up || !out) return MT_ERR_NULL;
    if (!aligned16(gate_up) || !aligned16(out)) return MT_ERR_ALIGN;
    int rc = check_device();
    if (rc != MT_OK) return rc;
    return launch_swiglu_interleaved(static_cast<cudaStream_t>(stream), gate_up, out, m, n, dtype);
}

int mt_rms_norm(void* stream, const void* x, const void* weight, void* out, int rows, int h, float eps, int dtype) {
    if (dtype != MT_F16 && dtype != MT_BF16) return MT_ERR_DTYPE;
    if (rows < 0 || h < 0 || h % 8 != 0 || !(eps > 0.f)) return MT_ERR_SHAPE;
    if (rows == 0 || h == 0) return MT_OK;
    if (!x || !weight || !out) return MT_ERR_NULL;
    if (!aligned16(x) || !aligned16(weight) || !aligned16(out)) return MT_ERR_ALIGN;
    int rc = check_device();
    if (rc != MT_OK) return rc;
    return launch_rms_norm(static_cast<cudaStream_t>(stream), x, weight, out, rows, h, eps, dtype);
}

int mt_rope_append(void* stream, const void* qkv, const float* cos_table, const float* sin_table, void* q_out, void* k_cache, void* v_cache,
                   int m, int hq, int hkv, int d, int offset, const int32_t* offset_dev, int capacity, int table_rows, int dtype) {
    if (dtype != MT_F16 && dtype != MT_BF16) return MT_ERR_DTYPE;
    if (m < 0 || hq < 1 || hkv < 1 || offset < 0 || capacity < 1 || table_rows < 1) return MT_ERR_SHAPE;
    if (d < 2 || d % 2 != 0 || d > 1024) return MT_ERR_UNSUPPORTED;
    if (!offset_dev && (offset + m > capacity || offset + m > table_rows)) return MT_ERR_SHAPE;
    if (m == 0) return MT_OK;
    if (!qkv || !cos_table || !sin_table || !q_out || !k_cache || !v_cache) return MT_ERR_NULL;
    int rc = check_device();
    if (rc != MT_OK) return rc;
    return launch_rope_append(static_cast<cudaStream_t>(stream), qkv, cos_table, sin_table, q_out, k_cache, v_cache, m, hq, hkv, d, offset,
                              offset_dev, capacity, table_rows, dtype);
}

int mt_attention(void* stream, const void* q, const void* k_cache, const void* v_cache, void* out, const int32_t* offsets_dev,
                 int batch, int m, int hq, int hkv, int d, int offset, int capacity, float scale, int dtype) {
    if (dtype != MT_F16 && dtype != MT_BF16) return MT_ERR_DTYPE;
    if (batch < 0 || m < 0 || hq < 1 || hkv < 1 || offset < 0 || capacity < 1) return MT_ERR_SHAPE;
    if (!offsets_dev && offset + m > capacity) return MT_ERR_SHAPE;
    if (batch == 0 || m == 0) return MT_OK;
    if (!q || !k_cache || !v_cache || !out) return MT_ERR_NULL;
    if (!aligned16(q) || !aligned16(k_cache) || !aligned16(v_cache) || !aligned16(out)) return MT_ERR_ALIGN;
    int rc = check_device();
    if (rc != MT_OK) return rc;
    return launch_attention_rows(static_cast<cudaStream_t>(stream), q, k_cache, v_cache, out, offsets_dev, batch, m, hq, hkv, d, offset,
                                 capacity, scale, dtype);
}

int mt_qgemm_rope_append(void* stream, const void* x, const uint32_t* qweight, const uint32_t* qzeros, const void* scales, const void* bias,
                         const float* cos_table, const float* sin_table, void* q_out, void* k_cache, void* v_cache, void* scratch,
                         int m, int hq, int hkv, int d, int k, int nr_groups, int bits, int dtype,
                         int offset, const int32_t* offset_dev, int capacity, int table_rows,
                         void* workspace, size_t workspace_bytes, int flags) {
    if (hq < 1 || hkv < 1 || offset < 0 || capacity < 1 || table_rows < 1) return MT_ERR_SHAPE;
    if (d < 2 || d % 2 != 0 || d > 1024) return MT_ERR_UNSUPPORTED;
    const int n = (hq + 2 * hkv) * d;
    int rc = validate_gptq(qweight, qzeros, scales, n, k, nr_groups, bits, dtype);
    if (rc != MT_OK) return rc;
    if (m < 0 || k == 0) return MT_ERR_SHAPE;
    if (!offset_dev && (offset + m > capacity || offset + m > table_rows)) return MT_ERR_SHAPE;
    if (m == 0) return MT_OK;
    if (!x || !cos_table || !sin_table || !q_out || !k_cache || !v_cache) return MT_ERR_NULL;
    if (!aligned16(x) || !aligned16(q_out) || !aligned16(k_cache) || !aligned16(v_cache) || (bias && !aligned16(bias)) ||
        (workspace && !aligned16(workspace))) return MT_ERR_ALIGN;
    if ((k / nr_groups) % (4 * (32 / bits)) != 0) return MT_ERR_SHAPE;
    if ((rc = check_device()) != MT_OK) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    QGemmArgs a = {};
    a.x = x; a.qweight = qweight; a.qzeros = qzeros; a.scales = scales; a.bias = bias; a.out = q_out;
    a.m = m; a.n = n; a.k = k; a.groups = nr_groups; a.bits = bits; a.dtype = dtype;
    a.workspace = workspace; a.workspace_bytes = workspace_bytes; a.flags = flags;
    const bool forced_other = (flags & (MT_FLAG_FORCE_SMALL | MT_FLAG_FORCE_TC | MT_FLAG_FORCE_UMMA)) != 0;
    if (m <= 2 && d == 128 && !forced_other && vec_supported(a)) {       // the GEMV's rotary epilogue is written for 128-wide heads
        RopeArgs r;
        r.cosv = cos_table; r.sinv = sin_table; r.q_out = q_out; r.k_cache = k_cache; r.v_cache = v_cache; r.offset_dev = offset_dev;
        r.hq = hq; r.hkv = hkv; r.offset = offset; r.capacity = capacity; r.table_rows = table_rows;
        a.rope = &r;
        return launch_vec(st, a);
    }
    if (!scratch) return MT_ERR_NULL;
    if (!aligned16(scratch)) return MT_ERR_ALIGN;
    rc = mt_qgemm(stream, x, qweight, nullptr, qzeros, scales, bias, scratch, m, n, k, nr_groups, bits, dtype, workspace, workspace_bytes, flags);
    if (rc == MT_OK) rc = launch_rope_append(st, scratch, cos_table, sin_table, q_out, k_cache, v_cache, m, hq, hkv, d, offset, offset_dev, capacity, table_rows, dtype);
    return rc;
}

size_t mt_attention_workspace_bytes(int m, int hkv, int max_len) {
    if (m < 1 || hkv < 1 || max_len < 1) return 0;
    return attention_workspace_bytes(m, hkv, max_len);
}

int mt_attention_decode(void* stream, const void* q, const void* k_cache, const void* v_cache, void* out, int m, int hq, int hkv, int d,
                        int offset, const int32_t* offset_dev, int max_len, float scale, void* workspace, size_t workspace_bytes, int dtype) {
    if (dtype != MT_F16 && dtype != MT_BF16) return MT_ERR_DTYPE;
    if (m < 0 || hq < 1 || hkv < 1 || offset < 0 || max_len < 1) return MT_ERR_SHAPE;
    if (!offset_dev && offset + m > max_len) return MT_ERR_SHAPE;
    if (m == 0) return MT_OK;
    if (!q || !k_cache || !v_cache || !out) return MT_ERR_NULL;
    if (!aligned16(q) || !aligned16(k_cache) || !aligned16(v_cache) || !aligned16(out)) return MT_ERR_ALIGN;
    if (!workspace) return MT_ERR_WORKSPACE;
    if (!aligned16(workspace)) return MT_ERR_ALIGN;
    int rc = check_device();
    if (rc != MT_OK) return rc;
    return launch_attention_decode(static_cast<cudaStream_t>(stream), q, k_cache, v_cache, out, m, hq, hkv, d, offset, offset_dev, max_len,
                                   scale, workspace, workspace_bytes, dtype);
}

int mt_decode_plan(int m, int n, int k, int nr_groups, int bits, size_t workspace_bytes, int flags) {
    if ((bits != 4 && bits != 8) || m < 1 || n < 1 || k < 1 || nr_groups < 1 || k % nr_groups != 0) return MT_ERR_SHAPE;
    if (check_device() != MT_OK) return MT_ERR_DEVICE;
    QGemmArgs a = {};
    a.m = m; a.n = n; a.k = k; a.groups = nr_groups; a.bits = bits; a.dtype = MT_F16;
    a.workspace = reinterpret_cast<void*>(16); a.workspace_bytes = workspace_bytes; a.flags = flags;   // only tested for null
    if (m > 2) return MT_ERR_UNSUPPORTED;
    return vec_plan(a);
}

size_t mt_allreduce_buffer_bytes(int m_max, int n_max, int world) {
    if (m_max < 1 || n_max < 1 || world < 1 || world > kArMaxWorld) return 0;
    const size_t slot = (((size_t)m_max * n_max * 8) + 255) & ~(size_t)255;   // 8-byte cells {value, epoch}
    return kArDataOffset + 2 * (size_t)world * slot;
}

int mt_w8_pack(void* stream, const int8_t* w, uint32_t* qweight, int n, int k) {
    if (n < 0 || k < 0 || n % 4 != 0 || k % 4 != 0) return MT_ERR_SHAPE;
    if (n == 0 || k == 0) return MT_OK;
    if (!w || !qweight) return MT_ERR_NULL;
    if (!aligned16(w) || !aligned16(qweight)) return MT_ERR_ALIGN;
    int rc = check_device();
    if (rc != MT_OK) return rc;
    return launch_w8_pack(static_cast<cudaStream_t>(stream), w, qweight, n, k);
}

int mt_act_order_perm(void* stream, const int32_t* g_idx, int32_t* perm, int* status, int k, int nr_groups) {
    if (k < 0 || nr_groups < 1 || k % nr_groups != 0) return MT_ERR_SHAPE;
    if (k == 0) return MT_OK;
    if (!g_idx || !perm) return MT_ERR_NULL;
    int rc = check_device();
    if (rc != MT_OK) return rc;
    return launch_act_order_perm(static_cast<cudaStream_t>(stream), g_idx, perm, status, k, nr_groups);
}

int mt_repack_rows(void* stream, const uint32_t* qweight, const int32_t* perm, uint32_t* qweight_out, int n, int k, int bits) {
    if (bits != 4 && bits != 8) return MT_ERR_BITS;
    if (n < 0 || k < 0 || k % (32 / bits) != 0) return MT_ERR_SHAPE;
    if (n == 0 || k == 0) return MT_OK;
    if (!qweight || !perm || !qweight_out) return MT_ERR_NULL;
    if (qweight == qweight_out) return MT_ERR_SHAPE;             // not in place: rows are gathered
    int rc = check_device();
    if (rc != MT_OK) return rc;
    return launch_repack_rows(static_cast<cudaStream_t>(stream), qweight, perm, qweight_out, n, k, bits);
}

int mt_gather_columns(void* stream, const void* x, const int32_t* perm, void* x_out, int m, int k, int dtype) {
    if (dtype != MT_F16 && dtype != MT_BF16) return MT_ERR_DTYPE;
    if (m < 0 || k < 0) return MT_ERR_SHAPE;
    if (m == 0 || k == 0) return MT_OK;
    if (!x || !perm || !x_out) return MT_ERR_NULL;
    if (x == x_out) return MT_ERR_SHAPE;
    int rc = check_device();
    if (rc != MT_OK) return rc;
    return launch_gather_columns(static_cast<cudaStream_t>(stream), x, perm, x_out, m, k);
}

int mt_qgemm_ordered(void* stream, const void* x, const int32_t* x_perm, void* x_scratch, const uint32_t* qweight,
                     const uint32_t* qzeros, const void* scales, const void* bias, void* out,
                     int m, int n, int k, int nr_groups, int bits, int dtype,
                     void* workspace, size_t workspace_bytes, int flags) {
    if (!x_perm) return mt_qgemm(stream, x, qweight, nullptr, qzeros, scales, bias, out, m, n, k, nr_groups, bits, dtype,
                                 workspace, workspace_bytes, flags);
    int rc = validate_gptq(qweight, qzeros, scales, n, k, nr_groups, bits, dtype);
    if (rc != MT_OK) return rc;
    if (m < 0) return MT_ERR_SHAPE;
    if (m == 0 || n == 0) return MT_OK;
    if (k == 0) return MT_ERR_SHAPE;
    if (!x || !out) return MT_ERR_NULL;
    if (!aligned16(x) || !aligned16(out) || !aligned16(x_perm) || (bias && !aligned16(bias))) return MT_ERR_ALIGN;
    if ((k / nr_groups) % (4 * (32 / bits)) != 0) return MT_ERR_SHAPE;
    if (workspace && !aligned16(workspace)) return MT_ERR_ALIGN;
    if ((rc = check_device()) != MT_OK) return rc;
    QGemmArgs a = {};
    a.x = x; a.qweight = qweight; a.qzeros = qzeros; a.scales = scales; a.bias = bias; a.out = out;
    a.m = m; a.n = n; a.k = k; a.groups = nr_groups; a.bits = bits; a.dtype = dtype;
    a.workspace = workspace; a.workspace_bytes = workspace_bytes; a.flags = flags;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool forced_other = (flags & (MT_FLAG_FORCE_SMALL | MT_FLAG_FORCE_TC | MT_FLAG_FORCE_UMMA)) != 0;
    if (m <= 2 && !forced_other && vec_supported(a)) {          // the GEMV gathers while it stages the activations
        a.x_perm = x_perm;
        return launch_vec(st, a);
    }
    if (!x_scratch) return MT_ERR_NULL;
    if (!aligned16(x_scratch)) return MT_ERR_ALIGN;
    if ((rc = launch_gather_columns(st, x, x_perm, x_scratch, m, k)) != MT_OK) return rc;
    return mt_qgemm(stream, x_scratch, qweight, nullptr, qzeros, scales, bias, out, m, n, k, nr_groups, bits, dtype,
                    workspace, workspace_bytes, flags);
}

int mt_w8_perchannel_gemm(void* stream, const void* x, const int8_t* w, const void* scales,
                          const void* bias, void* out, int m, int n, int k, int dtype,
                          void* workspace, size_t workspace_bytes, int flags) {
    if (dtype != MT_F16 && dtype != MT_BF16) return MT_ERR_DTYPE;
    if (m < 0 || n < 0 || k <= 0 || n % 16 != 0 || k % 16 != 0) return MT_ERR_SHAPE;
    if (m == 0 || n == 0) return MT_OK;
    if (!x || !w || !scales || !out) return MT_ERR_NULL;
    if (!aligned16(x) || !aligned16(w) || !aligned16(scales) || !aligned16(out) || (bias && !aligned16(bias)) ||
        (workspace && !aligned16(workspace))) return MT_ERR_ALIGN;
    int rc = check_device();
    if (rc != MT_OK) return rc;
    QGemmArgs a = {};
    a.x = x; a.w8 = w; a.scales = scales; a.bias = bias; a.out = out;
    a.m = m; a.n = n; a.k = k; a.groups = 1; a.bits = 8; a.dtype = dtype;
    a.workspace = workspace; a.workspace_bytes = workspace_bytes; a.flags = flags;
    if (!(flags & MT_FLAG_FORCE_SMALL) && m <= 2 && w8vec_supported(a)) return launch_w8vec(static_cast<cudaStream_t>(stream), a);
    return launch_small_w8(static_cast<cudaStream_t>(stream), a);
}

}  // extern "C"
