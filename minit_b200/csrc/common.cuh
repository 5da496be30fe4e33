// Shared device helpers for the quantized-linear kernels (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include "../../include/minit_b200.h"
#include "ar_mailbox.cuh"

namespace mt {

// ----------------------------------------------------------------------------------
// 16-bit float traits: register-level (uint32 = two packed elements) arithmetic
// ----------------------------------------------------------------------------------
template <typename T> struct F16x2;

template <> struct F16x2<__half> {
    static constexpr bool kIsBf16 = false;
    static __device__ __forceinline__ uint32_t sub(uint32_t a, uint32_t b) {
        uint32_t d; asm("sub.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d; }
    static __device__ __forceinline__ uint32_t mul(uint32_t a, uint32_t b) {
        uint32_t d; asm("mul.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d; }
    static __device__ __forceinline__ uint32_t fma(uint32_t a, uint32_t b, uint32_t c) {
        uint32_t d; asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c)); return d; }
    static __device__ __forceinline__ float to_float(uint16_t v) { return __half2float(__ushort_as_half(v)); }
    static __device__ __forceinline__ uint16_t from_float(float f) { return __half_as_ushort(__float2half_rn(f)); }
    static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
        __half2 h = __floats2half2_rn(lo, hi); return *reinterpret_cast<uint32_t*>(&h); }
};

template <> struct F16x2<__nv_bfloat16> {
    static constexpr bool kIsBf16 = true;
    static __device__ __forceinline__ uint32_t sub(uint32_t a, uint32_t b) {
        uint32_t d; asm("sub.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d; }
    static __device__ __forceinline__ uint32_t mul(uint32_t a, uint32_t b) {
        uint32_t d; asm("mul.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d; }
    static __device__ __forceinline__ uint32_t fma(uint32_t a, uint32_t b, uint32_t c) {
        uint32_t d; asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c)); return d; }
    static __device__ __forceinline__ float to_float(uint16_t v) { return __uint_as_float(uint32_t(v) << 16); }
    static __device__ __forceinline__ uint16_t from_float(float f) { return __bfloat16_as_ushort(__float2bfloat16_rn(f)); }
    static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
        __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi); return *reinterpret_cast<uint32_t*>(&h); }
};

// silu(g) * u in fp32: the activation of a gated feed-forward (examples/llama3_70b.py:44-45, 127-129)
__device__ __forceinline__ float silu_mul(float g, float u) { return g / (1.f + expf(-g)) * u; }

// (a & b) | c in one LOP3
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d; asm("lop3.b32 %0, %1, %2, %3, 0xea;" : "=r"(d) : "r"(a), "r"(b), "r"(c)); return d;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d; asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel)); return d;
}

// streaming 128-bit global load: weights are read exactly once, keep them out of L1
__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ldg_stream8(const void* p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}
// L2-coherent loads for data another CTA of the same grid has just written
__device__ __forceinline__ float4 ldcg_f4(const float* p) { return __ldcg(reinterpret_cast<const float4*>(p)); }

// f16x2 arithmetic on raw 32-bit registers (round to nearest, subnormals kept: the decode GEMVs multiply
// packed integers as fp16 subnormals)
__device__ __forceinline__ uint32_t hfma2(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d; asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c)); return d; }
__device__ __forceinline__ uint32_t hmul2(uint32_t a, uint32_t b) {
    uint32_t d; asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d; }
__device__ __forceinline__ uint32_t hadd2(uint32_t a, uint32_t b) {
    uint32_t d; asm("add.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d; }

// thread-block cluster barrier and a distributed-shared-memory store into the CTA of rank `cta_rank`
__device__ __forceinline__ void cluster_arrive_relaxed() { asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_arrive_release() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait_acquire() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ void st_cluster_f32(const float* local, unsigned cta_rank, float v) {
    const uint32_t la = (uint32_t)__cvta_generic_to_shared(local);
    uint32_t ra;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(la), "r"(cta_rank));
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(ra), "f"(v) : "memory");
}

__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// m16n8k16, A row-major (16x16), B col-major (16x8), fp32 accumulate
template <typename T>
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    if constexpr (F16x2<T>::kIsBf16) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    } else {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
}

// ----------------------------------------------------------------------------------
// host-side launch plumbing shared by the .cu files
// ----------------------------------------------------------------------------------
// Epilogue of the fused q/k/v linear at decode: rotary embedding of the q and k heads, q to its own tensor, k and v
// straight into the cache (what rope_append_kernel does as a separate launch).  cosv == nullptr: off.
struct RopeArgs {
    const float* cosv; const float* sinv;     // fp32 [table_rows, 64]
    void* q_out;                              // [M, hq, 128] T
    void* k_cache; void* v_cache;             // [capacity, hkv, 128] T
    const int* offset_dev;                    // device int32 or null: overrides offset
    int hq, hkv, offset, capacity, table_rows;
};

// One (even column, odd column) pair of a fused qkv row: rotate (q, k heads) or copy (v heads) and store.
template <typename T>
__device__ __forceinline__ void rope_store_pair(const RopeArgs& r, int off, int tok, int col, float re, float im) {
    using H = F16x2<T>;
    const int head = col >> 7, d = col & 127, pos = off + tok;
    if (head >= r.hq + r.hkv) {
        if (pos < r.capacity) reinterpret_cast<uint32_t*>(r.v_cache)[(((size_t)pos * r.hkv + (head - r.hq - r.hkv)) * 128 + d) >> 1] = H::pack(re, im);
        return;
    }
    const int tp = pos < r.table_rows ? pos : r.table_rows - 1;
    const float cs = __ldg(r.cosv + (size_t)tp * 64 + (d >> 1)), sn = __ldg(r.sinv + (size_t)tp * 64 + (d >> 1));
    const uint32_t o = H::pack(re * cs - im * sn, im * cs + re * sn);
    if (head < r.hq) reinterpret_cast<uint32_t*>(r.q_out)[(((size_t)tok * r.hq + head) * 128 + d) >> 1] = o;
    else if (pos < r.capacity) reinterpret_cast<uint32_t*>(r.k_cache)[(((size_t)pos * r.hkv + (head - r.hq)) * 128 + d) >> 1] = o;
}

struct QGemmArgs {
    const void* x;            // [M,K] T
    const uint32_t* qweight;  // [K/pack, N]
    const int32_t* g_idx;     // [K] or null
    const uint32_t* qzeros;   // [G, N/pack] or null
    const void* scales;       // [G,N] T (per-channel: [N])
    const void* bias;         // [N] T or null
    void* out;                // [M,N] T
    const int8_t* w8;         // per-channel path: [K,N] int8
    const int32_t* x_perm;    // [K] or null: rows of qweight were sorted by group (act-order), read x through this permutation
    int m, n, k, groups, bits, dtype;
    void* workspace;
    size_t workspace_bytes;
    int flags;
    // fused all-reduce (row-parallel): device array of the ranks' symmetric buffers, or null
    unsigned char* const* ar_peers;
    int ar_rank, ar_world;
    size_t ar_bytes;          // size of one symmetric buffer
    // fused epilogues (decode GEMV only; other kernels are followed by an elementwise launch)
    const void* residual;     // [M,N] T or null: out = residual + (x @ W + bias), added after the all-reduce
    int epilogue;             // MT_EPILOGUE_*: SWIGLU = out[M,N/2] from the gate / up interleaved layout
    const RopeArgs* rope;     // non-null: the output row is a fused q/k/v row, rotated and scattered (out unused)
};

// workspace layout: [0, kCounterBytes) tile counters (the last word is the error word) (kept zero between launches),
// then fp32 split-K partials.
constexpr size_t kCounterBytes = 16384;           // 4096 tile counters
constexpr int kMaxTiles = int(kCounterBytes / 4);

// all-reduce parameters of a launch (world 1 when the call has no peers)
inline ArParams make_ar_params(const QGemmArgs& a) {
    ArParams r;
    r.peers = a.ar_peers; r.rank = a.ar_rank; r.world = a.ar_peers ? a.ar_world : 1;
    r.err = a.workspace ? static_cast<unsigned*>(a.workspace) + (kMaxTiles - 1) : nullptr;
    r.slot_bytes = (a.ar_peers && a.ar_world > 0) ? ((a.ar_bytes - kArDataOffset) / (2 * (size_t)a.ar_world)) & ~(size_t)255 : 0;
    r.spin_limit = (a.flags & MT_FLAG_AR_SHORT_WAIT) ? (1 << 12) : (1 << 22);
    // two-shot exchange (only the kernels that exchange one value at a time implement it: the integer mid-batch kernel): by
    // flag only.  Measured on four ranks at 32 rows it loses to the one-shot form (19.1 against 18.3 ms per step): the
    // exchange is bound by its latency there, not by its bytes, and two-shot has two NVLink crossings in a row.
    r.two_shot = ((a.flags & MT_FLAG_AR_TWO_SHOT) && !(a.flags & MT_FLAG_AR_ONE_SHOT) && r.world > 1 && a.m >= 3) ? 1 : 0;
    r.cols_per_owner = r.world > 0 ? (a.n + r.world - 1) / r.world : a.n;
    if (r.cols_per_owner < 1) r.cols_per_owner = 1;
    return r;
}

int launch_dequant(cudaStream_t st, const uint32_t* qweight, const int32_t* g_idx, const uint32_t* qzeros,
                   const void* scales, void* w_out, int n, int k, int groups, int bits, int dtype);
int launch_dequant_unpacked(cudaStream_t st, const uint8_t* q, const int32_t* g_idx, const uint8_t* z, const void* scales,
                            void* w_out, int n, int k, int groups, int dtype);
int launch_w8_pack(cudaStream_t st, const int8_t* w, uint32_t* out, int n, int k);
int launch_act_order_perm(cudaStream_t st, const int32_t* g_idx, int32_t* perm, int* status, int k, int groups);
int launch_repack_rows(cudaStream_t st, const uint32_t* qw, const int32_t* perm, uint32_t* out, int n, int k, int bits);
int launch_gather_columns(cudaStream_t st, const void* x, const int32_t* perm, void* out, int m, int k);
int launch_unpack(cudaStream_t st, const uint32_t* packed, uint8_t* out, int rows, int cols, int bits, int axis);
int launch_small(cudaStream_t st, const QGemmArgs& a);          // GPTQ layout, M <= 64 per launch
int launch_small_w8(cudaStream_t st, const QGemmArgs& a);       // int8 [K,N] per-channel, M <= 64 per launch
int launch_w8vec(cudaStream_t st, const QGemmArgs& a);          // int8 [K,N] per-channel, CUDA-core GEMV, M <= 2, N % 256 == 0
bool w8vec_supported(const QGemmArgs& a);
int launch_vec(cudaStream_t st, const QGemmArgs& a);            // CUDA-core decode GEMV, M <= 2, contiguous groups
int launch_vec_chain(cudaStream_t st, const QGemmArgs* list, int count);   // several such linears in one resident launch
bool vec_supported(const QGemmArgs& a);
int vec_plan(const QGemmArgs& a);                               // > 0 split-K factor, 0 stream-K, < 0 MT_ERR_*
int launch_interleave_gate_up(cudaStream_t st, const uint32_t* qw_g, const uint32_t* qw_u, const uint32_t* qz_g, const uint32_t* qz_u,
                              const void* s_g, const void* s_u, const void* b_g, const void* b_u,
                              uint32_t* qw_out, uint32_t* qz_out, void* s_out, void* b_out, int half, int k, int groups, int bits);
int launch_swiglu_interleaved(cudaStream_t st, const void* in, void* out, int m, int n, int dtype);   // [M,N] interleaved -> [M,N/2]
int launch_add_residual(cudaStream_t st, void* io, const void* res, int m, int n, int dtype);        // io += res
int launch_rms_norm(cudaStream_t st, const void* x, const void* w, void* out, int rows, int h, float eps, int dtype);
int launch_rope_append(cudaStream_t st, const void* qkv, const float* cosv, const float* sinv, void* q_out, void* k_cache, void* v_cache,
                       int m, int hq, int hkv, int d, int offset, const int* offset_dev, int capacity, int table_rows, int dtype);
int launch_attention_rows(cudaStream_t st, const void* q, const void* k_cache, const void* v_cache, void* out, const int* offsets,
                          int batch, int m, int hq, int hkv, int d, int offset, int capacity, float scale, int dtype);
size_t attention_workspace_bytes(int m, int hkv, int max_len);
int launch_attention_decode(cudaStream_t st, const void* q, const void* k_cache, const void* v_cache, void* out,
                            int m, int hq, int hkv, int d, int offset, const int* offset_dev, int max_len, float scale,
                            void* workspace, size_t workspace_bytes, int dtype);
int launch_umma(cudaStream_t st, const QGemmArgs& a);           // tcgen05 with all-warp dequant, 2 < M <= 192, contiguous groups
bool umma_supported(const QGemmArgs& a);
size_t umma_workspace_bytes(int m, int n, int k);
int launch_mid(cudaStream_t st, const QGemmArgs& a);            // integer tensor-core kernel, 2 < M (passes of 64), contiguous groups of a multiple of 128
bool mid_supported(const QGemmArgs& a);
size_t mid_workspace_bytes(int m, int n, int k);
int launch_tc(cudaStream_t st, const QGemmArgs& a);             // tcgen05 path (any M), GPTQ layout without g_idx
bool tc_supported(const QGemmArgs& a);
size_t tcx_workspace_bytes(int m, int n, int k);     // fp32 partial tiles of the prefill kernel's split last wave
bool tcx_rows_supported(const QGemmArgs& a);          // up to 192 rows: one row of tiles of the tensor-memory-A prefill kernel, cut along K
size_t tcx_rows_workspace_bytes(int m, int n, int k);
int launch_tcx_rows(cudaStream_t st, const QGemmArgs& a);
bool tc_tmem_a_preferred(int m, int n, int bits);   // 65..128 rows: the tensor-memory-A prefill tile beats the mid-batch kernel

}  // namespace mt
