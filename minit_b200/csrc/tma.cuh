// mbarrier / TMA (cp.async.bulk.tensor) wrappers and the host-side tensor-map encoder, shared
// by the kernels that stage operands with TMA.  None of the loads carries a cluster qualifier
// beyond the destination state space: every CTA fetches its own tiles.
#pragma once
#include <cuda.h>
#include "common.cuh"

namespace mt {

// ---- PTX wrappers ----------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.b32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// One non-blocking look at a barrier.  The answer takes a few hundred cycles to come back whatever it is, so a thread that
// knows which barrier it will need next can ask early and read the answer behind other work.
__device__ __forceinline__ uint32_t mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.b32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok;
}
// Bounded wait: spins, then backs off with nanosleep; gives up after roughly a second.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    for (int i = 0; i < 4096; ++i) if (mbar_try_wait(bar, parity)) return true;
    for (int i = 0; i < (1 << 22); ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        __nanosleep(128);
    }
    *abort_flag = 1;
    return false;
}
// Bounded wait that SLEEPS between looks.  A warp that spins on try_wait takes issue slots from the warps of its
// scheduler and keeps the barrier unit busy; roles that wait long by design (an epilogue waiting for a whole tile, a
// producer that runs stages ahead) look every NS nanoseconds instead, and roles on the critical path every few tens.
template <int NS>
__device__ __forceinline__ bool mbar_wait_sleep(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    constexpr int LIMIT = NS >= 256 ? (1 << 22) : (1 << 25);          // about a second either way
    for (int i = 0; i < LIMIT; ++i) {
        if (mbar_test(bar, parity)) return true;
        if ((i & 63) == 63 && *abort_flag) return false;
        __nanosleep(NS);
    }
    *abort_flag = 1;
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
// cuTensorMapEncodeTiled through the runtime's driver entry point lookup (no link-time libcuda dependency)
EncodeTiledFn get_tensor_map_encoder();

}  // namespace mt
