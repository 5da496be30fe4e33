// Instantiations of the GPTQ streaming kernel for one (bits, dtype) pair; compiled once per
// pair with -DMT_INST_BITS={4,8} -DMT_INST_BF16={0,1} so the four pairs build in parallel.
#include "qgemm_small.cuh"

#ifndef MT_INST_BITS
#error "compile with -DMT_INST_BITS=4|8 -DMT_INST_BF16=0|1"
#endif

namespace mt {

#if MT_INST_BF16
using InstT = __nv_bfloat16;
#define MT_INST_NAME2(b) launch_small_i##b##_bf16
#else
using InstT = __half;
#define MT_INST_NAME2(b) launch_small_i##b##_f16
#endif
#define MT_INST_NAME1(b) MT_INST_NAME2(b)
#define MT_INST_NAME MT_INST_NAME1(MT_INST_BITS)

template <int MT, int WN, int GPC, bool ACT>
static int launch_one(cudaStream_t st, const SmallParams& p, dim3 grid, size_t smem) {
    auto kern = qgemm_small_kernel<MT_INST_BITS, InstT, MT, WN, GPC, ACT>;
    if (smem > 48 * 1024) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            cudaGetLastError();
            return MT_ERR_TOO_LARGE;
        }
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = dim3(WN * 32); cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = p.pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, p) == cudaSuccess ? MT_OK : MT_ERR_CUDA;
}

template <int MT, int WN>
static int launch_gpc(cudaStream_t st, const SmallParams& p, dim3 grid, size_t smem, int gpc, bool act) {
    if (act) return launch_one<MT, WN, 1, true>(st, p, grid, smem);
    switch (gpc) {
        case 1: return launch_one<MT, WN, 1, false>(st, p, grid, smem);
        case 2: return launch_one<MT, WN, 2, false>(st, p, grid, smem);
        case 8: return launch_one<MT, WN, 8, false>(st, p, grid, smem);
    }
    return MT_ERR_UNSUPPORTED;
}

// mt: batch tiles of 8 rows (1,2,4,8); wn: warps per CTA (2,4,8; 8 only for mt == 8)
int MT_INST_NAME(cudaStream_t st, const SmallParams& p, int mt, int wn, int gpc, bool act, dim3 grid, size_t smem) {
#define MT_CASE(M_, W_) if (mt == M_ && wn == W_) return launch_gpc<M_, W_>(st, p, grid, smem, gpc, act)
    MT_CASE(1, 8); MT_CASE(1, 4); MT_CASE(1, 2);
    MT_CASE(2, 8); MT_CASE(2, 4); MT_CASE(2, 2);
    MT_CASE(4, 8); MT_CASE(4, 4);
    MT_CASE(8, 8);
#undef MT_CASE
    return MT_ERR_UNSUPPORTED;
}

}  // namespace mt
