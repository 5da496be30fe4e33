// Instantiations + launcher of the int8 per-channel streaming kernel.
#include "qgemm_w8.cuh"

namespace mt {

template <typename T, int MT, int WN, int CPT>
static int launch_w8_one(cudaStream_t st, const W8Params& p, dim3 grid, size_t smem) {
    auto kern = qgemm_w8_kernel<T, MT, WN, CPT>;
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

template <typename T>
static int launch_w8_t(cudaStream_t st, const W8Params& p, int mt, int wn, int cpt, dim3 grid, size_t smem) {
#define MT_CASE(M_, W_, C_) if (mt == M_ && wn == W_ && cpt == C_) return launch_w8_one<T, M_, W_, C_>(st, p, grid, smem)
    MT_CASE(1, 2, 16); MT_CASE(1, 4, 16); MT_CASE(2, 2, 16); MT_CASE(2, 4, 16);
    MT_CASE(4, 4, 8); MT_CASE(8, 4, 8);
#undef MT_CASE
    return MT_ERR_UNSUPPORTED;
}

int launch_w8_inst(cudaStream_t st, const W8Params& p, int dtype, int mt, int wn, int cpt, dim3 grid, size_t smem) {
    return dtype == MT_F16 ? launch_w8_t<__half>(st, p, mt, wn, cpt, grid, smem)
                           : launch_w8_t<__nv_bfloat16>(st, p, mt, wn, cpt, grid, smem);
}

}  // namespace mt
