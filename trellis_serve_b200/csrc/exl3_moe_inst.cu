// Instantiates the grouped MoE GEMV for one bit rate.  Compiled once per K with -DEXL3_MOE_K=<2..8>.
#include "exl3_moe_kernel.cuh"

#ifndef EXL3_MOE_K
#error "compile with -DEXL3_MOE_K=<2..8>"
#endif

namespace exl3 {

template <int K>
int launch_moe_gemm_for_k(const MoeGemmLaunch& l, int mode, int family, int grid, size_t smem, cudaStream_t st);
template <int K>
int moe_set_attributes_for_k(int max_smem);

template <>
int launch_moe_gemm_for_k<EXL3_MOE_K>(const MoeGemmLaunch& l, int mode, int family, int grid, size_t smem, cudaStream_t st)
{
    constexpr int K = EXL3_MOE_K;
    if (family == FAM_MUL1) return launch_chained(moe_gemm_kernel<K, GEMV_PAIRED, FAM_MUL1>, dim3(grid), dim3(MOE_THREADS), smem, st, l);
    if (mode == GEMV_SPLIT) return launch_chained(moe_gemm_kernel<K, GEMV_SPLIT, FAM_HASH>, dim3(grid), dim3(MOE_THREADS), smem, st, l);
    return launch_chained(moe_gemm_kernel<K, GEMV_PAIRED, FAM_HASH>, dim3(grid), dim3(MOE_THREADS), smem, st, l);
}

template <>
int moe_set_attributes_for_k<EXL3_MOE_K>(int max_smem)
{
    constexpr int K = EXL3_MOE_K;
    int rc = cuda_status(cudaFuncSetAttribute(moe_gemm_kernel<K, GEMV_SPLIT, FAM_HASH>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem));
    if (rc == EXL3_OK) rc = cuda_status(cudaFuncSetAttribute(moe_gemm_kernel<K, GEMV_PAIRED, FAM_HASH>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem));
    if (rc == EXL3_OK) rc = cuda_status(cudaFuncSetAttribute(moe_gemm_kernel<K, GEMV_PAIRED, FAM_MUL1>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem));
    return rc;
}

}  // namespace exl3
