// Instantiates the decode GEMV for one bit rate.  Compiled once per K with -DEXL3_GEMV_K=<2..8>.
#include "exl3_gemv_kernel.cuh"

#ifndef EXL3_GEMV_K
#error "compile with -DEXL3_GEMV_K=<2..8>"
#endif

namespace exl3 {

template <int K, int MODE, int FAM, int MB, int XR, int XIN = 0, int EPI = 0>
static int launch_one(const GemvLaunch& l, size_t smem, cudaStream_t st)
{
    // Launched with programmatic stream serialization: its prologue and weight copies overlap the tail of the kernel
    // ahead of it; the kernel itself waits (griddepcontrol.wait) before touching anything that kernel wrote.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(l.grid);
    cfg.blockDim = dim3(GEMV_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cuda_status(cudaLaunchKernelEx(&cfg, gemv_kernel<K, MODE, FAM, MB, XR, XIN, EPI>, l));
}

template <int K, int MODE, int FAM, int MB, int XR, int XIN = 0, int EPI = 0>
static int set_attr(int max_smem)
{
    return cuda_status(cudaFuncSetAttribute(gemv_kernel<K, MODE, FAM, MB, XR, XIN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem));
}

template <int K, int MODE, int FAM>
static int launch_variant(const GemvLaunch& l, size_t smem, cudaStream_t st)
{
    if (l.a.x && l.a.norm_weight) {               // the kernel normalises the residual stream and rotates it
        if (l.a.rows == 1) return launch_one<K, MODE, FAM, 1, 1, 1>(l, smem, st);
        if (l.a.rows == 2) return launch_one<K, MODE, FAM, 1, 2, 1>(l, smem, st);
        return EXL3_ERR_UNSUPPORTED_ROWS;
    }
    if ((l.a.x || l.a.xf_staged) && l.a.res_out) {   // ... and its epilogue adds the residual stream
        if (l.a.rows == 1) return launch_one<K, MODE, FAM, 1, 1, 0, 1>(l, smem, st);
        if (l.a.rows == 2) return launch_one<K, MODE, FAM, 1, 2, 0, 1>(l, smem, st);
        return EXL3_ERR_UNSUPPORTED_ROWS;
    }
    if (l.a.x || l.a.xf_staged) {                 // the kernel rotates the input itself, or stages ready-made fragments
        if (l.a.rows == 1) return launch_one<K, MODE, FAM, 1, 1>(l, smem, st);
        if (l.a.rows == 2) return launch_one<K, MODE, FAM, 1, 2>(l, smem, st);
        return EXL3_ERR_UNSUPPORTED_ROWS;
    }
    return l.a.rows > 8 ? launch_one<K, MODE, FAM, 2, 0>(l, smem, st) : launch_one<K, MODE, FAM, 1, 0>(l, smem, st);
}

template <int K, int MODE, int FAM>
static int set_attr_variants(int max_smem)
{
    int rc = set_attr<K, MODE, FAM, 1, 0>(max_smem);
    if (rc == EXL3_OK) rc = set_attr<K, MODE, FAM, 2, 0>(max_smem);
    if (rc == EXL3_OK) rc = set_attr<K, MODE, FAM, 1, 1>(max_smem);
    if (rc == EXL3_OK) rc = set_attr<K, MODE, FAM, 1, 2>(max_smem);
    if (rc == EXL3_OK) rc = set_attr<K, MODE, FAM, 1, 1, 1>(max_smem);
    if (rc == EXL3_OK) rc = set_attr<K, MODE, FAM, 1, 2, 1>(max_smem);
    if (rc == EXL3_OK) rc = set_attr<K, MODE, FAM, 1, 1, 0, 1>(max_smem);
    if (rc == EXL3_OK) rc = set_attr<K, MODE, FAM, 1, 2, 0, 1>(max_smem);
    return rc;
}

template <>
int launch_gemv_for_k<EXL3_GEMV_K>(const GemvLaunch& l, size_t smem, cudaStream_t st)
{
    constexpr int K = EXL3_GEMV_K;
    const int fam = codebook_family(l.a.codebook);
    if (l.a.mode == GEMV_SPLIT && fam == FAM_HASH) return launch_variant<K, GEMV_SPLIT, FAM_HASH>(l, smem, st);
    if (fam == FAM_HASH) return launch_variant<K, GEMV_PAIRED, FAM_HASH>(l, smem, st);
    return launch_variant<K, GEMV_PAIRED, FAM_MUL1>(l, smem, st);
}

template <>
int gemv_set_attributes_for_k<EXL3_GEMV_K>(int max_smem)
{
    constexpr int K = EXL3_GEMV_K;
    int rc = set_attr_variants<K, GEMV_SPLIT, FAM_HASH>(max_smem);
    if (rc == EXL3_OK) rc = set_attr_variants<K, GEMV_PAIRED, FAM_HASH>(max_smem);
    if (rc == EXL3_OK) rc = set_attr_variants<K, GEMV_PAIRED, FAM_MUL1>(max_smem);
    return rc;
}

}  // namespace exl3
