// MoE layer pieces around the grouped GEMV (sm_100a): routing alignment, per-slot input rotations, SiLU-gated
// rotation for the down projection, router-weighted combine.  One MoE layer is
//   align -> had_in (gather, per-expert suh, gate and up) -> grouped GEMV gate|up -> glu_had_in -> grouped GEMV down -> combine
// the five-launch structure of cuda/src/sglang_exl3/kernels/marlin_moe.py:272-294 of 0xSero/trellis-serve, whose kernels
// are cuda/csrc/exl3_marlin_moe.cu:210-292 (per-slot transforms, combine) and :542-594 (decode-size align).
#include "exl3_moe_kernel.cuh"

namespace exl3 {

// ------------------------------------------------------------------------------------------------ align

// One CTA.  Slots (token, k) are grouped by expert into blocks of `block` rows: sorted_ids holds the slot of every
// row (numel = padding), expert_ids the expert of every block, num_post the padded row count.  Ids outside
// [0, E) are dropped.  The order of slots inside an expert is not specified (rows are independent).
// With expert_map (int [E_global]: global id -> id in [0, E), or -1) the ids are translated first, so one class of a
// mixed-bitrate expert set gets the blocks of its own slots only, with local expert ids.
__device__ __forceinline__ int moe_mapped_id(const int* topk_ids, int i, const int* expert_map, int E_global)
{
    const int e = topk_ids[i];
    if (!expert_map) return e;
    return (e >= 0 && e < E_global) ? expert_map[e] : -1;
}

__global__ void moe_align_kernel(const int* __restrict__ topk_ids, int numel, int E, int block, int cap, int* __restrict__ sorted_ids,
                                 int* __restrict__ expert_ids, int* __restrict__ num_post, const int* __restrict__ expert_map,
                                 int E_global)
{
    ptx::grid_launch_dependents();
    ptx::grid_dependency_wait();
    extern __shared__ int sh[];
    int* count = sh;              // [E]
    int* offset = sh + E;         // [E + 1]
    int* fill = sh + 2 * E + 1;   // [E]
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        count[e] = 0;
        fill[e] = 0;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < numel; i += blockDim.x) {
        const int e = moe_mapped_id(topk_ids, i, expert_map, E_global);
        if (e >= 0 && e < E) atomicAdd(&count[e], 1);
    }
    __syncthreads();
    // Exclusive prefix sum of the padded counts: warp scans by shuffle, warp totals through shared memory; experts are
    // taken in chunks of blockDim.x with a running carry.
    __shared__ int warp_total[32];
    __shared__ int carry_sh;
    if (threadIdx.x == 0) carry_sh = 0;
    __syncthreads();
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int e0 = 0; e0 < E; e0 += blockDim.x) {
        const int e = e0 + threadIdx.x;
        const int padded = e < E ? (count[e] + block - 1) / block * block : 0;
        int incl = padded;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int up = __shfl_up_sync(0xFFFFFFFFu, incl, d);
            if (lane >= d) incl += up;
        }
        if (lane == 31) warp_total[wid] = incl;
        __syncthreads();
        if (wid == 0) {
            int t = lane < nwarps ? warp_total[lane] : 0;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int up = __shfl_up_sync(0xFFFFFFFFu, t, d);
                if (lane >= d) t += up;
            }
            warp_total[lane] = t;                      // inclusive totals of the warps
        }
        __syncthreads();
        const int base = carry_sh + (wid > 0 ? warp_total[wid - 1] : 0);
        if (e < E) offset[e] = base + incl - padded;
        __syncthreads();
        if (threadIdx.x == blockDim.x - 1) carry_sh = base + incl;
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        offset[E] = carry_sh;
        *num_post = carry_sh;
    }
    __syncthreads();
    const int total = offset[E];
    for (int i = threadIdx.x; i < cap; i += blockDim.x) sorted_ids[i] = numel;
    for (int e = threadIdx.x; e < E; e += blockDim.x)
        for (int r = offset[e]; r < offset[e + 1]; r += block) expert_ids[r / block] = e;
    for (int i = total / block + threadIdx.x; i < cap / block; i += blockDim.x) expert_ids[i] = -1;
    __syncthreads();
    for (int i = threadIdx.x; i < numel; i += blockDim.x) {
        const int e = moe_mapped_id(topk_ids, i, expert_map, E_global);
        if (e >= 0 && e < E) sorted_ids[offset[e] + atomicAdd(&fill[e], 1)] = i;
    }
}

// ------------------------------------------------------------------------------------------------ fragments

template <int MODE>
__device__ __forceinline__ void store_fragments(uint32_t* out, long long elem_base, int lane, const __half (&h)[4])
{
    // lane holds rows r = 4*(lane&3) + e of 16-row tile lane/4; element = ((kt * 8 + row) * 4 + q), FW words each
    constexpr int FW = gemv_frag_words(MODE);
    const int rbase = 4 * (lane & 3);
    if constexpr (MODE == GEMV_SPLIT) {
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int r = rbase + e, q = (r & 7) >> 1, slot = (r & 1) + 2 * (r >> 3);
            const uint32_t hv = __half_as_ushort(h[e]);
            out[(elem_base + q) * FW + slot] = hv | (hv << 16);
        }
    } else {
#pragma unroll
        for (int e = 0; e < 4; e += 2) {
            const int r = rbase + e, q = (r & 7) >> 1, slot = r >> 3;
            out[(elem_base + q) * FW + slot] = (uint32_t)__half_as_ushort(h[e]) | ((uint32_t)__half_as_ushort(h[e + 1]) << 16);
        }
    }
}

// xf[shard][position p][k tile][q] = fragments of Had128(fp16(x[token(p)]) * suh[expert(p), shard]); zero rows for padding.
// One warp per (shard, p, 128-block).  Positions at or beyond num_post are left untouched.
template <int MODE>
__global__ void moe_had_in_kernel(const void* __restrict__ x, int x_bf16, const __half* __restrict__ suh, int shards, int hidden, int top_k,
                                  int numel, int cap, const int* __restrict__ sorted_ids, const int* __restrict__ expert_ids,
                                  const int* __restrict__ num_post, uint32_t* __restrict__ xf)
{
    ptx::grid_launch_dependents();
    ptx::grid_dependency_wait();
    const int lane = threadIdx.x & 31;
    const int kgs = hidden >> 7, KT = hidden >> 4;
    const long long item = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (long long)shards * cap * kgs) return;
    const int kg = (int)(item % kgs);
    const int p = (int)((item / kgs) % cap);
    const int s = (int)(item / ((long long)kgs * cap));
    if (p >= *num_post) return;
    const int slot = sorted_ids[p];
    const int b = p / MOE_BLOCK_ROWS, row = p % MOE_BLOCK_ROWS;
    __half h[4];
    if (slot < 0 || slot >= numel) {
#pragma unroll
        for (int e = 0; e < 4; e++) h[e] = __ushort_as_half(0);
    } else {
        const int token = slot / top_k, ex = expert_ids[b];
        float v[4];
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int col = kg * 128 + 4 * lane + e;
            float xv = x_bf16 ? __half2float(__float2half_rn(__bfloat162float(reinterpret_cast<const __nv_bfloat16*>(x)[(long long)token * hidden + col])))
                              : __half2float(reinterpret_cast<const __half*>(x)[(long long)token * hidden + col]);
            v[e] = xv * __half2float(suh[((long long)ex * shards + s) * hidden + col]);
        }
        fwht128(v[0], v[1], v[2], v[3], lane);
#pragma unroll
        for (int e = 0; e < 4; e++) h[e] = __float2half_rn(v[e] * HAD_SCALE);
    }
    const int kt = kg * 8 + (lane >> 2);
    const long long elem_base = (((long long)s * (cap / MOE_BLOCK_ROWS) + b) * KT + kt) * 32 + row * 4;
    store_fragments<MODE>(xf, elem_base, lane, h);
}

// xd fragments = Had128( fp16( silu(gate) * up ) * suh2[expert] ) per position; gu is [slots][2*inter] fp16.
template <int MODE>
__global__ void moe_glu_had_in_kernel(const __half* __restrict__ gu, const __half* __restrict__ suh2, int inter, int numel, int cap,
                                      const int* __restrict__ sorted_ids, const int* __restrict__ expert_ids,
                                      const int* __restrict__ num_post, uint32_t* __restrict__ xf)
{
    ptx::grid_launch_dependents();
    ptx::grid_dependency_wait();
    const int lane = threadIdx.x & 31;
    const int kgs = inter >> 7, KT = inter >> 4;
    const long long item = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (long long)cap * kgs) return;
    const int kg = (int)(item % kgs);
    const int p = (int)(item / kgs);
    if (p >= *num_post) return;
    const int slot = sorted_ids[p];
    const int b = p / MOE_BLOCK_ROWS, row = p % MOE_BLOCK_ROWS;
    __half h[4];
    if (slot < 0 || slot >= numel) {
#pragma unroll
        for (int e = 0; e < 4; e++) h[e] = __ushort_as_half(0);
    } else {
        const int ex = expert_ids[b];
        float v[4];
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int col = kg * 128 + 4 * lane + e;
            const float gv = __half2float(gu[(long long)slot * 2 * inter + col]);
            const float uv = __half2float(gu[(long long)slot * 2 * inter + inter + col]);
            const float act = __half2float(__float2half_rn(gv / (1.0f + __expf(-gv)) * uv));
            v[e] = act * __half2float(suh2[(long long)ex * inter + col]);
        }
        fwht128(v[0], v[1], v[2], v[3], lane);
#pragma unroll
        for (int e = 0; e < 4; e++) h[e] = __float2half_rn(v[e] * HAD_SCALE);
    }
    const int kt = kg * 8 + (lane >> 2);
    const long long elem_base = (((long long)b) * KT + kt) * 32 + row * 4;
    store_fragments<MODE>(xf, elem_base, lane, h);
}

// y[t, :] = sum_j w[t, j] * yd[t*top_k + j, :] in fp32, slot order, one rounding; ids outside [0, E) are skipped.
__global__ void moe_combine_kernel(const __half* __restrict__ yd, const float* __restrict__ w, const int* __restrict__ topk_ids, int tokens,
                                   int top_k, int hidden, int E, void* __restrict__ y, int y_bf16)
{
    ptx::grid_launch_dependents();
    ptx::grid_dependency_wait();
    const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;       // one thread per (token, 2 columns)
    const int half_h = hidden >> 1;
    if (idx >= (long long)tokens * half_h) return;
    const int t = (int)(idx / half_h), c = (int)(idx % half_h) * 2;
    float a0 = 0.f, a1 = 0.f;
    for (int j = 0; j < top_k; j++) {
        const int e = topk_ids[t * top_k + j];
        if (e < 0 || e >= E) continue;
        const __half2 v = *reinterpret_cast<const __half2*>(yd + ((long long)t * top_k + j) * hidden + c);
        const float wt = w[t * top_k + j];
        a0 += wt * __low2float(v);
        a1 += wt * __high2float(v);
    }
    const __half2 h = __floats2half2_rn(a0, a1);
    if (y_bf16) {
        reinterpret_cast<__nv_bfloat162*>(y)[idx] = __floats2bfloat162_rn(__low2float(h), __high2float(h));
    } else {
        reinterpret_cast<__half2*>(y)[idx] = h;
    }
}

// ------------------------------------------------------------------------------------------------ launchers

template <int K>
int launch_moe_gemm_for_k(const MoeGemmLaunch& l, int mode, int family, int grid, size_t smem, cudaStream_t st);
template <int K>
int moe_set_attributes_for_k(int max_smem);

int moe_init_device()
{
    const DeviceInfo* d = current_device_info();
    if (!d) return EXL3_ERR_NOT_INITIALISED;
    int rc = moe_set_attributes_for_k<2>(d->max_smem_optin);
    if (rc == EXL3_OK) rc = moe_set_attributes_for_k<3>(d->max_smem_optin);
    if (rc == EXL3_OK) rc = moe_set_attributes_for_k<4>(d->max_smem_optin);
    if (rc == EXL3_OK) rc = moe_set_attributes_for_k<5>(d->max_smem_optin);
    if (rc == EXL3_OK) rc = moe_set_attributes_for_k<6>(d->max_smem_optin);
    if (rc == EXL3_OK) rc = moe_set_attributes_for_k<7>(d->max_smem_optin);
    if (rc == EXL3_OK) rc = moe_set_attributes_for_k<8>(d->max_smem_optin);
    return rc;
}

static inline unsigned blocks_for(long long items, int per_block) { return (unsigned)((items + per_block - 1) / per_block); }

int launch_moe_align(const int* topk_ids, int numel, int E, int block, int cap, int* sorted_ids, int* expert_ids, int* num_post,
                     const int* expert_map, int E_global, cudaStream_t st)
{
    return launch_chained(moe_align_kernel, dim3(1), dim3(1024), (3 * E + 1) * sizeof(int), st, topk_ids, numel, E, block, cap, sorted_ids, expert_ids,
                          num_post, expert_map, E_global);
}

int launch_moe_had_in(const void* x, int x_bf16, const __half* suh, int shards, int hidden, int top_k, int numel, int cap,
                      const int* sorted_ids, const int* expert_ids, const int* num_post, uint32_t* xf, int mode, cudaStream_t st)
{
    const long long items = (long long)shards * cap * (hidden / 128);
    if (items == 0) return EXL3_OK;
    auto kernel = mode == GEMV_SPLIT ? moe_had_in_kernel<GEMV_SPLIT> : moe_had_in_kernel<GEMV_PAIRED>;
    return launch_chained(kernel, dim3(blocks_for(items, 8)), dim3(256), 0, st, x, x_bf16, suh, shards, hidden, top_k, numel, cap, sorted_ids,
                          expert_ids, num_post, xf);
}

int launch_moe_glu_had_in(const __half* gu, const __half* suh2, int inter, int numel, int cap, const int* sorted_ids,
                          const int* expert_ids, const int* num_post, uint32_t* xf, int mode, cudaStream_t st)
{
    const long long items = (long long)cap * (inter / 128);
    if (items == 0) return EXL3_OK;
    auto kernel = mode == GEMV_SPLIT ? moe_glu_had_in_kernel<GEMV_SPLIT> : moe_glu_had_in_kernel<GEMV_PAIRED>;
    return launch_chained(kernel, dim3(blocks_for(items, 8)), dim3(256), 0, st, gu, suh2, inter, numel, cap, sorted_ids, expert_ids, num_post, xf);
}

int launch_moe_combine(const __half* yd, const float* w, const int* topk_ids, int tokens, int top_k, int hidden, int E, void* y,
                       int y_bf16, cudaStream_t st)
{
    const long long items = (long long)tokens * (hidden / 2);
    if (items == 0) return EXL3_OK;
    return launch_chained(moe_combine_kernel, dim3(blocks_for(items, 256)), dim3(256), 0, st, yd, w, topk_ids, tokens, top_k, hidden, E, y, y_bf16);
}

int launch_moe_gemm(MoeGemmLaunch l, int K, int codebook, int mode, cudaStream_t st)
{
    const DeviceInfo* d = current_device_info();
    if (!d) return EXL3_ERR_NOT_INITIALISED;
    int grid = d->sm_count * MOE_CTAS_PER_SM;
    if (grid > GEMV_MAX_GRID) grid = GEMV_MAX_GRID;
    const uint32_t unit_bytes = 2048u * K;
    const uint32_t frag_bytes = 8u * MOE_BLOCK_ROWS * 4u * (uint32_t)gemv_frag_words(mode) * 4u;   // a unit's fragments ride with its weights
    int ups = (int)((24u * 1024u + unit_bytes - 1) / unit_bytes);
    const int UB = l.KG * l.NB;
    if (ups > UB) ups = UB;
    l.units_per_stage = ups;
    l.stage_stride = (uint32_t)ups * (unit_bytes + frag_bytes);
    const size_t fixed = 256 + GEMV_MAX_ROWS * 128 * 4;
    int stages = (int)((96u * 1024u) / l.stage_stride);
    const int cap = (int)((d->max_smem_optin / MOE_CTAS_PER_SM - 2048 - fixed) / l.stage_stride);
    if (stages > cap) stages = cap;
    if (stages > MOE_MAX_STAGES) stages = MOE_MAX_STAGES;
    if (stages < 2) return EXL3_ERR_UNSUPPORTED_ROWS;
    l.stages = stages;
    const CodebookConst c = codebook_const(codebook);
    l.mul = c.mul;
    l.add = c.add;
    l.pw = make_pow2();
    const size_t smem = fixed + (size_t)stages * l.stage_stride;
    const int fam = codebook_family(codebook);
    switch (K) {
        case 2: return launch_moe_gemm_for_k<2>(l, mode, fam, grid, smem, st);
        case 3: return launch_moe_gemm_for_k<3>(l, mode, fam, grid, smem, st);
        case 4: return launch_moe_gemm_for_k<4>(l, mode, fam, grid, smem, st);
        case 5: return launch_moe_gemm_for_k<5>(l, mode, fam, grid, smem, st);
        case 6: return launch_moe_gemm_for_k<6>(l, mode, fam, grid, smem, st);
        case 7: return launch_moe_gemm_for_k<7>(l, mode, fam, grid, smem, st);
        case 8: return launch_moe_gemm_for_k<8>(l, mode, fam, grid, smem, st);
    }
    return EXL3_ERR_UNSUPPORTED_K;
}

}  // namespace exl3
