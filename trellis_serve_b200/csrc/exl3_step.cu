// Caller side of the fused groups in a decode step: the element-wise kernels that sit between the EXL3 linears write the
// NEXT linear's rotated input as tensor-core fragments, once, so that the decode GEMV neither needs a rotation launch of
// its own nor rotates inside every CTA:
//
//   rmsnorm_rotate_kernel   residual += x;  normed = rmsnorm(residual) * weight;  fragments = Had128(fp16(normed) * suh[s])
//   silu_mul_rotate_kernel  act = silu(gate) * up;                                fragments = Had128(fp16(act) * suh)
//
// This is the residual / normalisation fusion around the reference's fused launch (cuda/csrc/exl3_marlin.cu:507-527 is the
// group launch; its engine runs residual add, RMSNorm and the activation as separate kernels ahead of had_in,
// cuda/csrc/exl3_marlin.cu:283-290).  The fragments are those of the stand-alone rotation kernel, bit for bit.
#include "exl3_internal.h"
#include "exl3_ptx.cuh"

namespace exl3 {

constexpr int STEP_THREADS = 1024;
constexpr int STEP_MAX_BLOCKS_PER_WARP = 8;            // 128-column blocks one warp keeps in registers: k <= 32768

__device__ __forceinline__ float to_f32(const void* p, long long i, bool bf16)
{
    return bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]) : __half2float(reinterpret_cast<const __half*>(p)[i]);
}

// Rounds to the activation type and returns the rounded value.
__device__ __forceinline__ float round_act(float v, bool bf16) { return bf16 ? __bfloat162float(__float2bfloat16_rn(v)) : __half2float(__float2half_rn(v)); }

__device__ __forceinline__ void store_act4(void* p, long long i, const float (&v)[4], bool bf16)
{
    if (bf16) {
        __nv_bfloat16 b[4];
#pragma unroll
        for (int e = 0; e < 4; e++) b[e] = __float2bfloat16_rn(v[e]);
        *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p) + i) = *reinterpret_cast<uint2*>(b);
    } else {
        __half h[4];
#pragma unroll
        for (int e = 0; e < 4; e++) h[e] = __float2half_rn(v[e]);
        *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(p) + i) = *reinterpret_cast<uint2*>(h);
    }
}

// One warp, one (shard, row, 128 block): a[e] are activation values already rounded to the activation type.  They are
// converted to fp16 as the rotation kernel does, scaled by suh, rotated and stored as fragments.
// mode 1: split-pair fragments (4 words per lane q), mode 2: paired (2 words); layouts of had_in_kernel.
__device__ __forceinline__ void rotate_store(const float (&a)[4], const __half* suh_blk, uint32_t* xf, int mode, int s, int kts, int rows,
                                             int row, int kg, int lane)
{
    float v[4];
    const uint2 sw = *reinterpret_cast<const uint2*>(suh_blk + 4 * lane);
    const __half2 s01 = *reinterpret_cast<const __half2*>(&sw.x), s23 = *reinterpret_cast<const __half2*>(&sw.y);
    v[0] = __half2float(__float2half_rn(a[0])) * __low2float(s01);
    v[1] = __half2float(__float2half_rn(a[1])) * __high2float(s01);
    v[2] = __half2float(__float2half_rn(a[2])) * __low2float(s23);
    v[3] = __half2float(__float2half_rn(a[3])) * __high2float(s23);
    fwht128(v[0], v[1], v[2], v[3], lane);
    uint32_t hv[4];
#pragma unroll
    for (int e = 0; e < 4; e++) hv[e] = __half_as_ushort(__float2half_rn(v[e] * HAD_SCALE));
    const int kt = kg * 8 + (lane >> 2);
    const int rbase = 4 * (lane & 3);
    if (mode == 1) {
        uint32_t* o = xf + (((long long)s * kts + kt) * rows + row) * 16;
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int r = rbase + e;
            o[((r & 7) >> 1) * 4 + (r & 1) + 2 * (r >> 3)] = hv[e] | (hv[e] << 16);
        }
    } else {
        uint32_t* o = xf + (((long long)s * kts + kt) * rows + row) * 8;
#pragma unroll
        for (int e = 0; e < 4; e += 2) {
            const int r = rbase + e;
            o[((r & 7) >> 1) * 2 + (r >> 3)] = hv[e] | (hv[e + 1] << 16);
        }
    }
}

// grid = rows, block = STEP_THREADS.  x [rows, k]; residual [rows, k] or null (in / out); weight [k]; suh [shards, k];
// normed [rows, k] or null.
__global__ void __launch_bounds__(STEP_THREADS) rmsnorm_rotate_kernel(const void* __restrict__ x, void* __restrict__ residual,
                                                                       const void* __restrict__ weight, float eps, int bf16,
                                                                       const __half* __restrict__ suh, int shards, int rows, int k,
                                                                       void* __restrict__ normed, uint32_t* __restrict__ xf, int mode)
{
    __shared__ float part[STEP_THREADS / 32];
    __shared__ float rstd_s;
    ptx::grid_launch_dependents();
    ptx::grid_dependency_wait();
    const int row = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kgs = k >> 7;
    const bool b = bf16 != 0;
    float h[STEP_MAX_BLOCKS_PER_WARP][4];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < STEP_MAX_BLOCKS_PER_WARP; j++) {
        const int kg = warp + j * (STEP_THREADS / 32);
        if (kg < kgs) {
            const long long i0 = (long long)row * k + kg * 128 + 4 * lane;
            float z[4];
#pragma unroll
            for (int e = 0; e < 4; e++) {
                z[e] = to_f32(x, i0 + e, b);
                if (residual) z[e] = round_act(z[e] + to_f32(residual, i0 + e, b), b);
                h[j][e] = z[e];
                ss += z[e] * z[e];
            }
            if (residual) store_act4(residual, i0, z, b);
        }
    }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, m);
    if (lane == 0) part[warp] = ss;
    __syncthreads();
    if (warp == 0) {
        float t = part[lane];                            // 32 warps: one partial per lane, added in a fixed order
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) t += __shfl_xor_sync(0xFFFFFFFFu, t, m);
        if (lane == 0) rstd_s = rsqrtf(t / (float)k + eps);
    }
    __syncthreads();
    const float rstd = rstd_s;
#pragma unroll
    for (int j = 0; j < STEP_MAX_BLOCKS_PER_WARP; j++) {
        const int kg = warp + j * (STEP_THREADS / 32);
        if (kg < kgs) {                                   // warp-uniform: all lanes take part in the rotation's shuffles
            const long long i0 = (long long)row * k + kg * 128 + 4 * lane;
            float a[4];
#pragma unroll
            for (int e = 0; e < 4; e++) a[e] = round_act(h[j][e] * rstd * to_f32(weight, kg * 128 + 4 * lane + e, b), b);
            if (normed) store_act4(normed, i0, a, b);
            for (int s = 0; s < shards; s++) rotate_store(a, suh + (long long)s * k + kg * 128, xf, mode, s, k >> 4, rows, row, kg, lane);
        }
    }
}

// One warp per (row, 128 block of the intermediate width).  gu [rows, 2 * inter] = gate | up.
__global__ void silu_mul_rotate_kernel(const void* __restrict__ gu, int bf16, const __half* __restrict__ suh, int rows, int inter,
                                       void* __restrict__ act, uint32_t* __restrict__ xf, int mode)
{
    ptx::grid_launch_dependents();
    ptx::grid_dependency_wait();
    const int lane = threadIdx.x & 31;
    const int kgs = inter >> 7;
    const long long item = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (long long)rows * kgs) return;
    const int kg = (int)(item % kgs), row = (int)(item / kgs);
    const bool b = bf16 != 0;
    float a[4];
#pragma unroll
    for (int e = 0; e < 4; e++) {
        const int col = kg * 128 + 4 * lane + e;
        const float g = to_f32(gu, (long long)row * 2 * inter + col, b), u = to_f32(gu, (long long)row * 2 * inter + inter + col, b);
        a[e] = round_act(g / (1.0f + __expf(-g)) * u, b);
    }
    if (act) store_act4(act, (long long)row * inter + kg * 128 + 4 * lane, a, b);
    rotate_store(a, suh + kg * 128, xf, mode, 0, inter >> 4, rows, row, kg, lane);
}

int launch_rmsnorm_rotate(const void* x, void* residual, const void* weight, float eps, int bf16, const __half* suh, int shards, int rows,
                          int k, void* normed, uint32_t* xf, int mode, cudaStream_t st)
{
    if (rows == 0 || k == 0) return EXL3_OK;
    if ((k >> 7) > STEP_MAX_BLOCKS_PER_WARP * (STEP_THREADS / 32)) return EXL3_ERR_BAD_SHAPE;
    return launch_chained(rmsnorm_rotate_kernel, dim3(rows), dim3(STEP_THREADS), 0, st, x, residual, weight, eps, bf16, suh, shards, rows, k,
                          normed, xf, mode);
}

int launch_silu_mul_rotate(const void* gu, int bf16, const __half* suh, int rows, int inter, void* act, uint32_t* xf, int mode,
                           cudaStream_t st)
{
    const long long items = (long long)rows * (inter / 128);
    if (items == 0) return EXL3_OK;
    return launch_chained(silu_mul_rotate_kernel, dim3((unsigned)((items + 7) / 8)), dim3(256), 0, st, gu, bf16, suh, rows, inter, act, xf,
                          mode);
}

}  // namespace exl3
