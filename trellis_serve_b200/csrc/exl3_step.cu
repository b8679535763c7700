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

// Four consecutive activations (8-byte aligned) as floats.
__device__ __forceinline__ void load_act4(const void* p, long long i, bool bf16, float (&v)[4])
{
    if (bf16) {
        const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(p) + i);
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), c = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
        v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(c); v[3] = __high2float(c);
    } else {
        const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const __half*>(p) + i);
        const __half2 a = *reinterpret_cast<const __half2*>(&raw.x), c = *reinterpret_cast<const __half2*>(&raw.y);
        v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(c); v[3] = __high2float(c);
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
// normed [rows, k] or null.  J = 128-column blocks a warp keeps in registers (k <= J * 4096).
template <int J>
__global__ void __launch_bounds__(STEP_THREADS) rmsnorm_rotate_kernel(const void* __restrict__ x, void* __restrict__ residual,
                                                                       const void* __restrict__ weight, float eps, int bf16,
                                                                       const __half* __restrict__ suh, int shards, int rows, int k,
                                                                       void* __restrict__ normed, uint32_t* __restrict__ xf, int mode,
                                                                       void* __restrict__ residual_out)
{
    __shared__ float part[STEP_THREADS / 32];
    __shared__ float rstd_s;
    const int row = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kgs = k >> 7;
    const bool b = bf16 != 0;
    // The norm weights are constants: they are fetched while the kernel ahead is still finishing.
    float wv[J][4];
#pragma unroll
    for (int j = 0; j < J; j++) {
        const int kg = warp + j * (STEP_THREADS / 32);
        if (kg < kgs) load_act4(weight, kg * 128 + 4 * lane, b, wv[j]);
    }
    ptx::grid_launch_dependents();
    ptx::grid_dependency_wait();
    float h[J][4];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < J; j++) {
        const int kg = warp + j * (STEP_THREADS / 32);
        if (kg < kgs) {
            const long long i0 = (long long)row * k + kg * 128 + 4 * lane;
            float z[4], r[4];
            load_act4(x, i0, b, z);
            if (residual) {
                load_act4(residual, i0, b, r);
#pragma unroll
                for (int e = 0; e < 4; e++) z[e] = round_act(z[e] + r[e], b);
                store_act4(residual_out ? residual_out : residual, i0, z, b);      // in place unless a second buffer is given
            }
#pragma unroll
            for (int e = 0; e < 4; e++) {
                h[j][e] = z[e];
                ss += z[e] * z[e];
            }
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
    for (int j = 0; j < J; j++) {
        const int kg = warp + j * (STEP_THREADS / 32);
        if (kg < kgs) {                                   // warp-uniform: all lanes take part in the rotation's shuffles
            const long long i0 = (long long)row * k + kg * 128 + 4 * lane;
            float a[4];
#pragma unroll
            for (int e = 0; e < 4; e++) a[e] = round_act(h[j][e] * rstd * wv[j][e], b);
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
    float a[4], gv[4], uv[4];
    load_act4(gu, (long long)row * 2 * inter + kg * 128 + 4 * lane, b, gv);
    load_act4(gu, (long long)row * 2 * inter + inter + kg * 128 + 4 * lane, b, uv);
#pragma unroll
    for (int e = 0; e < 4; e++) a[e] = round_act(gv[e] / (1.0f + __expf(-gv[e])) * uv[e], b);
    if (act) store_act4(act, (long long)row * inter + kg * 128 + 4 * lane, a, b);
    rotate_store(a, suh + kg * 128, xf, mode, 0, inter >> 4, rows, row, kg, lane);
}

// z = x (+ res_in, rounded to the activation type) -> res_out, and the sums of squares of z per (row, 128 columns) -> ssq.
// One warp per (row, block).  The start of a chain of residual blocks whose linears carry the stream in their epilogues.
__global__ void residual_ssq_kernel(const void* __restrict__ x, const void* __restrict__ res_in, int bf16, int rows, int k,
                                    void* __restrict__ res_out, float* __restrict__ ssq)
{
    ptx::grid_launch_dependents();
    ptx::grid_dependency_wait();
    const int lane = threadIdx.x & 31;
    const int kgs = k >> 7;
    const long long item = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (long long)rows * kgs) return;
    const bool b = bf16 != 0;
    const long long at = (item / kgs) * k + (item % kgs) * 128 + 4 * lane;
    float z[4], r[4];
    load_act4(x, at, b, z);
    if (res_in) {
        load_act4(res_in, at, b, r);
#pragma unroll
        for (int e = 0; e < 4; e++) z[e] = round_act(z[e] + r[e], b);
    }
    if (res_out) store_act4(res_out, at, z, b);
    float ss = z[0] * z[0] + z[1] * z[1] + z[2] * z[2] + z[3] * z[3];
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, m);
    if (lane == 0) ssq[item] = ss;
}

int launch_residual_ssq(const void* x, const void* res_in, int bf16, int rows, int k, void* res_out, float* ssq, cudaStream_t st)
{
    const long long items = (long long)rows * (k / 128);
    if (items == 0) return EXL3_OK;
    return launch_chained(residual_ssq_kernel, dim3((unsigned)((items + 7) / 8)), dim3(256), 0, st, x, res_in, bf16, rows, k, res_out, ssq);
}

int launch_rmsnorm_rotate(const void* x, void* residual, const void* weight, float eps, int bf16, const __half* suh, int shards, int rows,
                          int k, void* normed, uint32_t* xf, int mode, cudaStream_t st, void* residual_out)
{
    if (rows == 0 || k == 0) return EXL3_OK;
    if ((k >> 7) > STEP_MAX_BLOCKS_PER_WARP * (STEP_THREADS / 32)) return EXL3_ERR_BAD_SHAPE;
    const int per_warp = ((k >> 7) + STEP_THREADS / 32 - 1) / (STEP_THREADS / 32);
    auto kernel = per_warp <= 2 ? rmsnorm_rotate_kernel<2> : per_warp <= 4 ? rmsnorm_rotate_kernel<4> : rmsnorm_rotate_kernel<STEP_MAX_BLOCKS_PER_WARP>;
    return launch_chained(kernel, dim3(rows), dim3(STEP_THREADS), 0, st, x, residual, weight, eps, bf16, suh, shards, rows, k, normed, xf, mode,
                          residual_out);
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

// ------------------------------------------------------------------------------------------------ attention side of the step
//
// Between q|k|v and o a decode step applies the rotary embedding to q and k, appends k and v to the cache and attends over
// the cache.  None of it is quantized arithmetic; it is written here so that the step does not pay a dozen framework
// launches per layer.  Head dimension 128, grouped queries (q_heads a multiple of kv_heads), one new token per sequence.

namespace exl3 {

constexpr int ATT_D = 128;
constexpr int ATT_MAX_GROUP = 8;          // query heads per KV head
constexpr int ATT_WARPS = 4;
constexpr int ATT_CHUNK = ATT_WARPS * 32; // cache positions per CTA
constexpr int ATT_PART = ATT_D + 4;       // floats of one partial result: 128 weighted sums, maximum, normaliser (16-byte rows)

// One thread per (row, head, pair i < 64): x1' = x1 cos - x2 sin, x2' = x2 cos + x1 sin with x1 = x[i], x2 = x[i + 64]
// (the "rotate half" convention).  Query heads are rotated in place in qkv; key heads are rotated into the cache slot
// `pos`, value heads copied there.  cache layout [rows, kv_heads, t_max, 128].
__global__ void rope_append_kernel(void* __restrict__ qkv, int bf16, int rows, int q_heads, int kv_heads, const float* __restrict__ cos_t,
                                   const float* __restrict__ sin_t, void* __restrict__ k_cache, void* __restrict__ v_cache, int t_max,
                                   const int* __restrict__ pos_ptr)
{
    ptx::grid_launch_dependents();
    ptx::grid_dependency_wait();
    const int heads = q_heads + 2 * kv_heads;
    const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (idx >= (long long)rows * heads * 64) return;
    const int i = (int)(idx & 63), head = (int)((idx >> 6) % heads), row = (int)((idx >> 6) / heads);
    const int pos = *pos_ptr;
    const long long base = ((long long)row * heads + head) * ATT_D;
    const bool b = bf16 != 0;
    const float x1 = to_f32(qkv, base + i, b), x2 = to_f32(qkv, base + i + 64, b);
    auto put = [&](void* dst, long long at, float v) {
        if (b) reinterpret_cast<__nv_bfloat16*>(dst)[at] = __float2bfloat16_rn(v);
        else reinterpret_cast<__half*>(dst)[at] = __float2half_rn(v);
    };
    if (head < q_heads + kv_heads) {
        const float c = cos_t[(long long)pos * 64 + i], s = sin_t[(long long)pos * 64 + i];
        const float y1 = x1 * c - x2 * s, y2 = x2 * c + x1 * s;
        if (head < q_heads) {
            put(qkv, base + i, y1);
            put(qkv, base + i + 64, y2);
        } else {
            const long long at = (((long long)row * kv_heads + (head - q_heads)) * t_max + pos) * ATT_D;
            put(k_cache, at + i, y1);
            put(k_cache, at + i + 64, y2);
        }
    } else {
        const long long at = (((long long)row * kv_heads + (head - q_heads - kv_heads)) * t_max + pos) * ATT_D;
        put(v_cache, at + i, x1);
        put(v_cache, at + i + 64, x2);
    }
}

#ifdef EXL3_TIMELINE
// Measurement build only: thread 0 of every attention CTA stamps %globaltimer; the slot is derived from the cache address.
__device__ unsigned long long g_att_timeline[64][256][8];
extern "C" int exl3_debug_att_timeline(unsigned long long* host_out) { return (int)cudaMemcpyFromSymbol(host_out, g_att_timeline, sizeof(g_att_timeline)); }
#define ATT_STAMP(i)                                                                                                          \
    do {                                                                                                                      \
        if (threadIdx.x == 0) {                                                                                               \
            unsigned long long t_;                                                                                            \
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                                                            \
            g_att_timeline[(unsigned)(reinterpret_cast<unsigned long long>(k_cache) >> 22) & 63][blockIdx.x + gridDim.x * blockIdx.y][i] = t_; \
        }                                                                                                                     \
    } while (0)
#else
#define ATT_STAMP(i) do { } while (0)
#endif

// One warp, one (row, query head): lane l merges columns 4l..4l+3 of every partial of the head (fixed order: the same bits
// every time), writes the output and -- a head is exactly one 128-wide rotation block of the o projection's input --
// optionally the rotated fragments of that block for the linear that follows (suh != null).  The partials were written by
// other CTAs of the same launch, so they are read past the L1 cache.
__device__ __forceinline__ void attention_merge_head(const float* base, long long stride, int parts, int rows, int q_heads, int row, int qh,
                                                     int lane, void* out, bool bf16, const __half* suh, uint32_t* xf, int mode)
{
    // Sixteen partials per round of loads (one round up to 2048 cache positions), added in split order under a running
    // maximum.
    float mx = -INFINITY, num[4] = {0.f, 0.f, 0.f, 0.f}, den = 0.f;
    for (int s0 = 0; s0 < parts; s0 += 16) {
        float4 a[16];
        float ms[16], ls[16];
#pragma unroll
        for (int u = 0; u < 16; u++) {
            const bool in = s0 + u < parts;
            const float* ps = base + (long long)(in ? s0 + u : s0) * stride;
            a[u] = __ldcg(reinterpret_cast<const float4*>(ps + 4 * lane));
            ms[u] = in ? __ldcg(ps + ATT_D) : -INFINITY;
            ls[u] = __ldcg(ps + ATT_D + 1);
        }
        float bm = mx;
#pragma unroll
        for (int u = 0; u < 16; u++) bm = fmaxf(bm, ms[u]);
        const float keep = mx == -INFINITY ? 0.f : __expf(mx - bm);   // rescale what earlier rounds added
        mx = bm;
        den *= keep;
#pragma unroll
        for (int e = 0; e < 4; e++) num[e] *= keep;
#pragma unroll
        for (int u = 0; u < 16; u++) {
            const float w = ms[u] == -INFINITY ? 0.f : __expf(ms[u] - mx);
            num[0] += w * a[u].x;
            num[1] += w * a[u].y;
            num[2] += w * a[u].z;
            num[3] += w * a[u].w;
            den += w * ls[u];
        }
    }
    float y[4];
#pragma unroll
    for (int e = 0; e < 4; e++) y[e] = round_act(num[e] / den, bf16);
    if (out) store_act4(out, ((long long)row * q_heads + qh) * ATT_D + 4 * lane, y, bf16);
    if (suh) rotate_store(y, suh + qh * ATT_D, xf, mode, 0, (q_heads * ATT_D) >> 4, rows, row, qh, lane);
}

// The merge of all splits of one (row, KV head) by a whole CTA (ATT_WARPS warps).  `dry`: same instructions, no stores -- run
// once before the wait for the kernel ahead, while the CTA has nothing else to do, so that the real pass at the very end of
// the launch finds its code in the instruction cache.
template <int G>
static __device__ __noinline__ void attention_merge_cta(const float* part, float (*red)[G][ATT_PART], int row, int kvh, int kv_heads, int q_heads,
                                                        int splits, int rows, void* y_out, bool b, const __half* suh, uint32_t* xf, int mode,
                                                        bool dry)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float* base = part + ((long long)row * kv_heads + kvh) * splits * (G * ATT_PART);
    const long long stride = (long long)G * ATT_PART;
    if (splits > 32) {                                            // more than 4096 cache positions: one warp per head, split after split
        if (!dry)
            for (int g = warp; g < G; g += ATT_WARPS)
                attention_merge_head(base + g * ATT_PART, stride, splits, rows, q_heads, row, kvh * G + g, lane, y_out, b, suh, xf, mode);
        return;
    }
    // Up to 32 splits: the whole CTA merges all G heads together, in three short phases with one round of loads each, so the
    // tail of the launch is a few dependent memory round trips instead of one per head and warp.  Every sum has a fixed order.
    __shared__ float sm_ms[ATT_MAX_GROUP * 32], sm_ls[ATT_MAX_GROUP * 32], sm_w[ATT_MAX_GROUP * 32];
    // (1) maxima and normalisers of every (head, split)
    for (int i = threadIdx.x; i < G * splits; i += ATT_WARPS * 32) {
        const int g = i / splits, sp = i - g * splits;
        const float* ps = base + sp * stride + g * ATT_PART;
        sm_ms[g * 32 + sp] = __ldcg(ps + ATT_D);
        sm_ls[g * 32 + sp] = __ldcg(ps + ATT_D + 1);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < G * splits; i += ATT_WARPS * 32) {
        const int g = i / splits, sp = i - g * splits;
        float mx = -INFINITY;
#pragma unroll 1
        for (int t2 = 0; t2 < splits; t2++) mx = fmaxf(mx, sm_ms[g * 32 + t2]);
        const float ms = sm_ms[g * 32 + sp];
        sm_w[g * 32 + sp] = ms == -INFINITY ? 0.f : __expf(ms - mx);
    }
    __syncthreads();
    // (2) warp w adds the splits w, w + 4, ... of every head
    constexpr int JB = G <= 5 ? 5 : (G <= 6 ? 4 : 3);            // splits in flight per warp: JB x G 16-byte loads per lane
    float sum[G][4];
#pragma unroll
    for (int g = 0; g < G; g++)
#pragma unroll
        for (int e = 0; e < 4; e++) sum[g][e] = 0.f;
    const int per_warp = (splits + ATT_WARPS - 1) / ATT_WARPS;
#pragma unroll 1
    for (int j0 = 0; j0 < per_warp; j0 += JB) {
        float4 a[JB][G];
#pragma unroll
        for (int j = 0; j < JB; j++) {
            const int sp = warp + ATT_WARPS * (j0 + j);
#pragma unroll
            for (int g = 0; g < G; g++)
                a[j][g] = sp < splits ? __ldcg(reinterpret_cast<const float4*>(base + sp * stride + g * ATT_PART + 4 * lane)) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int j = 0; j < JB; j++) {
            const int sp = warp + ATT_WARPS * (j0 + j);
#pragma unroll
            for (int g = 0; g < G; g++) {
                const float w = sp < splits ? sm_w[g * 32 + sp] : 0.f;
                sum[g][0] += w * a[j][g].x;
                sum[g][1] += w * a[j][g].y;
                sum[g][2] += w * a[j][g].z;
                sum[g][3] += w * a[j][g].w;
            }
        }
    }
#pragma unroll
    for (int g = 0; g < G; g++) *reinterpret_cast<float4*>(&red[warp][g][4 * lane]) = make_float4(sum[g][0], sum[g][1], sum[g][2], sum[g][3]);
    __syncthreads();
    // (3) one warp per head: the warps' sums in warp order, the normaliser, the output and the next linear's fragments
    for (int g = warp; g < G; g += ATT_WARPS) {
        float num[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int w = 0; w < ATT_WARPS; w++) {
            const float4 v = *reinterpret_cast<const float4*>(&red[w][g][4 * lane]);
            num[0] += v.x;
            num[1] += v.y;
            num[2] += v.z;
            num[3] += v.w;
        }
        float den = lane < splits ? sm_w[g * 32 + lane] * sm_ls[g * 32 + lane] : 0.f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) den += __shfl_xor_sync(0xFFFFFFFFu, den, o);
        const int qh = kvh * G + g;
        float y[4];
#pragma unroll
        for (int e = 0; e < 4; e++) y[e] = round_act(num[e] / den, b);
        if (y_out && !dry) store_act4(y_out, ((long long)row * q_heads + qh) * ATT_D + 4 * lane, y, b);
        if (suh && !dry) rotate_store(y, suh + qh * ATT_D, xf, mode, 0, (q_heads * ATT_D) >> 4, rows, row, qh, lane);
    }
}

// Split-KV decode attention.  grid = (splits, kv_heads, rows); a CTA attends positions [split * ATT_CHUNK ...) of one KV
// head for its G query heads: every lane owns ONE position (reads its key row, G dot products against the queries held in
// shared memory, no shuffles), the warp then walks its 32 positions for the values (each lane four of the 128 columns).
// Partial results (running maximum, normaliser, G x 128 weighted sums per split) go to scratch; the last CTA of a (row, KV
// head) to arrive merges them.
// With cos_t / sin_t the kernel also does what rope_append_kernel does, with the same roundings: the queries are rotated as
// they are loaded (qkv itself is left as it is), and the warp that owns cache position `pos` rotates the new key into the
// cache and copies the new value there before it reads them back like any other position.
template <int G>
__global__ void __launch_bounds__(ATT_WARPS * 32) decode_attention_kernel(const void* __restrict__ qkv, int bf16, int q_heads, int kv_heads,
                                                                           void* k_cache, void* v_cache, int t_max,
                                                                           const int* __restrict__ pos_ptr, float scale,
                                                                           const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                                                           float* part, int* counters, int* err, int rows, void* __restrict__ y_out,
                                                                           const __half* __restrict__ suh, uint32_t* __restrict__ xf, int mode)
{
    // Dynamic shared memory: the CTA's chunk of keys and of values (ATT_CHUNK rows of 256 bytes each), brought in by two bulk
    // copies.  The loops over them are short and rolled: a kernel whose every instruction runs once is bound by instruction
    // fetch, not by arithmetic.
    extern __shared__ __align__(128) unsigned char att_smem[];
    unsigned char* ks = att_smem;
    unsigned char* vs = att_smem + ATT_CHUNK * ATT_D * 2;
    // queries, chunk-major: qs[g][half][chunk of 8 columns][4] so that lanes reading different chunks hit different banks
    __shared__ __align__(16) float qs[G][2][16][4];
    __shared__ __align__(16) float red[ATT_WARPS][G][ATT_PART];
    __shared__ __align__(8) uint64_t bar;
    ATT_STAMP(0);
    ptx::grid_launch_dependents();
    const int split = blockIdx.x, kvh = blockIdx.y, row = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pos = *pos_ptr;
    const int T = pos + 1;                                        // valid cache positions
    const int heads = q_heads + 2 * kv_heads;
    const bool b = bf16 != 0;
    const int chunk0 = split * ATT_CHUNK;
    const int t0 = chunk0 + warp * 32;
    const int t = t0 + lane;
    const long long rowbase = (((long long)row * kv_heads + kvh) * t_max) * ATT_D;
    // Cache rows below `pos` were written by earlier steps: like weights they are constants of this launch and are requested
    // before the wait for the kernel ahead, so their trip from memory overlaps that kernel's tail; row `pos` itself comes from
    // the kernel ahead or from this kernel's own append and is put in place after the wait.
    int old_rows = pos - chunk0;
    old_rows = old_rows < 0 ? 0 : (old_rows > ATT_CHUNK ? ATT_CHUNK : old_rows);
    if (threadIdx.x == 0) {
        ptx::mbar_init(&bar, 1);
        ptx::mbar_fence_init();
        if (old_rows > 0) {
            const uint32_t bytes = (uint32_t)old_rows * ATT_D * 2;
            ptx::mbar_arrive_expect_tx(&bar, 2 * bytes);
            ptx::bulk_g2s(ks, reinterpret_cast<const unsigned char*>(k_cache) + (rowbase + (long long)chunk0 * ATT_D) * 2, bytes, &bar);
            ptx::bulk_g2s(vs, reinterpret_cast<const unsigned char*>(v_cache) + (rowbase + (long long)chunk0 * ATT_D) * 2, bytes, &bar);
        }
    }
    // Nothing else to do until the kernel ahead has finished: walk through the merge code once without storing anything, so
    // that the CTA that ends up merging runs it from the instruction cache (it looks at last step's partials).
    attention_merge_cta<G>(part, red, row, kvh, kv_heads, q_heads, gridDim.x, rows, y_out, b, suh, xf, mode, true);
    ptx::grid_dependency_wait();
    ATT_STAMP(1);
    // queries (rotated here when the tables are given), scaled
    for (int e = threadIdx.x; e < G * (ATT_D / 2); e += ATT_WARPS * 32) {
        const int g = e / (ATT_D / 2), i = e % (ATT_D / 2);
        const long long at = ((long long)row * heads + kvh * G + g) * ATT_D;
        const float x1 = to_f32(qkv, at + i, b), x2 = to_f32(qkv, at + i + 64, b);
        float y1 = x1, y2 = x2;
        if (cos_t) {
            const float c = cos_t[(long long)pos * 64 + i], sn = sin_t[(long long)pos * 64 + i];
            y1 = round_act(x1 * c - x2 * sn, b);
            y2 = round_act(x2 * c + x1 * sn, b);
        }
        qs[g][(i >> 2) & 1][i >> 3][i & 3] = y1 * scale;
        qs[g][((i + 64) >> 2) & 1][(i + 64) >> 3][i & 3] = y2 * scale;
    }
    // the new row: rotated key and value into the cache (with the tables) and, either way, into this CTA's chunk
    if (pos >= t0 && pos < t0 + 32) {                             // warp-uniform: the warp that owns position `pos`
        const long long cat = rowbase + (long long)pos * ATT_D;
        const int r = pos - chunk0;
        if (cos_t) {
            const long long kat = ((long long)row * heads + q_heads + kvh) * ATT_D, vat = kat + (long long)kv_heads * ATT_D;
            for (int i = lane; i < 64; i += 32) {
                const float x1 = to_f32(qkv, kat + i, b), x2 = to_f32(qkv, kat + i + 64, b);
                const float c = cos_t[(long long)pos * 64 + i], sn = sin_t[(long long)pos * 64 + i];
                const float y1 = x1 * c - x2 * sn, y2 = x2 * c + x1 * sn;
                uint16_t h1, h2;
                if (b) {
                    h1 = __bfloat16_as_ushort(__float2bfloat16_rn(y1));
                    h2 = __bfloat16_as_ushort(__float2bfloat16_rn(y2));
                } else {
                    h1 = __half_as_ushort(__float2half_rn(y1));
                    h2 = __half_as_ushort(__float2half_rn(y2));
                }
                reinterpret_cast<uint16_t*>(k_cache)[cat + i] = h1;
                reinterpret_cast<uint16_t*>(k_cache)[cat + i + 64] = h2;
                reinterpret_cast<uint16_t*>(ks)[r * ATT_D + i] = h1;
                reinterpret_cast<uint16_t*>(ks)[r * ATT_D + i + 64] = h2;
            }
            const uint2 vv = reinterpret_cast<const uint2*>(reinterpret_cast<const unsigned char*>(qkv) + vat * 2)[lane];
            reinterpret_cast<uint2*>(reinterpret_cast<unsigned char*>(v_cache) + cat * 2)[lane] = vv;
            reinterpret_cast<uint2*>(vs + (size_t)r * ATT_D * 2)[lane] = vv;
        } else {
            reinterpret_cast<uint2*>(ks + (size_t)r * ATT_D * 2)[lane] = reinterpret_cast<const uint2*>(reinterpret_cast<const unsigned char*>(k_cache) + cat * 2)[lane];
            reinterpret_cast<uint2*>(vs + (size_t)r * ATT_D * 2)[lane] = reinterpret_cast<const uint2*>(reinterpret_cast<const unsigned char*>(v_cache) + cat * 2)[lane];
        }
    }
    __syncthreads();
    if (old_rows > 0 && !ptx::mbar_wait(&bar, 0) && lane == 0) atomicExch(err, 1);
    const int splits = gridDim.x;
    float* out = part + (((long long)row * kv_heads + kvh) * splits + split) * (G * ATT_PART);
    // scores: lane = position; its key row in 16 chunks of 8 columns, taken in an order rotated by the lane number so that
    // the lanes of a quarter warp read different banks (rows are 256 bytes apart); the query chunk follows the same order
    float sc[G];
#pragma unroll
    for (int g = 0; g < G; g++) sc[g] = 0.f;
    if (t < T) {
        const uint32_t krow = ptx::smem_addr(ks) + (uint32_t)(warp * 32 + lane) * (ATT_D * 2);
#pragma unroll 2
        for (int j = 0; j < 16; j++) {
            const int c = (j + lane) & 15;
            const uint4 w = ptx::lds128(krow + c * 16);
            const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
            float kf[8];
#pragma unroll
            for (int h2 = 0; h2 < 4; h2++) {
                if (b) {
                    const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(&ww[h2]);
                    kf[2 * h2] = __low2float(v);
                    kf[2 * h2 + 1] = __high2float(v);
                } else {
                    const __half2 v = *reinterpret_cast<const __half2*>(&ww[h2]);
                    kf[2 * h2] = __low2float(v);
                    kf[2 * h2 + 1] = __high2float(v);
                }
            }
#pragma unroll
            for (int g = 0; g < G; g++) {
                const float4 qa = *reinterpret_cast<const float4*>(&qs[g][0][c][0]), qb = *reinterpret_cast<const float4*>(&qs[g][1][c][0]);
                sc[g] += kf[0] * qa.x + kf[1] * qa.y + kf[2] * qa.z + kf[3] * qa.w + kf[4] * qb.x + kf[5] * qb.y + kf[6] * qb.z + kf[7] * qb.w;
            }
        }
    }
    ATT_STAMP(2);
    float m[G], l[G], p[G];
#pragma unroll
    for (int g = 0; g < G; g++) {
        float v = t < T ? sc[g] : -INFINITY;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
        m[g] = v;
        p[g] = (t < T) ? __expf(sc[g] - v) : 0.f;
        float s = p[g];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, o);
        l[g] = s;
    }
    // values: the warp walks its positions, each lane four of the 128 columns
    float acc[G][4];
#pragma unroll
    for (int g = 0; g < G; g++)
#pragma unroll
        for (int e = 0; e < 4; e++) acc[g][e] = 0.f;
    const int n = T - t0 < 32 ? (T - t0 < 0 ? 0 : T - t0) : 32;   // warp-uniform: positions of this warp that exist
    const uint32_t vrow = ptx::smem_addr(vs) + (uint32_t)(warp * 32) * (ATT_D * 2) + lane * 8;
#pragma unroll 4
    for (int u = 0; u < n; u++) {
        const uint2 w = ptx::lds64(vrow + u * (ATT_D * 2));
        float v[4];
        if (b) {
            const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&w.x), c = *reinterpret_cast<const __nv_bfloat162*>(&w.y);
            v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(c); v[3] = __high2float(c);
        } else {
            const __half2 a = *reinterpret_cast<const __half2*>(&w.x), c = *reinterpret_cast<const __half2*>(&w.y);
            v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(c); v[3] = __high2float(c);
        }
#pragma unroll
        for (int g = 0; g < G; g++) {
            const float pj = __shfl_sync(0xFFFFFFFFu, p[g], u);
#pragma unroll
            for (int e = 0; e < 4; e++) acc[g][e] += pj * v[e];
        }
    }
    ATT_STAMP(3);
    __shared__ float wgt[G][ATT_WARPS];
    __shared__ int last_s;
    // The four warps' partial results are merged inside the CTA (fixed warp order), so one partial per split goes out.
#pragma unroll
    for (int g = 0; g < G; g++) {
        *reinterpret_cast<float4*>(&red[warp][g][4 * lane]) = make_float4(acc[g][0], acc[g][1], acc[g][2], acc[g][3]);
        if (lane == 0) {
            red[warp][g][ATT_D] = n > 0 ? m[g] : -INFINITY;
            red[warp][g][ATT_D + 1] = n > 0 ? l[g] : 0.f;
        }
    }
    __syncthreads();
    if (threadIdx.x < G) {
        const int g = threadIdx.x;
        float mx = -INFINITY;
#pragma unroll
        for (int w = 0; w < ATT_WARPS; w++) mx = fmaxf(mx, red[w][g][ATT_D]);
        float den = 0.f;
#pragma unroll
        for (int w = 0; w < ATT_WARPS; w++) {
            const float mw = red[w][g][ATT_D];
            const float f = mw == -INFINITY ? 0.f : __expf(mw - mx);
            wgt[g][w] = f;
            den += f * red[w][g][ATT_D + 1];
        }
        out[g * ATT_PART + ATT_D] = mx;
        out[g * ATT_PART + ATT_D + 1] = den;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < G * (ATT_D / 4); e += ATT_WARPS * 32) {
        const int g = e / (ATT_D / 4), c = (e % (ATT_D / 4)) * 4;
        float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int w = 0; w < ATT_WARPS; w++) {
            const float f = wgt[g][w];
            const float4 a = *reinterpret_cast<const float4*>(&red[w][g][c]);
            sum.x += f * a.x;
            sum.y += f * a.y;
            sum.z += f * a.z;
            sum.w += f * a.w;
        }
        *reinterpret_cast<float4*>(out + g * ATT_PART + c) = sum;
    }
    // The CTA that is last to deliver its split for this (row, KV head) merges all of them: no second launch.  Its partial
    // stores are fenced before the count, the others' are read after it.
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        int* cnt = counters + row * kv_heads + kvh;
        const int arrived = atomicAdd(cnt, 1);
        last_s = arrived == splits - 1;
        if (last_s) *cnt = 0;                                     // everyone has counted: zero again for the next launch
    }
    __syncthreads();
    ATT_STAMP(4);
    if (!last_s) return;
    __threadfence();
    ATT_STAMP(5);
    attention_merge_cta<G>(part, red, row, kvh, kv_heads, q_heads, splits, rows, y_out, b, suh, xf, mode, false);
    ATT_STAMP(7);
}

// Scratch: an error word (set when the bounded wait for the cache copies gives up; exl3_device_error reads it), one arrival
// counter per (row, KV head) -- zero before the first launch, left zero by every launch -- then the partials.
constexpr size_t ATT_SCRATCH_HEADER = 256;
constexpr size_t ATT_DYN_SMEM = 2 * (size_t)ATT_CHUNK * ATT_D * 2;
static size_t attention_counter_bytes(int rows, int kv_heads) { return ((size_t)rows * kv_heads * sizeof(int) + 255) & ~(size_t)255; }

size_t attention_scratch_bytes(int rows, int q_heads, int kv_heads, int t_max)
{
    const int splits = (t_max + ATT_CHUNK - 1) / ATT_CHUNK;
    const int G = q_heads / (kv_heads > 0 ? kv_heads : 1);
    return ATT_SCRATCH_HEADER + attention_counter_bytes(rows, kv_heads) + (size_t)rows * kv_heads * splits * G * ATT_PART * sizeof(float);
}

// The kernels keep their cache chunk in dynamic shared memory beyond the default limit: opted in once per device.
int attention_init_device()
{
    int rc = cuda_status(cudaFuncSetAttribute(decode_attention_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ATT_DYN_SMEM));
    if (rc == EXL3_OK) rc = cuda_status(cudaFuncSetAttribute(decode_attention_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ATT_DYN_SMEM));
    if (rc == EXL3_OK) rc = cuda_status(cudaFuncSetAttribute(decode_attention_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ATT_DYN_SMEM));
    if (rc == EXL3_OK) rc = cuda_status(cudaFuncSetAttribute(decode_attention_kernel<5>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ATT_DYN_SMEM));
    if (rc == EXL3_OK) rc = cuda_status(cudaFuncSetAttribute(decode_attention_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ATT_DYN_SMEM));
    return rc;
}

int launch_rope_append(void* qkv, int bf16, int rows, int q_heads, int kv_heads, const float* cos_t, const float* sin_t, void* k_cache,
                       void* v_cache, int t_max, const int* pos, cudaStream_t st)
{
    const long long items = (long long)rows * (q_heads + 2 * kv_heads) * 64;
    if (items == 0) return EXL3_OK;
    return launch_chained(rope_append_kernel, dim3((unsigned)((items + 255) / 256)), dim3(256), 0, st, qkv, bf16, rows, q_heads, kv_heads, cos_t,
                          sin_t, k_cache, v_cache, t_max, pos);
}

template <int G>
static int launch_attention_g(const void* qkv, int bf16, int rows, int q_heads, int kv_heads, void* k_cache, void* v_cache, int t_max,
                              const int* pos, float scale, const float* cos_t, const float* sin_t, float* part, void* out, const __half* suh,
                              uint32_t* xf, int mode, cudaStream_t st)
{
    const int splits = (t_max + ATT_CHUNK - 1) / ATT_CHUNK;
    unsigned char* base = reinterpret_cast<unsigned char*>(part);
    int* err = reinterpret_cast<int*>(base);
    int* counters = reinterpret_cast<int*>(base + ATT_SCRATCH_HEADER);
    float* partials = reinterpret_cast<float*>(base + ATT_SCRATCH_HEADER + attention_counter_bytes(rows, kv_heads));
    return launch_chained(decode_attention_kernel<G>, dim3(splits, kv_heads, rows), dim3(ATT_WARPS * 32), ATT_DYN_SMEM, st, qkv, bf16, q_heads,
                          kv_heads, k_cache, v_cache, t_max, pos, scale, cos_t, sin_t, partials, counters, err, rows, out, suh, xf, mode);
}

int launch_decode_attention(const void* qkv, int bf16, int rows, int q_heads, int kv_heads, void* k_cache, void* v_cache, int t_max,
                            const int* pos, float scale, const float* cos_t, const float* sin_t, float* part, void* out, const __half* suh,
                            uint32_t* xf, int mode, cudaStream_t st)
{
    if (rows == 0) return EXL3_OK;
    if (kv_heads < 1 || q_heads % kv_heads) return EXL3_ERR_BAD_SHAPE;
    switch (q_heads / kv_heads) {
        case 1: return launch_attention_g<1>(qkv, bf16, rows, q_heads, kv_heads, k_cache, v_cache, t_max, pos, scale, cos_t, sin_t, part, out, suh, xf, mode, st);
        case 2: return launch_attention_g<2>(qkv, bf16, rows, q_heads, kv_heads, k_cache, v_cache, t_max, pos, scale, cos_t, sin_t, part, out, suh, xf, mode, st);
        case 4: return launch_attention_g<4>(qkv, bf16, rows, q_heads, kv_heads, k_cache, v_cache, t_max, pos, scale, cos_t, sin_t, part, out, suh, xf, mode, st);
        case 5: return launch_attention_g<5>(qkv, bf16, rows, q_heads, kv_heads, k_cache, v_cache, t_max, pos, scale, cos_t, sin_t, part, out, suh, xf, mode, st);
        case 8: return launch_attention_g<8>(qkv, bf16, rows, q_heads, kv_heads, k_cache, v_cache, t_max, pos, scale, cos_t, sin_t, part, out, suh, xf, mode, st);
    }
    return EXL3_ERR_BAD_SHAPE;
}

}  // namespace exl3
