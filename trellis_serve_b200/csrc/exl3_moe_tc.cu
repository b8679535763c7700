// Routed experts with many rows per expert (prefill-sized batches) on the tensor cores (sm_100a).
//
// The grouped GEMV of exl3_moe_kernel.cuh re-streams and re-decodes an expert's matrices once per 8 routed rows, which is
// right for decode batches and wasteful once experts see tens of rows.  The reference answers that by growing its moe
// block from 8 to 64 rows with T * top_k / E (cuda/src/sglang_exl3/kernels/marlin_moe.py:52-57 of 0xSero/trellis-serve)
// inside the same mma.sync kernel; here the routing is aligned to blocks of 128 rows -- the M of one tcgen05.mma -- and
// up to two blocks of one expert (four with the narrow tiling) share every decoded weight block in the grouped instances of
// gemm_tc_kernel:
//
//   align (blocks of 128) -> work items -> gather + suh + Had128 -> A layout        (gate and up inputs)
//   grouped tcgen05 GEMM gate|up  (rotated basis, fp16)
//   Had128 * svh -> SiLU(gate) * up -> fp16 -> * suh2 -> Had128 -> A layout
//   grouped tcgen05 GEMM down     (rotated basis, fp16)
//   Had128 * svh2 -> yd[slot, :]                                                     (the combine kernel closes the layer)
//
// Same arithmetic as the five-launch GEMV layer (cuda/csrc/exl3_marlin_moe.cu:210-292) up to one extra fp16 rounding of
// the rotated-basis GEMM outputs, which the dense many-row path has as well.
#include "exl3_internal.h"
#include "exl3_ptx.cuh"

namespace exl3 {

// One CTA.  Consecutive 128-row blocks of one expert are cut into work items of up to `max_len` blocks.  Block b starts an
// item when its distance to the first block of its expert is a multiple of max_len; items are numbered in block order.
__global__ void moe_tc_items_kernel(const int* __restrict__ expert_ids, const int* __restrict__ num_post, int max_len, int4* __restrict__ items,
                                    int* __restrict__ n_items)
{
    ptx::grid_launch_dependents();
    ptx::grid_dependency_wait();
    __shared__ int warp_total[32];
    __shared__ int carry_sh;
    const int blocks = *num_post / MOE_TC_BLOCK_ROWS;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    if (threadIdx.x == 0) carry_sh = 0;
    __syncthreads();
    for (int b0 = 0; b0 < blocks; b0 += blockDim.x) {
        const int b = b0 + threadIdx.x;
        int e = -1, len = 0, flag = 0;
        if (b < blocks) {
            e = expert_ids[b];
            int first = b;
            while (first > 0 && expert_ids[first - 1] == e) first--;
            if ((b - first) % max_len == 0) {
                flag = 1;
                len = 1;
                while (len < max_len && b + len < blocks && expert_ids[b + len] == e) len++;
            }
        }
        const unsigned ballot = __ballot_sync(0xFFFFFFFFu, flag);
        if (lane == 0) warp_total[wid] = __popc(ballot);
        __syncthreads();
        int before = carry_sh;
        for (int w = 0; w < wid; w++) before += warp_total[w];
        before += __popc(ballot & ((1u << lane) - 1));
        if (flag) items[before] = make_int4(e, b, len, 0);
        __syncthreads();
        if (threadIdx.x == 0) {
            int t = carry_sh;
            for (int w = 0; w < nwarps; w++) t += warp_total[w];
            carry_sh = t;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) *n_items = carry_sh;
}

constexpr int MOE_TC_GROUP = 8;           // positions per warp: one row group of the A layout, four lanes per position (fwht128_quad)

// Eight floats rounded to halves, as one 16-byte word.
__device__ __forceinline__ uint4 pack_h8(const float* v)
{
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const __half2 h = __floats2half2_rn(v[2 * j], v[2 * j + 1]);
        o[j] = *reinterpret_cast<const uint32_t*>(&h);
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
}

// A lane's 32 results as four whole 16-byte core-matrix rows of the A layout.
__device__ __forceinline__ void store_a32(__half* xa, int p, int col, int KB, const float (&v)[32])
{
#pragma unroll
    for (int i = 0; i < 4; i++) *reinterpret_cast<uint4*>(xa + tc_a_offset(p, col + 8 * i, KB)) = pack_h8(&v[8 * i]);
}

// xa[shard][position p] = Had128(fp16(x[token(p)]) * suh[expert(p), shard]) in the A-operand layout.  One warp per (shard,
// group of 8 positions, 128-block).  Padding positions are left as they are: a row of the product depends on its own row of
// A only, and nothing downstream uses the rows of padding positions.
__global__ void moe_tc_had_in_kernel(const void* __restrict__ x, int x_bf16, const __half* __restrict__ suh, int shards, int hidden,
                                     int top_k, int numel, int cap, const int* __restrict__ sorted_ids, const int* __restrict__ expert_ids,
                                     const int* __restrict__ num_post, __half* __restrict__ xa, long long shard_stride)
{
    ptx::grid_launch_dependents();
    ptx::grid_dependency_wait();
    const int lane = threadIdx.x & 31;
    const int kgs = hidden >> 7, groups = cap / MOE_TC_GROUP;
    const long long item = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (long long)shards * groups * kgs) return;
    const int kg = (int)(item % kgs);
    const int p0 = (int)((item / kgs) % groups) * MOE_TC_GROUP;
    const int s = (int)(item / ((long long)kgs * groups));
    if (p0 >= *num_post) return;
    const int p = p0 + (lane >> 2);
    const int ex = expert_ids[p0 / MOE_TC_BLOCK_ROWS];
    const int col = kg * 128 + 32 * (lane & 3);
    const int slot = sorted_ids[p];
    const bool valid = slot >= 0 && slot < numel;
    if (__ballot_sync(0xFFFFFFFFu, valid) == 0) return;       // a group of padding rows: nothing reads what the GEMM makes of them
    float v[32];
    if (valid) {
        float sg[32];
        load_half32(suh + ((long long)ex * shards + s) * hidden + col, sg);
        const long long at = (long long)(slot / top_k) * hidden + col;
        if (x_bf16) {
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const uint4 raw = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(x) + at)[i];
                const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const __nv_bfloat162 bb = *reinterpret_cast<const __nv_bfloat162*>(&w[j]);
                    v[8 * i + 2 * j] = __half2float(__float2half_rn(__low2float(bb)));
                    v[8 * i + 2 * j + 1] = __half2float(__float2half_rn(__high2float(bb)));
                }
            }
        } else {
            load_half32(reinterpret_cast<const __half*>(x) + at, v);
        }
#pragma unroll
        for (int i = 0; i < 32; i++) v[i] *= sg[i];
    } else {
#pragma unroll
        for (int i = 0; i < 32; i++) v[i] = 0.f;
    }
    fwht128_quad(v, lane);
#pragma unroll
    for (int i = 0; i < 32; i++) v[i] *= HAD_SCALE;
    if (valid) store_a32(xa + s * shard_stride, p, col, kgs * 2, v);
}

// 32 columns of a rotated-basis row back in the true basis: Had128(y) * svh, rounded to fp16 like the GEMV's output.
__device__ __forceinline__ void unrotate32(float (&v)[32], const __half* __restrict__ svh, int lane)
{
    float sv[32];
    load_half32(svh, sv);
    fwht128_quad(v, lane);
#pragma unroll
    for (int i = 0; i < 32; i++) v[i] = __half2float(__float2half_rn(v[i] * (HAD_SCALE * sv[i])));
}

// xa2[position p] = Had128( fp16( silu(gate) * up ) * suh2[expert] ) with gate | up = Had128(gu_rot[p]) * svh13[expert].
// One warp per (group of 8 positions, 128-block of the intermediate size).
__global__ void moe_tc_mid_kernel(const __half* __restrict__ gu_rot, const __half* __restrict__ svh13, const __half* __restrict__ suh2,
                                  int inter, int numel, int cap, const int* __restrict__ sorted_ids, const int* __restrict__ expert_ids,
                                  const int* __restrict__ num_post, __half* __restrict__ xa2)
{
    ptx::grid_launch_dependents();
    ptx::grid_dependency_wait();
    const int lane = threadIdx.x & 31;
    const int kgs = inter >> 7, groups = cap / MOE_TC_GROUP;
    const long long item = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (long long)groups * kgs) return;
    const int kg = (int)(item % kgs);
    const int p0 = (int)(item / kgs) * MOE_TC_GROUP;
    if (p0 >= *num_post) return;
    const int p = p0 + (lane >> 2);
    const int ex = expert_ids[p0 / MOE_TC_BLOCK_ROWS];
    const int col = kg * 128 + 32 * (lane & 3);
    const int slot = sorted_ids[p];
    const bool valid = slot >= 0 && slot < numel;
    if (__ballot_sync(0xFFFFFFFFu, valid) == 0) return;       // a group of padding rows
    float g[32], u[32];
#pragma unroll
    for (int i = 0; i < 32; i++) g[i] = u[i] = 0.f;
    if (valid) {
        load_half32(gu_rot + (long long)p * 2 * inter + col, g);
        load_half32(gu_rot + (long long)p * 2 * inter + inter + col, u);
    }
    unrotate32(g, svh13 + (long long)ex * 2 * inter + col, lane);
    unrotate32(u, svh13 + (long long)ex * 2 * inter + inter + col, lane);
    float s2[32];
    load_half32(suh2 + (long long)ex * inter + col, s2);
#pragma unroll
    for (int i = 0; i < 32; i++) {
        const float act = __half2float(__float2half_rn(g[i] / (1.0f + __expf(-g[i])) * u[i]));
        g[i] = valid ? act * s2[i] : 0.f;
    }
    fwht128_quad(g, lane);
#pragma unroll
    for (int i = 0; i < 32; i++) g[i] *= HAD_SCALE;
    if (valid) store_a32(xa2, p, col, kgs * 2, g);
}

// yd[slot(p), :] = fp16( Had128(yd_rot[p]) * svh2[expert] ) for the valid positions.  One warp per (group of 8 positions,
// 128 columns).
__global__ void moe_tc_out_kernel(const __half* __restrict__ yd_rot, const __half* __restrict__ svh2, int hidden, int numel, int cap,
                                  const int* __restrict__ sorted_ids, const int* __restrict__ expert_ids, const int* __restrict__ num_post,
                                  __half* __restrict__ yd)
{
    ptx::grid_launch_dependents();
    ptx::grid_dependency_wait();
    const int lane = threadIdx.x & 31;
    const int nbs = hidden >> 7, groups = cap / MOE_TC_GROUP;
    const long long item = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (long long)groups * nbs) return;
    const int nb = (int)(item % nbs);
    const int p0 = (int)(item / nbs) * MOE_TC_GROUP;
    if (p0 >= *num_post) return;
    const int p = p0 + (lane >> 2);
    const int ex = expert_ids[p0 / MOE_TC_BLOCK_ROWS];
    const int col = nb * 128 + 32 * (lane & 3);
    const int slot = sorted_ids[p];
    const bool valid = slot >= 0 && slot < numel;
    if (__ballot_sync(0xFFFFFFFFu, valid) == 0) return;       // a group of padding rows
    float v[32];
#pragma unroll
    for (int i = 0; i < 32; i++) v[i] = 0.f;
    if (valid) load_half32(yd_rot + (long long)p * hidden + col, v);
    unrotate32(v, svh2 + (long long)ex * hidden + col, lane);
    if (valid) {
        uint4* dst = reinterpret_cast<uint4*>(yd + (long long)slot * hidden + col);
#pragma unroll
        for (int i = 0; i < 4; i++) dst[i] = pack_h8(&v[8 * i]);
    }
}

// ------------------------------------------------------------------------------------------------ host side

static inline size_t up256(size_t v) { return (v + 255) & ~(size_t)255; }

size_t moe_tc_capacity(int slots, int num_local)
{
    if (slots <= 0 || num_local < 1) return 0;
    const size_t used = (size_t)(slots < num_local ? slots : num_local);           // experts that can receive a slot
    const size_t cap = (size_t)slots + used * (MOE_TC_BLOCK_ROWS - 1);
    return (cap + MOE_TC_BLOCK_ROWS - 1) / MOE_TC_BLOCK_ROWS * MOE_TC_BLOCK_ROWS;
}

struct MoeTcLayout {
    size_t sorted, experts, counts, items, xa13, gu, xa2, yd_rot, total;
    int cap, cap512;
};

static MoeTcLayout moe_tc_layout(int slots, int num_local, int hidden, int inter)
{
    MoeTcLayout l;
    l.cap = (int)moe_tc_capacity(slots, num_local);
    l.cap512 = (l.cap + TC_ROWS - 1) / TC_ROWS * TC_ROWS;
    size_t off = 256;                                                               // header: error word
    auto take = [&](size_t bytes) {
        const size_t at = off;
        off += up256(bytes);
        return at;
    };
    l.sorted = take((size_t)l.cap * 4);
    l.experts = take((size_t)(l.cap / MOE_TC_BLOCK_ROWS + 1) * 4);
    l.counts = take(8);                                                             // num_post, n_items
    l.items = take((size_t)(l.cap / MOE_TC_BLOCK_ROWS + 1) * sizeof(int4));
    l.xa13 = take((size_t)2 * l.cap512 * hidden * 2);
    l.gu = take((size_t)l.cap * 2 * inter * 2);
    l.xa2 = take((size_t)l.cap512 * inter * 2);
    l.yd_rot = take((size_t)l.cap * hidden * 2);
    l.total = off;
    return l;
}

size_t moe_tc_workspace_bytes(int slots, int num_local, int hidden, int inter)
{
    return moe_tc_layout(slots, num_local, hidden, inter).total;
}

static inline unsigned blocks_of(long long items, int per_block) { return (unsigned)((items + per_block - 1) / per_block); }

int launch_moe_tc_experts(const void* x, int x_bf16, int top_k, int hidden, int inter, const int* topk_ids, int slots, int num_experts,
                          const int* expert_map, int num_local, const uint32_t* w13, const __half* suh13, const __half* svh13,
                          const uint32_t* w2, const __half* suh2, const __half* svh2, int K, int codebook, __half* yd, unsigned char* ws,
                          cudaStream_t st)
{
    const MoeTcLayout l = moe_tc_layout(slots, num_local, hidden, inter);
    int* err = reinterpret_cast<int*>(ws);
    int* sorted_ids = reinterpret_cast<int*>(ws + l.sorted);
    int* expert_ids = reinterpret_cast<int*>(ws + l.experts);
    int* num_post = reinterpret_cast<int*>(ws + l.counts);
    int* n_items = num_post + 1;
    int4* items = reinterpret_cast<int4*>(ws + l.items);
    __half* xa13 = reinterpret_cast<__half*>(ws + l.xa13);
    __half* gu_rot = reinterpret_cast<__half*>(ws + l.gu);
    __half* xa2 = reinterpret_cast<__half*>(ws + l.xa2);
    __half* yd_rot = reinterpret_cast<__half*>(ws + l.yd_rot);
    const int cap = l.cap;

    if (int rc = launch_moe_align(topk_ids, slots, num_local, MOE_TC_BLOCK_ROWS, cap, sorted_ids, expert_ids, num_post, expert_map,
                                  expert_map ? num_experts : 0, st))
        return rc;
    // Wide tiles need column blocks that pair up inside gate, up and the down projection's output.
    const bool wide = (inter % 256) == 0 && (hidden % 256) == 0;
    const int groups = cap / MOE_TC_GROUP;
    if (int rc = launch_chained(moe_tc_items_kernel, dim3(1), dim3(1024), 0, st, expert_ids, num_post, wide ? TC_GROUPED_MT : 4, items, n_items))
        return rc;
    if (int rc = launch_chained(moe_tc_had_in_kernel, dim3(blocks_of((long long)2 * groups * (hidden / 128), 8)), dim3(256), 0, st, x, x_bf16,
                                suh13, 2, hidden, top_k, slots, cap, sorted_ids, expert_ids, num_post, xa13, (long long)l.cap512 * hidden))
        return rc;
    int ends[GEMV_MAX_SHARDS];
    for (int s = 0; s < GEMV_MAX_SHARDS; s++) ends[s] = 2 * inter / 128;
    ends[0] = inter / 128;
    if (int rc = launch_gemm_tc_grouped(w13, (long long)(2 * inter / 128) * (hidden / 128) * 512 * K, K, codebook, ends, 2, hidden, 2 * inter,
                                        xa13, l.cap512, gu_rot, items, n_items, wide, err, st))
        return rc;
    if (int rc = launch_chained(moe_tc_mid_kernel, dim3(blocks_of((long long)groups * (inter / 128), 8)), dim3(256), 0, st, gu_rot, svh13, suh2,
                                inter, slots, cap, sorted_ids, expert_ids, num_post, xa2))
        return rc;
    for (int s = 0; s < GEMV_MAX_SHARDS; s++) ends[s] = hidden / 128;
    if (int rc = launch_gemm_tc_grouped(w2, (long long)(hidden / 128) * (inter / 128) * 512 * K, K, codebook, ends, 1, inter, hidden, xa2,
                                        l.cap512, yd_rot, items, n_items, wide, err, st))
        return rc;
    return launch_chained(moe_tc_out_kernel, dim3(blocks_of((long long)groups * (hidden / 128), 8)), dim3(256), 0, st, yd_rot, svh2, hidden, slots,
                          cap, sorted_ids, expert_ids, num_post, yd);
}

}  // namespace exl3
