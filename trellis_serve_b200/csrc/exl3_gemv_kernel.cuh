// Decode GEMV / skinny GEMM of the EXL3 linear for 1..16 rows (sm_100a): the HBM-bound path.
//
//   out[r, :] = ( xh[r, :] @ W_inner ) -> optional Had128 * svh
//
// with W_inner decoded on the fly from the resident trellis.  This is the B200 counterpart of the reference's
// fused dense kernel (cuda/csrc/exl3_marlin.cu:489-527 -> cuda/csrc/exl3_marlin_template.h:271), rebuilt around
// the hardware rather than translated:
//
//   * persistent grid, one CTA per SM; the (column block, row block) units of the matrix are split evenly and
//     contiguously over the CTAs ("stream-K"), so every CTA streams ONE contiguous byte range of the weights;
//   * a producer warp feeds a ring of shared-memory stages with 1-D bulk async copies (TMA engine, mbarrier
//     byte counting, no multicast): one stage = one unit = 2048*K bytes of weights + its activation fragments;
//   * 16 consumer warps; warp (nt, kq) owns column tile nt of the block and four of the unit's eight row tiles.
//     A lane reads K words, gets 16-K bits from its neighbour by one shuffle per tile, extracts its eight
//     16-bit states in registers and hashes them.  The resulting registers ARE the A operand of
//     mma.sync.m16n8k16 with the weights transposed (output columns as M, batch rows as N), so one tile costs
//     one MMA (paired) or two (split) whatever the row count up to 8;
//   * partial sums of a column block that several CTAs share go to a workspace; the CTA that arrives last
//     (atomic counter, no spinning) adds them in a fixed order, applies Had128 * svh and stores.  Results are
//     therefore deterministic.
#pragma once
#include "exl3_internal.h"
#include "exl3_ptx.cuh"

namespace exl3 {

constexpr int GEMV_CONSUMER_WARPS = 16;
constexpr int GEMV_THREADS = (GEMV_CONSUMER_WARPS + 1) * 32;
constexpr int GEMV_MAX_STAGES = 12;

enum { GEMV_ERR_FULL_WAIT = 1, GEMV_ERR_EMPTY_WAIT = 2 };

struct GemvLaunch {
    GemvArgs a;
    int KG, NB, grid;
    int units_q, units_r;       // units per CTA: the first units_r CTAs take units_q + 1
    int stages;
    uint32_t stage_stride;      // bytes
    uint32_t xf_bytes;          // activation fragment bytes per unit
    uint32_t mul, add;
    long long xf_shard_stride;  // words between shards in xf
};

__host__ __device__ inline long long gemv_first_unit(int cta, int q, int r) { return (long long)cta * q + (cta < r ? cta : r); }

__device__ __forceinline__ int gemv_cta_of_unit(long long u, int q, int r)
{
    long long boundary = (long long)r * (q + 1);
    return u < boundary ? (int)(u / (q + 1)) : r + (int)((u - boundary) / q);
}

template <int K, int MODE, int FAM>
__device__ __forceinline__ void decode_tile_regs(const LaneTile<K>& lt, CodebookConst cbc, uint32_t (&w)[8])
{
    uint32_t s[8];
    s[0] = window<K, 0>(lt); s[1] = window<K, 1>(lt); s[2] = window<K, 2>(lt); s[3] = window<K, 3>(lt);
    s[4] = window<K, 4>(lt); s[5] = window<K, 5>(lt); s[6] = window<K, 6>(lt); s[7] = window<K, 7>(lt);
    if constexpr (MODE == GEMV_SPLIT) {
#pragma unroll
        for (int j = 0; j < 8; j++) w[j] = hash_pair(s[j], cbc);
    } else if constexpr (FAM == FAM_HASH) {
#pragma unroll
        for (int j = 0; j < 4; j++) w[j] = hash_pair_rounded(s[2 * j], s[2 * j + 1], cbc);
    } else {
#pragma unroll
        for (int j = 0; j < 4; j++) w[j] = mul1_pair(s[2 * j], s[2 * j + 1], cbc);
    }
}

// MODE: GEMV_SPLIT / GEMV_PAIRED.  FAM: FAM_HASH / FAM_MUL1 (split implies hash).  MB: 8-row groups (1 or 2).
template <int K, int MODE, int FAM, int MB>
__global__ void __launch_bounds__(GEMV_THREADS, 1) gemv_kernel(const GemvLaunch p)
{
    constexpr int FW = gemv_frag_words(MODE);
    constexpr uint32_t W_BYTES = 2048u * K;
    extern __shared__ __align__(128) unsigned char smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty = full + GEMV_MAX_STAGES;
    int* flag = reinterpret_cast<int*>(smem + 2 * GEMV_MAX_STAGES * 8);          // [0] last-arriver flag, [1] abort
    float* P = reinterpret_cast<float*>(smem + 256);                              // [16][128]
    unsigned char* stage0 = smem + 256 + GEMV_MAX_ROWS * 128 * 4;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int cta = blockIdx.x;
    const long long u0 = gemv_first_unit(cta, p.units_q, p.units_r);
    const long long u1 = gemv_first_unit(cta + 1, p.units_q, p.units_r);
    const int rows = p.a.rows;

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; s++) {
            ptx::mbar_init(&full[s], 1);
            ptx::mbar_init(&empty[s], GEMV_CONSUMER_WARPS);
        }
        flag[0] = 0;
        flag[1] = 0;
        ptx::mbar_fence_init();
    }
    __syncthreads();

    if (warp == GEMV_CONSUMER_WARPS) {
        // ------------------------------------------------------------------ producer
        if (lane == 0) {
            int nb = (int)(u0 / p.KG), kg = (int)(u0 % p.KG);
            int shard = 0;
            while (shard < p.a.n_shards - 1 && nb >= p.a.shard_end_blocks[shard]) shard++;
            int it = 0;
            for (long long u = u0; u < u1; u++, it++) {
                const int s = it % p.stages;
                if (it >= p.stages) {
                    if (!ptx::mbar_wait(&empty[s], ((it / p.stages) & 1) ^ 1)) {
                        atomicExch(p.a.err, GEMV_ERR_EMPTY_WAIT);
                        break;
                    }
                }
                unsigned char* dst = stage0 + (size_t)s * p.stage_stride;
                ptx::mbar_arrive_expect_tx(&full[s], W_BYTES + p.xf_bytes);
                ptx::bulk_g2s(dst, p.a.packed + u * (512ll * K), W_BYTES, &full[s]);
                const uint32_t* xsrc = p.a.xf + shard * p.xf_shard_stride + (long long)kg * 8 * rows * 4 * FW;
                ptx::bulk_g2s(dst + W_BYTES, xsrc, p.xf_bytes, &full[s]);
                if (++kg == p.KG) {
                    kg = 0;
                    nb++;
                    while (shard < p.a.n_shards - 1 && nb >= p.a.shard_end_blocks[shard]) shard++;
                }
            }
        }
        return;
    }

    // ---------------------------------------------------------------------- consumers
    const int nt = warp & 7, kq = warp >> 3;
    const int g = lane >> 2, q = lane & 3;
    const CodebookConst cbc = {p.mul, p.add};
    float acc[MB][4];
#pragma unroll
    for (int mb = 0; mb < MB; mb++)
#pragma unroll
        for (int e = 0; e < 4; e++) acc[mb][e] = 0.f;

    const uint32_t stage0_addr = ptx::smem_addr(stage0);
    const uint32_t w_off = (uint32_t)((nt * 2 + kq) * K) * 128u + lane * 4u;
    bool row_ok[MB];
#pragma unroll
    for (int mb = 0; mb < MB; mb++) row_ok[mb] = (g + 8 * mb) < rows;

    int nb = (int)(u0 / p.KG), kg = (int)(u0 % p.KG);
    bool dirty = false;
    int it = 0;

    auto flush = [&](int fnb) {
        // acc -> P (the two k-halves of a column tile add up), then either finish the block here or hand the
        // partial sums to the workspace and let the last CTA to arrive finish it.
        ptx::named_bar_sync(1, GEMV_CONSUMER_WARPS * 32);
#pragma unroll
        for (int half = 0; half < 2; half++) {
            if (kq == half) {
#pragma unroll
                for (int mb = 0; mb < MB; mb++)
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        int m = 8 * mb + 2 * q + (e & 1);
                        int col = nt * 16 + g + 8 * (e >> 1);
                        if (m < rows) {
                            float* dst = &P[m * 128 + col];
                            *dst = half == 0 ? acc[mb][e] : *dst + acc[mb][e];
                        }
                    }
            }
            ptx::named_bar_sync(1, GEMV_CONSUMER_WARPS * 32);
        }
        const long long ub = (long long)fnb * p.KG;
        const int c_first = gemv_cta_of_unit(ub, p.units_q, p.units_r);
        const int c_last = gemv_cta_of_unit(ub + p.KG - 1, p.units_q, p.units_r);
        const int tid = threadIdx.x;
        const int nelem = rows * 128;
        bool finish = true;
        if (c_first != c_last) {
            float* slot = p.a.partials + (size_t)(cta + fnb) * rows * 128;
            for (int e = tid; e < nelem; e += GEMV_CONSUMER_WARPS * 32) slot[e] = P[e];
            __threadfence();
            ptx::named_bar_sync(1, GEMV_CONSUMER_WARPS * 32);
            if (tid == 0) {
                int old = atomicAdd(&p.a.counters[fnb], 1);
                int last = (old == c_last - c_first);
                if (last) p.a.counters[fnb] = 0;          // leave the counter ready for the next launch
                flag[0] = last;
            }
            ptx::named_bar_sync(1, GEMV_CONSUMER_WARPS * 32);
            finish = flag[0] != 0;
            if (finish) {
                __threadfence();
                for (int e = tid; e < nelem; e += GEMV_CONSUMER_WARPS * 32) {
                    float sum = 0.f;
                    for (int c = c_first; c <= c_last; c++) sum += __ldcg(p.a.partials + (size_t)(c + fnb) * rows * 128 + e);
                    P[e] = sum;
                }
            }
            ptx::named_bar_sync(1, GEMV_CONSUMER_WARPS * 32);
        }
        if (finish && warp < rows) {
            const int m = warp;
            float v[4];
#pragma unroll
            for (int e = 0; e < 4; e++) v[e] = P[m * 128 + 4 * lane + e];
            const long long o = (long long)m * p.a.n_total + fnb * 128 + 4 * lane;
            if (p.a.rotated) {
                __half h[4];
#pragma unroll
                for (int e = 0; e < 4; e++) h[e] = __float2half_rn(v[e]);
                *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(p.a.out) + o) = *reinterpret_cast<uint2*>(h);
            } else {
                fwht128(v[0], v[1], v[2], v[3], lane);
                const uint2 sv = *reinterpret_cast<const uint2*>(p.a.svh + fnb * 128 + 4 * lane);
                const __half2 s01 = *reinterpret_cast<const __half2*>(&sv.x), s23 = *reinterpret_cast<const __half2*>(&sv.y);
                v[0] *= HAD_SCALE * __low2float(s01);
                v[1] *= HAD_SCALE * __high2float(s01);
                v[2] *= HAD_SCALE * __low2float(s23);
                v[3] *= HAD_SCALE * __high2float(s23);
                if (p.a.out_dtype == EXL3_F32) {
                    *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.a.out) + o) = make_float4(v[0], v[1], v[2], v[3]);
                } else {
                    __half h[4];
#pragma unroll
                    for (int e = 0; e < 4; e++) h[e] = __float2half_rn(v[e]);
                    if (p.a.out_dtype == EXL3_BF16) {
                        __nv_bfloat16 b[4];
#pragma unroll
                        for (int e = 0; e < 4; e++) b[e] = __float2bfloat16_rn(__half2float(h[e]));
                        *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.a.out) + o) = *reinterpret_cast<uint2*>(b);
                    } else {
                        *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(p.a.out) + o) = *reinterpret_cast<uint2*>(h);
                    }
                }
            }
        }
#pragma unroll
        for (int mb = 0; mb < MB; mb++)
#pragma unroll
            for (int e = 0; e < 4; e++) acc[mb][e] = 0.f;
    };

    for (long long u = u0; u < u1; u++, it++) {
        const int s = it % p.stages;
        if (!ptx::mbar_wait(&full[s], (it / p.stages) & 1)) {
            // Give up on the data but keep the control flow of every warp identical, so nothing deadlocks.
            if (lane == 0) atomicExch(p.a.err, GEMV_ERR_FULL_WAIT);
        }
        const uint32_t sbase = stage0_addr + (uint32_t)s * p.stage_stride;
        uint32_t L[K];
#pragma unroll
        for (int i = 0; i < K; i++) L[i] = ptx::lds32(sbase + w_off + i * 128u);
        const uint32_t xbase = sbase + W_BYTES;

        auto tile = [&](auto tconst) {
            constexpr int T = decltype(tconst)::value;
            uint32_t own[2];
            own_words<K, T>(L, own);
            const uint32_t prev0 = __shfl_sync(0xFFFFFFFFu, own[0], (lane + 31) & 31);
            const LaneTile<K> lt = assemble<K>(own, prev0);
            uint32_t w[8];
            decode_tile_regs<K, MODE, FAM>(lt, cbc, w);
            const int ktl = kq * 4 + T;
#pragma unroll
            for (int mb = 0; mb < MB; mb++) {
                const uint32_t xaddr = xbase + (uint32_t)(((ktl * rows + g + 8 * mb) * 4 + q) * FW) * 4u;
                if constexpr (MODE == GEMV_SPLIT) {
                    uint4 b = make_uint4(0, 0, 0, 0);
                    if (row_ok[mb]) b = ptx::lds128(xaddr);
                    ptx::mma_m16n8k16(acc[mb], w[0], w[4], w[1], w[5], b.x, b.y);
                    ptx::mma_m16n8k16(acc[mb], w[2], w[6], w[3], w[7], b.z, b.w);
                } else {
                    uint2 b = make_uint2(0, 0);
                    if (row_ok[mb]) b = ptx::lds64(xaddr);
                    ptx::mma_m16n8k16(acc[mb], w[0], w[2], w[1], w[3], b.x, b.y);
                }
            }
        };
        tile(std::integral_constant<int, 0>{});
        tile(std::integral_constant<int, 1>{});
        tile(std::integral_constant<int, 2>{});
        tile(std::integral_constant<int, 3>{});

        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&empty[s]);
        dirty = true;
        if (++kg == p.KG) {
            flush(nb);
            dirty = false;
            kg = 0;
            nb++;
        }
    }
    if (dirty) flush(nb);
}

template <int K>
int launch_gemv_for_k(const GemvLaunch& l, cudaStream_t st);
template <int K>
int gemv_set_attributes_for_k(int max_smem);

}  // namespace exl3
