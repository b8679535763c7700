// Grouped decode GEMV for routed MoE experts (sm_100a).
//
// Every (token, expert) slot is its own GEMV row because every expert has its own suh
// (cuda/src/sglang_exl3/kernels/marlin_moe.py:11-13 of 0xSero/trellis-serve).  The routing step sorts the slots by
// expert into "moe blocks" of 8 rows of one expert (sorted ids, block expert ids, padded count: the contract of
// cuda/csrc/exl3_marlin_moe.cu:542-594); this kernel multiplies each block by its expert's matrix.  It replaces the
// reference's grouped Marlin instances (cuda/csrc/exl3_marlin_moe_template.h, launch at exl3_marlin_moe.cu:376-408).
//
// Same machinery as the dense decode GEMV (exl3_gemv_kernel.cuh): persistent CTAs that split the unit list
// (moe block, column block, row block) evenly and contiguously, a producer thread streaming weights through a ring of
// bulk-copy stages, 16 consumer warps decoding in registers into transposed m16n8k16 MMAs, split-k partial sums
// finished by the last CTA to arrive.  Differences: the number of blocks is read on the device (CUDA-graph safe), a
// stage never crosses a moe block (the next block is another expert's matrix), activation fragments always hold 8
// rows per block (padding rows are zero), the epilogue uses the expert's svh and scatters rows to their slots.
#pragma once
#include "exl3_gemv_common.cuh"

namespace exl3 {

constexpr int MOE_BLOCK_ROWS = 8;
constexpr int MOE_CONSUMER_WARPS = 16;
constexpr int MOE_THREADS = (MOE_CONSUMER_WARPS + 1) * 32;        // 16 decode warps and a copy warp
constexpr int MOE_MAX_STAGES = 12;
constexpr int MOE_CTAS_PER_SM = 2;
// Largest expert count of one routing alignment: its single CTA keeps three counters per expert in the default 48 KB of
// shared memory ((3 * E + 1) * 4 bytes + 132 static).
constexpr int MOE_MAX_EXPERTS = 4064;

struct MoeGemmLaunch {
    const uint32_t* packed;          // [E][NB][KG][...] resident expert stack
    long long expert_stride;         // words between experts
    const uint32_t* xf;              // fragments [shard][moe block][k/16][8][4][FW]
    long long xf_shard_stride;       // elements (of FW words) between shards
    const __half* svh;               // [E][n_total]
    __half* out;                     // [slots][n_total] fp16
    const int* sorted_ids;           // [blocks * 8] slot of each row, >= numel for padding
    const int* expert_ids;           // [blocks]
    const int* num_post;             // device: padded slot count = blocks * 8
    float* partials;
    int* counters;
    int* err;
    int KG, NB, n_total, numel, shard_end_block;   // shard_end_block: first column block of shard 1 (NB if one shard)
    int stages, units_per_stage;
    uint32_t stage_stride, mul, add;
    int rotated;                     // 1: no output Hadamard / svh (identity read-out)
    Pow2 pw;
};

int launch_moe_gemm(MoeGemmLaunch l, int K, int codebook, int mode, cudaStream_t st);

template <int K, int MODE, int FAM>
__global__ void __launch_bounds__(MOE_THREADS, MOE_CTAS_PER_SM) moe_gemm_kernel(const MoeGemmLaunch p)
{
    constexpr int FW = gemv_frag_words(MODE);
    constexpr uint32_t W_BYTES = 2048u * K;
    // Fragments of one unit (8 k-tiles x 8 rows x 4 lanes x FW words): they are copied into the stage behind its weights,
    // [weights of units_per_stage units][fragments of units_per_stage units], so a fragment crosses the L2 once per CTA.
    constexpr uint32_t F_BYTES = 8u * MOE_BLOCK_ROWS * 4u * FW * 4u;
    using Frag = typename std::conditional<FW == 4, uint4, uint2>::type;
    extern __shared__ __align__(128) unsigned char smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty = full + MOE_MAX_STAGES;
    int* flag = reinterpret_cast<int*>(smem + 2 * MOE_MAX_STAGES * 8);
    float* P = reinterpret_cast<float*>(smem + 256);                              // [8][128]
    unsigned char* stage0 = smem + 256 + GEMV_MAX_ROWS * 128 * 4;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int cta = blockIdx.x;
    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; s++) {
            ptx::mbar_init(&full[s], 1);
            ptx::mbar_init(&empty[s], MOE_CONSUMER_WARPS);
        }
        flag[0] = 0;
        ptx::mbar_fence_init();
    }
    __syncthreads();
    // The routing lists come from kernels ahead of this one in the stream: nothing is read before they have finished.
    ptx::grid_launch_dependents();
    ptx::grid_dependency_wait();
    const int UB = p.NB * p.KG;                                  // units per moe block
    const int nblocks = *p.num_post / MOE_BLOCK_ROWS;
    const long long total = (long long)nblocks * UB;
    const int units_q = (int)(total / gridDim.x), units_r = (int)(total % gridDim.x);
    const long long u0 = gemv_first_unit(cta, units_q, units_r);
    const long long u1 = gemv_first_unit(cta + 1, units_q, units_r);
    if (u0 >= u1) return;

    // position of the first unit: moe block, unit inside the block
    int b = (int)(u0 / UB);
    int in_blk = (int)(u0 - (long long)b * UB);

    if (warp == MOE_CONSUMER_WARPS) {
        // ------------------------------------------------------------------ producer
        if (lane == 0) {
            int s = 0;
            uint32_t wait_parity = 1;
            bool first_lap = true;
            long long left = u1 - u0;
            while (left > 0) {
                int n = p.units_per_stage;
                if (n > UB - in_blk) n = UB - in_blk;          // a stage never crosses into the next expert's matrix
                if (n > left) n = (int)left;
                if (!first_lap && !ptx::mbar_wait(&empty[s], wait_parity)) {
                    atomicExch(p.err, GEMV_ERR_EMPTY_WAIT);
                    break;
                }
                const int e = p.expert_ids[b];
                const uint32_t bytes = (uint32_t)n * W_BYTES;
                ptx::mbar_arrive_expect_tx(&full[s], bytes + (uint32_t)n * F_BYTES);
                ptx::bulk_g2s(stage0 + (size_t)s * p.stage_stride, p.packed + e * p.expert_stride + (long long)in_blk * (512ll * K), bytes,
                              &full[s]);
                {   // the units' fragments: consecutive row blocks of a column block are consecutive in the fragment buffer
                    unsigned char* dst = stage0 + (size_t)s * p.stage_stride + (size_t)p.units_per_stage * W_BYTES;
                    int at = in_blk, todo = n;
                    while (todo > 0) {
                        const int fnb = at / p.KG, fkg = at - fnb * p.KG;
                        int run = p.KG - fkg;
                        if (run > todo) run = todo;
                        const long long shard = fnb >= p.shard_end_block ? 1 : 0;
                        const uint32_t* src = p.xf + (shard * p.xf_shard_stride + ((long long)b * (p.KG * 8) + fkg * 8) * 32) * FW;
                        ptx::bulk_g2s(dst, src, (uint32_t)run * F_BYTES, &full[s]);
                        dst += (size_t)run * F_BYTES;
                        at += run;
                        todo -= run;
                    }
                }
                left -= n;
                in_blk += n;
                if (in_blk == UB) {
                    in_blk = 0;
                    b++;
                }
                if (++s == p.stages) {
                    s = 0;
                    if (first_lap) { first_lap = false; wait_parity = 0; } else wait_parity ^= 1;
                }
            }
        }
        return;
    }

    // ---------------------------------------------------------------------- consumers
    const int nt = warp & 7, kq = warp >> 3;
    const int g = lane >> 2, q = lane & 3;
    const CodebookConst cbc = {p.mul, p.add};
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    const uint32_t stage0_addr = ptx::smem_addr(stage0);
    const uint32_t w_off = (uint32_t)((nt * 2 + kq) * K) * 128u + lane * 4u;
    int nb = in_blk / p.KG, kg = in_blk - nb * p.KG;
    bool aborted = false;

    auto wait_stage = [&](int slot, uint32_t phase) {
        if (!aborted && !ptx::mbar_wait(&full[slot], phase)) {
            aborted = true;
            if (lane == 0) atomicExch(p.err, GEMV_ERR_FULL_WAIT);
        }
    };

    auto flush = [&]() {
        ptx::named_bar_sync(1, MOE_CONSUMER_WARPS * 32);
#pragma unroll
        for (int half = 0; half < 2; half++) {
            if (kq == half) {
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    float* dst = &P[(2 * q + (e & 1)) * 128 + nt * 16 + g + 8 * (e >> 1)];
                    *dst = half == 0 ? acc[e] : *dst + acc[e];
                }
            }
            ptx::named_bar_sync(1, MOE_CONSUMER_WARPS * 32);
        }
        const int gb = b * p.NB + nb;                           // global column block
        const long long ub = (long long)gb * p.KG;
        const int c_first = gemv_cta_of_unit(ub, units_q, units_r);
        const int c_last = gemv_cta_of_unit(ub + p.KG - 1, units_q, units_r);
        const int tid = threadIdx.x;
        constexpr int nelem = MOE_BLOCK_ROWS * 128;
        bool finish = true;
        if (c_first != c_last) {
            float* slot = p.partials + (size_t)(cta + gb) * nelem;
            for (int e = tid; e < nelem; e += MOE_CONSUMER_WARPS * 32) slot[e] = P[e];
            ptx::named_bar_sync(1, MOE_CONSUMER_WARPS * 32);
            if (tid == 0) {
                __threadfence();          // publishes every thread's stores (ordered before it by the barrier) ahead of the counter
                const int old = atomicAdd(&p.counters[gb], 1);
                const int last = (old == c_last - c_first);
                if (last) p.counters[gb] = 0;
                flag[0] = last;
            }
            ptx::named_bar_sync(1, MOE_CONSUMER_WARPS * 32);
            finish = flag[0] != 0;
            if (finish) {
                __threadfence();
                for (int e = tid; e < nelem; e += MOE_CONSUMER_WARPS * 32) {
                    float sum = 0.f;
                    for (int c = c_first; c <= c_last; c++) sum += __ldcg(p.partials + (size_t)(c + gb) * nelem + e);
                    P[e] = sum;
                }
            }
            ptx::named_bar_sync(1, MOE_CONSUMER_WARPS * 32);
        }
        if (finish && warp < MOE_BLOCK_ROWS) {
            const int slot_id = p.sorted_ids[b * MOE_BLOCK_ROWS + warp];
            if (slot_id >= 0 && slot_id < p.numel) {
                float v[4];
#pragma unroll
                for (int e = 0; e < 4; e++) v[e] = P[warp * 128 + 4 * lane + e];
                if (!p.rotated) {
                    fwht128(v[0], v[1], v[2], v[3], lane);
                    const int ex = p.expert_ids[b];
                    const uint2 sv = *reinterpret_cast<const uint2*>(p.svh + (size_t)ex * p.n_total + nb * 128 + 4 * lane);
                    const __half2 s01 = *reinterpret_cast<const __half2*>(&sv.x), s23 = *reinterpret_cast<const __half2*>(&sv.y);
                    v[0] *= HAD_SCALE * __low2float(s01);
                    v[1] *= HAD_SCALE * __high2float(s01);
                    v[2] *= HAD_SCALE * __low2float(s23);
                    v[3] *= HAD_SCALE * __high2float(s23);
                }
                __half h[4];
#pragma unroll
                for (int e = 0; e < 4; e++) h[e] = __float2half_rn(v[e]);
                *reinterpret_cast<uint2*>(p.out + (size_t)slot_id * p.n_total + nb * 128 + 4 * lane) = *reinterpret_cast<uint2*>(h);
            }
        }
#pragma unroll
        for (int e = 0; e < 4; e++) acc[e] = 0.f;
    };

    int slot = 0, in_stage = 0;
    uint32_t phase = 0;
    int left = (int)(u1 - u0);
    int stage_units = p.units_per_stage;
    if (stage_units > UB - in_blk) stage_units = UB - in_blk;
    if (stage_units > left) stage_units = left;
    uint32_t waddr = stage0_addr + w_off;
    const uint32_t f_off = (uint32_t)p.units_per_stage * W_BYTES + ((uint32_t)(g * 4 + q) + (uint32_t)(kq * 4) * 32u) * FW * 4u;
    uint32_t faddr = stage0_addr + f_off;
    bool dirty = false;
    wait_stage(0, 0);

    // Runs of units that end where something has to happen (stage used up, column block finished, range finished);
    // inside a run only the two read addresses advance.
    while (left > 0) {
        int run = p.KG - kg;
        if (run > stage_units - in_stage) run = stage_units - in_stage;
        if (run > left) run = left;
        left -= run;
        in_blk += run;
        in_stage += run;
        kg += run;
        dirty = true;
#pragma unroll 1
        for (; run > 0; run--) {
            uint32_t L[K];
#pragma unroll
            for (int i = 0; i < K; i++) L[i] = ptx::lds32(waddr + i * 128u);
            Frag bfrag[4];
#pragma unroll
            for (int T = 0; T < 4; T++) {
                if constexpr (FW == 4) bfrag[T] = ptx::lds128(faddr + T * 32u * FW * 4u);
                else bfrag[T] = ptx::lds64(faddr + T * 32u * FW * 4u);
            }

            auto tile = [&](auto tconst) {
                constexpr int T = decltype(tconst)::value;
                uint32_t own[2];
                own_words<K, T>(L, own);
                const uint32_t prev0 = __shfl_sync(0xFFFFFFFFu, own[0], (lane + 31) & 31);
                const LaneRegs<K> R = lane_regs<K>(own, prev0);
                uint32_t w[8];
                decode_tile_regs<K, MODE, FAM>(R, p.pw, cbc, w);
                if constexpr (MODE == GEMV_SPLIT) {
                    const uint4 bb = bfrag[T];
                    ptx::mma_m16n8k16(acc, w[0], w[4], w[1], w[5], bb.x, bb.y);
                    ptx::mma_m16n8k16(acc, w[2], w[6], w[3], w[7], bb.z, bb.w);
                } else {
                    const uint2 bb = bfrag[T];
                    ptx::mma_m16n8k16(acc, w[0], w[2], w[1], w[3], bb.x, bb.y);
                }
            };
            tile(std::integral_constant<int, 0>{});
            tile(std::integral_constant<int, 1>{});
            tile(std::integral_constant<int, 2>{});
            tile(std::integral_constant<int, 3>{});
            waddr += W_BYTES;
            faddr += F_BYTES;
        }
        const bool stage_done = in_stage == stage_units;
        if (stage_done) {
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&empty[slot]);
        }
        if (kg == p.KG) {                                        // column block of this moe block finished
            flush();
            dirty = false;
            kg = 0;
            if (++nb == p.NB) {                                  // next moe block: another expert, another 8 rows
                nb = 0;
                in_blk = 0;
                b++;
            }
        }
        if (stage_done && left > 0) {
            in_stage = 0;
            if (++slot == p.stages) {
                slot = 0;
                phase ^= 1;
            }
            stage_units = p.units_per_stage;
            if (stage_units > UB - in_blk) stage_units = UB - in_blk;
            if (stage_units > left) stage_units = left;
            waddr = stage0_addr + (uint32_t)slot * p.stage_stride + w_off;
            faddr = stage0_addr + (uint32_t)slot * p.stage_stride + f_off;
            wait_stage(slot, phase);
        }
    }
    if (dirty) flush();
}

}  // namespace exl3
