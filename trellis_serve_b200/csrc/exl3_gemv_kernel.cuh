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
//   * a ring of shared-memory stages is fed with 1-D bulk async copies (TMA engine, mbarrier byte counting, no
//     multicast), one copy of several units per stage; there is no copy warp: the warp that is last to finish a stage
//     (a shared-memory counter tells it) issues the copy that refills it;
//   * 16 consumer warps; warp (nt, kq) owns column tile nt of the block and four of the unit's eight row tiles.
//     A lane reads K words, gets 16-K bits from its neighbour by one shuffle per tile, extracts its eight
//     16-bit states in registers and hashes them.  The resulting registers ARE the A operand of
//     mma.sync.m16n8k16 with the weights transposed (output columns as M, batch rows as N), so one tile costs
//     one MMA (paired) or two (split) whatever the row count up to 8;
//   * partial sums of a column block that several CTAs share go to a workspace; the CTA that arrives last
//     (atomic counter, no spinning) adds them in a fixed order, applies Had128 * svh and stores.  Results are
//     therefore deterministic.
#pragma once
#include "exl3_gemv_common.cuh"

namespace exl3 {

constexpr int GEMV_CONSUMER_WARPS = 16;
constexpr int GEMV_THREADS = GEMV_CONSUMER_WARPS * 32;             // no copy warp: 512 threads leave 64 registers each
constexpr int GEMV_MAX_STAGES = 12;
constexpr int GEMV_CTAS_PER_SM = 2;         // two resident CTAs per SM: twice the warps to hide instruction latency

struct GemvLaunch {
    GemvArgs a;
    unsigned long long* tl;     // measurement builds only: where this launch stamps its timeline
    int KG, NB, grid;
    int units_q, units_r;       // units per CTA: the first units_r CTAs take units_q + 1
    int stages;
    uint32_t stage_stride;      // bytes
    int units_per_stage;        // units covered by one bulk copy
    const void* zeros;          // at least 16 bytes of zeros in global memory
    uint32_t mul, add;
    long long xf_shard_stride;  // words between shards in xf
    uint32_t xs_off;            // in-kernel rotation only: byte offset of the fragment slots in shared memory
    Pow2 pw;                    // powers of two for the multiply that cuts a window out (constant bank)
};

// Largest row count whose input rotation the GEMV does itself (one launch per linear instead of two).
constexpr int GEMV_FUSED_ROWS = 2;
// Shared memory of the in-kernel rotation: a block of zeros (read by lanes whose batch row does not exist) followed by
// one slot of fragments per unit of the CTA.
constexpr uint32_t GEMV_XS_ZERO_BYTES = 512;
__host__ __device__ constexpr uint32_t gemv_xs_slot_bytes(int mode, int rows) { return 8u * rows * 4u * gemv_frag_words(mode) * 4u; }

// MODE: GEMV_SPLIT / GEMV_PAIRED.  FAM: FAM_HASH / FAM_MUL1 (split implies hash).  MB: 8-row groups (1 or 2).
// XR: 0 = activation fragments come from the workspace (written by the rotation kernel ahead of this launch);
//     1, 2 = that many rows, and the kernel rotates the input itself: before the main loop every consumer warp turns
//     x * suh of a few of the CTA's units into fragments in shared memory (one slot per unit, in unit order), so the
//     linear is ONE launch and the main loop reads its activations with immediate-offset shared loads.
// XIN: what the in-kernel rotation (XR > 0) reads -- 0: x as it is (or gate | up, a run-time flag); 1: the residual stream, which
// it normalises on the way in.  EPI: 1 = the epilogue adds the residual stream and writes the new one with its sums of squares.
// Both are instances of their own so that the code of the plain kernel stays as it is.
template <int K, int MODE, int FAM, int MB, int XR, int XIN = 0, int EPI = 0>
__global__ void __launch_bounds__(GEMV_THREADS, GEMV_CTAS_PER_SM) gemv_kernel(const __grid_constant__ GemvLaunch p)
{
    static_assert(XR == 0 || MB == 1, "in-kernel rotation serves one 8-row group");
    constexpr int FW = gemv_frag_words(MODE);
    constexpr uint32_t W_BYTES = 2048u * K;
    extern __shared__ __align__(128) unsigned char smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    int* released = reinterpret_cast<int*>(smem + GEMV_MAX_STAGES * 8);           // per stage: warps that are done with it
    int* flag = reinterpret_cast<int*>(smem + 2 * GEMV_MAX_STAGES * 8);          // [0] last-arriver flag, [1] abort
    uint64_t* xbar = reinterpret_cast<uint64_t*>(smem + 2 * GEMV_MAX_STAGES * 8 + 16);   // staged fragments have landed
    float* P = reinterpret_cast<float*>(smem + 256);                              // [16][128]
    unsigned char* stage0 = smem + 256 + GEMV_MAX_ROWS * 128 * 4;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int cta = blockIdx.x;
    const long long u0 = gemv_first_unit(cta, p.units_q, p.units_r);
    const long long u1 = gemv_first_unit(cta + 1, p.units_q, p.units_r);
    const int rows = p.a.rows;

    // One bulk copy per stage and stages of several units: the copy engine has a fixed cost of a few hundred nanoseconds
    // per bulk copy, so small copies cap the stream far below HBM speed.  The CTA's units are contiguous in memory, so
    // stage number j is simply units [u0 + j * ups, +ups) and lives in slot j % stages.
    const int ups = p.units_per_stage;
    const int n_fills = (int)((u1 - u0 + ups - 1) / ups);
    // Without the in-kernel rotation (XR == 0: three rows and more) the activation fragments of a stage's units travel with
    // its weights: [weights of ups units][fragments of ups units], F_BYTES of fragments per unit, copied from the fragment
    // buffer the rotation kernel ahead wrote (units of a column block are consecutive there) -- every fragment crosses the
    // L2 once per CTA instead of once per warp and tile.
    const uint32_t F_BYTES = XR == 0 ? gemv_xs_slot_bytes(MODE, rows) : 0u;
    auto issue_frags = [&](long long u, int n, int slot) {      // one thread, after the wait for the kernel ahead
        unsigned char* dst = stage0 + (size_t)slot * p.stage_stride + (size_t)ups * W_BYTES;
        while (n > 0) {
            const int unb = (int)(u / p.KG), ukg = (int)(u - (long long)unb * p.KG);
            int run = p.KG - ukg;
            if (run > n) run = n;
            int s = 0;
            while (s < p.a.n_shards - 1 && unb >= p.a.shard_end_blocks[s]) s++;
            ptx::bulk_g2s(dst, p.a.xf + s * p.xf_shard_stride + (long long)ukg * (F_BYTES / 4), (uint32_t)run * F_BYTES, &full[slot]);
            dst += (size_t)run * F_BYTES;
            u += run;
            n -= run;
        }
    };
    auto issue_fill = [&](int j, int slot, bool frags) {       // one thread: start the copy of stage number j into `slot`
        const long long u = u0 + (long long)j * ups;
        const long long left = u1 - u;
        const int n = (int)(left < ups ? left : ups);
        const uint32_t bytes = (uint32_t)n * W_BYTES;
        ptx::mbar_arrive_expect_tx(&full[slot], bytes + (uint32_t)n * F_BYTES);
        ptx::bulk_g2s(stage0 + (size_t)slot * p.stage_stride, p.a.packed + (long long)u * (512 * K), bytes, &full[slot]);
        if constexpr (XR == 0)
            if (frags) issue_frags(u, n, slot);
    };
    EXL3_STAMP(0);
    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; s++) {
            ptx::mbar_init(&full[s], 1);
            released[s] = 0;
        }
        flag[0] = 0;
        flag[1] = 0;
        if constexpr (XR > 0) ptx::mbar_init(xbar, 1);
        ptx::mbar_fence_init();
        // Weights are constants: the first lap of copies starts before the kernel ahead of this one has finished.
        for (int j = 0; j < p.stages && j < n_fills; j++) issue_fill(j, j, false);
    }
    __syncthreads();

    ptx::grid_launch_dependents();             // the next kernel in the stream may begin its prologue

    // ---------------------------------------------------------------------- consumers
    // Everything below reads or writes memory other kernels write (activations, workspace, output) and so comes after
    // the wait for the kernel ahead; with the in-kernel rotation the (constant) sign vectors are fetched before it.
    if constexpr (XR == 0) {
        ptx::grid_dependency_wait();
        EXL3_STAMP(1);
        if (threadIdx.x == 0) {                 // the fragments of the first lap follow their weights now that they exist
            reinterpret_cast<uint4*>(smem + 224)[0] = make_uint4(0u, 0u, 0u, 0u);      // read by lanes whose batch row does not exist
            for (int j = 0; j < p.stages && j < n_fills; j++) {
                const long long u = u0 + (long long)j * ups;
                const long long left = u1 - u;
                issue_frags(u, (int)(left < ups ? left : ups), j);
            }
        }
        __syncthreads();
    }
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
    int nb = (int)(u0 / p.KG), kg = (int)(u0 % p.KG);

    uint32_t tp_epoch = 0;                      // call number of the fused exchange; read once the kernel ahead has finished
    // P -> out for column block fnb: one warp per batch row applies Had128 * svh (or stores the rotated-basis product).
    auto epilogue = [&](int fnb) {
        if (warp < rows) {
            const int m = warp;
            float v[4];
#pragma unroll
            for (int e = 0; e < 4; e++) v[e] = P[m * 128 + 4 * lane + e];
            const long long o = (long long)m * p.a.n_total + fnb * 128 + 4 * lane;
            if (p.a.rotated && p.a.out_dtype == EXL3_F32) {
                *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.a.out) + o) = make_float4(v[0], v[1], v[2], v[3]);
            } else if (p.a.rotated) {
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
                if constexpr (EPI == 1) {
                    gemv_residual_store(p.a, tp_epoch, v, o, m, fnb, lane);
                } else if (p.a.out_dtype == EXL3_F32) {
                    *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.a.out) + o) = make_float4(v[0], v[1], v[2], v[3]);
                } else if (p.a.tp.world > 1) {
                    gemv_exchange_store(p.a.tp, tp_epoch, p.a.out_dtype == EXL3_BF16, v, o, reinterpret_cast<uint16_t*>(p.a.out), p.a.err);
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
    };

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
        bool finish = true;
        if (c_first != c_last) {
            const int tid = threadIdx.x;
            const int nelem = rows * 128;
            float* slot = p.a.partials + (size_t)(cta + fnb) * rows * 128;
            for (int e = tid; e < nelem; e += GEMV_CONSUMER_WARPS * 32) slot[e] = P[e];
            ptx::named_bar_sync(1, GEMV_CONSUMER_WARPS * 32);
            if (tid == 0) {
                // The barrier orders every thread's stores before this thread; its fence then publishes them all
                // (fences are cumulative) ahead of the counter update.
                __threadfence();
                int old = atomicAdd(&p.a.counters[fnb], 1);
                int last = (old == c_last - c_first);
                if (last) p.a.counters[fnb] = 0;          // leave the counter ready for the next launch
                flag[0] = last;
            }
            ptx::named_bar_sync(1, GEMV_CONSUMER_WARPS * 32);
            EXL3_STAMP(6);
            finish = flag[0] != 0;
            if (finish) {                                 // the last CTA to arrive adds up in a fixed order
                __threadfence();
                const float* base = p.a.partials + (size_t)fnb * nelem;
                for (int e = tid; e < nelem; e += GEMV_CONSUMER_WARPS * 32) {
                    // The additions keep their order either way.  Which form is faster was measured per instance family: the
                    // plain loop in the instances without producer or residual code (the compiler overlaps its loads by
                    // itself there; a column block cut 40 ways on a tensor-parallel shard showed the difference), four
                    // explicit loads in flight in the others (the 64-layer decode step: 8.46 against 8.64 ms).
                    float sum = 0.f;
                    int c = c_first;
                    if constexpr (XIN != 0 || EPI != 0) {
                        for (; c + 3 <= c_last; c += 4) {
                            const float a0 = __ldcg(base + (size_t)c * nelem + e), a1 = __ldcg(base + (size_t)(c + 1) * nelem + e);
                            const float a2 = __ldcg(base + (size_t)(c + 2) * nelem + e), a3 = __ldcg(base + (size_t)(c + 3) * nelem + e);
                            sum += a0;
                            sum += a1;
                            sum += a2;
                            sum += a3;
                        }
                    }
                    for (; c <= c_last; c++) sum += __ldcg(base + (size_t)c * nelem + e);
                    P[e] = sum;
                }
            }
            ptx::named_bar_sync(1, GEMV_CONSUMER_WARPS * 32);
        }
        if (finish) epilogue(fnb);
        if (finish) EXL3_STAMP(7);
#pragma unroll
        for (int mb = 0; mb < MB; mb++)
#pragma unroll
            for (int e = 0; e < 4; e++) acc[mb][e] = 0.f;
    };

    // Activation fragments.  Fragment elements are FW words: element index = (k-tile * rows + row) * 4 + q.  Lanes whose
    // batch row does not exist read a block of zeros instead, so no select is needed per tile.
    //   XR == 0: straight from global memory (they are tiny and stay in L1/L2), written by the kernel ahead;
    //   XR  > 0: from the shared-memory slots filled below, slot i = unit u0 + i.
    using Frag = typename std::conditional<FW == 4, uint4, uint2>::type;
    uint32_t f_lane[MB], f_tile[MB], f_unit[MB];      // XR == 0: byte offsets in a stage's fragment area: lane, per tile, per unit
    uint32_t xaddr = 0, xstep = 0;                    // XR > 0: shared address of the lane's fragments, bytes per unit
    constexpr uint32_t XS_TILE = (uint32_t)(XR > 0 ? XR : 1) * 4u * FW * 4u;      // bytes per 16-row tile in a slot
    constexpr uint32_t XS_SLOT = 8u * XS_TILE;
    if constexpr (XR == 0) {
#pragma unroll
        for (int mb = 0; mb < MB; mb++) {
            const bool ok = (g + 8 * mb) < rows;
            f_lane[mb] = ok ? (uint32_t)ups * W_BYTES + (uint32_t)((kq * 4 * rows + g + 8 * mb) * 4 + q) * FW * 4u : 0u;
            f_tile[mb] = ok ? (uint32_t)(rows * 4) * FW * 4u : 0u;
            f_unit[mb] = ok ? F_BYTES : 0u;
        }
    } else {
        unsigned char* xs = smem + p.xs_off;
        uint32_t* slots = reinterpret_cast<uint32_t*>(xs + GEMV_XS_ZERO_BYTES);
        if (threadIdx.x < GEMV_XS_ZERO_BYTES / 4) reinterpret_cast<uint32_t*>(xs)[threadIdx.x] = 0u;
        bool waited = false;
        if (p.a.xf_staged) {
            // The kernel ahead in the stream (a normalisation, an activation, a plain rotation) has written the fragments
            // of every (shard, row block) once; this CTA copies those of its units into its slots: units are consecutive
            // row blocks of a column block, so one bulk copy per column block touched.
            ptx::grid_dependency_wait();
            EXL3_STAMP(1);
            if (threadIdx.x == 0) {
                ptx::mbar_arrive_expect_tx(xbar, (uint32_t)(u1 - u0) * XS_SLOT);
                int u = (int)u0;
                while (u < (int)u1) {
                    const int unb = u / p.KG, ukg = u - unb * p.KG;
                    int n = p.KG - ukg;
                    if (n > (int)u1 - u) n = (int)u1 - u;
                    int s = 0;
                    while (s < p.a.n_shards - 1 && unb >= p.a.shard_end_blocks[s]) s++;
                    ptx::bulk_g2s(slots + (size_t)(u - (int)u0) * (XS_SLOT / 4), p.a.xf + s * p.xf_shard_stride + (long long)ukg * (XS_SLOT / 4),
                                  (uint32_t)n * XS_SLOT, xbar);
                    u += n;
                }
            }
            if (!ptx::mbar_wait(xbar, 0) && lane == 0) atomicExch(p.a.err, GEMV_ERR_FULL_WAIT);
            waited = true;
        } else {
        const int items = (int)(u1 - u0) * XR;
        const bool bf16 = p.a.x_bf16 != 0;
        float rstd[XR];
#pragma unroll
        for (int r = 0; r < XR; r++) rstd[r] = 1.f;
        constexpr int BATCH = 3;                      // rotations in flight per warp: their loads overlap
        for (int it0 = warp; it0 < items; it0 += GEMV_CONSUMER_WARPS * BATCH) {
            float v[BATCH][4];
            long long xi[BATCH];
#pragma unroll
            for (int b = 0; b < BATCH; b++) {
                const int it = it0 + GEMV_CONSUMER_WARPS * b;
                xi[b] = 0;
                if (it < items) {
                    const int i = it / XR, row = it % XR;
                    const long long u = u0 + i;
                    const int unb = (int)(u / p.KG), ukg = (int)(u - (long long)unb * p.KG);
                    int s = 0;
                    while (s < p.a.n_shards - 1 && unb >= p.a.shard_end_blocks[s]) s++;
                    const long long col = (long long)ukg * 128 + 4 * lane;
                    xi[b] = (long long)row * (p.a.x_glu ? 2 * p.a.k : p.a.k) + col;
#pragma unroll
                    for (int e = 0; e < 4; e++) v[b][e] = __half2float(p.a.suh[(long long)s * p.a.k + col + e]);
                }
            }
            if (!waited) {
                ptx::grid_dependency_wait();
                waited = true;
                EXL3_STAMP(1);
                if constexpr (XIN == 1) {
#pragma unroll
                    for (int r = 0; r < XR; r++)
                        if (r < rows) rstd[r] = gemv_row_rstd(p.a.ssq_in + (size_t)r * p.KG, p.KG, p.a.k, p.a.norm_eps, lane);
                }
            }
#pragma unroll
            for (int b = 0; b < BATCH; b++) {
                if (it0 + GEMV_CONSUMER_WARPS * b < items) {
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        if constexpr (XIN == 1) {
                            const int row = (it0 + GEMV_CONSUMER_WARPS * b) % XR;
                            v[b][e] *= gemv_load_norm(p.a.x, p.a.norm_weight, xi[b] + e, xi[b] + e - (long long)row * p.a.k,
                                                      XR > 1 && row == 1 ? rstd[XR - 1] : rstd[0], bf16);
                        } else {
                            v[b][e] *= p.a.x_glu ? gemv_load_glu(p.a.x, xi[b] + e, p.a.k, bf16) : gemv_load_x(p.a.x, xi[b] + e, bf16);
                        }
                    }
                }
            }
#pragma unroll
            for (int b = 0; b < BATCH; b++) {
                const int it = it0 + GEMV_CONSUMER_WARPS * b;
                if (it < items) {                     // warp-uniform: every lane takes part in the shuffles
                    const int i = it / XR, row = it % XR;
                    fwht128(v[b][0], v[b][1], v[b][2], v[b][3], lane);
                    // the lane holds tile-local rows r = 4*(lane&3) + e of 16-row tile lane/4 of the unit
                    uint32_t* o = slots + (size_t)i * (XS_SLOT / 4) + (size_t)((lane >> 2) * XR + row) * 4 * FW;
                    const int rbase = 4 * (lane & 3);
                    uint32_t hv[4];
#pragma unroll
                    for (int e = 0; e < 4; e++) hv[e] = __half_as_ushort(__float2half_rn(v[b][e] * HAD_SCALE));
                    if constexpr (MODE == GEMV_SPLIT) {
#pragma unroll
                        for (int e = 0; e < 4; e++) {
                            const int r = rbase + e;
                            o[((r & 7) >> 1) * 4 + (r & 1) + 2 * (r >> 3)] = hv[e] | (hv[e] << 16);
                        }
                    } else {
#pragma unroll
                        for (int e = 0; e < 4; e += 2) {
                            const int r = rbase + e;
                            o[((r & 7) >> 1) * 2 + (r >> 3)] = hv[e] | (hv[e + 1] << 16);
                        }
                    }
                }
            }
        }
        }
        if (!waited) ptx::grid_dependency_wait();
        ptx::named_bar_sync(1, GEMV_CONSUMER_WARPS * 32);
        EXL3_STAMP(2);
        const bool ok = g < XR;
        xaddr = ptx::smem_addr(xs) + (ok ? GEMV_XS_ZERO_BYTES + (uint32_t)(kq * 4 * XR + g) * 4u * FW * 4u + (uint32_t)q * FW * 4u : 0u);
        xstep = ok ? XS_SLOT : 0u;
    }
    if (p.a.tp.world > 1) tp_epoch = (uint32_t)*reinterpret_cast<volatile int*>(p.a.tp.state) + 1u;
    bool aborted = false;

    auto wait_stage = [&](int slot, uint32_t phase) {
        if (!aborted && !ptx::mbar_wait(&full[slot], phase)) {
            // Give up on the data but keep the control flow of every warp identical, so nothing deadlocks.
            aborted = true;
            if (lane == 0) atomicExch(p.a.err, GEMV_ERR_FULL_WAIT);
        }
    };

    int shard = 0;
    while (shard < p.a.n_shards - 1 && nb >= p.a.shard_end_blocks[shard]) shard++;
    // The main loop is cut into runs of units that end where something has to happen (stage used up, column block
    // finished, range finished); inside a run only two addresses advance: no division, no 64-bit arithmetic, no
    // bookkeeping per unit.
    int slot = 0, stage_left = ups, stage_no = 0;
    uint32_t phase = 0;
    uint32_t waddr = stage0_addr + w_off;
    uint32_t fx[MB];                                  // XR == 0: shared address of the lane's fragments of the current unit
    const uint32_t zero_addr = ptx::smem_addr(smem + 224);
    if constexpr (XR == 0) {
#pragma unroll
        for (int mb = 0; mb < MB; mb++) fx[mb] = f_unit[mb] ? stage0_addr + f_lane[mb] : zero_addr;
    }
    int remaining = (int)(u1 - u0);
    if (remaining > 0) wait_stage(0, 0);
    EXL3_STAMP(3);
    EXL3_STAMP_CLK(8);
    EXL3_STAMP_SM(10);

    while (remaining > 0) {
        int run = p.KG - kg;
        if (run > stage_left) run = stage_left;
        if (run > remaining) run = remaining;
        remaining -= run;
        stage_left -= run;
        kg += run;
#pragma unroll 1
        for (; run > 0; run--) {
            uint32_t L[K];
#pragma unroll
            for (int i = 0; i < K; i++) L[i] = ptx::lds32(waddr + i * 128u);
            // All activation fragments of the unit are requested up front so that their latency hides behind the decode.
            Frag bfrag[MB][4];
            if constexpr (XR == 0) {
#pragma unroll
                for (int mb = 0; mb < MB; mb++)
#pragma unroll
                    for (int T = 0; T < 4; T++) {
                        if constexpr (FW == 4) bfrag[mb][T] = ptx::lds128(fx[mb] + T * f_tile[mb]);
                        else bfrag[mb][T] = ptx::lds64(fx[mb] + T * f_tile[mb]);
                    }
            } else {
#pragma unroll
                for (int T = 0; T < 4; T++) {
                    if constexpr (FW == 4) bfrag[0][T] = ptx::lds128(xaddr + T * XS_TILE);
                    else bfrag[0][T] = ptx::lds64(xaddr + T * XS_TILE);
                }
            }

            auto tile = [&](auto tconst) {
                constexpr int T = decltype(tconst)::value;
                uint32_t own[2];
                own_words<K, T>(L, own);
                const uint32_t prev0 = __shfl_sync(0xFFFFFFFFu, own[0], (lane + 31) & 31);
                const LaneRegs<K> R = lane_regs<K>(own, prev0);
                uint32_t w[8];
                decode_tile_regs<K, MODE, FAM>(R, p.pw, cbc, w);
#pragma unroll
                for (int mb = 0; mb < MB; mb++) {
                    if constexpr (MODE == GEMV_SPLIT) {
                        const uint4 b = bfrag[mb][T];
                        ptx::mma_m16n8k16(acc[mb], w[0], w[4], w[1], w[5], b.x, b.y);
                        ptx::mma_m16n8k16(acc[mb], w[2], w[6], w[3], w[7], b.z, b.w);
                    } else {
                        const uint2 b = bfrag[mb][T];
                        ptx::mma_m16n8k16(acc[mb], w[0], w[2], w[1], w[3], b.x, b.y);
                    }
                }
            };
            tile(std::integral_constant<int, 0>{});
            tile(std::integral_constant<int, 1>{});
            tile(std::integral_constant<int, 2>{});
            tile(std::integral_constant<int, 3>{});

            waddr += W_BYTES;
            if constexpr (XR == 0) {
#pragma unroll
                for (int mb = 0; mb < MB; mb++) fx[mb] += f_unit[mb];
            } else {
                xaddr += xstep;
            }
        }
        if (stage_left == 0 || remaining == 0) {            // stage finished: hand it back, move to the next one
            __syncwarp();
            // The warp that is last to finish with the stage refills it (its reads and those of the warps counted before
            // it are ordered ahead of the copy by the acquire-release counter update).
            if (lane == 0 && ptx::atom_add_acq_rel_cta_shared(&released[slot], 1) == GEMV_CONSUMER_WARPS - 1) {
                released[slot] = 0;
                if (stage_no + p.stages < n_fills) issue_fill(stage_no + p.stages, slot, true);
            }
            stage_no++;
            stage_left = ups;
            if (++slot == p.stages) {
                slot = 0;
                phase ^= 1;
            }
            waddr = stage0_addr + (uint32_t)slot * p.stage_stride + w_off;
            if constexpr (XR == 0) {
#pragma unroll
                for (int mb = 0; mb < MB; mb++) fx[mb] = f_unit[mb] ? stage0_addr + (uint32_t)slot * p.stage_stride + f_lane[mb] : zero_addr;
            }
            if (remaining > 0) wait_stage(slot, phase);
        }
        if (kg == p.KG) {                                    // column block finished
            flush(nb);
            kg = 0;
            nb++;

        }
    }
    EXL3_STAMP(4);
    EXL3_STAMP_CLK(9);
    if (kg != 0 && u1 > u0) flush(nb);
    EXL3_STAMP(5);
    if (p.a.tp.world > 1) {
        // The call number moves on once every CTA of this launch has read it: the last CTA to get here bumps it.
        ptx::named_bar_sync(1, GEMV_CONSUMER_WARPS * 32);
        if (threadIdx.x == 0) {
            __threadfence();
            if (atomicAdd(&p.a.tp.state[2], 1) == (int)gridDim.x - 1) {
                p.a.tp.state[2] = 0;
                p.a.tp.state[0] = (int)tp_epoch;
            }
        }
    }
}

template <int K>
int launch_gemv_for_k(const GemvLaunch& l, size_t smem, cudaStream_t st);
template <int K>
int gemv_set_attributes_for_k(int max_smem);

}  // namespace exl3
