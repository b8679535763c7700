// Prefill GEMM of the EXL3 linear on the 5th-generation tensor cores (sm_100a): out = Xh @ W_inner for many rows,
// with the weights decoded from the resident trellis straight into the shared-memory operand of tcgen05.mma.
//
// The reference has no fused many-row kernel: it materialises the fp16 weight and calls a library GEMM
// (cuda/src/sglang_exl3/runtime/ops.py:36-59 of 0xSero/trellis-serve).  Here one persistent CTA per SM owns an output
// tile of 512 rows x 128 columns at a time and walks the reduction dimension in blocks of 64:
//
//   warps 0-7   decode: warp w decodes column tile w of the 64 x 128 weight block from the resident layout (register
//               level decode of exl3_decode.cuh, weights rounded to fp16 exactly as the reference decoder) and stores
//               it K-major, in 8x8 core matrices, as the B operand; after the main loop the same warps read the
//               accumulators back from tensor memory (tcgen05.ld) and store fp16 rows
//   warp 8      A producer: one 64 KB bulk async copy per stage; the rotated activations are laid out in global
//               memory by had_in_tc_kernel exactly as the A operand wants them (four 128 x 64 K-major tiles)
//   warp 9      allocates tensor memory (512 columns = four 128 x 128 fp32 accumulators), issues
//               tcgen05.mma.cta_group::1.kind::f16 (M 128, N 128, K 16) from one elected lane and commits to the
//               mbarriers that release the stage / publish the accumulators
//
// Each weight block is decoded once per 512 rows and reused by 16 MMAs, so the kernel is bound by the tensor pipe,
// not by the decode.  Every wait is bounded (exl3_ptx.cuh); on a time-out the error word is set and the control flow
// continues unchanged to the common exit, where tensor memory is released.
#include <cstring>

#include "exl3_internal.h"
#include "exl3_ptx.cuh"

namespace exl3 {

constexpr uint32_t TC_A_TILE_BYTES = 128 * TC_KB * 2;                 // 16 KB: one 128-row A tile of a reduction block

// Tilings of the output.  Narrow: MT x 128 rows by 128 columns (MT = 4 or 3 accumulators), 8 decode warps, 2 stages.  Wide:
// 256 rows x 256 columns (two accumulators of 256 columns), 16 decode warps, 3 stages: an MMA of N = 256 reads 12 KB of
// operands for twice the MACs of an N = 128 one (8 KB), which is what the shared-memory port of the SM can sustain.
template <int MT, bool WIDE>
struct TcTile {
    static_assert(!WIDE || MT == 2, "the wide tiling has two accumulators");
    static constexpr int M_TILES = MT;
    static constexpr int NCOLS = WIDE ? 256 : 128;
    static constexpr int NBLK = NCOLS / 128;                                  // column blocks of 128 per tile
    static constexpr int ROWS = 128 * M_TILES;
    static constexpr int STAGES = WIDE ? 3 : 2;
    static constexpr int DECODE_WARPS = 8 * NBLK;
    static constexpr int THREADS = (DECODE_WARPS + 2) * 32;
    static constexpr uint32_t A_STAGE_BYTES = TC_A_TILE_BYTES * M_TILES;
    static constexpr uint32_t B_STAGE_BYTES = NCOLS * TC_KB * 2;
    static constexpr uint32_t STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
    static constexpr size_t SMEM_BYTES = 1024 + (size_t)STAGES * STAGE_BYTES;
    static constexpr uint32_t B_LBO = (NCOLS / 8) * 128;                      // bytes between k chunks of the B block
    // kind::f16, fp16 x fp16 -> fp32, both operands K-major, M = 128, N = NCOLS
    static constexpr uint32_t IDESC = (1u << 4) | ((uint32_t)(NCOLS >> 3) << 17) | ((128u >> 4) << 24);
};

enum { TC_ERR_WAIT = 3 };
constexpr int TC_GROUPED_EPILOGUE_WARPS = 4;       // the grouped instances read their tiles out on warps of their own

struct GemmTcLaunch {
    const uint32_t* packed;      // resident weights [NB][KG][8][2][K][32]
    const __half* xa;            // rotated activations in A-operand layout [MS][k/64][4][8][16][8][8]
    __half* out;                 // [rows][n_total] fp16, rotated basis
    int* err;
    int rows, KG, NB, MS;        // MS = ceil(rows / 512): super tiles of the A layout
    int n_total;
    int shard_end_block[GEMV_MAX_SHARDS];
    int n_shards;
    long long xa_shard_stride;   // halves between shards
    uint32_t mul, add;
    int ksplit;                  // > 1: the reduction of every tile is cut into this many parts, each on its own CTA
    int tail_first;              // pair tiling: tiles before this one are not cut ...
    void* y;                     // ... and leave the kernel rotated: y[rows][n_total] = fp16 or bf16 of Had128(fp16(acc)) * svh
    const __half* svh;
    int y_bf16;
    float* part;                 //      which stores its fp32 accumulators into slab [part index][rows][n_total]
    long long part_slab;         //      floats per slab
    // Grouped (routed experts): work items come from a device-side list built after the routing alignment.  Item i =
    // (expert, first 128-row block, blocks of that expert in the item (1..TC_GROUPED_MT), unused); the weights of expert e start
    // expert_stride words after `packed`, rows are positions of the alignment (blocks of 128 rows of one expert).
    const int4* items;
    const int* n_items;
    long long expert_stride;
    Pow2 pw;
};

// Operand layout shared by A tiles and the B block: 8 x 8 fp16 core matrices of 128 contiguous bytes, core (c, j) =
// (k chunk of 8, row group of 8) at (c * groups + j) * 128 bytes: `lbo` = groups * 128 bytes between k chunks (2048 for a
// 128-row operand, 4096 for the 256-column B block), 128 between row groups.
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t smem_byte_addr, uint32_t lbo)
{
    uint64_t d = 0;
    d |= (uint64_t)((smem_byte_addr >> 4) & 0x3FFF);          // start address
    d |= (uint64_t)(lbo >> 4) << 16;                          // leading byte offset: between the two k chunks of an MMA
    d |= (uint64_t)(128 >> 4) << 32;                          // stride byte offset: between 8-row groups
    d |= 1ull << 46;                                          // descriptor version of this architecture
    return d;                                                 // layout type 0: no swizzle
}

__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(tmem_d),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void tc_commit(uint64_t* bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(ptx::smem_addr(bar)) : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// 16 x 16 tile T of a reduction block: the warp's 16 columns x k 16T..16T+15, decoded from the warp's K x 32 words into the
// B operand block at `bst`.  Pair j of a lane: k chunk 2T + (j & 1), column group cg0 + (j >> 1), row lane / 4 of the core
// matrix, bytes 4 (lane % 4) .. + 3.
template <int K, int FAM, int NCOLS, int T>
__device__ __forceinline__ void tc_decode_tile(const uint32_t (&L)[K], unsigned char* bst, int cg0, int lane, const CodebookConst& cbc, const Pow2& pw)
{
    uint32_t own[2];
    own_words<K, T>(L, own);
    const uint32_t prev0 = __shfl_sync(0xFFFFFFFFu, own[0], (lane + 31) & 31);
    const LaneRegs<K> R = lane_regs<K>(own, prev0);
    uint32_t st[8];
    st[0] = window_low<K, 0>(R, pw); st[1] = window_low<K, 1>(R, pw); st[2] = window_low<K, 2>(R, pw);
    st[3] = window_low<K, 3>(R, pw); st[4] = window_low<K, 4>(R, pw); st[5] = window_low<K, 5>(R, pw);
    st[6] = window_low<K, 6>(R, pw); st[7] = window_low<K, 7>(R, pw);
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; j++) w[j] = FAM == FAM_HASH ? hash_pair_rounded(st[2 * j], st[2 * j + 1], cbc) : mul1_pair(st[2 * j], st[2 * j + 1], cbc);
    const int g = lane >> 2, q = lane & 3;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const int c = 2 * T + (j & 1), jn = cg0 + (j >> 1);
        *reinterpret_cast<uint32_t*>(bst + (c * (NCOLS / 8) + jn) * 128 + g * 16 + q * 4) = w[j];
    }
}

// The warp's 16 columns of one reduction block (64 deep): four tiles.
template <int K, int FAM, int NCOLS>
__device__ __forceinline__ void tc_decode_block(const uint32_t (&L)[K], unsigned char* bst, int cg0, int lane, const CodebookConst& cbc, const Pow2& pw)
{
    tc_decode_tile<K, FAM, NCOLS, 0>(L, bst, cg0, lane, cbc, pw);
    tc_decode_tile<K, FAM, NCOLS, 1>(L, bst, cg0, lane, cbc, pw);
    tc_decode_tile<K, FAM, NCOLS, 2>(L, bst, cg0, lane, cbc, pw);
    tc_decode_tile<K, FAM, NCOLS, 3>(L, bst, cg0, lane, cbc, pw);
}

// SPLIT: the reduction of a tile may be cut into p.ksplit parts (work items); without it the part count is the constant 1
// and the index arithmetic of the unsplit kernel folds away.
template <int K, int FAM, int MT_, bool WIDE, bool SPLIT, bool GROUPED = false>
__global__ void __launch_bounds__(TcTile<MT_, WIDE>::THREADS + (GROUPED ? TC_GROUPED_EPILOGUE_WARPS * 32 : 0), 1) gemm_tc_kernel(const GemmTcLaunch p)
{
    static_assert(!GROUPED || !SPLIT, "grouped work items carry whole reductions");
    using TT = TcTile<MT_, WIDE>;
    constexpr int DW = TT::DECODE_WARPS, STAGES = TT::STAGES;
    extern __shared__ __align__(1024) unsigned char smem[];
    uint64_t* a_full = reinterpret_cast<uint64_t*>(smem);            // [stages]
    uint64_t* b_full = a_full + STAGES;
    uint64_t* empty = b_full + STAGES;
    uint64_t* acc_full = empty + STAGES;
    uint64_t* acc_empty = acc_full + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 1);
    unsigned char* stage0 = smem + 1024;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            ptx::mbar_init(&a_full[s], 1);
            ptx::mbar_init(&b_full[s], DW);
            ptx::mbar_init(&empty[s], 1);
        }
        ptx::mbar_init(acc_full, 1);
        ptx::mbar_init(acc_empty, GROUPED ? TC_GROUPED_EPILOGUE_WARPS : DW);
        ptx::mbar_fence_init();
    }
    if (warp == DW + 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(ptx::smem_addr(tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if constexpr (GROUPED) ptx::grid_dependency_wait();      // the item list comes from the kernels ahead in the stream
    const int KB = p.KG * 2;                           // reduction blocks of 64
    const int MT = GROUPED ? 1 : (p.rows + TT::ROWS - 1) / TT::ROWS;   // row tiles
    const int NT = p.NB / TT::NBLK;                    // column tiles
    const int KS = SPLIT ? p.ksplit : 1;
    // work items: (tile, part of its reduction), part fastest; grouped: (item of the list, column tile), column fastest
    const long long n_tiles = GROUPED ? (long long)(*p.n_items) * NT : (long long)MT * NT * KS;
    auto kb_begin = [&](long long t) { return (int)((long long)KB * (t % KS) / KS); };
    auto kb_end = [&](long long t) { return (int)((long long)KB * (t % KS + 1) / KS); };
    bool failed = false;
    auto fail = [&]() {
        if (!failed) {
            failed = true;
            atomicExch(p.err, TC_ERR_WAIT);
        }
    };

    // Accumulators of a finished tile -> fp16 rows (or fp32 slabs of a split reduction).  `eq` = which of `ew` epilogue warps
    // this is: column group eq / 4 of ew / 4; a warp can only read the quarter warp % 4 of the tensor-memory lanes.
    auto epilogue = [&](int eq, int ew, int row0, int ct, int sp, int present, uint32_t acc_round) {
        const int cgroups = ew >> 2, ccols = TT::NCOLS / cgroups;
        if (!failed && !ptx::mbar_wait(acc_full, acc_round & 1)) fail();
        tc_fence_after();
        const int quarter = warp & 3, cgroup = eq >> 2;
#pragma unroll 1
        for (int mt = 0; mt < present; mt++) {
            const int row = row0 + mt * 128 + quarter * 32 + lane;
#pragma unroll 1
            for (int cc = 0; cc < ccols / 32; cc++) {
                const int col = cgroup * ccols + cc * 32;
                uint32_t r[32];
                tc_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(mt * TT::NCOLS + col), r);
                if (row < p.rows && KS > 1) {
                    // part of a split reduction: fp32 accumulators into this part's slab; the output rotation adds the slabs
                    float* dst = p.part + (size_t)sp * p.part_slab + (size_t)row * p.n_total + (size_t)ct * TT::NCOLS + col;
#pragma unroll
                    for (int v = 0; v < 32; v += 4)
                        *reinterpret_cast<uint4*>(dst + v) = make_uint4(r[v], r[v + 1], r[v + 2], r[v + 3]);
                } else if (GROUPED || row < p.rows) {
                    __half* dst = p.out + (size_t)row * p.n_total + (size_t)ct * TT::NCOLS + col;
#pragma unroll
                    for (int v = 0; v < 32; v += 8) {
                        uint4 o;
                        __half2 h0 = __floats2half2_rn(__uint_as_float(r[v]), __uint_as_float(r[v + 1]));
                        __half2 h1 = __floats2half2_rn(__uint_as_float(r[v + 2]), __uint_as_float(r[v + 3]));
                        __half2 h2 = __floats2half2_rn(__uint_as_float(r[v + 4]), __uint_as_float(r[v + 5]));
                        __half2 h3 = __floats2half2_rn(__uint_as_float(r[v + 6]), __uint_as_float(r[v + 7]));
                        o.x = *reinterpret_cast<uint32_t*>(&h0);
                        o.y = *reinterpret_cast<uint32_t*>(&h1);
                        o.z = *reinterpret_cast<uint32_t*>(&h2);
                        o.w = *reinterpret_cast<uint32_t*>(&h3);
                        *reinterpret_cast<uint4*>(dst + v) = o;
                    }
                }
            }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(acc_empty);
    };

    if (warp < DW) {
        // ------------------------------------------------------------------ decode + epilogue
        const int nt = warp & 7, nbh = warp >> 3;
        const CodebookConst cbc = {p.mul, p.add};
        uint32_t it = 0, acc_round = 0;
        // The warp's words of the next reduction block are requested one block ahead, so their L2 latency hides
        // behind the decode of the current block.
        // column block of a work item (64-bit divisions: once per work item, not per reduction block)
        auto block_of = [&](long long tile) { return (GROUPED ? (int)(tile % NT) : (int)((tile / KS) / MT)) * TT::NBLK + nbh; };
        auto base_of = [&](long long tile) {               // start of the tile's weight matrix
            if constexpr (GROUPED) return p.packed + (long long)p.items[tile / NT].x * p.expert_stride;
            else return p.packed;
        };
        auto words_ptr = [&](const uint32_t* base, int nb_, int kb) {
            return base + (((((long long)nb_ * p.KG + (kb >> 1)) * 8 + nt) * 2 + (kb & 1)) * K) * 32 + lane;
        };
        uint32_t Lnext[K];
        if ((long long)blockIdx.x < n_tiles) {
            const uint32_t* src = words_ptr(base_of(blockIdx.x), block_of(blockIdx.x), kb_begin(blockIdx.x));
#pragma unroll
            for (int i = 0; i < K; i++) Lnext[i] = __ldg(src + i * 32);
        }
        for (long long t = blockIdx.x; t < n_tiles; t += gridDim.x) {
            int ms = (int)((t / KS) % MT), ct = (int)((t / KS) / MT), row0, present = TT::M_TILES;
            const int sp = (int)(t % KS);
            if constexpr (GROUPED) {
                const int4 item = p.items[t / NT];
                ms = 0;
                ct = (int)(t % NT);
                row0 = item.y * 128;
                present = item.z;
            } else {
                row0 = ms * TT::ROWS;
            }
            const int kb0 = kb_begin(t), kb1 = kb_end(t);
            const long long t_next = t + gridDim.x;
            const uint32_t* base_cur = base_of(t);
            const uint32_t* base_next = t_next < n_tiles ? base_of(t_next) : p.packed;
            const int nb_cur = block_of(t), nb_next = t_next < n_tiles ? block_of(t_next) : 0;
            const int kb_next = t_next < n_tiles ? kb_begin(t_next) : 0;
            for (int kb = kb0; kb < kb1; kb++, it++) {
                const int s = it % STAGES;
                const uint32_t round = it / STAGES;
                uint32_t L[K];
#pragma unroll
                for (int i = 0; i < K; i++) L[i] = Lnext[i];
                {
                    const bool last = kb + 1 == kb1;
                    if (!last || t_next < n_tiles) {
                        const uint32_t* src = last ? words_ptr(base_next, nb_next, kb_next) : words_ptr(base_cur, nb_cur, kb + 1);
#pragma unroll
                        for (int i = 0; i < K; i++) Lnext[i] = __ldg(src + i * 32);
                    }
                }
                if (round > 0 && !failed && !ptx::mbar_wait(&empty[s], (round - 1) & 1)) fail();
                unsigned char* bst = stage0 + (size_t)s * TT::STAGE_BYTES + TT::A_STAGE_BYTES;
                tc_decode_block<K, FAM, TT::NCOLS>(L, bst, 2 * (8 * nbh + nt), lane, cbc, p.pw);
                fence_async_smem();                     // generic-proxy stores -> visible to the tensor core's reads
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&b_full[s]);
            }
            // Dense: the decode warps read out the tile themselves (each the 32 tensor-memory lanes of its quarter and 64 of
            // the tile's columns).  Grouped: warps of their own do, and these go on to the next item's weights.
            if constexpr (!GROUPED) epilogue(warp, DW, row0, ct, sp, present, acc_round);
            acc_round++;
        }
    } else if (warp == DW) {
        // ------------------------------------------------------------------ A producer
        if (lane == 0) {
            uint32_t it = 0;
            for (long long t = blockIdx.x; t < n_tiles; t += gridDim.x) {
                const int ms = (int)((t / KS) % MT), nb = (GROUPED ? (int)(t % NT) : (int)((t / KS) / MT)) * TT::NBLK;
                const int kb0 = kb_begin(t), kb1 = kb_end(t);
                int shard = 0;
                while (shard < p.n_shards - 1 && nb >= p.shard_end_block[shard]) shard++;
                // The A layout in global memory is in super tiles of 512 rows = four 128-row tiles of 16 KB per reduction
                // block; the tile's 128-row tiles are fetched one by one (a 384-row tile may straddle two super tiles, and
                // its last 128-row tiles may lie beyond the padded rows: those are not fetched, their products are never stored).
                int t128 = ms * TT::M_TILES;
                int present = p.MS * 4 - t128;
                if (present > TT::M_TILES) present = TT::M_TILES;
                if constexpr (GROUPED) {
                    const int4 item = p.items[t / NT];
                    t128 = item.y;
                    present = item.z;
                }
                for (int kb = kb0; kb < kb1; kb++, it++) {
                    const int s = it % STAGES;
                    const uint32_t round = it / STAGES;
                    if (round > 0 && !failed && !ptx::mbar_wait_relaxed(&empty[s], (round - 1) & 1)) fail();
                    ptx::mbar_arrive_expect_tx(&a_full[s], (uint32_t)present * TC_A_TILE_BYTES);
                    for (int mt = 0; mt < present; mt++) {
                        const int idx = t128 + mt;
                        const __half* src = p.xa + shard * p.xa_shard_stride + (((long long)(idx >> 2) * KB + kb) * 4 + (idx & 3)) * (TC_A_TILE_BYTES / 2);
                        ptx::bulk_g2s(stage0 + (size_t)s * TT::STAGE_BYTES + (size_t)mt * TC_A_TILE_BYTES, src, TC_A_TILE_BYTES, &a_full[s]);
                    }
                }
            }
        }
    } else if (GROUPED && warp >= DW + 2) {
        // ------------------------------------------------------------------ epilogue warps of the grouped instances: routed
        // experts' tiles are short (8 reduction blocks in a down projection), so reading a tile out while the next one
        // is being decoded matters
        uint32_t acc_round = 0;
        for (long long t = blockIdx.x; t < n_tiles; t += gridDim.x, acc_round++) {
            const int4 item = p.items[t / NT];
            epilogue(warp - (DW + 2), TC_GROUPED_EPILOGUE_WARPS, item.y * 128, (int)(t % NT), 0, item.z, acc_round);
        }
    } else if (warp == DW + 1) {
        // ------------------------------------------------------------------ MMA issue
        if (lane == 0) {
            uint32_t it = 0, acc_round = 0;
            for (long long t = blockIdx.x; t < n_tiles; t += gridDim.x) {
                if (acc_round > 0 && !failed && !ptx::mbar_wait(acc_empty, (acc_round - 1) & 1)) fail();
                tc_fence_after();
                const int kb0 = kb_begin(t), kb1 = kb_end(t);
                int present = TT::M_TILES;
                if constexpr (GROUPED) present = p.items[t / NT].z;
                for (int kb = kb0; kb < kb1; kb++, it++) {
                    const int s = it % STAGES;
                    const uint32_t round = it / STAGES;
                    if (!failed && !ptx::mbar_wait(&a_full[s], round & 1)) fail();
                    if (!failed && !ptx::mbar_wait(&b_full[s], round & 1)) fail();
                    tc_fence_after();
                    const uint32_t a_addr = ptx::smem_addr(stage0 + (size_t)s * TT::STAGE_BYTES);
                    const uint32_t b_addr = a_addr + TT::A_STAGE_BYTES;
#pragma unroll
                    for (int mt = 0; mt < TT::M_TILES; mt++)
#pragma unroll
                        for (int ks = 0; ks < TC_KB / 16; ks++)
                            if (!GROUPED || mt < present)
                                tc_mma(tmem_base + (uint32_t)(mt * TT::NCOLS), tc_smem_desc(a_addr + mt * TC_A_TILE_BYTES + ks * 4096, 2048),
                                   tc_smem_desc(b_addr + ks * 2 * TT::B_LBO, TT::B_LBO), TT::IDESC, (kb > kb0 || ks > 0) ? 1u : 0u);
                    tc_commit(&empty[s]);               // stage reusable once these MMAs have read it
                }
                tc_commit(acc_full);                    // accumulators complete
                acc_round++;
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == DW + 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

// ------------------------------------------------------------------------------------------------ CTA pairs
// Two CTAs of a cluster on neighbouring SMs work on one 512 x 256 output tile with 256 x 256 x 16 MMAs (cta_group::2): each
// CTA holds 128 rows of every MMA's A operand and accumulator and decodes 128 of the 256 columns of B; the tensor cores read
// the other half from the partner's shared memory.  Against the single-CTA 512 x 128 tile this halves the operand bytes an SM
// reads from shared memory per flop and the activation bytes it pulls from L2, at the same 512 rows per decoded weight.
struct TcPair {
    static constexpr int M_TILES = 2;                                        // 256-row MMAs stacked in a tile
    static constexpr int ROWS = 256 * M_TILES;
    static constexpr int STAGES = 3;
    static constexpr int DECODE_WARPS = 8;
    static constexpr int EPILOGUE_WARPS = 8;                                 // two per quarter of the tensor-memory lanes
    static constexpr int THREADS = (DECODE_WARPS + 2 + EPILOGUE_WARPS) * 32;
    static constexpr uint32_t A_STAGE_BYTES = TC_A_TILE_BYTES * M_TILES;    // this CTA's 128 rows of each MMA
    static constexpr uint32_t B_STAGE_BYTES = 128 * TC_KB * 2;              // this CTA's 128 columns
    static constexpr uint32_t STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
    // Output staging: per epilogue warp 32 rows x 128 fp16 columns, rows 16 bytes apart from a multiple of 128 so that the
    // lanes' 16-byte stores fall on different banks.
    static constexpr uint32_t OUT_PITCH = 128 * 2 + 16;
    static constexpr uint32_t OUT_WARP_BYTES = 32 * OUT_PITCH;
    static constexpr size_t SMEM_BYTES = 1024 + (size_t)STAGES * STAGE_BYTES + (size_t)EPILOGUE_WARPS * OUT_WARP_BYTES;
    static constexpr uint32_t B_LBO = (128 / 8) * 128;
    // fp16 x fp16 -> fp32, both operands K-major, N = 256, M = 256 over the pair
    static constexpr uint32_t IDESC = (1u << 4) | ((256u >> 3) << 17) | ((256u >> 4) << 24);
};

__device__ __forceinline__ void tc_mma_pair(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(tmem_d),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Arrives on the barrier at this shared-memory offset in both CTAs of the pair once the MMAs issued so far have completed.
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar)
{
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(ptx::smem_addr(bar)),
                 "h"((uint16_t)3)
                 : "memory");
}

// Launched as clusters of two CTAs.  Work items, dealt to the pairs in turn: the first p.tail_first tiles whole, then every
// remaining tile as p.ksplit parts of its reduction, so that the last wave of a tile count that does not divide by the
// pairs is short: its parts store fp32 accumulators, slab [(tile - tail_first) * ksplit + part][512][256], which the output
// rotation adds in part order.  Tile t = column tile t / row tiles, row tile t % row tiles.  Roles
// per CTA: 8 decode warps, an activation producer, a warp whose first lane issues the MMAs of the pair (rank 0) or reports
// this CTA's filled stages to rank 0 (rank 1), and 8 epilogue warps, so that the decode of the next tile fills the stages
// while a tile's accumulators are read out, rotated and sent.  Barriers sit at the same offsets in both CTAs; `empty` and
// `acc_full` are signalled in both by the tensor core, `peer_full` and `acc_empty` of rank 0 by threads of rank 1.
template <int K, int FAM>
__global__ void __launch_bounds__(TcPair::THREADS, 1) gemm_tc_pair_kernel(const GemmTcLaunch p)
{
    using TT = TcPair;
    constexpr int DW = TT::DECODE_WARPS, EW = TT::EPILOGUE_WARPS, STAGES = TT::STAGES;
    extern __shared__ __align__(1024) unsigned char smem[];
    uint64_t* a_full = reinterpret_cast<uint64_t*>(smem);            // [stages]
    uint64_t* b_full = a_full + STAGES;
    uint64_t* peer_full = b_full + STAGES;
    uint64_t* empty = peer_full + STAGES;
    uint64_t* acc_full = empty + STAGES;
    uint64_t* acc_empty = acc_full + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 1);
    unsigned char* stage0 = smem + 1024;
    unsigned char* out_stage = stage0 + (size_t)STAGES * TcPair::STAGE_BYTES;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = ptx::cluster_cta_rank();
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            ptx::mbar_init(&a_full[s], 1);
            ptx::mbar_init(&b_full[s], DW);
            ptx::mbar_init(&peer_full[s], 1);
            ptx::mbar_init(&empty[s], 1);
        }
        ptx::mbar_init(acc_full, 1);
        ptx::mbar_init(acc_empty, 2 * EW);
        ptx::mbar_fence_init();
    }
    if (warp == DW + 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(ptx::smem_addr(tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    ptx::cluster_sync_all();                           // the partner's barriers exist before anything arrives on them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int KB = p.KG * 2;                           // reduction blocks of 64
    const int MT = (p.rows + TT::ROWS - 1) / TT::ROWS; // row tiles
    const int NT = p.NB / 2;                           // column tiles
    const int KS = p.ksplit;
    const long long n_whole = p.tail_first;
    const long long n_tiles = n_whole + ((long long)MT * NT - n_whole) * KS;     // work items
    const long long first = blockIdx.x >> 1, step = gridDim.x >> 1;
    auto tile_of = [&](long long t) { return t < n_whole ? t : n_whole + (t - n_whole) / KS; };
    auto part_of = [&](long long t) { return t < n_whole ? 0 : (int)((t - n_whole) % KS); };
    auto kb_begin = [&](long long t) { return t < n_whole ? 0 : (int)((long long)KB * part_of(t) / KS); };
    auto kb_end = [&](long long t) { return t < n_whole ? KB : (int)((long long)KB * (part_of(t) + 1) / KS); };
    bool failed = false;
    auto fail = [&]() {
        if (!failed) {
            failed = true;
            atomicExch(p.err, TC_ERR_WAIT);
        }
    };

    if (warp < DW) {
        // ------------------------------------------------------------------ decode
        const int nt = warp;
        const CodebookConst cbc = {p.mul, p.add};
        uint32_t it = 0;
        auto block_of = [&](long long t) { return (int)(tile_of(t) / MT) * 2 + (int)rank; };
        auto words_ptr = [&](int nb_, int kb) {
            return p.packed + (((((long long)nb_ * p.KG + (kb >> 1)) * 8 + nt) * 2 + (kb & 1)) * K) * 32 + lane;
        };
        uint32_t Lnext[K];
        if (first < n_tiles) {
            const uint32_t* src = words_ptr(block_of(first), kb_begin(first));
#pragma unroll
            for (int i = 0; i < K; i++) Lnext[i] = __ldg(src + i * 32);
        }
        for (long long t = first; t < n_tiles; t += step) {
            const int kb0 = kb_begin(t), kb1 = kb_end(t);
            const long long t_next = t + step;
            const int nb_cur = block_of(t), nb_next = t_next < n_tiles ? block_of(t_next) : 0;
            const int kb_next = t_next < n_tiles ? kb_begin(t_next) : 0;
            for (int kb = kb0; kb < kb1; kb++, it++) {
                const int s = it % STAGES;
                const uint32_t round = it / STAGES;
                uint32_t L[K];
#pragma unroll
                for (int i = 0; i < K; i++) L[i] = Lnext[i];
                {
                    const bool last = kb + 1 == kb1;
                    if (!last || t_next < n_tiles) {
                        const uint32_t* src = last ? words_ptr(nb_next, kb_next) : words_ptr(nb_cur, kb + 1);
#pragma unroll
                        for (int i = 0; i < K; i++) Lnext[i] = __ldg(src + i * 32);
                    }
                }
                if (round > 0 && !failed && !ptx::mbar_wait(&empty[s], (round - 1) & 1)) fail();
                tc_decode_block<K, FAM, 128>(L, stage0 + (size_t)s * TT::STAGE_BYTES + TT::A_STAGE_BYTES, 2 * nt, lane, cbc, p.pw);
                fence_async_smem();                     // generic-proxy stores -> visible to the tensor cores' reads
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&b_full[s]);
            }
        }
    } else if (warp == DW) {
        // ------------------------------------------------------------------ activation producer: rows 128 rank .. + 127 of each MMA
        if (lane == 0) {
            uint32_t it = 0;
            for (long long t = first; t < n_tiles; t += step) {
                const int ms = (int)(tile_of(t) % MT), nb = (int)(tile_of(t) / MT) * 2;
                const int kb0 = kb_begin(t), kb1 = kb_end(t);
                int shard = 0;
                while (shard < p.n_shards - 1 && nb >= p.shard_end_block[shard]) shard++;
                for (int kb = kb0; kb < kb1; kb++, it++) {
                    const int s = it % STAGES;
                    const uint32_t round = it / STAGES;
                    if (round > 0 && !failed && !ptx::mbar_wait_relaxed(&empty[s], (round - 1) & 1)) fail();
                    ptx::mbar_arrive_expect_tx(&a_full[s], TT::A_STAGE_BYTES);
                    for (int mt = 0; mt < TT::M_TILES; mt++) {
                        // 128-row tile 2 mt + rank of the 512-row super tile ms
                        const __half* src = p.xa + shard * p.xa_shard_stride + (((long long)ms * KB + kb) * 4 + 2 * mt + (int)rank) * (TC_A_TILE_BYTES / 2);
                        ptx::bulk_g2s(stage0 + (size_t)s * TT::STAGE_BYTES + (size_t)mt * TC_A_TILE_BYTES, src, TC_A_TILE_BYTES, &a_full[s]);
                    }
                }
            }
            // The tensor core's last arrivals on `empty` land in this CTA's shared memory: seen before the CTA may leave.
            for (uint32_t j = it > (uint32_t)STAGES ? it - STAGES : 0; j < it; j++)
                if (!failed && !ptx::mbar_wait_relaxed(&empty[j % STAGES], (j / STAGES) & 1)) fail();
        }
    } else if (warp >= DW + 2) {
        // ------------------------------------------------------------------ epilogue
        const int quarter = warp & 3, cgroup = (warp - (DW + 2)) >> 2;
        unsigned char* slice = out_stage + (size_t)(warp - (DW + 2)) * TT::OUT_WARP_BYTES;
        unsigned char* my_row = slice + (size_t)lane * TT::OUT_PITCH;
        uint32_t acc_round = 0;
        for (long long t = first; t < n_tiles; t += step) {
            const long long tile = tile_of(t);
            const int ms = (int)(tile % MT), ct = (int)(tile / MT);
            // This CTA's 128 rows of both MMAs.  A warp reads the 32 tensor-memory lanes of its quarter and 128 of the tile's
            // 256 columns; a lane rounds its row to fp16 into the warp's staging slice, the warp applies the output rotation
            // and the svh vector there, and every lane sends its row's 256 bytes to y as one bulk copy.  Tensor memory is
            // handed back as soon as it has been read.  Parts of a cut tile store their fp32 accumulators directly.
            if (!failed && !ptx::mbar_wait(acc_full, acc_round & 1)) fail();
            tc_fence_after();
#pragma unroll 1
            for (int mt = 0; mt < TT::M_TILES; mt++) {
                const int row_in = mt * 256 + (int)rank * 128 + quarter * 32 + lane, row = ms * TT::ROWS + row_in;
                ptx::bulk_wait_read_all();              // the lane's previous copy has left its staging row ...
                __syncwarp();                           // ... and so has every other lane's (a row is rotated by four lanes)
#pragma unroll 1
                for (int cc = 0; cc < 4; cc++) {
                    const int col = cgroup * 128 + cc * 32;
                    uint32_t r[32];
                    tc_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(mt * 256 + col), r);
                    if (t >= n_whole) {
                        if (row < p.rows) {
                            float* dst = p.part + ((size_t)(tile - n_whole) * KS + part_of(t)) * (TT::ROWS * 256) + (size_t)row_in * 256 + col;
#pragma unroll
                            for (int v = 0; v < 32; v += 4)
                                *reinterpret_cast<uint4*>(dst + v) = make_uint4(r[v], r[v + 1], r[v + 2], r[v + 3]);
                        }
                    } else {
#pragma unroll
                        for (int v = 0; v < 32; v += 8) {
                            uint4 o;
                            __half2 h0 = __floats2half2_rn(__uint_as_float(r[v]), __uint_as_float(r[v + 1]));
                            __half2 h1 = __floats2half2_rn(__uint_as_float(r[v + 2]), __uint_as_float(r[v + 3]));
                            __half2 h2 = __floats2half2_rn(__uint_as_float(r[v + 4]), __uint_as_float(r[v + 5]));
                            __half2 h3 = __floats2half2_rn(__uint_as_float(r[v + 6]), __uint_as_float(r[v + 7]));
                            o.x = *reinterpret_cast<uint32_t*>(&h0);
                            o.y = *reinterpret_cast<uint32_t*>(&h1);
                            o.z = *reinterpret_cast<uint32_t*>(&h2);
                            o.w = *reinterpret_cast<uint32_t*>(&h3);
                            *reinterpret_cast<uint4*>(my_row + cc * 64 + v * 2) = o;
                        }
                    }
                }
                if (mt == TT::M_TILES - 1) {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        if (rank == 0) ptx::mbar_arrive(acc_empty);
                        else ptx::mbar_arrive_cluster(acc_empty, 0);
                    }
                }
                if (t < n_whole) {
                    // The warp's 32 rows x 128 columns are whole blocks of the output rotation: done here on the staged
                    // rows, eight rows at a time with four lanes per row (the arithmetic of had_out_kernel, same bits).
                    __syncwarp();
#pragma unroll 1
                    for (int pass = 0; pass < 4; pass++) {
                        __half* at = reinterpret_cast<__half*>(slice + (size_t)(pass * 8 + (lane >> 2)) * TT::OUT_PITCH) +
                                     32 * (lane & 3);
                        float v[32];
                        load_half32(at, v);
                        fwht128_quad(v, lane);
                        had_out_finish(v, p.svh, ct * 256 + cgroup * 128 + 32 * (lane & 3), at, 0, p.y_bf16);
                    }
                    fence_async_smem();                 // every lane's stores -> visible to the copy engine
                    __syncwarp();
                    if (row < p.rows) {
                        ptx::bulk_s2g(reinterpret_cast<uint16_t*>(p.y) + (size_t)row * p.n_total + (size_t)ct * 256 + cgroup * 128, my_row, 256);
                        ptx::bulk_commit();
                    }
                }
            }
            acc_round++;
        }
        ptx::bulk_wait_all();                           // the lane's output copies have completed
    } else if (lane == 0) {
        uint32_t it = 0, acc_round = 0;
        if (rank == 0) {
            // -------------------------------------------------------------- MMA issue for the pair
            for (long long t = first; t < n_tiles; t += step) {
                if (acc_round > 0 && !failed && !ptx::mbar_wait_cluster(acc_empty, (acc_round - 1) & 1)) fail();
                tc_fence_after();
                const int kb0 = kb_begin(t), kb1 = kb_end(t);
                for (int kb = kb0; kb < kb1; kb++, it++) {
                    const int s = it % STAGES;
                    const uint32_t round = it / STAGES;
                    if (!failed && !ptx::mbar_wait(&a_full[s], round & 1)) fail();
                    if (!failed && !ptx::mbar_wait(&b_full[s], round & 1)) fail();
                    if (!failed && !ptx::mbar_wait_cluster(&peer_full[s], round & 1)) fail();
                    tc_fence_after();
                    const uint32_t a_addr = ptx::smem_addr(stage0 + (size_t)s * TT::STAGE_BYTES);
                    const uint32_t b_addr = a_addr + TT::A_STAGE_BYTES;
#pragma unroll
                    for (int mt = 0; mt < TT::M_TILES; mt++)
#pragma unroll
                        for (int ks = 0; ks < TC_KB / 16; ks++)
                            tc_mma_pair(tmem_base + (uint32_t)(mt * 256), tc_smem_desc(a_addr + mt * TC_A_TILE_BYTES + ks * 4096, 2048),
                                        tc_smem_desc(b_addr + ks * 2 * TT::B_LBO, TT::B_LBO), TT::IDESC, (kb > kb0 || ks > 0) ? 1u : 0u);
                    tc_commit_pair(&empty[s]);          // the stage is reusable in both CTAs once these MMAs have read it
                }
                tc_commit_pair(acc_full);               // accumulators complete in both CTAs
                acc_round++;
            }
        } else {
            // -------------------------------------------------------------- this CTA's stages reported to rank 0
            for (long long t = first; t < n_tiles; t += step) {
                const int kb0 = kb_begin(t), kb1 = kb_end(t);
                for (int kb = kb0; kb < kb1; kb++, it++) {
                    const int s = it % STAGES;
                    const uint32_t round = it / STAGES;
                    if (!failed && !ptx::mbar_wait(&a_full[s], round & 1)) fail();
                    if (!failed && !ptx::mbar_wait(&b_full[s], round & 1)) fail();
                    ptx::mbar_arrive_cluster(&peer_full[s], 0);
                }
            }
        }
    }

    // Neither CTA may leave, nor free tensor memory, while its partner can still signal it or the pair's MMAs run.
    tc_fence_before();
    __syncthreads();
    ptx::cluster_sync_all();
    if (warp == DW + 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

// Rotated activations in the A-operand layout of gemm_tc_kernel.  One warp per (shard, group of 8 rows, 128-block), four lanes
// per row with 32 columns each (fwht128_quad): a lane's 32 results are four whole 16-byte core-matrix rows, and the eight
// lanes that share a column range fill a 128-byte core matrix.  Rows beyond `rows` inside the last group are written as
// zeros; those up to the next multiple of 512 must have been zero-filled by the caller.
constexpr int HAD_IN_TC_ROWS = 8;
__global__ void had_in_tc_kernel(const void* __restrict__ x, int x_bf16, const __half* __restrict__ suh, int shards, int rows, int k,
                                 __half* __restrict__ xa, long long shard_stride)
{
    const int lane = threadIdx.x & 31;
    const int kgs = k >> 7;
    const int groups = (rows + HAD_IN_TC_ROWS - 1) / HAD_IN_TC_ROWS;
    const long long item = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (long long)shards * groups * kgs) return;
    const int kg = (int)(item % kgs);
    const int row = (int)((item / kgs) % groups) * HAD_IN_TC_ROWS + (lane >> 2);
    const int s = (int)(item / ((long long)kgs * groups));
    const int col = kg * 128 + 32 * (lane & 3);
    float v[32];
    if (row < rows) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint4 raw = reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(x) + (long long)row * k + col)[i];
            const uint4 sraw = reinterpret_cast<const uint4*>(suh + (long long)s * k + col)[i];
            const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w}, sw[4] = {sraw.x, sraw.y, sraw.z, sraw.w};
#pragma unroll
            for (int j = 0; j < 4; j++) {
                float x0, x1;
                if (x_bf16) {
                    const __nv_bfloat162 bb = *reinterpret_cast<const __nv_bfloat162*>(&w[j]);
                    x0 = __half2float(__float2half_rn(__low2float(bb)));
                    x1 = __half2float(__float2half_rn(__high2float(bb)));
                } else {
                    const __half2 h = *reinterpret_cast<const __half2*>(&w[j]);
                    x0 = __low2float(h);
                    x1 = __high2float(h);
                }
                const __half2 sh = *reinterpret_cast<const __half2*>(&sw[j]);
                v[8 * i + 2 * j] = x0 * __low2float(sh);
                v[8 * i + 2 * j + 1] = x1 * __high2float(sh);
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < 32; i++) v[i] = 0.f;
    }
    fwht128_quad(v, lane);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const __half2 h = __floats2half2_rn(v[8 * i + 2 * j] * HAD_SCALE, v[8 * i + 2 * j + 1] * HAD_SCALE);
            o[j] = *reinterpret_cast<const uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(xa + s * shard_stride + tc_a_offset(row, col + 8 * i, kgs * 2)) = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

template <int K, int FAM, int MT, bool WIDE, bool SPLIT>
static int launch_tc_kernel(const GemmTcLaunch& l, int sm_count, cudaStream_t st)
{
    using TT = TcTile<MT, WIDE>;
    const long long work = (long long)((l.rows + TT::ROWS - 1) / TT::ROWS) * (l.NB / TT::NBLK) * l.ksplit;
    const int grid = work < sm_count ? (int)work : sm_count;
    gemm_tc_kernel<K, FAM, MT, WIDE, SPLIT><<<grid, TT::THREADS, TT::SMEM_BYTES, st>>>(l);
    return cuda_status(cudaGetLastError());
}

template <int K, int FAM, int MT, bool WIDE>
static int launch_tc_variant(const GemmTcLaunch& l, int sm_count, cudaStream_t st)
{
    return l.ksplit > 1 ? launch_tc_kernel<K, FAM, MT, WIDE, true>(l, sm_count, st) : launch_tc_kernel<K, FAM, MT, WIDE, false>(l, sm_count, st);
}

// CTA pairs that can be resident at once (clusters of two on neighbouring SMs); 0 until a device is initialised or when the
// query fails, which switches the pair tiling off.
static int g_tc_pairs = 0;

template <int K, int FAM>
static int launch_tc_pair(const GemmTcLaunch& l, cudaStream_t st)
{
    const long long tiles = (long long)((l.rows + TcPair::ROWS - 1) / TcPair::ROWS) * (l.NB / 2);
    const long long work = l.tail_first + (tiles - l.tail_first) * l.ksplit;
    const int pairs = work < g_tc_pairs ? (int)work : g_tc_pairs;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(TcPair::THREADS);
    cfg.dynamicSmemBytes = TcPair::SMEM_BYTES;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cuda_status(cudaLaunchKernelEx(&cfg, gemm_tc_pair_kernel<K, FAM>, l));
}

// tiling: 0 = 512 x 128, 1 = 256 x 256, 2 = 384 x 128, 3 = 512 x 256 on a CTA pair
template <int K, int FAM>
static int launch_tc_fam(const GemmTcLaunch& l, int tiling, int sm_count, cudaStream_t st)
{
    if (tiling == 3) return launch_tc_pair<K, FAM>(l, st);
    if (tiling == 1) return launch_tc_variant<K, FAM, 2, true>(l, sm_count, st);
    if (tiling == 2) return launch_tc_variant<K, FAM, 3, false>(l, sm_count, st);
    return launch_tc_variant<K, FAM, 4, false>(l, sm_count, st);
}

template <int K>
static int launch_tc_k(const GemmTcLaunch& l, int fam, int tiling, int sm_count, cudaStream_t st)
{
    return fam == FAM_HASH ? launch_tc_fam<K, FAM_HASH>(l, tiling, sm_count, st) : launch_tc_fam<K, FAM_MUL1>(l, tiling, sm_count, st);
}

// The opt-in to large dynamic shared memory is a per-device attribute of every kernel instance: set for all of them when a
// device is initialised (before any capture), never on the run path.
template <int K, int FAM, int MT, bool WIDE>
static int tc_set_attr_tile()
{
    using TT = TcTile<MT, WIDE>;
    int rc = cuda_status(cudaFuncSetAttribute(gemm_tc_kernel<K, FAM, MT, WIDE, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TT::SMEM_BYTES));
    if (rc == EXL3_OK)
        rc = cuda_status(cudaFuncSetAttribute(gemm_tc_kernel<K, FAM, MT, WIDE, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TT::SMEM_BYTES));
    return rc;
}

template <int K>
static int tc_set_attr_k()
{
    int rc = EXL3_OK;
    if (rc == EXL3_OK) rc = tc_set_attr_tile<K, FAM_HASH, 2, true>();
    if (rc == EXL3_OK) rc = tc_set_attr_tile<K, FAM_HASH, 3, false>();
    if (rc == EXL3_OK) rc = tc_set_attr_tile<K, FAM_HASH, 4, false>();
    if (rc == EXL3_OK) rc = tc_set_attr_tile<K, FAM_MUL1, 2, true>();
    if (rc == EXL3_OK) rc = tc_set_attr_tile<K, FAM_MUL1, 3, false>();
    if (rc == EXL3_OK) rc = tc_set_attr_tile<K, FAM_MUL1, 4, false>();
    using TN = TcTile<4, false>;
    if (rc == EXL3_OK)
        rc = cuda_status(cudaFuncSetAttribute(gemm_tc_kernel<K, FAM_HASH, 4, false, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TN::SMEM_BYTES));
    if (rc == EXL3_OK)
        rc = cuda_status(cudaFuncSetAttribute(gemm_tc_kernel<K, FAM_MUL1, 4, false, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TN::SMEM_BYTES));
    if (rc == EXL3_OK) rc = cuda_status(cudaFuncSetAttribute(gemm_tc_pair_kernel<K, FAM_HASH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TcPair::SMEM_BYTES));
    if (rc == EXL3_OK) rc = cuda_status(cudaFuncSetAttribute(gemm_tc_pair_kernel<K, FAM_MUL1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TcPair::SMEM_BYTES));
    using TG = TcTile<TC_GROUPED_MT, true>;
    if (rc == EXL3_OK)
        rc = cuda_status(cudaFuncSetAttribute(gemm_tc_kernel<K, FAM_HASH, TC_GROUPED_MT, true, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TG::SMEM_BYTES));
    if (rc == EXL3_OK)
        rc = cuda_status(cudaFuncSetAttribute(gemm_tc_kernel<K, FAM_MUL1, TC_GROUPED_MT, true, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TG::SMEM_BYTES));
    return rc;
}

int gemm_tc_init_device()
{
    int rc = tc_set_attr_k<2>();
    if (rc == EXL3_OK) rc = tc_set_attr_k<3>();
    if (rc == EXL3_OK) rc = tc_set_attr_k<4>();
    if (rc == EXL3_OK) rc = tc_set_attr_k<5>();
    if (rc == EXL3_OK) rc = tc_set_attr_k<6>();
    if (rc == EXL3_OK) rc = tc_set_attr_k<7>();
    if (rc == EXL3_OK) rc = tc_set_attr_k<8>();
    if (rc == EXL3_OK) {
        // How many clusters of two fit on the device at once (every instance has the same footprint).
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2);
        cfg.blockDim = dim3(TcPair::THREADS);
        cfg.dynamicSmemBytes = TcPair::SMEM_BYTES;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, gemm_tc_pair_kernel<4, FAM_HASH>, &cfg) != cudaSuccess) {
            cudaGetLastError();
            n = 0;
        }
        g_tc_pairs = n;
    }
    return rc;
}

int gemm_tc_pairs() { return g_tc_pairs; }

constexpr int TC_MAX_KSPLIT = 8;
constexpr int TC_PAIR_MAX_KSPLIT = 16;     // parts of a tile of the pair tiling's last wave
static int g_tc_ksplit = 0;           // 0 = choose; n >= 1 = at most n parts (1 switches the split off)
void gemm_tc_set_ksplit(int n) { g_tc_ksplit = n; }
static int g_tc_tiling = -1;          // -1 = choose; 0 = 512 x 128; 1 = 256 x 256 where the shape allows; 2 = 384 x 128; 3 = 512 x 256 on CTA pairs, same condition
void gemm_tc_set_tiling(int t) { g_tc_tiling = t; }

size_t gemm_tc_activation_bytes(int rows, int k, int shards)
{
    const size_t ms = (size_t)(rows + TC_ROWS - 1) / TC_ROWS;
    return (size_t)shards * ms * TC_ROWS * k * sizeof(__half);
}

// xa: gemm_tc_activation_bytes() of scratch.  out: [rows][n_total] fp16 in the rotated basis.
size_t gemm_tc_part_bytes(int rows, int n_total)
{
    // Slabs of a split reduction: parts x rows x n_total floats with parts * tiles <= SMs, so never more than this.
    const size_t want = (size_t)TC_MAX_KSPLIT * rows * n_total * sizeof(float);
    const size_t cap = (size_t)160 * 512 * 128 * sizeof(float);
    return want < cap ? want : cap;
}

int launch_gemm_tc(const void* x, int x_bf16, const __half* suh_cat, const uint32_t* packed, int K, int codebook, const int* shard_end_blocks,
                   int n_shards, int rows, int k, int n_total, __half* xa, __half* out, float* part, void* y, const __half* svh, int y_bf16, TcSplit* split_out, int* err,
                   cudaStream_t st)
{
    const DeviceInfo* d = current_device_info();
    if (!d) return EXL3_ERR_NOT_INITIALISED;
    GemmTcLaunch l;
    l.packed = packed;
    l.xa = xa;
    l.out = out;
    l.err = err;
    l.rows = rows;
    l.KG = k / 128;
    l.NB = n_total / 128;
    l.MS = (rows + TC_ROWS - 1) / TC_ROWS;
    l.n_total = n_total;
    l.n_shards = n_shards;
    for (int s = 0; s < GEMV_MAX_SHARDS; s++) l.shard_end_block[s] = shard_end_blocks[s];
    l.xa_shard_stride = (long long)l.MS * TC_ROWS * k;
    const CodebookConst c = codebook_const(codebook);
    l.mul = c.mul;
    l.add = c.add;
    l.pw = make_pow2();
    // Rows beyond `rows` inside the last 512-row super tile must read as zeros; with whole super tiles there are none.
    if (rows % TC_ROWS != 0)
        if (int rc = cuda_status(cudaMemsetAsync(xa, 0, gemm_tc_activation_bytes(rows, k, n_shards), st))) return rc;
    const long long items = (long long)n_shards * ((rows + HAD_IN_TC_ROWS - 1) / HAD_IN_TC_ROWS) * (k / 128);
    had_in_tc_kernel<<<(unsigned)((items + 7) / 8), 256, 0, st>>>(x, x_bf16, suh_cat, n_shards, rows, k, xa, l.xa_shard_stride);
    if (int rc = cuda_status(cudaGetLastError())) return rc;
    // Wide tiles (256 x 256) need column blocks that pair up inside every shard.  They halve the rows that share a decoded
    // weight block, which makes the decode the limiter at large row counts (measured: 823 against 851 TFLOP/s at 2048
    // rows), but they waste no rows when there are at most 256 (703 against 457 TFLOP/s): chosen only then.  Above that,
    // 384-row tiles are taken instead of 512-row ones when they finish in less time: cost = waves of tiles over the SMs x
    // rows per tile (160 tiles of 512 rows on 148 SMs are two waves; 240 tiles of 384 rows are two shorter ones).
    bool can_wide = (l.NB % 2) == 0;
    for (int s = 0; s < n_shards - 1; s++) can_wide = can_wide && (shard_end_blocks[s] % 2) == 0;
    // The CTA-pair tiling (512 x 256 on two SMs, same condition on the column blocks) shares a decoded block over 512 rows
    // like the narrow one but reads half the operand bytes per flop; when its tile count does not divide by the resident
    // pairs, the tiles of the last wave are cut along the reduction into parts that fill the pairs once (fp32 slabs per
    // tile, added by the output rotation): 80 tiles on 74 pairs are 1.08 waves instead of 2.
    const long long pair_tiles = (long long)((rows + TcPair::ROWS - 1) / TcPair::ROWS) * (l.NB / 2);
    long long pair_whole = pair_tiles, pair_parts = 1;
    if (g_tc_pairs > 0 && pair_tiles % g_tc_pairs != 0) {
        const long long rem = pair_tiles % g_tc_pairs;
        long long ks = g_tc_pairs / rem;
        if (ks > TC_PAIR_MAX_KSPLIT) ks = TC_PAIR_MAX_KSPLIT;
        if (ks > l.KG / 2) ks = l.KG / 2;                       // at least four reduction blocks per part
        while (ks > 1 && (size_t)rem * ks * TcPair::ROWS * 256 * sizeof(float) > gemm_tc_part_bytes(rows, n_total)) ks--;
        if (g_tc_ksplit >= 1 && ks > g_tc_ksplit) ks = g_tc_ksplit;
        if (part && ks > 1) {
            pair_parts = ks;
            pair_whole = pair_tiles - rem;
        }
    }
    int tiling = g_tc_tiling;
    if (tiling < 0) {
        auto cost = [&](int mt) {
            const long long tiles = (long long)((rows + 128 * mt - 1) / (128 * mt)) * l.NB;
            return (double)((tiles + d->sm_count - 1) / d->sm_count * mt);
        };
        tiling = rows <= 256 ? 1 : (cost(3) < cost(4) ? 2 : 0);
        if (rows > 256 && can_wide && g_tc_pairs > 0) {
            const double waves = pair_parts > 1 ? (double)(pair_whole / g_tc_pairs) + 1.0 / (double)pair_parts
                                                : (double)((pair_tiles + g_tc_pairs - 1) / g_tc_pairs);
            if (4.0 * waves <= (cost(3) < cost(4) ? cost(3) : cost(4))) tiling = 3;
        }
    }
    if ((tiling == 1 || tiling == 3) && !can_wide) tiling = 0;
    if (tiling == 3 && g_tc_pairs < 1) tiling = 0;
    l.part = part;
    l.part_slab = (long long)rows * n_total;
    l.tail_first = 0;
    if (tiling == 3) {
        l.ksplit = (int)pair_parts;
        l.tail_first = (int)pair_whole;
        l.y = y;
        l.svh = svh;
        l.y_bf16 = y_bf16;
        if (split_out) *split_out = TcSplit{l.ksplit, 1, l.tail_first, (rows + TcPair::ROWS - 1) / TcPair::ROWS};
    } else {
        // Few tiles (narrow outputs at small row counts) leave most SMs idle: the reduction of every tile is then cut into
        // parts that run on CTAs of their own and store fp32 slabs, which the output rotation adds in part order.
        const int tile_rows = tiling == 1 ? 256 : tiling == 2 ? 384 : 512;
        const long long tiles = (long long)((rows + tile_rows - 1) / tile_rows) * (l.NB / (tiling == 1 ? 2 : 1));
        long long parts = tiles > 0 ? d->sm_count / tiles : 1;
        if (parts > TC_MAX_KSPLIT) parts = TC_MAX_KSPLIT;
        if (parts > l.KG * 2) parts = l.KG * 2;
        while (parts > 1 && (size_t)parts * rows * n_total * sizeof(float) > gemm_tc_part_bytes(rows, n_total)) parts--;
        if (g_tc_ksplit >= 1 && parts > g_tc_ksplit) parts = g_tc_ksplit;
        l.ksplit = part && parts > 1 ? (int)parts : 1;
        if (split_out) *split_out = TcSplit{l.ksplit, 0, 0, 0};
    }
    const int fam = codebook_family(codebook);
    switch (K) {
        case 2: return launch_tc_k<2>(l, fam, tiling, d->sm_count, st);
        case 3: return launch_tc_k<3>(l, fam, tiling, d->sm_count, st);
        case 4: return launch_tc_k<4>(l, fam, tiling, d->sm_count, st);
        case 5: return launch_tc_k<5>(l, fam, tiling, d->sm_count, st);
        case 6: return launch_tc_k<6>(l, fam, tiling, d->sm_count, st);
        case 7: return launch_tc_k<7>(l, fam, tiling, d->sm_count, st);
        case 8: return launch_tc_k<8>(l, fam, tiling, d->sm_count, st);
    }
    return EXL3_ERR_UNSUPPORTED_K;
}

template <int K>
static int launch_tc_grouped_k(const GemmTcLaunch& l, int fam, bool wide, int sm_count, cudaStream_t st)
{
    if (!wide) {
        using TN = TcTile<4, false>;
        if (fam == FAM_HASH) gemm_tc_kernel<K, FAM_HASH, 4, false, false, true><<<sm_count, TN::THREADS + TC_GROUPED_EPILOGUE_WARPS * 32, TN::SMEM_BYTES, st>>>(l);
        else gemm_tc_kernel<K, FAM_MUL1, 4, false, false, true><<<sm_count, TN::THREADS + TC_GROUPED_EPILOGUE_WARPS * 32, TN::SMEM_BYTES, st>>>(l);
        return cuda_status(cudaGetLastError());
    }
    using TT = TcTile<TC_GROUPED_MT, true>;
    if (fam == FAM_HASH) gemm_tc_kernel<K, FAM_HASH, TC_GROUPED_MT, true, false, true><<<sm_count, TT::THREADS + TC_GROUPED_EPILOGUE_WARPS * 32, TT::SMEM_BYTES, st>>>(l);
    else gemm_tc_kernel<K, FAM_MUL1, TC_GROUPED_MT, true, false, true><<<sm_count, TT::THREADS + TC_GROUPED_EPILOGUE_WARPS * 32, TT::SMEM_BYTES, st>>>(l);
    return cuda_status(cudaGetLastError());
}

// Routed experts with many rows each: out[position, :] = xa[position, :] @ W_inner[expert of the position's block], for
// the work items of `items` (see GemmTcLaunch).  xa is in the A-operand layout over positions (blocks of 128 rows of one
// expert; padding rows may hold anything, a product row depends on its own row only), `cap512` positions per shard; out is
// [cap][n_total] fp16 in the rotated basis.  wide: the 256-column tiling with 16 decode warps and items of at most
// TC_GROUPED_MT blocks (column blocks must pair up inside every shard); otherwise 128-column tiles and items of at most 4
// blocks.
int launch_gemm_tc_grouped(const uint32_t* packed, long long expert_stride, int K, int codebook, const int* shard_end_blocks, int n_shards,
                           int k, int n_total, const __half* xa, int cap512, __half* out, const int4* items, const int* n_items, bool wide,
                           int* err, cudaStream_t st)
{
    const DeviceInfo* d = current_device_info();
    if (!d) return EXL3_ERR_NOT_INITIALISED;
    GemmTcLaunch l;
    memset(&l, 0, sizeof(l));
    l.packed = packed;
    l.expert_stride = expert_stride;
    l.xa = xa;
    l.out = out;
    l.err = err;
    l.rows = cap512;
    l.KG = k / 128;
    l.NB = n_total / 128;
    l.MS = cap512 / TC_ROWS;
    l.n_total = n_total;
    l.n_shards = n_shards;
    for (int s = 0; s < GEMV_MAX_SHARDS; s++) l.shard_end_block[s] = shard_end_blocks[s];
    l.xa_shard_stride = (long long)cap512 * k;
    const CodebookConst c = codebook_const(codebook);
    l.mul = c.mul;
    l.add = c.add;
    l.pw = make_pow2();
    l.ksplit = 1;
    l.items = items;
    l.n_items = n_items;
    const int fam = codebook_family(codebook);
    switch (K) {
        case 2: return launch_tc_grouped_k<2>(l, fam, wide, d->sm_count, st);
        case 3: return launch_tc_grouped_k<3>(l, fam, wide, d->sm_count, st);
        case 4: return launch_tc_grouped_k<4>(l, fam, wide, d->sm_count, st);
        case 5: return launch_tc_grouped_k<5>(l, fam, wide, d->sm_count, st);
        case 6: return launch_tc_grouped_k<6>(l, fam, wide, d->sm_count, st);
        case 7: return launch_tc_grouped_k<7>(l, fam, wide, d->sm_count, st);
        case 8: return launch_tc_grouped_k<8>(l, fam, wide, d->sm_count, st);
    }
    return EXL3_ERR_UNSUPPORTED_K;
}

}  // namespace exl3
