// Internal declarations shared by the .cu files of libexl3_b200 (not part of the C ABI).
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cstdint>
#include <type_traits>

#include "../../include/exl3_b200.h"
#include "exl3_decode.cuh"

namespace exl3 {

// Records a CUDA runtime error for exl3_last_cuda_error() and maps it to a status.
int cuda_status(cudaError_t e);

struct DeviceInfo {
    bool ready = false;
    int sm_count = 0;
    int max_smem_optin = 0;
};
// State of the current device, or nullptr if exl3_init_device() has not run for it.
const DeviceInfo* current_device_info();

// exl3_kernels.cu
int launch_repack(const uint16_t* trellis, int k, int n, int K, uint32_t* packed, cudaStream_t st);
int launch_unpack(const uint32_t* packed, int k, int n, int K, uint16_t* trellis, cudaStream_t st);
int launch_reconstruct_stored(const uint16_t* trellis, int kt, int nt, int K, int cb, __half* w, cudaStream_t st);
int launch_reconstruct_packed(const uint32_t* packed, int k, int n, int K, int cb, __half* w, cudaStream_t st);
int launch_had_in(const void* x, int x_bf16, const __half* suh, int shards, int rows, int k, void* out, int mode, cudaStream_t st);
int launch_to_fragments(const __half* xh, int shards, int rows, int k, uint32_t* out, int mode, cudaStream_t st);
int launch_had_out(const void* y, int y_f32, const __half* svh, int rows, int n, void* out, long long out_stride, int out_bf16,
                   cudaStream_t st);

// exl3_gemv.cu -------------------------------------------------------------------------------------------

// How decoded weights enter the tensor-core product.
//   GEMV_SPLIT   hash codebooks: each weight occupies two k slots of the MMA as its two fp16 summands, the
//                activation is duplicated; the fp32 accumulator adds them exactly (no fp16 add, no packing).
//   GEMV_PAIRED  any codebook: weights are rounded to fp16 and packed two per register.
enum { GEMV_SPLIT = 0, GEMV_PAIRED = 1 };

constexpr int GEMV_MAX_ROWS = 16;          // rows per launch
constexpr int GEMV_MAX_GRID = 512;         // upper bound of persistent CTAs assumed when sizing workspaces
constexpr int GEMV_MAX_SHARDS = 4;

// Words per lane of one activation fragment (four k values of a 16-row tile) in each mode.
__host__ __device__ constexpr int gemv_frag_words(int mode) { return mode == GEMV_SPLIT ? 4 : 2; }

// Tensor-parallel exchange fused into the GEMV (row-parallel linears): peer regions laid out as for the one-shot
// all-reduce (256-byte header, then per call parity `world` slots of slot_bytes, 4 bytes per output element).
constexpr int TP_MAX_WORLD = 16;
constexpr int TP_HEADER_BYTES = 256;
struct TpExchange {
    unsigned char* base[TP_MAX_WORLD];   // every rank's region, mapped into this process
    int rank, world;                      // world <= 1: no exchange
    unsigned int slot_bytes;
    int* state;                           // [0] calls completed, [1] error word, [2] CTAs arrived in the running call
};

struct GemvArgs {
    const uint32_t* packed;     // resident weights, n-blocks of all shards concatenated
    const uint32_t* xf;         // activation fragments [shard][k/16][rows][4][frag_words]
    const void* x;              // in-kernel rotation (rows <= 2): raw activations [rows, k], else nullptr
    const __half* suh;          //   and the input sign vectors [n_shards][k]
    int x_bf16;
    int x_glu;                  // x is gate | up [rows, 2k]: the input is silu(gate) * up (a down projection's activation)
    // Normalised input (consumer side of a residual block, XR > 0): x is the residual stream z [rows, k], its sums of squares
    // per 128 columns are in ssq [rows, k/128] (written by the epilogue of the linear ahead or by the stats kernel), and the
    // input proper is z * rsqrt(mean square + eps) * norm_weight.
    const void* norm_weight;
    const float* ssq_in;
    float norm_eps;
    // Residual epilogue (producer side): the output block y is added to res_in, the sum z (rounded to the output type) goes to
    // res_out and its sum of squares per (row, 128 columns) to ssq_out [rows, n_total/128]; y itself is stored only if `out` is set.
    const void* res_in;
    void* res_out;
    float* ssq_out;
    int xf_staged;              // rows <= 2 without x: the fragments in xf are copied to shared memory once (bulk copies)
                                //   instead of being read from global memory tile by tile
    const __half* svh;          // [n_total]; unused when rotated
    void* out;                  // [rows, n_total]
    float* partials;            // [(grid + NB)][rows][128]
    int* counters;              // [NB], zero between launches
    int* err;                   // device error word
    int K, codebook, mode;
    int rows, k, n_total;
    int n_shards;
    int shard_end_blocks[GEMV_MAX_SHARDS];   // n-block index where shard s ends (last = NB)
    int out_dtype;              // EXL3_F16 / EXL3_BF16 / EXL3_F32 (fp32 only with the output Hadamard)
    int rotated;                // 1: store the rotated-basis product as fp16, no output Hadamard
    TpExchange tp;              // world > 1: the output is summed over the ranks inside the kernel
};

// Preferred mode for a codebook (split for the hash codebooks, paired for MUL1).
int gemv_default_mode(int codebook);
void gemv_set_mode_override(int mode);      // -1 = default; test / measurement knob
// With a.x set the GEMV rotates the input itself (no rotation launch ahead of it); gemv_rotates_input() tells whether
// that variant can serve the problem (row count, shared-memory budget) and launch_gemv() then requires it to.
bool gemv_rotates_input(const GemvArgs& a);
int launch_gemv(const GemvArgs& a, cudaStream_t st);
int gemv_init_device();

// exl3_moe.cu -------------------------------------------------------------------------------------------
struct MoeGemmLaunch;
int moe_init_device();
int launch_moe_align(const int* topk_ids, int numel, int E, int block, int cap, int* sorted_ids, int* expert_ids, int* num_post,
                     const int* expert_map, int E_global, cudaStream_t st);
int launch_moe_had_in(const void* x, int x_bf16, const __half* suh, int shards, int hidden, int top_k, int numel, int cap,
                      const int* sorted_ids, const int* expert_ids, const int* num_post, uint32_t* xf, int mode, cudaStream_t st);
int launch_moe_glu_had_in(const __half* gu, const __half* suh2, int inter, int numel, int cap, const int* sorted_ids,
                          const int* expert_ids, const int* num_post, uint32_t* xf, int mode, cudaStream_t st);
int launch_moe_combine(const __half* yd, const float* w, const int* topk_ids, int tokens, int top_k, int hidden, int E, void* y,
                       int y_bf16, cudaStream_t st);

// exl3_step.cu ------------------------------------------------------------------------------------------
int launch_rmsnorm_rotate(const void* x, void* residual, const void* weight, float eps, int bf16, const __half* suh, int shards, int rows,
                          int k, void* normed, uint32_t* xf, int mode, cudaStream_t st, void* residual_out = nullptr);
int launch_residual_ssq(const void* x, const void* res_in, int bf16, int rows, int k, void* res_out, float* ssq, cudaStream_t st);
int launch_silu_mul_rotate(const void* gu, int bf16, const __half* suh, int rows, int inter, void* act, uint32_t* xf, int mode,
                           cudaStream_t st);
size_t attention_scratch_bytes(int rows, int q_heads, int kv_heads, int t_max);
int attention_init_device();
int launch_rope_append(void* qkv, int bf16, int rows, int q_heads, int kv_heads, const float* cos_t, const float* sin_t, void* k_cache,
                       void* v_cache, int t_max, const int* pos, cudaStream_t st);
int launch_decode_attention(const void* qkv, int bf16, int rows, int q_heads, int kv_heads, void* k_cache, void* v_cache, int t_max,
                            const int* pos, float scale, const float* cos_t, const float* sin_t, float* part, void* out, const __half* suh,
                            uint32_t* xf, int mode, cudaStream_t st);

// exl3_gemm_tc.cu ---------------------------------------------------------------------------------------
// A-operand layout of the tensor-core GEMM in global memory: super tiles of TC_ROWS rows; per reduction block of TC_KB
// columns four 128-row tiles of 16 KB, each in 8 x 8 fp16 core matrices (k chunk of 8 outermost, then row group of 8).
constexpr int TC_ROWS = 512;
constexpr int TC_KB = 64;
// Element offset of (row, col) for a matrix of KB reduction blocks; the halves of an aligned group of 8 columns are contiguous.
__host__ __device__ inline long long tc_a_offset(int row, int col, int KB)
{
    const int kb = col >> 6, c = (col & 63) >> 3, e0 = col & 7;
    const int ms = row / TC_ROWS, mt = (row % TC_ROWS) >> 7, j = (row & 127) >> 3, rr = row & 7;
    return ((((((long long)ms * KB + kb) * 4 + mt) * 8 + c) * 16 + j) * 8 + rr) * 8 + e0;
}

// The grouped instances: the wide tiling where column blocks pair up inside every shard -- 16 decode warps on a 64 x 256 weight
// block per step (routed experts have few rows each, so the decode bounds the kernel and needs the warps), items of up to
// TC_GROUPED_MT blocks of 128 rows of one expert -- else 128-column tiles with 8 decode warps and items of up to 4 blocks.
constexpr int TC_GROUPED_MT = 2;
int launch_gemm_tc_grouped(const uint32_t* packed, long long expert_stride, int K, int codebook, const int* shard_end_blocks, int n_shards,
                           int k, int n_total, const __half* xa, int cap512, __half* out, const int4* items, const int* n_items, bool wide,
                           int* err, cudaStream_t st);
// exl3_moe_tc.cu: routed experts through the grouped tensor-core GEMM (many rows per expert)
constexpr int MOE_TC_BLOCK_ROWS = 128;
size_t moe_tc_capacity(int slots, int num_local);
size_t moe_tc_workspace_bytes(int slots, int num_local, int hidden, int inter);
int launch_moe_tc_experts(const void* x, int x_bf16, int top_k, int hidden, int inter, const int* topk_ids, int slots, int num_experts,
                          const int* expert_map, int num_local, const uint32_t* w13, const __half* suh13, const __half* svh13,
                          const uint32_t* w2, const __half* suh2, const __half* svh2, int K, int codebook, __half* yd, unsigned char* ws,
                          cudaStream_t st);
// How launch_gemm_tc left its result: !tile_slabs: parts == 1: fp16 in `out` in the rotated basis (launch_had_out), parts > 1:
// `parts` fp32 slabs [rows][n_total] (launch_had_out_sum); tile_slabs (the CTA-pair tiling): the 512 x 256 tiles before
// tail_first are final in y, the others are `parts` fp32 slabs per tile (launch_had_out_tiles; row_tiles = 512-row tiles per
// column tile; nothing left to do when parts == 1).
struct TcSplit {
    int parts, tile_slabs, tail_first, row_tiles;
};
int gemm_tc_init_device();
size_t gemm_tc_activation_bytes(int rows, int k, int shards);
void gemm_tc_set_tiling(int t);             // -1 = choose; 0 = 512 x 128 tiles; 1 = 256 x 256 tiles where the shape allows; 2 = 384 x 128 tiles; 3 = 512 x 256 on CTA pairs
int gemm_tc_pairs();                        // CTA pairs of the pair tiling that fit on the device at once (0 = tiling unavailable)
size_t gemm_tc_part_bytes(int rows, int n_total);
void gemm_tc_set_ksplit(int n);             // 0 = choose; n >= 1 = at most n parts of the reduction per tile
int launch_gemm_tc(const void* x, int x_bf16, const __half* suh_cat, const uint32_t* packed, int K, int codebook, const int* shard_end_blocks,
                   int n_shards, int rows, int k, int n_total, __half* xa, __half* out, float* part, void* y, const __half* svh, int y_bf16, TcSplit* split_out, int* err,
                   cudaStream_t st);
int launch_had_out_tiles(const float* part, int parts, int tail_first, int row_tiles, const __half* svh, int rows, int n, void* out,
                         int out_bf16, cudaStream_t st);
int launch_had_out_sum(const float* part, int parts, long long slab, const __half* svh, int rows, int n, void* out, int out_bf16,
                       cudaStream_t st);

// exl3_allreduce.cu -------------------------------------------------------------------------------------
size_t allreduce_region_bytes(size_t max_elems);
int launch_allreduce(void* data, int bf16, size_t n, void* const* peer_bases_host, int rank, int world, size_t max_elems, int* state,
                     cudaStream_t st);

// Launch with programmatic stream serialization: the kernel may become resident while the kernel ahead of it in the stream
// is still finishing.  Every kernel launched this way executes griddepcontrol.wait before it touches global memory that
// is not constant, and does so in every thread (also those that leave early), so completion stays ordered along the stream.
template <typename... KArgs, typename... Args>
inline int launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cuda_status(cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...));
}

// Every workspace starts with a 256-byte header (error word, zeros) and a counters region of FIXED size: the counters
// must read zero at the start of every launch whatever the shapes of the launches before it, so nothing else may ever be
// laid over them; the regions behind are scratch that each launch overwrites.
constexpr size_t WS_HEADER_BYTES = 256;
constexpr size_t WS_MAX_COUNTERS = 131072;                       // column blocks (dense) or moe block x column block pairs
constexpr size_t WS_SCRATCH_OFF = WS_HEADER_BYTES + WS_MAX_COUNTERS * sizeof(int);

// Workspace carved up identically by every entry point that takes one.
struct WorkspaceLayout {
    size_t err_off, counters_off, xf_off, partials_off, total;
};
WorkspaceLayout workspace_layout(int rows, int k, int n_total, int n_shards);

}  // namespace exl3
