/*
 * exl3_b200 -- C ABI of the B200 (sm_100a) EXL3 quantized-linear kernels.
 *
 * This is the boundary a host plugin binds (ctypes, cffi, pybind, cgo ...).  It replaces the pybind/ATen
 * modules of 0xSero/trellis-serve, `trellis_exl3_kernels` (cuda/csrc/exl3_marlin.cu:562-585) and
 * `trellis_exl3_moe_kernels` (cuda/csrc/exl3_marlin_moe.cu:620-646).  Conventions:
 *
 *   - every pointer is a DEVICE pointer owned by the caller unless a comment says "host";
 *   - nothing here allocates device memory; scratch comes in through `workspace`;
 *   - every function returns a status (0 = ok); shape or argument errors are reported before any launch;
 *   - `stream` is a cudaStream_t passed as void*; launches are asynchronous on it;
 *   - tensors are contiguous; fp16 / bf16 are passed as raw 16-bit storage;
 *   - rows == 0 is a no-op that returns EXL3_OK (cuda/csrc/exl3_marlin.cu:499);
 *   - one host thread per device at a time (the reference's model: cuda/csrc/exl3_marlin.cu:84-100).
 *
 * EXL3 linear:  y = Had128( Had128(x * suh) @ W_inner ) * svh, W_inner decoded from the trellis
 * (core/src/trellis_core/reference.py:1-17, :145-153).
 */
#ifndef EXL3_B200_H
#define EXL3_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int exl3_status;

enum {
    EXL3_OK = 0,
    EXL3_ERR_BAD_SHAPE = 1,          /* k or n not a multiple of 128, negative sizes, shard ends out of order */
    EXL3_ERR_UNSUPPORTED_K = 2,      /* bits per weight outside 2..8 */
    EXL3_ERR_UNSUPPORTED_CODEBOOK = 3,
    EXL3_ERR_BAD_POINTER = 4,        /* null or misaligned pointer */
    EXL3_ERR_WORKSPACE = 5,          /* workspace missing or smaller than exl3_linear_workspace_bytes() */
    EXL3_ERR_CUDA = 6,               /* a CUDA runtime call failed; exl3_last_cuda_error() has the code */
    EXL3_ERR_DEVICE_WAIT = 7,        /* a bounded device-side wait gave up (reported by exl3_device_error) */
    EXL3_ERR_NOT_INITIALISED = 8,    /* exl3_init_device() was not called for the current device */
    EXL3_ERR_UNSUPPORTED_ROWS = 9,
    EXL3_ERR_UNSUPPORTED_DTYPE = 10,
    EXL3_ERR_STATIC_WORKSPACE = 11   /* exl3_linear_static: the problem needs more scratch than the built-in array holds */
};

enum { EXL3_CB_3INST = 0, EXL3_CB_MCG = 1, EXL3_CB_MUL1 = 2 };      /* core/src/trellis_core/reference.py:27 */
enum { EXL3_F16 = 0, EXL3_BF16 = 1, EXL3_F32 = 2 };

const char *exl3_status_str(exl3_status status);
int exl3_last_cuda_error(void);
int exl3_version(void);

/* Per-device state (SM count, kernel attributes).  Call once per device before any other entry point and
 * before any CUDA-graph capture.  Replaces init_device (cuda/csrc/exl3_marlin.cu:99-112, :537). */
exl3_status exl3_init_device(int device);
/* Multiprocessor count recorded by exl3_init_device for `device` (0 if it has not run): what the persistent grids and the
 * host's choice between the decode and the tensor-core kernel are sized by.  No counterpart in the reference. */
int exl3_device_sm_count(int device);

/* ---- resident layout ------------------------------------------------------------------------------------
 * Stored trellis: int16 [k/16, n/16, 16K].  Resident layout: uint32, same number of bytes, a permutation of
 * the stored bits.  Replaces repack_trellis / unpack_trellis (cuda/csrc/exl3_marlin.cu:344-408). */
size_t exl3_packed_bytes(int k, int n, int K);
exl3_status exl3_repack(const uint16_t *trellis, int k, int n, int K, uint32_t *packed, void *stream);
exl3_status exl3_unpack(const uint32_t *packed, int k, int n, int K, uint16_t *trellis, void *stream);

/* ---- decode to dense ------------------------------------------------------------------------------------
 * fp16 W_inner [k, n] row-major, bit-identical to reconstruct_inner (core/src/trellis_core/reference.py:102-115).
 * Stands in for exllamav3_ext.reconstruct (cuda/src/sglang_exl3/kernels/reference.py:71-80).
 * The stored form accepts any tile counts (k, n multiples of 16); the resident form needs multiples of 128. */
exl3_status exl3_reconstruct(const uint16_t *trellis, int k, int n, int K, int codebook, uint16_t *w_f16, void *stream);
exl3_status exl3_reconstruct_packed(const uint32_t *packed, int k, int n, int K, int codebook, uint16_t *w_f16,
                                    void *stream);

/* ---- Hadamard rotations ---------------------------------------------------------------------------------
 * xh[s*rows + r, :] = Had128(fp16(x[r, :]) * suh[s, :]), fp16, for every shard s.  suh may be NULL (no scale).
 * Replaces had_in_group_marlin (cuda/csrc/exl3_marlin.cu:283-290). */
exl3_status exl3_had_in(const void *x, int x_dtype, const uint16_t *suh, int shards, int rows, int k, uint16_t *xh,
                        void *stream);
/* out[r, j] = Had128(y[r, :])[j] * svh[j] for j < n, written with row stride out_stride (elements) so a fused
 * group can fill adjacent column spans.  y_dtype EXL3_F16 or EXL3_F32; out_dtype EXL3_F16 or EXL3_BF16.  y, out and svh are
 * 16-byte aligned and out_stride is a multiple of 8 (the kernel moves 16 bytes at a time).
 * Replaces had_out_into_marlin (cuda/csrc/exl3_marlin.cu:292-306). */
exl3_status exl3_had_out(const void *y, int y_dtype, const uint16_t *svh, int rows, int n, void *out, int64_t out_stride,
                         int out_dtype, void *stream);

/* ---- fused linear (decode path, any row count; rows are processed 16 at a time) -------------------------
 * One fused group: `n_shards` matrices that share the input x [rows, k] and write adjacent column spans of
 * y [rows, n_total].  packed = the matrices' resident layouts concatenated along n; suh_cat [n_shards, k];
 * svh_cat [n_total]; shard_ends (host, n_shards - 1 ints) = column where each matrix but the last ends,
 * multiples of 128.  x_dtype: EXL3_F16 or EXL3_BF16; y_dtype: EXL3_F16, EXL3_BF16 (the fp16 result converted) or
 * EXL3_F32 (the fp32 accumulators unrounded, for accuracy measurements).  y must be 16-byte aligned.
 * Replaces exl3_linear_marlin_out / exl3_linear_marlin_multi_out (cuda/csrc/exl3_marlin.cu:489-527).
 * packed, suh_cat and svh_cat are treated as constants: the kernel starts fetching them while the kernel ahead of it in the
 * stream is still running (programmatic dependent launch), so they must be complete (the work that wrote them finished, or
 * separated from this call by an event or a stream synchronisation) before the call is enqueued.  x and the workspace are
 * read only after the kernel ahead has finished, as usual.
 * The workspace must be zero-filled once after allocation; every call leaves it reusable, also by calls with other
 * shapes and by the MoE entry points: it starts with a 256-byte header and a fixed 512 KB of counters that every launch
 * leaves zero, and only scratch lies behind them (so n_total / 128, and for the MoE kernel moe blocks x column blocks,
 * may not exceed 131072: EXL3_ERR_BAD_SHAPE). */
size_t exl3_linear_workspace_bytes(int rows, int k, int n_total, int n_shards);
exl3_status exl3_linear(const void *x, int x_dtype, const uint32_t *packed, int K, int codebook, const uint16_t *suh_cat,
                        const uint16_t *svh_cat, const int *shard_ends, int n_shards, int rows, int k, int n_total, void *y,
                        int y_dtype, void *workspace, size_t workspace_bytes, void *stream);

/* ---- decode step: the kernels between the linears hand the next linear its rotated input ------------------------
 * In a decode step every EXL3 linear is preceded by an element-wise kernel (residual add + RMSNorm ahead of q|k|v and
 * gate|up, SiLU(gate) * up ahead of down, nothing but the rotation ahead of o).  These entry points fuse the linear's input
 * rotation into that kernel: it writes Had128(fp16(activation) * suh[s]) for every matrix s of the following fused group as
 * tensor-core fragments into `workspace`, once, and exl3_linear_prerotated runs the group from there (up to two rows its
 * CTAs copy the fragments of their units into shared memory with bulk copies; 3..16 rows read them tile by tile).  The
 * fragments, and so the results, are bit-identical to exl3_linear on the same activation.  rows <= 16; the workspace is the
 * one exl3_linear_workspace_bytes(rows, k, n_total, n_shards) sizes, shared by the whole chain in stream order.
 * The reference runs these steps as separate kernels ahead of had_in_group_marlin (cuda/csrc/exl3_marlin.cu:283-290,
 * group launch :507-527); the fusion has no counterpart there.
 *   exl3_rotate_fragments   activation x [rows, k] as it is.
 *   exl3_rmsnorm_rotate     residual (in/out, may be NULL) += x; a = rmsnorm(residual or x, eps) * weight, rounded to `dtype`;
 *                           `normed` (may be NULL) receives a.  x, residual, weight, normed share `dtype` (fp16 / bf16).
 *   exl3_silu_mul_rotate    a = silu(gate) * up of gate_up [rows, 2 * inter] (gate | up), rounded to `dtype`; `act` (may be
 *                           NULL) receives a [rows, inter].
 *   exl3_linear_prerotated  the fused group on those fragments; world > 1: row-parallel shard, summed over the ranks inside
 *                           the kernel as exl3_linear_allreduce does (peer arguments as there; world <= 1 ignores them). */
exl3_status exl3_rotate_fragments(const void *x, int x_dtype, const uint16_t *suh_cat, int n_shards, int rows, int k,
                                  int codebook, void *workspace, size_t workspace_bytes, void *stream);
exl3_status exl3_rmsnorm_rotate(const void *x, void *residual, const void *weight, float eps, int dtype,
                                const uint16_t *suh_cat, int n_shards, int rows, int k, int codebook, void *normed,
                                void *workspace, size_t workspace_bytes, void *stream);
exl3_status exl3_silu_mul_rotate(const void *gate_up, int dtype, const uint16_t *suh, int rows, int inter, int codebook,
                                 void *act, void *workspace, size_t workspace_bytes, void *stream);
exl3_status exl3_linear_prerotated(const uint32_t *packed, int K, int codebook, const uint16_t *svh_cat, const int *shard_ends,
                                   int n_shards, int rows, int k, int n_total, void *y, int y_dtype, void *workspace,
                                   size_t workspace_bytes, void *const *peer_regions, int rank, int world, size_t max_elems,
                                   int *state, const void *residual_in, void *residual_out, float *ssq_out, void *stream);

/* A down projection fed straight from the gate | up output: y = linear(fp16(silu(gate) * up)) with gate_up [rows, 2k] in
 * x_dtype, suh [k], n_shards = 1.  Up to two rows the activation is computed inside the GEMV's own input rotation (one launch,
 * no activation buffer); above that the library runs the activation kernel ahead of it.  Same bits as exl3_silu_mul_rotate
 * followed by exl3_linear_prerotated.  The exchange arguments are those of exl3_linear_prerotated (world <= 1: none).
 * The reference's engine runs its activation kernel between the two launches; no counterpart there.
 *
 * Residual stream carried by the linears (exl3_linear_prerotated and exl3_glu_linear, the row-parallel ends of a block):
 * with residual_in / residual_out / ssq_out set (all three or none) the epilogue adds the output block -- summed over the
 * ranks first, if there is an exchange -- to residual_in [rows, n_total], writes the sum, rounded to y_dtype, to residual_out
 * (a second buffer) and the sum of its squares per (row, 128 columns) to ssq_out [rows, n_total / 128]; y may then be NULL
 * (no exchange, up to two rows).  exl3_normed_linear is the consumer: the fused group on rmsnorm(z) * norm_weight, where z is
 * such a stream and ssq its sums of squares; up to two rows the GEMV normalises on the way into its own rotation, so a
 * transformer block is four launches plus attention.  exl3_residual_ssq starts a chain (z = x + residual_in, or x itself, and
 * its sums of squares); exl3_rmsnorm_linear = exl3_residual_ssq + exl3_normed_linear for a caller without a producer.
 * From three rows up the library runs its normalisation / stream kernels around a plain GEMV (y must then be given).
 * The reference's engine runs residual add and RMSNorm as kernels of its own ahead of had_in; no counterpart there. */
exl3_status exl3_glu_linear(const void *gate_up, int x_dtype, const uint32_t *packed, int K, int codebook, const uint16_t *suh,
                            const uint16_t *svh_cat, const int *shard_ends, int n_shards, int rows, int k, int n_total, void *y,
                            int y_dtype, void *workspace, size_t workspace_bytes, void *const *peer_regions, int rank, int world,
                            size_t max_elems, int *state, const void *residual_in, void *residual_out, float *ssq_out,
                            void *stream);
exl3_status exl3_residual_ssq(const void *x, const void *residual_in, int dtype, int rows, int k, void *residual_out, float *ssq,
                              void *stream);
exl3_status exl3_normed_linear(const void *z, int x_dtype, const float *ssq, const void *norm_weight, float eps,
                               const uint32_t *packed, int K, int codebook, const uint16_t *suh_cat, const uint16_t *svh_cat,
                               const int *shard_ends, int n_shards, int rows, int k, int n_total, void *y, int y_dtype,
                               void *workspace, size_t workspace_bytes, void *stream);
exl3_status exl3_rmsnorm_linear(const void *x, int x_dtype, const void *residual_in, void *residual_out, const void *norm_weight,
                                float eps, const uint32_t *packed, int K, int codebook, const uint16_t *suh_cat,
                                const uint16_t *svh_cat, const int *shard_ends, int n_shards, int rows, int k, int n_total, void *y,
                                int y_dtype, void *workspace, size_t workspace_bytes, void *stream);

/* The attention side of the same step (not quantized arithmetic; here so that a step is a handful of launches per layer):
 *   exl3_rope_append       qkv [rows, (q_heads + 2 kv_heads) * 128] holds q | k | v of one new token per row.  Rotary
 *                          embedding ("rotate half": pairs (i, i + 64)) with cos_table / sin_table [positions, 64] fp32 at
 *                          `*position` (device int, so a captured graph can move on): q in place, k into slot `*position` of
 *                          k_cache [rows, kv_heads, t_max, 128], v copied into v_cache.
 *   exl3_decode_attention  softmax(q k^T * scale) v over cache positions 0..*position for every query head (q_heads a
 *                          multiple of kv_heads, ratio 1, 2, 4, 5 or 8), split over the cache in chunks of 128 positions
 *                          and merged in a fixed order by the last CTA of each (row, KV head) to finish (one launch);
 *                          out [rows, q_heads * 128] in `dtype` (may be NULL).  scratch: exl3_attention_scratch_bytes(),
 *                          256-byte aligned, zero-filled once before its first use (an error word that exl3_device_error reads,
 *                          then arrival counters that every call leaves zero); exl3_init_device must have run.  suh_next != NULL: a head is one rotation block of the o
 *                          projection's input, so the merge also writes that linear's rotated fragments into `workspace`
 *                          (as exl3_rotate_fragments would from `out`) and exl3_linear_prerotated can follow directly.
 *   exl3_rope_decode_attention  the two above in one call and one launch: the attention kernel rotates
 *                          the queries as it loads them (qkv is left unrotated) and the warp that owns cache slot `*position`
 *                          rotates the new key into k_cache and copies the new value into v_cache before it reads them; same
 *                          roundings, same bits.  qkv must be 8-byte aligned.
 * Before it waits for the kernel ahead of it in the stream, an attention call reads `*position` and requests the cache rows
 * below it (like weights: they must be complete in memory before the call is enqueued behind this library's kernels; rows
 * written by earlier steps are), and walks through its merge code once on what the scratch buffer holds, storing nothing
 * (instruction-cache warm-up).  Row `*position` and qkv are read after the wait.
 * The reference leaves attention to its engine; no counterpart there. */
size_t exl3_attention_scratch_bytes(int rows, int q_heads, int kv_heads, int t_max);
exl3_status exl3_rope_append(void *qkv, int dtype, int rows, int q_heads, int kv_heads, int head_dim, const float *cos_table,
                             const float *sin_table, void *k_cache, void *v_cache, int t_max, const int *position,
                             void *stream);
exl3_status exl3_decode_attention(const void *qkv, int dtype, int rows, int q_heads, int kv_heads, int head_dim,
                                  const void *k_cache, const void *v_cache, int t_max, const int *position, float scale,
                                  void *scratch, size_t scratch_bytes, void *out, const uint16_t *suh_next, int codebook,
                                  void *workspace, size_t workspace_bytes, void *stream);
exl3_status exl3_rope_decode_attention(const void *qkv, int dtype, int rows, int q_heads, int kv_heads, int head_dim,
                                       const float *cos_table, const float *sin_table, void *k_cache, void *v_cache, int t_max,
                                       const int *position, float scale, void *scratch, size_t scratch_bytes, void *out,
                                       const uint16_t *suh_next, int codebook, void *workspace, size_t workspace_bytes,
                                       void *stream);

/* ---- fused linear for many rows (prefill) on the tcgen05 tensor cores -----------------------------------
 * Same contract as exl3_linear (fused group, dtypes, shard ends); built for hundreds to thousands of rows: the
 * weights are decoded once per 512 rows straight into the shared-memory operand of tcgen05.mma, accumulators live in
 * tensor memory; above 256 rows two CTAs of a cluster share a 512 x 256 tile (cta_group::2) and apply the output
 * rotation and svh inside their epilogue.  The reference has no fused many-row kernel; this replaces its decode +
 * library GEMM sequence `dense_group` (cuda/src/sglang_exl3/runtime/ops.py:36-59).  The workspace
 * (exl3_gemm_tc_workspace_bytes) holds the rotated activations, the rotated-basis product and the fp32 slabs of cut
 * reductions; its first 256 bytes must be zero (error word).  x, suh_cat, svh_cat and y must be 16-byte aligned. */
size_t exl3_gemm_tc_workspace_bytes(int rows, int k, int n_total, int n_shards);
exl3_status exl3_linear_tc(const void *x, int x_dtype, const uint32_t *packed, int K, int codebook, const uint16_t *suh_cat,
                           const uint16_t *svh_cat, const int *shard_ends, int n_shards, int rows, int k, int n_total, void *y,
                           int y_dtype, void *workspace, size_t workspace_bytes, void *stream);

/* The same fused linear for callers that can neither allocate device memory nor carry a workspace around: code
 * running inside another framework's captured or memory-pool-managed region, plugin hooks that only receive the
 * tensors of the call, hosts that hand out device memory once at start-up.  Its scratch is a fixed array of
 * EXL3_STATIC_WORKSPACE_BYTES that lives inside the library (every GPU that loads the library holds it until the
 * process exits); the entry point calls no cudaMalloc / cudaFree and no allocating library routine.
 *   - Problems whose scratch does not fit (see exl3_linear_workspace_bytes) are refused with EXL3_ERR_STATIC_WORKSPACE.
 *   - The first call on each device looks the array's device address up; make that first call before any stream
 *     capture on that device.
 *   - All calls on a device share the one array, which keeps what the previous call left there (the library keeps
 *     the parts that must be zero at zero).  Two calls that overlap on the GPU (different streams) race on it:
 *     keep calls to this entry point in one stream order per device.
 *   - A bounded device-side wait that gives up records its code in the array; exl3_device_error(NULL, 0, stream) reads and
 *     clears it for the current device (no allocation either).
 * Results are identical to exl3_linear.  No counterpart in the reference. */
#define EXL3_STATIC_WORKSPACE_BYTES (8u << 20)
exl3_status exl3_linear_static(const void *x, int x_dtype, const uint32_t *packed, int K, int codebook,
                               const uint16_t *suh_cat, const uint16_t *svh_cat, const int *shard_ends, int n_shards, int rows,
                               int k, int n_total, void *y, int y_dtype, void *stream);
size_t exl3_static_workspace_bytes(void);

/* Rotated-basis product without the Hadamards: out[r, :] = xh[s(col)*rows + r, :] @ W_inner, fp16 out.
 * Identity rows of xh read the decoded weights out exactly.  Replaces exl3_gemm_marlin / exl3_gemm_marlin_multi
 * (cuda/csrc/exl3_marlin.cu:410-487). */
exl3_status exl3_gemm_rotated(const uint16_t *xh, const uint32_t *packed, int K, int codebook, const int *shard_ends,
                              int n_shards, int rows, int k, int n_total, uint16_t *out, void *workspace,
                              size_t workspace_bytes, void *stream);
/* The same product with the fp32 accumulators stored unrounded: followed by exl3_had_out (y_dtype EXL3_F32) it is the
 * "output transform in a launch of its own" that the fused epilogue of exl3_linear must equal bit for bit, the check of
 * cuda/src/sglang_exl3/parity/marlin_parity.py:114-127. */
exl3_status exl3_gemm_rotated_f32(const uint16_t *xh, const uint32_t *packed, int K, int codebook, const int *shard_ends,
                                  int n_shards, int rows, int k, int n_total, float *out, void *workspace,
                                  size_t workspace_bytes, void *stream);

/* ---- tensor-parallel exchange step -------------------------------------------------------------------------
 * Row-parallel shards (o_proj, down_proj) produce partial sums (core/src/trellis_core/format/geometry.py:62-66); this
 * adds them over the ranks of one node, in place, with one latency-bound kernel over peer-mapped memory (ordinary peer
 * stores over NVLink of words tagged with the call number, polled for at the receiver; no multicast).  The reference itself has no collective (tensor parallelism is refused
 * at cuda/src/sglang_exl3/sglang_glue/linear.py:74-75).
 *   peer_regions (host array of `world` device pointers): every rank's symmetric region of
 *     exl3_allreduce_region_bytes(max_elems) bytes, zero-filled once, mapped into this process (peer_regions[rank] is
 *     this rank's own); state: 4 ints of this rank's device memory, zero-filled once (call counter, error word, ...).
 *   data: n fp16 / bf16 values (n % 8 == 0, n <= max_elems), summed in fp32 in rank order: every rank gets the same bits.
 * All ranks must make the same sequence of calls.  A peer that never arrives ends the bounded wait with a non-zero
 * state[1] instead of a hang. */
size_t exl3_allreduce_region_bytes(size_t max_elems);
/* exl3_linear with the exchange step inside the kernel, for row-parallel shards: the CTA that finishes a block of 128
 * output columns sends the rounded partial results straight to every peer and adds the peers' contributions as they
 * arrive, so no separate all-reduce launch follows the linear.  Same result bits as exl3_linear followed by
 * exl3_allreduce.  peer_regions / rank / world / max_elems as for exl3_allreduce (the two may share regions and state);
 * state: 4 ints, zero-filled once; y_dtype fp16 or bf16; min(rows, 16) * n_total <= max_elems.  A peer that never
 * arrives ends the bounded wait and exl3_device_error(workspace) reports it.  No counterpart in the reference. */
exl3_status exl3_linear_allreduce(const void *x, int x_dtype, const uint32_t *packed, int K, int codebook, const uint16_t *suh_cat,
                                  const uint16_t *svh_cat, const int *shard_ends, int n_shards, int rows, int k, int n_total,
                                  void *y, int y_dtype, void *workspace, size_t workspace_bytes, void *const *peer_regions, int rank,
                                  int world, size_t max_elems, int *state, void *stream);
exl3_status exl3_allreduce(void *data, int dtype, size_t n, void *const *peer_regions, int rank, int world, size_t max_elems,
                           int *state, void *stream);

/* ---- MoE layer (routed experts) ------------------------------------------------------------------------
 * One layer = align -> had_in (gate, up) -> grouped GEMV gate|up -> glu_had_in -> grouped GEMV down -> combine, the
 * launch structure of cuda/src/sglang_exl3/kernels/marlin_moe.py:272-294.  Slots are (token, k) pairs, slot = t*top_k+j.
 * Routing is consumed on the device (sorted_ids / expert_ids / num_post), so a captured CUDA graph replays with fresh
 * routing.  Blocks are 8 rows of one expert; padding rows carry slot id >= slots.
 *
 * exl3_moe_align       replaces moe_align_decode (cuda/csrc/exl3_marlin_moe.cu:542-594) and the engine's
 *                      moe_align_block_size: sorted_ids [cap] (padding = slots), expert_ids [cap/8] (-1 past the
 *                      end), num_post [1] = padded row count.  cap >= exl3_moe_sorted_capacity().  At most 4064
 *                      experts per alignment (EXL3_ERR_BAD_SHAPE beyond).  The later steps index the expert tensors
 *                      with these lists unchecked: pass only lists written by exl3_moe_align / exl3_moe_align_mapped.
 * exl3_moe_had_in      replaces moe_had_in (exl3_marlin_moe.cu:210-225): per position Had128(fp16(x[token]) * suh[e, s])
 *                      for `shards` input rotations (gate and up), written as MMA fragments.  suh is [E, shards, hidden].
 * exl3_moe_gemm        replaces moe_gemm (exl3_marlin_moe.cu:376-408): per moe block, rows @ W[e] -> Had128 * svh[e] ->
 *                      out[slot, :] fp16.  packed = [E] resident matrices; svh [E, n_total] (NULL: rotated basis, no
 *                      output transform); shard_end: first column fed by input rotation 1 (0 = single rotation).
 * exl3_moe_glu_had_in  replaces moe_glu_had_in (exl3_marlin_moe.cu:237-258): Had128(fp16(silu(g) * u) * suh2[e]);
 *                      gu is [slots, 2*inter] fp16 (gate | up).
 * exl3_moe_combine     replaces moe_combine (exl3_marlin_moe.cu:262-292): y[t] = sum_j w[t,j] * yd[t*top_k+j] in fp32,
 *                      slot order, one rounding; expert ids outside [0, E) are skipped.
 * The fragment buffers hold exl3_moe_fragment_bytes(); the GEMV workspace holds exl3_moe_workspace_bytes() and must be
 * zero-filled once. */
int exl3_moe_block_rows(void);
size_t exl3_moe_sorted_capacity(int slots, int num_experts);
exl3_status exl3_moe_align(const int32_t *topk_ids, int slots, int num_experts, int32_t *sorted_ids, int cap, int32_t *expert_ids,
                           int32_t *num_post, void *stream);
/* Alignment for one bitrate class of a mixed-K expert set (moe_align_decode with its expert_map list,
 * cuda/src/sglang_exl3/kernels/marlin_moe.py:195-213): expert_map is int32 [num_experts], global id -> id in
 * [0, num_local) or -1; slots of other classes are dropped, expert_ids come out local.  cap >=
 * exl3_moe_sorted_capacity(slots, num_local). */
exl3_status exl3_moe_align_mapped(const int32_t *topk_ids, int slots, int num_experts, const int32_t *expert_map, int num_local,
                                  int32_t *sorted_ids, int cap, int32_t *expert_ids, int32_t *num_post, void *stream);
size_t exl3_moe_fragment_bytes(int cap, int k, int shards, int codebook);
exl3_status exl3_moe_had_in(const void *x, int x_dtype, const uint16_t *suh, int shards, int hidden, int top_k, int slots,
                            const int32_t *sorted_ids, int cap, const int32_t *expert_ids, const int32_t *num_post, int codebook,
                            uint32_t *xf, void *stream);
exl3_status exl3_moe_glu_had_in(const uint16_t *gu, const uint16_t *suh2, int inter, int slots, const int32_t *sorted_ids, int cap,
                                const int32_t *expert_ids, const int32_t *num_post, int codebook, uint32_t *xf, void *stream);
size_t exl3_moe_workspace_bytes(int cap, int n_total);
exl3_status exl3_moe_gemm(const uint32_t *xf, const uint32_t *packed, int K, int codebook, const uint16_t *svh,
                          const int32_t *sorted_ids, const int32_t *expert_ids, const int32_t *num_post, int cap, int slots, int k,
                          int n_total, int shard_end, uint16_t *out, void *workspace, size_t workspace_bytes, void *stream);
exl3_status exl3_moe_combine(const uint16_t *yd, const float *topk_weights, const int32_t *topk_ids, int tokens, int top_k,
                             int hidden, int num_experts, void *y, int y_dtype, void *stream);

/* Routed experts with many rows per expert (prefill-sized batches) on the tensor cores.  The reference serves such batches
 * with the same grouped kernel and larger moe blocks (moe_block_size picks 8..64 rows from T * top_k / E,
 * cuda/src/sglang_exl3/kernels/marlin_moe.py:52-57; launch at cuda/csrc/exl3_marlin_moe.cu:376-408); here the routing is
 * aligned to blocks of exl3_moe_tc_block_rows() = 128 rows and up to two blocks of one expert (four when hidden or inter is
 * not a multiple of 256) share every decoded weight block in a grouped tcgen05 GEMM.  x, yd and the sign vectors must be
 * 16-byte aligned.  One call runs one bitrate class from the routing to the per-slot outputs:
 *   align (expert_map as in exl3_moe_align_mapped, or NULL with num_local == num_experts) -> gate|up -> SiLU(gate) * up
 *   -> down -> yd[slot, :] (fp16 [tokens * top_k, hidden]; slots of experts outside the class are not written).
 * exl3_moe_combine then closes the layer.  w13 / suh13 / svh13 / w2 / suh2 / svh2 are the resident expert stacks of
 * exl3_moe_gemm ([E][2I/128][H/128]..., [E][2][H], [E][2I], [E][H/128][I/128]..., [E][I], [E][H]).  The workspace holds
 * exl3_moe_tc_workspace_bytes(tokens * top_k, num_local, hidden, inter) bytes, 256-byte aligned, first 256 bytes zero. */
int exl3_moe_tc_block_rows(void);
size_t exl3_moe_tc_workspace_bytes(int slots, int num_local, int hidden, int inter);
exl3_status exl3_moe_tc_experts(const void *x, int x_dtype, int tokens, int top_k, int hidden, int inter, const int32_t *topk_ids,
                                int num_experts, const int32_t *expert_map, int num_local, const uint32_t *w13, const uint16_t *suh13,
                                const uint16_t *svh13, const uint32_t *w2, const uint16_t *suh2, const uint16_t *svh2, int K,
                                int codebook, uint16_t *yd, void *workspace, size_t workspace_bytes, void *stream);

/* Reads and clears the device-side error word kept in a workspace (set when a bounded wait in a kernel gave up).
 * workspace == NULL with workspace_bytes == 0 means the built-in scratch of exl3_linear_static on the current device.
 * Synchronises `stream`.  Returns EXL3_OK or EXL3_ERR_DEVICE_WAIT. */
exl3_status exl3_device_error(void *workspace, size_t workspace_bytes, void *stream);

/* Measurement / test knob: how weights of the 3INST and MCG codebooks enter the tensor-core product.
 * -1 = library default, 0 = split (each weight as its two fp16 summands, added exactly by the fp32 accumulator),
 * 1 = paired (weights rounded to fp16 first, as the reference decoder's table).  No counterpart in the reference. */
void exl3_set_gemv_mode(int mode);
/* Measurement / test knob: output tiling of exl3_linear_tc.  -1 = library default, 0 = 512 x 128 tiles, 1 = 256 x 256 tiles
 * (used only where the column blocks pair up inside every shard), 2 = 384 x 128 tiles, 3 = 512 x 256 tiles on pairs of CTAs
 * (clusters of two, cta_group::2 MMAs; same condition as 1).  No counterpart in the reference. */
void exl3_set_tc_tiling(int tiling);
/* Measurement / test knob: upper bound of the parts the reduction of a tile is cut into when exl3_linear_tc has fewer
 * tiles than SMs, or, with tiling 3, for the tiles of a last wave that does not fill the CTA pairs (0 = library default,
 * 1 = never split).  No counterpart in the reference. */
void exl3_set_tc_ksplit(int parts);

#ifdef __cplusplus
}
#endif
#endif /* EXL3_B200_H */
