// extern "C" entry points of libexl3_b200 (declared in include/exl3_b200.h): argument checks, workspace
// carving, launches.  No entry point allocates device memory.
#include <cstdio>
#include <cstring>

#include "exl3_internal.h"
#include "exl3_moe_kernel.cuh"

namespace exl3 {

static int g_last_cuda_error = 0;
static DeviceInfo g_devices[64];

int cuda_status(cudaError_t e)
{
    if (e == cudaSuccess) return EXL3_OK;
    g_last_cuda_error = (int)e;
    return EXL3_ERR_CUDA;
}

const DeviceInfo* current_device_info()
{
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    return g_devices[dev].ready ? &g_devices[dev] : nullptr;
}

static bool aligned(const void* p, size_t a) { return p != nullptr && (reinterpret_cast<uintptr_t>(p) % a) == 0; }

static int check_matrix(int k, int n, int K, int cb)
{
    if (k < 0 || n < 0 || (k % 128) || (n % 128)) return EXL3_ERR_BAD_SHAPE;
    if (K < 2 || K > 8) return EXL3_ERR_UNSUPPORTED_K;
    if (cb < 0 || cb > 2) return EXL3_ERR_UNSUPPORTED_CODEBOOK;
    return EXL3_OK;
}

static int fill_shards(GemvArgs& a, const int* shard_ends, int n_shards, int n_total)
{
    if (n_shards < 1 || n_shards > GEMV_MAX_SHARDS) return EXL3_ERR_BAD_SHAPE;
    if (n_shards > 1 && shard_ends == nullptr) return EXL3_ERR_BAD_POINTER;
    int prev = 0;
    for (int s = 0; s < n_shards - 1; s++) {
        int e = shard_ends[s];
        if (e <= prev || e >= n_total || (e % 128)) return EXL3_ERR_BAD_SHAPE;
        a.shard_end_blocks[s] = e / 128;
        prev = e;
    }
    for (int s = n_shards - 1; s < GEMV_MAX_SHARDS; s++) a.shard_end_blocks[s] = n_total / 128;
    a.n_shards = n_shards;
    return EXL3_OK;
}

}  // namespace exl3

using namespace exl3;

extern "C" {

const char* exl3_status_str(exl3_status s)
{
    switch (s) {
        case EXL3_OK: return "ok";
        case EXL3_ERR_BAD_SHAPE: return "bad shape: k and n must be non-negative multiples of 128, shard ends increasing multiples of 128";
        case EXL3_ERR_UNSUPPORTED_K: return "unsupported bit rate: K must be an integer in 2..8";
        case EXL3_ERR_UNSUPPORTED_CODEBOOK: return "unsupported codebook: 0 (3inst), 1 (mcg) or 2 (mul1)";
        case EXL3_ERR_BAD_POINTER: return "null or misaligned pointer";
        case EXL3_ERR_WORKSPACE: return "workspace missing or too small";
        case EXL3_ERR_CUDA: return "CUDA runtime error";
        case EXL3_ERR_DEVICE_WAIT: return "a bounded device-side wait gave up";
        case EXL3_ERR_NOT_INITIALISED: return "exl3_init_device was not called for the current device";
        case EXL3_ERR_UNSUPPORTED_ROWS: return "unsupported row count";
        case EXL3_ERR_UNSUPPORTED_DTYPE: return "unsupported dtype";
        case EXL3_ERR_STATIC_WORKSPACE: return "problem too large for the built-in scratch of exl3_linear_static: use exl3_linear with a workspace";
    }
    return "unknown status";
}

int exl3_last_cuda_error(void) { return g_last_cuda_error; }
int exl3_version(void) { return 100; }

exl3_status exl3_init_device(int device)
{
    if (device < 0 || device >= 64) return EXL3_ERR_BAD_SHAPE;
    int prev = -1;
    if (int rc = cuda_status(cudaGetDevice(&prev))) return rc;
    if (int rc = cuda_status(cudaSetDevice(device))) return rc;
    DeviceInfo& d = g_devices[device];
    int rc = EXL3_OK;
    if (!d.ready) {
        rc = cuda_status(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, device));
        if (rc == EXL3_OK) rc = cuda_status(cudaDeviceGetAttribute(&d.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device));
        if (rc == EXL3_OK) {
            d.ready = true;
            rc = gemv_init_device();
            if (rc == EXL3_OK) rc = moe_init_device();
            if (rc == EXL3_OK) rc = attention_init_device();
            if (rc == EXL3_OK) rc = gemm_tc_init_device();
            if (rc != EXL3_OK) d.ready = false;
        }
    }
    cudaSetDevice(prev);
    return rc;
}

int exl3_device_sm_count(int device)
{
    if (device < 0 || device >= 64 || !g_devices[device].ready) return 0;
    return g_devices[device].sm_count;
}

size_t exl3_packed_bytes(int k, int n, int K)
{
    if (k < 0 || n < 0 || K < 2 || K > 8) return 0;
    return (size_t)k * (size_t)n * (size_t)K / 8;
}

exl3_status exl3_repack(const uint16_t* trellis, int k, int n, int K, uint32_t* packed, void* stream)
{
    if (int rc = check_matrix(k, n, K, 0)) return rc;
    if ((long long)k * n == 0) return EXL3_OK;
    if (!aligned(trellis, 4) || !aligned(packed, 16)) return EXL3_ERR_BAD_POINTER;
    return launch_repack(trellis, k, n, K, packed, (cudaStream_t)stream);
}

exl3_status exl3_unpack(const uint32_t* packed, int k, int n, int K, uint16_t* trellis, void* stream)
{
    if (int rc = check_matrix(k, n, K, 0)) return rc;
    if ((long long)k * n == 0) return EXL3_OK;
    if (!aligned(trellis, 4) || !aligned(packed, 16)) return EXL3_ERR_BAD_POINTER;
    return launch_unpack(packed, k, n, K, trellis, (cudaStream_t)stream);
}

exl3_status exl3_reconstruct(const uint16_t* trellis, int k, int n, int K, int codebook, uint16_t* w, void* stream)
{
    if (k < 0 || n < 0 || (k % 16) || (n % 16)) return EXL3_ERR_BAD_SHAPE;
    if (K < 2 || K > 8) return EXL3_ERR_UNSUPPORTED_K;
    if (codebook < 0 || codebook > 2) return EXL3_ERR_UNSUPPORTED_CODEBOOK;
    if ((long long)k * n == 0) return EXL3_OK;
    if (!aligned(trellis, 4) || !aligned(w, 2)) return EXL3_ERR_BAD_POINTER;
    return launch_reconstruct_stored(trellis, k / 16, n / 16, K, codebook, reinterpret_cast<__half*>(w), (cudaStream_t)stream);
}

exl3_status exl3_reconstruct_packed(const uint32_t* packed, int k, int n, int K, int codebook, uint16_t* w, void* stream)
{
    if (int rc = check_matrix(k, n, K, codebook)) return rc;
    if ((long long)k * n == 0) return EXL3_OK;
    if (!aligned(packed, 16) || !aligned(w, 2)) return EXL3_ERR_BAD_POINTER;
    return launch_reconstruct_packed(packed, k, n, K, codebook, reinterpret_cast<__half*>(w), (cudaStream_t)stream);
}

exl3_status exl3_had_in(const void* x, int x_dtype, const uint16_t* suh, int shards, int rows, int k, uint16_t* xh, void* stream)
{
    if (rows < 0 || shards < 1 || k < 0 || (k % 128)) return EXL3_ERR_BAD_SHAPE;
    if (x_dtype != EXL3_F16 && x_dtype != EXL3_BF16) return EXL3_ERR_UNSUPPORTED_DTYPE;
    if (rows == 0 || k == 0) return EXL3_OK;
    if (!aligned(x, 2) || !aligned(xh, 8) || (suh && !aligned(suh, 2))) return EXL3_ERR_BAD_POINTER;
    return launch_had_in(x, x_dtype == EXL3_BF16, reinterpret_cast<const __half*>(suh), shards, rows, k, xh, 0, (cudaStream_t)stream);
}

exl3_status exl3_had_out(const void* y, int y_dtype, const uint16_t* svh, int rows, int n, void* out, int64_t out_stride,
                         int out_dtype, void* stream)
{
    if (rows < 0 || n < 0 || (n % 128) || out_stride < n || (out_stride % 8)) return EXL3_ERR_BAD_SHAPE;
    if ((y_dtype != EXL3_F16 && y_dtype != EXL3_F32) || (out_dtype != EXL3_F16 && out_dtype != EXL3_BF16))
        return EXL3_ERR_UNSUPPORTED_DTYPE;
    if (rows == 0 || n == 0) return EXL3_OK;
    if (!aligned(y, 16) || !aligned(out, 16) || (svh && !aligned(svh, 16))) return EXL3_ERR_BAD_POINTER;
    return launch_had_out(y, y_dtype == EXL3_F32, reinterpret_cast<const __half*>(svh), rows, n, out, out_stride,
                          out_dtype == EXL3_BF16, (cudaStream_t)stream);
}

size_t exl3_linear_workspace_bytes(int rows, int k, int n_total, int n_shards)
{
    if (k < 0 || n_total < 0 || n_shards < 1) return 0;
    return workspace_layout(rows, k, n_total, n_shards).total;
}

namespace {
struct NormArgs {                // consumer of a residual stream: x = z, normalised on the way in (exl3_normed_linear)
    const void* weight;
    const float* ssq;            // [rows, k/128]
    float eps;
};
struct ResidualArgs {            // producer: the epilogue adds res_in, writes the new stream and its sums of squares
    const void* res_in;
    void* res_out;
    float* ssq_out;              // [rows, n_total/128]
};
}  // namespace

static int linear_common(const void* x, int x_dtype, const uint16_t* xh_rowmajor, const uint32_t* packed, int K, int codebook,
                         const uint16_t* suh_cat, const uint16_t* svh_cat, const int* shard_ends, int n_shards, int rows, int k,
                         int n_total, void* y, int y_dtype, void* workspace, size_t workspace_bytes, cudaStream_t st, bool rotated,
                         const TpExchange* tp = nullptr, bool prerotated = false, bool glu = false, const NormArgs* norm = nullptr,
                         const ResidualArgs* res = nullptr)
{
    if (int rc = check_matrix(k, n_total, K, codebook)) return rc;
    if (rows < 0) return EXL3_ERR_BAD_SHAPE;
    GemvArgs a;
    memset(&a, 0, sizeof(a));
    if (int rc = fill_shards(a, shard_ends, n_shards, n_total)) return rc;
    if (!rotated && !prerotated && x_dtype != EXL3_F16 && x_dtype != EXL3_BF16) return EXL3_ERR_UNSUPPORTED_DTYPE;
    if (prerotated && rows > GEMV_MAX_ROWS) return EXL3_ERR_UNSUPPORTED_ROWS;
    if (y_dtype != EXL3_F16 && y_dtype != EXL3_F32 && !(y_dtype == EXL3_BF16 && !rotated)) return EXL3_ERR_UNSUPPORTED_DTYPE;
    if (rows == 0 || k == 0 || n_total == 0) return EXL3_OK;
    if ((size_t)(n_total / 128) > WS_MAX_COUNTERS) return EXL3_ERR_BAD_SHAPE;
    if (!current_device_info()) return EXL3_ERR_NOT_INITIALISED;
    if (!aligned(packed, 16) || (!aligned(y, 16) && !(res && y == nullptr))) return EXL3_ERR_BAD_POINTER;
    if (res && (!aligned(res->res_in, 8) || !aligned(res->res_out, 8) || !aligned(res->ssq_out, 4) || res->res_in == res->res_out ||
                (y_dtype != EXL3_F16 && y_dtype != EXL3_BF16)))
        return EXL3_ERR_BAD_POINTER;
    if (prerotated ? !aligned(svh_cat, 8)
                   : rotated ? !aligned(xh_rowmajor, 2) : (!aligned(x, 2) || !aligned(suh_cat, 2) || !aligned(svh_cat, 8)))
        return EXL3_ERR_BAD_POINTER;
    const WorkspaceLayout wl = workspace_layout(rows, k, n_total, n_shards);
    if (!aligned(workspace, 256) || workspace_bytes < wl.total) return EXL3_ERR_WORKSPACE;
    unsigned char* ws = reinterpret_cast<unsigned char*>(workspace);

    a.packed = packed;
    a.xf = reinterpret_cast<const uint32_t*>(ws + wl.xf_off);
    a.svh = reinterpret_cast<const __half*>(svh_cat);
    a.partials = reinterpret_cast<float*>(ws + wl.partials_off);
    a.counters = reinterpret_cast<int*>(ws + wl.counters_off);
    a.err = reinterpret_cast<int*>(ws + wl.err_off);
    a.K = K;
    a.codebook = codebook;
    a.mode = gemv_default_mode(codebook);
    a.k = k;
    a.n_total = n_total;
    a.out_dtype = y_dtype;
    a.rotated = rotated ? 1 : 0;
    if (tp) a.tp = *tp;
    const size_t esz = 2, osz = y_dtype == EXL3_F32 ? 4 : 2;
    for (int r0 = 0; r0 < rows; r0 += GEMV_MAX_ROWS) {
        const int r = rows - r0 < GEMV_MAX_ROWS ? rows - r0 : GEMV_MAX_ROWS;
        a.rows = r;
        a.out = y ? reinterpret_cast<unsigned char*>(y) + (size_t)r0 * n_total * osz : nullptr;
        if (res) {
            a.res_in = reinterpret_cast<const unsigned char*>(res->res_in) + (size_t)r0 * n_total * 2;
            a.res_out = reinterpret_cast<unsigned char*>(res->res_out) + (size_t)r0 * n_total * 2;
            a.ssq_out = res->ssq_out + (size_t)r0 * (n_total / 128);
        }
        int rc;
        if (prerotated) {
            // The fragments are in the workspace already (exl3_rotate_fragments, exl3_rmsnorm_rotate, exl3_silu_mul_rotate):
            // up to two rows the kernel copies those of its units into shared memory once, else it reads them tile by tile.
            a.x = nullptr;
            a.xf_staged = 1;
            if (!gemv_rotates_input(a)) a.xf_staged = 0;
            if (res && !a.xf_staged) {          // more rows than the residual epilogue serves: plain GEMV, then the stream kernel
                if (!y) return EXL3_ERR_BAD_POINTER;
                a.res_out = nullptr;
                rc = launch_gemv(a, st);
                if (rc) return rc;
                rc = launch_residual_ssq(a.out, a.res_in, y_dtype == EXL3_BF16, r, n_total, reinterpret_cast<unsigned char*>(res->res_out) + (size_t)r0 * n_total * 2,
                                         res->ssq_out + (size_t)r0 * (n_total / 128), st);
                if (rc) return rc;
                continue;
            }
        } else if (rotated) {
            // shard s reads slab s of xh: rows [s*rows + r0, s*rows + r0 + r)
            for (int s = 0; s < n_shards; s++) {
                const __half* src = reinterpret_cast<const __half*>(xh_rowmajor) + ((size_t)s * rows + r0) * k;
                uint32_t* dst = const_cast<uint32_t*>(a.xf) + (size_t)s * (k / 16) * r * 4 * gemv_frag_words(a.mode);
                rc = launch_to_fragments(src, 1, r, k, dst, a.mode == GEMV_SPLIT ? 1 : 2, st);
                if (rc) return rc;
            }
        } else {
            // Up to two rows: the GEMV rotates its own input (one launch); otherwise the rotation kernel runs ahead of it.
            // glu: x is gate | up with rows of 2k values and the input proper is silu(gate) * up.
            const unsigned char* xr = reinterpret_cast<const unsigned char*>(x) + (size_t)r0 * (glu ? 2 * k : k) * esz;
            a.x = xr;
            a.suh = reinterpret_cast<const __half*>(suh_cat);
            a.x_bf16 = x_dtype == EXL3_BF16;
            a.x_glu = glu ? 1 : 0;
            if (norm) {
                a.norm_weight = norm->weight;
                a.ssq_in = norm->ssq + (size_t)r0 * (k / 128);
                a.norm_eps = norm->eps;
            }
            if (!gemv_rotates_input(a)) {
                a.x = nullptr;
                if (norm || res) {
                    // more rows than the kernel rotates itself: the normalisation / activation kernel ahead of a plain GEMV, and
                    // the stream kernel behind it where the epilogue would have added the residual
                    a.norm_weight = nullptr;
                    void* res_out = a.res_out;
                    a.res_out = nullptr;
                    if (res && !y) return EXL3_ERR_BAD_POINTER;
                    if (norm)
                        rc = launch_rmsnorm_rotate(xr, nullptr, norm->weight, norm->eps, x_dtype == EXL3_BF16, reinterpret_cast<const __half*>(suh_cat),
                                                   n_shards, r, k, nullptr, const_cast<uint32_t*>(a.xf), a.mode == GEMV_SPLIT ? 1 : 2, st);
                    else if (glu)
                        rc = launch_silu_mul_rotate(xr, x_dtype == EXL3_BF16, reinterpret_cast<const __half*>(suh_cat), r, k, nullptr,
                                                    const_cast<uint32_t*>(a.xf), a.mode == GEMV_SPLIT ? 1 : 2, st);
                    else
                        rc = launch_had_in(xr, x_dtype == EXL3_BF16, reinterpret_cast<const __half*>(suh_cat), n_shards, r, k,
                                           const_cast<uint32_t*>(a.xf), a.mode == GEMV_SPLIT ? 1 : 2, st);
                    if (rc) return rc;
                    rc = launch_gemv(a, st);
                    if (rc) return rc;
                    if (res) {
                        rc = launch_residual_ssq(a.out, a.res_in, y_dtype == EXL3_BF16, r, n_total, res_out, a.ssq_out, st);
                        if (rc) return rc;
                    }
                    continue;
                }
                rc = glu ? launch_silu_mul_rotate(xr, x_dtype == EXL3_BF16, reinterpret_cast<const __half*>(suh_cat), r, k, nullptr,
                                                  const_cast<uint32_t*>(a.xf), a.mode == GEMV_SPLIT ? 1 : 2, st)
                         : launch_had_in(xr, x_dtype == EXL3_BF16, reinterpret_cast<const __half*>(suh_cat), n_shards, r, k,
                                         const_cast<uint32_t*>(a.xf), a.mode == GEMV_SPLIT ? 1 : 2, st);
                if (rc) return rc;
            }
        }
        rc = launch_gemv(a, st);
        if (rc) return rc;
    }
    return EXL3_OK;
}

exl3_status exl3_linear(const void* x, int x_dtype, const uint32_t* packed, int K, int codebook, const uint16_t* suh_cat,
                        const uint16_t* svh_cat, const int* shard_ends, int n_shards, int rows, int k, int n_total, void* y,
                        int y_dtype, void* workspace, size_t workspace_bytes, void* stream)
{
    return linear_common(x, x_dtype, nullptr, packed, K, codebook, suh_cat, svh_cat, shard_ends, n_shards, rows, k, n_total, y,
                         y_dtype, workspace, workspace_bytes, (cudaStream_t)stream, false);
}

exl3_status exl3_linear_allreduce(const void* x, int x_dtype, const uint32_t* packed, int K, int codebook, const uint16_t* suh_cat,
                                  const uint16_t* svh_cat, const int* shard_ends, int n_shards, int rows, int k, int n_total, void* y,
                                  int y_dtype, void* workspace, size_t workspace_bytes, void* const* peer_regions, int rank, int world,
                                  size_t max_elems, int* state, void* stream)
{
    if (world < 1 || world > TP_MAX_WORLD || rank < 0 || rank >= world) return EXL3_ERR_BAD_SHAPE;
    if (world == 1)
        return linear_common(x, x_dtype, nullptr, packed, K, codebook, suh_cat, svh_cat, shard_ends, n_shards, rows, k, n_total, y,
                             y_dtype, workspace, workspace_bytes, (cudaStream_t)stream, false);
    if (y_dtype != EXL3_F16 && y_dtype != EXL3_BF16) return EXL3_ERR_UNSUPPORTED_DTYPE;
    const size_t chunk_rows = rows < GEMV_MAX_ROWS ? (rows < 0 ? 0 : rows) : GEMV_MAX_ROWS;
    const size_t slot_bytes = (max_elems * 4 + 255) & ~(size_t)255;
    if (chunk_rows * (size_t)(n_total < 0 ? 0 : n_total) > max_elems || slot_bytes > 0xFFFFFFFFu) return EXL3_ERR_BAD_SHAPE;
    if (!peer_regions || !state || !aligned(state, 4)) return EXL3_ERR_BAD_POINTER;
    TpExchange tp;
    memset(&tp, 0, sizeof(tp));
    for (int r = 0; r < world; r++) {
        if (!aligned(peer_regions[r], 256)) return EXL3_ERR_BAD_POINTER;
        tp.base[r] = reinterpret_cast<unsigned char*>(peer_regions[r]);
    }
    tp.rank = rank;
    tp.world = world;
    tp.slot_bytes = (unsigned int)slot_bytes;
    tp.state = state;
    return linear_common(x, x_dtype, nullptr, packed, K, codebook, suh_cat, svh_cat, shard_ends, n_shards, rows, k, n_total, y, y_dtype,
                         workspace, workspace_bytes, (cudaStream_t)stream, false, &tp);
}

exl3_status exl3_gemm_rotated(const uint16_t* xh, const uint32_t* packed, int K, int codebook, const int* shard_ends, int n_shards,
                              int rows, int k, int n_total, uint16_t* out, void* workspace, size_t workspace_bytes, void* stream)
{
    return linear_common(nullptr, EXL3_F16, xh, packed, K, codebook, nullptr, nullptr, shard_ends, n_shards, rows, k, n_total, out,
                         EXL3_F16, workspace, workspace_bytes, (cudaStream_t)stream, true);
}

static void* static_workspace_of_current_device(int* status);

exl3_status exl3_gemm_rotated_f32(const uint16_t* xh, const uint32_t* packed, int K, int codebook, const int* shard_ends, int n_shards,
                                  int rows, int k, int n_total, float* out, void* workspace, size_t workspace_bytes, void* stream)
{
    return linear_common(nullptr, EXL3_F16, xh, packed, K, codebook, nullptr, nullptr, shard_ends, n_shards, rows, k, n_total, out,
                         EXL3_F32, workspace, workspace_bytes, (cudaStream_t)stream, true);
}

exl3_status exl3_device_error(void* workspace, size_t workspace_bytes, void* stream)
{
    if (workspace == nullptr && workspace_bytes == 0) {
        // The built-in scratch of exl3_linear_static on the current device (address looked up and cached, no allocation).
        int rc = EXL3_OK;
        workspace = static_workspace_of_current_device(&rc);
        if (rc) return rc;
        workspace_bytes = EXL3_STATIC_WORKSPACE_BYTES;
    }
    if (!aligned(workspace, 256) || workspace_bytes < 256) return EXL3_ERR_WORKSPACE;
    int code = 0;
    cudaStream_t st = (cudaStream_t)stream;
    if (int rc = cuda_status(cudaMemcpyAsync(&code, workspace, sizeof(int), cudaMemcpyDeviceToHost, st))) return rc;
    if (int rc = cuda_status(cudaStreamSynchronize(st))) return rc;
    if (code == 0) return EXL3_OK;
    if (int rc = cuda_status(cudaMemsetAsync(workspace, 0, sizeof(int), st))) return rc;
    return EXL3_ERR_DEVICE_WAIT;
}

/* ---- decode step: rotated fragments written by the kernel ahead of the linear -------------------------------------- */

static int fragment_mode(int codebook) { return gemv_default_mode(codebook) == GEMV_SPLIT ? 1 : 2; }

static int fragment_region(int rows, int k, int n_shards, void* workspace, size_t workspace_bytes, uint32_t** xf)
{
    if (rows < 0 || rows > GEMV_MAX_ROWS) return EXL3_ERR_UNSUPPORTED_ROWS;
    if (k < 0 || (k % 128) || n_shards < 1 || n_shards > GEMV_MAX_SHARDS) return EXL3_ERR_BAD_SHAPE;
    const WorkspaceLayout wl = workspace_layout(rows, k, 128, n_shards);
    if (!aligned(workspace, 256) || workspace_bytes < wl.partials_off) return EXL3_ERR_WORKSPACE;
    *xf = reinterpret_cast<uint32_t*>(reinterpret_cast<unsigned char*>(workspace) + wl.xf_off);
    return EXL3_OK;
}

exl3_status exl3_rotate_fragments(const void* x, int x_dtype, const uint16_t* suh_cat, int n_shards, int rows, int k, int codebook,
                                  void* workspace, size_t workspace_bytes, void* stream)
{
    if (x_dtype != EXL3_F16 && x_dtype != EXL3_BF16) return EXL3_ERR_UNSUPPORTED_DTYPE;
    if (codebook < 0 || codebook > 2) return EXL3_ERR_UNSUPPORTED_CODEBOOK;
    uint32_t* xf = nullptr;
    if (int rc = fragment_region(rows, k, n_shards, workspace, workspace_bytes, &xf)) return rc;
    if (rows == 0 || k == 0) return EXL3_OK;
    if (!aligned(x, 2) || !aligned(suh_cat, 8)) return EXL3_ERR_BAD_POINTER;
    return launch_had_in(x, x_dtype == EXL3_BF16, reinterpret_cast<const __half*>(suh_cat), n_shards, rows, k, xf, fragment_mode(codebook),
                         (cudaStream_t)stream);
}

exl3_status exl3_rmsnorm_rotate(const void* x, void* residual, const void* weight, float eps, int dtype, const uint16_t* suh_cat,
                                int n_shards, int rows, int k, int codebook, void* normed, void* workspace, size_t workspace_bytes,
                                void* stream)
{
    if (dtype != EXL3_F16 && dtype != EXL3_BF16) return EXL3_ERR_UNSUPPORTED_DTYPE;
    if (codebook < 0 || codebook > 2) return EXL3_ERR_UNSUPPORTED_CODEBOOK;
    uint32_t* xf = nullptr;
    if (int rc = fragment_region(rows, k, n_shards, workspace, workspace_bytes, &xf)) return rc;
    if (rows == 0 || k == 0) return EXL3_OK;
    if (!aligned(x, 8) || !aligned(weight, 8) || !aligned(suh_cat, 8) || (residual && !aligned(residual, 8)) || (normed && !aligned(normed, 8)))
        return EXL3_ERR_BAD_POINTER;
    return launch_rmsnorm_rotate(x, residual, weight, eps, dtype == EXL3_BF16, reinterpret_cast<const __half*>(suh_cat), n_shards, rows, k,
                                 normed, xf, fragment_mode(codebook), (cudaStream_t)stream);
}

exl3_status exl3_silu_mul_rotate(const void* gate_up, int dtype, const uint16_t* suh, int rows, int inter, int codebook, void* act,
                                 void* workspace, size_t workspace_bytes, void* stream)
{
    if (dtype != EXL3_F16 && dtype != EXL3_BF16) return EXL3_ERR_UNSUPPORTED_DTYPE;
    if (codebook < 0 || codebook > 2) return EXL3_ERR_UNSUPPORTED_CODEBOOK;
    uint32_t* xf = nullptr;
    if (int rc = fragment_region(rows, inter, 1, workspace, workspace_bytes, &xf)) return rc;
    if (rows == 0 || inter == 0) return EXL3_OK;
    if (!aligned(gate_up, 8) || !aligned(suh, 8) || (act && !aligned(act, 8))) return EXL3_ERR_BAD_POINTER;
    return launch_silu_mul_rotate(gate_up, dtype == EXL3_BF16, reinterpret_cast<const __half*>(suh), rows, inter, act, xf,
                                  fragment_mode(codebook), (cudaStream_t)stream);
}

static int make_exchange(TpExchange& tp, void* const* peer_regions, int rank, int world, size_t max_elems, int* state, int rows, int n_total,
                         int y_dtype)
{
    if (world > TP_MAX_WORLD || rank < 0 || rank >= world) return EXL3_ERR_BAD_SHAPE;
    if (y_dtype != EXL3_F16 && y_dtype != EXL3_BF16) return EXL3_ERR_UNSUPPORTED_DTYPE;
    const size_t slot_bytes = (max_elems * 4 + 255) & ~(size_t)255;
    if ((size_t)(rows < 0 ? 0 : rows) * (size_t)(n_total < 0 ? 0 : n_total) > max_elems || slot_bytes > 0xFFFFFFFFu) return EXL3_ERR_BAD_SHAPE;
    if (!peer_regions || !state || !aligned(state, 4)) return EXL3_ERR_BAD_POINTER;
    memset(&tp, 0, sizeof(tp));
    for (int r = 0; r < world; r++) {
        if (!aligned(peer_regions[r], 256)) return EXL3_ERR_BAD_POINTER;
        tp.base[r] = reinterpret_cast<unsigned char*>(peer_regions[r]);
    }
    tp.rank = rank;
    tp.world = world;
    tp.slot_bytes = (unsigned int)slot_bytes;
    tp.state = state;
    return EXL3_OK;
}

static int residual_args(ResidualArgs& r, const void* residual_in, void* residual_out, float* ssq_out, const void* y, int world)
{
    if (!residual_in && !residual_out && !ssq_out) return 0;
    if (!residual_in || !residual_out || !ssq_out) return EXL3_ERR_BAD_POINTER;
    if (world > 1 && !y) return EXL3_ERR_BAD_POINTER;              // the exchange sums in the output buffer
    r = {residual_in, residual_out, ssq_out};
    return 1;
}

exl3_status exl3_linear_prerotated(const uint32_t* packed, int K, int codebook, const uint16_t* svh_cat, const int* shard_ends,
                                   int n_shards, int rows, int k, int n_total, void* y, int y_dtype, void* workspace,
                                   size_t workspace_bytes, void* const* peer_regions, int rank, int world, size_t max_elems, int* state,
                                   const void* residual_in, void* residual_out, float* ssq_out, void* stream)
{
    ResidualArgs res;
    const int has = residual_args(res, residual_in, residual_out, ssq_out, y, world);
    if (has > 1) return has;
    TpExchange tp;
    if (world > 1)
        if (int rc = make_exchange(tp, peer_regions, rank, world, max_elems, state, rows, n_total, y_dtype)) return rc;
    return linear_common(nullptr, EXL3_F16, nullptr, packed, K, codebook, nullptr, svh_cat, shard_ends, n_shards, rows, k, n_total, y,
                         y_dtype, workspace, workspace_bytes, (cudaStream_t)stream, false, world > 1 ? &tp : nullptr, true, false, nullptr,
                         has ? &res : nullptr);
}

exl3_status exl3_glu_linear(const void* gate_up, int x_dtype, const uint32_t* packed, int K, int codebook, const uint16_t* suh,
                            const uint16_t* svh_cat, const int* shard_ends, int n_shards, int rows, int k, int n_total, void* y, int y_dtype,
                            void* workspace, size_t workspace_bytes, void* const* peer_regions, int rank, int world, size_t max_elems,
                            int* state, const void* residual_in, void* residual_out, float* ssq_out, void* stream)
{
    if (n_shards != 1) return EXL3_ERR_BAD_SHAPE;               // one input, one sign vector: a down projection is not a fused group
    if (rows > 0 && !aligned(gate_up, 8)) return EXL3_ERR_BAD_POINTER;
    ResidualArgs res;
    const int has = residual_args(res, residual_in, residual_out, ssq_out, y, world);
    if (has > 1) return has;
    TpExchange tp;
    if (world > 1)
        if (int rc = make_exchange(tp, peer_regions, rank, world, max_elems, state, rows, n_total, y_dtype)) return rc;
    return linear_common(gate_up, x_dtype, nullptr, packed, K, codebook, suh, svh_cat, shard_ends, n_shards, rows, k, n_total, y, y_dtype,
                         workspace, workspace_bytes, (cudaStream_t)stream, false, world > 1 ? &tp : nullptr, false, true, nullptr,
                         has ? &res : nullptr);
}

exl3_status exl3_residual_ssq(const void* x, const void* residual_in, int dtype, int rows, int k, void* residual_out, float* ssq, void* stream)
{
    if (dtype != EXL3_F16 && dtype != EXL3_BF16) return EXL3_ERR_UNSUPPORTED_DTYPE;
    if (rows < 0 || k <= 0 || k % 128) return EXL3_ERR_BAD_SHAPE;
    if (rows == 0) return EXL3_OK;
    if (!aligned(x, 8) || (residual_in && !aligned(residual_in, 8)) || (residual_out && !aligned(residual_out, 8)) || !aligned(ssq, 4))
        return EXL3_ERR_BAD_POINTER;
    return launch_residual_ssq(x, residual_in, dtype == EXL3_BF16, rows, k, residual_out, ssq, (cudaStream_t)stream);
}

exl3_status exl3_normed_linear(const void* z, int x_dtype, const float* ssq, const void* norm_weight, float eps, const uint32_t* packed, int K,
                               int codebook, const uint16_t* suh_cat, const uint16_t* svh_cat, const int* shard_ends, int n_shards, int rows,
                               int k, int n_total, void* y, int y_dtype, void* workspace, size_t workspace_bytes, void* stream)
{
    if (rows > 0 && (!aligned(z, 8) || !aligned(norm_weight, 8) || !aligned(suh_cat, 8) || !aligned(ssq, 4))) return EXL3_ERR_BAD_POINTER;
    NormArgs norm = {norm_weight, ssq, eps};
    return linear_common(z, x_dtype, nullptr, packed, K, codebook, suh_cat, svh_cat, shard_ends, n_shards, rows, k, n_total, y, y_dtype,
                         workspace, workspace_bytes, (cudaStream_t)stream, false, nullptr, false, false, &norm);
}

exl3_status exl3_rmsnorm_linear(const void* x, int x_dtype, const void* residual_in, void* residual_out, const void* norm_weight, float eps,
                                const uint32_t* packed, int K, int codebook, const uint16_t* suh_cat, const uint16_t* svh_cat,
                                const int* shard_ends, int n_shards, int rows, int k, int n_total, void* y, int y_dtype, void* workspace,
                                size_t workspace_bytes, void* stream)
{
    if (int rc = check_matrix(k, n_total, K, codebook)) return rc;
    if (rows <= 0) return rows < 0 ? EXL3_ERR_BAD_SHAPE : EXL3_OK;
    if (!aligned(x, 8) || !aligned(norm_weight, 8) || !aligned(suh_cat, 8)) return EXL3_ERR_BAD_POINTER;
    if (residual_in && (!aligned(residual_in, 8) || !aligned(residual_out, 8) || residual_in == residual_out)) return EXL3_ERR_BAD_POINTER;
    const WorkspaceLayout wl = workspace_layout(rows, k, n_total, n_shards);
    if (!aligned(workspace, 256) || workspace_bytes < wl.total) return EXL3_ERR_WORKSPACE;
    // The stream's sums of squares live where the fragments of a pre-rotated call would: this call has none (the GEMV rotates
    // its own input; from three rows up the normalisation kernel recomputes the statistics and overwrites the region).
    float* ssq = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(workspace) + wl.xf_off);
    if (int rc = launch_residual_ssq(x, residual_in, x_dtype == EXL3_BF16, rows, k, residual_in ? residual_out : nullptr, ssq, (cudaStream_t)stream))
        return rc;
    return exl3_normed_linear(residual_in ? residual_out : x, x_dtype, ssq, norm_weight, eps, packed, K, codebook, suh_cat, svh_cat, shard_ends,
                              n_shards, rows, k, n_total, y, y_dtype, workspace, workspace_bytes, stream);
}

size_t exl3_attention_scratch_bytes(int rows, int q_heads, int kv_heads, int t_max)
{
    if (rows < 0 || q_heads < 1 || kv_heads < 1 || t_max < 1) return 0;
    return attention_scratch_bytes(rows, q_heads, kv_heads, t_max);
}

exl3_status exl3_rope_append(void* qkv, int dtype, int rows, int q_heads, int kv_heads, int head_dim, const float* cos_table,
                             const float* sin_table, void* k_cache, void* v_cache, int t_max, const int* position, void* stream)
{
    if (dtype != EXL3_F16 && dtype != EXL3_BF16) return EXL3_ERR_UNSUPPORTED_DTYPE;
    if (rows < 0 || q_heads < 1 || kv_heads < 1 || head_dim != 128 || t_max < 1) return EXL3_ERR_BAD_SHAPE;
    if (!aligned(qkv, 2) || !aligned(cos_table, 4) || !aligned(sin_table, 4) || !aligned(k_cache, 16) || !aligned(v_cache, 16) || !aligned(position, 4))
        return EXL3_ERR_BAD_POINTER;
    return launch_rope_append(qkv, dtype == EXL3_BF16, rows, q_heads, kv_heads, cos_table, sin_table, k_cache, v_cache, t_max, position,
                              (cudaStream_t)stream);
}

static int attention_common(const void* qkv, int dtype, int rows, int q_heads, int kv_heads, int head_dim, const float* cos_table,
                            const float* sin_table, void* k_cache, void* v_cache, int t_max, const int* position, float scale, void* scratch,
                            size_t scratch_bytes, void* out, const uint16_t* suh_next, int codebook, void* workspace, size_t workspace_bytes,
                            void* stream)
{
    uint32_t* xf = nullptr;
    if (suh_next) {
        if (codebook < 0 || codebook > 2) return EXL3_ERR_UNSUPPORTED_CODEBOOK;
        if (!aligned(suh_next, 8)) return EXL3_ERR_BAD_POINTER;
        if (int rc = fragment_region(rows, q_heads * 128, 1, workspace, workspace_bytes, &xf)) return rc;
    }
    if (dtype != EXL3_F16 && dtype != EXL3_BF16) return EXL3_ERR_UNSUPPORTED_DTYPE;
    if (rows < 0 || q_heads < 1 || kv_heads < 1 || head_dim != 128 || t_max < 1 || q_heads % kv_heads) return EXL3_ERR_BAD_SHAPE;
    if (!aligned(qkv, 8) || !aligned(k_cache, 16) || !aligned(v_cache, 16) || !aligned(position, 4) || (out && !aligned(out, 8)) || (!out && !suh_next))
        return EXL3_ERR_BAD_POINTER;
    if (!aligned(scratch, 256) || scratch_bytes < attention_scratch_bytes(rows, q_heads, kv_heads, t_max)) return EXL3_ERR_WORKSPACE;
    if (!current_device_info()) return EXL3_ERR_NOT_INITIALISED;
    return launch_decode_attention(qkv, dtype == EXL3_BF16, rows, q_heads, kv_heads, k_cache, v_cache, t_max, position, scale, cos_table,
                                   sin_table, reinterpret_cast<float*>(scratch), out, reinterpret_cast<const __half*>(suh_next), xf,
                                   suh_next ? fragment_mode(codebook) : 0, (cudaStream_t)stream);
}

exl3_status exl3_decode_attention(const void* qkv, int dtype, int rows, int q_heads, int kv_heads, int head_dim, const void* k_cache,
                                  const void* v_cache, int t_max, const int* position, float scale, void* scratch, size_t scratch_bytes,
                                  void* out, const uint16_t* suh_next, int codebook, void* workspace, size_t workspace_bytes, void* stream)
{
    return attention_common(qkv, dtype, rows, q_heads, kv_heads, head_dim, nullptr, nullptr, const_cast<void*>(k_cache),
                            const_cast<void*>(v_cache), t_max, position, scale, scratch, scratch_bytes, out, suh_next, codebook, workspace,
                            workspace_bytes, stream);
}

exl3_status exl3_rope_decode_attention(const void* qkv, int dtype, int rows, int q_heads, int kv_heads, int head_dim, const float* cos_table,
                                       const float* sin_table, void* k_cache, void* v_cache, int t_max, const int* position, float scale,
                                       void* scratch, size_t scratch_bytes, void* out, const uint16_t* suh_next, int codebook,
                                       void* workspace, size_t workspace_bytes, void* stream)
{
    if (!aligned(cos_table, 4) || !aligned(sin_table, 4)) return EXL3_ERR_BAD_POINTER;
    return attention_common(qkv, dtype, rows, q_heads, kv_heads, head_dim, cos_table, sin_table, k_cache, v_cache, t_max, position, scale,
                            scratch, scratch_bytes, out, suh_next, codebook, workspace, workspace_bytes, stream);
}

/* ---- many-row (prefill) fused GEMM on tcgen05 ------------------------------------------------------------- */

static size_t tc_up(size_t v) { return (v + 255) & ~(size_t)255; }

size_t exl3_gemm_tc_workspace_bytes(int rows, int k, int n_total, int n_shards)
{
    if (rows < 0 || k < 0 || n_total < 0 || n_shards < 1) return 0;
    return 256 + tc_up(gemm_tc_activation_bytes(rows, k, n_shards)) + tc_up((size_t)rows * n_total * sizeof(__half)) +
           tc_up(gemm_tc_part_bytes(rows, n_total));
}

exl3_status exl3_linear_tc(const void* x, int x_dtype, const uint32_t* packed, int K, int codebook, const uint16_t* suh_cat,
                           const uint16_t* svh_cat, const int* shard_ends, int n_shards, int rows, int k, int n_total, void* y,
                           int y_dtype, void* workspace, size_t workspace_bytes, void* stream)
{
    if (int rc = check_matrix(k, n_total, K, codebook)) return rc;
    if (rows < 0) return EXL3_ERR_BAD_SHAPE;
    GemvArgs a;
    memset(&a, 0, sizeof(a));
    if (int rc = fill_shards(a, shard_ends, n_shards, n_total)) return rc;
    if ((x_dtype != EXL3_F16 && x_dtype != EXL3_BF16) || (y_dtype != EXL3_F16 && y_dtype != EXL3_BF16)) return EXL3_ERR_UNSUPPORTED_DTYPE;
    if (rows == 0 || k == 0 || n_total == 0) return EXL3_OK;
    if (!current_device_info()) return EXL3_ERR_NOT_INITIALISED;
    if (!aligned(x, 16) || !aligned(packed, 16) || !aligned(suh_cat, 16) || !aligned(svh_cat, 16) || !aligned(y, 16)) return EXL3_ERR_BAD_POINTER;
    if (!aligned(workspace, 256) || workspace_bytes < exl3_gemm_tc_workspace_bytes(rows, k, n_total, n_shards)) return EXL3_ERR_WORKSPACE;
    cudaStream_t st = (cudaStream_t)stream;
    unsigned char* ws = reinterpret_cast<unsigned char*>(workspace);
    __half* xa = reinterpret_cast<__half*>(ws + 256);
    __half* rot = reinterpret_cast<__half*>(ws + 256 + tc_up(gemm_tc_activation_bytes(rows, k, n_shards)));
    float* part = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(rot) + tc_up((size_t)rows * n_total * sizeof(__half)));
    TcSplit split = {1, 0, 0, 0};
    if (int rc = launch_gemm_tc(x, x_dtype == EXL3_BF16, reinterpret_cast<const __half*>(suh_cat), packed, K, codebook, a.shard_end_blocks,
                                n_shards, rows, k, n_total, xa, rot, part, y, reinterpret_cast<const __half*>(svh_cat), y_dtype == EXL3_BF16,
                                &split, reinterpret_cast<int*>(ws), st))
        return rc;
    if (split.tile_slabs) {
        if (split.parts == 1) return EXL3_OK;
        return launch_had_out_tiles(part, split.parts, split.tail_first, split.row_tiles, reinterpret_cast<const __half*>(svh_cat), rows,
                                    n_total, y, y_dtype == EXL3_BF16, st);
    }
    if (split.parts > 1)
        return launch_had_out_sum(part, split.parts, (long long)rows * n_total, reinterpret_cast<const __half*>(svh_cat), rows, n_total, y,
                                  y_dtype == EXL3_BF16, st);
    return launch_had_out(rot, 0, reinterpret_cast<const __half*>(svh_cat), rows, n_total, y, n_total, y_dtype == EXL3_BF16, st);
}

/* ---- tensor-parallel exchange step ------------------------------------------------------------------------ */

size_t exl3_allreduce_region_bytes(size_t max_elems) { return allreduce_region_bytes(max_elems); }

exl3_status exl3_allreduce(void* data, int dtype, size_t n, void* const* peer_regions, int rank, int world, size_t max_elems, int* state,
                           void* stream)
{
    if (world < 1 || world > 16 || rank < 0 || rank >= world || n > max_elems || (n % 8)) return EXL3_ERR_BAD_SHAPE;
    if (dtype != EXL3_F16 && dtype != EXL3_BF16) return EXL3_ERR_UNSUPPORTED_DTYPE;
    if (n == 0 || world == 1) return EXL3_OK;
    if (!aligned(data, 16) || peer_regions == nullptr || !aligned(state, 8)) return EXL3_ERR_BAD_POINTER;
    for (int r = 0; r < world; r++)
        if (!aligned(peer_regions[r], 256)) return EXL3_ERR_BAD_POINTER;
    return launch_allreduce(data, dtype == EXL3_BF16, n, peer_regions, rank, world, max_elems, state, (cudaStream_t)stream);
}

/* ---- MoE ------------------------------------------------------------------------------------------------------ */

namespace exl3 {
struct MoeWorkspace {
    size_t counters_off, partials_off, total;
};
static MoeWorkspace moe_workspace(int cap, int n_total)
{
    auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
    const size_t col_blocks = (size_t)(cap / MOE_BLOCK_ROWS) * (n_total / 128);
    MoeWorkspace w;
    w.counters_off = WS_HEADER_BYTES;
    w.partials_off = WS_SCRATCH_OFF;
    w.total = up(w.partials_off + (GEMV_MAX_GRID + col_blocks) * MOE_BLOCK_ROWS * 128 * sizeof(float));
    return w;
}
}  // namespace exl3

int exl3_moe_block_rows(void) { return MOE_BLOCK_ROWS; }

size_t exl3_moe_sorted_capacity(int slots, int num_experts)
{
    if (slots < 0 || num_experts < 1) return 0;
    size_t cap = (size_t)slots + (size_t)num_experts * (MOE_BLOCK_ROWS - 1);
    cap = (cap + MOE_BLOCK_ROWS - 1) / MOE_BLOCK_ROWS * MOE_BLOCK_ROWS;
    if (slots < num_experts && (size_t)slots * MOE_BLOCK_ROWS < cap) cap = (size_t)slots * MOE_BLOCK_ROWS;
    return cap;
}

exl3_status exl3_moe_align(const int32_t* topk_ids, int slots, int num_experts, int32_t* sorted_ids, int cap, int32_t* expert_ids,
                           int32_t* num_post, void* stream)
{
    if (slots < 0 || num_experts < 1 || num_experts > MOE_MAX_EXPERTS || cap < 0 || (cap % MOE_BLOCK_ROWS)) return EXL3_ERR_BAD_SHAPE;
    if ((size_t)cap < exl3_moe_sorted_capacity(slots, num_experts)) return EXL3_ERR_BAD_SHAPE;
    if (!aligned(num_post, 4) || (slots > 0 && !aligned(topk_ids, 4)) || (cap > 0 && (!aligned(sorted_ids, 4) || !aligned(expert_ids, 4))))
        return EXL3_ERR_BAD_POINTER;
    return launch_moe_align(topk_ids, slots, num_experts, MOE_BLOCK_ROWS, cap, sorted_ids, expert_ids, num_post, nullptr, 0,
                            (cudaStream_t)stream);
}

exl3_status exl3_moe_align_mapped(const int32_t* topk_ids, int slots, int num_experts, const int32_t* expert_map, int num_local,
                                  int32_t* sorted_ids, int cap, int32_t* expert_ids, int32_t* num_post, void* stream)
{
    if (slots < 0 || num_experts < 1 || num_local < 1 || num_local > MOE_MAX_EXPERTS || cap < 0 || (cap % MOE_BLOCK_ROWS)) return EXL3_ERR_BAD_SHAPE;
    if ((size_t)cap < exl3_moe_sorted_capacity(slots, num_local)) return EXL3_ERR_BAD_SHAPE;
    if (!expert_map || !aligned(expert_map, 4) || !aligned(num_post, 4) || (slots > 0 && !aligned(topk_ids, 4)) ||
        (cap > 0 && (!aligned(sorted_ids, 4) || !aligned(expert_ids, 4))))
        return EXL3_ERR_BAD_POINTER;
    return launch_moe_align(topk_ids, slots, num_local, MOE_BLOCK_ROWS, cap, sorted_ids, expert_ids, num_post, expert_map, num_experts,
                            (cudaStream_t)stream);
}

size_t exl3_moe_fragment_bytes(int cap, int k, int shards, int codebook)
{
    if (cap < 0 || k < 0 || shards < 1) return 0;
    return (size_t)shards * cap * (k / 16) * 4 * gemv_frag_words(gemv_default_mode(codebook)) * sizeof(uint32_t);
}

exl3_status exl3_moe_had_in(const void* x, int x_dtype, const uint16_t* suh, int shards, int hidden, int top_k, int slots,
                            const int32_t* sorted_ids, int cap, const int32_t* expert_ids, const int32_t* num_post, int codebook,
                            uint32_t* xf, void* stream)
{
    if (hidden < 0 || (hidden % 128) || shards < 1 || top_k < 1 || slots < 0 || cap < 0 || (cap % MOE_BLOCK_ROWS)) return EXL3_ERR_BAD_SHAPE;
    if (x_dtype != EXL3_F16 && x_dtype != EXL3_BF16) return EXL3_ERR_UNSUPPORTED_DTYPE;
    if (codebook < 0 || codebook > 2) return EXL3_ERR_UNSUPPORTED_CODEBOOK;
    if (cap == 0 || hidden == 0) return EXL3_OK;
    if (!aligned(x, 2) || !aligned(suh, 2) || !aligned(xf, 16) || !aligned(sorted_ids, 4) || !aligned(expert_ids, 4) || !aligned(num_post, 4))
        return EXL3_ERR_BAD_POINTER;
    return launch_moe_had_in(x, x_dtype == EXL3_BF16, reinterpret_cast<const __half*>(suh), shards, hidden, top_k, slots, cap, sorted_ids,
                             expert_ids, num_post, xf, gemv_default_mode(codebook), (cudaStream_t)stream);
}

exl3_status exl3_moe_glu_had_in(const uint16_t* gu, const uint16_t* suh2, int inter, int slots, const int32_t* sorted_ids, int cap,
                                const int32_t* expert_ids, const int32_t* num_post, int codebook, uint32_t* xf, void* stream)
{
    if (inter < 0 || (inter % 128) || slots < 0 || cap < 0 || (cap % MOE_BLOCK_ROWS)) return EXL3_ERR_BAD_SHAPE;
    if (codebook < 0 || codebook > 2) return EXL3_ERR_UNSUPPORTED_CODEBOOK;
    if (cap == 0 || inter == 0) return EXL3_OK;
    if (!aligned(gu, 2) || !aligned(suh2, 2) || !aligned(xf, 16) || !aligned(sorted_ids, 4) || !aligned(expert_ids, 4) || !aligned(num_post, 4))
        return EXL3_ERR_BAD_POINTER;
    return launch_moe_glu_had_in(reinterpret_cast<const __half*>(gu), reinterpret_cast<const __half*>(suh2), inter, slots, cap, sorted_ids,
                                 expert_ids, num_post, xf, gemv_default_mode(codebook), (cudaStream_t)stream);
}

size_t exl3_moe_workspace_bytes(int cap, int n_total)
{
    if (cap < 0 || n_total < 0) return 0;
    return moe_workspace(cap, n_total).total;
}

exl3_status exl3_moe_gemm(const uint32_t* xf, const uint32_t* packed, int K, int codebook, const uint16_t* svh, const int32_t* sorted_ids,
                          const int32_t* expert_ids, const int32_t* num_post, int cap, int slots, int k, int n_total, int shard_end,
                          uint16_t* out, void* workspace, size_t workspace_bytes, void* stream)
{
    if (int rc = check_matrix(k, n_total, K, codebook)) return rc;
    if (cap < 0 || (cap % MOE_BLOCK_ROWS) || slots < 0 || shard_end < 0 || shard_end > n_total || (shard_end % 128)) return EXL3_ERR_BAD_SHAPE;
    if (cap == 0 || k == 0 || n_total == 0) return EXL3_OK;
    if ((size_t)(cap / MOE_BLOCK_ROWS) * (size_t)(n_total / 128) > WS_MAX_COUNTERS) return EXL3_ERR_BAD_SHAPE;
    if (!current_device_info()) return EXL3_ERR_NOT_INITIALISED;
    if (!aligned(xf, 16) || !aligned(packed, 16) || !aligned(out, 8) || (svh && !aligned(svh, 8)) || !aligned(sorted_ids, 4) ||
        !aligned(expert_ids, 4) || !aligned(num_post, 4))
        return EXL3_ERR_BAD_POINTER;
    const MoeWorkspace wl = moe_workspace(cap, n_total);
    if (!aligned(workspace, 256) || workspace_bytes < wl.total) return EXL3_ERR_WORKSPACE;
    unsigned char* ws = reinterpret_cast<unsigned char*>(workspace);
    MoeGemmLaunch l;
    memset(&l, 0, sizeof(l));
    l.packed = packed;
    l.expert_stride = (long long)k * n_total * K / 32;
    l.xf = xf;
    l.xf_shard_stride = (long long)(cap / MOE_BLOCK_ROWS) * (k / 16) * 32;
    l.svh = reinterpret_cast<const __half*>(svh);
    l.out = reinterpret_cast<__half*>(out);
    l.sorted_ids = sorted_ids;
    l.expert_ids = expert_ids;
    l.num_post = num_post;
    l.partials = reinterpret_cast<float*>(ws + wl.partials_off);
    l.counters = reinterpret_cast<int*>(ws + wl.counters_off);
    l.err = reinterpret_cast<int*>(ws);
    l.KG = k / 128;
    l.NB = n_total / 128;
    l.n_total = n_total;
    l.numel = slots;
    l.shard_end_block = shard_end == 0 ? l.NB : shard_end / 128;
    l.rotated = svh == nullptr;
    return launch_moe_gemm(l, K, codebook, gemv_default_mode(codebook), (cudaStream_t)stream);
}

exl3_status exl3_moe_combine(const uint16_t* yd, const float* topk_weights, const int32_t* topk_ids, int tokens, int top_k, int hidden,
                             int num_experts, void* y, int y_dtype, void* stream)
{
    if (tokens < 0 || top_k < 1 || hidden < 0 || (hidden % 2) || num_experts < 1) return EXL3_ERR_BAD_SHAPE;
    if (y_dtype != EXL3_F16 && y_dtype != EXL3_BF16) return EXL3_ERR_UNSUPPORTED_DTYPE;
    if (tokens == 0 || hidden == 0) return EXL3_OK;
    if (!aligned(yd, 4) || !aligned(topk_weights, 4) || !aligned(topk_ids, 4) || !aligned(y, 4)) return EXL3_ERR_BAD_POINTER;
    return launch_moe_combine(reinterpret_cast<const __half*>(yd), topk_weights, topk_ids, tokens, top_k, hidden, num_experts, y,
                              y_dtype == EXL3_BF16, (cudaStream_t)stream);
}

int exl3_moe_tc_block_rows(void) { return MOE_TC_BLOCK_ROWS; }

size_t exl3_moe_tc_workspace_bytes(int slots, int num_local, int hidden, int inter)
{
    if (slots < 0 || num_local < 1 || hidden <= 0 || inter <= 0 || hidden % 128 || inter % 128) return 0;
    return moe_tc_workspace_bytes(slots, num_local, hidden, inter);
}

exl3_status exl3_moe_tc_experts(const void* x, int x_dtype, int tokens, int top_k, int hidden, int inter, const int32_t* topk_ids,
                                int num_experts, const int32_t* expert_map, int num_local, const uint32_t* w13, const uint16_t* suh13,
                                const uint16_t* svh13, const uint32_t* w2, const uint16_t* suh2, const uint16_t* svh2, int K, int codebook,
                                uint16_t* yd, void* workspace, size_t workspace_bytes, void* stream)
{
    if (int rc = check_matrix(hidden, 2 * inter, K, codebook)) return rc;
    if (int rc = check_matrix(inter, hidden, K, codebook)) return rc;
    if (tokens < 0 || top_k < 1 || num_experts < 1 || num_local < 1 || num_local > MOE_MAX_EXPERTS) return EXL3_ERR_BAD_SHAPE;
    if (!expert_map && num_local != num_experts) return EXL3_ERR_BAD_SHAPE;
    if ((long long)tokens * top_k > (1 << 24)) return EXL3_ERR_BAD_SHAPE;
    if (x_dtype != EXL3_F16 && x_dtype != EXL3_BF16) return EXL3_ERR_UNSUPPORTED_DTYPE;
    if (tokens == 0) return EXL3_OK;
    if (!current_device_info()) return EXL3_ERR_NOT_INITIALISED;
    if (!aligned(x, 16) || !aligned(topk_ids, 4) || !aligned(w13, 16) || !aligned(w2, 16) || !aligned(suh13, 16) || !aligned(svh13, 16) ||
        !aligned(suh2, 16) || !aligned(svh2, 16) || !aligned(yd, 16))
        return EXL3_ERR_BAD_POINTER;
    const int slots = tokens * top_k;
    if (!aligned(workspace, 256) || workspace_bytes < moe_tc_workspace_bytes(slots, num_local, hidden, inter)) return EXL3_ERR_WORKSPACE;
    return launch_moe_tc_experts(x, x_dtype == EXL3_BF16, top_k, hidden, inter, topk_ids, slots, num_experts, expert_map, num_local, w13,
                                 reinterpret_cast<const __half*>(suh13), reinterpret_cast<const __half*>(svh13), w2,
                                 reinterpret_cast<const __half*>(suh2), reinterpret_cast<const __half*>(svh2), K, codebook,
                                 reinterpret_cast<__half*>(yd), reinterpret_cast<unsigned char*>(workspace), (cudaStream_t)stream);
}

/* ---- exl3_linear_static: the fused linear for callers that cannot bring a workspace ---------------------------
 * Scratch (activation fragments, split-k partial sums, block counters, error word) lives in this file-scope device
 * array instead of a caller buffer.  Every GPU that loads the library holds the array until the process exits. */
static __device__ __align__(256) unsigned char g_static_workspace[EXL3_STATIC_WORKSPACE_BYTES];
static void* g_static_workspace_ptr[64];

// In host code the array's name is only a handle, not a device address: the address has to be asked for, once per
// device, with that device current.
static void* static_workspace_of_current_device(int* status)
{
    int dev = -1;
    *status = cuda_status(cudaGetDevice(&dev));
    if (*status) return nullptr;
    if (dev < 0 || dev >= 64) {
        *status = EXL3_ERR_BAD_SHAPE;
        return nullptr;
    }
    if (g_static_workspace_ptr[dev] == nullptr) {
        void* ptr = nullptr;
        *status = cuda_status(cudaGetSymbolAddress(&ptr, g_static_workspace));
        if (*status) return nullptr;
        if (ptr == nullptr) {
            *status = EXL3_ERR_CUDA;
            return nullptr;
        }
        g_static_workspace_ptr[dev] = ptr;
    }
    return g_static_workspace_ptr[dev];
}

exl3_status exl3_linear_static(const void* x, int x_dtype, const uint32_t* packed, int K, int codebook, const uint16_t* suh_cat,
                               const uint16_t* svh_cat, const int* shard_ends, int n_shards, int rows, int k, int n_total, void* y,
                               int y_dtype, void* stream)
{
    if (int rc = check_matrix(k, n_total, K, codebook)) return rc;
    if (rows < 0 || n_shards < 1) return EXL3_ERR_BAD_SHAPE;
    if (workspace_layout(rows, k, n_total, n_shards).total > EXL3_STATIC_WORKSPACE_BYTES) return EXL3_ERR_STATIC_WORKSPACE;
    int rc = EXL3_OK;
    void* ws = static_workspace_of_current_device(&rc);
    if (rc) return rc;
    return linear_common(x, x_dtype, nullptr, packed, K, codebook, suh_cat, svh_cat, shard_ends, n_shards, rows, k, n_total, y,
                         y_dtype, ws, EXL3_STATIC_WORKSPACE_BYTES, (cudaStream_t)stream, false);
}

size_t exl3_static_workspace_bytes(void) { return EXL3_STATIC_WORKSPACE_BYTES; }

/* Test / measurement knob: force how hash-codebook weights enter the MMA (-1 default, 0 split, 1 paired). */
void exl3_set_gemv_mode(int mode) { gemv_set_mode_override(mode); }

/* Test / measurement knob: output tiling of the many-row tensor-core GEMM (-1 choose, 0 = 512 x 128, 1 = 256 x 256, 2 = 384 x 128,
 * 3 = 512 x 256 on CTA pairs). */
void exl3_set_tc_tiling(int tiling) { gemm_tc_set_tiling(tiling); }

/* Test / measurement knob: at most `parts` parts of the reduction per tile in exl3_linear_tc (0 choose, 1 no split). */
void exl3_set_tc_ksplit(int parts) { gemm_tc_set_ksplit(parts); }

}  // extern "C"
