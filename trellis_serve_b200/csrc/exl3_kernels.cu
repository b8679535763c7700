// Layout, decode-to-dense and Hadamard kernels of the EXL3 linear (sm_100a).
//
//   repack / unpack        stored trellis <-> resident layout (exl3_decode.cuh), exact inverses
//                          (replaces repack_trellis / unpack_trellis, cuda/csrc/exl3_marlin.cu:344-408)
//   reconstruct            trellis -> fp16 W_inner [k, n]  (core/src/trellis_core/reference.py:102-115)
//   had_in / had_out       128-point rotations with the suh / svh vectors
//                          (cuda/csrc/exl3_marlin.cu:257-306, cuda/csrc/exl3_had.cuh:20-84)
#include "exl3_internal.h"

namespace exl3 {

// ------------------------------------------------------------------------------------------------ repack

// One thread per packed word.  Every bit is fetched from its place in the stored stream: load-time only.
__global__ void repack_kernel(const uint16_t* __restrict__ trellis, uint32_t* __restrict__ packed, int KG, int NB, int K,
                              long long total_words)
{
    long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (idx >= total_words) return;
    int lane = (int)(idx & 31);
    long long r = idx >> 5;
    int i = (int)(r % K);
    r /= K;
    int kq = (int)(r & 1);
    r >>= 1;
    int nt = (int)(r & 7);
    r >>= 3;
    int kg = (int)(r % KG);
    int nb = (int)(r / KG);
    const int ntiles_n = NB * 8;
    uint32_t out = 0;
    for (int b = 0; b < 32; b++) {
        int pos = 32 * i + b;                 // bit of the lane stream
        int t = pos / (8 * K);
        int o = pos % (8 * K);
        int sb = 8 * K * lane + o;            // bit of the tile's stream
        long long tile = (long long)(kg * 8 + kq * 4 + t) * ntiles_n + nb * 8 + nt;
        const uint16_t* tw = trellis + tile * 16 * K;
        int w = sb >> 5;
        uint32_t word = (uint32_t)tw[2 * w] | ((uint32_t)tw[2 * w + 1] << 16);
        out = (out << 1) | ((word >> (31 - (sb & 31))) & 1u);
    }
    packed[idx] = out;
}

// One thread per stored 32-bit stream word.
__global__ void unpack_kernel(const uint32_t* __restrict__ packed, uint16_t* __restrict__ trellis, int KG, int NB, int K,
                              long long total_words)
{
    long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (idx >= total_words) return;
    const int words_per_tile = 8 * K;
    int w = (int)(idx % words_per_tile);
    long long tile = idx / words_per_tile;
    const int ntiles_n = NB * 8;
    int tn = (int)(tile % ntiles_n);
    int tk = (int)(tile / ntiles_n);
    int nb = tn >> 3, nt = tn & 7, kg = tk >> 3, kq = (tk >> 2) & 1, t = tk & 3;
    uint32_t out = 0;
    for (int b = 0; b < 32; b++) {
        int sb = 32 * w + b;
        int lane = sb / (8 * K);
        int o = sb % (8 * K);
        int pos = 8 * K * t + o;
        int i = pos >> 5;
        long long pidx = ((((((long long)nb * KG + kg) * 8 + nt) * 2 + kq) * K + i) << 5) + lane;
        out = (out << 1) | ((packed[pidx] >> (31 - (pos & 31))) & 1u);
    }
    trellis[2 * idx] = (uint16_t)(out & 0xFFFF);
    trellis[2 * idx + 1] = (uint16_t)(out >> 16);
}

// ------------------------------------------------------------------------------------------------ reconstruct

// From the stored stream, any K: one warp per tile, lane l decodes elements 8l..8l+7 with run-time bit
// arithmetic (circular inside the tile).
__global__ void reconstruct_stored_kernel(const uint16_t* __restrict__ trellis, __half* __restrict__ w, int kt, int nt, int K,
                                          int family, CodebookConst cbc)
{
    const int lane = threadIdx.x & 31;
    long long tile = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);
    if (tile >= (long long)kt * nt) return;
    const uint32_t* tw = reinterpret_cast<const uint32_t*>(trellis + tile * 16 * K);   // 8K little-endian words
    const int nbits = 256 * K, nwords = 8 * K;
    const int ti = (int)(tile / nt), tj = (int)(tile % nt);
    const int n = nt * 16;
#pragma unroll
    for (int j = 0; j < 8; j++) {
        int t = 8 * lane + j;
        int b0 = (t * K + K - 16 + nbits) % nbits;       // first bit of the window
        int w0 = b0 >> 5, sh = b0 & 31;
        uint32_t hi = tw[w0], lo = tw[(w0 + 1) % nwords];
        uint32_t state = __funnelshift_l(lo, hi, sh) >> 16;
        __half v = decode_value(state, family, cbc);
        w[(long long)(ti * 16 + tile_row(lane, j)) * n + tj * 16 + tile_col(lane, j)] = v;
    }
}

// From the resident layout with the same lane-local extraction the GEMV / GEMM kernels use.
// One warp per (nb, kg, nt, kq): four tiles.
template <int K>
__global__ void reconstruct_packed_kernel(const uint32_t* __restrict__ packed, __half* __restrict__ w, int KG, int NB, int family,
                                          CodebookConst cbc)
{
    const int lane = threadIdx.x & 31;
    long long quad = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);
    if (quad >= (long long)NB * KG * 16) return;
    uint32_t L[K];
#pragma unroll
    for (int i = 0; i < K; i++) L[i] = packed[(quad * K + i) * 32 + lane];
    long long r = quad;
    int kq = (int)(r & 1);
    r >>= 1;
    int nt = (int)(r & 7);
    r >>= 3;
    int kg = (int)(r % KG);
    int nb = (int)(r / KG);
    const int n = NB * 128;
    const int col0 = nb * 128 + nt * 16;

    auto emit = [&](auto tconst) {
        constexpr int T = decltype(tconst)::value;
        uint32_t own[2];
        own_words<K, T>(L, own);
        uint32_t prev0 = __shfl_sync(0xFFFFFFFFu, own[0], (lane + 31) & 31);
        LaneTile<K> lt = assemble<K>(own, prev0);
        uint32_t s[8];
        s[0] = window<K, 0>(lt); s[1] = window<K, 1>(lt); s[2] = window<K, 2>(lt); s[3] = window<K, 3>(lt);
        s[4] = window<K, 4>(lt); s[5] = window<K, 5>(lt); s[6] = window<K, 6>(lt); s[7] = window<K, 7>(lt);
        const int row0 = (kg * 8 + kq * 4 + T) * 16;
#pragma unroll
        for (int j = 0; j < 8; j++)
            w[(long long)(row0 + tile_row(lane, j)) * n + col0 + tile_col(lane, j)] = decode_value(s[j], family, cbc);
    };
    emit(std::integral_constant<int, 0>{});
    emit(std::integral_constant<int, 1>{});
    emit(std::integral_constant<int, 2>{});
    emit(std::integral_constant<int, 3>{});
}

// ------------------------------------------------------------------------------------------------ Hadamard

__device__ __forceinline__ void ptx_grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void ptx_grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ float load_as_f16_value(const void* p, long long idx, bool bf16)
{
    // bf16 inputs are first converted to fp16 (round to nearest even, overflow to +-inf), the value
    // conversion torch's x.to(float16) performs; the GEMM always runs on fp16 activations.
    if (bf16) {
        float f = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[idx]);
        return __half2float(__float2half_rn(f));
    }
    return __half2float(reinterpret_cast<const __half*>(p)[idx]);
}

// xh = Had128(fp16(x) * suh[s]) for every shard s.  One warp per (shard, row, 128-block).
// MODE 0: row-major fp16 [shards*rows, k] (slab s = rows s*rows..).
// MODE 1: B-operand fragments for the split-pair MMA: [shard][k/16][rows][4 lanes q][4 words], every word one
//         fp16 value duplicated in both halves; word order x[2q], x[2q+1], x[2q+8], x[2q+9] of the 16-row tile.
// MODE 2: B-operand fragments for the paired MMA: [shard][k/16][rows][4 lanes q][2 words]:
//         (x[2q], x[2q+1]), (x[2q+8], x[2q+9]).
template <int MODE>
__global__ void had_in_kernel(const void* __restrict__ x, int x_bf16, const __half* __restrict__ suh, int shards, int rows, int k,
                              void* __restrict__ out)
{
    ptx_grid_launch_dependents();              // the GEMV behind this kernel may start streaming weights already
    ptx_grid_dependency_wait();                // x may be the output of the kernel ahead
    const int lane = threadIdx.x & 31;
    const int kgs = k >> 7;
    long long item = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (long long)shards * rows * kgs) return;
    const int kg = (int)(item % kgs);
    const int row = (int)((item / kgs) % rows);
    const int s = (int)(item / ((long long)kgs * rows));
    float v[4];
#pragma unroll
    for (int e = 0; e < 4; e++) {
        int col = kg * 128 + 4 * lane + e;
        float xv = load_as_f16_value(x, (long long)row * k + col, x_bf16 != 0);
        v[e] = suh ? xv * __half2float(suh[(long long)s * k + col]) : xv;
    }
    fwht128(v[0], v[1], v[2], v[3], lane);
    __half h[4];
#pragma unroll
    for (int e = 0; e < 4; e++) h[e] = __float2half_rn(v[e] * HAD_SCALE);

    if constexpr (MODE == 0) {
        __half* o = reinterpret_cast<__half*>(out) + ((long long)s * rows + row) * k + kg * 128 + 4 * lane;
        *reinterpret_cast<uint2*>(o) = make_uint2(
            (uint32_t)__half_as_ushort(h[0]) | ((uint32_t)__half_as_ushort(h[1]) << 16),
            (uint32_t)__half_as_ushort(h[2]) | ((uint32_t)__half_as_ushort(h[3]) << 16));
    } else {
        // lane holds tile-local rows r = 4*(lane&3) + e of 16-row tile kt = kg*8 + lane/4
        const int kt = kg * 8 + (lane >> 2);
        const int rbase = 4 * (lane & 3);
        if constexpr (MODE == 1) {
            uint32_t* o = reinterpret_cast<uint32_t*>(out) + (((long long)s * (k >> 4) + kt) * rows + row) * 16;
#pragma unroll
            for (int e = 0; e < 4; e++) {
                int r = rbase + e;
                int q = (r & 7) >> 1;
                int slot = (r & 1) + 2 * (r >> 3);
                uint32_t hv = __half_as_ushort(h[e]);
                o[q * 4 + slot] = hv | (hv << 16);
            }
        } else {
            uint32_t* o = reinterpret_cast<uint32_t*>(out) + (((long long)s * (k >> 4) + kt) * rows + row) * 8;
#pragma unroll
            for (int e = 0; e < 4; e += 2) {
                int r = rbase + e;
                int q = (r & 7) >> 1;
                int slot = r >> 3;
                o[q * 2 + slot] = (uint32_t)__half_as_ushort(h[e]) | ((uint32_t)__half_as_ushort(h[e + 1]) << 16);
            }
        }
    }
}

// Row-major fp16 xh [shards*rows, k] (already rotated) -> fragment layouts of had_in_kernel MODE 1 / 2.
template <int MODE>
__global__ void to_fragments_kernel(const __half* __restrict__ xh, int shards, int rows, int k, uint32_t* __restrict__ out)
{
    long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;      // one thread per (s, row, kt, q)
    const int kts = k >> 4;
    if (idx >= (long long)shards * rows * kts * 4) return;
    int q = (int)(idx & 3);
    long long r = idx >> 2;
    int kt = (int)(r % kts);
    r /= kts;
    int row = (int)(r % rows);
    int s = (int)(r / rows);
    const __half* src = xh + ((long long)s * rows + row) * k + kt * 16;
    uint32_t a = __half_as_ushort(src[2 * q]), b = __half_as_ushort(src[2 * q + 1]);
    uint32_t c = __half_as_ushort(src[2 * q + 8]), d = __half_as_ushort(src[2 * q + 9]);
    if constexpr (MODE == 1) {
        uint4* o = reinterpret_cast<uint4*>(out) + (((long long)s * kts + kt) * rows + row) * 4 + q;
        *o = make_uint4(a | (a << 16), b | (b << 16), c | (c << 16), d | (d << 16));
    } else {
        uint2* o = reinterpret_cast<uint2*>(out) + (((long long)s * kts + kt) * rows + row) * 4 + q;
        *o = make_uint2(a | (b << 16), c | (d << 16));
    }
}

__device__ __forceinline__ void store_out4(void* out, long long idx, const float (&v)[4], bool bf16)
{
    // Results are rounded to fp16 first; a bf16 output is that fp16 value converted (torch's y.to(bfloat16)).
    __half h[4];
#pragma unroll
    for (int e = 0; e < 4; e++) h[e] = __float2half_rn(v[e]);
    if (bf16) {
        __nv_bfloat16 b[4];
#pragma unroll
        for (int e = 0; e < 4; e++) b[e] = __float2bfloat16_rn(__half2float(h[e]));
        *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(out) + idx) = *reinterpret_cast<uint2*>(b);
    } else {
        *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(out) + idx) = *reinterpret_cast<uint2*>(h);
    }
}

// out[row, col0 + j] = Had128(y[row, :])[j] * svh[j].  y is fp16 (IN_F32 = false) or fp32 [rows, n].  One warp per (group of
// HAD_OUT_ROWS rows, 128 columns), four lanes per row with 32 columns each (fwht128_quad).
constexpr int HAD_OUT_ROWS = 8;
template <bool IN_F32>
__global__ void had_out_kernel(const void* __restrict__ y, const __half* __restrict__ svh, int rows, int n, void* __restrict__ out,
                               long long out_stride, int out_bf16)
{
    const int lane = threadIdx.x & 31;
    const int nbs = n >> 7;
    const int groups = (rows + HAD_OUT_ROWS - 1) / HAD_OUT_ROWS;
    long long item = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (long long)groups * nbs) return;
    const int nb = (int)(item % nbs);
    const int row = (int)(item / nbs) * HAD_OUT_ROWS + (lane >> 2);
    const int col = nb * 128 + 32 * (lane & 3);
    const bool live = row < rows;
    float v[32];
    if (live) {
        const long long base = (long long)row * n + col;
        if (IN_F32) {
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const float4 f = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(y) + base)[i];
                v[4 * i] = f.x; v[4 * i + 1] = f.y; v[4 * i + 2] = f.z; v[4 * i + 3] = f.w;
            }
        } else {
            load_half32(reinterpret_cast<const __half*>(y) + base, v);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 32; i++) v[i] = 0.f;
    }
    fwht128_quad(v, lane);                        // every lane takes part in the shuffles
    if (live) had_out_finish(v, svh, col, out, (long long)row * out_stride + col, out_bf16);
}

// The output rotation for the cut tiles of the CTA-pair tiling of the many-row GEMM (tiles of 512 rows x 256 columns; tile =
// column tile x row_tiles + row tile; the tiles before `tail_first` leave that kernel finished): the sum of `parts` fp32
// slabs part[(tile - tail_first) * parts + s][512][256], added in part order and rounded to fp16 once, as the kernel rounds
// the accumulators of a tile it did not cut.  One warp per (cut tile, 8 rows, 128 columns).
__global__ void had_out_tiles_kernel(const float* __restrict__ part, int parts, int tail_first, int row_tiles, int cut_tiles,
                                     const __half* __restrict__ svh, int rows, int n, void* __restrict__ out, int out_bf16)
{
    const int lane = threadIdx.x & 31;
    long long item = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (long long)cut_tiles * 128) return;
    const int j = (int)(item >> 7), rg = (int)(item & 127) >> 1, half = (int)(item & 1);
    const int tile = tail_first + j;
    const int row_in = rg * HAD_OUT_ROWS + (lane >> 2), row = (tile % row_tiles) * 512 + row_in;
    const int col = (tile / row_tiles) * 256 + half * 128 + 32 * (lane & 3);
    const bool live = row < rows;
    float v[32];
#pragma unroll
    for (int i = 0; i < 32; i++) v[i] = 0.f;
    if (live) {
        const float* src = part + (size_t)j * parts * (512 * 256) + (size_t)row_in * 256 + half * 128 + 32 * (lane & 3);
        for (int s = 0; s < parts; s++, src += 512 * 256) {
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const float4 f = reinterpret_cast<const float4*>(src)[i];
                v[4 * i] += f.x; v[4 * i + 1] += f.y; v[4 * i + 2] += f.z; v[4 * i + 3] += f.w;
            }
        }
#pragma unroll
        for (int i = 0; i < 32; i++) v[i] = __half2float(__float2half_rn(v[i]));
    }
    fwht128_quad(v, lane);
    if (live) had_out_finish(v, svh, col, out, (long long)row * n + col, out_bf16);
}

// out[row, :] = Had128(fp16(sum over parts of part[s][row, :])) * svh: the output rotation of the many-row path when the
// reduction was split over CTAs; the slabs are added in part order in fp32 and rounded to fp16 once, as the unsplit
// kernel rounds its accumulators.
__global__ void had_out_sum_kernel(const float* __restrict__ part, int parts, long long slab, const __half* __restrict__ svh, int rows,
                                   int n, void* __restrict__ out, int out_bf16)
{
    const int lane = threadIdx.x & 31;
    const int nbs = n >> 7;
    long long item = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (long long)rows * nbs) return;
    const int nb = (int)(item % nbs);
    const int row = (int)(item / nbs);
    const long long base = (long long)row * n + nb * 128 + 4 * lane;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < parts; s++) {
        const float4 v = *reinterpret_cast<const float4*>(part + s * slab + base);
        acc.x += v.x;
        acc.y += v.y;
        acc.z += v.z;
        acc.w += v.w;
    }
    float v[4] = {__half2float(__float2half_rn(acc.x)), __half2float(__float2half_rn(acc.y)), __half2float(__float2half_rn(acc.z)),
                  __half2float(__float2half_rn(acc.w))};
    fwht128(v[0], v[1], v[2], v[3], lane);
#pragma unroll
    for (int e = 0; e < 4; e++) {
        float sv = svh ? __half2float(svh[nb * 128 + 4 * lane + e]) : 1.0f;
        v[e] = v[e] * (HAD_SCALE * sv);          // the same order as the epilogues fused into the GEMV kernels
    }
    store_out4(out, base, v, out_bf16 != 0);
}

// ------------------------------------------------------------------------------------------------ launchers

static inline unsigned blocks_for(long long items, int per_block) { return (unsigned)((items + per_block - 1) / per_block); }

int launch_repack(const uint16_t* trellis, int k, int n, int K, uint32_t* packed, cudaStream_t st)
{
    long long words = (long long)k * n * K / 32;
    if (words == 0) return EXL3_OK;
    repack_kernel<<<blocks_for(words, 256), 256, 0, st>>>(trellis, packed, k / 128, n / 128, K, words);
    return cuda_status(cudaGetLastError());
}

int launch_unpack(const uint32_t* packed, int k, int n, int K, uint16_t* trellis, cudaStream_t st)
{
    long long words = (long long)k * n * K / 32;
    if (words == 0) return EXL3_OK;
    unpack_kernel<<<blocks_for(words, 256), 256, 0, st>>>(packed, trellis, k / 128, n / 128, K, words);
    return cuda_status(cudaGetLastError());
}

int launch_reconstruct_stored(const uint16_t* trellis, int kt, int nt, int K, int cb, __half* w, cudaStream_t st)
{
    long long tiles = (long long)kt * nt;
    if (tiles == 0) return EXL3_OK;
    reconstruct_stored_kernel<<<blocks_for(tiles, 8), 256, 0, st>>>(trellis, w, kt, nt, K, codebook_family(cb), codebook_const(cb));
    return cuda_status(cudaGetLastError());
}

template <int K>
static int launch_reconstruct_packed_k(const uint32_t* packed, int k, int n, int cb, __half* w, cudaStream_t st)
{
    long long quads = (long long)(n / 128) * (k / 128) * 16;
    reconstruct_packed_kernel<K><<<blocks_for(quads, 8), 256, 0, st>>>(packed, w, k / 128, n / 128, codebook_family(cb), codebook_const(cb));
    return cuda_status(cudaGetLastError());
}

int launch_reconstruct_packed(const uint32_t* packed, int k, int n, int K, int cb, __half* w, cudaStream_t st)
{
    if ((long long)k * n == 0) return EXL3_OK;
    switch (K) {
        case 2: return launch_reconstruct_packed_k<2>(packed, k, n, cb, w, st);
        case 3: return launch_reconstruct_packed_k<3>(packed, k, n, cb, w, st);
        case 4: return launch_reconstruct_packed_k<4>(packed, k, n, cb, w, st);
        case 5: return launch_reconstruct_packed_k<5>(packed, k, n, cb, w, st);
        case 6: return launch_reconstruct_packed_k<6>(packed, k, n, cb, w, st);
        case 7: return launch_reconstruct_packed_k<7>(packed, k, n, cb, w, st);
        case 8: return launch_reconstruct_packed_k<8>(packed, k, n, cb, w, st);
    }
    return EXL3_ERR_UNSUPPORTED_K;
}

int launch_had_in(const void* x, int x_bf16, const __half* suh, int shards, int rows, int k, void* out, int mode, cudaStream_t st)
{
    long long items = (long long)shards * rows * (k / 128);
    if (items == 0) return EXL3_OK;
    // programmatic stream serialization: see the GEMV launcher
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(blocks_for(items, 8));
    cfg.blockDim = dim3(256);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (mode == 0) return cuda_status(cudaLaunchKernelEx(&cfg, had_in_kernel<0>, x, x_bf16, suh, shards, rows, k, out));
    if (mode == 1) return cuda_status(cudaLaunchKernelEx(&cfg, had_in_kernel<1>, x, x_bf16, suh, shards, rows, k, out));
    return cuda_status(cudaLaunchKernelEx(&cfg, had_in_kernel<2>, x, x_bf16, suh, shards, rows, k, out));
}

int launch_to_fragments(const __half* xh, int shards, int rows, int k, uint32_t* out, int mode, cudaStream_t st)
{
    long long items = (long long)shards * rows * (k / 16) * 4;
    if (items == 0) return EXL3_OK;
    if (mode == 1) to_fragments_kernel<1><<<blocks_for(items, 256), 256, 0, st>>>(xh, shards, rows, k, out);
    else to_fragments_kernel<2><<<blocks_for(items, 256), 256, 0, st>>>(xh, shards, rows, k, out);
    return cuda_status(cudaGetLastError());
}

int launch_had_out(const void* y, int y_f32, const __half* svh, int rows, int n, void* out, long long out_stride, int out_bf16,
                   cudaStream_t st)
{
    long long items = (long long)((rows + HAD_OUT_ROWS - 1) / HAD_OUT_ROWS) * (n / 128);
    if (items == 0) return EXL3_OK;
    if (y_f32) had_out_kernel<true><<<blocks_for(items, 8), 256, 0, st>>>(y, svh, rows, n, out, out_stride, out_bf16);
    else had_out_kernel<false><<<blocks_for(items, 8), 256, 0, st>>>(y, svh, rows, n, out, out_stride, out_bf16);
    return cuda_status(cudaGetLastError());
}

int launch_had_out_tiles(const float* part, int parts, int tail_first, int row_tiles, const __half* svh, int rows, int n, void* out,
                         int out_bf16, cudaStream_t st)
{
    const int cut_tiles = row_tiles * (n / 256) - tail_first;
    if (cut_tiles <= 0) return EXL3_OK;
    had_out_tiles_kernel<<<blocks_for((long long)cut_tiles * 128, 8), 256, 0, st>>>(part, parts, tail_first, row_tiles, cut_tiles, svh, rows, n, out,
                                                                                  out_bf16);
    return cuda_status(cudaGetLastError());
}

int launch_had_out_sum(const float* part, int parts, long long slab, const __half* svh, int rows, int n, void* out, int out_bf16,
                       cudaStream_t st)
{
    long long items = (long long)rows * (n / 128);
    if (items == 0) return EXL3_OK;
    had_out_sum_kernel<<<blocks_for(items, 8), 256, 0, st>>>(part, parts, slab, svh, rows, n, out, out_bf16);
    return cuda_status(cudaGetLastError());
}

}  // namespace exl3
