// Pieces shared by the dense decode GEMV (exl3_gemv_kernel.cuh) and the grouped MoE GEMV (exl3_moe_kernel.cuh): the
// even, contiguous split of a unit list over persistent CTAs, the register-level decode of one 16x16 tile into MMA
// operands, and the tensor-parallel exchange that a row-parallel linear runs in its epilogue.
#pragma once
#include "exl3_internal.h"
#include "exl3_ptx.cuh"

namespace exl3 {

enum { GEMV_ERR_FULL_WAIT = 1, GEMV_ERR_EMPTY_WAIT = 2, GEMV_ERR_PEER_WAIT = 3 };    // 2: the grouped MoE kernel's copy warp
constexpr uint32_t GEMV_PEER_MAX_POLLS = 1u << 20;       // bounded wait for a peer's words: about a second

#ifdef EXL3_TIMELINE
// Measurement build only: thread 0 of every CTA stamps %globaltimer at a few points of the kernel.
constexpr int TL_POINTS = 12, TL_SLOTS = 128, TL_CTAS = 512;
__device__ __forceinline__ unsigned long long tl_now()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define EXL3_STAMP(i) do { if (threadIdx.x == 0) p.tl[(blockIdx.x) * TL_POINTS + (i)] = tl_now(); } while (0)
#define EXL3_STAMP_ANY(i) do { if ((threadIdx.x & 31) == 0) p.tl[(blockIdx.x) * TL_POINTS + (i)] = tl_now(); } while (0)
#define EXL3_STAMP_CLK(i) do { if (threadIdx.x == 0) p.tl[(blockIdx.x) * TL_POINTS + (i)] = (unsigned long long)clock64(); } while (0)
#define EXL3_STAMP_SM(i) do { if (threadIdx.x == 0) { unsigned s_; asm volatile("mov.u32 %0, %%smid;" : "=r"(s_)); p.tl[(blockIdx.x) * TL_POINTS + (i)] = s_; } } while (0)
#else
#define EXL3_STAMP(i) do { } while (0)
#define EXL3_STAMP_ANY(i) do { } while (0)
#define EXL3_STAMP_CLK(i) do { } while (0)
#define EXL3_STAMP_SM(i) do { } while (0)
#endif

// Unit indices fit 32 bits (the host refuses matrices with 2^31 or more units).
__host__ __device__ inline long long gemv_first_unit(int cta, int q, int r) { return (long long)cta * q + (cta < r ? cta : r); }

__device__ __forceinline__ int gemv_cta_of_unit(long long u, int q, int r)
{
    long long boundary = (long long)r * (q + 1);
    return u < boundary ? (int)(u / (q + 1)) : r + (int)((u - boundary) / q);
}

template <int K, int MODE, int FAM>
__device__ __forceinline__ void decode_tile_regs(const LaneRegs<K>& R, const Pow2& pw, CodebookConst cbc, uint32_t (&w)[8])
{
    uint32_t s[8];
    s[0] = window_low<K, 0>(R, pw); s[1] = window_low<K, 1>(R, pw); s[2] = window_low<K, 2>(R, pw); s[3] = window_low<K, 3>(R, pw);
    s[4] = window_low<K, 4>(R, pw); s[5] = window_low<K, 5>(R, pw); s[6] = window_low<K, 6>(R, pw); s[7] = window_low<K, 7>(R, pw);
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

__device__ __forceinline__ float gemv_load_x(const void* p, long long idx, bool bf16)
{
    // bf16 inputs are first converted to fp16 (round to nearest even), as the stand-alone rotation kernel does.
    if (bf16) return __half2float(__float2half_rn(__bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[idx])));
    return __half2float(reinterpret_cast<const __half*>(p)[idx]);
}

// The same for a down projection fed straight from gate | up (row stride 2k): the activation silu(gate) * up, rounded to the
// activation type as the stand-alone activation kernel stores it, then taken as fp16.
__device__ __forceinline__ float gemv_load_glu(const void* p, long long idx, int k, bool bf16)
{
    float g, u;
    if (bf16) {
        g = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[idx]);
        u = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[idx + k]);
    } else {
        g = __half2float(reinterpret_cast<const __half*>(p)[idx]);
        u = __half2float(reinterpret_cast<const __half*>(p)[idx + k]);
    }
    const float act = g / (1.0f + __expf(-g)) * u;
    return __half2float(__float2half_rn(bf16 ? __bfloat162float(__float2bfloat16_rn(act)) : act));
}

__device__ __forceinline__ float gemv_raw(const void* p, long long idx, bool bf16)
{
    return bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[idx]) : __half2float(reinterpret_cast<const __half*>(p)[idx]);
}

__device__ __forceinline__ float gemv_round_act(float v, bool bf16)
{
    return bf16 ? __bfloat162float(__float2bfloat16_rn(v)) : __half2float(__float2half_rn(v));
}

// The normalised activation z * rstd * weight, rounded to the activation type (as the stand-alone normalisation kernel stores
// it) and taken as fp16.
__device__ __forceinline__ float gemv_load_norm(const void* z, const void* weight, long long idx, long long col, float rstd, bool bf16)
{
    const float a = gemv_round_act(gemv_raw(z, idx, bf16) * rstd * gemv_raw(weight, col, bf16), bf16);
    return __half2float(__float2half_rn(a));
}

// 1 / sqrt(mean square + eps) of a row of the residual stream from its per-block sums of squares (one warp, every lane gets
// the value): lane-strided loads, then a shuffle tree -- the same order in every CTA and every launch.
__device__ __forceinline__ float gemv_row_rstd(const float* ssq_row, int blocks, int k, float eps, int lane)
{
    float t = 0.f;
    for (int i = lane; i < blocks; i += 32) t += ssq_row[i];
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) t += __shfl_xor_sync(0xFFFFFFFFu, t, m);
    return rsqrtf(t / (float)k + eps);
}

// Row-parallel shard: 4 consecutive columns (index o) of one output row are a partial sum.  They go, rounded to the
// output type and tagged with the call number, into this rank's slot at every peer (single 64-bit peer stores); then
// the same words of all ranks are awaited here (bounded), added in rank order in fp32 and rounded once: the bits a
// separate all-reduce of the rounded outputs gives.  Kept out of line: it runs once per 128 outputs and must not
// weigh on the register allocation of the decode loop.
static __device__ __noinline__ void gemv_exchange_store(const TpExchange& tp, uint32_t tp_epoch, bool bf, const float (&v)[4], long long o,
                                                 uint16_t* out, int* err)
{
    uint32_t w2[2];
#pragma unroll
    for (int e = 0; e < 2; e++) {
        const __half2 hh = __floats2half2_rn(v[2 * e], v[2 * e + 1]);
        if (bf) {
            const __nv_bfloat162 bb = __floats2bfloat162_rn(__low2float(hh), __high2float(hh));
            w2[e] = *reinterpret_cast<const uint32_t*>(&bb);
        } else {
            w2[e] = *reinterpret_cast<const uint32_t*>(&hh);
        }
    }
    const size_t set_off = (size_t)TP_HEADER_BYTES + (size_t)(tp_epoch & 1u) * tp.world * tp.slot_bytes;
    const size_t word = (size_t)(o >> 1);                    // 32-bit word of two values inside a slot
    const unsigned long long tag = (unsigned long long)tp_epoch << 32;
    for (int r = 0; r < tp.world; r++) {
        unsigned long long* dst = reinterpret_cast<unsigned long long*>(tp.base[r] + set_off + (size_t)tp.rank * tp.slot_bytes) + word;
        ptx::st_relaxed_sys_v2u64(dst, tag | w2[0], tag | w2[1]);          // word is even: 16-byte aligned
    }
    float a[4] = {0.f, 0.f, 0.f, 0.f};
    const unsigned char* own = tp.base[tp.rank] + set_off;
    bool gave_up = *reinterpret_cast<volatile int*>(err) != 0;       // a wait that already ran out is not repeated block after block
    constexpr int BATCH = 4;                      // ranks whose words are requested together: their latencies overlap
    for (int r0 = 0; r0 < tp.world; r0 += BATCH) {
        unsigned long long got[BATCH][2];
#pragma unroll
        for (int j = 0; j < BATCH; j++) {
            const int r = r0 + j < tp.world ? r0 + j : tp.world - 1;
            const unsigned long long* src = reinterpret_cast<const unsigned long long*>(own + (size_t)r * tp.slot_bytes) + word;
            ptx::ld_relaxed_sys_v2u64(src, got[j][0], got[j][1]);
        }
#pragma unroll
        for (int j = 0; j < BATCH; j++) {
            if (r0 + j < tp.world) {
                const unsigned long long* src = reinterpret_cast<const unsigned long long*>(own + (size_t)(r0 + j) * tp.slot_bytes) + word;
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    uint32_t polls = 0;
                    while ((uint32_t)(got[j][e] >> 32) != tp_epoch && !gave_up) {
                        if (++polls > GEMV_PEER_MAX_POLLS) {
                            gave_up = true;
                            atomicExch(err, GEMV_ERR_PEER_WAIT);
                            break;
                        }
                        got[j][e] = ptx::ld_relaxed_sys_u64(src + e);
                    }
                    const uint32_t lo = (uint32_t)got[j][e];
                    if (bf) {
                        const __nv_bfloat162 bb = *reinterpret_cast<const __nv_bfloat162*>(&lo);
                        a[2 * e] += __low2float(bb);
                        a[2 * e + 1] += __high2float(bb);
                    } else {
                        const __half2 hh = *reinterpret_cast<const __half2*>(&lo);
                        a[2 * e] += __low2float(hh);
                        a[2 * e + 1] += __high2float(hh);
                    }
                }
            }
        }
    }
    uint2 res;
    if (bf) {
        const __nv_bfloat162 b0 = __floats2bfloat162_rn(a[0], a[1]), b1 = __floats2bfloat162_rn(a[2], a[3]);
        res = make_uint2(*reinterpret_cast<const uint32_t*>(&b0), *reinterpret_cast<const uint32_t*>(&b1));
    } else {
        const __half2 h0 = __floats2half2_rn(a[0], a[1]), h1 = __floats2half2_rn(a[2], a[3]);
        res = make_uint2(*reinterpret_cast<const uint32_t*>(&h0), *reinterpret_cast<const uint32_t*>(&h1));
    }
    *reinterpret_cast<uint2*>(out + o) = res;
}

// Residual epilogue of one row's block of 128 outputs (one warp, four columns per lane): y -- summed over the ranks first, if
// there is an exchange -- rounded as it would be stored, plus the residual stream: the new stream goes to res_out, this block's
// share of its mean square to ssq_out, y itself to `out` only if that is set.  Out of line: once per 128 outputs.
static __device__ __noinline__ void gemv_residual_store(const GemvArgs& a, uint32_t tp_epoch, const float (&v)[4], long long o, int m, int fnb,
                                                        int lane)
{
    const bool bf = a.out_dtype == EXL3_BF16;
    float y[4];
    if (a.tp.world > 1) {
        gemv_exchange_store(a.tp, tp_epoch, bf, v, o, reinterpret_cast<uint16_t*>(a.out), a.err);
#pragma unroll
        for (int e = 0; e < 4; e++) y[e] = gemv_raw(a.out, o + e, bf);       // what the exchange stored
    } else {
#pragma unroll
        for (int e = 0; e < 4; e++) y[e] = gemv_round_act(__half2float(__float2half_rn(v[e])), bf);
        if (a.out) {
#pragma unroll
            for (int e = 0; e < 4; e++) {
                if (bf) reinterpret_cast<__nv_bfloat16*>(a.out)[o + e] = __float2bfloat16_rn(y[e]);
                else reinterpret_cast<__half*>(a.out)[o + e] = __float2half_rn(y[e]);
            }
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < 4; e++) {
        const float z = gemv_round_act(y[e] + gemv_raw(a.res_in, o + e, bf), bf);
        ss += z * z;
        if (bf) reinterpret_cast<__nv_bfloat16*>(a.res_out)[o + e] = __float2bfloat16_rn(z);
        else reinterpret_cast<__half*>(a.res_out)[o + e] = __float2half_rn(z);
    }
#pragma unroll
    for (int m2 = 16; m2 > 0; m2 >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, m2);
    if (lane == 0) a.ssq_out[(size_t)m * (a.n_total >> 7) + fnb] = ss;
}

}  // namespace exl3
