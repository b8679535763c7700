// EXL3 trellis decode primitives for sm_100a: lane-local window extraction for any K in 2..8, the three
// computed codebooks, and a 128-point Walsh-Hadamard transform held in one warp.
//
// Written from the format description, not from the reference's kernels.  What each piece corresponds to in
// 0xSero/trellis-serve:
//   windows / bit order   core/src/trellis_core/reference.py:81-99   (cuda/csrc/exl3_decode.cuh:149-360 for K=3..6)
//   codebooks             core/src/trellis_core/reference.py:53-73   (cuda/csrc/third_party/exllamav3/codebook.cuh:56-123)
//   tile placement        core/src/trellis_core/reference.py:30-45
//   Hadamard              core/src/trellis_core/reference.py:119-130 (cuda/csrc/exl3_had.cuh:20-84)
//
// Resident ("packed") layout used by every kernel here.  It is a pure permutation of the stored bits, so
// the packed-weight byte count is unchanged (k*n*K/8):
//
//   packed[nb][kg][nt][kq][i][lane]   uint32
//     nb   = output column block of 128            (n / 128)
//     kg   = input row block of 128                (k / 128)
//     nt   = 16-column tile inside the block       (8)
//     kq   = group of four 16-row tiles            (2)
//     i    = word of the lane's stream             (K)
//     lane = 32
//
// The "lane stream" of (nb, kg, nt, kq, lane) is B0|B1|B2|B3, where Bt are stream bits [8K*lane, 8K*(lane+1))
// of tile (row tile kg*8 + kq*4 + t, column tile nb*8 + nt), first stream bit in the most significant
// position.  Lane `lane` therefore owns stream elements 8*lane .. 8*lane+7 of each of its four tiles; the
// 16-K bits that element 8*lane also needs from the previous lane arrive by one warp shuffle per tile.
// One (nb, kg) unit is 2048*K contiguous bytes: a bulk-copy friendly stage.
#pragma once
#include <cstdint>
#include <cuda_fp16.h>
#include <cuda_bf16.h>

namespace exl3 {

constexpr int CB_3INST = 0;
constexpr int CB_MCG = 1;
constexpr int CB_MUL1 = 2;

constexpr uint32_t MUL_3INST = 89226354u;
constexpr uint32_t ADD_3INST = 64248484u;
constexpr uint32_t MUL_MCG = 0xCBAC1FEDu;
constexpr uint32_t MUL_MUL1 = 0x83DCD12Du;

// Codebook family as the kernels see it: the two "hash" codebooks differ only in two constants.
constexpr int FAM_HASH = 0;   // 3INST, MCG: x = s*mul + add; (x & 0x8FFF8FFF) ^ 0x3B603B60; value = lo + hi
constexpr int FAM_MUL1 = 1;   // MUL1: x = s*mul; value = fma(half(0x6400 + bytesum(x)), 0x1EEE, 0xC931)

struct CodebookConst {
    uint32_t mul;
    uint32_t add;
};

__host__ __device__ inline CodebookConst codebook_const(int cb)
{
    if (cb == CB_3INST) return {MUL_3INST, ADD_3INST};
    if (cb == CB_MCG) return {MUL_MCG, 0u};
    return {MUL_MUL1, 0u};
}

__host__ __device__ inline int codebook_family(int cb) { return cb == CB_MUL1 ? FAM_MUL1 : FAM_HASH; }

// ---------------------------------------------------------------------------------------------- bit helpers

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel)
{
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}

// 32 bits of the lane stream L (K words, bit b of the stream = bit 31-(b%32) of word b/32) that end at bit
// position END (exclusive), right-aligned.  Bits before the start of the stream read as zero.
template <int K, int END>
__device__ __forceinline__ uint32_t stream_bits_ending_at(const uint32_t (&L)[K])
{
    static_assert(END > 0 && END <= 32 * K, "window end outside the lane stream");
    constexpr int wi = END / 32;
    constexpr int r = END % 32;
    if constexpr (r == 0) {
        return L[wi - 1];
    } else if constexpr (wi == 0) {
        return L[0] >> (32 - r);
    } else {
        return __funnelshift_l(L[wi], L[wi - 1], r);
    }
}

// The lane's view of one tile: E = (last 16-K bits of the previous lane's share) | (own 8K bits),
// right-aligned in up to three words.  Element p (0..7) of the lane is E bits [K*(7-p), K*(7-p)+16).
template <int K>
struct LaneTile {
    uint32_t e[3];
};

// Own share of tile T (0..3) right-aligned: word 0 = last 32 own bits, word 1 = the 32 before, ...
// Words above the own share contain neighbouring bits of the stream; assemble() masks or replaces them.
template <int K, int T>
__device__ __forceinline__ void own_words(const uint32_t (&L)[K], uint32_t (&o)[2])
{
    constexpr int END = 8 * K * (T + 1);
    o[0] = stream_bits_ending_at<K, END>(L);
    if constexpr (8 * K > 32) {
        o[1] = stream_bits_ending_at<K, END - 32>(L);
    } else {
        o[1] = 0;
    }
}

// own: this lane's right-aligned words; prev0: word 0 of the previous lane's right-aligned share of the same tile.
template <int K>
__device__ __forceinline__ LaneTile<K> assemble(const uint32_t (&own)[2], uint32_t prev0)
{
    LaneTile<K> t;
    if constexpr (K == 2) {            // own 16 bits
        t.e[0] = prmt(own[0], prev0, 0x5410);
        t.e[1] = 0;
        t.e[2] = 0;
    } else if constexpr (K == 3) {     // own 24 bits
        t.e[0] = prmt(own[0], prev0, 0x4210);
        t.e[1] = prev0 >> 8;
        t.e[2] = 0;
    } else if constexpr (K == 4) {     // own 32 bits
        t.e[0] = own[0];
        t.e[1] = prev0;
        t.e[2] = 0;
    } else if constexpr (K == 5) {     // own 40 bits
        t.e[0] = own[0];
        t.e[1] = prmt(own[1], prev0, 0x6540);
        t.e[2] = 0;
    } else if constexpr (K == 6) {     // own 48 bits
        t.e[0] = own[0];
        t.e[1] = prmt(own[1], prev0, 0x5410);
        t.e[2] = 0;
    } else if constexpr (K == 7) {     // own 56 bits
        t.e[0] = own[0];
        t.e[1] = prmt(own[1], prev0, 0x4210);
        t.e[2] = prev0 >> 8;
    } else {                           // K == 8, own 64 bits
        t.e[0] = own[0];
        t.e[1] = own[1];
        t.e[2] = prev0;
    }
    return t;
}

// 16-bit trellis state of element P (0..7) of the lane.
template <int K, int P>
__device__ __forceinline__ uint32_t window(const LaneTile<K>& t)
{
    constexpr int lo = K * (7 - P);
    constexpr int wi = lo / 32;
    constexpr int sh = lo % 32;
    if constexpr (sh == 0) {
        return t.e[wi] & 0xFFFFu;
    } else if constexpr (sh == 16) {
        return t.e[wi] >> 16;
    } else if constexpr (sh + 16 <= 32) {
        return (t.e[wi] >> sh) & 0xFFFFu;
    } else {
        return __funnelshift_r(t.e[wi], t.e[wi + 1], sh) & 0xFFFFu;
    }
}

// ---------------------------------------------------------------------------------------------- pipe-balanced windows
//
// On sm_100 shifts, logic ops and byte permutes all issue on the ALU pipe (16 lanes per scheduler) while integer
// multiply-add issues on the equally wide FMA pipe, and the ALU pipe is what bounds the decode.  A shift-and-mask
// extraction costs two ALU slots per weight on top of the codebook's logic op.  Here a window is instead cut out with one
// multiply by a power of two (drops the bits above the window, FMA pipe) and one shift right by 16 (drops the bits below,
// ALU pipe): E is re-read as 32-bit registers R_j = E[16j, 16j+32), so every window lies inside one of them.  Windows
// that start on a byte boundary (all of them at K = 8, half at K = 4) take a single mask or byte permute.  The powers of
// two come from kernel parameters (constant bank) so that the multiply stays a multiply.

struct Pow2 {
    uint32_t v[32];          // v[c] = 1 << c
};

__host__ inline Pow2 make_pow2()
{
    Pow2 p;
    for (int c = 0; c < 32; c++) p.v[c] = 1u << c;
    return p;
}

template <int K>
struct LaneRegs {
    uint32_t r[4];           // r[j] = E bits [16j, 16j + 32)
};

template <int K>
__device__ __forceinline__ LaneRegs<K> lane_regs(const uint32_t (&own)[2], uint32_t prev0)
{
    LaneRegs<K> R;
    if constexpr (K == 2) {
        R.r[0] = prmt(own[0], prev0, 0x5410);
        R.r[1] = R.r[2] = R.r[3] = 0;
    } else if constexpr (K == 3) {
        R.r[0] = prmt(own[0], prev0, 0x4210);
        R.r[1] = prmt(own[0], prev0, 0x6542);
        R.r[2] = R.r[3] = 0;
    } else if constexpr (K == 4) {
        R.r[0] = own[0];
        R.r[1] = prmt(own[0], prev0, 0x5432);
        R.r[2] = R.r[3] = 0;
    } else {
        const LaneTile<K> t = assemble<K>(own, prev0);
        R.r[0] = t.e[0];
        R.r[1] = prmt(t.e[0], t.e[1], 0x5432);
        R.r[2] = t.e[1];
        R.r[3] = (K >= 7) ? prmt(t.e[1], t.e[2], 0x5432) : 0u;
    }
    return R;
}

// 16-bit trellis state of element P (0..7) of the lane, bits above it cleared.
template <int K, int P>
__device__ __forceinline__ uint32_t window_low(const LaneRegs<K>& R, const Pow2& pw)
{
    constexpr int lo = K * (7 - P);
    constexpr int j = lo / 16;
    constexpr int sh = lo % 16;
    static_assert(j < 4, "window outside the lane registers");
    if constexpr (sh == 0) {
        return R.r[j] & 0xFFFFu;
    } else if constexpr (sh == 8) {
        return prmt(R.r[j], 0u, 0x4421);          // byte-aligned window (K = 2, 4, 6, 8): one permute
    } else {
        return (R.r[j] * pw.v[16 - sh]) >> 16;
    }
}

// ---------------------------------------------------------------------------------------------- codebooks

// Hash codebooks: the register holds two fp16 numbers whose sum is the weight.
__device__ __forceinline__ uint32_t hash_pair(uint32_t state, CodebookConst c)
{
    // One multiply-add and ONE three-input logic op: with both masks in registers (a & b) ^ c is a single lop3;
    // written as C it compiles to two instructions because each can carry only one 32-bit immediate.
    uint32_t x = state * c.mul + c.add, d;
    asm("lop3.b32 %0, %1, %2, %3, 0x6a;" : "=r"(d) : "r"(x), "r"(0x8FFF8FFFu), "r"(0x3B603B60u));
    return d;
}

// One weight, fp16, rounded once: bit-identical to the codebook table of the reference decoder.
__device__ __forceinline__ __half decode_value(uint32_t state, int family, CodebookConst c)
{
    if (family == FAM_HASH) {
        uint32_t x = hash_pair(state, c);
        __half2 h = *reinterpret_cast<__half2*>(&x);
        return __hadd(__low2half(h), __high2half(h));
    }
    uint32_t x = state * c.mul;
    uint32_t bits = __dp4a(x, 0x01010101u, 0x6400u);
    __half h = __ushort_as_half(static_cast<unsigned short>(bits));
    return __hfma(h, __ushort_as_half(0x1EEE), __ushort_as_half(0xC931));
}

// Two MUL1 weights at once: states a, b -> half2(value(a), value(b)).
__device__ __forceinline__ uint32_t mul1_pair(uint32_t sa, uint32_t sb, CodebookConst c)
{
    uint32_t ha = __dp4a(sa * c.mul, 0x01010101u, 0x6400u);
    uint32_t hb = __dp4a(sb * c.mul, 0x01010101u, 0x6400u);
    uint32_t packed = prmt(ha, hb, 0x5410);
    __half2 h = *reinterpret_cast<__half2*>(&packed);
    const __half2 m = __half2half2(__ushort_as_half(0x1EEE));
    const __half2 a = __half2half2(__ushort_as_half(0xC931));
    __half2 v = __hfma2(h, m, a);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Two hash-codebook weights rounded to fp16: half2(value(a), value(b)).
__device__ __forceinline__ uint32_t hash_pair_rounded(uint32_t sa, uint32_t sb, CodebookConst c)
{
    uint32_t xa = hash_pair(sa, c), xb = hash_pair(sb, c);
    uint32_t lo = prmt(xa, xb, 0x5410), hi = prmt(xa, xb, 0x7632);
    __half2 v = __hadd2(*reinterpret_cast<__half2*>(&lo), *reinterpret_cast<__half2*>(&hi));
    return *reinterpret_cast<uint32_t*>(&v);
}

// ---------------------------------------------------------------------------------------------- placement

// Element j (0..7) of lane l sits at row 2*(l&3) + (j&1) + 8*((j>>1)&1), column (l>>2) + 8*(j>>2) of the tile.
__device__ __forceinline__ int tile_row(int lane, int j) { return 2 * (lane & 3) + (j & 1) + 8 * ((j >> 1) & 1); }
__device__ __forceinline__ int tile_col(int lane, int j) { return (lane >> 2) + 8 * (j >> 2); }

// ---------------------------------------------------------------------------------------------- Hadamard

// 128-point transform across a warp: lane l holds elements 4l..4l+3.  Unnormalised.
__device__ __forceinline__ void fwht128(float& v0, float& v1, float& v2, float& v3, int lane)
{
    float a0 = v0 + v1, a1 = v0 - v1, a2 = v2 + v3, a3 = v2 - v3;
    v0 = a0 + a2;
    v1 = a1 + a3;
    v2 = a0 - a2;
    v3 = a1 - a3;
#pragma unroll
    for (int m = 1; m < 32; m <<= 1) {
        float p0 = __shfl_xor_sync(0xFFFFFFFFu, v0, m);
        float p1 = __shfl_xor_sync(0xFFFFFFFFu, v1, m);
        float p2 = __shfl_xor_sync(0xFFFFFFFFu, v2, m);
        float p3 = __shfl_xor_sync(0xFFFFFFFFu, v3, m);
        const bool upper = (lane & m) != 0;
        v0 = upper ? p0 - v0 : v0 + p0;
        v1 = upper ? p1 - v1 : v1 + p1;
        v2 = upper ? p2 - v2 : v2 + p2;
        v3 = upper ? p3 - v3 : v3 + p3;
    }
}

// The same transform with a row spread over FOUR lanes (lane l holds elements 32 * (l & 3) .. + 31 of row l >> 2, eight rows
// per warp): five stages stay inside the lane and only two cross lanes, 64 shuffles for eight rows where the layout above
// needs 160 -- the shuffle unit is what bounds the rotation kernels of the many-row paths.  Same stage order (strides 1, 2, ...,
// 64) and the same sums and differences, so the results are the same bits.
__device__ __forceinline__ void fwht128_quad(float (&v)[32], int lane)
{
#pragma unroll
    for (int stride = 1; stride < 32; stride <<= 1) {
#pragma unroll
        for (int i = 0; i < 32; i++) {
            if ((i & stride) == 0) {
                const float lo = v[i], hi = v[i + stride];
                v[i] = lo + hi;
                v[i + stride] = lo - hi;
            }
        }
    }
#pragma unroll
    for (int m = 1; m < 4; m <<= 1) {
        const bool upper = (lane & m) != 0;
#pragma unroll
        for (int i = 0; i < 32; i++) {
            const float p = __shfl_xor_sync(0xFFFFFFFFu, v[i], m);
            v[i] = upper ? p - v[i] : v[i] + p;
        }
    }
}

constexpr float HAD_SCALE = 0.08838834764831845f;   // 1 / sqrt(128)

// 32 consecutive halves (64 bytes, 16-byte aligned) as floats.
__device__ __forceinline__ void load_half32(const __half* __restrict__ src, float (&v)[32])
{
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint4 raw = reinterpret_cast<const uint4*>(src)[i];
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const __half2 h = *reinterpret_cast<const __half2*>(&w[j]);
            v[8 * i + 2 * j] = __low2float(h);
            v[8 * i + 2 * j + 1] = __high2float(h);
        }
    }
}

// A lane's 32 rotated values -> out[at .. at + 31] = fp16(v * (scale * svh[col ..])), or that value converted to bf16: the
// order of the fused epilogues.
__device__ __forceinline__ void had_out_finish(const float (&v)[32], const __half* __restrict__ svh, int col, void* __restrict__ out, long long at,
                                               int out_bf16)
{
    uint32_t packed[16];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        uint4 sraw = make_uint4(0x3C003C00u, 0x3C003C00u, 0x3C003C00u, 0x3C003C00u);       // ones
        if (svh) sraw = reinterpret_cast<const uint4*>(svh + col)[i];
        const uint32_t sw[4] = {sraw.x, sraw.y, sraw.z, sraw.w};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const __half2 sh = *reinterpret_cast<const __half2*>(&sw[j]);
            const __half2 h = __floats2half2_rn(v[8 * i + 2 * j] * (HAD_SCALE * __low2float(sh)), v[8 * i + 2 * j + 1] * (HAD_SCALE * __high2float(sh)));
            if (out_bf16) {
                const __nv_bfloat162 bb = __floats2bfloat162_rn(__low2float(h), __high2float(h));
                packed[4 * i + j] = *reinterpret_cast<const uint32_t*>(&bb);
            } else {
                packed[4 * i + j] = *reinterpret_cast<const uint32_t*>(&h);
            }
        }
    }
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(out) + at);
#pragma unroll
    for (int i = 0; i < 4; i++) dst[i] = make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
}

}  // namespace exl3
