// One-shot all-reduce over peer-mapped memory (NVLink 5 / NVSwitch) for the partial outputs of row-parallel EXL3
// linears (o_proj, down_proj): [rows, hidden] fp16 or bf16, 10 KB at batch 1.  The reference has no collectives at
// all (tensor parallelism is refused at cuda/src/sglang_exl3/sglang_glue/linear.py:74-75); the exchange step follows
// from its slicing rules (core/src/trellis_core/format/geometry.py:62-66): row slices produce partial sums.
//
// Messages this small are latency-bound, so one kernel does everything: every rank copies its vector into its own
// peer-visible slot, raises a flag in every peer's memory, waits (bounded) until all peers have raised theirs, then
// reads all slots with ordinary peer loads and adds them in rank order in fp32 (deterministic, identical on all
// ranks).  Slots are double-buffered by call parity: a rank can be at most one call ahead of a peer, because it
// cannot pass the flag wait of call e+1 before that peer has finished call e.
//
// Per-rank symmetric region: [world flags, 128 bytes apart][slot 0][slot 1].  No multicast, no multimem.
#include "exl3_internal.h"

namespace exl3 {

constexpr int AR_FLAG_STRIDE = 32;            // uint32 units: one 128-byte line per peer flag
constexpr int AR_MAX_WORLD = 16;
constexpr uint32_t AR_MAX_POLLS = 1u << 21;   // bounded wait: about a second, then give up
enum { AR_ERR_WAIT = 4 };

struct ArPeers {
    unsigned char* base[AR_MAX_WORLD];
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) { asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p)
{
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// state[0] = number of calls completed (epoch), state[1] = error word.  One CTA.
template <bool BF16>
__global__ void __launch_bounds__(1024, 1) allreduce_oneshot_kernel(uint16_t* __restrict__ data, size_t n, ArPeers peers, int rank, int world,
                                                                    size_t slot_bytes, int* __restrict__ state)
{
    const uint32_t epoch = (uint32_t)state[0] + 1u;
    const size_t slot_off = (size_t)AR_MAX_WORLD * AR_FLAG_STRIDE * 4 + (size_t)(epoch & 1u) * slot_bytes;
    const size_t n16 = n / 8;                                   // 16-byte chunks (n is a multiple of 8)
    uint4* mine = reinterpret_cast<uint4*>(peers.base[rank] + slot_off);
    const uint4* src = reinterpret_cast<const uint4*>(data);
    for (size_t i = threadIdx.x; i < n16; i += blockDim.x) mine[i] = src[i];
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < world) {
        // tell peer p that this rank's slot for this call is complete ...
        st_release_sys(reinterpret_cast<uint32_t*>(peers.base[threadIdx.x]) + rank * AR_FLAG_STRIDE, epoch);
        // ... and wait until peer p has told us the same
        const uint32_t* flag = reinterpret_cast<const uint32_t*>(peers.base[rank]) + threadIdx.x * AR_FLAG_STRIDE;
        uint32_t polls = 0;
        while ((int32_t)(ld_acquire_sys(flag) - epoch) < 0) {
            if (++polls > AR_MAX_POLLS) {
                atomicExch(&state[1], AR_ERR_WAIT);
                break;
            }
        }
    }
    __syncthreads();
    uint4* dst = reinterpret_cast<uint4*>(data);
    for (size_t i = threadIdx.x; i < n16; i += blockDim.x) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int r = 0; r < world; r++) {
            uint4 v;                              // plain peer load, not cached in L1 across calls
            asm volatile("ld.global.cv.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(peers.base[r] + slot_off + i * 16) : "memory");
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int e = 0; e < 4; e++) {
                if (BF16) {
                    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&w[e]);
                    acc[2 * e] += __low2float(b);
                    acc[2 * e + 1] += __high2float(b);
                } else {
                    const __half2 h = *reinterpret_cast<const __half2*>(&w[e]);
                    acc[2 * e] += __low2float(h);
                    acc[2 * e + 1] += __high2float(h);
                }
            }
        }
        uint32_t o[4];
#pragma unroll
        for (int e = 0; e < 4; e++) {
            if (BF16) {
                const __nv_bfloat162 b = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
                o[e] = *reinterpret_cast<const uint32_t*>(&b);
            } else {
                const __half2 h = __floats2half2_rn(acc[2 * e], acc[2 * e + 1]);
                o[e] = *reinterpret_cast<const uint32_t*>(&h);
            }
        }
        dst[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
    __syncthreads();
    if (threadIdx.x == 0) state[0] = (int)epoch;
}

size_t allreduce_region_bytes(size_t max_elems) { return (size_t)AR_MAX_WORLD * AR_FLAG_STRIDE * 4 + 2 * ((max_elems * 2 + 255) & ~(size_t)255); }

int launch_allreduce(void* data, int bf16, size_t n, void* const* peer_bases_host, int rank, int world, size_t max_elems, int* state,
                     cudaStream_t st)
{
    ArPeers peers;
    for (int r = 0; r < AR_MAX_WORLD; r++) peers.base[r] = r < world ? reinterpret_cast<unsigned char*>(peer_bases_host[r]) : nullptr;
    const size_t slot_bytes = (max_elems * 2 + 255) & ~(size_t)255;
    if (bf16) allreduce_oneshot_kernel<true><<<1, 1024, 0, st>>>(reinterpret_cast<uint16_t*>(data), n, peers, rank, world, slot_bytes, state);
    else allreduce_oneshot_kernel<false><<<1, 1024, 0, st>>>(reinterpret_cast<uint16_t*>(data), n, peers, rank, world, slot_bytes, state);
    return cuda_status(cudaGetLastError());
}

}  // namespace exl3
