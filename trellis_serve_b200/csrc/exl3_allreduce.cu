// One-shot all-reduce over peer-mapped memory (NVLink 5 / NVSwitch) for the partial outputs of row-parallel EXL3
// linears (o_proj, down_proj): [rows, hidden] fp16 or bf16, 10 KB at batch 1.  The reference has no collectives at
// all (tensor parallelism is refused at cuda/src/sglang_exl3/sglang_glue/linear.py:74-75); the exchange step follows
// from its slicing rules (core/src/trellis_core/format/geometry.py:62-66): row slices produce partial sums.
//
// Messages this small are latency-bound, so one kernel does everything, nothing is ever loaded across NVLink and
// there is no separate flag round: every rank PUSHES its vector into its own slot of every peer's region as 8-byte
// words {two values, call number} written with single 64-bit stores; a receiver polls (bounded) each word of its own
// region until it carries the current call number, which proves that its two values have arrived, and adds the slots
// in rank order in fp32 (deterministic, identical on all ranks).  One NVLink store flight is the whole exchange: no
// fence, no flag store behind the data.  Slot sets are double-buffered by call parity: a rank can be at most one call
// ahead of a peer, because it cannot finish call e before it has received that peer's words of call e, which the peer
// sends only after it has finished reading call e-1.  The kernel is launched with programmatic stream serialization,
// so its launch overlaps the tail of the linear ahead of it.
//
// Per-rank symmetric region: [256-byte header][parity 0: world slots][parity 1: world slots], slot = 4 bytes per element.
// No multicast, no multimem.
#include "exl3_internal.h"
#include "exl3_ptx.cuh"

namespace exl3 {

constexpr int AR_HEADER_BYTES = TP_HEADER_BYTES;
constexpr int AR_MAX_WORLD = TP_MAX_WORLD;
constexpr uint32_t AR_MAX_POLLS = 1u << 20;   // bounded wait per word: about a second, then give up
enum { AR_ERR_WAIT = 4 };

struct ArPeers {
    unsigned char* base[AR_MAX_WORLD];
};

// state[0] = number of calls completed (epoch), state[1] = error word.  One CTA.
template <bool BF16>
__global__ void __launch_bounds__(1024, 1) allreduce_oneshot_kernel(uint16_t* __restrict__ data, size_t n, ArPeers peers, int rank, int world,
                                                                    size_t slot_bytes, int* __restrict__ state)
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // data is the output of the kernel ahead; the call counter was written by the previous call, which is certain to be
    // complete only once the kernels between it and this one are (each of them waits for the one ahead of it).
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t epoch = (uint32_t)state[0] + 1u;
    const size_t set_off = (size_t)AR_HEADER_BYTES + (size_t)(epoch & 1u) * world * slot_bytes;
    const size_t nw = n / 2;                                    // 32-bit words of two values (n is a multiple of 8)
    const uint32_t* src = reinterpret_cast<const uint32_t*>(data);
    // push: this rank's words, tagged with the call number, into slot `rank` of every region (its own included)
    for (size_t i = threadIdx.x; i < nw; i += blockDim.x) {
        const unsigned long long tagged = (unsigned long long)src[i] | ((unsigned long long)epoch << 32);
        for (int r = 0; r < world; r++)
            ptx::st_relaxed_sys_u64(reinterpret_cast<unsigned long long*>(peers.base[r] + set_off + (size_t)rank * slot_bytes) + i, tagged);
    }
    uint32_t* dst = reinterpret_cast<uint32_t*>(data);
    const unsigned char* own = peers.base[rank] + set_off;
    bool gave_up = false;                         // once a wait has run out the thread stops waiting for the other words too
    constexpr int BATCH = 8;                      // ranks whose words are requested together: their latencies overlap
    for (size_t i = threadIdx.x; i < nw; i += blockDim.x) {
        float a0 = 0.f, a1 = 0.f;
        for (int r0 = 0; r0 < world; r0 += BATCH) {
            unsigned long long v[BATCH];
#pragma unroll
            for (int j = 0; j < BATCH; j++) {
                const int r = r0 + j < world ? r0 + j : world - 1;
                v[j] = ptx::ld_relaxed_sys_u64(reinterpret_cast<const unsigned long long*>(own + (size_t)r * slot_bytes) + i);
            }
#pragma unroll
            for (int j = 0; j < BATCH; j++) {
                if (r0 + j < world) {
                    const unsigned long long* w = reinterpret_cast<const unsigned long long*>(own + (size_t)(r0 + j) * slot_bytes) + i;
                    uint32_t polls = 0;
                    while ((uint32_t)(v[j] >> 32) != epoch && !gave_up) {
                        if (++polls > AR_MAX_POLLS) {
                            gave_up = true;
                            atomicExch(&state[1], AR_ERR_WAIT);
                            break;
                        }
                        v[j] = ptx::ld_relaxed_sys_u64(w);
                    }
                    const uint32_t lo = (uint32_t)v[j];
                    if (BF16) {
                        const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&lo);
                        a0 += __low2float(b);
                        a1 += __high2float(b);
                    } else {
                        const __half2 h = *reinterpret_cast<const __half2*>(&lo);
                        a0 += __low2float(h);
                        a1 += __high2float(h);
                    }
                }
            }
        }
        uint32_t o;
        if (BF16) {
            const __nv_bfloat162 b = __floats2bfloat162_rn(a0, a1);
            o = *reinterpret_cast<const uint32_t*>(&b);
        } else {
            const __half2 h = __floats2half2_rn(a0, a1);
            o = *reinterpret_cast<const uint32_t*>(&h);
        }
        dst[i] = o;
    }
    __syncthreads();
    if (threadIdx.x == 0) state[0] = (int)epoch;
}

size_t allreduce_region_bytes(size_t max_elems)
{
    return (size_t)AR_HEADER_BYTES + 2 * (size_t)AR_MAX_WORLD * ((max_elems * 4 + 255) & ~(size_t)255);
}

int launch_allreduce(void* data, int bf16, size_t n, void* const* peer_bases_host, int rank, int world, size_t max_elems, int* state,
                     cudaStream_t st)
{
    ArPeers peers;
    for (int r = 0; r < AR_MAX_WORLD; r++) peers.base[r] = r < world ? reinterpret_cast<unsigned char*>(peer_bases_host[r]) : nullptr;
    const size_t slot_bytes = (max_elems * 4 + 255) & ~(size_t)255;
    auto kernel = bf16 ? allreduce_oneshot_kernel<true> : allreduce_oneshot_kernel<false>;
    return launch_chained(kernel, dim3(1), dim3(1024), 0, st, reinterpret_cast<uint16_t*>(data), n, peers, rank, world, slot_bytes, state);
}

}  // namespace exl3
