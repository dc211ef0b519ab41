// Device side of the feature-slice all-gather over peer memory, shared by the gather kernels (peer.cu) and by the
// kernels that push their own output (the split-path fold of the matmuls, the split merge of decode attention).
//
// A kernel that produces this rank's slice out[rows, f] of a [rows, R*f] activation stores every element straight
// into columns [rank*f, (rank+1)*f) of the destination buffer of EVERY rank (plain stores through peer mappings,
// NVLink on the way) and ends with push_handshake(): fence system-wide; the last CTA of the launch raises this
// rank's epoch flag at every peer and, if asked to, waits (bounded) for theirs.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include "bi_common.cuh"
#include "bi_ptx.cuh"

namespace bi {

constexpr int MAX_RANKS = 8;
constexpr uint64_t GATHER_WAIT_NS = 2000000000ull;

struct PeerPtrs {
    void* p[MAX_RANKS];
};

// Where a pushing kernel sends its output. counters[0]: CTAs of the current launch that have pushed their part;
// counters[1]: epoch of the last gather. wait == 0: raise the flags and return; whoever reads the gathered buffer
// waits for the peers' flags itself.
struct PushSink {
    PeerPtrs dst, flags;
    unsigned* counters;
    int32_t* status;
    int rank, world, wait;
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* addr) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
    return v;
}

__device__ __forceinline__ void st_relaxed_sys(uint32_t* addr, uint32_t v) {
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}

// Called by every thread of every CTA of the launch, after its stores (no early return before it).
// Ordering: the CTA barrier puts every thread's stores before thread 0's system-wide fence (fences are cumulative),
// the fence before the CTA's arrival count; the last CTA to arrive fences once more (it has observed every other
// CTA's count, hence their fenced stores) and only then raises the flags, with relaxed stores that need not wait for
// one another: one NVLink round trip for all peers instead of one per peer.
__device__ __forceinline__ void push_handshake(int rank, int R, const PeerPtrs& flags, unsigned* counters, int32_t* status, int wait) {
    __syncthreads();
    if (threadIdx.x != 0) return;
    __threadfence_system();
    if (atomicAdd(&counters[0], 1u) != gridDim.x - 1) return;
    // last CTA of this rank: every store of the launch has been fenced
    atomicExch(&counters[0], 0u);
    const uint32_t epoch = counters[1] + 1u;
    counters[1] = epoch;
    __threadfence_system();
    for (int r = 0; r < R; ++r)
        if (r != rank) st_relaxed_sys(static_cast<uint32_t*>(flags.p[r]) + rank, epoch);
    if (!wait) return;
    const uint32_t* mine = static_cast<const uint32_t*>(flags.p[rank]);
    const uint64_t t0 = ptx::globaltimer_ns();
    for (int r = 0; r < R; ++r) {
        if (r == rank) continue;
        while ((int32_t)(ld_acquire_sys(mine + r) - epoch) < 0) {
            if (ptx::globaltimer_ns() - t0 > GATHER_WAIT_NS) {
                if (status) atomicCAS(status, 0, (int)(0x20000 | (r << 8) | (epoch & 0xff)));
                return;
            }
        }
    }
}
__device__ __forceinline__ void push_handshake(const PushSink& s) {
    push_handshake(s.rank, s.world, s.flags, s.counters, s.status, s.wait);
}

// Host: fill a PushSink from the C-ABI's pointer tables. `align` is what the pushing kernel's stores need.
inline int make_sink(const char* op, void* const* dst, void* const* flags, uint32_t* counters, int rank, int world, int wait,
                     int32_t* status, size_t align, PushSink* s) {
    if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world)
        return fail(BI_ERR_BAD_ARG, "%s: rank %d of %d (at most %d ranks)", op, rank, world, MAX_RANKS);
    if (!dst || !flags || !counters) return fail(BI_ERR_BAD_ARG, "%s: null pointer", op);
    *s = PushSink{};
    for (int r = 0; r < world; ++r) {
        if (!dst[r] || !flags[r]) return fail(BI_ERR_BAD_ARG, "%s: null peer pointer for rank %d", op, r);
        if (!aligned(dst[r], align)) return fail(BI_ERR_MISALIGNED, "%s: destination of rank %d is not %zu-byte aligned", op, r, align);
        s->dst.p[r] = dst[r];
        s->flags.p[r] = flags[r];
    }
    s->counters = counters;
    s->status = status;
    s->rank = rank;
    s->world = world;
    s->wait = wait;
    return BI_OK;
}

}  // namespace bi
