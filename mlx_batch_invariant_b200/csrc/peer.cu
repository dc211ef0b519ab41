// Feature-slice all-gather over peer memory, for the sharded decoder runner.
//
// Every rank owns a slice local[rows, f] of a [rows, R*f] activation and every rank needs the whole
// activation. One launch per rank: the CTAs store the local slice straight into columns
// [rank*f, (rank+1)*f) of the destination buffer of EVERY rank (plain 16-byte stores through peer
// mappings, NVLink on the way), fence system-wide, and the last CTA to finish raises this rank's flag
// in every peer's flag array and then waits until every peer has raised its flag in the local array.
// When the kernel returns, the local destination holds all R slices, already in [rows, R*f] order (no
// transpose copy afterwards, no library collective). Nothing but bytes moves, so the result cannot
// depend on R.
//
// Protocol state: flags are epochs (a device-side counter that every launch advances by one, so a
// captured CUDA graph can be replayed), destination buffers are used in rotation by the caller (three or
// more: a peer can run at most one gather ahead of the slowest rank, because it needs that rank's flag
// of the gather before). The wait is bounded (2 s by %globaltimer); on expiry the kernel stores a code in
// the caller's status word and returns.
//
// Buffers that peers write into are allocated here (cudaMalloc, so that a CUDA IPC handle can name
// them) and opened in the other ranks' processes by handle; exchanging the 64-byte handles is the
// caller's business (the runner uses its process group).
#include <cstring>
#include "bi_common.cuh"
#include "bi_ptx.cuh"
#include "peer_push.cuh"

namespace bi {
namespace {

__global__ void __launch_bounds__(256) push_gather_kernel(const uint4* __restrict__ local, long long rows, int f16, int rank,
                                                          int R, PeerPtrs dst, PeerPtrs flags, unsigned* counters,
                                                          int32_t* status, int wait) {
    ptx::grid_dep_launch();   // the next kernel of the stream may start its set-up
    ptx::grid_dep_wait();     // everything before this kernel has completed and is visible
    const long long total = rows * f16;
    const long long pitch = (long long)R * f16;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long m = i / f16;
        const long long o = m * pitch + (long long)rank * f16 + (i - m * f16);
        const uint4 v = local[i];
        for (int r = 0; r < R; ++r) static_cast<uint4*>(dst.p[r])[o] = v;
    }
    push_handshake(rank, R, flags, counters, status, wait);
}

// The SwiGLU gate and the gather that follows it, in one kernel: this rank's slice out[m, j] = T(silu(gu[m, j]) *
// gu[m, F + j]) (the arithmetic of bi_swiglu, element for element) is computed eight elements at a time and stored
// straight into columns [rank * F, (rank + 1) * F) of every rank's gathered activation -- the local slice never
// exists in memory, and the transfer overlaps the arithmetic piece by piece.
template <typename T>
__global__ void __launch_bounds__(256) push_gather_swiglu_kernel(const T* __restrict__ gu, long long rows, int F, int rank, int R,
                                                                 PeerPtrs dst, PeerPtrs flags, unsigned* counters,
                                                                 int32_t* status, int wait) {
    ptx::grid_dep_launch();   // the next kernel of the stream may start its set-up
    ptx::grid_dep_wait();     // everything before this kernel has completed and is visible
    constexpr int V = 16 / (int)sizeof(T);
    const int f16 = F / V;
    const long long total = rows * f16;
    const long long pitch = (long long)R * f16;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long m = i / f16;
        const int c = (int)(i - m * f16);
        const uint4 gq = *reinterpret_cast<const uint4*>(gu + m * 2 * F + (long long)c * V);
        const uint4 uq = *reinterpret_cast<const uint4*>(gu + m * 2 * F + F + (long long)c * V);
        const T* gp = reinterpret_cast<const T*>(&gq);
        const T* up = reinterpret_cast<const T*>(&uq);
        uint4 oq;
        T* op = reinterpret_cast<T*>(&oq);
#pragma unroll
        for (int e = 0; e < V; ++e) op[e] = Cvt<T>::down(swiglu_canon(Cvt<T>::up(gp[e]), Cvt<T>::up(up[e])));
        const long long o = m * pitch + (long long)rank * f16 + c;
        for (int r = 0; r < R; ++r) static_cast<uint4*>(dst.p[r])[o] = oq;
    }
    push_handshake(rank, R, flags, counters, status, wait);
}

}  // namespace
}  // namespace bi

extern "C" int bi_peer_alloc(void** ptr, size_t bytes) {
    using namespace bi;
    if (!ptr || bytes == 0) return fail(BI_ERR_BAD_ARG, "bi_peer_alloc: null pointer or zero size");
    cudaError_t e = cudaMalloc(ptr, bytes);
    if (e == cudaSuccess) e = cudaMemset(*ptr, 0, bytes);
    if (e != cudaSuccess) return fail(BI_ERR_CUDA, "bi_peer_alloc(%zu): %s", bytes, cudaGetErrorString(e));
    return BI_OK;
}

extern "C" int bi_peer_free(void* ptr) {
    using namespace bi;
    cudaError_t e = cudaFree(ptr);
    if (e != cudaSuccess) return fail(BI_ERR_CUDA, "bi_peer_free: %s", cudaGetErrorString(e));
    return BI_OK;
}

extern "C" int bi_peer_export(void* ptr, uint8_t handle[64]) {
    using namespace bi;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    if (!ptr || !handle) return fail(BI_ERR_BAD_ARG, "bi_peer_export: null pointer");
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, ptr);
    if (e != cudaSuccess) return fail(BI_ERR_CUDA, "bi_peer_export: %s", cudaGetErrorString(e));
    memcpy(handle, &h, 64);
    return BI_OK;
}

extern "C" int bi_peer_open(const uint8_t handle[64], void** ptr) {
    using namespace bi;
    if (!ptr || !handle) return fail(BI_ERR_BAD_ARG, "bi_peer_open: null pointer");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, 64);
    cudaError_t e = cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return fail(BI_ERR_CUDA, "bi_peer_open: %s", cudaGetErrorString(e));
    return BI_OK;
}

extern "C" int bi_peer_close(void* ptr) {
    using namespace bi;
    cudaError_t e = cudaIpcCloseMemHandle(ptr);
    if (e != cudaSuccess) return fail(BI_ERR_CUDA, "bi_peer_close: %s", cudaGetErrorString(e));
    return BI_OK;
}

extern "C" int bi_push_gather(const void* local, void* const* dst, void* const* flags, uint32_t* counters, int64_t rows,
                              int64_t row_bytes, int rank, int world, int wait, int32_t* status, void* stream) {
    using namespace bi;
    if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world)
        return fail(BI_ERR_BAD_ARG, "bi_push_gather: rank %d of %d (at most %d ranks)", rank, world, MAX_RANKS);
    if (rows < 0 || row_bytes <= 0) return fail(BI_ERR_BAD_ARG, "bi_push_gather: rows=%lld row_bytes=%lld", (long long)rows, (long long)row_bytes);
    if (rows == 0) return BI_OK;
    if (!local || !dst || !flags || !counters) return fail(BI_ERR_BAD_ARG, "bi_push_gather: null pointer");
    if (row_bytes % 16 != 0 || !aligned(local, 16)) return fail(BI_ERR_MISALIGNED, "bi_push_gather: slices must be 16-byte aligned rows of a multiple of 16 bytes");
    PeerPtrs d{}, f{};
    for (int r = 0; r < world; ++r) {
        if (!dst[r] || !flags[r]) return fail(BI_ERR_BAD_ARG, "bi_push_gather: null peer pointer for rank %d", r);
        if (!aligned(dst[r], 16)) return fail(BI_ERR_MISALIGNED, "bi_push_gather: destination of rank %d is not 16-byte aligned", r);
        d.p[r] = dst[r];
        f.p[r] = flags[r];
    }
    const long long f16 = row_bytes / 16;
    if (f16 >= (1LL << 31)) return fail(BI_ERR_UNSUPPORTED, "bi_push_gather: row too long");
    const long long total = rows * f16;
    long long blocks = (total + 256 * 4 - 1) / (256 * 4);   // four 16-byte pieces per thread
    if (blocks > 128) blocks = 128;
    if (blocks < 1) blocks = 1;
    launch_overlapped(push_gather_kernel, dim3((unsigned)blocks), dim3(256), 0, static_cast<cudaStream_t>(stream),
        static_cast<const uint4*>(local), rows, (int)f16, rank, world, d, f, counters, status, wait);
    return check_launch("bi_push_gather");
}

extern "C" int bi_push_gather_swiglu(const void* gate_up, void* const* dst, void* const* flags, uint32_t* counters, int64_t rows,
                                     int64_t F, int dtype, int rank, int world, int wait, int32_t* status, void* stream) {
    using namespace bi;
    if (!dtype_ok(dtype)) return fail(BI_ERR_UNSUPPORTED, "bi_push_gather_swiglu: dtype %d", dtype);
    if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world)
        return fail(BI_ERR_BAD_ARG, "bi_push_gather_swiglu: rank %d of %d (at most %d ranks)", rank, world, MAX_RANKS);
    if (rows < 0 || F <= 0) return fail(BI_ERR_BAD_ARG, "bi_push_gather_swiglu: rows=%lld F=%lld", (long long)rows, (long long)F);
    if (rows == 0) return BI_OK;
    if (!gate_up || !dst || !flags || !counters) return fail(BI_ERR_BAD_ARG, "bi_push_gather_swiglu: null pointer");
    const int64_t per = 16 / (int64_t)dtype_size(dtype);
    if (F % per != 0 || !aligned(gate_up, 16) || F / per >= (1LL << 31))
        return fail(BI_ERR_MISALIGNED, "bi_push_gather_swiglu: F must be a multiple of %lld elements and gate_up 16-byte aligned", (long long)per);
    PeerPtrs d{}, f{};
    for (int r = 0; r < world; ++r) {
        if (!dst[r] || !flags[r]) return fail(BI_ERR_BAD_ARG, "bi_push_gather_swiglu: null peer pointer for rank %d", r);
        if (!aligned(dst[r], 16)) return fail(BI_ERR_MISALIGNED, "bi_push_gather_swiglu: destination of rank %d is not 16-byte aligned", r);
        d.p[r] = dst[r];
        f.p[r] = flags[r];
    }
    const long long total = rows * (F / per);
    long long blocks = (total + 255) / 256;
    if (blocks > 128) blocks = 128;
    if (blocks < 1) blocks = 1;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
#define BI_PGS(TT) launch_overlapped(push_gather_swiglu_kernel<TT>, dim3((unsigned)blocks), dim3(256), 0, st, static_cast<const TT*>(gate_up), rows, (int)F, rank, world, d, f, counters, status, wait)
    if (dtype == BI_F32) BI_PGS(float); else if (dtype == BI_F16) BI_PGS(__half); else BI_PGS(__nv_bfloat16);
#undef BI_PGS
    return check_launch("bi_push_gather_swiglu");
}
