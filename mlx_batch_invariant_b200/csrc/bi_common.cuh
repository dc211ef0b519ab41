// Host-side plumbing shared by the .cu files: status codes, the thread-local
// error message, and launch checking.
#pragma once
#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdio>
#include <cstdint>
#include "../../include/bi_abi.h"
#include "bi_math.cuh"

namespace bi {

// Defined in abi.cu. Records `msg` for bi_last_error() and returns `code`.
int fail(int code, const char* fmt, ...);

// Defined in abi.cu: counts kernel launches of the library (read back by bi_launch_count()).
void count_launch();

inline int check_launch(const char* what) {
    count_launch();
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(BI_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
    return BI_OK;
}

// Defined in abi.cu: whether kernels are launched with programmatic dependent launch (BI_PDL=1 turns it on).
bool pdl_enabled();

// Launch `kernel` so that it may begin (block scheduling, barrier and tensor-memory set-up) while the kernel before it
// on the stream is still draining; the kernel itself waits (ptx::grid_dep_wait) before it touches global memory.
// Every kernel launched through here MUST execute ptx::grid_dep_wait() in every CTA: completion of this kernel then
// implies completion of everything before it, which is what the kernel after it relies on.
template <typename... KArgs, typename... Args>
inline void launch_overlapped(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);     // errors are picked up by check_launch()
}

inline bool aligned(const void* p, size_t n) { return (reinterpret_cast<uintptr_t>(p) % n) == 0; }

inline size_t dtype_size(int dtype) { return dtype == BI_F32 ? 4 : 2; }

inline bool dtype_ok(int dtype) { return dtype == BI_F32 || dtype == BI_F16 || dtype == BI_BF16; }

// Streaming multiprocessors of the current device (cached per device ordinal). Launch shapes are
// sized from it; no arithmetic depends on it.
inline int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (!cached[dev]) cudaDeviceGetAttribute(&cached[dev], cudaDevAttrMultiProcessorCount, dev);
    return cached[dev] > 0 ? cached[dev] : 148;
}

// Canonical constants of the arithmetic contract.
constexpr int GROUP_K = 256;  // K is folded in groups of this many elements, whatever M is

}  // namespace bi
