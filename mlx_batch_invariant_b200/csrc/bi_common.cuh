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
