// Library-wide entry points: version, the thread-local error message, and the
// device status word helper.
#include "bi_common.cuh"
#include <atomic>
#include <cstdlib>
#include <cstring>

namespace bi {
namespace {
thread_local char g_err[512] = "";
std::atomic<unsigned long long> g_launches{0};
}

void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

// Off unless BI_PDL=1: measured on the decoder step (418 kernels in one CUDA graph) it changed nothing for 16-bit
// weights (6.07 against 6.04 ms) and cost 5 % with 4-bit weights (8.36 against 7.98 ms): inside a graph the gaps
// between kernels are already short, and CTAs of the next kernel that sit resident take room from the running one.
bool pdl_enabled() {
    const char* v = getenv("BI_PDL");      // read per launch: a test can switch it for one call
    return v && v[0] == '1';
}

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}
}  // namespace bi

extern "C" int bi_version(void) { return 100; /* 0.1.0 */ }

extern "C" const char* bi_last_error(void) { return bi::g_err; }

extern "C" unsigned long long bi_launch_count(void) { return bi::g_launches.load(std::memory_order_relaxed); }

extern "C" int bi_read_device_status(const int32_t* status, int32_t* host_value, void* stream) {
    using namespace bi;
    if (!status || !host_value) return fail(BI_ERR_BAD_ARG, "bi_read_device_status: null pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemcpyAsync(host_value, status, sizeof(int32_t), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return fail(BI_ERR_CUDA, "bi_read_device_status: %s", cudaGetErrorString(e));
    if (*host_value != 0)
        return fail(BI_ERR_DEVICE_WAIT, "device wait ran out: code 0x%x (role %d, stage/buffer %d)", *host_value,
                    (*host_value >> 8) & 0xff, *host_value & 0xff);
    return BI_OK;
}
