// bi_attn_decode_static: decode attention for callers that cannot hand over scratch memory.
//
// bi_attn_decode needs a caller-allocated workspace for its per-split partials. Some hosts of
// this library have nothing to allocate it with: a plugin that lives inside another runtime
// (MLX, for one, allocates kernel outputs itself and offers C code no allocator to call), or a
// serving process that reserved almost all of HBM for its own pool at start-up, where a late
// cudaMalloc may fail, and in any case synchronises the whole device. For them this entry point
// keeps the partials in a fixed array inside the library image instead.
//
// What that costs and what to watch:
//   * every GPU on which the library is loaded gives up BI_ATTN_DECODE_STATIC_MAX_BYTES (8 MiB)
//     of device memory until the process exits;
//   * a problem whose partials need more than that is refused with BI_ERR_WORKSPACE - use
//     bi_attn_decode with your own workspace then;
//   * all calls on a device share the one array. Two calls whose kernels can overlap on the GPU
//     (different streams, no dependency between them) race on it; keep such calls on one stream
//     or order them with events. The array still holds the previous call's partials when a call
//     starts; nothing in it has to be zero, because every slot the combine step reads is written
//     by the same call first;
//   * the first call on each device looks up the array's device address (cudaGetSymbolAddress).
//     Make that first call during start-up, before any stream capture begins on that device.
//   * no cudaMalloc, cudaFree or allocating library routine is called, on the first call or later.
#include <mutex>
#include "bi_common.cuh"

namespace {

constexpr size_t SCRATCH_BYTES = BI_ATTN_DECODE_STATIC_MAX_BYTES;
constexpr int MAX_DEVICES = 64;

// In host code this name is only a handle for the runtime; the address kernels can use comes
// from cudaGetSymbolAddress below. Device code never touches it by name here.
static __device__ __align__(256) unsigned char g_decode_scratch[SCRATCH_BYTES];

std::mutex g_mu;
void* g_scratch_ptr[MAX_DEVICES] = {nullptr};

// Device address of the scratch array on the current device (looked up once per device).
int scratch_for_current_device(void** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return bi::fail(BI_ERR_CUDA, "bi_attn_decode_static: cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= MAX_DEVICES) return bi::fail(BI_ERR_UNSUPPORTED, "bi_attn_decode_static: device ordinal %d", dev);
    std::lock_guard<std::mutex> lock(g_mu);
    if (!g_scratch_ptr[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_decode_scratch);
        if (e != cudaSuccess || !p)
            return bi::fail(BI_ERR_CUDA, "bi_attn_decode_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        g_scratch_ptr[dev] = p;
    }
    *out = g_scratch_ptr[dev];
    return BI_OK;
}

}  // namespace

extern "C" int bi_attn_decode_static(const void* q, const void* k, const void* v, void* out, const int32_t* kv_lens,
                                     int64_t B, int64_t Hq, int64_t Hkv, int64_t L, int64_t D, int64_t kv_sb,
                                     int64_t kv_sh, int64_t kv_sl, float scale, int split_size, int dtype,
                                     void* stream) {
    const size_t need = bi_attn_decode_workspace_bytes(B, Hq, L, D, split_size);
    if (need > SCRATCH_BYTES)
        return bi::fail(BI_ERR_WORKSPACE,
                        "bi_attn_decode_static: B=%lld Hq=%lld L=%lld D=%lld needs %zu bytes of partials, the built-in "
                        "scratch holds %zu; call bi_attn_decode with a workspace of your own",
                        (long long)B, (long long)Hq, (long long)L, (long long)D, need, SCRATCH_BYTES);
    void* scratch = nullptr;
    int rc = scratch_for_current_device(&scratch);
    if (rc) return rc;
    // Same kernels, same arithmetic as bi_attn_decode; only the home of the partials differs.
    return bi_attn_decode(q, k, v, out, kv_lens, scratch, SCRATCH_BYTES, B, Hq, Hkv, L, D, kv_sb, kv_sh, kv_sl, scale,
                          split_size, dtype, stream);
}
