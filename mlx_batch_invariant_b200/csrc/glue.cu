// Elementwise glue of the decoder runner: rotary embedding fused with the KV-cache append, and the
// SwiGLU gate. Each output element depends on its own inputs only, through a fixed sequence of
// round-to-nearest fp32 operations, so these are batch-invariant by construction; they exist to
// replace a dozen framework launches per layer with two.
#include "bi_common.cuh"
#include "bi_ptx.cuh"

namespace bi {
namespace {

// qkv: [B*T, (Hq + 2*Hkv) * D] rows as the qkv projection wrote them. Token (b, t) sits at position
// pos0[0] + t. q -> q_out[B, Hq, T, D] rotated; k rotated and v -> caches [*, Hkv, cap, D] at that position.
//   rot(x)_d = x_d * cos_d + (d < D/2 ? -x_{d+D/2} : x_{d-D/2}) * sin_d     (two multiplies, one add, one rounding)
template <typename T>
__global__ void __launch_bounds__(256) rope_append_kernel(const T* __restrict__ qkv, const float* __restrict__ cosT,
                                                          const float* __restrict__ sinT, const int64_t* __restrict__ pos0,
                                                          T* __restrict__ q_out, T* __restrict__ kc, T* __restrict__ vc,
                                                          int B, int Tn, int Hq, int Hkv, int D, int64_t c_sb, int64_t c_sh,
                                                          int64_t c_sl, int64_t capacity, int32_t* status) {
    ptx::grid_dep_launch();   // the next kernel of the stream may start its set-up
    ptx::grid_dep_wait();     // everything before this kernel has completed and is visible
    const int H = Hq + 2 * Hkv;
    const int64_t total = (int64_t)B * Tn * H * D;
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int d = (int)(i % D);
    const int h = (int)((i / D) % H);
    const int64_t bt = i / ((int64_t)D * H);
    const int t = (int)(bt % Tn);
    const int b = (int)(bt / Tn);
    const int64_t p = pos0[0] + t;
    // The position comes from device memory (a replayed graph advances it): a position outside the cache or
    // the tables writes nothing and leaves a code in the status word instead.
    if (p < 0 || p >= capacity) {
        if (status) atomicCAS(status, 0, (int)(0x30000 | (int)(p & 0xffff)));
        return;
    }
    const float x = Cvt<T>::up(qkv[i]);
    if (h >= Hq + Hkv) {                                   // v: copied as is
        vc[(int64_t)b * c_sb + (int64_t)(h - Hq - Hkv) * c_sh + p * c_sl + d] = qkv[i];
        return;
    }
    const int half = D / 2;
    const float other = Cvt<T>::up(qkv[d < half ? i + half : i - half]);
    const float rot = d < half ? -other : other;
    const float o = add_rn(mul_rn(x, cosT[p * D + d]), mul_rn(rot, sinT[p * D + d]));
    if (h < Hq) q_out[(((int64_t)b * Hq + h) * Tn + t) * D + d] = Cvt<T>::down(o);
    else        kc[(int64_t)b * c_sb + (int64_t)(h - Hq) * c_sh + p * c_sl + d] = Cvt<T>::down(o);
}

// out[m, j] = T( silu(gu[m, j]) * gu[m, F + j] ),  silu(g) = g * sigmoid(g), sigmoid from exp(-|g|)
template <typename T>
__global__ void __launch_bounds__(256) swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int64_t M, int64_t F) {
    ptx::grid_dep_launch();   // the next kernel of the stream may start its set-up
    ptx::grid_dep_wait();     // everything before this kernel has completed and is visible
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= M * F) return;
    const int64_t m = i / F, j = i - m * F;
    const float g = Cvt<T>::up(gu[m * 2 * F + j]);
    const float u = Cvt<T>::up(gu[m * 2 * F + F + j]);
    out[i] = Cvt<T>::down(swiglu_canon(g, u));
}

}  // namespace
}  // namespace bi

extern "C" int bi_rope_append(const void* qkv, const float* cos_table, const float* sin_table, const int64_t* pos0,
                              void* q_out, void* k_cache, void* v_cache, int64_t B, int64_t T, int64_t Hq, int64_t Hkv,
                              int64_t D, int64_t cache_sb, int64_t cache_sh, int64_t cache_sl, int64_t capacity,
                              int32_t* status, int dtype, void* stream) {
    using namespace bi;
    if (!dtype_ok(dtype)) return fail(BI_ERR_UNSUPPORTED, "bi_rope_append: dtype %d", dtype);
    if (B < 0 || T <= 0 || Hq <= 0 || Hkv <= 0 || D <= 0 || D % 2 || capacity <= 0) return fail(BI_ERR_BAD_ARG, "bi_rope_append: bad sizes");
    if (B == 0) return BI_OK;
    if (!qkv || !cos_table || !sin_table || !pos0 || !q_out || !k_cache || !v_cache) return fail(BI_ERR_BAD_ARG, "bi_rope_append: null pointer");
    const int64_t total = B * T * (Hq + 2 * Hkv) * D;
    const int64_t blocks = (total + 255) / 256;
    if (blocks > 0x7fffffffLL) return fail(BI_ERR_UNSUPPORTED, "bi_rope_append: too large");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
#define BI_ROPE(TT) launch_overlapped(rope_append_kernel<TT>, dim3((unsigned)blocks), dim3(256), 0, st, static_cast<const TT*>(qkv), cos_table, sin_table, pos0, \
        static_cast<TT*>(q_out), static_cast<TT*>(k_cache), static_cast<TT*>(v_cache), (int)B, (int)T, (int)Hq, (int)Hkv, (int)D, cache_sb, cache_sh, cache_sl, capacity, status)
    if (dtype == BI_F32) BI_ROPE(float); else if (dtype == BI_F16) BI_ROPE(__half); else BI_ROPE(__nv_bfloat16);
#undef BI_ROPE
    return check_launch("bi_rope_append");
}

extern "C" int bi_swiglu(const void* gate_up, void* out, int64_t M, int64_t F, int dtype, void* stream) {
    using namespace bi;
    if (!dtype_ok(dtype)) return fail(BI_ERR_UNSUPPORTED, "bi_swiglu: dtype %d", dtype);
    if (M < 0 || F <= 0) return fail(BI_ERR_BAD_ARG, "bi_swiglu: bad sizes");
    if (M == 0) return BI_OK;
    if (!gate_up || !out) return fail(BI_ERR_BAD_ARG, "bi_swiglu: null pointer");
    const int64_t blocks = (M * F + 255) / 256;
    if (blocks > 0x7fffffffLL) return fail(BI_ERR_UNSUPPORTED, "bi_swiglu: too large");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == BI_F32) launch_overlapped(swiglu_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, st, static_cast<const float*>(gate_up), static_cast<float*>(out), M, F);
    else if (dtype == BI_F16) launch_overlapped(swiglu_kernel<__half>, dim3((unsigned)blocks), dim3(256), 0, st, static_cast<const __half*>(gate_up), static_cast<__half*>(out), M, F);
    else launch_overlapped(swiglu_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(256), 0, st, static_cast<const __nv_bfloat16*>(gate_up), static_cast<__nv_bfloat16*>(out), M, F);
    return check_launch("bi_swiglu");
}
