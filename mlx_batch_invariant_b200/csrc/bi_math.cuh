// Canonical scalar arithmetic shared by every kernel of the library.
//
// Each helper is a fixed sequence of IEEE-754 round-to-nearest operations
// (fma / mul / add / sub / max, integer exponent arithmetic), written with the
// explicit *_rn intrinsics so the compiler can neither contract nor reorder
// them. No fast-math function, no MUFU approximation: the same source compiled
// by any toolkit gives the same bits, and a plain C restatement on a CPU with a
// correctly rounded fmaf() reproduces them.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace bi {

__device__ __forceinline__ float fma_rn(float a, float b, float c) { return __fmaf_rn(a, b, c); }
__device__ __forceinline__ float mul_rn(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float add_rn(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ float sub_rn(float a, float b) { return __fsub_rn(a, b); }

// exp(x) for x <= 0 (the only arguments online softmax produces), <= 1.07 ulp.
//   n = rint(x * log2 e)           (magic-number rounding, exact)
//   r = x - n*ln2                  (two fma steps, hi/lo split of ln 2)
//   p = 1 + r*Q(r), Q degree 5     (six Horner fma steps)
//   result = p * 2^n               (integer add on the exponent field)
// Results below 2^-125 (x < -86.5, including -inf) are defined as exactly 0.
// exp(0) is exactly 1.
__device__ __forceinline__ float expf_canon(float x) {
    const float MAGIC = 12582912.0f;  // 1.5 * 2^23
    float t  = fma_rn(x, 1.4426950408889634f, MAGIC);
    float nf = sub_rn(t, MAGIC);
    float r  = fma_rn(nf, -0.693145751953125f, x);
    r        = fma_rn(nf, -1.42860682030941723212e-6f, r);
    float p  = 0.0013843559427186847f;
    p = fma_rn(p, r, 0.008374235592782497f);
    p = fma_rn(p, r, 0.041668009012937546f);
    p = fma_rn(p, r, 0.16666430234909058f);
    p = fma_rn(p, r, 0.4999999403953552f);
    p = fma_rn(p, r, 1.0f);
    p = fma_rn(p, r, 1.0f);
    int n = __float_as_int(t) - 0x4B400000;
    float res = __int_as_float(__float_as_int(p) + (n << 23));
    return (x < -86.5f) ? 0.0f : res;
}

// 1 / sqrt(v) as a correctly rounded sqrt followed by a correctly rounded divide.
__device__ __forceinline__ float rsqrt_canon(float v) { return __fdiv_rn(1.0f, __fsqrt_rn(v)); }
__device__ __forceinline__ float div_canon(float a, float b) { return __fdiv_rn(a, b); }

// silu(g) * u = (g * sigmoid(g)) * u with sigmoid from exp(-|g|): one exp, one divide, two multiplies.
__device__ __forceinline__ float swiglu_canon(float g, float u) {
    const float e = expf_canon(-fabsf(g));
    const float den = add_rn(1.0f, e);
    const float sig = g >= 0.0f ? div_canon(1.0f, den) : div_canon(e, den);
    return mul_rn(mul_rn(g, sig), u);
}

// Storage-type conversions. Upcasts are exact; downcasts round to nearest even once.
template <typename T> struct Cvt;
template <> struct Cvt<float> {
    static __device__ __forceinline__ float up(float v) { return v; }
    static __device__ __forceinline__ float down(float v) { return v; }
};
template <> struct Cvt<__nv_bfloat16> {
    static __device__ __forceinline__ float up(__nv_bfloat16 v) { return __bfloat162float(v); }
    static __device__ __forceinline__ __nv_bfloat16 down(float v) { return __float2bfloat16_rn(v); }
};
template <> struct Cvt<__half> {
    static __device__ __forceinline__ float up(__half v) { return __half2float(v); }
    static __device__ __forceinline__ __half down(float v) { return __float2half_rn(v); }
};

// Final rounding of an output element, with the optional bias of a linear layer: T(total), then -- as an
// elementwise add of two T arrays would -- T(float(T(total)) + float(bias)). Two roundings, the bits of the unfused
// sequence (product rounded to the output type first, bias added afterwards: mlx_batch_invariant/ops.py:54-62).
template <typename T>
__device__ __forceinline__ T round_out(float total, const T* bias, long long n) {
    const T r = Cvt<T>::down(total);
    return bias ? Cvt<T>::down(add_rn(Cvt<T>::up(r), Cvt<T>::up(bias[n]))) : r;
}

}  // namespace bi
