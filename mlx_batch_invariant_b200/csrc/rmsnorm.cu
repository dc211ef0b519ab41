// RMSNorm, one CTA of 256 threads per row.
//
// Canonical order per row (identical to the Metal kernel of the reference,
// mlx_batch_invariant/kernels/rmsnorm.py:19-47):
//   thread t:  ss_t = 0; for i = t, t+256, ...: ss_t = fma(x_i, x_i, ss_t)
//   tree:      for s = 128, 64, ..., 1: red[t] = red[t] + red[t+s]  (t < s)
//   inv  = 1 / sqrt(red[0] / float(D) + eps)
//   out_i = T((x_i * inv) * w_i)          two fp32 multiplies, one rounding
// How many rows share the launch never enters: a row sees only its own CTA.
//
// bi_add_rms_norm is the same kernel with a residual add in front: sum_i = T(x_i + delta_i) (fp32 add, one
// rounding -- what an elementwise add of two T arrays gives), written out, and the norm runs over the
// rounded sums exactly as if they had been read back from memory.
//
// Data movement is free to differ from the reference: the row is staged in
// shared memory with 16-byte loads, each thread then walks its stride-256
// elements there, results are written back in place and leave with 16-byte
// stores. Rows too long for shared memory, or not 16-byte aligned, take the
// same arithmetic straight from global memory.
#include "bi_common.cuh"
#include "bi_ptx.cuh"

namespace bi {
namespace {

constexpr int TG = 256;

__device__ __forceinline__ float block_tree_sum(float ss, float* red, int t) {
    red[t] = ss;
    __syncthreads();
    if (t < 128) red[t] = add_rn(red[t], red[t + 128]);
    __syncthreads();
    if (t < 64) red[t] = add_rn(red[t], red[t + 64]);
    __syncthreads();
    if (t < 32) {
        float v = add_rn(red[t], red[t + 32]);
        v = add_rn(v, __shfl_down_sync(0xffffffffu, v, 16));
        v = add_rn(v, __shfl_down_sync(0xffffffffu, v, 8));
        v = add_rn(v, __shfl_down_sync(0xffffffffu, v, 4));
        v = add_rn(v, __shfl_down_sync(0xffffffffu, v, 2));
        v = add_rn(v, __shfl_down_sync(0xffffffffu, v, 1));
        if (t == 0) red[0] = v;
    }
    __syncthreads();
    return red[0];
}

// `delta` may be the destination of a peer gather whose arrival nobody has waited for yet: the CTA then first
// waits (bounded, 2 s) until every peer's flag has reached *epoch; on expiry it records a code and goes on.
struct NormAwait {
    const uint32_t* flags;
    const uint32_t* epoch;
    int rank, world;
    int32_t* status;
};

template <typename T, bool STAGED, bool HAS_W, bool HAS_RES>
__global__ void __launch_bounds__(TG) rms_norm_kernel(const T* x, const T* __restrict__ delta, const T* __restrict__ w,
                                                      T* sum_out, T* __restrict__ out, int D, float eps, NormAwait aw) {
    ptx::grid_dep_launch();   // the next kernel of the stream may start its set-up
    ptx::grid_dep_wait();     // everything before this kernel has completed and is visible
    extern __shared__ uint4 stage_raw[];
    __shared__ float red[TG];
    const int t = threadIdx.x;
    if (HAS_RES && aw.flags != nullptr) {
        if (t < aw.world && t != aw.rank) {
            const uint32_t epoch = *aw.epoch;
            uint64_t t0;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
            while (true) {
                uint32_t seen;
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(aw.flags + t) : "memory");
                if ((int32_t)(seen - epoch) >= 0) break;
                uint64_t now;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
                if (now - t0 > 2000000000ull) {
                    if (aw.status) atomicCAS(aw.status, 0, (int)(0x20000 | (t << 8) | (epoch & 0xff)));
                    break;
                }
            }
        }
        __syncthreads();
    }
    const size_t row = blockIdx.x;
    const T* xr = x + row * (size_t)D;
    T* orow = out + row * (size_t)D;
    T* xs = reinterpret_cast<T*>(stage_raw);

    if (STAGED) {
        constexpr int VEC = 16 / sizeof(T);
        const uint4* src = reinterpret_cast<const uint4*>(xr);
        if (HAS_RES) {
            // x + delta, rounded to T, goes to shared memory for the norm and to sum_out (which may be x)
            const uint4* dsrc = reinterpret_cast<const uint4*>(delta + row * (size_t)D);
            uint4* sdst = reinterpret_cast<uint4*>(sum_out + row * (size_t)D);
            for (int i = t; i < D / VEC; i += TG) {
                uint4 a = src[i], b = dsrc[i];
                T* av = reinterpret_cast<T*>(&a);
                const T* bv = reinterpret_cast<const T*>(&b);
#pragma unroll
                for (int j = 0; j < VEC; ++j) av[j] = Cvt<T>::down(add_rn(Cvt<T>::up(av[j]), Cvt<T>::up(bv[j])));
                stage_raw[i] = a;
                sdst[i] = a;
            }
        } else {
            for (int i = t; i < D / VEC; i += TG) stage_raw[i] = __ldg(src + i);
        }
        __syncthreads();
    } else if (HAS_RES) {
        const T* dr = delta + row * (size_t)D;
        T* sr = sum_out + row * (size_t)D;
        for (int i = t; i < D; i += TG) sr[i] = Cvt<T>::down(add_rn(Cvt<T>::up(xr[i]), Cvt<T>::up(dr[i])));
        // each thread reads back only what it wrote
    }
    const T* xin = STAGED ? xs : (HAS_RES ? sum_out + row * (size_t)D : xr);

    // Rows of up to 256 * KEEP elements keep the thread's values in registers between the two passes (the second
    // pass then reads neither shared nor global memory for x); longer rows read them again.
    constexpr int KEEP = 16;
    const bool keep = D <= TG * KEEP;
    float kept[KEEP];
    float ss = 0.0f;
    if (keep) {
#pragma unroll
        for (int j = 0; j < KEEP; ++j) {
            const int i = t + j * TG;
            kept[j] = i < D ? Cvt<T>::up(xin[i]) : 0.0f;
            if (i < D) ss = fma_rn(kept[j], kept[j], ss);
        }
    } else {
        for (int i = t; i < D; i += TG) {
            float v = Cvt<T>::up(xin[i]);
            ss = fma_rn(v, v, ss);
        }
    }
    const float total = block_tree_sum(ss, red, t);
    const float inv = rsqrt_canon(add_rn(div_canon(total, (float)D), eps));

    if (keep) {
#pragma unroll
        for (int j = 0; j < KEEP; ++j) {
            const int i = t + j * TG;
            if (i < D) {
                const float v = mul_rn(kept[j], inv);
                const float wi = HAS_W ? Cvt<T>::up(w[i]) : 1.0f;
                const T o = Cvt<T>::down(mul_rn(v, wi));
                if (STAGED) xs[i] = o; else orow[i] = o;
            }
        }
    } else {
        for (int i = t; i < D; i += TG) {
            float v = mul_rn(Cvt<T>::up(xin[i]), inv);
            float wi = HAS_W ? Cvt<T>::up(w[i]) : 1.0f;
            T o = Cvt<T>::down(mul_rn(v, wi));
            if (STAGED) xs[i] = o; else orow[i] = o;
        }
    }
    if (STAGED) {
        constexpr int VEC = 16 / sizeof(T);
        __syncthreads();
        uint4* dst = reinterpret_cast<uint4*>(orow);
        for (int i = t; i < D / VEC; i += TG) dst[i] = stage_raw[i];
    }
}

// LayerNorm, one CTA of 256 threads per row, in the manner of the RMSNorm above (the reference lists a
// batch-invariant LayerNorm as future work, README.md:261-263 there; this is its canonical order here):
//   thread t:  s_t = 0;  for i = t, t+256, ...: s_t = s_t + x_i           tree 128..1 -> mean = sum / float(D)
//   thread t:  q_t = 0;  for i = t, t+256, ...: d = x_i - mean; q_t = fma(d, d, q_t)   tree -> var = q / float(D)
//   inv = 1 / sqrt(var + eps);  out_i = T((((x_i - mean) * inv) * w_i) + b_i)   (w, b optional; one rounding)
template <typename T, bool HAS_W, bool HAS_B>
__global__ void __launch_bounds__(TG) layer_norm_kernel(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ b,
                                                        T* __restrict__ out, int D, float eps) {
    ptx::grid_dep_launch();   // the next kernel of the stream may start its set-up
    ptx::grid_dep_wait();     // everything before this kernel has completed and is visible
    __shared__ float red[TG];
    const int t = threadIdx.x;
    const T* xr = x + (size_t)blockIdx.x * (size_t)D;
    T* orow = out + (size_t)blockIdx.x * (size_t)D;
    constexpr int KEEP = 16;                     // rows of up to 4096 elements stay in registers after the first read
    const bool keep = D <= TG * KEEP;
    float kept[KEEP];
    float s = 0.0f;
    if (keep) {
#pragma unroll
        for (int j = 0; j < KEEP; ++j) {
            const int i = t + j * TG;
            kept[j] = i < D ? Cvt<T>::up(xr[i]) : 0.0f;
            if (i < D) s = add_rn(s, kept[j]);
        }
    } else {
        for (int i = t; i < D; i += TG) s = add_rn(s, Cvt<T>::up(xr[i]));
    }
    const float mean = div_canon(block_tree_sum(s, red, t), (float)D);
    __syncthreads();                             // red[] is reused by the second reduction
    float q = 0.0f;
    if (keep) {
#pragma unroll
        for (int j = 0; j < KEEP; ++j) {
            const int i = t + j * TG;
            if (i < D) { const float d = sub_rn(kept[j], mean); q = fma_rn(d, d, q); }
        }
    } else {
        for (int i = t; i < D; i += TG) { const float d = sub_rn(Cvt<T>::up(xr[i]), mean); q = fma_rn(d, d, q); }
    }
    const float var = div_canon(block_tree_sum(q, red, t), (float)D);
    const float inv = rsqrt_canon(add_rn(var, eps));
    auto finish = [&](float xv, int i) {
        float y = mul_rn(sub_rn(xv, mean), inv);
        if (HAS_W) y = mul_rn(y, Cvt<T>::up(w[i]));
        if (HAS_B) y = add_rn(y, Cvt<T>::up(b[i]));
        orow[i] = Cvt<T>::down(y);
    };
    if (keep) {
#pragma unroll
        for (int j = 0; j < KEEP; ++j) {
            const int i = t + j * TG;
            if (i < D) finish(kept[j], i);
        }
    } else {
        for (int i = t; i < D; i += TG) finish(Cvt<T>::up(xr[i]), i);
    }
}

template <typename T>
int launch_layer_norm(const void* x, const void* w, const void* b, void* out, int64_t rows, int64_t D, float eps, cudaStream_t st) {
    const T* xp = static_cast<const T*>(x);
    const T* wp = static_cast<const T*>(w);
    const T* bp = static_cast<const T*>(b);
    T* op = static_cast<T*>(out);
    dim3 grid((unsigned)rows), block(TG);
    if (w && b) layer_norm_kernel<T, true, true><<<grid, block, 0, st>>>(xp, wp, bp, op, (int)D, eps);
    else if (w) layer_norm_kernel<T, true, false><<<grid, block, 0, st>>>(xp, wp, bp, op, (int)D, eps);
    else if (b) layer_norm_kernel<T, false, true><<<grid, block, 0, st>>>(xp, wp, bp, op, (int)D, eps);
    else layer_norm_kernel<T, false, false><<<grid, block, 0, st>>>(xp, wp, bp, op, (int)D, eps);
    return check_launch("bi_layer_norm");
}

template <typename T>
int launch(const void* x, const void* delta, const void* w, void* sum_out, void* out, int64_t rows, int64_t D, float eps,
           cudaStream_t st, const NormAwait& aw = NormAwait{nullptr, nullptr, 0, 0, nullptr}) {
    const size_t row_bytes = (size_t)D * sizeof(T);
    const bool staged = row_bytes % 16 == 0 && row_bytes <= 160 * 1024 && aligned(x, 16) && aligned(out, 16) &&
                        (!delta || (aligned(delta, 16) && aligned(sum_out, 16)));
    const T* xp = static_cast<const T*>(x);
    const T* dp = static_cast<const T*>(delta);
    const T* wp = static_cast<const T*>(w);
    T* sp = static_cast<T*>(sum_out);
    T* op = static_cast<T*>(out);
    dim3 grid((unsigned)rows), block(TG);
#define BI_RMS_LAUNCH2(ST, HW, HR)                                                                  \
    do {                                                                                            \
        auto kern = rms_norm_kernel<T, ST, HW, HR>;                                                 \
        size_t smem = ST ? row_bytes : 0;                                                           \
        if (smem > 48 * 1024) {                                                                     \
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                                 (int)smem);                                        \
            if (e != cudaSuccess) return fail(BI_ERR_CUDA, "rms_norm smem attr: %s",               \
                                              cudaGetErrorString(e));                               \
        }                                                                                           \
        launch_overlapped(kern, grid, block, smem, st, xp, dp, wp, sp, op, (int)D, eps, aw);                       \
    } while (0)
#define BI_RMS_LAUNCH(ST, HW) do { if (delta) BI_RMS_LAUNCH2(ST, HW, true); else BI_RMS_LAUNCH2(ST, HW, false); } while (0)
    if (staged) { if (w) BI_RMS_LAUNCH(true, true); else BI_RMS_LAUNCH(true, false); }
    else        { if (w) BI_RMS_LAUNCH(false, true); else BI_RMS_LAUNCH(false, false); }
#undef BI_RMS_LAUNCH
#undef BI_RMS_LAUNCH2
    return check_launch(delta ? "bi_add_rms_norm" : "bi_rms_norm");
}

}  // namespace
}  // namespace bi

extern "C" int bi_rms_norm(const void* x, const void* w, void* out, int64_t rows, int64_t D, float eps,
                           int dtype, void* stream) {
    using namespace bi;
    if (!dtype_ok(dtype)) return fail(BI_ERR_UNSUPPORTED, "bi_rms_norm: dtype %d", dtype);
    if (rows < 0 || D <= 0 || D > INT32_MAX) return fail(BI_ERR_BAD_ARG, "bi_rms_norm: rows=%lld D=%lld", (long long)rows, (long long)D);
    if (rows == 0) return BI_OK;
    if (!x || !out) return fail(BI_ERR_BAD_ARG, "bi_rms_norm: null pointer");
    if (rows > 0x7fffffffLL) return fail(BI_ERR_UNSUPPORTED, "bi_rms_norm: rows=%lld exceeds the grid limit", (long long)rows);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case BI_F32: return launch<float>(x, nullptr, w, nullptr, out, rows, D, eps, st);
        case BI_F16: return launch<__half>(x, nullptr, w, nullptr, out, rows, D, eps, st);
        default:     return launch<__nv_bfloat16>(x, nullptr, w, nullptr, out, rows, D, eps, st);
    }
}

extern "C" int bi_add_rms_norm(const void* x, const void* delta, const void* w, void* sum_out, void* out, int64_t rows,
                               int64_t D, float eps, int dtype, void* stream) {
    using namespace bi;
    if (!dtype_ok(dtype)) return fail(BI_ERR_UNSUPPORTED, "bi_add_rms_norm: dtype %d", dtype);
    if (rows < 0 || D <= 0 || D > INT32_MAX) return fail(BI_ERR_BAD_ARG, "bi_add_rms_norm: rows=%lld D=%lld", (long long)rows, (long long)D);
    if (rows == 0) return BI_OK;
    if (!x || !delta || !sum_out || !out) return fail(BI_ERR_BAD_ARG, "bi_add_rms_norm: null pointer");
    if (out == sum_out || out == x || out == delta) return fail(BI_ERR_BAD_ARG, "bi_add_rms_norm: out must not alias x, delta or sum_out");
    if (rows > 0x7fffffffLL) return fail(BI_ERR_UNSUPPORTED, "bi_add_rms_norm: rows=%lld exceeds the grid limit", (long long)rows);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case BI_F32: return launch<float>(x, delta, w, sum_out, out, rows, D, eps, st);
        case BI_F16: return launch<__half>(x, delta, w, sum_out, out, rows, D, eps, st);
        default:     return launch<__nv_bfloat16>(x, delta, w, sum_out, out, rows, D, eps, st);
    }
}

extern "C" int bi_add_rms_norm_awaiting(const void* x, const void* delta, const void* w, void* sum_out, void* out, int64_t rows,
                                        int64_t D, float eps, int dtype, void* stream, const uint32_t* flags,
                                        const uint32_t* epoch, int rank, int world, int32_t* status) {
    using namespace bi;
    if (!dtype_ok(dtype)) return fail(BI_ERR_UNSUPPORTED, "bi_add_rms_norm_awaiting: dtype %d", dtype);
    if (rows < 0 || D <= 0 || D > INT32_MAX) return fail(BI_ERR_BAD_ARG, "bi_add_rms_norm_awaiting: rows=%lld D=%lld", (long long)rows, (long long)D);
    if (rows == 0) return BI_OK;
    if (!x || !delta || !sum_out || !out) return fail(BI_ERR_BAD_ARG, "bi_add_rms_norm_awaiting: null pointer");
    if (out == sum_out || out == x || out == delta) return fail(BI_ERR_BAD_ARG, "bi_add_rms_norm_awaiting: out must not alias x, delta or sum_out");
    if (rows > 0x7fffffffLL) return fail(BI_ERR_UNSUPPORTED, "bi_add_rms_norm_awaiting: rows=%lld exceeds the grid limit", (long long)rows);
    if (flags && (!epoch || world < 1 || world > 8 || rank < 0 || rank >= world))
        return fail(BI_ERR_BAD_ARG, "bi_add_rms_norm_awaiting: bad gather to wait for (rank %d of %d)", rank, world);
    const NormAwait aw{flags, epoch, rank, world, status};
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case BI_F32: return launch<float>(x, delta, w, sum_out, out, rows, D, eps, st, aw);
        case BI_F16: return launch<__half>(x, delta, w, sum_out, out, rows, D, eps, st, aw);
        default:     return launch<__nv_bfloat16>(x, delta, w, sum_out, out, rows, D, eps, st, aw);
    }
}

extern "C" int bi_layer_norm(const void* x, const void* w, const void* b, void* out, int64_t rows, int64_t D, float eps,
                             int dtype, void* stream) {
    using namespace bi;
    if (!dtype_ok(dtype)) return fail(BI_ERR_UNSUPPORTED, "bi_layer_norm: dtype %d", dtype);
    if (rows < 0 || D <= 0 || D > INT32_MAX) return fail(BI_ERR_BAD_ARG, "bi_layer_norm: rows=%lld D=%lld", (long long)rows, (long long)D);
    if (rows == 0) return BI_OK;
    if (!x || !out) return fail(BI_ERR_BAD_ARG, "bi_layer_norm: null pointer");
    if (rows > 0x7fffffffLL) return fail(BI_ERR_UNSUPPORTED, "bi_layer_norm: rows=%lld exceeds the grid limit", (long long)rows);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case BI_F32: return launch_layer_norm<float>(x, w, b, out, rows, D, eps, st);
        case BI_F16: return launch_layer_norm<__half>(x, w, b, out, rows, D, eps, st);
        default:     return launch_layer_norm<__nv_bfloat16>(x, w, b, out, rows, D, eps, st);
    }
}
