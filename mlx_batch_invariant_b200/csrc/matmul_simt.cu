// CUDA-core matmul with the K-group contract, and the split-path combine kernel.
//
// Canonical order per output element on this path:
//   for each K group g (256 wide, ascending):  acc = 0;
//       for k ascending inside the group:      acc = fma(a[m,k], b[k,n], acc)
//   total = 0;  total = total + acc_g          (plain fp32 adds, g ascending)
//   out = T(total)                             (one rounding)
// Operands are upcast to fp32 exactly; every product/sum is a single fp32 fma.
// It serves fp32 inputs (Blackwell tensor cores have no full-precision fp32
// mode) and 16-bit weights whose rows cannot be described to TMA. Which path a
// weight takes depends on the weight alone, never on the batch.
//
// Two launch shapes, as in the reference (mlx_batch_invariant/kernels/matmul.py:279-314):
// fused (one CTA walks all groups and folds) and split (grid.z = group, raw fp32
// partials, then combine_kernel folds them). Both perform the same sequence of
// operations on every element.
#include "bi_common.cuh"
#include "bi_ptx.cuh"
#include "matmul_internal.cuh"

namespace bi {
namespace {

constexpr int BN = 64;
constexpr int BK = 16;
constexpr int THREADS = 256;

// Affine dequantization of one code: fma in fp32, then one rounding to the staged type T.
template <typename T>
__device__ __forceinline__ float dequant_code(uint32_t code, float s, float b) {
    return Cvt<T>::up(Cvt<T>::down(fma_rn((float)code, s, b)));
}

struct QuantArgs {
    const uint32_t* w;   // [N, K*bits/32]
    const void* scales;  // [N, K/gs]
    const void* biases;
    int bits, gs;
    const void* out_bias;  // optional [N] bias of the linear layer (dense and quantized alike), in T
};

// TM rows x 4 columns per thread; tile = (16*TM) x 64.
template <typename T, int TM, bool SPLIT, bool QUANT>
__global__ void __launch_bounds__(THREADS) simt_matmul_kernel(const T* __restrict__ a, const T* __restrict__ b,
                                                              QuantArgs qa, void* __restrict__ outp, int M, int N,
                                                              int K, int64_t a_sm, int64_t a_sk, int64_t b_sk,
                                                              int64_t b_sn) {
    ptx::grid_dep_launch();   // the next kernel of the stream may start its set-up
    ptx::grid_dep_wait();     // everything before this kernel has completed and is visible
    constexpr int BM = 16 * TM;
    __shared__ float As[BK][BM];
    __shared__ float Bs[BK][BN];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int n0 = blockIdx.x * BN, m0 = blockIdx.y * BM;
    const int ngroups = (K + GROUP_K - 1) / GROUP_K;
    const int g0 = SPLIT ? (int)blockIdx.z : 0;
    const int g1 = SPLIT ? g0 + 1 : ngroups;

    float total[TM][4];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) total[i][j] = 0.0f;

    for (int g = g0; g < g1; ++g) {
        float acc[TM][4];
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
        const int kg0 = g * GROUP_K;
        const int kg1 = min(K, kg0 + GROUP_K);
        for (int k0 = kg0; k0 < kg1; k0 += BK) {
            const int kc = min(BK, kg1 - k0);
            // stage A: k fastest when a is k-contiguous, else m fastest
            for (int e = tid; e < BM * BK; e += THREADS) {
                int kk, i;
                if (a_sk == 1) { kk = e % BK; i = e / BK; } else { i = e % BM; kk = e / BM; }
                const int m = m0 + i, k = k0 + kk;
                As[kk][i] = (m < M && kk < kc) ? Cvt<T>::up(a[(int64_t)m * a_sm + (int64_t)k * a_sk]) : 0.0f;
            }
            for (int e = tid; e < BN * BK; e += THREADS) {
                int kk, j;
                if (QUANT || b_sk == 1) { kk = e % BK; j = e / BK; } else { j = e % BN; kk = e / BN; }
                const int n = n0 + j, k = k0 + kk;
                float v = 0.0f;
                if (n < N && kk < kc) {
                    if (QUANT) {
                        const int per_word = 32 / qa.bits;
                        const uint32_t word = qa.w[(int64_t)n * (K / per_word) + k / per_word];
                        const uint32_t code = (word >> ((k % per_word) * qa.bits)) & ((1u << qa.bits) - 1u);
                        const int64_t gi = (int64_t)n * (K / qa.gs) + k / qa.gs;
                        const float s = Cvt<T>::up(static_cast<const T*>(qa.scales)[gi]);
                        const float bb = Cvt<T>::up(static_cast<const T*>(qa.biases)[gi]);
                        v = dequant_code<T>(code, s, bb);
                    } else {
                        v = Cvt<T>::up(b[(int64_t)k * b_sk + (int64_t)n * b_sn]);
                    }
                }
                Bs[kk][j] = v;
            }
            __syncthreads();
            for (int kk = 0; kk < kc; ++kk) {
                float av[TM], bv[4];
#pragma unroll
                for (int i = 0; i < TM; ++i) av[i] = As[kk][ty * TM + i];
#pragma unroll
                for (int j = 0; j < 4; ++j) bv[j] = Bs[kk][tx * 4 + j];
#pragma unroll
                for (int i = 0; i < TM; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[i][j] = fma_rn(av[i], bv[j], acc[i][j]);
            }
            __syncthreads();
        }
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) total[i][j] = SPLIT ? acc[i][j] : add_rn(total[i][j], acc[i][j]);
    }

#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            if (SPLIT) static_cast<float*>(outp)[((int64_t)g0 * M + m) * N + n] = total[i][j];
            else static_cast<T*>(outp)[(int64_t)m * N + n] = round_out<T>(total[i][j], static_cast<const T*>(qa.out_bias), n);
        }
    }
}

// out[idx] = T(((0 + p_0[idx]) + p_1[idx]) + ...): the fold of the split path
// (reference: bi_matmul_combine, mlx_batch_invariant/kernels/matmul.py:226-234).
// PUSH: the output is this rank's column slice of a gathered activation: out[m, n] goes to column rank * N + n of
// every rank's [M, world * N] destination, and the launch ends with the gather's handshake (peer_push.cuh) -- the
// fold and the all-gather that follows it are one kernel, the local slice never exists in memory.
template <typename T, int VEC, bool PUSH>
__global__ void __launch_bounds__(256) combine_kernel(const float* __restrict__ part, T* __restrict__ out, int G,
                                                      int64_t MN, const T* __restrict__ bias, int64_t N, PushSink sink) {
    ptx::grid_dep_launch();   // the next kernel of the stream may start its set-up
    ptx::grid_dep_wait();     // everything before this kernel has completed and is visible
    const int64_t i0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * VEC;
    if (i0 < MN) {
        float total[VEC];
#pragma unroll
        for (int v = 0; v < VEC; ++v) total[v] = 0.0f;
        for (int g = 0; g < G; ++g) {
            const float* p = part + (int64_t)g * MN + i0;
            if (VEC == 4) {
                const float4 x = *reinterpret_cast<const float4*>(p);
                total[0] = add_rn(total[0], x.x); total[1 % VEC] = add_rn(total[1 % VEC], x.y);
                total[2 % VEC] = add_rn(total[2 % VEC], x.z); total[3 % VEC] = add_rn(total[3 % VEC], x.w);
            } else {
                total[0] = add_rn(total[0], p[0]);
            }
        }
        if (PUSH) {
            // VEC consecutive outputs stay inside one row (N % VEC == 0 is checked by the launcher)
            const int64_t m = i0 / N, n = i0 - m * N;
            const int64_t o = m * N * sink.world + (int64_t)sink.rank * N + n;
            T vals[VEC];
#pragma unroll
            for (int v = 0; v < VEC; ++v) vals[v] = round_out<T>(total[v], bias, bias ? n + v : 0);
            for (int r = 0; r < sink.world; ++r) {
                T* d = static_cast<T*>(sink.dst.p[r]) + o;
#pragma unroll
                for (int v = 0; v < VEC; ++v) d[v] = vals[v];
            }
        } else {
#pragma unroll
            for (int v = 0; v < VEC; ++v) out[i0 + v] = round_out<T>(total[v], bias, bias ? (i0 + v) % N : 0);
        }
    }
    if (PUSH) push_handshake(sink);
}

template <typename T>
int combine_t(const float* part, void* out, int G, int64_t MN, cudaStream_t st, const void* bias_v, int64_t N,
              const PushSink* sink = nullptr) {
    const T* bias = static_cast<const T*>(bias_v);
    const bool vec_ok = MN % 4 == 0 && aligned(part, 16) && (!sink || N % 4 == 0);
    const PushSink none{};
#define BI_COMBINE(VEC, THREADS_)                                                                                        \
    do {                                                                                                                 \
        const unsigned blocks_ = (unsigned)(((THREADS_) + 255) / 256);                                                  \
        if (sink) launch_overlapped(combine_kernel<T, VEC, true>, dim3(blocks_), dim3(256), 0, st, part, (T*)nullptr, G, MN, bias, N, *sink); \
        else launch_overlapped(combine_kernel<T, VEC, false>, dim3(blocks_), dim3(256), 0, st, part, static_cast<T*>(out), G, MN, bias, N, none); \
    } while (0)
    if (vec_ok && MN >= (1 << 20)) {
        BI_COMBINE(4, MN / 4);
    } else {
        // few outputs: one per thread, so that enough loads are in flight to cover the L2 latency
        // (4096x14336 at M = 16: 31.1 -> 28.3 us for matmul + combine)
        BI_COMBINE(1, MN);
    }
#undef BI_COMBINE
    return check_launch("matmul combine");
}

// The fold of the split path for a decoder's qkv projection, with bi_rope_append's work done on the folded values
// before they ever reach memory. One thread per element, as in combine_kernel (enough loads in flight to cover the
// L2 latency): it folds its column, rounds to T (the bits combine_kernel would have stored), leaves the value in shared
// memory for the thread that holds the other half of the rotation pair (a block of 256 consecutive elements covers
// whole heads: 256 % D == 0), and then repeats rope_append_kernel's arithmetic: q and k heads rotated, v heads
// copied, positions outside the cache skipped with a status code.
template <typename T>
__global__ void __launch_bounds__(256) combine_rope_kernel(const float* __restrict__ part, int G, int64_t MN, RopeSink r) {
    ptx::grid_dep_launch();
    ptx::grid_dep_wait();
    __shared__ T rounded[256];
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const bool live = i < MN;
    float total = 0.0f;
    if (live)
        for (int g = 0; g < G; ++g) total = add_rn(total, part[(int64_t)g * MN + i]);
    const T x = Cvt<T>::down(total);
    rounded[threadIdx.x] = x;
    __syncthreads();
    if (!live) return;
    const int H = r.Hq + 2 * r.Hkv, half = r.D / 2;
    const int d = (int)(i % r.D);
    const int h = (int)((i / r.D) % H);
    const int64_t bt = i / ((int64_t)r.D * H);
    const int t = (int)(bt % r.T);
    const int b = (int)(bt / r.T);
    const int64_t pos = r.pos0[0] + t;
    if (pos < 0 || pos >= r.capacity) {
        if (r.status) atomicCAS(r.status, 0, (int)(0x30000 | (int)(pos & 0xffff)));
        return;
    }
    if (h >= r.Hq + r.Hkv) {                               // v: stored as is
        static_cast<T*>(r.v_cache)[(int64_t)b * r.c_sb + (int64_t)(h - r.Hq - r.Hkv) * r.c_sh + pos * r.c_sl + d] = x;
        return;
    }
    const float other = Cvt<T>::up(rounded[d < half ? threadIdx.x + half : threadIdx.x - half]);
    const float rot = d < half ? -other : other;
    const T o = Cvt<T>::down(add_rn(mul_rn(Cvt<T>::up(x), r.cos_table[pos * r.D + d]), mul_rn(rot, r.sin_table[pos * r.D + d])));
    if (h < r.Hq) static_cast<T*>(r.q_out)[(((int64_t)b * r.Hq + h) * r.T + t) * r.D + d] = o;
    else          static_cast<T*>(r.k_cache)[(int64_t)b * r.c_sb + (int64_t)(h - r.Hq) * r.c_sh + pos * r.c_sl + d] = o;
}

template <typename T, bool QUANT>
int simt_t(const void* a, const void* b, const QuantArgs& qa, void* out, float* part, int64_t M, int64_t N,
           int64_t K, int64_t a_sm, int64_t a_sk, int64_t b_sk, int64_t b_sn, bool split, cudaStream_t st) {
    const int G = (int)((K + GROUP_K - 1) / GROUP_K);
    const bool skinny = M <= 16;
    const int BM = skinny ? 16 : 64;
    dim3 grid((unsigned)((N + BN - 1) / BN), (unsigned)((M + BM - 1) / BM), split ? G : 1);
    if (grid.y > 65535) return fail(BI_ERR_UNSUPPORTED, "matmul (cuda-core path): M=%lld too large", (long long)M);
    const T* ap = static_cast<const T*>(a);
    const T* bp = static_cast<const T*>(b);
    void* dst = split ? static_cast<void*>(part) : out;
#define BI_SIMT(TMV, SP) simt_matmul_kernel<T, TMV, SP, QUANT><<<grid, THREADS, 0, st>>>(ap, bp, qa, dst, (int)M, (int)N, (int)K, a_sm, a_sk, b_sk, b_sn)
    if (skinny) { if (split) BI_SIMT(1, true); else BI_SIMT(1, false); }
    else        { if (split) BI_SIMT(4, true); else BI_SIMT(4, false); }
#undef BI_SIMT
    int rc = check_launch("matmul (cuda-core path)");
    if (rc || !split) return rc;
    return combine_t<T>(part, out, G, M * N, st, qa.out_bias, N);
}

}  // namespace

int launch_combine_rope(const float* part, int G, int64_t MN, int dtype, cudaStream_t st, const RopeSink& rope) {
    if (rope.D > 256 || 256 % rope.D != 0) return fail(BI_ERR_UNSUPPORTED, "matmul + rope: head_dim %d (must divide 256)", rope.D);
    const int64_t blocks = (MN + 255) / 256;
    if (blocks > 0x7fffffffLL) return fail(BI_ERR_UNSUPPORTED, "matmul + rope: too large");
    switch (dtype) {
        case BI_F32: launch_overlapped(combine_rope_kernel<float>, dim3((unsigned)blocks), dim3(256), 0, st, part, G, MN, rope); break;
        case BI_F16: launch_overlapped(combine_rope_kernel<__half>, dim3((unsigned)blocks), dim3(256), 0, st, part, G, MN, rope); break;
        default:     launch_overlapped(combine_rope_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(256), 0, st, part, G, MN, rope); break;
    }
    return check_launch("matmul fold + rope");
}

int launch_combine(const float* part, void* out, int G, int64_t MN, int dtype, cudaStream_t st, const void* bias, int64_t N,
                   const PushSink* sink) {
    switch (dtype) {
        case BI_F32: return combine_t<float>(part, out, G, MN, st, bias, N, sink);
        case BI_F16: return combine_t<__half>(part, out, G, MN, st, bias, N, sink);
        default:     return combine_t<__nv_bfloat16>(part, out, G, MN, st, bias, N, sink);
    }
}

int launch_simt_matmul(const void* a, const void* b, void* out, float* part, int64_t M, int64_t N, int64_t K,
                       int64_t a_sm, int64_t a_sk, int64_t b_sk, int64_t b_sn, int dtype, bool split,
                       cudaStream_t st, const void* bias) {
    QuantArgs qa{nullptr, nullptr, nullptr, 0, 0, bias};
    switch (dtype) {
        case BI_F32: return simt_t<float, false>(a, b, qa, out, part, M, N, K, a_sm, a_sk, b_sk, b_sn, split, st);
        case BI_F16: return simt_t<__half, false>(a, b, qa, out, part, M, N, K, a_sm, a_sk, b_sk, b_sn, split, st);
        default:     return simt_t<__nv_bfloat16, false>(a, b, qa, out, part, M, N, K, a_sm, a_sk, b_sk, b_sn, split, st);
    }
}

int launch_simt_qmm(const void* x, const uint32_t* w, const void* scales, const void* biases, void* out, float* part,
                    int64_t M, int64_t N, int64_t K, int64_t x_sm, int gs, int bits, int dtype, bool split,
                    cudaStream_t st) {
    QuantArgs qa{w, scales, biases, bits, gs, nullptr};
    switch (dtype) {
        case BI_F32: return simt_t<float, true>(x, nullptr, qa, out, part, M, N, K, x_sm, 1, 1, K, split, st);
        case BI_F16: return simt_t<__half, true>(x, nullptr, qa, out, part, M, N, K, x_sm, 1, 1, K, split, st);
        default:     return simt_t<__nv_bfloat16, true>(x, nullptr, qa, out, part, M, N, K, x_sm, 1, 1, K, split, st);
    }
}

}  // namespace bi
