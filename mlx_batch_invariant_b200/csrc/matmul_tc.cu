// Tensor-core matmul for 16-bit inputs on sm_100a: TMA -> shared memory ->
// tcgen05.mma -> TMEM -> registers.   out[M, N] = x[M, K] @ W[N, K]^T
//
// Canonical order per output element (what never changes with M):
//   * K is cut into groups of 256. Inside a group the tensor core runs sixteen
//     MMA steps of K = 16 in ascending k, all of the one instruction shape
//     tcgen05.mma.cta_group::1.kind::f16  M=128 (weight rows) x N=128 (batch rows) x K=16,
//     operands in the input dtype, fp32 accumulator. The first step of a group
//     overwrites the accumulator (accumulate off), so a group partial starts
//     from nothing.
//   * out = T(((0 + p_0) + p_1) + ... ), plain fp32 adds of the group partials,
//     g ascending, one rounding at the end.
// The weight is the 128-row "A" operand and the batch is the 128-column "B"
// operand, so a decode step with one row still issues exactly the instruction a
// 128-row prefill tile issues; batch rows beyond M are never loaded (their
// accumulator columns hold garbage that is never read -- every accumulator
// column depends on its own batch row only).
//
// Launch shapes (same arithmetic, reference: mlx_batch_invariant/kernels/matmul.py:279-314):
//   split : one job per (weight tile, batch tile, K group); the raw fp32 group
//           partial goes to the workspace and combine_kernel folds the groups.
//   fused : one unit per (weight tile, batch tile); the epilogue warps keep the
//           running total in registers and fold each group partial as it leaves TMEM.
// Both are one persistent kernel: CTA c takes a contiguous range of units, a
// TMA warp streams stages through a ring of shared-memory buffers, one thread
// issues the MMAs into one of two TMEM accumulators, four epilogue warps drain
// the other. For affine-quantized weights the TMA warp brings the packed codes
// instead and four more warps turn them into the same swizzled 16-bit tile the
// dense path would have loaded (fma(float(code), scale, bias) in fp32, one
// rounding -- mlx_batch_invariant/kernels/quantized.py:44-67), so the MMA
// sequence is the dense one.
//
// Every wait on a shared-memory barrier is bounded in time; a wait that runs
// out records a code in the caller's status word, raises a CTA-wide abort flag
// and the kernel drains its copies, frees its TMEM and returns.
#include <cuda.h>
#include <type_traits>
#include "bi_common.cuh"
#include "bi_ptx.cuh"
#include "matmul_internal.cuh"

namespace bi {
namespace {

constexpr int BLOCK_N = 128;  // weight rows per tile  (UMMA M)
constexpr int BLOCK_M = 128;  // batch rows per tile   (UMMA N)
constexpr int BLOCK_K = 64;   // elements per stage along K: 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int W_TILE_BYTES = BLOCK_N * BLOCK_K * 2;
constexpr int X_TILE_BYTES = BLOCK_M * BLOCK_K * 2;
constexpr int TMEM_COLS = 2 * BLOCK_M;  // two accumulators
constexpr uint64_t WAIT_LIMIT_NS = 2000000000ull;

constexpr int WARP_TMA = 0, WARP_MMA = 1, WARP_EPI0 = 2, WARP_DEQ0 = 6;

template <int QBITS> struct Cfg {
    static constexpr int RAW_BYTES = QBITS ? BLOCK_N * BLOCK_K * QBITS / 8 : 0;
    static constexpr int STAGE_BYTES = W_TILE_BYTES + X_TILE_BYTES + RAW_BYTES;
    static constexpr int STAGES = QBITS ? 5 : 6;
    static constexpr int THREADS = QBITS ? 320 : 192;
    static constexpr int BAR_BYTES = 512;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + BAR_BYTES + 1024;  // + alignment slack
};

struct Params {
    void* out;          // [M, N] in T (fused)
    float* part;        // [G, M, N] fp32 (split)
    const void* scales; // quantized only: [N, K/gs] in T
    const void* biases;
    int32_t* status;
    int M, N, K, G;
    int n_tiles, m_tiles;
    int split;          // 1: split jobs, 0: fused units
    int x_rows;         // rows of the activation TMA box
    int gs;
    long long units;
};

enum { ROLE_TMA = 1, ROLE_MMA = 2, ROLE_EPI = 3, ROLE_DEQ = 4 };

struct Ctl {
    int32_t* status;
    volatile int* abort_flag;  // shared memory
};

__device__ __forceinline__ void report(const Ctl& c, int role, int idx) {
    *c.abort_flag = 1;
    if (c.status) atomicCAS(c.status, 0, (int)(0x10000 | (role << 8) | (idx & 0xff)));
}

// Wait for barrier phase `parity` to complete. Gives up after WAIT_LIMIT_NS or when another
// role has raised the abort flag; returns false then.
__device__ __forceinline__ bool wait_bounded(uint32_t bar, uint32_t parity, const Ctl& c, int role, int idx) {
    for (int i = 0; i < 4096; ++i)
        if (ptx::mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = ptx::globaltimer_ns();
    while (true) {
        for (int i = 0; i < 256; ++i)
            if (ptx::mbar_try_wait(bar, parity)) return true;
        if (*c.abort_flag) return false;
        if (ptx::globaltimer_ns() - t0 > WAIT_LIMIT_NS) { report(c, role, idx); return false; }
    }
}

struct Unit {
    int n0, m0, g0, g1;
};
__device__ __forceinline__ Unit decode_unit(const Params& p, long long u) {
    Unit r;
    long long tile;
    if (p.split) { tile = u / p.G; r.g0 = (int)(u % p.G); r.g1 = r.g0 + 1; }
    else         { tile = u; r.g0 = 0; r.g1 = p.G; }
    r.n0 = (int)(tile / p.m_tiles) * BLOCK_N;
    r.m0 = (int)(tile % p.m_tiles) * BLOCK_M;
    return r;
}
__device__ __forceinline__ int stages_in_group(const Params& p, int g) {
    const int kg0 = g * GROUP_K;
    const int kg1 = min(p.K, kg0 + GROUP_K);
    return (kg1 - kg0 + BLOCK_K - 1) / BLOCK_K;
}

template <typename T> struct Pack2;
template <> struct Pack2<__nv_bfloat16> {
    static __device__ __forceinline__ uint32_t rn(float lo, float hi) {
        __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);  // .x = lo (low address)
        return *reinterpret_cast<uint32_t*>(&v);
    }
};
template <> struct Pack2<__half> {
    static __device__ __forceinline__ uint32_t rn(float lo, float hi) {
        __half2 v = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&v);
    }
};

// Eight consecutive codes -> eight T values packed for one 16-byte swizzle chunk.
template <typename T, int QBITS>
__device__ __forceinline__ uint4 dequant8(const uint32_t* words, float s, float b) {
    float f[8];
    if (QBITS == 4) {
        const uint32_t w = words[0];
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = fma_rn((float)((w >> (4 * i)) & 0xFu), s, b);
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = fma_rn((float)((words[i >> 2] >> (8 * (i & 3))) & 0xFFu), s, b);
    }
    uint4 o;
    o.x = Pack2<T>::rn(f[0], f[1]); o.y = Pack2<T>::rn(f[2], f[3]);
    o.z = Pack2<T>::rn(f[4], f[5]); o.w = Pack2<T>::rn(f[6], f[7]);
    return o;
}

template <typename T, int QBITS>
__global__ void __launch_bounds__(Cfg<QBITS>::THREADS, 1)
tc_matmul_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                 const Params p) {
    using C = Cfg<QBITS>;
    constexpr int STAGES = C::STAGES;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
    // stage s: [W tile 16 KB | X tile 16 KB | raw codes]
    auto w_tile = [&](int s) { return smem_base + (uint32_t)s * C::STAGE_BYTES; };
    auto x_tile = [&](int s) { return w_tile(s) + W_TILE_BYTES; };
    auto raw_tile = [&](int s) { return x_tile(s) + X_TILE_BYTES; };
    const uint32_t bar_base = smem_base + STAGES * C::STAGE_BYTES;
    auto bar_full = [&](int s) { return bar_base + 8u * s; };                  // operands ready for the MMA
    auto bar_empty = [&](int s) { return bar_base + 8u * (STAGES + s); };      // stage free again
    auto bar_raw = [&](int s) { return bar_base + 8u * (2 * STAGES + s); };    // TMA landed (quantized)
    auto bar_tfull = [&](int b) { return bar_base + 8u * (3 * STAGES + b); };  // accumulator complete
    auto bar_tempty = [&](int b) { return bar_base + 8u * (3 * STAGES + 2 + b); };
    uint8_t* misc = smem_gen + STAGES * C::STAGE_BYTES + 8 * (3 * STAGES + 4);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(misc);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(misc + 4);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const Ctl ctl{p.status, abort_flag};

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(bar_full(s), QBITS ? 4 : 1);
            ptx::mbar_init(bar_empty(s), 1);
            ptx::mbar_init(bar_raw(s), 1);
        }
        for (int b = 0; b < 2; ++b) { ptx::mbar_init(bar_tfull(b), 1); ptx::mbar_init(bar_tempty(b), 4); }
        ptx::fence_mbar_init();
        ptx::prefetch_tensormap(&tmap_w);
        ptx::prefetch_tensormap(&tmap_x);
    }
    if (warp == WARP_MMA) {
        ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const long long ub = p.units * blockIdx.x / gridDim.x;
    const long long ue = p.units * (blockIdx.x + 1) / gridDim.x;

    if (warp == WARP_TMA) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            const uint32_t tx_bytes = (uint32_t)p.x_rows * BLOCK_K * 2 + (QBITS ? C::RAW_BYTES : W_TILE_BYTES);
            int s = 0; uint32_t ph = 0; long long issued = 0; bool ok = true;
            for (long long u = ub; u < ue && ok; ++u) {
                const Unit un = decode_unit(p, u);
                for (int g = un.g0; g < un.g1 && ok; ++g) {
                    const int nst = stages_in_group(p, g);
                    for (int ks = 0; ks < nst; ++ks) {
                        if (!wait_bounded(bar_empty(s), ph ^ 1u, ctl, ROLE_TMA, s)) { ok = false; break; }
                        const int k0 = g * GROUP_K + ks * BLOCK_K;
                        const uint32_t bar = QBITS ? bar_raw(s) : bar_full(s);
                        ptx::mbar_expect_tx(bar, tx_bytes);
                        if (QBITS) ptx::tma_load_2d(raw_tile(s), &tmap_w, k0 * QBITS / 32, un.n0, bar);
                        else       ptx::tma_load_2d(w_tile(s), &tmap_w, k0, un.n0, bar);
                        ptx::tma_load_2d(x_tile(s), &tmap_x, k0, un.m0, bar);
                        ++issued;
                        if (++s == STAGES) { s = 0; ph ^= 1u; }
                    }
                }
            }
            if (!ok) {
                // Let the copies already in flight land before the CTA goes away.
                const long long n = issued < STAGES ? issued : STAGES;
                for (long long i = 0; i < n; ++i) {
                    int si = s - 1 - (int)i; uint32_t pi = ph;
                    if (si < 0) { si += STAGES; pi ^= 1u; }
                    const uint32_t bar = QBITS ? bar_raw(si) : bar_full(si);
                    const uint64_t t0 = ptx::globaltimer_ns();
                    while (!ptx::mbar_try_wait(bar, pi) && ptx::globaltimer_ns() - t0 < WAIT_LIMIT_NS) {}
                }
            }
        }
    } else if (warp == WARP_MMA) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t FMT = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
            constexpr uint32_t IDESC = (1u << 4) | (FMT << 7) | (FMT << 10) | ((uint32_t)(BLOCK_M >> 3) << 17) |
                                       ((uint32_t)(BLOCK_N >> 4) << 24);
            int s = 0; uint32_t ph = 0; long long job = 0; bool ok = true;
            for (long long u = ub; u < ue && ok; ++u) {
                const Unit un = decode_unit(p, u);
                for (int g = un.g0; g < un.g1 && ok; ++g, ++job) {
                    const int buf = (int)(job & 1);
                    if (!wait_bounded(bar_tempty(buf), (uint32_t)((job >> 1) & 1) ^ 1u, ctl, ROLE_MMA, 16 + buf)) { ok = false; break; }
                    ptx::tc_fence_after();
                    const uint32_t tmem_d = tmem_base + (uint32_t)buf * BLOCK_M;
                    const int kg0 = g * GROUP_K;
                    const int kg1 = min(p.K, kg0 + GROUP_K);
                    const int nst = stages_in_group(p, g);
                    for (int ks = 0; ks < nst; ++ks) {
                        if (!wait_bounded(bar_full(s), ph, ctl, ROLE_MMA, s)) { ok = false; break; }
                        ptx::tc_fence_after();
                        const int kleft = kg1 - (kg0 + ks * BLOCK_K);
                        const int nsteps = (min(kleft, BLOCK_K) + UMMA_K - 1) / UMMA_K;
                        for (int kk = 0; kk < nsteps; ++kk) {
                            const uint64_t da = ptx::smem_desc_sw128(w_tile(s) + kk * UMMA_K * 2);
                            const uint64_t db = ptx::smem_desc_sw128(x_tile(s) + kk * UMMA_K * 2);
                            ptx::umma_f16(tmem_d, da, db, IDESC, (ks | kk) ? 1u : 0u);
                        }
                        ptx::umma_commit(bar_empty(s));
                        if (++s == STAGES) { s = 0; ph ^= 1u; }
                    }
                    if (ok) ptx::umma_commit(bar_tfull(buf));
                }
            }
        }
    } else if (warp >= WARP_EPI0 && warp < WARP_EPI0 + 4) {
        // ------------------------------------------------------------ epilogue
        const int quad = warp & 3;  // TMEM lanes this warp may read: 32*quad .. 32*quad+31
        const int row = quad * 32 + lane;
        long long job = 0; bool ok = true;
        T* out = static_cast<T*>(p.out);
        for (long long u = ub; u < ue && ok; ++u) {
            const Unit un = decode_unit(p, u);
            const int n = un.n0 + row;
            const int ncols = min(BLOCK_M, p.M - un.m0);
            float total[BLOCK_M];
#pragma unroll
            for (int i = 0; i < BLOCK_M; ++i) total[i] = 0.0f;
            for (int g = un.g0; g < un.g1 && ok; ++g, ++job) {
                const int buf = (int)(job & 1);
                if (!wait_bounded(bar_tfull(buf), (uint32_t)((job >> 1) & 1), ctl, ROLE_EPI, 16 + buf)) { ok = false; break; }
                ptx::tc_fence_after();
                const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)buf * BLOCK_M;
#pragma unroll
                for (int c = 0; c < BLOCK_M / 32; ++c) {
                    if (c * 32 < ncols) {  // warp-uniform
                        uint32_t v[32];
                        ptx::tmem_ld_32x32(taddr + c * 32, v);
                        ptx::tmem_ld_wait();
                        if (p.split) {
                            if (n < p.N) {
#pragma unroll
                                for (int j = 0; j < 32; ++j) {
                                    const int m = un.m0 + c * 32 + j;
                                    if (m < p.M) p.part[((long long)g * p.M + m) * p.N + n] = __uint_as_float(v[j]);
                                }
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j) total[c * 32 + j] = add_rn(total[c * 32 + j], __uint_as_float(v[j]));
                        }
                    }
                }
                ptx::tc_fence_before();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(bar_tempty(buf));
            }
            if (!p.split && ok && n < p.N) {
#pragma unroll
                for (int i = 0; i < BLOCK_M; ++i) {
                    const int m = un.m0 + i;
                    if (i < ncols) out[(long long)m * p.N + n] = Cvt<T>::down(total[i]);
                }
            }
        }
    } else if (QBITS && warp >= WARP_DEQ0) {
        // ------------------------------------------------------------ dequantizers
        constexpr int QB = QBITS ? QBITS : 4;
        constexpr int ROW_BYTES = BLOCK_K * QB / 8;     // packed bytes per weight row per stage
        constexpr int WORDS_PER_CHUNK = QB / 4;         // 32-bit words behind one 16-byte output chunk
        const int row = (warp - WARP_DEQ0) * 32 + lane;
        const T* scales = static_cast<const T*>(p.scales);
        const T* biases = static_cast<const T*>(p.biases);
        const int groups_per_row = p.K / p.gs;
        int s = 0; uint32_t ph = 0; bool ok = true;
        for (long long u = ub; u < ue && ok; ++u) {
            const Unit un = decode_unit(p, u);
            const int n = un.n0 + row;
            const bool live = n < p.N;
            for (int g = un.g0; g < un.g1 && ok; ++g) {
                const int nst = stages_in_group(p, g);
                for (int ks = 0; ks < nst; ++ks) {
                    const int k0 = g * GROUP_K + ks * BLOCK_K;
                    // scale / bias of the (at most two) quantization groups this stage touches
                    float sc[2] = {0.0f, 0.0f}, bs[2] = {0.0f, 0.0f};
                    if (live) {
                        const long long gi = (long long)n * groups_per_row + k0 / p.gs;
                        sc[0] = Cvt<T>::up(scales[gi]); bs[0] = Cvt<T>::up(biases[gi]);
                        if (p.gs == 32) { sc[1] = Cvt<T>::up(scales[gi + 1]); bs[1] = Cvt<T>::up(biases[gi + 1]); }
                        else            { sc[1] = sc[0]; bs[1] = bs[0]; }
                    }
                    if (!wait_bounded(bar_raw(s), ph, ctl, ROLE_DEQ, s)) { ok = false; break; }
                    const uint4* raw = reinterpret_cast<const uint4*>(smem_gen + (raw_tile(s) - smem_base) + row * ROW_BYTES);
                    uint8_t* wt = smem_gen + (w_tile(s) - smem_base) + row * 128;
                    uint32_t rw[ROW_BYTES / 4];
#pragma unroll
                    for (int i = 0; i < ROW_BYTES / 16; ++i) {
                        const uint4 t = raw[i];
                        rw[4 * i] = t.x; rw[4 * i + 1] = t.y; rw[4 * i + 2] = t.z; rw[4 * i + 3] = t.w;
                    }
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        uint32_t words[2];
                        words[0] = rw[c * WORDS_PER_CHUNK];
                        words[1] = rw[c * WORDS_PER_CHUNK + (WORDS_PER_CHUNK - 1)];
                        const uint4 o = dequant8<T, QB>(words, sc[c >> 2], bs[c >> 2]);
                        *reinterpret_cast<uint4*>(wt + ((c ^ (row & 7)) << 4)) = o;
                    }
                    ptx::fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(bar_full(s));
                    if (++s == STAGES) { s = 0; ph ^= 1u; }
                }
            }
        }
    }

    ptx::tc_fence_before();
    __syncthreads();
    if (warp == WARP_MMA) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ---- host side -----------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// 2-D row-major tensor [rows, cols] with `ld` elements between rows; box = [box_rows, box_cols].
int make_map(CUtensorMap* m, CUtensorMapDataType dt, size_t esize, const void* base, uint64_t cols, uint64_t rows,
             uint64_t ld, uint32_t box_cols, uint32_t box_rows, CUtensorMapSwizzle sw) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(BI_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t gdim[2] = {cols, rows};
    cuuint64_t gstr[1] = {ld * esize};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(m, dt, 2, const_cast<void*>(base), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(BI_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return BI_OK;
}

int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (!cached[dev]) cudaDeviceGetAttribute(&cached[dev], cudaDevAttrMultiProcessorCount, dev);
    return cached[dev] > 0 ? cached[dev] : 148;
}

template <typename T, int QBITS>
int launch_t(const CUtensorMap& mw, const CUtensorMap& mx, const Params& p, cudaStream_t st) {
    using C = Cfg<QBITS>;
    auto kern = tc_matmul_kernel<T, QBITS>;
    static bool attr_done[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (!attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
        if (e != cudaSuccess) return fail(BI_ERR_CUDA, "matmul smem attr: %s", cudaGetErrorString(e));
        attr_done[dev] = true;
    }
    const long long grid = p.units < sm_count() ? p.units : sm_count();
    kern<<<(unsigned)grid, C::THREADS, C::SMEM_BYTES, st>>>(mw, mx, p);
    return check_launch("matmul (tensor-core path)");
}

}  // namespace

bool tc_matmul_supported(const void* x, int64_t x_ld, const void* w, int64_t w_ld, int64_t N, int64_t K, int dtype,
                         const TcQuant* q) {
    if (dtype != BI_F16 && dtype != BI_BF16) return false;
    if (K <= 0 || N <= 0 || K >= (1LL << 31) || N >= (1LL << 31)) return false;
    if (!aligned(x, 16) || (x_ld * 2) % 16 != 0) return false;
    if (q && q->codes) {
        if (q->bits != 4 && q->bits != 8) return false;
        if (q->gs != 32 && q->gs != 64 && q->gs != 128) return false;
        if (K % BLOCK_K != 0 || K % q->gs != 0) return false;
        if (!aligned(q->codes, 16) || ((K * q->bits / 8) % 16) != 0) return false;
        return true;
    }
    return aligned(w, 16) && (w_ld * 2) % 16 == 0 && K % 8 == 0;
}

int launch_tc_matmul(const void* x, int64_t x_ld, const void* w, int64_t w_ld, const TcQuant* q, void* out,
                     float* part, int64_t M, int64_t N, int64_t K, int dtype, bool split, int32_t* status,
                     cudaStream_t st) {
    const bool quant = q && q->codes;
    Params p{};
    p.out = out; p.part = part; p.status = status;
    p.scales = quant ? q->scales : nullptr; p.biases = quant ? q->biases : nullptr;
    p.M = (int)M; p.N = (int)N; p.K = (int)K;
    p.G = (int)((K + GROUP_K - 1) / GROUP_K);
    p.n_tiles = (int)((N + BLOCK_N - 1) / BLOCK_N);
    p.m_tiles = (int)((M + BLOCK_M - 1) / BLOCK_M);
    p.split = split ? 1 : 0;
    p.gs = quant ? q->gs : 0;
    p.units = (long long)p.n_tiles * p.m_tiles * (split ? p.G : 1);
    // Only the batch rows that exist are loaded; the box height is a launch-shape choice.
    const int64_t mr = M < BLOCK_M ? ((M + 7) / 8) * 8 : BLOCK_M;
    p.x_rows = (int)mr;

    const CUtensorMapDataType dt = dtype == BI_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUtensorMap mw, mx;
    int rc = make_map(&mx, dt, 2, x, (uint64_t)K, (uint64_t)M, (uint64_t)x_ld, BLOCK_K, (uint32_t)p.x_rows,
                      CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    if (quant) {
        const uint64_t words = (uint64_t)K * q->bits / 32;
        rc = make_map(&mw, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, q->codes, words, (uint64_t)N, words,
                      (uint32_t)(BLOCK_K * q->bits / 32), BLOCK_N, CU_TENSOR_MAP_SWIZZLE_NONE);
    } else {
        rc = make_map(&mw, dt, 2, w, (uint64_t)K, (uint64_t)N, (uint64_t)w_ld, BLOCK_K, BLOCK_N,
                      CU_TENSOR_MAP_SWIZZLE_128B);
    }
    if (rc) return rc;

    if (dtype == BI_BF16) {
        if (!quant) return launch_t<__nv_bfloat16, 0>(mw, mx, p, st);
        return q->bits == 4 ? launch_t<__nv_bfloat16, 4>(mw, mx, p, st) : launch_t<__nv_bfloat16, 8>(mw, mx, p, st);
    }
    if (!quant) return launch_t<__half, 0>(mw, mx, p, st);
    return q->bits == 4 ? launch_t<__half, 4>(mw, mx, p, st) : launch_t<__half, 8>(mw, mx, p, st);
}

}  // namespace bi
