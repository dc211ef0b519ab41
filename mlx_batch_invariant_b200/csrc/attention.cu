// Split-KV attention with a fixed split size, key-by-key online softmax.
//
// Canonical order per (batch, head, query) -- the order of the reference's
// lane-parallel Metal kernels (mlx_batch_invariant/kernels/attention.py:47-85):
//   * keys run in index order inside fixed splits of `split` keys (256);
//   * the head dimension is cut into 32 "virtual lanes" of DL = D/32 dims.
//     Virtual lane v forms part_v = fma chain over its dims of q_hat*k from 0,
//     q_hat = float(q) * scale. The 32 partials are summed by the xor-butterfly
//     tree 16, 8, 4, 2, 1:  a_v = part_v + part_{v+16}; b_v = a_v + a_{v+8};
//     c_v = b_v + b_{v+4}; d_v = c_v + c_{v+2}; s = d_0 + d_1;
//   * per key: m' = max(m, s); corr = exp(m - m'); p = exp(s - m');
//     l = fma(l, corr, p); acc_d = fma(acc_d, corr, p * v_d); m = m';
//     from m = -inf, l = 0, acc = 0 at the start of every split;
//   * split partials merge left to right: M' = max(M, m); c_old = exp(M - M');
//     c_new = exp(m - M'); L = fma(L, c_old, l * c_new);
//     A_d = fma(A_d, c_old, acc_d * c_new); out_d = T(A_d / L).
//
// Work layout on the GPU (free to differ, it moves no rounding): eight real
// lanes -- an "octet" -- carry one key stream. Real lane r owns virtual lanes
// r, r+8, r+16, r+24, so the first two tree levels are thread-local adds and
// only levels 4, 2, 1 cross lanes (three shuffles). A warp holds four octets
// that work on four different units at once.
//
// Of the two exponentials of a key step one always has argument exactly 0
// (m' equals m or s) and exp(0) is exactly 1, so one evaluation of
// exp(-|s - m|) yields both factors with unchanged bits.
//
// decode_kernel and prefill_kernel call the same key_update() and merge
// functions (merge_coeffs / merge_acc for the split fold), which is why a token's bits do not depend on which of the two
// produced it.
#include <algorithm>
#include "bi_common.cuh"
#include "bi_ptx.cuh"
#include "peer_push.cuh"

namespace bi {
namespace {

constexpr int OCT = 8;        // real lanes per key stream
constexpr int OCT_PER_WARP = 4;
constexpr int NCHUNK = 4;     // virtual lanes per real lane

template <typename T, int DL> struct alignas(sizeof(T) * DL) Chunk { T v[DL]; };

// Load the 4*DL dims of `row` owned by real lane r, upcast to fp32.
template <typename T, int DL>
__device__ __forceinline__ void load_slice(const T* __restrict__ row, int r, float (&dst)[NCHUNK * DL]) {
    using C = Chunk<T, DL>;
    const C* p = reinterpret_cast<const C*>(row);
#pragma unroll
    for (int j = 0; j < NCHUNK; ++j) {
        C c = p[r + OCT * j];
#pragma unroll
        for (int d = 0; d < DL; ++d) dst[j * DL + d] = Cvt<T>::up(c.v[d]);
    }
}

// One key against NQ query rows that share it. `act[iq]` says whether query iq sees the key.
template <int NQ, int DL>
__device__ __forceinline__ void key_update(const float (&kf)[NCHUNK * DL], const float (&vf)[NCHUNK * DL],
                                           const float (&q)[NQ][NCHUNK * DL], float (&m)[NQ], float (&l)[NQ],
                                           float (&acc)[NQ][NCHUNK * DL], const bool (&act)[NQ]) {
#pragma unroll
    for (int iq = 0; iq < NQ; ++iq) {
        float part[NCHUNK];
#pragma unroll
        for (int j = 0; j < NCHUNK; ++j) {
            float a = 0.0f;
#pragma unroll
            for (int d = 0; d < DL; ++d) a = fma_rn(q[iq][j * DL + d], kf[j * DL + d], a);
            part[j] = a;
        }
        // tree level 16 and 8 (thread-local), then 4, 2, 1 across the octet
        float s = add_rn(add_rn(part[0], part[2]), add_rn(part[1], part[3]));
        s = add_rn(s, __shfl_xor_sync(0xffffffffu, s, 4));
        s = add_rn(s, __shfl_xor_sync(0xffffffffu, s, 2));
        s = add_rn(s, __shfl_xor_sync(0xffffffffu, s, 1));

        const float m_old = m[iq];
        const float m_new = fmaxf(m_old, s);
        const float e = expf_canon(-fabsf(sub_rn(s, m_old)));
        const bool rises = s >= m_old;
        const float corr = rises ? e : 1.0f;
        const float p = rises ? 1.0f : e;
        const float l_new = fma_rn(l[iq], corr, p);
        if (act[iq]) {
            m[iq] = m_new;
            l[iq] = l_new;
#pragma unroll
            for (int d = 0; d < NCHUNK * DL; ++d) acc[iq][d] = fma_rn(acc[iq][d], corr, mul_rn(p, vf[d]));
        }
    }
}

// Fold one split's (m, l) into the running (M, L) and return the two factors
// the accumulators are folded with:  A_d = fma(A_d, c_old, acc_d * c_new).
__device__ __forceinline__ void merge_coeffs(float& M, float& L, float m, float l, float& c_old, float& c_new) {
    const float M_new = fmaxf(M, m);
    c_old = expf_canon(sub_rn(M, M_new));
    c_new = expf_canon(sub_rn(m, M_new));
    L = fma_rn(L, c_old, mul_rn(l, c_new));
    M = M_new;
}
__device__ __forceinline__ float merge_acc(float A, float c_old, float acc, float c_new) {
    return fma_rn(A, c_old, mul_rn(acc, c_new));
}

struct KvLayout {
    int64_t sb, sh, sl;  // element strides of k and v: batch (or page, when paged), kv head, key
    // Paged cache (table != nullptr): k and v are pools of pages [page, kv head, key in page, D]; keys
    // [i * page_size, (i + 1) * page_size) of sequence b live in page table[b * table_stride + i].
    const int32_t* table;
    int page_size, table_stride;
};

// ---- decode: unit = (batch, kv head, chunk of GU query heads, split) ----------
template <typename T, int DL, int GU>
__global__ void __launch_bounds__(128) decode_kernel(const T* __restrict__ q, const T* __restrict__ k,
                                                     const T* __restrict__ v, const int32_t* __restrict__ kv_lens,
                                                     float* __restrict__ pm, float* __restrict__ pl,
                                                     float* __restrict__ pacc, int B, int Hq, int Hkv, int L,
                                                     KvLayout lay, float scale, int split, int nsplit, int nchunk) {
    ptx::grid_dep_launch();   // the next kernel of the stream may start its set-up
    ptx::grid_dep_wait();     // everything before this kernel has completed and is visible
    constexpr int D = 32 * DL;
    constexpr int NL = NCHUNK * DL;
    const int lane = threadIdx.x & 31;
    const int r = lane & (OCT - 1);
    const long long oct = ((long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * OCT_PER_WARP + (lane >> 3);
    const long long units = (long long)B * Hkv * nchunk * nsplit;
    const bool unit_ok = oct < units;
    long long u = unit_ok ? oct : 0;
    const int sp = (int)(u % nsplit); u /= nsplit;
    const int chunk = (int)(u % nchunk); u /= nchunk;
    const int hk = (int)(u % Hkv); u /= Hkv;
    const int b = (int)u;
    const int G = Hq / Hkv;
    const int h0 = hk * G + chunk * GU;
    const int gcount = min(GU, G - chunk * GU);
    const int Lb = kv_lens ? min(kv_lens[b], L) : L;
    const int j0 = sp * split;
    const int nk = (unit_ok && j0 < Lb) ? (min(Lb, j0 + split) - j0) : 0;

    const T* kb = k + (int64_t)b * lay.sb + (int64_t)hk * lay.sh + (int64_t)j0 * lay.sl;
    const T* vb = v + (int64_t)b * lay.sb + (int64_t)hk * lay.sh + (int64_t)j0 * lay.sl;

    float qf[GU][NL];
    bool act_head[GU];
#pragma unroll
    for (int iq = 0; iq < GU; ++iq) {
        act_head[iq] = iq < gcount;
        const T* qr = q + ((int64_t)b * Hq + h0 + min(iq, gcount - 1)) * D;
        load_slice<T, DL>(qr, r, qf[iq]);
#pragma unroll
        for (int d = 0; d < NL; ++d) qf[iq][d] = mul_rn(qf[iq][d], scale);
    }
    float m[GU], l[GU], acc[GU][NL];
#pragma unroll
    for (int iq = 0; iq < GU; ++iq) {
        m[iq] = -INFINITY; l[iq] = 0.0f;
#pragma unroll
        for (int d = 0; d < NL; ++d) acc[iq][d] = 0.0f;
    }

    // The trip count is the warp maximum so the shuffles stay converged; an octet
    // past its own range re-reads its first key and discards the step.
    int nk_max = nk;
    nk_max = max(nk_max, __shfl_xor_sync(0xffffffffu, nk_max, 8));
    nk_max = max(nk_max, __shfl_xor_sync(0xffffffffu, nk_max, 16));
    constexpr bool PF = DL < 8;  // keep the next key's rows in registers while this one is processed
    float kf[NL], vf[NL];
    if (PF && nk_max > 0) {
        load_slice<T, DL>(kb, r, kf);
        load_slice<T, DL>(vb, r, vf);
    }
    for (int jj = 0; jj < nk_max; ++jj) {
        const bool on = jj < nk;
        bool act[GU];
#pragma unroll
        for (int iq = 0; iq < GU; ++iq) act[iq] = on && act_head[iq];
        if (PF) {
            float kn[NL], vn[NL];
            const int jn = (jj + 1 < nk) ? jj + 1 : 0;
            load_slice<T, DL>(kb + (int64_t)jn * lay.sl, r, kn);
            load_slice<T, DL>(vb + (int64_t)jn * lay.sl, r, vn);
            key_update<GU, DL>(kf, vf, qf, m, l, acc, act);
#pragma unroll
            for (int d = 0; d < NL; ++d) { kf[d] = kn[d]; vf[d] = vn[d]; }
        } else {
            const int jc = on ? jj : 0;
            load_slice<T, DL>(kb + (int64_t)jc * lay.sl, r, kf);
            load_slice<T, DL>(vb + (int64_t)jc * lay.sl, r, vf);
            key_update<GU, DL>(kf, vf, qf, m, l, acc, act);
        }
    }

    if (nk > 0) {
#pragma unroll
        for (int iq = 0; iq < GU; ++iq) {
            if (iq < gcount) {
                const int64_t po = ((int64_t)b * Hq + h0 + iq) * nsplit + sp;
                if (r == 0) { pm[po] = m[iq]; pl[po] = l[iq]; }
#pragma unroll
                for (int j = 0; j < NCHUNK; ++j)
#pragma unroll
                    for (int d = 0; d < DL; ++d)
                        pacc[po * D + (r + OCT * j) * DL + d] = acc[iq][j * DL + d];
            }
        }
    }
}

// ---- decode, streamed: same units and arithmetic as decode_kernel; K/V rows reach the lanes through a
// per-warp ring of shared-memory stages filled by 16-byte cp.async copies, so several keys per stream
// are in flight while one is processed. The fp32 work runs as packed f32x2 instructions (two
// independent round-to-nearest operations each: same bits as the scalar forms), pairing virtual
// lanes (r, r+8) and (r+16, r+24); and the scalar softmax step of a head is evaluated on one lane of
// the octet and handed to the others by shuffle instead of being repeated on all eight.
constexpr int DEC2_KC = 4;       // keys per stream per stage
constexpr int DEC2_STAGES = 2;
constexpr int DEC2_WARPS = 4;

template <typename T, int DL> struct Dec2Cfg {
    static constexpr int ROWB = 32 * DL * (int)sizeof(T);                  // bytes of one K or V row
    static constexpr int PITCH = ROWB + 64;                                // rows of the 4 streams land on different banks
    static constexpr int ROWS = 2 * DEC2_KC * OCT_PER_WARP;                // rows per stage: (k|v, key, stream)
    static constexpr int STAGE_BYTES = ROWS * PITCH;
    static constexpr int WARP_BYTES = DEC2_STAGES * STAGE_BYTES;
    static constexpr int SMEM_BYTES = DEC2_WARPS * WARP_BYTES;
};

// two T values (consecutive dims) packed in one 32-bit word -> fp32, for 16-bit T
template <typename T> __device__ __forceinline__ float word_lo(uint32_t w);
template <typename T> __device__ __forceinline__ float word_hi(uint32_t w);
template <> __device__ __forceinline__ float word_lo<__nv_bfloat16>(uint32_t w) { return __uint_as_float(w << 16); }
template <> __device__ __forceinline__ float word_hi<__nv_bfloat16>(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }
template <> __device__ __forceinline__ float word_lo<__half>(uint32_t w) { return __half2float(__ushort_as_half((unsigned short)(w & 0xFFFFu))); }
template <> __device__ __forceinline__ float word_hi<__half>(uint32_t w) { return __half2float(__ushort_as_half((unsigned short)(w >> 16))); }

// Slice of a row owned by real lane r, as packed pairs: dst[jp][d] = (x[(r + 16 jp) * DL + d], x[(r + 8 + 16 jp) * DL + d])
template <typename T, int DL>
__device__ __forceinline__ void load_slice_pairs(const uint8_t* row, int r, uint64_t (&dst)[2][DL]) {
    float f[NCHUNK][DL];
#pragma unroll
    for (int j = 0; j < NCHUNK; ++j) {
        const uint8_t* c = row + (r + OCT * j) * DL * sizeof(T);
        if constexpr (sizeof(T) == 4) {
#pragma unroll
            for (int d = 0; d < DL; ++d) f[j][d] = reinterpret_cast<const float*>(c)[d];
        } else if constexpr (DL == 1) {
            f[j][0] = Cvt<T>::up(*reinterpret_cast<const T*>(c));
        } else {
#pragma unroll
            for (int d2 = 0; d2 < DL / 2; ++d2) {
                const uint32_t w = reinterpret_cast<const uint32_t*>(c)[d2];
                f[j][2 * d2] = word_lo<T>(w);
                f[j][2 * d2 + 1] = word_hi<T>(w);
            }
        }
    }
#pragma unroll
    for (int jp = 0; jp < 2; ++jp)
#pragma unroll
        for (int d = 0; d < DL; ++d) dst[jp][d] = ptx::pack2(f[2 * jp][d], f[2 * jp + 1][d]);
}

template <typename T, int DL, int GU>
__global__ void __launch_bounds__(32 * DEC2_WARPS) decode_stream_kernel(
    const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, const int32_t* __restrict__ kv_lens,
    float* __restrict__ pm, float* __restrict__ pl, float* __restrict__ pacc, int B, int Hq, int Hkv, int L,
    KvLayout lay, float scale, int split, int nsplit, int nchunk) {
    ptx::grid_dep_launch();   // the next kernel of the stream may start its set-up
    ptx::grid_dep_wait();     // everything before this kernel has completed and is visible
    using C = Dec2Cfg<T, DL>;
    constexpr int D = 32 * DL;
    constexpr int SEGS = C::ROWB / 16;                 // 16-byte segments per row
    extern __shared__ __align__(16) uint8_t dec_smem[];
    const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = lane & (OCT - 1), o = lane >> 3;
    uint8_t* ring = dec_smem + wid * C::WARP_BYTES;
    const uint32_t ring_s = (uint32_t)__cvta_generic_to_shared(ring);

    const long long oct = ((long long)blockIdx.x * DEC2_WARPS + wid) * OCT_PER_WARP + o;
    const long long units = (long long)B * Hkv * nchunk * nsplit;
    const bool unit_ok = oct < units;
    long long u = unit_ok ? oct : 0;
    const int sp = (int)(u % nsplit); u /= nsplit;
    const int chunk = (int)(u % nchunk); u /= nchunk;
    const int hk = (int)(u % Hkv); u /= Hkv;
    const int b = (int)u;
    const int G = Hq / Hkv;
    const int h0 = hk * G + chunk * GU;
    const int gcount = min(GU, G - chunk * GU);
    const int Lb = kv_lens ? min(kv_lens[b], L) : L;
    const int j0 = sp * split;
    const int nk = (unit_ok && j0 < Lb) ? (min(Lb, j0 + split) - j0) : 0;
    int nk_max = nk;
    nk_max = max(nk_max, __shfl_xor_sync(0xffffffffu, nk_max, 8));
    nk_max = max(nk_max, __shfl_xor_sync(0xffffffffu, nk_max, 16));
    const int nstage = (nk_max + DEC2_KC - 1) / DEC2_KC;

    // copy stage `st` (keys st*KC .. st*KC+KC-1 of every stream) into ring slot st % STAGES. Each octet
    // copies its own stream's rows: eight lanes x 16 bytes = 128 contiguous bytes per instruction.
    const T* const kb = k + (int64_t)b * lay.sb + (int64_t)hk * lay.sh + (int64_t)j0 * lay.sl;
    const T* const vb = v + (int64_t)b * lay.sb + (int64_t)hk * lay.sh + (int64_t)j0 * lay.sl;
    const int last_key = max(nk - 1, 0);               // past the stream's end: re-read a valid row
    auto issue = [&](int st) {
        if (st < nstage) {
            const uint32_t dst0 = ring_s + (uint32_t)(st % DEC2_STAGES) * C::STAGE_BYTES + (uint32_t)o * C::PITCH + r * 16;
#pragma unroll
            for (int key = 0; key < DEC2_KC; ++key) {
                const int64_t off = (int64_t)min(st * DEC2_KC + key, last_key) * lay.sl;
                const uint8_t* ks = reinterpret_cast<const uint8_t*>(kb + off) + r * 16;
                const uint8_t* vs = reinterpret_cast<const uint8_t*>(vb + off) + r * 16;
#pragma unroll
                for (int sg = 0; sg < SEGS; sg += OCT) {
                    if (SEGS >= OCT || r < SEGS) {
                        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst0 + (key * 4) * C::PITCH + sg * 16), "l"(ks + sg * 16) : "memory");
                        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst0 + ((DEC2_KC + key) * 4) * C::PITCH + sg * 16), "l"(vs + sg * 16) : "memory");
                    }
                }
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    // queries of this unit, pre-scaled, as packed pairs
    uint64_t qp[GU][2][DL];
#pragma unroll
    for (int iq = 0; iq < GU; ++iq) {
        const T* qr = q + ((int64_t)b * Hq + h0 + min(iq, gcount - 1)) * D;
        float qf[NCHUNK * DL];
        load_slice<T, DL>(qr, r, qf);
#pragma unroll
        for (int jp = 0; jp < 2; ++jp)
#pragma unroll
            for (int d = 0; d < DL; ++d)
                qp[iq][jp][d] = ptx::pack2(mul_rn(qf[(2 * jp) * DL + d], scale), mul_rn(qf[(2 * jp + 1) * DL + d], scale));
    }
    uint64_t accp[GU][2][DL];
#pragma unroll
    for (int iq = 0; iq < GU; ++iq)
#pragma unroll
        for (int jp = 0; jp < 2; ++jp)
#pragma unroll
            for (int d = 0; d < DL; ++d) accp[iq][jp][d] = ptx::pack2(0.0f, 0.0f);
    // lane r keeps the softmax scalars (m, l) of head r % GU only
    const int my_head = r % GU;
    float m_own = -INFINITY, l_own = 0.0f;

    for (int st = 0; st < DEC2_STAGES - 1; ++st) issue(st);
    for (int st = 0; st < nstage; ++st) {
        asm volatile("cp.async.wait_group %0;" ::"n"(DEC2_STAGES - 2) : "memory");
        __syncwarp();                                      // stage st visible; slot of stage st-1 free
        issue(st + DEC2_STAGES - 1);
        const uint8_t* stage = ring + (st % DEC2_STAGES) * C::STAGE_BYTES;
        // Phase A: scores of every key of the stage (independent of the softmax state, so the
        // four keys' dot products and shuffle trees overlap). Phase B: the sequential softmax steps.
        float s[DEC2_KC][GU];
#pragma unroll
        for (int key = 0; key < DEC2_KC; ++key) {
            uint64_t kp[2][DL];
            load_slice_pairs<T, DL>(stage + (key * 4 + o) * C::PITCH, r, kp);
#pragma unroll
            for (int iq = 0; iq < GU; ++iq) {
                uint64_t p01 = ptx::pack2(0.0f, 0.0f), p23 = ptx::pack2(0.0f, 0.0f);
#pragma unroll
                for (int d = 0; d < DL; ++d) {
                    p01 = ptx::fma2_rn(qp[iq][0][d], kp[0][d], p01);   // virtual lanes r, r+8
                    p23 = ptx::fma2_rn(qp[iq][1][d], kp[1][d], p23);   // virtual lanes r+16, r+24
                }
                float a0, a1;
                ptx::unpack2(ptx::add2_rn(p01, p23), a0, a1);          // (part_r + part_{r+16}, part_{r+8} + part_{r+24})
                float t = add_rn(a0, a1);
                t = add_rn(t, __shfl_xor_sync(0xffffffffu, t, 4));
                t = add_rn(t, __shfl_xor_sync(0xffffffffu, t, 2));
                t = add_rn(t, __shfl_xor_sync(0xffffffffu, t, 1));
                s[key][iq] = t;
            }
        }
        // Softmax scalars of head `my_head` for every key of the stage, off the serial chain (see
        // decode_warp_stream_kernel): prefix maximum first, then independent exponentials.
        float e_own[DEC2_KC];
        bool rises_own[DEC2_KC];
        {
            const bool mine = my_head < gcount;
            float mrun = m_own;
#pragma unroll
            for (int key = 0; key < DEC2_KC; ++key) {
                float s_own = s[key][0];
#pragma unroll
                for (int iq = 1; iq < GU; ++iq) if (my_head == iq) s_own = s[key][iq];
                e_own[key] = expf_canon(-fabsf(sub_rn(s_own, mrun)));
                rises_own[key] = s_own >= mrun;
                if (mine && st * DEC2_KC + key < nk) mrun = fmaxf(mrun, s_own);
            }
            m_own = mrun;
        }
#pragma unroll
        for (int key = 0; key < DEC2_KC; ++key) {
            const int jj = st * DEC2_KC + key;
            if (jj >= nk_max) break;                       // warp-uniform
            const bool on = jj < nk;
            uint64_t vp[2][DL];
            load_slice_pairs<T, DL>(stage + ((DEC2_KC + key) * 4 + o) * C::PITCH, r, vp);
            const float corr_own = rises_own[key] ? e_own[key] : 1.0f;
            const float p_own = rises_own[key] ? 1.0f : e_own[key];
            if (on && my_head < gcount) l_own = fma_rn(l_own, corr_own, p_own);
#pragma unroll
            for (int iq = 0; iq < GU; ++iq) {
                const int src = (lane & 24) | iq;
                const float corr = __shfl_sync(0xffffffffu, corr_own, src);
                const float pw = __shfl_sync(0xffffffffu, p_own, src);
                if (on && iq < gcount) {
                    const uint64_t c2 = ptx::pack2(corr, corr), p2 = ptx::pack2(pw, pw);
#pragma unroll
                    for (int jp = 0; jp < 2; ++jp)
#pragma unroll
                        for (int d = 0; d < DL; ++d)
                            accp[iq][jp][d] = ptx::fma2_rn(accp[iq][jp][d], c2, ptx::mul2_rn(p2, vp[jp][d]));
                }
            }
        }
    }
    asm volatile("cp.async.wait_all;" ::: "memory");

    if (nk > 0) {
#pragma unroll
        for (int iq = 0; iq < GU; ++iq) {
            if (iq < gcount) {
                const int64_t po = ((int64_t)b * Hq + h0 + iq) * nsplit + sp;
                if (r == iq) { pm[po] = m_own; pl[po] = l_own; }
#pragma unroll
                for (int jp = 0; jp < 2; ++jp)
#pragma unroll
                    for (int d = 0; d < DL; ++d) {
                        float lo, hi;
                        ptx::unpack2(accp[iq][jp][d], lo, hi);
                        pacc[po * D + (r + OCT * (2 * jp)) * DL + d] = lo;
                        pacc[po * D + (r + OCT * (2 * jp + 1)) * DL + d] = hi;
                    }
            }
        }
    }
}

// ---- decode, one stream per warp: when there are few (batch, kv head, split) streams, the four octets
// of a warp take four query heads of the SAME stream instead of four streams. The K/V rows are copied
// into shared memory once per warp and read by all four octets, every lane carries one head's state
// only (few registers, many resident warps), so short caches no longer leave the GPU waiting on one
// sequential chain per stream. Arithmetic per head is unchanged.
constexpr int DECW_KC = 8;
constexpr int DECW_STAGES = 3;
constexpr int DECW_WARPS = 16;   // most warps a CTA may have; the launch picks the count (see launch_decode)

template <typename T, int DL> struct DecWCfg {
    static constexpr int ROWB = 32 * DL * (int)sizeof(T);
    static constexpr int ROWS = 2 * DECW_KC;                                // (k|v, key)
    static constexpr int STAGE_BYTES = ROWS * ROWB;
    static constexpr int WARP_BYTES = DECW_STAGES * STAGE_BYTES;
    static constexpr int SMEM_BYTES = DECW_WARPS * WARP_BYTES;
};

template <typename T, int DL, int MAXW>
__global__ void __launch_bounds__(32 * MAXW) decode_warp_stream_kernel(
    const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, const int32_t* __restrict__ kv_lens,
    float* __restrict__ pm, float* __restrict__ pl, float* __restrict__ pacc, int B, int Hq, int Hkv, int L,
    KvLayout lay, float scale, int split, int nsplit, int nchunk) {
    ptx::grid_dep_launch();   // the next kernel of the stream may start its set-up
    ptx::grid_dep_wait();     // everything before this kernel has completed and is visible
    using C = DecWCfg<T, DL>;
    constexpr int D = 32 * DL;
    constexpr int SEGS = C::ROWB / 16;
    extern __shared__ __align__(16) uint8_t dec_smem[];
    const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = lane & (OCT - 1), o = lane >> 3;
    uint8_t* ring = dec_smem + wid * C::WARP_BYTES;
    const uint32_t ring_s = (uint32_t)__cvta_generic_to_shared(ring);

    const long long stream = (long long)blockIdx.x * (blockDim.x >> 5) + wid; // (b, kv head, chunk of 4 heads, split)
    const long long streams = (long long)B * Hkv * nchunk * nsplit;
    if (stream >= streams) return;                                           // whole warp
    long long u = stream;
    const int sp = (int)(u % nsplit); u /= nsplit;
    const int chunk = (int)(u % nchunk); u /= nchunk;
    const int hk = (int)(u % Hkv); u /= Hkv;
    const int b = (int)u;
    const int G = Hq / Hkv;
    const int gcount = min(OCT_PER_WARP, G - chunk * OCT_PER_WARP);
    const bool head_ok = o < gcount;
    const int h = hk * G + chunk * OCT_PER_WARP + min(o, gcount - 1);
    const int Lb = kv_lens ? min(kv_lens[b], L) : L;
    const int j0 = sp * split;
    const int nk = j0 < Lb ? (min(Lb, j0 + split) - j0) : 0;               // warp-uniform
    if (nk == 0) return;
    const int nstage = (nk + DECW_KC - 1) / DECW_KC;
    const T* const kb = k + (int64_t)b * lay.sb + (int64_t)hk * lay.sh + (int64_t)j0 * lay.sl;
    const T* const vb = v + (int64_t)b * lay.sb + (int64_t)hk * lay.sh + (int64_t)j0 * lay.sl;

    auto issue = [&](int st) {
        if (st < nstage) {
            const uint32_t dst0 = ring_s + (uint32_t)(st % DECW_STAGES) * C::STAGE_BYTES;
#pragma unroll
            for (int i = lane; i < C::ROWS * SEGS; i += 32) {
                const int seg = i % SEGS, row = i / SEGS;                    // row = kv * KC + key
                const int key = row % DECW_KC;
                const int64_t off = (int64_t)min(st * DECW_KC + key, nk - 1) * lay.sl;
                const uint8_t* src = reinterpret_cast<const uint8_t*>((row >= DECW_KC ? vb : kb) + off) + seg * 16;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst0 + row * C::ROWB + seg * 16), "l"(src) : "memory");
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    uint64_t qp[2][DL];
    {
        const T* qr = q + ((int64_t)b * Hq + h) * D;
        float qf[NCHUNK * DL];
        load_slice<T, DL>(qr, r, qf);
#pragma unroll
        for (int jp = 0; jp < 2; ++jp)
#pragma unroll
            for (int d = 0; d < DL; ++d)
                qp[jp][d] = ptx::pack2(mul_rn(qf[(2 * jp) * DL + d], scale), mul_rn(qf[(2 * jp + 1) * DL + d], scale));
    }
    uint64_t accp[2][DL];
#pragma unroll
    for (int jp = 0; jp < 2; ++jp)
#pragma unroll
        for (int d = 0; d < DL; ++d) accp[jp][d] = ptx::pack2(0.0f, 0.0f);
    float m_own = -INFINITY, l_own = 0.0f;

    for (int st = 0; st < DECW_STAGES - 1; ++st) issue(st);
    for (int st = 0; st < nstage; ++st) {
        asm volatile("cp.async.wait_group %0;" ::"n"(DECW_STAGES - 2) : "memory");
        __syncwarp();
        issue(st + DECW_STAGES - 1);
        const uint8_t* stage = ring + (st % DECW_STAGES) * C::STAGE_BYTES;
        float s[DECW_KC];
#pragma unroll
        for (int key = 0; key < DECW_KC; ++key) {
            uint64_t kp[2][DL];
            load_slice_pairs<T, DL>(stage + key * C::ROWB, r, kp);
            uint64_t p01 = ptx::pack2(0.0f, 0.0f), p23 = ptx::pack2(0.0f, 0.0f);
#pragma unroll
            for (int d = 0; d < DL; ++d) {
                p01 = ptx::fma2_rn(qp[0][d], kp[0][d], p01);
                p23 = ptx::fma2_rn(qp[1][d], kp[1][d], p23);
            }
            float a0, a1;
            ptx::unpack2(ptx::add2_rn(p01, p23), a0, a1);
            float t = add_rn(a0, a1);
            t = add_rn(t, __shfl_xor_sync(0xffffffffu, t, 4));
            t = add_rn(t, __shfl_xor_sync(0xffffffffu, t, 2));
            t = add_rn(t, __shfl_xor_sync(0xffffffffu, t, 1));
            s[key] = t;
        }
        // Softmax scalars of the stage, off the serial chain: the running maximum before key j is a prefix
        // maximum of scores that are already known (max is exact, so evaluating it ahead changes no bit),
        // and with it every key's exp(-|s_j - m_j|) is independent of the others. What stays sequential
        // per key is l = fma(l, corr, p) and acc = fma(acc, corr, p * v): the same operations on the same
        // operands in the same order as the key-by-key form.
        float e[DECW_KC];
        bool rises[DECW_KC];
        {
            float mrun = m_own;
#pragma unroll
            for (int key = 0; key < DECW_KC; ++key) {
                e[key] = expf_canon(-fabsf(sub_rn(s[key], mrun)));
                rises[key] = s[key] >= mrun;
                if (st * DECW_KC + key < nk) mrun = fmaxf(mrun, s[key]);   // warp-uniform predicate
            }
            m_own = mrun;
        }
#pragma unroll
        for (int key = 0; key < DECW_KC; ++key) {
            if (st * DECW_KC + key >= nk) break;                            // warp-uniform
            uint64_t vp[2][DL];
            load_slice_pairs<T, DL>(stage + (DECW_KC + key) * C::ROWB, r, vp);
            const float corr = rises[key] ? e[key] : 1.0f;
            const float pw = rises[key] ? 1.0f : e[key];
            l_own = fma_rn(l_own, corr, pw);
            const uint64_t c2 = ptx::pack2(corr, corr), p2 = ptx::pack2(pw, pw);
#pragma unroll
            for (int jp = 0; jp < 2; ++jp)
#pragma unroll
                for (int d = 0; d < DL; ++d) accp[jp][d] = ptx::fma2_rn(accp[jp][d], c2, ptx::mul2_rn(p2, vp[jp][d]));
        }
    }
    asm volatile("cp.async.wait_all;" ::: "memory");

    if (head_ok) {
        const int64_t po = ((int64_t)b * Hq + h) * nsplit + sp;
        if (r == 0) { pm[po] = m_own; pl[po] = l_own; }
#pragma unroll
        for (int jp = 0; jp < 2; ++jp)
#pragma unroll
            for (int d = 0; d < DL; ++d) {
                float lo, hi;
                ptx::unpack2(accp[jp][d], lo, hi);
                pacc[po * D + (r + OCT * (2 * jp)) * DL + d] = lo;
                pacc[po * D + (r + OCT * (2 * jp + 1)) * DL + d] = hi;
            }
    }
}

// ---- decode, a key per lane: for 16-bit K/V with head_dim 128, the layout the hardware likes best.
// The canonical arithmetic is unchanged; what changes is who computes it:
//   * scores: lane j of the warp owns key j of a 32-key block and evaluates the whole dot product of that key
//     with each of the NH query heads that share the kv head -- the 32 virtual-lane fma chains and the xor tree
//     16, 8, 4, 2, 1 become local packed-pair arithmetic (virtual lanes 2i and 2i+1 ride in one f32x2), so
//     no shuffle is needed, each K element is converted once for all heads, and 32 keys proceed at once;
//   * softmax scalars: the running maximum before each key is a prefix maximum over lanes (max is exact, so a
//     parallel scan gives the bits of the sequential one), after which every lane computes its own key's
//     exp(-|s - m|) -- 32 exponentials per instruction instead of one;
//   * accumulation: lane d owns dims 4d..4d+3 of all NH heads and walks the block's keys in order:
//     l = fma(l, corr, p), acc = fma(acc, corr, p * v), the factors read back from shared memory.
// A warp is one work item (batch, kv head, chunk of NH heads, split) at a time; items are dealt to a
// persistent grid round-robin, full splits first.
// Launch-shape constants, from measurements on B200 (bf16, 32/8 heads): two K blocks per warp beat one (eight and ten
// warps with one K block: 53.7 / 65.7 us against 50.1 us with seven warps and two at 64 x 560 keys; ten warps cap the
// kernel at 168 registers). Eight warps with two K blocks fit once the softmax factors of a block live in that
// block's own K buffer, which nothing reads after the scores.
constexpr int KL_WARPS = 8;    // most warps per CTA (one CTA per SM): two per scheduler. With fewer than two work items per
                               // warp the launch uses seven: each warp is then faster and the tail is what counts
                               // (64 x 560 keys: 50.1 us with seven, 53.2 with eight; 64 x 4096 keys: 268 against 248 us)
constexpr int KL_KBUFS = 2;    // K blocks in shared memory per warp: the next block is fetched a whole block ahead
constexpr int KL_UNROLL = 8;   // keys of the accumulation loop in flight
constexpr int KL_KEYS = 32;
struct KLCfg {
    static constexpr int ROWB = 256;                       // bytes of a K or V row (128 x 16 bit)
    static constexpr int KPITCH = ROWB + 16;               // lanes read different rows at one column: no bank conflict
    static constexpr int KBUF = KL_KEYS * KPITCH;
    static constexpr int VBUF = KL_KEYS * ROWB;
    static constexpr int QBYTES = 4 * 128 * 4;             // scaled queries of up to four heads, as packed pairs
    static constexpr int CPBYTES = KL_KEYS * 4 * 16;       // (corr, corr, p, p) per key and head
    static constexpr bool CP_IN_KBUF = KL_KBUFS == 2;      // the factors overwrite the block's K rows once the scores exist
    static_assert(CPBYTES <= KBUF, "the factors of a block must fit its K buffer");
    static constexpr int WARP_BYTES = KL_KBUFS * KBUF + VBUF + QBYTES + (CP_IN_KBUF ? 0 : CPBYTES);
    static constexpr int SMEM_BYTES = KL_WARPS * WARP_BYTES;
};

// P_I for every head: the packed partial sums (part_{2I}, part_{2I+1}) of virtual lanes 2I and 2I+1 -- piece I of
// the key's row (dims 8I .. 8I+7) against the queries' same dims, each a four-step fma chain from zero.
template <typename T, int NH, int I>
__device__ __forceinline__ void kl_leaf(const uint8_t* krow, const uint8_t* qs, uint64_t (&out)[NH]) {
    const uint4 kw = *reinterpret_cast<const uint4*>(krow + 16 * I);
    uint64_t k2[4];
    k2[0] = ptx::pack2(word_lo<T>(kw.x), word_lo<T>(kw.z));   // (x0, x4)
    k2[1] = ptx::pack2(word_hi<T>(kw.x), word_hi<T>(kw.z));   // (x1, x5)
    k2[2] = ptx::pack2(word_lo<T>(kw.y), word_lo<T>(kw.w));   // (x2, x6)
    k2[3] = ptx::pack2(word_hi<T>(kw.y), word_hi<T>(kw.w));   // (x3, x7)
#pragma unroll
    for (int h = 0; h < NH; ++h) {
        const ulonglong2 qa = *reinterpret_cast<const ulonglong2*>(qs + h * 512 + I * 32);
        const ulonglong2 qb = *reinterpret_cast<const ulonglong2*>(qs + h * 512 + I * 32 + 16);
        uint64_t p = ptx::fma2_rn(qa.x, k2[0], ptx::pack2(0.0f, 0.0f));
        p = ptx::fma2_rn(qa.y, k2[1], p);
        p = ptx::fma2_rn(qb.x, k2[2], p);
        p = ptx::fma2_rn(qb.y, k2[3], p);
        out[h] = p;
    }
}
// The xor tree over pieces: stride 8 is tree level 16 (virtual lanes v and v+16 are pieces I and I+8), then 4, 2, 1.
template <typename T, int NH, int STRIDE, int I>
__device__ __forceinline__ void kl_node(const uint8_t* krow, const uint8_t* qs, uint64_t (&out)[NH]) {
    uint64_t a[NH], b[NH];
    if constexpr (STRIDE == 8) {
        kl_leaf<T, NH, I>(krow, qs, a);
        kl_leaf<T, NH, I + 8>(krow, qs, b);
    } else {
        kl_node<T, NH, STRIDE * 2, I>(krow, qs, a);
        kl_node<T, NH, STRIDE * 2, I + STRIDE>(krow, qs, b);
    }
#pragma unroll
    for (int h = 0; h < NH; ++h) out[h] = ptx::add2_rn(a[h], b[h]);
}

template <typename T, int NH, int NW>
__global__ void __launch_bounds__(32 * NW, 1) decode_keylane_kernel(
    const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, const int32_t* __restrict__ kv_lens,
    float* __restrict__ pm, float* __restrict__ pl, float* __restrict__ pacc, int B, int Hq, int Hkv, int L,
    KvLayout lay, float scale, int split, int nsplit, int nchunk) {
    ptx::grid_dep_launch();   // the next kernel of the stream may start its set-up
    ptx::grid_dep_wait();     // everything before this kernel has completed and is visible
    using C = KLCfg;
    constexpr int D = 128;
    extern __shared__ __align__(16) uint8_t dec_smem[];
    const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint8_t* base = dec_smem + wid * C::WARP_BYTES;
    uint8_t* kbuf = base;
    uint8_t* vbuf = base + KL_KBUFS * C::KBUF;
    uint8_t* qs = vbuf + C::VBUF;
    uint8_t* const cps_own = qs + C::QBYTES;               // used only when the factors have a buffer of their own
    const uint32_t kbuf_s = (uint32_t)__cvta_generic_to_shared(kbuf), vbuf_s = (uint32_t)__cvta_generic_to_shared(vbuf);
    const int G = Hq / Hkv;
    const long long per_split = (long long)B * Hkv * nchunk;
    const long long items = per_split * nsplit;

    for (long long item = (long long)blockIdx.x * NW + wid; item < items; item += (long long)gridDim.x * NW) {
        const int sp = (int)(item / per_split);
        long long u = item - (long long)sp * per_split;
        const int chunk = (int)(u % nchunk); u /= nchunk;
        const int hk = (int)(u % Hkv);
        const int b = (int)(u / Hkv);
        const int Lb = kv_lens ? min(kv_lens[b], L) : L;
        const int j0 = sp * split;
        const int nk = j0 < Lb ? (min(Lb, j0 + split) - j0) : 0;             // warp-uniform
        if (nk == 0) continue;
        const int h0 = hk * G + chunk * NH;
        const int gcount = min(NH, G - chunk * NH);
        const T* const kb = k + (int64_t)b * lay.sb + (int64_t)hk * lay.sh + (int64_t)j0 * lay.sl;
        const T* const vb = v + (int64_t)b * lay.sb + (int64_t)hk * lay.sh + (int64_t)j0 * lay.sl;
        const int nblk = (nk + KL_KEYS - 1) / KL_KEYS;
        // first row of key block `blk` of the split: contiguous cache, or the page that holds it (a page is a
        // multiple of 32 keys, so a block never straddles two)
        auto block_rows = [&](const T* pool, const T* contiguous, int blk) -> const T* {
            if (lay.table == nullptr) return contiguous + (int64_t)blk * KL_KEYS * lay.sl;
            const int key = j0 + blk * KL_KEYS;
            const int page = lay.table[(int64_t)b * lay.table_stride + key / lay.page_size];
            return pool + (int64_t)page * lay.sb + (int64_t)hk * lay.sh + (int64_t)(key % lay.page_size) * lay.sl;
        };

        // a block of 32 rows: 512 pieces of 16 bytes, 16 per lane, consecutive lanes on consecutive pieces
        // lane's first piece of a block: row (lane >> 4), segment (lane & 15); each further piece is two rows on
        const int64_t row_bytes = lay.sl * (int64_t)sizeof(T);
        auto issue_rows = [&](const T* pool, const T* contiguous, uint32_t dst, int pitch, int blk) {
            const T* src = block_rows(pool, contiguous, blk);                   // row 0 of the block
            const int r0 = lane >> 4;
            const int last = nk - 1 - blk * KL_KEYS;                            // last valid row of the block
            const uint32_t d0 = dst + (lane >> 4) * pitch + (lane & 15) * 16;
            if (last >= KL_KEYS - 1) {
                const uint8_t* g = reinterpret_cast<const uint8_t*>(src) + r0 * row_bytes + (lane & 15) * 16;
#pragma unroll
                for (int it = 0; it < 16; ++it)
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d0 + it * 2 * pitch), "l"(g + it * 2 * row_bytes) : "memory");
            } else {
#pragma unroll
                for (int it = 0; it < 16; ++it) {
                    const int64_t row = min(r0 + it * 2, last);                                   // past the end: re-read a valid row
                    const uint8_t* g = reinterpret_cast<const uint8_t*>(src) + row * row_bytes + (lane & 15) * 16;
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d0 + it * 2 * pitch), "l"(g) : "memory");
                }
            }
        };
        __syncwarp();                                                        // the previous item's reads are done
        issue_rows(k, kb, kbuf_s, C::KPITCH, 0);
        asm volatile("cp.async.commit_group;" ::: "memory");
        // scaled queries as packed pairs: pair (8i + d, 8i + 4 + d) at qs[h][i][d]
#pragma unroll
        for (int h = 0; h < NH; ++h) {
            const T* qr = q + ((int64_t)b * Hq + h0 + min(h, gcount - 1)) * D;
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                const int d = t * 32 + lane;
                const int i = d >> 3, w = d & 7;
                *reinterpret_cast<float*>(qs + h * 512 + i * 32 + (w & 3) * 8 + (w >> 2) * 4) = mul_rn(Cvt<T>::up(qr[d]), scale);
            }
        }
        float m[NH], l[NH];
        uint64_t acc[NH][2];
#pragma unroll
        for (int h = 0; h < NH; ++h) {
            m[h] = -INFINITY; l[h] = 0.0f;
            acc[h][0] = ptx::pack2(0.0f, 0.0f); acc[h][1] = ptx::pack2(0.0f, 0.0f);
        }
        for (int blk = 0; blk < nblk; ++blk) {
            issue_rows(v, vb, vbuf_s, C::ROWB, blk);                         // lands while the scores are computed
            if (KL_KBUFS == 2 && blk + 1 < nblk) issue_rows(k, kb, kbuf_s + ((blk + 1) & 1) * C::KBUF, C::KPITCH, blk + 1);
            asm volatile("cp.async.commit_group;" ::: "memory");
            asm volatile("cp.async.wait_group 1;" ::: "memory");            // this block's K rows have landed
            __syncwarp();
            const int cnt = min(KL_KEYS, nk - blk * KL_KEYS);
            const bool valid = lane < cnt;
            // ---- scores of key `lane` for every head
            uint64_t dd[NH];
            uint8_t* const kcur = kbuf + (KL_KBUFS == 2 ? (blk & 1) * C::KBUF : 0);
            kl_node<T, NH, 1, 0>(kcur + lane * C::KPITCH, qs, dd);
            uint8_t* const cps = C::CP_IN_KBUF ? kcur : cps_own;
            if (C::CP_IN_KBUF) __syncwarp();                                 // every lane has read its K row: the buffer is free
            // ---- softmax scalars of the block
#pragma unroll
            for (int h = 0; h < NH; ++h) {
                float d0, d1;
                ptx::unpack2(dd[h], d0, d1);
                const float s = add_rn(d0, d1);
                float x = valid ? s : -INFINITY;                              // inclusive prefix maximum over the lanes
#pragma unroll
                for (int off = 1; off < 32; off <<= 1) {
                    const float y = __shfl_up_sync(0xffffffffu, x, off);
                    if (lane >= off) x = fmaxf(x, y);
                }
                float before = __shfl_up_sync(0xffffffffu, x, 1);
                before = fmaxf(m[h], lane == 0 ? -INFINITY : before);         // running maximum before this key
                const float e = expf_canon(-fabsf(sub_rn(s, before)));
                const bool rises = s >= before;
                const float corr = rises ? e : 1.0f, p = rises ? 1.0f : e;
                *reinterpret_cast<float4*>(cps + (lane * NH + h) * 16) = make_float4(corr, corr, p, p);
                m[h] = fmaxf(m[h], __shfl_sync(0xffffffffu, x, 31));
            }
            if (KL_KBUFS == 2) {
                asm volatile("cp.async.wait_group 0;" ::: "memory");        // V rows (and the next K rows) have landed
            } else {
                __syncwarp();                                                // every lane has read its K row
                if (blk + 1 < nblk) issue_rows(k, kb, kbuf_s, C::KPITCH, blk + 1);  // lands while this block is accumulated
                asm volatile("cp.async.commit_group;" ::: "memory");
                asm volatile("cp.async.wait_group 1;" ::: "memory");        // this block's V rows have landed
            }
            __syncwarp();
            // ---- accumulation, key by key; lane owns dims 4*lane .. 4*lane+3 of every head
#pragma unroll KL_UNROLL
            for (int j = 0; j < cnt; ++j) {
                const uint2 vw = *reinterpret_cast<const uint2*>(vbuf + j * C::ROWB + lane * 8);
                const uint64_t v01 = ptx::pack2(word_lo<T>(vw.x), word_hi<T>(vw.x));
                const uint64_t v23 = ptx::pack2(word_lo<T>(vw.y), word_hi<T>(vw.y));
#pragma unroll
                for (int h = 0; h < NH; ++h) {
                    const ulonglong2 cp = *reinterpret_cast<const ulonglong2*>(cps + (j * NH + h) * 16);
                    float c, c_, p, p_;
                    ptx::unpack2(cp.x, c, c_);
                    ptx::unpack2(cp.y, p, p_);
                    l[h] = fma_rn(l[h], c, p);
                    acc[h][0] = ptx::fma2_rn(acc[h][0], cp.x, ptx::mul2_rn(cp.y, v01));
                    acc[h][1] = ptx::fma2_rn(acc[h][1], cp.x, ptx::mul2_rn(cp.y, v23));
                }
            }
            __syncwarp();                                                    // before the buffers are refilled
        }
#pragma unroll
        for (int h = 0; h < NH; ++h) {
            if (h < gcount) {
                const int64_t po = ((int64_t)b * Hq + h0 + h) * nsplit + sp;
                if (lane == 0) { pm[po] = m[h]; pl[po] = l[h]; }
                float a0, a1, a2, a3;
                ptx::unpack2(acc[h][0], a0, a1);
                ptx::unpack2(acc[h][1], a2, a3);
                *reinterpret_cast<float4*>(pacc + po * D + lane * 4) = make_float4(a0, a1, a2, a3);
            }
        }
    }
}


// PUSH: the merged output is this rank's head slice of a gathered activation [B, world * Hq * D]: element (b, h, d)
// goes to column rank * Hq * D + h * D + d of every rank's destination and the launch ends with the gather's
// handshake (peer_push.cuh): the split merge and the all-gather after it are one kernel.
template <typename T, bool PUSH>
__global__ void __launch_bounds__(256) decode_combine_kernel(const float* __restrict__ pm, const float* __restrict__ pl,
                                                             const float* __restrict__ pacc,
                                                             const int32_t* __restrict__ kv_lens, T* __restrict__ out,
                                                             int64_t BH, int Hq, int D, int L, int split, int nsplit,
                                                             PushSink sink) {
    ptx::grid_dep_launch();   // the next kernel of the stream may start its set-up
    ptx::grid_dep_wait();     // everything before this kernel has completed and is visible
    const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid < BH * D) {
        const int64_t bh = gid / D;
        const int d = (int)(gid % D);
        const int b = (int)(bh / Hq);
        const int Lb = kv_lens ? min(kv_lens[b], L) : L;
        const int ns = (Lb + split - 1) / split;
        float M = -INFINITY, Ls = 0.0f, A = 0.0f;
        for (int i = 0; i < ns; ++i) {
            const int64_t po = bh * nsplit + i;
            float c_old, c_new;
            merge_coeffs(M, Ls, pm[po], pl[po], c_old, c_new);
            A = merge_acc(A, c_old, pacc[po * D + d], c_new);
        }
        const T val = Cvt<T>::down(div_canon(A, Ls));
        if (PUSH) {
            const int64_t f = (int64_t)Hq * D;
            const int64_t o = (int64_t)b * f * sink.world + (int64_t)sink.rank * f + (gid - (int64_t)b * f);
            for (int r = 0; r < sink.world; ++r) static_cast<T*>(sink.dst.p[r])[o] = val;
        } else {
            out[bh * D + d] = val;
        }
    }
    if (PUSH) push_handshake(sink);
}

template <typename T>
int launch_decode_combine(const float* pm, const float* pl, const float* pacc, const int32_t* kv_lens, void* out, int64_t BH,
                          int Hq, int D, int L, int split, int nsplit, const PushSink* sink, cudaStream_t st) {
    const int64_t n = BH * D;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (sink) launch_overlapped(decode_combine_kernel<T, true>, dim3(blocks), dim3(256), 0, st, pm, pl, pacc, kv_lens, (T*)nullptr, BH, Hq, D, L, split, nsplit, *sink);
    else launch_overlapped(decode_combine_kernel<T, false>, dim3(blocks), dim3(256), 0, st, pm, pl, pacc, kv_lens, static_cast<T*>(out), BH, Hq, D, L, split, nsplit, PushSink{});
    return check_launch("bi_attn_decode combine");
}

// ---- prefill: unit = (batch, head, block of QB consecutive queries) -----------
// QB queries share each K/V row (4, or 2 for the widest heads to stay in registers); which
// queries are grouped is a launch choice, a query's arithmetic is the same in any group.
// The running merge state (M, L, A) is touched once per split, so it lives in shared
// memory, one private slot per thread, and the registers hold the per-key state.
constexpr int PREFILL_THREADS = 128;
template <int DL> struct PrefillCfg { static constexpr int QB = DL >= 8 ? 2 : 4; };

template <typename T, int DL>
__global__ void __launch_bounds__(PREFILL_THREADS) prefill_kernel(const T* __restrict__ q, const T* __restrict__ k,
                                                      const T* __restrict__ v, T* __restrict__ out, int B, int Hq,
                                                      int Hkv, int Tq, int L, KvLayout lay, float scale, int causal,
                                                      int split) {
    ptx::grid_dep_launch();   // the next kernel of the stream may start its set-up
    ptx::grid_dep_wait();     // everything before this kernel has completed and is visible
    constexpr int D = 32 * DL;
    constexpr int NL = NCHUNK * DL;
    constexpr int QB = PrefillCfg<DL>::QB;
    extern __shared__ float merge_state[];  // [(QB * (NL + 2))][PREFILL_THREADS]
    const int lane = threadIdx.x & 31;
    const int r = lane & (OCT - 1);
    const int nblk = (Tq + QB - 1) / QB;
    const long long units = (long long)B * Hq * nblk;
    const long long oct = ((long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * OCT_PER_WARP + (lane >> 3);
    const bool unit_ok = oct < units;
    long long u = unit_ok ? oct : 0;
    const int blk = (int)(u % nblk); u /= nblk;
    const int h = (int)(u % Hq); u /= Hq;
    const int b = (int)u;
    const int hk = h / (Hq / Hkv);
    const int q0 = blk * QB;

    const T* kb = k + (int64_t)b * lay.sb + (int64_t)hk * lay.sh;
    const T* vb = v + (int64_t)b * lay.sb + (int64_t)hk * lay.sh;

    int nkeys[QB];
    float qf[QB][NL];
    int nkeys_max = 0;
#pragma unroll
    for (int iq = 0; iq < QB; ++iq) {
        const int qi = min(q0 + iq, Tq - 1);
        nkeys[iq] = (unit_ok && q0 + iq < Tq) ? (causal ? (L - Tq + qi + 1) : L) : 0;
        nkeys_max = max(nkeys_max, nkeys[iq]);
        const T* qr = q + (((int64_t)b * Hq + h) * Tq + qi) * D;
        load_slice<T, DL>(qr, r, qf[iq]);
#pragma unroll
        for (int d = 0; d < NL; ++d) qf[iq][d] = mul_rn(qf[iq][d], scale);
    }
    int warp_max = nkeys_max;
    warp_max = max(warp_max, __shfl_xor_sync(0xffffffffu, warp_max, 8));
    warp_max = max(warp_max, __shfl_xor_sync(0xffffffffu, warp_max, 16));
    const int nsplit = (warp_max + split - 1) / split;

    float* const slot = merge_state + threadIdx.x;  // element e of this thread: slot[e * PREFILL_THREADS]
    constexpr int STRIDE = PREFILL_THREADS;
    float m[QB], l[QB], acc[QB][NL];
#pragma unroll
    for (int iq = 0; iq < QB; ++iq) {
        slot[(iq * (NL + 2) + 0) * STRIDE] = -INFINITY;
        slot[(iq * (NL + 2) + 1) * STRIDE] = 0.0f;
#pragma unroll
        for (int d = 0; d < NL; ++d) slot[(iq * (NL + 2) + 2 + d) * STRIDE] = 0.0f;
    }

    for (int sp = 0; sp < nsplit; ++sp) {
#pragma unroll
        for (int iq = 0; iq < QB; ++iq) {
            m[iq] = -INFINITY; l[iq] = 0.0f;
#pragma unroll
            for (int d = 0; d < NL; ++d) acc[iq][d] = 0.0f;
        }
        const int j0 = sp * split;
        const int j1 = min(warp_max, j0 + split);
        constexpr bool PF = DL < 4;  // wider heads have no registers left for a look-ahead row
        float kf[NL], vf[NL];
        if (PF) {
            load_slice<T, DL>(kb + (int64_t)j0 * lay.sl, r, kf);
            load_slice<T, DL>(vb + (int64_t)j0 * lay.sl, r, vf);
        }
        for (int j = j0; j < j1; ++j) {
            bool act[QB];
#pragma unroll
            for (int iq = 0; iq < QB; ++iq) act[iq] = j < nkeys[iq];
            if (PF) {
                float kn[NL], vn[NL];
                const int jn = (j + 1 < j1) ? j + 1 : j0;
                load_slice<T, DL>(kb + (int64_t)jn * lay.sl, r, kn);
                load_slice<T, DL>(vb + (int64_t)jn * lay.sl, r, vn);
                key_update<QB, DL>(kf, vf, qf, m, l, acc, act);
#pragma unroll
                for (int d = 0; d < NL; ++d) { kf[d] = kn[d]; vf[d] = vn[d]; }
            } else {
                load_slice<T, DL>(kb + (int64_t)j * lay.sl, r, kf);
                load_slice<T, DL>(vb + (int64_t)j * lay.sl, r, vf);
                key_update<QB, DL>(kf, vf, qf, m, l, acc, act);
            }
        }
#pragma unroll
        for (int iq = 0; iq < QB; ++iq) {
            if (j0 < nkeys[iq]) {
                float* st = slot + (iq * (NL + 2)) * STRIDE;
                float Mq = st[0], Lq = st[STRIDE], c_old, c_new;
                merge_coeffs(Mq, Lq, m[iq], l[iq], c_old, c_new);
                st[0] = Mq; st[STRIDE] = Lq;
#pragma unroll
                for (int d = 0; d < NL; ++d)
                    st[(2 + d) * STRIDE] = merge_acc(st[(2 + d) * STRIDE], c_old, acc[iq][d], c_new);
            }
        }
    }

#pragma unroll
    for (int iq = 0; iq < QB; ++iq) {
        if (unit_ok && q0 + iq < Tq) {
            T* o = out + (((int64_t)b * Hq + h) * Tq + q0 + iq) * D;
            using C = Chunk<T, DL>;
            const float* st = slot + (iq * (NL + 2)) * STRIDE;
            const float Lq = st[STRIDE];
#pragma unroll
            for (int j = 0; j < NCHUNK; ++j) {
                C c;
#pragma unroll
                for (int d = 0; d < DL; ++d) c.v[d] = Cvt<T>::down(div_canon(st[(2 + j * DL + d) * STRIDE], Lq));
                reinterpret_cast<C*>(o)[r + OCT * j] = c;
            }
        }
    }
}

int check_common(const char* op, const void* q, const void* k, const void* v, const void* out, int64_t B,
                 int64_t Hq, int64_t Hkv, int64_t Tq, int64_t L, int64_t D, const KvLayout& lay, int split,
                 int dtype) {
    if (!dtype_ok(dtype)) return fail(BI_ERR_UNSUPPORTED, "%s: dtype %d", op, dtype);
    if (B < 0 || Hq <= 0 || Hkv <= 0 || Tq <= 0 || L <= 0 || D <= 0 || split <= 0)
        return fail(BI_ERR_BAD_ARG, "%s: bad sizes B=%lld Hq=%lld Hkv=%lld Tq=%lld L=%lld D=%lld split=%d", op,
                    (long long)B, (long long)Hq, (long long)Hkv, (long long)Tq, (long long)L, (long long)D, split);
    if (Hq % Hkv != 0) return fail(BI_ERR_UNSUPPORTED, "%s: Hq=%lld not a multiple of Hkv=%lld", op, (long long)Hq, (long long)Hkv);
    if (D != 32 && D != 64 && D != 128 && D != 256)
        return fail(BI_ERR_UNSUPPORTED, "%s: head_dim %lld (supported: 32, 64, 128, 256)", op, (long long)D);
    if (B == 0) return BI_OK;
    if (!q || !k || !v || !out) return fail(BI_ERR_BAD_ARG, "%s: null pointer", op);
    const size_t cb = (size_t)(D / 32) * dtype_size(dtype);  // bytes of one chunk load
    const size_t al = cb > 16 ? 16 : cb;
    if (!aligned(q, al) || !aligned(k, al) || !aligned(v, al) || !aligned(out, al))
        return fail(BI_ERR_MISALIGNED, "%s: pointers must be %zu-byte aligned", op, al);
    const int64_t se = (int64_t)(al / dtype_size(dtype));
    if (se > 1 && (lay.sb % se || lay.sh % se || lay.sl % se))
        return fail(BI_ERR_MISALIGNED, "%s: k/v strides must be multiples of %lld elements", op, (long long)se);
    if (lay.sl < D) return fail(BI_ERR_BAD_ARG, "%s: key stride %lld < head_dim", op, (long long)lay.sl);
    if (L > (1 << 30) || B * Hq * Tq > (1LL << 40))
        return fail(BI_ERR_UNSUPPORTED, "%s: problem too large", op);
    return BI_OK;
}

template <typename T, int DL>
int launch_decode(const void* q, const void* k, const void* v, void* out, const int32_t* kv_lens, float* ws,
                  int64_t B, int64_t Hq, int64_t Hkv, int64_t L, const KvLayout& lay, float scale, int split,
                  cudaStream_t st, const PushSink* sink = nullptr) {
    constexpr int D = 32 * DL;
    const int G = (int)(Hq / Hkv);
    const int nsplit = (int)((L + split - 1) / split);
    const int64_t BH = B * Hq;
    float* pm = ws;
    float* pl = pm + BH * nsplit;
    float* pacc = pl + BH * nsplit;
    // Query heads of a kv head share each K/V row load, up to four per unit.
    // How they are grouped is a launch choice; a head's arithmetic is the same alone or grouped.
    // With few units the GPU is short of independent key streams, so the heads of a kv head stop
    // sharing a stream (the rows are then re-read through L2) until there are enough.
    int GU = (G >= 4 && DL < 8) ? 4 : (G >= 2 ? 2 : 1);
    const int64_t sms = sm_count();
    const int64_t enough = sms * 16;
    while (GU > 1 && B * Hkv * ((G + GU - 1) / GU) * nsplit < enough) GU >>= 1;
    const int nchunk = (G + GU - 1) / GU;
    const int64_t units = B * Hkv * nchunk * nsplit;
    const int warps = 4;
    const int64_t blocks = (units + warps * OCT_PER_WARP - 1) / (warps * OCT_PER_WARP);
    if (blocks > 0x7fffffffLL) return fail(BI_ERR_UNSUPPORTED, "bi_attn_decode: grid too large");
    const T* qp = static_cast<const T*>(q);
    const T* kp = static_cast<const T*>(k);
    const T* vp = static_cast<const T*>(v);
    dim3 grid((unsigned)blocks), block(32 * warps);
    // Streamed kernel when every K/V row starts on a 16-byte boundary (cp.async granularity);
    // otherwise the register-prefetch kernel. Same arithmetic, the choice depends on layout only.
    if constexpr (DL < 8) {
        const int64_t per16 = 16 / (int64_t)sizeof(T);
        const bool rows16 = aligned(k, 16) && aligned(v, 16) && lay.sb % per16 == 0 && lay.sh % per16 == 0 &&
                            lay.sl % per16 == 0 && (32 * DL * sizeof(T)) % 16 == 0;
        if constexpr (DL == 4 && sizeof(T) == 2) {
            // 16-bit K/V, head_dim 128: a key per lane (decode_keylane_kernel). Heads of a kv head share the warp in
            // chunks of four (two, one); with few work items every head gets a warp of its own instead.
            if (rows16 && (BH * nsplit) % 2 == 0) {
                int nh = G >= 3 ? 4 : (G == 2 ? 2 : 1);
                if (nh > 1 && B * Hkv * ((G + nh - 1) / nh) * nsplit < sms * 4) nh = 1;
                const int nck = (G + nh - 1) / nh;
                const int64_t items = B * Hkv * nck * nsplit;
                const int nw = items >= 2 * sms * KL_WARPS ? KL_WARPS : KL_WARPS - 1;
                const int64_t ctas = std::min<int64_t>(sms, (items + nw - 1) / nw);
#define BI_KL_LAUNCH(NHV, NWV)                                                                                         \
    do {                                                                                                                \
        auto kern = decode_keylane_kernel<T, NHV, (NWV)>;                                                                \
        static bool attr_set[64] = {false};                                                                             \
        int dev_ = 0;                                                                                                   \
        cudaGetDevice(&dev_);                                                                                           \
        if (dev_ < 0 || dev_ >= 64) dev_ = 0;                                                                           \
        if (!attr_set[dev_]) {                                                                                          \
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (NWV) * KLCfg::WARP_BYTES); \
            if (e != cudaSuccess) return fail(BI_ERR_CUDA, "bi_attn_decode smem attr: %s", cudaGetErrorString(e));      \
            attr_set[dev_] = true;                                                                                      \
        }                                                                                                               \
        launch_overlapped(kern, dim3((unsigned)ctas), dim3(32 * (NWV)), (size_t)((NWV) * KLCfg::WARP_BYTES), st, qp, kp, vp, kv_lens, pm, pl, pacc, \
                          (int)B, (int)Hq, (int)Hkv, (int)L, lay, scale, split, nsplit, nck);                           \
    } while (0)
#define BI_KL_LAUNCH_NH(NWV) do { if (nh == 4) BI_KL_LAUNCH(4, NWV); else if (nh == 2) BI_KL_LAUNCH(2, NWV); else BI_KL_LAUNCH(1, NWV); } while (0)
                if (nw == KL_WARPS) BI_KL_LAUNCH_NH(KL_WARPS); else BI_KL_LAUNCH_NH(KL_WARPS - 1);
#undef BI_KL_LAUNCH_NH
#undef BI_KL_LAUNCH
                int rck = check_launch("bi_attn_decode (key per lane)");
                if (rck) return rck;
                const int64_t n2k = BH * D;
                return launch_decode_combine<T>(pm, pl, pacc, kv_lens, out, BH, (int)Hq, D, (int)L, split, nsplit, sink, st);
            }
        }
        if (lay.table != nullptr)
            return fail(BI_ERR_UNSUPPORTED, "bi_attn_decode_paged: needs 16-byte aligned rows and an even number of (sequence, head, split) partials");
        const int nchunk4 = (G + 3) / 4;
        const int64_t streams = B * Hkv * nchunk4 * nsplit;
        if (rows16 && streams < sms * 24) {
            // few streams: one warp per stream, its octets on different heads
            using CW = DecWCfg<T, DL>;
            // Warps per CTA: the streams are dealt out so that every SM gets the same number of warps (CTAs land
            // on SMs whole; with a fixed four warps per CTA, 1536 streams put 8 warps on some SMs and 12 on others
            // and the kernel ran as long as the 12): k CTAs per SM, ceil(streams / (148 k)) warps each. The kernel
            // is instantiated for CTAs of up to 4, 12 and 16 warps so that the register budget fits the count.
            constexpr int SMEM_CAP = 200 * 1024;
            constexpr int MAXW = (SMEM_CAP / CW::WARP_BYTES) < DECW_WARPS ? (SMEM_CAP / CW::WARP_BYTES) : DECW_WARPS;
            int wpc = 1;
            for (int k = 1; k <= 64; ++k) {
                wpc = (int)((streams + sms * k - 1) / (sms * k));
                if (wpc <= MAXW) break;
            }
            if (wpc > MAXW) wpc = MAXW;
            // Below nine warps per SM a warp runs alone on its scheduler most of the time and the 4-warp
            // instantiation (more registers, more loads in flight per warp) is the faster code: measured 55 us
            // against 64 us at 768 streams, 40 against 54 us at 32.
            if (wpc < 9) wpc = 4;
            const size_t smem_w = (size_t)wpc * CW::WARP_BYTES;
            const int64_t blocksw = (streams + wpc - 1) / wpc;
#define BI_DECW_LAUNCH(MW)                                                                                              \
    do {                                                                                                                \
        auto kern = decode_warp_stream_kernel<T, DL, MW>;                                                               \
        static bool attr_set[64] = {false}; /* per instantiation and device: the attribute is per device */            \
        int dev_ = 0;                                                                                                   \
        cudaGetDevice(&dev_);                                                                                           \
        if (dev_ < 0 || dev_ >= 64) dev_ = 0;                                                                           \
        if (!attr_set[dev_] && MW * CW::WARP_BYTES > 40 * 1024) {                                                       \
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, MW * CW::WARP_BYTES); \
            if (e != cudaSuccess) return fail(BI_ERR_CUDA, "bi_attn_decode smem attr: %s", cudaGetErrorString(e));      \
            attr_set[dev_] = true;                                                                                      \
        }                                                                                                               \
        launch_overlapped(kern, dim3((unsigned)blocksw), dim3(32 * wpc), smem_w, st, qp, kp, vp, kv_lens, pm, pl, pacc, (int)B, (int)Hq, (int)Hkv, \
                                                          (int)L, lay, scale, split, nsplit, nchunk4);                  \
    } while (0)
            if (wpc <= 4) BI_DECW_LAUNCH(4);
            else if (wpc <= 12) { if constexpr (MAXW >= 12) BI_DECW_LAUNCH(12); }
            else { if constexpr (MAXW >= 16) BI_DECW_LAUNCH(16); }
#undef BI_DECW_LAUNCH
            int rcw = check_launch("bi_attn_decode (warp per stream)");
            if (rcw) return rcw;
            const int64_t n2w = BH * D;
            return launch_decode_combine<T>(pm, pl, pacc, kv_lens, out, BH, (int)Hq, D, (int)L, split, nsplit, sink, st);
        }
        if (rows16) {
            using C = Dec2Cfg<T, DL>;
            const int64_t blocks2 = (units + DEC2_WARPS * OCT_PER_WARP - 1) / (DEC2_WARPS * OCT_PER_WARP);
#define BI_DECODE2_LAUNCH(GUV)                                                                                   \
    do {                                                                                                         \
        auto kern = decode_stream_kernel<T, DL, GUV>;                                                            \
        if (C::SMEM_BYTES > 40 * 1024) { /* static shared memory counts toward the 48 KB default too */          \
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES); \
            if (e != cudaSuccess) return fail(BI_ERR_CUDA, "bi_attn_decode smem attr: %s", cudaGetErrorString(e)); \
        }                                                                                                        \
        launch_overlapped(kern, dim3((unsigned)blocks2), dim3(32 * DEC2_WARPS), C::SMEM_BYTES, st, qp, kp, vp, kv_lens, pm, pl, pacc, (int)B, \
                                                                          (int)Hq, (int)Hkv, (int)L, lay, scale, split, nsplit, nchunk); \
    } while (0)
            if (GU == 4) BI_DECODE2_LAUNCH(4); else if (GU == 2) BI_DECODE2_LAUNCH(2); else BI_DECODE2_LAUNCH(1);
#undef BI_DECODE2_LAUNCH
            int rc2 = check_launch("bi_attn_decode (streamed)");
            if (rc2) return rc2;
            const int64_t n2s = BH * D;
            return launch_decode_combine<T>(pm, pl, pacc, kv_lens, out, BH, (int)Hq, D, (int)L, split, nsplit, sink, st);
        }
    }
    if (lay.table != nullptr)
        return fail(BI_ERR_UNSUPPORTED, "bi_attn_decode_paged: paged caches are read by the 16-bit head_dim-128 kernel only");
#define BI_DECODE_LAUNCH(GUV)                                                                              \
    launch_overlapped(decode_kernel<T, DL, GUV>, grid, block, 0, st, qp, kp, vp, kv_lens, pm, pl, pacc, (int)B, (int)Hq, \
                                                      (int)Hkv, (int)L, lay, scale, split, nsplit, nchunk)
    if (GU == 4) {
        if constexpr (DL < 8) BI_DECODE_LAUNCH(4);
    } else if (GU == 2) {
        BI_DECODE_LAUNCH(2);
    } else {
        BI_DECODE_LAUNCH(1);
    }
#undef BI_DECODE_LAUNCH
    int rc = check_launch("bi_attn_decode");
    if (rc) return rc;
    const int64_t n2 = BH * D;
    return launch_decode_combine<T>(pm, pl, pacc, kv_lens, out, BH, (int)Hq, D, (int)L, split, nsplit, sink, st);
}

template <typename T, int DL>
int launch_prefill(const void* q, const void* k, const void* v, void* out, int64_t B, int64_t Hq, int64_t Hkv,
                   int64_t Tq, int64_t L, const KvLayout& lay, float scale, int causal, int split, cudaStream_t st) {
    constexpr int QB = PrefillCfg<DL>::QB;
    const int64_t nblk = (Tq + QB - 1) / QB;
    const int64_t units = B * Hq * nblk;
    constexpr int warps = PREFILL_THREADS / 32;
    const int64_t blocks = (units + warps * OCT_PER_WARP - 1) / (warps * OCT_PER_WARP);
    if (blocks > 0x7fffffffLL) return fail(BI_ERR_UNSUPPORTED, "bi_attn_prefill: grid too large");
    const size_t smem = (size_t)QB * (NCHUNK * DL + 2) * PREFILL_THREADS * sizeof(float);
    auto kern = prefill_kernel<T, DL>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(BI_ERR_CUDA, "bi_attn_prefill smem attr: %s", cudaGetErrorString(e));
    }
    kern<<<(unsigned)blocks, PREFILL_THREADS, smem, st>>>(
        static_cast<const T*>(q), static_cast<const T*>(k), static_cast<const T*>(v), static_cast<T*>(out), (int)B,
        (int)Hq, (int)Hkv, (int)Tq, (int)L, lay, scale, causal, split);
    return check_launch("bi_attn_prefill");
}

}  // namespace
}  // namespace bi

#define BI_DISPATCH_T_DL(FN, ...)                                                        \
    do {                                                                                 \
        const int dl_ = (int)(D / 32);                                                   \
        if (dtype == BI_F32) {                                                           \
            if (dl_ == 1) return FN<float, 1>(__VA_ARGS__);                              \
            if (dl_ == 2) return FN<float, 2>(__VA_ARGS__);                              \
            if (dl_ == 4) return FN<float, 4>(__VA_ARGS__);                              \
            return FN<float, 8>(__VA_ARGS__);                                            \
        } else if (dtype == BI_F16) {                                                    \
            if (dl_ == 1) return FN<__half, 1>(__VA_ARGS__);                             \
            if (dl_ == 2) return FN<__half, 2>(__VA_ARGS__);                             \
            if (dl_ == 4) return FN<__half, 4>(__VA_ARGS__);                             \
            return FN<__half, 8>(__VA_ARGS__);                                           \
        } else {                                                                         \
            if (dl_ == 1) return FN<__nv_bfloat16, 1>(__VA_ARGS__);                      \
            if (dl_ == 2) return FN<__nv_bfloat16, 2>(__VA_ARGS__);                      \
            if (dl_ == 4) return FN<__nv_bfloat16, 4>(__VA_ARGS__);                      \
            return FN<__nv_bfloat16, 8>(__VA_ARGS__);                                    \
        }                                                                                \
    } while (0)

extern "C" size_t bi_attn_decode_workspace_bytes(int64_t B, int64_t Hq, int64_t L, int64_t D, int split_size) {
    if (B <= 0 || Hq <= 0 || L <= 0 || D <= 0 || split_size <= 0) return 0;
    const int64_t nsplit = (L + split_size - 1) / split_size;
    return (size_t)(B * Hq * nsplit * (D + 2)) * sizeof(float);
}

extern "C" int bi_attn_decode(const void* q, const void* k, const void* v, void* out, const int32_t* kv_lens,
                              void* workspace, size_t workspace_bytes, int64_t B, int64_t Hq, int64_t Hkv, int64_t L,
                              int64_t D, int64_t kv_sb, int64_t kv_sh, int64_t kv_sl, float scale, int split_size,
                              int dtype, void* stream) {
    using namespace bi;
    KvLayout lay{kv_sb, kv_sh, kv_sl};
    int rc = check_common("bi_attn_decode", q, k, v, out, B, Hq, Hkv, 1, L, D, lay, split_size, dtype);
    if (rc || B == 0) return rc;
    const size_t need = bi_attn_decode_workspace_bytes(B, Hq, L, D, split_size);
    if (!workspace || workspace_bytes < need)
        return fail(BI_ERR_WORKSPACE, "bi_attn_decode: workspace %zu bytes, need %zu", workspace_bytes, need);
    if (!aligned(workspace, 16)) return fail(BI_ERR_MISALIGNED, "bi_attn_decode: workspace must be 16-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    float* ws = static_cast<float*>(workspace);
    BI_DISPATCH_T_DL(launch_decode, q, k, v, out, kv_lens, ws, B, Hq, Hkv, L, lay, scale, split_size, st);
}

// bi_attn_decode whose merged output is pushed, as this rank's head slice, into every rank's gathered activation
// [B, world * Hq * D] (the split merge is the gather kernel; see peer_push.cuh for the handshake).
extern "C" int bi_attn_decode_push(const void* q, const void* k, const void* v, const int32_t* kv_lens, void* workspace,
                                   size_t workspace_bytes, int64_t B, int64_t Hq, int64_t Hkv, int64_t L, int64_t D,
                                   int64_t kv_sb, int64_t kv_sh, int64_t kv_sl, float scale, int split_size, int dtype,
                                   void* stream, void* const* dst, void* const* peer_flags, uint32_t* counters, int rank,
                                   int world, int wait, int32_t* status) {
    using namespace bi;
    KvLayout lay{kv_sb, kv_sh, kv_sl};
    PushSink sink;
    int rc = make_sink("bi_attn_decode_push", dst, peer_flags, counters, rank, world, wait, status, dtype_ok(dtype) ? dtype_size(dtype) : 1, &sink);
    if (rc) return rc;
    rc = check_common("bi_attn_decode_push", q, k, v, dst[rank], B, Hq, Hkv, 1, L, D, lay, split_size, dtype);
    if (rc || B == 0) return rc;
    const size_t need = bi_attn_decode_workspace_bytes(B, Hq, L, D, split_size);
    if (!workspace || workspace_bytes < need)
        return fail(BI_ERR_WORKSPACE, "bi_attn_decode_push: workspace %zu bytes, need %zu", workspace_bytes, need);
    if (!aligned(workspace, 16)) return fail(BI_ERR_MISALIGNED, "bi_attn_decode_push: workspace must be 16-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    float* ws = static_cast<float*>(workspace);
    const PushSink* sp = &sink;
    void* out = nullptr;
    BI_DISPATCH_T_DL(launch_decode, q, k, v, out, kv_lens, ws, B, Hq, Hkv, L, lay, scale, split_size, st, sp);
}

extern "C" int bi_attn_prefill(const void* q, const void* k, const void* v, void* out, int64_t B, int64_t Hq,
                               int64_t Hkv, int64_t Tq, int64_t L, int64_t D, int64_t kv_sb, int64_t kv_sh,
                               int64_t kv_sl, float scale, int causal, int split_size, int dtype, void* stream) {
    using namespace bi;
    KvLayout lay{kv_sb, kv_sh, kv_sl};
    int rc = check_common("bi_attn_prefill", q, k, v, out, B, Hq, Hkv, Tq, L, D, lay, split_size, dtype);
    if (rc || B == 0) return rc;
    if (causal && Tq > L) return fail(BI_ERR_BAD_ARG, "bi_attn_prefill: causal needs Tq <= L (Tq=%lld L=%lld)", (long long)Tq, (long long)L);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    BI_DISPATCH_T_DL(launch_prefill, q, k, v, out, B, Hq, Hkv, Tq, L, lay, scale, causal, split_size, st);
}

extern "C" int bi_attn_decode_paged(const void* q, const void* k_pages, const void* v_pages, void* out, const int32_t* kv_lens,
                                    const int32_t* block_table, void* workspace, size_t workspace_bytes, int64_t B, int64_t Hq,
                                    int64_t Hkv, int64_t max_pages, int64_t page_size, int64_t D, int64_t pg_sp, int64_t pg_sh,
                                    int64_t pg_sl, int64_t table_stride, float scale, int split_size, int dtype, void* stream) {
    using namespace bi;
    if (!block_table || !kv_lens) return fail(BI_ERR_BAD_ARG, "bi_attn_decode_paged: block_table and kv_lens are required");
    if (page_size <= 0 || page_size % 32 != 0 || split_size % page_size != 0 && page_size % split_size != 0 || max_pages <= 0 ||
        table_stride < max_pages)
        return fail(BI_ERR_UNSUPPORTED, "bi_attn_decode_paged: page_size %lld must be a multiple of 32 that divides, or is a multiple of, the split size %d",
                    (long long)page_size, split_size);
    if (dtype == BI_F32 || D != 128) return fail(BI_ERR_UNSUPPORTED, "bi_attn_decode_paged: 16-bit caches with head_dim 128 only");
    const int64_t L = max_pages * page_size;
    KvLayout lay{pg_sp, pg_sh, pg_sl, block_table, (int)page_size, (int)table_stride};
    int rc = check_common("bi_attn_decode_paged", q, k_pages, v_pages, out, B, Hq, Hkv, 1, L, D, lay, split_size, dtype);
    if (rc || B == 0) return rc;
    const size_t need = bi_attn_decode_workspace_bytes(B, Hq, L, D, split_size);
    if (!workspace || workspace_bytes < need)
        return fail(BI_ERR_WORKSPACE, "bi_attn_decode_paged: workspace %zu bytes, need %zu", workspace_bytes, need);
    if (!aligned(workspace, 16)) return fail(BI_ERR_MISALIGNED, "bi_attn_decode_paged: workspace must be 16-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    float* ws = static_cast<float*>(workspace);
    if (dtype == BI_F16) return launch_decode<__half, 4>(q, k_pages, v_pages, out, kv_lens, ws, B, Hq, Hkv, L, lay, scale, split_size, st);
    return launch_decode<__nv_bfloat16, 4>(q, k_pages, v_pages, out, kv_lens, ws, B, Hq, Hkv, L, lay, scale, split_size, st);
}
