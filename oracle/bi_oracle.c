/*
 * CPU oracle for the batch-invariant hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * Nothing in the product imports, links or executes this file: it exists so that
 * tests/, the smoke check and the benchmark's CPU-baseline leg can compare the CUDA
 * kernels with an independent plain-C statement of the same arithmetic.
 *
 * PARITY UNPINNED: the reference (waseemh/mlx-batch-invariant) ships no numeric golden
 * vectors, and its kernels are Metal source that needs MLX and an Apple GPU, so nothing
 * here could be checked against reference outputs. What this file restates is the
 * reference's *algorithm*, function by function:
 *
 *   orc_rms_norm        mlx_batch_invariant/kernels/rmsnorm.py:19-47   (256 threads, stride-256
 *                       fma partials, shared-memory tree 128..1, rsqrt, two multiplies)
 *   orc_attn_decode     mlx_batch_invariant/kernels/attention.py:47-75  (per-key update, 32 lanes,
 *                       xor-butterfly 16,8,4,2,1), :87-147 (decode partials), :149-171 (combine)
 *   orc_attn_prefill    mlx_batch_invariant/kernels/attention.py:173-254 (QB queries per simdgroup,
 *                       per-query causal predicate, in-register merge :77-85)
 *   orc_matmul_f32      mlx_batch_invariant/kernels/matmul.py:1-15,166-177,226-234 (K groups of 256,
 *                       group partial from exact zero, left fold of fp32 partials, one rounding)
 *   orc_combine         mlx_batch_invariant/kernels/matmul.py:226-234
 *   orc_dequant         mlx_batch_invariant/kernels/quantized.py:44-67 (fma(float(code), scale, bias)
 *                       in fp32, one rounding to the staged dtype, codes packed low to high)
 *
 * Two things cannot be taken from the reference and are stated here instead:
 *   - exp and 1/sqrt: Metal's precise::exp / precise::rsqrt are not available off an Apple GPU.
 *     orc_expf is a fixed fma-only sequence (<= 1.07 ulp on [-86.5, 0], exp(0) == 1, exactly 0
 *     below -86.5); rsqrt is a correctly rounded sqrt followed by a correctly rounded divide.
 *   - the inner product of one K group on tensor cores (simdgroup MMA there, tcgen05 here) has a
 *     hardware-defined internal order. orc_matmul_f32 is therefore bit-exact only for the
 *     CUDA-core path (one fp32 fma per k, ascending); the tensor-core path is checked against the
 *     fp64 semantic reference by tolerance and against itself bit for bit.
 *
 * Element types: fp32, and bf16 / fp16 carried as uint16 bit patterns.
 * Build: gcc -O2 -ffp-contract=off -fopenmp -fPIC -shared (see oracle/build.py); the OpenMP loops run
 * over independent output elements, so thread count never changes a bit. fmaf() must be the
 * correctly rounded one (glibc's is, with or without hardware FMA).
 */
#include <math.h>
#include <stdint.h>
#include <string.h>
#include <stdlib.h>

enum { ORC_F32 = 0, ORC_F16 = 1, ORC_BF16 = 2 };

/* ---- scalar helpers ---------------------------------------------------------------- */
static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

static inline float bf16_up(uint16_t h) { return u2f((uint32_t)h << 16); }
static inline uint16_t bf16_down(float f) { /* round to nearest even */
    uint32_t u = f2u(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u); /* quiet NaN */
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;
    return (uint16_t)(u >> 16);
}
static inline float f16_up(uint16_t h) { _Float16 x; memcpy(&x, &h, 2); return (float)x; }
static inline uint16_t f16_down(float f) { _Float16 x = (_Float16)f; uint16_t h; memcpy(&h, &x, 2); return h; }

static inline float load_el(const void* p, int64_t i, int dt) {
    if (dt == ORC_F32) return ((const float*)p)[i];
    if (dt == ORC_F16) return f16_up(((const uint16_t*)p)[i]);
    return bf16_up(((const uint16_t*)p)[i]);
}
static inline void store_el(void* p, int64_t i, int dt, float v) {
    if (dt == ORC_F32) ((float*)p)[i] = v;
    else if (dt == ORC_F16) ((uint16_t*)p)[i] = f16_down(v);
    else ((uint16_t*)p)[i] = bf16_down(v);
}

/* exp(x) for x <= 0: n = rint(x*log2e) by magic-number rounding; r = x - n*ln2 in two fma
 * steps; degree-6 polynomial by six fma steps; scale by 2^n on the exponent field. */
float orc_expf(float x) {
    const float MAGIC = 12582912.0f;
    float t = fmaf(x, 1.4426950408889634f, MAGIC);
    float nf = t - MAGIC;
    float r = fmaf(nf, -0.693145751953125f, x);
    r = fmaf(nf, -1.42860682030941723212e-6f, r);
    float p = 0.0013843559427186847f;
    p = fmaf(p, r, 0.008374235592782497f);
    p = fmaf(p, r, 0.041668009012937546f);
    p = fmaf(p, r, 0.16666430234909058f);
    p = fmaf(p, r, 0.4999999403953552f);
    p = fmaf(p, r, 1.0f);
    p = fmaf(p, r, 1.0f);
    int32_t n = (int32_t)f2u(t) - 0x4B400000;
    float res = u2f((uint32_t)((int32_t)f2u(p) + n * (1 << 23)));
    return (x < -86.5f) ? 0.0f : res;
}
void orc_expf_array(const float* x, float* y, int64_t n) { for (int64_t i = 0; i < n; ++i) y[i] = orc_expf(x[i]); }

static inline float orc_rsqrt(float v) { return 1.0f / sqrtf(v); }

/* ---- RMSNorm ------------------------------------------------------------------------ */
void orc_rms_norm(const void* x, const void* w, void* out, int64_t rows, int64_t D, float eps, int dt) {
    enum { TG = 256 };
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        float red[TG];
        const int64_t base = r * D;
        for (int t = 0; t < TG; ++t) {
            float ss = 0.0f;
            for (int64_t i = t; i < D; i += TG) { float v = load_el(x, base + i, dt); ss = fmaf(v, v, ss); }
            red[t] = ss;
        }
        for (int s = TG / 2; s > 0; s >>= 1)
            for (int t = 0; t < s; ++t) red[t] = red[t] + red[t + s];
        const float inv = orc_rsqrt(red[0] / (float)D + eps);
        for (int64_t i = 0; i < D; ++i) {
            float v = load_el(x, base + i, dt) * inv;
            float wi = w ? load_el(w, i, dt) : 1.0f;
            store_el(out, base + i, dt, v * wi);
        }
    }
}

/* LayerNorm in the manner of orc_rms_norm. The reference has no LayerNorm kernel (it names one as future work,
 * README.md:261-263); this states the order the CUDA kernel defines: stride-256 fp32 partial sums and the same tree
 * for the mean, then for the squared deviations; out = T((((x - mean) * inv) * w) + b), one rounding. */
void orc_layer_norm(const void* x, const void* w, const void* b, void* out, int64_t rows, int64_t D, float eps, int dt) {
    enum { TG = 256 };
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        float red[TG];
        const int64_t base = r * D;
        for (int t = 0; t < TG; ++t) {
            float s = 0.0f;
            for (int64_t i = t; i < D; i += TG) s = s + load_el(x, base + i, dt);
            red[t] = s;
        }
        for (int s = TG / 2; s > 0; s >>= 1)
            for (int t = 0; t < s; ++t) red[t] = red[t] + red[t + s];
        const float mean = red[0] / (float)D;
        for (int t = 0; t < TG; ++t) {
            float q = 0.0f;
            for (int64_t i = t; i < D; i += TG) { float d = load_el(x, base + i, dt) - mean; q = fmaf(d, d, q); }
            red[t] = q;
        }
        for (int s = TG / 2; s > 0; s >>= 1)
            for (int t = 0; t < s; ++t) red[t] = red[t] + red[t + s];
        const float inv = orc_rsqrt(red[0] / (float)D + eps);
        for (int64_t i = 0; i < D; ++i) {
            float y = (load_el(x, base + i, dt) - mean) * inv;
            if (w) y = y * load_el(w, i, dt);
            if (b) y = y + load_el(b, i, dt);
            store_el(out, base + i, dt, y);
        }
    }
}

/* ---- attention ---------------------------------------------------------------------- */
#define MAXD 256
typedef struct { float m, l, acc[MAXD]; } split_state;

/* simdgroup butterfly: returns what lane 0 holds after xor 16, 8, 4, 2, 1 */
static float butterfly32(const float* part_in) {
    float a[32], b[32];
    memcpy(a, part_in, sizeof(a));
    for (int off = 16; off >= 1; off >>= 1) {
        for (int l = 0; l < 32; ++l) b[l] = a[l] + a[l ^ off];
        memcpy(a, b, sizeof(a));
    }
    return a[0];
}

/* one key against one query row: the per-key update of attention.py:47-75 */
static void key_update(const float* qhat, const void* k, const void* v, int64_t krow, int D, int dt, split_state* st) {
    const int DL = D / 32;
    float part[32];
    for (int lane = 0; lane < 32; ++lane) {
        float p = 0.0f;
        for (int d = 0; d < DL; ++d) p = fmaf(qhat[lane * DL + d], load_el(k, krow + lane * DL + d, dt), p);
        part[lane] = p;
    }
    const float s = butterfly32(part);
    const float m_new = fmaxf(st->m, s);
    const float corr = orc_expf(st->m - m_new);
    const float p = orc_expf(s - m_new);
    st->l = fmaf(st->l, corr, p);
    for (int d = 0; d < D; ++d) st->acc[d] = fmaf(st->acc[d], corr, p * load_el(v, krow + d, dt));
    st->m = m_new;
}

static void merge(float* M, float* L, float* A, const split_state* st, int D) {
    const float M_new = fmaxf(*M, st->m);
    const float c_old = orc_expf(*M - M_new);
    const float c_new = orc_expf(st->m - M_new);
    *L = fmaf(*L, c_old, st->l * c_new);
    for (int d = 0; d < D; ++d) A[d] = fmaf(A[d], c_old, st->acc[d] * c_new);
    *M = M_new;
}

static void reset_state(split_state* st, int D) {
    st->m = -INFINITY; st->l = 0.0f;
    for (int d = 0; d < D; ++d) st->acc[d] = 0.0f;
}

/* One query row against keys [0, nkeys) of one kv head, fixed splits, left-to-right merge. */
static void attend_row(const void* q, int64_t qoff, const void* k, const void* v, int64_t kvoff, int64_t sl, int nkeys,
                       int D, float scale, int split, int dt, void* out, int64_t ooff) {
    float qhat[MAXD], A[MAXD];
    for (int d = 0; d < D; ++d) { qhat[d] = load_el(q, qoff + d, dt) * scale; A[d] = 0.0f; }
    float M = -INFINITY, L = 0.0f;
    split_state st;
    const int nsplit = (nkeys + split - 1) / split;
    for (int sp = 0; sp < nsplit; ++sp) {
        reset_state(&st, D);
        const int j1 = nkeys < (sp + 1) * split ? nkeys : (sp + 1) * split;
        for (int j = sp * split; j < j1; ++j) key_update(qhat, k, v, kvoff + (int64_t)j * sl, D, dt, &st);
        merge(&M, &L, A, &st, D);
    }
    for (int d = 0; d < D; ++d) store_el(out, ooff + d, dt, A[d] / L);
}

/* q, out: [B, Hq, 1, D]; k, v: [B, Hkv, L, D] contiguous; kv_lens: NULL or int32[B]. */
void orc_attn_decode(const void* q, const void* k, const void* v, void* out, const int32_t* kv_lens, int64_t B,
                     int64_t Hq, int64_t Hkv, int64_t L, int64_t D, float scale, int split, int dt) {
    const int64_t G = Hq / Hkv;
#pragma omp parallel for collapse(2) schedule(dynamic)
    for (int64_t b = 0; b < B; ++b)
        for (int64_t h = 0; h < Hq; ++h) {
            const int64_t hk = h / G;
            int nk = kv_lens ? kv_lens[b] : (int)L;
            if (nk > L) nk = (int)L;
            attend_row(q, (b * Hq + h) * D, k, v, (b * Hkv + hk) * L * D, D, nk, (int)D, scale, split, dt, out,
                       (b * Hq + h) * D);
        }
}

/* q, out: [B, Hq, Tq, D]; causal queries are right-aligned to the end of the keys. */
void orc_attn_prefill(const void* q, const void* k, const void* v, void* out, int64_t B, int64_t Hq, int64_t Hkv,
                      int64_t Tq, int64_t L, int64_t D, float scale, int causal, int split, int dt) {
    const int64_t G = Hq / Hkv;
#pragma omp parallel for collapse(3) schedule(dynamic, 8)
    for (int64_t b = 0; b < B; ++b)
        for (int64_t h = 0; h < Hq; ++h)
            for (int64_t qi = 0; qi < Tq; ++qi) {
                const int nk = causal ? (int)(L - Tq + qi + 1) : (int)L;
                const int64_t o = ((b * Hq + h) * Tq + qi) * D;
                attend_row(q, o, k, v, (b * Hkv + h / G) * L * D, D, nk, (int)D, scale, split, dt, out, o);
            }
}

/* ---- matmul ------------------------------------------------------------------------- */
/* out[M,N] = a[M,K] @ b[K,N] with element strides; group partial by one fma per k. */
void orc_matmul_f32order(const void* a, const void* b, void* out, int64_t M, int64_t N, int64_t K, int64_t a_sm,
                         int64_t a_sk, int64_t b_sk, int64_t b_sn, int dt) {
    const int64_t GK = 256;
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t m = 0; m < M; ++m)
        for (int64_t n = 0; n < N; ++n) {
            float total = 0.0f;
            for (int64_t k0 = 0; k0 < K; k0 += GK) {
                const int64_t k1 = k0 + GK < K ? k0 + GK : K;
                float acc = 0.0f;
                for (int64_t kk = k0; kk < k1; ++kk)
                    acc = fmaf(load_el(a, m * a_sm + kk * a_sk, dt), load_el(b, kk * b_sk + n * b_sn, dt), acc);
                total = total + acc;
            }
            store_el(out, m * N + n, dt, total);
        }
}

/* part: [G, MN] fp32 -> out[MN] in dt */
void orc_combine(const float* part, void* out, int64_t G, int64_t MN, int dt) {
    for (int64_t i = 0; i < MN; ++i) {
        float total = 0.0f;
        for (int64_t g = 0; g < G; ++g) total = total + part[g * MN + i];
        store_el(out, i, dt, total);
    }
}

/* Affine dequantization to dt: w[N, K*bits/32] uint32, scales/biases [N, K/gs] in dt -> wd[N, K] in dt. */
void orc_dequant(const uint32_t* w, const void* scales, const void* biases, void* wd, int64_t N, int64_t K, int gs,
                 int bits, int dt) {
    const int per = 32 / bits;
    const uint32_t mask = (1u << bits) - 1u;
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n)
        for (int64_t k = 0; k < K; ++k) {
            const uint32_t word = w[n * (K / per) + k / per];
            const uint32_t code = (word >> ((k % per) * bits)) & mask;
            const float s = load_el(scales, n * (K / gs) + k / gs, dt);
            const float bb = load_el(biases, n * (K / gs) + k / gs, dt);
            store_el(wd, n * K + k, dt, fmaf((float)code, s, bb));
        }
}

/* round-trip helpers for the Python side */
void orc_round_array(const float* x, void* y, int64_t n, int dt) { for (int64_t i = 0; i < n; ++i) store_el(y, i, dt, x[i]); }
void orc_up_array(const void* x, float* y, int64_t n, int dt) { for (int64_t i = 0; i < n; ++i) y[i] = load_el(x, i, dt); }

/* Worker threads of the OpenMP loops above (a launcher may have pinned OMP_NUM_THREADS to 1 in the environment;
 * the timed CPU baseline wants every host core). The thread count never changes a bit of any result. */
#ifdef _OPENMP
#include <omp.h>
int orc_set_threads(int n) { if (n > 0) omp_set_num_threads(n); return omp_get_max_threads(); }
#else
int orc_set_threads(int n) { (void)n; return 1; }
#endif
