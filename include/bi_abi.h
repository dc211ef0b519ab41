/*
 * C ABI of the B200 batch-invariant kernel library (libbi_b200.so).
 *
 * Every entry point is a plain C function over raw device pointers, sizes and
 * element strides. The library owns no device memory (documented exceptions:
 * bi_attn_decode_static's built-in array, and bi_peer_alloc, which exists to
 * allocate): inputs, outputs and any scratch ("workspace") are
 * allocated by the caller; the matching *_workspace_bytes() call says how much
 * scratch an op needs. Launches go to
 * the caller's stream and never synchronise. The return value is a bi_status;
 * bi_last_error() gives a thread-local message for the last non-zero status.
 * Nothing throws or aborts across this boundary.
 *
 * The reference project has no C layer: its kernels are Metal source strings
 * handed to mx.fast.metal_kernel(...) with a grid, a threadgroup size and the
 * caller-declared output shapes (mlx_batch_invariant/kernels/matmul.py:257-263,
 * 290-297). Each function below replaces one such kernel call site; the
 * citation beside it names the reference wrapper whose launch it stands for.
 */
#ifndef BI_ABI_H_
#define BI_ABI_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    BI_OK = 0,
    BI_ERR_UNSUPPORTED = 1, /* shape / dtype / option has no kernel            */
    BI_ERR_BAD_ARG = 2,     /* null pointer, negative size, inconsistent dims  */
    BI_ERR_MISALIGNED = 3,  /* pointer or stride not aligned as the op needs   */
    BI_ERR_WORKSPACE = 4,   /* workspace missing or too small                  */
    BI_ERR_CUDA = 5,        /* a CUDA runtime / driver call failed             */
    BI_ERR_DEVICE_WAIT = 6  /* a bounded device-side wait ran out (see bi_read_device_status) */
} bi_status;

typedef enum { BI_F32 = 0, BI_F16 = 1, BI_BF16 = 2 } bi_dtype;

/* Library version, major*10000 + minor*100 + patch. */
int bi_version(void);

/* Message for the last non-zero status returned on this thread ("" if none). */
const char* bi_last_error(void);

/* Kernels this library has launched in this process so far (every launch of every entry point, counted on
 * the host when it is issued; a launch recorded into a CUDA graph counts once, when it is captured).
 * No counterpart in the reference; benchmarks use it to state how many of the library's kernels a step runs. */
unsigned long long bi_launch_count(void);

/*
 * Device status word. The tensor-core matmul kernels wait on shared-memory
 * barriers with an iteration limit; a wait that runs out stores a non-zero
 * code into *status (an int32 in device memory owned by the caller, zeroed by
 * the caller) and the kernel returns early instead of hanging. `status` may be
 * NULL (no reporting). bi_read_device_status copies the word to the host after
 * synchronising `stream` and returns BI_ERR_DEVICE_WAIT if it is non-zero.
 */
int bi_read_device_status(const int32_t* status, int32_t* host_value, void* stream);

/* ------------------------------------------------------------------------ *
 * RMSNorm: out[r, :] = T((x[r, :] * rsqrt(mean(x[r, :]^2) + eps)) * w)       *
 * replaces batch_invariant_rms_norm / bi_rms_norm                           *
 * (mlx_batch_invariant/kernels/rmsnorm.py:19-47, 64-79).                    *
 * x, out: [rows, D] contiguous; w: [D] or NULL (= ones).                    *
 * ------------------------------------------------------------------------ */
int bi_rms_norm(const void* x, const void* w, void* out, int64_t rows, int64_t D, float eps,
                int dtype, void* stream);

/* LayerNorm: out[r, :] = T((((x[r, :] - mean) * rsqrt(var + eps)) * w) + b), mean and variance of the row by
 * fixed-stride fp32 partials and the fixed tree of bi_rms_norm (two passes: sum, then squared deviations).
 * No kernel in the reference yet -- it lists a batch-invariant LayerNorm as future work (README.md:261-263); the
 * call it would replace is the framework's layer_norm. x, out: [rows, D] contiguous; w, b: [D] or NULL. */
int bi_layer_norm(const void* x, const void* w, const void* b, void* out, int64_t rows, int64_t D, float eps,
                  int dtype, void* stream);

/* ------------------------------------------------------------------------ *
 * Dense matmul: out[M, N] = a[M, K] @ b[K, N], K folded in 256-wide groups. *
 * replaces batch_invariant_matmul / launch_tiled / bi_matmul_* /            *
 * bi_matmul_combine (mlx_batch_invariant/kernels/matmul.py:226-234,         *
 * 279-340). Strides are in elements. out is [M, N] contiguous.              *
 * `path` picks the launch shape; AUTO chooses by M, N and K. Every choice   *
 * gives the same bits. The low byte is one of BI_MATMUL_AUTO / SPLIT (one   *
 * work unit per K group, fp32 partials in the workspace, a second kernel    *
 * folds them) / FUSED (one unit folds all groups of a tile in place) /      *
 * SPLIT_FOLD (split, but the CTA that finishes a tile last folds it: one    *
 * launch). Optional, ORed in:                                               *
 *   BI_MATMUL_WS_ZEROED      the first BI_MATMUL_COUNTER_BYTES of the       *
 *                            workspace are zero when the call starts; the   *
 *                            call leaves them zero (unless a device wait    *
 *                            ran out: zero them again then). The partials   *
 *                            follow that block. Lets AUTO use SPLIT_FOLD.   *
 *   BI_MATMUL_BATCH_TILE(n)  batch rows per tile: 16, 32, 64 or 128         *
 *   BI_QMM_STAGE_SMEM/_TMEM  bi_qmm only: stage the dequantized weight in   *
 *                            shared memory (tile body) or in tensor memory  *
 *                            (streaming; batch tiles of at most 64 rows)    *
 * ------------------------------------------------------------------------ */
enum { BI_MATMUL_AUTO = 0, BI_MATMUL_SPLIT = 1, BI_MATMUL_FUSED = 2, BI_MATMUL_SPLIT_FOLD = 3 };
#define BI_MATMUL_WS_ZEROED 0x100
#define BI_MATMUL_BATCH_TILE(n) ((n) << 16)
#define BI_QMM_STAGE_SMEM 0x1000000
#define BI_QMM_STAGE_TMEM 0x2000000
#define BI_MATMUL_COUNTER_BYTES 16384

size_t bi_matmul_workspace_bytes(int64_t M, int64_t N, int64_t K, int dtype);

int bi_matmul(const void* a, const void* b, void* out, void* workspace, size_t workspace_bytes,
              int64_t M, int64_t N, int64_t K, int64_t a_sm, int64_t a_sk, int64_t b_sk,
              int64_t b_sn, int dtype, int path, int32_t* status, void* stream);

/* bi_matmul with the bias of a linear layer added in the epilogue: out[m, n] = T(float(T(total)) + float(bias[n])),
 * bias: [N] in the output dtype (NULL = none). The bits of the reference's addmm with alpha = beta = 1
 * (mlx_batch_invariant/ops.py:54-62: the product is rounded to the output dtype, then c is added elementwise),
 * without the second pass over the output; the reference names this fusion as future work (README.md:261-263). */
int bi_matmul_bias(const void* a, const void* b, const void* bias, void* out, void* workspace, size_t workspace_bytes,
                   int64_t M, int64_t N, int64_t K, int64_t a_sm, int64_t a_sk, int64_t b_sk, int64_t b_sn,
                   int dtype, int path, int32_t* status, void* stream);

/* ------------------------------------------------------------------------ *
 * Affine quantized matmul: out[M, N] = x[M, K] @ dequant(w)[N, K]^T         *
 *   dequant(n, k) = T(fma(float(code(n, k)), float(scales[n, k/gs]),        *
 *                                           float(biases[n, k/gs])))        *
 * replaces batch_invariant_quantized_matmul / bi_quantized_matmul_*         *
 * (mlx_batch_invariant/kernels/quantized.py:33-67, 106-125).                *
 * x: [M, K] row stride x_sm (elements), unit k stride; w: uint32            *
 * [N, K*bits/32] contiguous, codes packed low to high; scales, biases:      *
 * [N, K/gs] contiguous in x's dtype; out: [M, N] contiguous, x's dtype.     *
 * ------------------------------------------------------------------------ */
size_t bi_qmm_workspace_bytes(int64_t M, int64_t N, int64_t K, int dtype);

int bi_qmm(const void* x, const uint32_t* w, const void* scales, const void* biases, void* out,
           void* workspace, size_t workspace_bytes, int64_t M, int64_t N, int64_t K, int64_t x_sm,
           int group_size, int bits, int dtype, int path, int32_t* status, void* stream);

/* ------------------------------------------------------------------------ *
 * Decode attention (one query per sequence).                                *
 * replaces batch_invariant_decode_attention / bi_attn_decode /              *
 * bi_attn_combine (mlx_batch_invariant/kernels/attention.py:87-171,         *
 * 326-365). q, out: [B, Hq, 1, D] contiguous. k, v: [B, Hkv, L, D] with     *
 * element strides (kv_sb, kv_sh, kv_sl) and unit stride along D.            *
 * kv_lens: optional int32[B] device array of per-sequence key counts        *
 * (<= L); NULL means every sequence has L keys.                             *
 * ------------------------------------------------------------------------ */
size_t bi_attn_decode_workspace_bytes(int64_t B, int64_t Hq, int64_t L, int64_t D, int split_size);

int bi_attn_decode(const void* q, const void* k, const void* v, void* out, const int32_t* kv_lens,
                   void* workspace, size_t workspace_bytes, int64_t B, int64_t Hq, int64_t Hkv,
                   int64_t L, int64_t D, int64_t kv_sb, int64_t kv_sh, int64_t kv_sl, float scale,
                   int split_size, int dtype, void* stream);

/* ------------------------------------------------------------------------ *
 * Decode attention without a caller workspace. No counterpart in the         *
 * reference: there the MLX runtime allocates every kernel output and         *
 * intermediate. Same inputs, outputs and arithmetic as bi_attn_decode; the   *
 * per-split partials live in an array built into the library                 *
 * (BI_ATTN_DECODE_STATIC_MAX_BYTES per GPU, held until the process exits),    *
 * so the call allocates nothing. Meant for hosts that cannot allocate on the  *
 * library's behalf: a plugin inside a runtime that exposes no allocator to C, *
 * or a server that has already reserved HBM for its own pool. Problems whose  *
 * partials (bi_attn_decode_workspace_bytes) exceed the limit return           *
 * BI_ERR_WORKSPACE. All calls on a device share the array: calls that may     *
 * overlap on the GPU race and must be ordered by the caller. The first call   *
 * on each device resolves the array's address; issue it at start-up, before   *
 * any stream capture on that device.                                          *
 * ------------------------------------------------------------------------ */
#define BI_ATTN_DECODE_STATIC_MAX_BYTES (8u << 20)

int bi_attn_decode_static(const void* q, const void* k, const void* v, void* out, const int32_t* kv_lens,
                          int64_t B, int64_t Hq, int64_t Hkv, int64_t L, int64_t D, int64_t kv_sb, int64_t kv_sh,
                          int64_t kv_sl, float scale, int split_size, int dtype, void* stream);

/* Decode attention over a PAGED cache: k_pages, v_pages are pools [pages, Hkv, page_size, D] (element strides
 * pg_sp, pg_sh, pg_sl; unit stride along D), block_table[b * table_stride + i] names the page that holds keys
 * [i * page_size, (i + 1) * page_size) of sequence b, kv_lens[b] its key count (<= max_pages * page_size).
 * page_size: a multiple of 32 that divides the split size (or a multiple of it). 16-bit dtypes, D = 128.
 * Same arithmetic as bi_attn_decode -- only where a key's row is found differs -- so the same bits as the same
 * keys laid out contiguously. The reference reads one contiguous cache (it lists paged caches as future work,
 * README.md:261-263); workspace as bi_attn_decode_workspace_bytes(B, Hq, max_pages * page_size, D, split_size). */
int bi_attn_decode_paged(const void* q, const void* k_pages, const void* v_pages, void* out, const int32_t* kv_lens,
                         const int32_t* block_table, void* workspace, size_t workspace_bytes, int64_t B, int64_t Hq,
                         int64_t Hkv, int64_t max_pages, int64_t page_size, int64_t D, int64_t pg_sp, int64_t pg_sh,
                         int64_t pg_sl, int64_t table_stride, float scale, int split_size, int dtype, void* stream);

/* ------------------------------------------------------------------------ *
 * Prefill attention (any number of queries, right-aligned to the cache end  *
 * when causal). replaces batch_invariant_prefill_attention /                *
 * bi_attn_prefill (mlx_batch_invariant/kernels/attention.py:173-254,        *
 * 368-390). q, out: [B, Hq, Tq, D] contiguous; k, v as for decode.          *
 * ------------------------------------------------------------------------ */
int bi_attn_prefill(const void* q, const void* k, const void* v, void* out, int64_t B, int64_t Hq,
                    int64_t Hkv, int64_t Tq, int64_t L, int64_t D, int64_t kv_sb, int64_t kv_sh,
                    int64_t kv_sl, float scale, int causal, int split_size, int dtype,
                    void* stream);

/* ------------------------------------------------------------------------ *
 * Decoder-runner glue. No counterpart in the reference (there mlx_lm's model *
 * code does this with framework ops). Elementwise, batch-invariant by         *
 * construction.                                                               *
 * bi_rope_append: qkv[B*T, (Hq+2*Hkv)*D] as the qkv projection wrote it;       *
 *   token (b, t) is at position pos0[0] + t (pos0: int64 on the device);       *
 *   q -> q_out[B, Hq, T, D] rotated with cos/sin tables fp32 [positions, D]    *
 *   (the two halves of a head share an angle); rotated k and plain v are       *
 *   written into the caches [*, Hkv, capacity, D] (element strides given).     *
 *   `capacity` bounds the position (cache length and rows of the tables): a    *
 *   token whose position falls outside writes nothing and stores               *
 *   0x30000 | position into *status (see bi_read_device_status).               *
 * bi_swiglu: out[M, F] = T(silu(gu[:, :F]) * gu[:, F:]) for gu[M, 2F].         *
 * bi_add_rms_norm: the residual add in front of a norm, in one launch:         *
 *   sum_out[r, :] = T(x[r, :] + delta[r, :])  (fp32 add, one rounding: the      *
 *   bits of an elementwise add of two T arrays), out = bi_rms_norm(sum_out).   *
 *   sum_out may be x (in-place residual stream); out aliases nothing.          *
 * ------------------------------------------------------------------------ */
int bi_rope_append(const void* qkv, const float* cos_table, const float* sin_table, const int64_t* pos0,
                   void* q_out, void* k_cache, void* v_cache, int64_t B, int64_t T, int64_t Hq, int64_t Hkv,
                   int64_t D, int64_t cache_sb, int64_t cache_sh, int64_t cache_sl, int64_t capacity,
                   int32_t* status, int dtype, void* stream);

int bi_swiglu(const void* gate_up, void* out, int64_t M, int64_t F, int dtype, void* stream);

int bi_add_rms_norm(const void* x, const void* delta, const void* w, void* sum_out, void* out, int64_t rows,
                    int64_t D, float eps, int dtype, void* stream);

/* ------------------------------------------------------------------------ *
 * Feature-slice all-gather over peer memory, for the sharded decoder runner.  *
 * No counterpart in the reference (single device). Rank r holds               *
 * local[rows, row_bytes]; after the call every rank's destination holds       *
 * [rows, world*row_bytes] with rank r's slice in columns                      *
 * [r*row_bytes, (r+1)*row_bytes). One launch per rank on its own GPU: plain    *
 * stores into every rank's destination through peer mappings, a system-wide    *
 * fence, then a flag hand-shake with a bounded wait (2 s; on expiry *status    *
 * gets 0x20000 | peer << 8 | epoch and the kernel returns). Only bytes move.   *
 *   dst[world], flags[world]: HOST arrays of device pointers, entry r = rank    *
 *     r's destination buffer / flag array (uint32[world]) as mapped in THIS      *
 *     process (own buffers directly, the others through bi_peer_open).           *
 *   counters: uint32[2] in local device memory, zero before the first call.      *
 *   wait: 1 = the kernel returns when every peer's slice has arrived; 0 = see     *
 *   "Fused wait" below.                                                          *
 *   Every rank must issue the same sequence of gathers, and rotate over at        *
 *   least three destination buffers (a peer can be one gather ahead).            *
 * bi_peer_alloc / bi_peer_free: zero-filled device memory that a CUDA IPC        *
 *   handle can name (cudaMalloc; the one place the library allocates, at the      *
 *   caller's explicit request). bi_peer_export: its 64-byte handle, to be sent    *
 *   to the other ranks' processes; bi_peer_open / bi_peer_close map and unmap     *
 *   a peer's buffer by handle.                                                   *
 * ------------------------------------------------------------------------ */
int bi_peer_alloc(void** ptr, size_t bytes);
int bi_peer_free(void* ptr);
int bi_peer_export(void* ptr, uint8_t handle[64]);
int bi_peer_open(const uint8_t handle[64], void** ptr);
int bi_peer_close(void* ptr);
int bi_push_gather(const void* local, void* const* dst, void* const* flags, uint32_t* counters, int64_t rows,
                   int64_t row_bytes, int rank, int world, int wait, int32_t* status, void* stream);

/* bi_push_gather with the SwiGLU gate computed on the way: gate_up is this rank's [rows, 2F] (gate columns, then
 * up columns); the [rows, F] result of bi_swiglu on it is stored directly into every rank's gathered [rows, world*F]
 * activation (same bits as bi_swiglu followed by bi_push_gather, one launch, no local copy). Same protocol state. */
int bi_push_gather_swiglu(const void* gate_up, void* const* dst, void* const* flags, uint32_t* counters, int64_t rows,
                          int64_t F, int dtype, int rank, int world, int wait, int32_t* status, void* stream);

/* Fused wait. With wait = 0 a push gather stores its slice, raises this rank's flag at every peer and returns
 * without waiting for theirs: the kernel that READS the gathered buffer waits instead, after it has started the
 * part of its work that does not depend on the buffer. The *_awaiting entry points are bi_matmul / bi_qmm /
 * bi_add_rms_norm with that wait in front of their first read of the activation (matmul: the weight tiles of the
 * whole ring are already streaming while the kernel waits; add_rms_norm: `delta` is the gathered buffer).
 *   flags: this rank's own flag array (the local one of the `flags` table given to the push);
 *   epoch: &counters[1] of the push (device memory: the epoch of the gather just issued on the same stream).
 * The wait is bounded (2 s); on expiry 0x20000 | peer << 8 | epoch lands in *status. flags == NULL: no wait.
 * Same bits as the plain entry points. No counterpart in the reference (single device). */
int bi_matmul_awaiting(const void* a, const void* b, void* out, void* workspace, size_t workspace_bytes,
                       int64_t M, int64_t N, int64_t K, int64_t a_sm, int64_t a_sk, int64_t b_sk, int64_t b_sn,
                       int dtype, int path, int32_t* status, void* stream, const uint32_t* flags,
                       const uint32_t* epoch, int rank, int world);
int bi_qmm_awaiting(const void* x, const uint32_t* w, const void* scales, const void* biases, void* out,
                    void* workspace, size_t workspace_bytes, int64_t M, int64_t N, int64_t K, int64_t x_sm,
                    int group_size, int bits, int dtype, int path, int32_t* status, void* stream,
                    const uint32_t* flags, const uint32_t* epoch, int rank, int world);
int bi_add_rms_norm_awaiting(const void* x, const void* delta, const void* w, void* sum_out, void* out, int64_t rows,
                             int64_t D, float eps, int dtype, void* stream, const uint32_t* flags,
                             const uint32_t* epoch, int rank, int world, int32_t* status);

/* Producer-side fusion: the kernel that finishes an op's output IS the gather. bi_matmul_push / bi_qmm_push are
 * bi_matmul / bi_qmm (tensor-core weights only; always the split launch shape, so the workspace must hold
 * ceil(K/256) * M * N * 4 bytes, + BI_MATMUL_COUNTER_BYTES with BI_MATMUL_WS_ZEROED) whose fold kernel stores
 * out[m, n] into column rank * N + n of every rank's [M, world * N] destination and ends with the push gather's
 * handshake; bi_attn_decode_push is bi_attn_decode whose split merge stores (b, h, d) into column
 * rank * Hq * D + h * D + d of every rank's [B, world * Hq * D] destination. dst / peer_flags / counters / wait /
 * status as in bi_push_gather (same protocol state, same epochs: the calls can be mixed with bi_push_gather on
 * one stream). await_flags / await_epoch (NULL: none): the activation is itself a gathered buffer nobody has
 * waited for yet, as in bi_matmul_awaiting. Same bits as the plain op followed by bi_push_gather. No counterpart
 * in the reference (single device). */
int bi_matmul_push(const void* a, const void* b, void* workspace, size_t workspace_bytes, int64_t M, int64_t N,
                   int64_t K, int64_t a_sm, int64_t a_sk, int64_t b_sk, int64_t b_sn, int dtype, int path,
                   int32_t* status, void* stream, const uint32_t* await_flags, const uint32_t* await_epoch,
                   void* const* dst, void* const* peer_flags, uint32_t* counters, int rank, int world, int wait);
int bi_qmm_push(const void* x, const uint32_t* w, const void* scales, const void* biases, void* workspace,
                size_t workspace_bytes, int64_t M, int64_t N, int64_t K, int64_t x_sm, int group_size, int bits,
                int dtype, int path, int32_t* status, void* stream, const uint32_t* await_flags,
                const uint32_t* await_epoch, void* const* dst, void* const* peer_flags, uint32_t* counters, int rank,
                int world, int wait);
int bi_attn_decode_push(const void* q, const void* k, const void* v, const int32_t* kv_lens, void* workspace,
                        size_t workspace_bytes, int64_t B, int64_t Hq, int64_t Hkv, int64_t L, int64_t D,
                        int64_t kv_sb, int64_t kv_sh, int64_t kv_sl, float scale, int split_size, int dtype,
                        void* stream, void* const* dst, void* const* peer_flags, uint32_t* counters, int rank,
                        int world, int wait, int32_t* status);

/* The qkv projection of a decoder with bi_rope_append folded into it: bi_matmul / bi_qmm (tensor-core weights only;
 * always the split launch shape: the workspace must hold ceil(K/256) * M * N * 4 bytes, + BI_MATMUL_COUNTER_BYTES
 * with BI_MATMUL_WS_ZEROED) whose fold kernel rounds the product [B*T, (Hq + 2*Hkv) * D] to the dtype and then does
 * what bi_rope_append does with it -- rotated q into q_out, rotated k and plain v into the caches at position
 * pos0[0] + t, positions outside `capacity` skipped with 0x30000 | position in *status. The product itself is never
 * stored. Same bits as bi_matmul / bi_qmm followed by bi_rope_append. No counterpart in the reference. */
int bi_matmul_rope(const void* a, const void* b, void* workspace, size_t workspace_bytes, int64_t M, int64_t N,
                   int64_t K, int64_t a_sm, int64_t a_sk, int64_t b_sk, int64_t b_sn, int dtype, int path,
                   int32_t* status, void* stream, const float* cos_table, const float* sin_table,
                   const int64_t* pos0, void* q_out, void* k_cache, void* v_cache, int64_t B, int64_t T, int64_t Hq,
                   int64_t Hkv, int64_t D, int64_t cache_sb, int64_t cache_sh, int64_t cache_sl, int64_t capacity);
int bi_qmm_rope(const void* x, const uint32_t* w, const void* scales, const void* biases, void* workspace,
                size_t workspace_bytes, int64_t M, int64_t N, int64_t K, int64_t x_sm, int group_size, int bits,
                int dtype, int path, int32_t* status, void* stream, const float* cos_table, const float* sin_table,
                const int64_t* pos0, void* q_out, void* k_cache, void* v_cache, int64_t B, int64_t T, int64_t Hq,
                int64_t Hkv, int64_t D, int64_t cache_sb, int64_t cache_sh, int64_t cache_sl, int64_t capacity);

#ifdef __cplusplus
}
#endif
#endif /* BI_ABI_H_ */
