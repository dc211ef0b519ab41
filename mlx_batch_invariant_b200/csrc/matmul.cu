// extern "C" entry points of the dense and quantized matmul: validation, the
// choice between the tensor-core and the CUDA-core path (a property of the
// weight, never of the batch) and between the split and fused launch shapes (a
// function of M that moves no rounding).
#include "bi_common.cuh"
#include "matmul_internal.cuh"

namespace bi {
namespace {

constexpr int64_t SPLIT_M_MAX = 64;             // up to here the CUDA-core path may split; the tensor-core path always may
constexpr int64_t SPLIT_PARTIAL_MAX = 80 << 20;  // beyond 64 rows: only while the fp32 partials stay L2-sized
constexpr int64_t FOLD_M_MAX = 0;               // AUTO never folds in the kernel: the fence / count / read-back chain of every unit measured slower than the second launch (M = 1: 16.4 us against 12.6 us)
constexpr size_t COUNTER_BYTES = BI_MATMUL_COUNTER_BYTES;

int64_t ngroups(int64_t K) { return (K + GROUP_K - 1) / GROUP_K; }

// AUTO launch shape for the tensor-core path. Fused needs enough (weight tile, batch tile) pairs to fill the
// GPU; cutting the batch into shorter tiles makes more of them at the price of re-reading the weight tile
// through L2 once per batch tile, which pays down to 32-row tiles (measured at N = K = 4096: M = 256 fused in
// 64-row tiles 19.7 us against 30.3 us split; M = 128 in 32-row tiles 17.4 against 17.9 us; M = 64 in 16-row
// tiles 14.8 against 14.5 us). Below that the K groups are spread over CTAs (split) while the fp32 partials
// stay L2-sized.
// Quantized weights at decode (the streaming variant, M <= 8) are bound by the dequantizers' instruction stream, so
// they want every SM: with fewer weight tiles than SMs they split (the partials of <= 8 rows are tiny) -- 4096 ->
// 14336 at M = 1: 26.4 us split over 148 CTAs against 27.5 us fused on 112.
TcShape tc_auto_shape(int64_t M, int64_t N, int64_t K, bool quant = false) {
    TcShape sh{false, 128, nullptr, TcShape::STAGE_AUTO, Await{nullptr, nullptr, 0, 0}, nullptr};
    const int64_t G = ngroups(K);
    const int64_t nt = (N + 127) / 128;
    if (quant && M <= 8 && G > 1 && nt < sm_count()) { sh.split = true; return sh; }
    const int64_t fill = (int64_t)sm_count() * 3 / 4;
    int bm_fill = 0;                               // tallest batch tile that still fills the GPU
    for (int bm = 128; bm >= 16; bm >>= 1)
        if (nt * ((M + bm - 1) / bm) >= fill) { bm_fill = bm; break; }
    if (G <= 1 || bm_fill >= 32) { sh.bm = bm_fill ? bm_fill : 16; return sh; }
    const bool partials_ok = M <= SPLIT_M_MAX || G * M * N * (int64_t)sizeof(float) <= SPLIT_PARTIAL_MAX;
    if (partials_ok) { sh.split = true; return sh; }
    sh.bm = bm_fill ? bm_fill : 16;
    return sh;
}
// AUTO launch shape for the CUDA-core path (reference rule: M <= 32 and more than one group).
bool simt_auto_split(int64_t M, int64_t K) { return ngroups(K) > 1 && M <= 32; }

// `path` as the ABI packs it -> kind, flags, forced batch tile, forced staging.
struct PathArg {
    int kind;       // BI_MATMUL_AUTO / SPLIT / FUSED / SPLIT_FOLD
    bool zeroed;    // BI_MATMUL_WS_ZEROED
    int bm;         // 0 = choose
    int stage;      // TcShape::STAGE_*
};
int parse_path(const char* op, int path, PathArg* pa) {
    pa->kind = path & 0xff;
    pa->zeroed = (path & BI_MATMUL_WS_ZEROED) != 0;
    pa->bm = (path >> 16) & 0xff;
    pa->stage = (path & BI_QMM_STAGE_SMEM) ? TcShape::STAGE_SMEM : ((path & BI_QMM_STAGE_TMEM) ? TcShape::STAGE_TMEM : TcShape::STAGE_AUTO);
    if (pa->kind > BI_MATMUL_SPLIT_FOLD) return fail(BI_ERR_BAD_ARG, "%s: unknown path %d", op, pa->kind);
    if (pa->bm != 0 && pa->bm != 16 && pa->bm != 32 && pa->bm != 64 && pa->bm != 128)
        return fail(BI_ERR_BAD_ARG, "%s: batch tile %d (16, 32, 64 or 128)", op, pa->bm);
    if (pa->kind == BI_MATMUL_SPLIT_FOLD && !pa->zeroed)
        return fail(BI_ERR_BAD_ARG, "%s: BI_MATMUL_SPLIT_FOLD needs BI_MATMUL_WS_ZEROED (a zeroed counter block)", op);
    return BI_OK;
}

// Resolve the launch shape of a tensor-core call and lay out the workspace: [counter block, if the caller says
// it keeps one][fp32 partials].
int tc_shape(const char* op, const PathArg& pa, void* ws, size_t ws_bytes, int64_t M, int64_t N, int64_t K,
             TcShape* sh, float** part, bool quant = false) {
    *sh = tc_auto_shape(M, N, K, quant);
    if (pa.kind == BI_MATMUL_SPLIT || pa.kind == BI_MATMUL_SPLIT_FOLD) { sh->split = true; sh->bm = 128; }
    if (pa.kind == BI_MATMUL_FUSED && sh->split) {
        sh->split = false;
        sh->bm = 128;
        const int64_t nt = (N + 127) / 128, fill = (int64_t)sm_count() * 3 / 4;
        while (sh->bm > 16 && nt * ((M + sh->bm - 1) / sh->bm) < fill) sh->bm >>= 1;
    }
    if (pa.bm) sh->bm = pa.bm;
    sh->stage = pa.stage;
    const int64_t tiles = ((N + 127) / 128) * ((M + sh->bm - 1) / sh->bm);
    const bool fold = sh->split && pa.zeroed && tiles * (int64_t)sizeof(unsigned) <= (int64_t)COUNTER_BYTES &&
                      (pa.kind == BI_MATMUL_SPLIT_FOLD || (pa.kind == BI_MATMUL_AUTO && M <= FOLD_M_MAX));
    if (pa.kind == BI_MATMUL_SPLIT_FOLD && !fold)
        return fail(BI_ERR_UNSUPPORTED, "%s: %lld tiles exceed the counter block", op, (long long)tiles);
    const size_t head = pa.zeroed ? COUNTER_BYTES : 0;
    const size_t need = sh->split ? head + (size_t)ngroups(K) * (size_t)M * (size_t)N * sizeof(float) : 0;
    if (sh->split) {
        if (!ws || ws_bytes < need) return fail(BI_ERR_WORKSPACE, "%s: split path needs %zu workspace bytes, got %zu", op, need, ws_bytes);
        if (!aligned(ws, 16)) return fail(BI_ERR_MISALIGNED, "%s: workspace must be 16-byte aligned", op);
    }
    sh->counters = fold ? static_cast<unsigned*>(ws) : nullptr;
    *part = sh->split ? reinterpret_cast<float*>(static_cast<char*>(ws) + head) : nullptr;
    return BI_OK;
}

int simt_shape(const char* op, const PathArg& pa, void* ws, size_t ws_bytes, int64_t M, int64_t N, int64_t K, bool* split,
               float** part) {
    *split = pa.kind == BI_MATMUL_AUTO ? simt_auto_split(M, K) : (pa.kind != BI_MATMUL_FUSED);
    const size_t head = pa.zeroed ? COUNTER_BYTES : 0;
    const size_t need = head + (size_t)ngroups(K) * (size_t)M * (size_t)N * sizeof(float);
    *part = nullptr;
    if (*split && pa.kind == BI_MATMUL_AUTO && (!ws || ws_bytes < need)) *split = false;   // AUTO: fold in place instead
    if (!*split) return BI_OK;
    if (!ws || ws_bytes < need) return fail(BI_ERR_WORKSPACE, "%s: split path needs %zu workspace bytes, got %zu", op, need, ws_bytes);
    if (!aligned(ws, 16)) return fail(BI_ERR_MISALIGNED, "%s: workspace must be 16-byte aligned", op);
    *part = reinterpret_cast<float*>(static_cast<char*>(ws) + head);
    return BI_OK;
}

}  // namespace
}  // namespace bi

extern "C" size_t bi_matmul_workspace_bytes(int64_t M, int64_t N, int64_t K, int dtype) {
    using namespace bi;
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    // Enough for the shape AUTO picks, with or without a counter block in front; a forced BI_MATMUL_SPLIT always
    // needs ceil(K/256) * M * N * 4 bytes (+ BI_MATMUL_COUNTER_BYTES with BI_MATMUL_WS_ZEROED). 16-bit weights follow
    // the tensor-core rule (a 16-bit weight that has to take the CUDA-core path folds in place under AUTO when the
    // workspace is too small for its split); fp32 follows the CUDA-core rule.
    if (ngroups(K) <= 1) return 0;
    const bool split = dtype == BI_F32 ? simt_auto_split(M, K) : tc_auto_shape(M, N, K).split;
    if (!split) return 0;
    return COUNTER_BYTES + (size_t)ngroups(K) * (size_t)M * (size_t)N * sizeof(float);
}

extern "C" size_t bi_qmm_workspace_bytes(int64_t M, int64_t N, int64_t K, int dtype) {
    using namespace bi;
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    if (dtype == BI_F32 || ngroups(K) <= 1) return bi_matmul_workspace_bytes(M, N, K, dtype);
    if (!tc_auto_shape(M, N, K, true).split) return 0;
    return COUNTER_BYTES + (size_t)ngroups(K) * (size_t)M * (size_t)N * sizeof(float);
}

namespace bi {
namespace {
int check_await(const char* op, const Await& aw) {
    if (!aw.flags) return BI_OK;
    if (!aw.epoch || aw.world < 1 || aw.world > 8 || aw.rank < 0 || aw.rank >= aw.world)
        return fail(BI_ERR_BAD_ARG, "%s: bad gather to wait for (rank %d of %d)", op, aw.rank, aw.world);
    return BI_OK;
}

int matmul_impl(const void* a, const void* b, void* out, void* workspace, size_t workspace_bytes, int64_t M,
                int64_t N, int64_t K, int64_t a_sm, int64_t a_sk, int64_t b_sk, int64_t b_sn, int dtype,
                int path, int32_t* status, void* stream, const Await& aw, const void* bias = nullptr,
                const PushSink* sink = nullptr, const RopeSink* rope = nullptr) {
    if (!dtype_ok(dtype)) return fail(BI_ERR_UNSUPPORTED, "bi_matmul: dtype %d", dtype);
    if (M < 0 || N < 0 || K <= 0) return fail(BI_ERR_BAD_ARG, "bi_matmul: M=%lld N=%lld K=%lld", (long long)M, (long long)N, (long long)K);
    if (M == 0 || N == 0) return BI_OK;
    if (!a || !b || (!out && !sink && !rope)) return fail(BI_ERR_BAD_ARG, "bi_matmul: null pointer");
    if (M >= (1LL << 31) || N >= (1LL << 31) || K >= (1LL << 31)) return fail(BI_ERR_UNSUPPORTED, "bi_matmul: dimension too large");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t es = dtype_size(dtype);

    // Tensor-core path: 16-bit weight stored as rows of K contiguous elements (the W.T view of
    // nn.Linear's W[N, K]) that TMA can address. Decided by the weight alone.
    const bool weight_tc = dtype != BI_F32 && b_sk == 1 && K % 8 == 0 && aligned(b, 16) && (b_sn * (int64_t)es) % 16 == 0 &&
                           (N == 1 || b_sn >= K);
    PathArg pa;
    int rc = parse_path("bi_matmul", path, &pa);
    if (rc) return rc;
    if (sink || rope) {      // the fold kernel is the one that pushes / rotates: always the split shape, folded by the second launch
        if (!weight_tc) return fail(BI_ERR_UNSUPPORTED, "bi_matmul_push / bi_matmul_rope: only weights on the tensor-core path");
        pa.kind = BI_MATMUL_SPLIT;
    }
    float* part = nullptr;
    if (weight_tc) {
        const int64_t x_ld = M == 1 ? K : a_sm;
        if (a_sk != 1 || !aligned(a, 16) || (x_ld * (int64_t)es) % 16 != 0 || x_ld < K)
            return fail(BI_ERR_MISALIGNED, "bi_matmul: activation must be k-contiguous, 16-byte aligned rows for this weight");
        TcShape sh;
        rc = tc_shape("bi_matmul", pa, workspace, workspace_bytes, M, N, K, &sh, &part);
        if (rc) return rc;
        sh.await = aw;
        sh.bias = bias;
        const int64_t w_ld = N == 1 ? K : b_sn;
        rc = launch_tc_matmul(a, x_ld, b, w_ld, nullptr, out, part, M, N, K, dtype, sh, status, st);
        if (rc || !sh.split || sh.counters) return rc;
        if (rope) return launch_combine_rope(part, (int)ngroups(K), M * N, dtype, st, *rope);
        return launch_combine(part, out, (int)ngroups(K), M * N, dtype, st, bias, N, sink);
    }
    if (aw.flags) return fail(BI_ERR_UNSUPPORTED, "bi_matmul_awaiting: only weights on the tensor-core path can wait for a gather");
    bool split;
    rc = simt_shape("bi_matmul", pa, workspace, workspace_bytes, M, N, K, &split, &part);
    if (rc) return rc;
    return launch_simt_matmul(a, b, out, part, M, N, K, a_sm, a_sk, b_sk, b_sn, dtype, split, st, bias);
}
}  // namespace
}  // namespace bi

extern "C" int bi_matmul(const void* a, const void* b, void* out, void* workspace, size_t workspace_bytes, int64_t M,
                         int64_t N, int64_t K, int64_t a_sm, int64_t a_sk, int64_t b_sk, int64_t b_sn, int dtype,
                         int path, int32_t* status, void* stream) {
    return bi::matmul_impl(a, b, out, workspace, workspace_bytes, M, N, K, a_sm, a_sk, b_sk, b_sn, dtype, path, status, stream,
                           bi::Await{nullptr, nullptr, 0, 0});
}

extern "C" int bi_matmul_bias(const void* a, const void* b, const void* bias, void* out, void* workspace, size_t workspace_bytes,
                              int64_t M, int64_t N, int64_t K, int64_t a_sm, int64_t a_sk, int64_t b_sk, int64_t b_sn, int dtype,
                              int path, int32_t* status, void* stream) {
    if (bias && !bi::aligned(bias, bi::dtype_ok(dtype) ? bi::dtype_size(dtype) : 1))
        return bi::fail(BI_ERR_MISALIGNED, "bi_matmul_bias: bias is not aligned to its element size");
    return bi::matmul_impl(a, b, out, workspace, workspace_bytes, M, N, K, a_sm, a_sk, b_sk, b_sn, dtype, path, status, stream,
                           bi::Await{nullptr, nullptr, 0, 0}, bias);
}

extern "C" int bi_matmul_awaiting(const void* a, const void* b, void* out, void* workspace, size_t workspace_bytes, int64_t M,
                                  int64_t N, int64_t K, int64_t a_sm, int64_t a_sk, int64_t b_sk, int64_t b_sn, int dtype,
                                  int path, int32_t* status, void* stream, const uint32_t* flags, const uint32_t* epoch,
                                  int rank, int world) {
    const bi::Await aw{flags, epoch, rank, world};
    int rc = bi::check_await("bi_matmul_awaiting", aw);
    if (rc) return rc;
    return bi::matmul_impl(a, b, out, workspace, workspace_bytes, M, N, K, a_sm, a_sk, b_sk, b_sn, dtype, path, status, stream, aw);
}

namespace bi {
namespace {
int qmm_impl(const void* x, const uint32_t* w, const void* scales, const void* biases, void* out,
             void* workspace, size_t workspace_bytes, int64_t M, int64_t N, int64_t K, int64_t x_sm,
             int group_size, int bits, int dtype, int path, int32_t* status, void* stream, const Await& aw,
             const PushSink* sink = nullptr, const RopeSink* rope = nullptr) {
    if (!dtype_ok(dtype)) return fail(BI_ERR_UNSUPPORTED, "bi_qmm: dtype %d", dtype);
    if (bits != 4 && bits != 8) return fail(BI_ERR_UNSUPPORTED, "bi_qmm: bits=%d (supported: 4, 8)", bits);
    if (group_size != 32 && group_size != 64 && group_size != 128)
        return fail(BI_ERR_UNSUPPORTED, "bi_qmm: group_size=%d (supported: 32, 64, 128)", group_size);
    if (M < 0 || N < 0 || K <= 0) return fail(BI_ERR_BAD_ARG, "bi_qmm: M=%lld N=%lld K=%lld", (long long)M, (long long)N, (long long)K);
    if (K % group_size != 0) return fail(BI_ERR_UNSUPPORTED, "bi_qmm: K=%lld is not a multiple of group_size=%d", (long long)K, group_size);
    if (M == 0 || N == 0) return BI_OK;
    if (!x || !w || !scales || !biases || (!out && !sink && !rope)) return fail(BI_ERR_BAD_ARG, "bi_qmm: null pointer");
    if (M >= (1LL << 31) || N >= (1LL << 31) || K >= (1LL << 31)) return fail(BI_ERR_UNSUPPORTED, "bi_qmm: dimension too large");
    if (M > 1 && x_sm < K) return fail(BI_ERR_BAD_ARG, "bi_qmm: row stride %lld < K", (long long)x_sm);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t es = dtype_size(dtype);

    TcQuant q{w, scales, biases, bits, group_size};
    const bool weight_tc = dtype != BI_F32 && K % 64 == 0 && aligned(w, 16) && ((K * bits / 8) % 16) == 0;
    PathArg pa;
    int rc = parse_path("bi_qmm", path, &pa);
    if (rc) return rc;
    if (sink || rope) {
        if (!weight_tc) return fail(BI_ERR_UNSUPPORTED, "bi_qmm_push / bi_qmm_rope: only weights on the tensor-core path");
        pa.kind = BI_MATMUL_SPLIT;
    }
    float* part = nullptr;
    if (weight_tc) {
        const int64_t x_ld = M == 1 ? K : x_sm;
        if (!aligned(x, 16) || (x_ld * (int64_t)es) % 16 != 0)
            return fail(BI_ERR_MISALIGNED, "bi_qmm: activation must have 16-byte aligned rows for this weight");
        TcShape sh;
        rc = tc_shape("bi_qmm", pa, workspace, workspace_bytes, M, N, K, &sh, &part, true);
        if (rc) return rc;
        sh.await = aw;
        rc = launch_tc_matmul(x, x_ld, nullptr, 0, &q, out, part, M, N, K, dtype, sh, status, st);
        if (rc || !sh.split || sh.counters) return rc;
        if (rope) return launch_combine_rope(part, (int)ngroups(K), M * N, dtype, st, *rope);
        return launch_combine(part, out, (int)ngroups(K), M * N, dtype, st, nullptr, N, sink);
    }
    if (aw.flags) return fail(BI_ERR_UNSUPPORTED, "bi_qmm_awaiting: only weights on the tensor-core path can wait for a gather");
    bool split;
    rc = simt_shape("bi_qmm", pa, workspace, workspace_bytes, M, N, K, &split, &part);
    if (rc) return rc;
    return launch_simt_qmm(x, w, scales, biases, out, part, M, N, K, M == 1 ? K : x_sm, group_size, bits, dtype, split, st);
}
}  // namespace
}  // namespace bi

extern "C" int bi_qmm(const void* x, const uint32_t* w, const void* scales, const void* biases, void* out,
                      void* workspace, size_t workspace_bytes, int64_t M, int64_t N, int64_t K, int64_t x_sm,
                      int group_size, int bits, int dtype, int path, int32_t* status, void* stream) {
    return bi::qmm_impl(x, w, scales, biases, out, workspace, workspace_bytes, M, N, K, x_sm, group_size, bits, dtype, path, status,
                        stream, bi::Await{nullptr, nullptr, 0, 0});
}

extern "C" int bi_qmm_awaiting(const void* x, const uint32_t* w, const void* scales, const void* biases, void* out,
                               void* workspace, size_t workspace_bytes, int64_t M, int64_t N, int64_t K, int64_t x_sm,
                               int group_size, int bits, int dtype, int path, int32_t* status, void* stream,
                               const uint32_t* flags, const uint32_t* epoch, int rank, int world) {
    const bi::Await aw{flags, epoch, rank, world};
    int rc = bi::check_await("bi_qmm_awaiting", aw);
    if (rc) return rc;
    return bi::qmm_impl(x, w, scales, biases, out, workspace, workspace_bytes, M, N, K, x_sm, group_size, bits, dtype, path, status,
                        stream, aw);
}

// ---- output pushed into every rank's gathered activation (the fold of the split shape is the gather kernel) ----
extern "C" int bi_matmul_push(const void* a, const void* b, void* workspace, size_t workspace_bytes, int64_t M, int64_t N,
                              int64_t K, int64_t a_sm, int64_t a_sk, int64_t b_sk, int64_t b_sn, int dtype, int path,
                              int32_t* status, void* stream, const uint32_t* await_flags, const uint32_t* await_epoch,
                              void* const* dst, void* const* peer_flags, uint32_t* counters, int rank, int world, int wait) {
    using namespace bi;
    const Await aw{await_flags, await_flags ? await_epoch : nullptr, await_flags ? rank : 0, await_flags ? world : 0};
    int rc = check_await("bi_matmul_push", aw);
    if (rc) return rc;
    PushSink sink;
    rc = make_sink("bi_matmul_push", dst, peer_flags, counters, rank, world, wait, status, dtype_ok(dtype) ? dtype_size(dtype) : 1, &sink);
    if (rc) return rc;
    return matmul_impl(a, b, nullptr, workspace, workspace_bytes, M, N, K, a_sm, a_sk, b_sk, b_sn, dtype, path, status, stream, aw,
                       nullptr, &sink);
}

extern "C" int bi_qmm_push(const void* x, const uint32_t* w, const void* scales, const void* biases, void* workspace,
                           size_t workspace_bytes, int64_t M, int64_t N, int64_t K, int64_t x_sm, int group_size, int bits,
                           int dtype, int path, int32_t* status, void* stream, const uint32_t* await_flags,
                           const uint32_t* await_epoch, void* const* dst, void* const* peer_flags, uint32_t* counters, int rank,
                           int world, int wait) {
    using namespace bi;
    const Await aw{await_flags, await_flags ? await_epoch : nullptr, await_flags ? rank : 0, await_flags ? world : 0};
    int rc = check_await("bi_qmm_push", aw);
    if (rc) return rc;
    PushSink sink;
    rc = make_sink("bi_qmm_push", dst, peer_flags, counters, rank, world, wait, status, dtype_ok(dtype) ? dtype_size(dtype) : 1, &sink);
    if (rc) return rc;
    return qmm_impl(x, w, scales, biases, nullptr, workspace, workspace_bytes, M, N, K, x_sm, group_size, bits, dtype, path, status,
                    stream, aw, &sink);
}

// ---- qkv projection whose fold applies the rotary embedding and appends to the KV cache ----
namespace bi {
namespace {
int make_rope(const char* op, int64_t M, int64_t N, const float* cos_table, const float* sin_table, const int64_t* pos0, void* q_out,
              void* k_cache, void* v_cache, int64_t B, int64_t T, int64_t Hq, int64_t Hkv, int64_t D, int64_t c_sb, int64_t c_sh,
              int64_t c_sl, int64_t capacity, int32_t* status, RopeSink* r) {
    if (B <= 0 || T <= 0 || Hq <= 0 || Hkv <= 0 || D <= 0 || D % 2 || capacity <= 0) return fail(BI_ERR_BAD_ARG, "%s: bad sizes", op);
    if (M != B * T || N != (Hq + 2 * Hkv) * D)
        return fail(BI_ERR_BAD_ARG, "%s: the product must be [B*T, (Hq + 2*Hkv) * D] (M=%lld N=%lld)", op, (long long)M, (long long)N);
    if (!cos_table || !sin_table || !pos0 || !q_out || !k_cache || !v_cache) return fail(BI_ERR_BAD_ARG, "%s: null pointer", op);
    *r = RopeSink{cos_table, sin_table, pos0, q_out, k_cache, v_cache, (int)B, (int)T, (int)Hq, (int)Hkv, (int)D, c_sb, c_sh, c_sl, capacity, status};
    return BI_OK;
}
}  // namespace
}  // namespace bi

extern "C" int bi_matmul_rope(const void* a, const void* b, void* workspace, size_t workspace_bytes, int64_t M, int64_t N,
                              int64_t K, int64_t a_sm, int64_t a_sk, int64_t b_sk, int64_t b_sn, int dtype, int path,
                              int32_t* status, void* stream, const float* cos_table, const float* sin_table,
                              const int64_t* pos0, void* q_out, void* k_cache, void* v_cache, int64_t B, int64_t T, int64_t Hq,
                              int64_t Hkv, int64_t D, int64_t cache_sb, int64_t cache_sh, int64_t cache_sl, int64_t capacity) {
    using namespace bi;
    RopeSink rope;
    int rc = make_rope("bi_matmul_rope", M, N, cos_table, sin_table, pos0, q_out, k_cache, v_cache, B, T, Hq, Hkv, D, cache_sb,
                       cache_sh, cache_sl, capacity, status, &rope);
    if (rc) return rc;
    return matmul_impl(a, b, nullptr, workspace, workspace_bytes, M, N, K, a_sm, a_sk, b_sk, b_sn, dtype, path, status, stream,
                       Await{nullptr, nullptr, 0, 0}, nullptr, nullptr, &rope);
}

extern "C" int bi_qmm_rope(const void* x, const uint32_t* w, const void* scales, const void* biases, void* workspace,
                           size_t workspace_bytes, int64_t M, int64_t N, int64_t K, int64_t x_sm, int group_size, int bits,
                           int dtype, int path, int32_t* status, void* stream, const float* cos_table, const float* sin_table,
                           const int64_t* pos0, void* q_out, void* k_cache, void* v_cache, int64_t B, int64_t T, int64_t Hq,
                           int64_t Hkv, int64_t D, int64_t cache_sb, int64_t cache_sh, int64_t cache_sl, int64_t capacity) {
    using namespace bi;
    RopeSink rope;
    int rc = make_rope("bi_qmm_rope", M, N, cos_table, sin_table, pos0, q_out, k_cache, v_cache, B, T, Hq, Hkv, D, cache_sb,
                       cache_sh, cache_sl, capacity, status, &rope);
    if (rc) return rc;
    return qmm_impl(x, w, scales, biases, nullptr, workspace, workspace_bytes, M, N, K, x_sm, group_size, bits, dtype, path, status,
                    stream, Await{nullptr, nullptr, 0, 0}, nullptr, &rope);
}
