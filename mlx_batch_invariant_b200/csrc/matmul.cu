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

int64_t ngroups(int64_t K) { return (K + GROUP_K - 1) / GROUP_K; }

// AUTO launch shape for the tensor-core path.
bool tc_auto_split(int64_t M, int64_t N, int64_t K) {
    if (ngroups(K) <= 1) return false;
    const int64_t tiles = ((N + 127) / 128) * ((M + 127) / 128);
    if (tiles >= 148) return false;  // enough tiles to fill the GPU without cutting K
    // too few tiles: spread the K groups over CTAs as well. Measured at N = K = 4096: M = 128 17 us split,
    // 35 us fused; M = 256 28 us against 35 us; the partials are written and read back through L2.
    return M <= SPLIT_M_MAX || ngroups(K) * M * N * (int64_t)sizeof(float) <= SPLIT_PARTIAL_MAX;
}
// AUTO launch shape for the CUDA-core path (reference rule: M <= 32 and more than one group).
bool simt_auto_split(int64_t M, int64_t K) { return ngroups(K) > 1 && M <= 32; }

int resolve_split(int path, bool auto_split, int64_t K, bool* split) {
    if (path == BI_MATMUL_AUTO) *split = auto_split;
    else if (path == BI_MATMUL_SPLIT) *split = true;
    else if (path == BI_MATMUL_FUSED) *split = false;
    else return fail(BI_ERR_BAD_ARG, "matmul: unknown path %d", path);
    (void)K;
    return BI_OK;
}

int check_ws(const char* op, bool split, void* ws, size_t ws_bytes, int64_t M, int64_t N, int64_t K) {
    if (!split) return BI_OK;
    const size_t need = (size_t)ngroups(K) * (size_t)M * (size_t)N * sizeof(float);
    if (!ws || ws_bytes < need) return fail(BI_ERR_WORKSPACE, "%s: split path needs %zu workspace bytes, got %zu", op, need, ws_bytes);
    if (!aligned(ws, 16)) return fail(BI_ERR_MISALIGNED, "%s: workspace must be 16-byte aligned", op);
    return BI_OK;
}

}  // namespace
}  // namespace bi

extern "C" size_t bi_matmul_workspace_bytes(int64_t M, int64_t N, int64_t K, int dtype) {
    using namespace bi;
    (void)dtype;
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    // Enough for whichever shape AUTO may pick; a forced BI_MATMUL_SPLIT always needs
    // ceil(K/256) * M * N * 4 bytes.
    if (ngroups(K) <= 1) return 0;
    if (M > SPLIT_M_MAX && !tc_auto_split(M, N, K)) return 0;
    return (size_t)ngroups(K) * (size_t)M * (size_t)N * sizeof(float);
}

extern "C" size_t bi_qmm_workspace_bytes(int64_t M, int64_t N, int64_t K, int dtype) {
    return bi_matmul_workspace_bytes(M, N, K, dtype);
}

extern "C" int bi_matmul(const void* a, const void* b, void* out, void* workspace, size_t workspace_bytes, int64_t M,
                         int64_t N, int64_t K, int64_t a_sm, int64_t a_sk, int64_t b_sk, int64_t b_sn, int dtype,
                         int path, int32_t* status, void* stream) {
    using namespace bi;
    if (!dtype_ok(dtype)) return fail(BI_ERR_UNSUPPORTED, "bi_matmul: dtype %d", dtype);
    if (M < 0 || N < 0 || K <= 0) return fail(BI_ERR_BAD_ARG, "bi_matmul: M=%lld N=%lld K=%lld", (long long)M, (long long)N, (long long)K);
    if (M == 0 || N == 0) return BI_OK;
    if (!a || !b || !out) return fail(BI_ERR_BAD_ARG, "bi_matmul: null pointer");
    if (M >= (1LL << 31) || N >= (1LL << 31) || K >= (1LL << 31)) return fail(BI_ERR_UNSUPPORTED, "bi_matmul: dimension too large");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t es = dtype_size(dtype);

    // Tensor-core path: 16-bit weight stored as rows of K contiguous elements (the W.T view of
    // nn.Linear's W[N, K]) that TMA can address. Decided by the weight alone.
    const bool weight_tc = dtype != BI_F32 && b_sk == 1 && K % 8 == 0 && aligned(b, 16) && (b_sn * (int64_t)es) % 16 == 0 &&
                           (N == 1 || b_sn >= K);
    bool split;
    if (weight_tc) {
        const int64_t x_ld = M == 1 ? K : a_sm;
        if (a_sk != 1 || !aligned(a, 16) || (x_ld * (int64_t)es) % 16 != 0 || x_ld < K)
            return fail(BI_ERR_MISALIGNED, "bi_matmul: activation must be k-contiguous, 16-byte aligned rows for this weight");
        int rc = resolve_split(path, tc_auto_split(M, N, K), K, &split);
        if (rc) return rc;
        rc = check_ws("bi_matmul", split, workspace, workspace_bytes, M, N, K);
        if (rc) return rc;
        const int64_t w_ld = N == 1 ? K : b_sn;
        rc = launch_tc_matmul(a, x_ld, b, w_ld, nullptr, out, static_cast<float*>(workspace), M, N, K, dtype, split, status, st);
        if (rc || !split) return rc;
        return launch_combine(static_cast<float*>(workspace), out, (int)ngroups(K), M * N, dtype, st);
    }
    int rc = resolve_split(path, simt_auto_split(M, K), K, &split);
    if (rc) return rc;
    rc = check_ws("bi_matmul", split, workspace, workspace_bytes, M, N, K);
    if (rc) return rc;
    return launch_simt_matmul(a, b, out, static_cast<float*>(workspace), M, N, K, a_sm, a_sk, b_sk, b_sn, dtype, split, st);
}

extern "C" int bi_qmm(const void* x, const uint32_t* w, const void* scales, const void* biases, void* out,
                      void* workspace, size_t workspace_bytes, int64_t M, int64_t N, int64_t K, int64_t x_sm,
                      int group_size, int bits, int dtype, int path, int32_t* status, void* stream) {
    using namespace bi;
    if (!dtype_ok(dtype)) return fail(BI_ERR_UNSUPPORTED, "bi_qmm: dtype %d", dtype);
    if (bits != 4 && bits != 8) return fail(BI_ERR_UNSUPPORTED, "bi_qmm: bits=%d (supported: 4, 8)", bits);
    if (group_size != 32 && group_size != 64 && group_size != 128)
        return fail(BI_ERR_UNSUPPORTED, "bi_qmm: group_size=%d (supported: 32, 64, 128)", group_size);
    if (M < 0 || N < 0 || K <= 0) return fail(BI_ERR_BAD_ARG, "bi_qmm: M=%lld N=%lld K=%lld", (long long)M, (long long)N, (long long)K);
    if (K % group_size != 0) return fail(BI_ERR_UNSUPPORTED, "bi_qmm: K=%lld is not a multiple of group_size=%d", (long long)K, group_size);
    if (M == 0 || N == 0) return BI_OK;
    if (!x || !w || !scales || !biases || !out) return fail(BI_ERR_BAD_ARG, "bi_qmm: null pointer");
    if (M >= (1LL << 31) || N >= (1LL << 31) || K >= (1LL << 31)) return fail(BI_ERR_UNSUPPORTED, "bi_qmm: dimension too large");
    if (M > 1 && x_sm < K) return fail(BI_ERR_BAD_ARG, "bi_qmm: row stride %lld < K", (long long)x_sm);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t es = dtype_size(dtype);

    TcQuant q{w, scales, biases, bits, group_size};
    const bool weight_tc = dtype != BI_F32 && K % 64 == 0 && aligned(w, 16) && ((K * bits / 8) % 16) == 0;
    bool split;
    if (weight_tc) {
        const int64_t x_ld = M == 1 ? K : x_sm;
        if (!aligned(x, 16) || (x_ld * (int64_t)es) % 16 != 0)
            return fail(BI_ERR_MISALIGNED, "bi_qmm: activation must have 16-byte aligned rows for this weight");
        int rc = resolve_split(path, tc_auto_split(M, N, K), K, &split);
        if (rc) return rc;
        rc = check_ws("bi_qmm", split, workspace, workspace_bytes, M, N, K);
        if (rc) return rc;
        rc = launch_tc_matmul(x, x_ld, nullptr, 0, &q, out, static_cast<float*>(workspace), M, N, K, dtype, split, status, st);
        if (rc || !split) return rc;
        return launch_combine(static_cast<float*>(workspace), out, (int)ngroups(K), M * N, dtype, st);
    }
    int rc = resolve_split(path, simt_auto_split(M, K), K, &split);
    if (rc) return rc;
    rc = check_ws("bi_qmm", split, workspace, workspace_bytes, M, N, K);
    if (rc) return rc;
    return launch_simt_qmm(x, w, scales, biases, out, static_cast<float*>(workspace), M, N, K, M == 1 ? K : x_sm,
                           group_size, bits, dtype, split, st);
}
