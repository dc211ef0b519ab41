// Launchers shared between the matmul translation units.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include "peer_push.cuh"

namespace bi {

// Split-path fold: out[i] = T(((0 + part[0][i]) + part[1][i]) + ...), part is [G][MN] fp32.
// bias: optional [N] in the output dtype (N = row length of out), added after the rounding.
// sink: when given (N must then be the row length), `out` is ignored and the result is pushed as this rank's column
// slice into every rank's gathered activation, handshake included.
int launch_combine(const float* part, void* out, int G, int64_t MN, int dtype, cudaStream_t st, const void* bias = nullptr,
                   int64_t N = 1, const PushSink* sink = nullptr);

// The qkv projection of a decoder: where the fold of its split partials sends the result instead of `out` -- rotated q
// into q_out[B, Hq, T, D], rotated k and plain v into the caches at position pos0[0] + t (the arguments of
// bi_rope_append, whose arithmetic and capacity guard the fold kernel repeats element for element).
struct RopeSink {
    const float* cos_table;
    const float* sin_table;
    const int64_t* pos0;
    void* q_out;
    void* k_cache;
    void* v_cache;
    int B, T, Hq, Hkv, D;
    int64_t c_sb, c_sh, c_sl, capacity;
    int32_t* status;
};
int launch_combine_rope(const float* part, int G, int64_t MN, int dtype, cudaStream_t st, const RopeSink& rope);

// CUDA-core path (fp32 inputs, or weights TMA cannot address).
int launch_simt_matmul(const void* a, const void* b, void* out, float* part, int64_t M, int64_t N, int64_t K,
                       int64_t a_sm, int64_t a_sk, int64_t b_sk, int64_t b_sn, int dtype, bool split,
                       cudaStream_t st, const void* bias = nullptr);
int launch_simt_qmm(const void* x, const uint32_t* w, const void* scales, const void* biases, void* out, float* part,
                    int64_t M, int64_t N, int64_t K, int64_t x_sm, int gs, int bits, int dtype, bool split,
                    cudaStream_t st);

// Tensor-core path (tcgen05 / TMEM / TMA), 16-bit inputs. `w_kn` describes the weight:
// dense -> pointer to W[N, K] rows with row stride w_ld elements; quantized -> packed codes.
struct TcQuant {
    const uint32_t* codes;  // nullptr for the dense kernel
    const void* scales;
    const void* biases;
    int bits, gs;
};
// Returns true when the tensor-core path can take this weight / activation layout.
bool tc_matmul_supported(const void* x, int64_t x_ld, const void* w, int64_t w_ld, int64_t N, int64_t K, int dtype,
                         const TcQuant* q);
// Launch shape of a tensor-core matmul (every choice gives the same bits):
//   split     one work unit per (tile, K group) writing raw fp32 partials; else one unit per tile folding in place
//   bm        batch rows per tile: 16, 32, 64 or 128
//   counters  split only: per-tile arrival counters (all zero) -> the last CTA of a tile folds the partials and
//             writes `out` itself; nullptr -> the caller launches the combine kernel
//   stage     quantized only: how the dequantized weight operand reaches the MMA
//   await     the activation is the destination of a peer gather whose arrival nobody has waited for yet: the
//             kernel starts streaming weights at once and reads the activation only after every peer's flag
//             has reached *epoch (bounded wait); flags == nullptr -> nothing to wait for
struct Await {
    const uint32_t* flags;   // this rank's flag array, one word per rank
    const uint32_t* epoch;   // the gather's epoch, in device memory
    int rank, world;
};
struct TcShape {
    enum { STAGE_AUTO = 0, STAGE_SMEM = 1, STAGE_TMEM = 2 };
    bool split;
    int bm;
    unsigned* counters;
    int stage;
    Await await;
    const void* bias;     // optional [N] bias in the output dtype, added after the output's rounding
};
int launch_tc_matmul(const void* x, int64_t x_ld, const void* w, int64_t w_ld, const TcQuant* q, void* out,
                     float* part, int64_t M, int64_t N, int64_t K, int dtype, const TcShape& shape, int32_t* status,
                     cudaStream_t st);

}  // namespace bi
