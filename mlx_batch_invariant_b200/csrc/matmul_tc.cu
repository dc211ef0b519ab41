// Tensor-core matmul for 16-bit inputs on sm_100a: TMA -> shared memory ->
// tcgen05.mma -> TMEM -> registers.   out[M, N] = x[M, K] @ W[N, K]^T
//
// Canonical order per output element (what never changes with M):
//   * K is cut into groups of 256. Inside a group the tensor core runs sixteen
//     MMA steps of K = 16 in ascending k,
//     tcgen05.mma.cta_group::1.kind::f16  M=128 (weight rows) x N (batch rows) x K=16,
//     operands in the input dtype, fp32 accumulator. N is the batch tile's row
//     count rounded up to 16 (16 ... 128): an accumulator column depends on its
//     own batch row only, and the tests compare every N the kernel can issue
//     with the bits of a batch of one. The first step of a group overwrites the
//     accumulator (accumulate off), so a group partial starts from nothing.
//   * out = T(((0 + p_0) + p_1) + ... ), plain fp32 adds of the group partials,
//     g ascending, one rounding at the end.
// The weight is the 128-row "A" operand and the batch is the "B" operand, so a
// decode step with one row issues the instruction of a 16-row tile; batch rows
// beyond M are never loaded (their accumulator columns hold garbage that is
// never read).
//
// Launch shapes (same arithmetic, reference: mlx_batch_invariant/kernels/matmul.py:279-314):
//   split : one job per (weight tile, batch tile, K group); the raw fp32 group
//           partial goes to the workspace and combine_kernel folds the groups.
//   fused : one unit per (weight tile, batch tile); the epilogue warps keep the
//           running total in registers and fold each group partial as it leaves TMEM.
// Both are one persistent kernel: CTA c takes a contiguous range of units, a
// TMA warp streams stages through a ring of shared-memory buffers, one thread
// issues the MMAs into one of two TMEM accumulators, four epilogue warps drain
// the other (the fused path keeps its running total in a third TMEM region).
// For affine-quantized weights the TMA ring carries the packed codes (a deep
// ring of small stages, so enough bytes are in flight to cover HBM latency)
// and dequantizer warps turn them into the 16-bit weight operand
// (fma(float(code), scale, bias) in fp32, one rounding --
// mlx_batch_invariant/kernels/quantized.py:44-67), so the MMA sequence is the
// dense one. Two stagings of that operand exist:
//   * tile body (batches above 64 rows): eight warps write the same swizzled
//     shared-memory tile the dense path would have loaded;
//   * streaming (decode, up to 64 rows): sixteen warps, one weight row per
//     thread, write the operand straight into tensor memory (tcgen05.st) and
//     the MMA reads its weight operand from there, so the dequantized tile
//     never crosses shared memory and needs no proxy fence.
//
// The split path can fold in the producing kernel: a CTA that has stored its
// group partial bumps a per-tile counter, and the CTA that arrives last reads
// the G partials of the tile back in ascending g and writes T(total) -- the adds
// and their order are those of combine_kernel, nobody waits for anybody.
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
constexpr int BLOCK_M = 128;  // most batch rows per tile (UMMA N); a launch may use 16, 32 or 64 (Params::bm)
constexpr int BLOCK_K = 64;   // elements per stage along K: 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int W_TILE_BYTES = BLOCK_N * BLOCK_K * 2;
constexpr int TMEM_COLS = 512;
// Tensor-memory columns: accumulator 0 at 0, accumulator 1 at acc_stride, the fused path's running total at
// 2 * acc_stride (acc_stride = 128; 64 or 32 in the streaming variant, whose batch tile is at most 64 rows), and
// in the streaming variant the weight-operand ring from column a_col0: w_slots chunks x 4 K steps x 32 columns
// (two chunks from column 256; three from column 128 when the batch tile is at most 32 rows).
constexpr int TMEM_A_STEP = BLOCK_K / 2;   // columns of one K step of the weight operand (two 16-bit values per column)
constexpr uint64_t WAIT_LIMIT_NS = 2000000000ull;
#ifndef BI_EPI_SLEEP_NS
#define BI_EPI_SLEEP_NS 100
#endif

constexpr int MAX_SLOTS = 8;     // ring depths and the chunk-completion barrier array (power of two)
constexpr int WARP_TMA = 0, WARP_MMA = 1, WARP_EPI0 = 2, WARP_DEQ0 = 6;
constexpr int SMEM_LIMIT = 227 * 1024;
constexpr int BAR_BYTES = 512;

// TSA: the weight ("A") operand of the MMA comes from tensor memory (streaming quantized variant).
template <int QBITS, bool TSA> struct Cfg {
    static constexpr int RAW_BYTES = QBITS ? BLOCK_N * BLOCK_K * QBITS / 8 : 0;
    static constexpr int N_DEQ_WARPS = QBITS ? (TSA ? 16 : 8) : 0;
    static constexpr int THREADS = 32 * (WARP_DEQ0 + N_DEQ_WARPS);
};
constexpr int TSA_SMEM_CAP = 164 * 1024;   // leaves the L1 its share: the streaming dequantizers read scales through it

// Shared memory, in this order (every tile 1024-byte aligned):
//   x ring     load_slots x ks x x_bytes  activation tiles (TMA, 128-byte swizzle). Only the batch rows
//                                         that exist are loaded; the MMA still reads 128 rows from the
//                                         tile base, so the ring sits first and what follows it is
//                                         valid (unread-result) memory.
//   W ring     dense: load_slots x ks x 16 KB (TMA)   quantized tile body: w_slots x ks x 16 KB (dequantizers)
//              streaming: none (the operand lives in tensor memory)
//   raw ring   quantized only: load_slots x ks x RAW_BYTES packed codes (TMA). A chunk's codes arrive as one
//              or two boxes of 128 weight rows x raw_span bytes (raw_span = the chunk's bytes of a row, at
//              most 128), swizzled so that threads reading one 16-byte piece per row meet no bank
//              conflict. The box is as wide as the chunk, not as a K step: the TMA unit and the memory
//              system work per row, and 32-byte rows streamed at a twentieth of the rate of 128-byte rows.
//   barriers
struct Params {
    void* out;          // [M, N] in T (fused)
    float* part;        // [G, M, N] fp32 (split)
    const void* scales; // quantized only: [N, K/gs] in T
    const void* biases;
    int32_t* status;
    const void* bias;   // optional [N] in T, added to the rounded output (fused and in-kernel-fold shapes)
    Await await;        // activation produced by a peer gather that has not been waited for (flags == nullptr: none)
    unsigned* counters; // split path with in-kernel fold: one arrival counter per (weight tile, batch tile), zero between calls
    int M, N, K, G;
    int n_tiles, m_tiles;
    int bm;             // batch rows per tile: 16, 32, 64 or 128 (launch shape; an output column's bits do not depend on it)
    int split;          // 1: split jobs, 0: fused units
    int x_rows;         // rows of the activation TMA box
    int box3d;          // 1: one TMA box holds a whole chunk (all K steps of a slot) of an operand
    int smem_bytes;     // dynamic shared memory of the launch
    int x_bytes;        // shared-memory bytes reserved per activation tile
    int ks;             // K steps (of 64) per chunk = per ring slot = per tcgen05.commit
    int load_slots;     // depth of the TMA ring, in chunks
    int w_slots;        // depth of the dequantized-weight ring (quantized), in chunks
    int w_ring_slots;   // slots of the ring the MMA reads weights from (w_slots, or load_slots when dense)
    int acc_stride;     // tensor-memory columns between the two accumulators
    int a_col0;         // streaming variant: first tensor-memory column of the weight-operand ring
    int uniform;        // every chunk is a whole K group (K % 256 == 0 and four K steps per chunk)
    int raw_span;       // quantized: bytes of one weight row in one box of packed codes (32, 64 or 128)
    int raw_boxes;      // quantized: boxes of packed codes per chunk (1 or 2)
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
    if (role == ROLE_EPI || role == ROLE_DEQ) {
        // whole warps wait here; back off so they do not take issue slots from the TMA and MMA threads
        for (int i = 0; i < 2048; ++i) {
            if (ptx::mbar_try_wait(bar, parity)) return true;
            __nanosleep(BI_EPI_SLEEP_NS);
        }
    } else {
        for (int i = 0; i < 4096; ++i)
            if (ptx::mbar_try_wait(bar, parity)) return true;
    }
    const uint64_t t0 = ptx::globaltimer_ns();
    while (true) {
        for (int i = 0; i < 256; ++i)
            if (ptx::mbar_try_wait(bar, parity)) return true;
        if (*c.abort_flag) return false;
        if (ptx::globaltimer_ns() - t0 > WAIT_LIMIT_NS) { report(c, role, idx); return false; }
    }
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

// Byte offset, inside a chunk's packed codes, of 16-byte piece `piece` of weight row `row` (pieces count along the
// row's bytes of the chunk). The codes lie as boxes of 128 rows x span bytes under the TMA swizzle of that span:
// the piece index inside a span is XORed with bits [7, 7 + log2(span / 16)) of the byte address.
__device__ __forceinline__ uint32_t raw_piece_offset(int row, int piece, int span) {
    const int per = span >> 4;                         // pieces per row of one box: 2, 4 or 8
    const int box = piece / per, pb = piece - box * per;
    const int sw = ((row * span) >> 7) & (per - 1);
    return (uint32_t)(box * (BLOCK_N * span) + row * span + ((pb ^ sw) << 4));
}

// Eight consecutive codes -> eight T values, one 16-byte swizzle chunk.
//   value = T(fma(float(code), scale, bias))   fp32 fma, one rounding.
// float(code) is formed exactly without an integer->float conversion: a byte permute drops the code
// into the low mantissa byte of 2^23 (0x4B0000cc = 8388608 + cc) and 2^23 is subtracted, which is
// exact. The subtract and the fma run as packed f32x2 instructions: two independent IEEE
// round-to-nearest operations each, same bits as the scalar forms.
template <typename T, int QBITS>
__device__ __forceinline__ uint4 dequant8(const uint32_t* words, uint64_t s2, uint64_t b2) {
    const uint64_t neg_magic = ptx::pack2(-8388608.0f, -8388608.0f);
    uint32_t src_even[4], src_odd[4];  // register + byte index holding codes 2i and 2i+1
    uint32_t o[4];
    if (QBITS == 4) {
        const uint32_t lo = words[0] & 0x0F0F0F0Fu;          // bytes: codes 0, 2, 4, 6
        const uint32_t hi = (words[0] >> 4) & 0x0F0F0F0Fu;   // bytes: codes 1, 3, 5, 7
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            src_even[i] = __byte_perm(lo, 0x4B000000u, 0x7540u + i);
            src_odd[i] = __byte_perm(hi, 0x4B000000u, 0x7540u + i);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            src_even[i] = __byte_perm(words[i >> 1], 0x4B000000u, 0x7540u + 2 * (i & 1));
            src_odd[i] = __byte_perm(words[i >> 1], 0x4B000000u, 0x7540u + 2 * (i & 1) + 1);
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint64_t v = ptx::pack2(__uint_as_float(src_even[i]), __uint_as_float(src_odd[i]));
        v = ptx::add2_rn(v, neg_magic);
        v = ptx::fma2_rn(v, s2, b2);
        float x, y;
        ptx::unpack2(v, x, y);
        o[i] = Pack2<T>::rn(x, y);
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
}

// Work is cut into "chunks": up to p.ks consecutive 64-wide K steps of one K group. A chunk is the
// unit of every ring slot and of MMA completion tracking: the issuing thread commits once per chunk
// (a tcgen05.commit drains the tensor pipe for ~200 cycles, so it is issued as rarely as the
// shared-memory budget allows), and everyone who needs "the MMAs of chunk c are done" -- the TMA
// thread before it refills a slot, the dequantizers before they overwrite a weight slot, the
// epilogue before it reads an accumulator -- waits on the same barrier done[c % 8].
struct ChunkIter {
    // Enumerates (unit, group, chunk) in the one order every role follows, and keeps the ring
    // positions of the current chunk. Only the constructor divides; stepping is increments.
    const Params& p;
    int left;                 // units still to go, including the current one
    int nt, mt;               // weight tile, batch tile of the current unit
    int g, g1;                // current K group, end of the unit's group range
    int nst, c, nchunk;       // K steps in the group, chunk index, chunks in the group
    int ci;                   // CTA-local running chunk index
    int l, w, d;              // load slot, weight slot, completion barrier of the chunk
    uint32_t lph, wph, dph;   // phase parities of those rings
    __device__ __forceinline__ ChunkIter(const Params& pp, int ub, int ue) : p(pp), left(ue - ub) {
        ci = 0; l = w = d = 0; lph = wph = dph = 0;
        nt = mt = g = g1 = nst = c = nchunk = 0;
        if (left <= 0) return;
        int tile;
        if (p.split) { tile = ub / p.G; g = ub - tile * p.G; g1 = g + 1; }
        else         { tile = ub; g = 0; g1 = p.G; }
        nt = tile / p.m_tiles; mt = tile - nt * p.m_tiles;
        start_group();
    }
    __device__ __forceinline__ void start_group() {
        const int kw = min(p.K - g * GROUP_K, GROUP_K);
        nst = (kw + BLOCK_K - 1) / BLOCK_K;
        nchunk = (nst + p.ks - 1) >> (p.ks >> 1);                  // ks is 1, 2 or 4
        c = 0;
    }
    __device__ __forceinline__ bool valid() const { return left > 0; }
    __device__ __forceinline__ int n0() const { return nt * BLOCK_N; }
    __device__ __forceinline__ int m0() const { return mt * p.bm; }
    __device__ __forceinline__ int ksteps() const { return min(p.ks, nst - c * p.ks); }
    __device__ __forceinline__ int k0() const { return g * GROUP_K + c * p.ks * BLOCK_K; }
    __device__ __forceinline__ bool first_in_group() const { return c == 0; }
    __device__ __forceinline__ bool last_in_group() const { return c == nchunk - 1; }
    // Branch-free on purpose: every role calls this once per chunk, and as a chain of dependent branches it cost
    // 300-400 cycles a call next to sixteen busy dequantizer warps (a dependent scalar instruction issues about
    // every ten cycles there). As selects the steps are mostly independent, and a caller can put the call in
    // front of its arithmetic so that the two interleave. Stepping past the last chunk leaves valid() false and
    // the other fields meaningless.
    __device__ __forceinline__ void next() {
        ++ci;
        { const int t = l + 1; const bool wr = t == p.load_slots; l = wr ? 0 : t; lph ^= wr ? 1u : 0u; }
        { const int t = w + 1; const bool wr = t == p.w_ring_slots; w = wr ? 0 : t; wph ^= wr ? 1u : 0u; }
        { const int t = d + 1; const bool wr = t == MAX_SLOTS; d = wr ? 0 : t; dph ^= wr ? 1u : 0u; }
        const int c1 = c + 1, gn = g + 1, mt1 = mt + 1;
        const bool stay = c1 < nchunk;                              // next chunk of the same K group
        const bool unit_end = !stay && gn >= g1;                    // else: next group of the same unit
        const bool tile_adv = unit_end && (!p.split || gn == p.G);  // a split unit is one (tile, group)
        const bool mwrap = mt1 == p.m_tiles;
        left -= unit_end ? 1 : 0;
        mt = tile_adv ? (mwrap ? 0 : mt1) : mt;
        nt += (tile_adv && mwrap) ? 1 : 0;
        g = stay ? g : (tile_adv ? 0 : gn);
        g1 = (unit_end && p.split) ? g + 1 : g1;
        const int kw = min(p.K - g * GROUP_K, GROUP_K);
        const int nst_n = (kw + BLOCK_K - 1) >> 6;
        static_assert(BLOCK_K == 64, "shift above");
        nchunk = stay ? nchunk : ((nst_n + p.ks - 1) >> (p.ks >> 1));      // ks is 1, 2 or 4
        nst = stay ? nst : nst_n;
        c = stay ? c1 : 0;
    }
};

// One weight row's 64 codes of K step `kstep` of a chunk -> 32 packed pairs of T, written to the row's
// tensor-memory lane at columns taddr .. taddr+31 (column c holds elements 2c and 2c+1 of the row, low half
// first) in two stores of 16 columns. `raw` is the chunk's packed codes as the TMA boxes left them (rows of 128
// bytes, 128-byte swizzle); (s2a, b2a) apply to codes 0..31, (s2b, b2b) to codes 32..63.
template <typename T, int QBITS>
__device__ __forceinline__ void dequant_row64_to_tmem(const uint8_t* raw, int row, int kstep, uint64_t s2a, uint64_t b2a,
                                                      uint64_t s2b, uint64_t b2b, uint32_t taddr) {
    constexpr int PIECES = BLOCK_K * QBITS / 8 / 16;     // 16-byte pieces behind 64 codes: 2 (4-bit) or 4 (8-bit)
    constexpr int HP = PIECES / 2;                       // pieces behind 32 codes
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint64_t s2 = h ? s2b : s2a, b2 = h ? b2b : b2a;
        uint32_t o[16];
#pragma unroll
        for (int cc = 0; cc < HP; ++cc) {
            const uint4 q = *reinterpret_cast<const uint4*>(raw + raw_piece_offset(row, kstep * PIECES + h * HP + cc, 128));
            const uint32_t w[4] = {q.x, q.y, q.z, q.w};
            if (QBITS == 4) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint4 v = dequant8<T, 4>(&w[i], s2, b2);
                    o[i * 4 + 0] = v.x; o[i * 4 + 1] = v.y; o[i * 4 + 2] = v.z; o[i * 4 + 3] = v.w;
                }
            } else {
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const uint4 v = dequant8<T, 8>(&w[2 * i], s2, b2);
                    o[(cc * 2 + i) * 4 + 0] = v.x; o[(cc * 2 + i) * 4 + 1] = v.y;
                    o[(cc * 2 + i) * 4 + 2] = v.z; o[(cc * 2 + i) * 4 + 3] = v.w;
                }
            }
        }
        ptx::tmem_st_32x16(taddr + 16u * h, o);
    }
}

template <typename T, int QBITS, bool TSA>
__global__ void __launch_bounds__((Cfg<QBITS, TSA>::THREADS), 1)
tc_matmul_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                 const Params p) {
    using C = Cfg<QBITS, TSA>;
    static_assert(!TSA || QBITS != 0, "the tensor-memory weight operand exists for quantized weights only");
    ptx::grid_dep_launch();   // the next kernel of the stream may start its set-up
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
    const int LS = p.load_slots, KS = p.ks;
    const int WS = QBITS ? p.w_slots : p.load_slots;                 // slots of the weight-operand ring
    const int WS_SMEM = TSA ? 0 : WS;                                // ... of which live in shared memory
    const uint32_t w_ring = smem_base + (uint32_t)(LS * KS) * p.x_bytes;
    const uint32_t raw_ring = w_ring + (uint32_t)(WS_SMEM * KS) * W_TILE_BYTES;
    const uint32_t bar_base = raw_ring + (uint32_t)(LS * KS) * C::RAW_BYTES;
    auto x_tile = [&](int l, int j) { return smem_base + (uint32_t)(l * KS + j) * p.x_bytes; };
    auto w_tile = [&](int w, int j) { return w_ring + (uint32_t)(w * KS + j) * W_TILE_BYTES; };
    auto raw_chunk = [&](int l) { return raw_ring + (uint32_t)(l * KS) * C::RAW_BYTES; };   // packed codes of slot l
    auto bar_lfull = [&](int l) { return bar_base + 8u * l; };                    // TMA landed (slot l)
    auto bar_wfull = [&](int w) { return bar_base + 8u * (MAX_SLOTS + w); };      // dequantized chunk ready
    auto bar_done = [&](int d) { return bar_base + 8u * (2 * MAX_SLOTS + d); };   // MMAs of a chunk complete
    auto bar_tempty = [&](int b) { return bar_base + 8u * (3 * MAX_SLOTS + b); }; // accumulator drained
    const uint32_t bar_epi = bar_base + 8u * (3 * MAX_SLOTS + 2);                 // the four epilogue warps meet here
    uint8_t* misc = smem_gen + (bar_base - smem_base) + 8 * (3 * MAX_SLOTS + 3);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(misc);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(misc + 4);
    volatile int* fold_flag = reinterpret_cast<volatile int*>(misc + 8);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const Ctl ctl{p.status, abort_flag};

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        *fold_flag = 0;
        for (int i = 0; i < MAX_SLOTS; ++i) {
            ptx::mbar_init(bar_lfull(i), 1);
            ptx::mbar_init(bar_wfull(i), C::N_DEQ_WARPS ? C::N_DEQ_WARPS : 1);
            ptx::mbar_init(bar_done(i), 1);
        }
        for (int b = 0; b < 2; ++b) ptx::mbar_init(bar_tempty(b), 4);
        ptx::mbar_init(bar_epi, 4);
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
    // Barriers, tensor memory and the tensor maps were set up while the kernel before this one was still draining;
    // from here on global memory is touched.
    ptx::grid_dep_wait();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_total = 2u * (uint32_t)p.acc_stride;

    const int ub = (int)(p.units * blockIdx.x / gridDim.x);
    const int ue = (int)(p.units * (blockIdx.x + 1) / gridDim.x);
    // wait until the MMAs of chunk `ci` (CTA-local running index) have completed
    auto wait_done = [&](int ci, int role) {   // MAX_SLOTS is a power of two: mask and shift, no division
        return wait_bounded(bar_done(ci & (MAX_SLOTS - 1)), (uint32_t)(ci >> 3) & 1u, ctl, role, 16 + (ci & (MAX_SLOTS - 1)));
    };
    static_assert(MAX_SLOTS == 8, "wait_done shifts by log2(MAX_SLOTS)");

    if (warp == WARP_TMA) {
        // ------------------------------------------------------------ TMA producer
        // The whole warp runs the loop (warp-uniform control flow and address arithmetic), one elected lane issues.
        {
            const bool leader = ptx::elect_one();
            // The TMA unit's cost is per instruction (a few hundred cycles each, whatever the box holds), so
            // with box3d one box brings all K steps of a chunk: the tensor map is a 3-D view
            // [K/64 blocks][rows][64 elements] whose box lands as consecutive K-step tiles. K steps of the
            // box that lie beyond K are zero-filled and still count towards the barrier's bytes.
            const uint32_t xb = (uint32_t)p.x_rows * BLOCK_K * 2;
            const uint32_t wb = (uint32_t)W_TILE_BYTES;
            const uint32_t raw_box_bytes = (uint32_t)(BLOCK_N * p.raw_span);
            const bool w3d = p.box3d && !QBITS;
            // Weight tiles go through L2 marked evict-first: they should not push the batch rows or the split
            // path's partials out (measured faster also where several batch tiles re-read a weight tile).
            const uint64_t w_policy = ptx::l2_policy_evict_first();
            bool ok = true;
            // weight side of a chunk: arm the slot's barrier with all of the chunk's bytes, start the weight copies
            auto issue_w = [&](const ChunkIter& c) {
                const int l = c.l, kc = c.ksteps();
                const uint32_t bar = bar_lfull(l);
                const uint32_t tx = xb * (uint32_t)(p.box3d ? KS : kc) +
                                    (QBITS ? raw_box_bytes * (uint32_t)p.raw_boxes : wb * (uint32_t)(w3d ? KS : kc));
                const int n0 = c.n0(), k0c = c.k0();
                if (leader) {
                    ptx::mbar_expect_tx(bar, tx);
                    if (QBITS) {
                        // the chunk's codes: whole boxes (columns past the end of a weight row are zero-filled)
                        for (int b = 0; b < p.raw_boxes; ++b)
                            ptx::tma_load_2d_hint(raw_chunk(l) + (uint32_t)b * raw_box_bytes, &tmap_w,
                                                  k0c * QBITS / 32 + b * (p.raw_span >> 2), n0, bar, w_policy);
                    }
                    if (w3d) ptx::tma_load_3d_hint(w_tile(l, 0), &tmap_w, 0, n0, k0c >> 6, bar, w_policy);
                    if (!QBITS && !w3d)
                        for (int j = 0; j < kc; ++j) ptx::tma_load_2d_hint(w_tile(l, j), &tmap_w, k0c + j * BLOCK_K, n0, bar, w_policy);
                }
            };
            // activation side of the same chunk
            auto issue_x = [&](const ChunkIter& c) {
                const int l = c.l, kc = c.ksteps();
                const uint32_t bar = bar_lfull(l);
                const int m0 = c.m0(), k0c = c.k0();
                if (leader) {
                    if (p.box3d) ptx::tma_load_3d(x_tile(l, 0), &tmap_x, 0, m0, k0c >> 6, bar);
                    else
                        for (int j = 0; j < kc; ++j) ptx::tma_load_2d(x_tile(l, j), &tmap_x, k0c + j * BLOCK_K, m0, bar);
                }
            };
            ChunkIter it(p, ub, ue);
            if (p.await.flags != nullptr && it.valid()) {
                // The activation is still arriving from the other ranks. Fill the ring with weights first, then wait
                // (bounded) for every peer's flag, then fetch the activation tiles of those chunks.
                ChunkIter first(it);
                int n = 0;
                for (; it.valid() && n < LS; it.next(), ++n) issue_w(it);
                const uint32_t epoch = *p.await.epoch;
                const uint64_t t0 = ptx::globaltimer_ns();
                bool arrived = true;                       // lane r watches rank r's flag: the polls overlap
                if (lane < p.await.world && lane != p.await.rank) {
                    uint32_t seen;
                    do {
                        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(p.await.flags + lane) : "memory");
                        if ((int32_t)(seen - epoch) >= 0) break;
                        if (ptx::globaltimer_ns() - t0 > WAIT_LIMIT_NS) {
                            *abort_flag = 1;
                            if (p.status) atomicCAS(p.status, 0, (int)(0x20000 | (lane << 8) | (epoch & 0xff)));
                            arrived = false;
                            break;
                        }
                    } while (true);
                }
                if (!__all_sync(0xffffffffu, arrived)) ok = false;
                asm volatile("fence.proxy.async.global;" ::: "memory");      // peers' stores, seen through the flags, before the TMA reads
                for (int i = 0; i < n; ++i, first.next()) issue_x(first);   // also after a failed wait: the armed barriers must complete
                __syncwarp();
            }
            for (; it.valid() && ok; it.next()) {
                if (it.ci >= LS && !wait_done(it.ci - LS, ROLE_TMA)) { ok = false; break; }
                issue_w(it);
                issue_x(it);
                __syncwarp();
            }
            if (!ok) {
                // Let the copies already in flight land before the CTA goes away.
                const int ci = it.ci;
                for (int cj = max(0, ci - LS); cj < ci; ++cj) {
                    const uint64_t t0 = ptx::globaltimer_ns();
                    while (!ptx::mbar_try_wait(bar_lfull(cj % LS), (uint32_t)(cj / LS) & 1u) &&
                           ptx::globaltimer_ns() - t0 < WAIT_LIMIT_NS) {}
                }
            }
        }
    } else if (warp == WARP_MMA) {
        // ------------------------------------------------------------ MMA issuer
        // The whole warp runs the loop, so that control flow and descriptor arithmetic are warp-uniform (a
        // single-lane branch forces them onto per-thread registers, each instruction waiting for the one
        // before: measured ~200 cycles per MMA); one elected lane issues the MMAs and the commit.
        const bool leader = ptx::elect_one();
        constexpr uint32_t FMT = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
        // The MMA's N is the batch rows that were loaded, rounded up to the 16 the instruction wants
        // (columns past the loaded rows see whatever follows in the ring and are never read back; an
        // accumulator column depends on its own batch row only, whatever N is).
        const uint32_t mma_n = (uint32_t)((p.x_rows + 15) & ~15);
        const uint32_t IDESC = (1u << 4) | (FMT << 7) | (FMT << 10) | ((mma_n >> 3) << 17) |
                               ((uint32_t)(BLOCK_N >> 4) << 24);
        // Operand descriptors: constant bits + the tile's shared address in 16-byte units. One K step of 64 is
        // one tile further (W: 1024 units, x: x_bytes / 16), a UMMA K step of 16 elements +32 bytes = +2.
        const uint64_t da0 = ptx::smem_desc_sw128(w_ring), db0 = ptx::smem_desc_sw128(smem_base);
        const uint32_t xstep = (uint32_t)p.x_bytes >> 4;
        constexpr uint32_t WSTEP = W_TILE_BYTES >> 4;
        int job = -1; bool ok = true;
        uint32_t tmem_d = tmem_base;
        if (p.uniform) {
            // Every chunk is one whole K group with its own accumulator: nothing to enumerate but ring positions.
            const int nch = (ue - ub) * (p.split ? 1 : p.G);
            int l = 0, w = 0, d = 0;
            uint32_t lph = 0, wph = 0;
            const int wring = QBITS ? WS : LS;
            uint64_t db_c = db0;
            uint64_t da_c = da0;
            uint32_t ta_c = tmem_base + (uint32_t)p.a_col0;
            for (int ci = 0; ci < nch && ok; ++ci) {
                const int buf = ci & 1;
                if (!wait_bounded(bar_tempty(buf), (uint32_t)((ci >> 1) & 1) ^ 1u, ctl, ROLE_MMA, 32 + buf)) { ok = false; break; }
                tmem_d = tmem_base + (uint32_t)(buf * p.acc_stride);
                if (!wait_bounded(QBITS ? bar_wfull(w) : bar_lfull(l), QBITS ? wph : lph, ctl, ROLE_MMA, QBITS ? 8 + w : l)) { ok = false; break; }
                ptx::tc_fence_after();
                if (leader) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint64_t db = db_c + (uint64_t)((uint32_t)j * xstep);
                        if constexpr (TSA) {
                            const uint32_t ta = ta_c + (uint32_t)(j * TMEM_A_STEP);
                            if (j == 0) ptx::umma_f16_ts_c<false>(tmem_d, ta, db, IDESC);
                            else        ptx::umma_f16_ts_c<true>(tmem_d, ta, db, IDESC);
                            ptx::umma_f16_ts_c<true>(tmem_d, ta + 8, db + 2, IDESC);
                            ptx::umma_f16_ts_c<true>(tmem_d, ta + 16, db + 4, IDESC);
                            ptx::umma_f16_ts_c<true>(tmem_d, ta + 24, db + 6, IDESC);
                        } else {
                            const uint64_t da = da_c + (uint64_t)(j * WSTEP);
                            if (j == 0) ptx::umma_f16_c<false>(tmem_d, da, db, IDESC);
                            else        ptx::umma_f16_c<true>(tmem_d, da, db, IDESC);
                            ptx::umma_f16_c<true>(tmem_d, da + 2, db + 2, IDESC);
                            ptx::umma_f16_c<true>(tmem_d, da + 4, db + 4, IDESC);
                            ptx::umma_f16_c<true>(tmem_d, da + 6, db + 6, IDESC);
                        }
                    }
                    ptx::umma_commit(bar_done(d));
                }
                __syncwarp();
                if (++d == MAX_SLOTS) d = 0;
                if (++l == LS) { l = 0; lph ^= 1u; }
                if (++w == wring) { w = 0; wph ^= 1u; }
                db_c = db0 + (uint64_t)((uint32_t)(l * 4) * xstep);
                da_c = da0 + (uint64_t)((uint32_t)((QBITS ? w : l) * 4) * WSTEP);
                ta_c = tmem_base + (uint32_t)(p.a_col0 + w * 4 * TMEM_A_STEP);
            }
        }
        for (ChunkIter it(p, ub, ue); !p.uniform && it.valid() && ok; it.next()) {
            if (it.first_in_group()) {
                ++job;
                const int buf = job & 1;
                if (!wait_bounded(bar_tempty(buf), (uint32_t)((job >> 1) & 1) ^ 1u, ctl, ROLE_MMA, 32 + buf)) { ok = false; break; }
                tmem_d = tmem_base + (uint32_t)(buf * p.acc_stride);
            }
            const int l = it.l, w = it.w;
            const uint32_t ready = QBITS ? bar_wfull(w) : bar_lfull(l);
            if (!wait_bounded(ready, QBITS ? it.wph : it.lph, ctl, ROLE_MMA, QBITS ? 8 + w : l)) { ok = false; break; }
            ptx::tc_fence_after();
            const int kc = it.ksteps();
            const uint64_t db_c = db0 + (uint64_t)((uint32_t)(l * KS) * xstep);
            const uint64_t da_c = da0 + (uint64_t)((uint32_t)((QBITS ? w : l) * KS) * WSTEP);
            const uint32_t ta_c = tmem_base + (uint32_t)(p.a_col0 + w * KS * TMEM_A_STEP);
            (void)da_c; (void)ta_c;
            if (p.box3d) {
                // K % 64 == 0: every K step of the chunk is whole -- four MMAs each, offsets known at compile time
#pragma unroll 1
                for (int j = 0; j < kc; ++j) {
                    const uint64_t db = db_c + (uint64_t)((uint32_t)j * xstep);
                    const uint32_t acc0 = (it.c | j) ? 1u : 0u;
                    if constexpr (TSA) {
                        const uint32_t ta = ta_c + (uint32_t)(j * TMEM_A_STEP);
                        if (leader) {
                            ptx::umma_f16_ts(tmem_d, ta, db, IDESC, acc0);
                            ptx::umma_f16_ts_c<true>(tmem_d, ta + 8, db + 2, IDESC);
                            ptx::umma_f16_ts_c<true>(tmem_d, ta + 16, db + 4, IDESC);
                            ptx::umma_f16_ts_c<true>(tmem_d, ta + 24, db + 6, IDESC);
                        }
                    } else {
                        const uint64_t da = da_c + (uint64_t)((uint32_t)j * WSTEP);
                        if (leader) {
                            ptx::umma_f16(tmem_d, da, db, IDESC, acc0);
                            ptx::umma_f16_c<true>(tmem_d, da + 2, db + 2, IDESC);
                            ptx::umma_f16_c<true>(tmem_d, da + 4, db + 4, IDESC);
                            ptx::umma_f16_c<true>(tmem_d, da + 6, db + 6, IDESC);
                        }
                    }
                }
            } else {
                const int kend = min(p.K, (it.g + 1) * GROUP_K);
                for (int j = 0; j < kc; ++j) {
                    const int kleft = kend - (it.k0() + j * BLOCK_K);
                    const int nsteps = kleft >= BLOCK_K ? BLOCK_K / UMMA_K : (kleft + UMMA_K - 1) / UMMA_K;
                    const uint64_t db = db_c + (uint64_t)((uint32_t)j * xstep);
                    const uint64_t da = da_c + (uint64_t)((uint32_t)j * WSTEP);
                    for (int kk = 0; kk < nsteps; ++kk)
                        if (leader) ptx::umma_f16(tmem_d, da + 2 * kk, db + 2 * kk, IDESC, (it.c | j | kk) ? 1u : 0u);
                }
            }
            if (leader) ptx::umma_commit(bar_done(it.d));
            __syncwarp();
        }
    } else if (warp >= WARP_EPI0 && warp < WARP_EPI0 + 4) {
        // ------------------------------------------------------------ epilogue
        const int quad = warp & 3;  // TMEM lanes this warp may touch: 32*quad .. 32*quad+31
        const int row = quad * 32 + lane;
        const uint32_t lane_base = tmem_base + ((uint32_t)(quad * 32) << 16);
        int job = -1; bool ok = true;
        uint32_t epi_ph = 0;
        // the four epilogue warps meet (bounded, like every other wait of the kernel)
        auto epi_sync = [&]() {
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(bar_epi);
            const bool r = wait_bounded(bar_epi, epi_ph, ctl, ROLE_EPI, 40);
            epi_ph ^= 1u;
            return r;
        };
        T* out = static_cast<T*>(p.out);
        const T* bias = static_cast<const T*>(p.bias);
        float small_total[8];                                        // running totals of a tile of at most 8 batch rows (fused)
#pragma unroll
        for (int j = 0; j < 8; ++j) small_total[j] = 0.0f;
        for (ChunkIter it(p, ub, ue); it.valid() && ok; it.next()) {
            if (it.first_in_group()) ++job;
            if (!it.last_in_group()) continue;
            const int buf = job & 1;
            if (!wait_bounded(bar_done(it.d), it.dph, ctl, ROLE_EPI, 16 + it.d)) { ok = false; break; }
            ptx::tc_fence_after();
            const int g = it.g;
            const int n = it.n0() + row;
            const int m0 = it.m0();
            const int ncols = min(p.bm, p.M - m0);
            const uint32_t acc = lane_base + (uint32_t)(buf * p.acc_stride);
            const bool first = g == 0, last = g == p.G - 1;
            if (ncols <= 8) {
                // Few batch rows (decode): a narrow accumulator read, and in the fused shape the running totals
                // stay in registers from group to group -- no round trip through tensor memory.
                {
                    constexpr int W = 8;
                    uint32_t v[W];
                    ptx::tmem_ld_32x8(acc, v);
                    ptx::tmem_ld_wait();
                    ptx::tc_fence_before();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(bar_tempty(buf));          // the accumulator is in registers
                    if (p.split) {
                        if (n < p.N) {
                            float* dst = p.part + ((long long)g * p.M + m0) * p.N + n;
#pragma unroll
                            for (int j = 0; j < W; ++j)
                                if (j < ncols) dst[(long long)j * p.N] = __uint_as_float(v[j]);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < W; ++j) small_total[j] = add_rn(first ? 0.0f : small_total[j], __uint_as_float(v[j]));
                        if (last && n < p.N) {
#pragma unroll
                            for (int j = 0; j < W; ++j)
                                if (j < ncols) out[(long long)(m0 + j) * p.N + n] = round_out<T>(small_total[j], bias, n);
                        }
                    }
                }
            } else if (p.split) {
                // A TMEM load queues behind the MMAs already issued for the next unit, so the loads of two
                // column blocks go out together and pay that wait once (the streaming variant, short of
                // registers with its sixteen dequantizer warps, takes one block at a time).
#pragma unroll 1
                for (int c = 0; c * 32 < ncols; c += (TSA ? 1 : 2)) {  // warp-uniform trip count
                    uint32_t v0[32], v1[TSA ? 1 : 32];
                    const bool two = !TSA && (c + 1) * 32 < ncols;
                    ptx::tmem_ld_32x32(acc + c * 32, v0);
                    if constexpr (!TSA) { if (two) ptx::tmem_ld_32x32(acc + c * 32 + 32, v1); }
                    ptx::tmem_ld_wait();
                    if ((c + (TSA ? 1 : 2)) * 32 >= ncols) {
                        // the accumulator is in registers: hand it back before the stores go out
                        ptx::tc_fence_before();
                        __syncwarp();
                        if (lane == 0) ptx::mbar_arrive(bar_tempty(buf));
                    }
                    if (n < p.N) {
                        float* dst = p.part + ((long long)g * p.M + m0 + c * 32) * p.N + n;
                        const int left = ncols - c * 32;
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (j < left) dst[(long long)j * p.N] = __uint_as_float(v0[j]);
                        if constexpr (!TSA) {
                            if (two) {
#pragma unroll
                                for (int j = 0; j < 32; ++j)
                                    if (32 + j < left) dst[(long long)(32 + j) * p.N] = __uint_as_float(v1[j]);
                            }
                        }
                    }
                }
            }
            if (p.split && p.counters) {
                // In-kernel fold. Every thread's partial stores are fenced device-wide, the four warps meet,
                // one thread counts this unit in; the CTA that counts in last (all G partials of the tile are
                // then visible) folds them in ascending g and writes the output. The counter goes back to 0.
                __threadfence();
                if (!epi_sync()) { ok = false; break; }
                if (warp == WARP_EPI0 && lane == 0) {
                    unsigned* ctr = p.counters + ((long long)it.nt * p.m_tiles + it.mt);
                    const unsigned old = atomicAdd(ctr, 1u);
                    const int mine = old == (unsigned)p.G - 1u;
                    if (mine) atomicExch(ctr, 0u);
                    *fold_flag = mine;
                }
                if (!epi_sync()) { ok = false; break; }
                if (*fold_flag) {
                    __threadfence();
                    if (n < p.N) {
                        const long long gstride = (long long)p.M * p.N;
#pragma unroll 1
                        for (int mm = 0; mm < ncols; mm += 4) {
                            const float* src = p.part + (long long)(m0 + mm) * p.N + n;
                            float tot[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll 4
                            for (int gg = 0; gg < p.G; ++gg) {
                                float v[4];
#pragma unroll
                                for (int u = 0; u < 4; ++u)
                                    v[u] = (mm + u < ncols) ? __ldcg(src + gg * gstride + (long long)u * p.N) : 0.0f;
#pragma unroll
                                for (int u = 0; u < 4; ++u) tot[u] = add_rn(tot[u], v[u]);
                            }
#pragma unroll
                            for (int u = 0; u < 4; ++u)
                                if (mm + u < ncols) out[(long long)(m0 + mm + u) * p.N + n] = round_out<T>(tot[u], bias, n);
                        }
                    }
                }
            }
            // fused: the running total lives in TMEM; total = total + p_g, from an exact 0. EW columns at a time
            // (16 in the streaming variant, which is short of registers).
            constexpr int EW = TSA ? 16 : 32;
#pragma unroll 1
            for (int c = 0; !p.split && ncols > 8 && c * EW < ncols; ++c) {  // warp-uniform trip count
                uint32_t v[EW], t[EW];
                if constexpr (TSA) {
                    ptx::tmem_ld_32x16(acc + c * EW, v);
                    if (!first) ptx::tmem_ld_32x16(lane_base + tmem_total + c * EW, t);
                } else {
                    ptx::tmem_ld_32x32(acc + c * EW, v);
                    if (!first) ptx::tmem_ld_32x32(lane_base + tmem_total + c * EW, t);
                }
                ptx::tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < EW; ++j)
                    t[j] = __float_as_uint(add_rn(first ? 0.0f : __uint_as_float(t[j]), __uint_as_float(v[j])));
                if (last) {
                    if (n < p.N) {
#pragma unroll
                        for (int j = 0; j < EW; ++j) {
                            const int m = m0 + c * EW + j;
                            if (c * EW + j < ncols) out[(long long)m * p.N + n] = round_out<T>(__uint_as_float(t[j]), bias, n);
                        }
                    }
                } else {
                    if constexpr (TSA) ptx::tmem_st_32x16(lane_base + tmem_total + c * EW, t);
                    else ptx::tmem_st_32x32(lane_base + tmem_total + c * EW, t);
                }
            }
            if (!p.split && ncols > 8) {
                if (!last) ptx::tmem_st_wait();
                ptx::tc_fence_before();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(bar_tempty(buf));
            }
        }
    } else if (QBITS && !TSA && warp >= WARP_DEQ0) {
        // ------------------------------------------------------------ dequantizers (tile body)
        // 256 threads: thread t turns half a weight row (32 codes) of every K step into four
        // 16-byte chunks of the swizzled tile. Two threads per row; its stores spread over all banks.
        constexpr int QB = QBITS ? QBITS : 4;
        constexpr int ROW_BYTES = BLOCK_K * QB / 8;     // packed bytes per weight row per K step
        constexpr int HALF_WORDS = ROW_BYTES / 8;       // 32-bit words behind 32 codes
        constexpr int WORDS_PER_CHUNK = QB / 4;
        const int t = threadIdx.x - WARP_DEQ0 * 32;
        const int row = t >> 1, half = t & 1;
        const T* scales = static_cast<const T*>(p.scales);
        const T* biases = static_cast<const T*>(p.biases);
        const int groups_per_row = p.K / p.gs;
        const int per_group = GROUP_K / p.gs;              // 8, 4 or 2 quantization groups per K group
        const int gs_shift = p.gs == 32 ? 5 : (p.gs == 64 ? 6 : 7);
        // Scale / bias entries of one K group (8, 4 or 2 of them), kept as the packed 16-bit words they are
        // in memory: fetched with one vector load each, a whole K group ahead of their use.
        const bool sb_vec = (groups_per_row * (int)sizeof(T)) % 16 == 0 && ((uintptr_t)scales % 16) == 0 && ((uintptr_t)biases % 16) == 0;
        auto fetch = [&](int n, int g, uint32_t (&sw)[4], uint32_t (&bw)[4]) {
#pragma unroll
            for (int i = 0; i < 4; ++i) { sw[i] = 0u; bw[i] = 0u; }
            if (n >= p.N) return;
            const int q0 = g * per_group;
            const int have = min(per_group, groups_per_row - q0);
            const T* sp = scales + (long long)n * groups_per_row + q0;
            const T* bp = biases + (long long)n * groups_per_row + q0;
            if (sb_vec && have == per_group) {
                if (per_group == 8) {
                    const uint4 a = __ldg(reinterpret_cast<const uint4*>(sp)), b = __ldg(reinterpret_cast<const uint4*>(bp));
                    sw[0] = a.x; sw[1] = a.y; sw[2] = a.z; sw[3] = a.w; bw[0] = b.x; bw[1] = b.y; bw[2] = b.z; bw[3] = b.w;
                } else if (per_group == 4) {
                    const uint2 a = __ldg(reinterpret_cast<const uint2*>(sp)), b = __ldg(reinterpret_cast<const uint2*>(bp));
                    sw[0] = a.x; sw[1] = a.y; bw[0] = b.x; bw[1] = b.y;
                } else {
                    sw[0] = __ldg(reinterpret_cast<const uint32_t*>(sp)); bw[0] = __ldg(reinterpret_cast<const uint32_t*>(bp));
                }
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    if (i < have) {
                        sw[i >> 1] |= (uint32_t)reinterpret_cast<const unsigned short*>(sp)[i] << (16 * (i & 1));
                        bw[i >> 1] |= (uint32_t)reinterpret_cast<const unsigned short*>(bp)[i] << (16 * (i & 1));
                    }
                }
            }
        };
        auto entry = [&](const uint32_t (&wds)[4], int qi) {   // float(entry qi) of a fetched group
            uint32_t wd = wds[0];
            if ((qi >> 1) == 1) wd = wds[1];
            if ((qi >> 1) == 2) wd = wds[2];
            if ((qi >> 1) == 3) wd = wds[3];
            const unsigned short h = (unsigned short)((qi & 1) ? (wd >> 16) : (wd & 0xffffu));
            T tv;
            *reinterpret_cast<unsigned short*>(&tv) = h;
            return Cvt<T>::up(tv);
        };
        uint32_t sw[4] = {0u, 0u, 0u, 0u}, bw[4] = {0u, 0u, 0u, 0u};      // current K group
        uint32_t sw_n[4], bw_n[4];                                        // next K group, in flight
        {
            ChunkIter first(p, ub, ue);
            if (first.valid()) fetch(first.n0() + row, first.g, sw_n, bw_n);
            else { for (int i = 0; i < 4; ++i) { sw_n[i] = 0u; bw_n[i] = 0u; } }
        }
        bool ok = true;
        for (ChunkIter it(p, ub, ue); it.valid() && ok; it.next()) {
            if (it.first_in_group()) {
#pragma unroll
                for (int i = 0; i < 4; ++i) { sw[i] = sw_n[i]; bw[i] = bw_n[i]; }
                ChunkIter nx(it);
                do { nx.next(); } while (nx.valid() && !nx.first_in_group());
                if (nx.valid()) fetch(nx.n0() + row, nx.g, sw_n, bw_n);
            }
            const int l = it.l, w = it.w;
            if (!wait_bounded(bar_lfull(l), it.lph, ctl, ROLE_DEQ, l)) { ok = false; break; }
            if (it.ci >= WS && !wait_done(it.ci - WS, ROLE_DEQ)) { ok = false; break; }
            const int kc = it.ksteps();
            for (int j = 0; j < kc; ++j) {
                const int qi = ((it.c * KS + j) * BLOCK_K + half * 32) >> gs_shift;  // index inside this K group
                const float sc = entry(sw, qi), bs = entry(bw, qi);
                const uint64_t s2 = ptx::pack2(sc, sc), b2 = ptx::pack2(bs, bs);
                const uint8_t* raw = smem_gen + (raw_chunk(l) - smem_base);
                constexpr int HALF_PIECES = HALF_WORDS / 4;      // 16-byte pieces behind 32 codes: 1 (4-bit) or 2 (8-bit)
                uint32_t rw[HALF_WORDS];
#pragma unroll
                for (int i = 0; i < HALF_PIECES; ++i) {
                    const uint4 q = *reinterpret_cast<const uint4*>(raw + raw_piece_offset(row, (j * 2 + half) * HALF_PIECES + i, p.raw_span));
                    rw[4 * i] = q.x; rw[4 * i + 1] = q.y; rw[4 * i + 2] = q.z; rw[4 * i + 3] = q.w;
                }
                uint8_t* wt = smem_gen + (w_tile(w, j) - smem_base) + row * 128;
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) {
                    const int c = half * 4 + jj;
                    const uint4 o = dequant8<T, QB>(&rw[jj * WORDS_PER_CHUNK], s2, b2);
                    *reinterpret_cast<uint4*>(wt + ((c ^ (row & 7)) << 4)) = o;
                }
            }
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(bar_wfull(w));
        }
    } else if (QBITS && TSA && warp >= WARP_DEQ0) {
        // ------------------------------------------------------------ dequantizers (streaming)
        // Sixteen warps. A warp may touch the 32 tensor-memory lanes of its quadrant (warp index mod 4)
        // only, so the four warps of a quadrant share its 32 weight rows by K step: warp (quadrant, j)
        // dequantizes K step j of every chunk -- one row, 64 codes, per thread -- and writes the 32
        // packed columns with one tcgen05.st. Scales and biases are read straight from global memory,
        // DEPTH chunks ahead of their use (a register queue), through the L1.
        constexpr int QB = QBITS ? QBITS : 4;
        constexpr int DEPTH = 2;   // chunks between a scale load and its use (each load touches 32 lines: a deeper queue only lengthens the burst before the first chunk)
        const int dw = warp - WARP_DEQ0;
        const int quad = warp & 3;
        const int jstep = dw >> 2;                                           // 0..3
        const int row = quad * 32 + lane;
        const unsigned short* scales = static_cast<const unsigned short*>(p.scales);
        const unsigned short* biases = static_cast<const unsigned short*>(p.biases);
        const int groups_per_row = p.K / p.gs;
        const int gs_shift = p.gs == 32 ? 5 : (p.gs == 64 ? 6 : 7);
        const bool two_entries = p.gs == 32;                                 // a K step of 64 spans two quantization groups
        // entries of (row n, K step starting at k): low half = first entry, high half = second (gs 32) or the same
        auto fetch = [&](const ChunkIter& c, uint32_t& sv, uint32_t& bv) {
            // Only the loads are issued here. Nothing may touch the loaded value before the chunk it belongs to is
            // dequantized, DEPTH chunks later: an instruction that uses it now would wait out the whole memory
            // latency in every iteration. No branches either: where there is nothing to fetch (past the last chunk,
            // a row beyond N, a K step the chunk does not have) entry 0 is loaded and never used for a stored output.
            const int n = c.n0() + row;
            const bool on = c.valid() && n < p.N && jstep < c.ksteps();
            const long long e = on ? (long long)n * groups_per_row + ((c.k0() + jstep * BLOCK_K) >> gs_shift) : 0ll;
            if (two_entries) {
                sv = __ldg(reinterpret_cast<const unsigned int*>(scales + e));
                bv = __ldg(reinterpret_cast<const unsigned int*>(biases + e));
            } else {
                sv = __ldg(scales + e);
                bv = __ldg(biases + e);
            }
        };
        auto to_f = [&](uint32_t h) {
            T tv;
            *reinterpret_cast<unsigned short*>(&tv) = (unsigned short)h;
            return Cvt<T>::up(tv);
        };
        uint32_t qs[DEPTH], qb[DEPTH];
        ChunkIter pf(p, ub, ue);
#pragma unroll
        for (int i = 0; i < DEPTH; ++i) { fetch(pf, qs[i], qb[i]); pf.next(); }
        const uint32_t a_lane = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)p.a_col0;
        bool ok = true;
        ChunkIter it(p, ub, ue);
        while (it.valid() && ok) {
            uint32_t sv = qs[0], bv = qb[0];
            if (!two_entries) { sv |= sv << 16; bv |= bv << 16; }             // one entry per K step: both halves use it
#pragma unroll
            for (int i = 0; i + 1 < DEPTH; ++i) { qs[i] = qs[i + 1]; qb[i] = qb[i + 1]; }
            const int l = it.l, w = it.w, kst = it.ksteps();
            if (!wait_bounded(bar_lfull(l), it.lph, ctl, ROLE_DEQ, l)) { ok = false; break; }
            if (it.ci >= WS && !wait_done(it.ci - WS, ROLE_DEQ)) { ok = false; break; }
            // The state of the next iteration and the scale prefetch do not depend on this chunk's data: placed in
            // front of the arithmetic, in the same basic block, their dependent scalar chains issue in its shadow.
            auto advance = [&]() {
                it.next();
                fetch(pf, qs[DEPTH - 1], qb[DEPTH - 1]);
                pf.next();
            };
            if (jstep < kst) {
                advance();
                ptx::tc_fence_after();
                const float s0 = to_f(sv & 0xffffu), s1 = to_f(sv >> 16), b0 = to_f(bv & 0xffffu), b1 = to_f(bv >> 16);
                dequant_row64_to_tmem<T, QB>(smem_gen + (raw_chunk(l) - smem_base), row, jstep, ptx::pack2(s0, s0), ptx::pack2(b0, b0),
                                             ptx::pack2(s1, s1), ptx::pack2(b1, b1),
                                             a_lane + (uint32_t)((w * KS + jstep) * TMEM_A_STEP));
                ptx::tmem_st_wait();
            } else {
                advance();
            }
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(bar_wfull(w));
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

// The same tensor seen as [K/64 blocks][rows][inner elements] (needs K % 64 == 0; inner = the elements that hold
// 64 values of K: 64 for 16-bit data, 8 or 16 words for packed codes): a box of `depth` blocks lands as `depth`
// consecutive K-step tiles of box_rows x (inner * esize) bytes.
int make_map3(CUtensorMap* m, CUtensorMapDataType dt, size_t esize, const void* base, uint64_t kblocks, uint64_t rows,
              uint64_t ld, uint32_t box_rows, uint32_t depth, uint32_t inner = BLOCK_K,
              CUtensorMapSwizzle sw = CU_TENSOR_MAP_SWIZZLE_128B) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(BI_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t gdim[3] = {(cuuint64_t)inner, rows, kblocks};
    cuuint64_t gstr[2] = {ld * esize, (cuuint64_t)inner * esize};
    cuuint32_t box[3] = {(cuuint32_t)inner, box_rows, depth};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(m, dt, 3, const_cast<void*>(base), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(BI_ERR_CUDA, "cuTensorMapEncodeTiled (3-D) failed with CUresult %d", (int)r);
    return BI_OK;
}

// Chunk size and ring depths from the shared-memory budget (a launch-shape choice; no arithmetic
// depends on it): the largest chunk that still leaves at least two slots in every ring. Measured: larger
// chunks beat deeper rings (each chunk costs the MMA thread one commit and one pass of its loop).
// raw_bytes: packed codes per K step of a quantized weight tile, 0 for dense weights.
// tsa: streaming quantized variant (weight operand in tensor memory: its ring of two chunks takes no shared memory).
bool pick_rings(Params& p, int raw_bytes, bool tsa) {
    const bool quant = raw_bytes != 0;
    const int avail = (tsa ? TSA_SMEM_CAP : SMEM_LIMIT) - 1024 - BAR_BYTES;
    p.w_slots = quant ? 2 : 0;
    p.ks = 0;
    for (int ks = 4; ks >= (tsa ? 4 : 1); ks >>= 1) {
        const int wring = (tsa ? 0 : p.w_slots) * ks * W_TILE_BYTES;
        const int slot = ks * (p.x_bytes + (quant ? raw_bytes : W_TILE_BYTES));
        const int ls = (avail - wring) / slot;
        if (ls >= 2) { p.ks = ks; p.load_slots = ls < MAX_SLOTS ? ls : MAX_SLOTS; break; }
    }
    if (!p.ks) return false;
    p.w_ring_slots = quant ? p.w_slots : p.load_slots;
    p.smem_bytes = 1024 + BAR_BYTES + p.load_slots * p.ks * (p.x_bytes + raw_bytes) +
                   (quant ? (tsa ? 0 : p.w_slots) : p.load_slots) * p.ks * W_TILE_BYTES;
    return true;
}

template <typename T, int QBITS, bool TSA>
int launch_t(const CUtensorMap& mw, const CUtensorMap& mx, const Params& p, cudaStream_t st) {
    using C = Cfg<QBITS, TSA>;
    auto kern = tc_matmul_kernel<T, QBITS, TSA>;
    static bool attr_done[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (!attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT);
        if (e != cudaSuccess) return fail(BI_ERR_CUDA, "matmul smem attr: %s", cudaGetErrorString(e));
        attr_done[dev] = true;
    }
    // Units go to CTAs in equal contiguous shares. With few units per CTA an uneven share costs a
    // whole unit on the critical path (224 tiles on 148 CTAs: some take two, the rest idle half the time), so
    // the grid shrinks to the largest size at which every CTA gets the same count.
    const long long sms = sm_count();
    long long grid = p.units < sms ? p.units : sms;
    const long long waves = (p.units + sms - 1) / sms;
    if (waves >= 2 && waves <= 16) grid = (p.units + waves - 1) / waves;
    launch_overlapped(kern, dim3((unsigned)grid), dim3(C::THREADS), p.smem_bytes, st, mw, mx, p);
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
                     float* part, int64_t M, int64_t N, int64_t K, int dtype, const TcShape& shape, int32_t* status,
                     cudaStream_t st) {
    const bool quant = q && q->codes;
    const bool split = shape.split;
    const int bm = shape.bm;
    if (bm != 16 && bm != 32 && bm != 64 && bm != BLOCK_M) return fail(BI_ERR_BAD_ARG, "matmul: batch tile %d (16, 32, 64 or 128)", bm);
    Params p{};
    p.out = out; p.part = part; p.status = status;
    p.await = shape.await;
    p.bias = shape.bias;
    p.counters = split ? shape.counters : nullptr;
    p.scales = quant ? q->scales : nullptr; p.biases = quant ? q->biases : nullptr;
    p.M = (int)M; p.N = (int)N; p.K = (int)K;
    p.G = (int)((K + GROUP_K - 1) / GROUP_K);
    p.bm = bm;
    p.n_tiles = (int)((N + BLOCK_N - 1) / BLOCK_N);
    p.m_tiles = (int)((M + bm - 1) / bm);
    p.split = split ? 1 : 0;
    p.gs = quant ? q->gs : 0;
    p.units = (long long)p.n_tiles * p.m_tiles * (split ? p.G : 1);
    if (p.units >= (1LL << 31)) return fail(BI_ERR_UNSUPPORTED, "matmul: %lld work units exceed the kernel's 32-bit unit index", p.units);
    // Only the batch rows that exist are loaded; the box height is a launch-shape choice.
    const int64_t mr = M < bm ? ((M + 7) / 8) * 8 : bm;
    p.x_rows = (int)mr;
    p.x_bytes = ((int)mr * BLOCK_K * 2 + 1023) / 1024 * 1024;
    p.box3d = K % BLOCK_K == 0 ? 1 : 0;
    // Quantized weights: the streaming staging (weight operand in tensor memory) serves batch tiles of up to
    // 64 rows, the tile body the rest. Same MMA sequence on the same operand values either way.
    bool tsa = quant && mr <= 64 && p.box3d && shape.stage != TcShape::STAGE_SMEM;
    if (quant && shape.stage == TcShape::STAGE_TMEM && !tsa)
        return fail(BI_ERR_UNSUPPORTED, "qmm: the tensor-memory staging needs a batch tile of at most 64 rows");

    if (!pick_rings(p, quant ? BLOCK_N * BLOCK_K * q->bits / 8 : 0, tsa)) {
        if (!tsa || shape.stage == TcShape::STAGE_TMEM || !pick_rings(p, BLOCK_N * BLOCK_K * q->bits / 8, false))
            return fail(BI_ERR_UNSUPPORTED, "matmul: no shared-memory configuration fits");
        tsa = false;
    }
    p.acc_stride = BLOCK_M;
    if (tsa) {
        // tensor-memory budget of the streaming variant: two accumulators + the running total, then the operand ring
        const bool small = mr <= 32;
        p.acc_stride = small ? 32 : 64;
        p.a_col0 = small ? 128 : 256;
        p.w_slots = p.w_ring_slots = small ? 3 : 2;
    }
    p.uniform = (K % GROUP_K == 0 && p.ks == 4) ? 1 : 0;

    const CUtensorMapDataType dt = dtype == BI_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUtensorMap mw, mx;
    int rc = BI_OK;
    if (p.box3d) {
        // A driver that refuses the 3-D view gets the per-K-step boxes instead; the bytes that land are the same.
        rc = make_map3(&mx, dt, 2, x, (uint64_t)(K / BLOCK_K), (uint64_t)M, (uint64_t)x_ld, (uint32_t)p.x_rows, (uint32_t)p.ks);
        if (!rc && !quant) rc = make_map3(&mw, dt, 2, w, (uint64_t)(K / BLOCK_K), (uint64_t)N, (uint64_t)w_ld, BLOCK_N, (uint32_t)p.ks);
        if (rc && tsa) return rc;
        if (rc) p.box3d = 0;
    }
    if (!p.box3d) {
        rc = make_map(&mx, dt, 2, x, (uint64_t)K, (uint64_t)M, (uint64_t)x_ld, BLOCK_K, (uint32_t)p.x_rows, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc) return rc;
        if (!quant) rc = make_map(&mw, dt, 2, w, (uint64_t)K, (uint64_t)N, (uint64_t)w_ld, BLOCK_K, BLOCK_N, CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc) return rc;
    }
    if (quant) {
        // A chunk's codes of one weight row are ks * 64 * bits / 8 bytes: one box per 128 of them.
        const uint64_t words = (uint64_t)K * q->bits / 32;
        const int chunk_row_bytes = p.ks * BLOCK_K * q->bits / 8;              // 32 .. 256
        p.raw_span = chunk_row_bytes < 128 ? chunk_row_bytes : 128;
        p.raw_boxes = chunk_row_bytes / p.raw_span;
        const CUtensorMapSwizzle sw = p.raw_span == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                                    : (p.raw_span == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
        rc = make_map(&mw, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, q->codes, words, (uint64_t)N, words, (uint32_t)(p.raw_span / 4),
                      BLOCK_N, sw);
        if (rc) return rc;
    }

#define BI_TC_LAUNCH(TT)                                                                                          \
    do {                                                                                                          \
        if (!quant) return launch_t<TT, 0, false>(mw, mx, p, st);                                                 \
        if (tsa) return q->bits == 4 ? launch_t<TT, 4, true>(mw, mx, p, st) : launch_t<TT, 8, true>(mw, mx, p, st); \
        return q->bits == 4 ? launch_t<TT, 4, false>(mw, mx, p, st) : launch_t<TT, 8, false>(mw, mx, p, st);      \
    } while (0)
    if (dtype == BI_BF16) BI_TC_LAUNCH(__nv_bfloat16);
    BI_TC_LAUNCH(__half);
#undef BI_TC_LAUNCH
}

}  // namespace bi
