// spg_gemv.cu -- K1: small-batch (1..8 rows) fused dequant-GEMV layer.
//
//   y[n][j] = act(bias[j] + w_scale * sum_k q[j][k] * x[n][k])
//
// The layer is bound by reading the packed weights once from HBM, so the kernel
// is a persistent weight stream: one CTA per SM walks a list of items, an item
// being 16 weight rows over the whole of K.  A producer thread keeps a ring of
// TMA boxes (16 rows x up to 256 bytes of the stored, still packed matrix; no
// multicast) in flight across item boundaries, so HBM never waits for a CTA to
// start up, and the eight boxes of a chunk are neighbours along K, so every
// row is read in contiguous kilobyte runs.  Each of the eight consumer warps
// takes one box of every chunk: a lane reads its two 128-bit row pieces from
// shared memory, expands the packed integers to bf16 in registers with
// mask/magic-number tricks (no per-element conversion instruction) and feeds the
// warp-level tensor path (mma.sync m16n8k16, bf16 x bf16 -> fp32) with the 16
// weight rows as M and the batch as N.  At the end of an item the eight partial
// accumulators meet in shared memory and scale, bias and activation are applied:
// no split-K traffic, no global synchronisation.
//
// To keep fp32-class accuracy the activations enter as two or three bf16 terms
// (x = x1 + x2 [+ x3]), each term in its own column of the N dimension, and
// weights that are not exact in bf16 enter as several exact bf16 terms too
// (INT8 = 16*high nibble + low nibble, FP16 = 8+3 bits, FP32 = 8+8+8 bits);
// integer and BF16 weights are exact in one term.  All products are exact; only
// the fp32 summation order differs from the reference's dot product
// (SIMD.c:190-240).
//
// The K order inside one MMA is arbitrary as long as both operands agree, so the
// activation terms are kept in global memory already in the order in which the
// mask tricks deliver the weights ("staged" input): a small kernel stages the
// first layer's input, and every later layer's input is staged by the epilogue
// of the layer before it.  A chunk's slice of the staged input reaches shared
// memory with one bulk copy and serves all eight warps.
//
// Integer path.  Files stored as INT8 / INT4 / INT2 take a cheaper route through the integer tensor
// path (mma.sync m16n8k32, u8/s8 -> s32): the packed weights become s8 operands with one or two
// logic operations per word (an INT4 nibble moved to the top of its byte IS 16*q in two's
// complement; INT8 bytes go in untouched), and each activation enters as four base-128 digits of a
// 28-bit fixed-point number V = round(x / S * (2^27 - 1)), one digit per column of N.  Integer
// accumulation is exact, so the only error is the fixed-point rounding of x (relative to the
// row's scale S).  S must be known before a layer's outputs exist, because the epilogue of layer l
// writes layer l+1's digits as the items finish: the first layer's S is the exact row maximum
// (the staging kernel computes it), later layers use the bound
//     |y_j| <= max|bias| + |w_scale| * max|q| * sum_k |x_k|
// whose last factor is exact integer arithmetic on the digits of the layer's input (each item
// leaves the partial sum of its |V| next to the staged data; no atomics, nothing to clear).
// The bound costs about seven of the 28 bits; what is left still exceeds bf16 hi+lo pairs.
//
// Scratch starts with a status word: it must be zero before first use.  Every
// mbarrier wait is bounded; on expiry the status word is set, waits turn into
// no-ops and the CTA runs to its end without computing further.
#include "spg_common.cuh"
#include <cuda.h>
#include <cstdio>
#include <mutex>

namespace {

constexpr int CONSUMER_WARPS = 16;         // two warps per 256-byte slice of a chunk (each takes half of its steps)
constexpr int CONSUMER_THREADS = 32 * CONSUMER_WARPS;
constexpr int GEMV_THREADS = CONSUMER_THREADS + 64;     // + one producer warp + one epilogue warp
constexpr int HANDOFF_THREADS = CONSUMER_THREADS + 32;  // parties of the consumer <-> epilogue named barriers
constexpr int ITEM_ROWS = 16;              // one MMA row group
constexpr int MAX_BATCH = 8;
constexpr uint32_t GEMV_WAIT_LIMIT = 1u << 22;
constexpr uint32_t HEAD_BYTES = 256;                     // status word at the start of scratch
constexpr int DIGITS = 4;                                // base-128 digits per activation on the integer path
constexpr double DIGIT_FULL = 134217727.0;               // 2^27 - 1: |V| <= this, so the top digit fits [-64, 63]
constexpr uint32_t INT_PATH_MAX_K = 131072;              // 127 * 128 * K must stay below 2^31

// Every staged-input buffer starts with a head: the scale of each batch row's digits, then (at byte 256)
// partial sums of |V| per producer item, int64 [nparts][8].  The bf16 path leaves the head unused.
struct StagedHead { float S[8]; uint32_t nparts; uint32_t pad[7]; };
__host__ __device__ inline size_t staged_head_bytes(uint32_t width)
{
    const size_t parts = (size_t)(width + 15) / 16 + 33 + 160;      // staging blocks of the first layer, or one entry per CTA of a launch (at most one CTA per SM)
    return 256 + ((parts * 64 + 255) & ~(size_t)255);
}

struct GemvParams {
    const float *bias;
    float scale;
    uint32_t in, out;
    int act;
    float *y; uint32_t ldy;
    uint32_t N, P, C;                       // rows, bf16 terms per row, C = N*P columns in use
    uint32_t items;                         // row groups of 16
    uint32_t nboxes, nchunks;               // boxes along K per item; chunks of 8 boxes
    uint32_t spb, box_bytes;                // steps (64 bytes per row) per box; bytes of one box = 16 * spb * 64
    uint32_t ring, xdepth, xchunk_bytes;    // ring depth in chunks (weights + staged input travel together), bytes of staged input per chunk
    int32_t *status;
    const uint4 *xin;                       // this layer's staged input (see staged_index)
    __nv_bfloat16 *xout;                    // staged input of the next layer, written by the epilogue (or NULL)
    int next_prec; uint32_t next_kpad;      // precision of the next layer's weights; its K rounded up to a whole chunk
    const uint8_t *in_head;                 // integer path: head of this layer's staged input
    uint8_t *out_head;                      // integer path: head of the next layer's staged input (or NULL)
    float bias_absmax;                      // integer path: caller's bound of |bias|, checked against every bias used
    int softmax;                            // the layer ends in a row softmax: the CTA that finishes last applies it
};

// One launch may run a whole run of layers (same stored precision, same batch, each feeding the next): the CTAs
// keep streaming weights across the layer boundaries and only the staged input of a layer waits for the layer
// before it (a device-wide counter the epilogue warps bump when their share of a layer is done).
constexpr uint32_t MAX_CHAIN = 8;
struct ChainMaps { CUtensorMap m[MAX_CHAIN]; };
struct ChainParams {
    GemvParams L[MAX_CHAIN];
    uint32_t n;                             // layers in this launch (1 = the plain single-layer call)
    int32_t *sync;                          // [MAX_CHAIN] layer-done counters + [1] exit ticket, all zero between launches
};

// elements covered by one 128-bit load, per stored precision
template <int PREC> struct Fmt;
template <> struct Fmt<SPG_P_I4>   { static constexpr int EL = 32; };
template <> struct Fmt<SPG_P_I2>   { static constexpr int EL = 64; };
template <> struct Fmt<SPG_P_I8>   { static constexpr int EL = 16; };
template <> struct Fmt<SPG_P_BF16> { static constexpr int EL = 8; };
template <> struct Fmt<SPG_P_F16>  { static constexpr int EL = 8; };
template <> struct Fmt<SPG_P_F32>  { static constexpr int EL = 4; };

// Position of element e (0..EL-1 of a lane's 128-bit load) in fragment order: which 4-element
// B block it belongs to and where inside the block [b0.lo, b0.hi, b1.lo, b1.hi].
__device__ __forceinline__ void frag_pos(int prec, uint32_t e, uint32_t &block, uint32_t &r)
{
    if (prec == SPG_P_I4) {            // word j = 8 nibbles; masks deliver pairs (i, i+4)
        const uint32_t j = e >> 3, i = e & 7u, low = i & 3u;
        block = 2 * j + (low >> 1); r = (low & 1u) * 2 + (i >> 2);
    } else if (prec == SPG_P_I2) {     // word j = 16 crumbs; masks deliver pairs (i, i+8)
        const uint32_t j = e >> 4, i = e & 15u, low = i & 7u;
        block = 4 * j + (low >> 1); r = (low & 1u) * 2 + (i >> 3);
    } else if (prec == SPG_P_I8) {     // word j = 4 bytes; masks deliver pairs (i, i+2)
        const uint32_t j = e >> 2, i = e & 3u;
        block = j; r = (i & 1u) * 2 + (i >> 1);
    } else {                           // 16-bit and 32-bit floats keep their natural order
        block = e >> 2; r = e & 3u;
    }
}

// Index (in bf16 units) of activation element k, column `col`, inside a staged-input buffer laid out as
// [step][block][tile][t][cw columns][4]: the order in which the weight loads of a layer stored in
// precision `prec` consume it.  cs = columns kept (4, 8 or 16), cw = min(cs, 8) columns per tile.
// All the quantities below are powers of two (elements per load, columns per tile), so the index is shifts
// and masks: the epilogue warp computes it for every value it stages.
__device__ __forceinline__ uint32_t el_log2_of(int prec)
{
    return prec == SPG_P_I4 ? 5u : prec == SPG_P_I2 ? 6u : prec == SPG_P_I8 ? 4u : prec == SPG_P_F32 ? 2u : 3u;
}
__device__ __forceinline__ uint64_t staged_index(int prec, uint32_t cs, uint32_t k, uint32_t col)
{
    const uint32_t el2 = el_log2_of(prec), nb = 1u << (el2 - 2);
    const uint32_t cw2 = cs < 8 ? 2u : 3u, tiles = cs >> cw2;
    const uint32_t step = k >> (el2 + 2), rem = k & ((4u << el2) - 1u), tt = rem >> el2, e = rem & ((1u << el2) - 1u);
    uint32_t block, r;
    frag_pos(prec, e, block, r);
    const uint64_t slot = (((((uint64_t)step * nb + block) * tiles + (col >> cw2)) * 4 + tt) << cw2) + (col & ((1u << cw2) - 1u));
    return slot * 4 + r;
}

// Splits v into P bf16 terms (term i = round(v - earlier terms)) and stores them for columns n*P .. n*P+P-1.
__device__ __forceinline__ void stage_value(__nv_bfloat16 *dst, int prec, uint32_t cs, uint32_t k, uint32_t n, uint32_t P, float v)
{
    for (uint32_t q = 0; q < P; q++) {
        const __nv_bfloat16 h = __float2bfloat16_rn(v);
        dst[staged_index(prec, cs, k, n * P + q)] = h;
        v -= __bfloat162float(h);
    }
}

// Stages a whole activation matrix x[N][in] (fp32) for a layer of precision `prec`: one thread per k.
// Elements k in [in, kpad) and the unused columns are written as zero.
__global__ void __launch_bounds__(256)
spg_gemv_stage_kernel(const float *__restrict__ x, uint32_t ldx, uint32_t N, uint32_t P, uint32_t in, uint32_t kpad,
                      int prec, uint32_t cs, __nv_bfloat16 *__restrict__ dst)
{
    const uint32_t k = blockIdx.x * 256 + threadIdx.x;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");     // the layer kernel behind this one may start fetching weights
    if (k >= kpad) return;
    for (uint32_t n = 0; n < N; n++) stage_value(dst, prec, cs, k, n, P, k < in ? x[(uint64_t)n * ldx + k] : 0.0f);
    for (uint32_t col = N * P; col < cs; col++) dst[staged_index(prec, cs, k, col)] = __float2bfloat16_rn(0.0f);
}

// ---- integer path: staged layout and staging -------------------------------------------------
// Position of element e of a lane's 128-bit load: which k32 MMA of the step consumes it (m) and which
// byte of the lane's B pair {b0, b1} must hold the matching activation digit (r = 0..7).
__device__ __forceinline__ void frag_pos_int(int prec, uint32_t e, uint32_t &m, uint32_t &r)
{
    if (prec == SPG_P_I4) {            // word m = 8 nibbles: even nibbles feed a0 (b0), odd nibbles a2 (b1)
        const uint32_t i = e & 7u;
        m = e >> 3; r = (i & 1u) * 4 + (i >> 1);
    } else if (prec == SPG_P_I2) {     // word j = 16 crumbs, two MMAs: crumbs 0/1 of every byte, then crumbs 2/3
        const uint32_t j = e >> 4, i = e & 15u, c = i & 3u;
        m = 2 * j + (c >> 1); r = (c & 1u) * 4 + (i >> 2);
    } else {                           // INT8: words 2m and 2m+1 are a0 and a2
        m = e >> 3; r = e & 7u;
    }
}

// Byte index of activation element k, column `col` (col = row * DIGITS + digit) in an integer staged buffer:
// [step][mma][tile][t][cw columns][8 bytes].
__device__ __forceinline__ uint64_t staged_index_int(int prec, uint32_t cs, uint32_t k, uint32_t col)
{
    const uint32_t el2 = el_log2_of(prec), nbi = 1u << (el2 - 3);
    const uint32_t cw2 = cs < 8 ? 2u : 3u, tiles = cs >> cw2;
    const uint32_t step = k >> (el2 + 2), rem = k & ((4u << el2) - 1u), tt = rem >> el2, e = rem & ((1u << el2) - 1u);
    uint32_t m, r;
    frag_pos_int(prec, e, m, r);
    const uint64_t slot = (((((uint64_t)step * nbi + m) * tiles + (col >> cw2)) * 4 + tt) << cw2) + (col & ((1u << cw2) - 1u));
    return slot * 8 + r;
}

// Fixed-point value of v at scale inv = DIGIT_FULL / S (0 when S is 0 or v is not finite).
__device__ __forceinline__ long long fixed_of(float v, double inv)
{
    if (!(fabsf(v) <= 3.0e38f)) return 0;
    double f = (double)v * inv;
    f = f > DIGIT_FULL ? DIGIT_FULL : (f < -DIGIT_FULL ? -DIGIT_FULL : f);
    return __double2ll_rn(f);
}

// The same in fp32, for the epilogue: y has 24 significant bits, so nothing is lost (the clamp is the largest
// float below 2^27).
__device__ __forceinline__ long long fixed_of_f(float v, float inv)
{
    if (!(fabsf(v) <= 3.0e38f)) return 0;
    const float f = fminf(fmaxf(v * inv, -134217720.0f), 134217720.0f);
    return (long long)__float2int_rn(f);
}

// Stores the four digits of V (three unsigned 7-bit digits and a signed top digit) for row n.
__device__ __forceinline__ void stage_digits(uint8_t *dst, int prec, uint32_t cs, uint32_t k, uint32_t n, long long V)
{
#pragma unroll
    for (int d = 0; d < DIGITS; d++) {
        const long long sh = V >> (7 * d);
        dst[staged_index_int(prec, cs, k, n * DIGITS + d)] = (uint8_t)(d + 1 < DIGITS ? (sh & 127) : (sh & 255));
    }
}

// Stages x[N][in] for the integer path: every block finds each row's exact maximum itself (the rows are a
// few KB and sit in L2), then writes the digits of its 256 k and the sum of |V| over them.
__global__ void __launch_bounds__(256)
spg_gemv_stage_int_kernel(const float *__restrict__ x, uint32_t ldx, uint32_t N, uint32_t in, uint32_t kpad,
                          int prec, uint32_t cs, uint8_t *__restrict__ head_raw, uint8_t *__restrict__ dst)
{
    __shared__ float wmax[8];
    __shared__ long long wsum[8];
    __shared__ int wbad[8];
    StagedHead *head = reinterpret_cast<StagedHead *>(head_raw);
    long long *parts = reinterpret_cast<long long *>(head_raw + 256);
    const uint32_t k = blockIdx.x * 256 + threadIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");     // the layer kernel behind this one may start fetching weights
    for (uint32_t n = 0; n < N; n++) {
        const float *row = x + (uint64_t)n * ldx;
        float m = 0.0f;
        int bad = 0;
        for (uint32_t i = threadIdx.x; i < in; i += 256) {
            const float a = fabsf(row[i]);
            bad |= !(a <= 3.0e38f);
            m = fmaxf(m, a);
        }
        m = spg_warp_max(m);
        bad = __any_sync(0xFFFFFFFFu, bad);
        if (lane == 0) { wmax[warp] = m; wbad[warp] = bad; }
        __syncthreads();
        m = 0.0f; bad = 0;
        for (int w = 0; w < 8; w++) { m = fmaxf(m, wmax[w]); bad |= wbad[w]; }
        // a row holding an infinity or a NaN cannot be put on a fixed-point grid: its scale becomes NaN,
        // which turns every output of the row into NaN
        const float S = bad ? __int_as_float(0x7FC00000) : m;
        const double inv = (!bad && m > 0.0f) ? DIGIT_FULL / (double)m : 0.0;
        long long V = 0;
        if (k < kpad) {
            V = k < in ? fixed_of(row[k], inv) : 0;
            stage_digits(dst, prec, cs, k, n, V);
        }
        long long a = V < 0 ? -V : V;
        for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xFFFFFFFFu, a, o);
        if (lane == 0) wsum[warp] = a;
        __syncthreads();
        if (threadIdx.x == 0) {
            long long t = 0;
            for (int w = 0; w < 8; w++) t += wsum[w];
            parts[(uint64_t)blockIdx.x * 8 + n] = t;
            if (blockIdx.x == 0) head->S[n] = S;
        }
        __syncthreads();
    }
    if (k < kpad) for (uint32_t col = N * DIGITS; col < cs; col++) dst[staged_index_int(prec, cs, k, col)] = 0;
    if (blockIdx.x == 0 && threadIdx.x == 0) head->nparts = gridDim.x;
}

__device__ __forceinline__ void mma_s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// (bits & mask) | 0x4300 per half = bf16 value 128 + field; subtracting `bias` (exact in bf16) leaves the
// signed integer the field encodes.
__device__ __forceinline__ uint32_t int_pair_to_bf16(uint32_t shifted, uint32_t mask, uint32_t bias_pair)
{
    uint32_t v = (shifted & mask) | 0x43004300u;
    __nv_bfloat162 r = __hsub2(*reinterpret_cast<__nv_bfloat162 *>(&v), *reinterpret_cast<const __nv_bfloat162 *>(&bias_pair));
    return *reinterpret_cast<uint32_t *>(&r);
}

__device__ __forceinline__ uint32_t hi16_pair(uint32_t f0, uint32_t f1) { return __byte_perm(f0, f1, 0x7632); }

// ---- mbarrier / TMA wrappers (bounded waits) --------------------------------------
__device__ __forceinline__ uint32_t gsmem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void gbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void gbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void gbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Returns false once the abort flag is up (then every later wait returns at once) or when the bound is hit.
__device__ __forceinline__ bool gbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int32_t *status, int code)
{
    if (*abort_flag) return false;
    for (uint32_t i = 0; i < GEMV_WAIT_LIMIT; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        if ((i & 255u) == 255u && *abort_flag) return false;
    }
    *abort_flag = 1;
    atomicCAS(status, 0, code);
    return false;
}
__device__ __forceinline__ void tma_box_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void bulk_copy_1d(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar)
{
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// Named barriers between the consumer warps and the epilogue warp: the side that hands something over
// only arrives (does not wait), the side that needs it waits.
__device__ __forceinline__ void handoff_arrive(uint32_t id) { asm volatile("bar.arrive %0, %1;" ::"r"(id), "n"(HANDOFF_THREADS) : "memory"); }
__device__ __forceinline__ void handoff_wait(uint32_t id) { asm volatile("bar.sync %0, %1;" ::"r"(id), "n"(HANDOFF_THREADS) : "memory"); }

// Bounded wait until `target` CTAs have finished a layer (device-scope acquire on the layer's counter).
__device__ __forceinline__ bool grid_wait(const int32_t *counter, uint32_t target, volatile int *abort_flag, int32_t *status, int code)
{
    if (*abort_flag) return false;
    for (uint32_t i = 0; i < (1u << 22); ++i) {
        int v;
        asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
        if ((uint32_t)v >= target) return true;
        if ((i & 63u) == 63u && *abort_flag) return false;
        __nanosleep(64);
    }
    *abort_flag = 1;
    atomicCAS(status, 0, code);
    return false;
}

// End of the launch, epilogue warp: the CTA that finishes last (an exit ticket) applies the row softmax of a
// final softmax layer (Activation.c:5-21 per row -- maximum from -FLT_MAX, expf(x - max), scaling by 1/sum only
// when the sum is positive) and puts the layer counters and the ticket back to zero for the next launch.
__device__ __forceinline__ void chain_finish(const ChainParams &ch, uint32_t lane)
{
    const GemvParams &p = ch.L[ch.n - 1];
    if (!p.softmax && ch.n == 1) return;
    __threadfence();                                           // this CTA's outputs are visible before its ticket
    uint32_t ticket = 0;
    if (lane == 0) ticket = atomicAdd(reinterpret_cast<unsigned int *>(ch.sync + MAX_CHAIN), 1u);
    ticket = __shfl_sync(0xFFFFFFFFu, ticket, 0);
    if (ticket != gridDim.x - 1) return;
    __threadfence();
    for (uint32_t n = 0; p.softmax && n < p.N; n++) {
        float *r = p.y + (uint64_t)n * p.ldy;
        if (p.out <= 1024) {
            // the whole row in registers: one trip to L2 and back
            float v[32];
            float mx = -FLT_MAX;
#pragma unroll
            for (int j = 0; j < 32; j++) { const uint32_t i = j * 32 + lane; v[j] = i < p.out ? __ldcg(r + i) : -FLT_MAX; if (v[j] > mx) mx = v[j]; }
            mx = spg_warp_max(mx);
            float sum = 0.0f;
#pragma unroll
            for (int j = 0; j < 32; j++) { const uint32_t i = j * 32 + lane; v[j] = i < p.out ? expf(v[j] - mx) : 0.0f; sum += v[j]; }
            sum = spg_warp_sum(sum);
            const float inv = sum > 0.0f ? 1.0f / sum : 1.0f;
#pragma unroll
            for (int j = 0; j < 32; j++) { const uint32_t i = j * 32 + lane; if (i < p.out) r[i] = v[j] * inv; }
            continue;
        }
        float mx = -FLT_MAX;
        for (uint32_t i = lane; i < p.out; i += 32u) { const float v = __ldcg(r + i); if (v > mx) mx = v; }
        mx = spg_warp_max(mx);
        float sum = 0.0f;
        for (uint32_t i = lane; i < p.out; i += 32u) { const float e = expf(__ldcg(r + i) - mx); r[i] = e; sum += e; }
        sum = spg_warp_sum(sum);
        if (sum > 0.0f) {
            const float inv = 1.0f / sum;
            for (uint32_t i = lane; i < p.out; i += 32u) r[i] *= inv;
        }
    }
    if (lane <= MAX_CHAIN) ch.sync[lane] = 0;                  // ready for the next launch
}

// One step of one warp: 16 rows x (4 lanes x EL elements).  ra / rbv are the lane's 128-bit pieces of rows
// g and g+8; xb points at this lane's slot of the step's staged activations (CW columns per tile).
template <int PREC, int T, int CW>
__device__ __forceinline__ void gemv_step(const uint4 &ra, const uint4 &rbv, const uint2 *xb, bool col_live,
                                          float (&acc)[T][4], float (&acc_hi)[T][4])
{
    constexpr int NB = Fmt<PREC>::EL / 4;
    const uint32_t wa[4] = { ra.x, ra.y, ra.z, ra.w };
    const uint32_t wb[4] = { rbv.x, rbv.y, rbv.z, rbv.w };
#pragma unroll
    for (int b = 0; b < NB; b++) {
        uint2 bf[T];
#pragma unroll
        for (int i = 0; i < T; i++) bf[i] = col_live ? xb[(b * T + i) * 4 * CW] : make_uint2(0u, 0u);   // lanes of columns not kept multiply by zero
        if (PREC == SPG_P_I4) {
            const int j = b >> 1, h = b & 1;
            const uint32_t va = wa[j] ^ 0x88888888u, vb = wb[j] ^ 0x88888888u;     // nibble + 8
            const uint32_t a0 = int_pair_to_bf16(va >> (8 * h), 0x000F000Fu, 0x43084308u);
            const uint32_t a2 = int_pair_to_bf16(va >> (8 * h + 4), 0x000F000Fu, 0x43084308u);
            const uint32_t a1 = int_pair_to_bf16(vb >> (8 * h), 0x000F000Fu, 0x43084308u);
            const uint32_t a3 = int_pair_to_bf16(vb >> (8 * h + 4), 0x000F000Fu, 0x43084308u);
#pragma unroll
            for (int i = 0; i < T; i++) mma_bf16(acc[i], a0, a1, a2, a3, bf[i].x, bf[i].y);
        } else if (PREC == SPG_P_I2) {
            const int j = b >> 2, h = b & 3;
            const uint32_t va = wa[j] ^ 0xAAAAAAAAu, vb = wb[j] ^ 0xAAAAAAAAu;     // crumb + 2
            const uint32_t a0 = int_pair_to_bf16(va >> (4 * h), 0x00030003u, 0x43024302u);
            const uint32_t a2 = int_pair_to_bf16(va >> (4 * h + 2), 0x00030003u, 0x43024302u);
            const uint32_t a1 = int_pair_to_bf16(vb >> (4 * h), 0x00030003u, 0x43024302u);
            const uint32_t a3 = int_pair_to_bf16(vb >> (4 * h + 2), 0x00030003u, 0x43024302u);
#pragma unroll
            for (int i = 0; i < T; i++) mma_bf16(acc[i], a0, a1, a2, a3, bf[i].x, bf[i].y);
        } else if (PREC == SPG_P_I8) {
            // q = 16*(q >> 4) + (q & 15): low nibbles are unsigned, high nibbles signed (+8 after the flip)
            const uint32_t va = wa[b] ^ 0x80808080u, vb = wb[b] ^ 0x80808080u;
            uint32_t a0 = int_pair_to_bf16(va, 0x000F000Fu, 0x43004300u);
            uint32_t a2 = int_pair_to_bf16(va >> 8, 0x000F000Fu, 0x43004300u);
            uint32_t a1 = int_pair_to_bf16(vb, 0x000F000Fu, 0x43004300u);
            uint32_t a3 = int_pair_to_bf16(vb >> 8, 0x000F000Fu, 0x43004300u);
#pragma unroll
            for (int i = 0; i < T; i++) mma_bf16(acc[i], a0, a1, a2, a3, bf[i].x, bf[i].y);
            a0 = int_pair_to_bf16(va >> 4, 0x000F000Fu, 0x43084308u);
            a2 = int_pair_to_bf16(va >> 12, 0x000F000Fu, 0x43084308u);
            a1 = int_pair_to_bf16(vb >> 4, 0x000F000Fu, 0x43084308u);
            a3 = int_pair_to_bf16(vb >> 12, 0x000F000Fu, 0x43084308u);
#pragma unroll
            for (int i = 0; i < T; i++) mma_bf16(acc_hi[i], a0, a1, a2, a3, bf[i].x, bf[i].y);
        } else if (PREC == SPG_P_BF16) {
#pragma unroll
            for (int i = 0; i < T; i++) mma_bf16(acc[i], wa[2 * b], wb[2 * b], wa[2 * b + 1], wb[2 * b + 1], bf[i].x, bf[i].y);
        } else if (PREC == SPG_P_F16) {
            // fp16 (11 significant bits) = bf16 head (8 bits) + bf16 tail (3 bits), both exact
            uint32_t hi[4], lo[4];
            const uint32_t src[4] = { wa[2 * b], wb[2 * b], wa[2 * b + 1], wb[2 * b + 1] };
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&src[q]));
                const uint32_t u0 = __float_as_uint(f.x) & 0xFFFF0000u, u1 = __float_as_uint(f.y) & 0xFFFF0000u;
                hi[q] = hi16_pair(u0, u1);
                lo[q] = hi16_pair(__float_as_uint(f.x - __uint_as_float(u0)), __float_as_uint(f.y - __uint_as_float(u1)));
            }
#pragma unroll
            for (int i = 0; i < T; i++) {
                mma_bf16(acc[i], hi[0], hi[1], hi[2], hi[3], bf[i].x, bf[i].y);
                mma_bf16(acc[i], lo[0], lo[1], lo[2], lo[3], bf[i].x, bf[i].y);
            }
        } else {
            // fp32 = three bf16 terms of 8 bits each (head, middle, tail), all exact
            uint32_t t0[4], t1[4], t2[4];
            const uint32_t src[8] = { wa[0], wa[1], wb[0], wb[1], wa[2], wa[3], wb[2], wb[3] };
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const float f0 = __uint_as_float(src[2 * q]), f1 = __uint_as_float(src[2 * q + 1]);
                const uint32_t h0 = src[2 * q] & 0xFFFF0000u, h1 = src[2 * q + 1] & 0xFFFF0000u;
                const float r0 = f0 - __uint_as_float(h0), r1 = f1 - __uint_as_float(h1);
                const uint32_t m0 = __float_as_uint(r0) & 0xFFFF0000u, m1 = __float_as_uint(r1) & 0xFFFF0000u;
                t0[q] = hi16_pair(h0, h1);
                t1[q] = hi16_pair(m0, m1);
                t2[q] = hi16_pair(__float_as_uint(r0 - __uint_as_float(m0)), __float_as_uint(r1 - __uint_as_float(m1)));
            }
#pragma unroll
            for (int i = 0; i < T; i++) {
                mma_bf16(acc[i], t0[0], t0[1], t0[2], t0[3], bf[i].x, bf[i].y);
                mma_bf16(acc[i], t1[0], t1[1], t1[2], t1[3], bf[i].x, bf[i].y);
                mma_bf16(acc[i], t2[0], t2[1], t2[2], t2[3], bf[i].x, bf[i].y);
            }
        }
    }
}

// Integer-path step: the same 16 rows x (4 lanes x EL elements), as EL / 8 k32 MMAs.  The weights become
// signed bytes holding q * SHIFT (SHIFT = 16 for INT4, 64 for INT2, 1 for INT8) with a shift and a mask.
template <int PREC> struct IntFmt;
template <> struct IntFmt<SPG_P_I4> { static constexpr int SHIFT = 16, QMAX = 8; };
template <> struct IntFmt<SPG_P_I2> { static constexpr int SHIFT = 64, QMAX = 2; };
template <> struct IntFmt<SPG_P_I8> { static constexpr int SHIFT = 1, QMAX = 128; };

template <int PREC, int T, int CW>
__device__ __forceinline__ void gemv_step_int(const uint4 &ra, const uint4 &rbv, const uint2 *xb, bool col_live, int (&acc)[T][4])
{
    constexpr int NBI = Fmt<PREC>::EL / 8;
    const uint32_t wa[4] = { ra.x, ra.y, ra.z, ra.w };
    const uint32_t wb[4] = { rbv.x, rbv.y, rbv.z, rbv.w };
#pragma unroll
    for (int m = 0; m < NBI; m++) {
        uint2 bf[T];
#pragma unroll
        for (int i = 0; i < T; i++) bf[i] = col_live ? xb[(m * T + i) * 4 * CW] : make_uint2(0u, 0u);
        uint32_t a0, a1, a2, a3;
        if (PREC == SPG_P_I4) {
            a0 = (wa[m] << 4) & 0xF0F0F0F0u; a2 = wa[m] & 0xF0F0F0F0u;
            a1 = (wb[m] << 4) & 0xF0F0F0F0u; a3 = wb[m] & 0xF0F0F0F0u;
        } else if (PREC == SPG_P_I2) {
            const int j = m >> 1, h = m & 1;
            a0 = (wa[j] << (6 - 4 * h)) & 0xC0C0C0C0u; a2 = (wa[j] << (4 - 4 * h)) & 0xC0C0C0C0u;
            a1 = (wb[j] << (6 - 4 * h)) & 0xC0C0C0C0u; a3 = (wb[j] << (4 - 4 * h)) & 0xC0C0C0C0u;
        } else {
            a0 = wa[2 * m]; a2 = wa[2 * m + 1];
            a1 = wb[2 * m]; a3 = wb[2 * m + 1];
        }
#pragma unroll
        for (int i = 0; i < T; i++) mma_s8(acc[i], a0, a1, a2, a3, bf[i].x, bf[i].y);
    }
}

template <int PREC, int T, int CW, bool INTP>
__global__ void __launch_bounds__(GEMV_THREADS, 1)
spg_gemv_kernel(const __grid_constant__ ChainMaps maps, const __grid_constant__ ChainParams ch)
{
    using F = Fmt<PREC>;
    constexpr uint32_t EL = F::EL, NB = EL / 4;                // per warp step: 4 lanes x EL elements; NB B-blocks per load
    constexpr uint32_t STEP_SLOTS = (INTP ? EL / 8 : NB) * T * 4 * CW;   // uint2 slots of staged input per step
    constexpr uint32_t CPAD = 8 * T;
    const GemvParams &p0 = ch.L[0];                             // chunk geometry, ring depth and batch are the same for every layer

    extern __shared__ uint8_t gemv_smem_raw[];
    const uint32_t raw = gsmem_u32(gemv_smem_raw);
    const uint32_t base = (raw + 127u) & ~127u;
    uint8_t *smem = gemv_smem_raw + (base - raw);
    // layout: ring of chunks, each = [16 rows x 8 warp slices of packed weights | staged input of the same K range];
    // then the reduction buffer, the barriers and the abort flag
    const uint32_t wchunk_bytes = 8 * p0.box_bytes;
    const uint32_t slot_bytes = wchunk_bytes + p0.xchunk_bytes;
    const uint32_t ring = p0.ring;
    const uint32_t red_off = ring * slot_bytes;
    constexpr uint32_t RED_FLOATS = (INTP ? 1 : CONSUMER_WARPS) * ITEM_ROWS * CPAD;   // integer path: one shared buffer of sums
    const uint32_t bar_off = red_off + 2 * RED_FLOATS * 4;       // two reduction buffers, used alternately
    const uint32_t full0 = base + bar_off, empty0 = full0 + 8 * ring;
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + bar_off + 16 * ring);
    float *red = reinterpret_cast<float *>(smem + red_off);
    int32_t *status = p0.status;

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u, g = lane >> 2, t = lane & 3u;
    if (INTP) for (uint32_t i = tid; i < 2 * RED_FLOATS; i += GEMV_THREADS) red[i] = 0.0f;      // integer zero too
    if (tid == 0) {
        for (uint32_t s = 0; s < ring; s++) { gbar_init(full0 + 8 * s, 1); gbar_init(empty0 + 8 * s, CONSUMER_WARPS); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        for (uint32_t l = 0; l < ch.n; l++) asm volatile("prefetch.tensormap [%0];" ::"l"(&maps.m[l]) : "memory");
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");      // the next kernel may start on SMs this grid leaves
    }
    __syncthreads();
    // items of this CTA over all layers (the consumer <-> epilogue hand-off counts them through)
    uint32_t my_total = 0;
    for (uint32_t l = 0; l < ch.n; l++) my_total += ch.L[l].items > blockIdx.x ? (ch.L[l].items - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;

    if (warp == CONSUMER_WARPS) {
        // ------------------------------ producer: two copies per chunk -------------------
        // The weights of a layer depend on nothing that runs before it, its staged input does: on the kernel before
        // this one in the stream (layer 0, programmatic dependent launch) or on every CTA's share of the layer
        // before (a device-wide counter).  So weight boxes are requested as far ahead as the ring allows, the
        // input copies of the chunks issued meanwhile are held back, and only when nothing else can be done does
        // the thread wait for the input to exist.  The HBM stream therefore runs through layer boundaries.
        if (lane == 0) {
            uint32_t s = 0, ph = 1, q = 0, npend = 0;
            uint32_t pend_slot[8], pend_c[8];
            bool alive = true;
            for (uint32_t l = 0; l < ch.n && alive; l++) {
                const GemvParams &p = ch.L[l];
                bool x_ready = false;
                auto make_ready = [&]() -> bool {
                    if (l == 0) asm volatile("griddepcontrol.wait;" ::: "memory");
                    else if (!grid_wait(ch.sync + (l - 1), gridDim.x, abort_flag, status, 7)) return false;
                    for (uint32_t i = 0; i < npend; i++)
                        bulk_copy_1d(base + pend_slot[i] * slot_bytes + wchunk_bytes,
                                     reinterpret_cast<const uint8_t *>(p.xin) + (size_t)pend_c[i] * p.xchunk_bytes, p.xchunk_bytes, full0 + 8 * pend_slot[i]);
                    npend = 0;
                    x_ready = true;
                    return true;
                };
                for (uint32_t item = blockIdx.x; item < p.items && alive; item += gridDim.x) {
                    for (uint32_t c = 0; c < p.nchunks; c++, q++) {
                        if (q >= ring) {
                            // a held-back input copy keeps its slot from ever filling: settle those before blocking on a slot
                            if (!x_ready && (npend == ring || npend == 8) && !make_ready()) { alive = false; break; }
                            if (!x_ready) {
                                uint32_t ok;
                                asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                                             : "=r"(ok) : "r"(empty0 + 8 * s), "r"(ph) : "memory");
                                if (!ok && !make_ready()) { alive = false; break; }
                            }
                            if (!gbar_wait(empty0 + 8 * s, ph, abort_flag, status, 1)) { alive = false; break; }
                        }
                        gbar_expect_tx(full0 + 8 * s, slot_bytes);
                        tma_box_2d(base + s * slot_bytes, &maps.m[l], full0 + 8 * s, (int)(c * (wchunk_bytes / ITEM_ROWS / 8)), (int)(item * ITEM_ROWS));
                        if (x_ready) {
                            bulk_copy_1d(base + s * slot_bytes + wchunk_bytes,
                                         reinterpret_cast<const uint8_t *>(p.xin) + (size_t)c * p.xchunk_bytes, p.xchunk_bytes, full0 + 8 * s);
                        } else {
                            pend_slot[npend] = s; pend_c[npend] = c; npend++;
                            if (npend == 8 && !make_ready()) { alive = false; break; }
                        }
                        if (++s == ring) { s = 0; ph ^= 1u; }
                    }
                }
                if (alive && npend && !make_ready()) alive = false;        // every chunk of the layer went out before its input existed
            }
        }
        return;
    }

    if (warp == CONSUMER_WARPS + 1) {
        // ------------------------------ epilogue warp ------------------------------
        // Sums the sixteen K slices and the activation terms of each finished item, applies scale, bias and
        // activation, writes y and stages the next layer's input, while the consumers stream the next item.
        uint32_t n_item = 0;
        bool dead = false;                                      // a bounded wait gave up: keep the hand-offs going, do no work
        for (uint32_t l = 0; l < ch.n; l++) {
        const GemvParams &p = ch.L[l];
        const uint32_t cs = CW * T, spare = cs - p.C;
        // everything this warp reads or writes is ordered after the kernel before (first layer) or after every
        // CTA's share of the layer before
        if (l == 0) asm volatile("griddepcontrol.wait;" ::: "memory");
        else if (!dead) {
            bool ok = true;
            if (lane == 0) ok = grid_wait(ch.sync + (l - 1), gridDim.x, abort_flag, status, 8);
            if (!__shfl_sync(0xFFFFFFFFu, ok ? 1 : 0, 0)) dead = true;
            __threadfence();
        }
        if (dead) {
            // the consumers still arrive at and wait on the named barriers: answer them so that nobody hangs
            for (uint32_t item = blockIdx.x; item < p.items; item += gridDim.x, n_item++) {
                handoff_wait(1 + (n_item & 1u));
                if (n_item + 2 < my_total) handoff_arrive(3 + (n_item & 1u));
            }
            continue;
        }
        if constexpr (INTP) {
            // ---- integer path: exact integer dot products; scales and the next layer's range bound first ----
            __shared__ float e_sc[MAX_BATCH], e_inv[MAX_BATCH];
            const StagedHead *ih = reinterpret_cast<const StagedHead *>(p.in_head);
            const long long *iparts = reinterpret_cast<const long long *>(p.in_head + 256);
            const float bmax = p.bias_absmax;
            for (uint32_t n = 0; n < p.N; n++) {
                // the head was written by other CTAs earlier in this launch (or by the kernel before): read it past L1,
                // which may still hold this buffer's lines from two layers ago
                const float S = __ldcg(&ih->S[n]);
                float inv_next = 0.0f;
                if (p.xout) {
                    long long l1 = 0;
                    const uint32_t nparts = __ldcg(&ih->nparts);
                    for (uint32_t i = lane; i < nparts; i += 32) l1 += __ldcg(iparts + (uint64_t)i * 8 + n);
                    for (int o = 16; o > 0; o >>= 1) l1 += __shfl_xor_sync(0xFFFFFFFFu, l1, o);
                    // |y| <= max|bias| + |scale| * max|q| * sum|x'|, x' = V * S / DIGIT_FULL the values the MMAs really see
                    double bound = (double)bmax + fabs((double)p.scale) * IntFmt<PREC>::QMAX * ((double)S / DIGIT_FULL) * (double)l1;
                    bound *= 1.0001;
                    if (p.act == SPG_ACT_SIGMOID) bound = 1.0;
                    else if (p.act == SPG_ACT_TANH) bound = bound < 1.0 ? bound : 1.0;
                    float Sn = __double2float_ru(bound);
                    if (!(Sn <= 3.0e38f)) Sn = __int_as_float(0x7FC00000);        // overflow or NaN input: the row turns into NaN
                    inv_next = (Sn > 0.0f) ? (float)(DIGIT_FULL / (double)Sn) : 0.0f;
                    if (blockIdx.x == 0 && lane == 0) reinterpret_cast<StagedHead *>(p.out_head)->S[n] = Sn;
                }
                if (lane == 0) {
                    e_sc[n] = (float)((double)p.scale * (double)S / (DIGIT_FULL * IntFmt<PREC>::SHIFT));
                    e_inv[n] = inv_next;
                }
            }
            if (p.xout && blockIdx.x == 0 && lane == 0) reinterpret_cast<StagedHead *>(p.out_head)->nparts = gridDim.x;
            __syncwarp();
            int *redi = reinterpret_cast<int *>(red);
            uint8_t *xo = reinterpret_cast<uint8_t *>(p.xout);
            long long *oparts = p.out_head ? reinterpret_cast<long long *>(p.out_head + 256) : nullptr;
            constexpr int PER_LANE = ITEM_ROWS * MAX_BATCH / 32;        // outputs of one item a lane may own
            long long abs_run[PER_LANE];                                // this CTA's sum of |V| per batch row (lanes 0 and 16 hold it)
#pragma unroll
            for (int u = 0; u < PER_LANE; u++) abs_run[u] = 0;
            // the biases of an item's rows are fetched one item ahead, so their latency never sits between two items
            float bias_nx[PER_LANE];
#pragma unroll
            for (int u = 0; u < PER_LANE; u++) {
                const uint32_t idx = u * 32 + lane, row = blockIdx.x * ITEM_ROWS + idx % ITEM_ROWS;
                bias_nx[u] = (idx < ITEM_ROWS * p.N && row < p.out) ? p.bias[row] : 0.0f;
            }
            for (uint32_t item = blockIdx.x; item < p.items; item += gridDim.x, n_item++) {
                const uint32_t rbuf = n_item & 1u;
                float bias_r[PER_LANE];
#pragma unroll
                for (int u = 0; u < PER_LANE; u++) {
                    bias_r[u] = bias_nx[u];
                    const uint32_t idx = u * 32 + lane, row = (item + gridDim.x) * ITEM_ROWS + idx % ITEM_ROWS;
                    bias_nx[u] = (idx < ITEM_ROWS * p.N && row < p.out) ? p.bias[row] : 0.0f;
                    if (xo && !(fabsf(bias_r[u]) <= bmax)) atomicCAS(p.status, 0, 9);       // the caller's bound is wrong
                }
                handoff_wait(1 + rbuf);
                int *redb = redi + rbuf * RED_FLOATS;
                long long tot[PER_LANE];
#pragma unroll
                for (int u = 0; u < PER_LANE; u++) {
                    const uint32_t idx = u * 32 + lane, n = idx / ITEM_ROWS, rl = idx % ITEM_ROWS;
                    tot[u] = 0;
                    if (idx < ITEM_ROWS * p.N) {
                        int *src = redb + rl * CPAD + n * DIGITS;
#pragma unroll
                        for (int d = 0; d < DIGITS; d++) { tot[u] += (long long)src[d] << (7 * d); src[d] = 0; }   // leave the sums cleared for the item after next
                    }
                }
                __syncwarp();
                if (n_item + 2 < my_total) handoff_arrive(3 + rbuf);   // the buffer is free again
#pragma unroll
                for (int u = 0; u < PER_LANE; u++) {
                    const uint32_t idx = u * 32 + lane, n = idx / ITEM_ROWS, rl = idx % ITEM_ROWS, row = item * ITEM_ROWS + rl;
                    if (u * 32 >= ITEM_ROWS * p.N) break;                  // warp-uniform
                    long long absV = 0;
                    if (n < p.N && row < p.out) {
                        const float yv = spg_activate(fmaf(__ll2float_rn(tot[u]), e_sc[n], bias_r[u]), p.act);
                        p.y[(uint64_t)n * p.ldy + row] = yv;
                        if (xo) {
                            const long long V = fixed_of_f(yv, e_inv[n]);
                            stage_digits(xo, p.next_prec, cs, row, n, V);
                            absV = V < 0 ? -V : V;
                        }
                    }
                    if (xo) {
                        // lanes 0..15 hold one batch row, lanes 16..31 the next: their |V| sums go beside the staged data
                        for (int o = 8; o > 0; o >>= 1) absV += __shfl_xor_sync(0xFFFFFFFFu, absV, o);
                        abs_run[u] += absV;
                    }
                }
                if (xo) {
                    for (uint32_t idx = lane; idx < ITEM_ROWS * spare; idx += 32) {
                        const uint32_t row = item * ITEM_ROWS + idx / spare;
                        if (row < p.out) xo[staged_index_int(p.next_prec, cs, row, p.C + idx % spare)] = 0;
                    }
                    if (item == p.items - 1)
                        for (uint32_t idx = lane; idx < (p.next_kpad - p.out) * cs; idx += 32)
                            xo[staged_index_int(p.next_prec, cs, p.out + idx / cs, idx % cs)] = 0;
                }
            }
            if (xo && (lane & 15u) == 0) {
#pragma unroll
                for (int u = 0; u < PER_LANE; u++) {
                    const uint32_t n = (u * 32 + lane) / ITEM_ROWS;
                    if (n < p.N) oparts[(uint64_t)blockIdx.x * 8 + n] = abs_run[u];
                }
            }
        } else {
        constexpr int PER_LANE = ITEM_ROWS * MAX_BATCH / 32;
        for (uint32_t item = blockIdx.x; item < p.items; item += gridDim.x, n_item++) {
            const uint32_t rbuf = n_item & 1u;
            float bias_r[PER_LANE], sum_r[PER_LANE];
#pragma unroll
            for (int u = 0; u < PER_LANE; u++) {
                const uint32_t idx = u * 32 + lane, row = item * ITEM_ROWS + idx % ITEM_ROWS;
                bias_r[u] = (idx < ITEM_ROWS * p.N && row < p.out) ? p.bias[row] : 0.0f;
            }
            handoff_wait(1 + rbuf);
            const float *redb = red + rbuf * RED_FLOATS;
#pragma unroll
            for (int u = 0; u < PER_LANE; u++) {
                const uint32_t idx = u * 32 + lane, n = idx / ITEM_ROWS, rl = idx % ITEM_ROWS;
                float sum = 0.0f;
                if (idx < ITEM_ROWS * p.N) {
#pragma unroll
                    for (int w = 0; w < CONSUMER_WARPS; w++) {
                        const float *src = redb + (w * ITEM_ROWS + rl) * CPAD + n * p.P;
                        float part = 0.0f;
                        for (uint32_t q = p.P; q-- > 0;) part += src[q];           // smallest term first
                        sum += part;
                    }
                }
                sum_r[u] = sum;
            }
            __syncwarp();
            if (n_item + 2 < my_total) handoff_arrive(3 + rbuf);   // only if a later item will wait for it
#pragma unroll
            for (int u = 0; u < PER_LANE; u++) {
                const uint32_t idx = u * 32 + lane, n = idx / ITEM_ROWS, row = item * ITEM_ROWS + idx % ITEM_ROWS;
                if (idx >= ITEM_ROWS * p.N || row >= p.out) continue;
                const float yv = spg_activate(fmaf(sum_r[u], p.scale, bias_r[u]), p.act);
                p.y[(uint64_t)n * p.ldy + row] = yv;
                if (p.xout) stage_value(p.xout, p.next_prec, cs, row, n, p.P, yv);
            }
            if (p.xout) {
                // columns that carry no sample stay zero in the next layer's staged input; so does its K tail
                for (uint32_t idx = lane; idx < ITEM_ROWS * spare; idx += 32) {
                    const uint32_t row = item * ITEM_ROWS + idx / spare;
                    if (row < p.out) p.xout[staged_index(p.next_prec, cs, row, p.C + idx % spare)] = __float2bfloat16_rn(0.0f);
                }
                if (item == p.items - 1)
                    for (uint32_t idx = lane; idx < (p.next_kpad - p.out) * cs; idx += 32)
                        p.xout[staged_index(p.next_prec, cs, p.out + idx / cs, idx % cs)] = __float2bfloat16_rn(0.0f);
            }
        }
        }
        // this CTA's share of the layer is done (outputs, staged input of the next layer, partial sums): tell the others
        if (l + 1 < ch.n) {
            __threadfence();
            __syncwarp();
            if (lane == 0) atomicAdd(ch.sync + l, 1);
        }
        }
        chain_finish(ch, lane);
        return;
    }

    // ------------------------------ consumers --------------------------------------
    const bool col_live = g < CW;                              // with 4 kept columns only lanes of columns 0..3 load
    uint32_t s = 0, ph = 0, n_item = 0;
    for (uint32_t l = 0; l < ch.n; l++) {
    const GemvParams &p = ch.L[l];
    const uint32_t row_pitch = 8 * p.spb * 64u;                // bytes of one chunk row (8 warp slices)
    for (uint32_t item = blockIdx.x; item < p.items; item += gridDim.x, n_item++) {
        // two accumulator sets (even / odd steps) keep two independent MMA chains in flight
        float acc[2][T][4], acc_hi[2][T][4];                   // acc_hi: INT8 only (the high-nibble term)
        int iacc[2][T][4];                                     // integer path (the unused set is optimised away)
#pragma unroll
        for (int e = 0; e < 2; e++)
#pragma unroll
            for (int i = 0; i < T; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) { acc[e][i][j] = 0.0f; acc_hi[e][i][j] = 0.0f; iacc[e][i][j] = 0; }

        for (uint32_t c = 0; c < p.nchunks; c++) {
            const bool ok = gbar_wait(full0 + 8 * s, ph, abort_flag, status, 2);
            const uint32_t slice = warp & 7u, sub = warp >> 3;             // which 8th of the chunk's K range, which half of its steps
            const uint32_t per_sub = p.spb > 1 ? p.spb / 2 : 1;
            if (ok && c * 8u + slice < p.nboxes && sub * per_sub < p.spb) {
                const uint8_t *box = smem + s * slot_bytes + g * row_pitch + slice * p.spb * 64u + t * 16;
                const uint2 *xs = reinterpret_cast<const uint2 *>(smem + s * slot_bytes + wchunk_bytes) +
                                  (size_t)slice * p.spb * STEP_SLOTS + t * CW + (col_live ? g : 0);
                for (uint32_t st = sub * per_sub; st < (sub + 1) * per_sub; st++) {
                    const uint4 ra0 = *reinterpret_cast<const uint4 *>(box + st * 64);
                    const uint4 rb0 = *reinterpret_cast<const uint4 *>(box + 8 * row_pitch + st * 64);
                    if constexpr (INTP) {
                        if (st & 1u) gemv_step_int<PREC, T, CW>(ra0, rb0, xs + (size_t)st * STEP_SLOTS, col_live, iacc[1]);
                        else gemv_step_int<PREC, T, CW>(ra0, rb0, xs + (size_t)st * STEP_SLOTS, col_live, iacc[0]);
                    } else {
                        if (st & 1u) gemv_step<PREC, T, CW>(ra0, rb0, xs + (size_t)st * STEP_SLOTS, col_live, acc[1], acc_hi[1]);
                        else gemv_step<PREC, T, CW>(ra0, rb0, xs + (size_t)st * STEP_SLOTS, col_live, acc[0], acc_hi[0]);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) gbar_arrive(empty0 + 8 * s);
            if (++s == ring) { s = 0; ph ^= 1u; }
        }

        // ---- the sixteen partial sums go to shared memory [warp][row][column]; the epilogue warp takes over ----
        const uint32_t rbuf = n_item & 1u;
        if (n_item >= 2) handoff_wait(3 + rbuf);               // the epilogue warp has read this buffer's previous contents
        float *redb = red + rbuf * RED_FLOATS;
        if constexpr (INTP) {
            // integer sums commute: every warp adds its partials into one [row][column] buffer
            int *redi = reinterpret_cast<int *>(red) + rbuf * RED_FLOATS;
#pragma unroll
            for (int i = 0; i < T; i++) {
                int *r0 = redi + g * CPAD + i * 8 + 2 * t;
                atomicAdd(r0, iacc[0][i][0] + iacc[1][i][0]); atomicAdd(r0 + 1, iacc[0][i][1] + iacc[1][i][1]);
                atomicAdd(r0 + 8 * CPAD, iacc[0][i][2] + iacc[1][i][2]); atomicAdd(r0 + 8 * CPAD + 1, iacc[0][i][3] + iacc[1][i][3]);
            }
        } else {
#pragma unroll
        for (int i = 0; i < T; i++) {
            float d0 = acc[0][i][0] + acc[1][i][0], d1 = acc[0][i][1] + acc[1][i][1];
            float d2 = acc[0][i][2] + acc[1][i][2], d3 = acc[0][i][3] + acc[1][i][3];
            if (PREC == SPG_P_I8) {
                d0 = fmaf(16.0f, acc_hi[0][i][0] + acc_hi[1][i][0], d0); d1 = fmaf(16.0f, acc_hi[0][i][1] + acc_hi[1][i][1], d1);
                d2 = fmaf(16.0f, acc_hi[0][i][2] + acc_hi[1][i][2], d2); d3 = fmaf(16.0f, acc_hi[0][i][3] + acc_hi[1][i][3], d3);
            }
            float *r0 = redb + ((warp * ITEM_ROWS + g) * CPAD) + i * 8 + 2 * t;
            r0[0] = d0; r0[1] = d1;
            r0[8 * CPAD] = d2; r0[8 * CPAD + 1] = d3;
        }
        }
        __threadfence_block();
        handoff_arrive(1 + rbuf);                              // no waiting: on to the next item
    }
    }
}

struct Plan {
    uint32_t P, C, cs, T, CW, spb, box_bytes, nboxes, nchunks, kpad, items, ring, xdepth, xchunk_bytes;
    size_t staged_bytes, smem;
    bool ok, intp;
};

bool g_int_path = true;         // integer tensor path for INT8 / INT4 / INT2 files (spgk_gemv_set_int_path)

inline bool int_path_for(const spgk_layer *L)
{
    return g_int_path && (L->precision == SPG_P_I8 || L->precision == SPG_P_I4 || L->precision == SPG_P_I2) && L->in <= INT_PATH_MAX_K;
}

Plan make_plan(const spgk_layer *L, uint32_t N)
{
    Plan pl{};
    pl.ok = false;
    if (!L || N == 0 || N > MAX_BATCH || (unsigned)L->precision >= SPG_P_COUNT || L->in == 0 || L->out == 0) return pl;
    const uint32_t bits = spg_bits_per_elem(L->precision), el = 128u / bits, ks = 4 * el;
    const uint64_t row_bytes = (uint64_t)L->in * bits / 8;
    // TMA needs 16-byte aligned packed rows; very short rows go to the general kernel
    if (L->in % el || ((uintptr_t)L->w & 15u) || row_bytes < 64) return pl;
    pl.intp = int_path_for(L);
    uint32_t per_spb;
    if (pl.intp) {
        // four digit columns per batch row; one staged byte per column and k
        pl.P = DIGITS;
        pl.C = N * DIGITS;
        pl.cs = N == 1 ? 4 : 8 * ((N + 1) / 2);
        pl.T = pl.cs <= 8 ? 1 : pl.cs / 8;
        pl.CW = pl.cs < 8 ? 4 : 8;
        per_spb = 8 * ks * pl.cs;
    } else {
        pl.P = N == 1 ? 3 : 2;
        pl.C = N * pl.P;
        pl.cs = pl.C <= 4 ? 4 : (pl.C <= 8 ? 8 : 16);
        pl.T = pl.cs == 16 ? 2 : 1;
        pl.CW = pl.cs < 8 ? 4 : 8;
        per_spb = 8 * ks * 2 * pl.cs;
    }
    // a chunk = 8 boxes (one per warp) of spb steps; its staged input should fit 32 KB (three in flight), at most 64 KB (two)
    pl.spb = 0;
    for (uint32_t s = 4; s >= 1; s >>= 1) if (per_spb * s <= 32768) { pl.spb = s; break; }
    if (!pl.spb) for (uint32_t s = 4; s >= 1; s >>= 1) if (per_spb * s <= 65536) { pl.spb = s; break; }
    if (!pl.spb) return pl;
    pl.xchunk_bytes = per_spb * pl.spb;
    pl.xdepth = pl.xchunk_bytes <= 32768 ? 3 : 2;
    pl.box_bytes = ITEM_ROWS * pl.spb * 64;
    pl.nboxes = (uint32_t)((row_bytes + pl.spb * 64 - 1) / (pl.spb * 64));
    pl.nchunks = (pl.nboxes + 7) / 8;
    pl.kpad = pl.nchunks * 8 * pl.spb * ks;
    pl.items = (L->out + ITEM_ROWS - 1) / ITEM_ROWS;
    pl.staged_bytes = ((size_t)pl.kpad * (pl.intp ? 1 : 2) * pl.cs + 255) & ~(size_t)255;
    const size_t red = 2 * (size_t)(pl.intp ? 1 : CONSUMER_WARPS) * ITEM_ROWS * 8 * pl.T * 4;
    const size_t slot = 8 * (size_t)pl.box_bytes + pl.xchunk_bytes;           // one chunk: weights + its staged input
    uint32_t ring = (uint32_t)((225u * 1024 - 128 - red - 1024) / slot);
    if (ring > 8) ring = 8;
    if (ring < 2) return pl;
    pl.ring = ring;
    pl.smem = 128 + (size_t)ring * slot + red + 16 * ring + 64;
    pl.ok = true;
    return pl;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// View of the packed matrix as [out rows][row_bytes / 8] 64-bit words, boxes of 16 rows x box_row_bytes.  Cached per matrix.
int weight_map(const spgk_layer *L, uint32_t box_row_bytes, CUtensorMap *out_map)
{
    struct Entry { const void *w; uint32_t in, out, box; int prec; CUtensorMap map; };
    static Entry cache[32];
    static int used = 0, next_slot = 0;
    static std::mutex mu;
    static EncodeTiledFn fn = nullptr;
    std::lock_guard<std::mutex> lock(mu);
    for (int i = 0; i < used; i++)
        if (cache[i].w == L->w && cache[i].in == L->in && cache[i].out == L->out && cache[i].prec == L->precision && cache[i].box == box_row_bytes) { *out_map = cache[i].map; return SPGK_OK; }
    if (!fn) {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) {
            spgk_set_error("cuTensorMapEncodeTiled", "driver entry point not available");
            return SPGK_E_CUDA;
        }
        fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    const cuuint64_t row_bytes = (cuuint64_t)L->in * spg_bits_per_elem(L->precision) / 8;
    cuuint64_t dims[2] = { row_bytes / 8, L->out };          // 8-byte elements: a box row may then span 2 KB
    cuuint64_t strides[1] = { row_bytes };
    cuuint32_t box[2] = { box_row_bytes / 8, ITEM_ROWS };
    cuuint32_t estr[2] = { 1, 1 };
    CUtensorMap m;
    CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, const_cast<void *>(L->w), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        char msg[64];
        snprintf(msg, sizeof msg, "CUresult %d", (int)r);
        spgk_set_error("cuTensorMapEncodeTiled (gemv weights)", msg);
        return SPGK_E_CUDA;
    }
    Entry &e = cache[used < 32 ? used++ : (next_slot++ % 32)];
    e.w = L->w; e.in = L->in; e.out = L->out; e.box = box_row_bytes; e.prec = L->precision; e.map = m;
    *out_map = m;
    return SPGK_OK;
}

template <int PREC, int T, int CW, bool INTP>
int launch(const ChainMaps &maps, const ChainParams &ch, uint32_t grid_items, const Plan &pl, cudaStream_t s)
{
    // the opt-in for large dynamic shared memory is a per-device function attribute
    static SpgOncePerDevice once;
    int dev = 0;
    SPGK_CUDA(cudaGetDevice(&dev));
    int rc = once.run(dev, [&]() -> int {
        SPGK_CUDA(cudaFuncSetAttribute(spg_gemv_kernel<PREC, T, CW, INTP>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
        return SPGK_OK;
    });
    if (rc) return rc;
    SpgDeviceProps dp;
    if ((rc = spg_device_props(&dp))) return rc;
    const int sms = dp.sm_count;
    // one CTA per SM at most (the shared-memory ring fills an SM), so all CTAs of a launch are resident together
    const uint32_t grid = grid_items < (uint32_t)sms ? grid_items : (uint32_t)sms;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(GEMV_THREADS); cfg.dynamicSmemBytes = pl.smem; cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    SPGK_CUDA(cudaLaunchKernelEx(&cfg, spg_gemv_kernel<PREC, T, CW, INTP>, maps, ch));
    return spgk_check_launch("spg_gemv_kernel");
}

template <int PREC>
int launch_t(const ChainMaps &maps, const ChainParams &ch, uint32_t grid_items, const Plan &pl, cudaStream_t s)
{
    if (pl.cs == 4) return launch<PREC, 1, 4, false>(maps, ch, grid_items, pl, s);
    if (pl.cs == 8) return launch<PREC, 1, 8, false>(maps, ch, grid_items, pl, s);
    return launch<PREC, 2, 8, false>(maps, ch, grid_items, pl, s);
}

template <int PREC>
int launch_int(const ChainMaps &maps, const ChainParams &ch, uint32_t grid_items, const Plan &pl, cudaStream_t s)
{
    switch (pl.cs) {
        case 4:  return launch<PREC, 1, 4, true>(maps, ch, grid_items, pl, s);
        case 8:  return launch<PREC, 1, 8, true>(maps, ch, grid_items, pl, s);
        case 16: return launch<PREC, 2, 8, true>(maps, ch, grid_items, pl, s);
        case 24: return launch<PREC, 3, 8, true>(maps, ch, grid_items, pl, s);
        default: return launch<PREC, 4, 8, true>(maps, ch, grid_items, pl, s);
    }
}

int launch_any(int precision, const ChainMaps &maps, const ChainParams &ch, uint32_t grid_items, const Plan &pl, cudaStream_t s)
{
    if (pl.intp) {
        switch (precision) {
            case SPG_P_I4: return launch_int<SPG_P_I4>(maps, ch, grid_items, pl, s);
            case SPG_P_I2: return launch_int<SPG_P_I2>(maps, ch, grid_items, pl, s);
            default:       return launch_int<SPG_P_I8>(maps, ch, grid_items, pl, s);
        }
    }
    switch (precision) {
        case SPG_P_I4:   return launch_t<SPG_P_I4>(maps, ch, grid_items, pl, s);
        case SPG_P_I2:   return launch_t<SPG_P_I2>(maps, ch, grid_items, pl, s);
        case SPG_P_I8:   return launch_t<SPG_P_I8>(maps, ch, grid_items, pl, s);
        case SPG_P_BF16: return launch_t<SPG_P_BF16>(maps, ch, grid_items, pl, s);
        case SPG_P_F16:  return launch_t<SPG_P_F16>(maps, ch, grid_items, pl, s);
        default:         return launch_t<SPG_P_F32>(maps, ch, grid_items, pl, s);
    }
}

// Everything of one layer's parameters that does not depend on where its input comes from or its output goes.
void layer_params(const spgk_layer *L, const Plan &pl, uint32_t N, float *y, uint32_t ldy, void *scratch, GemvParams &p)
{
    p.bias = L->bias; p.scale = L->w_scale; p.in = L->in; p.out = L->out; p.bias_absmax = L->bias_absmax;
    p.act = L->act == SPG_ACT_SOFTMAX ? SPG_ACT_NONE : L->act;
    p.softmax = (L->act == SPG_ACT_SOFTMAX && N == 1) ? 1 : 0;     // one warp finishes one row quickly; more rows are left to the caller
    p.y = y; p.ldy = ldy;
    p.N = N; p.P = pl.P; p.C = pl.C;
    p.items = pl.items; p.nboxes = pl.nboxes; p.nchunks = pl.nchunks; p.spb = pl.spb; p.box_bytes = pl.box_bytes;
    p.ring = pl.ring; p.xdepth = pl.xdepth; p.xchunk_bytes = pl.xchunk_bytes;
    p.status = reinterpret_cast<int32_t *>(scratch);
    p.xout = nullptr; p.out_head = nullptr; p.next_prec = 0; p.next_kpad = 0;
}

// Stages x for the first layer of a launch into the scratch buffer's own staged area; returns its head.
int stage_first(const spgk_layer *L, const Plan &pl, const float *x, uint32_t ldx, uint32_t N, void *scratch, cudaStream_t s, GemvParams &p)
{
    uint8_t *base = reinterpret_cast<uint8_t *>(scratch);
    uint8_t *own_head = base + HEAD_BYTES, *own = own_head + staged_head_bytes(L->in);
    if (pl.intp)
        spg_gemv_stage_int_kernel<<<(pl.kpad + 255) / 256, 256, 0, s>>>(x, ldx, N, L->in, pl.kpad, L->precision, pl.cs, own_head, own);
    else
        spg_gemv_stage_kernel<<<(pl.kpad + 255) / 256, 256, 0, s>>>(x, ldx, N, pl.P, L->in, pl.kpad, L->precision, pl.cs,
                                                                  reinterpret_cast<__nv_bfloat16 *>(own));
    int rc = spgk_check_launch("spg_gemv_stage_kernel");
    if (rc) return rc;
    p.in_head = own_head;
    p.xin = reinterpret_cast<const uint4 *>(own);
    return SPGK_OK;
}

}  // namespace

extern "C" {

size_t spgk_gemv_scratch_bytes(const spgk_layer *L, uint32_t N)
{
    Plan pl = make_plan(L, N);
    return pl.ok ? HEAD_BYTES + staged_head_bytes(L->in) + pl.staged_bytes : 0;
}

// Bytes of a staged-input buffer for a layer of `width` inputs at N rows: head + data in either path's layout.
size_t spgk_gemv_staged_bytes(uint32_t width, uint32_t N)
{
    if (N == 0 || N > MAX_BATCH) return 0;
    const uint32_t C = N * (N == 1 ? 3u : 2u), cs = C <= 4 ? 4 : (C <= 8 ? 8 : 16);
    const size_t bf = (size_t)((width + 4095u) & ~4095u) * 2 * cs;                   // K padded to the widest chunk
    const uint32_t csi = N == 1 ? 4 : 8 * ((N + 1) / 2);
    const size_t in = (size_t)((width + 8191u) & ~8191u) * csi;
    return staged_head_bytes(width) + (((bf > in ? bf : in) + 255) & ~(size_t)255);
}

void spgk_gemv_set_int_path(int on) { g_int_path = on != 0; }
int spgk_gemv_get_int_path(void) { return g_int_path ? 1 : 0; }

int spgk_layer_gemv_chain(const spgk_layer *L, const spgk_layer *next, const void *staged_in, void *staged_out,
                          const float *x, uint32_t ldx, float *y, uint32_t ldy, uint32_t N, void *scratch, void *stream)
{
    if (!L || !y || !L->w || !L->bias || (!x && !staged_in)) { spgk_set_error("spgk_layer_gemv", "bad argument"); return SPGK_E_ARG; }
    Plan pl = make_plan(L, N);
    if (!pl.ok) return SPGK_E_UNSUPPORTED;
    if (!scratch) { spgk_set_error("spgk_layer_gemv", "scratch is NULL"); return SPGK_E_ARG; }
    cudaStream_t s = (cudaStream_t)stream;
    ChainMaps maps;
    int rc = weight_map(L, 8 * pl.spb * 64, &maps.m[0]);
    if (rc) return rc;
    ChainParams ch{};
    ch.n = 1;
    ch.sync = reinterpret_cast<int32_t *>(scratch) + 8;
    GemvParams &p = ch.L[0];
    layer_params(L, pl, N, y, ldy, scratch, p);
    if (staged_in) {
        p.in_head = reinterpret_cast<const uint8_t *>(staged_in);
        p.xin = reinterpret_cast<const uint4 *>(p.in_head + staged_head_bytes(L->in));
    } else if ((rc = stage_first(L, pl, x, ldx, N, scratch, s, p))) return rc;
    // The epilogue can stage the next layer's input directly, when that layer will also run here on the same
    // path and this layer's output needs no further pass (softmax) first.
    if (next && staged_out && L->act != SPG_ACT_SOFTMAX && next->in == L->out) {
        Plan np = make_plan(next, N);
        if (np.ok && np.intp == pl.intp) {
            p.out_head = reinterpret_cast<uint8_t *>(staged_out);
            p.xout = reinterpret_cast<__nv_bfloat16 *>(p.out_head + staged_head_bytes(next->in));
            p.next_prec = next->precision; p.next_kpad = np.kpad;
        }
    }
    return launch_any(L->precision, maps, ch, pl.items, pl, s);
}

// A whole run of layers in ONE launch: layer l's CTAs never leave the SMs, weights of layer l+1 are already on
// their way while layer l finishes, and only the staged input of l+1 waits for l (see the kernel).  All layers must
// be eligible for the kernel on the same path with the same chunk geometry (same stored precision), each feed the
// next, and only the last may be a softmax layer; otherwise SPGK_E_UNSUPPORTED and the caller goes layer by layer.
// ys[l] receives layer l's fp32 output [N][out_l]; staged_a / staged_b are the two ping-pong staged-input buffers
// (spgk_gemv_staged_bytes of the widest layer each).
int spgk_gemv_forward_chain(const spgk_layer *layers, uint32_t n, const float *x, uint32_t ldx, float *const *ys, uint32_t N,
                            void *staged_a, void *staged_b, void *scratch, void *stream)
{
    if (!layers || n == 0 || !x || !ys || !scratch || !staged_a || !staged_b) { spgk_set_error("spgk_gemv_forward_chain", "bad argument"); return SPGK_E_ARG; }
    if (n > MAX_CHAIN) return SPGK_E_UNSUPPORTED;
    Plan pls[MAX_CHAIN];
    uint32_t max_items = 0;
    for (uint32_t l = 0; l < n; l++) {
        const spgk_layer *L = &layers[l];
        if (!L->w || !L->bias || !ys[l]) { spgk_set_error("spgk_gemv_forward_chain", "bad argument"); return SPGK_E_ARG; }
        pls[l] = make_plan(L, N);
        if (!pls[l].ok) return SPGK_E_UNSUPPORTED;
        if (l > 0 && (L->in != layers[l - 1].out || L->precision != layers[0].precision || pls[l].intp != pls[0].intp || pls[l].spb != pls[0].spb ||
                      pls[l].box_bytes != pls[0].box_bytes || pls[l].xchunk_bytes != pls[0].xchunk_bytes || pls[l].ring != pls[0].ring ||
                      pls[l].cs != pls[0].cs || pls[l].smem != pls[0].smem)) return SPGK_E_UNSUPPORTED;
        if (l + 1 < n && L->act == SPG_ACT_SOFTMAX) return SPGK_E_UNSUPPORTED;
        if (pls[l].items > max_items) max_items = pls[l].items;
    }
    cudaStream_t s = (cudaStream_t)stream;
    ChainMaps maps;
    ChainParams ch{};
    ch.n = n;
    ch.sync = reinterpret_cast<int32_t *>(scratch) + 8;
    void *stg[2] = { staged_a, staged_b };
    for (uint32_t l = 0; l < n; l++) {
        const spgk_layer *L = &layers[l];
        int rc = weight_map(L, 8 * pls[l].spb * 64, &maps.m[l]);
        if (rc) return rc;
        GemvParams &p = ch.L[l];
        layer_params(L, pls[l], N, ys[l], L->out, scratch, p);
        if (l == 0) {
            if ((rc = stage_first(L, pls[0], x, ldx, N, scratch, s, p))) return rc;
        } else {
            p.in_head = reinterpret_cast<const uint8_t *>(stg[l & 1]);
            p.xin = reinterpret_cast<const uint4 *>(p.in_head + staged_head_bytes(L->in));
        }
        if (l + 1 < n) {
            p.out_head = reinterpret_cast<uint8_t *>(stg[(l + 1) & 1]);
            p.xout = reinterpret_cast<__nv_bfloat16 *>(p.out_head + staged_head_bytes(layers[l + 1].in));
            p.next_prec = layers[l + 1].precision; p.next_kpad = pls[l + 1].kpad;
        }
    }
    return launch_any(layers[0].precision, maps, ch, max_items, pls[0], s);
}

// 1 if the call above staged (or would stage) `next`'s input: lets the caller know whether to pass it on
int spgk_gemv_chain_stages_next(const spgk_layer *L, const spgk_layer *next, uint32_t N)
{
    if (!L || !next || L->act == SPG_ACT_SOFTMAX || next->in != L->out) return 0;
    const Plan a = make_plan(L, N), b = make_plan(next, N);
    return a.ok && b.ok && a.intp == b.intp ? 1 : 0;
}

// 1 if spgk_layer_gemv / spgk_layer_gemv_chain complete a softmax layer themselves at this batch (else they leave logits)
int spgk_gemv_applies_softmax(uint32_t N) { return N == 1 ? 1 : 0; }

int spgk_layer_gemv(const spgk_layer *L, const float *x, uint32_t ldx, float *y, uint32_t ldy, uint32_t N,
                    void *scratch, void *stream)
{
    if (!x) { spgk_set_error("spgk_layer_gemv", "bad argument"); return SPGK_E_ARG; }
    return spgk_layer_gemv_chain(L, nullptr, nullptr, nullptr, x, ldx, y, ldy, N, scratch, stream);
}

// Reads back the status word at the start of a GEMV scratch buffer (synchronises the stream).
int spgk_gemv_status(void *scratch, void *stream)
{
    int32_t h = 0;
    SPGK_CUDA(cudaMemcpyAsync(&h, scratch, sizeof h, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    SPGK_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    if (h == 9) {
        spgk_set_error("spg_gemv_kernel", "spgk_layer.bias_absmax is smaller than a bias of the layer");
        SPGK_CUDA(cudaMemsetAsync(scratch, 0, HEAD_BYTES, (cudaStream_t)stream));
        return SPGK_E_ARG;
    }
    if (h != 0) {
        char msg[96];
        snprintf(msg, sizeof msg, "bounded wait %d gave up inside the GEMV kernel", (int)h);
        spgk_set_error("spg_gemv_kernel", msg);
        SPGK_CUDA(cudaMemsetAsync(scratch, 0, HEAD_BYTES, (cudaStream_t)stream));      // status word, layer counters, exit ticket
        return SPGK_E_TIMEOUT;
    }
    return SPGK_OK;
}

}  // extern "C"
