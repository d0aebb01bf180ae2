// spg_mlp_fused.cu -- a three-layer MLP (in -> N1 -> N2 -> head of at most 16 outputs) as ONE
// persistent tcgen05 kernel for large batches: the layer chain of batch_forward (reference
// Training.c:313-345) without any activation matrix in HBM.
//
// The grid is made of CTA pairs (clusters of two): a pair owns tiles of 256 "slots" (normally 256 batch rows), 128 per
// CTA, and runs them as one cta_group::2 MMA stream -- each CTA holds its own rows of the A operands and accumulators
// and only HALF of every weight tile, which halves the weight bytes per SM that have to come from L2 and sit in shared
// memory (the budget that the resident hidden layer leaves is small).  Per tile and CTA:
//   * an input-producer warp streams the fp32 input rows as [128 x 64] tiles (cp.async.bulk.tensor) into a two-slot staging
//     ring that borrows the hidden layer's shared memory while it is idle; four converter warps round them to the 16-bit
//     operand type and write [128 x 64] K-major, 128-byte-swizzled A tiles into a five-slot ring (two slots of its own,
//     three more in idle hidden tiles; no separate split pass, no 16-bit copy of the input in HBM);
//   * one TMA warp streams this CTA's half of the 16-bit weight tiles of layers 1 and 2 from L2 ([128 x 64] boxes, three-slot
//     ring; cp.async.bulk.tensor, no multicast, completion counted on the first CTA's barrier);
//   * one warp of the pair's first CTA issues tcgen05.mma (kind::f16, cta_group::2, M = 256 over the two CTAs), whole-warp
//     convergent with one elected lane: layer 1 as ONE pass over K = in whose two chunks of 256 output columns fill the two
//     256-column halves of each CTA's tensor memory side by side, then layer 2 in chunks of 256 columns over K = N1, the
//     fp32 accumulators alternating between the halves;
//   * eight epilogue warps drain the accumulators: a layer-1 chunk becomes act(scale*acc + bias) rounded to 16
//     bits and written straight into the shared-memory A operand of layer 2 (the hidden matrix never leaves
//     the SM); a layer-2 chunk is read from tensor memory in the fragment layout of the warp-level MMA, gets scale,
//     bias and activation in registers, is rounded to 16 bits and multiplied into the head's dot products with
//     mma.sync.m16n8k16 against the head's weights of the chunk (brought into shared memory a chunk ahead by bulk
//     copies), so the wide second hidden matrix is never stored anywhere; after the last chunk the row's
//     head sums get bias, softmax (Activation.c:5-21) or the head's activation, and the <= 16 outputs are
//     written.  Rows whose two largest logits are within `theta`, or whose logits are not finite, are appended to a
//     list (AUTO math mode).
//
// "Pair" mode computes rows exactly on the same one-term tensor-core pass: a row occupies two adjacent slots,
// one carrying the 16-bit rounding of each value and one the rounding error scaled by 2^11 (fp16) or 2^8
// (bf16); the two accumulator rows are recombined in the epilogue (hi + lo / scale), and the hidden
// activations are split the same way.  With integer, fp16 or bf16 weight files (exact 16-bit weights) every
// product is then exact and only the fp32 accumulation order differs from the reference.
//
// Waits and arrives are the cheap forms: a first plain try_wait (21 cycles when the phase is complete), CTA-scope
// semantics on barriers the other CTA of the pair arrives on (the waiter reads peer-written shared memory only through
// the tensor core, behind the writer's proxy fence; the cluster-scope release cost 1300 cycles per arrive here).
// Every mbarrier wait is bounded; on expiry the CTA records a code in `status`, raises a shared abort flag
// that all roles poll, lets its copies land, frees its tensor memory and returns.
#include "spg_common.cuh"
#include "spg_tc.cuh"
#include <cstdio>
#include <mutex>
#include <type_traits>

using namespace spgtc;

namespace {

constexpr uint32_t BM = 128;                    // slots per tile (UMMA M)
constexpr uint32_t BK = 64;                     // K elements per operand tile: one 128-byte swizzle row
constexpr uint32_t TILE_BYTES = BM * BK * 2;    // every operand tile here is [128 x 64] 16-bit = 16 KB
constexpr uint32_t W_STAGES = 3, H1_TILES = 8;
constexpr uint32_t XF_STAGES = 2;                                     // fp32 input staging slots ([128 rows x 64 columns] = 32 KB each), in hidden tiles 0..3
constexpr uint32_t X_PRIV = 2;                                        // 16-bit input tiles with a slot of their own
constexpr uint32_t X_STAGES = X_PRIV + (H1_TILES - 1 - 2 * XF_STAGES); // plus hidden tiles 4..6, idle while layer 1's MMAs run (tile 7: head-sum exchange)
constexpr uint32_t EPI_WARPS = 8, CVT_WARPS = 4;
constexpr uint32_t EPI_WARP0 = 2, CVT_WARP0 = EPI_WARP0 + EPI_WARPS;
constexpr uint32_t XPROD_WARP = CVT_WARP0 + CVT_WARPS;                // the input producer (TMA of fp32 input tiles)
constexpr uint32_t NUM_THREADS = 32 * (XPROD_WARP + 1);               // 480: weight TMA, MMA, 8 epilogue, 4 converter warps, input TMA
constexpr uint32_t XF_BYTES = BM * BK * 4;
constexpr int CVT_ITEMS = 128 * 16 / (32 * CVT_WARPS);                // float4 loads per converter thread and input tile
constexpr uint32_t SMEM_TILES = (H1_TILES + W_STAGES + X_PRIV) * TILE_BYTES;   // 208 KB
// the head's 16-bit weights of one layer-2 chunk, [16 outputs][256 columns], rows 16 bytes apart in the banks (pitch 528)
// so that the B-fragment reads of the warp-level MMA (8 rows x 4 words per instruction) are conflict-free; two buffers
constexpr uint32_t HEAD_PITCH = 256 * 2 + 16, HEAD_BUF = 16 * HEAD_PITCH;
constexpr uint32_t SMEM_HEAD = 2 * HEAD_BUF;
constexpr uint32_t SMEM_BARS = 384;                                              // the mbarrier table, padded
constexpr uint32_t SMEM_BIAS = 2 * 256 * 4;                                      // two chunks' biases (fp32), double-buffered
constexpr uint32_t SMEM_TOTAL = SMEM_TILES + SMEM_HEAD + SMEM_BARS + SMEM_BIAS;
static_assert(SMEM_TOTAL <= 232448, "more than the 227 KB a CTA can have");
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t MAX_N1 = H1_TILES * BK;      // the hidden operand of layer 2 must fit its 8 shared-memory tiles
constexpr uint32_t ROW_INVALID = 0xFFFFFFFFu;

struct FusedParams {
    const float *x; uint32_t ldx;               // fp32 input rows
    const uint32_t *rows_idx;                   // optional: logical row r is input/output row rows_idx[r]
    const uint32_t *rows_limit;                 // optional device-resident row count (the kernel uses min(M, *rows_limit))
    uint32_t M;                                 // logical rows (capacity)
    int pairs;                                  // 1: each row takes a hi and a lo slot
    uint32_t K1, N1, N2, HO;
    uint32_t kb1, kb2, nch1, nch2;
    float scale1, scale2, scale3;
    int act1, act2, act3, softmax3;
    const float *bias1, *bias2, *bias3;         // padded fp32: [nch1*256], [nch2*256], [16]
    const void *head16;                         // head weights as 16-bit operand: [16][nch2*256] (unscaled, zero padded)
    float *out; uint32_t ldo;
    float theta; uint32_t *margin_idx, *margin_count;
    int32_t *status;
    float lo_scale, lo_inv;
    unsigned long long *trace;                  // optional: cycle counters of CTA 0's roles (see spgk_mlp3_set_trace)
};

struct __align__(8) Bars {
    uint64_t w_full[W_STAGES], w_empty[W_STAGES], x_full[X_STAGES], x_empty[X_STAGES];
    uint64_t acc_full[2], acc_empty[2], h1_ready[H1_TILES], xchg_full[4];
    uint64_t xf_full[XF_STAGES], xf_empty[XF_STAGES], h1_free, hb_full[2];
    uint32_t tmem_slot;
    int abort_flag;
};

// a bounded wait whose duration is added to *cycles when tracing is on
__device__ __forceinline__ bool timed_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int32_t *status, int code,
                                           bool tracing, unsigned long long &cycles)
{
    if (!tracing) return mbar_wait(bar, parity, abort_flag, status, code);
    const long long t0 = clock64();
    const bool ok = mbar_wait(bar, parity, abort_flag, status, code);
    cycles += (unsigned long long)(clock64() - t0);
    return ok;
}

// the convergent-warp wait, timed when tracing (the clock reads cost the traced CTA some of its uniformity: a traced
// launch is for proportions, not for timing)
template <bool TRACE>
__device__ __forceinline__ void uwait(uint32_t bar, uint32_t parity, uint32_t abort_addr, int32_t *status, int code, bool tracing, unsigned long long &cycles)
{
    if (TRACE && tracing) {
        const long long t0 = clock64();
        mbar_wait_uniform_cluster(bar, parity, abort_addr, status, code);
        cycles += (unsigned long long)(clock64() - t0);
    } else {
        mbar_wait_uniform_cluster(bar, parity, abort_addr, status, code);
    }
}

template <typename T16> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b)
{
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&h);
}
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b)
{
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&h);
}
template <typename T16> __device__ __forceinline__ float round16(float a);
template <> __device__ __forceinline__ float round16<__half>(float a) { return __half2float(__float2half_rn(a)); }
template <> __device__ __forceinline__ float round16<__nv_bfloat16>(float a) { return __bfloat162float(__float2bfloat16_rn(a)); }

// the activation of a whole register block, resolved once per block (the switch is warp-uniform)
template <int COUNT, bool RELU = false>
__device__ __forceinline__ void activate_block(float (&v)[COUNT], int act)
{
    if (RELU) {                                      // known at compile time: no switch in the hot loop
#pragma unroll
        for (int i = 0; i < COUNT; i++) v[i] = v[i] > 0.0f ? v[i] : 0.0f;
        return;
    }
    switch (act) {
        case SPG_ACT_RELU:
#pragma unroll
            for (int i = 0; i < COUNT; i++) v[i] = v[i] > 0.0f ? v[i] : 0.0f;
            break;
        case SPG_ACT_LEAKY:
#pragma unroll
            for (int i = 0; i < COUNT; i++) v[i] = v[i] > 0.0f ? v[i] : 0.01f * v[i];
            break;
        case SPG_ACT_FOO52:
#pragma unroll
            for (int i = 0; i < COUNT; i++) v[i] = spg_activate(v[i], SPG_ACT_FOO52);
            break;
        case SPG_ACT_TANH:
#pragma unroll
            for (int i = 0; i < COUNT; i++) v[i] = tanhf(v[i]);
            break;
        case SPG_ACT_SIGMOID:
#pragma unroll
            for (int i = 0; i < COUNT; i++) v[i] = 1.0f / (1.0f + expf(-v[i]));
            break;
        default: break;
    }
}

// 16 accumulator columns of this thread's row (already in registers) -> scale*acc + bias, activation, 16-bit, and into the
// hidden tile (bias: this chunk's slice in shared memory, same address in every lane).  In pair mode the raw accumulators
// of the hi slot (even lane) and the lo slot (odd lane) first become hi + lo / lo_scale in both lanes.
template <typename T16, bool PAIRS, bool RELU>
__device__ __forceinline__ void finish_l1_half(const FusedParams &p, const uint32_t (&r)[16], const float *bias, uint32_t col0, uint32_t lane,
                                               uint8_t *trow, uint32_t chunk0, uint32_t row)
{
    float v[16];
    if (PAIRS) {
        const bool odd = lane & 1u;
#pragma unroll
        for (int i = 0; i < 16; i++) {
            const float mine = __uint_as_float(r[i]);
            const float other = __shfl_xor_sync(0xffffffffu, mine, 1);
            const float s = odd ? fmaf(mine, p.lo_inv, other) : fmaf(other, p.lo_inv, mine);
            v[i] = fmaf(s, p.scale1, bias[i]);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 16; i += 4) {
            const float4 b = *reinterpret_cast<const float4 *>(bias + i);
            v[i + 0] = fmaf(__uint_as_float(r[i + 0]), p.scale1, b.x); v[i + 1] = fmaf(__uint_as_float(r[i + 1]), p.scale1, b.y);
            v[i + 2] = fmaf(__uint_as_float(r[i + 2]), p.scale1, b.z); v[i + 3] = fmaf(__uint_as_float(r[i + 3]), p.scale1, b.w);
        }
    }
    activate_block<16, RELU>(v, p.act1);
    if (col0 + 16u > p.N1) {
#pragma unroll
        for (int i = 0; i < 16; i++) if (col0 + i >= p.N1) v[i] = 0.0f;
    }
    if (PAIRS && (lane & 1u)) {
#pragma unroll
        for (int i = 0; i < 16; i++) v[i] = (v[i] - round16<T16>(v[i])) * p.lo_scale;
    }
#pragma unroll
    for (uint32_t g = 0; g < 2; g++) {
        uint4 qv;
        qv.x = pack2<T16>(v[8 * g + 0], v[8 * g + 1]); qv.y = pack2<T16>(v[8 * g + 2], v[8 * g + 3]);
        qv.z = pack2<T16>(v[8 * g + 4], v[8 * g + 5]); qv.w = pack2<T16>(v[8 * g + 6], v[8 * g + 7]);
        *reinterpret_cast<uint4 *>(trow + (((chunk0 + g) ^ (row & 7u)) << 4)) = qv;
    }
}

// One layer-1 chunk (256 columns of the hidden layer): this warp's 128 columns -> 16-bit values in the
// shared-memory A operand of layer 2 (tile kb = column / 64, row = slot, 16-byte pieces XOR-swizzled by row & 7).
// The columns are walked in halves of 16 with the tensor-memory load of the next half in flight.
template <typename T16, bool PAIRS, bool RELU>
__device__ __forceinline__ void epilogue_l1(const FusedParams &p, uint32_t c1, uint32_t taddr, uint32_t q, uint32_t half, uint32_t lane,
                                            uint8_t *h1, uint32_t h1_ready0, const float *cbias)
{
    const uint32_t row = q * 32u + lane;
    const uint32_t cbase = c1 * 256u + half * 128u;
    const uint32_t kb_end = p.kb2;
    if ((cbase >> 6) >= kb_end) return;                         // beyond the hidden width: no tile to fill
    const float *bias = cbias + half * 128u;
    uint32_t ra[16], rb[16];
    tmem_ld16(taddr, ra);
#pragma unroll 1
    for (uint32_t pc = 0; pc < 4; pc++) {
        const uint32_t col0 = cbase + pc * 32u;
        const uint32_t kb = col0 >> 6;
        if (kb >= kb_end) break;
        uint8_t *trow = h1 + kb * TILE_BYTES + row * 128u;
        const uint32_t chunk0 = (col0 & 63u) >> 3;              // 0 or 4: which half of the 128-byte row
        tmem_ld_wait();
        tmem_ld16(taddr + pc * 32u + 16u, rb);
        finish_l1_half<T16, PAIRS, RELU>(p, ra, bias + pc * 32u, col0, lane, trow, chunk0, row);
        tmem_ld_wait();
        if (pc + 1 < 4 && ((col0 + 32u) >> 6) < kb_end) tmem_ld16(taddr + pc * 32u + 32u, ra);
        finish_l1_half<T16, PAIRS, RELU>(p, rb, bias + pc * 32u + 16u, col0 + 16u, lane, trow, chunk0 + 2u, row);
        if (pc & 1u) {
            // this warp's 32 rows of tile kb are complete
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(h1_ready0 + 8u * kb);       // a barrier of the pair's first CTA
        }
    }
    tmem_ld_wait();
}

// 16 rows x 32 columns of the accumulator in the fragment layout of the warp-level MMA: lane (g = lane/4, t = lane%4)
// gets, for each group n of 8 columns, rows g and g+8 at columns 8n+2t, 8n+2t+1 (r[4n..4n+1], r[4n+2..4n+3]).
__device__ __forceinline__ void tmem_ld_frag32(uint32_t taddr, uint32_t (&r)[16])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.16x256b.x4.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}

template <typename T16>
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    if constexpr (std::is_same<T16, __half>::value)
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    else
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// One layer-2 chunk: this warp's 32 rows x 128 columns of the second hidden layer never leave the registers.  They are
// read from tensor memory directly in the A-fragment layout of the warp-level MMA (tcgen05.ld 16x256b), get scale, bias
// and activation, are rounded to 16 bits and multiplied into the head's sums with mma.sync.m16n8k16 against B fragments
// of the head's weights (16-bit, [output][column]; this chunk's 256 columns are in shared memory, `hb`).  hd[mt][nt][4]: the head's accumulator fragments of
// row tile mt (rows 16*mt + g, +8) and output tile nt (outputs 8*nt + 2t, +1).
template <typename T16, int NT, bool PAIRS, bool RELU>
__device__ __forceinline__ void epilogue_l2(const FusedParams &p, uint32_t c2, uint32_t taddr, uint32_t half, uint32_t lane,
                                            float (&hd)[2][NT][4], const float *cbias, const uint8_t *hb)
{
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint32_t cbase = c2 * 256u + half * 128u;
    // this lane's B-fragment words: output row g (+ 8 per output tile), columns half*128 + 2t.. of the chunk
    const uint8_t *hlane = hb + g * HEAD_PITCH + (half * 128u + 2u * t) * 2u;
    // the accumulator rows of a 32-column block (two row tiles of 16) come from tensor memory while the block before
    // is worked on
    uint32_t r[2][16];
    if (cbase >= p.N2) return;
    tmem_ld_frag32(taddr, r[0]);
    tmem_ld_frag32(taddr + (16u << 16), r[1]);
#pragma unroll 1
    for (uint32_t pc = 0; pc < 4; pc++) {
        const uint32_t col0 = cbase + pc * 32u;
        if (col0 >= p.N2) break;
        const bool more = pc + 1 < 4 && col0 + 32u < p.N2;
        float2 bias[4];
#pragma unroll
        for (int n = 0; n < 4; n++) bias[n] = *reinterpret_cast<const float2 *>(cbias + half * 128u + pc * 32u + 8 * n + 2 * t);
        tmem_ld_wait();
        float v[2][16];
#pragma unroll
        for (int mt = 0; mt < 2; mt++)
#pragma unroll
            for (int i = 0; i < 16; i++) v[mt][i] = __uint_as_float(r[mt][i]);
        if (more) {                                           // the next block's rows: in flight during the arithmetic below
            tmem_ld_frag32(taddr + pc * 32u + 32u, r[0]);
            tmem_ld_frag32(taddr + pc * 32u + 32u + (16u << 16), r[1]);
        }
#pragma unroll
        for (int mt = 0; mt < 2; mt++) {
            if (PAIRS) {
                // rows 2i (hi) and 2i+1 (lo) sit in lanes that differ by 4: both get hi + lo / lo_scale
                const bool odd = g & 1u;
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    const float other = __shfl_xor_sync(0xffffffffu, v[mt][i], 4);
                    v[mt][i] = odd ? fmaf(v[mt][i], p.lo_inv, other) : fmaf(other, p.lo_inv, v[mt][i]);
                }
            }
#pragma unroll
            for (int n = 0; n < 4; n++) {
                v[mt][4 * n + 0] = fmaf(v[mt][4 * n + 0], p.scale2, bias[n].x); v[mt][4 * n + 1] = fmaf(v[mt][4 * n + 1], p.scale2, bias[n].y);
                v[mt][4 * n + 2] = fmaf(v[mt][4 * n + 2], p.scale2, bias[n].x); v[mt][4 * n + 3] = fmaf(v[mt][4 * n + 3], p.scale2, bias[n].y);
            }
            activate_block<16, RELU>(v[mt], p.act2);
            if (col0 + 32u > p.N2) {
                // columns beyond the layer's width were not written by this chunk's MMAs: keep stale tensor memory out
#pragma unroll
                for (int n = 0; n < 4; n++) {
                    if (col0 + 8 * n + 2 * t >= p.N2) { v[mt][4 * n] = 0.0f; v[mt][4 * n + 2] = 0.0f; }
                    if (col0 + 8 * n + 2 * t + 1 >= p.N2) { v[mt][4 * n + 1] = 0.0f; v[mt][4 * n + 3] = 0.0f; }
                }
            }
            if (PAIRS && (g & 1u)) {
#pragma unroll
                for (int i = 0; i < 16; i++) v[mt][i] = (v[mt][i] - round16<T16>(v[mt][i])) * p.lo_scale;
            }
        }
        // the warp-level MMAs of the block: k-step by k-step, the (row tile, output tile) accumulators are independent
#pragma unroll
        for (int ks = 0; ks < 2; ks++) {
            uint32_t a[2][4];
#pragma unroll
            for (int mt = 0; mt < 2; mt++) {
                a[mt][0] = pack2<T16>(v[mt][8 * ks + 0], v[mt][8 * ks + 1]);      // row g,   columns 16ks + 2t, +1
                a[mt][1] = pack2<T16>(v[mt][8 * ks + 2], v[mt][8 * ks + 3]);      // row g+8
                a[mt][2] = pack2<T16>(v[mt][8 * ks + 4], v[mt][8 * ks + 5]);      // row g,   columns 16ks + 8 + 2t, +1
                a[mt][3] = pack2<T16>(v[mt][8 * ks + 6], v[mt][8 * ks + 7]);      // row g+8
            }
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                const uint8_t *src = hlane + nt * 8 * HEAD_PITCH + (pc * 32u + ks * 16u) * 2u;
                const uint32_t b0 = *reinterpret_cast<const uint32_t *>(src), b1 = *reinterpret_cast<const uint32_t *>(src + 16);
#pragma unroll
                for (int mt = 0; mt < 2; mt++) mma_16816<T16>(hd[mt][nt], a[mt], b0, b1);
            }
        }
    }
    tmem_ld_wait();
}

// PAIRS: every row as a hi and a lo slot (p.pairs); RELU: both hidden activations are ReLU (known at compile time, the
// common case); otherwise they are resolved per register block at run time.
template <typename T16, int NT, bool PAIRS, bool RELU>
__global__ void __launch_bounds__(NUM_THREADS, 1)
spg_mlp3_fused_kernel(const __grid_constant__ CUtensorMap map_w1, const __grid_constant__ CUtensorMap map_w2,
                      const __grid_constant__ CUtensorMap map_x, const FusedParams p)
{
    // the whole shared memory of the SM is one dynamic block: operand tiles first (they need 1024-byte alignment
    // for the swizzle atoms, which the start of a CTA's shared window has), then the barrier table and the bias buffers
    extern __shared__ __align__(1024) uint8_t smem[];
    static_assert(sizeof(Bars) <= SMEM_BARS, "barrier table outgrew its slot");
    const uint32_t base = smem_u32(smem);
    if (base & 1023u) {                                        // never seen; checked because the tile addressing relies on it
        if (threadIdx.x == 0) atomicCAS(p.status, 0, 9);
        return;
    }
    Bars &bars = *reinterpret_cast<Bars *>(smem + SMEM_TILES + SMEM_HEAD);
    float *bias_buf = reinterpret_cast<float *>(smem + SMEM_TILES + SMEM_HEAD + SMEM_BARS);
    uint8_t *head_buf = smem + SMEM_TILES;
    uint8_t *h1 = smem;                                        // [8] layer-2 A operand tiles (hidden layer 1, 16-bit)
    const uint32_t h1_addr = base, wst_addr = base + H1_TILES * TILE_BYTES;
    // The 16-bit input tiles of layer 1: X_PRIV slots of their own, plus -- for rows in order -- the hidden tiles between
    // the fp32 staging slots and the last one (the head-sum exchange), which hold nothing while layer 1's MMAs run: their
    // contents come into being in layer 1's epilogue, after the last of those MMAs, and the next tile's input only
    // arrives once the last layer-2 MMA has read them (h1_free; rows taken through a list are fetched by the converters
    // ahead of that moment, so they wait for it themselves before a tile's first store).
    constexpr uint32_t xfn = XF_STAGES, xn = X_STAGES;
    auto x_stage_off = [&](uint32_t s) { return (s < X_PRIV ? H1_TILES + W_STAGES + s : 2u * XF_STAGES + (s - X_PRIV)) * TILE_BYTES; };

    const uint32_t w_full0 = smem_u32(bars.w_full), w_empty0 = smem_u32(bars.w_empty);
    const uint32_t x_full0 = smem_u32(bars.x_full), x_empty0 = smem_u32(bars.x_empty);
    const uint32_t acc_full0 = smem_u32(bars.acc_full), acc_empty0 = smem_u32(bars.acc_empty);
    const uint32_t h1_ready0 = smem_u32(bars.h1_ready), xchg_full0 = smem_u32(bars.xchg_full);
    const uint32_t xf_full0 = smem_u32(bars.xf_full), xf_empty0 = smem_u32(bars.xf_empty), h1_free0 = smem_u32(&bars.h1_free);
    const uint32_t hb_full0 = smem_u32(bars.hb_full);
    volatile int *abort_flag = &bars.abort_flag;

    // the warp index through a shuffle: provably warp-uniform, so role code stays in uniform registers
    const uint32_t warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31u;
    const uint32_t abort_addr = smem_u32(&bars.abort_flag);

    // The two CTAs of a cluster work as a pair: CTA `rank` owns slots 128*rank .. 128*rank+127 of a 256-slot tile.  The MMA
    // thread of rank 0 issues for both; the barriers it waits on live in ITS shared memory (both CTAs' warps arrive there),
    // and its commits arrive on the barriers at the same offsets in both CTAs.
    const uint32_t rank = cluster_rank();
    const uint32_t lead_x_full0 = mapa(x_full0, 0), lead_acc_empty0 = mapa(acc_empty0, 0), lead_h1_ready0 = mapa(h1_ready0, 0);
    const uint32_t lead_w_full0 = mapa(w_full0, 0);

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < W_STAGES; s++) { mbar_init(w_full0 + 8 * s, 1); mbar_init(w_empty0 + 8 * s, 1); }
        for (uint32_t s = 0; s < X_STAGES; s++) { mbar_init(x_full0 + 8 * s, 2 * CVT_WARPS); mbar_init(x_empty0 + 8 * s, 1); }
        for (uint32_t a = 0; a < 2; a++) { mbar_init(acc_full0 + 8 * a, 1); mbar_init(acc_empty0 + 8 * a, 2 * EPI_WARPS); }
        for (uint32_t k = 0; k < H1_TILES; k++) mbar_init(h1_ready0 + 8 * k, 2 * 4);
        for (uint32_t a = 0; a < 4; a++) mbar_init(xchg_full0 + 8 * a, 1);
        for (uint32_t s = 0; s < XF_STAGES; s++) { mbar_init(xf_full0 + 8 * s, 1); mbar_init(xf_empty0 + 8 * s, CVT_WARPS); }
        mbar_init(h1_free0, 1);
        for (uint32_t b = 0; b < 2; b++) mbar_init(hb_full0 + 8 * b, 1);
        bars.abort_flag = 0;
        mbar_fence_init();
        prefetch_map(&map_w1);
        prefetch_map(&map_w2);
    }
    if (warp == 1) tmem_alloc_pair(smem_u32(&bars.tmem_slot), TMEM_COLS);
    tc_fence_before();
    cluster_sync();                                            // both CTAs' barriers exist before anyone arrives on them
    tc_fence_after();
    const uint32_t tmem_base = bars.tmem_slot;
    // everything above touched only this pair's own shared and tensor memory: it may overlap the tail of the
    // kernel in front; from here on earlier results (the row list, the count) are read
    spg_grid_trigger();
    spg_grid_wait();

    uint32_t rows = p.M;
    if (p.rows_limit) {
        const uint32_t m = *reinterpret_cast<const volatile uint32_t *>(p.rows_limit);
        rows = m < rows ? m : rows;
    }
    const uint32_t rpt = PAIRS ? BM / 2 : BM;                // rows per CTA and tile
    const uint32_t pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
    const uint32_t tiles = (rows + 2 * rpt - 1) / (2 * rpt);   // 256-slot tiles
    const uint32_t ntile = tiles > pair ? (tiles - pair + npairs - 1) / npairs : 0;
    const uint32_t nchunks = p.nch1 + p.nch2;
    constexpr bool TRACE = true;                               // the cycle counters are a run-time switch (p.trace)
    const bool tracing = p.trace != nullptr && blockIdx.x == 0;
    // first row of this CTA in the pair's tile number ti
    auto tile_row0 = [&](uint32_t ti) { return ((pair + ti * npairs) * 2u + rank) * rpt; };

    if (warp == 0) {
        // ------------------------------ weight producer (TMA) ------------------------------
        // Per k-block each CTA fetches ITS half of the chunk's weight rows ([128 x 64] box starting at row n/2 * rank of the
        // chunk); both loads complete on the first CTA's barrier.  The whole warp walks the loops convergently; one elected
        // lane issues.
        uint32_t it = 0;
        unsigned long long w_wait = 0;
        const long long t_begin = TRACE ? clock64() : 0;
        auto load_w = [&](const CUtensorMap *map, uint32_t kb, uint32_t row) {
            const uint32_t s = it % W_STAGES, ph = (it / W_STAGES) & 1u;
            uwait<TRACE>(w_empty0 + 8 * s, ph ^ 1u, abort_addr, p.status, 1, tracing, w_wait);
            if (elect_one()) {
                if (rank == 0) mbar_expect_tx(w_full0 + 8 * s, 2 * TILE_BYTES);
                tma_load_2d_pair(wst_addr + s * TILE_BYTES, map, lead_w_full0 + 8 * s, (int)(kb * BK), (int)row);
            }
            __syncwarp();
            it++;
        };
        for (uint32_t ti = 0; ti < ntile; ti++) {
            // layer 1: one pass over K with every chunk's tile per k-block (its chunks fill the accumulators side by side)
            for (uint32_t kb = 0; kb < p.kb1; kb++)
                for (uint32_t c = 0; c < p.nch1; c++) {
                    const uint32_t ncols = p.N1 - c * 256u < 256u ? p.N1 - c * 256u : 256u;
                    load_w(&map_w1, kb, c * 256u + rank * (((ncols + 31u) & ~31u) >> 1));
                }
            // layer 2: chunk after chunk
            for (uint32_t c = 0; c < p.nch2; c++) {
                const uint32_t ncols = p.N2 - c * 256u < 256u ? p.N2 - c * 256u : 256u;
                for (uint32_t kb = 0; kb < p.kb2; kb++) load_w(&map_w2, kb, c * 256u + rank * (((ncols + 31u) & ~31u) >> 1));
            }
        }
        if (tracing && lane == 0) { p.trace[24] = (unsigned long long)(clock64() - t_begin); p.trace[25] = w_wait; }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer (first CTA of the pair only) ------------------------------
        // the whole warp walks the loops convergently (all operands of tcgen05.mma stay warp-uniform); one elected lane issues
        if (rank == 0) {
            const uint32_t fmt = std::is_same<T16, __half>::value ? 0u : 1u;
            uint32_t ws = 0, wph = 0, xs = 0, xph = 0, g = 0;   // weight and input ring positions (slot, phase), chunk counter
            const uint64_t w_desc0 = smem_desc_sw128(wst_addr);   // a slot further on adds its offset / 16 to the address field
            unsigned long long t_acc = 0, t_x = 0, t_h1 = 0, t_w = 0, t_issue = 0, t_commit = 0;
            const long long t_begin = TRACE ? clock64() : 0;
            // one k-block of MMAs: A tile at a_addr, this k-block's weight slot, accumulator `acc`, N = n
            auto kblock = [&](uint32_t a_addr, uint32_t kdim, uint32_t kb, uint32_t acc, uint32_t idesc, bool x_done, bool acc_done, bool h1_done) {
                const uint32_t s = ws;
                uwait<TRACE>(w_full0 + 8 * s, wph, abort_addr, p.status, 5, tracing, t_w);
                const uint32_t kleft = kdim - kb * BK;
                const uint32_t ksteps = kleft >= BK ? BK / 16u : (kleft + 15u) / 16u;
                const uint64_t da = smem_desc_sw128(a_addr);
                const uint64_t db = w_desc0 + (uint64_t)(s * (TILE_BYTES >> 4));
                const uint32_t d = tmem_base + acc * 256u;
                if (elect_one()) {
                    const long long t0 = (TRACE && tracing) ? clock64() : 0;
                    if (ksteps == BK / 16u) {
#pragma unroll
                        for (uint32_t k = 0; k < BK / 16u; k++) umma_f16_pair(d, da + 2 * k, db + 2 * k, idesc, (kb | k) ? 1u : 0u);
                    } else {
                        for (uint32_t k = 0; k < ksteps; k++) umma_f16_pair(d, da + 2 * k, db + 2 * k, idesc, (kb | k) ? 1u : 0u);
                    }
                    const long long t1 = (TRACE && tracing) ? clock64() : 0;
                    umma_commit_pair(w_empty0 + 8 * s);              // both CTAs' weight slots are free once these MMAs have read them
                    if (x_done) umma_commit_pair(x_empty0 + 8 * xs);
                    if (acc_done) umma_commit_pair(acc_full0 + 8 * acc);
                    if (h1_done) umma_commit_pair(h1_free0);         // the hidden tiles may be overwritten (input staging of the next tile)
                    if (TRACE && tracing) { t_issue += (unsigned long long)(t1 - t0); t_commit += (unsigned long long)(clock64() - t1); }
                }
                __syncwarp();
                if (++ws == W_STAGES) { ws = 0; wph ^= 1u; }
            };
            const uint32_t idesc1[2] = {idesc_f16_pair(fmt, fmt, ((p.N1 < 256u ? p.N1 : 256u) + 31u) & ~31u),
                                        idesc_f16_pair(fmt, fmt, ((p.N1 > 256u ? (p.N1 - 256u < 256u ? p.N1 - 256u : 256u) : 32u) + 31u) & ~31u)};
            for (uint32_t ti = 0; ti < ntile; ti++) {
                // ---- layer 1: ONE pass over the input; chunk c accumulates in accumulator (g + c) & 1 (at most two chunks) ----
                for (uint32_t c = 0; c < p.nch1; c++)
                    uwait<TRACE>(acc_empty0 + 8 * ((g + c) & 1u), (((g + c) >> 1) & 1u) ^ 1u, abort_addr, p.status, 2, tracing, t_acc);
                tc_fence_after();
                for (uint32_t kb = 0; kb < p.kb1; kb++) {
                    uwait<TRACE>(x_full0 + 8 * xs, xph, abort_addr, p.status, 3, tracing, t_x);
                    const uint32_t a_addr = base + x_stage_off(xs);
                    for (uint32_t c = 0; c < p.nch1; c++)
                        kblock(a_addr, p.K1, kb, (g + c) & 1u, idesc1[c], c + 1 == p.nch1, kb + 1 == p.kb1, false);
                    if (++xs == xn) { xs = 0; xph ^= 1u; }
                }
                g += p.nch1;
                // ---- layer 2: chunk after chunk, the hidden tiles as A operand ----
                for (uint32_t c = 0; c < p.nch2; c++, g++) {
                    const uint32_t ncols = p.N2 - c * 256u < 256u ? p.N2 - c * 256u : 256u;
                    const uint32_t acc = g & 1u;
                    const uint32_t idesc2 = idesc_f16_pair(fmt, fmt, (ncols + 31u) & ~31u);
                    uwait<TRACE>(acc_empty0 + 8 * acc, ((g >> 1) & 1u) ^ 1u, abort_addr, p.status, 2, tracing, t_acc);
                    tc_fence_after();
                    for (uint32_t kb = 0; kb < p.kb2; kb++) {
                        if (c == 0) uwait<TRACE>(h1_ready0 + 8 * kb, ti & 1u, abort_addr, p.status, 4, tracing, t_h1);
                        kblock(h1_addr + kb * TILE_BYTES, p.N1, kb, acc, idesc2, false, kb + 1 == p.kb2, c + 1 == p.nch2 && kb + 1 == p.kb2);
                    }
                }
            }
            if (tracing && lane == 0) {
                p.trace[0] = (unsigned long long)(clock64() - t_begin);
                p.trace[1] = t_acc; p.trace[2] = t_x; p.trace[3] = t_h1; p.trace[4] = t_w;
            }
            if (tracing && elect_one()) { p.trace[5] = t_issue; p.trace[6] = t_commit; }
        }
    } else if (warp < CVT_WARP0) {
        // ------------------------------ epilogue ------------------------------
        const uint32_t q = warp & 3u, half = (warp - EPI_WARP0) >> 2;    // TMEM lane quadrant of this warp; column half of a chunk
        const uint32_t slot = q * 32u + lane;
        // head-sum exchange in the last hidden tile (idle at that time): [column half][slot][16] fp32
        float *xbuf = reinterpret_cast<float *>(h1 + (H1_TILES - 1) * TILE_BYTES);
        constexpr int HP = 8 * NT;
        const uint32_t fg = lane >> 2, ft = lane & 3u;
        const uint32_t et = threadIdx.x - 32u * EPI_WARP0;                  // 0..255 among the epilogue threads
        float next_bias = __ldg(p.bias1 + et);                               // chunk 0 of the first tile
        uint32_t g = 0;
        bool alive = true;
        unsigned long long t_full = 0, t_l1 = 0, t_l2 = 0, t_x = 0, t_bar = 0;
        const long long t_begin = clock64();
        for (uint32_t ti = 0; ti < ntile; ti++) {
            const uint32_t r = tile_row0(ti) + (PAIRS ? slot >> 1 : slot);
            uint32_t orow = ROW_INVALID;
            if (r < rows && !(PAIRS && (lane & 1u))) orow = p.rows_idx ? p.rows_idx[r] : r;
            float hd[2][NT][4];
#pragma unroll
            for (int mt = 0; mt < 2; mt++)
#pragma unroll
                for (int nt = 0; nt < NT; nt++)
#pragma unroll
                    for (int i = 0; i < 4; i++) hd[mt][nt][i] = 0.0f;
            for (uint32_t ch = 0; ch < nchunks; ch++, g++) {
                const uint32_t acc = g & 1u;
                // This chunk's 256 biases go to shared memory (one value per epilogue thread, fetched while the chunk before
                // was worked on); every thread then reads its row's columns from there with broadcast loads.
                float *cbias = bias_buf + (g & 1u) * 256u;
                cbias[et] = next_bias;
                {
                    const uint32_t nch = ch + 1 < nchunks ? ch + 1 : 0;           // the chunk after this one (of this or the next tile)
                    next_bias = nch < p.nch1 ? __ldg(p.bias1 + nch * 256u + et) : __ldg(p.bias2 + (nch - p.nch1) * 256u + et);
                }
                const long long tb0 = tracing ? clock64() : 0;
                asm volatile("bar.sync 1, %0;" ::"r"(32u * EPI_WARPS) : "memory");   // the epilogue warps only
                if (tracing) t_bar += (unsigned long long)(clock64() - tb0);
                // Every epilogue warp is past the chunk before: the head-weight buffer that chunk used is free.  When the
                // chunk after this one is a layer-2 chunk, its 16 x 256 head weights are asked for now (16 bulk copies of
                // 512 bytes, one per output row), a whole chunk ahead of their first use.
                if (alive && warp == EPI_WARP0 && ch + 1 < nchunks && ch + 1 >= p.nch1) {
                    const uint32_t c2n = ch + 1 - p.nch1, hidx = ti * p.nch2 + c2n, hbuf = hidx & 1u;
                    if (lane == 0) mbar_expect_tx(hb_full0 + 8 * hbuf, 16u * 512u);
                    __syncwarp();
                    if (lane < 16)
                        bulk_load(smem_u32(head_buf + hbuf * HEAD_BUF + lane * HEAD_PITCH),
                                  reinterpret_cast<const uint8_t *>(p.head16) + ((size_t)lane * p.nch2 * 256u + c2n * 256u) * 2u, 512u, hb_full0 + 8 * hbuf);
                }
                // after a wait has given up the warp keeps walking its chunks (the named barrier above needs every epilogue
                // warp every time) but does no more work: all later waits end at once
                if (alive && !timed_wait(acc_full0 + 8 * acc, (g >> 1) & 1u, abort_flag, p.status, 6, tracing, t_full)) alive = false;
                if (!alive) continue;
                tc_fence_after();
                const uint32_t taddr = tmem_base + acc * 256u + half * 128u + ((q * 32u) << 16);
                const bool last = ch + 1 == nchunks;
                const long long t_work = tracing ? clock64() : 0;
                if (ch < p.nch1) epilogue_l1<T16, PAIRS, RELU>(p, ch, taddr, q, half, lane, h1, lead_h1_ready0, cbias);
                else {
                    const uint32_t hidx = ti * p.nch2 + (ch - p.nch1);
                    if (!timed_wait(hb_full0 + 8 * (hidx & 1u), (hidx >> 1) & 1u, abort_flag, p.status, 13, tracing, t_full)) { alive = false; continue; }
                    epilogue_l2<T16, NT, PAIRS, RELU>(p, ch - p.nch1, taddr, half, lane, hd, cbias, head_buf + (hidx & 1u) * HEAD_BUF);
                }
                if (tracing) { if (ch < p.nch1) t_l1 += (unsigned long long)(clock64() - t_work); else t_l2 += (unsigned long long)(clock64() - t_work); }
                if (last) {
                    // the rows are complete: both warps of a quadrant lay their fragments out per row; the warp of the upper
                    // column half then signals, the warp of the lower half adds the two and finishes the rows
                    float *mine = xbuf + (size_t)half * BM * 16u + (size_t)(q * 32u) * 16u;
#pragma unroll
                    for (int mt = 0; mt < 2; mt++)
#pragma unroll
                        for (int nt = 0; nt < NT; nt++) {
                            *reinterpret_cast<float2 *>(mine + (16 * mt + fg) * 16u + 8 * nt + 2 * ft) = make_float2(hd[mt][nt][0], hd[mt][nt][1]);
                            *reinterpret_cast<float2 *>(mine + (16 * mt + fg + 8) * 16u + 8 * nt + 2 * ft) = make_float2(hd[mt][nt][2], hd[mt][nt][3]);
                        }
                    __syncwarp();
                    if (half == 1) {
                        if (lane == 0) mbar_arrive(xchg_full0 + 8 * q);
                    } else if (!timed_wait(xchg_full0 + 8 * q, ti & 1u, abort_flag, p.status, 7, tracing, t_x)) { alive = false; continue; }
                }
                float hacc[HP];
                if (last && half == 0) {
                    const float *lo_half = xbuf + (size_t)slot * 16u, *hi_half = lo_half + (size_t)BM * 16u;
#pragma unroll
                    for (int j = 0; j < HP; j += 4) {
                        const float4 a = *reinterpret_cast<const float4 *>(lo_half + j), b = *reinterpret_cast<const float4 *>(hi_half + j);
                        hacc[j] = a.x + b.x; hacc[j + 1] = a.y + b.y; hacc[j + 2] = a.z + b.z; hacc[j + 3] = a.w + b.w;
                    }
                    __syncwarp();
                }
                // hand the accumulator back (after the exchange has been read: the next writer of that shared
                // memory is a layer-1 epilogue that can only start once this accumulator has been reused)
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(lead_acc_empty0 + 8 * acc);
                if (!(last && half == 0)) continue;
                if (PAIRS) {
                    // the sums of the hi slot (even lane) and the lo slot (odd lane) of a row
#pragma unroll
                    for (int j = 0; j < HP; j++) {
                        const float other = __shfl_xor_sync(0xffffffffu, hacc[j], 1);
                        hacc[j] = (lane & 1u) ? fmaf(hacc[j], p.lo_inv, other) : fmaf(other, p.lo_inv, hacc[j]);
                    }
                }
                float z[HP];
#pragma unroll
                for (int j = 0; j < HP; j++) z[j] = (uint32_t)j < p.HO ? fmaf(hacc[j], p.scale3, __ldg(p.bias3 + j)) : -FLT_MAX;
                if (p.softmax3) {
                    float mx = -FLT_MAX, second = -FLT_MAX, sum = 0.0f;
#pragma unroll
                    for (int j = 0; j < HP; j++) if ((uint32_t)j < p.HO) { if (z[j] > mx) { second = mx; mx = z[j]; } else if (z[j] > second) second = z[j]; }
#pragma unroll
                    for (int j = 0; j < HP; j++) if ((uint32_t)j < p.HO) { z[j] = expf(z[j] - mx); sum += z[j]; }
                    const float inv = sum > 0.0f ? 1.0f / sum : 1.0f;
#pragma unroll
                    for (int j = 0; j < HP; j++) z[j] *= inv;
                    // log p1 - log p2 of the softmax equals the gap of the two largest logits
                    // (a row whose one-term pass left the 16-bit range -- non-finite logits or sum -- is listed as well)
                    if (p.margin_idx && orow != ROW_INVALID && p.HO >= 2 && (!(mx - second >= p.theta) || !(sum < FLT_MAX))) p.margin_idx[atomicAdd(p.margin_count, 1u)] = orow;
                } else {
                    activate_block<HP>(z, p.act3);
                }
                if (orow != ROW_INVALID) {
                    float *o = p.out + (size_t)orow * p.ldo;
#pragma unroll
                    for (int j = 0; j < HP; j++) if ((uint32_t)j < p.HO) o[j] = z[j];
                }
            }
        }
        if (tracing && warp == EPI_WARP0 + 2 && lane == 0) {       // quadrant 0, lower column half
            p.trace[8] = (unsigned long long)(clock64() - t_begin);
            p.trace[9] = t_full; p.trace[10] = t_l1; p.trace[11] = t_l2; p.trace[12] = t_x;
            p.trace[13] = t_bar;
        }
    } else if (warp == XPROD_WARP) {
        // ------------------------------ input producer (TMA) ------------------------------
        // While layer 1 of a tile runs, the hidden tiles in shared memory are idle (their next contents only come into being
        // in layer 1's epilogue): the first 64 KB of that region serve as a two-slot ring of fp32 input tiles, filled by
        // bulk-tensor copies that need no registers; the converters empty a slot into registers as soon as it lands, so the
        // next copy is under way while they round and store.  Rows addressed through a list take the converters' own loads instead.
        if (!p.rows_idx) {
            uint32_t xfit = 0;
            for (uint32_t ti = 0; ti < ntile; ti++) {
                // the hidden tiles of the tile before must have been read by its last layer-2 MMA
                mbar_wait_uniform_cluster(h1_free0, (ti & 1u) ^ 1u, abort_addr, p.status, 10);
                const uint32_t row0 = tile_row0(ti);
                for (uint32_t kb = 0; kb < p.kb1; kb++, xfit++) {
                    const uint32_t s = xfit % xfn;
                    mbar_wait_uniform_cluster(xf_empty0 + 8 * s, ((xfit / xfn) & 1u) ^ 1u, abort_addr, p.status, 11);
                    if (elect_one()) {
                        mbar_expect_tx(xf_full0 + 8 * s, XF_BYTES);
                        tma_load_2d(h1_addr + s * XF_BYTES, &map_x, xf_full0 + 8 * s, (int)(kb * BK), (int)row0);
                    }
                    __syncwarp();
                }
            }
        }
    } else {
        // ------------------------------ input converters ------------------------------
        // A step is one [128 slots x 64 columns] tile of the input: thread (cw, lane) handles, for j = 0..15, slot
        // j*8 + cw*2 + lane/16 and the four columns 4*(lane%16).., so a warp instruction covers two rows x 256 bytes.
        // The fp32 values come from the staging ring (rows in order) or, for a row list, from global memory.
        const uint32_t cw = warp - CVT_WARP0;
        const uint32_t sub = lane >> 4, c4 = lane & 15u;
        const uint32_t steps_per_tile = p.kb1;                  // layer 1 makes one pass over the input per tile
        const uint32_t total = ntile * steps_per_tile;
        unsigned long long t_empty = 0, t_cvt = 0;
        const long long t_begin = clock64();
        // rounds, packs and writes one [128 x 64] A tile; arrives on the first CTA's barrier
        auto store_tile = [&](uint32_t step, const float4 (&buf)[CVT_ITEMS]) -> bool {
            const uint32_t xs = step % xn;
            if (!timed_wait(x_empty0 + 8 * xs, ((step / xn) & 1u) ^ 1u, abort_flag, p.status, 8, tracing, t_empty)) return false;
            uint8_t *tile = smem + x_stage_off(xs);
#pragma unroll
            for (int j = 0; j < CVT_ITEMS; j++) {
                const uint32_t slot = j * (2u * CVT_WARPS) + cw * 2u + sub;
                float4 v = buf[j];
                if (PAIRS && (slot & 1u)) {
                    v.x = (v.x - round16<T16>(v.x)) * p.lo_scale; v.y = (v.y - round16<T16>(v.y)) * p.lo_scale;
                    v.z = (v.z - round16<T16>(v.z)) * p.lo_scale; v.w = (v.w - round16<T16>(v.w)) * p.lo_scale;
                }
                uint2 o;
                o.x = pack2<T16>(v.x, v.y); o.y = pack2<T16>(v.z, v.w);
                *reinterpret_cast<uint2 *>(tile + slot * 128u + (((c4 >> 1) ^ (slot & 7u)) << 4) + ((c4 & 1u) << 3)) = o;
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(lead_x_full0 + 8 * xs);
            return true;
        };
        if (!p.rows_idx) {
            // ---- rows in order: fp32 tiles arrive in the staging ring ----
            for (uint32_t step = 0; step < total; step++) {
                const uint32_t s = step % xfn;
                const uint32_t ti = step / steps_per_tile;
                if (!timed_wait(xf_full0 + 8 * s, (step / xfn) & 1u, abort_flag, p.status, 12, tracing, t_empty)) break;
                const long long t_work = tracing ? clock64() : 0;
                const float4 *stg = reinterpret_cast<const float4 *>(h1 + s * XF_BYTES);
                const uint32_t row0 = tile_row0(ti);
                float4 buf[CVT_ITEMS];
#pragma unroll
                for (int j = 0; j < CVT_ITEMS; j++) {
                    const uint32_t slot = j * (2u * CVT_WARPS) + cw * 2u + sub;
                    const uint32_t rl = PAIRS ? slot >> 1 : slot;                 // staging row of this slot
                    buf[j] = stg[rl * 16u + c4];
                    if (row0 + rl >= rows) buf[j] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                }
                // the slot can be refilled as soon as every converter warp has its values in registers
                __syncwarp();
                if (lane == 0) mbar_arrive(xf_empty0 + 8 * s);
                if (!store_tile(step, buf)) break;
                if (tracing) t_cvt += (unsigned long long)(clock64() - t_work);
            }
        } else {
            // ---- a row list: each thread fetches its rows itself, one step ahead of the tile it writes ----
            uint32_t srow[CVT_ITEMS];
            float4 buf[CVT_ITEMS];
            auto issue = [&](uint32_t step) {
                const uint32_t ti = step / steps_per_tile, kb = step % steps_per_tile;
                if (kb == 0) {
                    const uint32_t row0 = tile_row0(ti);
#pragma unroll
                    for (int j = 0; j < CVT_ITEMS; j++) {
                        const uint32_t slot = j * (2u * CVT_WARPS) + cw * 2u + sub;
                        const uint32_t r = row0 + (PAIRS ? slot >> 1 : slot);
                        srow[j] = r < rows ? p.rows_idx[r] : ROW_INVALID;
                    }
                }
                const uint32_t col = kb * BK + c4 * 4u;
#pragma unroll
                for (int j = 0; j < CVT_ITEMS; j++) {
                    buf[j] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                    if (srow[j] != ROW_INVALID && col < p.K1) buf[j] = __ldg(reinterpret_cast<const float4 *>(p.x + (size_t)srow[j] * p.ldx + col));
                }
            };
            // the listed rows of a tile are brought into L2 as a whole (one bulk prefetch per row) before its first loads
            auto prefetch_rows = [&](uint32_t ti) {
                const uint32_t t = cw * 32u + lane;                       // 0..127: one slot each
                if (PAIRS && (t & 1u)) return;
                const uint32_t r = tile_row0(ti) + (PAIRS ? t >> 1 : t);
                if (ti >= ntile || r >= rows) return;
                const float *row = p.x + (size_t)p.rows_idx[r] * p.ldx;
                asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(row), "r"(p.K1 * 4u) : "memory");
            };
            if (total) { prefetch_rows(0); prefetch_rows(1); issue(0); }
            for (uint32_t step = 0; step < total; step++) {
                if (step % steps_per_tile == 0) {
                    if (step) prefetch_rows(step / steps_per_tile + 1);
                    // some input slots are hidden tiles: the tile before must be through its last layer-2 MMA
                    if (!timed_wait(h1_free0, ((step / steps_per_tile) & 1u) ^ 1u, abort_flag, p.status, 14, tracing, t_empty)) break;
                }
                const long long t_work = tracing ? clock64() : 0;
                if (!store_tile(step, buf)) break;
                if (step + 1 < total) issue(step + 1);
                if (tracing) t_cvt += (unsigned long long)(clock64() - t_work);
            }
        }
        if (tracing && warp == CVT_WARP0 && lane == 0) {
            p.trace[16] = (unsigned long long)(clock64() - t_begin);
            p.trace[17] = t_empty; p.trace[18] = t_cvt;
        }
    }

    // ------------------------------ common tail ------------------------------
    tc_fence_before();
    __syncthreads();
    if (bars.abort_flag && threadIdx.x == 0) {
        // a wait gave up: give weight tiles that may still be in flight time to land before the shared memory goes away
        for (int i = 0; i < 256; i++) __nanosleep(1000);
    }
    cluster_sync();            // neither CTA leaves while the other may still read its shared memory or arrive on its barriers
    if (warp == 1) {
        tc_fence_after();
        tmem_free_pair(tmem_base, TMEM_COLS);
    }
}

// parameter block of the fused kernel: fp32 bias1 [n1p] | bias2 [n2p] | head bias [16] | then the head's weights as a
// 16-bit operand [16][n2p] (unscaled stored values, zero beyond the head's real size)
template <typename T16>
__global__ void __launch_bounds__(256)
spg_mlp3_params_kernel(const float *__restrict__ b1, uint32_t n1, uint32_t n1p, const float *__restrict__ b2, uint32_t n2, uint32_t n2p,
                       const void *__restrict__ w3, int precision, uint32_t ho, const float *__restrict__ b3, float *__restrict__ dst)
{
    const uint32_t nf = n1p + n2p + 16u, total = nf + 16u * n2p;
    T16 *head = reinterpret_cast<T16 *>(dst + nf);
    for (uint32_t i = blockIdx.x * 256u + threadIdx.x; i < total; i += gridDim.x * 256u) {
        if (i < n1p) dst[i] = i < n1 ? b1[i] : 0.0f;
        else if (i < n1p + n2p) { const uint32_t c = i - n1p; dst[i] = c < n2 ? b2[c] : 0.0f; }
        else if (i < nf) { const uint32_t j = i - n1p - n2p; dst[i] = j < ho ? b3[j] : 0.0f; }
        else {
            const uint32_t e = i - nf, j = e / n2p, c = e % n2p;
            const float v = (c < n2 && j < ho) ? spg_decode_elem(w3, (uint64_t)j * n2 + c, precision) : 0.0f;
            if constexpr (std::is_same<T16, __half>::value) head[e] = __float2half_rn(v); else head[e] = __float2bfloat16_rn(v);
        }
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn()
{
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// 2-D map over a row-major [rows][ld] 16-bit weight operand whose first K columns are valid, boxes of [128 rows x 64 columns]
int weight_map(CUtensorMap *map, const void *base, int type16, uint32_t K, uint32_t rows, uint32_t ld)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) { spgk_set_error("cuTensorMapEncodeTiled", "driver entry point not available"); return SPGK_E_CUDA; }
    if (((uintptr_t)base & 15u) || (ld & 7u)) { spgk_set_error("tensor map", "weight operand is not 16-byte aligned"); return SPGK_E_ARG; }
    cuuint64_t dims[2] = { K, rows };
    cuuint64_t strides[1] = { (cuuint64_t)ld * 2 };
    cuuint32_t box[2] = { BK, 128 };
    cuuint32_t estr[2] = { 1, 1 };
    CUresult r = fn(map, type16 == SPGK_T_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                    const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        char msg[64];
        snprintf(msg, sizeof msg, "CUresult %d", (int)r);
        spgk_set_error("cuTensorMapEncodeTiled", msg);
        return SPGK_E_CUDA;
    }
    return SPGK_OK;
}

thread_local unsigned long long *tls_trace = nullptr;

// 2-D map over the fp32 input rows [rows][ld] whose first K columns are valid, boxes of [128 rows x 64 columns], no swizzle
int input_map(CUtensorMap *map, const float *x, uint32_t K, uint32_t rows, uint32_t ld)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) { spgk_set_error("cuTensorMapEncodeTiled", "driver entry point not available"); return SPGK_E_CUDA; }
    cuuint64_t dims[2] = { K, rows };
    cuuint64_t strides[1] = { (cuuint64_t)ld * 4 };
    cuuint32_t box[2] = { BK, BM };
    cuuint32_t estr[2] = { 1, 1 };
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(x), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        char msg[64];
        snprintf(msg, sizeof msg, "CUresult %d", (int)r);
        spgk_set_error("cuTensorMapEncodeTiled (input)", msg);
        return SPGK_E_CUDA;
    }
    return SPGK_OK;
}

template <typename T16, int NT, bool PAIRS, bool RELU>
int launch_fused_t(const CUtensorMap &m1, const CUtensorMap &m2, const CUtensorMap &mx, const FusedParams &p, uint32_t grid, cudaStream_t stream)
{
    static SpgOncePerDevice once;
    int dev = 0;
    SPGK_CUDA(cudaGetDevice(&dev));
    const size_t smem = SMEM_TOTAL;
    int rc = once.run(dev, [&]() -> int {
        SPGK_CUDA(cudaFuncSetAttribute(spg_mlp3_fused_kernel<T16, NT, PAIRS, RELU>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        return SPGK_OK;
    });
    if (rc) return rc;
    // clusters of two CTAs (one MMA pair per cluster); programmatic stream serialisation as for the other chained kernels
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(NUM_THREADS); cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 2;
    SPGK_CUDA(cudaLaunchKernelEx(&cfg, spg_mlp3_fused_kernel<T16, NT, PAIRS, RELU>, m1, m2, mx, p));
    return spgk_check_launch("spg_mlp3_fused_kernel");
}

template <typename T16>
int launch_fused(const CUtensorMap &m1, const CUtensorMap &m2, const CUtensorMap &mx, const FusedParams &p, bool relu, uint32_t grid, cudaStream_t stream)
{
    // the warp-level MMA of the head always covers 16 outputs (two tiles of 8)
    if (p.pairs) return relu ? launch_fused_t<T16, 2, true, true>(m1, m2, mx, p, grid, stream) : launch_fused_t<T16, 2, true, false>(m1, m2, mx, p, grid, stream);
    return relu ? launch_fused_t<T16, 2, false, true>(m1, m2, mx, p, grid, stream) : launch_fused_t<T16, 2, false, false>(m1, m2, mx, p, grid, stream);
}

}  // namespace

extern "C" {

void spgk_mlp3_set_trace(unsigned long long *trace32) { tls_trace = trace32; }

int spgk_mlp3_supported(const spgk_layer *L1, const spgk_layer *L2, const spgk_layer *L3, uint32_t ldx)
{
    if (!L1 || !L2 || !L3 || !L1->w || !L2->w || !L3->w || !L1->bias || !L2->bias || !L3->bias) return 0;
    if (L2->in != L1->out || L3->in != L2->out) return 0;
    if (L1->act == SPG_ACT_SOFTMAX || L2->act == SPG_ACT_SOFTMAX) return 0;
    if (L1->in < 16 || (L1->in & 3u) || (ldx & 3u) || ldx < L1->in) return 0;          // 16-byte vector loads of the input rows
    if (L1->out < 16 || L1->out > MAX_N1 || (L1->out & 7u)) return 0;                  // hidden operand in shared memory; TMA rows of W2
    if (L2->out < 16 || L3->out == 0 || L3->out > 16) return 0;
    if ((unsigned)L3->precision >= SPG_P_COUNT) return 0;
    SpgDeviceProps dp;
    if (spg_device_props(&dp) != SPGK_OK) return 0;
    return (dp.cc == 100 && dp.smem_optin >= SMEM_TOTAL) ? 1 : 0;
}

size_t spgk_mlp3_params_bytes(const spgk_layer *L1, const spgk_layer *L2, const spgk_layer *L3)
{
    if (!L1 || !L2 || !L3) return 0;
    const size_t n1p = (size_t)((L1->out + 255u) / 256u) * 256u, n2p = (size_t)((L2->out + 255u) / 256u) * 256u;
    return (n1p + n2p + 16u) * sizeof(float) + 16u * n2p * 2u;
}

int spgk_mlp3_params(const spgk_layer *L1, const spgk_layer *L2, const spgk_layer *L3, int type16, float *dst, void *stream)
{
    if (!L1 || !L2 || !L3 || !dst || (type16 != SPGK_T_F16 && type16 != SPGK_T_BF16)) { spgk_set_error("spgk_mlp3_params", "bad argument"); return SPGK_E_ARG; }
    const uint32_t n1p = ((L1->out + 255u) / 256u) * 256u, n2p = ((L2->out + 255u) / 256u) * 256u;
    const uint32_t total = n1p + n2p + 16u + 16u * n2p;
    if (type16 == SPGK_T_F16)
        spg_mlp3_params_kernel<__half><<<(total + 255u) / 256u, 256, 0, (cudaStream_t)stream>>>(L1->bias, L1->out, n1p, L2->bias, L2->out, n2p,
                                                                                                 L3->w, L3->precision, L3->out, L3->bias, dst);
    else
        spg_mlp3_params_kernel<__nv_bfloat16><<<(total + 255u) / 256u, 256, 0, (cudaStream_t)stream>>>(L1->bias, L1->out, n1p, L2->bias, L2->out, n2p,
                                                                                                        L3->w, L3->precision, L3->out, L3->bias, dst);
    return spgk_check_launch("spg_mlp3_params_kernel");
}

int spgk_mlp3_forward(const spgk_layer *L1, const void *w1_16, uint32_t ldw1,
                      const spgk_layer *L2, const void *w2_16, uint32_t ldw2,
                      const spgk_layer *L3, const float *params, int type16,
                      const float *x, uint32_t ldx, const uint32_t *rows_idx, const uint32_t *rows_limit, uint32_t rows_expected,
                      int pairs, float *out, uint32_t ldo, uint32_t N,
                      float theta, uint32_t *margin_idx, uint32_t *margin_count,
                      int32_t *status, void *stream)
{
    if (!w1_16 || !w2_16 || !params || !x || !out || !status || (type16 != SPGK_T_F16 && type16 != SPGK_T_BF16) ||
        ((uintptr_t)x & 15u) || !spgk_mlp3_supported(L1, L2, L3, ldx) || ldo < L3->out) {
        spgk_set_error("spgk_mlp3_forward", "bad argument or unsupported shape");
        return SPGK_E_ARG;
    }
    if (N == 0) return SPGK_OK;
    SpgDeviceProps dp;
    int rc = spg_device_props(&dp);
    if (rc) return rc;
    FusedParams p{};
    p.x = x; p.ldx = ldx; p.rows_idx = rows_idx; p.rows_limit = rows_limit; p.M = N; p.pairs = pairs ? 1 : 0;
    p.K1 = L1->in; p.N1 = L1->out; p.N2 = L2->out; p.HO = L3->out;
    p.kb1 = (p.K1 + BK - 1) / BK; p.kb2 = (p.N1 + BK - 1) / BK;
    p.nch1 = (p.N1 + 255u) / 256u; p.nch2 = (p.N2 + 255u) / 256u;
    p.scale1 = L1->w_scale; p.scale2 = L2->w_scale; p.scale3 = L3->w_scale;
    p.act1 = L1->act; p.act2 = L2->act;
    p.softmax3 = L3->act == SPG_ACT_SOFTMAX ? 1 : 0;
    p.act3 = p.softmax3 ? SPG_ACT_NONE : L3->act;
    const uint32_t n1p = p.nch1 * 256u, n2p = p.nch2 * 256u;
    p.bias1 = params; p.bias2 = params + n1p; p.bias3 = params + n1p + n2p; p.head16 = params + n1p + n2p + 16u;
    p.out = out; p.ldo = ldo;
    if (margin_idx && margin_count && !pairs) { p.theta = theta; p.margin_idx = margin_idx; p.margin_count = margin_count; }
    p.status = status;
    p.trace = tls_trace;
    p.lo_scale = type16 == SPGK_T_F16 ? 2048.0f : 256.0f;
    p.lo_inv = 1.0f / p.lo_scale;

    CUtensorMap m1, m2;
    if ((rc = weight_map(&m1, w1_16, type16, L1->in, L1->out, ldw1))) return rc;
    if ((rc = weight_map(&m2, w2_16, type16, L2->in, L2->out, ldw2))) return rc;
    CUtensorMap mx = m1;                                         // unused with a row list
    if (!rows_idx && (rc = input_map(&mx, x, L1->in, N, ldx))) return rc;

    const uint32_t rpt2 = pairs ? BM : 2 * BM;                  // rows of a 256-slot tile (one per CTA pair)
    uint32_t guess = N;
    if (rows_limit && rows_expected && rows_expected < N) guess = rows_expected * 2u + rpt2;      // a selection: few tiles expected
    if (guess > N) guess = N;
    uint32_t tiles = (guess + rpt2 - 1) / rpt2;
    // A pair walks tiles pair + i * pairs, so any grid size covers every tile the device-side count can produce; the guess
    // only avoids launching pairs that would find nothing to do.
    const uint32_t max_pairs = (uint32_t)dp.sm_count / 2u;
    const uint32_t npairs = tiles < max_pairs ? (tiles ? tiles : 1u) : max_pairs;
    const uint32_t grid = 2u * npairs;
    cudaStream_t st = (cudaStream_t)stream;
    const bool relu = L1->act == SPG_ACT_RELU && L2->act == SPG_ACT_RELU;
    if (type16 == SPGK_T_F16) return launch_fused<__half>(m1, m2, mx, p, relu, grid, st);
    return launch_fused<__nv_bfloat16>(m1, m2, mx, p, relu, grid, st);
}

}  // extern "C"
