// spg_mlp_fused.cu -- a three-layer MLP (in -> N1 -> N2 -> head of at most 16 outputs) as ONE
// persistent tcgen05 kernel for large batches: the layer chain of batch_forward (reference
// Training.c:313-345) without any activation matrix in HBM.
//
// A CTA owns tiles of 128 "slots" (normally 128 batch rows).  Per tile:
//   * eight converter warps read the fp32 input rows (ld.global, rows prefetched into L2 one tile ahead),
//     round them to the 16-bit operand type and write [128 x 64] K-major, 128-byte-swizzled A tiles into a
//     two-slot ring (no separate split pass, no 16-bit copy of the input in HBM);
//   * one TMA lane streams the 16-bit weight operands of layers 1 and 2 from L2 in [128 x 64] tiles through a
//     four-slot ring (cp.async.bulk.tensor, no multicast);
//   * one lane issues tcgen05.mma (kind::f16, M = 128): layer 1 in chunks of 256 output columns over K = in,
//     then layer 2 in chunks of 256 columns over K = N1, the fp32 accumulators alternating between the two
//     256-column halves of tensor memory;
//   * eight epilogue warps drain the accumulators: a layer-1 chunk becomes act(scale*acc + bias) rounded to 16
//     bits and written straight into the shared-memory A operand of layer 2 (the hidden matrix never leaves
//     the SM); a layer-2 chunk stays in registers as fp32 and is multiplied into the head's dot products
//     (fp32 FMAs), so the wide second hidden matrix is never stored anywhere; after the last chunk the row's
//     head sums get bias, softmax (Activation.c:5-21) or the head's activation, and the <= 16 outputs are
//     written.  Rows whose two largest logits are within `theta` are appended to a list (AUTO math mode).
//
// "Pair" mode computes rows exactly on the same one-term tensor-core pass: a row occupies two adjacent slots,
// one carrying the 16-bit rounding of each value and one the rounding error scaled by 2^11 (fp16) or 2^8
// (bf16); the two accumulator rows are recombined in the epilogue (hi + lo / scale), and the hidden
// activations are split the same way.  With integer, fp16 or bf16 weight files (exact 16-bit weights) every
// product is then exact and only the fp32 accumulation order differs from the reference.
//
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
constexpr uint32_t W_STAGES = 4, X_STAGES = 2, H1_TILES = 8;
constexpr uint32_t EPI_WARPS = 8, CVT_WARPS = 8;
constexpr uint32_t EPI_WARP0 = 2, CVT_WARP0 = EPI_WARP0 + EPI_WARPS;
constexpr uint32_t NUM_THREADS = 32 * (CVT_WARP0 + CVT_WARPS);        // 576: TMA, MMA, 8 epilogue, 8 converter warps
constexpr int CVT_ITEMS = 128 * 16 / (32 * CVT_WARPS);                // float4 loads per converter thread and input tile
constexpr uint32_t SMEM_TILES = (H1_TILES + W_STAGES + X_STAGES) * TILE_BYTES;   // 224 KB
constexpr uint32_t SMEM_BARS = 256;                                              // the mbarrier table, padded
constexpr uint32_t SMEM_BIAS = 2 * 256 * 4;                                      // two chunks' biases (fp32), double-buffered
constexpr uint32_t SMEM_TOTAL = SMEM_TILES + SMEM_BARS + SMEM_BIAS;
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
        mbar_wait_uniform(bar, parity, abort_addr, status, code);
        cycles += (unsigned long long)(clock64() - t0);
    } else {
        mbar_wait_uniform(bar, parity, abort_addr, status, code);
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
template <int COUNT>
__device__ __forceinline__ void activate_block(float (&v)[COUNT], int act)
{
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

// 32 accumulator columns of this thread's row -> scale*acc + bias (bias: this chunk's slice in shared memory, same address in every lane)
__device__ __forceinline__ void load_block(uint32_t taddr, float scale, const float *bias, float (&v)[32])
{
    uint32_t r0[16], r1[16];
    tmem_ld16(taddr, r0);
    tmem_ld16(taddr + 16, r1);
    tmem_ld_wait();
#pragma unroll
    for (int i = 0; i < 16; i += 4) {
        const float4 b0 = *reinterpret_cast<const float4 *>(bias + i);
        const float4 b1 = *reinterpret_cast<const float4 *>(bias + 16 + i);
        v[i + 0] = fmaf(__uint_as_float(r0[i + 0]), scale, b0.x); v[i + 1] = fmaf(__uint_as_float(r0[i + 1]), scale, b0.y);
        v[i + 2] = fmaf(__uint_as_float(r0[i + 2]), scale, b0.z); v[i + 3] = fmaf(__uint_as_float(r0[i + 3]), scale, b0.w);
        v[16 + i + 0] = fmaf(__uint_as_float(r1[i + 0]), scale, b1.x); v[16 + i + 1] = fmaf(__uint_as_float(r1[i + 1]), scale, b1.y);
        v[16 + i + 2] = fmaf(__uint_as_float(r1[i + 2]), scale, b1.z); v[16 + i + 3] = fmaf(__uint_as_float(r1[i + 3]), scale, b1.w);
    }
}
// pair mode: the raw accumulators of the hi slot (even lane) and the lo slot (odd lane) become hi + lo / lo_scale in both lanes
__device__ __forceinline__ void load_block_pairs(uint32_t taddr, float scale, const float *bias, float lo_inv, uint32_t lane, float (&v)[32])
{
    uint32_t r0[16], r1[16];
    tmem_ld16(taddr, r0);
    tmem_ld16(taddr + 16, r1);
    tmem_ld_wait();
    const bool odd = lane & 1u;
#pragma unroll
    for (int i = 0; i < 32; i++) {
        const float mine = __uint_as_float(i < 16 ? r0[i] : r1[i - 16]);
        const float other = __shfl_xor_sync(0xffffffffu, mine, 1);
        const float s = odd ? fmaf(mine, lo_inv, other) : fmaf(other, lo_inv, mine);
        v[i] = fmaf(s, scale, bias[i]);
    }
}

// One layer-1 chunk (256 columns of the hidden layer): this warp's 128 columns -> 16-bit values in the
// shared-memory A operand of layer 2 (tile kb = column / 64, row = slot, 16-byte pieces XOR-swizzled by row & 7).
template <typename T16>
__device__ __forceinline__ void epilogue_l1(const FusedParams &p, uint32_t c1, uint32_t taddr, uint32_t q, uint32_t half, uint32_t lane,
                                            uint8_t *h1, uint32_t h1_ready0, const float *cbias)
{
    const uint32_t row = q * 32u + lane;
#pragma unroll 1
    for (uint32_t pc = 0; pc < 4; pc++) {
        const uint32_t col0 = c1 * 256u + half * 128u + pc * 32u;
        const uint32_t kb = col0 >> 6;
        if (kb >= p.kb2) break;                                   // beyond the hidden width: no tile to fill
        float v[32];
        if (p.pairs) load_block_pairs(taddr + pc * 32u, p.scale1, cbias + half * 128u + pc * 32u, p.lo_inv, lane, v);
        else load_block(taddr + pc * 32u, p.scale1, cbias + half * 128u + pc * 32u, v);
        activate_block<32>(v, p.act1);
        if (col0 + 32u > p.N1) {
#pragma unroll
            for (int i = 0; i < 32; i++) if (col0 + i >= p.N1) v[i] = 0.0f;
        }
        if (p.pairs && (lane & 1u)) {
#pragma unroll
            for (int i = 0; i < 32; i++) v[i] = (v[i] - round16<T16>(v[i])) * p.lo_scale;
        }
        uint8_t *trow = h1 + kb * TILE_BYTES + row * 128u;
        const uint32_t cbase = (col0 & 63u) >> 3;                 // 0 or 4: which half of the 128-byte row
#pragma unroll
        for (uint32_t g = 0; g < 4; g++) {
            uint4 qv;
            qv.x = pack2<T16>(v[8 * g + 0], v[8 * g + 1]); qv.y = pack2<T16>(v[8 * g + 2], v[8 * g + 3]);
            qv.z = pack2<T16>(v[8 * g + 4], v[8 * g + 5]); qv.w = pack2<T16>(v[8 * g + 6], v[8 * g + 7]);
            *reinterpret_cast<uint4 *>(trow + (((cbase + g) ^ (row & 7u)) << 4)) = qv;
        }
        if (pc & 1u) {
            // this warp's 32 rows of tile kb are complete
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(h1_ready0 + 8u * kb);
        }
    }
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
// of the head's weights (16-bit, [output][column], read from L1/L2).  hd[mt][nt][4]: the head's accumulator fragments of
// row tile mt (rows 16*mt + g, +8) and output tile nt (outputs 8*nt + 2t, +1).
template <typename T16, int NT>
__device__ __forceinline__ void load_bfrag(const T16 *head, uint32_t ld16, uint32_t col0, uint32_t g, uint32_t t, uint32_t (&bf)[2][NT][2])
{
#pragma unroll
    for (int ks = 0; ks < 2; ks++)
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            const T16 *src = head + (size_t)(nt * 8 + g) * ld16 + col0 + ks * 16 + 2 * t;
            bf[ks][nt][0] = __ldg(reinterpret_cast<const uint32_t *>(src));
            bf[ks][nt][1] = __ldg(reinterpret_cast<const uint32_t *>(src + 8));
        }
}

template <typename T16, int NT>
__device__ __forceinline__ void epilogue_l2(const FusedParams &p, uint32_t c2, uint32_t taddr, uint32_t half, uint32_t lane,
                                            float (&hd)[2][NT][4], const float *cbias)
{
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint32_t ld16 = p.nch2 * 256u;
    const T16 *head = reinterpret_cast<const T16 *>(p.head16);
    const uint32_t cbase = c2 * 256u + half * 128u;
    // B fragments of a 32-column block (two k-steps of 16), fetched one block ahead of their use
    uint32_t bf[2][NT][2], bf_next[2][NT][2];
    if (cbase < p.N2) load_bfrag<T16, NT>(head, ld16, cbase, g, t, bf);
#pragma unroll 1
    for (uint32_t pc = 0; pc < 4; pc++) {
        const uint32_t col0 = cbase + pc * 32u;
        if (col0 >= p.N2) break;
        if (pc + 1 < 4 && col0 + 32u < p.N2) load_bfrag<T16, NT>(head, ld16, col0 + 32u, g, t, bf_next);
        float2 bias[4];
#pragma unroll
        for (int n = 0; n < 4; n++) bias[n] = *reinterpret_cast<const float2 *>(cbias + half * 128u + pc * 32u + 8 * n + 2 * t);
#pragma unroll
        for (int mt = 0; mt < 2; mt++) {
            uint32_t r[16];
            tmem_ld_frag32(taddr + pc * 32u + ((uint32_t)(16 * mt) << 16), r);      // rows 16*mt .. 16*mt+15 of this warp's quadrant
            tmem_ld_wait();
            float v[16];
#pragma unroll
            for (int i = 0; i < 16; i++) v[i] = __uint_as_float(r[i]);
            if (p.pairs) {
                // rows 2i (hi) and 2i+1 (lo) sit in lanes that differ by 4: both get hi + lo / lo_scale
                const bool odd = g & 1u;
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    const float other = __shfl_xor_sync(0xffffffffu, v[i], 4);
                    v[i] = odd ? fmaf(v[i], p.lo_inv, other) : fmaf(other, p.lo_inv, v[i]);
                }
            }
#pragma unroll
            for (int n = 0; n < 4; n++) {
                v[4 * n + 0] = fmaf(v[4 * n + 0], p.scale2, bias[n].x); v[4 * n + 1] = fmaf(v[4 * n + 1], p.scale2, bias[n].y);
                v[4 * n + 2] = fmaf(v[4 * n + 2], p.scale2, bias[n].x); v[4 * n + 3] = fmaf(v[4 * n + 3], p.scale2, bias[n].y);
            }
            activate_block<16>(v, p.act2);
            if (col0 + 32u > p.N2) {
                // columns beyond the layer's width were not written by this chunk's MMAs: keep stale tensor memory out
#pragma unroll
                for (int n = 0; n < 4; n++) {
                    if (col0 + 8 * n + 2 * t >= p.N2) { v[4 * n] = 0.0f; v[4 * n + 2] = 0.0f; }
                    if (col0 + 8 * n + 2 * t + 1 >= p.N2) { v[4 * n + 1] = 0.0f; v[4 * n + 3] = 0.0f; }
                }
            }
            if (p.pairs && (g & 1u)) {
#pragma unroll
                for (int i = 0; i < 16; i++) v[i] = (v[i] - round16<T16>(v[i])) * p.lo_scale;
            }
#pragma unroll
            for (int ks = 0; ks < 2; ks++) {
                uint32_t a[4];
                a[0] = pack2<T16>(v[8 * ks + 0], v[8 * ks + 1]);      // row g,   columns 16ks + 2t, +1
                a[1] = pack2<T16>(v[8 * ks + 2], v[8 * ks + 3]);      // row g+8
                a[2] = pack2<T16>(v[8 * ks + 4], v[8 * ks + 5]);      // row g,   columns 16ks + 8 + 2t, +1
                a[3] = pack2<T16>(v[8 * ks + 6], v[8 * ks + 7]);      // row g+8
#pragma unroll
                for (int nt = 0; nt < NT; nt++) mma_16816<T16>(hd[mt][nt], a, bf[ks][nt][0], bf[ks][nt][1]);
            }
        }
#pragma unroll
        for (int ks = 0; ks < 2; ks++)
#pragma unroll
            for (int nt = 0; nt < NT; nt++) { bf[ks][nt][0] = bf_next[ks][nt][0]; bf[ks][nt][1] = bf_next[ks][nt][1]; }
    }
}

template <typename T16, int NT, bool TRACE>
__global__ void __launch_bounds__(NUM_THREADS, 1)
spg_mlp3_fused_kernel(const __grid_constant__ CUtensorMap map_w1, const __grid_constant__ CUtensorMap map_w2, const FusedParams p)
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
    Bars &bars = *reinterpret_cast<Bars *>(smem + SMEM_TILES);
    float *bias_buf = reinterpret_cast<float *>(smem + SMEM_TILES + SMEM_BARS);
    uint8_t *h1 = smem;                                        // [8] layer-2 A operand tiles (hidden layer 1, 16-bit)
    const uint32_t h1_addr = base, wst_addr = base + H1_TILES * TILE_BYTES, xst_addr = wst_addr + W_STAGES * TILE_BYTES;
    uint8_t *xst = smem + (H1_TILES + W_STAGES) * TILE_BYTES;

    const uint32_t w_full0 = smem_u32(bars.w_full), w_empty0 = smem_u32(bars.w_empty);
    const uint32_t x_full0 = smem_u32(bars.x_full), x_empty0 = smem_u32(bars.x_empty);
    const uint32_t acc_full0 = smem_u32(bars.acc_full), acc_empty0 = smem_u32(bars.acc_empty);
    const uint32_t h1_ready0 = smem_u32(bars.h1_ready), xchg_full0 = smem_u32(bars.xchg_full);
    volatile int *abort_flag = &bars.abort_flag;

    // the warp index through a shuffle: provably warp-uniform, so role code stays in uniform registers
    const uint32_t warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31u;
    const uint32_t abort_addr = smem_u32(&bars.abort_flag);

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < W_STAGES; s++) { mbar_init(w_full0 + 8 * s, 1); mbar_init(w_empty0 + 8 * s, 1); }
        for (uint32_t s = 0; s < X_STAGES; s++) { mbar_init(x_full0 + 8 * s, CVT_WARPS); mbar_init(x_empty0 + 8 * s, 1); }
        for (uint32_t a = 0; a < 2; a++) { mbar_init(acc_full0 + 8 * a, 1); mbar_init(acc_empty0 + 8 * a, EPI_WARPS); }
        for (uint32_t k = 0; k < H1_TILES; k++) mbar_init(h1_ready0 + 8 * k, 4);
        for (uint32_t a = 0; a < 4; a++) mbar_init(xchg_full0 + 8 * a, 1);
        bars.abort_flag = 0;
        mbar_fence_init();
        prefetch_map(&map_w1);
        prefetch_map(&map_w2);
    }
    if (warp == 1) tmem_alloc(smem_u32(&bars.tmem_slot), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = bars.tmem_slot;
    // everything above touched only this CTA's own shared and tensor memory: it may overlap the tail of the
    // kernel in front; from here on earlier results (the row list, the count) are read
    spg_grid_trigger();
    spg_grid_wait();

    uint32_t rows = p.M;
    if (p.rows_limit) {
        const uint32_t m = *reinterpret_cast<const volatile uint32_t *>(p.rows_limit);
        rows = m < rows ? m : rows;
    }
    const uint32_t rpt = p.pairs ? BM / 2 : BM;                // rows per tile
    const uint32_t tiles = (rows + rpt - 1) / rpt;
    const uint32_t ntile = tiles > blockIdx.x ? (tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    const uint32_t nchunks = p.nch1 + p.nch2;
    const bool tracing = TRACE && p.trace != nullptr && blockIdx.x == 0;

    if (warp == 0) {
        // ------------------------------ weight producer (TMA) ------------------------------
        // the whole warp walks the loops convergently; one elected lane issues
        uint32_t it = 0;
        unsigned long long w_wait = 0;
        const long long t_begin = TRACE ? clock64() : 0;
        for (uint32_t ti = 0; ti < ntile; ti++) {
            for (uint32_t ch = 0; ch < nchunks; ch++) {
                const bool l1 = ch < p.nch1;
                const uint32_t c = l1 ? ch : ch - p.nch1;
                const uint32_t width = l1 ? p.N1 : p.N2;
                const uint32_t ncols = width - c * 256u < 256u ? width - c * 256u : 256u;
                const uint32_t nh = ncols > 128u ? 2u : 1u;
                const uint32_t kbs = l1 ? p.kb1 : p.kb2;
                const CUtensorMap *map = l1 ? &map_w1 : &map_w2;
                for (uint32_t kb = 0; kb < kbs; kb++) {
                    for (uint32_t h = 0; h < nh; h++, it++) {
                        const uint32_t s = it % W_STAGES, ph = (it / W_STAGES) & 1u;
                        uwait<TRACE>(w_empty0 + 8 * s, ph ^ 1u, abort_addr, p.status, 1, tracing, w_wait);
                        if (elect_one()) {
                            mbar_expect_tx(w_full0 + 8 * s, TILE_BYTES);
                            tma_load_2d(wst_addr + s * TILE_BYTES, map, w_full0 + 8 * s, (int)(kb * BK), (int)(c * 256u + h * 128u));
                        }
                        __syncwarp();
                    }
                }
            }
        }
        if (tracing && lane == 0) { p.trace[24] = (unsigned long long)(clock64() - t_begin); p.trace[25] = w_wait; }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        // the whole warp walks the loops convergently (all operands of tcgen05.mma stay warp-uniform); one elected lane issues
        const uint32_t fmt = std::is_same<T16, __half>::value ? 0u : 1u;
        uint32_t it = 0, xit = 0, g = 0;
        unsigned long long t_acc = 0, t_x = 0, t_h1 = 0, t_w = 0, t_issue = 0, t_commit = 0;
        const long long t_begin = TRACE ? clock64() : 0;
        for (uint32_t ti = 0; ti < ntile; ti++) {
            for (uint32_t ch = 0; ch < nchunks; ch++, g++) {
                const bool l1 = ch < p.nch1;
                const uint32_t c = l1 ? ch : ch - p.nch1;
                const uint32_t width = l1 ? p.N1 : p.N2;
                const uint32_t ncols = width - c * 256u < 256u ? width - c * 256u : 256u;
                const uint32_t nh = ncols > 128u ? 2u : 1u;
                const uint32_t kbs = l1 ? p.kb1 : p.kb2;
                const uint32_t kdim = l1 ? p.K1 : p.N1;
                const uint32_t acc = g & 1u;
                uwait<TRACE>(acc_empty0 + 8 * acc, ((g >> 1) & 1u) ^ 1u, abort_addr, p.status, 2, tracing, t_acc);
                tc_fence_after();
                for (uint32_t kb = 0; kb < kbs; kb++) {
                    uint32_t a_addr;
                    if (l1) {
                        const uint32_t xs = xit % X_STAGES;
                        uwait<TRACE>(x_full0 + 8 * xs, (xit / X_STAGES) & 1u, abort_addr, p.status, 3, tracing, t_x);
                        a_addr = xst_addr + xs * TILE_BYTES;
                    } else {
                        if (c == 0) uwait<TRACE>(h1_ready0 + 8 * kb, ti & 1u, abort_addr, p.status, 4, tracing, t_h1);
                        a_addr = h1_addr + kb * TILE_BYTES;
                    }
                    tc_fence_after();
                    const uint32_t kleft = kdim - kb * BK;
                    const uint32_t ksteps = kleft >= BK ? BK / 16u : (kleft + 15u) / 16u;
                    const uint64_t da = smem_desc_sw128(a_addr);
                    for (uint32_t h = 0; h < nh; h++, it++) {
                        const uint32_t s = it % W_STAGES;
                        uwait<TRACE>(w_full0 + 8 * s, (it / W_STAGES) & 1u, abort_addr, p.status, 5, tracing, t_w);
                        tc_fence_after();
                        const uint32_t nleft = ncols - h * 128u;
                        const uint32_t n = nleft >= 128u ? 128u : (nleft + 15u) & ~15u;
                        const uint32_t idesc = idesc_f16(fmt, fmt, n);
                        const uint64_t db = smem_desc_sw128(wst_addr + s * TILE_BYTES);
                        const uint32_t d = tmem_base + acc * 256u + h * 128u;
                        if (elect_one()) {
                            const long long t0 = (TRACE && tracing) ? clock64() : 0;
                            if (ksteps == BK / 16u) {
#pragma unroll
                                for (uint32_t k = 0; k < BK / 16u; k++) umma_f16(d, da + 2 * k, db + 2 * k, idesc, (kb | k) ? 1u : 0u);
                            } else {
                                for (uint32_t k = 0; k < ksteps; k++) umma_f16(d, da + 2 * k, db + 2 * k, idesc, (kb | k) ? 1u : 0u);
                            }
                            const long long t1 = (TRACE && tracing) ? clock64() : 0;
                            umma_commit(w_empty0 + 8 * s);               // the weight slot is free once these MMAs have read it
                            if (l1 && h + 1 == nh) umma_commit(x_empty0 + 8 * (xit % X_STAGES));
                            if (kb + 1 == kbs && h + 1 == nh) umma_commit(acc_full0 + 8 * acc);
                            if (TRACE && tracing) { t_issue += (unsigned long long)(t1 - t0); t_commit += (unsigned long long)(clock64() - t1); }
                        }
                        __syncwarp();
                    }
                    if (l1) xit++;
                }
            }
        }
        if (tracing && lane == 0) {
            p.trace[0] = (unsigned long long)(clock64() - t_begin);
            p.trace[1] = t_acc; p.trace[2] = t_x; p.trace[3] = t_h1; p.trace[4] = t_w;
        }
        if (tracing && elect_one()) { p.trace[5] = t_issue; p.trace[6] = t_commit; }
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
        unsigned long long t_full = 0, t_l1 = 0, t_l2 = 0, t_x = 0;
        const long long t_begin = clock64();
        for (uint32_t ti = 0; ti < ntile; ti++) {
            const uint32_t tile = blockIdx.x + ti * gridDim.x;
            const uint32_t r = tile * rpt + (p.pairs ? slot >> 1 : slot);
            uint32_t orow = ROW_INVALID;
            if (r < rows && !(p.pairs && (lane & 1u))) orow = p.rows_idx ? p.rows_idx[r] : r;
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
                asm volatile("bar.sync 1, %0;" ::"r"(32u * EPI_WARPS) : "memory");   // the epilogue warps only
                // after a wait has given up the warp keeps walking its chunks (the named barrier above needs every epilogue
                // warp every time) but does no more work: all later waits end at once
                if (alive && !timed_wait(acc_full0 + 8 * acc, (g >> 1) & 1u, abort_flag, p.status, 6, tracing, t_full)) alive = false;
                if (!alive) continue;
                tc_fence_after();
                const uint32_t taddr = tmem_base + acc * 256u + half * 128u + ((q * 32u) << 16);
                const bool last = ch + 1 == nchunks;
                const long long t_work = tracing ? clock64() : 0;
                if (ch < p.nch1) epilogue_l1<T16>(p, ch, taddr, q, half, lane, h1, h1_ready0, cbias);
                else epilogue_l2<T16, NT>(p, ch - p.nch1, taddr, half, lane, hd, cbias);
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
                if (lane == 0) mbar_arrive(acc_empty0 + 8 * acc);
                if (!(last && half == 0)) continue;
                if (p.pairs) {
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
                    if (p.margin_idx && orow != ROW_INVALID && p.HO >= 2 && mx - second < p.theta) p.margin_idx[atomicAdd(p.margin_count, 1u)] = orow;
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
        }
    } else {
        // ------------------------------ input converters ------------------------------
        // A step is one [128 slots x 64 columns] tile of the input: thread (cw, lane) handles, for j = 0..7, slot
        // j*16 + cw*2 + lane/16 and the four columns 4*(lane%16).., so a warp instruction reads two rows x 256 bytes.
        const uint32_t cw = warp - CVT_WARP0;
        const uint32_t sub = lane >> 4, c4 = lane & 15u;
        const uint32_t steps_per_tile = p.nch1 * p.kb1;
        const uint32_t total = ntile * steps_per_tile;
        uint32_t srow[CVT_ITEMS];
        unsigned long long t_empty = 0, t_cvt = 0;
        const long long t_begin = clock64();
        auto prefetch_tile = [&](uint32_t ti) {
            // the input rows of a whole tile into L2, one bulk prefetch per row
            if (ti >= ntile) return;
            const uint32_t t = cw * 32u + lane;
            if (t >= BM || (p.pairs && (t & 1u))) return;
            const uint32_t tile = blockIdx.x + ti * gridDim.x;
            const uint32_t r = tile * rpt + (p.pairs ? t >> 1 : t);
            if (r >= rows) return;
            const uint32_t src = p.rows_idx ? p.rows_idx[r] : r;
            const float *row = p.x + (size_t)src * p.ldx;
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(row), "r"(p.K1 * 4u) : "memory");
        };
        auto issue = [&](uint32_t step, float4 (&buf)[CVT_ITEMS]) {
            const uint32_t ti = step / steps_per_tile, kb = (step % steps_per_tile) % p.kb1;
            if (step % steps_per_tile == 0) {
                const uint32_t tile = blockIdx.x + ti * gridDim.x;
#pragma unroll
                for (int j = 0; j < CVT_ITEMS; j++) {
                    const uint32_t slot = j * (2u * CVT_WARPS) + cw * 2u + sub;
                    const uint32_t r = tile * rpt + (p.pairs ? slot >> 1 : slot);
                    srow[j] = r < rows ? (p.rows_idx ? p.rows_idx[r] : r) : ROW_INVALID;
                }
                prefetch_tile(ti + 1);
            }
            const uint32_t col = kb * BK + c4 * 4u;
#pragma unroll
            for (int j = 0; j < CVT_ITEMS; j++) {
                buf[j] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                if (srow[j] != ROW_INVALID && col < p.K1) buf[j] = __ldg(reinterpret_cast<const float4 *>(p.x + (size_t)srow[j] * p.ldx + col));
            }
        };
        auto convert = [&](uint32_t step, const float4 (&buf)[CVT_ITEMS]) -> bool {
            const uint32_t xs = step % X_STAGES;
            if (!timed_wait(x_empty0 + 8 * xs, ((step / X_STAGES) & 1u) ^ 1u, abort_flag, p.status, 8, tracing, t_empty)) return false;
            const long long t_work = tracing ? clock64() : 0;
            uint8_t *tile = xst + xs * TILE_BYTES;
#pragma unroll
            for (int j = 0; j < CVT_ITEMS; j++) {
                const uint32_t slot = j * (2u * CVT_WARPS) + cw * 2u + sub;
                float4 v = buf[j];
                if (p.pairs && (slot & 1u)) {
                    v.x = (v.x - round16<T16>(v.x)) * p.lo_scale; v.y = (v.y - round16<T16>(v.y)) * p.lo_scale;
                    v.z = (v.z - round16<T16>(v.z)) * p.lo_scale; v.w = (v.w - round16<T16>(v.w)) * p.lo_scale;
                }
                uint2 o;
                o.x = pack2<T16>(v.x, v.y); o.y = pack2<T16>(v.z, v.w);
                *reinterpret_cast<uint2 *>(tile + slot * 128u + (((c4 >> 1) ^ (slot & 7u)) << 4) + ((c4 & 1u) << 3)) = o;
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(x_full0 + 8 * xs);
            if (tracing) t_cvt += (unsigned long long)(clock64() - t_work);
            return true;
        };
        if (total) {
            // two register buffers: the loads of step s+1 are in flight while step s is converted
            prefetch_tile(0);
            float4 buf_a[CVT_ITEMS], buf_b[CVT_ITEMS];
            issue(0, buf_a);
            for (uint32_t step = 0; step < total; step += 2) {
                if (step + 1 < total) issue(step + 1, buf_b);
                if (!convert(step, buf_a)) break;
                if (step + 1 >= total) break;
                if (step + 2 < total) issue(step + 2, buf_a);
                if (!convert(step + 1, buf_b)) break;
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
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_free(tmem_base, TMEM_COLS);
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

template <typename T16, int NT, bool TRACE>
int launch_fused_t(const CUtensorMap &m1, const CUtensorMap &m2, const FusedParams &p, uint32_t grid, cudaStream_t stream)
{
    static SpgOncePerDevice once;
    int dev = 0;
    SPGK_CUDA(cudaGetDevice(&dev));
    const size_t smem = SMEM_TOTAL;
    int rc = once.run(dev, [&]() -> int {
        SPGK_CUDA(cudaFuncSetAttribute(spg_mlp3_fused_kernel<T16, NT, TRACE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        return SPGK_OK;
    });
    if (rc) return rc;
    SPGK_CUDA(spg_launch_chained(spg_mlp3_fused_kernel<T16, NT, TRACE>, dim3(grid), dim3(NUM_THREADS), smem, stream, m1, m2, p));
    return spgk_check_launch("spg_mlp3_fused_kernel");
}

template <typename T16, int NT>
int launch_fused(const CUtensorMap &m1, const CUtensorMap &m2, const FusedParams &p, uint32_t grid, cudaStream_t stream)
{
    return p.trace ? launch_fused_t<T16, NT, true>(m1, m2, p, grid, stream) : launch_fused_t<T16, NT, false>(m1, m2, p, grid, stream);
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

    const uint32_t rpt = pairs ? BM / 2 : BM;
    uint32_t guess = N;
    if (rows_limit && rows_expected && rows_expected < N) guess = rows_expected * 2u + rpt;      // a selection: few tiles expected
    if (guess > N) guess = N;
    uint32_t tiles = (guess + rpt - 1) / rpt;
    const uint32_t cap_tiles = (N + rpt - 1) / rpt;
    // the grid must cover every tile the device-side count can produce: a CTA walks tiles blockIdx.x + i * gridDim.x,
    // so any grid size is correct; the guess only avoids launching CTAs that would find nothing to do
    if (tiles > cap_tiles) tiles = cap_tiles;
    const uint32_t grid = tiles < (uint32_t)dp.sm_count ? (tiles ? tiles : 1u) : (uint32_t)dp.sm_count;
    cudaStream_t st = (cudaStream_t)stream;
    const bool narrow = L3->out <= 8;        // one or two 8-wide output tiles of the warp-level MMA
    if (type16 == SPGK_T_F16) return narrow ? launch_fused<__half, 1>(m1, m2, p, grid, st) : launch_fused<__half, 2>(m1, m2, p, grid, st);
    return narrow ? launch_fused<__nv_bfloat16, 1>(m1, m2, p, grid, st) : launch_fused<__nv_bfloat16, 2>(m1, m2, p, grid, st);
}

}  // extern "C"
