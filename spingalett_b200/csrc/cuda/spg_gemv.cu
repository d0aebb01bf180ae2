// spg_gemv.cu -- K1: small-batch (1..8 rows) fused dequant-GEMV layer.
//
//   y[n][j] = act(bias[j] + w_scale * sum_k q[j][k] * x[n][k])
//
// The layer is bound by reading the packed weights once from HBM, so the kernel
// is organised around that stream: every lane issues 128-bit loads of two weight
// rows (rows g and g+8 of a 16-row group), a warp walks 4 such loads (= 4 lanes
// per row) per step along K, several steps are kept in flight, and the packed
// integers are expanded to bf16 in registers with mask/magic-number tricks (no
// per-element conversion instruction).  The multiply-accumulate runs on the
// warp-level tensor path (mma.sync m16n8k16, bf16 x bf16 -> fp32): the 16 weight
// rows are the M dimension and the batch is the N dimension.  To keep fp32-class
// accuracy the activations enter as two or three bf16 terms (x = x1 + x2 [+ x3]),
// each term occupying its own column of the N dimension, and weights that are not
// exact in bf16 enter as several exact bf16 terms too (INT8 = 16*high nibble + low
// nibble, FP16 = 8+3 bits, FP32 = 8+8+8 bits); integer and BF16 weights are exact
// in one term.  All products are therefore exact and only the fp32 summation
// order differs from the reference's fp32 dot product (SIMD.c:190-240).
//
// Because the K order inside one MMA is arbitrary as long as both operands agree,
// the activation chunk is staged in shared memory in exactly the order in which
// the mask tricks deliver the weights ("fragment order"), so no shuffles are needed.
//
// Grid: (row blocks of 128 rows) x (K splits).  Each CTA writes fp32 partial sums;
// the last CTA to finish a row block (atomic ticket) reduces the splits and the
// activation terms, applies scale, bias and activation and writes y.  The ticket
// counters live at the start of the scratch buffer, must be zero before the first
// use and are left at zero.
#include "spg_common.cuh"
#include <cstdio>

namespace {

constexpr int GEMV_THREADS = 256;          // 8 warps x 16 rows = 128 rows per CTA
constexpr int ROWS_PER_CTA = 128;
constexpr int MAX_BATCH = 8;

struct GemvParams {
    const void *w;
    const float *bias;
    float scale;
    uint32_t in, out;
    int act;
    const float *x; uint32_t ldx;
    float *y; uint32_t ldy;
    uint32_t N, P, C;                       // rows, bf16 terms per row, C = N*P columns in use
    uint32_t kchunk, splits, row_blocks;
    uint32_t *tickets;                      // [row_blocks]
    float *partial;                         // [splits][row_blocks*128][8*T]
    const uint4 *xin;                       // this layer's staged input (see staged_index)
    __nv_bfloat16 *xout;                    // staged input of the next layer, written by the finishing CTAs (or NULL)
    int next_prec; uint32_t next_kpad;      // precision of the next layer's weights; its K rounded up to a whole step
};

// elements covered by one 128-bit load, per stored precision
template <int PREC> struct Fmt;
template <> struct Fmt<SPG_P_I4>   { static constexpr int EL = 32, BITS = 4; };
template <> struct Fmt<SPG_P_I2>   { static constexpr int EL = 64, BITS = 2; };
template <> struct Fmt<SPG_P_I8>   { static constexpr int EL = 16, BITS = 8; };
template <> struct Fmt<SPG_P_BF16> { static constexpr int EL = 8,  BITS = 16; };
template <> struct Fmt<SPG_P_F16>  { static constexpr int EL = 8,  BITS = 16; };
template <> struct Fmt<SPG_P_F32>  { static constexpr int EL = 4,  BITS = 32; };

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

__host__ __device__ inline uint32_t elems_per_load(int prec) { return 128u / spg_bits_per_elem(prec); }

// Index (in bf16 units) of activation element k, column `col`, inside a staged-input buffer laid out as
// [step][block][tile][t][8 columns][4]: the order in which the weight loads of a layer stored in
// precision `prec` consume it.  T = column tiles of 8.
__device__ __forceinline__ uint64_t staged_index(int prec, uint32_t T, uint32_t k, uint32_t col)
{
    const uint32_t el = elems_per_load(prec), ks = 4 * el, nb = el / 4;
    const uint32_t step = k / ks, rem = k % ks, tt = rem / el, e = rem % el;
    uint32_t block, r;
    frag_pos(prec, e, block, r);
    const uint64_t slot = ((((uint64_t)step * nb + block) * T + (col >> 3)) * 4 + tt) * 8 + (col & 7u);
    return slot * 4 + r;
}

// Splits v into P bf16 terms (term i = round(v - earlier terms)) and stores them for columns n*P .. n*P+P-1.
__device__ __forceinline__ void stage_value(__nv_bfloat16 *dst, int prec, uint32_t T, uint32_t k, uint32_t n, uint32_t P, float v)
{
    for (uint32_t q = 0; q < P; q++) {
        const __nv_bfloat16 h = __float2bfloat16_rn(v);
        dst[staged_index(prec, T, k, n * P + q)] = h;
        v -= __bfloat162float(h);
    }
}

// Stages a whole activation matrix x[N][in] (fp32) for a layer of precision `prec`: one thread per k.
// Elements k in [in, kpad) are written as zero so that the last partial step multiplies by zero.
__global__ void __launch_bounds__(256)
spg_gemv_stage_kernel(const float *__restrict__ x, uint32_t ldx, uint32_t N, uint32_t P, uint32_t in, uint32_t kpad,
                      int prec, uint32_t T, __nv_bfloat16 *__restrict__ dst)
{
    const uint32_t k = blockIdx.x * 256 + threadIdx.x;
    if (k >= kpad) return;
    for (uint32_t n = 0; n < N; n++) stage_value(dst, prec, T, k, n, P, k < in ? x[(uint64_t)n * ldx + k] : 0.0f);
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

template <int PREC, int T>
__global__ void __launch_bounds__(GEMV_THREADS)
spg_gemv_kernel(const GemvParams p)
{
    using F = Fmt<PREC>;
    constexpr int EL = F::EL, KS = 4 * EL, NB = EL / 4;       // per warp step: 4 lanes x EL elements; NB B-blocks per load
    constexpr int CPAD = 8 * T;
    extern __shared__ uint2 xs[];                             // [step][block][tile][t][8 columns] of 4 bf16
    __shared__ int s_last;

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u, g = lane >> 2, t = lane & 3u;
    const uint32_t rb = blockIdx.x, split = blockIdx.y;
    const uint32_t k0 = split * p.kchunk;
    const uint32_t kend = min(k0 + p.kchunk, p.in);
    const uint32_t steps = (kend - k0 + KS - 1) / KS;

    // ---- issue the first weight loads before staging x, so the two overlap ----
    const uint32_t row_a = rb * ROWS_PER_CTA + warp * 16 + g, row_b = row_a + 8;
    const uint8_t *wbase = reinterpret_cast<const uint8_t *>(p.w);
    auto load_row = [&](uint32_t row, uint32_t step) -> uint4 {
        const uint32_t kk = k0 + step * KS + t * EL;
        if (row < p.out && kk < kend)
            return __ldcs(reinterpret_cast<const uint4 *>(wbase + (((uint64_t)row * p.in + kk) * F::BITS >> 3)));
        return make_uint4(0, 0, 0, 0);                         // zero bits decode to zero in every format
    };
    constexpr int U = 4;                                       // steps in flight per thread (8 x 128-bit loads)
    uint4 ra[U], rbw[U];
#pragma unroll
    for (int u = 0; u < U; u++) { ra[u] = load_row(row_a, u); rbw[u] = load_row(row_b, u); }

    // ---- copy this chunk of the staged input (already split into bf16 terms, in fragment order) ----
    {
        const uint32_t per_step = NB * T * 16;                 // 16-byte units per step
        const uint4 *src = p.xin + (size_t)(k0 / KS) * per_step;
        uint4 *dst = reinterpret_cast<uint4 *>(xs);
        for (uint32_t i = tid; i < steps * per_step; i += GEMV_THREADS) dst[i] = __ldg(src + i);
    }
    __syncthreads();

    float acc[T][4];
    float acc_hi[T][4];                                        // INT8 only: the high-nibble term
#pragma unroll
    for (int i = 0; i < T; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) { acc[i][j] = 0.0f; acc_hi[i][j] = 0.0f; }

    for (uint32_t s0 = 0; s0 < steps; s0 += U) {
        uint4 ca[U], cb[U];
#pragma unroll
        for (int u = 0; u < U; u++) { ca[u] = ra[u]; cb[u] = rbw[u]; }
#pragma unroll
        for (int u = 0; u < U; u++) {                          // next group's loads go out before this group's math
            ra[u] = load_row(row_a, s0 + U + u);
            rbw[u] = load_row(row_b, s0 + U + u);
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
            const uint32_t step = s0 + u;
            if (step >= steps) break;
            const uint32_t wa[4] = { ca[u].x, ca[u].y, ca[u].z, ca[u].w };
            const uint32_t wb[4] = { cb[u].x, cb[u].y, cb[u].z, cb[u].w };
            const uint2 *xb = xs + (size_t)step * NB * T * 32 + t * 8 + g;
#pragma unroll
            for (int b = 0; b < NB; b++) {
                uint2 bf[T];
#pragma unroll
                for (int i = 0; i < T; i++) bf[i] = xb[(b * T + i) * 32];
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
    }

    // ---- partial sums of this K split: [split][row][column] ----
    const uint32_t out_pad = p.row_blocks * ROWS_PER_CTA;
    float *pp = p.partial + ((uint64_t)split * out_pad) * CPAD;
#pragma unroll
    for (int i = 0; i < T; i++) {
        float d0 = acc[i][0], d1 = acc[i][1], d2 = acc[i][2], d3 = acc[i][3];
        if (PREC == SPG_P_I8) {
            d0 = fmaf(16.0f, acc_hi[i][0], d0); d1 = fmaf(16.0f, acc_hi[i][1], d1);
            d2 = fmaf(16.0f, acc_hi[i][2], d2); d3 = fmaf(16.0f, acc_hi[i][3], d3);
        }
        __stcg(reinterpret_cast<float2 *>(pp + (uint64_t)row_a * CPAD + i * 8 + 2 * t), make_float2(d0, d1));
        __stcg(reinterpret_cast<float2 *>(pp + (uint64_t)row_b * CPAD + i * 8 + 2 * t), make_float2(d2, d3));
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const uint32_t ticket = atomicAdd(&p.tickets[rb], 1u);
        s_last = ticket == p.splits - 1;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();

    // ---- the last CTA of this row block finishes it: sum splits and terms, scale, bias, activation ----
    for (uint32_t idx = tid; idx < ROWS_PER_CTA * p.N; idx += GEMV_THREADS) {
        const uint32_t n = idx / ROWS_PER_CTA, row = rb * ROWS_PER_CTA + idx % ROWS_PER_CTA;
        if (row >= p.out) continue;
        float sum = 0.0f;
        for (uint32_t s = 0; s < p.splits; s++) {
            const float *src = p.partial + ((uint64_t)s * out_pad + row) * CPAD + n * p.P;
            float part = 0.0f;
            for (uint32_t q = p.P; q-- > 0;) part += __ldcg(src + q);      // smallest term first
            sum += part;
        }
        const float yv = spg_activate(fmaf(sum, p.scale, p.bias[row]), p.act);
        p.y[(uint64_t)n * p.ldy + row] = yv;
        if (p.xout) stage_value(p.xout, p.next_prec, T, row, n, p.P, yv);
    }
    if (p.xout && rb == p.row_blocks - 1) {
        // zero the tail of the next layer's last step (k in [out, next_kpad)), all columns
        for (uint32_t idx = tid; idx < (p.next_kpad - p.out) * CPAD; idx += GEMV_THREADS)
            p.xout[staged_index(p.next_prec, T, p.out + idx / CPAD, idx % CPAD)] = __float2bfloat16_rn(0.0f);
    }
    if (tid == 0) p.tickets[rb] = 0;                           // leave the counter ready for the next call
}

struct Plan { uint32_t P, C, T, kchunk, splits, row_blocks, kpad; size_t tickets_bytes, partial_bytes, staged_bytes, smem; bool ok; };

int bits_of(int prec) { return (int)spg_bits_per_elem(prec); }

Plan make_plan(const spgk_layer *L, uint32_t N)
{
    Plan pl{};
    pl.ok = false;
    if (!L || N == 0 || N > MAX_BATCH || (unsigned)L->precision >= SPG_P_COUNT) return pl;
    const uint32_t el = 128u / (uint32_t)bits_of(L->precision), ks = 4 * el;
    // 128-bit loads need 16-byte aligned packed rows
    if (L->in % el || ((uintptr_t)L->w & 15u)) return pl;
    pl.P = N <= 2 ? 3 : 2;
    pl.C = N * pl.P;
    pl.T = (pl.C + 7) / 8;
    pl.row_blocks = (L->out + ROWS_PER_CTA - 1) / ROWS_PER_CTA;
    // enough CTAs for ~4 per SM, K chunks a multiple of the widest step (256), shared memory <= 64 KB
    uint32_t want = (148u * 4 + pl.row_blocks - 1) / pl.row_blocks;
    uint32_t kchunk = (L->in + want - 1) / want;
    kchunk = (kchunk + 255u) & ~255u;
    if (kchunk < 512) kchunk = 512;
    const uint32_t cap = 65536u / (16u * pl.T);                 // bytes per k element = 8*T columns * 2
    if (kchunk > cap) kchunk = cap;
    kchunk = kchunk / ks * ks;
    pl.kchunk = kchunk;
    pl.splits = (L->in + kchunk - 1) / kchunk;
    pl.tickets_bytes = ((size_t)pl.row_blocks * 4 + 255) & ~(size_t)255;
    pl.partial_bytes = (size_t)pl.splits * pl.row_blocks * ROWS_PER_CTA * 8 * pl.T * sizeof(float);
    pl.smem = (size_t)((kchunk + ks - 1) / ks) * ks * 16 * pl.T;
    pl.kpad = (L->in + ks - 1) / ks * ks;
    pl.staged_bytes = ((size_t)pl.kpad * 16 * pl.T + 255) & ~(size_t)255;
    pl.ok = true;
    return pl;
}

template <int PREC, int T>
int launch(const GemvParams &p, const Plan &pl, cudaStream_t s)
{
    static bool attr_done = false;
    if (!attr_done) {
        SPGK_CUDA(cudaFuncSetAttribute(spg_gemv_kernel<PREC, T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536));
        attr_done = true;
    }
    dim3 grid(pl.row_blocks, pl.splits);
    spg_gemv_kernel<PREC, T><<<grid, GEMV_THREADS, pl.smem, s>>>(p);
    return spgk_check_launch("spg_gemv_kernel");
}

template <int PREC>
int launch_t(const GemvParams &p, const Plan &pl, cudaStream_t s)
{
    return pl.T == 1 ? launch<PREC, 1>(p, pl, s) : launch<PREC, 2>(p, pl, s);
}

}  // namespace

extern "C" {

size_t spgk_gemv_scratch_bytes(const spgk_layer *L, uint32_t N)
{
    Plan pl = make_plan(L, N);
    return pl.ok ? pl.tickets_bytes + pl.partial_bytes + pl.staged_bytes : 0;
}

size_t spgk_gemv_staged_bytes(uint32_t width, uint32_t N)
{
    if (N == 0 || N > MAX_BATCH) return 0;
    const uint32_t T = (N * (N <= 2 ? 3u : 2u) + 7) / 8;
    return ((size_t)((width + 255u) & ~255u) * 16 * T + 255) & ~(size_t)255;
}

int spgk_layer_gemv_chain(const spgk_layer *L, const spgk_layer *next, const void *staged_in, void *staged_out,
                          const float *x, uint32_t ldx, float *y, uint32_t ldy, uint32_t N, void *scratch, void *stream)
{
    if (!L || !y || !L->w || !L->bias || (!x && !staged_in)) { spgk_set_error("spgk_layer_gemv", "bad argument"); return SPGK_E_ARG; }
    Plan pl = make_plan(L, N);
    if (!pl.ok) return SPGK_E_UNSUPPORTED;
    if (!scratch) { spgk_set_error("spgk_layer_gemv", "scratch is NULL"); return SPGK_E_ARG; }
    cudaStream_t s = (cudaStream_t)stream;
    GemvParams p{};
    p.w = L->w; p.bias = L->bias; p.scale = L->w_scale; p.in = L->in; p.out = L->out;
    p.act = L->act == SPG_ACT_SOFTMAX ? SPG_ACT_NONE : L->act;
    p.x = x; p.ldx = ldx; p.y = y; p.ldy = ldy;
    p.N = N; p.P = pl.P; p.C = pl.C;
    p.kchunk = pl.kchunk; p.splits = pl.splits; p.row_blocks = pl.row_blocks;
    uint8_t *base = reinterpret_cast<uint8_t *>(scratch);
    p.tickets = reinterpret_cast<uint32_t *>(base);
    p.partial = reinterpret_cast<float *>(base + pl.tickets_bytes);
    if (staged_in) {
        p.xin = reinterpret_cast<const uint4 *>(staged_in);
    } else {
        // split x into bf16 terms in the order this layer's weight loads consume them
        __nv_bfloat16 *own = reinterpret_cast<__nv_bfloat16 *>(base + pl.tickets_bytes + pl.partial_bytes);
        spg_gemv_stage_kernel<<<(pl.kpad + 255) / 256, 256, 0, s>>>(x, ldx, N, pl.P, L->in, pl.kpad, L->precision, pl.T, own);
        int rc = spgk_check_launch("spg_gemv_stage_kernel");
        if (rc) return rc;
        p.xin = reinterpret_cast<const uint4 *>(own);
    }
    // The finishing CTAs can stage the next layer's input directly, when that layer will also run here
    // and this layer's output needs no further pass (softmax) first.
    p.xout = nullptr; p.next_prec = 0; p.next_kpad = 0;
    if (next && staged_out && L->act != SPG_ACT_SOFTMAX && next->in == L->out) {
        Plan np = make_plan(next, N);
        if (np.ok) { p.xout = reinterpret_cast<__nv_bfloat16 *>(staged_out); p.next_prec = next->precision; p.next_kpad = np.kpad; }
    }
    switch (L->precision) {
        case SPG_P_I4:   return launch_t<SPG_P_I4>(p, pl, s);
        case SPG_P_I2:   return launch_t<SPG_P_I2>(p, pl, s);
        case SPG_P_I8:   return launch_t<SPG_P_I8>(p, pl, s);
        case SPG_P_BF16: return launch_t<SPG_P_BF16>(p, pl, s);
        case SPG_P_F16:  return launch_t<SPG_P_F16>(p, pl, s);
        default:         return launch_t<SPG_P_F32>(p, pl, s);
    }
}

// 1 if the call above staged (or would stage) `next`'s input: lets the caller know whether to pass it on
int spgk_gemv_chain_stages_next(const spgk_layer *L, const spgk_layer *next, uint32_t N)
{
    if (!L || !next || L->act == SPG_ACT_SOFTMAX || next->in != L->out) return 0;
    return make_plan(L, N).ok && make_plan(next, N).ok ? 1 : 0;
}

int spgk_layer_gemv(const spgk_layer *L, const float *x, uint32_t ldx, float *y, uint32_t ldy, uint32_t N,
                    void *scratch, void *stream)
{
    if (!x) { spgk_set_error("spgk_layer_gemv", "bad argument"); return SPGK_E_ARG; }
    return spgk_layer_gemv_chain(L, nullptr, nullptr, nullptr, x, ldx, y, ldy, N, scratch, stream);
}

}  // extern "C"
