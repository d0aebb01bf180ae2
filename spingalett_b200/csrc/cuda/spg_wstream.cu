// spg_wstream.cu -- weight-streaming dense layer for small and medium batches (1..128 rows) on the
// 5th-generation tensor cores, with the dequantisation done in shared memory.
//
//   y[n][j] = act(bias[j] + w_scale * sum_k q[j][k] * x[n][k])
//
// In this regime the layer is bound by reading the packed weights once from HBM, so the roles of the two
// GEMM operands are swapped with respect to the large-batch kernel: the 128 rows of the UMMA tile are 128
// output neurons (weight rows) and its N dimension holds the batch -- every activation row as two or three
// bf16 terms (x = x1 + x2 [+ x3], one tile column per term), so that all products are exact and the fp32
// accumulation in tensor memory is the only rounding.
//
// Per CTA (persistent, one per SM, items = 128 weight rows x one K range):
//   warp 0      producer: TMA boxes of the stored, still packed matrix (128 rows x 128 bytes, 128-byte
//               swizzle, no multicast) into a raw ring, and [columns x 64] activation tiles into a B ring
//   warps 6-13  converters: unpack a raw box (INT4 / INT2 / INT8 two's complement) to bf16 with mask and
//               magic-number tricks and write it as the K-major, 128-byte-swizzled A operand tile
//               (BF16 files need no conversion: the raw box already is that tile)
//   warp 1      issues tcgen05.mma (kind::f16, M = 128, N = columns, K = 16), accumulator in TMEM
//   warps 2-5   epilogue: tcgen05.ld, sum of the terms, scale, bias, activation; write y (fp32) and the next
//               layer's activation operand (bf16 terms); with K split over several items the partial sums go
//               through global memory and the last item of a row tile (atomic ticket) finishes it.
//
// The K order inside a 16-wide MMA step is free as long as both operands agree, so the unpacking keeps the
// order the mask tricks deliver (e.g. nibbles 0,4,1,5,2,6,3,7 of a word) and the activation operand is
// stored with the same permutation of K.  Every mbarrier wait is bounded.
#include "spg_common.cuh"
#include "spg_tc.cuh"
#include <cstdio>
#include <mutex>

namespace {

using namespace spgtc;

constexpr uint32_t WS_THREADS = 448;        // 14 warps
constexpr uint32_t CONV_WARPS = 8, CONV_WARP0 = 6;
constexpr uint32_t TILE_ROWS = 128;
constexpr uint32_t RAW_BYTES = 128 * TILE_ROWS;          // one raw box
constexpr uint32_t A_TILE = 128 * TILE_ROWS;             // one bf16 operand tile (64 k)
constexpr uint32_t MAX_COLS = 256;

struct WsParams {
    uint32_t in, out; int prec, act; float scale; const float *bias;
    uint32_t N, P, C, NC;                   // rows, terms per row, columns in use, columns of the tile (multiple of 16)
    uint32_t m_tiles, splits, items;
    uint32_t kb_total, kb_per_split, kbr;   // 64-wide k-blocks over K, per item, per raw box
    uint32_t RS, AS, BS, a_slot_bytes, b_slot_bytes;
    uint32_t direct;                        // BF16 weights: the raw box is the A tile
    float *y; uint32_t ldy;
    __nv_bfloat16 *xnext; uint32_t next_ld; int next_prec; uint32_t next_in;
    float *partial; uint32_t *tickets; int32_t *status;
    uint32_t idesc;
};

// Where element e of a group of 16 consecutive k lands inside the group, for activations that meet weights of
// the given stored precision (the order in which the unpacking delivers those weights).
__host__ __device__ inline uint32_t k_position(int prec, uint32_t k)
{
    const uint32_t base = k & ~15u, e = k & 15u;
    if (prec == SPG_P_I4) {                 // per word of 8 nibbles: 0,4,1,5,2,6,3,7
        const uint32_t i = e & 7u;
        return base + (e & 8u) + ((i & 3u) << 1) + (i >> 2);
    }
    if (prec == SPG_P_I2) {                 // per word of 16 crumbs: 0,8,1,9,2,10,3,11 | 4,12,5,13,6,14,7,15
        const uint32_t i = e & 7u, hi = e >> 3;
        return base + ((i >> 2) << 3) + ((i & 3u) << 1) + hi;
    }
    if (prec == SPG_P_I8) {                 // per word of 4 bytes: 0,2,1,3
        const uint32_t i = e & 3u;
        return base + (e & 12u) + ((i & 1u) << 1) + (i >> 1);
    }
    return k;
}

// fp32 rows -> bf16 term columns of the activation operand [NC][ld], K permuted for `prec`; unused columns and
// the K tail are zero.
__global__ void __launch_bounds__(256)
spg_ws_stage_kernel(const float *__restrict__ x, uint32_t ldx, uint32_t N, uint32_t P, uint32_t in, uint32_t ld,
                    uint32_t NC, int prec, __nv_bfloat16 *__restrict__ dst)
{
    const uint32_t k = blockIdx.x * 256 + threadIdx.x;
    if (k >= ld) return;
    const uint32_t pos = k_position(prec, k);
    for (uint32_t c = 0; c < NC; c += P) {
        const uint32_t n = c / P;
        float v = (n < N && k < in) ? x[(uint64_t)n * ldx + k] : 0.0f;
        for (uint32_t q = 0; q < P && c + q < NC; q++) {
            const __nv_bfloat16 h = __float2bfloat16_rn(v);
            dst[(uint64_t)(c + q) * ld + pos] = h;
            v -= __bfloat162float(h);
        }
    }
}

// (bits & mask) | 0x4300 per half = bf16 value 128 + field; subtracting the bias pair leaves the signed integer
__device__ __forceinline__ uint32_t field_pair(uint32_t shifted, uint32_t mask, uint32_t bias_pair)
{
    uint32_t v = (shifted & mask) | 0x43004300u;
    __nv_bfloat162 r = __hsub2(*reinterpret_cast<__nv_bfloat162 *>(&v), *reinterpret_cast<const __nv_bfloat162 *>(&bias_pair));
    return *reinterpret_cast<uint32_t *>(&r);
}
// ((128 + field) - 136) * 16 in one exact bf16 fma: the high nibble of an INT8 weight, already scaled
__device__ __forceinline__ uint32_t high_nibble_pair(uint32_t shifted)
{
    uint32_t v = (shifted & 0x000F000Fu) | 0x43004300u;
    const uint32_t sixteen = 0x41804180u, minus = 0xC508C508u;         // 16.0 and -2176.0 as bf16 pairs
    __nv_bfloat162 r = __hfma2(*reinterpret_cast<__nv_bfloat162 *>(&v), *reinterpret_cast<const __nv_bfloat162 *>(&sixteen),
                               *reinterpret_cast<const __nv_bfloat162 *>(&minus));
    return *reinterpret_cast<uint32_t *>(&r);
}

__device__ __forceinline__ void epi_sync() { asm volatile("bar.sync 2, 128;" ::: "memory"); }      // the four epilogue warps

// One finished output value: scale, bias, activation; fp32 result and, if a next layer follows, its bf16 terms
// in that layer's activation operand (K position permuted for that layer's stored precision).
__device__ __forceinline__ void ws_finish(const WsParams &p, uint32_t n, uint32_t row, float sum)
{
    if (row >= p.out || n >= p.N) return;
    float v = spg_activate(fmaf(sum, p.scale, p.bias[row]), p.act);
    p.y[(uint64_t)n * p.ldy + row] = v;
    if (p.xnext) {
        const uint32_t pos = k_position(p.next_prec, row);
        for (uint32_t q = 0; q < p.P; q++) {
            const __nv_bfloat16 h = __float2bfloat16_rn(v);
            p.xnext[(uint64_t)(n * p.P + q) * p.next_ld + pos] = h;
            v -= __bfloat162float(h);
        }
    }
}

// Epilogue role (warps 2..5): thread = one weight row (TMEM lane) of the item, walking the tile's columns.
__device__ __forceinline__ void ws_epilogue(const WsParams &p, uint32_t tmem_base, uint32_t tfull0, uint32_t tempty0,
                                            volatile int *abort_flag, int *s_last, uint32_t warp, uint32_t lane)
{
    const uint32_t q = warp & 3u, et = (warp - 2u) * 32u + lane;
    const uint32_t out_pad = p.m_tiles * TILE_ROWS;
    uint32_t tcount = 0;
    for (uint32_t item = blockIdx.x; item < p.items; item += gridDim.x, tcount++) {
        const uint32_t mt = item % p.m_tiles, split = item / p.m_tiles;
        const uint32_t acc = tcount & 1u;
        const bool ok = mbar_wait(tfull0 + 8 * acc, (tcount >> 1) & 1u, abort_flag, p.status, 9);
        tc_fence_after();
        const uint32_t row = mt * TILE_ROWS + q * 32u + lane;
        const uint32_t taddr = tmem_base + acc * p.NC + ((q * 32u) << 16);
        float sum = 0.0f;
        for (uint32_t c0 = 0; c0 < p.C; c0 += 16) {
            uint32_t r[16];
            tmem_ld16(taddr + c0, r);
            tmem_ld_wait();
            if (!ok) continue;
            if (p.splits == 1) {
#pragma unroll
                for (uint32_t i = 0; i < 16; i++) {
                    const uint32_t col = c0 + i;
                    if (col < p.C) {
                        sum += __uint_as_float(r[i]);
                        if (col % p.P == p.P - 1) { ws_finish(p, col / p.P, row, sum); sum = 0.0f; }
                    }
                }
            } else {
#pragma unroll
                for (uint32_t i = 0; i < 16; i++) {
                    const uint32_t col = c0 + i;
                    if (col < p.C) __stcg(p.partial + ((uint64_t)split * p.C + col) * out_pad + row, __uint_as_float(r[i]));
                }
            }
        }
        tc_fence_before();
        mbar_arrive(tempty0 + 8 * acc);                    // the accumulator may be overwritten
        if (p.splits > 1) {
            __threadfence();
            epi_sync();
            if (et == 0) *s_last = atomicAdd(&p.tickets[mt], 1u) == p.splits - 1;
            epi_sync();
            if (*s_last) {
                __threadfence();
                for (uint32_t n = 0; n < p.N; n++) {
                    float total = 0.0f;
                    for (uint32_t s = 0; s < p.splits; s++) {
                        float part = 0.0f;
                        for (uint32_t t = p.P; t-- > 0;)      // smallest term first
                            part += __ldcg(p.partial + ((uint64_t)s * p.C + n * p.P + t) * out_pad + row);
                        total += part;
                    }
                    ws_finish(p, n, row, total);
                }
                if (et == 0) p.tickets[mt] = 0;                // ready for the next call
            }
            epi_sync();
        }
        // the K tail of the next layer's operand (k in [out, next_ld)) stays zero
        if (p.xnext && mt == p.m_tiles - 1 && (p.splits == 1 || *s_last))
            for (uint32_t idx = et; idx < (p.next_ld - p.out) * p.C; idx += 128)
                p.xnext[(uint64_t)(idx % p.C) * p.next_ld + k_position(p.next_prec, p.out + idx / p.C)] = __float2bfloat16_rn(0.0f);
    }
}

__global__ void __launch_bounds__(WS_THREADS, 1)
spg_wstream_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const WsParams p)
{
    extern __shared__ uint8_t ws_smem_raw[];
    const uint32_t raw = smem_u32(ws_smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *smem = ws_smem_raw + (base - raw);
    // layout: raw ring | A ring (absent for BF16 weights) | B ring | barriers | flags
    const uint32_t a_off = p.RS * RAW_BYTES;
    const uint32_t b_off = a_off + (p.direct ? 0u : p.AS * p.a_slot_bytes);
    const uint32_t bar_off = b_off + p.BS * p.b_slot_bytes;
    const uint32_t rfull0 = base + bar_off, rempty0 = rfull0 + 8 * p.RS;
    const uint32_t afull0 = rempty0 + 8 * p.RS, aempty0 = afull0 + 8 * p.AS;
    const uint32_t bfull0 = aempty0 + 8 * p.AS, bempty0 = bfull0 + 8 * p.BS;
    const uint32_t tfull0 = bempty0 + 8 * p.BS, tempty0 = tfull0 + 16;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + bar_off + 16 * (p.RS + p.AS + p.BS) + 32);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    int *s_last = const_cast<int *>(abort_flag) + 1;

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t tmem_cols = 2 * p.NC < 32 ? 32 : (2 * p.NC <= 64 ? 64 : (2 * p.NC <= 128 ? 128 : (2 * p.NC <= 256 ? 256 : 512)));

    if (tid == 0) {
        for (uint32_t s = 0; s < p.RS; s++) { mbar_init(rfull0 + 8 * s, 1); mbar_init(rempty0 + 8 * s, p.direct ? 1 : CONV_WARPS); }
        for (uint32_t s = 0; s < p.AS; s++) { mbar_init(afull0 + 8 * s, CONV_WARPS / p.AS); mbar_init(aempty0 + 8 * s, 1); }
        for (uint32_t s = 0; s < p.BS; s++) { mbar_init(bfull0 + 8 * s, 1); mbar_init(bempty0 + 8 * s, 1); }
        for (uint32_t a = 0; a < 2; a++) { mbar_init(tfull0 + 8 * a, 1); mbar_init(tempty0 + 8 * a, 128); }
        *abort_flag = 0;
        mbar_fence_init();
        prefetch_map(&map_w);
        prefetch_map(&map_x);
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), tmem_cols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // item -> (row tile, K split); k-blocks [kb0, kb1) of the item
#define WS_ITEM_RANGE(item)                                                              \
    const uint32_t mt = (item) % p.m_tiles, split = (item) / p.m_tiles;                  \
    const uint32_t kb0 = split * p.kb_per_split;                                         \
    const uint32_t kb1 = min(kb0 + p.kb_per_split, p.kb_total);                          \
    const uint32_t nraw = (kb1 - kb0 + p.kbr - 1) / p.kbr;

    const uint32_t abort_addr = smem_u32(const_cast<int *>(abort_flag));
    if (warp == 0) {
        // ------------------------------ producer ----------------------------------
        // The whole warp walks the loops convergently (ring positions are counted up, never divided out), one elected
        // lane issues the copies.  After an abort the waits end at once; the flag is looked at once per raw box so that
        // no copy is started into shared memory that is about to be given up.
        uint32_t rs = 0, rph = 0, bs = 0, bph = 0;
        for (uint32_t item = blockIdx.x; item < p.items; item += gridDim.x) {
            WS_ITEM_RANGE(item)
            for (uint32_t r = 0; r < nraw; r++) {
                if (*abort_flag) goto ws_role_done;
                mbar_wait_uniform(rempty0 + 8 * rs, rph ^ 1u, abort_addr, p.status, 1);
                if (elect_one()) {
                    mbar_expect_tx(rfull0 + 8 * rs, RAW_BYTES);
                    tma_load_2d(base + rs * RAW_BYTES, &map_w, rfull0 + 8 * rs, (int)((kb0 / p.kbr + r) * 128u), (int)(mt * TILE_ROWS));
                }
                __syncwarp();
                const uint32_t kbs = min(p.kbr, kb1 - kb0 - r * p.kbr);
                for (uint32_t j = 0; j < kbs; j++) {
                    mbar_wait_uniform(bempty0 + 8 * bs, bph ^ 1u, abort_addr, p.status, 2);
                    if (*abort_flag) goto ws_role_done;
                    if (elect_one()) {
                        mbar_expect_tx(bfull0 + 8 * bs, p.b_slot_bytes);
                        tma_load_2d(base + b_off + bs * p.b_slot_bytes, &map_x, bfull0 + 8 * bs, (int)((kb0 + r * p.kbr + j) * 64u), 0);
                    }
                    __syncwarp();
                    if (++bs == p.BS) { bs = 0; bph ^= 1u; }
                }
                if (++rs == p.RS) { rs = 0; rph ^= 1u; }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer --------------------------------
        // Convergent as well: descriptors, ring positions and the accumulator address stay warp-uniform (tcgen05.mma takes
        // them from uniform registers), the waits are single try_waits when the data is already there.
        uint32_t rs = 0, rph = 0, as = 0, aph = 0, bs = 0, bph = 0, tcount = 0;
        const uint32_t terms = p.prec == SPG_P_I8 ? 2u : 1u;           // INT8: low-nibble tile + high-nibble tile
        const uint64_t r_desc0 = smem_desc_sw128(base), a_desc0 = smem_desc_sw128(base + a_off), b_desc0 = smem_desc_sw128(base + b_off);
        const uint32_t a_step = p.a_slot_bytes >> 4, b_step = p.b_slot_bytes >> 4;
        for (uint32_t item = blockIdx.x; item < p.items; item += gridDim.x, tcount++) {
            WS_ITEM_RANGE(item)
            (void)mt;
            const uint32_t acc = tcount & 1u;
            mbar_wait_uniform(tempty0 + 8 * acc, ((tcount >> 1) & 1u) ^ 1u, abort_addr, p.status, 3);
            if (*abort_flag) goto ws_role_done;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + acc * p.NC;
            uint32_t accum = 0;
            for (uint32_t r = 0; r < nraw; r++) {
                const uint32_t kbs = min(p.kbr, kb1 - kb0 - r * p.kbr);
                if (p.direct) mbar_wait_uniform(rfull0 + 8 * rs, rph, abort_addr, p.status, 4);
                for (uint32_t j = 0; j < kbs; j++) {
                    uint64_t da;
                    if (p.direct) {
                        da = r_desc0 + (uint64_t)(rs * (RAW_BYTES >> 4));
                    } else {
                        mbar_wait_uniform(afull0 + 8 * as, aph, abort_addr, p.status, 5);
                        da = a_desc0 + (uint64_t)(as * a_step);
                    }
                    mbar_wait_uniform(bfull0 + 8 * bs, bph, abort_addr, p.status, 6);
                    tc_fence_after();
                    const uint64_t db = b_desc0 + (uint64_t)(bs * b_step);
                    if (elect_one()) {
                        for (uint32_t tm = 0; tm < terms; tm++) {
#pragma unroll
                            for (uint32_t k = 0; k < 4; k++) { umma_f16(d_tmem, da + tm * (A_TILE >> 4) + 2 * k, db + 2 * k, p.idesc, accum); accum = 1; }
                        }
                        umma_commit(bempty0 + 8 * bs);
                        if (!p.direct) umma_commit(aempty0 + 8 * as);
                    }
                    __syncwarp();
                    accum = 1;
                    if (++bs == p.BS) { bs = 0; bph ^= 1u; }
                    if (!p.direct && ++as == p.AS) { as = 0; aph ^= 1u; }
                }
                if (p.direct) {
                    if (elect_one()) umma_commit(rempty0 + 8 * rs);
                    __syncwarp();
                }
                if (++rs == p.RS) { rs = 0; rph ^= 1u; }
                if (*abort_flag) goto ws_role_done;
            }
            if (elect_one()) umma_commit(tfull0 + 8 * acc);
            __syncwarp();
        }
    } else if (warp >= CONV_WARP0) {
        // ------------------------------ converters --------------------------------
        // G groups of 8/G warps, G = slots of the operand ring (4 or 2); group g takes the k-blocks whose running number
        // is g mod G -- always ring slot g, so a group only ever waits for its own previous tile to be consumed -- and G
        // operand tiles are being written at any time: the latency of one (load, unpack, store, proxy fence, arrive) is
        // hidden behind the others.  A thread handles G (row, half k-block) units of its group's k-block: all raw words
        // are loaded first, then unpacked and stored.  Every warp waits for every raw box and arrives on its "empty"
        // barrier once it is through it, whether or not one of its k-blocks was in it.
        if (!p.direct) {
            const uint32_t G = p.AS, wpg = CONV_WARPS / G, TG = 32u * wpg;
            const uint32_t cw = warp - CONV_WARP0, grp = cw / wpg;
            const uint32_t ctg = (cw % wpg) * 32u + lane;              // 0..TG-1 inside the group
            uint32_t rs = 0, rph = 0, as = 0, aph = 0;
            for (uint32_t item = blockIdx.x; item < p.items; item += gridDim.x) {
                WS_ITEM_RANGE(item)
                (void)mt;
                for (uint32_t r = 0; r < nraw; r++) {
                    const bool okr = mbar_wait(rfull0 + 8 * rs, rph, abort_flag, p.status, 7);
                    const uint8_t *rawbox = smem + rs * RAW_BYTES;
                    const uint32_t kbs = min(p.kbr, kb1 - kb0 - r * p.kbr);
                    for (uint32_t j = 0; j < kbs; j++) {
                        if (as == grp) {
                            const bool ok = okr && mbar_wait(aempty0 + 8 * as, aph ^ 1u, abort_flag, p.status, 8);
                            if (ok) {
                                uint8_t *atile = smem + a_off + as * p.a_slot_bytes;
                                if (p.prec == SPG_P_I4) {
                                    // 32 nibbles = one 16-byte piece (piece j*2+h of the raw row) -> chunks h*4 .. h*4+3
                                    uint4 w[4];
#pragma unroll
                                    for (uint32_t u = 0; u < 4; u++) {
                                        if (u >= G) break;
                                        const uint32_t ct = u * TG + ctg, r7 = ct & 7u, h = (ct >> 3) & 1u, row = (ct >> 4) * 8u + r7;
                                        w[u] = *reinterpret_cast<const uint4 *>(rawbox + row * 128u + (((j * 2u + h) ^ r7) << 4));
                                    }
#pragma unroll
                                    for (uint32_t u = 0; u < 4; u++) {
                                        if (u >= G) break;
                                        const uint32_t ct = u * TG + ctg, r7 = ct & 7u, h = (ct >> 3) & 1u, row = (ct >> 4) * 8u + r7;
                                        uint8_t *arow = atile + row * 128u;
                                        const uint32_t ws[4] = { w[u].x, w[u].y, w[u].z, w[u].w };
#pragma unroll
                                        for (uint32_t q = 0; q < 4; q++) {
                                            const uint32_t v = ws[q] ^ 0x88888888u;
                                            uint4 o;
                                            o.x = field_pair(v, 0x000F000Fu, 0x43084308u);
                                            o.y = field_pair(v >> 4, 0x000F000Fu, 0x43084308u);
                                            o.z = field_pair(v >> 8, 0x000F000Fu, 0x43084308u);
                                            o.w = field_pair(v >> 12, 0x000F000Fu, 0x43084308u);
                                            *reinterpret_cast<uint4 *>(arow + (((h * 4u + q) ^ r7) << 4)) = o;
                                        }
                                    }
                                } else if (p.prec == SPG_P_I2) {
                                    // 32 crumbs = 8 bytes (half of piece j) -> chunks h*4 .. h*4+3
                                    uint2 w[4];
#pragma unroll
                                    for (uint32_t u = 0; u < 4; u++) {
                                        if (u >= G) break;
                                        const uint32_t ct = u * TG + ctg, r7 = ct & 7u, h = (ct >> 3) & 1u, row = (ct >> 4) * 8u + r7;
                                        w[u] = *reinterpret_cast<const uint2 *>(rawbox + row * 128u + ((j ^ r7) << 4) + h * 8u);
                                    }
#pragma unroll
                                    for (uint32_t u = 0; u < 4; u++) {
                                        if (u >= G) break;
                                        const uint32_t ct = u * TG + ctg, r7 = ct & 7u, h = (ct >> 3) & 1u, row = (ct >> 4) * 8u + r7;
                                        uint8_t *arow = atile + row * 128u;
                                        const uint32_t ws[2] = { w[u].x, w[u].y };
#pragma unroll
                                        for (uint32_t q = 0; q < 2; q++) {
                                            const uint32_t v = ws[q] ^ 0xAAAAAAAAu;
#pragma unroll
                                            for (uint32_t c2 = 0; c2 < 2; c2++) {
                                                uint4 o;
                                                o.x = field_pair(v >> (8 * c2), 0x00030003u, 0x43024302u);
                                                o.y = field_pair(v >> (8 * c2 + 2), 0x00030003u, 0x43024302u);
                                                o.z = field_pair(v >> (8 * c2 + 4), 0x00030003u, 0x43024302u);
                                                o.w = field_pair(v >> (8 * c2 + 6), 0x00030003u, 0x43024302u);
                                                *reinterpret_cast<uint4 *>(arow + (((h * 4u + q * 2u + c2) ^ r7) << 4)) = o;
                                            }
                                        }
                                    }
                                } else {
                                    // INT8: 32 bytes = pieces j*4 + h*2 + {0,1}; low nibbles -> tile 0, high nibbles * 16 -> tile 1
#pragma unroll
                                    for (uint32_t u = 0; u < 4; u++) {
                                        if (u >= G) break;
                                        const uint32_t ct = u * TG + ctg, r7 = ct & 7u, h = (ct >> 3) & 1u, row = (ct >> 4) * 8u + r7;
                                        const uint8_t *rawrow = rawbox + row * 128u;
                                        uint8_t *arow = atile + row * 128u;
                                        uint4 w2[2];
#pragma unroll
                                        for (uint32_t pc = 0; pc < 2; pc++) w2[pc] = *reinterpret_cast<const uint4 *>(rawrow + (((j * 4u + h * 2u + pc) ^ r7) << 4));
#pragma unroll
                                        for (uint32_t pc = 0; pc < 2; pc++) {
                                            const uint32_t ws[4] = { w2[pc].x, w2[pc].y, w2[pc].z, w2[pc].w };
#pragma unroll
                                            for (uint32_t q = 0; q < 2; q++) {
                                                const uint32_t v0 = ws[2 * q] ^ 0x80808080u, v1 = ws[2 * q + 1] ^ 0x80808080u;
                                                uint4 lo, hi;
                                                lo.x = field_pair(v0, 0x000F000Fu, 0x43004300u); lo.y = field_pair(v0 >> 8, 0x000F000Fu, 0x43004300u);
                                                lo.z = field_pair(v1, 0x000F000Fu, 0x43004300u); lo.w = field_pair(v1 >> 8, 0x000F000Fu, 0x43004300u);
                                                hi.x = high_nibble_pair(v0 >> 4); hi.y = high_nibble_pair(v0 >> 12);
                                                hi.z = high_nibble_pair(v1 >> 4); hi.w = high_nibble_pair(v1 >> 12);
                                                const uint32_t chunk = ((h * 4u + pc * 2u + q) ^ r7) << 4;
                                                *reinterpret_cast<uint4 *>(arow + chunk) = lo;
                                                *reinterpret_cast<uint4 *>(arow + A_TILE + chunk) = hi;
                                            }
                                        }
                                    }
                                }
                            }
                            fence_async_smem();                        // make the tile visible to the tensor core's reads
                            __syncwarp();
                            if (lane == 0) mbar_arrive(afull0 + 8 * as);
                        }
                        if (++as == p.AS) { as = 0; aph ^= 1u; }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(rempty0 + 8 * rs);
                    if (++rs == p.RS) { rs = 0; rph ^= 1u; }
                }
            }
        }
    } else {
        ws_epilogue(p, tmem_base, tfull0, tempty0, abort_flag, s_last, warp, lane);
    }
#undef WS_ITEM_RANGE
ws_role_done:
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        // a wait gave up: give copies that may still be in flight time to land before the shared memory goes away
        if (tid == 0) for (int i = 0; i < 256; i++) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 1) { tc_fence_after(); tmem_free(tmem_base, tmem_cols); }
}

struct WsPlan {
    uint32_t P, C, NC, kbr, kb_total, kb_per_split, m_tiles, splits, items, RS, AS, BS, a_slot, b_slot, ld, direct;
    size_t tickets_bytes, partial_bytes, operand_bytes, smem;
    bool ok;
};

constexpr size_t WS_HEAD = 256;             // status word at the start of scratch

WsPlan ws_plan(const spgk_layer *L, uint32_t N)
{
    WsPlan pl{};
    pl.ok = false;
    if (!L || N == 0 || L->in == 0 || L->out == 0) return pl;
    const int prec = L->precision;
    if (prec != SPG_P_I4 && prec != SPG_P_I2 && prec != SPG_P_I8 && prec != SPG_P_BF16) return pl;
    const uint32_t bits = spg_bits_per_elem(prec);
    const uint64_t row_bytes = (uint64_t)L->in * bits / 8;
    if ((L->in * bits) % 128 || ((uintptr_t)L->w & 15u)) return pl;      // TMA: 16-byte aligned packed rows
    pl.P = N == 1 ? 3 : 2;
    pl.C = N * pl.P;
    if (pl.C > MAX_COLS) return pl;
    pl.NC = (pl.C + 15u) & ~15u;
    pl.kbr = 16u / bits;
    pl.direct = prec == SPG_P_BF16;
    pl.kb_total = (L->in + 63u) / 64u;
    pl.ld = pl.kb_total * 64u;
    pl.m_tiles = (L->out + TILE_ROWS - 1) / TILE_ROWS;
    // K splits: enough items to balance 148 persistent CTAs, but partial sums must stay a small fraction of the weight bytes
    uint32_t want = (148u * 4 + pl.m_tiles - 1) / pl.m_tiles;
    const uint32_t cap = (uint32_t)(row_bytes / (80ull * pl.C));
    if (want > cap) want = cap;
    if (want < 1) want = 1;
    uint32_t per = (pl.kb_total + want - 1) / want;
    per = (per + pl.kbr - 1) / pl.kbr * pl.kbr;
    pl.kb_per_split = per;
    pl.splits = (pl.kb_total + per - 1) / per;
    pl.items = pl.m_tiles * pl.splits;
    pl.a_slot = prec == SPG_P_I8 ? 2 * A_TILE : A_TILE;
    pl.b_slot = pl.NC * 128u;
    // ring depths: as deep as shared memory allows, never less than two slots each
    // (the operand ring has 4 or 2 slots: one per converter group)
    bool fits = false;
    size_t a_bytes = 0;
    static const uint32_t depths[5][2] = { {4, 4}, {4, 3}, {4, 2}, {2, 3}, {2, 2} };
    for (int d = 0; d < 5 && !fits; d++) {
        pl.AS = pl.direct ? 1 : depths[d][0];
        pl.BS = depths[d][1];
        a_bytes = pl.direct ? 0 : (size_t)pl.AS * pl.a_slot;
        const size_t fixed = 1024 + a_bytes + (size_t)pl.BS * pl.b_slot + 1024;
        if (fixed + 2 * RAW_BYTES <= 225u * 1024) {
            pl.RS = (uint32_t)((225u * 1024 - fixed) / RAW_BYTES);
            if (pl.RS > 8) pl.RS = 8;
            fits = true;
        }
    }
    if (!fits) return pl;
    pl.smem = 1024 + (size_t)pl.RS * RAW_BYTES + a_bytes + (size_t)pl.BS * pl.b_slot + 16 * (pl.RS + pl.AS + pl.BS) + 32 + 64;
    // fixed size: layers of different shapes share one scratch buffer and the counters must stay zero between calls
    pl.tickets_bytes = 16384;
    if (pl.m_tiles > 4096) return pl;
    pl.partial_bytes = pl.splits > 1 ? (size_t)pl.splits * pl.C * pl.m_tiles * TILE_ROWS * 4 : 0;
    pl.partial_bytes = (pl.partial_bytes + 255) & ~(size_t)255;
    pl.operand_bytes = ((size_t)pl.NC * pl.ld * 2 + 255) & ~(size_t)255;
    pl.ok = true;
    return pl;
}

typedef CUresult (*WsEncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                               const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// 2-D tiled map with 128-byte swizzle; small cache keyed by everything that defines the map.
int ws_map(const void *ptr, CUtensorMapDataType dt, uint32_t esize, uint64_t d0, uint64_t d1, uint64_t pitch_bytes,
           uint32_t b0, uint32_t b1, CUtensorMap *out)
{
    struct Entry { const void *ptr; uint64_t d0, d1, pitch; uint32_t b0, b1; int dt; CUtensorMap map; };
    static Entry cache[64];
    static int used = 0, victim = 0;
    static std::mutex mu;
    static WsEncodeFn fn = nullptr;
    std::lock_guard<std::mutex> lock(mu);
    for (int i = 0; i < used; i++) {
        const Entry &e = cache[i];
        if (e.ptr == ptr && e.d0 == d0 && e.d1 == d1 && e.pitch == pitch_bytes && e.b0 == b0 && e.b1 == b1 && e.dt == (int)dt) { *out = e.map; return SPGK_OK; }
    }
    if (!fn) {
        void *f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) {
            spgk_set_error("cuTensorMapEncodeTiled", "driver entry point not available");
            return SPGK_E_CUDA;
        }
        fn = reinterpret_cast<WsEncodeFn>(f);
    }
    (void)esize;
    cuuint64_t dims[2] = { d0, d1 };
    cuuint64_t strides[1] = { pitch_bytes };
    cuuint32_t box[2] = { b0, b1 };
    cuuint32_t estr[2] = { 1, 1 };
    CUtensorMap m;
    CUresult r = fn(&m, dt, 2, const_cast<void *>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        char msg[64];
        snprintf(msg, sizeof msg, "CUresult %d", (int)r);
        spgk_set_error("cuTensorMapEncodeTiled (weight stream)", msg);
        return SPGK_E_CUDA;
    }
    Entry &e = cache[used < 64 ? used++ : (victim++ % 64)];
    e.ptr = ptr; e.d0 = d0; e.d1 = d1; e.pitch = pitch_bytes; e.b0 = b0; e.b1 = b1; e.dt = (int)dt; e.map = m;
    *out = m;
    return SPGK_OK;
}

}  // namespace

extern "C" {

size_t spgk_wstream_scratch_bytes(const spgk_layer *L, uint32_t N)
{
    WsPlan pl = ws_plan(L, N);
    return pl.ok ? WS_HEAD + pl.tickets_bytes + pl.partial_bytes + pl.operand_bytes : 0;
}

size_t spgk_wstream_operand_bytes(uint32_t width, uint32_t N)
{
    const uint32_t C = N * (N == 1 ? 3u : 2u);
    if (N == 0 || C > MAX_COLS) return 0;
    return ((size_t)((C + 15u) & ~15u) * ((width + 63u) & ~63u) * 2 + 255) & ~(size_t)255;
}

int spgk_wstream_stages_next(const spgk_layer *L, const spgk_layer *next, uint32_t N)
{
    if (!L || !next || L->act == SPG_ACT_SOFTMAX || next->in != L->out) return 0;
    return ws_plan(L, N).ok && ws_plan(next, N).ok ? 1 : 0;
}

int spgk_layer_wstream(const spgk_layer *L, const spgk_layer *next, const void *operand_in, void *operand_out,
                       const float *x, uint32_t ldx, float *y, uint32_t ldy, uint32_t N, void *scratch, void *stream)
{
    if (!L || !y || !L->w || !L->bias || (!x && !operand_in)) { spgk_set_error("spgk_layer_wstream", "bad argument"); return SPGK_E_ARG; }
    WsPlan pl = ws_plan(L, N);
    if (!pl.ok) return SPGK_E_UNSUPPORTED;
    if (!scratch) { spgk_set_error("spgk_layer_wstream", "scratch is NULL"); return SPGK_E_ARG; }
    SpgDeviceProps dp;
    int rc;
    if ((rc = spg_device_props(&dp))) return rc;
    if (dp.cc != 100) return SPGK_E_UNSUPPORTED;                        // tcgen05 / TMEM exist on sm_100 only
    const int sms = dp.sm_count;
    {
        // the opt-in for large dynamic shared memory is a per-device function attribute
        static SpgOncePerDevice once;
        int dev = 0;
        SPGK_CUDA(cudaGetDevice(&dev));
        rc = once.run(dev, [&]() -> int {
            SPGK_CUDA(cudaFuncSetAttribute(spg_wstream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
            return SPGK_OK;
        });
        if (rc) return rc;
    }
    cudaStream_t s = (cudaStream_t)stream;
    uint8_t *base = reinterpret_cast<uint8_t *>(scratch);
    const void *xop = operand_in;
    if (!xop) {
        __nv_bfloat16 *own = reinterpret_cast<__nv_bfloat16 *>(base + WS_HEAD + pl.tickets_bytes + pl.partial_bytes);
        spg_ws_stage_kernel<<<(pl.ld + 255) / 256, 256, 0, s>>>(x, ldx, N, pl.P, L->in, pl.ld, pl.NC, L->precision, own);
        if ((rc = spgk_check_launch("spg_ws_stage_kernel"))) return rc;
        xop = own;
    }
    CUtensorMap map_w, map_x;
    const uint64_t row_bytes = (uint64_t)L->in * spg_bits_per_elem(L->precision) / 8;
    if ((rc = ws_map(L->w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, row_bytes, L->out, row_bytes, 128, TILE_ROWS, &map_w))) return rc;
    if ((rc = ws_map(xop, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, pl.ld, pl.NC, (uint64_t)pl.ld * 2, 64, pl.NC, &map_x))) return rc;

    WsParams p{};
    p.in = L->in; p.out = L->out; p.prec = L->precision;
    p.act = L->act == SPG_ACT_SOFTMAX ? SPG_ACT_NONE : L->act;
    p.scale = L->w_scale; p.bias = L->bias;
    p.N = N; p.P = pl.P; p.C = pl.C; p.NC = pl.NC;
    p.m_tiles = pl.m_tiles; p.splits = pl.splits; p.items = pl.items;
    p.kb_total = pl.kb_total; p.kb_per_split = pl.kb_per_split; p.kbr = pl.kbr;
    p.RS = pl.RS; p.AS = pl.AS; p.BS = pl.BS; p.a_slot_bytes = pl.a_slot; p.b_slot_bytes = pl.b_slot; p.direct = pl.direct;
    p.y = y; p.ldy = ldy;
    p.status = reinterpret_cast<int32_t *>(base);
    p.tickets = reinterpret_cast<uint32_t *>(base + WS_HEAD);
    p.partial = reinterpret_cast<float *>(base + WS_HEAD + pl.tickets_bytes);
    p.idesc = idesc_f16(1, 1, pl.NC);
    p.xnext = nullptr;
    if (next && operand_out && L->act != SPG_ACT_SOFTMAX && next->in == L->out) {
        WsPlan np = ws_plan(next, N);
        if (np.ok) { p.xnext = reinterpret_cast<__nv_bfloat16 *>(operand_out); p.next_ld = np.ld; p.next_prec = next->precision; p.next_in = next->in; }
    }
    const uint32_t grid = pl.items < (uint32_t)sms ? pl.items : (uint32_t)sms;
    spg_wstream_kernel<<<grid, WS_THREADS, pl.smem, s>>>(map_w, map_x, p);
    return spgk_check_launch("spg_wstream_kernel");
}

int spgk_wstream_status(void *scratch, void *stream)
{
    int32_t h = 0;
    SPGK_CUDA(cudaMemcpyAsync(&h, scratch, sizeof h, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    SPGK_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    if (h != 0) {
        char msg[96];
        snprintf(msg, sizeof msg, "bounded wait %d gave up inside the weight-streaming kernel", (int)h);
        spgk_set_error("spg_wstream_kernel", msg);
        SPGK_CUDA(cudaMemsetAsync(scratch, 0, sizeof h, (cudaStream_t)stream));
        return SPGK_E_TIMEOUT;
    }
    return SPGK_OK;
}

}  // extern "C"
