// spg_gemm_tc.cu -- large-batch dense layer on the 5th-generation tensor cores.
//
//   C[M][N] = act(bias + scale * sum over passes  A_pa[M][K] * W_pw[N][K]^T)
//
// Both operands are 16-bit and K-major (activations row-major [rows][K], weights
// row-major [out][in] exactly as Spingalett lays them out), so a tile of either
// is a stack of 128-byte rows: TMA (cp.async.bulk.tensor, 128-byte swizzle, no
// multicast) brings [128 x 64] A tiles and [BN x 64] W tiles into shared memory,
// one elected thread issues tcgen05.mma (kind::f16, M=128, N=BN, K=16) with the
// fp32 accumulator in tensor memory, and eight epilogue warps read it back with
// tcgen05.ld, apply scale, bias, activation (optionally the row softmax) and
// write either the 16-bit operand planes of the next layer or the final fp32
// output.  The kernel is persistent (one CTA per SM walks a tile list) and the
// accumulator is double-buffered in TMEM so the epilogue of tile i overlaps the
// main loop of tile i+1.
//
// Every wait on an mbarrier is bounded: when the bound is hit the CTA records a
// code in `status`, raises a shared abort flag that all roles poll, drains, frees
// its tensor memory and returns; the launcher turns that into SPGK_E_TIMEOUT.
#include "spg_common.cuh"
#include "spg_tc.cuh"
#include <cuda.h>
#include <cstdio>
#include <mutex>
#include <type_traits>

namespace {

constexpr uint32_t BM = 128;            // rows of C per tile (UMMA M)
constexpr uint32_t BK = 64;             // K elements per stage: 64 * 2 B = one 128-byte swizzle row
constexpr uint32_t UMMA_K = 16;
constexpr uint32_t A_TILE_BYTES = BM * BK * 2;
constexpr uint32_t EPI_WARPS = 8;       // two warps per TMEM lane quadrant, each taking half of the tile's columns
constexpr uint32_t NUM_THREADS = 64 + 32 * EPI_WARPS;   // warp 0 TMA, warp 1 MMA + TMEM owner, warps 2.. epilogue
constexpr uint32_t WAIT_LIMIT = 1u << 16;    // attempts; each may suspend the warp for up to SPG_WAIT_HINT_NS
constexpr uint32_t MAX_PASSES = 4;
constexpr uint32_t SOFTMAX_FUSE_MAX = 256;       // a row that fits one tile
constexpr uint32_t SOFTMAX_WIDE_MAX = 1024;      // a row over up to four column tiles of a CTA that owns the row tile
constexpr uint32_t STG_PITCH = 80;                        // bytes per staged row: 32 columns x 2 bytes + 16 (bank spread for 16-byte accesses)
constexpr uint32_t PATCH_BYTES = 32 * 128;                 // TMA-store patch: 32 rows x 64 columns, 128-byte swizzled rows
constexpr uint32_t STG_BYTES = EPI_WARPS * PATCH_BYTES;    // per epilogue warp: one patch (the register-store path uses 32 x STG_PITCH of it)

struct GemmParams {
    uint32_t M, N, K;
    uint32_t BN, stages, kblocks;
    uint32_t npass;
    uint32_t pass_a[MAX_PASSES], pass_w[MAX_PASSES];
    uint32_t m_tiles, n_tiles, group_m;
    uint32_t idesc;
    float scale;
    const float *bias;
    int act;
    int softmax;
    void *out16; uint32_t ldo16; uint64_t o_plane; int out_parts; int type16;
    float *out32; uint32_t ldo32;
    int32_t *status;
    // optional narrow last layer ("head") finished inside this layer's epilogue: out = head_act(head_bias + head_scale * Wh * act(...))
    uint32_t own_rows;            // a CTA owns whole row tiles and walks their column tiles in order (fused head, wide fused softmax)
    const float *head_w;          // [round_up(N, 32)][HP] fp32, unscaled, rows beyond N zero (staged into shared memory)
    const float *head_bias; float head_scale; uint32_t head_out, head_hp; int head_act, head_softmax;
    uint32_t stg_bytes;           // bytes of the epilogue's shared-memory region (patches, or head weights + exchange)
    float margin_theta; uint32_t *margin_idx, *margin_count;
    const uint32_t *out_rows;     // optional scatter of the fp32 output rows   // fused-softmax rows with top-two logit gap < theta are appended here (optional)
    int tma_store;                // 16-bit output leaves through TMA stores (one plane, tiles at least 128 wide)
    const uint32_t *m_limit;      // optional device-resident row count: the kernel works on min(M, *m_limit) rows
};

struct RowLimit { uint32_t m_tiles, group_m; };   // tile counts for the rows actually present (<= the launch's capacity)

// ---- PTX wrappers: the shared ones of spg_tc.cuh, plus what only this kernel uses -----------------
using spgtc::smem_u32; using spgtc::mbar_init; using spgtc::mbar_arrive; using spgtc::tc_fence_before; using spgtc::tc_fence_after;
using spgtc::umma_f16; using spgtc::umma_commit; using spgtc::tmem_ld16; using spgtc::tmem_ld_wait; using spgtc::fence_async_smem;
using spgtc::mbar_wait_uniform; using spgtc::elect_one;

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) { spgtc::mbar_expect_tx(bar, bytes); }
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) { return spgtc::smem_desc_sw128(saddr); }
// Bounded wait of the epilogue warps.  Returns false when the abort flag is up or the bound was hit
// (in which case it raises the flag and records `code`).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int32_t *status, int code)
{
    return spgtc::mbar_wait(bar, parity, abort_flag, status, code, WAIT_LIMIT);
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1, int c2)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}

__device__ __forceinline__ void tile_coords(const GemmParams &p, const RowLimit &rl, uint32_t t, uint32_t &m_tile, uint32_t &n_tile)
{
    // Tiles are walked in bands of group_m row-tiles, row-tile fastest inside a band,
    // so CTAs running at the same time share W tiles and a small set of A tiles in L2.
    const uint32_t band = rl.group_m * p.n_tiles;
    const uint32_t g = t / band, r = t % band;
    const uint32_t rows_here = min(rl.group_m, rl.m_tiles - g * rl.group_m);
    m_tile = g * rl.group_m + r % rows_here;
    n_tile = r / rows_here;
}


// The tiles of this CTA, in order.  Normally tile blockIdx.x + i * gridDim.x of the banded walk; with a fused head
// a CTA owns whole row tiles (all their column tiles in a row), because the head sums over every column of a row.
__device__ __forceinline__ uint32_t my_tile_count(const GemmParams &p, const RowLimit &rl)
{
    if (p.own_rows) {
        const uint32_t rt = rl.m_tiles > blockIdx.x ? (rl.m_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
        return rt * p.n_tiles;
    }
    const uint32_t total = rl.m_tiles * p.n_tiles;
    return total > blockIdx.x ? (total - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
}
__device__ __forceinline__ void my_tile(const GemmParams &p, const RowLimit &rl, uint32_t i, uint32_t &m_tile, uint32_t &n_tile)
{
    if (p.own_rows) { m_tile = blockIdx.x + (i / p.n_tiles) * gridDim.x; n_tile = i % p.n_tiles; }
    else tile_coords(p, rl, blockIdx.x + i * gridDim.x, m_tile, n_tile);
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

// 16 accumulator columns of one row -> scale, bias, activation.  `full` says all 16 columns exist.
template <int ACT>
__device__ __forceinline__ void finish16(const GemmParams &p, const uint32_t (&r)[16], uint32_t col0, bool full, float (&v)[16])
{
    if (full) {
#pragma unroll
        for (int i = 0; i < 16; i += 4) {
            const float4 b = __ldg(reinterpret_cast<const float4 *>(p.bias + col0 + i));   // same address in every lane
            v[i + 0] = spg_activate(fmaf(__uint_as_float(r[i + 0]), p.scale, b.x), ACT);
            v[i + 1] = spg_activate(fmaf(__uint_as_float(r[i + 1]), p.scale, b.y), ACT);
            v[i + 2] = spg_activate(fmaf(__uint_as_float(r[i + 2]), p.scale, b.z), ACT);
            v[i + 3] = spg_activate(fmaf(__uint_as_float(r[i + 3]), p.scale, b.w), ACT);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 16; i++) {
            const float b = col0 + i < p.N ? p.bias[col0 + i] : 0.0f;
            v[i] = spg_activate(fmaf(__uint_as_float(r[i]), p.scale, b), ACT);
        }
    }
}

__device__ __forceinline__ void write32(const GemmParams &p, uint32_t row, uint32_t col0, const float (&v)[16])
{
    float *o = p.out32 + (uint64_t)(p.out_rows ? p.out_rows[row] : row) * p.ldo32 + col0;
    if ((p.ldo32 & 3u) == 0 && col0 + 16 <= p.N) {
#pragma unroll
        for (int i = 0; i < 16; i += 4)
            *reinterpret_cast<float4 *>(o + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
    } else {
#pragma unroll
        for (int i = 0; i < 16; i++) if (col0 + i < p.N) o[i] = v[i];
    }
}

__device__ __forceinline__ void tma_store_3d(const CUtensorMap *map, uint32_t src, int c0, int c1, int c2)
{
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
                 ::"l"(map), "r"(src), "r"(c0), "r"(c1), "r"(c2) : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// 16-bit output of a 32-row x 32-column patch.  Each thread owns one row of the accumulator, so writing
// straight from registers would send every 16-byte store of a warp to a different row of C (32 cache lines
// per instruction -- measured: a third of the kernel's time).  The patch goes through shared memory instead:
// written row-wise by its owners, read back so that a store instruction covers 8 rows x 64 contiguous bytes.
template <typename T16>
__device__ __forceinline__ void store_patch(const GemmParams &p, uint32_t rows, uint8_t *stg, uint32_t lane, uint32_t row0, uint32_t col0,
                                            const float (&v0)[16], const float (&v1)[16], bool second)
{
    const uint32_t pieces = second ? 4u : 2u;
    for (int part = 0; part < p.out_parts; part++) {
        uint4 q[4];
#pragma unroll
        for (int g = 0; g < 4; g++) {
            const float *v = g < 2 ? v0 + 8 * g : v1 + 8 * (g - 2);
            float w[8];
#pragma unroll
            for (int i = 0; i < 8; i++) w[i] = part == 0 ? v[i] : v[i] - round16<T16>(v[i]);
            q[g].x = pack2<T16>(w[0], w[1]); q[g].y = pack2<T16>(w[2], w[3]);
            q[g].z = pack2<T16>(w[4], w[5]); q[g].w = pack2<T16>(w[6], w[7]);
        }
#pragma unroll
        for (int g = 0; g < 4; g++) if ((uint32_t)g < pieces) *reinterpret_cast<uint4 *>(stg + lane * STG_PITCH + g * 16) = q[g];
        __syncwarp();
        T16 *plane = reinterpret_cast<T16 *>(p.out16) + (uint64_t)part * p.o_plane;
#pragma unroll
        for (int pass = 0; pass < 4; pass++) {
            const uint32_t rr = pass * 8 + (lane >> 2), piece = lane & 3u;
            const uint32_t row = row0 + rr, col = col0 + piece * 8;
            if (piece < pieces && row < rows && col < p.ldo16)
                *reinterpret_cast<uint4 *>(plane + (uint64_t)row * p.ldo16 + col) = *reinterpret_cast<const uint4 *>(stg + rr * STG_PITCH + piece * 16);
        }
        __syncwarp();
    }
}

// Epilogue role.  Warp w reads TMEM lanes 32*(w%4).. (its quadrant) and, of the tile's BN columns,
// the half selected by (w-2)/4; each thread therefore owns one row of C and walks its columns in
// chunks of 32 (two tcgen05.ld in flight per wait).
template <int ACT, int HP>
__device__ __forceinline__ void epilogue_loop(const GemmParams &p, const RowLimit &rl, uint32_t rows, uint32_t tmem_base, uint32_t tfull0, uint32_t tempty0,
                                              volatile int *abort_flag, uint32_t warp, uint32_t lane, uint8_t *stage,
                                              const CUtensorMap *map_o, uint32_t hx0)
{
    uint8_t *stg = stage + (warp - 2u) * PATCH_BYTES;          // 1024-byte aligned: a swizzle atom is 8 rows x 128 bytes
    const uint32_t stg_addr = smem_u32(stg);
    const uint32_t q = warp & 3u, half = (warp - 2u) >> 2;
    const uint32_t ntile = my_tile_count(p, rl);
    const uint32_t span = p.BN >= 32 ? p.BN / 2 : p.BN;            // columns per warp
    const uint32_t c_begin = p.BN >= 32 ? half * span : 0;
    const bool idle = p.BN < 32 && half == 1;                      // a 16-wide tile has work for one warp per quadrant
    const bool vec_bias = (reinterpret_cast<uintptr_t>(p.bias) & 15u) == 0;
    float hacc[HP > 0 ? HP : 1];
    const float *headw = reinterpret_cast<const float *>(stage);               // head mode: the staged head weights
    float *xch = reinterpret_cast<float *>(stage + p.stg_bytes - 4 * 2 * 32 * 16 * 4) ;   // head mode: [parity][quadrant][lane][16] exchange
    for (uint32_t tcount = 0; tcount < ntile; tcount++) {
        uint32_t mt, nt;
        my_tile(p, rl, tcount, mt, nt);
        const uint32_t acc = tcount & 1u, acc_ph = (tcount >> 1) & 1u;
        if (!mbar_wait(tfull0 + 8 * acc, acc_ph, abort_flag, p.status, 4)) break;
        tc_fence_after();
        const uint32_t row = mt * BM + q * 32u + lane;
        const uint32_t n0 = nt * p.BN;
        if (HP > 0 && nt == 0) {
#pragma unroll
            for (int j = 0; j < (HP > 0 ? HP : 1); j++) hacc[j] = 0.0f;
        }
        const uint32_t taddr = tmem_base + acc * p.BN + ((q * 32u) << 16);
        const bool row_ok = row < rows;
        if (!idle) {
            for (uint32_t c0 = c_begin; c0 < c_begin + span; c0 += 32) {
                if (n0 + c0 >= p.N) break;                         // only zero-filled W rows beyond N
                const bool second = c0 + 16 < c_begin + span && n0 + c0 + 16 < p.N;
                uint32_t r0[16], r1[16];
                tmem_ld16(taddr + c0, r0);
                if (second) tmem_ld16(taddr + c0 + 16, r1);
                tmem_ld_wait();
                float v[16], v2[16];
                finish16<ACT>(p, r0, n0 + c0, vec_bias && n0 + c0 + 16 <= p.N, v);
                if (second) finish16<ACT>(p, r1, n0 + c0 + 16, vec_bias && n0 + c0 + 32 <= p.N, v2);
                if (HP > 0) {
                    // the head's partial dot products over these columns (its weights beyond N are zero in shared memory)
                    const float *hw = headw + (size_t)(n0 + c0) * HP;
#pragma unroll
                    for (int i = 0; i < 16; i++) {
#pragma unroll
                        for (int j = 0; j < HP; j += 4) {
                            const float4 w4 = *reinterpret_cast<const float4 *>(hw + i * HP + j);
                            hacc[j] = fmaf(v[i], w4.x, hacc[j]); hacc[j + 1] = fmaf(v[i], w4.y, hacc[j + 1]);
                            hacc[j + 2] = fmaf(v[i], w4.z, hacc[j + 2]); hacc[j + 3] = fmaf(v[i], w4.w, hacc[j + 3]);
                        }
                    }
                    if (second) {
#pragma unroll
                        for (int i = 0; i < 16; i++) {
#pragma unroll
                            for (int j = 0; j < HP; j += 4) {
                                const float4 w4 = *reinterpret_cast<const float4 *>(hw + (16 + i) * HP + j);
                                hacc[j] = fmaf(v2[i], w4.x, hacc[j]); hacc[j + 1] = fmaf(v2[i], w4.y, hacc[j + 1]);
                                hacc[j + 2] = fmaf(v2[i], w4.z, hacc[j + 2]); hacc[j + 3] = fmaf(v2[i], w4.w, hacc[j + 3]);
                            }
                        }
                    }
                } else if (p.tma_store) {
                    // Two 32-column chunks fill one 64-column patch: 128-byte rows in the swizzled order the tensor
                    // map expects, then one bulk store moves the patch (rows and columns outside C are clipped).
                    const uint32_t h32 = ((c0 - c_begin) >> 5) & 1u;
                    if (h32 == 0) { if (lane == 0) tma_store_wait_read(); __syncwarp(); }     // the store before has read the patch
                    if (!second) {
#pragma unroll
                        for (int i = 0; i < 16; i++) v2[i] = 0.0f;
                    }
#pragma unroll
                    for (int g = 0; g < 4; g++) {
                        const float *w = g < 2 ? v + 8 * g : v2 + 8 * (g - 2);
                        uint4 qv;
                        if (p.type16 == SPGK_T_F16) {
                            qv.x = pack2<__half>(w[0], w[1]); qv.y = pack2<__half>(w[2], w[3]);
                            qv.z = pack2<__half>(w[4], w[5]); qv.w = pack2<__half>(w[6], w[7]);
                        } else {
                            qv.x = pack2<__nv_bfloat16>(w[0], w[1]); qv.y = pack2<__nv_bfloat16>(w[2], w[3]);
                            qv.z = pack2<__nv_bfloat16>(w[4], w[5]); qv.w = pack2<__nv_bfloat16>(w[6], w[7]);
                        }
                        const uint32_t chunk = (h32 * 4u + g) ^ (lane & 7u);
                        *reinterpret_cast<uint4 *>(stg + lane * 128u + chunk * 16u) = qv;
                    }
                    const bool patch_done = h32 == 1 || c0 + 32 >= c_begin + span || n0 + c0 + 32 >= p.N;
                    if (patch_done) {
                        fence_async_smem();
                        __syncwarp();
                        if (lane == 0) tma_store_3d(map_o, stg_addr, (int)(n0 + c0 - 32u * h32), (int)(mt * BM + q * 32u), 0);
                    }
                } else if (p.out16) {
                    if (p.type16 == SPGK_T_F16) store_patch<__half>(p, rows, stg, lane, mt * BM + q * 32u, n0 + c0, v, v2, second);
                    else store_patch<__nv_bfloat16>(p, rows, stg, lane, mt * BM + q * 32u, n0 + c0, v, v2, second);
                }
                if (HP == 0 && p.out32 && row_ok) {
                    write32(p, row, n0 + c0, v);
                    if (second) write32(p, row, n0 + c0 + 16, v2);
                }
            }
        }
        tc_fence_before();
        mbar_arrive(tempty0 + 8 * acc);                            // every epilogue thread hands the accumulator back
        if (HP > 0 && nt == p.n_tiles - 1) {
            // The row is complete: the warp of the upper column half hands its sums to the warp of the lower half
            // (same rows), which adds bias, applies the head's activation or softmax and writes the outputs.
            float *slot = xch + ((((tcount / p.n_tiles) & 1u) * 4 + q) * 32 + lane) * 16;
            if (half == 1) {
#pragma unroll
                for (int j = 0; j < HP; j += 4) *reinterpret_cast<float4 *>(slot + j) = make_float4(hacc[j], hacc[j + 1], hacc[j + 2], hacc[j + 3]);
            }
            const uint32_t rt = tcount / p.n_tiles;                  // this CTA's row-tile counter: exchange phase and slot parity
            if (half == 1) mbar_arrive(hx0 + 8 * q);
            else if (!mbar_wait(hx0 + 8 * q, rt & 1u, abort_flag, p.status, 5)) break;
            if (half == 0) {
                float z[HP > 0 ? HP : 1];
#pragma unroll
                for (int j = 0; j < HP; j++)
                    z[j] = (uint32_t)j < p.head_out ? fmaf(hacc[j] + slot[j], p.head_scale, p.head_bias[j]) : -FLT_MAX;
                if (p.head_softmax) {
                    float mx = -FLT_MAX, second = -FLT_MAX, sum = 0.0f;
#pragma unroll
                    for (int j = 0; j < HP; j++) if ((uint32_t)j < p.head_out) { if (z[j] > mx) { second = mx; mx = z[j]; } else if (z[j] > second) second = z[j]; }
#pragma unroll
                    for (int j = 0; j < HP; j++) if ((uint32_t)j < p.head_out) { z[j] = expf(z[j] - mx); sum += z[j]; }
                    const float inv = sum > 0.0f ? 1.0f / sum : 1.0f;
#pragma unroll
                    for (int j = 0; j < HP; j++) z[j] *= inv;
                    if (p.margin_idx && row < rows && p.head_out >= 2 && (!(mx - second >= p.margin_theta) || !(sum < FLT_MAX))) p.margin_idx[atomicAdd(p.margin_count, 1u)] = row;
                } else {
#pragma unroll
                    for (int j = 0; j < HP; j++) z[j] = spg_activate(z[j], p.head_act);
                }
                if (row < rows) {
                    const uint64_t orow = p.out_rows ? p.out_rows[row] : row;
#pragma unroll
                    for (int j = 0; j < HP; j++) if ((uint32_t)j < p.head_out) p.out32[orow * p.ldo32 + j] = z[j];
                }
            }
        }
    }
    if (p.tma_store && lane == 0) tma_store_wait_all();            // shared memory must outlive the last bulk store
}

// Fused row softmax (reference Activation.c:5-21): the whole row (N <= BN) sits in one TMEM lane, so
// one thread per row sweeps it three times: running max from -FLT_MAX, sum of expf(v - max), then
// expf(v - max) / sum written out (the division happens only when the sum is positive).
__device__ __forceinline__ void epilogue_softmax(const GemmParams &p, const RowLimit &rl, uint32_t rows, uint32_t tmem_base, uint32_t tfull0, uint32_t tempty0,
                                                 volatile int *abort_flag, uint32_t warp, uint32_t lane)
{
    const uint32_t q = warp & 3u, half = (warp - 2u) >> 2;
    const uint32_t ntile = my_tile_count(p, rl);
    for (uint32_t tcount = 0; tcount < ntile; tcount++) {
        uint32_t mt, nt;
        my_tile(p, rl, tcount, mt, nt);
        const uint32_t acc = tcount & 1u, acc_ph = (tcount >> 1) & 1u;
        if (!mbar_wait(tfull0 + 8 * acc, acc_ph, abort_flag, p.status, 4)) break;
        tc_fence_after();
        if (half == 0) {
            const uint32_t row = mt * BM + q * 32u + lane;
            const uint32_t taddr = tmem_base + acc * p.BN + ((q * 32u) << 16);
            float mx = -FLT_MAX, second = -FLT_MAX, sum = 0.0f;
            for (uint32_t c0 = 0; c0 < p.N; c0 += 16) {
                uint32_t r[16];
                tmem_ld16(taddr + c0, r);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 16; i++)
                    if (c0 + i < p.N) {
                        const float v = fmaf(__uint_as_float(r[i]), p.scale, p.bias[c0 + i]);
                        if (v > mx) { second = mx; mx = v; } else if (v > second) second = v;
                    }
            }
            for (uint32_t c0 = 0; c0 < p.N; c0 += 16) {
                uint32_t r[16];
                tmem_ld16(taddr + c0, r);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 16; i++)
                    if (c0 + i < p.N) sum += expf(fmaf(__uint_as_float(r[i]), p.scale, p.bias[c0 + i]) - mx);
            }
            // log p1 - log p2 of the softmax equals the gap of the two largest logits; a row whose one-term pass left the
            // 16-bit range (non-finite logits or sum) is listed as well
            if (p.margin_idx && row < rows && p.N >= 2 && (!(mx - second >= p.margin_theta) || !(sum < FLT_MAX))) p.margin_idx[atomicAdd(p.margin_count, 1u)] = row;
            const float inv = sum > 0.0f ? 1.0f / sum : 1.0f;
            for (uint32_t c0 = 0; c0 < p.N; c0 += 16) {
                uint32_t r[16];
                tmem_ld16(taddr + c0, r);
                tmem_ld_wait();
                if (row < rows) {
                    const uint64_t orow = p.out_rows ? p.out_rows[row] : row;
#pragma unroll
                    for (int i = 0; i < 16; i++)
                        if (c0 + i < p.N)
                            p.out32[orow * p.ldo32 + c0 + i] =
                                expf(fmaf(__uint_as_float(r[i]), p.scale, p.bias[c0 + i]) - mx) * inv;
                }
            }
        }
        tc_fence_before();
        mbar_arrive(tempty0 + 8 * acc);
    }
}

// Fused row softmax for rows wider than one tile (up to SOFTMAX_WIDE_MAX columns; the CTA owns the row tile and walks its
// column tiles in order).  Per column tile the row's thread (lower column-half warps, one thread per TMEM lane) adds
// scale and bias, keeps the two largest logits seen so far and writes the raw logits to the output.  After the last
// column tile both warps of a quadrant share the tile's rows: a row at a time, lanes across the columns (coalesced),
// they read the row's logits once into registers, sum expf(v - max), apply the margin test and write expf(v - max) / sum
// -- the arithmetic of the reference's three sweeps (Activation.c:5-21), the division only when the sum is positive.
__device__ __forceinline__ void epilogue_softmax_wide(const GemmParams &p, const RowLimit &rl, uint32_t rows, uint32_t tmem_base, uint32_t tfull0,
                                                      uint32_t tempty0, uint32_t hx0, volatile int *abort_flag, uint32_t warp, uint32_t lane,
                                                      uint8_t *stage)
{
    const uint32_t q = warp & 3u, half = (warp - 2u) >> 2;
    const uint32_t ntile = my_tile_count(p, rl);
    float4 *slots = reinterpret_cast<float4 *>(stage);           // [2 row-tile parities][128 rows] {max, second, output row, row}
    float mx = -FLT_MAX, second = -FLT_MAX;
    for (uint32_t tcount = 0; tcount < ntile; tcount++) {
        uint32_t mt, nt;
        my_tile(p, rl, tcount, mt, nt);
        const uint32_t acc = tcount & 1u, acc_ph = (tcount >> 1) & 1u;
        if (!mbar_wait(tfull0 + 8 * acc, acc_ph, abort_flag, p.status, 4)) break;
        tc_fence_after();
        const uint32_t row = mt * BM + q * 32u + lane;
        const uint32_t orow = row < rows ? (p.out_rows ? p.out_rows[row] : row) : 0xFFFFFFFFu;
        if (half == 0) {
            if (nt == 0) { mx = -FLT_MAX; second = -FLT_MAX; }
            const uint32_t col0 = nt * p.BN, cols = p.N - col0 < p.BN ? p.N - col0 : p.BN;
            const uint32_t taddr = tmem_base + acc * p.BN + ((q * 32u) << 16);
            float *orow_ptr = p.out32 + (uint64_t)orow * p.ldo32 + col0;
            const bool vec = (p.ldo32 & 3u) == 0 && (reinterpret_cast<uintptr_t>(p.out32) & 15u) == 0;      // 16-byte stores (BN is a multiple of 4)
            for (uint32_t c0 = 0; c0 < cols; c0 += 16) {
                uint32_t r[16];
                tmem_ld16(taddr + c0, r);
                tmem_ld_wait();
                float v[16];
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    v[i] = c0 + i < cols ? fmaf(__uint_as_float(r[i]), p.scale, p.bias[col0 + c0 + i]) : -FLT_MAX;
                    if (v[i] > mx) { second = mx; mx = v[i]; } else if (v[i] > second) second = v[i];
                }
                if (orow != 0xFFFFFFFFu) {
                    if (vec && c0 + 16 <= cols) {
#pragma unroll
                        for (int i = 0; i < 16; i += 4) *reinterpret_cast<float4 *>(orow_ptr + c0 + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
                    } else {
#pragma unroll
                        for (int i = 0; i < 16; i++) if (c0 + i < cols) orow_ptr[c0 + i] = v[i];
                    }
                }
            }
        }
        tc_fence_before();
        mbar_arrive(tempty0 + 8 * acc);
        if (nt + 1 != p.n_tiles) continue;
        // ---- the row tile is complete ----
        const uint32_t rt = tcount / p.n_tiles;                   // this CTA's row-tile counter: slot and barrier parity
        float4 *slot = slots + (rt & 1u) * BM + q * 32u;
        if (half == 0) {
            slot[lane] = make_float4(mx, second, __uint_as_float(orow), __uint_as_float(row));
            __threadfence_block();                               // the raw logits and the slot, before the other warp is told
            mbar_arrive(hx0 + 8 * q);                            // (the barrier counts 32 arrivals: every lane)
            __syncwarp();
        } else if (!mbar_wait(hx0 + 8 * q, rt & 1u, abort_flag, p.status, 5)) break;
        for (uint32_t rr = 0; rr < 16; rr++) {
            const float4 st = slot[half * 16u + rr];
            const uint32_t o = __float_as_uint(st.z);
            if (o == 0xFFFFFFFFu) continue;                      // a row beyond the batch (the same for the whole warp)
            float *out = p.out32 + (uint64_t)o * p.ldo32;
            // the whole row in registers (32 values per lane, all loads in flight at once), each value through expf once
            float e[SOFTMAX_WIDE_MAX / 32];
#pragma unroll
            for (uint32_t j = 0; j < SOFTMAX_WIDE_MAX / 32; j++) {
                const uint32_t c = lane + 32u * j;
                e[j] = c < p.N ? out[c] : 0.0f;
            }
            float sum = 0.0f;
#pragma unroll
            for (uint32_t j = 0; j < SOFTMAX_WIDE_MAX / 32; j++)
                if (lane + 32u * j < p.N) { e[j] = expf(e[j] - st.x); sum += e[j]; }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
            // log p1 - log p2 of the softmax equals the gap of the two largest logits; a row whose one-term pass left the
            // 16-bit range (non-finite logits or sum) is listed as well
            if (lane == 0 && p.margin_idx && p.N >= 2 && (!(st.x - st.y >= p.margin_theta) || !(sum < FLT_MAX)))
                p.margin_idx[atomicAdd(p.margin_count, 1u)] = __float_as_uint(st.w);
            const float inv = sum > 0.0f ? 1.0f / sum : 1.0f;
#pragma unroll
            for (uint32_t j = 0; j < SOFTMAX_WIDE_MAX / 32; j++)
                if (lane + 32u * j < p.N) out[lane + 32u * j] = e[j] * inv;
        }
    }
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
spg_gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                   const __grid_constant__ CUtensorMap map_o, const GemmParams p)
{
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment of the operand tiles (required by the 128-byte swizzle atoms)
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *smem = smem_raw + (base - raw);

    const uint32_t b_tile_bytes = p.BN * BK * 2;
    const uint32_t a_off = 0, b_off = p.stages * A_TILE_BYTES;
    const uint32_t stg_off = b_off + p.stages * b_tile_bytes;        // epilogue patches, 1024-byte aligned like the tiles
    const uint32_t bar_off = stg_off + p.stg_bytes;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + bar_off);
    // barrier table: full[stages], empty[stages], tmem_full[2], tmem_empty[2], head_exchange[4]
    const uint32_t full0 = base + bar_off, empty0 = full0 + 8 * p.stages;
    const uint32_t tfull0 = empty0 + 8 * p.stages, tempty0 = tfull0 + 16, hx0 = tempty0 + 16;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * p.stages + 8);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    uint8_t *stage = smem + stg_off;

    // the warp index through a shuffle: provably warp-uniform, so the role code below keeps uniform values in uniform registers
    const uint32_t warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31u;
    const uint32_t abort_addr = smem_u32(const_cast<int *>(abort_flag));
    const uint32_t tmem_cols = 2 * p.BN < 32 ? 32 : 2 * p.BN;       // power of two: BN in {16,32,64,128,256}

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < p.stages; s++) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (uint32_t a = 0; a < 2; a++) { mbar_init(tfull0 + 8 * a, 1); mbar_init(tempty0 + 8 * a, 32 * EPI_WARPS); }
        for (uint32_t a = 0; a < 4; a++) mbar_init(hx0 + 8 * a, 32);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Everything above touched only this CTA's shared and tensor memory, so it may overlap the tail of the kernel
    // before this one in the stream; from here on its results are needed.
    spg_grid_trigger();
    spg_grid_wait();
    // rows may be limited by a count that only exists on the device (every role derives the same tile list from it);
    // the effective sizes live in their own small struct: the kernel parameters themselves stay untouched
    uint32_t rows = p.M;
    if (p.m_limit) {
        const uint32_t m = *reinterpret_cast<const volatile uint32_t *>(p.m_limit);
        rows = m < rows ? m : rows;
    }
    RowLimit rl;
    rl.m_tiles = (rows + BM - 1) / BM;
    rl.group_m = (rl.m_tiles && p.group_m > rl.m_tiles) ? rl.m_tiles : p.group_m;

    const uint32_t ntile = my_tile_count(p, rl);
    const uint32_t iters_per_tile = p.npass * p.kblocks;
    if (p.head_w) {
        // the head's weights (a few tens of KB) live in shared memory for the whole kernel
        const uint32_t n4 = ((p.N + 31u) & ~31u) * p.head_hp / 4;
        const float4 *src = reinterpret_cast<const float4 *>(p.head_w);
        float4 *dst = reinterpret_cast<float4 *>(stage);
        for (uint32_t i = threadIdx.x; i < n4; i += NUM_THREADS) dst[i] = src[i];
        __syncthreads();
    }

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        // The whole warp walks the loops convergently and one elected lane issues: every operand of the bulk-tensor
        // copies then stays warp-uniform (uniform registers) instead of being moved over per instruction.
        uint32_t it = 0;
        for (uint32_t ti = 0; ti < ntile; ti++) {
            uint32_t mt, nt;
            my_tile(p, rl, ti, mt, nt);
            // k-block outermost, the passes of a multi-term product inside: the weight tile of a k-block is fetched for every
            // pass, and fetched back to back the second fetch is an L2 hit -- with the passes outermost a small batch on a
            // large layer (weight panel of a tile beyond L2) streamed the weights from HBM once per pass
            for (uint32_t kb = 0; kb < p.kblocks; kb++) {
                for (uint32_t ps = 0; ps < p.npass; ps++, it++) {
                    const uint32_t s = it % p.stages, ph = (it / p.stages) & 1u;
                    mbar_wait_uniform(empty0 + 8 * s, ph ^ 1u, abort_addr, p.status, 1, WAIT_LIMIT);
                    if (elect_one()) {
                        mbar_arrive_expect_tx(full0 + 8 * s, A_TILE_BYTES + b_tile_bytes);
                        tma_load_3d(base + a_off + s * A_TILE_BYTES, &map_a, full0 + 8 * s,
                                    (int)(kb * BK), (int)(mt * BM), (int)p.pass_a[ps]);
                        tma_load_3d(base + b_off + s * b_tile_bytes, &map_w, full0 + 8 * s,
                                    (int)(kb * BK), (int)(nt * p.BN), (int)p.pass_w[ps]);
                    }
                    __syncwarp();
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer --------------------------------
        // Convergent like the producer: descriptors, addresses and counters stay in uniform registers, which is
        // where tcgen05.mma takes them from.  A wait that gives up only raises the abort flag (every later wait then
        // ends at once); the MMAs issued after that work on stale tiles, and the host discards the launch.
        uint32_t it = 0;
        for (uint32_t tcount = 0; tcount < ntile; tcount++) {
            const uint32_t acc = tcount & 1u, acc_ph = (tcount >> 1) & 1u;
            mbar_wait_uniform(tempty0 + 8 * acc, acc_ph ^ 1u, abort_addr, p.status, 2, WAIT_LIMIT);
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + acc * p.BN;
            for (uint32_t i = 0; i < iters_per_tile; i++, it++) {
                const uint32_t s = it % p.stages, ph = (it / p.stages) & 1u;
                mbar_wait_uniform(full0 + 8 * s, ph, abort_addr, p.status, 3, WAIT_LIMIT);
                tc_fence_after();
                const uint64_t da = make_smem_desc(base + a_off + s * A_TILE_BYTES);
                const uint64_t db = make_smem_desc(base + b_off + s * b_tile_bytes);
                if (elect_one()) {
#pragma unroll
                    for (uint32_t k = 0; k < BK / UMMA_K; k++)
                        umma_f16(d_tmem, da + 2 * k, db + 2 * k, p.idesc, (i | k) ? 1u : 0u);   // +32 bytes per K step
                    umma_commit(empty0 + 8 * s);          // frees the stage once these MMAs have read it
                    if (i + 1 == iters_per_tile) umma_commit(tfull0 + 8 * acc);  // accumulator complete
                }
                __syncwarp();
            }
        }
    } else {
        // ------------------------------ epilogue ----------------------------------
        // The activation is resolved once, outside every loop, so the per-element code is branch-free.
        // The activation (and the width of a fused head) is resolved once, outside every loop.
#define SPG_EPI(ACTV) \
        if (p.head_hp == 0) epilogue_loop<ACTV, 0>(p, rl, rows, tmem_base, tfull0, tempty0, abort_flag, warp, lane, stage, &map_o, hx0); \
        else if (p.head_hp == 12) epilogue_loop<ACTV, 12>(p, rl, rows, tmem_base, tfull0, tempty0, abort_flag, warp, lane, stage, &map_o, hx0); \
        else epilogue_loop<ACTV, 16>(p, rl, rows, tmem_base, tfull0, tempty0, abort_flag, warp, lane, stage, &map_o, hx0)
        switch (p.softmax ? -1 : p.act) {
            case -1:
                if (p.n_tiles == 1) epilogue_softmax(p, rl, rows, tmem_base, tfull0, tempty0, abort_flag, warp, lane);
                else epilogue_softmax_wide(p, rl, rows, tmem_base, tfull0, tempty0, hx0, abort_flag, warp, lane, stage);
                break;
            case SPG_ACT_RELU:     SPG_EPI(SPG_ACT_RELU); break;
            case SPG_ACT_LEAKY:    SPG_EPI(SPG_ACT_LEAKY); break;
            case SPG_ACT_FOO52:    SPG_EPI(SPG_ACT_FOO52); break;
            case SPG_ACT_TANH:     SPG_EPI(SPG_ACT_TANH); break;
            case SPG_ACT_SIGMOID:  SPG_EPI(SPG_ACT_SIGMOID); break;
            default:               SPG_EPI(SPG_ACT_NONE); break;
        }
#undef SPG_EPI
    }

    // ------------------------------ common tail -----------------------------------
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
    }
}

// ---------------------------------------------------------------------------------
// 16-bit weight operand preparation: any stored precision -> `parts` planes of
// [out][ldw] 16-bit values (plane 0 = round(q), plane 1 = round(q - plane 0)).
// Integer formats are exact in one plane; the per-array scale stays outside.
// ---------------------------------------------------------------------------------
template <typename T16>
__global__ void __launch_bounds__(256)
spg_dequant16_kernel(const void *__restrict__ w, int precision, uint32_t in, uint32_t out,
                     T16 *__restrict__ dst, uint32_t ldw, uint64_t plane, int parts)
{
    const uint64_t total = (uint64_t)out * ldw;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t j = (uint32_t)(i / ldw), k = (uint32_t)(i % ldw);
        float v = k < in ? spg_decode_elem(w, (uint64_t)j * in + k, precision) : 0.0f;
        for (int pt = 0; pt < parts; pt++) {
            T16 h;
            float back;
            if constexpr (std::is_same<T16, __half>::value) { h = __float2half_rn(v); back = __half2float(h); }
            else { h = __float2bfloat16_rn(v); back = __bfloat162float(h); }
            dst[(uint64_t)pt * plane + i] = h;
            v -= back;
        }
    }
}

// Head weights for the fused narrow last layer: dst[c][j] = q(H.w[j][c]) (unscaled), c < round_up(in, 32), j < hp;
// entries beyond the layer's real size are zero.
__global__ void __launch_bounds__(256)
spg_head_weights_kernel(const void *__restrict__ w, int precision, uint32_t in, uint32_t out, uint32_t hp, uint32_t rows, float *__restrict__ dst)
{
    const uint32_t total = rows * hp;
    for (uint32_t i = blockIdx.x * 256 + threadIdx.x; i < total; i += gridDim.x * 256) {
        const uint32_t c = i / hp, j = i % hp;
        dst[i] = (c < in && j < out) ? spg_decode_elem(w, (uint64_t)j * in + c, precision) : 0.0f;
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
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// 3-D map over `parts` planes of a row-major [rows][ld] 16-bit matrix whose first K columns are valid.
int make_map(CUtensorMap *map, const void *base, int type16, uint32_t K, uint32_t rows, uint32_t ld, uint64_t plane,
             int parts, uint32_t box_rows)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) { spgk_set_error("cuTensorMapEncodeTiled", "driver entry point not available"); return SPGK_E_CUDA; }
    if (((uintptr_t)base & 15u) || (ld & 7u) || (parts > 1 && (plane & 7u))) {
        spgk_set_error("tensor map", "operand is not 16-byte aligned");
        return SPGK_E_ARG;
    }
    cuuint64_t dims[3] = { K, rows, (cuuint64_t)parts };
    cuuint64_t plane_bytes = parts > 1 ? plane * 2 : (cuuint64_t)rows * ld * 2;
    plane_bytes = (plane_bytes + 15) & ~(cuuint64_t)15;
    cuuint64_t strides[2] = { (cuuint64_t)ld * 2, plane_bytes };
    cuuint32_t box[3] = { BK, box_rows, 1 };
    cuuint32_t estr[3] = { 1, 1, 1 };
    CUresult r = fn(map, type16 == SPGK_T_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3,
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

uint32_t pick_bn(uint32_t out)
{
    if (out > 128) return 256;
    uint32_t bn = 16;
    while (bn < out) bn <<= 1;
    return bn;
}

}  // namespace

extern "C" {

uint32_t spgk_gemm_tc_softmax_max(void) { return SOFTMAX_FUSE_MAX; }

// Whether a softmax layer of this width is finished inside the GEMM's epilogue for a batch of `rows`: always when the row
// fits one tile; up to SOFTMAX_WIDE_MAX columns when there are enough row tiles to give most SMs one (a CTA then owns
// whole row tiles), and not for a device-resident row count (a handful of rows would leave the layer to a few CTAs).
int spgk_gemm_tc_softmax_fusable(uint32_t width, uint32_t rows, int dynamic_rows)
{
    if (width <= SOFTMAX_FUSE_MAX) return 1;
    return (width <= SOFTMAX_WIDE_MAX && !dynamic_rows && rows >= 64u * BM) ? 1 : 0;
}

int spgk_gemm_tc_supported(const spgk_layer *L)
{
    if (!L || L->in == 0 || L->out == 0) return 0;
    SpgDeviceProps dp;
    if (spg_device_props(&dp) != SPGK_OK) return 0;
    return dp.cc == 100 ? 1 : 0;     // tcgen05 / TMEM exist on sm_100 only
}

int spgk_weights16_direct(const spgk_layer *L, int type16)
{
    if ((L->in & 7u) || ((uintptr_t)L->w & 15u)) return 0;
    return (L->precision == SPG_P_F16 && type16 == SPGK_T_F16) || (L->precision == SPG_P_BF16 && type16 == SPGK_T_BF16);
}

size_t spgk_weights16_bytes(const spgk_layer *L, int parts)
{
    return (size_t)L->out * ((L->in + 7u) & ~7u) * 2u * (size_t)parts;
}

int spgk_dequant16(const spgk_layer *L, void *dst, uint32_t ldw, uint64_t plane, int parts, int type16, void *stream)
{
    if (!L || !dst || ldw < L->in || (ldw & 7u) || parts < 1 || parts > 2) { spgk_set_error("spgk_dequant16", "bad argument"); return SPGK_E_ARG; }
    const uint64_t total = (uint64_t)L->out * ldw;
    const uint32_t blocks = (uint32_t)((total + 255) / 256 < 148ull * 32 ? (total + 255) / 256 : 148ull * 32);
    if (type16 == SPGK_T_F16)
        spg_dequant16_kernel<__half><<<blocks, 256, 0, (cudaStream_t)stream>>>(L->w, L->precision, L->in, L->out, (__half *)dst, ldw, plane, parts);
    else
        spg_dequant16_kernel<__nv_bfloat16><<<blocks, 256, 0, (cudaStream_t)stream>>>(L->w, L->precision, L->in, L->out, (__nv_bfloat16 *)dst, ldw, plane, parts);
    return spgk_check_launch("spg_dequant16_kernel");
}

size_t spgk_head_weights_bytes(const spgk_layer *H);
static uint32_t head_hp(const spgk_layer *H) { return H->out <= 12 ? 12u : 16u; }

int spgk_gemm_tc_head_supported(const spgk_layer *L, const spgk_layer *H)
{
    // a head of at most 16 outputs behind a layer of more than one 256-wide column tile whose weights fit shared memory
    if (!L || !H || H->in != L->out || H->out == 0 || H->out > 16 || L->out <= 256 || L->act == SPG_ACT_SOFTMAX) return 0;
    if ((unsigned)H->precision >= SPG_P_COUNT || !H->w || !H->bias) return 0;
    return spgk_head_weights_bytes(H) <= 96u * 1024 ? 1 : 0;
}

size_t spgk_head_weights_bytes(const spgk_layer *H)
{
    return H ? (size_t)((H->in + 31u) & ~31u) * head_hp(H) * sizeof(float) : 0;
}

int spgk_head_weights(const spgk_layer *H, float *dst, void *stream)
{
    if (!H || !dst || !H->w) { spgk_set_error("spgk_head_weights", "bad argument"); return SPGK_E_ARG; }
    const uint32_t rows = (H->in + 31u) & ~31u, hp = head_hp(H);
    uint32_t blocks = (rows * hp + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    spg_head_weights_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(H->w, H->precision, H->in, H->out, hp, rows, dst);
    return spgk_check_launch("spg_head_weights_kernel");
}

static int gemm_launch(const spgk_layer *L,
                       const void *w16, uint32_t ldw, uint64_t w_plane, int w_parts, int w_type16,
                       const void *a16, uint32_t lda, uint64_t a_plane, int a_parts, int type16,
                       void *out16, uint32_t ldo16, uint64_t o_plane, int out_parts,
                       float *out32, uint32_t ldo32,
                       uint32_t N, int softmax_fused, int32_t *status, void *stream,
                       const spgk_layer *head, const float *head_w)
{
    if (!L || !w16 || !a16 || !L->bias || (!out16 && !out32) || !status || a_parts < 1 || a_parts > 2 || w_parts < 1 || w_parts > 2 ||
        (out16 && (ldo16 & 7u)) || (softmax_fused && (!out32 || L->out > SOFTMAX_WIDE_MAX))) {
        spgk_set_error("spgk_layer_gemm_tc", "bad argument");
        return SPGK_E_ARG;
    }
    if (N == 0) return SPGK_OK;
    SpgDeviceProps dp;
    {
        const int prc = spg_device_props(&dp);
        if (prc) return prc;
        // the opt-in for large dynamic shared memory is a per-device function attribute
        static SpgOncePerDevice once;
        int dev = 0;
        SPGK_CUDA(cudaGetDevice(&dev));
        const int orc = once.run(dev, [&]() -> int {
            SPGK_CUDA(cudaFuncSetAttribute(spg_gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dp.smem_optin));
            return SPGK_OK;
        });
        if (orc) return orc;
    }
    const int sm_count = dp.sm_count;
    const size_t smem_max = dp.smem_optin;
    GemmParams p{};
    p.M = N; p.N = L->out; p.K = L->in;
    p.BN = pick_bn(L->out);
    // a device-resident row count usually means a small selection of a large batch: when the caller's estimate of
    // it gives fewer tiles than SMs, narrower tiles spread the work (at the price of re-reading the rows more often)
    if (spg_tls_rows_limit && spg_tls_rows_expected && !softmax_fused) {
        const uint32_t mt = (spg_tls_rows_expected + BM - 1) / BM;
        while (p.BN > 64 && mt * ((L->out + p.BN - 1) / p.BN) < (uint32_t)sm_count) p.BN >>= 1;
    }
    p.kblocks = (L->in + BK - 1) / BK;
    // passes: hi*hi first, then the correction terms (lo*hi, hi*lo); lo*lo is below fp32 resolution
    p.npass = 0;
    p.pass_a[p.npass] = 0; p.pass_w[p.npass] = 0; p.npass++;
    if (a_parts > 1) { p.pass_a[p.npass] = 1; p.pass_w[p.npass] = 0; p.npass++; }
    if (w_parts > 1) { p.pass_a[p.npass] = 0; p.pass_w[p.npass] = 1; p.npass++; }
    const uint32_t stage_bytes = A_TILE_BYTES + p.BN * BK * 2;
    if (head) {
        p.head_w = head_w; p.head_bias = head->bias; p.head_scale = head->w_scale; p.head_out = head->out; p.head_hp = head_hp(head);
        p.head_softmax = head->act == SPG_ACT_SOFTMAX ? 1 : 0;
        p.head_act = head->act == SPG_ACT_SOFTMAX ? SPG_ACT_NONE : head->act;
        p.stg_bytes = (uint32_t)((spgk_head_weights_bytes(head) + 1023) & ~(size_t)1023) + 4 * 2 * 32 * 16 * 4;
    } else {
        p.stg_bytes = STG_BYTES;
    }
    const size_t fixed = 1024 /*alignment slack*/ + 8 * (2 * 12 + 8) + 64 + p.stg_bytes;
    uint32_t stages = (uint32_t)((smem_max - fixed) / stage_bytes);
    if (stages > 12) stages = 12;
    if (stages < 2) { spgk_set_error("spgk_layer_gemm_tc", "not enough shared memory"); return SPGK_E_UNSUPPORTED; }
    p.stages = stages;
    p.m_tiles = (N + BM - 1) / BM;
    p.n_tiles = (L->out + p.BN - 1) / p.BN;
    p.group_m = p.m_tiles < 16 ? p.m_tiles : 16;
    p.idesc = (1u << 4) | ((uint32_t)type16 << 7) | ((uint32_t)w_type16 << 10) | ((p.BN >> 3) << 17) | ((BM >> 4) << 24);
    p.scale = L->w_scale; p.bias = L->bias;
    p.act = L->act == SPG_ACT_SOFTMAX ? SPG_ACT_NONE : L->act;
    p.softmax = softmax_fused ? 1 : 0;
    if (softmax_fused && p.n_tiles != 1 && L->out > SOFTMAX_WIDE_MAX) { spgk_set_error("spgk_layer_gemm_tc", "softmax row wider than the fused epilogue takes"); return SPGK_E_ARG; }
    p.own_rows = (head || (softmax_fused && p.n_tiles != 1)) ? 1u : 0u;
    p.out16 = out16; p.ldo16 = ldo16; p.o_plane = o_plane; p.out_parts = out_parts; p.type16 = type16;
    p.out32 = out32; p.ldo32 = ldo32;
    p.status = status;
    p.m_limit = spg_tls_rows_limit;
    if ((softmax_fused || (head && head->act == SPG_ACT_SOFTMAX)) && spg_tls_margin_idx) { p.margin_theta = spg_tls_margin_theta; p.margin_idx = spg_tls_margin_idx; p.margin_count = spg_tls_margin_count; }
    p.out_rows = spg_tls_out_rows;

    CUtensorMap map_a, map_w;
    int rc = make_map(&map_a, a16, type16, L->in, N, lda, a_plane, a_parts, BM);
    if (rc) return rc;
    rc = make_map(&map_w, w16, w_type16, L->in, L->out, ldw, w_plane, w_parts, p.BN);
    if (rc) return rc;

    // 16-bit output through TMA stores when it is one plane and the tiles are wide enough for 64-column patches
    CUtensorMap map_o = map_a;
    p.tma_store = (out16 && out_parts == 1 && p.BN >= 128 && !softmax_fused && !head) ? 1 : 0;
    if (p.tma_store) {
        rc = make_map(&map_o, out16, type16, ldo16, N, ldo16, o_plane, 1, 32);
        if (rc) return rc;
    }
    const uint32_t tiles = p.own_rows ? p.m_tiles : p.m_tiles * p.n_tiles;   // with a head or a wide softmax a CTA owns whole row tiles
    const uint32_t grid = tiles < (uint32_t)sm_count ? tiles : (uint32_t)sm_count;
    const size_t smem = 1024 + (size_t)stages * stage_bytes + p.stg_bytes + 8 * (2 * stages + 8) + 64;
    SPGK_CUDA(spg_launch_chained(spg_gemm_tc_kernel, dim3(grid), dim3(NUM_THREADS), smem, (cudaStream_t)stream, map_a, map_w, map_o, p));
    return spgk_check_launch("spg_gemm_tc_kernel");
}

int spgk_layer_gemm_tc(const spgk_layer *L,
                       const void *w16, uint32_t ldw, uint64_t w_plane, int w_parts, int w_type16,
                       const void *a16, uint32_t lda, uint64_t a_plane, int a_parts, int type16,
                       void *out16, uint32_t ldo16, uint64_t o_plane, int out_parts,
                       float *out32, uint32_t ldo32,
                       uint32_t N, int softmax_fused, int32_t *status, void *stream)
{
    return gemm_launch(L, w16, ldw, w_plane, w_parts, w_type16, a16, lda, a_plane, a_parts, type16,
                       out16, ldo16, o_plane, out_parts, out32, ldo32, N, softmax_fused, status, stream, nullptr, nullptr);
}

int spgk_layer_gemm_tc_head(const spgk_layer *L,
                            const void *w16, uint32_t ldw, uint64_t w_plane, int w_parts, int w_type16,
                            const void *a16, uint32_t lda, uint64_t a_plane, int a_parts, int type16,
                            const spgk_layer *head, const float *head_w, float *out32, uint32_t ldo32,
                            uint32_t N, int32_t *status, void *stream)
{
    if (!head || !head_w || !out32 || !spgk_gemm_tc_head_supported(L, head)) { spgk_set_error("spgk_layer_gemm_tc_head", "bad argument"); return SPGK_E_ARG; }
    return gemm_launch(L, w16, ldw, w_plane, w_parts, w_type16, a16, lda, a_plane, a_parts, type16,
                       nullptr, 0, 0, 1, out32, ldo32, N, 0, status, stream, head, head_w);
}

// Reads back and clears the status word the GEMM kernels report bounded-wait
// failures in (synchronises the stream).
int spgk_gemm_tc_status(int32_t *status, void *stream)
{
    int32_t h = 0;
    SPGK_CUDA(cudaMemcpyAsync(&h, status, sizeof h, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    SPGK_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    if (h != 0) {
        char msg[96];
        snprintf(msg, sizeof msg, "bounded wait %d gave up inside the tcgen05 GEMM", (int)h);
        spgk_set_error("spg_gemm_tc_kernel", msg);
        SPGK_CUDA(cudaMemsetAsync(status, 0, sizeof h, (cudaStream_t)stream));
        return SPGK_E_TIMEOUT;
    }
    return SPGK_OK;
}

}  // extern "C"

namespace {
// A barrier nobody ever arrives on, waited for with the same bounded waits the tensor-core kernels use (no copy, no MMA and
// no tensor memory involved): both give up after `limit` attempts, record their code, raise the abort flag and return.
__global__ void spg_wait_selftest_kernel(int32_t *status, uint32_t limit)
{
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) { mbar_init(smem_u32(&bar), 1); abort_flag = 0; spgtc::mbar_fence_init(); }
    __syncthreads();
    if (threadIdx.x < 32) {
        // warp 0: the convergent-warp wait; its expiry raises the flag ...
        mbar_wait_uniform(smem_u32(&bar), 0, smem_u32(&abort_flag), status, 41, limit);
    }
    __syncthreads();
    if (threadIdx.x >= 32) {
        // ... which the per-thread wait of warp 1 then finds up at once (it returns false without recording its own code)
        const bool ok = spgtc::mbar_wait(smem_u32(&bar), 0, &abort_flag, status + 1, 42, limit);
        if (threadIdx.x == 32) status[2] = ok ? 1 : 2;
    }
}
}  // namespace

extern "C" {

// Failure-path check: makes a bounded device wait run out on purpose (the kernel returns normally; nothing faults) and
// reports through the same status word and call the GEMM uses: SPGK_E_TIMEOUT with the wait's code in the message.
int spgk_selftest_bounded_wait(int32_t *status3, uint32_t limit, void *stream)
{
    if (!status3 || limit == 0 || limit > 4096) { spgk_set_error("spgk_selftest_bounded_wait", "bad argument"); return SPGK_E_ARG; }
    SPGK_CUDA(cudaMemsetAsync(status3, 0, 3 * sizeof(int32_t), (cudaStream_t)stream));
    spg_wait_selftest_kernel<<<1, 64, 0, (cudaStream_t)stream>>>(status3, limit);
    int rc = spgk_check_launch("spg_wait_selftest_kernel");
    if (rc) return rc;
    return spgk_gemm_tc_status(status3, stream);
}

// ---------------------------------------------------------------------------------
// Allocation-free variant of the layer GEMM.
//
// Some callers must not allocate device memory at all: a serving process that gave
// the whole of HBM to its own arena at start-up has nothing left for cudaMalloc to
// hand out, and a latency-critical loop cannot afford the device-wide
// synchronisation that cudaMalloc / cudaFree imply.  For them the scratch this layer
// needs -- the 16-bit weight operand expanded from the packed payload, and the word
// the kernel reports a bounded wait in -- lives in a fixed array inside the library's
// device image.  Every GPU that loads the library carries that array until the
// process exits, which is why its size is modest and fixed.
// ---------------------------------------------------------------------------------
constexpr size_t NOALLOC_HEAD_BYTES = 256;                               // status word, padded
constexpr size_t NOALLOC_WEIGHT_BYTES = SPGK_NOALLOC_MAX_WEIGHT_BYTES;   // 16-bit weight operand
static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_HEAD_BYTES + NOALLOC_WEIGHT_BYTES];

constexpr int NOALLOC_MAX_DEVICES = 64;
static void *g_noalloc_dev_ptr[NOALLOC_MAX_DEVICES];      // device address of the array, per device
static std::mutex g_noalloc_mutex;

int spgk_layer_gemm_tc_noalloc(const spgk_layer *L,
                               const void *a16, uint32_t lda, uint64_t a_plane, int a_parts, int type16,
                               void *out16, uint32_t ldo16, uint64_t o_plane, int out_parts,
                               float *out32, uint32_t ldo32,
                               uint32_t N, int softmax_fused, void *stream)
{
    if (!L || !L->w) { spgk_set_error("spgk_layer_gemm_tc_noalloc", "bad argument"); return SPGK_E_ARG; }
    const bool direct = spgk_weights16_direct(L, type16) != 0;
    const int w_parts = (!direct && L->precision == SPG_P_F32 && a_parts == 2) ? 2 : 1;
    const size_t need = direct ? 0 : spgk_weights16_bytes(L, w_parts);
    if (need > NOALLOC_WEIGHT_BYTES) {
        char msg[160];
        snprintf(msg, sizeof msg, "layer needs %zu bytes of weight-operand scratch, the built-in array holds %zu "
                 "(use spgk_layer_gemm_tc with caller-provided scratch)", need, (size_t)NOALLOC_WEIGHT_BYTES);
        spgk_set_error("spgk_layer_gemm_tc_noalloc", msg);
        return SPGK_E_ARG;
    }
    // Set-up, once per device and with that device current: in host code the array's name is only a
    // stand-in, the address a kernel can use comes from cudaGetSymbolAddress.
    int dev = 0;
    SPGK_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= NOALLOC_MAX_DEVICES) { spgk_set_error("spgk_layer_gemm_tc_noalloc", "device index out of range"); return SPGK_E_ARG; }
    void *base = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_noalloc_mutex);
        if (!g_noalloc_dev_ptr[dev]) {
            void *p = nullptr;
            SPGK_CUDA(cudaGetSymbolAddress(&p, g_noalloc_scratch));
            g_noalloc_dev_ptr[dev] = p;
        }
        base = g_noalloc_dev_ptr[dev];
    }
    int32_t *status = reinterpret_cast<int32_t *>(base);
    void *w16_scratch = static_cast<unsigned char *>(base) + NOALLOC_HEAD_BYTES;
    // The array keeps whatever the previous call left: the status word must start at zero; the weight
    // operand is rewritten in full (padding columns included) by the expansion below.
    SPGK_CUDA(cudaMemsetAsync(status, 0, sizeof(int32_t), (cudaStream_t)stream));
    const void *w16 = L->w;
    uint32_t ldw = L->in;
    uint64_t w_plane = 0;
    if (!direct) {
        ldw = (L->in + 7u) & ~7u;
        w_plane = (uint64_t)L->out * ldw;
        int rc = spgk_dequant16(L, w16_scratch, ldw, w_plane, w_parts, type16, stream);
        if (rc) return rc;
        w16 = w16_scratch;
    }
    int rc = spgk_layer_gemm_tc(L, w16, ldw, w_plane, w_parts, type16, a16, lda, a_plane, a_parts, type16,
                                out16, ldo16, o_plane, out_parts, out32, ldo32, N, softmax_fused, status, stream);
    if (rc) return rc;
    return spgk_gemm_tc_status(status, stream);
}

}  // extern "C"
