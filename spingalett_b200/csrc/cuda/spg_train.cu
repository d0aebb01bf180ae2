// spg_train.cu -- kernels of one mini-batch training step (cross-entropy + Adam)
// and the NCCL plumbing for its data-parallel gradient exchange.
//
// The step follows the reference's batched trainer (Src/Spingalett.Training.c):
//   forward   C = act(A W^T + b)                         batch_forward            :313-345
//   delta_L   = a_L - t                                  batch_compute_deltas     :366-371
//   delta_l   = (delta_{l+1} W_l) * act'(a_l)            batch_compute_deltas     :374-393
//   gW_l      = s * delta_{l+1}^T a_l,  gB_l = s * colsum batch_accumulate_gradients :396-419
//   Adam      eps inside the square root                  SIMD.c:279-328
// Everything is fp32, as in the reference.  The step is latency-bound (about
// 1.2 GFLOP per 256-row batch of the 784-512-1000-10 MLP), so the GEMMs are a
// plain shared-memory tiled fp32 kernel with the three operand layouts the step
// needs and the elementwise work fused into its epilogue.
#include "spg_common.cuh"
#include <dlfcn.h>
#include <chrono>
#include <condition_variable>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <mutex>
#include <thread>

namespace {

constexpr int TK = 16;      // k depth of a staged tile; the CTA tile is TS x TS, (TS/4)^2 threads with 4x4 outputs each

enum { GEMM_FWD = 0, GEMM_DELTA = 1, GEMM_GRAD = 2 };

// Four consecutive floats at `base`: one 128-bit load when `vec`, else element-wise with zeros where the row is
// outside the matrix (`row_ok` false) or the element index first+j reaches `limit`.
__device__ __forceinline__ float4 train_load4(const float *base, bool vec, bool row_ok, uint32_t first, uint32_t limit)
{
    if (vec) return *reinterpret_cast<const float4 *>(base);
    float4 v;
    v.x = row_ok && first < limit ? base[0] : 0.0f;
    v.y = row_ok && first + 1 < limit ? base[1] : 0.0f;
    v.z = row_ok && first + 2 < limit ? base[2] : 0.0f;
    v.w = row_ok && first + 3 < limit ? base[3] : 0.0f;
    return v;
}

// MODE 0: C[M][N] = act(A[M][K] . B[N][K]^T + bias[N])        (A = activations, B = weights [out][in])
// MODE 1: C[M][N] = (A[M][K] . B[K][N]) * act'(aux[M][N])      (A = delta_{l+1}, B = weights [next][cur])
// MODE 2: C[M][N] = alpha * A[K][M]^T . B[K][N]                 (A = delta [rows][out], B = activations [rows][in])
// The A tile is staged as As[k][m] and the B tile as Bs[k][n].  Every thread owns R groups of four elements of each
// operand, consecutive along that operand's contiguous axis; the groups of the next k-tile are loaded into registers
// before the products of the current one are formed, so the global-memory latency hides behind the arithmetic.
// KS > 1 puts KS such thread groups ("slices") in the CTA: slice s takes the k-tiles s, s+KS, ... and the partial sums are
// added in slice order through shared memory at the end, so the result does not depend on timing.  It is what keeps an SM
// busy when the whole product has fewer tiles than the GPU has SMs and a CTA would otherwise be two warps waiting on loads.
template <int MODE, int TS, int KS>
__global__ void __launch_bounds__((TS / 4) * (TS / 4) * KS)
spg_train_gemm_kernel(const float *__restrict__ A, uint32_t lda, const float *__restrict__ B, uint32_t ldb,
                      float *__restrict__ C, uint32_t ldc, uint32_t M, uint32_t N, uint32_t K,
                      float alpha, const float *__restrict__ bias, const float *__restrict__ aux, uint32_t ldaux, int act,
                      float *__restrict__ colsum)
{
    constexpr int TM = TS, TN = TS, NT = (TS / 4) * (TS / 4), Q = TS / 4;     // Q: groups of four per tile row along m or n
    constexpr int R = TS * TK / 4 / NT;                                       // groups per thread per operand
    constexpr bool a_km = MODE == GEMM_GRAD;                    // A stored [K][M] (contiguous in m); otherwise [M][K]
    constexpr bool b_nk = MODE == GEMM_FWD;                     // B stored [N][K] (contiguous in k); otherwise [K][N]
    static_assert(KS == 1 || (KS - 1) * NT * 20 <= KS * 2 * TK * (TS + 4), "the partial sums reuse the staging memory");
    __shared__ __align__(16) float sm[KS][2][TK][TS + 4];
    const uint32_t slice = threadIdx.x / NT, tid = threadIdx.x % NT, tx = tid % Q, ty = tid / Q;
    float (*As)[TS + 4] = sm[slice][0];
    float (*Bs)[TS + 4] = sm[slice][1];
    const uint32_t m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
    const bool a_al = (lda & 3u) == 0 && (reinterpret_cast<uintptr_t>(A) & 15u) == 0 && m0 + TM <= M;
    const bool b_al = (ldb & 3u) == 0 && (reinterpret_cast<uintptr_t>(B) & 15u) == 0 && n0 + TN <= N;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.0f;
    float4 ra[R], rb[R];
    // MODE 2 with `colsum`: the CTAs of the first tile column also sum their A tile over k, colsum[m] = alpha * sum_k A[k][m]
    // (the bias gradient beside the weight gradient); one thread per group of four m carries those sums
    const bool cs = MODE == GEMM_GRAD && colsum != nullptr && blockIdx.x == 0 && tx == 0;
    float bs[4] = { 0.0f, 0.0f, 0.0f, 0.0f };

    auto fetch = [&](uint32_t k0) {
        const bool whole = k0 + TK <= K;
#pragma unroll
        for (int r = 0; r < R; r++) {
            const uint32_t i = tid + r * NT;
            if (a_km) {
                const uint32_t k = i / Q, m = (i % Q) * 4;
                ra[r] = train_load4(A + (uint64_t)(k0 + k) * lda + m0 + m, a_al && whole, k0 + k < K, m0 + m, M);
            } else {
                const uint32_t m = i / (TK / 4), k = (i % (TK / 4)) * 4;
                ra[r] = train_load4(A + (uint64_t)(m0 + m) * lda + k0 + k, a_al && whole, m0 + m < M, k0 + k, K);
            }
            if (b_nk) {
                const uint32_t n = i / (TK / 4), k = (i % (TK / 4)) * 4;
                rb[r] = train_load4(B + (uint64_t)(n0 + n) * ldb + k0 + k, b_al && whole, n0 + n < N, k0 + k, K);
            } else {
                const uint32_t k = i / Q, n = (i % Q) * 4;
                rb[r] = train_load4(B + (uint64_t)(k0 + k) * ldb + n0 + n, b_al && whole, k0 + k < K, n0 + n, N);
            }
        }
    };
    auto stage = [&]() {
#pragma unroll
        for (int r = 0; r < R; r++) {
            const uint32_t i = tid + r * NT;
            if (a_km) {
                *reinterpret_cast<float4 *>(&As[i / Q][(i % Q) * 4]) = ra[r];
            } else {
                const uint32_t m = i / (TK / 4), k = (i % (TK / 4)) * 4;
                As[k][m] = ra[r].x; As[k + 1][m] = ra[r].y; As[k + 2][m] = ra[r].z; As[k + 3][m] = ra[r].w;
            }
            if (b_nk) {
                const uint32_t n = i / (TK / 4), k = (i % (TK / 4)) * 4;
                Bs[k][n] = rb[r].x; Bs[k + 1][n] = rb[r].y; Bs[k + 2][n] = rb[r].z; Bs[k + 3][n] = rb[r].w;
            } else {
                *reinterpret_cast<float4 *>(&Bs[i / Q][(i % Q) * 4]) = rb[r];
            }
        }
    };

    // every slice runs the same number of rounds (a tile beyond K loads as zeros), so the CTA-wide barriers line up
    fetch(slice * TK);
    for (uint32_t kb = 0; kb < K; kb += KS * TK) {
        stage();
        __syncthreads();
        if (kb + KS * TK < K) fetch(kb + (KS + slice) * TK);
#pragma unroll
        for (int k = 0; k < TK; k++) {
            const float4 av = *reinterpret_cast<const float4 *>(&As[k][ty * 4]);
            const float4 bv = *reinterpret_cast<const float4 *>(&Bs[k][tx * 4]);
            const float a[4] = { av.x, av.y, av.z, av.w }, b[4] = { bv.x, bv.y, bv.z, bv.w };
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
            if (cs) {
#pragma unroll
                for (int i = 0; i < 4; i++) bs[i] += a[i];
            }
        }
        __syncthreads();
    }
    if (KS > 1) {
        float *red = &sm[0][0][0][0];
        if (slice > 0) {
#pragma unroll
            for (int i = 0; i < 16; i++) red[((slice - 1) * 20 + i) * NT + tid] = acc[i >> 2][i & 3];
            if (cs) {
#pragma unroll
                for (int i = 0; i < 4; i++) red[((slice - 1) * 20 + 16 + i) * NT + tid] = bs[i];
            }
        }
        __syncthreads();
        if (slice > 0) return;
        for (int sl = 0; sl < KS - 1; sl++) {
#pragma unroll
            for (int i = 0; i < 16; i++) acc[i >> 2][i & 3] += red[(sl * 20 + i) * NT + tid];
            if (cs) {
#pragma unroll
                for (int i = 0; i < 4; i++) bs[i] += red[(sl * 20 + 16 + i) * NT + tid];
            }
        }
    }
    if (cs) {
#pragma unroll
        for (int i = 0; i < 4; i++)
            if (m0 + ty * 4 + i < M) colsum[m0 + ty * 4 + i] = alpha * bs[i];
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint32_t m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const uint32_t n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (MODE == GEMM_FWD) v = spg_activate(v + bias[n], act);
            else if (MODE == GEMM_DELTA) v *= spg_derivative(aux[(uint64_t)m * ldaux + n], act);
            else v *= alpha;
            C[(uint64_t)m * ldc + n] = v;
        }
    }
}

// ---- the same three products on the tensor cores, with fp32-level error -------------------------------------------------
// An fp32 value x is split into hi = tf32(x) and lo = tf32(x - hi); a*b is formed as a_lo*b_hi + a_hi*b_lo + a_hi*b_hi by
// three mma.m16n8k8.tf32 with fp32 accumulation (the dropped a_lo*b_lo term is below 2^-22 of the product).  CTA tile
// 32 x 32, KS k-slices of two warps each (a warp owns 16 rows x 32 columns of the slice's partial sum); staging, slice
// order and the fixed-order addition of the partial sums are those of spg_train_gemm_kernel.  The staged tiles have a
// pitch of 40 floats, which makes the fragment reads As[k][m], k = lane%4 (+4), m = lane/4 (+8), conflict-free.
__device__ __forceinline__ void tf32_split(float x, uint32_t &hi, uint32_t &lo)
{
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hi) : "f"(x));
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(lo) : "f"(x - __uint_as_float(hi)));
}

__device__ __forceinline__ void mma_tf32(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int MODE, int KS>
__global__ void __launch_bounds__(64 * KS)
spg_train_mma_kernel(const float *__restrict__ A, uint32_t lda, const float *__restrict__ B, uint32_t ldb,
                     float *__restrict__ C, uint32_t ldc, uint32_t M, uint32_t N, uint32_t K,
                     float alpha, const float *__restrict__ bias, const float *__restrict__ aux, uint32_t ldaux, int act,
                     float *__restrict__ colsum)
{
    constexpr int TS = 32, NT = 64, Q = 8, R = 2, P = TS + 8;
    constexpr bool a_km = MODE == GEMM_GRAD;
    constexpr bool b_nk = MODE == GEMM_FWD;
    static_assert((KS - 1) * (NT * 16 + TS) <= KS * 2 * TK * P, "the partial sums reuse the staging memory");
    __shared__ __align__(16) float sm[KS][2][TK][P];
    const uint32_t slice = threadIdx.x / NT, tid = threadIdx.x % NT, lane = tid & 31u, mh = tid >> 5, g = lane >> 2, t = lane & 3u;
    float (*As)[P] = sm[slice][0];
    float (*Bs)[P] = sm[slice][1];
    const uint32_t m0 = blockIdx.y * TS, n0 = blockIdx.x * TS;
    const bool a_al = (lda & 3u) == 0 && (reinterpret_cast<uintptr_t>(A) & 15u) == 0 && m0 + TS <= M;
    const bool b_al = (ldb & 3u) == 0 && (reinterpret_cast<uintptr_t>(B) & 15u) == 0 && n0 + TS <= N;
    float acc[4][4];                                            // [8-column block][fragment register]
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.0f;
    float4 ra[R], rb[R];
    const bool cs = MODE == GEMM_GRAD && colsum != nullptr && blockIdx.x == 0 && tid < (uint32_t)TS;    // thread tid sums column m0+tid
    float bsum = 0.0f;

    auto fetch = [&](uint32_t k0) {
        const bool whole = k0 + TK <= K;
#pragma unroll
        for (int r = 0; r < R; r++) {
            const uint32_t i = tid + r * NT;
            if (a_km) {
                const uint32_t k = i / Q, m = (i % Q) * 4;
                ra[r] = train_load4(A + (uint64_t)(k0 + k) * lda + m0 + m, a_al && whole, k0 + k < K, m0 + m, M);
            } else {
                const uint32_t m = i / (TK / 4), k = (i % (TK / 4)) * 4;
                ra[r] = train_load4(A + (uint64_t)(m0 + m) * lda + k0 + k, a_al && whole, m0 + m < M, k0 + k, K);
            }
            if (b_nk) {
                const uint32_t n = i / (TK / 4), k = (i % (TK / 4)) * 4;
                rb[r] = train_load4(B + (uint64_t)(n0 + n) * ldb + k0 + k, b_al && whole, n0 + n < N, k0 + k, K);
            } else {
                const uint32_t k = i / Q, n = (i % Q) * 4;
                rb[r] = train_load4(B + (uint64_t)(k0 + k) * ldb + n0 + n, b_al && whole, k0 + k < K, n0 + n, N);
            }
        }
    };
    auto stage = [&]() {
#pragma unroll
        for (int r = 0; r < R; r++) {
            const uint32_t i = tid + r * NT;
            if (a_km) {
                *reinterpret_cast<float4 *>(&As[i / Q][(i % Q) * 4]) = ra[r];
            } else {
                const uint32_t m = i / (TK / 4), k = (i % (TK / 4)) * 4;
                As[k][m] = ra[r].x; As[k + 1][m] = ra[r].y; As[k + 2][m] = ra[r].z; As[k + 3][m] = ra[r].w;
            }
            if (b_nk) {
                const uint32_t n = i / (TK / 4), k = (i % (TK / 4)) * 4;
                Bs[k][n] = rb[r].x; Bs[k + 1][n] = rb[r].y; Bs[k + 2][n] = rb[r].z; Bs[k + 3][n] = rb[r].w;
            } else {
                *reinterpret_cast<float4 *>(&Bs[i / Q][(i % Q) * 4]) = rb[r];
            }
        }
    };

    fetch(slice * TK);
    for (uint32_t kb = 0; kb < K; kb += KS * TK) {
        stage();
        __syncthreads();
        if (kb + KS * TK < K) fetch(kb + (KS + slice) * TK);
#pragma unroll
        for (int ks = 0; ks < TK; ks += 8) {
            uint32_t ah[4], al[4];
            tf32_split(As[ks + t][mh * 16 + g], ah[0], al[0]);
            tf32_split(As[ks + t][mh * 16 + g + 8], ah[1], al[1]);
            tf32_split(As[ks + t + 4][mh * 16 + g], ah[2], al[2]);
            tf32_split(As[ks + t + 4][mh * 16 + g + 8], ah[3], al[3]);
#pragma unroll
            for (int nb = 0; nb < 4; nb++) {
                uint32_t bh0, bl0, bh1, bl1;
                tf32_split(Bs[ks + t][nb * 8 + g], bh0, bl0);
                tf32_split(Bs[ks + t + 4][nb * 8 + g], bh1, bl1);
                mma_tf32(acc[nb], al, bh0, bh1);
                mma_tf32(acc[nb], ah, bl0, bl1);
                mma_tf32(acc[nb], ah, bh0, bh1);
            }
        }
        if (cs) {
#pragma unroll
            for (int k = 0; k < TK; k++) bsum += As[k][tid];
        }
        __syncthreads();
    }
    {
        float *red = &sm[0][0][0][0];
        if (slice > 0) {
#pragma unroll
            for (int i = 0; i < 16; i++) red[(slice - 1) * (NT * 16 + TS) + i * NT + tid] = acc[i >> 2][i & 3];
            if (cs) red[(slice - 1) * (NT * 16 + TS) + NT * 16 + tid] = bsum;
        }
        __syncthreads();
        if (slice > 0) return;
        for (int sl = 0; sl < KS - 1; sl++) {
#pragma unroll
            for (int i = 0; i < 16; i++) acc[i >> 2][i & 3] += red[sl * (NT * 16 + TS) + i * NT + tid];
            if (cs) bsum += red[sl * (NT * 16 + TS) + NT * 16 + tid];
        }
    }
    if (cs && m0 + tid < M) colsum[m0 + tid] = alpha * bsum;
#pragma unroll
    for (int nb = 0; nb < 4; nb++) {
#pragma unroll
        for (int c = 0; c < 4; c++) {
            const uint32_t m = m0 + mh * 16 + g + (c >> 1) * 8, n = n0 + nb * 8 + 2 * t + (c & 1);
            if (m >= M || n >= N) continue;
            float v = acc[nb][c];
            if (MODE == GEMM_FWD) v = spg_activate(v + bias[n], act);
            else if (MODE == GEMM_DELTA) v *= spg_derivative(aux[(uint64_t)m * ldaux + n], act);
            else v *= alpha;
            C[(uint64_t)m * ldc + n] = v;
        }
    }
}

// Forward product of a narrow layer (N <= 16 outputs, e.g. the class scores): one warp per row of A, the lanes striding
// over k, every lane keeping N partial sums that a shuffle tree adds at the end.  The N rows of B are read by every warp
// and stay in L1.  C[m][n] = act(sum_k A[m][k] B[n][k] + bias[n]).
// FUSE 1 / 2 make it the whole output end of a training step in one launch: the row's softmax (1) or sigmoid (2) is formed
// in the warp, C gets the activation, delta[m][n] = C[m][n] - T[m][n], and the row's cross-entropy is added to *loss when
// loss is not null (same formulas as spg_softmax_rows_kernel and spg_ce_delta_kernel).
template <bool VEC, int FUSE>
__global__ void __launch_bounds__(256)
spg_train_fwd_narrow_kernel(const float *__restrict__ A, uint32_t lda, const float *__restrict__ B, uint32_t ldb,
                            float *__restrict__ C, uint32_t ldc, uint32_t M, uint32_t N, uint32_t K,
                            const float *__restrict__ bias, int act, const float *__restrict__ T, float *__restrict__ delta,
                            float *loss)
{
    const uint32_t lane = threadIdx.x & 31u, m = blockIdx.x * 8u + (threadIdx.x >> 5);
    if (m >= M) return;
    const float *a = A + (uint64_t)m * lda;
    float acc[16];
#pragma unroll
    for (int n = 0; n < 16; n++) acc[n] = 0.0f;
    if (VEC) {
        for (uint32_t k = lane * 4u; k < K; k += 128u) {
            const float4 av = *reinterpret_cast<const float4 *>(a + k);
#pragma unroll
            for (int n = 0; n < 16; n++) {
                if ((uint32_t)n < N) {
                    const float4 bv = __ldg(reinterpret_cast<const float4 *>(B + (uint64_t)n * ldb + k));
                    acc[n] = fmaf(av.x, bv.x, fmaf(av.y, bv.y, fmaf(av.z, bv.z, fmaf(av.w, bv.w, acc[n]))));
                }
            }
        }
    } else {
        for (uint32_t k = lane; k < K; k += 32u) {
            const float av = a[k];
#pragma unroll
            for (int n = 0; n < 16; n++)
                if ((uint32_t)n < N) acc[n] = fmaf(av, __ldg(B + (uint64_t)n * ldb + k), acc[n]);
        }
    }
#pragma unroll
    for (int n = 0; n < 16; n++) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc[n] += __shfl_xor_sync(0xffffffffu, acc[n], o);
    }
    float v = 0.0f;
#pragma unroll
    for (int n = 0; n < 16; n++)
        if (lane == (uint32_t)n) v = acc[n];
    const bool mine = lane < N;
    const float z = mine ? v + bias[lane] : 0.0f;
    if (FUSE == 0) {
        if (mine) C[(uint64_t)m * ldc + lane] = spg_activate(z, act);
        return;
    }
    float o;
    if (FUSE == 1) {
        const float mx = spg_warp_max(mine ? z : -FLT_MAX);
        const float e = mine ? expf(z - mx) : 0.0f;
        const float sum = spg_warp_sum(e);
        o = sum > 0.0f ? e * (1.0f / sum) : e;
    } else {
        o = spg_activate(z, SPG_ACT_SIGMOID);
    }
    float local = 0.0f;
    if (mine) {
        const float tg = T[(uint64_t)m * N + lane];
        C[(uint64_t)m * ldc + lane] = o;
        delta[(uint64_t)m * N + lane] = o - tg;
        if (loss) {
            if (FUSE == 2) {
                const float c = fminf(fmaxf(o, 1e-9f), 1.0f - 1e-9f);
                local = -(tg * logf(c) + (1.0f - tg) * logf(1.0f - c));
            } else {
                local = -tg * logf(fmaxf(o, 1e-9f));
            }
        }
    }
    if (loss) {
        local = spg_warp_sum(local);
        if (lane == 0) atomicAdd(loss, local);
    }
}

// delta = a - t over `count` elements; optionally adds the cross-entropy of each row to *loss
// (softmax output: -sum t*log(max(o,1e-9)); sigmoid output: the two-sided form, SIMD.c:533-549).
__global__ void __launch_bounds__(256)
spg_ce_delta_kernel(const float *__restrict__ a, const float *__restrict__ t, float *__restrict__ delta,
                    uint64_t count, float *loss, int sigmoid_output)
{
    float local = 0.0f;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (uint64_t)gridDim.x * blockDim.x) {
        const float o = a[i], tg = t[i];
        delta[i] = o - tg;
        if (loss) {
            if (sigmoid_output) {
                float c = fminf(fmaxf(o, 1e-9f), 1.0f - 1e-9f);
                local -= tg * logf(c) + (1.0f - tg) * logf(1.0f - c);
            } else {
                local -= tg * logf(fmaxf(o, 1e-9f));
            }
        }
    }
    if (loss) {
        local = spg_warp_sum(local);
        if ((threadIdx.x & 31u) == 0) atomicAdd(loss, local);
    }
}

// out[j] = scale * sum over rows of d[row][j]  (bias gradient, Training.c:413-417)
__global__ void __launch_bounds__(256)
spg_col_sums_kernel(const float *__restrict__ d, uint32_t rows, uint32_t cols, float scale, float *__restrict__ out)
{
    const uint32_t j = blockIdx.x * 32 + (threadIdx.x & 31u), part = threadIdx.x >> 5;
    __shared__ float red[8][33];
    float s = 0.0f;
    if (j < cols)
        for (uint32_t r = part; r < rows; r += 8) s += d[(uint64_t)r * cols + j];
    red[part][threadIdx.x & 31u] = s;
    __syncthreads();
    if (part == 0 && j < cols) {
        float tsum = 0.0f;
#pragma unroll
        for (int q = 0; q < 8; q++) tsum += red[q][threadIdx.x];
        out[j] = scale * tsum;
    }
}

// gather rows: dst[i][:] = src[idx[i]][:]
__global__ void __launch_bounds__(256)
spg_gather_rows_kernel(const float *__restrict__ src, const uint32_t *__restrict__ idx, float *__restrict__ dst,
                       uint32_t rows, uint32_t width, const uint32_t *__restrict__ limit)
{
    spg_grid_trigger();
    spg_grid_wait();
    rows = spg_limit_rows(rows, limit);
    const uint64_t total = (uint64_t)rows * width;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t r = (uint32_t)(i / width), c = (uint32_t)(i % width);
        dst[i] = src[(uint64_t)idx[r] * width + c];
    }
}

// What changes from one optimiser step to the next, kept on the device so that a step's launches have the same
// arguments every time and can be replayed as a CUDA graph: the position in the epoch (first row of the step in the
// shuffled order) and Adam's running powers of beta1 / beta2 with the bias corrections made of them.  The host
// computes the same values with the same fp32 operations (Training.c:480-500), so both ways give the same bits.
struct SpgStepState { uint32_t step, start; float b1pow, b2pow, mf, vf; };

// first launch of a step: this step's values, then the position moves on
__global__ void spg_train_state_kernel(SpgStepState *st, uint32_t steps_per_epoch, uint32_t batch, float b1, float b2)
{
    st->start = st->step * batch;
    st->step = st->step + 1 == steps_per_epoch ? 0u : st->step + 1;
    st->b1pow *= b1;
    st->b2pow *= b2;
    st->mf = 1.0f / (1.0f - st->b1pow);
    st->vf = 1.0f / (1.0f - st->b2pow);
}

struct SpgGraph { cudaGraphExec_t exec; uint32_t nodes; };

// the device step state that the launchers below hand to their kernels (NULL: arguments come from the host)
thread_local const SpgStepState *tls_step_state = nullptr;

// gather the same rows of two tables (a mini-batch's inputs and targets) in one launch
__global__ void __launch_bounds__(256)
spg_gather_rows2_kernel(const float *__restrict__ src_a, uint32_t wa, float *__restrict__ dst_a, const float *__restrict__ src_b,
                        uint32_t wb, float *__restrict__ dst_b, const uint32_t *__restrict__ idx, uint32_t rows,
                        const SpgStepState *__restrict__ state)
{
    if (state) idx += state->start;                    // the step's first row of the shuffled order, kept on the device
    const uint32_t w = wa + wb;
    const uint64_t total = (uint64_t)rows * w;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t r = (uint32_t)(i / w), c = (uint32_t)(i % w);
        const uint64_t from = idx[r];
        if (c < wa) dst_a[(uint64_t)r * wa + c] = src_a[from * wa + c];
        else dst_b[(uint64_t)r * wb + (c - wa)] = src_b[from * wb + (c - wa)];
    }
}

// Fused Adam over one flat buffer (weights and biases of every layer laid end to end).  The gradient
// is first scaled by gscale (1/ranks after a sum all-reduce).  Same operation order as the reference:
// m = b1*m + (1-b1)*g ; v = b2*v + (1-b2)*g*g ; w -= lr * (m*mf) / sqrt(v*vf + eps).
__global__ void __launch_bounds__(256)
spg_adam_kernel(float *__restrict__ w, float *__restrict__ m, float *__restrict__ v, const float *__restrict__ g, uint64_t n,
                float lr, float b1, float b2, float mf, float vf, float eps, float gscale, const SpgStepState *__restrict__ state)
{
    if (state) { mf = state->mf; vf = state->vf; }     // bias corrections of this step, advanced on the device
    const float omb1 = 1.0f - b1, omb2 = 1.0f - b2;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        const float gi = g[i] * gscale;
        const float mi = fmaf(b1, m[i], omb1 * gi);
        const float vi = fmaf(b2, v[i], omb2 * (gi * gi));
        m[i] = mi;
        v[i] = vi;
        w[i] -= lr * ((mi * mf) / sqrtf(vi * vf + eps));
    }
}


// Output-layer delta for the combinations cross-entropy does not cover (reference Training.c:357-376), one warp per row:
//   mse_softmax: delta_j = a_j * ((a_j - t_j) - sum_k (a_k - t_k) a_k)          (Training.c:357-367)
//   otherwise:   delta_j = (a_j - t_j) * act'(a_j)                              (Training.c:373-375)
// and, when loss is not null, the batch's summed loss: squared error (loss_ce == 0, SIMD.c:527-531) or cross-entropy
// -sum t*log(max(a, 1e-9)) (loss_ce != 0 with an output activation other than softmax / sigmoid, SIMD.c:543-548).
__global__ void __launch_bounds__(256)
spg_output_delta_kernel(const float *__restrict__ a, const float *__restrict__ t, float *__restrict__ delta,
                        uint32_t rows, uint32_t width, int act, int mse_softmax, int loss_ce, float *loss)
{
    const uint32_t lane = threadIdx.x & 31u;
    float local = 0.0f;
    for (uint32_t r = blockIdx.x * 8u + (threadIdx.x >> 5); r < rows; r += gridDim.x * 8u) {
        const float *ar = a + (uint64_t)r * width, *tr = t + (uint64_t)r * width;
        float *dr = delta + (uint64_t)r * width;
        float sum = 0.0f;
        if (mse_softmax) {
            for (uint32_t j = lane; j < width; j += 32u) sum += (ar[j] - tr[j]) * ar[j];
            sum = spg_warp_sum(sum);
        }
        for (uint32_t j = lane; j < width; j += 32u) {
            const float diff = ar[j] - tr[j];
            dr[j] = mse_softmax ? ar[j] * (diff - sum) : diff * spg_derivative(ar[j], act);
            if (loss) local += loss_ce ? -tr[j] * logf(fmaxf(ar[j], 1e-9f)) : diff * diff;
        }
    }
    if (loss) {
        local = spg_warp_sum(local);
        if (lane == 0 && local != 0.0f) atomicAdd(loss, local);
    }
}

// sum of squares of a flat buffer (for the global gradient norm, SIMD.c:496-507), added to *out
__global__ void __launch_bounds__(256)
spg_sumsq_kernel(const float *__restrict__ g, uint64_t n, float *out)
{
    float local = 0.0f;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) local = fmaf(g[i], g[i], local);
    local = spg_warp_sum(local);
    __shared__ float part[8];
    if ((threadIdx.x & 31u) == 0) part[threadIdx.x >> 5] = local;
    __syncthreads();
    if (threadIdx.x == 0) {
        float s = 0.0f;
        for (int i = 0; i < 8; i++) s += part[i];
        atomicAdd(out, s);
    }
}

// One fused pass of any of the reference's update rules over the flat parameter buffer [weights | biases]
// (Training.c:439-507, SIMD.c:279-494).  The first n_w elements are weights (weight decay applies to them only),
// the rest biases.  g is scaled first by gscale (1/ranks after a sum exchange) and, when sumsq is given, by the
// global-norm clip factor max_norm / norm if norm > max_norm (SIMD.c:509-518; *sumsq holds the sum of squares of
// the UNSCALED buffer).
//   kind 0 SGD:      w -= lr * (g + decay*w)
//   kind 1 MOMENTUM: m = mom*m + decay*w + g ; w -= lr*m
//   kind 2 RMSPROP:  v = b2*v + (1-b2)*g*g ; w -= lr * (decay*w + g / sqrt(v + eps))
//   kind 3 ADAM:     g += decay*w (weights) ; m, v as Adam ; w -= lr * (m*mf) / sqrt(v*vf + eps)
//   kind 4 ADAMW:    m, v as Adam ; w = w*(1 - lr*decay) - lr * (m*mf) / sqrt(v*vf + eps)
__global__ void __launch_bounds__(256)
spg_optimizer_kernel(int kind, float *__restrict__ w, float *__restrict__ m, float *__restrict__ v, const float *__restrict__ g,
                     uint64_t n, uint64_t n_w, float lr, float momentum, float b1, float b2, float mf, float vf, float eps,
                     float decay, float gscale, const float *sumsq, float max_norm, const SpgStepState *__restrict__ state)
{
    if (state) { mf = state->mf; vf = state->vf; }
    float gs = gscale;
    if (sumsq) {
        const float norm = sqrtf(*sumsq) * gscale;
        if (norm > max_norm) gs *= max_norm / norm;
    }
    const float omb1 = 1.0f - b1, omb2 = 1.0f - b2;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        const float d = i < n_w ? decay : 0.0f;
        float gi = g[i] * gs, wi = w[i];
        switch (kind) {
            case 0: wi -= lr * fmaf(d, wi, gi); break;
            case 1: { const float mi = fmaf(momentum, m[i], fmaf(d, wi, gi)); m[i] = mi; wi -= lr * mi; break; }
            case 2: { const float vi = fmaf(b2, v[i], omb2 * (gi * gi)); v[i] = vi; wi -= lr * fmaf(d, wi, gi / sqrtf(vi + eps)); break; }
            default: {
                if (kind == 3) gi = fmaf(d, wi, gi);
                const float mi = fmaf(b1, m[i], omb1 * gi);
                const float vi = fmaf(b2, v[i], omb2 * (gi * gi));
                m[i] = mi; v[i] = vi;
                const float step = lr * ((mi * mf) / sqrtf(vi * vf + eps));
                wi = kind == 4 && d > 0.0f ? wi * (1.0f - lr * d) - step : wi - step;
            }
        }
        w[i] = wi;
    }
}

__global__ void __launch_bounds__(256)
spg_nonfinite_kernel(const float *__restrict__ w, uint64_t n, int *flag)
{
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x)
        if (!isfinite(w[i])) *flag = 1;
}

uint32_t blocks_for(uint64_t n) { uint64_t b = (n + 255) / 256; return (uint32_t)(b < 148ull * 8 ? (b ? b : 1) : 148ull * 8); }

// ---- NCCL through dlopen: the library has no link-time dependency on it ----------
typedef struct { char internal[128]; } nccl_uid;
typedef void *nccl_comm;
struct NcclApi {
    void *handle;
    int (*GetUniqueId)(nccl_uid *);
    int (*CommInitRank)(nccl_comm *, int, nccl_uid, int);
    int (*AllReduce)(const void *, void *, size_t, int, int, nccl_comm, cudaStream_t);
    int (*CommDestroy)(nccl_comm);
    int (*CommAbort)(nccl_comm);
    int (*GroupStart)(void);
    int (*GroupEnd)(void);
    const char *(*GetErrorString)(int);
};
NcclApi g_nccl;

int nccl_load()
{
    if (g_nccl.handle) return SPGK_OK;
    const char *names[] = { "libnccl.so.2", "libnccl.so" };
    void *h = nullptr;
    for (const char *n : names) { h = dlopen(n, RTLD_NOW | RTLD_GLOBAL); if (h) break; }
    if (!h) { spgk_set_error("dlopen(libnccl.so.2)", dlerror()); return SPGK_E_CUDA; }
    g_nccl.GetUniqueId = (int (*)(nccl_uid *))dlsym(h, "ncclGetUniqueId");
    g_nccl.CommInitRank = (int (*)(nccl_comm *, int, nccl_uid, int))dlsym(h, "ncclCommInitRank");
    g_nccl.AllReduce = (int (*)(const void *, void *, size_t, int, int, nccl_comm, cudaStream_t))dlsym(h, "ncclAllReduce");
    g_nccl.CommDestroy = (int (*)(nccl_comm))dlsym(h, "ncclCommDestroy");
    g_nccl.CommAbort = (int (*)(nccl_comm))dlsym(h, "ncclCommAbort");
    g_nccl.GetErrorString = (const char *(*)(int))dlsym(h, "ncclGetErrorString");
    g_nccl.GroupStart = (int (*)(void))dlsym(h, "ncclGroupStart");
    g_nccl.GroupEnd = (int (*)(void))dlsym(h, "ncclGroupEnd");
    if (!g_nccl.GetUniqueId || !g_nccl.CommInitRank || !g_nccl.AllReduce || !g_nccl.CommDestroy || !g_nccl.GroupStart || !g_nccl.GroupEnd) {
        spgk_set_error("libnccl", "missing symbols");
        return SPGK_E_CUDA;
    }
    g_nccl.handle = h;
    return SPGK_OK;
}

int nccl_check(int rc, const char *what)
{
    if (rc == 0) return SPGK_OK;
    spgk_set_error(what, g_nccl.GetErrorString ? g_nccl.GetErrorString(rc) : "NCCL error");
    return SPGK_E_CUDA;
}

}  // namespace

extern "C" {

static int train_gemm(int mode, const float *A, uint32_t lda, const float *B, uint32_t ldb, float *C, uint32_t ldc,
                      uint32_t M, uint32_t N, uint32_t K, float alpha, const float *bias, const float *aux, uint32_t ldaux,
                      int act, float *colsum, void *stream)
{
    if (!A || !B || !C || M == 0 || N == 0 || K == 0 || (mode == GEMM_FWD && !bias) || (mode == GEMM_DELTA && !aux)) {
        spgk_set_error("spgk_train_gemm", "bad argument");
        return SPGK_E_ARG;
    }
    cudaStream_t s = (cudaStream_t)stream;
    if (act == SPG_ACT_SOFTMAX && mode == GEMM_FWD) act = SPG_ACT_NONE;      // softmax rows are finished separately
    if (mode != GEMM_FWD && mode != GEMM_DELTA && mode != GEMM_GRAD) { spgk_set_error("spgk_train_gemm", "unknown mode"); return SPGK_E_ARG; }
    if (mode == GEMM_FWD && N <= 16u) {
        const bool vec = (K & 3u) == 0 && (lda & 3u) == 0 && (ldb & 3u) == 0 &&
                         ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B)) & 15u) == 0;
        if (vec) spg_train_fwd_narrow_kernel<true, 0><<<(M + 7) / 8, 256, 0, s>>>(A, lda, B, ldb, C, ldc, M, N, K, bias, act, nullptr, nullptr, nullptr);
        else spg_train_fwd_narrow_kernel<false, 0><<<(M + 7) / 8, 256, 0, s>>>(A, lda, B, ldb, C, ldc, M, N, K, bias, act, nullptr, nullptr, nullptr);
        return spgk_check_launch("spg_train_fwd_narrow_kernel");
    }
    // Products of at least 148 64 x 64 tiles: the SIMT kernel with that tile.  Smaller ones - on a 256-row step of a
    // 784-512-1000-10 network that is every product - take 32 x 32 tiles on the tensor cores with the k range of a tile
    // split over four two-warp slices of the CTA, eight when there are at most 32 tiles.
    const uint32_t tiles64 = ((N + 63) / 64) * ((M + 63) / 64), tiles32 = ((N + 31) / 32) * ((M + 31) / 32);
    const int shape = tiles64 >= 148u ? 0 : tiles32 > 32u ? 1 : 2;
#define SPG_TRAIN_ARGS A, lda, B, ldb, C, ldc, M, N, K, alpha, bias, aux, ldaux, act, colsum
#define SPG_TRAIN_SHAPES(MODEV) \
    do { const dim3 g32((N + 31) / 32, (M + 31) / 32); \
         if (shape == 0) spg_train_gemm_kernel<MODEV, 64, 1><<<dim3((N + 63) / 64, (M + 63) / 64), 256, 0, s>>>(SPG_TRAIN_ARGS); \
         else if (shape == 1) spg_train_mma_kernel<MODEV, 4><<<g32, 256, 0, s>>>(SPG_TRAIN_ARGS); \
         else spg_train_mma_kernel<MODEV, 8><<<g32, 512, 0, s>>>(SPG_TRAIN_ARGS); } while (0)
    if (mode == GEMM_FWD) SPG_TRAIN_SHAPES(GEMM_FWD);
    else if (mode == GEMM_DELTA) SPG_TRAIN_SHAPES(GEMM_DELTA);
    else SPG_TRAIN_SHAPES(GEMM_GRAD);
#undef SPG_TRAIN_SHAPES
#undef SPG_TRAIN_ARGS
    return spgk_check_launch("spg_train_gemm_kernel");
}

int spgk_train_gemm(int mode, const float *A, uint32_t lda, const float *B, uint32_t ldb, float *C, uint32_t ldc,
                    uint32_t M, uint32_t N, uint32_t K, float alpha, const float *bias, const float *aux, uint32_t ldaux,
                    int act, void *stream)
{
    return train_gemm(mode, A, lda, B, ldb, C, ldc, M, N, K, alpha, bias, aux, ldaux, act, nullptr, stream);
}

int spgk_train_grad(const float *delta, uint32_t ldd, const float *a, uint32_t lda, float *gw, uint32_t ldg, float *gb,
                    uint32_t out, uint32_t in, uint32_t rows, float scale, void *stream)
{
    if (!gb) { spgk_set_error("spgk_train_grad", "bad argument"); return SPGK_E_ARG; }
    return train_gemm(GEMM_GRAD, delta, ldd, a, lda, gw, ldg, out, in, rows, scale, nullptr, nullptr, 0, 0, gb, stream);
}

int spgk_train_output(const float *x, uint32_t ldx, const float *w, uint32_t ldw, const float *bias, float *y, const float *t,
                      float *delta, float *loss, uint32_t rows, uint32_t out, uint32_t in, int sigmoid_output, void *stream)
{
    if (!x || !w || !bias || !y || !t || !delta || rows == 0 || in == 0 || out == 0 || out > 16u) {
        spgk_set_error("spgk_train_output", "bad argument");
        return SPGK_E_ARG;
    }
    cudaStream_t s = (cudaStream_t)stream;
    const bool vec = (in & 3u) == 0 && (ldx & 3u) == 0 && (ldw & 3u) == 0 &&
                     ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15u) == 0;
    const dim3 grid((rows + 7) / 8);
#define SPG_OUT_LAUNCH(VECV, FUSEV) \
    spg_train_fwd_narrow_kernel<VECV, FUSEV><<<grid, 256, 0, s>>>(x, ldx, w, ldw, y, out, rows, out, in, bias, 0, t, delta, loss)
    if (sigmoid_output) { if (vec) SPG_OUT_LAUNCH(true, 2); else SPG_OUT_LAUNCH(false, 2); }
    else { if (vec) SPG_OUT_LAUNCH(true, 1); else SPG_OUT_LAUNCH(false, 1); }
#undef SPG_OUT_LAUNCH
    return spgk_check_launch("spg_train_fwd_narrow_kernel");
}

// ---- device step state and graph replay of a training step --------------------------------------------------------------
size_t spgk_train_state_bytes(void) { return sizeof(SpgStepState); }

// starts a run of steps: position 0, beta powers 1 (Training.c:480-500 starts them there at every train() call)
int spgk_train_state_reset(void *state, void *stream)
{
    if (!state) { spgk_set_error("spgk_train_state_reset", "bad argument"); return SPGK_E_ARG; }
    const SpgStepState init = { 0u, 0u, 1.0f, 1.0f, 0.0f, 0.0f };
    SPGK_CUDA(cudaMemcpyAsync(state, &init, sizeof init, cudaMemcpyHostToDevice, (cudaStream_t)stream));
    SPGK_CUDA(cudaStreamSynchronize((cudaStream_t)stream));      // `init` is on this stack
    return SPGK_OK;
}

// first launch of a step: sets the step's first row and bias corrections in `state` and moves the position on
int spgk_train_state_step(void *state, uint32_t steps_per_epoch, uint32_t batch, float b1, float b2, void *stream)
{
    if (!state || steps_per_epoch == 0) { spgk_set_error("spgk_train_state_step", "bad argument"); return SPGK_E_ARG; }
    spg_train_state_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(static_cast<SpgStepState *>(state), steps_per_epoch, batch, b1, b2);
    return spgk_check_launch("spg_train_state_kernel");
}

// from now on spgk_gather_rows2 (row offset), spgk_adam and spgk_optimizer_step (bias corrections) of this thread take
// those values from `state` instead of their arguments; NULL switches back
void spgk_train_use_state(const void *state) { tls_step_state = static_cast<const SpgStepState *>(state); }

// Stream capture of a step's launches into a graph, and its replay.  begin .. end must enclose only launches and
// memsets on `stream`; end returns the executable graph (NULL and an error code if the capture did not come off).
int spgk_graph_begin(void *stream)
{
    SPGK_CUDA(cudaStreamBeginCapture((cudaStream_t)stream, cudaStreamCaptureModeRelaxed));
    return SPGK_OK;
}
int spgk_graph_end(void *stream, void **exec_out)
{
    if (!exec_out) return SPGK_E_ARG;
    *exec_out = nullptr;
    cudaGraph_t g = nullptr;
    cudaError_t e = cudaStreamEndCapture((cudaStream_t)stream, &g);
    if (e != cudaSuccess || !g) { spgk_set_error("cudaStreamEndCapture", cudaGetErrorString(e)); cudaGetLastError(); return SPGK_E_CUDA; }
    size_t nodes = 0;
    cudaGraphGetNodes(g, nullptr, &nodes);
    cudaGraphExec_t x = nullptr;
    e = cudaGraphInstantiate(&x, g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) { spgk_set_error("cudaGraphInstantiate", cudaGetErrorString(e)); cudaGetLastError(); return SPGK_E_CUDA; }
    *exec_out = new SpgGraph{ x, (uint32_t)nodes };
    return SPGK_OK;
}
int spgk_graph_launch(void *exec, void *stream)
{
    SpgGraph *gr = static_cast<SpgGraph *>(exec);
    if (!gr) return SPGK_E_ARG;
    SPGK_CUDA(cudaGraphLaunch(gr->exec, (cudaStream_t)stream));
    for (uint32_t i = 0; i < gr->nodes; i++) spgk_count_launch();      // the launch counter counts kernels, replayed or not
    return SPGK_OK;
}
void spgk_graph_destroy(void *exec)
{
    SpgGraph *gr = static_cast<SpgGraph *>(exec);
    if (!gr) return;
    cudaGraphExecDestroy(gr->exec);
    delete gr;
}

int spgk_gather_rows2(const float *src_a, uint32_t width_a, float *dst_a, const float *src_b, uint32_t width_b, float *dst_b,
                      const uint32_t *idx, uint32_t rows, void *stream)
{
    if (!src_a || !dst_a || !src_b || !dst_b || !idx) { spgk_set_error("spgk_gather_rows2", "bad argument"); return SPGK_E_ARG; }
    if (rows == 0 || width_a + width_b == 0) return SPGK_OK;
    spg_gather_rows2_kernel<<<blocks_for((uint64_t)rows * (width_a + width_b)), 256, 0, (cudaStream_t)stream>>>(
        src_a, width_a, dst_a, src_b, width_b, dst_b, idx, rows, tls_step_state);
    return spgk_check_launch("spg_gather_rows2_kernel");
}

int spgk_ce_delta(const float *a, const float *t, float *delta, uint64_t count, float *loss, int sigmoid_output, void *stream)
{
    if (!a || !t || !delta) { spgk_set_error("spgk_ce_delta", "bad argument"); return SPGK_E_ARG; }
    if (count == 0) return SPGK_OK;
    spg_ce_delta_kernel<<<blocks_for(count), 256, 0, (cudaStream_t)stream>>>(a, t, delta, count, loss, sigmoid_output);
    return spgk_check_launch("spg_ce_delta_kernel");
}

int spgk_col_sums(const float *d, uint32_t rows, uint32_t cols, float scale, float *out, void *stream)
{
    if (!d || !out || cols == 0) { spgk_set_error("spgk_col_sums", "bad argument"); return SPGK_E_ARG; }
    spg_col_sums_kernel<<<(cols + 31) / 32, 256, 0, (cudaStream_t)stream>>>(d, rows, cols, scale, out);
    return spgk_check_launch("spg_col_sums_kernel");
}

int spgk_gather_rows(const float *src, const uint32_t *idx, float *dst, uint32_t rows, uint32_t width, void *stream)
{
    if (!src || !idx || !dst) { spgk_set_error("spgk_gather_rows", "bad argument"); return SPGK_E_ARG; }
    if (rows == 0 || width == 0) return SPGK_OK;
    SPGK_CUDA(spg_launch_chained(spg_gather_rows_kernel, dim3(blocks_for((uint64_t)rows * width)), dim3(256), 0, (cudaStream_t)stream, src, idx, dst, rows, width, spg_tls_rows_limit));
    return spgk_check_launch("spg_gather_rows_kernel");
}

int spgk_adam(float *w, float *m, float *v, const float *g, uint64_t n, float lr, float b1, float b2,
              float mf, float vf, float eps, float gscale, void *stream)
{
    if (!w || !m || !v || !g) { spgk_set_error("spgk_adam", "bad argument"); return SPGK_E_ARG; }
    if (n == 0) return SPGK_OK;
    spg_adam_kernel<<<blocks_for(n), 256, 0, (cudaStream_t)stream>>>(w, m, v, g, n, lr, b1, b2, mf, vf, eps, gscale, tls_step_state);
    return spgk_check_launch("spg_adam_kernel");
}


int spgk_output_delta(const float *a, const float *t, float *delta, uint32_t rows, uint32_t width, int act, int mse_softmax,
                      int loss_ce, float *loss, void *stream)
{
    if (!a || !t || !delta || width == 0) { spgk_set_error("spgk_output_delta", "bad argument"); return SPGK_E_ARG; }
    if (rows == 0) return SPGK_OK;
    uint32_t blocks = (rows + 7u) / 8u;
    if (blocks > 148u * 8u) blocks = 148u * 8u;
    spg_output_delta_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(a, t, delta, rows, width, act, mse_softmax, loss_ce, loss);
    return spgk_check_launch("spg_output_delta_kernel");
}

int spgk_sumsq(const float *g, uint64_t n, float *out_dev, void *stream)
{
    if (!g || !out_dev) { spgk_set_error("spgk_sumsq", "bad argument"); return SPGK_E_ARG; }
    if (n == 0) return SPGK_OK;
    spg_sumsq_kernel<<<blocks_for(n), 256, 0, (cudaStream_t)stream>>>(g, n, out_dev);
    return spgk_check_launch("spg_sumsq_kernel");
}

int spgk_optimizer_step(int kind, float *w, float *m, float *v, const float *g, uint64_t n, uint64_t n_weights,
                        float lr, float momentum, float b1, float b2, float mf, float vf, float eps, float decay,
                        float gscale, const float *sumsq_dev, float max_norm, void *stream)
{
    if (!w || !g || kind < 0 || kind > 4 || (kind != 0 && kind != 2 && !m) || (kind >= 2 && !v) || n_weights > n) {
        spgk_set_error("spgk_optimizer_step", "bad argument");
        return SPGK_E_ARG;
    }
    if (n == 0) return SPGK_OK;
    spg_optimizer_kernel<<<blocks_for(n), 256, 0, (cudaStream_t)stream>>>(kind, w, m, v, g, n, n_weights, lr, momentum, b1, b2, mf, vf,
                                                                         eps, decay, gscale, sumsq_dev, max_norm, tls_step_state);
    return spgk_check_launch("spg_optimizer_kernel");
}

int spgk_nonfinite(const float *w, uint64_t n, int *flag_dev, void *stream)
{
    if (!w || !flag_dev) { spgk_set_error("spgk_nonfinite", "bad argument"); return SPGK_E_ARG; }
    if (n == 0) return SPGK_OK;
    spg_nonfinite_kernel<<<blocks_for(n), 256, 0, (cudaStream_t)stream>>>(w, n, flag_dev);
    return spgk_check_launch("spg_nonfinite_kernel");
}

int spgk_nccl_unique_id(void *id128)
{
    int rc = nccl_load();
    if (rc) return rc;
    nccl_uid id;
    rc = nccl_check(g_nccl.GetUniqueId(&id), "ncclGetUniqueId");
    if (rc) return rc;
    memcpy(id128, &id, sizeof id);
    return SPGK_OK;
}

}  // extern "C"

namespace {

// Runs `fn` on a helper thread and waits for it at most timeout_ms.  A rendezvous that never completes (a rank that died
// before it joined) must not hold the caller for ever: on expiry the caller gets SPGK_E_TIMEOUT and carries on; the
// helper thread stays parked inside the call it cannot leave and is abandoned (it owns only its own heap block).
struct TimedCall { std::mutex m; std::condition_variable cv; bool done = false; int rc = 0; };

template <typename Fn>
int run_with_timeout(Fn fn, int timeout_ms, const char *what)
{
    auto st = std::make_shared<TimedCall>();
    std::thread([st, fn]() {
        const int rc = fn();
        std::lock_guard<std::mutex> g(st->m);
        st->rc = rc; st->done = true;
        st->cv.notify_all();
    }).detach();
    std::unique_lock<std::mutex> g(st->m);
    if (!st->cv.wait_for(g, std::chrono::milliseconds(timeout_ms), [&] { return st->done; })) {
        char msg[96];
        snprintf(msg, sizeof msg, "no answer within %d ms (a rank that never joined?)", timeout_ms);
        spgk_set_error(what, msg);
        return SPGK_E_TIMEOUT;
    }
    return st->rc;
}

int dist_timeout_ms()
{
    const char *e = getenv("SPINGALETT_DIST_TIMEOUT_MS");
    const int v = e ? atoi(e) : 0;
    return v > 0 ? v : 120000;
}

}  // namespace

extern "C" {

// Host-only check of the timeout wrapper (no NCCL, no CUDA): a call that answers after answer_ms against a limit of
// timeout_ms.  Returns what the wrapper returned (0, or SPGK_E_TIMEOUT).
int spgk_selftest_timed_call(int answer_ms, int timeout_ms)
{
    return run_with_timeout([answer_ms]() -> int { std::this_thread::sleep_for(std::chrono::milliseconds(answer_ms)); return 0; },
                            timeout_ms, "selftest");
}

int spgk_nccl_init(void **comm, int rank, int world, const void *id128)
{
    int rc = nccl_load();
    if (rc) return rc;
    nccl_uid id;
    memcpy(&id, id128, sizeof id);
    int dev = 0;
    SPGK_CUDA(cudaGetDevice(&dev));
    auto slot = std::make_shared<nccl_comm>(nullptr);
    // ncclCommInitRank blocks until every rank has arrived: bounded by SPINGALETT_DIST_TIMEOUT_MS (default 120 s)
    rc = run_with_timeout([slot, world, id, rank, dev]() -> int {
        if (cudaSetDevice(dev) != cudaSuccess) return -1;
        return g_nccl.CommInitRank(slot.get(), world, id, rank);
    }, dist_timeout_ms(), "ncclCommInitRank");
    if (rc == SPGK_E_TIMEOUT) return rc;
    if ((rc = nccl_check(rc, "ncclCommInitRank"))) return rc;
    *comm = *slot;
    return SPGK_OK;
}

// Waits for the stream at most SPINGALETT_DIST_TIMEOUT_MS (polling, no blocking call): an exchange whose peer has gone
// never finishes, and the caller then aborts the communicator instead of hanging.
int spgk_stream_sync_bounded(void *stream)
{
    const auto t0 = std::chrono::steady_clock::now();
    const int limit = dist_timeout_ms();
    for (;;) {
        const cudaError_t e = cudaStreamQuery((cudaStream_t)stream);
        if (e == cudaSuccess) return SPGK_OK;
        if (e != cudaErrorNotReady) { spgk_set_error("cudaStreamQuery", cudaGetErrorString(e)); return SPGK_E_CUDA; }
        if (std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count() > limit) {
            spgk_set_error("stream wait", "the gradient exchange did not finish in time (a rank has gone?)");
            return SPGK_E_TIMEOUT;
        }
        std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
}

int spgk_nccl_abort(void *comm)
{
    if (!comm || !g_nccl.handle || !g_nccl.CommAbort) return SPGK_OK;
    return nccl_check(g_nccl.CommAbort(comm), "ncclCommAbort");
}

int spgk_nccl_allreduce_sum(void *comm, float *buf, uint64_t count, void *stream)
{
    if (!comm || !g_nccl.handle) { spgk_set_error("spgk_nccl_allreduce_sum", "no communicator"); return SPGK_E_ARG; }
    return nccl_check(g_nccl.AllReduce(buf, buf, (size_t)count, 7 /* ncclFloat32 */, 0 /* ncclSum */, comm, (cudaStream_t)stream),
                      "ncclAllReduce");
}

int spgk_nccl_allreduce_sum2(void *comm, float *buf_a, uint64_t count_a, float *buf_b, uint64_t count_b, void *stream)
{
    if (!comm || !g_nccl.handle) { spgk_set_error("spgk_nccl_allreduce_sum2", "no communicator"); return SPGK_E_ARG; }
    int rc = nccl_check(g_nccl.GroupStart(), "ncclGroupStart");
    if (rc != SPGK_OK) return rc;
    int ra = g_nccl.AllReduce(buf_a, buf_a, (size_t)count_a, 7 /* ncclFloat32 */, 0 /* ncclSum */, comm, (cudaStream_t)stream);
    int rb = g_nccl.AllReduce(buf_b, buf_b, (size_t)count_b, 7, 0, comm, (cudaStream_t)stream);
    int re = g_nccl.GroupEnd();                     // always closed, so that a failed call does not leave the group open
    if ((rc = nccl_check(ra, "ncclAllReduce")) != SPGK_OK || (rc = nccl_check(rb, "ncclAllReduce")) != SPGK_OK) return rc;
    return nccl_check(re, "ncclGroupEnd");
}

int spgk_nccl_destroy(void *comm)
{
    if (!comm || !g_nccl.handle) return SPGK_OK;
    return nccl_check(g_nccl.CommDestroy(comm), "ncclCommDestroy");
}

}  // extern "C"
