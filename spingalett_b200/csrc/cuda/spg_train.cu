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
#include <cstdio>
#include <cstring>

namespace {

constexpr int TM = 64, TN = 64, TK = 16;      // CTA tile; 256 threads, 4x4 outputs each

enum { GEMM_FWD = 0, GEMM_DELTA = 1, GEMM_GRAD = 2 };

// MODE 0: C[M][N] = act(A[M][K] . B[N][K]^T + bias[N])        (A = activations, B = weights [out][in])
// MODE 1: C[M][N] = (A[M][K] . B[K][N]) * act'(aux[M][N])      (A = delta_{l+1}, B = weights [next][cur])
// MODE 2: C[M][N] = alpha * A[K][M]^T . B[K][N]                 (A = delta [rows][out], B = activations [rows][in])
template <int MODE>
__global__ void __launch_bounds__(256)
spg_train_gemm_kernel(const float *__restrict__ A, uint32_t lda, const float *__restrict__ B, uint32_t ldb,
                      float *__restrict__ C, uint32_t ldc, uint32_t M, uint32_t N, uint32_t K,
                      float alpha, const float *__restrict__ bias, const float *__restrict__ aux, uint32_t ldaux, int act)
{
    __shared__ float As[TK][TM + 4];
    __shared__ float Bs[TK][TN + 4];
    const uint32_t tid = threadIdx.x, tx = tid & 15u, ty = tid >> 4;
    const uint32_t m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.0f;

    for (uint32_t k0 = 0; k0 < K; k0 += TK) {
        // stage A tile as As[k][m] and B tile as Bs[k][n]
        for (uint32_t i = tid; i < TM * TK; i += 256) {
            uint32_t m, k;
            float v = 0.0f;
            if (MODE == GEMM_GRAD) { m = i % TM; k = i / TM; if (m0 + m < M && k0 + k < K) v = A[(uint64_t)(k0 + k) * lda + m0 + m]; }
            else { k = i % TK; m = i / TK; if (m0 + m < M && k0 + k < K) v = A[(uint64_t)(m0 + m) * lda + k0 + k]; }
            As[k][m] = v;
        }
        for (uint32_t i = tid; i < TN * TK; i += 256) {
            uint32_t n, k;
            float v = 0.0f;
            if (MODE == GEMM_FWD) { k = i % TK; n = i / TK; if (n0 + n < N && k0 + k < K) v = B[(uint64_t)(n0 + n) * ldb + k0 + k]; }
            else { n = i % TN; k = i / TN; if (n0 + n < N && k0 + k < K) v = B[(uint64_t)(k0 + k) * ldb + n0 + n]; }
            Bs[k][n] = v;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < TK; k++) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; i++) a[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; j++) b[j] = Bs[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
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

// Fused Adam over one flat buffer (weights and biases of every layer laid end to end).  The gradient
// is first scaled by gscale (1/ranks after a sum all-reduce).  Same operation order as the reference:
// m = b1*m + (1-b1)*g ; v = b2*v + (1-b2)*g*g ; w -= lr * (m*mf) / sqrt(v*vf + eps).
__global__ void __launch_bounds__(256)
spg_adam_kernel(float *__restrict__ w, float *__restrict__ m, float *__restrict__ v, const float *__restrict__ g, uint64_t n,
                float lr, float b1, float b2, float mf, float vf, float eps, float gscale)
{
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
    g_nccl.GetErrorString = (const char *(*)(int))dlsym(h, "ncclGetErrorString");
    if (!g_nccl.GetUniqueId || !g_nccl.CommInitRank || !g_nccl.AllReduce || !g_nccl.CommDestroy) {
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

int spgk_train_gemm(int mode, const float *A, uint32_t lda, const float *B, uint32_t ldb, float *C, uint32_t ldc,
                    uint32_t M, uint32_t N, uint32_t K, float alpha, const float *bias, const float *aux, uint32_t ldaux,
                    int act, void *stream)
{
    if (!A || !B || !C || M == 0 || N == 0 || K == 0 || (mode == GEMM_FWD && !bias) || (mode == GEMM_DELTA && !aux)) {
        spgk_set_error("spgk_train_gemm", "bad argument");
        return SPGK_E_ARG;
    }
    dim3 grid((N + TN - 1) / TN, (M + TM - 1) / TM);
    cudaStream_t s = (cudaStream_t)stream;
    if (act == SPG_ACT_SOFTMAX && mode == GEMM_FWD) act = SPG_ACT_NONE;      // softmax rows are finished separately
    if (mode == GEMM_FWD) spg_train_gemm_kernel<GEMM_FWD><<<grid, 256, 0, s>>>(A, lda, B, ldb, C, ldc, M, N, K, alpha, bias, aux, ldaux, act);
    else if (mode == GEMM_DELTA) spg_train_gemm_kernel<GEMM_DELTA><<<grid, 256, 0, s>>>(A, lda, B, ldb, C, ldc, M, N, K, alpha, bias, aux, ldaux, act);
    else if (mode == GEMM_GRAD) spg_train_gemm_kernel<GEMM_GRAD><<<grid, 256, 0, s>>>(A, lda, B, ldb, C, ldc, M, N, K, alpha, bias, aux, ldaux, act);
    else { spgk_set_error("spgk_train_gemm", "unknown mode"); return SPGK_E_ARG; }
    return spgk_check_launch("spg_train_gemm_kernel");
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
    spg_adam_kernel<<<blocks_for(n), 256, 0, (cudaStream_t)stream>>>(w, m, v, g, n, lr, b1, b2, mf, vf, eps, gscale);
    return spgk_check_launch("spg_adam_kernel");
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

int spgk_nccl_init(void **comm, int rank, int world, const void *id128)
{
    int rc = nccl_load();
    if (rc) return rc;
    nccl_uid id;
    memcpy(&id, id128, sizeof id);
    nccl_comm c = nullptr;
    rc = nccl_check(g_nccl.CommInitRank(&c, world, id, rank), "ncclCommInitRank");
    if (rc) return rc;
    *comm = c;
    return SPGK_OK;
}

int spgk_nccl_allreduce_sum(void *comm, float *buf, uint64_t count, void *stream)
{
    if (!comm || !g_nccl.handle) { spgk_set_error("spgk_nccl_allreduce_sum", "no communicator"); return SPGK_E_ARG; }
    return nccl_check(g_nccl.AllReduce(buf, buf, (size_t)count, 7 /* ncclFloat32 */, 0 /* ncclSum */, comm, (cudaStream_t)stream),
                      "ncclAllReduce");
}

int spgk_nccl_destroy(void *comm)
{
    if (!comm || !g_nccl.handle) return SPGK_OK;
    return nccl_check(g_nccl.CommDestroy(comm), "ncclCommDestroy");
}

}  // extern "C"
