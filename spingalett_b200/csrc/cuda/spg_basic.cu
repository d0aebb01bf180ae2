// spg_basic.cu -- device plumbing of the C shim, the general SIMT layer kernel
// (any precision, any shape), the row softmax and the 16-bit activation split.
#include "spg_common.cuh"
#include <atomic>
#include <cstdio>
#include <cstring>

static thread_local char g_err[512] = "no error";
static std::atomic<uint64_t> g_launches{0};

void spgk_set_error(const char *what, const char *detail)
{
    snprintf(g_err, sizeof g_err, "%s: %s", what ? what : "?", detail ? detail : "?");
}
void spgk_count_launch(unsigned n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
int spgk_check_launch(const char *kernel_name)
{
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { spgk_set_error(kernel_name, cudaGetErrorString(e)); return SPGK_E_CUDA; }
    spgk_count_launch();
    return SPGK_OK;
}

int spg_device_props(SpgDeviceProps *out)
{
    static SpgDeviceProps table[SPG_MAX_DEVICES];
    static SpgOncePerDevice once;
    int dev = 0;
    SPGK_CUDA(cudaGetDevice(&dev));
    const int rc = once.run(dev, [&]() -> int {
        int sms = 0, optin = 0, major = 0, minor = 0;
        SPGK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        SPGK_CUDA(cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
        SPGK_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
        SPGK_CUDA(cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev));
        table[dev].cc = major * 10 + minor; table[dev].sm_count = sms; table[dev].smem_optin = (size_t)optin;
        return SPGK_OK;
    });
    if (rc) return rc;
    *out = table[dev];
    return SPGK_OK;
}

extern "C" {

// Host-only check of the once-per-device bookkeeping the launchers use (no CUDA call): `calls` rounds over
// `devices` fake device indices, the set-up of device `fail_first` failing on its first attempt.  Returns the
// number of set-ups that ran, or -1 if an out-of-range index was accepted.
int spgk_selftest_once_per_device(int devices, int calls, int fail_first)
{
    SpgOncePerDevice once;
    int ran = 0;
    bool failed_once = false;
    for (int c = 0; c < calls; c++)
        for (int d = 0; d < devices; d++)
            once.run(d, [&]() -> int {
                ran++;
                if (d == fail_first && !failed_once) { failed_once = true; return SPGK_E_CUDA; }
                return SPGK_OK;
            });
    if (once.run(-1, [] { return SPGK_OK; }) == SPGK_OK || once.run(SPG_MAX_DEVICES, [] { return SPGK_OK; }) == SPGK_OK) return -1;
    return ran;
}

const char *spgk_error_string(void) { return g_err; }
uint64_t spgk_launch_count(void) { return g_launches.load(); }

int spgk_device_count(int *count)
{
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) { *count = 0; spgk_set_error("cudaGetDeviceCount", cudaGetErrorString(e)); return SPGK_E_CUDA; }
    *count = n;
    return SPGK_OK;
}
int spgk_set_device(int device) { SPGK_CUDA(cudaSetDevice(device)); return SPGK_OK; }
int spgk_get_device(int *device) { SPGK_CUDA(cudaGetDevice(device)); return SPGK_OK; }
int spgk_device_info(int *cc, int *sm_count, size_t *total_mem)
{
    int dev = 0;
    SPGK_CUDA(cudaGetDevice(&dev));
    cudaDeviceProp p;
    SPGK_CUDA(cudaGetDeviceProperties(&p, dev));
    if (cc) *cc = p.major * 10 + p.minor;
    if (sm_count) *sm_count = p.multiProcessorCount;
    if (total_mem) *total_mem = p.totalGlobalMem;
    return SPGK_OK;
}
// test hook: the k-th device allocation from now fails as if the device were out of memory (k <= 0: off)
static std::atomic<int> g_fail_malloc_in{0};
void spgk_fail_malloc_after(int k) { g_fail_malloc_in.store(k > 0 ? k : 0); }

int spgk_malloc(void **dev, size_t bytes)
{
    *dev = nullptr;
    if (g_fail_malloc_in.load(std::memory_order_relaxed) > 0 && g_fail_malloc_in.fetch_sub(1) == 1) {
        spgk_set_error("cudaMalloc", "out of memory (injected by spgk_fail_malloc_after)");
        return SPGK_E_NOMEM;
    }
    SPGK_CUDA(cudaMalloc(dev, bytes ? bytes : 256));
    return SPGK_OK;
}
int spgk_mem_info(size_t *free_bytes, size_t *total_bytes)
{
    size_t f = 0, t = 0;
    SPGK_CUDA(cudaMemGetInfo(&f, &t));
    if (free_bytes) *free_bytes = f;
    if (total_bytes) *total_bytes = t;
    return SPGK_OK;
}
int spgk_free(void *dev) { if (dev) SPGK_CUDA(cudaFree(dev)); return SPGK_OK; }
int spgk_host_alloc(void **host, size_t bytes)
{
    *host = nullptr;
    SPGK_CUDA(cudaHostAlloc(host, bytes ? bytes : 64, cudaHostAllocDefault));
    return SPGK_OK;
}
int spgk_host_free(void *host) { if (host) SPGK_CUDA(cudaFreeHost(host)); return SPGK_OK; }
int spgk_memcpy_h2d(void *dev, const void *host, size_t bytes, void *stream)
{
    SPGK_CUDA(cudaMemcpyAsync(dev, host, bytes, cudaMemcpyHostToDevice, (cudaStream_t)stream));
    return SPGK_OK;
}
int spgk_memcpy_d2h(void *host, const void *dev, size_t bytes, void *stream)
{
    SPGK_CUDA(cudaMemcpyAsync(host, dev, bytes, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    return SPGK_OK;
}
int spgk_memcpy_d2d(void *dst, const void *src, size_t bytes, void *stream)
{
    SPGK_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
    return SPGK_OK;
}
int spgk_memset(void *dev, int value, size_t bytes, void *stream)
{
    SPGK_CUDA(cudaMemsetAsync(dev, value, bytes, (cudaStream_t)stream));
    return SPGK_OK;
}
int spgk_stream_sync(void *stream) { SPGK_CUDA(cudaStreamSynchronize((cudaStream_t)stream)); return SPGK_OK; }
int spgk_event_create(void **event)
{
    cudaEvent_t e;
    SPGK_CUDA(cudaEventCreate(&e));
    *event = e;
    return SPGK_OK;
}
int spgk_event_destroy(void *event) { if (event) SPGK_CUDA(cudaEventDestroy((cudaEvent_t)event)); return SPGK_OK; }
int spgk_event_record(void *event, void *stream) { SPGK_CUDA(cudaEventRecord((cudaEvent_t)event, (cudaStream_t)stream)); return SPGK_OK; }
int spgk_stream_create(void **stream) { cudaStream_t s; SPGK_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking)); *stream = s; return SPGK_OK; }
int spgk_stream_destroy(void *stream) { if (stream) SPGK_CUDA(cudaStreamDestroy((cudaStream_t)stream)); return SPGK_OK; }
int spgk_stream_wait_event(void *stream, void *event) { SPGK_CUDA(cudaStreamWaitEvent((cudaStream_t)stream, (cudaEvent_t)event, 0)); return SPGK_OK; }
int spgk_event_elapsed_ms(void *start, void *stop, float *ms) { SPGK_CUDA(cudaEventElapsedTime(ms, (cudaEvent_t)start, (cudaEvent_t)stop)); return SPGK_OK; }
int spgk_event_sync(void *event) { SPGK_CUDA(cudaEventSynchronize((cudaEvent_t)event)); return SPGK_OK; }
// 1: page-locked host memory (cudaMallocHost, cudaHostRegister), 0: ordinary (pageable) host memory or unknown
int spgk_is_pinned_host_pointer(const void *ptr)
{
    cudaPointerAttributes a;
    cudaError_t e = cudaPointerGetAttributes(&a, ptr);
    if (e != cudaSuccess) { cudaGetLastError(); return 0; }
    return a.type == cudaMemoryTypeHost ? 1 : 0;
}
int spgk_is_device_pointer(const void *ptr)
{
    cudaPointerAttributes a;
    cudaError_t e = cudaPointerGetAttributes(&a, ptr);
    if (e != cudaSuccess) { cudaGetLastError(); return 0; }
    return (a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged) ? 1 : 0;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// K0: general layer.  One warp per output neuron j and tile of up to NB batch
// rows; lanes stride over k.  Every stored element is decoded individually, so
// rows of packed formats may start in the middle of a byte.
// ---------------------------------------------------------------------------
template <int NB>
__global__ void __launch_bounds__(256)
spg_layer_simt_kernel(const void *__restrict__ w, const float *__restrict__ bias, float w_scale,
                      uint32_t in, uint32_t out, int precision, int act,
                      const float *__restrict__ x, uint32_t ldx, float *__restrict__ y, uint32_t ldy, uint32_t N)
{
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t j = blockIdx.x * 8u + warp;
    const uint32_t n0 = blockIdx.y * NB;
    if (j >= out) return;
    float acc[NB];
#pragma unroll
    for (int b = 0; b < NB; b++) acc[b] = 0.0f;
    const uint64_t row0 = (uint64_t)j * in;
    for (uint32_t k = lane; k < in; k += 32u) {
        float q = spg_decode_elem(w, row0 + k, precision);
#pragma unroll
        for (int b = 0; b < NB; b++) {
            uint32_t n = n0 + b;
            float xv = n < N ? x[(uint64_t)n * ldx + k] : 0.0f;
            acc[b] = fmaf(q, xv, acc[b]);
        }
    }
#pragma unroll
    for (int b = 0; b < NB; b++) acc[b] = spg_warp_sum(acc[b]);
    if (lane == 0) {
        float bj = bias ? bias[j] : 0.0f;
#pragma unroll
        for (int b = 0; b < NB; b++) {
            uint32_t n = n0 + b;
            if (n < N) y[(uint64_t)n * ldy + j] = spg_activate(fmaf(acc[b], w_scale, bj), act);
        }
    }
}

// Row softmax, one warp per row (Activation.c:5-21).
__global__ void __launch_bounds__(256)
spg_softmax_rows_kernel(float *__restrict__ y, uint32_t ldy, uint32_t N, uint32_t width, const uint32_t *__restrict__ limit)
{
    N = spg_limit_rows(N, limit);
    const uint32_t lane = threadIdx.x & 31u;
    for (uint32_t row = blockIdx.x * 8u + (threadIdx.x >> 5); row < N; row += gridDim.x * 8u) {
    float *r = y + (uint64_t)row * ldy;
    float mx = -FLT_MAX;
    for (uint32_t i = lane; i < width; i += 32u) { float v = r[i]; if (v > mx) mx = v; }
    mx = spg_warp_max(mx);
    float sum = 0.0f;
    for (uint32_t i = lane; i < width; i += 32u) { float e = expf(r[i] - mx); r[i] = e; sum += e; }
    sum = spg_warp_sum(sum);
    if (sum > 0.0f) {
        float inv = 1.0f / sum;
        for (uint32_t i = lane; i < width; i += 32u) r[i] *= inv;
    }
    }
}

// Row softmax for a handful of rows: one 256-thread block per row, so a single wide row (batch 1,
// width 1000) is not left to one warp.
__global__ void __launch_bounds__(256)
spg_softmax_block_kernel(float *__restrict__ y, uint32_t ldy, uint32_t width)
{
    __shared__ float red[8];
    __shared__ float bcast;
    float *r = y + (uint64_t)blockIdx.x * ldy;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    float mx = -FLT_MAX;
    for (uint32_t i = tid; i < width; i += 256) { float v = r[i]; if (v > mx) mx = v; }
    mx = spg_warp_max(mx);
    if (lane == 0) red[warp] = mx;
    __syncthreads();
    if (tid == 0) { float m = red[0]; for (int q = 1; q < 8; q++) m = fmaxf(m, red[q]); bcast = m; }
    __syncthreads();
    mx = bcast;
    float sum = 0.0f;
    for (uint32_t i = tid; i < width; i += 256) { float e = expf(r[i] - mx); r[i] = e; sum += e; }
    sum = spg_warp_sum(sum);
    __syncthreads();
    if (lane == 0) red[warp] = sum;
    __syncthreads();
    if (tid == 0) { float t = 0.0f; for (int q = 0; q < 8; q++) t += red[q]; bcast = t; }
    __syncthreads();
    sum = bcast;
    if (sum > 0.0f) {
        const float inv = 1.0f / sum;
        for (uint32_t i = tid; i < width; i += 256) r[i] *= inv;
    }
}

// Rows whose two largest outputs are closer than `theta` in log space (log p1 - log p2 < theta), and rows with a
// non-finite output, are appended to `idx` (order unspecified) and counted in *count.  One warp per row.
__global__ void __launch_bounds__(256)
spg_margin_select_kernel(const float *__restrict__ probs, uint32_t ldp, uint32_t N, uint32_t width, float theta,
                         uint32_t *__restrict__ idx, uint32_t *__restrict__ count)
{
    const uint32_t row = blockIdx.x * 8u + (threadIdx.x >> 5), lane = threadIdx.x & 31u;
    if (row >= N) return;
    const float *r = probs + (uint64_t)row * ldp;
    float a = -FLT_MAX, b = -FLT_MAX;                          // largest, second largest seen by this lane
    bool bad = false;                                          // a non-finite output: the one-term pass left the 16-bit range
    for (uint32_t i = lane; i < width; i += 32u) {
        const float v = r[i];
        bad |= !(fabsf(v) <= FLT_MAX);
        if (v > a) { b = a; a = v; } else if (v > b) b = v;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {                         // merge the (largest, second) pairs across lanes
        const float oa = __shfl_xor_sync(0xffffffffu, a, o), ob = __shfl_xor_sync(0xffffffffu, b, o);
        if (oa > a) { b = fmaxf(a, ob); a = oa; } else b = fmaxf(b, oa);
    }
    bad = __any_sync(0xffffffffu, bad);
    if (lane == 0 && (bad || (b > 0.0f && logf(a) - logf(b) < theta))) idx[atomicAdd(count, 1u)] = row;
}

// Largest change of the top-two log gap between two sets of row outputs: for every row, the two largest entries
// of `exact` define the pair (i1, i2); the result is max over rows of |log(f[i1]/f[i2]) - log(e[i1]/e[i2])|,
// accumulated with atomicMax on the float's bit pattern (the values are non-negative).  One warp per row.
__global__ void __launch_bounds__(256)
spg_gap_error_kernel(const float *__restrict__ fast, const float *__restrict__ exact, uint32_t ld, uint32_t N, uint32_t width,
                     uint32_t *__restrict__ max_bits)
{
    const uint32_t row = blockIdx.x * 8u + (threadIdx.x >> 5), lane = threadIdx.x & 31u;
    if (row >= N) return;
    const float *e = exact + (uint64_t)row * ld, *f = fast + (uint64_t)row * ld;
    float a = -FLT_MAX, b = -FLT_MAX;
    uint32_t ia = 0, ib = 0;
    for (uint32_t i = lane; i < width; i += 32u) {
        const float v = e[i];
        if (v > a) { b = a; ib = ia; a = v; ia = i; } else if (v > b) { b = v; ib = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float oa = __shfl_xor_sync(0xffffffffu, a, o), ob = __shfl_xor_sync(0xffffffffu, b, o);
        const uint32_t oia = __shfl_xor_sync(0xffffffffu, ia, o), oib = __shfl_xor_sync(0xffffffffu, ib, o);
        if (oa > a || (oa == a && oia < ia)) {
            if (a > ob || (a == ob && ia < oib)) { b = a; ib = ia; } else { b = ob; ib = oib; }
            a = oa; ia = oia;
        } else if (oa > b || (oa == b && oia < ib)) { b = oa; ib = oia; }
    }
    if (lane == 0 && b > 0.0f && f[ia] > 0.0f && f[ib] > 0.0f) {
        const float err = fabsf((logf(f[ia]) - logf(f[ib])) - (logf(a) - logf(b)));
        if (isfinite(err)) atomicMax(max_bits, __float_as_uint(err));
    }
}

// dst[idx[i]][:] = src[i][:]
__global__ void __launch_bounds__(256)
spg_scatter_rows_kernel(const float *__restrict__ src, const uint32_t *__restrict__ idx, float *__restrict__ dst,
                        uint32_t rows, uint32_t width, uint32_t ldd, const uint32_t *__restrict__ limit)
{
    spg_grid_trigger();
    spg_grid_wait();
    rows = spg_limit_rows(rows, limit);
    const uint64_t total = (uint64_t)rows * width;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t rr = (uint32_t)(i / width), c = (uint32_t)(i % width);
        dst[(uint64_t)idx[rr] * ldd + c] = src[i];
    }
}

// fp32 -> `parts` 16-bit planes (term p = round(x - sum of earlier terms)).
template <typename T16>
__device__ __forceinline__ T16 spg_to16(float v);
template <> __device__ __forceinline__ __half spg_to16<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 spg_to16<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <typename T16>
__device__ __forceinline__ float spg_from16(T16 v);
template <> __device__ __forceinline__ float spg_from16<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float spg_from16<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// One thread converts 8 consecutive columns of one row: two 128-bit loads (when the row is
// 16-byte aligned) and one 128-bit store per plane.  ld16 is a multiple of 8.
template <typename T16, bool VEC>
__global__ void __launch_bounds__(256)
spg_split16_kernel(const float *__restrict__ x, uint32_t ldx, uint32_t N, uint32_t in,
                   T16 *__restrict__ dst, uint32_t ld16, uint64_t plane_elems, int parts, const uint32_t *__restrict__ limit,
                   const uint32_t *__restrict__ rows_idx)
{
    spg_grid_trigger();
    spg_grid_wait();
    N = spg_limit_rows(N, limit);
    const uint32_t chunks = ld16 >> 3;
    const uint64_t total = (uint64_t)N * chunks;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t n = (uint32_t)(i / chunks), k0 = (uint32_t)(i % chunks) << 3;
        const float *src = x + (uint64_t)(rows_idx ? rows_idx[n] : n) * ldx + k0;      // optional gather: row n comes from row rows_idx[n]
        float v[8];
        if (VEC && k0 + 8 <= in) {
            const float4 a = __ldg(reinterpret_cast<const float4 *>(src));
            const float4 b = __ldg(reinterpret_cast<const float4 *>(src) + 1);
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        } else {
#pragma unroll
            for (int j = 0; j < 8; j++) v[j] = k0 + j < in ? src[j] : 0.0f;
        }
        T16 *out = dst + (uint64_t)n * ld16 + k0;
        for (int p = 0; p < parts; p++) {
            union { uint4 q; T16 h[8]; } pk;
#pragma unroll
            for (int j = 0; j < 8; j++) { pk.h[j] = spg_to16<T16>(v[j]); v[j] -= spg_from16<T16>(pk.h[j]); }
            *reinterpret_cast<uint4 *>(out + (uint64_t)p * plane_elems) = pk.q;
        }
    }
}


thread_local const uint32_t *spg_tls_rows_limit = nullptr;
thread_local uint32_t spg_tls_rows_expected = 0;
thread_local float spg_tls_margin_theta = 0.0f;
thread_local uint32_t *spg_tls_margin_idx = nullptr, *spg_tls_margin_count = nullptr;
thread_local const uint32_t *spg_tls_out_rows = nullptr;

extern "C" {

void spgk_set_dynamic_rows(const uint32_t *rows_dev, uint32_t expected) { spg_tls_rows_limit = rows_dev; spg_tls_rows_expected = rows_dev ? expected : 0; }
void spgk_set_output_rows(const uint32_t *rows_idx) { spg_tls_out_rows = rows_idx; }
void spgk_set_margin_sink(float theta, uint32_t *idx, uint32_t *count)
{
    spg_tls_margin_theta = theta; spg_tls_margin_idx = idx; spg_tls_margin_count = idx ? count : nullptr;
    if (!count) spg_tls_margin_idx = nullptr;
}

int spgk_layer_simt(const spgk_layer *L, const float *x, uint32_t ldx, float *y, uint32_t ldy, uint32_t N, void *stream)
{
    if (!L || !x || !y || !L->w || L->in == 0 || L->out == 0 || (unsigned)L->precision >= SPG_P_COUNT) {
        spgk_set_error("spgk_layer_simt", "bad argument");
        return SPGK_E_ARG;
    }
    if (N == 0) return SPGK_OK;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 block(256);
    uint32_t gx = (L->out + 7u) / 8u;
    int act = L->act == SPG_ACT_SOFTMAX ? SPG_ACT_NONE : L->act;
    // gridDim.y is limited to 65535: walk the batch in slabs
    const uint32_t NB = N >= 8 ? 8 : (N >= 4 ? 4 : (N >= 2 ? 2 : 1));
    const uint32_t slab = 65535u * NB;
    for (uint32_t n0 = 0; n0 < N; n0 += slab) {
        uint32_t n = N - n0 < slab ? N - n0 : slab;
        dim3 grid(gx, (n + NB - 1) / NB);
        const float *xs = x + (uint64_t)n0 * ldx;
        float *ys = y + (uint64_t)n0 * ldy;
#define SPG_LAUNCH_SIMT(NBV) spg_layer_simt_kernel<NBV><<<grid, block, 0, s>>>(L->w, L->bias, L->w_scale, L->in, L->out, L->precision, act, xs, ldx, ys, ldy, n)
        if (NB == 8) SPG_LAUNCH_SIMT(8); else if (NB == 4) SPG_LAUNCH_SIMT(4); else if (NB == 2) SPG_LAUNCH_SIMT(2); else SPG_LAUNCH_SIMT(1);
#undef SPG_LAUNCH_SIMT
        int rc = spgk_check_launch("spg_layer_simt_kernel");
        if (rc) return rc;
    }
    return SPGK_OK;
}

int spgk_softmax_rows(float *y, uint32_t ldy, uint32_t N, uint32_t width, void *stream)
{
    if (!y || width == 0 || width > 65535u) { spgk_set_error("spgk_softmax_rows", "bad argument"); return SPGK_E_ARG; }
    if (N == 0) return SPGK_OK;
    if (N <= 64 && width > 64 && !spg_tls_rows_limit) {
        spg_softmax_block_kernel<<<N, 256, 0, (cudaStream_t)stream>>>(y, ldy, width);
        return spgk_check_launch("spg_softmax_block_kernel");
    }
    uint32_t blocks = (N + 7u) / 8u;
    if (blocks > 148u * 64u) blocks = 148u * 64u;
    spg_softmax_rows_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(y, ldy, N, width, spg_tls_rows_limit);
    return spgk_check_launch("spg_softmax_rows_kernel");
}

int spgk_margin_select(const float *probs, uint32_t ldp, uint32_t N, uint32_t width, float theta,
                       uint32_t *idx, uint32_t *count, void *stream)
{
    if (!probs || !idx || !count || width < 2) { spgk_set_error("spgk_margin_select", "bad argument"); return SPGK_E_ARG; }
    if (N == 0) return SPGK_OK;
    spg_margin_select_kernel<<<(N + 7u) / 8u, 256, 0, (cudaStream_t)stream>>>(probs, ldp, N, width, theta, idx, count);
    return spgk_check_launch("spg_margin_select_kernel");
}

int spgk_gap_error(const float *fast, const float *exact, uint32_t ld, uint32_t N, uint32_t width, uint32_t *max_bits, void *stream)
{
    if (!fast || !exact || !max_bits || width < 2) { spgk_set_error("spgk_gap_error", "bad argument"); return SPGK_E_ARG; }
    if (N == 0) return SPGK_OK;
    spg_gap_error_kernel<<<(N + 7u) / 8u, 256, 0, (cudaStream_t)stream>>>(fast, exact, ld, N, width, max_bits);
    return spgk_check_launch("spg_gap_error_kernel");
}

int spgk_scatter_rows(const float *src, const uint32_t *idx, float *dst, uint32_t rows, uint32_t width, uint32_t ldd, void *stream)
{
    if (!src || !idx || !dst) { spgk_set_error("spgk_scatter_rows", "bad argument"); return SPGK_E_ARG; }
    if (rows == 0 || width == 0) return SPGK_OK;
    uint64_t total = (uint64_t)rows * width;
    uint32_t blocks = (uint32_t)((total + 255) / 256 < 148ull * 8 ? (total + 255) / 256 : 148ull * 8);
    SPGK_CUDA(spg_launch_chained(spg_scatter_rows_kernel, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, src, idx, dst, rows, width, ldd, spg_tls_rows_limit));
    return spgk_check_launch("spg_scatter_rows_kernel");
}

int spgk_split16(const float *x, uint32_t ldx, uint32_t N, uint32_t in, void *dst, uint32_t ld16,
                 uint64_t plane_elems, int parts, int type, void *stream)
{
    return spgk_split16_rows(x, ldx, nullptr, N, in, dst, ld16, plane_elems, parts, type, stream);
}

int spgk_split16_rows(const float *x, uint32_t ldx, const uint32_t *rows_idx, uint32_t N, uint32_t in, void *dst, uint32_t ld16,
                      uint64_t plane_elems, int parts, int type, void *stream)
{
    if (!x || !dst || parts < 1 || parts > 3 || ld16 < in) { spgk_set_error("spgk_split16", "bad argument"); return SPGK_E_ARG; }
    if (N == 0) return SPGK_OK;
    if ((ld16 & 7u) || (plane_elems & 7u) || ((uintptr_t)dst & 15u)) { spgk_set_error("spgk_split16", "destination planes must be 16-byte aligned"); return SPGK_E_ARG; }
    const uint64_t total = (uint64_t)N * (ld16 >> 3);
    const uint32_t blocks = (uint32_t)((total + 255) / 256 < 148ull * 16 ? (total + 255) / 256 : 148ull * 16);
    const bool vec = ((uintptr_t)x & 15u) == 0 && (ldx & 3u) == 0;
    cudaStream_t st = (cudaStream_t)stream;
    if (type == SPGK_T_F16) {
        if (vec) SPGK_CUDA(spg_launch_chained(spg_split16_kernel<__half, true>, dim3(blocks), dim3(256), 0, st, x, ldx, N, in, (__half *)dst, ld16, plane_elems, parts, spg_tls_rows_limit, rows_idx));
        else SPGK_CUDA(spg_launch_chained(spg_split16_kernel<__half, false>, dim3(blocks), dim3(256), 0, st, x, ldx, N, in, (__half *)dst, ld16, plane_elems, parts, spg_tls_rows_limit, rows_idx));
    } else {
        if (vec) SPGK_CUDA(spg_launch_chained(spg_split16_kernel<__nv_bfloat16, true>, dim3(blocks), dim3(256), 0, st, x, ldx, N, in, (__nv_bfloat16 *)dst, ld16, plane_elems, parts, spg_tls_rows_limit, rows_idx));
        else SPGK_CUDA(spg_launch_chained(spg_split16_kernel<__nv_bfloat16, false>, dim3(blocks), dim3(256), 0, st, x, ldx, N, in, (__nv_bfloat16 *)dst, ld16, plane_elems, parts, spg_tls_rows_limit, rows_idx));
    }
    return spgk_check_launch("spg_split16_kernel");
}

}  // extern "C"
