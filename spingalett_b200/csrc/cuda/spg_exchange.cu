// spg_exchange.cu -- the gradient exchange of data-parallel training as ONE kernel per step over peer memory:
// reduce-scatter by peer loads, the optimiser update on the own shard, all-gather of the new weights by peer stores.
//
// Every rank (one process per GPU) owns an "arena" allocated with cudaMalloc and exported with cudaIpcGetMemHandle:
//
//     [ flags | G: gradients | W: parameters | M: first moments | V: second moments ]        (flat fp32, np_pad each)
//
// The flat buffers are cut into `world` shards of `shard` elements (a multiple of 4, np_pad = shard * world).  In a
// step, rank r
//   1. tells every peer that its gradients are complete and waits until every peer has said so (flag phase 0),
//   2. sums shard r of every rank's G in rank order 0..world-1 (peer loads; the order is fixed, so the result does not
//      depend on timing), writes the sum into its own G, applies the update rule to shard r of its W / M / V and stores
//      the new weights of the shard into EVERY rank's W (peer stores),
//   3. tells every peer that its stores are done and waits for all of theirs (flag phase 1): when the kernel ends on a
//      rank, that rank's W is complete and nobody reads its G any more.
// M and V are therefore current only in the owner's shard; spgk_xchg_gather collects the shards of G, M and V when
// the host wants them (end of training, autosave).  The reference's update rules: Training.c:439-507, SIMD.c:279-494;
// its own data parallelism is OpenMP threads summing into one gradient buffer (Training.c:396-419).
//
// A barrier between the ranks is hierarchical, because a system-scope fence is the expensive part (measured on two
// B200s: 1.3 us for a flag round trip without fences, 3.5 us more per __threadfence_system(), and 15.5 us per barrier
// when each of 296 CTAs issues its own): every CTA makes its peer stores performed with a device-scope fence and
// counts itself on a local counter; thread 0 of CTA 0 waits for the count, issues ONE system fence (only where peer
// stores precede the barrier), writes this rank's flag into every peer's arena, waits for the peers' flags in its own
// and releases the other CTAs through a local flag (device scope).  That needs all CTAs resident at once: the kernels
// are launched cooperatively.  Counters and flags carry the running number of the collective and are never reset.
// Every wait is bounded: when it gives up, a status word is set, the kernel carries on to its end and the host
// reports the failure.  No TMA, no multicast, no NVLS: plain ld/st on peer pointers.
//
// The ranks' kernels wait for one another, so they must run at the same time: one rank per GPU, never two ranks'
// kernels on one device.
#include "spg_common.cuh"
#include <cstdio>
#include <cstring>

namespace {

constexpr uint32_t XG_MAX_WORLD = 8;
constexpr uint32_t XG_THREADS = 256;
// words of the arena's head, each on a 128-byte line of its own: [phase][source rank] flags written by the peers,
// then per phase the local CTA counter and the local release flag, then the status word
constexpr uint32_t XG_LINE = 32;
constexpr uint32_t XG_FLAG0 = 0, XG_CNT0 = 2 * XG_MAX_WORLD * XG_LINE, XG_GO0 = XG_CNT0 + 2 * XG_LINE, XG_STATUS_WORD = XG_GO0 + 2 * XG_LINE;
constexpr uint32_t XG_SEQ_WORD = XG_STATUS_WORD + XG_LINE;   // running number of this rank's collectives (advanced by the kernels themselves)
constexpr int XG_UNROLL = 2;                            // elements of 4 floats a thread works on at a time: the loads of every rank's copy of them (up to 16 x 16 bytes) are issued before the first is used -- a warp issues in order, so a sum placed between two loads would make the second wait for the first's round trip over NVLink
constexpr size_t XG_HEAD_BYTES = 16384;                 // flags + status, padded (keeps the buffers 256-byte aligned)
constexpr uint32_t XG_WAIT_LIMIT = 1u << 23;            // polls of 50 ns or more each before a wait gives up (about half a second)

struct XchgParams {
    float *arena[XG_MAX_WORLD];                         // every rank's arena (own: the local pointer)
    uint32_t rank, world, seq;                          // seq: running number of this collective, >= 1 (filled in by the kernel from the arena)
    const float *mfvf;                                  // optional: the step's Adam bias corrections {mf, vf} on the device
    uint64_t shard, np_pad, n_w;                        // n_w: the first n_w elements are weights (decay applies to them)
    int kind;
    float lr, momentum, b1, b2, mf, vf, eps, decay, gscale;
};

struct Xchg {
    void *arena;
    void *peer[XG_MAX_WORLD];
    int rank, world;
    uint64_t np, shard, np_pad;
    uint32_t grid;                                      // CTAs per launch: all resident at once (cooperative launch)
};

__device__ __forceinline__ float4 ld_peer(const float *p)
{
    float4 v;
    asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_peer(float *p, float4 v)
{
    asm volatile("st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

__device__ __forceinline__ float *xg_buf(float *arena, int which, uint64_t np_pad)
{
    return reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(arena) + XG_HEAD_BYTES) + (uint64_t)which * np_pad;
}

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t *p)
{
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_gpu(uint32_t *p, uint32_t v) { asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ void st_flag_sys(uint32_t *p, uint32_t v) { asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ uint32_t ld_flag_sys(const uint32_t *p)
{
    uint32_t v;
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// polls until *p has reached `want` (wrap-safe); false when the bound was hit (status word set, caller carries on)
template <bool SYS>
__device__ __forceinline__ bool xg_wait(const uint32_t *p, uint32_t want, uint32_t *status, uint32_t code, uint32_t limit = XG_WAIT_LIMIT)
{
    uint32_t polls = 0;
    while ((int32_t)((SYS ? ld_flag_sys(p) : ld_acquire_gpu(p)) - want) < 0) {
        if (++polls > limit) { atomicExch(status, code); return false; }
        if (polls > 64) __nanosleep(50);
    }
    return true;
}

// All CTAs of all ranks.  `stores_before`: peer stores of this kernel precede the barrier and must have landed when a
// peer passes it; otherwise the barrier only says "this rank has got here" (what earlier kernels of the stream wrote
// into local memory is visible to peer loads without a fence of this kernel).
__device__ __forceinline__ void xg_barrier(const XchgParams &p, uint32_t phase, bool stores_before)
{
    __syncthreads();                                     // this CTA's earlier loads and stores are issued
    if (threadIdx.x == 0) {
        uint32_t *head = reinterpret_cast<uint32_t *>(p.arena[p.rank]);
        uint32_t *status = head + XG_STATUS_WORD;
        if (stores_before) __threadfence();              // this CTA's peer stores have been performed
        atomicAdd(head + XG_CNT0 + phase * XG_LINE, 1u);
        if (blockIdx.x == 0) {
            xg_wait<false>(head + XG_CNT0 + phase * XG_LINE, p.seq * gridDim.x, status, 1u + phase);
            if (stores_before) __threadfence_system();   // ... and are visible to the peers before this rank's flag is
            for (uint32_t q = 0; q < p.world; q++)
                if (q != p.rank) st_flag_sys(reinterpret_cast<uint32_t *>(p.arena[q]) + XG_FLAG0 + (phase * XG_MAX_WORLD + p.rank) * XG_LINE, p.seq);
            for (uint32_t q = 0; q < p.world; q++)
                if (q != p.rank) xg_wait<true>(head + XG_FLAG0 + (phase * XG_MAX_WORLD + q) * XG_LINE, p.seq, status, 3u + phase);
            st_release_gpu(head + XG_GO0 + phase * XG_LINE, p.seq);
        } else {
            xg_wait<false>(head + XG_GO0 + phase * XG_LINE, p.seq, status, 5u + phase);
        }
    }
    __syncthreads();
}

// One update rule on one element (the formulas of the single-GPU optimiser kernels, operation for operation).
__device__ __forceinline__ void xg_update(const XchgParams &p, float &w, float &m, float &v, float g, bool is_weight, float omb1, float omb2)
{
    const float d = is_weight ? p.decay : 0.0f;
    float gi = g * p.gscale;
    switch (p.kind) {
        case 0: w -= p.lr * fmaf(d, w, gi); break;
        case 1: { const float mi = fmaf(p.momentum, m, fmaf(d, w, gi)); m = mi; w -= p.lr * mi; break; }
        case 2: { const float vi = fmaf(p.b2, v, omb2 * (gi * gi)); v = vi; w -= p.lr * fmaf(d, w, gi / sqrtf(vi + p.eps)); break; }
        default: {
            if (p.kind == 3) gi = fmaf(d, w, gi);
            const float mi = fmaf(p.b1, m, omb1 * gi);
            const float vi = fmaf(p.b2, v, omb2 * (gi * gi));
            m = mi; v = vi;
            const float step = p.lr * ((mi * p.mf) / sqrtf(vi * p.vf + p.eps));
            w = p.kind == 4 && d > 0.0f ? w * (1.0f - p.lr * d) - step : w - step;
        }
    }
}

__global__ void __launch_bounds__(XG_THREADS)
spg_xchg_step_kernel(const XchgParams p0)
{
    // the collective's number comes from the arena and is advanced at the end, so that every launch has the same
    // arguments (the step can be replayed as a graph); every CTA has read it before any CTA passes the first barrier
    XchgParams p = p0;
    uint32_t *seq_word = reinterpret_cast<uint32_t *>(p.arena[p.rank]) + XG_SEQ_WORD;
    p.seq = *reinterpret_cast<volatile uint32_t *>(seq_word) + 1u;
    if (p.mfvf) { p.mf = p.mfvf[0]; p.vf = p.mfvf[1]; }
    xg_barrier(p, 0, false);                             // every rank's gradients are complete
    const uint64_t base = (uint64_t)p.rank * p.shard;
    const uint64_t per = ((p.shard + gridDim.x - 1) / gridDim.x + 3) & ~(uint64_t)3;
    const uint64_t lo = (uint64_t)blockIdx.x * per, hi = lo + per < p.shard ? lo + per : p.shard;
    float *G = xg_buf(p.arena[p.rank], 0, p.np_pad), *W = xg_buf(p.arena[p.rank], 1, p.np_pad);
    float *M = xg_buf(p.arena[p.rank], 2, p.np_pad), *V = xg_buf(p.arena[p.rank], 3, p.np_pad);
    const float omb1 = 1.0f - p.b1, omb2 = 1.0f - p.b2;
    for (uint64_t i0 = lo + 4ull * threadIdx.x; i0 < hi; i0 += 4ull * XG_THREADS * XG_UNROLL) {
        float4 g[XG_MAX_WORLD][XG_UNROLL];
#pragma unroll
        for (uint32_t q = 0; q < XG_MAX_WORLD; q++) {
            if (q < p.world) {
                const float *Gq = q == p.rank ? G : xg_buf(p.arena[q], 0, p.np_pad);
#pragma unroll
                for (int u = 0; u < XG_UNROLL; u++) {
                    const uint64_t i = i0 + 4ull * XG_THREADS * u;
                    g[q][u] = i < hi ? ld_peer(Gq + base + i) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                }
            }
        }
        float4 s[XG_UNROLL];
#pragma unroll
        for (int u = 0; u < XG_UNROLL; u++) s[u] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
        for (uint32_t q = 0; q < XG_MAX_WORLD; q++) {     // rank order: the sum is the same whoever computes it
            if (q < p.world) {
#pragma unroll
                for (int u = 0; u < XG_UNROLL; u++) { s[u].x += g[q][u].x; s[u].y += g[q][u].y; s[u].z += g[q][u].z; s[u].w += g[q][u].w; }
            }
        }
#pragma unroll
        for (int u = 0; u < XG_UNROLL; u++) {
            const uint64_t i = i0 + 4ull * XG_THREADS * u;
            if (i >= hi) break;
            const uint64_t idx = base + i;
            *reinterpret_cast<float4 *>(G + idx) = s[u];    // nobody else reads this shard of this rank's G
            float4 w = *reinterpret_cast<const float4 *>(W + idx), m = *reinterpret_cast<const float4 *>(M + idx), v = *reinterpret_cast<const float4 *>(V + idx);
            xg_update(p, w.x, m.x, v.x, s[u].x, idx + 0 < p.n_w, omb1, omb2);
            xg_update(p, w.y, m.y, v.y, s[u].y, idx + 1 < p.n_w, omb1, omb2);
            xg_update(p, w.z, m.z, v.z, s[u].z, idx + 2 < p.n_w, omb1, omb2);
            xg_update(p, w.w, m.w, v.w, s[u].w, idx + 3 < p.n_w, omb1, omb2);
            *reinterpret_cast<float4 *>(M + idx) = m;
            *reinterpret_cast<float4 *>(V + idx) = v;
            for (uint32_t q = 0; q < p.world; q++) {
                if (q == p.rank) *reinterpret_cast<float4 *>(W + idx) = w;
                else st_peer(xg_buf(p.arena[q], 1, p.np_pad) + idx, w);
            }
        }
    }
    xg_barrier(p, 1, true);                              // every rank's weight stores have landed
    if (blockIdx.x == 0 && threadIdx.x == 0) *seq_word = p.seq;
}

// Shards of G (summed gradients), M and V from their owners into this rank's arena.
__global__ void __launch_bounds__(XG_THREADS)
spg_xchg_gather_kernel(const XchgParams p0)
{
    XchgParams p = p0;
    uint32_t *seq_word = reinterpret_cast<uint32_t *>(p.arena[p.rank]) + XG_SEQ_WORD;
    p.seq = *reinterpret_cast<volatile uint32_t *>(seq_word) + 1u;
    xg_barrier(p, 0, false);
    const uint64_t per = ((p.shard + gridDim.x - 1) / gridDim.x + 3) & ~(uint64_t)3;
    const uint64_t lo = (uint64_t)blockIdx.x * per, hi = lo + per < p.shard ? lo + per : p.shard;
    for (uint32_t q = 0; q < p.world; q++) {
        if (q == p.rank) continue;
        const uint64_t base = (uint64_t)q * p.shard;
        for (int which = 0; which < 4; which++) {
            if (which == 1) continue;                    // W is complete everywhere already
            const float *src = xg_buf(p.arena[q], which, p.np_pad) + base;
            float *dst = xg_buf(p.arena[p.rank], which, p.np_pad) + base;
            for (uint64_t i = lo + 4ull * threadIdx.x; i < hi; i += 4ull * XG_THREADS) *reinterpret_cast<float4 *>(dst + i) = ld_peer(src + i);
        }
    }
    xg_barrier(p, 1, false);                             // nobody reads this rank's shards any more
    if (blockIdx.x == 0 && threadIdx.x == 0) *seq_word = p.seq;
}

// the exchange's wait on a flag that nobody sets, with a small bound: out[0] = 1 when the wait reported the time-out,
// out[1] = the status word it left, out[2] = 7 once the thread has carried on past it
__global__ void spg_xchg_wait_selftest_kernel(uint32_t *words, uint32_t limit, int sys_scope)
{
    const bool ok = sys_scope ? xg_wait<true>(words + 8, 1u, words + 1, 42u, limit) : xg_wait<false>(words + 8, 1u, words + 1, 42u, limit);
    words[0] = ok ? 0u : 1u;
    words[2] = 7u;
}

void xg_fill(const Xchg *x, XchgParams *p)
{
    memset(p, 0, sizeof *p);
    for (int q = 0; q < x->world; q++) p->arena[q] = reinterpret_cast<float *>(q == x->rank ? x->arena : x->peer[q]);
    p->rank = (uint32_t)x->rank; p->world = (uint32_t)x->world;
    p->shard = x->shard; p->np_pad = x->np_pad;
}

// cooperative launch: the driver refuses it unless every CTA can be resident at once, which the grid barrier needs
int xg_launch(const void *kernel, Xchg *x, XchgParams *p, void *stream, const char *name)
{
    if (!x->grid) {
        int per_sm = 0, dev = 0, sms = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, spg_xchg_step_kernel, XG_THREADS, 0) != cudaSuccess || per_sm < 1 ||
            cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1) {
            spgk_set_error(name, "occupancy query failed");
            cudaGetLastError();
            return SPGK_E_CUDA;
        }
        x->grid = (uint32_t)sms * (per_sm > 2 ? 2u : (uint32_t)per_sm);
    }
    void *args[] = { p };
    if (cudaLaunchCooperativeKernel(kernel, dim3(x->grid), dim3(XG_THREADS), args, 0, (cudaStream_t)stream) != cudaSuccess) {
        spgk_set_error(name, cudaGetErrorString(cudaGetLastError()));
        return SPGK_E_CUDA;
    }
    return spgk_check_launch(name);
}

}  // namespace

extern "C" {

// Collective over the ranks of `comm`: allocates this rank's arena for `np` parameters, exchanges the IPC handles
// (through a sum all-reduce of byte values, so no other channel is needed) and maps the peers' arenas.
int spgk_xchg_create(void **out, int rank, int world, uint64_t np, void *comm, void *stream)
{
    if (!out || world < 2 || world > (int)XG_MAX_WORLD || rank < 0 || rank >= world || !np || !comm) {
        spgk_set_error("spgk_xchg_create", "bad argument (2..8 ranks)");
        return SPGK_E_ARG;
    }
    *out = nullptr;
    Xchg *x = new Xchg();
    x->rank = rank; x->world = world; x->np = np;
    x->shard = (((np + world - 1) / world) + 3) & ~(uint64_t)3;
    x->np_pad = x->shard * world;
    const size_t bytes = XG_HEAD_BYTES + 4 * x->np_pad * sizeof(float);
    cudaStream_t st = (cudaStream_t)stream;
    float *d_h = nullptr;
    float h[XG_MAX_WORLD * 64];
    cudaIpcMemHandle_t mine;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    int rc = SPGK_E_CUDA;
    bool ok = true;
    if (cudaMalloc(&x->arena, bytes) != cudaSuccess) { spgk_set_error("spgk_xchg_create: cudaMalloc", cudaGetErrorString(cudaGetLastError())); rc = SPGK_E_NOMEM; ok = false; }
    if (ok && cudaMemsetAsync(x->arena, 0, bytes, st) != cudaSuccess) ok = false;
    if (ok && cudaIpcGetMemHandle(&mine, x->arena) != cudaSuccess) { spgk_set_error("cudaIpcGetMemHandle", cudaGetErrorString(cudaGetLastError())); ok = false; }
    if (ok && cudaMalloc(&d_h, sizeof h) != cudaSuccess) { rc = SPGK_E_NOMEM; ok = false; }
    // every rank takes part in the all-reduce, also one whose set-up failed (its row carries 1000 in every slot:
    // no byte value), so that the others learn of it instead of waiting
    memset(h, 0, sizeof h);
    for (int i = 0; i < 64; i++) h[rank * 64 + i] = ok ? (float)reinterpret_cast<const unsigned char *>(&mine)[i] : 1000.0f;
    if (d_h) {
        if (cudaMemcpyAsync(d_h, h, sizeof h, cudaMemcpyHostToDevice, st) != cudaSuccess) ok = false;
        if (spgk_nccl_allreduce_sum(comm, d_h, (uint64_t)world * 64, st) != SPGK_OK) ok = false;
        if (cudaMemcpyAsync(h, d_h, sizeof h, cudaMemcpyDeviceToHost, st) != cudaSuccess) ok = false;
        if (cudaStreamSynchronize(st) != cudaSuccess) ok = false;
        cudaFree(d_h);
    }
    for (int q = 0; q < world && ok; q++)
        for (int i = 0; i < 64; i++) if (h[q * 64 + i] > 255.0f) { spgk_set_error("spgk_xchg_create", "a rank could not set up its exchange arena"); ok = false; break; }
    for (int q = 0; q < world && ok; q++) {
        if (q == rank) continue;
        cudaIpcMemHandle_t theirs;
        for (int i = 0; i < 64; i++) reinterpret_cast<unsigned char *>(&theirs)[i] = (unsigned char)h[q * 64 + i];
        if (cudaIpcOpenMemHandle(&x->peer[q], theirs, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
            spgk_set_error("cudaIpcOpenMemHandle", cudaGetErrorString(cudaGetLastError()));
            x->peer[q] = nullptr;
            ok = false;
        }
    }
    if (!ok) {
        for (int q = 0; q < world; q++) if (x->peer[q]) cudaIpcCloseMemHandle(x->peer[q]);
        if (x->arena) cudaFree(x->arena);
        delete x;
        cudaGetLastError();
        return rc;
    }
    *out = x;
    return SPGK_OK;
}

// The peers must be through with this rank's arena (no collective in flight) before it goes away.
void spgk_xchg_destroy(void *xv)
{
    Xchg *x = static_cast<Xchg *>(xv);
    if (!x) return;
    for (int q = 0; q < x->world; q++) if (x->peer[q]) cudaIpcCloseMemHandle(x->peer[q]);
    cudaFree(x->arena);
    delete x;
}

// Failure-path check without a failure: runs the exchange's bounded wait on a flag that is never written.  words3
// (device, 3 x uint32 of the caller) receives {1, 42, 7}: timed out, status code recorded, thread carried on.
int spgk_selftest_xchg_wait(uint32_t *words16_dev, uint32_t limit, int sys_scope, void *stream)
{
    if (!words16_dev || limit == 0 || limit > (1u << 20)) { spgk_set_error("spgk_selftest_xchg_wait", "bad argument"); return SPGK_E_ARG; }
    if (cudaMemsetAsync(words16_dev, 0, 64, (cudaStream_t)stream) != cudaSuccess) { spgk_set_error("spgk_selftest_xchg_wait", cudaGetErrorString(cudaGetLastError())); return SPGK_E_CUDA; }
    spg_xchg_wait_selftest_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(words16_dev, limit, sys_scope);
    return spgk_check_launch("spg_xchg_wait_selftest_kernel");
}

uint64_t spgk_xchg_capacity(const void *xv) { return xv ? static_cast<const Xchg *>(xv)->np : 0; }

// which: 0 gradients, 1 parameters, 2 first moments, 3 second moments (np_pad floats each, this rank's own)
float *spgk_xchg_buffer(void *xv, int which)
{
    Xchg *x = static_cast<Xchg *>(xv);
    if (!x || which < 0 || which > 3) return nullptr;
    return reinterpret_cast<float *>(static_cast<uint8_t *>(x->arena) + XG_HEAD_BYTES) + (uint64_t)which * x->np_pad;
}

int spgk_xchg_step(void *xv, int kind, uint64_t n_weights, float lr, float momentum, float b1, float b2, float mf, float vf, float eps,
                   float decay, float gscale, const float *mfvf_dev, void *stream)
{
    Xchg *x = static_cast<Xchg *>(xv);
    if (!x || kind < 0 || kind > 4) { spgk_set_error("spgk_xchg_step", "bad argument"); return SPGK_E_ARG; }
    XchgParams p;
    xg_fill(x, &p);
    p.n_w = n_weights; p.kind = kind; p.lr = lr; p.momentum = momentum; p.b1 = b1; p.b2 = b2; p.mf = mf; p.vf = vf; p.eps = eps;
    p.decay = decay; p.gscale = gscale; p.mfvf = mfvf_dev;
    return xg_launch(reinterpret_cast<const void *>(spg_xchg_step_kernel), x, &p, stream, "spg_xchg_step_kernel");
}

int spgk_xchg_gather(void *xv, void *stream)
{
    Xchg *x = static_cast<Xchg *>(xv);
    if (!x) { spgk_set_error("spgk_xchg_gather", "bad argument"); return SPGK_E_ARG; }
    XchgParams p;
    xg_fill(x, &p);
    return xg_launch(reinterpret_cast<const void *>(spg_xchg_gather_kernel), x, &p, stream, "spg_xchg_gather_kernel");
}

// After the stream has been synchronised: SPGK_OK, or SPGK_E_TIMEOUT when a wait for a peer gave up (the status word
// is cleared again).
int spgk_xchg_status(void *xv, void *stream)
{
    Xchg *x = static_cast<Xchg *>(xv);
    if (!x) return SPGK_OK;
    uint32_t w = 0;
    uint32_t *d = reinterpret_cast<uint32_t *>(x->arena) + XG_STATUS_WORD;
    if (cudaMemcpyAsync(&w, d, 4, cudaMemcpyDeviceToHost, (cudaStream_t)stream) != cudaSuccess || cudaStreamSynchronize((cudaStream_t)stream) != cudaSuccess) {
        spgk_set_error("spgk_xchg_status", cudaGetErrorString(cudaGetLastError()));
        return SPGK_E_CUDA;
    }
    if (!w) return SPGK_OK;
    cudaMemsetAsync(d, 0, 4, (cudaStream_t)stream);
    char msg[96];
    snprintf(msg, sizeof msg, "a bounded wait for a peer rank gave up (phase %u): a rank is missing or far behind", w - 1);
    spgk_set_error("gradient exchange", msg);
    return SPGK_E_TIMEOUT;
}

}  // extern "C"
