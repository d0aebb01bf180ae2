/* Device residency of a network and the orchestration of the layer chain.
 *
 * The weights go to the GPU exactly as stored (packed INT8/INT4/INT2, FP16,
 * BF16 or FP32 images, one 256-byte aligned allocation per matrix); biases go
 * as fp32.  Two chains exist: the small-batch chain (fused dequant-GEMV per
 * layer, fp32 activations) and the large-batch chain (tcgen05 GEMM per layer,
 * 16-bit activations between layers).  Shapes a fast kernel does not take run
 * on the general SIMT kernel -- still on the GPU; nothing here computes on
 * the CPU. */
#include "spg_internal.h"
#include <pthread.h>
#include <stdlib.h>
#include <math.h>
#include <string.h>
#include <unistd.h>

int spg_map_kernel_error(int rc, const char *where)
{
    if (rc == SPGK_OK) return SPINGALETT_OK;
    int code = rc == SPGK_E_NOMEM ? SPINGALETT_ERR_ALLOC
             : (rc == SPGK_E_ARG || rc == SPGK_E_UNSUPPORTED) ? SPINGALETT_ERR_INVALID
             : SPINGALETT_ERR_DEVICE;
    spg_set_errorf(code, "%s: %s", where, spgk_error_string());
    spg_log(LOG_ERROR, "%s: %s", where, spgk_error_string());
    return code;
}

static _Thread_local int t_device = -1;     /* device chosen with spingalett_set_device */

int spingalett_set_device(int device)
{
    int rc = spg_map_kernel_error(spgk_set_device(device), "set_device");
    if (rc == SPINGALETT_OK) t_device = device;
    return rc;
}

int spingalett_get_device_count(void)
{
    int n = 0;
    if (spgk_device_count(&n) != SPGK_OK) return 0;
    return n;
}

/* ---- batch sharding over several GPUs of one process ------------------------------------------------
 * spingalett_set_devices(ids, n): host-pointer batches of forward_batch are cut into n contiguous row shares
 * ([g*N/n, (g+1)*N/n), sizes differing by at most one) and share g runs on device ids[g] from a replica of the
 * net's weights there, one host thread per device, no peer access and no collective.  n <= 1 (or ids == NULL)
 * switches it off.  An id may appear more than once (two replicas on one GPU). */
#define SPG_MAX_FANOUT 16
static int g_fan_ids[SPG_MAX_FANOUT];
static int g_fan_n = 0;
static pthread_mutex_t g_fan_lock = PTHREAD_MUTEX_INITIALIZER;

int spingalett_set_devices(const int *ids, int n)
{
    int count = spingalett_get_device_count();
    if (n < 0 || n > SPG_MAX_FANOUT || (n > 0 && !ids)) { spg_set_error(SPINGALETT_ERR_INVALID, "set_devices: bad list"); return SPINGALETT_ERR_INVALID; }
    for (int i = 0; i < n; i++)
        if (ids[i] < 0 || ids[i] >= count) { spg_set_errorf(SPINGALETT_ERR_INVALID, "set_devices: no device %d", ids[i]); return SPINGALETT_ERR_INVALID; }
    pthread_mutex_lock(&g_fan_lock);
    g_fan_n = n > 1 ? n : 0;
    for (int i = 0; i < g_fan_n; i++) g_fan_ids[i] = ids[i];
    pthread_mutex_unlock(&g_fan_lock);
    return SPINGALETT_OK;
}

void spingalett_split_rows(uint32_t rows, uint32_t shares, uint32_t share, uint32_t *lo, uint32_t *hi)
{
    const uint32_t base = shares ? rows / shares : 0, extra = shares ? rows % shares : 0;
    const uint32_t b = share * base + (share < extra ? share : extra);
    if (lo) *lo = b;
    if (hi) *hi = b + base + (share < extra ? 1u : 0u);
}

void spingalett_set_stream(NeuralNetwork *net, void *cuda_stream)
{
    if (net) spg_priv(net)->stream = cuda_stream;
}

static void shadows_release(spg_net *n)
{
    for (int g = 0; g < SPG_MAX_FANOUT; g++) {
        spg_net *sh = n->shadow[g];
        if (!sh) continue;
        spg_dev_release(sh);
        spgk_host_free(sh->h_out);
        free(sh);
        n->shadow[g] = NULL;
    }
}

void spg_dev_invalidate(spg_net *n) { shadows_release(n); if (n->dev_ready) spg_dev_release(n); }

static int bind_device(spg_net *n)
{
    if (n->device < 0) {
        int count = 0;
        if (spgk_device_count(&count) != SPGK_OK || count <= 0) {
            spg_set_error(SPINGALETT_ERR_DEVICE, "no CUDA device available (this library has no CPU compute path)");
            spg_log(LOG_ERROR, "no CUDA device available");
            return SPINGALETT_ERR_DEVICE;
        }
        int cur = 0;
        if (t_device >= 0) cur = t_device;
        else if (spgk_get_device(&cur) != SPGK_OK) cur = 0;
        n->device = cur;
    }
    return spg_map_kernel_error(spgk_set_device(n->device), "bind device");
}

void spg_dev_release(spg_net *n)
{
    if (!n->is_shadow) shadows_release(n);
    if (n->device >= 0) spgk_set_device(n->device);
    for (uint32_t l = 0; l < n->dev_layers; l++) {
        if (n->d_w) spgk_free(n->d_w[l]);
        if (n->d_bias) spgk_free(n->d_bias[l]);
    }
    free(n->d_w); free(n->d_bias); free(n->klayers);
    n->d_w = NULL; n->d_bias = NULL; n->klayers = NULL; n->dev_layers = 0;
    spgk_free(n->d_small); n->d_small = NULL; n->small_cap = 0;
    spgk_free(n->d_gemv_scratch); n->d_gemv_scratch = NULL; n->gemv_scratch_bytes = 0;
    for (int i = 0; i < 2; i++) { spgk_free(n->d_staged[i]); n->d_staged[i] = NULL; n->staged_bytes[i] = 0; }
    for (int i = 0; i < 2; i++) { spgk_free(n->d_operand[i]); n->d_operand[i] = NULL; n->operand_bytes[i] = 0; }
    spgk_free(n->d_ws_scratch); n->d_ws_scratch = NULL; n->ws_scratch_bytes = 0;
    spgk_free(n->d_rep_idx); n->d_rep_idx = NULL; n->rep_idx_bytes = 0;
    n->auto_calibrated = false;
    n->auto_calls = 0;
    n->bf16_fits_f16 = 0;
    spgk_free(n->d_rep_in); n->d_rep_in = NULL; n->rep_in_bytes = 0;
    spgk_free(n->d_rep_out); n->d_rep_out = NULL; n->rep_out_bytes = 0;
    spgk_free(n->d_in32); n->d_in32 = NULL; n->in32_bytes = 0;
    spgk_free(n->d_out32); n->d_out32 = NULL; n->out32_bytes = 0;
    for (int i = 0; i < 2; i++) {
        spgk_free(n->d_act16[i]); n->d_act16[i] = NULL;
        spgk_free(n->d_act32[i]); n->d_act32[i] = NULL;
    }
    n->act16_bytes = 0; n->act32_bytes = 0;
    spgk_free(n->d_status); n->d_status = NULL;
    spgk_free(n->d_w16); n->d_w16 = NULL; n->w16_bytes = 0;
    spgk_free(n->d_head_w); n->d_head_w = NULL;
    spgk_free(n->d_fused_params); n->d_fused_params = NULL;
    spgk_host_free(n->h_count); n->h_count = NULL; n->count_pending = false; n->count_seen = false;
    for (int i = 0; i <= SPG_PIPE_MAX; i++) { if (n->copy_ev[i]) spgk_event_destroy(n->copy_ev[i]); n->copy_ev[i] = NULL; }
    spgk_stream_destroy(n->copy_stream); n->copy_stream = NULL;
    for (int i = 0; i < 2; i++) { spgk_host_free(n->h_chunk[i]); n->h_chunk[i] = NULL; }
    n->h_chunk_bytes = 0;
    for (int t = 0; t < 2; t++) {
        if (n->d_w16c[t]) for (uint32_t l = 0; l < n->dev_layers; l++) spgk_free(n->d_w16c[t][l]);
        free(n->d_w16c[t]); n->d_w16c[t] = NULL;
        free(n->w16c_parts[t]); n->w16c_parts[t] = NULL;
    }
    for (uint32_t i = 0; i < n->prof_cap; i++) spgk_event_destroy(n->prof_ev[i]);
    free(n->prof_ev); n->prof_ev = NULL; n->prof_cap = 0; n->prof_used = 0;
    n->dev_ready = false;
}

int spg_dev_ensure(spg_net *n)
{
    if (n->dev_ready) return spg_map_kernel_error(spgk_set_device(n->device), "bind device");
    NeuralNetwork *p = &n->pub;
    if (p->layers < 2) { spg_set_error(SPINGALETT_ERR_INVALID, "network has no weight layer"); return SPINGALETT_ERR_INVALID; }
    int rc = bind_device(n);
    if (rc) return rc;
    uint32_t wl = p->layers - 1;
    n->d_w = calloc(wl, sizeof *n->d_w);
    n->d_bias = calloc(wl, sizeof *n->d_bias);
    n->klayers = calloc(wl, sizeof *n->klayers);
    if (!n->d_w || !n->d_bias || !n->klayers) {
        spg_set_error(SPINGALETT_ERR_ALLOC, "device descriptor allocation failed");
        free(n->d_w); free(n->d_bias); free(n->klayers);
        n->d_w = NULL; n->d_bias = NULL; n->klayers = NULL;
        return SPINGALETT_ERR_ALLOC;
    }
    n->dev_layers = wl;
    const bool packed = n->payload_layers == wl && n->payload_w;
    for (uint32_t l = 0; l < wl; l++) {
        uint32_t in = p->topology[l], out = p->topology[l + 1];
        const void *src;
        size_t bytes;
        float scale = 1.0f;
        PrecisionMode prec;
        if (packed) {
            src = n->payload_w[l]; bytes = n->payload_w_bytes[l]; prec = n->store_precision;
            if (prec >= PRECISION_INT8) {
                float amax = n->amax_w[l];
                scale = amax > 0.0f ? amax / spg_precision_q(prec) : 0.0f;     /* Serialize.c:232 */
            }
        } else {
            src = p->weights + p->weight_offsets[l]; bytes = (size_t)in * out * sizeof(float); prec = PRECISION_FLOAT32;
        }
        /* slack so that whole-vector loads at the tail of the last row stay inside the allocation */
        if ((rc = spg_map_kernel_error(spgk_malloc(&n->d_w[l], bytes + 256), "weight allocation"))) goto fail;
        if ((rc = spg_map_kernel_error(spgk_memset((char *)n->d_w[l] + bytes, 0, 256, n->stream), "weight tail clear"))) goto fail;
        if ((rc = spg_map_kernel_error(spgk_memcpy_h2d(n->d_w[l], src, bytes, n->stream), "weight upload"))) goto fail;
        void *db = NULL;
        if ((rc = spg_map_kernel_error(spgk_malloc(&db, (size_t)out * sizeof(float)), "bias allocation"))) goto fail;
        n->d_bias[l] = db;
        if ((rc = spg_map_kernel_error(spgk_memcpy_h2d(db, p->biases + p->bias_offsets[l], (size_t)out * sizeof(float), n->stream), "bias upload"))) goto fail;
        float babs = 0.0f;
        for (uint32_t j = 0; j < out; j++) {
            const float a = fabsf(p->biases[p->bias_offsets[l] + j]);
            if (a > babs) babs = a;
        }
        n->klayers[l] = (spgk_layer){ .w = n->d_w[l], .bias = n->d_bias[l], .w_scale = scale, .in = in, .out = out,
                                      .precision = (int32_t)prec, .act = (int32_t)p->act_func[l], .bias_absmax = babs };
    }
    void *st = NULL;
    if ((rc = spg_map_kernel_error(spgk_malloc(&st, 64), "status allocation"))) goto fail;
    n->d_status = st;
    if ((rc = spg_map_kernel_error(spgk_memset(st, 0, 64, n->stream), "status clear"))) goto fail;
    if ((rc = spg_map_kernel_error(spgk_stream_sync(n->stream), "upload sync"))) goto fail;
    n->dev_ready = true;
    return SPINGALETT_OK;
fail:
    spg_dev_release(n);
    return rc;
}

static void prof_collect(spg_net *n);
static void prof_mark(spg_net *n);

/* Wait for the net's stream, then surface a bounded-wait failure reported by a
 * tensor-core kernel and fold the timing events in. */
static int finish(spg_net *n)
{
    int rc;
    if (n->ws_pending) {
        n->ws_pending = false;
        if ((rc = spg_map_kernel_error(spgk_wstream_status(n->d_ws_scratch, n->stream), "weight-stream kernel"))) return rc;
    }
    if (n->gemv_pending) {
        n->gemv_pending = false;
        if ((rc = spg_map_kernel_error(spgk_gemv_status(n->d_gemv_scratch, n->stream), "GEMV"))) return rc;
    }
    if (n->status_pending) {
        n->status_pending = false;
        if ((rc = spg_map_kernel_error(spgk_gemm_tc_status(n->d_status, n->stream), "tcgen05 GEMM"))) return rc;
    } else if ((rc = spg_map_kernel_error(spgk_stream_sync(n->stream), "stream sync"))) return rc;
    prof_collect(n);
    return SPINGALETT_OK;
}

int spingalett_synchronize(NeuralNetwork *net)
{
    if (!net) { spg_set_error(SPINGALETT_ERR_INVALID, "synchronize: net is NULL"); return SPINGALETT_ERR_INVALID; }
    spg_net *n = spg_priv(net);
    if (!n->dev_ready) return SPINGALETT_OK;
    int rc = spg_map_kernel_error(spgk_set_device(n->device), "bind device");
    return rc ? rc : finish(n);
}

int spingalett_sync_weights(NeuralNetwork *net)
{
    if (!net) { spg_set_error(SPINGALETT_ERR_INVALID, "sync_weights: net is NULL"); return SPINGALETT_ERR_INVALID; }
    spg_net *n = spg_priv(net);
    spg_dev_invalidate(n);
    spg_net_drop_payload(n);            /* the host fp32 arrays are now the truth */
    return SPINGALETT_OK;
}

uint32_t spingalett_last_repaired(NeuralNetwork *net)
{
    if (!net) return 0;
    spg_net *n = spg_priv(net);
    if (n->count_pending) {                       /* the count was copied asynchronously: wait for it */
        n->count_pending = false;
        if (spgk_stream_sync(n->stream) == 0 && n->h_count) {
            n->last_repaired = 0;
            for (uint32_t i = 0; i < n->count_slots_used; i++) n->last_repaired += n->h_count[i];
        }
    }
    return n->last_repaired;
}
float spingalett_net_margin(NeuralNetwork *net) { return net ? spg_priv(net)->auto_theta : 0.0f; }

/* ---- optional timing of the layer kernels -------------------------------- */
void spingalett_profile(NeuralNetwork *net, bool enable)
{
    if (!net) return;
    spg_net *n = spg_priv(net);
    n->prof_on = enable;
    n->prof_ms = 0.0; n->prof_launches = 0; n->prof_used = 0;
}

void spingalett_profile_read(NeuralNetwork *net, double *kernel_ms, uint64_t *launches)
{
    spg_net *n = spg_priv(net);
    if (kernel_ms) *kernel_ms = n->prof_ms;
    if (launches) *launches = n->prof_launches;
    n->prof_ms = 0.0; n->prof_launches = 0;
}

static void prof_mark(spg_net *n)
{
    if (!n->prof_on) return;
    if (n->prof_used == n->prof_cap) {
        uint32_t cap = n->prof_cap ? n->prof_cap * 2 : 16;
        void **ev = realloc(n->prof_ev, cap * sizeof *ev);
        if (!ev) return;
        for (uint32_t i = n->prof_cap; i < cap; i++) ev[i] = NULL;
        n->prof_ev = ev; n->prof_cap = cap;
    }
    if (!n->prof_ev[n->prof_used] && spgk_event_create(&n->prof_ev[n->prof_used]) != SPGK_OK) return;
    spgk_event_record(n->prof_ev[n->prof_used], n->stream);
    n->prof_used++;
}

/* after the stream has been synchronised: add up the (start, stop) pairs */
static void prof_collect(spg_net *n)
{
    for (uint32_t i = 0; i + 1 < n->prof_used; i += 2) {
        float ms = 0.0f;
        if (spgk_event_elapsed_ms(n->prof_ev[i], n->prof_ev[i + 1], &ms) == SPGK_OK) { n->prof_ms += ms; n->prof_launches++; }
    }
    n->prof_used = 0;
}

/* grow-only device buffer */
static int reserve(void **buf, size_t *have, size_t need, const char *what)
{
    if (*have >= need && *buf) return SPINGALETT_OK;
    spgk_free(*buf); *buf = NULL; *have = 0;
    int rc = spg_map_kernel_error(spgk_malloc(buf, need), what);
    if (rc == SPINGALETT_OK) *have = need;
    return rc;
}

/* ------------------------------------------------------------------------ */
/* small-batch chain                                                         */
/* ------------------------------------------------------------------------ */

/* device buffer that must start zero-filled (status words, ticket counters) */
static int reserve_zeroed(spg_net *n, void **buf, size_t *have, size_t need, const char *what)
{
    if (!need || (*have >= need && *buf)) return SPINGALETT_OK;
    int rc = reserve(buf, have, need, what);
    if (rc) return rc;
    return spg_map_kernel_error(spgk_memset(*buf, 0, need, n->stream), what);
}

static int small_reserve(spg_net *n, uint32_t N)
{
    NeuralNetwork *p = &n->pub;
    if (n->small_cap < N || !n->d_small) {
        spgk_free(n->d_small); n->d_small = NULL; n->small_cap = 0;
        void *b = NULL;
        int rc = spg_map_kernel_error(spgk_malloc(&b, (size_t)N * p->total_neurons * sizeof(float)), "small-batch workspace");
        if (rc) return rc;
        n->d_small = b; n->small_cap = N;
    }
    size_t gemv = 0, staged = 0, ws = 0, operand = 0;
    for (uint32_t l = 0; l < n->dev_layers; l++) {
        const spgk_layer *L = &n->klayers[l];
        size_t s = N <= SPGK_GEMV_MAX_BATCH ? spgk_gemv_scratch_bytes(L, N) : 0;
        if (s) {
            if (s > gemv) gemv = s;
            s = spgk_gemv_staged_bytes(L->in, N);
            if (s > staged) staged = s;
            continue;
        }
        s = spgk_wstream_scratch_bytes(L, N);
        if (s > ws) ws = s;
        if (s && (s = spgk_wstream_operand_bytes(L->in, N)) > operand) operand = s;
    }
    int rc;
    for (int i = 0; i < 2; i++) {
        if (staged && (rc = reserve(&n->d_staged[i], &n->staged_bytes[i], staged, "gemv staged input"))) return rc;
        if (operand && (rc = reserve(&n->d_operand[i], &n->operand_bytes[i], operand, "activation operand"))) return rc;
    }
    if ((rc = reserve_zeroed(n, &n->d_gemv_scratch, &n->gemv_scratch_bytes, gemv, "gemv scratch"))) return rc;
    return reserve_zeroed(n, &n->d_ws_scratch, &n->ws_scratch_bytes, ws, "weight-stream scratch");
}

/* 1 if every layer can run on the weight-streaming tensor-core kernel at this batch */
static bool all_wstream(const spg_net *n, uint32_t N)
{
    for (uint32_t l = 0; l < n->dev_layers; l++)
        if (!spgk_wstream_scratch_bytes(&n->klayers[l], N)) return false;
    return true;
}

/* Small / medium batches (fp32 activations between layers; every layer streams its packed weights once).
 * Per layer, in order of preference: the weight-streaming tcgen05 kernel, the mma.sync GEMV (<= 8 rows),
 * the general SIMT kernel.  d_x == NULL means the caller already placed the input rows in slot 0 of the
 * workspace (after a reservation-only call, see forward()). */
int spg_dev_forward_small(spg_net *n, const float *d_x, uint32_t ldx, uint32_t N, float **d_last, float *d_final)
{
    NeuralNetwork *p = &n->pub;
    int rc = small_reserve(n, N);
    if (rc) return rc;
    if (!d_last) return SPINGALETT_OK;          /* reservation only */
    const float *x = d_x ? d_x : n->d_small;
    uint32_t xld = d_x ? ldx : p->topology[0];
    const char *path = NULL;
    const void *staged = NULL, *operand = NULL;      /* input of the layer in flight, already in a kernel's own order */
    if (N <= SPGK_GEMV_MAX_BATCH && n->dev_layers <= 8 && n->d_staged[0] && n->d_staged[1] && n->d_gemv_scratch) {
        /* every layer in one launch when the kernel takes them all: the weight stream then runs through the layer boundaries */
        float *ys[8];
        for (uint32_t l = 0; l < n->dev_layers; l++)
            ys[l] = (d_final && l + 1 == n->dev_layers) ? d_final : n->d_small + (size_t)N * p->neuron_offsets[l + 1];
        prof_mark(n);
        int k = spgk_gemv_forward_chain(n->klayers, n->dev_layers, x, xld, ys, N, n->d_staged[0], n->d_staged[1], n->d_gemv_scratch, n->stream);
        prof_mark(n);
        if (k == SPGK_OK) {
            n->gemv_pending = true;
            const spgk_layer *Ll = &n->klayers[n->dev_layers - 1];
            if (Ll->act == ACT_SOFTMAX && !spgk_gemv_applies_softmax(N) &&
                (rc = spg_map_kernel_error(spgk_softmax_rows(ys[n->dev_layers - 1], Ll->out, N, Ll->out, n->stream), "softmax"))) return rc;
            spg_note_path("gemv");
            *d_last = ys[n->dev_layers - 1];
            return SPINGALETT_OK;
        }
        if (n->prof_used >= 2) n->prof_used -= 2;          /* nothing was launched between the two marks */
        if (k != SPGK_E_UNSUPPORTED && (rc = spg_map_kernel_error(k, "layers (small batch)"))) return rc;
    }
    for (uint32_t l = 0; l < n->dev_layers; l++) {
        const spgk_layer *L = &n->klayers[l];
        const spgk_layer *next = l + 1 < n->dev_layers ? &n->klayers[l + 1] : NULL;
        float *y = (d_final && l + 1 == n->dev_layers) ? d_final : n->d_small + (size_t)N * p->neuron_offsets[l + 1];
        /* up to 8 rows: the mma.sync GEMV first (measured faster there), then the tcgen05 streaming kernel;
         * more rows: the streaming kernel only */
        const char *used = "gemv";
        int k = SPGK_E_UNSUPPORTED;
        prof_mark(n);
        if (N <= SPGK_GEMV_MAX_BATCH) {
            k = spgk_layer_gemv_chain(L, next, staged, n->d_staged[(l + 1) & 1], x, xld, y, L->out, N, n->d_gemv_scratch, n->stream);
            if (k == SPGK_OK) n->gemv_pending = true;
        }
        if (k == SPGK_E_UNSUPPORTED) {
            used = "wstream";
            k = spgk_layer_wstream(L, next, operand, n->d_operand[(l + 1) & 1], x, xld, y, L->out, N, n->d_ws_scratch, n->stream);
            if (k == SPGK_OK) n->ws_pending = true;
        }
        operand = (k == SPGK_OK && used[0] == 'w' && next && spgk_wstream_stages_next(L, next, N)) ? n->d_operand[(l + 1) & 1] : NULL;
        staged = (k == SPGK_OK && used[0] == 'g' && next && spgk_gemv_chain_stages_next(L, next, N)) ? n->d_staged[(l + 1) & 1] : NULL;
        prof_mark(n);
        if (k == SPGK_E_UNSUPPORTED) {
            if (n->prof_used >= 2) n->prof_used -= 2;      /* nothing was launched between the two marks */
            used = "simt";
            k = spgk_layer_simt(L, x, xld, y, L->out, N, n->stream);
        }
        if ((rc = spg_map_kernel_error(k, "layer (small batch)"))) return rc;
        /* at one row the GEMV applies the softmax itself (its last CTA to finish does it); otherwise the layer left logits */
        if (L->act == ACT_SOFTMAX && !(used[0] == 'g' && spgk_gemv_applies_softmax(N)) &&
            (rc = spg_map_kernel_error(spgk_softmax_rows(y, L->out, N, L->out, n->stream), "softmax"))) return rc;
        if (!path || used[0] == 's' || (used[0] == 'w' && path[0] == 'g')) path = used;    /* report the most general kernel used */
        x = y; xld = L->out;
    }
    spg_note_path(path ? path : "none");
    *d_last = d_final ? d_final : n->d_small + (size_t)N * p->neuron_offsets[p->layers - 1];
    return SPINGALETT_OK;
}

/* ------------------------------------------------------------------------ */
/* large-batch chain                                                         */
/* ------------------------------------------------------------------------ */

static uint32_t round8(uint32_t v) { return (v + 7u) & ~7u; }

/* Expanded 16-bit weight operands are kept between calls up to this many bytes per net and type (4 GiB unless
 * SPINGALETT_W16_KEEP_MB says otherwise; 0 = expand per call).  A quantised file costs up to 4x (INT4) or 8x (INT2) its
 * packed size per kept type; nets beyond the budget are expanded into a scratch buffer on every call. */
static size_t w16_keep_max(void)
{
    static size_t cached = (size_t)-1;
    if (cached == (size_t)-1) {
        const char *e = getenv("SPINGALETT_W16_KEEP_MB");
        cached = (e && *e) ? (size_t)strtoull(e, NULL, 10) << 20 : (size_t)4096 << 20;
    }
    return cached;
}
#define SPG_W16_KEEP_MAX w16_keep_max()    /* keep expanded 16-bit weight operands between calls up to this many bytes per net and type */

static int large_simt(spg_net *n, const float *d_x, uint32_t N, float *d_out)
{
    NeuralNetwork *p = &n->pub;
    uint32_t maxw = 0;
    for (uint32_t l = 1; l < p->layers; l++) if (p->topology[l] > maxw) maxw = p->topology[l];
    size_t need = (size_t)N * maxw * sizeof(float);
    if (n->act32_bytes < need) {
        for (int i = 0; i < 2; i++) { spgk_free(n->d_act32[i]); n->d_act32[i] = NULL; }
        n->act32_bytes = 0;
        for (int i = 0; i < 2; i++) {
            void *b = NULL;
            int rc = spg_map_kernel_error(spgk_malloc(&b, need), "fp32 activation workspace");
            if (rc) return rc;
            n->d_act32[i] = b;
        }
        n->act32_bytes = need;
    }
    const float *x = d_x;
    uint32_t xld = p->topology[0];
    for (uint32_t l = 0; l < n->dev_layers; l++) {
        const spgk_layer *L = &n->klayers[l];
        bool last = l + 1 == n->dev_layers;
        float *y = last ? d_out : n->d_act32[l & 1];
        int rc = spg_map_kernel_error(spgk_layer_simt(L, x, xld, y, L->out, N, n->stream), "layer (simt)");
        if (rc) return rc;
        if (L->act == ACT_SOFTMAX && (rc = spg_map_kernel_error(spgk_softmax_rows(y, L->out, N, L->out, n->stream), "softmax"))) return rc;
        x = y; xld = L->out;
    }
    spg_note_path("simt");
    return SPINGALETT_OK;
}

/* The 16-bit K-major operand of layer l in flavour `type` with `w_parts` planes: the stored payload itself when
 * TMA can read it in place, else an expansion that is made once and kept with the net (while the whole net's
 * expansions stay below SPG_W16_KEEP_MAX; `keep` says so), else *w16 = NULL and the caller expands per call. */
static int kept_weight_operand(spg_net *n, int type, uint32_t l, int w_parts, bool keep, const void **w16, uint32_t *ldw, uint64_t *w_plane)
{
    const spgk_layer *L = &n->klayers[l];
    int rc;
    *w16 = NULL;
    if (spgk_weights16_direct(L, type)) { *w16 = L->w; *ldw = L->in; *w_plane = 0; return SPINGALETT_OK; }
    *ldw = round8(L->in);
    *w_plane = (uint64_t)L->out * *ldw;
    if (!keep) return SPINGALETT_OK;
    if (!n->d_w16c[type]) {
        n->d_w16c[type] = calloc(n->dev_layers, sizeof(void *));
        n->w16c_parts[type] = calloc(n->dev_layers, 1);
        if (!n->d_w16c[type] || !n->w16c_parts[type]) { spg_set_error(SPINGALETT_ERR_ALLOC, "weight operand table"); return SPINGALETT_ERR_ALLOC; }
    }
    if (n->d_w16c[type][l] && n->w16c_parts[type][l] != w_parts) { spgk_free(n->d_w16c[type][l]); n->d_w16c[type][l] = NULL; }
    if (!n->d_w16c[type][l]) {
        if ((rc = spg_map_kernel_error(spgk_malloc(&n->d_w16c[type][l], spgk_weights16_bytes(L, w_parts)), "kept weight operand"))) return rc;
        n->w16c_parts[type][l] = (uint8_t)w_parts;
        if ((rc = spg_map_kernel_error(spgk_dequant16(L, n->d_w16c[type][l], *ldw, *w_plane, w_parts, type, n->stream), "weight operand"))) return rc;
    }
    *w16 = n->d_w16c[type][l];
    return SPINGALETT_OK;
}

/* whether the expanded 16-bit operands of the whole net (flavour `type`) are small enough to keep between calls */
static bool weights_keepable(const spg_net *n, int type, bool exact)
{
    size_t wtotal = 0;
    for (uint32_t l = 0; l < n->dev_layers; l++) {
        const spgk_layer *L = &n->klayers[l];
        if (!spgk_weights16_direct(L, type)) wtotal += spgk_weights16_bytes(L, (exact && L->precision == PRECISION_FLOAT32) ? 2 : 1);
    }
    return wtotal <= SPG_W16_KEEP_MAX;
}

/* The one-term pass of a BF16 file takes fp16 operands when every weight is within fp16's range (any trained or
 * initialised net: the check is one pass over the host mirror, once per upload): fp16 carries 11 significant bits of an
 * activation against bf16's 8, an eighth of the rounding error, so AUTO lists about an eighth of the rows for the exact
 * recomputation (which keeps bf16: two terms, fp32 range).  bf16 weights are exact in fp16 down to 6.1e-5; smaller
 * ones keep an absolute error below 6e-8. */
static bool bf16_file_as_f16(spg_net *n)
{
    if (!n->bf16_fits_f16) {
        const NeuralNetwork *p = &n->pub;
        float mx = 0.0f;
        bool finite = true;
        for (uint64_t i = 0; i < p->total_weights; i++) {
            const float a = fabsf(p->weights[i]);
            if (!(a <= 3.0e38f)) finite = false;
            if (a > mx) mx = a;
        }
        n->bf16_fits_f16 = (finite && mx < 60000.0f) ? 1 : 2;
    }
    return n->bf16_fits_f16 == 1;
}

static _Thread_local bool dynamic_rows = false;      /* true around the repair chain of the AUTO mode */
static _Thread_local const uint32_t *repair_rows = NULL;   /* repair chain: input row i is row repair_rows[i] of d_x, and its result goes back there */

static int large_chain(spg_net *n, const float *d_x, uint32_t N, float *d_out, bool exact)
{
    NeuralNetwork *p = &n->pub;
    bool tc = true;
    for (uint32_t l = 0; l < n->dev_layers; l++) tc = tc && spgk_gemm_tc_supported(&n->klayers[l]);
    for (uint32_t l = 0; l + 1 < n->dev_layers; l++) tc = tc && n->klayers[l].act != ACT_SOFTMAX;   /* softmax only as the last layer */
    if (!tc) return large_simt(n, d_x, N, d_out);

    const int prec = n->klayers[0].precision;
    /* 16-bit flavour: the file's own 16-bit type when it has one (exact
     * weights); otherwise fp16 for the one-term mode (11 significant bits) and
     * bf16 for the two-term mode (fp32 range, 16 bits over two terms). */
    const int type = prec == PRECISION_FP16 ? SPGK_T_F16
                   : prec == PRECISION_BFLOAT16 ? ((exact || !bf16_file_as_f16(n)) ? SPGK_T_BF16 : SPGK_T_F16)
                   : exact ? SPGK_T_BF16 : SPGK_T_F16;
    const int parts = exact ? 2 : 1;
    uint32_t maxld = 0;
    for (uint32_t l = 0; l + 1 < p->layers; l++) if (round8(p->topology[l]) > maxld) maxld = round8(p->topology[l]);
    const uint64_t plane = (uint64_t)N * maxld;
    size_t need = (size_t)plane * 2u * (size_t)parts;
    if (n->act16_bytes < need) {
        for (int i = 0; i < 2; i++) { spgk_free(n->d_act16[i]); n->d_act16[i] = NULL; }
        n->act16_bytes = 0;
        for (int i = 0; i < 2; i++) {
            int rc = spg_map_kernel_error(spgk_malloc(&n->d_act16[i], need), "16-bit activation workspace");
            if (rc) return rc;
        }
        n->act16_bytes = need;
    }
    /* 16-bit weight operand of layers that are not stored as one: expanded once and kept while the whole net's
     * operands fit the budget below (the benchmark MLP: 1.8 MB), otherwise expanded into a scratch per call */
    size_t wneed = 0, wtotal = 0;
    for (uint32_t l = 0; l < n->dev_layers; l++) {
        const spgk_layer *L = &n->klayers[l];
        if (!spgk_weights16_direct(L, type)) {
            size_t b = spgk_weights16_bytes(L, (exact && L->precision == PRECISION_FLOAT32) ? 2 : 1);
            if (b > wneed) wneed = b;
            wtotal += b;
        }
    }
    const bool keep = wtotal && wtotal <= SPG_W16_KEEP_MAX;
    int rc;
    if (!keep && wneed && (rc = reserve(&n->d_w16, &n->w16_bytes, wneed, "16-bit weight operand scratch"))) return rc;
    rc = spg_map_kernel_error(spgk_split16_rows(d_x, p->topology[0], repair_rows, N, p->topology[0], n->d_act16[0],
                                                round8(p->topology[0]), plane, parts, type, n->stream), "input split");
    if (rc) return rc;
    for (uint32_t l = 0; l < n->dev_layers; l++) {
        const spgk_layer *L = &n->klayers[l];
        bool last = l + 1 == n->dev_layers;
        bool fuse_sm = L->act == ACT_SOFTMAX && spgk_gemm_tc_softmax_fusable(L->out, N, dynamic_rows ? 1 : 0);
        void *o16 = last ? NULL : n->d_act16[(l + 1) & 1];
        float *o32 = last ? d_out : NULL;
        const void *w16 = NULL;
        uint32_t ldw = 0;
        uint64_t w_plane = 0;
        const int w_parts = (!spgk_weights16_direct(L, type) && exact && L->precision == PRECISION_FLOAT32) ? 2 : 1;
        if ((rc = kept_weight_operand(n, type, l, w_parts, keep, &w16, &ldw, &w_plane))) return rc;
        if (!w16) {
            w16 = n->d_w16;
            if ((rc = spg_map_kernel_error(spgk_dequant16(L, n->d_w16, ldw, w_plane, w_parts, type, n->stream), "weight operand"))) return rc;
        }
        /* Measured on the benchmark MLP at 65536 rows: it wins in the two-term mode (141.8 us against 155.5 us for two
         * kernels), ties in the one-term mode where the epilogue's fp32 FMAs become the limit (106.7 / 105.4 us), and
         * loses for few rows, because a CTA owns whole row tiles there: so only full exact passes over large batches. */
        if (l + 2 == n->dev_layers && exact && !dynamic_rows && N >= 16384 && spgk_gemm_tc_head_supported(L, &n->klayers[l + 1])) {
            /* the narrow last layer rides in this layer's epilogue: its input matrix is never written */
            const spgk_layer *H = &n->klayers[l + 1];
            if (!n->d_head_w) {
                void *hw = NULL;
                if ((rc = spg_map_kernel_error(spgk_malloc(&hw, spgk_head_weights_bytes(H)), "head weights"))) return rc;
                n->d_head_w = hw;
                if ((rc = spg_map_kernel_error(spgk_head_weights(H, n->d_head_w, n->stream), "head weights"))) return rc;
            }
            prof_mark(n);
            rc = spg_map_kernel_error(spgk_layer_gemm_tc_head(L, w16, ldw, w_plane, w_parts, type,
                                                              n->d_act16[l & 1], round8(L->in), plane, parts, type,
                                                              H, n->d_head_w, d_out, H->out, N, n->d_status, n->stream), "layer + head (tcgen05)");
            prof_mark(n);
            if (rc) return rc;
            break;
        }
        if (!dynamic_rows) prof_mark(n);                 /* the timing marks cover the full passes, not the repair of a few rows */
        if (last) spgk_set_output_rows(repair_rows);
        rc = spg_map_kernel_error(spgk_layer_gemm_tc(L, w16, ldw, w_plane, w_parts, type,
                                                     n->d_act16[l & 1], round8(L->in), plane, parts, type,
                                                     o16, round8(L->out), plane, parts, o32, L->out,
                                                     N, (last && fuse_sm) ? 1 : 0, n->d_status, n->stream), "layer (tcgen05)");
        spgk_set_output_rows(NULL);
        if (!dynamic_rows) prof_mark(n);
        if (rc) return rc;
        if (last && L->act == ACT_SOFTMAX && !fuse_sm &&
            (rc = spg_map_kernel_error(spgk_softmax_rows(d_out, L->out, N, L->out, n->stream), "softmax"))) return rc;
    }
    n->status_pending = true;
    spg_note_path("tcgen05");
    return SPINGALETT_OK;
}

/* ---- the three-layer net in one launch ------------------------------------ */

#define SPG_AUTO_EXACT_ROWS 512u     /* AUTO runs batches of up to this many rows in EXACT */
#define SPG_AUTO_RECAL 1024u         /* large AUTO calls between two measurements of the margin */
#define SPG_FUSED_MIN_ROWS 1024u     /* below this a handful of 128-row tiles cannot fill the GPU: the per-layer chain spreads better */

/* 16-bit flavour of the one-term pass: fp16, except for a BF16 file with weights beyond fp16's range */
static int fast_type(spg_net *n)
{
    const int prec = n->klayers[0].precision;
    return prec == PRECISION_BFLOAT16 && !bf16_file_as_f16(n) ? SPGK_T_BF16 : SPGK_T_F16;
}

static bool fused_eligible(spg_net *n, const float *d_x, uint32_t N)
{
    if (n->dev_layers != 3 || N < SPG_FUSED_MIN_ROWS || ((uintptr_t)d_x & 15u)) return false;
    if (!spgk_mlp3_supported(&n->klayers[0], &n->klayers[1], &n->klayers[2], n->pub.topology[0])) return false;
    return weights_keepable(n, fast_type(n), false);
}

/* one launch over N rows (or over the rows of a device-resident list): the one-term pass, or with pairs the
 * two-term recomputation of the listed rows written over their one-term results */
static int fused_pass(spg_net *n, const float *d_x, uint32_t N, float *d_out, bool pairs,
                      const uint32_t *rows_idx, const uint32_t *rows_limit, uint32_t expected,
                      float theta, uint32_t *margin_idx, uint32_t *margin_count)
{
    const int type = fast_type(n);
    const spgk_layer *L1 = &n->klayers[0], *L2 = &n->klayers[1], *L3 = &n->klayers[2];
    int rc;
    if (!n->d_fused_params) {
        void *b = NULL;
        if ((rc = spg_map_kernel_error(spgk_malloc(&b, spgk_mlp3_params_bytes(L1, L2, L3)), "fused MLP parameters"))) return rc;
        n->d_fused_params = b;
        if ((rc = spg_map_kernel_error(spgk_mlp3_params(L1, L2, L3, type, n->d_fused_params, n->stream), "fused MLP parameters"))) return rc;
    }
    const void *w1 = NULL, *w2 = NULL;
    uint32_t ld1 = 0, ld2 = 0;
    uint64_t plane = 0;
    if ((rc = kept_weight_operand(n, type, 0, 1, true, &w1, &ld1, &plane))) return rc;
    if ((rc = kept_weight_operand(n, type, 1, 1, true, &w2, &ld2, &plane))) return rc;
    prof_mark(n);
    rc = spg_map_kernel_error(spgk_mlp3_forward(L1, w1, ld1, L2, w2, ld2, L3, n->d_fused_params, type,
                                                d_x, n->pub.topology[0], rows_idx, rows_limit, expected, pairs ? 1 : 0,
                                                d_out, L3->out, N, theta, margin_idx, margin_count, n->d_status, n->stream),
                              "three-layer MLP (tcgen05)");
    prof_mark(n);
    if (rc) return rc;
    n->status_pending = true;
    n->fused_ran = true;
    spg_note_path("tcgen05-fused");
    return SPINGALETT_OK;
}

/* Large-batch forward in the selected math mode.  AUTO = the one-term pass, then an exact recomputation of
 * the rows whose top-two softmax outputs are within the margin (their argmax is the only thing the one-term
 * pass could have changed), written over the fast result. */
int spg_dev_forward_large(spg_net *n, const float *d_x, uint32_t N, float *d_out)
{
    NeuralNetwork *p = &n->pub;
    const SpingalettMathMode mode = spingalett_get_math_mode();
    const uint32_t in0 = p->topology[0], outw = p->topology[p->layers - 1];
    const bool softmax_out = p->act_func[p->layers - 2] == ACT_SOFTMAX && outw >= 2;
    /* a three-layer net with a narrow last layer runs its one-term passes as ONE kernel (no activation matrix in HBM) */
    const bool fused = fused_eligible(n, d_x, N);
    if (mode == SPINGALETT_MATH_FAST && fused) return fused_pass(n, d_x, N, d_out, false, NULL, NULL, 0, 0.0f, NULL, NULL);
    if (mode != SPINGALETT_MATH_AUTO) return large_chain(n, d_x, N, d_out, mode == SPINGALETT_MATH_EXACT);
    if (!softmax_out) return large_chain(n, d_x, N, d_out, true);
    /* Few rows: the chain is bound by streaming the weights (or by latency), where the exact chain's second pass over K
     * is nearly free, while the one-term pass plus the recomputation chain costs two chains: 0.70 ms against 1.05 ms at
     * 256 rows of the large INT4 net, 1.00 against 1.20 at 512 (the curves cross near 700 rows). */
    if (N <= SPG_AUTO_EXACT_ROWS) return large_chain(n, d_x, N, d_out, true);

    int rc;
    if ((rc = reserve((void **)&n->d_rep_idx, &n->rep_idx_bytes, (size_t)N * 4 + 256, "repair index"))) return rc;
    uint32_t *d_count = n->d_rep_idx + N;
    float theta = spingalett_get_auto_margin();
    if (theta <= 0.0f && n->auto_calibrated) theta = n->auto_theta;
    /* with the margin known in advance, the softmax epilogue of the last layer picks the rows out itself */
    const spgk_layer *Llast = &n->klayers[n->dev_layers - 1];
    const bool sink = theta > 0.0f && (fused || spgk_gemm_tc_softmax_fusable(Llast->out, N, 0));
    if (sink && (rc = spg_map_kernel_error(spgk_memset(d_count, 0, 4, n->stream), "repair count clear"))) return rc;
    if (fused) {
        rc = fused_pass(n, d_x, N, d_out, false, NULL, NULL, 0, theta, sink ? n->d_rep_idx : NULL, sink ? d_count : NULL);
    } else {
        if (sink) spgk_set_margin_sink(theta, n->d_rep_idx, d_count);
        rc = large_chain(n, d_x, N, d_out, false);
        spgk_set_margin_sink(0.0f, NULL, NULL);
    }
    if (rc) return rc;
    if (strncmp(spingalett_last_path(), "tcgen05", 7) != 0) return SPINGALETT_OK;  /* the fp32 chain ran: nothing to repair */
    const bool fused_pass_ran = fused;
    theta = spingalett_get_auto_margin();
    if (theta <= 0.0f) {
        /* Self-calibration, once per device image of the net: run both modes on up to 2048 rows, measure the
         * largest change of the top-two log gap the one-term pass causes, and use four times that as margin. */
        /* ... and again on every SPG_AUTO_RECAL-th call, on that call's rows: the margin only ever grows, so inputs that
         * have drifted to where the one-term pass errs more widen it (one extra exact pass over 2048 rows and a host
         * read, a millisecond in a thousand calls) */
        const bool again = n->auto_calibrated && ++n->auto_calls % SPG_AUTO_RECAL == 0;
        if (!n->auto_calibrated || again) {
            const uint32_t rows = N < 2048 ? N : 2048;
            if ((rc = reserve((void **)&n->d_rep_out, &n->rep_out_bytes, (size_t)rows * outw * 4, "calibration outputs"))) return rc;
            if ((rc = large_chain(n, d_x, rows, n->d_rep_out, true))) return rc;          /* exact rows; d_out already holds the fast ones */
            /* (a word of its own: on a repeated measurement d_count already holds this call's number of listed rows) */
            uint32_t *d_gap = d_count + 8;
            if ((rc = spg_map_kernel_error(spgk_memset(d_gap, 0, 4, n->stream), "calibration clear"))) return rc;
            if ((rc = spg_map_kernel_error(spgk_gap_error(d_out, n->d_rep_out, outw, rows, outw, d_gap, n->stream), "calibration"))) return rc;
            float emax = 0.0f;
            if ((rc = spg_map_kernel_error(spgk_memcpy_d2h(&emax, d_gap, 4, n->stream), "calibration read"))) return rc;
            if ((rc = spg_map_kernel_error(spgk_stream_sync(n->stream), "calibration sync"))) return rc;
            const float measured = emax * 4.0f > 1e-4f ? emax * 4.0f : 1e-4f;
            n->auto_theta = again && n->auto_theta > measured ? n->auto_theta : measured;
            n->auto_calibrated = true;
            spg_log(LOG_DEBUG, "auto math mode: largest top-two log-gap change on %u rows %.3g, margin %.3g", rows, (double)emax, (double)n->auto_theta);
        }
        theta = n->auto_theta;
    }
    if (!sink) {
        if ((rc = spg_map_kernel_error(spgk_memset(d_count, 0, 4, n->stream), "repair count clear"))) return rc;
        if ((rc = spg_map_kernel_error(spgk_margin_select(d_out, outw, N, outw, theta, n->d_rep_idx, d_count, n->stream), "margin check"))) return rc;
    }
    /* The row count stays on the device: the gather, the exact chain and the scatter below are launched for
     * N rows of capacity and read the count when they run, so the call needs no host round trip.  A copy
     * travels to pinned host memory for spingalett_last_repaired(). */
    if (!n->h_count) {
        void *h = NULL;
        if ((rc = spg_map_kernel_error(spgk_host_alloc(&h, 256), "repair count (host)"))) return rc;
        n->h_count = h;
        memset(h, 0, 256);
    }
    uint32_t *h_slot = n->h_count + n->count_slot;
    const uint32_t expected = n->count_seen ? *(volatile uint32_t *)h_slot : 0;    /* the count of the call before: a guide to tile shapes only */
    /* (the copy is queued behind the repair kernels: nothing sits between the one-term pass and the repair, so the
     * repair's prologue overlaps the tail of the pass under programmatic dependent launch) */
    if (n->count_slot + 1 > n->count_slots_used) n->count_slots_used = n->count_slot + 1;
    if (Llast->act == ACT_SOFTMAX && Llast->out > spgk_gemm_tc_softmax_max()) {
        if ((rc = reserve((void **)&n->d_rep_in, &n->rep_in_bytes, (size_t)N * in0 * 4, "repair inputs"))) return rc;
        if ((rc = reserve((void **)&n->d_rep_out, &n->rep_out_bytes, (size_t)N * outw * 4, "repair outputs"))) return rc;
    }
    /* The flagged rows are a percent or two of the batch, so either repair is one latency-bound pass over a handful of
     * tiles.  Measured on the benchmark MLP at 65536 rows: the per-layer exact chain takes 67 us, the one-launch kernel
     * in pair mode 93 us (a single 128-row tile runs its 13 + 32 k-blocks and six epilogues back to back), so the chain
     * is the default; SPINGALETT_REPAIR=fused selects the other for comparisons. */
    static int repair_fused = -1;
    if (repair_fused < 0) { const char *e = getenv("SPINGALETT_REPAIR"); repair_fused = (e && strcmp(e, "fused") == 0) ? 1 : 0; }
    if (fused && repair_fused && n->klayers[0].precision != PRECISION_FLOAT32) {
        /* files whose weights are exact in 16 bits: the flagged rows again through the same kernel, each as a
         * hi/lo pair of tile rows, written over their one-term results */
        if ((rc = fused_pass(n, d_x, N, d_out, true, n->d_rep_idx, d_count, expected, 0.0f, NULL, NULL))) return rc;
        if ((rc = spg_map_kernel_error(spgk_memcpy_d2h(h_slot, d_count, 4, n->stream), "repair count"))) return rc;
        n->count_pending = true; n->count_seen = true;
        return SPINGALETT_OK;
    }
    spgk_set_dynamic_rows(d_count, expected);
    dynamic_rows = true;
    if (Llast->act != ACT_SOFTMAX || Llast->out <= spgk_gemm_tc_softmax_max()) {
        /* the split reads the flagged rows in place and the last layer's epilogue writes them back in place */
        repair_rows = n->d_rep_idx;
        rc = large_chain(n, d_x, N, d_out, true);
        repair_rows = NULL;
    } else {
        rc = spg_map_kernel_error(spgk_gather_rows(d_x, n->d_rep_idx, n->d_rep_in, N, in0, n->stream), "repair gather");
        if (!rc) rc = large_chain(n, n->d_rep_in, N, n->d_rep_out, true);
        if (!rc) rc = spg_map_kernel_error(spgk_scatter_rows(n->d_rep_out, n->d_rep_idx, d_out, N, outw, outw, n->stream), "repair scatter");
    }
    spgk_set_dynamic_rows(NULL, 0);
    dynamic_rows = false;
    if (rc) return rc;
    if ((rc = spg_map_kernel_error(spgk_memcpy_d2h(h_slot, d_count, 4, n->stream), "repair count"))) return rc;
    n->count_pending = true; n->count_seen = true;
    spg_note_path(fused_pass_ran ? "tcgen05-fused" : "tcgen05");
    return SPINGALETT_OK;
}

/* ------------------------------------------------------------------------ */
/* batched inference entry point                                             */
/* ------------------------------------------------------------------------ */

static float *forward_batch_on(spg_net *n, ForwardBatchArgs a);

/* A pageable source is copied into page-locked staging by several host threads at once: one thread (what a cudaMemcpy
 * from pageable memory amounts to) moves about 11 GB/s, a third of what the host link takes. */
#define SPG_STAGE_THREADS 16    /* most; SPINGALETT_STAGE_THREADS in the environment asks for fewer */
typedef struct { char *dst; const char *src; size_t bytes; } stage_job;
static void *stage_worker(void *arg)
{
    stage_job *j = arg;
    memcpy(j->dst, j->src, j->bytes);
    return NULL;
}
static void stage_copy(void *dst, const void *src, size_t bytes)
{
    static int want = 0;
    if (!want) {
        const char *e = getenv("SPINGALETT_STAGE_THREADS");
        const long cores = sysconf(_SC_NPROCESSORS_ONLN);
        want = e && atoi(e) > 0 ? atoi(e) : (cores >= 16 ? 8 : cores >= 4 ? (int)(cores / 2) : 1);
        if (want > SPG_STAGE_THREADS) want = SPG_STAGE_THREADS;
    }
    int nt = want;
    if (bytes < ((size_t)4 << 20)) nt = 1;
    pthread_t th[SPG_STAGE_THREADS];
    stage_job jobs[SPG_STAGE_THREADS];
    const size_t share = ((bytes / (size_t)nt) + 4095) & ~(size_t)4095;
    int started = 0;
    for (int t = 1; t < nt; t++) {
        const size_t off = (size_t)t * share;
        if (off >= bytes) break;
        jobs[t] = (stage_job){ (char *)dst + off, (const char *)src + off, bytes - off < share ? bytes - off : share };
        if (pthread_create(&th[t], NULL, stage_worker, &jobs[t]) != 0) {        /* no thread: this one copies the rest */
            memcpy((char *)dst + off, (const char *)src + off, bytes - off);
            break;
        }
        started = t;
    }
    memcpy(dst, src, bytes < share || nt == 1 ? bytes : share);
    for (int t = 1; t <= started; t++) pthread_join(th[t], NULL);
}

/* a replica record for device `dev`: shares the host arrays and the packed payload of `n`, owns its device image */
static spg_net *shadow_for(spg_net *n, int slot, int dev)
{
    spg_net *sh = n->shadow[slot];
    if (sh && sh->device == dev) return sh;
    if (sh) { spg_dev_release(sh); spgk_host_free(sh->h_out); free(sh); n->shadow[slot] = NULL; }
    sh = calloc(1, sizeof *sh);
    if (!sh) return NULL;
    sh->pub = n->pub;
    sh->magic = n->magic;
    sh->is_shadow = true;
    sh->store_precision = n->store_precision;
    sh->payload_w = n->payload_w; sh->payload_w_bytes = n->payload_w_bytes; sh->amax_w = n->amax_w; sh->payload_layers = n->payload_layers;
    sh->device = dev;
    sh->auto_calibrated = n->auto_calibrated; sh->auto_theta = n->auto_theta;
    n->shadow[slot] = sh;
    return sh;
}

typedef struct { spg_net *net; ForwardBatchArgs args; int rc; char msg[SPG_ERRMSG_MAX]; } fan_job;

static void *fan_worker(void *arg)
{
    fan_job *j = arg;
    spingalett_clear_error();
    j->rc = forward_batch_on(j->net, j->args) ? SPINGALETT_OK : spingalett_last_error_code();
    if (j->rc) {                                  /* the error state is per thread: hand the text to the caller */
        const char *m = spingalett_last_error_message();
        strncpy(j->msg, m ? m : "", sizeof j->msg - 1);
        if (j->rc == SPINGALETT_OK) j->rc = SPINGALETT_ERR_DEVICE;
    }
    return NULL;
}

float *forward_batch_struct_arguments(ForwardBatchArgs a)
{
    NeuralNetwork *p = a.net;
    if (!p || !a.inputs) { spg_set_error(SPINGALETT_ERR_INVALID, "forward_batch: net or inputs is NULL"); return NULL; }
    if (p->layers < 2) { spg_set_error(SPINGALETT_ERR_INVALID, "Network must have at least 2 layers for forward pass"); return NULL; }
    spg_net *n = spg_priv(p);
    int ids[SPG_MAX_FANOUT], G;
    pthread_mutex_lock(&g_fan_lock);
    G = g_fan_n;
    memcpy(ids, g_fan_ids, sizeof ids);
    pthread_mutex_unlock(&g_fan_lock);
    const bool host_in = spgk_is_device_pointer(a.inputs) != 1, host_out = !a.outputs || spgk_is_device_pointer(a.outputs) != 1;
    if (G < 2 || !host_in || !host_out || a.sample_count < 2u * (uint32_t)G) return forward_batch_on(n, a);

    /* fan-out: one host thread per device, each on its own contiguous share of the rows */
    const uint32_t in0 = p->topology[0], outw = p->topology[p->layers - 1];
    float *result = a.outputs;
    if (!result) {
        const size_t out_bytes = (size_t)a.sample_count * outw * sizeof(float);
        if (n->h_out_bytes < out_bytes || !n->h_out) {
            spgk_host_free(n->h_out); n->h_out = NULL; n->h_out_bytes = 0;
            void *h = NULL;
            if (spg_map_kernel_error(spgk_host_alloc(&h, out_bytes), "forward_batch: output buffer")) return NULL;
            n->h_out = h; n->h_out_bytes = out_bytes;
        }
        result = n->h_out;
    }
    fan_job jobs[SPG_MAX_FANOUT];
    pthread_t th[SPG_MAX_FANOUT];
    bool started[SPG_MAX_FANOUT] = { false };
    int failed = SPINGALETT_OK;
    const char *why = NULL;
    for (int g = 0; g < G; g++) {
        uint32_t lo, hi;
        spingalett_split_rows(a.sample_count, (uint32_t)G, (uint32_t)g, &lo, &hi);
        /* share 0 runs on the net's own record when that is (or can be) bound to the first device of the list */
        spg_net *target = (g == 0 && (n->device < 0 || n->device == ids[0])) ? n : shadow_for(n, g, ids[g]);
        if (!target) { failed = SPINGALETT_ERR_ALLOC; why = "forward_batch: replica allocation failed"; break; }
        if (target == n && n->device < 0) n->device = ids[0];
        jobs[g] = (fan_job){ .net = target, .rc = 0,
                             .args = { .net = &target->pub, .inputs = a.inputs + (size_t)lo * in0, .sample_count = hi - lo,
                                       .outputs = result + (size_t)lo * outw } };
        jobs[g].msg[0] = 0;
        if (pthread_create(&th[g], NULL, fan_worker, &jobs[g]) != 0) { failed = SPINGALETT_ERR_ALLOC; why = "forward_batch: thread creation failed"; break; }
        started[g] = true;
    }
    for (int g = 0; g < G; g++) {
        if (!started[g]) continue;
        pthread_join(th[g], NULL);
        if (jobs[g].rc && !failed) { failed = jobs[g].rc; why = jobs[g].msg; }
    }
    if (n->device >= 0) spgk_set_device(n->device);
    if (failed) { spg_set_errorf(failed, "forward_batch (device fan-out): %s", why ? why : "failed"); return NULL; }
    spg_note_path("fan-out");
    return result;
}

static float *forward_batch_on(spg_net *n, ForwardBatchArgs a)
{
    NeuralNetwork *p = &n->pub;
    const uint32_t N = a.sample_count;
    const uint32_t in0 = p->topology[0], outw = p->topology[p->layers - 1];
    if (spg_dev_ensure(n) != SPINGALETT_OK) return NULL;
    const size_t in_bytes = (size_t)N * in0 * sizeof(float), out_bytes = (size_t)N * outw * sizeof(float);

    float *result = a.outputs;
    const bool out_dev = a.outputs && spgk_is_device_pointer(a.outputs) == 1;
    if (!a.outputs) {
        if (n->h_out_bytes < out_bytes || !n->h_out) {
            spgk_host_free(n->h_out); n->h_out = NULL; n->h_out_bytes = 0;
            void *h = NULL;
            if (spg_map_kernel_error(spgk_host_alloc(&h, out_bytes), "forward_batch: output buffer")) return NULL;
            n->h_out = h; n->h_out_bytes = out_bytes;
        }
        result = n->h_out;
    }
    if (N == 0) return result;

    const float *d_x = a.inputs;
    const bool in_dev = spgk_is_device_pointer(a.inputs) == 1;
    /* Large host batches are cut into chunks whose copies run on a second stream ahead of the compute: the
     * call is bound by the host link, and this hides all compute but the last chunk's behind the copies. */
    const uint32_t chunk_rows = 16384;
    const uint32_t chunks = (N + chunk_rows - 1) / chunk_rows;
    const bool pipelined = !in_dev && N >= 2 * chunk_rows && chunks <= SPG_PIPE_MAX;
    /* pageable inputs of a pipelined call go through two page-locked chunk buffers filled by several host threads */
    static int stage_off = -1;
    if (stage_off < 0) { const char *e = getenv("SPINGALETT_NO_STAGING"); stage_off = (e && *e && *e != '0') ? 1 : 0; }
    bool staged = pipelined && !stage_off && !spgk_is_pinned_host_pointer(a.inputs);
    if (staged) {
        const size_t need = (size_t)chunk_rows * in0 * sizeof(float);
        if (n->h_chunk_bytes < need) {
            for (int i = 0; i < 2; i++) { spgk_host_free(n->h_chunk[i]); n->h_chunk[i] = NULL; }
            n->h_chunk_bytes = 0;
            void *b0 = NULL, *b1 = NULL;
            if (spgk_host_alloc(&b0, need) == SPGK_OK && spgk_host_alloc(&b1, need) == SPGK_OK) {
                n->h_chunk[0] = b0; n->h_chunk[1] = b1; n->h_chunk_bytes = need;
            } else {
                spgk_host_free(b0); spgk_host_free(b1);
                spingalett_clear_error();
                staged = false;                                   /* no page-locked memory to be had: plain copies */
            }
        }
    }
    if (!in_dev) {
        if (reserve((void **)&n->d_in32, &n->in32_bytes, in_bytes, "forward_batch: input staging")) return NULL;
        d_x = n->d_in32;
        if (pipelined) {
            if (!n->copy_stream && spg_map_kernel_error(spgk_stream_create(&n->copy_stream), "forward_batch: copy stream")) return NULL;
            for (uint32_t c = 0; c <= chunks; c++)
                if (!n->copy_ev[c] && spg_map_kernel_error(spgk_event_create(&n->copy_ev[c]), "forward_batch: copy event")) return NULL;
            /* the staging buffer may still be read by earlier work on the compute stream */
            if (spg_map_kernel_error(spgk_event_record(n->copy_ev[0], n->stream), "forward_batch: pipeline") ||
                spg_map_kernel_error(spgk_stream_wait_event(n->copy_stream, n->copy_ev[0]), "forward_batch: pipeline")) return NULL;
        } else if (spg_map_kernel_error(spgk_memcpy_h2d(n->d_in32, a.inputs, in_bytes, n->stream), "forward_batch: input copy")) return NULL;
    }

    /* Up to 8 rows always take the weight-streaming chain; up to 512 rows do so (in groups of at most 128
     * rows, each group streaming the packed weights once) when every layer is eligible for the tensor-core
     * streaming kernel; everything else is the large-batch GEMM chain. */
    /* 9 to 24 rows on a net the GEMV takes whole: groups of 8 rows through the GEMV (0.2 ms per group on the large
     * INT4 net) beat one pass of the tensor-core streaming kernel (0.7 - 0.8 ms there) */
    bool gemv_groups = N > SPGK_GEMV_MAX_BATCH && N <= 3 * SPGK_GEMV_MAX_BATCH;
    for (uint32_t l = 0; l < n->dev_layers && gemv_groups; l++)
        if (!spgk_gemv_scratch_bytes(&n->klayers[l], SPGK_GEMV_MAX_BATCH)) gemv_groups = false;
    const uint32_t group = N <= SPGK_GEMV_MAX_BATCH ? N : (gemv_groups ? SPGK_GEMV_MAX_BATCH : 128u);
    /* from about a hundred rows on the GEMM chain on kept 16-bit operands (0.70 ms at 128 and at 256 rows of the large
     * INT4 net, two-term) beats the streaming kernel (0.58 ms at 64 rows, 0.88 ms at 128, 1.77 ms for the two passes of
     * 256) whenever those operands fit the keep budget */
    const bool chain_kept = N > 96 && weights_keepable(n, fast_type(n), false) && weights_keepable(n, SPGK_T_BF16, true);
    if (N <= SPGK_GEMV_MAX_BATCH || gemv_groups || (N <= 512 && !chain_kept && all_wstream(n, N < group ? N : group))) {
        for (uint32_t r0 = 0; r0 < N; r0 += group) {
            const uint32_t rows = N - r0 < group ? N - r0 : group;
            float *d_last = NULL;
            float *dst_dev = out_dev ? result + (size_t)r0 * outw : NULL;
            if (spg_dev_forward_small(n, d_x + (size_t)r0 * in0, in0, rows, &d_last, dst_dev)) return NULL;
            if (!out_dev && spg_map_kernel_error(spgk_memcpy_d2h(result + (size_t)r0 * outw, d_last, (size_t)rows * outw * sizeof(float), n->stream),
                                                 "forward_batch: output copy")) return NULL;
        }
    } else {
        float *d_out = result;
        if (!out_dev) {
            if (reserve((void **)&n->d_out32, &n->out32_bytes, out_bytes, "forward_batch: output staging")) return NULL;
            d_out = n->d_out32;
        }
        n->count_slot = 0; n->count_slots_used = 0;
        if (pipelined) {
            /* compute on chunk c starts as soon as its copy has landed, while the copies of the later chunks go on */
            /* copy c is queued before compute c-1 is launched, so a pageable source (whose copies block the host)
             * overlaps as well as a pinned one */
            for (uint32_t c = 0; c <= chunks; c++) {
                if (c < chunks) {
                    const size_t r0 = (size_t)c * chunk_rows, rows = N - r0 < chunk_rows ? N - r0 : chunk_rows;
                    const float *src = a.inputs + r0 * in0;
                    if (staged) {
                        /* the staging buffer of chunk c was last read by the copy of chunk c-2 */
                        if (c >= 2 && spg_map_kernel_error(spgk_event_sync(n->copy_ev[c - 1]), "forward_batch: staging")) return NULL;
                        stage_copy(n->h_chunk[c & 1], src, rows * in0 * sizeof(float));
                        src = n->h_chunk[c & 1];
                    }
                    if (spg_map_kernel_error(spgk_memcpy_h2d(n->d_in32 + r0 * in0, src, rows * in0 * sizeof(float), n->copy_stream),
                                             "forward_batch: input copy") ||
                        spg_map_kernel_error(spgk_event_record(n->copy_ev[c + 1], n->copy_stream), "forward_batch: pipeline")) return NULL;
                }
                if (c >= 1) {
                    const uint32_t k = c - 1, r0 = k * chunk_rows, rows = N - r0 < chunk_rows ? N - r0 : chunk_rows;
                    if (spg_map_kernel_error(spgk_stream_wait_event(n->stream, n->copy_ev[k + 1]), "forward_batch: pipeline")) return NULL;
                    n->count_slot = k;
                    const int rc = spg_dev_forward_large(n, d_x + (size_t)r0 * in0, rows, d_out + (size_t)r0 * outw);
                    n->count_slot = 0;
                    if (rc) return NULL;
                }
            }
        } else if (spg_dev_forward_large(n, d_x, N, d_out)) return NULL;
        if (!out_dev && spg_map_kernel_error(spgk_memcpy_d2h(result, d_out, out_bytes, n->stream), "forward_batch: output copy")) return NULL;
    }
    /* device-to-device calls are stream-ordered like any CUDA library call: the caller
     * synchronises (spingalett_synchronize or its own stream sync); host buffers are
     * complete on return */
    if (!(in_dev && out_dev) && finish(n)) return NULL;
    return result;
}
