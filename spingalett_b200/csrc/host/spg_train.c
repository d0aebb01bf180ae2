/* train(): the reference's training loop on the GPU.
 *
 * Control flow and argument handling follow the reference's trainer
 * (Src/Spingalett.Training.c:584-920): defaults for unset fields (:593-597), the
 * same validation and messages (:602-626), batch-size defaults (:628-631),
 * optional optimizer reset (:633-640), per-epoch shuffle with the library
 * generator and batches cut from the shuffled order (:748-767), gradients scaled
 * by 1/batch (:753), time_step and the running powers of beta advanced before
 * every update (:777-779; the powers restart at 1 on every call, :687-688), loss
 * reported as summed batch loss / sample_count (:784), NaN scan (:788-793),
 * autosave (:795-799, :536-578), callback (:801-806).
 *
 * Every combination the reference trains runs on the GPU: MODE_ARRAY with
 * STRATEGY_FULL_BATCH, STRATEGY_SMALL_BATCH or STRATEGY_SAMPLE (one sample per
 * update, in order, :78-250); SGD, MOMENTUM, RMSPROP, ADAM, ADAMW with weight decay
 * (:439-507); global-norm gradient clipping for the batched strategies (:451-452);
 * LOSS_MSE and LOSS_CROSS_ENTROPY with any output activation (:347-376).  There
 * is no CPU trainer behind this library.
 *
 * The device buffers (parameters, optimiser moments, workspaces, the caller's
 * samples) stay allocated between train() calls on the same net; save_spingalett
 * called from inside a train() call (autosave, or the caller's callback) encodes
 * straight from those device buffers.
 *
 * Data parallelism: after spingalett_dist_init() every process (one per GPU)
 * trains on its own samples; the flat gradient buffer [gW | gB] is summed across
 * ranks with one NCCL all-reduce per step and the fused Adam kernel divides by the
 * number of ranks, so replicas stay bit-identical without a broadcast. */
#include "spg_internal.h"
#include <stdlib.h>
#include <stdio.h>
#include <string.h>
#include <time.h>

typedef struct {
    float *params, *grads, *m, *v;          /* flat device buffers: [weights | biases] */
    float *acts, *deltas;                    /* [batch][total_neurons]-sized, layer after layer */
    float *data_x, *data_t;                  /* the caller's samples, resident */
    float *batch_x, *batch_t;                /* gathered mini-batch */
    uint32_t *idx;
    float *words;                            /* [0] loss, [1] non-finite flag, [2] sum of squared gradients, [8..] rank agreement */
    size_t cap[12];                          /* bytes held by each of the buffers above, in declaration order */
    uint64_t np;                             /* parameters the flat buffers were sized for */
    void *stream;                            /* a stream of the library's own for nets that sit on the legacy default stream */
} train_state;

/* process-wide communicator for the gradient exchange */
static void *s_comm = NULL;
static int s_rank = 0, s_world = 1;
/* the exchange runs on a stream of its own so that one layer's gradients cross NVLink while the next layer's are computed:
   s_ev_ready orders it after the gradient kernels, s_ev_done orders the optimiser after it */
static void *s_ar_stream = NULL, *s_ev_ready = NULL, *s_ev_done = NULL;
/* the one-kernel exchange over peer memory (spgk_xchg_*): created by the first data-parallel train() call for its
   parameter count, kept for later calls; NULL = the NCCL exchange */
static void *s_xchg = NULL;

static void dist_release(void)
{
    if (s_xchg) spgk_xchg_destroy(s_xchg);
    s_xchg = NULL;
    if (s_ev_ready) spgk_event_destroy(s_ev_ready);
    if (s_ev_done) spgk_event_destroy(s_ev_done);
    if (s_ar_stream) spgk_stream_destroy(s_ar_stream);
    if (s_comm) spgk_nccl_destroy(s_comm);
    s_ev_ready = s_ev_done = s_ar_stream = s_comm = NULL;
}

int spingalett_dist_unique_id(void *id128)
{
    return spg_map_kernel_error(spgk_nccl_unique_id(id128), "dist_unique_id");
}

int spingalett_dist_init(int rank, int world, const void *id128)
{
    if (world < 1 || rank < 0 || rank >= world || (world > 1 && !id128)) {
        spg_set_error(SPINGALETT_ERR_INVALID, "dist_init: bad rank/world/id");
        return SPINGALETT_ERR_INVALID;
    }
    dist_release();
    s_rank = rank; s_world = world;
    if (world == 1) return SPINGALETT_OK;
    int rc = spgk_nccl_init(&s_comm, rank, world, id128);
    if (rc == SPGK_OK) rc = spgk_stream_create(&s_ar_stream);
    if (rc == SPGK_OK) rc = spgk_event_create(&s_ev_ready);
    if (rc == SPGK_OK) rc = spgk_event_create(&s_ev_done);
    if (rc != SPGK_OK) { dist_release(); s_rank = 0; s_world = 1; }
    return spg_map_kernel_error(rc, "dist_init");
}

void spingalett_dist_shutdown(void)
{
    dist_release();
    s_rank = 0; s_world = 1;
}

int spingalett_dist_world(void) { return s_world; }

/* grow-only device buffer number `slot` of the state */
static int state_reserve(train_state *t, int slot, void **buf, size_t bytes, const char *what)
{
    if (*buf && t->cap[slot] >= bytes) return SPINGALETT_OK;
    spgk_free(*buf); *buf = NULL; t->cap[slot] = 0;
    int rc = spg_map_kernel_error(spgk_malloc(buf, bytes ? bytes : 256), what);
    if (rc == SPINGALETT_OK) t->cap[slot] = bytes;
    return rc;
}

static void state_free(train_state *t)
{
    if (!t) return;
    void *bufs[] = { t->params, t->grads, t->m, t->v, t->acts, t->deltas, t->data_x, t->data_t, t->batch_x, t->batch_t,
                     t->idx, t->words };
    for (size_t i = 0; i < sizeof bufs / sizeof bufs[0]; i++) spgk_free(bufs[i]);
    spgk_stream_destroy(t->stream);
    free(t);
}

void spg_train_release(spg_net *n)
{
    n->live_params = n->live_m = n->live_v = NULL;
    if (!n->train) return;
    if (n->device >= 0) spgk_set_device(n->device);
    state_free((train_state *)n->train);
    n->train = NULL;
}

/* same rule as the reference (Training.c:580-582) */
static bool should_report(size_t epoch, size_t epochs, size_t interval)
{
    return interval > 0 && (epoch % interval == 0 || epoch == epochs);
}

/* ---- agreement between ranks ------------------------------------------------------------------
 * Before a data-parallel train() every rank must be about to issue the same sequence of exchanges,
 * or a rank is left waiting in a collective for ever.  Each rank packs what determines that sequence
 * (sample count, batch size, epochs, strategy / optimiser / loss, intervals) into bytes, one float per
 * byte plus its square; after a SUM over ranks every byte b must satisfy sum = world*b and sum of
 * squares = world*b*b (equality holds only if all ranks hold the same byte; exact in fp32 up to 256
 * ranks).  Exported so that the check can be exercised with any transport (the CPU tests use gloo). */
#define SPG_AGREE_BYTES 40
int spingalett_dist_agreement_floats(void) { return 2 * SPG_AGREE_BYTES; }

void spingalett_dist_pack_agreement(const TrainArgs *a, float *out)
{
    uint8_t b[SPG_AGREE_BYTES];
    memset(b, 0, sizeof b);
    const uint64_t v[4] = { a->sample_count, a->batch_size, (uint64_t)a->epochs,
                            (uint64_t)a->training_strategy | ((uint64_t)a->optimizer_type << 8) | ((uint64_t)(a->callback ? 1 : 0) << 16) |
                            ((uint64_t)(a->max_grad_norm > 0.0f ? 1 : 0) << 17) };
    memcpy(b, v, 32);
    const uint32_t iv[2] = { (uint32_t)a->nan_check_interval, (uint32_t)(a->callback ? a->callback_interval : 0) };
    memcpy(b + 32, iv, 8);
    for (int i = 0; i < SPG_AGREE_BYTES; i++) { out[i] = (float)b[i]; out[SPG_AGREE_BYTES + i] = (float)b[i] * (float)b[i]; }
}

/* 1 if the summed buffer says every rank packed the same bytes as `mine` */
int spingalett_dist_check_agreement(const float *summed, const float *mine, int world)
{
    for (int i = 0; i < 2 * SPG_AGREE_BYTES; i++)
        if (summed[i] != mine[i] * (float)world) return 0;
    return 1;
}

/* Waiting for the stream inside train(): with several ranks the wait is bounded (SPINGALETT_DIST_TIMEOUT_MS), because an
 * exchange whose peer has left never finishes; when the limit is hit the communicator is aborted, so that this rank's
 * process can go on (and report the error) instead of hanging. */
static int train_sync(void *st)
{
    if (s_world <= 1) return spgk_stream_sync(st);
    const int rc = spgk_stream_sync_bounded(st);
    if (rc == SPGK_E_TIMEOUT && s_comm) {
        spg_log(LOG_ERROR, "train: the gradient exchange timed out; aborting the communicator");
        spgk_nccl_abort(s_comm);
        s_comm = NULL;
        dist_release();
        s_rank = 0; s_world = 1;
    }
    return rc;
}

#define DEV(call, what) do { int rc__ = spg_map_kernel_error((call), what); if (rc__) goto fail; } while (0)
/* inside the step: a failure while the step is being captured into a graph only ends the capture */
#define SDEV(call, what) do { int rc__ = spg_map_kernel_error((call), what); if (rc__) { if (in_capture) goto capture_abort; goto fail; } } while (0)

void train_struct_arguments(TrainArgs a)
{
    NeuralNetwork *p = a.net;
    if (a.learning_rate <= 0.0f) a.learning_rate = 0.01f;
    if (a.momentum <= 0.0f) a.momentum = 0.9f;
    if (a.beta1 <= 0.0f) a.beta1 = 0.9f;
    if (a.beta2 <= 0.0f) a.beta2 = 0.999f;
    if (a.epsilon <= 0.0f) a.epsilon = 1e-8f;
    if (a.callback && a.callback_interval == 0) a.callback_interval = 1;

    if (a.training_mode == MODE_GENERATOR_FUNCTION) {
        spg_set_error(SPINGALETT_ERR_INVALID, "Generator function training mode is not implemented yet");
        spg_log(LOG_ERROR, "Generator function training mode is not implemented yet");
        return;
    }
    if (!p || a.sample_count == 0 || a.epochs == 0 || !a.inputs || !a.targets) {
        spg_set_error(SPINGALETT_ERR_INVALID, "Invalid training arguments (NULL net/inputs/targets or zero count/epochs)");
        spg_log(LOG_ERROR, "Invalid training arguments");
        return;
    }
    if (p->layers < 2) {
        spg_set_error(SPINGALETT_ERR_INVALID, "Network must have at least 2 layers for training");
        spg_log(LOG_ERROR, "Network must have at least 2 layers for training");
        return;
    }
    for (uint32_t l = 1; l + 1 < p->layers; l++)
        if (p->act_func[l - 1] == ACT_SOFTMAX) {
            spg_set_error(SPINGALETT_ERR_INVALID, "Softmax is not supported in hidden layers");
            spg_log(LOG_ERROR, "Softmax in hidden layer %u is not supported. Use softmax only in the output layer.", l);
            return;
        }
    if ((unsigned)a.training_strategy > STRATEGY_SMALL_BATCH || (unsigned)a.optimizer_type > OPTIMIZER_ADAMW ||
        (unsigned)p->loss_func > LOSS_CROSS_ENTROPY) {
        spg_set_error(SPINGALETT_ERR_INVALID, "train: unknown strategy, optimizer or loss");
        spg_log(LOG_ERROR, "train: unknown strategy, optimizer or loss");
        return;
    }
    const ActivationFunction out_act = p->act_func[p->layers - 2];
    if (a.training_strategy == STRATEGY_SMALL_BATCH && a.batch_size == 0) a.batch_size = 32;
    if (a.training_strategy == STRATEGY_SMALL_BATCH && a.batch_size > a.sample_count) a.batch_size = a.sample_count;

    spg_net *n = spg_priv(p);
    if (spg_net_ensure_train_arrays(n) != SPINGALETT_OK) return;
    if (a.reset_optimizer) {
        memset(p->opt_m_weights, 0, p->total_weights * sizeof(float));
        memset(p->opt_v_weights, 0, p->total_weights * sizeof(float));
        memset(p->opt_m_biases, 0, p->total_biases * sizeof(float));
        memset(p->opt_v_biases, 0, p->total_biases * sizeof(float));
        p->time_step = 0;
        spg_log(LOG_INFO, "Optimizer state reset");
    }
    if (spg_dev_ensure(n) != SPINGALETT_OK) return;          /* binds the device (and validates it exists) */

    /* STRATEGY_SAMPLE is a batch of one sample per update, in the caller's order (Training.c:894-897, :78-250) */
    const bool mini = a.training_strategy == STRATEGY_SMALL_BATCH, online = a.training_strategy == STRATEGY_SAMPLE;
    const uint32_t batch = mini ? a.batch_size : online ? 1u : a.sample_count;
    const uint32_t in0 = p->topology[0], outw = p->topology[p->layers - 1], last = p->layers - 1;
    const uint64_t tw = p->total_weights, tb = p->total_biases, np = tw + tb, tn = p->total_neurons;
    static const char *const strat_names[] = { "SAMPLE", "FULL_BATCH", "SMALL_BATCH" };
    static const char *const opt_names[] = { "SGD", "MOMENTUM", "RMSPROP", "ADAM", "ADAMW" };
    spg_log(LOG_INFO, "Starting training: loss=%s, strategy=%s, optimizer=%s, compute=CUDA, batch_size=%u, ranks=%d",
            spg_loss_name(p->loss_func), strat_names[a.training_strategy], opt_names[a.optimizer_type], batch, s_world);

    /* the device state of an earlier call is reused when it was made for the same parameter count */
    train_state *t = (train_state *)n->train;
    if (t && t->np != np) { spg_train_release(n); t = NULL; }
    if (!t) {
        t = calloc(1, sizeof *t);
        if (!t) { spg_set_error(SPINGALETT_ERR_ALLOC, "train: state allocation failed"); return; }
        t->np = np;
        n->train = t;
    }
    /* The legacy default stream cannot be captured into a graph: a net that runs on it trains on a stream of the
       library's own for the length of this call (everything the call touches, autosave and the callback's saves
       included, follows n->stream, so it is switched and put back at the end).  Earlier work of the net is awaited first;
       the call itself ends with a synchronisation, so later work on the caller's stream is ordered behind it. */
    void *const caller_stream = n->stream;
    if ((uintptr_t)n->stream <= 2) {
        if (!t->stream && spgk_stream_create(&t->stream) != SPGK_OK) { spingalett_clear_error(); t->stream = NULL; }
        if (t->stream && spgk_stream_sync(n->stream) == SPGK_OK) n->stream = t->stream;
    }
    void *st = n->stream;
    uint32_t *order = NULL;
    float *h_pinned = NULL;
    bool failed = true;
    void *graph_exec = NULL;                 /* the step as an executable CUDA graph, once captured */
    bool graph_failed = false, in_capture = false;

    if (state_reserve(t, 0, (void **)&t->params, np * 4, "train: parameters") || state_reserve(t, 1, (void **)&t->grads, np * 4, "train: gradients") ||
        state_reserve(t, 2, (void **)&t->m, np * 4, "train: first moments") || state_reserve(t, 3, (void **)&t->v, np * 4, "train: second moments") ||
        state_reserve(t, 4, (void **)&t->acts, (size_t)batch * tn * 4, "train: activations") ||
        state_reserve(t, 5, (void **)&t->deltas, (size_t)batch * tn * 4, "train: deltas") ||
        state_reserve(t, 6, (void **)&t->data_x, (size_t)a.sample_count * in0 * 4, "train: inputs") ||
        state_reserve(t, 7, (void **)&t->data_t, (size_t)a.sample_count * outw * 4, "train: targets") ||
        state_reserve(t, 11, (void **)&t->words, 1024, "train: status words")) goto fail;
    if (mini) {
        if (state_reserve(t, 8, (void **)&t->batch_x, (size_t)batch * in0 * 4, "train: batch inputs") ||
            state_reserve(t, 9, (void **)&t->batch_t, (size_t)batch * outw * 4, "train: batch targets")) goto fail;
        if (state_reserve(t, 10, (void **)&t->idx, (size_t)a.sample_count * 4, "train: shuffle order")) goto fail;
        order = malloc((size_t)a.sample_count * sizeof *order);
        if (!order) { spg_set_error(SPINGALETT_ERR_ALLOC, "Mini-batch allocation failed"); goto fail; }
        for (uint32_t i = 0; i < a.sample_count; i++) order[i] = i;
    }
    float *d_loss = t->words, *d_sumsq = t->words + 2, *d_agree = t->words + 8;
    int *d_flag = (int *)(t->words + 1);
    DEV(spgk_host_alloc((void **)&h_pinned, 1024), "train: pinned words");

    /* the host arrays are the truth between calls (callers may edit them): upload them every time */
    DEV(spgk_memcpy_h2d(t->params, p->weights, tw * 4, st), "train: upload weights");
    DEV(spgk_memcpy_h2d(t->params + tw, p->biases, tb * 4, st), "train: upload biases");
    DEV(spgk_memcpy_h2d(t->m, p->opt_m_weights, tw * 4, st), "train: upload m");
    DEV(spgk_memcpy_h2d(t->m + tw, p->opt_m_biases, tb * 4, st), "train: upload m");
    DEV(spgk_memcpy_h2d(t->v, p->opt_v_weights, tw * 4, st), "train: upload v");
    DEV(spgk_memcpy_h2d(t->v + tw, p->opt_v_biases, tb * 4, st), "train: upload v");
    DEV(spgk_memcpy_h2d(t->data_x, a.inputs, (size_t)a.sample_count * in0 * 4, st), "train: upload inputs");
    DEV(spgk_memcpy_h2d(t->data_t, a.targets, (size_t)a.sample_count * outw * 4, st), "train: upload targets");
    DEV(spgk_memset(t->grads, 0, np * 4, st), "train: clear gradients");

    if (s_world > 1) {
        /* all ranks must be about to run the same loop, or one of them waits in an exchange for ever */
        float mine[2 * SPG_AGREE_BYTES];
        spingalett_dist_pack_agreement(&a, mine);
        memcpy(h_pinned, mine, sizeof mine);
        DEV(spgk_memcpy_h2d(d_agree, h_pinned, sizeof mine, st), "train: agreement");
        DEV(spgk_nccl_allreduce_sum(s_comm, d_agree, 2 * SPG_AGREE_BYTES, st), "train: agreement");
        DEV(spgk_memcpy_d2h(h_pinned, d_agree, sizeof mine, st), "train: agreement");
        DEV(train_sync(st), "train: agreement");
        if (!spingalett_dist_check_agreement(h_pinned, mine, s_world)) {
            spg_set_error(SPINGALETT_ERR_INVALID, "train: the ranks disagree on sample_count, batch_size, epochs, strategy, optimizer or "
                                                  "callback / check intervals; a data-parallel run needs them equal on every rank");
            spg_log(LOG_ERROR, "train: ranks disagree on the training arguments");
            goto fail;
        }
    }

    /* Several ranks: the exchange of a step is one kernel over peer memory (sum of the gradient shards by peer loads, the
       update on the own shard, the new weights stored into every replica) unless gradient clipping needs the global norm
       first or SPINGALETT_EXCHANGE=nccl asks for the NCCL all-reduce.  Its buffers live in an arena the peers can map:
       the step's kernels write gradients there and read parameters from there.  Setting it up is collective, and a rank
       on which it fails takes all of them to the NCCL path. */
    float *P = t->params, *G = t->grads, *M = t->m, *V = t->v;
    const bool clip = a.max_grad_norm > 0.0f && a.training_strategy != STRATEGY_SAMPLE;
    bool fused_x = false;
    if (s_world > 1) {
        const char *mode = getenv("SPINGALETT_EXCHANGE");
        const bool want = !clip && !(mode && strcmp(mode, "nccl") == 0);
        /* first vote: does every rank want it, and does every rank still hold an arena of this size from an earlier call? */
        h_pinned[32] = want ? 1.0f : 0.0f;
        h_pinned[33] = want && s_xchg && spgk_xchg_capacity(s_xchg) == np ? 1.0f : 0.0f;
        DEV(spgk_memcpy_h2d(d_agree, h_pinned + 32, 8, st), "train: exchange vote");
        DEV(spgk_nccl_allreduce_sum(s_comm, d_agree, 2, st), "train: exchange vote");
        DEV(spgk_memcpy_d2h(h_pinned + 32, d_agree, 8, st), "train: exchange vote");
        DEV(train_sync(st), "train: exchange vote");
        const bool all_want = h_pinned[32] == (float)s_world, all_have = h_pinned[33] == (float)s_world;
        if (s_xchg && !(all_want && all_have)) { spgk_xchg_destroy(s_xchg); s_xchg = NULL; }
        if (all_want) {
            bool mine_ok = true;
            if (!s_xchg && spgk_xchg_create(&s_xchg, s_rank, s_world, np, s_comm, st) != SPGK_OK) {
                spg_log(LOG_INFO, "train: no peer-memory exchange here (%s); NCCL all-reduce instead", spgk_error_string());
                s_xchg = NULL; mine_ok = false;
            }
            /* second vote: did the set-up work everywhere? */
            h_pinned[32] = mine_ok ? 0.0f : 1.0f;
            DEV(spgk_memcpy_h2d(d_agree, h_pinned + 32, 4, st), "train: exchange vote");
            DEV(spgk_nccl_allreduce_sum(s_comm, d_agree, 1, st), "train: exchange vote");
            DEV(spgk_memcpy_d2h(h_pinned + 32, d_agree, 4, st), "train: exchange vote");
            DEV(train_sync(st), "train: exchange vote");
            fused_x = h_pinned[32] == 0.0f;
            if (!fused_x && s_xchg) { spgk_xchg_destroy(s_xchg); s_xchg = NULL; }
        }
        if (fused_x) {
            P = spgk_xchg_buffer(s_xchg, 1); G = spgk_xchg_buffer(s_xchg, 0); M = spgk_xchg_buffer(s_xchg, 2); V = spgk_xchg_buffer(s_xchg, 3);
            DEV(spgk_memcpy_d2d(P, t->params, np * 4, st), "train: parameters into the exchange arena");
            DEV(spgk_memcpy_d2d(M, t->m, np * 4, st), "train: moments into the exchange arena");
            DEV(spgk_memcpy_d2d(V, t->v, np * 4, st), "train: moments into the exchange arena");
            DEV(spgk_memset(G, 0, np * 4, st), "train: clear gradients");
        }
        spg_log(LOG_INFO, "train: gradient exchange over %s", fused_x ? "peer memory (one kernel per step)" : "NCCL all-reduce");
    }

    /* save_spingalett called while this call runs (autosave, the callback) reads the device buffers */
    n->live_params = P; n->live_m = M; n->live_v = V;

    /* which output-layer path: cross-entropy over softmax / sigmoid has delta = a - t (Training.c:368-371) and, for at most
       16 outputs, a one-launch output end; everything else goes through the general delta kernel */
    const bool ce_direct = p->loss_func == LOSS_CROSS_ENTROPY && (out_act == ACT_SOFTMAX || out_act == ACT_SIGMOID);
    const bool fused_out = ce_direct && outw <= 16;
    float b1pow = 1.0f, b2pow = 1.0f;
    /* Replay of the step as a CUDA graph: with one rank or the peer-memory exchange, a strategy whose steps are all the same size and more than a
       handful of steps, the launches of a step take what changes between steps (position in the epoch, Adam's bias
       corrections) from a small device record, so the first step runs directly, the second is captured, and every later
       one is a single graph launch -- the host thread is then out of the step's critical path (ten launches per 0.12 ms
       step otherwise: two identical train() calls differed by 20 % with the host's load).  SPINGALETT_TRAIN_GRAPH=0
       keeps the direct launches. */
    const uint32_t steps_per_epoch = (a.sample_count + batch - 1) / batch;
    bool graph_mode = (s_world == 1 || fused_x) && !online && a.sample_count % batch == 0 && (uint64_t)steps_per_epoch * a.epochs >= 4;
    { const char *e = getenv("SPINGALETT_TRAIN_GRAPH"); if (e && *e == '0') graph_mode = false; }
    void *step_state = (void *)(t->words + 128);      /* clear of the loss / flag / norm words and of the rank-agreement floats */
    uint64_t steps_done = 0;
    if (graph_mode) {
        DEV(spgk_train_state_reset(step_state, st), "train: step state");
        spgk_train_use_state(step_state);
    }
    for (size_t epoch = 1; epoch <= a.epochs; epoch++) {
        const bool need_loss = should_report(epoch, a.epochs, a.report_interval) ||
                               (a.callback && should_report(epoch, a.epochs, a.callback_interval));
        if (need_loss || graph_mode) DEV(spgk_memset(d_loss, 0, 4, st), "train: clear loss");
        float *const loss_ptr = (need_loss || graph_mode) ? d_loss : NULL;      /* a replayed step always adds to the loss word */
        if (mini) {
            spg_shuffle(order, a.sample_count);
            DEV(spgk_memcpy_h2d(t->idx, order, (size_t)a.sample_count * 4, st), "train: upload order");
            DEV(train_sync(st), "train: order sync");        /* `order` is reshuffled next epoch */
        }
        const uint32_t nb = (a.sample_count + batch - 1) / batch;
        for (uint32_t bi = 0; bi < nb; bi++) {
            const uint32_t start = bi * batch;
            const uint32_t cur = start + batch > a.sample_count ? a.sample_count - start : batch;
            const float *bx = t->data_x + (size_t)(mini ? 0 : start) * in0, *bt = t->data_t + (size_t)(mini ? 0 : start) * outw;
            p->time_step++;
            b1pow *= a.beta1;
            b2pow *= a.beta2;
            const float mf = 1.0f / (1.0f - b1pow), vf = 1.0f / (1.0f - b2pow);
            steps_done++;
            if (graph_exec) {                                        /* every step after the second */
                DEV(spgk_graph_launch(graph_exec, st), "train: step (graph)");
                continue;
            }
            bool capture = graph_mode && !graph_failed && steps_done == 2;
          for (;;) {
            if (capture) {
                if (spgk_graph_begin(st) == SPGK_OK) in_capture = true;
                else { spingalett_clear_error(); graph_failed = true; capture = false; }
            }
            if (graph_mode) SDEV(spgk_train_state_step(step_state, steps_per_epoch, batch, a.beta1, a.beta2, st), "train: step state");
            if (mini) {
                /* (with the device record the kernel adds the step's first row itself) */
                SDEV(spgk_gather_rows2(t->data_x, in0, t->batch_x, t->data_t, outw, t->batch_t, graph_mode ? t->idx : t->idx + start, cur, st),
                    "train: gather mini-batch");
                bx = t->batch_x; bt = t->batch_t;
            }
            /* forward: activations of layer l live at acts + cur*neuron_offsets[l], [cur][width] */
            float *d_last = t->deltas + (size_t)cur * p->neuron_offsets[last];
            const float *x = bx;
            for (uint32_t l = 0; l < last; l++) {
                const uint32_t fi = p->topology[l], fo = p->topology[l + 1];
                float *y = t->acts + (size_t)cur * p->neuron_offsets[l + 1];
                if (l + 1 == last && fused_out) {
                    SDEV(spgk_train_output(x, fi, P + p->weight_offsets[l], fi, P + tw + p->bias_offsets[l], y, bt,
                                          d_last, loss_ptr, cur, fo, fi, out_act == ACT_SIGMOID, st),
                        "train: output layer");
                    break;
                }
                SDEV(spgk_train_gemm(0, x, fi, P + p->weight_offsets[l], fi, y, fo, cur, fo, fi, 1.0f,
                                    P + tw + p->bias_offsets[l], NULL, 0, (int)p->act_func[l], st), "train: forward");
                if (p->act_func[l] == ACT_SOFTMAX) SDEV(spgk_softmax_rows(y, fo, cur, fo, st), "train: softmax");
                x = y;
            }
            if (!fused_out) {
                const float *a_last = t->acts + (size_t)cur * p->neuron_offsets[last];
                if (ce_direct)
                    SDEV(spgk_ce_delta(a_last, bt, d_last, (uint64_t)cur * outw, loss_ptr, out_act == ACT_SIGMOID, st),
                        "train: output delta");
                else
                    SDEV(spgk_output_delta(a_last, bt, d_last, cur, outw, (int)out_act,
                                          p->loss_func == LOSS_MSE && out_act == ACT_SOFTMAX ? 1 : 0,
                                          p->loss_func == LOSS_MSE ? 0 : 1, loss_ptr, st), "train: output delta");
            }
            /* backwards through the layers: the gradients of layer l (from delta l+1 and activation l) go into the flat
               buffer and, with several replicas, start their all-reduce on the exchange stream at once, so that it runs
               under the delta and gradient products of the layers below */
            const float gs = 1.0f / (float)cur;
            for (uint32_t l = last; l-- > 0;) {
                const uint32_t fi = p->topology[l], fo = p->topology[l + 1];
                const float *dl = t->deltas + (size_t)cur * p->neuron_offsets[l + 1];
                const float *al = l == 0 ? bx : t->acts + (size_t)cur * p->neuron_offsets[l];
                SDEV(spgk_train_grad(dl, fo, al, fi, G + p->weight_offsets[l], fi, G + tw + p->bias_offsets[l],
                                    fo, fi, cur, gs, st), "train: gradients");
                if (s_world > 1 && !fused_x) {
                    SDEV(spgk_event_record(s_ev_ready, st), "train: exchange order");
                    SDEV(spgk_stream_wait_event(s_ar_stream, s_ev_ready), "train: exchange order");
                    if (l == 0)             /* the bias gradients of every layer are complete now: one launch for both */
                        SDEV(spgk_nccl_allreduce_sum2(s_comm, G + p->weight_offsets[l], (uint64_t)fi * fo, G + tw, tb,
                                                     s_ar_stream), "train: all-reduce");
                    else
                        SDEV(spgk_nccl_allreduce_sum(s_comm, G + p->weight_offsets[l], (uint64_t)fi * fo, s_ar_stream),
                            "train: all-reduce");
                }
                if (l > 0)
                    SDEV(spgk_train_gemm(1, dl, fo, P + p->weight_offsets[l], fi,
                                        t->deltas + (size_t)cur * p->neuron_offsets[l], fi, cur, fi, fo, 1.0f, NULL,
                                        t->acts + (size_t)cur * p->neuron_offsets[l], fi, (int)p->act_func[l - 1], st), "train: delta");
            }
            if (s_world > 1 && !fused_x) {
                SDEV(spgk_event_record(s_ev_done, s_ar_stream), "train: exchange order");
                SDEV(spgk_stream_wait_event(st, s_ev_done), "train: exchange order");
            }
            if (clip) {
                SDEV(spgk_memset(d_sumsq, 0, 4, st), "train: clear norm");
                SDEV(spgk_sumsq(G, np, d_sumsq, st), "train: gradient norm");
            }
            if (fused_x)
                SDEV(spgk_xchg_step(s_xchg, (int)a.optimizer_type, tw, a.learning_rate, a.momentum, a.beta1, a.beta2, mf, vf, a.epsilon,
                                   a.weight_decay > 0.0f ? a.weight_decay : 0.0f, 1.0f / (float)s_world,
                                   graph_mode ? (const float *)step_state + 4 : NULL, st), "train: exchange and update");
            else if (a.optimizer_type == OPTIMIZER_ADAM && a.weight_decay <= 0.0f && !clip)
                SDEV(spgk_adam(P, M, V, G, np, a.learning_rate, a.beta1, a.beta2, mf, vf, a.epsilon,
                              1.0f / (float)s_world, st), "train: adam");
            else
                SDEV(spgk_optimizer_step((int)a.optimizer_type, P, M, V, G, np, tw, a.learning_rate, a.momentum,
                                        a.beta1, a.beta2, mf, vf, a.epsilon, a.weight_decay > 0.0f ? a.weight_decay : 0.0f,
                                        1.0f / (float)s_world, clip ? d_sumsq : NULL, a.max_grad_norm, st), "train: update");
            if (!capture) break;
            /* the launches above were recorded, not run: make the graph and run it, or -- if that fails -- issue them again */
            in_capture = false;
            if (spgk_graph_end(st, &graph_exec) == SPGK_OK) { DEV(spgk_graph_launch(graph_exec, st), "train: step (graph)"); break; }
          capture_abort:
            /* a launch that cannot be recorded, or a graph that cannot be made: give the capture up for good and issue the
               step's launches directly (nothing of the step has run yet) */
            if (in_capture) { void *x = NULL; spgk_graph_end(st, &x); spgk_graph_destroy(x); in_capture = false; }
            spg_log(LOG_DEBUG, "train: no graph replay (%s)", spgk_error_string());
            spingalett_clear_error();
            graph_exec = NULL; graph_failed = true; capture = false;
          }
        }
        /* end of the epoch: loss, NaN scan and the stop decision.  With several ranks the loss is summed and a stop wanted
           by any rank (its callback, a non-finite weight) stops all of them, so nobody is left in an exchange alone. */
        const bool nan_now = a.nan_check_interval > 0 && epoch % a.nan_check_interval == 0;
        const bool cb_now = a.callback && should_report(epoch, a.epochs, a.callback_interval);
        float current_error = 0.0f;
        bool stop = false, nan_found = false;
        if (nan_now) {
            DEV(spgk_memset(d_flag, 0, 4, st), "train: clear flag");
            DEV(spgk_nonfinite(P, np, d_flag, st), "train: nan scan");
        }
        if (need_loss || nan_now) {
            DEV(spgk_memcpy_d2h(h_pinned, t->words, 8, st), "train: read loss");
            DEV(train_sync(st), "train: loss sync");
            current_error = need_loss ? h_pinned[0] / (float)a.sample_count : 0.0f;
            nan_found = nan_now && ((int *)h_pinned)[1] != 0;
        }
        if (should_report(epoch, a.epochs, a.report_interval))
            spg_log(LOG_INFO, "Epoch: %zu/%zu, Error: %f", epoch, a.epochs, (double)current_error);
        if (nan_found) {
            spg_log(LOG_ERROR, "NaN/Inf detected in weights at epoch %zu, stopping training", epoch);
            stop = true;
        }
        if (!stop && a.autosave_mode != AUTOSAVE_OFF && a.autosave_interval > 0 && a.autosave_path &&
            should_report(epoch, a.epochs, a.autosave_interval)) {
            /* the moments are current in their owners' shards only: collect them (every rank takes part) before rank 0 writes */
            if (fused_x && !a.autosave_do_not_save_optimizer) DEV(spgk_xchg_gather(s_xchg, st), "train: gather optimiser state");
            if (s_rank == 0) spg_autosave(n, &a, epoch);
        }
        if (!stop && cb_now) {
            /* the callback may read the net: bring the host mirror up to date first */
            DEV(spgk_memcpy_d2h(p->weights, P, tw * 4, st), "train: weights to host");
            DEV(spgk_memcpy_d2h(p->biases, P + tw, tb * 4, st), "train: biases to host");
            DEV(train_sync(st), "train: callback sync");
            if (a.callback(p, epoch, current_error)) {
                spg_log(LOG_INFO, "Training interrupted by callback at epoch %zu", epoch);
                stop = true;
            }
        }
        if (s_world > 1 && (nan_now || cb_now)) {
            h_pinned[16] = stop ? 1.0f : 0.0f;
            DEV(spgk_memcpy_h2d(d_agree, h_pinned + 16, 4, st), "train: stop vote");
            DEV(spgk_nccl_allreduce_sum(s_comm, d_agree, 1, st), "train: stop vote");
            DEV(spgk_memcpy_d2h(h_pinned + 16, d_agree, 4, st), "train: stop vote");
            DEV(train_sync(st), "train: stop vote");
            if (h_pinned[16] > 0.0f && !stop) spg_log(LOG_INFO, "Training stopped at epoch %zu because another rank stopped", epoch);
            stop = h_pinned[16] > 0.0f;
        }
        if (stop) break;
    }
    if (fused_x) DEV(spgk_xchg_gather(s_xchg, st), "train: gather gradients and optimiser state");
    /* host mirrors of everything the reference leaves in the public struct */
    DEV(spgk_memcpy_d2h(p->weights, P, tw * 4, st), "train: weights to host");
    DEV(spgk_memcpy_d2h(p->biases, P + tw, tb * 4, st), "train: biases to host");
    DEV(spgk_memcpy_d2h(p->grad_weights, G, tw * 4, st), "train: gradients to host");
    DEV(spgk_memcpy_d2h(p->grad_biases, G + tw, tb * 4, st), "train: gradients to host");
    DEV(spgk_memcpy_d2h(p->opt_m_weights, M, tw * 4, st), "train: m to host");
    DEV(spgk_memcpy_d2h(p->opt_m_biases, M + tw, tb * 4, st), "train: m to host");
    DEV(spgk_memcpy_d2h(p->opt_v_weights, V, tw * 4, st), "train: v to host");
    DEV(spgk_memcpy_d2h(p->opt_v_biases, V + tw, tb * 4, st), "train: v to host");
    DEV(train_sync(st), "train: final sync");
    if (fused_x) DEV(spgk_xchg_status(s_xchg, st), "train: gradient exchange");
    spg_log(LOG_INFO, "Training completed.");
    failed = false;
fail:
    n->stream = caller_stream;
    if (in_capture) { void *x = NULL; spgk_graph_end(st, &x); spgk_graph_destroy(x); }      /* never leave the stream capturing */
    spgk_graph_destroy(graph_exec);
    spgk_train_use_state(NULL);
    free(order);
    spgk_host_free(h_pinned);
    n->live_params = n->live_m = n->live_v = NULL;
    if (failed) spg_train_release(n);          /* after an error nothing of the device state is trusted */
    if (failed && s_xchg) { spgk_xchg_destroy(s_xchg); s_xchg = NULL; }
    /* the inference image on the device (possibly a packed payload) no longer matches the weights */
    spg_dev_invalidate(n);
    spg_net_drop_payload(n);
}

/* Autosave (Training.c:536-578): the same file naming as the reference -- AUTOSAVE_OVERWRITE writes autosave_path itself,
 * AUTOSAVE_NEW_FILES inserts "_epoch_<n>" in front of the extension (or appends it when the name has none). */
void spg_autosave(spg_net *n, const TrainArgs *a, size_t epoch)
{
    SaveArgs sa = { .net = &n->pub, .filename = a->autosave_path, .do_not_save_optimizer = a->autosave_do_not_save_optimizer,
                    .precision = a->autosave_precision };
    if (a->autosave_mode == AUTOSAVE_OVERWRITE) { save_spingalett_struct_arguments(sa); return; }
    if (a->autosave_mode != AUTOSAVE_NEW_FILES) return;
    const char *path = a->autosave_path;
    const size_t len = strlen(path);
    const char *dot = strrchr(path, '.'), *slash = strrchr(path, '/'), *back = strrchr(path, '\\');
    const char *sep = slash && back ? (slash > back ? slash : back) : (slash ? slash : back);
    const bool has_ext = dot && (!sep || dot > sep);
    char *buf = malloc(len + 64);
    if (!buf) return;
    if (has_ext) snprintf(buf, len + 64, "%.*s_epoch_%zu%s", (int)(dot - path), path, epoch, dot);
    else snprintf(buf, len + 64, "%s_epoch_%zu", path, epoch);
    sa.filename = buf;
    save_spingalett_struct_arguments(sa);
    free(buf);
}
