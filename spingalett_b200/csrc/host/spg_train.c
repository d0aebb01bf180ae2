/* train(): the mini-batch / full-batch training loop on the GPU.
 *
 * Control flow and argument handling follow the reference's batched trainer
 * (Src/Spingalett.Training.c:584-817): defaults for unset fields (:593-597), the
 * same validation and messages (:602-626), batch-size defaults (:628-631),
 * optional optimizer reset (:633-640), per-epoch shuffle with the library
 * generator and batches cut from the shuffled order (:748-767), gradients scaled
 * by 1/batch (:753), time_step and the running powers of beta advanced before
 * every update (:777-779; the powers restart at 1 on every call, :687-688), loss
 * reported as summed batch loss / sample_count (:784), NaN scan, callback.
 *
 * What runs on the GPU here: MODE_ARRAY with STRATEGY_FULL_BATCH or
 * STRATEGY_SMALL_BATCH, OPTIMIZER_ADAM (no weight decay, no gradient clipping),
 * LOSS_CROSS_ENTROPY over a softmax or sigmoid output layer.  Anything else is
 * refused with SPINGALETT_ERR_INVALID -- there is no CPU trainer behind this
 * library.  Autosave is not implemented.
 *
 * Data parallelism: after spingalett_dist_init() every process (one per GPU)
 * trains on its own samples; the flat gradient buffer [gW | gB] is summed across
 * ranks with one NCCL all-reduce per step and the fused Adam kernel divides by the
 * number of ranks, so replicas stay bit-identical without a broadcast. */
#include "spg_internal.h"
#include <stdlib.h>
#include <string.h>

typedef struct {
    float *params, *grads, *m, *v;          /* flat device buffers: [weights | biases] */
    float *acts, *deltas;                    /* [batch][total_neurons]-sized, layer after layer */
    float *data_x, *data_t;                  /* the caller's samples, resident */
    float *batch_x, *batch_t;                /* gathered mini-batch */
    uint32_t *idx;
    float *loss; int *flag;
    uint32_t batch_cap; uint64_t data_rows;
} train_state;

/* process-wide communicator for the gradient exchange */
static void *s_comm = NULL;
static int s_rank = 0, s_world = 1;
/* the exchange runs on a stream of its own so that one layer's gradients cross NVLink while the next layer's are computed:
   s_ev_ready orders it after the gradient kernels, s_ev_done orders the optimiser after it */
static void *s_ar_stream = NULL, *s_ev_ready = NULL, *s_ev_done = NULL;

static void dist_release(void)
{
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

static void state_free(train_state *t)
{
    if (!t) return;
    void *bufs[] = { t->params, t->grads, t->m, t->v, t->acts, t->deltas, t->data_x, t->data_t, t->batch_x, t->batch_t,
                     t->idx, t->loss, t->flag };
    for (size_t i = 0; i < sizeof bufs / sizeof bufs[0]; i++) spgk_free(bufs[i]);
    free(t);
}

void spg_train_release(spg_net *n)
{
    if (!n->train) return;
    if (n->device >= 0) spgk_set_device(n->device);
    state_free((train_state *)n->train);
    n->train = NULL;
}

static bool should_report(size_t epoch, size_t epochs, size_t interval)
{
    if (interval == 0) return false;
    return epoch == 1 || epoch == epochs || epoch % interval == 0;
}

#define DEV(call, what) do { int rc__ = spg_map_kernel_error((call), what); if (rc__) goto fail; } while (0)

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
    const ActivationFunction out_act = p->act_func[p->layers - 2];
    if ((a.training_strategy != STRATEGY_FULL_BATCH && a.training_strategy != STRATEGY_SMALL_BATCH) ||
        a.optimizer_type != OPTIMIZER_ADAM || p->loss_func != LOSS_CROSS_ENTROPY ||
        (out_act != ACT_SOFTMAX && out_act != ACT_SIGMOID) || a.weight_decay > 0.0f || a.max_grad_norm > 0.0f ||
        a.autosave_mode != AUTOSAVE_OFF) {
        spg_set_error(SPINGALETT_ERR_INVALID,
                      "train: the CUDA trainer takes FULL_BATCH/SMALL_BATCH + ADAM + CROSS_ENTROPY over softmax/sigmoid "
                      "(no weight decay, clipping or autosave); there is no CPU trainer in this library");
        spg_log(LOG_ERROR, "train: unsupported combination for the CUDA trainer");
        return;
    }
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

    const bool mini = a.training_strategy == STRATEGY_SMALL_BATCH;
    const uint32_t batch = mini ? a.batch_size : a.sample_count;
    const uint32_t in0 = p->topology[0], outw = p->topology[p->layers - 1], last = p->layers - 1;
    const uint64_t tw = p->total_weights, tb = p->total_biases, np = tw + tb, tn = p->total_neurons;
    spg_log(LOG_INFO, "Starting training: loss=%s, strategy=%s, optimizer=ADAM, compute=CUDA, batch_size=%u, ranks=%d",
            spg_loss_name(p->loss_func), mini ? "SMALL_BATCH" : "FULL_BATCH", batch, s_world);

    spg_train_release(n);
    train_state *t = calloc(1, sizeof *t);
    if (!t) { spg_set_error(SPINGALETT_ERR_ALLOC, "train: state allocation failed"); return; }
    n->train = t;
    void *st = n->stream;
    uint32_t *order = NULL;
    float *h_pinned = NULL;

    DEV(spgk_malloc((void **)&t->params, np * 4), "train: parameters");
    DEV(spgk_malloc((void **)&t->grads, np * 4), "train: gradients");
    DEV(spgk_malloc((void **)&t->m, np * 4), "train: adam m");
    DEV(spgk_malloc((void **)&t->v, np * 4), "train: adam v");
    DEV(spgk_malloc((void **)&t->acts, (size_t)batch * tn * 4), "train: activations");
    DEV(spgk_malloc((void **)&t->deltas, (size_t)batch * tn * 4), "train: deltas");
    DEV(spgk_malloc((void **)&t->data_x, (size_t)a.sample_count * in0 * 4), "train: inputs");
    DEV(spgk_malloc((void **)&t->data_t, (size_t)a.sample_count * outw * 4), "train: targets");
    DEV(spgk_malloc((void **)&t->loss, 256), "train: loss word");
    DEV(spgk_malloc((void **)&t->flag, 256), "train: flag word");
    if (mini) {
        DEV(spgk_malloc((void **)&t->batch_x, (size_t)batch * in0 * 4), "train: batch inputs");
        DEV(spgk_malloc((void **)&t->batch_t, (size_t)batch * outw * 4), "train: batch targets");
        DEV(spgk_malloc((void **)&t->idx, (size_t)a.sample_count * 4), "train: shuffle order");
        order = malloc((size_t)a.sample_count * sizeof *order);
        if (!order) { spg_set_error(SPINGALETT_ERR_ALLOC, "Mini-batch allocation failed"); goto fail; }
        for (uint32_t i = 0; i < a.sample_count; i++) order[i] = i;
    }
    DEV(spgk_memcpy_h2d(t->params, p->weights, tw * 4, st), "train: upload weights");
    DEV(spgk_memcpy_h2d(t->params + tw, p->biases, tb * 4, st), "train: upload biases");
    DEV(spgk_memcpy_h2d(t->m, p->opt_m_weights, tw * 4, st), "train: upload m");
    DEV(spgk_memcpy_h2d(t->m + tw, p->opt_m_biases, tb * 4, st), "train: upload m");
    DEV(spgk_memcpy_h2d(t->v, p->opt_v_weights, tw * 4, st), "train: upload v");
    DEV(spgk_memcpy_h2d(t->v + tw, p->opt_v_biases, tb * 4, st), "train: upload v");
    DEV(spgk_memcpy_h2d(t->data_x, a.inputs, (size_t)a.sample_count * in0 * 4, st), "train: upload inputs");
    DEV(spgk_memcpy_h2d(t->data_t, a.targets, (size_t)a.sample_count * outw * 4, st), "train: upload targets");
    DEV(spgk_memset(t->grads, 0, np * 4, st), "train: clear gradients");
    DEV(spgk_host_alloc((void **)&h_pinned, 256), "train: pinned word");

    float b1pow = 1.0f, b2pow = 1.0f;
    for (size_t epoch = 1; epoch <= a.epochs; epoch++) {
        const bool need_loss = should_report(epoch, a.epochs, a.report_interval) ||
                               (a.callback && should_report(epoch, a.epochs, a.callback_interval));
        if (need_loss) DEV(spgk_memset(t->loss, 0, 4, st), "train: clear loss");
        if (mini) {
            spg_shuffle(order, a.sample_count);
            DEV(spgk_memcpy_h2d(t->idx, order, (size_t)a.sample_count * 4, st), "train: upload order");
            DEV(spgk_stream_sync(st), "train: order sync");        /* `order` is reshuffled next epoch */
        }
        const uint32_t nb = (a.sample_count + batch - 1) / batch;
        for (uint32_t bi = 0; bi < nb; bi++) {
            const uint32_t start = bi * batch;
            const uint32_t cur = start + batch > a.sample_count ? a.sample_count - start : batch;
            const float *bx = t->data_x, *bt = t->data_t;
            if (mini) {
                DEV(spgk_gather_rows2(t->data_x, in0, t->batch_x, t->data_t, outw, t->batch_t, t->idx + start, cur, st),
                    "train: gather mini-batch");
                bx = t->batch_x; bt = t->batch_t;
            }
            /* forward: activations of layer l live at acts + cur*neuron_offsets[l], [cur][width].  An output layer of at
               most 16 units is finished in one launch: product, softmax or sigmoid, delta and (when someone will read
               it) the loss; otherwise product, softmax rows and the delta kernel follow one another */
            float *d_last = t->deltas + (size_t)cur * p->neuron_offsets[last];
            const bool fused_out = outw <= 16;
            const float *x = bx;
            for (uint32_t l = 0; l < last; l++) {
                const uint32_t fi = p->topology[l], fo = p->topology[l + 1];
                float *y = t->acts + (size_t)cur * p->neuron_offsets[l + 1];
                if (l + 1 == last && fused_out) {
                    DEV(spgk_train_output(x, fi, t->params + p->weight_offsets[l], fi, t->params + tw + p->bias_offsets[l], y, bt,
                                          d_last, need_loss ? t->loss : NULL, cur, fo, fi, out_act == ACT_SIGMOID, st),
                        "train: output layer");
                    break;
                }
                DEV(spgk_train_gemm(0, x, fi, t->params + p->weight_offsets[l], fi, y, fo, cur, fo, fi, 1.0f,
                                    t->params + tw + p->bias_offsets[l], NULL, 0, (int)p->act_func[l], st), "train: forward");
                if (p->act_func[l] == ACT_SOFTMAX) DEV(spgk_softmax_rows(y, fo, cur, fo, st), "train: softmax");
                x = y;
            }
            if (!fused_out)
                DEV(spgk_ce_delta(t->acts + (size_t)cur * p->neuron_offsets[last], bt, d_last, (uint64_t)cur * outw,
                                  need_loss ? t->loss : NULL, out_act == ACT_SIGMOID, st), "train: output delta");
            /* backwards through the layers: the gradients of layer l (from delta l+1 and activation l) go into the flat
               buffer and, with several replicas, start their all-reduce on the exchange stream at once, so that it runs
               under the delta and gradient products of the layers below */
            const float gs = 1.0f / (float)cur;
            for (uint32_t l = last; l-- > 0;) {
                const uint32_t fi = p->topology[l], fo = p->topology[l + 1];
                const float *dl = t->deltas + (size_t)cur * p->neuron_offsets[l + 1];
                const float *al = l == 0 ? bx : t->acts + (size_t)cur * p->neuron_offsets[l];
                DEV(spgk_train_grad(dl, fo, al, fi, t->grads + p->weight_offsets[l], fi, t->grads + tw + p->bias_offsets[l],
                                    fo, fi, cur, gs, st), "train: gradients");
                if (s_world > 1) {
                    DEV(spgk_event_record(s_ev_ready, st), "train: exchange order");
                    DEV(spgk_stream_wait_event(s_ar_stream, s_ev_ready), "train: exchange order");
                    if (l == 0)             /* the bias gradients of every layer are complete now: one launch for both */
                        DEV(spgk_nccl_allreduce_sum2(s_comm, t->grads + p->weight_offsets[l], (uint64_t)fi * fo, t->grads + tw, tb,
                                                     s_ar_stream), "train: all-reduce");
                    else
                        DEV(spgk_nccl_allreduce_sum(s_comm, t->grads + p->weight_offsets[l], (uint64_t)fi * fo, s_ar_stream),
                            "train: all-reduce");
                }
                if (l > 0)
                    DEV(spgk_train_gemm(1, dl, fo, t->params + p->weight_offsets[l], fi,
                                        t->deltas + (size_t)cur * p->neuron_offsets[l], fi, cur, fi, fo, 1.0f, NULL,
                                        t->acts + (size_t)cur * p->neuron_offsets[l], fi, (int)p->act_func[l - 1], st), "train: delta");
            }
            if (s_world > 1) {
                DEV(spgk_event_record(s_ev_done, s_ar_stream), "train: exchange order");
                DEV(spgk_stream_wait_event(st, s_ev_done), "train: exchange order");
            }
            p->time_step++;
            b1pow *= a.beta1;
            b2pow *= a.beta2;
            const float mf = 1.0f / (1.0f - b1pow), vf = 1.0f / (1.0f - b2pow);
            DEV(spgk_adam(t->params, t->m, t->v, t->grads, np, a.learning_rate, a.beta1, a.beta2, mf, vf, a.epsilon,
                          1.0f / (float)s_world, st), "train: adam");
        }
        float current_error = 0.0f;
        if (need_loss) {
            DEV(spgk_memcpy_d2h(h_pinned, t->loss, 4, st), "train: read loss");
            DEV(spgk_stream_sync(st), "train: loss sync");
            current_error = h_pinned[0] / (float)a.sample_count;
        }
        if (should_report(epoch, a.epochs, a.report_interval))
            spg_log(LOG_INFO, "Epoch: %zu/%zu, Error: %f", epoch, a.epochs, (double)current_error);
        if (a.nan_check_interval > 0 && epoch % a.nan_check_interval == 0) {
            DEV(spgk_memset(t->flag, 0, 4, st), "train: clear flag");
            DEV(spgk_nonfinite(t->params, np, t->flag, st), "train: nan scan");
            DEV(spgk_memcpy_d2h(h_pinned, t->flag, 4, st), "train: read flag");
            DEV(spgk_stream_sync(st), "train: flag sync");
            if (*(int *)h_pinned) {
                spg_log(LOG_ERROR, "NaN/Inf detected in weights at epoch %zu, stopping training", epoch);
                break;
            }
        }
        if (a.callback && should_report(epoch, a.epochs, a.callback_interval)) {
            /* the callback may read the net: bring the host mirror up to date first */
            DEV(spgk_memcpy_d2h(p->weights, t->params, tw * 4, st), "train: weights to host");
            DEV(spgk_memcpy_d2h(p->biases, t->params + tw, tb * 4, st), "train: biases to host");
            DEV(spgk_stream_sync(st), "train: callback sync");
            if (a.callback(p, epoch, current_error)) {
                spg_log(LOG_INFO, "Training interrupted by callback at epoch %zu", epoch);
                break;
            }
        }
    }
    /* host mirrors of everything the reference leaves in the public struct */
    DEV(spgk_memcpy_d2h(p->weights, t->params, tw * 4, st), "train: weights to host");
    DEV(spgk_memcpy_d2h(p->biases, t->params + tw, tb * 4, st), "train: biases to host");
    DEV(spgk_memcpy_d2h(p->grad_weights, t->grads, tw * 4, st), "train: gradients to host");
    DEV(spgk_memcpy_d2h(p->grad_biases, t->grads + tw, tb * 4, st), "train: gradients to host");
    DEV(spgk_memcpy_d2h(p->opt_m_weights, t->m, tw * 4, st), "train: m to host");
    DEV(spgk_memcpy_d2h(p->opt_m_biases, t->m + tw, tb * 4, st), "train: m to host");
    DEV(spgk_memcpy_d2h(p->opt_v_weights, t->v, tw * 4, st), "train: v to host");
    DEV(spgk_memcpy_d2h(p->opt_v_biases, t->v + tw, tb * 4, st), "train: v to host");
    DEV(spgk_stream_sync(st), "train: final sync");
    spg_log(LOG_INFO, "Training completed.");
fail:
    free(order);
    spgk_host_free(h_pinned);
    spg_train_release(n);
    /* the inference image on the device (possibly a packed payload) no longer matches the weights */
    spg_dev_invalidate(n);
    spg_net_drop_payload(n);
}
