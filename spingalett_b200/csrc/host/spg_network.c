/* Model container and the single-sample forward entry point.
 *
 * The public struct keeps the reference's flat layout (weights: concatenated
 * row-major [out][in] matrices; offsets as in Network.c:16-32), but a layer is
 * appended by growing each array in place of the reference's copy-everything
 * step, and the gradient / optimizer arrays are only created when training
 * first needs them.  forward() never computes on the CPU: it uploads the
 * sample, runs the layer chain on the GPU and copies the activations back
 * into net->neurons. */
#include "spg_internal.h"
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

/* 64-byte aligned, zero-filled fp32 array of `count` elements (count 0 -> 64 bytes) */
static float *zeros_f32(uint64_t count)
{
    size_t bytes = (size_t)count * sizeof(float);
    bytes = (bytes + 63u) & ~(size_t)63u;
    if (bytes == 0) bytes = 64;
    return calloc(1, bytes);
}

/* Grow *arr to new_count elements, new tail zero-filled.  realloc lets the allocator extend large
 * blocks in place (mremap) instead of copying, which matters for nets with 1e8..1e9 weights. */
static bool grow_f32(float **arr, uint64_t old_count, uint64_t new_count)
{
    if (!*arr) {
        *arr = zeros_f32(new_count);
        return *arr != NULL;
    }
    size_t bytes = (size_t)new_count * sizeof(float);
    float *p = realloc(*arr, bytes ? bytes : 64);
    if (!p) return false;
    if (new_count > old_count) memset(p + old_count, 0, (size_t)(new_count - old_count) * sizeof(float));
    *arr = p;
    return true;
}

static void recompute_offsets(NeuralNetwork *n)
{
    uint64_t no = 0, wo = 0, bo = 0;
    for (uint32_t l = 0; l < n->layers; l++) {
        n->neuron_offsets[l] = no;
        no += n->topology[l];
        if (l + 1 < n->layers) {
            n->weight_offsets[l] = wo;
            n->bias_offsets[l] = bo;
            wo += (uint64_t)n->topology[l] * n->topology[l + 1];
            bo += n->topology[l + 1];
        }
    }
    n->neuron_offsets[n->layers] = no;
    n->total_neurons = no;
    n->total_weights = wo;
    n->total_biases = bo;
}

NeuralNetwork *new_spingalett_struct_arguments(NeuralNetworkArgs args)
{
    if ((unsigned)args.loss_func >= LOSS_COUNT) {
        spg_set_error(SPINGALETT_ERR_INVALID, "Invalid loss function");
        return NULL;
    }
    spg_log(LOG_INFO, "Creating new network with %s loss function", spg_loss_name(args.loss_func));
    spg_net *n = calloc(1, sizeof *n);
    if (!n) { spg_set_error(SPINGALETT_ERR_ALLOC, "NeuralNetwork calloc failed"); return NULL; }
    n->magic = SPG_NET_MAGIC;
    n->pub.loss_func = args.loss_func;
    n->store_precision = PRECISION_FLOAT32;
    n->device = -1;
    return &n->pub;
}

void spg_net_drop_payload(spg_net *n)
{
    for (uint32_t l = 0; l < n->payload_layers; l++) free(n->payload_w[l]);
    free(n->payload_w); free(n->payload_w_bytes); free(n->amax_w);
    n->payload_w = NULL; n->payload_w_bytes = NULL; n->amax_w = NULL;
    n->payload_layers = 0;
    n->store_precision = PRECISION_FLOAT32;
}

void layer_struct_arguments(LayerArgs args)
{
    NeuralNetwork *n = args.net;
    if (!n || args.neurons_amount == 0) {
        spg_set_error(SPINGALETT_ERR_INVALID, "Net is NULL or neurons amount is 0");
        return;
    }
    spg_net *pn = spg_priv(n);
    const bool has_weights = n->layers > 0;          /* this call adds a weight matrix */
    if (!has_weights) {
        spg_log(LOG_INFO, "Layer #0: Neurons amount: %u", args.neurons_amount);
    } else {
        if ((unsigned)args.act_func >= ACT_COUNT) {
            spg_set_error(SPINGALETT_ERR_INVALID, "Invalid activation function");
            return;
        }
        if ((unsigned)args.weight_initialization >= WEIGHT_INITIALIZATION_COUNT) {
            spg_set_error(SPINGALETT_ERR_INVALID, "Invalid weight initialization");
            return;
        }
        spg_log(LOG_INFO, "Layer #%u: Neurons amount: %u, Activation function: %s", n->layers,
                args.neurons_amount, spg_act_name(args.act_func));
    }

    const uint32_t nl = n->layers + 1;
    const uint32_t fan_in = has_weights ? n->topology[n->layers - 1] : 0;
    const uint64_t add_w = (uint64_t)fan_in * args.neurons_amount;
    const uint64_t add_b = has_weights ? args.neurons_amount : 0;
    const uint64_t old_w = n->total_weights, old_b = n->total_biases, old_n = n->total_neurons;

    uint32_t *topo = realloc(n->topology, nl * sizeof *topo);
    if (topo) n->topology = topo;
    uint64_t *noff = realloc(n->neuron_offsets, (nl + 1) * sizeof *noff);
    if (noff) n->neuron_offsets = noff;
    uint64_t *woff = realloc(n->weight_offsets, nl * sizeof *woff);
    if (woff) n->weight_offsets = woff;
    uint64_t *boff = realloc(n->bias_offsets, nl * sizeof *boff);
    if (boff) n->bias_offsets = boff;
    ActivationFunction *acts = n->act_func;
    if (has_weights) {
        acts = realloc(n->act_func, (nl - 1) * sizeof *acts);
        if (acts) n->act_func = acts;
    }
    bool ok = topo && noff && woff && boff && (!has_weights || acts);
    ok = ok && grow_f32(&n->neurons, old_n, old_n + args.neurons_amount);
    if (ok && has_weights) {
        ok = grow_f32(&n->weights, old_w, old_w + add_w) && grow_f32(&n->biases, old_b, old_b + add_b);
        /* arrays that only exist once training has run keep their contents too */
        if (ok && n->grad_weights)
            ok = grow_f32(&n->grad_weights, old_w, old_w + add_w) && grow_f32(&n->grad_biases, old_b, old_b + add_b) &&
                 grow_f32(&n->opt_m_weights, old_w, old_w + add_w) && grow_f32(&n->opt_m_biases, old_b, old_b + add_b) &&
                 grow_f32(&n->opt_v_weights, old_w, old_w + add_w) && grow_f32(&n->opt_v_biases, old_b, old_b + add_b);
    }
    if (!ok) {
        spg_set_error(SPINGALETT_ERR_ALLOC, "Layer allocation failed");
        return;
    }

    n->topology[n->layers] = args.neurons_amount;
    if (has_weights) {
        n->act_func[n->layers - 1] = args.act_func;
        /* Network.c:150-162: HE = N(0,1)*sqrt(2/fan_in), "XAVIER" = N(0,1)*sqrt(1/fan_in),
         * RANDOM = U(-1,1), NONE leaves zeros; biases start at zero. */
        float *w = n->weights + old_w;
        switch (args.weight_initialization) {
            case WEIGHT_INITIALIZATION_RANDOM:
                for (uint64_t i = 0; i < add_w; i++) w[i] = spg_rand_uniform_pm1();
                break;
            case WEIGHT_INITIALIZATION_XAVIER: {
                float s = sqrtf(1.0f / (float)fan_in);
                for (uint64_t i = 0; i < add_w; i++) w[i] = spg_rand_normal() * s;
                break;
            }
            case WEIGHT_INITIALIZATION_HE: {
                float s = sqrtf(2.0f / (float)fan_in);
                for (uint64_t i = 0; i < add_w; i++) w[i] = spg_rand_normal() * s;
                break;
            }
            default: break;
        }
    }
    n->layers = nl;
    recompute_offsets(n);
    /* the device image and any packed payload no longer describe this net */
    spg_dev_invalidate(pn);
    if (pn->payload_layers) spg_net_drop_payload(pn);
}

int spg_net_ensure_train_arrays(spg_net *pn)
{
    NeuralNetwork *n = &pn->pub;
    if (n->grad_weights) return SPINGALETT_OK;
    float **w[] = { &n->grad_weights, &n->opt_m_weights, &n->opt_v_weights };
    float **b[] = { &n->grad_biases, &n->opt_m_biases, &n->opt_v_biases };
    for (int i = 0; i < 3; i++) {
        *w[i] = zeros_f32(n->total_weights);
        *b[i] = zeros_f32(n->total_biases);
        if (!*w[i] || !*b[i]) {
            for (int k = 0; k < 3; k++) { free(*w[k]); free(*b[k]); *w[k] = NULL; *b[k] = NULL; }
            spg_set_error(SPINGALETT_ERR_ALLOC, "training array allocation failed");
            return SPINGALETT_ERR_ALLOC;
        }
    }
    return SPINGALETT_OK;
}

float activate(float x, ActivationFunction a)
{
    switch (a) {
        case ACT_SIGMOID:    return 1.0f / (1.0f + expf(-x));
        case ACT_RELU:       return x > 0.0f ? x : 0.0f;
        case ACT_TANH:       return tanhf(x);
        case ACT_LEAKY_RELU: return x > 0.0f ? x : 0.01f * x;
        case ACT_FOO52:      return x < 0.0f ? 0.01f * x : (x > 1.0f ? 1.0f + 0.01f * (x - 1.0f) : x);
        default:             return x;
    }
}

float derivative(float a, ActivationFunction f)
{
    switch (f) {
        case ACT_SIGMOID: case ACT_SOFTMAX: return a * (1.0f - a);
        case ACT_RELU:       return a > 0.0f ? 1.0f : 0.0f;
        case ACT_TANH:       return 1.0f - a * a;
        case ACT_LEAKY_RELU: return a > 0.0f ? 1.0f : 0.01f;
        case ACT_FOO52:      return (a < 0.0f || a > 1.0f) ? 0.01f : 1.0f;
        default:             return 1.0f;
    }
}

float *forward_struct_arguments(ForwardArgs args)
{
    NeuralNetwork *n = args.net;
    if (!n || !args.input) return NULL;                       /* silent, as Network.c:207 */
    if (n->layers < 2) {
        spg_set_error(SPINGALETT_ERR_INVALID, "Network must have at least 2 layers for forward pass");
        return NULL;
    }
    spg_net *pn = spg_priv(n);
    if (spg_dev_ensure(pn) != SPINGALETT_OK) return NULL;
    /* stage the sample in pinned memory so the copy is a true async DMA */
    size_t need = (size_t)n->total_neurons * sizeof(float);
    if (pn->h_stage_bytes < need) {
        spgk_host_free(pn->h_stage); pn->h_stage = NULL; pn->h_stage_bytes = 0;
        void *p = NULL;
        if (spg_map_kernel_error(spgk_host_alloc(&p, need), "forward: pinned staging")) return NULL;
        pn->h_stage = p; pn->h_stage_bytes = need;
    }
    memcpy(pn->h_stage, args.input, (size_t)n->topology[0] * sizeof(float));
    /* the workspace holds every layer's activations; slot 0 is the input */
    if (spg_dev_forward_small(pn, NULL, 0, 1, NULL, NULL) != SPINGALETT_OK) return NULL;      /* reserve */
    if (spg_map_kernel_error(spgk_memcpy_h2d(pn->d_small, pn->h_stage, (size_t)n->topology[0] * sizeof(float), pn->stream),
                             "forward: input copy")) return NULL;
    float *d_last = NULL;
    if (spg_dev_forward_small(pn, NULL, 0, 1, &d_last, NULL) != SPINGALETT_OK) return NULL;
    if (spg_map_kernel_error(spgk_memcpy_d2h(pn->h_stage, pn->d_small, need, pn->stream), "forward: copy back")) return NULL;
    if (spg_map_kernel_error(spgk_stream_sync(pn->stream), "forward: sync")) return NULL;
    memcpy(n->neurons, pn->h_stage, need);
    return n->neurons + n->neuron_offsets[n->layers - 1];
}

void print_parameters(NeuralNetwork *n)
{
    if (!n) return;
    spg_log(LOG_INFO, "========== NETWORK PARAMETERS ==========");
    spg_log(LOG_INFO, "Loss: %s, stored precision on device: %s", spg_loss_name(n->loss_func),
            spg_precision_name(spg_priv(n)->store_precision));
    for (uint32_t l = 0; l + 1 < n->layers; l++) {
        uint32_t in = n->topology[l], out = n->topology[l + 1];
        spg_log(LOG_INFO, "[Layer %u (%u) -> Layer %u (%u), activation %s]", l, in, l + 1, out, spg_act_name(n->act_func[l]));
        for (uint32_t j = 0; j < out; j++)
            spg_log(LOG_INFO, "    bias[%u] = %12.6g", j, (double)n->biases[n->bias_offsets[l] + j]);
        for (uint32_t k = 0; k < in; k++)
            for (uint32_t j = 0; j < out; j++)
                spg_log(LOG_INFO, "    L%u N%u -> L%u N%u: %12.6g", l, k, l + 1, j,
                        (double)n->weights[n->weight_offsets[l] + (uint64_t)j * in + k]);
    }
    spg_log(LOG_INFO, "========================================");
}

void free_network(NeuralNetwork *n)
{
    if (!n) return;
    spg_net *pn = spg_priv(n);
    spg_train_release(pn);
    spg_dev_release(pn);
    spgk_host_free(pn->h_out);
    spgk_host_free(pn->h_stage);
    spg_net_drop_payload(pn);
    free(n->neurons); free(n->weights); free(n->biases);
    free(n->grad_weights); free(n->grad_biases);
    free(n->opt_m_weights); free(n->opt_m_biases);
    free(n->opt_v_weights); free(n->opt_v_biases);
    free(n->neuron_offsets); free(n->weight_offsets); free(n->bias_offsets);
    free(n->topology); free(n->act_func);
    pn->magic = 0;
    free(pn);
    spg_log(LOG_DEBUG, "Memory freed.");
}
