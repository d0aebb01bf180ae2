/*
 * ref_harness.c -- test-only window into the UNMODIFIED reference.
 *
 * Compiled together with the reference's own sources where they lie (never
 * copied), this translation unit textually includes the reference's
 * Src/Spingalett.Training.c so that its file-static batched routines
 * (batch_forward :313, batch_compute_deltas :347, batch_accumulate_gradients
 * :396) become callable, and re-exports the internal seeding hook rng_seed
 * (Src/Spingalett.Random.c:18) that the public API hides.  Used to generate
 * golden fixtures and as the "reference" CPU baseline; never linked into the
 * product.
 */
#include "Spingalett.Training.c"

#define REFH_API __attribute__((visibility("default")))

REFH_API void refh_rng_seed(uint64_t seed) { rng_seed(seed); }

REFH_API int refh_has_blas(void)
{
#if defined(SPINGALETT_HAS_OPENBLAS)
    return 1;
#else
    return 0;
#endif
}

REFH_API void refh_blas_threads(int n)
{
#if defined(SPINGALETT_HAS_OPENBLAS)
    openblas_set_num_threads(n);
#else
    (void)n;
#endif
}

/* Batched forward of N rows; outputs [N][out_last].  With OpenBLAS this is the
 * reference's own batch_forward(); without it, a loop over its forward(). */
REFH_API int refh_batch_forward(NeuralNetwork *net, const float *inputs, uint32_t N, float *outputs)
{
    uint32_t last = net->layers - 1, nout = net->topology[last];
#if defined(SPINGALETT_HAS_OPENBLAS)
    BatchWorkspace *ws = batch_workspace_create(net, N);
    if (!ws) return -1;
    batch_forward(net, ws, inputs, N);
    memcpy(outputs, ws->act[last], (size_t)N * nout * sizeof(float));
    batch_workspace_free(ws);
#else
    for (uint32_t s = 0; s < N; s++) {
        float *o = forward_struct_arguments((ForwardArgs){ net, inputs + (size_t)s * net->topology[0] });
        if (!o) return -1;
        memcpy(outputs + (size_t)s * nout, o, nout * sizeof(float));
    }
#endif
    return 0;
}

/* Persistent-workspace variant for timing: create once, run many. */
REFH_API void *refh_ws_create(NeuralNetwork *net, uint32_t N)
{
#if defined(SPINGALETT_HAS_OPENBLAS)
    return batch_workspace_create(net, N);
#else
    (void)net; (void)N; return NULL;
#endif
}
REFH_API void refh_ws_free(void *ws)
{
#if defined(SPINGALETT_HAS_OPENBLAS)
    batch_workspace_free((BatchWorkspace *)ws);
#else
    (void)ws;
#endif
}
REFH_API const float *refh_ws_forward(NeuralNetwork *net, void *ws, const float *inputs, uint32_t N)
{
#if defined(SPINGALETT_HAS_OPENBLAS)
    batch_forward(net, (BatchWorkspace *)ws, inputs, N);
    return ((BatchWorkspace *)ws)->act[net->layers - 1];
#else
    (void)net; (void)ws; (void)inputs; (void)N; return NULL;
#endif
}

/* Gradients of one batch exactly as the reference's mini-batch path forms
 * them: results land in net->grad_weights / net->grad_biases. */
REFH_API int refh_batch_gradients(NeuralNetwork *net, const float *inputs, const float *targets,
                                  uint32_t N, float scale)
{
#if defined(SPINGALETT_HAS_OPENBLAS)
    BatchWorkspace *ws = batch_workspace_create(net, N);
    if (!ws) return -1;
    batch_forward(net, ws, inputs, N);
    batch_compute_deltas(net, ws, targets, N);
    batch_accumulate_gradients(net, ws, N, scale);
    batch_workspace_free(ws);
    return 0;
#else
    (void)net; (void)inputs; (void)targets; (void)N; (void)scale;
    return -2;
#endif
}

REFH_API void refh_adam(float *w, float *m, float *v, const float *g, uint64_t n,
                        float lr, float b1, float b2, float mf, float vf, float eps)
{
    spingalett_adam_update_avx(w, m, v, g, n, lr, b1, b2, 1.0f - b1, 1.0f - b2, mf, vf, eps);
}

REFH_API float refh_dot(const float *a, const float *b, uint64_t n) { return spingalett_dot_product(a, b, n); }
REFH_API void refh_softmax(float *row, uint32_t n) { apply_softmax(row, n); }
REFH_API void refh_activation_bulk(float *d, uint64_t n, int act) { apply_activation_bulk(d, n, (ActivationFunction)act); }
REFH_API float refh_normal(void) { return random_normal_weight(); }
REFH_API float refh_uniform(void) { return random_uniform_weight(); }
REFH_API uint32_t refh_rng_next(void) { return rng_next(); }
REFH_API size_t refh_sizeof_net(void) { return sizeof(NeuralNetwork); }
REFH_API size_t refh_sizeof_trainargs(void) { return sizeof(TrainArgs); }
