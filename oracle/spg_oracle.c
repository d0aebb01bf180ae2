/*
 * spg_oracle.c -- CPU restatement of Spingalett's forward-inference path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker that the CUDA library is
 * compared against; nothing in the shipped library links, loads or calls it.
 * Only the test-suite, the smoke check and the CPU-baseline leg of the
 * benchmark may use it.
 *
 * Every function restates, in plain C, what the named part of the reference
 * (pka-human/Spingalett, paths relative to that project) computes.  Parity of
 * this restatement with the reference itself is pinned by fixtures that were
 * produced by running the reference's own code (tests/golden/), because the
 * reference ships no test vectors of its own.
 */
#include <math.h>
#include <float.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#if defined(_OPENMP)
#include <omp.h>
#endif

#define SPGO_API __attribute__((visibility("default")))

/* enum values as in Include/Spingalett/Spingalett.h:38-47 and :93-101 */
enum { A_SIGMOID = 0, A_RELU, A_TANH, A_LEAKY, A_FOO52, A_SOFTMAX, A_NONE, A_COUNT };
enum { P_F32 = 0, P_F16, P_BF16, P_I8, P_I4, P_I2, P_COUNT };

/* ------------------------------------------------------------------------- */
/* 16-bit codecs: Src/Spingalett.Serialize.c:12-85                            */
/* ------------------------------------------------------------------------- */

static uint32_t f2u(float x) { uint32_t u; memcpy(&u, &x, 4); return u; }
static float u2f(uint32_t u) { float x; memcpy(&x, &u, 4); return x; }

/* Serialize.c:12-43 -- truncating fp32 -> fp16 (no rounding), fp32 denormals
 * flush to signed zero, overflow saturates to inf, NaN becomes 0x7E00. */
SPGO_API uint16_t spgo_f32_to_f16(float x)
{
    uint32_t u = f2u(x);
    uint16_t s = (uint16_t)((u >> 16) & 0x8000u);
    int e8 = (int)((u >> 23) & 0xFFu);
    uint32_t m = u & 0x7FFFFFu;
    if (e8 == 0) return s;
    if (e8 == 0xFF) return (uint16_t)(s | (m ? 0x7E00u : 0x7C00u));
    int e = e8 - 127;
    if (e > 15) return (uint16_t)(s | 0x7C00u);
    if (e < -24) return s;
    if (e < -14) return (uint16_t)(s | (uint16_t)((m | 0x800000u) >> (-1 - e)));
    return (uint16_t)(s | ((uint32_t)(e + 15) << 10) | (m >> 13));
}

/* Serialize.c:45-72 -- exact fp16 -> fp32 (subnormals renormalised). */
SPGO_API float spgo_f16_to_f32(uint16_t h)
{
    uint32_t s = (uint32_t)(h & 0x8000u) << 16;
    uint32_t e = (h >> 10) & 0x1Fu, m = h & 0x3FFu;
    if (e == 0) {
        if (m == 0) return u2f(s);
        int sh = 0;
        while (!(m & 0x400u)) { m <<= 1; sh++; }
        return u2f(s | ((uint32_t)(113 - sh) << 23) | ((m & 0x3FFu) << 13));
    }
    if (e == 31) return u2f(s | (m ? 0x7FC00000u : 0x7F800000u));
    return u2f(s | ((e + 112u) << 23) | (m << 13));
}

/* Serialize.c:74-85 -- bf16 is the upper half of the fp32 word (truncation). */
SPGO_API uint16_t spgo_f32_to_bf16(float x) { return (uint16_t)(f2u(x) >> 16); }
SPGO_API float spgo_bf16_to_f32(uint16_t h) { return u2f((uint32_t)h << 16); }

/* ------------------------------------------------------------------------- */
/* array payloads                                                             */
/* ------------------------------------------------------------------------- */

/* Bytes one array of `count` elements occupies in a file of this precision
 * (Serialize.c:87-193: integer formats carry one leading float, abs-max). */
SPGO_API uint64_t spgo_array_bytes(uint64_t count, int precision)
{
    switch (precision) {
        case P_F32: return 4 * count;
        case P_F16: case P_BF16: return 2 * count;
        case P_I8: return 4 + count;
        case P_I4: return 4 + (count + 1) / 2;
        case P_I2: return 4 + (count + 3) / 4;
        default: return 0;
    }
}

/* Serialize.c:195-297 -- decode one stored array into fp32. */
SPGO_API void spgo_decode_array(const uint8_t *src, uint64_t count, int precision, float *dst)
{
    if (precision == P_F32) { memcpy(dst, src, 4 * count); return; }
    if (precision == P_F16 || precision == P_BF16) {
        for (uint64_t i = 0; i < count; i++) {
            uint16_t h; memcpy(&h, src + 2 * i, 2);
            dst[i] = precision == P_F16 ? spgo_f16_to_f32(h) : spgo_bf16_to_f32(h);
        }
        return;
    }
    float amax; memcpy(&amax, src, 4);
    const uint8_t *q = src + 4;
    if (!(amax > 0.0f)) { memset(dst, 0, 4 * count); return; }   /* Serialize.c:232-237 */
    if (precision == P_I8) {
        for (uint64_t i = 0; i < count; i++)
            dst[i] = ((float)(int8_t)q[i] / 127.0f) * amax;           /* :234 */
    } else if (precision == P_I4) {
        for (uint64_t i = 0; i < count; i++) {
            uint8_t nib = (i & 1u) ? (uint8_t)(q[i >> 1] >> 4) : (uint8_t)(q[i >> 1] & 0xFu);
            int v = (nib & 8u) ? (int)nib - 16 : (int)nib;            /* :257 sign-extend */
            dst[i] = ((float)v / 7.0f) * amax;                         /* :258 */
        }
    } else { /* P_I2 */
        for (uint64_t i = 0; i < count; i++) {
            uint8_t two = (uint8_t)((q[i >> 2] >> ((i & 3u) * 2u)) & 3u);
            int v = (two & 2u) ? (int)two - 4 : (int)two;             /* :284 */
            dst[i] = (float)v * amax;                                  /* :285 */
        }
    }
}

/* Serialize.c:87-193 -- encode fp32 into a stored array; returns bytes written. */
SPGO_API uint64_t spgo_encode_array(const float *src, uint64_t count, int precision, uint8_t *dst)
{
    uint64_t nbytes = spgo_array_bytes(count, precision);
    if (precision == P_F32) { memcpy(dst, src, 4 * count); return nbytes; }
    if (precision == P_F16 || precision == P_BF16) {
        for (uint64_t i = 0; i < count; i++) {
            uint16_t h = precision == P_F16 ? spgo_f32_to_f16(src[i]) : spgo_f32_to_bf16(src[i]);
            memcpy(dst + 2 * i, &h, 2);
        }
        return nbytes;
    }
    float amax = 0.0f;
    for (uint64_t i = 0; i < count; i++) { float a = fabsf(src[i]); if (a > amax) amax = a; }
    memcpy(dst, &amax, 4);
    uint8_t *q = dst + 4;
    memset(q, 0, nbytes - 4);
    if (!(amax > 0.0f)) return nbytes;
    if (precision == P_I8) {
        for (uint64_t i = 0; i < count; i++)
            q[i] = (uint8_t)(int8_t)roundf((src[i] / amax) * 127.0f);              /* :124 */
    } else if (precision == P_I4) {
        for (uint64_t i = 0; i < count; i++) {
            int v = (int)(int8_t)roundf((src[i] / amax) * 7.0f);                   /* :144-147 */
            if (v > 7) v = 7;
            if (v < -8) v = -8;
            q[i >> 1] |= (uint8_t)(((unsigned)v & 0xFu) << ((i & 1u) * 4u));       /* :148-152 */
        }
    } else {
        for (uint64_t i = 0; i < count; i++) {
            float r = src[i] / amax;
            int v = r > 0.5f ? 1 : (r < -0.5f ? -1 : 0);                           /* :176-179 */
            q[i >> 2] |= (uint8_t)(((unsigned)v & 3u) << ((i & 3u) * 2u));         /* :180-183 */
        }
    }
    return nbytes;
}

/* ------------------------------------------------------------------------- */
/* .nn container: Serialize.c:348-372 (header), :385-407 (payload order)      */
/* ------------------------------------------------------------------------- */

typedef struct {
    uint32_t layers;
    uint32_t *topology;        /* [layers]   */
    uint8_t *act;              /* [layers-1] */
    float *weights;            /* concat of row-major [out][in] matrices (Private.h:16) */
    float *biases;
    uint64_t *w_off, *b_off;   /* [layers-1] */
    uint64_t total_w, total_b;
    uint8_t loss, has_opt, precision;
    uint64_t time_step;
    int truncated;
} spgo_net;

SPGO_API void spgo_free(spgo_net *n)
{
    if (!n) return;
    free(n->topology); free(n->act); free(n->weights); free(n->biases);
    free(n->w_off); free(n->b_off); free(n);
}

/* Parse an in-memory .nn image (Serialize.c:438-528 header, :567-591 payload).
 * Returns NULL where load_spingalett returns NULL; on a short payload the net
 * is returned with `truncated` set and the unread tail left at zero, which is
 * what the reference does (:596-608). */
SPGO_API spgo_net *spgo_parse(const uint8_t *buf, uint64_t len)
{
    uint64_t p = 0;
#define NEED(n) do { if (p + (n) > len) goto bad; } while (0)
    spgo_net *n = (spgo_net *)calloc(1, sizeof *n);
    if (!n) return NULL;
    uint16_t ver;
    NEED(2); memcpy(&ver, buf + p, 2); p += 2;
    if (ver != 1) goto bad;
    NEED(4); memcpy(&n->layers, buf + p, 4); p += 4;
    if (n->layers < 2) goto bad;
    NEED(1); n->loss = buf[p++];
    if (n->loss >= 2) goto bad;
    NEED(1); n->has_opt = buf[p++];
    if (n->has_opt) { NEED(8); memcpy(&n->time_step, buf + p, 8); p += 8; }
    NEED(1); n->precision = buf[p++];
    if (n->precision >= P_COUNT) goto bad;
    if ((uint64_t)n->layers * 4 > len) goto bad;
    n->topology = (uint32_t *)malloc(4 * (size_t)n->layers);
    n->act = (uint8_t *)malloc(n->layers - 1);
    n->w_off = (uint64_t *)malloc(8 * (size_t)(n->layers - 1));
    n->b_off = (uint64_t *)malloc(8 * (size_t)(n->layers - 1));
    NEED(4ull * n->layers); memcpy(n->topology, buf + p, 4ull * n->layers); p += 4ull * n->layers;
    for (uint32_t l = 0; l + 1 < n->layers; l++) {
        NEED(1); n->act[l] = buf[p++];
        if (n->act[l] >= A_COUNT) goto bad;
    }
    for (uint32_t l = 0; l < n->layers; l++)
        if (n->topology[l] == 0) goto bad;            /* layer() rejects 0 neurons, Network.c:53 */
    for (uint32_t l = 0; l + 1 < n->layers; l++) {
        n->w_off[l] = n->total_w; n->b_off[l] = n->total_b;
        n->total_w += (uint64_t)n->topology[l] * n->topology[l + 1];
        n->total_b += n->topology[l + 1];
    }
    n->weights = (float *)calloc(n->total_w ? n->total_w : 1, 4);
    n->biases = (float *)calloc(n->total_b ? n->total_b : 1, 4);
    for (uint32_t l = 0; l + 1 < n->layers; l++) {
        /* element counts are 32-bit in the file format (Serialize.c:390) */
        uint32_t wc = n->topology[l] * n->topology[l + 1], bc = n->topology[l + 1];
        uint64_t wb = spgo_array_bytes(wc, n->precision), bb = spgo_array_bytes(bc, n->precision);
        if (p + wb > len) { n->truncated = 1; break; }
        spgo_decode_array(buf + p, wc, n->precision, n->weights + n->w_off[l]); p += wb;
        if (n->has_opt) { if (p + 2 * wb > len) { n->truncated = 1; break; } p += 2 * wb; }
        if (p + bb > len) { n->truncated = 1; break; }
        spgo_decode_array(buf + p, bc, n->precision, n->biases + n->b_off[l]); p += bb;
        if (n->has_opt) { if (p + 2 * bb > len) { n->truncated = 1; break; } p += 2 * bb; }
    }
    return n;
bad:
    spgo_free(n);
    return NULL;
#undef NEED
}

/* Build an oracle net directly from fp32 arrays (for cases that never touch a file). */
SPGO_API spgo_net *spgo_from_arrays(uint32_t layers, const uint32_t *topology, const uint8_t *act,
                                    const float *weights, const float *biases)
{
    spgo_net *n = (spgo_net *)calloc(1, sizeof *n);
    n->layers = layers;
    n->topology = (uint32_t *)malloc(4 * (size_t)layers);
    n->act = (uint8_t *)malloc(layers - 1);
    n->w_off = (uint64_t *)malloc(8 * (size_t)(layers - 1));
    n->b_off = (uint64_t *)malloc(8 * (size_t)(layers - 1));
    memcpy(n->topology, topology, 4 * (size_t)layers);
    memcpy(n->act, act, layers - 1);
    for (uint32_t l = 0; l + 1 < layers; l++) {
        n->w_off[l] = n->total_w; n->b_off[l] = n->total_b;
        n->total_w += (uint64_t)topology[l] * topology[l + 1];
        n->total_b += topology[l + 1];
    }
    n->weights = (float *)malloc(4 * n->total_w);
    n->biases = (float *)malloc(4 * n->total_b);
    memcpy(n->weights, weights, 4 * n->total_w);
    memcpy(n->biases, biases, 4 * n->total_b);
    return n;
}

SPGO_API uint32_t spgo_layers(const spgo_net *n) { return n->layers; }
SPGO_API const uint32_t *spgo_topology(const spgo_net *n) { return n->topology; }
SPGO_API const uint8_t *spgo_acts(const spgo_net *n) { return n->act; }
SPGO_API float *spgo_weights(spgo_net *n) { return n->weights; }
SPGO_API float *spgo_biases(spgo_net *n) { return n->biases; }
SPGO_API uint64_t spgo_total_weights(const spgo_net *n) { return n->total_w; }
SPGO_API uint64_t spgo_total_biases(const spgo_net *n) { return n->total_b; }
SPGO_API int spgo_precision(const spgo_net *n) { return n->precision; }
SPGO_API int spgo_truncated(const spgo_net *n) { return n->truncated; }
SPGO_API int spgo_has_optimizer(const spgo_net *n) { return n->has_opt; }
SPGO_API uint64_t spgo_time_step(const spgo_net *n) { return n->time_step; }
SPGO_API int spgo_loss(const spgo_net *n) { return n->loss; }

/* ------------------------------------------------------------------------- */
/* activations: Src/Spingalett.Activation.c                                   */
/* ------------------------------------------------------------------------- */

/* Activation.c:23-38.  Strict comparisons: ReLU(0)=0, FOO52(0)=0, FOO52(1)=1;
 * softmax/none/unknown are the identity here. */
SPGO_API float spgo_activate(float x, int act)
{
    switch (act) {
        case A_RELU:    return x > 0.0f ? x : 0.0f;
        case A_LEAKY:   return x > 0.0f ? x : 0.01f * x;
        case A_SIGMOID: return 1.0f / (1.0f + expf(-x));
        case A_TANH:    return tanhf(x);
        case A_FOO52:   return x > 1.0f ? 1.0f + 0.01f * (x - 1.0f) : (x < 0.0f ? 0.01f * x : x);
        default:        return x;
    }
}

/* Activation.c:40-56 -- derivative expressed through the activation OUTPUT. */
SPGO_API float spgo_derivative(float a, int act)
{
    switch (act) {
        case A_RELU:    return a > 0.0f ? 1.0f : 0.0f;
        case A_LEAKY:   return a > 0.0f ? 1.0f : 0.01f;
        case A_SIGMOID: case A_SOFTMAX: return a * (1.0f - a);
        case A_TANH:    return 1.0f - a * a;
        case A_FOO52:   return (a > 1.0f || a < 0.0f) ? 0.01f : 1.0f;
        default:        return 1.0f;
    }
}

/* Activation.c:5-21 -- running max from -FLT_MAX, exp(x-max), normalise only
 * when the sum is positive (a NaN row therefore stays un-normalised). */
SPGO_API void spgo_softmax(float *row, uint32_t n)
{
    float mx = -FLT_MAX;
    for (uint32_t i = 0; i < n; i++) if (row[i] > mx) mx = row[i];
    float sum = 0.0f;
    for (uint32_t i = 0; i < n; i++) { row[i] = expf(row[i] - mx); sum += row[i]; }
    if (sum > 0.0f) {
        float inv = 1.0f / sum;
        for (uint32_t i = 0; i < n; i++) row[i] *= inv;
    }
}

/* SIMD.c:21-88 -- dispatch: softmax on the whole vector, else elementwise. */
static void apply_act(float *v, uint32_t n, int act)
{
    if (act == A_SOFTMAX) { spgo_softmax(v, n); return; }
    if (act == A_NONE || act >= A_COUNT) return;
    for (uint32_t i = 0; i < n; i++) v[i] = spgo_activate(v[i], act);
}

/* SIMD.c:190-240 -- the reference's dot product keeps four 8-lane running
 * sums over strides of 32, folds 8-wide leftovers into the first, combines
 * (s0+s1)+(s2+s3), reduces the 8 lanes as ((l0+l4)+(l1+l5))+((l2+l6)+(l3+l7))
 * and finishes the tail serially.  Restated with the same association so the
 * two agree to the last bit on FMA hardware. */
SPGO_API float spgo_dot(const float *a, const float *b, uint64_t n)
{
    float s[4][8];
    memset(s, 0, sizeof s);
    uint64_t i = 0;
    for (; i + 32 <= n; i += 32)
        for (int g = 0; g < 4; g++)
            for (int l = 0; l < 8; l++)
                s[g][l] = fmaf(a[i + 8 * g + l], b[i + 8 * g + l], s[g][l]);
    for (; i + 8 <= n; i += 8)
        for (int l = 0; l < 8; l++)
            s[0][l] = fmaf(a[i + l], b[i + l], s[0][l]);
    float v[8];
    for (int l = 0; l < 8; l++) v[l] = (s[0][l] + s[1][l]) + (s[2][l] + s[3][l]);
    float q0 = v[0] + v[4], q1 = v[1] + v[5], q2 = v[2] + v[6], q3 = v[3] + v[7];
    float sum = (q0 + q1) + (q2 + q3);
    for (; i < n; i++) sum += a[i] * b[i];
    return sum;
}

/* ------------------------------------------------------------------------- */
/* forward: Src/Spingalett.Network.c:202-251                                  */
/* ------------------------------------------------------------------------- */

SPGO_API uint32_t spgo_max_width(const spgo_net *n)
{
    uint32_t m = 0;
    for (uint32_t l = 0; l < n->layers; l++) if (n->topology[l] > m) m = n->topology[l];
    return m;
}

/* One sample through the chain.  scratch holds 2*max_width floats.
 * Per layer: y = bias (Network.c:227), y[j] += dot(x, row_j) (:241-244),
 * then the activation over the whole vector (:247).  If `acts_out` is given,
 * every layer's activations are appended to it (input included), matching the
 * reference's `neurons` buffer. */
static void forward_one(const spgo_net *n, const float *x, float *out, float *scratch, float *acts_out)
{
    uint32_t mw = spgo_max_width(n);
    float *cur = scratch, *nxt = scratch + mw;
    memcpy(cur, x, 4 * (size_t)n->topology[0]);
    uint64_t apos = 0;
    if (acts_out) { memcpy(acts_out, cur, 4 * (size_t)n->topology[0]); apos = n->topology[0]; }
    for (uint32_t l = 0; l + 1 < n->layers; l++) {
        uint32_t in = n->topology[l], outw = n->topology[l + 1];
        const float *W = n->weights + n->w_off[l];
        const float *b = n->biases + n->b_off[l];
        for (uint32_t j = 0; j < outw; j++)
            nxt[j] = b[j] + spgo_dot(cur, W + (uint64_t)j * in, in);
        apply_act(nxt, outw, n->act[l]);
        if (acts_out) { memcpy(acts_out + apos, nxt, 4 * (size_t)outw); apos += outw; }
        float *t = cur; cur = nxt; nxt = t;
    }
    memcpy(out, cur, 4 * (size_t)n->topology[n->layers - 1]);
}

SPGO_API void spgo_forward(const spgo_net *n, const float *x, float *out)
{
    float *scratch = (float *)malloc(8 * (size_t)spgo_max_width(n));
    forward_one(n, x, out, scratch, NULL);
    free(scratch);
}

/* Batched forward.  The reference's batched form (Training.c:313-345: sgemm,
 * rank-1 bias add, in-place activation / per-row softmax) computes, row by
 * row, the same function as forward(); rows are independent, so the batch is
 * restated as a loop over rows (threads over rows when built with OpenMP).
 * inputs: row-major [N][in]; outputs: row-major [N][out_last]. */
SPGO_API void spgo_forward_batch(const spgo_net *n, const float *inputs, uint64_t N, float *outputs)
{
    uint32_t in0 = n->topology[0], outl = n->topology[n->layers - 1];
    uint32_t mw = spgo_max_width(n);
#if defined(_OPENMP)
#pragma omp parallel
#endif
    {
        float *scratch = (float *)malloc(8 * (size_t)mw);
#if defined(_OPENMP)
#pragma omp for schedule(static)
#endif
        for (int64_t s = 0; s < (int64_t)N; s++)
            forward_one(n, inputs + (uint64_t)s * in0, outputs + (uint64_t)s * outl, scratch, NULL);
        free(scratch);
    }
}

/* Same, keeping every layer's activations: acts is [N][sum(topology)]. */
SPGO_API void spgo_forward_batch_acts(const spgo_net *n, const float *inputs, uint64_t N, float *acts)
{
    uint32_t in0 = n->topology[0], outl = n->topology[n->layers - 1];
    uint32_t mw = spgo_max_width(n);
    uint64_t tn = 0;
    for (uint32_t l = 0; l < n->layers; l++) tn += n->topology[l];
    float *scratch = (float *)malloc(8 * (size_t)mw);
    float *o = (float *)malloc(4 * (size_t)outl);
    for (uint64_t s = 0; s < N; s++)
        forward_one(n, inputs + s * in0, o, scratch, acts + s * tn);
    free(o); free(scratch);
}

/* ------------------------------------------------------------------------- */
/* one mini-batch training step (cross-entropy, Adam)                         */
/* ------------------------------------------------------------------------- */

/* Gradients of one batch, restating Training.c:347-419 for the case the
 * training configuration uses (cross-entropy with a softmax or sigmoid output
 * layer):  delta_L = a_L - t (:366-371);  delta_l = (delta_{l+1} W_l) * act'(a_l)
 * (:374-393);  gW_l = scale * delta_{l+1}^T a_l, gB_l = scale * column sums
 * (:396-419).  Sums run in double so the result is a tight reference for the
 * GPU's fp32 reductions.  grads: [gW (total_w) | gB (total_b)]. */
SPGO_API void spgo_batch_gradients(const spgo_net *n, const float *inputs, const float *targets,
                                   uint32_t N, float scale, float *grads)
{
    uint32_t L = n->layers;
    uint64_t tn = 0;
    for (uint32_t l = 0; l < L; l++) tn += n->topology[l];
    float *acts = (float *)malloc(4 * (size_t)(tn * N));
    spgo_forward_batch_acts(n, inputs, N, acts);
    uint64_t *noff = (uint64_t *)malloc(8 * (size_t)L);
    uint64_t o = 0;
    for (uint32_t l = 0; l < L; l++) { noff[l] = o; o += n->topology[l]; }
    float *delta = (float *)calloc((size_t)(tn * N), 4);
    uint32_t last = L - 1, nout = n->topology[last];
    for (uint32_t s = 0; s < N; s++)
        for (uint32_t j = 0; j < nout; j++)
            delta[s * tn + noff[last] + j] = acts[s * tn + noff[last] + j] - targets[(uint64_t)s * nout + j];
    for (uint32_t l = last - 1; l > 0; l--) {
        uint32_t cur = n->topology[l], nxt = n->topology[l + 1];
        const float *W = n->weights + n->w_off[l];
        int act = n->act[l - 1];
#if defined(_OPENMP)
#pragma omp parallel for schedule(static)
#endif
        for (int64_t s = 0; s < (int64_t)N; s++) {
            for (uint32_t k = 0; k < cur; k++) {
                double acc = 0.0;
                for (uint32_t j = 0; j < nxt; j++)
                    acc += (double)delta[s * tn + noff[l + 1] + j] * (double)W[(uint64_t)j * cur + k];
                delta[s * tn + noff[l] + k] = (float)acc * spgo_derivative(acts[s * tn + noff[l] + k], act);
            }
        }
    }
    float *gW = grads, *gB = grads + n->total_w;
    for (uint32_t l = 0; l < last; l++) {
        uint32_t in = n->topology[l], out = n->topology[l + 1];
#if defined(_OPENMP)
#pragma omp parallel for schedule(static)
#endif
        for (int64_t j = 0; j < (int64_t)out; j++) {
            double bs = 0.0;
            for (uint32_t s = 0; s < N; s++) bs += delta[s * tn + noff[l + 1] + j];
            gB[n->b_off[l] + j] = scale * (float)bs;
            for (uint32_t k = 0; k < in; k++) {
                double acc = 0.0;
                for (uint32_t s = 0; s < N; s++)
                    acc += (double)delta[s * tn + noff[l + 1] + j] * (double)acts[s * tn + noff[l] + k];
                gW[n->w_off[l] + (uint64_t)j * in + k] = scale * (float)acc;
            }
        }
    }
    free(delta); free(noff); free(acts);
}

/* SIMD.c:279-328 -- Adam with epsilon INSIDE the square root:
 * m = b1 m + (1-b1) g;  v = b2 v + (1-b2) g^2;
 * w -= lr * (m*mf) / sqrt(v*vf + eps),  mf = 1/(1-b1^t), vf = 1/(1-b2^t)
 * (factors formed by the caller as in Training.c:480-482). */
SPGO_API void spgo_adam(float *w, float *m, float *v, const float *g, uint64_t n,
                        float lr, float b1, float b2, float mf, float vf, float eps)
{
    float omb1 = 1.0f - b1, omb2 = 1.0f - b2;
    for (uint64_t i = 0; i < n; i++) {
        m[i] = fmaf(b1, m[i], omb1 * g[i]);
        v[i] = fmaf(b2, v[i], omb2 * (g[i] * g[i]));
        float mh = m[i] * mf, vh = v[i] * vf + eps;
        w[i] -= lr * (mh / sqrtf(vh));
    }
}

/* SIMD.c:522-552 (cross-entropy branch): -sum t*log(max(o,1e-9)). */
SPGO_API float spgo_cross_entropy(const float *out, const float *target, uint32_t n)
{
    float e = 0.0f;
    for (uint32_t i = 0; i < n; i++) {
        float o = out[i] > 1e-9f ? out[i] : 1e-9f;
        e -= target[i] * logf(o);
    }
    return e;
}

SPGO_API int spgo_threads(void)
{
#if defined(_OPENMP)
    return omp_get_max_threads();
#else
    return 1;
#endif
}
