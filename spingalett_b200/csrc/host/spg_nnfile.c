/* .nn files: load_spingalett / save_spingalett.
 *
 * Layout (little-endian, unpadded; reference Serialize.c:348-372 header,
 * :385-407 payload order): u16 version=1, u32 layers, u8 loss,
 * u8 has_optimizer, [u64 time_step], u8 precision, u32 topology[layers],
 * u8 act[layers-1]; then per weight layer: W [mW vW] b [mB vB], every array in
 * the file's precision.
 *
 * The loader keeps each packed weight matrix as read so the GPU can hold it
 * in its stored precision, and fills net->weights / net->biases with the fp32
 * values the reference loader produces (:567-591). */
#include "spg_internal.h"
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

typedef struct { const uint8_t *p; size_t len, pos; } cursor;

static bool take(cursor *c, void *dst, size_t n)
{
    if (c->len - c->pos < n) return false;
    memcpy(dst, c->p + c->pos, n);
    c->pos += n;
    return true;
}

static uint8_t *slurp(const char *path, size_t *len)
{
    FILE *f = fopen(path, "rb");
    if (!f) return NULL;
    uint8_t *buf = NULL;
    if (fseek(f, 0, SEEK_END) == 0) {
        long sz = ftell(f);
        if (sz >= 0 && fseek(f, 0, SEEK_SET) == 0) {
            buf = malloc((size_t)sz + 1);
            if (buf && fread(buf, 1, (size_t)sz, f) != (size_t)sz) { free(buf); buf = NULL; }
            *len = (size_t)sz;
        }
    }
    fclose(f);
    return buf;
}

/* read one stored array: decode to fp32 and optionally keep the packed bytes */
static bool read_array(cursor *c, uint32_t count, PrecisionMode p, float *dst, uint8_t **keep, size_t *keep_bytes, float *amax)
{
    size_t nbytes = spg_array_bytes(count, p);
    if (c->len - c->pos < nbytes) return false;
    const uint8_t *src = c->p + c->pos;
    spg_decode_array(src, count, p, dst);
    if (keep) {
        size_t skip = p >= PRECISION_INT8 ? 4 : 0;
        if (skip) memcpy(amax, src, 4); else *amax = 0.0f;
        *keep_bytes = nbytes - skip;
        *keep = malloc(*keep_bytes ? *keep_bytes : 1);
        if (!*keep) return false;
        memcpy(*keep, src + skip, *keep_bytes);
    }
    c->pos += nbytes;
    return true;
}

NeuralNetwork *load_spingalett(const char *filename)
{
    if (!filename) { spg_set_error(SPINGALETT_ERR_INVALID, "load: filename is NULL"); return NULL; }
    size_t len = 0;
    uint8_t *buf = slurp(filename, &len);
    if (!buf) { spg_set_error(SPINGALETT_ERR_INVALID, "load: cannot open file for reading"); return NULL; }
    cursor c = { buf, len, 0 };
    NeuralNetwork *net = NULL;
    uint32_t *topo = NULL;
    uint8_t *acts = NULL;

    uint16_t version = 0;
    if (!take(&c, &version, 2)) { spg_set_error(SPINGALETT_ERR_INVALID, "load: failed to read format version"); goto fail; }
    if (version != SPINGALETT_FORMAT_VERSION) {
        spg_set_error(SPINGALETT_ERR_INVALID, "load: unsupported format version");
        spg_log(LOG_ERROR, "Unsupported file format version %u (expected %u)", (unsigned)version, (unsigned)SPINGALETT_FORMAT_VERSION);
        goto fail;
    }
    uint32_t layers = 0;
    if (!take(&c, &layers, 4)) { spg_set_error(SPINGALETT_ERR_INVALID, "load: failed to read layer count"); goto fail; }
    if (layers < 2) { spg_set_error(SPINGALETT_ERR_INVALID, "load: network must have at least 2 layers"); goto fail; }
    uint8_t loss = 0, has_opt = 0, prec8 = 0;
    if (!take(&c, &loss, 1) || loss >= LOSS_COUNT) { spg_set_error(SPINGALETT_ERR_INVALID, "load: invalid loss type"); goto fail; }
    if (!take(&c, &has_opt, 1)) { spg_set_error(SPINGALETT_ERR_INVALID, "load: failed to read optimizer flag"); goto fail; }
    uint64_t time_step = 0;
    if (has_opt && !take(&c, &time_step, 8)) { spg_set_error(SPINGALETT_ERR_INVALID, "load: failed to read time step"); goto fail; }
    if (!take(&c, &prec8, 1) || prec8 >= PRECISION_COUNT) { spg_set_error(SPINGALETT_ERR_INVALID, "load: invalid precision type"); goto fail; }
    const PrecisionMode prec = (PrecisionMode)prec8;
    if ((size_t)layers * 4 > c.len - c.pos) { spg_set_error(SPINGALETT_ERR_INVALID, "load: failed to read topology"); goto fail; }
    topo = malloc((size_t)layers * 4);
    acts = malloc(layers - 1);
    if (!topo || !acts) { spg_set_error(SPINGALETT_ERR_ALLOC, "load: topology allocation failed"); goto fail; }
    take(&c, topo, (size_t)layers * 4);
    for (uint32_t l = 0; l + 1 < layers; l++) {
        if (!take(&c, &acts[l], 1) || acts[l] >= ACT_COUNT) { spg_set_error(SPINGALETT_ERR_INVALID, "load: invalid activation function"); goto fail; }
    }

    net = new_spingalett_struct_arguments((NeuralNetworkArgs){ .loss_func = (LossFunction)loss });
    if (!net) { spg_set_error(SPINGALETT_ERR_ALLOC, "load: network creation failed"); goto fail; }
    net->time_step = time_step;
    for (uint32_t l = 0; l < layers; l++) {
        layer_struct_arguments((LayerArgs){ .net = net, .neurons_amount = topo[l],
                                            .act_func = l ? (ActivationFunction)acts[l - 1] : ACT_SIGMOID,
                                            .weight_initialization = WEIGHT_INITIALIZATION_NONE });
        /* the error state is sticky: any error left pending (even an older
         * one) aborts the load, as in the reference (Serialize.c:556) */
        if (spingalett_last_error_code() != SPINGALETT_OK) goto fail;
    }
    spg_net *pn = spg_priv(net);
    const uint32_t wl = layers - 1;
    if (has_opt && spg_net_ensure_train_arrays(pn) != SPINGALETT_OK) goto fail;
    pn->payload_w = calloc(wl, sizeof *pn->payload_w);
    pn->payload_w_bytes = calloc(wl, sizeof *pn->payload_w_bytes);
    pn->amax_w = calloc(wl, sizeof *pn->amax_w);
    if (!pn->payload_w || !pn->payload_w_bytes || !pn->amax_w) { spg_set_error(SPINGALETT_ERR_ALLOC, "load: payload table allocation failed"); goto fail; }
    pn->payload_layers = wl;
    pn->store_precision = prec;

    bool ok = true;
    for (uint32_t l = 0; l < wl && ok; l++) {
        /* element counts are 32-bit in the format (Serialize.c:390) */
        uint32_t wc = net->topology[l] * net->topology[l + 1], bc = net->topology[l + 1];
        uint64_t wo = net->weight_offsets[l], bo = net->bias_offsets[l];
        ok = read_array(&c, wc, prec, net->weights + wo, &pn->payload_w[l], &pn->payload_w_bytes[l], &pn->amax_w[l]);
        if (ok && has_opt)
            ok = read_array(&c, wc, prec, net->opt_m_weights + wo, NULL, NULL, NULL) &&
                 read_array(&c, wc, prec, net->opt_v_weights + wo, NULL, NULL, NULL);
        if (ok) ok = read_array(&c, bc, prec, net->biases + bo, NULL, NULL, NULL);
        if (ok && has_opt)
            ok = read_array(&c, bc, prec, net->opt_m_biases + bo, NULL, NULL, NULL) &&
                 read_array(&c, bc, prec, net->opt_v_biases + bo, NULL, NULL, NULL);
    }
    if (!ok) {
        /* partly filled net is still handed back (Serialize.c:596-608); the GPU
         * then works from the fp32 arrays because the packed set is incomplete */
        spg_net_drop_payload(pn);
        spg_set_error(SPINGALETT_ERR_INVALID, "load: file appears truncated or corrupt");
        spg_log(LOG_WARNING, "Network file may be truncated: %s", filename);
    }
    spg_log(LOG_INFO, "Network loaded from %s", filename);
    spg_log(LOG_INFO, "Load info: format=v%u, layers=%u, weights=%llu, biases=%llu, precision=%s, optimizer=%s",
            (unsigned)version, layers, (unsigned long long)net->total_weights, (unsigned long long)net->total_biases,
            spg_precision_name(prec), has_opt ? "ON" : "OFF");
    free(topo); free(acts); free(buf);
    return net;
fail:
    free(topo); free(acts); free(buf);
    free_network(net);
    return NULL;
}

/* Arrays of a million elements or more are quantised on the GPU when one is there (upload, encode kernels, read
 * the packed bytes back: the scalar host loops below take seconds on a half-billion-weight net); the bytes are
 * the same either way, and without a device, with SPINGALETT_HOST_ENCODE set in the environment, or if anything on
 * that route fails, the host encoder does the work. */
#define SPG_DEV_ENCODE_MIN (1u << 20)
typedef struct { float *d_src; uint8_t *d_dst; bool ok; } dev_encoder;

static void dev_encoder_open(dev_encoder *de, uint32_t max_count)
{
    de->d_src = NULL; de->d_dst = NULL; de->ok = false;
    int count = 0;
    if (max_count < SPG_DEV_ENCODE_MIN || getenv("SPINGALETT_HOST_ENCODE") || spgk_device_count(&count) != 0 || count <= 0) return;
    void *a = NULL, *b = NULL;
    if (spgk_malloc(&a, (size_t)max_count * 4) == 0 && spgk_malloc(&b, (size_t)max_count * 4 + 16) == 0) {
        de->d_src = a; de->d_dst = b; de->ok = true;
    } else {
        spgk_free(a); spgk_free(b);
    }
}

static void dev_encoder_close(dev_encoder *de) { spgk_free(de->d_src); spgk_free(de->d_dst); de->ok = false; }

/* dsrc != NULL: the array currently lives on the device (a train() call is running and these are its buffers): it is
 * encoded there and only the file bytes come back; the host array `src` is stale then and not looked at. */
static bool write_array(FILE *f, const float *src, const float *dsrc, uint32_t count, PrecisionMode p, uint8_t *scratch, dev_encoder *de)
{
    size_t n = 0;
    if (dsrc) {
        if (p == PRECISION_FLOAT32) {
            n = (size_t)count * 4;
            if (spgk_memcpy_d2h(scratch, dsrc, n, NULL) || spgk_stream_sync(NULL)) return false;
        } else {
            if (!de || !de->d_dst) return false;
            n = spgk_encoded_bytes(count, (int)p);
            if (spgk_encode_array(dsrc, count, (int)p, de->d_dst, NULL) || spgk_memcpy_d2h(scratch, de->d_dst, n, NULL) ||
                spgk_stream_sync(NULL)) return false;
        }
        return fwrite(scratch, 1, n, f) == n;
    }
    if (de && de->ok && count >= SPG_DEV_ENCODE_MIN && p != PRECISION_FLOAT32) {
        n = spgk_encoded_bytes(count, (int)p);
        if (spgk_memcpy_h2d(de->d_src, src, (size_t)count * 4, NULL) || spgk_encode_array(de->d_src, count, (int)p, de->d_dst, NULL) ||
            spgk_memcpy_d2h(scratch, de->d_dst, n, NULL) || spgk_stream_sync(NULL)) {
            spg_log(LOG_DEBUG, "save: device encoder unavailable, using the host encoder");
            de->ok = false;
            n = 0;
        }
    }
    if (!n) n = spg_encode_array(src, count, p, scratch);
    return fwrite(scratch, 1, n, f) == n;
}

void save_spingalett_struct_arguments(SaveArgs a)
{
    if (!a.net || !a.filename) { spg_set_error(SPINGALETT_ERR_INVALID, "save: net or filename is NULL"); return; }
    if ((unsigned)a.precision >= PRECISION_COUNT) { spg_set_error(SPINGALETT_ERR_INVALID, "save: invalid precision mode"); return; }
    NeuralNetwork *n = a.net;
    if (n->layers < 1) { spg_set_error(SPINGALETT_ERR_INVALID, "save: network has no layers"); return; }

    /* ".nn" is appended when the last path component has no dot (Serialize.c:321-336) */
    const char *base = a.filename;
    for (const char *q = a.filename; *q; q++) if (*q == '/' || *q == '\\') base = q + 1;
    size_t len = strlen(a.filename);
    char *path = malloc(len + 4);
    if (!path) { spg_set_error(SPINGALETT_ERR_ALLOC, "save: filename allocation failed"); return; }
    memcpy(path, a.filename, len + 1);
    if (!strchr(base, '.')) memcpy(path + len, ".nn", 4);

    FILE *f = fopen(path, "wb");
    if (!f) { spg_set_error(SPINGALETT_ERR_INVALID, "save: cannot open file for writing"); free(path); return; }

    uint8_t head[32];
    size_t h = 0;
    uint16_t version = SPINGALETT_FORMAT_VERSION;
    uint8_t has_opt = a.do_not_save_optimizer ? 0 : 1;
    memcpy(head + h, &version, 2); h += 2;
    memcpy(head + h, &n->layers, 4); h += 4;
    head[h++] = (uint8_t)n->loss_func;
    head[h++] = has_opt;
    if (has_opt) { memcpy(head + h, &n->time_step, 8); h += 8; }
    head[h++] = (uint8_t)a.precision;
    bool ok = fwrite(head, 1, h, f) == h && fwrite(n->topology, 4, n->layers, f) == n->layers;
    for (uint32_t l = 0; l + 1 < n->layers && ok; l++) {
        uint8_t act = (uint8_t)n->act_func[l];
        ok = fwrite(&act, 1, 1, f) == 1;
    }
    if (!ok) {
        spg_set_error(SPINGALETT_ERR_INVALID, "save: failed to write header");
        spg_log(LOG_ERROR, "Failed to write file header to %s", path);
        fclose(f); free(path);
        return;
    }

    uint32_t maxc = 1;
    for (uint32_t l = 0; l + 1 < n->layers; l++) {
        uint32_t wc = n->topology[l] * n->topology[l + 1];
        if (wc > maxc) maxc = wc;
        if (n->topology[l + 1] > maxc) maxc = n->topology[l + 1];
    }
    uint8_t *scratch = malloc((size_t)maxc * 4 + 8);
    float *zeros = NULL;
    if (has_opt && !n->opt_m_weights) zeros = calloc(maxc, sizeof(float));   /* never trained: state is all zero */
    if (!scratch || (has_opt && !n->opt_m_weights && !zeros)) {
        spg_set_error(SPINGALETT_ERR_ALLOC, "save: write buffer allocation failed");
        free(scratch); free(zeros); fclose(f); free(path);
        return;
    }
    /* inside a train() call (autosave, or a save from the caller's callback) the parameters and moments are the flat
     * device buffers [weights | biases] of the trainer: encode straight from them */
    spg_net *pn = spg_priv(n);
    const float *lw = pn->live_params, *lm = pn->live_m, *lv = pn->live_v;
    const uint64_t tw = n->total_weights;
    dev_encoder de;
    dev_encoder_open(&de, a.precision != PRECISION_FLOAT32 ? maxc : 0);
    if (lw) {
        /* the kernels of the step in flight must have finished before their buffers are read on the legacy stream */
        if (spgk_set_device(pn->device) || spgk_stream_sync(pn->stream)) ok = false;
        if (ok && a.precision != PRECISION_FLOAT32 && !de.d_dst) {
            void *b = NULL;
            if (spgk_malloc(&b, (size_t)maxc * 4 + 16) == 0) de.d_dst = b; else ok = false;
        }
    }
    for (uint32_t l = 0; l + 1 < n->layers && ok; l++) {
        uint32_t wc = n->topology[l] * n->topology[l + 1], bc = n->topology[l + 1];
        uint64_t wo = n->weight_offsets[l], bo = n->bias_offsets[l];
        ok = write_array(f, n->weights + wo, lw ? lw + wo : NULL, wc, a.precision, scratch, &de);
        if (ok && has_opt)
            ok = write_array(f, zeros ? zeros : n->opt_m_weights + wo, lw ? lm + wo : NULL, wc, a.precision, scratch, &de) &&
                 write_array(f, zeros ? zeros : n->opt_v_weights + wo, lw ? lv + wo : NULL, wc, a.precision, scratch, &de);
        if (ok) ok = write_array(f, n->biases + bo, lw ? lw + tw + bo : NULL, bc, a.precision, scratch, &de);
        if (ok && has_opt)
            ok = write_array(f, zeros ? zeros : n->opt_m_biases + bo, lw ? lm + tw + bo : NULL, bc, a.precision, scratch, &de) &&
                 write_array(f, zeros ? zeros : n->opt_v_biases + bo, lw ? lv + tw + bo : NULL, bc, a.precision, scratch, &de);
    }
    dev_encoder_close(&de);
    free(scratch); free(zeros);
    if (fclose(f) != 0) ok = false;
    if (!ok) {
        spg_set_error(SPINGALETT_ERR_INVALID, "save: write error (disk full?)");
        spg_log(LOG_ERROR, "Write error saving to %s", path);
    } else {
        spg_log(LOG_INFO, "Network saved to %s", path);
        spg_log(LOG_INFO, "Save info: format=v%u, layers=%u, weights=%llu, biases=%llu, precision=%s, optimizer=%s",
                (unsigned)version, n->layers, (unsigned long long)n->total_weights, (unsigned long long)n->total_biases,
                spg_precision_name(a.precision), has_opt ? "ON" : "OFF");
    }
    free(path);
}
