/*
 * spg_internal.h -- private declarations of the C23 host library.
 *
 * A NeuralNetwork handed to callers is the first member of a larger private
 * record (spg_net) that carries the packed weight payloads, the device
 * buffers and the workspaces.  The library allocates and frees that record
 * (as the reference does with its own struct, Network.c:41 and :299), so the
 * extra fields are invisible to programs compiled against the public header.
 */
#pragma once

#include "spingalett_b200.h"
#include "spingalett_b200_kernels.h"
#include <stdint.h>
#include <stdbool.h>
#define SPG_PIPE_MAX 16        /* most chunks a host-input batch is cut into */
#include <stddef.h>

#define SPG_ERRMSG_MAX 256
#define SPG_NET_MAGIC 0x4E475053u /* "SPGN" */
#define SPG_HIDDEN __attribute__((visibility("hidden")))

typedef struct spg_net_s {
    NeuralNetwork pub;          /* MUST stay first: &net->pub == (NeuralNetwork *)net */
    uint32_t magic;

    /* Weights as stored.  For a net read from a .nn file these are the packed
     * arrays of the file (without the abs-max prefix, which is kept in
     * amax_*); for a net built with layer() they are NULL and the device gets
     * an fp32 image of pub.weights. */
    PrecisionMode store_precision;
    uint8_t **payload_w;        /* [layers-1] host copies of the packed matrices */
    size_t   *payload_w_bytes;
    float    *amax_w;           /* [layers-1] abs-max of integer formats */
    uint32_t  payload_layers;   /* length of the three arrays above */

    /* device side (all NULL until the first compute call) */
    bool   dev_ready;
    int    device;
    void  *stream;
    uint32_t dev_layers;
    void **d_w;                 /* [layers-1] */
    float **d_bias;             /* [layers-1] */
    spgk_layer *klayers;        /* [layers-1] descriptors with device pointers */

    /* small-batch workspace: fp32 activations of every layer for up to
     * small_cap rows, laid out layer after layer ([rows][width] each) */
    float *d_small; uint32_t small_cap;
    void *d_gemv_scratch; size_t gemv_scratch_bytes; bool gemv_pending;
    void *d_staged[2]; size_t staged_bytes[2];   /* ping-pong staged inputs of the GEMV chain */
    void *d_operand[2]; size_t operand_bytes[2]; /* ping-pong activation operands of the weight-streaming chain */
    void *d_ws_scratch; size_t ws_scratch_bytes; bool ws_pending;
    /* AUTO math mode: rows recomputed exactly after the one-term pass */
    uint32_t *d_rep_idx; size_t rep_idx_bytes; float *d_rep_in; size_t rep_in_bytes; float *d_rep_out; size_t rep_out_bytes;
    uint32_t last_repaired; bool auto_calibrated; float auto_theta;
    uint8_t bf16_fits_f16;                /* BF16 file: 0 not looked at yet, 1 every weight is within fp16's range, 2 not */
    uint32_t auto_calls;                  /* large AUTO calls since the calibration: every SPG_AUTO_RECAL-th one measures again */
    uint32_t *h_count; bool count_pending, count_seen;      /* pinned: [slot] repaired-row counts of the last AUTO call (one slot per pipelined chunk) */
    uint32_t count_slot, count_slots_used;
    void *copy_stream; void *copy_ev[SPG_PIPE_MAX + 1];      /* host-input pipeline: copies run ahead of compute */
    float *h_chunk[2]; size_t h_chunk_bytes;                /* page-locked staging for pageable inputs: two chunks */

    /* large-batch workspace */
    float *d_in32;  size_t in32_bytes;      /* staging for host inputs */
    float *d_out32; size_t out32_bytes;     /* fp32 outputs of the last layer */
    void  *d_act16[2]; size_t act16_bytes;  /* ping-pong 16-bit activation planes */
    float *d_act32[2]; size_t act32_bytes;  /* ping-pong fp32 activations (SIMT chain) */
    int32_t *d_status; bool status_pending;
    void *d_w16; size_t w16_bytes;         /* 16-bit weight operand of the layer in flight */
    /* 16-bit weight operands kept between calls (nets whose expanded weights are small): [fp16 | bf16][layer] */
    void **d_w16c[2]; uint8_t *w16c_parts[2];
    float *d_head_w;                       /* fp32 weights of a narrow last layer fused into the layer before it */
    float *d_fused_params;                 /* padded biases + head weights of the one-launch three-layer kernel */
    bool fused_ran;                        /* the one-launch kernel has served this net at least once */

    float *h_out; size_t h_out_bytes;       /* library-owned pinned output buffer */
    float *h_stage; size_t h_stage_bytes;   /* pinned staging for forward() */

    /* optional kernel timing (spingalett_profile): event pairs around the layer kernels */
    bool prof_on; void **prof_ev; uint32_t prof_cap, prof_used;
    double prof_ms; uint64_t prof_launches;

    /* replicas of the device image on other GPUs (spingalett_set_devices): records that share this net's host arrays and
     * packed payload and own only their device side; slot g serves share g of a batch */
    struct spg_net_s *shadow[16];
    bool is_shadow;

    /* training state on the device (created by the first train() call, kept between calls) */
    void *train;
    /* while a train() call runs: the flat device buffers [weights | biases] that hold the current parameters and
     * optimiser moments; save_spingalett encodes from them instead of the (stale) host arrays */
    const float *live_params, *live_m, *live_v;
} spg_net;

static inline spg_net *spg_priv(NeuralNetwork *n) { return (spg_net *)(void *)n; }

/* error.c */
SPG_HIDDEN void spg_set_error(int code, const char *msg);
SPG_HIDDEN void spg_set_errorf(int code, const char *fmt, ...);
/* settings.c */
SPG_HIDDEN void spg_log(LogLevel level, const char *fmt, ...);
SPG_HIDDEN const char *spg_act_name(unsigned a);
SPG_HIDDEN const char *spg_precision_name(unsigned p);
SPG_HIDDEN const char *spg_loss_name(unsigned l);
SPG_HIDDEN void spg_note_path(const char *name);
/* rng.c */
SPG_HIDDEN float spg_rand_uniform_pm1(void);
SPG_HIDDEN float spg_rand_normal(void);
SPG_HIDDEN uint32_t spg_rand_u32(void);
SPG_HIDDEN void spg_shuffle(uint32_t *idx, uint32_t n);
/* codec.c */
SPG_HIDDEN size_t spg_array_bytes(uint64_t count, PrecisionMode p);
SPG_HIDDEN void spg_decode_array(const uint8_t *src, uint64_t count, PrecisionMode p, float *dst);
SPG_HIDDEN size_t spg_encode_array(const float *src, uint64_t count, PrecisionMode p, uint8_t *dst);
SPG_HIDDEN float spg_precision_q(PrecisionMode p);
/* network.c */
SPG_HIDDEN int spg_net_ensure_train_arrays(spg_net *n);
SPG_HIDDEN void spg_net_drop_payload(spg_net *n);
/* device.c */
SPG_HIDDEN int spg_dev_ensure(spg_net *n);           /* upload if needed */
SPG_HIDDEN void spg_dev_release(spg_net *n);
SPG_HIDDEN void spg_dev_invalidate(spg_net *n);
SPG_HIDDEN int spg_dev_forward_small(spg_net *n, const float *d_x, uint32_t ldx, uint32_t N, float **d_last, float *d_final);
SPG_HIDDEN int spg_dev_forward_large(spg_net *n, const float *d_x, uint32_t N, float *d_out);
SPG_HIDDEN int spg_map_kernel_error(int rc, const char *where);
/* train.c */
SPG_HIDDEN void spg_train_release(spg_net *n);
SPG_HIDDEN void spg_autosave(spg_net *n, const TrainArgs *a, size_t epoch);
