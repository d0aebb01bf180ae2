/*
 * spingalett_b200_kernels.h -- the thin C shim between the C23 host library
 * and the hand-written sm_100a kernels.
 *
 * Everything here is `extern "C"`, takes plain pointers and sizes, and runs on
 * the CUDA device that is current on the calling thread.  Device pointers are
 * marked "dev".  Every function returns 0 on success or a negative SPGK_E_*
 * code; spgk_error_string() describes the last failure on the calling thread.
 * None of these functions has a CPU implementation: with no CUDA device they
 * fail.
 *
 * Each compute entry point names the reference routine (pka-human/Spingalett,
 * path:line) whose work it does on the GPU.
 */
#pragma once

#include <stdint.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#ifndef SPGK_API
#  define SPGK_API __attribute__((visibility("default")))
#endif

#define SPGK_OK            0
#define SPGK_E_CUDA       -1   /* a CUDA runtime/driver call failed            */
#define SPGK_E_ARG        -2   /* argument outside what the kernel supports   */
#define SPGK_E_NOMEM      -3   /* device or pinned-host allocation failed     */
#define SPGK_E_TIMEOUT    -4   /* a bounded device-side wait gave up          */
#define SPGK_E_UNSUPPORTED -5  /* shape/format not handled by this fast path  */

/* One dense layer as the kernels see it.  `w` is the weight matrix exactly as
 * Serialize.c stores it (row-major [out][in], packing running across rows),
 * WITHOUT the leading abs-max float of the integer formats; that scalar
 * arrives pre-divided in w_scale (abs_max/127, /7, /1; 1.0 for float
 * formats), so value = q * w_scale (reference Serialize.c:222-294). */
typedef struct {
    const void  *w;          /* dev, 256-byte aligned                        */
    const float *bias;       /* dev, fp32 [out], already dequantised          */
    float        w_scale;
    uint32_t     in;
    uint32_t     out;
    int32_t      precision;  /* PrecisionMode: 0 f32, 1 f16, 2 bf16, 3 i8, 4 i4, 5 i2 */
    int32_t      act;        /* ActivationFunction                            */
    float        bias_absmax;/* an upper bound of |bias[j]|.  Only the chained integer GEMV reads it
                              * (for the range of the values it hands to the next layer); a bound
                              * below a real bias makes that call fail with SPGK_E_ARG.            */
} spgk_layer;

/* 16-bit operand flavour used on the tensor-core paths. */
#define SPGK_T_F16   0
#define SPGK_T_BF16  1

SPGK_API const char *spgk_error_string(void);

/* ---- device plumbing ---------------------------------------------------- */
SPGK_API int spgk_device_count(int *count);
SPGK_API int spgk_set_device(int device);
SPGK_API int spgk_get_device(int *device);
/* compute capability major*10+minor and SM count of the current device */
SPGK_API int spgk_device_info(int *cc, int *sm_count, size_t *total_mem);
SPGK_API int spgk_malloc(void **dev, size_t bytes);
SPGK_API int spgk_free(void *dev);
SPGK_API int spgk_host_alloc(void **host, size_t bytes);     /* pinned */
SPGK_API int spgk_host_free(void *host);
SPGK_API int spgk_memcpy_h2d(void *dev, const void *host, size_t bytes, void *stream);
SPGK_API int spgk_memcpy_d2h(void *host, const void *dev, size_t bytes, void *stream);
SPGK_API int spgk_memcpy_d2d(void *dst, const void *src, size_t bytes, void *stream);
SPGK_API int spgk_memset(void *dev, int value, size_t bytes, void *stream);
SPGK_API int spgk_stream_sync(void *stream);
/* 1 if ptr is device (or managed) memory, 0 if host, <0 on error */
SPGK_API int spgk_is_device_pointer(const void *ptr);
SPGK_API int spgk_is_pinned_host_pointer(const void *ptr);   /* 1: page-locked host memory, 0: pageable or unknown */
/* number of kernel launches made through this shim by the calling process */
SPGK_API uint64_t spgk_launch_count(void);

/* CUDA events for timing on the launching stream */
SPGK_API int spgk_event_create(void **event);
SPGK_API int spgk_event_destroy(void *event);
SPGK_API int spgk_event_record(void *event, void *stream);
SPGK_API int spgk_event_sync(void *event);                    /* the host waits for the event */
SPGK_API int spgk_event_elapsed_ms(void *start, void *stop, float *ms);
/* a second (non-blocking) stream and cross-stream ordering, for copies that overlap compute */
SPGK_API int spgk_stream_create(void **stream);
SPGK_API int spgk_stream_destroy(void *stream);
SPGK_API int spgk_stream_wait_event(void *stream, void *event);

/* ---- K0: general layer, fp32 SIMT ---------------------------------------
 * y[n][j] = act(bias[j] + w_scale * sum_k q[j][k] * x[n][k]) for any
 * precision and any shape (odd widths, packed rows starting mid-byte).
 * x: dev fp32 [N][in] (row stride ldx floats), y: dev fp32 [N][out] (ldy).
 * ACT_SOFTMAX is NOT applied here (use spgk_softmax_rows afterwards).
 * Does the work of forward()'s layer step, reference Network.c:218-247. */
SPGK_API int spgk_layer_simt(const spgk_layer *L, const float *x, uint32_t ldx,
                             float *y, uint32_t ldy, uint32_t N, void *stream);

/* ---- softmax over rows, in place ----------------------------------------
 * Reference Activation.c:5-21 per row: max from -FLT_MAX, expf(x-max), scale
 * by 1/sum only if sum > 0.  width <= 65535. */
SPGK_API int spgk_softmax_rows(float *y, uint32_t ldy, uint32_t N, uint32_t width, void *stream);

/* ---- margin check of the one-term mode ---------------------------------------
 * spgk_margin_select appends to idx (and counts in *count, which the caller zeroes)
 * every row of probs [N][width] whose two largest entries are within `theta` in log
 * space; spgk_scatter_rows writes recomputed rows back: dst[idx[i]] = src[i].
 * (No reference counterpart: they let the fast one-term tensor-core pass be followed
 * by an exact recomputation of just the rows whose argmax it could have changed.) */
/* Row counts that exist only on the device.  After spgk_set_dynamic_rows(ptr, expected) the row-wise calls made by
 * this thread -- spgk_split16, spgk_gather_rows, spgk_scatter_rows, spgk_softmax_rows, spgk_layer_gemm_tc --
 * treat their row argument as a capacity and work on min(rows, *ptr) rows, *ptr being read by the kernels
 * when they run, so a selection made on the device (spgk_margin_select) can be followed up without a host
 * round trip.  `expected` is the caller's guess of the count (0 = none); it only steers tile shapes.  NULL
 * switches it off.  (No reference counterpart.) */
SPGK_API void spgk_set_dynamic_rows(const uint32_t *rows_dev, uint32_t expected);
/* After spgk_set_margin_sink(theta, idx, count) the next spgk_layer_gemm_tc calls of this thread that finish a
 * softmax row in their epilogue (softmax_fused = 1) do the work of spgk_margin_select on the way: rows whose two
 * largest logits are within theta are appended to idx and counted in *count (which the caller zeroes).
 * idx == NULL switches it off. */
SPGK_API void spgk_set_margin_sink(float theta, uint32_t *idx, uint32_t *count);
/* After spgk_set_output_rows(idx) the fp32 output of this thread's spgk_layer_gemm_tc calls is scattered: row r of the
 * result is written to row idx[r] of out32 (the counterpart of spgk_split16_rows).  NULL switches it off. */
SPGK_API void spgk_set_output_rows(const uint32_t *rows_idx);
SPGK_API int spgk_margin_select(const float *probs, uint32_t ldp, uint32_t N, uint32_t width, float theta,
                                uint32_t *idx, uint32_t *count, void *stream);
/* max over rows of the change in the top-two log gap between a fast and an exact result (float bits in *max_bits,
 * which the caller zeroes): the calibration measurement behind the margin. */
SPGK_API int spgk_gap_error(const float *fast, const float *exact, uint32_t ld, uint32_t N, uint32_t width,
                            uint32_t *max_bits, void *stream);
SPGK_API int spgk_scatter_rows(const float *src, const uint32_t *idx, float *dst, uint32_t rows, uint32_t width,
                               uint32_t ldd, void *stream);

/* ---- split fp32 activations into 16-bit terms ----------------------------
 * dst holds `parts` planes of [N][ld16] 16-bit values (plane stride
 * plane_elems): plane 0 = round(x), plane 1 = round(x - plane0), ...
 * Columns in..ld16 are zero-filled.  type = SPGK_T_F16 / SPGK_T_BF16. */
SPGK_API int spgk_split16(const float *x, uint32_t ldx, uint32_t N, uint32_t in,
                          void *dst, uint32_t ld16, uint64_t plane_elems,
                          int parts, int type, void *stream);
/* the same with a gather in front: plane row n is built from x row rows_idx[n] (device array) */
SPGK_API int spgk_split16_rows(const float *x, uint32_t ldx, const uint32_t *rows_idx, uint32_t N, uint32_t in,
                          void *dst, uint32_t ld16, uint64_t plane_elems,
                          int parts, int type, void *stream);

/* ---- array encoders of the .nn format on the device -------------------------
 * dst receives exactly the bytes write_array_compressed (Serialize.c:87-193) writes for src[0..count): fp32 copy,
 * truncated fp16 / bf16 words, or [abs-max float][packed INT8 / INT4 / INT2].  dst: dev, spgk_encoded_bytes(count,
 * precision) bytes, 4-byte aligned for the integer formats.  Stream-ordered, no host synchronisation. */
SPGK_API size_t spgk_encoded_bytes(uint64_t count, int precision);
SPGK_API int spgk_encode_array(const float *src, uint64_t count, int precision, uint8_t *dst, void *stream);

/* ---- K1: small-batch fused dequant-GEMV ----------------------------------
 * Whole layer for 1 <= N <= SPGK_GEMV_MAX_BATCH rows: streams the packed
 * weights once (TMA boxes into a shared-memory ring), unpacks them in registers
 * and multiplies on the warp-level tensor path -- integer files against base-128
 * digits of a fixed-point x with exact s32 accumulation, float files against a
 * two/three-term bf16 split of x with fp32 accumulation -- then applies bias and
 * activation; a softmax layer is completed by the CTA that finishes last when N == 1
 * (spgk_gemv_applies_softmax(N) == 1) and left as logits for spgk_softmax_rows otherwise.
 * Memory-bound by design.
 * Needs 16-byte aligned packed rows of at least 64 bytes (TMA boxes of the packed
 * matrix); returns SPGK_E_UNSUPPORTED otherwise so the caller can use spgk_layer_simt.
 * scratch: dev, at least spgk_gemv_scratch_bytes(L, N) bytes, ZERO-FILLED before
 * its first use (it starts with the status word a bounded wait that gave up is
 * reported in; read it with spgk_gemv_status).  Calls sharing a scratch buffer must not overlap.
 * Does forward()'s layer step, reference Network.c:218-247 / SIMD.c:190-240. */
#define SPGK_GEMV_MAX_BATCH 8
SPGK_API size_t spgk_gemv_scratch_bytes(const spgk_layer *L, uint32_t N);
SPGK_API int spgk_gemv_applies_softmax(uint32_t N);
SPGK_API int spgk_layer_gemv(const spgk_layer *L, const float *x, uint32_t ldx,
                             float *y, uint32_t ldy, uint32_t N,
                             void *scratch, void *stream);
/* Chained form for a run of layers.  The kernel consumes its input as bf16 terms
 * laid out in the order its weight loads need them ("staged" input).
 * staged_in : this layer's staged input, produced by the previous call; NULL makes
 *             the call stage x itself (one small extra kernel).
 * staged_out: if `next` is given, also eligible for this kernel and L is not a
 *             softmax layer (spgk_gemv_chain_stages_next() == 1), the CTAs that
 *             finish the layer write next's staged input here, so the following
 *             call needs no staging kernel.  spgk_gemv_staged_bytes(width, N) bytes
 *             for a layer whose `in` is `width`.
 * y (fp32) is always written as well. */
SPGK_API size_t spgk_gemv_staged_bytes(uint32_t width, uint32_t N);
/* The whole run of layers of a small-batch forward in ONE launch (the CTAs stay on their SMs, weights of the next layer
 * stream in while a layer finishes, a device-wide counter orders only the staged inputs).  Returns SPGK_E_UNSUPPORTED
 * unless every layer is eligible with the same stored precision and chunk geometry and only the last is a softmax
 * layer: then call spgk_layer_gemv_chain layer by layer.  ys[l]: fp32 output of layer l, [N][out_l]. */
SPGK_API int spgk_gemv_forward_chain(const spgk_layer *layers, uint32_t n, const float *x, uint32_t ldx, float *const *ys, uint32_t N,
                                     void *staged_a, void *staged_b, void *scratch, void *stream);
/* status word at the start of scratch: SPGK_E_TIMEOUT if a bounded wait inside the kernel gave up (synchronises) */
SPGK_API int spgk_gemv_status(void *scratch, void *stream);
SPGK_API int spgk_gemv_chain_stages_next(const spgk_layer *L, const spgk_layer *next, uint32_t N);
/* INT8 / INT4 / INT2 layers normally run through the integer tensor path (activations as four base-128
 * digits of a 28-bit fixed-point number, exact integer accumulation); 0 switches them to the bf16
 * hi/lo-term path that the floating-point formats use.  Process-wide; meant for tests and comparisons. */
SPGK_API void spgk_gemv_set_int_path(int on);
SPGK_API int spgk_gemv_get_int_path(void);
SPGK_API int spgk_layer_gemv_chain(const spgk_layer *L, const spgk_layer *next, const void *staged_in, void *staged_out,
                                   const float *x, uint32_t ldx, float *y, uint32_t ldy, uint32_t N,
                                   void *scratch, void *stream);

/* ---- K3: weight-streaming tensor-core layer, 1..128 rows --------------------
 * The memory-bound regime on tcgen05: the 128 rows of the MMA tile are weight
 * rows, its columns are the batch (each row as two or three bf16 terms, so all
 * products are exact), the packed INT4 / INT2 / INT8 weights arrive by TMA and
 * are dequantised in shared memory by converter warps into the K-major operand
 * tile (BF16 weights are used in place), the accumulator lives in tensor memory.
 * Needs 16-byte aligned packed rows and N*terms <= 256 columns; FP16/FP32 files
 * and other shapes return SPGK_E_UNSUPPORTED (use spgk_layer_gemv / _simt).
 * operand_in : this layer's activation operand as written by the previous call
 *              (bf16 terms, K order permuted to match the unpacking); NULL makes
 *              the call build it from x (one small extra kernel).
 * operand_out: if spgk_wstream_stages_next(L, next, N) == 1 the epilogue writes
 *              next's operand there (spgk_wstream_operand_bytes(next->in, N) bytes).
 * scratch    : spgk_wstream_scratch_bytes(L, N) bytes, ZERO-FILLED before first use
 *              (status word + ticket counters; both are left at zero).
 * y (fp32 [N][ldy]) is always written; ACT_SOFTMAX is left to spgk_softmax_rows.
 * Does forward()/batch_forward()'s layer step, reference Network.c:218-247,
 * Training.c:327-343, with the decode of Serialize.c:222-294 fused in. */
SPGK_API size_t spgk_wstream_scratch_bytes(const spgk_layer *L, uint32_t N);
SPGK_API size_t spgk_wstream_operand_bytes(uint32_t width, uint32_t N);
SPGK_API int spgk_wstream_stages_next(const spgk_layer *L, const spgk_layer *next, uint32_t N);
SPGK_API int spgk_layer_wstream(const spgk_layer *L, const spgk_layer *next, const void *operand_in, void *operand_out,
                                const float *x, uint32_t ldx, float *y, uint32_t ldy, uint32_t N,
                                void *scratch, void *stream);
SPGK_API int spgk_wstream_status(void *scratch, void *stream);

/* ---- K2: large-batch tcgen05 GEMM layer ----------------------------------
 * C[N][out] = act(bias + w_scale * A[N][in] * W^T) with the accumulator in
 * tensor memory; both operands reach shared memory by TMA (no multicast).
 *
 * A is the 16-bit split produced by spgk_split16 or by the previous layer's
 * epilogue (`a_parts` planes, row stride lda elements, plane stride a_plane).
 * W is a 16-bit K-major operand [out][ldw] in `w_parts` planes: for FP16/BF16
 * files with 16-byte aligned rows it is the stored payload itself
 * (spgk_weights16_direct() == 1, ldw = in); every other precision or shape is
 * first expanded by spgk_dequant16 into scratch of spgk_weights16_bytes()
 * bytes (integers are exact in one plane; the per-array scale is applied in
 * the epilogue).  Passes run hi*hi, then lo*hi and hi*lo when a second plane
 * exists, all into the same fp32 accumulator.  The two operands may use
 * different 16-bit flavours (w_type16 for W, type16 for A and the output).
 *
 * Output: if out16 != NULL, `out_parts` 16-bit planes for the next layer (row
 * stride ldo16, a multiple of 8; plane stride o_plane); if out32 != NULL, fp32
 * [N][ldo32].  softmax_fused != 0 applies the row softmax in the epilogue
 * (needs out <= spgk_gemm_tc_softmax_max() and out32); otherwise a softmax
 * layer needs spgk_softmax_rows afterwards.
 * status: dev int32 the kernel reports a bounded wait that gave up in; read it
 * with spgk_gemm_tc_status() (which synchronises the stream).
 * Does batch_forward()'s layer step, reference Training.c:318-343. */
SPGK_API int spgk_gemm_tc_supported(const spgk_layer *L);
SPGK_API uint32_t spgk_gemm_tc_softmax_max(void);
/* whether spgk_layer_gemm_tc finishes a softmax layer of `width` columns in its own epilogue for `rows` rows: rows that fit one
 * tile (256 columns) always; up to 1024 columns when the batch has at least 64 row tiles and its row count is known on the
 * host (the CTA then owns whole row tiles: logits written, then normalised row by row; Activation.c:5-21) */
SPGK_API int spgk_gemm_tc_softmax_fusable(uint32_t width, uint32_t rows, int dynamic_rows);
SPGK_API int spgk_weights16_direct(const spgk_layer *L, int type16);
SPGK_API size_t spgk_weights16_bytes(const spgk_layer *L, int parts);
SPGK_API int spgk_dequant16(const spgk_layer *L, void *dst, uint32_t ldw, uint64_t plane, int parts,
                            int type16, void *stream);
SPGK_API int spgk_layer_gemm_tc(const spgk_layer *L,
                                const void *w16, uint32_t ldw, uint64_t w_plane, int w_parts, int w_type16,
                                const void *a16, uint32_t lda, uint64_t a_plane, int a_parts, int type16,
                                void *out16, uint32_t ldo16, uint64_t o_plane, int out_parts,
                                float *out32, uint32_t ldo32,
                                uint32_t N, int softmax_fused, int32_t *status, void *stream);
/* The same layer with the network's narrow last layer ("head", at most 16 outputs) finished in its epilogue:
 * each epilogue thread keeps the head's dot products of its row in registers (fp32 FMAs against head weights
 * staged in shared memory) while it walks the row's column tiles, so the wide activation matrix is never
 * written and the head needs no kernel of its own.  out32 [N][head->out] receives head_act(bias_h + scale_h *
 * Wh * act(...)), a softmax head included (and the margin sink, if set, is served).  head_w comes from
 * spgk_head_weights (spgk_head_weights_bytes bytes; it depends only on the head's weights and can be kept).
 * Replaces the last two iterations of the layer loop of batch_forward (Training.c:327-343). */
SPGK_API int spgk_gemm_tc_head_supported(const spgk_layer *L, const spgk_layer *head);
SPGK_API size_t spgk_head_weights_bytes(const spgk_layer *head);
SPGK_API int spgk_head_weights(const spgk_layer *head, float *dst, void *stream);
SPGK_API int spgk_layer_gemm_tc_head(const spgk_layer *L,
                                     const void *w16, uint32_t ldw, uint64_t w_plane, int w_parts, int w_type16,
                                     const void *a16, uint32_t lda, uint64_t a_plane, int a_parts, int type16,
                                     const spgk_layer *head, const float *head_w, float *out32, uint32_t ldo32,
                                     uint32_t N, int32_t *status, void *stream);
SPGK_API int spgk_gemm_tc_status(int32_t *status, void *stream);

/* ---- K2f: a three-layer MLP in one launch (large batches) ----------------------
 * out[N][L3->out] = head(act2(L2(act1(L1(x))))) for a net of exactly three weight layers whose last
 * layer ("head") has at most 16 outputs -- the whole layer loop of batch_forward (reference
 * Training.c:313-345) in ONE persistent tcgen05 kernel: the fp32 input rows are rounded to the 16-bit
 * operand type inside the kernel, the first hidden matrix lives only in shared memory (as the A
 * operand of layer 2), the second only in registers (rounded to 16 bits and multiplied into the head's sums
 * by warp-level MMAs whose A fragments come straight from tensor memory),
 * and bias / activation / row softmax (Activation.c:5-38) are applied on the way.  No activation
 * matrix is written to or read from HBM.
 *   w1_16 / w2_16: the 16-bit K-major weight operands of layers 1 and 2 ([out][ldw], flavour type16):
 *     the stored payload itself for FP16/BF16 files (spgk_weights16_direct), else spgk_dequant16 output.
 *   params: spgk_mlp3_params_bytes() bytes filled once per net and 16-bit flavour by spgk_mlp3_params
 *     (padded biases, and the head's weights as a 16-bit operand: exact for INT8/INT4/INT2/FP16/BF16 files).
 *   x: dev fp32 rows, 16-byte aligned, ldx a multiple of 4.  rows_idx (optional, dev): logical row r
 *     reads input row rows_idx[r] and writes output row rows_idx[r].  rows_limit (optional, dev): the
 *     kernel works on min(N, *rows_limit) rows, read when it runs; rows_expected is the caller's
 *     guess of that count (0 = none) and only sizes the grid.
 *   pairs != 0: every row is computed from a two-term split (16-bit rounding + scaled remainder) of the
 *     input and of the hidden activations, carried as two adjacent rows of the same one-term tensor
 *     pass and recombined in the epilogue: exact products for INT8/INT4/INT2/FP16/BF16 files at twice
 *     the tensor work per row.
 *   margin_idx / margin_count (optional, dev; pairs == 0, softmax head): rows whose two largest logits
 *     are within theta are appended to margin_idx and counted in *margin_count (the caller zeroes it).
 *   status: dev int32, as for spgk_layer_gemm_tc (read with spgk_gemm_tc_status).
 * spgk_mlp3_supported() == 0 (other depths, hidden width above 512, head wider than 16, unaligned
 * input rows) means: run the layers one by one with spgk_layer_gemm_tc. */
SPGK_API int spgk_mlp3_supported(const spgk_layer *L1, const spgk_layer *L2, const spgk_layer *L3, uint32_t ldx);
SPGK_API size_t spgk_mlp3_params_bytes(const spgk_layer *L1, const spgk_layer *L2, const spgk_layer *L3);
SPGK_API int spgk_mlp3_params(const spgk_layer *L1, const spgk_layer *L2, const spgk_layer *L3, int type16, float *dst, void *stream);
SPGK_API int spgk_mlp3_forward(const spgk_layer *L1, const void *w1_16, uint32_t ldw1,
                               const spgk_layer *L2, const void *w2_16, uint32_t ldw2,
                               const spgk_layer *L3, const float *params, int type16,
                               const float *x, uint32_t ldx, const uint32_t *rows_idx, const uint32_t *rows_limit,
                               uint32_t rows_expected, int pairs, float *out, uint32_t ldo, uint32_t N,
                               float theta, uint32_t *margin_idx, uint32_t *margin_count,
                               int32_t *status, void *stream);

/* Profiling hook of the one-launch MLP (no reference counterpart): after spgk_mlp3_set_trace(buf) the
 * spgk_mlp3_forward calls of this thread make CTA 0 write cycle counters of its four roles into buf (dev, 32
 * uint64: [0..4] MMA issuer total / waits for accumulator, input tile, hidden tile, weight tile; [8..12] one
 * epilogue warp total / wait for accumulator / layer-1 work / layer-2 work / exchange wait; [16..18] one
 * converter warp total / wait for a free slot / work; [24..25] weight producer total / wait for a free slot).
 * NULL switches it off. */
SPGK_API void spgk_mlp3_set_trace(unsigned long long *trace32);

/* ---- training step (fp32, as the reference) -------------------------------
 * spgk_train_gemm modes:
 *   0  C[M][N] = act(A[M][K] B[N][K]^T + bias[N])      forward, batch_forward (Training.c:327-343);
 *                                                        ACT_SOFTMAX is left to spgk_softmax_rows
 *   1  C[M][N] = (A[M][K] B[K][N]) * act'(aux[M][N])   delta back-propagation (Training.c:383-392);
 *                                                        the derivative takes the activation OUTPUT
 *   2  C[M][N] = alpha * A[K][M]^T B[K][N]             weight gradient (Training.c:405-411)
 * spgk_ce_delta: delta = a - t (cross-entropy over softmax or sigmoid, Training.c:366-371); if
 *   loss != NULL the batch's summed cross-entropy (SIMD.c:533-549) is added to *loss.
 * spgk_col_sums: out[j] = scale * sum_rows d[row][j]   bias gradient (Training.c:413-417).
 * spgk_train_grad: both gradients of one layer in one launch (Training.c:405-417):
 *   gw[out][in] = scale * delta[rows][out]^T a[rows][in],  gb[out] = scale * sum_rows delta[row][out].
 * spgk_gather_rows: dst[i] = src[idx[i]]                mini-batch assembly (Training.c:759-767).
 * spgk_gather_rows2: the same rows of two tables (inputs and targets) in one launch.
 * spgk_train_output: the output end of a step in one launch, for an output layer of at most 16 units:
 *   y = softmax (or sigmoid) of x w^T + bias, delta = y - t, *loss += cross-entropy of the rows (loss may be NULL);
 *   replaces mode 0 + spgk_softmax_rows + spgk_ce_delta (Training.c:327-343, :366-371).
 * spgk_adam: one fused pass over a flat parameter buffer; g is scaled by gscale first
 *   (1/ranks after a sum all-reduce); epsilon inside the square root (SIMD.c:279-328).
 * spgk_nonfinite: sets *flag_dev to 1 if any element is NaN/Inf (Training.c:11-19). */
SPGK_API int spgk_train_gemm(int mode, const float *A, uint32_t lda, const float *B, uint32_t ldb,
                             float *C, uint32_t ldc, uint32_t M, uint32_t N, uint32_t K, float alpha,
                             const float *bias, const float *aux, uint32_t ldaux, int act, void *stream);
SPGK_API int spgk_ce_delta(const float *a, const float *t, float *delta, uint64_t count, float *loss,
                           int sigmoid_output, void *stream);
SPGK_API int spgk_col_sums(const float *d, uint32_t rows, uint32_t cols, float scale, float *out, void *stream);
SPGK_API int spgk_train_grad(const float *delta, uint32_t ldd, const float *a, uint32_t lda, float *gw, uint32_t ldg,
                             float *gb, uint32_t out, uint32_t in, uint32_t rows, float scale, void *stream);
SPGK_API int spgk_gather_rows(const float *src, const uint32_t *idx, float *dst, uint32_t rows, uint32_t width,
                              void *stream);
SPGK_API int spgk_gather_rows2(const float *src_a, uint32_t width_a, float *dst_a, const float *src_b, uint32_t width_b,
                               float *dst_b, const uint32_t *idx, uint32_t rows, void *stream);
SPGK_API int spgk_train_output(const float *x, uint32_t ldx, const float *w, uint32_t ldw, const float *bias, float *y,
                               const float *t, float *delta, float *loss, uint32_t rows, uint32_t out, uint32_t in,
                               int sigmoid_output, void *stream);
SPGK_API int spgk_adam(float *w, float *m, float *v, const float *g, uint64_t n, float lr, float b1, float b2,
                       float mf, float vf, float eps, float gscale, void *stream);
SPGK_API int spgk_nonfinite(const float *w, uint64_t n, int *flag_dev, void *stream);
/* spgk_output_delta: the output deltas the direct cross-entropy form does not cover (Training.c:357-376): mse_softmax != 0
 *   gives delta_j = a_j*((a_j - t_j) - sum_k (a_k - t_k) a_k), otherwise delta_j = (a_j - t_j) * act'(a_j); if loss != NULL the
 *   batch's summed loss is added to *loss: squared error (loss_ce == 0, SIMD.c:527-531) or -sum t*log(max(a, 1e-9))
 *   (loss_ce != 0, SIMD.c:543-548).
 * spgk_sumsq: *out_dev += sum g[i]^2 (global gradient norm, SIMD.c:496-507).
 * spgk_optimizer_step: one fused pass of SGD (0), MOMENTUM (1), RMSPROP (2), ADAM (3) or ADAMW (4) over the flat buffer
 *   [weights | biases] exactly as apply_gradients_batch_prescaled does it layer by layer (Training.c:439-507, SIMD.c:279-494):
 *   weight decay acts on the first n_weights elements only (L2 term for SGD / MOMENTUM / RMSPROP / ADAM, decoupled for
 *   ADAMW); g is scaled by gscale and, if sumsq_dev != NULL, clipped to max_norm by the global norm sqrt(*sumsq_dev)*gscale
 *   (SIMD.c:509-518). */
SPGK_API int spgk_output_delta(const float *a, const float *t, float *delta, uint32_t rows, uint32_t width, int act, int mse_softmax,
                               int loss_ce, float *loss, void *stream);
SPGK_API int spgk_sumsq(const float *g, uint64_t n, float *out_dev, void *stream);
SPGK_API int spgk_optimizer_step(int kind, float *w, float *m, float *v, const float *g, uint64_t n, uint64_t n_weights,
                                 float lr, float momentum, float b1, float b2, float mf, float vf, float eps, float decay,
                                 float gscale, const float *sumsq_dev, float max_norm, void *stream);

/* ---- gradient exchange: NCCL, loaded with dlopen at first use -----------------
 * One communicator per process (one process per GPU).  Rank 0 makes a 128-byte id with
 * spgk_nccl_unique_id and hands it to the other ranks by any host channel. */
/* A training step whose launches have the same arguments every time, so that it can be replayed as a CUDA graph: what
 * changes from step to step -- the first row of the step in the shuffled order, Adam's bias corrections -- lives in a small
 * device record (spgk_train_state_bytes) that spgk_train_state_step advances as the first launch of every step, with
 * the host's own fp32 operations (Training.c:480-500).  After spgk_train_use_state(state) this thread's
 * spgk_gather_rows2 offsets its index list by the record's position and spgk_adam / spgk_optimizer_step take mf and vf
 * from it; NULL switches back.  spgk_graph_begin / _end capture the launches issued on `stream` in between
 * (relaxed capture mode) and return an executable graph; _launch replays it; a capture that fails returns an error and
 * leaves the stream usable. */
SPGK_API size_t spgk_train_state_bytes(void);
SPGK_API int spgk_train_state_reset(void *state, void *stream);
SPGK_API int spgk_train_state_step(void *state, uint32_t steps_per_epoch, uint32_t batch, float b1, float b2, void *stream);
SPGK_API void spgk_train_use_state(const void *state);
SPGK_API int spgk_graph_begin(void *stream);
SPGK_API int spgk_graph_end(void *stream, void **exec);
SPGK_API int spgk_graph_launch(void *exec, void *stream);
SPGK_API void spgk_graph_destroy(void *exec);
SPGK_API int spgk_nccl_unique_id(void *id128);
SPGK_API int spgk_nccl_init(void **comm, int rank, int world, const void *id128);
SPGK_API int spgk_nccl_allreduce_sum(void *comm, float *buf, uint64_t count, void *stream);
/* two buffers summed in one grouped NCCL launch */
SPGK_API int spgk_nccl_allreduce_sum2(void *comm, float *buf_a, uint64_t count_a, float *buf_b, uint64_t count_b,
                                     void *stream);
SPGK_API int spgk_nccl_destroy(void *comm);

/* ---- K5: the gradient exchange of data-parallel training in one kernel over peer memory ---------------------------
 * (no counterpart in the reference, whose data parallelism is OpenMP threads adding into one gradient buffer,
 * Training.c:396-419; the update rules are those of Training.c:439-507 / SIMD.c:279-494.)
 * spgk_xchg_create is collective over the ranks of `comm` (2..8, one process and one GPU each, all on one node): every
 * rank allocates an arena [flags | G | W | M | V] for np parameters, the IPC handles travel through a sum all-reduce
 * and the peers' arenas are mapped.  spgk_xchg_buffer gives this rank's own G (0), W (1), M (2), V (3): the training
 * kernels write gradients into G and read parameters from W.  spgk_xchg_step then does, in one launch on every rank:
 * sum of shard r of all ranks' G in rank order (peer loads), update rule `kind` (0 SGD, 1 MOMENTUM, 2 RMSPROP, 3 ADAM,
 * 4 ADAMW; arguments as spgk_optimizer_step) on shard r of W / M / V, new weights of the shard into every rank's W
 * (peer stores).  Afterwards all W are identical bit for bit; M and V are current in the owner's shard only, and
 * spgk_xchg_gather (collective as well) brings the shards of G (the summed gradients), M and V to every rank.
 * The ranks' kernels wait for one another through flags in peer memory, every wait bounded (about half a second):
 * spgk_xchg_status, called after a stream synchronisation, returns SPGK_E_TIMEOUT when one gave up.  All ranks must
 * issue the same sequence of step / gather calls (the running number of the collective lives in the arena and is advanced
 * by the kernels, and mfvf_dev -- two floats on the device, optional -- overrides mf and vf: a step's launch then has
 * the same arguments every time and can be part of a replayed graph).  No TMA, multicast or NVLS is involved. */
SPGK_API int spgk_xchg_create(void **xchg, int rank, int world, uint64_t np, void *comm, void *stream);
SPGK_API void spgk_xchg_destroy(void *xchg);
SPGK_API uint64_t spgk_xchg_capacity(const void *xchg);
SPGK_API float *spgk_xchg_buffer(void *xchg, int which);
SPGK_API int spgk_xchg_step(void *xchg, int kind, uint64_t n_weights, float lr, float momentum, float b1, float b2, float mf, float vf,
                            float eps, float decay, float gscale, const float *mfvf_dev, void *stream);
SPGK_API int spgk_xchg_gather(void *xchg, void *stream);
SPGK_API int spgk_xchg_status(void *xchg, void *stream);
/* the exchange's bounded wait on a flag nobody writes (16 uint32 of device scratch): leaves {1, 42, 7} in the first
 * three words -- timed out, status code recorded, thread carried on; limit = polls (at most 2^20) */
SPGK_API int spgk_selftest_xchg_wait(uint32_t *words16_dev, uint32_t limit, int sys_scope, void *stream);
/* Failure handling of the exchange (all on the host; nothing here makes a GPU fault or hang):
 * spgk_nccl_init waits for the rendezvous at most SPINGALETT_DIST_TIMEOUT_MS milliseconds (environment, default 120000) and
 * returns SPGK_E_TIMEOUT when a rank never arrives; spgk_stream_sync_bounded waits for a stream by polling with the same
 * limit, so an exchange whose peer has gone ends in SPGK_E_TIMEOUT instead of a blocked host thread, after which
 * spgk_nccl_abort (ncclCommAbort) releases the communicator. */
SPGK_API int spgk_stream_sync_bounded(void *stream);
SPGK_API int spgk_nccl_abort(void *comm);

/* ---- failure-path hooks (for tests; none of them faults, traps or hangs a GPU) ------------------
 * spgk_fail_malloc_after(k): the k-th spgk_malloc from now returns SPGK_E_NOMEM (k <= 0 switches it off);
 *   spgk_mem_info reads the device's free / total bytes, so a test can see that a failed call gave everything back.
 * spgk_selftest_bounded_wait: launches one small kernel that waits on a barrier nobody arrives on with the kernels' own
 *   bounded waits and `limit` attempts (<= 4096; each attempt may suspend the warp for 20 us); the kernel returns by itself,
 *   status3[0] holds the wait's code, and the call returns SPGK_E_TIMEOUT exactly as a GEMM whose wait gave up does.
 * spgk_selftest_timed_call: host only: a call that answers after answer_ms under the rendezvous timeout wrapper with a
 *   limit of timeout_ms: 0 or SPGK_E_TIMEOUT.
 * spgk_selftest_once_per_device: host only: the once-per-device bookkeeping of the launchers over `devices` fake indices and
 *   `calls` rounds, device `fail_first` failing its first set-up: returns the number of set-ups that ran. */
SPGK_API void spgk_fail_malloc_after(int k);
SPGK_API int spgk_mem_info(size_t *free_bytes, size_t *total_bytes);
SPGK_API int spgk_selftest_bounded_wait(int32_t *status3, uint32_t limit, void *stream);
SPGK_API int spgk_selftest_timed_call(int answer_ms, int timeout_ms);
SPGK_API int spgk_selftest_once_per_device(int devices, int calls, int fail_first);

/* ---- K2 without allocations ----------------------------------------------
 * (No counterpart in the reference: it has no GPU code and no scratch memory.)
 * The same layer as spgk_layer_gemm_tc, for callers that cannot allocate device
 * memory: a server that handed all of HBM to its own arena at start-up, or a
 * latency-critical loop that cannot take the device-wide synchronisation hidden
 * in cudaMalloc/cudaFree.  The caller still passes the packed layer, the 16-bit
 * activations and the output buffers; the scratch (the 16-bit weight operand
 * expanded from the packed payload, and the kernel's status word) is a fixed
 * array inside the library's device image.  Every GPU that loads the library
 * holds that array until the process exits.
 *   - Limit: the expanded weight operand, out * round_up(in, 8) * 2 bytes (twice
 *     that for FP32 files with a_parts == 2), must fit
 *     SPGK_NOALLOC_MAX_WEIGHT_BYTES; larger layers are refused with SPGK_E_ARG
 *     and a message naming both sizes.  FP16/BF16 payloads that TMA can read in
 *     place need no weight scratch at all.
 *   - The first call on each device looks up the array's device address.  With
 *     CUDA's lazy module loading the array's memory is reserved when the
 *     library's device code is first used on a device, not when the library is
 *     loaded: make one warm-up call per device (or load modules eagerly) BEFORE
 *     the caller's arena takes the remaining memory.  Every call waits for its
 *     stream before it returns (it reads the status word back).
 *   - All calls share the one array and it keeps the previous call's contents
 *     (this function clears what has to start at zero), so two calls that
 *     overlap on the GPU -- different streams, different host threads -- race.
 *   - The call calls no cudaMalloc, cudaFree or allocating library routine, and
 *     returns after the stream has finished the layer (it reads the status word
 *     back): SPGK_OK, or SPGK_E_TIMEOUT if a bounded wait gave up. */
#define SPGK_NOALLOC_MAX_WEIGHT_BYTES (8u << 20)
SPGK_API int spgk_layer_gemm_tc_noalloc(const spgk_layer *L,
                                        const void *a16, uint32_t lda, uint64_t a_plane, int a_parts, int type16,
                                        void *out16, uint32_t ldo16, uint64_t o_plane, int out_parts,
                                        float *out32, uint32_t ldo32,
                                        uint32_t N, int softmax_fused, void *stream);

#ifdef __cplusplus
}
#endif
