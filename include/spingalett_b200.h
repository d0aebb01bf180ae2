/*
 * spingalett_b200.h -- public C ABI of the B200-native Spingalett library.
 *
 * PART 1 is the binary interface of pka-human/Spingalett
 * (Include/Spingalett/Spingalett.h in that project): the same enumerator
 * values, the same struct layouts (x86-64 SysV: NeuralNetwork 160 bytes,
 * LayerArgs 24, ForwardArgs 16, TrainArgs 152, SaveArgs 24), the same 21
 * exported functions and the same call macros, so that a program built against
 * the reference links against this library unchanged.  Behind it every
 * forward/train call runs hand-written sm_100a CUDA kernels; there is no CPU
 * compute path and no fallback -- without a usable CUDA device the compute
 * entry points fail with SPINGALETT_ERR_DEVICE.
 *
 * PART 2 lists the entry points this library adds.  They exist because the
 * reference has no public batched inference call (its batched forward is a
 * file-static helper of the trainer, Src/Spingalett.Training.c:313-345).
 */
#pragma once

#include <stdint.h>
#include <stdbool.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#ifndef SPINGALETT_API
#  define SPINGALETT_API __attribute__((visibility("default")))
#endif

/* ======================================================================== */
/* PART 1 -- the reference ABI                                               */
/* ======================================================================== */

/* File format revision understood by load/save (reference Spingalett.h:26). */
#define SPINGALETT_FORMAT_VERSION 1

/* Spingalett.h:28-34 */
typedef enum { LOG_DEBUG, LOG_INFO, LOG_WARNING, LOG_ERROR, LOG_NONE } LogLevel;
typedef void (*LogCallback)(LogLevel level, const char *message);

/* Spingalett.h:38-47.  Stored as one byte per layer in .nn files, so the
 * numeric values are part of the file format. */
typedef enum {
    ACT_SIGMOID,      /* 1/(1+exp(-x))                                  */
    ACT_RELU,         /* x>0 ? x : 0                                    */
    ACT_TANH,         /* tanh(x)                                        */
    ACT_LEAKY_RELU,   /* x>0 ? x : 0.01x                                */
    ACT_FOO52,        /* x<0 ? 0.01x : x>1 ? 1+0.01(x-1) : x            */
    ACT_SOFTMAX,      /* over the whole layer                           */
    ACT_NONE,         /* identity                                       */
    ACT_COUNT
} ActivationFunction;

/* Spingalett.h:49-53 */
typedef enum { LOSS_MSE, LOSS_CROSS_ENTROPY, LOSS_COUNT } LossFunction;

/* Spingalett.h:55-61.  XAVIER here means N(0,1)*sqrt(1/fan_in), HE means
 * N(0,1)*sqrt(2/fan_in), RANDOM means U(-1,1) (reference Network.c:150-162). */
typedef enum {
    WEIGHT_INITIALIZATION_RANDOM,
    WEIGHT_INITIALIZATION_XAVIER,
    WEIGHT_INITIALIZATION_HE,
    WEIGHT_INITIALIZATION_NONE,
    WEIGHT_INITIALIZATION_COUNT
} WeightInitialization;

/* Spingalett.h:63-67 */
typedef enum { MODE_ARRAY, MODE_GENERATOR_FUNCTION, MODE_COUNT } TrainingMode;

/* Spingalett.h:69-74 */
typedef enum { STRATEGY_SAMPLE, STRATEGY_FULL_BATCH, STRATEGY_SMALL_BATCH, STRATEGY_COUNT } TrainingStrategy;

/* Spingalett.h:76-83 */
typedef enum {
    OPTIMIZER_SGD, OPTIMIZER_MOMENTUM, OPTIMIZER_RMSPROP, OPTIMIZER_ADAM, OPTIMIZER_ADAMW, OPTIMIZER_COUNT
} OptimizerType;

/* Spingalett.h:85-91.  Accepted and recorded for compatibility; this library
 * always computes on CUDA whatever the recorded mode is. */
typedef enum {
    COMPUTE_SINGLE_THREADED, COMPUTE_OPENMP, COMPUTE_OPENBLAS, COMPUTE_CUDA, COMPUTE_COUNT
} ComputeMode;

/* Spingalett.h:93-101.  One byte in the .nn header; selects the array codec:
 *   FLOAT32  raw little-endian floats
 *   FP16     IEEE half, produced by truncation
 *   BFLOAT16 upper 16 bits of the float
 *   INT8/4/2 one float abs-max in front of the array, then signed integers
 *            q with value q*max/127, q*max/7, q*max (ternary); INT4 packs the
 *            even element in the low nibble; INT2 packs element i at bits
 *            2*(i%4); packing runs across matrix rows. */
typedef enum {
    PRECISION_FLOAT32, PRECISION_FP16, PRECISION_BFLOAT16,
    PRECISION_INT8, PRECISION_INT4, PRECISION_INT2, PRECISION_COUNT
} PrecisionMode;

/* Spingalett.h:103-107 */
typedef enum { AUTOSAVE_OFF, AUTOSAVE_OVERWRITE, AUTOSAVE_NEW_FILES } AutoSaveMode;

/* Spingalett.h:109-136.  The network is a public, caller-visible struct.
 * weights: concatenation over layers of row-major [out][in] matrices
 * (weights[weight_offsets[l] + j*topology[l] + k]); biases: concatenation of
 * [out] vectors; neurons: one sample's activations, layer after layer.  In
 * this library these host arrays are fp32 mirrors: the GPU holds the weights
 * in the precision they were loaded in.  grad_* and opt_* stay NULL until the
 * first train() call on the network.  After writing to weights/biases by hand
 * call spingalett_sync_weights(). */
typedef struct {
    uint32_t layers;
    uint32_t *topology;
    ActivationFunction *act_func;

    float *weights;
    float *biases;
    float *neurons;

    float *grad_weights;
    float *grad_biases;

    float *opt_m_weights;
    float *opt_m_biases;
    float *opt_v_weights;
    float *opt_v_biases;

    uint64_t *neuron_offsets;
    uint64_t *weight_offsets;
    uint64_t *bias_offsets;

    uint64_t total_neurons;
    uint64_t total_weights;
    uint64_t total_biases;

    uint64_t time_step;
    LossFunction loss_func;
} NeuralNetwork;

/* Spingalett.h:138 */
typedef bool (*TrainCallback)(NeuralNetwork *net, size_t epoch, float current_error);

/* Argument records (Spingalett.h:140-196).  Passed BY VALUE; a field left out
 * of the initialiser is zero, and zero selects the first enumerator. */
typedef struct { LossFunction loss_func; } NeuralNetworkArgs;

typedef struct {
    NeuralNetwork *net;
    uint32_t neurons_amount;
    ActivationFunction act_func;
    WeightInitialization weight_initialization;
} LayerArgs;

typedef struct {
    NeuralNetwork *net;
    const float *input;
} ForwardArgs;

typedef struct {
    NeuralNetwork *net;
    TrainingMode training_mode;
    TrainingStrategy training_strategy;
    OptimizerType optimizer_type;

    float *inputs;
    float *targets;
    uint32_t sample_count;
    uint32_t batch_size;
    size_t epochs;

    float learning_rate;
    float weight_decay;
    float momentum;
    float beta1;
    float beta2;
    float epsilon;
    float max_grad_norm;

    bool reset_optimizer;
    size_t nan_check_interval;

    size_t report_interval;

    AutoSaveMode autosave_mode;
    size_t autosave_interval;
    const char *autosave_path;
    bool autosave_do_not_save_optimizer;
    PrecisionMode autosave_precision;

    TrainCallback callback;
    size_t callback_interval;
} TrainArgs;

typedef struct {
    NeuralNetwork *net;
    const char *filename;
    bool do_not_save_optimizer;
    PrecisionMode precision;
} SaveArgs;

/* Error codes (Spingalett.h:198-200) plus one added code for CUDA failures. */
#define SPINGALETT_OK           0
#define SPINGALETT_ERR_ALLOC    1
#define SPINGALETT_ERR_INVALID  2
#define SPINGALETT_ERR_DEVICE   3   /* extension: CUDA/NCCL call failed or no device */

/* Thread-local, sticky until cleared (reference Error.c:9-22). */
SPINGALETT_API int spingalett_last_error_code(void);                 /* Spingalett.h:202 */
SPINGALETT_API const char *spingalett_last_error_message(void);      /* :203 */
SPINGALETT_API void spingalett_clear_error(void);                    /* :204 */

SPINGALETT_API ComputeMode spingalett_get_compute_mode(void);        /* :206 */
SPINGALETT_API void spingalett_set_compute_mode(ComputeMode mode);   /* :207 */
SPINGALETT_API unsigned spingalett_get_num_threads(void);            /* :208 */
SPINGALETT_API void spingalett_set_num_threads(unsigned n);          /* :209 */

SPINGALETT_API void spingalett_set_log_callback(LogCallback cb);     /* :211 */
SPINGALETT_API void spingalett_set_log_level(LogLevel level);        /* :212 */
SPINGALETT_API void spingalett_set_verbose(bool enabled);            /* :214 */
SPINGALETT_API bool spingalett_get_verbose(void);                    /* :215 */

/* The call macros take positional or designated initialisers and need a C
 * compiler (compound literals); C++ callers use the *_struct_arguments names. */
#ifndef __cplusplus
#define new_spingalett(...)  new_spingalett_struct_arguments((NeuralNetworkArgs){__VA_ARGS__})
#define layer(...)           layer_struct_arguments((LayerArgs){__VA_ARGS__})
#define forward(...)         forward_struct_arguments((ForwardArgs){__VA_ARGS__})
#define train(...)           train_struct_arguments((TrainArgs){__VA_ARGS__})
#define save_spingalett(...) save_spingalett_struct_arguments((SaveArgs){__VA_ARGS__})
#endif

/* :218 -- empty network; NULL + ERR_INVALID on a bad loss value. */
SPINGALETT_API NeuralNetwork *new_spingalett_struct_arguments(NeuralNetworkArgs args);

/* :221 -- append a layer; the first call adds the input layer, later calls add
 * a weight matrix [neurons_amount][previous] initialised as requested.
 * NULL net or 0 neurons -> ERR_INVALID (reference Network.c:53-56). */
SPINGALETT_API void layer_struct_arguments(LayerArgs args);

/* :223-224 -- scalar activation and its derivative (the derivative takes the
 * activation OUTPUT, reference Activation.c:40-56). */
SPINGALETT_API float activate(float x, ActivationFunction act_func);
SPINGALETT_API float derivative(float x, ActivationFunction act_func);

/* :227 -- one sample through the network ON THE GPU.  `input` holds
 * topology[0] floats in host memory.  Returns a pointer into net->neurons
 * (the last layer's slice), valid until the next call on this net.  NULL net
 * or input returns NULL without touching the error state; fewer than two
 * layers is ERR_INVALID (reference Network.c:207-212). */
SPINGALETT_API float *forward_struct_arguments(ForwardArgs args);

/* :230 -- training.  Supported on the GPU: MODE_ARRAY with
 * STRATEGY_FULL_BATCH or STRATEGY_SMALL_BATCH, OPTIMIZER_ADAM,
 * LOSS_CROSS_ENTROPY over a softmax or sigmoid output layer.  Other
 * combinations (other optimizers, weight decay, gradient clipping, autosave, MSE)
 * are rejected with ERR_INVALID (no CPU path exists here).  On return the host
 * arrays of the net (weights, biases, grad_*, opt_*) hold the trained state. */
SPINGALETT_API void train_struct_arguments(TrainArgs args);

/* :233 -- write a .nn file in the requested precision; ".nn" is appended when
 * the name has no extension (reference Serialize.c:321-336). */
SPINGALETT_API void save_spingalett_struct_arguments(SaveArgs args);

/* :235 -- read a .nn file.  The packed payload goes to the GPU as stored (no
 * fp32 expansion on the device); net->weights/biases receive the dequantised
 * fp32 values the reference loader would produce.  A truncated payload sets
 * ERR_INVALID but still returns the partly filled net (Serialize.c:596-608). */
SPINGALETT_API NeuralNetwork *load_spingalett(const char *filename);

SPINGALETT_API void print_parameters(NeuralNetwork *net);            /* :237 */
SPINGALETT_API void free_network(NeuralNetwork *net);                /* :238, NULL-safe */

/* ======================================================================== */
/* PART 2 -- additions of this library (no counterpart in the reference ABI) */
/* ======================================================================== */

/* Batched inference: the public form of the reference's static
 * batch_forward() (Training.c:313-345).  inputs is row-major
 * [sample_count][topology[0]], outputs row-major [sample_count][topology[last]].
 * Either pointer may be host memory or memory of the current CUDA device
 * (detected per call).  outputs == NULL selects a library-owned host buffer
 * that stays valid until the next batched call on the net.  Returns the
 * output pointer, or NULL with the error state set.  With host buffers the
 * call returns when the result is complete; when BOTH pointers are device
 * memory the call is stream-ordered and returns after enqueueing -- use
 * spingalett_synchronize() (or synchronise the stream) before reading. */
typedef struct {
    NeuralNetwork *net;
    const float *inputs;
    uint32_t sample_count;
    float *outputs;
} ForwardBatchArgs;
#ifndef __cplusplus
#define forward_batch(...) forward_batch_struct_arguments((ForwardBatchArgs){__VA_ARGS__})
#endif
SPINGALETT_API float *forward_batch_struct_arguments(ForwardBatchArgs args);
/* Waits for the net's stream and reports a kernel-side failure, if any. */
SPINGALETT_API int spingalett_synchronize(NeuralNetwork *net);

/* How activations are fed to the tensor cores on the large-batch path.
 * EXACT : two 16-bit terms hi+lo (>= 16 significant bits) at twice the tensor
 *         work; products with 16-bit or integer weights are exact and only the
 *         fp32 accumulation order differs from the reference.
 * FAST  : one fp16 term per operand (11 significant bits; a BF16 file's weights
 *         are exact in fp16 while they lie within its range -- checked once per
 *         upload -- else bf16 terms, 8 bits, are used).  Measured on the
 *         784-512-1000-10 MLP: ~99.95 % argmax agreement with the reference with
 *         fp16, ~99.7 % with bf16, i.e. at or below the 99.9 % parity bar.
 * AUTO (default): the FAST pass, then every row whose two largest softmax
 *         outputs are within a margin (log p1 - log p2 < margin) is recomputed
 *         in EXACT mode and written over the fast result (so is a row whose
 *         FAST result is not finite: an input or hidden value beyond the fp16
 *         range); the argmax is then expected to be the EXACT one at close to
 *         FAST cost, and the probabilities of the other rows keep the FAST
 *         error (<= 3e-4 measured with fp16, against a 2e-3 bar).
 *         The margin is measured, not guessed: on the first AUTO call after a
 *         net's weights reach the GPU both modes run on up to 2048 rows of the
 *         batch and the margin becomes four times the largest change of the
 *         top-two log gap that the FAST pass caused there (measured range: the
 *         change is below 0.002 with fp16 operands, 0.013 with bf16).
 *         spingalett_set_auto_margin(m > 0) fixes the margin instead; 0 returns
 *         to calibration.  Networks that do not end in softmax run EXACT.
 *         LIMIT: the calibration is a measurement on up to 2048 rows of the
 *         first large batch a net sees, repeated on every 1024th large call
 *         (the margin then only grows); between two measurements inputs of a
 *         different character are judged by the old margin.  AUTO's agreement
 *         with EXACT is that measurement's expectation (the parity tests allow
 *         3 differing rows in 16384), not a guarantee.  Callers that need the
 *         guarantee use SPINGALETT_MATH_EXACT.
 * The small-batch paths always use exact products (they are memory-bound), and
 * AUTO runs batches of up to 512 rows in EXACT: a chain that is bound by
 * streaming the weights pays next to nothing for the second term. */
typedef enum { SPINGALETT_MATH_FAST = 0, SPINGALETT_MATH_EXACT = 1, SPINGALETT_MATH_AUTO = 2 } SpingalettMathMode;
SPINGALETT_API void spingalett_set_math_mode(SpingalettMathMode mode);
SPINGALETT_API SpingalettMathMode spingalett_get_math_mode(void);
SPINGALETT_API void spingalett_set_auto_margin(float log_gap);
SPINGALETT_API float spingalett_get_auto_margin(void);
/* rows the last AUTO-mode call on this net recomputed exactly */
SPINGALETT_API uint32_t spingalett_last_repaired(NeuralNetwork *net);
/* the calibrated margin of this net (0 before its first AUTO call) */
SPINGALETT_API float spingalett_net_margin(NeuralNetwork *net);

/* CUDA device used by the calling process for nets created afterwards
 * (default: the current device).  Returns 0 or an error code. */
SPINGALETT_API int spingalett_set_device(int device);
SPINGALETT_API int spingalett_get_device_count(void);
/* Batch sharding over several GPUs of this process: after spingalett_set_devices(ids, n) with n >= 2, forward_batch
 * calls with HOST input and output buffers cut the batch into n contiguous row shares (share g = rows
 * [g*N/n, (g+1)*N/n), sizes differing by at most one: spingalett_split_rows) and run share g on device ids[g] from a
 * replica of the weights there -- one host thread and one stream per device, weights replicated, no peer access and
 * no collective.  n <= 1 switches it off; an id may be listed twice.  Device-pointer batches and batches of fewer than
 * 2n rows run on the net's own device as before.  (No reference counterpart: its forward is CPU code.) */
SPINGALETT_API int spingalett_set_devices(const int *ids, int n);
SPINGALETT_API void spingalett_split_rows(uint32_t rows, uint32_t shares, uint32_t share, uint32_t *lo, uint32_t *hi);

/* CUDA stream (a cudaStream_t passed as void*) on which this net's kernels
 * and copies are issued; NULL selects the legacy default stream. */
SPINGALETT_API void spingalett_set_stream(NeuralNetwork *net, void *cuda_stream);

/* Re-upload after the caller edited net->weights / net->biases in place.  The
 * device copy becomes an fp32 image of the host arrays. */
SPINGALETT_API int spingalett_sync_weights(NeuralNetwork *net);

/* Seed the calling thread's weight-initialisation generator (the reference
 * keeps the equivalent hook private, Src/Spingalett.Random.c:18). */
SPINGALETT_API void spingalett_seed(uint64_t seed);

/* Data-parallel training, one process per GPU.  Rank 0 creates a 128-byte id
 * (spingalett_dist_unique_id) and passes it to the other ranks over any host
 * channel; every rank then calls spingalett_dist_init(rank, world, id).  From
 * then on every step of train() sums the flat gradient buffer [gW | gB] across
 * ranks and applies the update with the 1/world average folded in: by default in
 * one kernel per rank over peer memory (CUDA IPC between the processes of one
 * node; shard r is summed in rank order and updated by rank r, the new weights
 * are stored into every replica), else with NCCL all-reduces (when a rank cannot
 * map its peers, with gradient clipping, or with SPINGALETT_EXCHANGE=nccl in the
 * environment; the ranks vote, so all take the same way).  Either way the
 * replicas stay bit-identical.  The reference has no multi-process mode; single-rank train()
 * behaves like its batched trainer (Training.c:691-817). */
SPINGALETT_API int spingalett_dist_unique_id(void *id128);
SPINGALETT_API int spingalett_dist_init(int rank, int world, const void *id128);
SPINGALETT_API void spingalett_dist_shutdown(void);
SPINGALETT_API int spingalett_dist_world(void);
/* A data-parallel train() first makes sure that every rank is about to run the same loop (equal sample_count,
 * batch_size, epochs, strategy, optimizer, callback / NaN-check intervals): otherwise the ranks would issue different
 * numbers of gradient exchanges and one of them would wait for ever.  The check is a SUM over ranks of
 * spingalett_dist_agreement_floats() floats written by spingalett_dist_pack_agreement; a rank whose
 * spingalett_dist_check_agreement(summed, own, world) returns 0 refuses to train (SPINGALETT_ERR_INVALID).  During
 * training the epoch's stop decision (callback, non-finite weights) is summed the same way, so all ranks stop together.
 * The three functions are exported so that the check can be run over any transport. */
SPINGALETT_API int spingalett_dist_agreement_floats(void);
SPINGALETT_API void spingalett_dist_pack_agreement(const TrainArgs *args, float *out);
SPINGALETT_API int spingalett_dist_check_agreement(const float *summed, const float *own, int world);

/* Kernel timing for benchmarks: while enabled, the library brackets each
 * large-batch layer kernel with CUDA events on the net's stream;
 * spingalett_profile_read returns (and resets) the summed device time in
 * milliseconds and the number of kernels timed. */
SPINGALETT_API void spingalett_profile(NeuralNetwork *net, bool enable);
SPINGALETT_API void spingalett_profile_read(NeuralNetwork *net, double *kernel_ms, uint64_t *launches);

/* Number of kernels this library has launched in the calling process, and the
 * name of the compute path the last batched/forward call took ("gemv",
 * "wstream", "tcgen05", "tcgen05-fused" -- the three-layer net in one launch --, "simt").  For benchmarks and tests. */
SPINGALETT_API uint64_t spingalett_kernel_launches(void);
SPINGALETT_API const char *spingalett_last_path(void);

#ifdef __cplusplus
}
#endif
