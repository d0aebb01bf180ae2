/* Process-wide settings (C11 atomics) and logging, mirroring the behaviour of
 * the reference's Src/Spingalett.Settings.c: level filter, then the verbose
 * gate for anything below a warning, then callback or "[LEVEL] text" on
 * stdout/stderr (:59-80).  The compute mode and thread count are recorded and
 * reported back but do not select a backend: everything runs on CUDA. */
#include "spg_internal.h"
#include <stdarg.h>
#include <stdatomic.h>
#include <stdio.h>

static _Atomic int      s_mode = COMPUTE_SINGLE_THREADED;
static _Atomic unsigned s_threads = 0;
static _Atomic int      s_level = LOG_INFO;
static _Atomic(LogCallback) s_cb = NULL;
static _Atomic bool     s_verbose = true;
static _Atomic int      s_math = SPINGALETT_MATH_AUTO;
static _Atomic float    s_margin = 0.0f;                /* 0 = calibrate per net */
static _Atomic bool     s_mode_note_done = false;
static _Thread_local const char *t_path = "none";

ComputeMode spingalett_get_compute_mode(void) { return (ComputeMode)atomic_load(&s_mode); }

void spingalett_set_compute_mode(ComputeMode mode)
{
    if ((unsigned)mode >= COMPUTE_COUNT) return;          /* out-of-range values are ignored, Settings.c:27 */
    atomic_store(&s_mode, (int)mode);
    if (mode != COMPUTE_CUDA && !atomic_exchange(&s_mode_note_done, true))
        spg_log(LOG_DEBUG, "compute mode recorded; this build always computes on CUDA");
}

unsigned spingalett_get_num_threads(void) { return atomic_load(&s_threads); }
void spingalett_set_num_threads(unsigned n) { atomic_store(&s_threads, n); }
void spingalett_set_log_callback(LogCallback cb) { atomic_store(&s_cb, cb); }
void spingalett_set_log_level(LogLevel level) { atomic_store(&s_level, (int)level); }
void spingalett_set_verbose(bool enabled) { atomic_store(&s_verbose, enabled); }
bool spingalett_get_verbose(void) { return atomic_load(&s_verbose); }

void spingalett_set_math_mode(SpingalettMathMode mode)
{
    if (mode == SPINGALETT_MATH_FAST || mode == SPINGALETT_MATH_EXACT || mode == SPINGALETT_MATH_AUTO) atomic_store(&s_math, (int)mode);
}
SpingalettMathMode spingalett_get_math_mode(void) { return (SpingalettMathMode)atomic_load(&s_math); }
void spingalett_set_auto_margin(float log_gap) { atomic_store(&s_margin, log_gap > 0.0f ? log_gap : 0.0f); }
float spingalett_get_auto_margin(void) { return atomic_load(&s_margin); }

void spg_note_path(const char *name) { t_path = name; }
const char *spingalett_last_path(void) { return t_path; }
uint64_t spingalett_kernel_launches(void) { return spgk_launch_count(); }

void spg_log(LogLevel level, const char *fmt, ...)
{
    if ((int)level < atomic_load(&s_level)) return;
    if (!atomic_load(&s_verbose) && level < LOG_WARNING) return;
    char line[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(line, sizeof line, fmt, ap);
    va_end(ap);
    LogCallback cb = atomic_load(&s_cb);
    if (cb) { cb(level, line); return; }
    static const char *const tag[] = { "DEBUG", "INFO", "WARN", "ERROR", "NONE" };
    fprintf(level >= LOG_WARNING ? stderr : stdout, "[%s] %s\n", tag[level < LOG_NONE ? level : LOG_NONE], line);
}

const char *spg_act_name(unsigned a)
{
    static const char *const t[] = { "SIGMOID", "RELU", "TANH", "LEAKY_RELU", "FOO52", "SOFTMAX", "NONE" };
    return a < ACT_COUNT ? t[a] : "UNKNOWN";
}
const char *spg_precision_name(unsigned p)
{
    static const char *const t[] = { "FLOAT32", "FP16", "BFLOAT16", "INT8", "INT4", "INT2" };
    return p < PRECISION_COUNT ? t[p] : "UNKNOWN";
}
const char *spg_loss_name(unsigned l)
{
    static const char *const t[] = { "MSE", "CROSS_ENTROPY" };
    return l < LOSS_COUNT ? t[l] : "UNKNOWN";
}
