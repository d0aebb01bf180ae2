// spg_common.cuh -- helpers shared by the sm_100a kernels: error plumbing,
// launch accounting, activation math and the element decoders for the six
// stored weight precisions.
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <float.h>
#include <mutex>
#include "spingalett_b200_kernels.h"

// enum values of the public header (ActivationFunction / PrecisionMode)
enum { SPG_ACT_SIGMOID = 0, SPG_ACT_RELU, SPG_ACT_TANH, SPG_ACT_LEAKY, SPG_ACT_FOO52, SPG_ACT_SOFTMAX, SPG_ACT_NONE };
enum { SPG_P_F32 = 0, SPG_P_F16, SPG_P_BF16, SPG_P_I8, SPG_P_I4, SPG_P_I2, SPG_P_COUNT };

void spgk_set_error(const char *what, const char *detail);
void spgk_count_launch(unsigned n = 1);
int  spgk_check_launch(const char *kernel_name);

#define SPGK_CUDA(call)                                                          \
    do {                                                                         \
        cudaError_t e__ = (call);                                                \
        if (e__ != cudaSuccess) {                                                \
            spgk_set_error(#call, cudaGetErrorString(e__));                      \
            return e__ == cudaErrorMemoryAllocation ? SPGK_E_NOMEM : SPGK_E_CUDA; \
        }                                                                        \
    } while (0)

// ---- per-device launcher state ----------------------------------------------
// SM count, compute capability and the opt-in shared-memory limit of a device, looked up once per
// device (a process may use several: spingalett_set_device, per-net device binding).
#define SPG_MAX_DEVICES 64
struct SpgDeviceProps { int cc; int sm_count; size_t smem_optin; };
// properties of the CURRENT device (cached per device under a mutex); SPGK_OK or an error code
int spg_device_props(SpgDeviceProps *out);

// Work that has to happen once per device and per kernel -- cudaFuncSetAttribute is per device -- keyed by
// the device index: `fn` runs the first time `device` is seen (and again if it failed), under a mutex.
struct SpgOncePerDevice {
    std::mutex lock;
    uint64_t done = 0;
    template <typename Fn> int run(int device, Fn fn)
    {
        if (device < 0 || device >= SPG_MAX_DEVICES) { spgk_set_error("device table", "device index out of range"); return SPGK_E_ARG; }
        std::lock_guard<std::mutex> g(lock);
        if ((done >> device) & 1u) return SPGK_OK;
        const int rc = fn();
        if (rc == SPGK_OK) done |= (uint64_t)1 << device;
        return rc;
    }
};

// Scalar activation, same comparisons as the reference (Activation.c:23-38):
// strict > and <, so ReLU(0)=0, FOO52(0)=0, FOO52(1)=1.  Softmax and "none"
// pass through.  expf/tanhf are the accurate CUDA versions (<= 2 ulp).
__device__ __forceinline__ float spg_activate(float x, int act)
{
    switch (act) {
        case SPG_ACT_RELU:    return x > 0.0f ? x : 0.0f;
        case SPG_ACT_LEAKY:   return x > 0.0f ? x : 0.01f * x;
        case SPG_ACT_SIGMOID: return 1.0f / (1.0f + expf(-x));
        case SPG_ACT_TANH:    return tanhf(x);
        case SPG_ACT_FOO52:   return x > 1.0f ? 1.0f + 0.01f * (x - 1.0f) : (x < 0.0f ? 0.01f * x : x);
        default:              return x;
    }
}

// Derivative through the activation OUTPUT (Activation.c:40-56).
__device__ __forceinline__ float spg_derivative(float a, int act)
{
    switch (act) {
        case SPG_ACT_RELU:    return a > 0.0f ? 1.0f : 0.0f;
        case SPG_ACT_LEAKY:   return a > 0.0f ? 1.0f : 0.01f;
        case SPG_ACT_SIGMOID:
        case SPG_ACT_SOFTMAX: return a * (1.0f - a);
        case SPG_ACT_TANH:    return 1.0f - a * a;
        case SPG_ACT_FOO52:   return (a > 1.0f || a < 0.0f) ? 0.01f : 1.0f;
        default:              return 1.0f;
    }
}

// Unscaled value of element `idx` of a stored array (multiply by w_scale for
// the integer formats).  Bit positions as written by Serialize.c:148-152
// (INT4: even index -> low nibble) and :180-183 (INT2: element i at bits
// 2*(i%4)); sign extension as read back at :257 and :284.
__device__ __forceinline__ float spg_decode_elem(const void *base, uint64_t idx, int precision)
{
    switch (precision) {
        case SPG_P_F32:  return reinterpret_cast<const float *>(base)[idx];
        case SPG_P_F16:  return __half2float(reinterpret_cast<const __half *>(base)[idx]);
        case SPG_P_BF16: return __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(base)[idx]);
        case SPG_P_I8:   return (float)reinterpret_cast<const int8_t *>(base)[idx];
        case SPG_P_I4: {
            uint32_t b = reinterpret_cast<const uint8_t *>(base)[idx >> 1];
            int v = (int)((b >> ((idx & 1u) * 4u)) & 0xFu);
            return (float)(v >= 8 ? v - 16 : v);
        }
        default: {
            uint32_t b = reinterpret_cast<const uint8_t *>(base)[idx >> 2];
            int v = (int)((b >> ((idx & 3u) * 2u)) & 0x3u);
            return (float)(v >= 2 ? v - 4 : v);
        }
    }
}

// bytes per 8 consecutive elements of a stored array
__host__ __device__ inline uint32_t spg_bits_per_elem(int precision)
{
    switch (precision) {
        case SPG_P_F32: return 32;
        case SPG_P_F16: case SPG_P_BF16: return 16;
        case SPG_P_I8: return 8;
        case SPG_P_I4: return 4;
        default: return 2;
    }
}

__device__ __forceinline__ float spg_warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float spg_warp_max(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Device-resident row count set by spgk_set_dynamic_rows for the calling thread (NULL = off): the row-wise
// kernels launched afterwards process min(rows argument, *limit) rows, the limit being read on the device.
extern thread_local const uint32_t *spg_tls_rows_limit;
extern thread_local uint32_t spg_tls_rows_expected;      // the caller's estimate of *limit (0 = none)
// margin sink set by spgk_set_margin_sink for the calling thread (idx == NULL: off)
extern thread_local float spg_tls_margin_theta;
extern thread_local uint32_t *spg_tls_margin_idx, *spg_tls_margin_count;
extern thread_local const uint32_t *spg_tls_out_rows;      // spgk_set_output_rows: fp32 output row r of the tensor-core layer goes to row out_rows[r]
__device__ __forceinline__ uint32_t spg_limit_rows(uint32_t rows, const uint32_t *limit)
{
    if (!limit) return rows;
    const uint32_t v = *limit;
    return v < rows ? v : rows;
}

// Programmatic dependent launch.  A kernel started through spg_launch_chained may be scheduled while the kernel
// before it in the stream is still draining; it must call spg_grid_wait() before it reads or writes anything
// that an earlier kernel of the stream touches, and spg_grid_trigger() lets the kernel behind it do the same.
__device__ __forceinline__ void spg_grid_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void spg_grid_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t spg_launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

