// spg_codec.cu -- the .nn array encoders on the device (reference Serialize.c:12-43 fp16 truncation, :74-78 bf16
// truncation, :110-190 per-array abs-max INT8 / INT4 / INT2), bit for bit: save_spingalett quantises a network
// of half a billion weights in milliseconds instead of seconds of scalar host code.
//
//   FP32            dst = src
//   FP16 / BF16     one 16-bit word per element, mantissa truncated (not rounded), fp32 denormals -> 0
//   INT8/INT4/INT2  [float abs-max][packed q], q = round-half-away(x / max * Q) (INT2: the sign of x/max beyond 0.5),
//                   INT4 two per byte (even index in the low nibble), INT2 four per byte; max <= 0 -> all zero
#include "spg_common.cuh"

namespace {

__device__ __forceinline__ uint16_t enc_f16_trunc(float x)
{
    const uint32_t u = __float_as_uint(x);
    const uint32_t sign = (u >> 16) & 0x8000u, ebits = (u >> 23) & 0xFFu, man = u & 0x7FFFFFu;
    if (ebits == 0) return (uint16_t)sign;
    if (ebits == 0xFF) return (uint16_t)(sign | (man ? 0x7E00u : 0x7C00u));
    const int e = (int)ebits - 127;
    if (e > 15) return (uint16_t)(sign | 0x7C00u);
    if (e < -24) return (uint16_t)sign;
    if (e < -14) return (uint16_t)(sign | ((man | 0x800000u) >> (-1 - e)));
    return (uint16_t)(sign | ((uint32_t)(e + 15) << 10) | (man >> 13));
}

// largest |x| of the array into *amax_bits (zeroed by the caller): non-negative floats order like their bit patterns
__global__ void __launch_bounds__(256)
spg_absmax_kernel(const float *__restrict__ src, uint64_t count, uint32_t *__restrict__ amax_bits)
{
    float m = 0.0f;
    for (uint64_t i = (uint64_t)blockIdx.x * 256 + threadIdx.x; i < count; i += (uint64_t)gridDim.x * 256) {
        const float a = fabsf(src[i]);
        if (a > m) m = a;                                     // a NaN never wins, as in the reference's loop
    }
    m = spg_warp_max(m);
    if ((threadIdx.x & 31u) == 0 && m > 0.0f) atomicMax(amax_bits, __float_as_uint(m));
}

__device__ __forceinline__ int quant(float x, float amax, int precision)
{
    if (precision == SPG_P_I8) return (int)(signed char)roundf(__fdiv_rn(x, amax) * 127.0f);
    if (precision == SPG_P_I4) {
        int v = (int)(signed char)roundf(__fdiv_rn(x, amax) * 7.0f);
        return v > 7 ? 7 : (v < -8 ? -8 : v);
    }
    const float r = __fdiv_rn(x, amax);
    return r > 0.5f ? 1 : (r < -0.5f ? -1 : 0);
}

// one thread per output byte of the packed payload (INT8: 1 element, INT4: 2, INT2: 4)
__global__ void __launch_bounds__(256)
spg_pack_int_kernel(const float *__restrict__ src, uint64_t count, int precision, const uint32_t *__restrict__ amax_bits, uint8_t *__restrict__ q)
{
    const float amax = __uint_as_float(*amax_bits);
    const uint32_t per = precision == SPG_P_I8 ? 1u : (precision == SPG_P_I4 ? 2u : 4u), bits = 8u / per;
    const uint64_t nbytes = (count + per - 1) / per;
    for (uint64_t b = (uint64_t)blockIdx.x * 256 + threadIdx.x; b < nbytes; b += (uint64_t)gridDim.x * 256) {
        uint32_t byte = 0;
        if (amax > 0.0f) {
            for (uint32_t j = 0; j < per; j++) {
                const uint64_t i = b * per + j;
                if (i < count) byte |= ((uint32_t)quant(src[i], amax, precision) & ((1u << bits) - 1u)) << (j * bits);
            }
        }
        q[b] = (uint8_t)byte;
    }
}

__global__ void __launch_bounds__(256)
spg_pack16_kernel(const float *__restrict__ src, uint64_t count, int precision, uint8_t *__restrict__ dst)
{
    for (uint64_t i = (uint64_t)blockIdx.x * 256 + threadIdx.x; i < count; i += (uint64_t)gridDim.x * 256) {
        const uint16_t h = precision == SPG_P_F16 ? enc_f16_trunc(src[i]) : (uint16_t)(__float_as_uint(src[i]) >> 16);
        dst[2 * i] = (uint8_t)(h & 0xFFu);                      // byte stores: the file offset of an array is arbitrary
        dst[2 * i + 1] = (uint8_t)(h >> 8);
    }
}

uint32_t blocks_for(uint64_t n) { const uint64_t b = (n + 255) / 256; return (uint32_t)(b < 148ull * 16 ? (b ? b : 1) : 148ull * 16); }

}  // namespace

extern "C" {

size_t spgk_encoded_bytes(uint64_t count, int precision)
{
    switch (precision) {
        case SPG_P_F32: return (size_t)(4 * count);
        case SPG_P_F16: case SPG_P_BF16: return (size_t)(2 * count);
        case SPG_P_I8: return (size_t)(4 + count);
        case SPG_P_I4: return (size_t)(4 + (count + 1) / 2);
        case SPG_P_I2: return (size_t)(4 + (count + 3) / 4);
        default: return 0;
    }
}

int spgk_encode_array(const float *src, uint64_t count, int precision, uint8_t *dst, void *stream)
{
    if (!src || !dst || (unsigned)precision >= SPG_P_COUNT) { spgk_set_error("spgk_encode_array", "bad argument"); return SPGK_E_ARG; }
    cudaStream_t st = (cudaStream_t)stream;
    if (count == 0) {
        if (precision >= SPG_P_I8) SPGK_CUDA(cudaMemsetAsync(dst, 0, 4, st));
        return SPGK_OK;
    }
    if (precision == SPG_P_F32) { SPGK_CUDA(cudaMemcpyAsync(dst, src, 4 * count, cudaMemcpyDeviceToDevice, st)); return SPGK_OK; }
    if (precision == SPG_P_F16 || precision == SPG_P_BF16) {
        spg_pack16_kernel<<<blocks_for(count), 256, 0, st>>>(src, count, precision, dst);
        return spgk_check_launch("spg_pack16_kernel");
    }
    if ((uintptr_t)dst & 3u) { spgk_set_error("spgk_encode_array", "integer formats start with a float: dst must be 4-byte aligned"); return SPGK_E_ARG; }
    SPGK_CUDA(cudaMemsetAsync(dst, 0, 4, st));
    spg_absmax_kernel<<<blocks_for(count), 256, 0, st>>>(src, count, reinterpret_cast<uint32_t *>(dst));
    int rc = spgk_check_launch("spg_absmax_kernel");
    if (rc) return rc;
    const uint32_t per = precision == SPG_P_I8 ? 1u : (precision == SPG_P_I4 ? 2u : 4u);
    spg_pack_int_kernel<<<blocks_for((count + per - 1) / per), 256, 0, st>>>(src, count, precision, reinterpret_cast<const uint32_t *>(dst), dst + 4);
    return spgk_check_launch("spg_pack_int_kernel");
}

}  // extern "C"
