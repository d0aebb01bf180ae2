/* Host-side array codecs of the .nn format (used by load/save; the GPU reads
 * the packed bytes directly).  Behaviour follows the reference's
 * Src/Spingalett.Serialize.c: truncating fp16/bf16 encoders (:12-43, :74-78),
 * exact decoders (:45-72, :80-85), symmetric per-array abs-max integer
 * formats (:110-190 write, :222-294 read). */
#include "spg_internal.h"
#include <math.h>
#include <string.h>

static uint32_t bits_of(float x) { uint32_t u; memcpy(&u, &x, 4); return u; }
static float float_of(uint32_t u) { float x; memcpy(&x, &u, 4); return x; }

static uint16_t enc_f16(float x)
{
    uint32_t u = bits_of(x);
    uint32_t sign = (u >> 16) & 0x8000u, ebits = (u >> 23) & 0xFFu, man = u & 0x7FFFFFu;
    if (ebits == 0) return (uint16_t)sign;                       /* zero and fp32 denormals */
    if (ebits == 0xFF) return (uint16_t)(sign | (man ? 0x7E00u : 0x7C00u));
    int e = (int)ebits - 127;
    if (e > 15) return (uint16_t)(sign | 0x7C00u);
    if (e < -24) return (uint16_t)sign;
    if (e < -14) return (uint16_t)(sign | ((man | 0x800000u) >> (-1 - e)));
    return (uint16_t)(sign | ((uint32_t)(e + 15) << 10) | (man >> 13));
}

static float dec_f16(uint16_t h)
{
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16, e = (h >> 10) & 0x1Fu, m = h & 0x3FFu;
    if (e == 31) return float_of(sign | (m ? 0x7FC00000u : 0x7F800000u));
    if (e) return float_of(sign | ((e + 112u) << 23) | (m << 13));
    if (!m) return float_of(sign);
    uint32_t ex = 113;
    while (!(m & 0x400u)) { m <<= 1; ex--; }
    return float_of(sign | (ex << 23) | ((m & 0x3FFu) << 13));
}

float spg_precision_q(PrecisionMode p)
{
    return p == PRECISION_INT8 ? 127.0f : p == PRECISION_INT4 ? 7.0f : 1.0f;
}

size_t spg_array_bytes(uint64_t count, PrecisionMode p)
{
    switch (p) {
        case PRECISION_FLOAT32: return (size_t)(4 * count);
        case PRECISION_FP16: case PRECISION_BFLOAT16: return (size_t)(2 * count);
        case PRECISION_INT8: return (size_t)(4 + count);
        case PRECISION_INT4: return (size_t)(4 + (count + 1) / 2);
        case PRECISION_INT2: return (size_t)(4 + (count + 3) / 4);
        default: return 0;
    }
}

void spg_decode_array(const uint8_t *src, uint64_t count, PrecisionMode p, float *dst)
{
    if (p == PRECISION_FLOAT32) { memcpy(dst, src, 4 * count); return; }
    if (p == PRECISION_FP16 || p == PRECISION_BFLOAT16) {
        for (uint64_t i = 0; i < count; i++) {
            uint16_t h; memcpy(&h, src + 2 * i, 2);
            dst[i] = p == PRECISION_FP16 ? dec_f16(h) : float_of((uint32_t)h << 16);
        }
        return;
    }
    float amax; memcpy(&amax, src, 4);
    src += 4;
    if (!(amax > 0.0f)) { memset(dst, 0, 4 * count); return; }
    if (p == PRECISION_INT8) {
        for (uint64_t i = 0; i < count; i++) dst[i] = ((float)(int8_t)src[i] / 127.0f) * amax;
    } else if (p == PRECISION_INT4) {
        for (uint64_t i = 0; i < count; i++) {
            int v = (src[i >> 1] >> ((i & 1) * 4)) & 0xF;
            if (v & 8) v -= 16;
            dst[i] = ((float)v / 7.0f) * amax;
        }
    } else {
        for (uint64_t i = 0; i < count; i++) {
            int v = (src[i >> 2] >> ((i & 3) * 2)) & 3;
            if (v & 2) v -= 4;
            dst[i] = (float)v * amax;
        }
    }
}

size_t spg_encode_array(const float *src, uint64_t count, PrecisionMode p, uint8_t *dst)
{
    size_t total = spg_array_bytes(count, p);
    if (p == PRECISION_FLOAT32) { memcpy(dst, src, 4 * count); return total; }
    if (p == PRECISION_FP16 || p == PRECISION_BFLOAT16) {
        for (uint64_t i = 0; i < count; i++) {
            uint16_t h = p == PRECISION_FP16 ? enc_f16(src[i]) : (uint16_t)(bits_of(src[i]) >> 16);
            memcpy(dst + 2 * i, &h, 2);
        }
        return total;
    }
    float amax = 0.0f;
    for (uint64_t i = 0; i < count; i++) { float a = fabsf(src[i]); if (a > amax) amax = a; }
    memcpy(dst, &amax, 4);
    uint8_t *q = dst + 4;
    memset(q, 0, total - 4);
    if (!(amax > 0.0f)) return total;
    if (p == PRECISION_INT8) {
        for (uint64_t i = 0; i < count; i++) q[i] = (uint8_t)(int8_t)roundf((src[i] / amax) * 127.0f);
    } else if (p == PRECISION_INT4) {
        for (uint64_t i = 0; i < count; i++) {
            int v = (int)(int8_t)roundf((src[i] / amax) * 7.0f);
            v = v > 7 ? 7 : (v < -8 ? -8 : v);
            q[i >> 1] |= (uint8_t)((v & 0xF) << ((i & 1) * 4));
        }
    } else {
        for (uint64_t i = 0; i < count; i++) {
            float r = src[i] / amax;
            int v = r > 0.5f ? 1 : (r < -0.5f ? -1 : 0);
            q[i >> 2] |= (uint8_t)((v & 3) << ((i & 3) * 2));
        }
    }
    return total;
}
