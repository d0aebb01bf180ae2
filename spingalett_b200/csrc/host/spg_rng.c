/* Weight-initialisation generator.  Same stream as the reference's
 * Src/Spingalett.Random.c so that a seeded net is reproducible across the two
 * libraries: xoshiro128+ state filled by four SplitMix64 steps (:18-31),
 * 24-bit uniforms (:58-60), Box-Muller cosine branch with u1 clamped at 1e-6
 * and pi written as 3.14159265f (:66-71), Fisher-Yates with modulo (:73-81).
 * State is per thread; an unseeded thread seeds itself from the clocks. */
#include "spg_internal.h"
#include <math.h>
#include <time.h>

static _Thread_local uint32_t t_s[4];
static _Thread_local bool t_seeded = false;

void spingalett_seed(uint64_t seed)
{
    uint64_t x = seed;
    for (int i = 0; i < 4; i++) {
        x += 0x9e3779b97f4a7c15ULL;
        uint64_t z = x;
        z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ULL;
        z = (z ^ (z >> 27)) * 0x94d049bb133111ebULL;
        t_s[i] = (uint32_t)(z ^ (z >> 31));
    }
    if (!(t_s[0] | t_s[1] | t_s[2] | t_s[3])) t_s[0] = 1;
    t_seeded = true;
}

uint32_t spg_rand_u32(void)
{
    if (!t_seeded) {
        uint64_t s = (uint64_t)time(NULL) ^ ((uint64_t)clock() * 6364136223846793005ULL);
        volatile int marker = 0;
        s ^= (uint64_t)(uintptr_t)&marker;
        spingalett_seed(s);
    }
    uint32_t r = t_s[0] + t_s[3];
    uint32_t t = t_s[1] << 9;
    t_s[2] ^= t_s[0];
    t_s[3] ^= t_s[1];
    t_s[1] ^= t_s[2];
    t_s[0] ^= t_s[3];
    t_s[2] ^= t;
    t_s[3] = (t_s[3] << 11) | (t_s[3] >> 21);
    return r;
}

static float unit_float(void) { return (float)(spg_rand_u32() >> 8) / 16777216.0f; }

float spg_rand_uniform_pm1(void) { return unit_float() * 2.0f - 1.0f; }

float spg_rand_normal(void)
{
    float u1 = unit_float();
    float u2 = unit_float();
    if (u1 < 1e-6f) u1 = 1e-6f;
    return sqrtf(-2.0f * logf(u1)) * cosf(2.0f * 3.14159265f * u2);
}

void spg_shuffle(uint32_t *idx, uint32_t n)
{
    if (n < 2) return;
    for (uint32_t i = n - 1; i > 0; i--) {
        uint32_t j = spg_rand_u32() % (i + 1);
        uint32_t t = idx[i]; idx[i] = idx[j]; idx[j] = t;
    }
}
