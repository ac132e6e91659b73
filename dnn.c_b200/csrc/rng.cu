// Host random numbers for weight initialisation.
// replaces src/rng.c:6-78 of the reference: xorshift128+ (Vigna) seeded through
// two SplitMix64 rounds, a 53-bit uniform, single-sample Box-Muller and a
// mask-and-reject bounded integer.  The draw order of every consumer matches
// the reference so that the same seed gives the same weights.
#include "common.cuh"

namespace {

inline uint64_t splitmix64(uint64_t x) {
    x += 0x9e3779b97f4a7c15ULL;
    x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ULL;
    x = (x ^ (x >> 27)) * 0x94d049bb133111ebULL;
    return x ^ (x >> 31);
}

inline uint64_t next_u64(dnn_rng *r) {
    uint64_t a = r->s[0];
    const uint64_t b = r->s[1];
    r->s[0] = b;
    a ^= a << 23;
    r->s[1] = a ^ b ^ (a >> 18) ^ (b >> 5);
    return r->s[1] + b;
}

thread_local dnn_rng g_default_rng = {{1, 2}};

}  // namespace

extern "C" {

dnn_rng dnn_rng_seed(uint64_t seed) {
    dnn_rng r;
    r.s[0] = splitmix64(seed);
    r.s[1] = splitmix64(r.s[0]);
    return r;
}

float dnn_rng_uniform(dnn_rng *rng) {
    return (float)(next_u64(rng) >> 11) * 0x1.0p-53f;
}

float dnn_rng_normal(dnn_rng *rng) {
    float u1;
    do { u1 = dnn_rng_uniform(rng); } while (u1 == 0.0f);
    float u2 = dnn_rng_uniform(rng);
    return sqrtf(-2.0f * logf(u1)) * cosf(6.283185307179586f * u2);
}

int dnn_rng_uniform_int(dnn_rng *rng, int n) {
    if (n <= 1) return 0;
    uint32_t limit = (uint32_t)n, mask = limit;
    mask |= mask >> 1; mask |= mask >> 2; mask |= mask >> 4; mask |= mask >> 8; mask |= mask >> 16;
    uint32_t v;
    do { v = (uint32_t)(next_u64(rng) >> 32) & mask; } while (v >= limit);
    return (int)v;
}

dnn_rng *dnn_get_rng(void) { return &g_default_rng; }
void dnn_seed(uint64_t seed) { g_default_rng = dnn_rng_seed(seed); }

}  // extern "C"
