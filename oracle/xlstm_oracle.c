/*
 * TEST INFRASTRUCTURE — CPU oracle for the xLSTM hot path (see xlstm_oracle_impl.h for
 * what it restates and its parity status: PARITY UNPINNED at the bit level).
 *
 * Builds one shared object exporting every function twice: <name>_f32 and <name>_f64.
 * Also exports the reference's seeded generator so its seeded problem instances can be
 * regenerated exactly.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define CAT_(a, b) a##b
#define CAT(a, b) CAT_(a, b)

#define REAL float
#define FN(name) CAT(name, _f32)
#define R_EXP expf
#define R_LOG logf
#define R_TANH tanhf
#define R_SQRT sqrtf
#define R_FABS fabsf
#define R_POW powf
#include "xlstm_oracle_impl.h"
#undef REAL
#undef FN
#undef R_EXP
#undef R_LOG
#undef R_TANH
#undef R_SQRT
#undef R_FABS
#undef R_POW

#define REAL double
#define FN(name) CAT(name, _f64)
#define R_EXP exp
#define R_LOG log
#define R_TANH tanh
#define R_SQRT sqrt
#define R_FABS fabs
#define R_POW pow
#include "xlstm_oracle_impl.h"

/* src/tensor/mod.rs:97-119 — SplitMix64, top 24 bits -> [0,1) -> [-scale, scale). */
void random_seeded_f32(float* out, size_t n, float scale, uint64_t seed) {
    uint64_t state = seed + 0x9E3779B97F4A7C15ull;
    for (size_t i = 0; i < n; ++i) {
        state += 0x9E3779B97F4A7C15ull;
        uint64_t z = state;
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        z ^= z >> 31;
        float u = (float)(z >> 40) / (float)(1u << 24);
        out[i] = (u * 2.0f - 1.0f) * scale;
    }
}
