// Counter-based synthetic values: element `index` of matrix `matrix_id` under `seed`.
// The same arithmetic is restated in numpy (rng.py of the package) and in C (the oracle), so any
// element can be recomputed in isolation on either side.
#pragma once

#include <stdint.h>

namespace b200 {

__host__ __device__ inline uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

// dist 0: uniform[-1, 1) on a 2^-23 grid; dist 1: normal(0, 1) by Box-Muller evaluated in double
// (so that host and device agree after rounding to float); dist 2: zero.
__host__ __device__ inline float synth_value(uint64_t seed, uint64_t matrix_id, uint64_t index, int dist) {
    const uint64_t u = splitmix64(seed * 0x9E3779B97F4A7C15ull + matrix_id * 0xD1B54A32D192ED03ull + index);
    if (dist == 0) return static_cast<float>(static_cast<double>(u >> 40) * (1.0 / 8388608.0) - 1.0);
    if (dist == 1) {
        const double u1 = (static_cast<double>(u >> 40) + 1.0) * (1.0 / 16777216.0);           // (0, 1]
        const double u2 = static_cast<double>((u >> 16) & 0xFFFFFFull) * (1.0 / 16777216.0);  // [0, 1)
        return static_cast<float>(sqrt(-2.0 * log(u1)) * cos(6.283185307179586476925 * u2));
    }
    return 0.0f;
}

}  // namespace b200
