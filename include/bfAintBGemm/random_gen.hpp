// Host-side fills of the fp32 master copies.
// The four rand_vector_2d* functions keep the names, arguments and value sets of the reference's
// bfAintBGemm/random_gen.hpp:5-66 (uniform floats; integers in {-2,-1,0,1}).  The reference seeds std::rand from
// the clock, so its runs cannot be repeated; here the generator is a counter-based hash seeded by rand_seed()
// (default seed 0), and seeded fills with the distributions of the benchmark configurations are added.
#pragma once
#include <cmath>
#include <cstddef>
#include <cstdint>

namespace afb_rng {
inline std::uint64_t& seed_ref() { static std::uint64_t s = 0; return s; }
inline std::uint64_t mix(std::uint64_t z) {  // splitmix64 finaliser
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
// Value of stream `tensor` at position `idx`: any element can be recomputed on its own.
inline std::uint64_t at(std::uint64_t tensor, std::uint64_t idx) { return mix(mix(seed_ref() ^ (tensor << 56)) + idx); }
inline float unit(std::uint64_t h) { return static_cast<float>(h >> 40) * (1.0f / 16777216.0f); }  // [0,1)
}  // namespace afb_rng

inline void rand_seed(std::uint64_t seed) { afb_rng::seed_ref() = seed; }

static inline void rand_vector_2d(float* v, int row, int col, int ld, float min_v = 0, float max_v = 1) {
    for (int r = 0; r < row; ++r)
        for (int c = 0; c < col; ++c) v[(std::size_t)r * ld + c] = min_v + afb_rng::unit(afb_rng::at(0, (std::uint64_t)r * col + c)) * (max_v - min_v);
}
namespace afb_rng {
inline void fill_small_int(float* v, int row, int col, int ld, std::uint64_t tensor) {  // integers in {-2,-1,0,1}
    for (int r = 0; r < row; ++r)
        for (int c = 0; c < col; ++c) v[(std::size_t)r * ld + c] = static_cast<float>(static_cast<int>(at(tensor, (std::uint64_t)r * col + c) & 3u) - 2);
}
}  // namespace afb_rng
static inline void rand_vector_2d_int_a(float* v, int row, int col, int ld) { afb_rng::fill_small_int(v, row, col, ld, 1); }
static inline void rand_vector_2d_int_b(float* v, int row, int col, int ld) { afb_rng::fill_small_int(v, row, col, ld, 2); }
static inline void rand_vector_2d_int_scale(float* v, int row, int col, int ld) { afb_rng::fill_small_int(v, row, col, ld, 3); }
static inline void rand_vector_2d_int(float* v, int row, int col, int ld) {
    for (int r = 0; r < row; ++r)
        for (int c = 0; c < col; ++c) v[(std::size_t)r * ld + c] = static_cast<float>(c % 3 + 1);
}

// ---- distributions of the benchmark configurations ----
static inline void rand_vector_2d_normal(float* v, int row, int col, int ld, std::uint64_t tensor = 1) {  // N(0,1), Box-Muller
    for (int r = 0; r < row; ++r)
        for (int c = 0; c < col; ++c) {
            const std::uint64_t i = (std::uint64_t)r * col + c;
            const float u1 = 1.0f - afb_rng::unit(afb_rng::at(tensor, 2 * i)), u2 = afb_rng::unit(afb_rng::at(tensor, 2 * i + 1));
            v[(std::size_t)r * ld + c] = std::sqrt(-2.0f * std::log(u1)) * std::cos(6.28318530718f * u2);
        }
}
static inline void rand_vector_2d_uniform(float* v, int row, int col, int ld, float lo, float hi, std::uint64_t tensor = 3) {
    for (int r = 0; r < row; ++r)
        for (int c = 0; c < col; ++c) v[(std::size_t)r * ld + c] = lo + afb_rng::unit(afb_rng::at(tensor, (std::uint64_t)r * col + c)) * (hi - lo);
}
static inline void rand_vector_2d_int_range(float* v, int row, int col, int ld, int lo, int hi, std::uint64_t tensor = 2) {  // integers in [lo,hi]
    const std::uint64_t span = (std::uint64_t)(hi - lo + 1);
    for (int r = 0; r < row; ++r)
        for (int c = 0; c < col; ++c) v[(std::size_t)r * ld + c] = static_cast<float>(lo + static_cast<int>(afb_rng::at(tensor, (std::uint64_t)r * col + c) % span));
}
