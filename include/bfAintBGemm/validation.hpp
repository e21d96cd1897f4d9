// Result check of the host driver (interface of the reference's bfAintBGemm/validation.hpp:7-46: NRMS plus a
// per-element relative test, first mismatches printed).  Two things differ on purpose:
//   * the per-element error is |r - p| / max(|r|, floor); the reference divides by the signed r (:27), so it can
//     never flag an entry whose reference value is negative, and 0/0 gives NaN;
//   * the tolerances are parameters (the reference hard-codes 1e-3, which only its integer-valued test data meets).
#pragma once
#include <cmath>
#include <cstdint>
#include <cstdio>
#include "datatype.hpp"

#define PER_PIXEL_CHECK
#define ASSERT_ON_FAIL

template <typename T>
static inline bool valid_vector(const float* ref, const T* pred, int n, float nrms = 1e-3f, float rel_tol = 1e-2f, float floor_frac = 0.05f) {
    double sum_d2 = 0.0, sum_r2 = 0.0;
    for (int i = 0; i < n; ++i) {
        const double r = ref[i], p = type_convert<float, T>(pred[i]);
        sum_d2 += (r - p) * (r - p);
        sum_r2 += r * r;
    }
    const double rms = n > 0 ? std::sqrt(sum_r2 / n) : 0.0;
    const double floor_abs = rms * floor_frac > 1e-30 ? rms * floor_frac : 1e-30;
    int bad = 0;
    double worst = 0.0;
#ifdef PER_PIXEL_CHECK
    for (int i = 0; i < n; ++i) {
        const double r = ref[i], p = type_convert<float, T>(pred[i]);
        const double den = std::fabs(r) > floor_abs ? std::fabs(r) : floor_abs;
        const double rel = std::fabs(r - p) / den;
        if (rel > worst) worst = rel;
        if (!(rel <= rel_tol)) {
#ifdef ASSERT_ON_FAIL
            if (bad < 100) std::printf("diff at %4d, ref:%lf, pred:%lf(0x%04x), d:%lf\n", i, r, p, (unsigned)((const std::uint16_t*)pred)[i], rel);
#endif
            ++bad;
        }
    }
#endif
    const double got_nrms = sum_r2 > 0 ? std::sqrt(sum_d2 / (2.0 * sum_r2)) : (sum_d2 > 0 ? 1e30 : 0.0);
    std::printf("pp_crr:%d, pp_err:%d, crr_ratio:%.3f, nrms:%lf, max_rel:%lf, s0:%lf, s1:%lf\n", n - bad, bad,
                n ? (float)(n - bad) / (float)n : 1.f, got_nrms, worst, sum_d2, 2.0 * sum_r2);
    return got_nrms < nrms && bad == 0;
}
