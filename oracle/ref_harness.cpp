// C-callable shim around the REFERENCE's own native header kernels.
//
// TEST INFRASTRUCTURE ONLY.  This translation unit contains no arithmetic of
// its own: it includes the reference project's header
// `ojasx2/math/csrc/ojasx_math_core.hpp` from where the reference checkout
// lies (include path given by the Makefile) and forwards to
//   ojasx::math::lattice::fused_ternary_e8_gemm_forward<float>   (:580-634)
//   ojasx::math::lattice::get_ternary_rank_to_coords             (:549-573)
// The built library lands in oracle/_ref/ (git-ignored).  It validates the C
// restatement in e8t_oracle.c and serves as the timed "reference" CPU baseline.
// Threading mirrors the reference's ATen wrapper, which parallelises over the
// rows of x only (ojasx_math_bindings.cpp:454-468).
#include "ojasx_math_core.hpp"

#include <cstdint>
#include <thread>
#include <vector>

extern "C" {

const int8_t* ojx_ref_rank_to_coords() {
    return ojasx::math::lattice::get_ternary_rank_to_coords();
}

void ojx_ref_ternary_forward(const float* x, const uint8_t* packed, const float* scales,
                             const float* bias, float* y, int64_t M, int64_t K, int64_t N,
                             int64_t group, int threads) {
    using ojasx::math::lattice::fused_ternary_e8_gemm_forward;
    if (threads <= 1 || M <= 1) {
        fused_ternary_e8_gemm_forward<float>(x, packed, scales, bias, y,
                                             (size_t)M, (size_t)K, (size_t)N, (size_t)group);
        return;
    }
    int nt = threads < M ? threads : (int)M;
    std::vector<std::thread> pool;
    for (int t = 0; t < nt; ++t) {
        int64_t m0 = M * t / nt, m1 = M * (t + 1) / nt;
        pool.emplace_back([=] {
            fused_ternary_e8_gemm_forward<float>(x + m0 * K, packed, scales, bias, y + m0 * N,
                                                 (size_t)(m1 - m0), (size_t)K, (size_t)N, (size_t)group);
        });
    }
    for (auto& th : pool) th.join();
}

}  // extern "C"
