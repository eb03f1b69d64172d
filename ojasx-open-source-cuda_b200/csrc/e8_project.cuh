// Nearest point of the E8 lattice (Conway-Sloane decoder) for every 8-vector, and the forward of the
// straight-through quantizer built on it.  fp32, one thread per 8-vector, 32 bytes in and 32 bytes out.
//
// Follows conway_sloane_e8_project and _E8STEFunction.forward (ojasx2/math/lattice.py:162-203, 853-867)
// operation by operation as torch evaluates them on fp32 tensors: round-half-even, squared distances and
// squared norms summed left to right with every partial result rounded, true divisions, no fused
// multiply-adds, the first index wins an argmax tie, sign(0) counts as +1, the integer candidate wins a
// distance tie.
#pragma once

#include "common.cuh"

namespace ojx {

// Nearest point of D8 (integer vectors with an even coordinate sum): round, and when the sum is odd move the
// coordinate with the largest rounding error one step towards the input.
__device__ __forceinline__ void d8_nearest(const float (&v)[8], float (&c)[8]) {
    float sum = 0.f, worst_err = -1.f, worst_diff = 0.f;
    int worst = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float f = rintf(v[i]);
        c[i] = f;
        sum = __fadd_rn(sum, f);
        const float d = __fsub_rn(v[i], f);
        if (fabsf(d) > worst_err) { worst_err = fabsf(d); worst = i; worst_diff = d; }
    }
    if (((long long)sum) & 1LL) {
        const float step = worst_diff < 0.f ? -1.f : 1.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) c[i] = (i == worst) ? __fadd_rn(c[i], step) : c[i];
    }
}

__device__ __forceinline__ void e8_nearest(const float (&v)[8], float (&out)[8]) {
    float c1[8], c2[8], vs[8];
    d8_nearest(v, c1);
#pragma unroll
    for (int i = 0; i < 8; ++i) vs[i] = __fsub_rn(v[i], 0.5f);
    d8_nearest(vs, c2);
    float d1 = 0.f, d2 = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        c2[i] = __fadd_rn(c2[i], 0.5f);
        const float e1 = __fsub_rn(v[i], c1[i]), e2 = __fsub_rn(v[i], c2[i]);
        d1 = __fadd_rn(d1, __fmul_rn(e1, e1));
        d2 = __fadd_rn(d2, __fmul_rn(e2, e2));
    }
    const bool first = d1 <= d2;
#pragma unroll
    for (int i = 0; i < 8; ++i) out[i] = first ? c1[i] : c2[i];
}

// kSte: divide the group by rms + 1e-8 before the projection and multiply back after it.
template <bool kSte>
__global__ void __launch_bounds__(256) e8_project_kernel(const float* __restrict__ x, float* __restrict__ out, int64_t total) {
    const int64_t groups = (total + 7) / 8;
    for (int64_t gi = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; gi < groups; gi += (int64_t)gridDim.x * blockDim.x) {
        const int64_t base = gi * 8;
        const bool full = base + 8 <= total;
        float v[8];
        if (full) {
            const float4 a = __ldg(reinterpret_cast<const float4*>(x + base)), b = __ldg(reinterpret_cast<const float4*>(x + base) + 1);
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = base + i < total ? x[base + i] : 0.f;
        }
        float scale = 1.f;
        if constexpr (kSte) {
            float s = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) s = __fadd_rn(s, __fmul_rn(v[i], v[i]));
            scale = __fadd_rn(__fdiv_rn(__fsqrt_rn(s), 2.8284271247461903f), 1e-8f);
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = __fdiv_rn(v[i], scale);
        }
        float q[8];
        e8_nearest(v, q);
        if constexpr (kSte) {
#pragma unroll
            for (int i = 0; i < 8; ++i) q[i] = __fmul_rn(q[i], scale);
        }
        if (full) {
            reinterpret_cast<float4*>(out + base)[0] = make_float4(q[0], q[1], q[2], q[3]);
            reinterpret_cast<float4*>(out + base)[1] = make_float4(q[4], q[5], q[6], q[7]);
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (base + i < total) out[base + i] = q[i];
        }
    }
}

int32_t e8_project_impl(const float* x, int64_t count, float* out, bool ste, cudaStream_t s) {
    OJX_RETURN_IF(!x || !out, OJX_ERR_NULL);
    OJX_RETURN_IF(count <= 0 || (!ste && count % 8 != 0), OJX_ERR_SHAPE);
    OJX_RETURN_IF(((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15) != 0, OJX_ERR_ALIGN);
    OJX_RETURN_IF(check_arch() != OJX_OK, OJX_ERR_ARCH);
    const int64_t groups = (count + 7) / 8;
    int64_t blocks = (groups + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    if (ste) e8_project_kernel<true><<<(unsigned)blocks, 256, 0, s>>>(x, out, count);
    else e8_project_kernel<false><<<(unsigned)blocks, 256, 0, s>>>(x, out, count);
    return launch_status();
}

}  // namespace ojx
