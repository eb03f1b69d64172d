// Encoder and decoder of the 2.0-bit format: four 2-bit codes per byte, weight = (code - 1.5) * scale with one
// fp16 rms scale per group of g consecutive weights (g a positive multiple of 8).
//
// Follows E8LatticePacker.pack / unpack (ojasx2/math/lattice.py:210-279) operation by operation in fp32: the
// scale as in the ternary encoder (eight lane accumulators of separately rounded squares, lanes added 0..7,
// sqrt, true division by sqrt(g), + 1e-8); every 8-block of x / scale is shifted by -1/2, rounded half-to-even
// and clamped to [-2, 1]; when the sum of an 8-block is odd, the coordinate whose move to its other neighbour
// (clamped as well) raises the squared error least - the first one on ties - is moved.  code = value + 2.
#pragma once

#include "codec.cuh"

namespace ojx {

// 16 bits of codes for eight consecutive values (kExactRcp: x / scale through the group's reciprocal, see codec.cuh).
template <bool kExactRcp>
__device__ __forceinline__ uint32_t encode2_block8(const float* x, float scale, float rcp) {
    uint32_t bits = 0;
    float sum = 0.f, best = 0.f;
    int best_step = 0;                                  // (alt - value) << (2 * index) of the cheapest move
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        float v;
        if (kExactRcp) {
            const float q0 = __fmul_rn(x[i], rcp);
            v = __fmaf_rn(__fmaf_rn(-scale, q0, x[i]), rcp, q0);
        } else {
            v = __fdiv_rn(x[i], scale);
        }
        const float xs = __fsub_rn(v, 0.5f);
        const float f = fminf(fmaxf(rintf(xs), -2.0f), 1.0f);
        const float alt = (xs >= f) ? fminf(f + 1.0f, 1.0f) : fmaxf(f - 1.0f, -2.0f);
        const float da = __fsub_rn(alt, xs), df = __fsub_rn(f, xs);
        const float pen = __fsub_rn(__fmul_rn(da, da), __fmul_rn(df, df));
        sum = __fadd_rn(sum, f);
        bits |= (uint32_t)((int)f + 2) << (2 * i);
        if (i == 0 || pen < best) { best = pen; best_step = (int)(alt - f) * (1 << (2 * i)); }
    }
    if (((int)sum) & 1) bits = (uint32_t)((int)bits + best_step);
    return bits & 0xFFFFu;
}

template <typename T, int GROUP>
__global__ void __launch_bounds__(128) encode2_kernel(const T* __restrict__ w, int64_t total, int group_rt, float sqrt_group,
                                                       uint8_t* __restrict__ packed, uint16_t* __restrict__ scales, int64_t ngroups) {
    const int group = GROUP > 0 ? GROUP : group_rt;
    for (int64_t gi = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; gi < ngroups; gi += (int64_t)gridDim.x * blockDim.x) {
        const int64_t base = gi * group;
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        float xr[GROUP > 0 ? GROUP : 8];
        if (GROUP > 0) {
            const bool vec = base + GROUP <= total && ((reinterpret_cast<uintptr_t>(w + base) & 15) == 0);
            if (vec) {
                constexpr int per = 16 / sizeof(T);
                const uint4* src = reinterpret_cast<const uint4*>(w + base);
#pragma unroll
                for (int c = 0; c < GROUP / per; ++c) {
                    const uint4 u = __ldg(src + c);
                    const T* e = reinterpret_cast<const T*>(&u);
#pragma unroll
                    for (int j = 0; j < per; ++j) xr[c * per + j] = to_f32<T>(e[j]);
                }
            } else {
#pragma unroll
                for (int i = 0; i < GROUP; ++i) xr[i] = (base + i < total) ? to_f32<T>(w[base + i]) : 0.f;
            }
#pragma unroll
            for (int d = 0; d < GROUP; d += 8)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] = __fadd_rn(acc[j], __fmul_rn(xr[d + j], xr[d + j]));
        } else {
            for (int d = 0; d < group; d += 8)
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float x = (base + d + j < total) ? to_f32<T>(w[base + d + j]) : 0.f;
                    acc[j] = __fadd_rn(acc[j], __fmul_rn(x, x));
                }
        }
        float s = acc[0];
#pragma unroll
        for (int j = 1; j < 8; ++j) s = __fadd_rn(s, acc[j]);
        const float scale = __fadd_rn(__fdiv_rn(__fsqrt_rn(s), sqrt_group), 1e-8f);
        scales[gi] = __half_as_ushort(__float2half_rn(scale));
        const bool fast = scale >= 1e-7f && scale <= 1e30f;
        const float rcp = fast ? __frcp_rn(scale) : 0.f;
        uint8_t* out = packed + gi * (int64_t)(group / 4);
        for (int b = 0; b < group; b += 8) {
            float t[8];
            if (GROUP > 0) {
#pragma unroll
                for (int i = 0; i < 8; ++i) t[i] = xr[(GROUP > 0 ? b : 0) + i];
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) t[i] = (base + b + i < total) ? to_f32<T>(w[base + b + i]) : 0.f;
            }
            const uint32_t bits = fast ? encode2_block8<true>(t, scale, rcp) : encode2_block8<false>(t, scale, rcp);
            out[b / 4] = (uint8_t)bits;
            out[b / 4 + 1] = (uint8_t)(bits >> 8);
        }
    }
}

template <typename T>
static int32_t encode2_typed(const void* w, int64_t total, int group, uint8_t* packed, uint16_t* scales, cudaStream_t s) {
    const int64_t ngroups = (total + group - 1) / group;
    const float sg = (float)sqrt((double)group);
    const int threads = 128;
    int64_t blocks = (ngroups + threads - 1) / threads;
    if (blocks > 148 * 64) blocks = 148 * 64;
    const T* wp = static_cast<const T*>(w);
    if (group == 8) encode2_kernel<T, 8><<<(unsigned)blocks, threads, 0, s>>>(wp, total, group, sg, packed, scales, ngroups);
    else if (group == 32) encode2_kernel<T, 32><<<(unsigned)blocks, threads, 0, s>>>(wp, total, group, sg, packed, scales, ngroups);
    else encode2_kernel<T, 0><<<(unsigned)blocks, threads, 0, s>>>(wp, total, group, sg, packed, scales, ngroups);
    return launch_status();
}

int32_t encode2_impl(const void* w, int w_dtype, int64_t rows, int64_t cols, int group, uint8_t* packed, uint16_t* scales,
                     cudaStream_t s) {
    OJX_RETURN_IF(!w || !packed || !scales, OJX_ERR_NULL);
    OJX_RETURN_IF(rows <= 0 || cols <= 0 || group <= 0 || group % 8 != 0, OJX_ERR_SHAPE);
    OJX_RETURN_IF(check_arch() != OJX_OK, OJX_ERR_ARCH);
    const int64_t total = rows * cols;
    switch (w_dtype) {
        case OJX_F32: return encode2_typed<float>(w, total, group, packed, scales, s);
        case OJX_F16: return encode2_typed<__half>(w, total, group, packed, scales, s);
        case OJX_BF16: return encode2_typed<__nv_bfloat16>(w, total, group, packed, scales, s);
        default: return OJX_ERR_DTYPE;
    }
}

// Decoder: one thread per 8 weights (two bytes of codes, one scale).
template <typename T>
__global__ void __launch_bounds__(256) decode2_kernel(const uint8_t* __restrict__ packed, const uint16_t* __restrict__ scales,
                                                       int64_t total, int group, T* __restrict__ out) {
    const int64_t blocks8 = (total + 7) / 8;
    for (int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; b < blocks8; b += (int64_t)gridDim.x * blockDim.x) {
        const uint32_t bits = (uint32_t)packed[2 * b] | ((uint32_t)packed[2 * b + 1] << 8);
        const float sc = decode_scale<T>(scales[(b * 8) / group]);
        T vals[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) vals[i] = from_f32<T>(__fmul_rn((float)((bits >> (2 * i)) & 3u) - 1.5f, sc));
        T* dst = out + b * 8;
        if (b * 8 + 8 <= total && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
            const uint4* v = reinterpret_cast<const uint4*>(vals);
#pragma unroll
            for (int c = 0; c < (int)(8 * sizeof(T) / 16); ++c) reinterpret_cast<uint4*>(dst)[c] = v[c];
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (b * 8 + i < total) dst[i] = vals[i];
        }
    }
}

template <typename T>
static int32_t decode2_typed(const uint8_t* packed, const uint16_t* scales, int64_t total, int group, void* out, cudaStream_t s) {
    const int64_t blocks8 = (total + 7) / 8;
    int64_t blocks = (blocks8 + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    decode2_kernel<T><<<(unsigned)blocks, 256, 0, s>>>(packed, scales, total, group, static_cast<T*>(out));
    return launch_status();
}

int32_t decode2_impl(const uint8_t* packed, const uint16_t* scales, int64_t rows, int64_t cols, int group, int out_dtype,
                     void* out, cudaStream_t s) {
    OJX_RETURN_IF(!packed || !scales || !out, OJX_ERR_NULL);
    OJX_RETURN_IF(rows <= 0 || cols <= 0 || group <= 0 || group % 8 != 0, OJX_ERR_SHAPE);
    OJX_RETURN_IF(check_arch() != OJX_OK, OJX_ERR_ARCH);
    const int64_t total = rows * cols;
    switch (out_dtype) {
        case OJX_F32: return decode2_typed<float>(packed, scales, total, group, out, s);
        case OJX_F16: return decode2_typed<__half>(packed, scales, total, group, out, s);
        case OJX_BF16: return decode2_typed<__nv_bfloat16>(packed, scales, total, group, out, s);
        default: return OJX_ERR_DTYPE;
    }
}

}  // namespace ojx
