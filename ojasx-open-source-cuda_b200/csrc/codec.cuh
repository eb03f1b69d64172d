// Encoder, decoder and seeded generator kernels for the ternary-E8 format.
//
// Encoder arithmetic follows TernaryE8LatticePacker.pack (ojasx2/math/lattice.py:338-384)
// operation by operation; every float operation is an explicit round-to-nearest
// intrinsic so the compiler cannot contract a multiply and an add into an FMA.
#pragma once

#include "common.cuh"

namespace ojx {

// ---------------------------------------------------------------------------------------------
// Encoder: one thread per scale group.
// ---------------------------------------------------------------------------------------------

// Code of eight consecutive values given the unrounded fp32 group scale.
__device__ __forceinline__ uint32_t encode_block8(const float* x, float scale) {
    float v[8], q[8], alt[8];
    int sum = 0;
    float best = 0.f;
    int worst = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        v[i] = __fdiv_rn(x[i], scale);
        float r = rintf(v[i]);
        q[i] = fminf(fmaxf(r, -1.0f), 1.0f);
        sum += (int)q[i];
        alt[i] = (q[i] == 0.0f) ? (v[i] >= 0.0f ? 1.0f : -1.0f) : 0.0f;
        float da = __fsub_rn(alt[i], v[i]);
        float dq = __fsub_rn(q[i], v[i]);
        float pen = __fsub_rn(__fmul_rn(da, da), __fmul_rn(dq, dq));
        if (i == 0 || pen < best) { best = pen; worst = i; }   // first index wins ties
    }
    const bool odd = (sum & 1) != 0;
    uint32_t raw = 0, p3 = 1;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        float qi = (odd && i == worst) ? alt[i] : q[i];
        raw += (uint32_t)((int)qi + 1) * p3;
        p3 *= 3;
    }
    return g_raw_to_rank[raw];
}

template <typename T, int GROUP>
__global__ void __launch_bounds__(128) encode_kernel(const T* __restrict__ w, int64_t total, int group_rt,
                                                      float sqrt_group, uint8_t* __restrict__ packed,
                                                      uint16_t* __restrict__ scales, int64_t ngroups) {
    const int group = GROUP > 0 ? GROUP : group_rt;
    for (int64_t gi = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; gi < ngroups;
         gi += (int64_t)gridDim.x * blockDim.x) {
        const int64_t base = gi * group;
        // Sum of squares in the order torch.norm uses on a contiguous last dimension: eight lane
        // accumulators, products rounded on their own, lanes added 0..7.
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        float xr[GROUP > 0 ? GROUP : 8];
        if (GROUP > 0) {
            const bool full = base + GROUP <= total;
            const bool vec = full && ((reinterpret_cast<uintptr_t>(w + base) & 15) == 0);
            if (vec) {
                constexpr int per = 16 / sizeof(T);
                const uint4* src = reinterpret_cast<const uint4*>(w + base);
#pragma unroll
                for (int c = 0; c < GROUP / per; ++c) {
                    uint4 u = __ldg(src + c);
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
                    float x = (base + d + j < total) ? to_f32<T>(w[base + d + j]) : 0.f;
                    acc[j] = __fadd_rn(acc[j], __fmul_rn(x, x));
                }
        }
        float s = acc[0];
#pragma unroll
        for (int j = 1; j < 8; ++j) s = __fadd_rn(s, acc[j]);
        const float scale = __fadd_rn(__fdiv_rn(__fsqrt_rn(s), sqrt_group), 1e-8f);
        scales[gi] = __half_as_ushort(__float2half_rn(scale));

        uint8_t* out = packed + gi * (int64_t)(group / 16) * 3;
#pragma unroll
        for (int b = 0; b < group; b += 16) {
            uint32_t c[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                if (GROUP > 0) {
                    c[h] = encode_block8(&xr[(GROUP > 0 ? b : 0) + h * 8], scale);
                } else {
                    float t[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        int64_t idx = base + b + h * 8 + i;
                        t[i] = idx < total ? to_f32<T>(w[idx]) : 0.f;
                    }
                    c[h] = encode_block8(t, scale);
                }
            }
            out[0] = (uint8_t)(c[0] & 0xFF);
            out[1] = (uint8_t)(((c[0] >> 8) & 0x0F) | ((c[1] & 0x0F) << 4));
            out[2] = (uint8_t)((c[1] >> 4) & 0xFF);
            out += 3;
        }
    }
}

template <typename T>
static int32_t encode_typed(const void* w, int64_t total, int group, uint8_t* packed, uint16_t* scales,
                            cudaStream_t s) {
    const int64_t ngroups = (total + group - 1) / group;
    const float sg = (float)sqrt((double)group);
    const int threads = 128;
    int64_t blocks = (ngroups + threads - 1) / threads;
    if (blocks > 148 * 64) blocks = 148 * 64;
    if (blocks < 1) blocks = 1;
    const T* wp = static_cast<const T*>(w);
    if (group == 32)
        encode_kernel<T, 32><<<(unsigned)blocks, threads, 0, s>>>(wp, total, group, sg, packed, scales, ngroups);
    else
        encode_kernel<T, 0><<<(unsigned)blocks, threads, 0, s>>>(wp, total, group, sg, packed, scales, ngroups);
    return launch_status();
}

int32_t encode_impl(const void* w, int w_dtype, int64_t rows, int64_t cols, int group,
                    uint8_t* packed, uint16_t* scales, cudaStream_t s) {
    OJX_RETURN_IF(!w || !packed || !scales, OJX_ERR_NULL);
    OJX_RETURN_IF(rows <= 0 || cols <= 0, OJX_ERR_SHAPE);
    OJX_RETURN_IF(check_arch() != OJX_OK, OJX_ERR_ARCH);
    group = effective_group(group);
    const int64_t total = rows * cols;
    switch (w_dtype) {
        case OJX_F32: return encode_typed<float>(w, total, group, packed, scales, s);
        case OJX_F16: return encode_typed<__half>(w, total, group, packed, scales, s);
        case OJX_BF16: return encode_typed<__nv_bfloat16>(w, total, group, packed, scales, s);
        default: return OJX_ERR_DTYPE;
    }
}

// ---------------------------------------------------------------------------------------------
// Decoder: one thread per 3-byte triplet (16 weights).
// ---------------------------------------------------------------------------------------------

template <typename T> __device__ __forceinline__ float decode_scale(uint16_t bits);
template <> __device__ __forceinline__ float decode_scale<float>(uint16_t b) { return __half2float(__ushort_as_half(b)); }
template <> __device__ __forceinline__ float decode_scale<__half>(uint16_t b) { return __half2float(__ushort_as_half(b)); }
// The reference casts the fp16 scale to the output dtype before multiplying (lattice.py:418).
template <> __device__ __forceinline__ float decode_scale<__nv_bfloat16>(uint16_t b) {
    return __bfloat162float(__float2bfloat16_rn(__half2float(__ushort_as_half(b))));
}

template <typename T>
__global__ void __launch_bounds__(256) decode_kernel(const uint8_t* __restrict__ packed,
                                                      const uint16_t* __restrict__ scales, int64_t total,
                                                      int group, T* __restrict__ out) {
    __shared__ uint32_t lut[kNumPoints];
    for (int i = threadIdx.x; i < kNumPoints; i += blockDim.x) lut[i] = g_trit_nibbles[i];
    __syncthreads();
    const int64_t ntrip = (total + 15) / 16;
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < ntrip;
         t += (int64_t)gridDim.x * blockDim.x) {
        const uint8_t* p = packed + t * 3;
        uint32_t c0, c1;
        triplet_to_codes(p[0], p[1], p[2], c0, c1);
        c0 = min(c0, (uint32_t)(kNumPoints - 1));     // corrupt input must not read outside the table
        c1 = min(c1, (uint32_t)(kNumPoints - 1));
        const int64_t base = t * 16;
        const float sc = decode_scale<T>(scales[base / group]);
        const uint32_t n0 = lut[c0], n1 = lut[c1];
        __align__(16) T vals[16];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            vals[i] = from_f32<T>((float)nibble_coord(n0, i) * sc);
            vals[8 + i] = from_f32<T>((float)nibble_coord(n1, i) * sc);
        }
        if (base + 16 <= total && ((reinterpret_cast<uintptr_t>(out + base) & 15) == 0)) {
            uint4* dst = reinterpret_cast<uint4*>(out + base);
            const uint4* src = reinterpret_cast<const uint4*>(vals);
#pragma unroll
            for (int i = 0; i < (int)(16 * sizeof(T) / 16); ++i) dst[i] = src[i];
        } else {
            for (int i = 0; i < 16; ++i)
                if (base + i < total) out[base + i] = vals[i];
        }
    }
}

int32_t decode_impl(const uint8_t* packed, const uint16_t* scales, int64_t rows, int64_t cols,
                    int group, int out_dtype, void* out, cudaStream_t s) {
    OJX_RETURN_IF(!packed || !scales || !out, OJX_ERR_NULL);
    OJX_RETURN_IF(rows <= 0 || cols <= 0, OJX_ERR_SHAPE);
    OJX_RETURN_IF(check_arch() != OJX_OK, OJX_ERR_ARCH);
    group = effective_group(group);
    const int64_t total = rows * cols;
    const int64_t ntrip = (total + 15) / 16;
    int64_t blocks = (ntrip + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    switch (out_dtype) {
        case OJX_F32:
            decode_kernel<float><<<(unsigned)blocks, 256, 0, s>>>(packed, scales, total, group, (float*)out);
            break;
        case OJX_F16:
            decode_kernel<__half><<<(unsigned)blocks, 256, 0, s>>>(packed, scales, total, group, (__half*)out);
            break;
        case OJX_BF16:
            decode_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, s>>>(packed, scales, total, group,
                                                                          (__nv_bfloat16*)out);
            break;
        default: return OJX_ERR_DTYPE;
    }
    return launch_status();
}

// ---------------------------------------------------------------------------------------------
// Seeded generator (integer-exact Irwin-Hall over splitmix64).
// ---------------------------------------------------------------------------------------------

__device__ __forceinline__ uint64_t mix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

template <typename T>
__global__ void __launch_bounds__(256) generate_kernel(T* __restrict__ out, int64_t count, uint64_t base,
                                                        int64_t start, float sigma) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count;
         i += (int64_t)gridDim.x * blockDim.x) {
        const uint64_t e = (uint64_t)(start + i);
        int64_t sum = 0;
#pragma unroll
        for (int j = 0; j < 6; ++j) {
            uint64_t h = mix64(base + e * 6ull + (uint64_t)j);
            sum += (int64_t)(h & 0xFFFFFFull) + (int64_t)((h >> 32) & 0xFFFFFFull);
        }
        sum -= 6ll * (1ll << 24);
        const float x = __fmul_rn((float)sum, 5.9604644775390625e-08f);   // exact: |sum| < 2^27, times 2^-24
        out[i] = from_f32<T>(__fmul_rn(x, sigma));
    }
}

int32_t generate_impl(void* out, int dtype, int64_t count, uint64_t seed, int64_t start, float sigma,
                      cudaStream_t s) {
    OJX_RETURN_IF(!out, OJX_ERR_NULL);
    OJX_RETURN_IF(count <= 0 || start < 0, OJX_ERR_SHAPE);
    OJX_RETURN_IF(check_arch() != OJX_OK, OJX_ERR_ARCH);
    const uint64_t base = seed * 0xD1342543DE82EF95ull;
    int64_t blocks = (count + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    switch (dtype) {
        case OJX_F32: generate_kernel<float><<<(unsigned)blocks, 256, 0, s>>>((float*)out, count, base, start, sigma); break;
        case OJX_F16: generate_kernel<__half><<<(unsigned)blocks, 256, 0, s>>>((__half*)out, count, base, start, sigma); break;
        case OJX_BF16: generate_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, s>>>((__nv_bfloat16*)out, count, base, start, sigma); break;
        default: return OJX_ERR_DTYPE;
    }
    return launch_status();
}

}  // namespace ojx
