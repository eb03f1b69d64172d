// Encoder, decoder and seeded generator kernels for the ternary-E8 format.
//
// Encoder arithmetic follows TernaryE8LatticePacker.pack (ojasx2/math/lattice.py:338-384)
// operation by operation; every float operation is an explicit round-to-nearest
// intrinsic so the compiler cannot contract a multiply and an add into an FMA.
#pragma once

#include "common.cuh"
#include "fwht.cuh"

namespace ojx {

// ---------------------------------------------------------------------------------------------
// Encoder: one thread per scale group.
//
// Facts the kernels rely on (all checked by the bit-exact tests against the reference's output):
//   * a ternary vector is valid when its coordinate sum is even, i.e. when raw = sum (q_i + 1) 3^i is even,
//     so the rank of a valid raw value (its position among the valid ones) is raw / 2: no table;
//   * clamp(rint(v), -1, 1) and the "other candidate" alt_i share one sign t = (v >= 0 ? +1 : -1): for
//     q = 0 the candidate is t and the penalty (t - v)^2 - v^2; for q = +-1 (= t) the candidate is 0 and the
//     penalty is the exact negation v^2 - (t - v)^2 - every operation rounded as the reference rounds it;
//   * x / scale, correctly rounded, equals fma(fma(-scale, q0, x), r, q0) with r = RN(1 / scale) and
//     q0 = RN(x r) (one reciprocal per group instead of a division per weight); groups whose scale is
//     outside [1e-7, 1e30] (all-zero groups, overflowing inputs) take true divisions.
// ---------------------------------------------------------------------------------------------

struct Block8 {
    float rawf;        // sum q_i 3^i               (exact: |.| <= 3280)
    float sumq;        // sum q_i                   (exact)
    float best;        // smallest penalty so far
    float delta;       // (alt - q) 3^i of that coordinate
};

// One coordinate of an 8-block.  kFirst: coordinate 0 (takes the penalty unconditionally: first index wins ties).
template <bool kFirst>
__device__ __forceinline__ void encode_coord(Block8& b, float v, float p3) {
    const float q = fminf(fmaxf(rintf(v), -1.0f), 1.0f);
    const float t = (v >= 0.0f) ? 1.0f : -1.0f;
    const float a = __fsub_rn(t, v);
    const float pen0 = __fsub_rn(__fmul_rn(a, a), __fmul_rn(v, v));
    const bool qz = (q == 0.0f);
    const float pen = qz ? pen0 : -pen0;
    const float dsel = qz ? t : -t;                    // alt - q
    b.rawf = __fmaf_rn(q, p3, b.rawf);
    b.sumq = __fadd_rn(b.sumq, q);
    if (kFirst || pen < b.best) { b.best = pen; b.delta = __fmul_rn(dsel, p3); }
}

__device__ __forceinline__ uint32_t block8_rank(const Block8& b) {
    const int odd = ((int)b.sumq) & 1;
    const float raw = __fadd_rn(__fadd_rn(b.rawf, 3280.0f), odd ? b.delta : 0.0f);     // sum (q_i + 1) 3^i
    return (uint32_t)((int)raw >> 1);
}

// Code of eight consecutive values given the unrounded fp32 group scale (true divisions).
__device__ __forceinline__ uint32_t encode_block8(const float* x, float scale) {
    Block8 b = {0.f, 0.f, 0.f, 0.f};
    float p3 = 1.0f;
    encode_coord<true>(b, __fdiv_rn(x[0], scale), p3);
#pragma unroll
    for (int i = 1; i < 8; ++i) {
        p3 *= 3.0f;
        encode_coord<false>(b, __fdiv_rn(x[i], scale), p3);
    }
    return block8_rank(b);
}

// Same, with the group's reciprocal: two fused multiply-adds per quotient.
__device__ __forceinline__ uint32_t encode_block8_rcp(const float* x, float scale, float rcp) {
    Block8 b = {0.f, 0.f, 0.f, 0.f};
    float p3 = 1.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float q0 = __fmul_rn(x[i], rcp);
        const float v = __fmaf_rn(__fmaf_rn(-scale, q0, x[i]), rcp, q0);
        if (i == 0) encode_coord<true>(b, v, p3);
        else encode_coord<false>(b, v, p3);
        p3 *= 3.0f;
    }
    return block8_rank(b);
}

// kHad: the group is first rotated by the 32-point Walsh-Hadamard transform in T's arithmetic (what
// _pack_row_block / E8LatticeLinear.from_linear do with use_hadamard, ojasx2/streaming_e8.py:112-125), in registers.
template <typename T, int GROUP, bool kHad = false>
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
            if constexpr (kHad && GROUP == 32) fwht32_values<T>(xr);
#pragma unroll
            for (int d = 0; d < GROUP; d += 8)
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    // the square of a 16-bit float is exact in fp32, so one fused multiply-add rounds exactly
                    // like the reference's separately rounded product and sum
                    if (sizeof(T) == 2) acc[j] = __fmaf_rn(xr[d + j], xr[d + j], acc[j]);
                    else acc[j] = __fadd_rn(acc[j], __fmul_rn(xr[d + j], xr[d + j]));
                }
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
        if (GROUP == 32) {
            uint32_t c[4];
            if (scale >= 1e-7f && scale <= 1e30f) {
                const float rcp = __frcp_rn(scale);
#pragma unroll
                for (int h = 0; h < 4; ++h) c[h] = encode_block8_rcp(&xr[h * 8], scale, rcp);
            } else {
#pragma unroll
                for (int h = 0; h < 4; ++h) c[h] = encode_block8(&xr[h * 8], scale);
            }
            // six bytes per group: two triplets b0 = c0 & 0xFF, b1 = (c0 >> 8) | ((c1 & 0xF) << 4), b2 = c1 >> 4
            const uint32_t h0 = (c[0] | (c[1] << 12)) & 0xFFFFu, h1 = ((c[1] >> 4) | (c[2] << 8)) & 0xFFFFu,
                           h2 = ((c[2] >> 8) | (c[3] << 4)) & 0xFFFFu;
            if ((reinterpret_cast<uintptr_t>(out) & 1) == 0) {
                uint16_t* o16 = reinterpret_cast<uint16_t*>(out);
                o16[0] = (uint16_t)h0; o16[1] = (uint16_t)h1; o16[2] = (uint16_t)h2;
            } else {
                out[0] = (uint8_t)h0; out[1] = (uint8_t)(h0 >> 8); out[2] = (uint8_t)h1;
                out[3] = (uint8_t)(h1 >> 8); out[4] = (uint8_t)h2; out[5] = (uint8_t)(h2 >> 8);
            }
        } else {
#pragma unroll
        for (int b = 0; b < group; b += 16) {
            uint32_t c[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                float t[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    int64_t idx = base + b + h * 8 + i;
                    t[i] = idx < total ? to_f32<T>(w[idx]) : 0.f;
                }
                c[h] = encode_block8(t, scale);
            }
            out[0] = (uint8_t)(c[0] & 0xFF);
            out[1] = (uint8_t)(((c[0] >> 8) & 0x0F) | ((c[1] & 0x0F) << 4));
            out[2] = (uint8_t)((c[1] >> 4) & 0xFF);
            out += 3;
        }
        }
    }
}

template <typename T>
static int32_t encode_typed(const void* w, int64_t total, int group, bool hadamard, uint8_t* packed,
                            uint16_t* scales, cudaStream_t s) {
    const int64_t ngroups = (total + group - 1) / group;
    const float sg = (float)sqrt((double)group);
    const int threads = 128;
    int64_t blocks = (ngroups + threads - 1) / threads;
    if (blocks > 148 * 64) blocks = 148 * 64;
    if (blocks < 1) blocks = 1;
    const T* wp = static_cast<const T*>(w);
    if (hadamard)
        encode_kernel<T, 32, true><<<(unsigned)blocks, threads, 0, s>>>(wp, total, group, sg, packed, scales, ngroups);
    else if (group == 32)
        encode_kernel<T, 32><<<(unsigned)blocks, threads, 0, s>>>(wp, total, group, sg, packed, scales, ngroups);
    else
        encode_kernel<T, 0><<<(unsigned)blocks, threads, 0, s>>>(wp, total, group, sg, packed, scales, ngroups);
    return launch_status();
}

int32_t encode_impl(const void* w, int w_dtype, int64_t rows, int64_t cols, int group, uint32_t flags,
                    uint8_t* packed, uint16_t* scales, cudaStream_t s) {
    OJX_RETURN_IF(!w || !packed || !scales, OJX_ERR_NULL);
    OJX_RETURN_IF(rows <= 0 || cols <= 0, OJX_ERR_SHAPE);
    OJX_RETURN_IF(check_arch() != OJX_OK, OJX_ERR_ARCH);
    group = effective_group(group);
    OJX_RETURN_IF((flags & ~(uint32_t)OJX_ENCODE_HADAMARD) != 0, OJX_ERR_UNSUPPORTED);
    const bool had = (flags & OJX_ENCODE_HADAMARD) != 0;
    OJX_RETURN_IF(had && (group != 32 || cols % 32 != 0), OJX_ERR_SHAPE);
    const int64_t total = rows * cols;
    switch (w_dtype) {
        case OJX_F32: return encode_typed<float>(w, total, group, had, packed, scales, s);
        case OJX_F16: return encode_typed<__half>(w, total, group, had, packed, scales, s);
        case OJX_BF16: return encode_typed<__nv_bfloat16>(w, total, group, had, packed, scales, s);
        default: return OJX_ERR_DTYPE;
    }
}

// ---------------------------------------------------------------------------------------------
// Decoder: one thread per 3-byte triplet (16 weights, 32 or 64 bytes of output).
// ---------------------------------------------------------------------------------------------

template <typename T> __device__ __forceinline__ float decode_scale(uint16_t bits);
template <> __device__ __forceinline__ float decode_scale<float>(uint16_t b) { return __half2float(__ushort_as_half(b)); }
template <> __device__ __forceinline__ float decode_scale<__half>(uint16_t b) { return __half2float(__ushort_as_half(b)); }
// The reference casts the fp16 scale to the output dtype before multiplying (lattice.py:418).
template <> __device__ __forceinline__ float decode_scale<__nv_bfloat16>(uint16_t b) {
    return __bfloat162float(__float2bfloat16_rn(__half2float(__ushort_as_half(b))));
}

// Bit pattern of the scale in the output's 16-bit type (fp32 output goes through fp16, which holds coord * scale exactly).
template <typename T> __device__ __forceinline__ uint32_t decode_scale_bits(uint16_t b) { return b; }
template <> __device__ __forceinline__ uint32_t decode_scale_bits<__nv_bfloat16>(uint16_t b) {
    return __bfloat16_as_ushort(__float2bfloat16_rn(__half2float(__ushort_as_half(b))));
}

// A weight is 0, +scale or -scale, so its 16-bit pattern is assembled from the bytes of the scale with byte permutes
// (two weights per permute; selectors from the table the GEMV uses) instead of being computed: about seven
// instructions per weight became about three, which leaves the kernel to the memory system.  Two variants that were
// measured and lost (145 and 137 us against 132 us for 28672 x 8192 to fp16): one 16-byte output chunk per lane, so
// that every store instruction writes whole 32-byte sectors, and the same with four chunks in flight per thread.
template <typename T>
__global__ void __launch_bounds__(256) decode_kernel(const uint8_t* __restrict__ packed,
                                                      const uint16_t* __restrict__ scales, int64_t total,
                                                      int group, T* __restrict__ out) {
    __shared__ uint2 lut[kNumPoints];                       // rank -> four 16-bit permute selectors (26 KB)
    for (int i = threadIdx.x; i < kNumPoints; i += blockDim.x) lut[i] = reinterpret_cast<const uint2*>(g_lut_f16sel)[2 * i];
    __syncthreads();
    const int64_t ntrip = (total + 15) / 16;
    const bool words = (reinterpret_cast<uintptr_t>(packed) & 3) == 0;
    for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < ntrip;
         t += (int64_t)gridDim.x * blockDim.x) {
        uint32_t bits;                                      // the triplet: two 12-bit ranks
        if (words && t + 2 < ntrip) {                       // two aligned words always cover bytes 3t .. 3t+2
            const uint32_t* wp = reinterpret_cast<const uint32_t*>(packed) + ((3 * t) >> 2);
            bits = __funnelshift_r(__ldg(wp), __ldg(wp + 1), 8 * (int)((3 * t) & 3));
        } else {
            const uint8_t* p = packed + t * 3;
            bits = (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16);
        }
        const uint32_t c0 = min(bits & 0xFFFu, (uint32_t)(kNumPoints - 1));           // corrupt input must not read
        const uint32_t c1 = min((bits >> 12) & 0xFFFu, (uint32_t)(kNumPoints - 1));   // outside the table
        const int64_t base = t * 16;
        const uint32_t h = decode_scale_bits<T>(scales[base / group]);
        const uint32_t pa = prmt(h, 0u, 0x4004u), pb = prmt(h, 0u, 0x4114u) ^ 0x00800000u;   // {0, lo, lo, 0}, {0, hi, -hi, 0}
        const uint2 s0 = lut[c0], s1 = lut[c1];
        uint32_t v[8];                                      // sixteen 16-bit values
        v[0] = prmt(pa, pb, s0.x); v[1] = prmt(pa, pb, s0.x >> 16); v[2] = prmt(pa, pb, s0.y); v[3] = prmt(pa, pb, s0.y >> 16);
        v[4] = prmt(pa, pb, s1.x); v[5] = prmt(pa, pb, s1.x >> 16); v[6] = prmt(pa, pb, s1.y); v[7] = prmt(pa, pb, s1.y >> 16);
        const bool whole = base + 16 <= total && ((reinterpret_cast<uintptr_t>(out + base) & 15) == 0);
        if constexpr (sizeof(T) == 2) {
            if (whole) {
                uint4* dst = reinterpret_cast<uint4*>(out + base);
                dst[0] = make_uint4(v[0], v[1], v[2], v[3]);
                dst[1] = make_uint4(v[4], v[5], v[6], v[7]);
            } else {
                uint16_t* o16 = reinterpret_cast<uint16_t*>(out);
                for (int i = 0; i < 16; ++i)
                    if (base + i < total) o16[base + i] = (uint16_t)(v[i >> 1] >> (16 * (i & 1)));
            }
        } else {
            float f[16];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float2 p2 = __half22float2(*reinterpret_cast<const __half2*>(&v[i]));
                f[2 * i] = p2.x; f[2 * i + 1] = p2.y;
            }
            if (whole) {
                float4* dst = reinterpret_cast<float4*>(out + base);
#pragma unroll
                for (int i = 0; i < 4; ++i) dst[i] = make_float4(f[4 * i], f[4 * i + 1], f[4 * i + 2], f[4 * i + 3]);
            } else {
                for (int i = 0; i < 16; ++i)
                    if (base + i < total) out[base + i] = f[i];
            }
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
    if (blocks > 148 * 8) blocks = 148 * 8;       // every block loads the 26 KB table once: one resident wave, grid-stride loop
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
