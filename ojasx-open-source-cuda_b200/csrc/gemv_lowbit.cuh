// Decode-shape linear (1..8 activation rows) for the 2.0-bit and 1.0-bit formats on the ordinary fp32 pipes.
//
//   y[m, n] = sum over scale groups of  scale * ( sum_k u[n,k] x[m,k]  -  off * sum_k x[m,k] )
//
// with u = the unsigned code itself for 2 bits (off = 1.5) and coordinate + 2 for 1 bit (off = 2): the per-group sums
// of x do not depend on the weight row, so they are formed once per CTA.  Replaces the 2.0-bit / 1.0-bit branches of
// _FusedE8GEMMFunction.forward (ojasx2/math/lattice.py:596-624) and the native fused_e8_gemm_forward<T>
// (ojasx2/math/csrc/ojasx_math_core.hpp:444) for small batches.
//
// One warp per weight row; a lane takes units of 16 consecutive weights (4 bytes of 2-bit codes, 2 code bytes of the
// 1-bit format), so a warp reads 128 (64) contiguous bytes of codes per step.  x sits in shared memory as fp32, 16
// values + 4 floats of padding per unit (the eight lanes of a 128-bit shared-memory access then fall on distinct
// banks).  A code becomes a float without an integer conversion: one byte permute drops it into the mantissa of 2^23,
// one subtraction removes 2^23.
#pragma once

#include "gemv.cuh"

namespace ojx {

constexpr int kLowbitUnitFloats = 20;            // 16 activations + 4 floats of padding

__host__ __device__ inline size_t lowbit_smem_bytes(int64_t M, int64_t K, int fmt) {
    return (size_t)(M * (K / 16) * kLowbitUnitFloats * 4 + M * (K / 8) * 4 + (fmt == 1 ? 2048 : 0));
}

// Byte j of `word` as a float (0..255), exactly.
template <int J>
__device__ __forceinline__ float byte_to_float(uint32_t word) {
    return __uint_as_float(prmt(word, 0x4B000000u, 0x7540u | J)) - 8388608.0f;
}

template <int kFmt, int kM>
__global__ void __launch_bounds__(256) lowbit_gemv_kernel(const void* __restrict__ x, int x_dtype, int M,
                                                           const uint8_t* __restrict__ packed, const uint16_t* __restrict__ scales,
                                                           const void* __restrict__ bias, int N, int K, int group, int group_shift,
                                                           void* __restrict__ y, int y_dtype) {
    extern __shared__ __align__(16) float lb_smem[];
    const int units = K / 16;
    float* xs = lb_smem;                                         // [M][units][20]
    float* xsum = lb_smem + (size_t)M * units * kLowbitUnitFloats;   // [M][K / 8]: sums of 8 consecutive activations
    uint32_t* lut = reinterpret_cast<uint32_t*>(xsum + (size_t)M * (K / 8));   // 1-bit: code -> eight bytes coordinate + 2
    // x (16-byte aligned, K % 16 == 0) arrives eight values per load: a thread's loads do not depend on one another
    for (int i = threadIdx.x; i < M * K / 8; i += blockDim.x) {
        const int e = i * 8, m = e / K, k = e - m * K;
        float v[8];
        if (x_dtype == OJX_F32) {
            const float4 a = __ldg(reinterpret_cast<const float4*>(x) + 2 * i), c = __ldg(reinterpret_cast<const float4*>(x) + 2 * i + 1);
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = c.x; v[5] = c.y; v[6] = c.z; v[7] = c.w;
        } else {
            const uint4 q = __ldg(reinterpret_cast<const uint4*>(x) + i);
            const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (x_dtype == OJX_BF16) {
                    v[2 * j] = __uint_as_float(w[j] << 16);
                    v[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
                } else {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
                    v[2 * j] = f.x; v[2 * j + 1] = f.y;
                }
            }
        }
        float* dst = xs + ((size_t)m * units + (k >> 4)) * kLowbitUnitFloats + (k & 15);
        *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(dst + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
    if (kFmt == 1)
        for (int i = threadIdx.x; i < 512; i += blockDim.x) {      // every int8 coordinate -2..2 becomes the byte 0..4
            const uint32_t c = g_root_coords[i];
            lut[i] = ((c & 0x7F7F7F7Fu) + 0x02020202u) ^ (c & 0x80808080u);    // byte-wise add without carries between bytes
        }
    __syncthreads();
    for (int i = threadIdx.x; i < M * (K / 8); i += blockDim.x) {
        const int m = i / (K / 8), h = i - m * (K / 8);
        const float* p = xs + ((size_t)m * units + (h >> 1)) * kLowbitUnitFloats + (h & 1) * 8;
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) s += p[j];
        xsum[i] = s;
    }
    __syncthreads();

    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    const float off = kFmt == 2 ? 1.5f : 2.0f;
    const int xrow = units * kLowbitUnitFloats, srow = K / 8;      // strides between activation rows in xs and xsum
    for (int n = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; n < N; n += warps) {
        float acc[kM];
#pragma unroll
        for (int m = 0; m < kM; ++m) acc[m] = 0.f;
        const int64_t row0 = (int64_t)n * K;
        // eight steps (8 x 32 units) at a time: all of their code words and scales are requested before the first one is
        // used, so a row costs one memory latency per 4096 weights instead of one per step
        constexpr int kAhead = 8;
        for (int u0 = lane; u0 < units; u0 += 32 * kAhead) {
            uint32_t cw[kAhead];
            uint16_t sw[kAhead][2];
#pragma unroll
            for (int j = 0; j < kAhead; ++j) {
                const int u = u0 + 32 * j;
                cw[j] = 0u; sw[j][0] = sw[j][1] = 0;
                if (u < units) {
                    if (kFmt == 2) cw[j] = __ldg(reinterpret_cast<const uint32_t*>(packed + (row0 >> 2)) + u);
                    else cw[j] = __ldg(reinterpret_cast<const uint16_t*>(packed + (row0 >> 3)) + u);
                    const int64_t at = row0 + 16 * (int64_t)u;
                    sw[j][0] = __ldg(scales + (group_shift >= 0 ? (at >> group_shift) : (at / group)));
                    sw[j][1] = __ldg(scales + (group_shift >= 0 ? ((at + 8) >> group_shift) : ((at + 8) / group)));
                }
            }
#pragma unroll
            for (int j = 0; j < kAhead; ++j) {
                const int u = u0 + 32 * j;
                if (u < units) {
                    // 2 bits: stage word t holds codes t, 4 + t, 8 + t, 12 + t in its four bytes;
                    // 1 bit:  words 0, 1 hold coordinates 0-3, 4-7 (+2) of the first code, words 2, 3 those of the second
                    uint32_t st[4];
                    if (kFmt == 2) {
#pragma unroll
                        for (int t = 0; t < 4; ++t) st[t] = (cw[j] >> (2 * t)) & 0x03030303u;
                    } else {
                        const uint32_t c0 = cw[j] & 0xFFu, c1 = (cw[j] >> 8) & 0xFFu;
                        st[0] = lut[2 * c0]; st[1] = lut[2 * c0 + 1]; st[2] = lut[2 * c1]; st[3] = lut[2 * c1 + 1];
                    }
                    const float* xu = xs + (size_t)u * kLowbitUnitFloats;
                    const float* su = xsum + 2 * u;
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const float sc = __half2float(__ushort_as_half(sw[j][h]));
                        float cf[8];                             // the eight unsigned code values of this half
                        if (kFmt == 2) {
                            if (h == 0) {
                                cf[0] = byte_to_float<0>(st[0]); cf[1] = byte_to_float<0>(st[1]); cf[2] = byte_to_float<0>(st[2]); cf[3] = byte_to_float<0>(st[3]);
                                cf[4] = byte_to_float<1>(st[0]); cf[5] = byte_to_float<1>(st[1]); cf[6] = byte_to_float<1>(st[2]); cf[7] = byte_to_float<1>(st[3]);
                            } else {
                                cf[0] = byte_to_float<2>(st[0]); cf[1] = byte_to_float<2>(st[1]); cf[2] = byte_to_float<2>(st[2]); cf[3] = byte_to_float<2>(st[3]);
                                cf[4] = byte_to_float<3>(st[0]); cf[5] = byte_to_float<3>(st[1]); cf[6] = byte_to_float<3>(st[2]); cf[7] = byte_to_float<3>(st[3]);
                            }
                        } else {
                            const uint32_t lo = st[2 * h], hi = st[2 * h + 1];
                            cf[0] = byte_to_float<0>(lo); cf[1] = byte_to_float<1>(lo); cf[2] = byte_to_float<2>(lo); cf[3] = byte_to_float<3>(lo);
                            cf[4] = byte_to_float<0>(hi); cf[5] = byte_to_float<1>(hi); cf[6] = byte_to_float<2>(hi); cf[7] = byte_to_float<3>(hi);
                        }
#pragma unroll
                        for (int m = 0; m < kM; ++m) {
                            if (kM == 1 || m < M) {
                                const float* xp = xu + m * xrow + 8 * h;
                                const float4 xa = *reinterpret_cast<const float4*>(xp), xb = *reinterpret_cast<const float4*>(xp + 4);
                                float p0 = -off * su[m * srow + h], p1 = 0.f;          // two chains: half the dependent latency
                                p0 = fmaf(cf[0], xa.x, p0); p1 = fmaf(cf[1], xa.y, p1);
                                p0 = fmaf(cf[2], xa.z, p0); p1 = fmaf(cf[3], xa.w, p1);
                                p0 = fmaf(cf[4], xb.x, p0); p1 = fmaf(cf[5], xb.y, p1);
                                p0 = fmaf(cf[6], xb.z, p0); p1 = fmaf(cf[7], xb.w, p1);
                                acc[m] = fmaf(sc, p0 + p1, acc[m]);
                            }
                        }
                    }
                }
            }
        }
#pragma unroll
        for (int m = 0; m < kM; ++m) {
            float v = acc[m];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
            if (lane == 0 && m < M) {
                if (bias != nullptr) v += load_any(bias, x_dtype, n);
                store_any(y, y_dtype, (int64_t)m * N + n, v);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// The same idea for the ternary codes, for the decode shapes the tensor-core kernels do not take: scale groups other
// than 32 (the reference layer's default group size of 8 becomes 16 for this format, ojasx2/math/lattice.py:750-751)
// and fp32 activations.  One warp per weight row; a lane takes units of 64 consecutive weights = eight 12-bit ranks =
// three 32-bit words; a rank is looked up in a table of eight bytes coordinate + 1 (4096 entries, so a corrupt rank
// stays inside it) and y accumulates scale * (sum_k u x - sum_k x) in fp32, every product exact.
// ---------------------------------------------------------------------------------------------
constexpr int kTernUnitFloats = 68;              // 64 activations + 4 floats of padding

__host__ __device__ inline size_t ternary_small_smem_bytes(int64_t M, int64_t K) {
    return (size_t)(M * (K / 64) * kTernUnitFloats * 4 + M * (K / 8) * 4 + 4096 * 8);
}

template <int kM>
__global__ void __launch_bounds__(256) ternary_small_gemv_kernel(const void* __restrict__ x, int x_dtype, int M,
                                                                  const uint8_t* __restrict__ packed, const uint16_t* __restrict__ scales,
                                                                  const void* __restrict__ bias, int N, int K, int group_shift,
                                                                  void* __restrict__ y, int y_dtype) {
    extern __shared__ __align__(16) float ts_smem[];
    const int units = K / 64;
    float* xs = ts_smem;                                              // [M][units][68]
    float* xsum = ts_smem + (size_t)M * units * kTernUnitFloats;       // [M][K / 8]: sums of 8 consecutive activations
    uint2* lut = reinterpret_cast<uint2*>(xsum + (size_t)M * (K / 8)); // rank -> eight bytes coordinate + 1
    for (int i = threadIdx.x; i < M * K / 8; i += blockDim.x) {       // x is 16-byte aligned, K % 64 == 0
        const int e = i * 8, m = e / K, k = e - m * K;
        float v[8];
        if (x_dtype == OJX_F32) {
            const float4 a = __ldg(reinterpret_cast<const float4*>(x) + 2 * i), c = __ldg(reinterpret_cast<const float4*>(x) + 2 * i + 1);
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = c.x; v[5] = c.y; v[6] = c.z; v[7] = c.w;
        } else {
            const uint4 q = __ldg(reinterpret_cast<const uint4*>(x) + i);
            const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (x_dtype == OJX_BF16) {
                    v[2 * j] = __uint_as_float(w[j] << 16);
                    v[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
                } else {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
                    v[2 * j] = f.x; v[2 * j + 1] = f.y;
                }
            }
        }
        float* dst = xs + ((size_t)m * units + (k >> 6)) * kTernUnitFloats + (k & 63);
        *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(dst + 4) = make_float4(v[4], v[5], v[6], v[7]);
        xsum[i] = ((v[0] + v[1]) + (v[2] + v[3])) + ((v[4] + v[5]) + (v[6] + v[7]));
    }
    for (int i = threadIdx.x; i < 4096; i += blockDim.x) {
        const uint32_t nib = i < kNumPoints ? g_trit_nibbles[i] : 0u;  // field: 0 zero, 1 plus, 2 minus
        uint32_t b[2] = {0u, 0u};
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const uint32_t f = (nib >> (4 * c)) & 0xFu;
            b[c >> 2] |= (f == 0u ? 1u : (f == 1u ? 2u : 0u)) << (8 * (c & 3));
        }
        lut[i] = make_uint2(b[0], b[1]);
    }
    __syncthreads();

    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    const int xrow = units * kTernUnitFloats, srow = K / 8;
    const int64_t row_bytes = (int64_t)K * 3 / 16;
    for (int n = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; n < N; n += warps) {
        float acc[kM];
#pragma unroll
        for (int m = 0; m < kM; ++m) acc[m] = 0.f;
        const uint32_t* crow = reinterpret_cast<const uint32_t*>(packed + n * row_bytes);
        const int64_t row0 = (int64_t)n * K;
        constexpr int kAhead = 4;                        // units in flight per lane: a row of 8192 weights costs one memory latency
        for (int u0 = lane; u0 < units; u0 += 32 * kAhead) {
            uint32_t cw[kAhead][3];
            uint16_t sw[kAhead][4];                      // the scales of the unit's four 16-weight quarters
#pragma unroll
            for (int j = 0; j < kAhead; ++j) {
                const int u = u0 + 32 * j;
                cw[j][0] = cw[j][1] = cw[j][2] = 0u;
                sw[j][0] = sw[j][1] = sw[j][2] = sw[j][3] = 0;
                if (u < units) {
                    cw[j][0] = __ldg(crow + 3 * u); cw[j][1] = __ldg(crow + 3 * u + 1); cw[j][2] = __ldg(crow + 3 * u + 2);
#pragma unroll
                    for (int q = 0; q < 4; ++q) sw[j][q] = __ldg(scales + ((row0 + 64 * (int64_t)u + 16 * q) >> group_shift));
                }
            }
#pragma unroll
            for (int j = 0; j < kAhead; ++j) {
                const int u = u0 + 32 * j;
                if (u < units) {
                    const float* xu = xs + (size_t)u * kTernUnitFloats;
                    const float* su = xsum + 8 * u;
#pragma unroll
                    for (int r = 0; r < 8; ++r) {        // rank r of the unit: weights 8r .. 8r + 7
                        const int bit = 12 * r, w = bit >> 5, sh = bit & 31;
                        uint32_t rank;
                        if (sh + 12 <= 32) rank = cw[j][w] >> sh;
                        else rank = __funnelshift_r(cw[j][w], cw[j][w + 1 < 3 ? w + 1 : 2], sh);
                        const uint2 e = lut[rank & 0xFFFu];
                        float cf[8];
                        cf[0] = byte_to_float<0>(e.x); cf[1] = byte_to_float<1>(e.x); cf[2] = byte_to_float<2>(e.x); cf[3] = byte_to_float<3>(e.x);
                        cf[4] = byte_to_float<0>(e.y); cf[5] = byte_to_float<1>(e.y); cf[6] = byte_to_float<2>(e.y); cf[7] = byte_to_float<3>(e.y);
                        const float sc = __half2float(__ushort_as_half(sw[j][r >> 1]));
#pragma unroll
                        for (int m = 0; m < kM; ++m) {
                            if (kM == 1 || m < M) {
                                const float* xp = xu + m * xrow + 8 * r;
                                const float4 xa = *reinterpret_cast<const float4*>(xp), xb = *reinterpret_cast<const float4*>(xp + 4);
                                float p0 = -su[m * srow + r], p1 = 0.f;      // coordinate = byte - 1
                                p0 = fmaf(cf[0], xa.x, p0); p1 = fmaf(cf[1], xa.y, p1);
                                p0 = fmaf(cf[2], xa.z, p0); p1 = fmaf(cf[3], xa.w, p1);
                                p0 = fmaf(cf[4], xb.x, p0); p1 = fmaf(cf[5], xb.y, p1);
                                p0 = fmaf(cf[6], xb.z, p0); p1 = fmaf(cf[7], xb.w, p1);
                                acc[m] = fmaf(sc, p0 + p1, acc[m]);
                            }
                        }
                    }
                }
            }
        }
#pragma unroll
        for (int m = 0; m < kM; ++m) {
            float v = acc[m];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
            if (lane == 0 && m < M) {
                if (bias != nullptr) v += load_any(bias, x_dtype, n);
                store_any(y, y_dtype, (int64_t)m * N + n, v);
            }
        }
    }
}

}  // namespace ojx
