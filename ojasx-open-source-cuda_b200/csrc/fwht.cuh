// 32-point normalised Walsh-Hadamard transform over consecutive blocks of 32 elements, computed in the
// element type's own arithmetic exactly as fwht_block32 does (ojasx2/math/lattice.py:91-102): five
// butterfly stages (spans 1, 2, 4, 8, 16; each sum and difference rounded to the element type), then one
// multiplication by float32(1/sqrt(32)) in fp32, rounded to the element type.
//
// 16-bit types run on packed pairs: add/sub/fma.rn.{bf16x2,f16x2} round once to the 16-bit type, which
// equals the reference's "add in fp32, round to 16 bits" - the exact sum of two 16-bit floats is either
// representable in fp32 or so far from every 16-bit rounding boundary that the intermediate rounding
// cannot move it across one.
#pragma once

#include "common.cuh"

namespace ojx {

__device__ __forceinline__ float fwht_norm() { return 0.1767766952966369f; }

__device__ __forceinline__ void fwht32_f32(float* x) {
#pragma unroll
    for (int span = 1; span < 32; span <<= 1) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            if ((i & span) == 0) {
                const float a = x[i], b = x[i + span];
                x[i] = __fadd_rn(a, b);
                x[i + span] = __fsub_rn(a, b);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 32; ++i) x[i] = __fmul_rn(x[i], fwht_norm());
}

template <typename T> struct Pair16;

template <> struct Pair16<__nv_bfloat16> {
    static constexpr uint32_t kPlusMinusOne = 0xBF803F80u;          // low half +1.0, high half -1.0
    static __device__ __forceinline__ uint32_t add(uint32_t a, uint32_t b) {
        uint32_t d; asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d;
    }
    static __device__ __forceinline__ uint32_t sub(uint32_t a, uint32_t b) {
        uint32_t d; asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d;
    }
    static __device__ __forceinline__ uint32_t fma(uint32_t a, uint32_t b, uint32_t c) {
        uint32_t d; asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c)); return d;
    }
    static __device__ __forceinline__ float lo(uint32_t w) { return __uint_as_float(w << 16); }
    static __device__ __forceinline__ float hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }
    static __device__ __forceinline__ uint32_t pack(float lo_v, float hi_v) {
        uint32_t d; asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi_v), "f"(lo_v)); return d;
    }
};

template <> struct Pair16<__half> {
    static constexpr uint32_t kPlusMinusOne = 0xBC003C00u;
    static __device__ __forceinline__ uint32_t add(uint32_t a, uint32_t b) {
        uint32_t d; asm("add.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d;
    }
    static __device__ __forceinline__ uint32_t sub(uint32_t a, uint32_t b) {
        uint32_t d; asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d;
    }
    static __device__ __forceinline__ uint32_t fma(uint32_t a, uint32_t b, uint32_t c) {
        uint32_t d; asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c)); return d;
    }
    static __device__ __forceinline__ float lo(uint32_t w) { return __half2float(__ushort_as_half((uint16_t)(w & 0xFFFFu))); }
    static __device__ __forceinline__ float hi(uint32_t w) { return __half2float(__ushort_as_half((uint16_t)(w >> 16))); }
    static __device__ __forceinline__ uint32_t pack(float lo_v, float hi_v) {
        uint32_t d; asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi_v), "f"(lo_v)); return d;
    }
};

// w[j] holds elements (2j, 2j+1) of the block in its (low, high) halves.
template <typename T>
__device__ __forceinline__ void fwht32_pairs(uint32_t* w) {
    using P = Pair16<T>;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        const uint32_t swapped = __byte_perm(w[j], 0u, 0x1032);
        w[j] = P::fma(w[j], P::kPlusMinusOne, swapped);              // (lo + hi, lo - hi)
    }
#pragma unroll
    for (int d = 1; d < 16; d <<= 1) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            if ((j & d) == 0) {
                const uint32_t a = w[j], b = w[j + d];
                w[j] = P::add(a, b);
                w[j + d] = P::sub(a, b);
            }
        }
    }
#pragma unroll
    for (int j = 0; j < 16; ++j)
        w[j] = P::pack(__fmul_rn(P::lo(w[j]), fwht_norm()), __fmul_rn(P::hi(w[j]), fwht_norm()));
}

// Transform of 32 values held as fp32 copies of T values; results are again T values held as fp32.
template <typename T>
__device__ __forceinline__ void fwht32_values(float* x) {
    if constexpr (sizeof(T) == 4) {
        fwht32_f32(x);
    } else {
        uint32_t w[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) w[j] = Pair16<T>::pack(x[2 * j], x[2 * j + 1]);
        fwht32_pairs<T>(w);
#pragma unroll
        for (int j = 0; j < 16; ++j) { x[2 * j] = Pair16<T>::lo(w[j]); x[2 * j + 1] = Pair16<T>::hi(w[j]); }
    }
}

// One thread per block of 32 elements; x and out 16-byte aligned (they may be the same buffer).
template <typename T>
__global__ void __launch_bounds__(128) fwht32_kernel(const T* __restrict__ x, T* __restrict__ out, int64_t blocks32) {
    constexpr int kVecs = 32 * sizeof(T) / 16;
    for (int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; b < blocks32; b += (int64_t)gridDim.x * blockDim.x) {
        const uint4* src = reinterpret_cast<const uint4*>(x + b * 32);
        uint4* dst = reinterpret_cast<uint4*>(out + b * 32);
        uint32_t w[kVecs * 4];
#pragma unroll
        for (int c = 0; c < kVecs; ++c) {
            const uint4 u = __ldg(src + c);
            w[c * 4 + 0] = u.x; w[c * 4 + 1] = u.y; w[c * 4 + 2] = u.z; w[c * 4 + 3] = u.w;
        }
        if constexpr (sizeof(T) == 4) {
            float* f = reinterpret_cast<float*>(w);
            fwht32_f32(f);
        } else {
            fwht32_pairs<T>(w);
        }
#pragma unroll
        for (int c = 0; c < kVecs; ++c) dst[c] = make_uint4(w[c * 4 + 0], w[c * 4 + 1], w[c * 4 + 2], w[c * 4 + 3]);
    }
}

template <typename T>
static int32_t fwht32_typed(const void* x, void* out, int64_t blocks32, cudaStream_t s) {
    const int threads = 128;
    int64_t blocks = (blocks32 + threads - 1) / threads;
    if (blocks > 148 * 32) blocks = 148 * 32;
    fwht32_kernel<T><<<(unsigned)blocks, threads, 0, s>>>(static_cast<const T*>(x), static_cast<T*>(out), blocks32);
    return launch_status();
}

int32_t fwht32_impl(const void* x, int dtype, int64_t count, void* out, cudaStream_t s) {
    OJX_RETURN_IF(!x || !out, OJX_ERR_NULL);
    OJX_RETURN_IF(count <= 0 || count % 32 != 0, OJX_ERR_SHAPE);
    OJX_RETURN_IF(((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15) != 0, OJX_ERR_ALIGN);
    OJX_RETURN_IF(check_arch() != OJX_OK, OJX_ERR_ARCH);
    switch (dtype) {
        case OJX_F32: return fwht32_typed<float>(x, out, count / 32, s);
        case OJX_F16: return fwht32_typed<__half>(x, out, count / 32, s);
        case OJX_BF16: return fwht32_typed<__nv_bfloat16>(x, out, count / 32, s);
        default: return OJX_ERR_DTYPE;
    }
}

}  // namespace ojx
