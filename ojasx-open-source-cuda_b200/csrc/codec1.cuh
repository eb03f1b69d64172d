// Encoder and decoder of the 1.0-bit format: one byte per 8-block, the index of one of 256 vectors (the 240 roots of
// E8 and 16 axis vectors, all doubled: coordinates 0, +-1, +-2), weight = coordinate * scale with one fp16
// least-squares scale per group of g consecutive weights.
//
// Follows RootE8LatticePacker.pack / unpack (ojasx2/math/lattice.py:475-537).  The reference picks the code with
// argmax over torch.matmul(v, normalize(table)^T); on its CPU path every entry of that product is the chain
// acc = fma(v[k], t[k], acc), k = 0..7, from acc = 0, and the first maximum wins.  The same chains are evaluated
// here, sharing what the table's structure lets them share:
//   * two non-zeros +-c (c = fl(2 / sqrt 8)) at i < j:   fma(v[j], +-c, fl(v[i] * +-c))               112 codes
//   * (+-d)^8, even number of minus signs (d = c / 2):    a binary tree over the first seven signs, the eighth fixed by
//     parity; flipping all eight signs negates the chain exactly, so only the half with a leading minus is walked
//     and the other half is read off its minima                                                        128 codes
//   * one non-zero +-1 at i:                              -+v[i]                                        16 codes
// The scale is <w, q> / <q, q> with the sum in torch.sum's CPU order (chunks of eight into four vector accumulators in
// turn, accumulators added 0..3, lanes 0..7).
#pragma once

#include "codec.cuh"

namespace ojx {

struct RootBest {
    float val;
    int idx;
};

// Index of the best of the 256 table vectors for one 8-block of normalised weights.
__device__ __forceinline__ int root_argmax(const float (&v)[8]) {
    const float c = __uint_as_float(0x3f3504f3u);            // 0.70710677: 2 / fl(sqrt(8))
    const float d = __uint_as_float(0x3eb504f3u);            // 0.35355338: 1 / fl(sqrt(8))
    RootBest best;
    // --- 112 codes with two non-zeros: index = 4 * pair + 2 * (s1 > 0) + (s2 > 0), pairs (i, j) in lexicographic order
    {
        float p[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) p[i] = __fmul_rn(v[i], c);
        best.val = __fmaf_rn(v[1], -c, -p[0]);
        best.idx = 0;
        int idx = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int j = i + 1; j < 8; ++j)
#pragma unroll
                for (int s = 0; s < 4; ++s) {
                    const float dot = __fmaf_rn(v[j], (s & 1) ? c : -c, (s & 2) ? p[i] : -p[i]);
                    if (dot > best.val) { best.val = dot; best.idx = idx; }
                    ++idx;
                }
    }
    // --- 128 codes (+-d)^8: bits b0..b6 of B choose the first seven signs (0 = minus), the eighth makes the number of
    // minus signs even; index = 112 + (B >> 1) over the 8-bit patterns in increasing order.  Walk b0 = 0 only.
    {
        float hi = 0.f, lo = 0.f;          // largest chain value (first occurrence) and smallest (last occurrence)
        int hi_at = -1, lo_at = -1;        // as 7-bit prefixes
        const float a0 = -__fmul_rn(v[0], d);
#pragma unroll
        for (int b = 0; b < 64; ++b) {     // bits b1..b6 of the pattern are bits 5..0 of b
            float acc = a0;
#pragma unroll
            for (int k = 1; k < 7; ++k) acc = __fmaf_rn(v[k], ((b >> (6 - k)) & 1) ? d : -d, acc);
            const int ones = __popc(b);                                   // plus signs among the first seven (b0 = 0)
            const bool last_plus = (ones & 1) != 0;                       // even number of minus signs over all eight
            acc = __fmaf_rn(v[7], last_plus ? d : -d, acc);
            if (hi_at < 0 || acc > hi) { hi = acc; hi_at = b; }
            if (lo_at < 0 || acc <= lo) { lo = acc; lo_at = b; }
        }
        // first half: pattern B = (0, b, last) -> index 112 + b; second half: the complement of (0, b, last) has
        // prefix 127 - b -> index 112 + 127 - b, value -acc; its first maximum is the LAST minimum of the first half
        if (hi > best.val) { best.val = hi; best.idx = 112 + hi_at; }
        if (-lo > best.val) { best.val = -lo; best.idx = 112 + 127 - lo_at; }
    }
    // --- 16 codes with one non-zero: index 240 + 2 i + (sign > 0), value -+v[i]
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        if (-v[i] > best.val) { best.val = -v[i]; best.idx = 240 + 2 * i; }
        if (v[i] > best.val) { best.val = v[i]; best.idx = 241 + 2 * i; }
    }
    return best.idx;
}

template <typename T>
__global__ void __launch_bounds__(128) encode1_kernel(const T* __restrict__ w, int64_t total, int group, float sqrt_group,
                                                       uint8_t* __restrict__ packed, uint16_t* __restrict__ scales, int64_t ngroups) {
    for (int64_t gi = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; gi < ngroups; gi += (int64_t)gridDim.x * blockDim.x) {
        const int64_t base = gi * group;
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        for (int dd = 0; dd < group; dd += 8)
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float x = (base + dd + j < total) ? to_f32<T>(w[base + dd + j]) : 0.f;
                acc[j] = __fadd_rn(acc[j], __fmul_rn(x, x));
            }
        float s = acc[0];
#pragma unroll
        for (int j = 1; j < 8; ++j) s = __fadd_rn(s, acc[j]);
        const float scale = __fadd_rn(__fdiv_rn(__fsqrt_rn(s), sqrt_group), 1e-8f);
        const bool fast = scale >= 1e-7f && scale <= 1e30f;             // x / scale through the reciprocal, exactly (codec.cuh)
        const float rcp = fast ? __frcp_rn(scale) : 0.f;
        float dotacc[4][8];                                             // <w, q> in torch.sum's order
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
            for (int j = 0; j < 8; ++j) dotacc[u][j] = 0.f;
        float qq = 0.f;                                                 // <q, q>: small integers, exact in any order
        uint8_t* out = packed + gi * (int64_t)(group / 8);
        for (int b = 0; b < group / 8; ++b) {
            float x[8], v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int64_t at = base + b * 8 + i;
                x[i] = at < total ? to_f32<T>(w[at]) : 0.f;
                if (fast) {
                    const float q0 = __fmul_rn(x[i], rcp);
                    v[i] = __fmaf_rn(__fmaf_rn(-scale, q0, x[i]), rcp, q0);
                } else {
                    v[i] = __fdiv_rn(x[i], scale);
                }
            }
            const int code = root_argmax(v);
            out[b] = (uint8_t)code;
            const uint32_t lo = g_root_coords[2 * code], hi = g_root_coords[2 * code + 1];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float q = (float)(int)(int8_t)(((i < 4 ? lo : hi) >> (8 * (i & 3))) & 0xFFu);
                const float pr = __fmul_rn(x[i], q);
                qq = __fadd_rn(qq, __fmul_rn(q, q));
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if ((b & 3) == u) dotacc[u][i] = __fadd_rn(dotacc[u][i], pr);
            }
        }
        float lanes[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
            lanes[j] = __fadd_rn(__fadd_rn(__fadd_rn(dotacc[0][j], dotacc[1][j]), dotacc[2][j]), dotacc[3][j]);
        float dot = lanes[0];
#pragma unroll
        for (int j = 1; j < 8; ++j) dot = __fadd_rn(dot, lanes[j]);
        scales[gi] = __half_as_ushort(__float2half_rn(__fdiv_rn(dot, fmaxf(qq, 1e-8f))));
    }
}

int32_t encode1_impl(const void* w, int w_dtype, int64_t rows, int64_t cols, int group, uint8_t* packed, uint16_t* scales,
                     cudaStream_t s) {
    OJX_RETURN_IF(!w || !packed || !scales, OJX_ERR_NULL);
    OJX_RETURN_IF(rows <= 0 || cols <= 0, OJX_ERR_SHAPE);
    OJX_RETURN_IF(check_arch() != OJX_OK, OJX_ERR_ARCH);
    if (group <= 0 || group % 8 != 0) group = 8;              // as the reference does (lattice.py:485-486)
    const int64_t total = rows * cols;
    const int64_t ngroups = (total + group - 1) / group;
    const float sg = (float)sqrt((double)group);
    int64_t blocks = (ngroups + 127) / 128;
    if (blocks > 148 * 64) blocks = 148 * 64;
    switch (w_dtype) {
        case OJX_F32: encode1_kernel<float><<<(unsigned)blocks, 128, 0, s>>>(static_cast<const float*>(w), total, group, sg, packed, scales, ngroups); break;
        case OJX_F16: encode1_kernel<__half><<<(unsigned)blocks, 128, 0, s>>>(static_cast<const __half*>(w), total, group, sg, packed, scales, ngroups); break;
        case OJX_BF16: encode1_kernel<__nv_bfloat16><<<(unsigned)blocks, 128, 0, s>>>(static_cast<const __nv_bfloat16*>(w), total, group, sg, packed, scales, ngroups); break;
        default: return OJX_ERR_DTYPE;
    }
    return launch_status();
}

// Decoder: one thread per 8 weights (one code byte, one scale).
template <typename T>
__global__ void __launch_bounds__(256) decode1_kernel(const uint8_t* __restrict__ packed, const uint16_t* __restrict__ scales,
                                                       int64_t total, int group, T* __restrict__ out) {
    const int64_t blocks8 = (total + 7) / 8;
    for (int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; b < blocks8; b += (int64_t)gridDim.x * blockDim.x) {
        const int code = packed[b];
        const uint32_t lo = g_root_coords[2 * code], hi = g_root_coords[2 * code + 1];
        const float sc = decode_scale<T>(scales[(b * 8) / group]);
        T vals[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
            vals[i] = from_f32<T>(__fmul_rn((float)(int)(int8_t)(((i < 4 ? lo : hi) >> (8 * (i & 3))) & 0xFFu), sc));
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

int32_t decode1_impl(const uint8_t* packed, const uint16_t* scales, int64_t rows, int64_t cols, int group, int out_dtype,
                     void* out, cudaStream_t s) {
    OJX_RETURN_IF(!packed || !scales || !out, OJX_ERR_NULL);
    OJX_RETURN_IF(rows <= 0 || cols <= 0 || group <= 0 || group % 8 != 0, OJX_ERR_SHAPE);
    OJX_RETURN_IF(check_arch() != OJX_OK, OJX_ERR_ARCH);
    const int64_t total = rows * cols;
    int64_t blocks = ((total + 7) / 8 + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    switch (out_dtype) {
        case OJX_F32: decode1_kernel<float><<<(unsigned)blocks, 256, 0, s>>>(packed, scales, total, group, static_cast<float*>(out)); break;
        case OJX_F16: decode1_kernel<__half><<<(unsigned)blocks, 256, 0, s>>>(packed, scales, total, group, static_cast<__half*>(out)); break;
        case OJX_BF16: decode1_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, s>>>(packed, scales, total, group, static_cast<__nv_bfloat16*>(out)); break;
        default: return OJX_ERR_DTYPE;
    }
    return launch_status();
}

}  // namespace ojx
