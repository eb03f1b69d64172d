// Decode GEMV for the 2.0-bit format and 1..8 activation rows on int8 tensor cores, with no lookup table at all.
//
//   y[m, n] = sum over scale groups of  scale[n, g] * ( sum_k code[n,k] x[m,k]  -  1.5 * sum_k x[m,k] )      (+ bias)
//
// Replaces the 2.0-bit branch of _FusedE8GEMMFunction.forward (ojasx2/math/lattice.py:596-624) and the native
// fused_e8_gemm_forward<T> (ojasx2/math/csrc/ojasx_math_core.hpp:444) for small batches, group size 32, K % 2048 == 0.
// With several activation rows the decoded operand registers of a scale group are used once per row (the rows take
// turns on the same eight accumulator columns), so the decode cost is shared and only MMAs and the per-group scaling
// repeat.
//
// Why this format is cheap: a 32-bit word holds sixteen 2-bit codes, and (word >> 2t) & 0x03030303, t = 0..3, ARE four
// int8 operand registers of mma.sync.m16n8k32 (codes t, 4+t, 8+t, 12+t in the four bytes) - seven shift/mask
// operations per sixteen weights, no table, no permute.  The order of k inside an MMA does not matter as long as the
// activation operand uses the same order, and a word never crosses a scale group.
//
// Work decomposition: a CTA is two groups of 8 warps, one CTA per SM; each group takes tiles of 16 weight rows on its
// own (its own named barrier and partial-sum buffers), while the operands of x are built once by all sixteen warps and
// shared.  Inside a group the 256-wide rounds of K are dealt to the warps
// in turn (round r to warp r mod 8), so one tile's codes are read by all eight warps at once, 64 contiguous bytes per
// row and round, straight from global memory into registers (three rounds in flight per warp; no shared-memory ring is
// needed because nothing is shared between rows).  Lane (g, t) owns rows g and g + 8 and the 64 codes 64t..64t+63 of
// the round (two scale groups); its eight steps (word q = 0..3, register pair p = 0, 1) feed two MMAs each.
//
// Activations: 28-bit fixed point per scale group exactly as in the ternary one-row kernel (gemv_a16.cuh, kI8): the
// group's largest finite magnitude fixes the exponent, the integers are split into four base-128 digits; accumulator
// column 2t' + h takes digits 2h, 2h + 1 of the group that lane quarter t' decodes, so only lane (g, t) with
// g >> 1 == t supplies a non-zero operand.  The operand words depend on the round only, so every CTA builds them once
// (each warp for its own rounds: quantise, then sixteen 16-bit stores per lane, no shuffles) and keeps them in shared
// memory in the byte order of the shift/mask code words, with the groups' sums of x for the -1.5 term.  A row of x that holds Inf or NaN sends the whole CTA down a scalar fp32 path,
// which reproduces the dense product's NaN / Inf pattern.
#pragma once

#include "gemv_a16.cuh"

namespace ojx {

constexpr int kB2Warps = 8;                       // warps of a tile group
constexpr int kB2Ahead = 3;                       // rounds in flight per warp

__host__ __device__ inline size_t b2_smem_bytes(int M, int groups, int K) {
    const int rounds = K / 256;
    return (size_t)M * rounds * (8 * 32 * 4 + 8 * 4 * 4) + (size_t)groups * M * kB2Warps * 16 * 4 * 2;   // operands, group factors, partial sums
}

// The optional adapter term of output (activation row m, weight row n): sum_r t[m, r] * B[r, n] in fp32, t = scaling * x . A
// prepared by the caller, B in the activations' dtype.  Out of line: rare, and the epilogue has no registers to spare.
__device__ __noinline__ float lowbit_lora_term(const float* t, const void* b, int rank, int dtype, int m, int n, int N) {
    float acc = 0.f;
    for (int r = 0; r < rank; ++r) acc = fmaf(t[m * rank + r], load_any(b, dtype, (int64_t)r * N + n), acc);
    return acc;
}

struct B2Loads {
    uint4 ca, cb;                                 // 64 codes of rows g and g + 8
    uint32_t sa, sb;                              // their two fp16 scales each
};

template <int kM, int kB2Groups, bool kLora = false>   // rows of x handled by the unrolled loops; tile groups of 8 warps; adapter term in the epilogue
__global__ void __launch_bounds__(kB2Groups * kB2Warps * 32, 1)
gemv_b2_kernel(const void* __restrict__ x, int x_dtype, int M, const uint8_t* __restrict__ packed, const uint16_t* __restrict__ scales,
               const void* __restrict__ bias, int N, int K, void* __restrict__ y, int y_dtype,
               const float* __restrict__ lora_t, const void* __restrict__ lora_b, int lora_rank) {
    extern __shared__ __align__(16) uint8_t b2_smem[];
    const int rounds = K / 256;
    uint32_t* frag = reinterpret_cast<uint32_t*>(b2_smem);                             // [m][round][digit][word group 0..15][4 words]
    float* gf = reinterpret_cast<float*>(b2_smem + (size_t)M * rounds * 8 * 32 * 4);   // [m][round][group 0..7][ua, ub, -1.5 sum x, pad]
    float* red_all = gf + (size_t)M * rounds * 8 * 4;                                  // [group][2][warp][m][16 rows]

    const int tid = threadIdx.x, lane = tid & 31;
    const int cta_warp = tid >> 5, grp = cta_warp >> 3, warp = cta_warp & (kB2Warps - 1);   // warp: index inside its tile group
    float* red = red_all + (size_t)grp * 2 * kB2Warps * M * 16;
    const int first_tile = blockIdx.x * kB2Groups + grp, tile_step = gridDim.x * kB2Groups;   // this group's tiles
    const int g = lane >> 2, t = lane & 3;

    const int tiles = (N + 15) / 16;
    const int64_t row_codes = K / 4, row_scales = K / 32;
    // ---- this warp's (tile, round) pairs in order, kB2Ahead of them in flight: the first loads are issued before the
    // prologue, whose shared-memory work then hides their latency ----
    const int my_rounds = (rounds - warp + kB2Warps - 1) / kB2Warps;              // rounds warp, warp + 8, ...
    const int my_tiles = first_tile < tiles ? (tiles - first_tile + tile_step - 1) / tile_step : 0;
    const int64_t total = (int64_t)my_tiles * my_rounds;
    // The fetcher and the consumer each walk the (tile, round) pairs with their own counters: no divisions, 32-bit offsets
    // from two row pointers that move once per tile.
    int f_ti = 0, f_ri = 0;
    const uint8_t* f_ca = nullptr; const uint8_t* f_cb = nullptr;
    const uint16_t* f_sa = nullptr; const uint16_t* f_sb = nullptr;
    auto fetch_rows = [&]() {
        const int tile = first_tile + f_ti * tile_step;
        const int na = min(tile * 16 + g, N - 1), nb = min(tile * 16 + g + 8, N - 1);     // rows beyond N re-read the last row
        f_ca = packed + na * row_codes + t * 16; f_cb = packed + nb * row_codes + t * 16;
        f_sa = scales + na * row_scales + t * 2; f_sb = scales + nb * row_scales + t * 2;
    };
    auto fetch = [&](B2Loads& L) {
        const int r = warp + f_ri * kB2Warps;
        L.ca = __ldg(reinterpret_cast<const uint4*>(f_ca + r * 64));
        L.cb = __ldg(reinterpret_cast<const uint4*>(f_cb + r * 64));
        L.sa = __ldg(reinterpret_cast<const uint32_t*>(f_sa + r * 8));
        L.sb = __ldg(reinterpret_cast<const uint32_t*>(f_sb + r * 8));
        if (++f_ri == my_rounds) {
            f_ri = 0;
            ++f_ti;
            if (f_ti < my_tiles) fetch_rows();
        }
    };
    B2Loads ring[kB2Ahead];
    if (total > 0) fetch_rows();
#pragma unroll
    for (int i = 0; i < kB2Ahead; ++i)
        if (i < total) fetch(ring[i]);

    // ---- prologue: fixed-point digits of x in the operand layout, once per CTA ----
    bool any_bad = false;                                                         // Inf or NaN seen by this warp
#pragma unroll 2
    for (int mr = cta_warp; mr < M * rounds; mr += kB2Groups * kB2Warps) {
        const int xm = mr / rounds, r = mr - xm * rounds;                         // activation row, round
        const int64_t x0 = (int64_t)xm * K + (int64_t)r * 256 + lane * 8;
        float v[8];                                                               // x is 16-byte aligned: one or two vector loads
        if (x_dtype == OJX_F32) {
            const float4* src = reinterpret_cast<const float4*>(x) + x0 / 4;
            const float4 a = __ldg(src), c = __ldg(src + 1);
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = c.x; v[5] = c.y; v[6] = c.z; v[7] = c.w;
        } else {
            const uint4 qv = __ldg(reinterpret_cast<const uint4*>(x) + x0 / 8);
            const uint32_t w[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (x_dtype == OJX_BF16) {
                    v[2 * i] = __uint_as_float(w[i] << 16);
                    v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
                } else {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
                    v[2 * i] = f.x; v[2 * i + 1] = f.y;
                }
            }
        }
        uint32_t amax = 0;
        bool bad = false;
        float sum8 = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t mag = __float_as_uint(v[i]) & 0x7FFFFFFFu;
            if (mag >= 0x7F800000u) bad = true;
            else amax = max(amax, mag);
            sum8 += v[i];
        }
        any_bad |= bad;
        amax = max(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
        amax = max(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));                 // the four lanes of a group
        sum8 += __shfl_xor_sync(0xFFFFFFFFu, sum8, 1);
        sum8 += __shfl_xor_sync(0xFFFFFFFFu, sum8, 2);                           // sum of the group's 32 activations
        const int ex = (int)(amax >> 23);
        const int shift = 26 - (ex == 0 ? -126 : ex - 127);                      // in [-101, 152]: applied as two factors
        const int sa = shift >> 1, sb = shift - sa;
        const float fa = __uint_as_float((uint32_t)(127 + sa) << 23), fb = __uint_as_float((uint32_t)(127 + sb) << 23);
        uint32_t dw[4][2] = {{0u, 0u}, {0u, 0u}, {0u, 0u}, {0u, 0u}};             // [digit][values 0-3, 4-7] as int8 x 4
#pragma unroll
        for (int h = 0; h < 2; ++h) {                                           // values 4h .. 4h + 3: one operand word per digit
            int dg[4][4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int q0 = __float2int_rn(v[4 * h + j] * fa * fb);
                const int q1 = (q0 + 64) >> 7, q2 = (q1 + 64) >> 7;
                dg[0][j] = (q2 + 64) >> 7;
                dg[1][j] = q2 - (dg[0][j] << 7);
                dg[2][j] = q1 - (q2 << 7);
                dg[3][j] = q0 - (q1 << 7);
            }
#pragma unroll
            for (int d = 0; d < 4; ++d)                                            // low bytes of four integers into one word
                dw[d][h] = prmt(prmt((uint32_t)dg[d][0], (uint32_t)dg[d][1], 0x0040u), prmt((uint32_t)dg[d][2], (uint32_t)dg[d][3], 0x0040u), 0x5410u);
        }
        // Operand layout in shared memory: frag[round][digit][word group 0..15][c 0..3] - the 32-bit word (group, c) holds
        // the digit bytes of k = 16 group + c + {0, 4, 8, 12}, exactly the bytes that meet the code bytes of
        // (code word >> 2c) & 0x03030303.  This lane holds k = 8 lane .. 8 lane + 7: values c and c + 4 are the low (even
        // lane) or high (odd lane) half of word (lane >> 1, c).
        uint16_t* half = reinterpret_cast<uint16_t*>(frag + (size_t)mr * 256) + (lane >> 1) * 8 + (lane & 1);
#pragma unroll
        for (int d = 0; d < 4; ++d)
#pragma unroll
            for (int c = 0; c < 4; ++c)
                half[d * 128 + c * 2] = (uint16_t)prmt(dw[d][0], dw[d][1], 0x4040u | (uint32_t)c | ((uint32_t)(4 + c) << 4));
        if (t == 0) {                                                           // lane 4G describes group G of the round
            float* f = gf + ((size_t)mr * 8 + g) * 4;
            f[0] = __uint_as_float((uint32_t)(127 - sa) << 23);
            f[1] = __uint_as_float((uint32_t)(127 - sb) << 23);
            f[2] = -1.5f * sum8;
            f[3] = 0.f;
        }
    }
    if (__syncthreads_or(any_bad)) {
        // Inf / NaN in x: every product in fp32, one warp per weight row
        for (int n = blockIdx.x * kB2Groups * kB2Warps + cta_warp; n < N; n += gridDim.x * kB2Groups * kB2Warps) {
            for (int m = 0; m < M; ++m) {
                float acc = 0.f;
                for (int k = lane; k < K; k += 32) {
                    const float w = ((float)((packed[n * row_codes + (k >> 2)] >> (2 * (k & 3))) & 3) - 1.5f) *
                                    __half2float(__ushort_as_half(scales[n * row_scales + (k >> 5)]));
                    acc = fmaf(load_any(x, x_dtype, (int64_t)m * K + k), w, acc);
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
                if (lane == 0) {
                    if (bias != nullptr) acc += load_any(bias, x_dtype, n);
                    if (kLora && lora_rank > 0) acc += lowbit_lora_term(lora_t, lora_b, lora_rank, x_dtype, m, n, N);
                    store_any(y, y_dtype, (int64_t)m * N + n, acc);
                }
            }
        }
        return;
    }


    const bool owner = (g >> 1) == t;
    float og[kM], og8[kM];                          // this warp's partial sums of rows g and g + 8 of the current tile, per row of x
#pragma unroll
    for (int m = 0; m < kM; ++m) og[m] = og8[m] = 0.f;
    int tiles_done = 0, ti = 0, ri = 0;             // the consumer's position
    for (int64_t it0 = 0; it0 < total; it0 += kB2Ahead) {
#pragma unroll
        for (int slot = 0; slot < kB2Ahead; ++slot) {
            const int64_t it = it0 + slot;
            if (it >= total) break;
            const B2Loads L = ring[slot];
            if (it + kB2Ahead < total) fetch(ring[slot]);
            const int r = warp + ri * kB2Warps;
            const uint32_t wa[4] = {L.ca.x, L.ca.y, L.ca.z, L.ca.w}, wb[4] = {L.cb.x, L.cb.y, L.cb.z, L.cb.w};
#pragma unroll
            for (int h = 0; h < 2; ++h) {                                          // scale group 2t + h of the round: words 2h, 2h + 1
                // the sixteen operand registers of the group (rows g and g + 8, two words), decoded once for all rows of x
                uint32_t ar[2][4], br[2][4];
#pragma unroll
                for (int qq = 0; qq < 2; ++qq)
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        ar[qq][c] = (wa[2 * h + qq] >> (2 * c)) & 0x03030303u;
                        br[qq][c] = (wb[2 * h + qq] >> (2 * c)) & 0x03030303u;
                    }
                const float wsa = __half2float(__ushort_as_half((uint16_t)(h ? (L.sa >> 16) : (L.sa & 0xFFFFu))));
                const float wsb = __half2float(__ushort_as_half((uint16_t)(h ? (L.sb >> 16) : (L.sb & 0xFFFFu))));
#pragma unroll
                for (int m = 0; m < kM; ++m) {
                    if (kM > 1 && m >= M) break;
                    // this lane's operand words (owners only): digits 2 (g & 1) and 2 (g & 1) + 1 of word groups 4t .. 4t + 3
                    const uint32_t* xf = frag + ((size_t)m * rounds + r) * 256 + (size_t)(2 * (g & 1)) * 64 + 16 * t;
                    int c0[4] = {0, 0, 0, 0}, c1[4] = {0, 0, 0, 0};
#pragma unroll
                    for (int qq = 0; qq < 2; ++qq) {
                        const int q = 2 * h + qq;
                        uint4 xa = make_uint4(0u, 0u, 0u, 0u), xb = make_uint4(0u, 0u, 0u, 0u);
                        if (owner) {                                               // words c = 0..3 of the first and the second digit
                            xa = *reinterpret_cast<const uint4*>(xf + q * 4);
                            xb = *reinterpret_cast<const uint4*>(xf + 64 + q * 4);
                        }
                        // codes {0,4,8,12} and {1,5,9,13} of the word, then {2,6,10,14} and {3,7,11,15}; c0 / c1: the two digits
                        mma_s8(c0, ar[qq][0], br[qq][0], ar[qq][1], br[qq][1], xa.x, xa.y);
                        mma_s8(c1, ar[qq][0], br[qq][0], ar[qq][1], br[qq][1], xb.x, xb.y);
                        mma_s8(c0, ar[qq][2], br[qq][2], ar[qq][3], br[qq][3], xa.z, xa.w);
                        mma_s8(c1, ar[qq][2], br[qq][2], ar[qq][3], br[qq][3], xb.z, xb.w);
                    }
                    // column 2t: digits 0 (c0) and 1 (c1); column 2t + 1: digits 2 and 3; rows g (0, 1) and g + 8 (2, 3)
                    const float4 f = *reinterpret_cast<const float4*>(gf + (((size_t)m * rounds + r) * 8 + 2 * t + h) * 4);
                    const float sg = fmaf((float)(c0[0] * 128 + c1[0]), 16384.f, (float)(c0[1] * 128 + c1[1]));
                    const float sg8 = fmaf((float)(c0[2] * 128 + c1[2]), 16384.f, (float)(c0[3] * 128 + c1[3]));
                    og[m] = fmaf(wsa, fmaf(sg * f.x, f.y, f.z), og[m]);
                    og8[m] = fmaf(wsb, fmaf(sg8 * f.x, f.y, f.z), og8[m]);
                }
            }
            if (ri == my_rounds - 1) {
                // the warp's last round of this tile: combine the four lane quarters, park, and let warp 0 add the warps
                float* mybuf = red + ((size_t)(tiles_done & 1) * kB2Warps + warp) * M * 16;
#pragma unroll
                for (int m = 0; m < kM; ++m) {
                    if (kM > 1 && m >= M) break;
                    float a = og[m], b = og8[m];
                    a += __shfl_xor_sync(0xFFFFFFFFu, a, 1);
                    b += __shfl_xor_sync(0xFFFFFFFFu, b, 1);
                    a += __shfl_xor_sync(0xFFFFFFFFu, a, 2);
                    b += __shfl_xor_sync(0xFFFFFFFFu, b, 2);
                    if (t == 0) { mybuf[m * 16 + g] = a; mybuf[m * 16 + g + 8] = b; }
                    og[m] = og8[m] = 0.f;
                }
                asm volatile("bar.sync %0, %1;" ::"r"(1 + grp), "r"(kB2Warps * 32) : "memory");   // the group's warps reach their tile ends in the same order
                if (warp == 0) {
                    const int tile = first_tile + ti * tile_step;
                    for (int e = lane; e < M * 16; e += 32) {                           // element (m, row) of the tile
                        const int m = e >> 4, n = tile * 16 + (e & 15);
                        if (n < N) {
                            const float* b = red + (size_t)(tiles_done & 1) * kB2Warps * M * 16 + e;
                            float sum = 0.f;
#pragma unroll
                            for (int w = 0; w < kB2Warps; ++w) sum += b[(size_t)w * M * 16];   // the host only launches with rounds % 8 == 0
                            if (bias != nullptr) sum += load_any(bias, x_dtype, n);
                            if (kLora && lora_rank > 0) sum += lowbit_lora_term(lora_t, lora_b, lora_rank, x_dtype, m, n, N);
                            store_any(y, y_dtype, (int64_t)m * N + n, sum);
                        }
                    }
                }
                ++tiles_done;
            }
            if (++ri == my_rounds) { ri = 0; ++ti; }
        }
    }
}

}  // namespace ojx
