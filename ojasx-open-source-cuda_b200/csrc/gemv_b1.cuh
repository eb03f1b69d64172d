// Decode GEMV for the 1.0-bit format and 1..8 activation rows on int8 tensor cores.
//
//   y[m, n] = sum over scale groups G of  scale[n, G] * sum_{k in G} coord[n, k] x[m, k]      (+ bias)
//
// Replaces the 1.0-bit branch of _FusedE8GEMMFunction.forward (ojasx2/math/lattice.py:596-624) and the native
// fused_e8_gemm_forward<T> (ojasx2/math/csrc/ojasx_math_core.hpp:444) for small batches, group size 32, K % 2048 == 0.
//
// Why this format suits mma.sync.m16n8k32: a code byte names eight coordinates in {0, +-1, +-2}, i.e. eight int8
// operand bytes = the two A registers one lane supplies for one weight row, and the four code bytes of a scale group of
// 32 are exactly the four lanes of a quad.  One 64-bit read of a table in shared memory per code byte is the whole
// decode, one MMA covers one scale group of 16 weight rows, and every k of the MMA belongs to the same group - so all
// eight accumulator columns carry work: column 4 (m & 1) + d holds digit d of activation row m.  The 2 KB table is kept
// sixteen times, entry e of copy c in the 64-bit slot 16 e + c: the sixteen lanes that share a 64-bit shared-memory
// access then read sixteen different bank pairs whatever their codes are (one copy measured 55 % of all shared-memory
// wavefronts as bank conflicts).
//
// Work decomposition as in the 2.0-bit kernel: one CTA per SM, two groups of 8 warps that take tiles of 16 weight rows
// independently and share the table and the operands of x; the 256-wide rounds of K are dealt to a group's warps in
// turn.  A round's 32 code bytes and 8 scales per row (768 bytes for the 16 rows) travel by
// 16-byte cp.async copies into a ring in shared memory that belongs to the warp alone (three rounds in flight, no
// registers held by loads in flight, no CTA-wide synchronisation); the four lanes of a quad then read the same 32
// bytes and each uses its own byte of every group.
//
// Activations: 28-bit fixed point per scale group (the group's largest finite magnitude fixes the exponent), split into
// four base-128 digits; digits 2p and 2p + 1 of a row of x land in the two accumulator columns of one lane, which joins
// them in integers, converts once and scales by the weight scale times the group's power of two (exact also where that
// power is subnormal; groups whose largest magnitude is below 2^-123 keep fewer than 28 bits).  The operand bytes depend
// on the round only: every CTA builds them once.  A row of x that holds Inf or NaN sends the whole CTA down a scalar
// fp32 path, which reproduces the dense product's NaN / Inf pattern.
#pragma once

#include "gemv_b2.cuh"

namespace ojx {

constexpr int kB1Warps = 8;                       // warps of a tile group
constexpr int kB1Ahead = 3;                       // rounds in flight per warp
constexpr int kB1RoundBytes = 16 * 32 + 16 * 16;  // one round of a 16-row tile: code bytes, then scales

__host__ __device__ inline size_t b1_smem_bytes(int cbs, int copies, int groups, int K) {      // cbs: column blocks (pairs of activation rows)
    const int rounds = K / 256;
    // operands [cb][round][group pair][lane][32 B], group factors [2 cb][round][parity][group] x 4 B, table copies, the
    // warps' rings, partial sums
    return (size_t)cbs * rounds * 2048 + (size_t)2 * cbs * rounds * 64 + (size_t)2048 * copies +
           (size_t)groups * kB1Warps * kB1Ahead * kB1RoundBytes + (size_t)groups * 2 * kB1Warps * 2 * cbs * 16 * 4;
}

// D = A . B with a zero accumulator operand: no registers to clear before the instruction.
__device__ __forceinline__ void mma_s8_from_zero(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}


template <int kCB, int kB1Copies, int kB1Groups>  // column blocks (pairs of activation rows); copies of the code table (16 or 8); tile groups of 8 warps
__global__ void __launch_bounds__(kB1Groups * kB1Warps * 32, 1)
gemv_b1_kernel(const void* __restrict__ x, int x_dtype, int M, const uint8_t* __restrict__ packed, const uint16_t* __restrict__ scales,
               const void* __restrict__ bias, int N, int K, void* __restrict__ y, int y_dtype,
               const float* __restrict__ lora_t, const void* __restrict__ lora_b, int lora_rank) {
    extern __shared__ __align__(16) uint8_t b1_smem[];
    const int rounds = K / 256;
    uint2* frag = reinterpret_cast<uint2*>(b1_smem);                                   // [cb][round][group pair][col 0..7][quarter 0..3][group & 1]
    float* gf = reinterpret_cast<float*>(b1_smem + (size_t)kCB * rounds * 2048);       // [m < 2 kCB][round][parity][group]
    uint2* lut = reinterpret_cast<uint2*>(gf + (size_t)2 * kCB * rounds * 16);         // slot 16 code + copy -> coordinates 0-3, 4-7
    uint8_t* rings = reinterpret_cast<uint8_t*>(lut + 256 * kB1Copies);                // [warp][slot][768 B]
    float* red_all = reinterpret_cast<float*>(rings + kB1Groups * kB1Warps * kB1Ahead * kB1RoundBytes);   // [group][2][warp][m < 2 kCB][16 rows]

    const int tid = threadIdx.x, lane = tid & 31;
    const int cta_warp = tid >> 5, grp = cta_warp >> 3, warp = cta_warp & (kB1Warps - 1);   // warp: index inside its tile group
    float* red = red_all + (size_t)grp * 2 * kB1Warps * 2 * kCB * 16;
    const int first_tile = blockIdx.x * kB1Groups + grp, tile_step = gridDim.x * kB1Groups;   // this group's tiles
    const int g = lane >> 2, t = lane & 3;
    const int tiles = (N + 15) / 16;
    const int64_t row_codes = K / 8, row_scales = K / 32;
    // ---- this warp's (tile, round) pairs in order, kB1Ahead of them in flight: the first loads are issued before the
    // prologue, whose shared-memory work then hides their latency ----
    const int my_rounds = (rounds - warp + kB1Warps - 1) / kB1Warps;              // rounds warp, warp + 8, ...
    const int my_tiles = first_tile < tiles ? (tiles - first_tile + tile_step - 1) / tile_step : 0;
    const int64_t total = (int64_t)my_tiles * my_rounds;
    int f_ti = 0, f_ri = 0;                                                       // the fetcher's position
    // lane l copies half l & 1 of the code bytes of tile row l >> 1, and (lanes 0-15) the scales of tile row l
    const uint8_t* f_code = nullptr;
    const uint16_t* f_scale = nullptr;
    const uint32_t ring0 = smem_u32(rings + cta_warp * kB1Ahead * kB1RoundBytes);
    auto fetch_rows = [&]() {
        const int tile = first_tile + f_ti * tile_step;
        const int nc = min(tile * 16 + (lane >> 1), N - 1), ns = min(tile * 16 + (lane & 15), N - 1);   // rows beyond N re-read the last row
        f_code = packed + nc * row_codes + (lane & 1) * 16;
        f_scale = scales + ns * row_scales;
    };
    auto fetch = [&](int slot) {                                                  // one commit group per call, also when nothing is left
        if (f_ti < my_tiles) {
            const int r = warp + f_ri * kB1Warps;
            const uint32_t dst = ring0 + slot * kB1RoundBytes;
            cp_async16(dst + lane * 16, f_code + r * 32);
            if (lane < 16) cp_async16(dst + 512 + lane * 16, f_scale + r * 8);
            if (++f_ri == my_rounds) {
                f_ri = 0;
                ++f_ti;
                if (f_ti < my_tiles) fetch_rows();
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (total > 0) fetch_rows();
#pragma unroll
    for (int i = 0; i < kB1Ahead; ++i) fetch(i);

    if (tid < 256) {   // thread `tid` writes all copies of code `tid`, starting at a copy that depends on the code: sixteen lanes, sixteen bank pairs
        const uint2 entry = make_uint2(g_root_coords[2 * tid], g_root_coords[2 * tid + 1]);
#pragma unroll
        for (int c = 0; c < kB1Copies; ++c) lut[tid * kB1Copies + ((c + tid) & (kB1Copies - 1))] = entry;
    }

    // ---- prologue: fixed-point digits of x in the operand layout, once per CTA.  Lane l of (row m, round r) holds
    // k = 8 l .. 8 l + 7 of the round: group l >> 2, quarter l & 3 - one 64-bit operand cell per digit. ----
    bool any_bad = false;                                                         // Inf or NaN seen by this warp
#pragma unroll 2
    for (int mr = cta_warp; mr < 2 * kCB * rounds; mr += kB1Groups * kB1Warps) {
        const int xm = mr / rounds, r = mr - xm * rounds;                         // activation row, round
        uint32_t dw[4][2] = {{0u, 0u}, {0u, 0u}, {0u, 0u}, {0u, 0u}};             // [digit][values 0-3, 4-7] as int8 x 4
        float f0 = 0.f;
        if (xm < M) {                                                             // rows beyond M: zero operands, zero factors
            const int64_t x0 = (int64_t)xm * K + (int64_t)r * 256 + lane * 8;
            float v[8];                                                           // x is 16-byte aligned: one or two vector loads
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
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const uint32_t mag = __float_as_uint(v[i]) & 0x7FFFFFFFu;
                if (mag >= 0x7F800000u) bad = true;
                else amax = max(amax, mag);
            }
            any_bad |= bad;
            amax = max(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
            amax = max(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));             // the four lanes of a group
            const int ex = (int)(amax >> 23);
            const int shift = min(26 - (ex == 0 ? -126 : ex - 127), 149);        // in [-101, 149]: 2^shift applied as two factors
            const int sa = shift >> 1, sb = shift - sa;
            const float fa = __uint_as_float((uint32_t)(127 + sa) << 23), fb = __uint_as_float((uint32_t)(127 + sb) << 23);
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
            f0 = __uint_as_float(shift <= 126 ? (uint32_t)(127 - shift) << 23 : 1u << (149 - shift));   // 2^-shift, exact
        }
        // this lane: group g, quarter t; digit d of row xm is column 4 (xm & 1) + d
        uint2* cell = frag + (((((xm >> 1) * rounds + r) * 4 + (g >> 1)) * 8 + (xm & 1) * 4) * 4 + t) * 2 + (g & 1);
#pragma unroll
        for (int d = 0; d < 4; ++d) cell[d * 8] = make_uint2(dw[d][0], dw[d][1]);
        if (t == 0) {                                                           // lane 4G describes group G of the round
            float* f = gf + (xm * rounds + r) * 16 + g;
            f[0] = f0 * 16384.f;                                                // digits 0, 1: the high pair
            f[8] = f0;                                                          // digits 2, 3
        }
    }
    if (__syncthreads_or(any_bad)) {
        asm volatile("cp.async.wait_all;" ::: "memory");                           // nothing of this thread is still in flight into shared memory
        // Inf / NaN in x: every product in fp32, one warp per weight row
        for (int n = blockIdx.x * kB1Groups * kB1Warps + cta_warp; n < N; n += gridDim.x * kB1Groups * kB1Warps) {
            for (int m = 0; m < M; ++m) {
                float acc = 0.f;
                for (int k = lane; k < K; k += 32) {
                    const uint2 e = lut[kB1Copies * packed[n * row_codes + (k >> 3)]];
                    const float w = (float)(int)(int8_t)((((k & 4) ? e.y : e.x) >> (8 * (k & 3))) & 0xFFu) *
                                    __half2float(__ushort_as_half(scales[n * row_scales + (k >> 5)]));
                    acc = fmaf(load_any(x, x_dtype, (int64_t)m * K + k), w, acc);
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
                if (lane == 0) {
                    if (bias != nullptr) acc += load_any(bias, x_dtype, n);
                    if (lora_rank > 0) acc += lowbit_lora_term(lora_t, lora_b, lora_rank, x_dtype, m, n, N);
                    store_any(y, y_dtype, (int64_t)m * N + n, acc);
                }
            }
        }
        return;
    }


    float og[kCB], og8[kCB];                        // partial sums of (row g | g + 8, activation row 2 cb + (t >> 1)), this lane's digit pair
#pragma unroll
    for (int cb = 0; cb < kCB; ++cb) og[cb] = og8[cb] = 0.f;
    const uint32_t byte_sel = 0x4440u | (uint32_t)t;                               // byte t of a word, zero-extended
    const uint8_t* lut_mine = reinterpret_cast<const uint8_t*>(lut + (lane & (kB1Copies - 1)));   // this lane's copy: slot stride 128 B
    int tiles_done = 0, ti = 0, ri = 0;             // the consumer's position
    for (int64_t it0 = 0; it0 < total; it0 += kB1Ahead) {
#pragma unroll
        for (int slot = 0; slot < kB1Ahead; ++slot) {
            const int64_t it = it0 + slot;
            if (it >= total) break;
            // the slot is complete when at most kB1Ahead - 1 newer groups are pending; the copies were made by other lanes
            asm volatile("cp.async.wait_group %0;" ::"n"(kB1Ahead - 1) : "memory");
            __syncwarp();
            const uint8_t* rs = rings + (cta_warp * kB1Ahead + slot) * kB1RoundBytes;
            const uint4 ca0 = *reinterpret_cast<const uint4*>(rs + g * 32), ca1 = *reinterpret_cast<const uint4*>(rs + g * 32 + 16);
            const uint4 cb0 = *reinterpret_cast<const uint4*>(rs + (g + 8) * 32), cb1 = *reinterpret_cast<const uint4*>(rs + (g + 8) * 32 + 16);
            const uint4 sva = *reinterpret_cast<const uint4*>(rs + 512 + g * 16), svb = *reinterpret_cast<const uint4*>(rs + 512 + (g + 8) * 16);
            __syncwarp();                                                          // every lane has read the slot: refill it
            fetch(slot);
            const int r = warp + ri * kB1Warps;
            const uint32_t wa[8] = {ca0.x, ca0.y, ca0.z, ca0.w, ca1.x, ca1.y, ca1.z, ca1.w};
            const uint32_t wb[8] = {cb0.x, cb0.y, cb0.z, cb0.w, cb1.x, cb1.y, cb1.z, cb1.w};
            const uint32_t sa[4] = {sva.x, sva.y, sva.z, sva.w}, sb[4] = {svb.x, svb.y, svb.z, svb.w};
#pragma unroll
            for (int h = 0; h < 2; ++h) {                                          // scale groups 4h .. 4h + 3 of the round
                // the four groups' table reads first: they depend on nothing but the loaded words
                uint2 ea[4], eb[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    ea[j] = *reinterpret_cast<const uint2*>(lut_mine + prmt(wa[4 * h + j], 0u, byte_sel) * (8 * kB1Copies));
                    eb[j] = *reinterpret_cast<const uint2*>(lut_mine + prmt(wb[4 * h + j], 0u, byte_sel) * (8 * kB1Copies));
                }
#pragma unroll
                for (int cb = 0; cb < kCB; ++cb) {
                    // this lane's accumulator columns 2t, 2t + 1: digits 2 (t & 1), 2 (t & 1) + 1 of activation row 2 cb + (t >> 1)
                    const float4 f4 = *reinterpret_cast<const float4*>(gf + ((2 * cb + (t >> 1)) * rounds + r) * 16 + (t & 1) * 8 + 4 * h);
                    const float fG[4] = {f4.x, f4.y, f4.z, f4.w};
                    const uint4* xo = reinterpret_cast<const uint4*>(frag) + ((cb * rounds + r) * 4 + 2 * h) * 32 + lane;
#pragma unroll
                    for (int p = 0; p < 2; ++p) {                                  // scale groups 4h + 2p, 4h + 2p + 1: one MMA each
                        const uint4 xb = xo[p * 32];
                        const float2 wsa = __half22float2(*reinterpret_cast<const __half2*>(&sa[2 * h + p]));
                        const float2 wsb = __half22float2(*reinterpret_cast<const __half2*>(&sb[2 * h + p]));
                        int c[4], e[4];
                        mma_s8_from_zero(c, ea[2 * p].x, eb[2 * p].x, ea[2 * p].y, eb[2 * p].y, xb.x, xb.y);
                        mma_s8_from_zero(e, ea[2 * p + 1].x, eb[2 * p + 1].x, ea[2 * p + 1].y, eb[2 * p + 1].y, xb.z, xb.w);
                        og[cb] = fmaf(wsa.x * fG[2 * p], (float)(c[0] * 128 + c[1]), og[cb]);
                        og8[cb] = fmaf(wsb.x * fG[2 * p], (float)(c[2] * 128 + c[3]), og8[cb]);
                        og[cb] = fmaf(wsa.y * fG[2 * p + 1], (float)(e[0] * 128 + e[1]), og[cb]);
                        og8[cb] = fmaf(wsb.y * fG[2 * p + 1], (float)(e[2] * 128 + e[3]), og8[cb]);
                    }
                }
            }
            if (ri == my_rounds - 1) {
                // the warp's last round of this tile: join the two digit pairs, park, and let warp 0 add the warps
                float* mybuf = red + ((size_t)(tiles_done & 1) * kB1Warps + warp) * 2 * kCB * 16;
#pragma unroll
                for (int cb = 0; cb < kCB; ++cb) {
                    float a = og[cb], b = og8[cb];
                    a += __shfl_xor_sync(0xFFFFFFFFu, a, 1);
                    b += __shfl_xor_sync(0xFFFFFFFFu, b, 1);
                    if ((t & 1) == 0) {
                        const int m = 2 * cb + (t >> 1);
                        mybuf[m * 16 + g] = a;
                        mybuf[m * 16 + g + 8] = b;
                    }
                    og[cb] = og8[cb] = 0.f;
                }
                asm volatile("bar.sync %0, %1;" ::"r"(1 + grp), "r"(kB1Warps * 32) : "memory");   // the group's warps reach their tile ends in the same order
                if (warp == 0) {
                    const int tile = first_tile + ti * tile_step;
                    for (int e = lane; e < M * 16; e += 32) {                           // element (m, row) of the tile
                        const int m = e >> 4, n = tile * 16 + (e & 15);
                        if (n < N) {
                            const float* b = red + (size_t)(tiles_done & 1) * kB1Warps * 2 * kCB * 16 + e;
                            float sum = 0.f;
#pragma unroll
                            for (int w = 0; w < kB1Warps; ++w) sum += b[(size_t)w * 2 * kCB * 16];   // the host only launches with rounds % 8 == 0
                            if (bias != nullptr) sum += load_any(bias, x_dtype, n);
                            if (lora_rank > 0) sum += lowbit_lora_term(lora_t, lora_b, lora_rank, x_dtype, m, n, N);
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
