// Decode GEMV for 2..16 bf16 activation rows: int8 tensor cores for 2-8 rows, fp16 tensor cores with
// scale-folded weights for 9-16 rows (template parameter kF16, described at the kernel).
//
// Same work items, cp.async ring and deterministic deferred reduction as gemv_b1.cuh; the MMA is turned
// around so that several activation rows cost one instruction:
//   * the decoded weights are the "B" operand of mma.sync.m16n8k32.s8: eight weight rows x one scale
//     group (32 k) per instruction; lane (g, t) supplies rank t of the group of row g as its two B
//     registers (two byte permutes of the looked-up selector word);
//   * the activations are the "A" operand (16 x 32): rows 0-7 carry the HIGH int8 term of activation rows
//     0-7 and rows 8-15 their LOW term (x * 2^-e = 128 hi + lo, 13-bit fixed point relative to the
//     slice maximum of each activation row, see gemv_b1.cuh), so ONE MMA yields both partial products of
//     eight activation rows and they land in the same lane; 9-16 rows use a second A block;
//   * per group the lane combines hi and lo in integers, converts once and multiplies by the group's
//     scale (fp32 FMA), i.e. the reference's order: acc += (sum_k x * coord) * scale.
#pragma once

#include "gemv_b1.cuh"

namespace ojx {

template <int NBLK> struct BnCfg {
    static constexpr int kStages = NBLK == 1 ? 4 : 3;
    static constexpr int kAhead = 2;
    static constexpr int kRed = 2;                                          // reduction buffers
    static constexpr int kRedLag = 1;
    static constexpr int kCopies = 4;                                       // interleaved copies of the lookup table
    static constexpr int kLutBytes = ((kNumPoints * kCopies * 4 + 1023) / 1024) * 1024;
    static constexpr int kRedFloats = kGemvWarps * 256 * NBLK;              // per buffer: 16 warps x 32 rows x 8 NBLK
    static constexpr size_t kSmem = (size_t)kLutBytes + (size_t)kStages * kB1StageBytes +
                                    (size_t)kRed * kRedFloats * sizeof(float) + 256;
};

// m16n8k32 int8 MMA with a zero accumulator input (the zero registers cost no instructions).
__device__ __forceinline__ void mma_s8_zero(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

// fp16 MMA with fp32 accumulation: D (16 x 8) += A (16 x 16, row-major) * B (16 x 8, column-major).
__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint2 lds_u64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}

// kF16 (9-16 activation rows): the weights enter the MMA as EXACT fp16 values coord * scale, built by byte
// permutes from a {0, +scale, -scale} byte pool with selectors fetched from a 64-bit table, and the activations
// as fp16 (x * 2^-e per row and slice, exact for bf16 inputs), sixteen rows per mma.sync.m16n8k16 with fp32
// accumulation across all eight groups of the slice - so no per-group integer combine, convert and scale
// multiply remain, which is what the int8 form spends most of its instructions on at 16 rows.
template <int NBLK, bool kF16, bool kXF16>
__global__ void __launch_bounds__(kGemvThreads, 1)
gemv_bn_kernel(const ojx_e8t_gemv_problem* __restrict__ probs_dev, const __grid_constant__ ojx_e8t_gemv_problem single,
               int count, int total_items, int M, int y_dtype, const __grid_constant__ PeerMap peers) {
    using Cfg = BnCfg<NBLK>;
    static_assert(kF16 || !kXF16, "fp16 activations take the fp16 form");
    const ojx_e8t_gemv_problem* probs = probs_dev != nullptr ? probs_dev : &single;
    extern __shared__ __align__(128) uint8_t smem[];
    uint32_t* lut = reinterpret_cast<uint32_t*>(smem);
    const uint32_t ring = smem_u32(smem) + Cfg::kLutBytes;
    float* red = reinterpret_cast<float*>(smem + Cfg::kLutBytes + Cfg::kStages * kB1StageBytes);
    uint8_t* tail = smem + Cfg::kLutBytes + Cfg::kStages * kB1StageBytes + Cfg::kRed * Cfg::kRedFloats * sizeof(float);
    const uint32_t bar_full = smem_u32(tail), bar_empty = bar_full + 8 * Cfg::kStages;
    const uint32_t bar_rfull = bar_empty + 8 * Cfg::kStages, bar_rempty = bar_rfull + 8 * Cfg::kRed;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tail + 16 * Cfg::kStages + 16 * Cfg::kRed);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    constexpr uint32_t kItemDescOffset = kB1Rows * kGemvMaxCodePitch - 16;      // free: row pitches end in 16 bytes of padding
    const uint32_t red_desc = smem_u32(tail) + 128;                              // one 16-byte item descriptor per reduction buffer
    const uint32_t bar_lut = smem_u32(tail) + 176;

    if (tid == 0) {
        for (int s = 0; s < Cfg::kStages; ++s) {
            mbar_init(bar_full + 8 * s, kGemvThreads);
            mbar_init(bar_empty + 8 * s, kGemvWarps);
        }
        for (int b = 0; b < Cfg::kRed; ++b) {
            mbar_init(bar_rfull + 8 * b, kGemvWarps);       // every warp has parked its partial sums
            mbar_init(bar_rempty + 8 * b, kGemvWarps);      // every warp has summed its share of the outputs
        }
        mbar_init(bar_lut, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        // the lookup table's shared-memory image arrives as ONE bulk copy while the kernel sets itself up
        mbar_expect_tx(bar_lut, kNumPoints * 16);
        bulk_load(smem_u32(lut), kF16 ? g_lut_f16sel : g_lut_i8x4, kNumPoints * 16, bar_lut);
    }
    __syncthreads();

    const int64_t per = ((int64_t)total_items + gridDim.x - 1) / gridDim.x;
    const int i0 = (int)min((int64_t)total_items, per * blockIdx.x);
    const int i1 = (int)min((int64_t)total_items, per * (blockIdx.x + 1));
    if (i0 >= i1) return;
    const int nitems = i1 - i0;
    const int p0 = find_problem(probs, count, i0, 1);

    // ---- loader (identical to the single-row kernel) ----
    const int lr = tid >> 4, ls = tid & 15;
    B1Cursor ic;
    b1_seek(ic, probs, p0, i0);
    int issued = 0;
    auto issue_next = [&]() {
        const int n = issued, s = n % Cfg::kStages;
        b1_wait(bar_empty + 8 * s, ((uint32_t)(n / Cfg::kStages) & 1u) ^ 1u, abort_flag, 41);
        const int row = ic.tile * kB1Rows + lr;
        if (row < ic.N) {
            const ojx_e8t_gemv_problem& P = probs[ic.prob];
            const int cchunks = 3 * ic.act;
            const uint32_t cb = ic.act * 48, sb = ic.act * 16;
            const uint32_t stage = ring + s * kB1StageBytes;
            const uint8_t* csrc = P.packed + (int64_t)row * (ic.K * 3 / 16) + (int64_t)ic.chunk * cb + ls * 16;
            const uint32_t cdst = stage + lr * (cb + 16) + ls * 16;
#pragma unroll
            for (int j = 0; j < 3; ++j)
                if (ls + 16 * j < cchunks) cp_async16(cdst + 256 * j, csrc + 256 * j);
            if (ls < ic.act)
                cp_async16(stage + kB1Rows * kGemvMaxCodePitch + lr * (sb + 16) + ls * 16,
                           reinterpret_cast<const uint8_t*>(P.scales) + (int64_t)row * (ic.K / 16) + (int64_t)ic.chunk * sb + ls * 16);
        }
        // The item's coordinates travel with its data (in the padding behind the last row's codes), so that
        // only the loader keeps a cursor in registers.
        if (tid == 0)
            sts_u128(ring + s * kB1StageBytes + kItemDescOffset, make_uint4((uint32_t)ic.prob, (uint32_t)ic.chunk, (uint32_t)ic.tile, (uint32_t)ic.act));
        cp_async_arrive(bar_full + 8 * s);
        ++issued;
        b1_next(ic, probs, count);
    };
    for (int n = 0; n < Cfg::kAhead && n < nitems; ++n) issue_next();


    // ---- reduction: every warp sums 16 * NBLK of the item's 256 * NBLK outputs over the 16 warps, in warp order ----
    int reduced = 0;
    auto reduce_next = [&]() {
        const int n = reduced, b = n % Cfg::kRed;
        b1_wait(bar_rfull + 8 * b, (uint32_t)(n / Cfg::kRed) & 1u, abort_flag, 43);
        const float* rbuf = red + (size_t)b * Cfg::kRedFloats;
        if (lane < 16 * NBLK) {
            const uint4 desc = lds_u128(red_desc + 16 * b);          // {problem, K chunk, 32-row tile, -} of item n
            const ojx_e8t_gemv_problem& P = probs[desc.x];
            const int rN = P.N, rchunk = (int)desc.y, rtile = (int)desc.z;
            const int o = warp * 16 * NBLK + lane;                 // output slot inside a warp's 256*NBLK block
            // slot layout: ((blk * 4 + tile8) * 32 + lane') * 2 + j   with lane' = (batch g', rank lane t')
            const int j = o & 1, lp = (o >> 1) & 31, tile8 = (o >> 6) & 3, blk = o >> 8;
            const int row = rtile * kB1Rows + tile8 * 8 + ((lp & 3) << 1) + j;
            const int col = blk * 8 + (lp >> 2);
            float sum = 0.f;
            if (col < M) {                                         // activation rows beyond M hold zeros: nothing to add up
#pragma unroll
                for (int w = 0; w < kGemvWarps; ++w) sum += rbuf[w * 256 * NBLK + o];
            }
            if (row < rN && col < M) {
                if (P.partial != nullptr) P.partial[((int64_t)rchunk * M + col) * rN + row] = sum;
                else {
                    if (P.bias != nullptr) sum += load_any(P.bias, kXF16 ? OJX_F16 : OJX_BF16, row);
                    store_any(P.y, y_dtype, (int64_t)col * rN + row, sum);
                    if (peers.world > 1) store_peers(peers, P.y, y_dtype, (int64_t)col * rN + row, sum);
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_rempty + 8 * b);
        ++reduced;
    };

    // ---- lane constants: this lane takes rank t of every scale group (byte window + nibble shift) ----
    const uint32_t lut_lane = smem_u32(lut) + (kF16 ? ((lane & 1) << 3) : ((lane & (Cfg::kCopies - 1)) << 2));
    constexpr uint32_t kTritBytes = 0x00FF0100u;
    constexpr uint32_t kEntryBytes = Cfg::kCopies * 4;                         // table stride
    const uint32_t bt = (t == 0) ? 0u : (t == 1) ? 1u : (t == 2) ? 3u : 4u;     // first byte of this lane's rank
    const uint32_t sel_even = bt | ((bt + 1) << 4);
    const uint32_t sel_odd = (bt + 2) | ((bt + 3) << 4);
    // the rank sits in bits 0-11 (even t) or 4-15 (odd t) of the 16-bit window: mask, then one multiply-add
    // turns it into the table address (stride 16 bytes)
    static_assert(kEntryBytes == 16, "the multiply-add below assumes a 16-byte table stride");
    const uint32_t win_mask = (t & 1) ? 0xFFF0u : 0x0FFFu;
    const uint32_t win_mul = (t & 1) ? 1u : 16u;

    // A fragments.  int8 form: [block][group][a0 hi, a1 lo, a2 hi, a3 lo].  fp16 form (flattened as
    // [k half j = index 0][group][a0, a1, a2, a3]): rows g and g + 8 of the sixteen activation rows.
    uint32_t xa[NBLK][8][4];
    float upscale[NBLK];
    int cur_prob = -1, cur_chunk = -1;
    struct { int prob, chunk, tile, act, K; } cc;
    cc.K = 0;

    b1_wait(bar_lut, 0u, abort_flag, 45);                          // the table has landed
    for (int n = 0; n < nitems; ++n) {
        const int s = n % Cfg::kStages, b = n % Cfg::kRed;
        if (issued < nitems) issue_next();

        b1_wait(bar_full + 8 * s, (uint32_t)(n / Cfg::kStages) & 1u, abort_flag, 42);
        {
            const uint4 desc = lds_u128(ring + s * kB1StageBytes + kItemDescOffset);
            cc.prob = (int)desc.x; cc.chunk = (int)desc.y; cc.tile = (int)desc.z; cc.act = (int)desc.w;
        }
        if (cc.prob != cur_prob || cc.chunk != cur_chunk) {
            if (cc.prob != cur_prob) cc.K = probs[cc.prob].K;
            cur_prob = cc.prob;
            cur_chunk = cc.chunk;
            const uint16_t* xp = static_cast<const uint16_t*>(probs[cc.prob].x);
            const int slice = cc.chunk * cc.act + warp;
            if constexpr (kF16) {
                static_assert(!kF16 || NBLK == 2, "the fp16 form holds sixteen activation rows");
#pragma unroll
                for (int hrow = 0; hrow < 2; ++hrow) {             // activation rows g and g + 8
                    const int m = hrow * 8 + g;
                    const bool on = warp < cc.act && m < M;
                    uint4 q[8];
                    uint32_t amax = 0;
#pragma unroll
                    for (int grp = 0; grp < 8; ++grp) {
                        q[grp] = make_uint4(0, 0, 0, 0);
                        if (on) q[grp] = __ldg(reinterpret_cast<const uint4*>(xp + (int64_t)m * cc.K + slice * 256 + grp * 32 + t * 8));
                        const uint32_t w[4] = {q[grp].x, q[grp].y, q[grp].z, q[grp].w};
#pragma unroll
                        for (int i = 0; i < 4; ++i) amax = max(amax, max((w[i] << 16) & 0x7FFFFFFFu, w[i] & 0x7FFF0000u));
                    }
                    if constexpr (kXF16) {                         // fp16 activations are MMA operands as they are
                        upscale[hrow] = 1.0f;
#pragma unroll
                        for (int grp = 0; grp < 8; ++grp) {
                            xa[0][grp][hrow] = q[grp].x; xa[0][grp][2 + hrow] = q[grp].y;
                            xa[1][grp][hrow] = q[grp].z; xa[1][grp][2 + hrow] = q[grp].w;
                        }
                        continue;
                    }
                    (void)amax;
                    amax = max(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
                    amax = max(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));  // the four lanes of activation row m
                    int e = 0;
                    const int ex = (int)((amax >> 23) & 0xFFu);
                    if (ex != 0 && ex != 0xFF) e = max(-100, min(100, ex - 127 - 14));   // row maximum -> [2^14, 2^15)
                    const float down = __uint_as_float((uint32_t)(127 - e) << 23);
                    upscale[hrow] = __uint_as_float((uint32_t)(127 + e) << 23);
#pragma unroll
                    for (int grp = 0; grp < 8; ++grp) {
                        const uint32_t w[4] = {q[grp].x, q[grp].y, q[grp].z, q[grp].w};
                        uint32_t h[4];                             // this lane's eight k of the group as four fp16 pairs
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const __half2 v = __floats2half2_rn(__uint_as_float(w[i] << 16) * down, __uint_as_float(w[i] & 0xFFFF0000u) * down);
                            h[i] = *reinterpret_cast<const uint32_t*>(&v);
                        }
                        // k half 0 multiplies coordinates 0-3 of the lane's rank, k half 1 coordinates 4-7
                        xa[0][grp][hrow] = h[0]; xa[0][grp][2 + hrow] = h[1];
                        xa[1][grp][hrow] = h[2]; xa[1][grp][2 + hrow] = h[3];
                    }
                }
            } else {
#pragma unroll
            for (int blk = 0; blk < NBLK; ++blk) {
                const int m = blk * 8 + g;
                const bool on = warp < cc.act && m < M;
                uint4 q[8];
                float amax = 0.f;
#pragma unroll
                for (int grp = 0; grp < 8; ++grp) {
                    q[grp] = make_uint4(0, 0, 0, 0);
                    if (on) q[grp] = __ldg(reinterpret_cast<const uint4*>(xp + (int64_t)m * cc.K + slice * 256 + grp * 32 + t * 8));
                    const uint32_t w[4] = {q[grp].x, q[grp].y, q[grp].z, q[grp].w};
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        amax = fmaxf(amax, fmaxf(fabsf(__uint_as_float(w[i] << 16)), fabsf(__uint_as_float(w[i] & 0xFFFF0000u))));
                }
                amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
                amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));      // the four lanes of activation row m
                int e = 0;
                if (amax > 0.f) e = max(-100, min(100, (int)((__float_as_uint(amax) >> 23) & 0xFFu) - 127 - 12));
                const float down = __uint_as_float((uint32_t)(127 - e) << 23);
                upscale[blk] = __uint_as_float((uint32_t)(127 + e) << 23);
#pragma unroll
                for (int grp = 0; grp < 8; ++grp) {
                    const uint32_t w[4] = {q[grp].x, q[grp].y, q[grp].z, q[grp].w};
                    uint32_t hw[2] = {0u, 0u}, lw[2] = {0u, 0u};
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float v = (i & 1) ? __uint_as_float(w[i >> 1] & 0xFFFF0000u) : __uint_as_float(w[i >> 1] << 16);
                        const int X = __float2int_rn(v * down);
                        const int hi = (X + 64) >> 7, lo = X - (hi << 7);
                        hw[i >> 2] |= (uint32_t)(hi & 0xFF) << (8 * (i & 3));
                        lw[i >> 2] |= (uint32_t)(lo & 0xFF) << (8 * (i & 3));
                    }
                    xa[blk][grp][0] = hw[0]; xa[blk][grp][1] = lw[0]; xa[blk][grp][2] = hw[1]; xa[blk][grp][3] = lw[1];
                }
            }
            }
        }

        // the reduction buffer of this item must have been drained (it was last used kRed items ago)
        b1_wait(bar_rempty + 8 * b, ((uint32_t)(n / Cfg::kRed) & 1u) ^ 1u, abort_flag, 44);
        float* rbuf = red + (size_t)b * Cfg::kRedFloats + warp * 256 * NBLK;

        if (warp < cc.act) {
            const uint32_t cb = cc.act * 48, sb = cc.act * 16;
            const uint32_t stage = ring + s * kB1StageBytes;
            if constexpr (kF16) {
#pragma unroll
                for (int tl = 0; tl < 4; ++tl) {
                    // [activation row g | g + 8][weight row 2t | 2t + 1]; kChains independent accumulation chains
                    // keep the MMA pipe from waiting on its own latency
                    constexpr int kChains = 1;
                    float acc[kChains][4];
#pragma unroll
                    for (int c = 0; c < kChains; ++c) acc[c][0] = acc[c][1] = acc[c][2] = acc[c][3] = 0.f;
                    const uint32_t ca = stage + (tl * 8 + g) * (cb + 16) + warp * 48;
                    const uint32_t sa = stage + kB1Rows * kGemvMaxCodePitch + (tl * 8 + g) * (sb + 16) + warp * 16;
                    const uint4 q0 = lds_u128(ca), q1 = lds_u128(ca + 16), q2 = lds_u128(ca + 32);
                    const uint4 s0 = lds_u128(sa);                     // the eight group scales of weight row g of the tile
                    if (tl == 3) {                                     // everything of this stage is in registers now
                        __syncwarp();
                        if (lane == 0) mbar_arrive(bar_empty + 8 * s);
                    }
                    const uint32_t cw[12] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w, q2.x, q2.y, q2.z, q2.w};
                    const uint32_t sw[4] = {s0.x, s0.y, s0.z, s0.w};
#pragma unroll
                    for (int grp = 0; grp < 8; ++grp) {
                        const int w0 = (grp & 1) ? (3 * grp - 1) / 2 : (3 * grp) / 2;
                        const uint32_t win = prmt(cw[w0], cw[w0 + 1], (grp & 1) ? sel_odd : sel_even);
                        const uint2 sel = lds_u64((win & win_mask) * win_mul + lut_lane);
                        // byte pools {0, lo, lo, 0} and {0, hi, hi ^ 0x80, 0} of the group's fp16 scale
                        const uint32_t pa = prmt(sw[grp >> 1], 0u, (grp & 1) ? 0x4224u : 0x4004u);
                        const uint32_t pb = prmt(sw[grp >> 1], 0u, (grp & 1) ? 0x4334u : 0x4114u) ^ 0x00800000u;
                        mma_f16(acc[(2 * grp) % kChains], xa[0][grp][0], xa[0][grp][1], xa[0][grp][2], xa[0][grp][3],
                                prmt(pa, pb, sel.x), prmt(pa, pb, sel.x >> 16));
                        mma_f16(acc[(2 * grp + 1) % kChains], xa[1][grp][0], xa[1][grp][1], xa[1][grp][2], xa[1][grp][3],
                                prmt(pa, pb, sel.y), prmt(pa, pb, sel.y >> 16));
                    }
                    float sum[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        sum[i] = acc[0][i];
#pragma unroll
                        for (int c = 1; c < kChains; ++c) sum[i] += acc[c][i];
                    }
                    *reinterpret_cast<float2*>(rbuf + ((0 * 4 + tl) * 32 + lane) * 2) = make_float2(sum[0] * upscale[0], sum[1] * upscale[0]);
                    *reinterpret_cast<float2*>(rbuf + ((1 * 4 + tl) * 32 + lane) * 2) = make_float2(sum[2] * upscale[1], sum[3] * upscale[1]);
                }
            } else {
#pragma unroll
            for (int tl = 0; tl < 4; ++tl) {
                float out[NBLK][2];                                // [block][weight row 2t | 2t+1] of this 8-row tile
#pragma unroll
                for (int blk = 0; blk < NBLK; ++blk) out[blk][0] = out[blk][1] = 0.f;
                const uint32_t ca = stage + (tl * 8 + g) * (cb + 16) + warp * 48;
                const uint32_t sa = stage + kB1Rows * kGemvMaxCodePitch + (tl * 8 + 2 * t) * (sb + 16) + warp * 16;
                const uint4 q0 = lds_u128(ca), q1 = lds_u128(ca + 16), q2 = lds_u128(ca + 32);
                const uint4 s0 = lds_u128(sa), s1 = lds_u128(sa + sb + 16);      // scales of rows 2t and 2t+1 of the tile
                if (tl == 3) {                                     // everything of this stage is in registers now
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_empty + 8 * s);
                }
                const uint32_t cw[12] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w, q2.x, q2.y, q2.z, q2.w};
                const __half2* h0 = reinterpret_cast<const __half2*>(&s0);
                const __half2* h1 = reinterpret_cast<const __half2*>(&s1);
#pragma unroll
                for (int grp = 0; grp < 8; ++grp) {
                    const int w0 = (grp & 1) ? (3 * grp - 1) / 2 : (3 * grp) / 2;
                    const uint32_t win = prmt(cw[w0], cw[w0 + 1], (grp & 1) ? sel_odd : sel_even);
                    const uint32_t nib = lds_u32((win & win_mask) * win_mul + lut_lane);
                    const uint32_t b0 = prmt(kTritBytes, 0u, nib), b1 = prmt(kTritBytes, 0u, nib >> 16);
                    const float f0 = (grp & 1) ? __high2float(h0[grp >> 1]) : __low2float(h0[grp >> 1]);
                    const float f1 = (grp & 1) ? __high2float(h1[grp >> 1]) : __low2float(h1[grp >> 1]);
#pragma unroll
                    for (int blk = 0; blk < NBLK; ++blk) {
                        int d[4];
                        mma_s8_zero(d, xa[blk][grp][0], xa[blk][grp][1], xa[blk][grp][2], xa[blk][grp][3], b0, b1);
                        // d[0], d[1]: high term for weight rows 2t, 2t+1;  d[2], d[3]: low term (same activation row g)
                        out[blk][0] = fmaf((float)(d[0] * 128 + d[2]), f0, out[blk][0]);
                        out[blk][1] = fmaf((float)(d[1] * 128 + d[3]), f1, out[blk][1]);
                    }
                }
#pragma unroll
                for (int blk = 0; blk < NBLK; ++blk)
                    *reinterpret_cast<float2*>(rbuf + ((blk * 4 + tl) * 32 + lane) * 2) =
                        make_float2(out[blk][0] * upscale[blk], out[blk][1] * upscale[blk]);
            }
            }
        } else {
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_empty + 8 * s);
#pragma unroll
            for (int i = 0; i < 4 * NBLK; ++i) *reinterpret_cast<float2*>(rbuf + (i * 32 + lane) * 2) = make_float2(0.f, 0.f);
        }
        if (tid == 0) sts_u128(red_desc + 16 * b, make_uint4((uint32_t)cc.prob, (uint32_t)cc.chunk, (uint32_t)cc.tile, 0u));
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_rfull + 8 * b);
        if (n >= Cfg::kRedLag) reduce_next();
    }
    while (reduced < nitems) reduce_next();

    __syncthreads();
    if (tid == 0 && *abort_flag != 0) atomicCAS(&g_device_status, 0, *abort_flag);
}

template <int NBLK, bool kF16, bool kXF16>
static int32_t launch_gemv_bn(const ojx_e8t_gemv_problem* probs, const ojx_e8t_gemv_problem& single, int count, int total,
                              int M, int y_dtype, const PeerMap& peers, cudaStream_t s) {
    static bool configured = false;
    if (!configured) {
        const cudaError_t e = cudaFuncSetAttribute(gemv_bn_kernel<NBLK, kF16, kXF16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                   (int)BnCfg<NBLK>::kSmem);
        if (e != cudaSuccess) { last_cuda_error() = e; return OJX_ERR_LAUNCH; }
        configured = true;
    }
    const int sms = num_sms();
    const int per = (total + sms - 1) / sms;
    const int grid = (total + per - 1) / per;
    gemv_bn_kernel<NBLK, kF16, kXF16><<<grid, kGemvThreads, BnCfg<NBLK>::kSmem, s>>>(probs, single, count, total, M, y_dtype, peers);
    return launch_status();
}

}  // namespace ojx
