// Decode GEMV for ONE activation row (M == 1, bf16): the path that is driven to HBM rate.
//
//   y[n] = sum_k x[k] * coord[n,k] * scale[n, k/32]  (+ bias)          fp32 result, cast on store
//
// Work decomposition (same as the multi-row kernel in gemv.cuh): a CTA of 16 warps walks a contiguous
// range of work items; an item is 32 weight rows x one K chunk, warp w owns the 256-wide slice w of the
// chunk.  Items stream HBM -> shared memory through a 5-stage ring of 16-byte cp.async copies (three
// items always in flight), completion counted on mbarriers.
//
// What makes this path cheap per weight:
//   * int8 tensor-core MACs (mma.sync.m16n8k32.s8, native on sm_100a).  A ternary coordinate is one
//     byte, so a rank's eight trits become the lane's two A registers with two byte permutes of a
//     4-bit-selector word fetched by ONE shared-memory lookup; nothing is widened to 16 bits.
//   * A lane owns 8 consecutive ranks of a row (12 contiguous bytes): no redundant loads, compile-time
//     bit positions.
//   * The eight accumulator columns serve as eight SCALE GROUPS instead of eight batch rows: lane
//     (g, t) feeds x only into column 2t + (step >> 2), so after the sixteen MMAs of a row tile column
//     n holds the integer partial sum of group n.  Group scales are then applied once per tile (not per
//     step) and the four lanes sharing a row are combined with two shuffles.
//   * Activations are quantised once per CTA and slice to 13-bit fixed point relative to the slice's
//     absolute maximum, X = rint(x * 2^-e) = 128 * hi + lo with int8 hi, lo; the two MMAs (hi, lo) share
//     the decoded weights and integer accumulation is exact.  Elements within 2^-5 of the slice maximum
//     are represented exactly, smaller ones to within 2^-13 of that maximum - a relative-L2 contribution
//     of ~1e-4 against the 2e-3 contract (the bf16 output rounding alone is 1.7e-3).
//   * Warps never meet at a block-wide barrier inside the loop; partial sums are combined in warp order
//     (deterministic) by a rotating warp two items late.
#pragma once

#include "gemv.cuh"

namespace ojx {

constexpr int kB1Rows = 32;                                   // weight rows per work item
constexpr int kB1Stages = 5;
constexpr int kB1Ahead = 3;
constexpr int kB1Red = 4;
constexpr int kB1RedLag = 2;
constexpr int kB1Copies = 4;                                  // interleaved copies of the lookup table
// Only the 3281 real entries are stored; a corrupt 12-bit rank (up to 4095) would read at most 64 KB past
// the table start, which is still inside this kernel's shared-memory allocation (ring and buffers follow).
constexpr int kB1LutBytes = ((kNumPoints * kB1Copies * 4 + 1023) / 1024) * 1024;   // 53248
constexpr int kB1StageBytes = kB1Rows * (kGemvMaxCodePitch + kGemvMaxScalePitch);   // 33792
constexpr int kB1RedFloats = kGemvWarps * kB1Rows;            // 512 floats per buffer
constexpr size_t kB1SmemBytes = (size_t)kB1LutBytes + (size_t)kB1Stages * kB1StageBytes +
                                (size_t)kB1Red * kB1RedFloats * sizeof(float) + 256;

__host__ __device__ inline int b1_row_tiles(int N) { return (N + kB1Rows - 1) / kB1Rows; }

__device__ __forceinline__ void mma_s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Slow path of a bounded wait, kept out of line so the loop body stays small.
__device__ __noinline__ void b1_wait_slow(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code) {
    if (*abort_flag != 0) return;               // some wait already gave up: run on so that barrier counts stay matched
    mbar_wait(bar, parity, abort_flag, code);
}
__device__ __forceinline__ void b1_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code) {
    if (!mbar_try_wait(bar, parity)) b1_wait_slow(bar, parity, abort_flag, code);
}

struct B1Cursor {
    int prob, chunk, tile;          // position
    int N, K, act, tiles, kchunks;  // of the current problem
};
__device__ __forceinline__ void b1_load_problem(B1Cursor& c, const ojx_e8t_gemv_problem* probs) {
    c.N = probs[c.prob].N;
    c.K = probs[c.prob].K;
    c.act = gemv_active_warps(c.K);
    c.tiles = b1_row_tiles(c.N);
    c.kchunks = (c.K / 256) / c.act;
}
__device__ __forceinline__ void b1_seek(B1Cursor& c, const ojx_e8t_gemv_problem* probs, int p, int item) {
    c.prob = p;
    b1_load_problem(c, probs);
    const int local = item - probs[p].tile_begin;
    c.chunk = local / c.tiles;
    c.tile = local - c.chunk * c.tiles;
}
__device__ __forceinline__ void b1_next(B1Cursor& c, const ojx_e8t_gemv_problem* probs, int count) {
    if (++c.tile == c.tiles) {
        c.tile = 0;
        if (++c.chunk == c.kchunks) {
            c.chunk = 0;
            if (c.prob + 1 < count) {
                ++c.prob;
                b1_load_problem(c, probs);
            }
        }
    }
}

__global__ void __launch_bounds__(kGemvThreads, 1)
gemv_b1_kernel(const ojx_e8t_gemv_problem* __restrict__ probs_dev, const __grid_constant__ ojx_e8t_gemv_problem single,
               int count, int total_items, int y_dtype, const __grid_constant__ PeerMap peers) {
    const ojx_e8t_gemv_problem* probs = probs_dev != nullptr ? probs_dev : &single;
    extern __shared__ __align__(128) uint8_t smem[];
    uint32_t* lut = reinterpret_cast<uint32_t*>(smem);
    const uint32_t ring = smem_u32(smem) + kB1LutBytes;
    float* red = reinterpret_cast<float*>(smem + kB1LutBytes + kB1Stages * kB1StageBytes);
    uint8_t* tail = smem + kB1LutBytes + kB1Stages * kB1StageBytes + kB1Red * kB1RedFloats * sizeof(float);
    const uint32_t bar_full = smem_u32(tail), bar_empty = bar_full + 8 * kB1Stages;
    const uint32_t bar_rfull = bar_empty + 8 * kB1Stages, bar_rempty = bar_rfull + 8 * kB1Red;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tail + 16 * kB1Stages + 16 * kB1Red);
    const uint32_t bar_lut = smem_u32(tail) + 16 * kB1Stages + 16 * kB1Red + 16;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;

    if (tid == 0) {
        for (int s = 0; s < kB1Stages; ++s) {
            mbar_init(bar_full + 8 * s, kGemvThreads);      // every thread's cp.async arrive
            mbar_init(bar_empty + 8 * s, kGemvWarps);       // every warp has pulled its slice
        }
        for (int b = 0; b < kB1Red; ++b) {
            mbar_init(bar_rfull + 8 * b, kGemvWarps);       // every warp has parked its partial sums
            mbar_init(bar_rempty + 8 * b, 1);               // the summing warp is done with the buffer
        }
        mbar_init(bar_lut, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        // the lookup table's shared-memory image (every entry four times) arrives as ONE bulk copy while the kernel
        // sets itself up; nobody builds it
        mbar_expect_tx(bar_lut, kNumPoints * 16);
        bulk_load(smem_u32(lut), g_lut_i8x4, kNumPoints * 16, bar_lut);
    }
    __syncthreads();

    const int64_t per = ((int64_t)total_items + gridDim.x - 1) / gridDim.x;
    const int i0 = (int)min((int64_t)total_items, per * blockIdx.x);
    const int i1 = (int)min((int64_t)total_items, per * (blockIdx.x + 1));
    if (i0 >= i1) return;
    const int nitems = i1 - i0;
    const int p0 = find_problem(probs, count, i0, 1);

    // ---- loader: thread (lr, ls) copies chunks ls, ls+16, ls+32 of row lr's codes and chunk ls of its scales ----
    const int lr = tid >> 4, ls = tid & 15;
    B1Cursor ic;
    b1_seek(ic, probs, p0, i0);
    const B1Cursor first = ic;                                     // the other two cursors start from the same item
    int issued = 0;
    auto issue_next = [&]() {
        const int n = issued, s = n % kB1Stages;
        b1_wait(bar_empty + 8 * s, ((uint32_t)(n / kB1Stages) & 1u) ^ 1u, abort_flag, 31);
        const int row = ic.tile * kB1Rows + lr;
        if (row < ic.N) {
            const ojx_e8t_gemv_problem& P = probs[ic.prob];
            const int cchunks = 3 * ic.act;                          // 16-byte chunks of codes per row and K chunk
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
        cp_async_arrive(bar_full + 8 * s);
        ++issued;
        b1_next(ic, probs, count);
    };
    for (int n = 0; n < kB1Ahead && n < nitems; ++n) issue_next();


    // ---- reduction of item n by warp n mod 16, kB1RedLag items after it was computed ----
    B1Cursor rc = first;
    int reduced = 0;
    auto reduce_next = [&]() {
        const int n = reduced, b = n % kB1Red;
        if (warp == (n & (kGemvWarps - 1))) {
            b1_wait(bar_rfull + 8 * b, (uint32_t)(n / kB1Red) & 1u, abort_flag, 33);
            const float* rbuf = red + (size_t)b * kB1RedFloats;
            float sum = 0.f;
#pragma unroll
            for (int w = 0; w < kGemvWarps; ++w) sum += rbuf[w * kB1Rows + lane];
            const int row = rc.tile * kB1Rows + lane;
            if (row < rc.N) {
                const ojx_e8t_gemv_problem& P = probs[rc.prob];
                if (P.partial != nullptr) P.partial[(int64_t)rc.chunk * rc.N + row] = sum;
                else {
                    if (P.bias != nullptr) sum += __bfloat162float(static_cast<const __nv_bfloat16*>(P.bias)[row]);
                    store_any(P.y, y_dtype, row, sum);
                    if (peers.world > 1) store_peers(peers, P.y, y_dtype, row, sum);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_rempty + 8 * b);
        }
        ++reduced;
        b1_next(rc, probs, count);
    };

    // ---- lane constants ----
    const uint32_t lut_lane = smem_u32(lut) + ((lane & (kB1Copies - 1)) << 2);
    constexpr uint32_t kTritBytes = 0x00FF0100u;      // selector 0 -> 0, 1 -> +1, 2 -> -1 (int8)
    constexpr uint32_t kEntryMask = 0xFFFu << 4;      // rank * 16 = byte offset of a table entry (4 copies x 4 bytes)

    uint32_t xh[8][2], xl[8][2];                      // int8 activation fragments (hi, lo) for the 8 steps
    float upscale = 1.f;                              // 2^e of this warp's slice
    int cur_prob = -1, cur_chunk = -1;
    B1Cursor cc = first;

    b1_wait(bar_lut, 0u, abort_flag, 35);                          // the table has landed
    for (int n = 0; n < nitems; ++n) {
        const int s = n % kB1Stages, b = n % kB1Red;
        if (issued < nitems) issue_next();                         // keeps kB1Ahead items in flight

        if (cc.prob != cur_prob || cc.chunk != cur_chunk) {
            // Quantise this warp's 256 activations.  Every lane converts the eight it loads (one 16-byte load) and
            // the MMA fragments are then handed out by shuffles: lane (g, t) with g >> 1 == t owns
            // x[64t + 32(g&1) + 0..31], i.e. what lanes 8t + 4(g&1) + 0..3 converted.
            cur_prob = cc.prob;
            cur_chunk = cc.chunk;
            const bool live = warp < cc.act;
            const uint16_t* xp = static_cast<const uint16_t*>(probs[cc.prob].x) + (cc.chunk * cc.act + warp) * 256 + lane * 8;
            uint4 q = make_uint4(0, 0, 0, 0);
            if (live) q = __ldg(reinterpret_cast<const uint4*>(xp));
            const uint32_t w[4] = {q.x, q.y, q.z, q.w};
            float v[8];
            float amax = 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                v[2 * i] = __uint_as_float(w[i] << 16);
                v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
                amax = fmaxf(amax, fmaxf(fabsf(v[2 * i]), fabsf(v[2 * i + 1])));
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
            int e = 0;
            if (amax > 0.f) e = max(-100, min(100, (int)((__float_as_uint(amax) >> 23) & 0xFFu) - 127 - 12));
            const float down = __uint_as_float((uint32_t)(127 - e) << 23);
            upscale = __uint_as_float((uint32_t)(127 + e) << 23);
            uint32_t hw[2] = {0u, 0u}, lw[2] = {0u, 0u};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int X = __float2int_rn(v[i] * down);                         // |X| < 8192
                const int hi = (X + 64) >> 7, lo = X - (hi << 7);                 // X = 128 hi + lo, lo in [-64, 63]
                hw[i >> 2] |= (uint32_t)(hi & 0xFF) << (8 * (i & 3));
                lw[i >> 2] |= (uint32_t)(lo & 0xFF) << (8 * (i & 3));
            }
            const bool owner = (g >> 1) == t;
            const int src = 8 * t + 4 * (g & 1);
#pragma unroll
            for (int j = 0; j < 4; ++j) {                                          // steps 0-3 feed group 2t, steps 4-7 group 2t+1
                const uint32_t h0 = __shfl_sync(0xFFFFFFFFu, hw[0], src + j), h1 = __shfl_sync(0xFFFFFFFFu, hw[1], src + j);
                const uint32_t l0 = __shfl_sync(0xFFFFFFFFu, lw[0], src + j), l1 = __shfl_sync(0xFFFFFFFFu, lw[1], src + j);
                const bool lo_half = owner && (g & 1) == 0, hi_half = owner && (g & 1) == 1;
                xh[j][0] = lo_half ? h0 : 0u; xh[j][1] = lo_half ? h1 : 0u;
                xl[j][0] = lo_half ? l0 : 0u; xl[j][1] = lo_half ? l1 : 0u;
                xh[j + 4][0] = hi_half ? h0 : 0u; xh[j + 4][1] = hi_half ? h1 : 0u;
                xl[j + 4][0] = hi_half ? l0 : 0u; xl[j + 4][1] = hi_half ? l1 : 0u;
            }
        }

        b1_wait(bar_full + 8 * s, (uint32_t)(n / kB1Stages) & 1u, abort_flag, 32);

        float out[2][2] = {{0.f, 0.f}, {0.f, 0.f}};               // [row tile][row g | row g+8]
        if (warp < cc.act) {
            const uint32_t cb = cc.act * 48, sb = cc.act * 16;
            const uint32_t stage = ring + s * kB1StageBytes;
            uint32_t cw[2][2][3], sw[2][2];                        // [row tile][row g | g+8][word]
#pragma unroll
            for (int rt = 0; rt < 2; ++rt)
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int r = rt * 16 + h * 8 + g;
                    const uint32_t ca = stage + r * (cb + 16) + warp * 48 + t * 12;
                    cw[rt][h][0] = lds_u32(ca); cw[rt][h][1] = lds_u32(ca + 4); cw[rt][h][2] = lds_u32(ca + 8);
                    sw[rt][h] = lds_u32(stage + kB1Rows * kGemvMaxCodePitch + r * (sb + 16) + warp * 16 + t * 4);
                }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_empty + 8 * s);         // the stage may be refilled
            int dh[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}}, dl[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}};
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int bit = 12 * j, w = bit >> 5, sh = bit & 31;
#pragma unroll
                for (int rt = 0; rt < 2; ++rt) {
                    uint32_t ra, rb;                               // rank * 16 straight from the packed words
                    if (sh + 12 <= 32) {
                        ra = sh >= 4 ? (cw[rt][0][w] >> (sh - 4)) : (cw[rt][0][w] << (4 - sh));
                        rb = sh >= 4 ? (cw[rt][1][w] >> (sh - 4)) : (cw[rt][1][w] << (4 - sh));
                    } else {
                        ra = __funnelshift_r(cw[rt][0][w], cw[rt][0][w + 1 < 3 ? w + 1 : 2], sh - 4);
                        rb = __funnelshift_r(cw[rt][1][w], cw[rt][1][w + 1 < 3 ? w + 1 : 2], sh - 4);
                    }
                    const uint32_t na = lds_u32((ra & kEntryMask) + lut_lane);
                    const uint32_t nb = lds_u32((rb & kEntryMask) + lut_lane);
                    const uint32_t a0 = prmt(kTritBytes, 0u, na), a2 = prmt(kTritBytes, 0u, na >> 16);
                    const uint32_t a1 = prmt(kTritBytes, 0u, nb), a3 = prmt(kTritBytes, 0u, nb >> 16);
                    mma_s8(dh[rt], a0, a1, a2, a3, xh[j][0], xh[j][1]);
                    mma_s8(dl[rt], a0, a1, a2, a3, xl[j][0], xl[j][1]);
                }
            }
#pragma unroll
            for (int rt = 0; rt < 2; ++rt) {
                const __half2 s0 = *reinterpret_cast<const __half2*>(&sw[rt][0]), s1 = *reinterpret_cast<const __half2*>(&sw[rt][1]);
                // columns 2t, 2t+1 of this lane = groups 2t, 2t+1 of rows g (regs 0,1) and g+8 (regs 2,3)
                const float f0 = (float)(dh[rt][0] * 128 + dl[rt][0]), f1 = (float)(dh[rt][1] * 128 + dl[rt][1]);
                const float f2 = (float)(dh[rt][2] * 128 + dl[rt][2]), f3 = (float)(dh[rt][3] * 128 + dl[rt][3]);
                float oa = fmaf(f0, __low2float(s0), f1 * __high2float(s0));
                float ob = fmaf(f2, __low2float(s1), f3 * __high2float(s1));
                oa += __shfl_xor_sync(0xFFFFFFFFu, oa, 1);
                ob += __shfl_xor_sync(0xFFFFFFFFu, ob, 1);
                oa += __shfl_xor_sync(0xFFFFFFFFu, oa, 2);
                ob += __shfl_xor_sync(0xFFFFFFFFu, ob, 2);
                out[rt][0] = oa * upscale;
                out[rt][1] = ob * upscale;
            }
        } else {
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_empty + 8 * s);
        }

        b1_wait(bar_rempty + 8 * b, ((uint32_t)(n / kB1Red) & 1u) ^ 1u, abort_flag, 34);
        if (t == 0) {
            float* rbuf = red + (size_t)b * kB1RedFloats + warp * kB1Rows;
            rbuf[g] = out[0][0]; rbuf[g + 8] = out[0][1]; rbuf[16 + g] = out[1][0]; rbuf[24 + g] = out[1][1];
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_rfull + 8 * b);
        if (n >= kB1RedLag) reduce_next();
        b1_next(cc, probs, count);
    }
    while (reduced < nitems) reduce_next();

    __syncthreads();
    if (tid == 0 && *abort_flag != 0) atomicCAS(&g_device_status, 0, *abort_flag);
}

static int32_t launch_gemv_b1(const ojx_e8t_gemv_problem* probs, const ojx_e8t_gemv_problem& single, int count, int total,
                              int y_dtype, const PeerMap& peers, cudaStream_t s) {
    static bool configured = false;
    if (!configured) {
        const cudaError_t e = cudaFuncSetAttribute(gemv_b1_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kB1SmemBytes);
        if (e != cudaSuccess) { last_cuda_error() = e; return OJX_ERR_LAUNCH; }
        configured = true;
    }
    const int sms = num_sms();
    const int per = (total + sms - 1) / sms;
    const int grid = (total + per - 1) / per;
    gemv_b1_kernel<<<grid, kGemvThreads, kB1SmemBytes, s>>>(probs, single, count, total, y_dtype, peers);
    return launch_status();
}

}  // namespace ojx
