// Decode-shape fused linear: y[M,N] = x[M,K] . dequant(W)[N,K]^T for small M.
//
// Replaces, for small batches, _FusedE8GEMMFunction.forward (ojasx2/math/lattice.py:551-640)
// and the reference's scalar fused kernel (ojasx2/math/csrc/ojasx_math_core.hpp:580-634):
// per (m, n) the result is sum over groups of (sum_k x*coord) * scale, accumulated in fp32.
//
// Fast path (K % 256 == 0, bf16/fp16 activations, M <= 16)
//   * one CTA = 16 warps; warp w owns one 256-wide slice of K and keeps that slice of x in
//     registers as mma.m16n8k16 B fragments, so activations are read once per CTA;
//   * a work item is 16 weight rows x one K chunk (= all slices of the CTA); a producer warp keeps a
//     4-deep ring of items (~16 KB each) in flight with 1-D bulk copies (cp.async.bulk + mbarrier),
//     so ~64 KB per SM is always on its way from HBM; consumer lanes then pick up 48 B of codes +
//     16 B of scales per row with 128-bit shared-memory loads;
//   * a 12-bit rank is turned into eight trits by ONE shared-memory lookup; the table is stored
//     eight times (stride 32 B) so that lanes of different lane%8 never collide on a bank;
//   * trits become +-2.0 / 0 fp16|bf16 operand registers with byte permutes, the MACs run on the
//     tensor cores, and the group scale (times 1/2) is applied to the fp32 fragment per group;
//   * warps' partial sums are combined in a fixed order through shared memory (deterministic), two
//     items late and by a different warp each time, so the loop has no block-wide barrier.
// K larger than one CTA's 16 slices is split into chunks whose fp32 partials go to caller-owned
// scratch and are summed, again in a fixed order, by a second small kernel.
#pragma once

#include "common.cuh"

namespace ojx {

constexpr int kGemvWarps = 16;
constexpr int kGemvThreads = kGemvWarps * 32;
constexpr int kLutEntries = 4096;                                  // any 12-bit code stays in bounds

__host__ __device__ inline int gemv_active_warps(int K) {
    const int slices = K / 256;
    for (int w = kGemvWarps; w > 1; --w)
        if (slices % w == 0) return w;
    return 1;
}
__host__ __device__ inline int gemv_kchunks(int K) { return (K / 256) / gemv_active_warps(K); }
__host__ __device__ inline int gemv_row_tiles(int N) { return (N + 15) / 16; }

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}

template <bool kBf16>
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    if (kBf16) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    } else {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
}

__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

__device__ __forceinline__ void store_any(void* y, int y_dtype, int64_t idx, float v) {
    if (y_dtype == OJX_BF16) static_cast<__nv_bfloat16*>(y)[idx] = __float2bfloat16_rn(v);
    else if (y_dtype == OJX_F16) static_cast<__half*>(y)[idx] = __float2half_rn(v);
    else static_cast<float*>(y)[idx] = v;
}
template <bool kBf16> __device__ __forceinline__ float load_act(const void* p, int64_t idx) {
    if (kBf16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[idx]);
    return __half2float(static_cast<const __half*>(p)[idx]);
}

__device__ __forceinline__ uint4 lds_u128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

// Position of a work item: problem, K chunk, 16-row tile; plus the few per-problem numbers the
// inner loop needs, refreshed only when the problem changes (no divisions per item).
struct Cursor {
    int prob, chunk, tile;
    int N, K, act, tiles, kchunks;
};

__device__ __forceinline__ void cursor_load_problem(Cursor& c, const ojx_e8t_gemv_problem* probs) {
    c.N = probs[c.prob].N;
    c.K = probs[c.prob].K;
    c.act = gemv_active_warps(c.K);
    c.tiles = gemv_row_tiles(c.N);
    c.kchunks = (c.K / 256) / c.act;
}
__device__ __forceinline__ void cursor_seek(Cursor& c, const ojx_e8t_gemv_problem* probs, int count, int item) {
    int p = 0;
    while (p + 1 < count && probs[p + 1].tile_begin <= item) ++p;
    c.prob = p;
    cursor_load_problem(c, probs);
    const int local = item - probs[p].tile_begin;
    c.chunk = local / c.tiles;
    c.tile = local - c.chunk * c.tiles;
}
__device__ __forceinline__ void cursor_next(Cursor& c, const ojx_e8t_gemv_problem* probs, int count) {
    if (++c.tile == c.tiles) {
        c.tile = 0;
        if (++c.chunk == c.kchunks) {
            c.chunk = 0;
            if (c.prob + 1 < count) {
                ++c.prob;
                cursor_load_problem(c, probs);
            }
        }
    }
}

// Shared-memory plan of the fast kernel.
//   lut    COPIES interleaved copies of the rank -> trit-nibble table (entry r, copy c at (r*COPIES + c)*4)
//   ring   kGemvStages work items; an item holds 16 rows of codes (pitch = bytes + 16, so the 8 rows a
//          128-bit load touches fall on distinct banks) followed by 16 rows of scales (same rule)
//   red    kGemvRed buffers of per-warp fragments for the deterministic cross-warp sum
constexpr int kGemvStages = 4;
constexpr int kGemvRed = 4;
constexpr int kGemvRedLag = 2;                              // an item is summed two items after it was computed
constexpr int kGemvMaxCodePitch = kGemvWarps * 48 + 16;     // 784
constexpr int kGemvMaxScalePitch = kGemvWarps * 16 + 16;    // 272
constexpr int kGemvStageBytes = 16 * (kGemvMaxCodePitch + kGemvMaxScalePitch);   // 16896
constexpr int kGemvBlock = kGemvThreads;

template <int NB, int COPIES> constexpr size_t gemv_smem_bytes() {
    return (size_t)kLutEntries * COPIES * 4 + (size_t)kGemvStages * kGemvStageBytes +
           (size_t)kGemvRed * kGemvWarps * 32 * 4 * NB * sizeof(float) + 256;
}

// All 16 warps are symmetric.  For item n (counted from the CTA's first item):
//   * warp (n mod 16) issued its bulk copies kGemvStages-1 items earlier, after waiting for the ring stage
//     to be released by all warps ("empty" barrier);
//   * every warp waits for the bytes ("full" barrier), pulls its rows' slice into registers, releases
//     the stage, decodes and multiplies, and parks its fragment in a reduction buffer ("rfull" barrier);
//   * warp ((n - 2) mod 16) then adds up the sixteen fragments of item n-2 in warp order and writes
//     the outputs ("rempty" barrier frees the buffer).  No block-wide barrier in the loop.
template <bool kBf16, int NB, int COPIES>
__global__ void __launch_bounds__(kGemvBlock, 1)
gemv_mma_kernel(const ojx_e8t_gemv_problem* __restrict__ probs_dev, const __grid_constant__ ojx_e8t_gemv_problem single,
                int count, int total_items, int M, int y_dtype) {
    // A single problem travels by value in the kernel parameters; a list lives in device memory.
    const ojx_e8t_gemv_problem* probs = probs_dev != nullptr ? probs_dev : &single;
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int kLutB = kLutEntries * COPIES * 4;
    constexpr int kRedFloats = kGemvWarps * 32 * 4 * NB;
    uint32_t* lut = reinterpret_cast<uint32_t*>(smem);
    const uint32_t ring = smem_u32(smem) + kLutB;
    float* red = reinterpret_cast<float*>(smem + kLutB + kGemvStages * kGemvStageBytes);
    uint8_t* tail = smem + kLutB + kGemvStages * kGemvStageBytes + kGemvRed * kRedFloats * sizeof(float);
    const uint32_t bar_full = smem_u32(tail), bar_empty = bar_full + 8 * kGemvStages;
    const uint32_t bar_rfull = bar_empty + 8 * kGemvStages, bar_rempty = bar_rfull + 8 * kGemvRed;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tail + 16 * kGemvStages + 16 * kGemvRed);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;

    for (int i = tid; i < kLutEntries * COPIES; i += kGemvBlock) {
        const int r = i / COPIES;
        lut[i] = r < kNumPoints ? g_trit_nibbles[r] : 0u;
    }
    if (tid == 0) {
        for (int s = 0; s < kGemvStages; ++s) {
            mbar_init(bar_full + 8 * s, 1);                 // the issuing lane's expect_tx arrive
            mbar_init(bar_empty + 8 * s, kGemvWarps);       // every warp has pulled its slice
        }
        for (int b = 0; b < kGemvRed; ++b) {
            mbar_init(bar_rfull + 8 * b, kGemvWarps);       // every warp has parked its fragment
            mbar_init(bar_rempty + 8 * b, 1);               // the summing warp is done with the buffer
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    const int64_t per = ((int64_t)total_items + gridDim.x - 1) / gridDim.x;
    const int i0 = (int)min((int64_t)total_items, per * blockIdx.x);
    const int i1 = (int)min((int64_t)total_items, per * (blockIdx.x + 1));
    if (i0 >= i1) return;
    const int nitems = i1 - i0;

    // Bounded wait; once any wait has given up, later waits return at once and the loop runs on (on stale
    // data) so that every barrier keeps its arrival count.  The failure is reported in g_device_status.
    auto wait = [&](uint32_t bar, uint32_t parity, int code) {
        if (*abort_flag == 0) mbar_wait(bar, parity, abort_flag, code);
    };

    // ---- issue: bulk copies of item n into ring stage n mod S ----
    Cursor ic;                                  // cursor of the next item to be issued
    cursor_seek(ic, probs, count, i0);
    int issued = 0;
    auto issue_next = [&]() {
        const int n = issued, s = n % kGemvStages;
        if (warp == (n & (kGemvWarps - 1))) {
            wait(bar_empty + 8 * s, ((uint32_t)(n / kGemvStages) & 1u) ^ 1u, 11);
            const ojx_e8t_gemv_problem& P = probs[ic.prob];
            const uint32_t cb = ic.act * 48, sb = ic.act * 16;
            const int rows = min(16, ic.N - ic.tile * 16);
            const uint32_t stage = ring + s * kGemvStageBytes;
            if (lane == 0) mbar_expect_tx(bar_full + 8 * s, (uint32_t)rows * (cb + sb));
            __syncwarp();
            const int r = lane & 15;
            if (r < rows) {
                const int64_t row = (int64_t)ic.tile * 16 + r;
                if (lane < 16)
                    bulk_load(stage + r * (cb + 16), P.packed + row * ((int64_t)ic.K * 3 / 16) + (int64_t)ic.chunk * cb, cb, bar_full + 8 * s);
                else
                    bulk_load(stage + 16 * kGemvMaxCodePitch + r * (sb + 16),
                              reinterpret_cast<const uint8_t*>(P.scales) + row * ((int64_t)ic.K / 16) + (int64_t)ic.chunk * sb, sb, bar_full + 8 * s);
            }
        }
        ++issued;
        cursor_next(ic, probs, count);
    };
    for (int n = 0; n < kGemvStages - 1 && n < nitems; ++n) issue_next();

    // ---- reduction of item n (done by warp n mod 16, kGemvRedLag items late) ----
    Cursor rc;                                  // cursor of the next item to be summed
    cursor_seek(rc, probs, count, i0);
    int reduced = 0;
    auto reduce_next = [&]() {
        const int n = reduced, b = n % kGemvRed;
        if (warp == (n & (kGemvWarps - 1))) {
            wait(bar_rfull + 8 * b, (uint32_t)(n / kGemvRed) & 1u, 13);
            const float* rbuf = red + (size_t)b * kRedFloats;
            const ojx_e8t_gemv_problem& P = probs[rc.prob];
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
                float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int w = 0; w < kGemvWarps; ++w) {
                    const float4 v = *reinterpret_cast<const float4*>(rbuf + ((size_t)(w * 32 + lane) * NB + nb) * 4);
                    sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
                }
                const float vals[4] = {sum.x * 0.5f, sum.y * 0.5f, sum.z * 0.5f, sum.w * 0.5f};   // operands hold +-2.0
#pragma unroll
                for (int reg = 0; reg < 4; ++reg) {
                    const int row = rc.tile * 16 + g + ((reg >> 1) << 3);
                    const int col = nb * 8 + (t << 1) + (reg & 1);
                    if (row < rc.N && col < M) {
                        float v = vals[reg];
                        if (P.partial != nullptr) {
                            P.partial[((int64_t)rc.chunk * M + col) * rc.N + row] = v;
                        } else {
                            if (P.bias != nullptr) v += load_act<kBf16>(P.bias, row);
                            store_any(P.y, y_dtype, (int64_t)col * rc.N + row, v);
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_rempty + 8 * b);
        }
        ++reduced;
        cursor_next(rc, probs, count);
    };

    // lane-constant decode parameters
    const uint32_t bt = (t == 0) ? 0u : (t == 1) ? 1u : (t == 2) ? 3u : 4u;     // first byte of this lane's rank
    const uint32_t sel_even = bt | ((bt + 1) << 4);
    const uint32_t sel_odd = (bt + 2) | ((bt + 3) << 4);
    constexpr int kEntryShift = COPIES == 8 ? 5 : (COPIES == 4 ? 4 : (COPIES == 2 ? 3 : 2));   // log2(COPIES * 4)
    const uint32_t lsh = (t & 1) ? (uint32_t)(kEntryShift - 4) : (uint32_t)kEntryShift;
    constexpr uint32_t kEntryMask = 0xFFFu << kEntryShift;
    const uint32_t lut_lane = smem_u32(lut) + ((lane & (COPIES - 1)) << 2);
    constexpr uint32_t kConstH = 0x00C04000u;                     // byte 1: +2.0 high byte, byte 2: -2.0

    uint32_t xf[NB][8][4];
    int cur_prob = -1, cur_chunk = -1;
    Cursor cc;
    cursor_seek(cc, probs, count, i0);
    for (int n = 0; n < nitems; ++n) {
        const int s = n % kGemvStages, b = n % kGemvRed;
        if (issued < nitems) issue_next();                       // keeps kGemvStages-1 items in flight

        // (re)load this warp's activations when the problem or the K chunk changes
        if (cc.prob != cur_prob || cc.chunk != cur_chunk) {
            cur_prob = cc.prob;
            cur_chunk = cc.chunk;
            if (warp < cc.act) {
                const uint16_t* xp = static_cast<const uint16_t*>(probs[cc.prob].x);
                const int slice = cc.chunk * cc.act + warp;
#pragma unroll
                for (int nb = 0; nb < NB; ++nb) {
                    const int m = nb * 8 + g;
#pragma unroll
                    for (int grp = 0; grp < 8; ++grp) {
                        uint4 v = make_uint4(0, 0, 0, 0);
                        if (m < M) v = __ldg(reinterpret_cast<const uint4*>(xp + (int64_t)m * cc.K + slice * 256 + grp * 32 + t * 8));
                        xf[nb][grp][0] = v.x; xf[nb][grp][1] = v.y; xf[nb][grp][2] = v.z; xf[nb][grp][3] = v.w;
                    }
                }
            }
        }

        wait(bar_full + 8 * s, (uint32_t)(n / kGemvStages) & 1u, 12);

        float acc[NB][4];
#pragma unroll
        for (int nb = 0; nb < NB; ++nb)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[nb][i] = 0.f;

        if (warp < cc.act) {
            const uint32_t cb = cc.act * 48, sb = cc.act * 16;
            const uint32_t stage = ring + s * kGemvStageBytes;
            const uint32_t ca_addr = stage + g * (cb + 16) + warp * 48, cb_addr = ca_addr + 8 * (cb + 16);
            const uint32_t sa_addr = stage + 16 * kGemvMaxCodePitch + g * (sb + 16) + warp * 16, sb_addr = sa_addr + 8 * (sb + 16);
            uint4 qa[3] = {lds_u128(ca_addr), lds_u128(ca_addr + 16), lds_u128(ca_addr + 32)};
            uint4 qb[3] = {lds_u128(cb_addr), lds_u128(cb_addr + 16), lds_u128(cb_addr + 32)};
            uint4 qsa = lds_u128(sa_addr), qsb = lds_u128(sb_addr);
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_empty + 8 * s);           // the stage may be refilled
            const uint32_t* ca = reinterpret_cast<const uint32_t*>(qa);
            const uint32_t* cbw = reinterpret_cast<const uint32_t*>(qb);
            const __half2* sa = reinterpret_cast<const __half2*>(&qsa);
            const __half2* sbh = reinterpret_cast<const __half2*>(&qsb);
#pragma unroll
            for (int grp = 0; grp < 8; ++grp) {
                const int w0 = (grp & 1) ? (3 * grp - 1) / 2 : (3 * grp) / 2;
                const uint32_t sel = (grp & 1) ? sel_odd : sel_even;
                const uint32_t wa = prmt(ca[w0], ca[w0 + 1], sel);
                const uint32_t wb = prmt(cbw[w0], cbw[w0 + 1], sel);
                const uint32_t na_ = lds_u32(((wa << lsh) & kEntryMask) + lut_lane);
                const uint32_t nb_ = lds_u32(((wb << lsh) & kEntryMask) + lut_lane);
                const uint32_t ha_lo = prmt(kConstH, 0u, na_), ha_hi = prmt(kConstH, 0u, na_ >> 16);
                const uint32_t hb_lo = prmt(kConstH, 0u, nb_), hb_hi = prmt(kConstH, 0u, nb_ >> 16);
                uint32_t a1[4], a2[4];
                a1[0] = prmt(ha_lo, 0u, 0x1404u); a1[2] = prmt(ha_lo, 0u, 0x3424u);
                a1[1] = prmt(hb_lo, 0u, 0x1404u); a1[3] = prmt(hb_lo, 0u, 0x3424u);
                a2[0] = prmt(ha_hi, 0u, 0x1404u); a2[2] = prmt(ha_hi, 0u, 0x3424u);
                a2[1] = prmt(hb_hi, 0u, 0x1404u); a2[3] = prmt(hb_hi, 0u, 0x3424u);
                const float fa = (grp & 1) ? __high2float(sa[grp >> 1]) : __low2float(sa[grp >> 1]);
                const float fb = (grp & 1) ? __high2float(sbh[grp >> 1]) : __low2float(sbh[grp >> 1]);
#pragma unroll
                for (int nb = 0; nb < NB; ++nb) {
                    float d[4] = {0.f, 0.f, 0.f, 0.f};
                    mma16816<kBf16>(d, a1, xf[nb][grp][0], xf[nb][grp][1]);
                    mma16816<kBf16>(d, a2, xf[nb][grp][2], xf[nb][grp][3]);
                    acc[nb][0] = fmaf(d[0], fa, acc[nb][0]);
                    acc[nb][1] = fmaf(d[1], fa, acc[nb][1]);
                    acc[nb][2] = fmaf(d[2], fb, acc[nb][2]);
                    acc[nb][3] = fmaf(d[3], fb, acc[nb][3]);
                }
            }
        } else {
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_empty + 8 * s);
        }

        // park this warp's fragment; the sum over warps happens kGemvRedLag items later
        wait(bar_rempty + 8 * b, ((uint32_t)(n / kGemvRed) & 1u) ^ 1u, 14);
        float* rbuf = red + (size_t)b * kRedFloats;
#pragma unroll
        for (int nb = 0; nb < NB; ++nb)
            *reinterpret_cast<float4*>(rbuf + ((size_t)(warp * 32 + lane) * NB + nb) * 4) =
                make_float4(acc[nb][0], acc[nb][1], acc[nb][2], acc[nb][3]);
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_rfull + 8 * b);
        if (n >= kGemvRedLag) reduce_next();
        cursor_next(cc, probs, count);
    }
    while (reduced < nitems) reduce_next();

    __syncthreads();
    if (tid == 0 && *abort_flag != 0) {
        // copies that were issued but never consumed get a bounded time to land before shared memory is released
        for (int s = 0; s < kGemvStages; ++s)
            for (uint32_t i = 0; i < (1u << 16); ++i)
                if (mbar_try_wait(bar_full + 8 * s, 0) || mbar_try_wait(bar_full + 8 * s, 1)) break;
        atomicCAS(&g_device_status, 0, *abort_flag);
    }
}

// Sums the K-chunk partials of every problem that has them (fixed order), adds bias, casts.
template <bool kBf16>
__global__ void __launch_bounds__(256) gemv_reduce_kernel(const ojx_e8t_gemv_problem* __restrict__ probs_dev,
                                                           const __grid_constant__ ojx_e8t_gemv_problem single,
                                                           int count, int M, int y_dtype) {
    const ojx_e8t_gemv_problem* probs = probs_dev != nullptr ? probs_dev : &single;
    for (int p = blockIdx.y; p < count; p += gridDim.y) {
        const ojx_e8t_gemv_problem& P = probs[p];
        if (P.partial == nullptr) continue;
        const int kc = gemv_kchunks(P.K);
        const int64_t total = (int64_t)M * P.N;
        for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
             i += (int64_t)gridDim.x * blockDim.x) {
            float s = 0.f;
            for (int c = 0; c < kc; ++c) s += P.partial[(int64_t)c * total + i];
            if (P.bias != nullptr) s += load_act<kBf16>(P.bias, i % P.N);
            store_any(P.y, y_dtype, i, s);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Generic path: any N, K (flat packing where groups may cross rows included), any dtypes.
// One warp per output feature; correctness path for shapes the fast kernels do not cover.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float load_any(const void* p, int dt, int64_t i) {
    if (dt == OJX_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
    if (dt == OJX_F16) return __half2float(static_cast<const __half*>(p)[i]);
    return static_cast<const float*>(p)[i];
}

__global__ void __launch_bounds__(256) generic_linear_kernel(const void* __restrict__ x, int x_dtype, int64_t M,
                                                              const uint8_t* __restrict__ packed,
                                                              const uint16_t* __restrict__ scales,
                                                              const void* __restrict__ bias, int64_t N, int64_t K,
                                                              int group, void* __restrict__ y, int y_dtype) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t n = warp; n < N; n += nwarps) {
        for (int64_t m0 = 0; m0 < M; m0 += 8) {
            float acc[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = 0.f;
            for (int64_t k = lane; k < K; k += 32) {
                const int64_t flat = n * K + k;
                const int64_t code_idx = flat >> 3;
                const uint8_t* tp = packed + (code_idx >> 1) * 3;
                uint32_t c0, c1;
                triplet_to_codes(tp[0], tp[1], tp[2], c0, c1);
                uint32_t code = (code_idx & 1) ? c1 : c0;
                code = min(code, (uint32_t)(kNumPoints - 1));
                const float w = (float)nibble_coord(g_trit_nibbles[code], (int)(flat & 7)) *
                                __half2float(__ushort_as_half(scales[flat / group]));
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if (m0 + j < M) acc[j] = fmaf(load_any(x, x_dtype, (m0 + j) * K + k), w, acc[j]);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                float v = acc[j];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
                if (lane == 0 && m0 + j < M) {
                    if (bias != nullptr) v += load_any(bias, x_dtype, n);
                    store_any(y, y_dtype, (m0 + j) * N + n, v);
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
inline bool gemv_fast_ok(int64_t M, int64_t N, int64_t K, int group, int x_dtype) {
    return M >= 1 && M <= 16 && K % 256 == 0 && group == 32 && (x_dtype == OJX_BF16 || x_dtype == OJX_F16) &&
           N >= 1 && N < (1 << 30) && K < (1 << 30);
}

int32_t gemv_tiles_impl(int64_t N, int64_t K) {
    if (N <= 0 || K <= 0 || K % 256 != 0) return 0;
    return gemv_row_tiles((int)N) * gemv_kchunks((int)K);
}
int32_t gemv_kchunks_impl(int64_t K) { return (K > 0 && K % 256 == 0) ? gemv_kchunks((int)K) : 0; }

// Scratch of the single-problem entry point: fp32 partials [kchunks][M][N], needed only when K
// spans more than one chunk of the CTA's 16 slices.
size_t gemv_workspace_bytes_impl(int64_t M, int64_t N, int64_t K) {
    if (M <= 0 || M > 16 || N <= 0 || K <= 0 || K % 256 != 0) return 0;
    const int kc = gemv_kchunks((int)K);
    return kc > 1 ? (size_t)kc * M * N * sizeof(float) : 0;
}

static int g_num_sms = 0;
static int num_sms() {
    if (g_num_sms == 0) {
        int dev = 0, n = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        g_num_sms = n > 0 ? n : 148;
    }
    return g_num_sms;
}

template <bool kBf16, int NB>
static int32_t launch_gemv(const ojx_e8t_gemv_problem* probs, const ojx_e8t_gemv_problem& single, int count, int total,
                           int M, int y_dtype, cudaStream_t s) {
    static bool configured = false;
    constexpr int COPIES = NB == 1 ? 8 : 4;
    const size_t smem = gemv_smem_bytes<NB, COPIES>();
    if (!configured) {
        const cudaError_t e = cudaFuncSetAttribute(gemv_mma_kernel<kBf16, NB, COPIES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) { last_cuda_error() = e; return OJX_ERR_LAUNCH; }
        configured = true;
    }
    const int sms = num_sms();
    const int per = (total + sms - 1) / sms;
    const int grid = (total + per - 1) / per;
    gemv_mma_kernel<kBf16, NB, COPIES><<<grid, kGemvBlock, smem, s>>>(probs, single, count, total, M, y_dtype);
    return launch_status();
}

int32_t gemv_grouped_impl(const ojx_e8t_gemv_problem* problems, int count, int total_tiles, int64_t M,
                          int x_dtype, int y_dtype, int needs_reduce, cudaStream_t s) {
    OJX_RETURN_IF(!problems, OJX_ERR_NULL);
    OJX_RETURN_IF(count <= 0 || total_tiles <= 0 || M < 1 || M > 16, OJX_ERR_SHAPE);
    OJX_RETURN_IF(x_dtype != OJX_BF16 && x_dtype != OJX_F16, OJX_ERR_DTYPE);
    OJX_RETURN_IF(y_dtype != OJX_BF16 && y_dtype != OJX_F16 && y_dtype != OJX_F32, OJX_ERR_DTYPE);
    OJX_RETURN_IF(check_arch() != OJX_OK, OJX_ERR_ARCH);
    int32_t st;
    const bool bf = x_dtype == OJX_BF16;
    ojx_e8t_gemv_problem none = {};
    if (M <= 8) st = bf ? launch_gemv<true, 1>(problems, none, count, total_tiles, (int)M, y_dtype, s)
                        : launch_gemv<false, 1>(problems, none, count, total_tiles, (int)M, y_dtype, s);
    else st = bf ? launch_gemv<true, 2>(problems, none, count, total_tiles, (int)M, y_dtype, s)
                 : launch_gemv<false, 2>(problems, none, count, total_tiles, (int)M, y_dtype, s);
    OJX_RETURN_IF(st != OJX_OK, st);
    if (!needs_reduce) return OJX_OK;
    // Problems whose K spans several chunks carry a partial buffer; the reduce pass skips the rest.
    dim3 grid(64, count > 64 ? 64 : count);
    if (bf) gemv_reduce_kernel<true><<<grid, 256, 0, s>>>(problems, none, count, (int)M, y_dtype);
    else gemv_reduce_kernel<false><<<grid, 256, 0, s>>>(problems, none, count, (int)M, y_dtype);
    return launch_status();
}

int32_t gemv_impl(const void* x, int x_dtype, int64_t M, const uint8_t* packed, const uint16_t* scales,
                  const void* bias, int64_t N, int64_t K, int group, void* y, int y_dtype,
                  void* workspace, size_t workspace_bytes, cudaStream_t s) {
    OJX_RETURN_IF(!x || !packed || !scales || !y, OJX_ERR_NULL);
    OJX_RETURN_IF(M <= 0 || N <= 0 || K <= 0, OJX_ERR_SHAPE);
    OJX_RETURN_IF(dtype_size(x_dtype) == 0 || dtype_size(y_dtype) == 0, OJX_ERR_DTYPE);
    OJX_RETURN_IF(check_arch() != OJX_OK, OJX_ERR_ARCH);
    group = effective_group(group);
    const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(packed) |
                           reinterpret_cast<uintptr_t>(scales)) & 15) == 0;
    if (gemv_fast_ok(M, N, K, group, x_dtype) && aligned) {
        const size_t need = gemv_workspace_bytes_impl(M, N, K);
        OJX_RETURN_IF(need > 0 && (!workspace || workspace_bytes < need), OJX_ERR_WORKSPACE);
        OJX_RETURN_IF(need > 0 && (reinterpret_cast<uintptr_t>(workspace) & 15) != 0, OJX_ERR_ALIGN);
        ojx_e8t_gemv_problem h;
        h.x = x; h.packed = packed; h.scales = scales; h.bias = bias; h.y = y;
        const int kc = gemv_kchunks((int)K);
        h.partial = kc > 1 ? static_cast<float*>(workspace) : nullptr;
        h.N = (int)N; h.K = (int)K; h.tile_begin = 0; h.reserved = 0;
        const int total = gemv_row_tiles((int)N) * kc;
        int32_t st;
        const bool bf = x_dtype == OJX_BF16;
        if (M <= 8) st = bf ? launch_gemv<true, 1>(nullptr, h, 1, total, (int)M, y_dtype, s) : launch_gemv<false, 1>(nullptr, h, 1, total, (int)M, y_dtype, s);
        else st = bf ? launch_gemv<true, 2>(nullptr, h, 1, total, (int)M, y_dtype, s) : launch_gemv<false, 2>(nullptr, h, 1, total, (int)M, y_dtype, s);
        OJX_RETURN_IF(st != OJX_OK, st);
        if (kc > 1) {
            dim3 grid(64, 1);
            if (bf) gemv_reduce_kernel<true><<<grid, 256, 0, s>>>(nullptr, h, 1, (int)M, y_dtype);
            else gemv_reduce_kernel<false><<<grid, 256, 0, s>>>(nullptr, h, 1, (int)M, y_dtype);
        }
        return launch_status();
    }
    // generic path
    int64_t warps_needed = N;
    int64_t blocks = (warps_needed * 32 + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    generic_linear_kernel<<<(unsigned)blocks, 256, 0, s>>>(x, x_dtype, M, packed, scales, bias, N, K, group, y, y_dtype);
    return launch_status();
}

}  // namespace ojx
