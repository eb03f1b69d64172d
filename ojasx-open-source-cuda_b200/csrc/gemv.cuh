// Decode-shape fused linear: y[M,N] = x[M,K] . dequant(W)[N,K]^T for small M.
//
// Replaces, for small batches, _FusedE8GEMMFunction.forward (ojasx2/math/lattice.py:551-640)
// and the reference's scalar fused kernel (ojasx2/math/csrc/ojasx_math_core.hpp:580-634):
// per (m, n) the result is sum over groups of (sum_k x*coord) * scale, accumulated in fp32.
//
// Fast path (K % 256 == 0, bf16/fp16 activations, M <= 16)
//   * one CTA = 16 warps; warp w owns one 256-wide slice of K and keeps that slice of x in
//     registers as mma.m16n8k16 B fragments, so activations are read once per CTA;
//   * a work item is 16 weight rows x one K chunk (= all slices of the CTA); three items (~16 KB each)
//     beyond the current one are always in flight from HBM into a 5-stage shared-memory ring
//     (16-byte cp.async copies issued by all threads, completion on mbarriers); lanes then pick up
//     their rows' codes and scales with shared-memory loads;
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
// The public tile unit is 32 rows (ojx_e8t_gemv_tiles); this kernel walks them as two 16-row halves.
__host__ __device__ inline int gemv_row_tiles32(int N) { return (N + 31) / 32; }
__host__ __device__ inline int gemv_row_tiles(int N) { return 2 * gemv_row_tiles32(N); }

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
// Output-column sharding across GPUs: every rank owns an identically laid out output window, and a kernel
// can store its results into all of them (its own at offset 0, the peers' through their mapped addresses)
// instead of leaving the exchange to a separate all-gather.  delta[r] is the byte distance from this GPU's
// window to rank r's; world == 1 with delta[0] == 0 is the single-GPU case.
struct PeerMap {
    int64_t delta[8];
    int world;
    int pad;
};
inline PeerMap peer_map_self() { PeerMap m = {}; m.world = 1; return m; }
// The copies for the other ranks (delta != 0), kept out of line: rare, and the callers run at the register cap.
__device__ __noinline__ void store_peers(const PeerMap& pm, void* y, int y_dtype, int64_t idx, float v) {
    for (int r = 0; r < pm.world; ++r)
        if (pm.delta[r] != 0) store_any(static_cast<uint8_t*>(y) + pm.delta[r], y_dtype, idx, v);
}
template <bool kBf16> __device__ __forceinline__ float load_act(const void* p, int64_t idx) {
    if (kBf16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[idx]);
    return __half2float(static_cast<const __half*>(p)[idx]);
}

__device__ __forceinline__ void sts_u128(uint32_t addr, uint4 v) {
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
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
// Index of the problem that owns work item `item` (tile_begin ascends): the whole CTA counts the entries that
// start at or before it, one coalesced pass over the table instead of a chain of dependent loads (a 64-entry
// table walked entry by entry cost the last CTAs ~40 us at the start of every grouped launch).  Every thread of
// the CTA must call this.
__device__ __forceinline__ int find_problem(const ojx_e8t_gemv_problem* probs, int count, int item, int scale) {
    if (count == 1) return 0;                                  // single-problem launches (a layer at a time) skip the pass
    int found = 0;
    for (int base = 0; base < count; base += (int)blockDim.x) {
        const int t = base + (int)threadIdx.x;
        found += __syncthreads_count(t < count && scale * probs[t].tile_begin <= item);
    }
    return max(found - 1, 0);
}

__device__ __forceinline__ void cursor_seek(Cursor& c, const ojx_e8t_gemv_problem* probs, int p, int item) {
    c.prob = p;
    cursor_load_problem(c, probs);
    const int local = item - 2 * probs[p].tile_begin;
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

// 16-byte asynchronous copy global -> shared (L2 only, no L1 allocation) and the mbarrier arrive that
// fires when all of this thread's earlier copies have landed.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_arrive(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}

// Shared-memory plan of the fast kernel.
//   lut    COPIES interleaved copies of the rank -> trit-nibble table (entry r, copy c at (r*COPIES + c)*4)
//   ring   kGemvStages work items; an item holds 16 rows of codes (pitch = bytes + 16, so the 8 rows one
//          shared-memory load touches fall on distinct banks) followed by 16 rows of scales (same rule);
//          filled by all 512 threads with 16-byte cp.async copies (two per thread and item), completion
//          counted on an mbarrier.  One bulk (TMA) copy per padded row was tried first and capped the
//          kernel near 1 TB/s: ~32 small bulk copies per 16 KB item cost ~140 cycles each per SM.
//   red    kGemvRed buffers of per-warp fragments for the deterministic cross-warp sum
constexpr int kGemvStages = 5;                              // ring depth
constexpr int kGemvAhead = 3;                               // items in flight beyond the one being decoded
constexpr int kGemvRed = 4;
constexpr int kGemvRedLag = 2;                              // an item is summed two items after it was computed
constexpr int kGemvMaxCodePitch = kGemvWarps * 48 + 16;     // 784
constexpr int kGemvMaxScalePitch = kGemvWarps * 16 + 16;    // 272
constexpr int kGemvStageBytes = 16 * (kGemvMaxCodePitch + kGemvMaxScalePitch);   // 16896
constexpr int kGemvBlock = kGemvThreads;

// Per-thread share of filling ring stages: every thread copies up to two 16-byte chunks of each item.
// The chunk -> (row, column) mapping depends only on the problem's K, so it is recomputed when the
// issue cursor moves to another problem, not per item.
struct ItemLoader {
    uint32_t ring, bar_full, bar_empty;
    int tid;
    int prob;                      // problem the mapping below belongs to (-1: none)
    uint32_t dst[2];               // byte offset inside a stage
    int64_t src[2];                // byte offset from the tile's first row (codes) / first scale row
    int row[2];                    // row inside the tile, -1: this thread has no chunk
    bool is_scale[2];

    __device__ __forceinline__ void map_problem(const Cursor& c) {
        prob = c.prob;
        const int cb = c.act * 48, sb = c.act * 16;
        const int code_chunks = 48 * c.act, all_chunks = 64 * c.act;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int ch = tid + j * kGemvThreads;
            if (ch < code_chunks) {
                const int r = ch / (3 * c.act), col = ch - r * 3 * c.act;
                row[j] = r; is_scale[j] = false;
                dst[j] = (uint32_t)(r * (cb + 16) + col * 16);
                src[j] = (int64_t)r * (c.K * 3 / 16) + col * 16;
            } else if (ch < all_chunks) {
                const int cs = ch - code_chunks;
                const int r = cs / c.act, col = cs - r * c.act;
                row[j] = r; is_scale[j] = true;
                dst[j] = (uint32_t)(16 * kGemvMaxCodePitch + r * (sb + 16) + col * 16);
                src[j] = (int64_t)r * (c.K / 16) + col * 16;
            } else {
                row[j] = -1; is_scale[j] = false; dst[j] = 0; src[j] = 0;
            }
        }
    }

    // Copies item number n of this CTA (cursor c) into stage n mod S once the stage has been released.
    template <typename WaitFn>
    __device__ __forceinline__ void issue(const Cursor& c, const ojx_e8t_gemv_problem* probs, int n, WaitFn&& wait) {
        if (c.prob != prob) map_problem(c);
        const int s = n % kGemvStages;
        wait(bar_empty + 8 * s, ((uint32_t)(n / kGemvStages) & 1u) ^ 1u, 11);
        const ojx_e8t_gemv_problem& P = probs[c.prob];
        const int rows = min(16, c.N - c.tile * 16);
        const uint32_t stage = ring + s * kGemvStageBytes;
        const int64_t code_base = (int64_t)c.tile * 16 * (c.K * 3 / 16) + (int64_t)c.chunk * c.act * 48;
        const int64_t scale_base = (int64_t)c.tile * 16 * (c.K / 16) + (int64_t)c.chunk * c.act * 16;
#pragma unroll
        for (int j = 0; j < 2; ++j)
            if (row[j] >= 0 && row[j] < rows) {
                const uint8_t* sp = is_scale[j] ? reinterpret_cast<const uint8_t*>(P.scales) + scale_base + src[j]
                                                : P.packed + code_base + src[j];
                cp_async16(stage + dst[j], sp);
            }
        cp_async_arrive(bar_full + 8 * s);
    }
};

template <int NB, int COPIES> constexpr size_t gemv_smem_bytes() {
    return (size_t)kLutEntries * COPIES * 4 + (size_t)kGemvStages * kGemvStageBytes +
           (size_t)kGemvRed * kGemvWarps * 32 * 4 * NB * sizeof(float) + 256;
}

// All 16 warps are symmetric.  For item n (counted from the CTA's first item):
//   * all threads issued its cp.async copies kGemvAhead items earlier, after waiting for the ring stage to
//     be released by all warps ("empty" barrier); the stage being refilled was last used two items ago;
//   * every warp waits for the bytes ("full" barrier), pulls its rows' slice into registers, releases
//     the stage, decodes and multiplies, and parks its fragment in a reduction buffer ("rfull" barrier);
//   * warp ((n - 2) mod 16) then adds up the sixteen fragments of item n-2 in warp order and writes
//     the outputs ("rempty" barrier frees the buffer).  No block-wide barrier in the loop.
template <bool kBf16, int NB, int COPIES>
__global__ void __launch_bounds__(kGemvBlock, 1)
gemv_mma_kernel(const ojx_e8t_gemv_problem* __restrict__ probs_dev, const __grid_constant__ ojx_e8t_gemv_problem single,
                int count, int total_items, int M, int y_dtype, const __grid_constant__ PeerMap peers) {
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
            mbar_init(bar_full + 8 * s, kGemvThreads);      // every thread's cp.async arrive
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
    const int p0 = find_problem(probs, count, i0, 2);        // tile_begin counts 32-row tiles, items are 16-row halves

    // Bounded wait; once any wait has given up, later waits return at once and the loop runs on (on stale
    // data) so that every barrier keeps its arrival count.  The failure is reported in g_device_status.
    auto wait = [&](uint32_t bar, uint32_t parity, int code) {
        if (*abort_flag == 0) mbar_wait(bar, parity, abort_flag, code);
    };

    // ---- issue: every thread copies its chunks of item n into ring stage n mod S ----
    Cursor ic;                                  // cursor of the next item to be issued
    cursor_seek(ic, probs, p0, i0);
    const Cursor first = ic;                                       // the other two cursors start from the same item
    int issued = 0;
    ItemLoader loader;
    loader.ring = ring; loader.bar_full = bar_full; loader.bar_empty = bar_empty; loader.tid = tid; loader.prob = -1;
    auto issue_next = [&]() {
        loader.issue(ic, probs, issued, wait);
        ++issued;
        cursor_next(ic, probs, count);
    };
    for (int n = 0; n < kGemvAhead && n < nitems; ++n) issue_next();

    // ---- reduction of item n (done by warp n mod 16, kGemvRedLag items late) ----
    Cursor rc;                                  // cursor of the next item to be summed
    cursor_seek(rc, probs, p0, i0);
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
                            if (peers.world > 1) store_peers(peers, P.y, y_dtype, (int64_t)col * rc.N + row, v);
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
    Cursor cc = first;
    for (int n = 0; n < nitems; ++n) {
        const int s = n % kGemvStages, b = n % kGemvRed;
        if (issued < nitems) issue_next();                       // keeps kGemvAhead items in flight

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
__global__ void __launch_bounds__(256, 3) gemv_reduce_kernel(const ojx_e8t_gemv_problem* __restrict__ probs_dev,
                                                           const __grid_constant__ ojx_e8t_gemv_problem single,
                                                           int count, int M, int y_dtype, const __grid_constant__ PeerMap peers) {
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
#pragma unroll 1
            for (int r = 0; r < peers.world; ++r)                  // the other ranks' windows (nothing when world == 1)
                if (peers.delta[r] != 0) store_any(static_cast<uint8_t*>(P.y) + peers.delta[r], y_dtype, i, s);
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

}  // namespace ojx
