// Decode-shape linear for 1..16 activation rows (bf16 or fp16) on fp16 tensor cores, weights as the
// row ("A") operand of mma.sync.m16n8k16; one bf16 row on int8 tensor cores (see "kI8" below).
//
//   y[m, n] = sum_k x[m, k] * coord[n, k] * scale[n, k / 32]  (+ bias)      fp32 accumulation
//
// Replaces the reference's scalar fused kernel (ojasx2/math/csrc/ojasx_math_core.hpp:580-634) and, for
// small batches, _FusedE8GEMMFunction.forward (ojasx2/math/lattice.py:551-640).
//
// Work decomposition: a CTA of 16 warps walks a contiguous range of work items; an item is 32 weight
// rows x one K chunk (up to 16 slices of 256 k), warp w owns slice w.  Items stream HBM -> shared memory
// through a ring of 16-byte cp.async copies issued by all threads (row pitch padded by 16 bytes so that
// the eight rows one shared-memory load touches fall on distinct banks); completion is counted on one
// mbarrier per stage.  ONE block-wide barrier per item both releases the item's stage and publishes the
// warps' partial sums, which the first 256 (512 for 9-16 rows) threads then add up in warp order
// (deterministic) while the other warps already decode the next item.  The alternative without a block-wide
// barrier - "empty" / "partials parked" / "partials summed" mbarriers and a reduction one item late, as the
// one-row int8 kernel does - was measured with this arithmetic and lost (163 vs 145 us for the profiled launch
// at 4 rows, 263 vs 190 us at 16 rows where its extra state spills).
//
// What one lane does: lane (g, t) of a warp owns ranks 8t..8t+7 of its slice for weight rows g and g + 8
// of a 16-row tile: 12 contiguous bytes per row, i.e. 64 consecutive k = two scale groups.  A rank becomes
// four operand registers (eight EXACT fp16 weights coord * scale) with four byte permutes: the permute
// selectors come from one 64-bit shared-memory lookup (3281 entries, two interleaved copies), the permuted
// bytes from two "pools" {0, lo, lo, 0} / {0, hi, hi ^ 0x80, 0} of the group's fp16 scale, built once per
// (row, group).  The activations sit in registers as fp16 "B" fragments (64 k x 8 rows per lane and block of
// eight activation rows) for as long as the CTA stays inside one problem and K chunk; bf16 activations are
// rescaled per (row, slice) by a power of two so that the slice maximum lands in [2^14, 2^15) - exact for
// every element within 2^-29 of the maximum, Inf / NaN pass through - and the partial sums are scaled back
// before they are combined.  Because the scale is folded into the weights, fp32 accumulation runs across the
// whole slice and nothing is left to do per group.
//
// One bf16 activation row (kI8) keeps the skeleton - loader, ring, barrier, reduction, output - and swaps the
// arithmetic for int8 MMAs (mma.sync.m16n8k32.s8): a rank becomes its two operand registers with TWO byte permutes
// of a 32-bit entry (eight 4-bit selectors into {0, +1, -1}; four interleaved copies of the table, so a lookup costs
// ~2.8 shared-memory wavefronts instead of ~6.2), the activations are 28-bit fixed point per scale group, split into
// four base-128 digits.  The eight accumulator columns serve as (lane quarter, digit pair): lane (g, t) feeds its
// digits only into column g and only when g >> 1 == t, so after the four steps of a scale group column 2t holds the
// group's integer sums for digits 0, 1 and column 2t + 1 for digits 2, 3 (two MMAs per step share the decoded
// weights); they are combined, converted and scaled by weight scale * 2^exponent once per group.
//
// A conflict-free alternative to the 3281-entry table was built and measured: a rank r is the base-3 number
// 2r, so its low and high four digits can index one 81-entry table stored once per lane.  It removed every
// bank conflict (14.3 M -> 8 k per launch) but needs a multiply-high and two multiply-adds per rank, and ran
// 3-10 % slower; the kernels here are bound by instruction issue, not by shared-memory wavefronts.
#pragma once

#include <type_traits>

#include "gemv.cuh"

namespace ojx {

constexpr int kA16Rows = 32;                                              // weight rows per work item
constexpr int kA16StageBytes = kA16Rows * (kGemvMaxCodePitch + kGemvMaxScalePitch);   // 33792
constexpr uint32_t kA16ScaleOff = kA16Rows * kGemvMaxCodePitch;           // scales follow the 32 padded code rows
constexpr uint32_t kA16DescOff = kA16ScaleOff - 16;                       // free: every code row ends in 16 bytes of padding

__host__ __device__ inline int a16_row_tiles(int N) { return (N + kA16Rows - 1) / kA16Rows; }

template <int NB> struct A16Cfg {
    static constexpr int kStages = NB == 1 ? 4 : 3;                       // all but one are in flight while an item is decoded
    static constexpr int kRed = 2;                                        // reduction buffers (written at item n, n + 2, ...)
    static constexpr int kLutBytes = ((kNumPoints * 16 + 1023) / 1024) * 1024;   // two interleaved copies of 8-byte entries
    static constexpr int kRedFloats = kGemvWarps * 256 * NB;              // per buffer: 16 warps x 32 rows x 8 NB columns
    static constexpr int kOutStageBytes = 16 * kA16Rows * 2;              // an item's outputs as 16-bit values, [column][row]
    static constexpr size_t kSmem = (size_t)kLutBytes + (size_t)kStages * kA16StageBytes + (size_t)kRed * kRedFloats * sizeof(float) + 256 + kOutStageBytes;
};

__device__ __forceinline__ uint2 lds_u64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}

// fp16 MMA with fp32 accumulation: D (16 x 8) += A (16 x 16, row-major) * B (16 x 8, column-major).
__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// int8 MMA with int32 accumulation: D (16 x 8) += A (16 x 32, row-major) * B (32 x 8, column-major).
__device__ __forceinline__ void mma_s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Slow path of a bounded wait, kept out of line so the loop body stays small.
__device__ __noinline__ void a16_wait_slow(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code, uint32_t limit) {
    if (*abort_flag != 0) return;               // some wait already gave up: the CTA is only running out its loop
    mbar_wait(bar, parity, abort_flag, code, limit);
}
__device__ __forceinline__ void a16_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code, uint32_t limit) {
    if (!mbar_try_wait(bar, parity)) a16_wait_slow(bar, parity, abort_flag, code, limit);
}

// Rank J (0..7) of a lane's 96-bit window, moved so that it starts at bit POS (bits outside the field are junk).
template <int J, int POS>
__device__ __forceinline__ uint32_t a16_field(uint32_t w0, uint32_t w1, uint32_t w2) {
    constexpr int bit = 12 * J, word = bit >> 5, off = bit & 31;
    const uint32_t lo = word == 0 ? w0 : (word == 1 ? w1 : w2);
    if constexpr (off + 12 <= 32) {
        if constexpr (off > POS) return lo >> (off - POS);
        else if constexpr (off < POS) return lo << (POS - off);
        else return lo;
    } else {
        const uint32_t hi = word == 0 ? w1 : w2;
        return __funnelshift_r(lo, hi, off - POS);
    }
}

// The four operand registers of rank J: weights {0,1}, {2,3}, {4,5}, {6,7}, each an fp16 pair coord * scale.
// `lut` is the table's shared-memory address plus this lane's copy offset is OR-ed into the entry address.
template <int J>
__device__ __forceinline__ void a16_decode(uint32_t (&a)[4], uint32_t w0, uint32_t w1, uint32_t w2, uint32_t pa, uint32_t pb,
                                           uint32_t lut, uint32_t lane_or) {
    const uint32_t addr = (a16_field<J, 4>(w0, w1, w2) & 0xFFF0u) | lane_or;
    const uint2 sel = lds_u64(lut + addr);
    a[0] = prmt(pa, pb, sel.x); a[1] = prmt(pa, pb, sel.x >> 16);
    a[2] = prmt(pa, pb, sel.y); a[3] = prmt(pa, pb, sel.y >> 16);
}

template <int NB, bool kXF16, bool kI8 = false>
__global__ void __launch_bounds__(kGemvThreads, 1)
gemv_a16_kernel(const ojx_e8t_gemv_problem* __restrict__ probs_dev, const __grid_constant__ ojx_e8t_gemv_problem single,
                int count, int total_items, int M, int y_dtype, int overlap, const __grid_constant__ PeerMap peers) {
    static_assert(!kI8 || (NB == 1 && !kXF16), "the int8 path serves one bf16 activation row");
    using Cfg = A16Cfg<NB>;
    constexpr int S = Cfg::kStages;
    const ojx_e8t_gemv_problem* probs = probs_dev != nullptr ? probs_dev : &single;
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t lut = smem_u32(smem);
    const uint32_t ring = lut + Cfg::kLutBytes;
    float* red = reinterpret_cast<float*>(smem + Cfg::kLutBytes + S * kA16StageBytes);
    uint8_t* tail = smem + Cfg::kLutBytes + S * kA16StageBytes + Cfg::kRed * Cfg::kRedFloats * sizeof(float);
    const uint32_t bar_full = smem_u32(tail), bar_lut = bar_full + 8 * S;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tail + 64);
    uint16_t* ost = reinterpret_cast<uint16_t*>(tail + 256);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;

    if (tid == 0) {
        for (int s = 0; s < S; ++s) mbar_init(bar_full + 8 * s, kGemvThreads);      // every thread's cp.async arrive
        mbar_init(bar_lut, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        // the lookup table's shared-memory image arrives as ONE bulk copy while the kernel sets itself up.  int8 path:
        // 32-bit entries (eight 4-bit byte-permute selectors), every entry four times so that the four lanes of a row
        // read four different banks; fp16 path: 64-bit entries, two copies
        mbar_expect_tx(bar_lut, kNumPoints * 16);
        bulk_load(lut, kI8 ? g_lut_i8x4 : g_lut_f16sel, kNumPoints * 16, bar_lut);
    }
    __syncthreads();

    const int64_t per = ((int64_t)total_items + gridDim.x - 1) / gridDim.x;
    const int i0 = (int)min((int64_t)total_items, per * blockIdx.x);
    const int i1 = (int)min((int64_t)total_items, per * (blockIdx.x + 1));
    // the launch that follows in the stream may start its own set-up once every CTA of this one is past this point
    if (overlap) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // with partial sums the outputs are stored (and signalled) by the reduce kernel that follows
    const bool signal = peers.sync != nullptr && (peers.mode & OJX_GEMV_SIGNAL_PEERS) != 0 && (peers.mode & 0x100) == 0;
    if (i0 >= i1) {
        if (signal && tid == 0) {
            if (overlap == 1) asm volatile("griddepcontrol.wait;" ::: "memory");
            peer_signal(peers);
        }
        return;
    }
    const int nitems = i1 - i0;
    const int p0 = find_problem(probs, count, i0, 1);

    // ---- loader: thread (lr, ls) copies chunks ls, ls+16, ls+32 of row lr's codes and chunk ls of its scales.
    // The plan of a (problem, K chunk) - source pointers of this thread's chunks, destination offsets, which
    // chunks exist - is made once; from one row tile to the next only the two pointers move. ----
    const int lr = tid >> 4, ls = tid & 15;
    int l_prob = p0, l_chunk, l_tile, l_tiles = 1, l_kchunks = 1, l_act = 1, l_N = 0;
    const uint8_t* l_pc = nullptr;
    const uint8_t* l_ps = nullptr;
    int l_step_c = 0, l_step_s = 0;
    uint32_t l_dc = 0, l_ds = 0;
    bool l_c0 = false, l_c1 = false, l_c2 = false, l_cs = false;
    auto plan = [&]() {
        const ojx_e8t_gemv_problem& P = probs[l_prob];
        l_N = P.N;
        const int K = P.K;
        l_act = gemv_active_warps(K);
        l_tiles = a16_row_tiles(l_N);
        l_kchunks = (K / 256) / l_act;
        const uint32_t cb = l_act * 48, sb = l_act * 16;
        const int64_t rowc = K * 3 / 16, rows = K / 16;
        l_pc = P.packed + (int64_t)(l_tile * kA16Rows + lr) * rowc + (int64_t)l_chunk * cb + ls * 16;
        l_ps = reinterpret_cast<const uint8_t*>(P.scales) + (int64_t)(l_tile * kA16Rows + lr) * rows + (int64_t)l_chunk * sb + ls * 16;
        l_step_c = (int)(kA16Rows * rowc);
        l_step_s = (int)(kA16Rows * rows);
        l_dc = lr * (cb + 16) + ls * 16;
        l_ds = kA16ScaleOff + lr * (sb + 16) + ls * 16;
        l_c0 = ls < 3 * l_act; l_c1 = ls + 16 < 3 * l_act; l_c2 = ls + 32 < 3 * l_act; l_cs = ls < l_act;
    };
    {
        const int local = i0 - probs[p0].tile_begin;
        const int tiles0 = a16_row_tiles(probs[p0].N);
        l_chunk = local / tiles0;
        l_tile = local - l_chunk * tiles0;
        plan();
    }
    int issued = 0, istage = 0;
    auto issue_next = [&]() {                                      // the caller knows that stage `istage` is free
        const uint32_t stage = ring + istage * kA16StageBytes;
        if (l_tile * kA16Rows + lr < l_N) {
            if (l_c0) cp_async16(stage + l_dc, l_pc);
            if (l_c1) cp_async16(stage + l_dc + 256, l_pc + 256);
            if (l_c2) cp_async16(stage + l_dc + 512, l_pc + 512);
            if (l_cs) cp_async16(stage + l_ds, l_ps);
        }
        // the item's coordinates travel with its data, so only the loader keeps a cursor
        if (tid == 0) sts_u128(stage + kA16DescOff, make_uint4((uint32_t)l_prob, (uint32_t)l_chunk, (uint32_t)l_tile, (uint32_t)l_act));
        if (!(peers.lose_copy && issued == 0 && tid == 0)) cp_async_arrive(bar_full + 8 * istage);
        ++issued;
        if (++istage == S) istage = 0;
        if (++l_tile < l_tiles) {
            l_pc += l_step_c;
            l_ps += l_step_s;
        } else {
            l_tile = 0;
            if (++l_chunk == l_kchunks) {
                l_chunk = 0;
                if (l_prob + 1 < count) ++l_prob;
            }
            plan();
        }
    };
    // packed weights never depend on the previous launch: their copies start before that launch has drained
    for (int n = 0; n < S - 1 && n < nitems; ++n) issue_next();
    // activations (and the output buffers) do, unless the caller declared the launch independent (overlap == 2)
    if (overlap == 1) asm volatile("griddepcontrol.wait;" ::: "memory");
    // ... and, in a column-sharded chain, on the same launch of every other rank
    if (peers.sync != nullptr && (peers.mode & OJX_GEMV_WAIT_PEERS)) {
        if (tid == 0) peer_wait(peers);
        __syncthreads();
    }

    const uint32_t lane_or = (uint32_t)((lane & 1) << 3);
    uint32_t xb[NB][8][4];                      // B fragments: [block][rank j][k 0-1, 2-3, 4-5, 6-7 of the rank]
    float up[NB][2];                            // 2^e of activation rows 2t, 2t+1 of the block (this lane's output columns)
    // int8 path (one activation row): B fragments [rank j][digit pair][k 0-3, 4-7 of the rank] - non-zero only in the lane
    // that feeds the accumulator column - and the two factors of 2^-shift of this lane's scale groups 2t and 2t + 1
    uint32_t xq[8][2][2];
    float ua[2] = {1.f, 1.f}, ub[2] = {1.f, 1.f};
    bool xbad = false;                          // the slice holds Inf or NaN (same value in every lane of the warp)
    int cur_prob = -1, cur_chunk = -1, cur_K = 0;

    a16_wait(bar_lut, 0u, abort_flag, 55, peers.wait_limit);        // the table has landed
    int cstage = 0;
    uint32_t cparity = 0;
    for (int n = 0; n < nitems; ++n) {
        if (issued < nitems) issue_next();                          // into the stage the previous item's barrier released
        a16_wait(bar_full + 8 * cstage, cparity, abort_flag, 52, peers.wait_limit);
        // Once a wait has given up nothing in shared memory can be trusted (not even the item's coordinates): the
        // warp then only keeps the block-wide barriers matched until the loop ends.
        const bool dead = __any_sync(0xFFFFFFFFu, *abort_flag != 0);
        const uint32_t stage = ring + cstage * kA16StageBytes;
        uint4 desc = make_uint4(0, 0, 0, 0);
        if (!dead) desc = lds_u128(stage + kA16DescOff);
        const int prob = (int)desc.x, chunk = (int)desc.y, tile = (int)desc.z, act = dead ? 0 : (int)desc.w;
        if (++cstage == S) { cstage = 0; cparity ^= 1u; }

        if (!dead && (prob != cur_prob || chunk != cur_chunk)) {
            if (prob != cur_prob) cur_K = probs[prob].K;
            cur_prob = prob;
            cur_chunk = chunk;
            const uint16_t* xp = static_cast<const uint16_t*>(probs[prob].x);
            const int slice = chunk * act + warp;
            if constexpr (kI8) {
                // Fixed point per scale group: lane l holds x[8l .. 8l+7] of the slice (rank l); the 32 values of a group
                // (four lanes) share the exponent E of their largest finite magnitude and become integers
                // q = rint(x 2^(26 - E)), |q| <= 2^27, written in balanced base 128: q = 128^3 d0 + 128^2 d1 + 128 d2 + d3,
                // digits in [-64, 64].  Values within 2^-19 of the group's maximum are exact (bf16 carries 8 bits), the
                // others are rounded at 2^-27 of that maximum.  Inf / NaN become 0 here and are added back in fp32 below.
                const uint4 q = warp < act ? __ldcg(reinterpret_cast<const uint4*>(xp + slice * 256 + lane * 8)) : make_uint4(0, 0, 0, 0);
                const uint32_t w[4] = {q.x, q.y, q.z, q.w};
                uint32_t vb[8];
                uint32_t amax = 0;
                bool bad = false;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    vb[i] = (i & 1) ? (w[i >> 1] & 0xFFFF0000u) : (w[i >> 1] << 16);
                    const uint32_t mag = vb[i] & 0x7FFFFFFFu;
                    if (mag >= 0x7F800000u) { bad = true; vb[i] = 0u; }
                    else amax = max(amax, mag);
                }
                xbad = __any_sync(0xFFFFFFFFu, bad);
                amax = max(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
                amax = max(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));          // the four lanes of a group
                const int ex = (int)(amax >> 23);
                const int shift = 26 - (ex == 0 ? -126 : ex - 127);               // in [-101, 152]: applied as two factors
                const int sa = shift >> 1, sb = shift - sa;
                const float fa = __uint_as_float((uint32_t)(127 + sa) << 23), fb = __uint_as_float((uint32_t)(127 + sb) << 23);
                uint32_t dw[4][2] = {{0u, 0u}, {0u, 0u}, {0u, 0u}, {0u, 0u}};          // [digit][values 0-3, 4-7] as int8 x 4
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int q0 = __float2int_rn(__uint_as_float(vb[i]) * fa * fb);
                    const int q1 = (q0 + 64) >> 7, d3 = q0 - (q1 << 7);
                    const int q2 = (q1 + 64) >> 7, d2 = q1 - (q2 << 7);
                    const int d0 = (q2 + 64) >> 7, d1 = q2 - (d0 << 7);
                    const int sh = 8 * (i & 3);
                    dw[0][i >> 2] |= (uint32_t)(d0 & 0xFF) << sh;
                    dw[1][i >> 2] |= (uint32_t)(d1 & 0xFF) << sh;
                    dw[2][i >> 2] |= (uint32_t)(d2 & 0xFF) << sh;
                    dw[3][i >> 2] |= (uint32_t)(d3 & 0xFF) << sh;
                }
                // Accumulator column c = 2t' + h takes digits 2h and 2h + 1 of the group that lane quarter t' decodes, so
                // only lane (g, t) with g >> 1 == t feeds its column (g); every other lane's fragment is zero.
                const bool owner = (g >> 1) == t;
                const bool hi_digits = (g & 1) != 0;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int src = 8 * t + j;                                      // the lane that holds rank j of quarter t
#pragma unroll
                    for (int m = 0; m < 2; ++m)
#pragma unroll
                        for (int r = 0; r < 2; ++r) {
                            const uint32_t lo = __shfl_sync(0xFFFFFFFFu, dw[m][r], src);
                            const uint32_t hi = __shfl_sync(0xFFFFFFFFu, dw[2 + m][r], src);
                            xq[j][m][r] = owner ? (hi_digits ? hi : lo) : 0u;
                        }
                }
                const float una = __uint_as_float((uint32_t)(127 - sa) << 23), unb = __uint_as_float((uint32_t)(127 - sb) << 23);
                ua[0] = __shfl_sync(0xFFFFFFFFu, una, 8 * t);     ub[0] = __shfl_sync(0xFFFFFFFFu, unb, 8 * t);       // group 2t
                ua[1] = __shfl_sync(0xFFFFFFFFu, una, 8 * t + 4); ub[1] = __shfl_sync(0xFFFFFFFFu, unb, 8 * t + 4);   // group 2t + 1
            } else {
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
                const int m = nb * 8 + g;
                const bool on = warp < act && m < M;
                const uint4* xrow = reinterpret_cast<const uint4*>(xp + (int64_t)m * cur_K + slice * 256 + t * 64);
                float upg = 1.0f;
                if constexpr (kXF16) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        uint4 q = make_uint4(0, 0, 0, 0);
                        if (on) q = __ldcg(xrow + j);            // L2: in a sharded chain x was written by other GPUs
                        xb[nb][j][0] = q.x; xb[nb][j][1] = q.y; xb[nb][j][2] = q.z; xb[nb][j][3] = q.w;
                    }
                } else {
                    // two passes over the lane's 128 bytes (the second one hits the cache): maximum first, then convert,
                    // so that the raw words never have to be held beside the converted ones
                    uint32_t amax = 0;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        uint4 q = make_uint4(0, 0, 0, 0);
                        if (on) q = __ldcg(xrow + j);            // L2: in a sharded chain x was written by other GPUs
                        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                        for (int i = 0; i < 4; ++i) amax = max(amax, max((w[i] << 16) & 0x7FFFFFFFu, w[i] & 0x7FFF0000u));
                    }
                    amax = max(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
                    amax = max(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));      // the four lanes of activation row m
                    int e = 0;
                    const int ex = (int)((amax >> 23) & 0xFFu);
                    if (ex != 0 && ex != 0xFF) e = max(-100, min(100, ex - 127 - 14));   // slice maximum -> [2^14, 2^15)
                    const float down = __uint_as_float((uint32_t)(127 - e) << 23);
                    upg = __uint_as_float((uint32_t)(127 + e) << 23);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        uint4 q = make_uint4(0, 0, 0, 0);
                        if (on) q = __ldcg(xrow + j);            // L2: in a sharded chain x was written by other GPUs
                        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const __half2 v = __floats2half2_rn(__uint_as_float(w[i] << 16) * down, __uint_as_float(w[i] & 0xFFFF0000u) * down);
                            xb[nb][j][i] = *reinterpret_cast<const uint32_t*>(&v);
                        }
                    }
                }
                up[nb][0] = __shfl_sync(0xFFFFFFFFu, upg, 8 * t);          // lane (g' = 2t, *) holds activation row 2t
                up[nb][1] = __shfl_sync(0xFFFFFFFFu, upg, 8 * t + 4);
            }
            }
        }


        // buffer n & 1 was last read after the barrier of item n - 2, which every thread has passed
        float* rbuf = red + (size_t)(n & 1) * Cfg::kRedFloats + warp * (256 * NB);

        if (warp < act) {
            const uint32_t cpitch = act * 48 + 16, spitch = act * 16 + 16;
#pragma unroll
            for (int tl = 0; tl < 2; ++tl) {
                // this lane's words of the tile: rows g and g + 8, three code words and one scale word (groups 2t, 2t+1) each
                const uint32_t ca = stage + (tl * 16 + g) * cpitch + warp * 48 + t * 12, cb2 = ca + 8 * cpitch;
                const uint32_t sa = stage + kA16ScaleOff + (tl * 16 + g) * spitch + warp * 16 + t * 4;
                const uint32_t a0 = lds_u32(ca), a1 = lds_u32(ca + 4), a2 = lds_u32(ca + 8);
                const uint32_t b0 = lds_u32(cb2), b1 = lds_u32(cb2 + 4), b2 = lds_u32(cb2 + 8);
                const uint32_t ssa = lds_u32(sa), ssb = lds_u32(sa + 8 * spitch);
                if constexpr (kI8) {
                    // Ranks 0-3 of the lane belong to scale group 2t, ranks 4-7 to group 2t + 1: four steps of two MMAs
                    // (digit pairs) each, then the integer sums of the group are put together and scaled once.
                    const uint32_t lane_or4 = (uint32_t)(t << 2);
                    constexpr uint32_t kTritBytes = 0x00FF0100u;          // selector 0 -> 0, 1 -> +1, 2 -> -1
                    float og = 0.f, og8 = 0.f;                            // rows g and g + 8 of the tile
                    auto half_group = [&](auto htag) {
                        constexpr int H = decltype(htag)::value;
                        int c0[4] = {0, 0, 0, 0}, c1[4] = {0, 0, 0, 0};
                        auto step = [&](auto jtag) {
                            constexpr int J = decltype(jtag)::value;
                            const uint32_t ea = lds_u32(lut + ((a16_field<J, 4>(a0, a1, a2) & 0xFFF0u) | lane_or4));
                            const uint32_t eb = lds_u32(lut + ((a16_field<J, 4>(b0, b1, b2) & 0xFFF0u) | lane_or4));
                            const uint32_t r0 = prmt(kTritBytes, 0u, ea), r2 = prmt(kTritBytes, 0u, ea >> 16);
                            const uint32_t r1 = prmt(kTritBytes, 0u, eb), r3 = prmt(kTritBytes, 0u, eb >> 16);
                            mma_s8(c0, r0, r1, r2, r3, xq[J][0][0], xq[J][0][1]);
                            mma_s8(c1, r0, r1, r2, r3, xq[J][1][0], xq[J][1][1]);
                        };
                        step(std::integral_constant<int, 4 * H + 0>{});
                        step(std::integral_constant<int, 4 * H + 1>{});
                        step(std::integral_constant<int, 4 * H + 2>{});
                        step(std::integral_constant<int, 4 * H + 3>{});
                        // column 2t holds digits 0 (c0) and 1 (c1), column 2t + 1 digits 2 and 3; rows g (0, 1) and g + 8 (2, 3)
                        const float sg = fmaf((float)(c0[0] * 128 + c1[0]), 16384.f, (float)(c0[1] * 128 + c1[1]));
                        const float sg8 = fmaf((float)(c0[2] * 128 + c1[2]), 16384.f, (float)(c0[3] * 128 + c1[3]));
                        const float wa = __half2float(__ushort_as_half((uint16_t)(H ? (ssa >> 16) : (ssa & 0xFFFFu))));
                        const float wb = __half2float(__ushort_as_half((uint16_t)(H ? (ssb >> 16) : (ssb & 0xFFFFu))));
                        og = fmaf(sg * ua[H], wa * ub[H], og);
                        og8 = fmaf(sg8 * ua[H], wb * ub[H], og8);
                    };
                    half_group(std::integral_constant<int, 0>{});
                    half_group(std::integral_constant<int, 1>{});
                    og += __shfl_xor_sync(0xFFFFFFFFu, og, 1);
                    og8 += __shfl_xor_sync(0xFFFFFFFFu, og8, 1);
                    og += __shfl_xor_sync(0xFFFFFFFFu, og, 2);
                    og8 += __shfl_xor_sync(0xFFFFFFFFu, og8, 2);
                    // the summing threads read activation row 0 only: components 0 (row g) and 2 (row g + 8) of the lanes t == 0
                    if (t == 0) *reinterpret_cast<float4*>(rbuf + (tl * 32 + lane) * 4) = make_float4(og, 0.f, og8, 0.f);
                } else {
                float acc[NB][4];
#pragma unroll
                for (int nb = 0; nb < NB; ++nb) acc[nb][0] = acc[nb][1] = acc[nb][2] = acc[nb][3] = 0.f;

                auto rank_pair = [&](auto jtag, uint32_t paa, uint32_t pba, uint32_t pab, uint32_t pbb) {
                    constexpr int J = decltype(jtag)::value;
                    uint32_t ra[4], rb[4];
                    a16_decode<J>(ra, a0, a1, a2, paa, pba, lut, lane_or);
                    a16_decode<J>(rb, b0, b1, b2, pab, pbb, lut, lane_or);
#pragma unroll
                    for (int nb = 0; nb < NB; ++nb) {
                        mma_f16(acc[nb], ra[0], rb[0], ra[1], rb[1], xb[nb][J][0], xb[nb][J][1]);
                        mma_f16(acc[nb], ra[2], rb[2], ra[3], rb[3], xb[nb][J][2], xb[nb][J][3]);
                    }
                };
                {   // group 2t: byte pools {0, lo, lo, 0} and {0, hi, hi ^ 0x80, 0} of the scale in the low half
                    const uint32_t paa = prmt(ssa, 0u, 0x4004u), pba = prmt(ssa, 0u, 0x4114u) ^ 0x00800000u;
                    const uint32_t pab = prmt(ssb, 0u, 0x4004u), pbb = prmt(ssb, 0u, 0x4114u) ^ 0x00800000u;
                    rank_pair(std::integral_constant<int, 0>{}, paa, pba, pab, pbb);
                    rank_pair(std::integral_constant<int, 1>{}, paa, pba, pab, pbb);
                    rank_pair(std::integral_constant<int, 2>{}, paa, pba, pab, pbb);
                    rank_pair(std::integral_constant<int, 3>{}, paa, pba, pab, pbb);
                }
                {   // group 2t + 1: the scale in the high half
                    const uint32_t paa = prmt(ssa, 0u, 0x4224u), pba = prmt(ssa, 0u, 0x4334u) ^ 0x00800000u;
                    const uint32_t pab = prmt(ssb, 0u, 0x4224u), pbb = prmt(ssb, 0u, 0x4334u) ^ 0x00800000u;
                    rank_pair(std::integral_constant<int, 4>{}, paa, pba, pab, pbb);
                    rank_pair(std::integral_constant<int, 5>{}, paa, pba, pab, pbb);
                    rank_pair(std::integral_constant<int, 6>{}, paa, pba, pab, pbb);
                    rank_pair(std::integral_constant<int, 7>{}, paa, pba, pab, pbb);
                }
#pragma unroll
                for (int nb = 0; nb < NB; ++nb)
                    *reinterpret_cast<float4*>(rbuf + ((tl * NB + nb) * 32 + lane) * 4) =
                        make_float4(acc[nb][0] * up[nb][0], acc[nb][1] * up[nb][1], acc[nb][2] * up[nb][0], acc[nb][3] * up[nb][1]);
                }
            }
        }
        if constexpr (kI8) {
            if (xbad && warp < act) {
                // Inf / NaN in this warp's slice (they were fed to the MMAs as 0): lane r adds, in fp32, the products of
                // weight row r with those activations - Inf * 0 and anything * NaN give NaN, as in fp32 arithmetic.
                const uint32_t cpitch = act * 48 + 16, spitch = act * 16 + 16;
                const uint16_t* xp = static_cast<const uint16_t*>(probs[prob].x) + (chunk * act + warp) * 256;
                const uint4 q = __ldcg(reinterpret_cast<const uint4*>(xp + lane * 8));
                const uint32_t w[4] = {q.x, q.y, q.z, q.w};
                bool mine = false;
#pragma unroll
                for (int i = 0; i < 4; ++i) mine = mine || ((w[i] << 16) & 0x7FFFFFFFu) >= 0x7F800000u || (w[i] & 0x7FFF0000u) >= 0x7F800000u;
                uint32_t holders = __ballot_sync(0xFFFFFFFFu, mine);
                const uint8_t* codes = smem + (stage - lut) + lane * cpitch + warp * 48;        // weight row `lane` of the item
                const uint16_t* scl = reinterpret_cast<const uint16_t*>(smem + (stage - lut) + kA16ScaleOff + lane * spitch + warp * 16);
                float corr = 0.f;
                while (holders != 0u) {
                    const int l = __ffs(holders) - 1;                      // rank l of the slice = the eight values lane l holds
                    holders &= holders - 1u;
                    uint32_t xv[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) xv[i] = __shfl_sync(0xFFFFFFFFu, w[i], l);
                    const uint32_t b0 = codes[(3 * l) >> 1], b1 = codes[((3 * l) >> 1) + 1];
                    const uint32_t rank = (l & 1) ? ((b0 >> 4) | (b1 << 4)) : (b0 | ((b1 & 0xFu) << 8));
                    const uint32_t entry = g_trit_nibbles[rank < (uint32_t)kNumPoints ? rank : 0u];
                    const float sc = __half2float(__ushort_as_half(scl[l >> 2]));
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const uint32_t bits = (i & 1) ? (xv[i >> 1] & 0xFFFF0000u) : (xv[i >> 1] << 16);
                        if ((bits & 0x7FFFFFFFu) >= 0x7F800000u) {
                            const uint32_t sel = (entry >> (4 * i)) & 0xFu;
                            const float coord = sel == 1u ? 1.f : (sel == 2u ? -1.f : 0.f);
                            corr += (coord * sc) * __uint_as_float(bits);
                        }
                    }
                }
                __syncwarp();                                              // the lanes' own partial sums are written
                rbuf[((lane >> 4) * 32 + (lane & 7) * 4) * 4 + (((lane >> 3) & 1) << 1)] += corr;
            }
        }
        __syncthreads();           // the stage is free again and every warp's partial sums are visible

        // ---- sum over the warps in warp order; thread tid owns element tid of the 256 NB fragment values.
        // 16-bit outputs of a full 32-row tile are first collected in shared memory ([column][row]) and then written as
        // 16-byte vectors - to this rank's buffer and, in a column-sharded launch, to every peer's window - instead of one
        // 2-byte store per value and target. ----
        if (tid < 256 * NB) {
            const int comp = tid & 3, lp = (tid >> 2) & 31, nb = (tid >> 7) % NB, tl = tid / (128 * NB);
            const int rin = tl * 16 + (lp >> 2) + ((comp >> 1) << 3);        // row inside the item
            const int row = tile * kA16Rows + rin;
            const int col = nb * 8 + ((lp & 3) << 1) + (comp & 1);
            bool vec = false;
            int64_t ld = 0;
            void* ybase = nullptr;
            if (!dead) {
                const ojx_e8t_gemv_problem& P = probs[prob];
                const int rN = P.N;
                ld = P.ldy > 0 ? P.ldy : rN;
                ybase = P.y;
                vec = P.partial == nullptr && y_dtype != OJX_F32 && tile * kA16Rows + kA16Rows <= rN && (ld & 7) == 0 &&
                      (reinterpret_cast<uintptr_t>(P.y) & 15) == 0;
                if (row < rN && col < M) {                           // activation rows beyond M hold zeros: nothing to add up
                    const float* rb = red + (size_t)(n & 1) * Cfg::kRedFloats + tid;
                    float sum = 0.f;
#pragma unroll
                    for (int w = 0; w < kGemvWarps; ++w)
                        if (w < act) sum += rb[w * 256 * NB];
                    if (P.partial != nullptr) P.partial[((int64_t)chunk * M + col) * rN + row] = sum;
                    else {
                        if (P.bias != nullptr) sum += load_any(P.bias, kXF16 ? OJX_F16 : OJX_BF16, row);
                        if constexpr (NB == 1) {                         // the host refuses the low-rank term beyond eight rows
                            if (P.lora_rank > 0) sum += lora_term<!kXF16>(P, col, row);
                        }
                        if (vec) {
                            ost[col * kA16Rows + rin] = y_dtype == OJX_BF16 ? __bfloat16_as_ushort(__float2bfloat16_rn(sum))
                                                                            : __half_as_ushort(__float2half_rn(sum));
                        } else {
                            const int64_t at = (int64_t)col * ld + row;
                            store_any(P.y, y_dtype, at, sum);
                            if (peers.world > 1) store_peers(peers, P.y, y_dtype, at, sum);
                        }
                    }
                }
            }
            // every summing thread, whatever it did above, so that the count of the named barrier is always met
            asm volatile("bar.sync 1, %0;" ::"r"(256 * NB) : "memory");
            if (vec && tid < M * 4 * peers.world) {
                const int target = tid / (M * 4), v = tid - target * (M * 4), vcol = v >> 2, q = v & 3;
                const uint4 val = *reinterpret_cast<const uint4*>(ost + vcol * kA16Rows + q * 8);
                uint8_t* dst = static_cast<uint8_t*>(ybase) + peers.delta[target] + ((int64_t)vcol * ld + tile * kA16Rows + q * 8) * 2;
                *reinterpret_cast<uint4*>(dst) = val;
            }
        }
    }

    asm volatile("cp.async.wait_all;" ::: "memory");               // nothing of this thread is still in flight into shared memory
    if (tid == 0 && *abort_flag != 0) {
        atomicCAS(&g_device_status, 0, *abort_flag);
        if (peers.host_status != nullptr) *reinterpret_cast<volatile int*>(peers.host_status) = *abort_flag;
    }
    if (signal) {
        __syncthreads();
        if (tid == 0) peer_signal(peers);
    }
}

}  // namespace ojx
