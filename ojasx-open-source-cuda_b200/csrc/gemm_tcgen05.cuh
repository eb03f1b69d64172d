// Prefill-shape fused linear on the 5th-generation tensor cores (tcgen05 + TMEM + TMA).
//
//   y[M, N] = x[M, K] . dequant(W)[N, K]^T (+ bias)       M large (tokens), fp32 accumulation
//
// Replaces the reference's TileLang builder (ojasx2/tilelang_kernels.py:277-363) and its
// unpack + F.linear path (ojasx2/math/lattice.py:613-624).
//
// The product is computed transposed: decoded weights are the MMA "A" operand (two blocks of 128
// weight rows = 128 TMEM lanes each per CTA tile) and the tokens are the "B"/N side (256 per tile),
// so each decoded weight feeds 256 MACs and every x tile fetched from L2 feeds 256 weight rows.
// (With 128-row tiles the x tiles alone needed 64 B/clk/SM from L2 at full tensor rate and the
// kernel stalled at 40 % tensor activity; 256-row tiles halve that traffic.)
//
// Per CTA (448 threads, persistent over tiles, 3-stage ring of 64-wide K blocks):
//   warp 12     TMA producer: x tile [256 tokens x 64 k] -> shared memory, 128-byte swizzle
//   warps 4-11  decoders: thread r owns weight row r of the 256-row tile; streams
//               48 B of codes + 16 B of scales per 256 k with 128-bit loads, turns each 12-bit rank into
//               eight EXACT fp16 weights (coord * fp16 scale is exact in fp16) and stores them as one
//               16-byte chunk of the swizzled K-major A tile
//   warp 13     one thread issues tcgen05.mma (kind::f16, A = fp16 weights, B = fp16 activations,
//               fp32 accumulator in TMEM) and commits to the stage's "empty" barrier
//   warps 0-3   epilogue: tcgen05.ld the two finished 128 x 256 accumulators (all 512 TMEM columns),
//               add bias, cast, store y
// Every mbarrier wait is bounded; on expiry the kernel records a status word and drains.
//
// Operand types.  The weight tile must be fp16: coord * fp16 scale is exact in fp16 but not in bf16,
// and bf16-rounded weights together with bf16 outputs exceed the 2e-3 relative-L2 contract.  On B200
// a kind::f16 MMA whose A and B formats differ (fp16 x bf16) is rejected as an illegal instruction,
// so bf16 activations are first rewritten as fp16 by a small pre-pass into caller-owned scratch
// (one read-convert-write pass that also finds max|x|; a second pass runs only if rescaling is needed):
// x * 2^-e with e chosen from the tensor's absolute maximum so nothing overflows (e = 0, i.e. an
// exact copy, whenever |x| < 32768); the epilogue multiplies the fp32 result by 2^e.
#pragma once

#include <cuda.h>

#include "common.cuh"
#include "gemv.cuh"

namespace ojx {

constexpr int kGemmBM = 256;            // weight rows per tile: two MMA row blocks of 128 sharing every x tile
constexpr int kGemmHalf = 128;          // MMA M
constexpr int kGemmBN = 256;            // tokens per tile (MMA N)
constexpr int kGemmBK = 64;             // k per stage (one 128-byte swizzle row of 16-bit elements)
constexpr int kGemmStages = 3;
constexpr int kGemmThreads = 448;          // 4 epilogue + 8 decoder + 1 TMA + 1 MMA warps
constexpr int kGemmDecoderWarps = 8;
constexpr uint32_t kXStageBytes = kGemmBN * kGemmBK * 2;      // 32768
constexpr uint32_t kAStageBytes = kGemmBM * kGemmBK * 2;      // 32768 (rows 0-127, then rows 128-255)
constexpr uint32_t kGemmLutBytes = 4096 * 8;                  // rank -> eight fp16 high bytes (+1.0 / -1.0 / 0); any 12-bit rank in bounds
constexpr uint32_t kGemmSmemBytes = kGemmStages * (kXStageBytes + kAStageBytes) + kGemmLutBytes + 256 + 1024;

struct GemmParams {
    const uint8_t* packed;
    const uint16_t* scales;
    const void* bias;
    void* y;
    int32_t* status;
    int M, N, K;
    int y_dtype;
    int bias_dtype;
    uint32_t idesc;
    int rows;                      // weight rows per CTA tile: 128 or 256
    int bn;                        // tokens per CTA tile (MMA N): 128 or 256
    const uint32_t* amax_bits;     // fp32 bit pattern of max|x| when activations were rescaled, else null
};

// Power-of-two exponent e >= 0 with max|x| * 2^-e < 2^15.
__device__ __forceinline__ int prescale_exponent(uint32_t amax_bits) {
    const int ex = (int)((amax_bits >> 23) & 0xFFu) - 127;
    return ex > 14 ? ex - 14 : 0;
}

// Pass 1 (always): fp16 copy of the bf16 activations assuming no rescaling is needed, plus the tensor's
// absolute maximum.  Pass 2 does the rescaled copy only when the maximum turned out to be >= 32768.
__global__ void __launch_bounds__(256) convert_bf16_to_f16_kernel(const __nv_bfloat16* __restrict__ x,
                                                                   __half* __restrict__ out, int64_t count,
                                                                   uint32_t* __restrict__ amax_bits) {
    uint32_t m = 0;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i * 8 < count; i += (int64_t)gridDim.x * blockDim.x) {
        if (i * 8 + 8 <= count) {
            const uint4 v = __ldg(reinterpret_cast<const uint4*>(x) + i);
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
            uint32_t o[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                m = max(m, (w[j] << 16) & 0x7FFFFFFFu);
                m = max(m, w[j] & 0x7FFF0000u);
                const __half2 h = __floats2half2_rn(__uint_as_float(w[j] << 16), __uint_as_float(w[j] & 0xFFFF0000u));
                o[j] = *reinterpret_cast<const uint32_t*>(&h);
            }
            reinterpret_cast<uint4*>(out)[i] = make_uint4(o[0], o[1], o[2], o[3]);
        } else {
            for (int64_t j = i * 8; j < count; ++j) {
                m = max(m, ((uint32_t)__bfloat16_as_ushort(x[j]) << 16) & 0x7FFFFFFFu);
                out[j] = __float2half_rn(__bfloat162float(x[j]));
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    if ((threadIdx.x & 31) == 0 && m != 0) atomicMax(amax_bits, m);      // positive floats order like integers
}

__global__ void __launch_bounds__(256) rescale_bf16_to_f16_kernel(const __nv_bfloat16* __restrict__ x,
                                                                   __half* __restrict__ out, int64_t count,
                                                                   const uint32_t* __restrict__ amax_bits) {
    const int e = prescale_exponent(*amax_bits);
    if (e == 0) return;                                                   // pass 1 was already exact
    const float down = __int_as_float((127 - e) << 23);
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (int64_t)gridDim.x * blockDim.x)
        out[i] = __float2half_rn(__bfloat162float(x[i]) * down);
}

// ---- PTX wrappers (mbarrier helpers live in common.cuh) ------------------------------------------
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tmap, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(tmap), "r"(c0), "r"(c1), "r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// K-major operand tile whose rows are 128 bytes (64 16-bit elements) with the 128-byte swizzle:
// 8-row groups are 1024 bytes apart (stride byte offset); leading byte offset is unused.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);            // start address, 16-byte units
    d |= (uint64_t)1 << 16;                                  // leading byte offset (ignored for swizzled K-major)
    d |= (uint64_t)(1024u >> 4) << 32;                       // stride byte offset
    d |= (uint64_t)1 << 46;                                  // descriptor version for sm_100
    d |= (uint64_t)2 << 61;                                  // SWIZZLE_128B
    return d;
}
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Eight exact fp16 weights (coord * scale) of one rank as a 16-byte chunk; `hb` holds the eight fp16 high
// bytes of +-1.0 / 0 (the low bytes are zero), `scale2` the group scale in both halves.
__device__ __forceinline__ uint4 decode_chunk_f16(uint2 hb, uint32_t scale2) {
    uint32_t p[4] = {prmt(hb.x, 0u, 0x1404u), prmt(hb.x, 0u, 0x3424u), prmt(hb.y, 0u, 0x1404u), prmt(hb.y, 0u, 0x3424u)};
    uint4 out;
    uint32_t* o = reinterpret_cast<uint32_t*>(&out);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        __half2 v = __hmul2(*reinterpret_cast<__half2*>(&p[i]), *reinterpret_cast<__half2*>(&scale2));
        o[i] = *reinterpret_cast<uint32_t*>(&v);
    }
    return out;
}

__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_x, const GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;                       // tiles need 1024-byte alignment
    uint8_t* smem = smem_raw + (base - raw);
    const uint32_t x_base = base;
    const uint32_t a_base = base + kGemmStages * kXStageBytes;
    uint32_t* lut = reinterpret_cast<uint32_t*>(smem + kGemmStages * (kXStageBytes + kAStageBytes));
    const uint32_t bar_base = base + kGemmStages * (kXStageBytes + kAStageBytes) + kGemmLutBytes;
    // barriers: full[S], empty[S], tmem_full[2], tmem_empty[2]; then tmem pointer; then abort flag
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (kGemmStages + s); };
    auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * kGemmStages + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * kGemmStages + 2 + a); };
    uint8_t* bar_ptr = smem + kGemmStages * (kXStageBytes + kAStageBytes) + kGemmLutBytes;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bar_ptr + 8 * (2 * kGemmStages + 4));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_ptr + 8 * (2 * kGemmStages + 4) + 8);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // 64-bit table: byte i = high byte of the fp16 value of coordinate i (0x3C: +1.0, 0xBC: -1.0, 0: 0)
    for (int i = tid; i < 4096; i += kGemmThreads) {
        const uint32_t nib = i < kNumPoints ? g_trit_nibbles[i] : 0u;
        const uint32_t lo = prmt(0x00BC3C00u, 0u, nib), hi = prmt(0x00BC3C00u, 0u, nib >> 16);
        reinterpret_cast<uint2*>(lut)[i] = make_uint2(lo, hi);
    }
    if (tid == 0) {
        for (int s = 0; s < kGemmStages; ++s) {
            mbar_init(full_bar(s), 1 + p.rows / 32);        // TMA transaction + one arrive per active decoder warp
            mbar_init(empty_bar(s), 1);             // tcgen05.commit
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tfull_bar(a), 1);             // tcgen05.commit after the tile's last k block
            mbar_init(tempty_bar(a), 4);            // one arrive per epilogue warp
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 13) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;"
                     ::"r"(smem_u32(const_cast<uint32_t*>(tmem_slot))) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int n_blocks = (p.N + p.rows - 1) / p.rows;
    const int m_blocks = (p.M + p.bn - 1) / p.bn;
    const uint32_t x_bytes = (uint32_t)p.bn * kGemmBK * 2;
    const int tiles = n_blocks * m_blocks;
    const int k_blocks = p.K / kGemmBK;

    if (warp == 12) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
                const int m_blk = tile / n_blocks;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % kGemmStages;
                    const uint32_t ph = (it / kGemmStages) & 1u;
                    if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, 1)) { ok = false; break; }
                    mbar_expect_tx(full_bar(s), x_bytes);
                    tma_load_2d(x_base + s * kXStageBytes, &tmap_x, kb * kGemmBK, m_blk * p.bn, full_bar(s));
                }
            }
            if (!ok) {
                // Loads already issued still complete on their barriers; give them a bounded time to land
                // before the CTA's shared memory is released.
                for (uint32_t back = 0; back < (uint32_t)kGemmStages && back < it; ++back) {
                    const uint32_t j = it - 1 - back;
                    const int s = j % kGemmStages;
                    const uint32_t ph = (j / kGemmStages) & 1u;
                    for (uint32_t i = 0; i < (1u << 16); ++i)
                        if (mbar_try_wait(full_bar(s), ph)) break;
                }
            }
        }
    } else if (warp == 13) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            uint32_t it = 0, tcount = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++tcount) {
                // both accumulators (columns 0-255: rows 0-127, columns 256-511: rows 128-255) must have been drained
                if (!mbar_wait(tempty_bar(0), (tcount & 1u) ^ 1u, abort_flag, 2)) { ok = false; break; }
                tc_fence_after();
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % kGemmStages;
                    const uint32_t ph = (it / kGemmStages) & 1u;
                    if (!mbar_wait(full_bar(s), ph, abort_flag, 3)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = a_base + s * kAStageBytes, x_addr = x_base + s * kXStageBytes;
#pragma unroll
                    for (int k = 0; k < kGemmBK / 16; ++k) {
                        const uint64_t bd = umma_desc_sw128(x_addr + k * 32);
                        tc_mma_f16(tmem_base, umma_desc_sw128(a_addr + k * 32), bd, p.idesc, (kb > 0 || k > 0) ? 1u : 0u);
                        if (p.rows == kGemmBM)
                            tc_mma_f16(tmem_base + kGemmBN, umma_desc_sw128(a_addr + kGemmHalf * 128 + k * 32), bd, p.idesc,
                                       (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    tc_commit(empty_bar(s));           // frees the stage once these MMAs have read it
                }
                if (ok) tc_commit(tfull_bar(0));       // accumulators complete -> epilogue
            }
        }
    } else if (warp >= 4 && (warp - 4) * 32 < p.rows) {
        // ---------------- decoders (warps beyond the tile's rows stay idle) ----------------
        const int r = (warp - 4) * 32 + lane;           // row of the 256-row tile
        uint32_t it = 0;
        bool ok = true;
        const int64_t row_bytes = (int64_t)p.K * 3 / 16, row_scales = p.K / 32;
        for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
            const int n_blk = tile % n_blocks;
            const int row = min(n_blk * p.rows + r, p.N - 1);
            const uint4* cptr = reinterpret_cast<const uint4*>(p.packed + row * row_bytes);
            const uint4* sptr = reinterpret_cast<const uint4*>(p.scales + row * row_scales);
            const int chunks = p.K / 256;
            uint4 c0 = __ldg(cptr), c1 = __ldg(cptr + 1), c2 = __ldg(cptr + 2), sc = __ldg(sptr);
            for (int ch = 0; ch < chunks && ok; ++ch) {
                uint32_t cw[12] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w, c2.x, c2.y, c2.z, c2.w};
                uint32_t sw[4] = {sc.x, sc.y, sc.z, sc.w};
                if (ch + 1 < chunks) {                   // prefetch the next 256 k of this row
                    c0 = __ldg(cptr + 3 * (ch + 1)); c1 = __ldg(cptr + 3 * (ch + 1) + 1);
                    c2 = __ldg(cptr + 3 * (ch + 1) + 2); sc = __ldg(sptr + ch + 1);
                }
#pragma unroll
                for (int q = 0; q < 4; ++q, ++it) {
                    const int s = it % kGemmStages;
                    const uint32_t ph = (it / kGemmStages) & 1u;
                    if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, 4)) { ok = false; break; }
                    uint8_t* arow = smem + kGemmStages * kXStageBytes + s * kAStageBytes + r * 128;
                    // All eight table lookups are issued before the first store: the compiler must assume a
                    // shared-memory store may alias the table, so interleaving them would serialise the ranks.
                    uint2 hb[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int c = q * 8 + j;                 // rank index inside the 48-byte chunk
                        const int bit = 12 * c, w = bit >> 5, sh = bit & 31;
                        uint32_t off;                            // rank * 8 = byte offset into the 64-bit table
                        if (sh + 12 <= 32) off = sh >= 3 ? (cw[w] >> (sh - 3)) : (cw[w] << (3 - sh));
                        else off = __funnelshift_r(cw[w], cw[w + 1 < 12 ? w + 1 : 11], sh - 3);
                        hb[j] = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint8_t*>(lut) + (off & 0x7FF8u));
                    }
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int grp = (q * 8 + j) >> 2;        // scale group inside the chunk
                        const uint32_t sp = sw[grp >> 1];
                        const uint32_t s16 = (grp & 1) ? (sp >> 16) : (sp & 0xFFFFu);
                        const uint4 v = decode_chunk_f16(hb[j], s16 | (s16 << 16));
                        *reinterpret_cast<uint4*>(arow + ((j ^ (r & 7)) << 4)) = v;
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> async proxy (UMMA)
                    __syncwarp();
                    if (lane == 0) mbar_arrive(full_bar(s));
                }
            }
        }
    } else if (warp < 4) {
        // ---------------- epilogue (warps 0-3 own TMEM lanes 32*warp ..) ----------------
        uint32_t tcount = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++tcount) {
            const int n_blk = tile % n_blocks, m_blk = tile / n_blocks;
            ok = mbar_wait(tfull_bar(0), tcount & 1u, abort_flag, 5);
            ok = __all_sync(0xFFFFFFFFu, ok);          // warp-uniform decision before the aligned TMEM loads
            if (!ok) break;
            tc_fence_after();
            const float up = p.amax_bits != nullptr ? __int_as_float((127 + prescale_exponent(*p.amax_bits)) << 23) : 1.0f;
#pragma unroll 1
            for (int h = 0; h < p.rows / kGemmHalf; ++h) {
                const int n = n_blk * p.rows + h * kGemmHalf + warp * 32 + lane;
                float bias = 0.f;
                if (p.bias != nullptr && n < p.N) bias = load_any(p.bias, p.bias_dtype, n);
                const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + h * kGemmBN;
#pragma unroll 1
                for (int cb = 0; cb < p.bn / 32; ++cb) {
                    uint32_t v[32];
                    tmem_ld_32x32b_x32(taddr + cb * 32, v);
                    tmem_ld_wait();
                    const int m0 = m_blk * p.bn + cb * 32;
                    if (n < p.N) {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (m0 + i < p.M) store_any(p.y, p.y_dtype, (int64_t)(m0 + i) * p.N + n, fmaf(__uint_as_float(v[i]), up, bias));
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar(0));
        }
    }

    tc_fence_before();
    __syncthreads();
    if (tid == 0 && *abort_flag != 0 && p.status != nullptr) atomicCAS(p.status, 0, *abort_flag);
    if (warp == 13) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
    }
}

// ---- host side --------------------------------------------------------------------------------------
typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static PFN_encodeTiled get_encode_tiled() {
    static PFN_encodeTiled fn = nullptr;
    if (fn == nullptr) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<PFN_encodeTiled>(ptr);
    }
    return fn;
}

inline bool gemm_fast_ok(int64_t M, int64_t N, int64_t K, int group, int x_dtype) {
    return M >= 1 && N >= 1 && K >= 256 && K % 256 == 0 && group == 32 &&
           (x_dtype == OJX_BF16 || x_dtype == OJX_F16) && M < (1 << 30) && N < (1 << 30) && K < (1 << 30);
}

// Scratch: a 256-byte status block (word 0: give-up code of a bounded wait, word 1: bit pattern of
// max|x|; zeroed by every call) followed by room for an fp16 copy of the activations.
size_t gemm_workspace_bytes_impl(int64_t M, int64_t N, int64_t K) {
    (void)N;
    if (M <= 0 || K <= 0) return 256;
    return 256 + (size_t)M * (size_t)K * 2;
}

int32_t gemm_impl(const void* x, int x_dtype, int64_t M, const uint8_t* packed, const uint16_t* scales,
                  const void* bias, int64_t N, int64_t K, int group, void* y, int y_dtype,
                  void* workspace, size_t workspace_bytes, cudaStream_t s) {
    OJX_RETURN_IF(!x || !packed || !scales || !y, OJX_ERR_NULL);
    OJX_RETURN_IF(M <= 0 || N <= 0 || K <= 0, OJX_ERR_SHAPE);
    OJX_RETURN_IF(dtype_size(x_dtype) == 0 || dtype_size(y_dtype) == 0, OJX_ERR_DTYPE);
    OJX_RETURN_IF(check_arch() != OJX_OK, OJX_ERR_ARCH);
    group = effective_group(group);
    OJX_RETURN_IF(!gemm_fast_ok(M, N, K, group, x_dtype), OJX_ERR_UNSUPPORTED);
    OJX_RETURN_IF(((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(packed) |
                    reinterpret_cast<uintptr_t>(scales)) & 15) != 0, OJX_ERR_ALIGN);
    const bool convert = x_dtype == OJX_BF16;
    const size_t need = convert ? gemm_workspace_bytes_impl(M, N, K) : 256;
    OJX_RETURN_IF(!workspace || workspace_bytes < need, OJX_ERR_WORKSPACE);
    OJX_RETURN_IF((reinterpret_cast<uintptr_t>(workspace) & 255) != 0, OJX_ERR_ALIGN);
    PFN_encodeTiled encode = get_encode_tiled();
    OJX_RETURN_IF(encode == nullptr, OJX_ERR_LAUNCH);

    CUtensorMap tmap;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    // Tile shape: the choice that minimises (waves over the SMs) x (work per tile), with a small
    // penalty for the shapes that reuse each fetched x tile or decoded weight tile less.
    int rows = kGemmBM, bn = kGemmBN;
    {
        double best = 1e30;
        const int cand_rows[2] = {256, 128}, cand_bn[2] = {256, 128};
        for (int ri = 0; ri < 2; ++ri)
            for (int bi = 0; bi < 2; ++bi) {
                const int64_t t = ((N + cand_rows[ri] - 1) / cand_rows[ri]) * ((M + cand_bn[bi] - 1) / cand_bn[bi]);
                const int64_t waves = (t + num_sms() - 1) / num_sms();
                const double penalty = (cand_rows[ri] == 128 ? 1.25 : 1.0) * (cand_bn[bi] == 128 ? 1.5 : 1.0);   // measured
                const double cost = (double)waves * cand_rows[ri] * cand_bn[bi] * penalty;
                if (cost < best) { best = cost; rows = cand_rows[ri]; bn = cand_bn[bi]; }
            }
    }
    const cuuint32_t box[2] = {(cuuint32_t)kGemmBK, (cuuint32_t)bn};
    const cuuint32_t estr[2] = {1, 1};
    uint32_t* status_words = static_cast<uint32_t*>(workspace);
    void* x_f16 = convert ? static_cast<void*>(static_cast<uint8_t*>(workspace) + 256) : const_cast<void*>(x);
    if (encode(&tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, x_f16, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return OJX_ERR_LAUNCH;

    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(gemm_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kGemmSmemBytes) != cudaSuccess)
            return OJX_ERR_LAUNCH;
        configured = true;
    }
    if (cudaMemsetAsync(workspace, 0, 256, s) != cudaSuccess) return OJX_ERR_LAUNCH;
    if (convert) {
        const int64_t count = M * K;
        int64_t blocks = (count / 8 + 255) / 256 + 1;
        if (blocks > 148 * 8) blocks = 148 * 8;
        convert_bf16_to_f16_kernel<<<(unsigned)blocks, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x),
                                                                    static_cast<__half*>(x_f16), count, status_words + 1);
        rescale_bf16_to_f16_kernel<<<(unsigned)blocks, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x),
                                                                    static_cast<__half*>(x_f16), count, status_words + 1);
        if (cudaGetLastError() != cudaSuccess) return OJX_ERR_LAUNCH;
    }

    GemmParams prm;
    prm.packed = packed; prm.scales = scales; prm.bias = bias; prm.y = y;
    prm.status = static_cast<int32_t*>(workspace);
    prm.M = (int)M; prm.N = (int)N; prm.K = (int)K;
    prm.y_dtype = y_dtype; prm.bias_dtype = x_dtype;
    prm.amax_bits = convert ? status_words + 1 : nullptr;
    // instruction descriptor: fp32 accumulate (bits 4-5 = 1), A and B both fp16 (format 0), both K-major,
    // N >> 3 at bits 17-22, M >> 4 at bits 24-28
    prm.rows = rows; prm.bn = bn;
    prm.idesc = (1u << 4) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(kGemmHalf >> 4) << 24);

    const int tiles = (int)(((N + rows - 1) / rows) * ((M + bn - 1) / bn));
    const int grid = tiles < num_sms() ? tiles : num_sms();
    gemm_tcgen05_kernel<<<grid, kGemmThreads, kGemmSmemBytes, s>>>(tmap, prm);
    return launch_status();
}

int32_t gemm_status_impl(const void* workspace, cudaStream_t s) {
    OJX_RETURN_IF(!workspace, OJX_ERR_NULL);
    int32_t h = 0;
    if (cudaMemcpyAsync(&h, workspace, sizeof(h), cudaMemcpyDeviceToHost, s) != cudaSuccess) return OJX_ERR_LAUNCH;
    if (cudaStreamSynchronize(s) != cudaSuccess) return OJX_ERR_LAUNCH;
    return h == 0 ? OJX_OK : OJX_ERR_TIMEOUT;
}

}  // namespace ojx
