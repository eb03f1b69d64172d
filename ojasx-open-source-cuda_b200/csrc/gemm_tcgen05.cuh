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
// so bf16 activations are first rewritten as fp16 by a small pre-pass into caller-owned scratch:
// every token row is multiplied by its own power of two 2^-e so that its largest magnitude lands in
// [2^14, 2^15) (exact for every element within 28 binades of the row maximum; smaller ones keep an
// absolute error below 2^-39 of that maximum), and the epilogue multiplies the token's outputs by 2^e.
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
constexpr int kGemmDigitCopies = 16;
constexpr uint32_t kGemmLutBytes = 16384;                     // digit table: 81 x 16 copies x 8 bytes = 10368; a corrupt rank (up to 4095) stays inside
constexpr uint32_t kGemmSmemBytes = kGemmStages * (kXStageBytes + kAStageBytes) + kGemmLutBytes + 256 + 1024;

struct GemmParams {
    const uint8_t* packed;
    const uint16_t* scales;
    const void* bias;
    void* y;
    int32_t* status;
    int M, N, K;
    int y_stride;                  // elements between consecutive token rows of y (N of the whole matrix)
    int tile_limit;                // process only the first tile_limit tiles of the enumeration
    int y_dtype;
    int bias_dtype;
    uint32_t idesc;
    int rows;                      // weight rows per CTA tile: 128 or 256
    int bn;                        // tokens per CTA tile (MMA N): 128 or 256
    const float* up;               // per-token output factors 2^e written by the pre-pass (null: 1)
};

// Activation pre-pass: a group of TPR threads (a warp for rows of up to 4096 elements, else the whole CTA)
// takes one token row, finds its largest magnitude, then writes the row as fp16 scaled by the power of two
// that brings that magnitude into [2^14, 2^15), and the inverse factor for the epilogue.  Rows of up to
// TPR * 8 * VECS elements stay in registers between the two steps (one global read); longer rows are read
// twice.  The first thread also clears the status word the GEMM kernel reports through.
template <int TPR, int VECS>
__global__ void __launch_bounds__(256) normalize_rows_bf16_to_f16_kernel(const __nv_bfloat16* __restrict__ x,
                                                                          __half* __restrict__ out, float* __restrict__ up,
                                                                          int64_t M, int64_t K, int32_t* __restrict__ status) {
    __shared__ uint32_t warp_max[8];
    constexpr int kRowsPerCta = 256 / TPR;
    const int t = threadIdx.x % TPR;
    const int64_t row = (int64_t)blockIdx.x * kRowsPerCta + threadIdx.x / TPR;
    if (blockIdx.x == 0 && threadIdx.x == 0 && status != nullptr) *status = 0;
    const bool live = row < M;                                            // whole warps share `live`
    const uint4* src = reinterpret_cast<const uint4*>(x + (live ? row : 0) * K);   // K % 256 == 0: rows are 16-byte aligned
    uint4* dst = reinterpret_cast<uint4*>(out + (live ? row : 0) * K);
    const int64_t vecs = live ? K / 8 : 0;
    const bool resident = vecs <= (int64_t)TPR * VECS;
    uint4 keep[VECS];
    uint32_t m = 0;
    if (resident) {
#pragma unroll
        for (int j = 0; j < VECS; ++j) {
            const int64_t i = t + TPR * j;
            keep[j] = i < vecs ? __ldg(src + i) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int j = 0; j < VECS; ++j) {
            const uint32_t w[4] = {keep[j].x, keep[j].y, keep[j].z, keep[j].w};
#pragma unroll
            for (int q = 0; q < 4; ++q) m = max(m, max((w[q] << 16) & 0x7FFFFFFFu, w[q] & 0x7FFF0000u));
        }
    } else {
        for (int64_t i = t; i < vecs; i += TPR) {
            const uint4 v = __ldg(src + i);
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) m = max(m, max((w[q] << 16) & 0x7FFFFFFFu, w[q] & 0x7FFF0000u));
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    if (TPR > 32) {
        if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = m;
        __syncthreads();
#pragma unroll
        for (int w = 0; w < 8; ++w) m = max(m, warp_max[w]);
    }
    int e = 0;
    const int ex = (int)((m >> 23) & 0xFFu);
    if (ex != 0 && ex != 0xFF) e = max(-100, min(100, ex - 127 - 14));
    const float down = __int_as_float((127 - e) << 23);
    if (t == 0 && live) up[row] = __int_as_float((127 + e) << 23);
    auto convert = [&](const uint4& v) {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        uint32_t o[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const __half2 h = __floats2half2_rn(__uint_as_float(w[q] << 16) * down, __uint_as_float(w[q] & 0xFFFF0000u) * down);
            o[q] = *reinterpret_cast<const uint32_t*>(&h);
        }
        return make_uint4(o[0], o[1], o[2], o[3]);
    };
    if (resident) {
#pragma unroll
        for (int j = 0; j < VECS; ++j) {
            const int64_t i = t + TPR * j;
            if (i < vecs) dst[i] = convert(keep[j]);
        }
    } else {
        for (int64_t i = t; i < vecs; i += TPR) dst[i] = convert(__ldg(src + i));
    }
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
// MN-major operand tile with the 128-byte swizzle (used for the transposed product dX = dY . W): 64 consecutive
// "M" elements (here: k) are contiguous (one 128-byte row), eight consecutive "K" indices (here: weight rows n)
// form a 1024-byte swizzle atom; atoms follow each other along K every `kDxSbo` bytes and along M every `kDxLbo`.
constexpr uint32_t kDxSbo = 1024, kDxLbo = 8192;
__device__ __forceinline__ uint64_t umma_desc_mn_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);            // start address, 16-byte units
    d |= (uint64_t)(kDxLbo >> 4) << 16;                      // leading byte offset: next block of 64 M elements
    d |= (uint64_t)(kDxSbo >> 4) << 32;                      // stride byte offset: next group of eight K indices
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

// Thirty-two consecutive tokens of one weight row: scale by the token's power of two (lane i of `up_lane`
// holds the factor of token m0 + i), add bias, cast, store.  Lanes = consecutive weight rows, so every store
// instruction writes one contiguous run of y.
template <typename T>
__device__ __forceinline__ void gemm_store32(T* __restrict__ y, int64_t N, int n, int m0, int M, const uint32_t (&v)[32],
                                             float up_lane, float bias, bool live) {
    float f[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) f[i] = __shfl_sync(0xFFFFFFFFu, up_lane, i);     // all lanes, before any divergence
    if (!live) return;
    T* dst = y + (int64_t)m0 * N + n;
    if (m0 + 32 <= M) {                                                            // straight-line: the stores pipeline
#pragma unroll
        for (int i = 0; i < 32; ++i) dst[(int64_t)i * N] = static_cast<T>(fmaf(__uint_as_float(v[i]), f[i], bias));
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
            if (m0 + i < M) dst[(int64_t)i * N] = static_cast<T>(fmaf(__uint_as_float(v[i]), f[i], bias));
    }
}

// One epilogue warp's share of a finished tile: TMEM lanes 32 * warp .. of both row blocks, all token columns.
// Kept out of line so that its registers are allocated independently of the decoders' inner loop.
__device__ __noinline__ void gemm_drain_tile(void* __restrict__ y, int y_dtype, const void* __restrict__ bias_ptr, int bias_dtype,
                                             const float* __restrict__ up, int M, int N, int y_stride, int rows, int bn,
                                             uint32_t tmem_base, int warp, int lane, int n_blk, int m_blk) {
    const int blocks = bn / 32;
    for (int h = 0; h < rows / kGemmHalf; ++h) {
        const int n = n_blk * rows + h * kGemmHalf + warp * 32 + lane;
        const bool live = n < N;
        float bias = 0.f;
        if (bias_ptr != nullptr && live) bias = load_any(bias_ptr, bias_dtype, n);
        const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + h * kGemmBN;
        // Token factors (lane l keeps the factor of token m0 + l) and accumulator blocks both travel one
        // 32-token block ahead of their use, so neither the global nor the TMEM load latency is exposed.
        auto load_up = [&](int cb) {
            const int m = m_blk * bn + cb * 32 + lane;
            return (up != nullptr && cb < blocks && m < M) ? __ldg(up + m) : 1.0f;
        };
        auto store = [&](int cb, const uint32_t (&v)[32], float up_lane) {
            const int m0 = m_blk * bn + cb * 32;
            if (m0 >= M) return;                                   // warp-uniform
            if (y_dtype == OJX_BF16) gemm_store32(static_cast<__nv_bfloat16*>(y), y_stride, n, m0, M, v, up_lane, bias, live);
            else if (y_dtype == OJX_F16) gemm_store32(static_cast<__half*>(y), y_stride, n, m0, M, v, up_lane, bias, live);
            else gemm_store32(static_cast<float*>(y), y_stride, n, m0, M, v, up_lane, bias, live);
        };
        uint32_t va[32], vb[32];
        float ua = load_up(0), ub;
        tmem_ld_32x32b_x32(taddr, va);
#pragma unroll 1
        for (int cb = 0; cb < blocks; cb += 2) {                   // blocks is 4 or 8
            tmem_ld_wait();
            tmem_ld_32x32b_x32(taddr + (cb + 1) * 32, vb);
            ub = load_up(cb + 1);
            store(cb, va, ua);
            tmem_ld_wait();
            if (cb + 2 < blocks) tmem_ld_32x32b_x32(taddr + (cb + 2) * 32, va);
            ua = load_up(cb + 2);
            store(cb + 1, vb, ub);
        }
    }
}

__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
    const __half2 v = __hmul2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
    return *reinterpret_cast<const uint32_t*>(&v);
}

// kDX = false: y[M, N] = x . W^T, contraction over K (the weights' row direction), p.N = weight rows, p.K = columns.
// kDX = true:  dX[M, K] = dY . W, contraction over the weight ROWS.  The roles are swapped in the parameters: p.N is
//              the number of weight COLUMNS (the output's feature dimension, tiled like N above) and p.K the number
//              of weight rows (the contraction length, any positive value: the last block is zero-filled).  The
//              decoded weights enter the MMA as an MN-major operand, so a decoded rank is still one 16-byte store.
template <bool kDX, int kFmt = 0, int kG = 32> // kFmt: 0 ternary codes, 2 the 2.0-bit format, 1 the 1.0-bit format; kG: weights per scale (8 and 16 only for the sibling formats)
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

    // Digit table: entry e < 81 holds the four base-3 digits of e, each minus one, as fp16 (+-1.0 / 0), in sixteen
    // interleaved copies (one per lane of a half warp, so the 64-bit lookups never meet in a bank).  A rank r is
    // the base-3 number 2r (even coordinate sums are exactly the even numbers), so its eight coordinates are the
    // digits of (2r) mod 81 followed by those of (2r) div 81.
    if constexpr (kFmt == 0) {
        for (int i = tid; i < 81 * kGemmDigitCopies; i += kGemmThreads) {
            int e = i / kGemmDigitCopies;
            uint32_t h[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) { const int d = e % 3; e /= 3; h[k] = d == 0 ? 0xBC00u : (d == 1 ? 0u : 0x3C00u); }
            reinterpret_cast<uint2*>(lut)[i] = make_uint2(h[0] | (h[1] << 16), h[2] | (h[3] << 16));
        }
    } else if constexpr (kFmt == 2) {
        // 2.0-bit format: a code byte (four codes, code j in bits 2j) -> four fp16 values code - 1.5, eight interleaved copies
        for (int i = tid; i < 256 * 8; i += kGemmThreads) {
            const int e = i >> 3;
            uint32_t h[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) { const int c = (e >> (2 * k)) & 3; h[k] = c == 0 ? 0xBE00u : (c == 1 ? 0xB800u : (c == 2 ? 0x3800u : 0x3E00u)); }
            reinterpret_cast<uint2*>(lut)[i] = make_uint2(h[0] | (h[1] << 16), h[2] | (h[3] << 16));
        }
    } else {
        // 1.0-bit format: a code -> its eight coordinates (0, +-1, +-2) as fp16, four interleaved copies
        for (int i = tid; i < 256 * 4; i += kGemmThreads) {
            const int e = i >> 2;
            const uint32_t cw[2] = {g_root_coords[2 * e], g_root_coords[2 * e + 1]};
            uint32_t h[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const int c = (int)(int8_t)((cw[k >> 2] >> (8 * (k & 3))) & 0xFFu);
                h[k] = c == 0 ? 0u : (c == 1 ? 0x3C00u : (c == -1 ? 0xBC00u : (c == 2 ? 0x4000u : 0xC000u)));
            }
            reinterpret_cast<uint4*>(lut)[i] = make_uint4(h[0] | (h[1] << 16), h[2] | (h[3] << 16), h[4] | (h[5] << 16), h[6] | (h[7] << 16));
        }
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
    const int tiles = min(n_blocks * m_blocks, p.tile_limit);
    const int k_blocks = (p.K + kGemmBK - 1) / kGemmBK;

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
                        const uint32_t acc = (kb > 0 || k > 0) ? 1u : 0u;
                        if constexpr (kDX) {
                            // sixteen weight rows = two swizzle atoms along the contraction; 128 outputs = two 64-wide blocks
                            tc_mma_f16(tmem_base, umma_desc_mn_sw128(a_addr + k * 2 * kDxSbo), bd, p.idesc, acc);
                            if (p.rows == kGemmBM)
                                tc_mma_f16(tmem_base + kGemmBN, umma_desc_mn_sw128(a_addr + 2 * kDxLbo + k * 2 * kDxSbo), bd, p.idesc, acc);
                        } else {
                            tc_mma_f16(tmem_base, umma_desc_sw128(a_addr + k * 32), bd, p.idesc, acc);
                            if (p.rows == kGemmBM)
                                tc_mma_f16(tmem_base + kGemmBN, umma_desc_sw128(a_addr + kGemmHalf * 128 + k * 32), bd, p.idesc, acc);
                        }
                    }
                    tc_commit(empty_bar(s));           // frees the stage once these MMAs have read it
                }
                if (ok) tc_commit(tfull_bar(0));       // accumulators complete -> epilogue
            }
        }
    } else if (warp >= 4 && (warp - 4) * 32 < p.rows) {
        // ---------------- decoders (warps beyond the tile's rows stay idle) ----------------
        if constexpr (kDX) {
            // Thread (j, kq) of a stage decodes weight row kb*64 + j, columns [64 kq, 64 kq + 64) of the tile's column range:
            // eight ranks = 12 bytes of codes and two scales, each rank one 16-byte chunk of the MN-major tile.
            const int r = (warp - 4) * 32 + lane;
            const int j = r & 63, kq = r >> 6;
            // (the sibling formats: 16 or 8 bytes of codes; one or two reads of their table per 8 weights)
            const uint8_t* digit_lane = reinterpret_cast<const uint8_t*>(lut) +
                                        (kFmt == 0 ? (lane & (kGemmDigitCopies - 1)) * 8 : (kFmt == 2 ? (lane & 7) * 8 : (lane & 3) * 16));
            constexpr int kWords = kFmt == 0 ? 3 : (kFmt == 2 ? 4 : 2);            // 32-bit words of codes per 64 columns
            constexpr int kSW = 32 / kG;                                           // 32-bit words of scales per 64 columns
            const int64_t row_bytes = kFmt == 0 ? (int64_t)p.N * 3 / 16 : (kFmt == 2 ? p.N / 4 : p.N / 8), row_scales = p.N / kG;
            uint32_t it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
                const int n_blk = tile % n_blocks;
                const int col0 = n_blk * p.rows + kq * 64;                       // first weight column of this thread
                const uint8_t* cbase = p.packed + (kFmt == 0 ? (int64_t)col0 * 3 / 16 : (kFmt == 2 ? col0 / 4 : col0 / 8));
                const uint16_t* sbase = p.scales + col0 / kG;
                auto fetch = [&](int kb, uint32_t (&cw)[4], uint32_t (&sw)[kSW]) {
                    const int row = kb * kGemmBK + j;
                    if (row < p.K && col0 < p.N) {
                        const uint32_t* cp = reinterpret_cast<const uint32_t*>(cbase + (int64_t)row * row_bytes);
#pragma unroll
                        for (int i = 0; i < kWords; ++i) cw[i] = __ldg(cp + i);
#pragma unroll
                        for (int i = 0; i < kSW; ++i) sw[i] = __ldg(reinterpret_cast<const uint32_t*>(sbase + (int64_t)row * row_scales) + i);
                    } else if (kFmt == 0) {                                      // beyond the matrix: rank of the zero vector, scale 0
                        cw[0] = 0x68668668u; cw[1] = 0x86686686u; cw[2] = 0x66866866u;               // rank 1640 eight times
#pragma unroll
                        for (int i = 0; i < kSW; ++i) sw[i] = 0u;
                    } else {                                                     // any code, scale 0
                        cw[0] = cw[1] = cw[2] = cw[3] = 0u;
#pragma unroll
                        for (int i = 0; i < kSW; ++i) sw[i] = 0u;
                    }
                };
                uint32_t nw[4] = {0u, 0u, 0u, 0u}, ns[kSW];
                fetch(0, nw, ns);
                for (int kb = 0; kb < k_blocks && ok; ++kb, ++it) {
                    uint32_t cw[4] = {nw[0], nw[1], nw[2], kWords == 4 ? nw[3] : 0u};
                    uint32_t sw[kSW];
#pragma unroll
                    for (int i = 0; i < kSW; ++i) sw[i] = ns[i];
                    if (kb + 1 < k_blocks) fetch(kb + 1, nw, ns);                // the next stage's words travel during this one's decode
                    const int s = it % kGemmStages;
                    const uint32_t ph = (it / kGemmStages) & 1u;
                    if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, 4)) { ok = false; break; }
                    uint8_t* arow = smem + kGemmStages * kXStageBytes + s * kAStageBytes + kq * kDxLbo + (j >> 3) * kDxSbo + (j & 7) * 128;
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        uint2 lo8[4], hi8[4];
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const int c = half * 4 + q;
                            if constexpr (kFmt == 0) {
                                const int bit = 12 * c, w = bit >> 5, sh = bit & 31;
                                uint32_t R;                              // 2 * rank
                                if (sh + 12 <= 32) R = sh >= 1 ? (cw[w] >> (sh - 1)) : (cw[w] << 1);
                                else R = __funnelshift_r(cw[w], cw[w + 1], sh - 1);
                                R &= 0x1FFEu;
                                const uint32_t v = (R * 6473u) >> 19;    // R div 81 (exact for R < 6562)
                                const uint32_t u = R - 81u * v;
                                lo8[q] = *reinterpret_cast<const uint2*>(digit_lane + u * (kGemmDigitCopies * 8));
                                hi8[q] = *reinterpret_cast<const uint2*>(digit_lane + v * (kGemmDigitCopies * 8));
                            } else if constexpr (kFmt == 2) {            // two code bytes: codes 0-3 and 4-7 of the chunk
                                const uint32_t word = cw[c >> 1];
                                lo8[q] = *reinterpret_cast<const uint2*>(digit_lane + prmt(word, 0u, 0x4440u | (uint32_t)(2 * (c & 1))) * 64u);
                                hi8[q] = *reinterpret_cast<const uint2*>(digit_lane + prmt(word, 0u, 0x4440u | (uint32_t)(2 * (c & 1) + 1)) * 64u);
                            } else {                                     // one code byte
                                const uint4 e = *reinterpret_cast<const uint4*>(digit_lane + prmt(cw[c >> 2], 0u, 0x4440u | (uint32_t)(c & 3)) * 64u);
                                lo8[q] = make_uint2(e.x, e.y);
                                hi8[q] = make_uint2(e.z, e.w);
                            }
                        }
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const int c = half * 4 + q;
                            const int si = 8 * c / kG;                              // scale of this 8-weight chunk
                            const uint32_t sc2 = prmt(sw[si >> 1], 0u, (si & 1) == 0 ? 0x1010u : 0x3232u);
                            const uint4 v = make_uint4(hmul2_u32(lo8[q].x, sc2), hmul2_u32(lo8[q].y, sc2),
                                                       hmul2_u32(hi8[q].x, sc2), hmul2_u32(hi8[q].y, sc2));
                            *reinterpret_cast<uint4*>(arow + ((c ^ (j & 7)) << 4)) = v;
                        }
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) mbar_arrive(full_bar(s));
                }
            }
        } else if constexpr (kFmt != 0) {
        // The sibling formats: thread r owns weight row r of the tile; 256 k are 64 (2.0-bit) or 32 (1.0-bit) bytes of
        // codes and eight scales; every 8 weights are one table read (two for 2 bits) and four packed multiplies.
        const int r = (warp - 4) * 32 + lane;
        constexpr int kVec = kFmt == 2 ? 4 : 2;          // 16-byte vectors of codes per 256 k
        const uint8_t* tab_lane = reinterpret_cast<const uint8_t*>(lut) + (kFmt == 2 ? (lane & 7) * 8 : (lane & 3) * 16);   // entry stride 64 B
        uint32_t it = 0;
        bool ok = true;
        constexpr int kSV = 32 / kG;                     // 16-byte vectors of scales per 256 k
        const int64_t row_bytes = kFmt == 2 ? p.K / 4 : p.K / 8, row_scales = p.K / kG;
        for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
            const int n_blk = tile % n_blocks;
            const int row = min(n_blk * p.rows + r, p.N - 1);
            const uint4* cptr = reinterpret_cast<const uint4*>(p.packed + row * row_bytes);
            const uint4* sptr = reinterpret_cast<const uint4*>(p.scales + row * row_scales);
            const int chunks = p.K / 256;
            uint4 cv[kVec], sv[kSV];
#pragma unroll
            for (int i = 0; i < kVec; ++i) cv[i] = __ldg(cptr + i);
#pragma unroll
            for (int i = 0; i < kSV; ++i) sv[i] = __ldg(sptr + i);
            for (int ch = 0; ch < chunks && ok; ++ch) {
                uint32_t cw[4 * kVec], sw[4 * kSV];
#pragma unroll
                for (int i = 0; i < kVec; ++i) { cw[4 * i] = cv[i].x; cw[4 * i + 1] = cv[i].y; cw[4 * i + 2] = cv[i].z; cw[4 * i + 3] = cv[i].w; }
#pragma unroll
                for (int i = 0; i < kSV; ++i) { sw[4 * i] = sv[i].x; sw[4 * i + 1] = sv[i].y; sw[4 * i + 2] = sv[i].z; sw[4 * i + 3] = sv[i].w; }
                if (ch + 1 < chunks) {                   // prefetch the next 256 k of this row
#pragma unroll
                    for (int i = 0; i < kVec; ++i) cv[i] = __ldg(cptr + kVec * (ch + 1) + i);
#pragma unroll
                    for (int i = 0; i < kSV; ++i) sv[i] = __ldg(sptr + kSV * (ch + 1) + i);
                }
#pragma unroll
                for (int q = 0; q < 4; ++q, ++it) {
                    const int s = it % kGemmStages;
                    const uint32_t ph = (it / kGemmStages) & 1u;
                    if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, 4)) { ok = false; break; }
                    uint8_t* arow = smem + kGemmStages * kXStageBytes + s * kAStageBytes + r * 128;
#pragma unroll
                    for (int half = 0; half < 2; ++half) {                         // one scale group (32 k) = four 8-weight chunks
                        uint2 lo8[4], hi8[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const int jj = half * 4 + j;                           // chunk of the stage: k = 64 q + 8 jj ..
                            if constexpr (kFmt == 2) {                             // two code bytes
                                const uint32_t word = cw[4 * q + (jj >> 1)];
                                lo8[j] = *reinterpret_cast<const uint2*>(tab_lane + prmt(word, 0u, 0x4440u | (uint32_t)(2 * (jj & 1))) * 64u);
                                hi8[j] = *reinterpret_cast<const uint2*>(tab_lane + prmt(word, 0u, 0x4440u | (uint32_t)(2 * (jj & 1) + 1)) * 64u);
                            } else {                                               // one code byte
                                const uint32_t word = cw[2 * q + (jj >> 2)];
                                const uint4 e = *reinterpret_cast<const uint4*>(tab_lane + prmt(word, 0u, 0x4440u | (uint32_t)(jj & 3)) * 64u);
                                lo8[j] = make_uint2(e.x, e.y);
                                hi8[j] = make_uint2(e.z, e.w);
                            }
                        }
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const int jj = half * 4 + j;
                            const int si = (64 * q + 8 * jj) / kG;                 // scale of this 8-weight chunk inside the 256 k
                            const uint32_t sc2 = prmt(sw[si >> 1], 0u, (si & 1) == 0 ? 0x1010u : 0x3232u);
                            const uint4 v = make_uint4(hmul2_u32(lo8[j].x, sc2), hmul2_u32(lo8[j].y, sc2),
                                                       hmul2_u32(hi8[j].x, sc2), hmul2_u32(hi8[j].y, sc2));
                            *reinterpret_cast<uint4*>(arow + ((jj ^ (r & 7)) << 4)) = v;
                        }
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> async proxy (UMMA)
                    __syncwarp();
                    if (lane == 0) mbar_arrive(full_bar(s));
                }
            }
        }
        } else {
        const int r = (warp - 4) * 32 + lane;           // row of the 256-row tile
        const uint8_t* digit_lane = reinterpret_cast<const uint8_t*>(lut) + (lane & (kGemmDigitCopies - 1)) * 8;
        uint32_t it = 0;
        bool ok = true;
        constexpr int kSV = 32 / kG;                     // 16-byte vectors of scales per 256 k (groups of 32 or 16)
        const int64_t row_bytes = (int64_t)p.K * 3 / 16, row_scales = p.K / kG;
        for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
            const int n_blk = tile % n_blocks;
            const int row = min(n_blk * p.rows + r, p.N - 1);
            const uint4* cptr = reinterpret_cast<const uint4*>(p.packed + row * row_bytes);
            const uint4* sptr = reinterpret_cast<const uint4*>(p.scales + row * row_scales);
            const int chunks = p.K / 256;
            uint4 c0 = __ldg(cptr), c1 = __ldg(cptr + 1), c2 = __ldg(cptr + 2), sv[kSV];
#pragma unroll
            for (int i = 0; i < kSV; ++i) sv[i] = __ldg(sptr + i);
            for (int ch = 0; ch < chunks && ok; ++ch) {
                uint32_t cw[12] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w, c2.x, c2.y, c2.z, c2.w};
                uint32_t sw[4 * kSV];
#pragma unroll
                for (int i = 0; i < kSV; ++i) { sw[4 * i] = sv[i].x; sw[4 * i + 1] = sv[i].y; sw[4 * i + 2] = sv[i].z; sw[4 * i + 3] = sv[i].w; }
                if (ch + 1 < chunks) {                   // prefetch the next 256 k of this row
                    c0 = __ldg(cptr + 3 * (ch + 1)); c1 = __ldg(cptr + 3 * (ch + 1) + 1);
                    c2 = __ldg(cptr + 3 * (ch + 1) + 2);
#pragma unroll
                    for (int i = 0; i < kSV; ++i) sv[i] = __ldg(sptr + kSV * (ch + 1) + i);
                }
#pragma unroll
                for (int q = 0; q < 4; ++q, ++it) {
                    const int s = it % kGemmStages;
                    const uint32_t ph = (it / kGemmStages) & 1u;
                    if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, 4)) { ok = false; break; }
                    uint8_t* arow = smem + kGemmStages * kXStageBytes + s * kAStageBytes + r * 128;
                    // Four ranks at a time: their lookups are issued before the first store (the compiler must
                    // assume a shared-memory store may alias the table).
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        uint2 lo8[4], hi8[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const int c = q * 8 + half * 4 + j;      // rank index inside the 48-byte chunk
                            const int bit = 12 * c, w = bit >> 5, sh = bit & 31;
                            uint32_t R;                              // 2 * rank
                            if (sh + 12 <= 32) R = sh >= 1 ? (cw[w] >> (sh - 1)) : (cw[w] << 1);
                            else R = __funnelshift_r(cw[w], cw[w + 1 < 12 ? w + 1 : 11], sh - 1);
                            R &= 0x1FFEu;
                            const uint32_t v = (R * 6473u) >> 19;    // R div 81 (exact for R < 6562)
                            const uint32_t u = R - 81u * v;
                            lo8[j] = *reinterpret_cast<const uint2*>(digit_lane + u * (kGemmDigitCopies * 8));   // coordinates 0-3
                            hi8[j] = *reinterpret_cast<const uint2*>(digit_lane + v * (kGemmDigitCopies * 8));   // coordinates 4-7
                        }
                        // the four ranks of a half are one scale group of 32, or two of 16
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const int jj = half * 4 + j;
                            const int si = (64 * q + 8 * jj) / kG;
                            const uint32_t sc2 = prmt(sw[si >> 1], 0u, (si & 1) == 0 ? 0x1010u : 0x3232u);
                            const uint4 v = make_uint4(hmul2_u32(lo8[j].x, sc2), hmul2_u32(lo8[j].y, sc2),
                                                       hmul2_u32(hi8[j].x, sc2), hmul2_u32(hi8[j].y, sc2));
                            *reinterpret_cast<uint4*>(arow + ((jj ^ (r & 7)) << 4)) = v;
                        }
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> async proxy (UMMA)
                    __syncwarp();
                    if (lane == 0) mbar_arrive(full_bar(s));
                }
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
            gemm_drain_tile(p.y, p.y_dtype, p.bias, p.bias_dtype, p.up, p.M, p.N, p.y_stride, p.rows, p.bn, tmem_base, warp, lane, n_blk, m_blk);
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

// The kernel instance for a format and a scale-group size (null: not built), and its slot in the per-kernel tables.
using GemmKernelFn = void (*)(const CUtensorMap, const GemmParams);
template <bool kDX>
inline GemmKernelFn gemm_kernel_for(int fmt, int group, int* slot) {
    if (fmt == 0 && group == 32) { *slot = 0; return gemm_tcgen05_kernel<kDX, 0, 32>; }
    if (fmt == 0 && group == 16) { *slot = 7; return gemm_tcgen05_kernel<kDX, 0, 16>; }
    if (fmt == 2 && group == 32) { *slot = 1; return gemm_tcgen05_kernel<kDX, 2, 32>; }
    if (fmt == 2 && group == 16) { *slot = 2; return gemm_tcgen05_kernel<kDX, 2, 16>; }
    if (fmt == 2 && group == 8) { *slot = 3; return gemm_tcgen05_kernel<kDX, 2, 8>; }
    if (fmt == 1 && group == 32) { *slot = 4; return gemm_tcgen05_kernel<kDX, 1, 32>; }
    if (fmt == 1 && group == 16) { *slot = 5; return gemm_tcgen05_kernel<kDX, 1, 16>; }
    if (fmt == 1 && group == 8) { *slot = 6; return gemm_tcgen05_kernel<kDX, 1, 8>; }
    return nullptr;
}

inline bool gemm_fast_ok(int64_t M, int64_t N, int64_t K, int group, int x_dtype) {
    return M >= 1 && N >= 1 && K >= 256 && K % 256 == 0 && group == 32 &&
           (x_dtype == OJX_BF16 || x_dtype == OJX_F16) && M < (1 << 30) && N < (1 << 30) && K < (1 << 30);
}

// Scratch: a 256-byte status block (word 0: give-up code of a bounded wait; zeroed by every call), the
// per-token output factors (M floats, padded to 256 bytes), then room for an fp16 copy of the activations.
inline size_t gemm_up_bytes(int64_t M) { return (((size_t)M * 4) + 255) & ~(size_t)255; }
size_t gemm_workspace_bytes_impl(int64_t M, int64_t N, int64_t K) {
    (void)N;
    if (M <= 0 || K <= 0) return 256;
    return 256 + gemm_up_bytes(M) + (size_t)M * (size_t)K * 2;
}

// fmt: 0 ternary codes (3 bytes per 16 weights), 2 the 2.0-bit format (one byte per 4 weights, weight =
// (code - 1.5) * scale rounded to fp16 once, exactly the fp16 output of its decoder), 1 the 1.0-bit format (one byte
// per 8 weights, coordinate * scale exact in fp16).
int32_t gemm_fmt_impl(int fmt, const void* x, int x_dtype, int64_t M, const uint8_t* packed, const uint16_t* scales,
                      const void* bias, int64_t N, int64_t K, int group, void* y, int y_dtype,
                      void* workspace, size_t workspace_bytes, cudaStream_t s) {
    OJX_RETURN_IF(!x || !packed || !scales || !y, OJX_ERR_NULL);
    OJX_RETURN_IF(fmt != 0 && fmt != 1 && fmt != 2, OJX_ERR_UNSUPPORTED);
    OJX_RETURN_IF(M <= 0 || N <= 0 || K <= 0, OJX_ERR_SHAPE);
    OJX_RETURN_IF(dtype_size(x_dtype) == 0 || dtype_size(y_dtype) == 0, OJX_ERR_DTYPE);
    OJX_RETURN_IF(check_arch() != OJX_OK, OJX_ERR_ARCH);
    if (fmt == 0) group = effective_group(group);
    int slot = 0;
    const GemmKernelFn kernel = gemm_kernel_for<false>(fmt, group, &slot);      // sibling formats: groups of 8, 16 or 32
    OJX_RETURN_IF(kernel == nullptr || !gemm_fast_ok(M, N, K, 32, x_dtype), OJX_ERR_UNSUPPORTED);
    OJX_RETURN_IF(((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(packed) |
                    reinterpret_cast<uintptr_t>(scales)) & 15) != 0, OJX_ERR_ALIGN);
    const bool convert = x_dtype == OJX_BF16;
    const size_t need = convert ? gemm_workspace_bytes_impl(M, N, K) : 256;
    OJX_RETURN_IF(!workspace || workspace_bytes < need, OJX_ERR_WORKSPACE);
    OJX_RETURN_IF((reinterpret_cast<uintptr_t>(workspace) & 255) != 0, OJX_ERR_ALIGN);
    PFN_encodeTiled encode = get_encode_tiled();
    OJX_RETURN_IF(encode == nullptr, OJX_ERR_LAUNCH);

    float* up = convert ? reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + 256) : nullptr;
    void* x_f16 = convert ? static_cast<void*>(static_cast<uint8_t*>(workspace) + 256 + gemm_up_bytes(M)) : const_cast<void*>(x);

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

    static std::atomic<uint64_t> configured[8];                  // per kernel; one bit per device: the opt-in is per context
    OJX_RETURN_IF(ensure_dynamic_smem(kernel, kGemmSmemBytes, configured[slot]) != OJX_OK, OJX_ERR_LAUNCH);
    if (convert) {
        if (K <= 4096)
            normalize_rows_bf16_to_f16_kernel<32, 16><<<(unsigned)((M + 7) / 8), 256, 0, s>>>(
                static_cast<const __nv_bfloat16*>(x), static_cast<__half*>(x_f16), up, M, K, static_cast<int32_t*>(workspace));
        else
            normalize_rows_bf16_to_f16_kernel<256, 8><<<(unsigned)M, 256, 0, s>>>(
                static_cast<const __nv_bfloat16*>(x), static_cast<__half*>(x_f16), up, M, K, static_cast<int32_t*>(workspace));
        if (cudaGetLastError() != cudaSuccess) return OJX_ERR_LAUNCH;
    } else if (cudaMemsetAsync(workspace, 0, 4, s) != cudaSuccess) {
        return OJX_ERR_LAUNCH;
    }

    // One launch over the rectangle of weight rows [n0, N) x tokens [m0, M) of the problem, in tiles of
    // rows x bn, stopping after tile_limit tiles of the enumeration (token block major, weight-row block minor).
    auto launch_region = [&](int64_t n0, int64_t m0, int rows, int bn, int tile_limit) -> int32_t {
        const int64_t Ns = N - n0, Ms = M - m0;
        CUtensorMap tmap;
        const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)Ms};
        const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
        const cuuint32_t box[2] = {(cuuint32_t)kGemmBK, (cuuint32_t)bn};
        const cuuint32_t estr[2] = {1, 1};
        void* xs = static_cast<uint8_t*>(x_f16) + (size_t)m0 * (size_t)K * 2;
        if (encode(&tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, xs, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return OJX_ERR_LAUNCH;
        GemmParams prm;
        prm.packed = packed + (fmt == 0 ? (size_t)n0 * (size_t)K * 3 / 16 : (size_t)n0 * (size_t)K / (fmt == 2 ? 4 : 8));
        prm.scales = scales + (size_t)n0 * (size_t)K / (size_t)group;
        prm.bias = bias ? static_cast<const uint8_t*>(bias) + (size_t)n0 * dtype_size(x_dtype) : nullptr;
        prm.y = static_cast<uint8_t*>(y) + ((size_t)m0 * (size_t)N + (size_t)n0) * dtype_size(y_dtype);
        prm.status = static_cast<int32_t*>(workspace);
        prm.M = (int)Ms; prm.N = (int)Ns; prm.K = (int)K;
        prm.y_stride = (int)N;
        prm.y_dtype = y_dtype; prm.bias_dtype = x_dtype;
        prm.up = up ? up + m0 : nullptr;
        prm.rows = rows; prm.bn = bn;
        // instruction descriptor: fp32 accumulate (bits 4-5 = 1), A and B both fp16 (format 0), both K-major,
        // N >> 3 at bits 17-22, M >> 4 at bits 24-28
        prm.idesc = (1u << 4) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(kGemmHalf >> 4) << 24);
        const int64_t all = ((Ns + rows - 1) / rows) * ((Ms + bn - 1) / bn);
        prm.tile_limit = (int)(all < tile_limit ? all : tile_limit);
        const int grid = prm.tile_limit < num_sms() ? prm.tile_limit : num_sms();
        kernel<<<grid, kGemmThreads, kGemmSmemBytes, s>>>(tmap, prm);
        return launch_status();
    };

    // Tail splitting: when the last wave of big tiles would leave most SMs idle, the big tiles stop at a whole
    // number of waves and the remaining rectangle (the end of the last token block) runs as small tiles.
    const int sms = num_sms();
    const int64_t n_blocks = (N + rows - 1) / rows, m_blocks = (M + bn - 1) / bn;
    const int64_t tiles = n_blocks * m_blocks;
    const int64_t full = (tiles / sms) * sms, leftover = tiles - full;
    if (rows == kGemmBM && bn == kGemmBN && full > 0 && leftover > 0 && leftover <= n_blocks && 4 * leftover <= 2 * sms) {
        const int32_t st = launch_region(0, 0, rows, bn, (int)full);
        if (st != OJX_OK) return st;
        return launch_region((n_blocks - leftover) * rows, (m_blocks - 1) * bn, kGemmHalf, 128, 1 << 30);
    }
    return launch_region(0, 0, rows, bn, 1 << 30);
}

int32_t gemm_impl(const void* x, int x_dtype, int64_t M, const uint8_t* packed, const uint16_t* scales,
                  const void* bias, int64_t N, int64_t K, int group, void* y, int y_dtype,
                  void* workspace, size_t workspace_bytes, cudaStream_t s) {
    return gemm_fmt_impl(0, x, x_dtype, M, packed, scales, bias, N, K, group, y, y_dtype, workspace, workspace_bytes, s);
}

// dX[M, K] = dY[M, N] . W[N, K] without ever materialising W (the backward of the linear with respect to its
// input: ojasx2/math/lattice.py:642-717, native form ojasx2/math/csrc/ojasx_math_core.hpp:641-702).
// Same pipeline as the forward kernel; the contraction runs over the weight rows.
inline bool gemm_dx_ok(int64_t M, int64_t N, int64_t K, int group, int gy_dtype) {
    return M >= 1 && N >= 8 && N % 8 == 0 && K >= 256 && K % 256 == 0 && group == 32 &&
           (gy_dtype == OJX_BF16 || gy_dtype == OJX_F16) && M < (1 << 30) && N < (1 << 30) && K < (1 << 30);
}
size_t gemm_dx_workspace_bytes_impl(int64_t M, int64_t N, int64_t K) {
    (void)K;
    if (M <= 0 || N <= 0) return 256;
    return 256 + gemm_up_bytes(M) + (size_t)M * (size_t)N * 2;
}

int32_t gemm_dx_fmt_impl(int fmt, const void* gy, int gy_dtype, int64_t M, const uint8_t* packed, const uint16_t* scales,
                         int64_t N, int64_t K, int group, void* dx, int dx_dtype,
                         void* workspace, size_t workspace_bytes, cudaStream_t s) {
    OJX_RETURN_IF(!gy || !packed || !scales || !dx, OJX_ERR_NULL);
    OJX_RETURN_IF(fmt != 0 && fmt != 1 && fmt != 2, OJX_ERR_UNSUPPORTED);
    OJX_RETURN_IF(M <= 0 || N <= 0 || K <= 0, OJX_ERR_SHAPE);
    OJX_RETURN_IF(dtype_size(gy_dtype) == 0 || dtype_size(dx_dtype) == 0, OJX_ERR_DTYPE);
    OJX_RETURN_IF(check_arch() != OJX_OK, OJX_ERR_ARCH);
    if (fmt == 0) group = effective_group(group);
    int slot = 0;
    const GemmKernelFn kernel = gemm_kernel_for<true>(fmt, group, &slot);
    OJX_RETURN_IF(kernel == nullptr || !gemm_dx_ok(M, N, K, 32, gy_dtype), OJX_ERR_UNSUPPORTED);
    OJX_RETURN_IF(((reinterpret_cast<uintptr_t>(gy) | reinterpret_cast<uintptr_t>(packed) |
                    reinterpret_cast<uintptr_t>(scales)) & 15) != 0, OJX_ERR_ALIGN);
    const bool convert = gy_dtype == OJX_BF16;
    const size_t need = convert ? gemm_dx_workspace_bytes_impl(M, N, K) : 256;
    OJX_RETURN_IF(!workspace || workspace_bytes < need, OJX_ERR_WORKSPACE);
    OJX_RETURN_IF((reinterpret_cast<uintptr_t>(workspace) & 255) != 0, OJX_ERR_ALIGN);
    PFN_encodeTiled encode = get_encode_tiled();
    OJX_RETURN_IF(encode == nullptr, OJX_ERR_LAUNCH);

    float* up = convert ? reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + 256) : nullptr;
    void* gy_f16 = convert ? static_cast<void*>(static_cast<uint8_t*>(workspace) + 256 + gemm_up_bytes(M)) : const_cast<void*>(gy);

    // tile shape over (K outputs) x (M tokens): same cost model as the forward launch
    int rows = kGemmBM, bn = kGemmBN;
    {
        double best = 1e30;
        const int cand_rows[2] = {256, 128}, cand_bn[2] = {256, 128};
        for (int ri = 0; ri < 2; ++ri)
            for (int bi = 0; bi < 2; ++bi) {
                const int64_t t = ((K + cand_rows[ri] - 1) / cand_rows[ri]) * ((M + cand_bn[bi] - 1) / cand_bn[bi]);
                const int64_t waves = (t + num_sms() - 1) / num_sms();
                const double penalty = (cand_rows[ri] == 128 ? 1.25 : 1.0) * (cand_bn[bi] == 128 ? 1.5 : 1.0);
                const double cost = (double)waves * cand_rows[ri] * cand_bn[bi] * penalty;
                if (cost < best) { best = cost; rows = cand_rows[ri]; bn = cand_bn[bi]; }
            }
    }
    static std::atomic<uint64_t> configured[8];
    OJX_RETURN_IF(ensure_dynamic_smem(kernel, kGemmSmemBytes, configured[slot]) != OJX_OK, OJX_ERR_LAUNCH);
    if (convert) {
        // per-token power-of-two factors exactly as in the forward launch; rows here are N long (any multiple of 8)
        if (N <= 4096)
            normalize_rows_bf16_to_f16_kernel<32, 16><<<(unsigned)((M + 7) / 8), 256, 0, s>>>(
                static_cast<const __nv_bfloat16*>(gy), static_cast<__half*>(gy_f16), up, M, N, static_cast<int32_t*>(workspace));
        else
            normalize_rows_bf16_to_f16_kernel<256, 8><<<(unsigned)M, 256, 0, s>>>(
                static_cast<const __nv_bfloat16*>(gy), static_cast<__half*>(gy_f16), up, M, N, static_cast<int32_t*>(workspace));
        if (cudaGetLastError() != cudaSuccess) return OJX_ERR_LAUNCH;
    } else if (cudaMemsetAsync(workspace, 0, 4, s) != cudaSuccess) {
        return OJX_ERR_LAUNCH;
    }
    CUtensorMap tmap;
    const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)M};
    const cuuint64_t strides[1] = {(cuuint64_t)N * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kGemmBK, (cuuint32_t)bn};
    const cuuint32_t estr[2] = {1, 1};
    if (encode(&tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, gy_f16, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return OJX_ERR_LAUNCH;
    GemmParams prm;
    prm.packed = packed; prm.scales = scales; prm.bias = nullptr;
    prm.y = dx;
    prm.status = static_cast<int32_t*>(workspace);
    prm.M = (int)M;
    prm.N = (int)K;                    // roles swapped: the output's feature dimension is the weight columns ...
    prm.K = (int)N;                    // ... and the contraction runs over the weight rows
    prm.y_stride = (int)K;
    prm.y_dtype = dx_dtype; prm.bias_dtype = gy_dtype;
    prm.up = up;
    prm.rows = rows; prm.bn = bn;
    // as the forward descriptor, plus bit 15: the A operand is MN-major
    prm.idesc = (1u << 4) | (1u << 15) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(kGemmHalf >> 4) << 24);
    const int64_t all = ((K + rows - 1) / rows) * ((M + bn - 1) / bn);
    prm.tile_limit = (int)(all < (1 << 30) ? all : (1 << 30));
    const int grid = prm.tile_limit < num_sms() ? prm.tile_limit : num_sms();
    kernel<<<grid, kGemmThreads, kGemmSmemBytes, s>>>(tmap, prm);
    return launch_status();
}

int32_t gemm_dx_impl(const void* gy, int gy_dtype, int64_t M, const uint8_t* packed, const uint16_t* scales,
                     int64_t N, int64_t K, int group, void* dx, int dx_dtype,
                     void* workspace, size_t workspace_bytes, cudaStream_t s) {
    return gemm_dx_fmt_impl(0, gy, gy_dtype, M, packed, scales, N, K, group, dx, dx_dtype, workspace, workspace_bytes, s);
}

int32_t gemm_status_impl(const void* workspace, cudaStream_t s) {
    OJX_RETURN_IF(!workspace, OJX_ERR_NULL);
    int32_t h = 0;
    if (cudaMemcpyAsync(&h, workspace, sizeof(h), cudaMemcpyDeviceToHost, s) != cudaSuccess) return OJX_ERR_LAUNCH;
    if (cudaStreamSynchronize(s) != cudaSuccess) return OJX_ERR_LAUNCH;
    return h == 0 ? OJX_OK : OJX_ERR_TIMEOUT;
}

}  // namespace ojx
