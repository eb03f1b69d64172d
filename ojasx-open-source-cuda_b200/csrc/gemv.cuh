// Decode-shape fused linear: y[M,N] = x[M,K] . dequant(W)[N,K]^T for small M.
//
// Replaces, for small batches, _FusedE8GEMMFunction.forward (ojasx2/math/lattice.py:551-640)
// and the reference's scalar fused kernel (ojasx2/math/csrc/ojasx_math_core.hpp:580-634):
// per (m, n) the result is sum over groups of (sum_k x*coord) * scale, accumulated in fp32.
//
// Fast path (K % 256 == 0, bf16/fp16 activations, M <= 16)
//   * one CTA = 16 warps; warp w owns one 256-wide slice of K and keeps that slice of x in
//     registers as mma.m16n8k16 B fragments, so activations are read once per CTA;
//   * a work item is 16 weight rows x one K chunk (= all slices of the CTA); per item a lane
//     streams 48 B of codes + 16 B of scales per row with 128-bit loads (the next item's loads
//     are issued before the current item is decoded);
//   * a 12-bit rank is turned into eight trits by ONE shared-memory lookup; the table is stored
//     eight times (stride 32 B) so that lanes of different lane%8 never collide on a bank;
//   * trits become +-2.0 / 0 fp16|bf16 operand registers with byte permutes, the MACs run on the
//     tensor cores, and the group scale (times 1/2) is applied to the fp32 fragment per group;
//   * warps' partial sums are combined in a fixed order through shared memory (deterministic).
// K larger than one CTA's 16 slices is split into chunks whose fp32 partials go to caller-owned
// scratch and are summed, again in a fixed order, by a second small kernel.
#pragma once

#include "common.cuh"

namespace ojx {

constexpr int kGemvWarps = 16;
constexpr int kGemvThreads = kGemvWarps * 32;
constexpr int kLutCopies = 8;
constexpr int kLutEntries = 4096;                                  // any 12-bit code stays in bounds
constexpr int kLutBytes = kLutEntries * kLutCopies * 4;            // 131072

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

// One row's share of a work item: 48 B of codes (32 ranks = 8 groups) and 8 fp16 scales.
struct RowSlice {
    uint4 c[3];
    uint4 s;
};

__device__ __forceinline__ void load_row_slice(RowSlice& r, const uint8_t* codes, const uint16_t* scales) {
    const uint4* cp = reinterpret_cast<const uint4*>(codes);
    r.c[0] = __ldg(cp);
    r.c[1] = __ldg(cp + 1);
    r.c[2] = __ldg(cp + 2);
    r.s = __ldg(reinterpret_cast<const uint4*>(scales));
}

struct ItemCtx {
    int prob, chunk, tile;
};

__device__ __forceinline__ ItemCtx locate_item(const ojx_e8t_gemv_problem* probs, int count, int item, int hint) {
    int p = hint;
    while (p + 1 < count && probs[p + 1].tile_begin <= item) ++p;
    const int local = item - probs[p].tile_begin;
    const int tiles = gemv_row_tiles(probs[p].N);
    ItemCtx c;
    c.prob = p;
    c.chunk = local / tiles;
    c.tile = local - c.chunk * tiles;
    return c;
}

template <typename T> __device__ __forceinline__ void store_out(void* y, int y_dtype, int64_t idx, float v) {
    (void)y_dtype;
    static_cast<T*>(y)[idx] = from_f32<T>(v);
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

template <bool kBf16, int NB>
__global__ void __launch_bounds__(kGemvThreads, 1)
gemv_mma_kernel(const ojx_e8t_gemv_problem* __restrict__ probs_dev, const __grid_constant__ ojx_e8t_gemv_problem single,
                int count, int total_items, int M, int y_dtype) {
    // A single problem travels by value in the kernel parameters; a list lives in device memory.
    const ojx_e8t_gemv_problem* probs = probs_dev != nullptr ? probs_dev : &single;
    extern __shared__ __align__(16) uint8_t smem[];
    uint32_t* lut = reinterpret_cast<uint32_t*>(smem);
    float* red = reinterpret_cast<float*>(smem + kLutBytes);        // [2][warps][32][4*NB]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;

    for (int i = tid; i < kLutEntries * kLutCopies; i += kGemvThreads) {
        const int r = i >> 3;
        lut[i] = r < kNumPoints ? g_trit_nibbles[r] : 0u;
    }
    __syncthreads();

    const int64_t per = ((int64_t)total_items + gridDim.x - 1) / gridDim.x;
    const int i0 = (int)min((int64_t)total_items, per * blockIdx.x);
    const int i1 = (int)min((int64_t)total_items, per * (blockIdx.x + 1));
    if (i0 >= i1) return;

    // lane-constant decode parameters
    const uint32_t bt = (t == 0) ? 0u : (t == 1) ? 1u : (t == 2) ? 3u : 4u;     // first byte of this lane's rank
    const uint32_t sel_even = bt | ((bt + 1) << 4);
    const uint32_t sel_odd = (bt + 2) | ((bt + 3) << 4);
    const uint32_t lsh = (t & 1) ? 1u : 5u;
    const uint32_t lut_lane = smem_u32(lut) + ((lane & 7) << 2);
    constexpr uint32_t kConstH = 0x00C04000u;                         // byte 1: +2.0 high byte, byte 2: -2.0

    uint32_t xf[NB][8][4];
    int cur_prob = -1, cur_chunk = -1;
    int hint = 0;

    ItemCtx ctx = locate_item(probs, count, i0, 0);
    hint = ctx.prob;
    RowSlice ra, rb;                       // current item
    ra.c[0] = ra.c[1] = ra.c[2] = ra.s = make_uint4(0, 0, 0, 0);
    rb = ra;
    int active = 0;
    {
        const ojx_e8t_gemv_problem& P = probs[ctx.prob];
        active = gemv_active_warps(P.K);
        if (warp < active) {
            const int64_t row_bytes = (int64_t)P.K * 3 / 16, row_scales = P.K / 32;
            const int slice = ctx.chunk * active + warp;
            const int r0 = min(ctx.tile * 16 + g, P.N - 1), r1 = min(ctx.tile * 16 + g + 8, P.N - 1);
            load_row_slice(ra, P.packed + r0 * row_bytes + slice * 48, P.scales + r0 * row_scales + slice * 8);
            load_row_slice(rb, P.packed + r1 * row_bytes + slice * 48, P.scales + r1 * row_scales + slice * 8);
        }
    }

    int buf = 0;
    for (int item = i0; item < i1; ++item) {
        const ojx_e8t_gemv_problem& P = probs[ctx.prob];
        const int act = active;
        // (re)load this warp's activations when the problem or the K chunk changes
        if (ctx.prob != cur_prob || ctx.chunk != cur_chunk) {
            cur_prob = ctx.prob;
            cur_chunk = ctx.chunk;
            if (warp < act) {
                const int slice = ctx.chunk * act + warp;
#pragma unroll
                for (int nb = 0; nb < NB; ++nb) {
                    const int m = nb * 8 + g;
#pragma unroll
                    for (int grp = 0; grp < 8; ++grp) {
                        uint4 v = make_uint4(0, 0, 0, 0);
                        if (m < M)
                            v = __ldg(reinterpret_cast<const uint4*>(
                                static_cast<const uint16_t*>(P.x) + (int64_t)m * P.K + slice * 256 + grp * 32 + t * 8));
                        xf[nb][grp][0] = v.x; xf[nb][grp][1] = v.y; xf[nb][grp][2] = v.z; xf[nb][grp][3] = v.w;
                    }
                }
            }
        }

        // issue the next item's loads before decoding this one
        ItemCtx nctx = ctx;
        RowSlice na = ra, nbq = rb;
        int nactive = act;
        const bool has_next = item + 1 < i1;
        if (has_next) {
            nctx = locate_item(probs, count, item + 1, hint);
            hint = nctx.prob;
            const ojx_e8t_gemv_problem& Q = probs[nctx.prob];
            nactive = gemv_active_warps(Q.K);
            if (warp < nactive) {
                const int64_t row_bytes = (int64_t)Q.K * 3 / 16, row_scales = Q.K / 32;
                const int slice = nctx.chunk * nactive + warp;
                const int r0 = min(nctx.tile * 16 + g, Q.N - 1), r1 = min(nctx.tile * 16 + g + 8, Q.N - 1);
                load_row_slice(na, Q.packed + r0 * row_bytes + slice * 48, Q.scales + r0 * row_scales + slice * 8);
                load_row_slice(nbq, Q.packed + r1 * row_bytes + slice * 48, Q.scales + r1 * row_scales + slice * 8);
            }
        }

        float acc[NB][4];
#pragma unroll
        for (int nb = 0; nb < NB; ++nb)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[nb][i] = 0.f;

        if (warp < act) {
            const uint32_t* ca = reinterpret_cast<const uint32_t*>(ra.c);
            const uint32_t* cb = reinterpret_cast<const uint32_t*>(rb.c);
            const uint32_t* sa = reinterpret_cast<const uint32_t*>(&ra.s);
            const uint32_t* sb = reinterpret_cast<const uint32_t*>(&rb.s);
#pragma unroll
            for (int grp = 0; grp < 8; ++grp) {
                constexpr int dummy = 0; (void)dummy;
                const int w0 = (grp & 1) ? (3 * grp - 1) / 2 : (3 * grp) / 2;
                const uint32_t sel = (grp & 1) ? sel_odd : sel_even;
                const uint32_t wa = prmt(ca[w0], ca[w0 + 1], sel);
                const uint32_t wb = prmt(cb[w0], cb[w0 + 1], sel);
                const uint32_t na_ = lds_u32(((wa << lsh) & 0x1FFE0u) + lut_lane);
                const uint32_t nb_ = lds_u32(((wb << lsh) & 0x1FFE0u) + lut_lane);
                const uint32_t ha_lo = prmt(kConstH, 0u, na_), ha_hi = prmt(kConstH, 0u, na_ >> 16);
                const uint32_t hb_lo = prmt(kConstH, 0u, nb_), hb_hi = prmt(kConstH, 0u, nb_ >> 16);
                uint32_t a1[4], a2[4];
                a1[0] = prmt(ha_lo, 0u, 0x1404u); a1[2] = prmt(ha_lo, 0u, 0x3424u);
                a1[1] = prmt(hb_lo, 0u, 0x1404u); a1[3] = prmt(hb_lo, 0u, 0x3424u);
                a2[0] = prmt(ha_hi, 0u, 0x1404u); a2[2] = prmt(ha_hi, 0u, 0x3424u);
                a2[1] = prmt(hb_hi, 0u, 0x1404u); a2[3] = prmt(hb_hi, 0u, 0x3424u);
                const uint32_t spa = sa[grp >> 1], spb = sb[grp >> 1];
                const float fa = 0.5f * __half2float(__ushort_as_half((uint16_t)((grp & 1) ? (spa >> 16) : (spa & 0xFFFFu))));
                const float fb = 0.5f * __half2float(__ushort_as_half((uint16_t)((grp & 1) ? (spb >> 16) : (spb & 0xFFFFu))));
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
        }

        // deterministic cross-warp sum through shared memory
        float* rbuf = red + (size_t)buf * kGemvWarps * 32 * 4 * NB;
#pragma unroll
        for (int nb = 0; nb < NB; ++nb)
            *reinterpret_cast<float4*>(rbuf + ((size_t)(warp * 32 + lane) * NB + nb) * 4) =
                make_float4(acc[nb][0], acc[nb][1], acc[nb][2], acc[nb][3]);
        __syncthreads();
        if (tid < 128 * NB) {
            const int nb = tid >> 7, l = (tid & 127) >> 2, reg = tid & 3;
            float sum = 0.f;
            for (int w = 0; w < act; ++w) sum += rbuf[((size_t)(w * 32 + l) * NB + nb) * 4 + reg];
            const int row = ctx.tile * 16 + (l >> 2) + ((reg >> 1) << 3);
            const int col = nb * 8 + ((l & 3) << 1) + (reg & 1);
            if (row < P.N && col < M) {
                if (P.partial != nullptr) {
                    P.partial[((int64_t)ctx.chunk * M + col) * P.N + row] = sum;
                } else {
                    if (P.bias != nullptr) sum += load_act<kBf16>(P.bias, row);
                    store_any(P.y, y_dtype, (int64_t)col * P.N + row, sum);
                }
            }
        }
        buf ^= 1;
        ctx = nctx;
        active = nactive;
        ra = na;
        rb = nbq;
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
    const size_t smem = kLutBytes + (size_t)2 * kGemvWarps * 32 * 4 * NB * sizeof(float);
    if (!configured) {
        if (cudaFuncSetAttribute(gemv_mma_kernel<kBf16, NB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return OJX_ERR_LAUNCH;
        configured = true;
    }
    const int sms = num_sms();
    const int per = (total + sms - 1) / sms;
    const int grid = (total + per - 1) / per;
    gemv_mma_kernel<kBf16, NB><<<grid, kGemvThreads, smem, s>>>(probs, single, count, total, M, y_dtype);
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
