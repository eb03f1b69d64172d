// Shared pieces of the decode-shape fused linear  y[M,N] = x[M,K] . dequant(W)[N,K]^T  for small M:
// work-item geometry, shared-memory and cp.async helpers, the output-window map for column-sharded
// launches, the partial-sum reduce kernel for K larger than one chunk, and the generic correctness kernel
// for shapes and dtypes the tensor-core kernel (gemv_a16.cuh) does not cover.
//
// Replaces, for small batches, _FusedE8GEMMFunction.forward (ojasx2/math/lattice.py:551-640)
// and the reference's scalar fused kernel (ojasx2/math/csrc/ojasx_math_core.hpp:580-634):
// per (m, n) the result is sum over groups of (sum_k x*coord) * scale, accumulated in fp32.
#pragma once

#include "common.cuh"

namespace ojx {

constexpr int kGemvWarps = 16;
constexpr int kGemvThreads = kGemvWarps * 32;

__host__ __device__ inline int gemv_active_warps(int K) {
    const int slices = K / 256;
    for (int w = kGemvWarps; w > 1; --w)
        if (slices % w == 0) return w;
    return 1;
}
__host__ __device__ inline int gemv_kchunks(int K) { return (K / 256) / gemv_active_warps(K); }
// The public tile unit (ojx_e8t_gemv_tiles) is 32 weight rows x one K chunk.
__host__ __device__ inline int gemv_row_tiles32(int N) { return (N + 31) / 32; }

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
    int mode;                      // OJX_GEMV_SIGNAL_PEERS | OJX_GEMV_WAIT_PEERS, only with a sync block
    ojx_e8t_peer_sync* sync;       // this rank's block inside the window (peers' blocks at + delta[r]), or null
    // not about peers, but travelling in the same kernel argument:
    int* host_status;              // mapped host word that receives the code of a wait that gave up (may be null)
    uint32_t wait_limit;           // polls before a wait on a copy gives up
    int lose_copy;                 // tests: never report the first item's copies complete
};
inline PeerMap peer_map_self() { PeerMap m = {}; m.world = 1; m.wait_limit = kSpinLimit; return m; }
// The copies for the other ranks (delta != 0), kept out of line: rare, and the callers run at the register cap.
__device__ __noinline__ void store_peers(const PeerMap& pm, void* y, int y_dtype, int64_t idx, float v) {
    for (int r = 0; r < pm.world; ++r)
        if (pm.delta[r] != 0) store_any(static_cast<uint8_t*>(y) + pm.delta[r], y_dtype, idx, v);
}

// ---- device-side ordering between the ranks of a column-sharded chain (see ojx_e8t_gemv_grouped_ex) ----
constexpr int kPeerSpinDefault = 1 << 21;                      // polls of a system-scope load: about a second

__device__ __forceinline__ int ld_acquire_sys(const int* p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(int* p, int v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Called by ONE thread of every CTA after the CTA's last result store (and a __syncthreads): the CTA that
// arrives last publishes this rank's next epoch into every rank's block.
__device__ __noinline__ void peer_signal(const PeerMap& pm) {
    __threadfence_system();                                    // the CTA's stores, local and remote, before the count
    ojx_e8t_peer_sync* sy = pm.sync;
    if (atomicAdd(&sy->arrived, 1) != (int)gridDim.x * (int)gridDim.y - 1) return;
    __threadfence_system();                                    // every CTA's stores before the flags
    sy->arrived = 0;
    const int e = sy->epoch + 1;
    int self = 0;
    for (int r = 0; r < pm.world; ++r)
        if (pm.delta[r] == 0) self = r;
    for (int r = 0; r < pm.world; ++r) {
        ojx_e8t_peer_sync* dst = reinterpret_cast<ojx_e8t_peer_sync*>(reinterpret_cast<uint8_t*>(sy) + pm.delta[r]);
        st_release_sys(&dst->flag[self], e);
    }
    st_release_sys(&sy->epoch, e);
}

// Called by ONE thread of every CTA before the CTA's first read of x (followed by a __syncthreads).  Returns false
// when a wait ran out; the failure is recorded and the kernel carries on.
__device__ __noinline__ bool peer_wait(const PeerMap& pm) {
    ojx_e8t_peer_sync* sy = pm.sync;
    const int e = ld_acquire_sys(&sy->epoch);
    const int limit = sy->spin_limit > 0 ? sy->spin_limit : kPeerSpinDefault;
    bool ok = true;
    for (int q = 0; q < pm.world && ok; ++q) {
        int i = 0;
        while (ld_acquire_sys(&sy->flag[q]) - e < 0) {
            if (++i >= limit) { ok = false; break; }
            __nanosleep(64);
        }
    }
    if (!ok) {
        atomicCAS(&sy->status, 0, (int)OJX_ERR_TIMEOUT);
        atomicCAS(&g_device_status, 0, 60);
        if (pm.host_status != nullptr) *reinterpret_cast<volatile int*>(pm.host_status) = 60;
    }
    return ok;
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

// 16-byte asynchronous copy global -> shared (L2 only, no L1 allocation) and the mbarrier arrive that
// fires when all of this thread's earlier copies have landed.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_arrive(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}

// Geometry of a work item in shared memory: 32 rows of codes, then 32 rows of scales; a row holds one
// 48-byte (codes) / 16-byte (scales) piece per 256-wide slice of the K chunk and ends in 16 bytes of padding,
// so that the eight rows one shared-memory load touches fall on distinct banks.
constexpr int kGemvMaxCodePitch = kGemvWarps * 48 + 16;     // 784
constexpr int kGemvMaxScalePitch = kGemvWarps * 16 + 16;    // 272

__device__ __forceinline__ float load_any(const void* p, int dt, int64_t i) {
    if (dt == OJX_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
    if (dt == OJX_F16) return __half2float(static_cast<const __half*>(p)[i]);
    return static_cast<const float*>(p)[i];
}

// The optional low-rank term of a problem for output (activation row col, weight row row).
// Kept out of line: it is rare, and inlined into the decode kernels' epilogue it costs them registers they do not have.
template <bool kBf16>
__device__ __noinline__ float lora_term(const ojx_e8t_gemv_problem& P, int64_t col, int64_t row) {
    float acc = 0.f;
    const float* t = P.lora_t + col * P.lora_rank;
    for (int r = 0; r < P.lora_rank; ++r) acc = fmaf(t[r], load_act<kBf16>(P.lora_b, (int64_t)r * P.N + row), acc);
    return acc;
}

// Sums the K-chunk partials of every problem that has them (fixed order), adds bias and the low-rank term, casts,
// stores - to this rank's buffer and to every peer's window.  16-bit outputs whose rows come in multiples of eight
// are handled eight rows (one 16-byte vector) per thread.
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
        const int64_t ld = P.ldy > 0 ? P.ldy : P.N;
        const bool vec = y_dtype != OJX_F32 && (P.N & 7) == 0 && (ld & 7) == 0 && (reinterpret_cast<uintptr_t>(P.y) & 15) == 0 &&
                         (reinterpret_cast<uintptr_t>(P.partial) & 31) == 0;
        if (vec) {
            const int64_t per_col = P.N / 8;
            for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < (int64_t)M * per_col;
                 v += (int64_t)gridDim.x * blockDim.x) {
                const int64_t col = v / per_col, row = (v - col * per_col) * 8;
                float s8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                for (int c = 0; c < kc; ++c) {
                    const float4* src = reinterpret_cast<const float4*>(P.partial + (int64_t)c * total + col * P.N + row);
                    const float4 a = __ldcg(src), b = __ldcg(src + 1);
                    s8[0] += a.x; s8[1] += a.y; s8[2] += a.z; s8[3] += a.w;
                    s8[4] += b.x; s8[5] += b.y; s8[6] += b.z; s8[7] += b.w;
                }
                uint32_t w[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float lo = s8[2 * i], hi = s8[2 * i + 1];
                    if (P.bias != nullptr) { lo += load_act<kBf16>(P.bias, row + 2 * i); hi += load_act<kBf16>(P.bias, row + 2 * i + 1); }
                    if (P.lora_rank > 0) { lo += lora_term<kBf16>(P, col, row + 2 * i); hi += lora_term<kBf16>(P, col, row + 2 * i + 1); }
                    if (y_dtype == OJX_BF16) {
                        const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
                        w[i] = *reinterpret_cast<const uint32_t*>(&h);
                    } else {
                        const __half2 h = __floats2half2_rn(lo, hi);
                        w[i] = *reinterpret_cast<const uint32_t*>(&h);
                    }
                }
                const uint4 val = make_uint4(w[0], w[1], w[2], w[3]);
                uint8_t* dst = static_cast<uint8_t*>(P.y) + (col * ld + row) * 2;
#pragma unroll 1
                for (int r = 0; r < peers.world; ++r)              // delta is 0 for this rank itself
                    *reinterpret_cast<uint4*>(dst + peers.delta[r]) = val;
            }
            continue;
        }
        for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
             i += (int64_t)gridDim.x * blockDim.x) {
            float s = 0.f;
            for (int c = 0; c < kc; ++c) s += P.partial[(int64_t)c * total + i];
            const int64_t col = i / P.N, row = i - col * P.N;
            if (P.bias != nullptr) s += load_act<kBf16>(P.bias, row);
            if (P.lora_rank > 0) s += lora_term<kBf16>(P, col, row);
            const int64_t at = col * ld + row;
            store_any(P.y, y_dtype, at, s);
#pragma unroll 1
            for (int r = 0; r < peers.world; ++r)                  // the other ranks' windows (nothing when world == 1)
                if (peers.delta[r] != 0) store_any(static_cast<uint8_t*>(P.y) + peers.delta[r], y_dtype, at, s);
        }
    }
    if (peers.sync != nullptr && (peers.mode & OJX_GEMV_SIGNAL_PEERS)) {
        __syncthreads();
        if (threadIdx.x == 0) peer_signal(peers);
    }
}

// ---------------------------------------------------------------------------------------------
// Generic path: any N, K (flat packing where groups may cross rows included), any dtypes.
// One warp per output feature; correctness path for shapes the fast kernels do not cover.
// ---------------------------------------------------------------------------------------------
// kFmt: 0 ternary (1.5 bits), 2 two-bit codes, (code - 1.5) * scale (E8LatticePacker, ojasx2/math/lattice.py:210-279),
// 1 one byte per 8-block indexing the 256-vector table (RootE8LatticePacker, ojasx2/math/lattice.py:475-537).
template <int kFmt>
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
                float w;
                if constexpr (kFmt == 2) {
                    w = ((float)((packed[flat >> 2] >> (2 * (int)(flat & 3))) & 3) - 1.5f) *
                        __half2float(__ushort_as_half(scales[flat / group]));
                } else if constexpr (kFmt == 1) {
                    const uint32_t word = g_root_coords[2 * (int)packed[flat >> 3] + (int)((flat >> 2) & 1)];
                    w = (float)(int)(int8_t)((word >> (8 * (int)(flat & 3))) & 0xFFu) *
                        __half2float(__ushort_as_half(scales[flat / group]));
                } else {
                    const int64_t code_idx = flat >> 3;
                    const uint8_t* tp = packed + (code_idx >> 1) * 3;
                    uint32_t c0, c1;
                    triplet_to_codes(tp[0], tp[1], tp[2], c0, c1);
                    uint32_t code = (code_idx & 1) ? c1 : c0;
                    code = min(code, (uint32_t)(kNumPoints - 1));
                    w = (float)nibble_coord(g_trit_nibbles[code], (int)(flat & 7)) *
                        __half2float(__ushort_as_half(scales[flat / group]));
                }
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

// Multiprocessor count of the current device (cached per device ordinal).
static int num_sms() {
    static int cached[64] = {0};
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        cached[dev] = n > 0 ? n : 148;
    }
    return cached[dev];
}

}  // namespace ojx
