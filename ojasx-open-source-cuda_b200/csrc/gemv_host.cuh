// Host-side routing of the decode-shape entry points to the kernels in gemv.cuh and gemv_a16.cuh.
#pragma once

#include <atomic>
#include <mutex>
#include <utility>

#include "gemv.cuh"
#include "gemv_a16.cuh"
#include "gemv_lowbit.cuh"
#include "gemv_b2.cuh"
#include "gemv_b1.cuh"

namespace ojx {

inline bool gemv_fast_ok(int64_t M, int64_t N, int64_t K, int group, int x_dtype) {
    return M >= 1 && M <= 16 && K % 256 == 0 && group == 32 && (x_dtype == OJX_BF16 || x_dtype == OJX_F16) &&
           N >= 1 && N < (1 << 30) && K < (1 << 30);
}

int32_t gemv_tiles_impl(int64_t N, int64_t K) {
    if (N <= 0 || K <= 0 || K % 256 != 0 || N >= (1 << 30) || K >= (1 << 30)) return 0;
    return gemv_row_tiles32((int)N) * gemv_kchunks((int)K);
}
int32_t gemv_kchunks_impl(int64_t K) { return (K > 0 && K % 256 == 0 && K < (1 << 30)) ? gemv_kchunks((int)K) : 0; }

// Scratch of the single-problem entry point: fp32 partials [kchunks][M][N], needed only when K
// spans more than one chunk of the CTA's 16 slices.
size_t gemv_workspace_bytes_impl(int64_t M, int64_t N, int64_t K) {
    if (M <= 0 || M > 16 || N <= 0 || K <= 0 || K % 256 != 0 || N >= (1 << 30) || K >= (1 << 30)) return 0;
    const int kc = gemv_kchunks((int)K);
    return kc > 1 ? (size_t)kc * M * N * sizeof(float) : 0;
}

// Opting in to more than 48 KB of dynamic shared memory is a per-device (per-context) attribute of a kernel:
// `done` keeps one bit per device ordinal.
template <typename Kernel>
static int32_t ensure_dynamic_smem(Kernel kernel, size_t bytes, std::atomic<uint64_t>& done) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return OJX_ERR_LAUNCH;
    const uint64_t bit = 1ull << dev;
    if (done.load(std::memory_order_acquire) & bit) return OJX_OK;
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) { last_cuda_error() = e; return OJX_ERR_LAUNCH; }
    done.fetch_or(bit, std::memory_order_release);
    return OJX_OK;
}

// Launch with the "programmatic stream serialization" attribute when `overlap` is set: the kernel may then start
// (and run up to its griddepcontrol.wait) while the previous kernel of the stream is still draining.
template <typename... Params, typename... Args>
static int32_t launch_maybe_overlapped(void (*kernel)(Params...), int grid, int block, size_t smem, cudaStream_t s, bool overlap,
                                       Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3((unsigned)block);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = overlap ? 1 : 0;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
    if (e != cudaSuccess) { last_cuda_error() = e; (void)cudaGetLastError(); return OJX_ERR_LAUNCH; }
    return OJX_OK;
}

template <int NB, bool kXF16, bool kI8 = false>
static int32_t launch_gemv_a16(const ojx_e8t_gemv_problem* probs, const ojx_e8t_gemv_problem& single, int count, int total,
                               int M, int y_dtype, const PeerMap& peers_in, int overlap, cudaStream_t s) {
    PeerMap peers = peers_in;
    peers.host_status = host_status_device_ptr();
    peers.wait_limit = wait_limit_override() != 0 ? wait_limit_override() : kSpinLimit;
    static std::atomic<uint64_t> configured{0};
    using Cfg = A16Cfg<NB>;
    const int32_t st = ensure_dynamic_smem(gemv_a16_kernel<NB, kXF16, kI8>, Cfg::kSmem, configured);
    OJX_RETURN_IF(st != OJX_OK, st);
    const int sms = num_sms();
    const int per = (total + sms - 1) / sms;
    const int grid = (total + per - 1) / per;
    return launch_maybe_overlapped(gemv_a16_kernel<NB, kXF16, kI8>, grid, kGemvThreads, Cfg::kSmem, s, overlap != 0,
                                   probs, single, count, total, M, y_dtype, overlap, peers);
}

// One bf16 activation row takes the int8 path; one to eight rows take one block of eight columns per fp16 MMA, nine to
// sixteen take two.
static int32_t dispatch_gemv(bool bf16, const ojx_e8t_gemv_problem* probs, const ojx_e8t_gemv_problem& single, int count,
                             int total, int M, int y_dtype, const PeerMap& peers, int overlap, cudaStream_t s) {
    if (bf16 && M == 1) return launch_gemv_a16<1, false, true>(probs, single, count, total, M, y_dtype, peers, overlap, s);
    if (bf16) return M <= 8 ? launch_gemv_a16<1, false>(probs, single, count, total, M, y_dtype, peers, overlap, s)
                            : launch_gemv_a16<2, false>(probs, single, count, total, M, y_dtype, peers, overlap, s);
    return M <= 8 ? launch_gemv_a16<1, true>(probs, single, count, total, M, y_dtype, peers, overlap, s)
                  : launch_gemv_a16<2, true>(probs, single, count, total, M, y_dtype, peers, overlap, s);
}

int32_t gemv_grouped_impl(const ojx_e8t_gemv_problem* problems, int count, int total_tiles, int64_t M,
                          int x_dtype, int y_dtype, int needs_reduce, const int64_t* peer_delta, int world,
                          ojx_e8t_peer_sync* peer_sync, int flags, cudaStream_t s) {
    OJX_RETURN_IF(world < 1 || world > 8 || (world > 1 && !peer_delta), OJX_ERR_SHAPE);
    PeerMap peers = peer_map_self();
    if (peer_delta != nullptr) {
        peers.world = world;
        for (int r = 0; r < world; ++r) peers.delta[r] = peer_delta[r];
    }
    OJX_RETURN_IF(!problems, OJX_ERR_NULL);
    OJX_RETURN_IF(count <= 0 || total_tiles <= 0 || M < 1 || M > 16, OJX_ERR_SHAPE);
    OJX_RETURN_IF(x_dtype != OJX_BF16 && x_dtype != OJX_F16, OJX_ERR_DTYPE);
    OJX_RETURN_IF(y_dtype != OJX_BF16 && y_dtype != OJX_F16 && y_dtype != OJX_F32, OJX_ERR_DTYPE);
    OJX_RETURN_IF(check_arch() != OJX_OK, OJX_ERR_ARCH);
    const bool bf = x_dtype == OJX_BF16;
    ojx_e8t_gemv_problem none = {};
    constexpr int kKnown = OJX_GEMV_STATIC_WEIGHTS | OJX_GEMV_SIGNAL_PEERS | OJX_GEMV_WAIT_PEERS | OJX_GEMV_TEST_LOSE_COPY |
                           OJX_GEMV_INDEPENDENT;
    OJX_RETURN_IF((flags & ~kKnown) != 0, OJX_ERR_UNSUPPORTED);
    OJX_RETURN_IF((flags & OJX_GEMV_INDEPENDENT) != 0 && (flags & (OJX_GEMV_SIGNAL_PEERS | OJX_GEMV_WAIT_PEERS)) != 0, OJX_ERR_UNSUPPORTED);
    const int sync_mode = flags & (OJX_GEMV_SIGNAL_PEERS | OJX_GEMV_WAIT_PEERS);
    OJX_RETURN_IF(sync_mode != 0 && peer_sync == nullptr, OJX_ERR_NULL);
    OJX_RETURN_IF((reinterpret_cast<uintptr_t>(peer_sync) & 3) != 0, OJX_ERR_ALIGN);
    if (peer_sync != nullptr) {
        peers.sync = peer_sync;
        // bit 8 tells the main kernel that a reduce kernel follows and stores (and signals) in its place
        peers.mode = sync_mode | (needs_reduce ? 0x100 : 0);
    }
    peers.lose_copy = (flags & OJX_GEMV_TEST_LOSE_COPY) ? 1 : 0;
    // 0: ordered like any kernel; 1: starts early, waits for its predecessor before touching x and y; 2: never waits
    const int overlap = (flags & OJX_GEMV_INDEPENDENT) ? 2 : ((flags & OJX_GEMV_STATIC_WEIGHTS) ? 1 : 0);
    const int32_t st = dispatch_gemv(bf, problems, none, count, total_tiles, (int)M, y_dtype, peers, overlap, s);
    OJX_RETURN_IF(st != OJX_OK, st);
    if (!needs_reduce) return OJX_OK;
    // Problems whose K spans several chunks carry a partial buffer; the reduce pass skips the rest.
    dim3 grid(64, count > 64 ? 64 : count);
    if (bf) gemv_reduce_kernel<true><<<grid, 256, 0, s>>>(problems, none, count, (int)M, y_dtype, peers);
    else gemv_reduce_kernel<false><<<grid, 256, 0, s>>>(problems, none, count, (int)M, y_dtype, peers);
    return launch_status();
}

__global__ void peer_wait_kernel(const __grid_constant__ PeerMap peers) {
    if (threadIdx.x == 0) peer_wait(peers);
}

// Orders everything that follows in `s` after the launch that every rank signalled last (bounded, see peer_wait).
int32_t peer_wait_impl(ojx_e8t_peer_sync* peer_sync, int world, cudaStream_t s) {
    OJX_RETURN_IF(!peer_sync, OJX_ERR_NULL);
    OJX_RETURN_IF(world < 1 || world > 8, OJX_ERR_SHAPE);
    OJX_RETURN_IF(check_arch() != OJX_OK, OJX_ERR_ARCH);
    PeerMap peers = peer_map_self();
    peers.world = world;
    peers.sync = peer_sync;
    peers.mode = OJX_GEMV_WAIT_PEERS;
    peers.host_status = host_status_device_ptr();
    peer_wait_kernel<<<1, 32, 0, s>>>(peers);
    return launch_status();
}

int32_t gemv_impl(const void* x, int x_dtype, int64_t M, const uint8_t* packed, const uint16_t* scales,
                  const void* bias, int64_t N, int64_t K, int group, void* y, int y_dtype,
                  void* workspace, size_t workspace_bytes, cudaStream_t s,
                  const float* lora_t, const void* lora_b, int lora_rank) {
    OJX_RETURN_IF(!x || !packed || !scales || !y, OJX_ERR_NULL);
    OJX_RETURN_IF(lora_rank < 0 || lora_rank > 64 || (lora_rank > 0 && (!lora_t || !lora_b)), OJX_ERR_SHAPE);
    OJX_RETURN_IF(lora_rank > 0 && M > 8, OJX_ERR_UNSUPPORTED);        // the 9-16 row kernels have no registers to spare for it
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
        h.N = (int)N; h.K = (int)K; h.tile_begin = 0; h.ldy = 0;
        h.lora_t = lora_t; h.lora_b = lora_b; h.lora_rank = lora_rank; h.reserved = 0;
        const int total = gemv_row_tiles32((int)N) * kc;
        const bool bf = x_dtype == OJX_BF16;
        const int32_t st = dispatch_gemv(bf, nullptr, h, 1, total, (int)M, y_dtype, peer_map_self(), false, s);
        OJX_RETURN_IF(st != OJX_OK, st);
        if (kc > 1) {
            dim3 grid(64, 1);
            if (bf) gemv_reduce_kernel<true><<<grid, 256, 0, s>>>(nullptr, h, 1, (int)M, y_dtype, peer_map_self());
            else gemv_reduce_kernel<false><<<grid, 256, 0, s>>>(nullptr, h, 1, (int)M, y_dtype, peer_map_self());
        }
        return launch_status();
    }
    OJX_RETURN_IF(lora_rank > 0, OJX_ERR_UNSUPPORTED);          // the low-rank epilogue exists in the tensor-core kernels only
    // up to eight rows, any power-of-two group from 16 and any activation dtype: the shared-memory fp32 kernel
    {
        int shift = -1;
        for (int b = 4; b < 20; ++b)
            if ((1 << b) == group) shift = b;
        const size_t smem = ternary_small_smem_bytes(M, K);
        if (shift > 0 && M <= 8 && K % 64 == 0 && K <= (1 << 24) && N < (1 << 30) && smem <= 200 * 1024 &&
            (reinterpret_cast<uintptr_t>(packed) & 3) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
            const int per_sm = (int)((220 * 1024) / (smem + 1024)) < 1 ? 1 : (int)((220 * 1024) / (smem + 1024));
            int64_t blocks = (N + 31) / 32;                       // at least four weight rows per warp: every CTA stages x once
            const int64_t cap = (int64_t)num_sms() * (per_sm > 8 ? 8 : per_sm);
            if (blocks > cap) blocks = cap;
            auto run = [&](auto kernel, std::atomic<uint64_t>& done) -> int32_t {
                const int32_t sc = ensure_dynamic_smem(kernel, 200 * 1024, done);
                OJX_RETURN_IF(sc != OJX_OK, sc);
                kernel<<<(unsigned)blocks, 256, smem, s>>>(x, x_dtype, (int)M, packed, scales, bias, (int)N, (int)K, shift, y, y_dtype);
                return launch_status();
            };
            static std::atomic<uint64_t> done1{0}, done4{0}, done8{0};
            if (M == 1) return run(ternary_small_gemv_kernel<1>, done1);
            if (M <= 4) return run(ternary_small_gemv_kernel<4>, done4);
            return run(ternary_small_gemv_kernel<8>, done8);
        }
    }
    // generic path
    int64_t warps_needed = N;
    int64_t blocks = (warps_needed * 32 + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    generic_linear_kernel<0><<<(unsigned)blocks, 256, 0, s>>>(x, x_dtype, M, packed, scales, bias, N, K, group, y, y_dtype);
    return launch_status();
}

// Routes a low-bit decode-shape linear to lowbit_gemv_kernel when its shared-memory image of x fits; returns false when
// the caller has to use the generic kernel.
template <int kFmt>
static bool launch_lowbit_gemv(const void* x, int x_dtype, int64_t M, const uint8_t* packed, const uint16_t* scales,
                               const void* bias, int64_t N, int64_t K, int group, void* y, int y_dtype, cudaStream_t s,
                               int32_t* status) {
    const size_t smem = lowbit_smem_bytes(M, K, kFmt);
    if (M < 1 || M > 8 || K % 16 != 0 || K > (1 << 24) || N >= (1 << 30) || smem > 200 * 1024 ||
        (reinterpret_cast<uintptr_t>(packed) & 3) != 0 || (reinterpret_cast<uintptr_t>(x) & 15) != 0)
        return false;
    const int sms = num_sms();
    const int per_sm = (int)((220 * 1024) / (smem + 1024)) < 1 ? 1 : (int)((220 * 1024) / (smem + 1024));
    int64_t blocks = (N + 31) / 32;                           // at least four weight rows per warp: every CTA stages x once
    const int64_t cap = (int64_t)sms * (per_sm > 8 ? 8 : per_sm);
    if (blocks > cap) blocks = cap;
    int shift = -1;
    for (int b = 3; b < 20; ++b)
        if ((1 << b) == group) shift = b;
    auto run = [&](auto kernel, std::atomic<uint64_t>& done) {
        *status = ensure_dynamic_smem(kernel, 200 * 1024, done);
        if (*status != OJX_OK) return;
        kernel<<<(unsigned)blocks, 256, smem, s>>>(x, x_dtype, (int)M, packed, scales, bias, (int)N, (int)K, group, shift, y, y_dtype);
        *status = launch_status();
    };
    static std::atomic<uint64_t> done1{0}, done4{0}, done8{0};
    if (M == 1) run(lowbit_gemv_kernel<kFmt, 1>, done1);
    else if (M <= 4) run(lowbit_gemv_kernel<kFmt, 4>, done4);
    else run(lowbit_gemv_kernel<kFmt, 8>, done8);
    return true;
}

// y = x . W^T (+ bias) for the 2.0-bit (bits == 2) and 1.0-bit (bits == 1) formats: the fused fp32 kernel (one warp per
// output feature), any shape.
int32_t linear_lowbit_impl(int bits, const void* x, int x_dtype, int64_t M, const uint8_t* packed, const uint16_t* scales,
                           const void* bias, int64_t N, int64_t K, int group, void* y, int y_dtype, cudaStream_t s,
                           const float* lora_t, const void* lora_b, int lora_rank) {
    OJX_RETURN_IF(!x || !packed || !scales || !y, OJX_ERR_NULL);
    OJX_RETURN_IF(lora_rank < 0 || lora_rank > 64 || (lora_rank > 0 && (!lora_t || !lora_b)), OJX_ERR_SHAPE);
    OJX_RETURN_IF(M <= 0 || N <= 0 || K <= 0 || group <= 0 || group % 8 != 0, OJX_ERR_SHAPE);
    OJX_RETURN_IF(dtype_size(x_dtype) == 0 || dtype_size(y_dtype) == 0, OJX_ERR_DTYPE);
    OJX_RETURN_IF(check_arch() != OJX_OK, OJX_ERR_ARCH);
    // up to eight rows of the 2.0-bit format with groups of 32 and K a multiple of 2048: int8 tensor cores, no table
    if (bits == 2 && M >= 1 && M <= 8 && group == 32 && K % 2048 == 0 && K <= (1 << 20) && N < (1 << 30) &&
        b2_smem_bytes((int)M, 2, (int)K) <= 227 * 1024 &&
        ((reinterpret_cast<uintptr_t>(packed) | reinterpret_cast<uintptr_t>(x)) & 15) == 0 &&
        (reinterpret_cast<uintptr_t>(scales) & 3) == 0) {
        // one CTA per SM, two groups of eight warps (three and four groups were measured: coarser tile sets and fewer
        // registers per thread cost more than the extra warps hide)
        const int groups = 2;
        const size_t smem = b2_smem_bytes((int)M, groups, (int)K);
        const int tile_sets = (int)((N + 16 * groups - 1) / (16 * groups));
        const int grid = tile_sets < num_sms() ? tile_sets : num_sms();
        auto run = [&](auto kernel, std::atomic<uint64_t>& done) -> int32_t {
            const int32_t sc = ensure_dynamic_smem(kernel, 227 * 1024, done);
            OJX_RETURN_IF(sc != OJX_OK, sc);
            kernel<<<grid, groups * kB2Warps * 32, smem, s>>>(x, x_dtype, (int)M, packed, scales, bias, (int)N, (int)K, y, y_dtype,
                                                              lora_t, lora_b, lora_rank);
            return launch_status();
        };
        static std::atomic<uint64_t> d1{0}, d2{0}, d4{0}, d8{0}, l1{0}, l2{0}, l4{0}, l8{0};
        if (lora_rank > 0) {                                  // the variants that carry the adapter term are kept apart
            if (M == 1) return run(gemv_b2_kernel<1, 2, true>, l1);
            if (M == 2) return run(gemv_b2_kernel<2, 2, true>, l2);
            if (M <= 4) return run(gemv_b2_kernel<4, 2, true>, l4);
            return run(gemv_b2_kernel<8, 2, true>, l8);
        }
        if (M == 1) return run(gemv_b2_kernel<1, 2>, d1);
        if (M == 2) return run(gemv_b2_kernel<2, 2>, d2);
        if (M <= 4) return run(gemv_b2_kernel<4, 2>, d4);
        return run(gemv_b2_kernel<8, 2>, d8);
    }
    // the same shapes of the 1.0-bit format: int8 tensor cores, one table read per code byte
    if (bits == 1 && M >= 1 && M <= 8 && group == 32 && K % 2048 == 0 && K <= (1 << 20) && N < (1 << 30) &&
        b1_smem_bytes(M <= 2 ? 1 : (M <= 4 ? 2 : 4), 8, 2, (int)K) <= 227 * 1024 &&
        ((reinterpret_cast<uintptr_t>(packed) | reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(scales)) & 15) == 0) {
        const int cbs = M <= 2 ? 1 : (M <= 4 ? 2 : 4);
        const int groups = 2;                                                // one CTA per SM, two groups of eight warps
        const bool narrow = b1_smem_bytes(cbs, 16, groups, (int)K) > 227 * 1024;      // sixteen copies of the table, eight where sixteen do not fit
        const size_t smem = b1_smem_bytes(cbs, narrow ? 8 : 16, groups, (int)K);
        const int tile_sets = (int)((N + 16 * groups - 1) / (16 * groups));
        const int grid = tile_sets < num_sms() ? tile_sets : num_sms();
        auto run = [&](auto kernel, std::atomic<uint64_t>& done) -> int32_t {
            const int32_t sc = ensure_dynamic_smem(kernel, 227 * 1024, done);
            OJX_RETURN_IF(sc != OJX_OK, sc);
            kernel<<<grid, groups * kB1Warps * 32, smem, s>>>(x, x_dtype, (int)M, packed, scales, bias, (int)N, (int)K, y, y_dtype,
                                                              lora_t, lora_b, lora_rank);
            return launch_status();
        };
        static std::atomic<uint64_t> d1{0}, d2{0}, d4{0}, d1n{0}, d2n{0}, d4n{0};
        if (cbs == 1) return narrow ? run(gemv_b1_kernel<1, 8, 2>, d1n) : run(gemv_b1_kernel<1, 16, 2>, d1);
        if (cbs == 2) return narrow ? run(gemv_b1_kernel<2, 8, 2>, d2n) : run(gemv_b1_kernel<2, 16, 2>, d2);
        return narrow ? run(gemv_b1_kernel<4, 8, 2>, d4n) : run(gemv_b1_kernel<4, 16, 2>, d4);
    }
    OJX_RETURN_IF(lora_rank > 0, OJX_ERR_UNSUPPORTED);          // the adapter epilogue exists in the tensor-core kernels only
    int32_t st = OJX_OK;                                      // small batches: the shared-memory kernel when x fits
    if (bits == 2 ? launch_lowbit_gemv<2>(x, x_dtype, M, packed, scales, bias, N, K, group, y, y_dtype, s, &st)
                  : launch_lowbit_gemv<1>(x, x_dtype, M, packed, scales, bias, N, K, group, y, y_dtype, s, &st))
        return st;
    int64_t blocks = (N * 32 + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    if (bits == 2) generic_linear_kernel<2><<<(unsigned)blocks, 256, 0, s>>>(x, x_dtype, M, packed, scales, bias, N, K, group, y, y_dtype);
    else generic_linear_kernel<1><<<(unsigned)blocks, 256, 0, s>>>(x, x_dtype, M, packed, scales, bias, N, K, group, y, y_dtype);
    return launch_status();
}


// ---------------------------------------------------------------------------------------------
// Decode-shape linear that brings its own scratch.
//
// Some hosts hand a plug-in nothing but its input and output buffers: an inference server whose
// device memory is carved up front by its own arena, a callback running where cudaMalloc is
// forbidden (it synchronises the whole device), a sandboxed worker without allocation rights.
// For them the fp32 partial sums that K > 4096 needs live in this file-scope device array instead
// of a caller buffer.  Every GPU that loads the library carries the array until the process ends.
// ---------------------------------------------------------------------------------------------
constexpr size_t kStaticScratchFloats = (size_t)1 << 20;                     // 4 MiB per GPU
static __device__ __align__(256) float g_static_scratch[kStaticScratchFloats];

// In host code the array's name is only a handle; the device address is asked for once per device,
// with that device current, and cached.
static float* static_scratch_ptr(int32_t* status) {
    static float* cached[64] = {nullptr};
    static std::mutex mtx;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { *status = OJX_ERR_LAUNCH; return nullptr; }
    std::lock_guard<std::mutex> lock(mtx);
    if (cached[dev] == nullptr) {
        float* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_static_scratch);
        if (e != cudaSuccess || p == nullptr) { last_cuda_error() = e; *status = OJX_ERR_LAUNCH; return nullptr; }
        cached[dev] = p;
    }
    *status = OJX_OK;
    return cached[dev];
}

size_t gemv_static_scratch_capacity_impl() { return kStaticScratchFloats * sizeof(float); }

int32_t gemv_static_scratch_impl(const void* x, int x_dtype, int64_t M, const uint8_t* packed, const uint16_t* scales,
                                 const void* bias, int64_t N, int64_t K, int group, void* y, int y_dtype, cudaStream_t s) {
    OJX_RETURN_IF(!x || !packed || !scales || !y, OJX_ERR_NULL);
    OJX_RETURN_IF(M <= 0 || N <= 0 || K <= 0, OJX_ERR_SHAPE);
    // scratch is only needed on the tensor-core route (same test as in gemv_impl); the plain kernel uses none
    const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(packed) |
                           reinterpret_cast<uintptr_t>(scales)) & 15) == 0;
    const size_t need = (gemv_fast_ok(M, N, K, effective_group(group), x_dtype) && aligned) ? gemv_workspace_bytes_impl(M, N, K) : 0;
    // larger problems do not fit the built-in array: the caller has to use ojx_e8t_gemv with its own scratch
    OJX_RETURN_IF(need > kStaticScratchFloats * sizeof(float), OJX_ERR_WORKSPACE);
    float* scratch = nullptr;
    if (need > 0) {
        int32_t st = OJX_OK;
        scratch = static_scratch_ptr(&st);
        OJX_RETURN_IF(st != OJX_OK, st);
    }
    // Every partial sum is written by exactly one work item before the reduce pass reads it, so the
    // array's previous contents never matter and nothing has to be cleared.
    return gemv_impl(x, x_dtype, M, packed, scales, bias, N, K, group, y, y_dtype, scratch, need, s);
}

}  // namespace ojx
