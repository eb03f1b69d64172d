// Shared device/host helpers for the ternary-E8 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/ojx_e8t.h"

namespace ojx {

constexpr int kNumPoints = 3281;

// Device copies of the generated tables.  The whole library is one translation unit
// (ojx_e8t.cu includes every kernel file), so file-scope statics are shared by all kernels.
//   g_trit_nibbles[rank]  eight 4-bit fields, field i = coordinate i as {0: 0, 1: +1, 2: -1}
#define OJX_TABLE_QUAL static __device__ __align__(16)
#define OJX_TABLE_NAME(x) g_##x
#include "e8t_tables.inc"
#undef OJX_TABLE_QUAL
#undef OJX_TABLE_NAME

__host__ __device__ inline int effective_group(int group) {
    // The reference replaces anything that is not a positive multiple of 16 by 16
    // (ojasx2/math/lattice.py:346-347).
    return (group <= 0 || group % 16 != 0) ? 16 : group;
}

inline int dtype_size(int dt) {
    switch (dt) {
        case OJX_F32: return 4;
        case OJX_F16: return 2;
        case OJX_BF16: return 2;
        default: return 0;
    }
}

// Byte permute: byte i of the result is byte sel[4i+3:4i] of the eight bytes {b, a}.
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Two 12-bit ranks from one 3-byte triplet (ojasx2/math/lattice.py:397-405).
__device__ __forceinline__ void triplet_to_codes(uint32_t b0, uint32_t b1, uint32_t b2, uint32_t& c0, uint32_t& c1) {
    c0 = b0 | ((b1 & 0x0Fu) << 8);
    c1 = ((b1 >> 4) & 0x0Fu) | (b2 << 4);
}

// Coordinate i (-1, 0, +1) of a nibble-encoded trit vector.
__device__ __forceinline__ int nibble_coord(uint32_t nib, int i) {
    uint32_t f = (nib >> (4 * i)) & 0xFu;
    return f == 0 ? 0 : (f == 1 ? 1 : -1);
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier helpers (shared by the GEMV ring and the tcgen05 pipeline) -------------------------
constexpr uint32_t kSpinLimit = 1u << 24;                     // bounded waits: ~seconds, then give up
__device__ __forceinline__ void mbar_init(uint32_t addr, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(addr), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t addr) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(addr) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t addr, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(addr), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t addr, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false (and raises the CTA-wide abort flag) when the limit is reached or
// another thread already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t addr, uint32_t parity, volatile int* abort_flag, int code,
                                          uint32_t limit = kSpinLimit) {
    for (uint32_t i = 0; i < limit; ++i) {
        if (mbar_try_wait(addr, parity)) return true;
        if ((i & 1023u) == 1023u && *abort_flag != 0) return false;
    }
    atomicCAS(const_cast<int*>(abort_flag), 0, code);
    return false;
}

// 1-D bulk copy global -> shared, completion counted in bytes on an mbarrier.  Both addresses and
// the size must be multiples of 16 bytes.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// Device-side status word: a bounded wait that gave up records its code here (0 = none).
static __device__ int g_device_status = 0;

// The same event for the host, without a synchronisation: one page of host memory that is part of the
// library image, pinned and mapped on first use, into which a kernel that gave up on a wait writes its code.
// Kernels receive its device address as an argument (null when the mapping failed: then only
// g_device_status is written).
int* host_status_device_ptr();
int  host_status_take();                       // returns the recorded code (0: none) and clears it
uint32_t& wait_limit_override();               // 0: the built-in limit; set by ojx_e8t_set_wait_limit (tests)

// Validates the device once per process per device: kernels are built for sm_100a only.
int check_arch();

#define OJX_RETURN_IF(cond, code) do { if (cond) return (code); } while (0)

// Last CUDA runtime error seen by this library on the calling thread (for diagnostics only).
inline cudaError_t& last_cuda_error() {
    static thread_local cudaError_t e = cudaSuccess;
    return e;
}
inline int32_t launch_status() {
    const cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) return OJX_OK;
    last_cuda_error() = e;
    return OJX_ERR_LAUNCH;
}

// Entry points implemented in the individual .cu files (called by api.cu).
int32_t encode_impl(const void* w, int w_dtype, int64_t rows, int64_t cols, int group, uint32_t flags,
                    uint8_t* packed, uint16_t* scales, cudaStream_t s);
int32_t decode_impl(const uint8_t* packed, const uint16_t* scales, int64_t rows, int64_t cols,
                    int group, int out_dtype, void* out, cudaStream_t s);
int32_t generate_impl(void* out, int dtype, int64_t count, uint64_t seed, int64_t start, float sigma,
                      cudaStream_t s);
size_t  gemv_workspace_bytes_impl(int64_t M, int64_t N, int64_t K);
int32_t gemv_impl(const void* x, int x_dtype, int64_t M, const uint8_t* packed, const uint16_t* scales,
                  const void* bias, int64_t N, int64_t K, int group, void* y, int y_dtype,
                  void* workspace, size_t workspace_bytes, cudaStream_t s,
                  const float* lora_t = nullptr, const void* lora_b = nullptr, int lora_rank = 0);
size_t  gemv_static_scratch_capacity_impl();
int32_t gemv_static_scratch_impl(const void* x, int x_dtype, int64_t M, const uint8_t* packed, const uint16_t* scales,
                                 const void* bias, int64_t N, int64_t K, int group, void* y, int y_dtype, cudaStream_t s);
int32_t gemv_tiles_impl(int64_t N, int64_t K);
int32_t gemv_kchunks_impl(int64_t K);
int32_t gemv_grouped_impl(const ojx_e8t_gemv_problem* problems, int count, int total_tiles, int64_t M,
                          int x_dtype, int y_dtype, int needs_reduce, const int64_t* peer_delta, int world,
                          ojx_e8t_peer_sync* peer_sync, int flags, cudaStream_t s);
int32_t peer_wait_impl(ojx_e8t_peer_sync* peer_sync, int world, cudaStream_t s);
size_t  gemm_workspace_bytes_impl(int64_t M, int64_t N, int64_t K);
int32_t gemm_impl(const void* x, int x_dtype, int64_t M, const uint8_t* packed, const uint16_t* scales,
                  const void* bias, int64_t N, int64_t K, int group, void* y, int y_dtype,
                  void* workspace, size_t workspace_bytes, cudaStream_t s);
int32_t gemm_status_impl(const void* workspace, cudaStream_t s);
size_t  gemm_dx_workspace_bytes_impl(int64_t M, int64_t N, int64_t K);
int32_t gemm_dx_impl(const void* gy, int gy_dtype, int64_t M, const uint8_t* packed, const uint16_t* scales,
                     int64_t N, int64_t K, int group, void* dx, int dx_dtype,
                     void* workspace, size_t workspace_bytes, cudaStream_t s);

}  // namespace ojx
