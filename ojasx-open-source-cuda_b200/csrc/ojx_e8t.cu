// The whole library is this one translation unit: C ABI entry points (declared in
// include/ojx_e8t.h) in front of the kernel files included below.  Built for sm_100a only.
#include <mutex>

#include "common.cuh"
#include "codec.cuh"
#include "codec2.cuh"
#include "codec1.cuh"
#include "e8_project.cuh"
#include "gemv.cuh"
#include "gemv_a16.cuh"
#include "gemv_host.cuh"
#include "gemm_tcgen05.cuh"

namespace ojx {

int check_arch() {
    static int cached[64] = {0};          // 0 unknown, 1 ok, -1 wrong architecture
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return OJX_ERR_LAUNCH;
    if (dev < 0 || dev >= 64) return OJX_ERR_ARCH;
    if (cached[dev] == 0) {
        int major = 0;
        if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return OJX_ERR_LAUNCH;
        cached[dev] = (major == 10) ? 1 : -1;
    }
    return cached[dev] == 1 ? OJX_OK : OJX_ERR_ARCH;
}

alignas(4096) static volatile int g_host_status_page[1024];

int* host_status_device_ptr() {
    static std::once_flag once;
    static bool registered = false;
    std::call_once(once, [] {
        const cudaError_t e = cudaHostRegister(const_cast<int*>(g_host_status_page), sizeof(g_host_status_page), cudaHostRegisterMapped);
        registered = (e == cudaSuccess || e == cudaErrorHostMemoryAlreadyRegistered);
        (void)cudaGetLastError();
    });
    if (!registered) return nullptr;
    static int* cached[64] = {nullptr};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (cached[dev] == nullptr) {
        int* p = nullptr;
        if (cudaHostGetDevicePointer(reinterpret_cast<void**>(&p), const_cast<int*>(g_host_status_page), 0) != cudaSuccess) {
            (void)cudaGetLastError();
            return nullptr;
        }
        cached[dev] = p;
    }
    return cached[dev];
}

int host_status_take() {
    const int v = g_host_status_page[0];
    if (v != 0) g_host_status_page[0] = 0;
    return v;
}

uint32_t& wait_limit_override() {
    static uint32_t v = 0;
    return v;
}

}  // namespace ojx

extern "C" {

int32_t ojx_e8t_version(void) { return 300; }

const char* ojx_e8t_status_string(int32_t st) {
    switch (st) {
        case OJX_OK: return "OJX_OK";
        case OJX_ERR_NULL: return "OJX_ERR_NULL";
        case OJX_ERR_SHAPE: return "OJX_ERR_SHAPE";
        case OJX_ERR_ALIGN: return "OJX_ERR_ALIGN";
        case OJX_ERR_DTYPE: return "OJX_ERR_DTYPE";
        case OJX_ERR_ARCH: return "OJX_ERR_ARCH";
        case OJX_ERR_LAUNCH: return "OJX_ERR_LAUNCH";
        case OJX_ERR_TIMEOUT: return "OJX_ERR_TIMEOUT";
        case OJX_ERR_WORKSPACE: return "OJX_ERR_WORKSPACE";
        case OJX_ERR_UNSUPPORTED: return "OJX_ERR_UNSUPPORTED";
        default: return "OJX_ERR_UNKNOWN";
    }
}

const char* ojx_e8t_last_cuda_error(void) { return cudaGetErrorString(ojx::last_cuda_error()); }

int32_t ojx_e8t_device_status(void) {
    int h = 0;
    const int zero = 0;
    if (cudaDeviceSynchronize() != cudaSuccess) { ojx::last_cuda_error() = cudaGetLastError(); return OJX_ERR_LAUNCH; }
    if (cudaMemcpyFromSymbol(&h, ojx::g_device_status, sizeof(int)) != cudaSuccess) return OJX_ERR_LAUNCH;
    if (h != 0 && cudaMemcpyToSymbol(ojx::g_device_status, &zero, sizeof(int)) != cudaSuccess) return OJX_ERR_LAUNCH;
    (void)ojx::host_status_take();
    return h == 0 ? OJX_OK : OJX_ERR_TIMEOUT;
}

int32_t ojx_e8t_poll_status(void) { return ojx::host_status_take() == 0 ? OJX_OK : OJX_ERR_TIMEOUT; }

void ojx_e8t_set_wait_limit(uint32_t polls) { ojx::wait_limit_override() = polls; }

int32_t ojx_e8t_encode(const void* w, int32_t w_dtype, int64_t rows, int64_t cols, int32_t group,
                       uint8_t* packed_out, uint16_t* scales_out, void* stream) {
    return ojx::encode_impl(w, w_dtype, rows, cols, group, 0u, packed_out, scales_out, (cudaStream_t)stream);
}

int32_t ojx_e8t_encode_ex(const void* w, int32_t w_dtype, int64_t rows, int64_t cols, int32_t group, uint32_t flags,
                          uint8_t* packed_out, uint16_t* scales_out, void* stream) {
    return ojx::encode_impl(w, w_dtype, rows, cols, group, flags, packed_out, scales_out, (cudaStream_t)stream);
}

int32_t ojx_e8t_encode_2bit(const void* w, int32_t w_dtype, int64_t rows, int64_t cols, int32_t group,
                            uint8_t* packed_out, uint16_t* scales_out, void* stream) {
    return ojx::encode2_impl(w, w_dtype, rows, cols, group, packed_out, scales_out, (cudaStream_t)stream);
}

int32_t ojx_e8t_decode_2bit(const uint8_t* packed, const uint16_t* scales, int64_t rows, int64_t cols, int32_t group,
                            int32_t out_dtype, void* out, void* stream) {
    return ojx::decode2_impl(packed, scales, rows, cols, group, out_dtype, out, (cudaStream_t)stream);
}

int32_t ojx_e8t_linear_2bit(const void* x, int32_t x_dtype, int64_t M, const uint8_t* packed, const uint16_t* scales,
                            const void* bias, int64_t N, int64_t K, int32_t group, void* y, int32_t y_dtype, void* stream) {
    return ojx::linear_lowbit_impl(2, x, x_dtype, M, packed, scales, bias, N, K, group, y, y_dtype, (cudaStream_t)stream, nullptr, nullptr, 0);
}

int32_t ojx_e8t_encode_1bit(const void* w, int32_t w_dtype, int64_t rows, int64_t cols, int32_t group,
                            uint8_t* packed_out, uint16_t* scales_out, void* stream) {
    return ojx::encode1_impl(w, w_dtype, rows, cols, group, packed_out, scales_out, (cudaStream_t)stream);
}

int32_t ojx_e8t_decode_1bit(const uint8_t* packed, const uint16_t* scales, int64_t rows, int64_t cols, int32_t group,
                            int32_t out_dtype, void* out, void* stream) {
    return ojx::decode1_impl(packed, scales, rows, cols, group, out_dtype, out, (cudaStream_t)stream);
}

int32_t ojx_e8t_linear_1bit(const void* x, int32_t x_dtype, int64_t M, const uint8_t* packed, const uint16_t* scales,
                            const void* bias, int64_t N, int64_t K, int32_t group, void* y, int32_t y_dtype, void* stream) {
    return ojx::linear_lowbit_impl(1, x, x_dtype, M, packed, scales, bias, N, K, group, y, y_dtype, (cudaStream_t)stream, nullptr, nullptr, 0);
}

int32_t ojx_e8t_linear_lowbit_lora(int32_t bits, const void* x, int32_t x_dtype, int64_t M, const uint8_t* packed,
                                   const uint16_t* scales, const void* bias, int64_t N, int64_t K, int32_t group,
                                   const float* lora_t, const void* lora_b, int32_t lora_rank,
                                   void* y, int32_t y_dtype, void* stream) {
    if (bits != 1 && bits != 2) return OJX_ERR_UNSUPPORTED;
    if (lora_rank <= 0) return OJX_ERR_SHAPE;
    return ojx::linear_lowbit_impl(bits, x, x_dtype, M, packed, scales, bias, N, K, group, y, y_dtype, (cudaStream_t)stream,
                                   lora_t, lora_b, lora_rank);
}

int32_t ojx_e8t_project(const float* x, int64_t vectors, float* out, void* stream) {
    if (vectors <= 0 || vectors > (INT64_MAX >> 3)) return OJX_ERR_SHAPE;
    return ojx::e8_project_impl(x, vectors * 8, out, false, (cudaStream_t)stream);
}

int32_t ojx_e8t_ste_quantize(const float* w, int64_t count, float* out, void* stream) {
    return ojx::e8_project_impl(w, count, out, true, (cudaStream_t)stream);
}

int32_t ojx_e8t_fwht32(const void* x, int32_t dtype, int64_t count, void* out, void* stream) {
    return ojx::fwht32_impl(x, dtype, count, out, (cudaStream_t)stream);
}

int32_t ojx_e8t_decode(const uint8_t* packed, const uint16_t* scales, int64_t rows, int64_t cols,
                       int32_t group, int32_t out_dtype, void* out, void* stream) {
    return ojx::decode_impl(packed, scales, rows, cols, group, out_dtype, out, (cudaStream_t)stream);
}

size_t ojx_e8t_gemv_workspace_bytes(int64_t M, int64_t N, int64_t K) { return ojx::gemv_workspace_bytes_impl(M, N, K); }

int32_t ojx_e8t_gemv(const void* x, int32_t x_dtype, int64_t M, const uint8_t* packed, const uint16_t* scales,
                     const void* bias, int64_t N, int64_t K, int32_t group, void* y, int32_t y_dtype,
                     void* workspace, size_t workspace_bytes, void* stream) {
    return ojx::gemv_impl(x, x_dtype, M, packed, scales, bias, N, K, group, y, y_dtype, workspace, workspace_bytes,
                          (cudaStream_t)stream);
}

int32_t ojx_e8t_gemv_lora(const void* x, int32_t x_dtype, int64_t M, const uint8_t* packed, const uint16_t* scales,
                          const void* bias, int64_t N, int64_t K, int32_t group, const float* lora_t, const void* lora_b,
                          int32_t lora_rank, void* y, int32_t y_dtype, void* workspace, size_t workspace_bytes, void* stream) {
    return ojx::gemv_impl(x, x_dtype, M, packed, scales, bias, N, K, group, y, y_dtype, workspace, workspace_bytes,
                          (cudaStream_t)stream, lora_t, lora_b, lora_rank);
}

size_t ojx_e8t_gemv_static_scratch_capacity(void) { return ojx::gemv_static_scratch_capacity_impl(); }

int32_t ojx_e8t_gemv_static_scratch(const void* x, int32_t x_dtype, int64_t M, const uint8_t* packed, const uint16_t* scales,
                                    const void* bias, int64_t N, int64_t K, int32_t group, void* y, int32_t y_dtype,
                                    void* stream) {
    return ojx::gemv_static_scratch_impl(x, x_dtype, M, packed, scales, bias, N, K, group, y, y_dtype, (cudaStream_t)stream);
}

int32_t ojx_e8t_gemv_tiles(int64_t N, int64_t K) { return ojx::gemv_tiles_impl(N, K); }
int32_t ojx_e8t_gemv_kchunks(int64_t K) { return ojx::gemv_kchunks_impl(K); }

int32_t ojx_e8t_gemv_grouped(const ojx_e8t_gemv_problem* problems, int32_t count, int32_t total_tiles, int64_t M,
                             int32_t x_dtype, int32_t y_dtype, int32_t needs_reduce, void* stream) {
    return ojx::gemv_grouped_impl(problems, count, total_tiles, M, x_dtype, y_dtype, needs_reduce, nullptr, 1, nullptr, 0, (cudaStream_t)stream);
}

int32_t ojx_e8t_gemv_grouped_peers(const ojx_e8t_gemv_problem* problems, int32_t count, int32_t total_tiles, int64_t M,
                                   int32_t x_dtype, int32_t y_dtype, int32_t needs_reduce,
                                   const int64_t* peer_delta, int32_t world, void* stream) {
    OJX_RETURN_IF(!peer_delta, OJX_ERR_NULL);
    return ojx::gemv_grouped_impl(problems, count, total_tiles, M, x_dtype, y_dtype, needs_reduce, peer_delta, world, nullptr, 0, (cudaStream_t)stream);
}

int32_t ojx_e8t_gemv_grouped_ex(const ojx_e8t_gemv_problem* problems, int32_t count, int32_t total_tiles, int64_t M,
                                int32_t x_dtype, int32_t y_dtype, int32_t needs_reduce,
                                const int64_t* peer_delta, int32_t world, ojx_e8t_peer_sync* peer_sync, int32_t flags,
                                void* stream) {
    return ojx::gemv_grouped_impl(problems, count, total_tiles, M, x_dtype, y_dtype, needs_reduce, peer_delta,
                                  peer_delta ? world : 1, peer_sync, flags, (cudaStream_t)stream);
}

int32_t ojx_e8t_peer_wait(ojx_e8t_peer_sync* peer_sync, int32_t world, void* stream) {
    return ojx::peer_wait_impl(peer_sync, world, (cudaStream_t)stream);
}

int32_t ojx_e8t_enable_peer_access(int32_t peer_device) {
    int cur = -1, can = 0;
    if (cudaGetDevice(&cur) != cudaSuccess) { ojx::last_cuda_error() = cudaGetLastError(); return OJX_ERR_LAUNCH; }
    if (peer_device == cur) return OJX_OK;
    if (cudaDeviceCanAccessPeer(&can, cur, peer_device) != cudaSuccess) { ojx::last_cuda_error() = cudaGetLastError(); return OJX_ERR_LAUNCH; }
    if (!can) return OJX_ERR_UNSUPPORTED;
    const cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) { (void)cudaGetLastError(); return OJX_OK; }
    if (e != cudaSuccess) { ojx::last_cuda_error() = e; (void)cudaGetLastError(); return OJX_ERR_LAUNCH; }
    return OJX_OK;
}

size_t ojx_e8t_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K) { return ojx::gemm_workspace_bytes_impl(M, N, K); }

int32_t ojx_e8t_gemm(const void* x, int32_t x_dtype, int64_t M, const uint8_t* packed, const uint16_t* scales,
                     const void* bias, int64_t N, int64_t K, int32_t group, void* y, int32_t y_dtype,
                     void* workspace, size_t workspace_bytes, void* stream) {
    return ojx::gemm_impl(x, x_dtype, M, packed, scales, bias, N, K, group, y, y_dtype, workspace, workspace_bytes,
                          (cudaStream_t)stream);
}

int32_t ojx_e8t_gemm_lowbit(int32_t bits, const void* x, int32_t x_dtype, int64_t M, const uint8_t* packed, const uint16_t* scales,
                            const void* bias, int64_t N, int64_t K, int32_t group, void* y, int32_t y_dtype,
                            void* workspace, size_t workspace_bytes, void* stream) {
    if (bits != 1 && bits != 2) return OJX_ERR_UNSUPPORTED;
    return ojx::gemm_fmt_impl(bits, x, x_dtype, M, packed, scales, bias, N, K, group, y, y_dtype, workspace, workspace_bytes,
                              (cudaStream_t)stream);
}

size_t ojx_e8t_gemm_dx_workspace_bytes(int64_t M, int64_t N, int64_t K) { return ojx::gemm_dx_workspace_bytes_impl(M, N, K); }

int32_t ojx_e8t_gemm_dx(const void* grad_y, int32_t gy_dtype, int64_t M, const uint8_t* packed, const uint16_t* scales,
                        int64_t N, int64_t K, int32_t group, void* dx, int32_t dx_dtype,
                        void* workspace, size_t workspace_bytes, void* stream) {
    return ojx::gemm_dx_impl(grad_y, gy_dtype, M, packed, scales, N, K, group, dx, dx_dtype, workspace, workspace_bytes,
                             (cudaStream_t)stream);
}

int32_t ojx_e8t_gemm_dx_lowbit(int32_t bits, const void* grad_y, int32_t gy_dtype, int64_t M, const uint8_t* packed,
                               const uint16_t* scales, int64_t N, int64_t K, int32_t group, void* dx, int32_t dx_dtype,
                               void* workspace, size_t workspace_bytes, void* stream) {
    if (bits != 1 && bits != 2) return OJX_ERR_UNSUPPORTED;
    return ojx::gemm_dx_fmt_impl(bits, grad_y, gy_dtype, M, packed, scales, N, K, group, dx, dx_dtype, workspace, workspace_bytes,
                                 (cudaStream_t)stream);
}

int32_t ojx_e8t_gemm_status(const void* workspace, void* stream) {
    return ojx::gemm_status_impl(workspace, (cudaStream_t)stream);
}

int32_t ojx_e8t_generate(void* out, int32_t dtype, int64_t count, uint64_t seed, int64_t start, float sigma,
                         void* stream) {
    return ojx::generate_impl(out, dtype, count, seed, start, sigma, (cudaStream_t)stream);
}

}  // extern "C"
