/*
 * ojx_e8t.h - C ABI of the B200 (sm_100a) ternary-E8 quantized-linear kernels.
 *
 * Packed format (identical to the reference's, so buffers are interchangeable):
 *   codes   uint8[P*3/16]  every 3 bytes hold two 12-bit lattice ranks c0,c1 covering 16
 *                          consecutive weights: b0=c0&0xFF, b1=(c0>>8)|((c1&0xF)<<4), b2=c1>>4
 *   scales  fp16[P/g]      one RMS scale per group of g consecutive weights (g = 32 by default)
 *   P = rows*cols rounded up to a multiple of g; weights are taken row-major.  When cols % g == 0
 *   every row owns whole groups: row n starts at byte n*cols*3/16 and at scale n*cols/g.
 *
 * Conventions for every entry point
 *   - returns an ojx_status (0 = ok, negative = error); never throws, never traps;
 *   - never allocates device or host memory: every buffer, including scratch, is owned by the
 *     caller (one documented exception below carries its own static scratch);
 *   - asynchronous: work is enqueued on `stream` (a cudaStream_t passed as void*);
 *   - all pointers are device pointers unless stated otherwise.
 *
 * The functions replace the following parts of the reference project (file:line inside it):
 *   ojx_e8t_encode        TernaryE8LatticePacker.pack            ojasx2/math/lattice.py:338-384
 *                         (and its row-block caller)             ojasx2/streaming_e8.py:112-159
 *   ojx_e8t_decode        TernaryE8LatticePacker.unpack          ojasx2/math/lattice.py:386-419
 *                         workspace reconstruction               ojasx2/math/lattice.py:62-84,412-416
 *   ojx_e8t_fwht32        fwht_block32                           ojasx2/math/lattice.py:91-102
 *   ojx_e8t_project       conway_sloane_e8_project               ojasx2/math/lattice.py:162-203
 *   ojx_e8t_ste_quantize  _E8STEFunction.forward                 ojasx2/math/lattice.py:853-867
 *   ojx_e8t_gemv/_gemm    _FusedE8GEMMFunction.forward           ojasx2/math/lattice.py:551-640
 *                         dispatch_tilelang_e8_gemm              ojasx2/tilelang_kernels.py:370-419
 *                         _build_tl_ternary_e8_1_5bit_gemm       ojasx2/tilelang_kernels.py:277-363
 *                         fused_ternary_e8_gemm_forward<T>       ojasx2/math/csrc/ojasx_math_core.hpp:580-634
 *                         op schema fused_ternary_e8_gemm_fwd    ojasx2/math/csrc/ojasx_math_bindings.cpp:586-595
 */
#ifndef OJX_E8T_H
#define OJX_E8T_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    OJX_OK = 0,
    OJX_ERR_NULL = -1,        /* a required pointer is null */
    OJX_ERR_SHAPE = -2,       /* sizes are zero/negative or violate the layout rules */
    OJX_ERR_ALIGN = -3,       /* a pointer or row stride is not aligned as required */
    OJX_ERR_DTYPE = -4,       /* unknown or unsupported element type */
    OJX_ERR_ARCH = -5,        /* the current device is not sm_100 */
    OJX_ERR_LAUNCH = -6,      /* the CUDA runtime rejected a launch or a set-up call */
    OJX_ERR_TIMEOUT = -7,     /* a bounded device-side wait gave up (reported by ojx_e8t_gemm_status) */
    OJX_ERR_WORKSPACE = -8,   /* scratch buffer missing or too small */
    OJX_ERR_UNSUPPORTED = -9  /* valid request that this build does not implement */
} ojx_status;

typedef enum { OJX_F32 = 0, OJX_F16 = 1, OJX_BF16 = 2 } ojx_dtype;

/* Library version: major*10000 + minor*100 + patch. */
int32_t ojx_e8t_version(void);

/* Static, human readable name of a status code. */
const char* ojx_e8t_status_string(int32_t status);

/*
 * Diagnostics (no counterpart in the reference).
 * ojx_e8t_last_cuda_error: text of the last CUDA runtime error that made an entry point return
 *   OJX_ERR_LAUNCH on the calling thread.
 * Every wait inside the kernels (on a copy in flight, on another rank) is bounded; a kernel whose wait runs
 * out stops working on its inputs, returns, and records the fact in two places:
 * ojx_e8t_device_status: synchronises the current device, returns OJX_ERR_TIMEOUT if a wait gave up since the
 *   last call, else OJX_OK, and clears the record.
 * ojx_e8t_poll_status: the same answer WITHOUT synchronising - the kernels also write into a page of pinned
 *   host memory that belongs to the library - so a wrapper can check it cheaply at the start of every call
 *   and raise; it reports launches that have already run into the limit, and clears the record.
 *   (The page is pinned on the first decode-shape call of the process: make that call before a stream capture.)
 * ojx_e8t_set_wait_limit: polls before a wait on a copy gives up (0 restores the default of 2^24, seconds);
 *   for tests of the error path.
 */
const char* ojx_e8t_last_cuda_error(void);
int32_t ojx_e8t_device_status(void);
int32_t ojx_e8t_poll_status(void);
void    ojx_e8t_set_wait_limit(uint32_t polls);

/*
 * Encoder.  Replaces TernaryE8LatticePacker.pack (ojasx2/math/lattice.py:338-384); bit-exact.
 *   w         [rows, cols] row-major, dtype w_dtype (fp32 / fp16 / bf16), any alignment of rows
 *   group     scale group size; values that are not a positive multiple of 16 are replaced by 16,
 *             exactly as the reference does (lattice.py:346-347)
 *   packed_out uint8[P*3/16], scales_out fp16[P/g] with P = rows*cols padded up to g
 */
int32_t ojx_e8t_encode(const void* w, int32_t w_dtype, int64_t rows, int64_t cols, int32_t group,
                       uint8_t* packed_out, uint16_t* scales_out, void* stream);

/*
 * Encoder with options.  flags = 0 is ojx_e8t_encode.  OJX_ENCODE_HADAMARD rotates every block of 32
 * consecutive weights of a row by the normalised Walsh-Hadamard transform in registers before encoding it, in
 * w's own arithmetic - the bytes equal pack(fwht_block32(w)), which is what the reference's _pack_row_block
 * (ojasx2/streaming_e8.py:112-125) and E8LatticeLinear.from_linear (ojasx2/math/lattice.py:783-812) compute with
 * use_hadamard=True, without the rotated copy of w in memory.  Needs group == 32 and cols % 32 == 0
 * (OJX_ERR_SHAPE otherwise); unknown flag bits return OJX_ERR_UNSUPPORTED.
 */
#define OJX_ENCODE_HADAMARD 1u
int32_t ojx_e8t_encode_ex(const void* w, int32_t w_dtype, int64_t rows, int64_t cols, int32_t group, uint32_t flags,
                          uint8_t* packed_out, uint16_t* scales_out, void* stream);

/*
 * 32-point normalised Walsh-Hadamard transform of every block of 32 consecutive elements.  Replaces
 * fwht_block32 (ojasx2/math/lattice.py:91-102) bit for bit: butterflies and the final scaling are rounded to the
 * element type exactly where the reference's tensor operations round.  count % 32 == 0; x and out 16-byte
 * aligned; out may be x.
 */
int32_t ojx_e8t_fwht32(const void* x, int32_t dtype, int64_t count, void* out, void* stream);

/*
 * The 2.0-bit sibling format (four 2-bit codes per byte, weight = (code - 1.5) * scale, one fp16 rms scale per
 * group of `group` consecutive weights of the flattened matrix; group a positive multiple of 8, anything else
 * returns OJX_ERR_SHAPE where the reference raises ValueError).
 *   ojx_e8t_encode_2bit   replaces E8LatticePacker.pack   (ojasx2/math/lattice.py:210-248), bit-exact:
 *                         packed_out uint8[P/4], scales_out fp16[P/group], P = rows*cols padded up to group
 *   ojx_e8t_decode_2bit   replaces E8LatticePacker.unpack (ojasx2/math/lattice.py:250-279): fp32 and fp16 exact,
 *                         bf16 multiplies by the bf16-rounded scale as the reference does
 *   ojx_e8t_linear_2bit   y[M, N] = x[M, K] . W^T (+ bias) from the packed codes in one fp32 kernel (any shape,
 *                         any of the three dtypes for x, bias (x's dtype) and y); replaces the 2.0-bit branch of
 *                         _FusedE8GEMMFunction.forward (ojasx2/math/lattice.py:596-624) and the native
 *                         fused_e8_gemm_forward<T> (ojasx2/math/csrc/ojasx_math_core.hpp:444).  One to eight rows
 *                         with group 32, K % 2048 == 0 and 16-byte aligned operands run on int8 tensor cores
 *                         (activations as 28-bit fixed point per scale group, as in ojx_e8t_gemv for one bf16 row;
 *                         Inf / NaN in x give the dense product's pattern); other shapes of up to eight rows with
 *                         K % 16 == 0 and 16-byte aligned x run a shared-memory fp32 kernel (a row of x with Inf
 *                         comes out as NaN there), everything else a scalar fp32 kernel.
 */
int32_t ojx_e8t_encode_2bit(const void* w, int32_t w_dtype, int64_t rows, int64_t cols, int32_t group,
                            uint8_t* packed_out, uint16_t* scales_out, void* stream);
int32_t ojx_e8t_decode_2bit(const uint8_t* packed, const uint16_t* scales, int64_t rows, int64_t cols, int32_t group,
                            int32_t out_dtype, void* out, void* stream);
int32_t ojx_e8t_linear_2bit(const void* x, int32_t x_dtype, int64_t M, const uint8_t* packed, const uint16_t* scales,
                            const void* bias, int64_t N, int64_t K, int32_t group, void* y, int32_t y_dtype, void* stream);

/*
 * The 1.0-bit sibling format (one byte per 8 weights: the index of one of 256 vectors - the 240 roots of E8 and 16 axis
 * vectors, doubled; weight = coordinate * scale, one fp16 least-squares scale per group; group a positive multiple of
 * 8, anything else is replaced by 8 in the encoder, as the reference does).
 *   ojx_e8t_encode_1bit   replaces RootE8LatticePacker.pack   (ojasx2/math/lattice.py:475-512): packed_out uint8[P/8],
 *                         scales_out fp16[P/group].  Bit-exact with the reference's CPU path, where each entry of
 *                         torch.matmul(v, normalize(table)^T) is a chain of fused multiply-adds over k = 0..7 and
 *                         torch.sum adds chunks of eight into four vector accumulators in turn; a BLAS that rounds the
 *                         8-term dot products differently may pick the other of two nearly equal candidates.
 *   ojx_e8t_decode_1bit   replaces RootE8LatticePacker.unpack (ojasx2/math/lattice.py:514-537)
 *   ojx_e8t_linear_1bit   y = x . W^T (+ bias) from the codes; the same three kernels as for 2 bits: int8 tensor
 *                         cores for one to eight rows with group 32 and K % 2048 == 0 (a code byte is looked up as
 *                         eight int8 operand bytes), the shared-memory fp32 kernel, the scalar fp32 kernel
 */
int32_t ojx_e8t_encode_1bit(const void* w, int32_t w_dtype, int64_t rows, int64_t cols, int32_t group,
                            uint8_t* packed_out, uint16_t* scales_out, void* stream);
int32_t ojx_e8t_decode_1bit(const uint8_t* packed, const uint16_t* scales, int64_t rows, int64_t cols, int32_t group,
                            int32_t out_dtype, void* out, void* stream);
int32_t ojx_e8t_linear_1bit(const void* x, int32_t x_dtype, int64_t M, const uint8_t* packed, const uint16_t* scales,
                            const void* bias, int64_t N, int64_t K, int32_t group, void* y, int32_t y_dtype, void* stream);

/*
 * Decode-shape linear of the 2.0-bit (`bits` 2) or 1.0-bit (`bits` 1) format with the adapter term in the epilogue:
 * y = x . W^T (+ bias) + lora_t . lora_b, lora_t fp32 [M, lora_rank] = scaling * (x . A) prepared by the caller,
 * lora_b [lora_rank, N] in x's dtype, accumulated in fp32 before the single rounding (the reference adds the term with
 * three more tensor operations, ojasx2/math/lattice.py:839-842).  Only the shapes of the int8 tensor-core kernels are
 * served (1 <= M <= 8, group 32, K % 2048 == 0, 16-byte aligned operands, 1 <= lora_rank <= 64); anything else returns
 * OJX_ERR_UNSUPPORTED and the caller adds the term itself.
 */
int32_t ojx_e8t_linear_lowbit_lora(int32_t bits, const void* x, int32_t x_dtype, int64_t M, const uint8_t* packed,
                                   const uint16_t* scales, const void* bias, int64_t N, int64_t K, int32_t group,
                                   const float* lora_t, const void* lora_b, int32_t lora_rank,
                                   void* y, int32_t y_dtype, void* stream);

/*
 * Nearest point of the E8 lattice (integer vectors with an even sum, or all of them shifted by 1/2) for
 * each of `vectors` consecutive 8-vectors.  Replaces conway_sloane_e8_project (ojasx2/math/lattice.py:162-203;
 * native form ojasx_math_core.hpp:385-425) bit for bit on fp32 input: round-half-even, first index wins the
 * "largest rounding error" tie, an exact integer moves up when the parity has to be fixed, the integer candidate
 * wins a distance tie, squared distances summed left to right without fused multiply-adds.  x and out fp32,
 * 16-byte aligned; out may be x.  NaN input gives unspecified output for that vector.
 */
int32_t ojx_e8t_project(const float* x, int64_t vectors, float* out, void* stream);

/*
 * Forward of the straight-through E8 quantizer.  Replaces _E8STEFunction.forward
 * (ojasx2/math/lattice.py:853-867) bit for bit on fp32 input: every group of eight consecutive elements of the
 * flattened tensor (the last one zero-padded) is divided by its rms + 1e-8, projected to E8 and multiplied
 * back, in one pass.  w and out fp32, 16-byte aligned, `count` elements; out may be w.
 */
int32_t ojx_e8t_ste_quantize(const float* w, int64_t count, float* out, void* stream);

/*
 * Decoder.  Replaces TernaryE8LatticePacker.unpack (ojasx2/math/lattice.py:386-419).
 * out[rows, cols] = coord * cast(scale): fp32 and fp16 outputs are exact; bf16 output multiplies
 * by the bf16-rounded scale, as the reference does when asked for bf16.
 */
int32_t ojx_e8t_decode(const uint8_t* packed, const uint16_t* scales, int64_t rows, int64_t cols,
                       int32_t group, int32_t out_dtype, void* out, void* stream);

/*
 * Decode-shape linear (small M): y[M, N] = x[M, K] . W^T (+ bias), W given packed.
 * Replaces _FusedE8GEMMFunction.forward for small batches (ojasx2/math/lattice.py:551-640) and the
 * reference's native fused kernel (ojasx_math_core.hpp:580-634).  fp32 accumulation.
 * Shapes outside the tensor-core path: up to eight rows with K % 64 == 0, a power-of-two group from 16 and 16-byte
 * aligned x (any of the three dtypes) run a shared-memory fp32 kernel with exact products; everything else a scalar
 * fp32 kernel.
 * Numerics of the tensor-core path (M <= 16, K % 256 == 0, group 32, bf16 or fp16 x): the weights enter the
 * MMAs as exact fp16 values coord * scale; fp16 activations are used as they are; bf16 activations are
 * multiplied by a power of two per (row, 256-wide slice of K) so that the slice maximum lies in [2^14, 2^15)
 * and converted to fp16 - exact for every element within 2^-29 of its slice maximum, so an activation
 * outlier does not degrade its neighbours; products are exact and accumulate in fp32.  Inf and NaN in x reach
 * every output of that activation row (0 * Inf = NaN, as in a dense product).
 * One bf16 activation row (M == 1, the decode case) runs on int8 tensor cores instead: the 32 activations of a
 * scale group share the exponent of their largest finite magnitude and become 28-bit integers (four signed
 * base-128 digits, one int8 MMA operand each), the ternary coordinates are int8, the integer dot product of a
 * group is exact and is scaled once by weight scale * 2^exponent in fp32.  Every activation within 2^-19 of
 * its group's maximum is represented exactly, smaller ones are rounded at 2^-27 of that maximum (below the
 * rounding of the fp32 accumulation itself); scaling x by a power of two scales y by exactly that power.
 * Inf / NaN activations are left out of the integer product and their products with the weights are added in
 * fp32, which yields the same NaN / +-Inf pattern as a dense fp32 product.
 * Other shapes and fp32 activations run a plain fp32 kernel.
 *   x, y       row-major, dtypes x_dtype / y_dtype (bf16, fp16 or fp32)
 *   bias       [N] in x_dtype, or null
 *   group      must be 32 and K % 32 == 0 (every row owns whole groups)
 *   workspace  scratch of at least ojx_e8t_gemv_workspace_bytes(M, N, K) bytes (may be null when
 *              that function returns 0); contents need not be initialised
 */
size_t  ojx_e8t_gemv_workspace_bytes(int64_t M, int64_t N, int64_t K);
int32_t ojx_e8t_gemv(const void* x, int32_t x_dtype, int64_t M,
                     const uint8_t* packed, const uint16_t* scales, const void* bias,
                     int64_t N, int64_t K, int32_t group,
                     void* y, int32_t y_dtype,
                     void* workspace, size_t workspace_bytes, void* stream);

/*
 * ojx_e8t_gemv with the adapter term of E8LatticeLinear.forward_fused (ojasx2/math/lattice.py:826-842) fused into the
 * epilogue: y = x . W^T (+ bias) + lora_t . lora_b, where lora_t [M, lora_rank] fp32 = scaling * (x . A) and lora_b
 * [lora_rank, N] has x's dtype.  Only the tensor-core decode shapes up to eight rows are served (1 <= M <= 8, K % 256 == 0, group 32,
 * 16-bit x, 16-byte aligned buffers, lora_rank <= 64); anything else returns OJX_ERR_UNSUPPORTED and the caller adds
 * the term itself.
 */
int32_t ojx_e8t_gemv_lora(const void* x, int32_t x_dtype, int64_t M,
                          const uint8_t* packed, const uint16_t* scales, const void* bias,
                          int64_t N, int64_t K, int32_t group,
                          const float* lora_t, const void* lora_b, int32_t lora_rank,
                          void* y, int32_t y_dtype,
                          void* workspace, size_t workspace_bytes, void* stream);

/*
 * ojx_e8t_gemv for callers that cannot hand over scratch memory (no counterpart in the reference).
 * Meant for hosts where a plug-in only ever sees its input and output buffers: a serving process whose
 * device memory is pre-carved by its own arena, a callback that runs where cudaMalloc is not allowed
 * (it synchronises the device), a worker without allocation rights.  The fp32 partial sums that
 * K > 4096 needs are kept in a 4 MiB array that is part of the library image on every GPU that loads
 * it; the call allocates nothing and frees nothing.
 *   - Same arguments and results as ojx_e8t_gemv, minus the workspace.
 *   - Limit: ojx_e8t_gemv_workspace_bytes(M, N, K) must not exceed
 *     ojx_e8t_gemv_static_scratch_capacity() (4 MiB; e.g. K = 14336, N = 4096, M = 16 needs 1 MiB);
 *     larger problems return OJX_ERR_WORKSPACE and must use ojx_e8t_gemv with caller scratch.
 *   - The first call on each device looks up the array's device address (a driver query, done once
 *     per device with that device current); make that first call before starting a stream capture.
 *   - All calls share the one array.  It keeps whatever the last call left; nothing needs clearing
 *     because every element is written before it is read.  Two calls that run on the GPU at the same
 *     time (different streams, or different threads) would overwrite each other's partial sums:
 *     serialise them.
 */
size_t  ojx_e8t_gemv_static_scratch_capacity(void);
int32_t ojx_e8t_gemv_static_scratch(const void* x, int32_t x_dtype, int64_t M,
                                    const uint8_t* packed, const uint16_t* scales, const void* bias,
                                    int64_t N, int64_t K, int32_t group,
                                    void* y, int32_t y_dtype, void* stream);

/*
 * Several independent decode-shape linears in ONE launch (for example q/k/v, or gate/up, or a
 * rotation of matrices in a benchmark).  `problems` is a DEVICE array of `count` descriptors;
 * `total_tiles` is the sum over problems of ojx_e8t_gemv_tiles(N, K).  All problems share M,
 * x_dtype and y_dtype; every K must be a multiple of 256.  Pass needs_reduce != 0 when any problem
 * has ojx_e8t_gemv_kchunks(K) > 1 (its `partial` scratch is then summed by a second small kernel).  No counterpart in the reference, which runs one layer per call.
 */
typedef struct {
    const void*     x;        /* [M, K] */
    const uint8_t*  packed;   /* [N, K*3/16] */
    const uint16_t* scales;   /* [N, K/32] */
    const void*     bias;     /* [N] or null */
    void*           y;        /* [M, N] */
    float*          partial;  /* scratch [kchunks, M, N] fp32 when kchunks > 1, else null */
    int32_t         N, K;
    int32_t         tile_begin;   /* exclusive prefix sum of tiles over the problem list */
    int32_t         ldy;          /* distance in elements between consecutive rows of y; 0 means N.  A larger value lets
                                     y be a column block of a wider [M, ldy] matrix (the place of one rank's shard in
                                     the full output of a column-sharded linear) */
    /* Optional low-rank term added in the epilogue, in fp32, before the one rounding to y's type:
     *   y[m, n] += sum_r lora_t[m, r] * lora_b[r, n]
     * lora_t = scaling * (x . A) as fp32 [M, lora_rank] (computed by the caller; it is read after the product, so it may
     * be produced by work queued just ahead of the launch), lora_b [lora_rank, N] in x's dtype.  lora_rank == 0: none;
     * honoured for M <= 8.
     * This is the adapter term of E8LatticeLinear.forward_fused (ojasx2/math/lattice.py:839-842). */
    const float*    lora_t;
    const void*     lora_b;
    int32_t         lora_rank;
    int32_t         reserved;
} ojx_e8t_gemv_problem;

int32_t ojx_e8t_gemv_tiles(int64_t N, int64_t K);
int32_t ojx_e8t_gemv_kchunks(int64_t K);
int32_t ojx_e8t_gemv_grouped(const ojx_e8t_gemv_problem* problems, int32_t count, int32_t total_tiles,
                             int64_t M, int32_t x_dtype, int32_t y_dtype, int32_t needs_reduce, void* stream);

/*
 * Grouped decode-shape launch whose results go straight into EVERY rank's output window (fused
 * all-gather for output-column sharding; no counterpart in the reference, which is single-device).
 * Every rank holds an identically laid out output window; problems[i].y points into THIS rank's
 * window at the place of this rank's shard, and peer_delta[r] (r < world, world <= 8) is the byte
 * distance from this rank's window to rank r's window as mapped into this process (0 for this rank;
 * e.g. from CUDA IPC handles).  The kernel stores each result `world` times - plain stores over
 * NVLink, no device-side waiting, nothing is loaded from a peer.  The caller orders the exchange: a peer may
 * read its window only after this launch has completed on this rank's stream and the ranks have met
 * (one small collective or barrier per step instead of one all-gather per launch).
 */
int32_t ojx_e8t_gemv_grouped_peers(const ojx_e8t_gemv_problem* problems, int32_t count, int32_t total_tiles,
                                   int64_t M, int32_t x_dtype, int32_t y_dtype, int32_t needs_reduce,
                                   const int64_t* peer_delta, int32_t world, void* stream);
/*
 * The general form of the two grouped launches above (they call it with peer_sync = null and flags = 0;
 * peer_delta may be null, which means a single rank).  No counterpart in the reference.
 *
 * peer_sync (optional) points at an ojx_e8t_peer_sync block that lives INSIDE the peer-mapped output window
 * (same offset on every rank, so the deltas of the window reach every rank's block) and is zeroed once by
 * its owner.  It lets a chain of column-sharded launches - each one reading, as its activations, the full
 * output its predecessor stored into this rank's window from all ranks - run without a collective or a host
 * round trip in between: every rank must issue the same sequence of launches on the block.
 *
 * Flags:
 *   OJX_GEMV_STATIC_WEIGHTS  the caller promises that no kernel still running or queued ahead of this launch in
 *       `stream` WRITES the packed codes or scales of any problem (they were produced earlier and the producer
 *       has finished, the normal case for inference).  The launch is then allowed to start while its
 *       predecessor in the stream drains: it sets itself up and starts streaming weights, and waits for the
 *       predecessor only before its first read of x and its first write of y (programmatic dependent launch).
 *       Activations, outputs, bias and partial buffers may depend on the predecessor as usual.  Without the flag
 *       the launch is ordered like any other kernel.  Works inside stream capture.
 *   OJX_GEMV_INDEPENDENT     (implies OJX_GEMV_STATIC_WEIGHTS) the caller promises more: NOTHING this launch reads
 *       or writes - activations, bias, outputs, partial buffers - is written or read by the kernels queued ahead of
 *       it in `stream` that may still be running (for example the previous launches of a sweep over different
 *       matrices with their own outputs).  The launch then never waits for its predecessor: its CTAs start as
 *       multiprocessors become free, so the tail of one launch is filled by the head of the next.  Work queued
 *       AFTER the launch is ordered after it as usual.  Not allowed together with the peer flags.
 *   OJX_GEMV_SIGNAL_PEERS    (needs peer_sync and peer_delta) once every result of the launch has been stored into
 *       every rank's window, this rank publishes its next epoch into flag[this rank] of every rank's block
 *       (release at system scope, plain stores over NVLink) and advances its own epoch.
 *   OJX_GEMV_WAIT_PEERS      (needs peer_sync) before the first read of x every CTA waits until flag[q] of the
 *       local block has reached this rank's current epoch for every rank q, i.e. until all ranks have finished
 *       the launch that produced x.  The wait is bounded (spin_limit polls per rank, default about a second):
 *       when it runs out the kernel records OJX_ERR_TIMEOUT in the block's status word and in the device
 *       status (ojx_e8t_device_status), finishes on whatever x holds, and returns - nothing hangs.
 * Nothing is ever loaded from a peer's memory.
 */
typedef struct {
    int32_t epoch;       /* signalled launches of the chain completed on this rank */
    int32_t arrived;     /* CTAs of the running launch that have stored their results */
    int32_t status;      /* 0, or OJX_ERR_TIMEOUT after a wait that gave up */
    int32_t spin_limit;  /* polls per awaited rank before giving up; 0 selects the default */
    int32_t flag[8];     /* flag[q]: the epoch rank q has published into this rank's window */
} ojx_e8t_peer_sync;

#define OJX_GEMV_STATIC_WEIGHTS 1
#define OJX_GEMV_SIGNAL_PEERS   2
#define OJX_GEMV_WAIT_PEERS     4
#define OJX_GEMV_INDEPENDENT    16
#define OJX_GEMV_TEST_LOSE_COPY 8   /* tests only: the first work item's copies are never reported complete, so the
                                       wait on them runs into its limit (set a small one) and the error path runs */
int32_t ojx_e8t_gemv_grouped_ex(const ojx_e8t_gemv_problem* problems, int32_t count, int32_t total_tiles,
                                int64_t M, int32_t x_dtype, int32_t y_dtype, int32_t needs_reduce,
                                const int64_t* peer_delta, int32_t world, ojx_e8t_peer_sync* peer_sync,
                                int32_t flags, void* stream);

/*
 * The wait of OJX_GEMV_WAIT_PEERS on its own, for work of another library that reads a window (an element-wise
 * kernel between two sharded linears, say): everything enqueued in `stream` after this call runs once every rank
 * has published the launch this rank signalled last.  Bounded like the wait inside the kernels.  No counterpart in
 * the reference.
 */
int32_t ojx_e8t_peer_wait(ojx_e8t_peer_sync* peer_sync, int32_t world, void* stream);

/* Lets kernels of the current device address memory that lives on `peer_device` (same node, NVLink or PCIe
 * peer): OJX_OK when access is (already) enabled, OJX_ERR_UNSUPPORTED when the two devices cannot be peers.
 * Required once per peer before ojx_e8t_gemv_grouped_peers stores into that peer's window.  No counterpart in
 * the reference. */
int32_t ojx_e8t_enable_peer_access(int32_t peer_device);

/*
 * Prefill-shape linear (large M) on the tcgen05 tensor cores.  Same contract as ojx_e8t_gemv;
 * replaces the reference's TileLang builder (ojasx2/tilelang_kernels.py:277-363) and the
 * unpack + F.linear path (lattice.py:613-624).  Requires K % 256 == 0, group 32 or 16, bf16 or fp16 x (any M >= 1:
 * groups of 16, which have no decode-shape kernel of their own, are best sent here at every batch size).
 * `workspace` (256-byte aligned, size from ojx_e8t_gemm_workspace_bytes) holds a status block and,
 * for bf16 activations, one power-of-two factor per token row and the fp16 copy of the activations
 * scaled by it (each row's largest magnitude is brought into [2^14, 2^15); the row's outputs are
 * scaled back): the tensor cores need both operands in one 16-bit format and the weights are only
 * exact in fp16.  Calls that share a workspace must not overlap on the GPU.
 * ojx_e8t_gemm_status reads back (synchronising the stream) whether any bounded wait inside the
 * last gemm on that workspace expired.
 */
size_t  ojx_e8t_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K);
int32_t ojx_e8t_gemm(const void* x, int32_t x_dtype, int64_t M,
                     const uint8_t* packed, const uint16_t* scales, const void* bias,
                     int64_t N, int64_t K, int32_t group,
                     void* y, int32_t y_dtype,
                     void* workspace, size_t workspace_bytes, void* stream);
int32_t ojx_e8t_gemm_status(const void* workspace, void* stream);

/*
 * The same prefill kernel for the two sibling formats (`bits` 2 or 1; group 8, 16 or 32, K % 256 == 0, 16-bit activations,
 * workspace and status exactly as for ojx_e8t_gemm): the decoder warps read the 2-bit / 1-bit codes instead of the
 * ternary ranks.  Replaces the 2.0-bit / 1.0-bit branches of _FusedE8GEMMFunction.forward
 * (ojasx2/math/lattice.py:596-624) for batches of tokens.  The weights enter the tensor cores as fp16: for 1 bit
 * coordinate * scale is exact; for 2 bits (code - 1.5) * scale is rounded to fp16 once, i.e. the product equals
 * x . decode_2bit(fp16)^T with fp32 accumulation.
 */
int32_t ojx_e8t_gemm_lowbit(int32_t bits, const void* x, int32_t x_dtype, int64_t M,
                            const uint8_t* packed, const uint16_t* scales, const void* bias,
                            int64_t N, int64_t K, int32_t group,
                            void* y, int32_t y_dtype,
                            void* workspace, size_t workspace_bytes, void* stream);

/*
 * Backward of the packed linear with respect to its input: dX[M, K] = dY[M, N] . W[N, K], W given packed, on the
 * same tcgen05 pipeline (the contraction runs over the weight rows; the decoded weights enter the MMAs as an
 * MN-major operand, so no dense or transposed copy of W ever exists).  Replaces the decode-then-matmul of
 * _FusedE8GEMMFunction.backward (ojasx2/math/lattice.py:642-717) and the reference's native
 * fused_ternary_e8_gemm_backward_dx (ojasx2/math/csrc/ojasx_math_core.hpp:641-702, schema
 * ojasx_math_bindings.cpp:594).  Requires K % 256 == 0, N % 8 == 0, group 32 or 16, bf16 or fp16 dY; fp32 accumulation;
 * workspace as for ojx_e8t_gemm (size from ojx_e8t_gemm_dx_workspace_bytes; ojx_e8t_gemm_status reports on it).
 */
size_t  ojx_e8t_gemm_dx_workspace_bytes(int64_t M, int64_t N, int64_t K);
int32_t ojx_e8t_gemm_dx(const void* grad_y, int32_t gy_dtype, int64_t M,
                        const uint8_t* packed, const uint16_t* scales,
                        int64_t N, int64_t K, int32_t group,
                        void* dx, int32_t dx_dtype,
                        void* workspace, size_t workspace_bytes, void* stream);
/* The same for the 2.0-bit and 1.0-bit formats (`bits` 2 or 1; the weights enter as fp16 exactly as in
 * ojx_e8t_gemm_lowbit): dX = dY . decode(fp16 W). */
int32_t ojx_e8t_gemm_dx_lowbit(int32_t bits, const void* grad_y, int32_t gy_dtype, int64_t M,
                               const uint8_t* packed, const uint16_t* scales,
                               int64_t N, int64_t K, int32_t group,
                               void* dx, int32_t dx_dtype,
                               void* workspace, size_t workspace_bytes, void* stream);

/*
 * Seeded synthetic data, generated on the device: element i of stream `seed` is a sum of twelve
 * 24-bit uniforms from splitmix64, scaled to ~N(0, sigma), then rounded to `dtype`.  Integer-exact,
 * so host and device produce identical bits.  Used by the benchmark to fill 70B-shaped weights
 * without a host copy.  No counterpart in the reference.
 */
int32_t ojx_e8t_generate(void* out, int32_t dtype, int64_t count, uint64_t seed, int64_t start,
                         float sigma, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* OJX_E8T_H */
