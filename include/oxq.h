/*
 * oxq.h -- C ABI of liboxq_b200.so: hand-written sm_100a kernels for the OxiCUDA quantized-inference
 * path (oxicuda-quant quantize/dequantize kernels and the oxicuda-blas low-precision GEMMs).
 *
 * The reference is a Rust workspace with no FFI boundary of its own on this path: its two public
 * surfaces are ordinary Rust APIs.  Each entry point below names the reference interface it stands
 * behind (paths relative to the reference workspace root).  A Rust shim binds these symbols with
 * `extern "C"` declarations and keeps the reference's type names on top.
 *
 * Conventions
 *   - Every pointer named *_dev or documented "device" is a device pointer owned by the caller
 *     (reference: MatrixDesc borrows a CUdeviceptr, crates/oxicuda-blas/src/types.rs:443-455).
 *   - Every call is asynchronous on the handle's stream and performs no host synchronisation
 *     (reference: dispatch() launches and returns, crates/oxicuda-blas/src/level3/gemm/dispatch.rs:198-203).
 *   - No call allocates device memory.  Kernels that need scratch take a caller-provided workspace.
 *   - A handle is not thread-safe: one per host thread, exactly the BlasHandle rule
 *     (crates/oxicuda-blas/src/handle.rs:37-40).
 *   - There is no CPU fallback: on a machine without an sm_100 device every launch returns an error.
 *   - Matrices are row-major.  GEMMs compute Y[M x N] = X[M x K] * W[N x K]^T with K contiguous in
 *     both operands (the weight layout of ColumnLinearShard,
 *     crates/oxicuda-dist-infer/src/tensor_parallel/column_parallel.rs:77-95).
 *
 * Status codes: 0 = OK; 1..9 mirror QuantError (crates/oxicuda-quant/src/error.rs:10-58);
 * 10..19 mirror BlasError (crates/oxicuda-blas/src/error.rs:16-59); 100 = a bounded device-side
 * wait expired; 1000 + n = cudaError_t n; 2000 + n = ncclResult_t n.
 */
#ifndef OXQ_H_
#define OXQ_H_

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define OXQ_API __attribute__((visibility("default")))
#else
#define OXQ_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef struct oxq_handle oxq_handle;

enum {
    OXQ_OK = 0,
    /* QuantError */
    OXQ_ERR_EMPTY_INPUT = 1,
    OXQ_ERR_GROUP_SIZE_MISMATCH = 2,
    OXQ_ERR_INVALID_SCALE = 3,
    OXQ_ERR_QUANT_DIMENSION_MISMATCH = 4,
    OXQ_ERR_NON_FINITE_FP8 = 5,
    OXQ_ERR_INVALID_BIT_WIDTH = 6,
    OXQ_ERR_SINGULAR_HESSIAN = 7,      /* QuantError::SingularHessian; raised by host wrappers that read `info` of oxq_gptq_quantize_layer */
    /* BlasError */
    OXQ_ERR_INVALID_DIMENSION = 10,
    OXQ_ERR_BUFFER_TOO_SMALL = 11,
    OXQ_ERR_DIMENSION_MISMATCH = 12,
    OXQ_ERR_UNSUPPORTED_OPERATION = 13,
    OXQ_ERR_LAUNCH_FAILED = 14,
    OXQ_ERR_INVALID_ARGUMENT = 15,
    /* device side */
    OXQ_ERR_DEVICE_TIMEOUT = 100,
    OXQ_ERR_CUDA_BASE = 1000,
    OXQ_ERR_NCCL_BASE = 2000           /* 2000 + n = ncclResult_t n */
};

/* element types of floating-point tensors handed to the quantizers */
enum { OXQ_F32 = 0, OXQ_BF16 = 1, OXQ_F16 = 2 };
/* integer rounding of x/scale: HALF_EVEN is cvt.rni (crates/oxicuda-quant/src/ptx_kernels.rs:166-172),
 * HALF_AWAY is f32::round as used by MinMaxQuantizer (crates/oxicuda-quant/src/scheme/minmax.rs:263). */
enum { OXQ_ROUND_HALF_EVEN = 0, OXQ_ROUND_HALF_AWAY = 1 };
/* FP8 conversion: SPEC_RNE = round-to-nearest-even, saturating (cvt.rn.satfinite.e4m3x2.f32, the
 * conversion the reference's PTX builder documents, crates/oxicuda-ptx/src/builder/body_builder/mod.rs:1309-1323);
 * REFCOMPAT = the literal bit manipulation of Fp8Codec (crates/oxicuda-quant/src/scheme/fp8.rs:163-208). */
enum { OXQ_FP8_SPEC_RNE = 0, OXQ_FP8_REFCOMPAT = 1 };

/* ---- handle: stands in for BlasHandle (crates/oxicuda-blas/src/handle.rs:41-52) ---------------- */
OXQ_API int32_t oxq_handle_create(int device, void* cuda_stream, oxq_handle** out);
OXQ_API int32_t oxq_handle_destroy(oxq_handle* h);
OXQ_API int32_t oxq_set_stream(oxq_handle* h, void* cuda_stream);          /* BlasHandle::set_stream, handle.rs:134-154 */
OXQ_API const char* oxq_last_error_string(const oxq_handle* h);
OXQ_API const char* oxq_status_name(int32_t status);
OXQ_API int32_t oxq_version(void);
/* Reads and clears the device-side status word that bounded waits write (0 = none).  Synchronises the stream. */
OXQ_API int32_t oxq_device_status(oxq_handle* h, int32_t* status_out);

/* ---- INT8 symmetric per-row: MinMaxQuantizer::calibrate_2d + quantize_grouped(group = cols)
 *      (crates/oxicuda-quant/src/scheme/minmax.rs:179-207, :275-299); device API shape of
 *      quantize_to_int8 (crates/oxicuda-dnn/src/quantize/int8_quantize.rs:33-92).
 *      scale[r] = max(absmax_row, 1e-8)/127; q = clamp(round(x/scale), -127, 127). ------------------ */
OXQ_API int32_t oxq_int8_quant_rows(oxq_handle* h, const float* x_dev, int64_t rows, int64_t cols,
                            int8_t* q_dev, float* scales_dev, int rounding);
/* MinMaxQuantizer::dequantize_grouped (minmax.rs:309-324): y = q * scale[row]. */
OXQ_API int32_t oxq_int8_dequant_rows(oxq_handle* h, const int8_t* q_dev, const float* scales_dev,
                              int64_t rows, int64_t cols, float* y_dev);

/* ---- FP8 E4M3 per tensor: Fp8Codec::encode / decode (crates/oxicuda-quant/src/scheme/fp8.rs:115-142)
 *      with the per-tensor absmax/448 scaling of quantize_to_fp8
 *      (crates/oxicuda-dnn/src/quantize/fp8_quantize.rs:47-111). ------------------------------------- */
/* absmax_dev[0] = max |x| (NaNs skipped).  One pass over x. */
OXQ_API int32_t oxq_absmax(oxq_handle* h, const void* x_dev, int x_dtype, int64_t n, float* absmax_dev);
/* q = e4m3(x / *scale_dev). */
OXQ_API int32_t oxq_fp8_quant(oxq_handle* h, const void* x_dev, int x_dtype, int64_t n, const float* scale_dev,
                      uint8_t* q_dev, int fp8_mode);
/* absmax pass + quantize pass; stats_dev[0] = absmax, stats_dev[1] = scale = absmax/448 (1.0 if absmax == 0). */
OXQ_API int32_t oxq_fp8_quant_dynamic(oxq_handle* h, const void* x_dev, int x_dtype, int64_t n, uint8_t* q_dev,
                              float* stats_dev);
/* y = decode(q) * *scale_dev. */
OXQ_API int32_t oxq_fp8_dequant(oxq_handle* h, const uint8_t* q_dev, int64_t n, const float* scale_dev,
                        void* y_dev, int y_dtype, int fp8_mode);

/* ---- uint4 group-wise asymmetric: MinMaxQuantizer::int4_per_group / calibrate(PerGroup, Asymmetric)
 *      (minmax.rs:146-167, :226-232) + pack_int4 bit positions (crates/oxicuda-blas/src/precision/int_ops.rs:375-399);
 *      device API shape of quantize_to_int4 (crates/oxicuda-dnn/src/quantize/int4_quantize.rs:132-218).
 *      Groups run along k; scales are f16 [rows x k/group]; zero-points are packed 8 per u32 in
 *      linear group order; codes 8 per u32, element j at bits [4j, 4j+4). ---------------------------- */
OXQ_API int32_t oxq_int4g_quant_pack(oxq_handle* h, const void* x_dev, int x_dtype, int64_t rows, int64_t k, int group,
                             uint32_t* codes_dev, uint16_t* scales_f16_dev, uint32_t* zeros_packed_dev, int rounding);
OXQ_API int32_t oxq_int4g_dequant(oxq_handle* h, const uint32_t* codes_dev, const uint16_t* scales_f16_dev,
                          const uint32_t* zeros_packed_dev, int64_t rows, int64_t k, int group,
                          void* y_dev, int y_dtype);

/* The same quantizer in MinMaxQuantizer's own parameter types -- f32 scales and i32 zero-points per group
 * (QuantParams, minmax.rs:50-60) -- so that a caller holding reference results can compare value for value:
 *   scale = max(max - min, 1e-8) / 15, zp = clamp(round(-min / scale), 0, 15)            (minmax.rs:226-232)
 *   q = clamp(round(x / scale + zp), 0, 15), packed 8 per u32 like pack_int4              (minmax.rs:275-299)
 *   y = (q - zp) as f32 * scale                                                            (minmax.rs:302-324)
 * x is f32 [rows x k].  A group that holds an infinity gets a non-finite scale where the reference returns
 * QuantError::InvalidScale; the call is asynchronous, so it is the host wrapper that looks at the scales. */
OXQ_API int32_t oxq_int4g_quant_pack_f32(oxq_handle* h, const float* x_dev, int64_t rows, int64_t k, int group, uint32_t* codes_dev,
                                 float* scales_dev, int32_t* zero_points_dev, int rounding);
OXQ_API int32_t oxq_int4g_dequant_f32(oxq_handle* h, const uint32_t* codes_dev, const float* scales_dev, const int32_t* zero_points_dev,
                              int64_t rows, int64_t k, int group, float* y_dev);

/* ---- MicroScalingQuantizer::quantize_fp4 / dequantize_fp4 as the reference defines them
 *      (crates/oxicuda-blas/src/precision/fp4_fp6_ops.rs:763-782, :849-897): an f32 scale max|x| / 6 per block of
 *      32, 64 or 128 elements (1 for an all-zero block, the last block may be short), codes from the floor-type
 *      E2M1 encoder Fp4Quantizer::quantize_one (:645-661) applied to x / scale, two per byte with the even element
 *      in the low nibble (PackedFp4::pack, :465-472).  packed_dev holds ceil(n / 2) bytes, scales_dev ceil(n / block)
 *      floats.  n == 0 returns OXQ_OK. ------------------------------------------------------------------ */
OXQ_API int32_t oxq_fp4_microscale_quant(oxq_handle* h, const float* x_dev, int64_t n, int64_t block, uint8_t* packed_dev, float* scales_dev);
OXQ_API int32_t oxq_fp4_microscale_dequant(oxq_handle* h, const uint8_t* packed_dev, const float* scales_dev, int64_t n, int64_t block,
                                   float* y_dev);

/* ---- block-scaled formats: MicroScalingQuantizer::quantize_fp4 and Fp4GemmConfig
 *      (crates/oxicuda-blas/src/precision/fp4_fp6_ops.rs:337-395, :746-898) re-defined on the OCP MX / NVFP4
 *      formats the benchmark configurations name.  Scale factors are written twice: row-major
 *      [rows x k/block], and (if sf_mma_dev != NULL) in the 128-row x 4-column tiled order the
 *      tensor-core scale-factor loads consume; oxq_sf_mma_bytes gives the size of the latter. -------- */
OXQ_API size_t oxq_sf_mma_bytes(int64_t rows, int64_t sf_cols);
OXQ_API int32_t oxq_mxfp8_quant(oxq_handle* h, const void* x_dev, int x_dtype, int64_t rows, int64_t k,
                        uint8_t* codes_dev, uint8_t* sf_rowmajor_dev, uint8_t* sf_mma_dev);
OXQ_API int32_t oxq_mxfp8_dequant(oxq_handle* h, const uint8_t* codes_dev, const uint8_t* sf_rowmajor_dev,
                          int64_t rows, int64_t k, void* y_dev, int y_dtype);
/* stats_dev[0] = absmax (input, from oxq_absmax), stats_dev[1] = global scale g (output). */
OXQ_API int32_t oxq_nvfp4_quant(oxq_handle* h, const void* x_dev, int x_dtype, int64_t rows, int64_t k,
                        float* stats_dev, uint8_t* packed_dev, uint8_t* sf_rowmajor_dev, uint8_t* sf_mma_dev);
OXQ_API int32_t oxq_nvfp4_dequant(oxq_handle* h, const uint8_t* packed_dev, const uint8_t* sf_rowmajor_dev,
                          const float* stats_dev, int64_t rows, int64_t k, void* y_dev, int y_dtype);

/* ---- SwiGLU on an interleaved gate/up product: h = silu(gate) * up (crates/oxicuda-lm/src/layer/ffn.rs:25-27, :245-249).
 *      gu_dev is [m x 2n] bf16 in blocks of 128 gate columns followed by the 128 matching up columns; n % 128 == 0. */
OXQ_API int32_t oxq_swiglu_interleaved(oxq_handle* h, const void* gu_bf16_dev, int64_t m, int64_t n, void* h_bf16_dev);

/* ---- GEMMs: stand behind gemm<T> (crates/oxicuda-blas/src/level3/gemm_api.rs:73-138) for the element
 *      types that entry point cannot run in the reference, and behind the low-precision configs of
 *      crates/oxicuda-blas/src/precision/{int_ops,fp8_ops,fp4_fp6_ops}.rs.
 *      Zero dimensions are errors (gemm_api.rs:88-92).  Outputs are bf16 unless noted.
 *      Kernel choice is internal: large M runs tcgen05 kernels with TMA-fed operands and accumulators in tensor
 *      memory; oxq_gemm_fp8, oxq_gemm_fp8_swiglu, oxq_gemm_w8a8, oxq_gemm_mxfp8 and oxq_gemm_nvfp4 with m <= 32 run a
 *      weight-streaming tensor-core kernel (the weight is the 128-row operand of the MMA, the batch its narrow side),
 *      the decode entry points (oxq_gemm_w4a16 with m <= 8, oxq_gemm_w8a32, oxq_gemm_nf4) mma.sync streams.  Operands may be
 *      produced by the call just before on the same stream (a quantizer followed directly by the GEMM): no kernel
 *      reads an operand before its producer has finished. ---------------- */
/* FP8 E4M3: Y = bf16((X . W^T) * (*sx_dev * *sw_dev)), f32 accumulate.  K % 16 == 0, ldy % 8 == 0. */
OXQ_API int32_t oxq_gemm_fp8(oxq_handle* h, int64_t m, int64_t n, int64_t k, const uint8_t* x_dev, int64_t ldx,
                     const uint8_t* w_dev, int64_t ldw, const float* sx_dev, const float* sw_dev,
                     void* y_bf16_dev, int64_t ldy);
/* The same FP8 GEMM with the SwiGLU of SwiGluFfn::forward (crates/oxicuda-lm/src/layer/ffn.rs:235-254) fused into
 * its epilogue.  w_gu_dev holds the gate and up projection weights interleaved in blocks of 128 rows
 * ([gate rows 0..127][up rows 0..127][gate rows 128..255]...), n2 = 2 * intermediate rows in total (multiple of 256);
 * H[m x n2/2] = bf16(silu(g) * u) with g, u = the scaled gate / up products. */
/* gemm's general form (crates/oxicuda-blas/src/level3/gemm_api.rs:73-82: C = alpha * op(A) * op(B) + beta * C) for the operand
 * layout of this library (X row-major [M x K], W row-major [N x K], i.e. op(B) = W^T): Y = alpha * (X . W^T) * sx * sw + beta * Y,
 * one rounding to bf16.  With beta == 0 the old contents of Y are not read (NaNs there do not propagate), as in BLAS. */
OXQ_API int32_t oxq_gemm_fp8_ex(oxq_handle* h, int64_t m, int64_t n, int64_t k, float alpha, const uint8_t* x_dev, int64_t ldx,
                        const uint8_t* w_dev, int64_t ldw, const float* sx_dev, const float* sw_dev, float beta, void* y_bf16_dev, int64_t ldy);
OXQ_API int32_t oxq_gemm_bf16_ex(oxq_handle* h, int64_t m, int64_t n, int64_t k, float alpha, const void* x_bf16_dev, int64_t ldx,
                         const void* w_bf16_dev, int64_t ldw, float beta, void* y_bf16_dev, int64_t ldy);
/* gemm's operand forms (trans_a, trans_b and MatrixDesc.layout, gemm_api.rs:73-82, types.rs:60-90, :443-455).  C = alpha * op(A) * op(B)
 * + beta * C with op(A) [m x k] and op(B) [k x n]; what matters to the kernel is which index is contiguous in memory:
 *   a_major  OXQ_OP_K_MAJOR   A is stored [m x lda], k contiguous   (NoTrans + RowMajor, or Trans + ColMajor)
 *            OXQ_OP_MN_MAJOR  A is stored [k x lda], m contiguous   (Trans + RowMajor, or NoTrans + ColMajor)
 *   b_major  OXQ_OP_K_MAJOR   B is stored [n x ldb], k contiguous   (Trans + RowMajor, or NoTrans + ColMajor): the weight layout W[N x K]
 *            OXQ_OP_MN_MAJOR  B is stored [k x ldb], n contiguous   (NoTrans + RowMajor: the reference's default call)
 * so a reference caller's gemm(NoTrans, NoTrans, ...) on row-major matrices is (K_MAJOR, MN_MAJOR) and needs no transposed copy.
 * The output is row-major [m x ldy] bf16; a column-major C is the row-major C^T = op(B)^T * op(A)^T, i.e. the same call with the
 * operands exchanged and their flags flipped (the host mirror does that).  MN-major tiles go through the shared-memory descriptor
 * and the major bits of the tcgen05 instruction descriptor.  Leading dimensions are multiples of 16 bytes; k is a multiple of
 * 16 bytes' worth of elements when an operand is K-major.  Errors: InvalidDimension (zero sizes, a leading dimension smaller
 * than the contiguous extent), InvalidArgument (alignment, unknown flag). */
enum { OXQ_OP_K_MAJOR = 0, OXQ_OP_MN_MAJOR = 1 };
OXQ_API int32_t oxq_gemm_fp8_op(oxq_handle* h, int64_t m, int64_t n, int64_t k, float alpha, const uint8_t* a_dev, int64_t lda, int a_major,
                        const uint8_t* b_dev, int64_t ldb, int b_major, const float* sa_dev, const float* sb_dev, float beta,
                        void* y_bf16_dev, int64_t ldy);
OXQ_API int32_t oxq_gemm_bf16_op(oxq_handle* h, int64_t m, int64_t n, int64_t k, float alpha, const void* a_bf16_dev, int64_t lda, int a_major,
                         const void* b_bf16_dev, int64_t ldb, int b_major, float beta, void* y_bf16_dev, int64_t ldy);
OXQ_API int32_t oxq_gemm_fp8_swiglu(oxq_handle* h, int64_t m, int64_t n2, int64_t k, const uint8_t* x_dev, int64_t ldx,
                            const uint8_t* w_gu_dev, int64_t ldw, const float* sx_dev, const float* sw_dev,
                            void* h_bf16_dev, int64_t ldh);
/* bf16 GEMM behind gemm<bf16> (gemm_api.rs:73-138; alpha = 1, beta = 0, op(B) = W^T): the consumer of weights
 * dequantised to bf16 (W4A16 at prefill shapes) and its SwiGLU-fused form.  K % 8 == 0. */
OXQ_API int32_t oxq_gemm_bf16(oxq_handle* h, int64_t m, int64_t n, int64_t k, const void* x_bf16_dev, int64_t ldx,
                      const void* w_bf16_dev, int64_t ldw, void* y_bf16_dev, int64_t ldy);
OXQ_API int32_t oxq_gemm_bf16_swiglu(oxq_handle* h, int64_t m, int64_t n2, int64_t k, const void* x_bf16_dev, int64_t ldx,
                             const void* w_gu_bf16_dev, int64_t ldw, void* h_bf16_dev, int64_t ldh);
/* W8A8 (Int8GemmConfig, int_ops.rs:79-189): Y = bf16(s32(X . W^T) * sx_rows[m] * sw_rows[n]). */
OXQ_API int32_t oxq_gemm_w8a8(oxq_handle* h, int64_t m, int64_t n, int64_t k, const int8_t* x_dev, int64_t ldx,
                      const int8_t* w_dev, int64_t ldw, const float* sx_rows_dev, const float* sw_rows_dev,
                      void* y_bf16_dev, int64_t ldy);
/* W8A32 decode GEMM of benchmark configuration 1: Y_f32 = X_f32 . (W_i8 * sw_rows)^T, f32 accumulate. */
OXQ_API int32_t oxq_gemm_w8a32(oxq_handle* h, int64_t m, int64_t n, int64_t k, const float* x_dev,
                       const int8_t* w_dev, const float* sw_rows_dev, float* y_dev);
/* W4A16 weight-only (Int4GemmConfig, int_ops.rs:215-355; quantized operand is the weight):
 * Y = bf16(X_bf16 . dequant(W)^T).  Three regimes, all reading the packed weight once per 32 batch rows or less:
 *   m <= 8           HBM-bound mma.sync kernel, one CTA per 16 weight rows over the whole K (no workspace traffic);
 *   9 <= m <= 64     (group 128, k % 1024 == 0) tensor-core kernel with the dequantisation fused in: codes are
 *                    unpacked straight into tensor memory as the row operand of tcgen05.mma, per-group scales are
 *                    applied to the group's accumulator, partial K ranges are combined in the workspace; one pass
 *                    over the weight for up to 16, 32 or 64 batch rows;
 *                    other shapes with m <= 32 use a split-K mma.sync kernel (partial sums in the workspace);
 *   otherwise        the weight is dequantised to bf16 in the workspace and the bf16 tensor-core GEMM runs
 *                    (n % 8 == 0).
 * Workspace: oxq_gemm_w4a16_workspace_bytes(m, n, k) bytes, 256-byte aligned.  Its first
 * oxq_gemm_w4a16_workspace_bytes(min(m, 32), n, k) bytes hold the partial sums of the decode kernels: they must be
 * zero before a call with m <= 32 and every call, whatever its m, leaves them zero (a call with m > 32 keeps its
 * dequantised weight behind that region and clears what it uses itself), so one workspace sized for the largest m
 * serves prefill and decode calls in any order. */
OXQ_API size_t oxq_gemm_w4a16_workspace_bytes(int64_t m, int64_t n, int64_t k);
OXQ_API int32_t oxq_gemm_w4a16(oxq_handle* h, int64_t m, int64_t n, int64_t k, const void* x_bf16_dev,
                       const uint32_t* codes_dev, const uint16_t* scales_f16_dev, const uint32_t* zeros_packed_dev,
                       int group, void* y_bf16_dev, void* workspace_dev, size_t workspace_bytes);
/* Same product as oxq_gemm_w4a16 for callers that cannot allocate device memory at all: code that
 * runs where cudaMalloc is off limits (inside a framework's caching-allocator region, under a memory
 * budget enforced by someone else, in a plugin whose host forbids allocations after start-up) and so
 * can neither create an oxq_handle nor provide a workspace.  It has no counterpart in the reference.
 * It takes the stream directly, works on the current device, and keeps its split-K partial sums in an
 * array built into the library image (2 MiB + 32 KiB per GPU that loads the library, held until the
 * process exits).  Limit: m <= 32 and m * n <= 524288 outputs; larger shapes return
 * OXQ_ERR_BUFFER_TOO_SMALL.  The first call on each device looks up the array's device address and
 * reads three device attributes; make that first call before any stream capture begins.  Every call
 * clears the part of the array it uses and all calls share the one array, so two calls that overlap
 * on the GPU (different streams, no ordering between them) race and give wrong sums.  The first call
 * on a device also fills a small per-device record on the host without a lock: let one host thread
 * make that first call before other threads use the entry point on the same device. */
OXQ_API int32_t oxq_gemm_w4a16_static(void* cuda_stream, int64_t m, int64_t n, int64_t k, const void* x_bf16_dev,
                              const uint32_t* codes_dev, const uint16_t* scales_f16_dev, const uint32_t* zeros_packed_dev,
                              int group, void* y_bf16_dev);
/* ---- quantizers next to the hot path --------------------------------------------------------------------
 * Per-tensor INT8 with the arithmetic of oxicuda-dnn's quantize_to_int8 / dequantize_from_int8
 * (crates/oxicuda-dnn/src/quantize/int8_quantize.rs:33-92, :101-157): scale_dev[0] = max(absmax / 127, 1e-12),
 * q = rint(clamp(x / scale, -127, 127)) (half to even); y = (float)q * scale_dev[0].  n == 0 returns OXQ_OK. */
OXQ_API int32_t oxq_int8_quant_tensor(oxq_handle* h, const void* x_dev, int dtype, int64_t n, int8_t* q_dev, float* scale_dev);
OXQ_API int32_t oxq_int8_dequant_tensor(oxq_handle* h, const int8_t* q_dev, const float* scale_dev, int64_t n, void* y_dev, int y_dtype);
/* BlockQuantizedInt8::quantize / dequantize (int8_quantize.rs:404-451) on device buffers: one scale per `block`
 * contiguous elements (the last block may be short), scale = max|x| / 127 or 1 for an all-zero block,
 * q = clamp(round_half_away(x / scale), -128, 127).  scales_dev holds ceil(n / block) floats. */
OXQ_API int32_t oxq_int8_block_quant(oxq_handle* h, const float* x_dev, int64_t n, int64_t block, int8_t* q_dev, float* scales_dev);
OXQ_API int32_t oxq_int8_block_dequant(oxq_handle* h, const int8_t* q_dev, const float* scales_dev, int64_t n, int64_t block, float* y_dev);
/* quantize_to_int4 / dequantize_int4 of the DNN layer (crates/oxicuda-dnn/src/quantize/int4_quantize.rs:132-218, :229-300)
 * with the arithmetic of its generated kernels: groups of group_size contiguous elements (the last may be short);
 * symmetric: scale = max(absmax, 1e-12) / 7, q = trunc(clamp(x / scale, -8, 7) + 8), y = (q - 8) * scale;
 * asymmetric: scale = max(max - min, 1e-12) / 15, zeros = -min / scale (a float, written but not used by the codes),
 * q = trunc(clamp(x / scale, 0, 15)), y = q * scale.  Two codes per byte, even element in the low nibble; packed_dev
 * holds ceil(n / 2) bytes, scales_dev and zeros_dev ceil(n / group_size) floats (zeros_dev may be NULL when symmetric).
 * n == 0 returns OXQ_OK. */
OXQ_API int32_t oxq_dnn_int4_quant(oxq_handle* h, const float* x_dev, int64_t n, int64_t group_size, int symmetric, uint8_t* packed_dev,
                           float* scales_dev, float* zeros_dev);
OXQ_API int32_t oxq_dnn_int4_dequant(oxq_handle* h, const uint8_t* packed_dev, const float* scales_dev, int64_t n, int64_t group_size,
                             int symmetric, float* y_dev);
/* quantize_block_scaled of the DNN layer (crates/oxicuda-dnn/src/quantize/block_scale.rs:53-140): per block of block_size
 * elements (a power of two, at least 16; the last block may be short) scale = max(absmax / 6, 1e-12),
 * out = clamp(int(rint(clamp(x / scale, -6, 6))) + 6, 0, 255) as one byte per element. */
OXQ_API int32_t oxq_dnn_block_scaled_quant(oxq_handle* h, const void* x_dev, int dtype, int64_t n, int64_t block_size, uint8_t* out_dev,
                                   float* scales_dev);
/* The fused dequantise + GEMV of the DNN layer's weight-only plan (dnn_fused_dequant_gemv_f32 of
 * WeightQuantPlan::generate_fused_dequant_gemv_ptx, crates/oxicuda-dnn/src/quantize/gptq_awq.rs:867-994):
 *   y[row] = sum over col of (code[row, col] * scale[row, col / group_size]) * x[col],   f32 throughout,
 * codes unsigned, `bits` wide, packed LSB-first in u32 words (element `sub` of a word at bit sub * bits, :936-945),
 * packed_w_dev [rows x cols * bits / 32] words, scales_dev [rows x cols / group_size] f32, no zero-point (the reference's
 * kernel takes a zero pointer and does not read it).  One pass over the packed weight.  The reference adds the products
 * of a row one after the other; here they are summed by lanes and shuffles, so results agree to f32 summation error.
 * bits in {2, 4, 8}; cols a multiple of four packed words (128 / bits columns) and of group_size; group_size a multiple of
 * 32 / bits; packed_w_dev and x_dev 16-byte aligned. */
OXQ_API int32_t oxq_dnn_fused_dequant_gemv(oxq_handle* h, const uint32_t* packed_w_dev, const float* scales_dev, const float* x_dev, float* y_dev,
                                   int64_t rows, int64_t cols, int64_t group_size, int bits);
/* Nf4Quantizer::encode / decode (crates/oxicuda-quant/src/scheme/nf4.rs:93-155): per block absmax (floored at
 * 1e-8), x / absmax clamped to [-1, 1], nearest of the 16 NormalFloat4 levels (the lower index on a tie), two
 * codes per byte with the even element in the low nibble.  packed_dev holds n / 2 bytes, absmax_dev n / block
 * floats.  Errors as the reference: EmptyInput, GroupSizeMismatch (encode), DimensionMismatch (decode). */
/* The 15 decision thresholds of the NF4 encoder (host call, no device work): out15[i] is the largest f32 whose nearest
 * level under the reference's f32 comparison (nf4.rs:186-205) is i; the encoder's code is the number of thresholds below x. */
OXQ_API int32_t oxq_nf4_thresholds(float* out15);
OXQ_API int32_t oxq_nf4_quant(oxq_handle* h, const float* x_dev, int64_t n, int64_t block, uint8_t* packed_dev, float* absmax_dev);
OXQ_API int32_t oxq_nf4_dequant(oxq_handle* h, const uint8_t* packed_dev, const float* absmax_dev, int64_t n, int64_t block,
                                void* y_dev, int y_dtype);
/* Decode-shaped GEMM on NF4 weights, dequantisation fused in: Y[m x n] (bf16) = X[m x k] (bf16) . W^T with
 * W[r][c] = level[code] * absmax[(r * k + c) / block], the tensors of oxq_nf4_quant on a row-major [n x k] weight.  The
 * reference has the elementwise nf4_dequant kernel only (crates/oxicuda-quant/src/ptx_kernels.rs:261-396); this replaces
 * dequantise + GEMV by one pass over the packed bytes.  m <= 8; block a multiple of 64 that divides k.  The levels enter
 * the tensor core rounded to bf16; accumulation is f32. */
OXQ_API int32_t oxq_gemm_nf4(oxq_handle* h, int64_t m, int64_t n, int64_t k, const void* x_bf16_dev, const uint8_t* packed_dev,
                             const float* absmax_dev, int64_t block, void* y_bf16_dev);
/* RmsNorm::forward (crates/oxicuda-lm/src/layer/norm.rs:73-95; y = x / sqrt(mean(x^2) + eps) * weight) fused with the per-row
 * symmetric INT8 quantizer of oxq_int8_quant_rows (half to even): the activation path in front of oxq_gemm_w8a8, one pass over
 * the row.  cols % 8 == 0, cols <= 16384.  y_opt (same dtype as x) also receives the normalised row when it is not NULL. */
OXQ_API int32_t oxq_rmsnorm_int8_quant_rows(oxq_handle* h, const void* x_dev, int dtype, const float* weight_dev, int64_t rows, int64_t cols,
                                            float eps, int8_t* q_dev, float* scales_dev, void* y_opt_dev);
/* The FP8 forms of the fused activation paths, at a calibrated per-tensor scale (scale_dev[0], as oxq_fp8_quant takes it):
 *   oxq_rmsnorm_fp8_quant_rows  RmsNorm::forward (norm.rs:73-95) then E4M3 (RNE, saturating) of y / scale: the input of oxq_gemm_fp8;
 *   oxq_silu_gate_fp8_quant     silu_gate (crates/oxicuda-lm/src/ptx_kernels.rs:222-290, out = gate / (1 + exp(-gate)) * up,
 *                               SwiGluFfn::forward at crates/oxicuda-lm/src/layer/ffn.rs:202-254) then E4M3 of out / scale: the
 *                               input of the down projection, written as one byte per element instead of a bf16 round trip.
 * x, gate and up share `dtype` (OXQ_F32 / OXQ_BF16 / OXQ_F16); the arithmetic is f32 before the one conversion. */
OXQ_API int32_t oxq_rmsnorm_fp8_quant_rows(oxq_handle* h, const void* x_dev, int dtype, const float* weight_dev, int64_t rows, int64_t cols,
                                           float eps, const float* scale_dev, uint8_t* q_dev);
OXQ_API int32_t oxq_silu_gate_fp8_quant(oxq_handle* h, const void* gate_dev, const void* up_dev, int dtype, int64_t n,
                                        const float* scale_dev, uint8_t* q_dev);
/* SmoothQuantMigrator (crates/oxicuda-quant/src/scheme/smooth_quant.rs) on device buffers, f32 row-major:
 *   oxq_smooth_col_absmax  compute_act_stats / compute_weight_stats (:125-196): stats[j] = max_r |x[r, j]|;
 *   oxq_smooth_scales      compute_migration_scales (:84-113): s_j = max(|a_j|,1e-8)^alpha / max(|w_j|,1e-8)^(1-alpha);
 *   oxq_smooth_apply       divide != 0: smooth_activations (:198-222), x[r, j] /= max(s_j, 1e-12);
 *                          divide == 0: smooth_weights (:231-254), x[r, j] *= s_j.  In place. */
OXQ_API int32_t oxq_smooth_col_absmax(oxq_handle* h, const float* x_dev, int64_t rows, int64_t cols, float* stats_dev);
OXQ_API int32_t oxq_smooth_scales(oxq_handle* h, const float* act_max_dev, const float* weight_max_dev, int64_t n, float alpha, float* scales_dev);
OXQ_API int32_t oxq_smooth_apply(oxq_handle* h, float* x_dev, int64_t rows, int64_t cols, const float* scales_dev, int divide);
/* y[m, n] += bias[n] on a bf16 matrix (the bias term of ColumnLinearShard::forward / RowLinearShard::forward_partial,
 * crates/oxicuda-dist-infer/src/tensor_parallel/column_parallel.rs:77-95, row_parallel.rs:67-90); n and ldy multiples of 8. */
OXQ_API int32_t oxq_bias_add_bf16(oxq_handle* h, void* y_bf16_dev, int64_t ldy, const float* bias_dev, int64_t m, int64_t n);
/* Block-scaled GEMMs (Fp4GemmConfig, fp4_fp6_ops.rs:337-395).  Scale factors in the tiled order. */
OXQ_API int32_t oxq_gemm_mxfp8(oxq_handle* h, int64_t m, int64_t n, int64_t k, const uint8_t* x_dev, const uint8_t* sfx_mma_dev,
                       const uint8_t* w_dev, const uint8_t* sfw_mma_dev, void* y_bf16_dev, int64_t ldy);
OXQ_API int32_t oxq_gemm_nvfp4(oxq_handle* h, int64_t m, int64_t n, int64_t k, const uint8_t* x_dev, const uint8_t* sfx_mma_dev,
                       const float* gx_dev, const uint8_t* w_dev, const uint8_t* sfw_mma_dev, const float* gw_dev,
                       void* y_bf16_dev, int64_t ldy);

/* ---- tensor-parallel combine: RowLinear::all_reduce (crates/oxicuda-dist-infer/src/tensor_parallel/row_parallel.rs:199-223),
 *      which sums the rank partials on the host, done in place over the NVSwitch multicast mapping of a symmetric
 *      bf16 buffer: this rank reduces elements [rank*numel/world, (rank+1)*numel/world) across all replicas (f32
 *      accumulation in the switch) and broadcasts the sums.  The caller provides the cross-rank barriers: every
 *      rank's partial must be complete before the call starts anywhere, and nobody may read the result before every
 *      rank's call has finished.  numel % (8 * world) == 0. */
OXQ_API int32_t oxq_multimem_all_reduce_bf16(oxq_handle* h, void* multicast_ptr, int64_t numel, int rank, int world);
/* The same over a column block of a row-major bf16 matrix ([rows x cols] at multicast_ptr, leading dimension ld elements):
 * rank r reduces rows [r * rows / world, (r + 1) * rows / world).  cols and ld multiples of 8, rows a multiple of world. */
OXQ_API int32_t oxq_multimem_all_reduce_bf16_2d(oxq_handle* h, void* multicast_ptr, int64_t rows, int64_t cols, int64_t ld, int rank, int world);
/* The same with the cross-rank synchronisation inside the kernel: no barrier before or after it.  The call is stream-ordered
 * behind the kernel that wrote this rank's partial; when it has finished on a rank, that rank's replica holds the complete
 * sums.  flags_*: this rank's replica and the multicast address of four 32-bit words of symmetric memory (16-byte aligned,
 * zero before the first call, never written by the host afterwards: the calls are counted on the device, so a CUDA graph
 * that holds such a call may be replayed).  Every rank makes the same sequence of calls on these words.  Waits on other
 * ranks are bounded (OXQ_ERR_DEVICE_TIMEOUT in the status word). */
OXQ_API int32_t oxq_multimem_all_reduce_bf16_2d_sync(oxq_handle* h, void* multicast_ptr, int64_t rows, int64_t cols, int64_t ld, int rank, int world,
                                             uint32_t* flags_local_dev, uint32_t* flags_multicast_dev);
/* ---- RowLinear::forward_partial + RowLinear::all_reduce in one kernel (crates/oxicuda-dist-infer/src/tensor_parallel/
 *      row_parallel.rs:67-90, :199-223): Y = sum over ranks of (X_r . W_r^T) * sx_r * sw_r, every rank's K-shard an FP8 GEMM as in
 *      oxq_gemm_fp8.  y_local_dev is this rank's replica of a symmetric bf16 buffer [m x ldy] and y_multicast_dev the same
 *      buffer through the NVSwitch multicast mapping; flags_* are this rank's replica and the multicast address of
 *      flag_words >= 2 * (ceil(m / 256) * ceil(n / 256) + 1) + 1 32-bit words of symmetric memory, zero before the first
 *      call and never written by the host afterwards (the last word counts the calls on the device, so a replayed CUDA
 *      graph behaves like a sequence of host calls; calls alternate between two sets of words).  Every rank of the group
 *      makes the same sequence of calls with the same shapes.  Tiles are reduced in the switch while
 *      later tiles are still being multiplied; when the call's kernel has finished on a rank, that rank's replica holds the
 *      complete sum (no barrier needed after it; the buffer may be rewritten by the next call).  Waits on other ranks are
 *      bounded (OXQ_ERR_DEVICE_TIMEOUT in the status word).  n % 8 == 0, 2 <= world <= 64. */
OXQ_API int32_t oxq_gemm_fp8_all_reduce(oxq_handle* h, int64_t m, int64_t n, int64_t k, const uint8_t* x_dev, int64_t ldx,
                                const uint8_t* w_dev, int64_t ldw, const float* sx_dev, const float* sw_dev, void* y_local_dev,
                                void* y_multicast_dev, int64_t ldy, uint32_t* flags_local_dev, uint32_t* flags_multicast_dev,
                                int64_t flag_words, int rank, int world);

/* ---- tensor-parallel layer behind the C ABI --------------------------------------------------------------------------
 * ColumnLinear / RowLinear / SwiGluFfn of the reference (crates/oxicuda-dist-infer/src/tensor_parallel/column_parallel.rs:103-204,
 * row_parallel.rs:97-223, crates/oxicuda-lm/src/layer/ffn.rs:202-254) hold f32 weights and add the ranks' partial sums on the
 * host.  Here every rank is one process with one GPU, holds its shard quantised, and the partial sums meet in one NCCL
 * all-reduce over NVLink.
 *   oxq_comm_unique_id  rank 0 makes the 128-byte identifier (ncclGetUniqueId) and hands it to the other ranks out of band
 *   oxq_comm_init       every rank joins with the same identifier (ncclCommInitRank on the handle's device); one communicator
 *                       per handle; the handle's stream carries the collectives
 *   oxq_comm_destroy    leaves the communicator (oxq_handle_destroy does it as well)
 * NCCL is bound at run time: the libnccl.so.2 the process already holds, else the one named by OXQ_NCCL_LIB, else the
 * loader's.  Without one, these calls return UnsupportedOperation; a handle without a communicator is a world of one rank. */
OXQ_API int32_t oxq_comm_unique_id(void* id_out_128);
OXQ_API int32_t oxq_comm_init(oxq_handle* h, const void* id_128, int nranks, int rank);
OXQ_API int32_t oxq_comm_destroy(oxq_handle* h);
OXQ_API int32_t oxq_comm_info(const oxq_handle* h, int* nranks_out, int* rank_out, int* nccl_version_out);
/* RowLinear::all_reduce (row_parallel.rs:199-223) and ColumnLinear::all_gather (column_parallel.rs:181-204) on device buffers,
 * asynchronous on the handle's stream.  The gather is rank-major: rank r's numel_local elements land at [r * numel_local, ...). */
OXQ_API int32_t oxq_all_reduce_bf16(oxq_handle* h, void* y_bf16_dev, int64_t numel);
OXQ_API int32_t oxq_all_gather_bf16(oxq_handle* h, const void* local_bf16_dev, int64_t numel_local, void* gathered_bf16_dev);
/* One rank's shard of the SwiGLU MLP.  inter_local = intermediate / nranks rows of the gate and of the up weight (interleaved in
 * blocks of 128 rows: [gate 0..127][up 0..127][gate 128..255]..., so w_gu is [2 * inter_local x hidden]) and the matching
 * inter_local input columns of the down weight ([hidden x inter_local]).
 *   OXQ_TP_FP8    w_gu / w_down are E4M3 bytes, w_gu_scales / w_down_scales one f32 each; the zeros are unused.  x is quantised
 *                 per tensor, h per shard (no maximum crosses ranks), both on the fly.
 *   OXQ_TP_W4A16  w_gu / w_down are uint4 codes (8 per u32, group 128 along K), the scales f16 per group, the zeros packed
 *                 nibbles: the tensors of oxq_int4g_quant_pack.
 * y_bf16 [m x hidden] receives the rank's partial and, with reduce != 0, the sum over the ranks (in place, bf16, one
 * all-reduce).  The workspace (oxq_mlp_swiglu_tp_workspace_bytes, 256-byte aligned) holds the intermediates; for
 * OXQ_TP_W4A16 it must be zero-filled once before its first use (the W4A16 decode kernels keep their partial sums there and
 * leave them zero).  Nothing is allocated and nothing synchronises. */
enum { OXQ_TP_FP8 = 0, OXQ_TP_W4A16 = 1 };
typedef struct oxq_tp_mlp_weights {
    int32_t variant;
    int64_t hidden, inter_local;
    const void* w_gu; const void* w_gu_scales; const void* w_gu_zeros;
    const void* w_down; const void* w_down_scales; const void* w_down_zeros;
} oxq_tp_mlp_weights;
OXQ_API int32_t oxq_mlp_swiglu_tp_workspace_bytes(int variant, int64_t m, int64_t hidden, int64_t inter_local, size_t* bytes_out);
OXQ_API int32_t oxq_mlp_swiglu_tp(oxq_handle* h, const oxq_tp_mlp_weights* w, int64_t m, const void* x_bf16_dev, void* y_bf16_dev,
                          void* workspace_dev, size_t workspace_bytes, int reduce);

/* ---- GPTQ weight preparation -------------------------------------------------------------------------------------
 * GptqQuantizer::quantize_layer (crates/oxicuda-quant/src/scheme/gptq.rs:133-257): dampen the Hessian by
 * percdamp * max(|mean diag|, 1e-8), factor it (cholesky_lower, :281-300), invert the factor (invert_lower, :305-318),
 * form H^-1 (hinv_row_starting, :328-332), then quantize column by column with per-column parameters
 * (col_quant_params, :242-276) and push each column's error into the later columns.  All in f32 on the device with
 * the reference's order of operations, so codes, scales and zero points equal the reference's bit for bit.
 *   weights      [n_rows x n_cols] f32 row-major (not modified);   hessian [n_cols x n_cols] f32 row-major, symmetric
 *   quantized    [n_rows x n_cols] i32;   scales [n_cols] f32;   zero_points [n_cols] i32 (0 when symmetric)
 *   info         2 words: info[0] = 1 when the dampened Hessian is not positive definite (the reference's
 *                SingularHessian; nothing else is written then), else 0; info[1] = bits of the smallest dampened
 *                diagonal entry (SingularHessian's min_diag).  The call is asynchronous: read info after the stream.
 *   workspace    oxq_gptq_workspace_bytes(n_rows, n_cols) bytes; on return its first n_cols^2 floats hold H^-1 (upper
 *                triangle), the next n_cols^2 the inverse of the Cholesky factor.
 * GptqConfig::block_size has no effect in the reference and has no parameter here.  The column loop runs as one
 * cooperative launch (one meeting point of all CTAs per column, bounded wait); n_rows <= ~60000, n_cols <= 32768.
 * Errors: EMPTY_INPUT (n_rows or n_cols == 0), INVALID_BIT_WIDTH (bits == 0 or > 16), BUFFER_TOO_SMALL. */
OXQ_API int32_t oxq_gptq_workspace_bytes(int64_t n_rows, int64_t n_cols, size_t* bytes);
OXQ_API int32_t oxq_gptq_quantize_layer(oxq_handle* h, const float* weights_dev, int64_t n_rows, int64_t n_cols, const float* hessian_dev,
                                int bits, int symmetric, double percdamp, int32_t* quantized_dev, float* scales_dev,
                                int32_t* zero_points_dev, int32_t* info_dev, void* workspace_dev, size_t workspace_bytes);

#ifdef __cplusplus
}
#endif
#endif /* OXQ_H_ */
