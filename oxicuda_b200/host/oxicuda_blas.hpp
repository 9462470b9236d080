// Host-side mirror of the oxicuda-blas surface on the quantized path over the C ABI of liboxq_b200:
// BlasHandle (crates/oxicuda-blas/src/handle.rs:41-52), MatrixDesc / MatrixDescMut (types.rs:443-643),
// E4M3 (types.rs:313-357), BlasError (error.rs:16-59) and the gemm entry point (level3/gemm_api.rs:73-138) for
// the element types the reference cannot run.  Device memory is caller-owned, calls are asynchronous on the
// handle's stream.  Header-only; link with -loxq_b200 -lcudart.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>
#include "../../include/oxq.h"

namespace oxicuda_blas {

struct BlasError : std::runtime_error {
    std::string variant; int32_t status;
    BlasError(int32_t st, const std::string& msg) : std::runtime_error(std::string(oxq_status_name(st)) + ": " + msg), variant(oxq_status_name(st)), status(st) {}
};

struct E4M3 { uint8_t bits; };                                           // #[repr(transparent)] u8; one = 0x38
enum class Layout { RowMajor, ColMajor };
enum class Transpose { NoTrans, Trans };

template <typename T> struct MatrixDesc {                                 // borrowed view, caller owns the memory
    const T* ptr; uint32_t rows, cols, ld; Layout layout;
};
template <typename T> struct MatrixDescMut { T* ptr; uint32_t rows, cols, ld; Layout layout; };

class BlasHandle {                                                       // Send, not Sync: one per thread
public:
    explicit BlasHandle(int device = 0, cudaStream_t stream = nullptr) {
        int32_t rc = oxq_handle_create(device, stream, &h_);
        if (rc) throw BlasError(rc, "oxq_handle_create");
    }
    ~BlasHandle() { if (h_) oxq_handle_destroy(h_); }
    BlasHandle(const BlasHandle&) = delete; BlasHandle& operator=(const BlasHandle&) = delete;
    void set_stream(cudaStream_t s) { check(oxq_set_stream(h_, s)); }
    oxq_handle* raw() const { return h_; }
    void check(int32_t rc) const { if (rc) throw BlasError(rc, oxq_last_error_string(h_)); }
private:
    oxq_handle* h_ = nullptr;
};

// C[M x N] (bf16) = (A[M x K] . B[N x K]^T) * (*scale_a * *scale_b): gemm::<E4M3> with op(B) = B^T, alpha folded
// into the scales, beta = 0.  Validation order and error variants follow gemm_api.rs:84-108.
inline void gemm_fp8(const BlasHandle& h, const MatrixDesc<E4M3>& a, const MatrixDesc<E4M3>& b_nk, const float* scale_a_dev,
                     const float* scale_b_dev, MatrixDescMut<uint16_t>& c_bf16) {
    if (a.rows == 0 || b_nk.rows == 0 || a.cols == 0) throw BlasError(OXQ_ERR_INVALID_DIMENSION, "GEMM dimensions must be non-zero");
    if (a.cols != b_nk.cols) throw BlasError(OXQ_ERR_DIMENSION_MISMATCH, "inner dimensions of op(A) and op(B) do not match");
    if (c_bf16.rows != a.rows || c_bf16.cols != b_nk.rows) throw BlasError(OXQ_ERR_DIMENSION_MISMATCH, "C shape does not match the GEMM result");
    h.check(oxq_gemm_fp8(h.raw(), a.rows, b_nk.rows, a.cols, reinterpret_cast<const uint8_t*>(a.ptr), a.ld,
                         reinterpret_cast<const uint8_t*>(b_nk.ptr), b_nk.ld, scale_a_dev, scale_b_dev, c_bf16.ptr, c_bf16.ld));
}

// The general form of gemm_api.rs:73-82, C = alpha * A * B^T * scales + beta * C; C is not read when beta == 0.
inline void gemm_fp8(const BlasHandle& h, float alpha, const MatrixDesc<E4M3>& a, const MatrixDesc<E4M3>& b_nk, const float* scale_a_dev,
                     const float* scale_b_dev, float beta, MatrixDescMut<uint16_t>& c_bf16) {
    if (a.rows == 0 || b_nk.rows == 0 || a.cols == 0) throw BlasError(OXQ_ERR_INVALID_DIMENSION, "GEMM dimensions must be non-zero");
    if (a.cols != b_nk.cols) throw BlasError(OXQ_ERR_DIMENSION_MISMATCH, "inner dimensions of op(A) and op(B) do not match");
    if (c_bf16.rows != a.rows || c_bf16.cols != b_nk.rows) throw BlasError(OXQ_ERR_DIMENSION_MISMATCH, "C shape does not match the GEMM result");
    h.check(oxq_gemm_fp8_ex(h.raw(), a.rows, b_nk.rows, a.cols, alpha, reinterpret_cast<const uint8_t*>(a.ptr), a.ld,
                            reinterpret_cast<const uint8_t*>(b_nk.ptr), b_nk.ld, scale_a_dev, scale_b_dev, beta, c_bf16.ptr, c_bf16.ld));
}

// ---- gemm<T> with the reference's operand forms --------------------------------------------------------------------
// gemm(handle, trans_a, trans_b, alpha, a, b, beta, c) of gemm_api.rs:73-138: op(A) is [m x k], op(B) is [k x n], every
// matrix row- or column-major.  Validation order and error variants follow gemm_api.rs:84-137: zero dimensions ->
// InvalidDimension, inner dimensions that disagree -> DimensionMismatch, C of another shape -> DimensionMismatch.  The
// library's kernels take either index of an operand as the contiguous one, so no combination is refused and nothing is
// copied; a column-major C is computed as the row-major C^T = op(B)^T * op(A)^T.  Per-tensor scales (device floats) are
// the E4M3 operands' dequantisation factors; C is bf16.
namespace detail {
// true when the operand's row index (of op(X)) is the contiguous one in memory
inline bool rows_contiguous(Transpose t, Layout l) { return (t == Transpose::Trans) == (l == Layout::RowMajor); }
inline uint32_t op_rows(Transpose t, uint32_t rows, uint32_t cols) { return t == Transpose::NoTrans ? rows : cols; }
inline uint32_t op_cols(Transpose t, uint32_t rows, uint32_t cols) { return t == Transpose::NoTrans ? cols : rows; }
}  // namespace detail

inline void gemm(const BlasHandle& h, Transpose trans_a, Transpose trans_b, float alpha, const MatrixDesc<E4M3>& a, const float* scale_a_dev,
                 const MatrixDesc<E4M3>& b, const float* scale_b_dev, float beta, MatrixDescMut<uint16_t>& c_bf16) {
    const uint32_t m = detail::op_rows(trans_a, a.rows, a.cols), k = detail::op_cols(trans_a, a.rows, a.cols);
    const uint32_t kb = detail::op_rows(trans_b, b.rows, b.cols), n = detail::op_cols(trans_b, b.rows, b.cols);
    if (m == 0 || n == 0 || k == 0) throw BlasError(OXQ_ERR_INVALID_DIMENSION, "GEMM dimensions must be non-zero");
    if (k != kb) throw BlasError(OXQ_ERR_DIMENSION_MISMATCH, "inner dimensions of op(A) and op(B) do not match");
    if (c_bf16.rows != m || c_bf16.cols != n) throw BlasError(OXQ_ERR_DIMENSION_MISMATCH, "C shape does not match the GEMM result");
    // op(A) [m x k]: MN-major when m is the contiguous index; op(B) [k x n]: K-major when k (its row index) is contiguous
    const int a_major = detail::rows_contiguous(trans_a, a.layout) ? OXQ_OP_MN_MAJOR : OXQ_OP_K_MAJOR;
    const int b_major = detail::rows_contiguous(trans_b, b.layout) ? OXQ_OP_K_MAJOR : OXQ_OP_MN_MAJOR;
    const uint8_t* ap = reinterpret_cast<const uint8_t*>(a.ptr);
    const uint8_t* bp = reinterpret_cast<const uint8_t*>(b.ptr);
    if (c_bf16.layout == Layout::RowMajor) {
        h.check(oxq_gemm_fp8_op(h.raw(), m, n, k, alpha, ap, a.ld, a_major, bp, b.ld, b_major, scale_a_dev, scale_b_dev, beta, c_bf16.ptr, c_bf16.ld));
    } else {
        // C^T [n x m] row-major = op(B)^T [n x k] * op(A)^T [k x m]: B takes A's place with the meaning of its flag kept
        // (K-major stays "k contiguous"), and likewise A
        h.check(oxq_gemm_fp8_op(h.raw(), n, m, k, alpha, bp, b.ld, b_major, ap, a.ld, a_major, scale_b_dev, scale_a_dev, beta, c_bf16.ptr, c_bf16.ld));
    }
}

// ---- low-precision GEMM configurations ----------------------------------------------------------------------------
// SmVersion of the reference's PTX layer (crates/oxicuda-ptx/src/arch.rs:20-37), ordered.
enum class SmVersion { Sm75 = 75, Sm80 = 80, Sm86 = 86, Sm89 = 89, Sm90 = 90, Sm90a = 91, Sm100 = 100, Sm120 = 120 };
enum class AccType { I32, F32 };

// Int8GemmConfig (precision/int_ops.rs:79-125).
struct Int8GemmConfig {
    uint32_t m, n, k;
    Layout layout_a = Layout::RowMajor, layout_b = Layout::RowMajor;
    AccType accumulator = AccType::I32;
    static constexpr uint32_t ELEMENT_BYTES = 1;
    static bool is_available(SmVersion sm) { return sm >= SmVersion::Sm75; }
    void validate(SmVersion sm) const {
        if (m == 0 || n == 0 || k == 0) throw BlasError(OXQ_ERR_INVALID_DIMENSION, "INT8 GEMM dimensions must be non-zero");
        if (k % 4 != 0) throw BlasError(OXQ_ERR_INVALID_DIMENSION, "INT8 GEMM K dimension must be a multiple of 4 for dp4a, got k=" + std::to_string(k));
        if (!is_available(sm)) throw BlasError(OXQ_ERR_UNSUPPORTED_OPERATION, "INT8 dp4a requires Turing+ (sm_75)");
    }
};

// Int4GemmConfig (precision/int_ops.rs:215-281).
struct Int4GemmConfig {
    uint32_t m, n, k;
    Layout layout_a = Layout::RowMajor, layout_b = Layout::RowMajor;
    uint32_t group_size = 128;
    static constexpr uint32_t PACKED_ELEMENT_BYTES = 4, VALUES_PER_U32 = 8;
    static bool is_available(SmVersion sm) { return sm >= SmVersion::Sm75; }
    void validate(SmVersion sm) const {
        if (m == 0 || n == 0 || k == 0) throw BlasError(OXQ_ERR_INVALID_DIMENSION, "INT4 GEMM dimensions must be non-zero");
        if (k % 8 != 0) throw BlasError(OXQ_ERR_INVALID_DIMENSION, "INT4 GEMM K dimension must be a multiple of 8 for packing, got k=" + std::to_string(k));
        if (group_size == 0 || (group_size & (group_size - 1)) != 0)
            throw BlasError(OXQ_ERR_INVALID_ARGUMENT, "INT4 group_size must be a positive power of 2, got " + std::to_string(group_size));
        if (k % group_size != 0) throw BlasError(OXQ_ERR_INVALID_ARGUMENT, "INT4 group_size must divide K evenly");
        if (!is_available(sm)) throw BlasError(OXQ_ERR_UNSUPPORTED_OPERATION, "INT4 GEMM requires Turing+ (sm_75)");
    }
};

// MicroScalingConfig (precision/fp4_fp6_ops.rs:190-225).
enum class ScalingFormat { E8M0, Fp16, Fp32 };
enum class ScalingGranularity { PerTensor, PerChannel, PerBlock };
struct MicroScalingConfig {
    uint32_t block_size = 32;
    ScalingFormat scaling_format = ScalingFormat::Fp32;
    ScalingGranularity scaling_granularity = ScalingGranularity::PerBlock;
    void validate() const {
        if (!(block_size == 32 || block_size == 64 || block_size == 128))
            throw BlasError(OXQ_ERR_INVALID_ARGUMENT, "MicroScaling block_size must be one of [32, 64, 128], got " + std::to_string(block_size));
    }
    uint32_t num_scales(uint32_t num_elements) const {
        switch (scaling_granularity) {
            case ScalingGranularity::PerTensor: return 1;
            case ScalingGranularity::PerChannel: return num_elements;
            default: return (num_elements + block_size - 1) / block_size;
        }
    }
};

// Fp4GemmConfig (precision/fp4_fp6_ops.rs:337-395).
enum class Fp4Format { E2M1, Int4 };
enum class SubByteAccumulator { F16, F32 };
struct Fp4GemmConfig {
    uint32_t m, n, k;
    Fp4Format format = Fp4Format::E2M1;
    SubByteAccumulator accumulator = SubByteAccumulator::F32;
    MicroScalingConfig micro_scaling;
    SmVersion sm_version = SmVersion::Sm100;
    static constexpr SmVersion MIN_SM = SmVersion::Sm100;
    void validate() const {
        if (m == 0 || n == 0 || k == 0) throw BlasError(OXQ_ERR_INVALID_DIMENSION, "FP4 GEMM dimensions must be non-zero");
        if (sm_version < MIN_SM) throw BlasError(OXQ_ERR_UNSUPPORTED_OPERATION, "FP4 Tensor Cores require Blackwell+ (sm_100)");
        if (k % 2 != 0) throw BlasError(OXQ_ERR_INVALID_DIMENSION, "FP4 GEMM K dimension must be even for packing, got k=" + std::to_string(k));
        micro_scaling.validate();
    }
    std::string kernel_name() const {
        return std::string("fp4_") + (format == Fp4Format::E2M1 ? "e2m1" : "int4") + "_gemm_" + std::to_string(m) + "x" + std::to_string(n) + "x" +
               std::to_string(k) + "_" + (accumulator == SubByteAccumulator::F32 ? "f32" : "f16");
    }
};

// PackedFp4 (precision/fp4_fp6_ops.rs:452-480): two 4-bit codes in a byte, the first in the low nibble.
struct PackedFp4 {
    uint8_t bits;
    std::pair<uint8_t, uint8_t> unpack() const { return {uint8_t(bits & 0xF), uint8_t(bits >> 4)}; }
};

// MicroScalingQuantizer (precision/fp4_fp6_ops.rs:736-898), the FP4 half: one f32 scale max|x| / 6 per block (1 for an
// all-zero block; the last block may be short), codes from the floor-type E2M1 encoder on x / scale; an odd length is
// padded with one zero code.  Host slices are staged through device buffers on
// device 0's default stream.  The device path covers Fp4Format::E2M1.
class MicroScalingQuantizer {
public:
    explicit MicroScalingQuantizer(const MicroScalingConfig& config) : config(config) {}
    MicroScalingConfig config;
    std::pair<std::vector<PackedFp4>, std::vector<float>> quantize_fp4(const std::vector<float>& values, Fp4Format format) const {
        config.validate();
        if (format != Fp4Format::E2M1) throw BlasError(OXQ_ERR_UNSUPPORTED_OPERATION, "the device path covers Fp4Format::E2M1");
        const size_t n = values.size(), bs = config.block_size;
        std::pair<std::vector<PackedFp4>, std::vector<float>> out{std::vector<PackedFp4>((n + 1) / 2), std::vector<float>((n + bs - 1) / bs)};
        if (n == 0) return out;
        BlasHandle h;
        Buf x(n * sizeof(float)), packed(out.first.size()), scales(out.second.size() * sizeof(float));
        cuda(cudaMemcpy(x.p, values.data(), n * sizeof(float), cudaMemcpyHostToDevice));
        h.check(oxq_fp4_microscale_quant(h.raw(), (const float*)x.p, (int64_t)n, (int64_t)bs, (uint8_t*)packed.p, (float*)scales.p));
        cuda(cudaDeviceSynchronize());
        cuda(cudaMemcpy(out.first.data(), packed.p, out.first.size(), cudaMemcpyDeviceToHost));
        cuda(cudaMemcpy(out.second.data(), scales.p, out.second.size() * sizeof(float), cudaMemcpyDeviceToHost));
        return out;
    }
    std::vector<float> dequantize_fp4(const std::vector<PackedFp4>& packed, const std::vector<float>& scales, Fp4Format format, size_t original_len) const {
        if (format != Fp4Format::E2M1) throw BlasError(OXQ_ERR_UNSUPPORTED_OPERATION, "the device path covers Fp4Format::E2M1");
        const size_t bs = config.block_size;
        const size_t n = original_len < packed.size() * 2 ? original_len : packed.size() * 2;   // .take(original_len) of what was packed
        std::vector<float> out(n);
        if (n == 0) return out;
        BlasHandle h;
        std::vector<float> sc((n + bs - 1) / bs, 1.0f);                    // a missing scale counts as 1 (scales.get(..).unwrap_or(1.0))
        for (size_t i = 0; i < sc.size() && i < scales.size(); i++) sc[i] = scales[i];
        Buf p((n + 1) / 2), s(sc.size() * sizeof(float)), y(n * sizeof(float));
        cuda(cudaMemcpy(p.p, packed.data(), (n + 1) / 2, cudaMemcpyHostToDevice));
        cuda(cudaMemcpy(s.p, sc.data(), sc.size() * sizeof(float), cudaMemcpyHostToDevice));
        h.check(oxq_fp4_microscale_dequant(h.raw(), (const uint8_t*)p.p, (const float*)s.p, (int64_t)n, (int64_t)bs, (float*)y.p));
        cuda(cudaDeviceSynchronize());
        cuda(cudaMemcpy(out.data(), y.p, n * sizeof(float), cudaMemcpyDeviceToHost));
        return out;
    }
private:
    static void cuda(cudaError_t e) { if (e != cudaSuccess) throw BlasError(OXQ_ERR_LAUNCH_FAILED, cudaGetErrorString(e)); }
    struct Buf {
        void* p = nullptr;
        explicit Buf(size_t bytes) { if (bytes) cuda(cudaMalloc(&p, bytes)); }
        ~Buf() { if (p) cudaFree(p); }
        Buf(const Buf&) = delete; Buf& operator=(const Buf&) = delete;
    };
};

// The GEMMs those configurations describe, over the library's kernels.  The quantised operand is the weight W[N x K]
// (the reference's generators quantise "A"; the roles are exchanged, C^T = W * X^T).
inline void gemm_w8a8(const BlasHandle& h, const Int8GemmConfig& cfg, const int8_t* x, const int8_t* w, const float* sx_rows, const float* sw_rows,
                      void* y_bf16) {
    cfg.validate(SmVersion::Sm100);
    h.check(oxq_gemm_w8a8(h.raw(), cfg.m, cfg.n, cfg.k, x, cfg.k, w, cfg.k, sx_rows, sw_rows, y_bf16, cfg.n));
}
inline void gemm_w4a16(const BlasHandle& h, const Int4GemmConfig& cfg, const void* x_bf16, const uint32_t* codes, const uint16_t* scales_f16,
                       const uint32_t* zeros, void* y_bf16, void* workspace, size_t workspace_bytes) {
    cfg.validate(SmVersion::Sm100);
    h.check(oxq_gemm_w4a16(h.raw(), cfg.m, cfg.n, cfg.k, x_bf16, codes, scales_f16, zeros, (int)cfg.group_size, y_bf16, workspace, workspace_bytes));
}
// NVFP4 operands (E2M1 codes, UE4M3 scale per 16, f32 tensor scale) as produced by oxq_nvfp4_quant
inline void gemm_nvfp4(const BlasHandle& h, const Fp4GemmConfig& cfg, const uint8_t* x, const uint8_t* sfx_mma, const float* gx, const uint8_t* w,
                       const uint8_t* sfw_mma, const float* gw, void* y_bf16) {
    cfg.validate();
    h.check(oxq_gemm_nvfp4(h.raw(), cfg.m, cfg.n, cfg.k, x, sfx_mma, gx, w, sfw_mma, gw, y_bf16, cfg.n));
}
// MXFP8 operands (E4M3 codes, one E8M0 scale per 32 elements along K) as produced by oxq_mxfp8_quant; the micro-scaling
// configuration is the one the format fixes (block 32, E8M0 scales)
inline void gemm_mxfp8(const BlasHandle& h, uint32_t m, uint32_t n, uint32_t k, const uint8_t* x, const uint8_t* sfx_mma, const uint8_t* w, const uint8_t* sfw_mma,
                       void* y_bf16) {
    if (m == 0 || n == 0 || k == 0) throw BlasError(OXQ_ERR_INVALID_DIMENSION, "MXFP8 GEMM dimensions must be non-zero");
    h.check(oxq_gemm_mxfp8(h.raw(), m, n, k, x, sfx_mma, w, sfw_mma, y_bf16, n));
}
// W8A32 decode GEMM (Int8GemmConfig with f32 activations): Y_f32 = X_f32 . (W_i8 * sw_rows)^T
inline void gemm_w8a32(const BlasHandle& h, const Int8GemmConfig& cfg, const float* x, const int8_t* w, const float* sw_rows, float* y_f32) {
    cfg.validate(SmVersion::Sm100);
    h.check(oxq_gemm_w8a32(h.raw(), cfg.m, cfg.n, cfg.k, x, w, sw_rows, y_f32));
}

}  // namespace oxicuda_blas
