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

// Int4GemmConfig (precision/int_ops.rs:215-355): validate() keeps the reference's rules.
struct Int4GemmConfig {
    uint32_t m, n, k, group_size;
    void validate() const {
        if (m == 0 || n == 0 || k == 0) throw BlasError(OXQ_ERR_INVALID_DIMENSION, "INT4 GEMM dimensions must be non-zero");
        if (k % 8 != 0) throw BlasError(OXQ_ERR_INVALID_ARGUMENT, "K must be a multiple of 8 for INT4 packing");
        if (!(group_size == 32 || group_size == 64 || group_size == 128 || group_size == 256))
            throw BlasError(OXQ_ERR_INVALID_ARGUMENT, "invalid group size");
    }
};
inline void gemm_w4a16(const BlasHandle& h, const Int4GemmConfig& cfg, const void* x_bf16, const uint32_t* codes, const uint16_t* scales_f16,
                       const uint32_t* zeros, void* y_bf16, void* workspace, size_t workspace_bytes) {
    cfg.validate();
    h.check(oxq_gemm_w4a16(h.raw(), cfg.m, cfg.n, cfg.k, x_bf16, codes, scales_f16, zeros, (int)cfg.group_size, y_bf16, workspace, workspace_bytes));
}

}  // namespace oxicuda_blas
