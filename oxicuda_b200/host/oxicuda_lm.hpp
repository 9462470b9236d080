// Host-side mirror of the SwiGLU feed-forward layer of oxicuda-lm over the C ABI of liboxq_b200:
//   WeightTensor (from_data, zeros, ones, eye)      crates/oxicuda-lm/src/weights.rs:15-76
//   silu                                             crates/oxicuda-lm/src/layer/ffn.rs:25-27
//   SwiGluFfn (new, forward)                         crates/oxicuda-lm/src/layer/ffn.rs:202-254
//   LmError                                          crates/oxicuda-lm/src/error.rs
// Same names, argument meaning and error variants as the reference.  The reference runs three f32 loops on the CPU; here
// forward is two tensor-core GEMMs on the GPU with bf16 operands and f32 accumulation: the gate and up projections in one
// pass with silu(gate) * up applied in the epilogue (oxq_gemm_bf16_swiglu on the weights interleaved in blocks of 128 rows),
// then the down projection (oxq_gemm_bf16).  Results therefore agree with the reference to bf16 precision (2^-8 relative
// per stage), not to its 1e-5.  The layer's weights are public host tensors as in the reference, so every forward stages
// them again; `SwiGluFfn::to_device()` gives a form whose weights stay on the GPU.  The quantized (FP8 / W4A16) and
// tensor-parallel form of the same layer is oxq_mlp_swiglu_tp.
// Header-only; link with -loxq_b200 -lcudart.  There is no CPU fallback: without a device forward throws.
#pragma once
#include <cuda_runtime.h>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>
#include "../../include/oxq.h"

namespace oxicuda_lm {

struct LmError : std::runtime_error {
    std::string variant;
    size_t expected = 0, got = 0;                                         // DimensionMismatch / WeightDataLengthMismatch
    LmError(const std::string& v, const std::string& msg, size_t expected_ = 0, size_t got_ = 0)
        : std::runtime_error(v + ": " + msg), variant(v), expected(expected_), got(got_) {}
};

struct WeightTensor {
    std::vector<float> data;
    std::vector<size_t> shape;
    static size_t product(const std::vector<size_t>& s) { size_t n = 1; for (size_t v : s) n *= v; return n; }
    static WeightTensor from_data(std::vector<float> data, std::vector<size_t> shape) {
        const size_t expected = product(shape);
        if (data.size() != expected) throw LmError("WeightDataLengthMismatch", "data length " + std::to_string(data.size()) + " != " + std::to_string(expected), expected, data.size());
        return {std::move(data), std::move(shape)};
    }
    static WeightTensor zeros(const std::vector<size_t>& shape) { return {std::vector<float>(product(shape), 0.0f), shape}; }
    static WeightTensor ones(const std::vector<size_t>& shape) { return {std::vector<float>(product(shape), 1.0f), shape}; }
    static WeightTensor eye(size_t rows, size_t cols) {
        WeightTensor t = zeros({rows, cols});
        for (size_t i = 0; i < rows && i < cols; i++) t.data[i * cols + i] = 1.0f;
        return t;
    }
    size_t n_elements() const { return data.size(); }
    size_t ndim() const { return shape.size(); }
};

inline float silu(float x) { return x / (1.0f + std::exp(-x)); }

namespace detail {
inline void cuda(cudaError_t e) { if (e != cudaSuccess) throw LmError("Cuda", cudaGetErrorString(e)); }
inline uint16_t f32_to_bf16(float f) {                                    // round to nearest even; NaN stays NaN
    uint32_t u; std::memcpy(&u, &f, 4);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return uint16_t((u >> 16) | 0x0040u);
    return uint16_t((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
}
inline float bf16_to_f32(uint16_t b) { const uint32_t u = uint32_t(b) << 16; float f; std::memcpy(&f, &u, 4); return f; }
inline size_t round_up(size_t v, size_t to) { return (v + to - 1) / to * to; }
struct DevMem {
    void* p = nullptr;
    explicit DevMem(size_t bytes) { if (bytes) cuda(cudaMalloc(&p, bytes)); }
    ~DevMem() { if (p) cudaFree(p); }
    DevMem(const DevMem&) = delete; DevMem& operator=(const DevMem&) = delete;
};
}  // namespace detail

// The layer with its weights resident on the GPU: gate/up interleaved in blocks of 128 rows [2 * inter_pad x hidden_pad]
// and down [out_pad x inter_pad], bf16, zero padded (hidden to a multiple of 64 as a K extent and of 8 as an output
// extent, intermediate to a multiple of 128; a padded intermediate channel has gate = up = 0, so it contributes nothing).
class DeviceSwiGluFfn {
public:
    size_t hidden_dim, intermediate_dim, hidden_pad, inter_pad, out_pad;
    DeviceSwiGluFfn(size_t hidden, size_t inter, const float* w_gate, const float* w_up, const float* w_down, int device = 0)
        : hidden_dim(hidden), intermediate_dim(inter), hidden_pad(detail::round_up(hidden, 64)), inter_pad(detail::round_up(inter, 128)),
          out_pad(detail::round_up(hidden, 8)) {
        detail::cuda(cudaSetDevice(device));
        const int32_t rc = oxq_handle_create(device, nullptr, &h_);
        if (rc) throw LmError(oxq_status_name(rc), "oxq_handle_create");
        try {
            w_gu_.reset(new detail::DevMem(2 * inter_pad * hidden_pad * 2));
            w_down_.reset(new detail::DevMem(out_pad * inter_pad * 2));
            std::vector<uint16_t> gu(2 * inter_pad * hidden_pad, 0), dn(out_pad * inter_pad, 0);
            for (size_t r = 0; r < inter; r++) {
                const size_t blk = r / 128, in_blk = r % 128;
                uint16_t* g = &gu[((2 * blk) * 128 + in_blk) * hidden_pad];
                uint16_t* u = &gu[((2 * blk + 1) * 128 + in_blk) * hidden_pad];
                for (size_t c = 0; c < hidden; c++) { g[c] = detail::f32_to_bf16(w_gate[r * hidden + c]); u[c] = detail::f32_to_bf16(w_up[r * hidden + c]); }
            }
            for (size_t r = 0; r < hidden; r++)
                for (size_t c = 0; c < inter; c++) dn[r * inter_pad + c] = detail::f32_to_bf16(w_down[r * inter + c]);
            detail::cuda(cudaMemcpy(w_gu_->p, gu.data(), gu.size() * 2, cudaMemcpyHostToDevice));
            detail::cuda(cudaMemcpy(w_down_->p, dn.data(), dn.size() * 2, cudaMemcpyHostToDevice));
        } catch (...) { oxq_handle_destroy(h_); h_ = nullptr; throw; }    // a constructor that throws runs no destructor
    }
    ~DeviceSwiGluFfn() { if (h_) oxq_handle_destroy(h_); }
    DeviceSwiGluFfn(const DeviceSwiGluFfn&) = delete; DeviceSwiGluFfn& operator=(const DeviceSwiGluFfn&) = delete;
    oxq_handle* library_handle() const { return h_; }
    // x bf16 [n_tokens x hidden_pad], h scratch bf16 [n_tokens x inter_pad], y bf16 [n_tokens x out_pad]; asynchronous
    void forward_device(const void* x_bf16_dev, size_t n_tokens, void* h_bf16_dev, void* y_bf16_dev) const {
        check(oxq_gemm_bf16_swiglu(h_, (int64_t)n_tokens, (int64_t)(2 * inter_pad), (int64_t)hidden_pad, x_bf16_dev, (int64_t)hidden_pad, w_gu_->p,
                                   (int64_t)hidden_pad, h_bf16_dev, (int64_t)inter_pad));
        check(oxq_gemm_bf16(h_, (int64_t)n_tokens, (int64_t)out_pad, (int64_t)inter_pad, h_bf16_dev, (int64_t)inter_pad, w_down_->p, (int64_t)inter_pad,
                            y_bf16_dev, (int64_t)out_pad));
    }
    // x f32 [n_tokens x hidden] -> f32 [n_tokens x hidden]
    std::vector<float> forward(const std::vector<float>& x, size_t n_tokens) const {
        if (n_tokens == 0) throw LmError("EmptyInput", "SwiGluFfn::forward n_tokens");
        if (x.size() != n_tokens * hidden_dim)
            throw LmError("DimensionMismatch", "expected " + std::to_string(n_tokens * hidden_dim) + ", got " + std::to_string(x.size()), n_tokens * hidden_dim, x.size());
        std::vector<uint16_t> xb(n_tokens * hidden_pad, 0), yb(n_tokens * out_pad);
        for (size_t t = 0; t < n_tokens; t++)
            for (size_t c = 0; c < hidden_dim; c++) xb[t * hidden_pad + c] = detail::f32_to_bf16(x[t * hidden_dim + c]);
        detail::DevMem xd(xb.size() * 2), hd(n_tokens * inter_pad * 2), yd(yb.size() * 2);
        detail::cuda(cudaMemcpy(xd.p, xb.data(), xb.size() * 2, cudaMemcpyHostToDevice));
        forward_device(xd.p, n_tokens, hd.p, yd.p);
        detail::cuda(cudaDeviceSynchronize());
        detail::cuda(cudaMemcpy(yb.data(), yd.p, yb.size() * 2, cudaMemcpyDeviceToHost));
        std::vector<float> out(n_tokens * hidden_dim);
        for (size_t t = 0; t < n_tokens; t++)
            for (size_t c = 0; c < hidden_dim; c++) out[t * hidden_dim + c] = detail::bf16_to_f32(yb[t * out_pad + c]);
        return out;
    }
private:
    void check(int32_t rc) const { if (rc) throw LmError(oxq_status_name(rc), oxq_last_error_string(h_)); }
    oxq_handle* h_ = nullptr;
    std::unique_ptr<detail::DevMem> w_gu_, w_down_;
};

// out = W_down . (silu(W_gate . x) * (W_up . x)), no biases; w_gate and w_up are [intermediate x hidden], w_down [hidden x intermediate].
struct SwiGluFfn {
    size_t hidden_dim, intermediate_dim;
    WeightTensor w_gate, w_up, w_down;
    SwiGluFfn(size_t hidden_dim, size_t intermediate_dim) : hidden_dim(hidden_dim), intermediate_dim(intermediate_dim) {
        if (hidden_dim == 0 || intermediate_dim == 0) throw LmError("InvalidConfig", "SwiGluFfn: dimensions must be > 0");
        w_gate = WeightTensor::zeros({intermediate_dim, hidden_dim});
        w_up = WeightTensor::zeros({intermediate_dim, hidden_dim});
        w_down = WeightTensor::zeros({hidden_dim, intermediate_dim});
    }
    std::unique_ptr<DeviceSwiGluFfn> to_device(int device = 0) const {
        check_weight(w_gate, intermediate_dim, hidden_dim);
        check_weight(w_up, intermediate_dim, hidden_dim);
        check_weight(w_down, hidden_dim, intermediate_dim);
        return std::unique_ptr<DeviceSwiGluFfn>(new DeviceSwiGluFfn(hidden_dim, intermediate_dim, w_gate.data.data(), w_up.data.data(), w_down.data.data(), device));
    }
    std::vector<float> forward(const std::vector<float>& x, size_t n_tokens) const {
        if (n_tokens == 0) throw LmError("EmptyInput", "SwiGluFfn::forward n_tokens");
        return to_device()->forward(x, n_tokens);
    }
private:
    static void check_weight(const WeightTensor& w, size_t rows, size_t cols) {
        if (w.shape.size() != 2) throw LmError("DimensionMismatch", "expected 2, got " + std::to_string(w.shape.size()), 2, w.shape.size());
        if (w.shape[0] != rows || w.shape[1] != cols || w.data.size() != rows * cols)
            throw LmError("DimensionMismatch", "expected " + std::to_string(rows * cols) + ", got " + std::to_string(w.data.size()), rows * cols, w.data.size());
    }
};

}  // namespace oxicuda_lm
