// Host-side mirror of the oxicuda-dnn quantize API over the C ABI of liboxq_b200 (include/oxq.h): device buffers in,
// device buffers out, asynchronous on the handle's stream, nothing allocated by the calls except where noted.
//   quantize_to_int8 / dequantize_from_int8       crates/oxicuda-dnn/src/quantize/int8_quantize.rs:33-157
//   quantize_to_fp8 / dequantize_from_fp8         crates/oxicuda-dnn/src/quantize/fp8_quantize.rs:47-170
//   Int4QuantConfig, quantize_to_int4, dequantize_int4   crates/oxicuda-dnn/src/quantize/int4_quantize.rs:60-300
//   quantize_block_scaled, Fp4BlockQuantizer      crates/oxicuda-dnn/src/quantize/block_scale.rs:53-140, :346-395
//   TensorDesc / TensorDescMut (matrix, from_raw, numel)   crates/oxicuda-dnn/src/types.rs:108-400
//   DnnError                                      crates/oxicuda-dnn/src/error.rs:13-60
// The order of the checks is the reference's.  BufferTooSmall carries byte counts, as error.rs documents the variant
// (the reference's call sites mix element and byte counts; for one-byte element types the two agree).
// Header-only; link with -loxq_b200 -lcudart.  There is no CPU fallback: without a device every call throws.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>
#include "../../include/oxq.h"

namespace oxicuda_dnn {

struct DnnError : std::runtime_error {
    std::string variant;
    size_t expected = 0, actual = 0;                                      // BufferTooSmall only
    DnnError(const std::string& v, const std::string& msg) : std::runtime_error(v + ": " + msg), variant(v) {}
    static DnnError buffer_too_small(size_t expected_bytes, size_t actual_bytes) {
        DnnError e("BufferTooSmall", "buffer too small: expected " + std::to_string(expected_bytes) + " bytes, got " + std::to_string(actual_bytes) + " bytes");
        e.expected = expected_bytes; e.actual = actual_bytes;
        return e;
    }
};

// element types: f32 is `float`; the 16-bit formats are carried as bit patterns
struct bf16 { uint16_t bits; };
struct f16 { uint16_t bits; };
template <typename T> struct GpuFloat;
template <> struct GpuFloat<float> { static constexpr int DTYPE = OXQ_F32; };
template <> struct GpuFloat<bf16> { static constexpr int DTYPE = OXQ_BF16; };
template <> struct GpuFloat<f16> { static constexpr int DTYPE = OXQ_F16; };

namespace detail {
inline void cuda(cudaError_t e) { if (e != cudaSuccess) throw DnnError("Cuda", cudaGetErrorString(e)); }
}  // namespace detail

// DeviceBuffer<T> of oxicuda-memory as this API uses it: an owned device allocation of `len` elements.
template <typename T> class DeviceBuffer {
public:
    static DeviceBuffer alloc(size_t n) { DeviceBuffer b; b.n_ = n; if (n) detail::cuda(cudaMalloc(&b.p_, n * sizeof(T))); return b; }
    static DeviceBuffer from_slice(const std::vector<T>& host) {
        DeviceBuffer b = alloc(host.size());
        if (b.n_) detail::cuda(cudaMemcpy(b.p_, host.data(), b.n_ * sizeof(T), cudaMemcpyHostToDevice));
        return b;
    }
    DeviceBuffer(DeviceBuffer&& o) noexcept : p_(o.p_), n_(o.n_) { o.p_ = nullptr; o.n_ = 0; }
    DeviceBuffer& operator=(DeviceBuffer&& o) noexcept { if (this != &o) { release(); p_ = o.p_; n_ = o.n_; o.p_ = nullptr; o.n_ = 0; } return *this; }
    DeviceBuffer(const DeviceBuffer&) = delete; DeviceBuffer& operator=(const DeviceBuffer&) = delete;
    ~DeviceBuffer() { release(); }
    size_t len() const { return n_; }
    bool is_empty() const { return n_ == 0; }
    T* as_device_ptr() const { return p_; }
    std::vector<T> to_vec() const {                                      // copy back on the default stream: synchronise a non-blocking stream first
        std::vector<T> out(n_);
        if (n_) detail::cuda(cudaMemcpy(out.data(), p_, n_ * sizeof(T), cudaMemcpyDeviceToHost));
        return out;
    }
private:
    DeviceBuffer() = default;
    void release() { if (p_) cudaFree(p_); p_ = nullptr; }
    T* p_ = nullptr; size_t n_ = 0;
};

// TensorDesc<T> / TensorDescMut<T>: a borrowed device pointer with dims and strides (in elements).
template <typename T> struct TensorDesc {
    const T* ptr = nullptr;
    std::vector<uint32_t> dims, strides;
    static TensorDesc matrix(const DeviceBuffer<T>& buf, uint32_t rows, uint32_t cols) {
        if (rows == 0) throw DnnError("InvalidDimension", "dimension 0 is zero");
        if (cols == 0) throw DnnError("InvalidDimension", "dimension 1 is zero");
        TensorDesc d; d.ptr = buf.as_device_ptr(); d.dims = {rows, cols}; d.strides = {cols, 1};
        if (buf.len() < d.numel()) throw DnnError::buffer_too_small(d.numel() * sizeof(T), buf.len() * sizeof(T));
        return d;
    }
    static TensorDesc from_raw(const T* ptr, std::vector<uint32_t> dims, std::vector<uint32_t> strides) {
        if (dims.size() != strides.size())
            throw DnnError("InvalidDimension", "dims length (" + std::to_string(dims.size()) + ") != strides length (" + std::to_string(strides.size()) + ")");
        if (dims.empty()) throw DnnError("InvalidDimension", "empty dims");
        TensorDesc d; d.ptr = ptr; d.dims = std::move(dims); d.strides = std::move(strides);
        return d;
    }
    size_t numel() const { size_t n = 1; for (uint32_t v : dims) n *= v; return n; }
    size_t ndim() const { return dims.size(); }
};
template <typename T> struct TensorDescMut {
    T* ptr = nullptr;
    std::vector<uint32_t> dims, strides;
    static TensorDescMut matrix(DeviceBuffer<T>& buf, uint32_t rows, uint32_t cols) {
        if (rows == 0) throw DnnError("InvalidDimension", "dimension 0 is zero");
        if (cols == 0) throw DnnError("InvalidDimension", "dimension 1 is zero");
        TensorDescMut d; d.ptr = buf.as_device_ptr(); d.dims = {rows, cols}; d.strides = {cols, 1};
        if (buf.len() < d.numel()) throw DnnError::buffer_too_small(d.numel() * sizeof(T), buf.len() * sizeof(T));
        return d;
    }
    size_t numel() const { size_t n = 1; for (uint32_t v : dims) n *= v; return n; }
    TensorDesc<T> as_immutable() const { TensorDesc<T> d; d.ptr = ptr; d.dims = dims; d.strides = strides; return d; }
};

// DnnHandle (crates/oxicuda-dnn/src/handle.rs:43-175): one library handle bound to a device and a stream.
class DnnHandle {
public:
    explicit DnnHandle(int device = 0, cudaStream_t stream = nullptr) : stream_(stream) {
        const int32_t rc = oxq_handle_create(device, stream, &h_);
        if (rc) throw DnnError(oxq_status_name(rc), "oxq_handle_create");
    }
    ~DnnHandle() { if (h_) oxq_handle_destroy(h_); }
    DnnHandle(const DnnHandle&) = delete; DnnHandle& operator=(const DnnHandle&) = delete;
    void set_stream(cudaStream_t s) { check(oxq_set_stream(h_, s)); stream_ = s; }
    cudaStream_t stream() const { return stream_; }
    oxq_handle* raw() const { return h_; }
    void check(int32_t rc) const { if (rc) throw DnnError(oxq_status_name(rc), oxq_last_error_string(h_)); }
private:
    oxq_handle* h_ = nullptr;
    cudaStream_t stream_ = nullptr;
};

// scale[0] = max(absmax / 127, 1e-12); output[i] = rint(clamp(input[i] / scale, -127, 127))
template <typename T>
inline void quantize_to_int8(const DnnHandle& handle, const TensorDesc<T>& input, DeviceBuffer<int8_t>& output, DeviceBuffer<float>& scale) {
    const size_t n = input.numel();
    if (n == 0) return;
    if (output.len() < n) throw DnnError::buffer_too_small(n, output.len());
    if (scale.is_empty()) throw DnnError::buffer_too_small(sizeof(float), 0);
    handle.check(oxq_int8_quant_tensor(handle.raw(), input.ptr, GpuFloat<T>::DTYPE, (int64_t)n, output.as_device_ptr(), scale.as_device_ptr()));
}
// output[i] = (float)input[i] * scale[0]
template <typename T>
inline void dequantize_from_int8(const DnnHandle& handle, const DeviceBuffer<int8_t>& input, const DeviceBuffer<float>& scale, TensorDescMut<T>& output, uint32_t n) {
    if (n == 0) return;
    if (input.len() < n) throw DnnError::buffer_too_small(n, input.len());
    if (scale.is_empty()) throw DnnError::buffer_too_small(sizeof(float), 0);
    if (output.numel() < n) throw DnnError::buffer_too_small((size_t)n * sizeof(T), output.numel() * sizeof(T));
    handle.check(oxq_int8_dequant_tensor(handle.raw(), input.as_device_ptr(), scale.as_device_ptr(), (int64_t)n, output.ptr, GpuFloat<T>::DTYPE));
}

// scale[0] = absmax / 448 (1 for an all-zero tensor); output[i] = E4M3(input[i] / scale), round to nearest even, saturating.
// The library's entry writes {absmax, scale} into two floats; this wrapper keeps the reference's one-float `scale`
// buffer by staging through a two-float device scratch (allocated and freed here, stream-ordered).
template <typename T>
inline void quantize_to_fp8(const DnnHandle& handle, const TensorDesc<T>& input, DeviceBuffer<uint8_t>& output, DeviceBuffer<float>& scale) {
    const size_t n = input.numel();
    if (n == 0) return;
    if (output.len() < n) throw DnnError::buffer_too_small(n, output.len());
    if (scale.is_empty()) throw DnnError::buffer_too_small(sizeof(float), 0);
    float* stats = nullptr;
    detail::cuda(cudaMallocAsync((void**)&stats, 2 * sizeof(float), handle.stream()));
    const int32_t rc = oxq_fp8_quant_dynamic(handle.raw(), input.ptr, GpuFloat<T>::DTYPE, (int64_t)n, output.as_device_ptr(), stats);
    if (rc == OXQ_OK) cudaMemcpyAsync(scale.as_device_ptr(), stats + 1, sizeof(float), cudaMemcpyDeviceToDevice, handle.stream());
    cudaFreeAsync(stats, handle.stream());
    handle.check(rc);
}
// output[i] = e4m3(input[i]) * scale[0]
template <typename T>
inline void dequantize_from_fp8(const DnnHandle& handle, const DeviceBuffer<uint8_t>& input, const DeviceBuffer<float>& scale, TensorDescMut<T>& output, uint32_t n) {
    if (n == 0) return;
    if (input.len() < n) throw DnnError::buffer_too_small(n, input.len());
    if (scale.is_empty()) throw DnnError::buffer_too_small(sizeof(float), 0);
    if (output.numel() < n) throw DnnError::buffer_too_small((size_t)n * sizeof(T), output.numel() * sizeof(T));
    handle.check(oxq_fp8_dequant(handle.raw(), input.as_device_ptr(), (int64_t)n, scale.as_device_ptr(), output.ptr, GpuFloat<T>::DTYPE, OXQ_FP8_SPEC_RNE));
}

struct Int4QuantConfig {
    size_t group_size; bool symmetric;
    Int4QuantConfig(size_t group_size, bool symmetric) : group_size(group_size), symmetric(symmetric) {
        if (group_size == 0) throw DnnError("InvalidArgument", "INT4 group_size must be non-zero");
    }
    size_t num_groups(size_t n) const { return (n + group_size - 1) / group_size; }
    size_t packed_bytes(size_t n) const { return (n + 1) / 2; }
};
// Per group of config.group_size contiguous elements: symmetric scale = max(absmax, 1e-12) / 7 and codes
// trunc(clamp(x / scale, -8, 7) + 8); asymmetric scale = max(max - min, 1e-12) / 15, zeros = -min / scale and codes
// trunc(clamp(x / scale, 0, 15)).  Two codes per byte, the even element in the low nibble.  f32 data.
inline void quantize_to_int4(const DnnHandle& handle, const DeviceBuffer<float>& input, DeviceBuffer<uint8_t>& output, DeviceBuffer<float>& scales,
                             DeviceBuffer<float>& zeros, size_t n, const Int4QuantConfig& config) {
    if (n == 0) return;
    const size_t num_groups = config.num_groups(n), packed_bytes = config.packed_bytes(n);
    if (input.len() < n) throw DnnError::buffer_too_small(n * sizeof(float), input.len() * sizeof(float));
    if (output.len() < packed_bytes) throw DnnError::buffer_too_small(packed_bytes, output.len());
    if (scales.len() < num_groups) throw DnnError::buffer_too_small(num_groups * sizeof(float), scales.len() * sizeof(float));
    if (!config.symmetric && zeros.len() < num_groups) throw DnnError::buffer_too_small(num_groups * sizeof(float), zeros.len() * sizeof(float));
    handle.check(oxq_dnn_int4_quant(handle.raw(), input.as_device_ptr(), (int64_t)n, (int64_t)config.group_size, config.symmetric ? 1 : 0,
                                    output.as_device_ptr(), scales.as_device_ptr(), config.symmetric ? nullptr : zeros.as_device_ptr()));
}
// symmetric: out = (code - 8) * scale; asymmetric: out = code * scale (the kernels of the reference do not read `zeros`)
inline void dequantize_int4(const DnnHandle& handle, const DeviceBuffer<uint8_t>& input, const DeviceBuffer<float>& scales, const DeviceBuffer<float>& zeros,
                            DeviceBuffer<float>& output, size_t n, const Int4QuantConfig& config) {
    if (n == 0) return;
    (void)zeros;
    const size_t num_groups = config.num_groups(n), packed_bytes = config.packed_bytes(n);
    if (input.len() < packed_bytes) throw DnnError::buffer_too_small(packed_bytes, input.len());
    if (scales.len() < num_groups) throw DnnError::buffer_too_small(num_groups * sizeof(float), scales.len() * sizeof(float));
    if (output.len() < n) throw DnnError::buffer_too_small(n * sizeof(float), output.len() * sizeof(float));
    handle.check(oxq_dnn_int4_dequant(handle.raw(), input.as_device_ptr(), scales.as_device_ptr(), (int64_t)n, (int64_t)config.group_size,
                                      config.symmetric ? 1 : 0, output.as_device_ptr()));
}

// Per block of block_size elements (a power of two, at least 16): scale = max(absmax / 6, 1e-12),
// output = clamp(int(rint(clamp(x / scale, -6, 6))) + 6, 0, 255), one byte per element.
template <typename T>
inline void quantize_block_scaled(const DnnHandle& handle, const TensorDesc<T>& input, DeviceBuffer<uint8_t>& output, DeviceBuffer<float>& scales,
                                  uint32_t block_size) {
    const size_t n = input.numel();
    if (n == 0) return;
    if (block_size == 0 || (block_size & (block_size - 1)) != 0)
        throw DnnError("InvalidArgument", "block_size must be a non-zero power of 2, got " + std::to_string(block_size));
    if (block_size < 16) throw DnnError("InvalidArgument", "block_size must be >= 16, got " + std::to_string(block_size));
    if (output.len() < n) throw DnnError::buffer_too_small(n, output.len());
    const size_t num_blocks = (n + block_size - 1) / block_size;
    if (scales.len() < num_blocks) throw DnnError::buffer_too_small(num_blocks * sizeof(float), scales.len() * sizeof(float));
    handle.check(oxq_dnn_block_scaled_quant(handle.raw(), input.ptr, GpuFloat<T>::DTYPE, (int64_t)n, (int64_t)block_size, output.as_device_ptr(),
                                            scales.as_device_ptr()));
}

// Fp4BlockQuantizer (crates/oxicuda-dnn/src/quantize/block_scale.rs:346-395): the host-side helper for blocks of 32 E2M1 codes.
struct Fp4BlockQuantizer {
    static constexpr float MAX_VALUE = 6.0f;
    static constexpr size_t REQUIRED_BLOCK_SIZE = 32;
    size_t block_size;
    explicit Fp4BlockQuantizer(size_t block_size) : block_size(block_size) {
        if (block_size != REQUIRED_BLOCK_SIZE) throw DnnError("InvalidArgument", "NVFP4/OCP MXFP4 block size must be 32, got " + std::to_string(block_size));
    }
    // max |x| / 6, or 1 for an all-zero block; NaN elements are skipped as f32::max skips them
    float compute_scale(const std::vector<float>& block) const {
        float max_abs = 0.0f;
        for (float v : block) { const float a = v < 0.0f ? -v : v; if (a > max_abs) max_abs = a; }
        return max_abs == 0.0f ? 1.0f : max_abs / MAX_VALUE;
    }
    size_t num_scales(size_t n) const { return (n + block_size - 1) / block_size; }
};

}  // namespace oxicuda_dnn
