// Host-side mirror of the oxicuda-quant quantizer types over the C ABI of liboxq_b200 (include/oxq.h).
// Same names, argument meaning and error behaviour as the reference (crates/oxicuda-quant/src/scheme/minmax.rs,
// scheme/fp8.rs, error.rs); the arithmetic runs on the GPU.  Host-slice methods stage through device buffers
// (H2D, kernel, D2H) exactly as the reference's signatures imply; *_device methods take device pointers.
// Header-only; link with -loxq_b200 -lcudart.  There is no CPU fallback: without a device every call throws.
#pragma once
#include <cuda_runtime.h>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>
#include "../../include/oxq.h"

namespace oxicuda_quant {

// QuantError (error.rs:10-58): `variant` carries the enum variant name.
struct QuantError : std::runtime_error {
    std::string variant;
    QuantError(const std::string& v, const std::string& msg) : std::runtime_error(v + ": " + msg), variant(v) {}
};

enum class QuantScheme { Symmetric, Asymmetric };                       // minmax.rs:27-33
struct QuantGranularity {                                               // minmax.rs:37-44
    enum Kind { PerTensor, PerChannel, PerGroup } kind = PerTensor;
    size_t channel_axis = 0, group_size = 0;
    static QuantGranularity per_tensor() { return {}; }
    static QuantGranularity per_channel(size_t axis) { QuantGranularity g; g.kind = PerChannel; g.channel_axis = axis; return g; }
    static QuantGranularity per_group(size_t gs) { QuantGranularity g; g.kind = PerGroup; g.group_size = gs; return g; }
};
struct QuantParams {                                                    // minmax.rs:50-79
    std::vector<float> scales;
    std::vector<int32_t> zero_points;
    uint32_t bits = 8;
    QuantScheme scheme = QuantScheme::Symmetric;
    float q_max() const { return scheme == QuantScheme::Symmetric ? float(1 << (bits - 1)) - 1.0f : float(1 << bits) - 1.0f; }
    float q_min() const { return scheme == QuantScheme::Symmetric ? -float(1 << (bits - 1)) : 0.0f; }
};

namespace detail {
inline void check(int32_t rc, oxq_handle* h) {
    if (rc == OXQ_OK) return;
    throw QuantError(oxq_status_name(rc), h ? oxq_last_error_string(h) : "");
}
inline void cuda(cudaError_t e) { if (e != cudaSuccess) throw QuantError("Cuda", cudaGetErrorString(e)); }
template <typename T> struct DevBuf {
    T* p = nullptr; size_t n = 0;
    explicit DevBuf(size_t count) : n(count) { if (n) cuda(cudaMalloc(&p, n * sizeof(T))); }
    ~DevBuf() { if (p) cudaFree(p); }
    DevBuf(const DevBuf&) = delete; DevBuf& operator=(const DevBuf&) = delete;
    void upload(const T* h) { if (n) cuda(cudaMemcpy(p, h, n * sizeof(T), cudaMemcpyHostToDevice)); }
    void download(T* h) const { if (n) cuda(cudaMemcpy(h, p, n * sizeof(T), cudaMemcpyDeviceToHost)); }
};
struct Handle {                                                          // owns one oxq_handle on the default stream
    oxq_handle* h = nullptr;
    explicit Handle(int device = 0) { check(oxq_handle_create(device, nullptr, &h), nullptr); }
    ~Handle() { if (h) oxq_handle_destroy(h); }
    Handle(const Handle&) = delete; Handle& operator=(const Handle&) = delete;
};
}  // namespace detail

// MinMaxQuantizer (minmax.rs:86-324).  The accelerated configurations are the two the hot path names:
// 8-bit symmetric per channel (calibrate_2d + quantize_grouped(group = cols)) and 4-bit asymmetric per group
// (f16 scales on the device side; see quantize_int4_per_group).  rounding follows OXQ_ROUND_*.
class MinMaxQuantizer {
public:
    MinMaxQuantizer(uint32_t bits, QuantScheme scheme, QuantGranularity gran, int rounding = OXQ_ROUND_HALF_AWAY)
        : bits_(bits), scheme_(scheme), gran_(gran), rounding_(rounding) {
        if (bits == 0 || bits > 16) throw std::invalid_argument("bits must be in [1, 16]");   // new() panics, minmax.rs:99-100
    }
    static MinMaxQuantizer int8_symmetric() { return {8, QuantScheme::Symmetric, QuantGranularity::per_tensor()}; }
    static MinMaxQuantizer int4_per_group(size_t g) { return {4, QuantScheme::Symmetric, QuantGranularity::per_group(g)}; }

    // calibrate_2d + quantize_grouped(group = cols) in one pass over the data: returns per-row params and int8 codes
    // widened to i32 as the reference's Vec<i32>.  (minmax.rs:179-207, :275-299)
    QuantParams calibrate_quantize_2d(const std::vector<float>& t, size_t rows, size_t cols, std::vector<int32_t>& codes) const {
        if (rows == 0) throw QuantError("EmptyInput", "calibrate_2d: rows == 0");
        if (cols == 0) throw QuantError("DimensionMismatch", "dimension mismatch: expected 1, got 0");
        if (bits_ != 8 || scheme_ != QuantScheme::Symmetric) throw QuantError("InvalidConfig", "device path covers 8-bit symmetric per channel");
        if (t.size() != rows * cols) throw QuantError("DimensionMismatch", "tensor length != rows * cols");
        detail::Handle h;
        detail::DevBuf<float> x(rows * cols), s(rows);
        detail::DevBuf<int8_t> q(rows * cols);
        x.upload(t.data());
        detail::check(oxq_int8_quant_rows(h.h, x.p, (int64_t)rows, (int64_t)cols, q.p, s.p, rounding_), h.h);
        detail::cuda(cudaDeviceSynchronize());
        QuantParams p;
        p.bits = 8; p.scheme = QuantScheme::Symmetric;
        p.scales.resize(rows); p.zero_points.assign(rows, 0);
        s.download(p.scales.data());
        for (float sc : p.scales)                                        // minmax.rs:234-236
            if (!std::isfinite(sc) || sc <= 0.0f) throw QuantError("InvalidScale", "invalid scale " + std::to_string(sc));
        std::vector<int8_t> q8(rows * cols);
        q.download(q8.data());
        codes.assign(q8.begin(), q8.end());
        return p;
    }
    // dequantize_grouped (minmax.rs:309-324) for the per-row INT8 case
    std::vector<float> dequantize_2d(const std::vector<int32_t>& codes, const QuantParams& p, size_t rows, size_t cols) const {
        detail::Handle h;
        std::vector<int8_t> q8(codes.begin(), codes.end());
        detail::DevBuf<int8_t> q(rows * cols);
        detail::DevBuf<float> s(rows), y(rows * cols);
        q.upload(q8.data()); s.upload(p.scales.data());
        detail::check(oxq_int8_dequant_rows(h.h, q.p, s.p, (int64_t)rows, (int64_t)cols, y.p), h.h);
        detail::cuda(cudaDeviceSynchronize());
        std::vector<float> out(rows * cols);
        y.download(out.data());
        return out;
    }
private:
    uint32_t bits_; QuantScheme scheme_; QuantGranularity gran_; int rounding_;
};

// Fp8Codec (fp8.rs:84-159), E4M3.  `refcompat` selects the literal reference bit manipulation; otherwise the
// hardware RNE/satfinite conversion.  Non-finite input is always an error (fp8.rs:116-118).
class Fp8Codec {
public:
    explicit Fp8Codec(bool refcompat = false) : mode_(refcompat ? OXQ_FP8_REFCOMPAT : OXQ_FP8_SPEC_RNE) {}
    static Fp8Codec e4m3() { return Fp8Codec(false); }
    std::vector<uint8_t> encode(const std::vector<float>& data) const {
        for (float v : data) if (!std::isfinite(v)) throw QuantError("NonFiniteFp8", "FP8 encoding received non-finite value");
        if (data.empty()) return {};
        detail::Handle h;
        detail::DevBuf<float> x(data.size()), one(1);
        detail::DevBuf<uint8_t> q(data.size());
        const float unit = 1.0f;
        x.upload(data.data()); one.upload(&unit);
        detail::check(oxq_fp8_quant(h.h, x.p, OXQ_F32, (int64_t)data.size(), one.p, q.p, mode_), h.h);
        detail::cuda(cudaDeviceSynchronize());
        std::vector<uint8_t> out(data.size());
        q.download(out.data());
        return out;
    }
    std::vector<float> decode(const std::vector<uint8_t>& data) const {
        if (data.empty()) return {};
        detail::Handle h;
        detail::DevBuf<uint8_t> q(data.size());
        detail::DevBuf<float> y(data.size()), one(1);
        const float unit = 1.0f;
        q.upload(data.data()); one.upload(&unit);
        detail::check(oxq_fp8_dequant(h.h, q.p, (int64_t)data.size(), one.p, y.p, OXQ_F32, mode_), h.h);
        detail::cuda(cudaDeviceSynchronize());
        std::vector<float> out(data.size());
        y.download(out.data());
        return out;
    }
private:
    int mode_;
};

// Nf4Quantizer (crates/oxicuda-quant/src/scheme/nf4.rs:56-172): blocks of `block_size` elements share an absmax.
class Nf4Quantizer {
public:
    explicit Nf4Quantizer(size_t block_size = 64) : block_size(block_size) {
        if (block_size == 0) throw std::invalid_argument("block_size must be > 0");          // the reference panics
    }
    size_t block_size;
    // (packed bytes, per-block absmax)
    std::pair<std::vector<uint8_t>, std::vector<float>> encode(const std::vector<float>& tensor) const {
        if (tensor.empty()) throw QuantError("EmptyInput", "Nf4Quantizer::encode");
        if (tensor.size() % block_size != 0) throw QuantError("GroupSizeMismatch", "length is not a multiple of the block size");
        detail::Handle h;
        detail::DevBuf<float> x(tensor.size()), am(tensor.size() / block_size);
        detail::DevBuf<uint8_t> packed(tensor.size() / 2);
        x.upload(tensor.data());
        detail::check(oxq_nf4_quant(h.h, x.p, (int64_t)tensor.size(), (int64_t)block_size, packed.p, am.p), h.h);
        detail::cuda(cudaDeviceSynchronize());
        std::pair<std::vector<uint8_t>, std::vector<float>> out{std::vector<uint8_t>(tensor.size() / 2), std::vector<float>(tensor.size() / block_size)};
        packed.download(out.first.data());
        am.download(out.second.data());
        return out;
    }
    std::vector<float> decode(const std::vector<uint8_t>& packed, const std::vector<float>& absmaxs) const {
        const size_t n = packed.size() * 2;
        if (absmaxs.size() != n / block_size) throw QuantError("DimensionMismatch", "absmax count does not match the packed length");
        if (n == 0) return {};
        detail::Handle h;
        detail::DevBuf<uint8_t> p(packed.size());
        detail::DevBuf<float> am(absmaxs.size()), y(n);
        p.upload(packed.data()); am.upload(absmaxs.data());
        detail::check(oxq_nf4_dequant(h.h, p.p, am.p, (int64_t)n, (int64_t)block_size, y.p, OXQ_F32), h.h);
        detail::cuda(cudaDeviceSynchronize());
        std::vector<float> out(n);
        y.download(out.data());
        return out;
    }
    float quantization_mse(const std::vector<float>& tensor) const {
        auto enc = encode(tensor);
        std::vector<float> dec = decode(enc.first, enc.second);
        double acc = 0.0;
        for (size_t i = 0; i < tensor.size(); i++) acc += (double)(tensor[i] - dec[i]) * (double)(tensor[i] - dec[i]);
        return (float)(acc / (double)tensor.size());
    }
};

// BlockQuantizedInt8 (crates/oxicuda-dnn/src/quantize/int8_quantize.rs:387-471).
struct BlockQuantizedInt8 {
    std::vector<int8_t> data;
    std::vector<float> scales;
    size_t block_size = 0, orig_len = 0;
    static BlockQuantizedInt8 quantize(const std::vector<float>& input, size_t block_size) {
        if (block_size == 0) throw std::invalid_argument("block_size must be > 0");
        BlockQuantizedInt8 r;
        r.block_size = block_size; r.orig_len = input.size();
        r.data.resize(input.size());
        r.scales.resize((input.size() + block_size - 1) / block_size);
        if (input.empty()) return r;
        detail::Handle h;
        detail::DevBuf<float> x(input.size()), s(r.scales.size());
        detail::DevBuf<int8_t> q(input.size());
        x.upload(input.data());
        detail::check(oxq_int8_block_quant(h.h, x.p, (int64_t)input.size(), (int64_t)block_size, q.p, s.p), h.h);
        detail::cuda(cudaDeviceSynchronize());
        q.download(r.data.data());
        s.download(r.scales.data());
        return r;
    }
    std::vector<float> dequantize() const {
        std::vector<float> out(orig_len);
        if (orig_len == 0) return out;
        detail::Handle h;
        detail::DevBuf<int8_t> q(orig_len);
        detail::DevBuf<float> s(scales.size()), y(orig_len);
        q.upload(data.data()); s.upload(scales.data());
        detail::check(oxq_int8_block_dequant(h.h, q.p, s.p, (int64_t)orig_len, (int64_t)block_size, y.p), h.h);
        detail::cuda(cudaDeviceSynchronize());
        y.download(out.data());
        return out;
    }
    size_t num_blocks() const { return scales.size(); }
    float compression_ratio() const {
        const size_t qb = data.size() + scales.size() * 4;
        return qb == 0 ? 1.0f : (float)(orig_len * 4) / (float)qb;
    }
};

// SmoothQuantMigrator (crates/oxicuda-quant/src/scheme/smooth_quant.rs:54-293).  Activations are [n_tokens x n_channels],
// weights [n_out x n_channels], both row-major f32 host slices staged through device buffers; the checks and their order
// are the reference's.
struct SmoothQuantConfig { float alpha = 0.5f; };
class SmoothQuantMigrator {
public:
    explicit SmoothQuantMigrator(float alpha) { config.alpha = alpha; }
    SmoothQuantConfig config;
    // s[j] = max(|act_max[j]|, 1e-8)^alpha / max(|weight_max[j]|, 1e-8)^(1 - alpha)        (smooth_quant.rs:84-113)
    std::vector<float> compute_migration_scales(const std::vector<float>& act_max, const std::vector<float>& weight_max) const {
        if (act_max.empty()) throw QuantError("EmptyInput", "SmoothQuantMigrator::compute_migration_scales");
        if (act_max.size() != weight_max.size())
            throw QuantError("DimensionMismatch", "dimension mismatch: expected " + std::to_string(act_max.size()) + ", got " + std::to_string(weight_max.size()));
        detail::Handle h;
        detail::DevBuf<float> a(act_max.size()), w(weight_max.size()), s(act_max.size());
        a.upload(act_max.data()); w.upload(weight_max.data());
        detail::check(oxq_smooth_scales(h.h, a.p, w.p, (int64_t)act_max.size(), config.alpha, s.p), h.h);
        detail::cuda(cudaDeviceSynchronize());
        std::vector<float> out(act_max.size());
        s.download(out.data());
        return out;
    }
    // per-channel max |x| over the rows                                                    (smooth_quant.rs:125-196)
    static std::vector<float> compute_act_stats(const std::vector<float>& acts, size_t n_tokens, size_t n_channels) {
        return col_absmax(acts, n_tokens, n_channels, "compute_act_stats: empty activations");
    }
    static std::vector<float> compute_weight_stats(const std::vector<float>& weights, size_t n_out, size_t n_channels) {
        return col_absmax(weights, n_out, n_channels, "compute_weight_stats: empty weights");
    }
    // acts[t, j] /= max(scales[j], 1e-12), in place                                        (smooth_quant.rs:198-222)
    static void smooth_activations(std::vector<float>& acts, const std::vector<float>& scales, size_t n_tokens, size_t n_channels) {
        apply(acts, scales, n_tokens, n_channels, 1);
    }
    // weights[r, j] *= scales[j], in place                                                 (smooth_quant.rs:231-254)
    static void smooth_weights(std::vector<float>& weights, const std::vector<float>& scales, size_t n_out, size_t n_channels) {
        apply(weights, scales, n_out, n_channels, 0);
    }
    // statistics, scales and both in-place updates; returns the scales                     (smooth_quant.rs:274-293)
    std::vector<float> smooth_layer(std::vector<float>& acts, std::vector<float>& weights, size_t n_tokens, size_t n_channels, size_t n_out) const {
        const std::vector<float> act_stats = compute_act_stats(acts, n_tokens, n_channels);
        const std::vector<float> weight_stats = compute_weight_stats(weights, n_out, n_channels);
        const std::vector<float> scales = compute_migration_scales(act_stats, weight_stats);
        smooth_activations(acts, scales, n_tokens, n_channels);
        smooth_weights(weights, scales, n_out, n_channels);
        return scales;
    }
private:
    static std::vector<float> col_absmax(const std::vector<float>& x, size_t rows, size_t cols, const char* empty_msg) {
        if (x.empty()) throw QuantError("EmptyInput", empty_msg);
        if (x.size() != rows * cols)
            throw QuantError("DimensionMismatch", "dimension mismatch: expected " + std::to_string(rows * cols) + ", got " + std::to_string(x.size()));
        detail::Handle h;
        detail::DevBuf<float> d(x.size()), st(cols);
        d.upload(x.data());
        detail::check(oxq_smooth_col_absmax(h.h, d.p, (int64_t)rows, (int64_t)cols, st.p), h.h);
        detail::cuda(cudaDeviceSynchronize());
        std::vector<float> out(cols);
        st.download(out.data());
        return out;
    }
    static void apply(std::vector<float>& x, const std::vector<float>& scales, size_t rows, size_t cols, int divide) {
        if (x.size() != rows * cols)
            throw QuantError("DimensionMismatch", "dimension mismatch: expected " + std::to_string(rows * cols) + ", got " + std::to_string(x.size()));
        if (scales.size() != cols)
            throw QuantError("DimensionMismatch", "dimension mismatch: expected " + std::to_string(cols) + ", got " + std::to_string(scales.size()));
        if (x.empty()) return;                                            // the reference's loops run zero times
        detail::Handle h;
        detail::DevBuf<float> d(x.size()), s(cols);
        d.upload(x.data()); s.upload(scales.data());
        detail::check(oxq_smooth_apply(h.h, d.p, (int64_t)rows, (int64_t)cols, s.p, divide), h.h);
        detail::cuda(cudaDeviceSynchronize());
        d.download(x.data());
    }
};

// GptqConfig / GptqOutput / GptqQuantizer (crates/oxicuda-quant/src/scheme/gptq.rs:30-257): the whole layer is
// quantized on the device by oxq_gptq_quantize_layer; results equal the reference's CPU loop bit for bit.
struct GptqConfig {
    uint32_t bits = 4;
    size_t block_size = 128;                                              // unused by the reference's algorithm as well
    double percdamp = 0.01;
    bool symmetric = true;
};
struct GptqOutput {
    std::vector<int32_t> quantized;
    std::vector<float> scales;
    std::vector<int32_t> zero_points;
    size_t n_rows = 0, n_cols = 0;
    std::vector<float> dequantize() const {
        std::vector<float> out(n_rows * n_cols);
        for (size_t i = 0; i < n_rows; i++)
            for (size_t j = 0; j < n_cols; j++) out[i * n_cols + j] = ((float)quantized[i * n_cols + j] - (float)zero_points[j]) * scales[j];
        return out;
    }
    float reconstruction_mse(const std::vector<float>& original) const {
        const std::vector<float> deq = dequantize();
        float acc = 0.0f;
        for (size_t i = 0; i < deq.size() && i < original.size(); i++) acc += (deq[i] - original[i]) * (deq[i] - original[i]);
        return acc / (float)(deq.empty() ? 1 : deq.size());
    }
};
class GptqQuantizer {
public:
    explicit GptqQuantizer(const GptqConfig& config = GptqConfig()) : config(config) {}
    GptqConfig config;
    GptqOutput quantize_layer(const std::vector<float>& weights, size_t n_rows, size_t n_cols, const std::vector<float>& hessian) const {
        if (weights.empty()) throw QuantError("EmptyInput", "GptqQuantizer::quantize_layer");
        if (weights.size() != n_rows * n_cols) throw QuantError("DimensionMismatch", "weights length does not match n_rows * n_cols");
        if (hessian.size() != n_cols * n_cols) throw QuantError("DimensionMismatch", "hessian length does not match n_cols * n_cols");
        if (config.bits == 0 || config.bits > 16) throw QuantError("InvalidBitWidth", "bits must be in 1..=16");
        detail::Handle h;
        size_t ws_bytes = 0;
        detail::check(oxq_gptq_workspace_bytes((int64_t)n_rows, (int64_t)n_cols, &ws_bytes), h.h);
        detail::DevBuf<float> w(weights.size()), hs(hessian.size()), sc(n_cols);
        detail::DevBuf<int32_t> q(weights.size()), zp(n_cols), info(2);
        detail::DevBuf<uint8_t> ws(ws_bytes);
        w.upload(weights.data()); hs.upload(hessian.data());
        detail::check(oxq_gptq_quantize_layer(h.h, w.p, (int64_t)n_rows, (int64_t)n_cols, hs.p, (int)config.bits, config.symmetric ? 1 : 0,
                                              config.percdamp, q.p, sc.p, zp.p, info.p, ws.p, ws_bytes), h.h);
        detail::cuda(cudaDeviceSynchronize());
        int32_t host_info[2] = {0, 0};
        info.download(host_info);
        if (host_info[0] != 0) {
            float md; memcpy(&md, &host_info[1], sizeof(md));
            throw QuantError("SingularHessian", "min diagonal = " + std::to_string(md));
        }
        GptqOutput out;
        out.n_rows = n_rows; out.n_cols = n_cols;
        out.quantized.resize(weights.size()); out.scales.resize(n_cols); out.zero_points.resize(n_cols);
        q.download(out.quantized.data()); sc.download(out.scales.data()); zp.download(out.zero_points.data());
        return out;
    }
};

}  // namespace oxicuda_quant
