// Host-side mirror of the tensor-parallel linear layers of oxicuda-dist-infer over the C ABI of liboxq_b200:
//   ParallelismConfig, RankCoordinates, DistInferHandle   crates/oxicuda-dist-infer/src/handle.rs:40-240
//   ColumnLinear (from_full_weight, local_forward, all_gather)               tensor_parallel/column_parallel.rs:103-204
//   RowLinear (from_full_weight, slice_input, local_forward, all_reduce)     tensor_parallel/row_parallel.rs:97-223
//   TpSwiGluMlp: SwiGluFfn (crates/oxicuda-lm/src/layer/ffn.rs:202-254) over weights cut the same way, FP8, one fused call
// Same names, argument meaning, check order and error variants as the reference.  The reference computes the shard's
// product with f32 loops on the CPU; here the shard lives on the GPU as bf16 and the product is one tensor-core GEMM
// (oxq_gemm_bf16, f32 accumulation, bf16 result) followed by the bias add (oxq_bias_add_bf16).  Host slices are
// converted to bf16 (round to nearest even) and staged through device buffers; *_device methods take device pointers.
// The static all_gather / all_reduce are the reference's host-side helpers over a list of per-rank results; on device
// buffers the collectives are oxq_all_gather_bf16 / oxq_all_reduce_bf16 on a handle that holds a communicator.
// Header-only; link with -loxq_b200 -lcudart.  There is no CPU fallback: without a device every forward throws.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>
#include <cstring>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>
#include "../../include/oxq.h"

namespace oxicuda_dist_infer {

struct DistInferError : std::runtime_error {
    std::string variant;
    size_t a = 0, b = 0;                                                  // the variant's two numbers, in declaration order
    DistInferError(const std::string& v, const std::string& msg, size_t a_ = 0, size_t b_ = 0)
        : std::runtime_error(v + ": " + msg), variant(v), a(a_), b(b_) {}
};

struct SmVersion { uint32_t value; };

struct ParallelismConfig {                                                // handle.rs:40-75
    size_t tp = 1, sp = 1, ep = 1;
    size_t world_size() const { return tp * sp * ep; }
    void validate() const {
        if (tp == 0 || sp == 0 || ep == 0) throw DistInferError("InvalidWorldSize", "all parallelism degrees must be >= 1", tp * sp * ep);
    }
};

struct RankCoordinates {                                                  // handle.rs:96-150: tp is the fastest-varying axis
    size_t tp_rank = 0, sp_rank = 0, ep_rank = 0, global_rank = 0;
    static RankCoordinates from_global(size_t global_rank, const ParallelismConfig& c) {
        const size_t ws = c.world_size();
        if (global_rank >= ws) throw DistInferError("RankOutOfRange", "rank " + std::to_string(global_rank) + " outside a world of " + std::to_string(ws), global_rank, ws);
        return {global_rank % c.tp, (global_rank / c.tp) % c.sp, global_rank / (c.tp * c.sp), global_rank};
    }
    size_t to_global(const ParallelismConfig& c) const { return ep_rank * (c.tp * c.sp) + sp_rank * c.tp + tp_rank; }
    size_t peer_tp(size_t r, const ParallelismConfig& c) const { return ep_rank * (c.tp * c.sp) + sp_rank * c.tp + r; }
    size_t peer_sp(size_t r, const ParallelismConfig& c) const { return ep_rank * (c.tp * c.sp) + r * c.tp + tp_rank; }
    size_t peer_ep(size_t r, const ParallelismConfig& c) const { return r * (c.tp * c.sp) + sp_rank * c.tp + tp_rank; }
};

struct DistInferHandle {                                                  // handle.rs:159-240
    int device = 0;
    SmVersion sm_version{100};
    ParallelismConfig config;
    RankCoordinates coords;
    DistInferHandle(int device, SmVersion sm, size_t global_rank, const ParallelismConfig& cfg) : device(device), sm_version(sm), config(cfg) {
        config.validate();
        coords = RankCoordinates::from_global(global_rank, config);
    }
    static DistInferHandle single_rank(uint32_t sm) { return DistInferHandle(0, SmVersion{sm}, 0, ParallelismConfig()); }
    size_t world_size() const { return config.world_size(); }
    size_t global_rank() const { return coords.global_rank; }
    size_t tp_rank() const { return coords.tp_rank; }
    size_t sp_rank() const { return coords.sp_rank; }
    size_t ep_rank() const { return coords.ep_rank; }
};

namespace detail {
inline void cuda(cudaError_t e) { if (e != cudaSuccess) throw DistInferError("Cuda", cudaGetErrorString(e)); }
inline uint16_t f32_to_bf16(float f) {                                    // round to nearest even; NaN stays NaN
    uint32_t u; std::memcpy(&u, &f, 4);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return uint16_t((u >> 16) | 0x0040u);
    return uint16_t((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
}
inline float bf16_to_f32(uint16_t b) { const uint32_t u = uint32_t(b) << 16; float f; std::memcpy(&f, &u, 4); return f; }
inline size_t round_up(size_t v, size_t to) { return (v + to - 1) / to * to; }

// One rank's shard on the GPU: bf16 weight [n_pad x k_pad] (zero padding: k to a multiple of 64, n to a multiple of 8,
// so that every row is a whole number of 16-byte units whatever the layer's sizes), optional f32 bias [n_pad].
struct DeviceShard {
    oxq_handle* h = nullptr;
    void* w = nullptr; float* bias = nullptr;
    size_t n = 0, k = 0, n_pad = 0, k_pad = 0;
    DeviceShard(int device, const float* weight, size_t n_, size_t k_, size_t src_ld, const float* bias_or_null) : n(n_), k(k_) {
        n_pad = round_up(n, 8); k_pad = round_up(k, 64);
        cuda(cudaSetDevice(device));
        const int32_t rc = oxq_handle_create(device, nullptr, &h);
        if (rc) throw DistInferError(oxq_status_name(rc), "oxq_handle_create");
        try {
            std::vector<uint16_t> wb(n_pad * k_pad, 0);
            for (size_t r = 0; r < n; r++)
                for (size_t c = 0; c < k; c++) wb[r * k_pad + c] = f32_to_bf16(weight[r * src_ld + c]);
            cuda(cudaMalloc(&w, wb.size() * 2));
            cuda(cudaMemcpy(w, wb.data(), wb.size() * 2, cudaMemcpyHostToDevice));
            if (bias_or_null) {
                std::vector<float> bb(n_pad, 0.0f);
                for (size_t i = 0; i < n; i++) bb[i] = bias_or_null[i];
                cuda(cudaMalloc((void**)&bias, n_pad * sizeof(float)));
                cuda(cudaMemcpy(bias, bb.data(), n_pad * sizeof(float), cudaMemcpyHostToDevice));
            }
        } catch (...) { release(); throw; }                               // a constructor that throws runs no destructor
    }
    ~DeviceShard() { release(); }
    void release() {
        if (w) cudaFree(w);
        if (bias) cudaFree(bias);
        if (h) oxq_handle_destroy(h);
        w = nullptr; bias = nullptr; h = nullptr;
    }
    DeviceShard(const DeviceShard&) = delete; DeviceShard& operator=(const DeviceShard&) = delete;
    void check(int32_t rc) const { if (rc) throw DistInferError(oxq_status_name(rc), oxq_last_error_string(h)); }
    // y[batch x n_pad] (bf16, ld = n_pad) = x[batch x k_pad] (bf16, ld = k_pad) . W^T (+ bias); asynchronous on the handle's stream
    void forward_device(const void* x_bf16_dev, size_t batch, void* y_bf16_dev) const {
        check(oxq_gemm_bf16(h, (int64_t)batch, (int64_t)n_pad, (int64_t)k_pad, x_bf16_dev, (int64_t)k_pad, w, (int64_t)k_pad, y_bf16_dev, (int64_t)n_pad));
        if (bias) check(oxq_bias_add_bf16(h, y_bf16_dev, (int64_t)n_pad, bias, (int64_t)batch, (int64_t)n_pad));
    }
    // host slices: x [batch x k] f32 -> [batch x n] f32
    std::vector<float> forward_host(const float* x, size_t batch) const {
        std::vector<uint16_t> xb(batch * k_pad, 0);
        for (size_t r = 0; r < batch; r++)
            for (size_t c = 0; c < k; c++) xb[r * k_pad + c] = f32_to_bf16(x[r * k + c]);
        void *xd = nullptr, *yd = nullptr;
        cuda(cudaMalloc(&xd, xb.size() * 2));
        cuda(cudaMalloc(&yd, batch * n_pad * 2));
        std::vector<uint16_t> yb(batch * n_pad);
        try {
            cuda(cudaMemcpy(xd, xb.data(), xb.size() * 2, cudaMemcpyHostToDevice));
            forward_device(xd, batch, yd);
            cuda(cudaDeviceSynchronize());
            cuda(cudaMemcpy(yb.data(), yd, yb.size() * 2, cudaMemcpyDeviceToHost));
        } catch (...) { cudaFree(xd); cudaFree(yd); throw; }
        cudaFree(xd); cudaFree(yd);
        std::vector<float> out(batch * n);
        for (size_t r = 0; r < batch; r++)
            for (size_t c = 0; c < n; c++) out[r * n + c] = bf16_to_f32(yb[r * n_pad + c]);
        return out;
    }
};
}  // namespace detail

// Rank r owns output rows [r * total_out / tp, (r + 1) * total_out / tp) of W [total_out x in_features].
class ColumnLinear {
public:
    DistInferHandle handle;
    size_t in_features = 0, local_out = 0, col_offset = 0, total_out = 0;
    static ColumnLinear from_full_weight(const DistInferHandle& handle, size_t in_features, size_t total_out, const std::vector<float>& weight,
                                         const std::vector<float>* bias = nullptr) {
        const size_t tp = handle.config.tp;
        if (total_out % tp != 0) throw DistInferError("TpFeaturesMisaligned", "features " + std::to_string(total_out) + " not divisible by degree " + std::to_string(tp), total_out, tp);
        ColumnLinear l(handle);
        l.in_features = in_features; l.total_out = total_out;
        l.local_out = total_out / tp; l.col_offset = handle.tp_rank() * l.local_out;
        if (weight.size() != total_out * in_features)
            throw DistInferError("DimensionMismatch", "expected " + std::to_string(total_out * in_features) + ", got " + std::to_string(weight.size()), total_out * in_features, weight.size());
        if (bias && bias->size() != total_out)
            throw DistInferError("DimensionMismatch", "expected " + std::to_string(total_out) + ", got " + std::to_string(bias->size()), total_out, bias->size());
        if (l.local_out == 0 || in_features == 0) throw DistInferError("ShardShapeMismatch", "empty shard", l.local_out, in_features);
        l.shard_ = std::make_shared<detail::DeviceShard>(handle.device, weight.data() + l.col_offset * in_features, l.local_out, in_features, in_features,
                                                         bias ? bias->data() + l.col_offset : nullptr);
        return l;
    }
    // input [batch x in_features] -> this rank's [batch x local_out]
    std::vector<float> local_forward(const std::vector<float>& input, size_t batch) const {
        if (input.size() != batch * in_features)
            throw DistInferError("DimensionMismatch", "expected " + std::to_string(batch * in_features) + ", got " + std::to_string(input.size()), batch * in_features, input.size());
        if (batch == 0) return {};
        return shard_->forward_host(input.data(), batch);
    }
    // device form: x bf16 [batch x k_pad()], y bf16 [batch x n_pad()], asynchronous on library_handle()'s stream
    void local_forward_device(const void* x_bf16_dev, size_t batch, void* y_bf16_dev) const { shard_->forward_device(x_bf16_dev, batch, y_bf16_dev); }
    size_t k_pad() const { return shard_->k_pad; }
    size_t n_pad() const { return shard_->n_pad; }
    oxq_handle* library_handle() const { return shard_->h; }
    // the reference's host-side all-gather: shard r's columns land at [r * local_out, (r + 1) * local_out)
    static std::vector<float> all_gather(size_t total_out, size_t batch, const std::vector<std::vector<float>>& shards) {
        const size_t tp = shards.size();
        if (tp == 0) throw DistInferError("TooFewRanks", "needed 1, world_size 0", 1, 0);
        const size_t local_out = total_out / tp;
        std::vector<float> out(batch * total_out, 0.0f);
        for (size_t rank = 0; rank < tp; rank++)
            for (size_t b = 0; b < batch; b++)
                for (size_t o = 0; o < local_out; o++) out[b * total_out + rank * local_out + o] = shards[rank][b * local_out + o];
        return out;
    }
private:
    explicit ColumnLinear(const DistInferHandle& h) : handle(h) {}
    std::shared_ptr<detail::DeviceShard> shard_;
};

// Rank r owns input columns [r * total_in / tp, (r + 1) * total_in / tp) of W [out_features x total_in]; the bias lives on
// rank 0 only, so the sum over ranks counts it once.
class RowLinear {
public:
    DistInferHandle handle;
    size_t out_features = 0, total_in = 0, local_in = 0, row_offset = 0;
    bool has_bias = false;
    static RowLinear from_full_weight(const DistInferHandle& handle, size_t out_features, size_t total_in, const std::vector<float>& weight,
                                      const std::vector<float>* bias = nullptr) {
        const size_t tp = handle.config.tp;
        if (total_in % tp != 0) throw DistInferError("TpInputMisaligned", "features " + std::to_string(total_in) + " not divisible by degree " + std::to_string(tp), total_in, tp);
        RowLinear l(handle);
        l.out_features = out_features; l.total_in = total_in;
        l.local_in = total_in / tp; l.row_offset = handle.tp_rank() * l.local_in;
        if (weight.size() != out_features * total_in)
            throw DistInferError("DimensionMismatch", "expected " + std::to_string(out_features * total_in) + ", got " + std::to_string(weight.size()), out_features * total_in, weight.size());
        const float* b = nullptr;
        if (handle.tp_rank() == 0 && bias) {
            if (bias->size() != out_features)
                throw DistInferError("DimensionMismatch", "expected " + std::to_string(out_features) + ", got " + std::to_string(bias->size()), out_features, bias->size());
            b = bias->data();
        }
        l.has_bias = b != nullptr;
        if (out_features == 0 || l.local_in == 0) throw DistInferError("ShardShapeMismatch", "empty shard", out_features, l.local_in);
        l.shard_ = std::make_shared<detail::DeviceShard>(handle.device, weight.data() + l.row_offset, out_features, l.local_in, total_in, b);
        return l;
    }
    // this rank's columns of full_input [batch x total_in]
    std::vector<float> slice_input(const std::vector<float>& full_input, size_t batch) const {
        if (full_input.size() != batch * total_in)
            throw DistInferError("DimensionMismatch", "expected " + std::to_string(batch * total_in) + ", got " + std::to_string(full_input.size()), batch * total_in, full_input.size());
        std::vector<float> s(batch * local_in);
        for (size_t b = 0; b < batch; b++)
            for (size_t i = 0; i < local_in; i++) s[b * local_in + i] = full_input[b * total_in + row_offset + i];
        return s;
    }
    // input_slice [batch x local_in] -> this rank's partial [batch x out_features]
    std::vector<float> forward_partial(const std::vector<float>& input_slice, size_t batch) const {
        if (input_slice.size() != batch * local_in)
            throw DistInferError("DimensionMismatch", "expected " + std::to_string(batch * local_in) + ", got " + std::to_string(input_slice.size()), batch * local_in, input_slice.size());
        if (batch == 0) return {};
        return shard_->forward_host(input_slice.data(), batch);
    }
    std::vector<float> local_forward(const std::vector<float>& full_input, size_t batch) const { return forward_partial(slice_input(full_input, batch), batch); }
    void forward_partial_device(const void* x_slice_bf16_dev, size_t batch, void* y_bf16_dev) const { shard_->forward_device(x_slice_bf16_dev, batch, y_bf16_dev); }
    size_t k_pad() const { return shard_->k_pad; }
    size_t n_pad() const { return shard_->n_pad; }
    oxq_handle* library_handle() const { return shard_->h; }
    // the reference's host-side all-reduce: partials summed in rank order
    static std::vector<float> all_reduce(const std::vector<std::vector<float>>& partials) {
        if (partials.empty()) throw DistInferError("TooFewRanks", "needed 1, world_size 0", 1, 0);
        std::vector<float> acc = partials[0];
        for (size_t r = 1; r < partials.size(); r++) {
            if (partials[r].size() != acc.size())
                throw DistInferError("DimensionMismatch", "expected " + std::to_string(acc.size()) + ", got " + std::to_string(partials[r].size()), acc.size(), partials[r].size());
            for (size_t i = 0; i < acc.size(); i++) acc[i] += partials[r][i];
        }
        return acc;
    }
private:
    explicit RowLinear(const DistInferHandle& h) : handle(h) {}
    std::shared_ptr<detail::DeviceShard> shard_;
};

// One rank's shard of a tensor-parallel SwiGLU MLP with FP8 (E4M3) weights: SwiGluFfn (crates/oxicuda-lm/src/layer/ffn.rs:202-254)
// with w_gate / w_up cut by rows as ColumnLinear::from_full_weight cuts them and w_down by columns as RowLinear::from_full_weight
// does, so that the sum of the ranks' outputs is the layer's output.  The shard is quantised once on the device (one scale for
// the gate/up tensor, interleaved in blocks of 128 rows, one for the down tensor); a forward is one call of oxq_mlp_swiglu_tp:
// x quantised per tensor, gate/up GEMM with silu(gate) * up in the epilogue, h quantised per shard, down GEMM and, when asked
// and a communicator exists, the all-reduce.  Sizes: hidden a multiple of 16, inter / tp a multiple of 128.
class TpSwiGluMlp {
public:
    DistInferHandle handle;
    size_t hidden = 0, inter = 0, inter_local = 0;
    TpSwiGluMlp(const DistInferHandle& handle, size_t hidden, size_t inter, const std::vector<float>& w_gate, const std::vector<float>& w_up,
                const std::vector<float>& w_down)
        : handle(handle), hidden(hidden), inter(inter) {
        const size_t tp = handle.config.tp;
        if (inter % tp != 0) throw DistInferError("TpFeaturesMisaligned", "features " + std::to_string(inter) + " not divisible by degree " + std::to_string(tp), inter, tp);
        inter_local = inter / tp;
        for (const std::vector<float>* w : {&w_gate, &w_up, &w_down})
            if (w->size() != inter * hidden)
                throw DistInferError("DimensionMismatch", "expected " + std::to_string(inter * hidden) + ", got " + std::to_string(w->size()), inter * hidden, w->size());
        if (inter_local == 0 || inter_local % 128 != 0 || hidden == 0 || hidden % 16 != 0)
            throw DistInferError("ShardShapeMismatch", "the shard needs hidden % 16 == 0 and inter / tp % 128 == 0", inter_local, hidden);
        detail::cuda(cudaSetDevice(handle.device));
        const int32_t rc = oxq_handle_create(handle.device, nullptr, &h_);
        if (rc) throw DistInferError(oxq_status_name(rc), "oxq_handle_create");
        try {
            const size_t r0 = handle.tp_rank() * inter_local, n_gu = 2 * inter_local * hidden, n_d = hidden * inter_local;
            std::vector<float> gu(n_gu), dn(n_d);
            for (size_t r = 0; r < inter_local; r++) {
                const size_t blk = r / 128, in_blk = r % 128;
                std::memcpy(&gu[((2 * blk) * 128 + in_blk) * hidden], &w_gate[(r0 + r) * hidden], hidden * sizeof(float));
                std::memcpy(&gu[((2 * blk + 1) * 128 + in_blk) * hidden], &w_up[(r0 + r) * hidden], hidden * sizeof(float));
            }
            for (size_t o = 0; o < hidden; o++) std::memcpy(&dn[o * inter_local], &w_down[o * inter + r0], inter_local * sizeof(float));
            detail::cuda(cudaMalloc(&w_gu_, n_gu));
            detail::cuda(cudaMalloc(&w_down_, n_d));
            detail::cuda(cudaMalloc((void**)&stats_, 4 * sizeof(float)));
            void* stage = nullptr;
            detail::cuda(cudaMalloc(&stage, (n_gu > n_d ? n_gu : n_d) * sizeof(float)));
            int32_t q = OXQ_OK;
            if (cudaMemcpy(stage, gu.data(), n_gu * sizeof(float), cudaMemcpyHostToDevice) != cudaSuccess) q = OXQ_ERR_LAUNCH_FAILED;
            if (!q) q = oxq_fp8_quant_dynamic(h_, stage, OXQ_F32, (int64_t)n_gu, (uint8_t*)w_gu_, stats_);
            if (!q && cudaDeviceSynchronize() != cudaSuccess) q = OXQ_ERR_LAUNCH_FAILED;
            if (!q && cudaMemcpy(stage, dn.data(), n_d * sizeof(float), cudaMemcpyHostToDevice) != cudaSuccess) q = OXQ_ERR_LAUNCH_FAILED;
            if (!q) q = oxq_fp8_quant_dynamic(h_, stage, OXQ_F32, (int64_t)n_d, (uint8_t*)w_down_, stats_ + 2);
            if (!q && cudaDeviceSynchronize() != cudaSuccess) q = OXQ_ERR_LAUNCH_FAILED;
            cudaFree(stage);
            check(q);
        } catch (...) { release(); throw; }
    }
    ~TpSwiGluMlp() { release(); }
    TpSwiGluMlp(const TpSwiGluMlp&) = delete; TpSwiGluMlp& operator=(const TpSwiGluMlp&) = delete;
    oxq_handle* library_handle() const { return h_; }
    // joins the tensor-parallel group: `id_128` is the identifier rank 0 got from oxq_comm_unique_id
    void init_comm(const void* id_128) { check(oxq_comm_init(h_, id_128, (int)handle.config.tp, (int)handle.tp_rank())); }
    oxq_tp_mlp_weights weights() const {
        oxq_tp_mlp_weights w{};
        w.variant = OXQ_TP_FP8; w.hidden = (int64_t)hidden; w.inter_local = (int64_t)inter_local;
        w.w_gu = w_gu_; w.w_gu_scales = stats_ + 1; w.w_down = w_down_; w.w_down_scales = stats_ + 3;
        return w;
    }
    // x bf16 [m x hidden] -> y bf16 [m x hidden]: this rank's partial, or the sum over the ranks when `reduce` is set and a
    // communicator exists.  Asynchronous on the library handle's stream; the workspace is kept and grows with m.
    void forward_device(const void* x_bf16_dev, size_t m, void* y_bf16_dev, bool reduce) {
        size_t need = 0;
        check(oxq_mlp_swiglu_tp_workspace_bytes(OXQ_TP_FP8, (int64_t)m, (int64_t)hidden, (int64_t)inter_local, &need));
        if (need > ws_bytes_) {
            detail::cuda(cudaDeviceSynchronize());
            if (ws_) cudaFree(ws_);
            ws_ = nullptr; ws_bytes_ = 0;
            detail::cuda(cudaMalloc(&ws_, need));
            ws_bytes_ = need;
        }
        const oxq_tp_mlp_weights w = weights();
        check(oxq_mlp_swiglu_tp(h_, &w, (int64_t)m, x_bf16_dev, y_bf16_dev, ws_, ws_bytes_, reduce ? 1 : 0));
    }
    // host slices: x f32 [batch x hidden] (rounded to bf16) -> f32 [batch x hidden]
    std::vector<float> forward_partial(const std::vector<float>& x, size_t batch) { return forward_host(x, batch, false); }
    std::vector<float> forward(const std::vector<float>& x, size_t batch) { return forward_host(x, batch, true); }
private:
    void check(int32_t rc) const { if (rc) throw DistInferError(oxq_status_name(rc), oxq_last_error_string(h_)); }
    void release() {
        if (w_gu_) cudaFree(w_gu_);
        if (w_down_) cudaFree(w_down_);
        if (stats_) cudaFree(stats_);
        if (ws_) cudaFree(ws_);
        if (h_) oxq_handle_destroy(h_);
        w_gu_ = w_down_ = ws_ = nullptr; stats_ = nullptr; h_ = nullptr;
    }
    std::vector<float> forward_host(const std::vector<float>& x, size_t batch, bool reduce) {
        if (x.size() != batch * hidden)
            throw DistInferError("DimensionMismatch", "expected " + std::to_string(batch * hidden) + ", got " + std::to_string(x.size()), batch * hidden, x.size());
        if (batch == 0) return {};
        std::vector<uint16_t> xb(x.size()), yb(x.size());
        for (size_t i = 0; i < x.size(); i++) xb[i] = detail::f32_to_bf16(x[i]);
        void *xd = nullptr, *yd = nullptr;
        detail::cuda(cudaMalloc(&xd, xb.size() * 2));
        if (cudaMalloc(&yd, yb.size() * 2) != cudaSuccess) { cudaFree(xd); throw DistInferError("Cuda", "cudaMalloc"); }
        try {
            detail::cuda(cudaMemcpy(xd, xb.data(), xb.size() * 2, cudaMemcpyHostToDevice));
            forward_device(xd, batch, yd, reduce);
            detail::cuda(cudaDeviceSynchronize());
            detail::cuda(cudaMemcpy(yb.data(), yd, yb.size() * 2, cudaMemcpyDeviceToHost));
        } catch (...) { cudaFree(xd); cudaFree(yd); throw; }
        cudaFree(xd); cudaFree(yd);
        std::vector<float> out(x.size());
        for (size_t i = 0; i < out.size(); i++) out[i] = detail::bf16_to_f32(yb[i]);
        return out;
    }
    oxq_handle* h_ = nullptr;
    void *w_gu_ = nullptr, *w_down_ = nullptr, *ws_ = nullptr;
    float* stats_ = nullptr;
    size_t ws_bytes_ = 0;
};

}  // namespace oxicuda_dist_infer
