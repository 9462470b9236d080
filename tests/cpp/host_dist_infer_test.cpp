// Drives the C++ mirror of the tensor-parallel linear layers (oxicuda_b200/host/oxicuda_dist_infer.hpp).
//   host_dist_infer_test host        the reference's handle / coordinate / error tests: no device needed
//   host_dist_infer_test <out.bin>   the reference's layer tests on the GPU (every rank's shard built in this process, as
//                                    the reference's own tests do), then a 256 -> 512 -> 256 column / row pair at tp = 4 whose
//                                    results are written to the file for the Python side to compare with the oracle, then
//                                    the FP8 tensor-parallel SwiGLU MLP at tp = 2 (fused entry against its four steps, h and
//                                    the partials into the same file)
// Exit code 0 on success, else the number of the failed check.
#include <cstdio>
#include <cstring>
#include <vector>
#include "../../oxicuda_b200/host/oxicuda_dist_infer.hpp"

using namespace oxicuda_dist_infer;
typedef std::vector<float> V;

static DistInferHandle make_handle(size_t tp, size_t rank) { return DistInferHandle(0, SmVersion{100}, rank, ParallelismConfig{tp, 1, 1}); }
static V eye(size_t rows, size_t cols) { V m(rows * cols, 0.0f); for (size_t i = 0; i < rows && i < cols; i++) m[i * cols + i] = 1.0f; return m; }

static int host_checks() {
    // handle.rs:246-360
    DistInferHandle s = DistInferHandle::single_rank(80);
    if (s.world_size() != 1 || s.global_rank() != 0 || s.tp_rank() != 0 || s.sp_rank() != 0 || s.ep_rank() != 0) return 40;
    ParallelismConfig c222{2, 2, 2};
    RankCoordinates c1 = RankCoordinates::from_global(1, c222), c2 = RankCoordinates::from_global(2, c222), c7 = RankCoordinates::from_global(7, c222);
    if (c1.tp_rank != 1 || c1.sp_rank != 0 || c1.ep_rank != 0 || c2.tp_rank != 0 || c2.sp_rank != 1 || c2.ep_rank != 0) return 41;
    if (c7.tp_rank != 1 || c7.sp_rank != 1 || c7.ep_rank != 1 || c7.to_global(c222) != 7) return 42;
    int errs = 0;
    try { RankCoordinates::from_global(4, ParallelismConfig{2, 2, 1}); } catch (const DistInferError& e) { errs += e.variant == "RankOutOfRange" && e.a == 4 && e.b == 4; }
    try { ParallelismConfig{0, 1, 1}.validate(); } catch (const DistInferError& e) { errs += e.variant == "InvalidWorldSize"; }
    if (errs != 2) return 43;
    ParallelismConfig c4{4, 1, 1}, c24{2, 4, 1};
    if (RankCoordinates::from_global(0, c4).peer_tp(3, c4) != 3 || RankCoordinates::from_global(0, c24).peer_sp(3, c24) != 6) return 44;
    DistInferHandle h4(0, SmVersion{90}, 2, c4);
    if (h4.world_size() != 4 || h4.tp_rank() != 2) return 45;
    // the layers' argument checks come before any device work (column_parallel.rs:298-330, row_parallel.rs:322-360)
    errs = 0;
    try { ColumnLinear::from_full_weight(make_handle(3, 0), 2, 4, V(8, 0.0f)); } catch (const DistInferError& e) { errs += e.variant == "TpFeaturesMisaligned" && e.a == 4 && e.b == 3; }
    try { RowLinear::from_full_weight(make_handle(3, 0), 4, 4, V(16, 0.0f)); } catch (const DistInferError& e) { errs += e.variant == "TpInputMisaligned" && e.a == 4 && e.b == 3; }
    try { ColumnLinear::from_full_weight(make_handle(2, 0), 4, 4, V(15, 0.0f)); } catch (const DistInferError& e) { errs += e.variant == "DimensionMismatch" && e.a == 16 && e.b == 15; }
    V short_bias(3, 0.0f);
    try { ColumnLinear::from_full_weight(make_handle(2, 0), 4, 4, V(16, 0.0f), &short_bias); } catch (const DistInferError& e) { errs += e.variant == "DimensionMismatch" && e.a == 4 && e.b == 3; }
    try { ColumnLinear::all_gather(4, 1, {}); } catch (const DistInferError& e) { errs += e.variant == "TooFewRanks" && e.a == 1 && e.b == 0; }
    try { RowLinear::all_reduce({}); } catch (const DistInferError& e) { errs += e.variant == "TooFewRanks"; }
    try { RowLinear::all_reduce({V(4, 1.0f), V(3, 1.0f)}); } catch (const DistInferError& e) { errs += e.variant == "DimensionMismatch"; }
    if (errs != 7) return 46;
    if (ColumnLinear::all_gather(4, 2, {V{1, 2, 5, 6}, V{3, 4, 7, 8}}) != V{1, 2, 3, 4, 5, 6, 7, 8}) return 47;
    if (RowLinear::all_reduce({V{1, 2}, V{10, 20}, V{100, 200}}) != V{111, 222}) return 48;
    return 0;
}

static int device_checks(const char* out_path) {
    // column_linear_identity_weight (column_parallel.rs:240-262)
    {
        std::vector<V> shards;
        for (size_t r = 0; r < 2; r++) shards.push_back(ColumnLinear::from_full_weight(make_handle(2, r), 4, 4, eye(4, 4)).local_forward({1, 2, 3, 4}, 1));
        if (shards[0].size() != 2 || ColumnLinear::all_gather(4, 1, shards) != V{1, 2, 3, 4}) return 3;
    }
    // column_linear_batch2 (:264-285): tp = 4, ones weight, two tokens of ones
    {
        std::vector<V> shards;
        for (size_t r = 0; r < 4; r++) shards.push_back(ColumnLinear::from_full_weight(make_handle(4, r), 2, 4, V(8, 1.0f)).local_forward(V(4, 1.0f), 2));
        if (ColumnLinear::all_gather(4, 2, shards) != V(8, 2.0f)) return 4;
    }
    // column_linear_bias_added (:287-307): zero weight, bias [10, 20]
    {
        V bias{10.0f, 20.0f};
        std::vector<V> shards;
        for (size_t r = 0; r < 2; r++) shards.push_back(ColumnLinear::from_full_weight(make_handle(2, r), 2, 2, V(4, 0.0f), &bias).local_forward({0, 0}, 1));
        if (ColumnLinear::all_gather(2, 1, shards) != V{10, 20}) return 5;
    }
    // row_linear_identity_weight, bias_on_rank0_only, tp4_ones_weight, slice_input_correctness (row_parallel.rs:243-350)
    {
        std::vector<V> parts;
        for (size_t r = 0; r < 2; r++) parts.push_back(RowLinear::from_full_weight(make_handle(2, r), 4, 4, eye(4, 4)).local_forward({1, 2, 3, 4}, 1));
        if (RowLinear::all_reduce(parts) != V{1, 2, 3, 4}) return 6;
        V bias{5.0f, 7.0f};
        parts.clear();
        for (size_t r = 0; r < 2; r++) {
            RowLinear l = RowLinear::from_full_weight(make_handle(2, r), 2, 2, V(4, 0.0f), &bias);
            if (l.has_bias != (r == 0)) return 7;
            parts.push_back(l.local_forward({0, 0}, 1));
        }
        if (RowLinear::all_reduce(parts) != V{5, 7}) return 8;
        parts.clear();
        for (size_t r = 0; r < 4; r++) parts.push_back(RowLinear::from_full_weight(make_handle(4, r), 3, 4, V(12, 1.0f)).local_forward(V(8, 1.0f), 2));
        if (RowLinear::all_reduce(parts) != V(6, 4.0f)) return 9;
        RowLinear l0 = RowLinear::from_full_weight(make_handle(2, 0), 4, 4, V(16, 0.0f)), l1 = RowLinear::from_full_weight(make_handle(2, 1), 4, 4, V(16, 0.0f));
        if (l0.slice_input({10, 20, 30, 40}, 1) != V{10, 20} || l1.slice_input({10, 20, 30, 40}, 1) != V{30, 40}) return 10;
        int errs = 0;
        try { l0.local_forward(V(5, 0.0f), 1); } catch (const DistInferError& e) { errs += e.variant == "DimensionMismatch" && e.a == 4 && e.b == 5; }
        try { l0.forward_partial(V(3, 0.0f), 1); } catch (const DistInferError& e) { errs += e.variant == "DimensionMismatch" && e.a == 2 && e.b == 3; }
        if (errs != 2) return 11;
    }
    // e2e_tp_column_row_roundtrip (lib.rs:118-160): column -> all-gather -> row -> all-reduce with identity weights at tp = 4
    {
        std::vector<V> shards, parts;
        for (size_t r = 0; r < 4; r++) shards.push_back(ColumnLinear::from_full_weight(make_handle(4, r), 8, 8, eye(8, 8)).local_forward(V(8, 1.0f), 1));
        const V gathered = ColumnLinear::all_gather(8, 1, shards);
        if (gathered != V(8, 1.0f)) return 12;
        for (size_t r = 0; r < 4; r++) parts.push_back(RowLinear::from_full_weight(make_handle(4, r), 8, 8, eye(8, 8)).local_forward(gathered, 1));
        if (RowLinear::all_reduce(parts) != V(8, 1.0f)) return 13;
    }
    // a layer-sized pair for the oracle: x [5 x 256] -> column 512 (+ bias) -> row 256 (+ bias), tp = 4
    const size_t tp = 4, in_f = 256, mid = 512, batch = 5;
    auto pattern = [](size_t n, uint32_t salt, float amp) {
        V v(n);
        for (size_t i = 0; i < n; i++) v[i] = amp * (float)((int)((((uint32_t)i + salt) * 2654435761u) >> 20 & 1023) - 512) / 512.0f;
        return v;
    };
    const V x = pattern(batch * in_f, 1, 1.0f), w1 = pattern(mid * in_f, 7, 0.05f), b1 = pattern(mid, 11, 0.5f), w2 = pattern(in_f * mid, 13, 0.05f),
            b2 = pattern(in_f, 17, 0.5f);
    std::vector<V> shards, parts;
    for (size_t r = 0; r < tp; r++) shards.push_back(ColumnLinear::from_full_weight(make_handle(tp, r), in_f, mid, w1, &b1).local_forward(x, batch));
    const V h = ColumnLinear::all_gather(mid, batch, shards);
    for (size_t r = 0; r < tp; r++) parts.push_back(RowLinear::from_full_weight(make_handle(tp, r), in_f, mid, w2, &b2).local_forward(h, batch));
    const V y = RowLinear::all_reduce(parts);
    FILE* f = fopen(out_path, "wb");
    if (!f) return 9;
    for (const V* v : {&x, &w1, &b1, &w2, &b2, &h, &y}) fwrite(v->data(), sizeof(float), v->size(), f);
    // TpSwiGluMlp (FP8) at tp = 2, both ranks' shards in this process: hidden 512, intermediate 2048, five tokens.  Each rank's
    // partial from the fused entry must equal, bit for bit, the same four steps issued one by one (which also yields h for the
    // oracle); the file gets x (as bf16 values), the weights, and per rank h and the partial.
    {
        const size_t hid = 512, inter = 2048, m = 5, mtp = 2, il = inter / mtp;
        const V wg = pattern(inter * hid, 21, 0.08f), wu = pattern(inter * hid, 23, 0.08f), wd = pattern(hid * inter, 29, 0.08f);
        V xs = pattern(m * hid, 31, 1.0f);
        std::vector<uint16_t> xb(xs.size());
        for (size_t i = 0; i < xs.size(); i++) { xb[i] = detail::f32_to_bf16(xs[i]); xs[i] = detail::bf16_to_f32(xb[i]); }
        int errs = 0;
        try { TpSwiGluMlp(make_handle(3, 0), hid, inter, wg, wu, wd); } catch (const DistInferError& e) { errs += e.variant == "TpFeaturesMisaligned"; }
        try { TpSwiGluMlp(make_handle(2, 0), hid, inter, wg, V(7, 0.0f), wd); } catch (const DistInferError& e) { errs += e.variant == "DimensionMismatch"; }
        try { TpSwiGluMlp(make_handle(32, 0), hid, inter, wg, wu, wd); } catch (const DistInferError& e) { errs += e.variant == "ShardShapeMismatch"; }
        if (errs != 3) { fclose(f); return 14; }
        fwrite(xs.data(), sizeof(float), xs.size(), f);
        for (const V* v : {&wg, &wu, &wd}) fwrite(v->data(), sizeof(float), v->size(), f);
        std::vector<V> partials;
        for (size_t r = 0; r < mtp; r++) {
            TpSwiGluMlp mlp(make_handle(mtp, r), hid, inter, wg, wu, wd);
            const V part = mlp.forward_partial(xs, m);
            if (mlp.forward(xs, m) != part) { fclose(f); return 15; }        // no communicator: a world of one, the sum is the partial
            // the same steps one by one on the layer's own handle and weights
            oxq_handle* lh = mlp.library_handle();
            const oxq_tp_mlp_weights w = mlp.weights();
            void *xd, *xq, *hb, *hq, *yd; float* st;
            detail::cuda(cudaMalloc(&xd, m * hid * 2)); detail::cuda(cudaMalloc(&xq, m * hid)); detail::cuda(cudaMalloc(&hb, m * il * 2));
            detail::cuda(cudaMalloc(&hq, m * il)); detail::cuda(cudaMalloc(&yd, m * hid * 2)); detail::cuda(cudaMalloc((void**)&st, 4 * sizeof(float)));
            detail::cuda(cudaMemcpy(xd, xb.data(), xb.size() * 2, cudaMemcpyHostToDevice));
            int32_t rc = oxq_fp8_quant_dynamic(lh, xd, OXQ_BF16, (int64_t)(m * hid), (uint8_t*)xq, st);
            if (!rc) rc = oxq_gemm_fp8_swiglu(lh, (int64_t)m, (int64_t)(2 * il), (int64_t)hid, (const uint8_t*)xq, (int64_t)hid, (const uint8_t*)w.w_gu, (int64_t)hid, st + 1,
                                              (const float*)w.w_gu_scales, hb, (int64_t)il);
            if (!rc) rc = oxq_fp8_quant_dynamic(lh, hb, OXQ_BF16, (int64_t)(m * il), (uint8_t*)hq, st + 2);
            if (!rc) rc = oxq_gemm_fp8(lh, (int64_t)m, (int64_t)hid, (int64_t)il, (const uint8_t*)hq, (int64_t)il, (const uint8_t*)w.w_down, (int64_t)il, st + 3,
                                       (const float*)w.w_down_scales, yd, (int64_t)hid);
            if (rc) { fprintf(stderr, "staged step failed: %d %s\n", rc, oxq_last_error_string(lh)); fclose(f); return 16; }
            detail::cuda(cudaDeviceSynchronize());
            std::vector<uint16_t> hh(m * il), yy(m * hid);
            detail::cuda(cudaMemcpy(hh.data(), hb, hh.size() * 2, cudaMemcpyDeviceToHost));
            detail::cuda(cudaMemcpy(yy.data(), yd, yy.size() * 2, cudaMemcpyDeviceToHost));
            cudaFree(xd); cudaFree(xq); cudaFree(hb); cudaFree(hq); cudaFree(yd); cudaFree(st);
            for (size_t i = 0; i < yy.size(); i++) if (detail::bf16_to_f32(yy[i]) != part[i]) { fclose(f); return 17; }
            V hf(hh.size());
            for (size_t i = 0; i < hh.size(); i++) hf[i] = detail::bf16_to_f32(hh[i]);
            fwrite(hf.data(), sizeof(float), hf.size(), f);
            fwrite(part.data(), sizeof(float), part.size(), f);
            partials.push_back(part);
        }
        const V ysum = RowLinear::all_reduce(partials);
        fwrite(ysum.data(), sizeof(float), ysum.size(), f);
    }
    fclose(f);
    return 0;
}

int main(int argc, char** argv) {
    if (argc < 2) return 2;
    try {
        if (int rc = host_checks()) return rc;
        if (strcmp(argv[1], "host") == 0) return 0;
        return device_checks(argv[1]);
    } catch (const std::exception& e) {
        fprintf(stderr, "exception: %s\n", e.what());
        return 1;
    }
}
