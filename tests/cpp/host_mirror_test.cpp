// Drives the C++ host mirror (oxicuda_quant.hpp / oxicuda_blas.hpp) on a GPU and prints results that the Python
// test compares with the oracle.  Usage: host_mirror_test <out.bin>; exit code 0 on success.
#include <cmath>
#include <cstdio>
#include <cstring>
#include <stdexcept>
#include <vector>
#include "../../oxicuda_b200/host/oxicuda_blas.hpp"
#include "../../oxicuda_b200/host/oxicuda_quant.hpp"

int main(int argc, char** argv) {
    using namespace oxicuda_quant;
    if (argc < 2) return 2;
    try {
        // reference test `calibrate_2d_per_row` (minmax.rs:428-439) through the device path
        std::vector<float> t = {0.0f, 1.0f, -1.0f, 0.5f, 0.0f, 2.0f, -2.0f, 1.5f};
        MinMaxQuantizer q(8, QuantScheme::Symmetric, QuantGranularity::per_channel(0), OXQ_ROUND_HALF_AWAY);
        std::vector<int32_t> codes;
        QuantParams p = q.calibrate_quantize_2d(t, 2, 4, codes);
        if (p.scales.size() != 2 || !(p.scales[1] > p.scales[0])) return 3;
        if (p.q_max() != 127.0f || p.q_min() != -128.0f) return 4;
        std::vector<float> deq = q.dequantize_2d(codes, p, 2, 4);
        // a larger seeded-free pattern for the Python side to check against the oracle
        std::vector<float> big(64 * 256);
        for (size_t i = 0; i < big.size(); i++) big[i] = 0.02f * (float)((int)((i * 2654435761u) >> 20 & 1023) - 512) / 512.0f;
        std::vector<int32_t> big_codes;
        QuantParams bp = q.calibrate_quantize_2d(big, 64, 256, big_codes);
        // error behaviour: rows == 0 -> EmptyInput, cols == 0 -> DimensionMismatch, NaN -> NonFiniteFp8
        int errs = 0;
        try { q.calibrate_quantize_2d({}, 0, 4, codes); } catch (const QuantError& e) { errs += e.variant == "EmptyInput"; }
        try { q.calibrate_quantize_2d({}, 2, 0, codes); } catch (const QuantError& e) { errs += e.variant == "DimensionMismatch"; }
        Fp8Codec c = Fp8Codec::e4m3();
        try { c.encode({1.0f, NAN}); } catch (const QuantError& e) { errs += e.variant == "NonFiniteFp8"; }
        if (errs != 3) return 5;
        std::vector<uint8_t> enc = c.encode({0.0f, -0.0f, 1.0f, 1.9375f, 1000.0f});
        if (enc[0] != 0x00 || enc[1] != 0x80 || enc[2] != 0x38 || enc[4] != 0x7E) return 6;   // fp8.rs:288-292, types.rs:355-357
        std::vector<uint8_t> enc_ref = Fp8Codec(true).encode({1.9375f, 256.0f});
        if (enc_ref[0] != 0x3F || enc_ref[1] != 0x7E) return 7;                                // literal codec truncates
        // blas side: zero dimension -> InvalidDimension before anything is launched (gemm_api.rs:88-92)
        oxicuda_blas::BlasHandle bh;
        oxicuda_blas::MatrixDesc<oxicuda_blas::E4M3> a{nullptr, 0, 16, 16, oxicuda_blas::Layout::RowMajor}, b{nullptr, 8, 16, 16, oxicuda_blas::Layout::RowMajor};
        oxicuda_blas::MatrixDescMut<uint16_t> cm{nullptr, 0, 8, 8, oxicuda_blas::Layout::RowMajor};
        int berr = 0;
        try { oxicuda_blas::gemm_fp8(bh, a, b, nullptr, nullptr, cm); } catch (const oxicuda_blas::BlasError& e) { berr = e.variant == "InvalidDimension"; }
        if (!berr) return 8;
        berr = 0;
        try { oxicuda_blas::gemm_fp8(bh, 2.0f, a, b, nullptr, nullptr, 1.0f, cm); } catch (const oxicuda_blas::BlasError& e) { berr = e.variant == "InvalidDimension"; }
        if (!berr) return 8;
        // Nf4Quantizer: the reference's round-trip, all-zero and error tests (nf4.rs:243-310)
        {
            Nf4Quantizer nq(64);
            std::vector<float> ramp(128);
            for (int i = 0; i < 128; i++) ramp[i] = (float)i / 64.0f - 1.0f;
            auto enc = nq.encode(ramp);
            if (enc.first.size() != 64 || enc.second.size() != 2) return 10;
            if (!(nq.quantization_mse(ramp) < 0.01f)) return 11;
            auto z = Nf4Quantizer().encode(std::vector<float>(64, 0.0f));
            for (uint8_t b : z.first) if (b != 0x77) return 12;
            int nerr = 0;
            try { nq.encode(std::vector<float>(65, 0.5f)); } catch (const QuantError& e) { nerr += e.variant == "GroupSizeMismatch"; }
            try { nq.decode(std::vector<uint8_t>(32, 0), std::vector<float>(5, 1.0f)); } catch (const QuantError& e) { nerr += e.variant == "DimensionMismatch"; }
            try { nq.encode({}); } catch (const QuantError& e) { nerr += e.variant == "EmptyInput"; }
            if (nerr != 3) return 13;
        }
        // BlockQuantizedInt8: block counts, ragged tail, saturation (int8_quantize.rs:541-577)
        {
            std::vector<float> in(100);
            for (int i = 0; i < 100; i++) in[i] = (float)i;
            BlockQuantizedInt8 bq = BlockQuantizedInt8::quantize(in, 64);
            if (bq.num_blocks() != 2 || bq.dequantize().size() != 100) return 14;
            BlockQuantizedInt8 sat = BlockQuantizedInt8::quantize({1e30f, -1e30f, 0.0f, 1e30f}, 4);
            std::vector<float> d = sat.dequantize();
            if (!(d[0] > 0.0f && d[1] < 0.0f && d[2] == 0.0f) || sat.data[0] != 127 || sat.data[1] != -127) return 15;
            BlockQuantizedInt8 known;
            known.data = {-128, 0, 127}; known.scales = {0.1f}; known.block_size = 3; known.orig_len = 3;
            std::vector<float> kd = known.dequantize();
            if (std::fabs(kd[0] + 12.8f) > 1e-4f || kd[1] != 0.0f || std::fabs(kd[2] - 12.7f) > 1e-4f) return 16;
        }
        // GptqQuantizer: the reference's own tests (gptq.rs:422-520)
        {
            auto eye = [](size_t n) { std::vector<float> m(n * n, 0.0f); for (size_t i = 0; i < n; i++) m[i * n + i] = 1.0f; return m; };
            int gerr = 0;
            GptqConfig nodamp; nodamp.percdamp = 0.0;
            try { GptqQuantizer(nodamp).quantize_layer(std::vector<float>(4, 0.5f), 2, 2, std::vector<float>(4, 0.0f)); }
            catch (const QuantError& e) { gerr += e.variant == "SingularHessian"; }
            try { GptqQuantizer().quantize_layer(std::vector<float>(3, 0.5f), 1, 4, eye(4)); } catch (const QuantError& e) { gerr += e.variant == "DimensionMismatch"; }
            GptqConfig zero_bits; zero_bits.bits = 0;
            try { GptqQuantizer(zero_bits).quantize_layer(std::vector<float>(4, 0.5f), 2, 2, eye(2)); } catch (const QuantError& e) { gerr += e.variant == "InvalidBitWidth"; }
            if (gerr != 3) return 17;
            GptqConfig int8; int8.bits = 8;
            std::vector<float> gw(32);
            for (int i = 0; i < 32; i++) gw[i] = (float)i / 16.0f - 1.0f;
            GptqOutput go = GptqQuantizer(int8).quantize_layer(gw, 4, 8, eye(8));
            if (!(go.reconstruction_mse(gw) < 1e-4f) || go.quantized.size() != 32 || go.scales.size() != 8 || go.zero_points.size() != 8) return 18;
            GptqConfig asym; asym.symmetric = false;
            std::vector<float> aw = {-0.6f, 0.4f, -0.2f, 0.8f, 0.6f, -0.4f, 0.2f, -0.8f};
            if (!(GptqQuantizer(asym).quantize_layer(aw, 2, 4, eye(4)).reconstruction_mse(aw) < 0.05f)) return 19;
        }
        // SmoothQuantMigrator: the reference's own tests (smooth_quant.rs:311-440)
        {
            auto near = [](float a, float b, float eps) { return std::fabs(a - b) <= eps; };
            std::vector<float> sc = SmoothQuantMigrator(0.5f).compute_migration_scales({4.0f, 1.0f, 9.0f}, {1.0f, 4.0f, 1.0f});
            if (!near(sc[0], 2.0f, 1e-5f) || !near(sc[1], 0.5f, 1e-5f) || !near(sc[2], 3.0f, 1e-5f)) return 20;
            sc = SmoothQuantMigrator(1.0f).compute_migration_scales({2.0f, 5.0f}, {3.0f, 7.0f});
            if (!near(sc[0], 2.0f, 1e-5f) || !near(sc[1], 5.0f, 1e-5f)) return 21;
            sc = SmoothQuantMigrator(0.0f).compute_migration_scales({4.0f, 1.0f}, {2.0f, 5.0f});
            if (!near(sc[0], 0.5f, 1e-5f) || !near(sc[1], 0.2f, 1e-5f)) return 22;
            std::vector<float> st = SmoothQuantMigrator::compute_act_stats({1.0f, -5.0f, 2.0f, -3.0f, 4.0f, 1.0f}, 2, 3);
            if (st[0] != 3.0f || st[1] != 5.0f || st[2] != 2.0f) return 23;
            st = SmoothQuantMigrator::compute_weight_stats({0.5f, -2.0f, 1.0f, -1.5f, 0.3f, 3.0f}, 2, 3);
            if (st[0] != 1.5f || st[1] != 2.0f || st[2] != 3.0f) return 24;
            int serr = 0;
            try { SmoothQuantMigrator(0.5f).compute_migration_scales(std::vector<float>(3, 1.0f), std::vector<float>(4, 1.0f)); }
            catch (const QuantError& e) { serr += e.variant == "DimensionMismatch"; }
            try { SmoothQuantMigrator(0.5f).compute_migration_scales({}, {}); } catch (const QuantError& e) { serr += e.variant == "EmptyInput"; }
            try { SmoothQuantMigrator::compute_act_stats(std::vector<float>(5, 1.0f), 2, 3); } catch (const QuantError& e) { serr += e.variant == "DimensionMismatch"; }
            if (serr != 3) return 25;
            // smoothing_preserves_layer_output: Y = X W^T is unchanged by the migration
            const size_t n_tok = 3, n_ch = 4, n_out = 2;
            std::vector<float> acts(n_tok * n_ch), w(n_out * n_ch);
            for (size_t i = 0; i < acts.size(); i++) acts[i] = (float)i * 0.3f - 1.0f;
            for (size_t i = 0; i < w.size(); i++) w[i] = (float)i * 0.2f - 0.5f;
            auto matmul_nt = [&](const std::vector<float>& x, const std::vector<float>& ww) {
                std::vector<float> y(n_tok * n_out, 0.0f);
                for (size_t t = 0; t < n_tok; t++)
                    for (size_t o = 0; o < n_out; o++)
                        for (size_t j = 0; j < n_ch; j++) y[t * n_out + o] += x[t * n_ch + j] * ww[o * n_ch + j];
                return y;
            };
            const std::vector<float> y0 = matmul_nt(acts, w);
            SmoothQuantMigrator(0.5f).smooth_layer(acts, w, n_tok, n_ch, n_out);
            const std::vector<float> y1 = matmul_nt(acts, w);
            for (size_t i = 0; i < y0.size(); i++) if (!near(y0[i], y1[i], 1e-4f)) return 26;
            // smoothing_reduces_act_channel_range_imbalance
            std::vector<float> a2 = {100.0f, 1.0f, -100.0f, 1.0f, 100.0f, -1.0f, -100.0f, -1.0f}, w2 = {0.5f, 0.5f, -0.5f, 0.5f};
            sc = SmoothQuantMigrator(0.5f).smooth_layer(a2, w2, 4, 2, 2);
            float m0 = 0.0f, m1 = 0.0f;
            for (int t = 0; t < 4; t++) { m0 = std::fmax(m0, std::fabs(a2[t * 2])); m1 = std::fmax(m1, std::fabs(a2[t * 2 + 1])); }
            if (!(sc[0] > 1.0f) || !(m0 / std::fmax(m1, 1e-8f) < 100.0f)) return 27;
        }
        // MicroScalingQuantizer, FP4 half (fp4_fp6_ops.rs:763-897): scale = block max / 6, 1 for an all-zero block, odd lengths padded
        {
            using namespace oxicuda_blas;
            MicroScalingQuantizer mq{MicroScalingConfig()};
            std::vector<float> v(64);
            for (int i = 0; i < 64; i++) v[i] = (float)i * 0.25f - 4.0f;
            auto enc = mq.quantize_fp4(v, Fp4Format::E2M1);
            if (enc.first.size() != 32 || enc.second.size() != 2 || enc.second[0] != 4.0f / 6.0f || enc.second[1] != 11.75f / 6.0f) return 28;
            if (enc.first[0].unpack().first != 0xF) return 29;                 // -4 / (4/6) = -6: sign bit + the top code
            std::vector<float> rec = mq.dequantize_fp4(enc.first, enc.second, Fp4Format::E2M1, 64);
            if (rec.size() != 64 || rec[0] != -4.0f) return 30;
            for (int i = 0; i < 64; i++) if (std::fabs(rec[i] - v[i]) > 11.75f * 0.35f) return 31;
            auto z = mq.quantize_fp4(std::vector<float>(33, 0.0f), Fp4Format::E2M1);
            if (z.first.size() != 17 || z.second.size() != 2 || z.second[0] != 1.0f || z.second[1] != 1.0f) return 32;
            if (mq.dequantize_fp4(z.first, z.second, Fp4Format::E2M1, 33).size() != 33) return 33;
            int merr = 0;
            MicroScalingConfig bad; bad.block_size = 16;
            try { MicroScalingQuantizer(bad).quantize_fp4(v, Fp4Format::E2M1); } catch (const BlasError& e) { merr += e.variant == "InvalidArgument"; }
            if (merr != 1) return 34;
        }
        // blas mirror: the block-scaled and W8A32 GEMM wrappers against host products of the dequantised operands
        {
            using namespace oxicuda_blas;
            auto pattern = [](size_t n, uint32_t salt, float amp) {
                std::vector<float> v(n);
                for (size_t i = 0; i < n; i++) v[i] = amp * (float)((int)((((uint32_t)i + salt) * 2654435761u) >> 20 & 1023) - 512) / 512.0f;
                return v;
            };
            struct Dev {
                void* p = nullptr;
                explicit Dev(size_t bytes) { if (cudaMalloc(&p, bytes ? bytes : 16) != cudaSuccess) throw std::runtime_error("cudaMalloc"); }
                ~Dev() { cudaFree(p); }
                Dev(const Dev&) = delete; Dev& operator=(const Dev&) = delete;
            };
            auto bf16_to_f32 = [](uint16_t b) { uint32_t u = (uint32_t)b << 16; float f; memcpy(&f, &u, 4); return f; };
            // |y - ref| <= tol * max |ref| over [m x n]; ref accumulated in double from the dequantised operands
            auto close = [&](const std::vector<float>& y, const std::vector<float>& a, const std::vector<float>& b, size_t m, size_t n, size_t k, double tol) {
                std::vector<double> ref(m * n);
                double mx = 0.0;
                for (size_t i = 0; i < m; i++)
                    for (size_t j = 0; j < n; j++) {
                        double acc = 0.0;
                        for (size_t c = 0; c < k; c++) acc += (double)a[i * k + c] * (double)b[j * k + c];
                        ref[i * n + j] = acc; mx = std::fmax(mx, std::fabs(acc));
                    }
                for (size_t i = 0; i < m * n; i++) if (!(std::fabs((double)y[i] - ref[i]) <= tol * mx)) return false;
                return mx > 0.0;
            };
            const size_t shapes[2][3] = {{128, 384, 256}, {3, 200, 512}};         // a prefill tile and a decode shape
            for (const auto& sh : shapes) {
                const size_t m = sh[0], n = sh[1], k = sh[2];
                const std::vector<float> xa = pattern(m * k, 41, 1.0f), wb = pattern(n * k, 43, 1.0f);
                Dev xd(m * k * 4), wd(n * k * 4), yd(m * n * 2), xdq(m * k * 4), wdq(n * k * 4);
                cudaMemcpy(xd.p, xa.data(), m * k * 4, cudaMemcpyHostToDevice);
                cudaMemcpy(wd.p, wb.data(), n * k * 4, cudaMemcpyHostToDevice);
                std::vector<float> xq(m * k), wq(n * k), y(m * n);
                std::vector<uint16_t> yb(m * n);
                {   // MXFP8: E4M3 codes, E8M0 scale per 32
                    Dev xc(m * k), wc(n * k), xs(m * k / 32), ws(n * k / 32), xsm(oxq_sf_mma_bytes((int64_t)m, (int64_t)(k / 32))), wsm(oxq_sf_mma_bytes((int64_t)n, (int64_t)(k / 32)));
                    bh.check(oxq_mxfp8_quant(bh.raw(), xd.p, OXQ_F32, (int64_t)m, (int64_t)k, (uint8_t*)xc.p, (uint8_t*)xs.p, (uint8_t*)xsm.p));
                    bh.check(oxq_mxfp8_quant(bh.raw(), wd.p, OXQ_F32, (int64_t)n, (int64_t)k, (uint8_t*)wc.p, (uint8_t*)ws.p, (uint8_t*)wsm.p));
                    gemm_mxfp8(bh, (uint32_t)m, (uint32_t)n, (uint32_t)k, (const uint8_t*)xc.p, (const uint8_t*)xsm.p, (const uint8_t*)wc.p, (const uint8_t*)wsm.p, yd.p);
                    bh.check(oxq_mxfp8_dequant(bh.raw(), (const uint8_t*)xc.p, (const uint8_t*)xs.p, (int64_t)m, (int64_t)k, xdq.p, OXQ_F32));
                    bh.check(oxq_mxfp8_dequant(bh.raw(), (const uint8_t*)wc.p, (const uint8_t*)ws.p, (int64_t)n, (int64_t)k, wdq.p, OXQ_F32));
                    if (cudaDeviceSynchronize() != cudaSuccess) return 35;
                    cudaMemcpy(xq.data(), xdq.p, m * k * 4, cudaMemcpyDeviceToHost); cudaMemcpy(wq.data(), wdq.p, n * k * 4, cudaMemcpyDeviceToHost);
                    cudaMemcpy(yb.data(), yd.p, m * n * 2, cudaMemcpyDeviceToHost);
                    for (size_t i = 0; i < m * n; i++) y[i] = bf16_to_f32(yb[i]);
                    if (!close(y, xq, wq, m, n, k, 1.0 / 128.0)) return 36;
                }
                {   // NVFP4: E2M1 codes, UE4M3 scale per 16, f32 tensor scale
                    Fp4GemmConfig cfg{(uint32_t)m, (uint32_t)n, (uint32_t)k};
                    Dev xc(m * k / 2), wc(n * k / 2), xs(m * k / 16), ws(n * k / 16), xsm(oxq_sf_mma_bytes((int64_t)m, (int64_t)(k / 16))), wsm(oxq_sf_mma_bytes((int64_t)n, (int64_t)(k / 16))), stx(8), stw(8);
                    bh.check(oxq_absmax(bh.raw(), xd.p, OXQ_F32, (int64_t)(m * k), (float*)stx.p));
                    bh.check(oxq_absmax(bh.raw(), wd.p, OXQ_F32, (int64_t)(n * k), (float*)stw.p));
                    bh.check(oxq_nvfp4_quant(bh.raw(), xd.p, OXQ_F32, (int64_t)m, (int64_t)k, (float*)stx.p, (uint8_t*)xc.p, (uint8_t*)xs.p, (uint8_t*)xsm.p));
                    bh.check(oxq_nvfp4_quant(bh.raw(), wd.p, OXQ_F32, (int64_t)n, (int64_t)k, (float*)stw.p, (uint8_t*)wc.p, (uint8_t*)ws.p, (uint8_t*)wsm.p));
                    gemm_nvfp4(bh, cfg, (const uint8_t*)xc.p, (const uint8_t*)xsm.p, (const float*)stx.p + 1, (const uint8_t*)wc.p, (const uint8_t*)wsm.p, (const float*)stw.p + 1, yd.p);
                    bh.check(oxq_nvfp4_dequant(bh.raw(), (const uint8_t*)xc.p, (const uint8_t*)xs.p, (const float*)stx.p, (int64_t)m, (int64_t)k, xdq.p, OXQ_F32));
                    bh.check(oxq_nvfp4_dequant(bh.raw(), (const uint8_t*)wc.p, (const uint8_t*)ws.p, (const float*)stw.p, (int64_t)n, (int64_t)k, wdq.p, OXQ_F32));
                    if (cudaDeviceSynchronize() != cudaSuccess) return 37;
                    cudaMemcpy(xq.data(), xdq.p, m * k * 4, cudaMemcpyDeviceToHost); cudaMemcpy(wq.data(), wdq.p, n * k * 4, cudaMemcpyDeviceToHost);
                    cudaMemcpy(yb.data(), yd.p, m * n * 2, cudaMemcpyDeviceToHost);
                    for (size_t i = 0; i < m * n; i++) y[i] = bf16_to_f32(yb[i]);
                    if (!close(y, xq, wq, m, n, k, 1.0 / 128.0)) return 38;
                }
            }
            {   // W8A32 (benchmark configuration 1): per-row INT8 weights, f32 activations and result
                const size_t m = 13, n = 100, k = 1040;
                Int8GemmConfig cfg{(uint32_t)m, (uint32_t)n, (uint32_t)k};
                const std::vector<float> xa = pattern(m * k, 47, 1.0f), wb = pattern(n * k, 53, 0.05f);
                Dev xd(m * k * 4), wd(n * k * 4), wq8(n * k), sw(n * 4), yd(m * n * 4), wdq(n * k * 4);
                cudaMemcpy(xd.p, xa.data(), m * k * 4, cudaMemcpyHostToDevice);
                cudaMemcpy(wd.p, wb.data(), n * k * 4, cudaMemcpyHostToDevice);
                bh.check(oxq_int8_quant_rows(bh.raw(), (const float*)wd.p, (int64_t)n, (int64_t)k, (int8_t*)wq8.p, (float*)sw.p, OXQ_ROUND_HALF_EVEN));
                gemm_w8a32(bh, cfg, (const float*)xd.p, (const int8_t*)wq8.p, (const float*)sw.p, (float*)yd.p);
                bh.check(oxq_int8_dequant_rows(bh.raw(), (const int8_t*)wq8.p, (const float*)sw.p, (int64_t)n, (int64_t)k, (float*)wdq.p));
                if (cudaDeviceSynchronize() != cudaSuccess) return 39;
                std::vector<float> wq(n * k), y(m * n);
                cudaMemcpy(wq.data(), wdq.p, n * k * 4, cudaMemcpyDeviceToHost); cudaMemcpy(y.data(), yd.p, m * n * 4, cudaMemcpyDeviceToHost);
                if (!close(y, xa, wq, m, n, k, 1e-4)) return 40;
            }
        }
        FILE* f = fopen(argv[1], "wb");
        if (!f) return 9;
        fwrite(big.data(), sizeof(float), big.size(), f);
        fwrite(bp.scales.data(), sizeof(float), bp.scales.size(), f);
        fwrite(big_codes.data(), sizeof(int32_t), big_codes.size(), f);
        fwrite(deq.data(), sizeof(float), deq.size(), f);
        fclose(f);
    } catch (const std::exception& e) {
        fprintf(stderr, "exception: %s\n", e.what());
        return 1;
    }
    return 0;
}
