// Drives the C++ host mirror (oxicuda_quant.hpp / oxicuda_blas.hpp) on a GPU and prints results that the Python
// test compares with the oracle.  Usage: host_mirror_test <out.bin>; exit code 0 on success.
#include <cstdio>
#include <cstring>
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
