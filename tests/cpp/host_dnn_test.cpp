// Drives the C++ mirror of the oxicuda-dnn quantize API (oxicuda_b200/host/oxicuda_dnn.hpp) on a GPU: known answers and
// the reference's buffer checks are verified here; the results on a 4100-element pattern are written to a file that the
// Python test compares with the oracle bit for bit.  Usage: host_dnn_test <out.bin> (on a GPU) or host_dnn_test host (the
// configuration types and Fp4BlockQuantizer only, no device); exit code 0 on success.
#include <cmath>
#include <cstdio>
#include <string>
#include <vector>
#include "../../oxicuda_b200/host/oxicuda_dnn.hpp"

using namespace oxicuda_dnn;

template <typename T> static void put(FILE* f, const std::vector<T>& v) { fwrite(v.data(), sizeof(T), v.size(), f); }

// host-only checks: Int4QuantConfig (int4_quantize.rs:971-996) and Fp4BlockQuantizer (block_scale.rs:475-610)
static int host_checks() {
    Int4QuantConfig cfg(128, true);
    if (cfg.num_groups(256) != 2 || cfg.num_groups(257) != 3 || cfg.packed_bytes(256) != 128 || cfg.packed_bytes(257) != 129) return 40;
    int errs = 0;
    try { Int4QuantConfig(0, true); } catch (const DnnError& e) { errs += e.variant == "InvalidArgument"; }
    try { Fp4BlockQuantizer(16); } catch (const DnnError& e) { errs += e.variant == "InvalidArgument"; }
    try { Fp4BlockQuantizer(64); } catch (const DnnError& e) { errs += e.variant == "InvalidArgument"; }
    if (errs != 3) return 41;
    if (Fp4BlockQuantizer::MAX_VALUE != 6.0f || Fp4BlockQuantizer::REQUIRED_BLOCK_SIZE != 32) return 42;
    Fp4BlockQuantizer q(32);
    if (q.block_size != 32 || q.num_scales(32) != 1 || q.num_scales(96) != 3 || q.num_scales(33) != 2 || q.num_scales(0) != 0) return 43;
    if (q.compute_scale(std::vector<float>(32, 0.0f)) != 1.0f || std::fabs(q.compute_scale(std::vector<float>(32, 6.0f)) - 1.0f) > 1e-6f ||
        std::fabs(q.compute_scale(std::vector<float>(32, 12.0f)) - 2.0f) > 1e-6f) return 44;
    std::vector<float> block(32, 0.0f);
    block[0] = -6.0f; block[1] = 3.0f; block[2] = 1.5f;
    if (std::fabs(q.compute_scale(block) - 1.0f) > 1e-6f) return 45;
    try { TensorDesc<float>::from_raw(nullptr, {}, {}); } catch (const DnnError& e) { errs += e.variant == "InvalidDimension"; }
    try { TensorDesc<float>::from_raw(nullptr, {2, 4}, {4}); } catch (const DnnError& e) { errs += e.variant == "InvalidDimension"; }
    if (errs != 5) return 46;
    if (TensorDesc<float>::from_raw(nullptr, {2, 3, 4}, {12, 4, 1}).numel() != 24) return 47;
    return 0;
}

int main(int argc, char** argv) {
    if (argc < 2) return 2;
    try {
        if (int rc = host_checks()) return rc;
        if (std::string(argv[1]) == "host") return 0;
        DnnHandle handle;
        // ---- per-tensor INT8: scale = absmax / 127, codes, round trip (int8_quantize.rs:26-29)
        {
            auto x = DeviceBuffer<float>::from_slice({1.0f, -2.0f, 3.0f, 127.0f, -127.0f, 0.0f, 64.0f, 10.0f});
            auto q = DeviceBuffer<int8_t>::alloc(8);
            auto s = DeviceBuffer<float>::alloc(1);
            quantize_to_int8(handle, TensorDesc<float>::matrix(x, 2, 4), q, s);
            auto y = DeviceBuffer<float>::alloc(8);
            auto yd = TensorDescMut<float>::matrix(y, 2, 4);
            dequantize_from_int8(handle, q, s, yd, 8);
            detail::cuda(cudaDeviceSynchronize());
            const std::vector<int8_t> qh = q.to_vec();
            const int8_t want[8] = {1, -2, 3, 127, -127, 0, 64, 10};
            if (s.to_vec()[0] != 1.0f) return 3;
            for (int i = 0; i < 8; i++) if (qh[i] != want[i]) return 4;
            const std::vector<float> yh = y.to_vec();
            for (int i = 0; i < 8; i++) if (yh[i] != (float)want[i]) return 5;
            // undersized buffers: output, then scale, in the reference's order (int8_quantize.rs:44-55)
            int errs = 0;
            auto small_q = DeviceBuffer<int8_t>::alloc(7);
            auto no_s = DeviceBuffer<float>::alloc(0);
            try { quantize_to_int8(handle, TensorDesc<float>::matrix(x, 2, 4), small_q, no_s); }
            catch (const DnnError& e) { errs += e.variant == "BufferTooSmall" && e.expected == 8 && e.actual == 7; }
            try { quantize_to_int8(handle, TensorDesc<float>::matrix(x, 2, 4), q, no_s); }
            catch (const DnnError& e) { errs += e.variant == "BufferTooSmall" && e.expected == 4 && e.actual == 0; }
            try { TensorDesc<float>::matrix(x, 3, 4); } catch (const DnnError& e) { errs += e.variant == "BufferTooSmall" && e.expected == 48 && e.actual == 32; }
            try { TensorDesc<float>::matrix(x, 0, 4); } catch (const DnnError& e) { errs += e.variant == "InvalidDimension"; }
            try { TensorDesc<float>::from_raw(x.as_device_ptr(), {2, 4}, {4}); } catch (const DnnError& e) { errs += e.variant == "InvalidDimension"; }
            auto small_y = DeviceBuffer<float>::alloc(4);
            auto small_yd = TensorDescMut<float>::matrix(small_y, 1, 4);
            try { dequantize_from_int8(handle, q, s, small_yd, 8); } catch (const DnnError& e) { errs += e.variant == "BufferTooSmall" && e.expected == 32 && e.actual == 16; }
            if (errs != 6) return 6;
        }
        // ---- per-tensor FP8: scale = absmax / 448, E4M3 codes (fp8_quantize.rs:47-170)
        {
            auto x = DeviceBuffer<float>::from_slice({448.0f, -224.0f, 1.0f, 0.0f});
            auto q = DeviceBuffer<uint8_t>::alloc(4);
            auto s = DeviceBuffer<float>::alloc(1);
            quantize_to_fp8(handle, TensorDesc<float>::matrix(x, 1, 4), q, s);
            auto y = DeviceBuffer<float>::alloc(4);
            auto yd = TensorDescMut<float>::matrix(y, 1, 4);
            dequantize_from_fp8(handle, q, s, yd, 4);
            detail::cuda(cudaDeviceSynchronize());
            const std::vector<uint8_t> qh = q.to_vec();
            if (s.to_vec()[0] != 1.0f || qh[0] != 0x7E || qh[1] != 0xF6 || qh[2] != 0x38 || qh[3] != 0x00) return 7;
            const std::vector<float> yh = y.to_vec();
            if (yh[0] != 448.0f || yh[1] != -224.0f || yh[2] != 1.0f || yh[3] != 0.0f) return 8;
            int errs = 0;
            auto small_q = DeviceBuffer<uint8_t>::alloc(3);
            try { quantize_to_fp8(handle, TensorDesc<float>::matrix(x, 1, 4), small_q, s); } catch (const DnnError& e) { errs += e.variant == "BufferTooSmall" && e.expected == 4 && e.actual == 3; }
            if (errs != 1) return 9;
        }
        // ---- Int4QuantConfig (int4_quantize.rs:971-996) and the symmetric / asymmetric definitions on one group
        {
            Int4QuantConfig cfg(128, true);
            if (cfg.num_groups(256) != 2 || cfg.num_groups(257) != 3 || cfg.packed_bytes(256) != 128 || cfg.packed_bytes(257) != 129) return 10;
            int errs = 0;
            try { Int4QuantConfig(0, true); } catch (const DnnError& e) { errs += e.variant == "InvalidArgument"; }
            if (errs != 1) return 11;
            Int4QuantConfig g4(4, true);
            auto x = DeviceBuffer<float>::from_slice({7.0f, -7.0f, 1.0f, 0.0f});
            auto packed = DeviceBuffer<uint8_t>::alloc(2);
            auto scales = DeviceBuffer<float>::alloc(1);
            auto zeros = DeviceBuffer<float>::alloc(1);
            quantize_to_int4(handle, x, packed, scales, zeros, 4, g4);
            auto y = DeviceBuffer<float>::alloc(4);
            dequantize_int4(handle, packed, scales, zeros, y, 4, g4);
            detail::cuda(cudaDeviceSynchronize());
            const std::vector<uint8_t> ph = packed.to_vec();
            // scale 1: codes 15, 1, 9, 8 -> bytes 0x1F, 0x89
            if (scales.to_vec()[0] != 1.0f || ph[0] != 0x1F || ph[1] != 0x89) return 12;
            const std::vector<float> yh = y.to_vec();
            if (yh[0] != 7.0f || yh[1] != -7.0f || yh[2] != 1.0f || yh[3] != 0.0f) return 13;
            Int4QuantConfig a4(4, false);
            auto xa = DeviceBuffer<float>::from_slice({0.0f, 15.0f, 7.5f, 3.0f});
            quantize_to_int4(handle, xa, packed, scales, zeros, 4, a4);
            detail::cuda(cudaDeviceSynchronize());
            const std::vector<uint8_t> pa = packed.to_vec();
            // scale 1, zero 0: codes 0, 15, 7 (truncation), 3 -> bytes 0xF0, 0x37
            if (scales.to_vec()[0] != 1.0f || zeros.to_vec()[0] != 0.0f || pa[0] != 0xF0 || pa[1] != 0x37) return 14;
            auto no_z = DeviceBuffer<float>::alloc(0);
            try { quantize_to_int4(handle, xa, packed, scales, no_z, 4, a4); } catch (const DnnError& e) { errs += e.variant == "BufferTooSmall" && e.expected == 4 && e.actual == 0; }
            auto small_p = DeviceBuffer<uint8_t>::alloc(1);
            try { quantize_to_int4(handle, xa, small_p, scales, zeros, 4, a4); } catch (const DnnError& e) { errs += e.variant == "BufferTooSmall" && e.expected == 2 && e.actual == 1; }
            if (errs != 3) return 15;
        }
        // ---- quantize_block_scaled: argument checks (block_scale.rs:65-94) and one block with scale 1
        {
            std::vector<float> v(16, 0.0f);
            v[0] = 6.0f; v[1] = -6.0f; v[2] = 1.0f; v[3] = 2.5f; v[4] = 3.5f;
            auto x = DeviceBuffer<float>::from_slice(v);
            auto out = DeviceBuffer<uint8_t>::alloc(16);
            auto scales = DeviceBuffer<float>::alloc(1);
            quantize_block_scaled(handle, TensorDesc<float>::matrix(x, 1, 16), out, scales, 16);
            detail::cuda(cudaDeviceSynchronize());
            const std::vector<uint8_t> oh = out.to_vec();
            // 6 -> 12, -6 -> 0, 1 -> 7, 2.5 -> 8 and 3.5 -> 10 (ties to even), 0 -> 6
            if (scales.to_vec()[0] != 1.0f || oh[0] != 12 || oh[1] != 0 || oh[2] != 7 || oh[3] != 8 || oh[4] != 10 || oh[5] != 6) return 16;
            int errs = 0;
            try { quantize_block_scaled(handle, TensorDesc<float>::matrix(x, 1, 16), out, scales, 24); } catch (const DnnError& e) { errs += e.variant == "InvalidArgument"; }
            try { quantize_block_scaled(handle, TensorDesc<float>::matrix(x, 1, 16), out, scales, 8); } catch (const DnnError& e) { errs += e.variant == "InvalidArgument"; }
            auto no_s = DeviceBuffer<float>::alloc(0);
            try { quantize_block_scaled(handle, TensorDesc<float>::matrix(x, 1, 16), out, no_s, 16); } catch (const DnnError& e) { errs += e.variant == "BufferTooSmall" && e.expected == 4 && e.actual == 0; }
            if (errs != 3) return 17;
        }
        // ---- a ragged pattern for the oracle: 4100 elements (ragged against groups of 128 and blocks of 32)
        const size_t n = 4100;
        std::vector<float> big(n);
        for (size_t i = 0; i < n; i++) big[i] = 0.05f * (float)((int)((i * 2654435761u) >> 19 & 2047) - 1024) / 1024.0f * (1.0f + (float)(i % 7));
        auto x = DeviceBuffer<float>::from_slice(big);
        auto xd = TensorDesc<float>::from_raw(x.as_device_ptr(), {(uint32_t)n}, {1});
        auto q8 = DeviceBuffer<int8_t>::alloc(n);
        auto s8 = DeviceBuffer<float>::alloc(1);
        quantize_to_int8(handle, xd, q8, s8);
        auto qf = DeviceBuffer<uint8_t>::alloc(n);
        auto sf = DeviceBuffer<float>::alloc(1);
        quantize_to_fp8(handle, xd, qf, sf);
        Int4QuantConfig sym(128, true), asym(128, false);
        auto p4s = DeviceBuffer<uint8_t>::alloc(sym.packed_bytes(n));
        auto s4s = DeviceBuffer<float>::alloc(sym.num_groups(n));
        auto z4s = DeviceBuffer<float>::alloc(0);
        quantize_to_int4(handle, x, p4s, s4s, z4s, n, sym);
        auto p4a = DeviceBuffer<uint8_t>::alloc(asym.packed_bytes(n));
        auto s4a = DeviceBuffer<float>::alloc(asym.num_groups(n));
        auto z4a = DeviceBuffer<float>::alloc(asym.num_groups(n));
        quantize_to_int4(handle, x, p4a, s4a, z4a, n, asym);
        auto y4a = DeviceBuffer<float>::alloc(n);
        dequantize_int4(handle, p4a, s4a, z4a, y4a, n, asym);
        auto ob = DeviceBuffer<uint8_t>::alloc(n);
        auto sb = DeviceBuffer<float>::alloc((n + 31) / 32);
        quantize_block_scaled(handle, xd, ob, sb, 32);
        detail::cuda(cudaDeviceSynchronize());
        FILE* f = fopen(argv[1], "wb");
        if (!f) return 9;
        put(f, big); put(f, q8.to_vec()); put(f, s8.to_vec()); put(f, qf.to_vec()); put(f, sf.to_vec());
        put(f, p4s.to_vec()); put(f, s4s.to_vec()); put(f, p4a.to_vec()); put(f, s4a.to_vec()); put(f, z4a.to_vec()); put(f, y4a.to_vec());
        put(f, ob.to_vec()); put(f, sb.to_vec());
        fclose(f);
    } catch (const std::exception& e) {
        fprintf(stderr, "exception: %s\n", e.what());
        return 1;
    }
    return 0;
}
