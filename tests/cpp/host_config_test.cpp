// Host-only checks of the low-precision GEMM configuration types of the C++ host mirror (oxicuda_blas.hpp): the
// reference's own validate() tests restated (crates/oxicuda-blas/src/precision/int_ops.rs:787-944,
// fp4_fp6_ops.rs tests of MicroScalingConfig / Fp4GemmConfig), and the mapping from (Transpose, Layout) to the
// library's operand flags.  No device call is made; exit code 0 on success, else the number of the failed check.
#include <cstdio>
#include <string>
#include "../../oxicuda_b200/host/oxicuda_blas.hpp"

using namespace oxicuda_blas;

template <typename F>
static std::string variant_of(F&& f) {
    try { f(); } catch (const BlasError& e) { return e.variant; }
    return "Ok";
}

int main() {
    // int8_config_valid / zero_dim / k_not_multiple_of_4 / sm_75 accepted
    if (variant_of([] { Int8GemmConfig{128, 128, 64}.validate(SmVersion::Sm80); }) != "Ok") return 1;
    if (variant_of([] { Int8GemmConfig{0, 128, 64}.validate(SmVersion::Sm80); }) != "InvalidDimension") return 2;
    try { Int8GemmConfig{128, 128, 33}.validate(SmVersion::Sm80); return 3; }
    catch (const BlasError& e) { if (e.variant != "InvalidDimension" || std::string(e.what()).find("multiple of 4") == std::string::npos) return 3; }
    { Int8GemmConfig c{64, 64, 32}; c.accumulator = AccType::F32; if (variant_of([&] { c.validate(SmVersion::Sm75); }) != "Ok") return 4; }
    // int4_config_valid / zero_dim / k_not_multiple_of_8 / invalid_group_size / group_size_not_divides_k
    auto i4 = [](uint32_t m, uint32_t n, uint32_t k, uint32_t g) { Int4GemmConfig c{m, n, k}; c.group_size = g; return c; };
    if (variant_of([&] { i4(128, 128, 128, 32).validate(SmVersion::Sm80); }) != "Ok") return 5;
    if (variant_of([&] { i4(128, 0, 128, 32).validate(SmVersion::Sm80); }) != "InvalidDimension") return 6;
    if (variant_of([&] { i4(128, 128, 100, 32).validate(SmVersion::Sm80); }) != "InvalidDimension") return 7;
    if (variant_of([&] { i4(128, 128, 128, 3).validate(SmVersion::Sm80); }) != "InvalidArgument") return 8;
    if (variant_of([&] { i4(128, 128, 48, 32).validate(SmVersion::Sm80); }) != "InvalidArgument") return 9;
    // MicroScalingConfig: block sizes 32 / 64 / 128 only; num_scales per granularity
    for (uint32_t b : {32u, 64u, 128u}) { MicroScalingConfig c; c.block_size = b; if (variant_of([&] { c.validate(); }) != "Ok") return 10; }
    for (uint32_t b : {0u, 16u, 48u, 256u}) { MicroScalingConfig c; c.block_size = b; if (variant_of([&] { c.validate(); }) != "InvalidArgument") return 11; }
    { MicroScalingConfig c; if (c.num_scales(100) != 4) return 12; c.scaling_granularity = ScalingGranularity::PerTensor; if (c.num_scales(100) != 1) return 12;
      c.scaling_granularity = ScalingGranularity::PerChannel; if (c.num_scales(7) != 7) return 12; }
    // Fp4GemmConfig: zero dimension, architecture below sm_100, odd K, bad block size, kernel name
    { Fp4GemmConfig c{128, 128, 256}; if (variant_of([&] { c.validate(); }) != "Ok") return 13;
      if (c.kernel_name() != "fp4_e2m1_gemm_128x128x256_f32") return 13; }
    { Fp4GemmConfig c{0, 128, 256}; if (variant_of([&] { c.validate(); }) != "InvalidDimension") return 14; }
    { Fp4GemmConfig c{128, 128, 256}; c.sm_version = SmVersion::Sm90; if (variant_of([&] { c.validate(); }) != "UnsupportedOperation") return 15; }
    { Fp4GemmConfig c{128, 128, 255}; if (variant_of([&] { c.validate(); }) != "InvalidDimension") return 16; }
    { Fp4GemmConfig c{128, 128, 256}; c.micro_scaling.block_size = 16; if (variant_of([&] { c.validate(); }) != "InvalidArgument") return 17; }
    // (Transpose, Layout) -> which index is contiguous
    if (detail::rows_contiguous(Transpose::NoTrans, Layout::RowMajor)) return 18;          // A [m x k] row-major: k contiguous
    if (!detail::rows_contiguous(Transpose::Trans, Layout::RowMajor)) return 18;
    if (!detail::rows_contiguous(Transpose::NoTrans, Layout::ColMajor)) return 18;
    if (detail::rows_contiguous(Transpose::Trans, Layout::ColMajor)) return 18;
    std::puts("host config checks ok");
    return 0;
}
