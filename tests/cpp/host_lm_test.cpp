// Drives the C++ mirror of the SwiGLU feed-forward layer (oxicuda_b200/host/oxicuda_lm.hpp).
//   host_lm_test host        WeightTensor constructors, silu and the argument errors: no device needed
//   host_lm_test <out.bin>   the reference's SwiGluFfn tests (crates/oxicuda-lm/src/layer/ffn.rs:357-395) on the GPU at bf16
//                            precision, then a 256 / 200 layer on 5 tokens whose result goes to the file for the Python side
//                            to compare with the oracle (200 exercises the padding of the intermediate extent to 128)
// Exit code 0 on success, else the number of the failed check.
#include <cmath>
#include <cstdio>
#include <cstring>
#include <vector>
#include "../../oxicuda_b200/host/oxicuda_lm.hpp"

using namespace oxicuda_lm;
typedef std::vector<float> V;

static int host_checks() {
    if (std::fabs(silu(0.0f)) > 1e-6f || std::fabs(silu(10.0f) - 10.0f) > 1e-3f || !(silu(1.0f) > 0.0f) || !(silu(-1.0f) < 0.0f)) return 40;   // ffn.rs:279-296
    WeightTensor e = WeightTensor::eye(2, 3);
    if (e.shape != std::vector<size_t>{2, 3} || e.data != V{1, 0, 0, 0, 1, 0} || WeightTensor::ones({2, 2}).data != V(4, 1.0f) || WeightTensor::zeros({3}).n_elements() != 3) return 41;
    int errs = 0;
    try { WeightTensor::from_data(V(5, 0.0f), {2, 3}); } catch (const LmError& x) { errs += x.variant == "WeightDataLengthMismatch" && x.expected == 6 && x.got == 5; }
    try { SwiGluFfn(4, 0); } catch (const LmError& x) { errs += x.variant == "InvalidConfig"; }                                            // swiglu_ffn_zero_dim_error
    try { SwiGluFfn(0, 4); } catch (const LmError& x) { errs += x.variant == "InvalidConfig"; }
    try { SwiGluFfn(4, 8).forward(V(4, 1.0f), 0); } catch (const LmError& x) { errs += x.variant == "EmptyInput"; }
    SwiGluFfn bad(4, 8);
    bad.w_up = WeightTensor::zeros({8, 3});
    try { bad.to_device(); } catch (const LmError& x) { errs += x.variant == "DimensionMismatch"; }
    if (errs != 5) return 42;
    return 0;
}

static int device_checks(const char* out_path) {
    // swiglu_ffn_zero_weights_zero_output
    {
        const V out = SwiGluFfn(4, 8).forward(V(4, 1.0f), 1);
        if (out.size() != 4) return 3;
        for (float v : out) if (std::fabs(v) > 1e-6f) return 4;
    }
    // swiglu_ffn_gate_identity: gate = up = down = I, x = 2 -> silu(2) * 2 (here to bf16 precision)
    {
        SwiGluFfn ffn(4, 4);
        ffn.w_gate = WeightTensor::eye(4, 4); ffn.w_up = WeightTensor::eye(4, 4); ffn.w_down = WeightTensor::eye(4, 4);
        const V out = ffn.forward(V(4, 2.0f), 1);
        const float expected = silu(2.0f) * 2.0f;
        for (float v : out) if (std::fabs(v - expected) > expected / 128.0f) return 5;
    }
    // swiglu_ffn_batch_tokens
    if (SwiGluFfn(4, 8).forward(V(12, 0.0f), 3).size() != 12) return 6;
    {
        int errs = 0;
        try { SwiGluFfn(4, 8).forward(V(11, 0.0f), 3); } catch (const LmError& x) { errs += x.variant == "DimensionMismatch" && x.expected == 12 && x.got == 11; }
        if (errs != 1) return 7;
    }
    // a layer for the oracle
    const size_t hidden = 256, inter = 200, tokens = 5;
    auto pattern = [](size_t n, uint32_t salt, float amp) {
        V v(n);
        for (size_t i = 0; i < n; i++) v[i] = amp * (float)((int)((((uint32_t)i + salt) * 2654435761u) >> 20 & 1023) - 512) / 512.0f;
        return v;
    };
    SwiGluFfn ffn(hidden, inter);
    ffn.w_gate = WeightTensor::from_data(pattern(inter * hidden, 3, 0.08f), {inter, hidden});
    ffn.w_up = WeightTensor::from_data(pattern(inter * hidden, 5, 0.08f), {inter, hidden});
    ffn.w_down = WeightTensor::from_data(pattern(hidden * inter, 9, 0.08f), {hidden, inter});
    const V x = pattern(tokens * hidden, 1, 1.0f);
    const V y = ffn.forward(x, tokens);
    const V y2 = ffn.to_device()->forward(x, tokens);                     // the resident form computes the same thing
    if (y != y2) return 8;
    FILE* f = fopen(out_path, "wb");
    if (!f) return 9;
    const V* parts[5] = {&x, &ffn.w_gate.data, &ffn.w_up.data, &ffn.w_down.data, &y};
    for (const V* v : parts) fwrite(v->data(), sizeof(float), v->size(), f);
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
