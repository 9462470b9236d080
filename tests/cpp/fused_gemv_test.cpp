// Drives oxq_dnn_fused_dequant_gemv through the C ABI: argument errors, then four shapes (4-bit ragged rows, the 14336 x 4096
// projection of the decode configuration, 8-bit, 2-bit) whose inputs and results go to a file that the Python test compares
// with the oracle's sequential restatement of the reference kernel.
//   fused_gemv_test <out.bin> [time]     `time` also prints the device time of the 14336 x 4096 case over rotating weight copies
// Exit code 0 on success, else the number of the failed check.
#include <cuda_runtime.h>
#include <cstdio>
#include <cstring>
#include <vector>
#include "../../include/oxq.h"

static uint32_t hash32(uint32_t i, uint32_t salt) { uint32_t v = (i + salt) * 2654435761u; v ^= v >> 15; v *= 2246822519u; v ^= v >> 13; return v; }

struct Case { int64_t rows, cols, group; int bits; };

int main(int argc, char** argv) {
    if (argc < 2) return 2;
    const bool timing = argc > 2 && strcmp(argv[2], "time") == 0;
    oxq_handle* h = nullptr;
    if (oxq_handle_create(0, nullptr, &h) != OXQ_OK) return 3;
    void* dummy = nullptr;
    if (cudaMalloc(&dummy, 4096) != cudaSuccess) return 3;
    const uint32_t* dw = (const uint32_t*)dummy; const float* df = (const float*)dummy; float* dy = (float*)dummy;
    if (oxq_dnn_fused_dequant_gemv(h, dw, df, df, dy, 0, 256, 64, 4) != OXQ_ERR_INVALID_DIMENSION) return 4;
    if (oxq_dnn_fused_dequant_gemv(h, dw, df, df, dy, 4, 256, 64, 3) != OXQ_ERR_UNSUPPORTED_OPERATION) return 5;
    if (oxq_dnn_fused_dequant_gemv(h, dw, df, df, dy, 4, 256, 96, 4) != OXQ_ERR_GROUP_SIZE_MISMATCH) return 6;
    if (oxq_dnn_fused_dequant_gemv(h, dw, df, df, dy, 4, 264, 8, 4) != OXQ_ERR_INVALID_ARGUMENT) return 7;      // 33 words: not a multiple of four
    if (oxq_dnn_fused_dequant_gemv(h, nullptr, df, df, dy, 4, 256, 64, 4) != OXQ_ERR_INVALID_ARGUMENT) return 8;
    cudaFree(dummy);

    const Case cases[4] = {{100, 256, 64, 4}, {14336, 4096, 128, 4}, {67, 512, 128, 8}, {33, 1024, 64, 2}};
    FILE* f = fopen(argv[1], "wb");
    if (!f) return 9;
    for (int c = 0; c < 4; c++) {
        const Case& k = cases[c];
        const size_t words = (size_t)(k.rows * k.cols * k.bits / 32), ngroups = (size_t)(k.rows * k.cols / k.group);
        std::vector<uint32_t> w(words);
        std::vector<float> s(ngroups), x((size_t)k.cols), y((size_t)k.rows);
        for (size_t i = 0; i < words; i++) w[i] = hash32((uint32_t)i, 101u + (uint32_t)c);
        for (size_t i = 0; i < ngroups; i++) s[i] = 0.001f + 0.01f * (float)(hash32((uint32_t)i, 211u + (uint32_t)c) & 1023u) / 1024.0f;
        for (size_t i = 0; i < x.size(); i++) x[i] = (float)((int)(hash32((uint32_t)i, 307u + (uint32_t)c) & 2047u) - 1024) / 1024.0f;
        void *wd, *sd, *xd, *yd;
        if (cudaMalloc(&wd, words * 4) != cudaSuccess || cudaMalloc(&sd, ngroups * 4) != cudaSuccess || cudaMalloc(&xd, x.size() * 4) != cudaSuccess ||
            cudaMalloc(&yd, y.size() * 4) != cudaSuccess) return 10;
        cudaMemcpy(wd, w.data(), words * 4, cudaMemcpyHostToDevice);
        cudaMemcpy(sd, s.data(), ngroups * 4, cudaMemcpyHostToDevice);
        cudaMemcpy(xd, x.data(), x.size() * 4, cudaMemcpyHostToDevice);
        cudaMemset(yd, 0xFF, y.size() * 4);
        const int32_t rc = oxq_dnn_fused_dequant_gemv(h, (const uint32_t*)wd, (const float*)sd, (const float*)xd, (float*)yd, k.rows, k.cols, k.group, k.bits);
        if (rc != OXQ_OK) { fprintf(stderr, "case %d: %d %s\n", c, rc, oxq_last_error_string(h)); return 11; }
        if (cudaDeviceSynchronize() != cudaSuccess) return 12;
        cudaMemcpy(y.data(), yd, y.size() * 4, cudaMemcpyDeviceToHost);
        const int64_t hdr[4] = {k.rows, k.cols, k.group, k.bits};
        fwrite(hdr, sizeof(int64_t), 4, f);
        fwrite(w.data(), 4, words, f); fwrite(s.data(), 4, ngroups, f); fwrite(x.data(), 4, x.size(), f); fwrite(y.data(), 4, y.size(), f);
        if (timing && c == 1) {
            // eight copies of the packed weight (235 MB, more than the L2 holds) taken in turn; 5 warm-up launches, 40 timed
            const int copies = 8, launches = 40;
            std::vector<void*> wc(copies);
            for (int i = 0; i < copies; i++) { if (cudaMalloc(&wc[i], words * 4) != cudaSuccess) return 13; cudaMemcpy(wc[i], wd, words * 4, cudaMemcpyDeviceToDevice); }
            cudaEvent_t e0, e1;
            cudaEventCreate(&e0); cudaEventCreate(&e1);
            for (int i = 0; i < 5; i++) oxq_dnn_fused_dequant_gemv(h, (const uint32_t*)wc[i % copies], (const float*)sd, (const float*)xd, (float*)yd, k.rows, k.cols, k.group, k.bits);
            cudaEventRecord(e0, 0);
            for (int i = 0; i < launches; i++) oxq_dnn_fused_dequant_gemv(h, (const uint32_t*)wc[i % copies], (const float*)sd, (const float*)xd, (float*)yd, k.rows, k.cols, k.group, k.bits);
            cudaEventRecord(e1, 0);
            if (cudaEventSynchronize(e1) != cudaSuccess) return 14;
            float ms = 0.0f;
            cudaEventElapsedTime(&ms, e0, e1);
            const double us = 1000.0 * ms / launches, bytes = (double)words * 4 + (double)ngroups * 4 + (double)x.size() * 4 + (double)y.size() * 4;
            printf("fused_dequant_gemv 14336x4096 g128 4-bit: %.2f us per launch, %.0f GB/s of %.1f MB algorithmic bytes\n", us, bytes / us * 1e-3, bytes * 1e-6);
            for (void* p : wc) cudaFree(p);
        }
        cudaFree(wd); cudaFree(sd); cudaFree(xd); cudaFree(yd);
    }
    fclose(f);
    int32_t st = -1;
    if (oxq_device_status(h, &st) != OXQ_OK || st != 0) return 15;
    oxq_handle_destroy(h);
    return 0;
}
