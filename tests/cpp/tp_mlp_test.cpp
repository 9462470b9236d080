// Drives the tensor-parallel SwiGLU MLP through the C ABI alone (no Python, no torch in the ranks): one process per rank and
// GPU, NCCL bound by the library at run time.
//
//   tp_mlp_test <dir> <nranks> <m> <hidden> <inter_local>           parent: makes the NCCL identifier, starts the ranks
//   tp_mlp_test <dir> <nranks> <m> <hidden> <inter_local> <rank> <id-hex>   one rank
//
// Every rank reads x.bin (bf16 [m x hidden], the same on all ranks) and its own shard rank<r>_wgu.bin (bf16, gate/up rows
// interleaved in blocks of 128, [2 * inter_local x hidden]) and rank<r>_wd.bin (bf16 [hidden x inter_local]) from <dir>,
// quantises the shard to E4M3 on the device, runs the layer without and with the all-reduce, gathers a slice of the partials,
// and writes rank<r>_partial.bin, rank<r>_y.bin and rank<r>_gather.bin (bf16).  Exit code 0 on success.
#include <cuda_runtime.h>
#include <sys/wait.h>
#include <unistd.h>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>
#include "../../include/oxq.h"

#define CK(expr) do { int32_t rc__ = (expr); if (rc__ != 0) { std::fprintf(stderr, "rank %d: %s -> %d (%s) %s\n", g_rank, #expr, rc__, oxq_status_name(rc__), g_h ? oxq_last_error_string(g_h) : ""); return 10; } } while (0)
#define CU(expr) do { cudaError_t e__ = (expr); if (e__ != cudaSuccess) { std::fprintf(stderr, "rank %d: %s -> %s\n", g_rank, #expr, cudaGetErrorString(e__)); return 11; } } while (0)

static int g_rank = -1;
static oxq_handle* g_h = nullptr;

static bool read_file(const std::string& path, std::vector<uint16_t>& v, size_t n) {
    v.resize(n);
    FILE* f = std::fopen(path.c_str(), "rb");
    if (!f) return false;
    const size_t got = std::fread(v.data(), 2, n, f);
    std::fclose(f);
    return got == n;
}
static bool write_file(const std::string& path, const void* p, size_t bytes) {
    FILE* f = std::fopen(path.c_str(), "wb");
    if (!f) return false;
    const size_t put = std::fwrite(p, 1, bytes, f);
    std::fclose(f);
    return put == bytes;
}

static int run_rank(const std::string& dir, int nranks, int64_t m, int64_t hidden, int64_t il, int rank, const char* id_hex) {
    g_rank = rank;
    unsigned char id[128];
    if (std::strlen(id_hex) != 256) return 2;
    for (int i = 0; i < 128; i++) { unsigned v; std::sscanf(id_hex + 2 * i, "%2x", &v); id[i] = (unsigned char)v; }
    int ndev = 0;
    CU(cudaGetDeviceCount(&ndev));
    if (ndev < nranks) { std::fprintf(stderr, "needs %d GPUs, found %d\n", nranks, ndev); return 3; }
    CU(cudaSetDevice(rank));
    cudaStream_t stream;
    CU(cudaStreamCreate(&stream));
    CK(oxq_handle_create(rank, stream, &g_h));
    CK(oxq_comm_init(g_h, id, nranks, rank));
    int nr = 0, rk = -1, ver = 0;
    CK(oxq_comm_info(g_h, &nr, &rk, &ver));
    if (nr != nranks || rk != rank) return 4;

    std::vector<uint16_t> x, wgu, wd;
    const std::string r = dir + "/rank" + std::to_string(rank);
    if (!read_file(dir + "/x.bin", x, (size_t)(m * hidden)) || !read_file(r + "_wgu.bin", wgu, (size_t)(2 * il * hidden)) ||
        !read_file(r + "_wd.bin", wd, (size_t)(hidden * il))) { std::fprintf(stderr, "rank %d: input files missing\n", rank); return 5; }
    void *d_x, *d_wgu, *d_wd, *d_wgu_q, *d_wd_q, *d_y, *d_part, *d_gather, *d_ws;
    float *d_st;
    CU(cudaMalloc(&d_x, x.size() * 2)); CU(cudaMalloc(&d_wgu, wgu.size() * 2)); CU(cudaMalloc(&d_wd, wd.size() * 2));
    CU(cudaMalloc(&d_wgu_q, wgu.size())); CU(cudaMalloc(&d_wd_q, wd.size()));
    CU(cudaMalloc(&d_y, (size_t)(m * hidden) * 2)); CU(cudaMalloc(&d_part, (size_t)(m * hidden) * 2));
    CU(cudaMalloc(&d_gather, (size_t)nranks * 1024 * 2)); CU(cudaMalloc((void**)&d_st, 4 * sizeof(float)));
    CU(cudaMemcpyAsync(d_x, x.data(), x.size() * 2, cudaMemcpyHostToDevice, stream));
    CU(cudaMemcpyAsync(d_wgu, wgu.data(), wgu.size() * 2, cudaMemcpyHostToDevice, stream));
    CU(cudaMemcpyAsync(d_wd, wd.data(), wd.size() * 2, cudaMemcpyHostToDevice, stream));
    // the shard's weights, quantised once: one scale for the fused gate/up tensor, one for the down tensor (stats = [absmax, scale])
    CK(oxq_fp8_quant_dynamic(g_h, d_wgu, OXQ_BF16, (int64_t)wgu.size(), (uint8_t*)d_wgu_q, d_st));
    CK(oxq_fp8_quant_dynamic(g_h, d_wd, OXQ_BF16, (int64_t)wd.size(), (uint8_t*)d_wd_q, d_st + 2));
    oxq_tp_mlp_weights w{};
    w.variant = OXQ_TP_FP8; w.hidden = hidden; w.inter_local = il;
    w.w_gu = d_wgu_q; w.w_gu_scales = d_st + 1; w.w_down = d_wd_q; w.w_down_scales = d_st + 3;
    size_t ws_bytes = 0;
    CK(oxq_mlp_swiglu_tp_workspace_bytes(OXQ_TP_FP8, m, hidden, il, &ws_bytes));
    CU(cudaMalloc(&d_ws, ws_bytes));
    CK(oxq_mlp_swiglu_tp(g_h, &w, m, d_x, d_part, d_ws, ws_bytes, /*reduce=*/0));
    CK(oxq_mlp_swiglu_tp(g_h, &w, m, d_x, d_y, d_ws, ws_bytes, /*reduce=*/1));
    CK(oxq_all_gather_bf16(g_h, d_part, 1024, d_gather));
    // a workspace that is too small is refused before anything runs
    if (oxq_mlp_swiglu_tp(g_h, &w, m, d_x, d_y, d_ws, 256, 1) != OXQ_ERR_BUFFER_TOO_SMALL) return 6;
    std::vector<uint16_t> part((size_t)(m * hidden)), y((size_t)(m * hidden)), gath((size_t)nranks * 1024);
    CU(cudaMemcpyAsync(part.data(), d_part, part.size() * 2, cudaMemcpyDeviceToHost, stream));
    CU(cudaMemcpyAsync(y.data(), d_y, y.size() * 2, cudaMemcpyDeviceToHost, stream));
    CU(cudaMemcpyAsync(gath.data(), d_gather, gath.size() * 2, cudaMemcpyDeviceToHost, stream));
    CU(cudaStreamSynchronize(stream));
    int32_t st = -1;
    CK(oxq_device_status(g_h, &st));
    if (st != 0) return 7;
    if (!write_file(r + "_partial.bin", part.data(), part.size() * 2) || !write_file(r + "_y.bin", y.data(), y.size() * 2) ||
        !write_file(r + "_gather.bin", gath.data(), gath.size() * 2)) return 8;
    CK(oxq_comm_destroy(g_h));
    CK(oxq_handle_destroy(g_h));
    return 0;
}

int main(int argc, char** argv) {
    if (argc != 6 && argc != 8) { std::fprintf(stderr, "usage: tp_mlp_test <dir> <nranks> <m> <hidden> <inter_local> [<rank> <id-hex>]\n"); return 1; }
    const std::string dir = argv[1];
    const int nranks = std::atoi(argv[2]);
    const int64_t m = std::atoll(argv[3]), hidden = std::atoll(argv[4]), il = std::atoll(argv[5]);
    if (argc == 8) return run_rank(dir, nranks, m, hidden, il, std::atoi(argv[6]), argv[7]);
    unsigned char id[128];
    const int32_t rc = oxq_comm_unique_id(id);
    if (rc != 0) { std::fprintf(stderr, "oxq_comm_unique_id -> %d (%s)\n", rc, oxq_status_name(rc)); return 20; }
    char hex[257];
    for (int i = 0; i < 128; i++) std::snprintf(hex + 2 * i, 3, "%02x", id[i]);
    std::vector<pid_t> kids;
    for (int r = 0; r < nranks; r++) {
        const pid_t pid = fork();
        if (pid == 0) {
            const std::string rs = std::to_string(r);
            execl(argv[0], argv[0], argv[1], argv[2], argv[3], argv[4], argv[5], rs.c_str(), hex, (char*)nullptr);
            _exit(127);
        }
        kids.push_back(pid);
    }
    int worst = 0;
    for (pid_t pid : kids) {
        int status = 0;
        waitpid(pid, &status, 0);
        const int code = WIFEXITED(status) ? WEXITSTATUS(status) : 99;
        if (code > worst) worst = code;
    }
    return worst;
}
