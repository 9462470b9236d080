// Tensor-parallel SwiGLU MLP behind the C ABI: one rank's shard of the layer, the rank's four kernels and the one exchange
// step, for hosts that have no torch.distributed to lean on.
//
// Sharding is the reference's (ColumnLinear / RowLinear::from_full_weight, crates/oxicuda-dist-infer/src/tensor_parallel/
// column_parallel.rs:115-166, row_parallel.rs:109-168): gate and up weights by output rows, the down weight by input
// columns, h = silu(gate) * up local to the rank, every rank's [M x hidden] partial summed by one all-reduce
// (RowLinear::all_reduce, row_parallel.rs:199-223, which adds the partials on the host; here ncclAllReduce over NVLink).
//
// NCCL is bound at run time (dlopen): a process that already holds an NCCL (a Python host with torch) keeps using that
// one, a plain C / Rust host gets libnccl.so.2 from the loader's search path or from OXQ_NCCL_LIB.  Only NCCL's stable
// host API is used.
#include "oxq_common.cuh"
#include <dlfcn.h>
#include <nccl.h>
#include <new>
#include <stdlib.h>

namespace {

struct NcclApi {
    ncclResult_t (*GetVersion)(int*);
    ncclResult_t (*GetUniqueId)(ncclUniqueId*);
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int);
    ncclResult_t (*CommDestroy)(ncclComm_t);
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t);
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t);
    const char* (*GetErrorString)(ncclResult_t);
    bool ok;
};

NcclApi* nccl_api() {
    static NcclApi api = [] {
        NcclApi a{};
        void* lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);                       // the one the process already uses
        if (!lib) { const char* e = getenv("OXQ_NCCL_LIB"); if (e && e[0]) lib = dlopen(e, RTLD_NOW | RTLD_GLOBAL); }
        if (!lib) lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!lib) return a;
        a.GetVersion = (decltype(a.GetVersion))dlsym(lib, "ncclGetVersion");
        a.GetUniqueId = (decltype(a.GetUniqueId))dlsym(lib, "ncclGetUniqueId");
        a.CommInitRank = (decltype(a.CommInitRank))dlsym(lib, "ncclCommInitRank");
        a.CommDestroy = (decltype(a.CommDestroy))dlsym(lib, "ncclCommDestroy");
        a.AllReduce = (decltype(a.AllReduce))dlsym(lib, "ncclAllReduce");
        a.AllGather = (decltype(a.AllGather))dlsym(lib, "ncclAllGather");
        a.GetErrorString = (decltype(a.GetErrorString))dlsym(lib, "ncclGetErrorString");
        a.ok = a.GetVersion && a.GetUniqueId && a.CommInitRank && a.CommDestroy && a.AllReduce && a.AllGather && a.GetErrorString;
        return a;
    }();
    return &api;
}

#define OXQ_NCCL(h, expr)                                                                    \
    do {                                                                                     \
        ncclResult_t r__ = (expr);                                                           \
        if (r__ != ncclSuccess) {                                                            \
            snprintf((h)->last_error, sizeof((h)->last_error), "%s: %s", #expr, nccl_api()->GetErrorString(r__)); \
            return OXQ_ERR_NCCL_BASE + (int32_t)r__;                                         \
        }                                                                                    \
    } while (0)

inline size_t up256(size_t v) { return (v + 255) & ~(size_t)255; }

// workspace layout of the FP8 variant: codes of x, h in bf16, codes of h, two pairs of (absmax, scale)
struct Fp8Ws { size_t xq, h, hq, stats, end; };
Fp8Ws fp8_ws(int64_t m, int64_t hidden, int64_t inter_local) {
    Fp8Ws w;
    w.xq = 0;
    w.h = up256((size_t)m * hidden);
    w.hq = w.h + up256((size_t)m * inter_local * 2);
    w.stats = w.hq + up256((size_t)m * inter_local);
    w.end = w.stats + 256;
    return w;
}
// W4A16 variant: the workspaces of the two W4A16 GEMMs first (each keeps its own: their leading parts are the decode
// kernels' partial sums, zero between calls), then the interleaved gate/up product and h in bf16
struct W4Ws { size_t gemm1, gemm1_bytes, gemm2, gemm2_bytes, gu, h, end; };
W4Ws w4_ws(int64_t m, int64_t hidden, int64_t inter_local) {
    W4Ws w;
    w.gemm1 = 0;
    w.gemm1_bytes = up256(oxq_gemm_w4a16_workspace_bytes(m, 2 * inter_local, hidden));
    w.gemm2 = w.gemm1 + w.gemm1_bytes;
    w.gemm2_bytes = up256(oxq_gemm_w4a16_workspace_bytes(m, hidden, inter_local));
    w.gu = w.gemm2 + w.gemm2_bytes;
    w.h = w.gu + up256((size_t)m * 2 * inter_local * 2);
    w.end = w.h + up256((size_t)m * inter_local * 2);
    return w;
}

}  // namespace

extern "C" {

int32_t oxq_comm_unique_id(void* id_out_128) {
    if (!id_out_128) return OXQ_ERR_INVALID_ARGUMENT;
    NcclApi* a = nccl_api();
    if (!a->ok) return OXQ_ERR_UNSUPPORTED_OPERATION;
    ncclUniqueId id;
    const ncclResult_t r = a->GetUniqueId(&id);
    if (r != ncclSuccess) return OXQ_ERR_NCCL_BASE + (int32_t)r;
    static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId is 128 bytes");
    memcpy(id_out_128, &id, 128);
    return OXQ_OK;
}

int32_t oxq_comm_init(oxq_handle* h, const void* id_128, int nranks, int rank) {
    OXQ_CHECK_HANDLE(h);
    if (!id_128 || nranks < 1 || rank < 0 || rank >= nranks) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "rank %d outside a world of %d", rank, nranks);
    if (h->comm) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "the handle already has a communicator");
    NcclApi* a = nccl_api();
    if (!a->ok) OXQ_FAIL(h, OXQ_ERR_UNSUPPORTED_OPERATION, "libnccl.so.2 could not be loaded (set OXQ_NCCL_LIB to its path)");
    OXQ_CUDA(h, cudaSetDevice(h->device));
    ncclUniqueId id;
    memcpy(&id, id_128, 128);
    ncclComm_t comm = nullptr;
    OXQ_NCCL(h, a->CommInitRank(&comm, nranks, id, rank));
    h->comm = comm; h->nranks = nranks; h->rank = rank;
    return OXQ_OK;
}

int32_t oxq_comm_destroy(oxq_handle* h) {
    OXQ_CHECK_HANDLE(h);
    if (!h->comm) return OXQ_OK;
    OXQ_NCCL(h, nccl_api()->CommDestroy((ncclComm_t)h->comm));
    h->comm = nullptr; h->nranks = 1; h->rank = 0;
    return OXQ_OK;
}

int32_t oxq_comm_info(const oxq_handle* h, int* nranks_out, int* rank_out, int* nccl_version_out) {
    if (!h) return OXQ_ERR_INVALID_ARGUMENT;
    if (nranks_out) *nranks_out = h->comm ? h->nranks : 1;
    if (rank_out) *rank_out = h->comm ? h->rank : 0;
    if (nccl_version_out) { int v = 0; if (nccl_api()->ok) nccl_api()->GetVersion(&v); *nccl_version_out = v; }
    return OXQ_OK;
}

int32_t oxq_all_reduce_bf16(oxq_handle* h, void* y_bf16, int64_t numel) {
    OXQ_CHECK_HANDLE(h);
    if (numel <= 0) OXQ_FAIL(h, OXQ_ERR_EMPTY_INPUT, "all_reduce: empty input");
    if (!y_bf16) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null pointer");
    if (!h->comm || h->nranks == 1) return OXQ_OK;                                   // a world of one: the partial is the sum
    OXQ_NCCL(h, nccl_api()->AllReduce(y_bf16, y_bf16, (size_t)numel, ncclBfloat16, ncclSum, (ncclComm_t)h->comm, h->stream));
    return OXQ_OK;
}

int32_t oxq_all_gather_bf16(oxq_handle* h, const void* local_bf16, int64_t numel_local, void* gathered_bf16) {
    OXQ_CHECK_HANDLE(h);
    if (numel_local <= 0) OXQ_FAIL(h, OXQ_ERR_EMPTY_INPUT, "all_gather: empty input");
    if (!local_bf16 || !gathered_bf16) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null pointer");
    if (!h->comm || h->nranks == 1) {
        if (local_bf16 != gathered_bf16) OXQ_CUDA(h, cudaMemcpyAsync(gathered_bf16, local_bf16, (size_t)numel_local * 2, cudaMemcpyDeviceToDevice, h->stream));
        return OXQ_OK;
    }
    OXQ_NCCL(h, nccl_api()->AllGather(local_bf16, gathered_bf16, (size_t)numel_local, ncclBfloat16, (ncclComm_t)h->comm, h->stream));
    return OXQ_OK;
}

int32_t oxq_mlp_swiglu_tp_workspace_bytes(int variant, int64_t m, int64_t hidden, int64_t inter_local, size_t* bytes_out) {
    if (!bytes_out || m <= 0 || hidden <= 0 || inter_local <= 0) return OXQ_ERR_INVALID_ARGUMENT;
    if (variant == OXQ_TP_FP8) *bytes_out = fp8_ws(m, hidden, inter_local).end;
    else if (variant == OXQ_TP_W4A16) *bytes_out = w4_ws(m, hidden, inter_local).end;
    else return OXQ_ERR_INVALID_ARGUMENT;
    return OXQ_OK;
}

int32_t oxq_mlp_swiglu_tp(oxq_handle* h, const oxq_tp_mlp_weights* w, int64_t m, const void* x_bf16, void* y_bf16, void* workspace,
                          size_t workspace_bytes, int reduce) {
    OXQ_CHECK_HANDLE(h);
    if (!w || !x_bf16 || !y_bf16 || !workspace) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null pointer");
    if (m <= 0 || w->hidden <= 0 || w->inter_local <= 0) OXQ_FAIL(h, OXQ_ERR_INVALID_DIMENSION, "layer dimensions must be non-zero");
    if (w->inter_local % 128 != 0) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "the intermediate shard (%lld rows) must be a multiple of 128: gate and up rows are interleaved in blocks of 128", (long long)w->inter_local);
    if ((uintptr_t)workspace & 255u) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "workspace must be 256-byte aligned");
    if (!w->w_gu || !w->w_gu_scales || !w->w_down || !w->w_down_scales) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null weight pointer");
    const int64_t hidden = w->hidden, il = w->inter_local;
    char* ws = (char*)workspace;
    if (w->variant == OXQ_TP_FP8) {
        const Fp8Ws L = fp8_ws(m, hidden, il);
        if (workspace_bytes < L.end) OXQ_FAIL(h, OXQ_ERR_BUFFER_TOO_SMALL, "workspace: expected at least %zu bytes, got %zu", L.end, workspace_bytes);
        uint8_t* xq = (uint8_t*)(ws + L.xq);
        void* hb = ws + L.h;
        uint8_t* hq = (uint8_t*)(ws + L.hq);
        float* st_x = (float*)(ws + L.stats);
        float* st_h = st_x + 2;
        // x per tensor; h per shard (each rank's partial is in real units before the reduce, so no maximum crosses ranks)
        if (int32_t rc = oxq_fp8_quant_dynamic(h, x_bf16, OXQ_BF16, m * hidden, xq, st_x)) return rc;
        if (int32_t rc = oxq_gemm_fp8_swiglu(h, m, 2 * il, hidden, xq, hidden, (const uint8_t*)w->w_gu, hidden, st_x + 1, (const float*)w->w_gu_scales, hb, il)) return rc;
        if (int32_t rc = oxq_fp8_quant_dynamic(h, hb, OXQ_BF16, m * il, hq, st_h)) return rc;
        if (int32_t rc = oxq_gemm_fp8(h, m, hidden, il, hq, il, (const uint8_t*)w->w_down, il, st_h + 1, (const float*)w->w_down_scales, y_bf16, hidden)) return rc;
    } else if (w->variant == OXQ_TP_W4A16) {
        if (!w->w_gu_zeros || !w->w_down_zeros) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null zero-point pointer");
        const W4Ws L = w4_ws(m, hidden, il);
        if (workspace_bytes < L.end) OXQ_FAIL(h, OXQ_ERR_BUFFER_TOO_SMALL, "workspace: expected at least %zu bytes, got %zu", L.end, workspace_bytes);
        void* gu = ws + L.gu;
        void* hb = ws + L.h;
        if (int32_t rc = oxq_gemm_w4a16(h, m, 2 * il, hidden, x_bf16, (const uint32_t*)w->w_gu, (const uint16_t*)w->w_gu_scales, (const uint32_t*)w->w_gu_zeros, 128, gu, ws + L.gemm1, L.gemm1_bytes)) return rc;
        if (int32_t rc = oxq_swiglu_interleaved(h, gu, m, il, hb)) return rc;
        if (int32_t rc = oxq_gemm_w4a16(h, m, hidden, il, hb, (const uint32_t*)w->w_down, (const uint16_t*)w->w_down_scales, (const uint32_t*)w->w_down_zeros, 128, y_bf16, ws + L.gemm2, L.gemm2_bytes)) return rc;
    } else {
        OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "unknown variant %d", w->variant);
    }
    if (reduce) return oxq_all_reduce_bf16(h, y_bf16, m * hidden);
    return OXQ_OK;
}

}  // extern "C"
