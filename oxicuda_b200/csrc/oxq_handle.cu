// Handle lifecycle and status plumbing of liboxq_b200.
#include "oxq_common.cuh"
#include <new>
#include <stdlib.h>

extern "C" {

int32_t oxq_version(void) { return 100; }

const char* oxq_status_name(int32_t s) {
    switch (s) {
        case OXQ_OK: return "Ok";
        case OXQ_ERR_EMPTY_INPUT: return "EmptyInput";
        case OXQ_ERR_GROUP_SIZE_MISMATCH: return "GroupSizeMismatch";
        case OXQ_ERR_INVALID_SCALE: return "InvalidScale";
        case OXQ_ERR_QUANT_DIMENSION_MISMATCH: return "DimensionMismatch";
        case OXQ_ERR_NON_FINITE_FP8: return "NonFiniteFp8";
        case OXQ_ERR_INVALID_BIT_WIDTH: return "InvalidBitWidth";
        case OXQ_ERR_SINGULAR_HESSIAN: return "SingularHessian";
        case OXQ_ERR_INVALID_DIMENSION: return "InvalidDimension";
        case OXQ_ERR_BUFFER_TOO_SMALL: return "BufferTooSmall";
        case OXQ_ERR_DIMENSION_MISMATCH: return "DimensionMismatch";
        case OXQ_ERR_UNSUPPORTED_OPERATION: return "UnsupportedOperation";
        case OXQ_ERR_LAUNCH_FAILED: return "LaunchFailed";
        case OXQ_ERR_INVALID_ARGUMENT: return "InvalidArgument";
        case OXQ_ERR_DEVICE_TIMEOUT: return "DeviceTimeout";
        default: return s >= OXQ_ERR_NCCL_BASE ? "Nccl" : (s >= OXQ_ERR_CUDA_BASE ? "Cuda" : "Unknown");
    }
}

int32_t oxq_handle_create(int device, void* cuda_stream, oxq_handle** out) {
    if (!out) return OXQ_ERR_INVALID_ARGUMENT;
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess) return OXQ_ERR_CUDA_BASE + (int32_t)e;
    if (device < 0 || device >= count) return OXQ_ERR_INVALID_ARGUMENT;
    e = cudaSetDevice(device);
    if (e != cudaSuccess) return OXQ_ERR_CUDA_BASE + (int32_t)e;
    cudaDeviceProp prop;
    e = cudaGetDeviceProperties(&prop, device);
    if (e != cudaSuccess) return OXQ_ERR_CUDA_BASE + (int32_t)e;
    oxq_handle* h = new (std::nothrow) oxq_handle();
    if (!h) return OXQ_ERR_INVALID_ARGUMENT;
    h->device = device;
    h->stream = (cudaStream_t)cuda_stream;
    h->sm_count = prop.multiProcessorCount;
    h->cc_major = prop.major;
    h->cc_minor = prop.minor;
    h->last_error[0] = 0;
    h->comm = nullptr; h->nranks = 1; h->rank = 0;
    h->dev_status = nullptr;
    // The only allocation the library ever makes: 128 bytes per handle (status word + self-cleaning reduction cells).
    h->dev_scratch = nullptr;
    e = cudaMalloc(&h->dev_status, 128);
    if (e == cudaSuccess) e = cudaMemset(h->dev_status, 0, 128);
    if (e == cudaSuccess) h->dev_scratch = reinterpret_cast<uint32_t*>(h->dev_status) + 16;
    if (e != cudaSuccess) { delete h; return OXQ_ERR_CUDA_BASE + (int32_t)e; }
    *out = h;
    return OXQ_OK;
}

int32_t oxq_handle_destroy(oxq_handle* h) {
    if (!h) return OXQ_ERR_INVALID_ARGUMENT;
    if (h->comm) oxq_comm_destroy(h);
    if (h->dev_status) cudaFree(h->dev_status);
    delete h;
    return OXQ_OK;
}

int32_t oxq_set_stream(oxq_handle* h, void* cuda_stream) {
    OXQ_CHECK_HANDLE(h);
    h->stream = (cudaStream_t)cuda_stream;
    return OXQ_OK;
}

const char* oxq_last_error_string(const oxq_handle* h) { return h ? h->last_error : "null handle"; }

int32_t oxq_device_status(oxq_handle* h, int32_t* status_out) {
    OXQ_CHECK_HANDLE(h);
    if (!status_out) return OXQ_ERR_INVALID_ARGUMENT;
    int32_t v = 0;
    OXQ_CUDA(h, cudaMemcpyAsync(&v, h->dev_status, sizeof(v), cudaMemcpyDeviceToHost, h->stream));
    OXQ_CUDA(h, cudaStreamSynchronize(h->stream));
    if (v != 0) OXQ_CUDA(h, cudaMemsetAsync(h->dev_status, 0, sizeof(int32_t), h->stream));
    *status_out = v;
    return OXQ_OK;
}

}  // extern "C"

bool oxq_pdl_enabled() {
    static int v = -1;
    if (v < 0) { const char* e = getenv("OXQ_PDL"); v = e ? (atoi(e) != 0) : 1; }
    return v != 0;
}

int32_t oxq_require_sm100(oxq_handle* h) {
    if (h->cc_major != 10)
        OXQ_FAIL(h, OXQ_ERR_UNSUPPORTED_OPERATION,
                 "device %d is compute capability %d.%d; this library runs on sm_100 only and has no fallback",
                 h->device, h->cc_major, h->cc_minor);
    return OXQ_OK;
}
