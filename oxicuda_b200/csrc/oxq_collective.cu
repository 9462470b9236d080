// All-reduce of the tensor-parallel partial sums through the NVSwitch multicast path (NVLS): every rank owns
// 1/world of the buffer, pulls the sum of all replicas of its slice with multimem.ld_reduce (the switch adds,
// f32 accumulation) and pushes the result back to every replica with multimem.st.  Each byte crosses a GPU's
// links about once per direction, half of what a ring moves.  The kernel does not wait on other GPUs: the
// caller brackets it with cross-rank barriers (all partials written before, all slices written after).
#include "oxq_common.cuh"
#include "oxq_tc.cuh"

namespace oxq {

__device__ __forceinline__ uint4 mm_ld_reduce(const uint4* p) {
    uint4 r;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p) : "memory");
    return r;
}
__device__ __forceinline__ void mm_st(uint4* p, const uint4& r) {
    asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};"
                 ::"l"(p), "r"(r.x), "r"(r.y), "r"(r.z), "r"(r.w) : "memory");
}

// four reductions in flight per thread: a round trip through the switch takes microseconds
__global__ void __launch_bounds__(512) multimem_all_reduce_bf16_kernel(uint4* mc, int64_t vec_lo, int64_t vec_hi) {
    pdl_trigger();
    pdl_wait();
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    int64_t v = vec_lo + blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    for (; v + 3 * stride < vec_hi; v += 4 * stride) {
        const uint4 a = mm_ld_reduce(mc + v), b = mm_ld_reduce(mc + v + stride), c = mm_ld_reduce(mc + v + 2 * stride),
                    d = mm_ld_reduce(mc + v + 3 * stride);
        mm_st(mc + v, a); mm_st(mc + v + stride, b); mm_st(mc + v + 2 * stride, c); mm_st(mc + v + 3 * stride, d);
    }
    for (; v < vec_hi; v += stride) mm_st(mc + v, mm_ld_reduce(mc + v));
}

// The same over a column range of a row-major matrix: rows [row_lo, row_hi) x vec_cols 16-byte vectors per row, rows
// ld_vecs vectors apart (the all-reduce of one column block of the output while the GEMM still produces the next).
__global__ void __launch_bounds__(512) multimem_all_reduce_bf16_2d_kernel(uint4* mc, int64_t row_lo, int64_t row_hi, int64_t vec_cols,
                                                                          int64_t ld_vecs) {
    pdl_trigger();
    pdl_wait();
    const int64_t total = (row_hi - row_lo) * vec_cols;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    auto at = [&](int64_t v) { const int64_t r = v / vec_cols; return mc + (row_lo + r) * ld_vecs + (v - r * vec_cols); };
    int64_t v = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    for (; v + 3 * stride < total; v += 4 * stride) {
        uint4* p0 = at(v); uint4* p1 = at(v + stride); uint4* p2 = at(v + 2 * stride); uint4* p3 = at(v + 3 * stride);
        const uint4 a = mm_ld_reduce(p0), b = mm_ld_reduce(p1), c = mm_ld_reduce(p2), d = mm_ld_reduce(p3);
        mm_st(p0, a); mm_st(p1, b); mm_st(p2, c); mm_st(p3, d);
    }
    for (; v < total; v += stride) { uint4* q = at(v); mm_st(q, mm_ld_reduce(q)); }
}

// The same with the cross-rank synchronisation inside the kernel (no barrier kernels around it): one thread signals on
// every rank that this rank's partial is written (the kernel is stream-ordered behind its producer), every CTA waits until
// all ranks have signalled, reduces its share, and the last CTA to finish signals "this rank's slice is broadcast" on
// every rank and leaves only when all ranks have said so -- the kernel that follows in the stream finds the complete sums.
// flags (symmetric memory, zero before the first call): [0] arrivals, [1] finished ranks, both running totals that are
// never cleared; [2] this rank's CTAs that are done, cleared by the last one; [3] this rank's finished calls.  The
// target of a call is world * (finished calls + 1): counted on the device, so the same launch replayed from a CUDA graph
// waits for its own generation of signals.  [3] changes only when every CTA of the grid is done, so all CTAs read one value.
__global__ void __launch_bounds__(512) multimem_all_reduce_bf16_2d_sync_kernel(uint4* mc, int64_t row_lo, int64_t row_hi, int64_t vec_cols,
                                                                               int64_t ld_vecs, uint32_t* flags, uint32_t* mc_flags, uint32_t world,
                                                                               int32_t* status) {
    using namespace oxq::tc;
    pdl_trigger();
    pdl_wait();
    __shared__ int s_ok;
    const uint32_t target = world * (*reinterpret_cast<const volatile uint32_t*>(flags + 3) + 1u);
    if (threadIdx.x == 0) {
        if (blockIdx.x == 0) mm_red_add_u32(mc_flags, 1u);
        s_ok = wait_word_at_least(flags, target, 200) ? 1 : 0;
        if (!s_ok) atomicExch(status, OXQ_ERR_DEVICE_TIMEOUT);
    }
    __syncthreads();
    if (s_ok) {
        const int64_t total = (row_hi - row_lo) * vec_cols;
        const int64_t stride = (int64_t)gridDim.x * blockDim.x;
        auto at = [&](int64_t v) { const int64_t r = v / vec_cols; return mc + (row_lo + r) * ld_vecs + (v - r * vec_cols); };
        int64_t v = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
        for (; v + 3 * stride < total; v += 4 * stride) {
            uint4* p0 = at(v); uint4* p1 = at(v + stride); uint4* p2 = at(v + 2 * stride); uint4* p3 = at(v + 3 * stride);
            const uint4 a = mm_ld_reduce(p0), b = mm_ld_reduce(p1), c = mm_ld_reduce(p2), d = mm_ld_reduce(p3);
            mm_st(p0, a); mm_st(p1, b); mm_st(p2, c); mm_st(p3, d);
        }
        for (; v < total; v += stride) { uint4* q = at(v); mm_st(q, mm_ld_reduce(q)); }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        if (atomicAdd(flags + 2, 1u) == gridDim.x - 1) {         // the last CTA of this rank
            __threadfence_system();
            flags[2] = 0u;
            mm_red_add_u32(mc_flags + 1, 1u);
            if (!wait_word_at_least(flags + 1, target, 200)) atomicExch(status, OXQ_ERR_DEVICE_TIMEOUT);
            *reinterpret_cast<volatile uint32_t*>(flags + 3) = target / world;      // this call is finished
            __threadfence();
        }
    }
}

}  // namespace oxq

extern "C" int32_t oxq_multimem_all_reduce_bf16_2d_sync(oxq_handle* h, void* multicast_ptr, int64_t rows, int64_t cols, int64_t ld, int rank, int world,
                                                        uint32_t* flags_local, uint32_t* flags_multicast) {
    OXQ_CHECK_HANDLE(h);
    if (rows <= 0 || cols <= 0) OXQ_FAIL(h, OXQ_ERR_EMPTY_INPUT, "all_reduce: empty input");
    if (world < 1 || world > 1024 || rank < 0 || rank >= world) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "rank %d outside world of %d", rank, world);
    if (!multicast_ptr || ((uintptr_t)multicast_ptr & 15u) || !flags_local || !flags_multicast || ((uintptr_t)flags_local & 15u) || ((uintptr_t)flags_multicast & 15u))
        OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null or misaligned multicast / flag pointer");
    if ((cols & 7) || (ld & 7) || ld < cols || rows % world != 0)
        OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "cols and ld must be multiples of 8 elements, ld >= cols, rows a multiple of world");
    if (int32_t rc = oxq_require_sm100(h)) return rc;
    const int64_t per = rows / world, total = per * (cols / 8);
    int64_t blocks = (total + 512 * 4 - 1) / (512 * 4);
    if (blocks > h->sm_count) blocks = h->sm_count;              // one CTA per SM at most: every CTA of the grid is resident
    if (blocks < 1) blocks = 1;
    oxq_launch(oxq::multimem_all_reduce_bf16_2d_sync_kernel, (int)blocks, 512, 0, h->stream, (uint4*)multicast_ptr, per * rank, per * (rank + 1), cols / 8,
               ld / 8, flags_local, flags_multicast, (uint32_t)world, h->dev_status);
    OXQ_LAUNCH_CHECK(h);
    return OXQ_OK;
}

extern "C" int32_t oxq_multimem_all_reduce_bf16_2d(oxq_handle* h, void* multicast_ptr, int64_t rows, int64_t cols, int64_t ld, int rank, int world) {
    OXQ_CHECK_HANDLE(h);
    if (rows <= 0 || cols <= 0) OXQ_FAIL(h, OXQ_ERR_EMPTY_INPUT, "all_reduce: empty input");
    if (world < 1 || rank < 0 || rank >= world) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "rank %d outside world of %d", rank, world);
    if (!multicast_ptr || ((uintptr_t)multicast_ptr & 15u)) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null or misaligned multicast pointer");
    if ((cols & 7) || (ld & 7) || ld < cols || rows % world != 0)
        OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "cols and ld must be multiples of 8 elements, ld >= cols, rows a multiple of world");
    if (int32_t rc = oxq_require_sm100(h)) return rc;
    const int64_t per = rows / world, total = per * (cols / 8);
    int64_t blocks = (total + 512 * 4 - 1) / (512 * 4);
    if (blocks > h->sm_count) blocks = h->sm_count;
    if (blocks < 1) blocks = 1;
    oxq_launch(oxq::multimem_all_reduce_bf16_2d_kernel, (int)blocks, 512, 0, h->stream, (uint4*)multicast_ptr, per * rank, per * (rank + 1), cols / 8, ld / 8);
    OXQ_LAUNCH_CHECK(h);
    return OXQ_OK;
}

extern "C" int32_t oxq_multimem_all_reduce_bf16(oxq_handle* h, void* multicast_ptr, int64_t numel, int rank, int world) {
    OXQ_CHECK_HANDLE(h);
    if (numel <= 0) OXQ_FAIL(h, OXQ_ERR_EMPTY_INPUT, "all_reduce: empty input");
    if (world < 1 || rank < 0 || rank >= world) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "rank %d outside world of %d", rank, world);
    if (!multicast_ptr || ((uintptr_t)multicast_ptr & 15u)) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null or misaligned multicast pointer");
    if (numel % (8 * (int64_t)world) != 0) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "numel %lld must be a multiple of 8 * world", (long long)numel);
    if (int32_t rc = oxq_require_sm100(h)) return rc;
    const int64_t vecs = numel / 8, per = vecs / world;
    const int64_t lo = per * rank, hi = lo + per;
    int64_t blocks = (per + 512 * 4 - 1) / (512 * 4);
    if (blocks > h->sm_count) blocks = h->sm_count;
    if (blocks < 1) blocks = 1;
    oxq_launch(oxq::multimem_all_reduce_bf16_kernel, (int)blocks, 512, 0, h->stream, (uint4*)multicast_ptr, lo, hi);
    OXQ_LAUNCH_CHECK(h);
    return OXQ_OK;
}
