// Shared declarations of liboxq_b200: the handle, status plumbing and small device helpers.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>
#include <atomic>
#include "../../include/oxq.h"

struct oxq_handle {
    int device;
    cudaStream_t stream;
    int sm_count;
    int cc_major, cc_minor;
    int32_t* dev_status;      // one word in device memory, written by bounded waits that expire
    uint32_t* dev_scratch;    // 16 words after the status word: reduction cells that kernels leave zeroed (absmax)
    void* comm;               // ncclComm_t of oxq_comm_init (tensor-parallel entry points), or null
    int nranks, rank;
    char last_error[256];
};

#define OXQ_FAIL(h, code, ...)                                           \
    do {                                                                 \
        if (h) snprintf((h)->last_error, sizeof((h)->last_error), __VA_ARGS__); \
        return (code);                                                   \
    } while (0)

#define OXQ_CUDA(h, expr)                                                \
    do {                                                                 \
        cudaError_t e__ = (expr);                                        \
        if (e__ != cudaSuccess) {                                        \
            if (h) snprintf((h)->last_error, sizeof((h)->last_error), "%s: %s", #expr, cudaGetErrorString(e__)); \
            return OXQ_ERR_CUDA_BASE + (int32_t)e__;                     \
        }                                                                \
    } while (0)

#define OXQ_CHECK_HANDLE(h)                                              \
    do { if (!(h)) return OXQ_ERR_INVALID_ARGUMENT; (h)->last_error[0] = 0; } while (0)

// Reports a launch-time error of the kernel just launched (asynchronous faults surface later).
#define OXQ_LAUNCH_CHECK(h)                                              \
    do {                                                                 \
        cudaError_t e__ = cudaGetLastError();                            \
        if (e__ != cudaSuccess) {                                        \
            snprintf((h)->last_error, sizeof((h)->last_error), "kernel launch failed: %s", cudaGetErrorString(e__)); \
            return OXQ_ERR_CUDA_BASE + (int32_t)e__;                     \
        }                                                                \
    } while (0)

// Launch settings that belong to a device (a kernel's dynamic shared-memory limit, occupancy figures) are cached per
// device ordinal, not per process: one process may hold handles on several GPUs, and function attributes set on one
// device say nothing about another.  A slot holds 0 until its value is known; two host threads that both find 0 both
// compute the same value and store it, which is harmless.
constexpr int OXQ_MAX_DEVICES = 64;
struct OxqPerDevice {
    std::atomic<int> v[OXQ_MAX_DEVICES];
    int get(int device) const { return (unsigned)device < (unsigned)OXQ_MAX_DEVICES ? v[device].load(std::memory_order_acquire) : 0; }
    void set(int device, int value) { if ((unsigned)device < (unsigned)OXQ_MAX_DEVICES) v[device].store(value, std::memory_order_release); }
};

// Refuses to launch on anything but a compute-capability 10.x device: there is no fallback path.
int32_t oxq_require_sm100(oxq_handle* h);

// Every kernel of the library is launched with the programmatic-dependent-launch attribute (OXQ_PDL=0 turns it
// off): a kernel may be scheduled while the one before it in the stream is still draining, which hides the few
// microseconds a launch costs when kernels that last 5-30 us follow one another.  Kernels call pdl_trigger() first
// (the next launch may be scheduled) and pdl_wait() before their first access to anything an earlier kernel may
// have written or may still read; both are no-ops in a launch without the attribute.
bool oxq_pdl_enabled();

template <bool PDL = true, typename... P, typename... A>
static inline cudaError_t oxq_launch(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, A&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = (PDL && oxq_pdl_enabled()) ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<P>(args)...);
}

// Cooperative launch: the driver either makes every CTA of the grid resident at once or refuses the launch, which is
// what a kernel with a grid-wide meeting point needs when other streams may hold part of the GPU.
template <typename... P, typename... A>
static inline cudaError_t oxq_launch_cooperative(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, A&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeCooperative;
    attr.val.cooperative = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<P>(args)...);
}

// FP8 (or, with int8 = true, W8A8 with per-row scales) GEMM for up to 8 batch rows (csrc/oxq_gemm_fp8_gemv.cu);
// arguments already validated by the entry points.
cudaError_t oxq_fp8_gemv_launch(oxq_handle* h, int m, int n, int k, const uint8_t* x, int64_t ldx, const uint8_t* w, int64_t ldw,
                                const float* sx, const float* sw, float alpha, void* y, int64_t ldy, bool swiglu, bool int8 = false);

namespace oxq {

__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Brings a line into the L2 without returning data.  The weight-streaming kernels use it for their first weights
// before pdl_wait(): the kernel before this one in the stream may still be writing those weights (a quantizer
// followed directly by the GEMM), so nothing may be *read* yet, but the L2 is the point of coherence and a line
// that is written after it was prefetched is simply updated there.
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Loads `V` consecutive elements of dtype T as floats.  p must be aligned to V * sizeof(T).
template <typename T> struct Elem;
template <> struct Elem<float> {
    static constexpr int kDtype = OXQ_F32;
    __device__ static __forceinline__ float to_f32(float v) { return v; }
    __device__ static __forceinline__ float from_f32(float v) { return v; }
};
template <> struct Elem<__nv_bfloat16> {
    static constexpr int kDtype = OXQ_BF16;
    __device__ static __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
    __device__ static __forceinline__ __nv_bfloat16 from_f32(float v) { return __float2bfloat16_rn(v); }
};
template <> struct Elem<__half> {
    static constexpr int kDtype = OXQ_F16;
    __device__ static __forceinline__ float to_f32(__half v) { return __half2float(v); }
    __device__ static __forceinline__ __half from_f32(float v) { return __float2half_rn(v); }
};

// 16-byte vector of T
template <typename T> struct alignas(16) Vec16 {
    static constexpr int N = 16 / sizeof(T);
    T v[N];
};

template <typename T>
__device__ __forceinline__ Vec16<T> ld16(const T* p) {
    Vec16<T> r;
    *reinterpret_cast<uint4*>(&r) = __ldg(reinterpret_cast<const uint4*>(p));
    return r;
}
// streaming variant: data that is read exactly once should not displace what must stay in L2
template <typename T>
__device__ __forceinline__ Vec16<T> ld16_stream(const T* p) {
    Vec16<T> r;
    uint4 u;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(u.x), "=r"(u.y), "=r"(u.z), "=r"(u.w) : "l"(p));
    *reinterpret_cast<uint4*>(&r) = u;
    return r;
}

__device__ __forceinline__ float round_mode(float v, int rounding) {
    // HALF_EVEN: rintf (cvt.rni).  HALF_AWAY: roundf, the reference's f32::round.
    return rounding == OXQ_ROUND_HALF_AWAY ? roundf(v) : rintf(v);
}

// two f32 -> two E4M3 bytes (RNE, satfinite); `lo` lands in bits [0,8)
__device__ __forceinline__ uint16_t cvt_e4m3x2(float lo, float hi) {
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    return r;
}
// two f32 -> two E2M1 nibbles in one byte (RNE, satfinite); `lo` lands in bits [0,4)
__device__ __forceinline__ uint8_t cvt_e2m1x2(float lo, float hi) {
    uint16_t r;
    asm("{ .reg .b8 t; cvt.rn.satfinite.e2m1x2.f32 t, %1, %2; cvt.u16.u8 %0, t; }" : "=h"(r) : "f"(hi), "f"(lo));
    return (uint8_t)r;
}
__device__ __forceinline__ float e4m3_to_f32(uint8_t b) {
    uint32_t h2;
    uint16_t in = b;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(in));
    return __half2float(__ushort_as_half((unsigned short)(h2 & 0xFFFFu)));
}
__device__ __forceinline__ float e2m1_to_f32(uint32_t nib) {
    // {0, .5, 1, 1.5, 2, 3, 4, 6} with sign bit 3
    uint32_t e = (nib >> 1) & 3u, m = nib & 1u;
    float v = e == 0 ? 0.5f * (float)m : (1.0f + 0.5f * (float)m) * (float)(1u << (e - 1));
    return (nib & 8u) ? -v : v;
}
// exact 2^e for e in [-127, 127]
__device__ __forceinline__ float pow2_of(int e) {
    return e >= -126 ? __uint_as_float((uint32_t)(e + 127) << 23) : __uint_as_float(0x00400000u);
}

// IEEE-exact x / s for a positive divisor that is shared by many elements: the correctly rounded reciprocal
// y = RN(1/s) is computed once; each quotient is then q0 = RN(x*y), r = x - s*q0 (exact, one FMA),
// q = RN(q0 + r*y), which equals RN(x/s) (Markstein's theorem) -- three FMA-pipe operations instead of a
// division sequence that re-evaluates the reciprocal for every element.  Outside the divisor range where
// the remainder is exactly representable the true division is used instead.
struct InvDiv {
    float s, y;
    bool fast;
};
__device__ __forceinline__ InvDiv make_invdiv(float s) {
    InvDiv d;
    d.s = s;
    d.y = __frcp_rn(s);
    d.fast = s >= 0x1p-60f && s <= 0x1p60f;
    return d;
}
// Variant for callers that know |x / s| cannot overflow (s was derived from the maximum of the data, so a
// non-finite x would have made s non-finite and taken the slow path) and that do not care about the sign of a
// zero quotient (integer codes): the multiply and the two FMAs only.
__device__ __forceinline__ float div_exact_bounded(float x, const InvDiv& d) {
    if (!d.fast) return __fdiv_rn(x, d.s);
    const float q0 = x * d.y;
    return fmaf(fmaf(-d.s, q0, x), d.y, q0);
}
// Same, keeping the sign of zero (FP8 / FP4 codes show it).
__device__ __forceinline__ float div_exact_bounded_signed(float x, const InvDiv& d) {
    if (!d.fast) return __fdiv_rn(x, d.s);
    const float q0 = x * d.y;
    return copysignf(fmaf(fmaf(-d.s, q0, x), d.y, q0), x);
}
__device__ __forceinline__ float div_exact(float x, const InvDiv& d) {
    if (!d.fast) return __fdiv_rn(x, d.s);
    const float q0 = x * d.y;
    float q = fmaf(fmaf(-d.s, q0, x), d.y, q0);
    // s > 0, so the quotient carries the sign of x; forcing it keeps -0 (the correction step would give +0),
    // which shows in FP8 / FP4 codes
    q = copysignf(q, x);
    // an infinite q0 (x = +-Inf, or overflow) makes the remainder NaN: return q0 then.  NaN inputs give NaN both ways.
    return q != q ? q0 : q;
}

// offset of scale factor (row r, sf column c) in the tiled order consumed by the tensor-core scale
// loads: tiles of 128 rows x 4 columns (512 bytes), tile order row-tile major; inside a tile the
// byte of (r, c) sits at (r % 32) * 16 + (r % 128) / 32 * 4 + c % 4.
__host__ __device__ __forceinline__ size_t sf_mma_offset(int64_t r, int64_t c, int64_t sf_cols) {
    int64_t col_tiles = (sf_cols + 3) / 4;
    return (size_t)(((r >> 7) * col_tiles + (c >> 2)) * 512 + (r & 31) * 16 + ((r & 127) >> 5) * 4 + (c & 3));
}

// 32-bit form for the kernels (row < 2^31 / 128 tiles etc. is checked on the host)
__device__ __forceinline__ uint32_t sf_mma_offset32(uint32_t r, uint32_t c, uint32_t col_tiles) {
    return ((r >> 7) * col_tiles + (c >> 2)) * 512u + (r & 31u) * 16u + ((r & 127u) >> 5) * 4u + (c & 3u);
}

}  // namespace oxq
