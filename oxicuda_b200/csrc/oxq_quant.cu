// Memory-bound quantize / dequantize kernels: every element of the input crosses HBM once, with
// 128-bit coalesced accesses, row or block statistics reduced by warp shuffles, codes packed in
// registers.  Rounding rules are the ones the CPU oracle states; divisions are IEEE (__fdiv_rn).
#include "oxq_common.cuh"
#include <stdlib.h>

namespace oxq {

// ------------------------------------------------------------------------------------------------
// INT8 symmetric per-row
// ------------------------------------------------------------------------------------------------

// x / scale -> int8 code in the low byte of the result.  The scale comes from the row's own maximum, so
// |x / scale| <= 127 (+ rounding) for every finite x and an Inf in the row takes the slow path of div_exact.
// Rounding happens in the FMA pipe: adding 1.5 * 2^23 leaves round-to-nearest-even(v) in the low mantissa
// bits (two's complement), so no conversion instruction is needed.  Half-away differs from half-even only at
// exact ties whose even neighbour is the one nearer zero.
__device__ __forceinline__ uint32_t quant_i8(float x, const InvDiv& scale, int rounding) {
    float v = div_exact_bounded(x, scale);
    v = v != v ? 0.0f : v;                                  // NaN -> code 0 (Rust `as i32`)
    v = fminf(fmaxf(v, -127.0f), 127.0f);
    const float m = v + 12582912.0f;                        // RNE(v) + 1.5 * 2^23
    uint32_t code = __float_as_uint(m);
    if (rounding == OXQ_ROUND_HALF_AWAY) {
        const float r = m - 12582912.0f;                    // RNE(v) as a float
        if (fabsf(v - r) == 0.5f && fabsf(r) < fabsf(v)) code += v < 0.0f ? 0xFFFFFFFFu : 1u;
    }
    return code & 0xFFu;
}

// Fast form for a scale derived from the row's own maximum and inside the exact-division range: finite inputs give
// quotients within +-127 (+ rounding), so no clamp; a NaN gives code 0.  ROUND is a compile-time constant here.
// Half away from zero is trunc(v + copysign(pred(0.5), v)): the sum rounds to the next integer exactly when the
// fraction of |v| is at least one half.
template <int ROUND>
__device__ __forceinline__ uint32_t quant_i8_fast(float x, const InvDiv& d) {
    const float q0 = x * d.y;
    float v = fmaf(fmaf(-d.s, q0, x), d.y, q0);
    v = v != v ? 0.0f : v;
    if (ROUND == OXQ_ROUND_HALF_AWAY) {
        const float half = __uint_as_float((__float_as_uint(v) & 0x80000000u) | 0x3EFFFFFFu);
        return (uint32_t)__float2int_rz(v + half);
    }
    return __float_as_uint(v + 12582912.0f);                // RNE(v) in the low mantissa byte
}
__device__ __forceinline__ uint32_t pack4_low(uint32_t a, uint32_t b, uint32_t c, uint32_t e) {
    return __byte_perm(__byte_perm(a, b, 0x0040), __byte_perm(c, e, 0x0040), 0x5410);
}

// One CTA per row at a time (grid-stride over rows).  Each thread keeps up to NV float4 of the row in
// registers, so a row of up to 256*4*NV floats is read from HBM exactly once (longer rows are read a second
// time for the quantize pass), and the next row of the CTA is already being fetched while the current one is
// reduced, quantised and stored.
template <int NV, int ROUND>
__global__ void __launch_bounds__(256) int8_quant_rows_kernel(const float* __restrict__ x, int64_t rows, int64_t cols,
                                                              int8_t* __restrict__ q, float* __restrict__ scales) {
    constexpr int rounding = ROUND;
    pdl_trigger();
    pdl_wait();
    __shared__ float s_red[2][8];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t nvec = cols >> 2;
    float4 cur[NV], nxt[NV];
    int64_t row = blockIdx.x;
    if (row < rows) {
        const float4* xr = reinterpret_cast<const float4*>(x + row * cols);
#pragma unroll
        for (int i = 0; i < NV; i++) {
            const int64_t idx = tid + (int64_t)i * 256;
            cur[i] = idx < nvec ? __ldcs(xr + idx) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    int par = 0;
    for (; row < rows; row += gridDim.x, par ^= 1) {
        const int64_t next = row + gridDim.x;
        if (next < rows) {
            const float4* xn = reinterpret_cast<const float4*>(x + next * cols);
#pragma unroll
            for (int i = 0; i < NV; i++) {
                const int64_t idx = tid + (int64_t)i * 256;
                nxt[i] = idx < nvec ? __ldcs(xn + idx) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
        const float4* xr = reinterpret_cast<const float4*>(x + row * cols);
        float amax = 0.0f;
#pragma unroll
        for (int i = 0; i < NV; i++)
            amax = fmaxf(amax, fmaxf(fmaxf(fabsf(cur[i].x), fabsf(cur[i].y)), fmaxf(fabsf(cur[i].z), fabsf(cur[i].w))));
        for (int64_t idx = tid + (int64_t)NV * 256; idx < nvec; idx += 256) {
            float4 t = __ldg(xr + idx);
            amax = fmaxf(amax, fmaxf(fmaxf(fabsf(t.x), fabsf(t.y)), fmaxf(fabsf(t.z), fabsf(t.w))));
        }
        amax = warp_max(amax);
        if (lane == 0) s_red[par][warp] = amax;             // double-buffered: one barrier per row is enough
        __syncthreads();
        amax = s_red[par][0];
#pragma unroll
        for (int w = 1; w < 8; w++) amax = fmaxf(amax, s_red[par][w]);
        const float scale_f = __fdiv_rn(fmaxf(amax, 1e-8f), 127.0f);
        if (tid == 0) scales[row] = scale_f;
        const InvDiv scale = make_invdiv(scale_f);
        uint32_t* qr = reinterpret_cast<uint32_t*>(q + row * cols);
        if (scale.fast) {                                    // the whole CTA takes the same side
#pragma unroll
            for (int i = 0; i < NV; i++) {
                const int64_t idx = tid + (int64_t)i * 256;
                if (idx < nvec)
                    __stcs(qr + idx, pack4_low(quant_i8_fast<ROUND>(cur[i].x, scale), quant_i8_fast<ROUND>(cur[i].y, scale),
                                               quant_i8_fast<ROUND>(cur[i].z, scale), quant_i8_fast<ROUND>(cur[i].w, scale)));
            }
        } else {
#pragma unroll
            for (int i = 0; i < NV; i++) {
                const int64_t idx = tid + (int64_t)i * 256;
                if (idx < nvec) {
                    uint32_t p = quant_i8(cur[i].x, scale, rounding) | (quant_i8(cur[i].y, scale, rounding) << 8) |
                                 (quant_i8(cur[i].z, scale, rounding) << 16) | (quant_i8(cur[i].w, scale, rounding) << 24);
                    __stcs(qr + idx, p);
                }
            }
        }
        for (int64_t idx = tid + (int64_t)NV * 256; idx < nvec; idx += 256) {
            float4 t = __ldg(xr + idx);
            qr[idx] = quant_i8(t.x, scale, rounding) | (quant_i8(t.y, scale, rounding) << 8) |
                      (quant_i8(t.z, scale, rounding) << 16) | (quant_i8(t.w, scale, rounding) << 24);
        }
#pragma unroll
        for (int i = 0; i < NV; i++) cur[i] = nxt[i];
    }
}

// Any cols / alignment: scalar accesses.
__global__ void __launch_bounds__(256) int8_quant_rows_scalar_kernel(const float* __restrict__ x, int64_t rows, int64_t cols,
                                                                     int8_t* __restrict__ q, float* __restrict__ scales,
                                                                     int rounding) {
    pdl_trigger();
    pdl_wait();
    __shared__ float s_red[8];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const float* xr = x + row * cols;
        float amax = 0.0f;
        for (int64_t i = tid; i < cols; i += 256) amax = fmaxf(amax, fabsf(xr[i]));
        amax = warp_max(amax);
        __syncthreads();
        if (lane == 0) s_red[warp] = amax;
        __syncthreads();
        amax = s_red[0];
        for (int w = 1; w < 8; w++) amax = fmaxf(amax, s_red[w]);
        const float scale_f = __fdiv_rn(fmaxf(amax, 1e-8f), 127.0f);
        if (tid == 0) scales[row] = scale_f;
        const InvDiv scale = make_invdiv(scale_f);
        for (int64_t i = tid; i < cols; i += 256) q[row * cols + i] = (int8_t)quant_i8(xr[i], scale, rounding);
    }
}

// 16 codes per thread: one 16-byte load, four 16-byte stores.
__global__ void __launch_bounds__(256) int8_dequant_rows_kernel(const int8_t* __restrict__ q, const float* __restrict__ scales,
                                                                int64_t rows, int64_t cols, float* __restrict__ y) {
    pdl_trigger();
    pdl_wait();
    const int64_t nchunk = rows * cols / 16;
    for (int64_t c = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; c < nchunk; c += (int64_t)gridDim.x * blockDim.x) {
        const int64_t e = c * 16;
        const float s = __ldg(scales + e / cols);
        uint4 u = __ldcs(reinterpret_cast<const uint4*>(q + e));
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
        float4* yo = reinterpret_cast<float4*>(y + e);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            float4 o;
            o.x = (float)(int8_t)(w[i] & 0xFF) * s;
            o.y = (float)(int8_t)((w[i] >> 8) & 0xFF) * s;
            o.z = (float)(int8_t)((w[i] >> 16) & 0xFF) * s;
            o.w = (float)(int8_t)(w[i] >> 24) * s;
            __stcs(yo + i, o);
        }
    }
}
__global__ void __launch_bounds__(256) int8_dequant_rows_scalar_kernel(const int8_t* __restrict__ q, const float* __restrict__ scales,
                                                                       int64_t rows, int64_t cols, float* __restrict__ y) {
    pdl_trigger();
    pdl_wait();
    const int64_t n = rows * cols;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        y[i] = (float)q[i] * scales[i / cols];
}

// ------------------------------------------------------------------------------------------------
// absmax (per tensor)
// ------------------------------------------------------------------------------------------------

// Each CTA folds a strided slice of the tensor, then one atomicMax per CTA on the bit pattern of
// the non-negative result (ordering of non-negative floats == ordering of their bits).
// |x| and max are taken on packed pairs for the 16-bit types (one logic and one packed-max instruction per two
// elements), so the kernel stays limited by HBM rather than by the ALU pipe.  NaNs are skipped, as fmaxf does.
template <typename T> struct AbsMaxAcc;
template <> struct AbsMaxAcc<float> {
    float m = 0.0f;
    __device__ __forceinline__ void add(const uint4& u) {
        m = fmaxf(m, fmaxf(fmaxf(fabsf(__uint_as_float(u.x)), fabsf(__uint_as_float(u.y))),
                           fmaxf(fabsf(__uint_as_float(u.z)), fabsf(__uint_as_float(u.w)))));
    }
    __device__ __forceinline__ float result() const { return m; }
};
template <> struct AbsMaxAcc<__nv_bfloat16> {
    __nv_bfloat162 m = __floats2bfloat162_rn(0.0f, 0.0f);
    __device__ __forceinline__ void add1(uint32_t w) {
        const uint32_t a = w & 0x7FFF7FFFu;
        m = __hmax2(m, *reinterpret_cast<const __nv_bfloat162*>(&a));
    }
    __device__ __forceinline__ void add(const uint4& u) { add1(u.x); add1(u.y); add1(u.z); add1(u.w); }
    __device__ __forceinline__ float result() const { return fmaxf(__low2float(m), __high2float(m)); }
};
template <> struct AbsMaxAcc<__half> {
    __half2 m = __floats2half2_rn(0.0f, 0.0f);
    __device__ __forceinline__ void add1(uint32_t w) {
        const uint32_t a = w & 0x7FFF7FFFu;
        m = __hmax2(m, *reinterpret_cast<const __half2*>(&a));
    }
    __device__ __forceinline__ void add(const uint4& u) { add1(u.x); add1(u.y); add1(u.z); add1(u.w); }
    __device__ __forceinline__ float result() const { return fmaxf(__low2float(m), __high2float(m)); }
};

// cells[0] accumulates the maximum, cells[1] counts finished CTAs; the last CTA publishes the result and puts
// both cells back to zero, so no memset is needed between calls.
template <typename T>
__global__ void __launch_bounds__(256) absmax_kernel(const T* __restrict__ x, int64_t n, float* __restrict__ out, unsigned int* __restrict__ cells) {
    pdl_trigger();
    pdl_wait();
    constexpr int V = Vec16<T>::N;
    __shared__ float s_red[8];
    const int64_t nvec = n / V;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const uint4* xv = reinterpret_cast<const uint4*>(x);
    AbsMaxAcc<T> a0, a1, a2, a3;
    int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    for (; i + 7 * stride < nvec; i += 8 * stride) {
        const uint4 u0 = __ldg(xv + i), u1 = __ldg(xv + i + stride), u2 = __ldg(xv + i + 2 * stride), u3 = __ldg(xv + i + 3 * stride);
        const uint4 u4 = __ldg(xv + i + 4 * stride), u5 = __ldg(xv + i + 5 * stride), u6 = __ldg(xv + i + 6 * stride), u7 = __ldg(xv + i + 7 * stride);
        a0.add(u0); a1.add(u1); a2.add(u2); a3.add(u3);
        a0.add(u4); a1.add(u5); a2.add(u6); a3.add(u7);
    }
    for (; i < nvec; i += stride) a0.add(__ldg(xv + i));
    float m = fmaxf(fmaxf(a0.result(), a1.result()), fmaxf(a2.result(), a3.result()));
    if (blockIdx.x == 0) {
        for (int64_t t = nvec * V + threadIdx.x; t < n; t += blockDim.x) m = fmaxf(m, fabsf(Elem<T>::to_f32(x[t])));
    }
    m = warp_max(m);
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; w++) m = fmaxf(m, s_red[w]);
        atomicMax(cells, __float_as_uint(m));
        __threadfence();
        if (atomicAdd(cells + 1, 1u) == gridDim.x - 1) {
            __threadfence();
            out[0] = __uint_as_float(atomicExch(cells, 0u));
            cells[1] = 0u;
        }
    }
}

// ------------------------------------------------------------------------------------------------
// FP8 E4M3 per tensor
// ------------------------------------------------------------------------------------------------

// Literal Fp8Codec::fp32_to_fp8 for E4M3 (truncation, |v| >= 256 -> 448, subnormal shift).
__device__ __forceinline__ uint8_t e4m3_refcompat(float v) {
    v = fminf(fmaxf(v, -448.0f), 448.0f);
    uint32_t bits = __float_as_uint(v);
    uint32_t sign = bits >> 31;
    int exp32 = (int)((bits >> 23) & 0xFF);
    uint32_t man32 = bits & 0x007FFFFFu;
    if (v == 0.0f) return (uint8_t)(sign << 7);
    int e = exp32 - 127 + 7;
    if (e <= 0) {
        uint32_t full = (man32 | 0x00800000u) >> 1;
        uint32_t shift = (uint32_t)(1 - e) + 20u;
        if (shift >= 24) return (uint8_t)(sign << 7);
        return (uint8_t)((sign << 7) | ((full >> shift) & 7u));
    }
    if (e >= 15) return (uint8_t)((sign << 7) | 0x7E);
    return (uint8_t)((sign << 7) | ((uint32_t)e << 3) | ((man32 >> 20) & 7u));
}
// Literal Fp8Codec::fp8_to_fp32 for E4M3 (subnormals decode as 2^-6 * (1 + m/8)).
__device__ __forceinline__ float e4m3_refcompat_decode(uint8_t b) {
    uint32_t sign = b >> 7, e = (b >> 3) & 0xF, m = b & 7;
    if (e == 15 && m == 7) return __uint_as_float(0x7FC00000u);
    if (e == 0) return m == 0 ? __uint_as_float(sign << 31) : __uint_as_float((sign << 31) | (121u << 23) | (m << 20));
    return __uint_as_float((sign << 31) | ((e + 120u) << 23) | (m << 20));
}

// Items of 8 elements (one 8-byte store); every thread keeps FP8_ILP items in flight, item j of a thread is
// FP8_ILP-strided by the warp so each load instruction of a warp covers one contiguous span.  If
// stats != nullptr the scale is derived from stats[0] (absmax) as absmax/448 (1.0 when absmax == 0) and
// thread 0 records it in stats[1].
constexpr int FP8_ILP = 4;
template <typename T, int MODE, bool BOUNDED>
__global__ void __launch_bounds__(256) fp8_quant_kernel(const T* __restrict__ x, int64_t n, const float* __restrict__ scale_ptr,
                                                        float* __restrict__ stats, uint8_t* __restrict__ q) {
    pdl_trigger();
    pdl_wait();
    constexpr int V = Vec16<T>::N;                          // elements per 16-byte load (8 or 4)
    constexpr int L = 8 / V;                                // 16-byte loads per item (1 or 2)
    float scale_f;
    if (stats) {
        const float am = stats[0];
        scale_f = am > 0.0f ? __fdiv_rn(am, 448.0f) : 1.0f;
        if (blockIdx.x == 0 && threadIdx.x == 0) stats[1] = scale_f;
    } else {
        scale_f = __ldg(scale_ptr);
    }
    const InvDiv scale = make_invdiv(scale_f);
    const int64_t nitems = n / 8;
    const int lane = threadIdx.x & 31;
    const int64_t warp_global = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t base = warp_global * (32 * FP8_ILP); base < nitems; base += nwarps * (32 * FP8_ILP)) {
        Vec16<T> in[FP8_ILP][L];
#pragma unroll
        for (int j = 0; j < FP8_ILP; j++) {
            const int64_t it = base + j * 32 + lane;
            if (it < nitems) {
#pragma unroll
                for (int l = 0; l < L; l++) in[j][l] = ld16_stream(x + it * 8 + l * V);
            }
        }
#pragma unroll
        for (int j = 0; j < FP8_ILP; j++) {
            const int64_t it = base + j * 32 + lane;
            if (it < nitems) {
                float f[8];
#pragma unroll
                for (int l = 0; l < L; l++)
#pragma unroll
                    for (int e = 0; e < V; e++)
                        f[l * V + e] = BOUNDED ? div_exact_bounded_signed(Elem<T>::to_f32(in[j][l].v[e]), scale) : div_exact(Elem<T>::to_f32(in[j][l].v[e]), scale);
                uint32_t w[2];
#pragma unroll
                for (int i = 0; i < 2; i++) {
                    if (MODE == OXQ_FP8_SPEC_RNE) {
                        w[i] = (uint32_t)cvt_e4m3x2(f[4 * i], f[4 * i + 1]) | ((uint32_t)cvt_e4m3x2(f[4 * i + 2], f[4 * i + 3]) << 16);
                    } else {
                        w[i] = (uint32_t)e4m3_refcompat(f[4 * i]) | ((uint32_t)e4m3_refcompat(f[4 * i + 1]) << 8) |
                               ((uint32_t)e4m3_refcompat(f[4 * i + 2]) << 16) | ((uint32_t)e4m3_refcompat(f[4 * i + 3]) << 24);
                    }
                }
                __stcs(reinterpret_cast<uint2*>(q + it * 8), make_uint2(w[0], w[1]));
            }
        }
    }
    if (blockIdx.x == 0) {                                  // ragged tail
        for (int64_t t = nitems * 8 + threadIdx.x; t < n; t += blockDim.x) {
            const float f = div_exact(Elem<T>::to_f32(x[t]), scale);
            q[t] = MODE == OXQ_FP8_SPEC_RNE ? (uint8_t)(cvt_e4m3x2(f, 0.0f) & 0xFF) : e4m3_refcompat(f);
        }
    }
}

// absmax and quantize in one launch.  All CTAs are resident (a cooperative launch with the grid sized from the
// occupancy: the driver refuses it rather than run part of the grid), so after the first pass they meet at a counter
// in the handle's cells, read the maximum and run the second pass over the tensor in reverse order: what the first
// pass read last is still in L2 (a whole activation tensor of tens of MB is).  The wait on the counter is bounded; on
// expiry the status word is set and stats[0] and stats[1] become NaN, so the partial maximum cannot pass for a result.
// cells[0] maximum, cells[1] arrivals, cells[2] departures, cells[3] set by a CTA whose wait expired; the last CTA to
// leave puts all four back to zero.
template <typename T>
__global__ void __launch_bounds__(256) fp8_quant_dynamic_fused_kernel(const T* __restrict__ x, int64_t n, float* __restrict__ stats,
                                                                      uint8_t* __restrict__ q, unsigned int* __restrict__ cells,
                                                                      int32_t* __restrict__ status) {
    pdl_trigger();
    pdl_wait();
    constexpr int V = Vec16<T>::N;
    constexpr int L = 8 / V;
    __shared__ float s_red[8];
    __shared__ float s_amax;
    // ---- pass 1: maximum --------------------------------------------------------------------------
    {
        const int64_t nvec = n / V;
        const int64_t stride = (int64_t)gridDim.x * blockDim.x;
        const uint4* xv = reinterpret_cast<const uint4*>(x);
        AbsMaxAcc<T> a0, a1, a2, a3;
        int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
        for (; i + 7 * stride < nvec; i += 8 * stride) {
            const uint4 u0 = __ldg(xv + i), u1 = __ldg(xv + i + stride), u2 = __ldg(xv + i + 2 * stride), u3 = __ldg(xv + i + 3 * stride);
            const uint4 u4 = __ldg(xv + i + 4 * stride), u5 = __ldg(xv + i + 5 * stride), u6 = __ldg(xv + i + 6 * stride), u7 = __ldg(xv + i + 7 * stride);
            a0.add(u0); a1.add(u1); a2.add(u2); a3.add(u3);
            a0.add(u4); a1.add(u5); a2.add(u6); a3.add(u7);
        }
        for (; i < nvec; i += stride) a0.add(__ldg(xv + i));
        float m = fmaxf(fmaxf(a0.result(), a1.result()), fmaxf(a2.result(), a3.result()));
        if (blockIdx.x == 0) {
            for (int64_t t = nvec * V + threadIdx.x; t < n; t += blockDim.x) m = fmaxf(m, fabsf(Elem<T>::to_f32(x[t])));
        }
        m = warp_max(m);
        if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = m;
        __syncthreads();
        if (threadIdx.x == 0) {
            for (int w = 1; w < 8; w++) m = fmaxf(m, s_red[w]);
            atomicMax(cells, __float_as_uint(m));
            __threadfence();
            atomicAdd(cells + 1, 1u);
            // every CTA of the grid is resident, so the others arrive; give up after two seconds all the same
            uint64_t t0, t1;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
            const volatile unsigned int* arrivals = cells + 1;
            for (uint32_t it = 0; *arrivals < gridDim.x; ++it) {
                if ((it & 1023u) == 1023u) {
                    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t1));
                    if (t1 - t0 > 2000000000ull) { atomicExch(status, OXQ_ERR_DEVICE_TIMEOUT); atomicExch(cells + 3, 1u); break; }
                }
            }
            __threadfence();
            s_amax = __uint_as_float(*reinterpret_cast<const volatile unsigned int*>(cells));
        }
        __syncthreads();
    }
    const float am = s_amax;
    const float scale_f = am > 0.0f ? __fdiv_rn(am, 448.0f) : 1.0f;
    if (blockIdx.x == 0 && threadIdx.x == 0) { stats[0] = am; stats[1] = scale_f; }
    const InvDiv scale = make_invdiv(scale_f);
    // ---- pass 2: codes, from the end of the tensor backwards ---------------------------------------------
    const int64_t nitems = n / 8;
    const int lane = threadIdx.x & 31;
    const int64_t warp_global = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const int64_t nchunks = (nitems + 32 * FP8_ILP - 1) / (32 * FP8_ILP);
    for (int64_t c = nchunks - 1 - warp_global; c >= 0; c -= nwarps) {
        const int64_t base = c * (32 * FP8_ILP);
        Vec16<T> in[FP8_ILP][L];
#pragma unroll
        for (int j = 0; j < FP8_ILP; j++) {
            const int64_t it = base + j * 32 + lane;
            if (it < nitems) {
#pragma unroll
                for (int l = 0; l < L; l++) in[j][l] = ld16_stream(x + it * 8 + l * V);
            }
        }
#pragma unroll
        for (int j = 0; j < FP8_ILP; j++) {
            const int64_t it = base + j * 32 + lane;
            if (it < nitems) {
                float f[8];
#pragma unroll
                for (int l = 0; l < L; l++)
#pragma unroll
                    for (int e = 0; e < V; e++) f[l * V + e] = div_exact_bounded_signed(Elem<T>::to_f32(in[j][l].v[e]), scale);
                const uint32_t w0 = (uint32_t)cvt_e4m3x2(f[0], f[1]) | ((uint32_t)cvt_e4m3x2(f[2], f[3]) << 16);
                const uint32_t w1 = (uint32_t)cvt_e4m3x2(f[4], f[5]) | ((uint32_t)cvt_e4m3x2(f[6], f[7]) << 16);
                __stcs(reinterpret_cast<uint2*>(q + it * 8), make_uint2(w0, w1));
            }
        }
    }
    if (blockIdx.x == 0) {                                  // ragged tail
        for (int64_t t = nitems * 8 + threadIdx.x; t < n; t += blockDim.x)
            q[t] = (uint8_t)(cvt_e4m3x2(div_exact(Elem<T>::to_f32(x[t]), scale), 0.0f) & 0xFF);
    }
    // ---- leave the cells as they were found --------------------------------------------------------------------
    __syncthreads();
    if (threadIdx.x == 0 && atomicAdd(cells + 2, 1u) == gridDim.x - 1) {
        __threadfence();
        if (*reinterpret_cast<const volatile unsigned int*>(cells + 3) != 0u) {        // some CTA gave up waiting: no valid maximum
            stats[0] = __uint_as_float(0x7FC00000u); stats[1] = __uint_as_float(0x7FC00000u);
        }
        cells[0] = 0u; cells[1] = 0u; cells[2] = 0u; cells[3] = 0u;
        __threadfence();
    }
}

// Small tensors (a decode step's activations): one CTA does both passes, the second from L1 / L2, so the dynamic
// quantizer is one launch of a few microseconds instead of two.  Same arithmetic as the two-launch form.
constexpr int64_t FP8_SMALL_MAX = 131072;
template <typename T>
__global__ void __launch_bounds__(1024) fp8_quant_dynamic_small_kernel(const T* __restrict__ x, int64_t n, float* __restrict__ stats,
                                                                       uint8_t* __restrict__ q) {
    pdl_trigger();
    pdl_wait();
    constexpr int V = Vec16<T>::N;
    constexpr int L = 8 / V;
    __shared__ float s_red[32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t nvec = n / V;
    const uint4* xv = reinterpret_cast<const uint4*>(x);
    AbsMaxAcc<T> acc;
    for (int64_t i = tid; i < nvec; i += 1024) acc.add(__ldg(xv + i));
    float m = acc.result();
    for (int64_t t = nvec * V + tid; t < n; t += 1024) m = fmaxf(m, fabsf(Elem<T>::to_f32(x[t])));
    m = warp_max(m);
    if (lane == 0) s_red[warp] = m;
    __syncthreads();
    m = s_red[0];
#pragma unroll
    for (int w = 1; w < 32; w++) m = fmaxf(m, s_red[w]);
    const float scale_f = m > 0.0f ? __fdiv_rn(m, 448.0f) : 1.0f;
    if (tid == 0) { stats[0] = m; stats[1] = scale_f; }
    const InvDiv scale = make_invdiv(scale_f);
    const int64_t nitems = n / 8;
    for (int64_t it = tid; it < nitems; it += 1024) {
        float f[8];
#pragma unroll
        for (int l = 0; l < L; l++) {
            const Vec16<T> in = ld16(x + it * 8 + l * V);
#pragma unroll
            for (int e = 0; e < V; e++) f[l * V + e] = div_exact_bounded_signed(Elem<T>::to_f32(in.v[e]), scale);
        }
        const uint32_t w0 = (uint32_t)cvt_e4m3x2(f[0], f[1]) | ((uint32_t)cvt_e4m3x2(f[2], f[3]) << 16);
        const uint32_t w1 = (uint32_t)cvt_e4m3x2(f[4], f[5]) | ((uint32_t)cvt_e4m3x2(f[6], f[7]) << 16);
        *reinterpret_cast<uint2*>(q + it * 8) = make_uint2(w0, w1);
    }
    for (int64_t t = nitems * 8 + tid; t < n; t += 1024)
        q[t] = (uint8_t)(cvt_e4m3x2(div_exact(Elem<T>::to_f32(x[t]), scale), 0.0f) & 0xFF);
}

template <typename T, int MODE>
__global__ void __launch_bounds__(256) fp8_dequant_kernel(const uint8_t* __restrict__ q, int64_t n, const float* __restrict__ scale_ptr,
                                                          T* __restrict__ y) {
    pdl_trigger();
    pdl_wait();
    const float scale = __ldg(scale_ptr);
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        float v = MODE == OXQ_FP8_SPEC_RNE ? e4m3_to_f32(q[i]) : e4m3_refcompat_decode(q[i]);
        y[i] = Elem<T>::from_f32(v * scale);
    }
}

// ------------------------------------------------------------------------------------------------
// uint4 group-wise asymmetric with f16 scales
// ------------------------------------------------------------------------------------------------

// One warp owns 8 consecutive groups (so it also owns one packed zero-point word).  Per group the
// lanes hold group/32 elements each in 4-element pieces; min/max by shuffles; the four nibbles of a
// piece are merged with the neighbour lane's so even lanes store whole u32 words.
template <typename T, int GROUP>
__global__ void __launch_bounds__(256) int4g_quant_kernel(const T* __restrict__ x, int64_t ngroups, int rounding,
                                                          uint32_t* __restrict__ codes, uint16_t* __restrict__ scales,
                                                          uint32_t* __restrict__ zeros) {
    pdl_trigger();
    pdl_wait();
    constexpr int PIECES = GROUP / 128 > 0 ? GROUP / 128 : 1;  // 4-element pieces per lane per group
    constexpr int ACTIVE = GROUP >= 128 ? 32 : GROUP / 4;      // lanes that hold data
    const int lane = threadIdx.x & 31;
    const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t g0 = warp * 8; g0 < ngroups; g0 += nwarps * 8) {
        float v[8][PIECES][4];
#pragma unroll
        for (int g = 0; g < 8; g++) {
#pragma unroll
            for (int p = 0; p < PIECES; p++) {
                const int64_t e = (g0 + g) * GROUP + p * 128 + lane * 4;
                if (g0 + g < ngroups && lane < ACTIVE) {
                    if (sizeof(T) == 4) {
                        float4 t = __ldcs(reinterpret_cast<const float4*>(x + e));
                        v[g][p][0] = t.x; v[g][p][1] = t.y; v[g][p][2] = t.z; v[g][p][3] = t.w;
                    } else {
                        uint2 t = __ldcs(reinterpret_cast<const uint2*>(x + e));
                        const T* h = reinterpret_cast<const T*>(&t);
#pragma unroll
                        for (int j = 0; j < 4; j++) v[g][p][j] = Elem<T>::to_f32(h[j]);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 4; j++) v[g][p][j] = 0.0f;
                }
            }
        }
        uint32_t zword = 0;
#pragma unroll
        for (int g = 0; g < 8; g++) {
            float mn = INFINITY, mx = -INFINITY;
            if (lane < ACTIVE) {
#pragma unroll
                for (int p = 0; p < PIECES; p++)
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        // NaNs are skipped exactly as `if v < fmin` / `if v > fmax` skip them
                        mn = fminf(mn, v[g][p][j]);
                        mx = fmaxf(mx, v[g][p][j]);
                    }
            }
            mn = warp_min(mn);
            mx = warp_max(mx);
            float s32 = __fdiv_rn(fmaxf(mx - mn, 1e-8f), 15.0f);
            __half sh = __float2half_rn(s32);
            if ((__half_as_ushort(sh) & 0x7FFFu) == 0) sh = __ushort_as_half(1);
            const float s = __half2float(sh);
            const InvDiv sd = make_invdiv(s);
            float zf = roundf(div_exact(-mn, sd));
            zf = zf != zf ? 0.0f : fminf(fmaxf(zf, 0.0f), 15.0f);
            const uint32_t zp = (uint32_t)zf;
            if (g0 + g < ngroups) {
                zword |= zp << (4 * g);
                if (lane == 0) scales[g0 + g] = __half_as_ushort(sh);
#pragma unroll
                for (int p = 0; p < PIECES; p++) {
                    uint32_t nib4 = 0;
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        float t = round_mode(div_exact(v[g][p][j], sd) + zf, rounding);
                        t = t != t ? 0.0f : fminf(fmaxf(t, 0.0f), 15.0f);
                        nib4 |= ((uint32_t)t) << (4 * j);
                    }
                    const uint32_t other = __shfl_down_sync(0xffffffffu, nib4, 1);
                    if ((lane & 1) == 0 && lane < ACTIVE)
                        codes[((g0 + g) * GROUP + p * 128 + lane * 4) >> 3] = nib4 | (other << 16);
                }
            }
        }
        if (lane == 0) zeros[g0 >> 3] = zword;
    }
}

// Group 128, the shape the GEMMs use: 8 lanes share a group (16 elements each, as two runs of 8 consecutive
// elements = two whole code words, so no nibble exchange), a warp works on 4 groups at once and on 8 groups per
// pass, so it owns one packed zero-point word.  min / max need 3 + 3 shuffles per 16 elements.  Rounding runs in
// the FMA pipe: after the clamp to [0, 15] (which also maps NaN to 0), adding 1.5 * 2^23 leaves
// round-to-nearest-even in the low mantissa bits; half-away differs only at exact ties rounded down.
__device__ __forceinline__ uint32_t quant_u4(float x, const InvDiv& sd, float zf, int rounding) {
    const float t = fminf(fmaxf(div_exact_bounded(x, sd) + zf, 0.0f), 15.0f);
    const float m = t + 12582912.0f;
    uint32_t code = __float_as_uint(m);
    if (rounding == OXQ_ROUND_HALF_AWAY && t - (m - 12582912.0f) == 0.5f) code += 1u;
    return code & 0xFu;
}

template <typename T>
__global__ void __launch_bounds__(256) int4g128_quant_kernel(const T* __restrict__ x, int64_t ngroups, int rounding,
                                                             uint32_t* __restrict__ codes, uint16_t* __restrict__ scales,
                                                             uint32_t* __restrict__ zeros) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31, sub = lane >> 3, sl = lane & 7;
    const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t g0 = warp * 8; g0 < ngroups; g0 += nwarps * 8) {
        float v[2][2][8];                                   // [pass][run][element]
#pragma unroll
        for (int ps = 0; ps < 2; ps++) {
            const int64_t g = g0 + ps * 4 + sub;
#pragma unroll
            for (int j = 0; j < 2; j++) {
                const int64_t e = g * 128 + j * 64 + sl * 8;
                if (g < ngroups) {
                    if (sizeof(T) == 4) {
                        const float4 a = __ldg(reinterpret_cast<const float4*>(x + e)), b = __ldg(reinterpret_cast<const float4*>(x + e) + 1);
                        v[ps][j][0] = a.x; v[ps][j][1] = a.y; v[ps][j][2] = a.z; v[ps][j][3] = a.w;
                        v[ps][j][4] = b.x; v[ps][j][5] = b.y; v[ps][j][6] = b.z; v[ps][j][7] = b.w;
                    } else {
                        const uint4 u = __ldcs(reinterpret_cast<const uint4*>(x + e));
                        const T* hh = reinterpret_cast<const T*>(&u);
#pragma unroll
                        for (int q = 0; q < 8; q++) v[ps][j][q] = Elem<T>::to_f32(hh[q]);
                    }
                } else {
#pragma unroll
                    for (int q = 0; q < 8; q++) v[ps][j][q] = 0.0f;
                }
            }
        }
        uint32_t zcontrib = 0;
#pragma unroll
        for (int ps = 0; ps < 2; ps++) {
            const int64_t g = g0 + ps * 4 + sub;
            float mn = INFINITY, mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < 2; j++)
#pragma unroll
                for (int q = 0; q < 8; q++) { mn = fminf(mn, v[ps][j][q]); mx = fmaxf(mx, v[ps][j][q]); }   // NaNs skipped like `if v < fmin`
#pragma unroll
            for (int o = 4; o > 0; o >>= 1) {
                mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            }
            const float s32 = __fdiv_rn(fmaxf(mx - mn, 1e-8f), 15.0f);
            __half sh = __float2half_rn(s32);
            if ((__half_as_ushort(sh) & 0x7FFFu) == 0) sh = __ushort_as_half(1);
            const float sc = __half2float(sh);
            InvDiv sd = make_invdiv(sc);
            sd.fast = sd.fast && fmaxf(fabsf(mn), fabsf(mx)) < 0x1p100f;      // quotients of this group cannot overflow
            float zf = roundf(div_exact(-mn, sd));
            zf = zf != zf ? 0.0f : fminf(fmaxf(zf, 0.0f), 15.0f);
            if (g < ngroups) {
                if (sl == 0) {
                    scales[g] = __half_as_ushort(sh);
                    zcontrib |= ((uint32_t)zf) << (4 * (ps * 4 + sub));
                }
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    uint32_t w = 0;
#pragma unroll
                    for (int q = 0; q < 8; q++) w |= quant_u4(v[ps][j][q], sd, zf, rounding) << (4 * q);
                    __stcs(codes + ((g * 128 + j * 64 + sl * 8) >> 3), w);
                }
            }
        }
        const uint32_t zword = __reduce_or_sync(0xffffffffu, zcontrib);
        if (lane == 0) zeros[g0 >> 3] = zword;
    }
}

template <typename T>
__global__ void __launch_bounds__(256) int4g_dequant_kernel(const uint32_t* __restrict__ codes, const uint16_t* __restrict__ scales,
                                                            const uint32_t* __restrict__ zeros, int64_t nwords, int group,
                                                            T* __restrict__ y) {
    pdl_trigger();
    pdl_wait();
    for (int64_t w = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; w < nwords; w += (int64_t)gridDim.x * blockDim.x) {
        const int64_t gi = (w * 8) / group;
        const float s = __half2float(__ushort_as_half(scales[gi]));
        const int zp = (int)((zeros[gi >> 3] >> ((gi & 7) * 4)) & 0xF);
        const uint32_t c = __ldcs(codes + w);
        T o[8];
#pragma unroll
        for (int j = 0; j < 8; j++) o[j] = Elem<T>::from_f32((float)((int)((c >> (4 * j)) & 0xF) - zp) * s);
        if (sizeof(T) == 4) {
            float4* yo = reinterpret_cast<float4*>(y + w * 8);
            yo[0] = *reinterpret_cast<float4*>(&o[0]);
            yo[1] = *reinterpret_cast<float4*>(&o[4]);
        } else {
            *reinterpret_cast<uint4*>(y + w * 8) = *reinterpret_cast<uint4*>(&o[0]);
        }
    }
}

// ------------------------------------------------------------------------------------------------
// MXFP8 (E4M3 codes, E8M0 scale per 32) and NVFP4 (E2M1 codes, E4M3 scale per 16, f32 tensor scale)
// ------------------------------------------------------------------------------------------------

template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&f)[8]) {
    if (sizeof(T) == 4) {
        float4 a = __ldcs(reinterpret_cast<const float4*>(p)), b = __ldcs(reinterpret_cast<const float4*>(p) + 1);
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    } else {
        uint4 u = __ldcs(reinterpret_cast<const uint4*>(p));
        const T* h = reinterpret_cast<const T*>(&u);
#pragma unroll
        for (int j = 0; j < 8; j++) f[j] = Elem<T>::to_f32(h[j]);
    }
}

// 8 elements per item, 4 adjacent lanes form one 32-element block; BS_ILP items per thread in flight.
constexpr int BS_ILP = 4;
template <typename T>
__global__ void __launch_bounds__(256) mxfp8_quant_kernel(const T* __restrict__ x, int64_t rows, int64_t k,
                                                          uint8_t* __restrict__ codes, uint8_t* __restrict__ sf_rm,
                                                          uint8_t* __restrict__ sf_mma) {
    pdl_trigger();
    pdl_wait();
    const int64_t nitems = rows * k / 8;
    const int64_t sf_cols = k / 32;
    const uint32_t sf_col_tiles = (uint32_t)((sf_cols + 3) / 4);
    const int lane = threadIdx.x & 31;
    const int64_t warp_global = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    // warp-uniform trip count: the shuffles below need every lane of the warp
    for (int64_t base = warp_global * (32 * BS_ILP); base < nitems; base += nwarps * (32 * BS_ILP)) {
        float f[BS_ILP][8];
#pragma unroll
        for (int j = 0; j < BS_ILP; j++) {
            const int64_t t = base + j * 32 + lane;
            if (t < nitems) load8(x + t * 8, f[j]);
            else {
#pragma unroll
                for (int e = 0; e < 8; e++) f[j][e] = 0.0f;
            }
        }
#pragma unroll
        for (int j = 0; j < BS_ILP; j++) {
            const int64_t t = base + j * 32 + lane;
            float am = 0.0f;
#pragma unroll
            for (int e = 0; e < 8; e++) am = fmaxf(am, fabsf(f[j][e]));
            am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 1));
            am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 2));
            if (t >= nitems) continue;
            int byte = 0;
            if (am > 0.0f) {
                const uint32_t b = __float_as_uint(am);
                const int e = (b >> 23) != 0 ? (int)(b >> 23) - 127 : -118 - __clz(b);   // floor(log2(am))
                byte = e - 8 + 127;
                byte = byte < 0 ? 0 : (byte > 254 ? 254 : byte);
            }
            const float inv = pow2_of(127 - byte);
            uint32_t lo = (uint32_t)cvt_e4m3x2(f[j][0] * inv, f[j][1] * inv) | ((uint32_t)cvt_e4m3x2(f[j][2] * inv, f[j][3] * inv) << 16);
            uint32_t hi = (uint32_t)cvt_e4m3x2(f[j][4] * inv, f[j][5] * inv) | ((uint32_t)cvt_e4m3x2(f[j][6] * inv, f[j][7] * inv) << 16);
            __stcs(reinterpret_cast<uint2*>(codes + t * 8), make_uint2(lo, hi));
            if ((t & 3) == 0) {
                const uint32_t blk = (uint32_t)(t >> 2);                     // host guarantees < 2^31 blocks
                const uint32_t r = blk / (uint32_t)sf_cols, c = blk - r * (uint32_t)sf_cols;
                if (sf_rm) sf_rm[blk] = (uint8_t)byte;
                if (sf_mma) sf_mma[sf_mma_offset32(r, c, sf_col_tiles)] = (uint8_t)byte;
            }
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(256) mxfp8_dequant_kernel(const uint8_t* __restrict__ codes, const uint8_t* __restrict__ sf_rm,
                                                            int64_t n, T* __restrict__ y) {
    pdl_trigger();
    pdl_wait();
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        y[i] = Elem<T>::from_f32(e4m3_to_f32(codes[i]) * pow2_of((int)sf_rm[i >> 5] - 127));
}

// eight f32 -> eight E2M1 nibbles in one word (RNE, satfinite), element e at bits [4e, 4e+4)
__device__ __forceinline__ uint32_t cvt_e2m1x8(const float (&q)[8]) {
    uint32_t w;
    asm("{ .reg .b8 t0, t1, t2, t3;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 t0, %2, %1;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 t1, %4, %3;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 t2, %6, %5;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 t3, %8, %7;\n\t"
        "mov.b32 %0, {t0, t1, t2, t3}; }"
        : "=r"(w) : "f"(q[0]), "f"(q[1]), "f"(q[2]), "f"(q[3]), "f"(q[4]), "f"(q[5]), "f"(q[6]), "f"(q[7]));
    return w;
}

// 8 elements per item, 2 adjacent lanes form one 16-element block; BS_ILP items per thread in flight.
// A block's divisor g * ue4m3(s8) takes one of 127 values per launch: its reciprocal comes from a table in shared
// memory instead of a reciprocal sequence per block, and the block's (row, column) for the tiled scale layout is
// carried along instead of divided out.
template <typename T>
__global__ void __launch_bounds__(256) nvfp4_quant_kernel(const T* __restrict__ x, int64_t rows, int64_t k, float* __restrict__ stats,
                                                          uint8_t* __restrict__ packed, uint8_t* __restrict__ sf_rm,
                                                          uint8_t* __restrict__ sf_mma) {
    pdl_trigger();
    pdl_wait();
    __shared__ float2 lut[128];                               // (divisor, its reciprocal; NaN = divide the slow way)
    const float tmax = stats[0];
    const float g = tmax > 0.0f ? __fdiv_rn(tmax, 448.0f * 6.0f) : 1.0f;
    if (blockIdx.x == 0 && threadIdx.x == 0) stats[1] = g;
    if (threadIdx.x < 128) {
        const InvDiv d = make_invdiv(g * e4m3_to_f32((uint8_t)threadIdx.x));
        lut[threadIdx.x] = make_float2(d.s, d.fast ? d.y : __int_as_float(0x7FC00000));
    }
    __syncthreads();
    const InvDiv six_g = make_invdiv(6.0f * g);
    const int64_t nitems = rows * k / 8;
    const uint32_t sf_cols = (uint32_t)(k / 16);
    const uint32_t sf_col_tiles = (sf_cols + 3) / 4;
    const int lane = threadIdx.x & 31;
    const int64_t warp_global = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t base = warp_global * (32 * BS_ILP); base < nitems; base += nwarps * (32 * BS_ILP)) {
        float f[BS_ILP][8];
#pragma unroll
        for (int j = 0; j < BS_ILP; j++) {
            const int64_t t = base + j * 32 + lane;
            if (t < nitems) load8(x + t * 8, f[j]);
            else {
#pragma unroll
                for (int e = 0; e < 8; e++) f[j][e] = 0.0f;
            }
        }
        // (row, column) of this lane's first block; the next items are 16 blocks further each
        uint32_t blk = (uint32_t)((base + lane) >> 1);                       // host guarantees < 2^31 blocks
        uint32_t r = blk / sf_cols, c = blk - r * sf_cols;
#pragma unroll
        for (int j = 0; j < BS_ILP; j++) {
            const int64_t t = base + j * 32 + lane;
            float am = 0.0f;
#pragma unroll
            for (int e = 0; e < 8; e++) am = fmaxf(am, fabsf(f[j][e]));
            am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 1));
            if (t < nitems) {
                const uint32_t s8 = cvt_e4m3x2(div_exact_bounded(am, six_g), 0.0f) & 0xFFu;       // am <= tensor max: quotient <= 448
                uint32_t w = 0;
                if (s8 == 0) {
#pragma unroll
                    for (int e = 0; e < 8; e++) w |= ((__float_as_uint(f[j][e]) >> 28) & 8u) << (4 * e);
                } else {
                    const float2 le = lut[s8 & 127u];
                    InvDiv d;
                    d.s = le.x; d.y = le.y; d.fast = le.y == le.y;
                    float q[8];
#pragma unroll
                    for (int e = 0; e < 8; e++) q[e] = div_exact_bounded_signed(f[j][e], d);      // |x| <= block max: no overflow
                    w = cvt_e2m1x8(q);
                }
                __stcs(reinterpret_cast<uint32_t*>(packed + t * 4), w);
                if ((t & 1) == 0) {
                    if (sf_rm) sf_rm[blk] = (uint8_t)s8;
                    if (sf_mma) sf_mma[sf_mma_offset32(r, c, sf_col_tiles)] = (uint8_t)s8;
                }
            }
            blk += 16; c += 16;
            while (c >= sf_cols) { c -= sf_cols; r++; }
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(256) nvfp4_dequant_kernel(const uint8_t* __restrict__ packed, const uint8_t* __restrict__ sf_rm,
                                                            const float* __restrict__ stats, int64_t n, T* __restrict__ y) {
    pdl_trigger();
    pdl_wait();
    const float g = stats[1];
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const uint32_t nib = (packed[i >> 1] >> ((i & 1) * 4)) & 0xF;
        y[i] = Elem<T>::from_f32(e2m1_to_f32(nib) * e4m3_to_f32(sf_rm[i >> 4]) * g);
    }
}

// h[m, j] = silu(gu[m, blk*256 + j%128]) * gu[m, blk*256 + 128 + j%128], blk = j / 128: the SwiGLU of
// SwiGluFfn::forward on a gate/up product stored in the interleaved 128-column block order.
__global__ void __launch_bounds__(256) swiglu_interleaved_kernel(const __nv_bfloat16* __restrict__ gu, int64_t m, int64_t n,
                                                                 __nv_bfloat16* __restrict__ out) {
    pdl_trigger();
    pdl_wait();
    const int64_t nvec = m * n / 8;
    for (int64_t v = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; v < nvec; v += (int64_t)gridDim.x * blockDim.x) {
        const int64_t e = v * 8, row = e / n, j = e - row * n;
        const __nv_bfloat16* g = gu + row * 2 * n + (j >> 7) * 256 + (j & 127);
        Vec16<__nv_bfloat16> a = ld16(g), b = ld16(g + 128), o;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const float gt = __bfloat162float(a.v[i]);
            o.v[i] = __float2bfloat16_rn(__fdividef(gt, 1.0f + __expf(-gt)) * __bfloat162float(b.v[i]));
        }
        *reinterpret_cast<uint4*>(out + e) = *reinterpret_cast<uint4*>(&o);
    }
}

static inline int grid_for(oxq_handle* h, int64_t work_items, int block, int ctas_per_sm) {
    int64_t need = (work_items + block - 1) / block;
    int64_t cap = (int64_t)h->sm_count * ctas_per_sm;
    if (need < 1) need = 1;
    return (int)(need < cap ? need : cap);
}

}  // namespace oxq

using namespace oxq;

#define DISPATCH_DTYPE(dtype, ...)                                           \
    switch (dtype) {                                                         \
        case OXQ_F32: { using T = float; __VA_ARGS__; break; }               \
        case OXQ_BF16: { using T = __nv_bfloat16; __VA_ARGS__; break; }      \
        case OXQ_F16: { using T = __half; __VA_ARGS__; break; }              \
        default: OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "unknown dtype %d", dtype); \
    }

static inline bool aligned16(const void* p) { return ((uintptr_t)p & 15u) == 0; }
static inline size_t dtype_size(int dt) { return dt == OXQ_F32 ? 4 : 2; }

extern "C" {

int32_t oxq_int8_quant_rows(oxq_handle* h, const float* x, int64_t rows, int64_t cols, int8_t* q, float* scales, int rounding) {
    OXQ_CHECK_HANDLE(h);
    if (rows <= 0) OXQ_FAIL(h, OXQ_ERR_EMPTY_INPUT, "calibrate_2d: rows == 0");
    if (cols <= 0) OXQ_FAIL(h, OXQ_ERR_QUANT_DIMENSION_MISMATCH, "dimension mismatch: expected 1, got 0");
    if (!x || !q || !scales) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null pointer");
    if (rounding != OXQ_ROUND_HALF_EVEN && rounding != OXQ_ROUND_HALF_AWAY) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "rounding %d", rounding);
    if (int32_t rc = oxq_require_sm100(h)) return rc;
    const int grid = (int)(rows < (int64_t)h->sm_count * 6 ? rows : (int64_t)h->sm_count * 6);
    if ((cols & 3) == 0 && aligned16(x) && (((uintptr_t)q & 3u) == 0)) {
        const bool away = rounding == OXQ_ROUND_HALF_AWAY;
        if (cols <= 4096) {
            if (away) oxq_launch(int8_quant_rows_kernel<4, OXQ_ROUND_HALF_AWAY>, grid, 256, 0, h->stream, x, rows, cols, q, scales);
            else oxq_launch(int8_quant_rows_kernel<4, OXQ_ROUND_HALF_EVEN>, grid, 256, 0, h->stream, x, rows, cols, q, scales);
        } else {
            if (away) oxq_launch(int8_quant_rows_kernel<8, OXQ_ROUND_HALF_AWAY>, grid, 256, 0, h->stream, x, rows, cols, q, scales);
            else oxq_launch(int8_quant_rows_kernel<8, OXQ_ROUND_HALF_EVEN>, grid, 256, 0, h->stream, x, rows, cols, q, scales);
        }
    } else {
        oxq_launch(int8_quant_rows_scalar_kernel, grid, 256, 0, h->stream, x, rows, cols, q, scales, rounding);
    }
    OXQ_LAUNCH_CHECK(h);
    return OXQ_OK;
}

int32_t oxq_int8_dequant_rows(oxq_handle* h, const int8_t* q, const float* scales, int64_t rows, int64_t cols, float* y) {
    OXQ_CHECK_HANDLE(h);
    if (rows <= 0 || cols <= 0) OXQ_FAIL(h, OXQ_ERR_EMPTY_INPUT, "dequantize: empty input");
    if (!y || !q || !scales) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null pointer");
    if (int32_t rc = oxq_require_sm100(h)) return rc;
    if ((cols & 15) == 0 && aligned16(q) && aligned16(y))
        oxq_launch(int8_dequant_rows_kernel, grid_for(h, rows * cols / 16, 256, 16), 256, 0, h->stream, q, scales, rows, cols, y);
    else
        oxq_launch(int8_dequant_rows_scalar_kernel, grid_for(h, rows * cols, 256, 16), 256, 0, h->stream, q, scales, rows, cols, y);
    OXQ_LAUNCH_CHECK(h);
    return OXQ_OK;
}

int32_t oxq_absmax(oxq_handle* h, const void* x, int dtype, int64_t n, float* absmax_dev) {
    OXQ_CHECK_HANDLE(h);
    if (n <= 0) OXQ_FAIL(h, OXQ_ERR_EMPTY_INPUT, "absmax: empty input");
    if (!x || !absmax_dev || !aligned16(x)) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null or misaligned pointer");
    if (int32_t rc = oxq_require_sm100(h)) return rc;
    if (!h->dev_scratch) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "handle has no reduction cells");
    DISPATCH_DTYPE(dtype, oxq_launch(absmax_kernel<T>, grid_for(h, n / Vec16<T>::N / 8 + 1, 256, 8), 256, 0, h->stream, (const T*)x, n, absmax_dev, h->dev_scratch));
    OXQ_LAUNCH_CHECK(h);
    return OXQ_OK;
}

static int32_t fp8_quant_launch(oxq_handle* h, const void* x, int dtype, int64_t n, const float* scale, float* stats, uint8_t* q, int mode) {
    const int grid = grid_for(h, n / (8 * FP8_ILP) + 1, 256, 8);
    if (mode == OXQ_FP8_SPEC_RNE && stats) {
        // scale = absmax / 448 of this very tensor: quotients are bounded by 448, no overflow handling needed
        DISPATCH_DTYPE(dtype, oxq_launch(fp8_quant_kernel<T, OXQ_FP8_SPEC_RNE, true>, grid, 256, 0, h->stream, (const T*)x, n, scale, stats, q));
    } else if (mode == OXQ_FP8_SPEC_RNE) {
        DISPATCH_DTYPE(dtype, oxq_launch(fp8_quant_kernel<T, OXQ_FP8_SPEC_RNE, false>, grid, 256, 0, h->stream, (const T*)x, n, scale, stats, q));
    } else if (mode == OXQ_FP8_REFCOMPAT) {
        DISPATCH_DTYPE(dtype, oxq_launch(fp8_quant_kernel<T, OXQ_FP8_REFCOMPAT, false>, grid, 256, 0, h->stream, (const T*)x, n, scale, stats, q));
    } else {
        OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "fp8 mode %d", mode);
    }
    OXQ_LAUNCH_CHECK(h);
    return OXQ_OK;
}

int32_t oxq_fp8_quant(oxq_handle* h, const void* x, int dtype, int64_t n, const float* scale_dev, uint8_t* q, int mode) {
    OXQ_CHECK_HANDLE(h);
    if (n <= 0) OXQ_FAIL(h, OXQ_ERR_EMPTY_INPUT, "fp8 encode: empty input");
    if (!x || !q || !scale_dev || !aligned16(x) || !aligned16(q)) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null or misaligned pointer");
    if (int32_t rc = oxq_require_sm100(h)) return rc;
    return fp8_quant_launch(h, x, dtype, n, scale_dev, nullptr, q, mode);
}

int32_t oxq_fp8_quant_dynamic(oxq_handle* h, const void* x, int dtype, int64_t n, uint8_t* q, float* stats_dev) {
    OXQ_CHECK_HANDLE(h);
    if (n <= 0) OXQ_FAIL(h, OXQ_ERR_EMPTY_INPUT, "fp8 encode: empty input");
    if (!x || !q || !stats_dev || !aligned16(x) || !aligned16(q)) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null or misaligned pointer");
    if (n <= FP8_SMALL_MAX && (dtype == OXQ_F32 || dtype == OXQ_BF16 || dtype == OXQ_F16)) {       // one CTA, one launch
        if (int32_t rc = oxq_require_sm100(h)) return rc;
        DISPATCH_DTYPE(dtype, oxq_launch(fp8_quant_dynamic_small_kernel<T>, 1, 1024, 0, h->stream, (const T*)x, n, stats_dev, q));
        OXQ_LAUNCH_CHECK(h);
        return OXQ_OK;
    }
    // one launch with a grid-wide meeting point between the two passes (OXQ_FP8_FUSED_DYNAMIC=0: two launches)
    static int fused = -1;
    if (fused < 0) { const char* e = getenv("OXQ_FP8_FUSED_DYNAMIC"); fused = e ? (atoi(e) != 0) : 1; }
    // it pays from tensors of about half the L2 on (8192 x 8192 bf16: 66.4 -> 61.8 us); below that the second launch
    // finds the whole tensor in L2 anyway and the two-launch form is as fast
    const int64_t bytes = n * (dtype == OXQ_F32 ? 4 : 2);
    if (fused && bytes >= (int64_t)48 << 20 && h->dev_scratch && (dtype == OXQ_F32 || dtype == OXQ_BF16 || dtype == OXQ_F16)) {
        if (int32_t rc = oxq_require_sm100(h)) return rc;
        static OxqPerDevice occ_cache[3];
        const int di = dtype == OXQ_F32 ? 0 : (dtype == OXQ_BF16 ? 1 : 2);
        int occ[3] = {0, 0, 0};
        occ[di] = occ_cache[di].get(h->device);
        if (occ[di] == 0) {
            int o = 0;
            cudaError_t e = cudaSuccess;
            if (di == 0) e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&o, fp8_quant_dynamic_fused_kernel<float>, 256, 0);
            else if (di == 1) e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&o, fp8_quant_dynamic_fused_kernel<__nv_bfloat16>, 256, 0);
            else e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&o, fp8_quant_dynamic_fused_kernel<__half>, 256, 0);
            occ[di] = (e == cudaSuccess && o > 0) ? o : -1;
            occ_cache[di].set(h->device, occ[di]);
        }
        if (occ[di] > 0) {
            const int per_sm = occ[di] < 6 ? occ[di] : 6;
            const int grid = grid_for(h, n / (8 * FP8_ILP) + 1, 256, per_sm);          // never more CTAs than fit at once
            unsigned int* cells = h->dev_scratch + 8;                                   // cells 8-11; 0-1 and 4 have other owners
            // Cooperative: other streams of the process may occupy part of the GPU, and a grid that is only partly resident
            // would wait at the meeting point for CTAs that cannot start.  If the driver cannot place the whole grid the
            // launch fails here and the two-launch form below runs instead.
            cudaError_t le = cudaSuccess;
            DISPATCH_DTYPE(dtype, le = oxq_launch_cooperative(fp8_quant_dynamic_fused_kernel<T>, grid, 256, 0, h->stream, (const T*)x, n, stats_dev, q, cells, h->dev_status));
            if (le == cudaSuccess) return OXQ_OK;
            (void)cudaGetLastError();                                                   // clear the refused launch, fall through
        }
    }
    if (int32_t rc = oxq_absmax(h, x, dtype, n, stats_dev)) return rc;
    return fp8_quant_launch(h, x, dtype, n, nullptr, stats_dev, q, OXQ_FP8_SPEC_RNE);
}

int32_t oxq_fp8_dequant(oxq_handle* h, const uint8_t* q, int64_t n, const float* scale_dev, void* y, int y_dtype, int mode) {
    OXQ_CHECK_HANDLE(h);
    if (n <= 0) OXQ_FAIL(h, OXQ_ERR_EMPTY_INPUT, "fp8 decode: empty input");
    if (!y || !q || !scale_dev) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null pointer");
    if (int32_t rc = oxq_require_sm100(h)) return rc;
    const int grid = grid_for(h, n, 256, 16);
    if (mode == OXQ_FP8_SPEC_RNE) {
        DISPATCH_DTYPE(y_dtype, oxq_launch(fp8_dequant_kernel<T, OXQ_FP8_SPEC_RNE>, grid, 256, 0, h->stream, q, n, scale_dev, (T*)y));
    } else {
        DISPATCH_DTYPE(y_dtype, oxq_launch(fp8_dequant_kernel<T, OXQ_FP8_REFCOMPAT>, grid, 256, 0, h->stream, q, n, scale_dev, (T*)y));
    }
    OXQ_LAUNCH_CHECK(h);
    return OXQ_OK;
}

int32_t oxq_int4g_quant_pack(oxq_handle* h, const void* x, int dtype, int64_t rows, int64_t k, int group, uint32_t* codes,
                             uint16_t* scales, uint32_t* zeros, int rounding) {
    OXQ_CHECK_HANDLE(h);
    if (rows <= 0 || k <= 0) OXQ_FAIL(h, OXQ_ERR_EMPTY_INPUT, "MinMaxQuantizer::calibrate");
    if (!(group == 32 || group == 64 || group == 128 || group == 256))   // Int4GemmConfig::VALID_GROUP_SIZES
        OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "group size %d not in {32,64,128,256}", group);
    if (k % group != 0) OXQ_FAIL(h, OXQ_ERR_GROUP_SIZE_MISMATCH, "tensor length %lld is not divisible by group size %d", (long long)k, group);
    if (!x || !codes || !scales || !zeros || !aligned16(x)) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null or misaligned pointer");
    if (int32_t rc = oxq_require_sm100(h)) return rc;
    const int64_t ngroups = rows * (k / group);
    const int grid = grid_for(h, (ngroups + 7) / 8 * 32, 256, 8);
#define LAUNCH_G(G) oxq_launch(int4g_quant_kernel<T, G>, grid, 256, 0, h->stream, (const T*)x, ngroups, rounding, codes, scales, zeros)
    DISPATCH_DTYPE(dtype, if (group == 32) LAUNCH_G(32); else if (group == 64) LAUNCH_G(64);
                   else if (group == 128) oxq_launch(int4g128_quant_kernel<T>, grid, 256, 0, h->stream, (const T*)x, ngroups, rounding, codes, scales, zeros);
                   else LAUNCH_G(256));
#undef LAUNCH_G
    OXQ_LAUNCH_CHECK(h);
    return OXQ_OK;
}

int32_t oxq_int4g_dequant(oxq_handle* h, const uint32_t* codes, const uint16_t* scales, const uint32_t* zeros, int64_t rows, int64_t k,
                          int group, void* y, int y_dtype) {
    OXQ_CHECK_HANDLE(h);
    if (rows <= 0 || k <= 0) OXQ_FAIL(h, OXQ_ERR_EMPTY_INPUT, "dequantize: empty input");
    if (group <= 0 || k % group != 0 || group % 8 != 0) OXQ_FAIL(h, OXQ_ERR_GROUP_SIZE_MISMATCH, "k %lld vs group %d", (long long)k, group);
    if (!y || !codes || !scales || !zeros || !aligned16(y)) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null or misaligned pointer");
    if (int32_t rc = oxq_require_sm100(h)) return rc;
    const int64_t nwords = rows * k / 8;
    DISPATCH_DTYPE(y_dtype, oxq_launch(int4g_dequant_kernel<T>, grid_for(h, nwords, 256, 16), 256, 0, h->stream, codes, scales, zeros, nwords, group, (T*)y));
    OXQ_LAUNCH_CHECK(h);
    return OXQ_OK;
}

int32_t oxq_swiglu_interleaved(oxq_handle* h, const void* gu, int64_t m, int64_t n, void* out) {
    OXQ_CHECK_HANDLE(h);
    if (m <= 0 || n <= 0) OXQ_FAIL(h, OXQ_ERR_EMPTY_INPUT, "swiglu: empty input");
    if (n % 128 != 0) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "n must be a multiple of 128, got %lld", (long long)n);
    if (!gu || !out || !aligned16(gu) || !aligned16(out)) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null or misaligned pointer");
    if (int32_t rc = oxq_require_sm100(h)) return rc;
    oxq_launch(swiglu_interleaved_kernel, grid_for(h, m * n / 8, 256, 8), 256, 0, h->stream, (const __nv_bfloat16*)gu, m, n, (__nv_bfloat16*)out);
    OXQ_LAUNCH_CHECK(h);
    return OXQ_OK;
}

size_t oxq_sf_mma_bytes(int64_t rows, int64_t sf_cols) {
    if (rows <= 0 || sf_cols <= 0) return 0;
    return (size_t)((rows + 127) / 128) * (size_t)((sf_cols + 3) / 4) * 512;
}

int32_t oxq_mxfp8_quant(oxq_handle* h, const void* x, int dtype, int64_t rows, int64_t k, uint8_t* codes, uint8_t* sf_rm, uint8_t* sf_mma) {
    OXQ_CHECK_HANDLE(h);
    if (rows <= 0 || k <= 0) OXQ_FAIL(h, OXQ_ERR_EMPTY_INPUT, "mxfp8 quantize: empty input");
    if (k % 32 != 0) OXQ_FAIL(h, OXQ_ERR_GROUP_SIZE_MISMATCH, "k %lld is not divisible by block size 32", (long long)k);
    if (!x || !codes || (!sf_rm && !sf_mma) || !aligned16(x)) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null or misaligned pointer");
    if (rows * (k / 32) >= ((int64_t)1 << 31)) OXQ_FAIL(h, OXQ_ERR_INVALID_DIMENSION, "more than 2^31 scale blocks");
    if (int32_t rc = oxq_require_sm100(h)) return rc;
    if (sf_mma && ((rows & 127) || ((k / 32) & 3)))          // pad bytes of partial tiles must not hold garbage
        OXQ_CUDA(h, cudaMemsetAsync(sf_mma, 0, oxq_sf_mma_bytes(rows, k / 32), h->stream));
    DISPATCH_DTYPE(dtype, oxq_launch(mxfp8_quant_kernel<T>, grid_for(h, rows * k / (8 * BS_ILP) + 1, 256, 8), 256, 0, h->stream, (const T*)x, rows, k, codes, sf_rm, sf_mma));
    OXQ_LAUNCH_CHECK(h);
    return OXQ_OK;
}

int32_t oxq_mxfp8_dequant(oxq_handle* h, const uint8_t* codes, const uint8_t* sf_rm, int64_t rows, int64_t k, void* y, int y_dtype) {
    OXQ_CHECK_HANDLE(h);
    if (rows <= 0 || k <= 0) OXQ_FAIL(h, OXQ_ERR_EMPTY_INPUT, "mxfp8 dequantize: empty input");
    if (k % 32 != 0) OXQ_FAIL(h, OXQ_ERR_GROUP_SIZE_MISMATCH, "k %lld is not divisible by block size 32", (long long)k);
    if (!y || !codes || !sf_rm) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null pointer");
    if (int32_t rc = oxq_require_sm100(h)) return rc;
    DISPATCH_DTYPE(y_dtype, oxq_launch(mxfp8_dequant_kernel<T>, grid_for(h, rows * k, 256, 16), 256, 0, h->stream, codes, sf_rm, rows * k, (T*)y));
    OXQ_LAUNCH_CHECK(h);
    return OXQ_OK;
}

int32_t oxq_nvfp4_quant(oxq_handle* h, const void* x, int dtype, int64_t rows, int64_t k, float* stats, uint8_t* packed, uint8_t* sf_rm,
                        uint8_t* sf_mma) {
    OXQ_CHECK_HANDLE(h);
    if (rows <= 0 || k <= 0) OXQ_FAIL(h, OXQ_ERR_EMPTY_INPUT, "nvfp4 quantize: empty input");
    if (k % 16 != 0) OXQ_FAIL(h, OXQ_ERR_GROUP_SIZE_MISMATCH, "k %lld is not divisible by block size 16", (long long)k);
    if (!x || !packed || !stats || (!sf_rm && !sf_mma) || !aligned16(x)) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null or misaligned pointer");
    if (rows * (k / 16) >= ((int64_t)1 << 31)) OXQ_FAIL(h, OXQ_ERR_INVALID_DIMENSION, "more than 2^31 scale blocks");
    if (int32_t rc = oxq_require_sm100(h)) return rc;
    if (sf_mma && ((rows & 127) || ((k / 16) & 3)))
        OXQ_CUDA(h, cudaMemsetAsync(sf_mma, 0, oxq_sf_mma_bytes(rows, k / 16), h->stream));
    DISPATCH_DTYPE(dtype, oxq_launch(nvfp4_quant_kernel<T>, grid_for(h, rows * k / (8 * BS_ILP) + 1, 256, 8), 256, 0, h->stream, (const T*)x, rows, k, stats, packed, sf_rm, sf_mma));
    OXQ_LAUNCH_CHECK(h);
    return OXQ_OK;
}

int32_t oxq_nvfp4_dequant(oxq_handle* h, const uint8_t* packed, const uint8_t* sf_rm, const float* stats, int64_t rows, int64_t k, void* y,
                          int y_dtype) {
    OXQ_CHECK_HANDLE(h);
    if (rows <= 0 || k <= 0) OXQ_FAIL(h, OXQ_ERR_EMPTY_INPUT, "nvfp4 dequantize: empty input");
    if (k % 16 != 0) OXQ_FAIL(h, OXQ_ERR_GROUP_SIZE_MISMATCH, "k %lld is not divisible by block size 16", (long long)k);
    if (!y || !packed || !sf_rm || !stats) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null pointer");
    if (int32_t rc = oxq_require_sm100(h)) return rc;
    DISPATCH_DTYPE(y_dtype, oxq_launch(nvfp4_dequant_kernel<T>, grid_for(h, rows * k, 256, 16), 256, 0, h->stream, packed, sf_rm, stats, rows * k, (T*)y));
    OXQ_LAUNCH_CHECK(h);
    return OXQ_OK;
}

}  // extern "C"
