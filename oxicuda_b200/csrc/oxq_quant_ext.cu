// Quantizers next to the hot path: the per-tensor INT8 form of the DNN crate's device API, its per-block INT8
// container, and NF4.  All are memory-bound streaming kernels with the same conventions as oxq_quant.cu:
// caller-owned device buffers, stream-ordered, 128-bit accesses where the layout allows, IEEE divisions.
#include "oxq_common.cuh"

namespace oxq {

// ------------------------------------------------------------------------------------------------
// INT8, one scale for the whole tensor
// ------------------------------------------------------------------------------------------------

template <typename T>
__device__ __forceinline__ void load8f(const T* p, float (&f)[8]);
template <>
__device__ __forceinline__ void load8f<float>(const float* p, float (&f)[8]) {
    const float4 a = __ldcs(reinterpret_cast<const float4*>(p)), b = __ldcs(reinterpret_cast<const float4*>(p) + 1);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
template <>
__device__ __forceinline__ void load8f<__nv_bfloat16>(const __nv_bfloat16* p, float (&f)[8]) {
    const uint4 u = __ldcs(reinterpret_cast<const uint4*>(p));
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; i++) { f[2 * i] = __uint_as_float(w[i] << 16); f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u); }
}
template <>
__device__ __forceinline__ void load8f<__half>(const __half* p, float (&f)[8]) {
    const uint4 u = __ldcs(reinterpret_cast<const uint4*>(p));
    const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; i++) { const float2 v = __half22float2(h[i]); f[2 * i] = v.x; f[2 * i + 1] = v.y; }
}

// the same eight elements as raw 16-byte words (requested early, converted when needed)
template <typename T> struct Raw8 { uint4 a; };
template <> struct Raw8<float> { uint4 a, b; };
template <typename T>
__device__ __forceinline__ Raw8<T> load8raw(const T* p) {
    Raw8<T> r;
    r.a = __ldcs(reinterpret_cast<const uint4*>(p));
    if constexpr (sizeof(T) == 4) r.b = __ldcs(reinterpret_cast<const uint4*>(p) + 1);
    return r;
}
__device__ __forceinline__ void raw8_to_f32(const Raw8<float>& r, float (&f)[8]) {
    f[0] = __uint_as_float(r.a.x); f[1] = __uint_as_float(r.a.y); f[2] = __uint_as_float(r.a.z); f[3] = __uint_as_float(r.a.w);
    f[4] = __uint_as_float(r.b.x); f[5] = __uint_as_float(r.b.y); f[6] = __uint_as_float(r.b.z); f[7] = __uint_as_float(r.b.w);
}
__device__ __forceinline__ void raw8_to_f32(const Raw8<__nv_bfloat16>& r, float (&f)[8]) {
    const uint32_t w[4] = {r.a.x, r.a.y, r.a.z, r.a.w};
#pragma unroll
    for (int i = 0; i < 4; i++) { f[2 * i] = __uint_as_float(w[i] << 16); f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u); }
}
__device__ __forceinline__ void raw8_to_f32(const Raw8<__half>& r, float (&f)[8]) {
    const __half2* h = reinterpret_cast<const __half2*>(&r.a);
#pragma unroll
    for (int i = 0; i < 4; i++) { const float2 v = __half22float2(h[i]); f[2 * i] = v.x; f[2 * i + 1] = v.y; }
}

// clamp(x / scale, -127, 127) rounded half to even, left in the low byte of the returned float's bit pattern.  The
// scale comes from the tensor's own maximum, so finite inputs give quotients within +-127 (+ rounding) and only
// the lower clamp is kept: it sends a NaN to -127, as the max.f32 of the reference's kernel does.  An Inf in the
// tensor makes the scale Inf, which takes the true-division path.
__device__ __forceinline__ uint32_t quant_i8_rne_bits(float x, const InvDiv& d) {
    const float v = fminf(fmaxf(div_exact_bounded(x, d), -127.0f), 127.0f);
    return __float_as_uint(v + 12582912.0f);                // RNE(v) in the low mantissa byte of v + 1.5 * 2^23
}
__device__ __forceinline__ uint32_t quant_i8_rne(float x, const InvDiv& d) { return quant_i8_rne_bits(x, d) & 0xFFu; }
// low bytes of four words -> one word
__device__ __forceinline__ uint32_t pack_low_bytes(uint32_t a, uint32_t b, uint32_t c, uint32_t e) {
    return __byte_perm(__byte_perm(a, b, 0x0040), __byte_perm(c, e, 0x0040), 0x5410);
}

constexpr int I8T_ILP = 4;                                  // items of 8 elements in flight per thread

// scale[0] = max(absmax / 127, 1e-12); q = rint(clamp(x / scale, -127, 127)).  The maximum was left in
// `absmax` (a cell of the handle) by the reduction kernel that ran just before on the same stream.
template <typename T>
__global__ void __launch_bounds__(256) int8_tensor_quant_kernel(const T* __restrict__ x, int64_t n, const float* __restrict__ absmax,
                                                                int8_t* __restrict__ q, float* __restrict__ scale_out) {
    pdl_trigger();
    pdl_wait();
    const float sc = fmaxf(__fdiv_rn(*absmax, 127.0f), 1e-12f);
    if (blockIdx.x == 0 && threadIdx.x == 0) *scale_out = sc;
    const InvDiv d = make_invdiv(sc);
    const int64_t nitems = n >> 3;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t t0 = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t0 < nitems; t0 += stride * I8T_ILP) {
        float f[I8T_ILP][8];
#pragma unroll
        for (int j = 0; j < I8T_ILP; j++)
            if (t0 + j * stride < nitems) load8f(x + (t0 + j * stride) * 8, f[j]);
#pragma unroll
        for (int j = 0; j < I8T_ILP; j++) {
            const int64_t t = t0 + j * stride;
            if (t < nitems) {
                uint2 o;
                o.x = pack_low_bytes(quant_i8_rne_bits(f[j][0], d), quant_i8_rne_bits(f[j][1], d), quant_i8_rne_bits(f[j][2], d), quant_i8_rne_bits(f[j][3], d));
                o.y = pack_low_bytes(quant_i8_rne_bits(f[j][4], d), quant_i8_rne_bits(f[j][5], d), quant_i8_rne_bits(f[j][6], d), quant_i8_rne_bits(f[j][7], d));
                __stcs(reinterpret_cast<uint2*>(q + t * 8), o);
            }
        }
    }
    // ragged tail (n not a multiple of 8)
    if (blockIdx.x == 0) {
        for (int64_t i = (nitems << 3) + threadIdx.x; i < n; i += blockDim.x) q[i] = (int8_t)quant_i8_rne(Elem<T>::to_f32(x[i]), d);
    }
}

template <typename T>
__global__ void __launch_bounds__(256) int8_tensor_dequant_kernel(const int8_t* __restrict__ q, int64_t n, const float* __restrict__ scale,
                                                                  T* __restrict__ y) {
    pdl_trigger();
    pdl_wait();
    const float sc = *scale;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        y[i] = Elem<T>::from_f32((float)q[i] * sc);
}

// ------------------------------------------------------------------------------------------------
// INT8, one scale per block of contiguous elements (the last block may be short)
// ------------------------------------------------------------------------------------------------

// A warp per block: maximum, then q = clamp(round_half_away(x / scale), -128, 127).  The second pass finds the
// block in L1 / L2.
__global__ void __launch_bounds__(256) int8_block_quant_kernel(const float* __restrict__ x, int64_t n, int64_t block, int64_t nblocks,
                                                               int8_t* __restrict__ q, float* __restrict__ scales) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5, nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t b = warp0; b < nblocks; b += nwarps) {
        const int64_t b0 = b * block;
        const int64_t len = n - b0 < block ? n - b0 : block;
        float am = 0.0f;
        for (int64_t i = lane; i < len; i += 32) am = fmaxf(am, fabsf(x[b0 + i]));
        am = warp_max(am);
        const float sc = am > 0.0f ? __fdiv_rn(am, 127.0f) : 1.0f;
        if (lane == 0) scales[b] = sc;
        for (int64_t i = lane; i < len; i += 32) {
            float v = roundf(__fdiv_rn(x[b0 + i], sc));
            v = v != v ? 0.0f : fminf(fmaxf(v, -128.0f), 127.0f);          // NaN -> 0 (Rust `as i8`)
            q[b0 + i] = (int8_t)(int)v;
        }
    }
}

__global__ void __launch_bounds__(256) int8_block_dequant_kernel(const int8_t* __restrict__ q, const float* __restrict__ scales, int64_t n,
                                                                 int64_t block, float* __restrict__ y) {
    pdl_trigger();
    pdl_wait();
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        y[i] = (float)q[i] * __ldg(scales + i / block);
}

// ------------------------------------------------------------------------------------------------
// NF4
// ------------------------------------------------------------------------------------------------

__constant__ float c_nf4[16] = {-1.0f, -0.69619286f, -0.52507305f, -0.3949175f, -0.28444138f, -0.18477343f, -0.09105003f, 0.0f,
                                0.0795803f, 0.1609302f, 0.2461123f, 0.33791524f, 0.44070983f, 0.562617f, 0.72295684f, 1.0f};

// Index of the level nearest to v in [-1, 1]; between two levels the lower index wins a tie (nf4.rs:186-205: first
// index whose level is >= v, then |v - level[lo-1]| <= |level[lo] - v| in f32).  Both distances are monotone in v, so
// for every pair of neighbours there is one f32 value up to which the lower level wins: kNf4Thr[i] is the largest
// f32 whose nearest level is i under exactly that f32 comparison (found by bisection over bit patterns against the
// reference's function; they sit within an ulp or two of the arithmetic midpoints).  The code is then the number of
// thresholds below v: four comparisons against constants picked by the earlier outcomes, no table and no memory.
// NaN compares false everywhere and gives 0, as in the reference.
#define NF4_THR_BITS {0xBF591CD9u, 0xBF1C5271u, 0xBEEB8480u, 0xBEADEA77u, 0xBE703CEDu, 0xBE0D38BCu, 0xBD3A7870u, 0x3D22FAFFu, \
                      0x3DF64862u, 0x3E5067E0u, 0x3E9582D4u, 0x3EC753F9u, 0x3F006D03u, 0x3F248DAFu, 0x3F5C89D9u}
__device__ __forceinline__ uint32_t nearest_nf4(float v, const float* thr) {
    // thr: the 15 thresholds (and +Inf as a 16th) in shared memory; 16 words in 16 banks, so any mix of indices in a
    // warp is served in one pass.  The two upper levels of the search use constants, the two lower ones the table.
    constexpr uint32_t T[15] = NF4_THR_BITS;
    const bool b3 = v > __uint_as_float(T[7]);
    const bool b2 = v > (b3 ? __uint_as_float(T[11]) : __uint_as_float(T[3]));
    uint32_t lo = (b3 ? 8u : 0u) + (b2 ? 4u : 0u);
    lo += thr[lo + 1] < v ? 2u : 0u;
    lo += thr[lo] < v ? 1u : 0u;
    return lo;
}
__device__ __forceinline__ void nf4_load_thresholds(float* thr) {
    constexpr uint32_t T[15] = NF4_THR_BITS;
    if (threadIdx.x < 16) {
        uint32_t bits = 0x7F800000u;
#pragma unroll
        for (int i = 0; i < 15; i++) bits = threadIdx.x == i ? T[i] : bits;
        thr[threadIdx.x] = __uint_as_float(bits);
    }
    __syncthreads();
}

// Eight consecutive elements per lane (one packed word); LPB lanes share a block of 8 * LPB elements.
template <int LPB>
__global__ void __launch_bounds__(256, 5) nf4_quant_kernel(const float* __restrict__ x, int64_t n, uint8_t* __restrict__ packed,
                                                        float* __restrict__ absmaxs) {
    pdl_trigger();
    pdl_wait();
    __shared__ float thr[16];
    nf4_load_thresholds(thr);
    const int64_t nitems = n >> 3;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    // whole warps iterate together so the shuffles below always have their partners; two items per lane and trip, both
    // requested before either is encoded
    constexpr int ILP = 2;
    for (int64_t t0 = blockIdx.x * (int64_t)blockDim.x + (threadIdx.x & ~31); t0 < nitems; t0 += ILP * stride) {
        float f[ILP][8];
#pragma unroll
        for (int j = 0; j < ILP; j++) {
            const int64_t t = t0 + j * stride + (threadIdx.x & 31);
            if (t < nitems) load8f(x + t * 8, f[j]);
            else {
#pragma unroll
                for (int e = 0; e < 8; e++) f[j][e] = 0.0f;
            }
        }
#pragma unroll
        for (int j = 0; j < ILP; j++) {
            const int64_t t = t0 + j * stride + (threadIdx.x & 31);
            float am = 0.0f;
#pragma unroll
            for (int e = 0; e < 8; e++) am = fmaxf(am, fabsf(f[j][e]));
#pragma unroll
            for (int o = LPB / 2; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
            am = am < 1e-8f ? 1e-8f : am;
            if (t >= nitems) continue;
            const InvDiv d = make_invdiv(am);
            uint32_t w = 0;
#pragma unroll
            for (int e = 0; e < 8; e++) {
                // |x| <= absmax, so the quotient is already in [-1, 1] (the reference's clamp never acts); a NaN stays
                // NaN and takes code 0, +-0 both take code 7
                w |= nearest_nf4(div_exact_bounded(f[j][e], d), thr) << (4 * e);
            }
            __stcs(reinterpret_cast<uint32_t*>(packed) + t, w);
            if ((t & (LPB - 1)) == 0) absmaxs[t / LPB] = am;
        }
    }
}

// Any even block size: a warp per block, two elements (one byte) per lane and step.
__global__ void __launch_bounds__(256) nf4_quant_generic_kernel(const float* __restrict__ x, int64_t nblocks, int64_t block,
                                                                uint8_t* __restrict__ packed, float* __restrict__ absmaxs) {
    pdl_trigger();
    pdl_wait();
    __shared__ float thr[16];
    nf4_load_thresholds(thr);
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5, nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t b = warp0; b < nblocks; b += nwarps) {
        const float* xb = x + b * block;
        float am = 0.0f;
        for (int64_t i = lane; i < block; i += 32) am = fmaxf(am, fabsf(xb[i]));
        am = warp_max(am);
        am = am < 1e-8f ? 1e-8f : am;
        if (lane == 0) absmaxs[b] = am;
        for (int64_t i = lane; i < block / 2; i += 32) {
            const float v0 = fminf(fmaxf(__fdiv_rn(xb[2 * i], am), -1.0f), 1.0f), v1 = fminf(fmaxf(__fdiv_rn(xb[2 * i + 1], am), -1.0f), 1.0f);
            packed[b * (block / 2) + i] = (uint8_t)(nearest_nf4(v0, thr) | (nearest_nf4(v1, thr) << 4));
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(256) nf4_dequant_kernel(const uint8_t* __restrict__ packed, const float* __restrict__ absmaxs, int64_t n,
                                                          int64_t block, T* __restrict__ y) {
    pdl_trigger();
    pdl_wait();
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const uint32_t code = (packed[i >> 1] >> ((i & 1) * 4)) & 0xFu;
        y[i] = Elem<T>::from_f32(c_nf4[code] * __ldg(absmaxs + i / block));
    }
}

// ------------------------------------------------------------------------------------------------
// RMSNorm fused with the per-row INT8 quantizer (the activation path in front of a W8A8 GEMM)
// ------------------------------------------------------------------------------------------------

// One CTA per row at a time; the row (up to 256 * 8 * NV elements) stays in registers between the three phases:
// sum of squares -> inv_rms, y = x * inv_rms * weight and its maximum -> scale, codes.  Two block reductions.
__device__ __forceinline__ float block_reduce_sum(float v, float* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = (threadIdx.x & 31) < 8 ? red[threadIdx.x & 31] : 0.0f;
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    t = __shfl_sync(0xffffffffu, t, 0);
    __syncthreads();
    return t;
}
__device__ __forceinline__ float block_reduce_max(float v, float* red) {
    v = warp_max(v);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = (threadIdx.x & 31) < 8 ? red[threadIdx.x & 31] : 0.0f;
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, o));
    t = __shfl_sync(0xffffffffu, t, 0);
    __syncthreads();
    return t;
}

template <typename T, int NV>
__global__ void __launch_bounds__(256) rmsnorm_int8_rows_kernel(const T* __restrict__ x, const float* __restrict__ weight, int64_t rows,
                                                                int64_t cols, float eps, int8_t* __restrict__ q, float* __restrict__ scales,
                                                                T* __restrict__ y_out) {
    pdl_trigger();
    pdl_wait();
    __shared__ float red[8];
    const int64_t nitems = cols >> 3;
    Raw8<T> nxt[NV];                                          // the next row of this CTA, requested a row ahead
    if ((int64_t)blockIdx.x < rows) {
#pragma unroll
        for (int i = 0; i < NV; i++) {
            const int64_t it = threadIdx.x + (int64_t)i * 256;
            if (it < nitems) nxt[i] = load8raw(x + (int64_t)blockIdx.x * cols + it * 8);
        }
    }
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        float f[NV][8];
        float ss = 0.0f;
#pragma unroll
        for (int i = 0; i < NV; i++) {
            const int64_t it = threadIdx.x + (int64_t)i * 256;
            if (it < nitems) {
                raw8_to_f32(nxt[i], f[i]);
#pragma unroll
                for (int e = 0; e < 8; e++) ss = fmaf(f[i][e], f[i][e], ss);
            }
        }
        if (row + gridDim.x < rows) {
#pragma unroll
            for (int i = 0; i < NV; i++) {
                const int64_t it = threadIdx.x + (int64_t)i * 256;
                if (it < nitems) nxt[i] = load8raw(x + (row + gridDim.x) * cols + it * 8);
            }
        }
        ss = block_reduce_sum(ss, red);
        const float inv_rms = __fdiv_rn(1.0f, sqrtf(__fdiv_rn(ss, (float)cols) + eps));
        float am = 0.0f;
#pragma unroll
        for (int i = 0; i < NV; i++) {
            const int64_t it = threadIdx.x + (int64_t)i * 256;
            if (it < nitems) {
                const float4 w0 = __ldg(reinterpret_cast<const float4*>(weight + it * 8)), w1 = __ldg(reinterpret_cast<const float4*>(weight + it * 8) + 1);
                const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
                for (int e = 0; e < 8; e++) {
                    f[i][e] = f[i][e] * inv_rms * wv[e];                   // the reference's order of the two multiplications
                    am = fmaxf(am, fabsf(f[i][e]));
                }
                if (y_out) {
                    T o[8];
#pragma unroll
                    for (int e = 0; e < 8; e++) o[e] = Elem<T>::from_f32(f[i][e]);
                    if (sizeof(T) == 4) {
                        float4* yo = reinterpret_cast<float4*>(y_out + row * cols + it * 8);
                        yo[0] = *reinterpret_cast<float4*>(&o[0]); yo[1] = *reinterpret_cast<float4*>(&o[4]);
                    } else {
                        *reinterpret_cast<uint4*>(y_out + row * cols + it * 8) = *reinterpret_cast<uint4*>(&o[0]);
                    }
                }
            }
        }
        am = block_reduce_max(am, red);
        // per-row symmetric INT8 as in the row quantizer: scale = max(absmax, 1e-8) / 127, codes rounded half to even
        const float sc = __fdiv_rn(fmaxf(am, 1e-8f), 127.0f);
        if (threadIdx.x == 0) scales[row] = sc;
        const InvDiv d = make_invdiv(sc);
#pragma unroll
        for (int i = 0; i < NV; i++) {
            const int64_t it = threadIdx.x + (int64_t)i * 256;
            if (it < nitems) {
                uint2 o;
                o.x = pack_low_bytes(quant_i8_rne_bits(f[i][0], d), quant_i8_rne_bits(f[i][1], d), quant_i8_rne_bits(f[i][2], d), quant_i8_rne_bits(f[i][3], d));
                o.y = pack_low_bytes(quant_i8_rne_bits(f[i][4], d), quant_i8_rne_bits(f[i][5], d), quant_i8_rne_bits(f[i][6], d), quant_i8_rne_bits(f[i][7], d));
                *reinterpret_cast<uint2*>(q + row * cols + it * 8) = o;
            }
        }
    }
}

// RMSNorm fused with the E4M3 quantizer at a calibrated (static) per-tensor scale: the activation path in front of
// an FP8 GEMM.  Same structure as the INT8 form, minus the second reduction.
template <typename T, int NV>
__global__ void __launch_bounds__(256) rmsnorm_fp8_rows_kernel(const T* __restrict__ x, const float* __restrict__ weight, int64_t rows,
                                                               int64_t cols, float eps, const float* __restrict__ scale_ptr,
                                                               uint8_t* __restrict__ q) {
    pdl_trigger();
    pdl_wait();
    __shared__ float red[8];
    const InvDiv d = make_invdiv(__ldg(scale_ptr));
    const int64_t nitems = cols >> 3;
    Raw8<T> nxt[NV];
    if ((int64_t)blockIdx.x < rows) {
#pragma unroll
        for (int i = 0; i < NV; i++) {
            const int64_t it = threadIdx.x + (int64_t)i * 256;
            if (it < nitems) nxt[i] = load8raw(x + (int64_t)blockIdx.x * cols + it * 8);
        }
    }
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        float f[NV][8];
        float ss = 0.0f;
#pragma unroll
        for (int i = 0; i < NV; i++) {
            const int64_t it = threadIdx.x + (int64_t)i * 256;
            if (it < nitems) {
                raw8_to_f32(nxt[i], f[i]);
#pragma unroll
                for (int e = 0; e < 8; e++) ss = fmaf(f[i][e], f[i][e], ss);
            }
        }
        if (row + gridDim.x < rows) {
#pragma unroll
            for (int i = 0; i < NV; i++) {
                const int64_t it = threadIdx.x + (int64_t)i * 256;
                if (it < nitems) nxt[i] = load8raw(x + (row + gridDim.x) * cols + it * 8);
            }
        }
        ss = block_reduce_sum(ss, red);
        const float inv_rms = __fdiv_rn(1.0f, sqrtf(__fdiv_rn(ss, (float)cols) + eps));
#pragma unroll
        for (int i = 0; i < NV; i++) {
            const int64_t it = threadIdx.x + (int64_t)i * 256;
            if (it < nitems) {
                const float4 w0 = __ldg(reinterpret_cast<const float4*>(weight + it * 8)), w1 = __ldg(reinterpret_cast<const float4*>(weight + it * 8) + 1);
                const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
                float v[8];
#pragma unroll
                for (int e = 0; e < 8; e++) v[e] = div_exact(f[i][e] * inv_rms * wv[e], d);
                uint2 o;
                o.x = (uint32_t)cvt_e4m3x2(v[0], v[1]) | ((uint32_t)cvt_e4m3x2(v[2], v[3]) << 16);
                o.y = (uint32_t)cvt_e4m3x2(v[4], v[5]) | ((uint32_t)cvt_e4m3x2(v[6], v[7]) << 16);
                *reinterpret_cast<uint2*>(q + row * cols + it * 8) = o;
            }
        }
    }
}

// silu_gate of the reference (crates/oxicuda-lm/src/ptx_kernels.rs:222-290: out = gate / (1 + exp(-gate)) * up) fused
// with the E4M3 quantizer at a static scale: the activation of a SwiGLU MLP written once, as one byte per element.
template <typename T>
__global__ void __launch_bounds__(256) silu_gate_fp8_kernel(const T* __restrict__ gate, const T* __restrict__ up, int64_t n,
                                                            const float* __restrict__ scale_ptr, uint8_t* __restrict__ q) {
    pdl_trigger();
    pdl_wait();
    const InvDiv d = make_invdiv(__ldg(scale_ptr));
    const int64_t nitems = n >> 3;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t it = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; it < nitems; it += 2 * stride) {
        const int64_t it2 = it + stride;
        const bool two = it2 < nitems;
        Raw8<T> g0 = load8raw(gate + it * 8), u0 = load8raw(up + it * 8), g1 = g0, u1 = u0;
        if (two) { g1 = load8raw(gate + it2 * 8); u1 = load8raw(up + it2 * 8); }
#pragma unroll
        for (int h = 0; h < 2; h++) {
            if (h == 1 && !two) break;
            float g[8], u[8], v[8];
            raw8_to_f32(h ? g1 : g0, g);
            raw8_to_f32(h ? u1 : u0, u);
#pragma unroll
            for (int e = 0; e < 8; e++) v[e] = div_exact(__fdividef(g[e], 1.0f + __expf(-g[e])) * u[e], d);   // a few f32 ulp, far below an E4M3 step
            uint2 o;
            o.x = (uint32_t)cvt_e4m3x2(v[0], v[1]) | ((uint32_t)cvt_e4m3x2(v[2], v[3]) << 16);
            o.y = (uint32_t)cvt_e4m3x2(v[4], v[5]) | ((uint32_t)cvt_e4m3x2(v[6], v[7]) << 16);
            __stcs(reinterpret_cast<uint2*>(q + (h ? it2 : it) * 8), o);
        }
    }
    if (blockIdx.x == 0) {                                    // ragged tail
        for (int64_t i = nitems * 8 + threadIdx.x; i < n; i += blockDim.x) {
            const float g = Elem<T>::to_f32(gate[i]), u = Elem<T>::to_f32(up[i]);
            q[i] = (uint8_t)(cvt_e4m3x2(div_exact(__fdividef(g, 1.0f + __expf(-g)) * u, d), 0.0f) & 0xFF);
        }
    }
}

// ------------------------------------------------------------------------------------------------
// SmoothQuant migration (per-channel scale folded from the activations into the weights)
// ------------------------------------------------------------------------------------------------

// Per-column max |x| of a row-major [rows x cols] f32 matrix: a thread owns four columns, a CTA row covers 1024
// columns, CTAs along y split the rows; the partial maxima meet in `stats` (zero on entry) through integer
// atomicMax on the bit patterns of the non-negative floats.
__global__ void __launch_bounds__(256) col_absmax_kernel(const float* __restrict__ x, int64_t rows, int64_t cols, float* __restrict__ stats) {
    pdl_trigger();
    pdl_wait();
    const int64_t c = ((int64_t)blockIdx.x * 256 + threadIdx.x) * 4;
    if (c >= cols) return;
    float4 m = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c + 4 <= cols && ((cols & 3) == 0)) {
        for (int64_t r = blockIdx.y; r < rows; r += gridDim.y) {
            const float4 v = __ldcs(reinterpret_cast<const float4*>(x + r * cols + c));
            m.x = fmaxf(m.x, fabsf(v.x)); m.y = fmaxf(m.y, fabsf(v.y)); m.z = fmaxf(m.z, fabsf(v.z)); m.w = fmaxf(m.w, fabsf(v.w));
        }
    } else {
        float* mm = &m.x;
        for (int64_t r = blockIdx.y; r < rows; r += gridDim.y)
            for (int e = 0; e < 4 && c + e < cols; e++) mm[e] = fmaxf(mm[e], fabsf(x[r * cols + c + e]));
    }
    const float mv[4] = {m.x, m.y, m.z, m.w};
    for (int e = 0; e < 4 && c + e < cols; e++)
        if (mv[e] > 0.0f) atomicMax(reinterpret_cast<int*>(stats) + c + e, __float_as_int(mv[e]));
}

// s_j = max(|a_j|, 1e-8)^alpha / max(|w_j|, 1e-8)^(1 - alpha)
__global__ void __launch_bounds__(256) smooth_scales_kernel(const float* __restrict__ a, const float* __restrict__ w, int64_t n, float alpha,
                                                            float* __restrict__ s) {
    pdl_trigger();
    pdl_wait();
    const int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= n) return;
    const float av = fmaxf(fabsf(a[j]), 1e-8f), wv = fmaxf(fabsf(w[j]), 1e-8f);
    s[j] = __fdiv_rn(powf(av, alpha), powf(wv, 1.0f - alpha));
}

// DIVIDE: x[r, j] /= max(s_j, 1e-12) (activations); otherwise x[r, j] *= s_j (weights).  In place.
template <bool DIVIDE>
__global__ void __launch_bounds__(256) smooth_apply_kernel(float* __restrict__ x, int64_t rows, int64_t cols, const float* __restrict__ s) {
    pdl_trigger();
    pdl_wait();
    const int64_t total = rows * cols;
    if ((cols & 3) == 0) {
        const int64_t nvec = total >> 2, cv = cols >> 2;
        for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += (int64_t)gridDim.x * blockDim.x) {
            const int64_t j = (v % cv) << 2;
            float4 d = *reinterpret_cast<float4*>(x + (v << 2));
            const float4 sc = __ldg(reinterpret_cast<const float4*>(s + j));
            if (DIVIDE) {
                d.x = __fdiv_rn(d.x, fmaxf(sc.x, 1e-12f)); d.y = __fdiv_rn(d.y, fmaxf(sc.y, 1e-12f));
                d.z = __fdiv_rn(d.z, fmaxf(sc.z, 1e-12f)); d.w = __fdiv_rn(d.w, fmaxf(sc.w, 1e-12f));
            } else {
                d.x *= sc.x; d.y *= sc.y; d.z *= sc.z; d.w *= sc.w;
            }
            *reinterpret_cast<float4*>(x + (v << 2)) = d;
        }
    } else {
        for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
            const float sc = s[i % cols];
            x[i] = DIVIDE ? __fdiv_rn(x[i], fmaxf(sc, 1e-12f)) : x[i] * sc;
        }
    }
}

// y[m, n] += bias[n] on a bf16 matrix with leading dimension ldy (f32 add, one rounding); 8 columns per thread.
__global__ void __launch_bounds__(256) bias_add_bf16_kernel(__nv_bfloat16* __restrict__ y, int64_t ldy, const float* __restrict__ bias,
                                                            int64_t m, int64_t n) {
    pdl_trigger();
    pdl_wait();
    const int64_t per_row = n >> 3;
    for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < m * per_row; t += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = t / per_row, c = (t - r * per_row) << 3;
        uint4* p = reinterpret_cast<uint4*>(y + r * ldy + c);
        uint4 u = *p;
        uint32_t w[4] = {u.x, u.y, u.z, u.w};
        const float4 b0 = __ldg(reinterpret_cast<const float4*>(bias + c)), b1 = __ldg(reinterpret_cast<const float4*>(bias + c) + 1);
        const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float lo = __uint_as_float(w[i] << 16) + b[2 * i], hi = __uint_as_float(w[i] & 0xFFFF0000u) + b[2 * i + 1];
            const __nv_bfloat162 o = __floats2bfloat162_rn(lo, hi);
            w[i] = *reinterpret_cast<const uint32_t*>(&o);
        }
        *p = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

static inline int grid_cap(oxq_handle* h, int64_t threads_needed, int block, int ctas_per_sm) {
    int64_t need = (threads_needed + block - 1) / block;
    const int64_t cap = (int64_t)h->sm_count * ctas_per_sm;
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

extern "C" {

int32_t oxq_int8_quant_tensor(oxq_handle* h, const void* x, int dtype, int64_t n, int8_t* q, float* scale_dev) {
    OXQ_CHECK_HANDLE(h);
    if (n == 0) return OXQ_OK;                                 // quantize_to_int8 returns Ok(()) on an empty tensor
    if (n < 0) OXQ_FAIL(h, OXQ_ERR_INVALID_DIMENSION, "negative element count");
    if (!x || !q || !scale_dev || !aligned16(x) || ((uintptr_t)q & 7u)) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null or misaligned pointer");
    if (!h->dev_scratch) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "handle has no reduction cells");
    float* absmax = reinterpret_cast<float*>(h->dev_scratch + 4);          // cells 0-1 belong to the reduction itself
    if (int32_t rc = oxq_absmax(h, x, dtype, n, absmax)) return rc;
    DISPATCH_DTYPE(dtype, oxq_launch(int8_tensor_quant_kernel<T>, grid_cap(h, n / (8 * I8T_ILP) + 1, 256, 8), 256, 0, h->stream, (const T*)x, n, absmax, q, scale_dev));
    OXQ_LAUNCH_CHECK(h);
    return OXQ_OK;
}

int32_t oxq_int8_dequant_tensor(oxq_handle* h, const int8_t* q, const float* scale_dev, int64_t n, void* y, int y_dtype) {
    OXQ_CHECK_HANDLE(h);
    if (n == 0) return OXQ_OK;
    if (n < 0) OXQ_FAIL(h, OXQ_ERR_INVALID_DIMENSION, "negative element count");
    if (!q || !scale_dev || !y) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null pointer");
    if (int32_t rc = oxq_require_sm100(h)) return rc;
    DISPATCH_DTYPE(y_dtype, oxq_launch(int8_tensor_dequant_kernel<T>, grid_cap(h, n, 256, 16), 256, 0, h->stream, q, n, scale_dev, (T*)y));
    OXQ_LAUNCH_CHECK(h);
    return OXQ_OK;
}

int32_t oxq_int8_block_quant(oxq_handle* h, const float* x, int64_t n, int64_t block, int8_t* q, float* scales) {
    OXQ_CHECK_HANDLE(h);
    if (block <= 0) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "block_size must be > 0");
    if (n == 0) return OXQ_OK;
    if (n < 0) OXQ_FAIL(h, OXQ_ERR_INVALID_DIMENSION, "negative element count");
    if (!x || !q || !scales) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null pointer");
    if (int32_t rc = oxq_require_sm100(h)) return rc;
    const int64_t nblocks = (n + block - 1) / block;
    oxq_launch(int8_block_quant_kernel, grid_cap(h, nblocks * 32, 256, 8), 256, 0, h->stream, x, n, block, nblocks, q, scales);
    OXQ_LAUNCH_CHECK(h);
    return OXQ_OK;
}

int32_t oxq_int8_block_dequant(oxq_handle* h, const int8_t* q, const float* scales, int64_t n, int64_t block, float* y) {
    OXQ_CHECK_HANDLE(h);
    if (block <= 0) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "block_size must be > 0");
    if (n == 0) return OXQ_OK;
    if (n < 0) OXQ_FAIL(h, OXQ_ERR_INVALID_DIMENSION, "negative element count");
    if (!q || !scales || !y) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null pointer");
    if (int32_t rc = oxq_require_sm100(h)) return rc;
    oxq_launch(int8_block_dequant_kernel, grid_cap(h, n, 256, 16), 256, 0, h->stream, q, scales, n, block, y);
    OXQ_LAUNCH_CHECK(h);
    return OXQ_OK;
}

int32_t oxq_rmsnorm_int8_quant_rows(oxq_handle* h, const void* x, int dtype, const float* weight, int64_t rows, int64_t cols, float eps,
                                    int8_t* q, float* scales, void* y_opt) {
    OXQ_CHECK_HANDLE(h);
    if (rows <= 0 || cols <= 0) OXQ_FAIL(h, OXQ_ERR_EMPTY_INPUT, "rmsnorm: empty input");
    if (cols % 8 != 0 || cols > 16384) OXQ_FAIL(h, OXQ_ERR_INVALID_DIMENSION, "rmsnorm + int8: cols must be a multiple of 8 and at most 16384, got %lld", (long long)cols);
    if (!x || !weight || !q || !scales || !aligned16(x) || !aligned16(weight) || ((uintptr_t)q & 7u) || (y_opt && !aligned16(y_opt)))
        OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null or misaligned pointer");
    if (dtype == OXQ_F32 && ((cols * 4) & 31)) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "f32 rows must be 32-byte multiples");
    if (int32_t rc = oxq_require_sm100(h)) return rc;
    const int64_t cap = (int64_t)h->sm_count * 6;
    const int grid = (int)(rows < cap ? rows : cap);
    const int nv = (int)((cols / 8 + 255) / 256);                            // items of 8 per thread
#define LAUNCH_RN(TT, NVV) oxq_launch(rmsnorm_int8_rows_kernel<TT, NVV>, grid, 256, 0, h->stream, (const TT*)x, weight, rows, cols, eps, q, scales, (TT*)y_opt)
#define PICK_RN(TT) do { if (nv <= 1) LAUNCH_RN(TT, 1); else if (nv <= 2) LAUNCH_RN(TT, 2); else if (nv <= 4) LAUNCH_RN(TT, 4); else LAUNCH_RN(TT, 8); } while (0)
    switch (dtype) {
        case OXQ_F32: PICK_RN(float); break;
        case OXQ_BF16: PICK_RN(__nv_bfloat16); break;
        case OXQ_F16: PICK_RN(__half); break;
        default: OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "unknown dtype %d", dtype);
    }
#undef PICK_RN
#undef LAUNCH_RN
    OXQ_LAUNCH_CHECK(h);
    return OXQ_OK;
}

int32_t oxq_rmsnorm_fp8_quant_rows(oxq_handle* h, const void* x, int dtype, const float* weight, int64_t rows, int64_t cols, float eps,
                                   const float* scale, uint8_t* q) {
    OXQ_CHECK_HANDLE(h);
    if (rows <= 0 || cols <= 0) OXQ_FAIL(h, OXQ_ERR_EMPTY_INPUT, "rmsnorm: empty input");
    if (cols % 8 != 0 || cols > 16384) OXQ_FAIL(h, OXQ_ERR_INVALID_DIMENSION, "rmsnorm + fp8: cols must be a multiple of 8 and at most 16384, got %lld", (long long)cols);
    if (!x || !weight || !q || !scale || !aligned16(x) || !aligned16(weight) || ((uintptr_t)q & 7u))
        OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null or misaligned pointer");
    if (dtype == OXQ_F32 && ((cols * 4) & 31)) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "f32 rows must be 32-byte multiples");
    if (int32_t rc = oxq_require_sm100(h)) return rc;
    const int64_t cap = (int64_t)h->sm_count * 6;
    const int grid = (int)(rows < cap ? rows : cap);
    const int nv = (int)((cols / 8 + 255) / 256);
#define LAUNCH_RF(TT, NVV) oxq_launch(rmsnorm_fp8_rows_kernel<TT, NVV>, grid, 256, 0, h->stream, (const TT*)x, weight, rows, cols, eps, scale, q)
#define PICK_RF(TT) do { if (nv <= 1) LAUNCH_RF(TT, 1); else if (nv <= 2) LAUNCH_RF(TT, 2); else if (nv <= 4) LAUNCH_RF(TT, 4); else LAUNCH_RF(TT, 8); } while (0)
    switch (dtype) {
        case OXQ_F32: PICK_RF(float); break;
        case OXQ_BF16: PICK_RF(__nv_bfloat16); break;
        case OXQ_F16: PICK_RF(__half); break;
        default: OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "unknown dtype %d", dtype);
    }
#undef PICK_RF
#undef LAUNCH_RF
    OXQ_LAUNCH_CHECK(h);
    return OXQ_OK;
}

int32_t oxq_silu_gate_fp8_quant(oxq_handle* h, const void* gate, const void* up, int dtype, int64_t n, const float* scale, uint8_t* q) {
    OXQ_CHECK_HANDLE(h);
    if (n == 0) return OXQ_OK;
    if (n < 0) OXQ_FAIL(h, OXQ_ERR_INVALID_DIMENSION, "negative element count");
    if (!gate || !up || !scale || !q || !aligned16(gate) || !aligned16(up) || ((uintptr_t)q & 7u)) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null or misaligned pointer");
    if (int32_t rc = oxq_require_sm100(h)) return rc;
    const int grid = grid_cap(h, n / 16 + 1, 256, 8);
    switch (dtype) {
        case OXQ_F32: oxq_launch(silu_gate_fp8_kernel<float>, grid, 256, 0, h->stream, (const float*)gate, (const float*)up, n, scale, q); break;
        case OXQ_BF16: oxq_launch(silu_gate_fp8_kernel<__nv_bfloat16>, grid, 256, 0, h->stream, (const __nv_bfloat16*)gate, (const __nv_bfloat16*)up, n, scale, q); break;
        case OXQ_F16: oxq_launch(silu_gate_fp8_kernel<__half>, grid, 256, 0, h->stream, (const __half*)gate, (const __half*)up, n, scale, q); break;
        default: OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "unknown dtype %d", dtype);
    }
    OXQ_LAUNCH_CHECK(h);
    return OXQ_OK;
}

int32_t oxq_smooth_col_absmax(oxq_handle* h, const float* x, int64_t rows, int64_t cols, float* stats) {
    OXQ_CHECK_HANDLE(h);
    if (rows <= 0 || cols <= 0) OXQ_FAIL(h, OXQ_ERR_EMPTY_INPUT, "compute_act_stats: empty input");
    if (!x || !stats || !aligned16(x)) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null or misaligned pointer");
    if (int32_t rc = oxq_require_sm100(h)) return rc;
    OXQ_CUDA(h, cudaMemsetAsync(stats, 0, (size_t)cols * sizeof(float), h->stream));
    const int64_t gx = (cols + 1023) / 1024;
    int64_t gy = ((int64_t)h->sm_count * 8 + gx - 1) / gx;
    if (gy > rows) gy = rows;
    if (gy > 65535) gy = 65535;
    oxq_launch(col_absmax_kernel, dim3((unsigned)gx, (unsigned)gy), 256, 0, h->stream, x, rows, cols, stats);
    OXQ_LAUNCH_CHECK(h);
    return OXQ_OK;
}

int32_t oxq_smooth_scales(oxq_handle* h, const float* act_max, const float* weight_max, int64_t n, float alpha, float* scales) {
    OXQ_CHECK_HANDLE(h);
    if (n <= 0) OXQ_FAIL(h, OXQ_ERR_EMPTY_INPUT, "SmoothQuantMigrator::compute_migration_scales");
    if (!act_max || !weight_max || !scales) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null pointer");
    if (int32_t rc = oxq_require_sm100(h)) return rc;
    oxq_launch(smooth_scales_kernel, (unsigned)((n + 255) / 256), 256, 0, h->stream, act_max, weight_max, n, alpha, scales);
    OXQ_LAUNCH_CHECK(h);
    return OXQ_OK;
}

int32_t oxq_smooth_apply(oxq_handle* h, float* x, int64_t rows, int64_t cols, const float* scales, int divide) {
    OXQ_CHECK_HANDLE(h);
    if (rows <= 0 || cols <= 0) OXQ_FAIL(h, OXQ_ERR_QUANT_DIMENSION_MISMATCH, "smooth: empty matrix");
    if (!x || !scales || !aligned16(x) || !aligned16(scales)) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null or misaligned pointer");
    if (int32_t rc = oxq_require_sm100(h)) return rc;
    const int grid = grid_cap(h, rows * cols / 4 + 1, 256, 8);
    if (divide) oxq_launch(smooth_apply_kernel<true>, grid, 256, 0, h->stream, x, rows, cols, scales);
    else oxq_launch(smooth_apply_kernel<false>, grid, 256, 0, h->stream, x, rows, cols, scales);
    OXQ_LAUNCH_CHECK(h);
    return OXQ_OK;
}

int32_t oxq_bias_add_bf16(oxq_handle* h, void* y, int64_t ldy, const float* bias, int64_t m, int64_t n) {
    OXQ_CHECK_HANDLE(h);
    if (m <= 0 || n <= 0) OXQ_FAIL(h, OXQ_ERR_INVALID_DIMENSION, "dimensions must be non-zero");
    if (!y || !bias || !aligned16(y) || !aligned16(bias) || (n & 7) || (ldy & 7)) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null or misaligned pointer, or n / ldy not a multiple of 8");
    if (int32_t rc = oxq_require_sm100(h)) return rc;
    oxq_launch(bias_add_bf16_kernel, grid_cap(h, m * n / 8, 256, 8), 256, 0, h->stream, (__nv_bfloat16*)y, ldy, bias, m, n);
    OXQ_LAUNCH_CHECK(h);
    return OXQ_OK;
}

int32_t oxq_nf4_thresholds(float* out15) {
    if (!out15) return OXQ_ERR_INVALID_ARGUMENT;
    const uint32_t t[15] = NF4_THR_BITS;
    memcpy(out15, t, sizeof(t));
    return OXQ_OK;
}

int32_t oxq_nf4_quant(oxq_handle* h, const float* x, int64_t n, int64_t block, uint8_t* packed, float* absmaxs) {
    OXQ_CHECK_HANDLE(h);
    if (block <= 0 || (block & 1)) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "block_size must be positive and even, got %lld", (long long)block);
    if (n <= 0) OXQ_FAIL(h, OXQ_ERR_EMPTY_INPUT, "Nf4Quantizer::encode");
    if (n % block != 0) OXQ_FAIL(h, OXQ_ERR_GROUP_SIZE_MISMATCH, "length %lld is not divisible by block size %lld", (long long)n, (long long)block);
    if (!x || !packed || !absmaxs) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null pointer");
    if (int32_t rc = oxq_require_sm100(h)) return rc;
    const bool vec = aligned16(x) && ((uintptr_t)packed & 3u) == 0;
    const int grid = grid_cap(h, n / 16 + 1, 256, 5);                 // five CTAs of this kernel fit an SM: one full wave, grid-stride loop
    if (vec && block == 32) oxq_launch(nf4_quant_kernel<4>, grid, 256, 0, h->stream, x, n, packed, absmaxs);
    else if (vec && block == 64) oxq_launch(nf4_quant_kernel<8>, grid, 256, 0, h->stream, x, n, packed, absmaxs);
    else if (vec && block == 128) oxq_launch(nf4_quant_kernel<16>, grid, 256, 0, h->stream, x, n, packed, absmaxs);
    else if (vec && block == 256) oxq_launch(nf4_quant_kernel<32>, grid, 256, 0, h->stream, x, n, packed, absmaxs);
    else oxq_launch(nf4_quant_generic_kernel, grid_cap(h, (n / block) * 32, 256, 8), 256, 0, h->stream, x, n / block, block, packed, absmaxs);
    OXQ_LAUNCH_CHECK(h);
    return OXQ_OK;
}

int32_t oxq_nf4_dequant(oxq_handle* h, const uint8_t* packed, const float* absmaxs, int64_t n, int64_t block, void* y, int y_dtype) {
    OXQ_CHECK_HANDLE(h);
    if (block <= 0 || (block & 1)) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "block_size must be positive and even, got %lld", (long long)block);
    if (n <= 0) OXQ_FAIL(h, OXQ_ERR_EMPTY_INPUT, "Nf4Quantizer::decode");
    if (n % block != 0) OXQ_FAIL(h, OXQ_ERR_QUANT_DIMENSION_MISMATCH, "length %lld is not divisible by block size %lld", (long long)n, (long long)block);
    if (!packed || !absmaxs || !y) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null pointer");
    if (int32_t rc = oxq_require_sm100(h)) return rc;
    DISPATCH_DTYPE(y_dtype, oxq_launch(nf4_dequant_kernel<T>, grid_cap(h, n, 256, 16), 256, 0, h->stream, packed, absmaxs, n, block, (T*)y));
    OXQ_LAUNCH_CHECK(h);
    return OXQ_OK;
}

}  // extern "C"
