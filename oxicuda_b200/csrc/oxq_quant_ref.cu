// Quantizers in the reference's own parameter types, so that their outputs can be compared with the reference's
// value for value (the benchmark forms in oxq_quant.cu store f16 scales, packed zero-points and hardware-rounded
// E2M1 / E4M3 codes, which the reference has no counterpart for):
//
//   * MinMaxQuantizer per group, asymmetric, with f32 scales and i32 zero-points
//     (crates/oxicuda-quant/src/scheme/minmax.rs:146-167, :226-232, :275-324);
//   * MicroScalingQuantizer::quantize_fp4 with f32 block scales and the floor-type E2M1 encoder of Fp4Quantizer
//     (crates/oxicuda-blas/src/precision/fp4_fp6_ops.rs:638-699, :763-897);
//   * quantize_to_int4 / dequantize_int4 of the DNN layer (crates/oxicuda-dnn/src/quantize/int4_quantize.rs:132-218,
//     scale kernel :403-545, pack kernel :548-701, unpack :780-826);
//   * quantize_block_scaled of the DNN layer (crates/oxicuda-dnn/src/quantize/block_scale.rs:53-140, kernels :145-345).
//   * the fused dequantise + GEMV of the DNN layer's weight-only plan (crates/oxicuda-dnn/src/quantize/gptq_awq.rs:867-994):
//     unsigned codes packed LSB-first in u32 words, f32 scales per group, f32 vector in and out (a stream over the
//     packed weight; its sums are ordered for the GPU, so it is compared within a tolerance, not bit for bit).
//
// Every division is the IEEE one the reference performs (f32 `/`, div.rn.f32) and sums are never contracted into
// FMAs, so codes, scales and zero-points are bit-exact against the CPU restatement of those lines.
#include "oxq_common.cuh"

namespace oxq {
namespace refq {

__device__ __forceinline__ void load8_f32(const float* p, float (&f)[8]) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p) + 1);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}

// ---- MinMaxQuantizer, per group, asymmetric ------------------------------------------------------------------------
// Items of 8 consecutive elements (one packed code word); LPG = group / 8 adjacent lanes hold one group.
//   range = max(fmax - fmin, 1e-8); scale = range / q_range; zp = clamp(round(-fmin / scale), 0, q_range)   (minmax.rs:226-232)
//   q = clamp(round(x / scale + zp), 0, q_range)                                                              (minmax.rs:65-79, :294)
// round = f32::round (half away from zero) or, with OXQ_ROUND_HALF_EVEN, rint.  NaN elements are skipped by the scan
// and get code 0; a group with an infinite element gets a non-finite scale (the reference returns InvalidScale: host
// wrappers look at the scales).
__global__ void __launch_bounds__(256) int4g_ref_quant_kernel(const float* __restrict__ x, int64_t nitems, int lpg, int rounding,
                                                              uint32_t* __restrict__ codes, float* __restrict__ scales,
                                                              int32_t* __restrict__ zps) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int64_t warp_global = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t base = warp_global * 32; base < nitems; base += nwarps * 32) {          // warp-uniform trip count
        const int64_t t = base + lane;
        const bool live = t < nitems;
        float f[8];
        if (live) load8_f32(x + t * 8, f);
        float mn = INFINITY, mx = -INFINITY;
        if (live) {
#pragma unroll
            for (int e = 0; e < 8; e++) { mn = fminf(mn, f[e]); mx = fmaxf(mx, f[e]); }     // `if v < fmin` / `if v > fmax`: NaNs skipped
        }
        for (int o = lpg >> 1; o > 0; o >>= 1) {
            mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        }
        if (!live) continue;
        const float scale = __fdiv_rn(fmaxf(__fsub_rn(mx, mn), 1e-8f), 15.0f);
        float zf = roundf(__fdiv_rn(-mn, scale));
        zf = zf != zf ? 0.0f : fminf(fmaxf(zf, 0.0f), 15.0f);                               // NaN.clamp() stays NaN, `as i32` gives 0
        uint32_t w = 0;
#pragma unroll
        for (int e = 0; e < 8; e++) {
            float q = round_mode(__fadd_rn(__fdiv_rn(f[e], scale), zf), rounding);
            q = q != q ? 0.0f : fminf(fmaxf(q, 0.0f), 15.0f);
            w |= (uint32_t)q << (4 * e);
        }
        codes[t] = w;
        if ((t % lpg) == 0) { scales[t / lpg] = scale; zps[t / lpg] = (int32_t)zf; }
    }
}

// (q - zp) as f32 * scale, the integer subtraction first (minmax.rs:305, :320)
__global__ void __launch_bounds__(256) int4g_ref_dequant_kernel(const uint32_t* __restrict__ codes, const float* __restrict__ scales,
                                                                const int32_t* __restrict__ zps, int64_t nitems, int lpg,
                                                                float* __restrict__ y) {
    pdl_trigger();
    pdl_wait();
    for (int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; t < nitems; t += (int64_t)gridDim.x * blockDim.x) {
        const float s = __ldg(scales + t / lpg);
        const int zp = __ldg(zps + t / lpg);
        const uint32_t w = __ldg(codes + t);
        float o[8];
#pragma unroll
        for (int e = 0; e < 8; e++) o[e] = __fmul_rn((float)((int)((w >> (4 * e)) & 0xFu) - zp), s);
        float4* yo = reinterpret_cast<float4*>(y + t * 8);
        yo[0] = make_float4(o[0], o[1], o[2], o[3]);
        yo[1] = make_float4(o[4], o[5], o[6], o[7]);
    }
}

// ---- MicroScalingQuantizer::quantize_fp4 ---------------------------------------------------------------------------
// Fp4Quantizer::quantize_one for E2M1 (fp4_fp6_ops.rs:645-661): 0 -> 0 (the sign of a zero is dropped), a = min(|v|, 6),
// exponent from floor(log2 a), mantissa bit = (significand - 1 >= 0.5).  The significand is a / 2^e exactly, so the code
// is a function of which of the intervals [0, .75) [.75, 1) [1, 1.5) [1.5, 2) [2, 3) [3, 4) [4, 6) [6, 6] holds a: the
// comparisons below are that function without the logarithm.  A NaN becomes +6 (`NaN.min(6.0)` is 6 and `NaN < 0` is false).
__device__ __forceinline__ uint32_t e2m1_floor_code(float v) {
    if (v == 0.0f) return 0u;
    const uint32_t sign = v < 0.0f ? 8u : 0u;
    const float a = fminf(fabsf(v), 6.0f);
    const uint32_t c = a < 0.75f ? 0u : a < 1.0f ? 1u : a < 1.5f ? 2u : a < 2.0f ? 3u : a < 3.0f ? 4u : a < 4.0f ? 5u : a < 6.0f ? 6u : 7u;
    return sign | c;
}

// Items of 8 elements; LPG = block / 8 lanes hold one block.  scale = max|x| / 6, or 1 for an all-zero block
// (compute_scales, :763-782); the last block may be short; codes of x / scale, two per byte, even element low (:465-472).
__global__ void __launch_bounds__(256) fp4_microscale_quant_kernel(const float* __restrict__ x, int64_t n, int lpg,
                                                                   uint8_t* __restrict__ packed, float* __restrict__ scales) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int64_t nitems = (n + 7) / 8;
    const int64_t warp_global = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const bool vec_ok = (reinterpret_cast<uintptr_t>(x) & 15u) == 0;
    for (int64_t base = warp_global * 32; base < nitems; base += nwarps * 32) {
        const int64_t t = base + lane;
        float f[8];
        if (t * 8 + 8 <= n && vec_ok) load8_f32(x + t * 8, f);
        else {
#pragma unroll
            for (int e = 0; e < 8; e++) f[e] = t * 8 + e < n ? x[t * 8 + e] : 0.0f;
        }
        float am = 0.0f;
#pragma unroll
        for (int e = 0; e < 8; e++) am = fmaxf(am, fabsf(f[e]));                           // f32::max: a NaN is ignored
        for (int o = lpg >> 1; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
        if (t >= nitems) continue;
        const float scale = am == 0.0f ? 1.0f : __fdiv_rn(am, 6.0f);
        if ((t % lpg) == 0) scales[t / lpg] = scale;
        uint32_t w = 0;
#pragma unroll
        for (int e = 0; e < 8; e++) w |= e2m1_floor_code(__fdiv_rn(f[e], scale)) << (4 * e);   // elements past n are 0 -> code 0
        const int64_t nbytes = (n + 1) / 2;
        if (t * 4 + 4 <= nbytes && (reinterpret_cast<uintptr_t>(packed) & 3u) == 0) *reinterpret_cast<uint32_t*>(packed + t * 4) = w;
        else {
            for (int b = 0; b < 4 && t * 4 + b < nbytes; b++) packed[t * 4 + b] = (uint8_t)(w >> (8 * b));
        }
    }
}

__global__ void __launch_bounds__(256) fp4_microscale_dequant_kernel(const uint8_t* __restrict__ packed, const float* __restrict__ scales,
                                                                     int64_t n, int64_t block, float* __restrict__ y) {
    pdl_trigger();
    pdl_wait();
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const uint32_t nib = (packed[i >> 1] >> ((i & 1) * 4)) & 0xFu;
        y[i] = __fmul_rn(e2m1_to_f32(nib), __ldg(scales + i / block));
    }
}

// ---- DNN quantize_to_int4 ------------------------------------------------------------------------------------------
// One warp per group (the reference walks a group with one thread; max and min do not depend on the order).
//   symmetric:  scale = max(absmax, 1e-12) / 7                       (int4_quantize.rs:440-468; INT4_SYM_MAX.abs() is 7)
//   asymmetric: scale = max(max - min, 1e-12) / 15, zero = -min / scale as a float   (:470-530)
__global__ void __launch_bounds__(256) dnn_int4_scale_kernel(const float* __restrict__ x, int64_t n, int64_t group, int64_t ngroups,
                                                             int symmetric, float* __restrict__ scales, float* __restrict__ zeros) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int64_t warp_global = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t g = warp_global; g < ngroups; g += nwarps) {
        const int64_t lo = g * group, hi = lo + group < n ? lo + group : n;
        float amax = 0.0f, mn = INFINITY, mx = -INFINITY;          // f64::MAX / f64::MIN as f32 immediates are +-inf
        for (int64_t i = lo + lane; i < hi; i += 32) {
            const float v = __ldg(x + i);
            amax = fmaxf(amax, fabsf(v));
            mn = mn > v ? v : mn;                                  // setp.gt + selp: a NaN never replaces the minimum
            mx = fmaxf(mx, v);
        }
        amax = warp_max(amax); mn = warp_min(mn); mx = warp_max(mx);
        if (lane == 0) {
            if (symmetric) {
                scales[g] = __fdiv_rn(fmaxf(amax, 1e-12f), 7.0f);
            } else {
                const float sc = __fdiv_rn(fmaxf(__fadd_rn(mx, __fmul_rn(mn, -1.0f)), 1e-12f), 15.0f);
                scales[g] = sc;
                zeros[g] = __fdiv_rn(__fmul_rn(mn, -1.0f), sc);
            }
        }
    }
}

// One output byte (two elements) per thread item, as the reference's pack kernel (:548-701):
//   symmetric:  q = min(trunc(clamp(x / scale, -8, 7) + 8), 15);   asymmetric: q = min(trunc(clamp(x / scale, 0, 15)), 15)
// (the asymmetric form ignores the zero point: the reference's kernel never reads it).  max.f32 returns the other
// operand for a NaN, so a NaN element lands on the lower clamp bound.
__device__ __forceinline__ uint32_t dnn_int4_code(float v, float scale, int symmetric) {
    float s = __fdiv_rn(v, scale);
    if (symmetric) {
        s = fmaxf(s, -8.0f);
        s = s > 7.0f ? 7.0f : s;
        const uint32_t q = (uint32_t)__float2uint_rz(__fadd_rn(s, 8.0f));
        return q > 15u ? 15u : q;
    }
    s = fmaxf(s, 0.0f);
    s = s > 15.0f ? 15.0f : s;
    const uint32_t q = (uint32_t)__float2uint_rz(s);
    return q > 15u ? 15u : q;
}
__global__ void __launch_bounds__(256) dnn_int4_pack_kernel(const float* __restrict__ x, const float* __restrict__ scales, int64_t n,
                                                            int64_t group, int symmetric, uint8_t* __restrict__ packed) {
    pdl_trigger();
    pdl_wait();
    const int64_t nbytes = (n + 1) / 2;
    for (int64_t b = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; b < nbytes; b += (int64_t)gridDim.x * blockDim.x) {
        const int64_t i0 = 2 * b, i1 = 2 * b + 1;
        const uint32_t lo = dnn_int4_code(__ldg(x + i0), __ldg(scales + i0 / group), symmetric);
        const uint32_t hi = i1 < n ? dnn_int4_code(__ldg(x + i1), __ldg(scales + i1 / group), symmetric) : 0u;
        packed[b] = (uint8_t)(lo | (hi << 4));
    }
}
// symmetric: (nibble + (-8)) * scale; asymmetric: nibble * scale (:780-826)
__global__ void __launch_bounds__(256) dnn_int4_unpack_kernel(const uint8_t* __restrict__ packed, const float* __restrict__ scales, int64_t n,
                                                              int64_t group, int symmetric, float* __restrict__ y) {
    pdl_trigger();
    pdl_wait();
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const float nib = (float)((packed[i >> 1] >> ((i & 1) * 4)) & 0xFu);
        const float s = __ldg(scales + i / group);
        y[i] = symmetric ? __fmul_rn(__fadd_rn(nib, -8.0f), s) : __fmul_rn(nib, s);
    }
}

// ---- DNN quantize_block_scaled -------------------------------------------------------------------------------------
//   scale[b] = max(absmax_b / 6, 1e-12)                                            (block_scale.rs:243-249)
//   out[i]   = clamp(int(rint(clamp(x / scale, -6, 6))) + 6, 0, 255) as u8         (:300-333)
template <typename T>
__global__ void __launch_bounds__(256) dnn_block_scale_kernel(const T* __restrict__ x, int64_t n, int64_t block, int64_t nblocks,
                                                              float* __restrict__ scales) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int64_t warp_global = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t b = warp_global; b < nblocks; b += nwarps) {
        const int64_t lo = b * block, hi = lo + block < n ? lo + block : n;
        float am = 0.0f;
        for (int64_t i = lo + lane; i < hi; i += 32) am = fmaxf(am, fabsf(Elem<T>::to_f32(x[i])));
        am = warp_max(am);
        if (lane == 0) scales[b] = fmaxf(__fdiv_rn(am, 6.0f), 1e-12f);
    }
}
template <typename T>
__global__ void __launch_bounds__(256) dnn_block_quant_kernel(const T* __restrict__ x, const float* __restrict__ scales, int64_t n,
                                                              int64_t block, uint8_t* __restrict__ out) {
    pdl_trigger();
    pdl_wait();
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        float s = __fdiv_rn(Elem<T>::to_f32(x[i]), __ldg(scales + i / block));
        s = fminf(fmaxf(s, -6.0f), 6.0f);
        int q = __float2int_rz(rintf(s)) + 6;
        q = q < 0 ? 0 : (q > 255 ? 255 : q);
        out[i] = (uint8_t)q;
    }
}

// ---- fused dequantise + GEMV: y[row] = sum_col (code[row, col] * scale[row, col / group]) * x[col] -------------------------
// dnn_fused_dequant_gemv_f32 (gptq_awq.rs:867-994) gives one thread a whole row.  Here a warp takes FGV_ROWS consecutive rows
// and walks them together: a lane loads 16 bytes of codes of each row per step (the warp 512 contiguous bytes per row) and
// the matching 4 * 32 / BITS elements of x once for all its rows, so x comes from L1 once per FGV_ROWS rows of weights and the
// packed weight is read from HBM exactly once.  Codes become floats by or-ing them into the mantissa of 2^23.  The per-word
// sum is scaled once (a word never straddles a group: group % (32 / BITS) == 0), lanes are summed by shuffles.
constexpr int FGV_ROWS = 4;
constexpr int FGV_WARPS = 4;
template <int BITS>
__global__ void __launch_bounds__(FGV_WARPS * 32) fused_dequant_gemv_kernel(const uint32_t* __restrict__ w, const float* __restrict__ scales,
                                                                            const float* __restrict__ x, float* __restrict__ y, int rows, int words,
                                                                            int group_words, int gpr) {
    pdl_trigger();
    pdl_wait();
    constexpr int EPW = 32 / BITS;                                    // elements per packed word
    constexpr uint32_t MASK = (1u << BITS) - 1u;
    const int lane = threadIdx.x & 31;
    const int row0 = (blockIdx.x * FGV_WARPS + (threadIdx.x >> 5)) * FGV_ROWS;
    if (row0 >= rows) return;
    float acc[FGV_ROWS];
    const uint32_t* wr[FGV_ROWS];
    const float* sr[FGV_ROWS];
#pragma unroll
    for (int r = 0; r < FGV_ROWS; r++) {
        const int row = min(row0 + r, rows - 1);                      // rows past the end repeat the last one and are not stored
        acc[r] = 0.0f;
        wr[r] = w + (size_t)row * words;
        sr[r] = scales + (size_t)row * gpr;
    }
    for (int i = lane * 4; i < words; i += 128) {                     // words % 4 == 0: every lane's four words exist together
        uint4 v[FGV_ROWS];
#pragma unroll
        for (int r = 0; r < FGV_ROWS; r++) v[r] = __ldcs(reinterpret_cast<const uint4*>(wr[r] + i));
#pragma unroll
        for (int q = 0; q < 4; q++) {
            float xv[EPW];
            const float4* xp = reinterpret_cast<const float4*>(x + (size_t)(i + q) * EPW);
#pragma unroll
            for (int e = 0; e < EPW / 4; e++) {
                const float4 t = __ldg(xp + e);
                xv[4 * e] = t.x; xv[4 * e + 1] = t.y; xv[4 * e + 2] = t.z; xv[4 * e + 3] = t.w;
            }
            const int g = (i + q) / group_words;
#pragma unroll
            for (int r = 0; r < FGV_ROWS; r++) {
                const uint32_t word = q == 0 ? v[r].x : q == 1 ? v[r].y : q == 2 ? v[r].z : v[r].w;
                float part = 0.0f;
#pragma unroll
                for (int e = 0; e < EPW; e++) {
                    const float c = __uint_as_float(((word >> (e * BITS)) & MASK) | 0x4B000000u) - 8388608.0f;
                    part = fmaf(c, xv[e], part);
                }
                acc[r] = fmaf(part, __ldg(sr[r] + g), acc[r]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < FGV_ROWS; r++) {
        float a = acc[r];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
        if (lane == 0 && row0 + r < rows) y[row0 + r] = a;
    }
}

static inline int grid_for(oxq_handle* h, int64_t threads_wanted, int ctas_per_sm) {
    int64_t need = (threads_wanted + 255) / 256;
    const int64_t cap = (int64_t)h->sm_count * ctas_per_sm;
    if (need < 1) need = 1;
    return (int)(need < cap ? need : cap);
}

}  // namespace refq
}  // namespace oxq

using namespace oxq;
using namespace oxq::refq;

extern "C" {

int32_t oxq_int4g_quant_pack_f32(oxq_handle* h, const float* x, int64_t rows, int64_t k, int group, uint32_t* codes, float* scales,
                                 int32_t* zero_points, int rounding) {
    OXQ_CHECK_HANDLE(h);
    if (rows <= 0 || k <= 0) OXQ_FAIL(h, OXQ_ERR_EMPTY_INPUT, "MinMaxQuantizer::calibrate");
    if (!(group == 32 || group == 64 || group == 128 || group == 256)) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "group size %d not in {32,64,128,256}", group);
    if (k % group != 0) OXQ_FAIL(h, OXQ_ERR_GROUP_SIZE_MISMATCH, "tensor length %lld is not divisible by group size %d", (long long)k, group);
    if (!x || !codes || !scales || !zero_points || ((uintptr_t)x & 15u)) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null or misaligned pointer");
    if (rounding != OXQ_ROUND_HALF_EVEN && rounding != OXQ_ROUND_HALF_AWAY) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "rounding %d", rounding);
    if (int32_t rc = oxq_require_sm100(h)) return rc;
    const int64_t nitems = rows * k / 8;
    OXQ_CUDA(h, oxq_launch(int4g_ref_quant_kernel, grid_for(h, nitems, 8), 256, 0, h->stream, x, nitems, group / 8, rounding, codes, scales, zero_points));
    return OXQ_OK;
}

int32_t oxq_int4g_dequant_f32(oxq_handle* h, const uint32_t* codes, const float* scales, const int32_t* zero_points, int64_t rows, int64_t k,
                              int group, float* y) {
    OXQ_CHECK_HANDLE(h);
    if (rows <= 0 || k <= 0) OXQ_FAIL(h, OXQ_ERR_EMPTY_INPUT, "dequantize: empty input");
    if (group <= 0 || group % 8 != 0 || k % group != 0) OXQ_FAIL(h, OXQ_ERR_GROUP_SIZE_MISMATCH, "k %lld vs group %d", (long long)k, group);
    if (!codes || !scales || !zero_points || !y || ((uintptr_t)y & 15u)) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null or misaligned pointer");
    if (int32_t rc = oxq_require_sm100(h)) return rc;
    const int64_t nitems = rows * k / 8;
    OXQ_CUDA(h, oxq_launch(int4g_ref_dequant_kernel, grid_for(h, nitems, 8), 256, 0, h->stream, codes, scales, zero_points, nitems, group / 8, y));
    return OXQ_OK;
}

int32_t oxq_fp4_microscale_quant(oxq_handle* h, const float* x, int64_t n, int64_t block, uint8_t* packed, float* scales) {
    OXQ_CHECK_HANDLE(h);
    // MicroScalingConfig::validate: block sizes 32, 64, 128 (fp4_fp6_ops.rs:202-214)
    if (!(block == 32 || block == 64 || block == 128)) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "micro-scaling block size must be 32, 64 or 128, got %lld", (long long)block);
    if (n <= 0) return OXQ_OK;                                    // an empty slice gives empty outputs in the reference
    if (!x || !packed || !scales) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null pointer");
    if (int32_t rc = oxq_require_sm100(h)) return rc;
    OXQ_CUDA(h, oxq_launch(fp4_microscale_quant_kernel, grid_for(h, (n + 7) / 8, 8), 256, 0, h->stream, x, n, (int)(block / 8), packed, scales));
    return OXQ_OK;
}

int32_t oxq_fp4_microscale_dequant(oxq_handle* h, const uint8_t* packed, const float* scales, int64_t n, int64_t block, float* y) {
    OXQ_CHECK_HANDLE(h);
    if (!(block == 32 || block == 64 || block == 128)) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "micro-scaling block size must be 32, 64 or 128, got %lld", (long long)block);
    if (n <= 0) return OXQ_OK;
    if (!packed || !scales || !y) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null pointer");
    if (int32_t rc = oxq_require_sm100(h)) return rc;
    OXQ_CUDA(h, oxq_launch(fp4_microscale_dequant_kernel, grid_for(h, n, 16), 256, 0, h->stream, packed, scales, n, block, y));
    return OXQ_OK;
}

int32_t oxq_dnn_int4_quant(oxq_handle* h, const float* x, int64_t n, int64_t group_size, int symmetric, uint8_t* packed, float* scales,
                           float* zeros) {
    OXQ_CHECK_HANDLE(h);
    if (group_size <= 0) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "INT4 group_size must be non-zero");      // Int4QuantConfig::new
    if (n <= 0) return OXQ_OK;                                                                           // quantize_to_int4: n == 0 is Ok(())
    if (!x || !packed || !scales || (!symmetric && !zeros)) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null pointer");
    if (int32_t rc = oxq_require_sm100(h)) return rc;
    const int64_t ngroups = (n + group_size - 1) / group_size;
    OXQ_CUDA(h, oxq_launch(dnn_int4_scale_kernel, grid_for(h, ngroups * 32, 8), 256, 0, h->stream, x, n, group_size, ngroups, symmetric ? 1 : 0, scales, zeros));
    OXQ_CUDA(h, oxq_launch(dnn_int4_pack_kernel, grid_for(h, (n + 1) / 2, 16), 256, 0, h->stream, x, (const float*)scales, n, group_size, symmetric ? 1 : 0, packed));
    return OXQ_OK;
}

int32_t oxq_dnn_int4_dequant(oxq_handle* h, const uint8_t* packed, const float* scales, int64_t n, int64_t group_size, int symmetric, float* y) {
    OXQ_CHECK_HANDLE(h);
    if (group_size <= 0) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "INT4 group_size must be non-zero");
    if (n <= 0) return OXQ_OK;
    if (!packed || !scales || !y) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null pointer");
    if (int32_t rc = oxq_require_sm100(h)) return rc;
    OXQ_CUDA(h, oxq_launch(dnn_int4_unpack_kernel, grid_for(h, n, 16), 256, 0, h->stream, packed, scales, n, group_size, symmetric ? 1 : 0, y));
    return OXQ_OK;
}

int32_t oxq_dnn_block_scaled_quant(oxq_handle* h, const void* x, int dtype, int64_t n, int64_t block_size, uint8_t* out, float* scales) {
    OXQ_CHECK_HANDLE(h);
    if (n <= 0) return OXQ_OK;                                                                           // quantize_block_scaled: n == 0 is Ok(())
    if (block_size <= 0 || (block_size & (block_size - 1)) != 0) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "block_size must be a non-zero power of 2, got %lld", (long long)block_size);
    if (block_size < 16) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "block_size must be >= 16, got %lld", (long long)block_size);
    if (!x || !out || !scales) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null pointer");
    if (int32_t rc = oxq_require_sm100(h)) return rc;
    const int64_t nblocks = (n + block_size - 1) / block_size;
    const int g1 = grid_for(h, nblocks * 32, 8), g2 = grid_for(h, n, 16);
    switch (dtype) {
        case OXQ_F32:
            OXQ_CUDA(h, oxq_launch(dnn_block_scale_kernel<float>, g1, 256, 0, h->stream, (const float*)x, n, block_size, nblocks, scales));
            OXQ_CUDA(h, oxq_launch(dnn_block_quant_kernel<float>, g2, 256, 0, h->stream, (const float*)x, (const float*)scales, n, block_size, out));
            break;
        case OXQ_BF16:
            OXQ_CUDA(h, oxq_launch(dnn_block_scale_kernel<__nv_bfloat16>, g1, 256, 0, h->stream, (const __nv_bfloat16*)x, n, block_size, nblocks, scales));
            OXQ_CUDA(h, oxq_launch(dnn_block_quant_kernel<__nv_bfloat16>, g2, 256, 0, h->stream, (const __nv_bfloat16*)x, (const float*)scales, n, block_size, out));
            break;
        case OXQ_F16:
            OXQ_CUDA(h, oxq_launch(dnn_block_scale_kernel<__half>, g1, 256, 0, h->stream, (const __half*)x, n, block_size, nblocks, scales));
            OXQ_CUDA(h, oxq_launch(dnn_block_quant_kernel<__half>, g2, 256, 0, h->stream, (const __half*)x, (const float*)scales, n, block_size, out));
            break;
        default: OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "unknown dtype %d", dtype);
    }
    return OXQ_OK;
}

int32_t oxq_dnn_fused_dequant_gemv(oxq_handle* h, const uint32_t* packed_w, const float* scales, const float* x, float* y, int64_t rows, int64_t cols,
                                   int64_t group_size, int bits) {
    OXQ_CHECK_HANDLE(h);
    if (rows <= 0 || cols <= 0) OXQ_FAIL(h, OXQ_ERR_INVALID_DIMENSION, "fused dequant GEMV: rows and cols must be non-zero");
    if (rows > INT32_MAX || cols > INT32_MAX) OXQ_FAIL(h, OXQ_ERR_INVALID_DIMENSION, "fused dequant GEMV: dimensions exceed 2^31-1");
    if (!(bits == 2 || bits == 4 || bits == 8)) OXQ_FAIL(h, OXQ_ERR_UNSUPPORTED_OPERATION, "fused dequant GEMV covers 2, 4 and 8 bits, got %d", bits);
    const int64_t epw = 32 / bits;
    if (group_size <= 0 || cols % group_size != 0) OXQ_FAIL(h, OXQ_ERR_GROUP_SIZE_MISMATCH, "cols %lld is not divisible by group size %lld", (long long)cols, (long long)group_size);
    if (group_size % epw != 0) OXQ_FAIL(h, OXQ_ERR_GROUP_SIZE_MISMATCH, "group size %lld is not a multiple of the %lld codes of a packed word", (long long)group_size, (long long)epw);
    if (cols % (4 * epw) != 0) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "cols must be a multiple of %lld (four packed words)", (long long)(4 * epw));
    if (!packed_w || !scales || !x || !y || ((uintptr_t)packed_w & 15u) || ((uintptr_t)x & 15u)) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null or misaligned pointer");
    if (int32_t rc = oxq_require_sm100(h)) return rc;
    const int words = (int)(cols / epw), group_words = (int)(group_size / epw), gpr = (int)(cols / group_size);
    const unsigned grid = (unsigned)((rows + FGV_WARPS * FGV_ROWS - 1) / (FGV_WARPS * FGV_ROWS));
    cudaError_t le;
    if (bits == 4) le = oxq_launch(fused_dequant_gemv_kernel<4>, grid, FGV_WARPS * 32, 0, h->stream, packed_w, scales, x, y, (int)rows, words, group_words, gpr);
    else if (bits == 8) le = oxq_launch(fused_dequant_gemv_kernel<8>, grid, FGV_WARPS * 32, 0, h->stream, packed_w, scales, x, y, (int)rows, words, group_words, gpr);
    else le = oxq_launch(fused_dequant_gemv_kernel<2>, grid, FGV_WARPS * 32, 0, h->stream, packed_w, scales, x, y, (int)rows, words, group_words, gpr);
    OXQ_CUDA(h, le);
    return OXQ_OK;
}

}  // extern "C"
