/*
 * oxq_oracle.c -- CPU restatement of the OxiCUDA quantized-inference path.
 *
 * THIS IS TEST INFRASTRUCTURE, NOT PRODUCT CODE.  It is the checker that the
 * parity tests, the smoke run and the CPU-baseline leg of the benchmark compare
 * the CUDA library against.  Nothing in the shipped library or its host layer
 * calls into this file.
 *
 * Two families of functions live here:
 *
 *   orc_ref_*   literal restatements of the reference's scalar CPU arithmetic
 *               ("refcompat").  Each cites the reference file:line it follows.
 *               They are pinned by the reference's own known-answer tests.
 *
 *   orc_spec_*  the arithmetic the benchmark configurations describe where the
 *               reference has no implementation at all (per-tensor FP8 scaling
 *               of bf16 tensors with RNE/satfinite conversion, uint4 g128 with
 *               f16 scales, MXFP8 with E8M0 scales, NVFP4 with E4M3 block
 *               scales and an f32 tensor scale).  PARITY UNPINNED: no reference
 *               code or vector exists for them; they follow the public format
 *               definitions (OCP Microscaling v1.0, the NVFP4 recipe) and the
 *               exact formulas stated beside each function.
 *
 * Build: gcc -O2 -ffp-contract=off -fno-fast-math -fopenmp -shared -fPIC
 * (see the Makefile in this directory).  -ffp-contract=off matters: a fused
 * multiply-add would change x/scale+zp rounding.
 */
#include <math.h>
#include <stdint.h>
#include <stddef.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_OK 0
#define ORC_ERR_EMPTY_INPUT 1
#define ORC_ERR_GROUP_SIZE_MISMATCH 2
#define ORC_ERR_INVALID_SCALE 3
#define ORC_ERR_DIMENSION_MISMATCH 4
#define ORC_ERR_NON_FINITE_FP8 5
#define ORC_ERR_INVALID_BITS 6
#define ORC_ERR_INVALID_ARGUMENT 8

#define ORC_SYMMETRIC 0
#define ORC_ASYMMETRIC 1
#define ORC_ROUND_HALF_EVEN 0
#define ORC_ROUND_HALF_AWAY 1

static inline float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

static inline float clampf(float v, float lo, float hi) {
    /* Rust f32::clamp: NaN stays NaN */
    if (v < lo) return lo;
    if (v > hi) return hi;
    return v;
}

static inline float round_mode(float v, int rounding) {
    /* Rust f32::round == roundf (half away from zero); spec mode == rintf (half to even). */
    return rounding == ORC_ROUND_HALF_AWAY ? roundf(v) : rintf(v);
}

/* Rust `as i32` on a float: NaN -> 0, saturating otherwise. */
static inline int32_t f32_as_i32(float v) {
    if (v != v) return 0;
    if (v >= 2147483648.0f) return INT32_MAX;
    if (v <= -2147483648.0f) return INT32_MIN;
    return (int32_t)v;
}

/* ------------------------------------------------------------------------- */
/* bf16 / f16 helpers                                                         */
/* ------------------------------------------------------------------------- */

uint16_t orc_f32_to_bf16(float f) {
    uint32_t u = f32_bits(f);
    if ((u & 0x7F800000u) == 0x7F800000u && (u & 0x007FFFFFu)) return (uint16_t)((u >> 16) | 0x0040u);
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7FFFu + lsb;
    return (uint16_t)(u >> 16);
}
float orc_bf16_to_f32(uint16_t h) { return bits_f32(((uint32_t)h) << 16); }

/* IEEE binary16 <- f32, round to nearest even, overflow to Inf. */
uint16_t orc_f32_to_f16(float f) {
    uint32_t x = f32_bits(f);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t ax = x & 0x7FFFFFFFu;
    if (ax >= 0x7F800000u) return (uint16_t)(sign | (ax > 0x7F800000u ? 0x7E00u : 0x7C00u));
    if (ax >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u);          /* rounds to >= 65520 -> Inf */
    if (ax < 0x33000001u) return (uint16_t)sign;                        /* <= 2^-25 -> 0 (tie at 2^-25 to even = 0) */
    int e = (int)(ax >> 23) - 127;
    uint32_t man = (ax & 0x007FFFFFu) | 0x00800000u;
    if (e < -14) {                                                      /* subnormal half */
        int shift = 13 + (-14 - e);                                     /* drop bits */
        uint32_t q = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1u);
        uint32_t half = 1u << (shift - 1);
        if (rem > half || (rem == half && (q & 1u))) q++;
        return (uint16_t)(sign | q);
    }
    uint32_t q = ((uint32_t)(e + 15) << 10) | ((man >> 13) & 0x3FFu);
    uint32_t rem = man & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (q & 1u))) q++;
    return (uint16_t)(sign | q);
}
float orc_f16_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t e = (h >> 10) & 0x1Fu, m = h & 0x3FFu;
    if (e == 0) {
        if (m == 0) return bits_f32(sign);
        float v = (float)m * 5.9604644775390625e-08f; /* m * 2^-24 */
        return sign ? -v : v;
    }
    if (e == 31) return bits_f32(sign | 0x7F800000u | (m << 13));
    return bits_f32(sign | ((e + 112u) << 23) | (m << 13));
}

/* ------------------------------------------------------------------------- */
/* A.1  MinMaxQuantizer  (crates/oxicuda-quant/src/scheme/minmax.rs)          */
/* ------------------------------------------------------------------------- */

/* calibrate_slice, minmax.rs:209-243 */
int orc_ref_minmax_calibrate_slice(const float* x, size_t n, int bits, int scheme,
                                   float* scale_out, int32_t* zp_out) {
    if (bits < 1 || bits > 16) return ORC_ERR_INVALID_BITS;      /* new() panics, minmax.rs:99-100 */
    float fmin = INFINITY, fmax = -INFINITY;
    for (size_t i = 0; i < n; i++) {
        float v = x[i];
        if (v < fmin) fmin = v;
        if (v > fmax) fmax = v;
    }
    float scale; int32_t zp;
    if (scheme == ORC_SYMMETRIC) {
        float q_max = (float)(1 << (bits - 1)) - 1.0f;
        float abs_max = fmaxf(fmaxf(fabsf(fmin), fabsf(fmax)), 1e-8f);
        scale = abs_max / q_max;
        zp = 0;
    } else {
        float q_range = (float)((1 << bits) - 1);
        float range = fmaxf(fmax - fmin, 1e-8f);
        scale = range / q_range;
        zp = f32_as_i32(clampf(roundf(-fmin / scale), 0.0f, q_range));
    }
    *scale_out = scale; *zp_out = zp;
    if (!isfinite(scale) || scale <= 0.0f) return ORC_ERR_INVALID_SCALE;
    return ORC_OK;
}

/* calibrate with PerGroup granularity, minmax.rs:134-172; group==0 means PerTensor. */
int orc_ref_minmax_calibrate(const float* x, size_t n, int bits, int scheme, size_t group,
                             float* scales, int32_t* zps) {
    if (n == 0) return ORC_ERR_EMPTY_INPUT;
    if (group == 0) return orc_ref_minmax_calibrate_slice(x, n, bits, scheme, scales, zps);
    if (n % group != 0) return ORC_ERR_GROUP_SIZE_MISMATCH;
    for (size_t g = 0; g < n / group; g++) {
        int rc = orc_ref_minmax_calibrate_slice(x + g * group, group, bits, scheme, scales + g, zps + g);
        if (rc) return rc;
    }
    return ORC_OK;
}

/* calibrate_2d, minmax.rs:179-207 */
int orc_ref_minmax_calibrate_2d(const float* x, size_t rows, size_t cols, int bits, int scheme,
                                float* scales, int32_t* zps) {
    if (rows == 0) return ORC_ERR_EMPTY_INPUT;
    if (cols == 0) return ORC_ERR_DIMENSION_MISMATCH;
    for (size_t r = 0; r < rows; r++) {
        int rc = orc_ref_minmax_calibrate_slice(x + r * cols, cols, bits, scheme, scales + r, zps + r);
        if (rc) return rc;
    }
    return ORC_OK;
}

/* quantize_grouped, minmax.rs:275-299 (quantize :252-268 is the group == n case with one scale).
 * `rounding` = HALF_AWAY and clamp_sym_lo127 = 0 reproduce the reference exactly;
 * HALF_EVEN with clamp_sym_lo127 = 1 is the benchmark-configuration ("spec") variant. */
int orc_minmax_quantize_grouped(const float* x, size_t n, const float* scales, const int32_t* zps,
                                size_t group, int bits, int scheme, int rounding, int clamp_sym_lo127,
                                int32_t* out) {
    if (group == 0 || n % group != 0) return ORC_ERR_GROUP_SIZE_MISMATCH;
    float q_max = scheme == ORC_SYMMETRIC ? (float)(1 << (bits - 1)) - 1.0f : (float)(1 << bits) - 1.0f;
    float q_min = scheme == ORC_SYMMETRIC ? -(float)(1 << (bits - 1)) : 0.0f;
    if (scheme == ORC_SYMMETRIC && clamp_sym_lo127) q_min = -q_max;
    for (size_t g = 0; g < n / group; g++) {
        float scale = scales[g];
        float zp = (float)zps[g];
        for (size_t i = 0; i < group; i++) {
            float v = x[g * group + i] / scale + zp;
            out[g * group + i] = f32_as_i32(clampf(round_mode(v, rounding), q_min, q_max));
        }
    }
    return ORC_OK;
}

/* dequantize_grouped, minmax.rs:309-324 */
void orc_ref_minmax_dequantize_grouped(const int32_t* codes, size_t n, const float* scales,
                                       const int32_t* zps, size_t group, float* out) {
    for (size_t g = 0; g < n / group; g++)
        for (size_t i = 0; i < group; i++)
            out[g * group + i] = (float)(codes[g * group + i] - zps[g]) * scales[g];
}

/* ------------------------------------------------------------------------- */
/* A.2  Fp8Codec (crates/oxicuda-quant/src/scheme/fp8.rs)                      */
/* ------------------------------------------------------------------------- */

static void fp8_params(int e5m2, int* exp_bits, int* man_bits, int* bias, float* maxv) {
    if (e5m2) { *exp_bits = 5; *man_bits = 2; *bias = 15; *maxv = 57344.0f; }
    else      { *exp_bits = 4; *man_bits = 3; *bias = 7;  *maxv = 448.0f; }
}

/* fp32_to_fp8, fp8.rs:163-208 (truncating, with the reference's subnormal shift). */
static uint8_t ref_fp32_to_fp8(float v, int e5m2) {
    int exp_bits, man_bits, bias8; float maxv;
    fp8_params(e5m2, &exp_bits, &man_bits, &bias8, &maxv);
    uint32_t bits = f32_bits(v);
    uint8_t sign = (uint8_t)(bits >> 31);
    int exp32 = (int)((bits >> 23) & 0xFF);
    uint32_t man32 = bits & 0x007FFFFFu;
    if (v == 0.0f) return (uint8_t)(sign << 7);
    int exp8_raw = exp32 - 127 + bias8;
    int man_shift = 23 - man_bits;
    if (exp8_raw <= 0) {
        uint32_t full_man = (man32 | 0x00800000u) >> 1;
        uint32_t shift = (uint32_t)(1 - exp8_raw) + (uint32_t)man_shift;
        if (shift >= 24) return (uint8_t)(sign << 7);
        uint8_t man8 = (uint8_t)(full_man >> shift) & (uint8_t)((1 << man_bits) - 1);
        return (uint8_t)((sign << 7) | man8);
    }
    int max_exp = (1 << exp_bits) - 1;
    if (exp8_raw >= max_exp) return (uint8_t)((sign << 7) | (e5m2 ? 0x7B : 0x7E));
    uint8_t man8 = (uint8_t)(man32 >> man_shift) & (uint8_t)((1 << man_bits) - 1);
    return (uint8_t)((sign << 7) | ((uint8_t)exp8_raw << man_bits) | man8);
}

/* encode_f32, fp8.rs:115-122 */
int orc_ref_fp8_encode(const float* x, size_t n, int e5m2, uint8_t* out) {
    int eb, mb, b; float maxv;
    fp8_params(e5m2, &eb, &mb, &b, &maxv);
    for (size_t i = 0; i < n; i++) {
        if (!isfinite(x[i])) return ORC_ERR_NON_FINITE_FP8;
        out[i] = ref_fp32_to_fp8(clampf(x[i], -maxv, maxv), e5m2);
    }
    return ORC_OK;
}

/* fp8_to_fp32, fp8.rs:210-261.  `leading` is always 0 there because leading_zeros()
 * is taken on a 32-bit value, so subnormals decode as 2^(1-bias) * (1 + m/2^man_bits). */
void orc_ref_fp8_decode(const uint8_t* in, size_t n, int e5m2, float* out) {
    int exp_bits, man_bits, bias8; float maxv;
    fp8_params(e5m2, &exp_bits, &man_bits, &bias8, &maxv);
    for (size_t i = 0; i < n; i++) {
        uint8_t b = in[i];
        uint32_t sign = b >> 7;
        uint32_t exp8 = (b >> man_bits) & ((1u << exp_bits) - 1u);
        uint32_t man8 = b & ((1u << man_bits) - 1u);
        uint32_t all_exp = (1u << exp_bits) - 1u;
        if (!e5m2) {
            if (exp8 == all_exp && man8 == (1u << man_bits) - 1u) { out[i] = NAN; continue; }
        } else if (exp8 == all_exp) {
            out[i] = man8 == 0 ? (sign ? -INFINITY : INFINITY) : NAN; continue;
        }
        int man_shift = 23 - man_bits;
        if (exp8 == 0) {
            if (man8 == 0) { out[i] = bits_f32(sign << 31); continue; }
            uint32_t exp32 = (uint32_t)(127 + 1 - bias8);
            uint32_t man32 = (man8 & ((1u << man_bits) - 1u)) << man_shift;
            out[i] = bits_f32((sign << 31) | (exp32 << 23) | man32); continue;
        }
        uint32_t exp32 = (uint32_t)((int)exp8 - bias8 + 127);
        out[i] = bits_f32((sign << 31) | (exp32 << 23) | (man8 << man_shift));
    }
}

/* IEEE-style conversions (what the hardware cvt.rn.satfinite.e4m3x2.f32 does): round to nearest
 * even, saturate finite overflow and +-Inf to +-448 (0x7E), NaN -> 0x7F.  Used by every orc_spec_*. */
uint8_t orc_e4m3_rne_sat(float v) {
    uint32_t u = f32_bits(v);
    uint8_t sign = (uint8_t)((u >> 24) & 0x80u);
    uint32_t au = u & 0x7FFFFFFFu;
    if (au > 0x7F800000u) return 0x7F;                      /* NaN (sign dropped by the hardware conversion) */
    float a = bits_f32(au);
    if (a >= 464.0f) return (uint8_t)(sign | 0x7E);         /* > max + half ulp(=16)... ties at 464 go to even=512 -> sat */
    if (a > 448.0f) return (uint8_t)(sign | 0x7E);
    /* scale so that one E4M3 step == 1.0, then rintf (RNE).  Subnormal step is 2^-9. */
    int e = (int)(au >> 23) - 127;
    if (e < -6) e = -6;
    float step = bits_f32((uint32_t)(e - 3 + 127) << 23);   /* 2^(e-3) */
    float q = rintf(a / step);                              /* exact division by a power of two */
    float r = q * step;
    if (r > 448.0f) r = 448.0f;
    if (r == 0.0f) return sign;
    uint32_t ru = f32_bits(r);
    int re = (int)(ru >> 23) - 127;
    if (re < -6) {                                          /* subnormal: m * 2^-9 */
        return (uint8_t)(sign | (uint8_t)(r * 512.0f));
    }
    return (uint8_t)(sign | ((uint32_t)(re + 7) << 3) | ((ru >> 20) & 7u));
}
float orc_e4m3_to_f32(uint8_t b) {
    uint32_t sign = b >> 7, e = (b >> 3) & 0xF, m = b & 7;
    float v;
    if (e == 15 && m == 7) return NAN;
    if (e == 0) v = (float)m * 0.001953125f;               /* m * 2^-9 */
    else v = bits_f32(((e + 120u) << 23) | (m << 20));
    return sign ? -v : v;
}

/* ------------------------------------------------------------------------- */
/* A.3  nibble packing (crates/oxicuda-blas/src/precision/int_ops.rs:375-428)  */
/* ------------------------------------------------------------------------- */

int orc_ref_pack_int4(const int8_t* v, size_t n, uint32_t* out) {
    if (n % 8 != 0) return ORC_ERR_INVALID_ARGUMENT;
    for (size_t i = 0; i < n; i++) if (v[i] < -8 || v[i] > 7) return ORC_ERR_INVALID_ARGUMENT;
    for (size_t w = 0; w < n / 8; w++) {
        uint32_t p = 0;
        for (int j = 0; j < 8; j++) p |= ((uint32_t)((uint8_t)v[w * 8 + j] & 0x0F)) << (j * 4);
        out[w] = p;
    }
    return ORC_OK;
}
void orc_ref_unpack_int4(const uint32_t* in, size_t words, int8_t* out) {
    for (size_t w = 0; w < words; w++)
        for (int j = 0; j < 8; j++) {
            uint8_t nib = (uint8_t)((in[w] >> (j * 4)) & 0x0F);
            out[w * 8 + j] = (nib & 0x08) ? (int8_t)(0xF0u | nib) : (int8_t)nib;
        }
}
/* Unsigned variant: same bit positions, no sign extension (GPTQ/AWQ u32 packing,
 * crates/oxicuda-dnn/src/quantize/gptq_awq.rs:936-945). */
void orc_pack_uint4(const uint8_t* v, size_t n, uint32_t* out) {
    for (size_t w = 0; w < n / 8; w++) {
        uint32_t p = 0;
        for (int j = 0; j < 8; j++) p |= ((uint32_t)(v[w * 8 + j] & 0x0F)) << (j * 4);
        out[w] = p;
    }
}
void orc_unpack_uint4(const uint32_t* in, size_t words, uint8_t* out) {
    for (size_t w = 0; w < words; w++)
        for (int j = 0; j < 8; j++) out[w * 8 + j] = (uint8_t)((in[w] >> (j * 4)) & 0x0F);
}

/* dnn_fused_dequant_gemv_f32 (crates/oxicuda-dnn/src/quantize/gptq_awq.rs:867-994): one sequential pass over a row,
 * codes of `bits` bits packed LSB-first in u32 words (element `sub` of a word at bit sub * bits, :936-945), an f32 scale
 * per group of group_size columns, no zero-point:
 *   acc = fma(rn(float(code) * scale[row, col / group_size]), x[col], acc)     (cvt.rn.f32.u32, mul.rn.f32, fma.rn.f32) */
void orc_ref_dnn_fused_dequant_gemv(const uint32_t* packed_w, const float* scales, const float* x, float* y, size_t rows, size_t cols,
                                    size_t group_size, int bits) {
    const size_t epu32 = (size_t)(32 / bits), packed_cols = cols / epu32, gpr = cols / group_size;
    const uint32_t mask = (1u << bits) - 1u;
    for (size_t row = 0; row < rows; row++) {
        float acc = 0.0f;
        for (size_t pw = 0; pw < packed_cols; pw++) {
            const uint32_t word = packed_w[row * packed_cols + pw];
            for (size_t sub = 0; sub < epu32; sub++) {
                const size_t col = pw * epu32 + sub;
                const float dq = (float)((word >> (sub * (size_t)bits)) & mask) * scales[row * gpr + col / group_size];
                acc = fmaf(dq, x[col], acc);
            }
        }
        y[row] = acc;
    }
}

/* ------------------------------------------------------------------------- */
/* A.4  E2M1 + micro-scaling (crates/oxicuda-blas/src/precision/fp4_fp6_ops.rs) */
/* ------------------------------------------------------------------------- */

/* Fp4Quantizer::quantize_one(E2M1), fp4_fp6_ops.rs:645-661 */
uint8_t orc_ref_e2m1_quantize_one(float value) {
    if (value == 0.0f) return 0;
    uint8_t sign = value < 0.0f ? 1 : 0;
    float a = fminf(fabsf(value), 6.0f);
    float l2 = log2f(a);
    int eu = (int)floorf(l2);
    int eb = eu + 1; if (eb < 0) eb = 0; if (eb > 3) eb = 3;
    int ea = eb - 1;
    float sig = a / powf(2.0f, (float)ea);
    uint8_t m = (sig - 1.0f) >= 0.5f ? 1 : 0;
    return (uint8_t)((sign << 3) | ((uint8_t)eb << 1) | m);
}
/* Fp4Quantizer::dequantize_one(E2M1), fp4_fp6_ops.rs:678-697 (also the IEEE E2M1 value). */
float orc_e2m1_to_f32(uint8_t raw) {
    uint8_t sign = (raw >> 3) & 1, e = (raw >> 1) & 3, m = raw & 1;
    float v;
    if (e == 0) v = (float)m * 0.5f;
    else v = (1.0f + (float)m * 0.5f) * (float)(1 << (e - 1));
    return sign ? -v : v;
}
/* MicroScalingQuantizer::compute_scales + quantize_fp4, fp4_fp6_ops.rs:763-782, :849-876.
 * PackedFp4::pack(v0, v1) = v0 | v1 << 4, :465-472.  block in {32,64,128} (:202-214). */
int orc_ref_microscale_fp4(const float* x, size_t n, size_t block, uint8_t* packed, float* scales) {
    if (!(block == 32 || block == 64 || block == 128)) return ORC_ERR_INVALID_ARGUMENT;
    size_t nb = (n + block - 1) / block;
    for (size_t b = 0; b < nb; b++) {
        size_t s = b * block, e = s + block < n ? s + block : n;
        float mx = 0.0f;
        for (size_t i = s; i < e; i++) mx = fmaxf(mx, fabsf(x[i]));
        scales[b] = mx == 0.0f ? 1.0f : mx / 6.0f;
    }
    size_t npad = n + (n & 1);
    for (size_t i = 0; i < npad; i += 2) {
        float v0 = x[i] / scales[i / block];
        float v1 = (i + 1 < n) ? x[i + 1] / scales[(i + 1) / block] : 0.0f;
        packed[i / 2] = (uint8_t)(orc_ref_e2m1_quantize_one(v0) | (orc_ref_e2m1_quantize_one(v1) << 4));
    }
    return ORC_OK;
}
void orc_ref_microscale_fp4_dequant(const uint8_t* packed, const float* scales, size_t n, size_t block, float* out) {
    for (size_t i = 0; i < n; i++) {
        uint8_t nib = (i & 1) ? (packed[i / 2] >> 4) : (packed[i / 2] & 0x0F);
        out[i] = orc_e2m1_to_f32(nib) * scales[i / block];
    }
}

/* Round-to-nearest-even onto the E2M1 grid {0,.5,1,1.5,2,3,4,6} with saturation
 * (the hardware cvt.rn.satfinite.e2m1x2.f32).  Sign is kept, so small negatives give 0x8. */
uint8_t orc_e2m1_rne_sat(float v) {
    uint8_t sign = (uint8_t)((f32_bits(v) >> 28) & 0x8u);
    float a = fabsf(v);
    uint8_t c;
    if (a != a) return 0x7;                       /* NaN -> +max, as the conversion instruction does */
    if (a <= 0.25f) c = 0;                        /* tie 0.25 -> code 0 (even) */
    else if (a < 0.75f) c = 1;
    else if (a <= 1.25f) c = 2;                   /* ties 0.75, 1.25 -> code 2 */
    else if (a < 1.75f) c = 3;
    else if (a <= 2.5f) c = 4;                    /* ties 1.75, 2.5 -> code 4 */
    else if (a < 3.5f) c = 5;
    else if (a <= 5.0f) c = 6;                    /* ties 3.5, 5.0 -> code 6 */
    else c = 7;
    return (uint8_t)(sign | c);
}

/* ------------------------------------------------------------------------- */
/* spec quantizers (PARITY UNPINNED: defined here, see file header)            */
/* ------------------------------------------------------------------------- */

/* INT8 symmetric per-row, benchmark configuration 1:
 * scale = max(absmax_row, 1e-8)/127 (same scale as minmax.rs:221-225); code = clamp(round(x/scale), -127, 127). */
void orc_spec_int8_quant_rows(const float* x, size_t rows, size_t cols, int rounding, int8_t* q, float* scales) {
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < rows; r++) {
        const float* p = x + r * cols;
        float fmin = INFINITY, fmax = -INFINITY;
        for (size_t i = 0; i < cols; i++) { float v = p[i]; if (v < fmin) fmin = v; if (v > fmax) fmax = v; }
        float s = fmaxf(fmaxf(fabsf(fmin), fabsf(fmax)), 1e-8f) / 127.0f;
        scales[r] = s;
        for (size_t i = 0; i < cols; i++)
            q[r * cols + i] = (int8_t)f32_as_i32(clampf(round_mode(p[i] / s, rounding), -127.0f, 127.0f));
    }
}
void orc_spec_int8_dequant_rows(const int8_t* q, const float* scales, size_t rows, size_t cols, float* y) {
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < rows; r++)
        for (size_t i = 0; i < cols; i++) y[r * cols + i] = (float)q[r * cols + i] * scales[r];
}

/* absmax over a tensor; NaNs are skipped exactly as fmaxf skips them. */
float orc_spec_absmax_f32(const float* x, size_t n) {
    float m = 0.0f;
#pragma omp parallel for reduction(max : m) schedule(static)
    for (size_t i = 0; i < n; i++) { float a = fabsf(x[i]); if (a > m) m = a; }
    return m;
}
float orc_spec_absmax_bf16(const uint16_t* x, size_t n) {
    float m = 0.0f;
#pragma omp parallel for reduction(max : m) schedule(static)
    for (size_t i = 0; i < n; i++) { float a = fabsf(orc_bf16_to_f32(x[i])); if (a > m) m = a; }
    return m;
}
/* FP8 E4M3 per-tensor, benchmark configuration 2: scale = absmax/448 (1.0 if the tensor is all zero);
 * code = e4m3_rne_sat(x / scale) with a true IEEE f32 divide. */
float orc_spec_fp8_scale(float absmax) { return absmax > 0.0f ? absmax / 448.0f : 1.0f; }
void orc_spec_fp8_quant_f32(const float* x, size_t n, float scale, uint8_t* out) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) out[i] = orc_e4m3_rne_sat(x[i] / scale);
}
void orc_spec_fp8_quant_bf16(const uint16_t* x, size_t n, float scale, uint8_t* out) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) out[i] = orc_e4m3_rne_sat(orc_bf16_to_f32(x[i]) / scale);
}
void orc_spec_fp8_dequant(const uint8_t* q, size_t n, float scale, float* out) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < n; i++) out[i] = orc_e4m3_to_f32(q[i]) * scale;
}

/* uint4 group-wise asymmetric with f16 scales, benchmark configuration 3.  Per group of `group`
 * consecutive K elements of a row:  s32 = max(max-min, 1e-8)/15 (minmax.rs:226-232);
 * s = f16_rne(s32), bumped to the smallest f16 subnormal if it rounds to zero;
 * zp = clamp(round_half_away(-min / f32(s)), 0, 15); q = clamp(round(x / f32(s) + zp), 0, 15).
 * Codes and zero-points are packed 8 per u32, element j at bits [4j, 4j+4). */
void orc_spec_int4g_quant(const float* x, size_t rows, size_t k, size_t group, int rounding,
                          uint32_t* codes, uint16_t* scales_f16, uint32_t* zeros_packed) {
    size_t gpr = k / group;
    size_t ngroups = rows * gpr;
    memset(zeros_packed, 0, ((ngroups + 7) / 8) * 4);
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < rows; r++) {
        for (size_t g = 0; g < gpr; g++) {
            const float* p = x + r * k + g * group;
            float fmin = INFINITY, fmax = -INFINITY;
            for (size_t i = 0; i < group; i++) { float v = p[i]; if (v < fmin) fmin = v; if (v > fmax) fmax = v; }
            float s32 = fmaxf(fmax - fmin, 1e-8f) / 15.0f;
            uint16_t sh = orc_f32_to_f16(s32);
            if ((sh & 0x7FFFu) == 0) sh = 1;
            float s = orc_f16_to_f32(sh);
            int32_t zp = f32_as_i32(clampf(roundf(-fmin / s), 0.0f, 15.0f));
            size_t gi = r * gpr + g;
            scales_f16[gi] = sh;
#pragma omp atomic
            zeros_packed[gi / 8] |= ((uint32_t)zp) << ((gi % 8) * 4);
            for (size_t w = 0; w < group / 8; w++) {
                uint32_t pk = 0;
                for (int j = 0; j < 8; j++) {
                    float v = p[w * 8 + j] / s + (float)zp;
                    uint32_t qv = (uint32_t)f32_as_i32(clampf(round_mode(v, rounding), 0.0f, 15.0f));
                    pk |= qv << (4 * j);
                }
                codes[(r * k + g * group) / 8 + w] = pk;
            }
        }
    }
}
void orc_spec_int4g_dequant(const uint32_t* codes, const uint16_t* scales_f16, const uint32_t* zeros_packed,
                            size_t rows, size_t k, size_t group, float* out) {
    size_t gpr = k / group;
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < rows; r++)
        for (size_t c = 0; c < k; c++) {
            size_t gi = r * gpr + c / group;
            int32_t zp = (int32_t)((zeros_packed[gi / 8] >> ((gi % 8) * 4)) & 0xF);
            int32_t q = (int32_t)((codes[(r * k + c) / 8] >> ((c % 8) * 4)) & 0xF);
            out[r * k + c] = (float)(q - zp) * orc_f16_to_f32(scales_f16[gi]);
        }
}

/* MXFP8 (OCP Microscaling v1.0): E4M3 elements, one E8M0 scale per 32 consecutive K elements.
 * e = floor(log2(absmax_blk)) - 8; scale byte = clamp(e + 127, 0, 254); all-zero block -> byte 0
 * and codes 0; otherwise code = e4m3_rne_sat(x * 2^-(byte-127)).  0xFF (NaN) is never written. */
static inline float pow2_of(int e) { /* exact 2^e for e in [-127, 127] */
    if (e >= -126) return bits_f32((uint32_t)(e + 127) << 23);
    return bits_f32(0x00400000u);     /* 2^-127, an f32 subnormal */
}
void orc_spec_mxfp8_quant(const float* x, size_t rows, size_t k, uint8_t* codes, uint8_t* sf) {
    size_t bpr = k / 32;
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < rows; r++)
        for (size_t b = 0; b < bpr; b++) {
            const float* p = x + r * k + b * 32;
            float mx = 0.0f;
            for (int i = 0; i < 32; i++) { float a = fabsf(p[i]); if (a > mx) mx = a; }
            uint8_t* c = codes + r * k + b * 32;
            if (mx == 0.0f) { sf[r * bpr + b] = 0; for (int i = 0; i < 32; i++) c[i] = (uint8_t)((f32_bits(p[i]) >> 24) & 0x80u); continue; }
            int e = ilogbf(mx) - 8;
            int byte = e + 127; if (byte < 0) byte = 0; if (byte > 254) byte = 254;
            sf[r * bpr + b] = (uint8_t)byte;
            float inv = pow2_of(-(byte - 127));
            for (int i = 0; i < 32; i++) c[i] = orc_e4m3_rne_sat(p[i] * inv);
        }
}
void orc_spec_mxfp8_dequant(const uint8_t* codes, const uint8_t* sf, size_t rows, size_t k, float* out) {
    size_t bpr = k / 32;
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < rows; r++)
        for (size_t c = 0; c < k; c++)
            out[r * k + c] = orc_e4m3_to_f32(codes[r * k + c]) * pow2_of((int)sf[r * bpr + c / 32] - 127);
}

/* NVFP4: E2M1 elements, one unsigned E4M3 scale per 16 consecutive K elements, one f32 scale per tensor.
 * g = absmax_tensor / (448*6) (1.0 if the tensor is all zero); SF = e4m3_rne_sat(absmax_blk / (6*g));
 * code = e2m1_rne_sat(x / (g * f32(SF))), all codes of a block are (signed) zero when SF == 0.
 * Two codes per byte, even element in the low nibble. */
float orc_spec_nvfp4_global_scale(float absmax) { return absmax > 0.0f ? absmax / (448.0f * 6.0f) : 1.0f; }
void orc_spec_nvfp4_quant(const float* x, size_t rows, size_t k, float g, uint8_t* packed, uint8_t* sf) {
    size_t bpr = k / 16;
    float six_g = 6.0f * g;
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < rows; r++)
        for (size_t b = 0; b < bpr; b++) {
            const float* p = x + r * k + b * 16;
            float mx = 0.0f;
            for (int i = 0; i < 16; i++) { float a = fabsf(p[i]); if (a > mx) mx = a; }
            uint8_t s8 = orc_e4m3_rne_sat(mx / six_g);
            sf[r * bpr + b] = s8;
            float d = g * orc_e4m3_to_f32(s8);
            uint8_t* o = packed + (r * k + b * 16) / 2;
            for (int i = 0; i < 16; i += 2) {
                uint8_t c0, c1;
                if (s8 == 0) { c0 = (uint8_t)((f32_bits(p[i]) >> 28) & 8u); c1 = (uint8_t)((f32_bits(p[i + 1]) >> 28) & 8u); }
                else { c0 = orc_e2m1_rne_sat(p[i] / d); c1 = orc_e2m1_rne_sat(p[i + 1] / d); }
                o[i / 2] = (uint8_t)(c0 | (c1 << 4));
            }
        }
}
void orc_spec_nvfp4_dequant(const uint8_t* packed, const uint8_t* sf, float g, size_t rows, size_t k, float* out) {
    size_t bpr = k / 16;
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < rows; r++)
        for (size_t c = 0; c < k; c++) {
            size_t idx = r * k + c;
            uint8_t nib = (idx & 1) ? (packed[idx / 2] >> 4) : (packed[idx / 2] & 0xF);
            out[idx] = orc_e2m1_to_f32(nib) * orc_e4m3_to_f32(sf[r * bpr + c / 16]) * g;
        }
}

/* ------------------------------------------------------------------------- */
/* A.5  f32 GEMM / SwiGLU / tensor-parallel helpers                            */
/* ------------------------------------------------------------------------- */
/* Rows that follow the hot path: NF4, per-block INT8, per-tensor INT8.          */
/* ------------------------------------------------------------------------- */

/* The 16 NormalFloat4 levels (crates/oxicuda-quant/src/scheme/nf4.rs:33-50). */
static const float NF4_LEVELS[16] = {
    -1.0f, -0.69619286f, -0.52507305f, -0.3949175f, -0.28444138f, -0.18477343f, -0.09105003f, 0.0f,
    0.0795803f, 0.1609302f, 0.2461123f, 0.33791524f, 0.44070983f, 0.562617f, 0.72295684f, 1.0f};

float orc_nf4_level(int i) { return NF4_LEVELS[i & 15]; }

/* nearest_nf4 (nf4.rs:186-205): first index whose level is >= v, then the closer neighbour, the lower
 * index on a tie. */
int orc_ref_nearest_nf4(float v) {
    int lo = 0, hi = 16;
    while (lo < hi) {
        int mid = lo + (hi - lo) / 2;
        if (NF4_LEVELS[mid] < v) lo = mid + 1; else hi = mid;
    }
    if (lo == 0) return 0;
    if (lo == 16) return 15;
    float d_lo = fabsf(v - NF4_LEVELS[lo - 1]);
    float d_hi = fabsf(NF4_LEVELS[lo] - v);
    return d_lo <= d_hi ? lo - 1 : lo;
}

/* Nf4Quantizer::encode (nf4.rs:93-130): per block absmax (floored at 1e-8), v / absmax clamped to [-1, 1],
 * nearest level, even element in the low nibble.  Returns 0, or -1 empty input, -2 length not a multiple of block. */
int orc_ref_nf4_encode(const float* x, size_t n, size_t block, uint8_t* packed, float* absmaxs) {
    if (n == 0) return -1;
    if (block == 0 || n % block != 0) return -2;
    memset(packed, 0, n / 2);
    for (size_t b = 0; b < n / block; b++) {
        const float* blk = x + b * block;
        float am = 0.0f;
        for (size_t i = 0; i < block; i++) am = fmaxf(am, fabsf(blk[i]));
        if (am < 1e-8f) am = 1e-8f;
        absmaxs[b] = am;
        size_t base = b * block / 2;
        for (size_t i = 0; i < block; i++) {
            float normed = clampf(blk[i] / am, -1.0f, 1.0f);
            uint8_t code = (uint8_t)orc_ref_nearest_nf4(normed);
            if (i % 2 == 0) packed[base + i / 2] = code; else packed[base + i / 2] |= (uint8_t)(code << 4);
        }
    }
    return 0;
}

/* Nf4Quantizer::decode (nf4.rs:137-155). */
void orc_ref_nf4_decode(const uint8_t* packed, const float* absmaxs, size_t n, size_t block, float* out) {
    for (size_t i = 0; i < n; i++) {
        uint8_t byte = packed[i / 2];
        int code = (i & 1) ? (byte >> 4) : (byte & 0x0F);
        out[i] = NF4_LEVELS[code] * absmaxs[i / block];
    }
}

/* BlockQuantizedInt8::quantize (crates/oxicuda-dnn/src/quantize/int8_quantize.rs:404-432): per block of
 * `block` contiguous elements (the last one may be short) scale = max|x| / 127, or 1 for an all-zero block;
 * q = clamp(round_half_away(x / scale), -128, 127). */
void orc_ref_block_int8_quant(const float* x, size_t n, size_t block, int8_t* q, float* scales) {
    for (size_t b0 = 0, bi = 0; b0 < n; b0 += block, bi++) {
        size_t len = n - b0 < block ? n - b0 : block;
        float am = 0.0f;
        for (size_t i = 0; i < len; i++) am = fmaxf(am, fabsf(x[b0 + i]));
        float scale = am > 0.0f ? am / 127.0f : 1.0f;
        scales[bi] = scale;
        for (size_t i = 0; i < len; i++) q[b0 + i] = (int8_t)clampf(roundf(x[b0 + i] / scale), -128.0f, 127.0f);
    }
}

/* BlockQuantizedInt8::dequantize (int8_quantize.rs:438-451). */
void orc_ref_block_int8_dequant(const int8_t* q, const float* scales, size_t n, size_t block, float* out) {
    for (size_t i = 0; i < n; i++) out[i] = (float)q[i] * scales[i / block];
}

/* quantize_to_int8 (int8_quantize.rs:33-92; arithmetic of its two generated kernels, :148-330):
 * scale[0] = max(absmax / 127, 1e-12); q = rint(clamp(x / scale, -127, 127)) (round half to even). */
void orc_ref_dnn_int8_quant(const float* x, size_t n, int8_t* q, float* scale) {
    float am = 0.0f;
    for (size_t i = 0; i < n; i++) am = fmaxf(am, fabsf(x[i]));
    float sc = fmaxf(am / 127.0f, 1e-12f);
    scale[0] = sc;
    for (size_t i = 0; i < n; i++) q[i] = (int8_t)rintf(fminf(fmaxf(x[i] / sc, -127.0f), 127.0f));
}

/* dequantize_from_int8 (int8_quantize.rs:101-157): out = (float)q * scale[0]. */
void orc_ref_dnn_int8_dequant(const int8_t* q, size_t n, float scale, float* out) {
    for (size_t i = 0; i < n; i++) out[i] = (float)q[i] * scale;
}

/* quantize_to_int4 (crates/oxicuda-dnn/src/quantize/int4_quantize.rs:132-218), the arithmetic of its two generated
 * kernels.  Scale kernel (:403-545): groups of `group` contiguous elements, the last may be short;
 *   symmetric   scale = max(absmax, 1e-12) / 7          (INT4_SYM_MAX.abs(), :468)
 *   asymmetric  scale = max(max - min, 1e-12) / 15, zero = (-min) / scale kept as a float (:518-536); min starts at
 *               f64::MAX and max at f64::MIN, which are +-inf as f32 immediates; setp.gt / max.f32 skip NaNs.
 * Pack kernel (:548-701): one byte per two elements, even element in the low nibble;
 *   symmetric   q = min(trunc(min(max(x / scale, -8), 7) + 8), 15)
 *   asymmetric  q = min(trunc(min(max(x / scale, 0), 15)), 15)      (the zero point is not read by this kernel)
 * max.f32 with a NaN operand returns the other operand; cvt.rzi truncates. */
void orc_ref_dnn_int4_quant(const float* x, size_t n, size_t group, int symmetric, uint8_t* packed, float* scales, float* zeros) {
    size_t ng = (n + group - 1) / group;
    for (size_t g = 0; g < ng; g++) {
        size_t lo = g * group, hi = lo + group < n ? lo + group : n;
        float amax = 0.0f, mn = INFINITY, mx = -INFINITY;
        for (size_t i = lo; i < hi; i++) {
            float v = x[i];
            amax = fmaxf(amax, fabsf(v));
            if (mn > v) mn = v;
            mx = fmaxf(mx, v);
        }
        if (symmetric) scales[g] = fmaxf(amax, 1e-12f) / 7.0f;
        else {
            float range = mx + mn * -1.0f;
            scales[g] = fmaxf(range, 1e-12f) / 15.0f;
            zeros[g] = (mn * -1.0f) / scales[g];
        }
    }
    for (size_t b = 0; b < (n + 1) / 2; b++) {
        uint32_t nib[2] = {0, 0};
        for (int j = 0; j < 2; j++) {
            size_t i = 2 * b + j;
            if (i >= n) continue;
            float s = x[i] / scales[i / group];
            float lo = symmetric ? -8.0f : 0.0f, hi = symmetric ? 7.0f : 15.0f;
            s = fmaxf(s, lo);
            if (s > hi) s = hi;
            if (symmetric) s = s + 8.0f;
            uint32_t q = (uint32_t)s;                    /* truncation; s is in [0, 15] */
            nib[j] = q > 15u ? 15u : q;
        }
        packed[b] = (uint8_t)(nib[0] | (nib[1] << 4));
    }
}

/* dequantize_int4 (int4_quantize.rs:780-826): symmetric (nibble + (-8)) * scale, asymmetric nibble * scale. */
void orc_ref_dnn_int4_dequant(const uint8_t* packed, const float* scales, size_t n, size_t group, int symmetric, float* out) {
    for (size_t i = 0; i < n; i++) {
        float nib = (float)((packed[i / 2] >> ((i & 1) * 4)) & 0x0F);
        out[i] = symmetric ? (nib + -8.0f) * scales[i / group] : nib * scales[i / group];
    }
}

/* quantize_block_scaled (crates/oxicuda-dnn/src/quantize/block_scale.rs:53-140), the arithmetic of its two generated
 * kernels: scale[b] = max(absmax_b / 6, 1e-12) (:243-249); out[i] = clamp(int(rint(min(max(x / scale, -6), 6))) + 6, 0, 255)
 * (:300-333; cvt.rni then cvt.rzi, bias FP4_MAX = 6).  The last block may be short. */
void orc_ref_dnn_block_scaled_quant(const float* x, size_t n, size_t block, uint8_t* out, float* scales) {
    size_t nb = (n + block - 1) / block;
    for (size_t b = 0; b < nb; b++) {
        size_t lo = b * block, hi = lo + block < n ? lo + block : n;
        float am = 0.0f;
        for (size_t i = lo; i < hi; i++) am = fmaxf(am, fabsf(x[i]));
        scales[b] = fmaxf(am / 6.0f, 1e-12f);
    }
    for (size_t i = 0; i < n; i++) {
        float s = x[i] / scales[i / block];
        s = fminf(fmaxf(s, -6.0f), 6.0f);
        int q = (int)rintf(s) + 6;
        out[i] = (uint8_t)(q < 0 ? 0 : (q > 255 ? 255 : q));
    }
}

/* Fp4BlockQuantizer::compute_scale (block_scale.rs:420-427): max|x| / 6, or 1 for an all-zero block. */
float orc_ref_fp4_block_compute_scale(const float* block, size_t n) {
    float mx = 0.0f;
    for (size_t i = 0; i < n; i++) mx = fmaxf(mx, fabsf(block[i]));
    return mx == 0.0f ? 1.0f : mx / 6.0f;
}

/* SmoothQuantMigrator (crates/oxicuda-quant/src/scheme/smooth_quant.rs).  compute_act_stats / compute_weight_stats
 * (:125-196): per-column maximum of |x| over the rows of a row-major [rows x cols] matrix. */
int orc_ref_smooth_col_absmax(const float* x, size_t rows, size_t cols, float* stats) {
    if (rows * cols == 0) return -1;
    for (size_t j = 0; j < cols; j++) stats[j] = 0.0f;
    for (size_t t = 0; t < rows; t++)
        for (size_t j = 0; j < cols; j++) {
            float v = fabsf(x[t * cols + j]);
            if (v > stats[j]) stats[j] = v;
        }
    return 0;
}

/* compute_migration_scales (:84-113): s_j = max(|a_j|, 1e-8)^alpha / max(|w_j|, 1e-8)^(1 - alpha). */
int orc_ref_smooth_scales(const float* act_max, const float* weight_max, size_t n, float alpha, float* scales) {
    if (n == 0) return -1;
    for (size_t j = 0; j < n; j++) {
        float a = fmaxf(fabsf(act_max[j]), 1e-8f), w = fmaxf(fabsf(weight_max[j]), 1e-8f);
        scales[j] = powf(a, alpha) / powf(w, 1.0f - alpha);
    }
    return 0;
}

/* smooth_activations (:198-222): x[t, j] /= max(s_j, 1e-12); smooth_weights (:231-254): w[r, j] *= s_j. */
void orc_ref_smooth_activations(float* x, const float* scales, size_t rows, size_t cols) {
    for (size_t t = 0; t < rows; t++)
        for (size_t j = 0; j < cols; j++) x[t * cols + j] /= fmaxf(scales[j], 1e-12f);
}
void orc_ref_smooth_weights(float* w, const float* scales, size_t rows, size_t cols) {
    for (size_t r = 0; r < rows; r++)
        for (size_t j = 0; j < cols; j++) w[r * cols + j] *= scales[j];
}

/* ------------------------------------------------------------------------- */
/* GPTQ (crates/oxicuda-quant/src/scheme/gptq.rs)                              */

/* cholesky_lower (gptq.rs:281-300): row by row, s = h[i][j] minus the products l[i][k] * l[j][k] in increasing k,
 * each product and each subtraction rounded on its own.  Returns 0, or 1 when a pivot is <= 0. */
int orc_ref_cholesky_lower(const float* h, size_t n, float* l) {
    memset(l, 0, n * n * sizeof(float));
    for (size_t i = 0; i < n; i++) {
        for (size_t j = 0; j <= i; j++) {
            float s = h[i * n + j];
            for (size_t k = 0; k < j; k++) s -= l[i * n + k] * l[j * n + k];
            if (i == j) {
                if (s <= 0.0f) return 1;
                l[i * n + i] = sqrtf(s);
            } else {
                l[i * n + j] = s / l[j * n + j];
            }
        }
    }
    return 0;
}

/* invert_lower (gptq.rs:305-318): forward substitution, s starts at 0 and adds l[i][k] * li[k][j] for k = j .. i-1. */
void orc_ref_invert_lower(const float* l, size_t n, float* li) {
    memset(li, 0, n * n * sizeof(float));
    for (size_t i = 0; i < n; i++) {
        li[i * n + i] = 1.0f / l[i * n + i];
        for (size_t j = 0; j < i; j++) {
            float s = 0.0f;
            for (size_t k = j; k < i; k++) s += l[i * n + k] * li[k * n + j];
            li[i * n + j] = -s / l[i * n + i];
        }
    }
}

/* hinv_row_starting (gptq.rs:328-332) for every j: hinv[j][k] = sum over m = k .. n-1 of li[m][j] * li[m][k], k >= j,
 * summed in increasing m.  Entries below the diagonal are left at zero. */
void orc_ref_hinv_upper(const float* li, size_t n, float* hinv) {
    memset(hinv, 0, n * n * sizeof(float));
    for (size_t j = 0; j < n; j++)
        for (size_t k = j; k < n; k++) {
            float s = 0.0f;
            for (size_t m = k; m < n; m++) s += li[m * n + j] * li[m * n + k];
            hinv[j * n + k] = s;
        }
}

static int32_t gptq_quant_scalar(float x, float scale, int32_t zp, int32_t q_min, int32_t q_max) {
    /* quant_scalar (gptq.rs:235-239) */
    return f32_as_i32(clampf(roundf(x / scale + (float)zp), (float)q_min, (float)q_max));
}

/* The column loop of GptqQuantizer::quantize_layer (gptq.rs:184-247) on a given upper-triangular H^-1: per-column
 * parameters from the current (already corrected) column (col_quant_params, gptq.rs:242-276), round to nearest,
 * error divided by the diagonal entry, and the correction of every later column, one rounded product and one rounded
 * subtraction per element.  `w` is overwritten with the corrected weights. */
void orc_ref_gptq_columns(float* w, size_t n_rows, size_t n_cols, const float* hinv, int bits, int symmetric,
                          int32_t* quantized, float* scales, int32_t* zero_points) {
    int32_t q_min, q_max;
    if (symmetric) { q_min = -(1 << (bits - 1)); q_max = (1 << (bits - 1)) - 1; }
    else { q_min = 0; q_max = (1 << bits) - 1; }
    float* errs = (float*)malloc(n_rows * sizeof(float));
    for (size_t j = 0; j < n_cols; j++) {
        float scale; int32_t zp = 0;
        if (symmetric) {
            float am = 0.0f;
            for (size_t i = 0; i < n_rows; i++) { float a = fabsf(w[i * n_cols + j]); if (a > am) am = a; }   /* f32::max skips NaN */
            if (!(am > 1e-8f)) am = 1e-8f;
            scale = am / (float)q_max;
        } else {
            float fmin = INFINITY, fmax = -INFINITY;
            for (size_t i = 0; i < n_rows; i++) { float v = w[i * n_cols + j]; if (v < fmin) fmin = v; if (v > fmax) fmax = v; }
            float range = fmax - fmin;
            if (!(range > 1e-8f)) range = 1e-8f;
            scale = range / (float)((1 << bits) - 1);
            zp = f32_as_i32(clampf(roundf(-fmin / scale), (float)q_min, (float)q_max));
        }
        scales[j] = scale; zero_points[j] = zp;
        const float hjj = hinv[j * n_cols + j];
        if (hjj < 1e-12f) {
            for (size_t i = 0; i < n_rows; i++) quantized[i * n_cols + j] = gptq_quant_scalar(w[i * n_cols + j], scale, zp, q_min, q_max);
            continue;
        }
        for (size_t i = 0; i < n_rows; i++) {
            const float wij = w[i * n_cols + j];
            const int32_t q = gptq_quant_scalar(wij, scale, zp, q_min, q_max);
            quantized[i * n_cols + j] = q;
            const float q_dq = ((float)q - (float)zp) * scale;
            errs[i] = (wij - q_dq) / hjj;
        }
        for (size_t k = j + 1; k < n_cols; k++) {
            const float hjk = hinv[j * n_cols + k];
            for (size_t i = 0; i < n_rows; i++) w[i * n_cols + k] -= errs[i] * hjk;
        }
    }
    free(errs);
}

/* GptqQuantizer::quantize_layer (gptq.rs:133-257).  Returns 0, 1 (EmptyInput), 6 (InvalidBitWidth) or 7
 * (SingularHessian, with *min_diag = the smallest dampened diagonal entry).  The length checks of the reference are
 * the caller's (the wrapper raises DimensionMismatch). */
int orc_ref_gptq_quantize_layer(const float* weights, size_t n_rows, size_t n_cols, const float* hessian, int bits, int symmetric,
                                double percdamp, int32_t* quantized, float* scales, int32_t* zero_points, float* min_diag) {
    if (n_rows * n_cols == 0) return ORC_ERR_EMPTY_INPUT;
    if (bits <= 0 || bits > 16) return ORC_ERR_INVALID_BITS;
    const size_t n = n_cols;
    float sum = 0.0f;
    for (size_t j = 0; j < n; j++) sum += hessian[j * n + j];
    const float mean_diag = sum / (float)n;
    float md = fabsf(mean_diag);
    if (!(md > 1e-8f)) md = 1e-8f;
    const float lambda = (float)percdamp * md;
    float* hd = (float*)malloc(n * n * sizeof(float));
    float* l = (float*)malloc(n * n * sizeof(float));
    float* li = (float*)malloc(n * n * sizeof(float));
    memcpy(hd, hessian, n * n * sizeof(float));
    for (size_t j = 0; j < n; j++) hd[j * n + j] += lambda;
    int rc = 0;
    if (orc_ref_cholesky_lower(hd, n, l)) {
        float m = INFINITY;
        for (size_t j = 0; j < n; j++) if (hd[j * n + j] < m) m = hd[j * n + j];
        if (min_diag) *min_diag = m;
        rc = 7;
    } else {
        orc_ref_invert_lower(l, n, li);
        orc_ref_hinv_upper(li, n, hd);
        float* w = (float*)malloc(n_rows * n_cols * sizeof(float));
        memcpy(w, weights, n_rows * n_cols * sizeof(float));
        orc_ref_gptq_columns(w, n_rows, n_cols, hd, bits, symmetric, quantized, scales, zero_points);
        free(w);
    }
    free(hd); free(l); free(li);
    return rc;
}

/* RmsNorm::forward (crates/oxicuda-lm/src/layer/norm.rs:73-95): per row, mean of squares summed left to right in
 * f32, inv_rms = 1 / sqrt(mean_sq + eps), out = x * inv_rms * weight (two multiplications, in that order). */
void orc_ref_rms_norm(const float* x, const float* weight, size_t rows, size_t dim, float eps, float* out) {
    for (size_t t = 0; t < rows; t++) {
        const float* row = x + t * dim;
        float sum = 0.0f;
        for (size_t i = 0; i < dim; i++) sum += row[i] * row[i];
        float mean_sq = sum / (float)dim;
        float inv_rms = 1.0f / sqrtf(mean_sq + eps);
        for (size_t i = 0; i < dim; i++) out[t * dim + i] = row[i] * inv_rms * weight[i];
    }
}

/* RmsNorm::forward with the sum of squares taken in the order of the fused device kernel instead of left to right:
 * the row is dealt out in items of 8 consecutive elements, thread t of 256 owns items t, t + 256, t + 512, ... and
 * chains them with fused multiply-adds; the 32 partial sums of a warp are combined by a butterfly (partner lanes
 * 16, 8, 4, 2, 1 apart, every lane adding its partner's value), then the 8 warp sums by a butterfly over 4, 2, 1.
 * Everything after the sum is the reference's arithmetic (crates/oxicuda-lm/src/layer/norm.rs:82-90).  Floating-point
 * addition is commutative, so the butterfly is the same expression on every lane.  dim is a multiple of 8. */
void orc_spec_rms_norm_blocked(const float* x, const float* weight, size_t rows, size_t dim, float eps, float* out) {
    size_t nitems = dim / 8;
    for (size_t t = 0; t < rows; t++) {
        const float* row = x + t * dim;
        float part[256];
        for (int th = 0; th < 256; th++) {
            float ss = 0.0f;
            for (size_t it = (size_t)th; it < nitems; it += 256)
                for (int e = 0; e < 8; e++) ss = fmaf(row[it * 8 + e], row[it * 8 + e], ss);
            part[th] = ss;
        }
        float wsum[8];
        for (int w = 0; w < 8; w++) {
            float v[32], n[32];
            for (int l = 0; l < 32; l++) v[l] = part[w * 32 + l];
            for (int o = 16; o > 0; o >>= 1) {
                for (int l = 0; l < 32; l++) n[l] = v[l] + v[l ^ o];
                for (int l = 0; l < 32; l++) v[l] = n[l];
            }
            wsum[w] = v[0];
        }
        for (int o = 4; o > 0; o >>= 1) {
            float n[8];
            for (int l = 0; l < 8; l++) n[l] = wsum[l] + wsum[l ^ o];
            for (int l = 0; l < 8; l++) wsum[l] = n[l];
        }
        float mean_sq = wsum[0] / (float)dim;
        float inv_rms = 1.0f / sqrtf(mean_sq + eps);
        for (size_t i = 0; i < dim; i++) out[t * dim + i] = row[i] * inv_rms * weight[i];
    }
}

/* ------------------------------------------------------------------------- */

/* Y[b,o] = bias[o] + sum_i X[b,i] * W[o,i], accumulated left to right in f32
 * (crates/oxicuda-dist-infer/src/tensor_parallel/column_parallel.rs:77-95;
 *  crates/oxicuda-lm/src/layer/ffn.rs:72-110 is the bias-free form).  `threads` <= 1 runs the
 * reference's single-threaded loop; otherwise rows of W are split over OpenMP threads (the
 * per-output summation order is unchanged, so results are identical). */
void orc_ref_linear_f32(const float* x, const float* w, const float* bias, size_t batch, size_t in_f, size_t out_f,
                        float* y, int threads) {
#ifdef _OPENMP
    int nt = threads <= 1 ? 1 : threads;
#pragma omp parallel for schedule(static) num_threads(nt)
#endif
    for (size_t o = 0; o < out_f; o++) {
        const float* wr = w + o * in_f;
        for (size_t b = 0; b < batch; b++) {
            float acc = bias ? bias[o] : 0.0f;
            const float* xr = x + b * in_f;
            for (size_t i = 0; i < in_f; i++) acc += xr[i] * wr[i];
            y[b * out_f + o] = acc;
        }
    }
}

/* silu(x) = x / (1 + exp(-x)), crates/oxicuda-lm/src/layer/ffn.rs:25-27;
 * h = silu(gate) * up, ffn.rs:245-249 */
void orc_ref_silu_mul(const float* gate, const float* up, size_t n, float* h) {
    for (size_t i = 0; i < n; i++) h[i] = (gate[i] / (1.0f + expf(-gate[i]))) * up[i];
}

/* RowLinear::all_reduce, crates/oxicuda-dist-infer/src/tensor_parallel/row_parallel.rs:202-223:
 * elementwise sum of the rank partials in rank order.  partials = [ranks][len] contiguous. */
void orc_ref_all_reduce_sum(const float* partials, size_t ranks, size_t len, float* out) {
    memcpy(out, partials, len * sizeof(float));
    for (size_t r = 1; r < ranks; r++)
        for (size_t i = 0; i < len; i++) out[i] += partials[r * len + i];
}

int orc_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
