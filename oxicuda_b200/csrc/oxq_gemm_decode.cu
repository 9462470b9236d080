// Decode-shaped (M <= 32) quantized GEMMs.  These are HBM-bound: the weight matrix is streamed once
// with 128-bit loads, unpacked in registers, and multiplied with mma.sync.
//
//   W4A16: uint4 codes -> bf16 in registers with the (0x4300 | nibble) trick, mma.sync m16n8k16 with the
//          weights as the row operand, per-group f32 scale and zero-point applied to the group's partial
//          sum.  Two kernels: w4a16_gemv_kernel (up to 8 batch rows: a CTA owns 16 weight rows over the
//          whole K, activations read from L1, nothing combined across CTAs) and w4a16_decode_kernel (up to
//          16 rows per pass, split along K across CTAs; partial sums are combined with f32 atomics in a
//          caller-provided workspace that the last CTA of each row block drains).
//   W8A32: int8 codes are exact in TF32, the f32 activations are split in two TF32 halves, mma.sync m16n8k8 (the
//          benchmark's CPU-runnable configuration).
#include "oxq_common.cuh"
#include <stdlib.h>

namespace oxq {
namespace decode {

// ------------------------------------------------------------------------------------------------
// W4A16
// ------------------------------------------------------------------------------------------------

constexpr int W4_ROWS_PER_CTA = 64;    // 4 warps x 16 weight rows
constexpr int W4_THREADS = 128;
constexpr int W4_SPANS = 4;            // 128-wide K spans per CTA (512 K)

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t sub_bf16x2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ uint4 ld_stream_u4(const void* p) {
    uint4 u;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(u.x), "=r"(u.y), "=r"(u.z), "=r"(u.w) : "l"(p));
    return u;
}

struct W4Params {
    int m, n, k, group;
    int kc;                      // K elements per split (multiple of 128, at most W4_SPANS * 128)
    int splits;
    const __nv_bfloat16* x;      // [m x k]
    const uint32_t* codes;       // [n x k/8]
    const uint16_t* scales;      // f16 [n x k/group]
    const uint32_t* zeros;       // packed, linear group order
    __nv_bfloat16* y;            // [m x n]
    float* ws;                   // [m x n] f32 partial sums, zero on entry and on exit
    int* counters;               // [ceil(n/64)], zero on entry and on exit
};

// NT = number of 8-wide batch tiles (M padded to 8*NT).  One CTA = 64 weight rows x one K chunk of up to
// SPANS spans of 128; many short CTAs, so load latency, the split-K combine and the grid tail overlap
// across the 8 or so CTAs an SM holds at once.
//
// The MMAs multiply the raw bf16 values 128 + code (0x4300 | nibble: one shift and one logic instruction per
// code pair); the zero-point and the 128 come out afterwards through the per-span sum of the activations:
//   sum_k (c_k - z) x_k = sum_k (128 + c_k) x_k - (128 + z) * sum_k x_k
// (the f32 accumulator carries about 5 bits more magnitude than the result, invisible at bf16 output).
// K order inside one MMA is free as long as both operands agree, so word i of a thread's 16-byte load
// (8 consecutive K) feeds MMAs 2i and 2i+1 directly, and the activation chunk is stored in shared memory
// already permuted to match.
template <int NT, int SPANS>
__global__ void __launch_bounds__(W4_THREADS) w4a16_decode_kernel(const W4Params p) {
    pdl_trigger();
    pdl_wait();
    __shared__ uint4 xs[SPANS * 4 * NT * 32];           // [span][word][nt][lane]: B fragments of two MMAs
    __shared__ float xsum[SPANS][NT * 8];               // [span][batch row]: sum of the activations
    __shared__ int s_last;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int split = blockIdx.y;
    const int k0 = split * p.kc;
    const int k1 = min(p.k, k0 + p.kc);
    const int spans = (k1 - k0) >> 7;

    // ---- request every weight byte and group parameter of this thread up front ---------------
    const int row_a = blockIdx.x * W4_ROWS_PER_CTA + warp * 16 + g, row_b = row_a + 8;
    const bool va = row_a < p.n, vb = row_b < p.n;
    const int wpr = p.k >> 3, gpr = p.k / p.group;
    const uint32_t* ca = p.codes + (size_t)(va ? row_a : 0) * wpr + ((k0 + 32 * t) >> 3);
    const uint32_t* cb = p.codes + (size_t)(vb ? row_b : 0) * wpr + ((k0 + 32 * t) >> 3);
    uint4 wa[SPANS], wb[SPANS];
    uint32_t sca[SPANS], scb[SPANS], zwa[SPANS], zwb[SPANS];
#pragma unroll
    for (int s = 0; s < SPANS; s++) {
        wa[s] = make_uint4(0, 0, 0, 0); wb[s] = wa[s];
        sca[s] = 0; scb[s] = 0; zwa[s] = 0; zwb[s] = 0;
        if (s < spans) {
            const int kg = (k0 + s * 128) / p.group;
            if (va) {
                wa[s] = ld_stream_u4(ca + s * 16);
                const int gi = row_a * gpr + kg;
                sca[s] = __ldg(p.scales + gi);
                zwa[s] = (__ldg(p.zeros + (gi >> 3)) >> ((gi & 7) * 4)) & 0xFu;
            }
            if (vb) {
                wb[s] = ld_stream_u4(cb + s * 16);
                const int gi = row_b * gpr + kg;
                scb[s] = __ldg(p.scales + gi);
                zwb[s] = (__ldg(p.zeros + (gi >> 3)) >> ((gi & 7) * 4)) & 0xFu;
            }
        }
    }

    // ---- stage the activation chunk, permuted into B-fragment order ---------------------------
    // One item = 8 consecutive K of one batch row = the K of one weight word.  For K offset o inside the chunk:
    // span = o/128, t' = (o%128)/32, word i = (o%32)/8; u32 q of the uint4 holds (x[q], x[q+4]).  The 16 items of
    // one (batch row, span) sit in 16 consecutive lanes, which also add up the span's sum.  Rows beyond m are zero.
    if (p.m < NT * 8) {
        for (int idx = tid; idx < SPANS * 4 * NT * 32; idx += W4_THREADS) xs[idx] = make_uint4(0, 0, 0, 0);
        for (int idx = tid; idx < SPANS * NT * 8; idx += W4_THREADS) (&xsum[0][0])[idx] = 0.0f;
        __syncthreads();
    }
    const int items = p.m * (spans * 16);
    for (int it0 = 0; it0 < items; it0 += W4_THREADS) {
        const int it = it0 + tid;
        const bool live = it < items;
        const int mrow = live ? it / (spans * 16) : 0, o8 = live ? it - mrow * (spans * 16) : 0;
        const int span = o8 >> 4, tt = (o8 >> 2) & 3, i = o8 & 3;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (live) v = __ldg(reinterpret_cast<const uint4*>(p.x + (size_t)mrow * p.k + k0 + o8 * 8));
        const uint32_t lo[4] = {v.x & 0xFFFFu, v.x >> 16, v.y & 0xFFFFu, v.y >> 16};
        const uint32_t hi[4] = {v.z & 0xFFFFu, v.z >> 16, v.w & 0xFFFFu, v.w >> 16};
        float sum = 0.0f;
#pragma unroll
        for (int q = 0; q < 4; q++) sum += __uint_as_float(lo[q] << 16) + __uint_as_float(hi[q] << 16);
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if (live) {
            uint4 o;
            o.x = lo[0] | (hi[0] << 16); o.y = lo[1] | (hi[1] << 16); o.z = lo[2] | (hi[2] << 16); o.w = lo[3] | (hi[3] << 16);
            const int nt = mrow >> 3, gg = mrow & 7;
            xs[((span * 4 + i) * NT + nt) * 32 + gg * 4 + tt] = o;
            if ((o8 & 15) == 0) xsum[span][mrow] = sum;
        }
    }
    __syncthreads();

    // ---- multiply -----------------------------------------------------------------------------------
    float total[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) { total[nt][0] = total[nt][1] = total[nt][2] = total[nt][3] = 0.0f; }
#pragma unroll
    for (int s = 0; s < SPANS; s++) {
        if (s < spans) {
            float part[NT][4];
#pragma unroll
            for (int nt = 0; nt < NT; nt++) { part[nt][0] = part[nt][1] = part[nt][2] = part[nt][3] = 0.0f; }
            const uint32_t wwa[4] = {wa[s].x, wa[s].y, wa[s].z, wa[s].w}, wwb[4] = {wb[s].x, wb[s].y, wb[s].z, wb[s].w};
#pragma unroll
            for (int i = 0; i < 4; i++) {
                uint32_t ra[4], rb4[4];
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    ra[q] = ((wwa[i] >> (4 * q)) & 0x000F000Fu) | 0x43004300u;           // bf16x2 (128 + c, 128 + c')
                    rb4[q] = ((wwb[i] >> (4 * q)) & 0x000F000Fu) | 0x43004300u;
                }
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    const uint4 b = xs[((s * 4 + i) * NT + nt) * 32 + lane];
                    mma_bf16_16816(part[nt], ra[0], rb4[0], ra[1], rb4[1], b.x, b.y);
                    mma_bf16_16816(part[nt], ra[2], rb4[2], ra[3], rb4[3], b.z, b.w);
                }
            }
            const float sa = __half2float(__ushort_as_half((unsigned short)sca[s])), sb = __half2float(__ushort_as_half((unsigned short)scb[s]));
            const float zca = -sa * (128.0f + (float)zwa[s]), zcb = -sb * (128.0f + (float)zwb[s]);   // -(128 + z) * scale
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                const float2 xsm = *reinterpret_cast<const float2*>(&xsum[s][nt * 8 + 2 * t]);
                total[nt][0] += fmaf(sa, part[nt][0], zca * xsm.x);
                total[nt][1] += fmaf(sa, part[nt][1], zca * xsm.y);
                total[nt][2] += fmaf(sb, part[nt][2], zcb * xsm.x);
                total[nt][3] += fmaf(sb, part[nt][3], zcb * xsm.y);
            }
        }
    }

    // ---- combine --------------------------------------------------------------------------------
    // accumulator element e of tile nt: weight row (e < 2 ? row_a : row_b), batch row nt*8 + 2t + (e & 1)
    if (p.splits == 1) {
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int mrow = nt * 8 + 2 * t + (e & 1), nrow = e < 2 ? row_a : row_b;
                if (mrow < p.m && nrow < p.n) p.y[(size_t)mrow * p.n + nrow] = __float2bfloat16_rn(total[nt][e]);
            }
        return;
    }
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int mrow = nt * 8 + 2 * t + (e & 1), nrow = e < 2 ? row_a : row_b;
            if (mrow < p.m && nrow < p.n) atomicAdd(p.ws + (size_t)mrow * p.n + nrow, total[nt][e]);
        }
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = atomicAdd(p.counters + blockIdx.x, 1) == p.splits - 1;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // last CTA of this row block: convert the sums and leave the workspace zeroed for the next call
    const int n_lo = blockIdx.x * W4_ROWS_PER_CTA;
    const int ncols = min(W4_ROWS_PER_CTA, p.n - n_lo);
    for (int idx = tid; idx < p.m * ncols; idx += W4_THREADS) {
        const int mrow = idx / ncols, c = idx - mrow * ncols;
        float* w = p.ws + (size_t)mrow * p.n + n_lo + c;
        p.y[(size_t)mrow * p.n + n_lo + c] = __float2bfloat16_rn(__ldcg(w));
        __stcg(w, 0.0f);
    }
    if (tid == 0) p.counters[blockIdx.x] = 0;
}

// ------------------------------------------------------------------------------------------------
// W4A16, up to 8 batch rows, no split across CTAs
// ------------------------------------------------------------------------------------------------
//
// A CTA owns 16 weight rows over the whole K range; its GV_WARPS warps split K among themselves and meet once
// in shared memory at the end, so there are no global atomics, no workspace and no second pass.  Inside a warp
// nothing is shared: lane (g, t) streams rows g and g + 8 (16 bytes = 32 codes per load, chunks of four spans
// of 128 K, the next chunk requested before the current one is multiplied), reads the matching 8 activations of
// batch row g straight from global memory (they stay in L1) and permutes them in registers into the K order of
// the unpacked codes.  0x4300 | nibble is the bf16 value 128 + code; a packed subtraction of 128 + z leaves the exact
// integer code - z in both halves, so the MMAs multiply the dequantised integers and only the group's scale is left.
constexpr int GV_WARPS = 8;
constexpr int GV_CHUNK = 4;            // spans per register buffer (the vector scale loads assume 4)

// a load the compiler keeps where it is written
__device__ __forceinline__ uint4 ld_pinned_u4(const void* p) {
    uint4 u;
    asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(u.x), "=r"(u.y), "=r"(u.z), "=r"(u.w) : "l"(p) : "memory");
    return u;
}

struct GvParams {
    int m, n, k, group;
    const __nv_bfloat16* x;      // [m x k]
    const uint32_t* codes;       // [n x k/8]
    const uint16_t* scales;      // f16 [n x k/group]
    const uint32_t* zeros;       // packed, linear group order
    __nv_bfloat16* y;            // [m x n]
    int scales_vec_ok;           // the scales pointer is 8-byte aligned, so four f16 scales may be read with one load
};

// PIPE: the warp's K range is longer than one chunk, so a second register buffer holds the next chunk's requests.
template <bool PIPE>
__global__ void __launch_bounds__(GV_WARPS * 32, 2) w4a16_gemv_kernel(const GvParams p) {
    __shared__ float red[GV_WARPS][16][8];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int spans = p.k >> 7;
    const int s_lo = (int)(((int64_t)warp * spans) / GV_WARPS), s_hi = (int)(((int64_t)(warp + 1) * spans) / GV_WARPS);
    const int row_a = min((int)blockIdx.x * 16 + g, p.n - 1), row_b = min((int)blockIdx.x * 16 + g + 8, p.n - 1);
    const int wpr = p.k >> 3, gpr = p.k / p.group;
    const uint32_t* ca = p.codes + (size_t)row_a * wpr + 4 * t;
    const uint32_t* cb = p.codes + (size_t)row_b * wpr + 4 * t;
    const bool has_x = g < p.m;
    const __nv_bfloat16* xr = p.x + (size_t)(has_x ? g : 0) * p.k + 32 * t;

    uint4 cur_a[GV_CHUNK], cur_b[GV_CHUNK], nxt_a[GV_CHUNK], nxt_b[GV_CHUNK];
    uint32_t cur_sa[GV_CHUNK], cur_sb[GV_CHUNK], nxt_sa[GV_CHUNK], nxt_sb[GV_CHUNK];     // f16 scale | zero-point << 16

    // With group 128, a chunk that starts at a multiple of four groups and whole rows of scales that are 8-byte aligned,
    // the chunk's four scales of a row are one 8-byte load and its zero-points sit in one word.
    const bool vec_meta = p.scales_vec_ok && p.group == 128 && (gpr & 7) == 0 && ((s_lo & 3) == 0) && (((s_hi - s_lo) & 3) == 0);

    auto fetch = [&](int s0, uint4 (&wa)[GV_CHUNK], uint4 (&wb)[GV_CHUNK], uint32_t (&sa)[GV_CHUNK], uint32_t (&sb)[GV_CHUNK]) {
#pragma unroll
        for (int j = 0; j < GV_CHUNK; j++) {
            const int s = s0 + j;
            wa[j] = make_uint4(0, 0, 0, 0); wb[j] = wa[j]; sa[j] = 0; sb[j] = 0;      // scale 0: the span contributes nothing
            if (s < s_hi) {
                wa[j] = ld_stream_u4(ca + s * 16);
                wb[j] = ld_stream_u4(cb + s * 16);
            }
        }
        if (vec_meta) {
            const int gia = row_a * gpr + s0, gib = row_b * gpr + s0;
            const uint2 qa = __ldg(reinterpret_cast<const uint2*>(p.scales + gia)), qb = __ldg(reinterpret_cast<const uint2*>(p.scales + gib));
            const uint32_t za = __ldg(p.zeros + (gia >> 3)) >> ((gia & 7) * 4), zb = __ldg(p.zeros + (gib >> 3)) >> ((gib & 7) * 4);
            sa[0] = (qa.x & 0xFFFFu) | ((za & 0xFu) << 16);         sb[0] = (qb.x & 0xFFFFu) | ((zb & 0xFu) << 16);
            sa[1] = (qa.x >> 16) | (((za >> 4) & 0xFu) << 16);      sb[1] = (qb.x >> 16) | (((zb >> 4) & 0xFu) << 16);
            sa[2] = (qa.y & 0xFFFFu) | (((za >> 8) & 0xFu) << 16);  sb[2] = (qb.y & 0xFFFFu) | (((zb >> 8) & 0xFu) << 16);
            sa[3] = (qa.y >> 16) | (((za >> 12) & 0xFu) << 16);     sb[3] = (qb.y >> 16) | (((zb >> 12) & 0xFu) << 16);
        } else {
#pragma unroll
            for (int j = 0; j < GV_CHUNK; j++) {
                const int s = s0 + j;
                if (s < s_hi) {
                    const int kg = (s << 7) / p.group;
                    const int gia = row_a * gpr + kg, gib = row_b * gpr + kg;
                    sa[j] = (uint32_t)__ldg(p.scales + gia) | (((__ldg(p.zeros + (gia >> 3)) >> ((gia & 7) * 4)) & 0xFu) << 16);
                    sb[j] = (uint32_t)__ldg(p.scales + gib) | (((__ldg(p.zeros + (gib >> 3)) >> ((gib & 7) * 4)) & 0xFu) << 16);
                }
            }
        }
    };

    float total[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    // Before the kernel ahead of this one in the stream has finished, the first codes are only prefetched into the L2
    // (it may be the quantizer that writes them); codes, scales and zero-points are read after the wait.
    pdl_trigger();
#pragma unroll
    for (int j = 0; j < GV_CHUNK; j++) {
        const int s = s_lo + j;
        if (s < s_hi) { prefetch_l2(ca + s * 16); prefetch_l2(cb + s * 16); }
    }
    pdl_wait();
    if (s_lo < s_hi) fetch(s_lo, cur_a, cur_b, cur_sa, cur_sb);
    for (int s0 = s_lo; s0 < s_hi; s0 += GV_CHUNK) {
        if (PIPE && s0 + GV_CHUNK < s_hi) fetch(s0 + GV_CHUNK, nxt_a, nxt_b, nxt_sa, nxt_sb);
#pragma unroll
        for (int j = 0; j < GV_CHUNK; j++) {
            const int s = s0 + j;
            if (s < s_hi) {
                float part[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                const uint32_t wwa[4] = {cur_a[j].x, cur_a[j].y, cur_a[j].z, cur_a[j].w}, wwb[4] = {cur_b[j].x, cur_b[j].y, cur_b[j].z, cur_b[j].w};
                // bf16x2 (128 + z): one packed subtraction per code pair takes the 128 and the zero-point out, exactly (all
                // values are small integers).  The legacy tensor path is the scarce unit of this kernel on sm_100 -- an
                // m16n8k16 occupies it for 8 cycles per SM -- so the sums of the activations are not formed by extra MMAs.
                const uint32_t za = cur_sa[j] >> 16, zb = cur_sb[j] >> 16;
                const uint32_t zz_a = 0x43004300u | za | (za << 16), zz_b = 0x43004300u | zb | (zb << 16);
                // the span's 32 activations of batch row g (L1-resident), requested here and not earlier: hoisting the
                // requests of all spans to the top would cost 64 registers
                const uint4* xp = reinterpret_cast<const uint4*>(xr + (size_t)s * 128);
                uint4 xv[4];
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    xv[i] = make_uint4(0, 0, 0, 0);
                    if (has_x) xv[i] = ld_pinned_u4(xp + i);
                }
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    // 8 consecutive activations, reordered to (x0,x4) (x1,x5) (x2,x6) (x3,x7)
                    const uint4 v = xv[i];
                    const uint32_t b0 = __byte_perm(v.x, v.z, 0x5410), b1 = __byte_perm(v.x, v.z, 0x7632);
                    const uint32_t b2 = __byte_perm(v.y, v.w, 0x5410), b3 = __byte_perm(v.y, v.w, 0x7632);
                    uint32_t ra[4], rb4[4];
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        ra[q] = sub_bf16x2(((wwa[i] >> (4 * q)) & 0x000F000Fu) | 0x43004300u, zz_a);   // bf16x2 (c - z, c' - z)
                        rb4[q] = sub_bf16x2(((wwb[i] >> (4 * q)) & 0x000F000Fu) | 0x43004300u, zz_b);
                    }
                    mma_bf16_16816(part, ra[0], rb4[0], ra[1], rb4[1], b0, b1);
                    mma_bf16_16816(part, ra[2], rb4[2], ra[3], rb4[3], b2, b3);
                }
                const float sa = __half2float(__ushort_as_half((unsigned short)(cur_sa[j] & 0xFFFFu)));
                const float sb = __half2float(__ushort_as_half((unsigned short)(cur_sb[j] & 0xFFFFu)));
                total[0] = fmaf(sa, part[0], total[0]);
                total[1] = fmaf(sa, part[1], total[1]);
                total[2] = fmaf(sb, part[2], total[2]);
                total[3] = fmaf(sb, part[3], total[3]);
            }
        }
        if (PIPE) {
#pragma unroll
            for (int j = 0; j < GV_CHUNK; j++) { cur_a[j] = nxt_a[j]; cur_b[j] = nxt_b[j]; cur_sa[j] = nxt_sa[j]; cur_sb[j] = nxt_sb[j]; }
        }
    }
    // accumulator element e: weight row (e < 2 ? g : g + 8), batch row 2t + (e & 1)
    red[warp][g][2 * t] = total[0]; red[warp][g][2 * t + 1] = total[1];
    red[warp][g + 8][2 * t] = total[2]; red[warp][g + 8][2 * t + 1] = total[3];
    __syncthreads();
    if (threadIdx.x < 128) {
        const int col = threadIdx.x >> 4, r = threadIdx.x & 15;                             // consecutive threads -> consecutive rows of y
        const int row = (int)blockIdx.x * 16 + r;
        float acc = 0.0f;
#pragma unroll
        for (int w = 0; w < GV_WARPS; w++) acc += red[w][r][col];
        if (col < p.m && row < p.n) p.y[(size_t)col * p.n + row] = __float2bfloat16_rn(acc);
    }
}

// ------------------------------------------------------------------------------------------------
// W8A32
// ------------------------------------------------------------------------------------------------

// four int8 codes of a word -> f32: the byte (xor 0x80, an unsigned 0..255) becomes the low mantissa byte of
// 2^23, and 2^23 + 128 is subtracted; exact, and on the FMA pipe instead of the conversion unit
__device__ __forceinline__ void i8x4_to_f32(uint32_t u, float (&f)[4]) {
    const uint32_t v = u ^ 0x80808080u;
    f[0] = __uint_as_float(__byte_perm(v, 0x4B000000u, 0x7540)) - 8388736.0f;
    f[1] = __uint_as_float(__byte_perm(v, 0x4B000000u, 0x7541)) - 8388736.0f;
    f[2] = __uint_as_float(__byte_perm(v, 0x4B000000u, 0x7542)) - 8388736.0f;
    f[3] = __uint_as_float(__byte_perm(v, 0x4B000000u, 0x7543)) - 8388736.0f;
}

// The shape of the W4A16 GEMV with f32 activations: a CTA owns 16 weight rows over the whole K range for 8 batch
// rows (or 16 / 32: the converted weights are shared), its warps split K in spans of 64 and meet once in shared memory.  Lane (g, t) streams 16 codes of rows g and
// g + 8 per span and the 16 matching activations of batch row g.  An int8 code is exact in TF32 (10 mantissa bits);
// an f32 activation is split into x_hi = tf32(x) and x_lo = tf32(x - x_hi), so two m16n8k8 TF32 MMAs give the product
// to about 2^-21 relative with f32 accumulation (an f32 FMA loop spends eight FMAs per weight on 8 batch rows).
constexpr int W8T_WARPS = 8;
constexpr int W8T_CHUNK = 4;           // 64-wide spans per register buffer

__device__ __forceinline__ void mma_tf32_1688(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t to_tf32(float v) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
    return r;
}

// NT: tiles of 8 batch rows handled by one CTA (the converted weights are shared by the tiles)
template <int NT>
__global__ void __launch_bounds__(W8T_WARPS * 32, 2) w8a32_tc_kernel(const float* __restrict__ x, const int8_t* __restrict__ w,
                                                                     const float* __restrict__ sw, float* __restrict__ y,
                                                                     int m, int n, int k) {
    __shared__ float red[W8T_WARPS][16][8 * NT];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int m0 = blockIdx.y * 8 * NT;
    const int spans = (k + 63) >> 6;
    const int s_lo = (int)(((int64_t)warp * spans) / W8T_WARPS), s_hi = (int)(((int64_t)(warp + 1) * spans) / W8T_WARPS);
    const int row_a = min((int)blockIdx.x * 16 + g, n - 1), row_b = min((int)blockIdx.x * 16 + g + 8, n - 1);
    const int8_t* pa = w + (size_t)row_a * k + 16 * t;
    const int8_t* pb = w + (size_t)row_b * k + 16 * t;

    uint4 cur_a[W8T_CHUNK], cur_b[W8T_CHUNK], nxt_a[W8T_CHUNK], nxt_b[W8T_CHUNK];
    auto fetch = [&](int s0, uint4 (&wa)[W8T_CHUNK], uint4 (&wb)[W8T_CHUNK]) {
#pragma unroll
        for (int j = 0; j < W8T_CHUNK; j++) {
            const int s = s0 + j;
            // codes of zero contribute nothing: a span past the warp's range, or the ragged end of K (k is a multiple of 16)
            wa[j] = make_uint4(0, 0, 0, 0); wb[j] = wa[j];
            if (s < s_hi && s * 64 + 16 * t < k) {
                wa[j] = ld_stream_u4(pa + (size_t)s * 64);
                wb[j] = ld_stream_u4(pb + (size_t)s * 64);
            }
        }
    };
    float acc[NT][4];
#pragma unroll
    for (int i = 0; i < NT; i++) { acc[i][0] = 0.0f; acc[i][1] = 0.0f; acc[i][2] = 0.0f; acc[i][3] = 0.0f; }
    // Before the kernel ahead of this one in the stream has finished, the first weights are only prefetched into the L2
    // (it may be the quantizer that writes them); they are read after the wait.
    pdl_trigger();
#pragma unroll
    for (int j = 0; j < W8T_CHUNK; j++) {
        const int s = s_lo + j;
        if (s < s_hi && s * 64 + 16 * t < k) { prefetch_l2(pa + (size_t)s * 64); prefetch_l2(pb + (size_t)s * 64); }
    }
    pdl_wait();
    if (s_lo < s_hi) fetch(s_lo, cur_a, cur_b);
    for (int s0 = s_lo; s0 < s_hi; s0 += W8T_CHUNK) {
        if (s0 + W8T_CHUNK < s_hi) fetch(s0 + W8T_CHUNK, nxt_a, nxt_b);
#pragma unroll
        for (int j = 0; j < W8T_CHUNK; j++) {
            const int s = s0 + j;
            if (s < s_hi) {
                const bool in_k = s * 64 + 16 * t < k;
                const uint32_t wwa[4] = {cur_a[j].x, cur_a[j].y, cur_a[j].z, cur_a[j].w}, wwb[4] = {cur_b[j].x, cur_b[j].y, cur_b[j].z, cur_b[j].w};
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    float fa[4], fb[4];
                    i8x4_to_f32(wwa[q], fa);
                    i8x4_to_f32(wwb[q], fb);
#pragma unroll
                    for (int i = 0; i < NT; i++) {
                        const int mrow = m0 + 8 * i + g;
                        float4 xv = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                        if (in_k && mrow < m) xv = __ldg(reinterpret_cast<const float4*>(x + (size_t)mrow * k + (size_t)s * 64 + 16 * t) + q);
                        const float xf[4] = {xv.x, xv.y, xv.z, xv.w};
                        uint32_t hi[4], lo[4];
#pragma unroll
                        for (int e = 0; e < 4; e++) { hi[e] = to_tf32(xf[e]); lo[e] = to_tf32(xf[e] - __uint_as_float(hi[e])); }
                        // code 4q + e of the lane meets activation 4q + e: k slots (t, t + 4) of one MMA take e = (0, 1), then (2, 3)
                        mma_tf32_1688(acc[i], __float_as_uint(fa[0]), __float_as_uint(fb[0]), __float_as_uint(fa[1]), __float_as_uint(fb[1]), hi[0], hi[1]);
                        mma_tf32_1688(acc[i], __float_as_uint(fa[0]), __float_as_uint(fb[0]), __float_as_uint(fa[1]), __float_as_uint(fb[1]), lo[0], lo[1]);
                        mma_tf32_1688(acc[i], __float_as_uint(fa[2]), __float_as_uint(fb[2]), __float_as_uint(fa[3]), __float_as_uint(fb[3]), hi[2], hi[3]);
                        mma_tf32_1688(acc[i], __float_as_uint(fa[2]), __float_as_uint(fb[2]), __float_as_uint(fa[3]), __float_as_uint(fb[3]), lo[2], lo[3]);
                    }
                }
            }
        }
#pragma unroll
        for (int j = 0; j < W8T_CHUNK; j++) { cur_a[j] = nxt_a[j]; cur_b[j] = nxt_b[j]; }
    }
    // accumulator element e of tile i: weight row (e < 2 ? g : g + 8), batch row 8i + 2t + (e & 1)
#pragma unroll
    for (int i = 0; i < NT; i++) {
        red[warp][g][8 * i + 2 * t] = acc[i][0]; red[warp][g][8 * i + 2 * t + 1] = acc[i][1];
        red[warp][g + 8][8 * i + 2 * t] = acc[i][2]; red[warp][g + 8][8 * i + 2 * t + 1] = acc[i][3];
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < 16 * 8 * NT; idx += W8T_WARPS * 32) {
        const int col = idx >> 4, r = idx & 15;                            // consecutive threads -> consecutive rows of y
        const int row = (int)blockIdx.x * 16 + r;
        float v = 0.0f;
#pragma unroll
        for (int wi = 0; wi < W8T_WARPS; wi++) v += red[wi][r][col];
        if (m0 + col < m && row < n) y[(size_t)(m0 + col) * n + row] = v * __ldg(sw + row);
    }
}

}  // namespace decode
}  // namespace oxq

using namespace oxq::decode;

// f32 partial sums of the split-K kernels: [m x n], rounded up to 256 bytes
static size_t split_sums_bytes(int64_t m, int64_t n) { return ((size_t)m * (size_t)n * sizeof(float) + 255) & ~(size_t)255; }
// workspace of the mma.sync kernel: the sums, then one counter per W4_ROWS_PER_CTA weight rows
static size_t mma_sync_ws_bytes(int64_t m, int64_t n) {
    return split_sums_bytes(m, n) + ((((size_t)(n + oxq::decode::W4_ROWS_PER_CTA - 1) / oxq::decode::W4_ROWS_PER_CTA) * sizeof(int) + 255) & ~(size_t)255);
}

// workspace of the tensor-core kernel: 32 f32 per weight row and pass of 32 batch rows, then one counter per 32 weight rows
static size_t w4tc_sums_bytes(int64_t m, int64_t n) { return (size_t)((m + 31) / 32) * (size_t)n * 32 * sizeof(float); }
static size_t w4tc_ws_bytes(int64_t m, int64_t n) {
    return w4tc_sums_bytes(m, n) + ((((size_t)(n + 31) / 32) * sizeof(int) + 255) & ~(size_t)255);
}

// defined in oxq_gemm_w4tc.cu
bool oxq_w4tc_supports(int64_t m, int64_t n, int64_t k, int group);
int32_t oxq_w4tc_launch(oxq_handle* h, int64_t m, int64_t n, int64_t k, const void* x, const uint32_t* codes, const uint16_t* scales,
                        const uint32_t* zeros, void* y, float* ws_sums, int* ws_counters);

static int32_t w4a16_impl(oxq_handle* h, int64_t m, int64_t n, int64_t k, const void* x, const uint32_t* codes, const uint16_t* scales,
                          const uint32_t* zeros, int group, void* y, void* ws, size_t ws_bytes, int mode);

extern "C" {

// Layout of the caller's workspace: [sums and counters of the decode kernels: zero between calls][bf16 copy of the
// dequantised weight (m > 32 only)].  The second part starts behind the largest decode region (64 batch rows), so a
// prefill call never dirties what a later decode call on the same workspace expects to find zeroed.
static size_t w4_clean_bytes(int64_t n) { return w4tc_ws_bytes(64, n); }

size_t oxq_gemm_w4a16_workspace_bytes(int64_t m, int64_t n, int64_t k) {
    if (m <= 0 || n <= 0) return 0;
    if (m > 32) return w4_clean_bytes(n) + ((((size_t)n * (size_t)k * 2) + 255) & ~(size_t)255);
    return w4tc_ws_bytes(m, n);                                                  // covers the mma.sync kernel's needs as well
}

int32_t oxq_gemm_w4a16(oxq_handle* h, int64_t m, int64_t n, int64_t k, const void* x, const uint32_t* codes, const uint16_t* scales,
                       const uint32_t* zeros, int group, void* y, void* ws, size_t ws_bytes) {
    // Measured on B200 (14336 x 4096): up to 8 batch rows the mma.sync kernels win (16-17 us against 21; the one
    // without a split across CTAs is as fast as the split-K one at one row, faster from two rows and on small
    // matrices: 6.2 against 7.6 us at 4096 x 4096), the tensor-core kernel from there on (22-23 us per pass of 32
    // rows against 30-61), and from 65 rows the dequantise-then-GEMM path (70 us whatever the batch) beats three or
    // more passes.  OXQ_W4A16_TC=0 uses neither of the two newer kernels, 2 uses the tensor-core kernel for every
    // batch it supports (for A/B runs).
    static int tc = -1;
    if (tc < 0) { const char* e = getenv("OXQ_W4A16_TC"); tc = e ? atoi(e) : 1; }
    return w4a16_impl(h, m, n, k, x, codes, scales, zeros, group, y, ws, ws_bytes, tc < 0 ? 0 : (tc > 2 ? 2 : tc));
}

}  // extern "C"

// OXQ_W4A16_GEMV=0 keeps batches of up to 8 rows on the split-K mma.sync kernel (for A/B runs)
static bool gemv_setting() {
    static int v = -1;
    if (v < 0) { const char* e = getenv("OXQ_W4A16_GEMV"); v = e ? (atoi(e) != 0) : 1; }
    return v != 0;
}

static int32_t w4a16_impl(oxq_handle* h, int64_t m, int64_t n, int64_t k, const void* x, const uint32_t* codes, const uint16_t* scales,
                          const uint32_t* zeros, int group, void* y, void* ws, size_t ws_bytes, int mode) {
    OXQ_CHECK_HANDLE(h);
    if (m <= 0 || n <= 0 || k <= 0) OXQ_FAIL(h, OXQ_ERR_INVALID_DIMENSION, "GEMM dimensions must be non-zero");
    if (!x || !codes || !scales || !zeros || !y) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null pointer");
    // Int4GemmConfig::validate: K % 8 == 0, group in {32,64,128,256} (crates/oxicuda-blas/src/precision/int_ops.rs:250-281)
    if (k % 8 != 0) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "K must be a multiple of 8 for INT4 packing, got %lld", (long long)k);
    if (!(group == 32 || group == 64 || group == 128 || group == 256)) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "group size %d not in {32,64,128,256}", group);
    if (k % group != 0) OXQ_FAIL(h, OXQ_ERR_GROUP_SIZE_MISMATCH, "k %lld is not divisible by group size %d", (long long)k, group);
    // mode 0: split-K mma.sync and dequantise-then-GEMM only (the allocation-free entry point); 1: by batch size; 2: the
    // fused tensor-core kernel wherever it applies
    const bool tc_ok = oxq_w4tc_supports(m, n, k, group);
    if ((mode == 2 && tc_ok) || (mode == 1 && tc_ok && m > 8 && m <= 64)) {
        // Tensor-core kernel with the dequantisation fused in: one pass over the weights per 32 batch rows.
        if (((uintptr_t)x & 15u) || ((uintptr_t)codes & 15u) || ((uintptr_t)scales & 15u)) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "x, codes and scales must be 16-byte aligned");
        if (int32_t rc = oxq_require_sm100(h)) return rc;
        const size_t sums = w4tc_sums_bytes(m, n);
        const size_t need = w4tc_ws_bytes(m, n);
        if (!ws || ws_bytes < need || ((uintptr_t)ws & 255u))
            OXQ_FAIL(h, OXQ_ERR_BUFFER_TOO_SMALL, "workspace: expected at least %zu bytes (256-byte aligned), got %zu", need, ws_bytes);
        // up to 32 rows the workspace is zero on entry by contract; a caller that only ever runs more rows never had to clear it
        if (m > 32) OXQ_CUDA(h, cudaMemsetAsync(ws, 0, need, h->stream));
        return oxq_w4tc_launch(h, m, n, k, x, codes, scales, zeros, y, (float*)ws, (int*)((char*)ws + sums));
    }
    if (m > 32) {
        // Prefill shapes are tensor-bound: dequantise the weight once to bf16 in the workspace (which needs
        // no zero fill on this path), then run the bf16 tensor-core GEMM.
        const size_t need = oxq_gemm_w4a16_workspace_bytes(m, n, k);
        if (!ws || ws_bytes < need || ((uintptr_t)ws & 255u))
            OXQ_FAIL(h, OXQ_ERR_BUFFER_TOO_SMALL, "workspace: expected at least %zu bytes (256-byte aligned), got %zu", need, ws_bytes);
        void* wdq = (char*)ws + w4_clean_bytes(n);           // behind the region the decode kernels keep zeroed
        if (int32_t rc = oxq_int4g_dequant(h, codes, scales, zeros, n, k, group, wdq, OXQ_BF16)) return rc;
        return oxq_gemm_bf16(h, m, n, k, x, k, wdq, k, y, n);
    }
    if (group % 128 != 0 || k % 128 != 0) OXQ_FAIL(h, OXQ_ERR_UNSUPPORTED_OPERATION, "decode kernel needs group and k to be multiples of 128");
    if (((uintptr_t)x & 15u) || ((uintptr_t)codes & 15u)) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "x and codes must be 16-byte aligned");
    if (n > (int64_t)INT32_MAX / 64 || k > INT32_MAX / 64) OXQ_FAIL(h, OXQ_ERR_INVALID_DIMENSION, "dimension too large");
    if (int32_t rc = oxq_require_sm100(h)) return rc;

    if (mode >= 1 && m <= 8 && gemv_setting()) {
        // up to 8 batch rows: one CTA per 16 weight rows over the whole K, nothing to combine across CTAs
        GvParams gp;
        gp.m = (int)m; gp.n = (int)n; gp.k = (int)k; gp.group = group;
        gp.x = (const __nv_bfloat16*)x; gp.codes = codes; gp.scales = scales; gp.zeros = zeros; gp.y = (__nv_bfloat16*)y;
        gp.scales_vec_ok = ((uintptr_t)scales & 7u) == 0;          // the C type promises 2-byte alignment only: unaligned scales take the scalar loads
        OXQ_CUDA(h, oxq_launch(w4a16_gemv_kernel<true>, (unsigned)((n + 15) / 16), GV_WARPS * 32, 0, h->stream, gp));
        return OXQ_OK;
    }
    const int row_blocks = (int)((n + W4_ROWS_PER_CTA - 1) / W4_ROWS_PER_CTA);
    // K chunks of 4 spans (512 K): many short CTAs, so the tail of the grid is short as well
    const int spans_total = (int)(k / 128);
    const int spans_per = spans_total < W4_SPANS ? spans_total : W4_SPANS;
    const int splits = (spans_total + spans_per - 1) / spans_per;
    float* ws_sums = nullptr;
    int* ws_counters = nullptr;
    if (splits > 1) {
        const size_t need = mma_sync_ws_bytes(m, n);
        if (!ws || ws_bytes < need || ((uintptr_t)ws & 255u))
            OXQ_FAIL(h, OXQ_ERR_BUFFER_TOO_SMALL, "workspace: expected at least %zu bytes (256-byte aligned), got %zu", need, ws_bytes);
        ws_sums = (float*)ws;
        ws_counters = (int*)((char*)ws + split_sums_bytes(m, n));
    }
    dim3 grid(row_blocks, splits);
    // Batches above 16 rows run as passes of 16: the legacy MMA path is the limit there, and the second pass
    // finds most of the weight bytes in L2.
    for (int64_t m0 = 0; m0 < m; m0 += 16) {
        const int mc = (int)(m - m0 < 16 ? m - m0 : 16);
        W4Params p;
        p.m = mc; p.n = (int)n; p.k = (int)k; p.group = group; p.kc = spans_per * 128; p.splits = splits;
        p.x = (const __nv_bfloat16*)x + m0 * k; p.codes = codes; p.scales = scales; p.zeros = zeros;
        p.y = (__nv_bfloat16*)y + m0 * n;
        p.ws = ws_sums ? ws_sums + m0 * n : nullptr; p.counters = ws_counters;
        if (mc <= 8) oxq_launch(w4a16_decode_kernel<1, W4_SPANS>, grid, W4_THREADS, 0, h->stream, p);
        else oxq_launch(w4a16_decode_kernel<2, W4_SPANS>, grid, W4_THREADS, 0, h->stream, p);
    }
    OXQ_LAUNCH_CHECK(h);
    return OXQ_OK;
}

extern "C" {

// ---- W4A16 without any allocation ---------------------------------------------------------------
// Scratch for oxq_gemm_w4a16_static: lives in the library image, so every GPU that loads the library
// carries these bytes until the process exits.  Layout: [kStaticW4MaxOut f32 partial sums][counters].
static constexpr size_t kStaticW4MaxOut = 512 * 1024;                       // m * n <= 524288 outputs (2 MiB of f32)
static constexpr size_t kStaticW4Counters = kStaticW4MaxOut / W4_ROWS_PER_CTA; // one counter per 64 weight rows (m >= 1)
static constexpr size_t kStaticW4Bytes = kStaticW4MaxOut * sizeof(float) + kStaticW4Counters * sizeof(int);
static __device__ __align__(256) unsigned char g_w4_static_scratch[kStaticW4Bytes];

static constexpr int kMaxDevices = 64;
struct StaticW4Device {
    bool ready;
    void* scratch;      // device address of g_w4_static_scratch on this device
    int sm_count, cc_major, cc_minor;
};
static StaticW4Device g_static_w4[kMaxDevices];

int32_t oxq_gemm_w4a16_static(void* cuda_stream, int64_t m, int64_t n, int64_t k, const void* x, const uint32_t* codes,
                              const uint16_t* scales, const uint32_t* zeros, int group, void* y) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return OXQ_ERR_CUDA_BASE + (int32_t)e;
    if (dev < 0 || dev >= kMaxDevices) return OXQ_ERR_INVALID_ARGUMENT;
    StaticW4Device& d = g_static_w4[dev];
    if (!d.ready) {
        // Once per device, with that device current.  In host code the array's name is only a handle
        // for the runtime; the address a kernel can use comes from cudaGetSymbolAddress.
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_w4_static_scratch);
        if (e != cudaSuccess) return OXQ_ERR_CUDA_BASE + (int32_t)e;
        if (!ptr || ((uintptr_t)ptr & 255u)) return OXQ_ERR_LAUNCH_FAILED;
        e = cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (e == cudaSuccess) e = cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev);
        if (e == cudaSuccess) e = cudaDeviceGetAttribute(&d.cc_minor, cudaDevAttrComputeCapabilityMinor, dev);
        if (e != cudaSuccess) return OXQ_ERR_CUDA_BASE + (int32_t)e;
        d.scratch = ptr;
        d.ready = true;
    }
    if (m <= 0 || n <= 0 || k <= 0) return OXQ_ERR_INVALID_DIMENSION;
    if (m > 32) return OXQ_ERR_UNSUPPORTED_OPERATION;
    if ((uint64_t)m * (uint64_t)n > kStaticW4MaxOut) return OXQ_ERR_BUFFER_TOO_SMALL;   // beyond the built-in scratch
    // The array keeps whatever the previous call left in it: clear the part this call accumulates into.
    const size_t sums = ((size_t)m * (size_t)n * sizeof(float) + 255) & ~(size_t)255;
    const size_t counters = (((size_t)(n + W4_ROWS_PER_CTA - 1) / W4_ROWS_PER_CTA) * sizeof(int) + 255) & ~(size_t)255;
    if (sums + counters > kStaticW4Bytes) return OXQ_ERR_BUFFER_TOO_SMALL;
    e = cudaMemsetAsync(d.scratch, 0, sums + counters, (cudaStream_t)cuda_stream);
    if (e != cudaSuccess) return OXQ_ERR_CUDA_BASE + (int32_t)e;
    oxq_handle tmp;
    tmp.device = dev; tmp.stream = (cudaStream_t)cuda_stream; tmp.sm_count = d.sm_count;
    tmp.cc_major = d.cc_major; tmp.cc_minor = d.cc_minor; tmp.dev_status = nullptr; tmp.dev_scratch = nullptr; tmp.comm = nullptr; tmp.nranks = 1; tmp.rank = 0; tmp.last_error[0] = 0;
    return w4a16_impl(&tmp, m, n, k, x, codes, scales, zeros, group, y, d.scratch, sums + counters, 0);
}

int32_t oxq_gemm_w8a32(oxq_handle* h, int64_t m, int64_t n, int64_t k, const float* x, const int8_t* w, const float* sw, float* y) {
    OXQ_CHECK_HANDLE(h);
    if (m <= 0 || n <= 0 || k <= 0) OXQ_FAIL(h, OXQ_ERR_INVALID_DIMENSION, "GEMM dimensions must be non-zero");
    if (!x || !w || !sw || !y) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null pointer");
    if ((k & 15) || ((uintptr_t)x & 15u) || ((uintptr_t)w & 15u)) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "k must be a multiple of 16 and x, w 16-byte aligned");
    if (m > 64) OXQ_FAIL(h, OXQ_ERR_UNSUPPORTED_OPERATION, "oxq_gemm_w8a32 covers decode shapes (m <= 64), got m = %lld", (long long)m);
    if (int32_t rc = oxq_require_sm100(h)) return rc;
    const unsigned gx = (unsigned)((n + 15) / 16);
    if (m <= 8) oxq_launch(w8a32_tc_kernel<1>, dim3(gx, 1), W8T_WARPS * 32, 0, h->stream, x, w, sw, y, (int)m, (int)n, (int)k);
    else if (m <= 16) oxq_launch(w8a32_tc_kernel<2>, dim3(gx, 1), W8T_WARPS * 32, 0, h->stream, x, w, sw, y, (int)m, (int)n, (int)k);
    else oxq_launch(w8a32_tc_kernel<4>, dim3(gx, (unsigned)((m + 31) / 32)), W8T_WARPS * 32, 0, h->stream, x, w, sw, y, (int)m, (int)n, (int)k);
    OXQ_LAUNCH_CHECK(h);
    return OXQ_OK;
}

}  // extern "C"
