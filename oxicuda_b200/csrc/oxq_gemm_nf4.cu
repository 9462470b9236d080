// Decode-shaped GEMM on NF4 weights (QLoRA's NormalFloat4): y[m][n] = sum_k x[m][k] * lut[code[n][k]] * absmax[n][k / block]
// for up to 8 batch rows, with the dequantisation fused in.  The weights are what Nf4Quantizer::encode produces
// (crates/oxicuda-quant/src/scheme/nf4.rs:93-125: two codes per byte, even element in the low nibble, one f32
// absmax per block); the reference only has the elementwise nf4_dequant kernel (crates/oxicuda-quant/src/ptx_kernels.rs:261-396),
// so this is dequantise-then-GEMV in one pass over the packed bytes.
//
// Same shape as the W4A16 GEMV: a CTA owns 16 weight rows over the whole K range, its 8 warps split K and meet once
// in shared memory.  Lane (g, t) streams rows g and g + 8, eight bytes (16 codes) per 64-wide span, so that a span
// never crosses an absmax block; each byte of codes indexes a 256-entry table of bf16 pairs (lut[low], lut[high]),
// kept in shared memory once per lane (entry i of lane l in bank l: no conflicts whatever the codes are), and the pair
// goes straight into the A operand of mma.sync m16n8k16 next to the matching two activations.  The span's partial
// sums are scaled by the two rows' absmax in f32.  The levels are rounded to bf16 (relative 2^-9) for the tensor
// core; the activations are bf16 anyway, accumulation is f32.
#include "oxq_common.cuh"

namespace oxq {
namespace {

constexpr int NG_WARPS = 8;
constexpr int NG_CHUNK = 4;            // 64-wide spans per register buffer

__constant__ float c_nf4_levels[16] = {-1.0f, -0.69619286f, -0.52507305f, -0.3949175f, -0.28444138f, -0.18477343f, -0.09105003f, 0.0f,
                                       0.0795803f, 0.1609302f, 0.2461123f, 0.33791524f, 0.44070983f, 0.562617f, 0.72295684f, 1.0f};

__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint2 ld_stream_u2(const void* p) {
    uint2 u;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(u.x), "=r"(u.y) : "l"(p));
    return u;
}
__device__ __forceinline__ uint4 ld_pinned_u4(const void* p) {
    uint4 u;
    asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(u.x), "=r"(u.y), "=r"(u.z), "=r"(u.w) : "l"(p) : "memory");
    return u;
}

struct Nf4Params {
    int m, n, k;
    int bpr;                     // absmax blocks per weight row
    int spb;                     // 64-wide spans per absmax block
    int spb_shift;               // log2(spb) when spb is a power of two, else -1
    const __nv_bfloat16* x;      // [m x k]
    const uint8_t* packed;       // [n x k/2]
    const float* absmax;         // [n x bpr]
    __nv_bfloat16* y;            // [m x n]
};

__global__ void __launch_bounds__(NG_WARPS * 32, 3) nf4_gemv_kernel(const Nf4Params p) {
    extern __shared__ __align__(16) uint32_t tab[];           // [256][32]: entry i of lane l at i * 32 + l
    __shared__ float red[NG_WARPS][16][8];
    __shared__ uint32_t lv[16];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    pdl_trigger();
    const uint32_t* tl = tab + lane;

    const int spans = p.k >> 6;
    const int s_lo = (int)(((int64_t)warp * spans) / NG_WARPS), s_hi = (int)(((int64_t)(warp + 1) * spans) / NG_WARPS);
    const int row_a = min((int)blockIdx.x * 16 + g, p.n - 1), row_b = min((int)blockIdx.x * 16 + g + 8, p.n - 1);
    const uint8_t* pa = p.packed + (size_t)row_a * (p.k >> 1) + 8 * t;
    const uint8_t* pb = p.packed + (size_t)row_b * (p.k >> 1) + 8 * t;
    const float* aa = p.absmax + (size_t)row_a * p.bpr;
    const float* ab = p.absmax + (size_t)row_b * p.bpr;
    const bool has_x = g < p.m;
    const __nv_bfloat16* xr = p.x + (size_t)(has_x ? g : 0) * p.k + 16 * t;

    uint2 cur_a[NG_CHUNK], cur_b[NG_CHUNK], nxt_a[NG_CHUNK], nxt_b[NG_CHUNK];
    float cur_sa[NG_CHUNK], cur_sb[NG_CHUNK], nxt_sa[NG_CHUNK], nxt_sb[NG_CHUNK];
    auto fetch = [&](int s0, uint2 (&wa)[NG_CHUNK], uint2 (&wb)[NG_CHUNK], float (&sa)[NG_CHUNK], float (&sb)[NG_CHUNK]) {
#pragma unroll
        for (int j = 0; j < NG_CHUNK; j++) {
            const int s = s0 + j;
            wa[j] = make_uint2(0, 0); wb[j] = wa[j]; sa[j] = 0.0f; sb[j] = 0.0f;     // scale 0: the span contributes nothing
            if (s < s_hi) {
                wa[j] = ld_stream_u2(pa + (size_t)s * 32);
                wb[j] = ld_stream_u2(pb + (size_t)s * 32);
                const int b = p.spb_shift >= 0 ? (s >> p.spb_shift) : (s / p.spb);
                sa[j] = __ldg(aa + b);
                sb[j] = __ldg(ab + b);
            }
        }
    };

    float total[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    // Before the kernel ahead of this one in the stream has finished, the first weights are only prefetched into the L2
    // (it may be the encoder that writes them); the table is built meanwhile and the weights are read after the wait.
#pragma unroll
    for (int j = 0; j < NG_CHUNK; j++) {
        const int s = s_lo + j;
        if (s < s_hi) { prefetch_l2(pa + (size_t)s * 32); prefetch_l2(pb + (size_t)s * 32); }
    }
    if (threadIdx.x < 16) lv[threadIdx.x] = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(c_nf4_levels[threadIdx.x]));
    __syncthreads();
    for (int e = threadIdx.x; e < 256 * 8; e += NG_WARPS * 32) {              // 16-byte stores: four lanes' copies at a time
        const int idx = e >> 3;
        const uint32_t v = lv[idx & 15] | (lv[idx >> 4] << 16);
        reinterpret_cast<uint4*>(tab)[e] = make_uint4(v, v, v, v);
    }
    __syncthreads();
    pdl_wait();
    if (s_lo < s_hi) fetch(s_lo, cur_a, cur_b, cur_sa, cur_sb);
    for (int s0 = s_lo; s0 < s_hi; s0 += NG_CHUNK) {
        if (s0 + NG_CHUNK < s_hi) fetch(s0 + NG_CHUNK, nxt_a, nxt_b, nxt_sa, nxt_sb);
#pragma unroll
        for (int j = 0; j < NG_CHUNK; j++) {
            const int s = s0 + j;
            if (s < s_hi) {
                const uint4* xp = reinterpret_cast<const uint4*>(xr + (size_t)s * 64);
                uint4 xv[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
                if (has_x) { xv[0] = ld_pinned_u4(xp); xv[1] = ld_pinned_u4(xp + 1); }
                float part[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                const uint32_t wwa[2] = {cur_a[j].x, cur_a[j].y}, wwb[2] = {cur_b[j].x, cur_b[j].y};
#pragma unroll
                for (int i = 0; i < 2; i++) {
                    // byte q of the word holds codes 2q and 2q + 1, which meet activations 2q and 2q + 1 of the same eight
                    const uint32_t a0 = tl[(wwa[i] & 0xFFu) << 5], a1 = tl[(wwb[i] & 0xFFu) << 5];
                    const uint32_t a2 = tl[((wwa[i] >> 8) & 0xFFu) << 5], a3 = tl[((wwb[i] >> 8) & 0xFFu) << 5];
                    mma_bf16(part, a0, a1, a2, a3, xv[i].x, xv[i].y);
                    const uint32_t c0 = tl[((wwa[i] >> 16) & 0xFFu) << 5], c1 = tl[((wwb[i] >> 16) & 0xFFu) << 5];
                    const uint32_t c2 = tl[(wwa[i] >> 24) << 5], c3 = tl[(wwb[i] >> 24) << 5];
                    mma_bf16(part, c0, c1, c2, c3, xv[i].z, xv[i].w);
                }
                total[0] = fmaf(cur_sa[j], part[0], total[0]);
                total[1] = fmaf(cur_sa[j], part[1], total[1]);
                total[2] = fmaf(cur_sb[j], part[2], total[2]);
                total[3] = fmaf(cur_sb[j], part[3], total[3]);
            }
        }
#pragma unroll
        for (int j = 0; j < NG_CHUNK; j++) { cur_a[j] = nxt_a[j]; cur_b[j] = nxt_b[j]; cur_sa[j] = nxt_sa[j]; cur_sb[j] = nxt_sb[j]; }
    }
    // accumulator element e: weight row (e < 2 ? g : g + 8), batch row 2t + (e & 1)
    red[warp][g][2 * t] = total[0]; red[warp][g][2 * t + 1] = total[1];
    red[warp][g + 8][2 * t] = total[2]; red[warp][g + 8][2 * t + 1] = total[3];
    __syncthreads();
    if (threadIdx.x < 128) {
        const int col = threadIdx.x >> 4, r = threadIdx.x & 15;
        const int row = (int)blockIdx.x * 16 + r;
        float acc = 0.0f;
#pragma unroll
        for (int w = 0; w < NG_WARPS; w++) acc += red[w][r][col];
        if (col < p.m && row < p.n) p.y[(size_t)col * p.n + row] = __float2bfloat16_rn(acc);
    }
}

}  // namespace
}  // namespace oxq

using namespace oxq;

extern "C" int32_t oxq_gemm_nf4(oxq_handle* h, int64_t m, int64_t n, int64_t k, const void* x, const uint8_t* packed, const float* absmax,
                                int64_t block, void* y) {
    OXQ_CHECK_HANDLE(h);
    if (m <= 0 || n <= 0 || k <= 0) OXQ_FAIL(h, OXQ_ERR_INVALID_DIMENSION, "GEMM dimensions must be non-zero");
    if (m > 8) OXQ_FAIL(h, OXQ_ERR_UNSUPPORTED_OPERATION, "the NF4 GEMM serves decode shapes, m <= 8 (got %lld): dequantise with oxq_nf4_dequant and use oxq_gemm_bf16 above that", (long long)m);
    if (block <= 0 || block % 64 != 0 || k % block != 0) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "block must be a multiple of 64 that divides k (block %lld, k %lld)", (long long)block, (long long)k);
    if (n > (1 << 27) || k > (1 << 24)) OXQ_FAIL(h, OXQ_ERR_INVALID_DIMENSION, "matrix too large");
    if (!x || !packed || !absmax || !y || ((uintptr_t)x & 15) || ((uintptr_t)packed & 15) || ((uintptr_t)absmax & 3))
        OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null or misaligned pointer");
    if (int32_t rc = oxq_require_sm100(h)) return rc;
    Nf4Params p;
    p.m = (int)m; p.n = (int)n; p.k = (int)k; p.bpr = (int)(k / block); p.spb = (int)(block / 64);
    p.spb_shift = -1;
    for (int sh = 0; sh < 20; sh++) if ((1 << sh) == p.spb) p.spb_shift = sh;
    p.x = (const __nv_bfloat16*)x; p.packed = packed; p.absmax = absmax; p.y = (__nv_bfloat16*)y;
    OXQ_CUDA(h, oxq_launch(nf4_gemv_kernel, (unsigned)((n + 15) / 16), NG_WARPS * 32, 256 * 32 * sizeof(uint32_t), h->stream, p));
    return OXQ_OK;
}
