// FP8 (E4M3 x E4M3) GEMM for decode shapes, up to 8 batch rows (the kernel is written for NT tiles of 8 rows that share
// the weight registers, but mma.sync is slow enough on this part that the 128-row kernels win from 16 rows on -- at
// 57344 x 8192, 16 / 64 rows took 124 / 363 us here against 115 / 116 us there -- so only NT = 1 is launched): Y = bf16(alpha * (X . W^T) * sx * sw), or the SwiGLU
// form on a gate/up-interleaved weight.  The 128-row tensor-memory kernels serve these shapes at half the HBM rate
// (one 128-row tile of X is almost empty and every CTA still pays the full pipeline set-up); here the weight stream
// is the only cost.  Same shape as the W4A16 GEMV: a CTA owns 16 weight rows over the whole K range, its 8 warps
// split K in spans of 64 codes and meet once in shared memory.  Lane (g, t) streams 16 bytes of rows g and g + 8 per
// span and 16 bytes of batch row g; the bytes go into mma.sync m16n8k32 e4m3 as they are -- no conversion, no
// shuffles: about ten instructions per 32 weights.
//
// SwiGLU form: the weight holds blocks of 128 gate rows followed by the 128 matching up rows.  The CTA takes 8 gate
// rows as its rows 0-7 and the 8 matching up rows as its rows 8-15, so the accumulator pair of a lane is (gate, up)
// of the same output column and silu(gate) * up needs no exchange.
#include "oxq_common.cuh"
#include <type_traits>

namespace oxq {
namespace {

constexpr int FG_WARPS = 8;
constexpr int FG_CHUNK = 2;            // 64-code spans per register buffer

__device__ __forceinline__ void mma_e4m3_16832(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_s8_16832(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_8bit(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) { mma_e4m3_16832(d, a0, a1, a2, a3, b0, b1); }
__device__ __forceinline__ void mma_8bit(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) { mma_s8_16832(d, a0, a1, a2, a3, b0, b1); }
__device__ __forceinline__ uint4 ld_stream_u4(const void* p) {
    uint4 u;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(u.x), "=r"(u.y), "=r"(u.z), "=r"(u.w) : "l"(p));
    return u;
}
__device__ __forceinline__ uint4 ld_pinned_u4(const void* p) {
    uint4 u;
    asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(u.x), "=r"(u.y), "=r"(u.z), "=r"(u.w) : "l"(p) : "memory");
    return u;
}

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// stores v at the same shared-memory offset in CTA `rank` of the cluster
__device__ __forceinline__ void st_cluster_b32(const void* local, uint32_t rank, uint32_t bits) {
    uint32_t a = (uint32_t)__cvta_generic_to_shared(local), ra;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(a), "r"(rank));
    asm volatile("st.shared::cluster.b32 [%0], %1;" ::"r"(ra), "r"(bits) : "memory");
}
__device__ __forceinline__ void st_cluster(const float* local, uint32_t rank, float v) { st_cluster_b32(local, rank, __float_as_uint(v)); }
__device__ __forceinline__ void st_cluster(const int* local, uint32_t rank, int v) { st_cluster_b32(local, rank, (uint32_t)v); }
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
}

struct FgParams {
    int m, n, k;                 // n: weight rows (SwiGLU: gate + up rows, a multiple of 256)
    int64_t ldx, ldw, ldy;
    const uint8_t* x;            // [m x k] E4M3
    const uint8_t* w;            // [n x k] E4M3
    const float* sx;             // FP8: one scale; W8A8: one per batch row
    const float* sw;             // FP8: one scale; W8A8: one per weight row
    float alpha;
    int ksplit;                  // CTAs of a cluster that share the K range of one row block (1, 2 or 4)
    __nv_bfloat16* y;            // [m x n], or [m x n/2] in the SwiGLU form
};

// NT: tiles of 8 batch rows (the weight registers are shared by the tiles)
// I8: int8 x int8 with an exact s32 accumulator and per-row scales (W8A8) instead of E4M3 x E4M3 with f32
template <bool I8, bool SWIGLU, int NT>
__global__ void __launch_bounds__(FG_WARPS * 32, NT == 1 ? 4 : 3) fp8_gemv_kernel(const FgParams p) {
    constexpr int NB = 8 * NT;                                // batch rows of a CTA
    using Acc = typename std::conditional<I8, int, float>::type;
    __shared__ Acc red[FG_WARPS][16][NB];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    // the cluster's CTAs (grid y) take consecutive parts of the K range; inside a CTA the warps split its part
    const uint32_t crank = p.ksplit > 1 ? cluster_rank() : 0u;
    const int all_spans = (p.k + 63) >> 6;
    const int c_lo = (int)(((int64_t)crank * all_spans) / p.ksplit), c_hi = (int)(((int64_t)(crank + 1) * all_spans) / p.ksplit);
    const int s_lo = c_lo + (int)(((int64_t)warp * (c_hi - c_lo)) / FG_WARPS), s_hi = c_lo + (int)(((int64_t)(warp + 1) * (c_hi - c_lo)) / FG_WARPS);
    int row_a, row_b;
    if (SWIGLU) {
        const int o = (int)blockIdx.x * 8 + g;                            // output column; 8 per CTA, never across a block of 128
        row_a = (o >> 7) * 256 + (o & 127);
        row_b = row_a + 128;
    } else {
        row_a = min((int)blockIdx.x * 16 + g, p.n - 1);
        row_b = min((int)blockIdx.x * 16 + g + 8, p.n - 1);
    }
    const uint8_t* pa = p.w + (size_t)row_a * p.ldw + 16 * t;
    const uint8_t* pb = p.w + (size_t)row_b * p.ldw + 16 * t;
    const uint8_t* xr = p.x + 16 * t;

    uint4 cur_a[FG_CHUNK], cur_b[FG_CHUNK], nxt_a[FG_CHUNK], nxt_b[FG_CHUNK];
    auto fetch = [&](int s0, uint4 (&wa)[FG_CHUNK], uint4 (&wb)[FG_CHUNK]) {
#pragma unroll
        for (int j = 0; j < FG_CHUNK; j++) {
            const int s = s0 + j;
            wa[j] = make_uint4(0, 0, 0, 0); wb[j] = wa[j];               // +0 codes: past the warp's range or the ragged end of K
            if (s < s_hi && s * 64 + 16 * t < p.k) {
                wa[j] = ld_stream_u4(pa + (size_t)s * 64);
                wb[j] = ld_stream_u4(pb + (size_t)s * 64);
            }
        }
    };
    Acc acc[NT][4];
#pragma unroll
    for (int i = 0; i < NT; i++) { acc[i][0] = 0; acc[i][1] = 0; acc[i][2] = 0; acc[i][3] = 0; }
    // Before the kernel ahead of this one in the stream has finished, the first weights are only prefetched into the L2
    // (it may be the quantizer that writes them); they are read after the wait.
    pdl_trigger();
#pragma unroll
    for (int j = 0; j < FG_CHUNK; j++) {
        const int s = s_lo + j;
        if (s < s_hi && s * 64 + 16 * t < p.k) { prefetch_l2(pa + (size_t)s * 64); prefetch_l2(pb + (size_t)s * 64); }
    }
    pdl_wait();
    if (s_lo < s_hi) fetch(s_lo, cur_a, cur_b);
    for (int s0 = s_lo; s0 < s_hi; s0 += FG_CHUNK) {
        if (s0 + FG_CHUNK < s_hi) fetch(s0 + FG_CHUNK, nxt_a, nxt_b);
#pragma unroll
        for (int j = 0; j < FG_CHUNK; j++) {
            const int s = s0 + j;
            if (s < s_hi) {
                const bool in_k = s * 64 + 16 * t < p.k;
#pragma unroll
                for (int i = 0; i < NT; i++) {
                    uint4 xv = make_uint4(0, 0, 0, 0);
                    if (in_k && 8 * i + g < p.m) xv = ld_pinned_u4(xr + (size_t)(8 * i + g) * p.ldx + (size_t)s * 64);
                    // word q of the lane's 16 codes meets word q of its 16 activations: k slots (4t.., 4t + 16..) take words (0, 1), then (2, 3)
                    if constexpr (I8) {
                        mma_8bit(acc[i], cur_a[j].x, cur_b[j].x, cur_a[j].y, cur_b[j].y, xv.x, xv.y);
                        mma_8bit(acc[i], cur_a[j].z, cur_b[j].z, cur_a[j].w, cur_b[j].w, xv.z, xv.w);
                    } else {
                        // The FP8 mma.sync path adds its products to the accumulator at reduced precision (about 13 bits
                        // relative to the accumulator's magnitude, measured as a 0.7 % drift over K = 8192 with one running
                        // accumulator).  A span's 64 products therefore go into a fresh accumulator and are promoted into
                        // the running f32 sum with ordinary additions.
                        Acc part4[4] = {0, 0, 0, 0};
                        mma_8bit(part4, cur_a[j].x, cur_b[j].x, cur_a[j].y, cur_b[j].y, xv.x, xv.y);
                        mma_8bit(part4, cur_a[j].z, cur_b[j].z, cur_a[j].w, cur_b[j].w, xv.z, xv.w);
                        acc[i][0] += part4[0]; acc[i][1] += part4[1]; acc[i][2] += part4[2]; acc[i][3] += part4[3];
                    }
                }
            }
        }
#pragma unroll
        for (int j = 0; j < FG_CHUNK; j++) { cur_a[j] = nxt_a[j]; cur_b[j] = nxt_b[j]; }
    }
    // accumulator element e of tile i: CTA row (e < 2 ? g : g + 8), batch row 8i + 2t + (e & 1)
#pragma unroll
    for (int i = 0; i < NT; i++) {
        red[warp][g][8 * i + 2 * t] = acc[i][0]; red[warp][g][8 * i + 2 * t + 1] = acc[i][1];
        red[warp][g + 8][8 * i + 2 * t] = acc[i][2]; red[warp][g + 8][8 * i + 2 * t + 1] = acc[i][3];
    }
    __syncthreads();
    __shared__ Acc part[3][16][NB];                           // sums of the cluster's other CTAs (written by them)
    __shared__ float fin[16][NB];
    constexpr int PER = (16 * NB + FG_WARPS * 32 - 1) / (FG_WARPS * 32);      // (row, batch row) pairs per thread
    Acc v[PER];
#pragma unroll
    for (int q = 0; q < PER; q++) {
        const int idx = threadIdx.x + q * FG_WARPS * 32;
        v[q] = 0;
        if (idx < 16 * NB) {
            const int col = idx >> 4, r = idx & 15;
#pragma unroll
            for (int wi = 0; wi < FG_WARPS; wi++) v[q] += red[wi][r][col];
        }
    }
    if (p.ksplit > 1) {
        if (crank != 0) {
#pragma unroll
            for (int q = 0; q < PER; q++) {
                const int idx = threadIdx.x + q * FG_WARPS * 32;
                if (idx < 16 * NB) st_cluster(&part[crank - 1][idx & 15][idx >> 4], 0, v[q]);
            }
        }
        cluster_sync_all();                                   // every thread of every CTA of the cluster
        if (crank != 0) return;
#pragma unroll
        for (int q = 0; q < PER; q++) {
            const int idx = threadIdx.x + q * FG_WARPS * 32;
            if (idx < 16 * NB)
                for (int c = 1; c < p.ksplit; c++) v[q] += part[c - 1][idx & 15][idx >> 4];
        }
    }
    const float scale = I8 ? 1.0f : __ldg(p.sx) * __ldg(p.sw) * p.alpha;
    if (SWIGLU) {
#pragma unroll
        for (int q = 0; q < PER; q++) {
            const int idx = threadIdx.x + q * FG_WARPS * 32;
            if (idx < 16 * NB) fin[idx & 15][idx >> 4] = (float)v[q];
        }
        __syncthreads();
        for (int idx = threadIdx.x; idx < 8 * NB; idx += FG_WARPS * 32) {
            const int bc = idx >> 3, oc = idx & 7;                        // batch row, output column inside the CTA
            const float gt = fin[oc][bc] * scale, up = fin[oc + 8][bc] * scale;
            const int o = (int)blockIdx.x * 8 + oc;
            if (bc < p.m) p.y[(size_t)bc * p.ldy + o] = __float2bfloat16_rn(__fdividef(gt, 1.0f + __expf(-gt)) * up);
        }
    } else {
#pragma unroll
        for (int q = 0; q < PER; q++) {
            const int idx = threadIdx.x + q * FG_WARPS * 32;
            const int col = idx >> 4, row = (int)blockIdx.x * 16 + (idx & 15);
            if (idx < 16 * NB && col < p.m && row < p.n) {
                // W8A8: the same expression as the 128-row kernel's epilogue, (float)acc * (sx[m] * sw[n])
                const float sc = I8 ? __ldg(p.sx + col) * p.alpha * __ldg(p.sw + row) : scale;
                p.y[(size_t)col * p.ldy + row] = __float2bfloat16_rn((float)v[q] * sc);
            }
        }
    }
}

}  // namespace
}  // namespace oxq

// Launches the GEMV; the caller has validated pointers, alignment (16 bytes, k / ldx / ldw multiples of 16) and m <= 8.
cudaError_t oxq_fp8_gemv_launch(oxq_handle* h, int m, int n, int k, const uint8_t* x, int64_t ldx, const uint8_t* w, int64_t ldw,
                                const float* sx, const float* sw, float alpha, void* y, int64_t ldy, bool swiglu, bool int8) {
    using namespace oxq;
    FgParams p;
    p.m = m; p.n = n; p.k = k; p.ldx = ldx; p.ldw = ldw; p.ldy = ldy; p.x = x; p.w = w; p.sx = sx; p.sw = sw; p.alpha = alpha;
    p.y = (__nv_bfloat16*)y;
    // Few row blocks for the machine (a long-K projection, or a small matrix): clusters of 2 or 4 CTAs split K and add
    // their sums through distributed shared memory, so that there are at least four waves of CTAs to balance.
    const int64_t blocks = swiglu ? n / 16 : (n + 15) / 16, slots = 4 * (int64_t)h->sm_count;
    int ks = 1;
    while (ks < 4 && blocks * ks < 4 * slots && (int64_t)16 * k / (2 * ks) >= 65536) ks *= 2;   // keep at least 64 KB of weights per CTA
    p.ksplit = ks;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)blocks, (unsigned)ks, 1); cfg.blockDim = dim3(FG_WARPS * 32, 1, 1); cfg.dynamicSmemBytes = 0; cfg.stream = h->stream;
    cudaLaunchAttribute attrs[2];
    int na = 0;
    if (ks > 1) {
        attrs[na].id = cudaLaunchAttributeClusterDimension;
        attrs[na].val.clusterDim.x = 1; attrs[na].val.clusterDim.y = (unsigned)ks; attrs[na].val.clusterDim.z = 1;
        na++;
    }
    if (oxq_pdl_enabled()) {
        attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attrs[na].val.programmaticStreamSerializationAllowed = 1;
        na++;
    }
    cfg.attrs = attrs; cfg.numAttrs = na;
    if (int8) return cudaLaunchKernelEx(&cfg, fp8_gemv_kernel<true, false, 1>, p);
    if (swiglu) return cudaLaunchKernelEx(&cfg, fp8_gemv_kernel<false, true, 1>, p);
    return cudaLaunchKernelEx(&cfg, fp8_gemv_kernel<false, false, 1>, p);
}
