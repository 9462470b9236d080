// Prefill-shaped low-precision GEMMs on the sm_100a tensor cores.
//
// One persistent, warp-specialised kernel template: a TMA producer warp streams 128-byte-swizzled
// operand tiles into a shared-memory ring, one thread issues tcgen05.mma with the accumulator in
// tensor memory (two accumulator buffers, so the epilogue of tile i overlaps the main loop of tile
// i+1), and four epilogue warps drain tensor memory with tcgen05.ld, apply the scales and store bf16.
// Block-scaled kinds additionally stream scale-factor chunks (bulk copies) and move them into
// tensor memory with tcgen05.cp before each group of MMAs.
//
//   Y[M x N] = X[M x K] * W[N x K]^T, both operands K-contiguous ("K-major"), f32 / s32 accumulate.
#include "oxq_common.cuh"
#include "oxq_tc.cuh"
#include <stdlib.h>

namespace oxq {
namespace tc {

// Epilogues: EPI_SCALE stores acc * scale; EPI_SWIGLU treats each 256-column tile as 128 gate columns
// followed by the 128 matching up columns and stores silu(gate) * up (SwiGluFfn::forward,
// crates/oxicuda-lm/src/layer/ffn.rs:235-254, fused into the gate/up projection).
enum { EPI_SCALE = 0, EPI_SWIGLU = 1 };

constexpr int BM = 128;               // rows of X per tile == tensor-memory lanes
constexpr int BKB = 128;              // bytes of K per stage == one swizzle atom
constexpr int NUM_THREADS = 192;      // warp 0: TMA, warp 1: MMA + tensor-memory owner, warps 2-5: epilogue
constexpr int SMEM_BUDGET = 227 * 1024;

struct GemmParams {
    int m, n, k_bytes;                // k_bytes: bytes of K per operand row (K for 8-bit, K/2 for 4-bit)
    void* y; int64_t ldy;             // bf16 output
    const float* s0; const float* s1; // epilogue scales (meaning depends on the kind)
    const uint8_t* sfa; const uint8_t* sfb;   // tiled scale factors (block-scaled kinds)
    int sf_col_tiles;                 // 4-column scale-factor tiles per row tile
    int sfa_row_tiles, sfb_row_tiles;
    int group_m;                      // M-tiles per rasterisation group (L2 reuse of the X panel)
    float alpha, beta;                // plain epilogue: y = alpha * (acc * scales) + beta * y (beta == 0: y is not read)
    int full_tiles, tail_split;       // CTA-pair dense kernel: tiles done whole, and the number of N-parts of each remaining tile
    int a_mn, b_mn;                   // CTA-pair dense kernel: operand stored MN-major (X as [K x M], W as [K x N]) instead of K-major
    int esize;                        // bytes per operand element (1 or 2)
    int32_t* status;
    // fused all-reduce form of the CTA-pair kernel: y is this rank's replica of a symmetric buffer
    void* ar_mc_y;                    // the same buffer through the multicast mapping
    uint32_t* ar_flags;               // this rank's replica of the flag words: two sets of ([items] arrivals, one word of finished units)
    uint32_t* ar_mc_flags;            // the flag words through the multicast mapping
    uint32_t* ar_calls;               // this rank's count of finished calls on these flag words (device memory: the parity picks the set,
                                      // so a replayed CUDA graph alternates like a sequence of host calls does)
    int ar_set_stride;                // words from one set to the other
    int ar_world, ar_rank;
    int ar_sleep_ns;                  // pause between two looks at a flag word (0: none)
};

template <int KIND, int BN>
struct Cfg {
    static constexpr bool kScaled = KIND == KIND_MXF8 || KIND == KIND_NVF4;
    // scale-factor chunks (128 rows x 4 scale columns, 512 bytes) per stage and operand row tile
    static constexpr int kSfChunks = KIND == KIND_MXF8 ? 1 : (KIND == KIND_NVF4 ? 4 : 0);
    static constexpr int kSfaBytes = kSfChunks * 512;
    static constexpr int kSfbBytes = kScaled ? 2 * kSfChunks * 512 : 0;   // two 128-row tiles cover BN <= 256
    static constexpr int kABytes = BM * BKB;
    static constexpr int kBBytes = BN * BKB;
    static constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;
    static constexpr int kStages = (SMEM_BUDGET - 2048) / kStageBytes > 8 ? 8 : (SMEM_BUDGET - 2048) / kStageBytes;
    static constexpr int kSmemBytes = kStages * kStageBytes + 2048;        // + alignment slack and barriers
    // tensor-memory columns: two accumulators, then scale factors
    static constexpr int kAccStride = BN == 192 ? 256 : BN;
    static constexpr int kSfaCol = BN == 256 ? 0 : (BN == 192 ? 448 : 256);   // unused when BN == 256
    static constexpr int kSfbCol = kSfaCol + 4 * kSfChunks;
    static_assert(!kScaled || BN != 256, "block-scaled kinds need tensor-memory columns for scale factors");
    static_assert(!kScaled || kSfbCol + 8 * kSfChunks <= 512, "tensor memory overflow");
};

// Tiles are walked in groups of `group_m` M-tiles: inside a group M runs fastest, then N, so the
// CTAs of one wave share a narrow X panel (it stays in L2 for the whole sweep over N) and each
// W tile is used by group_m CTAs at about the same time.
__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int group_m, int& tm, int& tn) {
    const int per_group = group_m * tiles_n;
    const int g = tile / per_group;
    const int first_m = g * group_m;
    const int gm = min(group_m, tiles_m - first_m);
    const int r = tile - g * per_group;
    tn = r / gm;
    tm = first_m + (r - tn * gm);
}

template <int KIND>
__device__ __forceinline__ void epilogue_store_scale(const uint32_t (&r)[32], int row, int col0, const GemmParams& p, float tensor_scale,
                                                     float row_scale, __nv_bfloat16* y) {
    if (row >= p.m || col0 >= p.n) return;
    float v[32];
#pragma unroll
    for (int j = 0; j < 32; j++) {
        if (KIND == KIND_I8) v[j] = (float)(int)r[j] * (row_scale * (col0 + j < p.n ? __ldg(p.s1 + col0 + j) : 0.0f));
        else v[j] = __uint_as_float(r[j]) * tensor_scale;
    }
    __nv_bfloat16* dst = y + (size_t)row * p.ldy + col0;
    if (col0 + 32 <= p.n) {
        if (p.beta != 0.0f) {                                    // gemm's beta * C term: read the old values, one rounding at the end
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const uint4 o = *reinterpret_cast<const uint4*>(dst + 8 * j);
                const uint32_t w[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    v[8 * j + 2 * e] = fmaf(p.beta, __uint_as_float(w[e] << 16), v[8 * j + 2 * e]);
                    v[8 * j + 2 * e + 1] = fmaf(p.beta, __uint_as_float(w[e] & 0xFFFF0000u), v[8 * j + 2 * e + 1]);
                }
            }
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            uint4 o;
            __nv_bfloat162 t0 = __floats2bfloat162_rn(v[8 * j + 0], v[8 * j + 1]);
            __nv_bfloat162 t1 = __floats2bfloat162_rn(v[8 * j + 2], v[8 * j + 3]);
            __nv_bfloat162 t2 = __floats2bfloat162_rn(v[8 * j + 4], v[8 * j + 5]);
            __nv_bfloat162 t3 = __floats2bfloat162_rn(v[8 * j + 6], v[8 * j + 7]);
            o.x = *reinterpret_cast<uint32_t*>(&t0); o.y = *reinterpret_cast<uint32_t*>(&t1);
            o.z = *reinterpret_cast<uint32_t*>(&t2); o.w = *reinterpret_cast<uint32_t*>(&t3);
            *reinterpret_cast<uint4*>(dst + 8 * j) = o;
        }
    } else {
        for (int j = 0; j < 32 && col0 + j < p.n; j++) {
            const float old = p.beta != 0.0f ? p.beta * __bfloat162float(dst[j]) : 0.0f;
            dst[j] = __float2bfloat16_rn(v[j] + old);
        }
    }
}

__device__ __forceinline__ void epilogue_store_swiglu(const uint32_t (&rg)[32], const uint32_t (&ru)[32], int row, int col0, int out_n,
                                                      const GemmParams& p, float tensor_scale, __nv_bfloat16* y) {
    if (row >= p.m || col0 >= out_n) return;
    float v[32];
#pragma unroll
    for (int j = 0; j < 32; j++) {
        const float gt = __uint_as_float(rg[j]) * tensor_scale, up = __uint_as_float(ru[j]) * tensor_scale;
        v[j] = __fdividef(gt, 1.0f + __expf(-gt)) * up;
    }
    __nv_bfloat16* dst = y + (size_t)row * p.ldy + col0;
    if (col0 + 32 <= out_n) {
#pragma unroll
        for (int j = 0; j < 4; j++) {
            uint4 o;
            __nv_bfloat162 t0 = __floats2bfloat162_rn(v[8 * j + 0], v[8 * j + 1]);
            __nv_bfloat162 t1 = __floats2bfloat162_rn(v[8 * j + 2], v[8 * j + 3]);
            __nv_bfloat162 t2 = __floats2bfloat162_rn(v[8 * j + 4], v[8 * j + 5]);
            __nv_bfloat162 t3 = __floats2bfloat162_rn(v[8 * j + 6], v[8 * j + 7]);
            o.x = *reinterpret_cast<uint32_t*>(&t0); o.y = *reinterpret_cast<uint32_t*>(&t1);
            o.z = *reinterpret_cast<uint32_t*>(&t2); o.w = *reinterpret_cast<uint32_t*>(&t3);
            *reinterpret_cast<uint4*>(dst + 8 * j) = o;
        }
    } else {
        for (int j = 0; j < 32 && col0 + j < out_n; j++) dst[j] = __float2bfloat16_rn(v[j]);
    }
}

// Work items of the CTA-pair dense kernel.  The first `full_tiles` items are whole 256 x 256 tiles; every tile after
// that (the last, partly filled wave) is cut along N into `tail_split` parts so that the pairs which would idle
// take a share: part p of a tile holds, of each 128-column half, the columns [p * half, (p + 1) * half).
struct WorkItem { int tile, part, n_cols; };                 // n_cols = 256 / tail_split for a part, else 256
__device__ __forceinline__ WorkItem work_item(int w, int full_tiles, int tail_split) {
    WorkItem it;
    if (w < full_tiles) { it.tile = w; it.part = 0; it.n_cols = 256; return it; }
    const int t = w - full_tiles;
    it.tile = full_tiles + t / tail_split;
    it.part = t - (t / tail_split) * tail_split;
    it.n_cols = 256 / tail_split;
    return it;
}

template <int KIND, int BN, int EPI>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b, const GemmParams p) {
    using C = Cfg<KIND, BN>;
    constexpr int S = C::kStages;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t sm_a = base;
    const uint32_t sm_b = sm_a + S * C::kABytes;
    const uint32_t sm_sfa = sm_b + S * C::kBBytes;
    const uint32_t sm_sfb = sm_sfa + S * C::kSfaBytes;
    const uint32_t sm_bar = sm_sfb + S * C::kSfbBytes;           // 8-byte aligned (all sizes are multiples of 512)
    const uint32_t bar_full = sm_bar, bar_empty = sm_bar + 8 * S;
    const uint32_t bar_tfull = sm_bar + 16 * S, bar_tempty = bar_tfull + 16;
    const uint32_t tmem_slot = bar_tempty + 16;
    uint32_t* tmem_slot_ptr = reinterpret_cast<uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_m = (p.m + BM - 1) / BM, tiles_n = (p.n + BN - 1) / BN;
    const int num_tiles = tiles_m * tiles_n;
    const int num_kb = (p.k_bytes + BKB - 1) / BKB;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; s++) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_empty + 8 * s, 1); }
        for (int a = 0; a < 2; a++) { mbar_init(bar_tfull + 8 * a, 1); mbar_init(bar_tempty + 8 * a, 4); }
        fence_barrier_init();
        prefetch_tmap(&tm_a);
        prefetch_tmap(&tm_b);
    }
    if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_ptr;
    pdl_trigger();                                               // barriers, tensor memory and descriptors are set up:
    pdl_wait();                                                  // only now wait for the kernel that produced the operands

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (whole warp, one elected lane issues)
        {
            int stage = 0; uint32_t phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                int tm, tn;
                tile_coords(tile, tiles_m, tiles_n, p.group_m, tm, tn);
                const int m0 = tm * BM, n0 = tn * BN;
                for (int kb = 0; kb < num_kb; kb++) {
                    if (!mbar_wait_warp(bar_empty + 8 * stage, phase ^ 1)) { ok = false; if (lane == 0) atomicExch(p.status, OXQ_ERR_DEVICE_TIMEOUT); break; }
                    const uint32_t full = bar_full + 8 * stage;
                    uint32_t bytes = C::kABytes + C::kBBytes;
                    if (C::kScaled) {
                        bytes += C::kSfaBytes;
                        const int rt0 = n0 >> 7;
                        bytes += (rt0 < p.sfb_row_tiles ? C::kSfaBytes : 0) + (rt0 + 1 < p.sfb_row_tiles ? C::kSfaBytes : 0);
                    }
                    if (elect_one()) {
                    mbar_arrive_expect_tx(full, bytes);
                    tma_load_2d(sm_a + stage * C::kABytes, &tm_a, kb * BKB, m0, full);
                    tma_load_2d(sm_b + stage * C::kBBytes, &tm_b, kb * BKB, n0, full);
                    if (C::kScaled) {
                        const size_t col_off = (size_t)kb * C::kSfaBytes;
                        const size_t row_stride = (size_t)p.sf_col_tiles * 512;
                        bulk_load(sm_sfa + stage * C::kSfaBytes, p.sfa + (size_t)(m0 >> 7) * row_stride + col_off, C::kSfaBytes, full);
                        const int rt0 = n0 >> 7;
                        if (rt0 < p.sfb_row_tiles)
                            bulk_load(sm_sfb + stage * C::kSfbBytes, p.sfb + (size_t)rt0 * row_stride + col_off, C::kSfaBytes, full);
                        if (rt0 + 1 < p.sfb_row_tiles)
                            bulk_load(sm_sfb + stage * C::kSfbBytes + C::kSfaBytes, p.sfb + (size_t)(rt0 + 1) * row_stride + col_off, C::kSfaBytes, full);
                    }
                    }
                    __syncwarp();
                    if (++stage == S) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (whole warp, one elected lane issues)
        {
            constexpr uint32_t idesc =
                KIND == KIND_F8 ? idesc_dense(1, 0, 0, BM, BN) :
                KIND == KIND_BF16 ? idesc_dense(1, 1, 1, BM, BN) :
                KIND == KIND_I8 ? idesc_dense(2, 1, 1, BM, BN) :
                KIND == KIND_MXF8 ? idesc_block_scaled(0, 0, 1, BM, BN) : idesc_block_scaled(1, 1, 0, BM, BN);
            int stage = 0; uint32_t phase = 0;
            int acc = 0; uint32_t acc_phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                int tm, tn;
                tile_coords(tile, tiles_m, tiles_n, p.group_m, tm, tn);
                const int n0 = tn * BN;
                if (!mbar_wait_warp(bar_tempty + 8 * acc, acc_phase ^ 1)) { ok = false; if (lane == 0) atomicExch(p.status, OXQ_ERR_DEVICE_TIMEOUT); break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * C::kAccStride;
                for (int kb = 0; kb < num_kb; kb++) {
                    if (!mbar_wait_warp(bar_full + 8 * stage, phase)) { ok = false; if (lane == 0) atomicExch(p.status, OXQ_ERR_DEVICE_TIMEOUT); break; }
                    tc_fence_after();
                    const uint64_t adesc = smem_desc_sw128(sm_a + stage * C::kABytes);
                    const uint64_t bdesc = smem_desc_sw128(sm_b + stage * C::kBBytes);
                    if (elect_one()) {
                    if (C::kScaled) {
#pragma unroll
                        for (int c = 0; c < C::kSfChunks; c++) {
                            tc_cp_32x128b_warpx4(tmem_base + C::kSfaCol + 4 * c, smem_desc_sf(sm_sfa + stage * C::kSfaBytes + c * 512));
                            // B scale factors: per K chunk, the two 128-row tiles side by side (8 columns = 256 rows)
                            tc_cp_32x128b_warpx4(tmem_base + C::kSfbCol + 8 * c, smem_desc_sf(sm_sfb + stage * C::kSfbBytes + c * 512));
                            tc_cp_32x128b_warpx4(tmem_base + C::kSfbCol + 8 * c + 4,
                                                 smem_desc_sf(sm_sfb + stage * C::kSfbBytes + C::kSfaBytes + c * 512));
                        }
                    }
#pragma unroll
                    for (int k = 0; k < BKB / 32; k++) {
                        // each MMA consumes 32 bytes of K: advance the start-address field by 32 >> 4
                        const uint64_t a = adesc + (uint64_t)(k * 2), b = bdesc + (uint64_t)(k * 2);
                        const uint32_t accum = (kb | k) != 0;
                        if (KIND == KIND_F8) mma_f8f6f4(d_tmem, a, b, idesc, accum);
                        else if (KIND == KIND_BF16) mma_f16(d_tmem, a, b, idesc, accum);
                        else if (KIND == KIND_I8) mma_i8(d_tmem, a, b, idesc, accum);
                        else {
                            // tile rows [n0, n0+BN) start (n0 % 128) / 32 row-groups into the first scale-factor tile
                            const uint32_t sfb_shift = (uint32_t)(n0 & 127) >> 5;
                            if (KIND == KIND_MXF8) {
                                // one scale per row and MMA: byte k of the chunk's 32-bit words
                                mma_mxf8f6f4(d_tmem, a, b, idesc_with_sf_ids(idesc, k, k), accum,
                                             tmem_base + C::kSfaCol, tmem_base + C::kSfbCol + sfb_shift);
                            } else {
                                // four scales per row and MMA: chunk k, all four bytes
                                mma_mxf4nvf4_x4(d_tmem, a, b, idesc, accum,
                                                tmem_base + C::kSfaCol + 4 * k, tmem_base + C::kSfbCol + 8 * k + sfb_shift);
                            }
                        }
                    }
                    tc_commit(bar_empty + 8 * stage);            // frees the stage once these MMAs have read it
                    }
                    __syncwarp();
                    if (++stage == S) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                if (elect_one()) tc_commit(bar_tfull + 8 * acc);  // accumulator complete
                __syncwarp();
                if (++acc == 2) { acc = 0; acc_phase ^= 1; }
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (4 warps)
        const int quarter = warp & 3;                            // tensor-memory lanes [32*quarter, +32)
        int acc = 0; uint32_t acc_phase = 0;
        float tensor_scale = 1.0f;
        if (KIND == KIND_F8 || KIND == KIND_NVF4) tensor_scale = __ldg(p.s0) * __ldg(p.s1);
        tensor_scale *= p.alpha;
        __nv_bfloat16* y = reinterpret_cast<__nv_bfloat16*>(p.y);
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
            int tm, tn;
            tile_coords(tile, tiles_m, tiles_n, p.group_m, tm, tn);
            const int m0 = tm * BM, n0 = tn * BN;
            bool ok = mbar_wait(bar_tfull + 8 * acc, acc_phase);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) { if (lane == 0) atomicExch(p.status, OXQ_ERR_DEVICE_TIMEOUT); break; }
            tc_fence_after();
            const int row = m0 + quarter * 32 + lane;
            const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * C::kAccStride;
            float row_scale = 1.0f;
            if (KIND == KIND_I8 && row < p.m) row_scale = __ldg(p.s0 + row) * p.alpha;
            if (EPI == EPI_SWIGLU) {
                // columns [0, BN/2) of the tile are gate, [BN/2, BN) the matching up columns
                const int out_n = p.n >> 1;
#pragma unroll 1
                for (int c = 0; c < BN / 64; c++) {
                    uint32_t rg[32], ru[32];
                    tmem_ld_32x32b_x32(t_row + c * 32, rg);
                    tmem_ld_32x32b_x32(t_row + BN / 2 + c * 32, ru);
                    tmem_ld_wait();
                    const int col0 = (n0 >> 1) + c * 32;
                    if (row < p.m && col0 < out_n) {
                        float v[32];
#pragma unroll
                        for (int j = 0; j < 32; j++) {
                            const float gt = __uint_as_float(rg[j]) * tensor_scale, up = __uint_as_float(ru[j]) * tensor_scale;
                            v[j] = __fdividef(gt, 1.0f + __expf(-gt)) * up;
                        }
                        __nv_bfloat16* dst = y + (size_t)row * p.ldy + col0;
                        if (col0 + 32 <= out_n) {
#pragma unroll
                            for (int j = 0; j < 4; j++) {
                                uint4 o;
                                __nv_bfloat162 t0 = __floats2bfloat162_rn(v[8 * j + 0], v[8 * j + 1]);
                                __nv_bfloat162 t1 = __floats2bfloat162_rn(v[8 * j + 2], v[8 * j + 3]);
                                __nv_bfloat162 t2 = __floats2bfloat162_rn(v[8 * j + 4], v[8 * j + 5]);
                                __nv_bfloat162 t3 = __floats2bfloat162_rn(v[8 * j + 6], v[8 * j + 7]);
                                o.x = *reinterpret_cast<uint32_t*>(&t0); o.y = *reinterpret_cast<uint32_t*>(&t1);
                                o.z = *reinterpret_cast<uint32_t*>(&t2); o.w = *reinterpret_cast<uint32_t*>(&t3);
                                *reinterpret_cast<uint4*>(dst + 8 * j) = o;
                            }
                        } else {
                            for (int j = 0; j < 32 && col0 + j < out_n; j++) dst[j] = __float2bfloat16_rn(v[j]);
                        }
                    }
                }
            } else {
#pragma unroll 1
                for (int c = 0; c < BN / 32; c++) {
                    uint32_t r[32];
                    tmem_ld_32x32b_x32(t_row + c * 32, r);
                    tmem_ld_wait();
                    epilogue_store_scale<KIND>(r, row, n0 + c * 32, p, tensor_scale, row_scale, y);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_tempty + 8 * acc);
            if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        }
    }

    // Teardown.  On the normal path the epilogue has seen the last accumulator complete, so every
    // MMA has finished and every TMA load has landed before tensor memory is released.
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

// ---- 2-CTA variant of the dense kinds --------------------------------------------------------------
// A cluster of two CTAs computes one 256 x 256 tile: CTA r loads rows [128r, 128r+128) of the X tile and
// rows [128r, 128r+128) of the W tile (so every operand byte is fetched by one CTA only and the W bytes per
// CTA halve), CTA 0 issues tcgen05.mma.cta_group::2 (M = 256 across the pair, N = 256), each CTA keeps its
// 128 accumulator rows in its own tensor memory and runs its own epilogue.  Full barriers live in CTA 0
// (both CTAs' TMA loads count bytes there), empty / accumulator-full barriers are signalled in both CTAs by
// a multicast commit, accumulator-empty arrivals go to CTA 0.
constexpr int T2_STAGES = 7;
constexpr int T2_STAGE_BYTES = 2 * BM * BKB;                      // 16 KB of X + 16 KB of W per CTA
constexpr int T2_SMEM_BYTES = T2_STAGES * T2_STAGE_BYTES + 2048;

// GENERIC = false is the K-major / K-major kernel; GENERIC = true reads the operands' major-ness from the parameters (the
// operand forms of gemm).  Two instantiations, so that the common form carries none of the other's address arithmetic.
// ---- all-reduce fused into the CTA-pair kernel (AR = true) ----------------------------------------------------------
// Every rank of a tensor-parallel group runs this kernel on its K-shard and writes its partial tiles into its replica of
// a symmetric buffer.  When an epilogue warp has stored its 32 rows of a tile it adds one to the tile's arrival word on
// every rank (multimem.red through the NVSwitch).  Tile w belongs to rank w % world: sixteen more warps per CTA, the
// reducers, take the owned tiles in strips of 8 rows, wait until every epilogue warp of every rank has arrived
// (8 * world), pull the sum of all replicas with multimem.ld_reduce (the switch adds in f32) and push it to every
// replica with multimem.st, then add one to the word of finished units on every rank.  CTA 0 leaves only when every
// unit of every rank is finished, so the kernel that follows in the stream finds the complete sum in its replica; it
// then clears this call's flag words (calls alternate between two sets of words, so a peer that is already a call
// ahead never meets a word that is still to be cleared).  The transfer of a tile overlaps the MMAs of the tiles after
// it; nothing waits on the reducers except the end of the kernel, and every wait is bounded.
constexpr int AR_WARPS = 16;                                       // reducer warps per CTA
constexpr int AR_THREADS = NUM_THREADS + 32 * AR_WARPS;

template <int KIND, int EPI, bool GENERIC = false, bool AR = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(AR ? AR_THREADS : NUM_THREADS, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b, const GemmParams p) {
    const bool a_mn = GENERIC && p.a_mn, b_mn = GENERIC && p.b_mn;
    constexpr int S = T2_STAGES;
    constexpr int BN2 = 256, BM2 = 256;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t sm_a = base;
    const uint32_t sm_b = sm_a + S * BM * BKB;
    const uint32_t sm_bar = sm_b + S * BM * BKB;
    const uint32_t bar_full = sm_bar, bar_empty = sm_bar + 8 * S;
    const uint32_t bar_tfull = sm_bar + 16 * S, bar_tempty = bar_tfull + 16;
    const uint32_t tmem_slot = bar_tempty + 16;
    uint32_t* tmem_slot_ptr = reinterpret_cast<uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t cta_rank = cluster_ctarank();
    const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;
    const int tiles_m = (p.m + BM2 - 1) / BM2, tiles_n = (p.n + BN2 - 1) / BN2;
    const int num_tiles = tiles_m * tiles_n;
    const int num_work = p.full_tiles + (num_tiles - p.full_tiles) * p.tail_split;
    const int num_kb = (p.k_bytes + BKB - 1) / BKB;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; s++) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_empty + 8 * s, 1); }
        for (int a = 0; a < 2; a++) { mbar_init(bar_tfull + 8 * a, 1); mbar_init(bar_tempty + 8 * a, 8); }
        fence_barrier_init();
        prefetch_tmap(&tm_a);
        prefetch_tmap(&tm_b);
    }
    if (warp == 1) { tmem_alloc_cg2(tmem_slot, 512); tmem_relinquish_cg2(); }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                                   // peer barriers are initialised and its tensor memory allocated
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_ptr;
    pdl_trigger();
    pdl_wait();
    // fused all-reduce: the set of flag words of this call.  The count of finished calls changes only when CTA 0 has seen every
    // unit of every rank finished, i.e. after every CTA of this grid has done its part, so all CTAs read the same value.
    uint32_t* ar_flags = nullptr; uint32_t* ar_mc_flags = nullptr;
    if (AR) {
        const uint32_t set = *reinterpret_cast<const volatile uint32_t*>(p.ar_calls) & 1u;
        ar_flags = p.ar_flags + set * p.ar_set_stride;
        ar_mc_flags = p.ar_mc_flags + set * p.ar_set_stride;
    }

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (whole warp, one elected lane issues; both CTAs)
        {
            int stage = 0; uint32_t phase = 0;
            bool ok = true;
            const int es_shift = p.esize == 2 ? 1 : 0;
            for (int w = cluster_id; w < num_work && ok; w += num_clusters) {
                const WorkItem wi = work_item(w, p.full_tiles, p.tail_split);
                int tm, tn;
                tile_coords(wi.tile, tiles_m, tiles_n, p.group_m, tm, tn);
                // this CTA's rows of W: its 128-row half of the tile, from the part's offset on (the 128-row box reads
                // past the part; the MMA uses the first n_cols / 2 rows)
                const int m0 = tm * BM2 + (int)cta_rank * BM, n0 = tn * BN2 + (int)cta_rank * BM + wi.part * (wi.n_cols >> 1);
                for (int kb = 0; kb < num_kb; kb++) {
                    if (!mbar_wait_warp(bar_empty + 8 * stage, phase ^ 1)) { ok = false; if (lane == 0) atomicExch(p.status, OXQ_ERR_DEVICE_TIMEOUT); break; }
                    const uint32_t full0 = mapa_shared(bar_full + 8 * stage, 0);
                    if (elect_one()) {
                    // the full barrier of the pair lives in CTA 0 and expects the bytes of both CTAs
                    if (cta_rank == 0) mbar_arrive_expect_tx(bar_full + 8 * stage, 2 * T2_STAGE_BYTES);
                    // K-major operand: one box of 128 rows x 128 bytes of K.  MN-major operand ([K x M] / [K x N] in memory):
                    // `esize` boxes of (128 / esize) K rows x 128 bytes of M / N, one swizzle atom each, side by side
                    // (esize is 1 or 2: the shifts below are the divisions by it).
                    if (!a_mn) tma_load_2d_cg2(sm_a + stage * BM * BKB, &tm_a, kb * BKB, m0, full0);
                    else for (int j = 0; j < p.esize; j++)
                        tma_load_2d_cg2(sm_a + stage * BM * BKB + j * ((BM * BKB) >> es_shift), &tm_a, (m0 << es_shift) + j * 128, kb * (BKB >> es_shift), full0);
                    if (!b_mn) tma_load_2d_cg2(sm_b + stage * BM * BKB, &tm_b, kb * BKB, n0, full0);
                    else for (int j = 0; j < p.esize; j++)
                        tma_load_2d_cg2(sm_b + stage * BM * BKB + j * ((BM * BKB) >> es_shift), &tm_b, (n0 << es_shift) + j * 128, kb * (BKB >> es_shift), full0);
                    }
                    __syncwarp();
                    if (++stage == S) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (warp 1 of CTA 0, one elected lane issues)
        if (cta_rank == 0) {
            constexpr uint32_t cf = KIND == KIND_I8 ? 2 : 1, af = KIND == KIND_F8 ? 0 : 1;
            int stage = 0; uint32_t phase = 0;
            int acc = 0; uint32_t acc_phase = 0;
            bool ok = true;
            // Per MMA (32 bytes of K) the start address moves 32 bytes along a K-major row, or 32 / esize rows of 128 bytes
            // (whole 1024-byte row groups) down an MN-major tile; an MN-major tile wider than 128 bytes is `esize` atoms apart
            // by the leading byte offset.  All of it is fixed per launch and kept out of the issue loop.
            const uint32_t es_shift = p.esize == 2 ? 1u : 0u;
            const uint32_t atom = (uint32_t)(BM * BKB) >> es_shift;
            const uint32_t ka = a_mn ? ((4096u >> es_shift) >> 4) : 2u, kbs = b_mn ? ((4096u >> es_shift) >> 4) : 2u;
            const uint64_t a_fixed = a_mn ? (smem_desc_mn_sw128(0, atom)) : smem_desc_sw128(0);
            const uint64_t b_fixed = b_mn ? (smem_desc_mn_sw128(0, atom)) : smem_desc_sw128(0);
            const uint32_t majors = idesc_majors((uint32_t)a_mn, (uint32_t)b_mn);
            for (int w = cluster_id; w < num_work && ok; w += num_clusters) {
                const uint32_t idesc = idesc_dense(cf, af, af, BM2, (uint32_t)work_item(w, p.full_tiles, p.tail_split).n_cols) | majors;
                if (!mbar_wait_warp(bar_tempty + 8 * acc, acc_phase ^ 1)) { ok = false; if (lane == 0) atomicExch(p.status, OXQ_ERR_DEVICE_TIMEOUT); break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN2;
                for (int kb = 0; kb < num_kb; kb++) {
                    if (!mbar_wait_warp(bar_full + 8 * stage, phase)) { ok = false; if (lane == 0) atomicExch(p.status, OXQ_ERR_DEVICE_TIMEOUT); break; }
                    tc_fence_after();
                    // descriptor = the launch's fixed fields + the stage's start address (bits [0, 14), in units of 16 bytes)
                    const uint64_t adesc = a_fixed | (uint64_t)(((sm_a + stage * BM * BKB) & 0x3FFFFu) >> 4);
                    const uint64_t bdesc = b_fixed | (uint64_t)(((sm_b + stage * BM * BKB) & 0x3FFFFu) >> 4);
                    if (elect_one()) {
#pragma unroll
                    for (int k = 0; k < BKB / 32; k++) {
                        const uint64_t a = adesc + (uint64_t)(k * ka), b = bdesc + (uint64_t)(k * kbs);
                        const uint32_t accum = (kb | k) != 0;
                        if (KIND == KIND_F8) mma_f8f6f4_cg2(d_tmem, a, b, idesc, accum);
                        else if (KIND == KIND_BF16) mma_f16_cg2(d_tmem, a, b, idesc, accum);
                        else mma_i8_cg2(d_tmem, a, b, idesc, accum);
                    }
                    tc_commit_cg2_mc(bar_empty + 8 * stage, 3);          // frees the stage in both CTAs
                    }
                    __syncwarp();
                    if (++stage == S) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                if (elect_one()) tc_commit_cg2_mc(bar_tfull + 8 * acc, 3);   // accumulator complete, both CTAs
                __syncwarp();
                if (++acc == 2) { acc = 0; acc_phase ^= 1; }
            }
        }
    } else if (!AR || warp < 6) {
        // ------------------------------------------------------------------ epilogue (4 warps, both CTAs)
        const int quarter = warp & 3;
        int acc = 0; uint32_t acc_phase = 0;
        float tensor_scale = 1.0f;
        if (KIND == KIND_F8) tensor_scale = __ldg(p.s0) * __ldg(p.s1);
        tensor_scale *= p.alpha;
        __nv_bfloat16* y = reinterpret_cast<__nv_bfloat16*>(p.y);
        for (int w = cluster_id; w < num_work; w += num_clusters) {
            const WorkItem wi = work_item(w, p.full_tiles, p.tail_split);
            int tm, tn;
            tile_coords(wi.tile, tiles_m, tiles_n, p.group_m, tm, tn);
            const int m0 = tm * BM2 + (int)cta_rank * BM, n0 = tn * BN2;
            const int half = wi.n_cols >> 1;                 // accumulator columns [0, half) come from CTA 0's rows of W, [half, n_cols) from CTA 1's
            bool ok = mbar_wait(bar_tfull + 8 * acc, acc_phase);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) { if (lane == 0) atomicExch(p.status, OXQ_ERR_DEVICE_TIMEOUT); break; }
            tc_fence_after();
            const int row = m0 + quarter * 32 + lane;
            const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN2;
            float row_scale = 1.0f;
            if (KIND == KIND_I8 && row < p.m) row_scale = __ldg(p.s0 + row) * p.alpha;
            if (EPI == EPI_SWIGLU) {
#pragma unroll 1
                for (int c = 0; c < half / 32; c++) {
                    uint32_t rg[32], ru[32];
                    tmem_ld_32x32b_x32(t_row + c * 32, rg);
                    tmem_ld_32x32b_x32(t_row + half + c * 32, ru);
                    tmem_ld_wait();
                    epilogue_store_swiglu(rg, ru, row, (n0 >> 1) + wi.part * half + c * 32, p.n >> 1, p, tensor_scale, y);
                }
            } else {
#pragma unroll 1
                for (int c = 0; c < wi.n_cols / 32; c++) {
                    uint32_t r[32];
                    tmem_ld_32x32b_x32(t_row + c * 32, r);
                    tmem_ld_wait();
                    const int cc = c * 32;
                    const int col0 = cc < half ? n0 + wi.part * half + cc : n0 + BM + wi.part * half + (cc - half);
                    epilogue_store_scale<KIND>(r, row, col0, p, tensor_scale, row_scale, y);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(mapa_shared(bar_tempty + 8 * acc, 0));
            if (++acc == 2) { acc = 0; acc_phase ^= 1; }
            if (AR) {
                // this warp's 32 rows of the tile are stored: one arrival on every rank (lane 0's release, after the warp
                // has met, covers the stores of all its lanes)
                if (lane == 0) mm_red_add_u32(ar_mc_flags + w, 1u);
            }
        }
    } else {
        // ------------------------------------------------------------------ reducers (AR only: 16 warps, both CTAs)
        // A unit is a strip of 8 rows x 256 columns of an owned tile; the reducer warps of the whole grid take the
        // units in order, each warp on its own (no CTA-wide meeting point anywhere in this role).
        const int world = p.ar_world;
        const int owned = num_work > p.ar_rank ? (num_work - p.ar_rank + world - 1) / world : 0;   // items w = rank, rank + world, ...
        const int units = owned * 32;
        const uint32_t arrive_target = 8u * (uint32_t)world;            // 2 CTAs x 4 epilogue warps per rank
        char* mc_y = reinterpret_cast<char*>(p.ar_mc_y);
        bool ok = true;
        for (int u = (int)blockIdx.x * AR_WARPS + (warp - 6); u < units && ok; u += (int)gridDim.x * AR_WARPS) {
            const int w = (u >> 5) * world + p.ar_rank, strip = u & 31;
            int tm, tn;
            tile_coords(w, tiles_m, tiles_n, p.group_m, tm, tn);
            if (lane == 0) ok = wait_word_at_least(ar_flags + w, arrive_target, p.ar_sleep_ns);
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) { if (lane == 0) atomicExch(p.status, OXQ_ERR_DEVICE_TIMEOUT); break; }
            // 8 rows x 256 columns of bf16 = 8 x 32 vectors of 16 bytes: eight vectors in flight per lane, one round trip
            const int row0 = tm * BM2 + strip * 8, col0 = tn * BN2 + (lane << 3);
            uint4 val[8];
            const bool col_in = col0 < p.n;
#pragma unroll
            for (int j = 0; j < 8; j++)
                if (col_in && row0 + j < p.m) val[j] = mm_ld_reduce_bf16x8(mc_y + ((size_t)(row0 + j) * p.ldy + col0) * 2);
#pragma unroll
            for (int j = 0; j < 8; j++)
                if (col_in && row0 + j < p.m) mm_st_bf16x8(mc_y + ((size_t)(row0 + j) * p.ldy + col0) * 2, val[j]);
            __syncwarp();
            if (lane == 0) mm_red_add_u32(ar_mc_flags + num_work, 1u);
        }
        if (blockIdx.x == 0 && warp == 6) {
            // the last to leave: every unit of every rank is finished (32 per item), then this call's words are cleared
            if (lane == 0 && ok && !wait_word_at_least(ar_flags + num_work, 32u * (uint32_t)num_work, p.ar_sleep_ns)) atomicExch(p.status, OXQ_ERR_DEVICE_TIMEOUT);
            __syncwarp();
            for (int i = lane; i <= num_work; i += 32) ar_flags[i] = 0u;
            __threadfence_system();
            __syncwarp();
            if (lane == 0) *reinterpret_cast<volatile uint32_t*>(p.ar_calls) = *reinterpret_cast<const volatile uint32_t*>(p.ar_calls) + 1u;
        }
    }

    // Teardown: both CTAs are past every access to the peer's barriers, shared and tensor memory before
    // either frees its tensor memory or exits.
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc_cg2(tmem_base, 512);
    }
}

// ---- 2-CTA variant of the block-scaled kinds -------------------------------------------------------
// Tile = 256 (M, two CTAs) x 192 (N).  CTA r loads rows [128r, +128) of the X tile with their scale chunks, rows
// [96r, +96) of the W tile, and the scale chunks of both 128-row W tiles that cover the 192 columns (every CTA
// needs the B scales of all columns).  CTA 0 issues tcgen05.cp.cta_group::2 (each CTA copies its own scale
// chunks into its own tensor memory) and tcgen05.mma.cta_group::2.  Tensor memory per CTA: accumulators at
// columns 0 and 256 (192 wide), A scales at 448, B scales at 464.  Scale factors travel as TMA tiles of
// 512-byte chunks (a [chunks x 128] u32 view of the tiled scale array) so that, like the operands, they can
// count their bytes on CTA 0's barrier.
// Two tile shapes.  256 x 192: two accumulators of 192 columns (the epilogue of a tile runs under the main loop of the next),
// scale factors behind them.  256 x 256: every operand byte in shared memory feeds twice as many MMA columns per byte of W as
// it costs to bring in (the shared-memory traffic per MMA cycle is what limits the 4-bit kind), but tensor memory then holds
// one accumulator only (256 + 48 scale columns), so the main loop of the next tile waits for the epilogue; the epilogue is
// spread over eight warps (two per lane quarter, 128 columns each) to keep that wait short.
template <int KIND, int BN2_>
struct Cfg2S {
    static constexpr int kSfChunks = KIND == KIND_MXF8 ? 1 : 4;
    static constexpr int kSfBytes = kSfChunks * 512;
    static constexpr int BN2 = BN2_;
    static constexpr int kAcc = BN2 == 256 ? 1 : 2;                                // accumulator buffers
    static constexpr int kEpiWarps = BN2 == 256 ? 8 : 4;
    static constexpr int kThreads = 32 * (2 + kEpiWarps);
    static constexpr int kABytes = BM * BKB, kBBytes = (BN2 / 2) * BKB;
    static constexpr int kStageBytes = kABytes + kBBytes + 3 * kSfBytes;           // A, B half, SFA, 2 x SFB
    static constexpr int kStages = (SMEM_BUDGET - 2048) / kStageBytes > 8 ? 8 : (SMEM_BUDGET - 2048) / kStageBytes;
    static constexpr int kSmemBytes = kStages * kStageBytes + 2048;
    static constexpr int kSfaCol = BN2 == 256 ? 256 : 448, kSfbCol = kSfaCol + 16;
    static_assert(BN2 == 192 || BN2 == 256, "tile widths of the CTA-pair block-scaled kernel");
};

template <int KIND, int BN2_>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(Cfg2S<KIND, BN2_>::kThreads, 1)
gemm_tc2_scaled_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                       const __grid_constant__ CUtensorMap tm_sfa, const __grid_constant__ CUtensorMap tm_sfb, const GemmParams p) {
    using C = Cfg2S<KIND, BN2_>;
    constexpr int S = C::kStages;
    constexpr int BN2 = C::BN2, BM2 = 256;
    constexpr int ACC = C::kAcc, EW = C::kEpiWarps;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t sm_a = base;
    const uint32_t sm_b = sm_a + S * C::kABytes;
    const uint32_t sm_sfa = sm_b + S * C::kBBytes;
    const uint32_t sm_sfb = sm_sfa + S * C::kSfBytes;
    const uint32_t sm_bar = sm_sfb + S * 2 * C::kSfBytes;
    const uint32_t bar_full = sm_bar, bar_empty = sm_bar + 8 * S;
    const uint32_t bar_tfull = sm_bar + 16 * S, bar_tempty = bar_tfull + 16;
    const uint32_t tmem_slot = bar_tempty + 16;
    uint32_t* tmem_slot_ptr = reinterpret_cast<uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t cta_rank = cluster_ctarank();
    const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;
    const int tiles_m = (p.m + BM2 - 1) / BM2, tiles_n = (p.n + BN2 - 1) / BN2;
    const int num_tiles = tiles_m * tiles_n;
    const int num_kb = (p.k_bytes + BKB - 1) / BKB;

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; s++) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_empty + 8 * s, 1); }
        for (int a = 0; a < 2; a++) { mbar_init(bar_tfull + 8 * a, 1); mbar_init(bar_tempty + 8 * a, 2 * EW); }
        fence_barrier_init();
        prefetch_tmap(&tm_a); prefetch_tmap(&tm_b); prefetch_tmap(&tm_sfa); prefetch_tmap(&tm_sfb);
    }
    if (warp == 1) { tmem_alloc_cg2(tmem_slot, 512); tmem_relinquish_cg2(); }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_ptr;
    pdl_trigger();
    pdl_wait();

    if (warp == 0) {
        {                                                         // whole warp; one elected lane issues
            int stage = 0; uint32_t phase = 0;
            bool ok = true;
            for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
                int tm, tn;
                tile_coords(tile, tiles_m, tiles_n, p.group_m, tm, tn);
                const int m0 = tm * BM2 + (int)cta_rank * BM, n0 = tn * BN2;
                const int sfa_row = (m0 >> 7) * p.sf_col_tiles, sfb_row = (n0 >> 7) * p.sf_col_tiles;
                for (int kb = 0; kb < num_kb; kb++) {
                    if (!mbar_wait_warp(bar_empty + 8 * stage, phase ^ 1)) { ok = false; if (lane == 0) atomicExch(p.status, OXQ_ERR_DEVICE_TIMEOUT); break; }
                    const uint32_t full0 = mapa_shared(bar_full + 8 * stage, 0);
                    if (elect_one()) {
                    if (cta_rank == 0) mbar_arrive_expect_tx(bar_full + 8 * stage, 2 * C::kStageBytes);
                    tma_load_2d_cg2(sm_a + stage * C::kABytes, &tm_a, kb * BKB, m0, full0);
                    tma_load_2d_cg2(sm_b + stage * C::kBBytes, &tm_b, kb * BKB, n0 + (int)cta_rank * (BN2 / 2), full0);
                    // scale chunks: rows of the [chunk x 128 u32] view; rows past the end read as zero
                    tma_load_2d_cg2(sm_sfa + stage * C::kSfBytes, &tm_sfa, 0, sfa_row + kb * C::kSfChunks, full0);
                    tma_load_2d_cg2(sm_sfb + stage * 2 * C::kSfBytes, &tm_sfb, 0, sfb_row + kb * C::kSfChunks, full0);
                    tma_load_2d_cg2(sm_sfb + stage * 2 * C::kSfBytes + C::kSfBytes, &tm_sfb, 0, sfb_row + p.sf_col_tiles + kb * C::kSfChunks, full0);
                    }
                    __syncwarp();
                    if (++stage == S) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        if (cta_rank == 0) {                                      // whole warp; one elected lane issues
            constexpr uint32_t idesc = KIND == KIND_MXF8 ? idesc_block_scaled(0, 0, 1, BM2, BN2) : idesc_block_scaled(1, 1, 0, BM2, BN2);
            int stage = 0; uint32_t phase = 0;
            int acc = 0; uint32_t acc_phase = 0;
            bool ok = true;
            for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
                int tm, tn;
                tile_coords(tile, tiles_m, tiles_n, p.group_m, tm, tn);
                const uint32_t sfb_shift = (uint32_t)((tn * BN2) & 127) >> 5;       // 0 or 2: odd tiles start 64 rows into a scale tile
                if (!mbar_wait_warp(bar_tempty + 8 * acc, acc_phase ^ 1)) { ok = false; if (lane == 0) atomicExch(p.status, OXQ_ERR_DEVICE_TIMEOUT); break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * 256;
                for (int kb = 0; kb < num_kb; kb++) {
                    if (!mbar_wait_warp(bar_full + 8 * stage, phase)) { ok = false; if (lane == 0) atomicExch(p.status, OXQ_ERR_DEVICE_TIMEOUT); break; }
                    tc_fence_after();
                    const uint64_t adesc = smem_desc_sw128(sm_a + stage * C::kABytes);
                    const uint64_t bdesc = smem_desc_sw128(sm_b + stage * C::kBBytes);
                    if (elect_one()) {
#pragma unroll
                    for (int c = 0; c < C::kSfChunks; c++) {
                        tc_cp_32x128b_warpx4_cg2(tmem_base + C::kSfaCol + 4 * c, smem_desc_sf(sm_sfa + stage * C::kSfBytes + c * 512));
                        tc_cp_32x128b_warpx4_cg2(tmem_base + C::kSfbCol + 8 * c, smem_desc_sf(sm_sfb + stage * 2 * C::kSfBytes + c * 512));
                        tc_cp_32x128b_warpx4_cg2(tmem_base + C::kSfbCol + 8 * c + 4, smem_desc_sf(sm_sfb + stage * 2 * C::kSfBytes + C::kSfBytes + c * 512));
                    }
#pragma unroll
                    for (int k = 0; k < BKB / 32; k++) {
                        const uint64_t a = adesc + (uint64_t)(k * 2), b = bdesc + (uint64_t)(k * 2);
                        const uint32_t accum = (kb | k) != 0;
                        if (KIND == KIND_MXF8)
                            mma_mxf8f6f4_cg2(d_tmem, a, b, idesc_with_sf_ids(idesc, k, k), accum, tmem_base + C::kSfaCol, tmem_base + C::kSfbCol + sfb_shift);
                        else
                            mma_mxf4nvf4_x4_cg2(d_tmem, a, b, idesc, accum, tmem_base + C::kSfaCol + 4 * k, tmem_base + C::kSfbCol + 8 * k + sfb_shift);
                    }
                    tc_commit_cg2_mc(bar_empty + 8 * stage, 3);
                    }
                    __syncwarp();
                    if (++stage == S) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                if (elect_one()) tc_commit_cg2_mc(bar_tfull + 8 * acc, 3);
                __syncwarp();
                if (++acc == ACC) { acc = 0; acc_phase ^= 1; }
            }
        }
    } else {
        const int quarter = warp & 3;
        // with eight epilogue warps, warps 2-5 take the first half of the tile's columns and warps 6-9 the second
        const int col_lo = EW == 8 ? ((warp - 2) >> 2) * (BN2 / 2) : 0, col_hi = EW == 8 ? col_lo + BN2 / 2 : BN2;
        int acc = 0; uint32_t acc_phase = 0;
        float tensor_scale = 1.0f;
        if (KIND == KIND_NVF4) tensor_scale = __ldg(p.s0) * __ldg(p.s1);
        tensor_scale *= p.alpha;
        __nv_bfloat16* y = reinterpret_cast<__nv_bfloat16*>(p.y);
        for (int tile = cluster_id; tile < num_tiles; tile += num_clusters) {
            int tm, tn;
            tile_coords(tile, tiles_m, tiles_n, p.group_m, tm, tn);
            const int m0 = tm * BM2 + (int)cta_rank * BM, n0 = tn * BN2;
            bool ok = mbar_wait(bar_tfull + 8 * acc, acc_phase);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) { if (lane == 0) atomicExch(p.status, OXQ_ERR_DEVICE_TIMEOUT); break; }
            tc_fence_after();
            const int row = m0 + quarter * 32 + lane;
            const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * 256;
#pragma unroll 1
            for (int c = col_lo / 32; c < col_hi / 32; c++) {
                uint32_t r[32];
                tmem_ld_32x32b_x32(t_row + c * 32, r);
                tmem_ld_wait();
                epilogue_store_scale<KIND_F8>(r, row, n0 + c * 32, p, tensor_scale, 1.0f, y);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(mapa_shared(bar_tempty + 8 * acc, 0));
            if (++acc == ACC) { acc = 0; acc_phase ^= 1; }
        }
    }

    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc_cg2(tmem_base, 512);
    }
}

// ---- host side ----------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &p, 12000, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// Row-major byte matrix [rows x row_bytes] with leading dimension ld_bytes, tiles of box_rows x 128 bytes.
static bool make_tmap_bytes(CUtensorMap* tm, const void* ptr, int64_t rows, int64_t row_bytes, int64_t ld_bytes, int box_rows) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)row_bytes, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld_bytes};
    cuuint32_t box[2] = {(cuuint32_t)BKB, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    return fn(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace tc
}  // namespace oxq

bool oxq_make_tmap_2d(CUtensorMap* tm, CUtensorMapDataType dtype, const void* ptr, uint64_t inner_elems, uint64_t rows,
                      uint64_t ld_bytes, uint32_t box_inner, uint32_t box_rows, CUtensorMapSwizzle swizzle) {
    oxq::tc::EncodeTiledFn fn = oxq::tc::get_encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)inner_elems, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld_bytes};
    cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    return fn(tm, dtype, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

namespace oxq {
namespace tc {

// M-tiles per rasterisation group; OXQ_GEMM_GROUP_M overrides the default for tuning runs.
static int group_m_setting() {
    static int v = 0;
    if (v == 0) {
        const char* e = getenv("OXQ_GEMM_GROUP_M");
        v = e ? atoi(e) : 32;
        if (v < 1) v = 1;
    }
    return v;
}

template <int KIND, int BN, int EPI = EPI_SCALE>
static int32_t launch(oxq_handle* h, const void* x, int64_t ldx_bytes, const void* w, int64_t ldw_bytes, GemmParams p) {
    using C = Cfg<KIND, BN>;
    CUtensorMap tm_a, tm_b;
    if (!make_tmap_bytes(&tm_a, x, p.m, p.k_bytes, ldx_bytes, BM) || !make_tmap_bytes(&tm_b, w, p.n, p.k_bytes, ldw_bytes, BN))
        OXQ_FAIL(h, OXQ_ERR_LAUNCH_FAILED, "cuTensorMapEncodeTiled failed (pointers must be 16-byte aligned, leading dimensions multiples of 16 bytes)");
    static OxqPerDevice attr_set;
    if (!attr_set.get(h->device)) {
        OXQ_CUDA(h, cudaFuncSetAttribute(gemm_tc_kernel<KIND, BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
        attr_set.set(h->device, 1);
    }
    const int tiles = ((p.m + BM - 1) / BM) * ((p.n + BN - 1) / BN);
    const int grid = tiles < h->sm_count ? tiles : h->sm_count;
    p.status = h->dev_status;
    p.group_m = group_m_setting();
    oxq_launch(gemm_tc_kernel<KIND, BN, EPI>, grid, NUM_THREADS, C::kSmemBytes, h->stream, tm_a, tm_b, p);
    OXQ_LAUNCH_CHECK(h);
    return OXQ_OK;
}

// 2-CTA launch: one cluster per pair of SMs.  OXQ_GEMM_2CTA=0 falls back to the 1-CTA kernel (for A/B runs).
static bool use_2cta_setting() {
    static int v = -1;
    if (v < 0) { const char* e = getenv("OXQ_GEMM_2CTA"); v = e ? (atoi(e) != 0) : 1; }
    return v != 0;
}

template <int KIND, int EPI = EPI_SCALE, bool GENERIC = false>
static int32_t launch2(oxq_handle* h, const void* x, int64_t ldx_bytes, const void* w, int64_t ldw_bytes, GemmParams p) {
    CUtensorMap tm_a, tm_b;
    if (p.esize != 2) p.esize = 1;
    // K-major: byte matrix [rows x K bytes], boxes of 128 rows x 128 bytes.  MN-major: byte matrix [K x rows * esize],
    // boxes of (128 / esize) K rows x 128 bytes.
    const int64_t k_elems = p.k_bytes / p.esize;
    const bool ok_a = p.a_mn ? make_tmap_bytes(&tm_a, x, k_elems, (int64_t)p.m * p.esize, ldx_bytes, BKB / p.esize)
                             : make_tmap_bytes(&tm_a, x, p.m, p.k_bytes, ldx_bytes, BM);
    const bool ok_b = p.b_mn ? make_tmap_bytes(&tm_b, w, k_elems, (int64_t)p.n * p.esize, ldw_bytes, BKB / p.esize)
                             : make_tmap_bytes(&tm_b, w, p.n, p.k_bytes, ldw_bytes, BM);
    if (!ok_a || !ok_b)
        OXQ_FAIL(h, OXQ_ERR_LAUNCH_FAILED, "cuTensorMapEncodeTiled failed (pointers must be 16-byte aligned, leading dimensions multiples of 16 bytes)");
    static OxqPerDevice cluster_cache;
    int max_clusters = cluster_cache.get(h->device);
    if (max_clusters == 0) {
        OXQ_CUDA(h, cudaFuncSetAttribute(gemm_tc2_kernel<KIND, EPI, GENERIC>, cudaFuncAttributeMaxDynamicSharedMemorySize, T2_SMEM_BYTES));
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(h->sm_count & ~1, 1, 1);
        cfg.blockDim = dim3(NUM_THREADS, 1, 1);
        cfg.dynamicSmemBytes = T2_SMEM_BYTES;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
        cfg.attrs = &attr; cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, gemm_tc2_kernel<KIND, EPI, GENERIC>, &cfg) != cudaSuccess || n < 1) n = h->sm_count / 2;
        max_clusters = n < h->sm_count / 2 ? n : h->sm_count / 2;
        cluster_cache.set(h->device, max_clusters);
    }
    const int tiles = ((p.m + 255) / 256) * ((p.n + 255) / 256);
    // The last wave: r tiles for max_clusters pairs.  Each of them is cut along N into up to four parts (64 accumulator
    // columns at least) so that the idle pairs take a share; OXQ_GEMM_TAIL_SPLIT caps the number of parts (1 = off).
    static int split_cap = 0;
    if (split_cap == 0) { const char* e = getenv("OXQ_GEMM_TAIL_SPLIT"); split_cap = e ? atoi(e) : 4; if (split_cap < 1) split_cap = 1; if (split_cap > 4) split_cap = 4; }
    int clusters, full, split = 1;
    if (tiles >= max_clusters) { clusters = max_clusters; full = (tiles / clusters) * clusters; } else { clusters = tiles; full = 0; }
    const int rest = tiles - full;
    if (rest > 0) {
        int sp = max_clusters / rest;
        if (sp > split_cap) sp = split_cap;
        if (sp >= 4) split = 4; else if (sp >= 2) split = 2;
        if (tiles < max_clusters) clusters = rest * split;
    }
    p.full_tiles = full; p.tail_split = split;
    p.status = h->dev_status;
    p.group_m = group_m_setting() / 2 > 0 ? group_m_setting() / 2 : 1;     // same panel height in rows as the 1-CTA walk
    oxq_launch(gemm_tc2_kernel<KIND, EPI, GENERIC>, 2 * clusters, NUM_THREADS, T2_SMEM_BYTES, h->stream, tm_a, tm_b, p);
    OXQ_LAUNCH_CHECK(h);
    return OXQ_OK;
}

// The CTA-pair FP8 kernel with the all-reduce fused in (whole 256 x 256 tiles only: no split of the last wave).
static int32_t launch2_ar(oxq_handle* h, const void* x, int64_t ldx_bytes, const void* w, int64_t ldw_bytes, GemmParams p) {
    CUtensorMap tm_a, tm_b;
    p.esize = 1; p.a_mn = 0; p.b_mn = 0;
    if (!make_tmap_bytes(&tm_a, x, p.m, p.k_bytes, ldx_bytes, BM) || !make_tmap_bytes(&tm_b, w, p.n, p.k_bytes, ldw_bytes, BM))
        OXQ_FAIL(h, OXQ_ERR_LAUNCH_FAILED, "cuTensorMapEncodeTiled failed (pointers must be 16-byte aligned, leading dimensions multiples of 16 bytes)");
    auto kernel = gemm_tc2_kernel<KIND_F8, EPI_SCALE, false, true>;
    static OxqPerDevice cluster_cache;
    int max_clusters = cluster_cache.get(h->device);
    if (max_clusters == 0) {
        OXQ_CUDA(h, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, T2_SMEM_BYTES));
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(h->sm_count & ~1, 1, 1);
        cfg.blockDim = dim3(AR_THREADS, 1, 1);
        cfg.dynamicSmemBytes = T2_SMEM_BYTES;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
        cfg.attrs = &attr; cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n < 1)
            OXQ_FAIL(h, OXQ_ERR_LAUNCH_FAILED, "the fused all-reduce kernel does not fit this device");
        max_clusters = n < h->sm_count / 2 ? n : h->sm_count / 2;
        cluster_cache.set(h->device, max_clusters);
    }
    const int tiles = ((p.m + 255) / 256) * ((p.n + 255) / 256);
    const int clusters = tiles < max_clusters ? tiles : max_clusters;
    p.full_tiles = tiles; p.tail_split = 1;
    p.status = h->dev_status;
    p.group_m = group_m_setting() / 2 > 0 ? group_m_setting() / 2 : 1;
    // Every CTA of the grid has to be resident (the reducers of one rank serve the epilogues of all ranks): the grid is
    // at most one cluster per SM pair, and the launch is plain stream order, without an early start under the kernel before.
    oxq_launch<false>(kernel, 2 * clusters, AR_THREADS, T2_SMEM_BYTES, h->stream, tm_a, tm_b, p);
    OXQ_LAUNCH_CHECK(h);
    return OXQ_OK;
}

// Dense kinds: 256 x 256 tiles on CTA pairs when there are at least two 128-row tiles of X, else 128 x 256.
template <int KIND, int EPI = EPI_SCALE>
static int32_t launch_dense(oxq_handle* h, const void* x, int64_t ldx_bytes, const void* w, int64_t ldw_bytes, const GemmParams& p) {
    if (use_2cta_setting() && p.m > 128) return launch2<KIND, EPI>(h, x, ldx_bytes, w, ldw_bytes, p);
    // One 128-row tile of X (decode shapes): the weight stream is the whole cost, so narrow tiles are used to
    // spread it over all SMs (N = 8192 gives 128 tiles of 64 columns instead of 32 of 256).
    if (EPI == EPI_SCALE && p.m <= 128 && (p.n + 255) / 256 < 2 * h->sm_count) return launch<KIND, 64, EPI_SCALE>(h, x, ldx_bytes, w, ldw_bytes, p);
    return launch<KIND, 256, EPI>(h, x, ldx_bytes, w, ldw_bytes, p);
}

// [chunks x 128] u32 view of a tiled scale-factor array: one row per 512-byte chunk, box = `box_chunks` rows.
static bool make_tmap_sf(CUtensorMap* tm, const void* ptr, int64_t total_chunks, int box_chunks) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {128, (cuuint64_t)total_chunks};
    cuuint64_t strides[1] = {512};
    cuuint32_t box[2] = {128, (cuuint32_t)box_chunks};
    cuuint32_t estr[2] = {1, 1};
    return fn(tm, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int KIND, int BN2_>
static int32_t launch2_scaled(oxq_handle* h, const void* x, int64_t ldx_bytes, const void* w, int64_t ldw_bytes, GemmParams p) {
    using C = Cfg2S<KIND, BN2_>;
    CUtensorMap tm_a, tm_b, tm_sfa, tm_sfb;
    if (!make_tmap_bytes(&tm_a, x, p.m, p.k_bytes, ldx_bytes, BM) || !make_tmap_bytes(&tm_b, w, p.n, p.k_bytes, ldw_bytes, C::BN2 / 2) ||
        !make_tmap_sf(&tm_sfa, p.sfa, (int64_t)p.sfa_row_tiles * p.sf_col_tiles, C::kSfChunks) ||
        !make_tmap_sf(&tm_sfb, p.sfb, (int64_t)p.sfb_row_tiles * p.sf_col_tiles, C::kSfChunks))
        OXQ_FAIL(h, OXQ_ERR_LAUNCH_FAILED, "cuTensorMapEncodeTiled failed (pointers must be 16-byte aligned, leading dimensions multiples of 16 bytes)");
    static OxqPerDevice cluster_cache;
    int max_clusters = cluster_cache.get(h->device);
    if (max_clusters == 0) {
        OXQ_CUDA(h, cudaFuncSetAttribute(gemm_tc2_scaled_kernel<KIND, BN2_>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(h->sm_count & ~1, 1, 1);
        cfg.blockDim = dim3(C::kThreads, 1, 1);
        cfg.dynamicSmemBytes = C::kSmemBytes;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
        cfg.attrs = &attr; cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, gemm_tc2_scaled_kernel<KIND, BN2_>, &cfg) != cudaSuccess || n < 1) n = h->sm_count / 2;
        max_clusters = n < h->sm_count / 2 ? n : h->sm_count / 2;
        cluster_cache.set(h->device, max_clusters);
    }
    const int tiles = ((p.m + 255) / 256) * ((p.n + C::BN2 - 1) / C::BN2);
    const int clusters = tiles < max_clusters ? tiles : max_clusters;
    p.status = h->dev_status;
    p.group_m = group_m_setting() / 2 > 0 ? group_m_setting() / 2 : 1;
    oxq_launch(gemm_tc2_scaled_kernel<KIND, BN2_>, 2 * clusters, C::kThreads, C::kSmemBytes, h->stream, tm_a, tm_b, tm_sfa, tm_sfb, p);
    OXQ_LAUNCH_CHECK(h);
    return OXQ_OK;
}

// tile width of the CTA-pair block-scaled kernel: OXQ_GEMM_SCALED_TILE = 192 or 256
static int scaled_tile_setting() {
    static int v = 0;
    if (v == 0) { const char* e = getenv("OXQ_GEMM_SCALED_TILE"); v = (e && atoi(e) == 256) ? 256 : 192; }
    return v;
}

static int32_t check_gemm_args(oxq_handle* h, int64_t m, int64_t n, int64_t k, const void* x, const void* w, const void* y, int64_t ldy) {
    // gemm(): zero dimensions are errors (crates/oxicuda-blas/src/level3/gemm_api.rs:88-92)
    if (m <= 0 || n <= 0 || k <= 0) OXQ_FAIL(h, OXQ_ERR_INVALID_DIMENSION, "GEMM dimensions must be non-zero");
    if (m > INT32_MAX || n > INT32_MAX || k > INT32_MAX) OXQ_FAIL(h, OXQ_ERR_INVALID_DIMENSION, "GEMM dimensions exceed 2^31-1");
    if (!x || !w || !y) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null pointer");
    if (((uintptr_t)x & 15u) || ((uintptr_t)w & 15u) || ((uintptr_t)y & 15u)) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "operands must be 16-byte aligned");
    if (ldy < n || (ldy & 7)) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "ldy must be >= n and a multiple of 8");
    return oxq_require_sm100(h);
}

}  // namespace tc
}  // namespace oxq

using namespace oxq::tc;

extern "C" {

// OXQ_FP8_GEMV=0 keeps decode shapes on the 128-row tensor-memory kernels
static bool fp8_gemv_setting() {
    static const bool on = [] { const char* e = getenv("OXQ_FP8_GEMV"); return !(e && e[0] == '0'); }();
    return on;
}

// FP8 / W8A8 GEMMs with dense_decode_min_m() < m <= dense_decode_max_m() batch rows take the tensor-core weight-streaming
// kernel (OXQ_DENSE_DECODE_MAX_M, 0..64, 0 = never; OXQ_DENSE_DECODE_MIN_M: batches up to this size stay on the GEMV).
static int dense_decode_max_m() {
    static const int v = [] { const char* e = getenv("OXQ_DENSE_DECODE_MAX_M"); const int x = e ? atoi(e) : 32; return x < 0 ? 0 : (x > 64 ? 64 : x); }();
    return v;
}
// 33..64 batch rows: the streaming kernel only where the row tiles alone fill the machine (no K split: with 64 batch columns
// the cluster's exchange of partial sums costs more than the 128-row kernel): 57344 x 8192 at 64 rows 82 us against 116,
// 14336 x 4096 16 against 19, but 4096 x 4096 14 against 10.
static bool dense_decode_takes(const oxq_handle* h, int64_t m, int64_t n) {
    static const int cap = [] { const char* e = getenv("OXQ_DENSE_DECODE_MAX_M"); return e ? atoi(e) : -1; }();
    if (cap >= 0) return m <= (cap > 64 ? 64 : cap);
    return m <= 32 || (m <= 64 && ((n + 127) / 128) * 10 >= (int64_t)h->sm_count * 7);
}
static int dense_decode_min_m() {
    static const int v = [] { const char* e = getenv("OXQ_DENSE_DECODE_MIN_M"); const int x = e ? atoi(e) : 0; return x < 0 ? 0 : x; }();
    return v;
}

// largest batch served by the GEMV (OXQ_FP8_GEMV_MAX_M, 0..8, default 8)
static int fp8_gemv_max_m() {
    static const int v = [] { const char* e = getenv("OXQ_FP8_GEMV_MAX_M"); const int x = e ? atoi(e) : 8; return x < 0 ? 0 : (x > 8 ? 8 : x); }();
    return v;
}

static int32_t gemm_fp8_impl(oxq_handle* h, int64_t m, int64_t n, int64_t k, const uint8_t* x, int64_t ldx, const uint8_t* w, int64_t ldw,
                             const float* sx, const float* sw, float alpha, float beta, void* y, int64_t ldy) {
    OXQ_CHECK_HANDLE(h);
    if (int32_t rc = check_gemm_args(h, m, n, k, x, w, y, ldy)) return rc;
    if (!sx || !sw) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null scale pointer");
    if ((k & 15) || ldx < k || ldw < k || (ldx & 15) || (ldw & 15)) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "k, ldx and ldw must be multiples of 16 and ld >= k");
    if (dense_decode_takes(h, m, n) && m > dense_decode_min_m() && beta == 0.0f)   // decode shapes: the weight stream is the whole cost
        return oxq_scaled_decode_launch(h, KIND_F8, (int)m, (int)n, (int)k, x, ldx, nullptr, w, ldw, nullptr, sx, sw, alpha, y, ldy);
    if (m <= fp8_gemv_max_m() && beta == 0.0f && fp8_gemv_setting()) {
        if (int32_t rc = oxq_require_sm100(h)) return rc;
        OXQ_CUDA(h, oxq_fp8_gemv_launch(h, (int)m, (int)n, (int)k, x, ldx, w, ldw, sx, sw, alpha, y, ldy, false));
        return OXQ_OK;
    }
    GemmParams p{};
    p.alpha = alpha; p.beta = beta;
    p.m = (int)m; p.n = (int)n; p.k_bytes = (int)k; p.y = y; p.ldy = ldy; p.s0 = sx; p.s1 = sw;
    return launch_dense<KIND_F8>(h, x, ldx, w, ldw, p);
}

int32_t oxq_gemm_fp8(oxq_handle* h, int64_t m, int64_t n, int64_t k, const uint8_t* x, int64_t ldx, const uint8_t* w, int64_t ldw,
                     const float* sx, const float* sw, void* y, int64_t ldy) {
    return gemm_fp8_impl(h, m, n, k, x, ldx, w, ldw, sx, sw, 1.0f, 0.0f, y, ldy);
}

int32_t oxq_gemm_fp8_ex(oxq_handle* h, int64_t m, int64_t n, int64_t k, float alpha, const uint8_t* x, int64_t ldx, const uint8_t* w, int64_t ldw,
                        const float* sx, const float* sw, float beta, void* y, int64_t ldy) {
    return gemm_fp8_impl(h, m, n, k, x, ldx, w, ldw, sx, sw, alpha, beta, y, ldy);
}

static int32_t gemm_bf16_impl(oxq_handle* h, int64_t m, int64_t n, int64_t k, const void* x, int64_t ldx, const void* w, int64_t ldw,
                              float alpha, float beta, void* y, int64_t ldy);

// gemm's operand forms: each operand K-major or MN-major in memory; the CTA-pair kernel takes either through the shared-memory
// descriptor and the instruction descriptor's major bits, whatever m (a single 128-row tile of X simply leaves the second CTA's rows empty)
static int32_t gemm_op_impl(oxq_handle* h, bool fp8, int64_t m, int64_t n, int64_t k, float alpha, const void* a, int64_t lda, int a_major,
                            const void* b, int64_t ldb, int b_major, const float* sa, const float* sb, float beta, void* y, int64_t ldy) {
    OXQ_CHECK_HANDLE(h);
    if (int32_t rc = check_gemm_args(h, m, n, k, a, b, y, ldy)) return rc;
    if (fp8 && (!sa || !sb)) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null scale pointer");
    if ((a_major != OXQ_OP_K_MAJOR && a_major != OXQ_OP_MN_MAJOR) || (b_major != OXQ_OP_K_MAJOR && b_major != OXQ_OP_MN_MAJOR))
        OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "operand layout must be OXQ_OP_K_MAJOR or OXQ_OP_MN_MAJOR");
    const int64_t es = fp8 ? 1 : 2, al = 16 / es;
    const int64_t need_a = a_major == OXQ_OP_K_MAJOR ? k : m, need_b = b_major == OXQ_OP_K_MAJOR ? k : n;
    if (lda < need_a || ldb < need_b) OXQ_FAIL(h, OXQ_ERR_INVALID_DIMENSION, "leading dimension smaller than the contiguous extent (lda %lld < %lld or ldb %lld < %lld)",
                                               (long long)lda, (long long)need_a, (long long)ldb, (long long)need_b);
    if ((lda % al) || (ldb % al)) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "leading dimensions must be multiples of %lld elements (16 bytes)", (long long)al);
    if ((a_major == OXQ_OP_K_MAJOR || b_major == OXQ_OP_K_MAJOR) && (k % al)) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "k must be a multiple of %lld for a K-major operand", (long long)al);
    if (a_major == OXQ_OP_K_MAJOR && b_major == OXQ_OP_K_MAJOR)
        return fp8 ? gemm_fp8_impl(h, m, n, k, (const uint8_t*)a, lda, (const uint8_t*)b, ldb, sa, sb, alpha, beta, y, ldy)
                   : gemm_bf16_impl(h, m, n, k, a, lda, b, ldb, alpha, beta, y, ldy);
    GemmParams p{};
    p.alpha = alpha; p.beta = beta;
    p.m = (int)m; p.n = (int)n; p.k_bytes = (int)(k * es); p.y = y; p.ldy = ldy; p.s0 = sa; p.s1 = sb;
    p.a_mn = a_major == OXQ_OP_MN_MAJOR; p.b_mn = b_major == OXQ_OP_MN_MAJOR; p.esize = (int)es;
    return fp8 ? launch2<KIND_F8, EPI_SCALE, true>(h, a, lda * es, b, ldb * es, p) : launch2<KIND_BF16, EPI_SCALE, true>(h, a, lda * es, b, ldb * es, p);
}

int32_t oxq_gemm_fp8_op(oxq_handle* h, int64_t m, int64_t n, int64_t k, float alpha, const uint8_t* a, int64_t lda, int a_major,
                        const uint8_t* b, int64_t ldb, int b_major, const float* sa, const float* sb, float beta, void* y, int64_t ldy) {
    return gemm_op_impl(h, true, m, n, k, alpha, a, lda, a_major, b, ldb, b_major, sa, sb, beta, y, ldy);
}

int32_t oxq_gemm_bf16_op(oxq_handle* h, int64_t m, int64_t n, int64_t k, float alpha, const void* a, int64_t lda, int a_major,
                         const void* b, int64_t ldb, int b_major, float beta, void* y, int64_t ldy) {
    return gemm_op_impl(h, false, m, n, k, alpha, a, lda, a_major, b, ldb, b_major, nullptr, nullptr, beta, y, ldy);
}

int32_t oxq_gemm_fp8_all_reduce(oxq_handle* h, int64_t m, int64_t n, int64_t k, const uint8_t* x, int64_t ldx, const uint8_t* w, int64_t ldw,
                                const float* sx, const float* sw, void* y_local, void* y_multicast, int64_t ldy, uint32_t* flags_local,
                                uint32_t* flags_multicast, int64_t flag_words, int rank, int world) {
    OXQ_CHECK_HANDLE(h);
    if (int32_t rc = check_gemm_args(h, m, n, k, x, w, y_local, ldy)) return rc;
    if (!sx || !sw) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null scale pointer");
    if ((k & 15) || ldx < k || ldw < k || (ldx & 15) || (ldw & 15)) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "k, ldx and ldw must be multiples of 16 and ld >= k");
    if (world < 2 || world > 64 || rank < 0 || rank >= world) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "rank %d outside a world of %d (2..64)", rank, world);
    if (!y_multicast || ((uintptr_t)y_multicast & 15u) || !flags_local || !flags_multicast || ((uintptr_t)flags_local & 3u) || ((uintptr_t)flags_multicast & 3u))
        OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null or misaligned multicast / flag pointer");
    if (n & 7) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "n must be a multiple of 8 (16-byte vectors through the switch)");
    const int64_t tiles = ((m + 255) / 256) * ((n + 255) / 256);
    if (flag_words < 2 * (tiles + 1) + 1) OXQ_FAIL(h, OXQ_ERR_BUFFER_TOO_SMALL, "flag words: expected at least %lld, got %lld", (long long)(2 * (tiles + 1) + 1), (long long)flag_words);
    GemmParams p{};
    p.alpha = 1.0f; p.beta = 0.0f;
    p.m = (int)m; p.n = (int)n; p.k_bytes = (int)k; p.y = y_local; p.ldy = ldy; p.s0 = sx; p.s1 = sw;
    // the last word counts this rank's finished calls; its parity picks one of the two sets of flag words in front of it
    p.ar_mc_y = y_multicast; p.ar_flags = flags_local; p.ar_mc_flags = flags_multicast;
    p.ar_set_stride = (int)((flag_words - 1) / 2); p.ar_calls = flags_local + (flag_words - 1);
    p.ar_world = world; p.ar_rank = rank;
    // pause between two looks at a flag word: 232 us for the tensor-parallel down projection on two GPUs at 1000 ns against 241 at 0
    static const int sleep_ns = [] { const char* e = getenv("OXQ_AR_SLEEP_NS"); const int v = e ? atoi(e) : 1000; return v < 0 ? 0 : v; }();
    p.ar_sleep_ns = sleep_ns;
    return launch2_ar(h, x, ldx, w, ldw, p);
}

int32_t oxq_gemm_fp8_swiglu(oxq_handle* h, int64_t m, int64_t n2, int64_t k, const uint8_t* x, int64_t ldx, const uint8_t* w_gu, int64_t ldw,
                            const float* sx, const float* sw, void* hout, int64_t ldh) {
    OXQ_CHECK_HANDLE(h);
    if (n2 % 256 != 0) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "interleaved gate/up weight needs a multiple of 256 rows, got %lld", (long long)n2);
    if (int32_t rc = check_gemm_args(h, m, n2 / 2, k, x, w_gu, hout, ldh)) return rc;
    if (!sx || !sw) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null scale pointer");
    if ((k & 15) || ldx < k || ldw < k || (ldx & 15) || (ldw & 15)) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "k, ldx and ldw must be multiples of 16 and ld >= k");
    if (m <= dense_decode_max_m() && m <= 32 && m > dense_decode_min_m())
        return oxq_scaled_decode_launch(h, KIND_F8, (int)m, (int)n2, (int)k, x, ldx, nullptr, w_gu, ldw, nullptr, sx, sw, 1.0f, hout, ldh, true);
    if (m <= fp8_gemv_max_m() && fp8_gemv_setting()) {
        if (int32_t rc = oxq_require_sm100(h)) return rc;
        OXQ_CUDA(h, oxq_fp8_gemv_launch(h, (int)m, (int)n2, (int)k, x, ldx, w_gu, ldw, sx, sw, 1.0f, hout, ldh, true));
        return OXQ_OK;
    }
    GemmParams p{};
    p.alpha = 1.0f; p.beta = 0.0f;
    p.m = (int)m; p.n = (int)n2; p.k_bytes = (int)k; p.y = hout; p.ldy = ldh; p.s0 = sx; p.s1 = sw;
    return launch_dense<KIND_F8, EPI_SWIGLU>(h, x, ldx, w_gu, ldw, p);
}

static int32_t gemm_bf16_impl(oxq_handle* h, int64_t m, int64_t n, int64_t k, const void* x, int64_t ldx, const void* w, int64_t ldw,
                              float alpha, float beta, void* y, int64_t ldy) {
    OXQ_CHECK_HANDLE(h);
    if (int32_t rc = check_gemm_args(h, m, n, k, x, w, y, ldy)) return rc;
    if ((k & 7) || ldx < k || ldw < k || (ldx & 7) || (ldw & 7)) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "k, ldx and ldw must be multiples of 8 and ld >= k");
    GemmParams p{};
    p.alpha = alpha; p.beta = beta;
    p.m = (int)m; p.n = (int)n; p.k_bytes = (int)(2 * k); p.y = y; p.ldy = ldy;
    return launch_dense<KIND_BF16>(h, x, 2 * ldx, w, 2 * ldw, p);
}

int32_t oxq_gemm_bf16(oxq_handle* h, int64_t m, int64_t n, int64_t k, const void* x, int64_t ldx, const void* w, int64_t ldw,
                      void* y, int64_t ldy) {
    return gemm_bf16_impl(h, m, n, k, x, ldx, w, ldw, 1.0f, 0.0f, y, ldy);
}

int32_t oxq_gemm_bf16_ex(oxq_handle* h, int64_t m, int64_t n, int64_t k, float alpha, const void* x, int64_t ldx, const void* w, int64_t ldw,
                         float beta, void* y, int64_t ldy) {
    return gemm_bf16_impl(h, m, n, k, x, ldx, w, ldw, alpha, beta, y, ldy);
}

int32_t oxq_gemm_bf16_swiglu(oxq_handle* h, int64_t m, int64_t n2, int64_t k, const void* x, int64_t ldx, const void* w_gu, int64_t ldw,
                             void* hout, int64_t ldh) {
    OXQ_CHECK_HANDLE(h);
    if (n2 % 256 != 0) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "interleaved gate/up weight needs a multiple of 256 rows, got %lld", (long long)n2);
    if (int32_t rc = check_gemm_args(h, m, n2 / 2, k, x, w_gu, hout, ldh)) return rc;
    if ((k & 7) || ldx < k || ldw < k || (ldx & 7) || (ldw & 7)) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "k, ldx and ldw must be multiples of 8 and ld >= k");
    GemmParams p{};
    p.alpha = 1.0f; p.beta = 0.0f;
    p.m = (int)m; p.n = (int)n2; p.k_bytes = (int)(2 * k); p.y = hout; p.ldy = ldh;
    return launch_dense<KIND_BF16, EPI_SWIGLU>(h, x, 2 * ldx, w_gu, 2 * ldw, p);
}

int32_t oxq_gemm_w8a8(oxq_handle* h, int64_t m, int64_t n, int64_t k, const int8_t* x, int64_t ldx, const int8_t* w, int64_t ldw,
                      const float* sx_rows, const float* sw_rows, void* y, int64_t ldy) {
    OXQ_CHECK_HANDLE(h);
    if (int32_t rc = check_gemm_args(h, m, n, k, x, w, y, ldy)) return rc;
    if (!sx_rows || !sw_rows) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null scale pointer");
    if ((k & 15) || ldx < k || ldw < k || (ldx & 15) || (ldw & 15)) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "k, ldx and ldw must be multiples of 16 and ld >= k");
    if (dense_decode_takes(h, m, n) && m > dense_decode_min_m())
        return oxq_scaled_decode_launch(h, KIND_I8, (int)m, (int)n, (int)k, (const uint8_t*)x, ldx, nullptr, (const uint8_t*)w, ldw, nullptr, sx_rows,
                                        sw_rows, 1.0f, y, ldy);
    if (m <= fp8_gemv_max_m() && fp8_gemv_setting()) {             // decode shapes: mma.sync s8 on the raw bytes, exact s32 sums
        OXQ_CUDA(h, oxq_fp8_gemv_launch(h, (int)m, (int)n, (int)k, (const uint8_t*)x, ldx, (const uint8_t*)w, ldw, sx_rows, sw_rows, 1.0f, y, ldy,
                                        false, true));
        return OXQ_OK;
    }
    GemmParams p{};
    p.alpha = 1.0f; p.beta = 0.0f;
    p.m = (int)m; p.n = (int)n; p.k_bytes = (int)k; p.y = y; p.ldy = ldy; p.s0 = sx_rows; p.s1 = sw_rows;
    return launch_dense<KIND_I8>(h, x, ldx, w, ldw, p);
}

// Block-scaled GEMMs with at most this many batch rows take the weight-streaming kernel (OXQ_SCALED_DECODE_MAX_M, 0..64; 0 = never).
// Every CTA of that kernel reads the batch again, m / 128 of the weight bytes on top of the weight stream: from about 32 rows
// on the 128-row kernels are as fast.
static int scaled_decode_max_m() {
    static const int v = [] { const char* e = getenv("OXQ_SCALED_DECODE_MAX_M"); const int x = e ? atoi(e) : 32; return x < 0 ? 0 : (x > 64 ? 64 : x); }();
    return v;
}

int32_t oxq_gemm_mxfp8(oxq_handle* h, int64_t m, int64_t n, int64_t k, const uint8_t* x, const uint8_t* sfx, const uint8_t* w,
                       const uint8_t* sfw, void* y, int64_t ldy) {
    OXQ_CHECK_HANDLE(h);
    if (int32_t rc = check_gemm_args(h, m, n, k, x, w, y, ldy)) return rc;
    if (!sfx || !sfw || ((uintptr_t)sfx & 15u) || ((uintptr_t)sfw & 15u)) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null or misaligned scale-factor pointer");
    if (k & 127) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "k must be a multiple of 128 for the MXFP8 GEMM");
    if (m <= scaled_decode_max_m())
        return oxq_scaled_decode_launch(h, KIND_MXF8, (int)m, (int)n, (int)k, x, k, sfx, w, k, sfw, nullptr, nullptr, 1.0f, y, ldy);
    GemmParams p{};
    p.alpha = 1.0f; p.beta = 0.0f;
    p.m = (int)m; p.n = (int)n; p.k_bytes = (int)k; p.y = y; p.ldy = ldy;
    p.sfa = sfx; p.sfb = sfw; p.sf_col_tiles = (int)(k / 32 + 3) / 4;
    p.sfa_row_tiles = (int)((m + 127) / 128); p.sfb_row_tiles = (int)((n + 127) / 128);
    if (use_2cta_setting() && m > 128) return scaled_tile_setting() == 256 ? launch2_scaled<KIND_MXF8, 256>(h, x, k, w, k, p) : launch2_scaled<KIND_MXF8, 192>(h, x, k, w, k, p);
    return launch<KIND_MXF8, 192>(h, x, k, w, k, p);
}

int32_t oxq_gemm_nvfp4(oxq_handle* h, int64_t m, int64_t n, int64_t k, const uint8_t* x, const uint8_t* sfx, const float* gx,
                       const uint8_t* w, const uint8_t* sfw, const float* gw, void* y, int64_t ldy) {
    OXQ_CHECK_HANDLE(h);
    if (int32_t rc = check_gemm_args(h, m, n, k, x, w, y, ldy)) return rc;
    if (!sfx || !sfw || !gx || !gw || ((uintptr_t)sfx & 15u) || ((uintptr_t)sfw & 15u)) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null or misaligned scale pointer");
    if (k & 255) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "k must be a multiple of 256 for the NVFP4 GEMM");
    if (m <= scaled_decode_max_m())
        return oxq_scaled_decode_launch(h, KIND_NVF4, (int)m, (int)n, (int)(k / 2), x, k / 2, sfx, w, k / 2, sfw, gx, gw, 1.0f, y, ldy);
    GemmParams p{};
    p.alpha = 1.0f; p.beta = 0.0f;
    p.m = (int)m; p.n = (int)n; p.k_bytes = (int)(k / 2); p.y = y; p.ldy = ldy; p.s0 = gx; p.s1 = gw;
    p.sfa = sfx; p.sfb = sfw; p.sf_col_tiles = (int)(k / 16 + 3) / 4;
    p.sfa_row_tiles = (int)((m + 127) / 128); p.sfb_row_tiles = (int)((n + 127) / 128);
    // The CTA-pair kernel is the default for prefill shapes (OXQ_GEMM_NVFP4_2CTA=0 keeps the single-CTA one for A/B runs).
    static int nv2 = -1;
    if (nv2 < 0) { const char* e = getenv("OXQ_GEMM_NVFP4_2CTA"); nv2 = e ? (atoi(e) != 0) : 1; }
    if (nv2 && use_2cta_setting() && m > 128)
        return scaled_tile_setting() == 256 ? launch2_scaled<KIND_NVF4, 256>(h, x, k / 2, w, k / 2, p) : launch2_scaled<KIND_NVF4, 192>(h, x, k / 2, w, k / 2, p);
    return launch<KIND_NVF4, 192>(h, x, k / 2, w, k / 2, p);
}

}  // extern "C"
