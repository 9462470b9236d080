// Decode shapes (1 to 64 batch rows) of the block-scaled GEMMs, Fp4GemmConfig's memory-bound regime
// (crates/oxicuda-blas/src/precision/fp4_fp6_ops.rs:337-395; the reference's kernel unpacks FP4 in registers,
// generate_fp4_gemm_ptx :1237-1362 and the dequantisation at :1481-1579), and of the FP8 and W8A8 GEMMs (no scale
// factors to move: the per-tensor or per-row scales are applied when the accumulator is drained).
//
// Here the operands swap sides: the weight W[N x K] is the 128-row A operand of tcgen05.mma and the batch X[M x K] its
// narrow N side (16, 32 or 64 columns), D[128 weight rows x batch] = W_tile . X^T.  Every byte of the weight stream
// then feeds a full-height MMA, the tensor core unpacks E2M1 / E4M3 and applies the block scales itself, and the SM
// only has to keep TMA loads in flight: the kernel runs at the speed of the weight stream.  A CTA owns one 128-row
// tile of W over a K range; a cluster of up to eight CTAs splits K and adds its partial sums through distributed
// shared memory in a fixed order (no atomics: the result does not depend on scheduling).  Two CTAs fit on an SM, so
// the set-up and the epilogue of one overlap the stream of the other.
//
//   warp 0: TMA producer    warp 1: tensor-memory owner + MMA issuer    warps 2-5: epilogue (one per 32 accumulator lanes)
#include "oxq_common.cuh"
#include "oxq_tc.cuh"
#include <stdlib.h>

namespace oxq {
namespace tcdec {

using namespace oxq::tc;

constexpr int BM = 128;               // weight rows per tile == tensor-memory lanes
constexpr int BKB = 128;              // bytes of K per stage == one swizzle atom
constexpr int NUM_THREADS = 192;
constexpr int SMEM_PER_CTA = 112 * 1024;    // two CTAs per SM

struct DecParams {
    int m, n, k_bytes;
    int ksplit;                       // CTAs of a cluster that share the K range of one tile
    const uint8_t* sfw; const uint8_t* sfx;   // tiled scale factors of W and X (block-scaled kinds)
    int sf_col_tiles;                 // 4-column scale-factor tiles per 128-row tile
    const float* gx; const float* gw; // NVFP4 / FP8: per-tensor scales; W8A8: per-row scales of X [m] and of W [n]
    float alpha;
    __nv_bfloat16* y; int64_t ldy;
    int32_t* status;
};

// SWIGLU (FP8 only): the weight holds blocks of 128 gate rows followed by the 128 matching up rows; a CTA takes one such
// pair of tiles into two accumulators, so a thread's lane holds gate and up of the same output column and stores
// silu(gate) * up (SwiGluFfn::forward, crates/oxicuda-lm/src/layer/ffn.rs:235-254).
template <int KIND, int BN, bool SWIGLU = false>
struct Cfg {
    static constexpr bool kScaled = KIND == KIND_MXF8 || KIND == KIND_NVF4;
    static constexpr int kSfChunks = KIND == KIND_MXF8 ? 1 : (KIND == KIND_NVF4 ? 4 : 0);   // 512-byte scale-factor chunks per stage and operand
    static constexpr int kSfBytes = kSfChunks * 512;
    static constexpr int kATiles = SWIGLU ? 2 : 1;
    static constexpr int kABytes = kATiles * BM * BKB;
    static constexpr int kBBytes = BN * BKB;
    static constexpr int kStageBytes = kABytes + kBBytes + 2 * kSfBytes;
    static constexpr int kStagesFit = (SMEM_PER_CTA - 2048) / kStageBytes;
    static constexpr int kStages = kStagesFit > 6 ? 6 : kStagesFit;
    static constexpr int kSmemBytes = kStages * kStageBytes + 2048;
    // tensor-memory columns: accumulator, then the scale factors of W and of X
    static constexpr int kSfaCol = 64, kSfbCol = 64 + 4 * kSfChunks, kCols = 128;
    static_assert(BN == 16 || BN == 32 || BN == 64, "batch tile");
    static_assert(kStages >= 3, "pipeline depth");
    static_assert((BN + 8) * kATiles * BM * 4 <= kStages * kABytes, "the partial sums reuse the weight stages");
    static_assert(!SWIGLU || (KIND == KIND_F8 && BN <= 32), "SwiGLU form: FP8, up to 32 batch rows");
};

template <int KIND, int BN, bool SWIGLU = false>
__global__ void __launch_bounds__(NUM_THREADS, 2)
scaled_decode_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x, const DecParams p) {
    using C = Cfg<KIND, BN, SWIGLU>;
    constexpr int AT = C::kATiles;
    constexpr int S = C::kStages;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t sm_a = base;
    const uint32_t sm_b = sm_a + S * C::kABytes;
    const uint32_t sm_sfa = sm_b + S * C::kBBytes;
    const uint32_t sm_sfb = sm_sfa + S * C::kSfBytes;
    const uint32_t sm_bar = sm_sfb + S * C::kSfBytes;
    const uint32_t bar_full = sm_bar, bar_empty = sm_bar + 8 * S, bar_tfull = sm_bar + 16 * S;
    const uint32_t tmem_slot = bar_tfull + 8;
    uint32_t* tmem_slot_ptr = reinterpret_cast<uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));
    float* part = reinterpret_cast<float*>(smem_raw + (sm_a - smem_u32(smem_raw)));   // [rank][batch rows owned][128] partial sums, over the weight stages once every MMA is done

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t crank = p.ksplit > 1 ? cluster_ctarank() : 0u;
    const int n0 = (int)blockIdx.x * BM * AT;                     // first weight row (SwiGLU: of the gate block; the up block follows)
    const int num_kb = (p.k_bytes + BKB - 1) / BKB;
    const int kb_lo = (int)(((int64_t)crank * num_kb) / p.ksplit), kb_hi = (int)(((int64_t)(crank + 1) * num_kb) / p.ksplit);

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; s++) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_empty + 8 * s, 1); }
        mbar_init(bar_tfull, 1);
        fence_barrier_init();
        prefetch_tmap(&tm_w);
        prefetch_tmap(&tm_x);
    }
    if (warp == 1) { tmem_alloc(tmem_slot, C::kCols); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_ptr;
    pdl_trigger();
    pdl_wait();                                                  // X (and its scales) may come from the kernel before this one

    bool done = kb_lo < kb_hi;                                   // epilogue: the accumulator holds this CTA's sum
    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (whole warp, one elected lane issues)
        int stage = 0; uint32_t phase = 0;
        const size_t row_stride = (size_t)p.sf_col_tiles * 512;
        const uint8_t* sfw_tile = p.sfw + (size_t)blockIdx.x * row_stride;
        // The CTAs of a wave would all ask the L2 for the same lines of X at the same moment; each tile therefore starts
        // its walk over the K blocks at a different block (a fixed function of the tile index, so the order of the sum is
        // the same in every run).
        const int cnt = kb_hi - kb_lo;
        int kb = cnt > 0 ? kb_lo + (int)((blockIdx.x * 5u) % (unsigned)cnt) : kb_lo;
        for (int it = 0; it < cnt; it++, kb = kb + 1 == kb_hi ? kb_lo : kb + 1) {
            if (!mbar_wait_warp(bar_empty + 8 * stage, phase ^ 1)) { if (lane == 0) atomicExch(p.status, OXQ_ERR_DEVICE_TIMEOUT); break; }
            const uint32_t full = bar_full + 8 * stage;
            if (elect_one()) {
                mbar_arrive_expect_tx(full, C::kStageBytes);
                tma_load_2d(sm_a + stage * C::kABytes, &tm_w, kb * BKB, n0, full);
                if (SWIGLU) tma_load_2d(sm_a + stage * C::kABytes + BM * BKB, &tm_w, kb * BKB, n0 + BM, full);
                tma_load_2d(sm_b + stage * C::kBBytes, &tm_x, kb * BKB, 0, full);
                if (C::kScaled) {
                    bulk_load(sm_sfa + stage * C::kSfBytes, sfw_tile + (size_t)kb * C::kSfBytes, C::kSfBytes, full);
                    bulk_load(sm_sfb + stage * C::kSfBytes, p.sfx + (size_t)kb * C::kSfBytes, C::kSfBytes, full);
                }
            }
            __syncwarp();
            if (++stage == S) { stage = 0; phase ^= 1; }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (whole warp, one elected lane issues)
        constexpr uint32_t idesc = KIND == KIND_F8 ? idesc_dense(1, 0, 0, BM, BN) : KIND == KIND_I8 ? idesc_dense(2, 1, 1, BM, BN) :
                                   KIND == KIND_MXF8 ? idesc_block_scaled(0, 0, 1, BM, BN) : idesc_block_scaled(1, 1, 0, BM, BN);
        int stage = 0; uint32_t phase = 0;
        bool ok = true;
        for (int it = 0; it < kb_hi - kb_lo; it++) {
            if (!mbar_wait_warp(bar_full + 8 * stage, phase)) { ok = false; if (lane == 0) atomicExch(p.status, OXQ_ERR_DEVICE_TIMEOUT); break; }
            tc_fence_after();
            const uint64_t adesc = smem_desc_sw128(sm_a + stage * C::kABytes);
            const uint64_t bdesc = smem_desc_sw128(sm_b + stage * C::kBBytes);
            if (elect_one()) {
#pragma unroll
                for (int c = 0; c < C::kSfChunks; c++) {
                    tc_cp_32x128b_warpx4(tmem_base + C::kSfaCol + 4 * c, smem_desc_sf(sm_sfa + stage * C::kSfBytes + c * 512));
                    tc_cp_32x128b_warpx4(tmem_base + C::kSfbCol + 4 * c, smem_desc_sf(sm_sfb + stage * C::kSfBytes + c * 512));
                }
#pragma unroll
                for (int k = 0; k < BKB / 32; k++) {
                    const uint64_t a = adesc + (uint64_t)(k * 2), b = bdesc + (uint64_t)(k * 2);
                    const uint32_t accum = (it | k) != 0;
                    if (KIND == KIND_F8) {
                        mma_f8f6f4(tmem_base, a, b, idesc, accum);
                        if (SWIGLU) mma_f8f6f4(tmem_base + 64, a + (uint64_t)((BM * BKB) >> 4), b, idesc, accum);   // the up tile, 16 KB further on
                    }
                    else if (KIND == KIND_I8) mma_i8(tmem_base, a, b, idesc, accum);
                    else if (KIND == KIND_MXF8)                   // one scale per row and MMA: byte k of the chunk's 32-bit words
                        mma_mxf8f6f4(tmem_base, a, b, idesc_with_sf_ids(idesc, k, k), accum, tmem_base + C::kSfaCol, tmem_base + C::kSfbCol);
                    else                                          // four scales per row and MMA: chunk k, all four bytes
                        mma_mxf4nvf4_x4(tmem_base, a, b, idesc, accum, tmem_base + C::kSfaCol + 4 * k, tmem_base + C::kSfbCol + 4 * k);
                }
                tc_commit(bar_empty + 8 * stage);
            }
            __syncwarp();
            if (++stage == S) { stage = 0; phase ^= 1; }
        }
        if (ok && elect_one()) tc_commit(bar_tfull);
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ epilogue (4 warps): accumulator -> registers
        const int quarter = warp & 3;
        const int i = quarter * 32 + lane;                       // row of the tile
        float acc[AT * BN];                                      // SwiGLU: gate sums, then up sums
#pragma unroll
        for (int j = 0; j < AT * BN; j++) acc[j] = 0.0f;
        if (done) {
            bool ok = mbar_wait(bar_tfull, 0);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) { done = false; if (lane == 0) atomicExch(p.status, OXQ_ERR_DEVICE_TIMEOUT); }
        }
        if (done) {
            tc_fence_after();
            const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16);
#pragma unroll
            for (int a = 0; a < AT; a++) {
#pragma unroll
                for (int c = 0; c < BN / 16; c++) {
                    uint32_t r[16];
                    tmem_ld_32x32b_x16(t_row + a * 64 + c * 16, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; j++) acc[a * BN + c * 16 + j] = __uint_as_float(r[j]);
                }
            }
        }
        // accumulator (or sum of the cluster's accumulators) of batch row j -> bf16 output.  W8A8 sums are exact integers and
        // take the same scale expression as the 128-row kernel, (float)acc * (sx[m] * alpha * sw[n]).
        const float scale = (KIND == KIND_NVF4 || KIND == KIND_F8) ? __ldg(p.gx) * __ldg(p.gw) * p.alpha : p.alpha;
        const float sw_row = (KIND == KIND_I8 && n0 + i < p.n) ? __ldg(p.gw + n0 + i) : 0.0f;
        auto emit = [&](int j, uint32_t bits, uint32_t up_bits) {
            if (SWIGLU) {
                const float gt = __uint_as_float(bits) * scale, up = __uint_as_float(up_bits) * scale;
                p.y[(size_t)j * p.ldy + (n0 >> 1) + i] = __float2bfloat16_rn(__fdividef(gt, 1.0f + __expf(-gt)) * up);
                return;
            }
            float v;
            if (KIND == KIND_I8) v = (float)(int)bits * ((__ldg(p.gx + j) * p.alpha) * sw_row);
            else v = __uint_as_float(bits) * scale;
            p.y[(size_t)j * p.ldy + n0 + i] = __float2bfloat16_rn(v);
        };
        if (p.ksplit == 1) {
            if (n0 + i < p.n) {
#pragma unroll
                for (int j = 0; j < BN; j++)
                    if (j < p.m) emit(j, __float_as_uint(acc[j]), SWIGLU ? __float_as_uint(acc[(AT - 1) * BN + j]) : 0u);
            }
        }
        tc_fence_before();
        if (p.ksplit > 1) {
            // The cluster's CTAs add their sums.  Batch row j belongs to CTA j % ksplit: once every CTA of the cluster has
            // finished its MMAs (first barrier: the weight stages are free everywhere) each CTA stores its partial sums of
            // row j into the owner's shared memory, slot [rank][j / ksplit][i]; after the second barrier the owner adds the
            // slots in rank order.  Remote stores do not wait for their completion, the barrier does.
            cluster_sync_all();
            const int per = (p.m + p.ksplit - 1) / p.ksplit;             // rows per owner
#pragma unroll
            for (int j = 0; j < BN; j++) {
                if (j < p.m) {
                    const int owner = j % p.ksplit, slot = j / p.ksplit;
#pragma unroll
                    for (int a = 0; a < AT; a++) {
                        const uint32_t local = sm_a + (uint32_t)(((((int)crank * per + slot) * AT + a) * BM + i) * 4);
                        const uint32_t ra = mapa_shared(local, (uint32_t)owner);
                        asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(ra), "f"(acc[a * BN + j]) : "memory");
                    }
                }
            }
            cluster_sync_all();
            for (int slot = 0, j = (int)crank; j < p.m; slot++, j += p.ksplit) {
                uint32_t bits, up_bits = 0u;
                if (KIND == KIND_I8) {
                    int v = 0;
                    for (int c = 0; c < p.ksplit; c++) v += (int)__float_as_uint(part[(c * per + slot) * BM + i]);
                    bits = (uint32_t)v;
                } else {
                    float v = 0.0f, u = 0.0f;
                    for (int c = 0; c < p.ksplit; c++) {
                        v += part[((c * per + slot) * AT) * BM + i];
                        if (SWIGLU) u += part[((c * per + slot) * AT + 1) * BM + i];
                    }
                    bits = __float_as_uint(v); up_bits = __float_as_uint(u);
                }
                if (n0 + i < p.n) emit(j, bits, up_bits);
            }
        }
    }
    if (p.ksplit > 1 && warp < 2) {                              // every thread of the cluster takes part in both barriers
        cluster_sync_all();
        cluster_sync_all();
    }

    // Teardown: every MMA has finished (the epilogue saw the accumulator complete, or a wait gave up) before tensor
    // memory is released.
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, C::kCols);
    }
}

// OXQ_DEC_KSPLIT = 1, 2, 4 or 8 fixes the K split (tuning runs); 0 or unset: chosen per shape.
static int ksplit_override() {
    static const int v = [] { const char* e = getenv("OXQ_DEC_KSPLIT"); const int x = e ? atoi(e) : 0; return (x == 1 || x == 2 || x == 4 || x == 8) ? x : 0; }();
    return v;
}

// Clusters cost scheduling freedom (their CTAs have to start together inside one GPC; sizes that are not powers of two
// pack badly), so K is split only when the row tiles alone leave much of the machine idle: the smallest power of two
// that gives at least 0.7 CTAs per SM.  Measured at 8 batch rows, MXFP8, K splits 1 / 2 / 4 / 8: 14336 x 4096 (112
// tiles) 12.5 / 13.5 / 16.8 / 22.8 us, 57344 x 8192 (448 tiles) 75 / 83 / 87 / 104 us, 4096 x 14336 (32 tiles) 28.2 /
// 17.9 / 13.8 / 13.8 us, 6144 x 4096 (48 tiles) 10.4 / 8.9 / 8.1 / 11.6 us.
static int choose_ksplit(int tiles, int num_kb, int sm_count) {
    if (const int o = ksplit_override()) return o <= num_kb ? o : 1;
    int ks = 1;
    while (ks < 8 && (int64_t)tiles * ks * 10 < (int64_t)sm_count * 7 && num_kb / (ks * 2) >= 2) ks *= 2;
    return ks;
}

template <int KIND, int BN, bool SWIGLU = false>
static int32_t launch(oxq_handle* h, const CUtensorMap& tm_w, const CUtensorMap& tm_x, DecParams p) {
    using C = Cfg<KIND, BN, SWIGLU>;
    static OxqPerDevice attr_set;
    if (!attr_set.get(h->device)) {
        OXQ_CUDA(h, cudaFuncSetAttribute(scaled_decode_kernel<KIND, BN, SWIGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
        attr_set.set(h->device, 1);
    }
    const int tiles = (p.n + BM * C::kATiles - 1) / (BM * C::kATiles);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)tiles, (unsigned)p.ksplit, 1); cfg.blockDim = dim3(NUM_THREADS, 1, 1);
    cfg.dynamicSmemBytes = C::kSmemBytes; cfg.stream = h->stream;
    cudaLaunchAttribute attrs[2];
    int na = 0;
    if (p.ksplit > 1) {
        attrs[na].id = cudaLaunchAttributeClusterDimension;
        attrs[na].val.clusterDim.x = 1; attrs[na].val.clusterDim.y = (unsigned)p.ksplit; attrs[na].val.clusterDim.z = 1;
        na++;
    }
    if (oxq_pdl_enabled()) {
        attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attrs[na].val.programmaticStreamSerializationAllowed = 1;
        na++;
    }
    cfg.attrs = attrs; cfg.numAttrs = na;
    OXQ_CUDA(h, cudaLaunchKernelEx(&cfg, scaled_decode_kernel<KIND, BN, SWIGLU>, tm_w, tm_x, p));
    return OXQ_OK;
}

}  // namespace tcdec
}  // namespace oxq

int32_t oxq_scaled_decode_launch(oxq_handle* h, int kind, int m, int n, int k_bytes, const uint8_t* x, int64_t ldx_bytes, const uint8_t* sfx,
                                 const uint8_t* w, int64_t ldw_bytes, const uint8_t* sfw, const float* gx, const float* gw, float alpha, void* y,
                                 int64_t ldy, bool swiglu) {
    using namespace oxq::tcdec;
    using namespace oxq::tc;
    const int bn = m <= 16 ? 16 : (m <= 32 ? 32 : 64);
    if (swiglu && (kind != KIND_F8 || m > 32 || (n & 255))) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "SwiGLU decode form: FP8, up to 32 batch rows, 256-row blocks");
    CUtensorMap tm_w, tm_x;
    if (!oxq_make_tmap_2d(&tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, w, (uint64_t)k_bytes, (uint64_t)n, (uint64_t)ldw_bytes, BKB, BM, CU_TENSOR_MAP_SWIZZLE_128B) ||
        !oxq_make_tmap_2d(&tm_x, CU_TENSOR_MAP_DATA_TYPE_UINT8, x, (uint64_t)k_bytes, (uint64_t)m, (uint64_t)ldx_bytes, BKB, (uint32_t)bn, CU_TENSOR_MAP_SWIZZLE_128B))
        OXQ_FAIL(h, OXQ_ERR_LAUNCH_FAILED, "cuTensorMapEncodeTiled failed (pointers must be 16-byte aligned, leading dimensions multiples of 16 bytes)");
    DecParams p;
    p.m = m; p.n = n; p.k_bytes = k_bytes;
    const int num_kb = (k_bytes + BKB - 1) / BKB;
    p.ksplit = choose_ksplit(swiglu ? n / (2 * BM) : (n + BM - 1) / BM, num_kb, h->sm_count);
    p.sfw = sfw; p.sfx = sfx;
    p.sf_col_tiles = kind == KIND_MXF8 ? (k_bytes / 32 + 3) / 4 : (k_bytes / 8 + 3) / 4;
    p.gx = gx; p.gw = gw; p.alpha = alpha; p.y = (__nv_bfloat16*)y; p.ldy = ldy; p.status = h->dev_status;
#define OXQ_DEC_DISPATCH(K)                                                     \
    do {                                                                        \
        if (bn == 16) return launch<K, 16>(h, tm_w, tm_x, p);                   \
        if (bn == 32) return launch<K, 32>(h, tm_w, tm_x, p);                   \
        return launch<K, 64>(h, tm_w, tm_x, p);                                 \
    } while (0)
    if (swiglu) {
        if (bn == 16) return launch<KIND_F8, 16, true>(h, tm_w, tm_x, p);
        return launch<KIND_F8, 32, true>(h, tm_w, tm_x, p);
    }
    if (kind == KIND_MXF8) OXQ_DEC_DISPATCH(KIND_MXF8);
    if (kind == KIND_NVF4) OXQ_DEC_DISPATCH(KIND_NVF4);
    if (kind == KIND_F8) OXQ_DEC_DISPATCH(KIND_F8);
    if (kind == KIND_I8) OXQ_DEC_DISPATCH(KIND_I8);
#undef OXQ_DEC_DISPATCH
    OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "operand kind %d has no decode kernel", kind);
}
