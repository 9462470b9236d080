// W4A16 for small batches (passes of up to 32 rows) on the sm_100a tensor cores, with the weights as the 128-row operand.
//
//   Y[M x N] = X[M x K] * dequant(W)[N x K]^T,  uint4 codes, group 128 along K, f16 scales, packed zero-points
//   (Int4GemmConfig, crates/oxicuda-blas/src/precision/int_ops.rs:215-355, with the roles swapped: the weight
//   is the quantised operand).
//
// The weight matrix is streamed exactly once, 128 weight rows x 256 K (16 KB of codes) per TMA load into a deep
// ring of raw tiles.  Eight unpack warps turn every nibble c of a group with zero-point z into the bf16 integer
// c - z (a byte permute and one logic instruction per code pair build 128 + c, one packed subtraction removes
// 128 + z; all exact) and store the row operand of the MMA straight into tensor memory with tcgen05.st: a thread
// owns one weight row, which is one tensor-memory lane, and a group of 128 K is 64 columns.  Expanding the
// weights four-fold through shared memory instead would make shared-memory bandwidth, not HBM, the limit.
// The activation tile of the same K range arrives by TMA; one thread issues tcgen05.mma (kind::f16, A from tensor
// memory, M = 128 weight rows, N = padded batch) per group into one of eight small accumulators; four epilogue
// warps drain each group's accumulator and add it, times the group's f32 scale, to per-row totals in registers.
//
// Work is split into units of (128 rows, 256 K) in row-major order and each CTA (one per SM) takes an equal
// contiguous range of units, so the tail of the grid is at most one unit.  A range may cover parts of several
// row blocks: a part that is not the whole K range is added into an f32 workspace with atomics, and the last
// contributor of each 32-row quarter (a counter of contributed groups tells) converts the sums to bf16 and leaves
// the workspace zeroed for the next call.  The workspace is weight-row major (32 f32 per row), so a thread adds its
// totals with 16-byte vector reductions.
#include "oxq_common.cuh"
#include "oxq_tc.cuh"

namespace oxq {
namespace w4tc {
using namespace oxq::tc;

constexpr int ROWS = 128;                  // weight rows per unit == tensor-memory lanes
constexpr int UNIT_K = 256;                // K per raw tile (128 bytes of codes per row)
constexpr int RAW_BYTES = ROWS * 128;      // 16 KB
constexpr int A_COLS = 128;                // tensor-memory columns of one unpacked unit (two groups of 128 bf16 per lane)
constexpr int A_SLOTS = 2;                 // units of unpacked weights in tensor memory
constexpr int U_SLOTS_MAX = 4;             // units of activations in shared memory == units of accumulators in tensor memory (2 for 64 batch rows)
constexpr int UNPACK_WARPS = 8;            // 8 or 16 (measured alike): with 8 a thread unpacks one group (128 codes) of a weight row per unit
constexpr int NUM_WARPS = 7 + UNPACK_WARPS; // 0: codes TMA, 1: X TMA, 2: MMA + tensor-memory owner, 3-6: epilogue, 7-: unpack
constexpr int NUM_THREADS = NUM_WARPS * 32;
constexpr int SMEM_BUDGET = 227 * 1024;
constexpr int PASS_ROWS = 32;              // batch rows per pass of the 16- and 32-row forms; the workspace keeps 32 f32 per weight row and pass
                                           // (the 64-row form is one pass with 64 f32 per weight row: the same bytes as two passes)

template <int NB>
struct Cfg {
    static constexpr int kUSlots = NB == 64 ? 2 : U_SLOTS_MAX;
    static constexpr int kPassRows = NB == 64 ? 64 : PASS_ROWS;
    static constexpr int kXBytes = NB * 512;                              // one unit of X: four sub-tiles of NB rows x 128 bytes
    static constexpr int kRawStages = (SMEM_BUDGET - 3072 - kUSlots * kXBytes) / RAW_BYTES;
    static constexpr int kSmemBytes = kUSlots * kXBytes + kRawStages * RAW_BYTES + 3072;
    // tensor memory: accumulators first (two per unit slot, one per group), then the unpacked units
    static constexpr int kACol0 = kUSlots * 2 * NB;
    static constexpr int kTmemCols = 512;
    static_assert(kACol0 + A_SLOTS * A_COLS <= 512, "tensor memory overflow");
    static_assert(kRawStages >= 4, "raw ring too shallow");
};

struct Params {
    int m, n, k;
    int gpr;                       // groups per row (k / 128)
    int upr;                       // units per row (k / 256)
    int total_units;
    const uint16_t* scales;        // f16 [n x gpr]
    const uint32_t* zeros;         // packed nibbles, linear group order
    __nv_bfloat16* y;              // [m x n]
    float* ws;                     // [n x PASS_ROWS] f32 partial sums (weight row major), zero on entry and on exit
    int* counters;                 // [ceil(n / 32)], zero on entry and on exit
    int32_t* status;
};

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t sub_bf16x2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
// two codes in the low nibbles of the two halves -> bf16 pair (c - z, c' - z)
__device__ __forceinline__ uint32_t unpack_pair(uint32_t halves, uint32_t zz) {
    return sub_bf16x2((halves & 0x000F000Fu) | 0x43004300u, zz);
}
// four consecutive f32 added to global memory in one reduction (16-byte aligned)
__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

__device__ __forceinline__ void fail(const Params& p) {
    if (p.status) atomicExch(p.status, OXQ_ERR_DEVICE_TIMEOUT);
}

template <int NB>
__global__ void __launch_bounds__(NUM_THREADS, 1)
w4a16_tc_kernel(const __grid_constant__ CUtensorMap tm_codes, const __grid_constant__ CUtensorMap tm_x, const Params p) {
    using C = Cfg<NB>;
    constexpr int RS = C::kRawStages;
    constexpr int U_SLOTS = C::kUSlots;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t sm_x = base;                                   // activation tiles, one unit each
    const uint32_t sm_raw = sm_x + U_SLOTS * C::kXBytes;          // packed codes, one unit each
    const uint32_t sm_bar = sm_raw + RS * RAW_BYTES;
    const uint32_t bar_raw_full = sm_bar, bar_raw_empty = bar_raw_full + 8 * RS;
    const uint32_t bar_x_full = bar_raw_empty + 8 * RS;           // [U_SLOTS] activations of the unit have landed
    const uint32_t bar_a_full = bar_x_full + 8 * U_SLOTS;         // [A_SLOTS] weights of the unit are in tensor memory
    const uint32_t bar_done = bar_a_full + 8 * A_SLOTS;           // [U_SLOTS] the unit's MMAs have completed
    const uint32_t bar_acc_empty = bar_done + 8 * U_SLOTS;        // [U_SLOTS] the unit's accumulators have been drained
    const uint32_t tmem_slot = bar_acc_empty + 8 * U_SLOTS;
    uint32_t* tmem_slot_ptr = reinterpret_cast<uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // this CTA's contiguous range of units
    const int unit0 = (int)(((int64_t)blockIdx.x * p.total_units) / gridDim.x);
    const int unit1 = (int)(((int64_t)(blockIdx.x + 1) * p.total_units) / gridDim.x);
    const int num_units = unit1 - unit0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < RS; s++) { mbar_init(bar_raw_full + 8 * s, 1); mbar_init(bar_raw_empty + 8 * s, UNPACK_WARPS); }
        for (int s = 0; s < U_SLOTS; s++) { mbar_init(bar_x_full + 8 * s, 1); mbar_init(bar_done + 8 * s, 1); mbar_init(bar_acc_empty + 8 * s, 4); }
        for (int s = 0; s < A_SLOTS; s++) mbar_init(bar_a_full + 8 * s, UNPACK_WARPS);
        fence_barrier_init();
        prefetch_tmap(&tm_codes);
        prefetch_tmap(&tm_x);
    }
    if (warp == 2) { tmem_alloc(tmem_slot, C::kTmemCols); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_ptr;
    // Everything set up so far (barriers, tensor memory, descriptors) overlaps the tail of the kernel before this one in
    // the stream; every role waits for it before its first global access -- the weights too, since that kernel may be
    // the quantizer that writes them.
    pdl_trigger();
    pdl_wait();

    // One completion barrier per unit slot serves three waiters: the epilogue (accumulators ready), the
    // activation producer (slot free again, four units later) and the unpack warps (tensor-memory slot of the
    // weights free again, two units later) -- a single tcgen05.commit per unit on the issuing thread.
    if (warp == 0) {
        // ------------------------------------------------------------------ codes producer (whole warp, one elected lane issues)
        for (int lu = 0; lu < num_units; lu++) {
            const int unit = unit0 + lu, rb = unit / p.upr, uk = unit - rb * p.upr;
            const int rs = lu % RS;
            if (!mbar_wait_warp(bar_raw_empty + 8 * rs, ((lu / RS) & 1) ^ 1)) { if (lane == 0) fail(p); break; }
            if (elect_one()) {
                mbar_arrive_expect_tx(bar_raw_full + 8 * rs, RAW_BYTES);
                tma_load_2d(sm_raw + rs * RAW_BYTES, &tm_codes, uk * 128, rb * ROWS, bar_raw_full + 8 * rs);
            }
            __syncwarp();
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ activation producer (whole warp, one elected lane issues)
        pdl_wait();
        for (int lu = 0; lu < num_units; lu++) {
            const int unit = unit0 + lu, rb = unit / p.upr, uk = unit - rb * p.upr;
            const int k0 = uk * UNIT_K;
            const int us = lu % U_SLOTS;
            if (!mbar_wait_warp(bar_done + 8 * us, ((lu / U_SLOTS) & 1) ^ 1)) { if (lane == 0) fail(p); break; }
            const uint32_t xdst = sm_x + us * C::kXBytes;
            if (elect_one()) {
                mbar_arrive_expect_tx(bar_x_full + 8 * us, C::kXBytes);
#pragma unroll
                for (int s = 0; s < 4; s++) tma_load_2d(xdst + s * (NB * 128), &tm_x, k0 + 64 * s, 0, bar_x_full + 8 * us);
            }
            __syncwarp();
        }
    } else if (warp == 2) {
        // ------------------------------------------------------------------ MMA issuer (whole warp, one elected lane issues)
        {
            constexpr uint32_t idesc = idesc_dense(1, 1, 1, ROWS, NB);
            for (int lu = 0; lu < num_units; lu++) {
                const int us = lu % U_SLOTS, as = lu % A_SLOTS;
                if (!mbar_wait_warp(bar_acc_empty + 8 * us, ((lu / U_SLOTS) & 1) ^ 1)) { if (lane == 0) fail(p); break; }
                if (!mbar_wait_warp(bar_x_full + 8 * us, (lu / U_SLOTS) & 1)) { if (lane == 0) fail(p); break; }
                if (!mbar_wait_warp(bar_a_full + 8 * as, (lu / A_SLOTS) & 1)) { if (lane == 0) fail(p); break; }    // weights unpacked into tensor memory
                tc_fence_after();
                const uint32_t x0 = sm_x + us * C::kXBytes;
                if (elect_one()) {
#pragma unroll
                for (int h = 0; h < 2; h++) {                 // the unit's two groups, one accumulator each
                    const uint32_t d_tmem = tmem_base + (us * 2 + h) * NB;
                    const uint32_t a_tmem = tmem_base + C::kACol0 + as * A_COLS + h * 64;
#pragma unroll
                    for (int s = 0; s < 2; s++) {
                        const uint64_t bdesc = smem_desc_sw128(x0 + (h * 2 + s) * (NB * 128));
#pragma unroll
                        for (int kk = 0; kk < 4; kk++)        // 16 bf16 of K per MMA: 8 columns of A, 32 bytes of X
                            mma_f16_ts(d_tmem, a_tmem + (s * 4 + kk) * 8, bdesc + (uint64_t)(kk * 2), idesc, (s | kk) != 0);
                    }
                }
                tc_commit(bar_done + 8 * us);
                }
                __syncwarp();
            }
        }
    } else if (warp < 7) {
        // ------------------------------------------------------------------ epilogue (4 warps, one weight row per thread)
        const int quarter = warp & 3;
        const int row_in_block = quarter * 32 + lane;
        pdl_wait();
        float total[NB];
#pragma unroll
        for (int j = 0; j < NB; j++) total[j] = 0.0f;
        int cur_rb = -1, seg_groups = 0;
        uint4 sc_cur = make_uint4(0, 0, 0, 0), sc_next = sc_cur;
        int sc_key = -1, sc_next_key = -1;
        bool ok = true;
        // A part that is not the whole K range goes into the workspace; whether this warp was the last contributor
        // of its 32 rows is looked at one segment later, so the counter's round trip is not waited for.
        int pend_rb = -1, pend_old = 0, pend_groups = 0;

        auto finish_pending = [&]() {
            if (pend_rb < 0) return;
            const int last = __shfl_sync(0xffffffffu, pend_old + pend_groups == p.gpr, 0);
            const int row = pend_rb * ROWS + row_in_block;
            const int rb = pend_rb;
            pend_rb = -1;
            if (!last) return;
            __threadfence();
            if (row < p.n) {
                float4* w = reinterpret_cast<float4*>(p.ws + (size_t)row * C::kPassRows);
                float4 v[NB / 4];
#pragma unroll
                for (int q = 0; q < NB / 4; q++) v[q] = __ldcg(w + q);
#pragma unroll
                for (int q = 0; q < NB / 4; q++) {
                    __stcg(w + q, make_float4(0.0f, 0.0f, 0.0f, 0.0f));
                    const float e[4] = {v[q].x, v[q].y, v[q].z, v[q].w};
#pragma unroll
                    for (int t = 0; t < 4; t++)
                        if (4 * q + t < p.m) p.y[(size_t)(4 * q + t) * p.n + row] = __float2bfloat16_rn(e[t]);
                }
            }
            if (lane == 0) p.counters[rb * 4 + quarter] = 0;
        };

        auto flush = [&](int rb, int groups) {
            const int row = rb * ROWS + row_in_block;
            if (rb * ROWS + quarter * 32 >= p.n) return;            // this quarter lies beyond the matrix
            if (groups == p.gpr) {
                if (row < p.n) {
#pragma unroll
                    for (int j = 0; j < NB; j++)
                        if (j < p.m) p.y[(size_t)j * p.n + row] = __float2bfloat16_rn(total[j]);
                }
                return;
            }
            finish_pending();
            if (row < p.n) {
                float* w = p.ws + (size_t)row * C::kPassRows;
#pragma unroll
                for (int q = 0; q < NB / 4; q++)
                    if (4 * q < p.m) red_add_v4(w + 4 * q, total[4 * q], total[4 * q + 1], total[4 * q + 2], total[4 * q + 3]);
            }
            __threadfence();
            __syncwarp();
            if (lane == 0) pend_old = atomicAdd(p.counters + rb * 4 + quarter, groups);
            pend_rb = rb; pend_groups = groups;
        };

        for (int lu = 0; lu < num_units && ok; lu++) {
            const int unit = unit0 + lu, rb = unit / p.upr, uk = unit - rb * p.upr;
            const int g = uk * 2;                                  // the unit's groups are g and g + 1 (same 16-byte scale load)
            if (rb != cur_rb) {
                if (cur_rb >= 0) flush(cur_rb, seg_groups);
#pragma unroll
                for (int j = 0; j < NB; j++) total[j] = 0.0f;
                cur_rb = rb; seg_groups = 0;
            }
            // the groups' scales: eight consecutive f16 of this row per 16-byte load, the next eight requested ahead
            const int row_c = min(rb * ROWS + row_in_block, p.n - 1);
            const int key = rb * (p.gpr >> 3) + (g >> 3);
            if (key != sc_key) {
                if (key == sc_next_key) sc_cur = sc_next;
                else sc_cur = __ldg(reinterpret_cast<const uint4*>(p.scales + (size_t)row_c * p.gpr + (g & ~7)));
                sc_key = key;
                if ((g & ~7) + 8 < p.gpr) {
                    sc_next = __ldg(reinterpret_cast<const uint4*>(p.scales + (size_t)row_c * p.gpr + (g & ~7) + 8));
                    sc_next_key = key + 1;
                }
            }
            const int gi = (g & 7) >> 1;
            const uint32_t sw = gi == 0 ? sc_cur.x : (gi == 1 ? sc_cur.y : (gi == 2 ? sc_cur.z : sc_cur.w));
            const float s_lo = __half2float(__ushort_as_half((unsigned short)(sw & 0xFFFFu)));
            const float s_hi = __half2float(__ushort_as_half((unsigned short)(sw >> 16)));

            const int us = lu % U_SLOTS;
            ok = mbar_wait(bar_done + 8 * us, (lu / U_SLOTS) & 1);
            if (!__all_sync(0xffffffffu, ok)) { ok = false; if (lane == 0) fail(p); break; }
            tc_fence_after();
            const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + us * 2 * NB;
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const float s = h ? s_hi : s_lo;
#pragma unroll
                for (int c = 0; c < NB / 16; c++) {
                    uint32_t r[16];
                    tmem_ld_32x32b_x16(t_row + h * NB + c * 16, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; j++) total[c * 16 + j] = fmaf(s, __uint_as_float(r[j]), total[c * 16 + j]);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_acc_empty + 8 * us);
            seg_groups += 2;
        }
        if (ok && cur_rb >= 0) flush(cur_rb, seg_groups);
        if (ok) finish_pending();
    } else {
        // ------------------------------------------------------------------ unpack (UNPACK_WARPS warps)
        // The first half of the unpack warps takes the first group of every unit, the second half the second; a warp
        // serves the tensor-memory lane quarter it may access (warp index mod 4) and a thread owns a group of one weight
        // row, or half of it with 16 warps: 64 (32) bytes of codes in, 64 (32) columns of bf16 pairs out.
        constexpr int JJ = 32 / UNPACK_WARPS;                    // 16-byte pieces of a row's group per thread
        const int part = (warp - 7) >> 2, half = part / (UNPACK_WARPS / 8), sub = part % (UNPACK_WARPS / 8), quarter = warp & 3;
        const int r = quarter * 32 + lane;                       // row inside the block == tensor-memory lane
        const uint32_t rsw = (uint32_t)(r & 7);
        uint32_t zw_cur = 0, zw_next = 0;
        int z_key = -1, z_next_key = -1;
        for (int lu = 0; lu < num_units; lu++) {
            const int unit = unit0 + lu, rb = unit / p.upr, uk = unit - rb * p.upr;
            const int g = uk * 2 + half;
            // zero-point: eight consecutive groups of this row per word, the next word requested ahead
            const int row_c = min(rb * ROWS + r, p.n - 1);
            const int key = rb * (p.gpr >> 3) + (g >> 3);
            if (key != z_key) {
                if (key == z_next_key) zw_cur = zw_next;
                else zw_cur = __ldg(p.zeros + (size_t)row_c * (p.gpr >> 3) + (g >> 3));
                z_key = key;
                if ((g >> 3) + 1 < (p.gpr >> 3)) {
                    zw_next = __ldg(p.zeros + (size_t)row_c * (p.gpr >> 3) + (g >> 3) + 1);
                    z_next_key = key + 1;
                }
            }
            const uint32_t z = (zw_cur >> ((g & 7) * 4)) & 0xFu;
            const uint32_t zz = 0x43004300u | z | (z << 16);

            const int rs = lu % RS, as = lu % A_SLOTS;
            bool ok = mbar_wait(bar_raw_full + 8 * rs, (lu / RS) & 1);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) { if (lane == 0) fail(p); break; }
            uint4 raw[JJ];
            const uint32_t raw_row = sm_raw + rs * RAW_BYTES + r * 128;
#pragma unroll
            for (int jj = 0; jj < JJ; jj++) raw[jj] = lds128(raw_row + ((((uint32_t)(half * 4 + sub * JJ + jj)) ^ rsw) << 4));
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_raw_empty + 8 * rs);   // the codes are in registers

            if (lu >= A_SLOTS) {
                // the tensor-memory slot was last read by the MMAs of unit lu - A_SLOTS
                const int pu = lu - A_SLOTS;
                ok = mbar_wait(bar_done + 8 * (pu % U_SLOTS), (pu / U_SLOTS) & 1);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) { if (lane == 0) fail(p); break; }
            }
            tc_fence_after();
            const uint32_t a_lane = tmem_base + ((uint32_t)(quarter * 32) << 16) + C::kACol0 + as * A_COLS + half * 64;
            {
#pragma unroll
                for (int jj = 0; jj < JJ; jj++) {
                    // 32 consecutive K of this row -> 16 columns, K pairs in their natural order
                    const uint32_t wv[4] = {raw[jj].x, raw[jj].y, raw[jj].z, raw[jj].w};
                    uint32_t o[16];
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const uint32_t w = wv[i], w4 = w >> 4;    // byte b of w4 has code 2b+1 in its low nibble
                        o[4 * i + 0] = unpack_pair(__byte_perm(w, w4, 0x4400), zz);
                        o[4 * i + 1] = unpack_pair(__byte_perm(w, w4, 0x5511), zz);
                        o[4 * i + 2] = unpack_pair(__byte_perm(w, w4, 0x6622), zz);
                        o[4 * i + 3] = unpack_pair(__byte_perm(w, w4, 0x7733), zz);
                    }
                    tmem_st_32x32b_x16(a_lane + 16 * (sub * JJ + jj), o);
                }
                tmem_st_wait();
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_a_full + 8 * as);
        }
    }

    // Teardown: on the normal path the epilogue has drained the last accumulator, so every MMA has finished and
    // every TMA load has landed before tensor memory is released.
    tc_fence_before();
    __syncthreads();
    if (warp == 2) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, C::kTmemCols);
    }
}

template <int NB>
static int32_t launch_nb(oxq_handle* h, const CUtensorMap& tm_codes, const void* x, Params p) {
    using C = Cfg<NB>;
    CUtensorMap tm_x;
    if (!oxq_make_tmap_2d(&tm_x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, x, (uint64_t)p.k, (uint64_t)p.m, (uint64_t)p.k * 2, 64, NB,
                          CU_TENSOR_MAP_SWIZZLE_128B))
        OXQ_FAIL(h, OXQ_ERR_LAUNCH_FAILED, "cuTensorMapEncodeTiled failed for the activations (16-byte aligned pointer needed)");
    static OxqPerDevice attr_set;
    if (!attr_set.get(h->device)) {
        OXQ_CUDA(h, cudaFuncSetAttribute(w4a16_tc_kernel<NB>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
        attr_set.set(h->device, 1);
    }
    const int grid = p.total_units < h->sm_count ? p.total_units : h->sm_count;
    oxq_launch(w4a16_tc_kernel<NB>, grid, NUM_THREADS, C::kSmemBytes, h->stream, tm_codes, tm_x, p);
    OXQ_LAUNCH_CHECK(h);
    return OXQ_OK;
}

}  // namespace w4tc
}  // namespace oxq

// Shapes this path covers: group 128, k a multiple of 1024 (whole units, and eight groups per scale / zero-point
// load), m <= 128 (batches above 32 rows run as passes of 32; the later passes find the weights in L2).
// `ws_sums` (32 f32 per weight row and pass: [ceil(m / 32)][n][32]) and `ws_counters` ([ceil(n / 32)]) must be zero
// on entry and are zero again on exit.
bool oxq_w4tc_supports(int64_t m, int64_t n, int64_t k, int group) {
    return m >= 1 && m <= 128 && group == 128 && k % 1024 == 0 && n >= 1 && n <= (int64_t)INT32_MAX / 256 && k <= INT32_MAX / 4;
}

int32_t oxq_w4tc_launch(oxq_handle* h, int64_t m, int64_t n, int64_t k, const void* x, const uint32_t* codes, const uint16_t* scales,
                        const uint32_t* zeros, void* y, float* ws_sums, int* ws_counters) {
    using namespace oxq::w4tc;
    CUtensorMap tm_codes;
    if (!oxq_make_tmap_2d(&tm_codes, CU_TENSOR_MAP_DATA_TYPE_UINT8, codes, (uint64_t)(k / 2), (uint64_t)n, (uint64_t)(k / 2), 128, ROWS,
                          CU_TENSOR_MAP_SWIZZLE_128B))
        OXQ_FAIL(h, OXQ_ERR_LAUNCH_FAILED, "cuTensorMapEncodeTiled failed for the codes (16-byte aligned pointer needed)");
    const int row_blocks = (int)((n + ROWS - 1) / ROWS);
    if (m > PASS_ROWS && m <= 64) {                            // one pass with 64 batch columns: the weights are unpacked once
        Params p;
        p.m = (int)m; p.n = (int)n; p.k = (int)k; p.gpr = (int)(k / 128); p.upr = (int)(k / UNIT_K);
        p.total_units = row_blocks * p.upr;
        p.scales = scales; p.zeros = zeros; p.y = (__nv_bfloat16*)y; p.ws = ws_sums; p.counters = ws_counters;
        p.status = h->dev_status;
        return launch_nb<64>(h, tm_codes, (const __nv_bfloat16*)x, p);
    }
    for (int64_t m0 = 0; m0 < m; m0 += PASS_ROWS) {
        Params p;
        p.m = (int)(m - m0 < PASS_ROWS ? m - m0 : PASS_ROWS); p.n = (int)n; p.k = (int)k; p.gpr = (int)(k / 128); p.upr = (int)(k / UNIT_K);
        p.total_units = row_blocks * p.upr;
        p.scales = scales; p.zeros = zeros; p.y = (__nv_bfloat16*)y + m0 * n; p.ws = ws_sums + (m0 / PASS_ROWS) * n * PASS_ROWS; p.counters = ws_counters;
        p.status = h->dev_status;
        const __nv_bfloat16* xp = (const __nv_bfloat16*)x + m0 * k;
        const int32_t rc = p.m <= 16 ? launch_nb<16>(h, tm_codes, xp, p) : launch_nb<32>(h, tm_codes, xp, p);
        if (rc != OXQ_OK) return rc;
    }
    return OXQ_OK;
}
