// GPTQ weight preparation on the device: GptqQuantizer::quantize_layer of the reference
// (crates/oxicuda-quant/src/scheme/gptq.rs:133-257) with its helpers cholesky_lower (:281-300), invert_lower
// (:305-318), hinv_row_starting (:328-332), col_quant_params (:242-276) and quant_scalar (:235-239).
//
// The reference is a sequential CPU loop in f32.  Every stage here is blocked and parallel, yet reproduces the
// reference bit for bit, because each output element still sees the same chain of individually rounded
// operations in the same order:
//   * Cholesky, right-looking in blocks of 32: element (i, j) starts from h[i][j] and has l[i][k] * l[j][k]
//     subtracted for k = 0, 1, ... in increasing k, then is divided by the pivot (or square-rooted) -- the
//     sequence of the reference's row-by-row loop.  Products and subtractions are never fused.
//   * Inverse of the factor, right-looking by blocks of 32 rows: s starts at +0 and accumulates l[i][k] * li[k][j]
//     in increasing k (a finished block of rows is pushed into every later row before the next block is finished);
//     terms with k < j multiply stored zeros and leave s at +0.
//   * H^-1 = (L^-1)^T L^-1 (upper triangle): sums over m in increasing m, again with stored zeros in front.
//   * The column loop: a column's correction by all earlier columns, w[i][k] -= err_j[i] * hinv[j][k] for
//     j = 0 .. k-1, is applied lazily but in increasing j, one rounded product and one rounded subtraction each.
//     Rows are independent except for the per-column scale (a maximum over all rows), which costs one grid-wide
//     meeting point per column: the kernel is launched cooperatively with every CTA resident, each CTA owns a
//     slice of rows and publishes its share of the maximum in a tagged slot that the others read (no atomics), and
//     the wait is bounded (two seconds, then OXQ_ERR_DEVICE_TIMEOUT in the status word).
#include "oxq_common.cuh"

namespace oxq {
namespace {

constexpr int NB = 32;                 // block edge of the factorisation and the inversion
constexpr int CB = 64;                 // columns per block of the column loop
constexpr int CBP = CB + 1;            // padded row stride of the column blocks in shared memory
constexpr float kDegenerate = 1e-12f;  // gptq.rs:209

// control words at the end of the workspace
enum { CTL_LAMBDA = 0, CTL_MIN_DIAG = 1, CTL_FAIL = 2, CTL_COUNTER = 3, CTL_WORDS = 16 };

__device__ __forceinline__ float mulsub(float s, float a, float b) { return __fsub_rn(s, __fmul_rn(a, b)); }
__device__ __forceinline__ float muladd(float s, float a, float b) { return __fadd_rn(s, __fmul_rn(a, b)); }
__device__ __forceinline__ uint32_t order_key(float v) {                  // monotone map of finite/inf floats to u32
    const uint32_t b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float order_unkey(uint32_t k) { return __uint_as_float((k & 0x80000000u) ? (k & 0x7FFFFFFFu) : ~k); }
__device__ __forceinline__ uint32_t ld_volatile(const uint32_t* p) { return *reinterpret_cast<const volatile uint32_t*>(p); }

// lambda = percdamp * max(|mean(diag H)|, 1e-8) with the diagonal summed left to right (gptq.rs:163-165), and the
// smallest dampened diagonal entry for the SingularHessian report (:172-176).
__global__ void __launch_bounds__(256) gptq_prepare_kernel(const float* __restrict__ H, int n, float percdamp, uint32_t* ctl, int32_t* info,
                                                           unsigned long long* slots, int nslots) {
    __shared__ float d[1024];
    for (int t = threadIdx.x; t < nslots; t += 256) slots[t] = 0ull;
    float sum = 0.0f;
    for (int base = 0; base < n; base += 1024) {
        __syncthreads();
        for (int t = threadIdx.x; t < 1024 && base + t < n; t += 256) d[t] = H[(size_t)(base + t) * n + base + t];
        __syncthreads();
        if (threadIdx.x == 0) {
            const int m = min(1024, n - base);
            for (int t = 0; t < m; t++) sum = __fadd_rn(sum, d[t]);
        }
    }
    if (threadIdx.x == 0) {
        float md = fabsf(__fdiv_rn(sum, (float)n));
        if (!(md > 1e-8f)) md = 1e-8f;
        const float lambda = __fmul_rn(percdamp, md);
        float mn = __int_as_float(0x7F800000);
        for (int j = 0; j < n; j++) {
            const float v = __fadd_rn(H[(size_t)j * n + j], lambda);
            if (v < mn) mn = v;
        }
        ctl[CTL_LAMBDA] = __float_as_uint(lambda);
        ctl[CTL_MIN_DIAG] = __float_as_uint(mn);
        ctl[CTL_FAIL] = 0;
        ctl[CTL_COUNTER] = 0;
        info[0] = 0;
        info[1] = __float_as_int(mn);
    }
}

__global__ void __launch_bounds__(256) gptq_damp_kernel(const float* __restrict__ H, float* __restrict__ A, int n, const uint32_t* ctl) {
    const float lambda = __uint_as_float(ctl[CTL_LAMBDA]);
    const int64_t total = (int64_t)n * n;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / n, c = i - r * n;
        const float v = H[i];
        A[i] = r == c ? __fadd_rn(v, lambda) : v;
    }
}

// The 32 x 32 diagonal block of one block column, factored in place by one CTA.
__global__ void __launch_bounds__(256) chol_diag_kernel(float* __restrict__ A, int n, int kb, uint32_t* ctl, int32_t* info) {
    if (ld_volatile(ctl + CTL_FAIL)) return;
    __shared__ float D[NB][NB + 1];
    __shared__ int s_fail;
    const int bw = min(NB, n - kb);
    for (int t = threadIdx.x; t < NB * NB; t += 256) {
        const int r = t / NB, c = t % NB;
        D[r][c] = (r < bw && c <= r) ? A[(size_t)(kb + r) * n + kb + c] : 0.0f;
    }
    if (threadIdx.x == 0) s_fail = 0;
    __syncthreads();
    for (int k = 0; k < bw; k++) {
        if (threadIdx.x == 0) {
            const float d = D[k][k];
            if (d <= 0.0f) s_fail = 1;                                    // gptq.rs:290-292
            else D[k][k] = __fsqrt_rn(d);
        }
        __syncthreads();
        if (s_fail) break;
        const float lkk = D[k][k];
        for (int i = k + 1 + threadIdx.x; i < bw; i += 256) D[i][k] = __fdiv_rn(D[i][k], lkk);
        __syncthreads();
        for (int t = threadIdx.x; t < NB * NB; t += 256) {
            const int i = t / NB, j = t % NB;
            if (j > k && j <= i && i < bw) D[i][j] = mulsub(D[i][j], D[i][k], D[j][k]);
        }
        __syncthreads();
    }
    if (s_fail) {
        if (threadIdx.x == 0) { ctl[CTL_FAIL] = 1; info[0] = 1; }
        return;
    }
    for (int t = threadIdx.x; t < NB * NB; t += 256) {
        const int r = t / NB, c = t % NB;
        if (c <= r && r < bw) A[(size_t)(kb + r) * n + kb + c] = D[r][c];
    }
}

// The panel below a factored diagonal block: one thread per row, 32 columns solved in order.
__global__ void __launch_bounds__(256) chol_panel_kernel(float* __restrict__ A, int n, int kb, const uint32_t* ctl) {
    if (ld_volatile(ctl + CTL_FAIL)) return;
    __shared__ float D[NB][NB + 1];
    for (int t = threadIdx.x; t < NB * NB; t += 256) {
        const int r = t / NB, c = t % NB;
        D[r][c] = c <= r ? A[(size_t)(kb + r) * n + kb + c] : 0.0f;
    }
    __syncthreads();
    const int i = kb + NB + blockIdx.x * 256 + threadIdx.x;
    if (i >= n) return;
    float a[NB];
    float* row = A + (size_t)i * n + kb;
#pragma unroll
    for (int c = 0; c < NB; c++) a[c] = row[c];
#pragma unroll
    for (int j = 0; j < NB; j++) {
        float s = a[j];
#pragma unroll
        for (int k = 0; k < j; k++) s = mulsub(s, a[k], D[j][k]);
        a[j] = __fdiv_rn(s, D[j][j]);
    }
#pragma unroll
    for (int c = 0; c < NB; c++) row[c] = a[c];
}

// Trailing update of one block column: a[i][j] -= sum over the 32 columns of the panel, in increasing k.
__global__ void __launch_bounds__(256) chol_trailing_kernel(float* __restrict__ A, int n, int kb, const uint32_t* ctl) {
    if (ld_volatile(ctl + CTL_FAIL)) return;
    const int ti = blockIdx.y, tj = blockIdx.x;
    if (tj > ti) return;
    __shared__ float Pi[64][NB + 1], Pj[64][NB + 1];
    const int t0 = kb + NB, i0 = t0 + ti * 64, j0 = t0 + tj * 64;
    for (int t = threadIdx.x; t < 64 * NB; t += 256) {
        const int r = t / NB, k = t % NB;
        Pi[r][k] = i0 + r < n ? A[(size_t)(i0 + r) * n + kb + k] : 0.0f;
        Pj[r][k] = j0 + r < n ? A[(size_t)(j0 + r) * n + kb + k] : 0.0f;
    }
    __syncthreads();
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    float acc[4][4];
#pragma unroll
    for (int u = 0; u < 4; u++)
#pragma unroll
        for (int v = 0; v < 4; v++) {
            const int i = i0 + ty + 16 * u, j = j0 + tx + 16 * v;
            acc[u][v] = (i < n && j <= i) ? A[(size_t)i * n + j] : 0.0f;
        }
#pragma unroll 8
    for (int k = 0; k < NB; k++) {
        float a[4], b[4];
#pragma unroll
        for (int u = 0; u < 4; u++) { a[u] = Pi[ty + 16 * u][k]; b[u] = Pj[tx + 16 * u][k]; }
#pragma unroll
        for (int u = 0; u < 4; u++)
#pragma unroll
            for (int v = 0; v < 4; v++) acc[u][v] = mulsub(acc[u][v], a[u], b[v]);
    }
#pragma unroll
    for (int u = 0; u < 4; u++)
#pragma unroll
        for (int v = 0; v < 4; v++) {
            const int i = i0 + ty + 16 * u, j = j0 + tx + 16 * v;
            if (i < n && j <= i) A[(size_t)i * n + j] = acc[u][v];
        }
}

// The inverse of the factor, right-looking by blocks of 32 rows.  Until a row block is finished, LI[i][j] holds
// the running sum s of invert_lower (gptq.rs:310-314); the trailing kernel below adds a finished block's 32 terms
// to every later row, in increasing k, and this kernel finishes rows [ib, ib + 32): the terms inside the block and
// the division by the diagonal, one thread per column.
__global__ void __launch_bounds__(64) invl_diag_kernel(const float* __restrict__ L, float* __restrict__ LI, int n, int ib, const uint32_t* ctl) {
    if (ld_volatile(ctl + CTL_FAIL)) return;
    __shared__ float Ld[NB][NB + 1];
    __shared__ float X[NB][64];
    const int bh = min(NB, n - ib);
    const int c = threadIdx.x, j = blockIdx.x * 64 + c;
    for (int t = threadIdx.x; t < NB * NB; t += 64) {
        const int r = t / NB, k = t % NB;
        Ld[r][k] = (r < bh && k <= r) ? L[(size_t)(ib + r) * n + ib + k] : 0.0f;
    }
    const bool live = j < ib + bh;
    if (live) {
        for (int r = 0; r < bh; r++) X[r][c] = LI[(size_t)(ib + r) * n + j];
    }
    __syncthreads();
    if (!live) return;
    for (int r = 0; r < bh; r++) {
        const int i = ib + r;
        if (j > i) continue;
        const float lii = Ld[r][r];
        float v;
        if (j == i) {
            v = __fdiv_rn(1.0f, lii);
        } else {
            float s = X[r][c];
            for (int kk = max(0, j - ib); kk < r; kk++) s = muladd(s, Ld[r][kk], X[kk][c]);
            v = __fdiv_rn(-s, lii);
        }
        X[r][c] = v;
        LI[(size_t)i * n + j] = v;
    }
}

// s[i][j] += l[i][k] * li[k][j] for the 32 finished rows k of block ib, every later row i and every column j that
// those rows reach; 64 x 64 tiles.
__global__ void __launch_bounds__(256) invl_trailing_kernel(const float* __restrict__ L, float* __restrict__ LI, int n, int ib, const uint32_t* ctl) {
    if (ld_volatile(ctl + CTL_FAIL)) return;
    __shared__ float Pa[64][NB + 1];
    __shared__ float Pb[NB][64];
    const int i0 = ib + NB + blockIdx.y * 64, j0 = blockIdx.x * 64, jend = ib + NB;
    for (int t = threadIdx.x; t < 64 * NB; t += 256) {
        const int r = t / NB, k = t % NB;
        Pa[r][k] = i0 + r < n ? L[(size_t)(i0 + r) * n + ib + k] : 0.0f;
        const int kk = t / 64, cc = t % 64;
        Pb[kk][cc] = j0 + cc < jend ? LI[(size_t)(ib + kk) * n + j0 + cc] : 0.0f;
    }
    __syncthreads();
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    float acc[4][4];
#pragma unroll
    for (int u = 0; u < 4; u++)
#pragma unroll
        for (int v = 0; v < 4; v++) {
            const int i = i0 + ty + 16 * u, j = j0 + tx + 16 * v;
            acc[u][v] = (i < n && j < jend) ? LI[(size_t)i * n + j] : 0.0f;
        }
#pragma unroll 8
    for (int k = 0; k < NB; k++) {
        float a[4], b[4];
#pragma unroll
        for (int u = 0; u < 4; u++) { a[u] = Pa[ty + 16 * u][k]; b[u] = Pb[k][tx + 16 * u]; }
#pragma unroll
        for (int u = 0; u < 4; u++)
#pragma unroll
            for (int v = 0; v < 4; v++) acc[u][v] = muladd(acc[u][v], a[u], b[v]);
    }
#pragma unroll
    for (int u = 0; u < 4; u++)
#pragma unroll
        for (int v = 0; v < 4; v++) {
            const int i = i0 + ty + 16 * u, j = j0 + tx + 16 * v;
            if (i < n && j < jend) LI[(size_t)i * n + j] = acc[u][v];
        }
}

// Upper triangle of H^-1 = (L^-1)^T L^-1 in 64 x 64 tiles; rows of L^-1 above the tile's first column are zero and
// are not visited.
__global__ void __launch_bounds__(256) hinv_kernel(const float* __restrict__ LI, float* __restrict__ HINV, int n, const uint32_t* ctl) {
    if (ld_volatile(ctl + CTL_FAIL)) return;
    const int tj = blockIdx.y, tk = blockIdx.x;
    if (tj > tk) return;
    __shared__ float Pj[NB][64], Pk[NB][64];
    const int j0 = tj * 64, k0 = tk * 64;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    float acc[4][4];
#pragma unroll
    for (int u = 0; u < 4; u++)
#pragma unroll
        for (int v = 0; v < 4; v++) acc[u][v] = 0.0f;
    for (int m0 = k0; m0 < n; m0 += NB) {
        __syncthreads();
        for (int t = threadIdx.x; t < NB * 64; t += 256) {
            const int mm = t / 64, cc = t % 64;
            const bool in = m0 + mm < n;
            Pj[mm][cc] = (in && j0 + cc < n) ? LI[(size_t)(m0 + mm) * n + j0 + cc] : 0.0f;
            Pk[mm][cc] = (in && k0 + cc < n) ? LI[(size_t)(m0 + mm) * n + k0 + cc] : 0.0f;
        }
        __syncthreads();
        const int mend = min(NB, n - m0);
#pragma unroll 4
        for (int mm = 0; mm < mend; mm++) {
            float a[4], b[4];
#pragma unroll
            for (int u = 0; u < 4; u++) { a[u] = Pj[mm][ty + 16 * u]; b[u] = Pk[mm][tx + 16 * u]; }
#pragma unroll
            for (int u = 0; u < 4; u++)
#pragma unroll
                for (int v = 0; v < 4; v++) acc[u][v] = muladd(acc[u][v], a[u], b[v]);
        }
    }
#pragma unroll
    for (int u = 0; u < 4; u++)
#pragma unroll
        for (int v = 0; v < 4; v++) {
            const int j = j0 + ty + 16 * u, k = k0 + tx + 16 * v;
            if (k < n && j <= k) HINV[(size_t)j * n + k] = acc[u][v];
        }
}

struct ColParams {
    const float* W;          // [R][n] original weights
    const float* HINV;       // [n][n], upper triangle
    float* ERRS;             // [R][n] per-row errors of every finished column
    unsigned long long* slots;   // [2][2][SLOT_MAX] published column statistics (see post_stats)
    uint32_t* ctl;
    int32_t* Q;              // [R][n]
    float* scales;           // [n]
    int32_t* zps;            // [n]
    int32_t* status;
    int R, n, rpc, bits, symmetric;
};

constexpr int SLOT_MAX = 1024;          // CTAs of the column loop at most

__device__ __forceinline__ float stat_init_max(int symmetric) { return symmetric ? 0.0f : __int_as_float(0xFF800000); }
// NaNs are skipped by the comparisons, as in the reference's folds (gptq.rs:253-268)
__device__ __forceinline__ void stat_add(int symmetric, float v, float& mx, float& mn) {
    if (symmetric) { const float a = fabsf(v); if (a > mx) mx = a; }
    else { if (v > mx) mx = v; if (v < mn) mn = v; }
}

// The meeting point of the column loop.  Each CTA publishes its statistics of column j as one 64-bit word per value,
// (j + 1) << 32 | ordered key, in its own slot; a reader takes a slot once it carries the tag of the column it waits
// for, so neither atomics nor fences are needed.  Two sets of slots alternate by the parity of j: a CTA can only
// publish column j + 2 after every CTA has published j + 1, i.e. after every CTA has finished reading column j.
__device__ __forceinline__ void post_stats(const ColParams& p, int j, float mx, float mn) {
    volatile unsigned long long* s = p.slots + (size_t)(j & 1) * 2 * SLOT_MAX;
    const unsigned long long tag = (unsigned long long)(uint32_t)(j + 1) << 32;
    s[blockIdx.x] = tag | order_key(mx);
    if (!p.symmetric) s[SLOT_MAX + blockIdx.x] = tag | order_key(mn);
}

// Warp-wide: waits (bounded: two seconds) for every CTA's slot of column j and reduces them; false on a timeout.
// A lane asks for all of its slots at once (eight per pass), so a pass costs one trip to the L2, not one per slot.
__device__ __forceinline__ bool collect_stats(const ColParams& p, int j, int lane, float& mx, float& mn) {
    const volatile unsigned long long* s = p.slots + (size_t)(j & 1) * 2 * SLOT_MAX;
    const uint32_t tag = (uint32_t)(j + 1);
    const int G = (int)gridDim.x;
    mx = stat_init_max(p.symmetric);
    mn = __int_as_float(0x7F800000);
    bool ok = true;
    uint64_t t0, t1;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
    for (int k0 = 0; k0 < G && ok; k0 += 256) {
        unsigned long long v[8], u[8];
        for (uint32_t it = 0;; ++it) {
            bool all = true;
#pragma unroll
            for (int x = 0; x < 8; x++) {
                const int k = k0 + 32 * x + lane;
                v[x] = k < G ? s[k] : (unsigned long long)tag << 32 | order_key(mx);
                u[x] = (k < G && !p.symmetric) ? s[SLOT_MAX + k] : (unsigned long long)tag << 32 | order_key(mn);
            }
#pragma unroll
            for (int x = 0; x < 8; x++) all = all && (uint32_t)(v[x] >> 32) == tag && (uint32_t)(u[x] >> 32) == tag;
            if (all) break;
            if ((it & 255u) == 255u) {
                asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t1));
                if (t1 - t0 > 2000000000ull) { ok = false; break; }
            }
        }
        if (ok) {
#pragma unroll
            for (int x = 0; x < 8; x++) { mx = fmaxf(mx, order_unkey((uint32_t)v[x])); mn = fminf(mn, order_unkey((uint32_t)u[x])); }
        }
    }
    ok = __all_sync(0xffffffffu, ok);
    mx = warp_max(mx);
    mn = warp_min(mn);
    return ok;
}

__device__ __forceinline__ int32_t quant_scalar(float x, float scale, float zpf, float lo, float hi) {
    float v = roundf(__fadd_rn(__fdiv_rn(x, scale), zpf));                // f32::round: half away from zero
    if (v < lo) v = lo;
    if (v > hi) v = hi;
    return v != v ? 0 : (int32_t)v;                                       // NaN as i32 == 0
}

__global__ void __launch_bounds__(256, 1) gptq_columns_kernel(ColParams p) {
    if (ld_volatile(p.ctl + CTL_FAIL)) return;
    extern __shared__ __align__(16) float smem[];
    float* w_s = smem;                                  // [rpc][CBP] current block of weights; finished columns hold the codes
    float* eb_s = w_s + (size_t)p.rpc * CBP;            // [rpc][CBP] errors of the block's columns
    float* E_s = smem + (((size_t)2 * p.rpc * CBP + 3) & ~(size_t)3);   // [32][CB] staged errors of earlier columns (16-byte aligned)
    float* H_s = E_s + 32 * CB;                         // [CB][CB]   staged tile of H^-1: rows = source columns, columns = this block
    __shared__ float Dg_s[CB];
    __shared__ float s_scale;
    __shared__ int s_zp, s_abort;
    const int n = p.n, tid = threadIdx.x;
    const int r0 = blockIdx.x * p.rpc;
    const int nr = min(p.rpc, p.R - r0);
    const int c = tid & 63, g = tid >> 6;
    const int q_min = p.symmetric ? -(1 << (p.bits - 1)) : 0;
    const int q_max = p.symmetric ? (1 << (p.bits - 1)) - 1 : (1 << p.bits) - 1;
    const float lo = (float)q_min, hi = (float)q_max;
    if (tid == 0) s_abort = 0;

    for (int b0 = 0; b0 < n; b0 += CB) {
        const int bw = min(CB, n - b0);
        for (int t = tid; t < nr * CB; t += 256) {
            const int r = t / CB, cc = t % CB;
            w_s[r * CBP + cc] = cc < bw ? p.W[(size_t)(r0 + r) * n + b0 + cc] : 0.0f;
        }
        __syncthreads();
        // corrections from every column before this block, in increasing column order
        if (b0 > 0) {
            for (int rc0 = 0; rc0 < nr; rc0 += 32) {
                float acc[8];
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    const int row = rc0 + g * 8 + u;
                    acc[u] = row < nr ? w_s[row * CBP + c] : 0.0f;
                }
                // tiles of 64 earlier columns: the next tile's errors and its rows of H^-1 are fetched into registers
                // while the current one is consumed from shared memory
                float er[8], hr[16], dg = 0.0f;
                auto fetch = [&](int jt) {
#pragma unroll
                    for (int x = 0; x < 8; x++) {
                        const int t = tid + 256 * x, r = t / CB, jj = t % CB, row = rc0 + r;
                        er[x] = row < nr ? p.ERRS[(size_t)(r0 + row) * n + jt + jj] : 0.0f;
                    }
#pragma unroll
                    for (int x = 0; x < 16; x++) {
                        const int t = tid + 256 * x, jj = t / CB, cc = t % CB;
                        hr[x] = __ldg(p.HINV + (size_t)(jt + jj) * n + b0 + min(cc, bw - 1));
                    }
                    if (tid < CB) dg = __ldg(p.HINV + (size_t)(jt + tid) * n + jt + tid);
                };
                fetch(0);
                for (int jt = 0; jt < b0; jt += CB) {
                    __syncthreads();
#pragma unroll
                    for (int x = 0; x < 8; x++) E_s[tid + 256 * x] = er[x];
#pragma unroll
                    for (int x = 0; x < 16; x++) H_s[tid + 256 * x] = hr[x];
                    if (tid < CB) Dg_s[tid] = dg;
                    __syncthreads();
                    if (jt + CB < b0) fetch(jt + CB);
#pragma unroll 2
                    for (int jj = 0; jj < CB; jj += 4) {
                        float h[4];
#pragma unroll
                        for (int x = 0; x < 4; x++) h[x] = H_s[(jj + x) * CB + c];
                        float4 e[8];
#pragma unroll
                        for (int u = 0; u < 8; u++) e[u] = *reinterpret_cast<const float4*>(&E_s[(g * 8 + u) * CB + jj]);
                        if (!(Dg_s[jj] < kDegenerate)) {
#pragma unroll
                            for (int u = 0; u < 8; u++) acc[u] = mulsub(acc[u], e[u].x, h[0]);
                        }
                        if (!(Dg_s[jj + 1] < kDegenerate)) {
#pragma unroll
                            for (int u = 0; u < 8; u++) acc[u] = mulsub(acc[u], e[u].y, h[1]);
                        }
                        if (!(Dg_s[jj + 2] < kDegenerate)) {
#pragma unroll
                            for (int u = 0; u < 8; u++) acc[u] = mulsub(acc[u], e[u].z, h[2]);
                        }
                        if (!(Dg_s[jj + 3] < kDegenerate)) {
#pragma unroll
                            for (int u = 0; u < 8; u++) acc[u] = mulsub(acc[u], e[u].w, h[3]);
                        }
                    }
                }
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    const int row = rc0 + g * 8 + u;
                    if (row < nr) w_s[row * CBP + c] = acc[u];
                }
            }
            __syncthreads();
        }
        // the block's own columns, one at a time; their rows of H^-1 (the part inside the block) wait in shared memory
        for (int t = tid; t < CB * CB; t += 256) {
            const int jj = t / CB, cc = t % CB;
            H_s[t] = (jj < bw && cc >= jj && cc < bw) ? __ldg(p.HINV + (size_t)(b0 + jj) * n + b0 + cc) : 0.0f;
        }
        __syncthreads();
        if (tid < 32) {                                                    // this CTA's statistics of the block's first column
            float mx = stat_init_max(p.symmetric), mn = __int_as_float(0x7F800000);
            for (int row = tid; row < nr; row += 32) stat_add(p.symmetric, w_s[row * CBP], mx, mn);
            mx = warp_max(mx);
            mn = warp_min(mn);
            if (tid == 0) post_stats(p, b0, mx, mn);
        }
        for (int jj = 0; jj < bw; jj++) {
            const int j = b0 + jj;
            if (tid < 32) {
                // every CTA's statistics of column j: the maximum over all rows of the layer
                float mx, mn;
                const bool ok = collect_stats(p, j, tid, mx, mn);
                if (tid == 0) {
                    if (!ok) { atomicExch(p.status, OXQ_ERR_DEVICE_TIMEOUT); s_abort = 1; }
                    float scale; int zp = 0;
                    if (p.symmetric) {
                        float am = mx;
                        if (!(am > 1e-8f)) am = 1e-8f;
                        scale = __fdiv_rn(am, hi);
                    } else {
                        float range = __fsub_rn(mx, mn);
                        if (!(range > 1e-8f)) range = 1e-8f;
                        scale = __fdiv_rn(range, (float)((1 << p.bits) - 1));
                        float z = roundf(__fdiv_rn(-mn, scale));
                        if (z < lo) z = lo;
                        if (z > hi) z = hi;
                        zp = z != z ? 0 : (int)z;
                    }
                    s_scale = scale; s_zp = zp;
                    if (blockIdx.x == 0) { p.scales[j] = scale; p.zps[j] = zp; }
                }
            }
            __syncthreads();
            if (s_abort) return;
            const float scale = s_scale, zpf = (float)s_zp;
            const float hjj = H_s[jj * CB + jj];
            const bool degenerate = hjj < kDegenerate;                    // gptq.rs:209-216: round to nearest, no correction
            for (int row = tid; row < nr; row += 256) {
                const float wij = w_s[row * CBP + jj];
                const int32_t q = quant_scalar(wij, scale, zpf, lo, hi);
                w_s[row * CBP + jj] = __int_as_float(q);
                float e = 0.0f;
                if (!degenerate) e = __fdiv_rn(__fsub_rn(wij, __fmul_rn(__fsub_rn((float)q, zpf), scale)), hjj);
                eb_s[row * CBP + jj] = e;
            }
            __syncthreads();
            if (tid < 32 && jj + 1 < bw) {
                // the next column first: correct it, take its statistics and post them, so that the other CTAs'
                // answers travel while the rest of the block is corrected
                const float h = H_s[jj * CB + jj + 1];
                float mx = stat_init_max(p.symmetric), mn = __int_as_float(0x7F800000);
                for (int row = tid; row < nr; row += 32) {
                    float v = w_s[row * CBP + jj + 1];
                    if (!degenerate) { v = mulsub(v, eb_s[row * CBP + jj], h); w_s[row * CBP + jj + 1] = v; }
                    stat_add(p.symmetric, v, mx, mn);
                }
                mx = warp_max(mx);
                mn = warp_min(mn);
                if (tid == 0) post_stats(p, j + 1, mx, mn);
            }
            if (!degenerate && c > jj + 1 && c < bw) {
                const float h = H_s[jj * CB + c];
                for (int row = g; row < nr; row += 4) w_s[row * CBP + c] = mulsub(w_s[row * CBP + c], eb_s[row * CBP + jj], h);
            }
            __syncthreads();
        }
        for (int t = tid; t < nr * CB; t += 256) {
            const int r = t / CB, cc = t % CB;
            if (cc < bw) {
                p.Q[(size_t)(r0 + r) * n + b0 + cc] = __float_as_int(w_s[r * CBP + cc]);
                p.ERRS[(size_t)(r0 + r) * n + b0 + cc] = eb_s[r * CBP + cc];
            }
        }
        __syncthreads();
    }
}

// workspace: A / H^-1 [n][n], L^-1 [n][n], errors [R][n], then (16-byte aligned) the control words and the slots
size_t gptq_tail_offset(int64_t R, int64_t n) { return (((size_t)(2 * n * n + R * n) * sizeof(float)) + 15) & ~(size_t)15; }
size_t gptq_ws_bytes(int64_t R, int64_t n) { return gptq_tail_offset(R, n) + CTL_WORDS * sizeof(uint32_t) + 4 * SLOT_MAX * sizeof(unsigned long long); }

}  // namespace
}  // namespace oxq

using namespace oxq;

extern "C" {

int32_t oxq_gptq_workspace_bytes(int64_t n_rows, int64_t n_cols, size_t* bytes) {
    if (!bytes || n_rows < 0 || n_cols < 0) return OXQ_ERR_INVALID_ARGUMENT;
    *bytes = gptq_ws_bytes(n_rows, n_cols);
    return OXQ_OK;
}

int32_t oxq_gptq_quantize_layer(oxq_handle* h, const float* weights, int64_t n_rows, int64_t n_cols, const float* hessian, int bits,
                                int symmetric, double percdamp, int32_t* quantized, float* scales, int32_t* zero_points, int32_t* info,
                                void* workspace, size_t workspace_bytes) {
    OXQ_CHECK_HANDLE(h);
    if (n_rows <= 0 || n_cols <= 0) OXQ_FAIL(h, OXQ_ERR_EMPTY_INPUT, "GptqQuantizer::quantize_layer");
    if (bits <= 0 || bits > 16) OXQ_FAIL(h, OXQ_ERR_INVALID_BIT_WIDTH, "bits = %d", bits);
    if (!weights || !hessian || !quantized || !scales || !zero_points || !info || !workspace) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "null pointer");
    if (n_cols > 32768 || n_rows * n_cols > (int64_t)1 << 31) OXQ_FAIL(h, OXQ_ERR_UNSUPPORTED_OPERATION, "layer too large: %lld x %lld", (long long)n_rows, (long long)n_cols);
    if (workspace_bytes < gptq_ws_bytes(n_rows, n_cols)) OXQ_FAIL(h, OXQ_ERR_BUFFER_TOO_SMALL, "workspace needs %zu bytes, got %zu", gptq_ws_bytes(n_rows, n_cols), workspace_bytes);
    if ((uintptr_t)workspace & 15) OXQ_FAIL(h, OXQ_ERR_INVALID_ARGUMENT, "workspace must be 16-byte aligned");
    if (int32_t rc = oxq_require_sm100(h)) return rc;
    const int n = (int)n_cols, R = (int)n_rows;
    float* A = (float*)workspace;                       // dampened Hessian -> L (lower) -> H^-1 (upper)
    float* LI = A + (size_t)n * n;
    float* ERRS = LI + (size_t)n * n;
    uint32_t* ctl = (uint32_t*)((char*)workspace + gptq_tail_offset(R, n));
    unsigned long long* slots = (unsigned long long*)(ctl + CTL_WORDS);
    cudaStream_t st = h->stream;

    // the column loop's grid: every CTA resident (cooperative launch), rows split evenly
    int rpc = (R + h->sm_count - 1) / h->sm_count;
    const size_t smem = ((((size_t)2 * rpc * CBP + 3) & ~(size_t)3) + 32 * CB + CB * CB) * sizeof(float);
    if (smem > 220 * 1024) OXQ_FAIL(h, OXQ_ERR_UNSUPPORTED_OPERATION, "n_rows = %d needs %zu bytes of shared memory per CTA", R, smem);
    OXQ_CUDA(h, cudaFuncSetAttribute(gptq_columns_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    int occ = 0;
    OXQ_CUDA(h, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, gptq_columns_kernel, 256, smem));
    const int grid_cols = (R + rpc - 1) / rpc;
    if (occ < 1 || grid_cols > occ * h->sm_count || grid_cols > SLOT_MAX) OXQ_FAIL(h, OXQ_ERR_LAUNCH_FAILED, "column kernel cannot be made resident (%d CTAs, occupancy %d)", grid_cols, occ);

    OXQ_CUDA(h, oxq_launch<false>(gptq_prepare_kernel, dim3(1), dim3(256), 0, st, hessian, n, (float)percdamp, ctl, info, slots, 4 * SLOT_MAX));
    OXQ_CUDA(h, oxq_launch<false>(gptq_damp_kernel, dim3(h->sm_count * 4), dim3(256), 0, st, hessian, A, n, (const uint32_t*)ctl));
    OXQ_CUDA(h, cudaMemsetAsync(LI, 0, (size_t)n * n * sizeof(float), st));
    for (int kb = 0; kb < n; kb += NB) {
        const int below = n - kb - NB;
        OXQ_CUDA(h, oxq_launch<false>(chol_diag_kernel, dim3(1), dim3(256), 0, st, A, n, kb, ctl, info));
        if (below > 0) {
            const int T = (below + 63) / 64;
            OXQ_CUDA(h, oxq_launch<false>(chol_panel_kernel, dim3((below + 255) / 256), dim3(256), 0, st, A, n, kb, (const uint32_t*)ctl));
            OXQ_CUDA(h, oxq_launch<false>(chol_trailing_kernel, dim3(T, T), dim3(256), 0, st, A, n, kb, (const uint32_t*)ctl));
        }
    }
    for (int ib = 0; ib < n; ib += NB) {
        const int cols = min(ib + NB, n), below = n - ib - NB;
        OXQ_CUDA(h, oxq_launch<false>(invl_diag_kernel, dim3((cols + 63) / 64), dim3(64), 0, st, (const float*)A, LI, n, ib, (const uint32_t*)ctl));
        if (below > 0)
            OXQ_CUDA(h, oxq_launch<false>(invl_trailing_kernel, dim3((cols + 63) / 64, (below + 63) / 64), dim3(256), 0, st, (const float*)A, LI, n, ib, (const uint32_t*)ctl));
    }
    {
        const int T = (n + 63) / 64;
        OXQ_CUDA(h, oxq_launch<false>(hinv_kernel, dim3(T, T), dim3(256), 0, st, (const float*)LI, A, n, (const uint32_t*)ctl));
    }
    ColParams p;
    p.W = weights; p.HINV = A; p.ERRS = ERRS; p.slots = slots; p.ctl = ctl; p.Q = quantized; p.scales = scales; p.zps = zero_points;
    p.status = h->dev_status; p.R = R; p.n = n; p.rpc = rpc; p.bits = bits; p.symmetric = symmetric ? 1 : 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid_cols); cfg.blockDim = dim3(256); cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeCooperative;
    attr.val.cooperative = 1;
    cfg.attrs = &attr; cfg.numAttrs = 1;
    OXQ_CUDA(h, cudaLaunchKernelEx(&cfg, gptq_columns_kernel, p));
    return OXQ_OK;
}

}  // extern "C"
