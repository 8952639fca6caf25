// Factored step for 2-D tensors: Adafactor (row / column second moments) and
// CAME (confidence-guided, with momentum).
//
// Reference semantics: _update_param_8bit factored branch on the pure-PyTorch
// route (optimizer.py:2202-2253 statistics and small-state EMAs, 2394-2399 and
// 2543-2549 dispatch), _factored_inv_std (optimizer.py:818-821),
// _compute_ut_clipped (optimizer.py:824-829), _fallback_2d_update
// (optimizer.py:920-970).
//
// Three kernels, each launched once for a whole table of tensors:
//   factored_stats_kernel   row and column sums of g*g, or of CAME's residual
//                           (U - M)^2 + eps, over 64 x 256 tiles.  Every product
//                           is rounded to binary32 as torch does and then
//                           accumulated in binary64, so the binary32 means do not
//                           depend on the order of accumulation.
//   factored_small_kernel   one CTA per tensor: means, EMA into the (tiny) row /
//                           column AL states with exact requantisation, mean of
//                           the row state, inverse-std vectors.
//   factored_update_kernel  flat chunks aligned to momentum blocks: the update
//                           itself, its sum of squares, the parameter write and
//                           the momentum requantisation.
#pragma once

#include <type_traits>

#include "common.cuh"
#include "fullrank_fast.cuh"
#include "fullrank_generic.cuh"
#include "fullrank_stat.cuh"
#include "tensormap.cuh"

namespace af8 {

constexpr int FSTAT_ROWS = 512;
constexpr int FSTAT_COLS = 256;
constexpr int FUPD_THREADS = 256;
constexpr int DEVERR_SRING_TIMEOUT = 4;      // a bulk copy of the statistic pass's input ring did not land

struct FactoredLaunch {
    const af8_factored_tensor *tensors;
    const af8_dyn_scalars *dyn;
    double *block_sumsq;
    int64_t total_units;
    int32_t n_tensors;
    int32_t grad_dtype, m_fmt, m_block, came, negate_grad, mode;
    float v_floor;
    int32_t param_dtype, sr;
};

__device__ __forceinline__ int find_factored_tile(const af8_factored_tensor *t, int n, int64_t id)
{
    int lo = 0, hi = n - 1;
    while (lo < hi) {
        int mid = (lo + hi + 1) >> 1;
        if (__ldg(&t[mid].first_tile) <= id) lo = mid; else hi = mid - 1;
    }
    return lo;
}
__device__ __forceinline__ int find_factored_chunk(const af8_factored_tensor *t, int n, int64_t id)
{
    int lo = 0, hi = n - 1;
    while (lo < hi) {
        int mid = (lo + hi + 1) >> 1;
        if (__ldg(&t[mid].first_chunk) <= id) lo = mid; else hi = mid - 1;
    }
    return lo;
}

// batches of matrices (batch_rows > 0): number of matrices, rows of one, and the stat tiles of one
__host__ __device__ __forceinline__ int64_t fact_mat_rows(const af8_factored_tensor &t) { return t.batch_rows > 0 ? t.batch_rows : t.rows; }
__host__ __device__ __forceinline__ int64_t fact_batch(const af8_factored_tensor &t) { return t.batch_rows > 0 ? t.rows / t.batch_rows : 1; }
__host__ __device__ __forceinline__ int64_t fact_tiles(const af8_factored_tensor &t)
{
    return fact_batch(t) * ((fact_mat_rows(t) + FSTAT_ROWS - 1) / FSTAT_ROWS) * ((t.cols + FSTAT_COLS - 1) / FSTAT_COLS);
}
// first entry of the column arrays for the matrix that holds row `row`
__device__ __forceinline__ int64_t fact_col_base(const af8_factored_tensor &t, int64_t row)
{
    return t.batch_rows > 0 ? (row / t.batch_rows) * t.cols : 0;
}

__device__ __forceinline__ float load_grad_any(const void *g, int dtype, int64_t i)
{
    if (dtype == AF8_F32) return static_cast<const float *>(g)[i];
    const uint32_t h = static_cast<const uint16_t *>(g)[i];
    return dtype == AF8_BF16 ? bf16_bits_to_f32(h) : f16_bits_to_f32(h);
}

// momentum before the EMA (optimizer.py:694-697): dequantised codes or the fp32 state
__device__ __forceinline__ float m_old_at(const af8_factored_tensor &T, int m_fmt, int m_block, int64_t flat)
{
    if (m_fmt == AF8_M_FP32) return T.m_f32[flat];
    return m_decode(T.m_q, __ldg(T.m_scale + flat / m_block), flat, m_fmt);
}

// Tensor.lerp_ with a weight that is the same for many elements: the choice between ATen's two
// forms is made once (LerpW), an element costs a subtraction, a select and one fma.
struct LerpW { float ww; bool small; };
__device__ __forceinline__ LerpW make_lerp(float w)
{
    LerpW l;
    l.small = fabsf(w) < 0.5f;
    l.ww = l.small ? w : __fsub_rn(w, 1.0f);
    return l;
}
__device__ __forceinline__ float lerp_w(float s, float e, const LerpW &l)
{
    return __fmaf_rn(l.ww, __fsub_rn(e, s), l.small ? s : e);
}

// U = g * inv_row * inv_col, then the RMS clip divisor (optimizer.py:825-828)
__device__ __forceinline__ float u_clipped(float g, float ir, float ic, float pre_div)
{
    float u = __fmul_rn(__fmul_rn(g, ir), ic);
    if (pre_div != 1.0f) u = __fdiv_rn(u, pre_div);
    return u;
}

// x / d for one divisor and many dividends: the correctly rounded reciprocal and one
// residual step give the IEEE quotient (checked against the division on 2e9 random
// normal operands; the unrefined product stands when it is infinite or NaN).
struct DivBy {
    float rcp, nd;
    bool one;
};
__device__ __forceinline__ DivBy make_div(float d)
{
    DivBy D;
    D.one = d == 1.0f;
    D.rcp = __frcp_rn(d);
    D.nd = -d;
    return D;
}
__device__ __forceinline__ float div_by(float x, const DivBy &D)
{
    if (D.one) return x;
    const float q = __fmul_rn(x, D.rcp);
    const float q2 = __fmaf_rn(__fmaf_rn(q, D.nd, x), D.rcp, q);
    return fabsf(q) <= 3.402823466e38f ? q2 : q;
}
__device__ __forceinline__ float u_clipped_fast(float g, float ir, float ic, const DivBy &D)
{
    return div_by(__fmul_rn(__fmul_rn(g, ir), ic), D);
}

// UF8 code of m for a block absmax a >= 1e-12 (optimizer.py:512): round(m / a * 128) clamped
// to [-128, 127], plus 128; the division as above
__device__ __forceinline__ uint32_t uf8_encode_fast(float m, const DivBy &A)
{
    const float q = __fmul_rn(m, A.rcp);
    const float q2 = __fmaf_rn(__fmaf_rn(q, A.nd, m), A.rcp, q);       // |q| <= 1: always finite
    const float kf = __fmaf_rn(q2, 128.0f, 12582912.0f);               // exact product, round half to even
    const int k = min(__float_as_int(kf), 0x4b400000 + 127);           // only +128 needs the clamp
    return (uint32_t)(k - 0x4b400000 + 128);
}

// The same helpers on pairs of elements with Blackwell's packed binary32 instructions (one
// instruction per pair; each component rounds exactly like the scalar operation).
__device__ __forceinline__ float2 div_by2(float2 x, const DivBy &D)
{
    if (D.one) return x;
    const float2 r2 = bc2(D.rcp);
    const float2 q = __fmul2_rn(x, r2);
    const float2 q2 = __ffma2_rn(__ffma2_rn(q, bc2(D.nd), x), r2, q);
    return make_float2(fabsf(q.x) <= 3.402823466e38f ? q2.x : q.x, fabsf(q.y) <= 3.402823466e38f ? q2.y : q.y);
}
__device__ __forceinline__ float2 lerp_w2(float2 s, float2 e, const LerpW &l)
{
    return __ffma2_rn(bc2(l.ww), sub2(e, s), l.small ? s : e);
}
// two UF8 codes, the first in the low byte
__device__ __forceinline__ uint32_t uf8_encode_fast2(float2 m, const DivBy &A)
{
    const float2 r2 = bc2(A.rcp);
    const float2 q = __fmul2_rn(m, r2);
    const float2 q2 = __ffma2_rn(__ffma2_rn(q, bc2(A.nd), m), r2, q);
    const float2 kf = __ffma2_rn(q2, bc2(128.0f), bc2(12582912.0f));
    const int k0 = min(__float_as_int(kf.x), 0x4b400000 + 127), k1 = min(__float_as_int(kf.y), 0x4b400000 + 127);
    return (uint32_t)(k0 - 0x4b400000 + 128) | ((uint32_t)(k1 - 0x4b400000 + 128) << 8);
}

// ---------------------------------------------------------------------------
// statistics
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
factored_stats_kernel(const FactoredLaunch L)
{
    __shared__ double s_col[FSTAT_COLS];
    __shared__ af8_factored_tensor sT;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    for (int64_t id = blockIdx.x; id < L.total_units; id += gridDim.x) {
        const int t = find_factored_tile(L.tensors, L.n_tensors, id);
        __syncthreads();
        if (tid < (int)(sizeof(af8_factored_tensor) / 4))
            reinterpret_cast<uint32_t *>(&sT)[tid] = __ldg(reinterpret_cast<const uint32_t *>(L.tensors + t) + tid);
        s_col[tid] = 0.0;
        __syncthreads();
        const int64_t C = sT.cols;
        const int64_t ntc = (C + FSTAT_COLS - 1) / FSTAT_COLS;
        const int64_t mr = fact_mat_rows(sT);                              // a tile lies inside one matrix of a batch
        const int64_t tpm = ((mr + FSTAT_ROWS - 1) / FSTAT_ROWS) * ntc;
        const int64_t local = id - sT.first_tile;
        const int64_t mat = local / tpm, lt = local - mat * tpm;
        const int64_t r0 = mat * mr + (lt / ntc) * FSTAT_ROWS;
        const int64_t R = (mat + 1) * mr;                                  // end of the matrix's rows
        const int64_t c0 = (lt % ntc) * FSTAT_COLS;
        const int64_t cb = sT.batch_rows > 0 ? mat * C : 0;               // the matrix's part of the column arrays
        float pre_div = 1.0f;
        if (L.mode == AF8_FSTAT_RESIDUAL) pre_div = L.dyn[t].pre_div;

        double cacc[FSTAT_COLS / 32];
        float icv[FSTAT_COLS / 32];
#pragma unroll
        for (int k = 0; k < FSTAT_COLS / 32; ++k) {
            cacc[k] = 0.0;
            const int64_t c = c0 + lane + 32 * k;
            icv[k] = (L.mode == AF8_FSTAT_RESIDUAL && c < C) ? sT.inv_col[cb + c] : 0.0f;
        }
        for (int rr = warp; rr < FSTAT_ROWS; rr += 8) {
            const int64_t r = r0 + rr;
            if (r >= R) break;
            const float ir = (L.mode == AF8_FSTAT_RESIDUAL) ? sT.inv_row[r] : 0.0f;
            double racc = 0.0;
#pragma unroll
            for (int k = 0; k < FSTAT_COLS / 32; ++k) {
                const int64_t c = c0 + lane + 32 * k;
                if (c < C) {
                    const int64_t flat = r * C + c;
                    float g = load_grad_any(sT.grad, L.grad_dtype, flat);
                    if (L.negate_grad) g = -g;
                    float x;
                    if (L.mode == AF8_FSTAT_GRADSQ) {
                        x = __fmul_rn(g, g);                                         // optimizer.py:2221
                    } else {
                        const float u = u_clipped(g, ir, icv[k], pre_div);           // optimizer.py:929
                        const float m = lerp_t(m_old_at(sT, L.m_fmt, L.m_block, flat), u, sT.m_w);   // optimizer.py:930
                        const float df = __fsub_rn(u, m);
                        x = __fadd_rn(__fmul_rn(df, df), sT.eps_came);               // optimizer.py:932
                    }
                    const double xd = (double)x;
                    racc += xd;
                    cacc[k] += xd;
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) racc += __shfl_xor_sync(0xffffffffu, racc, o);
            if (lane == 0) atomicAdd(sT.row_sum + r, racc);
        }
#pragma unroll
        for (int k = 0; k < FSTAT_COLS / 32; ++k) atomicAdd(&s_col[lane + 32 * k], cacc[k]);
        __syncthreads();
        if (c0 + tid < C) atomicAdd(sT.col_sum + cb + c0 + tid, s_col[tid]);
    }
}

// ---------------------------------------------------------------------------
// small states
// ---------------------------------------------------------------------------
// EMA + requantisation of block b of one small state of n elements (optimizer.py:2232-2238,
// 937-946, 2248-2251).  `out` receives the un-requantised values.  Returns this thread's partial
// sum of the block's values (binary64) for the mean of the row state.
__device__ double small_state_block(const af8_small_state &S, const double *sums, double count, int64_t n, int64_t b,
                                    float eps_add, float w, float floor_log, float *out, float *s_l, float (*s_red)[8])
{
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int block = S.block;
    double acc = 0.0;
    if (S.fmt == AF8_V_FP32) {
        const int64_t end = min(n, (b + 1) * (int64_t)block);
        for (int64_t i = b * block + tid; i < end; i += blockDim.x) {
            const float nv = __fadd_rn(__double2float_rn(sums[i] / count), eps_add);
            const float v = lerp_t(S.f32[i], nv, w);
            S.f32[i] = v;
            out[i] = v;
            acc += (double)v;
        }
        return acc;
    }
    const int bits = S.fmt;
    const float qm1 = bits == 16 ? 65534.0f : 254.0f;
    const int qmax = bits == 16 ? 65535 : 255;
    const float sc = S.scale[b], ml = S.min_log[b];
    float mn = INFINITY, mx = -INFINITY;
    for (int i = tid; i < block; i += blockDim.x) {
        const int64_t e = b * block + i;
        float v = 0.0f;                                       // padding re-enters as zeros (optimizer.py:303-305)
        if (e < n) {
            const uint32_t code = bits == 16 ? static_cast<const uint16_t *>(S.q)[e] : static_cast<const uint8_t *>(S.q)[e];
            const float nv = __fadd_rn(__double2float_rn(sums[e] / count), eps_add);
            v = lerp_t(al_decode(code, sc, ml, qm1), nv, w);
            out[e] = v;
            acc += (double)v;
        }
        const float l = al_log2(v);
        if (v != 0.0f) mn = fminf(mn, l);
        mx = fmaxf(mx, l);
        s_l[i] = (v != 0.0f) ? l : -INFINITY;
    }
    mn = warp_min(mn);
    mx = warp_max(mx);
    if (lane == 0) { s_red[0][warp] = mn; s_red[1][warp] = mx; }
    __syncthreads();
    for (int w8 = 0; w8 < 8; ++w8) { mn = fminf(mn, s_red[0][w8]); mx = fmaxf(mx, s_red[1][w8]); }
    float min_log, scale;
    al_range(mn, mx, floor_log, min_log, scale);
    for (int i = tid; i < block; i += blockDim.x) {
        const float l = s_l[i];
        const uint32_t code = (l == -INFINITY) ? 0u : al_encode(1.0f, l, min_log, scale, qm1, qmax);
        const int64_t e = b * block + i;
        if (bits == 16) static_cast<uint16_t *>(S.q)[e] = (uint16_t)code;
        else static_cast<uint8_t *>(S.q)[e] = (uint8_t)code;
    }
    if (tid == 0) { S.scale[b] = scale; S.min_log[b] = min_log; }
    return acc;
}

__device__ __forceinline__ int find_factored_small(const af8_factored_tensor *t, int n, int id)
{
    int lo = 0, hi = n - 1;
    while (lo < hi) {
        int mid = (lo + hi + 1) >> 1;
        if (__ldg(&t[mid].first_small) <= id) lo = mid; else hi = mid - 1;
    }
    return lo;
}

// One CTA per quantisation block of a row or column state: every block of every tensor in
// parallel (a 32000-row state has 125 blocks of 256; one CTA per tensor walked them in turn).
__global__ void __launch_bounds__(256)
factored_small_kernel(const af8_factored_tensor *tensors, int n_tensors, int conf, float floor_log)
{
    extern __shared__ float s_l[];
    __shared__ float s_red[2][8];
    __shared__ double s_acc[8];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int t = find_factored_small(tensors, n_tensors, (int)blockIdx.x);
    const af8_factored_tensor T = tensors[t];
    const int block = (conf ? T.conf_row : T.row_var).block;
    const int64_t nbr = (T.rows + block - 1) / block;
    const int64_t local = (int64_t)blockIdx.x - T.first_small;
    const bool is_row = local < nbr;
    const int64_t b = is_row ? local : local - nbr;
    const float w = conf ? T.c_w : T.v_w;
    const float eps_add = conf ? 0.0f : T.eps1;                 // optimizer.py:2222-2223 vs 933-934
    double part;
    // a batch of matrices: the states are flat over the batch (their blocks run across the matrices); a
    // column value is the mean over the rows of its own matrix
    if (is_row)
        part = small_state_block(conf ? T.conf_row : T.row_var, T.row_sum, (double)T.cols, T.rows, b, eps_add, w, floor_log,
                                 conf ? T.inv_row_conf : T.inv_row, s_l, s_red);
    else
        part = small_state_block(conf ? T.conf_col : T.col_var, T.col_sum, (double)fact_mat_rows(T), fact_batch(T) * T.cols, b, eps_add, w, floor_log,
                                 conf ? T.inv_col_conf : T.inv_col, s_l, s_red);
    if (!is_row) return;
    // the block's share of the mean of the row state goes where its first row sum was
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    if (lane == 0) s_acc[warp] = part;
    __syncthreads();                                            // (also: every thread has read its row sums)
    if (tid == 0) {
        double s = 0.0;
        for (int k = 0; k < 8; ++k) s += s_acc[k];
        T.row_sum[b * block] = s;
    }
}

// grid (n_tensors, slices): mean of the row state, clamped (optimizer.py:2236, 948), then the
// inverse-std vectors (optimizer.py:818-821); the CTAs of a tensor share its elements
__global__ void __launch_bounds__(256)
factored_inv_kernel(const af8_factored_tensor *tensors, int conf)
{
    __shared__ float s_rm;
    const af8_factored_tensor T = tensors[blockIdx.x];
    const int tid = threadIdx.x;
    float *inv_r = conf ? T.inv_row_conf : T.inv_row;
    float *inv_c = conf ? T.inv_col_conf : T.inv_col;
    const int block = (conf ? T.conf_row : T.row_var).block;
    const int64_t stride = (int64_t)blockDim.x * gridDim.y;
    const int64_t first = (int64_t)blockIdx.y * blockDim.x + tid;
    if (T.batch_rows > 0) {
        // a batch: the mean of each matrix's own row values (row_var.mean(dim=-2)), matrices dealt out to the
        // slices; the values are read before any of them is overwritten by this CTA's own threads
        __shared__ double s_red[8];
        const int64_t mr = T.batch_rows, nb = T.rows / mr;
        for (int64_t m = blockIdx.y; m < nb; m += gridDim.y) {
            double part = 0.0;
            for (int64_t i = tid; i < mr; i += blockDim.x) part += (double)inv_r[m * mr + i];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
            __syncthreads();
            if ((tid & 31) == 0) s_red[tid >> 5] = part;
            __syncthreads();
            double s = 0.0;
            for (int k = 0; k < 8; ++k) s += s_red[k];
            float rm = __double2float_rn(s / (double)mr);
            if (rm < T.eps1) rm = T.eps1;
            for (int64_t i = tid; i < mr; i += blockDim.x) inv_r[m * mr + i] = rsqrt_t(__fdiv_rn(inv_r[m * mr + i], rm));
        }
        for (int64_t j = first; j < nb * T.cols; j += stride) inv_c[j] = rsqrt_t(inv_c[j]);
        return;
    }
    if (tid == 0) {
        double s = 0.0;
        for (int64_t e = 0; e < T.rows; e += block) s += T.row_sum[e];      // fixed order
        float rm = __double2float_rn(s / (double)T.rows);
        if (rm < T.eps1) rm = T.eps1;
        s_rm = rm;
    }
    __syncthreads();
    const float rm = s_rm;
    for (int64_t i = first; i < T.rows; i += stride) inv_r[i] = rsqrt_t(__fdiv_rn(inv_r[i], rm));
    for (int64_t j = first; j < T.cols; j += stride) inv_c[j] = rsqrt_t(inv_c[j]);
}

// ---------------------------------------------------------------------------
// update
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(FUPD_THREADS)
factored_update_kernel(const FactoredLaunch L, int chunk)
{
    extern __shared__ float s_m[];                 // new momentum of the chunk (quantised formats)
    __shared__ af8_factored_tensor sT;
    __shared__ double s_acc[FUPD_THREADS / 32];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool has_m = L.m_fmt != AF8_M_NONE;
    const bool m_quant = has_m && L.m_fmt != AF8_M_FP32;
    const bool writes = L.mode == AF8_FUPD_APPLY || L.mode == AF8_FUPD_LAG;
    const bool sums = !writes || L.mode == AF8_FUPD_LAG;

    for (int64_t id = blockIdx.x; id < L.total_units; id += gridDim.x) {
        const int t = find_factored_chunk(L.tensors, L.n_tensors, id);
        __syncthreads();
        if (tid < (int)(sizeof(af8_factored_tensor) / 4))
            reinterpret_cast<uint32_t *>(&sT)[tid] = __ldg(reinterpret_cast<const uint32_t *>(L.tensors + t) + tid);
        __syncthreads();
        const int64_t C = sT.cols, numel = sT.rows * sT.cols;
        const int64_t base = (id - sT.first_chunk) * chunk;
        const int valid = (int)min((int64_t)chunk, numel - base);
        float pre_div = 1.0f, step_mul = -sT.alpha, fira = 1.0f;
        bool zero_upd = false;
        if (L.dyn != nullptr) {
            const af8_dyn_scalars ds = L.dyn[t];
            if (L.came) pre_div = ds.pre_div;
            if (writes) { step_mul = ds.step; fira = ds.fira; zero_upd = ds.zero != 0.0f; }
        }
        if (L.mode == AF8_FUPD_SUMSQ_U) pre_div = 1.0f;           // the clip divisor is what this pass measures

        int64_t row = (base + tid) / C;
        int64_t col = (base + tid) - row * C;
        double acc = 0.0;
        for (int i = tid; i < chunk; i += FUPD_THREADS) {
            float mj = 0.0f;
            if (i < valid) {
                const int64_t flat = base + i;
                float g = load_grad_any(sT.grad, L.grad_dtype, flat);
                if (L.negate_grad) g = -g;
                const int64_t cb = fact_col_base(sT, row);                         // (a batch of matrices: that matrix's columns)
                const float ir = sT.inv_row[row], ic = sT.inv_col[cb + col];
                float u;
                if (L.came) {
                    const float uc = u_clipped(g, ir, ic, pre_div);                  // optimizer.py:929
                    if (L.mode == AF8_FUPD_SUMSQ_U) {
                        u = uc;
                    } else {
                        mj = lerp_t(m_old_at(sT, L.m_fmt, L.m_block, flat), uc, sT.m_w);   // optimizer.py:930
                        u = __fmul_rn(__fmul_rn(mj, sT.inv_row_conf[row]), sT.inv_col_conf[cb + col]);   // optimizer.py:952
                    }
                } else if (has_m) {
                    mj = lerp_t(m_old_at(sT, L.m_fmt, L.m_block, flat), g, sT.m_w);        // optimizer.py:959
                    u = __fmul_rn(__fmul_rn(mj, ir), ic);                                  // optimizer.py:961
                } else {
                    u = __fmul_rn(__fmul_rn(g, ir), ic);                                   // optimizer.py:968-969
                }
                if (sums) acc += (double)__fmul_rn(u, u);
                if (writes) {
                    if (!m_quant && has_m) sT.m_f32[flat] = mj;
                    // optimizer.py:2039, 803, 874 (a zero update still applies the decay and the rounding)
                    const float uu = zero_upd ? 0.0f : __fmul_rn(u, fira);
                    const float pv = param_load(sT.param, flat, L.param_dtype);
                    const uint32_t pbits = param_step_bits(pv, sT.decay, step_mul, uu, L.param_dtype, L.sr, sT.sr_base, flat);
                    param_store_bits(sT.param, flat, pbits, L.param_dtype);
                    if (sT.param_copy != nullptr && L.param_dtype == AF8_F32)       // bf16 compute copy
                        static_cast<uint16_t *>(sT.param_copy)[flat] = (uint16_t)f32_to_bf16_rn_bits(__uint_as_float(pbits));
                }
            }
            if (writes && m_quant) s_m[i] = mj;
            col += FUPD_THREADS;
            while (col >= C) { col -= C; ++row; }
        }
        if (sums) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (lane == 0) s_acc[warp] = acc;
            __syncthreads();
            if (tid == 0) {
                double s = 0.0;
                for (int w = 0; w < FUPD_THREADS / 32; ++w) s += s_acc[w];
                L.block_sumsq[id] = s;
            }
            if (!writes) continue;
        }
        if (m_quant) {
            __syncthreads();
            const bool four_bit = (L.m_fmt == AF8_M_UF4 || L.m_fmt == AF8_M_D4);
            const int subs = chunk / L.m_block;
            for (int sb = warp; sb < subs; sb += FUPD_THREADS / 32) {
                const int s0 = sb * L.m_block;
                if (s0 >= valid) break;
                float am = 0.0f;
                for (int i = lane; i < L.m_block; i += 32) am = fmaxf(am, fabsf(s_m[s0 + i]));
                am = fmaxf(warp_max(am), 1e-12f);
                if (four_bit) {
                    for (int i = lane * 2; i < L.m_block; i += 64)
                        sT.m_q[(base + s0 + i) >> 1] = (uint8_t)((m_encode(s_m[s0 + i], am, L.m_fmt) << 4) | m_encode(s_m[s0 + i + 1], am, L.m_fmt));
                } else {
                    for (int i = lane; i < L.m_block; i += 32)
                        sT.m_q[base + s0 + i] = (uint8_t)m_encode(s_m[s0 + i], am, L.m_fmt);
                }
                if (lane == 0) sT.m_scale[(base + s0) / L.m_block] = am;
            }
        }
    }
}

// ---------------------------------------------------------------------------
// vectorised variants: every tensor has cols % 8 == 0 and 16-byte aligned arrays, the
// momentum block (if quantised) is 256.  A thread owns 8 consecutive elements of one row:
// 128-bit loads of the gradient, the parameter and the column vectors; a warp owns one
// momentum block, so its absmax is a warp reduction.  Same arithmetic as the kernels above.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void prefetch_l2(const void *p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }
#ifndef AF8_FUPD_PREFETCH_AHEAD
#define AF8_FUPD_PREFETCH_AHEAD 3      /* chunks ahead that the momentum-free write pass requests from L2; 0: off */
#endif
template <typename GradT> __host__ __device__ constexpr int sizeof_grad() { return std::is_same<GradT, float>::value ? 4 : 2; }

template <typename GradT>
__device__ __forceinline__ void load_g8(const void *grad, int64_t off, int negate, float (&g)[8])
{
    stat_load_g<GradT>(grad, off, g);
    if (negate) {
#pragma unroll
        for (int j = 0; j < 8; ++j) g[j] = -g[j];
    }
}

// 8 consecutive gradient elements as loaded, so that the load of the next chunk can be
// issued before the current one is processed
template <typename GradT> struct GradRaw8;
template <> struct GradRaw8<float> {
    float4 a, b;
    __device__ __forceinline__ void zero() { a = b = make_float4(0.f, 0.f, 0.f, 0.f); }
    __device__ __forceinline__ void load(const void *grad, int64_t off)
    {
        const float4 *p = reinterpret_cast<const float4 *>(static_cast<const float *>(grad) + off);
        a = __ldcs(p); b = __ldcs(p + 1);
    }
    __device__ __forceinline__ void from_shared(const unsigned char *p)
    {
        a = *reinterpret_cast<const float4 *>(p); b = *reinterpret_cast<const float4 *>(p + 16);
    }
    __device__ __forceinline__ void unpack(int negate, float (&g)[8]) const
    {
        g[0] = a.x; g[1] = a.y; g[2] = a.z; g[3] = a.w; g[4] = b.x; g[5] = b.y; g[6] = b.z; g[7] = b.w;
        if (negate) {
#pragma unroll
            for (int j = 0; j < 8; ++j) g[j] = -g[j];
        }
    }
};
template <> struct GradRaw8<bf16_tag> {
    uint4 a;
    __device__ __forceinline__ void zero() { a = make_uint4(0u, 0u, 0u, 0u); }
    __device__ __forceinline__ void load(const void *grad, int64_t off)
    {
        a = __ldcs(reinterpret_cast<const uint4 *>(static_cast<const uint16_t *>(grad) + off));
    }
    __device__ __forceinline__ void from_shared(const unsigned char *p) { a = *reinterpret_cast<const uint4 *>(p); }
    __device__ __forceinline__ void unpack(int negate, float (&g)[8]) const
    {
        const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            g[2 * k] = __uint_as_float(w[k] << 16);
            g[2 * k + 1] = __uint_as_float(w[k] & 0xffff0000u);
        }
        if (negate) {
#pragma unroll
            for (int j = 0; j < 8; ++j) g[j] = -g[j];
        }
    }
};

__device__ __forceinline__ void load_f8(const float *p, float (&x)[8])
{
    const float4 a = *reinterpret_cast<const float4 *>(p), b = *reinterpret_cast<const float4 *>(p + 4);
    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
}

__device__ __forceinline__ void load_f8_ro(const float *p, float (&x)[8])     // read-only data, kept in L1
{
    const float4 a = __ldg(reinterpret_cast<const float4 *>(p)), b = __ldg(reinterpret_cast<const float4 *>(p + 4));
    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
}

// old momentum of 8 consecutive elements (one momentum block)
// `pre`: the 8 UF8 codes if the caller has loaded them already (have_pre)
__device__ __forceinline__ void m_old8(const af8_factored_tensor &T, int m_fmt, int m_block, int64_t flat, float (&m)[8],
                                       bool have_pre = false, uint2 pre = make_uint2(0u, 0u))
{
    if (m_fmt == AF8_M_FP32) { load_f8(T.m_f32 + flat, m); return; }
    const float sc = __ldg(T.m_scale + flat / m_block);
    if (m_fmt == AF8_M_UF8) {
        const uint2 w = have_pre ? pre : *reinterpret_cast<const uint2 *>(T.m_q + flat);
        const float mc = __fmul_rn(sc, 0.0078125f);      // fl(scale / 128): a power-of-two divisor, scale >= 1e-12
#pragma unroll
        for (int j = 0; j < 8; ++j) m[j] = __fmul_rn(byte_minus_128(j < 4 ? w.x : w.y, j & 3), mc);   // no integer conversion
    } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) m[j] = m_decode(T.m_q, sc, flat + j, m_fmt);
    }
}

// Rows r0 + warp + 8k of the tile, NB at a time so that NB independent 128-bit loads per lane
// are in flight.  Column partials go to a per-warp shared array (no shared-memory atomics).
template <typename GradT, int NB, bool PREFETCH, bool RESIDUAL>
__device__ __forceinline__ void stats_rows(const FactoredLaunch &L, const af8_factored_tensor &sT, int64_t r0, int64_t row_end, int64_t c,
                                           bool col_ok, float pre_div, const float (&ic)[8], double (&cacc)[8])
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t R = row_end, C = sT.cols;          // row_end: end of the tile's matrix (the tensor's rows unless it is a batch)
    // PREFETCH: the loads of the next NB rows are issued before the current ones are processed
    GradRaw8<GradT> cur[NB], nxt[NB];
    auto fetch = [&](GradRaw8<GradT> (&dst)[NB], int k0) {
#pragma unroll
        for (int k = 0; k < NB; ++k) {
            const int64_t r = r0 + warp + 8 * (k0 + k);
            if (col_ok && r < R && k0 + k < FSTAT_ROWS / 8) dst[k].load(sT.grad, r * C + c);
            else dst[k].zero();
        }
    };
    if (PREFETCH) fetch(cur, 0);
    for (int k0 = 0; k0 < FSTAT_ROWS / 8; k0 += NB) {
        if (r0 + warp + 8 * k0 >= R) break;                       // uniform over the warp
        if (PREFETCH) fetch(nxt, k0 + NB);
        else fetch(cur, k0);
        float g[NB][8];
        double rsum[NB];
#pragma unroll
        for (int k = 0; k < NB; ++k) {
            cur[k].unpack(L.negate_grad, g[k]);
            if (PREFETCH) cur[k] = nxt[k];
        }
#pragma unroll
        for (int k = 0; k < NB; ++k) {
            const int64_t r = r0 + warp + 8 * (k0 + k);
            const bool live = col_ok && r < R;
            float x[8];
            if (!RESIDUAL) {
#pragma unroll
                for (int j = 0; j < 8; j += 2) {
                    const float2 gj = make_float2(g[k][j], g[k][j + 1]);
                    const float2 xx = __fmul2_rn(gj, gj);
                    x[j] = xx.x; x[j + 1] = xx.y;
                }
            } else if (live) {
                const int64_t flat = r * C + c;
                const float2 ir2 = bc2(sT.inv_row[r]);
                const DivBy D = make_div(pre_div);
                const LerpW LW = make_lerp(sT.m_w);
                const float2 eps2 = bc2(sT.eps_came);
                float mo[8];
                m_old8(sT, L.m_fmt, L.m_block, flat, mo);
#pragma unroll
                for (int j = 0; j < 8; j += 2) {       // pairs in packed binary32 arithmetic (bit-identical to element-wise)
                    const float2 u = div_by2(__fmul2_rn(__fmul2_rn(make_float2(g[k][j], g[k][j + 1]), ir2), make_float2(ic[j], ic[j + 1])), D);
                    const float2 m = lerp_w2(make_float2(mo[j], mo[j + 1]), u, LW);
                    const float2 df = sub2(u, m);
                    const float2 xx = __fadd2_rn(__fmul2_rn(df, df), eps2);
                    x[j] = xx.x; x[j + 1] = xx.y;
                }
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) x[j] = 0.0f;
            }
            double racc = 0.0;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const double xd = (double)x[j];
                racc += xd;
                cacc[j] += xd;
            }
            rsum[k] = racc;
        }
        // The NB row sums of the warp are reduced together: each exchange halves the number of
        // values a lane carries, so NB rows cost NB - 1 + (5 - log2 NB) shuffles instead of 5 NB.
        // The sum of row k0 + i ends up in lane 32 i / NB.
        static_assert(NB == 2 || NB == 4, "row-sum reduction is written for 2 or 4 rows");
        double v;
        if (NB == 4) {
            const bool hi = lane & 16;
            const double r0x = __shfl_xor_sync(0xffffffffu, hi ? rsum[0] : rsum[2], 16);
            const double r1x = __shfl_xor_sync(0xffffffffu, hi ? rsum[1] : rsum[NB - 1], 16);
            const double k0v = (hi ? rsum[2] : rsum[0]) + r0x;
            const double k1v = (hi ? rsum[NB - 1] : rsum[1]) + r1x;
            const bool h2 = lane & 8;
            v = (h2 ? k1v : k0v) + __shfl_xor_sync(0xffffffffu, h2 ? k0v : k1v, 8);
#pragma unroll
            for (int o = 4; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if ((lane & 7) == 0) {
                const int64_t r = r0 + warp + 8 * (k0 + (lane >> 3));
                if (r < R && k0 + (lane >> 3) < FSTAT_ROWS / 8) atomicAdd(sT.row_sum + r, v);
            }
        } else {
            const bool hi = lane & 16;
            v = (hi ? rsum[1] : rsum[0]) + __shfl_xor_sync(0xffffffffu, hi ? rsum[0] : rsum[1], 16);
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if ((lane & 15) == 0) {
                const int64_t r = r0 + warp + 8 * (k0 + (lane >> 4));
                if (r < R && k0 + (lane >> 4) < FSTAT_ROWS / 8) atomicAdd(sT.row_sum + r, v);
            }
        }
    }
}

// The same rows with the inputs of every row slice (256 columns: 512 or 1024 bytes of gradient and,
// for the residual, 256 momentum codes) requested SR_STAGES slices ahead by the warp's lane 0 with
// cp.async.bulk into the warp's own ring (one mbarrier per stage).  Needs cols % 256 == 0 (whole
// slices, 16-byte aligned runs) and, for the residual, a UF8 momentum.  NB rows are consumed per
// iteration so that their row sums are reduced jointly, as above.  Returns false after a time-out.
template <typename GradT> __host__ __device__ constexpr int sring_stages() { return sizeof_grad<GradT>() == 2 ? 8 : 4; }
template <typename GradT, bool RESIDUAL> __host__ __device__ constexpr int sring_stage_bytes() { return 256 * sizeof_grad<GradT>() + (RESIDUAL ? 256 : 0); }
template <typename GradT, bool RESIDUAL> __host__ __device__ constexpr size_t sring_smem_bytes() { return (size_t)8 * sring_stages<GradT>() * sring_stage_bytes<GradT, RESIDUAL>(); }

// 8 UF8 codes of one momentum block as floats: (code - 128) * mc, two elements per instruction; each
// component rounds like the scalar form in m_old8
__device__ __forceinline__ void uf8_decode8(uint2 w, float mc, float2 (&m)[4])
{
    const float2 off = bc2(-8388736.0f), mc2 = bc2(mc);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t word = j < 2 ? w.x : w.y;
        const float2 b = make_float2(__uint_as_float(__byte_perm(word, 0x4b000000u, 0x7540u | (uint32_t)((2 * j) & 3))),
                                     __uint_as_float(__byte_perm(word, 0x4b000000u, 0x7540u | (uint32_t)((2 * j + 1) & 3))));
        m[j] = __fmul2_rn(__fadd2_rn(b, off), mc2);
    }
}

// CAME's residual (U - M)^2 + eps of 8 elements, M the momentum after this step's EMA.
// ONE: the clip divisor is 1; SMALL: |momentum weight| < 0.5 (the form of lerp).  The quotient is taken
// without div_by's test for an infinite product.  The caller guarantees a divisor d >= 1 (or NaN), as the
// RMS clip produces: then a finite t = g * r * c has a finite product t * fl(1 / d), and an infinite or NaN t
// ends as x = NaN with the true quotient as well (U and M are both infinite, U - M is NaN).
template <bool ONE, bool SMALL>
__device__ __forceinline__ void residual_x8(const float (&g)[8], uint2 codes, float mc, float ir, const float (&ic)[8],
                                            const DivBy &D, float ww, float eps, float (&x)[8])
{
    const float2 ir2 = bc2(ir), r2 = bc2(D.rcp), nd2 = bc2(D.nd), ww2 = bc2(ww), eps2 = bc2(eps);
    float2 mo[4];
    uf8_decode8(codes, mc, mo);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 t = __fmul2_rn(__fmul2_rn(make_float2(g[2 * j], g[2 * j + 1]), ir2), make_float2(ic[2 * j], ic[2 * j + 1]));
        float2 u = t;
        if (!ONE) {
            const float2 q = __fmul2_rn(t, r2);
            u = __ffma2_rn(__ffma2_rn(q, nd2, t), r2, q);
        }
        const float2 m = __ffma2_rn(ww2, sub2(u, mo[j]), SMALL ? mo[j] : u);
        const float2 df = sub2(u, m);
        const float2 xx = __fadd2_rn(__fmul2_rn(df, df), eps2);
        x[2 * j] = xx.x; x[2 * j + 1] = xx.y;
    }
}

// The residual pass over the rows r0 + warp + 8 k of a tile whose 256-column row slices (gradient and UF8 codes,
// momentum block 256: a slice is one block) come through the warp's ring.  NB rows are consumed per iteration
// so that their row sums are reduced jointly.  The per-row scalars (inverse row factor, block absmax) of the
// next iteration are loaded while the current one computes; the sign of a negated gradient rides on the row
// factor ((-g) * r == g * (-r) bit for bit).  Returns false after a time-out.
template <typename GradT, int NB, bool ONE, bool SMALL>
__device__ __forceinline__ bool residual_rows_ring(const FactoredLaunch &L, const af8_factored_tensor &sT, int64_t r0, int64_t c0,
                                                   float pre_div, const float (&ic)[8], double (&cacc)[8],
                                                   unsigned char *ring, uint64_t *full, uint32_t &cons)
{
    constexpr int GB = sizeof_grad<GradT>(), NS = sring_stages<GradT>(), STAGE = sring_stage_bytes<GradT, true>();
    static_assert(NS % NB == 0 && (NS & (NS - 1)) == 0, "a ring holds whole groups of rows");
    static_assert(NB == 2 || NB == 4, "row-sum reduction is written for 2 or 4 rows");
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t C = sT.cols;
    const int64_t r_end = min(sT.rows, r0 + (int64_t)FSTAT_ROWS);
    const int64_t row0 = r0 + warp;
    const int nrows = row0 < r_end ? (int)((r_end - row0 + 7) / 8) : 0;          // rows row0 + 8 k of this warp
    // lanes 0 and 1 request the next slice: lane 0 its gradients (and the bytes to expect), lane 1 its codes,
    // both with the same instructions (a copy may complete before the bytes are announced: the phase also
    // needs lane 0's arrival)
    const int64_t estep = 8 * C;
    int64_t eoff = row0 * C + c0;                                // element offset of the next slice
    const unsigned char *src = lane == 0 ? static_cast<const unsigned char *>(sT.grad) : sT.m_q;
    const int esz = lane == 0 ? GB : 1;
    uint32_t prod = cons;                                        // (cons counts the slices consumed before this tile)
    auto issue = [&]() {                                         // lanes 0 and 1
        const int sl = (int)(prod & (uint32_t)(NS - 1));
        ++prod;
        unsigned char *dst = ring + sl * STAGE;
        if (lane == 0) mbar_expect_tx(&full[sl], (uint32_t)STAGE);
        bulk_g2s(dst + lane * (256 * GB), src + eoff * esz, 256 * esz, &full[sl]);
        eoff += estep;
    };
    if (lane < 2 && nrows > 0) {
        fence_proxy_async();
        for (int k = 0; k < min(NS, nrows); ++k) issue();
    }
    const DivBy D = make_div(pre_div);
    const LerpW LW = make_lerp(sT.m_w);
    const float eps = sT.eps_came, sgn = L.negate_grad ? -1.0f : 1.0f;
    // row row0 + 8 k: inverse row factor at index row0 + 8 k, block absmax at sc0 + k * scstep (both fit 32 bits:
    // a tensor has fewer than 2^31 rows and momentum blocks)
    const int scstep = (int)(8 * (C >> 8));
    const int sc0 = (int)(row0 * (C >> 8) + (c0 >> 8));
    float nir[NB], nsc[NB];                                      // the scalars of the next NB rows, signed and scaled
#pragma unroll
    for (int k = 0; k < NB; ++k) {
        nir[k] = 0.0f; nsc[k] = 0.0f;
        if (k < nrows) { nir[k] = __ldg(sT.inv_row + (int)row0 + 8 * k); nsc[k] = __ldg(sT.m_scale + sc0 + k * scstep); }
    }
    for (int k0 = 0; k0 < nrows; k0 += NB) {
        GradRaw8<GradT> cur[NB];
        uint2 cm[NB];
        bool landed = true;
#pragma unroll
        for (int k = 0; k < NB; ++k) {
            cm[k] = make_uint2(0u, 0u);
            if (k0 + k < nrows) {
                const uint32_t n = cons + (uint32_t)(k0 + k);
                const int sl = (int)(n & (uint32_t)(NS - 1));
                landed = landed && mbar_wait_bounded(&full[sl], (n / NS) & 1u);
                const unsigned char *st = ring + sl * STAGE;
                cur[k].from_shared(st + lane * (8 * GB));
                cm[k] = *reinterpret_cast<const uint2 *>(st + 256 * GB + lane * 8);
            } else cur[k].zero();
        }
        if (!__all_sync(0xffffffffu, landed)) return false;
        __syncwarp();                                            // the stages were read: they may be refilled
        if (lane < 2) {
            fence_proxy_async();
#pragma unroll
            for (int k = 0; k < NB; ++k)
                if (k0 + k + NS < nrows) issue();
        }
        double rsum[NB];
#pragma unroll
        for (int k = 0; k < NB; ++k) {
            double racc = 0.0;
            if (k0 + k < nrows) {
                float g[8], x[8];
                cur[k].unpack(0, g);
                // fl(scale / 128): a power-of-two divisor, scale >= 1e-12
                residual_x8<ONE, SMALL>(g, cm[k], __fmul_rn(nsc[k], 0.0078125f), __fmul_rn(nir[k], sgn), ic, D, LW.ww, eps, x);
                if (k0 + NB + k < nrows) {                       // this row's successor in the next iteration
                    nir[k] = __ldg(sT.inv_row + (int)row0 + 8 * (k0 + NB + k));
                    nsc[k] = __ldg(sT.m_scale + sc0 + (k0 + NB + k) * scstep);
                }
                double pr[4];                                   // (pairwise: a short dependency chain)
#pragma unroll
                for (int j = 0; j < 8; j += 2) {
                    const double xa = (double)x[j], xb = (double)x[j + 1];
                    cacc[j] += xa;
                    cacc[j + 1] += xb;
                    pr[j >> 1] = xa + xb;
                }
                racc = (pr[0] + pr[1]) + (pr[2] + pr[3]);
            }
            rsum[k] = racc;
        }
        double v;
        if (NB == 4) {
            const bool hi = lane & 16;
            const double r0x = __shfl_xor_sync(0xffffffffu, hi ? rsum[0] : rsum[2], 16);
            const double r1x = __shfl_xor_sync(0xffffffffu, hi ? rsum[1] : rsum[NB - 1], 16);
            const double k0v = (hi ? rsum[2] : rsum[0]) + r0x;
            const double k1v = (hi ? rsum[NB - 1] : rsum[1]) + r1x;
            const bool h2 = lane & 8;
            v = (h2 ? k1v : k0v) + __shfl_xor_sync(0xffffffffu, h2 ? k0v : k1v, 8);
#pragma unroll
            for (int o = 4; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if ((lane & 7) == 0 && k0 + (lane >> 3) < nrows) atomicAdd(sT.row_sum + row0 + 8 * (int64_t)(k0 + (lane >> 3)), v);
        } else {
            const bool hi = lane & 16;
            v = (hi ? rsum[1] : rsum[0]) + __shfl_xor_sync(0xffffffffu, hi ? rsum[0] : rsum[1], 16);
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if ((lane & 15) == 0 && k0 + (lane >> 4) < nrows) atomicAdd(sT.row_sum + row0 + 8 * (int64_t)(k0 + (lane >> 4)), v);
        }
    }
    cons += (uint32_t)nrows;
    return true;
}

// The same pass with the input of FBOX_ROWS consecutive rows per copy: one tiled bulk tensor copy brings their
// 256-column slices of the gradient (tensor map maps[0]: bf16 [rows][cols], box 256 x FBOX_ROWS), one their UF8 codes
// (maps[1]: bytes, same box) into a stage of the warp's two-stage ring, so that the instructions of a request -
// about 57 issue slots with one lane active - are spent once per FBOX_ROWS rows instead of once per row.  Warp w
// takes the row groups r0 + FBOX_ROWS (w + 8 k); rows past the end of the tensor arrive as zeros and are skipped.
// bf16 gradients only (a stage is 3 KB; the two stages fill the ring's 6 KB per warp).
constexpr int FBOX_ROWS = 4, FBOX_STAGES = 2;
constexpr int FBOX_G_BYTES = FBOX_ROWS * 512, FBOX_STAGE_BYTES = FBOX_G_BYTES + FBOX_ROWS * 256;
static_assert(FBOX_STAGES * FBOX_STAGE_BYTES <= sring_stages<bf16_tag>() * sring_stage_bytes<bf16_tag, true>(), "the boxes use the ring's memory");
static_assert(FSTAT_ROWS % (8 * FBOX_ROWS) == 0, "whole row groups per warp and tile");

template <bool ONE, bool SMALL>
__device__ __forceinline__ bool residual_rows_box(const FactoredLaunch &L, const af8_factored_tensor &sT, const CUtensorMap *maps,
                                                  int64_t r0, int64_t c0, float pre_div, const float (&ic)[8], double (&cacc)[8],
                                                  unsigned char *ring, uint64_t *full, uint32_t &cons)
{
    constexpr int BR = FBOX_ROWS, NS = FBOX_STAGES;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t C = sT.cols;
    const int r_end = (int)min(sT.rows, r0 + (int64_t)FSTAT_ROWS);
    const int row0 = (int)r0 + BR * warp;                        // first row of this warp's group 0; group g: + 8 * BR * g
    const int ngroups = row0 < r_end ? (r_end - row0 + 8 * BR - 1) / (8 * BR) : 0;
    auto issue = [&](int g) {                                    // lane 0: group g into its stage
        const int sl = (int)((cons + (uint32_t)g) & (uint32_t)(NS - 1));
        unsigned char *dst = ring + sl * FBOX_STAGE_BYTES;
        mbar_expect_tx(&full[sl], (uint32_t)FBOX_STAGE_BYTES);
        tma_load_2d(dst, maps, (int)c0, row0 + 8 * BR * g, &full[sl]);
        tma_load_2d(dst + FBOX_G_BYTES, maps + 1, (int)c0, row0 + 8 * BR * g, &full[sl]);
    };
    if (lane == 0 && ngroups > 0) {
        fence_proxy_async();
        for (int g = 0; g < min(NS, ngroups); ++g) issue(g);
    }
    const DivBy D = make_div(pre_div);
    const LerpW LW = make_lerp(sT.m_w);
    const float eps = sT.eps_came, sgn = L.negate_grad ? -1.0f : 1.0f;
    // row r: inverse row factor at index r, block absmax at r * (C / 256) + c0 / 256 (both fit 32 bits)
    const int scrow = (int)(C >> 8), scoff = (int)(c0 >> 8);
    float nir[2], nsc[2];                                        // the scalars of the next pair of rows
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        nir[k] = 0.0f; nsc[k] = 0.0f;
        if (row0 + k < r_end) { nir[k] = __ldg(sT.inv_row + row0 + k); nsc[k] = __ldg(sT.m_scale + (row0 + k) * scrow + scoff); }
    }
    for (int g = 0; g < ngroups; ++g) {
        const uint32_t n = cons + (uint32_t)g;
        const int sl = (int)(n & (uint32_t)(NS - 1));
        const bool landed = mbar_wait_bounded(&full[sl], (n / NS) & 1u);
        if (!__all_sync(0xffffffffu, landed)) return false;
        const unsigned char *st = ring + sl * FBOX_STAGE_BYTES;
        const int grow = row0 + 8 * BR * g;                      // first row of the group
#pragma unroll
        for (int h = 0; h < BR / 2; ++h) {                       // pairs of rows: their row sums are reduced jointly
            GradRaw8<bf16_tag> cur[2];
            uint2 cm[2];
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                cur[k].from_shared(st + (2 * h + k) * 512 + lane * 16);
                cm[k] = *reinterpret_cast<const uint2 *>(st + FBOX_G_BYTES + (2 * h + k) * 256 + lane * 8);
            }
            if (h == BR / 2 - 1) {                               // the stage was read: it may be refilled
                __syncwarp();
                if (lane == 0 && g + NS < ngroups) { fence_proxy_async(); issue(g + NS); }
            }
            double rsum[2];
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                const int r = grow + 2 * h + k;
                double racc = 0.0;
                const float ir = __fmul_rn(nir[k], sgn), mc = __fmul_rn(nsc[k], 0.0078125f);   // fl(scale / 128), scale >= 1e-12
                {   // this row's successor: the same place of the next pair
                    const int rn = (h == BR / 2 - 1) ? r + 8 * BR - (BR - 2) : r + 2;
                    if (rn < r_end) { nir[k] = __ldg(sT.inv_row + rn); nsc[k] = __ldg(sT.m_scale + rn * scrow + scoff); }
                }
                if (r < r_end) {
                    float gg[8], x[8];
                    cur[k].unpack(0, gg);
                    residual_x8<ONE, SMALL>(gg, cm[k], mc, ir, ic, D, LW.ww, eps, x);
                    double pr[4];                               // (pairwise: a short dependency chain)
#pragma unroll
                    for (int j = 0; j < 8; j += 2) {
                        const double xa = (double)x[j], xb = (double)x[j + 1];
                        cacc[j] += xa;
                        cacc[j + 1] += xb;
                        pr[j >> 1] = xa + xb;
                    }
                    racc = (pr[0] + pr[1]) + (pr[2] + pr[3]);
                }
                rsum[k] = racc;
            }
            const bool hi = lane & 16;
            double v = (hi ? rsum[1] : rsum[0]) + __shfl_xor_sync(0xffffffffu, hi ? rsum[0] : rsum[1], 16);
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            const int rr = grow + 2 * h + (lane >> 4);
            if ((lane & 15) == 0 && rr < r_end) atomicAdd(sT.row_sum + rr, v);
        }
    }
    cons += (uint32_t)ngroups;
    return true;
}

// RESIDUAL: CAME's (U - M)^2 + eps statistic; otherwise g^2 (separate instantiations, so that
// the lighter one keeps its lower register count)
// resident CTAs asked of the compiler (measured on B200: 3 for both passes; the g*g pass went
// from 1.02 to 0.76 ms on the TinyLlama set with it)
#ifndef AF8_FSTAT_MIN_CTAS
#define AF8_FSTAT_MIN_CTAS 3
#endif
#ifndef AF8_FSTAT_RES_NB
#define AF8_FSTAT_RES_NB 2
#endif
#ifndef AF8_FSTAT_RES_PREFETCH
#define AF8_FSTAT_RES_PREFETCH true
#endif
#ifndef AF8_FSTAT_MIN_CTAS_RES
#define AF8_FSTAT_MIN_CTAS_RES 3
#endif
template <typename GradT, bool RESIDUAL>
__global__ void __launch_bounds__(256, RESIDUAL ? AF8_FSTAT_MIN_CTAS_RES : AF8_FSTAT_MIN_CTAS)
factored_stats_vec_kernel(const FactoredLaunch L, const int use_ring, const CUtensorMap *__restrict__ maps)
{
    __shared__ double s_col[8][FSTAT_COLS];      // [warp][j * 32 + lane]
    __shared__ af8_factored_tensor sT;
    extern __shared__ __align__(128) unsigned char sr_smem[];            // the warps' input rings (use_ring)
    __shared__ __align__(8) uint64_t s_full[8][sring_stages<GradT>()];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    int cur_t = -1;
    uint32_t cons = 0;                           // row slices this warp has taken from its ring
    if (use_ring) {
        if (lane == 0) {
            for (int k = 0; k < sring_stages<GradT>(); ++k) mbar_init(&s_full[warp][k], 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        __syncthreads();
    }

    for (int64_t id = blockIdx.x; id < L.total_units; id += gridDim.x) {
        int t = cur_t;
        if (t < 0) t = find_factored_tile(L.tensors, L.n_tensors, id);
        else while (t + 1 < L.n_tensors && __ldg(&L.tensors[t + 1].first_tile) <= id) ++t;
        __syncthreads();                                           // s_col of the previous tile was read
        if (t != cur_t) {
            if (tid < (int)(sizeof(af8_factored_tensor) / 4))
                reinterpret_cast<uint32_t *>(&sT)[tid] = __ldg(reinterpret_cast<const uint32_t *>(L.tensors + t) + tid);
            cur_t = t;
            __syncthreads();
        }
        const int64_t C = sT.cols;
        const int64_t ntc = (C + FSTAT_COLS - 1) / FSTAT_COLS;
        const int64_t local = id - sT.first_tile;                  // (batches of matrices take the general kernel)
        const int64_t r0 = (local / ntc) * FSTAT_ROWS;
        const int64_t row_end = sT.rows;
        const int64_t c0 = (local % ntc) * FSTAT_COLS;
        const int64_t c = c0 + lane * 8;                           // this lane's 8 columns
        const bool col_ok = c < C;                                 // C % 8 == 0: all 8 or none
        float pre_div = 1.0f;
        float ic[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) ic[j] = 0.0f;
        if (RESIDUAL) {
            pre_div = L.dyn[t].pre_div;
            if (col_ok) load_f8_ro(sT.inv_col + c, ic);
        }
        double cacc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) cacc[j] = 0.0;
        // residual: whole 256-column slices of the gradient and the UF8 codes come through the warp's ring
        // (measured on Llama-2-7B: 11.9 -> 11.4 ms; the g*g pass and the sum passes, which only read the
        // gradient, were slower through a ring - 3.0 -> 4.3 ms and 4.6 -> 5.9 ms - and load directly)
        // (the ring's quotient wants a clip divisor >= 1 or NaN, which is what the RMS clip produces)
        bool done = false;
        if constexpr (RESIDUAL) {
            if (use_ring && (C % FSTAT_COLS) == 0 && L.m_fmt == AF8_M_UF8 && L.m_block == 256 && !(pre_div < 1.0f)) {
                done = true;
                unsigned char *ring = sr_smem + (size_t)warp * sring_stages<GradT>() * sring_stage_bytes<GradT, true>();
                constexpr int NB = AF8_FSTAT_RES_NB;
                const bool one = pre_div == 1.0f, small = fabsf(sT.m_w) < 0.5f;  // (uniform over the tensor)
                bool ok = true, boxes = false;
                if constexpr (std::is_same<GradT, bf16_tag>::value) {
                if (use_ring == 2) {                                             // boxes of rows through tensor maps
                    boxes = true;
                    const CUtensorMap *mp = maps + 2 * t;
                    if (one) ok = small ? residual_rows_box<true, true>(L, sT, mp, r0, c0, pre_div, ic, cacc, ring, s_full[warp], cons)
                                        : residual_rows_box<true, false>(L, sT, mp, r0, c0, pre_div, ic, cacc, ring, s_full[warp], cons);
                    else ok = small ? residual_rows_box<false, true>(L, sT, mp, r0, c0, pre_div, ic, cacc, ring, s_full[warp], cons)
                                    : residual_rows_box<false, false>(L, sT, mp, r0, c0, pre_div, ic, cacc, ring, s_full[warp], cons);
                }
                }
                if (boxes) { }
                else if (one) ok = small ? residual_rows_ring<GradT, NB, true, true>(L, sT, r0, c0, pre_div, ic, cacc, ring, s_full[warp], cons)
                                    : residual_rows_ring<GradT, NB, true, false>(L, sT, r0, c0, pre_div, ic, cacc, ring, s_full[warp], cons);
                else ok = small ? residual_rows_ring<GradT, NB, false, true>(L, sT, r0, c0, pre_div, ic, cacc, ring, s_full[warp], cons)
                                : residual_rows_ring<GradT, NB, false, false>(L, sT, r0, c0, pre_div, ic, cacc, ring, s_full[warp], cons);
                if (!ok) {
                    atomicExch(&g_device_error, DEVERR_SRING_TIMEOUT);
                    return;                      // (the whole warp; the others finish their rows and leave at the next barrier)
                }
            }
        }
        if (!RESIDUAL) stats_rows<GradT, 4, true, false>(L, sT, r0, row_end, c, col_ok, pre_div, ic, cacc);
        else if (!done) stats_rows<GradT, AF8_FSTAT_RES_NB, AF8_FSTAT_RES_PREFETCH, true>(L, sT, r0, row_end, c, col_ok, pre_div, ic, cacc);
#pragma unroll
        for (int j = 0; j < 8; ++j) s_col[warp][j * 32 + lane] = cacc[j];
        __syncthreads();
        // thread tid owns column c0 + tid = c0 + 8 * (tid >> 3) + (tid & 7)
        if (c0 + tid < C) {
            double sum = 0.0;
#pragma unroll
            for (int w = 0; w < 8; ++w) sum += s_col[w][(tid & 7) * 32 + (tid >> 3)];
            atomicAdd(sT.col_sum + c0 + tid, sum);
        }
    }
}

// chunk = 2048 elements = 8 warps x 256; requires m_block == 256 when the momentum is quantised
// PASS 0: a sum-of-squares pass (fewer values live, more resident CTAs); 1: the APPLY pass;
// 2: the LAG pass (APPLY plus the sums of this step's raw update)
// CTAS: resident CTAs per SM asked of the compiler.  Measured on B200: 4 for the sum passes; for the
// writing passes 3 with momentum (CAME, 0.78 ms per Llama-2-7B layer) and 2 without (Adafactor on the
// TinyLlama set: 2.51 -> 2.21 ms, no register spills).
template <typename GradT, int PASS, int CTAS>
__global__ void __launch_bounds__(FUPD_THREADS, CTAS)
factored_update_vec_kernel(const FactoredLaunch L)
{
    constexpr bool WRITES = PASS != 0;
    constexpr bool SUMS = PASS != 1;
    __shared__ af8_factored_tensor sT;
    __shared__ double s_acc2[1][FUPD_THREADS / 32];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool has_m = L.m_fmt != AF8_M_NONE;
    const bool m_quant = has_m && L.m_fmt != AF8_M_FP32;
    constexpr bool writes = WRITES;
    int cur_t = -1;
    GradRaw8<GradT> ng;
    float4 np0 = make_float4(0.f, 0.f, 0.f, 0.f), np1 = np0;
    uint2 nm = make_uint2(0u, 0u);
    bool have = false;
    ng.zero();

    // Every CTA takes a contiguous run of chunks, so a thread's position (flat index, row,
    // column) and the tensor's scalars advance incrementally: the division by the column
    // count and the table lookups happen once per tensor, not once per chunk.
    const int64_t per_cta = (L.total_units + gridDim.x - 1) / gridDim.x;
    const int64_t id_begin = (int64_t)blockIdx.x * per_cta;
    const int64_t id_end = min(id_begin + per_cta, L.total_units);
    int64_t next_first = 0, flat = 0, row = 0, col = 0;
    float pre_div = 1.0f, step_mul = 0.0f, fira = 1.0f;
    bool zero_upd = false;
    DivBy D = make_div(1.0f);

    // Sum-of-squares passes: a thread keeps one binary64 partial over all the chunks of a tensor
    // that its CTA processes; at the end of that run the CTA reduces it once and stores the total in
    // the slot of the run's first chunk and zero in the others (the finaliser adds a tensor's slots).
    double run_acc = 0.0;
    int64_t run_first = -1;
    auto flush_sums = [&](int64_t end) {
        double acc = run_acc;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (lane == 0) s_acc2[0][warp] = acc;
        __syncthreads();
        if (tid == 0) {
            double sum = 0.0;
            for (int w = 0; w < FUPD_THREADS / 32; ++w) sum += s_acc2[0][w];
            L.block_sumsq[run_first] = sum;
        }
        for (int64_t i = run_first + 1 + tid; i < end; i += FUPD_THREADS) L.block_sumsq[i] = 0.0;
        __syncthreads();
        run_acc = 0.0;
    };

    for (int64_t id = id_begin; id < id_end; ++id) {
        const int t = cur_t;
        if (cur_t < 0 || id >= next_first) {
            if (SUMS && run_first >= 0) flush_sums(id);
            run_first = id;
            int tn = cur_t;
            if (tn < 0) tn = find_factored_chunk(L.tensors, L.n_tensors, id);
            else while (tn + 1 < L.n_tensors && __ldg(&L.tensors[tn + 1].first_chunk) <= id) ++tn;
            __syncthreads();
            if (tid < (int)(sizeof(af8_factored_tensor) / 4))
                reinterpret_cast<uint32_t *>(&sT)[tid] = __ldg(reinterpret_cast<const uint32_t *>(L.tensors + tn) + tid);
            cur_t = tn;
            __syncthreads();
            next_first = tn + 1 < L.n_tensors ? __ldg(&L.tensors[tn + 1].first_chunk) : L.total_units;
            flat = (id - sT.first_chunk) * 2048 + tid * 8;
            row = flat / sT.cols;
            col = flat - row * sT.cols;
            have = false;
            pre_div = 1.0f; step_mul = -sT.alpha; fira = 1.0f; zero_upd = false;
            if (L.dyn != nullptr) {
                const af8_dyn_scalars ds = L.dyn[tn];
                if (L.came && L.mode != AF8_FUPD_SUMSQ_U) pre_div = ds.pre_div;
                if (writes) { step_mul = ds.step; fira = ds.fira; zero_upd = ds.zero != 0.0f; }
            }
            D = make_div(pre_div);
        } else {
            flat += 2048;
            col += 2048;
            if (sT.cols >= 2048) {
                if (col >= sT.cols) { col -= sT.cols; ++row; }
            } else {
                const uint32_t q = (uint32_t)col / (uint32_t)sT.cols;
                row += q;
                col -= (int64_t)q * sT.cols;
            }
        }
        (void)t;
        const int64_t numel = sT.rows * sT.cols;
        const bool ok = flat < numel;                                // numel % 8 == 0: all 8 or none
        // this chunk's streams, loaded one iteration ahead when the chunk is in the same tensor
        GradRaw8<GradT> cg;
        float4 cp0 = make_float4(0.f, 0.f, 0.f, 0.f), cp1 = cp0;
        uint2 cm = make_uint2(0u, 0u);
        const bool pre_m = has_m && L.m_fmt == AF8_M_UF8 && L.mode != AF8_FUPD_SUMSQ_U;
        float *const pbase = static_cast<float *>(sT.param);
        const bool lowp = L.param_dtype != AF8_F32;                  // 16-bit parameters: 8 of them in cp0
        const uint16_t *const hbase = static_cast<const uint16_t *>(sT.param);
        if (have) { cg = ng; cp0 = np0; cp1 = np1; cm = nm; }
        else if (ok) {
            cg.load(sT.grad, flat);
            if (writes) {
                if (lowp) cp0 = *reinterpret_cast<const float4 *>(hbase + flat);
                else { cp0 = *reinterpret_cast<const float4 *>(pbase + flat); cp1 = *reinterpret_cast<const float4 *>(pbase + flat + 4); }
            }
            if (pre_m) cm = *reinterpret_cast<const uint2 *>(sT.m_q + flat);
        } else cg.zero();
#if AF8_FUPD_PREFETCH_AHEAD > 0
        if (writes && !has_m) {
            // The momentum-free write pass asks L2 for the chunk a few iterations ahead (same tensor), one
            // request per 128-byte line: measured on the TinyLlama set 2.33 -> 1.89 ms (5.8 TB/s).  The
            // passes with momentum and the sum passes were measured slower with it (CAME apply 24.9 ->
            // 25.6 ms, sums 0.87 -> 0.94 ms), so they go without.
            const int64_t pf = flat + (int64_t)AF8_FUPD_PREFETCH_AHEAD * 2048;
            if (id + AF8_FUPD_PREFETCH_AHEAD < id_end && pf < numel) {
                constexpr int GB = sizeof_grad<GradT>();
                if ((tid & (GB == 2 ? 7 : 3)) == 0) prefetch_l2(static_cast<const char *>(sT.grad) + pf * GB);
                if (writes && (tid & (lowp ? 7 : 3)) == 0) prefetch_l2(static_cast<const char *>(sT.param) + pf * (lowp ? 2 : 4));
                if (pre_m && (tid & 15) == 0) prefetch_l2(sT.m_q + pf);
            }
        }
#endif
        {
            const int64_t nf = flat + 2048;                          // the next chunk of this CTA, if it is in this tensor
            have = id + 1 < id_end && nf < numel;
            if (have) {
                ng.load(sT.grad, nf);
                if (writes) {
                    if (lowp) np0 = *reinterpret_cast<const float4 *>(hbase + nf);
                    else { np0 = *reinterpret_cast<const float4 *>(pbase + nf); np1 = *reinterpret_cast<const float4 *>(pbase + nf + 4); }
                }
                if (pre_m) nm = *reinterpret_cast<const uint2 *>(sT.m_q + nf);
            }
        }
        float mj[8];
        double part = 0.0;
        if (ok) {
            float g[8], ic[8], u[8];
            const LerpW LW = make_lerp(sT.m_w);
            cg.unpack(L.negate_grad, g);
            load_f8_ro(sT.inv_col + col, ic);
            const float ir = __ldg(sT.inv_row + row);
            // pairs of elements in packed binary32 arithmetic (bit-identical to the element-wise form)
            const float2 ir2 = bc2(ir);
            if (L.came) {
                if (L.mode == AF8_FUPD_SUMSQ_U) {
#pragma unroll
                    for (int j = 0; j < 8; j += 2) {
                        const float2 uj = __fmul2_rn(__fmul2_rn(make_float2(g[j], g[j + 1]), ir2), make_float2(ic[j], ic[j + 1]));
                        u[j] = uj.x; u[j + 1] = uj.y;
                    }
                } else {
                    float mo[8], icc[8];
                    m_old8(sT, L.m_fmt, L.m_block, flat, mo, pre_m, cm);
                    load_f8_ro(sT.inv_col_conf + col, icc);
                    const float2 irc2 = bc2(__ldg(sT.inv_row_conf + row));
#pragma unroll
                    for (int j = 0; j < 8; j += 2) {
                        const float2 ut = div_by2(__fmul2_rn(__fmul2_rn(make_float2(g[j], g[j + 1]), ir2), make_float2(ic[j], ic[j + 1])), D);
                        const float2 mm = lerp_w2(make_float2(mo[j], mo[j + 1]), ut, LW);
                        const float2 uj = __fmul2_rn(__fmul2_rn(mm, irc2), make_float2(icc[j], icc[j + 1]));
                        mj[j] = mm.x; mj[j + 1] = mm.y; u[j] = uj.x; u[j + 1] = uj.y;
                    }
                }
            } else if (has_m) {
                float mo[8];
                m_old8(sT, L.m_fmt, L.m_block, flat, mo, pre_m, cm);
#pragma unroll
                for (int j = 0; j < 8; j += 2) {
                    const float2 mm = lerp_w2(make_float2(mo[j], mo[j + 1]), make_float2(g[j], g[j + 1]), LW);
                    const float2 uj = __fmul2_rn(__fmul2_rn(mm, ir2), make_float2(ic[j], ic[j + 1]));
                    mj[j] = mm.x; mj[j + 1] = mm.y; u[j] = uj.x; u[j + 1] = uj.y;
                }
            } else {
#pragma unroll
                for (int j = 0; j < 8; j += 2) {
                    const float2 uj = __fmul2_rn(__fmul2_rn(make_float2(g[j], g[j + 1]), ir2), make_float2(ic[j], ic[j + 1]));
                    u[j] = uj.x; u[j + 1] = uj.y;
                }
            }
            if (SUMS) {
                // The thread's eight squares are added in binary32 (two packed chains) and enter the binary64
                // partial as one number: the sum only feeds a norm (clip divisor, limiter), where a relative
                // 1e-7 is far below what the parameters can show, and it saves seven conversions and seven
                // binary64 additions per chunk.
                float2 a2 = __fmul2_rn(make_float2(u[0], u[1]), make_float2(u[0], u[1]));
#pragma unroll
                for (int j = 2; j < 8; j += 2) a2 = __ffma2_rn(make_float2(u[j], u[j + 1]), make_float2(u[j], u[j + 1]), a2);
                part += (double)__fadd_rn(a2.x, a2.y);
            }
            if (writes) {
                if (lowp) {
                    // bf16 / fp16 parameters: rounded after the decay and after the update, or once,
                    // stochastically (optimizer.py:873-881, 2033-2039)
                    const uint32_t w[4] = {__float_as_uint(cp0.x), __float_as_uint(cp0.y), __float_as_uint(cp0.z), __float_as_uint(cp0.w)};
                    uint32_t o[4];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const uint32_t h = (j & 1) ? (w[j >> 1] >> 16) : (w[j >> 1] & 0xffffu);
                        const float pv = L.param_dtype == AF8_BF16 ? bf16_bits_to_f32(h) : f16_bits_to_f32(h);
                        const float uu = zero_upd ? 0.0f : __fmul_rn(u[j], fira);
                        const uint32_t r = param_step_bits(pv, sT.decay, step_mul, uu, L.param_dtype, L.sr, sT.sr_base, flat + j);
                        if (j & 1) o[j >> 1] |= r << 16; else o[j >> 1] = r;
                    }
                    *reinterpret_cast<uint4 *>(const_cast<uint16_t *>(hbase) + flat) = make_uint4(o[0], o[1], o[2], o[3]);
                } else {
                    float *pp = pbase + flat;
                    float p[8] = {cp0.x, cp0.y, cp0.z, cp0.w, cp1.x, cp1.y, cp1.z, cp1.w};
                    const float2 decay2 = bc2(sT.decay), step2 = bc2(step_mul), fira2 = bc2(fira);
#pragma unroll
                    for (int j = 0; j < 8; j += 2) {
                        float2 pj = __fmul2_rn(make_float2(p[j], p[j + 1]), decay2);
                        if (!zero_upd) pj = __ffma2_rn(step2, __fmul2_rn(make_float2(u[j], u[j + 1]), fira2), pj);
                        p[j] = pj.x; p[j + 1] = pj.y;
                    }
                    *reinterpret_cast<float4 *>(pp) = make_float4(p[0], p[1], p[2], p[3]);
                    *reinterpret_cast<float4 *>(pp + 4) = make_float4(p[4], p[5], p[6], p[7]);
                    if (sT.param_copy != nullptr)                                    // bf16 compute copy
                        *reinterpret_cast<uint4 *>(static_cast<uint16_t *>(sT.param_copy) + flat) =
                            make_uint4(bf16x2_rn(p[0], p[1]), bf16x2_rn(p[2], p[3]), bf16x2_rn(p[4], p[5]), bf16x2_rn(p[6], p[7]));
                }
                if (has_m && !m_quant) {
                    *reinterpret_cast<float4 *>(sT.m_f32 + flat) = make_float4(mj[0], mj[1], mj[2], mj[3]);
                    *reinterpret_cast<float4 *>(sT.m_f32 + flat + 4) = make_float4(mj[4], mj[5], mj[6], mj[7]);
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) mj[j] = 0.0f;
        }
        if (SUMS) {
            run_acc += part;                 // reduced over the CTA once per tensor (flush_sums)
            if (!writes) continue;
        }
        if (m_quant) {
            // one warp = one momentum block of 256 (the block exists iff its first element does)
            const int64_t w0 = (id - sT.first_chunk) * 2048 + warp * 256;
            float am = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j) am = fmaxf(am, fabsf(mj[j]));
            am = fmaxf(warp_max(am), 1e-12f);
            if (w0 < numel) {
                if (L.m_fmt == AF8_M_UF8) {
                    const DivBy A = make_div(am);
                    const uint32_t o0 = uf8_encode_fast2(make_float2(mj[0], mj[1]), A) | (uf8_encode_fast2(make_float2(mj[2], mj[3]), A) << 16);
                    const uint32_t o1 = uf8_encode_fast2(make_float2(mj[4], mj[5]), A) | (uf8_encode_fast2(make_float2(mj[6], mj[7]), A) << 16);
                    if (ok) *reinterpret_cast<uint2 *>(sT.m_q + flat) = make_uint2(o0, o1);
                } else if (L.m_fmt == AF8_M_D8) {
                    uint32_t o0 = 0, o1 = 0;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        o0 |= m_encode(mj[j], am, L.m_fmt) << (8 * j);
                        o1 |= m_encode(mj[j + 4], am, L.m_fmt) << (8 * j);
                    }
                    if (ok) *reinterpret_cast<uint2 *>(sT.m_q + flat) = make_uint2(o0, o1);
                } else {
                    uint32_t o = 0;
#pragma unroll
                    for (int j = 0; j < 8; j += 2)
                        o |= ((m_encode(mj[j], am, L.m_fmt) << 4) | m_encode(mj[j + 1], am, L.m_fmt)) << (4 * j);
                    if (ok) *reinterpret_cast<uint32_t *>(sT.m_q + (flat >> 1)) = o;
                }
                if (lane == 0) sT.m_scale[w0 / 256] = am;
            }
        }
    }
    if (SUMS && run_first >= 0) flush_sums(id_end);
}

// ---------------------------------------------------------------------------
// The APPLY pass for fp32 parameters with a UF8 momentum (CAME, Adafactor with beta1), inputs
// through per-warp rings of bulk asynchronous copies.
//
// The register-pipelined kernel above has one chunk in flight per thread and was measured
// latency-bound in this configuration (CAME apply: half of the copy peak, long-scoreboard
// stalls on top).  Here a warp still owns one momentum block per chunk (256 consecutive
// elements: gradient, parameter and momentum codes are three contiguous runs of 512 or 1024,
// 1024 and 256 bytes), but its lane 0 requests them FRING_STAGES - 1 chunks ahead with
// cp.async.bulk into the warp's own ring; completion is an mbarrier per stage.  Warps do not
// synchronise with one another except when the CTA moves to its next tensor.  Copies never
// cross a tensor, and the (at most one) partial chunk at a tensor's end is loaded directly.
// Same arithmetic, element for element, as factored_update_vec_kernel.
// ---------------------------------------------------------------------------
#ifndef AF8_FRING_STAGES
#define AF8_FRING_STAGES 4
#endif
constexpr int FRING_STAGES = AF8_FRING_STAGES;
constexpr int DEVERR_FRING_TIMEOUT = 3;
template <typename GradT> __host__ __device__ constexpr int fring_stage_bytes() { return 256 * sizeof_grad<GradT>() + 1024 + 256; }
template <typename GradT> constexpr size_t fring_smem_bytes() { return (size_t)(FUPD_THREADS / 32) * FRING_STAGES * fring_stage_bytes<GradT>(); }

template <typename GradT, int CTAS>
__global__ void __launch_bounds__(FUPD_THREADS, CTAS)
factored_apply_ring_kernel(const FactoredLaunch L)
{
    constexpr int GB = sizeof_grad<GradT>();
    constexpr int P_OFF = 256 * GB, M_OFF = P_OFF + 1024, STAGE = fring_stage_bytes<GradT>(), NS = FRING_STAGES;
    extern __shared__ __align__(128) unsigned char fr_smem[];
    __shared__ af8_factored_tensor sT;
    __shared__ __align__(8) uint64_t s_full[FUPD_THREADS / 32][NS];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    unsigned char *const ring = fr_smem + (size_t)warp * NS * STAGE;
    if (lane == 0) {
        for (int k = 0; k < NS; ++k) mbar_init(&s_full[warp][k], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    const int64_t per_cta = (L.total_units + gridDim.x - 1) / gridDim.x;
    const int64_t id_begin = (int64_t)blockIdx.x * per_cta;
    const int64_t id_end = min(id_begin + per_cta, L.total_units);
    int cur_t = -1;
    int64_t next_first = 0, full_end = 0, flat = 0, row = 0, col = 0;
    float pre_div = 1.0f, step_mul = 0.0f, fira = 1.0f;
    bool zero_upd = false;
    DivBy D = make_div(1.0f);
    uint32_t cons = 0;            // chunks this warp has taken from its ring
    int inflight = 0;             // chunks from the current one on whose copies are issued

    for (int64_t id = id_begin; id < id_end; ++id) {
        if (cur_t < 0 || id >= next_first) {
            int tn = cur_t;
            if (tn < 0) tn = find_factored_chunk(L.tensors, L.n_tensors, id);
            else while (tn + 1 < L.n_tensors && __ldg(&L.tensors[tn + 1].first_chunk) <= id) ++tn;
            __syncthreads();
            if (tid < (int)(sizeof(af8_factored_tensor) / 4))
                reinterpret_cast<uint32_t *>(&sT)[tid] = __ldg(reinterpret_cast<const uint32_t *>(L.tensors + tn) + tid);
            cur_t = tn;
            __syncthreads();
            next_first = tn + 1 < L.n_tensors ? __ldg(&L.tensors[tn + 1].first_chunk) : L.total_units;
            full_end = min(id_end, sT.first_chunk + (sT.rows * sT.cols) / 2048);     // chunk ids below it are whole chunks of this tensor
            flat = (id - sT.first_chunk) * 2048 + tid * 8;
            row = flat / sT.cols;
            col = flat - row * sT.cols;
            pre_div = 1.0f; step_mul = -sT.alpha; fira = 1.0f; zero_upd = false;
            if (L.dyn != nullptr) {
                const af8_dyn_scalars ds = L.dyn[tn];
                if (L.came) pre_div = ds.pre_div;
                step_mul = ds.step; fira = ds.fira; zero_upd = ds.zero != 0.0f;
            }
            D = make_div(pre_div);
            inflight = 0;                                            // (copies never cross a tensor)
        } else {
            flat += 2048;
            col += 2048;
            if (sT.cols >= 2048) {
                if (col >= sT.cols) { col -= sT.cols; ++row; }
            } else {
                const uint32_t q = (uint32_t)col / (uint32_t)sT.cols;
                row += q;
                col -= (int64_t)q * sT.cols;
            }
        }
        const int64_t numel = sT.rows * sT.cols;
        const bool full = id < full_end;
        const bool ok = flat < numel;
        float *const pbase = static_cast<float *>(sT.param);

        // ---- request the chunks id .. id + NS - 1 that are whole chunks of this tensor ----
        int want = (int)min((int64_t)NS, full_end - id);
        if (want < 0) want = 0;
        if (lane == 0 && inflight < want) {
            fence_proxy_async();                                     // this warp's reads of the slots came first
            const unsigned char *gp = static_cast<const unsigned char *>(sT.grad);
            const unsigned char *pp = static_cast<const unsigned char *>(sT.param);
            for (int k = inflight; k < want; ++k) {
                const int64_t off = (id + k - sT.first_chunk) * 2048 + warp * 256;      // first element of the warp's run
                const int sl = (int)((cons + (uint32_t)k) % NS);
                unsigned char *dst = ring + sl * STAGE;
                mbar_expect_tx(&s_full[warp][sl], (uint32_t)STAGE);
                bulk_g2s(dst + P_OFF, pp + off * 4, 1024, &s_full[warp][sl]);
                bulk_g2s(dst, gp + off * GB, 256 * GB, &s_full[warp][sl]);
                bulk_g2s(dst + M_OFF, sT.m_q + off, 256, &s_full[warp][sl]);
            }
        }
        inflight = want > 0 ? want - 1 : 0;                          // as seen from the next chunk

        GradRaw8<GradT> cg;
        float4 cp0 = make_float4(0.f, 0.f, 0.f, 0.f), cp1 = cp0;
        uint2 cm = make_uint2(0u, 0u);
        if (full) {
            const int sl = (int)(cons % NS);
            const bool landed = mbar_wait_bounded(&s_full[warp][sl], (cons / NS) & 1u);
            if (!__all_sync(0xffffffffu, landed)) {                  // (uniform over the warp)
                atomicExch(&g_device_error, DEVERR_FRING_TIMEOUT);
                return;                                              // the other warps go on: nothing waits for this one
            }
            const unsigned char *st = ring + sl * STAGE;
            cg.from_shared(st + lane * (8 * GB));
            cp0 = *reinterpret_cast<const float4 *>(st + P_OFF + lane * 32);
            cp1 = *reinterpret_cast<const float4 *>(st + P_OFF + lane * 32 + 16);
            cm = *reinterpret_cast<const uint2 *>(st + M_OFF + lane * 8);
            ++cons;
            __syncwarp();                                            // the slot may be refilled from the next iteration on
        } else if (ok) {
            cg.load(sT.grad, flat);
            cp0 = *reinterpret_cast<const float4 *>(pbase + flat);
            cp1 = *reinterpret_cast<const float4 *>(pbase + flat + 4);
            cm = *reinterpret_cast<const uint2 *>(sT.m_q + flat);
        } else cg.zero();

        float mj[8];
        if (ok) {
            float g[8], ic[8], u[8], mo[8];
            const LerpW LW = make_lerp(sT.m_w);
            cg.unpack(L.negate_grad, g);
            load_f8_ro(sT.inv_col + col, ic);
            const float2 ir2 = bc2(__ldg(sT.inv_row + row));
            m_old8(sT, AF8_M_UF8, 256, flat, mo, true, cm);
            if (L.came) {
                float icc[8];
                load_f8_ro(sT.inv_col_conf + col, icc);
                const float2 irc2 = bc2(__ldg(sT.inv_row_conf + row));
#pragma unroll
                for (int j = 0; j < 8; j += 2) {
                    const float2 ut = div_by2(__fmul2_rn(__fmul2_rn(make_float2(g[j], g[j + 1]), ir2), make_float2(ic[j], ic[j + 1])), D);
                    const float2 mm = lerp_w2(make_float2(mo[j], mo[j + 1]), ut, LW);
                    const float2 uj = __fmul2_rn(__fmul2_rn(mm, irc2), make_float2(icc[j], icc[j + 1]));
                    mj[j] = mm.x; mj[j + 1] = mm.y; u[j] = uj.x; u[j + 1] = uj.y;
                }
            } else {
#pragma unroll
                for (int j = 0; j < 8; j += 2) {
                    const float2 mm = lerp_w2(make_float2(mo[j], mo[j + 1]), make_float2(g[j], g[j + 1]), LW);
                    const float2 uj = __fmul2_rn(__fmul2_rn(mm, ir2), make_float2(ic[j], ic[j + 1]));
                    mj[j] = mm.x; mj[j + 1] = mm.y; u[j] = uj.x; u[j + 1] = uj.y;
                }
            }
            float *pp = pbase + flat;
            float p[8] = {cp0.x, cp0.y, cp0.z, cp0.w, cp1.x, cp1.y, cp1.z, cp1.w};
            const float2 decay2 = bc2(sT.decay), step2 = bc2(step_mul), fira2 = bc2(fira);
#pragma unroll
            for (int j = 0; j < 8; j += 2) {
                float2 pj = __fmul2_rn(make_float2(p[j], p[j + 1]), decay2);
                if (!zero_upd) pj = __ffma2_rn(step2, __fmul2_rn(make_float2(u[j], u[j + 1]), fira2), pj);
                p[j] = pj.x; p[j + 1] = pj.y;
            }
            *reinterpret_cast<float4 *>(pp) = make_float4(p[0], p[1], p[2], p[3]);
            *reinterpret_cast<float4 *>(pp + 4) = make_float4(p[4], p[5], p[6], p[7]);
            if (sT.param_copy != nullptr)                                    // bf16 compute copy
                *reinterpret_cast<uint4 *>(static_cast<uint16_t *>(sT.param_copy) + flat) =
                    make_uint4(bf16x2_rn(p[0], p[1]), bf16x2_rn(p[2], p[3]), bf16x2_rn(p[4], p[5]), bf16x2_rn(p[6], p[7]));
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) mj[j] = 0.0f;
        }
        // one warp = one momentum block of 256 (the block exists iff its first element does)
        const int64_t w0 = (id - sT.first_chunk) * 2048 + warp * 256;
        float am = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) am = fmaxf(am, fabsf(mj[j]));
        am = fmaxf(warp_max(am), 1e-12f);
        if (w0 < numel) {
            const DivBy A = make_div(am);
            const uint32_t o0 = uf8_encode_fast2(make_float2(mj[0], mj[1]), A) | (uf8_encode_fast2(make_float2(mj[2], mj[3]), A) << 16);
            const uint32_t o1 = uf8_encode_fast2(make_float2(mj[4], mj[5]), A) | (uf8_encode_fast2(make_float2(mj[6], mj[7]), A) << 16);
            if (ok) *reinterpret_cast<uint2 *>(sT.m_q + flat) = make_uint2(o0, o1);
            if (lane == 0) sT.m_scale[w0 / 256] = am;
        }
    }
}

// ---------------------------------------------------------------------------
// factored_apply_ring_kernel in tile order, for tables whose tensors all have cols % 256 == 0: a CTA takes a
// 512 x 256 statistic tile, warp w its rows r0 + w, r0 + w + 8, ...; a row slice of 256 columns is 256
// consecutive elements that start on a multiple of 256, i.e. exactly one momentum block, so the warp still owns
// its block's absmax.  What changes is that a lane works on the same 8 columns for the whole tile and keeps
// their inverse column factors (and CAME's confidence factors) in registers instead of loading 32 or 64 bytes
// of them for every 8 elements.  Ring, arithmetic and stores as in factored_apply_ring_kernel; the copies of
// a warp run FRING_STAGES - 1 rows ahead inside a tile.
// ---------------------------------------------------------------------------
template <typename GradT, int CTAS>
__global__ void __launch_bounds__(FUPD_THREADS, CTAS)
factored_apply_tile_kernel(const FactoredLaunch L)
{
    constexpr int GB = sizeof_grad<GradT>();
    constexpr int P_OFF = 256 * GB, M_OFF = P_OFF + 1024, STAGE = fring_stage_bytes<GradT>(), NS = FRING_STAGES;
    extern __shared__ __align__(128) unsigned char fr_smem[];
    __shared__ af8_factored_tensor sT;
    __shared__ __align__(8) uint64_t s_full[FUPD_THREADS / 32][NS];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    unsigned char *const ring = fr_smem + (size_t)warp * NS * STAGE;
    if (lane == 0) {
        for (int k = 0; k < NS; ++k) mbar_init(&s_full[warp][k], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    int cur_t = -1;
    float pre_div = 1.0f, step_mul = 0.0f, fira = 1.0f;
    bool zero_upd = false;
    DivBy D = make_div(1.0f);
    uint32_t cons = 0;            // row slices this warp has taken from its ring

    for (int64_t id = blockIdx.x; id < L.total_units; id += gridDim.x) {
        int t = cur_t;
        if (t < 0) t = find_factored_tile(L.tensors, L.n_tensors, id);
        else while (t + 1 < L.n_tensors && __ldg(&L.tensors[t + 1].first_tile) <= id) ++t;
        if (t != cur_t) {
            __syncthreads();                                         // every warp has left the previous tensor
            if (tid < (int)(sizeof(af8_factored_tensor) / 4))
                reinterpret_cast<uint32_t *>(&sT)[tid] = __ldg(reinterpret_cast<const uint32_t *>(L.tensors + t) + tid);
            cur_t = t;
            __syncthreads();
            pre_div = 1.0f; step_mul = -sT.alpha; fira = 1.0f; zero_upd = false;
            if (L.dyn != nullptr) {
                const af8_dyn_scalars ds = L.dyn[t];
                if (L.came) pre_div = ds.pre_div;
                step_mul = ds.step; fira = ds.fira; zero_upd = ds.zero != 0.0f;
            }
            D = make_div(pre_div);
        }
        const int64_t R = sT.rows, C = sT.cols;
        const int64_t ntc = C / FSTAT_COLS;                          // (cols % 256 == 0)
        const int64_t local = id - sT.first_tile;
        const int64_t r0 = (local / ntc) * FSTAT_ROWS;
        const int64_t c0 = (local % ntc) * FSTAT_COLS;
        const int64_t c = c0 + lane * 8;                             // this lane's 8 columns
        const int64_t r_end = min(R, r0 + (int64_t)FSTAT_ROWS);
        const int nrows = r0 + warp < r_end ? (int)((r_end - (r0 + warp) + 7) / 8) : 0;
        float ic[8], icc[8];
        load_f8_ro(sT.inv_col + c, ic);
        if (L.came) load_f8_ro(sT.inv_col_conf + c, icc);
        float *const pbase = static_cast<float *>(sT.param);
        const unsigned char *gp = static_cast<const unsigned char *>(sT.grad);
        const LerpW LW = make_lerp(sT.m_w);
        const float2 decay2 = bc2(sT.decay), step2 = bc2(step_mul), fira2 = bc2(fira);

        auto issue = [&](int k) {                                    // lane 0: row slice k of this warp into its stage
            const int64_t off = (r0 + warp + 8 * (int64_t)k) * C + c0;
            const int sl = (int)((cons + (uint32_t)k) % NS);
            unsigned char *dst = ring + sl * STAGE;
            mbar_expect_tx(&s_full[warp][sl], (uint32_t)STAGE);
            bulk_g2s(dst + P_OFF, reinterpret_cast<const unsigned char *>(pbase) + off * 4, 1024, &s_full[warp][sl]);
            bulk_g2s(dst, gp + off * GB, 256 * GB, &s_full[warp][sl]);
            bulk_g2s(dst + M_OFF, sT.m_q + off, 256, &s_full[warp][sl]);
        };
        if (lane == 0 && nrows > 0) {
            fence_proxy_async();                                     // this warp's reads of the slots came first
            for (int k = 0; k < min(NS, nrows); ++k) issue(k);
        }
        // the per-row scalars (inverse row factors, block absmax) are loaded one row ahead; the sign of a
        // negated gradient rides on the row factor ((-g) * r == g * (-r) bit for bit; without CAME the
        // gradient itself enters the momentum and is negated when unpacked)
        const int64_t row0 = r0 + warp;
        const int64_t scstep = 8 * (C >> 8);
        float *const scp = sT.m_scale + row0 * (C >> 8) + (c0 >> 8);             // + scstep per row of this warp
        const float sgn = (L.came && L.negate_grad) ? -1.0f : 1.0f;
        float n_ir = 0.0f, n_irc = 0.0f, n_sc = 0.0f;
        if (nrows > 0) {
            n_ir = __ldg(sT.inv_row + row0); n_sc = __ldg(scp);
            if (L.came) n_irc = __ldg(sT.inv_row_conf + row0);
        }
        for (int k = 0; k < nrows; ++k) {
            const uint32_t n = cons + (uint32_t)k;
            const int sl = (int)(n % NS);
            const bool landed = mbar_wait_bounded(&s_full[warp][sl], (n / NS) & 1u);
            if (!__all_sync(0xffffffffu, landed)) {                  // (uniform over the warp)
                atomicExch(&g_device_error, DEVERR_FRING_TIMEOUT);
                return;
            }
            const unsigned char *st = ring + sl * STAGE;
            GradRaw8<GradT> cg;
            cg.from_shared(st + lane * (8 * GB));
            const float4 cp0 = *reinterpret_cast<const float4 *>(st + P_OFF + lane * 32);
            const float4 cp1 = *reinterpret_cast<const float4 *>(st + P_OFF + lane * 32 + 16);
            const uint2 cm = *reinterpret_cast<const uint2 *>(st + M_OFF + lane * 8);
            __syncwarp();                                            // the slot may be refilled
            if (lane == 0 && k + NS < nrows) { fence_proxy_async(); issue(k + NS); }

            const int64_t row = row0 + 8 * (int64_t)k;
            const int64_t flat = row * C + c;
            float g[8], u[8], mj[8];
            float2 mo[4];
            cg.unpack(L.came ? 0 : L.negate_grad, g);
            const float2 ir2 = bc2(__fmul_rn(n_ir, sgn)), irc2 = bc2(n_irc);
            uf8_decode8(cm, __fmul_rn(n_sc, 0.0078125f), mo);                    // fl(scale / 128), scale >= 1e-12
            if (k + 1 < nrows) {
                n_ir = __ldg(sT.inv_row + row + 8); n_sc = __ldg(scp + (k + 1) * scstep);
                if (L.came) n_irc = __ldg(sT.inv_row_conf + row + 8);
            }
            if (L.came) {
#pragma unroll
                for (int j = 0; j < 8; j += 2) {
                    const float2 ut = div_by2(__fmul2_rn(__fmul2_rn(make_float2(g[j], g[j + 1]), ir2), make_float2(ic[j], ic[j + 1])), D);
                    const float2 mm = lerp_w2(mo[j >> 1], ut, LW);
                    const float2 uj = __fmul2_rn(__fmul2_rn(mm, irc2), make_float2(icc[j], icc[j + 1]));
                    mj[j] = mm.x; mj[j + 1] = mm.y; u[j] = uj.x; u[j + 1] = uj.y;
                }
            } else {
#pragma unroll
                for (int j = 0; j < 8; j += 2) {
                    const float2 mm = lerp_w2(mo[j >> 1], make_float2(g[j], g[j + 1]), LW);
                    const float2 uj = __fmul2_rn(__fmul2_rn(mm, ir2), make_float2(ic[j], ic[j + 1]));
                    mj[j] = mm.x; mj[j + 1] = mm.y; u[j] = uj.x; u[j + 1] = uj.y;
                }
            }
            float p[8] = {cp0.x, cp0.y, cp0.z, cp0.w, cp1.x, cp1.y, cp1.z, cp1.w};
#pragma unroll
            for (int j = 0; j < 8; j += 2) {
                float2 pj = __fmul2_rn(make_float2(p[j], p[j + 1]), decay2);
                if (!zero_upd) pj = __ffma2_rn(step2, __fmul2_rn(make_float2(u[j], u[j + 1]), fira2), pj);
                p[j] = pj.x; p[j + 1] = pj.y;
            }
            float *pp = pbase + flat;
            *reinterpret_cast<float4 *>(pp) = make_float4(p[0], p[1], p[2], p[3]);
            *reinterpret_cast<float4 *>(pp + 4) = make_float4(p[4], p[5], p[6], p[7]);
            if (sT.param_copy != nullptr)                                    // bf16 compute copy
                *reinterpret_cast<uint4 *>(static_cast<uint16_t *>(sT.param_copy) + flat) =
                    make_uint4(bf16x2_rn(p[0], p[1]), bf16x2_rn(p[2], p[3]), bf16x2_rn(p[4], p[5]), bf16x2_rn(p[6], p[7]));
            // the row slice is one momentum block of 256
            float am = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j) am = fmaxf(am, fabsf(mj[j]));
            am = fmaxf(warp_max(am), 1e-12f);
            const DivBy A = make_div(am);
            const uint32_t o0 = uf8_encode_fast2(make_float2(mj[0], mj[1]), A) | (uf8_encode_fast2(make_float2(mj[2], mj[3]), A) << 16);
            const uint32_t o1 = uf8_encode_fast2(make_float2(mj[4], mj[5]), A) | (uf8_encode_fast2(make_float2(mj[6], mj[7]), A) << 16);
            *reinterpret_cast<uint2 *>(sT.m_q + flat) = make_uint2(o0, o1);
            if (lane == 0) scp[k * scstep] = am;
        }
        cons += (uint32_t)nrows;
    }
}

// ---------------------------------------------------------------------------
// The sum-of-squares pass over u = g * inv_row * inv_col (CAME's first sum, Adafactor without
// momentum): it only reads the gradient, 2 bytes per parameter, and with one 128-bit load per
// thread in flight (the kernel above) it was bound by memory latency.  Here a thread takes NE = 16
// consecutive elements per step of 4096 (8 where the columns are no multiple of 16) and the loads
// of its next step are issued before the current values are used: four times the bytes in flight.
// Partial sums as in factored_update_vec_kernel: one binary64 partial per thread over the chunks of
// a tensor that the CTA processes, reduced once per tensor into the slot of the run's first chunk.
// ---------------------------------------------------------------------------
template <typename GradT, int NE>
__device__ __forceinline__ double sumsq_span(const FactoredLaunch &L, const af8_factored_tensor &sT, int64_t e0, int64_t e1)
{
    constexpr int NV = NE / 8;                                   // 8-element vectors per thread and step
    constexpr int64_t STEP = (int64_t)FUPD_THREADS * NE;
    const int64_t C = sT.cols;
    double acc = 0.0;
    int64_t e = e0 + (int64_t)threadIdx.x * NE;
    if (e >= e1) return acc;
    int64_t row = e / C, col = e - row * C;
    GradRaw8<GradT> cur[NV], nxt[NV];
#pragma unroll
    for (int v = 0; v < NV; ++v) cur[v].load(sT.grad, e + 8 * v);
    for (; e < e1; e += STEP) {
        const bool more = e + STEP < e1;
        if (more) {
#pragma unroll
            for (int v = 0; v < NV; ++v) nxt[v].load(sT.grad, e + STEP + 8 * v);
        }
        const float2 ir2 = bc2(__ldg(sT.inv_row + row));
#pragma unroll
        for (int v = 0; v < NV; ++v) {
            float g[8], ic[8];
            cur[v].unpack(0, g);                                 // (the sign does not matter for the square)
            load_f8_ro(sT.inv_col + col + 8 * v, ic);
            float2 a2 = make_float2(0.0f, 0.0f);
#pragma unroll
            for (int j = 0; j < 8; j += 2) {
                const float2 uj = __fmul2_rn(__fmul2_rn(make_float2(g[j], g[j + 1]), ir2), make_float2(ic[j], ic[j + 1]));
                a2 = j == 0 ? __fmul2_rn(uj, uj) : __ffma2_rn(uj, uj, a2);
            }
            acc += (double)__fadd_rn(a2.x, a2.y);
            if (more) cur[v] = nxt[v];
        }
        col += STEP;
        if (col >= C) {
            if (C >= STEP) { col -= C; ++row; }
            else { const int64_t q = col / C; row += q; col -= q * C; }
        }
    }
    return acc;
}

template <typename GradT>
__global__ void __launch_bounds__(FUPD_THREADS, 4)
factored_sumsq_wide_kernel(const FactoredLaunch L)
{
    __shared__ af8_factored_tensor sT;
    __shared__ double s_acc2[FUPD_THREADS / 32];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int64_t per_cta = (L.total_units + gridDim.x - 1) / gridDim.x;
    const int64_t id_begin = (int64_t)blockIdx.x * per_cta;
    const int64_t id_end = min(id_begin + per_cta, L.total_units);
    int tn = -1;
    for (int64_t id = id_begin; id < id_end;) {
        if (tn < 0) tn = find_factored_chunk(L.tensors, L.n_tensors, id);
        else while (tn + 1 < L.n_tensors && __ldg(&L.tensors[tn + 1].first_chunk) <= id) ++tn;
        __syncthreads();
        if (tid < (int)(sizeof(af8_factored_tensor) / 4))
            reinterpret_cast<uint32_t *>(&sT)[tid] = __ldg(reinterpret_cast<const uint32_t *>(L.tensors + tn) + tid);
        __syncthreads();
        const int64_t next_first = tn + 1 < L.n_tensors ? __ldg(&L.tensors[tn + 1].first_chunk) : L.total_units;
        const int64_t run_end = min(id_end, next_first);         // this CTA's chunks of this tensor: id .. run_end - 1
        const int64_t e0 = (id - sT.first_chunk) * 2048;
        const int64_t e1 = min((run_end - sT.first_chunk) * 2048, sT.rows * sT.cols);
        double acc = (sT.cols % 16 == 0) ? sumsq_span<GradT, 16>(L, sT, e0, e1) : sumsq_span<GradT, 8>(L, sT, e0, e1);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (lane == 0) s_acc2[warp] = acc;
        __syncthreads();
        if (tid == 0) {
            double sum = 0.0;
            for (int w = 0; w < FUPD_THREADS / 32; ++w) sum += s_acc2[w];
            L.block_sumsq[id] = sum;
        }
        for (int64_t i = id + 1 + tid; i < run_end; i += FUPD_THREADS) L.block_sumsq[i] = 0.0;
        id = run_end;
    }
}

// The same sum over the 512 x 256 tiles of the statistic pass: a lane keeps the inverse column factors of
// its 8 columns in registers while its warp walks the tile's rows (the flat kernel above re-reads them for
// every element, twice the bytes of the gradient itself through L1), four rows' loads in flight.  A CTA adds
// its tile's sum to the slot of the tensor's first chunk; the caller clears the slots first.
template <typename GradT>
__global__ void __launch_bounds__(256, 4)
factored_sumsq_tile_kernel(const FactoredLaunch L)
{
    constexpr int NB = 4;
    __shared__ af8_factored_tensor sT;
    __shared__ double s_acc2[8];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    int cur_t = -1;
    for (int64_t id = blockIdx.x; id < L.total_units; id += gridDim.x) {
        int t = cur_t;
        if (t < 0) t = find_factored_tile(L.tensors, L.n_tensors, id);
        else while (t + 1 < L.n_tensors && __ldg(&L.tensors[t + 1].first_tile) <= id) ++t;
        __syncthreads();                                           // s_acc2 of the previous tile was read
        if (t != cur_t) {
            if (tid < (int)(sizeof(af8_factored_tensor) / 4))
                reinterpret_cast<uint32_t *>(&sT)[tid] = __ldg(reinterpret_cast<const uint32_t *>(L.tensors + t) + tid);
            cur_t = t;
            __syncthreads();
        }
        const int64_t R = sT.rows, C = sT.cols;
        const int64_t ntc = (C + FSTAT_COLS - 1) / FSTAT_COLS;
        const int64_t local = id - sT.first_tile;
        const int64_t r0 = (local / ntc) * FSTAT_ROWS;
        const int64_t c = (local % ntc) * FSTAT_COLS + lane * 8;   // this lane's 8 columns
        const bool col_ok = c < C;                                 // C % 8 == 0: all 8 or none
        float ic[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) ic[j] = 0.0f;
        if (col_ok) load_f8_ro(sT.inv_col + c, ic);
        double acc = 0.0;
        GradRaw8<GradT> cur[NB], nxt[NB];
        auto fetch = [&](GradRaw8<GradT> (&dst)[NB], int k0) {
#pragma unroll
            for (int k = 0; k < NB; ++k) {
                const int64_t r = r0 + warp + 8 * (k0 + k);
                if (col_ok && r < R && k0 + k < FSTAT_ROWS / 8) dst[k].load(sT.grad, r * C + c);
                else dst[k].zero();
            }
        };
        fetch(cur, 0);
        for (int k0 = 0; k0 < FSTAT_ROWS / 8; k0 += NB) {
            if (r0 + warp + 8 * k0 >= R) break;                    // uniform over the warp
            fetch(nxt, k0 + NB);
#pragma unroll
            for (int k = 0; k < NB; ++k) {
                const int64_t r = min(r0 + warp + 8 * (int64_t)(k0 + k), R - 1);     // (a row beyond the end carries zeros)
                const float2 ir2 = bc2(__ldg(sT.inv_row + r));
                float g[8];
                cur[k].unpack(0, g);                               // (the sign does not matter for the square)
                float2 a2 = make_float2(0.0f, 0.0f);
#pragma unroll
                for (int j = 0; j < 8; j += 2) {
                    const float2 uj = __fmul2_rn(__fmul2_rn(make_float2(g[j], g[j + 1]), ir2), make_float2(ic[j], ic[j + 1]));
                    a2 = j == 0 ? __fmul2_rn(uj, uj) : __ffma2_rn(uj, uj, a2);
                }
                acc += (double)__fadd_rn(a2.x, a2.y);
                cur[k] = nxt[k];
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (lane == 0) s_acc2[warp] = acc;
        __syncthreads();
        if (tid == 0) {
            double sum = 0.0;
            for (int w = 0; w < 8; ++w) sum += s_acc2[w];
            atomicAdd(L.block_sumsq + sT.first_chunk, sum);
        }
    }
}

inline int factored_chunk_for(int m_block)
{
    if (m_block <= 0) return 2048;
    int k = 2048 / m_block;
    if (k < 1) k = 1;
    return k * m_block;
}

inline int validate_factored(const af8_factored_cfg &c, const af8_factored_tensor *T, int n)
{
    const bool has_m = c.m_fmt != AF8_M_NONE;
    const bool m_quant = has_m && c.m_fmt != AF8_M_FP32;
    const int chunk = factored_chunk_for(m_quant ? c.m_block : 0);
    int64_t next_chunk = 0, next_tile = 0, next_small = 0;
    for (int i = 0; i < n; ++i) {
        const af8_factored_tensor &t = T[i];
        if (t.rows <= 0 || t.cols <= 0) return fail(AF8_ERR_INVALID, "factored tensor %d: empty shape", i);
        if (c.aligned8) {
            if (t.cols % 8 != 0) return fail(AF8_ERR_INVALID, "factored tensor %d: aligned8 needs cols %% 8 == 0", i);
            const void *ptrs[] = {t.param, t.grad, t.m_q, t.m_f32, t.inv_col, t.inv_col_conf, t.param_copy};
            for (const void *q : ptrs)
                if (q && (reinterpret_cast<uintptr_t>(q) & 15u)) return fail(AF8_ERR_INVALID, "factored tensor %d: aligned8 needs 16-byte aligned arrays", i);
        }
        if (t.rows * t.cols >= ((int64_t)1 << 40)) return fail(AF8_ERR_UNSUPPORTED, "factored tensor %d: too large", i);
        if (t.param_copy && c.param_dtype != AF8_F32) return fail(AF8_ERR_INVALID, "factored tensor %d: a bf16 copy exists only of fp32 parameters", i);
        if (!t.param || !t.grad || !t.row_sum || !t.col_sum || !t.inv_row || !t.inv_col)
            return fail(AF8_ERR_INVALID, "factored tensor %d: null pointer", i);
        if (c.came && (!t.inv_row_conf || !t.inv_col_conf)) return fail(AF8_ERR_INVALID, "factored tensor %d: CAME needs the confidence vectors", i);
        if (m_quant && (!t.m_q || !t.m_scale)) return fail(AF8_ERR_INVALID, "factored tensor %d: null quantised momentum", i);
        if (c.m_fmt == AF8_M_FP32 && !t.m_f32) return fail(AF8_ERR_INVALID, "factored tensor %d: null fp32 momentum", i);
        if (t.first_chunk != next_chunk) return fail(AF8_ERR_INVALID, "factored tensor %d: first_chunk %lld, expected %lld", i, (long long)t.first_chunk, (long long)next_chunk);
        if (t.first_tile != next_tile) return fail(AF8_ERR_INVALID, "factored tensor %d: first_tile %lld, expected %lld", i, (long long)t.first_tile, (long long)next_tile);
        next_chunk += (t.rows * t.cols + chunk - 1) / chunk;
        if (t.batch_rows < 0 || (t.batch_rows > 0 && t.rows % t.batch_rows != 0))
            return fail(AF8_ERR_INVALID, "factored tensor %d: batch_rows %lld does not divide rows %lld", i, (long long)t.batch_rows, (long long)t.rows);
        if (t.batch_rows > 0 && c.aligned8)
            return fail(AF8_ERR_INVALID, "factored tensor %d: a batch of matrices takes the general kernels (cfg.aligned8 = 0)", i);
        next_tile += fact_tiles(t);
        const af8_small_state *ss[4] = {&t.row_var, &t.col_var, &t.conf_row, &t.conf_col};
        const int sb = t.row_var.block;
        if (sb <= 0) return fail(AF8_ERR_INVALID, "factored tensor %d: small-state block must be positive", i);
        if (t.first_small != next_small) return fail(AF8_ERR_INVALID, "factored tensor %d: first_small %d, expected %lld", i, t.first_small, (long long)next_small);
        next_small += (t.rows + sb - 1) / sb + (fact_batch(t) * t.cols + sb - 1) / sb;
        if (next_small > 0x7fffffff) return fail(AF8_ERR_UNSUPPORTED, "factored table: too many small-state blocks");
        for (int k = 0; k < (c.came ? 4 : 2); ++k) {
            const af8_small_state &s = *ss[k];
            if (s.block != sb) return fail(AF8_ERR_INVALID, "factored tensor %d: the small states of a tensor must share one block size", i);
            if (s.fmt == AF8_V_FP32) {
                if (!s.f32) return fail(AF8_ERR_INVALID, "factored tensor %d: null fp32 small state %d", i, k);
            } else if (s.fmt == AF8_V_AL8 || s.fmt == AF8_V_AL16) {
                if (!s.q || !s.scale || !s.min_log) return fail(AF8_ERR_INVALID, "factored tensor %d: null quantised small state %d", i, k);
                if (s.block < 128 || s.block % 128 != 0 || s.block > GEN_MAX_BLOCK) return fail(AF8_ERR_INVALID, "factored tensor %d: bad block %d of small state %d", i, s.block, k);
            } else {
                return fail(AF8_ERR_INVALID, "factored tensor %d: bad format %d of small state %d", i, s.fmt, k);
            }
        }
    }
    return AF8_OK;
}

inline int check_factored_cfg(const af8_factored_cfg *cfg, const char *who)
{
    if (!cfg) return fail(AF8_ERR_INVALID, "%s: null cfg", who);
    if (cfg->param_dtype != AF8_F32 && cfg->param_dtype != AF8_BF16 && cfg->param_dtype != AF8_F16) return fail(AF8_ERR_INVALID, "%s: bad param_dtype %d", who, cfg->param_dtype);
    if (cfg->grad_dtype != AF8_F32 && cfg->grad_dtype != AF8_BF16 && cfg->grad_dtype != AF8_F16) return fail(AF8_ERR_INVALID, "%s: bad grad_dtype %d", who, cfg->grad_dtype);
    if (cfg->stochastic_round && cfg->param_dtype == AF8_F32) return fail(AF8_ERR_INVALID, "%s: stochastic rounding applies to bf16 / fp16 parameters only", who);
    if (cfg->m_fmt < AF8_M_NONE || cfg->m_fmt > AF8_M_FP32) return fail(AF8_ERR_INVALID, "%s: bad m_fmt %d", who, cfg->m_fmt);
    const bool m_quant = cfg->m_fmt != AF8_M_NONE && cfg->m_fmt != AF8_M_FP32;
    if (m_quant && (cfg->m_block < 32 || cfg->m_block % 4 != 0 || cfg->m_block > 2048)) return fail(AF8_ERR_INVALID, "%s: bad m_block %d", who, cfg->m_block);
    if (cfg->came && cfg->m_fmt == AF8_M_NONE) return fail(AF8_ERR_INVALID, "%s: CAME needs momentum", who);
    return AF8_OK;
}

inline FactoredLaunch make_factored_launch(const af8_factored_cfg &c, const af8_factored_tensor *dev, int n,
                                           int64_t units, const af8_dyn_scalars *dyn, double *sumsq)
{
    FactoredLaunch L;
    L.tensors = dev; L.dyn = dyn; L.block_sumsq = sumsq; L.total_units = units; L.n_tensors = n;
    L.grad_dtype = c.grad_dtype; L.m_fmt = c.m_fmt; L.m_block = c.m_block > 0 ? c.m_block : 256;
    L.came = c.came ? 1 : 0; L.negate_grad = c.negate_grad ? 1 : 0; L.mode = c.mode; L.v_floor = c.v_floor;
    L.param_dtype = c.param_dtype; L.sr = c.stochastic_round ? 1 : 0;
    return L;
}

}  // namespace af8

extern "C" int32_t af8_factored_chunk(int32_t m_block) { return af8::factored_chunk_for(m_block); }
extern "C" int32_t af8_factored_tile_rows(void) { return af8::FSTAT_ROWS; }
extern "C" int32_t af8_factored_tile_cols(void) { return af8::FSTAT_COLS; }

extern "C" int af8_factored_upload(const af8_factored_cfg *cfg, const af8_factored_tensor *host_tensors,
                                   af8_factored_tensor *dev_tensors, int32_t n_tensors, void *stream)
{
    using namespace af8;
    int rc = check_factored_cfg(cfg, "af8_factored_upload");
    if (rc) return rc;
    if (!host_tensors || !dev_tensors || n_tensors <= 0) return fail(AF8_ERR_INVALID, "af8_factored_upload: null or empty table");
    rc = validate_factored(*cfg, host_tensors, n_tensors);
    if (rc) return rc;
    AF8_CUDA_TRY(cudaMemcpyAsync(dev_tensors, host_tensors, sizeof(af8_factored_tensor) * (size_t)n_tensors,
                                 cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream)));
    return AF8_OK;
}

namespace af8 {
// the two tensor maps of a tensor for residual_rows_box: gradient (bf16) and UF8 codes as [rows][cols], boxes of
// 256 columns x FBOX_ROWS rows, no swizzle, zeros outside
inline int factored_box_maps(const af8_factored_tensor &t, CUtensorMap *out)
{
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return fail(AF8_ERR_CUDA, "cuTensorMapEncodeTiled is not available");
    const cuuint64_t dim[2] = {(cuuint64_t)t.cols, (cuuint64_t)t.rows};
    const cuuint32_t box[2] = {256, FBOX_ROWS}, es[2] = {1, 1};
    const cuuint64_t gstride[1] = {(cuuint64_t)t.cols * 2}, mstride[1] = {(cuuint64_t)t.cols};
    CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(t.grad), dim, gstride, box, es,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(AF8_ERR_CUDA, "cuTensorMapEncodeTiled (gradient rows) failed with %d", (int)r);
    r = enc(out + 1, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, t.m_q, dim, mstride, box, es,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(AF8_ERR_CUDA, "cuTensorMapEncodeTiled (momentum codes) failed with %d", (int)r);
    return AF8_OK;
}
}  // namespace af8

static int af8_factored_stats_impl(const af8_factored_cfg *cfg, const af8_factored_tensor *dev_tensors,
                                   const af8_factored_tensor *host_tensors, int32_t n_tensors,
                                   const af8_dyn_scalars *dyn, void *host_maps, void *dev_maps, void *stream)
{
    using namespace af8;
    int rc = check_factored_cfg(cfg, "af8_factored_stats");
    if (rc) return rc;
    if (!dev_tensors || !host_tensors || n_tensors <= 0) return fail(AF8_ERR_INVALID, "af8_factored_stats: null or empty table");
    if (cfg->mode != AF8_FSTAT_GRADSQ && cfg->mode != AF8_FSTAT_RESIDUAL) return fail(AF8_ERR_INVALID, "af8_factored_stats: bad mode %d", cfg->mode);
    if (cfg->mode == AF8_FSTAT_RESIDUAL && (!cfg->came || !dyn)) return fail(AF8_ERR_INVALID, "af8_factored_stats: the residual needs CAME and dyn");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int64_t tiles = 0;
    // clear the accumulators; ranges that follow one another in memory share one memset
    char *run_begin = nullptr, *run_end = nullptr;
    for (int i = 0; i < n_tensors; ++i) {
        const af8_factored_tensor &t = host_tensors[i];
        char *const ptr[2] = {reinterpret_cast<char *>(t.row_sum), reinterpret_cast<char *>(t.col_sum)};
        const size_t len[2] = {sizeof(double) * (size_t)t.rows, sizeof(double) * (size_t)(fact_batch(t) * t.cols)};
        for (int k = 0; k < 2; ++k) {
            if (ptr[k] == run_end) { run_end += len[k]; continue; }
            if (run_end != run_begin) AF8_CUDA_TRY(cudaMemsetAsync(run_begin, 0, (size_t)(run_end - run_begin), st));
            run_begin = ptr[k];
            run_end = ptr[k] + len[k];
        }
        tiles += fact_tiles(t);
    }
    if (run_end != run_begin) AF8_CUDA_TRY(cudaMemsetAsync(run_begin, 0, (size_t)(run_end - run_begin), st));
    FactoredLaunch L = make_factored_launch(*cfg, dev_tensors, n_tensors, tiles, dyn, nullptr);
    int64_t grid = (int64_t)sm_count() * 6;
    if (grid > tiles) grid = tiles;
    const bool bf = cfg->grad_dtype == AF8_BF16, res = cfg->mode == AF8_FSTAT_RESIDUAL;
    const bool vec = cfg->aligned8 && cfg->grad_dtype != AF8_F16;      // fp16 gradients take the general kernels
    static const bool ring_off = getenv("AF8_NO_FACTORED_RING") != nullptr;
    static const bool box_off = getenv("AF8_NO_FACTORED_BOXES") != nullptr;
    int ring = (ring_off || !res) ? 0 : 1;
    // residual pass over bf16 gradients and UF8 codes of tensors with cols % 256 == 0: boxes of rows through
    // tensor maps, when the caller has given room for the maps
    const CUtensorMap *maps = nullptr;
    if (ring && !box_off && vec && bf && host_maps && dev_maps && cfg->m_fmt == AF8_M_UF8 && cfg->m_block == 256 && cfg->cols_mult256) {
        bool ok = (reinterpret_cast<uintptr_t>(dev_maps) & 63) == 0;
        for (int i = 0; i < n_tensors && ok; ++i) {
            const af8_factored_tensor &t = host_tensors[i];
            ok = fact_batch(t) == 1 && t.rows < ((int64_t)1 << 31) && t.cols < ((int64_t)1 << 31) && (t.cols % 256) == 0 &&
                 t.rows * (t.cols >> 8) < ((int64_t)1 << 31);
        }
        if (ok) {
            CUtensorMap *hm = static_cast<CUtensorMap *>(host_maps);
            for (int i = 0; i < n_tensors; ++i) {
                rc = factored_box_maps(host_tensors[i], hm + 2 * i);
                if (rc) return rc;
            }
            AF8_CUDA_TRY(cudaMemcpyAsync(dev_maps, host_maps, sizeof(CUtensorMap) * 2 * (size_t)n_tensors, cudaMemcpyHostToDevice, st));
            maps = static_cast<const CUtensorMap *>(dev_maps);
            ring = 2;
        }
    }
#define AF8_LAUNCH_FSTAT(G, RES) do { \
        const size_t sm = ring ? sring_smem_bytes<G, RES>() : 0; \
        if (sm > 0) AF8_CUDA_TRY(cudaFuncSetAttribute(factored_stats_vec_kernel<G, RES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm)); \
        factored_stats_vec_kernel<G, RES><<<(int)grid, 256, sm, st>>>(L, ring, maps); } while (0)
    if (vec && bf && res) AF8_LAUNCH_FSTAT(bf16_tag, true);
    else if (vec && bf) AF8_LAUNCH_FSTAT(bf16_tag, false);
    else if (vec && res) AF8_LAUNCH_FSTAT(float, true);
    else if (vec) AF8_LAUNCH_FSTAT(float, false);
#undef AF8_LAUNCH_FSTAT
    else factored_stats_kernel<<<(int)grid, 256, 0, st>>>(L);
    AF8_CUDA_TRY(cudaGetLastError());
    return AF8_OK;
}

extern "C" int af8_factored_stats(const af8_factored_cfg *cfg, const af8_factored_tensor *dev_tensors,
                                  const af8_factored_tensor *host_tensors, int32_t n_tensors,
                                  const af8_dyn_scalars *dyn, void *stream)
{
    return af8_factored_stats_impl(cfg, dev_tensors, host_tensors, n_tensors, dyn, nullptr, nullptr, stream);
}

extern "C" int af8_factored_stats_boxes(const af8_factored_cfg *cfg, const af8_factored_tensor *dev_tensors,
                                        const af8_factored_tensor *host_tensors, int32_t n_tensors,
                                        const af8_dyn_scalars *dyn, void *host_maps, void *dev_maps, void *stream)
{
    return af8_factored_stats_impl(cfg, dev_tensors, host_tensors, n_tensors, dyn, host_maps, dev_maps, stream);
}

extern "C" int af8_factored_small(const af8_factored_cfg *cfg, const af8_factored_tensor *dev_tensors,
                                  int32_t n_tensors, int32_t conf, int32_t total_units, void *stream)
{
    using namespace af8;
    int rc = check_factored_cfg(cfg, "af8_factored_small");
    if (rc) return rc;
    if (!dev_tensors || n_tensors <= 0 || total_units <= 0) return fail(AF8_ERR_INVALID, "af8_factored_small: null or empty table");
    if (conf && !cfg->came) return fail(AF8_ERR_INVALID, "af8_factored_small: confidence states exist only with CAME");
    const size_t smem = sizeof(float) * GEN_MAX_BLOCK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    factored_small_kernel<<<total_units, 256, smem, st>>>(dev_tensors, n_tensors, conf, cfg->v_floor);
    AF8_CUDA_TRY(cudaGetLastError());
    factored_inv_kernel<<<dim3((unsigned)n_tensors, 8), 256, 0, st>>>(dev_tensors, conf);
    AF8_CUDA_TRY(cudaGetLastError());
    return AF8_OK;
}

extern "C" int af8_factored_update(const af8_factored_cfg *cfg, const af8_factored_tensor *dev_tensors,
                                   int32_t n_tensors, int64_t total_chunks, const af8_dyn_scalars *dyn,
                                   double *block_sumsq, void *stream)
{
    using namespace af8;
    int rc = check_factored_cfg(cfg, "af8_factored_update");
    if (rc) return rc;
    if (!dev_tensors || n_tensors <= 0 || total_chunks <= 0) return fail(AF8_ERR_INVALID, "af8_factored_update: null or empty table");
    if (cfg->mode < AF8_FUPD_SUMSQ_U || cfg->mode > AF8_FUPD_LAG) return fail(AF8_ERR_INVALID, "af8_factored_update: bad mode %d", cfg->mode);
    if (cfg->mode == AF8_FUPD_LAG && (cfg->came || !dyn)) return fail(AF8_ERR_INVALID, "af8_factored_update: the lag pass needs dyn and excludes CAME");
    if (cfg->mode != AF8_FUPD_APPLY && !block_sumsq) return fail(AF8_ERR_INVALID, "af8_factored_update: this mode needs block_sumsq");
    if (cfg->mode == AF8_FUPD_SUMSQ_U && !cfg->came) return fail(AF8_ERR_INVALID, "af8_factored_update: SUMSQ_U is a CAME pass");
    if (cfg->came && cfg->mode != AF8_FUPD_SUMSQ_U && !dyn) return fail(AF8_ERR_INVALID, "af8_factored_update: CAME passes need dyn");
    const bool m_quant = cfg->m_fmt != AF8_M_NONE && cfg->m_fmt != AF8_M_FP32;
    const int chunk = factored_chunk_for(m_quant ? cfg->m_block : 0);
    FactoredLaunch L = make_factored_launch(*cfg, dev_tensors, n_tensors, total_chunks, dyn, block_sumsq);
    const size_t smem = sizeof(float) * (size_t)chunk;
    int64_t grid = (int64_t)sm_count() * 6;
    if (grid > total_chunks) grid = total_chunks;
    const bool vec = cfg->aligned8 && chunk == 2048 && (!m_quant || cfg->m_block == 256) && cfg->grad_dtype != AF8_F16;
    const bool apply = cfg->mode == AF8_FUPD_APPLY || cfg->mode == AF8_FUPD_LAG;
    const bool lag = cfg->mode == AF8_FUPD_LAG;
    if (vec) {                                   // persistent: the CTAs that are resident together
        grid = (int64_t)sm_count() * (apply ? (cfg->m_fmt == AF8_M_NONE ? 2 : 3) : 4);
        if (grid > total_chunks) grid = total_chunks;
    }
    cudaStream_t cst = static_cast<cudaStream_t>(stream);
    const bool bf = cfg->grad_dtype == AF8_BF16;
    const bool no_m = cfg->m_fmt == AF8_M_NONE;
    static const bool ring_off = getenv("AF8_NO_FACTORED_RING") != nullptr;
    static const bool wide_off = getenv("AF8_NO_WIDE_SUMS") != nullptr;
    static const bool tile_off = getenv("AF8_NO_TILE_SUMS") != nullptr;
    const int64_t total_tiles = cfg->total_tiles;
    if (vec && !apply && !tile_off && total_tiles > 0 && cfg->grad_dtype != AF8_F16 && ((cfg->came && cfg->mode == AF8_FUPD_SUMSQ_U) || no_m)) {
        // the sum only needs the gradient: over the statistic tiles, column factors in registers
        AF8_CUDA_TRY(cudaMemsetAsync(block_sumsq, 0, sizeof(double) * (size_t)total_chunks, cst));
        FactoredLaunch LT = L;
        LT.total_units = total_tiles;
        int64_t tg = (int64_t)sm_count() * 8;
        if (tg > total_tiles) tg = total_tiles;
        if (bf) factored_sumsq_tile_kernel<bf16_tag><<<(int)tg, 256, 0, cst>>>(LT);
        else factored_sumsq_tile_kernel<float><<<(int)tg, 256, 0, cst>>>(LT);
        AF8_CUDA_TRY(cudaGetLastError());
        return AF8_OK;
    }
    if (vec && !apply && !wide_off && cfg->grad_dtype != AF8_F16 && ((cfg->came && cfg->mode == AF8_FUPD_SUMSQ_U) || no_m)) {
        // the sum only needs the gradient: 16 elements per thread, next step's loads in flight
        if (bf) factored_sumsq_wide_kernel<bf16_tag><<<(int)grid, FUPD_THREADS, 0, cst>>>(L);
        else factored_sumsq_wide_kernel<float><<<(int)grid, FUPD_THREADS, 0, cst>>>(L);
        AF8_CUDA_TRY(cudaGetLastError());
        return AF8_OK;
    }
    static const bool tile_apply_off = getenv("AF8_NO_TILE_APPLY") != nullptr;
    if (vec && cfg->mode == AF8_FUPD_APPLY && cfg->m_fmt == AF8_M_UF8 && cfg->param_dtype == AF8_F32 && !ring_off && !tile_apply_off &&
        cfg->total_tiles > 0 && cfg->cols_mult256) {
        // every row slice of 256 columns is one momentum block: tile order, column factors in registers
        FactoredLaunch LT = L;
        LT.total_units = cfg->total_tiles;
        if (bf) {
            int64_t tg = std::min<int64_t>((int64_t)sm_count() * 3, cfg->total_tiles);
            AF8_CUDA_TRY(cudaFuncSetAttribute(factored_apply_tile_kernel<bf16_tag, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fring_smem_bytes<bf16_tag>()));
            factored_apply_tile_kernel<bf16_tag, 3><<<(int)tg, FUPD_THREADS, fring_smem_bytes<bf16_tag>(), cst>>>(LT);
        } else {
            int64_t tg = std::min<int64_t>((int64_t)sm_count() * 2, cfg->total_tiles);
            AF8_CUDA_TRY(cudaFuncSetAttribute(factored_apply_tile_kernel<float, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fring_smem_bytes<float>()));
            factored_apply_tile_kernel<float, 2><<<(int)tg, FUPD_THREADS, fring_smem_bytes<float>(), cst>>>(LT);
        }
        AF8_CUDA_TRY(cudaGetLastError());
        return AF8_OK;
    }
    if (vec && cfg->mode == AF8_FUPD_APPLY && cfg->m_fmt == AF8_M_UF8 && cfg->param_dtype == AF8_F32 && !ring_off) {
        // fp32 parameters, UF8 momentum: inputs through per-warp rings of bulk copies
        if (bf) {
            AF8_CUDA_TRY(cudaFuncSetAttribute(factored_apply_ring_kernel<bf16_tag, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fring_smem_bytes<bf16_tag>()));
            factored_apply_ring_kernel<bf16_tag, 3><<<(int)grid, FUPD_THREADS, fring_smem_bytes<bf16_tag>(), cst>>>(L);
        } else {
            grid = std::min<int64_t>((int64_t)sm_count() * 2, total_chunks);
            AF8_CUDA_TRY(cudaFuncSetAttribute(factored_apply_ring_kernel<float, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fring_smem_bytes<float>()));
            factored_apply_ring_kernel<float, 2><<<(int)grid, FUPD_THREADS, fring_smem_bytes<float>(), cst>>>(L);
        }
        AF8_CUDA_TRY(cudaGetLastError());
        return AF8_OK;
    }
#define AF8_LAUNCH_FUPD(G, P, C) factored_update_vec_kernel<G, P, C><<<(int)grid, FUPD_THREADS, 0, cst>>>(L)
    if (vec && bf && lag) { if (no_m) AF8_LAUNCH_FUPD(bf16_tag, 2, 2); else AF8_LAUNCH_FUPD(bf16_tag, 2, 3); }
    else if (vec && lag) { if (no_m) AF8_LAUNCH_FUPD(float, 2, 2); else AF8_LAUNCH_FUPD(float, 2, 3); }
    else if (vec && bf && apply) { if (no_m) AF8_LAUNCH_FUPD(bf16_tag, 1, 2); else AF8_LAUNCH_FUPD(bf16_tag, 1, 3); }
    else if (vec && bf) AF8_LAUNCH_FUPD(bf16_tag, 0, 4);
    else if (vec && apply) { if (no_m) AF8_LAUNCH_FUPD(float, 1, 2); else AF8_LAUNCH_FUPD(float, 1, 3); }
    else if (vec) AF8_LAUNCH_FUPD(float, 0, 4);
#undef AF8_LAUNCH_FUPD
    else factored_update_kernel<<<(int)grid, FUPD_THREADS, smem, static_cast<cudaStream_t>(stream)>>>(L, chunk);
    AF8_CUDA_TRY(cudaGetLastError());
    return AF8_OK;
}
