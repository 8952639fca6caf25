// APOLLO: Adam statistics kept in a randomly projected low-rank space, applied to
// the full gradient through per-channel (or per-tensor) scaling factors.
//
// Reference semantics: _update_param_apollo without factorisation and without
// CAME (optimizer.py:2587-3084).  The step of one tensor G (rows x cols) is
//   1. g_low = G @ Pt ("right", rows >= cols, Pt is cols x rank) or Pt @ G
//      ("left", Pt is rank x rows)                        optimizer.py:2678-2681
//   2. EMA + requantisation of the low-rank V (AL) and M (UF/dynamic) states
//      over the flattened g_low, update_low = m / (sqrt(v) + eps)
//                                                         optimizer.py:2763-2959
//   3. scaling factor per channel = ||update_low|| / (||g_low|| + 1e-8), global
//      norm sqrt(sum ||G_channel||^2 * factor^2)          optimizer.py:2961-2988
//   4. Fira limiter on that norm, clip, bias correction   optimizer.py:2990-3023
//   5. p = p*decay + (update_scale * G) * final_scale      optimizer.py:3073-3079
// Step 2 is the full-rank kernel run on g_low (its "parameter" output, with decay
// 0 and step 1, is update_low); this file holds steps 3, 4 and 5, the helpers of step 1
// (channel norms, bf16 planes of Pt) and its exact SIMT form.  The tensor-core forms of
// step 1 are in apollo_umma.cuh (tcgen05 + TMA) and apollo_mma.cuh (mma.sync).
#pragma once

#include <cstdlib>
#include <cstring>

#include "common.cuh"
#include "fullrank_fast.cuh"
#include "apollo_mma.cuh"
#include "apollo_umma.cuh"

namespace af8 {

// gradient element with the reference's nan_to_num and maximize handling
// (optimizer.py:2601-2606)
__device__ __forceinline__ float apollo_grad(const void *g, int dtype, int64_t i, int negate)
{
    float x = dtype == AF8_BF16 ? bf16_bits_to_f32(static_cast<const uint16_t *>(g)[i]) : static_cast<const float *>(g)[i];
    if (!isfinite(x)) x = 0.0f;
    return negate ? -x : x;
}

__device__ __forceinline__ float apollo_grad_flag(const void *g, int dtype, int64_t i, bool &odd)
{
    float x = dtype == AF8_BF16 ? bf16_bits_to_f32(static_cast<const uint16_t *>(g)[i]) : static_cast<const float *>(g)[i];
    if (!isfinite(x)) { x = 0.0f; odd = true; }
    return x;
}

// ---------------------------------------------------------------------------
// 1. projection: C[M x N] = A[M x K] * B[K x N], A or B being the gradient.
//    Register-tiled SIMT kernel: 64 x 64 tile per CTA, 4 x 4 per thread, K step 16.
//    Products of two binary32 numbers are exact in binary64 and the accumulation runs in
//    binary64, so every output is the correctly rounded dot product whatever the order of
//    summation: the low-rank states that are quantised from it do not depend on tiling.
//    This is the path of fp32 gradients and odd shapes, and the bit-exact reference of the
//    tensor-core kernels, whose binary32 accumulation moves codes next to a block minimum.
// ---------------------------------------------------------------------------
constexpr int PJ_TM = 64, PJ_TN = 64, PJ_TK = 16;

// GRAD_IS_A: A is the gradient (right side: A = G, B = Pt); else B is the gradient (left: A = Pt, B = G)
template <bool GRAD_IS_A>
__global__ void __launch_bounds__(256)
apollo_project_kernel(const void *grad, int grad_dtype, int negate, const float *pt, float *out, int M, int N, int K)
{
    __shared__ float sA[PJ_TK][PJ_TM + 1];
    __shared__ float sB[PJ_TK][PJ_TN + 1];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * PJ_TM, n0 = blockIdx.x * PJ_TN;
    double acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0;

    for (int k0 = 0; k0 < K; k0 += PJ_TK) {
        // A tile: 64 rows x 16 k; B tile: 16 k x 64 cols (1024 elements each, 4 per thread)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int idx = tid + e * 256;
            {   // A[m][k], row-major M x K
                const int mm = idx / PJ_TK, kk = idx % PJ_TK;
                const int m = m0 + mm, k = k0 + kk;
                float v = 0.0f;
                if (m < M && k < K)
                    v = GRAD_IS_A ? apollo_grad(grad, grad_dtype, (int64_t)m * K + k, negate) : pt[(int64_t)m * K + k];
                sA[kk][mm] = v;
            }
            {   // B[k][n], row-major K x N
                const int kk = idx / PJ_TN, nn = idx % PJ_TN;
                const int k = k0 + kk, n = n0 + nn;
                float v = 0.0f;
                if (k < K && n < N)
                    v = GRAD_IS_A ? pt[(int64_t)k * N + n] : apollo_grad(grad, grad_dtype, (int64_t)k * N + n, negate);
                sB[kk][nn] = v;
            }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < PJ_TK; ++kk) {
            double a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = (double)sA[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = (double)sB[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fma(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
            if (m < M && n < N) out[(int64_t)m * N + n] = __double2float_rn(acc[i][j]);
        }
}

// squared channel norms of G in binary64: per row (right) or per column (left)
__global__ void __launch_bounds__(256)
apollo_channel_sumsq_kernel(const void *grad, int grad_dtype, int64_t rows, int64_t cols, int right, double *chan,
                            int *nonfinite_flag)
{
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    bool odd = false;                                  // met a non-finite entry (which counts as zero)
    if (right) {
        for (int64_t r = (int64_t)blockIdx.x * 8 + warp; r < rows; r += (int64_t)gridDim.x * 8) {
            double a = 0.0;
            for (int64_t c = lane; c < cols; c += 32) {
                const float x = apollo_grad_flag(grad, grad_dtype, r * cols + c, odd);
                a += (double)__fmul_rn(x, x);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
            if (lane == 0) chan[r] = a;
        }
    } else {
        // one thread per column, a block of rows per CTA, combined with binary64 atomics
        const int64_t c = (int64_t)blockIdx.x * 256 + tid;
        const int64_t r0 = (int64_t)blockIdx.y * 256;
        if (c < cols) {
            double a = 0.0;
            const int64_t r1 = min(rows, r0 + 256);
            for (int64_t r = r0; r < r1; ++r) {
                const float x = apollo_grad_flag(grad, grad_dtype, r * cols + c, odd);
                a += (double)__fmul_rn(x, x);
            }
            atomicAdd(chan + c, a);
        }
    }
    if (nonfinite_flag != nullptr && odd) atomicOr(nonfinite_flag, 1);
}

// the same for bf16 gradients with cols % 8 == 0: 8 columns per thread, 128-bit loads
__device__ __forceinline__ void bf16x8_squares(const uint4 a, double (&acc)[8], bool &odd)
{
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        float x = __uint_as_float(w[k] << 16), y = __uint_as_float(w[k] & 0xffff0000u);
        if (!isfinite(x)) { x = 0.0f; odd = true; }
        if (!isfinite(y)) { y = 0.0f; odd = true; }
        acc[2 * k] += (double)__fmul_rn(x, x);
        acc[2 * k + 1] += (double)__fmul_rn(y, y);
    }
}

__global__ void __launch_bounds__(256)
apollo_channel_sumsq_bf16_kernel(const uint16_t *__restrict__ grad, int64_t rows, int64_t cols, int right, double *chan,
                                 int *nonfinite_flag)
{
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    bool odd = false;
    if (right) {
        for (int64_t r = (int64_t)blockIdx.x * 8 + warp; r < rows; r += (int64_t)gridDim.x * 8) {
            double acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            const uint16_t *row = grad + r * cols;
            for (int64_t c = (int64_t)lane * 8; c < cols; c += 256)
                bf16x8_squares(__ldg(reinterpret_cast<const uint4 *>(row + c)), acc, odd);
            double a = ((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7]));
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
            if (lane == 0) chan[r] = a;
        }
    } else {
        // tile of 64 rows x 256 columns per CTA: a warp takes every 8th row, a lane 8 columns;
        // the warps' partial sums meet in shared memory, then one atomic per column
        __shared__ double s_col[8][256];
        const int64_t c = (int64_t)blockIdx.x * 256 + lane * 8;
        const int64_t r0 = (int64_t)blockIdx.y * 64;
        double acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (c < cols) {
            const int64_t r1 = min(rows, r0 + 64);
            for (int64_t r = r0 + warp; r < r1; r += 8)
                bf16x8_squares(__ldg(reinterpret_cast<const uint4 *>(grad + r * cols + c)), acc, odd);
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) s_col[warp][k * 32 + lane] = acc[k];
        __syncthreads();
        // thread tid owns column 8 * (tid >> 3) + (tid & 7) of the tile
        const int64_t cc = (int64_t)blockIdx.x * 256 + tid;
        if (cc < cols) {
            double a = 0.0;
#pragma unroll
            for (int w = 0; w < 8; ++w) a += s_col[w][(tid & 7) * 32 + (tid >> 3)];
            atomicAdd(chan + cc, a);
        }
    }
    if (nonfinite_flag != nullptr && odd) atomicOr(nonfinite_flag, 1);
}

// ---------------------------------------------------------------------------
// 3. scaling factors and the global norm
// ---------------------------------------------------------------------------
// One warp per channel: ||update_low|| / (||g_low|| + 1e-8) over the channel's `rank`
// entries (contiguous for "right", stride cols for "left"), then sum of ||G_ch||^2 * sf^2.
__global__ void __launch_bounds__(256)
apollo_scales_kernel(const float *upd, const float *g_low, const double *chan_g2, int64_t nch, int64_t rank,
                     int right, int front, float sqrt_scale, float *sf, double *total)
{
    __shared__ double s_part[8];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    double local = 0.0;
    for (int64_t ch = (int64_t)blockIdx.x * 8 + warp; ch < nch; ch += (int64_t)gridDim.x * 8) {
        double nu = 0.0, ng = 0.0;
        for (int64_t k = lane; k < rank; k += 32) {
            const int64_t idx = right ? ch * rank + k : k * nch + ch;
            const float u = upd[idx], g = g_low[idx];
            nu += (double)__fmul_rn(u, u);
            ng += (double)__fmul_rn(g, g);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            nu += __shfl_xor_sync(0xffffffffu, nu, o);
            ng += __shfl_xor_sync(0xffffffffu, ng, o);
        }
        if (lane == 0) {
            float s = __fdiv_rn(__double2float_rn(sqrt(nu)), __fadd_rn(__double2float_rn(sqrt(ng)), 1e-8f));   // optimizer.py:2964
            if (front) s = __fmul_rn(s, sqrt_scale);                       // optimizer.py:2969-2971
            sf[ch] = s;
            const float nG = __double2float_rn(sqrt(chan_g2[ch]));
            local += (double)__fmul_rn(__fmul_rn(nG, nG), __fmul_rn(s, s));   // optimizer.py:2975-2982
        }
    }
    if (lane == 0) s_part[warp] = local;
    __syncthreads();
    if (tid == 0) {
        double s = 0.0;
        for (int w = 0; w < 8; ++w) s += s_part[w];
        atomicAdd(total, s);
    }
}

// tensor-wide scaling (apollo_scale_type == "tensor", optimizer.py:2966, 2984-2988):
// sums[0..2] hold sum(update_low^2), sum(g_low^2), sum(G^2)
__global__ void __launch_bounds__(256)
apollo_tensor_sums_kernel(const float *upd, const float *g_low, int64_t nl, const double *chan_g2, int64_t nch, double *sums)
{
    __shared__ double s_part[3][8];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    double a = 0.0, b = 0.0, c = 0.0;
    for (int64_t i = (int64_t)blockIdx.x * 256 + tid; i < nl; i += (int64_t)gridDim.x * 256) {
        a += (double)__fmul_rn(upd[i], upd[i]);
        b += (double)__fmul_rn(g_low[i], g_low[i]);
    }
    for (int64_t i = (int64_t)blockIdx.x * 256 + tid; i < nch; i += (int64_t)gridDim.x * 256) c += chan_g2[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        a += __shfl_xor_sync(0xffffffffu, a, o);
        b += __shfl_xor_sync(0xffffffffu, b, o);
        c += __shfl_xor_sync(0xffffffffu, c, o);
    }
    if (lane == 0) { s_part[0][warp] = a; s_part[1][warp] = b; s_part[2][warp] = c; }
    __syncthreads();
    if (tid < 3) {
        double s = 0.0;
        for (int w = 0; w < 8; ++w) s += s_part[tid][w];
        atomicAdd(sums + tid, s);
    }
}

// ---------------------------------------------------------------------------
// 4. scalar chain of one tensor (one thread)
// ---------------------------------------------------------------------------
// alpha_decay: optional device pair (alpha_t, decay factor) from af8_param_scale (scale_parameter=True,
// optimizer.py:850-853, 3007-3013); NULL: in.alpha, and the decay travels as a kernel argument
__device__ __forceinline__ void apollo_finalize_one(const af8_apollo_scalars_in &in, const double *sums, float *sf_tensor,
                                                    float *fira_prev, af8_apollo_scalars *out, const float *alpha_decay = nullptr)
{
    float norm, s_tensor = 0.0f;
    if (in.scale_tensor) {
        s_tensor = __fdiv_rn(__double2float_rn(sqrt(sums[0])), __fadd_rn(__double2float_rn(sqrt(sums[1])), 1e-8f));
        if (in.scale_front) s_tensor = __fmul_rn(s_tensor, in.sqrt_scale);
        norm = __fmul_rn(__double2float_rn(sqrt(sums[2])), s_tensor);       // optimizer.py:2988
        *sf_tensor = s_tensor;
    } else {
        norm = __fsqrt_rn(__double2float_rn(sums[0]));                      // optimizer.py:2982
    }
    float fs = 1.0f;
    if (in.fira) {                                                          // optimizer.py:760-782, 2990-2994
        float nn = isfinite(norm) ? norm : 0.0f;
        if (in.fira_has_prev) {
            const float fp = *fira_prev;
            const bool reset = fp < 1e-6f;
            const float ratio = __fdiv_rn(nn, __fadd_rn(fp, 1e-8f));
            const float lim = __fdiv_rn(fmaxf(ratio, in.fira_margin1), in.fira_margin1);
            fs = reset ? 1.0f : __frcp_rn(lim);
            *fira_prev = reset ? nn : __fmul_rn(nn, fs);
        } else {
            *fira_prev = nn;
        }
    }
    float denom = 1.0f;
    if (in.d > 0.0f) {                                                      // optimizer.py:3003-3005
        const float x = __fdiv_rn(norm, in.clip_div);
        denom = (x >= 1.0f || isnan(x)) ? x : 1.0f;
    }
    const float alpha = alpha_decay ? alpha_decay[0] : in.alpha;
    float us = __fdiv_rn(-alpha, denom);                                    // optimizer.py:3013
    if (in.bc_mode == 1) us = __fmul_rn(us, in.bc);                         // optimizer.py:3021
    else if (in.bc_mode == 2) us = __fdiv_rn(us, in.bc);                    // optimizer.py:3023
    out->update_scale = us;
    out->fira = fs;
    out->norm = norm;
    out->decay = alpha_decay ? alpha_decay[1] : 1.0f;
}

__global__ void apollo_finalize_kernel(const float *alpha_decay, const af8_apollo_scalars_in in, const double *sums, float *sf_tensor,
                                       float *fira_prev, af8_apollo_scalars *out)
{
    apollo_finalize_one(in, sums, sf_tensor, fira_prev, out, alpha_decay);
}

// ---------------------------------------------------------------------------
// steps 3 and 4 for all tensors of a group in two launches (channel-wise scaling)
// ---------------------------------------------------------------------------
__device__ __forceinline__ int find_finish_tensor(const af8_apollo_finish_tensor *t, int n, int64_t unit)
{
    int lo = 0, hi = n - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (__ldg(&t[mid].first_unit) <= unit) lo = mid; else hi = mid - 1;
    }
    return lo;
}

// unit = 8 channels of one tensor.  Right case (a channel is a row of rank contiguous values): one
// warp per channel.  Left case (a channel is a column of the rank x cols array): the 8 channels of the
// unit are 32 contiguous bytes of every row, so 8 lanes take one row and the 32 groups of a CTA walk
// the rows together; the sums of a channel are then added over the groups in a fixed order.
__global__ void __launch_bounds__(256)
apollo_scales_multi_kernel(const af8_apollo_finish_tensor *__restrict__ T, int n, int64_t total_units)
{
    __shared__ double s_part[8];
    __shared__ double s_nu[8][8], s_ng[8][8];        // left case: [warp][channel of the unit]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    for (int64_t unit = blockIdx.x; unit < total_units; unit += gridDim.x) {
        const af8_apollo_finish_tensor *t = T + find_finish_tensor(T, n, unit);
        const int64_t rows = __ldg(&t->rows), cols = __ldg(&t->cols), rank = __ldg(&t->rank);
        const bool right = rows >= cols;
        const int64_t nch = right ? rows : cols;
        const int64_t ch0 = (unit - __ldg(&t->first_unit)) * 8;
        const int64_t ch = ch0 + warp;
        const float *upd = t->upd, *g_low = t->g_low;
        double local = 0.0;
        double nu = 0.0, ng = 0.0;
        if (right) {
            if (ch < nch) {
                for (int64_t k = lane; k < rank; k += 32) {
                    const int64_t idx = ch * rank + k;
                    const float u = upd[idx], g = g_low[idx];
                    nu += (double)__fmul_rn(u, u);
                    ng += (double)__fmul_rn(g, g);
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                nu += __shfl_xor_sync(0xffffffffu, nu, o);
                ng += __shfl_xor_sync(0xffffffffu, ng, o);
            }
        } else {
            const int64_t c = ch0 + (lane & 7);
            if (c < nch) {
                for (int64_t k = warp * 4 + (lane >> 3); k < rank; k += 32) {
                    const int64_t idx = k * nch + c;
                    const float u = upd[idx], g = g_low[idx];
                    nu += (double)__fmul_rn(u, u);
                    ng += (double)__fmul_rn(g, g);
                }
            }
            nu += __shfl_xor_sync(0xffffffffu, nu, 8);  ng += __shfl_xor_sync(0xffffffffu, ng, 8);
            nu += __shfl_xor_sync(0xffffffffu, nu, 16); ng += __shfl_xor_sync(0xffffffffu, ng, 16);
            if (lane < 8) { s_nu[warp][lane] = nu; s_ng[warp][lane] = ng; }
            __syncthreads();
            nu = ng = 0.0;
            if (lane == 0) {
#pragma unroll
                for (int w = 0; w < 8; ++w) { nu += s_nu[w][warp]; ng += s_ng[w][warp]; }
            }
        }
        if (lane == 0 && ch < nch) {
            float s = __fdiv_rn(__double2float_rn(sqrt(nu)), __fadd_rn(__double2float_rn(sqrt(ng)), 1e-8f));   // optimizer.py:2964
            if (__ldg(&t->in.scale_front)) s = __fmul_rn(s, __ldg(&t->in.sqrt_scale));                       // optimizer.py:2969-2971
            t->sf[ch] = s;
            const float nG = __double2float_rn(sqrt(t->chan_g2[ch]));
            local = (double)__fmul_rn(__fmul_rn(nG, nG), __fmul_rn(s, s));                                   // optimizer.py:2975-2982
        }
        __syncthreads();
        if (lane == 0) s_part[warp] = local;
        __syncthreads();
        if (tid == 0) {
            double s = 0.0;
            for (int w = 0; w < 8; ++w) s += s_part[w];
            atomicAdd(t->sums, s);
        }
    }
}

__global__ void apollo_finalize_multi_kernel(const af8_apollo_finish_tensor *T, int n)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        const af8_apollo_scalars_in in = T[i].in;
        apollo_finalize_one(in, T[i].sums, T[i].sf, T[i].fira_prev, T[i].out, T[i].alpha_decay);
    }
}

// ---------------------------------------------------------------------------
// 5. apply: p = p*decay + (us*G) * final_scale[channel]
// ---------------------------------------------------------------------------
// bf16 / fp16 parameters (optimizer.py:3043-3079).  Nearest rounding: the in-place ops of the fp32 rule,
// each rounded to the parameter's format (mul_ by the decay, then addcmul_ / add_).  Stochastic rounding:
// p*decay + (g * final_scale) * update_scale with every product and the sum rounded to binary32
// (optimizer.py:3061-3065), then one stochastic rounding with the counter generator.
struct ApolloLowp { int dtype, sr; uint64_t sr_base; };
__device__ __forceinline__ uint32_t apollo_lowp_bits(float p, float g, float f, float us, float decay, int has_decay,
                                                     int scale_tensor, const ApolloLowp &P, int64_t idx)
{
    if (!P.sr) {
        float x = has_decay ? param_round(__fmul_rn(p, decay), P.dtype) : p;
        x = scale_tensor ? __fmaf_rn(__fmul_rn(us, f), g, x) : __fmaf_rn(__fmul_rn(us, g), f, x);
        return P.dtype == AF8_BF16 ? f32_to_bf16_rn_bits(x) : f32_to_f16_rn_bits(x);
    }
    float x = has_decay ? __fmul_rn(p, decay) : p;
    x = __fadd_rn(x, __fmul_rn(__fmul_rn(g, f), us));
    const uint32_t r = sr_bits24(P.sr_base, (uint64_t)idx);
    return P.dtype == AF8_BF16 ? sr_bf16_bits(x, r) : sr_f16_bits(x, r);
}

__global__ void __launch_bounds__(256)
apollo_apply_lowp_kernel(void *param, const void *grad, int grad_dtype, int negate, const float *sf,
                         const af8_apollo_scalars *sc, int64_t rows, int64_t cols, int right, int scale_tensor,
                         int fira, int front, float sqrt_scale, float decay, int has_decay, const ApolloLowp P)
{
    const float us = sc->update_scale, fs = sc->fira;
    if (has_decay == 2) decay = sc->decay;               // computed on the device (parameter-scaled step)
    const int64_t n = rows * cols;
    for (int64_t idx = (int64_t)blockIdx.x * 256 + threadIdx.x; idx < n; idx += (int64_t)gridDim.x * 256) {
        const float g = apollo_grad(grad, grad_dtype, idx, negate);
        float f = scale_tensor ? sf[0] : (right ? sf[idx / cols] : sf[idx % cols]);
        if (fira) f = __fmul_rn(f, fs);                                  // optimizer.py:2994
        if (!front) f = __fmul_rn(f, sqrt_scale);                        // optimizer.py:3000
        const float pv = param_load(param, idx, P.dtype);
        static_cast<uint16_t *>(param)[idx] = (uint16_t)apollo_lowp_bits(pv, g, f, us, decay, has_decay, scale_tensor, P, idx);
    }
}

__global__ void __launch_bounds__(256)
apollo_apply_kernel(float *param, const void *grad, int grad_dtype, int negate, const float *sf,
                    const af8_apollo_scalars *sc, int64_t rows, int64_t cols, int right, int scale_tensor,
                    int fira, int front, float sqrt_scale, float decay, int has_decay, uint16_t *param_copy)
{
    const float us = sc->update_scale, fs = sc->fira;
    if (has_decay == 2) decay = sc->decay;               // computed on the device (parameter-scaled step)
    const int64_t n = rows * cols;
    for (int64_t i = ((int64_t)blockIdx.x * 256 + threadIdx.x) * 4; i < n; i += (int64_t)gridDim.x * 1024) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int64_t idx = i + e;
            if (idx >= n) break;
            const float g = apollo_grad(grad, grad_dtype, idx, negate);
            float f = scale_tensor ? sf[0] : (right ? sf[idx / cols] : sf[idx % cols]);
            if (fira) f = __fmul_rn(f, fs);                                  // optimizer.py:2994
            if (!front) f = __fmul_rn(f, sqrt_scale);                        // optimizer.py:3000
            float pv = param[idx];
            if (has_decay) pv = __fmul_rn(pv, decay);                        // optimizer.py:3075
            if (scale_tensor) pv = __fmaf_rn(__fmul_rn(us, f), g, pv);       // optimizer.py:3079
            else pv = __fmaf_rn(__fmul_rn(us, g), f, pv);                    // optimizer.py:3077
            param[idx] = pv;
            if (param_copy) param_copy[idx] = (uint16_t)f32_to_bf16_rn_bits(pv);   // bf16 compute copy
        }
    }
}

// 8 consecutive elements (group grp of the tensor) with 128-bit accesses (cols % 8 == 0, 16-byte aligned arrays,
// fewer than 2^34 elements); gpr: groups per row, st: the tensor-wise factor
// LOWP: the parameter is bf16 / fp16 (8 of them in one 128-bit word); P is ignored otherwise
template <bool BF16, bool LOWP>
__device__ __forceinline__ void apollo_apply_group(void *__restrict__ param_v, const void *__restrict__ grad, int negate,
                                                   const float *__restrict__ sf, float st, float us, float fs, uint32_t gpr, uint32_t grp,
                                                   int right, int scale_tensor, int fira, int front, float sqrt_scale, float decay,
                                                   int has_decay, const ApolloLowp &P, uint16_t *__restrict__ param_copy)
{
    float *const param = static_cast<float *>(param_v);
    const uint32_t row = grp / gpr, c8 = (grp - row * gpr) << 3;
    const int64_t idx = (int64_t)grp << 3;
    float g[8], f[8], pv[8];
    if (BF16) {
        const uint4 a = __ldcs(reinterpret_cast<const uint4 *>(static_cast<const uint16_t *>(grad) + idx));
        const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) { g[2 * k] = __uint_as_float(w[k] << 16); g[2 * k + 1] = __uint_as_float(w[k] & 0xffff0000u); }
    } else {
        const float4 a = __ldcs(reinterpret_cast<const float4 *>(static_cast<const float *>(grad) + idx));
        const float4 b = __ldcs(reinterpret_cast<const float4 *>(static_cast<const float *>(grad) + idx) + 1);
        g[0] = a.x; g[1] = a.y; g[2] = a.z; g[3] = a.w; g[4] = b.x; g[5] = b.y; g[6] = b.z; g[7] = b.w;
    }
    if (scale_tensor) {
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] = st;
    } else if (right) {
        const float fr = __ldg(sf + row);
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] = fr;
    } else {
        const float4 a = __ldg(reinterpret_cast<const float4 *>(sf + c8)), b = __ldg(reinterpret_cast<const float4 *>(sf + c8) + 1);
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    }
    if (LOWP) {
        uint4 *ph = reinterpret_cast<uint4 *>(static_cast<uint16_t *>(param_v) + idx);
        const uint4 pw = *ph;
        const uint32_t w[4] = {pw.x, pw.y, pw.z, pw.w};
        uint32_t o[4];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const uint32_t h = (e & 1) ? (w[e >> 1] >> 16) : (w[e >> 1] & 0xffffu);
            const float p = P.dtype == AF8_BF16 ? bf16_bits_to_f32(h) : f16_bits_to_f32(h);
            float ge = g[e];
            if (!isfinite(ge)) ge = 0.0f;
            if (negate) ge = -ge;
            float fe = f[e];
            if (fira) fe = __fmul_rn(fe, fs);
            if (!front) fe = __fmul_rn(fe, sqrt_scale);
            const uint32_t r = apollo_lowp_bits(p, ge, fe, us, decay, has_decay, scale_tensor, P, idx + e);
            if (e & 1) o[e >> 1] |= r << 16; else o[e >> 1] = r;
        }
        *ph = make_uint4(o[0], o[1], o[2], o[3]);
        return;
    }
    float4 *pp = reinterpret_cast<float4 *>(param + idx);
    const float4 p0 = pp[0], p1 = pp[1];
    pv[0] = p0.x; pv[1] = p0.y; pv[2] = p0.z; pv[3] = p0.w; pv[4] = p1.x; pv[5] = p1.y; pv[6] = p1.z; pv[7] = p1.w;
    // pairs of elements in packed binary32 arithmetic (each component rounds like the scalar operation)
    const float2 fs2 = bc2(fs), ss2 = bc2(sqrt_scale), us2 = bc2(us), decay2 = bc2(decay);
#pragma unroll
    for (int e = 0; e < 8; e += 2) {
        float2 ge = make_float2(isfinite(g[e]) ? g[e] : 0.0f, isfinite(g[e + 1]) ? g[e + 1] : 0.0f);   // optimizer.py:2606
        if (negate) ge = make_float2(-ge.x, -ge.y);
        float2 fe = make_float2(f[e], f[e + 1]);
        if (fira) fe = __fmul2_rn(fe, fs2);                              // optimizer.py:2994
        if (!front) fe = __fmul2_rn(fe, ss2);                            // optimizer.py:3000
        float2 x = make_float2(pv[e], pv[e + 1]);
        if (has_decay) x = __fmul2_rn(x, decay2);                        // optimizer.py:3075
        if (scale_tensor) x = __ffma2_rn(__fmul2_rn(us2, fe), ge, x);    // optimizer.py:3079
        else x = __ffma2_rn(__fmul2_rn(us2, ge), fe, x);                 // optimizer.py:3077
        pv[e] = x.x; pv[e + 1] = x.y;
    }
    pp[0] = make_float4(pv[0], pv[1], pv[2], pv[3]);
    pp[1] = make_float4(pv[4], pv[5], pv[6], pv[7]);
    if (param_copy) {                                                    // bf16 compute copy, round to nearest
        uint32_t o[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) o[k] = f32_to_bf16_rn_bits(pv[2 * k]) | (f32_to_bf16_rn_bits(pv[2 * k + 1]) << 16);
        *reinterpret_cast<uint4 *>(param_copy + idx) = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

// one tensor, grid-stride over its groups
template <bool BF16, bool LOWP>
__global__ void __launch_bounds__(256)
apollo_apply_vec_kernel(void *__restrict__ param_v, const void *__restrict__ grad, int negate, const float *__restrict__ sf,
                        const af8_apollo_scalars *__restrict__ sc, int64_t rows, int64_t cols, int right, int scale_tensor,
                        int fira, int front, float sqrt_scale, float decay, int has_decay, const ApolloLowp P,
                        uint16_t *__restrict__ param_copy)
{
    const float us = sc->update_scale, fs = sc->fira;
    if (has_decay == 2) decay = sc->decay;               // computed on the device (parameter-scaled step)
    const uint32_t gpr = (uint32_t)(cols >> 3);                 // groups of 8 per row
    const uint32_t ngroups = (uint32_t)((rows * cols) >> 3);
    const float st = scale_tensor ? __ldg(sf) : 0.0f;
    for (uint32_t grp = blockIdx.x * 256u + threadIdx.x; grp < ngroups; grp += gridDim.x * 256u)
        apollo_apply_group<BF16, LOWP>(param_v, grad, negate, sf, st, us, fs, gpr, grp, right, scale_tensor, fira, front, sqrt_scale,
                                       decay, has_decay, P, param_copy);
}

// all tensors of a table in one launch: a CTA takes chunks of 2048 elements (256 groups) in grid-stride order over
// the whole table and keeps the descriptor of its current tensor in shared memory
__device__ __forceinline__ int find_apply_chunk(const af8_apollo_apply_tensor *t, int n, int64_t id)
{
    int lo = 0, hi = n - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (__ldg(&t[mid].first_chunk) <= id) lo = mid; else hi = mid - 1;
    }
    return lo;
}
template <bool BF16, bool LOWP>
__global__ void __launch_bounds__(256)
apollo_apply_batch_kernel(const af8_apollo_apply_tensor *__restrict__ tensors, int n, int64_t total_chunks, int negate, int param_dtype)
{
    __shared__ af8_apollo_apply_tensor sT;
    static_assert(sizeof(af8_apollo_apply_tensor) % 4 == 0 && sizeof(af8_apollo_apply_tensor) / 4 <= 256, "descriptor copy");
    const int tid = threadIdx.x;
    int cur_t = -1;
    float us = 0.0f, fs = 0.0f, decay = 0.0f, st = 0.0f;
    uint32_t gpr = 1, ngroups = 0;
    int right = 0;
    ApolloLowp P{param_dtype, 0, 0};
    for (int64_t id = blockIdx.x; id < total_chunks; id += gridDim.x) {
        int t = cur_t;
        if (t < 0) t = find_apply_chunk(tensors, n, id);
        else while (t + 1 < n && __ldg(&tensors[t + 1].first_chunk) <= id) ++t;
        if (t != cur_t) {                                        // (uniform over the CTA)
            __syncthreads();                                     // every thread has left the previous tensor
            if (tid < (int)(sizeof(af8_apollo_apply_tensor) / 4))
                reinterpret_cast<uint32_t *>(&sT)[tid] = __ldg(reinterpret_cast<const uint32_t *>(tensors + t) + tid);
            cur_t = t;
            __syncthreads();
            us = sT.scalars->update_scale; fs = sT.scalars->fira;
            decay = sT.has_decay == 2 ? sT.scalars->decay : sT.decay;    // 2: computed on the device (parameter-scaled step)
            gpr = (uint32_t)(sT.cols >> 3);
            ngroups = (uint32_t)((sT.rows * sT.cols) >> 3);
            right = sT.rows >= sT.cols;
            st = sT.scale_tensor ? __ldg(sT.sf) : 0.0f;
            P.sr = sT.stochastic_round; P.sr_base = sT.sr_base;
        }
        const uint32_t grp = (uint32_t)(id - sT.first_chunk) * 256u + (uint32_t)tid;
        if (grp < ngroups)
            apollo_apply_group<BF16, LOWP>(sT.param, sT.grad, negate, sT.sf, st, us, fs, gpr, grp, right, sT.scale_tensor, sT.fira,
                                           sT.scale_front, sT.sqrt_scale, decay, sT.has_decay, P, static_cast<uint16_t *>(sT.param_copy));
    }
}

}  // namespace af8

namespace af8 {

constexpr int64_t APOLLO_WS_HEADER = 1024;    // flag at 0, the task of a single-tensor call at 128, planes after the header

inline int64_t apollo_workspace_bytes(int64_t rows, int64_t cols, int64_t rank)
{
    const int64_t k = rows >= cols ? cols : rows;              // the contracted dimension
    return APOLLO_WS_HEADER + 6 * k * rank;                    // header + three bf16 planes of Pt
}

inline int apollo_channel_norms(const void *grad, int32_t grad_dtype, int64_t rows, int64_t cols, double *chan_g2,
                                int *flag, cudaStream_t st)
{
    const int right = rows >= cols;
    const bool vec = grad_dtype == AF8_BF16 && cols % 8 == 0 && aligned16(grad);
    const uint16_t *gb = static_cast<const uint16_t *>(grad);
    if (right) {
        int64_t g = (rows + 7) / 8;
        if (g > 148 * 16) g = 148 * 16;
        if (vec) apollo_channel_sumsq_bf16_kernel<<<(int)g, 256, 0, st>>>(gb, rows, cols, 1, chan_g2, flag);
        else apollo_channel_sumsq_kernel<<<(int)g, 256, 0, st>>>(grad, grad_dtype, rows, cols, 1, chan_g2, flag);
    } else {
        AF8_CUDA_TRY(cudaMemsetAsync(chan_g2, 0, sizeof(double) * (size_t)cols, st));
        if (vec) {
            dim3 grid((unsigned)((cols + 255) / 256), (unsigned)((rows + 63) / 64));
            apollo_channel_sumsq_bf16_kernel<<<grid, 256, 0, st>>>(gb, rows, cols, 0, chan_g2, flag);
        } else {
            dim3 grid((unsigned)((cols + 255) / 256), (unsigned)((rows + 255) / 256));
            apollo_channel_sumsq_kernel<<<grid, 256, 0, st>>>(grad, grad_dtype, rows, cols, 0, chan_g2, flag);
        }
    }
    AF8_CUDA_TRY(cudaGetLastError());
    return AF8_OK;
}

inline bool apollo_tc_eligible(const af8_apollo_proj_desc &d, int32_t grad_dtype)
{
    return d.workspace != nullptr && grad_dtype == AF8_BF16 && d.rows % 8 == 0 && d.cols % 8 == 0 && d.rank % 8 == 0 &&
           d.workspace_bytes >= apollo_workspace_bytes(d.rows, d.cols, d.rank) &&
           (reinterpret_cast<uintptr_t>(d.workspace) & 255u) == 0 && aligned16(d.grad);
}

inline int apollo_check_desc(const af8_apollo_proj_desc &d, int32_t grad_dtype)
{
    if (!d.grad || !d.pt || !d.g_low || !d.chan_g2) return fail(AF8_ERR_INVALID, "af8_apollo_project: null argument");
    if (d.rows <= 0 || d.cols <= 0 || d.rank <= 0 || d.rows >= (1 << 30) || d.cols >= (1 << 30) || d.rank > 4096)
        return fail(AF8_ERR_INVALID, "af8_apollo_project: bad shape %lld x %lld, rank %lld", (long long)d.rows, (long long)d.cols, (long long)d.rank);
    if (grad_dtype != AF8_F32 && grad_dtype != AF8_BF16) return fail(AF8_ERR_UNSUPPORTED, "af8_apollo_project: gradients must be fp32 or bf16");
    return AF8_OK;
}

// correctly rounded dot products (SIMT, binary64 accumulation) + channel norms
inline int apollo_project_exact(const af8_apollo_proj_desc &d, int32_t grad_dtype, cudaStream_t st)
{
    if (d.rows >= d.cols) {
        dim3 grid((unsigned)((d.rank + PJ_TN - 1) / PJ_TN), (unsigned)((d.rows + PJ_TM - 1) / PJ_TM));
        apollo_project_kernel<true><<<grid, 256, 0, st>>>(d.grad, grad_dtype, d.negate, d.pt, d.g_low, (int)d.rows, (int)d.rank, (int)d.cols);
    } else {
        dim3 grid((unsigned)((d.cols + PJ_TN - 1) / PJ_TN), (unsigned)((d.rank + PJ_TM - 1) / PJ_TM));
        apollo_project_kernel<false><<<grid, 256, 0, st>>>(d.grad, grad_dtype, d.negate, d.pt, d.g_low, (int)d.rank, (int)d.cols, (int)d.rows);
    }
    AF8_CUDA_TRY(cudaGetLastError());
    return apollo_channel_norms(d.grad, grad_dtype, d.rows, d.cols, d.chan_g2, nullptr, st);
}

// tensor-core path, per tensor: bf16 planes of Pt (and, for the mma.sync kernel, the non-finite flag and the
// channel norms; the tcgen05 kernel produces both itself); fills the task
// true: this projection runs on tcgen05 (right case, rank a multiple of 16 up to 256)
// bytes of the transposed gradient that a left-case tensor needs on the tcgen05 path
inline int64_t apollo_transpose_need(const af8_apollo_proj_desc &d)
{
    return d.rows >= d.cols ? 0 : (d.rows * d.cols * 2 + 255) / 256 * 256;
}

// true: this projection runs on tcgen05 (rank a multiple of 16 up to 256; the left case also
// needs room for the transposed gradient, because the kernel takes both operands K-major)
inline bool apollo_umma_eligible(const af8_apollo_proj_desc &d, int64_t transpose_bytes)
{
    static const bool disabled = getenv("AF8_NO_UMMA") != nullptr;
    return !disabled && d.rank % 16 == 0 && d.rank >= 16 && d.rank <= UM_MAXN && apollo_transpose_need(d) <= transpose_bytes;
}

// gt: where the transposed gradient of a left-case tcgen05 task goes (nullptr otherwise)
inline int apollo_project_prepare(const af8_apollo_proj_desc &d, int32_t grad_dtype, ProjTask &task, int &next_tile, bool umma,
                                  cudaStream_t st, void *gt = nullptr)
{
    int *flag = static_cast<int *>(d.workspace);
    __nv_bfloat16 *planes = reinterpret_cast<__nv_bfloat16 *>(static_cast<char *>(d.workspace) + APOLLO_WS_HEADER);
    if (!umma) {       // the tcgen05 kernel finds non-finite entries and sums the channel norms itself
        AF8_CUDA_TRY(cudaMemsetAsync(flag, 0, sizeof(int), st));
        int rc = apollo_channel_norms(d.grad, grad_dtype, d.rows, d.cols, d.chan_g2, flag, st);
        if (rc) return rc;
    }
    const bool right = d.rows >= d.cols;
    const int64_t kdim = right ? d.cols : d.rows;
    const int64_t pn = kdim * d.rank;
    if (d.planes_valid) {
        // the planes of this pt are in the workspace already (same layout: it follows from the shape and the path)
    } else if (umma && right) {                              // planes transposed to [rank][cols]
        dim3 grid((unsigned)((kdim + 31) / 32), (unsigned)((d.rank + 31) / 32));
        apollo_split_transposed_kernel<<<grid, 256, 0, st>>>(d.pt, (int)kdim, (int)d.rank, planes);
    } else {                                                 // Pt is [rank][rows] already in the left case
        int64_t sg = (pn + 255) / 256;
        if (sg > 148 * 8) sg = 148 * 8;
        apollo_split_kernel<<<(int)sg, 256, 0, st>>>(d.pt, pn, planes);
    }
    AF8_CUDA_TRY(cudaGetLastError());
    task.grad = static_cast<const __nv_bfloat16 *>(d.grad);
    if (umma && !right) {                                    // the kernel reads G^T [cols][rows]
        dim3 grid((unsigned)((d.cols + 63) / 64), (unsigned)((d.rows + 63) / 64));
        apollo_transpose_bf16_kernel<<<grid, 256, 0, st>>>(static_cast<const uint16_t *>(d.grad), (int)d.rows, (int)d.cols,
                                                            static_cast<uint16_t *>(gt));
        AF8_CUDA_TRY(cudaGetLastError());
        task.grad = static_cast<const __nv_bfloat16 *>(gt);
    }
    task.planes = planes;
    task.out = d.g_low;
    task.nonfinite_flag = flag;
    task.M = (int)(right ? d.rows : d.cols);
    task.N = (int)d.rank;
    task.K = (int)kdim;
    task.right = right ? 1 : 0;
    task.negate = d.negate;
    task.first_tile = next_tile;
    task.tiles_n = umma ? 1 : (task.N + MM_BN - 1) / MM_BN;
    task.reserved = 0;
    const int64_t tiles = (int64_t)((task.M + MM_BM - 1) / MM_BM) * task.tiles_n;      // MM_BM == UM_BM
    if (tiles + next_tile >= (1ll << 31)) return fail(AF8_ERR_UNSUPPORTED, "af8_apollo_project: too many tiles in one launch");
    next_tile += (int)tiles;
    return AF8_OK;
}

// the two tensor maps of a tcgen05 task: G as [M][K] with boxes of 128 x 32, the planes as
// [3][N][K] with boxes of 3 x N x 32, both with the 64-byte swizzle and zero fill outside
inline int apollo_umma_maps(UmmaTask &u)
{
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return fail(AF8_ERR_CUDA, "cuTensorMapEncodeTiled is not available");
    const ProjTask &t = u.t;
    {
        const cuuint64_t dim[2] = {(cuuint64_t)t.K, (cuuint64_t)t.M}, stride[1] = {(cuuint64_t)t.K * 2};
        const cuuint32_t box[2] = {UM_BK, UM_BM}, es[2] = {1, 1};
        const CUresult r = enc(&u.map_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<__nv_bfloat16 *>(t.grad), dim, stride, box, es,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(AF8_ERR_CUDA, "cuTensorMapEncodeTiled (gradient) failed with %d", (int)r);
    }
    {
        const cuuint64_t dim[3] = {(cuuint64_t)t.K, (cuuint64_t)t.N, 3};
        const cuuint64_t stride[2] = {(cuuint64_t)t.K * 2, (cuuint64_t)t.K * t.N * 2};
        const cuuint32_t box[3] = {UM_BK, (cuuint32_t)t.N, 3}, es[3] = {1, 1, 1};
        const CUresult r = enc(&u.map_b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<__nv_bfloat16 *>(t.planes), dim, stride, box, es,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(AF8_ERR_CUDA, "cuTensorMapEncodeTiled (planes) failed with %d", (int)r);
    }
    return AF8_OK;
}

inline int apollo_project_launch_umma(const UmmaTask *dev_tasks, int n, int total_tiles, cudaStream_t st)
{
    static_assert(MM_BM == UM_BM, "tile height");
    auto kernel = apollo_project_umma_kernel;
    AF8_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)um_smem_bytes()));
    int grid = sm_count();
    if (grid > total_tiles) grid = total_tiles;
    kernel<<<grid, UM_THREADS, um_smem_bytes(), st>>>(dev_tasks, n, total_tiles);
    AF8_CUDA_TRY(cudaGetLastError());
    return AF8_OK;
}

inline int apollo_project_launch(const ProjTask *dev_tasks, int n, int total_tiles, cudaStream_t st)
{
    auto kernel = apollo_project_mma_kernel;
    AF8_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)mm_smem_bytes()));
    int grid = sm_count();                                   // one CTA per SM (shared memory and registers)
    if (grid > total_tiles) grid = total_tiles;
    kernel<<<grid, MM_THREADS, mm_smem_bytes(), st>>>(dev_tasks, n, total_tiles);
    AF8_CUDA_TRY(cudaGetLastError());
    return AF8_OK;
}

}  // namespace af8

extern "C" int af8_apollo_project(const void *grad, int32_t grad_dtype, int32_t negate, const float *pt,
                                  int64_t rows, int64_t cols, int64_t rank, float *g_low, double *chan_g2,
                                  void *stream)
{
    using namespace af8;
    af8_apollo_proj_desc d = {grad, pt, g_low, chan_g2, nullptr, 0, rows, cols, rank, negate, 0};
    int rc = apollo_check_desc(d, grad_dtype);
    if (rc) return rc;
    return apollo_project_exact(d, grad_dtype, static_cast<cudaStream_t>(stream));
}

extern "C" int64_t af8_apollo_project_workspace(int64_t rows, int64_t cols, int64_t rank)
{
    return af8::apollo_workspace_bytes(rows, cols, rank);
}

extern "C" int af8_apollo_project_ws(const void *grad, int32_t grad_dtype, int32_t negate, const float *pt,
                                     int64_t rows, int64_t cols, int64_t rank, float *g_low, double *chan_g2,
                                     void *workspace, int64_t workspace_bytes, void *stream)
{
    using namespace af8;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    af8_apollo_proj_desc d = {grad, pt, g_low, chan_g2, workspace, workspace_bytes, rows, cols, rank, negate, 0};
    int rc = apollo_check_desc(d, grad_dtype);
    if (rc) return rc;
    if (!apollo_tc_eligible(d, grad_dtype)) return apollo_project_exact(d, grad_dtype, st);
    ProjTask task;
    int tiles = 0;
    const bool umma = apollo_umma_eligible(d, 0);            // no room for a transposed gradient here: right case only
    rc = apollo_project_prepare(d, grad_dtype, task, tiles, umma, st);
    if (rc) return rc;
    // the task lives in the workspace between the flag and the planes; the copy from this
    // stack variable is staged by the runtime before the call returns (pageable source)
    char *slot = static_cast<char *>(workspace) + 128;
    if (umma) {
        UmmaTask u;
        memset(&u, 0, sizeof(u));
        u.t = task;
        u.chan_g2 = chan_g2;
        rc = apollo_umma_maps(u);
        if (rc) return rc;
        AF8_CUDA_TRY(cudaMemcpyAsync(slot, &u, sizeof(UmmaTask), cudaMemcpyHostToDevice, st));
        return apollo_project_launch_umma(reinterpret_cast<const UmmaTask *>(slot), 1, tiles, st);
    }
    AF8_CUDA_TRY(cudaMemcpyAsync(slot, &task, sizeof(ProjTask), cudaMemcpyHostToDevice, st));
    return apollo_project_launch(reinterpret_cast<const ProjTask *>(slot), 1, tiles, st);
}

extern "C" int32_t af8_apollo_project_task_bytes(void) { return (int32_t)sizeof(af8::UmmaTask); }

extern "C" int af8_apollo_project_batch(const af8_apollo_proj_desc *descs, int32_t n, int32_t grad_dtype,
                                        void *host_scratch, void *dev_scratch, void *transpose_scratch,
                                        int64_t transpose_bytes, void *stream)
{
    using namespace af8;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (!descs || n <= 0) return fail(AF8_ERR_INVALID, "af8_apollo_project_batch: null or empty table");
    if (!host_scratch || !dev_scratch) return fail(AF8_ERR_INVALID, "af8_apollo_project_batch: scratch buffers are required");
    // tensor-core tasks: the tcgen05 ones (with their tensor maps) first, then the mma.sync ones;
    // each kind is one launch.  The scratch holds n slots of sizeof(UmmaTask), 64-byte aligned.
    if ((reinterpret_cast<uintptr_t>(host_scratch) & 63u) || (reinterpret_cast<uintptr_t>(dev_scratch) & 63u))
        return fail(AF8_ERR_INVALID, "af8_apollo_project_batch: scratch buffers must be 64-byte aligned");
    if (transpose_bytes > 0 && (!transpose_scratch || (reinterpret_cast<uintptr_t>(transpose_scratch) & 255u)))
        return fail(AF8_ERR_INVALID, "af8_apollo_project_batch: transpose_scratch must be 256-byte aligned");
    int n_umma = 0, n_mma = 0;
    for (int i = 0; i < n; ++i) {
        int rc = apollo_check_desc(descs[i], grad_dtype);
        if (rc) return rc;
        if (apollo_tc_eligible(descs[i], grad_dtype)) { if (apollo_umma_eligible(descs[i], transpose_bytes)) ++n_umma; else ++n_mma; }
    }
    UmmaTask *host_u = static_cast<UmmaTask *>(host_scratch);
    const UmmaTask *dev_u = static_cast<const UmmaTask *>(dev_scratch);
    ProjTask *host_m = reinterpret_cast<ProjTask *>(host_u + n_umma);
    int iu = 0, im = 0, tiles_u = 0, tiles_m = 0;
    // The tcgen05 tasks go out in sub-batches: a new one starts when the transposed gradients
    // of the left-case tensors would no longer fit the scratch (stream order makes its reuse safe).
    int sub_start = 0;
    int64_t t_off = 0;
    auto launch_sub = [&](int end) -> int {
        if (end > sub_start) {
            AF8_CUDA_TRY(cudaMemcpyAsync(static_cast<char *>(dev_scratch) + sizeof(UmmaTask) * (size_t)sub_start, host_u + sub_start,
                                         sizeof(UmmaTask) * (size_t)(end - sub_start), cudaMemcpyHostToDevice, st));
            int rc = apollo_project_launch_umma(dev_u + sub_start, end - sub_start, tiles_u, st);
            if (rc) return rc;
        }
        sub_start = end;
        tiles_u = 0;
        t_off = 0;
        return AF8_OK;
    };
    for (int i = 0; i < n; ++i) {
        int rc;
        if (!apollo_tc_eligible(descs[i], grad_dtype)) {
            rc = apollo_project_exact(descs[i], grad_dtype, st);
        } else if (apollo_umma_eligible(descs[i], transpose_bytes)) {
            const int64_t need = apollo_transpose_need(descs[i]);
            if (need > 0 && t_off + need > transpose_bytes) {
                rc = launch_sub(iu);
                if (rc) return rc;
            }
            UmmaTask &u = host_u[iu++];
            memset(&u, 0, sizeof(u));
            rc = apollo_project_prepare(descs[i], grad_dtype, u.t, tiles_u, true, st, need > 0 ? static_cast<char *>(transpose_scratch) + t_off : nullptr);
            t_off += need;
            u.chan_g2 = descs[i].chan_g2;
            if (!rc) rc = apollo_umma_maps(u);
        } else {
            rc = apollo_project_prepare(descs[i], grad_dtype, host_m[im++], tiles_m, false, st);
        }
        if (rc) return rc;
    }
    int rc = launch_sub(iu);
    if (rc) return rc;
    if (n_mma) {
        ProjTask *dev_m = reinterpret_cast<ProjTask *>(static_cast<char *>(dev_scratch) + sizeof(UmmaTask) * (size_t)n_umma);
        AF8_CUDA_TRY(cudaMemcpyAsync(dev_m, host_m, sizeof(ProjTask) * (size_t)n_mma, cudaMemcpyHostToDevice, st));
        return apollo_project_launch(dev_m, n_mma, tiles_m, st);
    }
    return AF8_OK;
}

extern "C" int af8_apollo_scales(const float *upd, const float *g_low, const double *chan_g2, int64_t rows,
                                 int64_t cols, int64_t rank, const af8_apollo_scalars_in *in, float *sf,
                                 double *sums, float *fira_prev, af8_apollo_scalars *out, const float *alpha_decay,
                                 void *stream)
{
    using namespace af8;
    if (!upd || !g_low || !chan_g2 || !in || !sf || !sums || !out) return fail(AF8_ERR_INVALID, "af8_apollo_scales: null argument");
    if (in->fira && !fira_prev) return fail(AF8_ERR_INVALID, "af8_apollo_scales: the limiter needs fira_prev");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int right = rows >= cols;
    const int64_t nch = right ? rows : cols;
    AF8_CUDA_TRY(cudaMemsetAsync(sums, 0, sizeof(double) * 3, st));
    if (in->scale_tensor) {
        const int64_t nl = nch * rank;
        int64_t g = (nl + 255) / 256;
        if (g > 148 * 8) g = 148 * 8;
        apollo_tensor_sums_kernel<<<(int)g, 256, 0, st>>>(upd, g_low, nl, chan_g2, nch, sums);
    } else {
        int64_t g = (nch + 7) / 8;
        if (g > 148 * 16) g = 148 * 16;
        apollo_scales_kernel<<<(int)g, 256, 0, st>>>(upd, g_low, chan_g2, nch, rank, right, in->scale_front, in->sqrt_scale, sf, sums);
    }
    AF8_CUDA_TRY(cudaGetLastError());
    apollo_finalize_kernel<<<1, 1, 0, st>>>(alpha_decay, *in, sums, sf, fira_prev, out);
    AF8_CUDA_TRY(cudaGetLastError());
    return AF8_OK;
}

extern "C" int af8_apollo_scales_batch(const af8_apollo_finish_tensor *host_tensors, af8_apollo_finish_tensor *dev_tensors,
                                       int32_t n, int64_t total_units, void *stream)
{
    using namespace af8;
    if (!host_tensors || !dev_tensors || n <= 0) return fail(AF8_ERR_INVALID, "af8_apollo_scales_batch: null or empty table");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int64_t next = 0;
    char *run_begin = nullptr, *run_end = nullptr;
    for (int i = 0; i < n; ++i) {
        const af8_apollo_finish_tensor &t = host_tensors[i];
        if (!t.upd || !t.g_low || !t.chan_g2 || !t.sf || !t.sums || !t.out) return fail(AF8_ERR_INVALID, "af8_apollo_scales_batch: tensor %d: null pointer", i);
        if (t.in.scale_tensor) return fail(AF8_ERR_UNSUPPORTED, "af8_apollo_scales_batch: tensor-wise scaling takes af8_apollo_scales");
        if (t.in.fira && !t.fira_prev) return fail(AF8_ERR_INVALID, "af8_apollo_scales_batch: tensor %d: the limiter needs fira_prev", i);
        if (t.rows <= 0 || t.cols <= 0 || t.rank <= 0) return fail(AF8_ERR_INVALID, "af8_apollo_scales_batch: tensor %d: bad shape", i);
        if (t.first_unit != next) return fail(AF8_ERR_INVALID, "af8_apollo_scales_batch: tensor %d: first_unit %lld, expected %lld", i, (long long)t.first_unit, (long long)next);
        next += ((t.rows >= t.cols ? t.rows : t.cols) + 7) / 8;
        // clear the three accumulators of every tensor; neighbours in memory share one memset
        char *p = reinterpret_cast<char *>(t.sums);
        if (p == run_end) { run_end += 24; continue; }
        if (run_end != run_begin) AF8_CUDA_TRY(cudaMemsetAsync(run_begin, 0, (size_t)(run_end - run_begin), st));
        run_begin = p;
        run_end = p + 24;
    }
    if (run_end != run_begin) AF8_CUDA_TRY(cudaMemsetAsync(run_begin, 0, (size_t)(run_end - run_begin), st));
    if (next != total_units) return fail(AF8_ERR_INVALID, "af8_apollo_scales_batch: total_units is %lld but the table holds %lld", (long long)total_units, (long long)next);
    AF8_CUDA_TRY(cudaMemcpyAsync(dev_tensors, host_tensors, sizeof(af8_apollo_finish_tensor) * (size_t)n, cudaMemcpyHostToDevice, st));
    int64_t grid = (int64_t)sm_count() * 8;
    if (grid > total_units) grid = total_units;
    apollo_scales_multi_kernel<<<(int)grid, 256, 0, st>>>(dev_tensors, n, total_units);
    AF8_CUDA_TRY(cudaGetLastError());
    apollo_finalize_multi_kernel<<<(n + 127) / 128, 128, 0, st>>>(dev_tensors, n);
    AF8_CUDA_TRY(cudaGetLastError());
    return AF8_OK;
}

extern "C" int af8_apollo_apply(void *param, int32_t param_dtype, int32_t stochastic_round, uint64_t sr_base,
                                const void *grad, int32_t grad_dtype, int32_t negate, const float *sf,
                                const af8_apollo_scalars *scalars, int64_t rows, int64_t cols,
                                const af8_apollo_scalars_in *in, float decay, int32_t has_decay, void *param_copy,
                                void *stream)
{
    using namespace af8;
    if (!param || !grad || !sf || !scalars || !in) return fail(AF8_ERR_INVALID, "af8_apollo_apply: null argument");
    if (param_copy && (param_dtype != AF8_F32 || !aligned16(param_copy)))
        return fail(AF8_ERR_INVALID, "af8_apollo_apply: param_copy needs fp32 parameters and a 16-byte aligned address");
    uint16_t *const pc = static_cast<uint16_t *>(param_copy);
    if (grad_dtype != AF8_F32 && grad_dtype != AF8_BF16) return fail(AF8_ERR_UNSUPPORTED, "af8_apollo_apply: gradients must be fp32 or bf16");
    if (param_dtype != AF8_F32 && param_dtype != AF8_BF16 && param_dtype != AF8_F16) return fail(AF8_ERR_INVALID, "af8_apollo_apply: bad param_dtype %d", param_dtype);
    if (stochastic_round && param_dtype == AF8_F32) return fail(AF8_ERR_INVALID, "af8_apollo_apply: stochastic rounding applies to bf16 / fp16 parameters only");
    const bool lowp = param_dtype != AF8_F32;
    const ApolloLowp P{param_dtype, stochastic_round ? 1 : 0, sr_base};
    const int64_t n = rows * cols;
    const int right = rows >= cols ? 1 : 0;
    if (cols % 8 == 0 && n < ((int64_t)1 << 34) && aligned16(param) && aligned16(grad) && (right || in->scale_tensor || aligned16(sf))) {
        int64_t gv = (n / 8 + 255) / 256;
        if (gv > 148 * 8) gv = 148 * 8;
        cudaStream_t st = static_cast<cudaStream_t>(stream);
#define AF8_APOLLO_APPLY(B, L) apollo_apply_vec_kernel<B, L><<<(int)gv, 256, 0, st>>>(param, grad, negate, sf, scalars, rows, cols, right, \
        in->scale_tensor, in->fira, in->scale_front, in->sqrt_scale, decay, has_decay, P, pc)
        if (grad_dtype == AF8_BF16) { if (lowp) AF8_APOLLO_APPLY(true, true); else AF8_APOLLO_APPLY(true, false); }
        else { if (lowp) AF8_APOLLO_APPLY(false, true); else AF8_APOLLO_APPLY(false, false); }
#undef AF8_APOLLO_APPLY
        AF8_CUDA_TRY(cudaGetLastError());
        return AF8_OK;
    }
    if (lowp) {
        int64_t gl = (n + 255) / 256;
        if (gl > 148 * 16) gl = 148 * 16;
        apollo_apply_lowp_kernel<<<(int)gl, 256, 0, static_cast<cudaStream_t>(stream)>>>(
            param, grad, grad_dtype, negate, sf, scalars, rows, cols, right, in->scale_tensor, in->fira, in->scale_front,
            in->sqrt_scale, decay, has_decay, P);
        AF8_CUDA_TRY(cudaGetLastError());
        return AF8_OK;
    }
    int64_t g = (n + 1023) / 1024;
    if (g > 148 * 16) g = 148 * 16;
    apollo_apply_kernel<<<(int)g, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<float *>(param), grad, grad_dtype, negate, sf, scalars, rows, cols, rows >= cols ? 1 : 0,
        in->scale_tensor, in->fira, in->scale_front, in->sqrt_scale, decay, has_decay, pc);
    AF8_CUDA_TRY(cudaGetLastError());
    return AF8_OK;
}

extern "C" int af8_apollo_apply_batch(const af8_apollo_apply_tensor *host_tensors, af8_apollo_apply_tensor *dev_tensors,
                                      int32_t n, int64_t total_chunks, int32_t param_dtype, int32_t grad_dtype,
                                      int32_t negate, void *stream)
{
    using namespace af8;
    if (!host_tensors || !dev_tensors || n <= 0) return fail(AF8_ERR_INVALID, "af8_apollo_apply_batch: null table or n <= 0");
    if (grad_dtype != AF8_F32 && grad_dtype != AF8_BF16) return fail(AF8_ERR_UNSUPPORTED, "af8_apollo_apply_batch: gradients must be fp32 or bf16");
    if (param_dtype != AF8_F32 && param_dtype != AF8_BF16 && param_dtype != AF8_F16)
        return fail(AF8_ERR_INVALID, "af8_apollo_apply_batch: bad param_dtype %d", param_dtype);
    bool vec = true;
    int64_t chunks = 0;
    for (int i = 0; i < n; ++i) {
        const af8_apollo_apply_tensor &T = host_tensors[i];
        if (!T.param || !T.grad || !T.sf || !T.scalars || T.rows <= 0 || T.cols <= 0)
            return fail(AF8_ERR_INVALID, "af8_apollo_apply_batch: tensor %d: null pointer or empty shape", i);
        if (T.param_copy && (param_dtype != AF8_F32 || !aligned16(T.param_copy)))
            return fail(AF8_ERR_INVALID, "af8_apollo_apply_batch: tensor %d: param_copy needs fp32 parameters and a 16-byte aligned address", i);
        if (T.stochastic_round && param_dtype == AF8_F32)
            return fail(AF8_ERR_INVALID, "af8_apollo_apply_batch: stochastic rounding applies to bf16 / fp16 parameters only");
        if (T.has_decay < 0 || T.has_decay > 2) return fail(AF8_ERR_INVALID, "af8_apollo_apply_batch: tensor %d: bad has_decay %d", i, T.has_decay);
        if (T.first_chunk != chunks) return fail(AF8_ERR_INVALID, "af8_apollo_apply_batch: tensor %d: first_chunk out of sequence", i);
        const int64_t numel = T.rows * T.cols;
        chunks += (numel + 2047) / 2048;
        const bool right = T.rows >= T.cols;
        if (!(T.cols % 8 == 0 && numel < ((int64_t)1 << 34) && aligned16(T.param) && aligned16(T.grad) &&
              (right || T.scale_tensor || aligned16(T.sf))))
            vec = false;
    }
    if (chunks != total_chunks) return fail(AF8_ERR_INVALID, "af8_apollo_apply_batch: total_chunks does not match the table");
    if (!vec) {                                  // tensor by tensor
        for (int i = 0; i < n; ++i) {
            const af8_apollo_apply_tensor &T = host_tensors[i];
            af8_apollo_scalars_in in;
            memset(&in, 0, sizeof(in));
            in.scale_tensor = T.scale_tensor; in.fira = T.fira; in.scale_front = T.scale_front; in.sqrt_scale = T.sqrt_scale;
            const int rc = af8_apollo_apply(T.param, param_dtype, T.stochastic_round, T.sr_base, T.grad, grad_dtype, negate, T.sf,
                                            T.scalars, T.rows, T.cols, &in, T.decay, T.has_decay, T.param_copy, stream);
            if (rc != AF8_OK) return rc;
        }
        return AF8_OK;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    AF8_CUDA_TRY(cudaMemcpyAsync(dev_tensors, host_tensors, sizeof(af8_apollo_apply_tensor) * (size_t)n, cudaMemcpyHostToDevice, st));
    const bool lowp = param_dtype != AF8_F32;
    // one wave of resident CTAs, each walking the table in grid-stride order
#define AF8_APOLLO_APPLY_BATCH(B, L) do { \
        static int per_sm = 0; \
        if (per_sm == 0 && (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, apollo_apply_batch_kernel<B, L>, 256, 0) != cudaSuccess || per_sm <= 0)) \
            per_sm = 4; \
        const int64_t g = total_chunks < 148 * (int64_t)per_sm ? total_chunks : 148 * (int64_t)per_sm; \
        apollo_apply_batch_kernel<B, L><<<(int)g, 256, 0, st>>>(dev_tensors, n, total_chunks, negate, param_dtype); \
    } while (0)
    if (grad_dtype == AF8_BF16) { if (lowp) AF8_APOLLO_APPLY_BATCH(true, true); else AF8_APOLLO_APPLY_BATCH(true, false); }
    else { if (lowp) AF8_APOLLO_APPLY_BATCH(false, true); else AF8_APOLLO_APPLY_BATCH(false, false); }
#undef AF8_APOLLO_APPLY_BATCH
    AF8_CUDA_TRY(cudaGetLastError());
    return AF8_OK;
}
