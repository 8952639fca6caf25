// APOLLO: the low-rank state rules beyond the plain Adam one (which runs through the
// full-rank kernel).  Input: the projected gradient g_low [LR x LC]; output: update_low of
// the same shape, from which the scaling kernels take the channel factors.
//   factorize           fp32 row / column factors of g_low^2 (optimizer.py:2688-2706), update
//                       m / (sqrt(v_est) + eps) or g / (...) (2753-2760);
//   factorize + CAME    U = g * inv_row * inv_col, clipped; momentum of U; confidence vectors
//                       from (U - M)^2 + eps; update M * inv_row_conf * inv_col_conf (2708-2750);
//   CAME                U = g * rsqrt(max(v_low, eps^2)), clipped; momentum of U; instability
//                       state res_low shaped like g_low; update M * rsqrt(max(res_low, eps^2))
//                       (2801-2903, pure-PyTorch branch 2869-2894).
// The projected gradient is rank/min(rows, cols) of the tensor (a few per cent), so these
// passes are written for clarity: element-wise kernels over fp32 work arrays between the
// stand-alone codec kernels, all on the caller's stream, no host synchronisation.
#pragma once

#include "common.cuh"
#include "codec.cuh"

namespace af8 {

enum RuleMode {
    RM_VINIT = 0,       // out = (g*g) * w                               optimizer.py:2771
    RM_VLERP,           // out = lerp(a, g*g, w)                          optimizer.py:2790, 2798
    RM_U_FROM_V,        // out = g * rsqrt(max(a, eps_sq)); sum of squares optimizer.py:2871
    RM_U_FACTOR,        // out = (g * ir[row]) * ic[col]; sum of squares   optimizer.py:2715
    RM_M_RES,           // u = a / cf; m = lerp(b, u, w); out = m; out2 = (u - m)^2 + eps_came   optimizer.py:2720-2726, 2876-2881
    RM_LERP,            // out = lerp(a, b, w)                            (fp32 states, vectors)
    RM_UPD_RES,         // out = a * rsqrt(max(b, eps_sq))                optimizer.py:2894
    RM_UPD_CONF,        // out = (a * ir[row]) * ic[col]                  optimizer.py:2750
    RM_UPD_FACT,        // out = a / (sqrt((rv[row] * cv[col]) / div) + eps)   optimizer.py:2705, 2758, 2760
    RM_COPY,            // out = a
};

struct RuleEw {
    const float *g, *a, *b;
    float *out, *out2;
    const float *ir, *ic;          // row / column vectors
    const double *scal;            // device scalars: [0] sum of squares of U, [1] mean of row_var_low
    double *sumsq;                 // RM_U_*: receives the sum of squares (atomic, cleared by the caller)
    int64_t n, LC;
    int mode;
    float w, eps_sq, eps_came, eps, d, sqrt_n;
};

__global__ void __launch_bounds__(256)
apollo_rule_ew_kernel(const RuleEw a)
{
    __shared__ double s_part[8];
    const int tid = threadIdx.x;
    double acc = 0.0;
    float cf = 1.0f, div = 1.0f;
    if (a.mode == RM_M_RES && a.d > 0.0f) {                  // clamp(rms(U) / d, min=1)
        const float rms = __fdiv_rn(__double2float_rn(sqrt(a.scal[0])), a.sqrt_n);
        cf = fmaxf(__fdiv_rn(rms, a.d), 1.0f);
    }
    if (a.mode == RM_UPD_FACT) div = fmaxf(__double2float_rn(a.scal[1]), a.eps);      // clamp_(min=apollo_eps)
    for (int64_t i = (int64_t)blockIdx.x * 256 + tid; i < a.n; i += (int64_t)gridDim.x * 256) {
        const int64_t row = i / a.LC, col = i - row * a.LC;
        switch (a.mode) {
        case RM_VINIT: { const float g = a.g[i]; a.out[i] = __fmul_rn(__fmul_rn(g, g), a.w); break; }
        case RM_VLERP: { const float g = a.g[i]; a.out[i] = lerp_t(a.a[i], __fmul_rn(g, g), a.w); break; }
        case RM_U_FROM_V: {
            const float u = __fmul_rn(a.g[i], rsqrt_t(fmaxf(a.a[i], a.eps_sq)));
            a.out[i] = u;
            acc += (double)__fmul_rn(u, u);
            break;
        }
        case RM_U_FACTOR: {
            const float u = __fmul_rn(__fmul_rn(a.g[i], a.ir[row]), a.ic[col]);
            a.out[i] = u;
            acc += (double)__fmul_rn(u, u);
            break;
        }
        case RM_M_RES: {
            const float u = a.d > 0.0f ? __fdiv_rn(a.a[i], cf) : a.a[i];
            const float m = lerp_t(a.b[i], u, a.w);
            const float df = __fsub_rn(u, m);
            a.out[i] = m;
            a.out2[i] = __fadd_rn(__fmul_rn(df, df), a.eps_came);
            break;
        }
        case RM_LERP: a.out[i] = lerp_t(a.a[i], a.b[i], a.w); break;
        case RM_UPD_RES: a.out[i] = __fmul_rn(a.a[i], rsqrt_t(fmaxf(a.b[i], a.eps_sq))); break;
        case RM_UPD_CONF: a.out[i] = __fmul_rn(__fmul_rn(a.a[i], a.ir[row]), a.ic[col]); break;
        case RM_UPD_FACT: {
            const float ve = __fdiv_rn(__fmul_rn(a.ir[row], a.ic[col]), div);
            a.out[i] = __fdiv_rn(a.a[i], __fadd_rn(__fsqrt_rn(ve), a.eps));
            break;
        }
        default: a.out[i] = a.a[i]; break;
        }
    }
    if (a.mode == RM_U_FROM_V || a.mode == RM_U_FACTOR) {
        if (a.sumsq == nullptr) return;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if ((tid & 31) == 0) s_part[tid >> 5] = acc;
        __syncthreads();
        if (tid == 0) {
            double s = 0.0;
            for (int w = 0; w < 8; ++w) s += s_part[w];
            atomicAdd(a.sumsq, s);
        }
    }
}

// row sums (one warp per row) and column sums (a thread per column over a band of 64 rows) of
// x[LR][LC], or of its squares; binary64 accumulators cleared by the caller
__global__ void __launch_bounds__(256)
apollo_rule_sums_kernel(const float *__restrict__ x, int64_t LR, int64_t LC, int square, double *row_sum, double *col_sum)
{
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int64_t bands = (LR + 63) / 64;
    for (int64_t band = blockIdx.x; band < bands; band += gridDim.x) {
        const int64_t r0 = band * 64, r1 = min(r0 + 64, LR);
        for (int64_t r = r0 + warp; r < r1; r += 8) {
            double s = 0.0;
            for (int64_t c = lane; c < LC; c += 32) {
                const float v = x[r * LC + c];
                s += (double)(square ? __fmul_rn(v, v) : v);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            if (lane == 0) row_sum[r] = s;
        }
        for (int64_t c = tid; c < LC; c += 256) {
            double s = 0.0;
            for (int64_t r = r0; r < r1; ++r) {
                const float v = x[r * LC + c];
                s += (double)(square ? __fmul_rn(v, v) : v);
            }
            atomicAdd(col_sum + c, s);
        }
    }
}

// Vector stages, one CTA.  stage 0 (factors): means of g_low^2 + floor into row_var_low /
// col_var_low (optimizer.py:2691-2700); scal[1] = mean(row_var_low); with CAME also the inverse
// factors (optimizer.py:818-821 with the mean clamped at the floor, 2711-2713).
// stage 1: means of the sums into rmean / cmean (the new values of the confidence vectors).
// stage 2: inverse factors of the confidence vectors (optimizer.py:2747-2748).
struct RuleVec {
    const double *row_sum, *col_sum;
    float *rv, *cv;                // stage 0: the fp32 factors; stage 2: the confidence vectors (read only)
    float *inv_r, *inv_c;          // out
    double *scal;
    int64_t LR, LC;
    int stage, first, want_inv;
    float w, keep;
};

__device__ __forceinline__ double cta_sum_f64(double x, double *s_red)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = x;
    __syncthreads();
    double s = 0.0;
    for (int w = 0; w < 8; ++w) s += s_red[w];
    return s;
}

__global__ void __launch_bounds__(256)
apollo_rule_vec_kernel(const RuleVec a)
{
    __shared__ double s_red[8];
    const int tid = threadIdx.x;
    const float floor_v = 1.17549435e-38f;
    if (a.stage == 0) {
        double part = 0.0;
        for (int64_t i = tid; i < a.LR; i += 256) {
            const float t = __fadd_rn(__double2float_rn(a.row_sum[i] / (double)a.LC), floor_v);
            const float v = a.first ? __fmul_rn(t, a.w) : __fmaf_rn(a.w, t, __fmul_rn(a.rv[i], a.keep));
            a.rv[i] = v;
            part += (double)v;
        }
        for (int64_t j = tid; j < a.LC; j += 256) {
            const float t = __fadd_rn(__double2float_rn(a.col_sum[j] / (double)a.LR), floor_v);
            a.cv[j] = a.first ? __fmul_rn(t, a.w) : __fmaf_rn(a.w, t, __fmul_rn(a.cv[j], a.keep));
        }
        const double mean = cta_sum_f64(part, s_red) / (double)a.LR;
        if (tid == 0) a.scal[1] = mean;
        if (a.want_inv) {
            const float rm = fmaxf(__double2float_rn(mean), floor_v);
            for (int64_t i = tid; i < a.LR; i += 256) a.inv_r[i] = rsqrt_t(__fdiv_rn(a.rv[i], rm));
            for (int64_t j = tid; j < a.LC; j += 256) a.inv_c[j] = rsqrt_t(a.cv[j]);
        }
    } else if (a.stage == 1) {
        for (int64_t i = tid; i < a.LR; i += 256) a.inv_r[i] = __double2float_rn(a.row_sum[i] / (double)a.LC);
        for (int64_t j = tid; j < a.LC; j += 256) a.inv_c[j] = __double2float_rn(a.col_sum[j] / (double)a.LR);
    } else {
        double part = 0.0;
        for (int64_t i = tid; i < a.LR; i += 256) part += (double)a.rv[i];
        const double mean = cta_sum_f64(part, s_red) / (double)a.LR;
        const float cm = fmaxf(__double2float_rn(mean), floor_v);
        for (int64_t i = tid; i < a.LR; i += 256) a.inv_r[i] = rsqrt_t(__fdiv_rn(a.rv[i], cm));
        for (int64_t j = tid; j < a.LC; j += 256) a.inv_c[j] = rsqrt_t(a.cv[j]);
    }
}

inline int64_t align64(int64_t x) { return (x + 63) / 64 * 64; }

// workspace layout (floats unless noted): U[n] | M[n] | T[n] | vec 6 x (LR + LC) | doubles: row[LR] col[LC] scal[8]
struct RuleWork {
    float *U, *M, *T, *rmean, *cmean, *inv_r, *inv_c, *crow, *ccol;
    double *row_sum, *col_sum, *scal;
};
inline int64_t rule_work_bytes(int64_t LR, int64_t LC)
{
    const int64_t n = LR * LC;
    return 4 * (3 * align64(n) + 3 * (align64(LR) + align64(LC))) + 8 * (align64(LR) + align64(LC) + 64) + 256;
}
inline RuleWork rule_work(void *base, int64_t LR, int64_t LC)
{
    const int64_t n = LR * LC;
    RuleWork w;
    float *f = static_cast<float *>(base);
    w.U = f; f += align64(n);
    w.M = f; f += align64(n);
    w.T = f; f += align64(n);
    w.rmean = f; f += align64(LR);
    w.cmean = f; f += align64(LC);
    w.inv_r = f; f += align64(LR);
    w.inv_c = f; f += align64(LC);
    w.crow = f; f += align64(LR);
    w.ccol = f; f += align64(LC);
    double *dd = reinterpret_cast<double *>(f);
    w.row_sum = dd; dd += align64(LR);
    w.col_sum = dd; dd += align64(LC);
    w.scal = dd;
    return w;
}

inline int rule_ew(cudaStream_t st, int mode, int64_t n, int64_t LC, const float *g, const float *a, const float *b, float *out,
                   float *out2 = nullptr, const float *ir = nullptr, const float *ic = nullptr, const double *scal = nullptr,
                   double *sumsq = nullptr, float w = 0.0f, const af8_apollo_rule *r = nullptr)
{
    RuleEw e{};
    e.g = g; e.a = a; e.b = b; e.out = out; e.out2 = out2; e.ir = ir; e.ic = ic; e.scal = scal; e.sumsq = sumsq;
    e.n = n; e.LC = LC; e.mode = mode; e.w = w;
    if (r) { e.eps_sq = r->eps_sq; e.eps_came = r->eps_came; e.eps = r->apollo_eps; e.d = r->d; e.sqrt_n = (float)sqrt((double)(r->lr_rows * r->lr_cols)); }
    apollo_rule_ew_kernel<<<grid_for(n, 1024), 256, 0, st>>>(e);
    AF8_CUDA_TRY(cudaGetLastError());
    return AF8_OK;
}

// deq -> lerp_ -> requant of an AL-coded state, or lerp_ of the fp32 state; `vals` receives the
// un-requantised values (optimizer.py:2735-2746)
inline int rule_state_ema(cudaStream_t st, const af8_apollo_rule_state &s, const float *new_vals, float w, int32_t block, float *vals)
{
    int rc;
    if (s.fmt == AF8_V_FP32) {
        rc = rule_ew(st, RM_LERP, s.n, 1, nullptr, s.f32, new_vals, s.f32, nullptr, nullptr, nullptr, nullptr, nullptr, w);
        if (rc) return rc;
        return rule_ew(st, RM_COPY, s.n, 1, nullptr, s.f32, nullptr, vals);
    }
    const int bits = s.fmt == AF8_V_AL8 ? 8 : 16;
    rc = af8_al_dequant(s.q, s.scale, s.min_log, s.n, block, bits, vals, st);
    if (rc) return rc;
    rc = rule_ew(st, RM_LERP, s.n, 1, nullptr, vals, new_vals, vals, nullptr, nullptr, nullptr, nullptr, nullptr, w);
    if (rc) return rc;
    return af8_al_quant(vals, s.n, block, bits, -126.0f, s.q, s.scale, s.min_log, st);
}

// the low-rank momentum of x (optimizer.py:714-729): M receives the un-requantised values
inline int rule_momentum(cudaStream_t st, const af8_apollo_rule &r, const float *x, int64_t n, float *M)
{
    int rc;
    if (r.m_fmt == AF8_M_FP32) {
        rc = rule_ew(st, RM_LERP, n, 1, nullptr, r.m_f32, x, r.m_f32, nullptr, nullptr, nullptr, nullptr, nullptr, r.m_w);
        if (rc) return rc;
        return rule_ew(st, RM_COPY, n, 1, nullptr, r.m_f32, nullptr, M);
    }
    rc = af8_m_dequant(r.m_q, r.m_scale, n, r.m_block, r.m_fmt, M, st);
    if (rc) return rc;
    rc = rule_ew(st, RM_LERP, n, 1, nullptr, M, x, M, nullptr, nullptr, nullptr, nullptr, nullptr, r.m_w);
    if (rc) return rc;
    return af8_m_quant(M, n, r.m_block, r.m_fmt, r.m_q, r.m_scale, st);
}

}  // namespace af8

extern "C" int64_t af8_apollo_rule_workspace(int64_t lr_rows, int64_t lr_cols)
{
    if (lr_rows <= 0 || lr_cols <= 0) return 0;
    return af8::rule_work_bytes(lr_rows, lr_cols);
}

extern "C" int af8_apollo_rule_step(const af8_apollo_rule *rp, void *stream)
{
    using namespace af8;
    if (!rp) return fail(AF8_ERR_INVALID, "af8_apollo_rule_step: null rule");
    const af8_apollo_rule &r = *rp;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int64_t LR = r.lr_rows, LC = r.lr_cols, n = LR * LC;
    if (!r.g_low || !r.upd || !r.work || LR <= 0 || LC <= 0) return fail(AF8_ERR_INVALID, "af8_apollo_rule_step: null or empty argument");
    if (reinterpret_cast<uintptr_t>(r.work) & 255u) return fail(AF8_ERR_INVALID, "af8_apollo_rule_step: work must be 256-byte aligned");
    if (r.work_bytes < rule_work_bytes(LR, LC)) return fail(AF8_ERR_INVALID, "af8_apollo_rule_step: work holds %lld bytes, %lld needed", (long long)r.work_bytes, (long long)rule_work_bytes(LR, LC));
    if (!r.factorize && !r.came) return fail(AF8_ERR_INVALID, "af8_apollo_rule_step: the plain rule runs through af8_fullrank_step");
    const bool has_m = r.m_fmt != AF8_M_NONE;
    if (has_m && (r.m_fmt == AF8_M_FP32 ? !r.m_f32 : (!r.m_q || !r.m_scale || r.m_block <= 0)))
        return fail(AF8_ERR_INVALID, "af8_apollo_rule_step: momentum state missing");
    if (r.came && !has_m) return fail(AF8_ERR_INVALID, "af8_apollo_rule_step: CAME needs a momentum (beta1)");
    const RuleWork w = rule_work(r.work, LR, LC);
    AF8_CUDA_TRY(cudaMemsetAsync(w.row_sum, 0, sizeof(double) * (size_t)(align64(LR) + align64(LC) + 8), st));
    int rc;
    const int sum_grid = (int)std::min<int64_t>((LR + 63) / 64, 148 * 8);
    if (r.factorize) {
        if (!r.row_var_low || !r.col_var_low) return fail(AF8_ERR_INVALID, "af8_apollo_rule_step: row_var_low / col_var_low missing");
        apollo_rule_sums_kernel<<<sum_grid, 256, 0, st>>>(r.g_low, LR, LC, 1, w.row_sum, w.col_sum);
        AF8_CUDA_TRY(cudaGetLastError());
        RuleVec v{};
        v.row_sum = w.row_sum; v.col_sum = w.col_sum; v.rv = r.row_var_low; v.cv = r.col_var_low; v.inv_r = w.inv_r; v.inv_c = w.inv_c;
        v.scal = w.scal; v.LR = LR; v.LC = LC; v.stage = 0; v.first = r.first_factor; v.want_inv = r.came; v.w = r.v_w; v.keep = r.v_keep;
        apollo_rule_vec_kernel<<<1, 256, 0, st>>>(v);
        AF8_CUDA_TRY(cudaGetLastError());
        if (!r.came) {
            const float *x = r.g_low;
            if (has_m) { rc = rule_momentum(st, r, r.g_low, n, w.M); if (rc) return rc; x = w.M; }
            return rule_ew(st, RM_UPD_FACT, n, LC, nullptr, x, nullptr, r.upd, nullptr, r.row_var_low, r.col_var_low, w.scal, nullptr, 0.0f, &r);
        }
        if (r.conf_row.n != LR || r.conf_col.n != LC) return fail(AF8_ERR_INVALID, "af8_apollo_rule_step: confidence vectors must hold lr_rows / lr_cols values");
        rc = rule_ew(st, RM_U_FACTOR, n, LC, r.g_low, nullptr, nullptr, w.U, nullptr, w.inv_r, w.inv_c, nullptr, r.d > 0.0f ? w.scal : nullptr, 0.0f, &r);
        if (rc) return rc;
    } else {
        // second moment of the projected gradient (optimizer.py:2763-2799); T = its un-requantised values
        const bool v_quant = r.v.fmt != AF8_V_FP32;
        if (r.v.n != n) return fail(AF8_ERR_INVALID, "af8_apollo_rule_step: v_low must hold lr_rows * lr_cols values");
        if (v_quant) {
            const int bits = r.v.fmt == AF8_V_AL8 ? 8 : 16;
            if (r.first_v) rc = rule_ew(st, RM_VINIT, n, LC, r.g_low, nullptr, nullptr, w.T, nullptr, nullptr, nullptr, nullptr, nullptr, r.v_w);
            else {
                rc = af8_al_dequant(r.v.q, r.v.scale, r.v.min_log, n, r.block, bits, w.T, st);
                if (!rc) rc = rule_ew(st, RM_VLERP, n, LC, r.g_low, w.T, nullptr, w.T, nullptr, nullptr, nullptr, nullptr, nullptr, r.v_w);
            }
            if (!rc) rc = af8_al_quant(w.T, n, r.block, bits, r.first_v ? -126.0f : r.v_floor_later, r.v.q, r.v.scale, r.v.min_log, st);
        } else {
            if (r.first_v) rc = rule_ew(st, RM_VINIT, n, LC, r.g_low, nullptr, nullptr, r.v.f32, nullptr, nullptr, nullptr, nullptr, nullptr, r.v_w);
            else rc = rule_ew(st, RM_VLERP, n, LC, r.g_low, r.v.f32, nullptr, r.v.f32, nullptr, nullptr, nullptr, nullptr, nullptr, r.v_w);
            if (!rc) rc = rule_ew(st, RM_COPY, n, 1, nullptr, r.v.f32, nullptr, w.T);
        }
        if (rc) return rc;
        rc = rule_ew(st, RM_U_FROM_V, n, LC, r.g_low, w.T, nullptr, w.U, nullptr, nullptr, nullptr, nullptr, r.d > 0.0f ? w.scal : nullptr, 0.0f, &r);
        if (rc) return rc;
    }
    // CAME: momentum of the clipped U, instability (U - M)^2 + eps
    if (r.m_fmt == AF8_M_FP32) rc = rule_ew(st, RM_COPY, n, 1, nullptr, r.m_f32, nullptr, w.M);
    else rc = af8_m_dequant(r.m_q, r.m_scale, n, r.m_block, r.m_fmt, w.M, st);
    if (rc) return rc;
    rc = rule_ew(st, RM_M_RES, n, LC, nullptr, w.U, w.M, w.M, w.U, nullptr, nullptr, w.scal, nullptr, r.m_w, &r);     // M = momentum, U = instability
    if (rc) return rc;
    if (r.m_fmt == AF8_M_FP32) rc = rule_ew(st, RM_COPY, n, 1, nullptr, w.M, nullptr, r.m_f32);
    else rc = af8_m_quant(w.M, n, r.m_block, r.m_fmt, r.m_q, r.m_scale, st);
    if (rc) return rc;
    if (r.factorize) {
        AF8_CUDA_TRY(cudaMemsetAsync(w.row_sum, 0, sizeof(double) * (size_t)(align64(LR) + align64(LC)), st));
        apollo_rule_sums_kernel<<<sum_grid, 256, 0, st>>>(w.U, LR, LC, 0, w.row_sum, w.col_sum);
        AF8_CUDA_TRY(cudaGetLastError());
        RuleVec v{};
        v.row_sum = w.row_sum; v.col_sum = w.col_sum; v.inv_r = w.rmean; v.inv_c = w.cmean; v.LR = LR; v.LC = LC; v.stage = 1;
        apollo_rule_vec_kernel<<<1, 256, 0, st>>>(v);
        AF8_CUDA_TRY(cudaGetLastError());
        rc = rule_state_ema(st, r.conf_row, w.rmean, r.c_w, r.block, w.crow);
        if (!rc) rc = rule_state_ema(st, r.conf_col, w.cmean, r.c_w, r.block, w.ccol);
        if (rc) return rc;
        RuleVec v2{};
        v2.rv = w.crow; v2.cv = w.ccol; v2.inv_r = w.inv_r; v2.inv_c = w.inv_c; v2.LR = LR; v2.LC = LC; v2.stage = 2;
        apollo_rule_vec_kernel<<<1, 256, 0, st>>>(v2);
        AF8_CUDA_TRY(cudaGetLastError());
        return rule_ew(st, RM_UPD_CONF, n, LC, nullptr, w.M, nullptr, r.upd, nullptr, w.inv_r, w.inv_c);
    }
    if (r.res.n != n) return fail(AF8_ERR_INVALID, "af8_apollo_rule_step: res_low must hold lr_rows * lr_cols values");
    rc = rule_state_ema(st, r.res, w.U, r.c_w, r.block, w.T);
    if (rc) return rc;
    if (r.res.fmt != AF8_V_FP32) {                           // the requantised values are what the update uses (optimizer.py:2889)
        rc = af8_al_dequant(r.res.q, r.res.scale, r.res.min_log, n, r.block, r.res.fmt == AF8_V_AL8 ? 8 : 16, w.T, st);
        if (rc) return rc;
    }
    return rule_ew(st, RM_UPD_RES, n, LC, nullptr, w.M, w.T, r.upd, nullptr, nullptr, nullptr, nullptr, nullptr, 0.0f, &r);
}
