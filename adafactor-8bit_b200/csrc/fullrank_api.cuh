// Host side of the full-rank step: argument validation, kernel selection and
// launch (af8_fullrank_step), and the per-tensor norm / Fira / clip finaliser
// (af8_norm_finalize).
#pragma once

#include "common.cuh"
#include "fullrank_fast.cuh"
#include "fullrank_generic.cuh"
#include "fullrank_stat.cuh"

namespace af8 {

// ---------------------------------------------------------------------------
// norm finaliser: one CTA per tensor
// ---------------------------------------------------------------------------
// Reduces the tensor's per-block partial sums in a fixed order in binary64,
// then evaluates on one thread what the reference computes with 0-d tensors:
// _compute_fira_scale (optimizer.py:760-782), the clip denominators of
// _apply_fira_pytorch / _safe_rms_denom (optimizer.py:805-806, 859-863) and
// -alpha/denom (optimizer.py:874); in pre_div_mode 1 the RMS clip of the
// momentum-only rule (optimizer.py:897-899).
__global__ void __launch_bounds__(256)
norm_finalize_kernel(const af8_norm_tensor *tensors, const void *block_sumsq, af8_dyn_scalars *dyn)
{
    __shared__ double s_acc[256];
    const af8_norm_tensor T = tensors[blockIdx.x];
    const int tid = threadIdx.x;
    double acc = 0.0;
    if (T.partials_f64) {
        const double *ps = static_cast<const double *>(block_sumsq);
        for (int64_t i = tid; i < T.n_blocks; i += 256) acc += ps[T.first_block + i];
    } else {
        const float *ps = static_cast<const float *>(block_sumsq);
        for (int64_t i = tid; i < T.n_blocks; i += 256) acc += (double)ps[T.first_block + i];
    }
    s_acc[tid] = acc;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) {
        if (tid < o) s_acc[tid] += s_acc[tid + o];
        __syncthreads();
    }
    if (tid != 0) return;

    const double total = T.n_blocks < 0 ? *reinterpret_cast<const double *>(static_cast<uintptr_t>(T.first_block)) : s_acc[0];
    float norm = __double2float_rn(sqrt(total));
    const float alpha = T.alpha_dev ? *T.alpha_dev : T.alpha;
    af8_dyn_scalars out = dyn[blockIdx.x];
    out.norm = norm;
    if (T.pre_div_mode == 1) {
        const float rms = __fdiv_rn(norm, T.sqrt_n);
        float cf = __fdiv_rn(rms, T.d);
        cf = (cf >= 1.0f || isnan(cf)) ? cf : 1.0f;
        out.pre_div = cf;
        out.step = -alpha;
        out.fira = 1.0f;
        out.zero = 0.0f;
        dyn[blockIdx.x] = out;
        return;
    }
    float fs = 1.0f;
    float zero = 0.0f;
    if (T.fira_prev != nullptr) {
        if (!isfinite(norm)) { zero = 1.0f; norm = 0.0f; }       // optimizer.py:798-800
        if (T.fira_has_prev) {
            const float fp = *T.fira_prev;
            const bool reset = fp < 1e-6f;                          // optimizer.py:774
            const float ratio = __fdiv_rn(norm, __fadd_rn(fp, 1e-8f));
            const float lim = __fdiv_rn(fmaxf(ratio, T.fira_margin1), T.fira_margin1);
            fs = reset ? 1.0f : __frcp_rn(lim);                     // optimizer.py:777
            *T.fira_prev = reset ? norm : __fmul_rn(norm, fs);      // optimizer.py:778
        } else {
            *T.fira_prev = norm;                                    // optimizer.py:780-781
        }
    }
    float denom = 1.0f;
    if (T.clip_div > 0.0f) {
        const float x = __fdiv_rn(norm, T.clip_div);
        denom = (x >= 1.0f || isnan(x)) ? x : 1.0f;
    }
    out.step = __fdiv_rn(-alpha, denom);
    out.fira = fs;
    out.zero = zero;
    if (T.pre_div_mode != 2) out.pre_div = 1.0f;
    dyn[blockIdx.x] = out;
}

// One CTA per tensor: the scalars of the one-step-lag variant (af8_lag_scalars).
__global__ void __launch_bounds__(256)
lag_scalars_kernel(const af8_lag_tensor *tensors, int phase, const void *block_sumsq, af8_dyn_scalars *dyn)
{
    __shared__ double s_acc[256];
    const af8_lag_tensor T = tensors[blockIdx.x];
    const int tid = threadIdx.x;
    if (phase == 0) {
        if (tid != 0) return;
        const float alpha = T.alpha_dev ? *T.alpha_dev : T.alpha;
        const float fs = (T.lag_fira_scale != nullptr && T.has_lag_fira) ? *T.lag_fira_scale : 1.0f;
        const float alpha_eff = __fmul_rn(alpha, fs);                                      // optimizer.py:1062
        const float pn = *T.prev_update_norm;
        const float denom = T.clip_div > 0.0f ? fmaxf(1.0f, __fdiv_rn(pn, T.clip_div)) : 1.0f;   // kernels.cu:652-653
        af8_dyn_scalars out = dyn[blockIdx.x];
        out.fira = 1.0f;
        out.zero = 0.0f;
        out.step = -__fdiv_rn(alpha_eff, denom);
        out.pre_div = 1.0f;
        dyn[blockIdx.x] = out;
        return;
    }
    double acc = 0.0;
    if (T.partials_f64) {
        const double *ps = static_cast<const double *>(block_sumsq);
        for (int64_t i = tid; i < T.n_blocks; i += 256) acc += ps[T.first_block + i];
    } else {
        const float *ps = static_cast<const float *>(block_sumsq);
        for (int64_t i = tid; i < T.n_blocks; i += 256) acc += (double)ps[T.first_block + i];
    }
    s_acc[tid] = acc;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) {
        if (tid < o) s_acc[tid] += s_acc[tid + o];
        __syncthreads();
    }
    if (tid != 0) return;
    const float raw = __double2float_rn(sqrt(s_acc[0]));
    *T.prev_update_norm = raw;                                                              // optimizer.py:1066-1067
    dyn[blockIdx.x].norm = raw;
    if (T.lag_fira_scale == nullptr || T.fira_prev == nullptr) return;
    const float norm = isfinite(raw) ? raw : 0.0f;                                           // optimizer.py:767-768
    float fs = 1.0f;
    if (T.fira_has_prev) {
        const float fp = *T.fira_prev;
        const bool reset = fp < 1e-6f;
        const float ratio = __fdiv_rn(norm, __fadd_rn(fp, 1e-8f));
        const float lim = __fdiv_rn(fmaxf(ratio, T.fira_margin1), T.fira_margin1);
        fs = reset ? 1.0f : __frcp_rn(lim);
        *T.fira_prev = reset ? norm : __fmul_rn(norm, fs);
    } else {
        *T.fira_prev = norm;
    }
    *T.lag_fira_scale = fs;                                                                 // optimizer.py:1069-1070
}

// ---------------------------------------------------------------------------
// launch helpers
// ---------------------------------------------------------------------------
template <typename K>
inline int persistent_grid(K kernel, int threads, size_t smem, int64_t total_blocks, int *grid_out)
{
    int per_sm = 0;
    AF8_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, smem));
    if (per_sm < 1) return fail(AF8_ERR_CUDA, "kernel does not fit on an SM (threads=%d smem=%zu)", threads, smem);
    int64_t g = (int64_t)per_sm * sm_count();
    if (g > total_blocks) g = total_blocks;
    *grid_out = (int)g;
    return AF8_OK;
}

template <typename GradT, typename ParamT, int MODE>
inline int launch_fast(const FullrankLaunch &L, cudaStream_t st)
{
    using Ring = FastRing<GradT, ParamT, MODE>;
    auto kernel = fullrank_fast_kernel<GradT, ParamT, MODE>;
    // the ring lives in dynamic shared memory (up to 48-60 KB per CTA): opt in and ask for
    // the large shared-memory carve-out
    AF8_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Ring::SMEM_BYTES));
    AF8_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                      (int)cudaSharedmemCarveoutMaxShared));
    int grid = 0;
    int rc = persistent_grid(kernel, FAST_THREADS, Ring::SMEM_BYTES, L.total_blocks, &grid);
    if (rc) return rc;
    kernel<<<grid, FAST_THREADS, Ring::SMEM_BYTES, st>>>(L);
    AF8_CUDA_TRY(cudaGetLastError());
    return AF8_OK;
}

template <typename GradT>
inline int launch_stat(const FullrankLaunch &L, cudaStream_t st)
{
    auto kernel = fullrank_stat_kernel<GradT>;
    int per_sm = 0;
    AF8_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, STAT_THREADS, 0));
    if (per_sm < 1) return fail(AF8_ERR_CUDA, "statistic kernel does not fit on an SM");
    const int64_t warps_per_cta = STAT_THREADS / 32;
    int64_t grid = (int64_t)per_sm * sm_count();
    const int64_t need = (L.total_blocks + warps_per_cta - 1) / warps_per_cta;
    if (grid > need) grid = need;
    kernel<<<(int)grid, STAT_THREADS, 0, st>>>(L);
    AF8_CUDA_TRY(cudaGetLastError());
    return AF8_OK;
}

template <typename GradT, int MODE>
inline int launch_generic(const FullrankLaunch &L, const GenericCfg &C, cudaStream_t st)
{
    const size_t smem = (size_t)2 * C.block * sizeof(float);
    auto kernel = fullrank_generic_kernel<GradT, MODE>;
    if (smem > 48 * 1024)
        AF8_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    int grid = 0;
    int rc = persistent_grid(kernel, GEN_THREADS, smem, L.total_blocks, &grid);
    if (rc) return rc;
    kernel<<<grid, GEN_THREADS, smem, st>>>(L, C);
    AF8_CUDA_TRY(cudaGetLastError());
    return AF8_OK;
}

// the general kernel in any mode
template <typename GradT>
inline int dispatch_generic(int mode, const FullrankLaunch &L, const GenericCfg &C, cudaStream_t st)
{
    switch (mode) {
    case AF8_MODE_NOCLIP: return launch_generic<GradT, AF8_MODE_NOCLIP>(L, C, st);
    case AF8_MODE_SUMSQ: return launch_generic<GradT, AF8_MODE_SUMSQ>(L, C, st);
    case AF8_MODE_APPLY: return launch_generic<GradT, AF8_MODE_APPLY>(L, C, st);
    case AF8_MODE_LAG: return launch_generic<GradT, AF8_MODE_LAG>(L, C, st);
    default: return launch_generic<GradT, AF8_MODE_SUMSQ_M>(L, C, st);
    }
}

// the specialised kernels (AdamW UF8/AL8 layout): statistic pass, or the update pass for ParamT
template <typename GradT, typename ParamT>
inline int dispatch_fast(int mode, const FullrankLaunch &L, cudaStream_t st)
{
    switch (mode) {
    case AF8_MODE_NOCLIP: return launch_fast<GradT, ParamT, AF8_MODE_NOCLIP>(L, st);
    case AF8_MODE_SUMSQ: return launch_stat<GradT>(L, st);
    case AF8_MODE_LAG: return launch_fast<GradT, ParamT, AF8_MODE_LAG>(L, st);
    default: return launch_fast<GradT, ParamT, AF8_MODE_APPLY>(L, st);
    }
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline int validate_fullrank_table(const af8_fullrank_cfg &c, const af8_fullrank_tensor *T, int n, int64_t total_blocks)
{
    int64_t next = 0;
    const bool no_v = c.v_fmt == AF8_V_NONE;
    const bool v_quant = c.v_fmt != AF8_V_FP32 && !no_v;
    const bool has_m = c.m_fmt != AF8_M_NONE;
    const bool m_quant = has_m && c.m_fmt != AF8_M_FP32;
    for (int i = 0; i < n; ++i) {
        const af8_fullrank_tensor &t = T[i];
        if (t.numel <= 0) return fail(AF8_ERR_INVALID, "tensor %d: numel must be positive", i);
        if (t.numel >= ((int64_t)1 << 38)) return fail(AF8_ERR_UNSUPPORTED, "tensor %d: more than 2^38 elements", i);   // 32-bit block indices
        if (t.first_block != next) return fail(AF8_ERR_INVALID, "tensor %d: first_block %lld, expected %lld", i, (long long)t.first_block, (long long)next);
        next += (t.numel + c.block - 1) / c.block;
        if (!t.param || !t.grad) return fail(AF8_ERR_INVALID, "tensor %d: null param or grad", i);
        if (!aligned16(t.param) || !aligned16(t.grad)) return fail(AF8_ERR_INVALID, "tensor %d: param and grad must be 16-byte aligned", i);
        if (t.param_copy && (c.param_dtype != AF8_F32 || !aligned16(t.param_copy)))
            return fail(AF8_ERR_INVALID, "tensor %d: param_copy needs fp32 parameters and a 16-byte aligned address", i);
        if (v_quant) {
            if (!t.v_q || !t.v_scale || !t.v_min_log) return fail(AF8_ERR_INVALID, "tensor %d: null quantised V state", i);
            if (!aligned16(t.v_q)) return fail(AF8_ERR_INVALID, "tensor %d: v_q must be 16-byte aligned", i);
        } else if (!no_v && !t.v_f32) {
            return fail(AF8_ERR_INVALID, "tensor %d: null fp32 V state", i);
        }
        if (no_v && has_m && !(t.v_keep > 0.0f)) return fail(AF8_ERR_INVALID, "tensor %d: the SGD mode needs v_keep = 1 - beta1 > 0", i);
        if (m_quant) {
            if (!t.m_q || !t.m_scale) return fail(AF8_ERR_INVALID, "tensor %d: null quantised M state", i);
            if (!aligned16(t.m_q)) return fail(AF8_ERR_INVALID, "tensor %d: m_q must be 16-byte aligned", i);
        } else if (has_m && !t.m_f32) {
            return fail(AF8_ERR_INVALID, "tensor %d: null fp32 M state", i);
        }
    }
    if (next != total_blocks) return fail(AF8_ERR_INVALID, "total_blocks is %lld but the table holds %lld blocks", (long long)total_blocks, (long long)next);
    return AF8_OK;
}

}  // namespace af8

extern "C" int af8_fullrank_step(const af8_fullrank_cfg *cfg, const af8_fullrank_tensor *host_tensors,
                                 af8_fullrank_tensor *dev_tensors, int32_t n_tensors, int64_t total_blocks,
                                 const af8_dyn_scalars *dyn, float *block_sumsq, void *stream)
{
    using namespace af8;
    if (!cfg || !dev_tensors) return fail(AF8_ERR_INVALID, "af8_fullrank_step: null cfg or table");
    if (n_tensors <= 0 || total_blocks <= 0) return fail(AF8_ERR_INVALID, "af8_fullrank_step: empty launch (n_tensors=%d, total_blocks=%lld)", n_tensors, (long long)total_blocks);
    const af8_fullrank_cfg &c = *cfg;
    if (c.param_dtype != AF8_F32 && c.param_dtype != AF8_BF16 && c.param_dtype != AF8_F16) return fail(AF8_ERR_INVALID, "af8_fullrank_step: bad param_dtype %d", c.param_dtype);
    if (c.grad_dtype != AF8_F32 && c.grad_dtype != AF8_BF16 && c.grad_dtype != AF8_F16) return fail(AF8_ERR_INVALID, "af8_fullrank_step: bad grad_dtype %d", c.grad_dtype);
    if (c.stochastic_round && c.param_dtype == AF8_F32) return fail(AF8_ERR_INVALID, "af8_fullrank_step: stochastic rounding applies to bf16 / fp16 parameters only");
    if (c.v_fmt != AF8_V_FP32 && c.v_fmt != AF8_V_AL8 && c.v_fmt != AF8_V_AL16 && c.v_fmt != AF8_V_NONE) return fail(AF8_ERR_INVALID, "af8_fullrank_step: bad v_fmt %d", c.v_fmt);
    if (c.m_fmt < AF8_M_NONE || c.m_fmt > AF8_M_FP32) return fail(AF8_ERR_INVALID, "af8_fullrank_step: bad m_fmt %d", c.m_fmt);
    if (c.block < 128 || c.block % 128 != 0) return fail(AF8_ERR_INVALID, "af8_fullrank_step: block must be a multiple of 128, >= 128 (got %d)", c.block);
    if (c.block > GEN_MAX_BLOCK) return fail(AF8_ERR_UNSUPPORTED, "af8_fullrank_step: block %d exceeds the supported maximum %d", c.block, GEN_MAX_BLOCK);
    const bool m_quant = c.m_fmt != AF8_M_NONE && c.m_fmt != AF8_M_FP32;
    if (m_quant && (c.m_block < 32 || c.m_block % 4 != 0 || c.block % c.m_block != 0))
        return fail(AF8_ERR_INVALID, "af8_fullrank_step: m_block must be a multiple of 4, >= 32 and divide block (got %d, block %d)", c.m_block, c.block);
    if (c.mode < AF8_MODE_NOCLIP || c.mode > AF8_MODE_LAG) return fail(AF8_ERR_INVALID, "af8_fullrank_step: bad mode %d", c.mode);
    if ((c.mode == AF8_MODE_APPLY || c.mode == AF8_MODE_SUMSQ_M || c.mode == AF8_MODE_LAG) && !dyn) return fail(AF8_ERR_INVALID, "af8_fullrank_step: this mode needs dyn");
    if ((c.mode == AF8_MODE_SUMSQ || c.mode == AF8_MODE_SUMSQ_M || c.mode == AF8_MODE_LAG) && !block_sumsq) return fail(AF8_ERR_INVALID, "af8_fullrank_step: this mode needs block_sumsq");
    if (c.mode == AF8_MODE_LAG && c.momentum_only) return fail(AF8_ERR_UNSUPPORTED, "af8_fullrank_step: the lag mode does not cover the momentum-only rule");
    if (c.mode == AF8_MODE_SUMSQ_M && !(c.momentum_only && c.m_fmt != AF8_M_NONE)) return fail(AF8_ERR_INVALID, "af8_fullrank_step: SUMSQ_M needs the momentum-only rule");
    if (c.momentum_only && c.use_adam_denom) return fail(AF8_ERR_INVALID, "af8_fullrank_step: momentum_only excludes the Adam denominator");

    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (host_tensors) {
        int rc = validate_fullrank_table(c, host_tensors, n_tensors, total_blocks);
        if (rc) return rc;
        AF8_CUDA_TRY(cudaMemcpyAsync(dev_tensors, host_tensors, sizeof(af8_fullrank_tensor) * (size_t)n_tensors, cudaMemcpyHostToDevice, st));
    }

    FullrankLaunch L;
    L.tensors = dev_tensors;
    L.dyn = dyn;
    L.block_sumsq = block_sumsq;
    L.total_blocks = total_blocks;
    L.n_tensors = n_tensors;
    L.negate_grad = c.negate_grad ? 1 : 0;
    L.v_floor = c.v_floor;
    L.param_dtype = c.param_dtype;
    L.sr = c.stochastic_round ? 1 : 0;
    GenericCfg C{c.v_fmt, c.m_fmt, c.block, c.m_block, c.use_adam_denom ? 1 : 0, c.momentum_only ? 1 : 0};

    const bool fast = c.v_fmt == AF8_V_AL8 && c.m_fmt == AF8_M_UF8 && c.block == FAST_VBLOCK &&
                      c.m_block == FAST_MBLOCK && c.use_adam_denom && !c.momentum_only &&
                      c.mode != AF8_MODE_SUMSQ_M;
    // specialised kernels: fp32 parameters with fp32 / bf16 gradients, bf16 parameters with bf16 gradients
    if (fast && c.param_dtype == AF8_F32 && c.grad_dtype == AF8_BF16) return dispatch_fast<bf16_tag, float>(c.mode, L, st);
    if (fast && c.param_dtype == AF8_F32 && c.grad_dtype == AF8_F32) return dispatch_fast<float, float>(c.mode, L, st);
    if (fast && c.param_dtype == AF8_BF16 && c.grad_dtype == AF8_BF16) return dispatch_fast<bf16_tag, bf16_tag>(c.mode, L, st);
    if (c.grad_dtype == AF8_BF16) return dispatch_generic<bf16_tag>(c.mode, L, C, st);
    if (c.grad_dtype == AF8_F16) return dispatch_generic<f16_tag>(c.mode, L, C, st);
    return dispatch_generic<float>(c.mode, L, C, st);
}

extern "C" int af8_fullrank_upload(const af8_fullrank_cfg *cfg, const af8_fullrank_tensor *host_tensors,
                                   af8_fullrank_tensor *dev_tensors, int32_t n_tensors, int64_t total_blocks,
                                   void *stream)
{
    using namespace af8;
    if (!cfg || !host_tensors || !dev_tensors) return fail(AF8_ERR_INVALID, "af8_fullrank_upload: null argument");
    if (n_tensors <= 0 || cfg->block < 128 || cfg->block % 128 != 0) return fail(AF8_ERR_INVALID, "af8_fullrank_upload: bad sizes");
    int rc = validate_fullrank_table(*cfg, host_tensors, n_tensors, total_blocks);
    if (rc) return rc;
    AF8_CUDA_TRY(cudaMemcpyAsync(dev_tensors, host_tensors, sizeof(af8_fullrank_tensor) * (size_t)n_tensors,
                                 cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream)));
    return AF8_OK;
}

extern "C" int af8_device_status(int32_t *status_out, void *stream)
{
    using namespace af8;
    if (!status_out) return fail(AF8_ERR_INVALID, "af8_device_status: null output");
    int v = 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    AF8_CUDA_TRY(cudaMemcpyFromSymbolAsync(&v, g_device_error, sizeof(int), 0, cudaMemcpyDeviceToHost, st));
    AF8_CUDA_TRY(cudaStreamSynchronize(st));
    *status_out = v;
    return AF8_OK;
}

namespace af8 {
// Self-test of the bounded wait: one thread arms an mbarrier for 64 bytes, copies 32 (that copy
// completes; nothing stays in flight) and waits with the given limit.  The phase can never complete,
// so the wait must give up after the limit and record the time-out exactly as the step kernels do.
__global__ void bounded_wait_selftest_kernel(const unsigned char *src, uint64_t limit_ns, int *gave_up)
{
    __shared__ __align__(128) unsigned char s_dst[64];
    __shared__ __align__(8) uint64_t s_bar;
    if (threadIdx.x != 0) return;
    mbar_init(&s_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_proxy_async();
    mbar_expect_tx(&s_bar, 64);
    bulk_g2s(s_dst, src, 32, &s_bar);
    const bool done = mbar_wait_bounded(&s_bar, 0, limit_ns);
    if (!done) atomicExch(&g_device_error, DEVERR_COPY_TIMEOUT);
    *gave_up = done ? 0 : 1;
    // the 32-byte copy has landed long before the limit ran out; give it a (bounded) moment anyway
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 20000ull) { }
}
}  // namespace af8

extern "C" int af8_selftest_bounded_wait(const void *src32, int64_t limit_ns, int32_t *gave_up_dev, void *stream)
{
    using namespace af8;
    if (!src32 || !gave_up_dev) return fail(AF8_ERR_INVALID, "af8_selftest_bounded_wait: null argument");
    if (!aligned16(src32)) return fail(AF8_ERR_INVALID, "af8_selftest_bounded_wait: the source must be 16-byte aligned");
    if (limit_ns <= 0 || limit_ns > 1000000000ll) return fail(AF8_ERR_INVALID, "af8_selftest_bounded_wait: the limit must be 1 ns .. 1 s");
    bounded_wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const unsigned char *>(src32), (uint64_t)limit_ns, gave_up_dev);
    AF8_CUDA_TRY(cudaGetLastError());
    return AF8_OK;
}

extern "C" int af8_device_status_clear(void *stream)
{
    using namespace af8;
    const int zero = 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    AF8_CUDA_TRY(cudaMemcpyToSymbolAsync(g_device_error, &zero, sizeof(int), 0, cudaMemcpyHostToDevice, st));
    AF8_CUDA_TRY(cudaStreamSynchronize(st));
    return AF8_OK;
}

extern "C" int af8_lag_scalars(const af8_lag_tensor *tensors, int32_t n_tensors, int32_t phase, const void *block_sumsq,
                               af8_dyn_scalars *dyn, void *stream)
{
    using namespace af8;
    if (!tensors || !dyn) return fail(AF8_ERR_INVALID, "af8_lag_scalars: null argument");
    if (n_tensors <= 0) return fail(AF8_ERR_INVALID, "af8_lag_scalars: n_tensors must be positive");
    if (phase != 0 && phase != 1) return fail(AF8_ERR_INVALID, "af8_lag_scalars: phase must be 0 or 1");
    if (phase == 1 && !block_sumsq) return fail(AF8_ERR_INVALID, "af8_lag_scalars: phase 1 needs block_sumsq");
    lag_scalars_kernel<<<n_tensors, 256, 0, static_cast<cudaStream_t>(stream)>>>(tensors, phase, block_sumsq, dyn);
    AF8_CUDA_TRY(cudaGetLastError());
    return AF8_OK;
}

extern "C" int af8_norm_finalize(const af8_norm_tensor *tensors, int32_t n_tensors, const void *block_sumsq,
                                 af8_dyn_scalars *dyn, void *stream)
{
    using namespace af8;
    if (!tensors || !block_sumsq || !dyn) return fail(AF8_ERR_INVALID, "af8_norm_finalize: null argument");
    if (n_tensors <= 0) return fail(AF8_ERR_INVALID, "af8_norm_finalize: n_tensors must be positive");
    norm_finalize_kernel<<<n_tensors, 256, 0, static_cast<cudaStream_t>(stream)>>>(tensors, block_sumsq, dyn);
    AF8_CUDA_TRY(cudaGetLastError());
    return AF8_OK;
}
