// af8_fullrank_limited_step_noalloc: the two-pass full-rank step (statistic
// pass -> norm / Fira / clip scalars -> apply pass) for ONE tensor, with every
// byte of working memory taken from an array that is part of the library image.
//
// Who this is for.  The regular entry points expect the caller to hand in
// device buffers for the descriptor table, the per-tensor scalars and the
// per-block partial sums.  Some callers have no way to produce such buffers at
// the moment they step: a binding written in a language runtime that can pass
// pointers it was given but has no device allocator of its own, or a training
// process whose framework allocator already owns all of the GPU's memory, so
// that a raw cudaMalloc issued on the side would fail or stall the device.
// Those callers still own the parameter, the gradient and the optimizer states
// (the inputs and outputs); this entry point supplies the rest.
//
// This file must stay in the same translation unit as the host code that
// resolves the array's address: `static __device__` gives the array internal
// linkage, and in host code its name is only a handle for the runtime, not a
// device address.
#pragma once

#include <mutex>

#include "common.cuh"
#include "fullrank_api.cuh"

namespace af8 {

constexpr size_t NOALLOC_BYTES = 1u << 20;          // 1 MiB per GPU that loads the library
constexpr size_t NOALLOC_TABLE_OFF = 0;             // one af8_fullrank_tensor (144 B)
constexpr size_t NOALLOC_DYN_OFF = 160;             // one af8_dyn_scalars (32 B)
constexpr size_t NOALLOC_NORM_OFF = 192;            // one af8_norm_tensor (64 B)
constexpr size_t NOALLOC_SUMSQ_OFF = 256;           // float partial sums, one per V block
constexpr int64_t NOALLOC_MAX_BLOCKS = (int64_t)((NOALLOC_BYTES - NOALLOC_SUMSQ_OFF) / sizeof(float));

static_assert(sizeof(af8_fullrank_tensor) == 144, "table row layout");
static_assert(sizeof(af8_norm_tensor) == 64, "norm row layout");
static_assert(sizeof(af8_dyn_scalars) == 32, "dyn layout");

// The working memory.  Every GPU on which the library's module gets loaded
// holds one copy until the process exits.
static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_BYTES];

// Writes the descriptor rows into the array and clears the record that the
// finaliser reads before it writes.  The rows arrive as kernel arguments, so no
// host-to-device copy (and no staging buffer behind it) is involved.  Device
// code may name the array directly.
__global__ void noalloc_setup_kernel(const af8_fullrank_tensor row, const af8_norm_tensor nrow)
{
    *reinterpret_cast<af8_fullrank_tensor *>(g_noalloc_scratch + NOALLOC_TABLE_OFF) = row;
    *reinterpret_cast<af8_norm_tensor *>(g_noalloc_scratch + NOALLOC_NORM_OFF) = nrow;
    af8_dyn_scalars z;
    z.step = 0.0f; z.fira = 0.0f; z.pre_div = 0.0f; z.zero = 0.0f; z.norm = 0.0f;
    z.reserved[0] = z.reserved[1] = z.reserved[2] = 0.0f;
    *reinterpret_cast<af8_dyn_scalars *>(g_noalloc_scratch + NOALLOC_DYN_OFF) = z;
}

constexpr int NOALLOC_MAX_DEVICES = 64;

// Device address of the array on the current device.  Resolved once per device,
// with that device current, through cudaGetSymbolAddress.
inline int noalloc_scratch_address(unsigned char **out)
{
    static std::mutex mu;
    static unsigned char *addr[NOALLOC_MAX_DEVICES] = {nullptr};
    int dev = -1;
    AF8_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= NOALLOC_MAX_DEVICES)
        return fail(AF8_ERR_UNSUPPORTED, "af8 noalloc: device ordinal %d is outside 0..%d", dev, NOALLOC_MAX_DEVICES - 1);
    std::lock_guard<std::mutex> lock(mu);
    if (addr[dev] == nullptr) {
        unsigned char *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void **>(&p), g_noalloc_scratch);
        if (e != cudaSuccess)
            return fail(AF8_ERR_CUDA, "af8 noalloc: cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
        if (p == nullptr || (reinterpret_cast<uintptr_t>(p) & 255u) != 0)
            return fail(AF8_ERR_CUDA, "af8 noalloc: unusable scratch address %p on device %d", (void *)p, dev);
        addr[dev] = p;
    }
    *out = addr[dev];
    return AF8_OK;
}

}  // namespace af8

extern "C" int64_t af8_noalloc_max_numel(int32_t block)
{
    if (block < 128 || block % 128 != 0) return 0;
    return af8::NOALLOC_MAX_BLOCKS * (int64_t)block;
}

extern "C" int af8_fullrank_limited_step_noalloc(const af8_fullrank_cfg *cfg, const af8_fullrank_tensor *host_tensor,
                                                 float clip_d, int32_t fira, float fira_margin1, float *fira_prev,
                                                 int32_t fira_has_prev, float *norm_out, void *stream)
{
    using namespace af8;
    if (!cfg || !host_tensor) return fail(AF8_ERR_INVALID, "af8_fullrank_limited_step_noalloc: null cfg or tensor");
    af8_fullrank_cfg c = *cfg;
    if (c.param_dtype != AF8_F32) return fail(AF8_ERR_UNSUPPORTED, "af8_fullrank_limited_step_noalloc: only fp32 parameters are supported");
    if (c.stochastic_round) return fail(AF8_ERR_INVALID, "af8_fullrank_limited_step_noalloc: stochastic rounding applies to bf16 / fp16 parameters only");
    if (c.grad_dtype != AF8_F32 && c.grad_dtype != AF8_BF16) return fail(AF8_ERR_UNSUPPORTED, "af8_fullrank_limited_step_noalloc: gradients must be fp32 or bf16");
    if (c.v_fmt != AF8_V_FP32 && c.v_fmt != AF8_V_AL8 && c.v_fmt != AF8_V_AL16) return fail(AF8_ERR_INVALID, "af8_fullrank_limited_step_noalloc: bad v_fmt %d", c.v_fmt);
    if (c.m_fmt < AF8_M_NONE || c.m_fmt > AF8_M_FP32) return fail(AF8_ERR_INVALID, "af8_fullrank_limited_step_noalloc: bad m_fmt %d", c.m_fmt);
    if (c.block < 128 || c.block % 128 != 0 || c.block > GEN_MAX_BLOCK) return fail(AF8_ERR_INVALID, "af8_fullrank_limited_step_noalloc: unsupported block %d", c.block);
    const bool m_quant = c.m_fmt != AF8_M_NONE && c.m_fmt != AF8_M_FP32;
    if (m_quant && (c.m_block < 32 || c.m_block % 4 != 0 || c.block % c.m_block != 0))
        return fail(AF8_ERR_INVALID, "af8_fullrank_limited_step_noalloc: bad m_block %d for block %d", c.m_block, c.block);
    if (c.momentum_only) return fail(AF8_ERR_UNSUPPORTED, "af8_fullrank_limited_step_noalloc: the momentum-only rule is not covered");
    if (!(clip_d >= 0.0f) || (fira && !(fira_margin1 >= 1.0f))) return fail(AF8_ERR_INVALID, "af8_fullrank_limited_step_noalloc: clip_d must be >= 0 and fira_margin1 >= 1");
    if (fira && !fira_prev) return fail(AF8_ERR_INVALID, "af8_fullrank_limited_step_noalloc: the limiter needs fira_prev");

    af8_fullrank_tensor row = *host_tensor;
    row.first_block = 0;
    if (row.numel <= 0) return fail(AF8_ERR_INVALID, "af8_fullrank_limited_step_noalloc: numel must be positive");
    const int64_t n_blocks = (row.numel + c.block - 1) / c.block;
    if (n_blocks > NOALLOC_MAX_BLOCKS)
        return fail(AF8_ERR_UNSUPPORTED,
                    "af8_fullrank_limited_step_noalloc: %lld elements need %lld partial sums, the built-in scratch holds %lld "
                    "(at most %lld elements at block %d); use af8_fullrank_step with caller-provided scratch",
                    (long long)row.numel, (long long)n_blocks, (long long)NOALLOC_MAX_BLOCKS,
                    (long long)(NOALLOC_MAX_BLOCKS * (int64_t)c.block), c.block);
    int rc = validate_fullrank_table(c, &row, 1, n_blocks);
    if (rc) return rc;

    unsigned char *scratch = nullptr;
    rc = noalloc_scratch_address(&scratch);
    if (rc) return rc;
    af8_fullrank_tensor *d_table = reinterpret_cast<af8_fullrank_tensor *>(scratch + NOALLOC_TABLE_OFF);
    af8_norm_tensor *d_norm = reinterpret_cast<af8_norm_tensor *>(scratch + NOALLOC_NORM_OFF);
    af8_dyn_scalars *d_dyn = reinterpret_cast<af8_dyn_scalars *>(scratch + NOALLOC_DYN_OFF);
    float *d_sumsq = reinterpret_cast<float *>(scratch + NOALLOC_SUMSQ_OFF);

    af8_norm_tensor nrow;
    nrow.first_block = 0;
    nrow.n_blocks = n_blocks;
    nrow.fira_prev = fira ? fira_prev : nullptr;
    nrow.fira_has_prev = fira_has_prev ? 1 : 0;
    nrow.pre_div_mode = 0;
    nrow.alpha = row.alpha;
    const double sqrt_n = sqrt((double)row.numel);
    nrow.sqrt_n = (float)sqrt_n;
    nrow.d = clip_d;
    nrow.clip_div = clip_d > 0.0f ? (float)(sqrt_n * (double)clip_d) : 0.0f;
    nrow.fira_margin1 = fira_margin1;
    nrow.partials_f64 = 0;
    nrow.alpha_dev = nullptr;

    cudaStream_t st = static_cast<cudaStream_t>(stream);
    noalloc_setup_kernel<<<1, 1, 0, st>>>(row, nrow);
    AF8_CUDA_TRY(cudaGetLastError());

    FullrankLaunch L;
    L.tensors = d_table;
    L.dyn = d_dyn;
    L.block_sumsq = d_sumsq;
    L.total_blocks = n_blocks;
    L.n_tensors = 1;
    L.negate_grad = c.negate_grad ? 1 : 0;
    L.v_floor = c.v_floor;
    L.param_dtype = AF8_F32;
    L.sr = 0;
    GenericCfg C{c.v_fmt, c.m_fmt, c.block, c.m_block, c.use_adam_denom ? 1 : 0, 0};
    const bool fast = c.v_fmt == AF8_V_AL8 && c.m_fmt == AF8_M_UF8 && c.block == FAST_VBLOCK &&
                      c.m_block == FAST_MBLOCK && c.use_adam_denom;
    const bool bf16 = c.grad_dtype == AF8_BF16;

    auto pass = [&](int mode) {
        if (fast) return bf16 ? dispatch_fast<bf16_tag, float>(mode, L, st) : dispatch_fast<float, float>(mode, L, st);
        return bf16 ? dispatch_generic<bf16_tag>(mode, L, C, st) : dispatch_generic<float>(mode, L, C, st);
    };
    rc = pass(AF8_MODE_SUMSQ);
    if (rc) return rc;
    norm_finalize_kernel<<<1, 256, 0, st>>>(d_norm, d_sumsq, d_dyn);
    AF8_CUDA_TRY(cudaGetLastError());
    rc = pass(AF8_MODE_APPLY);
    if (rc) return rc;
    if (norm_out)   // device-to-device: lets the caller read the measured norm later
        AF8_CUDA_TRY(cudaMemcpyAsync(norm_out, &d_dyn->norm, sizeof(float), cudaMemcpyDeviceToDevice, st));
    return AF8_OK;
}
