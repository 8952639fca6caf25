// Stand-alone codecs between fp32 and the quantised state formats.  They are
// used for state migration, checkpoint conversion and tests; the fused step
// kernels carry their own inlined copies of the same per-element functions.
#pragma once

#include "common.cuh"
#include "fullrank_generic.cuh"

namespace af8 {

// _log_dequantize_nonneg (optimizer.py:328-353)
__global__ void __launch_bounds__(256)
al_dequant_kernel(const void *q, const float *scale, const float *min_log, int64_t n, int block, int bits, float *out)
{
    const float qm1 = bits == 16 ? 65534.0f : 254.0f;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t b = i / block;
        const uint32_t code = bits == 16 ? static_cast<const uint16_t *>(q)[i] : static_cast<const uint8_t *>(q)[i];
        out[i] = al_decode(code, __ldg(scale + b), __ldg(min_log + b), qm1);
    }
}

// _log_quantize_nonneg (optimizer.py:299-325): one CTA per block, elements
// beyond n are the zero padding.
__global__ void __launch_bounds__(256)
al_quant_kernel(const float *x, int64_t n, int block, int bits, float floor_log, void *q, float *scale, float *min_log)
{
    extern __shared__ float s_l[];
    __shared__ float s_red[2][8];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const float qm1 = bits == 16 ? 65534.0f : 254.0f;
    const int qmax = bits == 16 ? 65535 : 255;
    const int64_t nblocks = (n + block - 1) / block;
    for (int64_t b = blockIdx.x; b < nblocks; b += gridDim.x) {
        const int64_t base = b * block;
        float mn = INFINITY, mx = -INFINITY;
        __syncthreads();
        for (int i = tid; i < block; i += 256) {
            const float v = (base + i < n) ? x[base + i] : 0.0f;
            const float l = al_log2(v);
            if (v != 0.0f) mn = fminf(mn, l);
            mx = fmaxf(mx, l);
            s_l[i] = (v != 0.0f) ? l : -INFINITY;
        }
        mn = warp_min(mn);
        mx = warp_max(mx);
        if (lane == 0) { s_red[0][warp] = mn; s_red[1][warp] = mx; }
        __syncthreads();
        for (int w = 0; w < 8; ++w) { mn = fminf(mn, s_red[0][w]); mx = fmaxf(mx, s_red[1][w]); }
        float ml, sc;
        al_range(mn, mx, floor_log, ml, sc);
        for (int i = tid; i < block; i += 256) {
            const float l = s_l[i];
            const uint32_t code = (l == -INFINITY) ? 0u : al_encode(1.0f, l, ml, sc, qm1, qmax);
            if (bits == 16) static_cast<uint16_t *>(q)[base + i] = (uint16_t)code;
            else static_cast<uint8_t *>(q)[base + i] = (uint8_t)code;
        }
        if (tid == 0) { scale[b] = sc; min_log[b] = ml; }
    }
}

// _m_dequantize (optimizer.py:555-560)
__global__ void __launch_bounds__(256)
m_dequant_kernel(const uint8_t *q, const float *scale, int64_t n, int m_block, int fmt, float *out)
{
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        out[i] = m_decode(q, __ldg(scale + i / m_block), i, fmt);
}

// _m_quantize (optimizer.py:547-552): one warp per M block.
__global__ void __launch_bounds__(256)
m_quant_kernel(const float *m, int64_t n, int m_block, int fmt, uint8_t *q, float *scale)
{
    const int lane = threadIdx.x & 31;
    const int64_t nblocks = (n + m_block - 1) / m_block;
    const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
    const bool four_bit = fmt == AF8_M_UF4 || fmt == AF8_M_D4;
    for (int64_t b = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); b < nblocks; b += warps) {
        const int64_t base = b * m_block;
        float am = 0.0f;
        for (int i = lane; i < m_block; i += 32)
            if (base + i < n) am = fmaxf(am, fabsf(m[base + i]));
        am = fmaxf(warp_max(am), 1e-12f);
        if (four_bit) {
            for (int i = lane * 2; i < m_block; i += 64) {
                const float x0 = (base + i < n) ? m[base + i] : 0.0f;
                const float x1 = (base + i + 1 < n) ? m[base + i + 1] : 0.0f;
                q[(base + i) >> 1] = (uint8_t)((m_encode(x0, am, fmt) << 4) | m_encode(x1, am, fmt));
            }
        } else {
            for (int i = lane; i < m_block; i += 32) {
                const float x0 = (base + i < n) ? m[base + i] : 0.0f;
                q[base + i] = (uint8_t)m_encode(x0, am, fmt);
            }
        }
        if (lane == 0) scale[b] = am;
    }
}

inline int grid_for(int64_t work_items, int per_cta)
{
    int64_t g = (work_items + per_cta - 1) / per_cta;
    const int64_t cap = (int64_t)sm_count() * 8;
    if (g > cap) g = cap;
    if (g < 1) g = 1;
    return (int)g;
}

}  // namespace af8

extern "C" int af8_set_qmap(const float *host_map8, const float *host_map4, void *stream)
{
    using namespace af8;
    if (!host_map8 || !host_map4) return fail(AF8_ERR_INVALID, "af8_set_qmap: null codebook");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    AF8_CUDA_TRY(cudaMemcpyToSymbolAsync(c_qmap8, host_map8, sizeof(float) * 256, 0, cudaMemcpyHostToDevice, st));
    AF8_CUDA_TRY(cudaMemcpyToSymbolAsync(c_qmap4, host_map4, sizeof(float) * 16, 0, cudaMemcpyHostToDevice, st));
    return AF8_OK;
}

extern "C" int af8_al_dequant(const void *q, const float *scale, const float *min_log, int64_t numel,
                              int32_t block, int32_t bits, float *out, void *stream)
{
    using namespace af8;
    if (!q || !scale || !min_log || !out) return fail(AF8_ERR_INVALID, "af8_al_dequant: null argument");
    if (numel <= 0 || block <= 0 || (bits != 8 && bits != 16)) return fail(AF8_ERR_INVALID, "af8_al_dequant: bad size or bits");
    al_dequant_kernel<<<grid_for(numel, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(q, scale, min_log, numel, block, bits, out);
    AF8_CUDA_TRY(cudaGetLastError());
    return AF8_OK;
}

extern "C" int af8_al_quant(const float *x, int64_t numel, int32_t block, int32_t bits, float floor_log,
                            void *q, float *scale, float *min_log, void *stream)
{
    using namespace af8;
    if (!x || !q || !scale || !min_log) return fail(AF8_ERR_INVALID, "af8_al_quant: null argument");
    if (numel <= 0 || block <= 0 || (bits != 8 && bits != 16)) return fail(AF8_ERR_INVALID, "af8_al_quant: bad size or bits");
    if (block > 4 * GEN_MAX_BLOCK) return fail(AF8_ERR_UNSUPPORTED, "af8_al_quant: block %d too large", block);
    const size_t smem = sizeof(float) * (size_t)block;
    if (smem > 48 * 1024)
        AF8_CUDA_TRY(cudaFuncSetAttribute(al_quant_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int64_t nblocks = (numel + block - 1) / block;
    al_quant_kernel<<<grid_for(nblocks, 1), 256, smem, static_cast<cudaStream_t>(stream)>>>(x, numel, block, bits, floor_log, q, scale, min_log);
    AF8_CUDA_TRY(cudaGetLastError());
    return AF8_OK;
}

extern "C" int af8_m_dequant(const uint8_t *q, const float *scale, int64_t numel, int32_t m_block,
                             int32_t m_fmt, float *out, void *stream)
{
    using namespace af8;
    if (!q || !scale || !out) return fail(AF8_ERR_INVALID, "af8_m_dequant: null argument");
    if (numel <= 0 || m_block <= 0 || m_fmt < AF8_M_UF8 || m_fmt > AF8_M_D4) return fail(AF8_ERR_INVALID, "af8_m_dequant: bad size or format");
    m_dequant_kernel<<<grid_for(numel, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(q, scale, numel, m_block, m_fmt, out);
    AF8_CUDA_TRY(cudaGetLastError());
    return AF8_OK;
}

extern "C" int af8_m_quant(const float *m, int64_t numel, int32_t m_block, int32_t m_fmt, uint8_t *q,
                           float *scale, void *stream)
{
    using namespace af8;
    if (!m || !q || !scale) return fail(AF8_ERR_INVALID, "af8_m_quant: null argument");
    if (numel <= 0 || m_block < 2 || (m_block & 1) || m_fmt < AF8_M_UF8 || m_fmt > AF8_M_D4) return fail(AF8_ERR_INVALID, "af8_m_quant: bad size or format");
    const int64_t nblocks = (numel + m_block - 1) / m_block;
    m_quant_kernel<<<grid_for(nblocks, 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(m, numel, m_block, m_fmt, q, scale);
    AF8_CUDA_TRY(cudaGetLastError());
    return AF8_OK;
}
