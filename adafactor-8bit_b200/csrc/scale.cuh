// Parameter-scaled step size: alpha = max(RMS(p), eps2) * rho for every tensor
// of a launch table (_compute_alpha with scale_parameter=True,
// optimizer.py:850-853), followed by the bias-correction factor
// (optimizer.py:2020-2030) and the weight-decay factor (optimizer.py:2034-2039).
// The results are written straight into the `alpha` and `decay` fields of a
// device-resident tensor table, so the step kernels pick them up without a
// round trip to the host.
#pragma once

#include "common.cuh"

namespace af8 {

constexpr int SCALE_CHUNK = 4096;   // parameters per partial sum

struct ScaleLaunch {
    const af8_scale_tensor *tensors;
    float *block_sumsq;
    int64_t total_chunks;
    int32_t n_tensors;
};

__device__ __forceinline__ int find_scale_tensor(const af8_scale_tensor *tensors, int n, int64_t chunk)
{
    int lo = 0, hi = n - 1;
    while (lo < hi) {
        int mid = (lo + hi + 1) >> 1;
        if (__ldg(&tensors[mid].first_chunk) <= chunk) lo = mid; else hi = mid - 1;
    }
    return lo;
}

// one partial sum of squares per chunk of SCALE_CHUNK parameters
__global__ void __launch_bounds__(256)
param_sumsq_kernel(const ScaleLaunch L)
{
    __shared__ float s_red[8];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    for (int64_t chunk = blockIdx.x; chunk < L.total_chunks; chunk += gridDim.x) {
        const int t = find_scale_tensor(L.tensors, L.n_tensors, chunk);
        const void *p = L.tensors[t].param;
        const int pdt = L.tensors[t].param_dtype;
        const int64_t base = (chunk - L.tensors[t].first_chunk) * SCALE_CHUNK;
        const int64_t rem = L.tensors[t].numel - base;
        float acc = 0.0f;
        if (rem >= SCALE_CHUNK && pdt == AF8_F32) {
            const float4 *p4 = reinterpret_cast<const float4 *>(static_cast<const float *>(p) + base);
#pragma unroll
            for (int k = 0; k < SCALE_CHUNK / 4 / 256; ++k) {
                const float4 v = p4[tid + k * 256];
                acc = __fmaf_rn(v.x, v.x, acc); acc = __fmaf_rn(v.y, v.y, acc);
                acc = __fmaf_rn(v.z, v.z, acc); acc = __fmaf_rn(v.w, v.w, acc);
            }
        } else if (rem >= SCALE_CHUNK) {
            // bf16 / fp16 parameters enter the norm as binary32 (vector_norm(..., dtype=float32), optimizer.py:850-851)
            const uint2 *p2 = reinterpret_cast<const uint2 *>(static_cast<const uint16_t *>(p) + base);
#pragma unroll
            for (int k = 0; k < SCALE_CHUNK / 4 / 256; ++k) {
                const uint2 w = p2[tid + k * 256];
                float v[4];
                if (pdt == AF8_BF16) {
                    v[0] = __uint_as_float(w.x << 16); v[1] = __uint_as_float(w.x & 0xffff0000u);
                    v[2] = __uint_as_float(w.y << 16); v[3] = __uint_as_float(w.y & 0xffff0000u);
                } else {
                    v[0] = f16_bits_to_f32(w.x & 0xffffu); v[1] = f16_bits_to_f32(w.x >> 16);
                    v[2] = f16_bits_to_f32(w.y & 0xffffu); v[3] = f16_bits_to_f32(w.y >> 16);
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) acc = __fmaf_rn(v[j], v[j], acc);
            }
        } else {
            for (int i = tid; i < rem; i += 256) { const float v = param_load(p, base + i, pdt); acc = __fmaf_rn(v, v, acc); }
        }
        acc = warp_sum(acc);
        __syncthreads();
        if (lane == 0) s_red[warp] = acc;
        __syncthreads();
        if (tid == 0) {
            float s = 0.0f;
            for (int w = 0; w < 8; ++w) s = __fadd_rn(s, s_red[w]);
            L.block_sumsq[chunk] = s;
        }
    }
}

// one CTA per tensor: fixed-order binary64 reduction, then the scalar chain
__global__ void __launch_bounds__(256)
param_scale_finalize_kernel(const af8_scale_tensor *tensors, const float *block_sumsq,
                            uint8_t *table, int64_t stride, int64_t alpha_off, int64_t decay_off)
{
    __shared__ double s_acc[256];
    const af8_scale_tensor T = tensors[blockIdx.x];
    const int tid = threadIdx.x;
    const int64_t n_chunks = (T.numel + SCALE_CHUNK - 1) / SCALE_CHUNK;
    double acc = 0.0;
    for (int64_t i = tid; i < n_chunks; i += 256) acc += (double)block_sumsq[T.first_chunk + i];
    s_acc[tid] = acc;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) {
        if (tid < o) s_acc[tid] += s_acc[tid + o];
        __syncthreads();
    }
    if (tid != 0) return;
    const float norm = __double2float_rn(sqrt(T.total ? *T.total : s_acc[0]));
    const float rms = __fdiv_rn(norm, T.sqrt_n);                    // optimizer.py:851-852
    float alpha = __fmul_rn(fmaxf(rms, T.eps2), T.rho);             // optimizer.py:853
    if (T.bc_mode == 1) alpha = __fmul_rn(alpha, T.bc);             // optimizer.py:2026
    else if (T.bc_mode == 2) alpha = __fdiv_rn(alpha, T.bc);        // optimizer.py:2030
    float decay = 1.0f;
    if (T.weight_decay != 0.0f) {                                   // optimizer.py:2035-2039
        const float mult = T.scale_weight_decay ? alpha : T.rho;
        decay = __fsub_rn(1.0f, __fmul_rn(mult, T.weight_decay));
    }
    uint8_t *row = table + (int64_t)blockIdx.x * stride;
    *reinterpret_cast<float *>(row + alpha_off) = alpha;
    *reinterpret_cast<float *>(row + decay_off) = decay;
}

}  // namespace af8

namespace af8 {
inline int param_scale_layout_ok(int64_t table_stride, int64_t alpha_offset, int64_t decay_offset)
{
    return !(table_stride <= 0 || alpha_offset < 0 || decay_offset < 0 || alpha_offset + 4 > table_stride ||
             decay_offset + 4 > table_stride || (alpha_offset & 3) || (decay_offset & 3) || (table_stride & 3));
}
}  // namespace af8

extern "C" int af8_param_sumsq(const af8_scale_tensor *host_tensors, af8_scale_tensor *dev_tensors,
                               int32_t n_tensors, float *chunk_sumsq, void *stream)
{
    using namespace af8;
    if (!host_tensors || !dev_tensors || !chunk_sumsq) return fail(AF8_ERR_INVALID, "af8_param_sumsq: null argument");
    if (n_tensors <= 0) return fail(AF8_ERR_INVALID, "af8_param_sumsq: n_tensors must be positive");
    int64_t next = 0;
    for (int i = 0; i < n_tensors; ++i) {
        const af8_scale_tensor &t = host_tensors[i];
        if (!t.param || t.numel <= 0) return fail(AF8_ERR_INVALID, "af8_param_sumsq: tensor %d is empty", i);
        if (reinterpret_cast<uintptr_t>(t.param) & 15u) return fail(AF8_ERR_INVALID, "af8_param_sumsq: tensor %d: param must be 16-byte aligned", i);
        if (t.first_chunk != next) return fail(AF8_ERR_INVALID, "af8_param_sumsq: tensor %d: first_chunk %lld, expected %lld", i, (long long)t.first_chunk, (long long)next);
        next += (t.numel + SCALE_CHUNK - 1) / SCALE_CHUNK;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    AF8_CUDA_TRY(cudaMemcpyAsync(dev_tensors, host_tensors, sizeof(af8_scale_tensor) * (size_t)n_tensors, cudaMemcpyHostToDevice, st));
    ScaleLaunch L{dev_tensors, chunk_sumsq, next, n_tensors};
    int64_t grid = (int64_t)sm_count() * 8;
    if (grid > next) grid = next;
    param_sumsq_kernel<<<(int)grid, 256, 0, st>>>(L);
    AF8_CUDA_TRY(cudaGetLastError());
    return AF8_OK;
}

extern "C" int af8_param_scale_finish(const af8_scale_tensor *dev_tensors, int32_t n_tensors, const float *chunk_sumsq,
                                      void *dev_table, int64_t table_stride, int64_t alpha_offset, int64_t decay_offset,
                                      void *stream)
{
    using namespace af8;
    if (!dev_tensors || !chunk_sumsq || !dev_table) return fail(AF8_ERR_INVALID, "af8_param_scale_finish: null argument");
    if (n_tensors <= 0) return fail(AF8_ERR_INVALID, "af8_param_scale_finish: n_tensors must be positive");
    if (!param_scale_layout_ok(table_stride, alpha_offset, decay_offset)) return fail(AF8_ERR_INVALID, "af8_param_scale_finish: bad table layout");
    param_scale_finalize_kernel<<<n_tensors, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        dev_tensors, chunk_sumsq, static_cast<uint8_t *>(dev_table), table_stride, alpha_offset, decay_offset);
    AF8_CUDA_TRY(cudaGetLastError());
    return AF8_OK;
}

extern "C" int af8_param_scale(const af8_scale_tensor *host_tensors, af8_scale_tensor *dev_tensors,
                               int32_t n_tensors, float *chunk_sumsq, void *dev_table, int64_t table_stride,
                               int64_t alpha_offset, int64_t decay_offset, void *stream)
{
    using namespace af8;
    if (!dev_table) return fail(AF8_ERR_INVALID, "af8_param_scale: null argument");
    if (!param_scale_layout_ok(table_stride, alpha_offset, decay_offset)) return fail(AF8_ERR_INVALID, "af8_param_scale: bad table layout");
    int rc = af8_param_sumsq(host_tensors, dev_tensors, n_tensors, chunk_sumsq, stream);
    if (rc) return rc;
    return af8_param_scale_finish(dev_tensors, n_tensors, chunk_sumsq, dev_table, table_stride, alpha_offset, decay_offset, stream);
}

extern "C" int af8_scale_chunk(void) { return af8::SCALE_CHUNK; }
