// Statistic pass of the AdamW UF8/AL8 configuration: per V block, the sum of squares of
// the update u = m_new / (sqrt(v_new) + eps) that the APPLY pass is going to use
// (first pass of the NORM -> APPLY structure, optimizer.py:1048-1077).
//
// Nothing computed here reaches a stored state: the sums only produce the norm that
// feeds the Fira limiter and the RMS clip, i.e. fp32 parameters with a 1e-5 tolerance.
// So, unlike the update kernel, this pass decodes the second moment with the hardware
// exp2 (relative error 2^-22) instead of the exact sequence.  One WARP owns one V block
// (8 sub-steps of 256 elements, 8 per lane), keeps its sum in registers and writes one
// float: no block-wide barrier, plain coalesced 64/128-bit loads.  The 256 possible values
// of the block's codes go into a per-warp shared-memory table first (8 exp2 per lane and
// block instead of 64; entry 0 is the exact zero), guarded by warp-level syncs only.
//
// Per element: 2 special-function operations (sqrt, reciprocal) plus 1/8 for the table; the
// special-function pipe was the busiest unit with the decode per element (3 operations,
// 70 % busy): the table took the pass from 1.04 to 0.93 ms on the TinyLlama set.
// (Replacing the reciprocal by rsqrt and a short series was measured slower.)
#pragma once

#include "common.cuh"
#include "fullrank_fast.cuh"

namespace af8 {

constexpr int STAT_THREADS = 256;
#ifndef AF8_STAT_MIN_CTAS
#define AF8_STAT_MIN_CTAS 5
#endif
#ifndef AF8_STAT_UNROLL
#define AF8_STAT_UNROLL 4
#endif
#ifndef AF8_STAT_PREFETCH
#define AF8_STAT_PREFETCH 0      /* measured on the TinyLlama set: 0.972 ms with the requests, 0.955 ms without */
#endif
#define AF8_PRAGMA_(x) _Pragma(#x)
#define AF8_UNROLL_(n) AF8_PRAGMA_(unroll n)

__device__ __forceinline__ float ex2_approx(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <typename GradT>
__device__ __forceinline__ void stat_load_g(const void *grad, int64_t off, float (&g)[8]);

template <>
__device__ __forceinline__ void stat_load_g<float>(const void *grad, int64_t off, float (&g)[8])
{
    const float4 *p = reinterpret_cast<const float4 *>(static_cast<const float *>(grad) + off);
    const float4 a = __ldcs(p), b = __ldcs(p + 1);
    g[0] = a.x; g[1] = a.y; g[2] = a.z; g[3] = a.w; g[4] = b.x; g[5] = b.y; g[6] = b.z; g[7] = b.w;
}

template <>
__device__ __forceinline__ void stat_load_g<bf16_tag>(const void *grad, int64_t off, float (&g)[8])
{
    const uint4 a = __ldcs(reinterpret_cast<const uint4 *>(static_cast<const uint16_t *>(grad) + off));
    g[0] = __uint_as_float(a.x << 16); g[1] = __uint_as_float(a.x & 0xffff0000u);
    g[2] = __uint_as_float(a.y << 16); g[3] = __uint_as_float(a.y & 0xffff0000u);
    g[4] = __uint_as_float(a.z << 16); g[5] = __uint_as_float(a.z & 0xffff0000u);
    g[6] = __uint_as_float(a.w << 16); g[7] = __uint_as_float(a.w & 0xffff0000u);
}

template <typename GradT>
__global__ void __launch_bounds__(STAT_THREADS, AF8_STAT_MIN_CTAS)
fullrank_stat_kernel(const FullrankLaunch L)
{
    // per-warp decode table of the block's 256 second-moment codes: 8 exponentials per lane and block
    // instead of 64 (the special-function pipe is the busiest unit of this pass); entry 0 is exact zero
    __shared__ float s_dec[STAT_THREADS / 32][256];
    const int lane = threadIdx.x & 31;
    float *const dec = s_dec[threadIdx.x >> 5];
    const int64_t warps = (int64_t)gridDim.x * (STAT_THREADS / 32);
    const int64_t w0 = (int64_t)blockIdx.x * (STAT_THREADS / 32) + (threadIdx.x >> 5);

    int t = -1;
    int64_t cur_first = 0, cur_end = 0, numel = 0;
    const void *grad = nullptr;
    const uint8_t *mq = nullptr, *vq = nullptr;
    const float *m_scale = nullptr, *v_scale = nullptr, *v_min_log = nullptr;
    float v_w = 0.f, m_w = 0.f, eps_d = 0.f, eps_g = 0.f, v_wm1 = 0.f, m_wm1 = 0.f;
    bool small_w = true;

    for (int64_t blk = w0; blk < L.total_blocks; blk += warps) {
        if (t < 0 || blk >= cur_end) {            // uniform over the warp
            if (t < 0) t = find_tensor(L.tensors, L.n_tensors, blk);
            else while (t + 1 < L.n_tensors && __ldg(&L.tensors[t + 1].first_block) <= blk) ++t;
            const af8_fullrank_tensor *T = L.tensors + t;
            numel = __ldg(&T->numel);
            cur_first = __ldg(&T->first_block);
            cur_end = cur_first + (numel + FAST_VBLOCK - 1) / FAST_VBLOCK;
            grad = T->grad;
            mq = T->m_q; vq = static_cast<const uint8_t *>(T->v_q);
            m_scale = T->m_scale; v_scale = T->v_scale; v_min_log = T->v_min_log;
            v_w = __ldg(&T->v_w); m_w = __ldg(&T->m_w);
            eps_d = __ldg(&T->eps_denom); eps_g = __ldg(&T->eps_gradsq);
            v_wm1 = __fsub_rn(v_w, 1.0f); m_wm1 = __fsub_rn(m_w, 1.0f);
            small_w = fabsf(v_w) < 0.5f && fabsf(m_w) < 0.5f;
        }
        const int64_t b = blk - cur_first;
        const int64_t base = b * FAST_VBLOCK;
        const int64_t rem = numel - base;
#if AF8_STAT_PREFETCH
        // Optional: ask L2 for this warp's next block (same tensor, a full block) while this one is worked
        // on: the gradient is 32 lines of 128 bytes (one per lane), the two code arrays 16 lines each.
        {
            const int64_t nb = b + warps;
            if (blk + warps < cur_end && (nb + 1) * FAST_VBLOCK <= numel) {
                const int64_t nbase = nb * FAST_VBLOCK;
                constexpr int GBYTES = std::is_same<GradT, float>::value ? 4 : 2;
                const char *gp = static_cast<const char *>(grad) + nbase * GBYTES;
                asm volatile("prefetch.global.L2 [%0];" ::"l"(gp + lane * 128));
                if (GBYTES == 4) asm volatile("prefetch.global.L2 [%0];" ::"l"(gp + 4096 + lane * 128));
                const uint8_t *cp = (lane < 16 ? mq : vq) + nbase + (lane & 15) * 128;
                asm volatile("prefetch.global.L2 [%0];" ::"l"(cp));
            }
        }
#endif
        // decode v = 2^((code-1)*scale/254 + min_log) as 2^(code*a + c)
        const float sc = __ldg(v_scale + b), ml = __ldg(v_min_log + b);
        const float a = sc * (1.0f / 254.0f);
        const float c = ml - a;
        float acc = 0.0f;

        if (rem >= FAST_VBLOCK && small_w) {
            __syncwarp();                                   // the previous block's look-ups are done
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const int code = lane + 32 * k;
                dec[code] = code ? ex2_approx(__fmaf_rn((float)code, a, c)) : 0.0f;
            }
            __syncwarp();
            const float2 wv2 = bc2(v_w), wm2 = bc2(m_w), ed2 = bc2(eps_d);
            float2 acc2 = make_float2(0.0f, 0.0f);
AF8_UNROLL_(AF8_STAT_UNROLL)
            for (int s = 0; s < FAST_VBLOCK / FAST_MBLOCK; ++s) {
                const int64_t off = base + s * FAST_MBLOCK + lane * 8;
                float g[8];
                stat_load_g<GradT>(grad, off, g);
                if (L.negate_grad) {                       // maximize (optimizer.py:1973-1974)
#pragma unroll
                    for (int j = 0; j < 8; ++j) g[j] = -g[j];
                }
                const uint2 mw = __ldcs(reinterpret_cast<const uint2 *>(mq + off));
                const uint2 vw = __ldcs(reinterpret_cast<const uint2 *>(vq + off));
                const float2 mc2 = bc2(__ldg(m_scale + b * (FAST_VBLOCK / FAST_MBLOCK) + s) * 0.0078125f);
#pragma unroll
                for (int j = 0; j < 8; j += 2) {
                    const uint32_t mword = (j < 4) ? mw.x : mw.y, vword = (j < 4) ? vw.x : vw.y;
                    const float2 gj = make_float2(g[j], g[j + 1]);
                    float2 g2 = __fmul2_rn(gj, gj);
                    if (eps_g != 0.0f) g2 = __fadd2_rn(g2, bc2(eps_g));
                    const float2 v_old = make_float2(dec[__byte_perm(vword, 0u, 0x4440u | (uint32_t)(j & 3))],
                                                     dec[__byte_perm(vword, 0u, 0x4440u | (uint32_t)((j + 1) & 3))]);
                    const float2 vj = __ffma2_rn(wv2, sub2(g2, v_old), v_old);
                    const float2 mb = make_float2(__uint_as_float(__byte_perm(mword, 0x4b000000u, 0x7540u | (uint32_t)(j & 3))),
                                                  __uint_as_float(__byte_perm(mword, 0x4b000000u, 0x7540u | (uint32_t)((j + 1) & 3))));
                    const float2 m_old = __fmul2_rn(__fadd2_rn(mb, bc2(-8388736.0f)), mc2);
                    const float2 mj = __ffma2_rn(wm2, sub2(gj, m_old), m_old);
                    const float2 den = __fadd2_rn(make_float2(sqrt_approx(vj.x), sqrt_approx(vj.y)), ed2);
                    const float2 u = __fmul2_rn(mj, make_float2(rcp_approx(den.x), rcp_approx(den.y)));
                    acc2 = __ffma2_rn(u, u, acc2);
                }
            }
            acc = __fadd_rn(acc2.x, acc2.y);
        } else {
            // tail block of a tensor, or EMA weights >= 0.5: element-wise with guards
            for (int64_t i = lane; i < FAST_VBLOCK; i += 32) {
                if (i >= rem) break;
                const int64_t e = base + i;
                float gj = GradLoad<GradT>::load1(grad, e);
                if (L.negate_grad) gj = -gj;
                const float g2 = __fadd_rn(__fmul_rn(gj, gj), eps_g);
                const uint32_t code = vq[e];
                const float v_old = code ? ex2_approx(__fmaf_rn((float)code, a, c)) : 0.0f;
                const float vj = lerp_t(v_old, g2, v_w);
                const float m_old = __fmul_rn((float)((int)mq[e] - 128), __ldg(m_scale + e / FAST_MBLOCK) * 0.0078125f);
                const float mj = lerp_t(m_old, gj, m_w);
                const float u = __fmul_rn(mj, rcp_approx(__fadd_rn(sqrt_approx(vj), eps_d)));
                acc = __fmaf_rn(u, u, acc);
            }
        }
        acc = warp_sum(acc);
        if (lane == 0) L.block_sumsq[blk] = acc;
    }
    (void)v_wm1; (void)m_wm1;
}

}  // namespace af8
