// Full-rank fused step, specialised kernel: AdamW-style update with UF8
// momentum (M block 256) and AL8 second moment (V block 2048), fp32
// parameters, fp32 or bf16 gradients.
//
// Reference semantics: _update_param_8bit full-rank branch with the Adam
// denominator (optimizer.py:2115-2123), _fallback_1d_update
// (optimizer.py:903-910), _m_ema_pytorch (optimizer.py:690-700), the AL codec
// (optimizer.py:299-353) and the UF8 codec (optimizer.py:504-532).
//
// Work decomposition.  The launch covers a table of tensors; the unit of work
// is one V block (2048 consecutive elements of one tensor).  A persistent grid
// walks the flat block space with a grid stride.  One CTA of 256 threads owns a
// block; thread t owns elements [8t, 8t+8), so warp w owns exactly M block w of
// the V block and the momentum absmax is a pure warp reduction.  All global
// accesses of full blocks are 64- or 128-bit wide and contiguous across a warp.
// Everything a thread needs between the load and the requantisation stays in
// registers; shared memory only holds the 256-entry AL8 decode table of the
// block, the tensor descriptor and the cross-warp extrema.
#pragma once

#include "common.cuh"

namespace af8 {

constexpr int FAST_VBLOCK = 2048;
constexpr int FAST_MBLOCK = 256;
constexpr int FAST_THREADS = 256;
constexpr int FAST_EPT = 8;  // elements per thread

struct FullrankLaunch {
    const af8_fullrank_tensor *tensors;
    const af8_dyn_scalars *dyn;
    float *block_sumsq;
    int64_t total_blocks;
    int32_t n_tensors;
    int32_t negate_grad;
    float v_floor;
};

// Index of the tensor that owns flat block `blk` (first_block is ascending).
__device__ __forceinline__ int find_tensor(const af8_fullrank_tensor *tensors, int n, int64_t blk)
{
    int lo = 0, hi = n - 1;
    while (lo < hi) {
        int mid = (lo + hi + 1) >> 1;
        if (__ldg(&tensors[mid].first_block) <= blk) lo = mid; else hi = mid - 1;
    }
    return lo;
}

template <typename T> struct GradLoad;

template <> struct GradLoad<float> {
    static __device__ __forceinline__ void load8(const void *base, int64_t off, float (&g)[8])
    {
        const float4 *p = reinterpret_cast<const float4 *>(static_cast<const float *>(base) + off);
        float4 a = __ldcs(p), b = __ldcs(p + 1);
        g[0] = a.x; g[1] = a.y; g[2] = a.z; g[3] = a.w;
        g[4] = b.x; g[5] = b.y; g[6] = b.z; g[7] = b.w;
    }
    static __device__ __forceinline__ float load1(const void *base, int64_t off)
    {
        return static_cast<const float *>(base)[off];
    }
};

struct bf16_tag {};
template <> struct GradLoad<bf16_tag> {
    static __device__ __forceinline__ void load8(const void *base, int64_t off, float (&g)[8])
    {
        const uint4 *p = reinterpret_cast<const uint4 *>(static_cast<const uint16_t *>(base) + off);
        uint4 a = __ldcs(p);
        g[0] = __uint_as_float(a.x << 16); g[1] = __uint_as_float(a.x & 0xffff0000u);
        g[2] = __uint_as_float(a.y << 16); g[3] = __uint_as_float(a.y & 0xffff0000u);
        g[4] = __uint_as_float(a.z << 16); g[5] = __uint_as_float(a.z & 0xffff0000u);
        g[6] = __uint_as_float(a.w << 16); g[7] = __uint_as_float(a.w & 0xffff0000u);
    }
    static __device__ __forceinline__ float load1(const void *base, int64_t off)
    {
        return bf16_bits_to_f32(static_cast<const uint16_t *>(base)[off]);
    }
};

template <typename GradT, int MODE>
__global__ void __launch_bounds__(FAST_THREADS, 3)
fullrank_fast_kernel(const FullrankLaunch L)
{
    __shared__ af8_fullrank_tensor sT;
    __shared__ float s_tab[256];
    __shared__ float s_red[3][FAST_THREADS / 32];

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    int cur_t = -1;

    for (int64_t blk = blockIdx.x; blk < L.total_blocks; blk += gridDim.x) {
        // ---- locate the tensor (uniform over the CTA) ----
        int t = cur_t;
        if (t < 0) {
            t = find_tensor(L.tensors, L.n_tensors, blk);
        } else {
            while (t + 1 < L.n_tensors && __ldg(&L.tensors[t + 1].first_block) <= blk) ++t;
        }
        __syncthreads();  // previous iteration is done with sT, s_tab, s_red
        if (t != cur_t) {
            if (tid < (int)(sizeof(af8_fullrank_tensor) / 4))
                reinterpret_cast<uint32_t *>(&sT)[tid] =
                    __ldg(reinterpret_cast<const uint32_t *>(L.tensors + t) + tid);
            cur_t = t;
        }
        __syncthreads();

        const int64_t b = blk - sT.first_block;       // V block index inside the tensor
        const int64_t base = b * FAST_VBLOCK;         // first element of the block
        const int64_t rem = sT.numel - base;          // real elements from base on (> 0)
        const bool full = rem >= FAST_VBLOCK;
        const int e0 = tid * FAST_EPT;
        const bool m_exists = (int64_t)warp * FAST_MBLOCK < rem;  // this warp's M block is allocated

        // ---- loads ----
        float p[FAST_EPT], g[FAST_EPT];
        uint32_t mq0, mq1, vq0, vq1;
        float *pptr = static_cast<float *>(sT.param) + base + e0;
        {
            const uint2 vv = __ldcs(reinterpret_cast<const uint2 *>(static_cast<const uint8_t *>(sT.v_q) + base + e0));
            vq0 = vv.x; vq1 = vv.y;
        }
        if (m_exists) {
            const uint2 mm = __ldcs(reinterpret_cast<const uint2 *>(sT.m_q + base + e0));
            mq0 = mm.x; mq1 = mm.y;
        } else {
            mq0 = mq1 = 0x80808080u;
        }
        if (full) {
            const float4 a = *reinterpret_cast<const float4 *>(pptr);
            const float4 c = *reinterpret_cast<const float4 *>(pptr + 4);
            p[0] = a.x; p[1] = a.y; p[2] = a.z; p[3] = a.w;
            p[4] = c.x; p[5] = c.y; p[6] = c.z; p[7] = c.w;
            GradLoad<GradT>::load8(sT.grad, base + e0, g);
        } else {
#pragma unroll
            for (int j = 0; j < FAST_EPT; ++j) {
                const bool ok = e0 + j < rem;
                p[j] = ok ? pptr[j] : 0.0f;
                g[j] = ok ? GradLoad<GradT>::load1(sT.grad, base + e0 + j) : 0.0f;
            }
        }

        // ---- AL8 decode table of this block: 255 powers of two ----
        {
            const float sc = __ldg(sT.v_scale + b);
            const float ml = __ldg(sT.v_min_log + b);
            s_tab[tid] = al_decode((uint32_t)tid, sc, ml, 254.0f);
        }
        // fl(m_scale / 128) (optimizer.py:531)
        const float mc = m_exists ? __fdiv_rn(__ldg(sT.m_scale + b * (FAST_VBLOCK / FAST_MBLOCK) + warp), 128.0f) : 0.0f;
        __syncthreads();

        const float decay = sT.decay, v_w = sT.v_w, m_w = sT.m_w;
        const float eps_g = sT.eps_gradsq, eps_d = sT.eps_denom;
        float step_mul, fira = 1.0f;
        bool zero_upd = false;
        if (MODE == AF8_MODE_APPLY) {
            const af8_dyn_scalars ds = L.dyn[cur_t];
            step_mul = ds.step; fira = ds.fira; zero_upd = ds.zero != 0.0f;
        } else {
            step_mul = -sT.alpha;
        }

        float v[FAST_EPT], m[FAST_EPT];
        float acc = 0.0f;
#pragma unroll
        for (int j = 0; j < FAST_EPT; ++j) {
            const bool real = full || (e0 + j < rem);
            const uint32_t vcode = ((j < 4 ? vq0 : vq1) >> (8 * (j & 3))) & 0xffu;
            const uint32_t mcode = ((j < 4 ? mq0 : mq1) >> (8 * (j & 3))) & 0xffu;
            const float gj = L.negate_grad ? -g[j] : g[j];
            // second moment (optimizer.py:2117-2119)
            const float g2 = __fadd_rn(__fmul_rn(gj, gj), eps_g);
            float vj = lerp_t(s_tab[vcode], g2, v_w);
            // momentum (optimizer.py:528-531, 698)
            const float m_old = __fmul_rn((float)((int)mcode - 128), mc);
            float mj = lerp_t(m_old, gj, m_w);
            if (!real) { vj = 0.0f; mj = 0.0f; }
            v[j] = vj; m[j] = mj;
            // update from the un-requantised v and m (optimizer.py:905, 909)
            const float den = __fadd_rn(__fsqrt_rn(vj), eps_d);
            float u = __fmul_rn(mj, __frcp_rn(den));
            if (MODE == AF8_MODE_SUMSQ) {
                if (real) acc = __fmaf_rn(u, u, acc);
            } else {
                if (MODE == AF8_MODE_APPLY) u = zero_upd ? 0.0f : __fmul_rn(u, fira);  // optimizer.py:798-803
                const float p1 = __fmul_rn(p[j], decay);        // optimizer.py:2039
                p[j] = __fmaf_rn(step_mul, u, p1);              // optimizer.py:874
            }
        }

        if (MODE == AF8_MODE_SUMSQ) {
            acc = warp_sum(acc);
            if (lane == 0) s_red[2][warp] = acc;
            __syncthreads();
            if (tid == 0) {
                float s = 0.0f;
#pragma unroll
                for (int w = 0; w < FAST_THREADS / 32; ++w) s = __fadd_rn(s, s_red[2][w]);
                L.block_sumsq[blk] = s;
            }
            continue;
        }

        // ---- parameter store ----
        if (full) {
            *reinterpret_cast<float4 *>(pptr) = make_float4(p[0], p[1], p[2], p[3]);
            *reinterpret_cast<float4 *>(pptr + 4) = make_float4(p[4], p[5], p[6], p[7]);
        } else {
#pragma unroll
            for (int j = 0; j < FAST_EPT; ++j)
                if (e0 + j < rem) pptr[j] = p[j];
        }

        // ---- momentum requantisation: one warp = one M block (optimizer.py:510, 518) ----
        {
            float am = 0.0f;
#pragma unroll
            for (int j = 0; j < FAST_EPT; ++j) am = fmaxf(am, fabsf(m[j]));
            am = fmaxf(warp_max(am), 1e-12f);
            uint32_t o0 = 0, o1 = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                o0 |= uf8_encode(m[j], am) << (8 * j);
                o1 |= uf8_encode(m[j + 4], am) << (8 * j);
            }
            if (m_exists) {
                *reinterpret_cast<uint2 *>(sT.m_q + base + e0) = make_uint2(o0, o1);
                if (lane == 0) sT.m_scale[b * (FAST_VBLOCK / FAST_MBLOCK) + warp] = am;
            }
        }

        // ---- second-moment requantisation over the whole V block (optimizer.py:308-321) ----
        {
            float l[FAST_EPT];
            float mn = INFINITY, mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < FAST_EPT; ++j) {
                l[j] = al_log2(v[j]);
                if (v[j] != 0.0f) mn = fminf(mn, l[j]);
                mx = fmaxf(mx, l[j]);
            }
            mn = warp_min(mn);
            mx = warp_max(mx);
            if (lane == 0) { s_red[0][warp] = mn; s_red[1][warp] = mx; }
            __syncthreads();
#pragma unroll
            for (int w = 0; w < FAST_THREADS / 32; ++w) {
                mn = fminf(mn, s_red[0][w]);
                mx = fmaxf(mx, s_red[1][w]);
            }
            float min_log, scale;
            al_range(mn, mx, L.v_floor, min_log, scale);
            uint32_t o0 = 0, o1 = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                o0 |= al_encode(v[j], l[j], min_log, scale, 254.0f, 255) << (8 * j);
                o1 |= al_encode(v[j + 4], l[j + 4], min_log, scale, 254.0f, 255) << (8 * j);
            }
            *reinterpret_cast<uint2 *>(static_cast<uint8_t *>(sT.v_q) + base + e0) = make_uint2(o0, o1);
            if (tid == 0) { sT.v_scale[b] = scale; sT.v_min_log[b] = min_log; }
        }
    }
}

}  // namespace af8
