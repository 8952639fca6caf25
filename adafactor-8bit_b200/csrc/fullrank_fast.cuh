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
//
// Instruction budget.  At 14-16 bytes per parameter the HBM roofline leaves
// roughly 60 issue slots per parameter, so exact IEEE arithmetic is spent only
// where it decides a stored bit:
//   * the EMAs, the dequantisation and both requantisations are bit-exact
//     restatements of the torch ops;
//   * the block extrema are reduced on v itself (log2 is monotone) and the
//     exactly rounded log2 is taken of the two extreme values only;
//   * a second-moment code is first computed from the hardware log2
//     approximation; only when that estimate lies closer to a rounding
//     boundary than its own error bound is the exact sequence (binary64 log2,
//     IEEE division) evaluated, so the stored code is always the exact one;
//   * the momentum division m/absmax uses the correctly rounded reciprocal of
//     the block's absmax with one residual correction, which yields the IEEE
//     quotient;
//   * the parameter update u = m / (sqrt(v) + eps) feeds nothing but the fp32
//     parameter, whose tolerance is relative 1e-5; it uses the hardware
//     approximations of sqrt and reciprocal (relative error below 3e-7).
#pragma once

#include "common.cuh"

namespace af8 {

constexpr int FAST_VBLOCK = 2048;
constexpr int FAST_MBLOCK = 256;
constexpr int FAST_THREADS = 256;
constexpr int FAST_EPT = 8;  // elements per thread
constexpr int FAST_WARPS = FAST_THREADS / 32;

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

// hardware approximations, used only where the result does not reach a stored state
__device__ __forceinline__ float sqrt_approx(float x)
{
    float y;
    asm("sqrt.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float rcp_approx(float x)
{
    float y;
    asm("rcp.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float lg2_approx(float x)
{
    float y;
    asm("lg2.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// bound used for |lg2.approx(x) - log2(x)| / max(|log2(x)|, 1)
#define LG2_REL_BOUND 3.6e-7f   /* measured worst case on B200: 2.3e-7 */

#define AF8_MAGIC_F 12582912.0f       /* 1.5 * 2^23: adding it rounds to an integer (half to even) */
#define AF8_MAGIC_I 0x4b400000

// (byte j of a packed word) - 128 as a float, without a conversion instruction:
// the byte becomes the low mantissa bits of 2^23 + byte
__device__ __forceinline__ float byte_minus_128(uint32_t word, int j)
{
    return __uint_as_float(__byte_perm(word, 0x4b000000u, 0x7540u | (uint32_t)j)) - 8388736.0f;
}

// block-wide constants of the second-moment requantisation, produced by warp 0
struct __align__(16) VRange {
    float min_log;   // stored range
    float scale;
    float k;         // 254 / scale (estimate path)
    float c;         // -min_log * k
    float thr;       // an estimate is trusted when |t - rint(t)| <= thr
    float pad[3];
};

template <bool SMALL_W>
__device__ __forceinline__ float lerp_sel(float s, float e, float w, float wm1)
{
    const float d = __fsub_rn(e, s);
    return SMALL_W ? __fmaf_rn(w, d, s) : __fmaf_rn(wm1, d, e);
}

template <typename GradT, int MODE>
__global__ void __launch_bounds__(FAST_THREADS, 3)
fullrank_fast_kernel(const FullrankLaunch L)
{
    __shared__ af8_fullrank_tensor sT;
    __shared__ float s_tab[256];
    __shared__ float s_red[3][FAST_WARPS];
    __shared__ VRange s_vr;

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
        __syncthreads();  // previous iteration is done with sT, s_tab, s_red, s_vr
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
        uint32_t mq[2], vq[2];
        float *pptr = static_cast<float *>(sT.param) + base + e0;
        {
            const uint2 vv = __ldcs(reinterpret_cast<const uint2 *>(static_cast<const uint8_t *>(sT.v_q) + base + e0));
            vq[0] = vv.x; vq[1] = vv.y;
        }
        if (m_exists) {
            const uint2 mm = __ldcs(reinterpret_cast<const uint2 *>(sT.m_q + base + e0));
            mq[0] = mm.x; mq[1] = mm.y;
        } else {
            mq[0] = mq[1] = 0x80808080u;
        }
        if (full) {
            if (MODE != AF8_MODE_SUMSQ) {
                const float4 a = *reinterpret_cast<const float4 *>(pptr);
                const float4 c = *reinterpret_cast<const float4 *>(pptr + 4);
                p[0] = a.x; p[1] = a.y; p[2] = a.z; p[3] = a.w;
                p[4] = c.x; p[5] = c.y; p[6] = c.z; p[7] = c.w;
            }
            GradLoad<GradT>::load8(sT.grad, base + e0, g);
        } else {
#pragma unroll
            for (int j = 0; j < FAST_EPT; ++j) {
                const bool ok = e0 + j < rem;
                p[j] = (ok && MODE != AF8_MODE_SUMSQ) ? pptr[j] : 0.0f;
                g[j] = ok ? GradLoad<GradT>::load1(sT.grad, base + e0 + j) : 0.0f;
            }
        }

        // ---- AL8 decode table of this block: 255 powers of two (optimizer.py:341-349) ----
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
        if (MODE == AF8_MODE_APPLY) {
            const af8_dyn_scalars ds = L.dyn[cur_t];
            step_mul = ds.step;
            fira = (ds.zero != 0.0f) ? 0.0f : ds.fira;     // a non-finite norm zeroes the update (optimizer.py:798-800)
            if (ds.zero != 0.0f) step_mul = 0.0f;
        } else {
            step_mul = -sT.alpha;
        }

        // ---- EMAs and update: everything that reaches a state is exact ----
        float v[FAST_EPT], m[FAST_EPT];
        float acc = 0.0f;
        const bool small_w = fabsf(v_w) < 0.5f && fabsf(m_w) < 0.5f;   // ATen's lerp has two forms
        const float v_wm1 = __fsub_rn(v_w, 1.0f), m_wm1 = __fsub_rn(m_w, 1.0f);
#pragma unroll
        for (int j = 0; j < FAST_EPT; ++j) {
            const bool real = full || (e0 + j < rem);
            const uint32_t vcode = (vq[j >> 2] >> (8 * (j & 3))) & 0xffu;
            const float gj = L.negate_grad ? -g[j] : g[j];
            // second moment (optimizer.py:2117-2119)
            const float g2 = __fadd_rn(__fmul_rn(gj, gj), eps_g);
            const float v_old = s_tab[vcode];
            // momentum (optimizer.py:528-531, 698)
            const float m_old = __fmul_rn(byte_minus_128(mq[j >> 2], j & 3), mc);
            float vj, mj;
            if (small_w) {
                vj = lerp_sel<true>(v_old, g2, v_w, v_wm1);
                mj = lerp_sel<true>(m_old, gj, m_w, m_wm1);
            } else {
                vj = lerp_t(v_old, g2, v_w);
                mj = lerp_t(m_old, gj, m_w);
            }
            if (!real) { vj = 0.0f; mj = 0.0f; }
            v[j] = vj; m[j] = mj;
            // update from the un-requantised v and m (optimizer.py:905, 909); feeds the parameter only
            const float u = __fmul_rn(mj, rcp_approx(__fadd_rn(sqrt_approx(vj), eps_d)));
            if (MODE == AF8_MODE_SUMSQ) {
                acc = __fmaf_rn(u, u, acc);                       // padding contributes m = 0
            } else {
                const float us = (MODE == AF8_MODE_APPLY) ? __fmul_rn(u, fira) : u;   // optimizer.py:803
                const float p1 = __fmul_rn(p[j], decay);          // optimizer.py:2039
                p[j] = (MODE == AF8_MODE_APPLY && step_mul == 0.0f) ? p1 : __fmaf_rn(step_mul, us, p1);   // optimizer.py:874
            }
        }

        if (MODE == AF8_MODE_SUMSQ) {
            acc = warp_sum(acc);
            if (lane == 0) s_red[2][warp] = acc;
            __syncthreads();
            if (tid == 0) {
                float s = 0.0f;
#pragma unroll
                for (int w = 0; w < FAST_WARPS; ++w) s = __fadd_rn(s, s_red[2][w]);
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

        // ---- block extrema of v (log2 is monotone, so they locate min_log and max_log) ----
        {
            float vmin = INFINITY, vmax = 0.0f;
#pragma unroll
            for (int j = 0; j < FAST_EPT; ++j) {
                vmin = fminf(vmin, v[j] != 0.0f ? v[j] : INFINITY);
                vmax = fmaxf(vmax, v[j]);
            }
            vmin = warp_min(vmin);
            vmax = warp_max(vmax);
            if (lane == 0) { s_red[0][warp] = vmin; s_red[1][warp] = vmax; }
        }

        // ---- momentum requantisation: one warp = one M block (optimizer.py:510, 518) ----
        {
            float am = 0.0f;
#pragma unroll
            for (int j = 0; j < FAST_EPT; ++j) am = fmaxf(am, fabsf(m[j]));
            am = fmaxf(warp_max(am), 1e-12f);
            const float ra = __frcp_rn(am);
            uint32_t raw[FAST_EPT];
#pragma unroll
            for (int j = 0; j < FAST_EPT; ++j) {
                // IEEE m / am from the correctly rounded reciprocal and one residual step
                float q = __fmul_rn(m[j], ra);
                const float r = __fmaf_rn(-q, am, m[j]);
                q = __fmaf_rn(r, ra, q);
                // round(q * 128) (the product is exact), clamp to [-128, 127]
                int k = __float_as_int(__fmaf_rn(q, 128.0f, AF8_MAGIC_F));
                k = max(AF8_MAGIC_I - 128, min(k, AF8_MAGIC_I + 127));
                raw[j] = (uint32_t)k;
            }
            // low bytes hold k mod 256; k + 128 is that byte with its top bit flipped
            const uint32_t o0 = __byte_perm(__byte_perm(raw[0], raw[1], 0x0040), __byte_perm(raw[2], raw[3], 0x0040), 0x5410) ^ 0x80808080u;
            const uint32_t o1 = __byte_perm(__byte_perm(raw[4], raw[5], 0x0040), __byte_perm(raw[6], raw[7], 0x0040), 0x5410) ^ 0x80808080u;
            if (m_exists) {
                __stcs(reinterpret_cast<uint2 *>(sT.m_q + base + e0), make_uint2(o0, o1));
                if (lane == 0) sT.m_scale[b * (FAST_VBLOCK / FAST_MBLOCK) + warp] = am;
            }
        }

        // ---- block range: exact log2 of the two extreme values only (optimizer.py:308-318) ----
        __syncthreads();
        if (warp == 0) {
            float vmin = lane < FAST_WARPS ? s_red[0][lane] : INFINITY;
            float vmax = lane < FAST_WARPS ? s_red[1][lane] : 0.0f;
            vmin = warp_min(vmin);
            vmax = warp_max(vmax);
            if (lane == 0) {
                const float mn = (vmin == INFINITY) ? INFINITY : al_log2(vmin);
                const float mx = al_log2(vmax);
                VRange r;
                al_range(mn, mx, L.v_floor, r.min_log, r.scale);
                r.k = __fdiv_rn(254.0f, r.scale);
                r.c = -__fmul_rn(r.min_log, r.k);
                // error bound of the estimate in code units: the hardware log2 (taken as
                // 2^-21 relative and absolute, twice its specified bound), the roundings of
                // the estimate itself and of the exact sequence it must agree with
                const float lmax = fmaxf(fmaxf(fabsf(r.min_log), fabsf(mx)), 1.0f);
                const float err = __fmaf_rn(__fmul_rn(lmax, LG2_REL_BOUND), r.k, 2.0e-4f);
                r.thr = 0.5f - err;
                s_vr = r;
                sT.v_scale[b] = r.scale;
                sT.v_min_log[b] = r.min_log;
            }
        }
        __syncthreads();

        // ---- second-moment codes ----
        {
            const VRange r = s_vr;
            int kk[FAST_EPT];
            uint32_t ambiguous = 0;
#pragma unroll
            for (int j = 0; j < FAST_EPT; ++j) {
                const float le = lg2_approx(fmaxf(v[j], AF8_TINY));
                const float te = __fmaf_rn(le, r.k, r.c);
                const float s = __fadd_rn(te, AF8_MAGIC_F + 1.0f);          // rint(te) + 1 in the low bits
                const float rf = __fsub_rn(s, AF8_MAGIC_F + 1.0f);
                if (!(fabsf(__fsub_rn(te, rf)) <= r.thr) && (v[j] != 0.0f)) ambiguous |= 1u << j;
                kk[j] = __float_as_int(s);
            }
            if (__any_sync(0xffffffffu, ambiguous != 0)) {
                // rare: redo the codes in doubt with the exact sequence
#pragma unroll
                for (int j = 0; j < FAST_EPT; ++j)
                    if (ambiguous & (1u << j))
                        kk[j] = AF8_MAGIC_I + (int)al_encode(v[j], al_log2(v[j]), r.min_log, r.scale, 254.0f, 255);
            }
            uint32_t raw[FAST_EPT];
#pragma unroll
            for (int j = 0; j < FAST_EPT; ++j) {
                int k = max(AF8_MAGIC_I + 1, min(kk[j], AF8_MAGIC_I + 255));
                raw[j] = (v[j] == 0.0f) ? (uint32_t)AF8_MAGIC_I : (uint32_t)k;   // code 0 is reserved for exact zero
            }
            const uint32_t o0 = __byte_perm(__byte_perm(raw[0], raw[1], 0x0040), __byte_perm(raw[2], raw[3], 0x0040), 0x5410);
            const uint32_t o1 = __byte_perm(__byte_perm(raw[4], raw[5], 0x0040), __byte_perm(raw[6], raw[7], 0x0040), 0x5410);
            __stcs(reinterpret_cast<uint2 *>(static_cast<uint8_t *>(sT.v_q) + base + e0), make_uint2(o0, o1));
        }
    }
}

}  // namespace af8
