// Full-rank fused step, general kernel: every combination of state formats
// (V: fp32 / AL8 / AL16; M: none / UF8 / UF4 / d8 / d4 / fp32), block sizes and
// update rules that the reference's full-rank path accepts
// (_update_param_8bit, optimizer.py:2076-2194; _fallback_1d_update,
// optimizer.py:886-917).  The specialised kernel in fullrank_fast.cuh covers
// the AdamW UF8/AL8 configuration; this one covers the rest and the small
// fp32-state tensors (numel < min_8bit_size, optimizer.py:1640-1641).
//
// One CTA owns one V block of `block` elements.  The new second moment (as its
// log2) and the new momentum are staged in shared memory, because the block
// size is a run-time value; the requantisation passes then re-read them.
#pragma once

#include "common.cuh"
#include "fullrank_fast.cuh"

namespace af8 {

__constant__ float c_qmap8[256];
__constant__ float c_qmap4[16];

constexpr int GEN_THREADS = 256;
constexpr int GEN_MAX_BLOCK = 8192;

struct GenericCfg {
    int32_t v_fmt, m_fmt, block, m_block, use_adam_denom, momentum_only;
};

// nearest codebook entry with the reference's tie and sign rules
// (_quantize_dynamic_pytorch, optimizer.py:463-473).  map has L sorted entries.
__device__ __forceinline__ uint32_t dyn_encode(float m, float a, const float *map, int L)
{
    const float x = __fdiv_rn(m, a);
    int lo = 0, hi = L;
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (map[mid] < x) lo = mid + 1; else hi = mid;
    }
    int idx = min(lo, L - 1);
    const int prev = max(idx - 1, 0);
    const float cd = fabsf(__fsub_rn(x, map[idx]));
    const float pd = fabsf(__fsub_rn(x, map[prev]));
    if (pd < cd) idx = prev;
    const int os = (x > 0.0f) - (x < 0.0f);
    const float mv = map[idx];
    const int ms = (mv > 0.0f) - (mv < 0.0f);
    const bool flip = (os != ms) && (os != 0);
    if (flip && os > 0 && idx < L - 1) return (uint32_t)(idx + 1);
    if (flip && os < 0 && idx > 0) return (uint32_t)(idx - 1);
    return (uint32_t)idx;
}

__device__ __forceinline__ float m_decode(const uint8_t *q, float scale, int64_t i, int fmt)
{
    switch (fmt) {
    case AF8_M_UF8:
        return __fmul_rn((float)((int)q[i] - 128), __fdiv_rn(scale, 128.0f));
    case AF8_M_UF4: {
        const uint32_t byte = q[i >> 1];
        const uint32_t nib = (i & 1) ? (byte & 0xfu) : (byte >> 4);
        return __fmul_rn((float)((int)nib - 8), __fdiv_rn(scale, 8.0f));
    }
    case AF8_M_D8:
        return __fmul_rn(c_qmap8[q[i]], scale);
    default: {  // AF8_M_D4
        const uint32_t byte = q[i >> 1];
        const uint32_t nib = (i & 1) ? (byte & 0xfu) : (byte >> 4);
        return __fmul_rn(c_qmap4[nib], scale);
    }
    }
}

__device__ __forceinline__ uint32_t m_encode(float m, float a, int fmt)
{
    switch (fmt) {
    case AF8_M_UF8: return uf8_encode(m, a);
    case AF8_M_UF4: return uf4_encode(m, a);
    case AF8_M_D8: return dyn_encode(m, a, c_qmap8, 256);
    default: return dyn_encode(m, a, c_qmap4, 16);
    }
}

// MODE: AF8_MODE_NOCLIP / SUMSQ / APPLY, plus 3 = SUMSQ of the momentum update
// on the momentum-only path (reads dyn.pre_div like APPLY, writes nothing but
// the partial sums).
template <typename GradT, int MODE>
__global__ void __launch_bounds__(GEN_THREADS)
fullrank_generic_kernel(const FullrankLaunch L, const GenericCfg C)
{
    extern __shared__ float s_dyn[];
    float *s_l = s_dyn;                 // log2 of the new v, -inf marks exact zero
    float *s_m = s_dyn + C.block;       // new momentum
    __shared__ af8_fullrank_tensor sT;
    __shared__ float s_red[3][GEN_THREADS / 32];

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const bool no_v = C.v_fmt == AF8_V_NONE;     // SGD mode: no second moment (optimizer.py:2045-2071)
    const bool v_quant = C.v_fmt != AF8_V_FP32 && !no_v;
    const bool has_m = C.m_fmt != AF8_M_NONE;
    const bool m_quant = has_m && C.m_fmt != AF8_M_FP32;
    const bool writes = (MODE == AF8_MODE_NOCLIP || MODE == AF8_MODE_APPLY || MODE == AF8_MODE_LAG);
    constexpr bool DYN = MODE == AF8_MODE_APPLY || MODE == AF8_MODE_LAG;   // scalars of a statistic pass or of the previous step
    constexpr bool SUMS = MODE == AF8_MODE_SUMSQ || MODE == AF8_MODE_LAG;  // partial sums of squares of the raw update
    const float qm1 = (C.v_fmt == AF8_V_AL16) ? 65534.0f : 254.0f;
    const int qmax = (C.v_fmt == AF8_V_AL16) ? 65535 : 255;
    int cur_t = -1;

    for (int64_t blk = blockIdx.x; blk < L.total_blocks; blk += gridDim.x) {
        int t = cur_t;
        if (t < 0) {
            t = find_tensor(L.tensors, L.n_tensors, blk);
        } else {
            while (t + 1 < L.n_tensors && __ldg(&L.tensors[t + 1].first_block) <= blk) ++t;
        }
        __syncthreads();
        if (t != cur_t) {
            if (tid < (int)(sizeof(af8_fullrank_tensor) / 4))
                reinterpret_cast<uint32_t *>(&sT)[tid] =
                    __ldg(reinterpret_cast<const uint32_t *>(L.tensors + t) + tid);
            cur_t = t;
        }
        __syncthreads();

        const int64_t b = blk - sT.first_block;
        const int64_t base = b * C.block;
        const int64_t rem = sT.numel - base;
        const int valid = (int)(rem < C.block ? rem : C.block);
        const int subs_per_block = has_m && m_quant ? C.block / C.m_block : 0;

        float v_scale = 1.0f, v_min_log = 0.0f;
        if (v_quant) { v_scale = __ldg(sT.v_scale + b); v_min_log = __ldg(sT.v_min_log + b); }

        float step_mul = -sT.alpha, fira = 1.0f, pre_div = 1.0f;
        bool zero_upd = false;
        if (DYN || MODE == 3) {
            const af8_dyn_scalars ds = L.dyn[cur_t];
            pre_div = ds.pre_div;
            if (DYN) { step_mul = ds.step; fira = ds.fira; zero_upd = ds.zero != 0.0f; }
        }

        float acc = 0.0f, mn = INFINITY, mx = -INFINITY;

        for (int i = tid; i < C.block; i += GEN_THREADS) {
            const bool real = i < valid;
            float vj = 0.0f, mj = 0.0f;
            if (real) {
                float gj = GradLoad<GradT>::load1(sT.grad, base + i);
                if (L.negate_grad) gj = -gj;
                // ---- second moment ----
                if (no_v) {
                } else if (v_quant) {   // optimizer.py:2117-2119
                    uint32_t code = (C.v_fmt == AF8_V_AL16)
                                        ? static_cast<const uint16_t *>(sT.v_q)[base + i]
                                        : static_cast<const uint8_t *>(sT.v_q)[base + i];
                    const float v_old = al_decode(code, v_scale, v_min_log, qm1);
                    const float g2 = __fadd_rn(__fmul_rn(gj, gj), sT.eps_gradsq);
                    vj = lerp_t(v_old, g2, sT.v_w);
                } else if (sT.v_keep < 0.0f) {   // fp32 state updated with Tensor.lerp_ (APOLLO's low-rank V, optimizer.py:2797-2799)
                    vj = lerp_t(sT.v_f32[base + i], __fadd_rn(__fmul_rn(gj, gj), sT.eps_gradsq), sT.v_w);
                    if (writes) sT.v_f32[base + i] = vj;
                } else {         // optimizer.py:2186-2189
                    const float keep = __fmul_rn(sT.v_f32[base + i], sT.v_keep);
                    vj = __fmaf_rn(__fmul_rn(sT.v_w, gj), gj, keep);
                    if (sT.eps_gradsq > 0.0f) vj = __fadd_rn(vj, sT.v_eps_add);
                    if (writes) sT.v_f32[base + i] = vj;
                }
                // ---- normaliser ----
                float inv = 0.0f, den = 1.0f;
                if (no_v) {
                } else if (C.use_adam_denom) {
                    den = __fadd_rn(__fsqrt_rn(vj), sT.eps_denom);   // optimizer.py:905, 913
                    inv = __frcp_rn(den);
                } else {
                    inv = rsqrt_t(fmaxf(vj, sT.eps_sq));             // optimizer.py:895, 907, 915
                }
                // ---- momentum and update ----
                float u;
                if (no_v && !has_m) {
                    u = gj;                     // optimizer.py:2065-2066
                    if (SUMS) acc = __fmaf_rn(u, u, acc);
                } else if (has_m) {
                    float m_old;
                    if (m_quant) {
                        const int64_t sb = (base + i) / C.m_block;
                        m_old = m_decode(sT.m_q, __ldg(sT.m_scale + sb), base + i, C.m_fmt);
                    } else {
                        m_old = sT.m_f32[base + i];
                    }
                    if (no_v) {                 // optimizer.py:2047-2064: momentum / float(1 - beta1), kept in v_keep
                        mj = lerp_t(m_old, gj, sT.m_w);
                        u = __fdiv_rn(mj, sT.v_keep);
                        if (SUMS) acc = __fmaf_rn(u, u, acc);
                    } else if (C.momentum_only) {      // optimizer.py:894-901
                        float ut = __fmul_rn(gj, inv);
                        if (SUMS) {
                            acc = __fmaf_rn(ut, ut, acc);
                        }
                        ut = __fdiv_rn(ut, pre_div);
                        mj = lerp_t(m_old, ut, sT.m_w);
                        u = mj;
                        if (MODE == 3) acc = __fmaf_rn(u, u, acc);
                    } else {                    // optimizer.py:903-910
                        mj = lerp_t(m_old, gj, sT.m_w);
                        u = __fmul_rn(mj, inv);
                        if (SUMS) acc = __fmaf_rn(u, u, acc);
                    }
                    if (!m_quant && writes) sT.m_f32[base + i] = mj;
                } else {                        // optimizer.py:911-917
                    u = C.use_adam_denom ? __fdiv_rn(gj, den) : __fmul_rn(gj, inv);
                    if (SUMS) acc = __fmaf_rn(u, u, acc);
                }
                if (writes) {
                    if (DYN) u = zero_upd ? 0.0f : __fmul_rn(u, fira);
                    const float pv = param_load(sT.param, base + i, L.param_dtype);
                    const uint32_t pbits = param_step_bits(pv, sT.decay, step_mul, u, L.param_dtype, L.sr, sT.sr_base, base + i);
                    param_store_bits(sT.param, base + i, pbits, L.param_dtype);
                    if (sT.param_copy != nullptr && L.param_dtype == AF8_F32)       // bf16 compute copy
                        static_cast<uint16_t *>(sT.param_copy)[base + i] = (uint16_t)f32_to_bf16_rn_bits(__uint_as_float(pbits));
                }
            }
            if (writes) {
                if (v_quant) {
                    const float l = al_log2(vj);
                    if (vj != 0.0f) mn = fminf(mn, l);
                    mx = fmaxf(mx, l);
                    s_l[i] = (vj != 0.0f) ? l : -INFINITY;
                }
                if (m_quant) s_m[i] = mj;
            }
        }

        if (!writes || MODE == AF8_MODE_LAG) {
            acc = warp_sum(acc);
            if (lane == 0) s_red[2][warp] = acc;
            __syncthreads();
            if (tid == 0) {
                float s = 0.0f;
                for (int w = 0; w < GEN_THREADS / 32; ++w) s = __fadd_rn(s, s_red[2][w]);
                L.block_sumsq[blk] = s;
            }
            if (!writes) continue;
        }

        if (v_quant) {
            mn = warp_min(mn);
            mx = warp_max(mx);
            if (lane == 0) { s_red[0][warp] = mn; s_red[1][warp] = mx; }
        }
        __syncthreads();   // s_l, s_m and the warp extrema are visible
        if (v_quant) {
            for (int w = 0; w < GEN_THREADS / 32; ++w) {
                mn = fminf(mn, s_red[0][w]);
                mx = fmaxf(mx, s_red[1][w]);
            }
            float min_log, scale;
            al_range(mn, mx, L.v_floor, min_log, scale);
            for (int i = tid; i < C.block; i += GEN_THREADS) {
                const float l = s_l[i];
                const bool zero = (l == -INFINITY);
                const uint32_t code = zero ? 0u : al_encode(1.0f, l, min_log, scale, qm1, qmax);
                if (C.v_fmt == AF8_V_AL16) static_cast<uint16_t *>(sT.v_q)[base + i] = (uint16_t)code;
                else static_cast<uint8_t *>(sT.v_q)[base + i] = (uint8_t)code;
            }
            if (tid == 0) { sT.v_scale[b] = scale; sT.v_min_log[b] = min_log; }
        }
        if (m_quant) {
            // the M state is padded to a multiple of m_block only: sub-blocks that
            // start at or beyond numel do not exist
            const bool four_bit = (C.m_fmt == AF8_M_UF4 || C.m_fmt == AF8_M_D4);
            for (int sb = warp; sb < subs_per_block; sb += GEN_THREADS / 32) {
                const int s0 = sb * C.m_block;
                if (s0 >= valid) break;
                float am = 0.0f;
                for (int i = lane; i < C.m_block; i += 32) am = fmaxf(am, fabsf(s_m[s0 + i]));
                am = fmaxf(warp_max(am), 1e-12f);
                if (four_bit) {
                    for (int i = lane * 2; i < C.m_block; i += 64) {
                        const uint32_t hi = m_encode(s_m[s0 + i], am, C.m_fmt);
                        const uint32_t lo = m_encode(s_m[s0 + i + 1], am, C.m_fmt);
                        sT.m_q[(base + s0 + i) >> 1] = (uint8_t)((hi << 4) | lo);
                    }
                } else {
                    for (int i = lane; i < C.m_block; i += 32)
                        sT.m_q[base + s0 + i] = (uint8_t)m_encode(s_m[s0 + i], am, C.m_fmt);
                }
                if (lane == 0) sT.m_scale[(base + s0) / C.m_block] = am;
            }
        }
    }
}

}  // namespace af8
