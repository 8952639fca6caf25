// Full-rank fused step, AdamW UF8 (M block 256) / AL8 (V block 2048), fp32 parameters:
// the update passes (NOCLIP / APPLY / LAG) with ONE WARP per V block.
//
// fullrank_fast_kernel gives a V block to a CTA of eight warps; the block's range (the
// extrema of the new second moments over all 2048 elements) then costs two block-wide
// barriers per block, which that kernel's profile shows as its largest stall.  Here a warp
// walks the eight momentum blocks of its V block one after another (8 elements per lane and
// momentum block, 64 per V block), keeps the 64 new second moments in registers, reduces the
// extrema with two REDUX instructions and writes the codes at the end: no block-wide barrier
// after the start-up.  Inputs arrive through the warp's own ring of bulk asynchronous copies,
// one stage per momentum block (parameter 1024 B, gradient 512 / 1024 B, the two code runs
// 256 B each), requested FW_STAGES - 1 momentum blocks ahead, across the warp's V blocks of
// the same tensor.  Tail blocks load directly.  Arithmetic: the routines of
// fullrank_fast.cuh, element for element (same stored bits).
#pragma once

#include "fullrank_fast.cuh"

namespace af8 {

constexpr int FW_THREADS = 128;
constexpr int FW_WARPS = FW_THREADS / 32;
#ifndef AF8_FW_STAGES
#define AF8_FW_STAGES 4
#endif
constexpr int FW_STAGES = AF8_FW_STAGES;
#ifndef AF8_FW_MIN_CTAS
#define AF8_FW_MIN_CTAS 4
#endif
constexpr int DEVERR_FW_TIMEOUT = 5;
#ifndef AF8_FULLRANK_WARP_DEFAULT
#define AF8_FULLRANK_WARP_DEFAULT 0      /* which update kernel fp32 parameters take unless AF8_FULLRANK_WARP says otherwise */
#endif

template <typename GradT> struct FwRing {
    static constexpr int GB = GradBytes<GradT>::value;
    static constexpr int P_OFF = 0, G_OFF = 1024, MQ_OFF = G_OFF + 256 * GB, VQ_OFF = MQ_OFF + 256, STAGE = VQ_OFF + 256;
    static constexpr int WARP_BYTES = FW_STAGES * STAGE + 1024;       // the ring, then the 256-entry decode table
    static constexpr int SMEM_BYTES = FW_WARPS * WARP_BYTES;
};

template <typename GradT, int MODE>
__global__ void __launch_bounds__(FW_THREADS, AF8_FW_MIN_CTAS)
fullrank_warp_kernel(const FullrankLaunch L)
{
    using R = FwRing<GradT>;
    constexpr int GB = R::GB, NS = FW_STAGES, STAGE = R::STAGE;
    constexpr bool DYN = MODE == AF8_MODE_APPLY || MODE == AF8_MODE_LAG;
    extern __shared__ __align__(128) unsigned char fw_smem[];
    __shared__ __align__(8) uint64_t s_full[FW_WARPS][NS];
    __shared__ double s_exp2[32];
    __shared__ double2 s_log2[97];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    unsigned char *const ring = fw_smem + (size_t)warp * R::WARP_BYTES;
    float *const tab = reinterpret_cast<float *>(ring + NS * STAGE);
    if (tid < 32) s_exp2[tid] = c_exp2_tab[tid];
    if (tid < 97) s_log2[tid] = c_log2_tab[tid];
    if (lane == 0) {
        for (int k = 0; k < NS; ++k) mbar_init(&s_full[warp][k], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();                                   // the only block-wide barrier

    const int64_t W = (int64_t)gridDim.x * FW_WARPS;   // warps of the grid = stride of a warp's V blocks
    const int oa = lane * 4, ob = 128 + lane * 4;      // this lane's two 4-element groups inside a momentum block

    // the current tensor, cached per warp
    int t = -1;
    int64_t cur_first = 0, cur_end = 0, numel = 0, nfull = 0;
    float *param = nullptr;
    const unsigned char *grad = nullptr;
    uint8_t *m_q = nullptr, *v_q = nullptr;
    float *m_scale = nullptr, *v_scale = nullptr, *v_min_log = nullptr;
    uint16_t *param_copy = nullptr;
    StepScalars S;
    S.round_decay = false;
    bool small_w = true;
    uint32_t cons = 0;             // ring stages this warp has consumed
    int inflight = 0;              // momentum blocks from the current one on whose copies are issued

    for (int64_t blk = (int64_t)blockIdx.x * FW_WARPS + warp; blk < L.total_blocks; blk += W) {
        if (t < 0 || blk >= cur_end) {                 // uniform over the warp
            if (t < 0) t = find_tensor(L.tensors, L.n_tensors, blk);
            else while (t + 1 < L.n_tensors && __ldg(&L.tensors[t + 1].first_block) <= blk) ++t;
            const af8_fullrank_tensor *T = L.tensors + t;
            numel = __ldg(&T->numel);
            cur_first = __ldg(&T->first_block);
            cur_end = cur_first + (numel + FAST_VBLOCK - 1) / FAST_VBLOCK;
            nfull = numel / FAST_VBLOCK;
            param = static_cast<float *>(T->param);
            grad = static_cast<const unsigned char *>(T->grad);
            m_q = T->m_q; v_q = static_cast<uint8_t *>(T->v_q);
            m_scale = T->m_scale; v_scale = T->v_scale; v_min_log = T->v_min_log;
            param_copy = static_cast<uint16_t *>(T->param_copy);
            S.decay = __ldg(&T->decay); S.step_mul = -__ldg(&T->alpha);
            S.v_w = __ldg(&T->v_w); S.m_w = __ldg(&T->m_w);
            S.eps_g = __ldg(&T->eps_gradsq); S.eps_d = __ldg(&T->eps_denom);
            S.v_wm1 = __fsub_rn(S.v_w, 1.0f); S.m_wm1 = __fsub_rn(S.m_w, 1.0f);
            S.fira = 1.0f; S.zero_upd = false;
            if (DYN) {
                const af8_dyn_scalars ds = L.dyn[t];
                S.step_mul = ds.step; S.fira = ds.fira; S.zero_upd = ds.zero != 0.0f;
            }
            small_w = fabsf(S.v_w) < 0.5f && fabsf(S.m_w) < 0.5f;
            inflight = 0;                              // (copies never cross a tensor)
        }
        const int64_t b = blk - cur_first;             // V block inside the tensor
        const int64_t base = b * FAST_VBLOCK;
        const bool full = b < nfull;
        const int64_t rem = full ? FAST_VBLOCK : numel - base;

        // ---- decode table of this block's old second moments ----
        {
            const float sc = __ldg(v_scale + b), ml = __ldg(v_min_log + b);
            __syncwarp();                              // the previous block's look-ups are done
#pragma unroll
            for (int k = 0; k < 8; ++k) tab[lane + 32 * k] = al8_decode_fast((uint32_t)(lane + 32 * k), sc, ml, s_exp2);
            __syncwarp();
        }

        float vreg[64];                                // the block's new second moments (this lane's share)
        float fmn = INFINITY, fmx = 0.0f;
        float usq = 0.0f;
        // full blocks of this tensor that this warp still has after the current one
        const int64_t later = full ? (nfull - 1 - b) / W : 0;

#pragma unroll
        for (int s = 0; s < 8; ++s) {
            const int64_t e0 = base + s * FAST_MBLOCK;                   // first element of the momentum block
            const bool m_exists = (int64_t)s * FAST_MBLOCK < rem;
            float p[8], g[8], m[8];
            uint32_t mq[2], vq[2];
            int nva = 4, nvb = 4;
            if (full) {
                // ---- request the momentum blocks up to NS - 1 ahead (this block, then blk + W, ...) ----
                const int64_t chain = (8 - s) + 8 * later;
                const int want = (int)min((int64_t)NS, chain);
                if (lane == 0 && inflight < want) {
                    fence_proxy_async();
                    for (int k = inflight; k < want; ++k) {
                        const int sk = s + k;
                        const int64_t off = (b + (int64_t)(sk >> 3) * W) * FAST_VBLOCK + (sk & 7) * FAST_MBLOCK;
                        const int sl = (int)((cons + (uint32_t)k) % NS);
                        unsigned char *dst = ring + sl * STAGE;
                        mbar_expect_tx(&s_full[warp][sl], (uint32_t)STAGE);
                        bulk_g2s(dst + R::P_OFF, param + off, 1024, &s_full[warp][sl]);
                        bulk_g2s(dst + R::G_OFF, grad + off * GB, 256 * GB, &s_full[warp][sl]);
                        bulk_g2s(dst + R::MQ_OFF, m_q + off, 256, &s_full[warp][sl]);
                        bulk_g2s(dst + R::VQ_OFF, v_q + off, 256, &s_full[warp][sl]);
                    }
                }
                inflight = want - 1;
                const int sl = (int)(cons % NS);
                const bool landed = mbar_wait_bounded(&s_full[warp][sl], (cons / NS) & 1u);
                if (!__all_sync(0xffffffffu, landed)) {
                    atomicExch(&g_device_error, DEVERR_FW_TIMEOUT);
                    return;                            // this warp stops; nothing waits for it
                }
                const unsigned char *st = ring + sl * STAGE;
                {
                    const float4 a = *reinterpret_cast<const float4 *>(st + R::P_OFF + oa * 4);
                    const float4 c = *reinterpret_cast<const float4 *>(st + R::P_OFF + ob * 4);
                    p[0] = a.x; p[1] = a.y; p[2] = a.z; p[3] = a.w; p[4] = c.x; p[5] = c.y; p[6] = c.z; p[7] = c.w;
                }
                if (GB == 4) {
                    const float4 a = *reinterpret_cast<const float4 *>(st + R::G_OFF + oa * 4);
                    const float4 c = *reinterpret_cast<const float4 *>(st + R::G_OFF + ob * 4);
                    g[0] = a.x; g[1] = a.y; g[2] = a.z; g[3] = a.w; g[4] = c.x; g[5] = c.y; g[6] = c.z; g[7] = c.w;
                } else {
                    const uint2 a = *reinterpret_cast<const uint2 *>(st + R::G_OFF + oa * 2);
                    const uint2 c = *reinterpret_cast<const uint2 *>(st + R::G_OFF + ob * 2);
                    g[0] = __uint_as_float(a.x << 16); g[1] = __uint_as_float(a.x & 0xffff0000u);
                    g[2] = __uint_as_float(a.y << 16); g[3] = __uint_as_float(a.y & 0xffff0000u);
                    g[4] = __uint_as_float(c.x << 16); g[5] = __uint_as_float(c.x & 0xffff0000u);
                    g[6] = __uint_as_float(c.y << 16); g[7] = __uint_as_float(c.y & 0xffff0000u);
                }
                mq[0] = *reinterpret_cast<const uint32_t *>(st + R::MQ_OFF + oa);
                mq[1] = *reinterpret_cast<const uint32_t *>(st + R::MQ_OFF + ob);
                vq[0] = *reinterpret_cast<const uint32_t *>(st + R::VQ_OFF + oa);
                vq[1] = *reinterpret_cast<const uint32_t *>(st + R::VQ_OFF + ob);
                ++cons;
                __syncwarp();                          // the stage may be refilled from the next momentum block on
            } else {
                // tail block: guarded plain loads; the V state is padded to the block, the M state
                // only to its own 256-element blocks
                const int64_t left = rem - (int64_t)s * FAST_MBLOCK;
                nva = (int)max((int64_t)0, min((int64_t)4, left - oa));
                nvb = (int)max((int64_t)0, min((int64_t)4, left - ob));
                vq[0] = *reinterpret_cast<const uint32_t *>(v_q + e0 + oa);
                vq[1] = *reinterpret_cast<const uint32_t *>(v_q + e0 + ob);
                mq[0] = m_exists ? *reinterpret_cast<const uint32_t *>(m_q + e0 + oa) : 0x80808080u;
                mq[1] = m_exists ? *reinterpret_cast<const uint32_t *>(m_q + e0 + ob) : 0x80808080u;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int e = (j < 4) ? oa + j : ob + j - 4;
                    const bool ok = (j < 4) ? (j < nva) : (j - 4 < nvb);
                    p[j] = ok ? param[e0 + e] : 0.0f;
                    g[j] = ok ? GradLoad<GradT>::load1(grad, e0 + e) : 0.0f;
                }
            }
            if (L.negate_grad) {
#pragma unroll
                for (int j = 0; j < 8; ++j) g[j] = -g[j];
            }
            const float mc = m_exists ? __fmul_rn(__ldg(m_scale + b * (FAST_VBLOCK / FAST_MBLOCK) + s), 0.0078125f) : 0.0f;

            // ---- EMAs and update: everything that reaches a state is exact ----
            float v[8];
            if (small_w) {
                if (full) {
                    if (S.eps_g == 0.0f) ema_update<MODE, false, false>(g, p, mq, vq, tab, mc, S, nva, nvb, v, m, usq);
                    else ema_update<MODE, true, false>(g, p, mq, vq, tab, mc, S, nva, nvb, v, m, usq);
                } else {
                    ema_update<MODE, true, true>(g, p, mq, vq, tab, mc, S, nva, nvb, v, m, usq);
                }
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) {          // general lerp (weights >= 0.5): rare, kept simple
                    const bool real = (j < 4) ? (j < nva) : (j - 4 < nvb);
                    const uint32_t vcode = (vq[j >> 2] >> (8 * (j & 3))) & 0xffu;
                    const float g2 = __fadd_rn(__fmul_rn(g[j], g[j]), S.eps_g);
                    float vj = lerp_t(tab[vcode], g2, S.v_w);
                    float mj = lerp_t(__fmul_rn(byte_minus_128(mq[j >> 2], j & 3), mc), g[j], S.m_w);
                    if (!real) { vj = 0.0f; mj = 0.0f; }
                    v[j] = vj; m[j] = mj;
                    float u = __fmul_rn(mj, rcp_approx(__fadd_rn(sqrt_approx(vj), S.eps_d)));
                    if (!real) u = 0.0f;
                    float pj = __fmul_rn(p[j], S.decay);
                    if (MODE == AF8_MODE_LAG) usq = __fmaf_rn(u, u, usq);
                    const float us = DYN ? __fmul_rn(u, S.fira) : u;
                    if (!(DYN && S.zero_upd)) pj = __fmaf_rn(S.step_mul, us, pj);
                    p[j] = pj;
                }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                vreg[s * 8 + j] = v[j];
                fmn = fminf(fmn, v[j]);
                fmx = fmaxf(fmx, v[j]);
            }

            // ---- parameter store (and the optional bf16 compute copy) ----
            if (full) {
                *reinterpret_cast<float4 *>(param + e0 + oa) = make_float4(p[0], p[1], p[2], p[3]);
                *reinterpret_cast<float4 *>(param + e0 + ob) = make_float4(p[4], p[5], p[6], p[7]);
                if (param_copy != nullptr) {
                    *reinterpret_cast<uint2 *>(param_copy + e0 + oa) = make_uint2(bf16x2_rn(p[0], p[1]), bf16x2_rn(p[2], p[3]));
                    *reinterpret_cast<uint2 *>(param_copy + e0 + ob) = make_uint2(bf16x2_rn(p[4], p[5]), bf16x2_rn(p[6], p[7]));
                }
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (j < nva) { param[e0 + oa + j] = p[j]; if (param_copy) param_copy[e0 + oa + j] = (uint16_t)f32_to_bf16_rn_bits(p[j]); }
                    if (j < nvb) { param[e0 + ob + j] = p[j + 4]; if (param_copy) param_copy[e0 + ob + j] = (uint16_t)f32_to_bf16_rn_bits(p[j + 4]); }
                }
            }

            // ---- momentum requantisation of this momentum block (optimizer.py:510, 518) ----
            {
                float amx = 0.0f;
#pragma unroll
                for (int j = 0; j < 8; ++j) amx = fmaxf(amx, fabsf(m[j]));
                const float am = fmaxf(__uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(amx))), 1e-12f);
                const float2 ra2 = bc2(__frcp_rn(am)), nam2 = bc2(-am);
                uint32_t raw[8];
#pragma unroll
                for (int j = 0; j < 8; j += 2) {
                    const float2 mj = make_float2(m[j], m[j + 1]);
                    float2 q = __fmul2_rn(mj, ra2);
                    const float2 r = __ffma2_rn(q, nam2, mj);
                    q = __ffma2_rn(r, ra2, q);
                    const float2 kf = __ffma2_rn(q, bc2(128.0f), bc2(AF8_MAGIC_F));
                    raw[j] = (uint32_t)min(__float_as_int(kf.x), AF8_MAGIC_I + 127);
                    raw[j + 1] = (uint32_t)min(__float_as_int(kf.y), AF8_MAGIC_I + 127);
                }
                const uint32_t o0 = __byte_perm(__byte_perm(raw[0], raw[1], 0x0040), __byte_perm(raw[2], raw[3], 0x0040), 0x5410) ^ 0x80808080u;
                const uint32_t o1 = __byte_perm(__byte_perm(raw[4], raw[5], 0x0040), __byte_perm(raw[6], raw[7], 0x0040), 0x5410) ^ 0x80808080u;
                if (m_exists) {
                    *reinterpret_cast<uint32_t *>(m_q + e0 + oa) = o0;
                    *reinterpret_cast<uint32_t *>(m_q + e0 + ob) = o1;
                    if (lane == 0) m_scale[b * (FAST_VBLOCK / FAST_MBLOCK) + s] = am;
                }
            }
        }

        // ---- block extrema of v (non-negative: bit patterns order like the values); the minimum runs over
        //      the non-zero elements (optimizer.py:312-313) and travels as bits - 1 ----
        uint32_t umin = __reduce_min_sync(0xffffffffu, __float_as_uint(fmn));
        const uint32_t umax = __reduce_max_sync(0xffffffffu, __float_as_uint(fmx));
        if (umin == 0u) {                              // some lane holds a zero: rescan for the smallest non-zero
            uint32_t um = 0xffffffffu;
#pragma unroll
            for (int i = 0; i < 64; ++i) um = min(um, __float_as_uint(vreg[i]) - 1u);
            umin = __reduce_min_sync(0xffffffffu, um);
        } else {
            umin -= 1u;
        }
        // lane 0 takes the exact log2 of the minimum, lane 1 of the maximum (optimizer.py:308-318)
        const float lg = (lane == 0) ? ((umin == 0xffffffffu) ? INFINITY : al_log2_fast(__uint_as_float(umin + 1u), s_log2))
                                     : ((lane == 1) ? al_log2_fast(__uint_as_float(umax), s_log2) : 0.0f);
        const float mn = __shfl_sync(0xffffffffu, lg, 0), mx = __shfl_sync(0xffffffffu, lg, 1);
        VRange r;
        al_range(mn, mx, L.v_floor, r.min_log, r.scale);
        r.k = __fdiv_rn(254.0f, r.scale);
        r.c = -__fmul_rn(r.min_log, r.k);
        {
            const float lmax = fmaxf(fmaxf(fabsf(r.min_log), fabsf(mx)), 1.0f);
            const float err = __fmaf_rn(__fmul_rn(lmax, LG2_REL_BOUND), r.k, 2.0e-4f);
            r.thr = 0.5f - err;
            if (!(r.k >= 1.0f) || L.v_floor < -126.0f || mn < L.v_floor) r.thr = -1.0f;     // exact path for the whole block
        }
        if (lane == 0) {
            v_scale[b] = r.scale;
            v_min_log[b] = r.min_log;
        }
        if (MODE == AF8_MODE_LAG) {
            const float ws = warp_sum(usq);
            if (lane == 0) L.block_sumsq[blk] = ws;
        }

        // ---- second-moment codes ----
        const float2 k2 = bc2(r.k), c2 = bc2(r.c), mg2 = bc2(AF8_MAGIC_F + 1.0f), nmg2 = bc2(-(AF8_MAGIC_F + 1.0f));
#pragma unroll
        for (int s = 0; s < 8; ++s) {
            int kk[8];
            float dd[8];
            float dmax = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; j += 2) {
                const float2 le = make_float2(lg2_approx(vreg[s * 8 + j]), lg2_approx(vreg[s * 8 + j + 1]));
                const float2 te = __ffma2_rn(le, k2, c2);
                const float2 sm = __fadd2_rn(te, mg2);
                const float2 rf = __fadd2_rn(sm, nmg2);
                const float2 d = sub2(te, rf);
                dd[j] = d.x; dd[j + 1] = d.y;
                dmax = fmaxf(dmax, fmaxf(fabsf(d.x), fabsf(d.y)));
                kk[j] = __float_as_int(sm.x); kk[j + 1] = __float_as_int(sm.y);
            }
            if (__any_sync(0xffffffffu, dmax > r.thr)) {
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if (!(fabsf(dd[j]) <= r.thr))
                        kk[j] = AF8_MAGIC_I + (int)al_encode(vreg[s * 8 + j], al_log2_fast(vreg[s * 8 + j], s_log2), r.min_log, r.scale, 254.0f, 255);
            }
            uint32_t raw[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) raw[j] = (uint32_t)kk[j];
            const uint32_t o0 = __byte_perm(__byte_perm(raw[0], raw[1], 0x0040), __byte_perm(raw[2], raw[3], 0x0040), 0x5410);
            const uint32_t o1 = __byte_perm(__byte_perm(raw[4], raw[5], 0x0040), __byte_perm(raw[6], raw[7], 0x0040), 0x5410);
            uint8_t *vp = v_q + base + s * FAST_MBLOCK;
            *reinterpret_cast<uint32_t *>(vp + oa) = o0;
            *reinterpret_cast<uint32_t *>(vp + ob) = o1;
        }
    }
}

}  // namespace af8
