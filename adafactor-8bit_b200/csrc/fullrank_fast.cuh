// Full-rank fused step, specialised kernel: AdamW-style update with UF8
// momentum (M block 256) and AL8 second moment (V block 2048), fp32
// parameters with fp32 or bf16 gradients, or bf16 parameters (rounded to
// nearest or stochastically) with bf16 gradients.
//
// Reference semantics: _update_param_8bit full-rank branch with the Adam
// denominator (optimizer.py:2115-2123), _fallback_1d_update
// (optimizer.py:903-910), _m_ema_pytorch (optimizer.py:690-700), the AL codec
// (optimizer.py:299-353) and the UF8 codec (optimizer.py:504-532).
//
// Work decomposition.  The launch covers a table of tensors; the unit of work
// is one V block (2048 consecutive elements of one tensor).  A persistent grid
// walks the flat block space with a grid stride.  One CTA of 256 threads owns a
// block; warp w owns elements [256w, 256w+256), i.e. exactly M block w, so the
// momentum absmax is a pure warp reduction.  Lane l of the warp owns the two
// 4-element groups at 256w+4l and 256w+128+4l: every shared-memory read and
// every global store of a warp is one contiguous 128/256/512-byte run.
//
// Data movement.  The parameter, gradient and both code arrays of a full block
// are brought into a two-stage shared-memory ring by bulk asynchronous copies
// (cp.async.bulk, completion on an mbarrier).  While block i is being processed
// the copies of block i+1 of the same tensor are already in flight, and the
// 256-entry AL8 decode table of block i+1 is computed while warp 0 derives the
// range of block i.  Tail blocks (fewer than 2048 real elements) and the first
// block a CTA touches in a tensor take a plain-load path.  Every wait on an
// mbarrier is bounded; a wait that runs out raises the device error flag that
// af8_device_status() reports, the threads skip the stores of that block and
// the CTA stops at its next block-wide barrier.
//
// Instruction count.  At 14-16 bytes per parameter the HBM roofline leaves
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

#include <cstddef>

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
    int32_t param_dtype;    // AF8_F32 / AF8_BF16 / AF8_F16
    int32_t sr;             // stochastic rounding of 16-bit parameters
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
struct f16_tag {};
template <> struct GradLoad<f16_tag> {      // (general kernel only)
    static __device__ __forceinline__ float load1(const void *base, int64_t off)
    {
        return f16_bits_to_f32(static_cast<const uint16_t *>(base)[off]);
    }
};
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

// hardware approximations (flush-to-zero forms: one MUFU instruction each, no
// subnormal fix-up code), used only where the result does not reach a stored state
__device__ __forceinline__ float sqrt_approx(float x)
{
    float y;
    asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float rcp_approx(float x)
{
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float lg2_approx(float x)
{
    float y;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
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

// Blackwell packed binary32 arithmetic: one instruction works on a pair of floats held in
// a 64-bit register; each component rounds exactly like the scalar *_rn operation.
__device__ __forceinline__ float2 bc2(float x) { return make_float2(x, x); }
__device__ __forceinline__ float2 sub2(float2 a, float2 b) { return __ffma2_rn(bc2(-1.0f), b, a); }   // a - b, one rounding

// two binary32 numbers rounded to nearest bf16, packed (first one in the low half)
__device__ __forceinline__ uint32_t bf16x2_rn(float lo, float hi)
{
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

template <bool SMALL_W>
__device__ __forceinline__ float lerp_sel(float s, float e, float w, float wm1)
{
    const float d = __fsub_rn(e, s);
    return SMALL_W ? __fmaf_rn(w, d, s) : __fmaf_rn(wm1, d, e);
}

// ---------------------------------------------------------------------------
// device error flag, mbarrier and bulk-copy helpers
// ---------------------------------------------------------------------------
// Set (never cleared by kernels) when a bounded wait ran out.  Read back by
// af8_device_status().
__device__ int g_device_error = 0;
constexpr int DEVERR_COPY_TIMEOUT = 1;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ uint64_t global_timer_ns()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Wait for a phase of the barrier for at most `limit_ns` of wall time (two seconds unless told
// otherwise; a block's copies take microseconds).  Returns false when the time ran out.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity, uint64_t limit_ns = 2000000000ull)
{
    uint64_t t0 = 0;
    for (uint32_t i = 0;; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 0xffu) == 0xffu) {
            const uint64_t now = global_timer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > limit_ns) return false;
        }
    }
}
// global -> shared bulk copy of `bytes` (multiple of 16, both addresses 16-byte
// aligned); completion is signalled on `bar` as transaction bytes.
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

template <typename T> struct ParamElem { typedef float type; };
template <> struct ParamElem<bf16_tag> { typedef uint16_t type; };
template <typename T> struct GradBytes { static constexpr int value = 4; };
template <> struct GradBytes<bf16_tag> { static constexpr int value = 2; };

// ---------------------------------------------------------------------------
// EMAs and update of a thread's 8 elements
// ---------------------------------------------------------------------------
struct StepScalars {
    float decay, v_w, v_wm1, m_w, m_wm1, eps_g, eps_d, step_mul, fira;
    bool zero_upd;
    bool round_decay;   // bf16 parameter, nearest rounding: p*decay is rounded to bf16 before the update is added
};

// MODE: NOCLIP, APPLY (scalars of the statistic pass) or LAG (scalars of the previous step; the sum
// of squares of this step's raw update is added to usq)
template <int MODE, bool HAS_EPSG, bool TAIL>
__device__ __forceinline__ void ema_update(const float (&g)[8], float (&p)[8], const uint32_t (&mq)[2],
                                           const uint32_t (&vq)[2], const float *tab, float mc,
                                           const StepScalars &S, int nva, int nvb, float (&v)[8], float (&m)[8],
                                           float &usq)
{
    constexpr bool DYN = MODE == AF8_MODE_APPLY || MODE == AF8_MODE_LAG;
    const float2 w_v = bc2(S.v_w), w_m = bc2(S.m_w), mc2 = bc2(mc), eps_d2 = bc2(S.eps_d);
    const float2 decay2 = bc2(S.decay), step2 = bc2(S.step_mul), fira2 = bc2(S.fira);
#pragma unroll
    for (int j = 0; j < 8; j += 2) {
        const uint32_t c0 = __byte_perm(vq[j >> 2], 0u, 0x4440u | (uint32_t)(j & 3));
        const uint32_t c1 = __byte_perm(vq[j >> 2], 0u, 0x4440u | (uint32_t)((j + 1) & 3));
        const float2 gj = make_float2(g[j], g[j + 1]);
        // second moment (optimizer.py:2117-2119)
        float2 g2 = __fmul2_rn(gj, gj);
        if (HAS_EPSG) g2 = __fadd2_rn(g2, bc2(S.eps_g));          // 0 in Adam mode (optimizer.py:1967)
        const float2 v_old = make_float2(tab[c0], tab[c1]);
        float2 vj = __ffma2_rn(w_v, sub2(g2, v_old), v_old);
        // momentum (optimizer.py:528-531, 698): (byte - 128) * fl(scale / 128), then lerp
        const float2 mb = make_float2(__uint_as_float(__byte_perm(mq[j >> 2], 0x4b000000u, 0x7540u | (uint32_t)(j & 3))),
                                      __uint_as_float(__byte_perm(mq[j >> 2], 0x4b000000u, 0x7540u | (uint32_t)((j + 1) & 3))));
        const float2 m_old = __fmul2_rn(__fadd2_rn(mb, bc2(-8388736.0f)), mc2);
        float2 mj = __ffma2_rn(w_m, sub2(gj, m_old), m_old);
        bool real0 = true, real1 = true;
        if (TAIL) {
            real0 = (j < 4) ? (j < nva) : (j - 4 < nvb);
            real1 = (j < 4) ? (j + 1 < nva) : (j - 3 < nvb);
            if (!real0) { vj.x = 0.0f; mj.x = 0.0f; }
            if (!real1) { vj.y = 0.0f; mj.y = 0.0f; }
        }
        v[j] = vj.x; v[j + 1] = vj.y; m[j] = mj.x; m[j + 1] = mj.y;
        // update from the un-requantised v and m (optimizer.py:905, 909); feeds the parameter only
        const float2 den = __fadd2_rn(make_float2(sqrt_approx(vj.x), sqrt_approx(vj.y)), eps_d2);
        float2 u = __fmul2_rn(mj, make_float2(rcp_approx(den.x), rcp_approx(den.y)));
        if (TAIL) {                                               // padding (0 * inf when eps is 0)
            if (!real0) u.x = 0.0f;
            if (!real1) u.y = 0.0f;
        }
        float2 pj = __fmul2_rn(make_float2(p[j], p[j + 1]), decay2);     // optimizer.py:2039
        if (S.round_decay) {                                      // Tensor.mul_ on a bf16 tensor rounds to bf16
            const uint32_t pk = bf16x2_rn(pj.x, pj.y);
            pj = make_float2(__uint_as_float(pk << 16), __uint_as_float(pk & 0xffff0000u));
        }
        if (MODE == AF8_MODE_LAG) usq = __fmaf_rn(u.y, u.y, __fmaf_rn(u.x, u.x, usq));
        if (DYN) u = __fmul2_rn(u, fira2);                        // optimizer.py:803
        if (!(DYN && S.zero_upd))                                 // non-finite norm: zero update (optimizer.py:798-800)
            pj = __ffma2_rn(step2, u, pj);                        // optimizer.py:874
        p[j] = pj.x; p[j + 1] = pj.y;
    }
}

// ---------------------------------------------------------------------------
// the kernel
// ---------------------------------------------------------------------------
#ifndef AF8_FAST_MIN_CTAS
#define AF8_FAST_MIN_CTAS 4
#endif
#ifndef AF8_FAST_STAGES_UPDATE
#define AF8_FAST_STAGES_UPDATE 2      /* ring depth of the NOCLIP / APPLY passes, bf16 gradients */
#endif
#ifndef AF8_FAST_STAGES_UPDATE_F32
#define AF8_FAST_STAGES_UPDATE_F32 2  /* the same with fp32 gradients (20 KB per slot) */
#endif

// Measured on B200 (TinyLlama set): depths 2 / 3 / 4 / 6 change the pass times by a few
// per cent in the wrong direction (fewer resident CTAs), so the default stays at 2.
// Ring geometry of one kernel variant: byte offsets inside a slot and the slot count.
template <typename GradT, typename ParamT, int MODE> struct FastRing {
    static constexpr int GB = GradBytes<GradT>::value;
    static constexpr int PB = GradBytes<ParamT>::value;     // bytes per parameter: 4 (float) or 2 (bf16_tag)
    static_assert(MODE == AF8_MODE_NOCLIP || MODE == AF8_MODE_APPLY || MODE == AF8_MODE_LAG, "the statistic pass has its own kernel (fullrank_stat.cuh)");
    static constexpr int P_OFF = 0;
    static constexpr int G_OFF = FAST_VBLOCK * PB;
    static constexpr int MQ_OFF = G_OFF + FAST_VBLOCK * GB;
    static constexpr int VQ_OFF = MQ_OFF + FAST_VBLOCK;
    static constexpr int STAGE_BYTES = VQ_OFF + FAST_VBLOCK;
    static constexpr int NST = GB == 2 ? AF8_FAST_STAGES_UPDATE : AF8_FAST_STAGES_UPDATE_F32;
    static constexpr int SMEM_BYTES = NST * STAGE_BYTES;
    static_assert(NST >= 2 && NST <= 8, "ring depth");
};

template <typename GradT, typename ParamT, int MODE>
__global__ void __launch_bounds__(FAST_THREADS, AF8_FAST_MIN_CTAS)
fullrank_fast_kernel(const FullrankLaunch L)
{
    using Ring = FastRing<GradT, ParamT, MODE>;
    constexpr int GB = Ring::GB;
    constexpr int PB = Ring::PB;
    using PElem = typename ParamElem<ParamT>::type;
    constexpr int P_OFF = Ring::P_OFF, G_OFF = Ring::G_OFF, MQ_OFF = Ring::MQ_OFF, VQ_OFF = Ring::VQ_OFF;
    constexpr int STAGE_BYTES = Ring::STAGE_BYTES;
    constexpr int NST = Ring::NST;

    extern __shared__ __align__(128) unsigned char s_ring[];     // NST slots of STAGE_BYTES
    __shared__ __align__(8) uint64_t s_full[NST];
    __shared__ __align__(16) af8_fullrank_tensor sT;
    __shared__ float s_tab[2][256];
    __shared__ uint32_t s_redmin[FAST_WARPS];
    __shared__ uint32_t s_redmax[FAST_WARPS];
    __shared__ float s_usq[FAST_WARPS];
    __shared__ VRange s_vr;
    __shared__ int s_abort;
    __shared__ double s_exp2[32];            // copy of the exp2 table of the decode
    __shared__ double2 s_log2[97];           // copy of the log2 table of the range computation

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int oa = warp * FAST_MBLOCK + lane * 4;   // first 4-element group of this thread
    const int ob = oa + 128;                         // second group

    if (tid < 32) s_exp2[tid] = c_exp2_tab[tid];
    if (tid < 97) s_log2[tid] = c_log2_tab[tid];
    if (tid == 0) {
        for (int k = 0; k < NST; ++k) mbar_init(&s_full[k], 1);
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    int cur_t = -1;
    int64_t cur_first = 0, cur_end = 0;      // block range of the current tensor
    int nfull = 0;                           // number of full blocks of the current tensor
    const int G = (int)gridDim.x;
    uint32_t phase = 0;                      // bit k: parity to wait for on ring slot k
    int ahead = 0;                           // consecutive blocks from the current one whose copies are in flight
    bool staged = false;                     // this block's decode table and ranges were prepared last iteration
    float nsc = 0.f, nml = 0.f, nms = 0.f;   // prefetched range of the next block (v_scale, v_min_log, m_scale)
    float mscale_cur = 0.f;
    int n = 0;

    for (int64_t blk = blockIdx.x; blk < L.total_blocks; blk += gridDim.x, ++n) {
        // ---- tensor change (rare, uniform over the CTA) ----
        if (cur_t < 0 || blk >= cur_end) {
            int t = cur_t;
            if (t < 0) {
                t = find_tensor(L.tensors, L.n_tensors, blk);
            } else {
                while (t + 1 < L.n_tensors && __ldg(&L.tensors[t + 1].first_block) <= blk) ++t;
            }
            __syncthreads();
            if (tid < (int)(sizeof(af8_fullrank_tensor) / 4))
                reinterpret_cast<uint32_t *>(&sT)[tid] =
                    __ldg(reinterpret_cast<const uint32_t *>(L.tensors + t) + tid);
            __syncthreads();
            cur_t = t;
            cur_first = sT.first_block;
            cur_end = cur_first + (sT.numel + FAST_VBLOCK - 1) / FAST_VBLOCK;
            nfull = (int)(sT.numel / FAST_VBLOCK);   // a tensor has fewer than 2^31 blocks (checked on the host)
            staged = false;                          // (ahead is 0 here: copies never cross a tensor)
        }
        const int b = (int)(blk - cur_first);         // V block index inside the tensor
        const int64_t base = (int64_t)b * FAST_VBLOCK;   // first element of the block
        const bool full = b < nfull;
        const int64_t rem = full ? FAST_VBLOCK : sT.numel - base;   // real elements from base on (> 0), capped
        const int stage = n & 1;                      // decode-table / partial-sum buffer of this block
        const int slot = n % NST;                     // ring slot of this block
        const int b_next = b + G;
        // blocks blk, blk+G, ... that are full blocks of this tensor get their copies issued ahead
        int want = 0;
#pragma unroll
        for (int k = 0; k < NST; ++k)
            if (want == k && b + k * G < nfull) want = k + 1;
        const bool next_staged = want >= 2;           // the next block gets its table and ranges prepared here

        // ---- issue the bulk copies (one thread) ----
        if (tid == 0 && ahead < want) {
            const unsigned char *gp = static_cast<const unsigned char *>(sT.grad);
            const unsigned char *pp = static_cast<const unsigned char *>(sT.param);
            const unsigned char *vp = static_cast<const unsigned char *>(sT.v_q);
            fence_proxy_async();
            for (int k = ahead; k < want; ++k) {
                const int64_t nb = (int64_t)(b + k * G) * FAST_VBLOCK;
                const int sl = (n + k) % NST;
                unsigned char *dst = s_ring + sl * STAGE_BYTES;
                mbar_expect_tx(&s_full[sl], STAGE_BYTES);
                bulk_g2s(dst + P_OFF, pp + nb * PB, FAST_VBLOCK * PB, &s_full[sl]);
                bulk_g2s(dst + G_OFF, gp + nb * GB, FAST_VBLOCK * GB, &s_full[sl]);
                bulk_g2s(dst + MQ_OFF, sT.m_q + nb, FAST_VBLOCK, &s_full[sl]);
                bulk_g2s(dst + VQ_OFF, vp + nb, FAST_VBLOCK, &s_full[sl]);
            }
        }
        const int in_flight = want;                   // copies outstanding now, this block included
        ahead = want > 0 ? want - 1 : 0;              // ... as seen from the next block
        // ---- ranges of this block (if not prefetched) and of the next one ----
        const bool m_exists = (int64_t)warp * FAST_MBLOCK < rem;   // this warp's M block is allocated
        if (!staged) {
            const float sc = __ldg(sT.v_scale + b);
            const float ml = __ldg(sT.v_min_log + b);
            mscale_cur = m_exists ? __ldg(sT.m_scale + b * (FAST_VBLOCK / FAST_MBLOCK) + warp) : 0.0f;
            s_tab[stage][tid] = al8_decode_fast((uint32_t)tid, sc, ml, s_exp2);   // optimizer.py:341-349
            __syncthreads();
        }
        if (next_staged) {
            nsc = __ldg(sT.v_scale + b_next);
            nml = __ldg(sT.v_min_log + b_next);
            nms = __ldg(sT.m_scale + b_next * (FAST_VBLOCK / FAST_MBLOCK) + warp);
        }
        // fl(m_scale / 128) (optimizer.py:531): a power-of-two divisor, so the product is the
        // same number (m_scale >= 1e-12 keeps it far from the subnormal range)
        const float mc = __fmul_rn(mscale_cur, 0.0078125f);

        // ---- this thread's raw inputs ----
        float p[8], g[8];
        uint32_t mq[2], vq[2];
        int nva = 4, nvb = 4;
        bool bad = false;
        // (typed pointers: with byte pointers and a scaled offset the update pass ran 2.5 % slower)
        PElem *pa = static_cast<PElem *>(sT.param) + base + oa;
        PElem *pb = static_cast<PElem *>(sT.param) + base + ob;
        if (full) {
            if (!mbar_wait_bounded(&s_full[slot], (phase >> slot) & 1u)) {
                bad = true;      // this thread stores nothing for the block
                s_abort = 1;     // and the CTA stops at the next block-wide barrier
                atomicExch(&g_device_error, DEVERR_COPY_TIMEOUT);
            }
            phase ^= 1u << slot;
            const unsigned char *st = s_ring + slot * STAGE_BYTES;
            if (PB == 4) {
                const float4 a = *reinterpret_cast<const float4 *>(st + P_OFF + oa * 4);
                const float4 c = *reinterpret_cast<const float4 *>(st + P_OFF + ob * 4);
                p[0] = a.x; p[1] = a.y; p[2] = a.z; p[3] = a.w;
                p[4] = c.x; p[5] = c.y; p[6] = c.z; p[7] = c.w;
            } else {
                const uint2 a = *reinterpret_cast<const uint2 *>(st + P_OFF + oa * 2);
                const uint2 c = *reinterpret_cast<const uint2 *>(st + P_OFF + ob * 2);
                p[0] = __uint_as_float(a.x << 16); p[1] = __uint_as_float(a.x & 0xffff0000u);
                p[2] = __uint_as_float(a.y << 16); p[3] = __uint_as_float(a.y & 0xffff0000u);
                p[4] = __uint_as_float(c.x << 16); p[5] = __uint_as_float(c.x & 0xffff0000u);
                p[6] = __uint_as_float(c.y << 16); p[7] = __uint_as_float(c.y & 0xffff0000u);
            }
            if (GB == 4) {
                const float4 a = *reinterpret_cast<const float4 *>(st + G_OFF + oa * 4);
                const float4 c = *reinterpret_cast<const float4 *>(st + G_OFF + ob * 4);
                g[0] = a.x; g[1] = a.y; g[2] = a.z; g[3] = a.w;
                g[4] = c.x; g[5] = c.y; g[6] = c.z; g[7] = c.w;
            } else {
                const uint2 a = *reinterpret_cast<const uint2 *>(st + G_OFF + oa * 2);
                const uint2 c = *reinterpret_cast<const uint2 *>(st + G_OFF + ob * 2);
                g[0] = __uint_as_float(a.x << 16); g[1] = __uint_as_float(a.x & 0xffff0000u);
                g[2] = __uint_as_float(a.y << 16); g[3] = __uint_as_float(a.y & 0xffff0000u);
                g[4] = __uint_as_float(c.x << 16); g[5] = __uint_as_float(c.x & 0xffff0000u);
                g[6] = __uint_as_float(c.y << 16); g[7] = __uint_as_float(c.y & 0xffff0000u);
            }
            mq[0] = *reinterpret_cast<const uint32_t *>(st + MQ_OFF + oa);
            mq[1] = *reinterpret_cast<const uint32_t *>(st + MQ_OFF + ob);
            vq[0] = *reinterpret_cast<const uint32_t *>(st + VQ_OFF + oa);
            vq[1] = *reinterpret_cast<const uint32_t *>(st + VQ_OFF + ob);
        } else {
            // tail block: guarded plain loads; the V state is padded to the block, the M
            // state only to its own 256-element blocks
            nva = (int)max((int64_t)0, min((int64_t)4, rem - oa));
            nvb = (int)max((int64_t)0, min((int64_t)4, rem - ob));
            const uint8_t *vp = static_cast<const uint8_t *>(sT.v_q) + base;
            vq[0] = *reinterpret_cast<const uint32_t *>(vp + oa);
            vq[1] = *reinterpret_cast<const uint32_t *>(vp + ob);
            mq[0] = m_exists ? *reinterpret_cast<const uint32_t *>(sT.m_q + base + oa) : 0x80808080u;
            mq[1] = m_exists ? *reinterpret_cast<const uint32_t *>(sT.m_q + base + ob) : 0x80808080u;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int e = (j < 4) ? oa + j : ob + j - 4;
                const bool ok = (j < 4) ? (j < nva) : (j - 4 < nvb);
                p[j] = ok ? param_load(sT.param, base + e, PB == 4 ? AF8_F32 : AF8_BF16) : 0.0f;
                g[j] = ok ? GradLoad<GradT>::load1(sT.grad, base + e) : 0.0f;
            }
        }
        if (L.negate_grad) {
#pragma unroll
            for (int j = 0; j < 8; ++j) g[j] = -g[j];
        }

        // ---- scalars of the step ----
        StepScalars S;
        {   // three vector loads instead of six scalar ones (the descriptor is 16-byte aligned)
            static_assert(offsetof(af8_fullrank_tensor, decay) % 8 == 0 && offsetof(af8_fullrank_tensor, v_w) % 16 == 0 &&
                          offsetof(af8_fullrank_tensor, m_w) == offsetof(af8_fullrank_tensor, v_w) + 12 &&
                          offsetof(af8_fullrank_tensor, eps_gradsq) % 8 == 0 &&
                          offsetof(af8_fullrank_tensor, eps_denom) == offsetof(af8_fullrank_tensor, eps_gradsq) + 4, "descriptor layout");
            const float2 da = *reinterpret_cast<const float2 *>(&sT.decay);
            const float4 vw = *reinterpret_cast<const float4 *>(&sT.v_w);
            const float2 ep = *reinterpret_cast<const float2 *>(&sT.eps_gradsq);
            S.decay = da.x; S.step_mul = -da.y; S.v_w = vw.x; S.m_w = vw.w; S.eps_g = ep.x; S.eps_d = ep.y;
        }
        S.v_wm1 = __fsub_rn(S.v_w, 1.0f); S.m_wm1 = __fsub_rn(S.m_w, 1.0f);
        S.fira = 1.0f; S.zero_upd = false;
        S.round_decay = PB == 2 && !L.sr;
        constexpr bool DYN = MODE == AF8_MODE_APPLY || MODE == AF8_MODE_LAG;
        float usq = 0.0f;                    // LAG: this thread's sum of squares of the raw update
        if (DYN) {
            const af8_dyn_scalars ds = L.dyn[cur_t];
            S.step_mul = ds.step; S.fira = ds.fira; S.zero_upd = ds.zero != 0.0f;
        }

        // ---- EMAs and update: everything that reaches a state is exact ----
        float v[8], m[8];
        const bool small_w = fabsf(S.v_w) < 0.5f && fabsf(S.m_w) < 0.5f;   // ATen's lerp has two forms
        if (small_w) {
            if (full) {
                if (S.eps_g == 0.0f) ema_update<MODE, false, false>(g, p, mq, vq, s_tab[stage], mc, S, nva, nvb, v, m, usq);
                else ema_update<MODE, true, false>(g, p, mq, vq, s_tab[stage], mc, S, nva, nvb, v, m, usq);
            } else {
                ema_update<MODE, true, true>(g, p, mq, vq, s_tab[stage], mc, S, nva, nvb, v, m, usq);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) {   // general lerp (weights >= 0.5): rare, kept simple
                const bool real = (j < 4) ? (j < nva) : (j - 4 < nvb);
                const uint32_t vcode = (vq[j >> 2] >> (8 * (j & 3))) & 0xffu;
                const float g2 = __fadd_rn(__fmul_rn(g[j], g[j]), S.eps_g);
                float vj = lerp_t(s_tab[stage][vcode], g2, S.v_w);
                float mj = lerp_t(__fmul_rn(byte_minus_128(mq[j >> 2], j & 3), mc), g[j], S.m_w);
                if (!real) { vj = 0.0f; mj = 0.0f; }
                v[j] = vj; m[j] = mj;
                float u = __fmul_rn(mj, rcp_approx(__fadd_rn(sqrt_approx(vj), S.eps_d)));
                if (!real) u = 0.0f;
                float pj = __fmul_rn(p[j], S.decay);
                if (S.round_decay) pj = param_round(pj, AF8_BF16);
                if (MODE == AF8_MODE_LAG) usq = __fmaf_rn(u, u, usq);
                const float us = DYN ? __fmul_rn(u, S.fira) : u;
                if (!(DYN && S.zero_upd)) pj = __fmaf_rn(S.step_mul, us, pj);
                p[j] = pj;
            }
        }

        // ---- block extrema of v.  v >= 0, so the bit patterns order like the values.  The
        //      minimum runs over the non-zero elements (optimizer.py:312-313) and travels as
        //      bits-1, which sends "none" to the top; a warp that holds a zero (rare after the
        //      first steps, except in all-zero regions) rescans its registers for it ----
        {
            float fmn = v[0], fmx = v[0];
#pragma unroll
            for (int j = 1; j < 8; ++j) {
                fmn = fminf(fmn, v[j]);
                fmx = fmaxf(fmx, v[j]);
            }
            uint32_t umin = __reduce_min_sync(0xffffffffu, __float_as_uint(fmn));
            const uint32_t umax = __reduce_max_sync(0xffffffffu, __float_as_uint(fmx));
            if (umin == 0u) {                                    // uniform over the warp
                uint32_t um = 0xffffffffu;
#pragma unroll
                for (int j = 0; j < 8; ++j) um = min(um, __float_as_uint(v[j]) - 1u);
                umin = __reduce_min_sync(0xffffffffu, um);
            } else {
                umin -= 1u;
            }
            if (lane == 0) { s_redmin[warp] = umin; s_redmax[warp] = umax; }
            if (MODE == AF8_MODE_LAG) {      // the block's sum of squares travels with the extrema
                const float ws = warp_sum(usq);
                if (lane == 0) s_usq[warp] = ws;
            }
        }
        // ---- D: only warp 0 consumes the extrema; the other warps signal and move on ----
        if (warp == 0) asm volatile("bar.sync 1, %0;" ::"n"(FAST_THREADS) : "memory");
        else asm volatile("bar.arrive 1, %0;" ::"n"(FAST_THREADS) : "memory");

        // ---- warp 0: exact log2 of the two extreme values only (optimizer.py:308-318) ----
        if (warp == 0) {
            uint32_t umin = lane < FAST_WARPS ? s_redmin[lane] : 0xffffffffu;
            uint32_t umax = lane < FAST_WARPS ? s_redmax[lane] : 0u;
            umin = __reduce_min_sync(0xffffffffu, umin);
            umax = __reduce_max_sync(0xffffffffu, umax);
            // lane 0 takes the log of the minimum, lane 1 of the maximum
            float lg = (lane == 0) ? ((umin == 0xffffffffu) ? INFINITY : al_log2_fast(__uint_as_float(umin + 1u), s_log2))
                                   : ((lane == 1) ? al_log2_fast(__uint_as_float(umax), s_log2) : 0.0f);
            const float mx_l = __shfl_sync(0xffffffffu, lg, 1);
            if (lane == 0) {
                const float mn = lg;
                const float mx = mx_l;
                VRange r;
                al_range(mn, mx, L.v_floor, r.min_log, r.scale);
                r.k = __fdiv_rn(254.0f, r.scale);
                r.c = -__fmul_rn(r.min_log, r.k);
                // error bound of the estimate in code units: the hardware log2, the roundings
                // of the estimate and those of the exact sequence it must agree with
                const float lmax = fmaxf(fmaxf(fabsf(r.min_log), fabsf(mx)), 1.0f);
                const float err = __fmaf_rn(__fmul_rn(lmax, LG2_REL_BOUND), r.k, 2.0e-4f);
                r.thr = 0.5f - err;
                // Exact path for every element of the block when the range is absurd (NaN / inf)
                // or when some non-zero element lies below the floor (subnormal values with the
                // default floor): the estimate path has no lower clamp and flushes subnormals.
                if (!(r.k >= 1.0f) || L.v_floor < -126.0f || mn < L.v_floor) r.thr = -1.0f;
                s_vr = r;
                sT.v_scale[b] = r.scale;
                sT.v_min_log[b] = r.min_log;
                if (MODE == AF8_MODE_LAG) {
                    float s = 0.0f;
#pragma unroll
                    for (int w = 0; w < FAST_WARPS; ++w) s = __fadd_rn(s, s_usq[w]);
                    L.block_sumsq[blk] = s;
                }
            }
        }

        // ---- parameter store ----
        if (bad) {
        } else if (PB == 4 && full) {
            *reinterpret_cast<float4 *>(pa) = make_float4(p[0], p[1], p[2], p[3]);
            *reinterpret_cast<float4 *>(pb) = make_float4(p[4], p[5], p[6], p[7]);
        } else if (PB == 4) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (j < nva) pa[j] = p[j];
                if (j < nvb) pb[j] = p[j + 4];
            }
        } else {
            // bf16 parameters: the last rounding, to nearest or stochastic (optimizer.py:873-881)
            uint32_t w[4];
            if (L.sr) {
                uint32_t h[8];
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    h[j] = sr_bf16_bits(p[j], sr_bits24(sT.sr_base, (uint64_t)(base + ((j < 4) ? oa + j : ob + j - 4))));
#pragma unroll
                for (int j = 0; j < 4; ++j) w[j] = h[2 * j] | (h[2 * j + 1] << 16);
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) w[j] = bf16x2_rn(p[2 * j], p[2 * j + 1]);
            }
            if (full) {
                *reinterpret_cast<uint2 *>(pa) = make_uint2(w[0], w[1]);
                *reinterpret_cast<uint2 *>(pb) = make_uint2(w[2], w[3]);
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint32_t ha = (j & 1) ? (w[j >> 1] >> 16) : (w[j >> 1] & 0xffffu);
                    const uint32_t hb = (j & 1) ? (w[2 + (j >> 1)] >> 16) : (w[2 + (j >> 1)] & 0xffffu);
                    if (j < nva) pa[j] = (PElem)ha;
                    if (j < nvb) pb[j] = (PElem)hb;
                }
            }
        }

        // ---- optional bf16 compute copy of the fp32 parameter (round to nearest) ----
        if (PB == 4 && !bad && sT.param_copy != nullptr) {
            uint16_t *ca = static_cast<uint16_t *>(sT.param_copy) + base + oa;
            uint16_t *cb = static_cast<uint16_t *>(sT.param_copy) + base + ob;
            if (full) {
                *reinterpret_cast<uint2 *>(ca) = make_uint2(bf16x2_rn(p[0], p[1]), bf16x2_rn(p[2], p[3]));
                *reinterpret_cast<uint2 *>(cb) = make_uint2(bf16x2_rn(p[4], p[5]), bf16x2_rn(p[6], p[7]));
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (j < nva) ca[j] = (uint16_t)f32_to_bf16_rn_bits(p[j]);
                    if (j < nvb) cb[j] = (uint16_t)f32_to_bf16_rn_bits(p[j + 4]);
                }
            }
        }

        // ---- momentum requantisation: one warp = one M block (optimizer.py:510, 518) ----
        {
            float amx = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j) amx = fmaxf(amx, fabsf(m[j]));
            // non-negative floats order like their bit patterns: one REDUX instead of a shuffle tree
            const float am = fmaxf(__uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(amx))), 1e-12f);
            const float2 ra2 = bc2(__frcp_rn(am)), nam2 = bc2(-am);
            uint32_t raw[8];
#pragma unroll
            for (int j = 0; j < 8; j += 2) {
                // IEEE m / am from the correctly rounded reciprocal and one residual step
                const float2 mj = make_float2(m[j], m[j + 1]);
                float2 q = __fmul2_rn(mj, ra2);
                const float2 r = __ffma2_rn(q, nam2, mj);
                q = __ffma2_rn(r, ra2, q);
                // round(q * 128) (the product is exact); |q| <= 1, so only +128 needs the clamp to 127
                const float2 kf = __ffma2_rn(q, bc2(128.0f), bc2(AF8_MAGIC_F));
                raw[j] = (uint32_t)min(__float_as_int(kf.x), AF8_MAGIC_I + 127);
                raw[j + 1] = (uint32_t)min(__float_as_int(kf.y), AF8_MAGIC_I + 127);
            }
            // low bytes hold k mod 256; k + 128 is that byte with its top bit flipped
            const uint32_t o0 = __byte_perm(__byte_perm(raw[0], raw[1], 0x0040), __byte_perm(raw[2], raw[3], 0x0040), 0x5410) ^ 0x80808080u;
            const uint32_t o1 = __byte_perm(__byte_perm(raw[4], raw[5], 0x0040), __byte_perm(raw[6], raw[7], 0x0040), 0x5410) ^ 0x80808080u;
            if (m_exists && !bad) {
                *reinterpret_cast<uint32_t *>(sT.m_q + base + oa) = o0;
                *reinterpret_cast<uint32_t *>(sT.m_q + base + ob) = o1;
                if (lane == 0) sT.m_scale[b * (FAST_VBLOCK / FAST_MBLOCK) + warp] = am;
            }
        }

        // ---- decode table of the next block, while warp 0 finishes the range ----
        if (next_staged) s_tab[stage ^ 1][tid] = al8_decode_fast((uint32_t)tid, nsc, nml, s_exp2);
        __syncthreads();                     // ---- E ----
        if (s_abort) {       // a copy never completed: give the ones still in flight a bounded chance, then stop
            for (int k = 1; k < in_flight; ++k) mbar_wait_bounded(&s_full[(n + k) % NST], (phase >> ((n + k) % NST)) & 1u);
            break;
        }

        // ---- second-moment codes ----
        {
            const VRange r = s_vr;
            int kk[8];
            float dd[8];
            float dmax = 0.0f;
            const float2 k2 = bc2(r.k), c2 = bc2(r.c), mg2 = bc2(AF8_MAGIC_F + 1.0f), nmg2 = bc2(-(AF8_MAGIC_F + 1.0f));
#pragma unroll
            for (int j = 0; j < 8; j += 2) {
                // An exact zero estimates as -inf: te and sm are -inf, whose low byte is 0, the
                // reserved code, and d is NaN, which the tests below ignore.  Every other element
                // of a block that takes this path is a normal number at or above min_log, so
                // 0 <= t <= 254 up to the estimate's error and no clamp is needed.
                const float2 le = make_float2(lg2_approx(v[j]), lg2_approx(v[j + 1]));
                const float2 te = __ffma2_rn(le, k2, c2);
                const float2 sm = __fadd2_rn(te, mg2);             // rint(te) + 1 in the low bits
                const float2 rf = __fadd2_rn(sm, nmg2);
                const float2 d = sub2(te, rf);                     // distance to the chosen integer
                dd[j] = d.x; dd[j + 1] = d.y;
                dmax = fmaxf(dmax, fmaxf(fabsf(d.x), fabsf(d.y)));   // fmaxf drops NaN
                kk[j] = __float_as_int(sm.x); kk[j + 1] = __float_as_int(sm.y);
            }
            if (__any_sync(0xffffffffu, dmax > r.thr)) {
                // rare: redo the codes in doubt (and the zeros of this thread) with the exact sequence
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if (!(fabsf(dd[j]) <= r.thr))
                        kk[j] = AF8_MAGIC_I + (int)al_encode(v[j], al_log2_fast(v[j], s_log2), r.min_log, r.scale, 254.0f, 255);
            }
            uint32_t raw[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) raw[j] = (uint32_t)kk[j];
            const uint32_t o0 = __byte_perm(__byte_perm(raw[0], raw[1], 0x0040), __byte_perm(raw[2], raw[3], 0x0040), 0x5410);
            const uint32_t o1 = __byte_perm(__byte_perm(raw[4], raw[5], 0x0040), __byte_perm(raw[6], raw[7], 0x0040), 0x5410);
            uint8_t *vp = static_cast<uint8_t *>(sT.v_q) + base;
            *reinterpret_cast<uint32_t *>(vp + oa) = o0;       // (not reached after a failed wait: the CTA left at E)
            *reinterpret_cast<uint32_t *>(vp + ob) = o1;
        }
        staged = next_staged;
        mscale_cur = nms;
    }
}

}  // namespace af8
