/*
 * af8_oracle.c -- CPU restatement of the reference optimizer's pure-PyTorch
 * numerics (adafactor8bit/optimizer.py, the path taken with
 * use_cuda_kernel=False).
 *
 * THIS FILE IS TEST INFRASTRUCTURE.  It is the checker that the CUDA library
 * is compared against and the CPU baseline that the benchmark times.  Nothing
 * in the shipped package may call it.
 *
 * Every function cites the reference lines it follows, as
 * "optimizer.py:<first>-<last>".
 *
 * Arithmetic conventions (they restate what torch's CPU kernels compute):
 *   - all tensor arithmetic is IEEE binary32 with one rounding per torch op;
 *     this file must be compiled with -ffp-contract=off and without fast-math
 *     so that the only fused multiply-adds are the explicit fmaf() calls;
 *   - Tensor.lerp_(end, w)      = w < 0.5 ? fma(w, end-x, x)
 *                                         : fma(w-1, end-x, end)
 *   - Tensor.add_(u, alpha=s)   = fma(s, u, x)
 *   - Tensor.addcmul_(a,b,value=s) = fma(fl(s*a), b, x)
 *   - torch.round               = round-half-to-even (rintf in the default
 *                                 rounding mode)
 *   - torch.rsqrt(x)            = fl(1 / fl(sqrt(x)))
 *   - torch.log2 / torch.pow(2, x) are restated as the correctly rounded
 *     functions (evaluated in binary64, rounded once to binary32).  torch's own
 *     vector math differs from that by one ulp on a small share of inputs,
 *     which is inside the parity tolerances and is measured by the golden
 *     fixture tests.
 *   - full-tensor reductions (norms, means) accumulate in binary64 and round
 *     once; torch's float accumulation order is not reproduced.
 *
 * Parity status: pinned against outputs of the reference itself, produced by
 * tests/golden/gen_golden.py (which imports the reference package) and stored
 * as fixtures under tests/golden/.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <float.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define AF8O_API __attribute__((visibility("default")))

/* optimizer.py:23 */
#define LOG_QUANT_FLOOR 1.17549435e-38f

/* state formats */
enum { AF8O_V_FP32 = 0, AF8O_V_AL8 = 8, AF8O_V_AL16 = 16, AF8O_V_NONE = 1 };   /* NONE: the SGD mode, no second moment */
enum { AF8O_M_NONE = 0, AF8O_M_UF8 = 1, AF8O_M_UF4 = 2, AF8O_M_D8 = 3, AF8O_M_D4 = 4, AF8O_M_FP32 = 5 };
enum { AF8O_G_F32 = 0, AF8O_G_BF16 = 1, AF8O_G_F16 = 2 };  /* gradient and parameter formats */

AF8O_API int af8o_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

AF8O_API void af8o_set_num_threads(int n)
{
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* ------------------------------------------------------------------ */
/* scalar primitives                                                   */
/* ------------------------------------------------------------------ */
static inline float bf16_to_f32(uint16_t h)
{
    uint32_t u = ((uint32_t)h) << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

static inline float log2_cr(float x) { return (float)log2((double)x); }
static inline float pow2_cr(float x) { return (float)exp2((double)x); }
static inline float rsqrt_t(float x) { return 1.0f / sqrtf(x); }

/* Tensor.lerp_ (optimizer.py:698, 2119, 2234) */
static inline float lerp_t(float s, float e, float w)
{
    float d = e - s;
    return (fabsf(w) < 0.5f) ? fmaf(w, d, s) : fmaf(w - 1.0f, d, e);
}

static inline float f16_to_f32(uint16_t h)
{
    _Float16 x;
    memcpy(&x, &h, 2);
    return (float)x;
}

static inline float load_grad(const void *g, int dtype, int64_t i, int negate)
{
    float x = (dtype == AF8O_G_BF16) ? bf16_to_f32(((const uint16_t *)g)[i])
            : (dtype == AF8O_G_F16)  ? f16_to_f32(((const uint16_t *)g)[i])
                                     : ((const float *)g)[i];
    return negate ? -x : x;
}

/* ------------------------------------------------------------------ */
/* low-precision parameters and stochastic rounding                    */
/* ------------------------------------------------------------------ */

/* Tensor.to(torch.bfloat16) of a binary32 value: round to nearest even, NaN -> quiet NaN */
static inline uint16_t f32_to_bf16_rn(float x)
{
    uint32_t b;
    memcpy(&b, &x, 4);
    if ((b & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((b >> 16) | 0x0040u);
    b += 0x7fffu + ((b >> 16) & 1u);
    return (uint16_t)(b >> 16);
}
static inline uint16_t f32_to_f16_rn(float x)
{
    _Float16 h = (_Float16)x;
    uint16_t b;
    memcpy(&b, &h, 2);
    return b;
}

/* _stochastic_round_bf16_pytorch (optimizer.py:162-219): x lies between the bf16 numbers lo
 * (truncation) and hi = lo + one unit; hi is taken when rand < (x - lo) / (hi - lo).  No
 * step up out of an infinity or into one (finite overflow saturates); NaN keeps its sign. */
AF8O_API uint16_t af8o_sr_bf16(float x, float rnd)
{
    uint32_t b;
    memcpy(&b, &x, 4);
    const uint32_t lo = b & 0xffff0000u;
    const int is_nan = (b & 0x7f800000u) == 0x7f800000u && (b & 0x007fffffu) != 0;
    if (is_nan) return (uint16_t)(((b & 0x80000000u) | 0x7fc00000u) >> 16);
    const uint32_t hi = lo + 0x00010000u;
    const int lo_inf = (lo & 0x7f800000u) == 0x7f800000u;
    const int hi_inf = (hi & 0x7f800000u) == 0x7f800000u && (hi & 0x007fffffu) == 0;
    const int can_up = (b & 0xffffu) != 0 && !lo_inf && !hi_inf;
    if (!can_up) return (uint16_t)(lo >> 16);
    float flo, fhi;
    memcpy(&flo, &lo, 4);
    memcpy(&fhi, &hi, 4);
    const float prob = (x - flo) / (fhi - flo);
    return (uint16_t)(((rnd < prob) ? hi : lo) >> 16);
}

/* _stochastic_round_fp16_pytorch (optimizer.py:222-283): the two fp16 neighbours of x are found
 * from the nearest one; overflow saturates at the largest finite value, infinities and NaNs keep
 * their sign. */
AF8O_API uint16_t af8o_sr_f16(float x, float rnd)
{
    uint32_t xb;
    memcpy(&xb, &x, 4);
    const uint16_t sign = (xb & 0x80000000u) ? 0x8000u : 0u;
    if (x != x) return (uint16_t)(sign | 0x7e00u);
    if (isinf(x)) return (uint16_t)(sign | 0x7c00u);
    if (fabsf(x) > 65504.0f) return (uint16_t)(sign | 0x7bffu);
    const uint16_t q = f32_to_f16_rn(x);
    const float qf = f16_to_f32(q);
    if (qf == x) return q;
    uint16_t up, down;
    if (q == 0x8000u) up = 0x0001u; else up = (q & 0x8000u) ? (uint16_t)(q - 1) : (uint16_t)(q + 1);
    if (q == 0x0000u) down = 0x8001u; else down = (q & 0x8000u) ? (uint16_t)(q + 1) : (uint16_t)(q - 1);
    const uint16_t lo_b = (qf < x) ? q : down;
    const uint16_t hi_b = (qf < x) ? up : q;
    const float lo = f16_to_f32(lo_b), hi = f16_to_f32(hi_b);
    const float span = hi - lo;
    if (span == 0.0f) return lo_b;
    const float prob = (x - lo) / span;
    return (rnd < prob) ? hi_b : lo_b;
}

/* The uniform number of element idx: a counter-based generator, so that every element draws
 * independently of the launch geometry.  The counter mixes the per-parameter seed and the step
 * with the two odd constants of the reference's seeded stream (optimizer.py:205); the SplitMix64
 * finaliser (Steele, Lea, Flood 2014) of counter + golden-gamma gives 64 bits, of which the top
 * 24 become a number in [0, 1) (kernels.cu:48-65). */
AF8O_API float af8o_sr_uniform(uint64_t seed, uint64_t step, uint64_t idx)
{
    uint64_t z = seed * 0x9E3779B97F4A7C15ull + step * 0xD1B54A32D192ED03ull + idx;
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    return (float)((uint32_t)(z >> 32) >> 8) * (1.0f / 16777216.0f);
}

/* Format of the parameter tensor that the next step call updates.  The parameter array of every
 * step function holds binary32 numbers; for a bf16 / fp16 parameter they are the exactly
 * representable values, and every write rounds to that format.  (A process-wide setting: the
 * oracle steps one tensor at a time.) */
static struct {
    int32_t dtype;        /* AF8O_G_F32 / AF8O_G_BF16 / AF8O_G_F16 */
    int32_t sr;           /* stochastic_round_writeback and a low-precision parameter (optimizer.py:2032) */
    uint64_t seed, step;  /* state["sr_seed"], state["step"] (optimizer.py:2040) */
    float decay;          /* decay_factor of the step under way (optimizer.py:2036) */
} g_pf = {AF8O_G_F32, 0, 0, 0, 1.0f};

AF8O_API void af8o_set_param_format(int32_t dtype, int32_t sr, uint64_t seed, uint64_t step)
{
    g_pf.dtype = dtype;
    g_pf.sr = sr && dtype != AF8O_G_F32;
    g_pf.seed = seed;
    g_pf.step = step;
    g_pf.decay = 1.0f;
}

/* one-step-lag clipping / limiter for the next step call (see apply_update) */
static struct { int32_t on; float prev_norm, fira_scale; } g_lag = {0, 0.0f, 1.0f};

AF8O_API void af8o_set_lag(int32_t on, float prev_norm, float fira_scale)
{
    g_lag.on = on;
    g_lag.prev_norm = prev_norm;
    g_lag.fira_scale = fira_scale;
}

static inline float round_param(float x)
{
    if (g_pf.dtype == AF8O_G_BF16) return bf16_to_f32(f32_to_bf16_rn(x));
    if (g_pf.dtype == AF8O_G_F16) return f16_to_f32(f32_to_f16_rn(x));
    return x;
}

/* weight decay (optimizer.py:2033-2039): param.mul_(1 - wd_mult*wd) in the parameter's own
 * format, or, under stochastic rounding, a factor kept for the write (optimizer.py:2036) */
static inline float decay_param(float p, int has_decay, float decay)
{
    if (!has_decay || g_pf.sr) return p;
    return round_param(p * decay);
}
static void note_decay(int has_decay, float decay) { g_pf.decay = has_decay ? decay : 1.0f; }

/* the write of _apply_update_pytorch (optimizer.py:873-881): p + s*u in binary32, then the
 * parameter's format (nearest, or stochastic after the folded decay) */
static inline float write_param(float p, float s, float u, int64_t i)
{
    if (!g_pf.sr) return round_param(fmaf(s, u, p));
    float pf = p * g_pf.decay;                           /* optimizer.py:878 */
    pf = fmaf(s, u, pf);                                 /* optimizer.py:879 */
    const float rnd = af8o_sr_uniform(g_pf.seed, g_pf.step, (uint64_t)i);
    return (g_pf.dtype == AF8O_G_BF16) ? bf16_to_f32(af8o_sr_bf16(pf, rnd)) : f16_to_f32(af8o_sr_f16(pf, rnd));
}

/* ------------------------------------------------------------------ */
/* AL codec: adaptive log-space, code 0 reserved for exact zero        */
/* ------------------------------------------------------------------ */

/* One block of _log_quantize_nonneg (optimizer.py:299-325).  x holds the
 * `valid` real elements of the block; the remaining block-valid elements are
 * the zero padding that torch.nn.functional.pad appends (optimizer.py:303-305). */
static void al_quant_block(const float *x, int64_t valid, int64_t block,
                           float floor_log, int bits, void *q_out,
                           float *scale_out, float *min_log_out)
{
    const float qm1 = (bits == 16) ? 65534.0f : 254.0f;  /* q_max - 1 */
    const float qmax = (bits == 16) ? 65535.0f : 255.0f;
    const float l_zero = log2_cr(1e-38f);                 /* clamp(min=1e-38) */
    float mn = INFINITY, mx = -INFINITY;
    for (int64_t i = 0; i < block; ++i) {
        float v = (i < valid) ? x[i] : 0.0f;
        int is_zero = (v == 0.0f);
        float vs = (v < 1e-38f) ? 1e-38f : v;             /* optimizer.py:309 */
        float l = (vs == 1e-38f) ? l_zero : log2_cr(vs);  /* optimizer.py:310 */
        if (!is_zero && l < mn) mn = l;                   /* optimizer.py:312 */
        if (l > mx) mx = l;                               /* optimizer.py:313 */
    }
    if (mn < floor_log) mn = floor_log;                   /* optimizer.py:315 */
    if (mn >= mx) mn = mx - 1.0f;                         /* optimizer.py:316 */
    float scale = mx - mn;                                /* optimizer.py:318 */
    if (scale < 1e-12f) scale = 1e-12f;
    for (int64_t i = 0; i < block; ++i) {
        float v = (i < valid) ? x[i] : 0.0f;
        float code;
        if (v == 0.0f) {
            code = 0.0f;                                  /* optimizer.py:321 */
        } else {
            float vs = (v < 1e-38f) ? 1e-38f : v;
            float l = (vs == 1e-38f) ? l_zero : log2_cr(vs);
            float t = (l - mn) / scale;                   /* optimizer.py:320 */
            t = t * qm1;
            code = rintf(t) + 1.0f;
            if (code < 1.0f) code = 1.0f;
            if (code > qmax) code = qmax;
        }
        if (bits == 16) ((uint16_t *)q_out)[i] = (uint16_t)code;
        else ((uint8_t *)q_out)[i] = (uint8_t)code;
    }
    *scale_out = scale;
    *min_log_out = mn;
}

/* _log_quantize_nonneg over a whole flattened tensor (optimizer.py:299-325).
 * q has nblocks*block entries, scale/min_log have nblocks entries. */
AF8O_API int af8o_al_quantize(const float *x, int64_t n, int64_t block,
                              float floor_log, int bits, void *q, float *scale,
                              float *min_log)
{
    if (block <= 0 || (bits != 8 && bits != 16)) return 1;
    int64_t nblocks = (n + block - 1) / block;
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < nblocks; ++b) {
        int64_t start = b * block;
        int64_t valid = n - start < block ? n - start : block;
        void *qb = (bits == 16) ? (void *)((uint16_t *)q + start)
                                : (void *)((uint8_t *)q + start);
        al_quant_block(x + start, valid, block, floor_log, bits, qb, scale + b,
                       min_log + b);
    }
    return 0;
}

/* one element of _log_dequantize_nonneg (optimizer.py:341-349) */
static inline float al_deq1(uint32_t code, float scale, float min_log, float qm1)
{
    if (code == 0) return 0.0f;                           /* optimizer.py:349 */
    float t = ((float)code - 1.0f) * scale;               /* optimizer.py:347 */
    t = t / qm1;
    t = t + min_log;
    return pow2_cr(t);                                    /* optimizer.py:348 */
}

/* _log_dequantize_nonneg (optimizer.py:328-353); writes n values. */
AF8O_API int af8o_al_dequantize(const void *q, const float *scale,
                                const float *min_log, int64_t n, int64_t block,
                                int bits, float *out)
{
    if (block <= 0 || (bits != 8 && bits != 16)) return 1;
    const float qm1 = (bits == 16) ? 65534.0f : 254.0f;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        int64_t b = i / block;
        uint32_t code = (bits == 16) ? ((const uint16_t *)q)[i]
                                     : ((const uint8_t *)q)[i];
        out[i] = al_deq1(code, scale[b], min_log[b], qm1);
    }
    return 0;
}

/* ------------------------------------------------------------------ */
/* momentum codecs                                                     */
/* ------------------------------------------------------------------ */

/* block absmax with the 1e-12 floor (optimizer.py:462, 510) */
static float m_block_absmax(const float *m, int64_t valid)
{
    float a = 0.0f;
    for (int64_t i = 0; i < valid; ++i) {
        float t = fabsf(m[i]);
        if (t > a) a = t;
    }
    return a < 1e-12f ? 1e-12f : a;
}

/* _quantize_uniform_pytorch, 8-bit branch (optimizer.py:518) */
static inline uint8_t uf8_q1(float m, float a)
{
    float t = m / a;
    t = t * 128.0f;
    t = rintf(t);
    if (t < -128.0f) t = -128.0f;
    if (t > 127.0f) t = 127.0f;
    return (uint8_t)(t + 128.0f);
}

/* _quantize_uniform_pytorch, 4-bit branch (optimizer.py:512) */
static inline uint8_t uf4_q1(float m, float a)
{
    float t = m / a;
    t = t * 8.0f;
    t = rintf(t);
    if (t < -8.0f) t = -8.0f;
    if (t > 7.0f) t = 7.0f;
    return (uint8_t)(t + 8.0f);
}

/* _quantize_dynamic_pytorch for one element (optimizer.py:463-473).
 * map is sorted ascending with L entries. */
static inline uint8_t dyn_q1(float m, float a, const float *map, int L)
{
    float x = m / a;
    int lo = 0, hi = L;                 /* torch.searchsorted, side="left" */
    while (lo < hi) {
        int mid = (lo + hi) >> 1;
        if (map[mid] < x) lo = mid + 1; else hi = mid;
    }
    int idx = lo > L - 1 ? L - 1 : lo;
    int prev = idx - 1 < 0 ? 0 : idx - 1;
    float cd = fabsf(x - map[idx]);
    float pd = fabsf(x - map[prev]);
    if (pd < cd) idx = prev;
    int os = (x > 0.0f) - (x < 0.0f);
    int ms = (map[idx] > 0.0f) - (map[idx] < 0.0f);
    int flip = (os != ms) && (os != 0);
    int out = idx;
    if (flip && os > 0 && idx < L - 1) out = idx + 1;
    if (flip && os < 0 && out > 0 && idx > 0) out = out - 1;
    return (uint8_t)out;
}

/* _m_quantize (optimizer.py:547-552).  n real elements, padded with zeros to
 * a multiple of `block`.  8-bit formats write nblocks*block bytes, 4-bit
 * formats nblocks*block/2 bytes with the even element in the high nibble
 * (optimizer.py:513-515, 477-479).  map is only read for d8 / d4. */
AF8O_API int af8o_m_quantize(const float *m, int64_t n, int64_t block, int fmt,
                             const float *map, uint8_t *q, float *scale)
{
    if (block <= 0 || (block & 1)) return 1;
    if (fmt < AF8O_M_UF8 || fmt > AF8O_M_D4) return 1;
    int64_t nblocks = (n + block - 1) / block;
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < nblocks; ++b) {
        int64_t start = b * block;
        int64_t valid = n - start < block ? n - start : block;
        float a = m_block_absmax(m + start, valid);
        scale[b] = a;
        for (int64_t i = 0; i < block; i += 2) {
            float x0 = (i < valid) ? m[start + i] : 0.0f;
            float x1 = (i + 1 < valid) ? m[start + i + 1] : 0.0f;
            switch (fmt) {
            case AF8O_M_UF8:
                q[start + i] = uf8_q1(x0, a);
                q[start + i + 1] = uf8_q1(x1, a);
                break;
            case AF8O_M_D8:
                q[start + i] = dyn_q1(x0, a, map, 256);
                q[start + i + 1] = dyn_q1(x1, a, map, 256);
                break;
            case AF8O_M_UF4:
                q[(start + i) >> 1] = (uint8_t)((uf4_q1(x0, a) << 4) | uf4_q1(x1, a));
                break;
            default: /* AF8O_M_D4 */
                q[(start + i) >> 1] =
                    (uint8_t)((dyn_q1(x0, a, map, 16) << 4) | dyn_q1(x1, a, map, 16));
                break;
            }
        }
    }
    return 0;
}

static inline float m_deq1(const uint8_t *q, const float *scale, int64_t i,
                           int64_t block, int fmt, const float *map)
{
    float s = scale[i / block];
    switch (fmt) {
    case AF8O_M_UF8:   /* optimizer.py:528-531 */
        return ((float)q[i] - 128.0f) * (s / 128.0f);
    case AF8O_M_UF4: { /* optimizer.py:524-531 */
        uint8_t byte = q[i >> 1];
        uint8_t nib = (i & 1) ? (byte & 0x0F) : (byte >> 4);
        return ((float)nib - 8.0f) * (s / 8.0f);
    }
    case AF8O_M_D8:    /* optimizer.py:489-498 */
        return map[q[i]] * s;
    default: {         /* AF8O_M_D4 */
        uint8_t byte = q[i >> 1];
        uint8_t nib = (i & 1) ? (byte & 0x0F) : (byte >> 4);
        return map[nib] * s;
    }
    }
}

/* _m_dequantize (optimizer.py:555-560) */
AF8O_API int af8o_m_dequantize(const uint8_t *q, const float *scale, int64_t n,
                               int64_t block, int fmt, const float *map,
                               float *out)
{
    if (block <= 0) return 1;
    if (fmt < AF8O_M_UF8 || fmt > AF8O_M_D4) return 1;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) out[i] = m_deq1(q, scale, i, block, fmt, map);
    return 0;
}

/* ------------------------------------------------------------------ */
/* Fira norm-growth limiter on one scalar (optimizer.py:760-782)       */
/* ------------------------------------------------------------------ */
AF8O_API float af8o_fira_scale(float norm, float margin_plus_one, int *has_prev,
                               float *prev)
{
    if (!isfinite(norm)) norm = 0.0f;                    /* optimizer.py:768-769 */
    float fs;
    if (*has_prev) {
        float fp = *prev;
        int is_reset = fp < 1e-6f;                       /* optimizer.py:774 */
        float ratio = norm / (fp + 1e-8f);               /* optimizer.py:775 */
        float lim = (ratio < margin_plus_one ? margin_plus_one : ratio) /
                    margin_plus_one;                     /* optimizer.py:776 */
        fs = is_reset ? 1.0f : 1.0f / lim;               /* optimizer.py:777 */
        *prev = is_reset ? norm : norm * fs;             /* optimizer.py:778 */
    } else {
        fs = 1.0f;                                       /* optimizer.py:780-781 */
        *prev = norm;
        *has_prev = 1;
    }
    return fs;
}

/* sqrt(sum x^2) accumulated in binary64; stands in for
 * torch.linalg.vector_norm (optimizer.py:797, 827, 851, 861, 898). */
static float norm2_f64(const float *x, int64_t n)
{
    double acc = 0.0;
#pragma omp parallel for reduction(+ : acc) schedule(static)
    for (int64_t i = 0; i < n; ++i) acc += (double)x[i] * (double)x[i];
    return (float)sqrt(acc);
}

AF8O_API float af8o_norm2(const float *x, int64_t n) { return norm2_f64(x, n); }

/* ------------------------------------------------------------------ */
/* full-rank step ("1D" path): AdamW / RMSprop / unfactored Adafactor   */
/* ------------------------------------------------------------------ */

/* Host-computed scalars arrive already rounded to binary32 the way the
 * reference's 0-d tensors and Python floats are when they meet a tensor. */
typedef struct {
    int64_t numel;
    int64_t block;        /* V block size (state["block_size"]) */
    int64_t m_block;      /* M block size (state["m_block_size"]) */
    int32_t grad_dtype;   /* AF8O_G_* */
    int32_t v_fmt;        /* AF8O_V_* */
    int32_t m_fmt;        /* AF8O_M_*; AF8O_M_NONE when beta1 is None */
    int32_t negate_grad;  /* maximize (optimizer.py:1973-1974) */
    int32_t use_adam_denom;
    int32_t momentum_only;
    int32_t fira;
    int32_t has_decay;
    float decay;          /* 1 - wd_mult*wd (optimizer.py:2034-2039) */
    float alpha;          /* optimizer.py:2018-2030 */
    float v_w;            /* beta_val as the lerp weight (optimizer.py:2012-2017) */
    float v_keep;         /* float(1.0 - beta_val), fp32-state path (optimizer.py:2187);
                             with AF8O_V_NONE: float(1.0 - beta1), the divisor of the momentum (optimizer.py:2064) */
    float v_eps_add;      /* float(beta_val*eps_for_grad_sq) (optimizer.py:2189) */
    float m_w;            /* float(1.0 - beta1) (optimizer.py:698) */
    float eps_gradsq;     /* optimizer.py:1967 */
    float eps_denom;      /* optimizer.py:1966, 2028 */
    float eps_sq;         /* optimizer.py:1961 */
    float d;              /* clip threshold, 0 disables */
    float sqrt_n;         /* float(math.sqrt(numel)) */
    float clip_div;       /* float(math.sqrt(numel)*d) (optimizer.py:862) */
    float fira_margin1;   /* float(1.0 + fira_margin) */
    float v_floor;        /* min_log floor, -126 on this path (optimizer.py:299) */
} af8o_fullrank_cfg;

/* _apply_update_pytorch (optimizer.py:866-881) with _apply_fira_pytorch
 * (optimizer.py:796-810) and _safe_rms_denom (optimizer.py:859-863).
 * u is consumed (scaled in place).  Returns the update norm it measured, or
 * -1 when no norm was needed. */
static float apply_update(float *p, float *u, int64_t n, float alpha, float d,
                          float clip_div, int fira, float margin1,
                          int *fira_has_prev, float *fira_prev)
{
    float denom = 1.0f;
    float norm = -1.0f;
    if (g_lag.on && (fira || d > 0.0f)) {
        /* lag_norm=True as the reference's CUDA dispatcher runs it (optimizer.py:1056-1071,
         * kernels.cu:651-656; its pure-PyTorch path ignores the flag): the clip uses the previous
         * step's norm, alpha carries the limiter scale computed from it, and the norm of this
         * step's raw update is returned for the caller to store. */
        norm = norm2_f64(u, n);
        if (d > 0.0f) { denom = g_lag.prev_norm / clip_div; if (!(denom >= 1.0f)) denom = 1.0f; }
        const float alpha_eff = alpha * g_lag.fira_scale;
        const float sl = -(alpha_eff / denom);
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < n; ++i) p[i] = write_param(p[i], sl, u[i], i);
        return norm;
    }
    if (fira) {
        norm = norm2_f64(u, n);                          /* optimizer.py:797 */
        if (!isfinite(norm)) {                           /* optimizer.py:798-800 */
            memset(u, 0, (size_t)n * sizeof(float));
            norm = 0.0f;
        }
        float fs = af8o_fira_scale(norm, margin1, fira_has_prev, fira_prev);
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < n; ++i) u[i] = u[i] * fs; /* optimizer.py:803 */
        if (d > 0.0f) {                                  /* optimizer.py:805-806 */
            denom = norm / clip_div;
            if (denom < 1.0f) denom = 1.0f;
        }
    } else if (d > 0.0f) {                               /* optimizer.py:860-862 */
        norm = norm2_f64(u, n);
        denom = norm / clip_div;
        if (!(denom >= 1.0f)) denom = (denom != denom) ? denom : 1.0f;
    }
    float s = -alpha / denom;                            /* optimizer.py:874 */
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) p[i] = write_param(p[i], s, u[i], i);
    return norm;
}

/* _update_param_8bit, full-rank branch without the SGD mode
 * (optimizer.py:1957-2040 prologue scalars are inputs; 2076-2194 body) plus
 * _fallback_1d_update (optimizer.py:886-917) and _m_ema_pytorch
 * (optimizer.py:690-700).
 *
 * Quantised states are updated in place: v_q/v_scale/v_min_log (AL8/AL16,
 * nblocks*block codes) or v_f32; m_q/m_scale (n padded to m_block) or m_f32.
 * map is the dynamic codebook for d8/d4 (else NULL).
 * norm_out receives the update norm measured for clipping / Fira (or -1). */
AF8O_API int af8o_fullrank_step(const af8o_fullrank_cfg *c, float *p,
                                const void *grad, void *v_q, float *v_scale,
                                float *v_min_log, float *v_f32, uint8_t *m_q,
                                float *m_scale, float *m_f32, const float *map,
                                int *fira_has_prev, float *fira_prev,
                                float *norm_out)
{
    const int64_t n = c->numel;
    const int has_m = c->m_fmt != AF8O_M_NONE;
    const int m_quant = has_m && c->m_fmt != AF8O_M_FP32;
    if (c->v_fmt == AF8O_V_NONE) {
        /* SGD mode (optimizer.py:2045-2071): no second moment; the update is the gradient, or
         * the momentum divided by float(1 - beta1); then the common _apply_update_pytorch */
        float *gs = (float *)malloc((size_t)(n ? n : 1) * sizeof(float));
        float *us = (float *)malloc((size_t)(n ? n : 1) * sizeof(float));
        if (!gs || !us) { free(gs); free(us); return 2; }
        int rcs = 0;
    note_decay(c->has_decay, c->decay);
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < n; ++i) {
            gs[i] = load_grad(grad, c->grad_dtype, i, c->negate_grad);
            p[i] = decay_param(p[i], c->has_decay, c->decay);
        }
        if (has_m) {
            float *m = m_quant ? us : m_f32;
            if (m_quant) af8o_m_dequantize(m_q, m_scale, n, c->m_block, c->m_fmt, map, m);
#pragma omp parallel for schedule(static)
            for (int64_t i = 0; i < n; ++i) m[i] = lerp_t(m[i], gs[i], c->m_w);
            if (m_quant) rcs = af8o_m_quantize(m, n, c->m_block, c->m_fmt, map, m_q, m_scale);
#pragma omp parallel for schedule(static)
            for (int64_t i = 0; i < n; ++i) us[i] = m[i] / c->v_keep;
        } else {
            memcpy(us, gs, (size_t)n * sizeof(float));
        }
        float norms = apply_update(p, us, n, c->alpha, c->d, c->clip_div, c->fira, c->fira_margin1, fira_has_prev, fira_prev);
        if (norm_out) *norm_out = norms;
        free(gs);
        free(us);
        return rcs;
    }
    const int v_quant = c->v_fmt != AF8O_V_FP32;
    float *g = (float *)malloc((size_t)(n ? n : 1) * sizeof(float));
    float *v = v_quant ? (float *)malloc((size_t)(n ? n : 1) * sizeof(float)) : v_f32;
    float *u = (float *)malloc((size_t)(n ? n : 1) * sizeof(float));
    if (!g || !v || !u) { free(g); if (v_quant) free(v); free(u); return 2; }

    /* grad upcast (optimizer.py:1997), weight decay as its own pass
     * (optimizer.py:2039) */
    note_decay(c->has_decay, c->decay);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        g[i] = load_grad(grad, c->grad_dtype, i, c->negate_grad);
        p[i] = decay_param(p[i], c->has_decay, c->decay);
    }

    if (v_quant) {
        /* optimizer.py:2117-2121 */
        af8o_al_dequantize(v_q, v_scale, v_min_log, n, c->block, c->v_fmt, v);
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < n; ++i) {
            float g2 = g[i] * g[i];
            g2 = g2 + c->eps_gradsq;
            v[i] = lerp_t(v[i], g2, c->v_w);
        }
        af8o_al_quantize(v, n, c->block, c->v_floor, c->v_fmt, v_q, v_scale, v_min_log);
    } else {
        /* optimizer.py:2186-2189 */
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < n; ++i) {
            float t = v[i] * c->v_keep;
            t = fmaf(c->v_w * g[i], g[i], t);
            if (c->eps_gradsq > 0.0f) t = t + c->v_eps_add;
            v[i] = t;
        }
    }

    float norm = -1.0f;
    int rc = 0;
    if (has_m) {
        /* m_temp before the EMA: dequantised state or the fp32 state */
        float *m = m_quant ? u : m_f32;
        if (m_quant) af8o_m_dequantize(m_q, m_scale, n, c->m_block, c->m_fmt, map, m);
        if (c->momentum_only) {
            /* optimizer.py:894-901 */
            float *ut = g;  /* grad_fp32 * inv_std, reuse g */
#pragma omp parallel for schedule(static)
            for (int64_t i = 0; i < n; ++i) {
                float vc = v[i] < c->eps_sq ? c->eps_sq : v[i];
                ut[i] = g[i] * rsqrt_t(vc);
            }
            if (c->d > 0.0f) {
                float rms = norm2_f64(ut, n) / c->sqrt_n;
                float cf = rms / c->d;
                if (cf < 1.0f) cf = 1.0f;
#pragma omp parallel for schedule(static)
                for (int64_t i = 0; i < n; ++i) ut[i] = ut[i] / cf;
            }
#pragma omp parallel for schedule(static)
            for (int64_t i = 0; i < n; ++i) m[i] = lerp_t(m[i], ut[i], c->m_w);
            if (m_quant) rc = af8o_m_quantize(m, n, c->m_block, c->m_fmt, map, m_q, m_scale);
            float *upd = u;
            if (!m_quant) memcpy(u, m, (size_t)n * sizeof(float));
            norm = apply_update(p, upd, n, c->alpha, 0.0f, c->clip_div, c->fira,
                                c->fira_margin1, fira_has_prev, fira_prev);
        } else {
            /* optimizer.py:903-910 */
#pragma omp parallel for schedule(static)
            for (int64_t i = 0; i < n; ++i) m[i] = lerp_t(m[i], g[i], c->m_w);
            if (m_quant) rc = af8o_m_quantize(m, n, c->m_block, c->m_fmt, map, m_q, m_scale);
#pragma omp parallel for schedule(static)
            for (int64_t i = 0; i < n; ++i) {
                float inv;
                if (c->use_adam_denom) {
                    float den = sqrtf(v[i]) + c->eps_denom;
                    inv = 1.0f / den;
                } else {
                    float vc = v[i] < c->eps_sq ? c->eps_sq : v[i];
                    inv = rsqrt_t(vc);
                }
                u[i] = m[i] * inv;
            }
            norm = apply_update(p, u, n, c->alpha, c->d, c->clip_div, c->fira,
                                c->fira_margin1, fira_has_prev, fira_prev);
        }
    } else {
        /* optimizer.py:911-917 */
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < n; ++i) {
            if (c->use_adam_denom) {
                float den = sqrtf(v[i]) + c->eps_denom;
                u[i] = g[i] / den;
            } else {
                float vc = v[i] < c->eps_sq ? c->eps_sq : v[i];
                u[i] = g[i] * rsqrt_t(vc);
            }
        }
        norm = apply_update(p, u, n, c->alpha, c->d, c->clip_div, c->fira,
                            c->fira_margin1, fira_has_prev, fira_prev);
    }
    if (norm_out) *norm_out = norm;
    free(g);
    if (v_quant) free(v);
    free(u);
    return rc;
}

/* ------------------------------------------------------------------ */
/* factored step ("2D" path): Adafactor and CAME                       */
/* ------------------------------------------------------------------ */

/* A small second-moment / confidence state of n elements: quantised
 * (q/scale/min_log, fmt 8 or 16) or fp32 (f32, fmt 0). */
typedef struct {
    void *q;
    float *scale;
    float *min_log;
    float *f32;
    int64_t n;
    int32_t fmt;
    int32_t pad_;
} af8o_small_state;

typedef struct {
    int64_t rows, cols;
    int64_t block;        /* AL block of the row / col / conf states */
    int64_t m_block;
    int32_t grad_dtype;
    int32_t m_fmt;        /* AF8O_M_NONE when beta1 is None */
    int32_t came;         /* beta3 is not None */
    int32_t negate_grad;
    int32_t fira;
    int32_t has_decay;
    float decay;
    float alpha;
    float v_w;            /* beta_val */
    float m_w;            /* float(1 - beta1) */
    float c_w;            /* float(1 - beta3) */
    float eps1;
    float eps_came;
    float d;
    float sqrt_n;         /* float(sqrt(rows*cols)) */
    float clip_div;       /* float(sqrt(rows*cols)*d) */
    float fira_margin1;
    float v_floor;
} af8o_factored_cfg;

/* deq -> lerp_ -> requant of one small state (optimizer.py:2232-2238,
 * 937-946), or lerp_ of the fp32 state (optimizer.py:2248-2251).
 * out receives the un-requantised values. */
static void small_state_ema(af8o_small_state *s, const float *new_vals, float w,
                            int64_t block, float floor_log, float *out)
{
    const int64_t n = s->n;
    if (s->fmt == AF8O_V_FP32) {
        for (int64_t i = 0; i < n; ++i) {
            s->f32[i] = lerp_t(s->f32[i], new_vals[i], w);
            out[i] = s->f32[i];
        }
        return;
    }
    af8o_al_dequantize(s->q, s->scale, s->min_log, n, block, s->fmt, out);
    for (int64_t i = 0; i < n; ++i) out[i] = lerp_t(out[i], new_vals[i], w);
    af8o_al_quantize(out, n, block, floor_log, s->fmt, s->q, s->scale, s->min_log);
}

/* row means and column means of x[R][C], binary64 accumulation
 * (Tensor.mean(dim=-1) / mean(dim=-2), optimizer.py:2222-2223, 933-934) */
static void row_col_means(const float *x, int64_t R, int64_t C, float *rmean, float *cmean)
{
    double *cs = (double *)calloc((size_t)C, sizeof(double));
#pragma omp parallel
    {
        double *local = (double *)calloc((size_t)C, sizeof(double));
#pragma omp for schedule(static)
        for (int64_t i = 0; i < R; ++i) {
            double rs = 0.0;
            const float *row = x + i * C;
            for (int64_t j = 0; j < C; ++j) { rs += (double)row[j]; local[j] += (double)row[j]; }
            rmean[i] = (float)(rs / (double)C);
        }
#pragma omp critical
        for (int64_t j = 0; j < C; ++j) cs[j] += local[j];
        free(local);
    }
    for (int64_t j = 0; j < C; ++j) cmean[j] = (float)(cs[j] / (double)R);
    free(cs);
}

static float mean_f64(const float *x, int64_t n)
{
    double a = 0.0;
    for (int64_t i = 0; i < n; ++i) a += (double)x[i];
    return (float)(a / (double)n);
}

/* _update_param_8bit, factored branch on the pure-PyTorch route
 * (optimizer.py:2202-2253 statistics, 2394-2399 / 2543-2549 dispatch),
 * _factored_inv_std (optimizer.py:818-821), _compute_ut_clipped
 * (optimizer.py:824-829) and _fallback_2d_update (optimizer.py:920-970). */
/* The next af8o_factored_step treats its tensor as a batch of this many rows x cols matrices. */
static int64_t factored_batch = 1;
AF8O_API void af8o_factored_set_batch(int64_t b) { factored_batch = b; }

AF8O_API int af8o_factored_step(const af8o_factored_cfg *c, float *p, const void *grad,
                                af8o_small_state *row_var, af8o_small_state *col_var,
                                af8o_small_state *conf_row, af8o_small_state *conf_col,
                                uint8_t *m_q, float *m_scale, float *m_f32, const float *map,
                                int *fira_has_prev, float *fira_prev, float *norm_out)
{
    /* a tensor of more than two dimensions is a batch of B matrices (optimizer.py:2203-2207): rows / cols
     * describe one of them, the row states hold B*R values, the column states B*C, the means that
     * normalise the row factor are taken per matrix (row_var.mean(dim=-2)), norms over the whole tensor */
    const int64_t B = factored_batch > 0 ? factored_batch : 1;
    factored_batch = 1;
    const int64_t R = c->rows, C = c->cols, RC = R * C, n = B * RC;
#define COLI(i) (((i) / RC) * C + (i) % C)
    const int has_m = c->m_fmt != AF8O_M_NONE;
    const int m_quant = has_m && c->m_fmt != AF8O_M_FP32;
    float *g = (float *)malloc((size_t)n * sizeof(float));
    float *u = (float *)malloc((size_t)n * sizeof(float));
    float *rmean = (float *)malloc((size_t)(B * R) * sizeof(float));
    float *cmean = (float *)malloc((size_t)(B * C) * sizeof(float));
    float *row = (float *)malloc((size_t)(B * R) * sizeof(float));
    float *col = (float *)malloc((size_t)(B * C) * sizeof(float));
    float *inv_r = (float *)malloc((size_t)(B * R) * sizeof(float));
    float *inv_c = (float *)malloc((size_t)(B * C) * sizeof(float));
    if (!g || !u || !rmean || !cmean || !row || !col || !inv_r || !inv_c) return 2;

    note_decay(c->has_decay, c->decay);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        g[i] = load_grad(grad, c->grad_dtype, i, c->negate_grad);
        p[i] = decay_param(p[i], c->has_decay, c->decay);          /* optimizer.py:2039 */
        u[i] = g[i] * g[i];                                /* optimizer.py:2221 */
    }
    for (int64_t b = 0; b < B; ++b) row_col_means(u + b * RC, R, C, rmean + b * R, cmean + b * C);   /* optimizer.py:2222-2223 */
    for (int64_t i = 0; i < B * R; ++i) rmean[i] = rmean[i] + c->eps1;
    for (int64_t j = 0; j < B * C; ++j) cmean[j] = cmean[j] + c->eps1;

    /* optimizer.py:2232-2238 / 2248-2252 */
    small_state_ema(row_var, rmean, c->v_w, c->block, c->v_floor, row);
    small_state_ema(col_var, cmean, c->v_w, c->block, c->v_floor, col);
    for (int64_t b = 0; b < B; ++b) {
        float rm = mean_f64(row + b * R, R);
        if (rm < c->eps1) rm = c->eps1;
        for (int64_t i = b * R; i < (b + 1) * R; ++i) inv_r[i] = rsqrt_t(row[i] / rm);   /* optimizer.py:819 */
    }
    for (int64_t j = 0; j < B * C; ++j) inv_c[j] = rsqrt_t(col[j]);    /* optimizer.py:820 */

    float norm = -1.0f;
    int rc = 0;
    if (c->came && has_m) {
        /* optimizer.py:928-956 */
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < n; ++i) {
            float t = g[i] * inv_r[i / C];                 /* optimizer.py:825 */
            g[i] = t * inv_c[COLI(i)];
        }
        if (c->d > 0.0f) {                                 /* optimizer.py:826-828 */
            float rms = norm2_f64(g, n) / c->sqrt_n;
            float cf = rms / c->d;
            if (cf < 1.0f) cf = 1.0f;
#pragma omp parallel for schedule(static)
            for (int64_t i = 0; i < n; ++i) g[i] = g[i] / cf;
        }
        float *m = m_quant ? u : m_f32;
        if (m_quant) af8o_m_dequantize(m_q, m_scale, n, c->m_block, c->m_fmt, map, m);
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < n; ++i) m[i] = lerp_t(m[i], g[i], c->m_w);
        if (m_quant) rc = af8o_m_quantize(m, n, c->m_block, c->m_fmt, map, m_q, m_scale);
        /* res = (U - M)^2 + eps_came, in place in U (optimizer.py:932) */
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < n; ++i) {
            float t = g[i] - m[i];
            t = t * t;
            g[i] = t + c->eps_came;
        }
        for (int64_t b = 0; b < B; ++b) row_col_means(g + b * RC, R, C, rmean + b * R, cmean + b * C);   /* optimizer.py:933-934 */
        small_state_ema(conf_row, rmean, c->c_w, c->block, c->v_floor, row);   /* optimizer.py:937-946 */
        small_state_ema(conf_col, cmean, c->c_w, c->block, c->v_floor, col);
        for (int64_t b = 0; b < B; ++b) {
            float cm = mean_f64(row + b * R, R);           /* optimizer.py:948 */
            if (cm < c->eps1) cm = c->eps1;
            for (int64_t i = b * R; i < (b + 1) * R; ++i) inv_r[i] = rsqrt_t(row[i] / cm);
        }
        for (int64_t j = 0; j < B * C; ++j) inv_c[j] = rsqrt_t(col[j]);
        if (!m_quant) memcpy(u, m, (size_t)n * sizeof(float));
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < n; ++i) {                  /* optimizer.py:952, 955 */
            float t = u[i] * inv_r[i / C];
            u[i] = t * inv_c[COLI(i)];
        }
        norm = apply_update(p, u, n, c->alpha, 0.0f, c->clip_div, c->fira, c->fira_margin1,
                            fira_has_prev, fira_prev);
    } else if (has_m) {
        /* optimizer.py:958-965 */
        float *m = m_quant ? u : m_f32;
        if (m_quant) af8o_m_dequantize(m_q, m_scale, n, c->m_block, c->m_fmt, map, m);
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < n; ++i) m[i] = lerp_t(m[i], g[i], c->m_w);
        if (m_quant) rc = af8o_m_quantize(m, n, c->m_block, c->m_fmt, map, m_q, m_scale);
        if (!m_quant) memcpy(u, m, (size_t)n * sizeof(float));
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < n; ++i) {
            float t = u[i] * inv_r[i / C];
            u[i] = t * inv_c[COLI(i)];
        }
        norm = apply_update(p, u, n, c->alpha, c->d, c->clip_div, c->fira, c->fira_margin1,
                            fira_has_prev, fira_prev);
    } else {
        /* optimizer.py:967-970 */
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < n; ++i) {
            float t = g[i] * inv_r[i / C];
            u[i] = t * inv_c[COLI(i)];
        }
        norm = apply_update(p, u, n, c->alpha, c->d, c->clip_div, c->fira, c->fira_margin1,
                            fira_has_prev, fira_prev);
    }
    if (norm_out) *norm_out = norm;
    free(g); free(u); free(rmean); free(cmean); free(row); free(col); free(inv_r); free(inv_c);
#undef COLI
    return rc;
}

/* ------------------------------------------------------------------ */
/* APOLLO: low-rank projected Adam statistics, channel-wise scaling     */
/* ------------------------------------------------------------------ */
typedef struct {
    int64_t rows, cols, rank;
    int64_t block, m_block;
    int32_t grad_dtype;
    int32_t v_fmt;          /* AF8O_V_* of v_low */
    int32_t m_fmt;          /* AF8O_M_* of m_low; NONE when beta1 is None */
    int32_t negate_grad;
    int32_t first_step;     /* v_low does not exist yet (optimizer.py:2763) */
    int32_t scale_tensor;   /* apollo_scale_type == "tensor" */
    int32_t scale_front;
    int32_t fira;
    int32_t has_decay;
    float decay;
    float alpha;            /* alpha_t */
    float bc;               /* float(sqrt(bc2)/bc1), or bc1 when bc_mode == 2 */
    int32_t bc_mode;        /* 0 none, 1 multiply, 2 divide (optimizer.py:3015-3023) */
    float v_w;              /* beta_val */
    float m_w;              /* float(1 - beta1) */
    float apollo_eps;
    float sqrt_scale;       /* float(sqrt(apollo_scale)) */
    float d;
    float clip_div;         /* float(sqrt(numel)*d) */
    float fira_margin1;
    float v_floor_first;    /* -126 */
    float v_floor_later;    /* log2(max(apollo_eps^2, FLT_MIN)) (optimizer.py:2766-2767) */
} af8o_apollo_cfg;

/* _update_param_apollo without factorisation and without CAME
 * (optimizer.py:2587-3084): projection (2678-2681), low-rank V (2763-2799) and M
 * (2906-2953) states, update_low (2959), scaling factor (2961-2966), global norm
 * (2973-2988), Fira (2990-2996), write-back for fp32 parameters (3073-3079).
 * pt is proj_matrix_T: (cols, rank) when rows >= cols ("right"), else (rank, rows). */
/* Further low-rank state rules of _update_param_apollo, selected by the next af8o_apollo_step
 * after af8o_apollo_set_extra (cleared by that call):
 *   factorize            row / column factors of the projected gradient's squares instead of
 *                        v_low (optimizer.py:2688-2760), optionally with CAME's confidence
 *                        vectors on top (2708-2750);
 *   came, not factorize  CAME over the projected gradient: instability state res_low shaped
 *                        like it (optimizer.py:2801-2903, the pure-PyTorch branch 2869-2894). */
typedef struct {
    int32_t factorize;        /* apollo_factorize */
    int32_t came;             /* beta3 is not None */
    int32_t c_fmt;            /* AF8O_V_* of conf_row_low / conf_col_low / res_low */
    int32_t first_factor;     /* row_var_low does not exist yet (optimizer.py:2695) */
    float v_keep;             /* float(1 - beta_val) */
    float c_w;                /* float(1 - beta3) */
    float eps_came;
    float eps_sq;             /* max(apollo_eps^2, FLT_MIN) */
    float d;                  /* clip threshold of U_t (the low-rank one, optimizer.py:2716-2718) */
    float reserved;
    float *row_var_low;       /* fp32 [LR] */
    float *col_var_low;       /* fp32 [LC] */
    af8o_small_state conf_row, conf_col;      /* factorize + CAME */
    af8o_small_state res;                     /* CAME without factorisation: n = LR*LC */
} af8o_apollo_extra;
static const af8o_apollo_extra *apollo_extra = NULL;
AF8O_API void af8o_apollo_set_extra(const af8o_apollo_extra *x) { apollo_extra = x; }

/* U_t / clamp(rms(U_t)/d, 1) (optimizer.py:2716-2718, 2872-2874) */
static void clip_low(float *u, int64_t n, float d)
{
    if (d > 0.0f) {
        float rms = norm2_f64(u, n) / (float)sqrt((double)n);
        float cf = rms / d;
        if (cf < 1.0f) cf = 1.0f;
        for (int64_t i = 0; i < n; ++i) u[i] = u[i] / cf;
    }
}

/* the low-rank momentum (optimizer.py:714-729, 690-700): m receives the un-requantised values */
static int low_m_ema(const af8o_apollo_cfg *c, const float *x, int64_t nl, uint8_t *m_q, float *m_scale, float *m_f32,
                     const float *map, float *m)
{
    if (c->m_fmt != AF8O_M_FP32) {
        af8o_m_dequantize(m_q, m_scale, nl, c->m_block, c->m_fmt, map, m);
        for (int64_t i = 0; i < nl; ++i) m[i] = lerp_t(m[i], x[i], c->m_w);
        return af8o_m_quantize(m, nl, c->m_block, c->m_fmt, map, m_q, m_scale);
    }
    for (int64_t i = 0; i < nl; ++i) { m_f32[i] = lerp_t(m_f32[i], x[i], c->m_w); m[i] = m_f32[i]; }
    return 0;
}

/* Test hook: the next af8o_apollo_step takes this projected gradient (rows x rank or rank x cols
 * floats) instead of computing G*Pt, so that everything after the contraction can be compared
 * with a device run that started from the same projected values.  Cleared by that call. */
static const float *g_low_override = NULL;
AF8O_API void af8o_apollo_override_g_low(const float *g_low) { g_low_override = g_low; }

AF8O_API int af8o_apollo_step(const af8o_apollo_cfg *c, float *p, const void *grad, const float *pt,
                              void *v_q, float *v_scale, float *v_min_log, float *v_f32,
                              uint8_t *m_q, float *m_scale, float *m_f32, const float *map,
                              int *fira_has_prev, float *fira_prev, float *norm_out)
{
    const int64_t R = c->rows, C = c->cols, r = c->rank, n = R * C;
    const int right = R >= C;                                /* optimizer.py:2662 */
    const int64_t LR = right ? R : r, LC = right ? r : C, nl = LR * LC;
    const int has_m = c->m_fmt != AF8O_M_NONE;
    const int m_quant = has_m && c->m_fmt != AF8O_M_FP32;
    const int v_quant = c->v_fmt != AF8O_V_FP32;
    float *G = (float *)malloc((size_t)n * sizeof(float));
    float *gl = (float *)malloc((size_t)nl * sizeof(float));
    float *v = (float *)malloc((size_t)nl * sizeof(float));
    float *m = (float *)malloc((size_t)nl * sizeof(float));
    const int64_t nch = right ? R : C;                       /* channels */
    float *sf = (float *)malloc((size_t)nch * sizeof(float));
    if (!G || !gl || !v || !m || !sf) return 2;

#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {                        /* optimizer.py:2601-2606 */
        float x = load_grad(grad, c->grad_dtype, i, c->negate_grad);
        G[i] = isfinite(x) ? x : 0.0f;
    }
    /* optimizer.py:2678-2681, binary64 accumulation.  Each output element sums its products in
     * ascending order of the contracted index; the loops are arranged so that the innermost one
     * walks memory contiguously. */
    if (g_low_override) {
        memcpy(gl, g_low_override, (size_t)nl * sizeof(float));
        g_low_override = NULL;
    } else if (right) {
#pragma omp parallel
        {
            double *acc = (double *)malloc((size_t)r * sizeof(double));
#pragma omp for schedule(static)
            for (int64_t i = 0; i < R; ++i) {
                for (int64_t k = 0; k < r; ++k) acc[k] = 0.0;
                for (int64_t j = 0; j < C; ++j) {
                    const double gij = (double)G[i * C + j];
                    const float *prow = pt + j * r;
                    for (int64_t k = 0; k < r; ++k) acc[k] += gij * (double)prow[k];
                }
                for (int64_t k = 0; k < r; ++k) gl[i * r + k] = (float)acc[k];
            }
            free(acc);
        }
    } else {
#pragma omp parallel
        {
            double *acc = (double *)malloc((size_t)C * sizeof(double));
#pragma omp for schedule(static)
            for (int64_t k = 0; k < r; ++k) {
                for (int64_t j = 0; j < C; ++j) acc[j] = 0.0;
                for (int64_t i = 0; i < R; ++i) {
                    const double pki = (double)pt[k * R + i];
                    const float *grow = G + i * C;
                    for (int64_t j = 0; j < C; ++j) acc[j] += pki * (double)grow[j];
                }
                for (int64_t j = 0; j < C; ++j) gl[k * C + j] = (float)acc[j];
            }
            free(acc);
        }
    }
    const af8o_apollo_extra *x = apollo_extra;
    apollo_extra = NULL;
    int rc = 0;
    if (x && x->factorize) {
        /* optimizer.py:2688-2760.  update_low ends up in m. */
        float *sq = v;                                       /* grad_low.square() */
        float *rmean = (float *)malloc((size_t)LR * sizeof(float)), *cmean = (float *)malloc((size_t)LC * sizeof(float));
        float *crow = (float *)malloc((size_t)LR * sizeof(float)), *ccol = (float *)malloc((size_t)LC * sizeof(float));
        if (!rmean || !cmean || !crow || !ccol) return 2;
        for (int64_t i = 0; i < nl; ++i) sq[i] = gl[i] * gl[i];
        row_col_means(sq, LR, LC, rmean, cmean);             /* optimizer.py:2691-2692 */
        float *rv = x->row_var_low, *cv = x->col_var_low;
        for (int64_t i = 0; i < LR; ++i) {
            const float t = rmean[i] + LOG_QUANT_FLOOR;
            rv[i] = x->first_factor ? t * c->v_w : fmaf(c->v_w, t, rv[i] * x->v_keep);      /* optimizer.py:2695-2700 */
        }
        for (int64_t j = 0; j < LC; ++j) {
            const float t = cmean[j] + LOG_QUANT_FLOOR;
            cv[j] = x->first_factor ? t * c->v_w : fmaf(c->v_w, t, cv[j] * x->v_keep);
        }
        const float rvm = mean_f64(rv, LR);                  /* row_var.mean(dim=-2) */
        if (has_m && x->came) {                              /* optimizer.py:2708-2750 */
            float rmv = rvm < LOG_QUANT_FLOOR ? LOG_QUANT_FLOOR : rvm;
            for (int64_t i = 0; i < LR; ++i) crow[i] = rsqrt_t(rv[i] / rmv);               /* _factored_inv_std */
            for (int64_t j = 0; j < LC; ++j) ccol[j] = rsqrt_t(cv[j]);
            float *U = sq;
            for (int64_t i = 0; i < nl; ++i) { float t = gl[i] * crow[i / LC]; U[i] = t * ccol[i % LC]; }
            clip_low(U, nl, x->d);
            rc = low_m_ema(c, U, nl, m_q, m_scale, m_f32, map, m);
            for (int64_t i = 0; i < nl; ++i) { float t = U[i] - m[i]; t = t * t; U[i] = t + x->eps_came; }
            row_col_means(U, LR, LC, rmean, cmean);
            af8o_small_state cr = x->conf_row, cc = x->conf_col;
            small_state_ema(&cr, rmean, x->c_w, c->block, -126.0f, crow);
            small_state_ema(&cc, cmean, x->c_w, c->block, -126.0f, ccol);
            float cm = mean_f64(crow, LR);
            if (cm < LOG_QUANT_FLOOR) cm = LOG_QUANT_FLOOR;
            for (int64_t i = 0; i < LR; ++i) crow[i] = rsqrt_t(crow[i] / cm);
            for (int64_t j = 0; j < LC; ++j) ccol[j] = rsqrt_t(ccol[j]);
            for (int64_t i = 0; i < nl; ++i) { float t = m[i] * crow[i / LC]; m[i] = t * ccol[i % LC]; }   /* optimizer.py:2750 */
        } else {
            const float div = rvm < c->apollo_eps ? c->apollo_eps : rvm;                    /* optimizer.py:2705 */
            if (has_m) rc = low_m_ema(c, gl, nl, m_q, m_scale, m_f32, map, m);              /* optimizer.py:2753-2757 */
            else memcpy(m, gl, (size_t)nl * sizeof(float));
            for (int64_t i = 0; i < nl; ++i) {
                float ve = rv[i / LC] * cv[i % LC];
                ve = ve / div;
                m[i] = m[i] / (sqrtf(ve) + c->apollo_eps);   /* optimizer.py:2758, 2760 */
            }
        }
        free(rmean); free(cmean); free(crow); free(ccol);
        goto scaling;
    }
    /* low-rank second moment */
    if (c->first_step) {                                     /* optimizer.py:2770-2779 */
        for (int64_t i = 0; i < nl; ++i) { float t = gl[i] * gl[i]; v[i] = t * c->v_w; }
        if (v_quant) af8o_al_quantize(v, nl, c->block, c->v_floor_first, c->v_fmt, v_q, v_scale, v_min_log);
        else memcpy(v_f32, v, (size_t)nl * sizeof(float));
    } else if (v_quant) {                                    /* optimizer.py:2788-2795 */
        af8o_al_dequantize(v_q, v_scale, v_min_log, nl, c->block, c->v_fmt, v);
        for (int64_t i = 0; i < nl; ++i) v[i] = lerp_t(v[i], gl[i] * gl[i], c->v_w);
        af8o_al_quantize(v, nl, c->block, c->v_floor_later, c->v_fmt, v_q, v_scale, v_min_log);
    } else {                                                 /* optimizer.py:2797-2799 */
        for (int64_t i = 0; i < nl; ++i) { v_f32[i] = lerp_t(v_f32[i], gl[i] * gl[i], c->v_w); v[i] = v_f32[i]; }
    }
    if (x && x->came) {
        /* optimizer.py:2801-2903, pure-PyTorch branch; update_low ends up in m */
        float *U = (float *)malloc((size_t)nl * sizeof(float));
        if (!U) return 2;
        for (int64_t i = 0; i < nl; ++i) {
            const float vc = v[i] < x->eps_sq ? x->eps_sq : v[i];
            U[i] = gl[i] * rsqrt_t(vc);                      /* optimizer.py:2871, 2898 */
        }
        clip_low(U, nl, x->d);
        if (has_m) {
            rc = low_m_ema(c, U, nl, m_q, m_scale, m_f32, map, m);
            for (int64_t i = 0; i < nl; ++i) { float t = U[i] - m[i]; t = t * t; U[i] = t + x->eps_came; }   /* optimizer.py:2881 */
            af8o_small_state rs = x->res;
            if (rs.fmt == AF8O_V_FP32) {
                for (int64_t i = 0; i < nl; ++i) { rs.f32[i] = lerp_t(rs.f32[i], U[i], x->c_w); U[i] = rs.f32[i]; }
            } else {                                         /* optimizer.py:2884-2889: the requantised values are used */
                float *t2 = v;
                small_state_ema(&rs, U, x->c_w, c->block, -126.0f, t2);
                af8o_al_dequantize(rs.q, rs.scale, rs.min_log, nl, c->block, rs.fmt, U);
            }
            for (int64_t i = 0; i < nl; ++i) {
                const float rc_ = U[i] < x->eps_sq ? x->eps_sq : U[i];
                m[i] = m[i] * rsqrt_t(rc_);                  /* optimizer.py:2894 */
            }
        } else {
            memcpy(m, U, (size_t)nl * sizeof(float));        /* optimizer.py:2902 */
        }
        free(U);
        goto scaling;
    }
    /* low-rank momentum and update_low (optimizer.py:2906-2959) */
    if (has_m) {
        if (m_quant) {
            af8o_m_dequantize(m_q, m_scale, nl, c->m_block, c->m_fmt, map, m);
            for (int64_t i = 0; i < nl; ++i) m[i] = lerp_t(m[i], gl[i], c->m_w);
            rc = af8o_m_quantize(m, nl, c->m_block, c->m_fmt, map, m_q, m_scale);
        } else {
            for (int64_t i = 0; i < nl; ++i) { m_f32[i] = lerp_t(m_f32[i], gl[i], c->m_w); m[i] = m_f32[i]; }
        }
    } else {
        memcpy(m, gl, (size_t)nl * sizeof(float));
    }
    for (int64_t i = 0; i < nl; ++i) m[i] = m[i] / (sqrtf(v[i]) + c->apollo_eps);   /* update_low in m */

scaling:;
    /* scaling factor (optimizer.py:2961-2966) and squared channel norms of G (2975-2979) */
    double total = 0.0;
    float norm_unscaled = 0.0f;
    if (!c->scale_tensor) {
        /* per-channel sums in binary64, each in ascending index order; channels are independent,
         * the final sum over channels runs in channel order */
        double *nu = (double *)calloc((size_t)nch * 3, sizeof(double));
        if (!nu) return 2;
        double *ng = nu + nch, *nG = ng + nch;
        if (right) {
#pragma omp parallel for schedule(static)
            for (int64_t ch = 0; ch < nch; ++ch) {
                double a = 0.0, b = 0.0, cc = 0.0;
                for (int64_t k = 0; k < r; ++k) { a += (double)m[ch * r + k] * m[ch * r + k]; b += (double)gl[ch * r + k] * gl[ch * r + k]; }
                for (int64_t j = 0; j < C; ++j) cc += (double)G[ch * C + j] * G[ch * C + j];
                nu[ch] = a; ng[ch] = b; nG[ch] = cc;
            }
        } else {
            const int64_t strip = 512;                        /* columns per task: rows are walked contiguously */
#pragma omp parallel for schedule(static)
            for (int64_t c0 = 0; c0 < nch; c0 += strip) {
                const int64_t c1 = c0 + strip < nch ? c0 + strip : nch;
                for (int64_t k = 0; k < r; ++k)
                    for (int64_t ch = c0; ch < c1; ++ch) {
                        nu[ch] += (double)m[k * C + ch] * m[k * C + ch];
                        ng[ch] += (double)gl[k * C + ch] * gl[k * C + ch];
                    }
                for (int64_t i = 0; i < R; ++i)
                    for (int64_t ch = c0; ch < c1; ++ch) nG[ch] += (double)G[i * C + ch] * G[i * C + ch];
            }
        }
        for (int64_t ch = 0; ch < nch; ++ch) {
            float s = (float)sqrt(nu[ch]) / ((float)sqrt(ng[ch]) + 1e-8f);
            if (c->scale_front) s = s * c->sqrt_scale;        /* optimizer.py:2969-2971 */
            sf[ch] = s;
            float nGf = (float)sqrt(nG[ch]);
            float nG2 = nGf * nGf;                            /* vector_norm(...).square() */
            float s2 = s * s;
            total += (double)(nG2 * s2);
        }
        free(nu);
        norm_unscaled = sqrtf((float)total);                  /* optimizer.py:2982 */
    } else {
        float s = norm2_f64(m, nl) / (norm2_f64(gl, nl) + 1e-8f);
        if (c->scale_front) s = s * c->sqrt_scale;
        for (int64_t ch = 0; ch < nch; ++ch) sf[ch] = s;
        norm_unscaled = norm2_f64(G, n) * s;                  /* optimizer.py:2988 */
    }
    float fs = 1.0f;
    if (c->fira) fs = af8o_fira_scale(norm_unscaled, c->fira_margin1, fira_has_prev, fira_prev);   /* optimizer.py:2990-2994 */
    for (int64_t ch = 0; ch < nch; ++ch) {
        float f = c->fira ? sf[ch] * fs : sf[ch];
        if (!c->scale_front) f = f * c->sqrt_scale;           /* optimizer.py:2999-3000 */
        sf[ch] = f;
    }
    float denom = 1.0f;
    if (c->d > 0.0f) { denom = norm_unscaled / c->clip_div; if (denom < 1.0f) denom = 1.0f; }   /* optimizer.py:3003-3005 */
    float us = -c->alpha / denom;                             /* optimizer.py:3013 */
    if (c->bc_mode == 1) us = us * c->bc; else if (c->bc_mode == 2) us = us / c->bc;
    if (g_pf.sr) {
        /* bf16 / fp16 parameters with stochastic rounding (optimizer.py:3061-3067): separate tensor ops,
         * param*decay, grad*final_scale, *update_scale, +, each rounded to binary32 */
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < n; ++i) {
            float pf = c->has_decay ? p[i] * c->decay : p[i];
            const float f = c->scale_tensor ? sf[0] : (right ? sf[i / C] : sf[i % C]);
            float t = G[i] * f;
            t = t * us;
            pf = pf + t;
            const float rnd = af8o_sr_uniform(g_pf.seed, g_pf.step, (uint64_t)i);
            p[i] = (g_pf.dtype == AF8O_G_BF16) ? bf16_to_f32(af8o_sr_bf16(pf, rnd)) : f16_to_f32(af8o_sr_f16(pf, rnd));
        }
    } else if (!c->scale_tensor) {
        /* optimizer.py:3074-3077: mul_ then addcmul_ in place, each rounded to the parameter's format */
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < n; ++i) {
            float pv = c->has_decay ? round_param(p[i] * c->decay) : p[i];
            float f = right ? sf[i / C] : sf[i % C];
            p[i] = round_param(fmaf(us * G[i], f, pv));
        }
    } else {
        float a = us * sf[0];                                 /* optimizer.py:3079 */
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < n; ++i) {
            float pv = c->has_decay ? round_param(p[i] * c->decay) : p[i];
            p[i] = round_param(fmaf(a, G[i], pv));
        }
    }
    if (norm_out) *norm_out = norm_unscaled;
    free(G); free(gl); free(v); free(m); free(sf);
    return rc;
}
