// Shared host/device helpers of libaf8: error reporting, exactly rounded
// scalar primitives and warp/block reductions.
//
// Arithmetic contract.  The optimizer whose results this library must
// reproduce runs as a sequence of torch CPU ops, each of which rounds once to
// binary32 (reference: adafactor8bit/optimizer.py, pure-PyTorch path).  Every
// device function here therefore uses the explicitly rounded intrinsics
// (__fadd_rn, __fmul_rn, __fdiv_rn, __fsqrt_rn, __fmaf_rn), which the compiler
// never contracts or replaces by approximations, and the library is compiled
// with -fmad=false, without --use_fast_math and without flush-to-zero.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>
#include <math.h>

#include "../../include/af8.h"

namespace af8 {

// ---------------------------------------------------------------------------
// host: error reporting
// ---------------------------------------------------------------------------
inline char *error_buffer()
{
    static thread_local char buf[512] = {0};
    return buf;
}

inline int fail(int code, const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(error_buffer(), 512, fmt, ap);
    va_end(ap);
    return code;
}

#define AF8_CUDA_TRY(expr)                                                          \
    do {                                                                            \
        cudaError_t e__ = (expr);                                                   \
        if (e__ != cudaSuccess)                                                     \
            return af8::fail(AF8_ERR_CUDA, "%s failed: %s", #expr,                  \
                             cudaGetErrorString(e__));                              \
    } while (0)

inline int sm_count()
{
    static thread_local int cached_dev = -1;
    static thread_local int cached_sms = 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (dev != cached_dev) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
        cached_dev = dev;
        cached_sms = n;
    }
    return cached_sms;
}

// ---------------------------------------------------------------------------
// device: scalar primitives
// ---------------------------------------------------------------------------
// log2(1e-38f), the value torch.log2 returns for every element that
// clamp(min=1e-38) lifted (optimizer.py:309-310).
#define AF8_LOG2_TINY (-126.23327f)
#define AF8_TINY 1e-38f

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t h) { return __uint_as_float(h << 16); }

// ---------------------------------------------------------------------------
// bf16 / fp16 parameters: nearest and stochastic rounding
// (optimizer.py:162-292, 866-881; kernels.cu:48-161)
// ---------------------------------------------------------------------------
__device__ __forceinline__ float f16_bits_to_f32(uint32_t h) { return __half2float(__ushort_as_half((unsigned short)h)); }

// Tensor.to(bfloat16) / Tensor.to(float16) of a binary32 value: nearest even
__device__ __forceinline__ uint32_t f32_to_bf16_rn_bits(float x) { return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(x)); }
__device__ __forceinline__ uint32_t f32_to_f16_rn_bits(float x) { return (uint32_t)__half_as_ushort(__float2half_rn(x)); }

__device__ __forceinline__ float param_load(const void *p, int64_t i, int dtype)
{
    if (dtype == AF8_F32) return static_cast<const float *>(p)[i];
    const uint32_t h = static_cast<const uint16_t *>(p)[i];
    return dtype == AF8_BF16 ? bf16_bits_to_f32(h) : f16_bits_to_f32(h);
}
// x rounded to the nearest number of the parameter's format, as a binary32 value
__device__ __forceinline__ float param_round(float x, int dtype)
{
    if (dtype == AF8_BF16) return bf16_bits_to_f32(f32_to_bf16_rn_bits(x));
    if (dtype == AF8_F16) return f16_bits_to_f32(f32_to_f16_rn_bits(x));
    return x;
}

// The 24 random bits of element idx: SplitMix64 finaliser of counter + golden gamma, upper
// 32 bits, top 24 of those.  `base` = seed * 0x9E3779B97F4A7C15 + step * 0xD1B54A32D192ED03
// (mod 2^64) is computed on the host per parameter and step.
__device__ __forceinline__ uint32_t sr_bits24(uint64_t base, uint64_t idx)
{
    uint64_t z = base + idx + 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    return (uint32_t)(z >> 40);
}

// Stochastic rounding to bf16: the truncation lo, or lo + one unit with probability
// (x - lo) / unit = low16 / 65536.  The uniform number is r24 / 2^24, so "uniform < probability"
// is the integer comparison r24 < low16 * 256.  No step out of or into an infinity; NaN keeps
// its sign (optimizer.py:162-219).
__device__ __forceinline__ uint32_t sr_bf16_bits(float x, uint32_t r24)
{
    const uint32_t b = __float_as_uint(x);
    const uint32_t low = b & 0xffffu;
    const uint32_t lo = b >> 16;
    if ((b & 0x7fffffffu) > 0x7f800000u) return ((b >> 16) & 0x8000u) | 0x7fc0u;
    const bool can_up = low != 0u && (lo & 0x7f80u) != 0x7f80u && ((lo + 1u) & 0x7fffu) != 0x7f80u;
    return (can_up && r24 < (low << 8)) ? lo + 1u : lo;
}

// Stochastic rounding to fp16 between the two neighbours of x found from the nearest one;
// overflow saturates, infinities and NaNs keep their sign (optimizer.py:222-283).
__device__ __forceinline__ uint32_t sr_f16_bits(float x, uint32_t r24)
{
    const uint32_t sign = (__float_as_uint(x) >> 16) & 0x8000u;
    if (isnan(x)) return sign | 0x7e00u;
    if (isinf(x)) return sign | 0x7c00u;
    if (fabsf(x) > 65504.0f) return sign | 0x7bffu;
    const uint32_t q = f32_to_f16_rn_bits(x);
    const float qf = f16_bits_to_f32(q);
    if (qf == x) return q;
    const uint32_t up = (q == 0x8000u) ? 0x0001u : ((q & 0x8000u) ? q - 1u : q + 1u);
    const uint32_t down = (q == 0x0000u) ? 0x8001u : ((q & 0x8000u) ? q + 1u : q - 1u);
    const uint32_t lo_b = (qf < x) ? q : down, hi_b = (qf < x) ? up : q;
    const float lo = f16_bits_to_f32(lo_b), hi = f16_bits_to_f32(hi_b);
    const float span = __fsub_rn(hi, lo);
    if (span == 0.0f) return lo_b;
    const float prob = __fdiv_rn(__fsub_rn(x, lo), span);
    const float u = __fmul_rn((float)r24, 1.0f / 16777216.0f);
    return (u < prob) ? hi_b : lo_b;
}

// One parameter write of _apply_update_pytorch (optimizer.py:866-881) plus the weight decay
// of the prologue (optimizer.py:2033-2039):
//   fp32:            p*decay, then fma(step, u, .)
//   bf16/fp16:       the same two operations, each rounded to the parameter's format
//   stochastic:      fma(step, u, p*decay) in binary32, one stochastic rounding
// p is the loaded parameter as binary32; the result is the value to store (binary32 for fp32
// parameters, else the 16-bit pattern).
__device__ __forceinline__ uint32_t param_step_bits(float p, float decay, float step, float u, int dtype, int sr,
                                                    uint64_t sr_base, int64_t idx)
{
    if (dtype == AF8_F32) return __float_as_uint(__fmaf_rn(step, u, __fmul_rn(p, decay)));
    if (!sr) {
        const float p1 = param_round(__fmul_rn(p, decay), dtype);
        const float p2 = __fmaf_rn(step, u, p1);
        return dtype == AF8_BF16 ? f32_to_bf16_rn_bits(p2) : f32_to_f16_rn_bits(p2);
    }
    const float pf = __fmaf_rn(step, u, __fmul_rn(p, decay));
    const uint32_t r = sr_bits24(sr_base, (uint64_t)idx);
    return dtype == AF8_BF16 ? sr_bf16_bits(pf, r) : sr_f16_bits(pf, r);
}
__device__ __forceinline__ void param_store_bits(void *p, int64_t i, uint32_t bits, int dtype)
{
    if (dtype == AF8_F32) static_cast<uint32_t *>(p)[i] = bits;
    else static_cast<uint16_t *>(p)[i] = (uint16_t)bits;
}

// Tensor.lerp_(end, w) as ATen computes it (optimizer.py:698, 2119).
__device__ __forceinline__ float lerp_t(float s, float e, float w)
{
    float d = __fsub_rn(e, s);
    return (fabsf(w) < 0.5f) ? __fmaf_rn(w, d, s) : __fmaf_rn(__fsub_rn(w, 1.0f), d, e);
}

// Correctly rounded log2 of a positive finite float: evaluated in binary64
// (error below 1 ulp of binary64) and rounded once.
__device__ __forceinline__ float log2_cr(float x) { return __double2float_rn(log2((double)x)); }

// The same function with a short dependency chain, for the few calls that sit on a
// critical path (block extrema, codes in doubt): table-driven argument reduction in
// binary64.  x = 2^e * m with m in [0.75, 1.5); with c_j the nearest of 97 centres
// 0.75 + j/128 and inv_j = double(1/c_j):  log2(x) = e - log2(inv_j) + log2(1 + r),
// r = m*inv_j - 1 (one fma, |r| < 2^-7.5), log2(1 + r) by its Taylor series through
// r^7.  The table stores -log2(inv_j) for the stored inv_j, so the identity is exact;
// the centre c_32 = 1 has inv = 1 and a zero table entry, which keeps the result
// relatively accurate around x = 1.  Error about 2^-52 relative before the final
// rounding, like the library routine.  x must be positive and finite.
__constant__ double2 c_log2_tab[97] = {
#include "log2_table.inc"
};

__device__ __forceinline__ float log2_cr_fast(float x, const double2 *tab = c_log2_tab)
{
    const double xd = (double)x;
    const int hi = __double2hiint(xd);
    const int e = (hi - 0x3fe80000) >> 20;                 // 0x3fe80000: high word of 0.75
    const double m = __hiloint2double(hi - (e << 20), __double2loint(xd));
    const int j = __double2int_rn((m - 0.75) * 128.0);
    const double2 t = tab[j];
    const double r = fma(m, t.x, -1.0);
    double p = 0x1.a61762a7adedap-3;        //  1/(7 ln 2)
    p = fma(p, r, -0x1.ec709dc3a03fep-3);   // -1/(6 ln 2)
    p = fma(p, r, 0x1.2776c50ef9bfep-2);    //  1/(5 ln 2)
    p = fma(p, r, -0x1.71547652b82fep-2);   // -1/(4 ln 2)
    p = fma(p, r, 0x1.ec709dc3a03fep-2);    //  1/(3 ln 2)
    p = fma(p, r, -0x1.71547652b82fep-1);   // -1/(2 ln 2)
    p = fma(p, r, 0x1.71547652b82fep+0);    //  1/ln 2
    return __double2float_rn(fma(p, r, (double)e + t.y));
}

// Correctly rounded 2^x.
__device__ __forceinline__ float exp2_cr(float x) { return __double2float_rn(exp2((double)x)); }

// The same function for |x| <= 150 with a short instruction sequence, for the per-block
// decode tables: x = n/32 + r with n = rint(32 x), |r| <= 1/64 (both exact in binary64);
// 2^x = 2^(n >> 5) * 2^((n & 31)/32) * 2^r, the middle factor from a 32-entry table and
// 2^r = exp(r ln 2) by its Taylor series through r^6 (truncation below 2^-57).  Checked on
// the host, with the same operations, against (float)exp2((double)x) of the C library for
// every binary32 x in [-150, 150]: no difference.
#include "exp2_table.inc"
__constant__ double c_exp2_tab[32] = AF8_EXP2_TAB;

// `tab`: the 32-entry table, in constant memory (c_exp2_tab) or a copy of it in shared memory
// (indexed constant loads run on a slow path, which matters when every thread decodes)
__device__ __forceinline__ float exp2_cr_fast(float x, const double *tab = c_exp2_tab)
{
    const double xd = (double)x;
    const double z = fma(xd, 32.0, 0x1.8p52);               // n in the low word (round half to even)
    const int n = __double2loint(z);
    const double r = fma(z - 0x1.8p52, -0.03125, xd);
    double p = AF8_EXP2_C6;
    p = fma(p, r, AF8_EXP2_C5);
    p = fma(p, r, AF8_EXP2_C4);
    p = fma(p, r, AF8_EXP2_C3);
    p = fma(p, r, AF8_EXP2_C2);
    p = fma(p, r, AF8_EXP2_C1);
    p = fma(p, r, 1.0);
    const double y = tab[n & 31] * p;                       // in [1, 2.03)
    return __double2float_rn(__hiloint2double(__double2hiint(y) + ((n >> 5) << 20), __double2loint(y)));
}

// torch.rsqrt on CPU: one rounded sqrt, then one rounded reciprocal.
__device__ __forceinline__ float rsqrt_t(float x) { return __frcp_rn(__fsqrt_rn(x)); }

// log2 of a second-moment value as _log_quantize_nonneg sees it
// (optimizer.py:308-310): values below 1e-38 (zero included) are lifted to 1e-38.
__device__ __forceinline__ float al_log2(float v) { return (v > AF8_TINY) ? log2_cr(v) : AF8_LOG2_TINY; }
__device__ __forceinline__ float al_log2_fast(float v, const double2 *tab = c_log2_tab) { return (v > AF8_TINY) ? log2_cr_fast(v, tab) : AF8_LOG2_TINY; }

// AL dequantisation of one code (optimizer.py:341-349).  qm1 = levels - 2.
__device__ __forceinline__ float al_decode(uint32_t code, float scale, float min_log, float qm1)
{
    if (code == 0) return 0.0f;
    float t = __fmul_rn((float)(code - 1), scale);
    t = __fdiv_rn(t, qm1);
    t = __fadd_rn(t, min_log);
    return exp2_cr(t);
}

// AL8 dequantisation with the short sequences: x / 254 from the correctly rounded
// reciprocal and one residual step (equal to the IEEE quotient for every x >= 1e-13,
// checked exhaustively on the host; (code-1)*scale is 0 or at least 1e-12), then
// exp2_cr_fast.  min_log >= -127.3 and the block maximum is below 128, so |t| <= 150.
__device__ __forceinline__ float al8_decode_fast(uint32_t code, float scale, float min_log, const double *tab = c_exp2_tab)
{
    if (code == 0) return 0.0f;
    const float x = __fmul_rn((float)(code - 1), scale);
    const float rc = 0x1.020408p-8f;                        // fl(1 / 254)
    const float q0 = __fmul_rn(x, rc);
    const float q = __fmaf_rn(__fmaf_rn(-q0, 254.0f, x), rc, q0);
    return exp2_cr_fast(__fadd_rn(q, min_log), tab);
}

// Block range of _log_quantize_nonneg from the reduced extrema
// (optimizer.py:315-318).  mn = min of log2 over non-zero elements (+inf if
// none), mx = max over all elements.
__device__ __forceinline__ void al_range(float mn, float mx, float floor_log, float &min_log, float &scale)
{
    mn = fmaxf(mn, floor_log);
    if (mn >= mx) mn = __fsub_rn(mx, 1.0f);
    float s = __fsub_rn(mx, mn);
    scale = fmaxf(s, 1e-12f);
    min_log = mn;
}

// AL code of one element (optimizer.py:320-321).  l = al_log2(v).
__device__ __forceinline__ uint32_t al_encode(float v, float l, float min_log, float scale, float qm1, int qmax)
{
    if (v == 0.0f) return 0u;
    float t = __fdiv_rn(__fsub_rn(l, min_log), scale);
    t = __fmul_rn(t, qm1);
    int q = __float2int_rn(t) + 1;   // round half to even, like torch.round
    q = max(1, min(q, qmax));
    return (uint32_t)q;
}

// UF8 / UF4 code of one element (optimizer.py:512, 518).  a = block absmax >= 1e-12.
__device__ __forceinline__ uint32_t uf8_encode(float m, float a)
{
    float t = __fmul_rn(__fdiv_rn(m, a), 128.0f);
    int q = __float2int_rn(t);
    q = max(-128, min(q, 127));
    return (uint32_t)(q + 128);
}

__device__ __forceinline__ uint32_t uf4_encode(float m, float a)
{
    float t = __fmul_rn(__fdiv_rn(m, a), 8.0f);
    int q = __float2int_rn(t);
    q = max(-8, min(q, 7));
    return (uint32_t)(q + 8);
}

// ---------------------------------------------------------------------------
// device: reductions
// ---------------------------------------------------------------------------
__device__ __forceinline__ float warp_max(float x)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
    return x;
}

__device__ __forceinline__ float warp_min(float x)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x = fminf(x, __shfl_xor_sync(0xffffffffu, x, o));
    return x;
}

__device__ __forceinline__ float warp_sum(float x)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x = __fadd_rn(x, __shfl_xor_sync(0xffffffffu, x, o));
    return x;
}

}  // namespace af8
