// APOLLO projection, "right" case (rows >= cols), on the fifth-generation tensor cores:
//   g_low[M x N] = G[M x K] @ Pt[K x N],   M = rows, K = cols, N = rank
// with the same three-plane bf16 split of Pt as apollo_mma.cuh.  tcgen05.mma reads both
// operands from shared memory and accumulates in tensor memory (TMEM).
//
// Operands are K-major with the 64-byte swizzle: a stage holds 32 values of K, i.e. rows of
// 64 bytes, written by tiled bulk tensor copies (TMA) whose tensor maps use
// CU_TENSOR_MAP_SWIZZLE_64B; the matrix descriptors name the same swizzle, 512 bytes between
// 8-row groups, and advance by 32 bytes per 16 values of K.  The gradient already has K
// contiguous; the planes of Pt are written transposed ([3][N][K]) by the split kernel and
// arrive with one three-dimensional copy per stage.
//
// CTA = 320 threads, one CTA per SM, persistent over (task, M tile) pairs:
//   warps 0-7  read every gradient tile from shared memory before its MMAs: they add up the
//              squares of each row (the channel norms ||G_row||^2 that the scaling step needs,
//              so the gradient is read from memory once) and zero non-finite entries; then
//              drain the accumulator: warp w owns TMEM lanes 32 (w % 4) .. +31 and columns
//              128 (w / 4) .. +127, 128 totals per thread; then store g_low and the norms.
//   warp 8     allocates / frees TMEM; its lane 0 issues the MMAs and the commits
//   warp 9     lane 0 issues the copies
// Four 56 KB stages; a "full" barrier completes on the copies' transaction bytes, a "clean"
// barrier when the 256 workers have read (and, rarely, repaired) the gradient tile, an "empty"
// barrier on tcgen05.commit.
//
// The tensor cores add into their binary32 accumulators with truncation, whose error grows
// linearly with K (measured 1.4e-5 relative at K = 4096, as with mma.sync).  The accumulation
// is therefore cut into chunks of 256 values of K that alternate between two TMEM accumulators;
// while one is being filled the other is added, with rounding, into the workers' registers.
//
// Every wait is bounded (two seconds of %globaltimer); on a time-out the thread raises the
// device error flag and leaves; the others follow at their next wait or tile, and the tensor
// memory is freed after all have reported (or after a bounded wait).  After the start-up
// barrier no block-wide barrier is used, so a lost role cannot hang the others.  No copy
// uses cluster multicast.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>

#include "common.cuh"
#include "fullrank_fast.cuh"     // mbarrier helpers, g_device_error
#include "tensormap.cuh"         // tiled bulk tensor copies
#include "apollo_mma.cuh"        // ProjTask, clean_chunk

namespace af8 {

constexpr int UM_BM = 128, UM_BK = 32, UM_STAGES = 4, UM_THREADS = 320, UM_WORKERS = 256, UM_MMA_WARP = 8, UM_TMA_WARP = 9;
constexpr int UM_FLUSH = 8;        // stages (256 values of K) per accumulator chunk
constexpr int UM_MAXN = 256;
constexpr int UM_ROW_BYTES = UM_BK * 2;                       // 64
constexpr int UM_A_BYTES = UM_BM * UM_ROW_BYTES;              // 8 KB
constexpr int UM_B_BYTES = UM_MAXN * UM_ROW_BYTES;            // 16 KB per plane at N = 256
constexpr int UM_STAGE_BYTES = UM_A_BYTES + 3 * UM_B_BYTES;   // 56 KB
constexpr int UM_SBO = 8 * UM_ROW_BYTES;                      // 512 bytes between 8-row groups
constexpr int DEVERR_UMMA_TIMEOUT = 2;

// One projection of a tcgen05 launch: the mma.sync task plus the two tensor maps
struct __align__(64) UmmaTask {
    CUtensorMap map_a;       // G as [M][K], box 128 x 32
    CUtensorMap map_b;       // planes as [3][N][K], box 3 x N x 32
    ProjTask t;
    double *chan_g2;         // [M] sums of squares of the rows of G (non-finite entries count as zero)
    unsigned char pad[384 - 2 * sizeof(CUtensorMap) - sizeof(ProjTask) - sizeof(double *)];
};
static_assert(sizeof(CUtensorMap) == 128 && sizeof(UmmaTask) == 384, "task layout");

__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t smem_addr)
{
    // start address and stride byte offset in units of 16 bytes (the leading byte offset is not
    // used by swizzled K-major layouts); descriptor version 1; layout type 4 = 64-byte swizzle
    return (uint64_t)((smem_addr >> 4) & 0x3fffu) | ((uint64_t)1 << 16) | ((uint64_t)(UM_SBO >> 4) << 32) |
           (1ull << 46) | (4ull << 61);
}
// kind::f16 instruction descriptor: D = F32, A = B = BF16, both K-major, M = 128, N = n
__device__ __forceinline__ uint32_t umma_instr_desc(int n)
{
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(UM_BM >> 4) << 24);
}
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t *bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// G[R][C] (bf16) -> G^T[C][R], non-finite entries replaced by zero (optimizer.py:2606).
// 64 x 64 tiles.  A thread transposes 2 x 2 blocks in registers (two 32-bit loads from neighbouring
// rows become the two 32-bit words of neighbouring output rows), so shared memory only moves whole
// words through two 32 x 33 arrays, without bank conflicts; every global access of a warp is a
// contiguous run of 128 bytes.  R and C even.
__global__ void __launch_bounds__(256)
apollo_transpose_bf16_kernel(const uint16_t *__restrict__ in, int R, int C, uint16_t *__restrict__ out)
{
    __shared__ uint32_t t0[32][33], t1[32][33];       // [block column][block row]: output rows 2 bc and 2 bc + 1
    const int r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    uint32_t a[4], b[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {                      // block (row ty + 8 k, column tx): rows r, r + 1, columns c, c + 1
        const int r = r0 + 2 * (ty + 8 * k), c = c0 + 2 * tx;
        a[k] = b[k] = 0u;
        if (r < R && c < C) {
            a[k] = __ldg(reinterpret_cast<const uint32_t *>(in + (int64_t)r * C + c));
            b[k] = __ldg(reinterpret_cast<const uint32_t *>(in + (int64_t)(r + 1) * C + c));
        }
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        uint32_t x = a[k], y = b[k];
        if ((x & 0x7f80u) == 0x7f80u) x &= 0xffff0000u;
        if ((x & 0x7f800000u) == 0x7f800000u) x &= 0x0000ffffu;
        if ((y & 0x7f80u) == 0x7f80u) y &= 0xffff0000u;
        if ((y & 0x7f800000u) == 0x7f800000u) y &= 0x0000ffffu;
        t0[tx][ty + 8 * k] = __byte_perm(x, y, 0x5410);          // column c:     (row r, row r + 1)
        t1[tx][ty + 8 * k] = __byte_perm(x, y, 0x7632);          // column c + 1
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 4; ++k) {                      // output rows c, c + 1 of block column ty + 8 k; columns r, r + 1 of block row tx
        const int c = c0 + 2 * (ty + 8 * k), r = r0 + 2 * tx;
        if (c < C && r < R) {
            *reinterpret_cast<uint32_t *>(out + (int64_t)c * R + r) = t0[ty + 8 * k][tx];
            *reinterpret_cast<uint32_t *>(out + (int64_t)(c + 1) * R + r) = t1[ty + 8 * k][tx];
        }
    }
}

// Pt[K][N] (fp32) -> three bf16 planes stored [N][K]
__global__ void __launch_bounds__(256)
apollo_split_transposed_kernel(const float *__restrict__ p, int K, int N, __nv_bfloat16 *__restrict__ planes)
{
    __shared__ float tile[32][33];
    const int k0 = blockIdx.x * 32, n0 = blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;     // 32 x 8
    for (int r = ty; r < 32; r += 8) {
        const int k = k0 + r, n = n0 + tx;
        tile[r][tx] = (k < K && n < N) ? p[(int64_t)k * N + n] : 0.0f;
    }
    __syncthreads();
    const int64_t plane = (int64_t)K * N;
    for (int r = ty; r < 32; r += 8) {
        const int n = n0 + r, k = k0 + tx;
        if (n < N && k < K) {
            const float x = tile[tx][r];
            const __nv_bfloat16 h1 = __float2bfloat16_rn(x);
            const float r1 = __fsub_rn(x, __bfloat162float(h1));
            const __nv_bfloat16 h2 = __float2bfloat16_rn(r1);
            const float r2 = __fsub_rn(r1, __bfloat162float(h2));
            const int64_t o = (int64_t)n * K + k;
            planes[o] = h1;
            planes[plane + o] = h2;
            planes[2 * plane + o] = __float2bfloat16_rn(r2);
        }
    }
}

__device__ __forceinline__ int volatile_load(const int *p) { return *reinterpret_cast<const volatile int *>(p); }

// Sum of squares of the 8 bf16 values of a 16-byte chunk of a staged gradient tile.  The common
// case is eight binary32 multiply-adds; when that sum is not finite (a NaN or an infinity in the
// chunk, or squares beyond binary32) the non-finite entries are zeroed in shared memory, as the
// reference zeroes them in the gradient (optimizer.py:2606), and the sum is redone in binary64.
__device__ __forceinline__ double umma_chunk_sumsq(unsigned char *p, bool &wrote)
{
    uint4 v = *reinterpret_cast<uint4 *>(p);
    uint32_t w[4] = {v.x, v.y, v.z, v.w};
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float lo = __uint_as_float(w[i] << 16), hi = __uint_as_float(w[i] & 0xffff0000u);
        s = __fmaf_rn(lo, lo, s);
        s = __fmaf_rn(hi, hi, s);
    }
    if (s <= 3.0e38f) return (double)s;                          // false for NaN and infinity
    bool changed = false;
    double d = 0.0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if ((w[i] & 0x7f80u) == 0x7f80u) { w[i] &= 0xffff0000u; changed = true; }
        if ((w[i] & 0x7f800000u) == 0x7f800000u) { w[i] &= 0x0000ffffu; changed = true; }
        const double lo = (double)__uint_as_float(w[i] << 16), hi = (double)__uint_as_float(w[i] & 0xffff0000u);
        d += lo * lo;
        d += hi * hi;
    }
    if (changed) {
        *reinterpret_cast<uint4 *>(p) = make_uint4(w[0], w[1], w[2], w[3]);
        wrote = true;
    }
    return d;
}

__global__ void __launch_bounds__(UM_THREADS, 1)
apollo_project_umma_kernel(const UmmaTask *__restrict__ tasks, int n_tasks, int total_tiles)
{
    extern __shared__ __align__(1024) unsigned char um_smem[];
    __shared__ __align__(8) uint64_t s_full[UM_STAGES], s_clean[UM_STAGES], s_empty[UM_STAGES], s_acc_full[2], s_acc_empty[2], s_done;
    __shared__ uint32_t s_tmem;
    __shared__ int s_abort;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int s = 0; s < UM_STAGES; ++s) { mbar_init(&s_full[s], 1); mbar_init(&s_clean[s], UM_WORKERS); mbar_init(&s_empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&s_acc_full[b], 1); mbar_init(&s_acc_empty[b], UM_WORKERS); }
        mbar_init(&s_done, UM_THREADS);
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == UM_MMA_WARP) {   // all 512 columns of tensor memory: two 128 x 256 binary32 accumulators
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();             // the only block-wide barrier: after it the roles run on mbarriers alone
    tc_fence_after();
    const uint32_t tmem = s_tmem;
    const uint32_t smem_base = smem_u32(um_smem);

    // Running counters, advanced identically by every thread: stage fills and accumulator
    // chunks since the kernel started.  Use number n of a barrier = counter / ring size; the
    // consumer of use n waits for phase parity n & 1, the producer of use n >= 1 for (n-1) & 1.
    int fills = 0, gchunk = 0;
    int issued = 0;                 // producer only: stage fills issued so far

    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
        if (volatile_load(&s_abort)) break;
        int lo = 0, hi = n_tasks - 1;
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (__ldg(&tasks[mid].t.first_tile) <= tile) lo = mid; else hi = mid - 1;
        }
        const UmmaTask *U = tasks + lo;
        const ProjTask *T = &U->t;
        const int M = __ldg(&T->M), N = __ldg(&T->N), K = __ldg(&T->K);
        const int m0 = (tile - __ldg(&T->first_tile)) * UM_BM;
        const int ksteps = (K + UM_BK - 1) / UM_BK;
        const int nchunks = (ksteps + UM_FLUSH - 1) / UM_FLUSH;
        const int plane_bytes = N * UM_ROW_BYTES;
        bool failed = false;

        if (warp < UM_MMA_WARP) {
            // ---------------- workers (256 threads) ----------------
            // this thread's part of the accumulator: TMEM lanes 32 (warp % 4) + lane, columns 128 (warp / 4) ...
            const int row = (warp & 3) * 32 + lane, col_half = warp >> 2;
            float total[128];
#pragma unroll
            for (int i = 0; i < 128; ++i) total[i] = 0.0f;

            // add accumulator chunk c of this tile into the totals, with rounding, and hand the buffer back
            auto flush = [&](int c) -> bool {
                const int g = gchunk + c, buf = g & 1;
                if (!mbar_wait_bounded(&s_acc_full[buf], (uint32_t)(g >> 1) & 1u)) return false;
                tc_fence_after();
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    if (col_half * 128 + j * 16 < N) {           // uniform over the warp
                        uint32_t v[16];
                        const uint32_t taddr = tmem + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(buf * UM_MAXN + col_half * 128 + j * 16);
                        asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                                     : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                                       "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                                     : "r"(taddr));
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                        for (int e = 0; e < 16; ++e) total[j * 16 + e] = __fadd_rn(total[j * 16 + e], __uint_as_float(v[e]));
                    }
                }
                tc_fence_before();
                mbar_arrive(&s_acc_empty[buf]);
                return true;
            };
            // The 8 KB gradient tile of a stage is 512 chunks of 16 bytes, two per thread; chunk i lies in
            // row i / 4 of the tile (the swizzle permutes chunks within a row).  rs0 / rs1: this thread's
            // share of the squared norms of rows tid / 4 and 64 + tid / 4, over all of K.
            double rs0 = 0.0, rs1 = 0.0;
            auto scan = [&](int c) -> bool {
                const int k_end = min(ksteps, (c + 1) * UM_FLUSH);
                for (int ks = c * UM_FLUSH; ks < k_end; ++ks) {
                    const int f = fills + ks, slot = f % UM_STAGES;
                    if (!mbar_wait_bounded(&s_full[slot], (uint32_t)(f / UM_STAGES) & 1u)) return false;
                    unsigned char *st = um_smem + slot * UM_STAGE_BYTES;
                    bool wrote = false;
                    rs0 += umma_chunk_sumsq(st + tid * 16, wrote);
                    rs1 += umma_chunk_sumsq(st + (tid + UM_WORKERS) * 16, wrote);
                    if (wrote) fence_proxy_async();              // repaired entries must be visible to the MMAs
                    mbar_arrive(&s_clean[slot]);
                }
                return true;
            };
            for (int c = 0; c < nchunks && !failed; ++c) {
                if (!scan(c)) { failed = true; break; }
                if (c >= 1 && !flush(c - 1)) failed = true;
            }
            if (!failed && !flush(nchunks - 1)) failed = true;
            failed = __any_sync(0xffffffffu, failed);            // uniform over the warp from here on
            // ---------------- epilogue: the totals to g_low ----------------
            if (!failed) {
                const int m = m0 + row;
                const float sgn = __ldg(&T->negate) ? -1.0f : 1.0f;
                float *__restrict__ out = T->out;
                if (m < M && __ldg(&T->right)) {
#pragma unroll
                    for (int q = 0; q < 32; ++q) {
                        const int n = col_half * 128 + q * 4;
                        if (n < N)
                            *reinterpret_cast<float4 *>(out + (int64_t)m * N + n) =
                                make_float4(sgn * total[4 * q], sgn * total[4 * q + 1], sgn * total[4 * q + 2], sgn * total[4 * q + 3]);
                    }
                } else if (m < M) {
                    // left case computed as the transposed problem: g_low is [N][M]; a warp's 32
                    // rows are consecutive addresses of one output row
#pragma unroll
                    for (int e = 0; e < 128; ++e) {
                        const int n = col_half * 128 + e;
                        if (n < N) out[(int64_t)n * M + m] = sgn * total[e];
                    }
                }
                // the four threads that share a row add their parts; one of them stores the norm
                rs0 += __shfl_xor_sync(0xffffffffu, rs0, 1); rs0 += __shfl_xor_sync(0xffffffffu, rs0, 2);
                rs1 += __shfl_xor_sync(0xffffffffu, rs1, 1); rs1 += __shfl_xor_sync(0xffffffffu, rs1, 2);
                double *__restrict__ chan = U->chan_g2;
                if ((tid & 3) == 0 && chan != nullptr) {
                    const int ra = m0 + (tid >> 2), rb = ra + 64;
                    if (ra < M) chan[ra] = rs0;
                    if (rb < M) chan[rb] = rs1;
                }
            }
        } else if (warp == UM_MMA_WARP && lane == 0) {
            // ---------------- MMA issuer ----------------
            const uint32_t idesc = umma_instr_desc(N);
            for (int ks = 0; ks < ksteps; ++ks) {
                const int g = gchunk + ks / UM_FLUSH, buf = g & 1;
                const bool chunk_start = (ks % UM_FLUSH) == 0;
                if (chunk_start && g >= 2) {                    // the workers have drained this buffer
                    if (!mbar_wait_bounded(&s_acc_empty[buf], (uint32_t)((g >> 1) - 1) & 1u)) { failed = true; break; }
                    tc_fence_after();
                }
                const int f = fills + ks, slot = f % UM_STAGES, use = f / UM_STAGES;
                // the workers have read this stage (which also means that its copies have landed)
                if (!mbar_wait_bounded(&s_clean[slot], (uint32_t)use & 1u)) { failed = true; break; }
                if (!mbar_wait_bounded(&s_full[slot], (uint32_t)use & 1u)) { failed = true; break; }   // complete already: orders the copies before the MMAs in this thread
                tc_fence_after();
                const uint32_t a0 = smem_base + slot * UM_STAGE_BYTES;
                const uint32_t d = tmem + (uint32_t)(buf * UM_MAXN);
#pragma unroll
                for (int k16 = 0; k16 < UM_BK / 16; ++k16) {
                    const uint64_t ad = umma_smem_desc(a0 + k16 * 32);
#pragma unroll
                    for (int t = 2; t >= 0; --t) {              // smallest plane first
                        const uint64_t bd = umma_smem_desc(a0 + UM_A_BYTES + t * plane_bytes + k16 * 32);
                        umma_bf16(d, ad, bd, idesc, (!chunk_start || k16 > 0 || t < 2) ? 1u : 0u);
                    }
                }
                umma_commit(&s_empty[slot]);                    // frees the slot when these MMAs are done
                if ((ks % UM_FLUSH) == UM_FLUSH - 1 || ks == ksteps - 1) umma_commit(&s_acc_full[buf]);
            }
        } else if (warp == UM_TMA_WARP && lane == 0) {
            // ---------------- copies ----------------
            const uint32_t bytes = (uint32_t)(UM_A_BYTES + 3 * plane_bytes);
            for (int ks = 0; ks < ksteps; ++ks) {
                const int f = fills + ks, slot = f % UM_STAGES, use = f / UM_STAGES;
                if (use >= 1 && !mbar_wait_bounded(&s_empty[slot], (uint32_t)(use - 1) & 1u)) { failed = true; break; }
                unsigned char *st = um_smem + slot * UM_STAGE_BYTES;
                mbar_expect_tx(&s_full[slot], bytes);
                tma_load_2d(st, &U->map_a, ks * UM_BK, m0, &s_full[slot]);
                tma_load_3d(st + UM_A_BYTES, &U->map_b, ks * UM_BK, 0, 0, &s_full[slot]);
                issued = f + 1;
            }
        }
        if (failed) {
            s_abort = 1;
            atomicExch(&g_device_error, DEVERR_UMMA_TIMEOUT);
        }
        if (failed || volatile_load(&s_abort)) {
            // a role gave up: the producer gives its copies still in flight a bounded chance to land
            // before the block may end
            if (warp == UM_TMA_WARP && lane == 0)
                for (int back = 0; back < UM_STAGES && back < issued; ++back) {
                    const int f = issued - 1 - back;
                    mbar_wait_bounded(&s_full[f % UM_STAGES], (uint32_t)(f / UM_STAGES) & 1u);
                }
            break;
        }
        fills += ksteps;
        gchunk += nchunks;
    }

    // every thread reports in; the allocating warp frees the tensor memory once all have
    // (or after a bounded wait, when a role was lost to a time-out)
    mbar_arrive(&s_done);
    if (warp == UM_MMA_WARP) {
        mbar_wait_bounded(&s_done, 0u);
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
}

constexpr size_t um_smem_bytes() { return (size_t)UM_STAGES * UM_STAGE_BYTES + 1024; }

}  // namespace af8
