// APOLLO projection, "right" case (rows >= cols), on the fifth-generation tensor cores:
//   g_low[M x N] = G[M x K] @ Pt[K x N],   M = rows, K = cols, N = rank
// with the same three-plane bf16 split of Pt as apollo_mma.cuh.  tcgen05.mma reads both
// operands from shared memory and accumulates in tensor memory (TMEM); one thread issues
// the instructions, four warps feed shared memory and later drain the accumulator.
//
// Operands are K-major without swizzle: a tile is a grid of 8-row x 16-byte "core
// matrices" (128 contiguous bytes each); core matrices that follow one another along K are
// 128 bytes apart (leading byte offset), 8-row groups 512 bytes apart (stride byte offset)
// for the 32-element K step of a stage.  The gradient already has K contiguous; the planes
// of Pt are written transposed ([N][K]) by the split kernel.
//
// CTA = 160 threads, one CTA per SM, persistent over (task, M tile) pairs:
//   warps 0-3  cp.async loaders (128 threads), then epilogue: tcgen05.ld of the 128 x N
//              accumulator (warp w owns TMEM lanes 32w..32w+31) and stores to g_low
//   warp 4     allocates / frees TMEM; its lane 0 issues the MMAs and the commits
// Four 56 KB stages; "full" barriers are arrived on by the loaders after their copies have
// landed and been fenced for the asynchronous proxy, "empty" barriers by tcgen05.commit.
// Every wait is bounded (two seconds of %globaltimer); on a time-out the CTA raises the
// device error flag, skips its remaining work, frees its TMEM and returns.
#pragma once

#include <cuda_bf16.h>

#include "common.cuh"
#include "fullrank_fast.cuh"     // mbarrier helpers, g_device_error
#include "apollo_mma.cuh"        // ProjTask, cp_async16, clean_chunk

namespace af8 {

constexpr int UM_BM = 128, UM_BK = 32, UM_STAGES = 4, UM_THREADS = 288, UM_WORKERS = 256, UM_MMA_WARP = 8;
constexpr int UM_FLUSH = 8;        // stages (256 values of K) per accumulator chunk
constexpr int UM_MAXN = 256;
constexpr int UM_A_BYTES = UM_BM * UM_BK * 2;                 // 8 KB
constexpr int UM_B_BYTES = UM_MAXN * UM_BK * 2;               // 16 KB per plane
constexpr int UM_STAGE_BYTES = UM_A_BYTES + 3 * UM_B_BYTES;   // 56 KB
constexpr int UM_LBO = 128, UM_SBO = (UM_BK / 8) * 128;       // bytes
constexpr int DEVERR_UMMA_TIMEOUT = 2;

__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t smem_addr)
{
    // start address, leading and stride byte offsets in units of 16 bytes; descriptor version 1;
    // no swizzle (layout type 0)
    return (uint64_t)((smem_addr >> 4) & 0x3fffu) | ((uint64_t)(UM_LBO >> 4) << 16) | ((uint64_t)(UM_SBO >> 4) << 32) |
           (1ull << 46);
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

__global__ void __launch_bounds__(UM_THREADS, 1)
apollo_project_umma_kernel(const ProjTask *__restrict__ tasks, int n_tasks, int total_tiles)
{
    extern __shared__ __align__(1024) unsigned char um_smem[];
    __shared__ __align__(8) uint64_t s_full[UM_STAGES], s_empty[UM_STAGES], s_acc_full[2], s_acc_empty[2], s_done;
    __shared__ uint32_t s_tmem;
    __shared__ int s_abort;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int s = 0; s < UM_STAGES; ++s) { mbar_init(&s_full[s], UM_WORKERS); mbar_init(&s_empty[s], 1); }
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

    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
        if (volatile_load(&s_abort)) break;
        int lo = 0, hi = n_tasks - 1;
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (__ldg(&tasks[mid].first_tile) <= tile) lo = mid; else hi = mid - 1;
        }
        const ProjTask *T = tasks + lo;
        const int M = __ldg(&T->M), N = __ldg(&T->N), K = __ldg(&T->K);
        const int m0 = (tile - __ldg(&T->first_tile)) * UM_BM;
        const int ksteps = (K + UM_BK - 1) / UM_BK;
        const int nchunks = (ksteps + UM_FLUSH - 1) / UM_FLUSH;
        bool failed = false;

        if (warp < UM_MMA_WARP) {
            // ---------------- loaders / flushers (256 threads) ----------------
            const __nv_bfloat16 *__restrict__ grad = T->grad;
            const __nv_bfloat16 *__restrict__ planes = T->planes;
            const bool dirty = __ldg(T->nonfinite_flag) != 0;
            const int64_t plane_elems = (int64_t)K * N;
            const int kc = tid & 3, r_in = tid >> 2;            // 16-byte chunk along K; row inside a 64-row slab
            const uint32_t dst0 = (uint32_t)((r_in >> 3) * UM_SBO + kc * UM_LBO + (r_in & 7) * 16);
            const __nv_bfloat16 *a_src = grad + (int64_t)(m0 + r_in) * K + kc * 8;
            const __nv_bfloat16 *b_src = planes + (int64_t)r_in * K + kc * 8;
            const int64_t slab = (int64_t)64 * K;               // 64 rows further down
            // this thread's part of the accumulator: TMEM lanes 32 (warp % 4) + lane, columns 128 (warp / 4) ...
            const int row = (warp & 3) * 32 + lane, col_half = warp >> 2;
            float total[128];
#pragma unroll
            for (int i = 0; i < 128; ++i) total[i] = 0.0f;

            auto issue = [&](int ks) {
                unsigned char *st = um_smem + ((fills + ks) % UM_STAGES) * UM_STAGE_BYTES;
                const int k0 = ks * UM_BK;
                const bool kv = k0 + kc * 8 < K;
#pragma unroll
                for (int rr = 0; rr < 2; ++rr) {                // A: 128 rows
                    const bool v = kv && (m0 + rr * 64 + r_in < M);
                    cp_async16(st + dst0 + rr * 8 * UM_SBO, v ? a_src + rr * slab + k0 : grad, v);
                }
                for (int t = 0; t < 3; ++t) {
                    unsigned char *sb = st + UM_A_BYTES + t * UM_B_BYTES + dst0;
                    const __nv_bfloat16 *src = b_src + t * plane_elems + k0;
                    for (int rr = 0; rr * 64 < N; ++rr) {       // B plane t: N rows
                        const bool v = kv && (rr * 64 + r_in < N);
                        cp_async16(sb + rr * 8 * UM_SBO, v ? src + rr * slab : planes, v);
                    }
                }
            };
            auto publish = [&](int ks) {                        // this thread's copies of step ks have landed
                if (dirty) {
                    unsigned char *st = um_smem + ((fills + ks) % UM_STAGES) * UM_STAGE_BYTES;
#pragma unroll
                    for (int rr = 0; rr < 2; ++rr) clean_chunk(st + dst0 + rr * 8 * UM_SBO);
                }
                fence_proxy_async();
                mbar_arrive(&s_full[(fills + ks) % UM_STAGES]);
            };
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

            constexpr int LAG = UM_STAGES - 1;
            int flushed = 0;
            for (int ks = 0; ks < ksteps && !failed; ++ks) {
                if (ks >= LAG) {
                    cp_async_wait<LAG - 1>();                   // groups 0 .. ks-LAG are complete
                    publish(ks - LAG);
                }
                const int f = fills + ks, slot = f % UM_STAGES, use = f / UM_STAGES;
                if (use >= 1 && !mbar_wait_bounded(&s_empty[slot], (uint32_t)(use - 1) & 1u)) { failed = true; break; }
                issue(ks);
                cp_async_commit();
                // a chunk boundary: the chunk before the one just issued finished long ago
                if ((ks % UM_FLUSH) == UM_FLUSH - 1 && flushed < ks / UM_FLUSH) {
                    if (!flush(flushed)) { failed = true; break; }
                    ++flushed;
                }
            }
            cp_async_wait<0>();
            if (!failed)
                for (int ks = max(0, ksteps - LAG); ks < ksteps; ++ks) publish(ks);
            while (!failed && flushed < nchunks) {
                if (!flush(flushed)) failed = true;
                ++flushed;
            }
            // ---------------- epilogue: the totals to g_low ----------------
            if (!failed) {
                const int m = m0 + row;
                const float sgn = __ldg(&T->negate) ? -1.0f : 1.0f;
                float *__restrict__ out = T->out;
                if (m < M) {
#pragma unroll
                    for (int q = 0; q < 32; ++q) {
                        const int n = col_half * 128 + q * 4;
                        if (n < N)
                            *reinterpret_cast<float4 *>(out + (int64_t)m * N + n) =
                                make_float4(sgn * total[4 * q], sgn * total[4 * q + 1], sgn * total[4 * q + 2], sgn * total[4 * q + 3]);
                    }
                }
            }
        } else if (lane == 0) {
            // ---------------- MMA issuer ----------------
            const uint32_t idesc = umma_instr_desc(N);
            for (int ks = 0; ks < ksteps; ++ks) {
                const int g = gchunk + ks / UM_FLUSH, buf = g & 1;
                const bool chunk_start = (ks % UM_FLUSH) == 0;
                if (chunk_start && g >= 2) {                    // the flushers have drained this buffer
                    if (!mbar_wait_bounded(&s_acc_empty[buf], (uint32_t)((g >> 1) - 1) & 1u)) { failed = true; break; }
                    tc_fence_after();
                }
                const int f = fills + ks, slot = f % UM_STAGES, use = f / UM_STAGES;
                if (!mbar_wait_bounded(&s_full[slot], (uint32_t)use & 1u)) { failed = true; break; }
                tc_fence_after();
                const uint32_t a0 = smem_base + slot * UM_STAGE_BYTES;
                const uint32_t d = tmem + (uint32_t)(buf * UM_MAXN);
#pragma unroll
                for (int k16 = 0; k16 < UM_BK / 16; ++k16) {
                    const uint64_t ad = umma_smem_desc(a0 + k16 * 2 * UM_LBO);
#pragma unroll
                    for (int t = 2; t >= 0; --t) {              // smallest plane first
                        const uint64_t bd = umma_smem_desc(a0 + UM_A_BYTES + t * UM_B_BYTES + k16 * 2 * UM_LBO);
                        umma_bf16(d, ad, bd, idesc, (!chunk_start || k16 > 0 || t < 2) ? 1u : 0u);
                    }
                }
                umma_commit(&s_empty[slot]);                    // frees the slot when these MMAs are done
                if ((ks % UM_FLUSH) == UM_FLUSH - 1 || ks == ksteps - 1) umma_commit(&s_acc_full[buf]);
            }
        }
        if (failed) {
            s_abort = 1;
            atomicExch(&g_device_error, DEVERR_UMMA_TIMEOUT);
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
