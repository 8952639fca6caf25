// APOLLO projection on the tensor cores for bf16 gradients:
//   right (rows >= cols):  g_low[rows x rank] = G[rows x cols]  @ Pt[cols x rank]
//   left  (rows <  cols):  g_low[rank x cols] = Pt[rank x rows] @ G[rows x cols]
// (optimizer.py:2678-2681), for many tensors in one launch.  The gradient is bf16 already; the fp32 projection is split
// into three bf16 planes P = P1 + P2 + P3 (exact to 24 bits), so each product g * p_i is
// exact in binary32 and only the accumulation rounds - the accuracy class of the fp32
// matmul the reference calls, at three bf16 MMAs per fp32 one.
//
// Both cases run as C[M x N] = A[M x K] * B[K x N] with M the long gradient dimension:
//   right: A = G (K contiguous), B = planes of Pt stored [K][N] (N contiguous)
//   left : the transposed problem C^T = G^T * Pt^T: A = G^T, read from G's rows as a
//          tile [K][M] (M contiguous); B = planes of Pt stored [N][K] (K contiguous);
//          the epilogue stores C^T transposed.
// CTA tile 128 x 128, K step 32, 16 warps as 4 x 4 (warp tile 32 x 32), four-stage
// cp.async pipeline, ldmatrix fragment loads (.trans for the tiles whose contiguous
// dimension is M or N), mma.sync.m16n8k16 with binary32 accumulators.  Rows, columns and
// rank must be multiples of 8 (16-byte copies); edges are zero-filled.
//
// Non-finite gradient entries count as zero (optimizer.py:2606): the channel-norm kernel,
// which reads the whole gradient just before, raises a device flag when it meets one, and
// only then do the CTAs clean their gradient tiles in shared memory before using them.
#pragma once

#include <cuda_bf16.h>

#include "common.cuh"

namespace af8 {

constexpr int MM_BM = 128, MM_BN = 128, MM_BK = 32, MM_STAGES = 4, MM_THREADS = 512;
constexpr int MM_FLUSH = 8;          // k-steps (256 values of K) between two roundings of the MMA accumulators into the totals
constexpr int MM_KM_STRIDE = 40;     // elements per row of a tile whose rows are K-contiguous: [128][32] + pad
constexpr int MM_MN_STRIDE = 136;    // elements per row of a tile stored [32][128] + pad
constexpr int MM_KM_TILE = 128 * MM_KM_STRIDE;   // 5120 elements
constexpr int MM_MN_TILE = 32 * MM_MN_STRIDE;    // 4352 elements

__device__ __forceinline__ void cp_async16(void *dst, const void *src, bool valid)
{
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    const int n = valid ? 16 : 0;                  // 0 bytes read: the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void *p)
{
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void *p)
{
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// P (fp32, n elements) -> three bf16 planes of n elements each
__global__ void __launch_bounds__(256)
apollo_split_kernel(const float *p, int64_t n, __nv_bfloat16 *planes)
{
    for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (int64_t)gridDim.x * 256) {
        const float x = p[i];
        const __nv_bfloat16 h1 = __float2bfloat16_rn(x);
        const float r1 = __fsub_rn(x, __bfloat162float(h1));          // exact
        const __nv_bfloat16 h2 = __float2bfloat16_rn(r1);
        const float r2 = __fsub_rn(r1, __bfloat162float(h2));         // exact
        planes[i] = h1;
        planes[n + i] = h2;
        planes[2 * n + i] = __float2bfloat16_rn(r2);
    }
}

// zero the non-finite bf16 values of one 16-byte chunk in shared memory
__device__ __forceinline__ void clean_chunk(void *p)
{
    uint4 v = *reinterpret_cast<uint4 *>(p);
    uint32_t *w = reinterpret_cast<uint32_t *>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if ((w[i] & 0x7f80u) == 0x7f80u) w[i] &= 0xffff0000u;
        if ((w[i] & 0x7f800000u) == 0x7f800000u) w[i] &= 0x0000ffffu;
    }
    *reinterpret_cast<uint4 *>(p) = v;
}

// One projection of a multi-tensor launch.  M = long gradient dimension, N = rank,
// K = contracted gradient dimension; planes: three bf16 planes shaped like Pt.
struct ProjTask {
    const __nv_bfloat16 *grad;
    const __nv_bfloat16 *planes;
    float *out;
    const int *nonfinite_flag;
    int M, N, K;
    int right, negate;
    int first_tile, tiles_n;     // CTA tiles of this task start at first_tile; tiles_n tiles along N
    int reserved;
};

// The tensor cores add into their binary32 accumulators with truncation, whose error grows
// linearly with K (measured 1.4e-5 relative at K = 4096, twelve times a binary32 GEMM with
// rounded additions).  So the MMA accumulators only ever hold MM_FLUSH k-steps (256 values
// of K); they are then added, with rounding, into a second set of registers and cleared.
// Measured after that: 8e-7 relative (rms) at every K, the error class of an fp32 GEMM.
template <bool RIGHT>
__device__ __forceinline__ void project_tile(const ProjTask &T, int m0, int n0, __nv_bfloat16 *smem)
{
    constexpr int A_TILE = RIGHT ? MM_KM_TILE : MM_MN_TILE;
    constexpr int B_TILE = RIGHT ? MM_MN_TILE : MM_KM_TILE;
    constexpr int STAGE = A_TILE + 3 * B_TILE;                  // elements
    const __nv_bfloat16 *__restrict__ grad = T.grad;
    const __nv_bfloat16 *__restrict__ planes = T.planes;
    const int M = T.M, N = T.N, K = T.K;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int wm = warp >> 2, wn = warp & 3;                    // 4 x 4 warps, warp tile 32 x 32
    const int64_t plane_elems = (int64_t)K * N;                 // both layouts hold K*N elements
    const bool dirty = *T.nonfinite_flag != 0;                  // uniform over the task

    // copy slots: a tile is 512 chunks of 16 bytes, one per thread
    //   K-contiguous tile [128][32]: row = tid / 4, k offset = (tid % 4) * 8
    //   M/N-contiguous tile [32][128]: k = tid / 16, offset = (tid % 16) * 8
    const int km_row = tid >> 2, km_k = (tid & 3) * 8;
    const int mn_k = tid >> 4, mn_o = (tid & 15) * 8;

    auto load_stage = [&](int stage, int k0) {
        __nv_bfloat16 *sa = smem + stage * STAGE, *sb = sa + A_TILE;
        if (RIGHT) {
            const bool va = (m0 + km_row < M) && (k0 + km_k < K);                 // A = G[m][k]
            cp_async16(sa + km_row * MM_KM_STRIDE + km_k, va ? grad + (int64_t)(m0 + km_row) * K + k0 + km_k : grad, va);
            const bool vb = (k0 + mn_k < K) && (n0 + mn_o < N);                   // B planes = P[k][n]
            const int64_t off = vb ? (int64_t)(k0 + mn_k) * N + n0 + mn_o : 0;
#pragma unroll
            for (int t = 0; t < 3; ++t) cp_async16(sb + t * B_TILE + mn_k * MM_MN_STRIDE + mn_o, planes + t * plane_elems + off, vb);
        } else {
            const bool va = (k0 + mn_k < K) && (m0 + mn_o < M);                   // A = G^T: tile [k][m] of G[k][m]
            cp_async16(sa + mn_k * MM_MN_STRIDE + mn_o, va ? grad + (int64_t)(k0 + mn_k) * M + m0 + mn_o : grad, va);
            const bool vb = (n0 + km_row < N) && (k0 + km_k < K);                 // B planes = Pt[n][k]
            const int64_t off = vb ? (int64_t)(n0 + km_row) * K + k0 + km_k : 0;
#pragma unroll
            for (int t = 0; t < 3; ++t) cp_async16(sb + t * B_TILE + km_row * MM_KM_STRIDE + km_k, planes + t * plane_elems + off, vb);
        }
    };

    float acc[2][4][4], total[2][4][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) { acc[i][j][e] = 0.0f; total[i][j][e] = 0.0f; }

    const int ksteps = (K + MM_BK - 1) / MM_BK;
#pragma unroll
    for (int s = 0; s < MM_STAGES - 1; ++s) {
        if (s < ksteps) load_stage(s, s * MM_BK);
        cp_async_commit();
    }

    for (int ks = 0; ks < ksteps; ++ks) {
        cp_async_wait<MM_STAGES - 2>();             // the copies of step ks have landed (this thread's)
        __syncthreads();                            // ... everyone's; and step ks-1 has been consumed by all
        {
            const int nx = ks + MM_STAGES - 1;      // refill the slot that step ks-1 used
            if (nx < ksteps) load_stage(nx % MM_STAGES, nx * MM_BK);
            cp_async_commit();
        }
        __nv_bfloat16 *sa = smem + (ks % MM_STAGES) * STAGE, *sb = sa + A_TILE;
        if (dirty) {                                // rare: zero the non-finite gradient entries of this tile
            if (RIGHT) clean_chunk(sa + km_row * MM_KM_STRIDE + km_k);
            else clean_chunk(sa + mn_k * MM_MN_STRIDE + mn_o);
            __syncthreads();
        }
#pragma unroll
        for (int kk = 0; kk < MM_BK; kk += 16) {
            uint32_t af[2][4];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int mb = wm * 32 + i * 16;
                if (RIGHT) ldmatrix_x4(af[i], sa + (mb + (lane & 7) + ((lane >> 3) & 1) * 8) * MM_KM_STRIDE + kk + (lane >> 4) * 8);
                else ldmatrix_x4_trans(af[i], sa + (kk + (lane & 7) + (lane >> 4) * 8) * MM_MN_STRIDE + mb + ((lane >> 3) & 1) * 8);
            }
#pragma unroll
            for (int t = 2; t >= 0; --t) {          // smallest plane first
                const __nv_bfloat16 *pb = sb + t * B_TILE;
#pragma unroll
                for (int jj = 0; jj < 2; ++jj) {    // two n8 tiles per ldmatrix.x4
                    const int nb = wn * 32 + jj * 16;
                    uint32_t bf[4];
                    if (RIGHT) ldmatrix_x4_trans(bf, pb + (kk + (lane & 7) + ((lane >> 3) & 1) * 8) * MM_MN_STRIDE + nb + (lane >> 4) * 8);
                    else ldmatrix_x4(bf, pb + (nb + (lane & 7) + (lane >> 4) * 8) * MM_KM_STRIDE + kk + ((lane >> 3) & 1) * 8);
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        mma_bf16(acc[i][jj * 2], af[i], bf[0], bf[1]);
                        mma_bf16(acc[i][jj * 2 + 1], af[i], bf[2], bf[3]);
                    }
                }
            }
        }
        if ((ks % MM_FLUSH) == MM_FLUSH - 1 || ks == ksteps - 1) {
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        total[i][j][e] = __fadd_rn(total[i][j][e], acc[i][j][e]);
                        acc[i][j][e] = 0.0f;
                    }
        }
    }
    cp_async_wait<0>();
    __syncthreads();                                // the ring is reused by this CTA's next tile

    // epilogue: c0,c1 = (row g, cols 2t, 2t+1), c2,c3 = (row g + 8, same cols)
    const int g = lane >> 2, t4 = lane & 3;
    const float sgn = T.negate ? -1.0f : 1.0f;
    float *__restrict__ out = T.out;
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int m = m0 + wm * 32 + i * 16 + g + h * 8;
                const int n = n0 + wn * 32 + j * 8 + t4 * 2;
                if (m < M && n < N) {               // N is even: n + 1 < N as well
                    const float x = sgn * total[i][j][h * 2], y = sgn * total[i][j][h * 2 + 1];
                    if (RIGHT) {
                        *reinterpret_cast<float2 *>(out + (int64_t)m * N + n) = make_float2(x, y);
                    } else {                        // out is [N][M]
                        out[(int64_t)n * M + m] = x;
                        out[(int64_t)(n + 1) * M + m] = y;
                    }
                }
            }
}

// Multi-tensor launch: the CTA tiles of all tasks form one flat space walked with a grid
// stride; `tasks` is sorted by first_tile.
__global__ void __launch_bounds__(MM_THREADS, 1)
apollo_project_mma_kernel(const ProjTask *__restrict__ tasks, int n_tasks, int total_tiles)
{
    extern __shared__ __align__(128) unsigned char mm_smem[];
    __shared__ ProjTask sT;
    __nv_bfloat16 *smem = reinterpret_cast<__nv_bfloat16 *>(mm_smem);
    int cur = -1;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
        int lo = 0, hi = n_tasks - 1;
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (__ldg(&tasks[mid].first_tile) <= tile) lo = mid; else hi = mid - 1;
        }
        if (lo != cur) {
            __syncthreads();
            if (threadIdx.x < (int)(sizeof(ProjTask) / 4))
                reinterpret_cast<uint32_t *>(&sT)[threadIdx.x] = __ldg(reinterpret_cast<const uint32_t *>(tasks + lo) + threadIdx.x);
            cur = lo;
            __syncthreads();
        }
        const int local = tile - sT.first_tile;
        // tiles along N are neighbours, so the CTAs that share a gradient tile run together
        const int m0 = (local / sT.tiles_n) * MM_BM, n0 = (local % sT.tiles_n) * MM_BN;
        if (sT.right) project_tile<true>(sT, m0, n0, smem);
        else project_tile<false>(sT, m0, n0, smem);
    }
}

constexpr size_t mm_smem_bytes()
{
    return (size_t)MM_STAGES * (MM_MN_TILE + 3 * MM_KM_TILE) * 2;     // the larger (left) layout
}

}  // namespace af8
