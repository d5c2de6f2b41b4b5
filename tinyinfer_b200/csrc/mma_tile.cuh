// A 32 x 128 (MI = 2) or 64 x 128 (MI = 4) output tile of x . w^T on the warp-level tensor-core path (mma.sync m16n8k16, bfloat16 in, float32
// accumulators) for products whose row tiles are too short, too scattered or too many-shaped for the tcgen05
// kernels' 128-row tiles and tensor maps: the row tiles of routed experts (often a handful of rows an expert), the
// per-head and per-block products of the batched form. Four warps; warp w owns columns [32 w, 32 w + 32) of the
// tile for all rows. Operands come through a ring of three stages filled with 16-byte cp.async copies (rows
// and k beyond the operands are zero-filled), so a block streams its 128 weight rows at full width whatever the
// number of valid x rows. A row's result does not depend on the other rows of its tile, and k is walked in order.
//
// The caller supplies two functors: a_row(r) and b_row(n) return the address of row r of x / row n of w for this
// tile (k = 0), or nullptr for a row that does not exist. Every address and K must be a multiple of 8 elements.
// `safe`: any valid global address (the source operand of the copies that copy nothing).
#pragma once
#include "common.cuh"

namespace mt {
constexpr int BM = 32, BN = 128, BK = 32, STAGES = 3, THREADS = 128;
constexpr int LDS = BK + 8;                                   // halves per row in shared memory: ldmatrix without conflicts
constexpr int B_HALVES = BN * LDS;
template <int MI> struct Ring { static constexpr int BYTES = STAGES * (16 * MI * LDS + B_HALVES) * 2; };
constexpr int SMEM_BYTES = Ring<2>::BYTES;

__device__ __forceinline__ void cp16(void* dst, const void* src, bool valid) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void wait_group() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const __nv_bfloat16* p) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// acc[mi][ni][4]: rows 16 mi + (lane / 4) (+ 8 for elements 2, 3), columns 32 warp + 8 ni + 2 (lane % 4) (+ 1).
template <int MI, typename ARow, typename BRow>
__device__ __forceinline__ void tile_product(float (&acc)[MI][4][4], __nv_bfloat16* smem, ARow a_row, BRow b_row, int K,
                                             const __nv_bfloat16* safe) {
    constexpr int A_HALVES = 16 * MI * LDS;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    __nv_bfloat16* As = smem;
    __nv_bfloat16* Bs = smem + STAGES * A_HALVES;
#pragma unroll
    for (int mi = 0; mi < MI; ++mi)
#pragma unroll
        for (int ni = 0; ni < 4; ++ni)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[mi][ni][e] = 0.f;
    // what this thread copies in every stage: MI / 2 16-byte pieces of x, four of w
    const int a_r = tid >> 2, a_c = (tid & 3) * 8;
    const __nv_bfloat16* a_src[MI / 2];
#pragma unroll
    for (int i = 0; i < MI / 2; ++i) a_src[i] = a_row(a_r + 32 * i);
    const __nv_bfloat16* b_src[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) b_src[i] = b_row((tid >> 2) + 32 * i);
    const int steps = (K + BK - 1) / BK;
    auto load = [&](int step, int stage) {
        const int k = step * BK + a_c;
#pragma unroll
        for (int i = 0; i < MI / 2; ++i)
            cp16(As + stage * A_HALVES + (a_r + 32 * i) * LDS + a_c, (a_src[i] && k < K) ? a_src[i] + k : safe,
                 a_src[i] != nullptr && k < K);
#pragma unroll
        for (int i = 0; i < 4; ++i)
            cp16(Bs + stage * B_HALVES + ((tid >> 2) + 32 * i) * LDS + a_c, (b_src[i] && k < K) ? b_src[i] + k : safe,
                 b_src[i] != nullptr && k < K);
    };
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (s < steps) load(s, s);
        commit();
    }
    for (int step = 0; step < steps; ++step) {
        wait_group<STAGES - 2>();
        __syncthreads();
        if (step + STAGES - 1 < steps) load(step + STAGES - 1, (step + STAGES - 1) % STAGES);
        commit();
        const __nv_bfloat16* a = As + (step % STAGES) * A_HALVES;
        const __nv_bfloat16* b = Bs + (step % STAGES) * B_HALVES + warp * 32 * LDS;
#pragma unroll
        for (int kk = 0; kk < BK; kk += 16) {
            unsigned af[MI][4], bf[2][4];
#pragma unroll
            for (int mi = 0; mi < MI; ++mi)     // 16 x 16 of x: matrices (rows 0-7, k 0-7), (rows 8-15, k 0-7), (rows 0-7, k 8-15), (rows 8-15, k 8-15)
                ldmatrix_x4(af[mi], a + (mi * 16 + (lane & 15)) * LDS + kk + (lane >> 4) * 8);
#pragma unroll
            for (int nj = 0; nj < 2; ++nj)      // 16 columns x 16 of k: (n 0-7, k 0-7), (n 0-7, k 8-15), (n 8-15, k 0-7), (n 8-15, k 8-15)
                ldmatrix_x4(bf[nj], b + (nj * 16 + (lane & 7) + ((lane >> 4) << 3)) * LDS + kk + ((lane >> 3) & 1) * 8);
#pragma unroll
            for (int mi = 0; mi < MI; ++mi)
#pragma unroll
                for (int ni = 0; ni < 4; ++ni)
                    mma16816(acc[mi][ni], af[mi], bf[ni >> 1][(ni & 1) * 2], bf[ni >> 1][(ni & 1) * 2 + 1]);
        }
    }
    wait_group<0>();
    __syncthreads();                            // the ring may be filled again by the caller's next tile
}

// Calls f(row, col, value) for the two neighbouring columns (col, col + 1) a thread holds: f(row, col, v0, v1).
template <int MI, typename F>
__device__ __forceinline__ void for_each_pair(const float (&acc)[MI][4][4], F f) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
    for (int mi = 0; mi < MI; ++mi)
#pragma unroll
        for (int ni = 0; ni < 4; ++ni) {
            const int col = warp * 32 + ni * 8 + (lane & 3) * 2;
            const int row = mi * 16 + (lane >> 2);
            f(row, col, acc[mi][ni][0], acc[mi][ni][1]);
            f(row + 8, col, acc[mi][ni][2], acc[mi][ni][3]);
        }
}
}  // namespace mt
