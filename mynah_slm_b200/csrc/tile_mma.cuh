// A CTA's tile of a bfloat16 matrix product on tensor cores (mma.sync m16n8k16, fp32 accumulators) whose A rows are
// found through a list (gathered rows of one expert, or a head's slice of wider rows).
//
// The tile's rows (16 * MT of them) pass through shared memory in blocks of MMA_KC values of k; the weights stream from
// global memory (or L2, for the tiles that share a matrix) straight into the B fragments, 16 bytes a lane: lane (g, t)
// of a warp takes values [t * 8, t * 8 + 8) of row g of a k-block of 32, which feed two instructions. The instruction's
// k slots are thereby filled in another order than memory's; A is read from shared memory in the same order (values
// [t * 8, t * 8 + 8) of rows g and g + 8), and a sum over k does not care. Every output is one chain of instructions
// over ascending k-blocks whatever the tile, so a row's bits do not depend on the other rows, nor on the tile's height.
#pragma once

#include "common.cuh"

namespace tilemma {

constexpr int MMA_KC = 256;
constexpr int MMA_LDS = MMA_KC + 32;          // row stride in shared memory: 16 words off a multiple of 32 banks

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// acc[s][m][j]: stream s (one weight matrix each), m-th group of 16 rows, j-th group of 8 columns of this warp
template <int MT, int NT, int NS>
__device__ __forceinline__ void mma_tile(bf16 (*xs)[MMA_LDS], const int* row_s, const bf16* __restrict__ src, size_t ld_src,
                                         int src_div, const bf16* const (&wrow)[NS][NT], int K, float (&acc)[NS][MT][NT][4]) {
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int s = 0; s < NS; s++)
#pragma unroll
        for (int m = 0; m < MT; m++)
#pragma unroll
            for (int j = 0; j < NT; j++)
#pragma unroll
                for (int e = 0; e < 4; e++) acc[s][m][j][e] = 0.f;
    for (int k0 = 0; k0 < K; k0 += MMA_KC) {
        __syncthreads();
        for (int idx = threadIdx.x; idx < 16 * MT * (MMA_KC / 8); idx += blockDim.x) {
            const int r = idx / (MMA_KC / 8), kk = (idx % (MMA_KC / 8)) * 8;
            const int p = row_s[r];
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (p >= 0 && k0 + kk < K) v = *reinterpret_cast<const uint4*>(src + (size_t)(p / src_div) * ld_src + k0 + kk);
            *reinterpret_cast<uint4*>(&xs[r][kk]) = v;
        }
        __syncthreads();
        const int kend = min(MMA_KC, K - k0);
        // the weights of the k-blocks after the ones being multiplied are already on their way: one block ahead under
        // a tall tile (registers are the accumulators'), four under a 16-row tile (a decode step lives on loads in flight)
        constexpr int DEPTH = MT == 1 ? 4 : 1;
        auto fetch = [&](int kb, uint4 (&b)[DEPTH][NS][NT]) {
#pragma unroll
            for (int dd = 0; dd < DEPTH; dd++) {
                const bool in = kb + 32 * dd + t * 8 < kend;      // K is a multiple of 8: a lane's 8 values are all in or all out
#pragma unroll
                for (int s = 0; s < NS; s++)
#pragma unroll
                    for (int j = 0; j < NT; j++)
                        b[dd][s][j] = in ? __ldg(reinterpret_cast<const uint4*>(wrow[s][j] + k0 + kb + 32 * dd + t * 8))
                                         : make_uint4(0u, 0u, 0u, 0u);
            }
        };
        uint4 b[DEPTH][NS][NT], bn[DEPTH][NS][NT];
        fetch(0, b);
        for (int kb = 0; kb < kend; kb += 32 * DEPTH) {
            fetch(kb + 32 * DEPTH, bn);                           // beyond the block: zeros, not used
#pragma unroll
            for (int dd = 0; dd < DEPTH; dd++) {                  // (blocks beyond kend multiply zeros; they stay inside xs)
#pragma unroll
                for (int m = 0; m < MT; m++) {
                    const uint4 lo = *reinterpret_cast<const uint4*>(&xs[m * 16 + g][kb + 32 * dd + t * 8]);
                    const uint4 hi = *reinterpret_cast<const uint4*>(&xs[m * 16 + g + 8][kb + 32 * dd + t * 8]);
#pragma unroll
                    for (int s = 0; s < NS; s++)
#pragma unroll
                        for (int j = 0; j < NT; j++) {
                            mma_bf16(acc[s][m][j], lo.x, hi.x, lo.y, hi.y, b[dd][s][j].x, b[dd][s][j].y);
                            mma_bf16(acc[s][m][j], lo.z, hi.z, lo.w, hi.w, b[dd][s][j].z, b[dd][s][j].w);
                        }
                }
            }
#pragma unroll
            for (int dd = 0; dd < DEPTH; dd++)
#pragma unroll
                for (int s = 0; s < NS; s++)
#pragma unroll
                    for (int j = 0; j < NT; j++) b[dd][s][j] = bn[dd][s][j];
        }
    }
}


}  // namespace tilemma
