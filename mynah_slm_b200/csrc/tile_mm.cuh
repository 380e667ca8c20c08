// A CTA's tile of a matrix product whose A rows are found through a list of row pointers: the core of the
// products that the library's plain kernels cannot take because their rows are gathered (a token's rows of one
// expert) or their operands strided per head.
//
//   acc[i][j] = sum_k A_row(i)[k] * W[col0 + j][k]        i < BM, j < BN, k < K ascending
//
// 256 threads; thread (ty, tx) = (tid / 16, tid % 16) owns rows ty + 16 i and columns tx + 16 j. Both operands
// pass through shared memory as floats in blocks of 16 values of k; every output is ONE chain of fused
// multiply-adds over ascending k with an fp32 accumulator, so a row's result does not depend on which other rows
// share the tile, and the same code serves the bfloat16 run and the true 32-bit run.
#pragma once

#include "common.cuh"

namespace tilemm {

constexpr int THREADS = 256;
constexpr int BK = 16;

template <int BM, int BN>
struct Smem {
    float a[BK][BM + 1];
    float b[BK][BN + 1];
    const void* rows[BM];
};

// rows[i]: pointer to the first of the K values of A row i, or nullptr (a row of zeros). W: first of the
// weight's rows of this tile, `ldw` apart; rows from n_cols on read as zeros.
template <typename TA, int BM, int BN>
__device__ __forceinline__ void run(Smem<BM, BN>& s, const TA* __restrict__ W, size_t ldw, int n_cols, int K,
                                    float (&acc)[BM / 16][BN / 16]) {
    constexpr int TM = BM / 16, TN = BN / 16;
    const int tid = threadIdx.x, ty = tid / 16, tx = tid % 16;
#pragma unroll
    for (int i = 0; i < TM; i++)
#pragma unroll
        for (int j = 0; j < TN; j++) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += BK) {
        __syncthreads();
        for (int idx = tid; idx < BM * BK; idx += THREADS) {
            const int r = idx / BK, k = idx % BK;
            const TA* p = static_cast<const TA*>(s.rows[r]);
            s.a[k][r] = (p != nullptr && k0 + k < K) ? to_f32(p[k0 + k]) : 0.f;
        }
        for (int idx = tid; idx < BN * BK; idx += THREADS) {
            const int c = idx / BK, k = idx % BK;
            s.b[k][c] = (c < n_cols && k0 + k < K) ? to_f32(W[(size_t)c * ldw + k0 + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; k++) {
            float av[TM], bv[TN];
#pragma unroll
            for (int i = 0; i < TM; i++) av[i] = s.a[k][ty + 16 * i];
#pragma unroll
            for (int j = 0; j < TN; j++) bv[j] = s.b[k][tx + 16 * j];
#pragma unroll
            for (int i = 0; i < TM; i++)
#pragma unroll
                for (int j = 0; j < TN; j++) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
    }
}

}  // namespace tilemm
