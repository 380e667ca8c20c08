// Selective state-space scan (the recurrence of a Mamba-1 mixer) over the sequences of a ragged step.
//
// Per channel c and state index n, token after token:
//
//   dt      = softplus(dt_raw[t, c] + dt_bias[c])
//   S[c, n] = exp(dt * A[c, n]) * S[c, n] + dt * x[t, c] * B[t, n],        A = -exp(A_log)
//   y[t, c] = (sum_n S[c, n] * C[t, n] + D[c] * x[t, c]) * silu(z[t, c])
//
// S is fp32 [n_slots + 1][inner][N], carried from step to step per slot (the last row belongs to no sequence).
// Everything here is fp32 arithmetic; x, B, C and z are read in the type the projections left them in, dt_raw is fp32.
//
// A channel's N state values are spread over NL adjacent lanes (NL a power of two, 8 consecutive values a lane in
// registers), which add their parts of the read-out by shuffles in a fixed order. A CTA takes one sequence and
// 128 / NL channels and walks the sequence's rows in order, so a prompt run whole, in pieces or token by token
// performs the same operations in the same order.
#include "common.cuh"

namespace {

constexpr int SCAN_THREADS = 128;              // threads that compute; as many again stage the inputs
constexpr int SCAN_R = 8;                     // state values a lane
constexpr int SCAN_TB = 16;                   // tokens staged in shared memory at a time

struct ScanArgs {
    int B, inner, N, n_slots;
    int ldx, lddt, ldbc, ldz, ldy;
    int NL;                                   // lanes a channel
    int vec;                                  // 1: rows, strides and addresses fit 16-byte (fp32: 32-byte) vectors
    // Long prompts are cut into pieces of `piece` rows that run side by side, in two passes (mode 1, then mode 2):
    //   mode 0  a CTA walks a whole sequence's rows from the slot's state (decode steps, short prompts)
    //   mode 1  a CTA walks piece k (blockIdx.z) from a ZERO state and leaves its end state P_k and the sum of its
    //           step sizes; the CTA of piece 0 also copies the slot's state aside
    //   mode 2  a CTA forms its piece's true start state, S <- exp(A * sum_j) S + P_j over the pieces j before it
    //           (the decays of a piece multiply to exp(A * sum of its step sizes)), walks the piece again and writes
    //           y; the last piece stores the slot's new state
    int mode, piece;
    float* piece_state;                       // [pieces][inner][N] (P_k), pieces numbered cu_q[b] / piece + b + k
    float* piece_dt;                          // [pieces][inner]
    float* start_state;                       // [B][inner][N]: the slot's state as the step found it
};

__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }

// A CTA has 128 computing threads and 128 staging threads. Sixteen tokens at a time go through shared memory, in two
// buffers: while the computing threads walk block k, the staging threads bring block k+1 (the CTA's channels of x, of
// the step size with its softplus applied, of silu(z), and the tokens' B and C, each lane's SCAN_R values followed by
// 4 unused floats so that the lanes of a channel read 16-byte vectors from different banks) and write block k-1's
// y = (S.C + D x) silu(z) out in whole rows. The chain from token to token then waits on no load from global memory.
template <typename TX, typename TD>
__global__ void __launch_bounds__(2 * SCAN_THREADS)
selective_scan_kernel(const TX* __restrict__ x, const float* __restrict__ dt_raw, VecRef dt_bias, VecRef A_log, VecRef Dv,
                      const TD* __restrict__ Bm, const TD* __restrict__ Cm, const TX* __restrict__ z,
                      float* __restrict__ state, TX* __restrict__ y,
                      const int* __restrict__ cu_q, const int* __restrict__ slots, ScanArgs a) {
    extern __shared__ float sm[];
    griddep_wait();
    const int b = blockIdx.y;
    const int slot = slots[b];
    const int seq0 = cu_q[b], seq1 = cu_q[b + 1];
    if (slot < 0 || slot >= a.n_slots || seq1 <= seq0) return;
    const int piece_k = a.mode == 0 ? 0 : (int)blockIdx.z;
    const int q0 = a.mode == 0 ? seq0 : seq0 + piece_k * a.piece;
    if (q0 >= seq1) return;
    const int q1 = a.mode == 0 ? seq1 : min(seq1, q0 + a.piece);
    const size_t piece_id = (size_t)(seq0 / max(a.piece, 1) + b + piece_k);
    const int NL = a.NL;
    const int CB = SCAN_THREADS / NL;             // channels of this CTA
    const bool stager = threadIdx.x >= SCAN_THREADS;
    const int tid = threadIdx.x % SCAN_THREADS;
    const int l = tid % NL, cl = tid / NL;
    const int c0 = blockIdx.x * CB;
    const int c = c0 + cl;
    const bool on = c < a.inner;
    const int cc = on ? c : a.inner - 1;          // lanes past the last channel compute and store nothing
    constexpr int CS = SCAN_R + 4;
    const int brow = CS * NL;
    const int nx = SCAN_TB * CB, nb = SCAN_TB * brow;
    float* xs = sm;                               // [2][TB][CB]
    float* ds = xs + 2 * nx;                      // [2][TB][CB] step sizes
    float* zs = ds + 2 * nx;                      // [2][TB][CB] silu(z)
    float* ys = zs + 2 * nx;                      // [2][TB][CB]
    float* bs = ys + 2 * nx;                      // [2][TB][brow]
    float* cs = bs + 2 * nb;                      // [2][TB][brow]
    for (int i = threadIdx.x; i < 4 * nb; i += 2 * SCAN_THREADS) bs[i] = 0.f;     // the unused slots stay zero
    __syncthreads();

    auto stage = [&](int k) {                     // block k of the sequence's rows -> buffer k & 1
        const int t0 = q0 + k * SCAN_TB, nt = min(SCAN_TB, q1 - t0), buf = k & 1;
        if (a.vec) {
            // eight consecutive channels a thread (at most one such piece of x, z and the step a thread, since a CTA
            // has at most 64 channels), every load issued before the first is used
            const int per_row = CB / 8;
            const int tt = tid / per_row, c8 = (tid % per_row) * 8;
            const bool act = tid < nt * per_row && c0 + c8 < a.inner;
            float xv[8], zv[8], dv[8];
            if (act) {
                load8(x + (size_t)(t0 + tt) * a.ldx + c0 + c8, xv);
                if (a.mode != 1) load8(z + (size_t)(t0 + tt) * a.ldz + c0 + c8, zv);
                load8(dt_raw + (size_t)(t0 + tt) * a.lddt + c0 + c8, dv);
            }
            const int n8 = a.N / 8;
            for (int idx = tid; idx < nt * n8; idx += SCAN_THREADS) {
                const int bt = idx / n8, g8 = idx % n8;
                float bv[8], cv[8];
                load8(Bm + (size_t)(t0 + bt) * a.ldbc + g8 * 8, bv);
                load8(Cm + (size_t)(t0 + bt) * a.ldbc + g8 * 8, cv);
                store8(bs + buf * nb + bt * brow + g8 * CS, bv);
                store8(cs + buf * nb + bt * brow + g8 * CS, cv);
            }
            if (tid < nt * per_row) {
#pragma unroll
                for (int e = 0; e < 8; e++) {
                    xv[e] = act ? xv[e] : 0.f;
                    dv[e] = act ? softplus_f(dv[e] + (dt_bias.p ? dt_bias.at(c0 + c8 + e) : 0.f)) : 0.f;
                    zv[e] = act && a.mode != 1 ? zv[e] / (1.0f + expf(-zv[e])) : 0.f;
                }
                store8(xs + buf * nx + tt * CB + c8, xv);
                store8(ds + buf * nx + tt * CB + c8, dv);
                store8(zs + buf * nx + tt * CB + c8, zv);
            }
            return;
        }
#pragma unroll 4
        for (int idx = tid; idx < nt * CB; idx += SCAN_THREADS) {
            const int tt = idx / CB, ch = c0 + idx % CB;
            const bool ok = ch < a.inner;
            const float zv = ok && a.mode != 1 ? to_f32(z[(size_t)(t0 + tt) * a.ldz + ch]) : 0.f;
            xs[buf * nx + idx] = ok ? to_f32(x[(size_t)(t0 + tt) * a.ldx + ch]) : 0.f;
            ds[buf * nx + idx] = ok ? softplus_f(dt_raw[(size_t)(t0 + tt) * a.lddt + ch] + (dt_bias.p ? dt_bias.at(ch) : 0.f)) : 0.f;
            zs[buf * nx + idx] = zv / (1.0f + expf(-zv));
        }
#pragma unroll 4
        for (int idx = tid; idx < nt * a.N; idx += SCAN_THREADS) {
            const int tt = idx / a.N, n = idx % a.N;
            const int at = buf * nb + tt * brow + (n / SCAN_R) * CS + n % SCAN_R;
            bs[at] = to_f32(Bm[(size_t)(t0 + tt) * a.ldbc + n]);
            cs[at] = to_f32(Cm[(size_t)(t0 + tt) * a.ldbc + n]);
        }
    };
    auto write_out = [&](int k) {                 // y of block k, from buffer k & 1
        if (a.mode == 1) return;
        const int t0 = q0 + k * SCAN_TB, nt = min(SCAN_TB, q1 - t0), buf = k & 1;
        for (int idx = tid; idx < nt * CB; idx += SCAN_THREADS) {
            const int tt = idx / CB, ch = c0 + idx % CB;
            if (ch < a.inner) y[(size_t)(t0 + tt) * a.ldy + ch] = from_f32<TX>(ys[buf * nx + idx]);
        }
    };

    float S[SCAN_R], A[SCAN_R];
    float* st = state + ((size_t)slot * a.inner + cc) * a.N;
    float Dc = 0.f, dt_sum = 0.f;
    if (!stager) {
        const float* init = a.mode == 2 ? a.start_state + ((size_t)b * a.inner + cc) * a.N : st;
#pragma unroll
        for (int r = 0; r < SCAN_R; r++) {
            const int n = l * SCAN_R + r;
            S[r] = (n < a.N && a.mode != 1) ? init[n] : 0.f;
            A[r] = n < a.N ? -expf(A_log.at(cc * a.N + n)) : 0.f;
        }
        Dc = Dv.p ? Dv.at(cc) : 0.f;
        if (a.mode == 1 && piece_k == 0 && on) {              // the state as the step found it, for the second pass
            float* keep = a.start_state + ((size_t)b * a.inner + cc) * a.N;
#pragma unroll
            for (int r = 0; r < SCAN_R; r++) {
                const int n = l * SCAN_R + r;
                if (n < a.N) keep[n] = st[n];
            }
        }
        if (a.mode == 2) {
            for (int j = 0; j < piece_k; j++) {               // the pieces before this one, in order
                const size_t pj = piece_id - piece_k + j;
                const float sdt = a.piece_dt[pj * a.inner + cc];
                const float* P = a.piece_state + (pj * a.inner + cc) * a.N;
#pragma unroll
                for (int r = 0; r < SCAN_R; r++) {
                    const int n = l * SCAN_R + r;
                    if (n < a.N) S[r] = fmaf(expf(sdt * A[r]), S[r], P[n]);
                }
            }
        }
    } else {
        stage(0);
    }
    __syncthreads();
    const int n_blocks = (q1 - q0 + SCAN_TB - 1) / SCAN_TB;
    for (int k = 0; k < n_blocks; k++) {
        if (stager) {
            if (k + 1 < n_blocks) stage(k + 1);
            if (k > 0) write_out(k - 1);
        } else {
            const int nt = min(SCAN_TB, q1 - q0 - k * SCAN_TB), buf = k & 1;
            for (int tt = 0; tt < nt; tt++) {
                const float xv = xs[buf * nx + tt * CB + cl], dt = ds[buf * nx + tt * CB + cl];
                const float dx = dt * xv;
                dt_sum += dt;
                const float4* b4 = reinterpret_cast<const float4*>(bs + buf * nb + tt * brow + l * CS);
                const float4* c4 = reinterpret_cast<const float4*>(cs + buf * nb + tt * brow + l * CS);
                float a4[4] = {0.f, 0.f, 0.f, 0.f};             // four partial sums: short chains
#pragma unroll
                for (int r = 0; r < SCAN_R; r += 4) {
                    const float4 bb = b4[r >> 2], cv = c4[r >> 2];
                    S[r] = fmaf(expf(dt * A[r]), S[r], dx * bb.x);
                    S[r + 1] = fmaf(expf(dt * A[r + 1]), S[r + 1], dx * bb.y);
                    S[r + 2] = fmaf(expf(dt * A[r + 2]), S[r + 2], dx * bb.z);
                    S[r + 3] = fmaf(expf(dt * A[r + 3]), S[r + 3], dx * bb.w);
                    a4[0] = fmaf(S[r], cv.x, a4[0]);
                    a4[1] = fmaf(S[r + 1], cv.y, a4[1]);
                    a4[2] = fmaf(S[r + 2], cv.z, a4[2]);
                    a4[3] = fmaf(S[r + 3], cv.w, a4[3]);
                }
                float acc = (a4[0] + a4[1]) + (a4[2] + a4[3]);
                for (int o = NL >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
                if (l == 0) ys[buf * nx + tt * CB + cl] = (acc + Dc * xv) * zs[buf * nx + tt * CB + cl];
            }
        }
        __syncthreads();
    }
    if (stager) {
        write_out(n_blocks - 1);
    } else if (on && a.mode == 1) {
        float* P = a.piece_state + (piece_id * a.inner + cc) * a.N;
#pragma unroll
        for (int r = 0; r < SCAN_R; r++) {
            const int n = l * SCAN_R + r;
            if (n < a.N) P[n] = S[r];
        }
        if (l == 0) a.piece_dt[piece_id * a.inner + cc] = dt_sum;
    } else if (on && (a.mode == 0 || q1 == seq1)) {
#pragma unroll
        for (int r = 0; r < SCAN_R; r++) {
            const int n = l * SCAN_R + r;
            if (n < a.N) st[n] = S[r];
        }
    }
}

}  // namespace

// x, z, y: [T, ld*] in act_dtype; dt_raw fp32 [T, lddt] (the step projection's output before bias and softplus);
// Bm and Cm [T, ldbc] in proj_dtype (the type their projection was left in); dt_bias, D [inner] and A_log
// [inner, N] in w_dtype; state fp32.
MYNAH_API int mynah_selective_scan(const void* x, int ldx, const void* z, int ldz, void* y, int ldy, int act_dtype,
                                   const float* dt_raw, int lddt, const void* Bm, const void* Cm, int ldbc, int proj_dtype,
                                   const void* dt_bias, const void* A_log, const void* Dv, int w_dtype,
                                   float* state, int n_slots, const int* cu_q, const int* slots,
                                   int B, int inner, int N, int piece, int n_pieces, int max_q_len, float* scratch, cudaStream_t stream) {
    if (B == 0) return 0;
    MYNAH_REQUIRE(B > 0 && inner > 0 && N > 0, "selective_scan: bad sizes B=%d inner=%d N=%d", B, inner, N);
    MYNAH_REQUIRE(N <= 32 * SCAN_R, "selective_scan: a state of %d values a channel exceeds %d", N, 32 * SCAN_R);
    MYNAH_REQUIRE(B <= 65535, "selective_scan: %d sequences exceed one launch", B);
    int NL = 2;                                                 // at least two: a CTA then stages at most 64 channels
    while (NL * SCAN_R < N) NL <<= 1;
    auto fits = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 31) == 0; };
    const int vec = inner % 8 == 0 && N % 8 == 0 && ldx % 8 == 0 && ldz % 8 == 0 && lddt % 8 == 0 && ldbc % 8 == 0 &&
                    (SCAN_THREADS / NL) % 8 == 0 && fits(x) && fits(z) && fits(dt_raw) && fits(Bm) && fits(Cm);
    // piece > 0: the two passes over pieces of `piece` rows; scratch then holds n_pieces * inner * (N + 1) +
    // B * inner * N floats and n_pieces >= rows / piece + B + 1
    MYNAH_REQUIRE(piece == 0 || (piece > 0 && n_pieces > 0 && scratch != nullptr), "selective_scan: pieces need their scratch");
    ScanArgs a{B, inner, N, n_slots, ldx, lddt, ldbc, ldz, ldy, NL, vec, 0, piece, scratch,
               scratch ? scratch + (size_t)n_pieces * inner * N : nullptr,
               scratch ? scratch + (size_t)n_pieces * inner * (N + 1) : nullptr};
    const VecRef bias{dt_bias, w_dtype}, al{A_log, w_dtype}, dv{Dv, w_dtype};
    dim3 grid(ceil_div(inner, SCAN_THREADS / NL), B);
    const size_t smem = sizeof(float) * ((size_t)8 * SCAN_TB * (SCAN_THREADS / NL) + (size_t)4 * SCAN_TB * (SCAN_R + 4) * NL);
    auto launch_once = [&]() -> int {
#define SCAN_LAUNCH(TX, TD)                                                                                              \
    if (smem > 48 * 1024 &&                                                                                              \
        cudaFuncSetAttribute(selective_scan_kernel<TX, TD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) \
        return mynah_fail("selective_scan: %zu bytes of shared memory are not to be had", smem);                        \
    mynah_launch(selective_scan_kernel<TX, TD>, grid, dim3(2 * SCAN_THREADS), smem, stream, (const TX*)x, dt_raw, bias, al, \
                 dv, (const TD*)Bm, (const TD*)Cm, (const TX*)z, state, (TX*)y, cu_q, slots, a)
        if (act_dtype == MYNAH_F32 && proj_dtype == MYNAH_F32) { SCAN_LAUNCH(float, float); }
        else if (act_dtype == MYNAH_BF16 && proj_dtype == MYNAH_F32) { SCAN_LAUNCH(bf16, float); }
        else if (act_dtype == MYNAH_BF16 && proj_dtype == MYNAH_BF16) { SCAN_LAUNCH(bf16, bf16); }
        else return mynah_fail("selective_scan: unsupported dtypes %d, %d", act_dtype, proj_dtype);
#undef SCAN_LAUNCH
        return mynah_check_launch("selective_scan");
    };
    if (piece == 0) return launch_once();
    MYNAH_REQUIRE(max_q_len > 0 && ceil_div(max_q_len, piece) <= 65535, "selective_scan: too many pieces a sequence");
    grid.z = ceil_div(max_q_len, piece);
    a.mode = 1;
    if (launch_once()) return -1;
    a.mode = 2;
    return launch_once();
}
