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
// A channel's N state values are spread over NL adjacent lanes (NL a power of two, N / NL <= 8 values a lane in
// registers), which add their parts of the read-out by shuffles in a fixed order. A CTA takes one sequence and
// 128 / NL channels and walks the sequence's rows in order, so a prompt run whole, in pieces or token by token
// performs the same operations in the same order.
#include "common.cuh"

namespace {

constexpr int SCAN_THREADS = 128;
constexpr int SCAN_R = 8;                     // state values a lane

struct ScanArgs {
    int B, inner, N, n_slots;
    int ldx, lddt, ldbc, ldz, ldy;
    int NL;                                   // lanes a channel
};

__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }

template <typename TX, typename TD>
__global__ void __launch_bounds__(SCAN_THREADS)
selective_scan_kernel(const TX* __restrict__ x, const float* __restrict__ dt_raw, VecRef dt_bias, VecRef A_log, VecRef Dv,
                      const TD* __restrict__ Bm, const TD* __restrict__ Cm, const TX* __restrict__ z,
                      float* __restrict__ state, TX* __restrict__ y,
                      const int* __restrict__ cu_q, const int* __restrict__ slots, ScanArgs a) {
    griddep_wait();
    const int b = blockIdx.y;
    const int slot = slots[b];
    const int q0 = cu_q[b], q1 = cu_q[b + 1];
    if (slot < 0 || slot >= a.n_slots || q1 <= q0) return;
    const int NL = a.NL;
    const int l = threadIdx.x % NL;
    const int c = blockIdx.x * (SCAN_THREADS / NL) + threadIdx.x / NL;
    const bool on = c < a.inner;
    const int cc = on ? c : a.inner - 1;          // lanes past the last channel compute and store nothing

    float S[SCAN_R], A[SCAN_R];
    float* st = state + ((size_t)slot * a.inner + cc) * a.N;
#pragma unroll
    for (int r = 0; r < SCAN_R; r++) {
        const int n = l + r * NL;
        S[r] = n < a.N ? st[n] : 0.f;
        A[r] = n < a.N ? -expf(A_log.at(cc * a.N + n)) : 0.f;
    }
    const float bias = dt_bias.p ? dt_bias.at(cc) : 0.f;
    const float Dc = Dv.p ? Dv.at(cc) : 0.f;

    for (int t = q0; t < q1; t++) {
        const float xv = to_f32(x[(size_t)t * a.ldx + cc]);
        const float dt = softplus_f(dt_raw[(size_t)t * a.lddt + cc] + bias);
        const float dx = dt * xv;
        const TD* Bt = Bm + (size_t)t * a.ldbc;
        const TD* Ct = Cm + (size_t)t * a.ldbc;
        float acc = 0.f;
#pragma unroll
        for (int r = 0; r < SCAN_R; r++) {
            const int n = l + r * NL;
            if (n < a.N) {
                S[r] = fmaf(expf(dt * A[r]), S[r], dx * to_f32(Bt[n]));
                acc = fmaf(S[r], to_f32(Ct[n]), acc);
            }
        }
        for (int o = NL >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (on && l == 0) {
            const float zv = to_f32(z[(size_t)t * a.ldz + c]);
            const float out = (acc + Dc * xv) * (zv / (1.0f + expf(-zv)));
            y[(size_t)t * a.ldy + c] = from_f32<TX>(out);
        }
    }
    if (on) {
#pragma unroll
        for (int r = 0; r < SCAN_R; r++) {
            const int n = l + r * NL;
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
                                   int B, int inner, int N, cudaStream_t stream) {
    if (B == 0) return 0;
    MYNAH_REQUIRE(B > 0 && inner > 0 && N > 0, "selective_scan: bad sizes B=%d inner=%d N=%d", B, inner, N);
    MYNAH_REQUIRE(N <= 32 * SCAN_R, "selective_scan: a state of %d values a channel exceeds %d", N, 32 * SCAN_R);
    MYNAH_REQUIRE(B <= 65535, "selective_scan: %d sequences exceed one launch", B);
    int NL = 1;
    while (NL * SCAN_R < N) NL <<= 1;
    const ScanArgs a{B, inner, N, n_slots, ldx, lddt, ldbc, ldz, ldy, NL};
    const VecRef bias{dt_bias, w_dtype}, al{A_log, w_dtype}, dv{Dv, w_dtype};
    const dim3 grid(ceil_div(inner, SCAN_THREADS / NL), B);
#define SCAN_LAUNCH(TX, TD)                                                                                              \
    mynah_launch(selective_scan_kernel<TX, TD>, grid, dim3(SCAN_THREADS), 0, stream, (const TX*)x, dt_raw, bias, al, \
                 dv, (const TD*)Bm, (const TD*)Cm, (const TX*)z, state, (TX*)y, cu_q, slots, a)
    if (act_dtype == MYNAH_F32 && proj_dtype == MYNAH_F32) SCAN_LAUNCH(float, float);
    else if (act_dtype == MYNAH_BF16 && proj_dtype == MYNAH_F32) SCAN_LAUNCH(bf16, float);
    else if (act_dtype == MYNAH_BF16 && proj_dtype == MYNAH_BF16) SCAN_LAUNCH(bf16, bf16);
    else return mynah_fail("selective_scan: unsupported dtypes %d, %d", act_dtype, proj_dtype);
#undef SCAN_LAUNCH
    return mynah_check_launch("selective_scan");
}
