// Gated delta rule: a linear-attention recurrence whose per-head state S [dim x vd] is decayed, corrected
// towards the new value along the new key, and read with the query, token after token:
//
//   S <- g_t S;   u = beta_t (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T q_t
//
// (the read-out sees the token's own write). Three kernels:
//
//   delta_prep    q, k -> unit vectors per head, x / sqrt(sum(x^2) + 1e-6), q also times dim^(-1/2);
//                 beta = sigmoid(b_raw);  g = exp(-exp(A_log_h) * softplus(a_raw + dt_bias_h))       (fp32 out)
//   delta_rule    the recurrence. The columns of S are independent given k, q, g and beta, so a CTA takes a
//                 tile of columns of one head of one sequence; a column's dim values are spread over L adjacent
//                 lanes (at most 32 values a lane, in registers) that add their parts of the two dot products
//                 by shuffles in a fixed order. S is fp32 [n_slots + 1][H][dim][vd], carried per slot.
//   gated_rmsnorm out = o / rms(o over the head's vd) * w[d] * silu(gate)
//
// All arithmetic is fp32. A sequence's rows are walked in order, so a prompt run whole, in pieces or token by
// token performs the same operations in the same order.
#include "common.cuh"

namespace {

__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }

struct DeltaPrepArgs {
    int H, G, dim, ldc, ldab;
    float q_scale;
};

// one CTA a row; a warp a head of q or k
template <typename T>
__global__ void __launch_bounds__(128)
delta_prep_kernel(const T* __restrict__ qk, const T* __restrict__ a_raw, const T* __restrict__ b_raw,
                  VecRef A_log, VecRef dt_bias, float* __restrict__ qn, float* __restrict__ kn,
                  float* __restrict__ g_out, float* __restrict__ beta_out, DeltaPrepArgs a) {
    griddep_launch_small();
    griddep_wait();
    const int row = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const T* src = qk + (size_t)row * a.ldc;
    for (int hh = warp; hh < 2 * a.G; hh += 4) {
        const T* v = src + (size_t)hh * a.dim;                  // q heads, then k heads
        float ss = 0.f;
        for (int d = lane; d < a.dim; d += 32) {
            const float f = to_f32(v[d]);
            ss = fmaf(f, f, ss);
        }
        const float r = (1.0f / sqrtf(warp_sum(ss) + 1e-6f)) * (hh < a.G ? a.q_scale : 1.0f);
        float* dst = hh < a.G ? qn + ((size_t)row * a.G + hh) * a.dim : kn + ((size_t)row * a.G + (hh - a.G)) * a.dim;
        for (int d = lane; d < a.dim; d += 32) dst[d] = to_f32(v[d]) * r;
    }
    for (int h = threadIdx.x; h < a.H; h += blockDim.x) {
        const float av = to_f32(a_raw[(size_t)row * a.ldab + h]);
        const float bv = to_f32(b_raw[(size_t)row * a.ldab + h]);
        g_out[(size_t)row * a.H + h] = expf(-expf(A_log.at(h)) * softplus_f(av + dt_bias.at(h)));
        beta_out[(size_t)row * a.H + h] = 1.0f / (1.0f + expf(-bv));
    }
}

constexpr int DELTA_THREADS = 128;
constexpr int DELTA_R = 32;                 // state values a lane

struct DeltaArgs {
    int B, H, G, dim, vd, n_slots, ldv;
    int L;                                   // lanes a column
};

template <typename T>
__global__ void __launch_bounds__(DELTA_THREADS)
delta_rule_kernel(const float* __restrict__ qn, const float* __restrict__ kn, const T* __restrict__ v,
                  const float* __restrict__ g, const float* __restrict__ beta, float* __restrict__ state,
                  float* __restrict__ o, const int* __restrict__ cu_q, const int* __restrict__ slots, DeltaArgs a) {
    griddep_wait();
    const int b = blockIdx.z, h = blockIdx.y;
    const int slot = slots[b];
    const int q0 = cu_q[b], q1 = cu_q[b + 1];
    if (slot < 0 || slot >= a.n_slots || q1 <= q0) return;
    const int L = a.L;
    const int l = threadIdx.x % L;
    const int j = blockIdx.x * (DELTA_THREADS / L) + threadIdx.x / L;
    const bool on = j < a.vd;
    const int jj = on ? j : a.vd - 1;
    const int kvh = h / (a.H / a.G);

    float S[DELTA_R];
    float* st = state + (((size_t)slot * a.H + h) * a.dim) * a.vd + jj;
#pragma unroll
    for (int r = 0; r < DELTA_R; r++) {
        const int i = l + r * L;
        S[r] = i < a.dim ? st[(size_t)i * a.vd] : 0.f;
    }
    for (int t = q0; t < q1; t++) {
        const float* kt = kn + ((size_t)t * a.G + kvh) * a.dim;
        const float* qt = qn + ((size_t)t * a.G + kvh) * a.dim;
        const float gt = g[(size_t)t * a.H + h], bt = beta[(size_t)t * a.H + h];
        const float vt = to_f32(v[(size_t)t * a.ldv + (size_t)h * a.vd + jj]);
        float kr[DELTA_R];
        float dot = 0.f;
#pragma unroll
        for (int r = 0; r < DELTA_R; r++) {
            const int i = l + r * L;
            kr[r] = i < a.dim ? kt[i] : 0.f;
            S[r] *= gt;
            dot = fmaf(S[r], kr[r], dot);
        }
        for (int s = L >> 1; s > 0; s >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, s);
        const float u = bt * (vt - dot);
        float out = 0.f;
#pragma unroll
        for (int r = 0; r < DELTA_R; r++) {
            const int i = l + r * L;
            S[r] = fmaf(kr[r], u, S[r]);
            out = fmaf(S[r], i < a.dim ? qt[i] : 0.f, out);
        }
        for (int s = L >> 1; s > 0; s >>= 1) out += __shfl_xor_sync(0xffffffffu, out, s);
        if (on && l == 0) o[(size_t)t * a.H * a.vd + (size_t)h * a.vd + j] = out;
    }
    if (on) {
#pragma unroll
        for (int r = 0; r < DELTA_R; r++) {
            const int i = l + r * L;
            if (i < a.dim) st[(size_t)i * a.vd] = S[r];
        }
    }
}

// a warp a (row, head)
template <typename T>
__global__ void __launch_bounds__(128)
gated_rmsnorm_kernel(const float* __restrict__ o, const T* __restrict__ gate, int ldg, VecRef w, T* __restrict__ out,
                     int n_heads_total, int H, int vd, float eps) {
    griddep_launch_small();
    griddep_wait();
    const int idx = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (idx >= n_heads_total) return;
    const int lane = threadIdx.x & 31;
    const int row = idx / H, h = idx % H;
    const float* src = o + ((size_t)row * H + h) * vd;
    float ss = 0.f;
    for (int d = lane; d < vd; d += 32) ss = fmaf(src[d], src[d], ss);
    const float r = 1.0f / sqrtf(warp_sum(ss) / (float)vd + eps);
    const T* gt = gate + (size_t)row * ldg + (size_t)h * vd;
    T* dst = out + ((size_t)row * H + h) * vd;
    for (int d = lane; d < vd; d += 32) {
        const float z = to_f32(gt[d]);
        dst[d] = from_f32<T>(src[d] * r * w.at(d) * (z / (1.0f + expf(-z))));
    }
}

}  // namespace

// qk [T, ldc]: G*dim query then G*dim key values a row (after their convolution and activation); a_raw, b_raw
// [T, ldab] with H values a row; all in dtype. A_log, dt_bias [H] in w_dtype. Outputs fp32: qn, kn [T, G*dim],
// g, beta [T, H].
MYNAH_API int mynah_delta_prep(const void* qk, int ldc, const void* a_raw, const void* b_raw, int ldab, int dtype,
                               const void* A_log, const void* dt_bias, int w_dtype,
                               float* qn, float* kn, float* g, float* beta,
                               int T, int H, int G, int dim, cudaStream_t stream) {
    if (T == 0) return 0;
    MYNAH_REQUIRE(T > 0 && H > 0 && G > 0 && dim > 0 && H % G == 0, "delta_prep: bad sizes T=%d H=%d G=%d dim=%d", T, H, G, dim);
    const DeltaPrepArgs a{H, G, dim, ldc, ldab, 1.0f / sqrtf((float)dim)};
    const VecRef al{A_log, w_dtype}, db{dt_bias, w_dtype};
    if (dtype == MYNAH_F32)
        mynah_launch(delta_prep_kernel<float>, dim3(T), dim3(128), 0, stream, (const float*)qk, (const float*)a_raw,
                     (const float*)b_raw, al, db, qn, kn, g, beta, a);
    else if (dtype == MYNAH_BF16)
        mynah_launch(delta_prep_kernel<bf16>, dim3(T), dim3(128), 0, stream, (const bf16*)qk, (const bf16*)a_raw,
                     (const bf16*)b_raw, al, db, qn, kn, g, beta, a);
    else
        return mynah_fail("delta_prep: unsupported dtype %d", dtype);
    return mynah_check_launch("delta_prep");
}

// v [T, ldv] in dtype with head h at h*vd; state fp32 [n_slots + 1, H, dim, vd]; o fp32 [T, H*vd].
MYNAH_API int mynah_delta_rule(const float* qn, const float* kn, const void* v, int ldv, int dtype,
                               const float* g, const float* beta, float* state, int n_slots, float* o,
                               const int* cu_q, const int* slots, int B, int H, int G, int dim, int vd,
                               cudaStream_t stream) {
    if (B == 0) return 0;
    MYNAH_REQUIRE(B > 0 && H > 0 && G > 0 && dim > 0 && vd > 0 && H % G == 0, "delta_rule: bad sizes B=%d H=%d G=%d dim=%d vd=%d", B, H, G, dim, vd);
    MYNAH_REQUIRE(dim <= 32 * DELTA_R, "delta_rule: a key of %d values exceeds %d", dim, 32 * DELTA_R);
    MYNAH_REQUIRE(B <= 65535 && H <= 65535, "delta_rule: B=%d or H=%d exceeds one launch", B, H);
    int L = 1;
    while (L * DELTA_R < dim) L <<= 1;
    const DeltaArgs a{B, H, G, dim, vd, n_slots, ldv, L};
    const dim3 grid(ceil_div(vd, DELTA_THREADS / L), H, B);
    if (dtype == MYNAH_F32)
        mynah_launch(delta_rule_kernel<float>, grid, dim3(DELTA_THREADS), 0, stream, qn, kn, (const float*)v, g, beta, state, o,
                     cu_q, slots, a);
    else if (dtype == MYNAH_BF16)
        mynah_launch(delta_rule_kernel<bf16>, grid, dim3(DELTA_THREADS), 0, stream, qn, kn, (const bf16*)v, g, beta, state, o,
                     cu_q, slots, a);
    else
        return mynah_fail("delta_rule: unsupported dtype %d", dtype);
    return mynah_check_launch("delta_rule");
}

// out[t, h, :] = o[t, h, :] / rms(o[t, h, :]) * w * silu(gate[t, h, :]); o fp32 [T, H*vd], gate [T, ldg] and out
// [T, H*vd] in dtype, w [vd] in w_dtype.
MYNAH_API int mynah_gated_rmsnorm(const float* o, const void* gate, int ldg, int dtype, const void* w, int w_dtype,
                                  void* out, int T, int H, int vd, float eps, cudaStream_t stream) {
    if (T == 0) return 0;
    MYNAH_REQUIRE(T > 0 && H > 0 && vd > 0, "gated_rmsnorm: bad sizes T=%d H=%d vd=%d", T, H, vd);
    const long long total = (long long)T * H;
    MYNAH_REQUIRE(total <= 0x7fffffffLL, "gated_rmsnorm: too many heads");
    const VecRef wv{w, w_dtype};
    const dim3 grid((unsigned)ceil_div_ll(total, 4));
    if (dtype == MYNAH_F32)
        mynah_launch(gated_rmsnorm_kernel<float>, grid, dim3(128), 0, stream, o, (const float*)gate, ldg, wv, (float*)out,
                     (int)total, H, vd, eps);
    else if (dtype == MYNAH_BF16)
        mynah_launch(gated_rmsnorm_kernel<bf16>, grid, dim3(128), 0, stream, o, (const bf16*)gate, ldg, wv, (bf16*)out,
                     (int)total, H, vd, eps);
    else
        return mynah_fail("gated_rmsnorm: unsupported dtype %d", dtype);
    return mynah_check_launch("gated_rmsnorm");
}
