// Retention: linear attention with a fixed decay per head, no softmax and no denominator. Per head, with
// S [dim x vd] the state (fp32, carried per slot):
//
//   S_t = decay_h S_(t-1) + k_t v_t^T,      o_t = S_t^T q_t
//
// Kernels (the per-head unit RMS and the gate that follow are `gated_rmsnorm`):
//
//   retention_prep   q, k rows -> fp32, the first `rot` dims of every head rotated by the position's table row
//                    (pairs (i, i + rot/2), or (2i, 2i+1)), k then multiplied by k_scale
//   retention_scan   the recurrence. The columns of S are independent, so a CTA takes a tile of columns of one
//                    head of one sequence; a column's dim values lie in the registers of L adjacent lanes (up to
//                    32 values a lane), which add their parts of o by shuffles in a fixed order. Keys, queries and
//                    values of 32 tokens at a time pass through shared memory.
//   retention_chunk  the same recurrence for prompts, a chunk of tokens at a time (see below)
//
// All arithmetic is fp32. A sequence's rows are walked in order, so a prompt run whole, in pieces or token by
// token performs the same operations in the same order.
#include "layout.cuh"

namespace {

struct RetPrepArgs {
    int H, dim, ld, q_off, k_off;    // heads, head size, row stride, first columns of q and k
    int rot, interleaved, n_pos;
    float k_scale;
};

// one CTA a token
template <typename T>
__global__ void __launch_bounds__(128)
retention_prep_kernel(const T* __restrict__ qk, float* __restrict__ qn, float* __restrict__ kn,
                      const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                      const int* __restrict__ tok_seq, const int* __restrict__ tok_pos, RetPrepArgs a,
                      int* __restrict__ status) {
    griddep_launch_small();
    griddep_wait();
    const int t = blockIdx.x;
    if (tok_seq[t] < 0) return;
    const int pos = tok_pos[t];
    const bool rotate = a.rot > 0 && cos_t != nullptr;
    if (rotate && (pos < 0 || pos >= a.n_pos)) {
        if (threadIdx.x == 0) atomicOr(status, MYNAH_ST_POS_RANGE);
        return;
    }
    const int half = a.rot >> 1;
    const float* cr = rotate ? cos_t + (size_t)pos * half : nullptr;
    const float* sr = rotate ? sin_t + (size_t)pos * half : nullptr;
    const int n = a.H * a.dim;
    const T* row = qk + (size_t)t * a.ld;
    for (int idx = threadIdx.x; idx < 2 * n; idx += blockDim.x) {
        const bool is_k = idx >= n;
        const int e = is_k ? idx - n : idx;
        const int h = e / a.dim, d = e % a.dim;
        const T* src = row + (is_k ? a.k_off : a.q_off) + (size_t)h * a.dim;
        float v = to_f32(src[d]);
        if (rotate && d < a.rot) {
            int i, other;
            float sign;
            if (a.interleaved) {
                i = d >> 1; other = d ^ 1; sign = (d & 1) ? 1.f : -1.f;
            } else {
                i = d < half ? d : d - half; other = d < half ? d + half : d - half; sign = d < half ? -1.f : 1.f;
            }
            v = v * cr[i] + sign * to_f32(src[other]) * sr[i];
        }
        if (is_k) kn[(size_t)t * n + e] = v * a.k_scale;
        else qn[(size_t)t * n + e] = v;
    }
}

constexpr int RET_THREADS = 128;
constexpr int RET_TB = 32;                 // tokens staged in shared memory at a time
constexpr int RET_RMAX = 32;               // state values a lane keeps

struct RetArgs {
    int B, H, dim, vd, n_slots, ldv, v_off;
    int L, per;                            // lanes a column (a power of two <= 32), values a lane (<= RET_RMAX)
};

template <typename T>
__global__ void __launch_bounds__(RET_THREADS)
retention_scan_kernel(const float* __restrict__ qn, const float* __restrict__ kn, const T* __restrict__ v,
                      const float* __restrict__ decay, float* __restrict__ state, float* __restrict__ o,
                      const int* __restrict__ cu_q, const int* __restrict__ slots, RetArgs a) {
    extern __shared__ float sm[];
    griddep_wait();
    const int b = blockIdx.z, h = blockIdx.y;
    const int slot = slots[b];
    const int q0 = cu_q[b], q1 = cu_q[b + 1];
    if (slot < 0 || slot >= a.n_slots || q1 <= q0) return;
    const int L = a.L, per = a.per;
    const int JT = RET_THREADS / L;
    const int l = threadIdx.x % L, jl = threadIdx.x / L;
    const int j = blockIdx.x * JT + jl;
    const bool on = j < a.vd;
    const int CS = per + 1;                                      // floats of a lane's chunk (padded against bank conflicts)
    const int rowf = CS * L;
    float* ks = sm;                                              // [TB][rowf]
    float* qs = ks + RET_TB * rowf;                              // [TB][rowf]
    float* vs = qs + RET_TB * rowf;                              // [TB][JT]
    for (int i = threadIdx.x; i < 2 * RET_TB * rowf; i += RET_THREADS) ks[i] = 0.f;    // slots beyond dim stay zero
    const float g = decay[h];
    float S[RET_RMAX];
    float* sp = state + (((size_t)slot * a.H + h) * a.dim) * a.vd;
#pragma unroll
    for (int r = 0; r < RET_RMAX; r++) {
        const int i = l * per + r;
        S[r] = (on && r < per && i < a.dim) ? sp[(size_t)i * a.vd + j] : 0.f;
    }
    const int n = a.H * a.dim;
    for (int t0 = q0; t0 < q1; t0 += RET_TB) {
        const int nt = min(RET_TB, q1 - t0);
        __syncthreads();
        for (int idx = threadIdx.x; idx < nt * a.dim; idx += RET_THREADS) {
            const int tt = idx / a.dim, i = idx % a.dim;
            const size_t src = (size_t)(t0 + tt) * n + (size_t)h * a.dim + i;
            const int dst = tt * rowf + (i / per) * CS + i % per;
            ks[dst] = kn[src];
            qs[dst] = qn[src];
        }
        for (int idx = threadIdx.x; idx < nt * JT; idx += RET_THREADS) {
            const int tt = idx / JT, c = idx % JT;
            const int col = blockIdx.x * JT + c;
            vs[idx] = col < a.vd ? to_f32(v[(size_t)(t0 + tt) * a.ldv + a.v_off + (size_t)h * a.vd + col]) : 0.f;
        }
        __syncthreads();
        for (int tt = 0; tt < nt; tt++) {
            const float* kk = ks + tt * rowf + l * CS;
            const float* qq = qs + tt * rowf + l * CS;
            const float vj = vs[tt * JT + jl];
            float acc = 0.f;
#pragma unroll
            for (int r = 0; r < RET_RMAX; r++) {
                if (r < per) {
                    S[r] = fmaf(kk[r], vj, g * S[r]);
                    acc = fmaf(S[r], qq[r], acc);
                }
            }
            for (int m = 1; m < L; m <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, m);
            if (on && l == 0) o[(size_t)(t0 + tt) * a.H * a.vd + (size_t)h * a.vd + j] = acc;
        }
    }
    if (on) {
#pragma unroll
        for (int r = 0; r < RET_RMAX; r++) {
            const int i = l * per + r;
            if (r < per && i < a.dim) sp[(size_t)i * a.vd + j] = S[r];
        }
    }
}

// ---- the recurrence chunk by chunk, for prompts ----
// With a chunk of C tokens, S the state before it and g the head's decay:
//
//   o_t   = sum_{s <= t} g^(t-s) (q_t . k_s) v_s  +  g^(t+1) S^T q_t                      t, s inside the chunk
//   S_new = g^n S + sum_s g^(n-1-s) k_s v_s^T                                            n tokens in the chunk
//
// so the 2n dependent steps of a chunk become blocks of independent multiply-adds. Two kernels:
//
//   retention_scores  the decayed scores g^(t-s) (q_t . k_s) of every chunk of every sequence, side by side (they do
//                     not depend on the state): a CTA a chunk and head, register-tiled fp32, written to scratch
//                     [H][rows][C]
//   retention_chunk   the chain: a CTA takes JW columns (32, or 16 when the step has too few CTAs for the machine) of one
//                     head of one sequence and walks the sequence's chunks in order: scores times values, the read of
//                     the old state, the state's update. q and k of the chunk, the scores, the values and the state's
//                     columns lie in shared memory.
//
// The powers of g come from a table made by repeated multiplication. Sums run in another order than token by token:
// the two forms agree to rounding.
constexpr int RC_THREADS = 256;

struct RetChunkArgs {
    int H, dim, vd, n_slots, ldv, v_off, rows, B;
};

// grid (rows / C + B, H): the step's chunks are numbered sequence by sequence (layout.cuh: find_query_tile)
template <int C>
__global__ void __launch_bounds__(RC_THREADS)
retention_scores_kernel(const float* __restrict__ qn, const float* __restrict__ kn, const float* __restrict__ decay,
                        float* __restrict__ w_out, const int* __restrict__ cu_q, RetChunkArgs a) {
    constexpr int TT = C / 16;
    extern __shared__ __align__(16) float sm[];
    __shared__ float gp[C];
    griddep_wait();
    int b, tile;
    if (!find_query_tile(cu_q, a.B, C, (int)blockIdx.x, b, tile)) return;
    const int h = blockIdx.y, d = a.dim, ldr = d + 4;
    float* qs = sm;
    float* ks = qs + C * ldr;
    const int tid = threadIdx.x;
    const int t0 = cu_q[b] + tile * C, nt = min(C, cu_q[b + 1] - t0);
    if (tid == 0) {
        float p = 1.f;
        const float g = decay[h];
        for (int n = 0; n < C; n++) {
            gp[n] = p;
            p *= g;
        }
    }
    const size_t n = (size_t)a.H * d;
    for (int idx = tid; idx < C * (d / 4); idx += RC_THREADS) {
        const int tt = idx / (d / 4), i4 = (idx % (d / 4)) * 4;
        float4 qv = make_float4(0.f, 0.f, 0.f, 0.f), kv = qv;
        if (tt < nt) {
            const size_t src = (size_t)(t0 + tt) * n + (size_t)h * d + i4;
            qv = *reinterpret_cast<const float4*>(qn + src);
            kv = *reinterpret_cast<const float4*>(kn + src);
        }
        *reinterpret_cast<float4*>(qs + tt * ldr + i4) = qv;
        *reinterpret_cast<float4*>(ks + tt * ldr + i4) = kv;
    }
    __syncthreads();
    // thread (ta, sb) takes tokens ta + 16 u and keys sb + 16 w
    const int ta = tid >> 4, sb = tid & 15;
    float acc[TT][TT];
#pragma unroll
    for (int u = 0; u < TT; u++)
#pragma unroll
        for (int w = 0; w < TT; w++) acc[u][w] = 0.f;
#pragma unroll 2
    for (int i = 0; i < d; i += 4) {
        float4 qv[TT], kv[TT];
#pragma unroll
        for (int u = 0; u < TT; u++) qv[u] = *reinterpret_cast<const float4*>(qs + (ta + 16 * u) * ldr + i);
#pragma unroll
        for (int w = 0; w < TT; w++) kv[w] = *reinterpret_cast<const float4*>(ks + (sb + 16 * w) * ldr + i);
#pragma unroll
        for (int u = 0; u < TT; u++)
#pragma unroll
            for (int w = 0; w < TT; w++) {
                acc[u][w] = fmaf(qv[u].x, kv[w].x, acc[u][w]);
                acc[u][w] = fmaf(qv[u].y, kv[w].y, acc[u][w]);
                acc[u][w] = fmaf(qv[u].z, kv[w].z, acc[u][w]);
                acc[u][w] = fmaf(qv[u].w, kv[w].w, acc[u][w]);
            }
    }
    float* wo = w_out + ((size_t)h * a.rows + t0) * C;
#pragma unroll
    for (int u = 0; u < TT; u++)
#pragma unroll
        for (int w = 0; w < TT; w++) {
            const int t = ta + 16 * u, s = sb + 16 * w;
            if (t < nt) wo[(size_t)t * C + s] = s <= t ? gp[t - s] * acc[u][w] : 0.f;
        }
}

template <typename T, int C, int JW>
__global__ void __launch_bounds__(RC_THREADS)
retention_chunk_kernel(const float* __restrict__ qn, const float* __restrict__ kn, const T* __restrict__ v,
                       const float* __restrict__ decay, const float* __restrict__ w_in, float* __restrict__ state,
                       float* __restrict__ o, const int* __restrict__ cu_q, const int* __restrict__ slots, RetChunkArgs a) {
    constexpr int HS = 32 / JW;            // groups of lanes that share the CTA's columns (1 or 2)
    constexpr int TPW = C / 8 / HS;        // tokens a group of lanes takes in the products with the values and the state
    constexpr int LDW = C + 4;             // row stride of the decayed scores (rows stay 16-byte aligned)
    extern __shared__ __align__(16) float sm[];
    griddep_wait();
    const int b = blockIdx.z, h = blockIdx.y;
    const int slot = slots[b];
    const int q0 = cu_q[b], q1 = cu_q[b + 1];
    if (slot < 0 || slot >= a.n_slots || q1 <= q0) return;
    const int d = a.dim, ldr = d + 4;      // row stride of q and k in shared memory (16 bytes of padding)
    const int rpw = d / 8 / HS;            // state rows a group of lanes owns (a multiple of 4)
    float* qs = sm;                        // [C][ldr]
    float* ks = qs + C * ldr;              // [C][ldr]
    float* Ss = ks + C * ldr;              // [d][JW]
    float* Ws = Ss + d * JW;               // [C][LDW]
    float* vs = Ws + C * LDW;              // [C][JW]
    float* gp = vs + C * JW;               // [C + 1]: powers of the decay
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int grp = lane / JW, col = lane % JW;
    const int j = blockIdx.x * JW + col;
    const bool on = j < a.vd;
    const float g = decay[h];
    if (tid == 0) {
        float p = 1.f;
        for (int n = 0; n <= C; n++) {
            gp[n] = p;
            p *= g;
        }
    }
    float* sp = state + (((size_t)slot * a.H + h) * d) * a.vd;
    for (int idx = tid; idx < d * JW; idx += RC_THREADS) {
        const int i = idx / JW, c = blockIdx.x * JW + idx % JW;
        Ss[idx] = c < a.vd ? sp[(size_t)i * a.vd + c] : 0.f;
    }
    const size_t n = (size_t)a.H * d;
    // A chunk's q, k, scores and values travel through registers: the loads of chunk c + 1 are issued before chunk c
    // is computed, all at once, so that the chain waits on no load. (C * d <= 8192: at most 8 + 8 + 4 vectors a thread.)
    constexpr int QK_IT = 8, W_IT = C * (C / 4) / RC_THREADS > 0 ? C * (C / 4) / RC_THREADS : 1, V_IT = C * JW / RC_THREADS;
    float4 rq[QK_IT], rk[QK_IT], rw[W_IT];
    float rv[V_IT];
    const int qk_total = C * (d / 4);
    auto load_chunk = [&](int t0) {
        const int nt = min(C, q1 - t0);
        const float* wi = w_in + ((size_t)h * a.rows + t0) * C;
#pragma unroll
        for (int it = 0; it < QK_IT; it++) {
            const int idx = tid + it * RC_THREADS;
            const int tt = idx / (d / 4), i4 = (idx % (d / 4)) * 4;
            rq[it] = rk[it] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (idx < qk_total && tt < nt) {
                const size_t src = (size_t)(t0 + tt) * n + (size_t)h * d + i4;
                rq[it] = *reinterpret_cast<const float4*>(qn + src);
                rk[it] = *reinterpret_cast<const float4*>(kn + src);
            }
        }
#pragma unroll
        for (int it = 0; it < W_IT; it++) {
            const int idx = tid + it * RC_THREADS;
            const int tt = idx / (C / 4), s4 = (idx % (C / 4)) * 4;
            rw[it] = (idx < C * (C / 4) && tt < nt) ? *reinterpret_cast<const float4*>(wi + (size_t)tt * C + s4)
                                                     : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int it = 0; it < V_IT; it++) {
            const int idx = tid + it * RC_THREADS;
            const int tt = idx / JW, c = blockIdx.x * JW + idx % JW;
            rv[it] = (tt < nt && c < a.vd) ? to_f32(v[(size_t)(t0 + tt) * a.ldv + a.v_off + (size_t)h * a.vd + c]) : 0.f;
        }
    };
    auto store_chunk = [&]() {
#pragma unroll
        for (int it = 0; it < QK_IT; it++) {
            const int idx = tid + it * RC_THREADS;
            if (idx < qk_total) {
                const int tt = idx / (d / 4), i4 = (idx % (d / 4)) * 4;
                *reinterpret_cast<float4*>(qs + tt * ldr + i4) = rq[it];
                *reinterpret_cast<float4*>(ks + tt * ldr + i4) = rk[it];
            }
        }
#pragma unroll
        for (int it = 0; it < W_IT; it++) {
            const int idx = tid + it * RC_THREADS;
            if (idx < C * (C / 4)) *reinterpret_cast<float4*>(Ws + (idx / (C / 4)) * LDW + (idx % (C / 4)) * 4) = rw[it];
        }
#pragma unroll
        for (int it = 0; it < V_IT; it++) vs[tid + it * RC_THREADS] = rv[it];
    };
    load_chunk(q0);
    for (int t0 = q0; t0 < q1; t0 += C) {
        const int nt = min(C, q1 - t0);
        __syncthreads();                                         // the chunk before is done with q, k, v, the scores
        store_chunk();
        __syncthreads();
        if (t0 + C < q1) load_chunk(t0 + C);                     // in flight while this chunk is computed
        {   // o: lane group `grp` of warp `warp` takes tokens tb + u, its lanes the columns
            float intra[TPW], inter[TPW];
#pragma unroll
            for (int u = 0; u < TPW; u++) intra[u] = inter[u] = 0.f;
            const int tb = (warp * HS + grp) * TPW;
            const int s_end = min((tb + TPW + 3) & ~3, C);       // keys beyond the group's last token weigh nothing
            for (int s = 0; s < s_end; s += 4) {                 // (rows beyond nt hold zeros)
                const float v0 = vs[s * JW + col], v1 = vs[(s + 1) * JW + col];
                const float v2 = vs[(s + 2) * JW + col], v3 = vs[(s + 3) * JW + col];
#pragma unroll
                for (int u = 0; u < TPW; u++) {
                    const float4 w4 = *reinterpret_cast<const float4*>(Ws + (tb + u) * LDW + s);
                    intra[u] = fmaf(w4.x, v0, intra[u]);
                    intra[u] = fmaf(w4.y, v1, intra[u]);
                    intra[u] = fmaf(w4.z, v2, intra[u]);
                    intra[u] = fmaf(w4.w, v3, intra[u]);
                }
            }
#pragma unroll 2
            for (int i = 0; i < d; i += 4) {
                const float s0 = Ss[i * JW + col], s1 = Ss[(i + 1) * JW + col];
                const float s2 = Ss[(i + 2) * JW + col], s3 = Ss[(i + 3) * JW + col];
#pragma unroll
                for (int u = 0; u < TPW; u++) {
                    const float4 qv = *reinterpret_cast<const float4*>(qs + (tb + u) * ldr + i);
                    inter[u] = fmaf(qv.x, s0, inter[u]);
                    inter[u] = fmaf(qv.y, s1, inter[u]);
                    inter[u] = fmaf(qv.z, s2, inter[u]);
                    inter[u] = fmaf(qv.w, s3, inter[u]);
                }
            }
            if (on) {
#pragma unroll
                for (int u = 0; u < TPW; u++) {
                    const int t = tb + u;
                    if (t < nt) o[(size_t)(t0 + t) * a.H * a.vd + (size_t)h * a.vd + j] = fmaf(gp[t + 1], inter[u], intra[u]);
                }
            }
        }
        __syncthreads();                                         // every warp has read the old state
        {   // the state's rows (warp * HS + grp) * rpw + r, column `col`
            const float gn = gp[nt];
            float loc[32];                                       // rpw <= 32 rows (d <= 256)
#pragma unroll
            for (int r = 0; r < 32; r++) loc[r] = 0.f;
            const int row0 = (warp * HS + grp) * rpw;
            const float* kw = ks + row0;
#pragma unroll 2
            for (int s = 0; s < nt; s++) {
                const float vw = gp[nt - 1 - s] * vs[s * JW + col];
#pragma unroll
                for (int r4 = 0; r4 < 8; r4++) {
                    if (r4 * 4 < rpw) {
                        const float4 kv = *reinterpret_cast<const float4*>(kw + s * ldr + r4 * 4);
                        loc[r4 * 4] = fmaf(kv.x, vw, loc[r4 * 4]);
                        loc[r4 * 4 + 1] = fmaf(kv.y, vw, loc[r4 * 4 + 1]);
                        loc[r4 * 4 + 2] = fmaf(kv.z, vw, loc[r4 * 4 + 2]);
                        loc[r4 * 4 + 3] = fmaf(kv.w, vw, loc[r4 * 4 + 3]);
                    }
                }
            }
#pragma unroll
            for (int r = 0; r < 32; r++)
                if (r < rpw) {
                    float* sl = Ss + (row0 + r) * JW + col;
                    *sl = fmaf(gn, *sl, loc[r]);
                }
        }
    }
    __syncthreads();
    for (int idx = tid; idx < d * JW; idx += RC_THREADS) {
        const int i = idx / JW, c = blockIdx.x * JW + idx % JW;
        if (c < a.vd) sp[(size_t)i * a.vd + c] = Ss[idx];
    }
}

template <typename T, int C, int JW>
int launch_chain(const float* qn, const float* kn, const void* v, const float* decay, const float* w, float* state, float* o,
                 const int* cu_q, const int* slots, const RetChunkArgs& a, cudaStream_t stream) {
    const int d = a.dim;
    const size_t smem = ((size_t)2 * C * (d + 4) + (size_t)d * JW + (size_t)C * (C + 4) + (size_t)C * JW + C + 1 + 3) * sizeof(float);
    if (cudaFuncSetAttribute(retention_chunk_kernel<T, C, JW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return mynah_fail("retention_scan: %zu bytes of shared memory are not to be had", smem);
    mynah_launch(retention_chunk_kernel<T, C, JW>, dim3(ceil_div(a.vd, JW), a.H, a.B), dim3(RC_THREADS), smem, stream,
                 qn, kn, (const T*)v, decay, w, state, o, cu_q, slots, a);
    return mynah_check_launch("retention_scan (chunked)");
}

template <typename T, int C>
int launch_chunked(const float* qn, const float* kn, const void* v, const float* decay, float* w, float* state, float* o,
                   const int* cu_q, const int* slots, const RetChunkArgs& a, cudaStream_t stream) {
    const size_t smem = (size_t)2 * C * (a.dim + 4) * sizeof(float);
    if (cudaFuncSetAttribute(retention_scores_kernel<C>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return mynah_fail("retention_scan: %zu bytes of shared memory are not to be had", smem);
    MYNAH_REQUIRE(a.rows / C + a.B <= 65535 * 32, "retention_scan: too many chunks for one launch");
    mynah_launch(retention_scores_kernel<C>, dim3(a.rows / C + a.B, a.H), dim3(RC_THREADS), smem, stream, qn, kn, decay, w, cu_q, a);
    if (mynah_check_launch("retention_scan (scores)") != 0) return -1;
    // 16 columns a CTA when 32 would leave most of the machine idle (and the state's rows divide)
    const bool narrow = a.dim % 64 == 0 && (long long)a.B * a.H * ceil_div(a.vd, 32) < mynah_sm_count();
    return narrow ? launch_chain<T, C, 16>(qn, kn, v, decay, w, state, o, cu_q, slots, a, stream)
                  : launch_chain<T, C, 32>(qn, kn, v, decay, w, state, o, cu_q, slots, a, stream);
}

}  // namespace

// 0: every step walks token by token; otherwise prompts whose longest piece has at least this many tokens go chunk by chunk.
static int g_ret_chunk_min = 16;
MYNAH_API int mynah_retention_chunk_min(int n) {
    const int before = g_ret_chunk_min;
    g_ret_chunk_min = n;
    return before;
}

static bool retention_chunked(int dim, int max_q_len) {
    return g_ret_chunk_min > 0 && max_q_len >= g_ret_chunk_min && dim % 32 == 0 && dim <= 256;
}

// Floats of scratch that mynah_retention_scan wants for a step of `rows` rows (0: it walks token by token).
MYNAH_API long long mynah_retention_scratch_floats(int rows, int H, int dim, int max_q_len) {
    return retention_chunked(dim, max_q_len) ? (long long)rows * H * (dim <= 128 ? 64 : 32) : 0;
}


// qk: rows that hold every head's q from column q_off and every head's k from column k_off; qn, kn: fp32 [T][H*dim].
MYNAH_API int mynah_retention_prep(const void* qk, int ld, int q_off, int k_off, int dtype, float* qn, float* kn,
                                   int T, int H, int dim, const float* cos_t, const float* sin_t, int rot,
                                   int interleaved, int n_pos, float k_scale, const int* tok_seq, const int* tok_pos,
                                   int* status, cudaStream_t stream) {
    if (T == 0) return 0;
    MYNAH_REQUIRE(T > 0 && H > 0 && dim > 0, "retention_prep: bad sizes");
    MYNAH_REQUIRE(rot % 2 == 0 && rot <= dim, "retention_prep: %d rotated dims do not fit a head of %d", rot, dim);
    const RetPrepArgs a{H, dim, ld, q_off, k_off, cos_t ? rot : 0, interleaved, n_pos, k_scale};
    if (dtype == MYNAH_F32)
        mynah_launch(retention_prep_kernel<float>, dim3(T), dim3(128), 0, stream, (const float*)qk, qn, kn, cos_t, sin_t,
                     tok_seq, tok_pos, a, status);
    else if (dtype == MYNAH_BF16)
        mynah_launch(retention_prep_kernel<bf16>, dim3(T), dim3(128), 0, stream, (const bf16*)qk, qn, kn, cos_t, sin_t,
                     tok_seq, tok_pos, a, status);
    else
        return mynah_fail("retention_prep: unsupported dtype %d", dtype);
    return mynah_check_launch("retention_prep");
}

// v: rows whose columns [v_off + h * vd, ...) are head h's values; decay: fp32 [H]; state: fp32 [n_slots + 1][H][dim][vd];
// o: fp32 [T][H * vd]. max_q_len: the most tokens a sequence brings (chooses between the two forms of the recurrence);
// rows: the step's rows; scratch: mynah_retention_scratch_floats(...) floats, or null (token by token).
MYNAH_API int mynah_retention_scan(const float* qn, const float* kn, const void* v, int ldv, int v_off, int v_dtype,
                                   const float* decay, float* state, int n_slots, float* o, const int* cu_q,
                                   const int* slots, int B, int H, int dim, int vd, int max_q_len, int rows, float* scratch,
                                   cudaStream_t stream) {
    if (B == 0) return 0;
    MYNAH_REQUIRE(B > 0 && H > 0 && dim > 0 && vd > 0, "retention_scan: bad sizes");
    MYNAH_REQUIRE(dim <= 512, "retention_scan: keys of %d values exceed the 512 that the kernel stages", dim);
    MYNAH_REQUIRE(H <= 65535 && B <= 65535, "retention_scan: too many heads or sequences for one launch");
    MYNAH_REQUIRE(v_dtype == MYNAH_F32 || v_dtype == MYNAH_BF16, "retention_scan: unsupported dtype %d", v_dtype);
    if (retention_chunked(dim, max_q_len) && scratch != nullptr && (((uintptr_t)qn | (uintptr_t)kn | (uintptr_t)scratch) & 15) == 0) {
        const RetChunkArgs ca{H, dim, vd, n_slots, ldv, v_off, rows, B};
        if (v_dtype == MYNAH_F32)
            return dim <= 128 ? launch_chunked<float, 64>(qn, kn, v, decay, scratch, state, o, cu_q, slots, ca, stream)
                              : launch_chunked<float, 32>(qn, kn, v, decay, scratch, state, o, cu_q, slots, ca, stream);
        return dim <= 128 ? launch_chunked<bf16, 64>(qn, kn, v, decay, scratch, state, o, cu_q, slots, ca, stream)
                          : launch_chunked<bf16, 32>(qn, kn, v, decay, scratch, state, o, cu_q, slots, ca, stream);
    }
    int L = 1;
    while (L * RET_RMAX < dim) L <<= 1;
    const int per = ceil_div(dim, L);
    const int JT = RET_THREADS / L;
    const RetArgs a{B, H, dim, vd, n_slots, ldv, v_off, L, per};
    const size_t smem = ((size_t)2 * RET_TB * (per + 1) * L + (size_t)RET_TB * JT) * sizeof(float);
    const dim3 grid(ceil_div(vd, JT), H, B);
    if (v_dtype == MYNAH_F32) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(retention_scan_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        mynah_launch(retention_scan_kernel<float>, grid, dim3(RET_THREADS), smem, stream, qn, kn, (const float*)v, decay, state, o, cu_q, slots, a);
    } else if (v_dtype == MYNAH_BF16) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(retention_scan_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        mynah_launch(retention_scan_kernel<bf16>, grid, dim3(RET_THREADS), smem, stream, qn, kn, (const bf16*)v, decay, state, o, cu_q, slots, a);
    } else
        return mynah_fail("retention_scan: unsupported dtype %d", v_dtype);
    return mynah_check_launch("retention_scan");
}
