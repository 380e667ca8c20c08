// What lies between the q/k/v projection and the attention for mixers that norm the WHOLE projection:
//
//   q <- q / rms(q over all heads) * wq          (one RMS over the H*dim outputs, gain of that size; k likewise)
//   rotary positions on the first `rot` dimensions of each head of q and k, element i paired with i + rot/2:
//       (u, v) -> (u cos a - v sin a, v cos a + u sin a),   a = position * base^(-2i/rot)   (tables built in double)
//   v <- v / rms(v over the head's vd values)     (no gain)
//   v <- (1 - lambda) v + lambda v_first          (optional: v_first holds the same token's values of an earlier
//                                                  layer, written here by the layer that comes first)
//   q -> q_out, k and v -> the paged cache
//
// Everything is computed in fp32 from the projection's rows. Heads may be narrower than their storage: q_out and
// the cache hold dimp >= dim and vdp >= vd elements a head (multiples of 8), the rest written as zeros, which
// changes neither a score nor a used output column.
#include "layout.cuh"

namespace {

struct PrepArgs {
    int H, G, dim, vd, dimp, vdp, ld, ldq, rot, n_pos;
    float eps;
    int vmix;        // 0: none, 1: write v_first, 2: mix with v_first
    int vec;         // 1: the q and k heads go eight elements a thread (see norm_rotate_heads8)
};

constexpr int PREP_THREADS = 256;

// Norms and rotates one projection (n_heads heads of `dim`) of a row into dst, whose heads are `dimp` wide: the
// rotated pairs (i, i + rot/2) first, a thread a pair, so that each input, gain and table entry is read once; then
// the dimensions behind the rotated ones, and the zero padding.
template <typename T, typename TD>
__device__ __forceinline__ void norm_rotate_heads(const T* __restrict__ src, const VecRef& gain, float r, int n_heads,
                                                  int dim, int dimp, int rot, const float* __restrict__ cosr,
                                                  const float* __restrict__ sinr, TD* __restrict__ dst, size_t head_stride) {
    const int half = rot >> 1;
    for (int idx = threadIdx.x; idx < n_heads * half; idx += PREP_THREADS) {
        const int h = idx / half, i = idx % half;
        const int at = h * dim + i;
        const float u = to_f32(src[at]) * r * gain.at(at);
        const float v = to_f32(src[at + half]) * r * gain.at(at + half);
        const float c = cosr[i], sn = sinr[i];
        dst[h * head_stride + i] = from_f32<TD>(u * c - v * sn);
        dst[h * head_stride + i + half] = from_f32<TD>(v * c + u * sn);
    }
    const int rest = dimp - rot;
    for (int idx = threadIdx.x; idx < n_heads * rest; idx += PREP_THREADS) {
        const int h = idx / rest, d = rot + idx % rest;
        dst[h * head_stride + d] = from_f32<TD>(d < dim ? to_f32(src[h * dim + d]) * r * gain.at(h * dim + d) : 0.f);
    }
}

__device__ __forceinline__ void gain8(const VecRef& w, int i, float (&g)[8]) {
    if (w.dtype == MYNAH_F32) load8(static_cast<const float*>(w.p) + i, g);
    else load8(static_cast<const bf16*>(w.p) + i, g);
}

// The same for heads whose width, rotated part and storage fit 16-byte vectors (dim % 8 == 0, rot % 16 == 0, dimp ==
// dim, aligned rows): eight pairs, or eight unrotated dimensions, a thread; the same arithmetic per element.
template <typename T, typename TD>
__device__ __forceinline__ void norm_rotate_heads8(const T* __restrict__ src, const VecRef& gain, float r, int n_heads,
                                                   int dim, int rot, const float* __restrict__ cosr,
                                                   const float* __restrict__ sinr, TD* __restrict__ dst, size_t head_stride) {
    const int half = rot >> 1, h8 = half >> 3;
    for (int idx = threadIdx.x; idx < n_heads * h8; idx += PREP_THREADS) {
        const int h = idx / h8, i = (idx % h8) * 8;
        const int at = h * dim + i;
        float u[8], v[8], gu[8], gv[8], c[8], sn[8], o1[8], o2[8];
        load8(src + at, u);
        load8(src + at + half, v);
        gain8(gain, at, gu);
        gain8(gain, at + half, gv);
        load8(cosr + i, c);
        load8(sinr + i, sn);
#pragma unroll
        for (int e = 0; e < 8; e++) {
            const float uu = u[e] * r * gu[e], vv = v[e] * r * gv[e];
            o1[e] = uu * c[e] - vv * sn[e];
            o2[e] = vv * c[e] + uu * sn[e];
        }
        store8(dst + h * head_stride + i, o1);
        store8(dst + h * head_stride + i + half, o2);
    }
    const int rest8 = (dim - rot) >> 3;
    for (int idx = threadIdx.x; idx < n_heads * rest8; idx += PREP_THREADS) {
        const int h = idx / rest8, d = rot + (idx % rest8) * 8;
        float u[8], g[8];
        load8(src + h * dim + d, u);
        gain8(gain, h * dim + d, g);
#pragma unroll
        for (int e = 0; e < 8; e++) u[e] = u[e] * r * g[e];
        store8(dst + h * head_stride + d, u);
    }
}

template <typename T>
__device__ __forceinline__ float sum_squares(const T* __restrict__ src, int n, bool vec) {
    float s = 0.f;
    if (vec) {
        for (int i = threadIdx.x * 8; i < n; i += PREP_THREADS * 8) {
            float v[8];
            load8(src + i, v);
#pragma unroll
            for (int e = 0; e < 8; e++) s = fmaf(v[e], v[e], s);
        }
    } else {
        for (int i = threadIdx.x; i < n; i += PREP_THREADS) {
            const float v = to_f32(src[i]);
            s = fmaf(v, v, s);
        }
    }
    return s;
}

template <typename T>
__global__ void __launch_bounds__(PREP_THREADS)
attn_prep_kernel(const T* __restrict__ qkv, T* __restrict__ q_out, VecRef qw, VecRef kw,
                 const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                 const int* __restrict__ tok_seq, const int* __restrict__ tok_pos, PageTable pt,
                 T* __restrict__ k_cache, T* __restrict__ v_cache, float* __restrict__ v_first,
                 const float* __restrict__ lambda_p, PrepArgs a, int* __restrict__ status) {
    __shared__ float red[32];
    griddep_launch_small();
    griddep_wait();
    const int row = blockIdx.x;
    const int b = tok_seq[row];
    T* qo = q_out + (size_t)row * a.ldq;
    const int nq = a.H * a.dim, nk = a.G * a.dim;
    if (b < 0) {                                   // a padding row: defined zeros, nothing cached
        for (int i = threadIdx.x; i < a.H * a.dimp; i += PREP_THREADS) qo[i] = from_f32<T>(0.f);
        return;
    }
    const T* src = qkv + (size_t)row * a.ld;
    const int pos = tok_pos[row];
    if (a.rot > 0 && (pos < 0 || pos >= a.n_pos)) {
        if (threadIdx.x == 0) atomicOr(status, MYNAH_ST_POS_RANGE);
        return;
    }
    const float* cosr = a.rot > 0 ? cos_t + (size_t)pos * (a.rot >> 1) : nullptr;
    const float* sinr = a.rot > 0 ? sin_t + (size_t)pos * (a.rot >> 1) : nullptr;

    const float rq = 1.0f / sqrtf(block_sum(sum_squares(src, nq, a.vec), red) / (float)nq + a.eps);
    if (a.vec) norm_rotate_heads8(src, qw, rq, a.H, a.dim, a.rot, cosr, sinr, qo, (size_t)a.dimp);
    else norm_rotate_heads(src, qw, rq, a.H, a.dim, a.dimp, a.rot, cosr, sinr, qo, (size_t)a.dimp);
    if (k_cache == nullptr) return;                // this run reads a cache that another run wrote

    const int page = page_of(pt, b, pos);
    if (page < 0) {
        if (threadIdx.x == 0) atomicOr(status, MYNAH_ST_PAGE_RANGE);
        return;
    }
    const T* ksrc = src + nq;
    const float rk = 1.0f / sqrtf(block_sum(sum_squares(ksrc, nk, a.vec), red) / (float)nk + a.eps);
    const int in_page = pos % PAGE_TOKENS;
    T* kdst = k_cache + ((size_t)page * a.G * PAGE_TOKENS + in_page) * a.dimp;
    if (a.vec) norm_rotate_heads8(ksrc, kw, rk, a.G, a.dim, a.rot, cosr, sinr, kdst, (size_t)PAGE_TOKENS * a.dimp);
    else norm_rotate_heads(ksrc, kw, rk, a.G, a.dim, a.dimp, a.rot, cosr, sinr, kdst, (size_t)PAGE_TOKENS * a.dimp);

    // values: a warp a head
    const T* vsrc = ksrc + nk;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float lam = a.vmix == 2 ? *lambda_p : 0.f;
    for (int g = warp; g < a.G; g += PREP_THREADS / 32) {
        float sv = 0.f;
        for (int d = lane; d < a.vd; d += 32) {
            const float v = to_f32(vsrc[g * a.vd + d]);
            sv = fmaf(v, v, sv);
        }
        const float rv = 1.0f / sqrtf(warp_sum(sv) / (float)a.vd + a.eps);
        T* dst = v_cache + (((size_t)page * a.G + g) * PAGE_TOKENS + in_page) * a.vdp;
        float* vf = v_first ? v_first + ((size_t)row * a.G + g) * a.vd : nullptr;
        for (int d = lane; d < a.vdp; d += 32) {
            float v = 0.f;
            if (d < a.vd) {
                v = to_f32(vsrc[g * a.vd + d]) * rv;
                if (a.vmix == 1) vf[d] = v;
                else if (a.vmix == 2) v = (1.0f - lam) * v + lam * vf[d];
            }
            dst[d] = from_f32<T>(v);
        }
    }
}

// The vector form of the whole kernel (taken when `vec` holds and the values fit too: vd % 8 == 0, vdp == vd, at most
// 8 * 1024 elements a row): a thread fetches its eight-element pieces of q, k and v at once, the three kinds of
// sums of squares are formed together (q and k over the block, a value head over the lanes that hold it: vd / 8, a
// power of two up to 32), and every piece is normed, rotated with its partner piece (fetched again from L1) and stored.
template <typename T>
__global__ void __launch_bounds__(1024)
attn_prep_vec_kernel(const T* __restrict__ qkv, T* __restrict__ q_out, VecRef qw, VecRef kw,
                     const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                     const int* __restrict__ tok_seq, const int* __restrict__ tok_pos, PageTable pt,
                     T* __restrict__ k_cache, T* __restrict__ v_cache, float* __restrict__ v_first,
                     const float* __restrict__ lambda_p, PrepArgs a, int* __restrict__ status) {
    __shared__ float red[2][32];
    griddep_launch_small();
    griddep_wait();
    const int row = blockIdx.x;
    const int b = tok_seq[row];
    T* qo = q_out + (size_t)row * a.ldq;
    const int nq = a.H * a.dim, nk = a.G * a.dim, nv = a.G * a.vd;
    const int i = threadIdx.x * 8;                 // this thread's piece of the row: q, then k, then v
    const bool writes = k_cache != nullptr;
    const int n_all = nq + (writes ? nk + nv : 0);
    if (b < 0) {
        float zero[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (i < nq) store8(qo + i, zero);
        return;
    }
    const int pos = tok_pos[row];
    if (a.rot > 0 && (pos < 0 || pos >= a.n_pos)) {
        if (threadIdx.x == 0) atomicOr(status, MYNAH_ST_POS_RANGE);
        return;
    }
    const int page = writes ? page_of(pt, b, pos) : 0;
    if (page < 0) {
        if (threadIdx.x == 0) atomicOr(status, MYNAH_ST_PAGE_RANGE);
        return;
    }
    const T* src = qkv + (size_t)row * a.ld;
    float x[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (i < n_all) load8(src + i, x);
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < 8; e++) ss = fmaf(x[e], x[e], ss);
    const bool is_q = i < nq, is_k = !is_q && i < nq + nk, is_v = !is_q && !is_k && i < n_all;
    // q and k: two sums over the block, reduced together
    float sq = is_q ? ss : 0.f, sk = is_k ? ss : 0.f;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // a value head lies in vd / 8 consecutive threads of one warp (its start is a multiple of vd / 8 pieces)
    float sv = ss;
    for (int o = (a.vd >> 3) >> 1; o > 0; o >>= 1) sv += __shfl_xor_sync(0xffffffffu, sv, o);
    sq = warp_sum(sq);
    sk = warp_sum(sk);
    if (lane == 0) {
        red[0][warp] = sq;
        red[1][warp] = sk;
    }
    __syncthreads();
    float tq = 0.f, tk = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); w++) {
        tq += red[0][w];
        tk += red[1][w];
    }
    if (is_q || is_k) {
        const float r = 1.0f / sqrtf((is_q ? tq / (float)nq : tk / (float)nk) + a.eps);
        const int local = is_q ? i : i - nq;       // index inside the projection
        const int h = local / a.dim, d = local % a.dim;
        const VecRef& gain = is_q ? qw : kw;
        float g[8], out[8];
        gain8(gain, local, g);
#pragma unroll
        for (int e = 0; e < 8; e++) x[e] = x[e] * r * g[e];
        if (d < a.rot) {
            const int half = a.rot >> 1;
            const bool low = d < half;
            const int pd = low ? d + half : d - half;          // the partner piece
            float y[8], gy[8], c[8], sn[8];
            load8(src + (is_q ? 0 : nq) + h * a.dim + pd, y);
            gain8(gain, h * a.dim + pd, gy);
            const float* cosr = cos_t + (size_t)pos * half + (low ? d : pd);
            const float* sinr = sin_t + (size_t)pos * half + (low ? d : pd);
            load8(cosr, c);
            load8(sinr, sn);
#pragma unroll
            for (int e = 0; e < 8; e++) {
                const float yy = y[e] * r * gy[e];
                out[e] = low ? x[e] * c[e] - yy * sn[e] : x[e] * c[e] + yy * sn[e];
            }
        } else {
#pragma unroll
            for (int e = 0; e < 8; e++) out[e] = x[e];
        }
        if (is_q) store8(qo + h * a.dimp + d, out);
        else store8(k_cache + (((size_t)page * a.G + h) * PAGE_TOKENS + pos % PAGE_TOKENS) * a.dimp + d, out);
    } else if (is_v) {
        const int local = i - nq - nk;
        const int g = local / a.vd, d = local % a.vd;
        const float rv = 1.0f / sqrtf(sv / (float)a.vd + a.eps);
        float out[8];
#pragma unroll
        for (int e = 0; e < 8; e++) out[e] = x[e] * rv;
        if (a.vmix == 1) {
            store8(v_first + (size_t)row * nv + local, out);
        } else if (a.vmix == 2) {
            const float lam = *lambda_p;
            float f[8];
            load8(v_first + (size_t)row * nv + local, f);
#pragma unroll
            for (int e = 0; e < 8; e++) out[e] = (1.0f - lam) * out[e] + lam * f[e];
        }
        store8(v_cache + (((size_t)page * a.G + g) * PAGE_TOKENS + pos % PAGE_TOKENS) * a.vdp + d, out);
    }
}

}  // namespace

// qkv [T, ld]: H*dim query, then G*dim key, then G*vd value outputs a row. q_out [T, ldq] with head h at
// h*dimp. Caches [n_pages][G][PAGE_TOKENS][dimp | vdp]; null caches: only q is made. cos/sin [n_pos, rot/2]
// fp32 (rot 0: no rotation). v_first fp32 [T, G*vd]; lambda: one fp32 on the device.
MYNAH_API int mynah_attn_prep(const void* qkv, int dtype, int T, int ld, void* q_out, int ldq,
                              int H, int G, int dim, int vd, int dimp, int vdp,
                              const void* q_gain, const void* k_gain, int gain_dtype, float eps,
                              const float* cos_t, const float* sin_t, int rot, int n_pos,
                              const int* tok_seq, const int* tok_pos,
                              const int* page_indptr, const int* page_ids, const int* page_base, int n_pages,
                              void* k_cache, void* v_cache, float* v_first, const float* lambda_p, int vmix,
                              int* status, cudaStream_t stream) {
    if (T == 0) return 0;
    MYNAH_REQUIRE(T > 0 && H > 0 && G > 0 && dim > 0 && vd > 0, "attn_prep: bad sizes T=%d H=%d G=%d dim=%d vd=%d", T, H, G, dim, vd);
    MYNAH_REQUIRE(dimp >= dim && vdp >= vd, "attn_prep: stored heads are narrower than the heads");
    MYNAH_REQUIRE(rot >= 0 && rot % 2 == 0 && rot <= dim, "attn_prep: %d rotated dimensions do not fit a head of %d", rot, dim);
    MYNAH_REQUIRE(rot == 0 || (cos_t && sin_t), "attn_prep: no rotation tables given");
    MYNAH_REQUIRE(q_gain && k_gain, "attn_prep: no gains given");
    MYNAH_REQUIRE((k_cache == nullptr) == (v_cache == nullptr), "attn_prep: keys and values are cached together");
    MYNAH_REQUIRE(vmix == 0 || (v_first != nullptr && (vmix == 1 || lambda_p != nullptr)), "attn_prep: value mixing needs its buffers");
    auto fits = [](const void* p) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & 31) == 0; };
    const int vec = dim % 8 == 0 && dimp == dim && rot % 16 == 0 && ld % 8 == 0 && ldq % 8 == 0 && fits(qkv) && fits(q_out) &&
                    fits(q_gain) && fits(k_gain) && fits(cos_t) && fits(sin_t) && fits(k_cache);
    const PrepArgs a{H, G, dim, vd, dimp, vdp, ld, ldq, rot, n_pos, eps, vmix, vec};
    const PageTable pt{page_indptr, page_ids, page_base, n_pages};
    const VecRef qw{q_gain, gain_dtype}, kw{k_gain, gain_dtype};
    const int vd8 = vd / 8;
    const bool one_phase = vec && vd % 8 == 0 && vdp == vd && (vd8 & (vd8 - 1)) == 0 && vd8 <= 32 && fits(v_cache) && fits(v_first) &&
                           H * dim + G * dim + G * vd <= 8 * 1024 && ((H + G) * dim / 8) % vd8 == 0 &&
                           (dtype == MYNAH_F32 || dtype == MYNAH_BF16);
    if (one_phase) {
        const int n_all = H * dim + (k_cache ? G * (dim + vd) : 0);
        const int threads = (n_all / 8 + 31) / 32 * 32;
        if (dtype == MYNAH_F32)
            mynah_launch(attn_prep_vec_kernel<float>, dim3(T), dim3(threads), 0, stream, (const float*)qkv, (float*)q_out, qw, kw,
                         cos_t, sin_t, tok_seq, tok_pos, pt, (float*)k_cache, (float*)v_cache, v_first, lambda_p, a, status);
        else
            mynah_launch(attn_prep_vec_kernel<bf16>, dim3(T), dim3(threads), 0, stream, (const bf16*)qkv, (bf16*)q_out, qw, kw,
                         cos_t, sin_t, tok_seq, tok_pos, pt, (bf16*)k_cache, (bf16*)v_cache, v_first, lambda_p, a, status);
        return mynah_check_launch("attn_prep");
    }
    if (dtype == MYNAH_F32)
        mynah_launch(attn_prep_kernel<float>, dim3(T), dim3(PREP_THREADS), 0, stream, (const float*)qkv, (float*)q_out, qw, kw,
                     cos_t, sin_t, tok_seq, tok_pos, pt, (float*)k_cache, (float*)v_cache, v_first, lambda_p, a, status);
    else if (dtype == MYNAH_BF16)
        mynah_launch(attn_prep_kernel<bf16>, dim3(T), dim3(PREP_THREADS), 0, stream, (const bf16*)qkv, (bf16*)q_out, qw, kw,
                     cos_t, sin_t, tok_seq, tok_pos, pt, (bf16*)k_cache, (bf16*)v_cache, v_first, lambda_p, a, status);
    else
        return mynah_fail("attn_prep: unsupported dtype %d", dtype);
    return mynah_check_launch("attn_prep");
}
