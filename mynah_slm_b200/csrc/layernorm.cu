// Layer norm with weight and bias over the last dimension:
//
//   LN(v)[i] = (v[i] - mean) / sqrt(var + eps) * w[i] + b[i],   var = mean((v - mean)^2)
//
// Mean, variance and the result are fp32; the variance is taken from the deviations (second pass over the row,
// which a thread keeps in registers), not from E[v^2] - mean^2. Sums run in an order fixed by the thread layout.
//
// Two forms. `layernorm_rows`: out = LN(x[rows]) from the fp32 residual stream, for a model's last norm.
// `layernorm_add`: x += LN(y), for a block that norms a sublayer's OUTPUT before the residual add; it can also
// leave a copy of the new x in the activation type, which is what the next sublayer reads.
#include "common.cuh"

namespace {

constexpr int LN_THREADS = 256;
constexpr int LN_MAX_PER_THREAD = 32;       // rows of up to 8,192 elements stay in registers

template <typename TY>
__device__ __forceinline__ void ln_stats(const TY* __restrict__ v, int D, float* red, float (&keep)[LN_MAX_PER_THREAD],
                                         bool in_regs, float eps, float& mean, float& rstd) {
    float s = 0.f;
    if (in_regs) {
#pragma unroll
        for (int k = 0; k < LN_MAX_PER_THREAD; k++) {
            const int i = threadIdx.x + k * LN_THREADS;
            keep[k] = i < D ? to_f32(v[i]) : 0.f;
            s += keep[k];
        }
    } else {
        for (int i = threadIdx.x; i < D; i += LN_THREADS) s += to_f32(v[i]);
    }
    mean = block_sum(s, red) / (float)D;
    float q = 0.f;
    if (in_regs) {
#pragma unroll
        for (int k = 0; k < LN_MAX_PER_THREAD; k++) {
            const int i = threadIdx.x + k * LN_THREADS;
            const float d = keep[k] - mean;
            if (i < D) q = fmaf(d, d, q);
        }
    } else {
        for (int i = threadIdx.x; i < D; i += LN_THREADS) {
            const float d = to_f32(v[i]) - mean;
            q = fmaf(d, d, q);
        }
    }
    const float var = block_sum(q, red) / (float)D;
    rstd = 1.0f / sqrtf(var + eps);
}

template <typename TA>
__global__ void __launch_bounds__(LN_THREADS)
layernorm_rows_kernel(const float* __restrict__ x, const int* __restrict__ rows, VecRef w, VecRef b,
                      TA* __restrict__ out, int D, float eps) {
    __shared__ float red[32];
    griddep_launch_small();
    griddep_wait();
    const int r = rows ? rows[blockIdx.x] : blockIdx.x;
    const float* v = x + (size_t)r * D;
    float keep[LN_MAX_PER_THREAD];
    const bool in_regs = D <= LN_THREADS * LN_MAX_PER_THREAD;
    float mean, rstd;
    ln_stats<float>(v, D, red, keep, in_regs, eps, mean, rstd);
    TA* o = out + (size_t)blockIdx.x * D;
    for (int i = threadIdx.x; i < D; i += LN_THREADS)
        o[i] = from_f32<TA>((v[i] - mean) * rstd * w.at(i) + (b.p ? b.at(i) : 0.f));
}

template <typename TY, typename TA>
__global__ void __launch_bounds__(LN_THREADS)
layernorm_add_kernel(const TY* __restrict__ y, int ldy, VecRef w, VecRef b, float* __restrict__ x,
                     TA* __restrict__ x_copy, int D, float eps) {
    __shared__ float red[32];
    griddep_launch_small();
    griddep_wait();
    const int r = blockIdx.x;
    const TY* v = y + (size_t)r * ldy;
    float keep[LN_MAX_PER_THREAD];
    const bool in_regs = D <= LN_THREADS * LN_MAX_PER_THREAD;
    float mean, rstd;
    ln_stats<TY>(v, D, red, keep, in_regs, eps, mean, rstd);
    float* xr = x + (size_t)r * D;
    for (int i = threadIdx.x; i < D; i += LN_THREADS) {
        const float n = (to_f32(v[i]) - mean) * rstd * w.at(i) + (b.p ? b.at(i) : 0.f);
        const float s = xr[i] + n;
        xr[i] = s;
        if (x_copy) x_copy[(size_t)r * D + i] = from_f32<TA>(s);
    }
}

// The same two norms for rows whose width is a multiple of 8 and at most 8 * 1024: eight consecutive elements a
// thread, every access a 16-byte vector (two for fp32), the row held in registers between the passes.
template <typename TY>
__device__ __forceinline__ void ln_stats8(const float (&v)[8], bool active, int D, float* red, float eps, float& mean, float& rstd) {
    float s = 0.f;
    if (active) {
#pragma unroll
        for (int k = 0; k < 8; k++) s += v[k];
    }
    mean = block_sum(s, red) / (float)D;
    float q = 0.f;
    if (active) {
#pragma unroll
        for (int k = 0; k < 8; k++) {
            const float d = v[k] - mean;
            q = fmaf(d, d, q);
        }
    }
    rstd = 1.0f / sqrtf(block_sum(q, red) / (float)D + eps);
}

__device__ __forceinline__ void load_gain8(const VecRef& w, int i, float (&g)[8], float fill) {
    if (w.p == nullptr) {
#pragma unroll
        for (int k = 0; k < 8; k++) g[k] = fill;
    } else if (w.dtype == MYNAH_F32) {
        load8(static_cast<const float*>(w.p) + i, g);
    } else {
        load8(static_cast<const bf16*>(w.p) + i, g);
    }
}

template <typename TY, typename TA>
__global__ void __launch_bounds__(1024)
layernorm_add8_kernel(const TY* __restrict__ y, int ldy, VecRef w, VecRef b, float* __restrict__ x,
                      TA* __restrict__ x_copy, int D, float eps) {
    __shared__ float red[32];
    griddep_launch_small();
    griddep_wait();
    const int r = blockIdx.x, i = threadIdx.x * 8;
    const bool active = i < D;
    float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, xv[8], g[8], bb[8];
    if (active) {
        load8(y + (size_t)r * ldy + i, v);
        load8(x + (size_t)r * D + i, xv);
        load_gain8(w, i, g, 1.f);
        load_gain8(b, i, bb, 0.f);
    }
    float mean, rstd;
    ln_stats8<TY>(v, active, D, red, eps, mean, rstd);
    if (active) {
#pragma unroll
        for (int k = 0; k < 8; k++) xv[k] += (v[k] - mean) * rstd * g[k] + bb[k];
        store8(x + (size_t)r * D + i, xv);
        if (x_copy) store8(x_copy + (size_t)r * D + i, xv);
    }
}

template <typename TA>
__global__ void __launch_bounds__(1024)
layernorm_rows8_kernel(const float* __restrict__ x, const int* __restrict__ rows, VecRef w, VecRef b,
                       TA* __restrict__ out, int D, float eps) {
    __shared__ float red[32];
    griddep_launch_small();
    griddep_wait();
    const int r = rows ? rows[blockIdx.x] : blockIdx.x, i = threadIdx.x * 8;
    const bool active = i < D;
    float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, g[8], bb[8];
    if (active) {
        load8(x + (size_t)r * D + i, v);
        load_gain8(w, i, g, 1.f);
        load_gain8(b, i, bb, 0.f);
    }
    float mean, rstd;
    ln_stats8<float>(v, active, D, red, eps, mean, rstd);
    if (active) {
#pragma unroll
        for (int k = 0; k < 8; k++) v[k] = (v[k] - mean) * rstd * g[k] + bb[k];
        store8(out + (size_t)blockIdx.x * D + i, v);
    }
}

// Whether the eight-a-thread kernels take these rows: width, strides and addresses fit 16-byte vectors of every type.
inline bool vec8_ok(int D, int ld, const void* p0, const void* p1, const void* p2, const void* p3, const void* p4) {
    auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 31) == 0; };
    return D % 8 == 0 && D <= 8 * 1024 && ld % 8 == 0 && al(p0) && al(p1) && al(p2) && al(p3) && al(p4);
}

}  // namespace

// out[n, :] = LN(x[rows[n], :]) (rows null: every row). x fp32 [*, D]; out in out_dtype.
MYNAH_API int mynah_layernorm_rows(const float* x, const int* rows, const void* w, const void* b, int w_dtype,
                                   void* out, int out_dtype, int n, int D, float eps, cudaStream_t stream) {
    if (n == 0) return 0;
    MYNAH_REQUIRE(n > 0 && D > 0, "layernorm_rows: bad sizes n=%d D=%d", n, D);
    const VecRef wv{w, w_dtype}, bv{b, w_dtype};
    if (vec8_ok(D, D, x, w, b, out, nullptr) && (out_dtype == MYNAH_F32 || out_dtype == MYNAH_BF16)) {
        const int threads = (D / 8 + 31) / 32 * 32;
        if (out_dtype == MYNAH_F32)
            mynah_launch(layernorm_rows8_kernel<float>, dim3(n), dim3(threads), 0, stream, x, rows, wv, bv, (float*)out, D, eps);
        else
            mynah_launch(layernorm_rows8_kernel<bf16>, dim3(n), dim3(threads), 0, stream, x, rows, wv, bv, (bf16*)out, D, eps);
        return mynah_check_launch("layernorm_rows");
    }
    if (out_dtype == MYNAH_F32)
        mynah_launch(layernorm_rows_kernel<float>, dim3(n), dim3(LN_THREADS), 0, stream, x, rows, wv, bv, (float*)out, D, eps);
    else if (out_dtype == MYNAH_BF16)
        mynah_launch(layernorm_rows_kernel<bf16>, dim3(n), dim3(LN_THREADS), 0, stream, x, rows, wv, bv, (bf16*)out, D, eps);
    else
        return mynah_fail("layernorm_rows: unsupported dtype %d", out_dtype);
    return mynah_check_launch("layernorm_rows");
}

// x[r, :] += LN(y[r, :]) for r < n; y [n, ldy] in y_dtype; x fp32 [n, D]; x_copy (null or [n, D] in copy_dtype)
// receives the new x. A bfloat16 run may hand y over in fp32 (the product's accumulators, unrounded) and still ask
// for a bfloat16 copy.
MYNAH_API int mynah_layernorm_add(const void* y, int y_dtype, int ldy, const void* w, const void* b, int w_dtype,
                                  float* x, void* x_copy, int copy_dtype, int n, int D, float eps, cudaStream_t stream) {
    if (n == 0) return 0;
    MYNAH_REQUIRE(n > 0 && D > 0 && ldy >= D, "layernorm_add: bad sizes n=%d D=%d ldy=%d", n, D, ldy);
    const VecRef wv{w, w_dtype}, bv{b, w_dtype};
    if (x_copy == nullptr) copy_dtype = y_dtype;
    const int combo = y_dtype == MYNAH_F32 && copy_dtype == MYNAH_F32 ? 0
                      : (y_dtype == MYNAH_BF16 && copy_dtype == MYNAH_BF16 ? 1
                         : (y_dtype == MYNAH_F32 && copy_dtype == MYNAH_BF16 ? 2 : -1));
    MYNAH_REQUIRE(combo >= 0, "layernorm_add: unsupported dtypes %d -> %d", y_dtype, copy_dtype);
    if (vec8_ok(D, ldy, y, w, b, x, x_copy)) {
        const int threads = (D / 8 + 31) / 32 * 32;
        if (combo == 0)
            mynah_launch(layernorm_add8_kernel<float, float>, dim3(n), dim3(threads), 0, stream, (const float*)y, ldy, wv, bv,
                         x, (float*)x_copy, D, eps);
        else if (combo == 1)
            mynah_launch(layernorm_add8_kernel<bf16, bf16>, dim3(n), dim3(threads), 0, stream, (const bf16*)y, ldy, wv, bv,
                         x, (bf16*)x_copy, D, eps);
        else
            mynah_launch(layernorm_add8_kernel<float, bf16>, dim3(n), dim3(threads), 0, stream, (const float*)y, ldy, wv, bv,
                         x, (bf16*)x_copy, D, eps);
        return mynah_check_launch("layernorm_add");
    }
    if (combo == 0)
        mynah_launch(layernorm_add_kernel<float, float>, dim3(n), dim3(LN_THREADS), 0, stream, (const float*)y, ldy, wv, bv,
                     x, (float*)x_copy, D, eps);
    else if (combo == 1)
        mynah_launch(layernorm_add_kernel<bf16, bf16>, dim3(n), dim3(LN_THREADS), 0, stream, (const bf16*)y, ldy, wv, bv,
                     x, (bf16*)x_copy, D, eps);
    else
        mynah_launch(layernorm_add_kernel<float, bf16>, dim3(n), dim3(LN_THREADS), 0, stream, (const float*)y, ldy, wv, bv,
                     x, (bf16*)x_copy, D, eps);
    return mynah_check_launch("layernorm_add");
}
