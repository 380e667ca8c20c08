// Short causal convolution along each sequence of a ragged step, one filter per channel.
//
//   conv(x)[t, c] = bias[c] + sum_{j=0}^{taps-1} w[c, j] * x[t - (taps-1) + j, c]
//
// with zeros before a sequence's first position: the filter's last column weighs the current token. The inputs
// at the last taps-1 positions of every sequence are carried from step to step in a per-slot state
// [n_slots + 1][taps-1][C] (fp32; the last row belongs to no sequence and serves padding), so a prompt cut into
// pieces, or continued token by token, sums the same products in the same order (j ascending) as a prompt run
// whole. Output: act(conv(x)) or x + act(conv(x)); act: none or silu. All arithmetic is fp32.
//
// A step whose sequences bring more than one row reads the old state in the convolution and shifts it in a
// second launch; a decode step (one row a sequence) does both in one launch, a thread owning its sequence's
// channel.
#include "common.cuh"

namespace {

struct ConvArgs {
    int T, B, C, taps, ldx, ldo, n_slots;
    int act;          // 0: none, 1: silu
    int add_input;    // 1: out = x + act(conv(x))
    int update;       // 1: one row a sequence, shift the state here
};

__device__ __forceinline__ float silu_f(float v) { return v / (1.0f + expf(-v)); }

template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
causal_conv_kernel(const TI* __restrict__ x, VecRef w, VecRef bias, float* __restrict__ state, TO* __restrict__ out,
                   const int* __restrict__ tok_seq, const int* __restrict__ cu_q, const int* __restrict__ slots,
                   ConvArgs a) {
    griddep_launch_small();
    griddep_wait();
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    const int row = blockIdx.x;
    if (c >= a.C) return;
    const int b = tok_seq[row];
    TO* o = out + (size_t)row * a.ldo + c;
    if (b < 0 || b >= a.B) {                       // a padding row
        *o = from_f32<TO>(0.f);
        return;
    }
    const int i = row - cu_q[b];                   // place of the row in its sequence's piece
    int slot = slots[b];
    if (slot < 0 || slot >= a.n_slots) slot = a.n_slots;
    const int hist = a.taps - 1;
    float* st = state + (size_t)slot * hist * a.C + c;
    float acc = bias.p ? bias.at(c) : 0.f;
    const float cur = to_f32(x[(size_t)row * a.ldx + c]);
    for (int j = 0; j < a.taps; j++) {
        const int src = i - hist + j;              // place of the input in the piece; negative: before it
        float v;
        if (j == hist) v = cur;
        else if (src >= 0) v = to_f32(x[(size_t)(row - hist + j) * a.ldx + c]);
        else v = st[(size_t)(hist + src) * a.C];
        acc = fmaf(w.at(c * a.taps + j), v, acc);
    }
    if (a.act == 1) acc = silu_f(acc);
    if (a.add_input) acc += cur;
    *o = from_f32<TO>(acc);
    if (a.update) {                                // i == 0 and the piece is this row alone
        for (int k = 0; k + 1 < hist; k++) st[(size_t)k * a.C] = st[(size_t)(k + 1) * a.C];
        if (hist > 0) st[(size_t)(hist - 1) * a.C] = cur;
    }
}

// state[k] <- the input at the piece's place q_len - (taps-1) + k, which lies in the piece or, for a short
// piece, in the old state at k + q_len (read before any smaller k is written: one thread walks k upwards).
template <typename TI>
__global__ void __launch_bounds__(256)
conv_state_shift_kernel(const TI* __restrict__ x, float* __restrict__ state, const int* __restrict__ cu_q,
                        const int* __restrict__ slots, ConvArgs a) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int b = blockIdx.y;
    if (c >= a.C) return;
    const int slot = slots[b];
    if (slot < 0 || slot >= a.n_slots) return;
    const int q0 = cu_q[b], q_len = cu_q[b + 1] - q0;
    if (q_len <= 0) return;
    const int hist = a.taps - 1;
    float* st = state + (size_t)slot * hist * a.C + c;
    for (int k = 0; k < hist; k++) {
        const int src = q_len - hist + k;
        st[(size_t)k * a.C] = src >= 0 ? to_f32(x[(size_t)(q0 + src) * a.ldx + c]) : st[(size_t)(k + q_len) * a.C];
    }
}

// The same convolution, eight consecutive channels a thread with 16-byte accesses (channels, strides and
// addresses must fit them); the products are summed in the same order.
template <typename TI, typename TO>
__global__ void __launch_bounds__(128)
causal_conv8_kernel(const TI* __restrict__ x, VecRef w, VecRef bias, float* __restrict__ state, TO* __restrict__ out,
                    const int* __restrict__ tok_seq, const int* __restrict__ cu_q, const int* __restrict__ slots,
                    ConvArgs a) {
    griddep_launch_small();
    griddep_wait();
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
    const int row = blockIdx.x;
    if (c >= a.C) return;
    const int b = tok_seq[row];
    TO* o = out + (size_t)row * a.ldo + c;
    float acc[8], cur[8], v[8];
    if (b < 0 || b >= a.B) {
#pragma unroll
        for (int k = 0; k < 8; k++) acc[k] = 0.f;
        store8(o, acc);
        return;
    }
    const int i = row - cu_q[b];
    int slot = slots[b];
    if (slot < 0 || slot >= a.n_slots) slot = a.n_slots;
    const int hist = a.taps - 1;
    float* st = state + (size_t)slot * hist * a.C + c;
#pragma unroll
    for (int k = 0; k < 8; k++) acc[k] = bias.p ? bias.at(c + k) : 0.f;
    load8(x + (size_t)row * a.ldx + c, cur);
    for (int j = 0; j < a.taps; j++) {
        const int src = i - hist + j;
        if (j == hist) {
#pragma unroll
            for (int k = 0; k < 8; k++) v[k] = cur[k];
        } else if (src >= 0) {
            load8(x + (size_t)(row - hist + j) * a.ldx + c, v);
        } else {
            load8(st + (size_t)(hist + src) * a.C, v);
        }
#pragma unroll
        for (int k = 0; k < 8; k++) acc[k] = fmaf(w.at((c + k) * a.taps + j), v[k], acc[k]);
    }
#pragma unroll
    for (int k = 0; k < 8; k++) {
        if (a.act == 1) acc[k] = silu_f(acc[k]);
        if (a.add_input) acc[k] += cur[k];
    }
    store8(o, acc);
    if (a.update) {
        for (int k = 0; k + 1 < hist; k++) {
            load8(st + (size_t)(k + 1) * a.C, v);
            store8(st + (size_t)k * a.C, v);
        }
        if (hist > 0) store8(st + (size_t)(hist - 1) * a.C, cur);
    }
}

// Prompt steps: a thread takes eight channels of CONV_ROWS consecutive rows, keeps its 8 x taps weights and the last
// taps-1 inputs in registers and lets the rows slide through: every input is fetched once and every weight once a
// tile. A sequence that starts inside the tile (or the tile's first row) refills the window from the rows before it
// or from the state. Filters of up to 4 taps; the products are summed in the same order as in the other forms.
constexpr int CONV_ROWS = 4;
constexpr int CONV_MAXT = 4;

template <typename TI, typename TO>
__global__ void __launch_bounds__(128)
causal_conv8_rows_kernel(const TI* __restrict__ x, VecRef w, VecRef bias, const float* __restrict__ state,
                         TO* __restrict__ out, const int* __restrict__ tok_seq, const int* __restrict__ cu_q,
                         const int* __restrict__ slots, ConvArgs a) {
    griddep_launch_small();
    griddep_wait();
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
    if (c >= a.C) return;
    const int hist = a.taps - 1;
    float wr[CONV_MAXT][8], bb[8], win[CONV_MAXT - 1][8];
#pragma unroll
    for (int j = 0; j < CONV_MAXT; j++)
#pragma unroll
        for (int k = 0; k < 8; k++) wr[j][k] = j < a.taps ? w.at((c + k) * a.taps + j) : 0.f;
#pragma unroll
    for (int k = 0; k < 8; k++) bb[k] = bias.p ? bias.at(c + k) : 0.f;
    const int row0 = blockIdx.x * CONV_ROWS;
    int last_b = -2;
    float curs[CONV_ROWS][8];                      // every row's input is asked for before the first is used
#pragma unroll
    for (int r = 0; r < CONV_ROWS; r++)
        if (row0 + r < a.T) load8(x + (size_t)(row0 + r) * a.ldx + c, curs[r]);
#pragma unroll
    for (int r = 0; r < CONV_ROWS; r++) {
        const int row = row0 + r;
        if (row >= a.T) break;
        float (&cur)[8] = curs[r];
        const int b = tok_seq[row];
        TO* o = out + (size_t)row * a.ldo + c;
        float acc[8];
        if (b < 0 || b >= a.B) {
#pragma unroll
            for (int k = 0; k < 8; k++) acc[k] = 0.f;
            store8(o, acc);
            last_b = -2;
            continue;
        }
        const int i = row - cu_q[b];
        if (b != last_b) {                         // the window: win[m] is the input hist - m places back... filled oldest first
            int slot = slots[b];
            if (slot < 0 || slot >= a.n_slots) slot = a.n_slots;
            const float* st = state + (size_t)slot * hist * a.C + c;
#pragma unroll
            for (int m = 0; m < CONV_MAXT - 1; m++) {
                if (m < hist) {
                    const int src = i - hist + m;
                    if (src >= 0) load8(x + (size_t)(row - hist + m) * a.ldx + c, win[m]);
                    else load8(st + (size_t)(hist + src) * a.C, win[m]);
                }
            }
            last_b = b;
        }
#pragma unroll
        for (int k = 0; k < 8; k++) acc[k] = bb[k];
#pragma unroll
        for (int j = 0; j < CONV_MAXT; j++) {
            if (j < hist) {
#pragma unroll
                for (int k = 0; k < 8; k++) acc[k] = fmaf(wr[j][k], win[j][k], acc[k]);
            } else if (j == hist) {
#pragma unroll
                for (int k = 0; k < 8; k++) acc[k] = fmaf(wr[j][k], cur[k], acc[k]);
            }
        }
#pragma unroll
        for (int k = 0; k < 8; k++) {
            if (a.act == 1) acc[k] = silu_f(acc[k]);
            if (a.add_input) acc[k] += cur[k];
        }
        store8(o, acc);
#pragma unroll
        for (int m = 0; m < CONV_MAXT - 1; m++) {      // slide: drop the oldest, the current input becomes the newest
            if (m + 1 < hist) {
#pragma unroll
                for (int k = 0; k < 8; k++) win[m][k] = win[m + 1][k];
            } else if (m + 1 == hist) {
#pragma unroll
                for (int k = 0; k < 8; k++) win[m][k] = cur[k];
            }
        }
    }
}

template <typename TI, typename TO>
int launch_conv(const void* x, const VecRef& w, const VecRef& bias, float* state, void* out, const int* tok_seq,
                const int* cu_q, const int* slots, const ConvArgs& a, cudaStream_t stream) {
    const int threads = a.C >= 256 ? 256 : (a.C >= 128 ? 128 : 64);
    const dim3 grid(a.T, ceil_div(a.C, threads));
    auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 31) == 0; };
    const bool vec8 = a.C % 8 == 0 && a.ldx % 8 == 0 && a.ldo % 8 == 0 && al(x) && al(out) && al(state);
    const int t8 = a.C / 8 >= 128 ? 128 : (a.C / 8 >= 64 ? 64 : 32);
    if (vec8 && !a.update && a.taps <= CONV_MAXT && a.T >= 4 * CONV_ROWS) {
        // a prompt step: rows slide through registers
        mynah_launch(causal_conv8_rows_kernel<TI, TO>, dim3(ceil_div(a.T, CONV_ROWS), ceil_div(a.C / 8, t8)), dim3(t8), 0,
                     stream, (const TI*)x, w, bias, (const float*)state, (TO*)out, tok_seq, cu_q, slots, a);
    } else if (vec8) {
        mynah_launch(causal_conv8_kernel<TI, TO>, dim3(a.T, ceil_div(a.C / 8, t8)), dim3(t8), 0, stream, (const TI*)x, w, bias,
                     state, (TO*)out, tok_seq, cu_q, slots, a);
    } else {
        mynah_launch(causal_conv_kernel<TI, TO>, grid, dim3(threads), 0, stream, (const TI*)x, w, bias, state, (TO*)out,
                     tok_seq, cu_q, slots, a);
    }
    if (mynah_check_launch("causal_conv")) return -1;
    if (!a.update && a.taps > 1) {
        conv_state_shift_kernel<TI><<<dim3(ceil_div(a.C, threads), a.B), threads, 0, stream>>>((const TI*)x, state, cu_q, slots, a);
        return mynah_check_launch("conv_state_shift");
    }
    return 0;
}

}  // namespace

// x [T, ldx] (x_dtype), w [C, taps] and bias [C] or null (w_dtype), state [n_slots + 1, taps - 1, C] fp32,
// out [T, ldo] (out_dtype). one_row_each: every sequence of the step brings exactly one row and row b is
// sequence b (a decode step); the state is then shifted by the same launch.
MYNAH_API int mynah_causal_conv(const void* x, int x_dtype, int ldx, const void* w, const void* bias, int w_dtype,
                                float* state, int n_slots, void* out, int out_dtype, int ldo,
                                const int* tok_seq, const int* cu_q, const int* slots,
                                int T, int B, int C, int taps, int act, int add_input, int one_row_each,
                                cudaStream_t stream) {
    if (T == 0 || C == 0) return 0;
    MYNAH_REQUIRE(T > 0 && B > 0 && C > 0 && taps >= 1, "causal_conv: bad sizes T=%d B=%d C=%d taps=%d", T, B, C, taps);
    MYNAH_REQUIRE(ldx >= C && ldo >= C, "causal_conv: a row stride is smaller than the channels");
    MYNAH_REQUIRE(act == 0 || act == 1, "causal_conv: unknown activation %d", act);
    MYNAH_REQUIRE(taps == 1 || state != nullptr, "causal_conv: no state given");
    MYNAH_REQUIRE(B <= 65535 && ceil_div(C, 64) <= 65535, "causal_conv: B=%d or C=%d exceeds one launch", B, C);
    const ConvArgs a{T, B, C, taps, ldx, ldo, n_slots, act, add_input, one_row_each ? 1 : 0};
    const VecRef wv{w, w_dtype}, bv{bias, w_dtype};
    if (x_dtype == MYNAH_F32 && out_dtype == MYNAH_F32)
        return launch_conv<float, float>(x, wv, bv, state, out, tok_seq, cu_q, slots, a, stream);
    if (x_dtype == MYNAH_F32 && out_dtype == MYNAH_BF16)
        return launch_conv<float, bf16>(x, wv, bv, state, out, tok_seq, cu_q, slots, a, stream);
    if (x_dtype == MYNAH_BF16 && out_dtype == MYNAH_BF16)
        return launch_conv<bf16, bf16>(x, wv, bv, state, out, tok_seq, cu_q, slots, a, stream);
    if (x_dtype == MYNAH_BF16 && out_dtype == MYNAH_F32)
        return launch_conv<bf16, float>(x, wv, bv, state, out, tok_seq, cu_q, slots, a, stream);
    return mynah_fail("causal_conv: unsupported dtypes %d -> %d", x_dtype, out_dtype);
}
