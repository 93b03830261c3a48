// The residual sum of a block whose two parts read the same stream, fused with the norms of the next block:
//
//   v = x[r] + (d1[r] + d2[r])          float; written back to x when no rows are gathered
//   y1 = v / rms(v) * w1,   y2 = v / rms(v) * w2         one statistic, two weights, two outputs
//
// d1, d2, y1 and y2 may each be absent; a null weight with an output present gives y = v rounded once (for a part
// that reads the stream as it is).  Outputs have a pitch of their own, so that a row can land in a wider buffer.
// The stream, the sum and the statistic are float on both paths.  One block per row; the row waits in shared memory.
//
// Also here: the causal convolution over time, per channel, with its last inputs kept per sequence.
#include "common.cuh"

template <typename T>
__global__ void __launch_bounds__(256)
pair_add_rmsnorm_kernel(float* __restrict__ x, const T* __restrict__ d1, const T* __restrict__ d2,
                        const int* __restrict__ rows, const float* __restrict__ w1, T* __restrict__ y1, int ld1,
                        const float* __restrict__ w2, T* __restrict__ y2, int ld2, float eps, int d) {
    pdl_sync();
    extern __shared__ __align__(16) float row_s[];
    __shared__ float red[33];
    const int i = blockIdx.x;
    const size_t r = rows ? (size_t)rows[i] : (size_t)i;
    float ss = 0.f;
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
        float add = 0.f;
        if (d1) add = ldf(d1 + r * d + c);
        if (d2) add += ldf(d2 + r * d + c);
        const float v = x[r * d + c] + add;
        if (!rows && (d1 || d2)) x[r * d + c] = v;
        row_s[c] = v;
        ss += v * v;
    }
    if (!y1 && !y2) return;
    const bool normed = w1 || w2;
    float rs = 1.f;
    if (normed) rs = 1.0f / sqrtf(block_sum(ss, red) / (float)d + eps);
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
        const float v = row_s[c];
        if (y1) stf(y1 + (size_t)i * ld1 + c, w1 ? v * rs * w1[c] : v);
        if (y2) stf(y2 + (size_t)i * ld2 + c, w2 ? v * rs * w2[c] : v);
    }
}

// ---- causal convolution over time ------------------------------------------------------------------------
// y[t, c] = (residual ? u[t, c] : 0) + sum_j w[c, j] * u[t - taps + 1 + j, c]; the inputs before a step's first
// token come from the sequence's state, [taps - 1, C] floats, oldest first (zeros when the sequence starts).
// One thread per (token, channel).  In a step of one token per sequence (`roll`) the same thread also moves the
// state on; after any other step conv_roll_kernel does, once every token has read the old one.
template <typename T>
__global__ void __launch_bounds__(256)
causal_conv_kernel(const T* __restrict__ u, int ldu, const float* __restrict__ w, float* __restrict__ state,
                   long long state_pitch, T* __restrict__ y, int ldy, const int* __restrict__ tok_seq,
                   const int* __restrict__ seq_start, const int* __restrict__ slots, int nt, int C, int taps,
                   int residual, int roll) {
    pdl_sync();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)nt * C) return;
    const int t = (int)(idx / C), c = (int)(idx - (long long)t * C);
    const int b = tok_seq[t];
    const int tl = t - seq_start[b];
    float* st = state + (size_t)slots[b] * state_pitch;
    const float own = ldf(u + (size_t)t * ldu + c);
    float acc = residual ? own : 0.f;
    for (int j = 0; j < taps; ++j) {
        const int back = taps - 1 - j;                 // this tap reads the input `back` tokens earlier
        float v;
        if (back == 0) v = own;
        else if (tl - back >= 0) v = ldf(u + (size_t)(t - back) * ldu + c);
        else v = st[(size_t)(taps - 1 + tl - back) * C + c];
        acc += w[(size_t)c * taps + j] * v;
    }
    stf(y + (size_t)t * ldy + c, acc);
    if (roll) {            // tl == 0: the state moves on by one input
        for (int i = 0; i + 2 < taps; ++i) st[(size_t)i * C + c] = st[(size_t)(i + 1) * C + c];
        if (taps > 1) st[(size_t)(taps - 2) * C + c] = own;
    }
}

// The state after a step of n tokens: entry i is the input at local index n - (taps - 1) + i, which is one of the
// step's rows or, for a short step, an older entry.  One thread per (sequence, channel), so that what it reads of
// the old state it reads before it writes.
template <typename T>
__global__ void __launch_bounds__(256)
conv_roll_kernel(const T* __restrict__ u, int ldu, float* __restrict__ state, long long state_pitch,
                 const int* __restrict__ seq_start, const int* __restrict__ slots, int B, int C, int taps) {
    pdl_sync();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)B * C) return;
    const int b = (int)(idx / C), c = (int)(idx - (long long)b * C);
    const int t0 = seq_start[b], n = seq_start[b + 1] - t0;
    float* st = state + (size_t)slots[b] * state_pitch;
    float keep[15];
    const int m = taps - 1;
    for (int i = 0; i < m; ++i) {
        const int src = n - m + i;
        keep[i] = src >= 0 ? ldf(u + (size_t)(t0 + src) * ldu + c) : st[(size_t)(m + src) * C + c];
    }
    for (int i = 0; i < m; ++i) st[(size_t)i * C + c] = keep[i];
}

extern "C" {
#define TB_STREAM_PAIR(SFX, T)                                                                                        \
    int tb_pair_add_rmsnorm_##SFX(float* x, const void* d1, const void* d2, const int* rows, const float* w1,         \
                                  void* y1, int ld1, const float* w2, void* y2, int ld2, float eps, int n_out,        \
                                  int d, cudaStream_t s) {                                                            \
        if (n_out < 0 || d <= 0 || d > 48 * 1024 / 4) return TB_ERR_ARG;                                              \
        if ((y1 && ld1 < d) || (y2 && ld2 < d) || (w1 && !y1) || (w2 && !y2)) return TB_ERR_ARG;                      \
        if (n_out == 0) return 0;                                                                                     \
        TB_LAUNCH((pair_add_rmsnorm_kernel<T>), n_out, 256, (size_t)d * 4, s, x, (const T*)d1, (const T*)d2, rows,    \
                  w1, (T*)y1, ld1, w2, (T*)y2, ld2, eps, d);                                                          \
        return tb_last_error();                                                                                       \
    }                                                                                                                 \
    int tb_causal_conv_##SFX(const void* u, int ldu, const float* w, float* state, long long state_pitch, void* y,    \
                             int ldy, const int* tok_seq, const int* seq_start, const int* slots, int nt, int B,      \
                             int C, int taps, int residual, int decode, cudaStream_t s) {                             \
        if (nt < 0 || B <= 0 || C <= 0 || taps < 1 || taps > 16 || ldu < C || ldy < C) return TB_ERR_ARG;             \
        if (taps > 1 && (!state || state_pitch < (long long)(taps - 1) * C)) return TB_ERR_ARG;                       \
        if (nt == 0) return 0;                                                                                        \
        const long long n = (long long)nt * C;                                                                        \
        TB_LAUNCH((causal_conv_kernel<T>), (unsigned)((n + 255) / 256), 256, 0, s, (const T*)u, ldu, w, state,        \
                  state_pitch, (T*)y, ldy, tok_seq, seq_start, slots, nt, C, taps, residual, decode ? 1 : 0);         \
        int rc = tb_last_error();                                                                                     \
        if (rc || decode || taps == 1) return rc;                                                                     \
        TB_LAUNCH((conv_roll_kernel<T>), (unsigned)(((long long)B * C + 255) / 256), 256, 0, s, (const T*)u, ldu,     \
                  state, state_pitch, seq_start, slots, B, C, taps);                                                  \
        return tb_last_error();                                                                                       \
    }
#define TB_CONV_ROLL(SFX, T)                                                                                          \
    int tb_conv_roll_##SFX(const void* u, int ldu, float* state, long long state_pitch, const int* seq_start,         \
                           const int* slots, int B, int C, int taps, cudaStream_t s) {                                \
        if (B <= 0 || C <= 0 || taps < 1 || taps > 16 || ldu < C) return TB_ERR_ARG;                                  \
        if (taps == 1) return 0;                                                                                      \
        if (!state || state_pitch < (long long)(taps - 1) * C) return TB_ERR_ARG;                                     \
        TB_LAUNCH((conv_roll_kernel<T>), (unsigned)(((long long)B * C + 255) / 256), 256, 0, s, (const T*)u, ldu,     \
                  state, state_pitch, seq_start, slots, B, C, taps);                                                  \
        return tb_last_error();                                                                                       \
    }
TB_CONV_ROLL(f32, float)
TB_CONV_ROLL(bf16, __nv_bfloat16)
TB_STREAM_PAIR(f32, float)
TB_STREAM_PAIR(bf16, __nv_bfloat16)
}

#include "tape.h"
TB_TAPE_REGISTER(tb_pair_add_rmsnorm_f32)
TB_TAPE_REGISTER(tb_pair_add_rmsnorm_bf16)
TB_TAPE_REGISTER(tb_conv_roll_f32)
TB_TAPE_REGISTER(tb_conv_roll_bf16)
TB_TAPE_REGISTER(tb_causal_conv_f32)
TB_TAPE_REGISTER(tb_causal_conv_bf16)
