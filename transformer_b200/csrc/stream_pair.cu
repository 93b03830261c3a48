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

// The same with four neighbouring entries a thread and access (16 bytes of the float stream and of float inputs, 8
// of 16-bit ones), where the sizes and addresses allow it.
template <typename T>
__device__ __forceinline__ float4 ld4f(const T* p) {
    if constexpr (sizeof(T) == 2) {
        const uint2 raw = *reinterpret_cast<const uint2*>(p);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        return make_float4(a.x, a.y, b.x, b.y);
    } else {
        return *reinterpret_cast<const float4*>(p);
    }
}
template <typename T>
__device__ __forceinline__ void st4f(T* p, float4 v) {
    if constexpr (sizeof(T) == 2) {
        uint2 raw;
        *reinterpret_cast<__nv_bfloat162*>(&raw.x) = __floats2bfloat162_rn(v.x, v.y);
        *reinterpret_cast<__nv_bfloat162*>(&raw.y) = __floats2bfloat162_rn(v.z, v.w);
        *reinterpret_cast<uint2*>(p) = raw;
    } else {
        *reinterpret_cast<float4*>(p) = v;
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
pair_add_rmsnorm_vec_kernel(float* __restrict__ x, const T* __restrict__ d1, const T* __restrict__ d2,
                            const int* __restrict__ rows, const float* __restrict__ w1, T* __restrict__ y1, int ld1,
                            const float* __restrict__ w2, T* __restrict__ y2, int ld2, float eps, int d) {
    pdl_sync();
    extern __shared__ __align__(16) float row_s[];
    __shared__ float red[33];
    const int i = blockIdx.x;
    const size_t r = rows ? (size_t)rows[i] : (size_t)i;
    float ss = 0.f;
    for (int c = threadIdx.x * 4; c < d; c += blockDim.x * 4) {
        float4 add = make_float4(0.f, 0.f, 0.f, 0.f);
        if (d1) add = ld4f(d1 + r * d + c);
        if (d2) {
            const float4 b = ld4f(d2 + r * d + c);
            add.x += b.x; add.y += b.y; add.z += b.z; add.w += b.w;
        }
        float4 v = *reinterpret_cast<const float4*>(x + r * d + c);
        v.x += add.x; v.y += add.y; v.z += add.z; v.w += add.w;
        if (!rows && (d1 || d2)) *reinterpret_cast<float4*>(x + r * d + c) = v;
        *reinterpret_cast<float4*>(row_s + c) = v;
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    if (!y1 && !y2) return;
    const bool normed = w1 || w2;
    float rs = 1.f;
    if (normed) rs = 1.0f / sqrtf(block_sum(ss, red) / (float)d + eps);
    for (int c = threadIdx.x * 4; c < d; c += blockDim.x * 4) {
        const float4 v = *reinterpret_cast<const float4*>(row_s + c);
        if (y1) {
            float4 o = v;
            if (w1) {
                const float4 w = *reinterpret_cast<const float4*>(w1 + c);
                o = make_float4(v.x * rs * w.x, v.y * rs * w.y, v.z * rs * w.z, v.w * rs * w.w);
            }
            st4f(y1 + (size_t)i * ld1 + c, o);
        }
        if (y2) {
            float4 o = v;
            if (w2) {
                const float4 w = *reinterpret_cast<const float4*>(w2 + c);
                o = make_float4(v.x * rs * w.x, v.y * rs * w.y, v.z * rs * w.z, v.w * rs * w.w);
            }
            st4f(y2 + (size_t)i * ld2 + c, o);
        }
    }
}

// ---- causal convolution over time ------------------------------------------------------------------------
// y[t, c] = (residual ? u[t, c] : 0) + sum_j w[c, j] * u[t - taps + 1 + j, c]; the inputs before a step's first
// token come from the sequence's state, [taps - 1, C] floats, oldest first (zeros when the sequence starts).
// One thread per (token, V neighbouring channels): V entries of 16 bytes together where the layout allows it, else
// one.  In a step of one token per sequence (`roll`) the same thread also moves the state on; after any other step
// conv_roll_kernel does, once every token has read the old one.
template <typename T, int V>
struct ConvVec {
    float v[V];
    __device__ __forceinline__ void load(const T* p) {
        if constexpr (V == 1) {
            v[0] = ldf(p);
        } else if constexpr (sizeof(T) == 2) {
            const uint4 raw = *reinterpret_cast<const uint4*>(p);
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int i = 0; i < V / 2; ++i) {
                const float2 f = __bfloat1622float2(h[i]);
                v[2 * i] = f.x;
                v[2 * i + 1] = f.y;
            }
        } else {
            const float4 f = *reinterpret_cast<const float4*>(p);
            v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
        }
    }
    __device__ __forceinline__ void store(T* p) const {
        if constexpr (V == 1) {
            stf(p, v[0]);
        } else if constexpr (sizeof(T) == 2) {
            uint4 raw;
            __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
            for (int i = 0; i < V / 2; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            *reinterpret_cast<uint4*>(p) = raw;
        } else {
            *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
        }
    }
};

template <typename T, int V>
__global__ void __launch_bounds__(128)
causal_conv_kernel(const T* __restrict__ u, int ldu, const float* __restrict__ w, float* __restrict__ state,
                   long long state_pitch, T* __restrict__ y, int ldy, const int* __restrict__ tok_seq,
                   const int* __restrict__ seq_start, const int* __restrict__ slots, int nt, int C, int taps,
                   int residual, int roll) {
    pdl_sync();
    const int t = blockIdx.x;
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * V;
    if (c >= C) return;
    const int b = tok_seq[t];
    const int tl = t - seq_start[b];
    float* st = state ? state + (size_t)slots[b] * state_pitch : nullptr;
    ConvVec<T, V> own, in, acc;
    own.load(u + (size_t)t * ldu + c);
#pragma unroll
    for (int i = 0; i < V; ++i) acc.v[i] = residual ? own.v[i] : 0.f;
    for (int j = 0; j < taps; ++j) {
        const int back = taps - 1 - j;                 // this tap reads the input `back` tokens earlier
        if (back == 0) {
            in = own;
        } else if (tl - back >= 0) {
            in.load(u + (size_t)(t - back) * ldu + c);
        } else {
            const float* sp = st + (size_t)(taps - 1 + tl - back) * C + c;
#pragma unroll
            for (int i = 0; i < V; ++i) in.v[i] = sp[i];
        }
#pragma unroll
        for (int i = 0; i < V; ++i) acc.v[i] += w[(size_t)(c + i) * taps + j] * in.v[i];
    }
    acc.store(y + (size_t)t * ldy + c);
    if (roll && taps > 1) {            // tl == 0: the state moves on by one input
        for (int k = 0; k + 2 < taps; ++k)
#pragma unroll
            for (int i = 0; i < V; ++i) st[(size_t)k * C + c + i] = st[(size_t)(k + 1) * C + c + i];
#pragma unroll
        for (int i = 0; i < V; ++i) st[(size_t)(taps - 2) * C + c + i] = own.v[i];
    }
}

// The same sum for a prompt: a thread takes V neighbouring channels of a tile of consecutive tokens.  Its V x TAPS
// weights are fetched once (16 bytes at a time) and the last TAPS - 1 inputs slide along in registers, so every
// input is read once, and the tile's rows are all asked for before the first is used.  Where a sequence's portion
// starts inside the tile the window is filled from that sequence's state.
template <typename T, int V, int TAPS, int TILE>
__global__ void __launch_bounds__(64)
causal_conv_tile_kernel(const T* __restrict__ u, int ldu, const float* __restrict__ w, const float* __restrict__ state,
                        long long state_pitch, T* __restrict__ y, int ldy, const int* __restrict__ tok_seq,
                        const int* __restrict__ seq_start, const int* __restrict__ slots, int nt, int C, int residual) {
    pdl_sync();
    const int t0 = blockIdx.x * TILE;
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * V;
    if (c >= C) return;
    float wr[V * TAPS];                                   // wr[i * TAPS + j]: channel c + i, tap j
    {
        const float4* wp = reinterpret_cast<const float4*>(w + (size_t)c * TAPS);
#pragma unroll
        for (int k = 0; k < V * TAPS / 4; ++k) {
            const float4 f = wp[k];
            wr[4 * k] = f.x; wr[4 * k + 1] = f.y; wr[4 * k + 2] = f.z; wr[4 * k + 3] = f.w;
        }
    }
    uint4 raw[TILE];                                      // the tile's rows as they lie in memory, 16 bytes each
#pragma unroll
    for (int tt = 0; tt < TILE; ++tt)
        if (t0 + tt < nt) raw[tt] = *reinterpret_cast<const uint4*>(u + (size_t)(t0 + tt) * ldu + c);
    ConvVec<T, V> hist[TAPS - 1];                         // hist[k]: the input k + 1 tokens back
    {
        const int b = tok_seq[t0];
        const int tl = t0 - seq_start[b];
        const float* st = state + (size_t)slots[b] * state_pitch;
#pragma unroll
        for (int k = 0; k < TAPS - 1; ++k) {
            const int back = k + 1;
            if (tl - back >= 0) {
                hist[k].load(u + (size_t)(t0 - back) * ldu + c);
            } else {
                const float* sp = st + (size_t)(TAPS - 1 + tl - back) * C + c;
#pragma unroll
                for (int i = 0; i < V; ++i) hist[k].v[i] = sp[i];
            }
        }
    }
#pragma unroll
    for (int tt = 0; tt < TILE; ++tt) {
        const int t = t0 + tt;
        if (t >= nt) break;
        if (tt > 0) {
            const int b = tok_seq[t];
            if (t == seq_start[b]) {                      // another sequence's portion starts here
                const float* st = state + (size_t)slots[b] * state_pitch;
#pragma unroll
                for (int k = 0; k < TAPS - 1; ++k) {
                    const float* sp = st + (size_t)(TAPS - 2 - k) * C + c;
#pragma unroll
                    for (int i = 0; i < V; ++i) hist[k].v[i] = sp[i];
                }
            }
        }
        ConvVec<T, V> own, acc;
        own.load(reinterpret_cast<const T*>(&raw[tt]));
#pragma unroll
        for (int i = 0; i < V; ++i) {
            float a = residual ? own.v[i] : 0.f;
#pragma unroll
            for (int j = 0; j < TAPS - 1; ++j) a += wr[i * TAPS + j] * hist[TAPS - 2 - j].v[i];
            acc.v[i] = a + wr[i * TAPS + TAPS - 1] * own.v[i];
        }
        acc.store(y + (size_t)t * ldy + c);
#pragma unroll
        for (int k = TAPS - 2; k > 0; --k) hist[k] = hist[k - 1];
        hist[0] = own;
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
        const uintptr_t in_al = 4 * sizeof(T);                                                                        \
        const bool vec = d % 4 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)d1 % in_al == 0 &&                        \
                         (uintptr_t)d2 % in_al == 0 && (uintptr_t)y1 % in_al == 0 && (uintptr_t)y2 % in_al == 0 &&    \
                         ld1 % 4 == 0 && ld2 % 4 == 0 && (uintptr_t)w1 % 16 == 0 && (uintptr_t)w2 % 16 == 0;          \
        if (vec)                                                                                                      \
            TB_LAUNCH((pair_add_rmsnorm_vec_kernel<T>), n_out, 256, (size_t)d * 4, s, x, (const T*)d1, (const T*)d2,  \
                      rows, w1, (T*)y1, ld1, w2, (T*)y2, ld2, eps, d);                                                \
        else                                                                                                          \
            TB_LAUNCH((pair_add_rmsnorm_kernel<T>), n_out, 256, (size_t)d * 4, s, x, (const T*)d1, (const T*)d2, rows,\
                      w1, (T*)y1, ld1, w2, (T*)y2, ld2, eps, d);                                                      \
        return tb_last_error();                                                                                       \
    }                                                                                                                 \
    int tb_causal_conv_##SFX(const void* u, int ldu, const float* w, float* state, long long state_pitch, void* y,    \
                             int ldy, const int* tok_seq, const int* seq_start, const int* slots, int nt, int B,      \
                             int C, int taps, int residual, int decode, cudaStream_t s) {                             \
        if (nt < 0 || B <= 0 || C <= 0 || taps < 1 || taps > 16 || ldu < C || ldy < C) return TB_ERR_ARG;             \
        if (taps > 1 && (!state || state_pitch < (long long)(taps - 1) * C)) return TB_ERR_ARG;                       \
        if (nt == 0) return 0;                                                                                        \
        constexpr int V = 16 / sizeof(T);                                                                             \
        const bool vec = C % V == 0 && ldu % V == 0 && ldy % V == 0 && (uintptr_t)u % 16 == 0 && (uintptr_t)y % 16 == 0; \
        constexpr int TILE = 8;                                                                                       \
        const bool tiled = vec && !decode && nt >= 8 * TILE && taps >= 2 && taps <= 4 && (uintptr_t)w % 16 == 0;      \
        if (tiled) {                                                                                                  \
            const dim3 grid((nt + TILE - 1) / TILE, (C / V + 63) / 64);                                               \
            if (taps == 2)                                                                                            \
                TB_LAUNCH((causal_conv_tile_kernel<T, V, 2, TILE>), grid, 64, 0, s, (const T*)u, ldu, w, state,      \
                          state_pitch, (T*)y, ldy, tok_seq, seq_start, slots, nt, C, residual);                       \
            else if (taps == 3)                                                                                       \
                TB_LAUNCH((causal_conv_tile_kernel<T, V, 3, TILE>), grid, 64, 0, s, (const T*)u, ldu, w, state,      \
                          state_pitch, (T*)y, ldy, tok_seq, seq_start, slots, nt, C, residual);                       \
            else                                                                                                      \
                TB_LAUNCH((causal_conv_tile_kernel<T, V, 4, TILE>), grid, 64, 0, s, (const T*)u, ldu, w, state,      \
                          state_pitch, (T*)y, ldy, tok_seq, seq_start, slots, nt, C, residual);                       \
        } else if (vec) {                                                                                             \
            const dim3 grid(nt, (C / V + 127) / 128);                                                                 \
            TB_LAUNCH((causal_conv_kernel<T, V>), grid, 128, 0, s, (const T*)u, ldu, w, state, state_pitch, (T*)y,    \
                      ldy, tok_seq, seq_start, slots, nt, C, taps, residual, decode ? 1 : 0);                         \
        } else {                                                                                                      \
            const dim3 grid(nt, (C + 127) / 128);                                                                     \
            TB_LAUNCH((causal_conv_kernel<T, 1>), grid, 128, 0, s, (const T*)u, ldu, w, state, state_pitch, (T*)y,    \
                      ldy, tok_seq, seq_start, slots, nt, C, taps, residual, decode ? 1 : 0);                         \
        }                                                                                                             \
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
