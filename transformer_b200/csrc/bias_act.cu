// Biases of a feed-forward whose projections have them, applied to the products' results; and the squared relu of
// a feed-forward without a gate.
//
//   h[t, c] = silu(gu[t, c] + b[c]) * (gu[t, di + c] + b[di + c])        the (gate, up) pair with its biases
// Biases are float; the sums and the activation are float, one rounding at the store.
// h may have more columns than di (ldh > di): column di is then set to one and the rest to zero, so that a down
// projection whose weight carries its bias as column di adds it inside its own sum.
#include "common.cuh"

template <typename T>
__global__ void __launch_bounds__(256) bias_glu_kernel(const T* __restrict__ gu, const float* __restrict__ bias,
                                                       T* __restrict__ h, long long n, int di, int ldh) {
    pdl_sync();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / ldh;
        const int c = (int)(i - t * ldh);
        if (c >= di) {
            stf(h + i, c == di ? 1.f : 0.f);
            continue;
        }
        const float g = ldf(gu + t * 2 * di + c) + bias[c];
        const float u = ldf(gu + t * 2 * di + di + c) + bias[di + c];
        stf(h + i, g / (1.0f + expf(-g)) * u);
    }
}

// The same, eight entries per thread with 16-byte accesses (di and ldh multiples of 8).
template <typename T>
__global__ void __launch_bounds__(256) bias_glu_vec_kernel(const T* __restrict__ gu, const float* __restrict__ bias,
                                                           T* __restrict__ h, long long n8, int di, int ldh) {
    pdl_sync();
    const int per_row = ldh / 8;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / per_row;
        const int c = (int)(i - t * per_row) * 8;
        float o[8];
        if (c >= di) {
#pragma unroll
            for (int e = 0; e < 8; ++e) o[e] = (c + e == di) ? 1.f : 0.f;
        } else {
            float g[8], u[8], bg[8], bu[8];
            load8(gu + t * 2 * di + c, g);
            load8(gu + t * 2 * di + di + c, u);
            load8(bias + c, bg);
            load8(bias + di + c, bu);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float a = g[e] + bg[e];
                o[e] = a / (1.0f + expf(-a)) * (u[e] + bu[e]);
            }
        }
        store8(h + t * ldh + c, o);
    }
}

// h[i] = max(h[i], 0)^2 in place: the activation of a feed-forward without a gate, on its first product's result
template <typename T>
__global__ void __launch_bounds__(256) relu2_kernel(T* __restrict__ h, long long n) {
    pdl_sync();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const float v = fmaxf(ldf(h + i), 0.f);
        stf(h + i, v * v);
    }
}
template <typename T>
__global__ void __launch_bounds__(256) relu2_vec_kernel(T* __restrict__ h, long long n8) {
    pdl_sync();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
        float v[8];
        load8(h + i * 8, v);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            v[e] = fmaxf(v[e], 0.f);
            v[e] *= v[e];
        }
        store8(h + i * 8, v);
    }
}

static int grid_for(long long n) {
    const long long blocks = (n + 255) / 256;
    return (int)(blocks > 8192 ? 8192 : blocks);
}

extern "C" {
#define TB_BIAS(SFX, T)                                                                                               \
    int tb_bias_glu_##SFX(const void* gu, const float* bias, void* h, int nt, int di, int ldh, cudaStream_t s) {      \
        if (nt < 0 || di <= 0 || ldh < di || !bias) return TB_ERR_ARG;                                                \
        if (nt == 0) return 0;                                                                                        \
        const long long n = (long long)nt * ldh;                                                                      \
        if (di % 8 == 0 && ldh % 8 == 0 && (((uintptr_t)gu | (uintptr_t)h | (uintptr_t)bias) & 15) == 0)              \
            TB_LAUNCH((bias_glu_vec_kernel<T>), grid_for(n / 8), 256, 0, s, (const T*)gu, bias, (T*)h, n / 8, di, ldh); \
        else                                                                                                          \
            TB_LAUNCH((bias_glu_kernel<T>), grid_for(n), 256, 0, s, (const T*)gu, bias, (T*)h, n, di, ldh);           \
        return tb_last_error();                                                                                       \
    }
TB_BIAS(f32, float)
TB_BIAS(bf16, __nv_bfloat16)
#define TB_RELU2(SFX, T)                                                                                              \
    int tb_relu2_##SFX(void* h, long long n, cudaStream_t s) {                                                        \
        if (n < 0 || (n && !h)) return TB_ERR_ARG;                                                                    \
        if (n == 0) return 0;                                                                                         \
        if (n % 8 == 0 && ((uintptr_t)h & 15) == 0)                                                                   \
            TB_LAUNCH((relu2_vec_kernel<T>), grid_for(n / 8), 256, 0, s, (T*)h, n / 8);                               \
        else                                                                                                          \
            TB_LAUNCH((relu2_kernel<T>), grid_for(n), 256, 0, s, (T*)h, n);                                           \
        return tb_last_error();                                                                                       \
    }
TB_RELU2(f32, float)
TB_RELU2(bf16, __nv_bfloat16)
}

#include "tape.h"
TB_TAPE_REGISTER(tb_bias_glu_f32)
TB_TAPE_REGISTER(tb_bias_glu_bf16)
TB_TAPE_REGISTER(tb_relu2_f32)
TB_TAPE_REGISTER(tb_relu2_bf16)
