// Layer norm (mean taken off, weight and bias) fused with the residual sum, and, for blocks that norm what their
// parts produce, with the norm of that output as well.  Row r = rows ? rows[i] : i of the float stream x:
//
//   u    = delta(r)                 a part's output; or sum_j topk_w[r, j] * wy[pair_row[r, j]] (experts' rows,
//                                   unsummed; topk_w null: every weight is one); or nothing
//   u   <- N(u; post_w, post_b, post_eps, post_center)          when post_w is given
//   v    = x[r] + u                 float;  written back to x[r] when rows is null and there was a u
//   y[i] = N(v; w, b, eps, center)  one rounding to T;  w null: y[i] = v;  y null: nothing
//
//   N(a; w, b, eps, center) = (a - m) / sqrt(mean((a - m)^2) + eps) * w + b,   m = center ? mean(a) : 0,  b may be null
//
// The variance is the mean of the squared deviations from the mean that was taken first (two passes over the row,
// which lives in shared memory as floats between them).  One block per row.
#include "common.cuh"

struct LayerNormArgs {
    float* x;
    const void* delta;
    const void* wy;
    const int* pair_row;
    const float* topk_w;
    int k;
    const float* post_w;
    const float* post_b;
    float post_eps;
    int post_center;
    const int* rows;
    const float* w;
    const float* b;
    float eps;
    int center;
    void* y;
    int d;
};

// mean (or zero) and 1 / sqrt(var + eps) of the row in shared memory
__device__ __forceinline__ void ln_stats(const float* row, int d, bool center, float eps, float* red, float& mean,
                                         float& rstd) {
    mean = 0.f;
    if (center) {
        float s = 0.f;
        for (int c = threadIdx.x; c < d; c += blockDim.x) s += row[c];
        mean = block_sum(s, red) / (float)d;
    }
    float ss = 0.f;
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
        const float a = row[c] - mean;
        ss += a * a;
    }
    rstd = 1.0f / sqrtf(block_sum(ss, red) / (float)d + eps);
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(256) post_add_layernorm_kernel(const LayerNormArgs a) {
    pdl_sync();
    extern __shared__ __align__(16) float ln_row[];     // [d]
    __shared__ float red[33];
    const int i = blockIdx.x, d = a.d;
    const int r = a.rows ? a.rows[i] : i;
    float* xr = a.x + (size_t)r * d;
    const T* dr = a.delta ? static_cast<const T*>(a.delta) + (size_t)r * d : nullptr;
    const T* wy = static_cast<const T*>(a.wy);
    const bool has_u = dr != nullptr || wy != nullptr;
    constexpr int W = VEC ? 4 : 1;
    if (has_u) {
        for (int c = threadIdx.x * W; c < d; c += blockDim.x * W) {
            float u[W];
#pragma unroll
            for (int e = 0; e < W; ++e) u[e] = 0.f;
            if (dr) {
#pragma unroll
                for (int e = 0; e < W; ++e) u[e] = ldf(dr + c + e);
            } else {
                for (int j = 0; j < a.k; ++j) {
                    const float wj = a.topk_w ? a.topk_w[(size_t)r * a.k + j] : 1.f;
                    const T* src = wy + (size_t)a.pair_row[(size_t)r * a.k + j] * d + c;
#pragma unroll
                    for (int e = 0; e < W; ++e) u[e] += wj * ldf(src + e);
                }
            }
#pragma unroll
            for (int e = 0; e < W; ++e) ln_row[c + e] = u[e];
        }
        float mean = 0.f, rstd = 1.f;
        if (a.post_w) {
            __syncthreads();
            ln_stats(ln_row, d, a.post_center != 0, a.post_eps, red, mean, rstd);
        }
        // each thread goes on with the entries it wrote itself
        for (int c = threadIdx.x * W; c < d; c += blockDim.x * W) {
#pragma unroll
            for (int e = 0; e < W; ++e) {
                float u = ln_row[c + e];
                if (a.post_w) u = (u - mean) * rstd * a.post_w[c + e] + (a.post_b ? a.post_b[c + e] : 0.f);
                const float v = xr[c + e] + u;
                if (!a.rows) xr[c + e] = v;
                ln_row[c + e] = v;
            }
        }
    } else {
        if (!a.y) return;
        for (int c = threadIdx.x * W; c < d; c += blockDim.x * W) {
#pragma unroll
            for (int e = 0; e < W; ++e) ln_row[c + e] = xr[c + e];
        }
    }
    if (!a.y) return;
    T* yr = static_cast<T*>(a.y) + (size_t)i * d;
    if (!a.w) {
        for (int c = threadIdx.x * W; c < d; c += blockDim.x * W) {
#pragma unroll
            for (int e = 0; e < W; ++e) stf(yr + c + e, ln_row[c + e]);
        }
        return;
    }
    __syncthreads();
    float mean, rstd;
    ln_stats(ln_row, d, a.center != 0, a.eps, red, mean, rstd);
    for (int c = threadIdx.x * W; c < d; c += blockDim.x * W) {
#pragma unroll
        for (int e = 0; e < W; ++e)
            stf(yr + c + e, (ln_row[c + e] - mean) * rstd * a.w[c + e] + (a.b ? a.b[c + e] : 0.f));
    }
}

template <typename T>
static int post_add_layernorm_launch(const LayerNormArgs& a, int n_out, cudaStream_t s) {
    if (n_out < 0 || a.d <= 0 || !a.x) return TB_ERR_ARG;
    if (a.delta && a.wy) return TB_ERR_ARG;
    if (a.wy && (!a.pair_row || a.k <= 0)) return TB_ERR_ARG;
    if (a.post_w && !a.delta && !a.wy) return TB_ERR_ARG;
    if ((a.b && !a.w) || (a.post_b && !a.post_w) || (a.w && !a.y)) return TB_ERR_ARG;
    const size_t smem = (size_t)a.d * sizeof(float);
    if (smem > 160 * 1024) return TB_ERR_UNSUPPORTED;
    if (n_out == 0) return 0;
    static bool raised = false;
    if (smem > 48 * 1024 && !raised) {
        tb_note_error(cudaFuncSetAttribute(post_add_layernorm_kernel<T, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           160 * 1024));
        tb_note_error(cudaFuncSetAttribute(post_add_layernorm_kernel<T, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           160 * 1024));
        raised = true;
    }
    if (a.d % 4 == 0)
        TB_LAUNCH((post_add_layernorm_kernel<T, true>), n_out, 256, smem, s, a);
    else
        TB_LAUNCH((post_add_layernorm_kernel<T, false>), n_out, 256, smem, s, a);
    return tb_last_error();
}

extern "C" {
#define TB_LAYERNORM(SFX, T)                                                                                          \
    int tb_post_add_layernorm_##SFX(float* x, const void* delta, const void* wy, const int* pair_row,                 \
                                    const float* topk_w, int k, const float* post_w, const float* post_b,             \
                                    float post_eps, int post_center, const int* rows, const float* w,                 \
                                    const float* b, float eps, int center, void* y, int n_out, int d,                 \
                                    cudaStream_t s) {                                                                 \
        LayerNormArgs a{x, delta, wy, pair_row, topk_w, k, post_w, post_b, post_eps, post_center, rows, w, b, eps,    \
                        center, y, d};                                                                                \
        return post_add_layernorm_launch<T>(a, n_out, s);                                                             \
    }
TB_LAYERNORM(f32, float)
TB_LAYERNORM(bf16, __nv_bfloat16)
}

#include "tape.h"
TB_TAPE_REGISTER(tb_post_add_layernorm_f32)
TB_TAPE_REGISTER(tb_post_add_layernorm_bf16)
