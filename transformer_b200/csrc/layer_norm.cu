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
// The variance is the mean of the squared deviations from the mean: every thread takes the mean and the squared
// deviations of its own entries in two passes, and the threads' statistics are joined exactly (one reduction over
// the block instead of two).  One block per row.  Widths that are multiples of eight up to 8192 with 16-byte aligned
// addresses keep the row in registers and move 16 bytes at a time; any other width keeps it in shared memory as floats.
//
// A router may ride along (the form with the row in registers, up to 256 rows): the logits of the row just written,
// as stored, against the router's matrix, a warp per output, and the choice by the rules of router_pick.cuh.
#include "common.cuh"
#include "router_pick.cuh"

struct LayerNormTail {
    const void* w;          // [E, d] router matrix in the activations' type, or null: none
    const float* bias;      // the scored rule's correction, or null
    int* idx;               // [rows, k]
    float* wts;             // [rows, k]
    int E, k, rule;         // rule: RouterRule::scored
};

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
    LayerNormTail tail;
};

// Two partial statistics (count, mean, sum of squared deviations from that mean) joined into one: exact however
// the entries were dealt out, and as accurate as taking the mean first and the deviations in a second pass.
struct LnStat {
    float n, mean, m2;
};
__device__ __forceinline__ LnStat ln_join(const LnStat& a, const LnStat& b) {
    LnStat r;
    r.n = a.n + b.n;
    if (r.n == 0.f) {
        r.mean = r.m2 = 0.f;
        return r;
    }
    const float dm = b.mean - a.mean, fb = b.n / r.n;
    r.mean = a.mean + dm * fb;
    r.m2 = a.m2 + b.m2 + dm * dm * a.n * fb;
    return r;
}
__device__ __forceinline__ LnStat ln_block_join(LnStat v, float* red) {      // red: 3 * 32 + 3 floats
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        LnStat w{__shfl_xor_sync(0xffffffffu, v.n, o), __shfl_xor_sync(0xffffffffu, v.mean, o),
                 __shfl_xor_sync(0xffffffffu, v.m2, o)};
        v = ln_join(v, w);
    }
    __syncthreads();
    if (lane == 0) {
        red[3 * warp] = v.n;
        red[3 * warp + 1] = v.mean;
        red[3 * warp + 2] = v.m2;
    }
    __syncthreads();
    if (warp == 0) {
        LnStat t{0.f, 0.f, 0.f};
        if (lane < nw) t = LnStat{red[3 * lane], red[3 * lane + 1], red[3 * lane + 2]};
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            LnStat w{__shfl_xor_sync(0xffffffffu, t.n, o), __shfl_xor_sync(0xffffffffu, t.mean, o),
                     __shfl_xor_sync(0xffffffffu, t.m2, o)};
            t = ln_join(t, w);
        }
        if (lane == 0) {
            red[96] = t.n;
            red[97] = t.mean;
            red[98] = t.m2;
        }
    }
    __syncthreads();
    return LnStat{red[96], red[97], red[98]};
}

// mean (or zero) and 1 / sqrt(var + eps) of the row in shared memory; every thread takes the entries it wrote itself
template <int W>
__device__ __forceinline__ void ln_stats(const float* row, int d, bool center, float eps, float* red, float& mean,
                                         float& rstd) {
    float s = 0.f, cnt = 0.f;
    for (int c = threadIdx.x * W; c < d; c += blockDim.x * W) {
#pragma unroll
        for (int e = 0; e < W; ++e) s += center ? row[c + e] : row[c + e] * row[c + e];
        cnt += (float)W;
    }
    if (!center) {
        mean = 0.f;
        rstd = 1.0f / sqrtf(block_sum(s, red) / (float)d + eps);
        return;
    }
    LnStat mine{cnt, cnt > 0.f ? s / cnt : 0.f, 0.f};
    for (int c = threadIdx.x * W; c < d; c += blockDim.x * W) {
#pragma unroll
        for (int e = 0; e < W; ++e) {
            const float a = row[c + e] - mine.mean;
            mine.m2 += a * a;
        }
    }
    const LnStat all = ln_block_join(mine, red);
    mean = all.mean;
    rstd = 1.0f / sqrtf(all.m2 / (float)d + eps);
}

// W consecutive entries as floats, one 16-byte access per 8 bfloat16 or 4 floats where VEC says the layout allows it
template <typename T, bool VEC> __device__ __forceinline__ void ln_load(const T* p, float (&f)[VEC ? 8 : 1]) {
    if constexpr (VEC) load8(p, f);
    else f[0] = ldf(p);
}
template <typename T, bool VEC> __device__ __forceinline__ void ln_store(T* p, const float (&f)[VEC ? 8 : 1]) {
    if constexpr (VEC) store8(p, f);
    else stf(p, f[0]);
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(256) post_add_layernorm_kernel(const LayerNormArgs a) {
    pdl_sync();
    extern __shared__ __align__(16) float ln_row[];     // [d]
    __shared__ float red[99];
    const int i = blockIdx.x, d = a.d;
    const int r = a.rows ? a.rows[i] : i;
    float* xr = a.x + (size_t)r * d;
    const T* dr = a.delta ? static_cast<const T*>(a.delta) + (size_t)r * d : nullptr;
    const T* wy = static_cast<const T*>(a.wy);
    const bool has_u = dr != nullptr || wy != nullptr;
    constexpr int W = VEC ? 8 : 1;
    if (has_u) {
        for (int c = threadIdx.x * W; c < d; c += blockDim.x * W) {
            float u[W];
            if (dr) {
                ln_load<T, VEC>(dr + c, u);
            } else {
#pragma unroll
                for (int e = 0; e < W; ++e) u[e] = 0.f;
                for (int j = 0; j < a.k; ++j) {
                    const float wj = a.topk_w ? a.topk_w[(size_t)r * a.k + j] : 1.f;
                    float t[W];
                    ln_load<T, VEC>(wy + (size_t)a.pair_row[(size_t)r * a.k + j] * d + c, t);
#pragma unroll
                    for (int e = 0; e < W; ++e) u[e] += wj * t[e];
                }
            }
#pragma unroll
            for (int e = 0; e < W; ++e) ln_row[c + e] = u[e];
        }
        float mean = 0.f, rstd = 1.f;
        if (a.post_w) ln_stats<W>(ln_row, d, a.post_center != 0, a.post_eps, red, mean, rstd);
        // each thread goes on with the entries it wrote itself
        for (int c = threadIdx.x * W; c < d; c += blockDim.x * W) {
            float xv[W], pw[W], pb[W];
            ln_load<float, VEC>(xr + c, xv);
            if (a.post_w) ln_load<float, VEC>(a.post_w + c, pw);
            if (a.post_b) ln_load<float, VEC>(a.post_b + c, pb);
#pragma unroll
            for (int e = 0; e < W; ++e) {
                float u = ln_row[c + e];
                if (a.post_w) u = (u - mean) * rstd * pw[e] + (a.post_b ? pb[e] : 0.f);
                xv[e] += u;
                ln_row[c + e] = xv[e];
            }
            if (!a.rows) ln_store<float, VEC>(xr + c, xv);
        }
    } else {
        if (!a.y) return;
        for (int c = threadIdx.x * W; c < d; c += blockDim.x * W) {
            float xv[W];
            ln_load<float, VEC>(xr + c, xv);
#pragma unroll
            for (int e = 0; e < W; ++e) ln_row[c + e] = xv[e];
        }
    }
    if (!a.y) return;
    T* yr = static_cast<T*>(a.y) + (size_t)i * d;
    float mean = 0.f, rstd = 1.f;
    if (a.w) ln_stats<W>(ln_row, d, a.center != 0, a.eps, red, mean, rstd);
    for (int c = threadIdx.x * W; c < d; c += blockDim.x * W) {
        float o[W], w[W], b[W];
        if (a.w) ln_load<float, VEC>(a.w + c, w);
        if (a.b) ln_load<float, VEC>(a.b + c, b);
#pragma unroll
        for (int e = 0; e < W; ++e) {
            o[e] = ln_row[c + e];       // without weights: the sum itself, rounded once
            if (a.w) o[e] = (o[e] - mean) * rstd * w[e] + (a.b ? b[e] : 0.f);
        }
        ln_store<T, VEC>(yr + c, o);
    }
}

// The same with the row in registers: NCH pieces of eight entries a thread (widths that are multiples of eight up to
// 2048 * NCH, 16-byte aligned addresses).  Nothing goes through shared memory but the reductions.
template <int NCH>
__device__ __forceinline__ void ln_stats_reg(const float (&v)[NCH][8], int d, bool center, float eps, float* red,
                                             float& mean, float& rstd) {
    float s = 0.f, cnt = 0.f;
#pragma unroll
    for (int j = 0; j < NCH; ++j) {
        if ((int)(threadIdx.x + j * 256) * 8 < d) {
#pragma unroll
            for (int e = 0; e < 8; ++e) s += center ? v[j][e] : v[j][e] * v[j][e];
            cnt += 8.f;
        }
    }
    if (!center) {
        mean = 0.f;
        rstd = 1.0f / sqrtf(block_sum(s, red) / (float)d + eps);
        return;
    }
    LnStat mine{cnt, cnt > 0.f ? s / cnt : 0.f, 0.f};
#pragma unroll
    for (int j = 0; j < NCH; ++j) {
        if ((int)(threadIdx.x + j * 256) * 8 < d) {
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float a = v[j][e] - mine.mean;
                mine.m2 += a * a;
            }
        }
    }
    const LnStat all = ln_block_join(mine, red);
    mean = all.mean;
    rstd = 1.0f / sqrtf(all.m2 / (float)d + eps);
}

template <typename T, int NCH, bool TAIL>
__global__ void __launch_bounds__(256) post_add_layernorm_reg_kernel(const LayerNormArgs a) {
    pdl_sync();
    extern __shared__ __align__(16) unsigned char ln_tail_smem[];      // TAIL: the row as T [d], then logits [E] (or 2 E)
    __shared__ float red[99];
    const int i = blockIdx.x, d = a.d;
    const int r = a.rows ? a.rows[i] : i;
    float* xr = a.x + (size_t)r * d;
    const T* dr = a.delta ? static_cast<const T*>(a.delta) + (size_t)r * d : nullptr;
    const T* wy = static_cast<const T*>(a.wy);
    const bool has_u = dr != nullptr || wy != nullptr;
    float v[NCH][8];
    if (has_u) {
#pragma unroll
        for (int j = 0; j < NCH; ++j) {
            const int c = (threadIdx.x + j * 256) * 8;
#pragma unroll
            for (int e = 0; e < 8; ++e) v[j][e] = 0.f;
            if (c >= d) continue;
            if (dr) {
                load8(dr + c, v[j]);
            } else {
                for (int q = 0; q < a.k; ++q) {
                    const float wq = a.topk_w ? a.topk_w[(size_t)r * a.k + q] : 1.f;
                    float t[8];
                    load8(wy + (size_t)a.pair_row[(size_t)r * a.k + q] * d + c, t);
#pragma unroll
                    for (int e = 0; e < 8; ++e) v[j][e] += wq * t[e];
                }
            }
        }
        float mean = 0.f, rstd = 1.f;
        if (a.post_w) ln_stats_reg<NCH>(v, d, a.post_center != 0, a.post_eps, red, mean, rstd);
#pragma unroll
        for (int j = 0; j < NCH; ++j) {
            const int c = (threadIdx.x + j * 256) * 8;
            if (c >= d) continue;
            float xv[8], pw[8], pb[8];
            load8(xr + c, xv);
            if (a.post_w) load8(a.post_w + c, pw);
            if (a.post_b) load8(a.post_b + c, pb);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                float u = v[j][e];
                if (a.post_w) u = (u - mean) * rstd * pw[e] + (a.post_b ? pb[e] : 0.f);
                v[j][e] = xv[e] + u;
            }
            if (!a.rows) store8(xr + c, v[j]);
        }
    } else {
        if (!a.y) return;
#pragma unroll
        for (int j = 0; j < NCH; ++j) {
            const int c = (threadIdx.x + j * 256) * 8;
#pragma unroll
            for (int e = 0; e < 8; ++e) v[j][e] = 0.f;
            if (c < d) load8(xr + c, v[j]);
        }
    }
    if (!a.y) return;
    T* yr = static_cast<T*>(a.y) + (size_t)i * d;
    float mean = 0.f, rstd = 1.f;
    if (a.w) ln_stats_reg<NCH>(v, d, a.center != 0, a.eps, red, mean, rstd);
#pragma unroll
    for (int j = 0; j < NCH; ++j) {
        const int c = (threadIdx.x + j * 256) * 8;
        if (c >= d) continue;
        float o[8], w[8], b[8];
        if (a.w) load8(a.w + c, w);
        if (a.b) load8(a.b + c, b);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            o[e] = v[j][e];             // without weights: the sum itself, rounded once
            if (a.w) o[e] = (o[e] - mean) * rstd * w[e] + (a.b ? b[e] : 0.f);
        }
        store8(yr + c, o);
        if (TAIL) store8(reinterpret_cast<T*>(ln_tail_smem) + c, o);      // what the router reads: the row as stored
    }
    if (!TAIL) return;
    __syncthreads();
    constexpr int EPL = Vec16<T>::N;
    const T* ys = reinterpret_cast<const T*>(ln_tail_smem);
    float* lg = reinterpret_cast<float*>(ln_tail_smem + (size_t)d * sizeof(T));
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const LayerNormTail& t = a.tail;
    for (int e = warp; e < t.E; e += 8) {
        const T* we = static_cast<const T*>(t.w) + (size_t)e * d;
        float acc = 0.f;
        for (int c = lane * EPL; c < d; c += 32 * EPL) {
            float xf[EPL], wf[EPL];
            Vec16<T>::load(ys + c, xf);
            Vec16<T>::load(we + c, wf);
#pragma unroll
            for (int q = 0; q < EPL; ++q) acc += xf[q] * wf[q];
        }
        acc = warp_sum(acc);
        if (lane == 0) lg[e] = acc;
    }
    __syncthreads();
    if (warp == 0) {
        if (t.rule == 1)
            router_pick_scored(lg, lg + t.E, t.bias, t.idx + (size_t)i * t.k, t.wts + (size_t)i * t.k, t.E, t.k, lane);
        else
            router_pick(lg, t.idx + (size_t)i * t.k, t.wts + (size_t)i * t.k, t.E, t.k, lane, t.rule == 2);
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
    const uintptr_t all = (uintptr_t)a.x | (uintptr_t)a.delta | (uintptr_t)a.wy | (uintptr_t)a.post_w |
                          (uintptr_t)a.post_b | (uintptr_t)a.w | (uintptr_t)a.b | (uintptr_t)a.y;
    const bool vec = a.d % 8 == 0 && (all & 15) == 0;
    if (a.tail.w) {
        // the form that also routes: a few rows, the row in registers, the row as stored and the logits in 40 KB
        const LayerNormTail& t = a.tail;
        if (t.E <= 0 || t.k <= 0 || t.k > t.E || !t.idx || !t.wts || !a.y) return TB_ERR_ARG;
        const size_t tsm = (size_t)a.d * sizeof(T) + (size_t)t.E * sizeof(float) * (t.rule == 1 ? 2 : 1);
        if (!vec || a.d > 8192 || n_out > 256 || tsm > 40 * 1024 || ((uintptr_t)t.w & 15)) return TB_ERR_UNSUPPORTED;
        if (a.d <= 2048) TB_LAUNCH((post_add_layernorm_reg_kernel<T, 1, true>), n_out, 256, tsm, s, a);
        else if (a.d <= 4096) TB_LAUNCH((post_add_layernorm_reg_kernel<T, 2, true>), n_out, 256, tsm, s, a);
        else TB_LAUNCH((post_add_layernorm_reg_kernel<T, 4, true>), n_out, 256, tsm, s, a);
        return tb_last_error();
    }
    if (vec && a.d <= 8192) {       // the row in registers
        if (a.d <= 2048) TB_LAUNCH((post_add_layernorm_reg_kernel<T, 1, false>), n_out, 256, 0, s, a);
        else if (a.d <= 4096) TB_LAUNCH((post_add_layernorm_reg_kernel<T, 2, false>), n_out, 256, 0, s, a);
        else TB_LAUNCH((post_add_layernorm_reg_kernel<T, 4, false>), n_out, 256, 0, s, a);
        return tb_last_error();
    }
    static bool raised = false;
    if (smem > 48 * 1024 && !raised) {
        tb_note_error(cudaFuncSetAttribute(post_add_layernorm_kernel<T, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           160 * 1024));
        tb_note_error(cudaFuncSetAttribute(post_add_layernorm_kernel<T, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           160 * 1024));
        raised = true;
    }
    if (vec)
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
                        center, y, d, LayerNormTail{nullptr, nullptr, nullptr, nullptr, 0, 0, 0}};                    \
        return post_add_layernorm_launch<T>(a, n_out, s);                                                             \
    }                                                                                                                 \
    /* The same with a router riding along: router_w [E, d]; rule 0: the route_k largest logits with a softmax over   \
       the kept, 1: softmax over all and score + bias, 2: sigmoids as they are.  TB_ERR_UNSUPPORTED (nothing done)    \
       for more than 256 rows, widths or addresses the register form does not take. */                               \
    int tb_post_add_layernorm_router_##SFX(float* x, const void* delta, const void* wy, const int* pair_row,          \
                                           const float* topk_w, int k, const float* post_w, const float* post_b,      \
                                           float post_eps, int post_center, const int* rows, const float* w,          \
                                           const float* b, float eps, int center, void* y, int n_out, int d,          \
                                           const void* router_w, const float* route_bias, int* route_idx,             \
                                           float* route_w, int E, int route_k, int rule, cudaStream_t s) {            \
        if (!router_w || rule < 0 || rule > 2) return TB_ERR_ARG;                                                     \
        LayerNormArgs a{x, delta, wy, pair_row, topk_w, k, post_w, post_b, post_eps, post_center, rows, w, b, eps,    \
                        center, y, d, LayerNormTail{router_w, route_bias, route_idx, route_w, E, route_k, rule}};     \
        return post_add_layernorm_launch<T>(a, n_out, s);                                                             \
    }
TB_LAYERNORM(f32, float)
TB_LAYERNORM(bf16, __nv_bfloat16)
}

#include "tape.h"
TB_TAPE_REGISTER(tb_post_add_layernorm_f32)
TB_TAPE_REGISTER(tb_post_add_layernorm_bf16)
TB_TAPE_REGISTER(tb_post_add_layernorm_router_f32)
TB_TAPE_REGISTER(tb_post_add_layernorm_router_bf16)
