// A matrix memory with exponential gates (the mLSTM cell of xLSTM), token by token, state in float.
//
// Per head, with a state S [dim, vdim], n [dim] and a running maximum m (all zero when a sequence starts):
//
//   i_t = cap * tanh((zi_t + bi) / cap)                       log of the input gate
//   f_t = logsigmoid(cap * tanh((zf_t + bf) / cap))           log of the forget gate
//   m_t = max(f_t + m_{t-1}, i_t)
//   S_t = exp(f_t + m_{t-1} - m_t) S_{t-1} + exp(i_t - m_t) k_t v_t^T          n_t alike with k_t alone
//   o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)                      q scaled by dim^-1/2
//
// zi, zf are the gates' projections (float, computed by a product before this kernel), q, k, v the step's
// projections in the activation type.  Gates, decays, the state and the division are float on both paths.
//
// Work split: one block = one sequence x one head x 32 columns of v.  Lane = column, the block's 8 warps split
// the rows of S (warp w owns rows w, w + 8, ...: RPW registers per thread), so a block holds dim x 32 of the
// state in registers for all the tokens its sequence brings to the step, reads it once and writes it once.
// Every block keeps n and m for itself (they are cheap and every block needs them): the state holds one copy
// per block of columns, so that no block reads what another has already moved on.
//
// State of one (slot, head):  S [dim][vdim], then for each block of 32 columns: n [dim], m.
#include "common.cuh"

#define ML_WARPS 8
#define ML_COLS 32
#define ML_DENOM_FLOOR 1e-6f

struct MlstmArgs {
    const void* qkv;        // [nt, ld]: q heads | k heads | v heads (| anything else)
    const float* gates;     // [nt, 2 H]: zi of every head, then zf
    const float* bias;      // [2 H]
    float* state;           // [slots, H, state_size]
    float* out;             // [nt, H * vdim] unnormalized o
    const int* seq_start;   // [B + 1]
    const int* slots;       // [B]
    int ld, H, dim, vdim;
    float cap, qscale;
};

__device__ __forceinline__ float log_sigmoid(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

template <typename T, int RPW>
__global__ void __launch_bounds__(ML_WARPS * 32) mlstm_scan_kernel(const MlstmArgs a) {
    pdl_sync();
    constexpr int NQ = RPW * ML_WARPS / 32 > 0 ? RPW * ML_WARPS / 32 : 1;   // n entries per lane (dim <= 32 NQ)
    __shared__ float qk[2][2][RPW * ML_WARPS];      // [parity][q | k][dim]
    __shared__ float red[2][ML_WARPS][ML_COLS];
    const int b = blockIdx.x, h = blockIdx.y, cb = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, tid = threadIdx.x;
    const int dim = a.dim, vdim = a.vdim, H = a.H;
    const int col = cb * ML_COLS + lane;
    const bool has_col = col < vdim;
    const int t0 = a.seq_start[b], t1 = a.seq_start[b + 1];
    if (t0 >= t1) return;
    const int col_blocks = (vdim + ML_COLS - 1) / ML_COLS;
    const size_t state_size = (size_t)dim * vdim + (size_t)col_blocks * (dim + 1);
    float* S = a.state + ((size_t)a.slots[b] * H + h) * state_size;
    float* nvec = S + (size_t)dim * vdim + (size_t)cb * (dim + 1);
    float s[RPW], nq[NQ];
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
        const int r = warp + ML_WARPS * i;
        s[i] = (r < dim && has_col) ? S[(size_t)r * vdim + col] : 0.f;
    }
#pragma unroll
    for (int j = 0; j < NQ; ++j) {
        const int r = lane + 32 * j;
        nq[j] = r < dim ? nvec[r] : 0.f;
    }
    float m = nvec[dim];
    const T* X = static_cast<const T*>(a.qkv);
    const float bi = a.bias[h], bf = a.bias[H + h], cap = a.cap, inv_cap = 1.0f / a.cap;
    // the next token's values are asked for while this one is computed
    auto fetch = [&](int t, float& q_, float& k_, float& v_, float& zi_, float& zf_) {
        const T* row = X + (size_t)t * a.ld;
        q_ = tid < dim ? ldf(row + (size_t)h * dim + tid) * a.qscale : 0.f;
        k_ = tid < dim ? ldf(row + (size_t)(H + h) * dim + tid) : 0.f;
        v_ = has_col ? ldf(row + (size_t)2 * H * dim + (size_t)h * vdim + col) : 0.f;
        zi_ = a.gates[(size_t)t * 2 * H + h];
        zf_ = a.gates[(size_t)t * 2 * H + H + h];
    };
    float q_r, k_r, v_r, zi, zf;
    fetch(t0, q_r, k_r, v_r, zi, zf);
    for (int t = t0; t < t1; ++t) {
        const int par = (t - t0) & 1;
        if (tid < RPW * ML_WARPS) {
            qk[par][0][tid] = q_r;
            qk[par][1][tid] = k_r;
        }
        const float v_c = v_r, zi_c = zi, zf_c = zf;
        if (t + 1 < t1) fetch(t + 1, q_r, k_r, v_r, zi, zf);
        __syncthreads();
        const float ig = cap * tanhf((zi_c + bi) * inv_cap);
        const float fg = log_sigmoid(cap * tanhf((zf_c + bf) * inv_cap));
        const float m_new = fmaxf(fg + m, ig);
        const float keep = expf(fg + m - m_new), take = expf(ig - m_new);
        m = m_new;
        const float tv = take * v_c;
        float part = 0.f;
#pragma unroll
        for (int i = 0; i < RPW; ++i) {
            const int r = warp + ML_WARPS * i;       // rows beyond dim hold zeros in qk and stay zero
            s[i] = keep * s[i] + qk[par][1][r] * tv;
            part += s[i] * qk[par][0][r];
        }
        red[par][warp][lane] = part;
        float dot = 0.f;
        if (warp == 0) {
#pragma unroll
            for (int j = 0; j < NQ; ++j) {
                const int r = lane + 32 * j;
                if (r < RPW * ML_WARPS) {
                    nq[j] = keep * nq[j] + take * qk[par][1][r];
                    dot += nq[j] * qk[par][0][r];
                }
            }
            dot = warp_sum(dot);
        }
        __syncthreads();
        if (warp == 0 && has_col) {
            float o = 0.f;
#pragma unroll
            for (int w = 0; w < ML_WARPS; ++w) o += red[par][w][lane];
            const float den = fmaxf(fabsf(dot), expf(-m)) + ML_DENOM_FLOOR;
            a.out[(size_t)t * H * vdim + (size_t)h * vdim + col] = o / den;
        }
    }
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
        const int r = warp + ML_WARPS * i;
        if (r < dim && has_col) S[(size_t)r * vdim + col] = s[i];
    }
    if (warp == 0) {
#pragma unroll
        for (int j = 0; j < NQ; ++j) {
            const int r = lane + 32 * j;
            if (r < dim) nvec[r] = nq[j];
        }
        if (lane == 0) nvec[dim] = m;
    }
}


// ---- the same recurrence, a chunk of 64 tokens at a time -----------------------------------------------------------
// For prompts.  Inside a chunk that starts from (S', n', m') the recurrence has a closed form: with b_t the sum of the
// f up to t (inside the chunk) and M_t = max(m', max_{j<=t}(i_j - b_j)),
//
//   m_t = b_t + M_t                      g_t = e^{b_t + m' - m_t}          D_tj = e^{b_t - b_j + i_j - m_t}  (j <= t)
//   S_t^T q_t = g_t S'^T q_t + sum_j D_tj (k_j . q_t) v_j                  n_t . q_t = g_t n' . q_t + sum_j D_tj (k_j . q_t)
//   S_end = e^{b_L + m' - m_L} S' + sum_j e^{b_L - b_j + i_j - m_L} k_j v_j^T          (n_end alike)
//
// so the 64 tokens of a chunk are computed side by side and only the chunks follow one another: the scores
// C_tj = D_tj (k_j . q_t), then each token's numerator from the old state and from C, then the state's step.
// Every exponent is <= 0 by the choice of m_t; all arithmetic is float (CUDA cores), on both paths.
// One block = one sequence x one head x 32 columns of v, the state's layout is that of the kernel above.
#define MC_L 64
#define MC_THREADS 256

__device__ __forceinline__ float warp_scan_add(float v, int lane) {
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float u = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += u;
    }
    return v;
}
__device__ __forceinline__ float warp_scan_max(float v, int lane) {
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float u = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v = fmaxf(v, u);
    }
    return v;
}

template <typename T, bool FAST>
__global__ void __launch_bounds__(MC_THREADS) mlstm_chunk_kernel(const MlstmArgs a) {
    pdl_sync();
    extern __shared__ __align__(16) float mc[];
    const int dim = a.dim, vdim = a.vdim, H = a.H, dp = dim + 1;
    float* q_s = mc;                         // [64][dim + 1]
    float* k_s = q_s + MC_L * dp;            // [64][dim + 1]
    float* v_s = k_s + MC_L * dp;            // [64][32]   (a multiple of 4 floats from the start: dp * 128)
    float* C_s = v_s + MC_L * ML_COLS;       // [64][65]
    float* S_s = C_s + MC_L * (MC_L + 1);    // [dim][32]
    float* n_s = S_s + dim * ML_COLS;        // [dim]
    float* b_s = n_s + dim;                  // six arrays of 64, then two scalars
    float* ig_s = b_s + MC_L;
    float* m_s = ig_s + MC_L;
    float* g_s = m_s + MC_L;
    float* w_s = g_s + MC_L;
    float* den_s = w_s + MC_L;
    float* end_s = den_s + MC_L;             // b_L, m_L
    const int b = blockIdx.x, h = blockIdx.y, cb = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int t0 = a.seq_start[b], t1 = a.seq_start[b + 1];
    if (t0 >= t1) return;
    const int col_blocks = (vdim + ML_COLS - 1) / ML_COLS;
    const size_t state_size = (size_t)dim * vdim + (size_t)col_blocks * (dim + 1);
    float* S = a.state + ((size_t)a.slots[b] * H + h) * state_size;
    float* nvec = S + (size_t)dim * vdim + (size_t)cb * (dim + 1);
    for (int idx = tid; idx < dim * ML_COLS; idx += MC_THREADS) {
        const int r = idx / ML_COLS, col = cb * ML_COLS + idx % ML_COLS;
        S_s[idx] = col < vdim ? S[(size_t)r * vdim + col] : 0.f;
    }
    for (int r = tid; r < dim; r += MC_THREADS) n_s[r] = nvec[r];
    float m_prev = nvec[dim];
    const T* X = static_cast<const T*>(a.qkv);
    const float bi = a.bias[h], bf = a.bias[H + h], cap = a.cap, inv_cap = 1.0f / a.cap;
    const int cg = tid & 7, c4 = cg * 4, tp = tid >> 3;          // a thread's four columns; its pair of tokens / its rows
    // FAST: rows of q, k, v are fetched 16 bytes at a time, a chunk ahead of their use (registers pre_*)
    constexpr int QK_PER = FAST ? 8 : 1;                          // 64 x 256 / 8 pieces over 256 threads at most
    const int dim8 = dim / 8;
    uint4 pre_q[QK_PER], pre_k[QK_PER], pre_v;
    auto prefetch = [&](int base) {
        if (!FAST) return;
        const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
        const int left = t1 - base;
        const __nv_bfloat16* Xb = reinterpret_cast<const __nv_bfloat16*>(a.qkv);
#pragma unroll
        for (int u = 0; u < QK_PER; ++u) {
            const int idx = tid + u * MC_THREADS;
            pre_q[u] = pre_k[u] = zero;
            if (idx < MC_L * dim8) {
                const int t = idx / dim8, c = (idx - t * dim8) * 8;
                if (t < left) {
                    const __nv_bfloat16* row = Xb + (size_t)(base + t) * a.ld;
                    pre_q[u] = *reinterpret_cast<const uint4*>(row + (size_t)h * dim + c);
                    pre_k[u] = *reinterpret_cast<const uint4*>(row + (size_t)(H + h) * dim + c);
                }
            }
        }
        {
            const int t = tid >> 2, c = (tid & 3) * 8;            // 64 tokens x 32 columns = 256 pieces of 8
            pre_v = zero;
            if (t < left)
                pre_v = *reinterpret_cast<const uint4*>(Xb + (size_t)(base + t) * a.ld + (size_t)2 * H * dim +
                                                        (size_t)h * vdim + cb * ML_COLS + c);
        }
    };
    prefetch(t0);
    __syncthreads();
    for (int c0 = t0; c0 < t1; c0 += MC_L) {
        const int nc = min(MC_L, t1 - c0);
        // ---- 1. the chunk's q, k, v as floats; the gates and their scans by warp 0 ------------------------------
        if (FAST) {
            // the rows were asked for while the chunk before was computed: 16 bytes = 8 values at a time
#pragma unroll
            for (int u = 0; u < QK_PER; ++u) {
                const int idx = tid + u * MC_THREADS;
                if (idx < MC_L * dim8) {
                    const int t = idx / dim8, c = (idx - t * dim8) * 8;
                    float f[8];
                    Vec16<__nv_bfloat16>::unpack(pre_q[u], f);
#pragma unroll
                    for (int e = 0; e < 8; ++e) q_s[t * dp + c + e] = f[e] * a.qscale;
                    Vec16<__nv_bfloat16>::unpack(pre_k[u], f);
#pragma unroll
                    for (int e = 0; e < 8; ++e) k_s[t * dp + c + e] = f[e];
                }
            }
            {
                float f[8];
                Vec16<__nv_bfloat16>::unpack(pre_v, f);
#pragma unroll
                for (int e = 0; e < 8; ++e) v_s[tid * 8 + e] = f[e];
            }
        } else {
        for (int idx = tid; idx < MC_L * dim; idx += MC_THREADS) {
            const int t = idx / dim, c = idx - t * dim;
            float qv = 0.f, kv = 0.f;
            if (t < nc) {
                const T* row = X + (size_t)(c0 + t) * a.ld;
                qv = ldf(row + (size_t)h * dim + c) * a.qscale;
                kv = ldf(row + (size_t)(H + h) * dim + c);
            }
            q_s[t * dp + c] = qv;
            k_s[t * dp + c] = kv;
        }
        for (int idx = tid; idx < MC_L * ML_COLS; idx += MC_THREADS) {
            const int t = idx / ML_COLS, col = cb * ML_COLS + idx % ML_COLS;
            v_s[idx] = (t < nc && col < vdim)
                           ? ldf(X + (size_t)(c0 + t) * a.ld + (size_t)2 * H * dim + (size_t)h * vdim + col) : 0.f;
        }
        }
        if (warp == 0) {
            float fg[2], ig[2];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int t = lane + 32 * u;
                fg[u] = 0.f;
                ig[u] = -1e30f;            // a token that is not there: forgets nothing, writes nothing
                if (t < nc) {
                    const float zi = a.gates[(size_t)(c0 + t) * 2 * H + h], zf = a.gates[(size_t)(c0 + t) * 2 * H + H + h];
                    ig[u] = cap * tanhf((zi + bi) * inv_cap);
                    fg[u] = log_sigmoid(cap * tanhf((zf + bf) * inv_cap));
                }
            }
            float b0 = warp_scan_add(fg[0], lane);
            float b1 = warp_scan_add(fg[1], lane) + __shfl_sync(0xffffffffu, b0, 31);
            float x0 = warp_scan_max(ig[0] - b0, lane);
            float x1 = fmaxf(warp_scan_max(ig[1] - b1, lane), __shfl_sync(0xffffffffu, x0, 31));
            const float m0 = b0 + fmaxf(m_prev, x0), m1 = b1 + fmaxf(m_prev, x1);
            const float bL = __shfl_sync(0xffffffffu, b1, 31), mL = __shfl_sync(0xffffffffu, m1, 31);
            b_s[lane] = b0;            b_s[lane + 32] = b1;
            ig_s[lane] = ig[0];        ig_s[lane + 32] = ig[1];
            m_s[lane] = m0;            m_s[lane + 32] = m1;
            g_s[lane] = expf(b0 + m_prev - m0);
            g_s[lane + 32] = expf(b1 + m_prev - m1);
            w_s[lane] = expf(bL - b0 + ig[0] - mL);
            w_s[lane + 32] = expf(bL - b1 + ig[1] - mL);
            if (lane == 0) {
                end_s[0] = bL;
                end_s[1] = mL;
            }
        }
        __syncthreads();
        if (c0 + MC_L < t1) prefetch(c0 + MC_L);
        // ---- 2. C_tj = D_tj (q_t . k_j): a thread takes tokens ti + 16 u and keys ji + 16 u' ---------------------------
        {
            const int ti = tid >> 4, ji = tid & 15;
            float acc[4][4];
#pragma unroll
            for (int u = 0; u < 4; ++u)
#pragma unroll
                for (int w = 0; w < 4; ++w) acc[u][w] = 0.f;
            for (int c = 0; c < dim; ++c) {
                float qv[4], kv[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    qv[u] = q_s[(ti + 16 * u) * dp + c];
                    kv[u] = k_s[(ji + 16 * u) * dp + c];
                }
#pragma unroll
                for (int u = 0; u < 4; ++u)
#pragma unroll
                    for (int w = 0; w < 4; ++w) acc[u][w] += qv[u] * kv[w];
            }
#pragma unroll
            for (int u = 0; u < 4; ++u)
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    const int t = ti + 16 * u, j = ji + 16 * w;
                    C_s[t * (MC_L + 1) + j] = j <= t ? acc[u][w] * expf(b_s[t] - b_s[j] + ig_s[j] - m_s[t]) : 0.f;
                }
        }
        __syncthreads();
        // ---- 3. denominators (the first 64 threads), 4. numerators: a thread takes tokens tp, tp + 32 x 4 columns ---
        {
            // four neighbouring lanes share a token's dot products (q_t . n' and the row sum of C)
            const int t = tid >> 2, part = tid & 3;
            float dot = 0.f;
            for (int r = part; r < dim; r += 4) dot += q_s[t * dp + r] * n_s[r];
            dot *= g_s[t];
            for (int j = part; j <= t; j += 4) dot += C_s[t * (MC_L + 1) + j];
            dot += __shfl_xor_sync(0xffffffffu, dot, 1);
            dot += __shfl_xor_sync(0xffffffffu, dot, 2);
            if (part == 0) den_s[t] = fmaxf(fabsf(dot), expf(-m_s[t])) + ML_DENOM_FLOOR;
        }
        float na[4] = {0.f, 0.f, 0.f, 0.f}, nb[4] = {0.f, 0.f, 0.f, 0.f};
        {
            const float* qa = q_s + tp * dp;
            const float* qb = q_s + (tp + 32) * dp;
            for (int r = 0; r < dim; ++r) {
                const float4 s4 = *reinterpret_cast<const float4*>(S_s + r * ML_COLS + c4);
                const float x = qa[r], y = qb[r];
                na[0] += x * s4.x; na[1] += x * s4.y; na[2] += x * s4.z; na[3] += x * s4.w;
                nb[0] += y * s4.x; nb[1] += y * s4.y; nb[2] += y * s4.z; nb[3] += y * s4.w;
            }
            const float ga = g_s[tp], gb = g_s[tp + 32];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                na[e] *= ga;
                nb[e] *= gb;
            }
            const float* ca = C_s + tp * (MC_L + 1);
            const float* cbp = C_s + (tp + 32) * (MC_L + 1);
            for (int j = 0; j < MC_L; ++j) {
                const float4 v4 = *reinterpret_cast<const float4*>(v_s + j * ML_COLS + c4);
                const float x = ca[j], y = cbp[j];
                na[0] += x * v4.x; na[1] += x * v4.y; na[2] += x * v4.z; na[3] += x * v4.w;
                nb[0] += y * v4.x; nb[1] += y * v4.y; nb[2] += y * v4.z; nb[3] += y * v4.w;
            }
        }
        __syncthreads();
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int col = cb * ML_COLS + c4 + e;
            if (col < vdim) {
                if (tp < nc) a.out[(size_t)(c0 + tp) * H * vdim + (size_t)h * vdim + col] = na[e] / den_s[tp];
                if (tp + 32 < nc) a.out[(size_t)(c0 + tp + 32) * H * vdim + (size_t)h * vdim + col] = nb[e] / den_s[tp + 32];
            }
        }
        // ---- 5. the state's step: a thread takes rows tp + 32 i x its 4 columns -----------------------------------
        {
            const float G = expf(end_s[0] + m_prev - end_s[1]);
            float upd[8][4];
#pragma unroll
            for (int i = 0; i < 8; ++i) upd[i][0] = upd[i][1] = upd[i][2] = upd[i][3] = 0.f;
            for (int j = 0; j < MC_L; ++j) {
                float4 v4 = *reinterpret_cast<const float4*>(v_s + j * ML_COLS + c4);
                const float wj = w_s[j];
                v4.x *= wj; v4.y *= wj; v4.z *= wj; v4.w *= wj;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int r = tp + 32 * i;
                    if (r < dim) {
                        const float kv = k_s[j * dp + r];
                        upd[i][0] += kv * v4.x; upd[i][1] += kv * v4.y; upd[i][2] += kv * v4.z; upd[i][3] += kv * v4.w;
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int r = tp + 32 * i;
                if (r < dim) {
                    float4* sp = reinterpret_cast<float4*>(S_s + r * ML_COLS + c4);
                    float4 s4 = *sp;
                    s4.x = G * s4.x + upd[i][0]; s4.y = G * s4.y + upd[i][1];
                    s4.z = G * s4.z + upd[i][2]; s4.w = G * s4.w + upd[i][3];
                    *sp = s4;
                }
            }
            for (int r = tid; r < dim; r += MC_THREADS) {
                float acc = 0.f;
                for (int j = 0; j < MC_L; ++j) acc += w_s[j] * k_s[j * dp + r];
                n_s[r] = G * n_s[r] + acc;
            }
            m_prev = end_s[1];
        }
        __syncthreads();
    }
    for (int idx = tid; idx < dim * ML_COLS; idx += MC_THREADS) {
        const int r = idx / ML_COLS, col = cb * ML_COLS + idx % ML_COLS;
        if (col < vdim) S[(size_t)r * vdim + col] = S_s[idx];
    }
    for (int r = tid; r < dim; r += MC_THREADS) nvec[r] = n_s[r];
    if (tid == 0) nvec[dim] = m_prev;
}

template <typename T>
static int mlstm_chunk_launch(const MlstmArgs& a, int B, cudaStream_t s) {
    if (B < 0 || a.H <= 0 || a.dim <= 0 || a.vdim <= 0 || !(a.cap > 0.f)) return TB_ERR_ARG;
    if (a.dim > 256) return TB_ERR_UNSUPPORTED;
    if (B == 0) return 0;
    const size_t floats = (size_t)2 * MC_L * (a.dim + 1) + MC_L * ML_COLS + MC_L * (MC_L + 1) + (size_t)a.dim * ML_COLS +
                          a.dim + 6 * MC_L + 4;
    // v_s must start on a 16-byte boundary: 2 * 64 * (dim + 1) floats before it is a multiple of 4
    const size_t smem = floats * sizeof(float);
    if (smem > 200 * 1024) return TB_ERR_UNSUPPORTED;
    dim3 grid(B, a.H, (a.vdim + ML_COLS - 1) / ML_COLS);
    // bfloat16 rows whose pieces of 8 values lie on 16-byte boundaries take the form that fetches a chunk ahead
    constexpr bool is_bf16 = sizeof(T) == 2;
    const bool fast = is_bf16 && a.dim % 8 == 0 && a.vdim % ML_COLS == 0 && a.ld % 8 == 0 && ((a.H * a.dim) % 8 == 0) &&
                      !(reinterpret_cast<uintptr_t>(a.qkv) & 15);
    static bool raised = false;
    if (!raised) {
        tb_note_error(cudaFuncSetAttribute(mlstm_chunk_kernel<T, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        if (is_bf16)
            tb_note_error(cudaFuncSetAttribute(mlstm_chunk_kernel<T, is_bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        raised = true;
    }
    if (fast)
        TB_LAUNCH((mlstm_chunk_kernel<T, is_bf16>), grid, MC_THREADS, smem, s, a);
    else
        TB_LAUNCH((mlstm_chunk_kernel<T, false>), grid, MC_THREADS, smem, s, a);
    return tb_last_error();
}

// y[t, h, :] = o[t, h, :] / sqrt(mean_h(o^2) + eps) * w[h, :] * sigmoid(g[t, h, :])     one warp per (token, head)
template <typename T>
__global__ void __launch_bounds__(128)
mlstm_out_kernel(const float* __restrict__ o, const T* __restrict__ g, int ldg, const float* __restrict__ w,
                 T* __restrict__ y, int nt, int H, int vdim, float eps, int silu) {
    pdl_sync();
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (row >= nt * H) return;
    const int t = row / H, h = row - t * H;
    const float* orow = o + (size_t)t * H * vdim + (size_t)h * vdim;
    float ss = 0.f;
    for (int c = lane; c < vdim; c += 32) ss += orow[c] * orow[c];
    ss = warp_sum(ss);
    const float rs = 1.0f / sqrtf(ss / (float)vdim + eps);
    const T* grow = g + (size_t)t * ldg + (size_t)h * vdim;
    T* yrow = y + (size_t)t * H * vdim + (size_t)h * vdim;
    for (int c = lane; c < vdim; c += 32) {
        const float gz = ldf(grow + c);
        float gate = 1.0f / (1.0f + expf(-gz));
        if (silu) gate *= gz;
        stf(yrow + c, orow[c] * rs * w[(size_t)h * vdim + c] * gate);
    }
}

template <typename T>
static int mlstm_scan_launch(const MlstmArgs& a, int B, cudaStream_t s) {
    if (B < 0 || a.H <= 0 || a.dim <= 0 || a.vdim <= 0 || !(a.cap > 0.f)) return TB_ERR_ARG;
    if (a.dim > 32 * ML_WARPS) return TB_ERR_UNSUPPORTED;
    if (B == 0) return 0;
    dim3 grid(B, a.H, (a.vdim + ML_COLS - 1) / ML_COLS);
    const int rpw = (a.dim + ML_WARPS - 1) / ML_WARPS;
    if (rpw <= 4) TB_LAUNCH((mlstm_scan_kernel<T, 4>), grid, ML_WARPS * 32, 0, s, a);
    else if (rpw <= 8) TB_LAUNCH((mlstm_scan_kernel<T, 8>), grid, ML_WARPS * 32, 0, s, a);
    else if (rpw <= 16) TB_LAUNCH((mlstm_scan_kernel<T, 16>), grid, ML_WARPS * 32, 0, s, a);
    else TB_LAUNCH((mlstm_scan_kernel<T, 32>), grid, ML_WARPS * 32, 0, s, a);
    return tb_last_error();
}

extern "C" {
// Floats of state per (slot, head) for the given sizes.
int tb_mlstm_state_size(int dim, int vdim) {
    return dim * vdim + (vdim + ML_COLS - 1) / ML_COLS * (dim + 1);
}
#define TB_MLSTM(SFX, T)                                                                                              \
    int tb_mlstm_scan_##SFX(const void* qkv, const float* gates, const float* bias, float* state, float* out,         \
                            const int* seq_start, const int* slots, int B, int ld, int H, int dim, int vdim, float cap, \
                            float qscale, cudaStream_t s) {                                                           \
        MlstmArgs a{qkv, gates, bias, state, out, seq_start, slots, ld, H, dim, vdim, cap, qscale};                   \
        return mlstm_scan_launch<T>(a, B, s);                                                                         \
    }                                                                                                                 \
    int tb_mlstm_chunk_##SFX(const void* qkv, const float* gates, const float* bias, float* state, float* out,        \
                             const int* seq_start, const int* slots, int B, int ld, int H, int dim, int vdim, float cap, \
                             float qscale, cudaStream_t s) {                                                          \
        MlstmArgs a{qkv, gates, bias, state, out, seq_start, slots, ld, H, dim, vdim, cap, qscale};                   \
        return mlstm_chunk_launch<T>(a, B, s);                                                                        \
    }                                                                                                                 \
    int tb_mlstm_out_##SFX(const float* o, const void* g, int ldg, const float* w, void* y, int nt, int H, int vdim,  \
                           float eps, int silu, cudaStream_t s) {                                                     \
        if (nt < 0 || H <= 0 || vdim <= 0) return TB_ERR_ARG;                                                         \
        if (nt == 0) return 0;                                                                                        \
        TB_LAUNCH((mlstm_out_kernel<T>), (nt * H + 3) / 4, 128, 0, s, o, (const T*)g, ldg, w, (T*)y, nt, H, vdim, eps, \
                  silu);                                                                                              \
        return tb_last_error();                                                                                       \
    }
TB_MLSTM(f32, float)
TB_MLSTM(bf16, __nv_bfloat16)
}

#include "tape.h"
TB_TAPE_REGISTER(tb_mlstm_scan_f32)
TB_TAPE_REGISTER(tb_mlstm_scan_bf16)
TB_TAPE_REGISTER(tb_mlstm_chunk_f32)
TB_TAPE_REGISTER(tb_mlstm_chunk_bf16)
TB_TAPE_REGISTER(tb_mlstm_out_f32)
TB_TAPE_REGISTER(tb_mlstm_out_bf16)
