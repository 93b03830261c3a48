// Attention through a low-rank latent (multi-head latent attention), over a paged cache of latents.
//
// What is cached per token is ONE row for all heads: the normed latent c [rank] followed by a rotated key part
// kr [rot] that all heads share.  A head's plain key would be Wuk_h c and its value Wuv_h c; neither is ever
// formed for cached tokens.  Instead the query is taken to the latent's side,
//
//   score_h(t, j) = (q_h^plain . Wuk_h c_j + q_h^rot . kr_j) * scale = ((Wuk_h^T q_h^plain) . c_j + q_h^rot . kr_j) * scale
//   o_h(t)        = Wuv_h (sum_j p_h(t, j) c_j)
//
// so that the attention itself runs with one shared "key" [c | kr] of rank + rot entries and one shared
// "value" c, and the two products with Wuk_h^T and Wuv_h wrap it (batched over the heads, gemm_simt.cu).
// A query at position p sees the keys j with 0 <= p - j < window.  Scores, softmax and the output sum are float.
//
// Kernels here: the preparation (norm of the two latents, rotation of the shared key part, cache write), and
// the attention over the cache (CUDA cores, float or bfloat16 storage).
#include "common.cuh"

// ---- preparation -----------------------------------------------------------------------------------
// One block per token.  a[t] = [ zq: q_rank | zc: rank | zr: rot ] (the last two only for a layer that owns a
// latent; q_rank may be 0 for a mixer whose queries come straight from a projection).  cq[t] = zq / rms(zq) * wq;  cache row of (sequence, position) = [ zc / rms(zc) * wc | rotate(zr) ].
// rotate: entries i and i + rdims/2 (i < rdims/2) are a pair, angle = position * base^(-2i/rdims) from the
// tables cos/sin [positions, rdims/2]; entries from rdims on pass.
template <typename T>
__global__ void __launch_bounds__(128)
latent_prep_kernel(const T* __restrict__ a, int lda, const float* __restrict__ wq, const float* __restrict__ wc,
                   float eps, T* __restrict__ cq, T* __restrict__ cache, const int* __restrict__ tok_seq,
                   const int* __restrict__ tok_pos, const int* __restrict__ page_table, int max_pages,
                   const float* __restrict__ cosT, const float* __restrict__ sinT, int q_rank, int rank, int rot,
                   int rdims) {
    pdl_sync();
    __shared__ float red[33];
    const int t = blockIdx.x;
    const T* row = a + (size_t)t * lda;
    float ss = 0.f;
    for (int c = threadIdx.x; c < q_rank; c += blockDim.x) {
        const float v = ldf(row + c);
        ss += v * v;
    }
    ss = block_sum(ss, red);
    float rs = 1.0f / sqrtf(ss / (float)q_rank + eps);
    for (int c = threadIdx.x; c < q_rank; c += blockDim.x) stf(cq + (size_t)t * q_rank + c, ldf(row + c) * rs * wq[c]);
    if (!cache) return;
    const int pos = tok_pos[t];
    const int page = page_table[(size_t)tok_seq[t] * max_pages + pos / TB_PAGE];
    T* dst = cache + ((size_t)page * TB_PAGE + pos % TB_PAGE) * (rank + rot);
    const T* zc = row + q_rank;
    ss = 0.f;
    for (int c = threadIdx.x; c < rank; c += blockDim.x) {
        const float v = ldf(zc + c);
        ss += v * v;
    }
    ss = block_sum(ss, red);
    rs = 1.0f / sqrtf(ss / (float)rank + eps);
    for (int c = threadIdx.x; c < rank; c += blockDim.x) stf(dst + c, ldf(zc + c) * rs * wc[c]);
    const T* zr = zc + rank;
    const int half = rdims / 2;
    for (int c = threadIdx.x; c < rot; c += blockDim.x) {
        float v = ldf(zr + c);
        if (c < half) {
            const float co = cosT[(size_t)pos * half + c], si = sinT[(size_t)pos * half + c];
            v = v * co - ldf(zr + c + half) * si;
        } else if (c < rdims) {
            const float co = cosT[(size_t)pos * half + c - half], si = sinT[(size_t)pos * half + c - half];
            v = v * co + ldf(zr + c - half) * si;
        }
        stf(dst + rank + c, v);
    }
}

// ---- attention over the cache, general kernel ------------------------------------------------------------
// One block = a tile of query tokens of ONE sequence x up to 16 heads: LA_ROWS rows (token, head), all of which
// read the same keys.  A warp owns LA_ROWS / LA_WARPS rows; its 32 lanes are 32 keys for the scores and 32
// channels (NV times) for the output sum.  Keys come 32 at a time into shared memory as floats.
#define LA_WARPS 4
#define LA_ROWS 16
#define LA_RPW (LA_ROWS / LA_WARPS)
#define LA_KEYS 32

struct LatentArgs {
    const void* qa;         // [nt, H, rank]   queries on the latent's side
    const void* q;          // [nt, ldq]       raw queries; head h's rotated part starts at h * q_head + q_plain
    void* out;              // [nt, H, rank]
    const void* cache;      // [pages, TB_PAGE, rank + rot]
    const int* tile_seq;    // [tiles]
    const int* tile_t0;
    const int* tile_nq;
    const int* tok_pos;     // [nt]
    const int* page_table;  // [B, max_pages]
    const float* cosT;      // [positions, rdims / 2]
    const float* sinT;
    int max_pages, ldq, q_head, q_plain, H, rank, rot, rdims, window, heads_per_block, tokens_per_block;
    float scale;
    const float* sinks;     // [H] or null: a number per head that joins the softmax's denominator once
    const void* gate;       // [nt, ldg] or null: head h's output is multiplied by sigmoid(gate[t, h])
    int ldg;
};

template <typename T, int NV>
__global__ void __launch_bounds__(LA_WARPS * 32) latent_attention_kernel(const LatentArgs a) {
    pdl_sync();
    extern __shared__ __align__(16) float la_smem[];
    const int DK = a.rank + a.rot, DKP = (DK + 3) / 4 * 4;     // rows of q padded to float4
    float* q_s = la_smem;                                      // [LA_ROWS][DKP]
    float* k_s = q_s + LA_ROWS * DKP;                          // [LA_KEYS][DK + 1]
    float* p_s = k_s + LA_KEYS * (DK + 1);                     // [LA_WARPS][LA_RPW][LA_KEYS]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int tile = blockIdx.x, h0 = blockIdx.y * a.heads_per_block;
    const int seq = a.tile_seq[tile], t0 = a.tile_t0[tile], nq = a.tile_nq[tile];
    const int hc = a.heads_per_block;
    const T* QA = static_cast<const T*>(a.qa);
    const T* Q = static_cast<const T*>(a.q);
    const T* C = static_cast<const T*>(a.cache);
    // ---- the rows' queries: scaled, the rotated part rotated here -------------------------------------
    for (int idx = threadIdx.x; idx < LA_ROWS * DKP; idx += blockDim.x) {
        const int row = idx / DKP, c = idx - row * DKP;
        const int ti = row / hc, h = h0 + row % hc;
        float v = 0.f;
        if (ti < nq && ti < a.tokens_per_block && h < a.H && c < DK) {
            const int t = t0 + ti;
            if (c < a.rank) {
                v = ldf(QA + ((size_t)t * a.H + h) * a.rank + c);
            } else {
                const T* qr = Q + (size_t)t * a.ldq + (size_t)h * a.q_head + a.q_plain;
                const int r = c - a.rank, half = a.rdims / 2, pos = a.tok_pos[t];
                v = ldf(qr + r);
                if (r < half) {
                    const float co = a.cosT[(size_t)pos * half + r], si = a.sinT[(size_t)pos * half + r];
                    v = v * co - ldf(qr + r + half) * si;
                } else if (r < a.rdims) {
                    const float co = a.cosT[(size_t)pos * half + r - half], si = a.sinT[(size_t)pos * half + r - half];
                    v = v * co + ldf(qr + r - half) * si;
                }
            }
            v *= a.scale;
        }
        q_s[idx] = v;
    }
    int rpos[LA_RPW];
    bool live[LA_RPW];
#pragma unroll
    for (int rr = 0; rr < LA_RPW; ++rr) {
        const int row = warp * LA_RPW + rr;
        const int ti = row / hc, h = h0 + row % hc;
        live[rr] = ti < nq && ti < a.tokens_per_block && h < a.H;
        rpos[rr] = live[rr] ? a.tok_pos[t0 + ti] : -1;
    }
    const int n_tok = nq < a.tokens_per_block ? nq : a.tokens_per_block;
    const int p_first = a.tok_pos[t0], p_last = a.tok_pos[t0 + n_tok - 1];
    const int lo = p_first - a.window + 1 > 0 ? p_first - a.window + 1 : 0;
    float o[LA_RPW][NV], mx[LA_RPW], sum[LA_RPW];
#pragma unroll
    for (int rr = 0; rr < LA_RPW; ++rr) {
        mx[rr] = -INFINITY;
        sum[rr] = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i) o[rr][i] = 0.f;
    }
    const int* table = a.page_table + (size_t)seq * a.max_pages;
    for (int j0 = lo / LA_KEYS * LA_KEYS; j0 <= p_last; j0 += LA_KEYS) {
        __syncthreads();          // the last tile's readers are done (and q_s is written, the first time)
        for (int idx = threadIdx.x; idx < LA_KEYS * DK; idx += blockDim.x) {
            const int kk = idx / DK, c = idx - kk * DK;
            const int j = j0 + kk;
            float v = 0.f;
            if (j <= p_last) v = ldf(C + ((size_t)table[j / TB_PAGE] * TB_PAGE + j % TB_PAGE) * DK + c);
            k_s[kk * (DK + 1) + c] = v;
        }
        __syncthreads();
        // ---- scores: lane = key ---------------------------------------------------------------------
        float sc[LA_RPW];
#pragma unroll
        for (int rr = 0; rr < LA_RPW; ++rr) sc[rr] = 0.f;
        const float* kr = k_s + lane * (DK + 1);
        for (int c = 0; c < DKP; c += 4) {
            const float k0 = kr[c], k1 = c + 1 < DK ? kr[c + 1] : 0.f, k2 = c + 2 < DK ? kr[c + 2] : 0.f,
                        k3 = c + 3 < DK ? kr[c + 3] : 0.f;
#pragma unroll
            for (int rr = 0; rr < LA_RPW; ++rr) {
                const float4 qv = *reinterpret_cast<const float4*>(q_s + (warp * LA_RPW + rr) * DKP + c);
                sc[rr] += qv.x * k0 + qv.y * k1 + qv.z * k2 + qv.w * k3;
            }
        }
        const int j = j0 + lane;
#pragma unroll
        for (int rr = 0; rr < LA_RPW; ++rr) {
            const bool seen = live[rr] && j <= rpos[rr] && rpos[rr] - j < a.window;
            const float sv = seen ? sc[rr] : -INFINITY;
            const float m_new = fmaxf(mx[rr], warp_max(sv));
            float p = 0.f, corr = 1.f;
            if (m_new > -INFINITY) {
                p = seen ? expf(sv - m_new) : 0.f;
                corr = expf(mx[rr] - m_new);        // exp(-inf) = 0 the first time
            }
            mx[rr] = m_new;
            sum[rr] = sum[rr] * corr + warp_sum(p);
#pragma unroll
            for (int i = 0; i < NV; ++i) o[rr][i] *= corr;
            p_s[(warp * LA_RPW + rr) * LA_KEYS + lane] = p;
        }
        __syncwarp();
        // ---- output sum: lane = channel ------------------------------------------------------------------
        for (int kk = 0; kk < LA_KEYS; ++kk) {
            float pv[LA_RPW];
#pragma unroll
            for (int rr = 0; rr < LA_RPW; ++rr) pv[rr] = p_s[(warp * LA_RPW + rr) * LA_KEYS + kk];
            const float* vr = k_s + kk * (DK + 1);
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                const int c = lane + 32 * i;
                const float vv = c < a.rank ? vr[c] : 0.f;
#pragma unroll
                for (int rr = 0; rr < LA_RPW; ++rr) o[rr][i] += pv[rr] * vv;
            }
        }
        __syncwarp();
    }
    T* O = static_cast<T*>(a.out);
#pragma unroll
    for (int rr = 0; rr < LA_RPW; ++rr) {
        if (!live[rr]) continue;
        const int row = warp * LA_RPW + rr;
        const int t = t0 + row / hc, h = h0 + row % hc;
        float f = 1.f, l = sum[rr];
        if (a.sinks) {          // the sink has no key and no value: it only enters the maximum and the sum
            const float sk = a.sinks[h], m2 = fmaxf(mx[rr], sk);
            f = mx[rr] > -INFINITY ? expf(mx[rr] - m2) : 0.f;
            l = l * f + expf(sk - m2);
        }
        float inv = l > 0.f ? f / l : 0.f;
        if (a.gate) inv *= 1.0f / (1.0f + expf(-ldf(static_cast<const T*>(a.gate) + (size_t)t * a.ldg + h)));
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int c = lane + 32 * i;
            if (c < a.rank) stf(O + ((size_t)t * a.H + h) * a.rank + c, o[rr][i] * inv);
        }
    }
}

template <typename T, int NV>
static int latent_attention_go(const LatentArgs& a, int tiles, size_t smem, cudaStream_t s) {
    static bool raised = false;
    if (smem > 48 * 1024 && !raised) {
        tb_note_error(cudaFuncSetAttribute(latent_attention_kernel<T, NV>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           200 * 1024));
        raised = true;
    }
    dim3 grid(tiles, (a.H + a.heads_per_block - 1) / a.heads_per_block);
    TB_LAUNCH((latent_attention_kernel<T, NV>), grid, LA_WARPS * 32, smem, s, a);
    return tb_last_error();
}

template <typename T>
static int latent_attention_launch(LatentArgs a, int tiles, cudaStream_t s) {
    if (tiles < 0 || a.H <= 0 || a.rank <= 0 || a.rot < 0 || a.window <= 0 || a.rdims < 0 || a.rdims > a.rot ||
        a.rdims % 2)
        return TB_ERR_ARG;
    if (a.rank > 512) return TB_ERR_UNSUPPORTED;
    if (tiles == 0) return 0;
    a.heads_per_block = a.H < LA_ROWS ? a.H : LA_ROWS;
    a.tokens_per_block = LA_ROWS / a.heads_per_block;
    const int DK = a.rank + a.rot, DKP = (DK + 3) / 4 * 4;
    const size_t smem = sizeof(float) * ((size_t)LA_ROWS * DKP + (size_t)LA_KEYS * (DK + 1) + LA_ROWS * LA_KEYS);
    if (smem > 200 * 1024) return TB_ERR_UNSUPPORTED;
    if (a.rank <= 32) return latent_attention_go<T, 1>(a, tiles, smem, s);
    if (a.rank <= 64) return latent_attention_go<T, 2>(a, tiles, smem, s);
    if (a.rank <= 128) return latent_attention_go<T, 4>(a, tiles, smem, s);
    if (a.rank <= 256) return latent_attention_go<T, 8>(a, tiles, smem, s);
    return latent_attention_go<T, 16>(a, tiles, smem, s);
}

extern "C" {
// Query tokens of one sequence that a block of the general kernel takes, for a mixer of H heads (the step plans
// tiles of that many tokens).
int tb_latent_attention_tile_tokens(int H) {
    const int hc = H < LA_ROWS ? H : LA_ROWS;
    return LA_ROWS / (hc > 0 ? hc : 1);
}
#define TB_LATENT(SFX, T)                                                                                             \
    int tb_latent_prep_##SFX(const void* a, int lda, const float* wq, const float* wc, float eps, void* cq,           \
                             void* cache, const int* tok_seq, const int* tok_pos, const int* page_table,              \
                             int max_pages, const float* cosT, const float* sinT, int nt, int q_rank, int rank,       \
                             int rot, int rdims, cudaStream_t s) {                                                    \
        if (nt < 0 || q_rank < 0 || (q_rank && (!wq || !cq)) || rank <= 0 || rot < 0 || rdims < 0 || rdims > rot || rdims % 2) return TB_ERR_ARG; \
        if (cache && (!wc || !tok_seq || !tok_pos || !page_table || (rdims && (!cosT || !sinT)))) return TB_ERR_ARG;  \
        if (nt == 0) return 0;                                                                                        \
        TB_LAUNCH((latent_prep_kernel<T>), nt, 128, 0, s, (const T*)a, lda, wq, wc, eps, (T*)cq, (T*)cache, tok_seq,  \
                  tok_pos, page_table, max_pages, cosT, sinT, q_rank, rank, rot, rdims);                              \
        return tb_last_error();                                                                                       \
    }                                                                                                                 \
    int tb_latent_attention_##SFX(const void* qa, const void* q, void* out, const void* cache, const int* tile_seq,   \
                                  const int* tile_t0, const int* tile_nq, const int* tok_pos, const int* page_table,  \
                                  const float* cosT, const float* sinT, int tiles, int max_pages, int ldq,            \
                                  int q_head, int q_plain, int H, int rank, int rot, int rdims, int window,           \
                                  float scale, const float* sinks, const void* gate, int ldg, cudaStream_t s) {       \
        LatentArgs a{qa, q, out, cache, tile_seq, tile_t0, tile_nq, tok_pos, page_table, cosT, sinT, max_pages, ldq,  \
                     q_head, q_plain, H, rank, rot, rdims, window, 0, 0, scale, sinks, gate, ldg};                    \
        return latent_attention_launch<T>(a, tiles, s);                                                               \
    }
TB_LATENT(f32, float)
TB_LATENT(bf16, __nv_bfloat16)
}

#include "tape.h"
TB_TAPE_REGISTER(tb_latent_prep_f32)
TB_TAPE_REGISTER(tb_latent_prep_bf16)
TB_TAPE_REGISTER(tb_latent_attention_f32)
TB_TAPE_REGISTER(tb_latent_attention_bf16)
