// Attention over the cached latents on the tensor cores (bfloat16, mma.sync.m16n8k16), for prompts and decoding.
//
// The math is that of latent.cu: rows (token, head) of one sequence, all reading the same cached rows [c | kr]
// as keys and their first `rank` entries as values; a query at position p sees 0 <= p - j < window.
//
// One block = 16 rows (the M of one mma tile: up to 16 heads of a token, or several tokens of a few heads) x one
// slice of the key range.  Keys come a page (64 keys) at a time into shared memory with cp.async.  Per page:
//   1. scores: warp w takes keys 16 w .. 16 w + 15:  S_w = Q K_w^T over all rank + rot entries (A: the queries from
//      shared memory, B: the page's rows as they lie, both by ldmatrix), scaled, to shared memory as floats;
//   2. softmax: warp w takes rows 4 w .. 4 w + 3: mask by position and window, running maximum and sum (float, in
//      registers), the weights as bfloat16 and the rows' rescaling factors to shared memory;
//   3. values: warp w owns rank / 4 of the output's columns: O_w = O_w * factor + P V_w (B: the page's rows by
//      ldmatrix.trans), float accumulators in registers for the whole key range.
// With more than one slice a block leaves (maximum, sum, unnormalized output) and latent_merge_kernel joins them.
//
// Sizes: rank a multiple of 32 up to 512, rank + rot a multiple of 16; anything else goes to the general kernel.
#include "common.cuh"

// warps per block: 4 (any rank that is a multiple of 32), or 8 when the rank is a multiple of 64: twice the warps
// on an SM to hide the latencies of a k-step's chain of ldmatrix and mma (with four, no unit was busy for more than
// a third of the time and an SM held eight warps)
#define LM_ROWS 16
#define LM_KEYS TB_PAGE     // keys per tile = one page

struct LatentMmaArgs {
    const __nv_bfloat16* qa;     // [nt, H, rank]
    const __nv_bfloat16* q;      // [nt, ldq]; head h's rotated part at h * q_head + q_plain
    __nv_bfloat16* out;          // [nt, H, rank]
    float* partial;              // [nt, H, splits, rank + 2] when splits > 1
    const __nv_bfloat16* cache;  // [pages, TB_PAGE, rank + rot]
    const int* tile_seq;
    const int* tile_t0;
    const int* tile_nq;
    const int* tok_pos;
    const int* page_table;
    const float* cosT;
    const float* sinT;
    int max_pages, ldq, q_head, q_plain, H, rank, rot, rdims, window, heads_per_block, tokens_per_block, splits;
    float scale;
    const float* sinks;          // [H] or null: a number per head that joins the softmax's denominator once
    const __nv_bfloat16* gate;   // [nt, ldg] or null: head h's output is multiplied by sigmoid(gate[t, h])
    int ldg;
};

// What a sink and a gate make of a row's (maximum, sum): the factor for its unnormalized output.
__device__ __forceinline__ float lm_finish(float m, float l, const float* sinks, const __nv_bfloat16* gate, int ldg,
                                           int t, int h) {
    float f = 1.f;
    if (sinks) {
        const float sk = sinks[h], m2 = fmaxf(m, sk);
        f = m > -INFINITY ? __expf(m - m2) : 0.f;
        l = l * f + __expf(sk - m2);
    }
    f = l > 0.f ? f / l : 0.f;
    if (gate) f *= 1.0f / (1.0f + __expf(-__bfloat162float(gate[(size_t)t * ldg + h])));
    return f;
}

__device__ __forceinline__ void lm_ldmatrix_x4(unsigned (&r)[4], const void* p) {
    const unsigned addr = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void lm_ldmatrix_x4_trans(unsigned (&r)[4], const void* p) {
    const unsigned addr = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void lm_mma(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void lm_cp16(void* dst, const void* src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src));
}

// NT = n8 tiles of the output per warp (rank / 4 / 8, rounded up to the instantiated sizes)
template <int NT, int LM_WARPS>
__global__ void __launch_bounds__(LM_WARPS * 32) latent_mma_kernel(const LatentMmaArgs a) {
    constexpr int KPW = LM_KEYS / LM_WARPS;      // keys of a page per warp in the scores' phase: 16 or 8
    constexpr int RPW = LM_ROWS / LM_WARPS;      // rows per warp in the softmax phase: 4 or 2
    pdl_sync();
    extern __shared__ __align__(16) unsigned char lm_smem[];
    const int DK = a.rank + a.rot;
    const int pitch = DK + 8;                                   // in elements: rows 16 bytes apart modulo 128
    __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(lm_smem);                    // [16][pitch]
    __nv_bfloat16* k_s = q_s + LM_ROWS * pitch;                                         // [64][pitch]
    float* s_s = reinterpret_cast<float*>(k_s + LM_KEYS * pitch);                       // [16][64 + 1]
    __nv_bfloat16* p_s = reinterpret_cast<__nv_bfloat16*>(s_s + LM_ROWS * (LM_KEYS + 1));   // [16][64 + 8]
    float* corr_s = reinterpret_cast<float*>(p_s + LM_ROWS * (LM_KEYS + 8));            // [16] factors, then [16] sums
    int* pos_s = reinterpret_cast<int*>(corr_s + 2 * LM_ROWS);                          // [16] positions, -1: no row
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t4 = lane & 3;
    const int tile = blockIdx.x, h0 = blockIdx.y * a.heads_per_block, slice = blockIdx.z;
    const int seq = a.tile_seq[tile], t0 = a.tile_t0[tile];
    const int hc = a.heads_per_block;
    const int n_tok = min(a.tile_nq[tile], a.tokens_per_block);
    // ---- queries: the latent's side as it is (16 bytes at a time), the rotated part rotated here, both unscaled ----
    {
        const int chunks_q = a.rank / 8;
        for (int idx = threadIdx.x; idx < LM_ROWS * chunks_q; idx += blockDim.x) {
            const int row = idx / chunks_q, c = (idx - row * chunks_q) * 8;
            const int ti = row / hc, h = h0 + row % hc;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (ti < n_tok && h < a.H)
                v = *reinterpret_cast<const uint4*>(a.qa + ((size_t)(t0 + ti) * a.H + h) * a.rank + c);
            *reinterpret_cast<uint4*>(q_s + row * pitch + c) = v;
        }
        for (int idx = threadIdx.x; idx < LM_ROWS * a.rot; idx += blockDim.x) {
            const int row = idx / a.rot, r = idx - row * a.rot;
            const int ti = row / hc, h = h0 + row % hc;
            float v = 0.f;
            if (ti < n_tok && h < a.H) {
                const int t = t0 + ti;
                const __nv_bfloat16* qr = a.q + (size_t)t * a.ldq + (size_t)h * a.q_head + a.q_plain;
                const int half = a.rdims / 2, pos = a.tok_pos[t];
                v = __bfloat162float(qr[r]);
                if (r < half) {
                    const float co = a.cosT[(size_t)pos * half + r], si = a.sinT[(size_t)pos * half + r];
                    v = v * co - __bfloat162float(qr[r + half]) * si;
                } else if (r < a.rdims) {
                    const float co = a.cosT[(size_t)pos * half + r - half], si = a.sinT[(size_t)pos * half + r - half];
                    v = v * co + __bfloat162float(qr[r - half]) * si;
                }
            }
            q_s[row * pitch + a.rank + r] = __float2bfloat16_rn(v);
        }
    }
    if (threadIdx.x < LM_ROWS) {
        const int ti = threadIdx.x / hc, h = h0 + threadIdx.x % hc;
        pos_s[threadIdx.x] = (ti < n_tok && h < a.H) ? a.tok_pos[t0 + ti] : -1;
    }
    const int p_first = a.tok_pos[t0], p_last = a.tok_pos[t0 + n_tok - 1];
    const int lo = max(p_first - a.window + 1, 0);
    // pages of this slice
    const int pg_lo = lo / LM_KEYS, pg_hi = p_last / LM_KEYS;          // inclusive
    const int per = (pg_hi - pg_lo + 1 + a.splits - 1) / a.splits;
    const int pg0 = pg_lo + slice * per, pg1 = min(pg_hi, pg0 + per - 1);
    const int* table = a.page_table + (size_t)seq * a.max_pages;
    float acc[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    float mx[RPW], sum[RPW];           // of rows RPW warp .. (the same in every lane)
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
        mx[r] = -INFINITY;
        sum[r] = 0.f;
    }
    const int cols_w = a.rank / LM_WARPS;                                // output columns of this warp
    const int chunks = DK / 8;                                           // 16-byte pieces of a cached row
    __syncthreads();
    for (int pg = pg0; pg <= pg1; ++pg) {
        const __nv_bfloat16* src = a.cache + (size_t)table[pg] * TB_PAGE * DK;
        for (int idx = threadIdx.x; idx < LM_KEYS * chunks; idx += blockDim.x) {
            const int kk = idx / chunks, c8 = idx - kk * chunks;
            lm_cp16(k_s + kk * pitch + c8 * 8, src + (size_t)kk * DK + c8 * 8);
        }
        asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        // ---- 1. scores of this warp's keys ----------------------------------------------------------------------
        if constexpr (LM_WARPS == 8) {
            // 8 keys = one tile of 8 columns; one ldmatrix.x4 of the keys serves two k-steps
            float sc[4] = {0.f, 0.f, 0.f, 0.f}, sd[4] = {0.f, 0.f, 0.f, 0.f};
            const __nv_bfloat16* qa_p = q_s + (lane & 15) * pitch + (lane >> 4) * 8;
            const __nv_bfloat16* kb_p = k_s + (warp * 8 + (lane & 7)) * pitch + (lane >> 3) * 8;
            int k0 = 0;
#pragma unroll 2
            for (; k0 + 32 <= DK; k0 += 32) {
                unsigned af[4], ag[4], bf[4];
                lm_ldmatrix_x4(bf, kb_p + k0);
                lm_ldmatrix_x4(af, qa_p + k0);
                lm_ldmatrix_x4(ag, qa_p + k0 + 16);
                lm_mma(sc, af, bf[0], bf[1]);
                lm_mma(sd, ag, bf[2], bf[3]);
            }
            if (k0 < DK) {        // 16 entries left: the second half of the keys' fragment lies past them and is not used
                unsigned af[4], bf[4];
                lm_ldmatrix_x4(bf, kb_p + k0);
                lm_ldmatrix_x4(af, qa_p + k0);
                lm_mma(sc, af, bf[0], bf[1]);
            }
            const int c = warp * 8 + 2 * t4;
            s_s[g * (LM_KEYS + 1) + c] = (sc[0] + sd[0]) * a.scale;
            s_s[g * (LM_KEYS + 1) + c + 1] = (sc[1] + sd[1]) * a.scale;
            s_s[(g + 8) * (LM_KEYS + 1) + c] = (sc[2] + sd[2]) * a.scale;
            s_s[(g + 8) * (LM_KEYS + 1) + c + 1] = (sc[3] + sd[3]) * a.scale;
        } else
        {
            // two chains of sums (even and odd k-steps), so that a product does not wait for the one before it, and
            // the fragments of several k-steps in flight
            float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
            float sd[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
            const __nv_bfloat16* qa_p = q_s + (lane & 15) * pitch + (lane >> 4) * 8;
            const __nv_bfloat16* kb_p = k_s + (warp * 16 + (lane & 7) + ((lane >> 4) << 3)) * pitch + ((lane >> 3) & 1) * 8;
            int k0 = 0;
#pragma unroll 2
            for (; k0 + 32 <= DK; k0 += 32) {
                unsigned af[4], bf[4], ag[4], bg[4];
                lm_ldmatrix_x4(af, qa_p + k0);
                lm_ldmatrix_x4(bf, kb_p + k0);
                lm_ldmatrix_x4(ag, qa_p + k0 + 16);
                lm_ldmatrix_x4(bg, kb_p + k0 + 16);
                lm_mma(sc[0], af, bf[0], bf[1]);
                lm_mma(sc[1], af, bf[2], bf[3]);
                lm_mma(sd[0], ag, bg[0], bg[1]);
                lm_mma(sd[1], ag, bg[2], bg[3]);
            }
            if (k0 < DK) {
                unsigned af[4], bf[4];
                lm_ldmatrix_x4(af, qa_p + k0);
                lm_ldmatrix_x4(bf, kb_p + k0);
                lm_mma(sc[0], af, bf[0], bf[1]);
                lm_mma(sc[1], af, bf[2], bf[3]);
            }
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) sc[nt][e] += sd[nt][e];
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                const int c = warp * 16 + nt * 8 + 2 * t4;
                s_s[g * (LM_KEYS + 1) + c] = sc[nt][0] * a.scale;
                s_s[g * (LM_KEYS + 1) + c + 1] = sc[nt][1] * a.scale;
                s_s[(g + 8) * (LM_KEYS + 1) + c] = sc[nt][2] * a.scale;
                s_s[(g + 8) * (LM_KEYS + 1) + c + 1] = sc[nt][3] * a.scale;
            }
        }
        __syncthreads();
        // ---- 2. softmax of this warp's rows --------------------------------------------------------------------
#pragma unroll
        for (int r = 0; r < RPW; ++r) {
            const int row = warp * RPW + r, pos = pos_s[row];
            const int j0 = pg * LM_KEYS + lane, j1 = j0 + 32;
            const bool see0 = pos >= 0 && j0 <= pos && pos - j0 < a.window;
            const bool see1 = pos >= 0 && j1 <= pos && pos - j1 < a.window;
            const float v0 = see0 ? s_s[row * (LM_KEYS + 1) + lane] : -INFINITY;
            const float v1 = see1 ? s_s[row * (LM_KEYS + 1) + lane + 32] : -INFINITY;
            const float m_new = fmaxf(mx[r], warp_max(fmaxf(v0, v1)));
            float p0 = 0.f, p1 = 0.f, corr = 1.f;
            if (m_new > -INFINITY) {
                p0 = see0 ? __expf(v0 - m_new) : 0.f;
                p1 = see1 ? __expf(v1 - m_new) : 0.f;
                corr = __expf(mx[r] - m_new);
            }
            mx[r] = m_new;
            sum[r] = sum[r] * corr + warp_sum(p0 + p1);
            p_s[row * (LM_KEYS + 8) + lane] = __float2bfloat16_rn(p0);
            p_s[row * (LM_KEYS + 8) + lane + 32] = __float2bfloat16_rn(p1);
            if (lane == 0) corr_s[row] = corr;
        }
        __syncthreads();
        // ---- 3. this warp's columns of the output ----------------------------------------------------------------
        {
            const float c_lo = corr_s[g], c_hi = corr_s[g + 8];
#pragma unroll
            for (int i = 0; i < NT; ++i) {
                acc[i][0] *= c_lo;
                acc[i][1] *= c_lo;
                acc[i][2] *= c_hi;
                acc[i][3] *= c_hi;
            }
            const __nv_bfloat16* pa_p = p_s + (lane & 15) * (LM_KEYS + 8) + (lane >> 4) * 8;
            // .trans: lanes 0-7 keys k0..k0+7 of columns n0.., 8-15 keys k0+8.., 16-23 and 24-31 the same of n0+8..
            const __nv_bfloat16* vb_p = k_s + ((lane & 7) + ((lane >> 3) & 1) * 8) * pitch + warp * cols_w + (lane >> 4) * 8;
#pragma unroll
            for (int k0 = 0; k0 < LM_KEYS; k0 += 16) {
                unsigned af[4];
                lm_ldmatrix_x4(af, pa_p + k0);
#pragma unroll
                for (int i = 0; i < NT; i += 2) {
                    if (i * 8 < cols_w) {
                        unsigned bf[4];
                        lm_ldmatrix_x4_trans(bf, vb_p + (size_t)k0 * pitch + i * 8);
                        lm_mma(acc[i], af, bf[0], bf[1]);
                        if (i + 1 < NT && (i + 1) * 8 < cols_w) lm_mma(acc[i + 1], af, bf[2], bf[3]);
                    }
                }
            }
        }
        __syncthreads();        // the page's rows and the weights are free again
    }
    // ---- the end: sums to shared memory, then every warp stores its columns ------------------------------------
    float* sum_s = corr_s + LM_ROWS;
    float* max_s = s_s;             // free by now
    if (lane == 0) {
#pragma unroll
        for (int r = 0; r < RPW; ++r) {
            sum_s[warp * RPW + r] = sum[r];
            max_s[warp * RPW + r] = mx[r];
        }
    }
    __syncthreads();
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        const int row = g + 8 * hh;
        if (pos_s[row] < 0) continue;
        const int t = t0 + row / hc, h = h0 + row % hc;
        const float l = sum_s[row];
        if (a.splits == 1) {
            const float inv = lm_finish(max_s[row], l, a.sinks, a.gate, a.ldg, t, h);
            __nv_bfloat16* o = a.out + ((size_t)t * a.H + h) * a.rank + warp * cols_w;
#pragma unroll
            for (int i = 0; i < NT; ++i) {
                const int c = i * 8 + 2 * t4;
                if (c < cols_w)
                    *reinterpret_cast<__nv_bfloat162*>(o + c) =
                        __floats2bfloat162_rn(acc[i][2 * hh] * inv, acc[i][2 * hh + 1] * inv);
            }
        } else {
            float* o = a.partial + (((size_t)t * a.H + h) * a.splits + slice) * (a.rank + 2);
            if (warp == 0 && t4 == 0) {
                o[0] = max_s[row];
                o[1] = l;
            }
#pragma unroll
            for (int i = 0; i < NT; ++i) {
                const int c = i * 8 + 2 * t4;
                if (c < cols_w) {
                    o[2 + warp * cols_w + c] = acc[i][2 * hh];
                    o[2 + warp * cols_w + c + 1] = acc[i][2 * hh + 1];
                }
            }
        }
    }
}

// out[t, h] = sum_s e^{m_s - m} O_s / sum_s e^{m_s - m} l_s        one block per (token, head): the slices' factors
// once, then every thread its columns with the loads of all slices in flight together
#define LM_MAX_SPLITS 16
__global__ void __launch_bounds__(128)
latent_merge_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ out, int splits, int rank,
                    const float* __restrict__ sinks, const __nv_bfloat16* __restrict__ gate, int ldg, int H) {
    pdl_sync();
    __shared__ float f_s[LM_MAX_SPLITS];
    const float* p = partial + (size_t)blockIdx.x * splits * (rank + 2);
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        const float ms = lane < splits ? p[(size_t)lane * (rank + 2)] : -INFINITY;
        const float ls = lane < splits ? p[(size_t)lane * (rank + 2) + 1] : 0.f;
        const float m = warp_max(ms);
        const float f = ms > -INFINITY ? __expf(ms - m) : 0.f;
        const float l = warp_sum(f * ls);
        const float fin = lm_finish(m, l, sinks, gate, ldg, blockIdx.x / H, blockIdx.x % H);
        if (lane < splits) f_s[lane] = f * fin;
    }
    __syncthreads();
    for (int c = threadIdx.x; c < rank; c += blockDim.x) {
        float v[LM_MAX_SPLITS];
#pragma unroll
        for (int s = 0; s < LM_MAX_SPLITS; ++s) v[s] = s < splits ? p[(size_t)s * (rank + 2) + 2 + c] : 0.f;
        float acc = 0.f;
#pragma unroll
        for (int s = 0; s < LM_MAX_SPLITS; ++s)
            if (s < splits) acc += f_s[s] * v[s];
        out[(size_t)blockIdx.x * rank + c] = __float2bfloat16_rn(acc);
    }
}

template <int NT, int W>
static int latent_mma_go(const LatentMmaArgs& a, int tiles, size_t smem, cudaStream_t s) {
    static bool raised = false;
    if (smem > 48 * 1024 && !raised) {
        tb_note_error(cudaFuncSetAttribute(latent_mma_kernel<NT, W>, cudaFuncAttributeMaxDynamicSharedMemorySize, 120 * 1024));
        raised = true;
    }
    dim3 grid(tiles, (a.H + a.heads_per_block - 1) / a.heads_per_block, a.splits);
    TB_LAUNCH((latent_mma_kernel<NT, W>), grid, W * 32, smem, s, a);
    return tb_last_error();
}

extern "C" {
// As tb_latent_attention_bf16, on the tensor cores.  splits > 1: the key range of every block is cut into that many
// slices, `partial` [nt, H, splits, rank + 2] floats receives them and a second kernel joins them.
// TB_ERR_UNSUPPORTED for sizes it does not take (nothing has been done then).
int tb_latent_attention_mma_bf16(const void* qa, const void* q, void* out, float* partial, const void* cache,
                                 const int* tile_seq, const int* tile_t0, const int* tile_nq, const int* tok_pos,
                                 const int* page_table, const float* cosT, const float* sinT, int tiles, int nt,
                                 int max_pages, int ldq, int q_head, int H, int rank, int rot, int rdims, int window,
                                 int splits, float scale, const float* sinks, const void* gate, int ldg,
                                 cudaStream_t s) {
    const int q_plain = q_head - rot;      // a head's queries: the plain entries, then the rotated ones
    if (tiles < 0 || nt < 0 || H <= 0 || rank <= 0 || rot < 0 || window <= 0 || rdims < 0 || rdims > rot || rdims % 2 ||
        splits < 1 || splits > LM_MAX_SPLITS || (splits > 1 && !partial))
        return TB_ERR_ARG;
    if (rank % 32 || rank > 512 || (rank + rot) % 16 || ((((uintptr_t)cache) | ((uintptr_t)qa)) & 15))
        return TB_ERR_UNSUPPORTED;
    if (tiles == 0) return 0;
    const int hc = H < LM_ROWS ? H : LM_ROWS;
    LatentMmaArgs a{(const __nv_bfloat16*)qa, (const __nv_bfloat16*)q, (__nv_bfloat16*)out, partial,
                    (const __nv_bfloat16*)cache, tile_seq, tile_t0, tile_nq, tok_pos, page_table, cosT, sinT, max_pages,
                    ldq, q_head, q_plain, H, rank, rot, rdims, window, hc, LM_ROWS / hc, splits, scale, sinks,
                    (const __nv_bfloat16*)gate, ldg};
    const int DK = rank + rot, pitch = DK + 8;
    const size_t smem = (size_t)(LM_ROWS + LM_KEYS) * pitch * 2 + LM_ROWS * (LM_KEYS + 1) * 4 + LM_ROWS * (LM_KEYS + 8) * 2 +
                        2 * LM_ROWS * 4 + LM_ROWS * 4;
    if (smem > 120 * 1024) return TB_ERR_UNSUPPORTED;
    int rc;
    if (rank % 64 == 0) {               // eight warps: rank / 8 columns of the output each
        const int nt8 = rank / 8 / 8;
        if (nt8 <= 2) rc = latent_mma_go<2, 8>(a, tiles, smem, s);
        else if (nt8 <= 4) rc = latent_mma_go<4, 8>(a, tiles, smem, s);
        else rc = latent_mma_go<8, 8>(a, tiles, smem, s);
    } else {
        const int nt8 = rank / 4 / 8;
        if (nt8 <= 2) rc = latent_mma_go<2, 4>(a, tiles, smem, s);
        else if (nt8 <= 4) rc = latent_mma_go<4, 4>(a, tiles, smem, s);
        else if (nt8 <= 8) rc = latent_mma_go<8, 4>(a, tiles, smem, s);
        else rc = latent_mma_go<16, 4>(a, tiles, smem, s);
    }
    if (rc || splits == 1) return rc;
    TB_LAUNCH((latent_merge_kernel), nt * H, 128, 0, s, (const float*)partial, (__nv_bfloat16*)out, splits, rank, sinks,
              (const __nv_bfloat16*)gate, ldg, H);
    return tb_last_error();
}
}

#include "tape.h"
TB_TAPE_REGISTER(tb_latent_attention_mma_bf16)
