// Attention over the paged cache with a sliding window that keeps the first tokens, capped scores, key and value
// heads of different sizes and a gate on the output: the general kernel (CUDA cores, float or bfloat16).
//
//   score(q at position p, key at position j) = cap(q . k * scale),   cap(s) = softcap * tanh(s / softcap)  (softcap > 0)
//   visible iff j <= p and (p - j < window or j < keep_first) and (chunk == 0 or j / chunk == p / chunk)
//   out[t, h, :] = softmax over the visible keys . v  * sigmoid(gate[t, h, :])                (gate may be absent)
//   sink (may be absent): a number per head that joins the softmax's denominator as exp(sink_h), with no key and no
//       value, neither scaled nor capped
//   values cached rotated (may be absent): the head's output at position p is turned back before the gate, pair
//       (2m, 2m + 1) by -p * g_m, from the tables ocos / osin [positions, dv / 2]
//
// All arithmetic is float (scores, the cap, running maximum, sum, output accumulator).  Keys [pages, nkvh, 64, dk] and
// values [pages, nkvh, 64, dv] of the step's own tokens are already in the cache.  The cache keeps every position:
// the window is a mask, and a block visits only the 32-key tiles that hold a visible key -- those of the kept first
// tokens, then those of the window.
//
// Work split as in the general causal kernel: a block = one tile of query tokens of ONE sequence x one key/value
// head x up to 16 of its query heads x one slice of the visited key tiles; rows (token, head) share every key tile
// in shared memory; a warp owns rows warp, warp + 4, ...; its lanes are 32 keys for the scores and 32 output
// channels for P.V.  With more than one slice each block writes (max, sum, unnormalised output) and the merge
// kernel combines them and applies the gate.
#include "common.cuh"

#define AW_WARPS 4
#define AW_ROWS 16
#define AW_RPW (AW_ROWS / AW_WARPS)
#define AW_KEYS 32

struct WinArgs {
    const void* q;          // [nt, q_stride], first query head of each token
    void* out;              // [nt, nh * dv]
    const void* kc;         // [pages, nkvh, TB_PAGE, dk]
    const void* vc;         // [pages, nkvh, TB_PAGE, dv]
    const void* gate;       // [nt, gate_stride] pre-activation of the output gate, nh * dv wide, or null
    const int* tile_seq;
    const int* tile_t0;
    const int* tile_nq;
    const int* tok_pos;
    const int* page_table;
    float* partial;         // [nt, nh, splits, dv + 2] when splits > 1
    const float* sinks;     // [nh] or null
    const float* ocos;      // [positions, dv / 2] or null
    const float* osin;
    int chunk;              // 0: none
    int max_pages, q_stride, gate_stride, nh, nkvh, dk, dv, hc, splits, window, keep_first;
    float scale, softcap;
};

template <typename T, int DPL>
__global__ void __launch_bounds__(AW_WARPS * 32) attention_window_kernel(const WinArgs a) {
    pdl_sync();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int dk = a.dk, dv = a.dv;
    const int kstride = dk + (sizeof(T) == 4 ? 1 : 2);
    float* qs = reinterpret_cast<float*>(smem_raw);                 // [AW_ROWS][dk]
    T* ks = reinterpret_cast<T*>(qs + AW_ROWS * dk);                // [AW_KEYS][kstride]
    T* vs = ks + AW_KEYS * kstride;                                 // [AW_KEYS][dv]

    const int tile = blockIdx.x;
    const int group = a.nh / a.nkvh;
    const int chunks = (group + a.hc - 1) / a.hc;
    const int g = blockIdx.y / chunks;
    const int h0 = g * group + (blockIdx.y % chunks) * a.hc;
    const int nheads = min(a.hc, g * group + group - h0);
    const int split = blockIdx.z;
    const int b = a.tile_seq[tile], t0 = a.tile_t0[tile], nq = a.tile_nq[tile];
    const int rows = nq * nheads;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const T* qg = static_cast<const T*>(a.q);

    for (int idx = threadIdx.x; idx < rows * dk; idx += blockDim.x) {
        const int r = idx / dk, c = idx - r * dk;
        const int tq = r / nheads, hh = r - tq * nheads;
        qs[r * dk + c] = ldf(qg + (size_t)(t0 + tq) * a.q_stride + (size_t)(h0 + hh) * dk + c);
    }
    const int pos_first = a.tok_pos[t0];
    const int pos_last = pos_first + nq - 1;
    // the tiles to visit: those of the kept first tokens that lie before the window's, then the window's
    int win_lo = a.window > pos_first ? 0 : pos_first - a.window + 1;
    if (a.chunk > 0) win_lo = max(win_lo, pos_first / a.chunk * a.chunk);     // nothing before the first row's chunk
    const int win_t0 = win_lo / AW_KEYS, win_t1 = pos_last / AW_KEYS + 1;
    const int kept = min(a.keep_first, pos_last + 1);
    const int first = min((kept + AW_KEYS - 1) / AW_KEYS, win_t0);
    const int total = first + win_t1 - win_t0;
    const int per = (total + a.splits - 1) / a.splits;
    const int i_lo = split * per, i_hi = min(total, i_lo + per);

    float m[AW_RPW], l[AW_RPW], o[AW_RPW][DPL];
#pragma unroll
    for (int i = 0; i < AW_RPW; ++i) {
        m[i] = -INFINITY;
        l[i] = 0.f;
#pragma unroll
        for (int c = 0; c < DPL; ++c) o[i][c] = 0.f;
    }
    const T* kc = static_cast<const T*>(a.kc);
    const T* vc = static_cast<const T*>(a.vc);
    const float inv_cap = a.softcap > 0.f ? 1.0f / a.softcap : 0.f;

    for (int it = i_lo; it < i_hi; ++it) {
        const int kt = it < first ? it : win_t0 + (it - first);
        const int key0 = kt * AW_KEYS;
        const int page = a.page_table[(size_t)b * a.max_pages + key0 / TB_PAGE];
        const size_t row0 = ((size_t)page * a.nkvh + g) * TB_PAGE + (key0 % TB_PAGE);
        __syncthreads();
        for (int idx = threadIdx.x; idx < AW_KEYS * dk; idx += blockDim.x) {
            const int j = idx / dk, c = idx - j * dk;
            ks[j * kstride + c] = key0 + j <= pos_last ? kc[row0 * dk + idx] : T(0.f);
        }
        for (int idx = threadIdx.x; idx < AW_KEYS * dv; idx += blockDim.x) {
            const int j = idx / dv;
            vs[idx] = key0 + j <= pos_last ? vc[row0 * dv + idx] : T(0.f);
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < AW_RPW; ++i) {
            const int r = warp + i * AW_WARPS;
            if (r >= rows) continue;
            const int pos_r = pos_first + r / nheads;
            const float* qr = qs + r * dk;
            const T* kr = ks + lane * kstride;
            float s = 0.f;
            for (int c = 0; c < dk; ++c) s += qr[c] * ldf(kr + c);
            s *= a.scale;
            if (a.softcap > 0.f) s = a.softcap * tanhf(s * inv_cap);
            const int j = key0 + lane;
            const bool see = j <= pos_r && (pos_r - j < a.window || j < a.keep_first) &&
                             (a.chunk <= 0 || j / a.chunk == pos_r / a.chunk);
            s = see ? s : -INFINITY;
            const float m_new = fmaxf(m[i], warp_max(s));
            if (m_new == -INFINITY) continue;
            const float p = expf(s - m_new);
            const float corr = expf(m[i] - m_new);
            l[i] = l[i] * corr + warp_sum(p);
            m[i] = m_new;
#pragma unroll
            for (int c = 0; c < DPL; ++c) o[i][c] *= corr;
            for (int jj = 0; jj < AW_KEYS; ++jj) {
                const float pj = __shfl_sync(0xffffffffu, p, jj);
#pragma unroll
                for (int c = 0; c < DPL; ++c) {
                    const int ch = lane + 32 * c;
                    if (ch < dv) o[i][c] += pj * ldf(vs + jj * dv + ch);
                }
            }
        }
    }

#pragma unroll
    for (int i = 0; i < AW_RPW; ++i) {
        const int r = warp + i * AW_WARPS;
        if (r >= rows) continue;
        const int tq = r / nheads, hh = r - tq * nheads;
        const int t = t0 + tq, h = h0 + hh;
        if (a.splits == 1) {
            T* dst = static_cast<T*>(a.out) + ((size_t)t * a.nh + h) * dv;
            const T* gt = a.gate ? static_cast<const T*>(a.gate) + (size_t)t * a.gate_stride + (size_t)h * dv : nullptr;
            float lsum = l[i], keep = 1.f;
            if (a.sinks) {          // the sink joins the denominator; the larger of it and the maximum stays the reference
                const float sk = a.sinks[h];
                if (sk > m[i]) {
                    keep = expf(m[i] - sk);
                    lsum = lsum * keep + 1.f;
                } else {
                    lsum += expf(sk - m[i]);
                }
            }
            const float inv = keep / lsum;
            const int pos_t = a.ocos ? a.tok_pos[t] : 0;
#pragma unroll
            for (int c = 0; c < DPL; ++c) {
                const int ch = lane + 32 * c;
                float v = o[i][c] * inv;
                if (a.ocos) {       // the pair's other entry sits in the neighbouring lane
                    const float other = __shfl_xor_sync(0xffffffffu, v, 1);
                    if (ch < dv) {
                        const float co = a.ocos[(size_t)pos_t * (dv / 2) + (ch >> 1)];
                        const float si = a.osin[(size_t)pos_t * (dv / 2) + (ch >> 1)];
                        v = (ch & 1) ? v * co - other * si : v * co + other * si;
                    }
                }
                if (ch < dv) {
                    if (gt) v *= 1.0f / (1.0f + expf(-ldf(gt + ch)));
                    stf(dst + ch, v);
                }
            }
        } else {
            float* dst = a.partial + (((size_t)t * a.nh + h) * a.splits + split) * (dv + 2);
#pragma unroll
            for (int c = 0; c < DPL; ++c) {
                const int ch = lane + 32 * c;
                if (ch < dv) dst[ch] = o[i][c];
            }
            if (lane == 0) {
                dst[dv] = m[i];
                dst[dv + 1] = l[i];
            }
        }
    }
}

// out[t, h, :] = sum_s o_s exp(m_s - m) / sum_s l_s exp(m_s - m) * sigmoid(gate),  m = max_s m_s.
template <typename T>
__global__ void attention_window_merge_kernel(const float* __restrict__ partial, T* __restrict__ out,
                                              const T* __restrict__ gate, int gate_stride, int nh, int dv, int splits,
                                              const float* __restrict__ sinks, const float* __restrict__ ocos,
                                              const float* __restrict__ osin, const int* __restrict__ tok_pos) {
    pdl_sync();
    const int t = blockIdx.x, h = blockIdx.y;
    const float* p = partial + ((size_t)t * nh + h) * splits * (dv + 2);
    float m = sinks ? sinks[h] : -INFINITY;
    for (int s = 0; s < splits; ++s) m = fmaxf(m, p[s * (dv + 2) + dv]);
    float den = sinks ? expf(sinks[h] - m) : 0.f;
    for (int s = 0; s < splits; ++s) {
        const float ms = p[s * (dv + 2) + dv];
        if (ms != -INFINITY) den += p[s * (dv + 2) + dv + 1] * expf(ms - m);
    }
    for (int c = threadIdx.x; c < dv; c += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < splits; ++s) {
            const float ms = p[s * (dv + 2) + dv];
            if (ms != -INFINITY) acc += p[s * (dv + 2) + c] * expf(ms - m);
        }
        float v = acc / den;
        if (ocos) {             // turn the pair (c, c ^ 1) back: the other entry is summed here as well
            float other = 0.f;
            for (int s = 0; s < splits; ++s) {
                const float ms = p[s * (dv + 2) + dv];
                if (ms != -INFINITY) other += p[s * (dv + 2) + (c ^ 1)] * expf(ms - m);
            }
            other /= den;
            const float co = ocos[(size_t)tok_pos[t] * (dv / 2) + (c >> 1)], si = osin[(size_t)tok_pos[t] * (dv / 2) + (c >> 1)];
            v = (c & 1) ? v * co - other * si : v * co + other * si;
        }
        if (gate) v *= 1.0f / (1.0f + expf(-ldf(gate + (size_t)t * gate_stride + (size_t)h * dv + c)));
        stf(out + ((size_t)t * nh + h) * dv + c, v);
    }
}

template <typename T, int DPL>
static int window_launch_dpl(const WinArgs& a, int tiles, cudaStream_t s) {
    const int kstride = a.dk + (sizeof(T) == 4 ? 1 : 2);
    const size_t smem = (size_t)AW_ROWS * a.dk * 4 + (size_t)AW_KEYS * kstride * sizeof(T) + (size_t)AW_KEYS * a.dv * sizeof(T);
    static size_t configured = 0;
    if (smem > 48 * 1024 && smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_window_kernel<T, DPL>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = smem;
    }
    const int group = a.nh / a.nkvh;
    const int chunks = (group + a.hc - 1) / a.hc;
    dim3 grid(tiles, a.nkvh * chunks, a.splits);
    TB_LAUNCH((attention_window_kernel<T, DPL>), grid, AW_WARPS * 32, smem, s, a);
    return tb_last_error();
}

template <typename T>
static int window_launch(WinArgs a, int tiles, int nt, cudaStream_t s) {
    if (a.nh <= 0 || a.nkvh <= 0 || a.nh % a.nkvh || a.window <= 0 || a.keep_first < 0) return TB_ERR_ARG;
    if (a.dk <= 0 || a.dv <= 0 || a.dk > 256 || a.dv > 256) return TB_ERR_UNSUPPORTED;
    if (a.splits < 1 || (a.splits > 1 && !a.partial)) return TB_ERR_ARG;
    if (a.chunk < 0 || (a.ocos && (!a.osin || a.dv % 2))) return TB_ERR_ARG;
    if (tiles <= 0 || nt <= 0) return tiles == 0 || nt == 0 ? 0 : TB_ERR_ARG;
    const int group = a.nh / a.nkvh;
    a.hc = group < AW_ROWS ? group : AW_ROWS;
    int rc;
    switch ((a.dv + 31) / 32) {
        case 1: rc = window_launch_dpl<T, 1>(a, tiles, s); break;
        case 2: rc = window_launch_dpl<T, 2>(a, tiles, s); break;
        case 3: rc = window_launch_dpl<T, 3>(a, tiles, s); break;
        case 4: rc = window_launch_dpl<T, 4>(a, tiles, s); break;
        case 5: rc = window_launch_dpl<T, 5>(a, tiles, s); break;
        case 6: rc = window_launch_dpl<T, 6>(a, tiles, s); break;
        case 7: rc = window_launch_dpl<T, 7>(a, tiles, s); break;
        default: rc = window_launch_dpl<T, 8>(a, tiles, s); break;
    }
    if (rc) return rc;
    if (a.splits > 1) {
        dim3 grid(nt, a.nh);
        TB_LAUNCH((attention_window_merge_kernel<T>), grid, a.dv < 128 ? 64 : 128, 0, s, a.partial, (T*)a.out,
                  (const T*)a.gate, a.gate_stride, a.nh, a.dv, a.splits, a.sinks, a.ocos, a.osin, a.tok_pos);
        rc = tb_last_error();
    }
    return rc;
}

extern "C" {
#define TB_ATTENTION_WINDOW(NAME, T)                                                                                  \
    int NAME(const void* q, void* out, const void* kc, const void* vc, const void* gate, const int* tile_seq,         \
             const int* tile_t0, const int* tile_nq, const int* tok_pos, const int* page_table, float* partial,       \
             int tiles, int nt, int max_pages, int q_stride, int gate_stride, int nh, int nkvh, int dk, int dv,       \
             int splits, int window, int keep_first, float scale, float softcap, int chunk, const float* sinks,       \
             const float* ocos, const float* osin, cudaStream_t s) {                                                  \
        WinArgs a{q, out, kc, vc, gate, tile_seq, tile_t0, tile_nq, tok_pos, page_table, partial, sinks, ocos, osin,  \
                  chunk, max_pages, q_stride, gate_stride, nh, nkvh, dk, dv, 0, splits, window, keep_first, scale,    \
                  softcap};                                                                                           \
        return window_launch<T>(a, tiles, nt, s);                                                                     \
    }
TB_ATTENTION_WINDOW(tb_attention_window_f32, float)
TB_ATTENTION_WINDOW(tb_attention_window_bf16, __nv_bfloat16)
}

#include "tape.h"
TB_TAPE_REGISTER(tb_attention_window_f32)
TB_TAPE_REGISTER(tb_attention_window_bf16)
