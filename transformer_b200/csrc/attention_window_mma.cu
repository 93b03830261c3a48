// Windowed attention over the paged cache on the tensor cores, bfloat16: prompts, portions of prompts and decoding.
//
// Same mathematics as the general windowed kernel (attention_window.cu):
//   score = cap(q . k * scale), visible iff j <= p and (p - j < window or j < keep_first) and (no chunks or both in
//   the same chunk), an optional sink per head in the denominator, an optional turning back of the output's pairs, softmax in float,
//   out = softmax . v * sigmoid(gate); key heads of DK and value heads of DV entries.
//
// A block = one tile of query tokens of ONE sequence x ONE key/value head with ALL the query heads of its group:
// row r of the block's 64 is (token r / group, head r % group), so a page of K and V that is brought to shared
// memory serves every head that reads it (a tile holds 64 / group tokens; the host plans tiles of that size).  The
// block walks the pages (64 keys each) that hold a visible key -- those of the kept first tokens that lie before
// the window's, then the window's -- K double buffered and V behind the score product by cp.async with an XOR
// swizzle, S = Q K^T and O += P V as mma.sync.m16n8k16 fed by ldmatrix, the online softmax in registers.  Warps
// whose 16 rows hold no query (a decode step: the group's few heads are the block's only rows) copy and wait with
// the others and skip the arithmetic.  The visited pages may be cut into slices (grid z): every slice then writes
// (max, sum, unnormalised output) and the merge kernel of attention_window.cu's form combines them and applies
// the gate; that is how a few decoding sequences fill the GPU.
//
// The cap's tanh is 1 - 2 / (1 + 2^(2 y log2 e)) with the hardware's exponential and reciprocal (absolute error
// of a few 1e-7, times the cap), its constants folded with the score's multiplier and log2 e.  Head sizes: the instantiations at the end; others answer TB_ERR_UNSUPPORTED and
// the caller takes the general kernel.
#include "attention_prefill.cuh"

#define WM_ROWS 64
#define WM_KEYS 64
#define WM_THREADS 128

struct WinMmaArgs {
    const __nv_bfloat16* q;      // [nt, q_stride]
    __nv_bfloat16* out;          // [nt, nh * DV]
    const __nv_bfloat16* kc;     // [pages, nkvh, TB_PAGE, DK]
    const __nv_bfloat16* vc;     // [pages, nkvh, TB_PAGE, DV]
    const __nv_bfloat16* gate;   // [nt, gate_stride] or null
    const int* tile_seq;
    const int* tile_t0;
    const int* tile_nq;
    const int* tok_pos;
    const int* page_table;
    float* partial;              // [nt, nh, splits, DV + 2] when splits > 1
    const float* sinks;          // [nh] or null: a number per head in the softmax's denominator
    const float* ocos;           // [positions, DV / 2] or null: the output's pairs (2m, 2m + 1) are turned back
    const float* osin;
    int chunk;                   // > 0: position i sees j only if i / chunk == j / chunk
    int tiles, max_pages, q_stride, gate_stride, nh, nkvh, splits, window, keep_first;
    float scale, softcap;
};

__host__ __device__ constexpr int wm_blocks(int dk, int dv) { return (dk + dv) <= 256 ? 3 : 1; }

template <int DK, int DV>
__global__ void __launch_bounds__(WM_THREADS, wm_blocks(DK, DV)) attention_window_mma_kernel(const WinMmaArgs a) {
    pdl_sync();
    constexpr int CHK = DK / 8, CHV = DV / 8;          // 16-byte chunks in a row of K / of V
    constexpr int RSK = ap_row(DK), RSV = ap_row(DV);
    extern __shared__ __align__(128) __nv_bfloat16 sm[];
    __nv_bfloat16* sq = sm;                            // [64][RSK]
    __nv_bfloat16* sk = sq + WM_ROWS * RSK;            // [2][64][RSK]
    __nv_bfloat16* sv = sk + 2 * WM_KEYS * RSK;        // [64][RSV]
    auto swzk = [](int row, int chunk) { return row * RSK + ((chunk ^ (row & 7)) << 3); };
    auto swzv = [](int row, int chunk) { return row * RSV + ((chunk ^ (row & 7)) << 3); };

    const int tile = a.tiles - 1 - (int)blockIdx.x;
    const int g = blockIdx.y, split = blockIdx.z;
    const int group = a.nh / a.nkvh;
    const int b = a.tile_seq[tile], t0 = a.tile_t0[tile], nq = a.tile_nq[tile];
    const int rows = nq * group;
    const int pos_first = a.tok_pos[t0];
    const int pos_last = pos_first + nq - 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gid = lane >> 2, tid4 = lane & 3;
    const int* pt = a.page_table + (size_t)b * a.max_pages;
    const bool active = warp * 16 < rows;              // this warp's rows hold queries

    // the pages to visit
    int win_lo = a.window > pos_first ? 0 : pos_first - a.window + 1;
    if (a.chunk > 0) win_lo = max(win_lo, pos_first / a.chunk * a.chunk);     // nothing before the first row's chunk
    const int win_p0 = win_lo / WM_KEYS, win_p1 = pos_last / WM_KEYS + 1;
    const int kept = min(a.keep_first, pos_last + 1);
    const int first = min((kept + WM_KEYS - 1) / WM_KEYS, win_p0);
    const int total = first + win_p1 - win_p0;
    const int per = (total + a.splits - 1) / a.splits;
    const int i_lo = split * per, i_hi = min(total, i_lo + per);
    auto page_of = [&](int i) { return i < first ? i : win_p0 + (i - first); };

    auto load_k = [&](int i, __nv_bfloat16* dst_tile) {
        const __nv_bfloat16* src = a.kc + ((size_t)pt[page_of(i)] * a.nkvh + g) * TB_PAGE * DK;
        const uint32_t dst = (uint32_t)__cvta_generic_to_shared(dst_tile);
        for (int idx = threadIdx.x; idx < WM_KEYS * CHK; idx += WM_THREADS) {
            const int row = idx / CHK, c = idx - row * CHK;
            cp_async16(dst + swzk(row, c) * 2, src + row * DK + c * 8);
        }
    };
    auto load_v = [&](int i) {
        const __nv_bfloat16* src = a.vc + ((size_t)pt[page_of(i)] * a.nkvh + g) * TB_PAGE * DV;
        const uint32_t dst = (uint32_t)__cvta_generic_to_shared(sv);
        for (int idx = threadIdx.x; idx < WM_KEYS * CHV; idx += WM_THREADS) {
            const int row = idx / CHV, c = idx - row * CHV;
            cp_async16(dst + swzv(row, c) * 2, src + row * DV + c * 8);
        }
    };

    for (int idx = threadIdx.x; idx < WM_ROWS * CHK; idx += WM_THREADS) {
        const int row = idx / CHK, c = idx - row * CHK;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (row < rows) {
            const int tq = row / group, hh = row - tq * group;
            v = *reinterpret_cast<const uint4*>(a.q + (size_t)(t0 + tq) * a.q_stride + (size_t)(g * group + hh) * DK + c * 8);
        }
        *reinterpret_cast<uint4*>(sq + swzk(row, c)) = v;
    }
    if (i_lo < i_hi) load_k(i_lo, sk);
    cp_async_commit();

    float o[DV / 8][4];
#pragma unroll
    for (int i = 0; i < DV / 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) o[i][j] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const int row_a = warp * 16 + gid, row_b = row_a + 8;
    const int pos_a = pos_first + row_a / group, pos_b = pos_first + row_b / group;
    const uint32_t sq_addr = (uint32_t)__cvta_generic_to_shared(sq);
    const float LOG2E = 1.4426950408889634f;
    const float scale_l2 = a.scale * LOG2E, cap_l2 = a.softcap * LOG2E;
    const float pre_cap = a.softcap > 0.f ? a.scale / a.softcap * 2.0f * LOG2E : 0.f;

    for (int it = i_lo; it < i_hi; ++it) {
        const int buf = (it - i_lo) & 1;
        cp_async_wait<0>();
        __syncthreads();
        load_v(it);
        cp_async_commit();
        if (it + 1 < i_hi) load_k(it + 1, sk + (buf ^ 1) * WM_KEYS * RSK);
        cp_async_commit();
        const uint32_t sk_addr = (uint32_t)__cvta_generic_to_shared(sk + buf * WM_KEYS * RSK);
        const uint32_t sv_addr = (uint32_t)__cvta_generic_to_shared(sv);
        const int key0 = page_of(it) * WM_KEYS;

        uint32_t p[WM_KEYS / 8][2];
        if (active) {
            float s[WM_KEYS / 8][4];
#pragma unroll
            for (int i = 0; i < WM_KEYS / 8; ++i)
#pragma unroll
                for (int c = 0; c < 4; ++c) s[i][c] = 0.f;
#pragma unroll
            for (int ks = 0; ks < DK / 16; ++ks) {
                uint32_t a0, a1, a2, a3;
                {
                    const int row = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                    const int chunk = ks * 2 + (lane >> 4);
                    ldsm_x4(sq_addr + swzk(row, chunk) * 2, a0, a1, a2, a3);
                }
#pragma unroll
                for (int nb = 0; nb < WM_KEYS / 8; nb += 2) {
                    uint32_t b0, b1, b2, b3;
                    const int key = nb * 8 + (lane & 7) + (lane >> 4) * 8;
                    const int chunk = ks * 2 + ((lane >> 3) & 1);
                    ldsm_x4(sk_addr + swzk(key, chunk) * 2, b0, b1, b2, b3);
                    mma16816(s[nb], a0, a1, a2, a3, b0, b1);
                    mma16816(s[nb + 1], a0, a1, a2, a3, b2, b3);
                }
            }
            // every key of the page visible to every row of the block: not later than the first row's token, and
            // inside the last row's window or among the kept
            const bool open = key0 + WM_KEYS - 1 <= pos_first &&
                              (pos_last - key0 < a.window || key0 + WM_KEYS - 1 < a.keep_first) &&
                              (a.chunk <= 0 || key0 / a.chunk == pos_last / a.chunk);
            float mx[2] = {m_run[0], m_run[1]};
#pragma unroll
            for (int nb = 0; nb < WM_KEYS / 8; ++nb) {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    // score * log2 e, capped: cap tanh(y) = cap - 2 cap / (1 + e^{2y}), y = s * scale / cap
                    float v = a.softcap > 0.f ? cap_l2 - __fdividef(2.0f * cap_l2, 1.0f + exp2f(s[nb][c] * pre_cap))
                                              : s[nb][c] * scale_l2;
                    if (!open) {
                        const int key = key0 + nb * 8 + tid4 * 2 + (c & 1);
                        const int pos = (c & 2) ? pos_b : pos_a;
                        if (key > pos || (pos - key >= a.window && key >= a.keep_first) ||
                            (a.chunk > 0 && key / a.chunk != pos / a.chunk))
                            v = -INFINITY;
                    }
                    s[nb][c] = v;
                    mx[c >> 1] = fmaxf(mx[c >> 1], v);
                }
            }
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            }
            float corr[2], mref[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                mref[r] = (mx[r] == -INFINITY) ? 0.f : mx[r];
                corr[r] = exp2f(m_run[r] - mref[r]);
                m_run[r] = mx[r];
                l_run[r] *= corr[r];
            }
#pragma unroll
            for (int i = 0; i < DV / 8; ++i) {
                o[i][0] *= corr[0];
                o[i][1] *= corr[0];
                o[i][2] *= corr[1];
                o[i][3] *= corr[1];
            }
#pragma unroll
            for (int nb = 0; nb < WM_KEYS / 8; ++nb) {
                const float p0 = exp2f(s[nb][0] - mref[0]), p1 = exp2f(s[nb][1] - mref[0]);
                const float p2 = exp2f(s[nb][2] - mref[1]), p3 = exp2f(s[nb][3] - mref[1]);
                l_run[0] += p0 + p1;
                l_run[1] += p2 + p3;
                p[nb][0] = pack_bf16(p0, p1);
                p[nb][1] = pack_bf16(p2, p3);
            }
        }
        cp_async_wait<1>();
        __syncthreads();
        if (active) {
#pragma unroll
            for (int kk = 0; kk < WM_KEYS / 16; ++kk) {
                const uint32_t a0 = p[2 * kk][0], a1 = p[2 * kk][1], a2 = p[2 * kk + 1][0], a3 = p[2 * kk + 1][1];
#pragma unroll
                for (int db = 0; db < DV / 8; db += 2) {
                    uint32_t b0, b1, b2, b3;
                    const int key = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                    const int chunk = db + (lane >> 4);
                    ldsm_x4_t(sv_addr + swzv(key, chunk) * 2, b0, b1, b2, b3);
                    mma16816(o[db], a0, a1, a2, a3, b0, b1);
                    mma16816(o[db + 1], a0, a1, a2, a3, b2, b3);
                }
            }
        }
    }
    cp_async_wait<0>();

#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = r ? row_b : row_a;
        if (row >= rows) continue;
        const int tq = row / group, hh = row - tq * group;
        const int t = t0 + tq, h = g * group + hh;
        if (a.splits == 1) {
            float lsum = l_run[r], keep = 1.f;
            if (a.sinks) {      // the larger of the sink and the running maximum stays the reference
                const float sk = a.sinks[h] * LOG2E;
                if (sk > m_run[r]) {
                    keep = exp2f(m_run[r] - sk);
                    lsum = lsum * keep + 1.f;
                } else {
                    lsum += exp2f(sk - m_run[r]);
                }
            }
            const float inv = keep / lsum;
            const float* oc = a.ocos ? a.ocos + (size_t)a.tok_pos[t] * (DV / 2) + tid4 : nullptr;
            const float* os = a.ocos ? a.osin + (size_t)a.tok_pos[t] * (DV / 2) + tid4 : nullptr;
            __nv_bfloat16* dst = a.out + ((size_t)t * a.nh + h) * DV + tid4 * 2;
            const __nv_bfloat16* gt = a.gate ? a.gate + (size_t)t * a.gate_stride + (size_t)h * DV + tid4 * 2 : nullptr;
#pragma unroll
            for (int i = 0; i < DV / 8; ++i) {
                float v0 = o[i][2 * r] * inv, v1 = o[i][2 * r + 1] * inv;
                if (oc) {       // this thread holds the pair (2m, 2m + 1), m = 4 i + tid4
                    const float co = oc[i * 4], si = os[i * 4];
                    const float r0 = v0 * co + v1 * si, r1 = v1 * co - v0 * si;
                    v0 = r0;
                    v1 = r1;
                }
                if (gt) {
                    const float2 gg = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gt + i * 8));
                    v0 = __fdividef(v0, 1.0f + __expf(-gg.x));
                    v1 = __fdividef(v1, 1.0f + __expf(-gg.y));
                }
                *reinterpret_cast<uint32_t*>(dst + i * 8) = pack_bf16(v0, v1);
            }
        } else {
            float* dst = a.partial + (((size_t)t * a.nh + h) * a.splits + split) * (DV + 2);
#pragma unroll
            for (int i = 0; i < DV / 8; ++i) {
                dst[i * 8 + tid4 * 2] = o[i][2 * r];
                dst[i * 8 + tid4 * 2 + 1] = o[i][2 * r + 1];
            }
            if (tid4 == 0) {
                dst[DV] = m_run[r] * 0.6931471805599453f;       // the merge works with natural exponentials
                dst[DV + 1] = l_run[r];
            }
        }
    }
}

// the merge of attention_window.cu, for bfloat16 outputs
__global__ void attention_window_mma_merge_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ out,
                                                  const __nv_bfloat16* __restrict__ gate, int gate_stride, int nh, int dv,
                                                  int splits, const float* __restrict__ sinks,
                                                  const float* __restrict__ ocos, const float* __restrict__ osin,
                                                  const int* __restrict__ tok_pos) {
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
        if (gate) v *= 1.0f / (1.0f + expf(-__bfloat162float(gate[(size_t)t * gate_stride + (size_t)h * dv + c])));
        out[((size_t)t * nh + h) * dv + c] = __float2bfloat16_rn(v);
    }
}

template <int DK, int DV>
static int window_mma_launch(const WinMmaArgs& a, int nt, cudaStream_t s) {
    const size_t smem = ((size_t)(WM_ROWS + 2 * WM_KEYS) * ap_row(DK) + (size_t)WM_KEYS * ap_row(DV)) * sizeof(__nv_bfloat16);
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_window_mma_kernel<DK, DV>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid(a.tiles, a.nkvh, a.splits);
    TB_LAUNCH((attention_window_mma_kernel<DK, DV>), grid, WM_THREADS, smem, s, a);
    int rc = tb_last_error();
    if (rc || a.splits == 1) return rc;
    dim3 mgrid(nt, a.nh);
    TB_LAUNCH(attention_window_mma_merge_kernel, mgrid, DV < 128 ? 64 : 128, 0, s, a.partial, a.out, a.gate, a.gate_stride,
              a.nh, DV, a.splits, a.sinks, a.ocos, a.osin, a.tok_pos);
    return tb_last_error();
}

extern "C" {
// Query tokens of one sequence that a block takes when a key/value head serves `group` query heads (0: the kernel
// does not take such groups).
int tb_attention_window_mma_tile_tokens(int nh, int nkvh) {
    if (nh <= 0 || nkvh <= 0 || nh % nkvh) return 0;
    const int group = nh / nkvh;
    return group > WM_ROWS ? 0 : WM_ROWS / group;
}

int tb_attention_window_mma_bf16(const void* q, void* out, const void* kc, const void* vc, const void* gate,
                                 const int* tile_seq, const int* tile_t0, const int* tile_nq, const int* tok_pos,
                                 const int* page_table, float* partial, int tiles, int nt, int max_pages, int q_stride,
                                 int gate_stride, int nh, int nkvh, int dk, int dv, int splits, int window,
                                 int keep_first, float scale, float softcap, int chunk, const float* sinks,
                                 const float* ocos, const float* osin, cudaStream_t s) {
    if (nh <= 0 || nkvh <= 0 || nh % nkvh || tiles < 0 || window <= 0 || keep_first < 0 || splits < 1) return TB_ERR_ARG;
    if (chunk < 0 || (ocos && !osin)) return TB_ERR_ARG;
    if (splits > 1 && !partial) return TB_ERR_ARG;
    if (nh / nkvh > WM_ROWS) return TB_ERR_UNSUPPORTED;
    if (q_stride % 8 || gate_stride % 8 ||
        (((uintptr_t)q | (uintptr_t)out | (uintptr_t)kc | (uintptr_t)vc | (uintptr_t)gate) & 15))
        return TB_ERR_UNSUPPORTED;
    if (tiles == 0) return 0;
    WinMmaArgs a{(const __nv_bfloat16*)q, (__nv_bfloat16*)out, (const __nv_bfloat16*)kc, (const __nv_bfloat16*)vc,
                 (const __nv_bfloat16*)gate, tile_seq, tile_t0, tile_nq, tok_pos, page_table, partial, sinks, ocos, osin,
                 chunk, tiles, max_pages,
                 q_stride, gate_stride, nh, nkvh, splits, window, keep_first, scale, softcap};
#define WM_CASE(K, V) if (dk == K && dv == V) return window_mma_launch<K, V>(a, nt, s);
    WM_CASE(32, 32)
    WM_CASE(48, 48)
    WM_CASE(64, 64)
    WM_CASE(96, 96)
    WM_CASE(128, 128)
    WM_CASE(64, 128)
    WM_CASE(128, 64)
    WM_CASE(32, 96)
    WM_CASE(128, 256)
#undef WM_CASE
    return TB_ERR_UNSUPPORTED;
}
}

#include "tape.h"
TB_TAPE_REGISTER(tb_attention_window_mma_bf16)
