// What lies between the merged q-k-v product and the attention for a mixer with short convolutions on its
// projections, a norm per head and rotated values, in one kernel:
//
//   u = causal convolution over time of every channel of [q | k | v]     (taps wide, the last inputs kept per sequence)
//   q_h <- u_q,h / rms(u_q,h) * wq * temp_h,   k_g <- u_k,g / rms(u_k,g) * wk        (weights of one head, shared)
//   the first rdims entries of every query and key head turn by position * f_i in the pairs (2i, 2i + 1)
//   v <- (1 - l) v + l v_source      a blend with the values that an earlier layer left for the same token in
//                                    `vfirst` (float [nt, nkvh * dv]); without `vmix` (the number l) this layer is
//                                    that source and leaves its own values there
//   every pair (2m, 2m + 1) of a value head turns by position * g_m
//   queries go to `qout`, keys and values into the paged cache
//
// The convolution, the norm, the temperature and the rotations are optional (taps = 1, null weights, null tables).
// Everything is float; one rounding at each store.
//
// A warp takes ONE head (a query, key or value head) of a tile of consecutive tokens; a lane holds the pairs
// (2i, 2i + 1), i = lane, lane + 32, ..., of that head in registers from the convolution to the store, so nothing
// waits on another warp.  A block is four heads.  Two forms:
//   head_prep_kernel       any number of taps and any head sizes; one token a warp when a step has few (decoding:
//                          every (token, head) its own warp, which also moves the convolution's state on), else
//                          eight in turn with the head's weights waiting in shared memory, taps major
//   head_prep_tile_kernel  steps of many tokens, 1 to 4 taps, even head sizes: the taps and the pairs per lane are
//                          template parameters, HP_TILE tokens a warp, the window of earlier inputs in registers
// After a step that is not one token per sequence tb_conv_roll moves the state on.
#include "common.cuh"

constexpr int HP_WARPS = 4;
constexpr int HP_PAIRS = 4;      // pairs per lane: heads of up to 256 entries
constexpr int HP_TILE = 4;       // tokens a warp takes in the form for prompts

struct HeadPrepArgs {
    const void* z;          // [nt, ldz]  q | k | v as the product left them
    const float* conv;      // [C, taps] or null
    float* state;           // [slots, state_pitch]: [taps - 1, C]
    long long state_pitch;
    const float* wq;        // [dk] or null
    const float* wk;
    const float* temp;      // [nh] or null
    const float* cosT;      // [positions, rdims / 2]
    const float* sinT;
    const float* vcos;      // [positions, dv / 2] or null
    const float* vsin;
    void* qout;             // [nt, nh * dk]
    void* kc;               // [pages, nkvh, TB_PAGE, dk] or null (a run that reads another run's cache)
    void* vc;
    const int* tok_seq;
    const int* tok_pos;
    const int* seq_start;
    const int* slots;
    const int* page_table;
    int max_pages, ldz, nt, nh, nkvh, dk, dv, rdims, taps, decode, tok_tile, staged;
    float eps;
    float* vfirst;          // [nt, nkvh * dv] or null: the values of the blend's source
    const float* vmix;      // one number, or null
};

// two neighbouring entries, as one access where the layout allows it
template <typename T, bool VEC>
__device__ __forceinline__ void ld2(const T* p, bool two, float& x0, float& x1) {
    if constexpr (VEC) {
        if constexpr (sizeof(T) == 2) {
            const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
            x0 = f.x;
            x1 = f.y;
        } else {
            const float2 f = *reinterpret_cast<const float2*>(p);
            x0 = f.x;
            x1 = f.y;
        }
    } else {
        x0 = ldf(p);
        x1 = two ? ldf(p + 1) : 0.f;
    }
}
template <typename T, bool VEC>
__device__ __forceinline__ void st2(T* p, bool two, float x0, float x1) {
    if constexpr (VEC) {
        if constexpr (sizeof(T) == 2) *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(x0, x1);
        else *reinterpret_cast<float2*>(p) = make_float2(x0, x1);
    } else {
        stf(p, x0);
        if (two) stf(p + 1, x1);
    }
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(HP_WARPS * 32) head_prep_kernel(const HeadPrepArgs a) {
    pdl_sync();
    extern __shared__ __align__(16) float w_s[];       // [HP_WARPS][taps][dmax] when staged
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int h = blockIdx.y * HP_WARPS + warp;
    if (h >= a.nh + 2 * a.nkvh) return;
    const int C = (a.nh + a.nkvh) * a.dk + a.nkvh * a.dv;
    const int kind = h < a.nh ? 0 : h < a.nh + a.nkvh ? 1 : 2;             // query, key, value
    const int dim = kind == 2 ? a.dv : a.dk;
    const int coff = kind == 2 ? (a.nh + a.nkvh) * a.dk + (h - a.nh - a.nkvh) * a.dv : h * a.dk;
    if ((kind == 1 && !a.kc) || (kind == 2 && !a.vc)) {
        if (!(a.decode && a.conv && a.taps > 1)) return;                   // nothing to write, no state to move on
    }
    const int dmax = a.dk > a.dv ? a.dk : a.dv;
    const bool conv = a.conv != nullptr;        // one tap: a weight per channel, no state
    float* ws = w_s + (size_t)warp * a.taps * dmax;
    if (conv && a.staged) {
        for (int e = lane; e < dim * a.taps; e += 32) {
            const int c = e / a.taps, j = e - c * a.taps;
            ws[j * dmax + c] = a.conv[(size_t)(coff + c) * a.taps + j];
        }
        __syncwarp();
    }
    const T* z = static_cast<const T*>(a.z);
    const float* w = kind == 0 ? a.wq : kind == 1 ? a.wk : nullptr;
    const int half = kind == 2 ? (a.vcos ? a.dv / 2 : 0) : a.rdims / 2;
    const float* cosT = kind == 2 ? a.vcos : a.cosT;
    const float* sinT = kind == 2 ? a.vsin : a.sinT;
    const int t_end = min(a.nt, (int)(blockIdx.x + 1) * a.tok_tile);
    for (int t = blockIdx.x * a.tok_tile; t < t_end; ++t) {
        const int b = a.tok_seq[t], pos = a.tok_pos[t];
        const int tl = t - a.seq_start[b];
        float* st = a.state ? a.state + (size_t)a.slots[b] * a.state_pitch : nullptr;
        float x0[HP_PAIRS], x1[HP_PAIRS];
        float ss = 0.f;
#pragma unroll
        for (int r = 0; r < HP_PAIRS; ++r) {
            const int i = lane + 32 * r;
            x0[r] = x1[r] = 0.f;
            if (2 * i >= dim) continue;
            const bool two = 2 * i + 1 < dim;
            const int c = coff + 2 * i;
            float o0, o1;
            ld2<T, VEC>(z + (size_t)t * a.ldz + c, two, o0, o1);
            float a0 = o0, a1 = o1;
            if (conv) {
                a0 = a1 = 0.f;
                for (int j = 0; j < a.taps; ++j) {
                    const int back = a.taps - 1 - j;
                    float v0, v1;
                    if (back == 0) {
                        v0 = o0;
                        v1 = o1;
                    } else if (tl - back >= 0) {
                        ld2<T, VEC>(z + (size_t)(t - back) * a.ldz + c, two, v0, v1);
                    } else {
                        const float* sp = st + (size_t)(a.taps - 1 + tl - back) * C + c;
                        v0 = sp[0];
                        v1 = two ? sp[1] : 0.f;
                    }
                    float w0, w1;
                    if (a.staged) {
                        w0 = ws[j * dmax + 2 * i];
                        w1 = two ? ws[j * dmax + 2 * i + 1] : 0.f;
                    } else {
                        w0 = a.conv[(size_t)c * a.taps + j];
                        w1 = two ? a.conv[(size_t)(c + 1) * a.taps + j] : 0.f;
                    }
                    a0 += w0 * v0;
                    a1 += w1 * v1;
                }
                if (a.decode && a.taps > 1) {      // one token of this sequence in the step: its state moves on by one input
                    for (int k = 0; k + 2 < a.taps; ++k) {
                        st[(size_t)k * C + c] = st[(size_t)(k + 1) * C + c];
                        if (two) st[(size_t)k * C + c + 1] = st[(size_t)(k + 1) * C + c + 1];
                    }
                    st[(size_t)(a.taps - 2) * C + c] = o0;
                    if (two) st[(size_t)(a.taps - 2) * C + c + 1] = o1;
                }
            }
            x0[r] = a0;
            x1[r] = a1;
            ss += a0 * a0 + a1 * a1;
        }
        if (kind == 2 && a.vfirst) {
            float* vf = a.vfirst + ((size_t)t * a.nkvh + (h - a.nh - a.nkvh)) * a.dv;
            const float lam = a.vmix ? *a.vmix : 0.f;
#pragma unroll
            for (int r = 0; r < HP_PAIRS; ++r) {
                const int i = lane + 32 * r;
                if (2 * i >= dim) continue;
                const bool two = 2 * i + 1 < dim;
                if (a.vmix) {
                    x0[r] = (1.f - lam) * x0[r] + lam * vf[2 * i];
                    if (two) x1[r] = (1.f - lam) * x1[r] + lam * vf[2 * i + 1];
                } else {
                    vf[2 * i] = x0[r];
                    if (two) vf[2 * i + 1] = x1[r];
                }
            }
        }
        T* dst;
        if (kind == 0) {
            dst = static_cast<T*>(a.qout) + ((size_t)t * a.nh + h) * a.dk;
        } else {
            T* base = static_cast<T*>(kind == 1 ? a.kc : a.vc);
            if (!base) continue;
            const int page = a.page_table[(size_t)b * a.max_pages + pos / TB_PAGE];
            const int g = kind == 1 ? h - a.nh : h - a.nh - a.nkvh;
            dst = base + (((size_t)page * a.nkvh + g) * TB_PAGE + pos % TB_PAGE) * dim;
        }
        float rs = 1.f;
        if (w) rs = 1.0f / sqrtf(warp_sum(ss) / (float)dim + a.eps);
        if (kind == 0 && a.temp) rs *= a.temp[h];
#pragma unroll
        for (int r = 0; r < HP_PAIRS; ++r) {
            const int i = lane + 32 * r;
            if (2 * i >= dim) continue;
            const bool two = 2 * i + 1 < dim;
            float y0 = x0[r] * rs, y1 = x1[r] * rs;
            if (w) {
                y0 *= w[2 * i];
                if (two) y1 *= w[2 * i + 1];
            }
            if (i < half) {
                const float co = cosT[(size_t)pos * half + i], si = sinT[(size_t)pos * half + i];
                const float r0 = y0 * co - y1 * si, r1 = y1 * co + y0 * si;
                y0 = r0;
                y1 = r1;
            }
            st2<T, VEC>(dst + 2 * i, two, y0, y1);
        }
    }
}

// The form for prompts: the same warp per head and tile of tokens, with the taps and the pairs per lane known to the
// compiler.  The head's convolution weights sit in registers, the tile's rows are all asked for before the first is
// used, and the last TAPS - 1 inputs slide along in registers, so every projected value is read once.  Where a
// sequence's portion starts inside the tile the window is filled from that sequence's state.  Needs even head
// sizes (pairs as one access).  TAPS = 1 with no weights is the plain copy.
template <typename T, int TAPS, int PAIRS, int TILE>
__global__ void __launch_bounds__(HP_WARPS * 32, PAIRS <= 2 ? 6 : 3) head_prep_tile_kernel(const HeadPrepArgs a) {
    pdl_sync();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int h = blockIdx.y * HP_WARPS + warp;
    if (h >= a.nh + 2 * a.nkvh) return;
    const int C = (a.nh + a.nkvh) * a.dk + a.nkvh * a.dv;
    const int kind = h < a.nh ? 0 : h < a.nh + a.nkvh ? 1 : 2;             // query, key, value
    const int dim = kind == 2 ? a.dv : a.dk;
    const int coff = kind == 2 ? (a.nh + a.nkvh) * a.dk + (h - a.nh - a.nkvh) * a.dv : h * a.dk;
    if ((kind == 1 && !a.kc) || (kind == 2 && !a.vc)) return;
    constexpr int HIST = TAPS > 1 ? TAPS - 1 : 1;
    float wr[PAIRS][2 * TAPS];                      // wr[r][e * TAPS + j]: entry 2i + e of the head, tap j
#pragma unroll
    for (int r = 0; r < PAIRS; ++r) {
        const int i = lane + 32 * r;
        if (a.conv && 2 * i < dim) {                  // a pair's 2 TAPS weights lie together: 8 bytes at a time
            const float2* wp = reinterpret_cast<const float2*>(a.conv + (size_t)(coff + 2 * i) * TAPS);
#pragma unroll
            for (int k = 0; k < TAPS; ++k) {
                const float2 f = __ldg(wp + k);
                wr[r][2 * k] = f.x;
                wr[r][2 * k + 1] = f.y;
            }
        } else {
#pragma unroll
            for (int k = 0; k < 2 * TAPS; ++k) wr[r][k] = (k % TAPS == TAPS - 1) ? 1.f : 0.f;
        }
    }
    const T* z = static_cast<const T*>(a.z);
    const float* w = kind == 0 ? a.wq : kind == 1 ? a.wk : nullptr;
    const int half = kind == 2 ? (a.vcos ? a.dv / 2 : 0) : a.rdims / 2;
    const float* cosT = kind == 2 ? a.vcos : a.cosT;
    const float* sinT = kind == 2 ? a.vsin : a.sinT;
    float nw0[PAIRS], nw1[PAIRS];                     // the norm's weights of this lane's entries
#pragma unroll
    for (int r = 0; r < PAIRS; ++r) {
        const int i = lane + 32 * r;
        nw0[r] = (w && 2 * i < dim) ? w[2 * i] : 1.f;
        nw1[r] = (w && 2 * i < dim) ? w[2 * i + 1] : 1.f;
    }
    const float temp_h = (kind == 0 && a.temp) ? a.temp[h] : 1.f;
    const int t0 = blockIdx.x * TILE;
    float2 own[TILE][PAIRS];
#pragma unroll
    for (int tt = 0; tt < TILE; ++tt)
#pragma unroll
        for (int r = 0; r < PAIRS; ++r) {
            const int i = lane + 32 * r;
            own[tt][r] = make_float2(0.f, 0.f);
            if (t0 + tt < a.nt && 2 * i < dim)
                ld2<T, true>(z + (size_t)(t0 + tt) * a.ldz + coff + 2 * i, true, own[tt][r].x, own[tt][r].y);
        }
    // The rows before the tile are asked for with the tile's own, before it is known whether they are the same
    // sequence's: where they are not, the state's rows take their place below.
    float2 hist[HIST][PAIRS];                          // hist[k]: the input k + 1 tokens back
#pragma unroll
    for (int k = 0; k < HIST; ++k)
#pragma unroll
        for (int r = 0; r < PAIRS; ++r) {
            const int i = lane + 32 * r;
            hist[k][r] = make_float2(0.f, 0.f);
            if (TAPS > 1 && 2 * i < dim && t0 - (k + 1) >= 0)
                ld2<T, true>(z + (size_t)(t0 - (k + 1)) * a.ldz + coff + 2 * i, true, hist[k][r].x, hist[k][r].y);
        }
    // where each of the tile's tokens stands: lane tt looks it up, every lane asks that lane
    static_assert(TILE <= 32, "a lane per token of the tile");
    int my_pos = 0, my_page = 0, my_slot = 0, my_tl = 1 << 20;
    if (lane < TILE && t0 + lane < a.nt) {
        const int b = a.tok_seq[t0 + lane];
        my_pos = a.tok_pos[t0 + lane];
        my_tl = t0 + lane - a.seq_start[b];           // 0: the first token of its sequence's portion
        my_slot = a.slots ? a.slots[b] : 0;
        if (kind != 0) my_page = a.page_table[(size_t)b * a.max_pages + my_pos / TB_PAGE];
    }
    if constexpr (TAPS > 1) {
        const int tl = __shfl_sync(0xffffffffu, my_tl, 0);
        if (tl < TAPS - 1) {                           // the portion starts so shortly before the tile: the older inputs are state
            const float* st = a.state + (size_t)__shfl_sync(0xffffffffu, my_slot, 0) * a.state_pitch;
#pragma unroll
            for (int k = 0; k < TAPS - 1; ++k)
#pragma unroll
                for (int r = 0; r < PAIRS; ++r) {
                    const int i = lane + 32 * r;
                    const int back = k + 1;
                    if (2 * i >= dim || tl - back >= 0) continue;
                    const float* sp = st + (size_t)(TAPS - 1 + tl - back) * C + coff + 2 * i;
                    hist[k][r] = make_float2(sp[0], sp[1]);
                }
        }
    }
#pragma unroll
    for (int tt = 0; tt < TILE; ++tt) {
        const int t = t0 + tt;
        if (t >= a.nt) break;
        const int pos = __shfl_sync(0xffffffffu, my_pos, tt);
        if constexpr (TAPS > 1) {
            const int first = __shfl_sync(0xffffffffu, my_tl, tt) == 0, slot = __shfl_sync(0xffffffffu, my_slot, tt);
            if (tt > 0 && first) {                      // another sequence's portion starts here
                const float* st = a.state + (size_t)slot * a.state_pitch;
#pragma unroll
                for (int k = 0; k < TAPS - 1; ++k)
#pragma unroll
                    for (int r = 0; r < PAIRS; ++r) {
                        const int i = lane + 32 * r;
                        if (2 * i >= dim) continue;
                        const float* sp = st + (size_t)(TAPS - 2 - k) * C + coff + 2 * i;
                        hist[k][r] = make_float2(sp[0], sp[1]);
                    }
            }
        }
        float x0[PAIRS], x1[PAIRS];
        float ss = 0.f;
#pragma unroll
        for (int r = 0; r < PAIRS; ++r) {
            float a0 = wr[r][TAPS - 1] * own[tt][r].x, a1 = wr[r][2 * TAPS - 1] * own[tt][r].y;
            if constexpr (TAPS > 1) {
#pragma unroll
                for (int j = 0; j < TAPS - 1; ++j) {
                    a0 += wr[r][j] * hist[TAPS - 2 - j][r].x;
                    a1 += wr[r][TAPS + j] * hist[TAPS - 2 - j][r].y;
                }
            }
            x0[r] = a0;
            x1[r] = a1;
            ss += a0 * a0 + a1 * a1;
        }
        if (kind == 2 && a.vfirst) {
            float* vf = a.vfirst + ((size_t)t * a.nkvh + (h - a.nh - a.nkvh)) * a.dv;
            const float lam = a.vmix ? __ldg(a.vmix) : 0.f;
#pragma unroll
            for (int r = 0; r < PAIRS; ++r) {
                const int i = lane + 32 * r;
                if (2 * i >= dim) continue;
                float2* at = reinterpret_cast<float2*>(vf + 2 * i);
                if (a.vmix) {
                    const float2 f = *at;
                    x0[r] = (1.f - lam) * x0[r] + lam * f.x;
                    x1[r] = (1.f - lam) * x1[r] + lam * f.y;
                } else {
                    *at = make_float2(x0[r], x1[r]);
                }
            }
        }
        if constexpr (TAPS > 1) {
#pragma unroll
            for (int k = TAPS - 2; k > 0; --k)
#pragma unroll
                for (int r = 0; r < PAIRS; ++r) hist[k][r] = hist[k - 1][r];
#pragma unroll
            for (int r = 0; r < PAIRS; ++r) hist[0][r] = own[tt][r];
        }
        T* dst;
        if (kind == 0) {
            dst = static_cast<T*>(a.qout) + ((size_t)t * a.nh + h) * a.dk;
        } else {
            const int page = __shfl_sync(0xffffffffu, my_page, tt);
            const int g = kind == 1 ? h - a.nh : h - a.nh - a.nkvh;
            dst = static_cast<T*>(kind == 1 ? a.kc : a.vc) + (((size_t)page * a.nkvh + g) * TB_PAGE + pos % TB_PAGE) * dim;
        }
        float rs = 1.f;
        if (w) rs = 1.0f / sqrtf(warp_sum(ss) / (float)dim + a.eps);
        rs *= temp_h;
#pragma unroll
        for (int r = 0; r < PAIRS; ++r) {
            const int i = lane + 32 * r;
            if (2 * i >= dim) continue;
            float y0 = x0[r] * rs * nw0[r], y1 = x1[r] * rs * nw1[r];
            if (i < half) {
                const float co = __ldg(cosT + (size_t)pos * half + i), si = __ldg(sinT + (size_t)pos * half + i);
                const float r0 = y0 * co - y1 * si, r1 = y1 * co + y0 * si;
                y0 = r0;
                y1 = r1;
            }
            st2<T, true>(dst + 2 * i, true, y0, y1);
        }
    }
}

template <typename T, int TAPS>
static void head_prep_tile_launch(const HeadPrepArgs& a, dim3 grid, int dmax, cudaStream_t s) {
    constexpr int TILE = HP_TILE;
    if (dmax <= 64) TB_LAUNCH((head_prep_tile_kernel<T, TAPS, 1, TILE>), grid, HP_WARPS * 32, 0, s, a);
    else if (dmax <= 128) TB_LAUNCH((head_prep_tile_kernel<T, TAPS, 2, TILE>), grid, HP_WARPS * 32, 0, s, a);
    else TB_LAUNCH((head_prep_tile_kernel<T, TAPS, 4, TILE>), grid, HP_WARPS * 32, 0, s, a);
}

extern "C" {
#define TB_HEAD_PREP(SFX, T)                                                                                          \
    int tb_head_prep_##SFX(const void* z, int ldz, const float* conv, float* state, long long state_pitch,            \
                           const float* wq, const float* wk, const float* temp, float eps, const float* cosT,         \
                           const float* sinT, const float* vcos, const float* vsin, void* qout, void* kc, void* vc,   \
                           const int* tok_seq, const int* tok_pos, const int* seq_start, const int* slots,            \
                           const int* page_table, int max_pages, int nt, int nh, int nkvh, int dk, int dv, int rdims, \
                           int taps, int decode, float* vfirst, const float* vmix, cudaStream_t s) {                  \
        if (nt < 0 || nh <= 0 || nkvh <= 0 || dk <= 0 || dv <= 0 || rdims < 0 || rdims > dk || rdims % 2)             \
            return TB_ERR_ARG;                                                                                        \
        if (taps < 1 || taps > 16 || (conv && taps > 1 && !state) || (rdims && (!cosT || !sinT))) return TB_ERR_ARG;  \
        if (vcos && (dv % 2 || !vsin)) return TB_ERR_ARG;                                                             \
        if (vmix && !vfirst) return TB_ERR_ARG;                                                                       \
        const long long C = (long long)(nh + nkvh) * dk + (long long)nkvh * dv;                                       \
        if (ldz < C || (conv && taps > 1 && state_pitch < (taps - 1) * C)) return TB_ERR_ARG;                         \
        if (dk > 64 * HP_PAIRS || dv > 64 * HP_PAIRS) return TB_ERR_UNSUPPORTED;                                      \
        if (nt == 0) return 0;                                                                                        \
        const int heads = nh + 2 * nkvh, groups = (heads + HP_WARPS - 1) / HP_WARPS;                                  \
        /* the general form: eight tokens a warp in a step of many, else one */                                        \
        const int tile = nt >= 64 ? 8 : 1;                                                                            \
        size_t smem = conv ? (size_t)HP_WARPS * taps * (dk > dv ? dk : dv) * 4 : 0;                       \
        const int staged = smem > 0 && smem <= 48 * 1024 && tile > 1;                                                 \
        if (!staged) smem = 0;                                                                                        \
        HeadPrepArgs a{z, conv, state, state_pitch, wq, wk, temp, cosT, sinT, vcos, vsin, qout, kc, vc, tok_seq,      \
                       tok_pos, seq_start, slots, page_table, max_pages, ldz, nt, nh, nkvh, dk, dv, rdims, taps,      \
                       decode ? 1 : 0, tile, staged, eps, vfirst, vmix};                                              \
        const size_t es = sizeof(T);                                                                                  \
        const bool vec = dk % 2 == 0 && dv % 2 == 0 && ldz % 2 == 0 && (uintptr_t)z % (2 * es) == 0 &&                \
                         (uintptr_t)qout % (2 * es) == 0 && (uintptr_t)kc % (2 * es) == 0 &&                          \
                         (uintptr_t)vc % (2 * es) == 0 && (uintptr_t)vfirst % 8 == 0;                                 \
        const int taps_eff = conv ? taps : 1;                                                                         \
        if (vec && tile == 8 && !decode && taps_eff <= 4 && (uintptr_t)conv % 8 == 0) {                               \
            const int dmax = dk > dv ? dk : dv;                                                                       \
            const dim3 grid((nt + HP_TILE - 1) / HP_TILE, groups);                                                    \
            a.taps = taps_eff;                                                                                        \
            if (taps_eff == 1) head_prep_tile_launch<T, 1>(a, grid, dmax, s);                                         \
            else if (taps_eff == 2) head_prep_tile_launch<T, 2>(a, grid, dmax, s);                                    \
            else if (taps_eff == 3) head_prep_tile_launch<T, 3>(a, grid, dmax, s);                                    \
            else head_prep_tile_launch<T, 4>(a, grid, dmax, s);                                                       \
            return tb_last_error();                                                                                   \
        }                                                                                                             \
        const dim3 grid((nt + tile - 1) / tile, groups);                                                              \
        if (vec) TB_LAUNCH((head_prep_kernel<T, true>), grid, HP_WARPS * 32, smem, s, a);                             \
        else TB_LAUNCH((head_prep_kernel<T, false>), grid, HP_WARPS * 32, smem, s, a);                                \
        return tb_last_error();                                                                                       \
    }
TB_HEAD_PREP(f32, float)
TB_HEAD_PREP(bf16, __nv_bfloat16)
}

#include "tape.h"
TB_TAPE_REGISTER(tb_head_prep_f32)
TB_TAPE_REGISTER(tb_head_prep_bf16)
