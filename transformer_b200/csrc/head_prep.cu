// What lies between the merged q-k-v product and the attention for a mixer with short convolutions on its
// projections, a norm per head and rotated values, in one kernel:
//
//   u = causal convolution over time of every channel of [q | k | v]     (taps wide, the last inputs kept per sequence)
//   q_h <- u_q,h / rms(u_q,h) * wq * temp_h,   k_g <- u_k,g / rms(u_k,g) * wk        (weights of one head, shared)
//   the first rdims entries of every query and key head turn by position * f_i in the pairs (2i, 2i + 1)
//   every pair (2m, 2m + 1) of a value head turns by position * g_m
//   queries go to `qout`, keys and values into the paged cache
//
// The convolution, the norm, the temperature and the rotations are optional (taps = 1, null weights, null tables).
// Everything is float; one rounding at each store.  One block per token: the convolved row waits in shared memory,
// then a warp takes a head at a time.  In a step of one token per sequence the block also moves the convolution's
// state on; after any other step tb_causal_conv's roll kernel does.
#include "common.cuh"

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
    int max_pages, ldz, nh, nkvh, dk, dv, rdims, taps, decode;
    float eps;
};

template <typename T>
__global__ void __launch_bounds__(128) head_prep_kernel(const HeadPrepArgs a) {
    pdl_sync();
    extern __shared__ __align__(16) float u_s[];
    const int t = blockIdx.x;
    const int C = (a.nh + a.nkvh) * a.dk + a.nkvh * a.dv;
    const int b = a.tok_seq[t], pos = a.tok_pos[t];
    const int tl = t - a.seq_start[b];
    const T* z = static_cast<const T*>(a.z);
    float* st = a.state ? a.state + (size_t)a.slots[b] * a.state_pitch : nullptr;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        const float own = ldf(z + (size_t)t * a.ldz + c);
        float acc = own;
        if (a.conv) {
            acc = 0.f;
            for (int j = 0; j < a.taps; ++j) {
                const int back = a.taps - 1 - j;
                float v;
                if (back == 0) v = own;
                else if (tl - back >= 0) v = ldf(z + (size_t)(t - back) * a.ldz + c);
                else v = st[(size_t)(a.taps - 1 + tl - back) * C + c];
                acc += a.conv[(size_t)c * a.taps + j] * v;
            }
            if (a.decode) {
                for (int i = 0; i + 2 < a.taps; ++i) st[(size_t)i * C + c] = st[(size_t)(i + 1) * C + c];
                if (a.taps > 1) st[(size_t)(a.taps - 2) * C + c] = own;
            }
        }
        u_s[c] = acc;
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int page = a.page_table[(size_t)b * a.max_pages + pos / TB_PAGE];
    const int prow = pos % TB_PAGE;
    const int heads = a.nh + 2 * a.nkvh;
    const int half = a.rdims / 2;
    for (int h = warp; h < heads; h += nw) {
        if (h < a.nh + a.nkvh) {
            const bool is_q = h < a.nh;
            const float* src = u_s + (size_t)h * a.dk;
            const float* w = is_q ? a.wq : a.wk;
            float rs = 1.f;
            if (w) {
                float ss = 0.f;
                for (int c = lane; c < a.dk; c += 32) ss += src[c] * src[c];
                rs = 1.0f / sqrtf(warp_sum(ss) / (float)a.dk + a.eps);
            }
            if (is_q && a.temp) rs *= a.temp[h];
            T* dst;
            if (is_q) dst = static_cast<T*>(a.qout) + ((size_t)t * a.nh + h) * a.dk;
            else if (a.kc) dst = static_cast<T*>(a.kc) + (((size_t)page * a.nkvh + (h - a.nh)) * TB_PAGE + prow) * a.dk;
            else continue;
            for (int i = lane; 2 * i < a.dk; i += 32) {
                float x0 = src[2 * i] * rs, x1 = 2 * i + 1 < a.dk ? src[2 * i + 1] * rs : 0.f;
                if (w) {
                    x0 *= w[2 * i];
                    if (2 * i + 1 < a.dk) x1 *= w[2 * i + 1];
                }
                if (i < half) {
                    const float co = a.cosT[(size_t)pos * half + i], si = a.sinT[(size_t)pos * half + i];
                    const float r0 = x0 * co - x1 * si, r1 = x1 * co + x0 * si;
                    x0 = r0;
                    x1 = r1;
                }
                stf(dst + 2 * i, x0);
                if (2 * i + 1 < a.dk) stf(dst + 2 * i + 1, x1);
            }
        } else {
            if (!a.vc) continue;
            const int g = h - a.nh - a.nkvh;
            const float* src = u_s + (size_t)(a.nh + a.nkvh) * a.dk + (size_t)g * a.dv;
            T* dst = static_cast<T*>(a.vc) + (((size_t)page * a.nkvh + g) * TB_PAGE + prow) * a.dv;
            const int vhalf = a.dv / 2;
            for (int i = lane; 2 * i < a.dv; i += 32) {
                float x0 = src[2 * i], x1 = 2 * i + 1 < a.dv ? src[2 * i + 1] : 0.f;
                if (a.vcos && i < vhalf) {
                    const float co = a.vcos[(size_t)pos * vhalf + i], si = a.vsin[(size_t)pos * vhalf + i];
                    const float r0 = x0 * co - x1 * si, r1 = x1 * co + x0 * si;
                    x0 = r0;
                    x1 = r1;
                }
                stf(dst + 2 * i, x0);
                if (2 * i + 1 < a.dv) stf(dst + 2 * i + 1, x1);
            }
        }
    }
}

extern "C" {
#define TB_HEAD_PREP(SFX, T)                                                                                          \
    int tb_head_prep_##SFX(const void* z, int ldz, const float* conv, float* state, long long state_pitch,            \
                           const float* wq, const float* wk, const float* temp, float eps, const float* cosT,         \
                           const float* sinT, const float* vcos, const float* vsin, void* qout, void* kc, void* vc,   \
                           const int* tok_seq, const int* tok_pos, const int* seq_start, const int* slots,            \
                           const int* page_table, int max_pages, int nt, int nh, int nkvh, int dk, int dv, int rdims, \
                           int taps, int decode, cudaStream_t s) {                                                    \
        if (nt < 0 || nh <= 0 || nkvh <= 0 || dk <= 0 || dv <= 0 || rdims < 0 || rdims > dk || rdims % 2)             \
            return TB_ERR_ARG;                                                                                        \
        if (taps < 1 || taps > 16 || (conv && taps > 1 && !state) || (rdims && (!cosT || !sinT))) return TB_ERR_ARG;  \
        if (vcos && (dv % 2 || !vsin)) return TB_ERR_ARG;                                                             \
        const long long C = (long long)(nh + nkvh) * dk + (long long)nkvh * dv;                                       \
        if (ldz < C || (conv && taps > 1 && state_pitch < (taps - 1) * C)) return TB_ERR_ARG;                         \
        if (C * 4 > 48 * 1024) return TB_ERR_UNSUPPORTED;                                                             \
        if (nt == 0) return 0;                                                                                        \
        HeadPrepArgs a{z, conv, state, state_pitch, wq, wk, temp, cosT, sinT, vcos, vsin, qout, kc, vc, tok_seq,      \
                       tok_pos, seq_start, slots, page_table, max_pages, ldz, nh, nkvh, dk, dv, rdims, taps,          \
                       decode ? 1 : 0, eps};                                                                          \
        TB_LAUNCH((head_prep_kernel<T>), nt, 128, (size_t)C * 4, s, a);                                               \
        return tb_last_error();                                                                                       \
    }
TB_HEAD_PREP(f32, float)
TB_HEAD_PREP(bf16, __nv_bfloat16)
}

#include "tape.h"
TB_TAPE_REGISTER(tb_head_prep_f32)
TB_TAPE_REGISTER(tb_head_prep_bf16)
