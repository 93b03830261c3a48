// A gated delta rule with one decay per key channel, token by token, state in float.
//
// Per head h (its queries and keys come from key head h / (H / G)), with a state S [dim, vdim] that is zero when a
// sequence starts:
//
//   S <- diag(g_t) S;    u = beta_t (v_t - S^T k_t);    S <- S + k_t u^T;    o_t = S^T q_t
//
// What enters the recurrence is made by the kernel before it (delta_prep_kernel), in float on both paths:
//   q, k, v = silu(causal convolution over time of the step's projections, per channel, `taps` wide);
//   q and k unit vectors per head (x / sqrt(sum x^2 + 1e-6)), q also times dim^-1/2;
//   g = exp(-exp(A_log[h]) * softplus(a + dt_bias))  per head and key channel;   beta = sigmoid(b)  per head.
// The last taps - 1 inputs of every channel are state as well, so that a sequence may arrive in pieces.
//
// State of one slot (floats): S [H][dim][vdim], then the convolution's inputs [taps - 1][C], C = 2 G dim + H vdim.
//
// The scan reads o_t = (gS)^T q + u (k . q) from the SAME pass over the state that gives (gS)^T k, so a token costs
// one pass for the two sums, a reduction over the lanes that share a column, and one pass for the update.
// Work split of the scan: a block = one sequence x one head x 8 to 32 columns of the state; a column belongs to
// four to sixteen adjacent lanes, which split the rows (chunks of four rows, interleaved), RPT rows each in
// registers.  The first kernel leaves one contiguous record per (token, head), so the scan's staging is a plain
// 16-byte copy.
#include "common.cuh"
#include "attention_prefill.cuh"        // cp_async16, cp_async_commit, cp_async_wait

#define CD_UNIT_EPS 1e-6f
#define CD_THREADS 128
#define CD_MAX_TAPS 16
#define CD_TOK 4            // tokens staged in shared memory per barrier

// Rows that the scan's lanes cover for heads of `dim` key channels (dim rounded up to what its forms take), and the
// lanes that share a column.  A record of one (token, head) for the scan:  q [DP] | k [DP] | g [DP] | beta, k.q, 0, 0
// (rows beyond dim: q = k = 0, g = 1), then separately v [VP] with VP = vdim rounded up to 32.
__host__ __device__ inline int cd_rows(int dim) { return dim <= 16 ? 16 : dim <= 32 ? 32 : dim <= 64 ? 64 : dim <= 128 ? 128 : 256; }
__host__ __device__ inline int cd_record(int dim) { return 3 * cd_rows(dim) + 4; }
__host__ __device__ inline int cd_vpitch(int vdim) { return (vdim + 31) / 32 * 32; }

struct DeltaPrepArgs {
    const void* z;          // [nt, ldz]: q (G dim) | k (G dim) | v (H vdim) | whatever else the product made
    const float* wconv;     // [C, taps], the last column is the current token's
    float* state;           // [slots, state_stride]
    const float* a;         // [nt, H dim]  pre-activation of the decay
    const float* dt_bias;   // [H dim]
    const float* A_log;     // [H]
    const float* bz;        // [nt, H]      pre-activation of beta
    float* rec;             // out [nt, H, cd_record(dim)]
    float* vbuf;            // out [nt, H, cd_vpitch(vdim)]
    const int* tok_seq;
    const int* seq_start;
    const int* slots;
    long long state_stride, conv_offset;
    int ldz, G, H, dim, vdim, taps, update_state;
    int lda, ldb;           // row pitches of a and bz (floats)
    int head_decay;         // 1: one decay per head: a [nt, H], dt_bias [H], the same g for every key channel
};

__device__ __forceinline__ float cd_softplus(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }

// A block = up to four consecutive tokens of the step x one key head g: the convolutions of that head's query and
// key channels and of the value channels of the heads that read it (a thread keeps a channel's taps for the block's
// tokens), a warp per token for the two unit norms and k . q, then all threads write the group's records: q, k,
// decays, betas, and the values.  Four tokens a block for prompts, one for steps of few tokens (more blocks).
#define CD_PT 4
template <typename T>
__global__ void __launch_bounds__(32 * CD_PT) delta_prep_kernel(const DeltaPrepArgs p, int nt, int pt) {
    pdl_sync();
    extern __shared__ float y_all[];    // [pt][2 dim + per vdim] the convolution's outputs after silu: q, k, v of the group
    __shared__ float stats[CD_PT][3];   // per token: the query's and the key's multiplier, k . q
    const int tb = blockIdx.x * pt, g = blockIdx.y;
    const int ntok = min(pt, nt - tb);
    const int dim = p.dim, vdim = p.vdim, gd = p.G * dim, per = p.H / p.G, taps = p.taps;
    const int C = 2 * gd + p.H * vdim, n_loc = 2 * dim + per * vdim;
    const int DP = cd_rows(dim), PER = cd_record(dim), VP = cd_vpitch(vdim);
    const T* z = static_cast<const T*>(p.z);
    int li[CD_PT];                      // index of each token among its sequence's tokens of the step
    float* cs[CD_PT];                   // its sequence's convolution state [taps - 1][C]
#pragma unroll
    for (int tt = 0; tt < CD_PT; ++tt) {
        li[tt] = 0;
        cs[tt] = nullptr;
        if (tt < ntok) {
            const int b = p.tok_seq[tb + tt];
            li[tt] = tb + tt - p.seq_start[b];
            cs[tt] = p.state + (size_t)p.slots[b] * p.state_stride + p.conv_offset;
        }
    }
    for (int i = threadIdx.x; i < n_loc; i += blockDim.x) {
        // local entry i -> channel c of the row
        const int c = i < dim ? g * dim + i : i < 2 * dim ? gd + g * dim + (i - dim) : 2 * gd + g * per * vdim + (i - 2 * dim);
        float w[CD_MAX_TAPS];
        for (int j = 0; j < taps; ++j) w[j] = p.wconv[(size_t)c * taps + j];
#pragma unroll
        for (int tt = 0; tt < CD_PT; ++tt) {
            if (tt >= ntok) break;
            const int t = tb + tt;
            float acc = 0.f, old[CD_MAX_TAPS];
            for (int j = 0; j < taps; ++j) {
                const int back = taps - 1 - j, s = li[tt] - back;
                const float x = s >= 0 ? ldf(z + (size_t)(t - back) * p.ldz + c) : cs[tt][(size_t)(taps - 1 + s) * C + c];
                old[j] = x;
                acc += w[j] * x;
            }
            y_all[tt * n_loc + i] = acc / (1.0f + expf(-acc));
            if (p.update_state)     // a step of one token per sequence: this thread alone touches its channel's state
                for (int r = 0; r + 1 < taps; ++r) cs[tt][(size_t)r * C + c] = old[r + 1];
        }
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (warp < ntok) {
        const float* q = y_all + warp * n_loc;
        const float* k = q + dim;
        float sq = 0.f, sk = 0.f, dot = 0.f;
        for (int c = lane; c < dim; c += 32) {
            sq += q[c] * q[c];
            sk += k[c] * k[c];
            dot += q[c] * k[c];
        }
        sq = warp_sum(sq);
        sk = warp_sum(sk);
        dot = warp_sum(dot);
        if (lane == 0) {
            const float iq = rsqrtf((float)dim) / sqrtf(sq + CD_UNIT_EPS), ik = 1.0f / sqrtf(sk + CD_UNIT_EPS);
            stats[warp][0] = iq;
            stats[warp][1] = ik;
            stats[warp][2] = dot * iq * ik;
        }
    }
    __syncthreads();
    // the records of the block's tokens and the group's heads, q | k | g | beta, k.q, 0, 0, and their values: a warp
    // takes one of the four pieces of a (token, head) at a time
    for (int u = warp; u < ntok * per * 4; u += blockDim.x >> 5) {
        const int pair = u >> 2, piece = u & 3;
        const int tt = pair / per, h = pair - tt * per;
        const int t = tb + tt, hh = g * per + h;
        const float* y = y_all + tt * n_loc;
        float* r = p.rec + ((size_t)t * p.H + hh) * PER;
        if (piece == 0) {
            const float iq = stats[tt][0];
            for (int c = lane; c < DP; c += 32) r[c] = c < dim ? y[c] * iq : 0.f;
        } else if (piece == 1) {
            const float ik = stats[tt][1];
            for (int c = lane; c < DP; c += 32) r[DP + c] = c < dim ? y[dim + c] * ik : 0.f;
        } else if (piece == 2) {
            const float rate = expf(p.A_log[hh]);
            if (p.head_decay) {
                const float gh = expf(-rate * cd_softplus(p.a[(size_t)t * p.lda + hh] + p.dt_bias[hh]));
                for (int c = lane; c < DP; c += 32) r[2 * DP + c] = c < dim ? gh : 1.f;
            } else {
                const float* a = p.a + (size_t)t * p.lda + (size_t)hh * dim;
                const float* db = p.dt_bias + (size_t)hh * dim;
                for (int c = lane; c < DP; c += 32) r[2 * DP + c] = c < dim ? expf(-rate * cd_softplus(a[c] + db[c])) : 1.f;
            }
        } else {
            if (lane < 4)
                r[3 * DP + lane] = lane == 0 ? 1.0f / (1.0f + expf(-p.bz[(size_t)t * p.ldb + hh])) : lane == 1 ? stats[tt][2] : 0.f;
            float* vb = p.vbuf + ((size_t)t * p.H + hh) * VP;
            for (int c = lane; c < VP; c += 32) vb[c] = c < vdim ? y[2 * dim + h * vdim + c] : 0.f;
        }
    }
}

// After a step that brought a sequence more than one token: the last taps - 1 inputs of every channel, from the
// step's rows and, where the step was shorter than that, from what the state held.
template <typename T>
__global__ void __launch_bounds__(256) delta_conv_state_kernel(const DeltaPrepArgs p) {
    pdl_sync();
    const int b = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
    const int C = 2 * p.G * p.dim + p.H * p.vdim, keep = p.taps - 1;
    if (c >= C) return;
    const int t0 = p.seq_start[b], n = p.seq_start[b + 1] - t0;
    if (n <= 0) return;
    const T* z = static_cast<const T*>(p.z);
    float* cs = p.state + (size_t)p.slots[b] * p.state_stride + p.conv_offset;
    float fresh[CD_MAX_TAPS];
    for (int r = 0; r < keep; ++r) {
        const int li = n - keep + r;
        fresh[r] = li >= 0 ? ldf(z + (size_t)(t0 + li) * p.ldz + c) : cs[(size_t)(keep + li) * C + c];
    }
    for (int r = 0; r < keep; ++r) cs[(size_t)r * C + c] = fresh[r];
}

struct DeltaScanArgs {
    const float* rec;       // [nt, H, cd_record(dim)]
    const float* vbuf;      // [nt, H, cd_vpitch(vdim)]
    float* state;           // [slots, state_stride], S first
    float* out;             // [nt, H vdim]
    const int* seq_start;
    const int* slots;
    long long state_stride;
    int G, H, dim, vdim;
};

// RPT rows of a column per thread, SPLIT lanes per column: SPLIT * RPT = cd_rows(dim), CD_THREADS / SPLIT columns a
// block.  The records of four tokens at a time are copied to shared memory by cp.async while the four before them
// are computed; one barrier per four tokens.
template <int RPT, int SPLIT>
__global__ void __launch_bounds__(CD_THREADS) delta_scan_kernel(const DeltaScanArgs a) {
    pdl_sync();
    constexpr int DP = RPT * SPLIT;
    constexpr int COLS = CD_THREADS / SPLIT;
    constexpr int PER = 3 * DP + 4;                     // floats of a record
    constexpr int ROW = PER + COLS;                     // a token in shared memory: its record, then v of the block's columns
    constexpr int ROW4 = ROW / 4;
    __shared__ __align__(16) float sm[2][CD_TOK][ROW];
    const int b = blockIdx.x, h = blockIdx.y;
    const int tid = threadIdx.x, part = tid & (SPLIT - 1), cl = tid / SPLIT;
    const int col0 = blockIdx.z * COLS, col = col0 + cl;
    const int dim = a.dim, vdim = a.vdim, H = a.H;
    const bool has_col = col < vdim;
    const int t0 = a.seq_start[b], t1 = a.seq_start[b + 1];
    if (t0 >= t1) return;
    const int VP = cd_vpitch(vdim);
    float* S = a.state + (size_t)a.slots[b] * a.state_stride + (size_t)h * dim * vdim;
    float s[RPT];
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
        const int r = ((i >> 2) * SPLIT + part) * 4 + (i & 3);
        s[i] = (r < dim && has_col) ? S[(size_t)r * vdim + col] : 0.f;
    }
    auto issue = [&](int ts, int par) {
        const int ntok = min(CD_TOK, t1 - ts);
        for (int idx = tid; idx < ntok * ROW4; idx += CD_THREADS) {
            const int tt = idx / ROW4, e4 = idx - tt * ROW4;
            const float* src = e4 < PER / 4 ? a.rec + ((size_t)(ts + tt) * H + h) * PER + e4 * 4
                                            : a.vbuf + ((size_t)(ts + tt) * H + h) * VP + col0 + (e4 - PER / 4) * 4;
            cp_async16((uint32_t)__cvta_generic_to_shared(&sm[par][tt][e4 * 4]), src);
        }
        cp_async_commit();
    };
    issue(t0, 0);
    for (int ts = t0, st = 0; ts < t1; ts += CD_TOK, ++st) {
        const int par = st & 1;
        cp_async_wait<0>();
        __syncthreads();            // this stage has landed for everyone, and everyone is done with the stage before
        if (ts + CD_TOK < t1) issue(ts + CD_TOK, par ^ 1);
        const int ntok = min(CD_TOK, t1 - ts);
        float* o_tok = a.out + ((size_t)ts * H + h) * vdim + col;        // this thread's output of the stage's first token
#pragma unroll
        for (int tt = 0; tt < CD_TOK; ++tt) {
            if (tt >= ntok) break;
            const float* row = &sm[par][tt][0];
            const float4* Q4 = reinterpret_cast<const float4*>(row);
            const float4* K4 = reinterpret_cast<const float4*>(row + DP);
            const float4* G4 = reinterpret_cast<const float4*>(row + 2 * DP);
            float4 kk[RPT / 4];
            float dk[4] = {0.f, 0.f, 0.f, 0.f}, dq[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i4 = 0; i4 < RPT / 4; ++i4) {
                const int ch = i4 * SPLIT + part;
                const float4 q = Q4[ch], k = K4[ch], gg = G4[ch];
                kk[i4] = k;
                float* si = s + i4 * 4;
                si[0] *= gg.x; si[1] *= gg.y; si[2] *= gg.z; si[3] *= gg.w;
                dk[0] += si[0] * k.x; dk[1] += si[1] * k.y; dk[2] += si[2] * k.z; dk[3] += si[3] * k.w;
                dq[0] += si[0] * q.x; dq[1] += si[1] * q.y; dq[2] += si[2] * q.z; dq[3] += si[3] * q.w;
            }
            float sk = (dk[0] + dk[1]) + (dk[2] + dk[3]), sq = (dq[0] + dq[1]) + (dq[2] + dq[3]);
#pragma unroll
            for (int o = 1; o < SPLIT; o <<= 1) {
                sk += __shfl_xor_sync(0xffffffffu, sk, o);
                sq += __shfl_xor_sync(0xffffffffu, sq, o);
            }
            const float u = row[3 * DP] * (row[PER + cl] - sk);         // beta (v - S^T k)
#pragma unroll
            for (int i4 = 0; i4 < RPT / 4; ++i4) {
                float* si = s + i4 * 4;
                si[0] += kk[i4].x * u; si[1] += kk[i4].y * u; si[2] += kk[i4].z * u; si[3] += kk[i4].w * u;
            }
            if (part == 0 && has_col) o_tok[(size_t)tt * H * vdim] = sq + u * row[3 * DP + 1];
        }
    }
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
        const int r = ((i >> 2) * SPLIT + part) * 4 + (i & 3);
        if (r < dim && has_col) S[(size_t)r * vdim + col] = s[i];
    }
}

template <typename T>
static int delta_prep_launch(const DeltaPrepArgs& p, int nt, int B, cudaStream_t s) {
    if (nt < 0 || B < 0 || p.G <= 0 || p.H <= 0 || p.H % p.G || p.dim <= 0 || p.vdim <= 0) return TB_ERR_ARG;
    if (p.taps < 1 || p.taps > CD_MAX_TAPS) return TB_ERR_UNSUPPORTED;
    const int C = 2 * p.G * p.dim + p.H * p.vdim;
    const size_t smem = (size_t)CD_PT * (2 * p.dim + p.H / p.G * p.vdim) * sizeof(float);
    if (smem > 200 * 1024) return TB_ERR_UNSUPPORTED;
    if (nt == 0) return 0;
    static size_t configured = 0;
    if (smem > 48 * 1024 && smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(delta_prep_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = smem;
    }
    const int pt = nt >= 256 ? CD_PT : 1;
    dim3 pgrid((nt + pt - 1) / pt, p.G);
    TB_LAUNCH((delta_prep_kernel<T>), pgrid, 32 * CD_PT, smem, s, p, nt, pt);
    int rc = tb_last_error();
    if (rc || p.update_state || p.taps == 1) return rc;
    dim3 grid(B, (C + 255) / 256);
    TB_LAUNCH((delta_conv_state_kernel<T>), grid, 256, 0, s, p);
    return tb_last_error();
}

static int cd_scan_lanes_override = 0;      // measurements: lanes per column whatever the batch (0: by the rule below)

template <int RPT, int SPLIT>
static void delta_scan_go(const DeltaScanArgs& a, int B, bool early, cudaStream_t s) {
    dim3 grid(B, a.H, (a.vdim + CD_THREADS / SPLIT - 1) / (CD_THREADS / SPLIT));
    if (early)
        TB_LAUNCH((delta_scan_kernel<RPT, SPLIT>), grid, CD_THREADS, 0, s, a);
    else        // prompts: the blocks run for the whole sequence and want an SM each (see tb_launch_plain)
        tb_launch_plain(delta_scan_kernel<RPT, SPLIT>, grid, dim3(CD_THREADS), 0, s, a);
}

static int delta_scan_launch(const DeltaScanArgs& a, int nt, int B, cudaStream_t s) {
    if (B < 0 || a.G <= 0 || a.H <= 0 || a.H % a.G || a.dim <= 0 || a.vdim <= 0) return TB_ERR_ARG;
    if (a.dim > 256) return TB_ERR_UNSUPPORTED;
    if (B == 0) return 0;
    // Lanes per column.  Prompts: many lanes, since the chain of one token is what a sequence waits for (measured
    // with 16 heads of 128 x 128: one prompt of 2,048 tokens 0.71 ms with 16 lanes, 0.87 with 4; eight of 1,024
    // tokens 1.32 against 1.65).  Steps of a token or two per sequence: four lanes, since then the kernel is the
    // state's way in and out of the registers, and a thread's rows lie closer together (batch 64: 44 against 103 us).
    const int rows = cd_rows(a.dim);
    int lanes = rows >= 128 ? 16 : rows >= 32 ? 8 : 4;
    if (cd_scan_lanes_override > 0) lanes = cd_scan_lanes_override;
    else if (nt <= 2 * B) lanes = 4;
    const bool early = nt <= 2 * B;
    if (lanes > rows / 4) lanes = rows / 4;
    if (rows / lanes > 32) lanes = rows / 32;
    switch (rows / lanes * 100 + lanes) {       // rows per thread, lanes per column
        case 4 * 100 + 4: delta_scan_go<4, 4>(a, B, early, s); break;
        case 8 * 100 + 4: delta_scan_go<8, 4>(a, B, early, s); break;
        case 4 * 100 + 8: delta_scan_go<4, 8>(a, B, early, s); break;
        case 16 * 100 + 4: delta_scan_go<16, 4>(a, B, early, s); break;
        case 8 * 100 + 8: delta_scan_go<8, 8>(a, B, early, s); break;
        case 4 * 100 + 16: delta_scan_go<4, 16>(a, B, early, s); break;
        case 32 * 100 + 4: delta_scan_go<32, 4>(a, B, early, s); break;
        case 16 * 100 + 8: delta_scan_go<16, 8>(a, B, early, s); break;
        case 8 * 100 + 16: delta_scan_go<8, 16>(a, B, early, s); break;
        case 32 * 100 + 8: delta_scan_go<32, 8>(a, B, early, s); break;
        case 16 * 100 + 16: delta_scan_go<16, 16>(a, B, early, s); break;
        default: return TB_ERR_UNSUPPORTED;
    }
    return tb_last_error();
}

extern "C" {
// Floats of state per slot: the matrix memory of every head, then the convolution's last inputs.
int tb_delta_state_size(int G, int H, int dim, int vdim, int taps) {
    return H * dim * vdim + (taps - 1) * (2 * G * dim + H * vdim);
}
// For measurements: 4, 8 or 16 lanes per column in the scan whatever the batch; 0 gives the choice back to the rule.
int tb_delta_scan_lanes(int lanes) {
    cd_scan_lanes_override = lanes;
    return 0;
}
// Floats of a (token, head) record and of a (token, head) row of values between the two kernels.
int tb_delta_record_size(int dim) { return cd_record(dim); }
int tb_delta_value_pitch(int vdim) { return cd_vpitch(vdim); }
#define TB_DELTA_PREP(SFX, T)                                                                                         \
    int tb_delta_prep_##SFX(const void* z, int ldz, const float* wconv, float* state, const float* a,                 \
                            const float* dt_bias, const float* A_log, const float* bz, float* rec, float* vbuf,       \
                            const int* tok_seq, const int* seq_start, const int* slots, int nt, int B, int G, int H,  \
                            int dim, int vdim, int taps, int update_state, int lda, int ldb, int head_decay,          \
                            cudaStream_t s) {                                                                         \
        if (lda < (head_decay ? H : H * dim) || ldb < H) return TB_ERR_ARG;                                           \
        DeltaPrepArgs p{z, wconv, state, a, dt_bias, A_log, bz, rec, vbuf, tok_seq, seq_start, slots,                 \
                        (long long)tb_delta_state_size(G, H, dim, vdim, taps), (long long)H * dim * vdim, ldz, G, H,  \
                        dim, vdim, taps, update_state, lda, ldb, head_decay ? 1 : 0};                                 \
        return delta_prep_launch<T>(p, nt, B, s);                                                                     \
    }
TB_DELTA_PREP(f32, float)
TB_DELTA_PREP(bf16, __nv_bfloat16)

int tb_delta_scan(const float* rec, const float* vbuf, float* state, float* out, const int* seq_start,
                  const int* slots, int nt, int B, int G, int H, int dim, int vdim, int taps, cudaStream_t s) {
    if ((((uintptr_t)rec | (uintptr_t)vbuf) & 15)) return TB_ERR_ARG;
    DeltaScanArgs a{rec, vbuf, state, out, seq_start, slots, (long long)tb_delta_state_size(G, H, dim, vdim, taps), G, H,
                    dim, vdim};
    return delta_scan_launch(a, nt, B, s);
}
}

#include "tape.h"
TB_TAPE_REGISTER(tb_delta_prep_f32)
TB_TAPE_REGISTER(tb_delta_prep_bf16)
TB_TAPE_REGISTER(tb_delta_scan)
