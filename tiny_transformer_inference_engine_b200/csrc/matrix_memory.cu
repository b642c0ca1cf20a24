// Recurrent layers whose per-head state is a matrix S [key channels x value channels] that every token updates by a rank-one
// term: the RWKV-style time mix with a decay per key channel (wkv), the xLSTM matrix memory with scalar gates and a running
// maximum (mlstm), and retention, linear attention with one fixed decay per head and neither softmax nor denominator.  All of
// a recurrence is 32-bit: decays, gates, exponentials, rotated queries and keys, the state and the read-out.
//
// The scans share one layout.  A value column of S moves independently of the others, so a thread owns KPT consecutive key
// channels of one column (KPT = 4 for heads of up to 128 key channels, 8 up to 256, 16 up to 512: the fewest whose slices fit
// a warp, because the recurrence offers no other parallelism than its state's elements): a CTA is (columns x slices) threads
// for one (request, head), slices = key channels / KPT rounded up to a power of two, the lanes of a column's slices adjacent
// so that the read-out sum over key channels is a few shuffles.
// The state rows hold S as [head][value column][padded key channels] (a thread's channels are contiguous).  The step's tokens
// of a request are walked in order, a run of tokens at a time staged through shared memory in two stages: the next run's rows
// travel as asynchronous copies while this run is computed; decays and gates are evaluated before the walk, in parallel over
// the tokens.
// A request may be cut into steps anywhere because the walk starts from the state row and ends by writing it back.
//
//   token_shift_mix   mixes[m][t] = h_t + (h_(t-1) - h_t) * mu[m]; the previous token of a step's first token is the state row
//   wkv_decay         w = exp(-exp(wlog + w0)) per token and key channel
//   wkv_scan          o_t = (S + diag(u) k_t v_t^T)^T r_t, then S <- diag(w_t) S + k_t v_t^T;
//                     also stores the request's last mixer input as the next step's previous token
//   mlstm_gates       i = cap tanh(i'/cap), f = logsigmoid(cap tanh(f'/cap)), m' = max(f + m, i) as prefix operations of a warp;
//                     per token e^(f+m-m'), e^(i-m'), e^(-m'); also copies the normaliser state n for the scan to read
//   mlstm_scan        S <- e^(f+m-m') S + e^(i-m') k v^T, n likewise with k alone, o = S^T q / (max(|n.q|, e^(-m')) + 1e-6)
//   rotate_heads      float32 copies of `heads` head rows per token with the first `rot` values of each rotated at the token's
//                     position (either pairing) and the heads from `scale_from` on multiplied by a constant
//   retention_scan    S <- decay_h S + k v^T, o = S^T q, with q and k 32-bit (already rotated and scaled)
//   head_norm_gate    out = o / rms(o over the head) * weight * act(gate)   (act: silu or sigmoid; the weight is optional)
#include "common.cuh"
#include <math.h>
using namespace ttie;

namespace {


__device__ __forceinline__ int slot_row_(int slot, int num_rows) { return slot < 0 ? num_rows - 1 : slot; }

template <typename T>
__global__ void token_shift_mix_kernel(const T* __restrict__ x, long long ld, int T_, int d, int M, const float* __restrict__ mu,
                                       const float* __restrict__ prev, int prev_rows, const int* __restrict__ token_seq,
                                       const int* __restrict__ qsl, const int* __restrict__ slot_ids, T* __restrict__ out) {
    TTIE_PDL_ENTRY();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= d) return;
    for (int t = blockIdx.y; t < T_; t += gridDim.y) {
        const int s = token_seq[t];
        const float h = to_f32(x[(size_t)t * ld + c]);
        const float hp = t > qsl[s] ? to_f32(x[(size_t)(t - 1) * ld + c]) : prev[(size_t)slot_row_(slot_ids[s], prev_rows) * d + c];
        for (int m = 0; m < M; ++m)
            out[((size_t)m * T_ + t) * d + c] = from_f32<T>(fmaf(hp - h, mu[(size_t)m * d + c], h));
    }
}

// bfloat16, eight channels per thread (width and row stride multiples of 8, 16-byte aligned arrays)
__global__ void token_shift_mix_vec8_kernel(const __nv_bfloat16* __restrict__ x, long long ld, int T_, int d, int M, const float* __restrict__ mu,
                                            const float* __restrict__ prev, int prev_rows, const int* __restrict__ token_seq,
                                            const int* __restrict__ qsl, const int* __restrict__ slot_ids, __nv_bfloat16* __restrict__ out) {
    TTIE_PDL_ENTRY();
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (c >= d) return;
    for (int t = blockIdx.y; t < T_; t += gridDim.y) {
        const int s = token_seq[t];
        float h[8], hp[8];
        const uint4 xv = *reinterpret_cast<const uint4*>(x + (size_t)t * ld + c);
        const __nv_bfloat162* a = reinterpret_cast<const __nv_bfloat162*>(&xv);
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(a[i]); h[2 * i] = f.x; h[2 * i + 1] = f.y; }
        if (t > qsl[s]) {
            const uint4 pv = *reinterpret_cast<const uint4*>(x + (size_t)(t - 1) * ld + c);
            const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&pv);
#pragma unroll
            for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(b[i]); hp[2 * i] = f.x; hp[2 * i + 1] = f.y; }
        } else {
            const float* p = prev + (size_t)slot_row_(slot_ids[s], prev_rows) * d + c;
#pragma unroll
            for (int i = 0; i < 8; ++i) hp[i] = p[i];
        }
        for (int m = 0; m < M; ++m) {
            const float4 m0 = *reinterpret_cast<const float4*>(mu + (size_t)m * d + c), m1 = *reinterpret_cast<const float4*>(mu + (size_t)m * d + c + 4);
            const float w[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
            uint4 y;
            __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(&y);
#pragma unroll
            for (int i = 0; i < 4; ++i)
                o[i] = __floats2bfloat162_rn(fmaf(hp[2 * i] - h[2 * i], w[2 * i], h[2 * i]), fmaf(hp[2 * i + 1] - h[2 * i + 1], w[2 * i + 1], h[2 * i + 1]));
            *reinterpret_cast<uint4*>(out + ((size_t)m * T_ + t) * d + c) = y;
        }
    }
}

// decay of the time mix per token and key channel, once per step: w = exp(-exp(wlog + w0)), 32-bit
__global__ void wkv_decay_kernel(const float* __restrict__ wlog, long long ld, const float* __restrict__ w0, float* __restrict__ out,
                                 int T_, int HD) {
    TTIE_PDL_ENTRY();
    const long long total = (long long)T_ * HD;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
        const long long t = e / HD;
        const int c = (int)(e - t * HD);
        out[e] = expf(-expf(wlog[t * ld + c] + w0[c]));
    }
}

struct WkvArgs {
    const void* r; const void* k; const void* v; long long ld;       // [T, H*D] each, compute dtype
    const float* decay;                                               // [T, H*D] float32
    const float* u;
    float* state; int state_rows;                                     // [rows, H, D, Dpad]
    const void* x; long long ld_x; int d; float* prev; int prev_rows; // the mixer's input and the rows that keep its last token
    const int* qsl; const int* slot_ids;
    float* out;                                                       // [T, H*D] float32
    int H, D, Dpad, slices, tb; bool vec;                             // tb: tokens per stage; vec: rows can travel as 16-byte copies
};

// ---- staging of a run of tokens into shared memory
// Rows of D values per token and head go from global to shared memory as 16-byte asynchronous copies (no register in between,
// so a thread has all of a stage's copies in flight at once and the next stage travels while this one is computed); where the
// sizes or addresses do not allow that (`vec` false) the same rows are copied value by value.
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" :: "n"(N) : "memory"); }

template <typename E>
__device__ __forceinline__ void stage_rows(E* dst, int dst_ld, const E* src, long long src_ld, int rows, int D, bool vec) {
    if (vec) {
        constexpr int CE = 16 / sizeof(E);
        const int per_row = D / CE;
        for (int e = threadIdx.x; e < rows * per_row; e += blockDim.x) {
            const int tt = e / per_row, j = e - tt * per_row;
            cp_async16(dst + tt * dst_ld + j * CE, src + (size_t)tt * src_ld + j * CE);
        }
    } else {
        for (int e = threadIdx.x; e < rows * D; e += blockDim.x) {
            const int tt = e / D, j = e - tt * D;
            dst[tt * dst_ld + j] = src[(size_t)tt * src_ld + j];
        }
    }
}

// KPT consecutive staged values as floats, by vector loads from shared memory
template <int KPT>
__device__ __forceinline__ void lds_keys(const float* p, float* o) {
#pragma unroll
    for (int i = 0; i < KPT; i += 4) {
        const float4 x = *reinterpret_cast<const float4*>(p + i);
        o[i] = x.x; o[i + 1] = x.y; o[i + 2] = x.z; o[i + 3] = x.w;
    }
}
template <int KPT>
__device__ __forceinline__ void lds_keys(const __nv_bfloat16* p, float* o) {
#pragma unroll
    for (int i = 0; i < KPT; i += 4) {
        const uint2 x = *reinterpret_cast<const uint2*>(p + i);
        o[i] = __uint_as_float(x.x << 16); o[i + 1] = __uint_as_float(x.x & 0xffff0000u);
        o[i + 2] = __uint_as_float(x.y << 16); o[i + 3] = __uint_as_float(x.y & 0xffff0000u);
    }
}

// Sums over the SL adjacent lanes of a column of CNT values per lane at once (the partial read-outs of a run of tokens): at
// every step a lane hands half of its values to the partner and adds the partner's other half to the half it keeps, so the
// run costs CNT - 1 shuffles instead of CNT * log2(SL); once a lane is down to one value the remaining steps are plain
// butterfly additions.  Afterwards a lane holds, in v[0 ..], the totals of the tokens base, base + 1, ... (max(1, CNT / SL) of them).
template <int O, int CNT>
struct RunReduce {
    static __device__ __forceinline__ void run(float* v, int slice, int& base) {
        if constexpr (O >= 1) {
            if constexpr (CNT > 1) {
                constexpr int HALF = CNT / 2;
                const bool up = (slice & O) != 0;
#pragma unroll
                for (int i = 0; i < HALF; ++i) {
                    const float send = up ? v[i] : v[i + HALF];
                    const float keep = up ? v[i + HALF] : v[i];
                    v[i] = keep + __shfl_xor_sync(0xffffffffu, send, O);
                }
                if (up) base += HALF;
                RunReduce<O / 2, HALF>::run(v, slice, base);
            } else {
                v[0] += __shfl_xor_sync(0xffffffffu, v[0], O);
                RunReduce<O / 2, 1>::run(v, slice, base);
            }
        }
    }
};
// tokens a lane holds after RunReduce, and whether it is the one of several equal lanes that writes them
template <int SL, int N> struct RunOwner {
    static constexpr int COUNT = N >= SL ? N / SL : 1;
    static __device__ __forceinline__ bool writes(int slice) { return N >= SL ? true : (slice & (SL / N - 1)) == 0; }
};

// a request that brings this few tokens (decoded ones) is walked straight from global memory: nothing is staged
constexpr int DIRECT_TOKENS = 2;
template <int SL> __device__ __forceinline__ float slices_sum(float v) {
#pragma unroll
    for (int o = 1; o < SL; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

constexpr int MAXV = 16;            // staged tokens at most; also the most values of v (or gate weights) a thread carries ahead

template <typename T, int KPT, int SL>
__global__ void __launch_bounds__(128) wkv_scan_kernel(const WkvArgs a) {
    pdl_wait();                                                      // (the successor is let in at the end: its waiting CTAs would sit on the SMs of a long, latency-bound walk)
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int TB = 64 / KPT;                                     // tokens per stage: 16, 8 or 4
    const int cols = blockDim.x / SL;
    // two stages of [r | k] in the compute dtype and w in float32, rows of Dpad values; one array of the columns' v
    float* w_s = reinterpret_cast<float*>(smem_raw);                                  // [2][TB][Dpad]
    T* r_s = reinterpret_cast<T*>(w_s + 2 * TB * a.Dpad);                             // [2][TB][Dpad]
    T* k_s = r_s + 2 * TB * a.Dpad;
    float* v_s = reinterpret_cast<float*>(k_s + 2 * TB * a.Dpad);                     // [TB][cols]
    const int s = blockIdx.z, h = blockIdx.y;
    const int t0 = a.qsl[s], n = a.qsl[s + 1] - t0;
    const int slice = threadIdx.x % SL, cl = threadIdx.x / SL;
    const int col = blockIdx.x * cols + cl;
    const bool colv = col < a.D;
    const int HD = a.H * a.D;
    const int ch0 = slice * KPT;
    const size_t row = slot_row_(a.slot_ids[s], a.state_rows);
    float* sp = a.state + ((row * a.H + h) * a.D + (colv ? col : 0)) * a.Dpad + ch0;
    float S[KPT], ub[KPT];
#pragma unroll
    for (int i = 0; i < KPT; i += 4) {
        const float4 x4 = colv ? *reinterpret_cast<const float4*>(sp + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        S[i] = x4.x; S[i + 1] = x4.y; S[i + 2] = x4.z; S[i + 3] = x4.w;
    }
#pragma unroll
    for (int i = 0; i < KPT; ++i) ub[i] = ch0 + i < a.D ? a.u[h * a.D + ch0 + i] : 0.f;
    const T* rp = reinterpret_cast<const T*>(a.r) + (size_t)t0 * a.ld + h * a.D;
    const T* kp = reinterpret_cast<const T*>(a.k) + (size_t)t0 * a.ld + h * a.D;
    const T* vp = reinterpret_cast<const T*>(a.v) + (size_t)t0 * a.ld + h * a.D;
    const float* wp = a.decay + (size_t)t0 * HD + h * a.D;
    if (n <= DIRECT_TOKENS) {
        for (int tt = 0; tt < n; ++tt) {
            const float vj = colv ? to_f32(vp[(size_t)tt * a.ld + col]) : 0.f;
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < KPT; ++i) {
                const bool in = ch0 + i < a.D;
                const float kv = (in ? to_f32(kp[(size_t)tt * a.ld + ch0 + i]) : 0.f) * vj;
                acc = fmaf(in ? to_f32(rp[(size_t)tt * a.ld + ch0 + i]) : 0.f, fmaf(ub[i], kv, S[i]), acc);
                S[i] = fmaf(in ? wp[(size_t)tt * HD + ch0 + i] : 0.f, S[i], kv);
            }
            acc = slices_sum<SL>(acc);
            if (slice == 0 && colv) a.out[(size_t)(t0 + tt) * HD + h * a.D + col] = acc;
        }
    } else {
    // channels behind D (a head that does not fill its last slice) read as zero in every stage
    if (a.Dpad > a.D)
        for (int e = threadIdx.x; e < 2 * TB * a.Dpad; e += blockDim.x)
            if (e % a.Dpad >= a.D) { w_s[e] = 0.f; r_s[e] = from_f32<T>(0.f); k_s[e] = from_f32<T>(0.f); }
    auto stage = [&](int buf, int c0, int nb) {
        stage_rows<T>(r_s + buf * TB * a.Dpad, a.Dpad, rp + (size_t)c0 * a.ld, a.ld, nb, a.D, a.vec);
        stage_rows<T>(k_s + buf * TB * a.Dpad, a.Dpad, kp + (size_t)c0 * a.ld, a.ld, nb, a.D, a.vec);
        stage_rows<float>(w_s + buf * TB * a.Dpad, a.Dpad, wp + (size_t)c0 * HD, HD, nb, a.D, a.vec);
        cp_async_commit();
    };
    float vreg[MAXV];                                                // this thread's share of the next run's v
    auto fetch_v = [&](int c0, int nb) {
#pragma unroll
        for (int i = 0; i < MAXV; ++i) {
            const int e = i * blockDim.x + threadIdx.x;
            if (e < nb * cols) {
                const int tt = e / cols, c = blockIdx.x * cols + (e - tt * cols);
                vreg[i] = c < a.D ? to_f32(vp[(size_t)(c0 + tt) * a.ld + c]) : 0.f;
            }
        }
    };
    stage(0, 0, min(TB, n));
    fetch_v(0, min(TB, n));
    for (int c0 = 0, it = 0; c0 < n; c0 += TB, ++it) {
        const int nb = min(TB, n - c0), buf = it & 1;
        const bool more = c0 + TB < n;
        if (more) stage(buf ^ 1, c0 + TB, min(TB, n - c0 - TB));
#pragma unroll
        for (int i = 0; i < MAXV; ++i) {
            const int e = i * blockDim.x + threadIdx.x;
            if (e < nb * cols) v_s[e] = vreg[i];
        }
        if (more) { fetch_v(c0 + TB, min(TB, n - c0 - TB)); cp_async_wait<1>(); } else cp_async_wait<0>();
        __syncthreads();
        const T* rb = r_s + buf * TB * a.Dpad + ch0;
        const T* kb = k_s + buf * TB * a.Dpad + ch0;
        const float* wb = w_s + buf * TB * a.Dpad + ch0;
        float part[TB];                                              // this thread's share of every token's read-out
#pragma unroll
        for (int tt = 0; tt < TB; ++tt) {
            part[tt] = 0.f;
            if (tt < nb) {                                           // (the same for every thread of the CTA)
                const float vj = v_s[tt * cols + cl];
                float r_[KPT], k_[KPT], w_[KPT];
                lds_keys<KPT>(rb + tt * a.Dpad, r_);
                lds_keys<KPT>(kb + tt * a.Dpad, k_);
                lds_keys<KPT>(wb + tt * a.Dpad, w_);
                float acc = 0.f;
#pragma unroll
                for (int i = 0; i < KPT; ++i) {
                    const float kv = k_[i] * vj;
                    acc = fmaf(r_[i], fmaf(ub[i], kv, S[i]), acc);
                    S[i] = fmaf(w_[i], S[i], kv);
                }
                part[tt] = acc;
            }
        }
        int first = 0;
        RunReduce<SL / 2, TB>::run(part, slice, first);
        if (colv && RunOwner<SL, TB>::writes(slice)) {
#pragma unroll
            for (int j = 0; j < RunOwner<SL, TB>::COUNT; ++j)
                if (first + j < nb) a.out[(size_t)(t0 + c0 + first + j) * HD + h * a.D + col] = part[j];
        }
        __syncthreads();
    }
    }
    pdl_launch_dependents();
    if (colv) {
#pragma unroll
        for (int i = 0; i < KPT; i += 4) *reinterpret_cast<float4*>(sp + i) = make_float4(S[i], S[i + 1], S[i + 2], S[i + 3]);
    }
    if (blockIdx.x == 0 && blockIdx.y == 0 && n > 0) {               // the request's last input is the next step's previous token
        const T* x = reinterpret_cast<const T*>(a.x) + (size_t)(t0 + n - 1) * a.ld_x;
        float* p = a.prev + (size_t)slot_row_(a.slot_ids[s], a.prev_rows) * a.d;
        for (int c = threadIdx.x; c < a.d; c += blockDim.x) p[c] = to_f32(x[c]);
    }
}

__device__ __forceinline__ float logsigmoidf_(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

// The gates of the matrix memory for every token of the step: one CTA of GW warps per (request, head) walks the tokens
// 32 * GW at a time, a warp per 32 tokens.  With i, f the log gates and F_t the sum of f from a warp's first token to t, the
// running maximum m_t = max(f_t + m_(t-1), i_t) equals F_t + max(m_in, max over s <= t of (i_s - F_s)): a prefix sum and a
// prefix maximum over the lanes; a warp's m_in follows from the warps before it by the same rule applied to their totals.
// Writes per token (state decay e^(f + m_(t-1) - m_t), input weight e^(i - m_t), e^(-m_t)) and moves the request's running
// maximum in its state row.
constexpr int GW = 8;
__global__ void __launch_bounds__(32 * GW) mlstm_gates_kernel(const float* __restrict__ gates, long long ld_g, float* __restrict__ mx,
                                                              int state_rows, const int* __restrict__ qsl, const int* __restrict__ slot_ids,
                                                              float* __restrict__ out, int H, float cap,
                                                              const float* __restrict__ nrm, float* __restrict__ nsnap, int Dpad) {
    TTIE_PDL_ENTRY();
    __shared__ float tot_f[GW], tot_x[GW], carry;
    const int s = blockIdx.y, h = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t0 = qsl[s], n = qsl[s + 1] - t0;
    // a copy of the head's normaliser state as it stands before this step: the scan's CTAs all read it while one of them
    // writes the new one into the state row, which a CTA that starts late must not see
    for (int i = threadIdx.x; i < Dpad; i += blockDim.x)
        nsnap[((size_t)s * H + h) * Dpad + i] = nrm[((size_t)slot_row_(slot_ids[s], state_rows) * H + h) * Dpad + i];
    float* mrow = mx + (size_t)slot_row_(slot_ids[s], state_rows) * H + h;
    if (threadIdx.x == 0) carry = *mrow;
    for (int c0 = 0; c0 < n; c0 += 32 * GW) {
        const int t = c0 + warp * 32 + lane;
        const bool valid = t < n;
        float ig = -INFINITY, fg = 0.f;
        if (valid) {
            const float* g = gates + (size_t)(t0 + t) * ld_g;
            ig = cap * tanhf(g[h] / cap);
            fg = logsigmoidf_(cap * tanhf(g[H + h] / cap));
        }
        float F = fg;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const float y = __shfl_up_sync(0xffffffffu, F, o); if (lane >= o) F += y; }
        float X = ig - F;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const float y = __shfl_up_sync(0xffffffffu, X, o); if (lane >= o) X = fmaxf(X, y); }
        if (lane == 31) { tot_f[warp] = F; tot_x[warp] = X; }
        __syncthreads();
        float m_in = carry;
        for (int w = 0; w < warp; ++w) m_in = tot_f[w] + fmaxf(m_in, tot_x[w]);
        const float m_t = F + fmaxf(m_in, X);
        float m_prev = __shfl_up_sync(0xffffffffu, m_t, 1);
        if (lane == 0) m_prev = m_in;
        if (valid) {
            float* o3 = out + ((size_t)(t0 + t) * H + h) * 3;
            o3[0] = expf(fg + m_prev - m_t); o3[1] = expf(ig - m_t); o3[2] = expf(-m_t);
        }
        __syncthreads();
        if (warp == GW - 1 && lane == 31) carry = m_t;               // (lanes behind the last token pass the maximum on unchanged)
        __syncthreads();
    }
    if (threadIdx.x == 0) *mrow = carry;
}

struct MlstmArgs {
    const void* q; const void* k; const void* v; long long ld;        // q, k [T, H*D]; v [T, H*Dv]; one row stride
    const float* gates;                                               // [T, H, 3] from mlstm_gates
    float* S; float* nrm; int state_rows;                             // [rows, H, Dv, Dpad], [rows, H, Dpad]
    const float* nsnap;                                               // [requests, H, Dpad]: n as it stood before the step (mlstm_gates)
    const int* qsl; const int* slot_ids;
    float* out;                                                       // [T, H*Dv] float32
    int H, D, Dv, Dpad, slices, tb; float qscale; bool vec;
};

template <typename T, int KPT, int SL>
__global__ void __launch_bounds__(128) mlstm_scan_kernel(const MlstmArgs a) {
    pdl_wait();                                                      // (the successor is let in at the end: its waiting CTAs would sit on the SMs of a long, latency-bound walk)
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int TB = 64 / KPT;
    const int cols = blockDim.x / SL;
    T* q_s = reinterpret_cast<T*>(smem_raw);                                          // [2][TB][Dpad]
    T* k_s = q_s + 2 * TB * a.Dpad;
    float* v_s = reinterpret_cast<float*>(k_s + 2 * TB * a.Dpad);                     // [TB][cols]
    float* g_s = v_s + TB * cols;                                                     // [TB][3]: state decay, input weight, e^(-m)
    const int s = blockIdx.z, h = blockIdx.y;
    const int t0 = a.qsl[s], n = a.qsl[s + 1] - t0;
    const int slice = threadIdx.x % SL, cl = threadIdx.x / SL;
    const int col = blockIdx.x * cols + cl;
    const bool colv = col < a.Dv;
    const int ch0 = slice * KPT;
    const size_t row = slot_row_(a.slot_ids[s], a.state_rows);
    float* sp = a.S + ((row * a.H + h) * a.Dv + (colv ? col : 0)) * a.Dpad + ch0;
    float* np = a.nrm + (row * a.H + h) * a.Dpad + ch0;
    float S[KPT], nv[KPT];
#pragma unroll
    for (int i = 0; i < KPT; i += 4) {
        const float4 x4 = colv ? *reinterpret_cast<const float4*>(sp + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        S[i] = x4.x; S[i + 1] = x4.y; S[i + 2] = x4.z; S[i + 3] = x4.w;
        const float4 n4 = *reinterpret_cast<const float4*>(a.nsnap + ((size_t)s * a.H + h) * a.Dpad + ch0 + i);
        nv[i] = n4.x; nv[i + 1] = n4.y; nv[i + 2] = n4.z; nv[i + 3] = n4.w;
    }
    const T* qp = reinterpret_cast<const T*>(a.q) + (size_t)t0 * a.ld + h * a.D;
    const T* kp = reinterpret_cast<const T*>(a.k) + (size_t)t0 * a.ld + h * a.D;
    const T* vp = reinterpret_cast<const T*>(a.v) + (size_t)t0 * a.ld + h * a.Dv;
    const float* gp = a.gates + ((size_t)t0 * a.H + h) * 3;
    if (n <= DIRECT_TOKENS) {
        for (int tt = 0; tt < n; ++tt) {
            const float vj = colv ? to_f32(vp[(size_t)tt * a.ld + col]) : 0.f;
            const float fa = gp[(size_t)tt * a.H * 3], ib = gp[(size_t)tt * a.H * 3 + 1], em = gp[(size_t)tt * a.H * 3 + 2];
            float num = 0.f, nq = 0.f;
#pragma unroll
            for (int i = 0; i < KPT; ++i) {
                const bool in = ch0 + i < a.D;
                const float bk = ib * (in ? to_f32(kp[(size_t)tt * a.ld + ch0 + i]) : 0.f);
                const float qv = (in ? to_f32(qp[(size_t)tt * a.ld + ch0 + i]) : 0.f) * a.qscale;
                S[i] = fmaf(fa, S[i], bk * vj);
                nv[i] = fmaf(fa, nv[i], bk);
                num = fmaf(S[i], qv, num);
                nq = fmaf(nv[i], qv, nq);
            }
            num = slices_sum<SL>(num);
            nq = slices_sum<SL>(nq);
            if (slice == 0 && colv) a.out[(size_t)(t0 + tt) * a.H * a.Dv + h * a.Dv + col] = num / (fmaxf(fabsf(nq), em) + 1e-6f);
        }
    } else {
    if (a.Dpad > a.D)
        for (int e = threadIdx.x; e < 2 * TB * a.Dpad; e += blockDim.x)
            if (e % a.Dpad >= a.D) { q_s[e] = from_f32<T>(0.f); k_s[e] = from_f32<T>(0.f); }
    auto stage = [&](int buf, int c0, int nb) {
        stage_rows<T>(q_s + buf * TB * a.Dpad, a.Dpad, qp + (size_t)c0 * a.ld, a.ld, nb, a.D, a.vec);
        stage_rows<T>(k_s + buf * TB * a.Dpad, a.Dpad, kp + (size_t)c0 * a.ld, a.ld, nb, a.D, a.vec);
        cp_async_commit();
    };
    float vreg[MAXV], greg[2] = {0.f, 0.f};                          // this thread's share of the next run's v and gate weights
    auto fetch_v = [&](int c0, int nb) {
#pragma unroll
        for (int i = 0; i < MAXV; ++i) {
            const int e = i * blockDim.x + threadIdx.x;
            if (e < nb * cols) {
                const int tt = e / cols, c = blockIdx.x * cols + (e - tt * cols);
                vreg[i] = c < a.Dv ? to_f32(vp[(size_t)(c0 + tt) * a.ld + c]) : 0.f;
            }
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int e = i * blockDim.x + threadIdx.x;
            if (e < nb * 3) greg[i] = gp[(size_t)(c0 + e / 3) * a.H * 3 + e % 3];
        }
    };
    stage(0, 0, min(TB, n));
    fetch_v(0, min(TB, n));
    for (int c0 = 0, it = 0; c0 < n; c0 += TB, ++it) {
        const int nb = min(TB, n - c0), buf = it & 1;
        const bool more = c0 + TB < n;
        if (more) stage(buf ^ 1, c0 + TB, min(TB, n - c0 - TB));
#pragma unroll
        for (int i = 0; i < MAXV; ++i) {
            const int e = i * blockDim.x + threadIdx.x;
            if (e < nb * cols) v_s[e] = vreg[i];
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int e = i * blockDim.x + threadIdx.x;
            if (e < nb * 3) g_s[e] = greg[i];
        }
        if (more) { fetch_v(c0 + TB, min(TB, n - c0 - TB)); cp_async_wait<1>(); } else cp_async_wait<0>();
        __syncthreads();
        const T* qb = q_s + buf * TB * a.Dpad + ch0;
        const T* kb = k_s + buf * TB * a.Dpad + ch0;
        float pnum[TB], pden[TB];                                    // this thread's share of every token's S^T q and n . q
#pragma unroll
        for (int tt = 0; tt < TB; ++tt) {
            pnum[tt] = 0.f; pden[tt] = 0.f;
            if (tt < nb) {                                           // (the same for every thread of the CTA)
                const float vj = v_s[tt * cols + cl];
                const float fa = g_s[3 * tt], ib = g_s[3 * tt + 1];
                float q_[KPT], k_[KPT];
                lds_keys<KPT>(qb + tt * a.Dpad, q_);
                lds_keys<KPT>(kb + tt * a.Dpad, k_);
                float num = 0.f, nq = 0.f;
#pragma unroll
                for (int i = 0; i < KPT; ++i) {
                    const float bk = ib * k_[i];
                    const float qv = q_[i] * a.qscale;
                    S[i] = fmaf(fa, S[i], bk * vj);
                    nv[i] = fmaf(fa, nv[i], bk);
                    num = fmaf(S[i], qv, num);
                    nq = fmaf(nv[i], qv, nq);
                }
                pnum[tt] = num; pden[tt] = nq;
            }
        }
        int first = 0, first2 = 0;
        RunReduce<SL / 2, TB>::run(pnum, slice, first);
        RunReduce<SL / 2, TB>::run(pden, slice, first2);
        if (colv && RunOwner<SL, TB>::writes(slice)) {
#pragma unroll
            for (int j = 0; j < RunOwner<SL, TB>::COUNT; ++j)
                if (first + j < nb)
                    a.out[(size_t)(t0 + c0 + first + j) * a.H * a.Dv + h * a.Dv + col] =
                        pnum[j] / (fmaxf(fabsf(pden[j]), g_s[3 * (first + j) + 2]) + 1e-6f);
        }
        __syncthreads();
    }
    }
    pdl_launch_dependents();
    if (colv) {
#pragma unroll
        for (int i = 0; i < KPT; i += 4) *reinterpret_cast<float4*>(sp + i) = make_float4(S[i], S[i + 1], S[i + 2], S[i + 3]);
    }
    if (blockIdx.x == 0 && cl == 0) {
#pragma unroll
        for (int i = 0; i < KPT; i += 4) *reinterpret_cast<float4*>(np + i) = make_float4(nv[i], nv[i + 1], nv[i + 2], nv[i + 3]);
    }
}

// ---- retention
// float32 copies of head rows with the first `rot` values of each head rotated at the token's position: src [T, ld] holds
// `heads` rows of D values per token from column 0 on; cs [T, rot / 2] (cos, sin); style 0 pairs (2i, 2i + 1), 1 pairs
// (i, i + rot / 2).  Heads from `scale_from` on are multiplied by `scale` after the rotation.  Heads of an even size: one CTA
// row per token, one thread per pair of values (a rotated pair, or two neighbours behind the rotated part); else one thread
// per value.
template <typename T>
__global__ void __launch_bounds__(256) rotate_head_pairs_kernel(const T* __restrict__ src, long long ld, int heads, int D, int rot, int style,
                                                                const float2* __restrict__ cs, int scale_from, float scale, float* __restrict__ out) {
    TTIE_PDL_ENTRY();
    const int hd = D >> 1, half = rot >> 1;
    const int u = blockIdx.y * blockDim.x + threadIdx.x;               // pair u of the token's heads * D / 2
    if (u >= heads * hd) return;
    const long long t = blockIdx.x;
    const int h = u / hd, p = u - h * hd;
    const T* x = src + t * ld + (size_t)h * D;
    float* o = out + (t * heads + h) * D;
    const float sc = h >= scale_from ? scale : 1.0f;
    int ia, ib;
    if (p < half) {
        if (style == 1) { ia = p; ib = p + half; } else { ia = 2 * p; ib = ia + 1; }
        const float2 c = cs[t * half + p];
        const float a = to_f32(x[ia]), b = to_f32(x[ib]);
        const float ra = (a * c.x - b * c.y) * sc, rb = (b * c.x + a * c.y) * sc;
        if (style == 1) { o[ia] = ra; o[ib] = rb; }
        else *reinterpret_cast<float2*>(o + ia) = make_float2(ra, rb);      // (D is even: the pair is 8-byte aligned)
    } else {
        ia = 2 * p;
        *reinterpret_cast<float2*>(o + ia) = make_float2(to_f32(x[ia]) * sc, to_f32(x[ia + 1]) * sc);
    }
}


template <typename T>
__global__ void rotate_heads_kernel(const T* __restrict__ src, long long ld, int T_, int heads, int D, int rot, int style,
                                    const float2* __restrict__ cs, int scale_from, float scale, float* __restrict__ out) {
    TTIE_PDL_ENTRY();
    const long long total = (long long)T_ * heads * D;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
        const int i = (int)(e % D);
        const int h = (int)((e / D) % heads);
        const long long t = e / ((long long)D * heads);
        const T* x = src + t * ld + (size_t)h * D;
        float v = to_f32(x[i]);
        if (i < rot) {
            const int half = rot >> 1;
            const float2* c = cs + t * half;
            if (style == 1) {
                if (i < half) v = v * c[i].x - to_f32(x[i + half]) * c[i].y;
                else v = v * c[i - half].x + to_f32(x[i - half]) * c[i - half].y;
            } else {
                const float2 cc = c[i >> 1];
                v = (i & 1) ? v * cc.x + to_f32(x[i - 1]) * cc.y : v * cc.x - to_f32(x[i + 1]) * cc.y;
            }
        }
        out[e] = h >= scale_from ? v * scale : v;
    }
}

struct RetArgs {
    const float* q; const float* k; long long ld_qk;                  // [T, H*D] each, float32, one row stride
    const void* v; long long ld_v;                                    // [T, H*Dv], compute dtype
    const float* decay;                                               // [H]
    float* S; int state_rows;                                         // [rows, H, Dv, Dpad]
    const int* qsl; const int* slot_ids;
    float* out;                                                       // [T, H*Dv] float32
    int H, D, Dv, Dpad, slices, tb; bool vec;
    float* scratch; int parts, mode;                                  // [requests * parts, H, Dv, Dpad]; see below
};

// Long prompts in parts.  The decay is one number per head, so the state behind token t of a request is
//     decay^t S_0 + sum over the parts j that end at or before t of decay^(t - end_j) P_j,   P_j = sum_(u in part j) decay^(end_j - 1 - u) k_u v_u^T,
// and a part's P_j needs no other part.  With ``parts`` > 1 the kernel runs twice over a grid of requests x parts: mode 1 walks
// every part but a request's last from a zero state without reading out and leaves P_j in ``scratch`` (the unit of the last
// part copies the request's state row there meanwhile, so that the second launch reads nothing that it also writes); mode 0
// builds each part's first state from those, walks the part with read-out, and the request's last part writes the state row.
// A request's part is max(128, its tokens / parts rounded up to 64) tokens, so a request of few tokens is one part and runs as
// it does with parts == 1.
constexpr int PART_MIN_TOKENS = 128;

template <typename T, int KPT, int SL>
__global__ void __launch_bounds__(128) retention_scan_kernel(const RetArgs a) {
    pdl_wait();                                                      // (the successor is let in at the end, as in the other scans)
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int TB = 64 / KPT;
    const int cols = blockDim.x / SL;
    float* q_s = reinterpret_cast<float*>(smem_raw);                                  // [2][TB][Dpad]
    float* k_s = q_s + 2 * TB * a.Dpad;
    float* v_s = k_s + 2 * TB * a.Dpad;                                               // [TB][cols]
    const int s = blockIdx.z / a.parts, p = blockIdx.z - s * a.parts, h = blockIdx.y;
    int t0 = a.qsl[s], n = a.qsl[s + 1] - t0;
    int L = n, p_last = 0;                                           // tokens of a part, the part of the request's last token
    if (a.parts > 1 && n > 0) {
        L = max(PART_MIN_TOKENS, ((n + a.parts - 1) / a.parts + 63) / 64 * 64);
        p_last = (n - 1) / L;                                        // (< parts)
    }
    const bool local = a.mode == 1;
    const bool copies = local && p_last > 0 && p == a.parts - 1;     // (never a part that mode 1 walks: those lie before p_last)
    if (local ? (p >= p_last && !copies) : p > p_last) return;
    const int slice = threadIdx.x % SL, cl = threadIdx.x / SL;
    const int col = blockIdx.x * cols + cl;
    const bool colv = col < a.Dv;
    const int ch0 = slice * KPT;
    const size_t row = slot_row_(a.slot_ids[s], a.state_rows);
    float* sp = a.S + ((row * a.H + h) * a.Dv + (colv ? col : 0)) * a.Dpad + ch0;
    auto scratch_at = [&](int part) {
        return a.scratch + ((((size_t)s * a.parts + part) * a.H + h) * a.Dv + (colv ? col : 0)) * a.Dpad + ch0;
    };
    if (copies) {
        if (colv)
#pragma unroll
            for (int i = 0; i < KPT; i += 4) *reinterpret_cast<float4*>(scratch_at(p) + i) = *reinterpret_cast<const float4*>(sp + i);
        return;
    }
    const float decay = a.decay[h];
    float S[KPT];
#pragma unroll
    for (int i = 0; i < KPT; ++i) S[i] = 0.f;
    if (colv && !local) {
        if (p_last == 0) {
#pragma unroll
            for (int i = 0; i < KPT; i += 4) {
                const float4 x4 = *reinterpret_cast<const float4*>(sp + i);
                S[i] = x4.x; S[i + 1] = x4.y; S[i + 2] = x4.z; S[i + 3] = x4.w;
            }
        } else {                                                     // the state row as it was, then the parts before this one
            for (int j = -1; j < p; ++j) {
                const float f = powf(decay, (float)(p * L - (j + 1) * L));      // (0^0 = 1: a head that keeps nothing keeps its first state at p = 0)
                const float* src = scratch_at(j < 0 ? a.parts - 1 : j);
#pragma unroll
                for (int i = 0; i < KPT; i += 4) {
                    const float4 x4 = *reinterpret_cast<const float4*>(src + i);
                    S[i] = fmaf(f, x4.x, S[i]); S[i + 1] = fmaf(f, x4.y, S[i + 1]); S[i + 2] = fmaf(f, x4.z, S[i + 2]); S[i + 3] = fmaf(f, x4.w, S[i + 3]);
                }
            }
        }
    }
    t0 += p * L;
    n = min(L, n - p * L);
    const float* qp = a.q + (size_t)t0 * a.ld_qk + h * a.D;
    const float* kp = a.k + (size_t)t0 * a.ld_qk + h * a.D;
    const T* vp = reinterpret_cast<const T*>(a.v) + (size_t)t0 * a.ld_v + h * a.Dv;
    const size_t ld_o = (size_t)a.H * a.Dv;
    if (n <= DIRECT_TOKENS) {
        for (int tt = 0; tt < n; ++tt) {
            const float vj = colv ? to_f32(vp[(size_t)tt * a.ld_v + col]) : 0.f;
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < KPT; ++i) {
                const bool in = ch0 + i < a.D;
                const float kv = (in ? kp[(size_t)tt * a.ld_qk + ch0 + i] : 0.f) * vj;
                S[i] = fmaf(decay, S[i], kv);
                acc = fmaf(S[i], (in && !local) ? qp[(size_t)tt * a.ld_qk + ch0 + i] : 0.f, acc);
            }
            if (local) continue;
            acc = slices_sum<SL>(acc);
            if (slice == 0 && colv) a.out[(size_t)(t0 + tt) * ld_o + h * a.Dv + col] = acc;
        }
    } else {
    if (a.Dpad > a.D)
        for (int e = threadIdx.x; e < 2 * TB * a.Dpad; e += blockDim.x)
            if (e % a.Dpad >= a.D) { q_s[e] = 0.f; k_s[e] = 0.f; }
    auto stage = [&](int buf, int c0, int nb) {
        if (!local) stage_rows<float>(q_s + buf * TB * a.Dpad, a.Dpad, qp + (size_t)c0 * a.ld_qk, a.ld_qk, nb, a.D, a.vec);
        stage_rows<float>(k_s + buf * TB * a.Dpad, a.Dpad, kp + (size_t)c0 * a.ld_qk, a.ld_qk, nb, a.D, a.vec);
        cp_async_commit();
    };
    float vreg[MAXV];                                                // this thread's share of the next run's v
    auto fetch_v = [&](int c0, int nb) {
#pragma unroll
        for (int i = 0; i < MAXV; ++i) {
            const int e = i * blockDim.x + threadIdx.x;
            if (e < nb * cols) {
                const int tt = e / cols, c = blockIdx.x * cols + (e - tt * cols);
                vreg[i] = c < a.Dv ? to_f32(vp[(size_t)(c0 + tt) * a.ld_v + c]) : 0.f;
            }
        }
    };
    stage(0, 0, min(TB, n));
    fetch_v(0, min(TB, n));
    for (int c0 = 0, it = 0; c0 < n; c0 += TB, ++it) {
        const int nb = min(TB, n - c0), buf = it & 1;
        const bool more = c0 + TB < n;
        if (more) stage(buf ^ 1, c0 + TB, min(TB, n - c0 - TB));
#pragma unroll
        for (int i = 0; i < MAXV; ++i) {
            const int e = i * blockDim.x + threadIdx.x;
            if (e < nb * cols) v_s[e] = vreg[i];
        }
        if (more) { fetch_v(c0 + TB, min(TB, n - c0 - TB)); cp_async_wait<1>(); } else cp_async_wait<0>();
        __syncthreads();
        const float* qb = q_s + buf * TB * a.Dpad + ch0;
        const float* kb = k_s + buf * TB * a.Dpad + ch0;
        float part[TB];                                              // this thread's share of every token's read-out
#pragma unroll
        for (int tt = 0; tt < TB; ++tt) {
            part[tt] = 0.f;
            if (tt < nb) {                                           // (the same for every thread of the CTA)
                const float vj = v_s[tt * cols + cl];
                float q_[KPT], k_[KPT];
                lds_keys<KPT>(kb + tt * a.Dpad, k_);
#pragma unroll
                for (int i = 0; i < KPT; ++i) S[i] = fmaf(decay, S[i], k_[i] * vj);
                if (!local) {                                        // (the same for every thread of the grid)
                    lds_keys<KPT>(qb + tt * a.Dpad, q_);
                    float acc = 0.f;
#pragma unroll
                    for (int i = 0; i < KPT; ++i) acc = fmaf(S[i], q_[i], acc);
                    part[tt] = acc;
                }
            }
        }
        if (!local) {
            int first = 0;
            RunReduce<SL / 2, TB>::run(part, slice, first);
            if (colv && RunOwner<SL, TB>::writes(slice)) {
#pragma unroll
                for (int j = 0; j < RunOwner<SL, TB>::COUNT; ++j)
                    if (first + j < nb) a.out[(size_t)(t0 + c0 + first + j) * ld_o + h * a.Dv + col] = part[j];
            }
        }
        __syncthreads();
    }
    }
    pdl_launch_dependents();
    if (colv && (local || p == p_last)) {
        float* dst = local ? scratch_at(p) : sp;
#pragma unroll
        for (int i = 0; i < KPT; i += 4) *reinterpret_cast<float4*>(dst + i) = make_float4(S[i], S[i + 1], S[i + 2], S[i + 3]);
    }
}

// one warp per (token, head)
template <typename T>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, const T* __restrict__ gate, long long ld_g, const float* __restrict__ w,
                                      int T_, int H, int Dv, float eps, int act, T* __restrict__ out) {
    TTIE_PDL_ENTRY();
    const int lane = threadIdx.x & 31;
    const long long unit = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= (long long)T_ * H) return;
    const long long t = unit / H;
    const int h = (int)(unit - t * H);
    const float* src = o + (size_t)unit * Dv;
    float ss = 0.f;
    for (int j = lane; j < Dv; j += 32) { const float v = src[j]; ss = fmaf(v, v, ss); }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)Dv + eps);
    for (int j = lane; j < Dv; j += 32) {
        const float g = to_f32(gate[(size_t)t * ld_g + h * Dv + j]);
        const float sg = 1.0f / (1.0f + expf(-g));
        out[(size_t)unit * Dv + j] = from_f32<T>(src[j] * inv * (w ? w[h * Dv + j] : 1.0f) * (act == 0 ? g * sg : sg));
    }
}

// Key channels per thread for heads of D key channels: the fewest (the most threads per state) whose slices still fit a warp.
int keys_per_thread(int D) { return D <= 128 ? 4 : D <= 256 ? 8 : 16; }

int scan_shape(int D, int cols_total, int units, int* kpt, int* slices, int* threads) {
    const int k = keys_per_thread(D);
    int sl = 1;
    while (sl * k < D) sl <<= 1;
    if (sl > 32) return -1;
    *kpt = k; *slices = sl;
    // few (request, head) units: narrower CTAs so that the columns spread over more SMs
    int th = 128;
    while (th > 32 && (long long)units * ceil_div(cols_total, th / sl) < 2LL * num_sms()) th >>= 1;
    *threads = th;
    return 0;
}

}  // namespace

extern "C" int ttie_matrix_state_pad(int D) {                        // padded key channels of a state row
    const int k = keys_per_thread(D);
    int sl = 1;
    while (sl * k < D) sl <<= 1;
    return sl * k;
}

extern "C" int ttie_wkv_decay(const float* wlog, long long ld, const float* w0, float* out, int T, int HD, void* stream) {
    if (T <= 0) return 0;
    const long long total = (long long)T * HD;
    const int grid = (int)((total + 255) / 256 < 148LL * 16 ? (total + 255) / 256 : 148LL * 16);
    TTIE_LAUNCH(wkv_decay_kernel, grid, 256, 0, (cudaStream_t)stream, wlog, ld, w0, out, T, HD);
    TTIE_CHECK_LAUNCH("wkv_decay");
    return 0;
}

extern "C" int ttie_mlstm_gates(const float* gates, long long ld_g, float* mx, int state_rows, const int* qsl, const int* slot_ids,
                                int num_seqs, float* out, int H, float cap, const float* nrm, float* nsnap, int Dpad, void* stream) {
    if (num_seqs <= 0) return 0;
    TTIE_LAUNCH(mlstm_gates_kernel, dim3(H, num_seqs), 32 * GW, 0, (cudaStream_t)stream, gates, ld_g, mx, state_rows, qsl, slot_ids, out, H, cap,
                nrm, nsnap, Dpad);
    TTIE_CHECK_LAUNCH("mlstm_gates");
    return 0;
}

extern "C" int ttie_token_shift_mix(const void* x, long long ld, int T, int d, int M, const float* mu, const float* prev, int prev_rows,
                                    const int* token_seq, const int* qsl, const int* slot_ids, void* out, int dtype, void* stream) {
    if (T <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(ceil_div(d, 256), T < 65535 ? T : 65535);
    if (dtype == kBF16 && d % 8 == 0 && ld % 8 == 0 && !(((uintptr_t)x | (uintptr_t)out | (uintptr_t)mu) & 15)) {
        dim3 g8(ceil_div(d / 8, 128), T < 65535 ? T : 65535);
        TTIE_LAUNCH(token_shift_mix_vec8_kernel, g8, 128, 0, s, (const __nv_bfloat16*)x, ld, T, d, M, mu, prev, prev_rows, token_seq, qsl, slot_ids,
                    (__nv_bfloat16*)out);
        TTIE_CHECK_LAUNCH("token_shift_mix");
        return 0;
    }
    if (dtype == kF32) TTIE_LAUNCH(token_shift_mix_kernel<float>, grid, 256, 0, s, (const float*)x, ld, T, d, M, mu, prev, prev_rows, token_seq, qsl, slot_ids, (float*)out);
    else if (dtype == kBF16) TTIE_LAUNCH(token_shift_mix_kernel<__nv_bfloat16>, grid, 256, 0, s, (const __nv_bfloat16*)x, ld, T, d, M, mu, prev, prev_rows, token_seq, qsl, slot_ids, (__nv_bfloat16*)out);
    else TTIE_FAIL("token_shift_mix: unknown dtype %d", dtype);
    TTIE_CHECK_LAUNCH("token_shift_mix");
    return 0;
}

template <typename Args>
int launch_scan(void (*kernel)(const Args), const Args& a, dim3 grid, int threads, size_t smem, cudaStream_t s) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);   // (wide heads)
    return TTIE_LAUNCH(kernel, grid, threads, smem, s, a) == cudaSuccess ? 0 : -1;
}

// the kernel for a dtype, a number of key channels per thread and a number of slices (those of scan_shape: 4 channels with
// 1 to 32 slices, 8 or 16 channels with 32)
#define TTIE_SCAN_CASE(KERNEL, ARGS, K, L)                                                                            \
    if (kpt == K && a.slices == L) {                                                                                  \
        if (dtype == kF32) launch_scan<ARGS>(KERNEL<float, K, L>, a, grid, threads, smem, s);                        \
        else launch_scan<ARGS>(KERNEL<__nv_bfloat16, K, L>, a, grid, threads, smem, s);                              \
    }
#define TTIE_SCAN_DISPATCH(KERNEL, ARGS)                                                                              \
    do {                                                                                                              \
        if (dtype != kF32 && dtype != kBF16) TTIE_FAIL(#KERNEL ": unknown dtype %d", dtype);                           \
        TTIE_SCAN_CASE(KERNEL, ARGS, 4, 1) TTIE_SCAN_CASE(KERNEL, ARGS, 4, 2) TTIE_SCAN_CASE(KERNEL, ARGS, 4, 4)       \
        TTIE_SCAN_CASE(KERNEL, ARGS, 4, 8) TTIE_SCAN_CASE(KERNEL, ARGS, 4, 16) TTIE_SCAN_CASE(KERNEL, ARGS, 4, 32)     \
        TTIE_SCAN_CASE(KERNEL, ARGS, 8, 32) TTIE_SCAN_CASE(KERNEL, ARGS, 16, 32)                                       \
    } while (0)

extern "C" int ttie_wkv_scan(const void* r, const void* k, const void* v, long long ld, const float* decay, const float* u, float* state,
                             int state_rows, const void* x, long long ld_x, int d, float* prev, int prev_rows, const int* qsl,
                             const int* slot_ids, int num_seqs, float* out, int H, int D, int dtype, void* stream) {
    if (num_seqs <= 0) return 0;
    WkvArgs a;
    a.r = r; a.k = k; a.v = v; a.ld = ld; a.decay = decay; a.u = u; a.state = state; a.state_rows = state_rows;
    a.x = x; a.ld_x = ld_x; a.d = d; a.prev = prev; a.prev_rows = prev_rows; a.qsl = qsl; a.slot_ids = slot_ids; a.out = out;
    a.H = H; a.D = D;
    int threads, kpt;
    if (scan_shape(D, D, num_seqs * H, &kpt, &a.slices, &threads)) TTIE_FAIL("wkv_scan: %d key channels per head (at most 512)", D);
    a.Dpad = a.slices * kpt;
    const int cols = threads / a.slices;
    const int es = dtype == kF32 ? 4 : 2, ce = 16 / es;                // bytes per value of r and k; values per 16-byte copy
    a.tb = 64 / kpt;
    if (threads * MAXV < a.tb * cols) TTIE_FAIL("wkv_scan: internal: %d threads cannot carry %d x %d values", threads, a.tb, cols);
    const size_t smem = (size_t)2 * a.tb * a.Dpad * (4 + 2 * es) + (size_t)a.tb * cols * 4;
    a.vec = D % ce == 0 && D % 4 == 0 && ld % ce == 0 && !(((uintptr_t)r | (uintptr_t)k | (uintptr_t)decay) & 15);
    dim3 grid(ceil_div(D, cols), H, num_seqs);
    cudaStream_t s = (cudaStream_t)stream;
    TTIE_SCAN_DISPATCH(wkv_scan_kernel, WkvArgs);
    TTIE_CHECK_LAUNCH("wkv_scan");
    return 0;
}

extern "C" int ttie_mlstm_scan(const void* q, const void* k, const void* v, long long ld, const float* gates, float* S, float* nrm,
                               const float* nsnap, int state_rows, const int* qsl, const int* slot_ids, int num_seqs, float* out, int H, int D, int Dv,
                               float qscale, int dtype, void* stream) {
    if (num_seqs <= 0) return 0;
    MlstmArgs a;
    a.q = q; a.k = k; a.v = v; a.ld = ld; a.gates = gates; a.S = S; a.nrm = nrm; a.nsnap = nsnap; a.state_rows = state_rows;
    a.qsl = qsl; a.slot_ids = slot_ids; a.out = out; a.H = H; a.D = D; a.Dv = Dv; a.qscale = qscale;
    int threads, kpt;
    if (scan_shape(D, Dv, num_seqs * H, &kpt, &a.slices, &threads)) TTIE_FAIL("mlstm_scan: %d key channels per head (at most 512)", D);
    a.Dpad = a.slices * kpt;
    const int cols = threads / a.slices;
    const int es = dtype == kF32 ? 4 : 2, ce = 16 / es;
    a.tb = 64 / kpt;
    if (threads * MAXV < a.tb * cols || 2 * threads < a.tb * 3) TTIE_FAIL("mlstm_scan: internal: %d threads cannot carry %d x %d values", threads, a.tb, cols);
    const size_t smem = (size_t)2 * a.tb * a.Dpad * 2 * es + (size_t)a.tb * (cols + 3) * 4;
    a.vec = D % ce == 0 && ld % ce == 0 && !(((uintptr_t)q | (uintptr_t)k) & 15);
    dim3 grid(ceil_div(Dv, cols), H, num_seqs);
    cudaStream_t s = (cudaStream_t)stream;
    TTIE_SCAN_DISPATCH(mlstm_scan_kernel, MlstmArgs);
    TTIE_CHECK_LAUNCH("mlstm_scan");
    return 0;
}

extern "C" int ttie_rotate_heads(const void* src, long long ld, int T, int heads, int D, int rot, int style, const void* cs,
                                 int scale_from, float scale, float* out, int dtype, void* stream) {
    if (T <= 0 || heads <= 0) return 0;
    if (rot < 0 || rot > D || rot % 2) TTIE_FAIL("rotate_heads: %d rotated values of a head of %d", rot, D);
    if (rot > 0 && !cs) TTIE_FAIL("rotate_heads: a rotation needs the step's cos/sin table");
    const long long total = (long long)T * heads * D;
    const int grid = (int)((total + 255) / 256 < 148LL * 32 ? (total + 255) / 256 : 148LL * 32);
    cudaStream_t s = (cudaStream_t)stream;
    const long long units = (long long)heads * (D / 2);
    if (D % 2 == 0 && (units + 255) / 256 <= 65535) {
        const dim3 pg((unsigned)T, (unsigned)((units + 255) / 256));
        if (dtype == kF32) TTIE_LAUNCH(rotate_head_pairs_kernel<float>, pg, 256, 0, s, (const float*)src, ld, heads, D, rot, style, (const float2*)cs, scale_from, scale, out);
        else if (dtype == kBF16) TTIE_LAUNCH(rotate_head_pairs_kernel<__nv_bfloat16>, pg, 256, 0, s, (const __nv_bfloat16*)src, ld, heads, D, rot, style, (const float2*)cs, scale_from, scale, out);
        else TTIE_FAIL("rotate_heads: unknown dtype %d", dtype);
        TTIE_CHECK_LAUNCH("rotate_heads");
        return 0;
    }
    if (dtype == kF32) TTIE_LAUNCH(rotate_heads_kernel<float>, grid, 256, 0, s, (const float*)src, ld, T, heads, D, rot, style, (const float2*)cs, scale_from, scale, out);
    else if (dtype == kBF16) TTIE_LAUNCH(rotate_heads_kernel<__nv_bfloat16>, grid, 256, 0, s, (const __nv_bfloat16*)src, ld, T, heads, D, rot, style, (const float2*)cs, scale_from, scale, out);
    else TTIE_FAIL("rotate_heads: unknown dtype %d", dtype);
    TTIE_CHECK_LAUNCH("rotate_heads");
    return 0;
}

extern "C" int ttie_retention_scan(const float* q, const float* k, long long ld_qk, const void* v, long long ld_v, const float* decay,
                                   float* S, int state_rows, const int* qsl, const int* slot_ids, int num_seqs, float* out, int H, int D,
                                   int Dv, int parts, float* scratch, int dtype, void* stream) {
    if (num_seqs <= 0) return 0;
    if (parts < 1 || (parts > 1 && scratch == nullptr) || (long long)num_seqs * parts > 65535)
        TTIE_FAIL("retention_scan: %d parts for %d requests (scratch %p)", parts, num_seqs, (void*)scratch);
    RetArgs a;
    a.q = q; a.k = k; a.ld_qk = ld_qk; a.v = v; a.ld_v = ld_v; a.decay = decay; a.S = S; a.state_rows = state_rows;
    a.qsl = qsl; a.slot_ids = slot_ids; a.out = out; a.H = H; a.D = D; a.Dv = Dv; a.scratch = scratch; a.parts = parts; a.mode = 0;
    int threads, kpt;
    if (scan_shape(D, Dv, num_seqs * parts * H, &kpt, &a.slices, &threads)) TTIE_FAIL("retention_scan: %d key channels per head (at most 512)", D);
    a.Dpad = a.slices * kpt;
    const int cols = threads / a.slices;
    a.tb = 64 / kpt;
    if (threads * MAXV < a.tb * cols) TTIE_FAIL("retention_scan: internal: %d threads cannot carry %d x %d values", threads, a.tb, cols);
    const size_t smem = (size_t)2 * a.tb * a.Dpad * 2 * 4 + (size_t)a.tb * cols * 4;
    a.vec = D % 4 == 0 && ld_qk % 4 == 0 && !(((uintptr_t)q | (uintptr_t)k) & 15);
    dim3 grid(ceil_div(Dv, cols), H, num_seqs * parts);
    cudaStream_t s = (cudaStream_t)stream;
    if (parts > 1) {                                                 // every part's own sum, from a zero state
        a.mode = 1;
        TTIE_SCAN_DISPATCH(retention_scan_kernel, RetArgs);
        TTIE_CHECK_LAUNCH("retention_scan (parts)");
        a.mode = 0;
    }
    TTIE_SCAN_DISPATCH(retention_scan_kernel, RetArgs);
    TTIE_CHECK_LAUNCH("retention_scan");
    return 0;
}

extern "C" int ttie_head_norm_gate(const float* o, const void* gate, long long ld_g, const float* w, int T, int H, int Dv, float eps,
                                   int act, void* out, int dtype, void* stream) {
    if (T <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const long long units = (long long)T * H;
    const int grid = (int)((units + 7) / 8);
    if (dtype == kF32) TTIE_LAUNCH(head_norm_gate_kernel<float>, grid, 256, 0, s, o, (const float*)gate, ld_g, w, T, H, Dv, eps, act, (float*)out);
    else if (dtype == kBF16) TTIE_LAUNCH(head_norm_gate_kernel<__nv_bfloat16>, grid, 256, 0, s, o, (const __nv_bfloat16*)gate, ld_g, w, T, H, Dv, eps, act, (__nv_bfloat16*)out);
    else TTIE_FAIL("head_norm_gate: unknown dtype %d", dtype);
    TTIE_CHECK_LAUNCH("head_norm_gate");
    return 0;
}
