// What lies between the q/k/v projection and the paged attention kernels for attention layers whose projections pass a short
// causal convolution, whose query and key heads are normalised, whose rotation covers only the first `rot` values of a head,
// whose value size differs from the key size or whose values are the keys themselves; and the output gate behind the
// attention kernels.
//
//   qkv_conv_rope_store   one CTA per token and head.  The token's row [q | k | v] (Hq*D + Hkv*D + Hkv*Dv channels) is convolved over
//                         time, y_t[c] = sum_k w[k][c] * u_(t - taps + 1 + k)[c] in 32-bit (weights tap-major; inputs before
//                         the step's first token come from the request's state row, which holds the last taps - 1 projected
//                         rows, oldest first, and is zero for a new request); with norm weights every q and k head is divided
//                         by its root mean square (eps inside the root) and multiplied by a weight per channel that all heads
//                         share; q and k are rotated at the token's position (pairs (i, i + rot/2) or (2i, 2i + 1); cos/sin
//                         from the step's table); q is multiplied by 1 + coef * ln(floor((pos + 1) / every) + 1) where a
//                         query temperature is set; q is written as [T, Hq, Dp] and k, v into the pages
//                         [page, Hkv, slot, Dp]; Dp >= max(D, Dv), the rest zero.  v_from_k: the row has no v columns and a
//                         value head is the key head as it stands before norm and rotation.
//   conv_tail_update      moves the step's last taps - 1 projected rows into the state rows (a request that brought fewer
//                         keeps the newest of its old ones); runs after the kernel above has read the old rows.
//   stream_conv           the same convolution over the rows of the 32-bit residual stream (every channel of the model's width),
//                         for layers whose mixer reads x + conv(x): weights tap-major in 32-bit (the caller adds 1 to the last
//                         tap for the x itself), state rows as above with the last taps - 1 stream rows, output in the compute
//                         dtype; conv_tail_update (32-bit rows) advances the state
//   gate_head_rows        out[t, h, :Dv] = attn[t, h, :Dv] * sigmoid(gate) (gate optional: one number per head, gate[t, h], or
//                         one per value, gate[t, h * Dv + j]), dropping the padding.
#include "common.cuh"
using namespace ttie;

namespace {

__device__ __forceinline__ int slot_row_(int slot, int num_rows) { return slot < 0 ? num_rows - 1 : slot; }

struct QkvArgs {
    const void* proj; long long ld;
    int Hq, Hkv, D, Dv, Dp;
    int taps; const float* conv_w; const float* tail; int tail_rows;
    const int* positions; const int* token_seq; const int* qsl; const int* slot_ids;
    const float2* cs; int rot; int style;
    const float* norm_w; float norm_eps;                            // [2][D]: the query heads' weights, then the key heads'; null: no norm
    const float* row_inv;                                           // [T][2]: 1 / rms of the token's whole q and whole k projection (one norm over
                                                                    // all heads at once; norm_w is then [Hq*D + Hkv*D], a weight per channel); null: a norm per head
    int v_from_k;                                                   // the values are the key heads before norm and rotation
    float qt_coef; int qt_every;                                    // query temperature; every 0: none
    void* q_out; void* k_pages; void* v_pages;
    const int* block_table; int table_width, page_size, num_pages, write_kv;
};

// channels of a row [q | k | v], or [q | k] where the values are the keys
__device__ __forceinline__ int row_channels(const QkvArgs& a) { return a.Hq * a.D + a.Hkv * a.D + (a.v_from_k ? 0 : a.Hkv * a.Dv); }
// first channel of value head h
__device__ __forceinline__ int value_col0(const QkvArgs& a, int h) { return a.v_from_k ? a.Hq * a.D + h * a.D : (a.Hq + a.Hkv) * a.D + h * a.Dv; }
// what a query at position pos is multiplied by
__device__ __forceinline__ float query_temperature(const QkvArgs& a, int pos) {
    return a.qt_every > 0 ? 1.0f + a.qt_coef * logf((float)((pos + 1) / a.qt_every) + 1.0f) : 1.0f;
}

// first norm weight of head h of kind 0 (q) or 1 (k)
__device__ __forceinline__ int norm_w0(const QkvArgs& a, int kind, int h) {
    return a.row_inv ? (kind == 0 ? h * a.D : (a.Hq + h) * a.D) : kind * a.D;
}

// value i of a head row x after the rotation of its first `rot` values
__device__ __forceinline__ float rotated(const float* x, int i, int rot, int style, const float2* cs) {
    if (i >= rot) return x[i];
    const int half = rot >> 1;
    if (style == 1) {                                               // pairs (j, j + half)
        if (i < half) { const float2 c = cs[i]; return x[i] * c.x - x[i + half] * c.y; }
        const float2 c = cs[i - half];
        return x[i] * c.x + x[i - half] * c.y;
    }
    const float2 c = cs[i >> 1];                                    // pairs (2j, 2j + 1)
    return (i & 1) ? x[i] * c.x + x[i - 1] * c.y : x[i] * c.x - x[i + 1] * c.y;
}

// one CTA per (token, head of q, k or v): the head's channels are convolved into shared memory, then rotated and written
template <typename T>
__global__ void __launch_bounds__(128) qkv_conv_rope_store_kernel(const QkvArgs a) {
    TTIE_PDL_ENTRY();
    extern __shared__ float row[];                                  // the head's convolved channels
    __shared__ float red[32];
    const int t = blockIdx.x, unit = blockIdx.y;
    const int C = row_channels(a);
    const int kind = unit < a.Hq ? 0 : unit < a.Hq + a.Hkv ? 1 : 2; // q, k, v
    const int h = kind == 0 ? unit : kind == 1 ? unit - a.Hq : unit - a.Hq - a.Hkv;
    const int width = kind == 2 ? a.Dv : a.D;
    const int c0 = kind == 0 ? h * a.D : kind == 1 ? a.Hq * a.D + h * a.D : value_col0(a, h);
    if (kind != 0 && !a.write_kv) return;
    const T* proj = reinterpret_cast<const T*>(a.proj);
    const int s = a.token_seq[t];
    const int j = t - a.qsl[s];                                     // index among the request's tokens of this step
    if (a.taps > 1) {
        const float* tail = a.tail + (size_t)slot_row_(a.slot_ids[s], a.tail_rows) * (a.taps - 1) * C;
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            const int c = c0 + i;
            float acc = 0.f;
            for (int k = 0; k < a.taps; ++k) {
                const int src = j - (a.taps - 1) + k;
                const float u = src >= 0 ? to_f32(proj[(size_t)(t - j + src) * a.ld + c]) : tail[(size_t)(a.taps - 1 + src) * C + c];
                acc = fmaf(a.conv_w[(size_t)k * C + c], u, acc);
            }
            row[i] = acc;
        }
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            const float u = to_f32(proj[(size_t)t * a.ld + c0 + i]);
            row[i] = a.conv_w ? a.conv_w[c0 + i] * u : u;
        }
    }
    __syncthreads();
    if (a.norm_w && kind != 2) {                                    // the head over its root mean square, times the shared weight
        float inv;
        if (a.row_inv) inv = a.row_inv[2 * (size_t)t + kind];
        else {
            float ss = 0.f;
            for (int i = threadIdx.x; i < a.D; i += blockDim.x) ss = fmaf(row[i], row[i], ss);
            ss = block_sum(ss, red);
            inv = 1.0f / sqrtf(ss / (float)a.D + a.norm_eps);
        }
        const float* nw = a.norm_w + norm_w0(a, kind, h);
        for (int i = threadIdx.x; i < a.D; i += blockDim.x) row[i] = row[i] * inv * nw[i];
        __syncthreads();
    }
    const float2* cs = a.rot > 0 ? a.cs + (size_t)t * (a.rot >> 1) : nullptr;
    const int pos = a.positions[t];
    if (kind == 0) {
        T* q = reinterpret_cast<T*>(a.q_out) + ((size_t)t * a.Hq + h) * a.Dp;
        const float temp = query_temperature(a, pos);
        for (int i = threadIdx.x; i < a.Dp; i += blockDim.x)
            q[i] = from_f32<T>(i < a.D ? rotated(row, i, a.rot, a.style, cs) * temp : 0.f);
        return;
    }
    int page = a.block_table[(size_t)s * a.table_width + pos / a.page_size];
    if (page < 0 || page >= a.num_pages) page = 0;                  // validated on the host; never write outside
    const size_t dst = (((size_t)page * a.Hkv + h) * a.page_size + pos % a.page_size) * a.Dp;
    if (kind == 1) {
        T* kp = reinterpret_cast<T*>(a.k_pages) + dst;
        for (int i = threadIdx.x; i < a.Dp; i += blockDim.x)
            kp[i] = from_f32<T>(i < a.D ? rotated(row, i, a.rot, a.style, cs) : 0.f);
    } else {
        T* vp = reinterpret_cast<T*>(a.v_pages) + dst;
        for (int i = threadIdx.x; i < a.Dp; i += blockDim.x)
            vp[i] = from_f32<T>(i < a.Dv ? row[i] : 0.f);
    }
}

// ---- bfloat16, eight values per thread: no shared memory, no barrier, so that prompt portions run as a few waves of threads
// each with all its loads in flight.  A thread owns eight consecutive values of one head of one token; inside the rotated
// part it convolves its partner's eight values as well (pairs (i, i + rot/2): the chunk rot/2 away; pairs (2i, 2i + 1): its own).
// Sizes: D, Dv, Dp and the row stride multiples of 8; rot a multiple of 16 (half pairs) or of 8 (interleaved pairs).  With a
// query/key norm the threads of a head (Dp / 8 adjacent lanes, a power of two) add their squares up by shuffles.
__device__ __forceinline__ void conv8(const QkvArgs& a, const __nv_bfloat16* __restrict__ proj, const float* __restrict__ tail, int C,
                                      int t, int j, int c, float* acc) {
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (int k = 0; k < a.taps; ++k) {
        const int src = j - (a.taps - 1) + k;
        float u[8];
        if (src >= 0) {
            const uint4 x = *reinterpret_cast<const uint4*>(proj + (size_t)(t - j + src) * a.ld + c);
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&x);
#pragma unroll
            for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); u[2 * i] = f.x; u[2 * i + 1] = f.y; }
        } else {
            const float* p = tail + (size_t)(a.taps - 1 + src) * C + c;
            const float4 x = *reinterpret_cast<const float4*>(p), y = *reinterpret_cast<const float4*>(p + 4);
            u[0] = x.x; u[1] = x.y; u[2] = x.z; u[3] = x.w; u[4] = y.x; u[5] = y.y; u[6] = y.z; u[7] = y.w;
        }
        if (a.conv_w) {
            const float* wp = a.conv_w + (size_t)k * C + c;
            const float4 w0 = __ldg(reinterpret_cast<const float4*>(wp)), w1 = __ldg(reinterpret_cast<const float4*>(wp + 4));
            const float w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = fmaf(w[i], u[i], acc[i]);
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = u[i];
        }
    }
}

__global__ void __launch_bounds__(256) qkv_conv_rope_store_vec8_kernel(const QkvArgs a, int T_) {
    TTIE_PDL_ENTRY();
    const int chunks = a.Dp >> 3, units = a.Hq + 2 * a.Hkv;
    const long long id = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (id >= (long long)T_ * units * chunks) return;
    const int jc = (int)(id % chunks);
    const int unit = (int)((id / chunks) % units);
    const int t = (int)(id / ((long long)chunks * units));
    const int C = row_channels(a);
    const int kind = unit < a.Hq ? 0 : unit < a.Hq + a.Hkv ? 1 : 2;
    const int h = kind == 0 ? unit : kind == 1 ? unit - a.Hq : unit - a.Hq - a.Hkv;
    if (kind != 0 && !a.write_kv) return;
    const int width = kind == 2 ? a.Dv : a.D;
    const int c0 = kind == 0 ? h * a.D : kind == 1 ? a.Hq * a.D + h * a.D : value_col0(a, h);
    const int i0 = jc << 3;                                          // first of this thread's values within the head
    const __nv_bfloat16* proj = reinterpret_cast<const __nv_bfloat16*>(a.proj);
    const int s = a.token_seq[t];
    const int j = t - a.qsl[s];
    const float* tail = a.taps > 1 ? a.tail + (size_t)slot_row_(a.slot_ids[s], a.tail_rows) * (a.taps - 1) * C : nullptr;
    const bool inside = i0 < width;
    float out[8];
    if (inside) conv8(a, proj, tail, C, t, j, c0 + i0, out);
    else {
#pragma unroll
        for (int i = 0; i < 8; ++i) out[i] = 0.f;
    }
    float inv = 1.f;
    const bool normed = a.norm_w != nullptr && kind != 2;
    if (normed) {                                                    // (the same for all lanes of a head: they sit side by side)
        if (a.row_inv) inv = a.row_inv[2 * (size_t)t + kind];
        else {
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) ss = fmaf(out[i], out[i], ss);
            const unsigned lane = threadIdx.x & 31u;
            const unsigned group = chunks >= 32 ? 0xffffffffu : ((1u << chunks) - 1u) << (lane & ~(unsigned)(chunks - 1));
            for (int o = 1; o < chunks; o <<= 1) ss += __shfl_xor_sync(group, ss, o);
            inv = 1.0f / sqrtf(ss / (float)a.D + a.norm_eps);
        }
        if (inside) {
            const float* w = a.norm_w + norm_w0(a, kind, h) + i0;
#pragma unroll
            for (int i = 0; i < 8; ++i) out[i] = out[i] * inv * w[i];
        }
    }
    if (inside && kind != 2 && i0 < a.rot) {
        const float2* cs = a.cs + (size_t)t * (a.rot >> 1);
        if (a.style == 1) {
            const int half = a.rot >> 1;
            const bool low = i0 < half;
            const int ip = low ? i0 + half : i0 - half;              // the partner's first value
            float other[8];
            conv8(a, proj, tail, C, t, j, c0 + ip, other);
            if (normed) {
                const float* w = a.norm_w + norm_w0(a, kind, h) + ip;
#pragma unroll
                for (int i = 0; i < 8; ++i) other[i] = other[i] * inv * w[i];
            }
            const int f0 = low ? i0 : i0 - half;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float2 c = cs[f0 + i];
                out[i] = low ? out[i] * c.x - other[i] * c.y : out[i] * c.x + other[i] * c.y;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 8; i += 2) {
                const float2 c = cs[(i0 + i) >> 1];
                const float x = out[i], y = out[i + 1];
                out[i] = x * c.x - y * c.y; out[i + 1] = x * c.y + y * c.x;
            }
        }
    }
    const int pos = a.positions[t];
    if (kind == 0 && a.qt_every > 0) {
        const float temp = query_temperature(a, pos);
#pragma unroll
        for (int i = 0; i < 8; ++i) out[i] *= temp;
    }
    uint4 packed;
    __nv_bfloat162* ph = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
    for (int i = 0; i < 4; ++i) ph[i] = __floats2bfloat162_rn(out[2 * i], out[2 * i + 1]);
    if (kind == 0) {
        *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(a.q_out) + ((size_t)t * a.Hq + h) * a.Dp + i0) = packed;
        return;
    }
    int page = a.block_table[(size_t)s * a.table_width + pos / a.page_size];
    if (page < 0 || page >= a.num_pages) page = 0;                  // validated on the host; never write outside
    const size_t dst = (((size_t)page * a.Hkv + h) * a.page_size + pos % a.page_size) * a.Dp + i0;
    *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(kind == 1 ? a.k_pages : a.v_pages) + dst) = packed;
}

// one warp per token: 1 / sqrt(mean(x^2) + eps) over the token's nq query channels and over its nk key channels (one norm over
// the whole projection, before it is cut into heads); 32-bit
template <typename T>
__global__ void __launch_bounds__(128) proj_row_rms_kernel(const T* __restrict__ proj, long long ld, int T_, int nq, int nk, float eps,
                                                           float* __restrict__ inv) {
    TTIE_PDL_ENTRY();
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (t >= T_) return;
    const T* row = proj + (size_t)t * ld;
    float sq = 0.f, sk = 0.f;
    for (int i = lane; i < nq; i += 32) { const float v = to_f32(row[i]); sq = fmaf(v, v, sq); }
    for (int i = lane; i < nk; i += 32) { const float v = to_f32(row[nq + i]); sk = fmaf(v, v, sk); }
    sq = warp_sum(sq); sk = warp_sum(sk);
    if (lane == 0) {
        inv[2 * (size_t)t] = 1.0f / sqrtf(sq / (float)nq + eps);
        inv[2 * (size_t)t + 1] = 1.0f / sqrtf(sk / (float)nk + eps);
    }
}

// one thread per (tile of CONV_TOKENS tokens, four channels); x [T, C] 32-bit, w [taps][C], tail [slots + 1][taps - 1][C].  The tokens of a
// tile are independent: their look-ups and loads are all asked for before the first sum is needed (prompt portions: tiles of 8
// tokens; steps of a few tokens: one token per thread, so that every token has threads of its own).
template <typename TO, int V, int CONV_TOKENS>
__global__ void __launch_bounds__(128) stream_conv_kernel(const float* __restrict__ x, int T_, int C, int taps, const float* __restrict__ w,
                                                          float* tail, int tail_rows, const int* __restrict__ token_seq,
                                                          const int* __restrict__ qsl, const int* __restrict__ slot_ids, TO* __restrict__ out,
                                                          int update_tail) {
    TTIE_PDL_ENTRY();
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * V;
    if (c >= C) return;
    for (int t0 = blockIdx.y * CONV_TOKENS; t0 < T_; t0 += gridDim.y * CONV_TOKENS) {
        int js[CONV_TOKENS];
        float* mine[CONV_TOKENS];
#pragma unroll
        for (int m = 0; m < CONV_TOKENS; ++m) {
            const int t = min(t0 + m, T_ - 1);
            const int s = token_seq[t];
            js[m] = t - qsl[s];                                     // index among the request's tokens of this step
            mine[m] = taps > 1 ? tail + (size_t)slot_row_(slot_ids[s], tail_rows) * (taps - 1) * C : nullptr;
        }
        float acc[CONV_TOKENS][V];
#pragma unroll
        for (int m = 0; m < CONV_TOKENS; ++m)
#pragma unroll
            for (int i = 0; i < V; ++i) acc[m][i] = 0.f;
        for (int k = 0; k < taps; ++k) {
            const float* wk = w + (size_t)k * C + c;
            float wv[V];
            if (V == 4) { const float4 v4 = __ldg(reinterpret_cast<const float4*>(wk)); wv[0] = v4.x; wv[1 % V] = v4.y; wv[2 % V] = v4.z; wv[3 % V] = v4.w; }
            else wv[0] = wk[0];
#pragma unroll
            for (int m = 0; m < CONV_TOKENS; ++m) {
                const int t = min(t0 + m, T_ - 1);
                const int src = js[m] - (taps - 1) + k;
                const float* u = src >= 0 ? x + (size_t)(t - js[m] + src) * C + c : mine[m] + (size_t)(taps - 1 + src) * C + c;
                // update_tail (every request of the step brings one token, so this thread alone reads its request's state row for
                // its channels): the row that tap k read moves one place up; the token's own row becomes the newest
                float* up = (CONV_TOKENS == 1 && update_tail && k >= 1) ? mine[m] + (size_t)(k - 1) * C + c : nullptr;
                if (V == 4) {
                    const float4 uv = *reinterpret_cast<const float4*>(u);
                    acc[m][0] = fmaf(wv[0], uv.x, acc[m][0]); acc[m][1 % V] = fmaf(wv[1 % V], uv.y, acc[m][1 % V]);
                    acc[m][2 % V] = fmaf(wv[2 % V], uv.z, acc[m][2 % V]); acc[m][3 % V] = fmaf(wv[3 % V], uv.w, acc[m][3 % V]);
                    if (up) *reinterpret_cast<float4*>(up) = uv;
                } else {
                    const float u0 = u[0];
                    acc[m][0] = fmaf(wv[0], u0, acc[m][0]);
                    if (up) up[0] = u0;
                }
            }
        }
#pragma unroll
        for (int m = 0; m < CONV_TOKENS; ++m) {
            if (t0 + m >= T_) break;
            TO* o = out + (size_t)(t0 + m) * C + c;
            if (V == 4 && sizeof(TO) == 2) {                          // four bfloat16 values: one 8-byte store (C and c are multiples of 4)
                const __nv_bfloat162 lo = __floats2bfloat162_rn(acc[m][0], acc[m][1 % V]), hi = __floats2bfloat162_rn(acc[m][2 % V], acc[m][3 % V]);
                uint2 packed;
                packed.x = *reinterpret_cast<const unsigned*>(&lo);
                packed.y = *reinterpret_cast<const unsigned*>(&hi);
                *reinterpret_cast<uint2*>(o) = packed;
            } else if (V == 4) {
                *reinterpret_cast<float4*>(o) = make_float4(acc[m][0], acc[m][1 % V], acc[m][2 % V], acc[m][3 % V]);
            } else {
#pragma unroll
                for (int i = 0; i < V; ++i) o[i] = from_f32<TO>(acc[m][i]);
            }
        }
    }
}

template <typename T>
__global__ void conv_tail_update_kernel(const T* __restrict__ proj, long long ld, int C, int taps, float* __restrict__ tail,
                                        int tail_rows, const int* __restrict__ qsl, const int* __restrict__ slot_ids) {
    TTIE_PDL_ENTRY();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int s = blockIdx.y;
    const int t0 = qsl[s], n = qsl[s + 1] - t0;
    float* mine = tail + (size_t)slot_row_(slot_ids[s], tail_rows) * (taps - 1) * C + c;
    for (int i = 0; i < taps - 1; ++i) {                            // ascending: row i takes from an old row behind it, or from the step
        const int idx = n - (taps - 1) + i;
        mine[(size_t)i * C] = idx >= 0 ? to_f32(proj[(size_t)(t0 + idx) * ld + c]) : mine[(size_t)(taps - 1 + idx) * C];
    }
}

template <typename T>
__global__ void gate_head_rows_kernel(const T* __restrict__ attn, const T* __restrict__ gate, long long ld_gate, int per_value, int T_, int H,
                                      int Dv, int Dp, T* __restrict__ out) {
    TTIE_PDL_ENTRY();
    const int col = blockIdx.x * blockDim.x + threadIdx.x;           // grid: (columns of a token's output row, tokens)
    if (col >= H * Dv) return;
    const int h = col / Dv, j = col - h * Dv;
    for (size_t t = blockIdx.y; t < (size_t)T_; t += gridDim.y) {
        float v = to_f32(attn[(t * H + h) * Dp + j]);
        if (gate) v *= 1.0f / (1.0f + expf(-to_f32(gate[t * ld_gate + (per_value ? col : h)])));
        out[t * H * Dv + col] = from_f32<T>(v);
    }
}

// bfloat16, eight values per thread (value size and padded size multiples of 8, 16-byte aligned rows)
__global__ void gate_head_rows_vec8_kernel(const __nv_bfloat16* __restrict__ attn, const __nv_bfloat16* __restrict__ gate, long long ld_gate,
                                           int per_value, int T_, int H, int Dv, int Dp, __nv_bfloat16* __restrict__ out) {
    TTIE_PDL_ENTRY();
    const int col = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (col >= H * Dv) return;
    const int h = col / Dv, j = col - h * Dv;
    for (size_t t = blockIdx.y; t < (size_t)T_; t += gridDim.y) {
        const uint4 x = *reinterpret_cast<const uint4*>(attn + (t * H + h) * Dp + j);
        uint4 y;
        const __nv_bfloat162* a = reinterpret_cast<const __nv_bfloat162*>(&x);
        __nv_bfloat162* b = reinterpret_cast<__nv_bfloat162*>(&y);
        if (gate && per_value) {                                     // (the gate row is 16-byte aligned like the others: the caller checks)
            const uint4 gv = *reinterpret_cast<const uint4*>(gate + t * ld_gate + col);
            const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __bfloat1622float2(a[i]), g = __bfloat1622float2(g2[i]);
                b[i] = __floats2bfloat162_rn(f.x / (1.0f + expf(-g.x)), f.y / (1.0f + expf(-g.y)));
            }
        } else {
            const float g = gate ? 1.0f / (1.0f + expf(-__bfloat162float(gate[t * ld_gate + h]))) : 1.0f;
#pragma unroll
            for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(a[i]); b[i] = __floats2bfloat162_rn(f.x * g, f.y * g); }
        }
        *reinterpret_cast<uint4*>(out + t * H * Dv + col) = y;
    }
}

}  // namespace

extern "C" int ttie_qkv_conv_rope_store(const void* proj, long long ld, int T, int Hq, int Hkv, int D, int Dv, int Dp, int taps,
                                        const float* conv_w, const float* tail, int tail_rows, const int* positions,
                                        const int* token_seq, const int* qsl, const int* slot_ids, const void* cs, int rot, int style,
                                        const float* norm_w, float norm_eps, const float* row_inv, int v_from_k, float qt_coef, int qt_every,
                                        void* q_out, void* k_pages, void* v_pages, const int* block_table, int table_width,
                                        int page_size, int num_pages, int write_kv, int dtype, void* stream) {
    if (T <= 0) return 0;
    if (v_from_k && Dv != D) TTIE_FAIL("qkv_conv_rope_store: values that are the keys have the keys' size, not %d against %d", Dv, D);
    if (qt_every < 0) TTIE_FAIL("qkv_conv_rope_store: a query temperature every %d positions", qt_every);
    if (Dp < D || Dp < Dv) TTIE_FAIL("qkv_conv_rope_store: padded head size %d below %d / %d", Dp, D, Dv);
    if (rot < 0 || rot > D || rot % 2) TTIE_FAIL("qkv_conv_rope_store: %d rotated values of a head of %d", rot, D);
    if (rot > 0 && !cs) TTIE_FAIL("qkv_conv_rope_store: a rotation needs the step's cos/sin table");
    if (taps < 1 || (taps > 1 && (!conv_w || !tail))) TTIE_FAIL("qkv_conv_rope_store: %d taps need weights and state rows", taps);
    if (row_inv && (!norm_w || conv_w)) TTIE_FAIL("qkv_conv_rope_store: a norm over the whole projection needs weights and excludes a convolution");
    QkvArgs a;
    a.proj = proj; a.ld = ld; a.Hq = Hq; a.Hkv = Hkv; a.D = D; a.Dv = Dv; a.Dp = Dp; a.taps = taps; a.conv_w = conv_w; a.tail = tail;
    a.tail_rows = tail_rows; a.positions = positions; a.token_seq = token_seq; a.qsl = qsl; a.slot_ids = slot_ids;
    a.cs = (const float2*)cs; a.rot = rot; a.style = style; a.norm_w = norm_w; a.norm_eps = norm_eps; a.row_inv = row_inv; a.v_from_k = v_from_k;
    a.qt_coef = qt_coef; a.qt_every = qt_every; a.q_out = q_out; a.k_pages = k_pages; a.v_pages = v_pages;
    a.block_table = block_table; a.table_width = table_width; a.page_size = page_size; a.num_pages = num_pages; a.write_kv = write_kv;
    const size_t smem = (size_t)(D > Dv ? D : Dv) * sizeof(float);
    if (T > 2147483647 / 1 || Hq + 2 * Hkv > 65535) TTIE_FAIL("qkv_conv_rope_store: %d heads exceed the grid", Hq + 2 * Hkv);
    cudaStream_t s = (cudaStream_t)stream;
    const bool aligned = !(((uintptr_t)proj | (uintptr_t)q_out | (uintptr_t)k_pages | (uintptr_t)v_pages | (uintptr_t)conv_w | (uintptr_t)tail) & 15);
    const int lanes = Dp / 8;                                        // of a head in the eight-values form; a norm adds up over them by shuffles
    const bool norm_ok = !norm_w || row_inv || (Dp % 8 == 0 && lanes <= 32 && (lanes & (lanes - 1)) == 0);
    if (dtype == kBF16 && D % 8 == 0 && Dv % 8 == 0 && Dp % 8 == 0 && ld % 8 == 0 && aligned && norm_ok
        && (rot == 0 || rot % (style == 1 ? 16 : 8) == 0)) {
        const long long threads = (long long)T * (Hq + 2 * Hkv) * (Dp / 8);
        if ((threads + 255) / 256 > 2147483647LL) TTIE_FAIL("qkv_conv_rope_store: grid too large");
        TTIE_LAUNCH(qkv_conv_rope_store_vec8_kernel, (unsigned)((threads + 255) / 256), 256, 0, s, a, T);
        TTIE_CHECK_LAUNCH("qkv_conv_rope_store");
        return 0;
    }
    dim3 grid(T, Hq + 2 * Hkv);
    if (dtype == kF32) TTIE_LAUNCH(qkv_conv_rope_store_kernel<float>, grid, 128, smem, s, a);
    else if (dtype == kBF16) TTIE_LAUNCH(qkv_conv_rope_store_kernel<__nv_bfloat16>, grid, 128, smem, s, a);
    else TTIE_FAIL("qkv_conv_rope_store: unknown dtype %d", dtype);
    TTIE_CHECK_LAUNCH("qkv_conv_rope_store");
    return 0;
}

extern "C" int ttie_proj_row_rms(const void* proj, long long ld, int T, int nq, int nk, float eps, float* inv, int dtype, void* stream) {
    if (T <= 0) return 0;
    if (nq <= 0 || nk <= 0) TTIE_FAIL("proj_row_rms: %d query and %d key channels", nq, nk);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == kF32) TTIE_LAUNCH(proj_row_rms_kernel<float>, ceil_div(T, 4), 128, 0, s, (const float*)proj, ld, T, nq, nk, eps, inv);
    else if (dtype == kBF16) TTIE_LAUNCH(proj_row_rms_kernel<__nv_bfloat16>, ceil_div(T, 4), 128, 0, s, (const __nv_bfloat16*)proj, ld, T, nq, nk, eps, inv);
    else TTIE_FAIL("proj_row_rms: unknown dtype %d", dtype);
    TTIE_CHECK_LAUNCH("proj_row_rms");
    return 0;
}

// update_tail: also advance the state rows (only for a step in which every request brings exactly one token; any other step is
// followed by conv_tail_update)
extern "C" int ttie_stream_conv(const float* x, int T, int C, int taps, const float* w, float* tail, int tail_rows,
                                const int* token_seq, const int* qsl, const int* slot_ids, void* out, int out_dtype, int update_tail,
                                void* stream) {
    if (T <= 0) return 0;
    if (taps < 1 || (taps > 1 && !tail)) TTIE_FAIL("stream_conv: %d taps need state rows", taps);
    cudaStream_t s = (cudaStream_t)stream;
    const bool vec = C % 4 == 0 && !(((uintptr_t)x | (uintptr_t)w | (uintptr_t)tail | (uintptr_t)out) & 15);
    const bool tiled = T >= 64 && !update_tail;
    const int tiles = ceil_div(T, tiled ? 8 : 1);
    const dim3 grid(ceil_div(vec ? C / 4 : C, 128), tiles < 65535 ? tiles : 65535);
#define SC(TO, V) do { if (tiled) TTIE_LAUNCH((stream_conv_kernel<TO, V, 8>), grid, 128, 0, s, x, T, C, taps, w, tail, tail_rows, token_seq, qsl, slot_ids, (TO*)out, 0); \
                       else TTIE_LAUNCH((stream_conv_kernel<TO, V, 1>), grid, 128, 0, s, x, T, C, taps, w, tail, tail_rows, token_seq, qsl, slot_ids, (TO*)out, update_tail); } while (0)
    if (out_dtype == kF32) { if (vec) SC(float, 4); else SC(float, 1); }
    else if (out_dtype == kBF16) { if (vec) SC(__nv_bfloat16, 4); else SC(__nv_bfloat16, 1); }
    else TTIE_FAIL("stream_conv: unknown dtype %d", out_dtype);
#undef SC
    TTIE_CHECK_LAUNCH("stream_conv");
    return 0;
}

extern "C" int ttie_conv_tail_update(const void* proj, long long ld, int C, int taps, float* tail, int tail_rows, const int* qsl,
                                     const int* slot_ids, int num_seqs, int dtype, void* stream) {
    if (num_seqs <= 0 || taps <= 1) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(ceil_div(C, 256), num_seqs);
    if (dtype == kF32) TTIE_LAUNCH(conv_tail_update_kernel<float>, grid, 256, 0, s, (const float*)proj, ld, C, taps, tail, tail_rows, qsl, slot_ids);
    else if (dtype == kBF16) TTIE_LAUNCH(conv_tail_update_kernel<__nv_bfloat16>, grid, 256, 0, s, (const __nv_bfloat16*)proj, ld, C, taps, tail, tail_rows, qsl, slot_ids);
    else TTIE_FAIL("conv_tail_update: unknown dtype %d", dtype);
    TTIE_CHECK_LAUNCH("conv_tail_update");
    return 0;
}

extern "C" int ttie_gate_head_rows(const void* attn, const void* gate, long long ld_gate, int per_value, int T, int H, int Dv, int Dp,
                                   void* out, int dtype, void* stream) {
    if (T <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(ceil_div(H * Dv, 256), T < 65535 ? T : 65535);
    if (dtype == kBF16 && Dv % 8 == 0 && Dp % 8 == 0 && !(((uintptr_t)attn | (uintptr_t)out) & 15)
        && !(gate && per_value && (((uintptr_t)gate & 15) || ld_gate % 8))) {
        dim3 g8(ceil_div(H * Dv / 8, 128), T < 65535 ? T : 65535);
        TTIE_LAUNCH(gate_head_rows_vec8_kernel, g8, 128, 0, s, (const __nv_bfloat16*)attn, (const __nv_bfloat16*)gate, ld_gate, per_value, T, H,
                    Dv, Dp, (__nv_bfloat16*)out);
        TTIE_CHECK_LAUNCH("gate_head_rows");
        return 0;
    }
    if (dtype == kF32) TTIE_LAUNCH(gate_head_rows_kernel<float>, grid, 256, 0, s, (const float*)attn, (const float*)gate, ld_gate, per_value, T, H, Dv, Dp, (float*)out);
    else if (dtype == kBF16) TTIE_LAUNCH(gate_head_rows_kernel<__nv_bfloat16>, grid, 256, 0, s, (const __nv_bfloat16*)attn, (const __nv_bfloat16*)gate, ld_gate, per_value, T, H, Dv, Dp, (__nv_bfloat16*)out);
    else TTIE_FAIL("gate_head_rows: unknown dtype %d", dtype);
    TTIE_CHECK_LAUNCH("gate_head_rows");
    return 0;
}
