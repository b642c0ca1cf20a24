// Gated linear units with their constants as parameters, and a routed mixture of experts.
//   glu:            y = g' * sigmoid(alpha * g') * (u' + shift), g' = min(g, limit), u' = clamp(u, -limit, limit) (limit <= 0:
//                   no clamp); alpha = 1, shift = 0 is SwiGLU.  32-bit arithmetic, rounded once.
//   moe_route:      scores s = sigmoid(z), or softmax(z) over all experts, from 32-bit router logits; the choice is made by
//                   c = s + correction (a bias per expert, optional), the weights use s alone; expert e is in group
//                   e / (E / groups); a group is rated by adding up its `group_top` highest c, the `keep` best-rated
//                   groups stay eligible; the `top` highest c among eligible experts are taken (ties: the lower index),
//                   weighted s * scale, optionally renormalised to sum to `scale`.  One warp per token, all 32-bit.
//   moe_plan:       counting sort of the (token, choice) pairs by expert, on the device: offsets per expert, position of each
//                   pair, and a table of row tiles (expert, first row, rows) for the grouped product; nothing is read on the host.
//                   Only the first `tile_experts` experts get tiles: the ones behind them are identity experts, which own no
//                   matrices (their pairs are sorted like the others and no product touches their rows).
//   grouped_gemm:   C[pos, :] = A[row_of(pos), :] * W[expert_of_tile]^T for every tile of the table (FFMA, 32-bit accumulation,
//                   any sizes; operands in the compute dtype).
//   moe_combine:    out[t, :] = sum_k weight[t, k] * Y[pos(t, k), :] (+ shared[t, :]) in 32-bit, in the order of k; a choice k
//                   whose expert is an identity expert (idx >= first_identity) adds weight[t, k] * x[t, :] instead.
#include "common.cuh"
using namespace ttie;

namespace {

template <typename T>
__global__ void glu_kernel(const T* __restrict__ gu, long long ld, T* __restrict__ out, int F, size_t total, float alpha, float limit,
                           float shift) {
    TTIE_PDL_ENTRY();
    for (size_t e = blockIdx.x * (size_t)blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
        const size_t t = e / F;
        const int f = (int)(e % F);
        float g = to_f32(gu[t * ld + f]), u = to_f32(gu[t * ld + F + f]);
        if (limit > 0.f) { g = fminf(g, limit); u = fminf(fmaxf(u, -limit), limit); }
        out[e] = from_f32<T>(g / (1.0f + expf(-alpha * g)) * (u + shift));
    }
}

// bfloat16, 8 values per thread (F and the row stride multiples of 8, 16-byte aligned rows)
__global__ void glu_vec8_kernel(const __nv_bfloat16* __restrict__ gu, long long ld, __nv_bfloat16* __restrict__ out, int F8, size_t total8,
                                float alpha, float limit, float shift) {
    TTIE_PDL_ENTRY();
    for (size_t e = blockIdx.x * (size_t)blockDim.x + threadIdx.x; e < total8; e += (size_t)gridDim.x * blockDim.x) {
        const size_t t = e / F8;
        const int f = (int)(e % F8) * 8;
        const uint4 gv = *reinterpret_cast<const uint4*>(gu + t * ld + f);
        const uint4 uv = *reinterpret_cast<const uint4*>(gu + t * ld + (size_t)F8 * 8 + f);
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
        const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv);
        uint4 ov;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 g = __bfloat1622float2(g2[i]), u = __bfloat1622float2(u2[i]);
            if (limit > 0.f) {
                g.x = fminf(g.x, limit); g.y = fminf(g.y, limit);
                u.x = fminf(fmaxf(u.x, -limit), limit); u.y = fminf(fmaxf(u.y, -limit), limit);
            }
            o2[i] = __floats2bfloat162_rn(g.x / (1.0f + expf(-alpha * g.x)) * (u.x + shift), g.y / (1.0f + expf(-alpha * g.y)) * (u.y + shift));
        }
        *reinterpret_cast<uint4*>(out + t * (size_t)F8 * 8 + f) = ov;
    }
}

constexpr int MAX_EXPERTS = 512;

// One warp per token: the lanes share the experts (scores), the groups (ratings and ranks) and the search for the next
// largest score (a shuffle reduction per choice).  Shared memory per warp: E scores, then the groups' ratings and keep flags.
constexpr int ROUTE_WARPS = 4;
__global__ void __launch_bounds__(ROUTE_WARPS * 32)
moe_route_kernel(const float* __restrict__ logits, long long ld, int T_, int E, int groups, int keep, int group_top, int top,
                 float scale, int renorm, int softmax, const float* __restrict__ correction, int* __restrict__ idx,
                 float* __restrict__ wts) {
    extern __shared__ float sm[];
    TTIE_PDL_ENTRY();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * ROUTE_WARPS + warp;
    if (t >= T_) return;                                             // (whole warps leave; nothing below synchronises the block)
    float* s = sm + (size_t)warp * (2 * E + 2 * groups);             // the scores (weights), then what the choice is made by
    float* c = s + E;
    float* rating = c + E;
    float* kept = rating + groups;
    const int per = E / groups;
    if (softmax) {
        float mx = -INFINITY;
        for (int e = lane; e < E; e += 32) mx = fmaxf(mx, logits[(size_t)t * ld + e]);
        mx = warp_max(mx);
        float sum = 0.f;
        for (int e = lane; e < E; e += 32) { const float p = expf(logits[(size_t)t * ld + e] - mx); s[e] = p; sum += p; }
        sum = warp_sum(sum);
        for (int e = lane; e < E; e += 32) s[e] = s[e] / sum;
    } else {
        for (int e = lane; e < E; e += 32) s[e] = 1.0f / (1.0f + expf(-logits[(size_t)t * ld + e]));
    }
    // Sigmoid scores with nothing added and one group: the choice is made by the logits themselves.  The sigmoid is monotone, so
    // the order is the scores' own - also where two large logits round to the same score in 32-bit, which exact arithmetic tells apart.
    const bool by_logit = !softmax && !correction && groups == 1;
    for (int e = lane; e < E; e += 32) c[e] = by_logit ? logits[(size_t)t * ld + e] : correction ? s[e] + correction[e] : s[e];
    __syncwarp();
    for (int g = lane; g < groups; g += 32) {                        // a group's rating: the sum of its `group_top` (1 or 2) highest values
        float b0 = -INFINITY, b1 = -INFINITY;
        for (int e = 0; e < per; ++e) {
            const float v = c[g * per + e];
            if (v > b0) { b1 = b0; b0 = v; } else if (v > b1) b1 = v;
        }
        rating[g] = b0 + ((group_top > 1 && per > 1) ? b1 : 0.f);
    }
    __syncwarp();
    for (int g = lane; g < groups; g += 32) {                        // kept: fewer than `keep` groups rate higher (equal ratings: the lower index first)
        int ahead = 0;
        for (int h = 0; h < groups; ++h) ahead += (rating[h] > rating[g]) || (rating[h] == rating[g] && h < g);
        kept[g] = ahead < keep ? 1.f : 0.f;
    }
    __syncwarp();
    float total = 0.f;
    for (int k = 0; k < top; ++k) {
        float bv = -INFINITY;
        int be = -1;
        for (int e = lane; e < E; e += 32)                             // (taken experts are marked NaN and never compare greater; ascending e: the lower index wins a tie)
            if (kept[e / per] != 0.f && c[e] == c[e] && (be < 0 || c[e] > bv)) { bv = c[e]; be = e; }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oe = __shfl_xor_sync(0xffffffffu, be, o);
            if (oe >= 0 && (be < 0 || ov > bv || (ov == bv && oe < be))) { bv = ov; be = oe; }
        }
        if (be < 0) be = k;                                            // (nothing compared: the logits are not numbers; stay inside the tables)
        const float w = s[be];
        total += w;
        if (lane == 0) { idx[(size_t)t * top + k] = be; wts[(size_t)t * top + k] = w; }
        __syncwarp();
        if ((be & 31) == lane) c[be] = __int_as_float(0x7fc00000);
        __syncwarp();
    }
    for (int k = lane; k < top; k += 32) wts[(size_t)t * top + k] *= renorm ? scale / total : scale;
}

// one CTA.  pairs P = T * top.  tiles: int32 [max_tiles][4] = (expert, first row, rows, 0); meta[0] = number of tiles.
__global__ void __launch_bounds__(1024)
moe_plan_kernel(const int* __restrict__ idx, int P, int E, int tile_experts, int tile_rows, int max_tiles, int* __restrict__ offsets,
                int* __restrict__ pos_of_pair, int* __restrict__ pair_of_pos, int* __restrict__ tiles, int* __restrict__ meta) {
    __shared__ int count[MAX_EXPERTS], cursor[MAX_EXPERTS];
    TTIE_PDL_ENTRY();
    for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < P; p += blockDim.x) atomicAdd(&count[idx[p]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0, nt = 0;
        for (int e = 0; e < E; ++e) {
            offsets[e] = at; cursor[e] = at;
            for (int r = 0; e < tile_experts && r < count[e] && nt < max_tiles; r += tile_rows, ++nt) {
                tiles[4 * nt] = e; tiles[4 * nt + 1] = at + r; tiles[4 * nt + 2] = min(tile_rows, count[e] - r); tiles[4 * nt + 3] = 0;
            }
            at += count[e];
        }
        offsets[E] = at;
        meta[0] = nt;
    }
    __syncthreads();
    for (int p = threadIdx.x; p < P; p += blockDim.x) {
        const int at = atomicAdd(&cursor[idx[p]], 1);
        pos_of_pair[p] = at;
        pair_of_pos[at] = p;
    }
}

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

// An activation behind an ungated product, with the row's routing weight ahead of it: out = f(scale[row] * acc).  Scaling the
// product is scaling the expert's input (the product is linear), done in 32-bit.  act 0: none, 1: the square of relu.
// scale null: 1; scale_of (pair_of_pos) maps a sorted row to its (token, choice) pair, whose weight scale[] holds.
struct RowAct { int act; const float* scale; const int* scale_of; };
__device__ __forceinline__ float row_scale_of(const RowAct& ra, int pos) { return ra.scale ? ra.scale[ra.scale_of ? ra.scale_of[pos] : pos] : 1.0f; }
__device__ __forceinline__ float row_act(const RowAct& ra, float v, float scale) {
    v *= scale;
    if (ra.act == 1) { v = fmaxf(v, 0.f); v *= v; }
    return v;
}

// A rows: row_of[pos] / row_div (row_of null: pos itself).  W: [E, N, K] with expert stride.  C [P, N].
template <typename T, typename TO>
__global__ void __launch_bounds__(256)
grouped_gemm_kernel(const T* __restrict__ A, long long lda, const int* __restrict__ row_of, int row_div, const T* __restrict__ W,
                    long long w_stride, long long ldw, TO* __restrict__ C, long long ldc, const int* __restrict__ tiles,
                    const int* __restrict__ meta, int N, int K, RowAct ra) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    __shared__ int arow[BM];
    TTIE_PDL_ENTRY();
    const int tile = blockIdx.y;
    if (tile >= meta[0]) return;
    const int expert = tiles[4 * tile], r0 = tiles[4 * tile + 1], rows = tiles[4 * tile + 2];
    const int tid = threadIdx.x, n0 = blockIdx.x * BN;
    if (tid < BM) arow[tid] = tid < rows ? (row_of ? row_of[r0 + tid] / row_div : r0 + tid) : -1;
    __syncthreads();
    const T* We = W + (size_t)expert * w_stride;
    const int tx = tid % 16, ty = tid / 16;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int e = tid + i * 256;
            const int r = e / BK, kk = e % BK;
            const int gk = k0 + kk, gn = n0 + r, ar = arow[r];
            As[kk][r] = (ar >= 0 && gk < K) ? to_f32(A[(size_t)ar * lda + gk]) : 0.f;
            Ws[kk][r] = (gn < N && gk < K) ? to_f32(We[(size_t)gn * ldw + gk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], w[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) w[j] = Ws[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int r = ty * TM + i;
        if (r >= rows) continue;
        const float rs = row_scale_of(ra, r0 + r);
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int gn = n0 + tx * TN + j;
            if (gn < N) C[(size_t)(r0 + r) * ldc + gn] = from_f32<TO>(row_act(ra, acc[i][j], rs));
        }
    }
}

// ---- few rows (decode steps): every tile's weights are streamed once.  A warp owns GV_ROWS weight rows of the tile's expert,
// its lanes walk K in 16-byte steps, the tile's activation rows (a few, read by every warp) come through the cache MT at a
// time; lane-partial sums are added by shuffles in a fixed order.  K a multiple of the vector, rows 16-byte aligned.
constexpr int GV_WARPS = 8, GV_ROWS = 4;
template <typename T> struct VecOf;
template <> struct VecOf<float> { static constexpr int N = 4; using V = float4;
    static __device__ __forceinline__ void load(const float* p, float* o, bool stream) { const float4 v = stream ? __ldcs((const float4*)p) : __ldg((const float4*)p); o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w; } };
template <> struct VecOf<__nv_bfloat16> { static constexpr int N = 8; using V = uint4;
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* o, bool stream) {
        const uint4 v = stream ? __ldcs((const uint4*)p) : __ldg((const uint4*)p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); o[2 * i] = f.x; o[2 * i + 1] = f.y; } } };

// glu_F > 0: the matrix holds F gate rows, then F up rows; a warp then owns two gate rows and the two up rows that go with them
// and writes the gated unit's output [rows, F] (constants as in glu_kernel) - the [rows, 2F] product never leaves the SM.
struct GluConst { int F; float alpha, limit, shift; };
template <typename T, typename TO, int MT>
__global__ void __launch_bounds__(GV_WARPS * 32)
grouped_gemv_kernel(const T* __restrict__ A, long long lda, const int* __restrict__ row_of, int row_div, const T* __restrict__ W,
                    long long w_stride, long long ldw, TO* __restrict__ C, long long ldc, const int* __restrict__ tiles,
                    const int* __restrict__ meta, int N, int K, GluConst glu, RowAct ra) {
    constexpr int VN = VecOf<T>::N;
    TTIE_PDL_ENTRY();
    const int tile = blockIdx.y;
    if (tile >= meta[0]) return;
    const int expert = tiles[4 * tile], r0 = tiles[4 * tile + 1], rows = tiles[4 * tile + 2];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool gated = glu.F > 0;
    const int n0 = (blockIdx.x * GV_WARPS + warp) * (gated ? GV_ROWS / 2 : GV_ROWS);
    if (n0 >= (gated ? glu.F : N)) return;
    const T* wrow[GV_ROWS];
#pragma unroll
    for (int r = 0; r < GV_ROWS; ++r) {
        const int n = gated ? (r < 2 ? min(n0 + r, glu.F - 1) : glu.F + min(n0 + r - 2, glu.F - 1)) : min(n0 + r, N - 1);
        wrow[r] = W + (size_t)expert * w_stride + (size_t)n * ldw;
    }
    for (int m0 = 0; m0 < rows; m0 += MT) {
        const T* arow[MT];
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            const int pos = r0 + min(m0 + m, rows - 1);
            arow[m] = A + (size_t)(row_of ? row_of[pos] / row_div : pos) * lda;
        }
        float acc[MT][GV_ROWS];
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
            for (int r = 0; r < GV_ROWS; ++r) acc[m][r] = 0.f;
        for (int k = lane * VN; k < K; k += 32 * VN) {
            float w[GV_ROWS][VN], x[MT][VN];
#pragma unroll
            for (int r = 0; r < GV_ROWS; ++r) VecOf<T>::load(wrow[r] + k, w[r], m0 + MT >= rows);
#pragma unroll
            for (int m = 0; m < MT; ++m) VecOf<T>::load(arow[m] + k, x[m], false);
#pragma unroll
            for (int m = 0; m < MT; ++m)
#pragma unroll
                for (int r = 0; r < GV_ROWS; ++r)
#pragma unroll
                    for (int i = 0; i < VN; ++i) acc[m][r] = fmaf(x[m][i], w[r][i], acc[m][r]);
        }
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
            for (int r = 0; r < GV_ROWS; ++r) acc[m][r] = warp_sum(acc[m][r]);
        if (lane == 0 && gated) {
#pragma unroll
            for (int m = 0; m < MT; ++m)
#pragma unroll
                for (int r = 0; r < GV_ROWS / 2; ++r) {
                    if (m0 + m >= rows || n0 + r >= glu.F) continue;
                    float g = acc[m][r], u = acc[m][r + 2];
                    if (glu.limit > 0.f) { g = fminf(g, glu.limit); u = fminf(fmaxf(u, -glu.limit), glu.limit); }
                    C[(size_t)(r0 + m0 + m) * ldc + n0 + r] = from_f32<TO>(g / (1.0f + expf(-glu.alpha * g)) * (u + glu.shift));
                }
        } else if (lane == 0) {
#pragma unroll
            for (int m = 0; m < MT; ++m)
#pragma unroll
                for (int r = 0; r < GV_ROWS; ++r)
                    if (m0 + m < rows && n0 + r < N)
                        C[(size_t)(r0 + m0 + m) * ldc + n0 + r] = from_f32<TO>(row_act(ra, acc[m][r], row_scale_of(ra, r0 + m0 + m)));
        }
    }
}

// in place over rows sorted by expert: x[pos, :] = f(scale * x[pos, :]) (behind a library product, which has no epilogue)
template <typename T>
__global__ void row_scale_act_kernel(T* __restrict__ x, long long ld, int rows, int F, RowAct ra) {
    TTIE_PDL_ENTRY();
    const size_t total = (size_t)rows * F;
    for (size_t e = blockIdx.x * (size_t)blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
        const size_t r = e / F;
        T* p = x + r * ld + (e - r * F);
        *p = from_f32<T>(row_act(ra, to_f32(*p), row_scale_of(ra, (int)r)));
    }
}
__global__ void row_scale_act_vec8_kernel(__nv_bfloat16* __restrict__ x, long long ld, int rows, int F8, RowAct ra) {
    TTIE_PDL_ENTRY();
    const size_t total = (size_t)rows * F8;
    for (size_t e = blockIdx.x * (size_t)blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
        const size_t r = e / F8;
        uint4* p = reinterpret_cast<uint4*>(x + r * ld + (e - r * F8) * 8);
        const float rs = row_scale_of(ra, (int)r);
        uint4 v = *p;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); h[i] = __floats2bfloat162_rn(row_act(ra, f.x, rs), row_act(ra, f.y, rs)); }
        *p = v;
    }
}

// rows sorted by expert, gathered from the tokens: out[pos, :] = x[row_of[pos] / row_div, :]
template <typename T>
__global__ void gather_rows_kernel(const T* __restrict__ x, long long ldx, const int* __restrict__ row_of, int row_div, int rows, int d,
                                   T* __restrict__ out) {
    TTIE_PDL_ENTRY();
    const size_t total = (size_t)rows * d;
    for (size_t e = blockIdx.x * (size_t)blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
        const size_t r = e / d;
        out[e] = x[(size_t)(row_of[r] / row_div) * ldx + (e % d)];
    }
}

template <typename T, typename TY>
__global__ void moe_combine_kernel(const TY* __restrict__ Y, const int* __restrict__ pos_of_pair, const float* __restrict__ wts,
                                   const T* __restrict__ shared, int T_, int d, int top, float* __restrict__ out,
                                   const int* __restrict__ idx, int first_identity, const T* __restrict__ x, long long ldx,
                                   const float* __restrict__ shared_gate, long long ld_gate) {
    TTIE_PDL_ENTRY();
    const size_t total = (size_t)T_ * d;
    for (size_t e = blockIdx.x * (size_t)blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
        const size_t t = e / d;
        const int i = (int)(e % d);
        float acc = 0.f;
        for (int k = 0; k < top; ++k) {
            const bool same = idx && idx[t * top + k] >= first_identity;       // an identity expert: its output is the token's own row
            acc = fmaf(wts ? wts[t * top + k] : 1.0f, same ? to_f32(x[t * ldx + i]) : to_f32(Y[(size_t)pos_of_pair[t * top + k] * d + i]), acc);
        }
        if (shared) acc += to_f32(shared[e]) * (shared_gate ? 1.0f / (1.0f + expf(-shared_gate[t * ld_gate])) : 1.0f);
        out[e] = acc;
    }
}

// bfloat16 expert rows and shared rows, eight values per thread (d a multiple of 8)
__global__ void moe_combine_vec8_kernel(const __nv_bfloat16* __restrict__ Y, const int* __restrict__ pos_of_pair, const float* __restrict__ wts,
                                        const __nv_bfloat16* __restrict__ shared, int T_, int d8, int top, float* __restrict__ out,
                                        const int* __restrict__ idx, int first_identity, const __nv_bfloat16* __restrict__ x, long long ldx,
                                        const float* __restrict__ shared_gate, long long ld_gate) {
    TTIE_PDL_ENTRY();
    const size_t total = (size_t)T_ * d8;
    for (size_t e = blockIdx.x * (size_t)blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
        const size_t t = e / d8;
        const int i = (int)(e % d8) * 8;
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        for (int k = 0; k < top; ++k) {
            const float w = wts ? wts[t * top + k] : 1.0f;
            const bool same = idx && idx[t * top + k] >= first_identity;
            const uint4 v = *reinterpret_cast<const uint4*>(same ? x + t * ldx + i : Y + (size_t)pos_of_pair[t * top + k] * d8 * 8 + i);
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
            for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(h[j]); acc[2 * j] = fmaf(w, f.x, acc[2 * j]); acc[2 * j + 1] = fmaf(w, f.y, acc[2 * j + 1]); }
        }
        if (shared) {
            const uint4 v = *reinterpret_cast<const uint4*>(shared + t * d8 * 8 + i);
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
            const float sg = shared_gate ? 1.0f / (1.0f + expf(-shared_gate[t * ld_gate])) : 1.0f;
#pragma unroll
            for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(h[j]); acc[2 * j] = fmaf(sg, f.x, acc[2 * j]); acc[2 * j + 1] = fmaf(sg, f.y, acc[2 * j + 1]); }
        }
        float* o = out + t * d8 * 8 + i;
        *reinterpret_cast<float4*>(o) = make_float4(acc[0], acc[1], acc[2], acc[3]);
        *reinterpret_cast<float4*>(o + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
    }
}

inline int grid_for(size_t total) { return (int)((total + 255) / 256 < 8192 ? (total + 255) / 256 : 8192); }
}  // namespace

extern "C" int ttie_glu(const void* gate_up, long long ld, void* out, int T, int F, float alpha, float limit, float shift, int dtype,
                        void* stream) {
    if (T <= 0 || F <= 0) return 0;
    const size_t total = (size_t)T * F;
    if (dtype == kBF16 && F % 8 == 0 && ld % 8 == 0 && (((uintptr_t)gate_up | (uintptr_t)out) & 15) == 0) {
        TTIE_LAUNCH(glu_vec8_kernel, grid_for(total / 8), 256, 0, (cudaStream_t)stream, (const __nv_bfloat16*)gate_up, ld, (__nv_bfloat16*)out, F / 8,
                    total / 8, alpha, limit, shift);
        TTIE_CHECK_LAUNCH("glu");
        return 0;
    }
    if (dtype == kF32) TTIE_LAUNCH(glu_kernel<float>, grid_for(total), 256, 0, (cudaStream_t)stream, (const float*)gate_up, ld, (float*)out, F, total, alpha, limit, shift);
    else TTIE_LAUNCH(glu_kernel<__nv_bfloat16>, grid_for(total), 256, 0, (cudaStream_t)stream, (const __nv_bfloat16*)gate_up, ld, (__nv_bfloat16*)out, F, total, alpha, limit, shift);
    TTIE_CHECK_LAUNCH("glu");
    return 0;
}

extern "C" int ttie_moe_max_experts() { return MAX_EXPERTS; }
extern "C" int ttie_moe_tile_rows() { return BM; }

extern "C" int ttie_moe_route(const float* logits, long long ld, int T, int E, int groups, int keep, int group_top, int top, float scale, int renorm,
                              int softmax, const float* correction, int* idx, float* wts, void* stream) {
    if (T <= 0) return 0;
    if (E < 1 || E > MAX_EXPERTS || groups < 1 || E % groups || keep < 1 || keep > groups || top < 1 || top > keep * (E / groups)
        || group_top < 1 || group_top > 2)
        TTIE_FAIL("moe_route: %d experts in %d groups, keep %d, group score of %d, top %d", E, groups, keep, group_top, top);
    TTIE_LAUNCH(moe_route_kernel, ceil_div(T, ROUTE_WARPS), ROUTE_WARPS * 32, (size_t)ROUTE_WARPS * (2 * E + 2 * groups) * sizeof(float),
                (cudaStream_t)stream, logits, ld, T, E, groups, keep, group_top, top, scale, renorm, softmax, correction, idx, wts);
    TTIE_CHECK_LAUNCH("moe_route");
    return 0;
}

extern "C" int ttie_moe_plan(const int* idx, int P, int E, int tile_experts, int max_tiles, int* offsets, int* pos_of_pair, int* pair_of_pos,
                             int* tiles, int* meta, void* stream) {
    if (P <= 0) return 0;
    if (E > MAX_EXPERTS) TTIE_FAIL("moe_plan: %d experts (limit %d)", E, MAX_EXPERTS);
    if (tile_experts < 0 || tile_experts > E) TTIE_FAIL("moe_plan: %d of %d experts own matrices", tile_experts, E);
    TTIE_LAUNCH(moe_plan_kernel, 1, 1024, 0, (cudaStream_t)stream, idx, P, E, tile_experts, BM, max_tiles, offsets, pos_of_pair, pair_of_pos, tiles,
                meta);
    TTIE_CHECK_LAUNCH("moe_plan");
    return 0;
}

// act, row_scale, scale_of: an activation behind an ungated product, see RowAct (act 0 and row_scale null: the plain product)
extern "C" int ttie_grouped_gemm_act(const void* A, long long lda, const int* row_of, int row_div, const void* W, long long w_stride,
                                     long long ldw, void* C, long long ldc, const int* tiles, const int* meta, int max_tiles, int N, int K,
                                     int dtype, int out_dtype, int few_rows, int glu_F, float glu_alpha, float glu_limit, float glu_shift,
                                     int act, const float* row_scale, const int* scale_of, void* stream);

extern "C" int ttie_grouped_gemm(const void* A, long long lda, const int* row_of, int row_div, const void* W, long long w_stride,
                                 long long ldw, void* C, long long ldc, const int* tiles, const int* meta, int max_tiles, int N, int K,
                                 int dtype, int out_dtype, int few_rows, int glu_F, float glu_alpha, float glu_limit, float glu_shift,
                                 void* stream) {
    return ttie_grouped_gemm_act(A, lda, row_of, row_div, W, w_stride, ldw, C, ldc, tiles, meta, max_tiles, N, K, dtype, out_dtype, few_rows,
                                 glu_F, glu_alpha, glu_limit, glu_shift, 0, nullptr, nullptr, stream);
}

extern "C" int ttie_grouped_gemm_act(const void* A, long long lda, const int* row_of, int row_div, const void* W, long long w_stride,
                                     long long ldw, void* C, long long ldc, const int* tiles, const int* meta, int max_tiles, int N, int K,
                                     int dtype, int out_dtype, int few_rows, int glu_F, float glu_alpha, float glu_limit, float glu_shift,
                                     int act, const float* row_scale, const int* scale_of, void* stream) {
    if (max_tiles <= 0 || N <= 0) return 0;
    if (act < 0 || act > 1 || (glu_F > 0 && (act || row_scale))) TTIE_FAIL("grouped_gemm: activation %d (with a gated epilogue of width %d)", act, glu_F);
    const RowAct ra{act, row_scale, scale_of};
    if (max_tiles > 65535) TTIE_FAIL("grouped_gemm: %d row tiles in one launch", max_tiles);
    cudaStream_t s = (cudaStream_t)stream;
    const int vn = dtype == kF32 ? 4 : 8, esz = dtype == kF32 ? 4 : 2;
    if (few_rows && K % vn == 0 && lda % vn == 0 && ldw % vn == 0 && w_stride % vn == 0 && (((uintptr_t)A | (uintptr_t)W) & 15) == 0 && esz) {
        if (glu_F > 0 && N != 2 * glu_F) TTIE_FAIL("grouped_gemm: a gated epilogue of width %d on a matrix of %d rows", glu_F, N);
        const GluConst glu{glu_F, glu_alpha, glu_limit, glu_shift};
        const dim3 g(glu_F > 0 ? ceil_div(glu_F, GV_WARPS * GV_ROWS / 2) : ceil_div(N, GV_WARPS * GV_ROWS), max_tiles);
#define GV(TT, TO) TTIE_LAUNCH((grouped_gemv_kernel<TT, TO, 4>), g, GV_WARPS * 32, 0, s, (const TT*)A, lda, row_of, row_div > 0 ? row_div : 1, (const TT*)W, \
                               w_stride, ldw, (TO*)C, ldc, tiles, meta, N, K, glu, ra)
        if (dtype == kF32 && out_dtype == kF32) GV(float, float);
        else if (dtype == kBF16 && out_dtype == kBF16) GV(__nv_bfloat16, __nv_bfloat16);
        else if (dtype == kBF16 && out_dtype == kF32) GV(__nv_bfloat16, float);
        else TTIE_FAIL("grouped_gemm: operand dtype %d with output dtype %d", dtype, out_dtype);
#undef GV
        TTIE_CHECK_LAUNCH("grouped_gemm (few rows)");
        return 0;
    }
    if (glu_F > 0) TTIE_FAIL("grouped_gemm: the gated epilogue exists in the few-rows form only");
    const dim3 grid(ceil_div(N, BN), max_tiles);
#define GG(TT, TO) TTIE_LAUNCH((grouped_gemm_kernel<TT, TO>), grid, 256, 0, s, (const TT*)A, lda, row_of, row_div > 0 ? row_div : 1, (const TT*)W, \
                               w_stride, ldw, (TO*)C, ldc, tiles, meta, N, K, ra)
    if (dtype == kF32 && out_dtype == kF32) GG(float, float);
    else if (dtype == kBF16 && out_dtype == kBF16) GG(__nv_bfloat16, __nv_bfloat16);
    else if (dtype == kBF16 && out_dtype == kF32) GG(__nv_bfloat16, float);
    else TTIE_FAIL("grouped_gemm: operand dtype %d with output dtype %d", dtype, out_dtype);
#undef GG
    TTIE_CHECK_LAUNCH("grouped_gemm");
    return 0;
}

// dtype: of `shared`; y_dtype: of Y
extern "C" int ttie_gather_rows(const void* x, long long ldx, const int* row_of, int row_div, int rows, int d, void* out, int dtype, void* stream) {
    if (rows <= 0) return 0;
    const size_t total = (size_t)rows * d;
    if (dtype == kF32) TTIE_LAUNCH(gather_rows_kernel<float>, grid_for(total), 256, 0, (cudaStream_t)stream, (const float*)x, ldx, row_of, row_div > 0 ? row_div : 1, rows, d, (float*)out);
    else TTIE_LAUNCH(gather_rows_kernel<__nv_bfloat16>, grid_for(total), 256, 0, (cudaStream_t)stream, (const __nv_bfloat16*)x, ldx, row_of, row_div > 0 ? row_div : 1, rows, d, (__nv_bfloat16*)out);
    TTIE_CHECK_LAUNCH("gather_rows");
    return 0;
}

// idx, first_identity, x, ldx: the choices, the first identity expert and the tokens' own rows (compute dtype, row stride ldx);
// idx null: no identity experts
// wts null: every chosen expert's row counts once (its weight went in ahead of the expert); shared_gate: 32-bit logits, one per token
// ld_gate apart, whose sigmoid scales the shared expert's row (null: 1)
extern "C" int ttie_moe_combine_gated(const void* Y, int y_dtype, const int* pos_of_pair, const float* wts, const void* shared, int T, int d, int top,
                                      float* out, int dtype, const int* idx, int first_identity, const void* x, long long ldx,
                                      const float* shared_gate, long long ld_gate, void* stream);

extern "C" int ttie_moe_combine(const void* Y, int y_dtype, const int* pos_of_pair, const float* wts, const void* shared, int T, int d, int top,
                                float* out, int dtype, const int* idx, int first_identity, const void* x, long long ldx, void* stream) {
    return ttie_moe_combine_gated(Y, y_dtype, pos_of_pair, wts, shared, T, d, top, out, dtype, idx, first_identity, x, ldx, nullptr, 0, stream);
}

extern "C" int ttie_row_scale_act(void* x, long long ld, int rows, int F, int act, const float* row_scale, const int* scale_of, int dtype,
                                  void* stream) {
    if (rows <= 0 || F <= 0) return 0;
    if (act < 0 || act > 1) TTIE_FAIL("row_scale_act: activation %d", act);
    const RowAct ra{act, row_scale, scale_of};
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == kBF16 && F % 8 == 0 && ld % 8 == 0 && !((uintptr_t)x & 15))
        TTIE_LAUNCH(row_scale_act_vec8_kernel, grid_for((size_t)rows * F / 8), 256, 0, s, (__nv_bfloat16*)x, ld, rows, F / 8, ra);
    else if (dtype == kBF16) TTIE_LAUNCH(row_scale_act_kernel<__nv_bfloat16>, grid_for((size_t)rows * F), 256, 0, s, (__nv_bfloat16*)x, ld, rows, F, ra);
    else if (dtype == kF32) TTIE_LAUNCH(row_scale_act_kernel<float>, grid_for((size_t)rows * F), 256, 0, s, (float*)x, ld, rows, F, ra);
    else TTIE_FAIL("row_scale_act: unknown dtype %d", dtype);
    TTIE_CHECK_LAUNCH("row_scale_act");
    return 0;
}

extern "C" int ttie_moe_combine_gated(const void* Y, int y_dtype, const int* pos_of_pair, const float* wts, const void* shared, int T, int d, int top,
                                      float* out, int dtype, const int* idx, int first_identity, const void* x, long long ldx,
                                      const float* shared_gate, long long ld_gate, void* stream) {
    if (T <= 0) return 0;
    if (idx && !x) TTIE_FAIL("moe_combine: identity experts need the tokens' own rows");
    const size_t total = (size_t)T * d;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == kBF16 && y_dtype == kBF16 && d % 8 == 0 && ((((uintptr_t)Y) | ((uintptr_t)shared) | ((uintptr_t)out)) & 15) == 0
        && !(idx && ((((uintptr_t)x) & 15) || ldx % 8))) {
        TTIE_LAUNCH(moe_combine_vec8_kernel, grid_for(total / 8), 256, 0, s, (const __nv_bfloat16*)Y, pos_of_pair, wts, (const __nv_bfloat16*)shared, T, d / 8, top, out,
                    idx, first_identity, (const __nv_bfloat16*)x, ldx, shared_gate, ld_gate);
        TTIE_CHECK_LAUNCH("moe_combine");
        return 0;
    }
    if (dtype == kF32 && y_dtype == kF32) TTIE_LAUNCH((moe_combine_kernel<float, float>), grid_for(total), 256, 0, s, (const float*)Y, pos_of_pair, wts, (const float*)shared, T, d, top, out, idx, first_identity, (const float*)x, ldx, shared_gate, ld_gate);
    else if (y_dtype == kF32) TTIE_LAUNCH((moe_combine_kernel<__nv_bfloat16, float>), grid_for(total), 256, 0, s, (const float*)Y, pos_of_pair, wts, (const __nv_bfloat16*)shared, T, d, top, out, idx, first_identity, (const __nv_bfloat16*)x, ldx, shared_gate, ld_gate);
    else if (dtype == kBF16) TTIE_LAUNCH((moe_combine_kernel<__nv_bfloat16, __nv_bfloat16>), grid_for(total), 256, 0, s, (const __nv_bfloat16*)Y, pos_of_pair, wts, (const __nv_bfloat16*)shared, T, d, top, out, idx, first_identity, (const __nv_bfloat16*)x, ldx, shared_gate, ld_gate);
    else TTIE_FAIL("moe_combine: expert rows of dtype %d beside a shared expert of dtype %d", y_dtype, dtype);
    TTIE_CHECK_LAUNCH("moe_combine");
    return 0;
}
