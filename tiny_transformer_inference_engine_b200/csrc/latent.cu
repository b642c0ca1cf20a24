// Helpers of latent attention: attention whose cache holds, per token, one low-rank latent vector c (RMS-normed) and one
// rotated key part shared by all heads.  With the key up-projection folded into the query (q' = W_uk^T q) every head
// attends over the same cache rows [c | rotated part | zero padding], which also serve as the values: the paged attention
// kernels run it as multi-query attention whose key and value pages are the same array.
//   latent_store:  proj[t, col0 : col0 + rank + rot]  ->  page row (RMS norm with weight on the first `rank`, rotation of
//                  the last `rot` by the token's position), all in 32-bit, rounded once when stored
//   latent_query:  per head [folded query (rank) | rotated query part (rot) | zeros] in the attention kernels' layout
//   gate_heads:    out[t, h, :] = v[h, t, :] * sigmoid(gate[t, h]), or with a gate per value sigmoid(gate[t, h * vdim + j])
//   rmsnorm_cols:  out[t, :] = proj[t, col0 : col0 + width] / rms * weight (a query latent between its two projections), 32-bit inside
#include "common.cuh"
using namespace ttie;

namespace {

// one warp per token
template <typename T, typename W>
__global__ void __launch_bounds__(128)
latent_store_kernel(const T* __restrict__ proj, long long ld, int col0, int T_, int rank, int rot, int width,
                    const W* __restrict__ norm_w, float eps, const float2* __restrict__ cs, const int* __restrict__ positions,
                    const int* __restrict__ token_seq, T* __restrict__ pages, const int* __restrict__ block_table, int bt_stride,
                    int page_size, int num_pages) {
    TTIE_PDL_ENTRY();
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (t >= T_) return;
    const T* src = proj + (size_t)t * ld + col0;
    const int pos = positions[t];
    const int page = block_table[(size_t)token_seq[t] * bt_stride + pos / page_size];
    if (page < 0 || page >= num_pages) return;
    T* dst = pages + ((size_t)page * page_size + pos % page_size) * width;
    float sq = 0.f;
    for (int i = lane; i < rank; i += 32) { const float v = to_f32(src[i]); sq += v * v; }
    sq = warp_sum(sq);
    const float r = 1.0f / sqrtf(sq / (float)rank + eps);
    for (int i = lane; i < rank; i += 32) dst[i] = from_f32<T>(to_f32(src[i]) * r * to_f32(norm_w[i]));
    const int half = rot >> 1;
    for (int j = lane; j < half; j += 32) {
        const float2 c = cs[(size_t)t * half + j];
        const float u = to_f32(src[rank + 2 * j]), v = to_f32(src[rank + 2 * j + 1]);
        dst[rank + 2 * j] = from_f32<T>(u * c.x - v * c.y);
        dst[rank + 2 * j + 1] = from_f32<T>(v * c.x + u * c.y);
    }
    for (int i = rank + rot + lane; i < width; i += 32) dst[i] = from_f32<T>(0.f);
}

// one warp per token: columns col0 .. col0 + width of a projected row over their root mean square, times a weight
template <typename T, typename W>
__global__ void __launch_bounds__(128)
rmsnorm_cols_kernel(const T* __restrict__ proj, long long ld, int col0, int T_, int width, const W* __restrict__ w, float eps, T* __restrict__ out) {
    TTIE_PDL_ENTRY();
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (t >= T_) return;
    const T* src = proj + (size_t)t * ld + col0;
    float sq = 0.f;
    for (int i = lane; i < width; i += 32) { const float v = to_f32(src[i]); sq = fmaf(v, v, sq); }
    sq = warp_sum(sq);
    const float r = 1.0f / sqrtf(sq / (float)width + eps);
    for (int i = lane; i < width; i += 32) out[(size_t)t * width + i] = from_f32<T>(to_f32(src[i]) * r * to_f32(w[i]));
}

// q [T, H * (dim + rot)] (row stride ld), folded [H, T, rank] -> out [T, H, width]
template <typename T>
__global__ void latent_query_kernel(const T* __restrict__ q, long long ld, const T* __restrict__ folded, int T_, int H, int dim,
                                    int rank, int rot, int width, const float2* __restrict__ cs, T* __restrict__ out) {
    TTIE_PDL_ENTRY();
    const int half = rot >> 1, per_row = H * width;
    const int col = blockIdx.x * blockDim.x + threadIdx.x;           // grid: (columns of a token's row, tokens)
    if (col >= per_row) return;
    const int h = col / width, i = col - h * width;
    for (size_t t = blockIdx.y; t < (size_t)T_; t += gridDim.y) {
        const size_t e = t * per_row + col;
        float v = 0.f;
        if (i < rank) {
            v = to_f32(folded[((size_t)h * T_ + t) * rank + i]);
        } else if (i < rank + rot) {
            const int k = i - rank, j = k >> 1;
            const T* qr = q + t * ld + (size_t)h * (dim + rot) + dim;
            const float2 c = cs[t * half + j];
            const float a = to_f32(qr[2 * j]), b = to_f32(qr[2 * j + 1]);
            v = (k & 1) ? (b * c.x + a * c.y) : (a * c.x - b * c.y);
        }
        out[e] = from_f32<T>(v);
    }
}

// v [H, T, vdim]; gate logits gate[t * ld + h]; out [T, H * vdim]
template <typename T>
__global__ void gate_heads_kernel(const T* __restrict__ v, const T* __restrict__ gate, long long ld, int per_value, int T_, int H, int vdim,
                                  T* __restrict__ out) {
    TTIE_PDL_ENTRY();
    const int per_row = H * vdim;
    const int col = blockIdx.x * blockDim.x + threadIdx.x;           // grid: (columns of a token's row, tokens)
    if (col >= per_row) return;
    const int h = col / vdim, j = col - h * vdim;
    for (size_t t = blockIdx.y; t < (size_t)T_; t += gridDim.y) {
        const size_t e = t * per_row + col;
        const float g = 1.0f / (1.0f + expf(-to_f32(gate[t * ld + (per_value ? col : h)])));
        out[e] = from_f32<T>(to_f32(v[((size_t)h * T_ + t) * vdim + j]) * g);
    }
}

// ---- bfloat16, eight values per thread (every size a multiple of 8, rows 16-byte aligned)
__device__ __forceinline__ uint4 scale8(const uint4 v, float g) {
    uint4 o;
    const __nv_bfloat162* a = reinterpret_cast<const __nv_bfloat162*>(&v);
    __nv_bfloat162* b = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(a[i]); b[i] = __floats2bfloat162_rn(f.x * g, f.y * g); }
    return o;
}

__global__ void latent_query_vec8_kernel(const __nv_bfloat16* __restrict__ q, long long ld, const __nv_bfloat16* __restrict__ folded, int T_,
                                         int H, int dim, int rank, int rot, int width, const float2* __restrict__ cs,
                                         __nv_bfloat16* __restrict__ out) {
    TTIE_PDL_ENTRY();
    const int half = rot >> 1, per_row = H * width;
    const int col = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (col >= per_row) return;
    const int h = col / width, i = col - h * width;
    for (size_t t = blockIdx.y; t < (size_t)T_; t += gridDim.y) {
        uint4 o = make_uint4(0u, 0u, 0u, 0u);
        if (i < rank) {
            o = *reinterpret_cast<const uint4*>(folded + ((size_t)h * T_ + t) * rank + i);
        } else if (i < rank + rot) {
            const int k = i - rank;
            const uint4 v = *reinterpret_cast<const uint4*>(q + t * ld + (size_t)h * (dim + rot) + dim + k);
            const __nv_bfloat162* a = reinterpret_cast<const __nv_bfloat162*>(&v);
            __nv_bfloat162* b = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
            for (int p = 0; p < 4; ++p) {
                const float2 c = cs[t * half + (k >> 1) + p];
                const float2 f = __bfloat1622float2(a[p]);
                b[p] = __floats2bfloat162_rn(f.x * c.x - f.y * c.y, f.y * c.x + f.x * c.y);
            }
        }
        *reinterpret_cast<uint4*>(out + t * per_row + col) = o;
    }
}

__global__ void gate_heads_vec8_kernel(const __nv_bfloat16* __restrict__ v, const __nv_bfloat16* __restrict__ gate, long long ld, int per_value,
                                       int T_, int H, int vdim, __nv_bfloat16* __restrict__ out) {
    TTIE_PDL_ENTRY();
    const int per_row = H * vdim;
    const int col = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (col >= per_row) return;
    const int h = col / vdim, j = col - h * vdim;
    for (size_t t = blockIdx.y; t < (size_t)T_; t += gridDim.y) {
        const uint4 x = *reinterpret_cast<const uint4*>(v + ((size_t)h * T_ + t) * vdim + j);
        if (per_value) {                                             // (the gate row is 16-byte aligned like the others: the caller checks)
            const uint4 gv = *reinterpret_cast<const uint4*>(gate + t * ld + col);
            const __nv_bfloat162* a = reinterpret_cast<const __nv_bfloat162*>(&x);
            const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
            uint4 y;
            __nv_bfloat162* b = reinterpret_cast<__nv_bfloat162*>(&y);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __bfloat1622float2(a[i]), g = __bfloat1622float2(g2[i]);
                b[i] = __floats2bfloat162_rn(f.x / (1.0f + expf(-g.x)), f.y / (1.0f + expf(-g.y)));
            }
            *reinterpret_cast<uint4*>(out + t * per_row + col) = y;
            continue;
        }
        const float g = 1.0f / (1.0f + expf(-__bfloat162float(gate[t * ld + h])));
        *reinterpret_cast<uint4*>(out + t * per_row + col) = scale8(x, g);
    }
}

inline bool aligned16(const void* p) { return (((uintptr_t)p) & 15) == 0; }
inline int grid_for(size_t total) { return (int)((total + 255) / 256 < 8192 ? (total + 255) / 256 : 8192); }
}  // namespace

extern "C" int ttie_latent_store(const void* proj, long long ld, int col0, int T, int rank, int rot, int width, const void* norm_w,
                                 int w_dtype, float eps, const void* cs, const int* positions, const int* token_seq, void* pages,
                                 const int* block_table, int bt_stride, int page_size, int num_pages, int dtype, void* stream) {
    if (T <= 0) return 0;
    if (rot % 2 || rank <= 0 || width < rank + rot) TTIE_FAIL("latent_store: rank %d, rotated %d, row width %d", rank, rot, width);
    cudaStream_t s = (cudaStream_t)stream;
    const int grid = ceil_div(T, 4);
#define LS(TT, WW) TTIE_LAUNCH((latent_store_kernel<TT, WW>), grid, 128, 0, s, (const TT*)proj, ld, col0, T, rank, rot, width, (const WW*)norm_w, \
                               eps, (const float2*)cs, positions, token_seq, (TT*)pages, block_table, bt_stride, page_size, num_pages)
    if (dtype == kF32) { if (w_dtype != kF32) TTIE_FAIL("latent_store: a 32-bit run needs 32-bit norm weights"); LS(float, float); }
    else if (w_dtype == kF32) LS(__nv_bfloat16, float);
    else LS(__nv_bfloat16, __nv_bfloat16);
#undef LS
    TTIE_CHECK_LAUNCH("latent_store");
    return 0;
}

extern "C" int ttie_rmsnorm_cols(const void* proj, long long ld, int col0, int T, int width, const void* w, int w_dtype, float eps, void* out,
                                 int dtype, void* stream) {
    if (T <= 0) return 0;
    if (width <= 0) TTIE_FAIL("rmsnorm_cols: width %d", width);
    cudaStream_t s = (cudaStream_t)stream;
    const int grid = ceil_div(T, 4);
#define RC(TT, WW) TTIE_LAUNCH((rmsnorm_cols_kernel<TT, WW>), grid, 128, 0, s, (const TT*)proj, ld, col0, T, width, (const WW*)w, eps, (TT*)out)
    if (dtype == kF32) { if (w_dtype != kF32) TTIE_FAIL("rmsnorm_cols: a 32-bit run needs 32-bit norm weights"); RC(float, float); }
    else if (w_dtype == kF32) RC(__nv_bfloat16, float);
    else RC(__nv_bfloat16, __nv_bfloat16);
#undef RC
    TTIE_CHECK_LAUNCH("rmsnorm_cols");
    return 0;
}

extern "C" int ttie_latent_query(const void* q, long long ld, const void* folded, int T, int H, int dim, int rank, int rot, int width,
                                 const void* cs, void* out, int dtype, void* stream) {
    if (T <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == kBF16 && rank % 8 == 0 && rot % 8 == 0 && dim % 8 == 0 && width % 8 == 0 && ld % 8 == 0 && aligned16(q) && aligned16(folded) && aligned16(out)) {
        const dim3 g8(ceil_div(H * width / 8, 128), T < 65535 ? T : 65535);
        TTIE_LAUNCH(latent_query_vec8_kernel, g8, 128, 0, s, (const __nv_bfloat16*)q, ld, (const __nv_bfloat16*)folded, T, H, dim, rank, rot, width,
                    (const float2*)cs, (__nv_bfloat16*)out);
        TTIE_CHECK_LAUNCH("latent_query");
        return 0;
    }
    const dim3 grid(ceil_div(H * width, 256), T < 65535 ? T : 65535);
    if (dtype == kF32) TTIE_LAUNCH(latent_query_kernel<float>, grid, 256, 0, s, (const float*)q, ld, (const float*)folded, T, H, dim, rank, rot, width, (const float2*)cs, (float*)out);
    else TTIE_LAUNCH(latent_query_kernel<__nv_bfloat16>, grid, 256, 0, s, (const __nv_bfloat16*)q, ld, (const __nv_bfloat16*)folded, T, H, dim, rank, rot, width, (const float2*)cs, (__nv_bfloat16*)out);
    TTIE_CHECK_LAUNCH("latent_query");
    return 0;
}

extern "C" int ttie_gate_heads(const void* v, const void* gate, long long ld, int per_value, int T, int H, int vdim, void* out, int dtype,
                               void* stream) {
    if (T <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == kBF16 && vdim % 8 == 0 && aligned16(v) && aligned16(out) && !(per_value && (!aligned16(gate) || ld % 8))) {
        const dim3 g8(ceil_div(H * vdim / 8, 128), T < 65535 ? T : 65535);
        TTIE_LAUNCH(gate_heads_vec8_kernel, g8, 128, 0, s, (const __nv_bfloat16*)v, (const __nv_bfloat16*)gate, ld, per_value, T, H, vdim, (__nv_bfloat16*)out);
        TTIE_CHECK_LAUNCH("gate_heads");
        return 0;
    }
    const dim3 grid(ceil_div(H * vdim, 256), T < 65535 ? T : 65535);
    if (dtype == kF32) TTIE_LAUNCH(gate_heads_kernel<float>, grid, 256, 0, s, (const float*)v, (const float*)gate, ld, per_value, T, H, vdim, (float*)out);
    else TTIE_LAUNCH(gate_heads_kernel<__nv_bfloat16>, grid, 256, 0, s, (const __nv_bfloat16*)v, (const __nv_bfloat16*)gate, ld, per_value, T, H, vdim, (__nv_bfloat16*)out);
    TTIE_CHECK_LAUNCH("gate_heads");
    return 0;
}
