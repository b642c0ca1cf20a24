// LayerNorm over the 32-bit residual stream with the scaled residual add fused in (post-norm layers):
//     s = alpha * x + delta;   x <- (s - mean(s)) / sqrt(mean((s - mean)^2) + eps) * w + b
// x stays in 32-bit (the stream is rewritten in place) and a copy in the compute dtype is written for the
// sub-layer that reads it next.  With a row list the rows are gathered and the stream is left alone (the
// model's last norm at the places whose logits are wanted).  The sum, both moments and the affine step are
// 32-bit; the variance is the mean of the squared deviations (two passes over the row held in shared memory).
// delta: none, [R, d] in the compute dtype or in 32-bit, or 32-bit partial sums [S, R, d] of a K-split product.
// add_normed (layers that norm a sub-layer's output, not its input): the moments are those of delta alone and the stream
// takes the normed delta on top of what it holds,  x <- x + (delta - mean(delta)) / sqrt(var(delta) + eps) * w + b;  the
// copy in the compute dtype is of the new x.  A layer scale is folded into w by the caller.
#include "common.cuh"
using namespace ttie;

namespace {

template <typename T, typename W>
__global__ void __launch_bounds__(256)
scale_add_layernorm_kernel(float* __restrict__ resid, const T* __restrict__ delta, const float* __restrict__ dpart, int S,
                           long long part_stride, const int* __restrict__ rows, const W* __restrict__ weight,
                           const W* __restrict__ bias, T* __restrict__ out, float* __restrict__ out32, int d, float alpha, float eps,
                           int write_resid, int add_normed) {
    extern __shared__ float row[];
    __shared__ float scratch[32];
    TTIE_PDL_ENTRY();
    const int r = blockIdx.x;
    const size_t src = rows ? (size_t)rows[r] : (size_t)r;
    float* x = resid + src * d;
    float sum = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float v = add_normed ? 0.f : alpha * x[i];
        if (delta) v += to_f32(delta[src * d + i]);
        for (int s = 0; s < S; ++s) v += dpart[(size_t)s * part_stride + src * d + i];     // fixed order
        row[i] = v;
        sum += v;
    }
    const float mean = block_sum(sum, scratch) / (float)d;
    float sq = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) { const float c = row[i] - mean; sq += c * c; }
    const float rstd = 1.0f / sqrtf(block_sum(sq, scratch) / (float)d + eps);
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float y = (row[i] - mean) * rstd * to_f32(weight[i]) + (bias ? to_f32(bias[i]) : 0.f);
        if (add_normed) y += x[i];
        if (write_resid) x[i] = y;
        if (out) out[(size_t)r * d + i] = from_f32<T>(y);
        if (out32) out32[(size_t)r * d + i] = y;
    }
}

// The same with the row in registers: up to PER elements per thread, every load of the row (stream, delta, weight, bias)
// asked for before the first reduction, so a row costs one trip to memory and two block reductions.
template <typename T, typename W, int PER>
__global__ void __launch_bounds__(1024)
scale_add_layernorm_reg_kernel(float* __restrict__ resid, const T* __restrict__ delta, const float* __restrict__ dpart, int S,
                               long long part_stride, const int* __restrict__ rows, const W* __restrict__ weight,
                               const W* __restrict__ bias, T* __restrict__ out, float* __restrict__ out32, int d, float alpha, float eps,
                               int write_resid, int add_normed) {
    __shared__ float scratch[32];
    TTIE_PDL_ENTRY();
    const int r = blockIdx.x;
    const size_t src = rows ? (size_t)rows[r] : (size_t)r;
    float* x = resid + src * d;
    float v[PER], w[PER], b[PER], keep[PER];
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        v[j] = 0.f; w[j] = 0.f; b[j] = 0.f; keep[j] = 0.f;
        if (i < d) {
            if (add_normed) keep[j] = x[i]; else v[j] = alpha * x[i];
            if (delta) v[j] += to_f32(delta[src * d + i]);
            w[j] = to_f32(weight[i]);
            b[j] = bias ? to_f32(bias[i]) : 0.f;
        }
    }
    for (int s = 0; s < S; ++s)
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const int i = threadIdx.x + j * blockDim.x;
            if (i < d) v[j] += dpart[(size_t)s * part_stride + src * d + i];               // fixed order
        }
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < PER; ++j) sum += v[j];
    const float mean = block_sum(sum, scratch) / (float)d;
    float sq = 0.f;
#pragma unroll
    for (int j = 0; j < PER; ++j) { const float c = (threadIdx.x + j * blockDim.x < d) ? v[j] - mean : 0.f; sq += c * c; }
    const float rstd = 1.0f / sqrtf(block_sum(sq, scratch) / (float)d + eps);
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i >= d) continue;
        const float y = (v[j] - mean) * rstd * w[j] + b[j] + keep[j];
        if (write_resid) x[i] = y;
        if (out) out[(size_t)r * d + i] = from_f32<T>(y);
        if (out32) out32[(size_t)r * d + i] = y;
    }
}

// Four values per load (d a multiple of 4): two such vectors per thread.
__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ld4(const __nv_bfloat16* p) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x)), b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void st4(__nv_bfloat16* p, float4 v) {
    uint2 o;
    *reinterpret_cast<__nv_bfloat162*>(&o.x) = __floats2bfloat162_rn(v.x, v.y);
    *reinterpret_cast<__nv_bfloat162*>(&o.y) = __floats2bfloat162_rn(v.z, v.w);
    *reinterpret_cast<uint2*>(p) = o;
}

template <typename T, typename W>
__global__ void __launch_bounds__(1024)
scale_add_layernorm_vec_kernel(float* __restrict__ resid, const T* __restrict__ delta, const float* __restrict__ dpart, int S,
                               long long part_stride, const int* __restrict__ rows, const W* __restrict__ weight,
                               const W* __restrict__ bias, T* __restrict__ out, float* __restrict__ out32, int d, float alpha, float eps,
                               int write_resid, int add_normed) {
    constexpr int PER = 2;
    __shared__ float scratch[32];
    TTIE_PDL_ENTRY();
    const int r = blockIdx.x;
    const size_t src = rows ? (size_t)rows[r] : (size_t)r;
    float* x = resid + src * d;
    float4 v[PER], w[PER], b[PER], keep[PER];
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const int i = (threadIdx.x + j * blockDim.x) * 4;
        v[j] = w[j] = b[j] = keep[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < d) {
            const float4 xv = ld4(x + i);
            if (add_normed) keep[j] = xv; else v[j] = make_float4(alpha * xv.x, alpha * xv.y, alpha * xv.z, alpha * xv.w);
            if (delta) { const float4 dv = ld4(delta + src * d + i); v[j].x += dv.x; v[j].y += dv.y; v[j].z += dv.z; v[j].w += dv.w; }
            w[j] = ld4(weight + i);
            if (bias) b[j] = ld4(bias + i);
        }
    }
    for (int s = 0; s < S; ++s)
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            const int i = (threadIdx.x + j * blockDim.x) * 4;
            if (i < d) { const float4 p = ld4(dpart + (size_t)s * part_stride + src * d + i); v[j].x += p.x; v[j].y += p.y; v[j].z += p.z; v[j].w += p.w; }
        }
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < PER; ++j) sum += (v[j].x + v[j].y) + (v[j].z + v[j].w);
    const float mean = block_sum(sum, scratch) / (float)d;
    float sq = 0.f;
#pragma unroll
    for (int j = 0; j < PER; ++j)
        if ((threadIdx.x + j * blockDim.x) * 4 < d) {
            const float a0 = v[j].x - mean, a1 = v[j].y - mean, a2 = v[j].z - mean, a3 = v[j].w - mean;
            sq += (a0 * a0 + a1 * a1) + (a2 * a2 + a3 * a3);
        }
    const float rstd = 1.0f / sqrtf(block_sum(sq, scratch) / (float)d + eps);
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const int i = (threadIdx.x + j * blockDim.x) * 4;
        if (i >= d) continue;
        const float4 y = make_float4((v[j].x - mean) * rstd * w[j].x + b[j].x + keep[j].x, (v[j].y - mean) * rstd * w[j].y + b[j].y + keep[j].y,
                                     (v[j].z - mean) * rstd * w[j].z + b[j].z + keep[j].z, (v[j].w - mean) * rstd * w[j].w + b[j].w + keep[j].w);
        if (write_resid) st4(x + i, y);
        if (out) st4(out + (size_t)r * d + i, y);
        if (out32) st4(out32 + (size_t)r * d + i, y);
    }
}

template <typename T>
__global__ void cast_rows_kernel(const float* __restrict__ in, T* __restrict__ out, size_t n) {
    TTIE_PDL_ENTRY();
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) out[i] = from_f32<T>(in[i]);
}

template <typename T, typename W>
int launch_ln(float* resid, const void* delta, const float* dpart, int S, long long part_stride, const int* rows, const void* w,
              const void* b, void* out, float* out32, int R, int d, float alpha, float eps, int write_resid, int add_normed, cudaStream_t s) {
    const uintptr_t all = (uintptr_t)resid | (uintptr_t)delta | (uintptr_t)dpart | (uintptr_t)w | (uintptr_t)b | (uintptr_t)out | (uintptr_t)out32;
    if (d % 4 == 0 && d <= 8 * 1024 && (all & 15) == 0 && part_stride % 4 == 0) {
        const int threads = ((d / 8 + 31) / 32) * 32 < 32 ? 32 : ((d / 8 + 31) / 32) * 32;
        TTIE_LAUNCH((scale_add_layernorm_vec_kernel<T, W>), R, threads, 0, s, resid, (const T*)delta, dpart, S, part_stride, rows,
                    (const W*)w, (const W*)b, (T*)out, out32, d, alpha, eps, write_resid, add_normed);
        TTIE_CHECK_LAUNCH("scale_add_layernorm");
        return 0;
    }
    if (d <= 8 * 1024) {
        const int threads = d <= 1024 ? 128 : d <= 2048 ? 256 : d <= 4096 ? 512 : 1024;
        TTIE_LAUNCH((scale_add_layernorm_reg_kernel<T, W, 8>), R, threads, 0, s, resid, (const T*)delta, dpart, S, part_stride, rows,
                    (const W*)w, (const W*)b, (T*)out, out32, d, alpha, eps, write_resid, add_normed);
        TTIE_CHECK_LAUNCH("scale_add_layernorm");
        return 0;
    }
    TTIE_LAUNCH((scale_add_layernorm_kernel<T, W>), R, 256, (size_t)d * sizeof(float), s, resid, (const T*)delta, dpart, S, part_stride, rows,
                (const W*)w, (const W*)b, (T*)out, out32, d, alpha, eps, write_resid, add_normed);
    TTIE_CHECK_LAUNCH("scale_add_layernorm");
    return 0;
}
}  // namespace

// delta_dtype: the dtype code of `delta` (ignored if null); out_dtype: of `out`; w_dtype: of weight and bias.
extern "C" int ttie_scale_add_layernorm(float* resid, const void* delta, int delta_dtype, const float* dpart, int S, long long part_stride,
                                        const int* rows, const void* weight, const void* bias, int w_dtype, void* out, int out_dtype,
                                        int R, int d, float alpha, float eps, int write_resid, int add_normed, void* stream) {
    if (R <= 0) return 0;
    if (d <= 0 || (size_t)d * sizeof(float) > 200 * 1024) TTIE_FAIL("layernorm: width %d not supported", d);
    cudaStream_t s = (cudaStream_t)stream;
    static bool big = false;
    if ((size_t)d * sizeof(float) > 48 * 1024 && !big) {
        cudaFuncSetAttribute(scale_add_layernorm_kernel<float, float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        cudaFuncSetAttribute(scale_add_layernorm_kernel<__nv_bfloat16, float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        cudaFuncSetAttribute(scale_add_layernorm_kernel<__nv_bfloat16, __nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        big = true;
    }
    // a 32-bit delta beside a bfloat16 output goes in as one partial sum
    if (delta && delta_dtype == kF32 && out_dtype == kBF16) {
        if (S) TTIE_FAIL("layernorm: a 32-bit delta and partial sums together");
        dpart = (const float*)delta; S = 1; part_stride = 0; delta = nullptr;
    }
    if (delta && delta_dtype != out_dtype) TTIE_FAIL("layernorm: delta dtype %d with output dtype %d", delta_dtype, out_dtype);
    if (out_dtype == kF32) {
        if (w_dtype != kF32) TTIE_FAIL("layernorm: a 32-bit run needs 32-bit norm weights");
        return launch_ln<float, float>(resid, delta, dpart, S, part_stride, rows, weight, bias, nullptr, (float*)out, R, d, alpha, eps, write_resid, add_normed, s);
    }
    if (w_dtype == kF32)
        return launch_ln<__nv_bfloat16, float>(resid, delta, dpart, S, part_stride, rows, weight, bias, out, nullptr, R, d, alpha, eps, write_resid, add_normed, s);
    return launch_ln<__nv_bfloat16, __nv_bfloat16>(resid, delta, dpart, S, part_stride, rows, weight, bias, out, nullptr, R, d, alpha, eps, write_resid, add_normed, s);
}

extern "C" int ttie_cast_rows(const float* in, void* out, long long n, int out_dtype, void* stream) {
    if (n <= 0) return 0;
    const int grid = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
    if (out_dtype == kBF16) TTIE_LAUNCH(cast_rows_kernel<__nv_bfloat16>, grid, 256, 0, (cudaStream_t)stream, in, (__nv_bfloat16*)out, (size_t)n);
    else TTIE_LAUNCH(cast_rows_kernel<float>, grid, 256, 0, (cudaStream_t)stream, in, (float*)out, (size_t)n);
    TTIE_CHECK_LAUNCH("cast_rows");
    return 0;
}
