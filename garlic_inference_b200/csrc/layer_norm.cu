// Row-wise kernels around a mean-subtracting norm.
//
//   gi_add_layernorm   s = x (+ delta (+ delta2));  out = (s - mean(s)) / sqrt(var(s) + eps) * w (+ b), var the mean
//                      of the squared deviations; with write_residual the float32 sum goes back into x; `rows`
//                      picks input rows (nothing is written back then).  Two pending results serve arrangements
//                      whose mixer and feed-forward read one normed input and join the stream together.
//   gi_rmsnorm_rows    out = z / sqrt(mean(z^2) + eps) * w for rows that may be columns of a wider matrix (a
//                      latent between a down- and an up-projection)
//   gi_softcap         z <- cap * tanh(z / cap) in place, float32 (logits)
//
// Everything is float32 inside and rounded once on the way out; T is the activation type.  The block size depends
// on the row's width alone and sums run in a fixed order, so a row's result does not depend on what else is in
// the launch.  The mean is taken first and the variance from the deviations (two passes over registers or shared
// memory, one over global memory).  NikolayBlagoev/garlic-inference has RMSNorm only (src/src-cuda/norm.cu:3-101).
#include "common.cuh"
#include <math.h>

#define LN_MAX_PER_THREAD 16          // elements a thread keeps in registers: rows up to 512 * 16

template <typename T>
__global__ void __launch_bounds__(512)
add_layernorm_kernel(const T* __restrict__ delta, const T* __restrict__ delta2, float* __restrict__ residual,
                     const void* __restrict__ weight, const void* __restrict__ bias, int w_dtype, T* __restrict__ out,
                     const int* __restrict__ rows, int dim, float eps, int write_residual) {
    gi_pdl_start();
    __shared__ float red[33];
    const int r = blockIdx.x;
    const size_t i = rows ? (size_t)rows[r] : (size_t)r;
    float* res = residual + i * dim;
    const T* d1 = delta ? delta + i * dim : nullptr;
    const T* d2 = delta2 ? delta2 + i * dim : nullptr;
    float v[LN_MAX_PER_THREAD];
    float sum = 0.f;
#pragma unroll
    for (int it = 0; it < LN_MAX_PER_THREAD; ++it) {
        const int c = it * blockDim.x + threadIdx.x;
        v[it] = 0.f;
        if (c < dim) {
            float s = res[c];
            if (d1 && d2) s += to_f32(d1[c]) + to_f32(d2[c]);      // the sublayers' results are summed first
            else if (d1) s += to_f32(d1[c]);
            else if (d2) s += to_f32(d2[c]);
            if (write_residual && (d1 || d2)) res[c] = s;
            v[it] = s;
            sum += s;
        }
    }
    const float mean = block_sum(sum, red) / (float)dim;
    float sq = 0.f;
#pragma unroll
    for (int it = 0; it < LN_MAX_PER_THREAD; ++it) {
        const int c = it * blockDim.x + threadIdx.x;
        if (c < dim) { const float d = v[it] - mean; sq += d * d; }
    }
    const float inv = 1.f / sqrtf(block_sum(sq, red) / (float)dim + eps);
    T* o = out + (size_t)r * dim;
#pragma unroll
    for (int it = 0; it < LN_MAX_PER_THREAD; ++it) {
        const int c = it * blockDim.x + threadIdx.x;
        if (c < dim) {
            float y = (v[it] - mean) * inv * load_w(weight, w_dtype, c);
            if (bias) y += load_w(bias, w_dtype, c);
            o[c] = from_f32<T>(y);
        }
    }
}

// The same with four elements per thread and load (16-byte words of the stream, 8-byte words of bfloat16 results),
// the row in registers.  Taken when the width is a multiple of 4, at most 8,192, and everything starts on 16 bytes;
// the thread count depends on the width alone.  EARLY_W: the weight is fetched before the wait for the kernel that
// makes the pending results (it is nobody's output), which pays for a few rows.
#define LN_VEC_MAX_IT 8
template <typename T, int EARLY_W>
__global__ void __launch_bounds__(256)
add_layernorm_vec_kernel(const T* __restrict__ delta, const T* __restrict__ delta2, float* __restrict__ residual,
                         const void* __restrict__ weight, const void* __restrict__ bias, int w_dtype, T* __restrict__ out,
                         const int* __restrict__ rows, int dim, float eps, int write_residual) {
    gi_pdl_launch_dependents();
    __shared__ float red[33];
    const int r = blockIdx.x;
    float4 w4[EARLY_W ? LN_VEC_MAX_IT : 1];
    if (EARLY_W) {
#pragma unroll
        for (int it = 0; it < LN_VEC_MAX_IT; ++it) {
            const int c = (it * blockDim.x + threadIdx.x) * 4;
            if (c < dim) w4[it] = load4_w(weight, w_dtype, c);
        }
        if (!rows) {                                   // the stream's lines are asked back into L2 (a hint)
            const float* line = residual + (size_t)r * dim + threadIdx.x * 32;
            if (threadIdx.x * 32 < dim) asm volatile("prefetch.global.L2 [%0];" ::"l"(line));
        }
    }
    gi_pdl_wait();
    const size_t i = rows ? (size_t)rows[r] : (size_t)r;
    float* res = residual + i * dim;
    const T* d1 = delta ? delta + i * dim : nullptr;
    const T* d2 = delta2 ? delta2 + i * dim : nullptr;
    float4 v[LN_VEC_MAX_IT];
    float sum = 0.f;
#pragma unroll
    for (int it = 0; it < LN_VEC_MAX_IT; ++it) {
        const int c = (it * blockDim.x + threadIdx.x) * 4;
        if (c < dim) {
            float4 s = load4_f32(res + c);
            if (d1 && d2) {                            // the sublayers' results are summed first
                const float4 a = load4_act(d1 + c), b = load4_act(d2 + c);
                s.x += a.x + b.x; s.y += a.y + b.y; s.z += a.z + b.z; s.w += a.w + b.w;
            } else if (d1 || d2) {
                const float4 a = load4_act((d1 ? d1 : d2) + c);
                s.x += a.x; s.y += a.y; s.z += a.z; s.w += a.w;
            }
            if (write_residual && (d1 || d2)) *reinterpret_cast<float4*>(res + c) = s;
            v[it] = s;
            sum += s.x;                                // the same order of additions whatever the batch is
            sum += s.y;
            sum += s.z;
            sum += s.w;
        }
    }
    const float mean = block_sum(sum, red) / (float)dim;
    float sq = 0.f;
#pragma unroll
    for (int it = 0; it < LN_VEC_MAX_IT; ++it) {
        const int c = (it * blockDim.x + threadIdx.x) * 4;
        if (c < dim) {
            v[it].x -= mean; v[it].y -= mean; v[it].z -= mean; v[it].w -= mean;
            sq += v[it].x * v[it].x;
            sq += v[it].y * v[it].y;
            sq += v[it].z * v[it].z;
            sq += v[it].w * v[it].w;
        }
    }
    const float inv = 1.f / sqrtf(block_sum(sq, red) / (float)dim + eps);
    T* o = out + (size_t)r * dim;
#pragma unroll
    for (int it = 0; it < LN_VEC_MAX_IT; ++it) {
        const int c = (it * blockDim.x + threadIdx.x) * 4;
        if (c < dim) {
            const float4 w = EARLY_W ? w4[EARLY_W ? it : 0] : load4_w(weight, w_dtype, c);
            float4 y = make_float4(v[it].x * inv * w.x, v[it].y * inv * w.y, v[it].z * inv * w.z, v[it].w * inv * w.w);
            if (bias) {
                const float4 b = load4_w(bias, w_dtype, c);
                y.x += b.x; y.y += b.y; y.z += b.z; y.w += b.w;
            }
            store4_act(o + c, y);
        }
    }
}

extern "C" int gi_add_layernorm(const void* delta, const void* delta2, float* residual, const void* weight,
                                const void* bias, int w_dtype, void* out, int act_dtype, const int* rows, int n_rows,
                                int dim, float eps, int write_residual, void* stream) {
    GI_REQUIRE(n_rows >= 0 && dim > 0, "gi_add_layernorm: sizes must be positive");
    GI_REQUIRE(dim <= 512 * LN_MAX_PER_THREAD, "gi_add_layernorm: rows of %d are wider than %d", dim, 512 * LN_MAX_PER_THREAD);
    GI_REQUIRE(w_dtype == GI_DTYPE_F32 || w_dtype == GI_DTYPE_BF16, "gi_add_layernorm: weight dtype %d", w_dtype);
    GI_REQUIRE(!(rows && write_residual), "gi_add_layernorm: gathered rows cannot write the residual back");
    if (n_rows == 0) return 0;
    const bool aligned = ((uintptr_t)residual % 16 == 0) && ((uintptr_t)out % 16 == 0) && ((uintptr_t)weight % 16 == 0) &&
                         ((uintptr_t)bias % 16 == 0) && ((uintptr_t)delta % 16 == 0) && ((uintptr_t)delta2 % 16 == 0);
    if (dim % 4 == 0 && dim <= 256 * 4 * LN_VEC_MAX_IT && aligned) {
        int vt = ((dim / 4 + 31) / 32) * 32;
        vt = vt > 256 ? 256 : vt;
        const bool early = n_rows <= 256;
        cudaStream_t vs = (cudaStream_t)stream;
#define LAUNCH_LN(T, E) gi_launch(add_layernorm_vec_kernel<T, E>, dim3(n_rows), dim3(vt), 0, vs, (const T*)delta, (const T*)delta2, \
                                  residual, weight, bias, w_dtype, (T*)out, rows, dim, eps, write_residual)
        if (act_dtype == GI_DTYPE_F32) { if (early) LAUNCH_LN(float, 1); else LAUNCH_LN(float, 0); }
        else if (act_dtype == GI_DTYPE_BF16) { if (early) LAUNCH_LN(bf16, 1); else LAUNCH_LN(bf16, 0); }
#undef LAUNCH_LN
        else
            GI_REQUIRE(false, "gi_add_layernorm: activation dtype %d", act_dtype);
        return gi_check_launch("gi_add_layernorm");
    }
    int threads = ((dim + 3) / 4 + 31) / 32 * 32;             // from the width alone: four elements a thread,
    threads = threads < 64 ? 64 : (threads > 512 ? 512 : threads);   // more from 2,048 on
    cudaStream_t s = (cudaStream_t)stream;
    if (act_dtype == GI_DTYPE_F32)
        gi_launch(add_layernorm_kernel<float>, dim3(n_rows), dim3(threads), 0, s, (const float*)delta, (const float*)delta2,
                  residual, weight, bias, w_dtype, (float*)out, rows, dim, eps, write_residual);
    else if (act_dtype == GI_DTYPE_BF16)
        gi_launch(add_layernorm_kernel<bf16>, dim3(n_rows), dim3(threads), 0, s, (const bf16*)delta, (const bf16*)delta2,
                  residual, weight, bias, w_dtype, (bf16*)out, rows, dim, eps, write_residual);
    else
        GI_REQUIRE(false, "gi_add_layernorm: activation dtype %d", act_dtype);
    return gi_check_launch("gi_add_layernorm");
}

// ------------------------------------------------------------------ RMS norm of rows inside a wider matrix
template <typename T>
__global__ void rmsnorm_rows_kernel(const T* __restrict__ x, long long ld, const void* __restrict__ weight, int w_dtype,
                                    T* __restrict__ out, int dim, float eps) {
    gi_pdl_start();
    __shared__ float red[33];
    const T* row = x + (size_t)blockIdx.x * ld;
    float ss = 0.f;
    for (int c = threadIdx.x; c < dim; c += blockDim.x) { const float v = to_f32(row[c]); ss += v * v; }
    const float inv = 1.f / sqrtf(block_sum(ss, red) / (float)dim + eps);
    T* o = out + (size_t)blockIdx.x * dim;
    for (int c = threadIdx.x; c < dim; c += blockDim.x)
        o[c] = from_f32<T>(to_f32(row[c]) * inv * load_w(weight, w_dtype, c));
}

// Four elements per thread and load, the row in registers (widths that are multiples of 4 up to 8,192, rows that
// start on 16 bytes for float32 and on 8 for bfloat16).
template <typename T>
__global__ void __launch_bounds__(256)
rmsnorm_rows_vec_kernel(const T* __restrict__ x, long long ld, const void* __restrict__ weight, int w_dtype,
                        T* __restrict__ out, int dim, float eps) {
    gi_pdl_start();
    __shared__ float red[33];
    const T* row = x + (size_t)blockIdx.x * ld;
    float4 v[LN_VEC_MAX_IT];
    float ss = 0.f;
#pragma unroll
    for (int it = 0; it < LN_VEC_MAX_IT; ++it) {
        const int c = (it * blockDim.x + threadIdx.x) * 4;
        if (c < dim) {
            v[it] = load4_act(row + c);
            ss += v[it].x * v[it].x;
            ss += v[it].y * v[it].y;
            ss += v[it].z * v[it].z;
            ss += v[it].w * v[it].w;
        }
    }
    const float inv = 1.f / sqrtf(block_sum(ss, red) / (float)dim + eps);
    T* o = out + (size_t)blockIdx.x * dim;
#pragma unroll
    for (int it = 0; it < LN_VEC_MAX_IT; ++it) {
        const int c = (it * blockDim.x + threadIdx.x) * 4;
        if (c < dim) {
            const float4 w = load4_w(weight, w_dtype, c);
            store4_act(o + c, make_float4(v[it].x * inv * w.x, v[it].y * inv * w.y, v[it].z * inv * w.z, v[it].w * inv * w.w));
        }
    }
}

extern "C" int gi_rmsnorm_rows(const void* x, long long ld, const void* weight, int w_dtype, void* out, int act_dtype,
                               int n_rows, int dim, float eps, void* stream) {
    GI_REQUIRE(n_rows >= 0 && dim > 0 && ld >= dim, "gi_rmsnorm_rows: sizes");
    GI_REQUIRE(w_dtype == GI_DTYPE_F32 || w_dtype == GI_DTYPE_BF16, "gi_rmsnorm_rows: weight dtype %d", w_dtype);
    GI_REQUIRE(act_dtype == GI_DTYPE_F32 || act_dtype == GI_DTYPE_BF16, "gi_rmsnorm_rows: activation dtype %d", act_dtype);
    if (n_rows == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int esz = act_dtype == GI_DTYPE_F32 ? 4 : 2;
    if (dim % 4 == 0 && dim <= 256 * 4 * LN_VEC_MAX_IT && (uintptr_t)x % 16 == 0 && (ld * esz) % 16 == 0 &&
        (uintptr_t)out % 16 == 0 && (uintptr_t)weight % 16 == 0) {
        int vt = ((dim / 4 + 31) / 32) * 32;
        vt = vt > 256 ? 256 : vt;
        if (act_dtype == GI_DTYPE_F32)
            gi_launch(rmsnorm_rows_vec_kernel<float>, dim3(n_rows), dim3(vt), 0, s, (const float*)x, ld, weight, w_dtype, (float*)out, dim, eps);
        else
            gi_launch(rmsnorm_rows_vec_kernel<bf16>, dim3(n_rows), dim3(vt), 0, s, (const bf16*)x, ld, weight, w_dtype, (bf16*)out, dim, eps);
        return gi_check_launch("gi_rmsnorm_rows");
    }
    const int threads = dim >= 2048 ? 512 : (dim >= 512 ? 256 : (dim >= 128 ? 128 : 32));
    if (act_dtype == GI_DTYPE_F32)
        gi_launch(rmsnorm_rows_kernel<float>, dim3(n_rows), dim3(threads), 0, s, (const float*)x, ld, weight, w_dtype, (float*)out, dim, eps);
    else
        gi_launch(rmsnorm_rows_kernel<bf16>, dim3(n_rows), dim3(threads), 0, s, (const bf16*)x, ld, weight, w_dtype, (bf16*)out, dim, eps);
    return gi_check_launch("gi_rmsnorm_rows");
}

// ------------------------------------------------------------------ soft cap of logits
__global__ void softcap_kernel(float* __restrict__ z, long long n, float cap) {
    gi_pdl_start();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        z[i] = cap * tanhf(z[i] / cap);
}

extern "C" int gi_softcap(float* z, long long n, float cap, void* stream) {
    GI_REQUIRE(n >= 0 && cap > 0.f, "gi_softcap: a cap of %f", (double)cap);
    if (n == 0) return 0;
    const int blocks = (int)((n + 255) / 256 > 148 * 16 ? 148 * 16 : (n + 255) / 256);
    gi_launch(softcap_kernel, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, z, n, cap);
    return gi_check_launch("gi_softcap");
}
