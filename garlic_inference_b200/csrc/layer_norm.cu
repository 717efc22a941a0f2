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

extern "C" int gi_add_layernorm(const void* delta, const void* delta2, float* residual, const void* weight,
                                const void* bias, int w_dtype, void* out, int act_dtype, const int* rows, int n_rows,
                                int dim, float eps, int write_residual, void* stream) {
    GI_REQUIRE(n_rows >= 0 && dim > 0, "gi_add_layernorm: sizes must be positive");
    GI_REQUIRE(dim <= 512 * LN_MAX_PER_THREAD, "gi_add_layernorm: rows of %d are wider than %d", dim, 512 * LN_MAX_PER_THREAD);
    GI_REQUIRE(w_dtype == GI_DTYPE_F32 || w_dtype == GI_DTYPE_BF16, "gi_add_layernorm: weight dtype %d", w_dtype);
    GI_REQUIRE(!(rows && write_residual), "gi_add_layernorm: gathered rows cannot write the residual back");
    if (n_rows == 0) return 0;
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

extern "C" int gi_rmsnorm_rows(const void* x, long long ld, const void* weight, int w_dtype, void* out, int act_dtype,
                               int n_rows, int dim, float eps, void* stream) {
    GI_REQUIRE(n_rows >= 0 && dim > 0 && ld >= dim, "gi_rmsnorm_rows: sizes");
    GI_REQUIRE(w_dtype == GI_DTYPE_F32 || w_dtype == GI_DTYPE_BF16, "gi_rmsnorm_rows: weight dtype %d", w_dtype);
    if (n_rows == 0) return 0;
    const int threads = dim >= 2048 ? 512 : (dim >= 512 ? 256 : (dim >= 128 ? 128 : 32));
    cudaStream_t s = (cudaStream_t)stream;
    if (act_dtype == GI_DTYPE_F32)
        gi_launch(rmsnorm_rows_kernel<float>, dim3(n_rows), dim3(threads), 0, s, (const float*)x, ld, weight, w_dtype, (float*)out, dim, eps);
    else if (act_dtype == GI_DTYPE_BF16)
        gi_launch(rmsnorm_rows_kernel<bf16>, dim3(n_rows), dim3(threads), 0, s, (const bf16*)x, ld, weight, w_dtype, (bf16*)out, dim, eps);
    else
        GI_REQUIRE(false, "gi_rmsnorm_rows: activation dtype %d", act_dtype);
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
