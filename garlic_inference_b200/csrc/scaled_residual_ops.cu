// Row-wise kernels of layers whose sublayer results join the residual stream through a learned factor per
// channel (layer scale), whose norm is a Dynamic Tanh, and whose feed-forward gates with the tanh form of gelu.
//
//   gi_add_dyt              s = x (+ delta * scale);  out = tanh(alpha s) * w + b       x the float32 residual stream;
//                           no mean or variance is taken, alpha is one learned number; with write_residual the sum
//                           goes back into x; `rows` picks input rows (nothing is written back then)
//   gi_residual_add_scaled  x += delta * scale                                           (scale optional)
//   gi_glu                  out = act(g) * (u + up_shift) for rows [gate | up] (out may be columns of a wider matrix), g = min(gate, gate_max),
//                           u = clamp(up, -up_limit, up_limit) (infinite limits and a shift of 0: the plain unit);
//                           act 0: silu, 1: gelu in its tanh form, 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))),
//                           2: z sigmoid(alpha z)
//   gi_relu_squared         out = max(z, 0)^2
//   gi_scaled_sum           out = a * ca + b * cb                                        (two mixers side by side)
//
// Everything is float32 inside and rounded once on the way out; T is the activation type.  A row's result does
// not depend on what else is in the launch.  NikolayBlagoev/garlic-inference has none of these (its layer is
// pre-norm RMSNorm with a plain residual add, src/src-cuda/norm.cu:51-101).
#include "common.cuh"
#include "glu.cuh"
#include <math.h>

// ------------------------------------------------------------------ scaled add + Dynamic Tanh
template <typename T>
__global__ void add_dyt_kernel(const T* __restrict__ delta, const void* __restrict__ dscale, int s_dtype,
                               float* __restrict__ residual, const void* __restrict__ weight,
                               const void* __restrict__ bias, const void* __restrict__ alpha, int w_dtype,
                               T* __restrict__ out, const int* __restrict__ rows, int dim, int write_residual) {
    gi_pdl_start();
    const int r = blockIdx.x;
    const size_t i = rows ? (size_t)rows[r] : (size_t)r;
    float* res = residual + i * dim;
    const T* del = delta ? delta + i * dim : nullptr;
    const float a = load_w(alpha, w_dtype, 0);
    T* o = out + (size_t)r * dim;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < dim; c += gridDim.y * blockDim.x) {
        float s = res[c];
        if (del) {
            const float dv = to_f32(del[c]);
            s = dscale ? fmaf(dv, load_w(dscale, s_dtype, c), s) : s + dv;
            if (write_residual) res[c] = s;
        }
        o[c] = from_f32<T>(fmaf(tanhf(a * s), load_w(weight, w_dtype, c), load_w(bias, w_dtype, c)));
    }
}

extern "C" int gi_add_dyt(const void* delta, const void* dscale, int s_dtype, float* residual, const void* weight,
                          const void* bias, const void* alpha, int w_dtype, void* out, int act_dtype, const int* rows,
                          int n_rows, int dim, int write_residual, void* stream) {
    GI_REQUIRE(n_rows >= 0 && dim > 0, "gi_add_dyt: sizes must be positive");
    GI_REQUIRE(!(rows && write_residual), "gi_add_dyt: gathered rows are never written back");
    if (n_rows == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    // a row is cut over a few blocks when there are few rows: no sum ties a row's elements together
    const int per_row = n_rows >= 256 ? 1 : (dim + 1023) / 1024;
    dim3 grid(n_rows, per_row > 0 ? per_row : 1);
    if (act_dtype == GI_DTYPE_F32)
        gi_launch(add_dyt_kernel<float>, grid, dim3(256), 0, s, (const float*)delta, dscale, s_dtype, residual, weight, bias,
                  alpha, w_dtype, (float*)out, rows, dim, write_residual);
    else if (act_dtype == GI_DTYPE_BF16)
        gi_launch(add_dyt_kernel<bf16>, grid, dim3(256), 0, s, (const bf16*)delta, dscale, s_dtype, residual, weight, bias,
                  alpha, w_dtype, (bf16*)out, rows, dim, write_residual);
    else
        GI_REQUIRE(false, "gi_add_dyt: activation dtype %d", act_dtype);
    return gi_check_launch("gi_add_dyt");
}

template <typename T>
__global__ void residual_add_scaled_kernel(const T* __restrict__ delta, const void* __restrict__ dscale, int s_dtype,
                                           float* __restrict__ residual, long long n, int dim) {
    gi_pdl_start();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const float dv = to_f32(delta[i]);
        residual[i] = dscale ? fmaf(dv, load_w(dscale, s_dtype, (int)(i % dim)), residual[i]) : residual[i] + dv;
    }
}

extern "C" int gi_residual_add_scaled(const void* delta, int act_dtype, const void* dscale, int s_dtype, float* residual,
                                      int n_rows, int dim, void* stream) {
    GI_REQUIRE(n_rows >= 0 && dim > 0, "gi_residual_add_scaled: sizes must be positive");
    if (n_rows == 0) return 0;
    const long long n = (long long)n_rows * dim;
    const int blocks = (int)((n + 255) / 256 > 148 * 16 ? 148 * 16 : (n + 255) / 256);
    cudaStream_t s = (cudaStream_t)stream;
    if (act_dtype == GI_DTYPE_F32)
        gi_launch(residual_add_scaled_kernel<float>, dim3(blocks), dim3(256), 0, s, (const float*)delta, dscale, s_dtype, residual, n, dim);
    else if (act_dtype == GI_DTYPE_BF16)
        gi_launch(residual_add_scaled_kernel<bf16>, dim3(blocks), dim3(256), 0, s, (const bf16*)delta, dscale, s_dtype, residual, n, dim);
    else
        GI_REQUIRE(false, "gi_residual_add_scaled: activation dtype %d", act_dtype);
    return gi_check_launch("gi_residual_add_scaled");
}

// ------------------------------------------------------------------ gated linear unit, squared relu
template <typename T>
__global__ void glu_kernel(const T* __restrict__ gate_up, long long ld, T* __restrict__ out, long long ld_out, int n_rows,
                           int inter, GluShape p) {
    gi_pdl_start();
    const long long total = (long long)n_rows * inter;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / inter;
        const int c = (int)(i - r * inter);
        const T* row = gate_up + r * ld;
        out[r * ld_out + c] = from_f32<T>(glu_unit(to_f32(row[c]), to_f32(row[inter + c]), p));
    }
}

// Eight columns at a time with 16-byte loads and stores (bfloat16 rows whose halves start on 16 bytes).
__global__ void glu_vec_kernel(const bf16* __restrict__ gate_up, long long ld, bf16* __restrict__ out, long long ld_out,
                               int n_rows, int inter, GluShape p) {
    gi_pdl_start();
    const int per_row = inter / 8;
    const long long total = (long long)n_rows * per_row;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / per_row;
        const int c = (int)(i - r * per_row) * 8;
        const uint4 g = *reinterpret_cast<const uint4*>(gate_up + r * ld + c);
        const uint4 u = *reinterpret_cast<const uint4*>(gate_up + r * ld + inter + c);
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g);
        const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u);
        uint4 o;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 gf = __bfloat1622float2(g2[k]), uf = __bfloat1622float2(u2[k]);
            o2[k] = __floats2bfloat162_rn(glu_unit(gf.x, uf.x, p), glu_unit(gf.y, uf.y, p));
        }
        *reinterpret_cast<uint4*>(out + r * ld_out + c) = o;
    }
}

extern "C" int gi_glu(const void* gate_up, long long ld, void* out, long long ld_out, int act_dtype, int n_rows, int inter, int kind,
                      float alpha, float gate_max, float up_limit, float up_shift, void* stream) {
    GI_REQUIRE(n_rows >= 0 && inter > 0 && ld >= 2LL * inter && ld_out >= inter && kind >= 0 && kind <= 2, "gi_glu: sizes or activation");
    GI_REQUIRE(up_limit >= 0.f, "gi_glu: the up half is clamped to +-%f", (double)up_limit);
    if (n_rows == 0) return 0;
    const GluShape p = {kind, alpha, gate_max, up_limit, up_shift};
    const long long total = (long long)n_rows * inter;
    const int blocks = (int)((total + 255) / 256 > 148 * 16 ? 148 * 16 : (total + 255) / 256);
    cudaStream_t s = (cudaStream_t)stream;
    if (act_dtype == GI_DTYPE_F32)
        gi_launch(glu_kernel<float>, dim3(blocks), dim3(256), 0, s, (const float*)gate_up, ld, (float*)out, ld_out, n_rows, inter, p);
    else if (act_dtype == GI_DTYPE_BF16 && inter % 8 == 0 && ld % 8 == 0 && ld_out % 8 == 0 && (uintptr_t)gate_up % 16 == 0 &&
             (uintptr_t)out % 16 == 0) {
        const long long units = total / 8;
        const int vb = (int)((units + 255) / 256 > 148 * 16 ? 148 * 16 : (units + 255) / 256);
        gi_launch(glu_vec_kernel, dim3(vb), dim3(256), 0, s, (const bf16*)gate_up, ld, (bf16*)out, ld_out, n_rows, inter, p);
    } else if (act_dtype == GI_DTYPE_BF16)
        gi_launch(glu_kernel<bf16>, dim3(blocks), dim3(256), 0, s, (const bf16*)gate_up, ld, (bf16*)out, ld_out, n_rows, inter, p);
    else
        GI_REQUIRE(false, "gi_glu: activation dtype %d", act_dtype);
    return gi_check_launch("gi_glu");
}

template <typename T>
__global__ void relu_squared_kernel(const T* __restrict__ z, T* __restrict__ out, long long n) {
    gi_pdl_start();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const float v = fmaxf(to_f32(z[i]), 0.f);
        out[i] = from_f32<T>(v * v);
    }
}

extern "C" int gi_relu_squared(const void* z, void* out, int act_dtype, long long n, void* stream) {
    GI_REQUIRE(n >= 0, "gi_relu_squared: size");
    if (n == 0) return 0;
    const int blocks = (int)((n + 255) / 256 > 148 * 16 ? 148 * 16 : (n + 255) / 256);
    cudaStream_t s = (cudaStream_t)stream;
    if (act_dtype == GI_DTYPE_F32)
        gi_launch(relu_squared_kernel<float>, dim3(blocks), dim3(256), 0, s, (const float*)z, (float*)out, n);
    else if (act_dtype == GI_DTYPE_BF16)
        gi_launch(relu_squared_kernel<bf16>, dim3(blocks), dim3(256), 0, s, (const bf16*)z, (bf16*)out, n);
    else
        GI_REQUIRE(false, "gi_relu_squared: activation dtype %d", act_dtype);
    return gi_check_launch("gi_relu_squared");
}

// ------------------------------------------------------------------ two results side by side
template <typename T>
__global__ void scaled_sum_kernel(const T* __restrict__ a, float ca, const T* __restrict__ b, float cb,
                                  T* __restrict__ out, long long n) {
    gi_pdl_start();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        out[i] = from_f32<T>(fmaf(to_f32(a[i]), ca, to_f32(b[i]) * cb));
}

extern "C" int gi_scaled_sum(const void* a, float ca, const void* b, float cb, void* out, int act_dtype, long long n,
                             void* stream) {
    GI_REQUIRE(n >= 0, "gi_scaled_sum: size");
    if (n == 0) return 0;
    const int blocks = (int)((n + 255) / 256 > 148 * 16 ? 148 * 16 : (n + 255) / 256);
    cudaStream_t s = (cudaStream_t)stream;
    if (act_dtype == GI_DTYPE_F32)
        gi_launch(scaled_sum_kernel<float>, dim3(blocks), dim3(256), 0, s, (const float*)a, ca, (const float*)b, cb, (float*)out, n);
    else if (act_dtype == GI_DTYPE_BF16)
        gi_launch(scaled_sum_kernel<bf16>, dim3(blocks), dim3(256), 0, s, (const bf16*)a, ca, (const bf16*)b, cb, (bf16*)out, n);
    else
        GI_REQUIRE(false, "gi_scaled_sum: activation dtype %d", act_dtype);
    return gi_check_launch("gi_scaled_sum");
}
