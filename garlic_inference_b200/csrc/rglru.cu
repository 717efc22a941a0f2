// The real-gated linear recurrent unit: a recurrence with one number of state per channel, whose decay and input
// gate are made from the recurrence's own input by block-diagonal matrices.
//
//   gi_rglru_gates   per token, for channels in `blocks` equal blocks:  r = sigmoid(Wa[b] u_b + ba),
//                    i = sigmoid(Wi[b] u_b + bi);  log a = -c r softplus(lam);  a = exp(log a);
//                    b = sqrt(1 - a^2) i u.   Writes a and b as float32 [n, width].  u is float32 (the output of the
//                    short convolution).  1 - a^2 is taken as -expm1(2 log a), which keeps its digits when a is
//                    close to 1.
//   gi_rglru_scan    S_t = a_t S_(t-1) + b_t per channel along each sequence's rows of the step, from the slot's
//                    state row (float32, zero for a new sequence) and back into it; out = S_t * act(y_t + by)
//                    with act the tanh form of gelu, rounded once into the activation type.
//
// The gate matrices arrive transposed, [blocks, in, out], so that the threads of a block (one per output
// channel) read consecutive addresses; a block of threads handles a tile of tokens of one block of channels
// with the tokens' inputs in shared memory.  Every sum runs over the inputs in index order whatever the tile,
// and the scan walks a sequence's tokens in order, so a position's bits do not depend on how the tokens were cut
// into steps or on the batch.  NikolayBlagoev/garlic-inference has no recurrent mixer.
#include "common.cuh"
#include <math.h>

#define RG_TN 8              // tokens per tile of the gate kernel

__device__ __forceinline__ float rg_sigmoid(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float rg_softplus(float z) { return z > 20.f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float rg_gelu_tanh(float z) {
    return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename TW>
__global__ void __launch_bounds__(256)
rglru_gates_kernel(const float* __restrict__ u, const TW* __restrict__ wa_t, const TW* __restrict__ wi_t,
                   const void* __restrict__ ba, const void* __restrict__ bi, const void* __restrict__ lam, int vec_dtype,
                   float decay_scale, float* __restrict__ a_out, float* __restrict__ b_out, int n_rows, int width,
                   int bw) {
    gi_pdl_start();
    extern __shared__ __align__(16) float us[];                  // [RG_TN][bw]
    const int row0 = blockIdx.x * RG_TN, blk = blockIdx.y;
    const int rows = min(RG_TN, n_rows - row0);
    for (int i = threadIdx.x; i < RG_TN * bw; i += blockDim.x) {
        const int t = i / bw, k = i - t * bw;
        us[i] = t < rows ? u[(size_t)(row0 + t) * width + blk * bw + k] : 0.f;
    }
    __syncthreads();
    const TW* wa = wa_t + (size_t)blk * bw * bw;
    const TW* wi = wi_t + (size_t)blk * bw * bw;
    for (int o = blockIdx.z * blockDim.x + threadIdx.x; o < bw; o += gridDim.z * blockDim.x) {
        float ra[RG_TN], ri[RG_TN];
#pragma unroll
        for (int t = 0; t < RG_TN; ++t) ra[t] = ri[t] = 0.f;
        int k = 0;
        if (bw % 4 == 0) {
            for (; k < bw; k += 4) {
                float a4[4], i4[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    a4[j] = to_f32(wa[(size_t)(k + j) * bw + o]);
                    i4[j] = to_f32(wi[(size_t)(k + j) * bw + o]);
                }
#pragma unroll
                for (int t = 0; t < RG_TN; ++t) {
                    const float4 x = *reinterpret_cast<const float4*>(us + t * bw + k);
                    ra[t] = fmaf(a4[0], x.x, ra[t]); ra[t] = fmaf(a4[1], x.y, ra[t]);
                    ra[t] = fmaf(a4[2], x.z, ra[t]); ra[t] = fmaf(a4[3], x.w, ra[t]);
                    ri[t] = fmaf(i4[0], x.x, ri[t]); ri[t] = fmaf(i4[1], x.y, ri[t]);
                    ri[t] = fmaf(i4[2], x.z, ri[t]); ri[t] = fmaf(i4[3], x.w, ri[t]);
                }
            }
        } else {
            for (; k < bw; ++k) {
                const float a1 = to_f32(wa[(size_t)k * bw + o]), i1 = to_f32(wi[(size_t)k * bw + o]);
#pragma unroll
                for (int t = 0; t < RG_TN; ++t) {
                    ra[t] = fmaf(a1, us[t * bw + k], ra[t]);
                    ri[t] = fmaf(i1, us[t * bw + k], ri[t]);
                }
            }
        }
        const int c = blk * bw + o;
        const float bra = load_w(ba, vec_dtype, c), bri = load_w(bi, vec_dtype, c);
        const float sp = rg_softplus(load_w(lam, vec_dtype, c));
#pragma unroll
        for (int t = 0; t < RG_TN; ++t) {
            if (t >= rows) break;
            const float r = rg_sigmoid(ra[t] + bra), g = rg_sigmoid(ri[t] + bri);
            const float log_a = -decay_scale * r * sp;
            const float a = expf(log_a);
            const float keep = sqrtf(fmaxf(-expm1f(2.f * log_a), 0.f));
            a_out[(size_t)(row0 + t) * width + c] = a;
            b_out[(size_t)(row0 + t) * width + c] = keep * g * us[t * bw + o];
        }
    }
}

extern "C" int gi_rglru_gates(const float* u, const void* wa_t, const void* wi_t, int w_dtype, const void* ba,
                              const void* bi, const void* lam, int vec_dtype, float decay_scale, float* a_out,
                              float* b_out, int n_rows, int width, int blocks, void* stream) {
    GI_REQUIRE(n_rows >= 0 && width > 0 && blocks > 0 && width % blocks == 0, "gi_rglru_gates: %d channels in %d blocks", width, blocks);
    GI_REQUIRE(blocks <= 65535, "gi_rglru_gates: %d blocks is beyond 65535", blocks);
    if (n_rows == 0) return 0;
    const int bw = width / blocks;
    const size_t smem = (size_t)RG_TN * bw * sizeof(float);
    const int threads = bw >= 256 ? 256 : (bw + 31) / 32 * 32;
    // few tiles: the output channels of a block of channels are cut over several blocks of threads
    const int tiles = (n_rows + RG_TN - 1) / RG_TN;
    int cut = 1;
    while (cut * threads < bw && (long long)tiles * blocks * cut < 296) ++cut;
    dim3 grid(tiles, blocks, cut);
    cudaStream_t s = (cudaStream_t)stream;
    if (w_dtype == GI_DTYPE_F32) {
        if (int rc = gi_reserve_smem((const void*)rglru_gates_kernel<float>, smem, "gi_rglru_gates")) return rc;
        gi_launch(rglru_gates_kernel<float>, grid, dim3(threads), smem, s, u, (const float*)wa_t, (const float*)wi_t, ba, bi,
                  lam, vec_dtype, decay_scale, a_out, b_out, n_rows, width, bw);
    } else if (w_dtype == GI_DTYPE_BF16) {
        if (int rc = gi_reserve_smem((const void*)rglru_gates_kernel<bf16>, smem, "gi_rglru_gates")) return rc;
        gi_launch(rglru_gates_kernel<bf16>, grid, dim3(threads), smem, s, u, (const bf16*)wa_t, (const bf16*)wi_t, ba, bi,
                  lam, vec_dtype, decay_scale, a_out, b_out, n_rows, width, bw);
    } else {
        GI_REQUIRE(false, "gi_rglru_gates: weight dtype %d", w_dtype);
    }
    return gi_check_launch("gi_rglru_gates");
}

// spans [n_seq, 3] = {slot, first row, rows}, or null: every row is a sequence of its own with the slot of tok_slot.
#define RG_AHEAD 8           // tokens whose inputs a thread asks for before it walks them
template <typename T>
__global__ void __launch_bounds__(128)
rglru_scan_kernel(const float* __restrict__ a, const float* __restrict__ b, const T* __restrict__ y, long long ldy,
                  const void* __restrict__ y_bias, int bias_dtype, float* __restrict__ state, long long state_stride,
                  const int* __restrict__ spans, const int* __restrict__ tok_slot, T* __restrict__ out, long long ldo,
                  int width) {
    gi_pdl_start();
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= width) return;
    int slot, start, len;
    if (spans) { slot = spans[3 * blockIdx.x]; start = spans[3 * blockIdx.x + 1]; len = spans[3 * blockIdx.x + 2]; }
    else { slot = tok_slot[blockIdx.x]; start = blockIdx.x; len = 1; }
    if (slot < 0) {
        for (int t = 0; t < len; ++t) out[(size_t)(start + t) * ldo + c] = from_f32<T>(0.f);
        return;
    }
    const float yb = y_bias ? load_w(y_bias, bias_dtype, c) : 0.f;
    float S = state[(size_t)slot * state_stride + c];
    for (int t0 = 0; t0 < len; t0 += RG_AHEAD) {
        float av[RG_AHEAD], bv[RG_AHEAD], yv[RG_AHEAD];
#pragma unroll
        for (int j = 0; j < RG_AHEAD; ++j) {
            const bool in = t0 + j < len;
            const size_t r = (size_t)(start + (in ? t0 + j : 0));
            av[j] = in ? a[r * width + c] : 1.f;
            bv[j] = in ? b[r * width + c] : 0.f;
            yv[j] = in ? to_f32(y[r * ldy + c]) : 0.f;
        }
#pragma unroll
        for (int j = 0; j < RG_AHEAD; ++j) {
            if (t0 + j >= len) break;
            S = fmaf(av[j], S, bv[j]);
            out[(size_t)(start + t0 + j) * ldo + c] = from_f32<T>(S * rg_gelu_tanh(yv[j] + yb));
        }
    }
    state[(size_t)slot * state_stride + c] = S;
}

extern "C" int gi_rglru_scan(const float* a, const float* b, const void* y, long long ldy, int act_dtype, const void* y_bias,
                             int bias_dtype, float* state, long long state_stride, const int* spans, const int* tok_slot,
                             void* out, long long ldo, int n_seqs, int width, void* stream) {
    GI_REQUIRE(n_seqs >= 0 && width > 0 && ldy >= width && ldo >= width && state_stride >= width, "gi_rglru_scan: sizes");
    GI_REQUIRE((width + 127) / 128 <= 65535, "gi_rglru_scan: %d channels", width);
    if (n_seqs == 0) return 0;
    dim3 grid(n_seqs, (width + 127) / 128);
    cudaStream_t s = (cudaStream_t)stream;
    if (act_dtype == GI_DTYPE_F32)
        gi_launch(rglru_scan_kernel<float>, grid, dim3(128), 0, s, a, b, (const float*)y, ldy, y_bias, bias_dtype, state,
                  state_stride, spans, tok_slot, (float*)out, ldo, width);
    else if (act_dtype == GI_DTYPE_BF16)
        gi_launch(rglru_scan_kernel<bf16>, grid, dim3(128), 0, s, a, b, (const bf16*)y, ldy, y_bias, bias_dtype, state,
                  state_stride, spans, tok_slot, (bf16*)out, ldo, width);
    else
        GI_REQUIRE(false, "gi_rglru_scan: activation dtype %d", act_dtype);
    return gi_check_launch("gi_rglru_scan");
}
