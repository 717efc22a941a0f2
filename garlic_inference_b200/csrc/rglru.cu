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
// The gate matrices arrive transposed, [blocks, in, out]; a block of threads keeps a slice of output channels of
// both matrices in shared memory and streams tiles of tokens past them.  Every sum runs in an order that depends on
// the block width alone, and the scan walks a sequence's tokens in order, so a position's bits do not depend on
// how the tokens were cut into steps or on the batch.  NikolayBlagoev/garlic-inference has no recurrent mixer.
#include "common.cuh"
#include <math.h>

#define RG_KS 8              // lanes that share an output: lane s sums the inputs k = s, s + 8, s + 16, ...
#define RG_TG 8              // tokens per thread
#define RG_OG 4              // outputs per thread
#define RG_WPAD 8            // padding of a row of weights in shared memory: rows start on 16 bytes and spread over the banks

__device__ __forceinline__ float rg_sigmoid(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float rg_softplus(float z) { return z > 20.f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float rg_gelu_tanh(float z) {
    return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

__device__ __forceinline__ void rg_cp_async_4(float* smem, const float* gmem) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem));
}
__device__ __forceinline__ void rg_cp_async_16(void* smem, const void* gmem, int bytes) {      // the rest of the 16 is zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void rg_cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
__device__ __forceinline__ void rg_cp_async_wait_1() { asm volatile("cp.async.wait_group 1;\n" ::); }
__device__ __forceinline__ void rg_cp_async_wait_0() { asm volatile("cp.async.wait_group 0;\n" ::); }

template <typename TW> __device__ __forceinline__ void rg_load4(const TW* p, float (&w)[4]);
template <> __device__ __forceinline__ void rg_load4<float>(const float* p, float (&w)[4]) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
}
template <> __device__ __forceinline__ void rg_load4<bf16>(const bf16* p, float (&w)[4]) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
    const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
    w[0] = lo.x; w[1] = lo.y; w[2] = hi.x; w[3] = hi.y;
}

// One block of threads owns `orange` output channels of one block of channels: it copies their two slices of
// the gate matrices into shared memory once ([gate][input][output], rows padded by 8 elements) and then walks its
// share of the step's rows in tiles of `tt` tokens, whose inputs lie in shared memory transposed ([input][token],
// rows padded by 4 floats; two tiles, the next one copied in while this one is summed).  A thread holds 8 tokens x 4 outputs x 2 gates; the 8 lanes that share those outputs
// each sum every eighth input in rising order and their sums meet in a fixed butterfly, so a token's bits depend
// neither on the tile nor on the step's other rows.  The same launch shape serves a prompt (weights read once per
// block of threads, all tokens streamed past them) and a decode step (the weights land in shared memory with
// coalesced loads instead of a chain of dependent ones).
template <typename TW>
__global__ void __launch_bounds__(256)
rglru_gates_kernel(const float* __restrict__ u, const TW* __restrict__ wa_t, const TW* __restrict__ wi_t,
                   const void* __restrict__ ba, const void* __restrict__ bi, const void* __restrict__ lam, int vec_dtype,
                   float decay_scale, float* __restrict__ a_out, float* __restrict__ b_out, int n_rows, int width,
                   int bw, int orange, int tt, int rows_per_cta) {
    gi_pdl_start();
    extern __shared__ __align__(16) unsigned char rg_smem[];
    const int ws = orange + RG_WPAD, us_ld = tt + 4;
    TW* w_s = reinterpret_cast<TW*>(rg_smem);                                     // [2][bw][ws]
    float* u_s = reinterpret_cast<float*>(rg_smem + (((size_t)2 * bw * ws * sizeof(TW) + 15) & ~(size_t)15));   // [2][bw][us_ld]
    const int blk = blockIdx.x, o0 = blockIdx.y * orange;
    const int row_begin = blockIdx.z * rows_per_cta, row_end = min(n_rows, row_begin + rows_per_cta);
    if (row_begin >= row_end) return;
    // the two slices of weights: 16 bytes at a time and asynchronously where rows and slices start on 16 bytes (the
    // part of a chunk beyond the block's last output is zero-filled), element by element otherwise
    constexpr int EPC = 16 / (int)sizeof(TW);               // elements per chunk
    const bool wide = (bw % EPC == 0) && ((uintptr_t)wa_t % 16 == 0) && ((uintptr_t)wi_t % 16 == 0);
    for (int g = 0; g < 2; ++g) {
        const TW* src = (g ? wi_t : wa_t) + (size_t)blk * bw * bw;
        TW* dst = w_s + (size_t)g * bw * ws;
        if (wide) {
            const int cpr = orange / EPC, shift = __ffs(cpr) - 1;          // chunks per row: a power of two
            for (int i = threadIdx.x; i < bw * cpr; i += blockDim.x) {
                const int k = i >> shift, c = i & (cpr - 1), o = o0 + c * EPC;
                const int valid = max(0, min(EPC, bw - o)) * (int)sizeof(TW);
                rg_cp_async_16(dst + (size_t)k * ws + c * EPC, src + (size_t)k * bw + (valid ? o : 0), valid);
            }
        } else {
            for (int k = 0; k < bw; ++k)
                for (int oo = threadIdx.x; oo < orange; oo += blockDim.x)
                    dst[(size_t)k * ws + oo] = o0 + oo < bw ? src[(size_t)k * bw + o0 + oo] : from_f32<TW>(0.f);
        }
    }
    const int n_og = orange / RG_OG;
    const int ks = threadIdx.x % RG_KS, og = (threadIdx.x / RG_KS) % n_og, tg = threadIdx.x / (RG_KS * n_og);
    const int oo = og * RG_OG;                               // first of this thread's outputs within the slice
    // what the epilogue needs of this thread's outputs: biases and softplus(lam)
    float bra[RG_OG], bri[RG_OG], sp[RG_OG];
#pragma unroll
    for (int j = 0; j < RG_OG; ++j) {
        const int o = o0 + oo + j, c = blk * bw + min(o, bw - 1);
        bra[j] = load_w(ba, vec_dtype, c);
        bri[j] = load_w(bi, vec_dtype, c);
        sp[j] = rg_softplus(load_w(lam, vec_dtype, c));
    }
    // A tile's inputs go from global memory straight into their transposed places, four bytes at a time and
    // asynchronously; the tile after the present one is on its way while this one is summed.
    auto issue_tile = [&](int tile0, float* dst) {
        for (int t = 0; t < tt; ++t) {
            const int row = tile0 + t;
            if (row < row_end) {
                const float* src = u + (size_t)row * width + blk * bw;
                for (int k = threadIdx.x; k < bw; k += blockDim.x) rg_cp_async_4(dst + k * us_ld + t, src + k);
            } else {
                for (int k = threadIdx.x; k < bw; k += blockDim.x) dst[k * us_ld + t] = 0.f;
            }
        }
    };
    issue_tile(row_begin, u_s);
    rg_cp_async_commit();
    int it = 0;
    for (int tile0 = row_begin; tile0 < row_end; tile0 += tt, ++it) {
        const float* cur = u_s + (size_t)(it & 1) * bw * us_ld;
        if (tile0 + tt < row_end) issue_tile(tile0 + tt, u_s + (size_t)((it + 1) & 1) * bw * us_ld);
        rg_cp_async_commit();                                // an empty group when nothing is left: the count stays uniform
        rg_cp_async_wait_1();
        __syncthreads();                                     // every thread's copies of this tile have landed (and the weights)
        float ra[RG_TG][RG_OG], ri[RG_TG][RG_OG];
#pragma unroll
        for (int t = 0; t < RG_TG; ++t)
#pragma unroll
            for (int j = 0; j < RG_OG; ++j) ra[t][j] = ri[t][j] = 0.f;
#pragma unroll 2
        for (int k = ks; k < bw; k += RG_KS) {
            float wa4[4], wi4[4];
            rg_load4<TW>(w_s + (size_t)k * ws + oo, wa4);
            rg_load4<TW>(w_s + ((size_t)bw + k) * ws + oo, wi4);
            const float4 x0 = *reinterpret_cast<const float4*>(cur + k * us_ld + tg * RG_TG);
            const float4 x1 = *reinterpret_cast<const float4*>(cur + k * us_ld + tg * RG_TG + 4);
            const float x[RG_TG] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
            for (int t = 0; t < RG_TG; ++t)
#pragma unroll
                for (int j = 0; j < RG_OG; ++j) {
                    ra[t][j] = fmaf(wa4[j], x[t], ra[t][j]);
                    ri[t][j] = fmaf(wi4[j], x[t], ri[t][j]);
                }
        }
        // The 8 lanes' sums meet in a butterfly that also shares the tokens out: after the exchange with lane s ^ 4
        // a lane keeps the half of its tokens that its bit 2 names, then the quarter its bit 1 names, then one:
        // lane s ends with token s, summed as ((s0 + s4) + (s2 + s6)) + ((s1 + s5) + (s3 + s7)) for every token
        // (the pairs are the same whichever lane keeps the sum), with 56 exchanges instead of 192.
        const bool b2 = ks & 4, b1 = ks & 2, b0 = ks & 1;
        float a4[4][RG_OG], i4[4][RG_OG], a2[2][RG_OG], i2[2][RG_OG], a1[RG_OG], i1[RG_OG];
#pragma unroll
        for (int t = 0; t < 4; ++t)
#pragma unroll
            for (int j = 0; j < RG_OG; ++j) {
                a4[t][j] = (b2 ? ra[t + 4][j] : ra[t][j]) + __shfl_xor_sync(0xffffffffu, b2 ? ra[t][j] : ra[t + 4][j], 4);
                i4[t][j] = (b2 ? ri[t + 4][j] : ri[t][j]) + __shfl_xor_sync(0xffffffffu, b2 ? ri[t][j] : ri[t + 4][j], 4);
            }
#pragma unroll
        for (int t = 0; t < 2; ++t)
#pragma unroll
            for (int j = 0; j < RG_OG; ++j) {
                a2[t][j] = (b1 ? a4[t + 2][j] : a4[t][j]) + __shfl_xor_sync(0xffffffffu, b1 ? a4[t][j] : a4[t + 2][j], 2);
                i2[t][j] = (b1 ? i4[t + 2][j] : i4[t][j]) + __shfl_xor_sync(0xffffffffu, b1 ? i4[t][j] : i4[t + 2][j], 2);
            }
#pragma unroll
        for (int j = 0; j < RG_OG; ++j) {
            a1[j] = (b0 ? a2[1][j] : a2[0][j]) + __shfl_xor_sync(0xffffffffu, b0 ? a2[0][j] : a2[1][j], 1);
            i1[j] = (b0 ? i2[1][j] : i2[0][j]) + __shfl_xor_sync(0xffffffffu, b0 ? i2[0][j] : i2[1][j], 1);
        }
        const int row = tile0 + tg * RG_TG + ks;             // lane s finishes token s of the thread's eight
        if (row < row_end) {
#pragma unroll
            for (int j = 0; j < RG_OG; ++j) {
                const int o = o0 + oo + j;
                if (o >= bw) continue;
                const float r = rg_sigmoid(a1[j] + bra[j]), g = rg_sigmoid(i1[j] + bri[j]);
                const float log_a = -decay_scale * r * sp[j];
                const float keep = sqrtf(fmaxf(-expm1f(2.f * log_a), 0.f));
                const size_t at = (size_t)row * width + blk * bw + o;
                a_out[at] = expf(log_a);
                b_out[at] = keep * g * cur[o * us_ld + tg * RG_TG + ks];
            }
        }
        __syncthreads();                                     // this buffer is refilled by the next round's copies
    }
    rg_cp_async_wait_0();
}

// Blocks of channels too wide for the kernel above (their slices of weights and a tile of inputs pass shared
// memory): a tile of 8 tokens' inputs in shared memory, a thread per output channel, the weights read from global
// memory in input order.  Which of the two kernels runs follows from the block width alone, so a model's bits do not
// depend on the step.
#define RG_WIDE_TN 8
template <typename TW>
__global__ void __launch_bounds__(256)
rglru_gates_wide_kernel(const float* __restrict__ u, const TW* __restrict__ wa_t, const TW* __restrict__ wi_t,
                   const void* __restrict__ ba, const void* __restrict__ bi, const void* __restrict__ lam, int vec_dtype,
                   float decay_scale, float* __restrict__ a_out, float* __restrict__ b_out, int n_rows, int width,
                   int bw) {
    gi_pdl_start();
    extern __shared__ __align__(16) float us[];                  // [RG_WIDE_TN][bw]
    const int row0 = blockIdx.x * RG_WIDE_TN, blk = blockIdx.y;
    const int rows = min(RG_WIDE_TN, n_rows - row0);
    for (int i = threadIdx.x; i < RG_WIDE_TN * bw; i += blockDim.x) {
        const int t = i / bw, k = i - t * bw;
        us[i] = t < rows ? u[(size_t)(row0 + t) * width + blk * bw + k] : 0.f;
    }
    __syncthreads();
    const TW* wa = wa_t + (size_t)blk * bw * bw;
    const TW* wi = wi_t + (size_t)blk * bw * bw;
    for (int o = blockIdx.z * blockDim.x + threadIdx.x; o < bw; o += gridDim.z * blockDim.x) {
        float ra[RG_WIDE_TN], ri[RG_WIDE_TN];
#pragma unroll
        for (int t = 0; t < RG_WIDE_TN; ++t) ra[t] = ri[t] = 0.f;
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
                for (int t = 0; t < RG_WIDE_TN; ++t) {
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
                for (int t = 0; t < RG_WIDE_TN; ++t) {
                    ra[t] = fmaf(a1, us[t * bw + k], ra[t]);
                    ri[t] = fmaf(i1, us[t * bw + k], ri[t]);
                }
            }
        }
        const int c = blk * bw + o;
        const float bra = load_w(ba, vec_dtype, c), bri = load_w(bi, vec_dtype, c);
        const float sp = rg_softplus(load_w(lam, vec_dtype, c));
#pragma unroll
        for (int t = 0; t < RG_WIDE_TN; ++t) {
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
    GI_REQUIRE(w_dtype == GI_DTYPE_F32 || w_dtype == GI_DTYPE_BF16, "gi_rglru_gates: weight dtype %d", w_dtype);
    if (n_rows == 0) return 0;
    const int bw = width / blocks;
    const size_t wsize = w_dtype == GI_DTYPE_F32 ? 4 : 2;
    // outputs per block of threads and tokens per tile: as many as shared memory takes (the sizes depend on the
    // block width alone, never on the step)
    int orange = 32, tt = 32;
    auto smem_of = [&](int orng, int t) {
        return (((size_t)2 * bw * (orng + RG_WPAD) * wsize + 15) & ~(size_t)15) + (size_t)2 * bw * (t + 4) * sizeof(float);
    };
    while (smem_of(orange, tt) > 200 * 1024 && tt > 16) tt /= 2;
    while (smem_of(orange, tt) > 200 * 1024 && orange > 16) orange /= 2;      // beyond that: the kernel for wide blocks
    cudaStream_t s = (cudaStream_t)stream;
    if (smem_of(orange, tt) > 200 * 1024) {
        const size_t smem = (size_t)RG_WIDE_TN * bw * sizeof(float);
        GI_REQUIRE(smem <= 200 * 1024, "gi_rglru_gates: blocks of %d channels do not fit shared memory", bw);
        const int threads = bw >= 256 ? 256 : (bw + 31) / 32 * 32;
        const int tiles = (n_rows + RG_WIDE_TN - 1) / RG_WIDE_TN;
        int cut = 1;
        while (cut * threads < bw && (long long)tiles * blocks * cut < 296) ++cut;
        dim3 grid(tiles, blocks, cut);
        if (w_dtype == GI_DTYPE_F32) {
            if (int rc = gi_reserve_smem((const void*)rglru_gates_wide_kernel<float>, smem, "gi_rglru_gates")) return rc;
            gi_launch(rglru_gates_wide_kernel<float>, grid, dim3(threads), smem, s, u, (const float*)wa_t, (const float*)wi_t,
                      ba, bi, lam, vec_dtype, decay_scale, a_out, b_out, n_rows, width, bw);
        } else {
            if (int rc = gi_reserve_smem((const void*)rglru_gates_wide_kernel<bf16>, smem, "gi_rglru_gates")) return rc;
            gi_launch(rglru_gates_wide_kernel<bf16>, grid, dim3(threads), smem, s, u, (const bf16*)wa_t, (const bf16*)wi_t,
                      ba, bi, lam, vec_dtype, decay_scale, a_out, b_out, n_rows, width, bw);
        }
        return gi_check_launch("gi_rglru_gates");
    }
    const int threads = RG_KS * (orange / RG_OG) * (tt / RG_TG);
    const int slices = (bw + orange - 1) / orange;
    // many rows: the rows are cut over the grid's third axis until there are about eight blocks of threads to an SM
    // one after the other (an SM holds one or two at a time; with fewer, longer ones the last round would leave most
    // SMs idle, and a block's own copy of its weights costs little)
    const int tiles = (n_rows + tt - 1) / tt;
    long long cut = (8LL * 148 + (long long)blocks * slices - 1) / ((long long)blocks * slices);
    cut = cut < 1 ? 1 : (cut > tiles ? tiles : (cut > 65535 ? 65535 : cut));
    const int rows_per_cta = (int)((tiles + cut - 1) / cut) * tt;
    dim3 grid(blocks, slices, (unsigned)((n_rows + rows_per_cta - 1) / rows_per_cta));
    const size_t smem = smem_of(orange, tt);
    if (w_dtype == GI_DTYPE_F32) {
        if (int rc = gi_reserve_smem((const void*)rglru_gates_kernel<float>, smem, "gi_rglru_gates")) return rc;
        gi_launch(rglru_gates_kernel<float>, grid, dim3(threads), smem, s, u, (const float*)wa_t, (const float*)wi_t, ba, bi,
                  lam, vec_dtype, decay_scale, a_out, b_out, n_rows, width, bw, orange, tt, rows_per_cta);
    } else {
        if (int rc = gi_reserve_smem((const void*)rglru_gates_kernel<bf16>, smem, "gi_rglru_gates")) return rc;
        gi_launch(rglru_gates_kernel<bf16>, grid, dim3(threads), smem, s, u, (const bf16*)wa_t, (const bf16*)wi_t, ba, bi,
                  lam, vec_dtype, decay_scale, a_out, b_out, n_rows, width, bw, orange, tt, rows_per_cta);
    }
    return gi_check_launch("gi_rglru_gates");
}

// The gate branch's activation, the tanh form of gelu: with the library's tanh for a float32 engine; for bfloat16
// (the activation of a projection, whose result is rounded to 8 bits of mantissa right after) with the hardware's
// approximate tanh, which is good to about 11 bits.
template <typename T> __device__ __forceinline__ float rg_gate_act(float z) { return rg_gelu_tanh(z); }
template <> __device__ __forceinline__ float rg_gate_act<bf16>(float z) {
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.7978845608028654f * (z + 0.044715f * z * z * z)));
    return 0.5f * z * (1.f + t);
}

// spans [n_seq, 3] = {slot, first row, rows}, or null: every row is a sequence of its own with the slot of tok_slot.
#define RG_SUB 4             // tokens to a group of the scan's ring of inputs
#define RG_DEPTH 8           // groups in the ring: 32 tokens' inputs under way
#define RG_SCAN_THREADS 32    // one warp to a block: one long prompt of a few thousand channels then reaches every SM
template <typename T>
__global__ void __launch_bounds__(RG_SCAN_THREADS)
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
    if (len == 1) {                                          // a decode step's row: nothing to run ahead of
        const size_t r = (size_t)start;
        S = fmaf(a[r * width + c], S, b[r * width + c]);
        out[r * ldo + c] = from_f32<T>(S * rg_gate_act<T>(to_f32(y[r * ldy + c]) + yb));
        state[(size_t)slot * state_stride + c] = S;
        return;
    }
    // The inputs of the next 32 tokens are on their way while a token is walked: a ring of eight groups of four
    // tokens in registers, each refilled right after it was used; beyond that the lines of the 32 tokens after
    // those are asked into L2 (a hint: lane j names token j of them).  A group is walked in two passes: the chain of
    // dependent multiply-adds alone, then the gate branch's activation and the products, which wait for nothing.
    const int lane = threadIdx.x & 31;
    const size_t cw = (size_t)(c - lane);                    // the warp's first channel
    float ra[RG_DEPTH][RG_SUB], rb[RG_DEPTH][RG_SUB], ry[RG_DEPTH][RG_SUB];
    auto fetch = [&](int t0, float (&fa)[RG_SUB], float (&fb)[RG_SUB], float (&fy)[RG_SUB]) {
#pragma unroll
        for (int j = 0; j < RG_SUB; ++j) {
            const bool in = t0 + j < len;
            const size_t r = (size_t)(start + (in ? t0 + j : 0));
            fa[j] = in ? a[r * width + c] : 1.f;             // beyond the sequence: S stays as it is
            fb[j] = in ? b[r * width + c] : 0.f;
            fy[j] = in ? to_f32(y[r * ldy + c]) : 0.f;
        }
    };
#pragma unroll
    for (int d = 0; d < RG_DEPTH; ++d) fetch(d * RG_SUB, ra[d], rb[d], ry[d]);
    for (int t0 = 0; t0 < len; t0 += RG_DEPTH * RG_SUB) {
        if (t0 + 2 * RG_DEPTH * RG_SUB + lane < len) {
            const size_t r = (size_t)(start + t0 + 2 * RG_DEPTH * RG_SUB + lane);
            asm volatile("prefetch.global.L2 [%0];" ::"l"(a + r * width + cw));
            asm volatile("prefetch.global.L2 [%0];" ::"l"(b + r * width + cw));
            asm volatile("prefetch.global.L2 [%0];" ::"l"(y + r * ldy + cw));
        }
#pragma unroll
        for (int d = 0; d < RG_DEPTH; ++d) {
            const int t1 = t0 + d * RG_SUB;
            float sv[RG_SUB];
#pragma unroll
            for (int j = 0; j < RG_SUB; ++j) {
                S = fmaf(ra[d][j], S, rb[d][j]);
                sv[j] = S;
            }
#pragma unroll
            for (int j = 0; j < RG_SUB; ++j)
                if (t1 + j < len) out[(size_t)(start + t1 + j) * ldo + c] = from_f32<T>(sv[j] * rg_gate_act<T>(ry[d][j] + yb));
            fetch(t1 + RG_DEPTH * RG_SUB, ra[d], rb[d], ry[d]);
        }
    }
    state[(size_t)slot * state_stride + c] = S;
}

extern "C" int gi_rglru_scan(const float* a, const float* b, const void* y, long long ldy, int act_dtype, const void* y_bias,
                             int bias_dtype, float* state, long long state_stride, const int* spans, const int* tok_slot,
                             void* out, long long ldo, int n_seqs, int width, void* stream) {
    GI_REQUIRE(n_seqs >= 0 && width > 0 && ldy >= width && ldo >= width && state_stride >= width, "gi_rglru_scan: sizes");
    GI_REQUIRE((width + RG_SCAN_THREADS - 1) / RG_SCAN_THREADS <= 65535, "gi_rglru_scan: %d channels", width);
    if (n_seqs == 0) return 0;
    dim3 grid(n_seqs, (width + RG_SCAN_THREADS - 1) / RG_SCAN_THREADS);
    cudaStream_t s = (cudaStream_t)stream;
    if (act_dtype == GI_DTYPE_F32)
        gi_launch(rglru_scan_kernel<float>, grid, dim3(RG_SCAN_THREADS), 0, s, a, b, (const float*)y, ldy, y_bias, bias_dtype, state,
                  state_stride, spans, tok_slot, (float*)out, ldo, width);
    else if (act_dtype == GI_DTYPE_BF16)
        gi_launch(rglru_scan_kernel<bf16>, grid, dim3(RG_SCAN_THREADS), 0, s, a, b, (const bf16*)y, ldy, y_bias, bias_dtype, state,
                  state_stride, spans, tok_slot, (bf16*)out, ldo, width);
    else
        GI_REQUIRE(false, "gi_rglru_scan: activation dtype %d", act_dtype);
    return gi_check_launch("gi_rglru_scan");
}
