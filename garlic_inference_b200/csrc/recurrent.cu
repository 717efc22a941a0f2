// Mixers that carry a matrix of state per head from token to token, and the short causal convolution in
// front of one of them.  All state is float32 and lives in the cache's per-slot state rows.
//
//   gi_causal_conv_silu     y[t, c] = silu( sum_j taps[c, j] x[t - (K-1) + j, c] ), zeros before position 0; the
//                           K-1 inputs before this step's first token come from the slot's state
//   gi_conv_state_update    afterwards: the slot's state becomes its last K-1 inputs
//   gi_decay_scan           S_t = lam_h S_(t-1) + k_t v_t^T,  o_t = S_t^T q_t           (q, k, v = silu of the
//                           projections): linear attention with one fixed decay per head
//   gi_delta_scan           S <- g_t S;  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;  o_t = S^T q_t
//                           with q, k made unit vectors per head (q also times dim^-1/2),
//                           g_t = exp(-exp(A_h) softplus(a_t + dt_h)),  beta_t = sigmoid(b_t): the gated delta rule;
//                           the decay is one number per head, or one per head and key channel (row c of a head's
//                           state times g_t[c])
//
// A scan block owns one (sequence, head, slice of 32 value columns) and walks the sequence's tokens of this
// step in order, so prompts, portions of prompts and single tokens run the same instructions in the same
// order and give the same bits.  P lanes share one value column: a thread holds R of the column's keys in
// registers (4 consecutive keys out of every 4 P), and sums over the keys end with log2(P) shuffles.  P is 4 or
// 8 by the key dimension alone (8 from 64 keys on): with one long prompt there are only heads x columns / 32
// blocks, and it is the warps of a block that hide each other's latencies.  Measured at keys of 128, 32 heads
// (P = 4 / 8 / 16): a prompt of 2,048 tokens 0.91 / 0.71 / 0.70 ms (decay) and 1.61 / 1.23 / 1.04 ms (delta rule); a
// whole decode step of 64 sequences 1.72 / 1.80 / 1.89 ms.  P never depends on the batch or the cut, so a
// position's bits do not either.
// The delta rule's scan asks for the next chunk's inputs (into registers) before it walks the present chunk's
// tokens, when the rows allow 16-byte loads: a prompt of 2,048 tokens, 16 heads of 128 x 128, 1.20 -> 0.77 ms with a
// decay per head and 1.68 -> 1.07 ms with one per key channel; what is computed, and in which order, is the same.
// State rows are laid out [head][value column][key, padded to R P] so that a warp's loads and stores are
// whole runs of 16 P bytes.  NikolayBlagoev/garlic-inference has no recurrent mixer.
#include "common.cuh"
#include <math.h>

__device__ __forceinline__ float rc_sigmoid(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float rc_silu(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float rc_softplus(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// ------------------------------------------------------------------ short causal convolution
#define CONV_MAX_TAPS 16

// In-step predecessors of row r that belong to the same sequence, at most `most`.
__device__ __forceinline__ int rows_before(const int* __restrict__ tok_slot, int r, int slot, int most) {
    int have = 0;
    while (have < most && r - have - 1 >= 0 && tok_slot[r - have - 1] == slot) ++have;
    return have;
}

template <typename T>
__global__ void causal_conv_silu_kernel(const T* __restrict__ x, long long ldx, int C, const void* __restrict__ taps,
                                        int taps_dtype, int K, const float* __restrict__ state, long long state_stride,
                                        const int* __restrict__ tok_slot, float* __restrict__ out, int act,
                                        float* __restrict__ state_out, const void* __restrict__ in_bias,
                                        const void* __restrict__ out_bias, int bias_dtype) {
    gi_pdl_start();
    const int r = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int slot = tok_slot[r];
    const int have = slot < 0 ? 0 : rows_before(tok_slot, r, slot, K - 1);
    // a bias on the inputs belongs to the tokens (what the state holds has it already, and before a sequence's
    // first token there are zeros, not biases); a bias on the outputs starts the sum
    const float bin = in_bias ? load_w(in_bias, bias_dtype, c) : 0.f;
    float acc = out_bias ? load_w(out_bias, bias_dtype, c) : 0.f;
    float seen[CONV_MAX_TAPS];                       // the inputs, oldest first (for the state when it is renewed here)
    for (int j = K - 1; j >= 0; --j) {               // oldest input first, whatever its source
        float xv = 0.f;
        if (j <= have) xv = to_f32(x[(size_t)(r - j) * ldx + c]) + bin;
        else if (slot >= 0) xv = state[(size_t)slot * state_stride + (size_t)(K - 1 + have - j) * C + c];
        seen[K - 1 - j] = xv;
        acc = fmaf(load_w(taps, taps_dtype, c * K + (K - 1 - j)), xv, acc);
    }
    out[(size_t)r * C + c] = act ? rc_silu(acc) : acc;
    // Steps in which every row is a sequence of its own (decode steps): the slot's state becomes its last K - 1 inputs
    // here, by the one thread that read it, instead of in a launch of its own.
    if (state_out && slot >= 0)
        for (int m = 0; m < K - 1; ++m) state_out[(size_t)slot * state_stride + (size_t)m * C + c] = seen[m + 1];
}

template <typename T>
__global__ void conv_state_update_kernel(const T* __restrict__ x, long long ldx, int C, int K,
                                         float* __restrict__ state, long long state_stride,
                                         const int* __restrict__ tok_slot, int n_rows,
                                         const void* __restrict__ in_bias, int bias_dtype) {
    gi_pdl_start();
    const int r = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int slot = tok_slot[r];
    if (slot < 0 || (r + 1 < n_rows && tok_slot[r + 1] == slot)) return;      // only a sequence's last row acts
    const int have = rows_before(tok_slot, r, slot, K - 1);
    const float bin = in_bias ? load_w(in_bias, bias_dtype, c) : 0.f;
    float* st = state + (size_t)slot * state_stride;
    float vals[CONV_MAX_TAPS];
    for (int m = 0; m < K - 1; ++m) {
        const int j = K - 2 - m;                     // how far before the last row
        vals[m] = j <= have ? to_f32(x[(size_t)(r - j) * ldx + c]) + bin : st[(size_t)(K - 1 + have - j) * C + c];
    }
    for (int m = 0; m < K - 1; ++m) st[(size_t)m * C + c] = vals[m];
}

// `act` 1: silu of the filter's sum; 0: the sum itself.  update_state 2: the filter and the renewal of the state in
// one launch, for steps in which no two rows belong to one sequence (the caller's promise).
// `in_bias` (one per channel, added to every input of a token) and `out_bias` (one per channel, added to the sum)
// may be null; they share `bias_dtype`.
extern "C" int gi_causal_conv_biased(const void* x, long long ldx, int act_dtype, int C, const void* taps, int taps_dtype,
                                     int K, float* state, long long state_stride, const int* tok_slot, float* out,
                                     int n_rows, int update_state, int act, const void* in_bias, const void* out_bias,
                                     int bias_dtype, void* stream) {
    GI_REQUIRE(n_rows >= 0 && C > 0 && K >= 1 && K <= CONV_MAX_TAPS, "gi_causal_conv_silu: %d channels, %d taps (1 to %d)",
               C, K, CONV_MAX_TAPS);
    GI_REQUIRE(ldx >= C && state_stride >= (long long)(K - 1) * C, "gi_causal_conv_silu: strides shorter than the rows");
    GI_REQUIRE((C + 127) / 128 <= 65535, "gi_causal_conv_silu: %d channels is beyond %d", C, 65535 * 128);
    if (n_rows == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(n_rows, (C + 127) / 128);
    if (act_dtype == GI_DTYPE_F32) {
        if (update_state != 1) gi_launch(causal_conv_silu_kernel<float>, grid, dim3(128), 0, s, (const float*)x, ldx, C, taps, taps_dtype, K, (const float*)state, state_stride, tok_slot, out, act, update_state == 2 && K > 1 ? state : (float*)nullptr, in_bias, out_bias, bias_dtype);
        else if (K > 1) gi_launch(conv_state_update_kernel<float>, grid, dim3(128), 0, s, (const float*)x, ldx, C, K, state, state_stride, tok_slot, n_rows, in_bias, bias_dtype);
    } else if (act_dtype == GI_DTYPE_BF16) {
        if (update_state != 1) gi_launch(causal_conv_silu_kernel<bf16>, grid, dim3(128), 0, s, (const bf16*)x, ldx, C, taps, taps_dtype, K, (const float*)state, state_stride, tok_slot, out, act, update_state == 2 && K > 1 ? state : (float*)nullptr, in_bias, out_bias, bias_dtype);
        else if (K > 1) gi_launch(conv_state_update_kernel<bf16>, grid, dim3(128), 0, s, (const bf16*)x, ldx, C, K, state, state_stride, tok_slot, n_rows, in_bias, bias_dtype);
    } else {
        GI_REQUIRE(false, "gi_causal_conv_silu: activation dtype %d", act_dtype);
    }
    return gi_check_launch("gi_causal_conv_silu");
}

extern "C" int gi_causal_conv(const void* x, long long ldx, int act_dtype, int C, const void* taps, int taps_dtype,
                              int K, float* state, long long state_stride, const int* tok_slot, float* out,
                              int n_rows, int update_state, int act, void* stream) {
    return gi_causal_conv_biased(x, ldx, act_dtype, C, taps, taps_dtype, K, state, state_stride, tok_slot, out, n_rows,
                                 update_state, act, nullptr, nullptr, GI_DTYPE_F32, stream);
}

extern "C" int gi_causal_conv_silu(const void* x, long long ldx, int act_dtype, int C, const void* taps, int taps_dtype,
                                   int K, float* state, long long state_stride, const int* tok_slot, float* out,
                                   int n_rows, int update_state, void* stream) {
    return gi_causal_conv(x, ldx, act_dtype, C, taps, taps_dtype, K, state, state_stride, tok_slot, out, n_rows,
                          update_state, 1, stream);
}

// ------------------------------------------------------------------ scans
// Tokens staged in shared memory at a time: 32 (16 for the widest keys, to stay inside 48 KB).  A chunk costs one
// round trip to global memory that nothing hides when a block has its SM to itself (one long prompt), so the
// chunk is as long as shared memory allows; the results do not depend on it.
#define SCAN_TC(DP) ((DP) <= 128 ? 32 : 16)
#define SCAN_VS 32           // value columns per block; a block has 32 P threads

// Where a sequence's rows are: from `spans` [n_seq, 3] = {slot, first row, rows}, or, without spans, sequence
// i is row i alone (a decode step: the slot comes from tok_slot).
__device__ __forceinline__ void scan_span(const int* __restrict__ spans, const int* __restrict__ tok_slot, int seq,
                                          int& slot, int& start, int& len) {
    if (spans) { slot = spans[3 * seq]; start = spans[3 * seq + 1]; len = spans[3 * seq + 2]; }
    else { slot = tok_slot[seq]; start = seq; len = 1; }
}

// A thread's R state values: register e = 4 i + w holds key (P i + part) * 4 + w of its value column.
#define KEY_OF(i, part) (((i) * P + (part)) * 4)

template <int R, int P>
__device__ __forceinline__ void scan_load_state(float (&S)[R], const float* __restrict__ st, int part) {
#pragma unroll
    for (int i = 0; i < R / 4; ++i) {
        const float4 v = *reinterpret_cast<const float4*>(st + KEY_OF(i, part));
        S[4 * i] = v.x; S[4 * i + 1] = v.y; S[4 * i + 2] = v.z; S[4 * i + 3] = v.w;
    }
}
template <int R, int P>
__device__ __forceinline__ void scan_store_state(const float (&S)[R], float* __restrict__ st, int part) {
#pragma unroll
    for (int i = 0; i < R / 4; ++i)
        *reinterpret_cast<float4*>(st + KEY_OF(i, part)) = make_float4(S[4 * i], S[4 * i + 1], S[4 * i + 2], S[4 * i + 3]);
}
template <int P>
__device__ __forceinline__ float part_sum(float v) {               // over the P lanes of one value column
#pragma unroll
    for (int o = 1; o < P; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// ---- linear attention with a fixed decay per head
// qkv: T [n, ld], silu applied here; q at column q_off + h d, k at k_off + h d, v at v_off + h dv.
template <typename T, int R, int P>
__global__ void __launch_bounds__(SCAN_VS * P)
decay_scan_kernel(const T* __restrict__ qkv, long long ld, int q_off, int k_off, int v_off,
                  const float* __restrict__ decay, float* __restrict__ state, long long state_stride,
                  const int* __restrict__ spans, const int* __restrict__ tok_slot, float* __restrict__ out,
                  int H, int d, int dv, int vec_rows) {
    gi_pdl_start();
    const bool vec = sizeof(T) == 2 && vec_rows;       // rows that can be fetched 16 bytes at a time
    constexpr int DP = R * P;                          // padded key dimension
    constexpr int TC = SCAN_TC(DP);
    constexpr int SCAN_THREADS = SCAN_VS * P;
    __shared__ __align__(16) float q_s[TC][DP];
    __shared__ __align__(16) float k_s[TC][DP];
    __shared__ float v_s[TC][SCAN_VS];
    __shared__ float o_s[TC][SCAN_VS];
    int slot, start, len;
    scan_span(spans, tok_slot, blockIdx.x, slot, start, len);
    const int h = blockIdx.y, v0 = blockIdx.z * SCAN_VS;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int part = threadIdx.x % P, vl = threadIdx.x / P, v = v0 + vl;
    const bool live = v < dv;
    if (slot < 0) {
        for (int t = 0; t < len; ++t)
            if (live && part == 0) out[(size_t)(start + t) * H * dv + h * dv + v] = 0.f;
        return;
    }
    const float lam = decay[h];
    float* st = state + (size_t)slot * state_stride + ((size_t)h * dv + (live ? v : 0)) * DP;
    float S[R];
    if (live) scan_load_state<R, P>(S, st, part);
    else {
#pragma unroll
        for (int e = 0; e < R; ++e) S[e] = 0.f;
    }
    // Staging.  bfloat16 rows whose heads start on 16 bytes: every thread fetches NV vectors of 8 values of q and
    // k (and one of v) into registers, all at once, and the next chunk's are fetched before this chunk's tokens
    // are walked, so their latency hides behind the walk.  Otherwise: element by element.
    constexpr int VPT = DP / 8;                        // vectors per token and operand
    constexpr int NV = (TC * VPT * 2 + SCAN_THREADS - 1) / SCAN_THREADS;
    uint4 pre[NV], pre_v;
    auto fetch = [&](int t0) {
        const int tc = min(TC, len - t0);
#pragma unroll
        for (int n = 0; n < NV; ++n) {
            const int slot_i = threadIdx.x + SCAN_THREADS * n;
            const int which = slot_i / (TC * VPT), rem = slot_i - which * (TC * VPT);
            const int t = rem / VPT, vc = rem - t * VPT;
            pre[n] = make_uint4(0u, 0u, 0u, 0u);
            if (which < 2 && t < tc && vc * 8 < d)
                pre[n] = *reinterpret_cast<const uint4*>(qkv + (size_t)(start + t0 + t) * ld + (which ? k_off : q_off) + h * d + vc * 8);
        }
        const int t = threadIdx.x / (SCAN_VS / 8), vc = threadIdx.x - t * (SCAN_VS / 8);
        pre_v = make_uint4(0u, 0u, 0u, 0u);
        if (t < tc && v0 + vc * 8 < dv)
            pre_v = *reinterpret_cast<const uint4*>(qkv + (size_t)(start + t0 + t) * ld + v_off + h * dv + v0 + vc * 8);
    };
    auto silu8 = [](const uint4& w, float* dst) {
        const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&w);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(p2[i]);
            dst[2 * i] = rc_silu(f.x);
            dst[2 * i + 1] = rc_silu(f.y);
        }
    };
    if (vec) fetch(0);
    for (int t0 = 0; t0 < len; t0 += TC) {
        const int tc = min(TC, len - t0);
        __syncthreads();                               // the last chunk's o_s and inputs are done with
        if (vec) {
#pragma unroll
            for (int n = 0; n < NV; ++n) {
                const int slot_i = threadIdx.x + SCAN_THREADS * n;
                const int which = slot_i / (TC * VPT), rem = slot_i - which * (TC * VPT);
                const int t = rem / VPT, vc = rem - t * VPT;
                if (which < 2 && t < tc) silu8(pre[n], (which ? &k_s[t][0] : &q_s[t][0]) + vc * 8);   // silu(0) = 0: the padding
            }
            const int t = threadIdx.x / (SCAN_VS / 8), vc = threadIdx.x - t * (SCAN_VS / 8);
            if (t < tc) silu8(pre_v, &v_s[t][vc * 8]);
        } else {
            for (int i = threadIdx.x; i < tc * DP; i += SCAN_THREADS) {
                const int t = i / DP, c = i - t * DP;
                const T* row = qkv + (size_t)(start + t0 + t) * ld;
                q_s[t][c] = c < d ? rc_silu(to_f32(row[q_off + h * d + c])) : 0.f;
                k_s[t][c] = c < d ? rc_silu(to_f32(row[k_off + h * d + c])) : 0.f;
            }
            for (int i = threadIdx.x; i < tc * SCAN_VS; i += SCAN_THREADS) {
                const int t = i / SCAN_VS, c = i - t * SCAN_VS;
                v_s[t][c] = v0 + c < dv ? rc_silu(to_f32(qkv[(size_t)(start + t0 + t) * ld + v_off + h * dv + v0 + c])) : 0.f;
            }
        }
        __syncthreads();
        if (vec && t0 + TC < len) fetch(t0 + TC);
        for (int t = 0; t < tc; ++t) {
            const float vt = v_s[t][vl];
            float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;     // four chains instead of one of R dependent steps
#pragma unroll
            for (int i = 0; i < R / 4; ++i) {
                const float4 kk = *reinterpret_cast<const float4*>(&k_s[t][KEY_OF(i, part)]);
                const float4 qq = *reinterpret_cast<const float4*>(&q_s[t][KEY_OF(i, part)]);
                S[4 * i] = fmaf(lam, S[4 * i], kk.x * vt);          o0 = fmaf(S[4 * i], qq.x, o0);
                S[4 * i + 1] = fmaf(lam, S[4 * i + 1], kk.y * vt);  o1 = fmaf(S[4 * i + 1], qq.y, o1);
                S[4 * i + 2] = fmaf(lam, S[4 * i + 2], kk.z * vt);  o2 = fmaf(S[4 * i + 2], qq.z, o2);
                S[4 * i + 3] = fmaf(lam, S[4 * i + 3], kk.w * vt);  o3 = fmaf(S[4 * i + 3], qq.w, o3);
            }
            const float o = part_sum<P>((o0 + o1) + (o2 + o3));
            if (part == 0) o_s[t][vl] = o;
        }
        __syncthreads();
        for (int i = threadIdx.x; i < tc * SCAN_VS; i += SCAN_THREADS) {
            const int t = i / SCAN_VS, c = i - t * SCAN_VS;
            if (v0 + c < dv) out[(size_t)(start + t0 + t) * H * dv + h * dv + v0 + c] = o_s[t][c];
        }
    }
    if (live) scan_store_state<R, P>(S, st, part);
}

// ---- the gated delta rule
// qkv: float32 [n, ldq] (the convolution's output): q of key head kh at q_off + kh d, k at k_off + kh d, v of
// head h at v_off + h dv.  ab: float32 [n, ldab]: beta's logit of head h at column b_off + h, the decay's at
// a_off + h (float32 whatever the activation type is: the decay's logit is multiplied by exp(A_h) and goes
// through two exponentials, which would magnify a 16-bit rounding).
// CH = 1: a decay per head and key channel.  The logits are then [n, H d] (column a_off + h d + c), dt_bias has
// H d elements, and row c of a head's state is multiplied by g[c]; chunks are shorter so that the decays of a
// chunk fit shared memory beside its keys.
#define SCAN_TC_CH(DP) ((DP) <= 64 ? 32 : ((DP) <= 128 ? 16 : 8))
template <typename T, int R, int P, int CH>
__global__ void __launch_bounds__(SCAN_VS * P)
delta_scan_kernel(const float* __restrict__ qkv, long long ldq, int q_off, int k_off, int v_off,
                  const float* __restrict__ ab, long long ldab, int b_off, int a_off,
                  const float* __restrict__ al, long long ldal,
                  const void* __restrict__ A_log, const void* __restrict__ dt_bias, int p_dtype,
                  float* __restrict__ state, long long state_stride, const int* __restrict__ spans,
                  const int* __restrict__ tok_slot, float* __restrict__ out, int H, int Hk, int d, int dv,
                  float unit_eps, float q_scale, int vec) {
    gi_pdl_start();
    constexpr int DP = R * P;
    constexpr int TC = CH ? SCAN_TC_CH(DP) : SCAN_TC(DP);
    constexpr int SCAN_THREADS = SCAN_VS * P;
    __shared__ __align__(16) float q_s[TC][DP];
    __shared__ __align__(16) float k_s[TC][DP];
    __shared__ __align__(16) float gc_s[CH ? TC : 1][CH ? DP : 4];
    __shared__ float v_s[TC][SCAN_VS];
    __shared__ float o_s[TC][SCAN_VS];
    __shared__ float g_s[TC], b_s[TC];
    int slot, start, len;
    scan_span(spans, tok_slot, blockIdx.x, slot, start, len);
    const int h = blockIdx.y, v0 = blockIdx.z * SCAN_VS;
    const int kh = h / (H / Hk);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int part = threadIdx.x % P, vl = threadIdx.x / P, v = v0 + vl;
    const bool live = v < dv;
    if (slot < 0) {
        for (int t = 0; t < len; ++t)
            if (live && part == 0) out[(size_t)(start + t) * H * dv + h * dv + v] = 0.f;
        return;
    }
    const float rate = expf(load_w(A_log, p_dtype, h)), dt = CH ? 0.f : load_w(dt_bias, p_dtype, h);
    float* st = state + (size_t)slot * state_stride + ((size_t)h * dv + (live ? v : 0)) * DP;
    float S[R];
    if (live) scan_load_state<R, P>(S, st, part);
    else {
#pragma unroll
        for (int e = 0; e < R; ++e) S[e] = 0.f;
    }
    // Each warp stages tokens warp, warp + W, ... of a chunk (W warps).  When the rows allow 16-byte loads, the raw
    // values of the NEXT chunk's tokens are asked for into registers before this chunk's tokens are walked, so that
    // the walk hides their latency; what is done with them, and in which order, is the same either way.
    constexpr int TPW = TC / (SCAN_THREADS / 32);
    constexpr int NQ = (DP / 4 + 31) / 32;                 // 16-byte pieces of q (and of k) per lane and token
    constexpr int NA = CH ? (DP + 31) / 32 : 1;            // decay logits per lane and token
    float4 pq[TPW][NQ], pk[TPW][NQ];
    float pv[TPW], pa[TPW][NA], pb[TPW], dtc[NA];
#pragma unroll
    for (int n = 0; n < NA; ++n) {
        const int c = lane + 32 * n;
        dtc[n] = (CH && c < d) ? load_w(dt_bias, p_dtype, h * d + c) : 0.f;
    }
    auto fetch = [&](int t0) {
        const int tc = min(TC, len - t0);
#pragma unroll
        for (int i = 0; i < TPW; ++i) {
            const int t = warp + (SCAN_THREADS / 32) * i;
            if (t >= tc) continue;
            const float* row = qkv + (size_t)(start + t0 + t) * ldq;
            const float* abr = ab + (size_t)(start + t0 + t) * ldab;
            const float* alr = al + (size_t)(start + t0 + t) * ldal;
#pragma unroll
            for (int n = 0; n < NQ; ++n) {
                const int c4 = lane + 32 * n;
                pq[i][n] = make_float4(0.f, 0.f, 0.f, 0.f);
                pk[i][n] = pq[i][n];
                if (c4 < DP / 4 && c4 * 4 < d) {
                    pq[i][n] = *reinterpret_cast<const float4*>(row + q_off + kh * d + c4 * 4);
                    pk[i][n] = *reinterpret_cast<const float4*>(row + k_off + kh * d + c4 * 4);
                }
            }
            pv[i] = v0 + lane < dv ? row[v_off + h * dv + v0 + lane] : 0.f;
            if (CH) {
#pragma unroll
                for (int n = 0; n < NA; ++n) {
                    const int c = lane + 32 * n;
                    pa[i][n] = c < d ? alr[a_off + h * d + c] : 0.f;
                }
            } else {
                pa[i][0] = lane == 0 ? alr[a_off + h] : 0.f;
            }
            pb[i] = lane == 0 ? abr[b_off + h] : 0.f;
        }
    };
    if (vec) fetch(0);
    for (int t0 = 0; t0 < len; t0 += TC) {
        const int tc = min(TC, len - t0);
        __syncthreads();
        // raw q, k and v of a warp's tokens into shared memory, then q and k as unit vectors (sum of squares: a
        // lane's elements in order, then a tree over the lanes)
        float sq[TPW], sk[TPW];
#pragma unroll
        for (int i = 0; i < TPW; ++i) {
            const int t = warp + (SCAN_THREADS / 32) * i;
            sq[i] = 0.f; sk[i] = 0.f;
            if (t >= tc) continue;
            const float* row = qkv + (size_t)(start + t0 + t) * ldq;
            const float* abr = ab + (size_t)(start + t0 + t) * ldab;
            const float* alr = al + (size_t)(start + t0 + t) * ldal;
            if (vec) {
#pragma unroll
                for (int n = 0; n < NQ; ++n) {
                    const int c4 = lane + 32 * n;
                    if (c4 >= DP / 4) continue;
                    const float4 qv = pq[i][n], kv = pk[i][n];
                    *reinterpret_cast<float4*>(&q_s[t][c4 * 4]) = qv;
                    *reinterpret_cast<float4*>(&k_s[t][c4 * 4]) = kv;
                    sq[i] = fmaf(qv.x, qv.x, sq[i]); sq[i] = fmaf(qv.y, qv.y, sq[i]);
                    sq[i] = fmaf(qv.z, qv.z, sq[i]); sq[i] = fmaf(qv.w, qv.w, sq[i]);
                    sk[i] = fmaf(kv.x, kv.x, sk[i]); sk[i] = fmaf(kv.y, kv.y, sk[i]);
                    sk[i] = fmaf(kv.z, kv.z, sk[i]); sk[i] = fmaf(kv.w, kv.w, sk[i]);
                }
                v_s[t][lane] = pv[i];
                if (CH) {
#pragma unroll
                    for (int n = 0; n < NA; ++n) {
                        const int c = lane + 32 * n;
                        if (c < DP) gc_s[t][c] = c < d ? expf(-rate * rc_softplus(pa[i][n] + dtc[n])) : 1.f;
                    }
                }
                if (lane == 0) {
                    if (!CH) g_s[t] = expf(-rate * rc_softplus(pa[i][0] + dt));
                    b_s[t] = rc_sigmoid(pb[i]);
                }
                continue;
            }
            for (int c = lane; c < DP; c += 32) {
                const float qv = c < d ? row[q_off + kh * d + c] : 0.f;
                const float kv = c < d ? row[k_off + kh * d + c] : 0.f;
                q_s[t][c] = qv; k_s[t][c] = kv;
                sq[i] = fmaf(qv, qv, sq[i]); sk[i] = fmaf(kv, kv, sk[i]);
            }
            v_s[t][lane] = v0 + lane < dv ? row[v_off + h * dv + v0 + lane] : 0.f;
            if (CH) {
                for (int c = lane; c < DP; c += 32)
                    gc_s[t][c] = c < d ? expf(-rate * rc_softplus(alr[a_off + h * d + c] + load_w(dt_bias, p_dtype, h * d + c))) : 1.f;
            }
            if (lane == 0) {
                if (!CH) g_s[t] = expf(-rate * rc_softplus(alr[a_off + h] + dt));
                b_s[t] = rc_sigmoid(abr[b_off + h]);
            }
        }
#pragma unroll
        for (int i = 0; i < TPW; ++i) {
            const int t = warp + (SCAN_THREADS / 32) * i;
            if (t >= tc) continue;
            const float iq = q_scale / sqrtf(warp_sum(sq[i]) + unit_eps), ik = 1.f / sqrtf(warp_sum(sk[i]) + unit_eps);
            for (int c = lane; c < DP; c += 32) { q_s[t][c] *= iq; k_s[t][c] *= ik; }
        }
        __syncthreads();
        if (vec && t0 + TC < len) fetch(t0 + TC);
        for (int t = 0; t < tc; ++t) {
            const float g = CH ? 1.f : g_s[t];
            float r0 = 0.f, r1 = 0.f, r2 = 0.f, r3 = 0.f;     // four chains instead of one of R dependent steps
#pragma unroll
            for (int i = 0; i < R / 4; ++i) {
                const float4 kk = *reinterpret_cast<const float4*>(&k_s[t][KEY_OF(i, part)]);
                float4 gg = make_float4(g, g, g, g);
                if (CH) gg = *reinterpret_cast<const float4*>(&gc_s[t][KEY_OF(i, part)]);
                S[4 * i] *= gg.x;      r0 = fmaf(S[4 * i], kk.x, r0);
                S[4 * i + 1] *= gg.y;  r1 = fmaf(S[4 * i + 1], kk.y, r1);
                S[4 * i + 2] *= gg.z;  r2 = fmaf(S[4 * i + 2], kk.z, r2);
                S[4 * i + 3] *= gg.w;  r3 = fmaf(S[4 * i + 3], kk.w, r3);
            }
            const float r = part_sum<P>((r0 + r1) + (r2 + r3));
            const float u = b_s[t] * (v_s[t][vl] - r);
            float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
            for (int i = 0; i < R / 4; ++i) {
                const float4 kk = *reinterpret_cast<const float4*>(&k_s[t][KEY_OF(i, part)]);
                const float4 qq = *reinterpret_cast<const float4*>(&q_s[t][KEY_OF(i, part)]);
                S[4 * i] = fmaf(kk.x, u, S[4 * i]);          o0 = fmaf(S[4 * i], qq.x, o0);
                S[4 * i + 1] = fmaf(kk.y, u, S[4 * i + 1]);  o1 = fmaf(S[4 * i + 1], qq.y, o1);
                S[4 * i + 2] = fmaf(kk.z, u, S[4 * i + 2]);  o2 = fmaf(S[4 * i + 2], qq.z, o2);
                S[4 * i + 3] = fmaf(kk.w, u, S[4 * i + 3]);  o3 = fmaf(S[4 * i + 3], qq.w, o3);
            }
            const float o = part_sum<P>((o0 + o1) + (o2 + o3));
            if (part == 0) o_s[t][vl] = o;
        }
        __syncthreads();
        for (int i = threadIdx.x; i < tc * SCAN_VS; i += SCAN_THREADS) {
            const int t = i / SCAN_VS, c = i - t * SCAN_VS;
            if (v0 + c < dv) out[(size_t)(start + t0 + t) * H * dv + h * dv + v0 + c] = o_s[t][c];
        }
    }
    if (live) scan_store_state<R, P>(S, st, part);
}

// The padded key dimension for d: 16, 32, 64, 128 or 256 (0: too large).
static int scan_padded(int d) {
    for (int dp = 16; dp <= 256; dp *= 2)
        if (dp >= d) return dp;
    return 0;
}

// Floats of one head's state for key dimension d and value dimension dv, as the scans lay it out.
extern "C" long long gi_scan_state_floats(int d, int dv) {
    const int dp = scan_padded(d);
    return dp ? (long long)dv * dp : -1;
}

// (registers, lanes per column) by padded key dimension: 16 -> (4, 4), 32 -> (8, 4), 64 -> (8, 8), 128 -> (16, 8),
// 256 -> (32, 8)
#define SCAN_DISPATCH_X(KERNEL, TT, X, ...)                                                              \
    switch (DP) {                                                                                        \
        case 16:  gi_launch(KERNEL<TT, 4, 4 X>, grid, dim3(SCAN_VS * 4), 0, s, __VA_ARGS__); break;      \
        case 32:  gi_launch(KERNEL<TT, 8, 4 X>, grid, dim3(SCAN_VS * 4), 0, s, __VA_ARGS__); break;      \
        case 64:  gi_launch(KERNEL<TT, 8, 8 X>, grid, dim3(SCAN_VS * 8), 0, s, __VA_ARGS__); break;      \
        case 128: gi_launch(KERNEL<TT, 16, 8 X>, grid, dim3(SCAN_VS * 8), 0, s, __VA_ARGS__); break;     \
        default:  gi_launch(KERNEL<TT, 32, 8 X>, grid, dim3(SCAN_VS * 8), 0, s, __VA_ARGS__); break;     \
    }
#define SCAN_NOTHING
#define SCAN_COMMA(v) , v
#define SCAN_DISPATCH(KERNEL, TT, ...) SCAN_DISPATCH_X(KERNEL, TT, SCAN_NOTHING, __VA_ARGS__)

extern "C" int gi_decay_scan(const void* qkv, long long ld, int act_dtype, int q_off, int k_off, int v_off,
                             const float* decay, float* state, long long state_stride, const int* spans,
                             const int* tok_slot, float* out, int n_seq, int H, int d, int dv, void* stream) {
    const int DP = scan_padded(d);
    GI_REQUIRE(n_seq >= 0 && H > 0 && d > 0 && dv > 0 && DP > 0, "gi_decay_scan: key dimension %d (at most 256)", d);
    GI_REQUIRE(H <= 65535 && (dv + SCAN_VS - 1) / SCAN_VS <= 65535, "gi_decay_scan: %d heads of %d values", H, dv);
    GI_REQUIRE(state_stride >= (long long)H * dv * DP && state_stride % 4 == 0, "gi_decay_scan: state rows of %lld "
               "floats are shorter than %lld or no multiple of 4", state_stride, (long long)H * dv * DP);
    if (n_seq == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(n_seq, H, (dv + SCAN_VS - 1) / SCAN_VS);
    if (act_dtype == GI_DTYPE_F32) {
        SCAN_DISPATCH(decay_scan_kernel, float, (const float*)qkv, ld, q_off, k_off, v_off, decay, state, state_stride, spans, tok_slot, out, H, d, dv, 0)
    } else if (act_dtype == GI_DTYPE_BF16) {
        const int vec_rows = d % 8 == 0 && dv % 8 == 0 && ld % 8 == 0 && q_off % 8 == 0 && k_off % 8 == 0 && v_off % 8 == 0 &&
                             (uintptr_t)qkv % 16 == 0;
        SCAN_DISPATCH(decay_scan_kernel, bf16, (const bf16*)qkv, ld, q_off, k_off, v_off, decay, state, state_stride, spans, tok_slot, out, H, d, dv, vec_rows)
    } else {
        GI_REQUIRE(false, "gi_decay_scan: activation dtype %d", act_dtype);
    }
    return gi_check_launch("gi_decay_scan");
}

extern "C" int gi_delta_scan(const float* qkv, long long ldq, int q_off, int k_off, int v_off, const float* ab,
                             long long ldab, int b_off, int a_off, const float* a_sep, long long lda_sep,
                             const void* A_log, const void* dt_bias,
                             int p_dtype, float* state, long long state_stride, const int* spans, const int* tok_slot,
                             float* out, int n_seq, int H, int Hk, int d, int dv, float unit_eps, float q_scale,
                             int channel_decay, void* stream) {
    const int DP = scan_padded(d);
    GI_REQUIRE(n_seq >= 0 && H > 0 && Hk > 0 && H % Hk == 0 && d > 0 && dv > 0 && DP > 0,
               "gi_delta_scan: %d heads on %d key heads, key dimension %d (at most 256)", H, Hk, d);
    GI_REQUIRE(H <= 65535 && (dv + SCAN_VS - 1) / SCAN_VS <= 65535, "gi_delta_scan: %d heads of %d values", H, dv);
    GI_REQUIRE(state_stride >= (long long)H * dv * DP && state_stride % 4 == 0, "gi_delta_scan: state rows of %lld "
               "floats are shorter than %lld or no multiple of 4", state_stride, (long long)H * dv * DP);
    if (n_seq == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(n_seq, H, (dv + SCAN_VS - 1) / SCAN_VS);
    const int vec = d % 4 == 0 && ldq % 4 == 0 && q_off % 4 == 0 && k_off % 4 == 0 && (uintptr_t)qkv % 16 == 0;
    // the decay's logits: columns of `ab`, or a matrix of their own
    const float* al = a_sep ? a_sep : ab;
    const long long ldal = a_sep ? lda_sep : ldab;
    if (channel_decay) {
        SCAN_DISPATCH_X(delta_scan_kernel, float, SCAN_COMMA(1), qkv, ldq, q_off, k_off, v_off, ab, ldab, b_off, a_off, al, ldal, A_log, dt_bias, p_dtype, state, state_stride, spans, tok_slot, out, H, Hk, d, dv, unit_eps, q_scale, vec)
    } else {
        SCAN_DISPATCH_X(delta_scan_kernel, float, SCAN_COMMA(0), qkv, ldq, q_off, k_off, v_off, ab, ldab, b_off, a_off, al, ldal, A_log, dt_bias, p_dtype, state, state_stride, spans, tok_slot, out, H, Hk, d, dv, unit_eps, q_scale, vec)
    }
    return gi_check_launch("gi_delta_scan");
}
