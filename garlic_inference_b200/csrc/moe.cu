// A routed feed-forward: every token runs `top` of `experts` small feed-forwards and sums their results with
// the router's weights.
//
//   gi_router_logits   z = W_r x in float32 (float32 weight, the token's vector widened)
//   gi_router_topk     per token: the `top` largest of its float32 router logits (ties: the lower index), in
//                      falling order, and the softmax over those chosen logits alone
//   gi_router_select   per token: scores = softmax of its float32 router logits over all experts; the experts lie in
//                      `groups` equal groups of neighbours, a group's score is its best expert's, and only the
//                      `keep` best groups stay; the `top` largest scores among them are chosen (ties: the lower
//                      index), in falling order; the weights are those scores times `scale`, not renormalised.
//                      Options: scores = sigmoid of each logit instead of the softmax; a correction per expert added
//                      to the scores that choose (groups and experts) but not to the weights; a group's score the
//                      sum of its `group_top` best choosing scores; the weights divided by their sum (+ 1e-20)
//                      before the factor.  Experts of groups that do not stay cannot be chosen, whatever their scores.
//   gi_moe_up          a[t, j, :] = act( W_up[e_tj] x_t )          act: the square of relu (0) or silu (1); or (2)
//                      a gated unit: W_up[e] holds ff gate rows and then ff up rows, a = unit(gate, up) (glu.cuh)
//   gi_moe_down        part[t, j, :] = W_down[e_tj] a[t, j, :]
//   gi_moe_group       the (token, choice) pairs in the order of their experts: each pair's row, each expert's last
//                      row, and the tokens' vectors gathered into that order (a stable counting sort)
//   gi_moe_combine     y[t, :] = (add[t, :] +) sum_j w_tj buf[where[t, j], :]   in the router's order of j: over gi_moe_down's
//                      rows (where = none: row t top + j), or over rows that a grouped product wrote expert by expert
//
// gi_moe_up and gi_moe_down read only the chosen experts' weights and take the expert of a row from device
// memory, so a recorded decode step replays them for other tokens.  They are products of one row with a matrix,
// a warp per row of W, the token's vector in shared memory as float32: the right shape for a handful of tokens.
// Prompts go expert by expert through the matrix products (parts/moe.py) and gi_moe_combine.  Sums are float32 in a
// fixed order; a token's result does not depend on the other tokens of the step.
// NikolayBlagoev/garlic-inference's mixture-of-experts path is a different design (src/models/qwen3/qwen3-moe.cpp).
#include "common.cuh"
#include "glu.cuh"
#include <math.h>

// ------------------------------------------------------------------ router
__global__ void router_topk_kernel(const float* __restrict__ logits, long long ld, int E, int top,
                                   int* __restrict__ idx_out, float* __restrict__ w_out, int n_rows) {
    gi_pdl_start();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = blockIdx.x * (blockDim.x >> 5) + warp;
    if (r >= n_rows) return;
    const float* z = logits + (size_t)r * ld;
    float first = 0.f, sum = 0.f;
    float prev_v = INFINITY;
    int prev_i = -1;
    for (int j = 0; j < top; ++j) {
        // the largest logit after (prev_v, prev_i) in the order (value falling, index rising)
        float best = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = z[e];
            const bool after = v < prev_v || (v == prev_v && e > prev_i);
            if (after && (v > best || (v == best && e < bi))) { best = v; bi = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        if (j == 0) first = best;
        const float p = expf(best - first);
        sum += p;
        if (lane == 0) { idx_out[(size_t)r * top + j] = bi; w_out[(size_t)r * top + j] = p; }
        prev_v = best; prev_i = bi;
    }
    __syncwarp();
    if (lane == 0)
        for (int j = 0; j < top; ++j) w_out[(size_t)r * top + j] /= sum;
}

extern "C" int gi_router_topk(const float* logits, long long ld, int E, int top, int* idx_out, float* w_out, int n_rows,
                              void* stream) {
    GI_REQUIRE(n_rows >= 0 && E > 0 && top > 0 && top <= E && ld >= E, "gi_router_topk: %d of %d experts", top, E);
    if (n_rows == 0) return 0;
    gi_launch(router_topk_kernel, dim3((n_rows + 3) / 4), dim3(128), 0, (cudaStream_t)stream, logits, ld, E, top, idx_out,
              w_out, n_rows);
    return gi_check_launch("gi_router_topk");
}

// Scores over all experts, groups of neighbours, the best groups' best experts.  A warp per token; its scores and
// its groups' scores live in shared memory.
#define RS_WARPS 4
__global__ void __launch_bounds__(RS_WARPS * 32)
router_select_kernel(const float* __restrict__ logits, long long ld, int E, int top, int groups, int keep, float scale,
                     int* __restrict__ idx_out, float* __restrict__ w_out, int n_rows, int sigmoid_scores,
                     const float* __restrict__ correction, int group_top, int normalize) {
    gi_pdl_start();
    extern __shared__ float rs_smem[];                   // per warp: E scores that choose, E plain scores, `groups` group scores
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = blockIdx.x * RS_WARPS + warp;
    if (r >= n_rows) return;
    float* sc = rs_smem + (size_t)warp * (2 * E + groups);
    float* plain = sc + E;
    float* gs = plain + E;
    const float* z = logits + (size_t)r * ld;
    if (sigmoid_scores) {
        for (int e = lane; e < E; e += 32) plain[e] = 1.f / (1.f + expf(-z[e]));
    } else {
        float m = -INFINITY;
        for (int e = lane; e < E; e += 32) m = fmaxf(m, z[e]);
        m = warp_max(m);
        float sum = 0.f;
        for (int e = lane; e < E; e += 32) { const float p = expf(z[e] - m); plain[e] = p; sum += p; }
        sum = warp_sum(sum);
        __syncwarp();
        for (int e = lane; e < E; e += 32) plain[e] = plain[e] / sum;
    }
    __syncwarp();
    for (int e = lane; e < E; e += 32) sc[e] = correction ? plain[e] + correction[e] : plain[e];
    __syncwarp();
    const int per = E / groups;
    if (keep < groups) {
        for (int g = lane; g < groups; g += 32) {
            float b = -INFINITY, b2 = -INFINITY;         // the group's best and second best
            for (int k = 0; k < per; ++k) {
                const float v = sc[g * per + k];
                if (v > b) { b2 = b; b = v; } else if (v > b2) b2 = v;
            }
            gs[g] = group_top >= 2 && per >= 2 ? b + b2 : b;
        }
        __syncwarp();
        // the `keep` best groups in the order (score falling, index rising); the others' experts leave the choice
        float prev_v = INFINITY;
        int prev_i = -1;
        for (int j = 0; j < keep; ++j) {
            float best = -INFINITY;
            int bi = 0x7fffffff;
            for (int g = lane; g < groups; g += 32) {
                const float v = gs[g];
                const bool after = v < prev_v || (v == prev_v && g > prev_i);
                if (after && (v > best || (v == best && g < bi))) { best = v; bi = g; }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, best, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
            }
            prev_v = best; prev_i = bi;
        }
        __syncwarp();
        // a group stays if it comes no later than the last one kept in that order
        for (int g = lane; g < groups; g += 32) {
            const float v = gs[g];
            const bool kept = v > prev_v || (v == prev_v && g <= prev_i);
            gs[g] = kept ? 1.f : 0.f;
        }
        __syncwarp();
    }
    float prev_v = INFINITY;
    int prev_i = -1;
    for (int j = 0; j < top; ++j) {
        float best = -INFINITY;
        int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            if (keep < groups && gs[e / per] == 0.f) continue;
            const float v = sc[e];
            const bool after = v < prev_v || (v == prev_v && e > prev_i);
            if (after && (v > best || (v == best && e < bi))) { best = v; bi = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        if (lane == 0) { idx_out[(size_t)r * top + j] = bi; w_out[(size_t)r * top + j] = plain[bi]; }
        prev_v = best; prev_i = bi;
    }
    __syncwarp();
    if (lane == 0) {
        float mul = scale;
        if (normalize) {
            float sum = 0.f;
            for (int j = 0; j < top; ++j) sum += w_out[(size_t)r * top + j];
            mul = scale / (sum + 1e-20f);
        }
        for (int j = 0; j < top; ++j) w_out[(size_t)r * top + j] *= mul;
    }
}

extern "C" int gi_router_select(const float* logits, long long ld, int E, int top, int groups, int keep, float scale,
                                int* idx_out, float* w_out, int n_rows, int sigmoid_scores, const float* correction,
                                int group_top, int normalize, void* stream) {
    GI_REQUIRE(group_top == 1 || group_top == 2, "gi_router_select: a group is judged by its best or its two best experts");
    GI_REQUIRE(n_rows >= 0 && E > 0 && ld >= E, "gi_router_select: sizes");
    GI_REQUIRE(groups > 0 && E % groups == 0 && keep > 0 && keep <= groups, "gi_router_select: %d experts in %d groups of which %d stay", E, groups, keep);
    GI_REQUIRE(top > 0 && top <= keep * (E / groups), "gi_router_select: %d of the %d experts that stay", top, keep * (E / groups));
    const size_t smem = (size_t)RS_WARPS * (2 * E + groups) * sizeof(float);
    GI_REQUIRE(smem <= 48 * 1024, "gi_router_select: %d experts do not fit shared memory", E);
    if (n_rows == 0) return 0;
    gi_launch(router_select_kernel, dim3((n_rows + RS_WARPS - 1) / RS_WARPS), dim3(RS_WARPS * 32), smem, (cudaStream_t)stream,
              logits, ld, E, top, groups, keep, scale, idx_out, w_out, n_rows, sigmoid_scores, correction, group_top,
              normalize);
    return gi_check_launch("gi_router_select");
}

// ------------------------------------------------------------------ one row times a chosen expert's matrix
// (dot_row below also serves the router's logits.)
template <typename T> __device__ __forceinline__ float dot_row(const T* __restrict__ w, const float* __restrict__ x, int k, int lane);
template <> __device__ __forceinline__ float dot_row<float>(const float* __restrict__ w, const float* __restrict__ x, int k, int lane) {
    float s = 0.f;
    if (k % 4 == 0 && (uintptr_t)w % 16 == 0) {
        for (int c = lane * 4; c < k; c += 128) {
            const float4 v = *reinterpret_cast<const float4*>(w + c), xv = *reinterpret_cast<const float4*>(x + c);
            s = fmaf(v.x, xv.x, s); s = fmaf(v.y, xv.y, s); s = fmaf(v.z, xv.z, s); s = fmaf(v.w, xv.w, s);
        }
    } else {
        for (int c = lane; c < k; c += 32) s = fmaf(w[c], x[c], s);
    }
    return warp_sum(s);
}
// Eight weights (one 16-byte word) times eight of the token's values, which come out of shared memory as two
// 16-byte words (eight 4-byte reads at a stride of 32 bytes would meet the same bank from every fourth lane).
__device__ __forceinline__ float fma8(const uint4& w, const float* __restrict__ x, float s) {
    const float4 x0 = *reinterpret_cast<const float4*>(x), x1 = *reinterpret_cast<const float4*>(x + 4);
    const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&w);
    float2 f = __bfloat1622float2(p2[0]);
    s = fmaf(f.x, x0.x, s); s = fmaf(f.y, x0.y, s);
    f = __bfloat1622float2(p2[1]);
    s = fmaf(f.x, x0.z, s); s = fmaf(f.y, x0.w, s);
    f = __bfloat1622float2(p2[2]);
    s = fmaf(f.x, x1.x, s); s = fmaf(f.y, x1.y, s);
    f = __bfloat1622float2(p2[3]);
    s = fmaf(f.x, x1.z, s); s = fmaf(f.y, x1.w, s);
    return s;
}
template <> __device__ __forceinline__ float dot_row<bf16>(const bf16* __restrict__ w, const float* __restrict__ x, int k, int lane) {
    float s = 0.f;
    if (k % 8 == 0 && (uintptr_t)w % 16 == 0) {
        // four 16-byte loads of a lane are asked for before any is used: the row is one stream of memory latencies
        int c = lane * 8;
        for (; c + 3 * 256 < k; c += 4 * 256) {
            uint4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) v[u] = *reinterpret_cast<const uint4*>(w + c + u * 256);
#pragma unroll
            for (int u = 0; u < 4; ++u) s = fma8(v[u], x + c + u * 256, s);
        }
        for (; c < k; c += 256) s = fma8(*reinterpret_cast<const uint4*>(w + c), x + c, s);
    } else {
        for (int c = lane; c < k; c += 32) s = fmaf(__bfloat162float(w[c]), x[c], s);
    }
    return warp_sum(s);
}

// Two rows of W against the same vector (a gate row and its up row): the vector's values are read once for both.
template <typename T>
__device__ __forceinline__ void dot_rows2(const T* __restrict__ w0, const T* __restrict__ w1, const float* __restrict__ x, int k,
                                          int lane, float& r0, float& r1) {
    r0 = dot_row<T>(w0, x, k, lane);
    r1 = dot_row<T>(w1, x, k, lane);
}
template <>
__device__ __forceinline__ void dot_rows2<bf16>(const bf16* __restrict__ w0, const bf16* __restrict__ w1,
                                                const float* __restrict__ x, int k, int lane, float& r0, float& r1) {
    if (!(k % 8 == 0 && (uintptr_t)w0 % 16 == 0 && (uintptr_t)w1 % 16 == 0)) {
        r0 = dot_row<bf16>(w0, x, k, lane);
        r1 = dot_row<bf16>(w1, x, k, lane);
        return;
    }
    float s0 = 0.f, s1 = 0.f;
    int c = lane * 8;
    for (; c + 3 * 256 < k; c += 4 * 256) {             // the same order of additions as dot_row's, row by row
        uint4 a[4], b[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            a[u] = *reinterpret_cast<const uint4*>(w0 + c + u * 256);
            b[u] = *reinterpret_cast<const uint4*>(w1 + c + u * 256);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            s0 = fma8(a[u], x + c + u * 256, s0);
            s1 = fma8(b[u], x + c + u * 256, s1);
        }
    }
    for (; c < k; c += 256) {
        s0 = fma8(*reinterpret_cast<const uint4*>(w0 + c), x + c, s0);
        s1 = fma8(*reinterpret_cast<const uint4*>(w1 + c), x + c, s1);
    }
    r0 = warp_sum(s0);
    r1 = warp_sum(s1);
}

// Router logits z[t, e] = sum_c w[e, c] x[t, c] in float32: the weight is float32, the token's vector is widened
// into shared memory, a warp per expert.  The weight (experts x hidden floats) stays in L2 over the launch.
template <typename T>
__global__ void __launch_bounds__(256)
router_logits_kernel(const T* __restrict__ x, long long ldx, const float* __restrict__ w, float* __restrict__ z,
                     int E, int hidden) {
    gi_pdl_start();
    extern __shared__ __align__(16) float xs[];
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) xs[c] = to_f32(x[(size_t)t * ldx + c]);
    __syncthreads();
    for (int e = blockIdx.y * 8 + warp; e < min(E, (int)(blockIdx.y + 1) * 8); e += 8) {
        const float v = dot_row<float>(w + (size_t)e * hidden, xs, hidden, lane);
        if (lane == 0) z[(size_t)t * E + e] = v;
    }
}

extern "C" int gi_router_logits(const void* x, long long ldx, int act_dtype, const float* w, float* z, int n_rows, int E,
                                int hidden, void* stream) {
    GI_REQUIRE(n_rows >= 0 && E > 0 && hidden > 0 && ldx >= hidden && (E + 7) / 8 <= 65535, "gi_router_logits: sizes");
    if (n_rows == 0) return 0;
    const size_t smem = (size_t)hidden * sizeof(float);
    dim3 grid(n_rows, (E + 7) / 8);
    cudaStream_t s = (cudaStream_t)stream;
    if (act_dtype == GI_DTYPE_F32) {
        if (smem > 48 * 1024) { int rc = gi_reserve_smem((const void*)router_logits_kernel<float>, smem, "gi_router_logits"); if (rc) return rc; }
        gi_launch(router_logits_kernel<float>, grid, dim3(256), smem, s, (const float*)x, ldx, w, z, E, hidden);
    } else if (act_dtype == GI_DTYPE_BF16) {
        if (smem > 48 * 1024) { int rc = gi_reserve_smem((const void*)router_logits_kernel<bf16>, smem, "gi_router_logits"); if (rc) return rc; }
        gi_launch(router_logits_kernel<bf16>, grid, dim3(256), smem, s, (const bf16*)x, ldx, w, z, E, hidden);
    } else {
        GI_REQUIRE(false, "gi_router_logits: activation dtype %d", act_dtype);
    }
    return gi_check_launch("gi_router_logits");
}

#define MOE_WARPS 8
#define MOE_ROWS 32          // rows of W per block, at most

// Rows of W per block: 32 when that still makes a couple of thousand blocks, else 16 or 8 (one row per warp), so that
// a step of one or two tokens still has enough loads in flight on every SM.
static int moe_rows_per_block(int pairs, int n_out) {
    for (int rows = MOE_ROWS; rows > MOE_WARPS; rows /= 2)
        if ((long long)pairs * ((n_out + rows - 1) / rows) >= 2048) return rows;
    return MOE_WARPS;
}

// x [n, ldx] (T), w_up [E, ff, hidden], idx [n, top] -> a [n, top, ff]
template <typename T>
__global__ void __launch_bounds__(MOE_WARPS * 32)
moe_up_kernel(const T* __restrict__ x, long long ldx, const T* __restrict__ w_up, const int* __restrict__ idx,
              T* __restrict__ a, int top, int E, int ff, int hidden, int act, int rows_pb, GluShape unit) {
    gi_pdl_start();
    extern __shared__ __align__(16) float xs[];                   // hidden
    const int tj = blockIdx.x, t = tj / top;
    const int e = idx[tj];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) xs[c] = to_f32(x[(size_t)t * ldx + c]);
    __syncthreads();
    const bool ok = e >= 0 && e < E;
    for (int f = blockIdx.y * rows_pb + warp; f < min(ff, (int)(blockIdx.y + 1) * rows_pb); f += MOE_WARPS) {
        float z;
        if (act == 2) {                             // a gated unit: ff gate rows, then ff up rows
            const T* we = w_up + (size_t)e * 2 * ff * hidden;
            float g = 0.f, u = 0.f;
            if (ok) dot_rows2<T>(we + (size_t)f * hidden, we + (size_t)(ff + f) * hidden, xs, hidden, lane, g, u);
            z = glu_unit(g, u, unit);
        } else {
            z = ok ? dot_row<T>(w_up + ((size_t)e * ff + f) * hidden, xs, hidden, lane) : 0.f;
            if (act == 0) { z = fmaxf(z, 0.f); z = z * z; } else { z = z / (1.f + expf(-z)); }
        }
        if (lane == 0) a[(size_t)tj * ff + f] = from_f32<T>(z);
    }
}

// a [n, top, ff] (T), w_down [E, hidden, ff], idx [n, top] -> part [n, top, hidden]: every (token, choice) pair's
// own result; gi_moe_combine sums a token's pairs with the router's weights.  A block stages one pair's vector.
template <typename T>
__global__ void __launch_bounds__(MOE_WARPS * 32)
moe_down_kernel(const T* __restrict__ a, const T* __restrict__ w_down, const int* __restrict__ idx,
                T* __restrict__ part, int E, int ff, int hidden, int rows_pb) {
    gi_pdl_start();
    extern __shared__ __align__(16) float as[];                   // ff
    const int tj = blockIdx.x;
    const int e = idx[tj];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int c = threadIdx.x; c < ff; c += blockDim.x) as[c] = to_f32(a[(size_t)tj * ff + c]);
    __syncthreads();
    const bool ok = e >= 0 && e < E;
    for (int c = blockIdx.y * rows_pb + warp; c < min(hidden, (int)(blockIdx.y + 1) * rows_pb); c += MOE_WARPS) {
        const float z = ok ? dot_row<T>(w_down + ((size_t)e * hidden + c) * ff, as, ff, lane) : 0.f;
        if (lane == 0) part[(size_t)tj * hidden + c] = from_f32<T>(z);
    }
}

extern "C" int gi_moe_up(const void* x, long long ldx, const void* w_up, const int* idx, void* a, int act_dtype, int n_rows,
                         int top, int E, int ff, int hidden, int act, int unit_kind, float alpha, float gate_max,
                         float up_limit, float up_shift, void* stream) {
    const GluShape unit = {unit_kind, alpha, gate_max, up_limit, up_shift};
    GI_REQUIRE(n_rows >= 0 && top > 0 && E > 0 && ff > 0 && hidden > 0 && ldx >= hidden, "gi_moe_up: sizes");
    GI_REQUIRE((ff + MOE_WARPS - 1) / MOE_WARPS <= 65535 && act >= 0 && act <= 2, "gi_moe_up: %d rows per expert, activation %d", ff, act);
    GI_REQUIRE(act != 2 || (unit_kind >= 0 && unit_kind <= 2 && up_limit >= 0.f), "gi_moe_up: gated unit %d", unit_kind);
    if (n_rows == 0) return 0;
    const size_t smem = (size_t)hidden * sizeof(float);
    const int rows_pb = moe_rows_per_block(n_rows * top, ff);
    dim3 grid(n_rows * top, (ff + rows_pb - 1) / rows_pb);
    cudaStream_t s = (cudaStream_t)stream;
    if (act_dtype == GI_DTYPE_F32) {
        if (smem > 48 * 1024) { int rc = gi_reserve_smem((const void*)moe_up_kernel<float>, smem, "gi_moe_up"); if (rc) return rc; }
        gi_launch(moe_up_kernel<float>, grid, dim3(MOE_WARPS * 32), smem, s, (const float*)x, ldx, (const float*)w_up, idx, (float*)a, top, E, ff, hidden, act, rows_pb, unit);
    } else if (act_dtype == GI_DTYPE_BF16) {
        if (smem > 48 * 1024) { int rc = gi_reserve_smem((const void*)moe_up_kernel<bf16>, smem, "gi_moe_up"); if (rc) return rc; }
        gi_launch(moe_up_kernel<bf16>, grid, dim3(MOE_WARPS * 32), smem, s, (const bf16*)x, ldx, (const bf16*)w_up, idx, (bf16*)a, top, E, ff, hidden, act, rows_pb, unit);
    } else {
        GI_REQUIRE(false, "gi_moe_up: activation dtype %d", act_dtype);
    }
    return gi_check_launch("gi_moe_up");
}

extern "C" int gi_moe_down(const void* a, const void* w_down, const int* idx, void* part, int act_dtype,
                           int n_rows, int top, int E, int ff, int hidden, void* stream) {
    GI_REQUIRE(n_rows >= 0 && top > 0 && E > 0 && ff > 0 && hidden > 0, "gi_moe_down: sizes");
    GI_REQUIRE((hidden + MOE_WARPS - 1) / MOE_WARPS <= 65535, "gi_moe_down: %d output channels", hidden);
    if (n_rows == 0) return 0;
    const size_t smem = (size_t)ff * sizeof(float);
    GI_REQUIRE(smem <= 200 * 1024, "gi_moe_down: an expert of %d does not fit shared memory", ff);
    const int rows_pb = moe_rows_per_block(n_rows * top, hidden);
    dim3 grid(n_rows * top, (hidden + rows_pb - 1) / rows_pb);
    cudaStream_t s = (cudaStream_t)stream;
    if (act_dtype == GI_DTYPE_F32) {
        if (smem > 48 * 1024) { int rc = gi_reserve_smem((const void*)moe_down_kernel<float>, smem, "gi_moe_down"); if (rc) return rc; }
        gi_launch(moe_down_kernel<float>, grid, dim3(MOE_WARPS * 32), smem, s, (const float*)a, (const float*)w_down, idx, (float*)part, E, ff, hidden, rows_pb);
    } else if (act_dtype == GI_DTYPE_BF16) {
        if (smem > 48 * 1024) { int rc = gi_reserve_smem((const void*)moe_down_kernel<bf16>, smem, "gi_moe_down"); if (rc) return rc; }
        gi_launch(moe_down_kernel<bf16>, grid, dim3(MOE_WARPS * 32), smem, s, (const bf16*)a, (const bf16*)w_down, idx, (bf16*)part, E, ff, hidden, rows_pb);
    } else {
        GI_REQUIRE(false, "gi_moe_down: activation dtype %d", act_dtype);
    }
    return gi_check_launch("gi_moe_down");
}

// ------------------------------------------------------------------ (token, choice) pairs in the order of their experts
// For the grouped products: pair p = t top + j goes to row where[p] of a matrix whose rows are sorted by expert, the
// pairs of one expert in the order of p (a counting sort, stable, so the layout does not depend on timing).
//   moe_count    every block counts its MOE_SEG pairs per expert
//   moe_offsets  one block: where each expert's rows end (`ends`), and where each block's pairs of each expert start
//   moe_place    a pair's row: its block's start for the expert + the pairs of that expert before it in the block
//   moe_gather   rows[where[p]] = x[p / top]
#define MOE_SEG 1024

__global__ void __launch_bounds__(MOE_SEG)
moe_count_kernel(const int* __restrict__ idx, int n_pairs, int E, int* __restrict__ block_counts) {
    gi_pdl_start();
    extern __shared__ int cnt[];                        // E
    for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    const int p = blockIdx.x * MOE_SEG + threadIdx.x;
    if (p < n_pairs) {
        const int e = idx[p];
        if (e >= 0 && e < E) atomicAdd(&cnt[e], 1);
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) block_counts[(size_t)blockIdx.x * E + e] = cnt[e];
}

// block_counts [n_blocks, E] become each block's first row for each expert; ends [E].
__global__ void moe_offsets_kernel(int* __restrict__ block_counts, int n_blocks, int E, int* __restrict__ ends) {
    gi_pdl_start();
    extern __shared__ int total[];                      // E totals, then E starts
    int* first = total + E;
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        int t = 0;
        for (int b = 0; b < n_blocks; ++b) t += block_counts[(size_t)b * E + e];
        total[e] = t;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < E; ++e) { first[e] = at; at += total[e]; ends[e] = at; }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        int at = first[e];
        for (int b = 0; b < n_blocks; ++b) {
            const int c = block_counts[(size_t)b * E + e];
            block_counts[(size_t)b * E + e] = at;
            at += c;
        }
    }
}

__global__ void __launch_bounds__(MOE_SEG)
moe_place_kernel(const int* __restrict__ idx, int n_pairs, int E, const int* __restrict__ block_first,
                 int* __restrict__ where) {
    gi_pdl_start();
    extern __shared__ int wc[];                         // [32 warps][E]: a warp's pairs per expert, then their prefix
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
    for (int i = threadIdx.x; i < n_warps * E; i += blockDim.x) wc[i] = 0;
    __syncthreads();
    const int p = blockIdx.x * MOE_SEG + threadIdx.x;
    int e = p < n_pairs ? idx[p] : -1;
    if (e < 0 || e >= E) e = -1;
    const unsigned same = __match_any_sync(0xffffffffu, e);
    const int rank = __popc(same & ((1u << lane) - 1u));
    if (e >= 0 && rank == 0) wc[warp * E + e] = __popc(same);
    __syncthreads();
    for (int x = threadIdx.x; x < E; x += blockDim.x) {             // exclusive prefix over the warps, per expert
        int at = 0;
        for (int w = 0; w < n_warps; ++w) { const int c = wc[w * E + x]; wc[w * E + x] = at; at += c; }
    }
    __syncthreads();
    if (e >= 0) where[p] = block_first[(size_t)blockIdx.x * E + e] + wc[warp * E + e] + rank;
    else if (p < n_pairs) where[p] = 0;
}

template <typename T>
__global__ void moe_gather_kernel(const T* __restrict__ x, long long ldx, const int* __restrict__ where, int top,
                                  T* __restrict__ rows, int hidden, int vec) {
    gi_pdl_start();
    const int p = blockIdx.x;
    const T* src = x + (size_t)(p / top) * ldx;
    T* dst = rows + (size_t)where[p] * hidden;
    if (vec) {
        const int n16 = hidden * (int)sizeof(T) / 16;
        for (int i = threadIdx.x; i < n16; i += blockDim.x)
            reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
    } else {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = src[i];
    }
}

// idx [n_rows, top] -> where [n_rows * top], ends [E], rows [n_rows * top, hidden] (x's rows in the experts' order).
// scratch: int32 [ceil(n_rows top / 1024) * E].
extern "C" int gi_moe_group(const int* idx, const void* x, long long ldx, int act_dtype, int* where, int* ends, void* rows,
                            int* scratch, int n_rows, int top, int E, int hidden, void* stream) {
    GI_REQUIRE(n_rows >= 0 && top > 0 && E > 0 && hidden > 0 && ldx >= hidden, "gi_moe_group: sizes");
    GI_REQUIRE(E <= 1024, "gi_moe_group: %d experts (at most 1024)", E);
    const long long n_pairs = (long long)n_rows * top;
    GI_REQUIRE(n_pairs < (1LL << 31), "gi_moe_group: %lld pairs", n_pairs);
    cudaStream_t s = (cudaStream_t)stream;
    if (n_rows == 0) return 0;
    const int n_blocks = (int)((n_pairs + MOE_SEG - 1) / MOE_SEG);
    gi_launch(moe_count_kernel, dim3(n_blocks), dim3(MOE_SEG), (size_t)E * sizeof(int), s, idx, (int)n_pairs, E, scratch);
    gi_launch(moe_offsets_kernel, dim3(1), dim3(256), (size_t)2 * E * sizeof(int), s, scratch, n_blocks, E, ends);
    const size_t place_smem = (size_t)(MOE_SEG / 32) * E * sizeof(int);
    if (place_smem > 48 * 1024) { int rc = gi_reserve_smem((const void*)moe_place_kernel, place_smem, "gi_moe_group"); if (rc) return rc; }
    gi_launch(moe_place_kernel, dim3(n_blocks), dim3(MOE_SEG), place_smem, s, idx, (int)n_pairs, E, (const int*)scratch, where);
    const int esz = act_dtype == GI_DTYPE_F32 ? 4 : 2;
    const int vec = ((long long)hidden * esz) % 16 == 0 && (ldx * esz) % 16 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)rows % 16 == 0;
    if (act_dtype == GI_DTYPE_F32)
        gi_launch(moe_gather_kernel<float>, dim3((unsigned)n_pairs), dim3(128), 0, s, (const float*)x, ldx, (const int*)where, top, (float*)rows, hidden, vec);
    else if (act_dtype == GI_DTYPE_BF16)
        gi_launch(moe_gather_kernel<bf16>, dim3((unsigned)n_pairs), dim3(128), 0, s, (const bf16*)x, ldx, (const int*)where, top, (bf16*)rows, hidden, vec);
    else
        GI_REQUIRE(false, "gi_moe_group: activation dtype %d", act_dtype);
    return gi_check_launch("gi_moe_group");
}

// ------------------------------------------------------------------ the weighted sum over rows written expert by expert
template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ buf, const int* __restrict__ where, const float* __restrict__ wt,
                                   T* __restrict__ y, int top, int hidden, const T* __restrict__ add) {
    gi_pdl_start();
    const size_t t = blockIdx.x;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < hidden; c += gridDim.y * blockDim.x) {
        float acc = add ? to_f32(add[t * hidden + c]) : 0.f;      // what every token gets besides (a shared expert)
        for (int j = 0; j < top; ++j)
            acc = fmaf(wt[t * top + j], to_f32(buf[(size_t)(where ? where[t * top + j] : (int)(t * top + j)) * hidden + c]), acc);
        y[t * hidden + c] = from_f32<T>(acc);
    }
}

extern "C" int gi_moe_combine(const void* buf, const int* where, const float* wt, void* y, int act_dtype, int n_rows,
                              int top, int hidden, const void* add, void* stream) {
    GI_REQUIRE(n_rows >= 0 && top > 0 && hidden > 0, "gi_moe_combine: sizes");
    if (n_rows == 0) return 0;
    dim3 grid(n_rows, (hidden + 1023) / 1024);
    cudaStream_t s = (cudaStream_t)stream;
    if (act_dtype == GI_DTYPE_F32)
        gi_launch(moe_combine_kernel<float>, grid, dim3(256), 0, s, (const float*)buf, where, wt, (float*)y, top, hidden, (const float*)add);
    else if (act_dtype == GI_DTYPE_BF16)
        gi_launch(moe_combine_kernel<bf16>, grid, dim3(256), 0, s, (const bf16*)buf, where, wt, (bf16*)y, top, hidden, (const bf16*)add);
    else
        GI_REQUIRE(false, "gi_moe_combine: activation dtype %d", act_dtype);
    return gi_check_launch("gi_moe_combine");
}
