// The two ends of an attention mixer whose keys and values have shapes of their own, around the attention
// kernel itself.
//
//   gi_attn_prepare   per token: rotate the first n_rot dimensions of every query and key head by position x
//                     frequency (pairs (2r, 2r+1), or (r, r + n_rot/2) in the half layout; the angle is the float32
//                     product and its cosine and sine are taken here, so no table limits the positions), write the
//                     queries as [n, query rows, d] and put the token's keys and values into its cache page.  The
//                     inputs are columns of one wider matrix (a packed projection, or the output of the short
//                     convolutions, which is float32 whatever the activation type is).  With n_rot = 0 nothing
//                     turns; with k_off < 0 the layer has no keys and values of its own (it reads another layer's)
//                     and only the queries are written.  Before the rotation, optionally: a bias per column (`bias`,
//                     laid out [queries | keys | values] like the columns themselves); an RMS norm of all query
//                     columns of the token at once and another of all its key columns, each with a weight per column
//                     (`norm_w`, [queries | keys]; x / sqrt(mean(x^2) + eps) * w); and a factor on the queries that
//                     grows with the position p, 1 + temp_coef ln(floor((p + 1) / temp_every) + 1).  All float32.
//   gi_attn_finish    per token and head: o = a_1 - lam a_2 for mixers with two softmax maps per head (lam one
//                     number on the device), o = a_1 otherwise; optionally o / sqrt(mean(o^2) + eps); times a
//                     constant; times sigmoid(gate logit of the head); rounded once into the activation type.
//
// Key pools are [pages, key heads, page_size, d], value pools [pages, value heads, page_size, dv].
// NikolayBlagoev/garlic-inference rotates by table and appends equal-shaped keys and values
// (src/src-cuda/rope.cu:41-79, src/src-cuda/kvcache.cu:61-84).
#include "common.cuh"
#include <math.h>

template <typename TI, typename T>
__global__ void attn_prepare_kernel(const TI* __restrict__ src, long long ld, int q_off, int k_off, int v_off,
                                    const float* __restrict__ freq, int n_rot, int half_layout,
                                    const int* __restrict__ tok_pos, const int* __restrict__ tok_slot,
                                    const int* __restrict__ block_table, T* __restrict__ k_pool, T* __restrict__ v_pool,
                                    T* __restrict__ q_out, int n_qh, int n_kh, int n_vh, int d, int dv, int page_size,
                                    int max_pages, int n_pool_pages, int append, int* __restrict__ status,
                                    const void* __restrict__ bias, int bias_dtype, const void* __restrict__ norm_w,
                                    int norm_dtype, float norm_eps, float temp_coef, int temp_every) {
    gi_pdl_start();
    extern __shared__ float cs[];                 // cos [n_rot/2], sin [n_rot/2]
    __shared__ float red[33];
    const int t = blockIdx.x;
    const int slot = tok_slot[t], pos = tok_pos[t];
    const TI* row = src + (size_t)t * ld;
    const int pairs = n_rot / 2;
    const int nq = n_qh * d, nk = k_off >= 0 ? n_kh * d : 0;
    // element i of the token's queries (i < nq) or keys (i - nq) as float32, with its bias
    auto raw = [&](int i) {
        const float x = to_f32(row[i < nq ? q_off + i : k_off + (i - nq)]);
        return bias ? x + load_w(bias, bias_dtype, i) : x;
    };
    float q_mul = 1.f, k_mul = 1.f;
    if (norm_w) {
        float sq = 0.f, sk = 0.f;
        for (int i = threadIdx.x; i < nq; i += blockDim.x) { const float x = raw(i); sq = fmaf(x, x, sq); }
        for (int i = nq + threadIdx.x; i < nq + nk; i += blockDim.x) { const float x = raw(i); sk = fmaf(x, x, sk); }
        sq = block_sum(sq, red);
        __syncthreads();
        sk = block_sum(sk, red);
        q_mul = 1.f / sqrtf(sq / (float)nq + norm_eps);
        if (nk) k_mul = 1.f / sqrtf(sk / (float)nk + norm_eps);
    }
    if (temp_every > 0) q_mul *= 1.f + temp_coef * logf((float)((max(pos, 0) + 1) / temp_every) + 1.f);
    // the same element as the attention reads it: normed, weighted, and (queries) times the position's factor
    auto val = [&](int i) {
        const float x = raw(i) * (i < nq ? q_mul : k_mul);
        return norm_w ? x * load_w(norm_w, norm_dtype, i) : x;
    };
    for (int r = threadIdx.x; r < pairs; r += blockDim.x) {
        float s, c;
        sincosf((float)pos * freq[r], &s, &c);
        cs[r] = c;
        cs[pairs + r] = s;
    }
    __syncthreads();
    // where this token's keys and values go
    long long page = -1;
    if (append && k_off >= 0 && slot >= 0) {
        if (pos < 0 || pos / page_size >= max_pages) {
            if (threadIdx.x == 0) atomicExch(status, 1);
        } else {
            page = block_table[(size_t)slot * max_pages + pos / page_size];
            if (page < 0 || page >= n_pool_pages) {
                if (threadIdx.x == 0) atomicExch(status, 2);
                page = -1;
            }
        }
    }
    const int in_page = pos >= 0 ? pos % page_size : 0;
    const int heads = n_qh + (k_off >= 0 ? n_kh : 0);
    // rotated pairs of the query and key heads
    for (int i = threadIdx.x; i < heads * pairs; i += blockDim.x) {
        const int h = i / pairs, r = i - h * pairs;
        const int a = half_layout ? r : 2 * r, b = half_layout ? r + pairs : 2 * r + 1;
        const bool is_q = h < n_qh;
        const float u = val(h * d + a), v = val(h * d + b);
        const float c = cs[r], s = cs[pairs + r];
        const float ua = u * c - v * s, vb = v * c + u * s;
        if (is_q) {
            T* o = q_out + ((size_t)t * n_qh + h) * d;
            o[a] = from_f32<T>(ua);
            o[b] = from_f32<T>(vb);
        } else if (page >= 0) {
            T* o = k_pool + ((page * n_kh + (h - n_qh)) * page_size + in_page) * d;
            o[a] = from_f32<T>(ua);
            o[b] = from_f32<T>(vb);
        }
    }
    // the dimensions that pass
    const int rest = d - n_rot;
    for (int i = threadIdx.x; i < heads * rest; i += blockDim.x) {
        const int h = i / rest, c = n_rot + (i - h * rest);
        const bool is_q = h < n_qh;
        const float x = val(h * d + c);
        if (is_q) q_out[((size_t)t * n_qh + h) * d + c] = from_f32<T>(x);
        else if (page >= 0) k_pool[((page * n_kh + (h - n_qh)) * page_size + in_page) * d + c] = from_f32<T>(x);
    }
    if (page >= 0) {
        for (int i = threadIdx.x; i < n_vh * dv; i += blockDim.x) {
            const int h = i / dv, c = i - h * dv;
            const float x = to_f32(row[v_off + i]);
            v_pool[((page * n_vh + h) * page_size + in_page) * dv + c] =
                from_f32<T>(bias ? x + load_w(bias, bias_dtype, nq + nk + i) : x);
        }
    }
}

extern "C" int gi_attn_prepare(const void* src, int src_dtype, long long ld, int q_off, int k_off, int v_off,
                               const float* freq, int n_rot, int half_layout, const int* tok_pos, const int* tok_slot,
                               const int* block_table, void* k_pool, void* v_pool, void* q_out, int act_dtype,
                               int n_tokens, int n_qh, int n_kh, int n_vh, int d, int dv, int page_size, int max_pages,
                               int n_pool_pages, int append, int* status, const void* bias, int bias_dtype,
                               const void* norm_w, int norm_dtype, float norm_eps, float temp_coef, int temp_every,
                               void* stream) {
    GI_REQUIRE(n_tokens >= 0 && n_qh > 0 && d > 0 && dv > 0, "gi_attn_prepare: sizes must be positive");
    GI_REQUIRE(temp_every >= 0 && (!norm_w || norm_eps > 0.f), "gi_attn_prepare: the queries' factor and the norm's eps");
    GI_REQUIRE(n_rot >= 0 && n_rot % 2 == 0 && n_rot <= d, "gi_attn_prepare: %d rotated dimensions of heads of %d", n_rot, d);
    GI_REQUIRE(k_off < 0 || (n_kh > 0 && n_vh > 0 && page_size > 0 && max_pages > 0), "gi_attn_prepare: key/value sizes");
    if (n_tokens == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem = (size_t)n_rot * sizeof(float);
    const int work = (n_qh + (k_off >= 0 ? n_kh : 0)) * d;
    const int threads = work >= 2048 ? 256 : 128;
#define AP_LAUNCH(TI, T)                                                                                             \
    gi_launch(attn_prepare_kernel<TI, T>, dim3(n_tokens), dim3(threads), smem, s, (const TI*)src, ld, q_off, k_off,   \
              v_off, freq, n_rot, half_layout, tok_pos, tok_slot, block_table, (T*)k_pool, (T*)v_pool, (T*)q_out,     \
              n_qh, n_kh, n_vh, d, dv, page_size, max_pages, n_pool_pages, append, status, bias, bias_dtype, norm_w,     \
              norm_dtype, norm_eps, temp_coef, temp_every)
    if (src_dtype == GI_DTYPE_F32 && act_dtype == GI_DTYPE_F32) AP_LAUNCH(float, float);
    else if (src_dtype == GI_DTYPE_F32 && act_dtype == GI_DTYPE_BF16) AP_LAUNCH(float, bf16);
    else if (src_dtype == GI_DTYPE_BF16 && act_dtype == GI_DTYPE_BF16) AP_LAUNCH(bf16, bf16);
    else GI_REQUIRE(false, "gi_attn_prepare: source dtype %d with activation dtype %d", src_dtype, act_dtype);
#undef AP_LAUNCH
    return gi_check_launch("gi_attn_prepare");
}

// att float32 [n, heads * maps, dv] (a head's maps side by side); gate: logit of head h at gate[r * ldg + h];
// out [n, ld_out] gets the head's dv values at column h * dv.
template <typename TA, typename T>
__global__ void attn_finish_kernel(const TA* __restrict__ att, int maps, const float* __restrict__ lam, float eps,
                                   int norm, float mul, const T* __restrict__ gate, long long ldg,
                                   T* __restrict__ out, long long ld_out, int heads, int dv) {
    gi_pdl_start();
    __shared__ float red[33];
    const size_t r = blockIdx.x;
    const int h = blockIdx.y;
    const TA* a1 = att + (r * heads + h) * (size_t)maps * dv;
    const float l = maps > 1 ? lam[0] : 0.f;
    float g = 1.f;
    if (gate) g = 1.f / (1.f + expf(-to_f32(gate[r * ldg + h])));
    float ss = 0.f;
    for (int c = threadIdx.x; c < dv; c += blockDim.x) {
        const float o = maps > 1 ? to_f32(a1[c]) - l * to_f32(a1[dv + c]) : to_f32(a1[c]);
        ss += o * o;
    }
    float inv = 1.f;
    if (norm) {
        ss = block_sum(ss, red);
        inv = 1.f / sqrtf(ss / (float)dv + eps);
    }
    for (int c = threadIdx.x; c < dv; c += blockDim.x) {
        const float o = maps > 1 ? to_f32(a1[c]) - l * to_f32(a1[dv + c]) : to_f32(a1[c]);
        out[r * ld_out + (size_t)h * dv + c] = from_f32<T>(o * inv * mul * g);
    }
}

extern "C" int gi_attn_finish(const void* att, int att_dtype, int maps, const float* lam, float eps, int norm, float mul,
                              const void* gate, long long ldg, void* out, long long ld_out, int act_dtype, int n_rows,
                              int heads, int dv, void* stream) {
    GI_REQUIRE(n_rows >= 0 && heads > 0 && heads <= 65535 && dv > 0 && (maps == 1 || maps == 2),
               "gi_attn_finish: %d heads of %d values in %d maps", heads, dv, maps);
    GI_REQUIRE(maps == 1 || lam, "gi_attn_finish: two maps need their factor");
    GI_REQUIRE(ld_out >= (long long)heads * dv, "gi_attn_finish: output rows shorter than the heads");
    if (n_rows == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = dv > 128 ? 128 : (dv > 64 ? 64 : 32);
    dim3 grid(n_rows, heads);
    if (att_dtype == GI_DTYPE_F32 && act_dtype == GI_DTYPE_F32)
        gi_launch(attn_finish_kernel<float, float>, grid, dim3(threads), 0, s, (const float*)att, maps, lam, eps, norm, mul,
                  (const float*)gate, ldg, (float*)out, ld_out, heads, dv);
    else if (att_dtype == GI_DTYPE_F32 && act_dtype == GI_DTYPE_BF16)
        gi_launch(attn_finish_kernel<float, bf16>, grid, dim3(threads), 0, s, (const float*)att, maps, lam, eps, norm, mul,
                  (const bf16*)gate, ldg, (bf16*)out, ld_out, heads, dv);
    else if (att_dtype == GI_DTYPE_BF16 && act_dtype == GI_DTYPE_BF16)
        gi_launch(attn_finish_kernel<bf16, bf16>, grid, dim3(threads), 0, s, (const bf16*)att, maps, lam, eps, norm, mul,
                  (const bf16*)gate, ldg, (bf16*)out, ld_out, heads, dv);
    else
        GI_REQUIRE(false, "gi_attn_finish: attention dtype %d with activation dtype %d", att_dtype, act_dtype);
    return gi_check_launch("gi_attn_finish");
}
