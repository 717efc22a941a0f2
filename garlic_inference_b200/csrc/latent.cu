// Latent attention, the step between the projections and the attention kernel: the new token's latent row
// goes into the paged cache and the queries are put into the form the attention kernel reads.
//
// A token's cache row is [ c (kv_rank) | rotated shared key part (rot_dim) | zeros up to the row's width ],
// c = rmsnorm(first kv_rank columns of the down-projection) * w.  Every head's key is W_uk,h c beside the
// shared rotated part and its value is W_uv,h c, so with q'_h = W_uk,h^T q_h (made by a per-head product
// before this kernel) the score is  q'_h . c + rot(q_rot,h) . rot(k_rot),  attention over the cache rows
// themselves gives sum_j p_j c_j, and W_uv,h is applied to that afterwards: the cache is read once for all
// heads and keys and values are never expanded.
//
// Rotation: pair (2i, 2i+1) of the rotated part (or, in the half layout, pair (i, i + n_rot/2)), i < n_rot / 2,
// turns by the float32 product position * freq[i]; cosine and sine are multiplied by `magnitude`; dimensions from
// n_rot on pass.  The queries may come from a matrix of their own (an up-projection behind a normed latent), and a
// layer that reads another layer's cache rows brings no latent to append (kv_src = null).
// NikolayBlagoev/garlic-inference has one attention (grouped-query, src/models/qwen3/qwen3.cpp:140-179) and
// the rotate-half layout (src/src-cuda/rope.cu:41-79).
#include "common.cuh"
#include <math.h>

// Element j < n_rot of a rotated part `x` after the turn (cs, sn: the pairs' cosines and sines).
template <typename T>
__device__ __forceinline__ float turned(const T* x, int j, int n_rot, int half, const float* cs, const float* sn) {
    if (half) {
        const int h = n_rot >> 1;
        return j < h ? to_f32(x[j]) * cs[j] - to_f32(x[j + h]) * sn[j]
                     : to_f32(x[j]) * cs[j - h] + to_f32(x[j - h]) * sn[j - h];
    }
    const float a = to_f32(x[j & ~1]), b = to_f32(x[j | 1]);
    return (j & 1) ? b * cs[j >> 1] + a * sn[j >> 1] : a * cs[j >> 1] - b * sn[j >> 1];
}

template <typename T>
__global__ void latent_prepare_kernel(const T* __restrict__ q_src, long long ldq, int q_off,
                                      const T* __restrict__ kv_src, long long ld, int c_off, int half,
                                      const T* __restrict__ q_lat, const void* __restrict__ norm_w, int w_dtype,
                                      float eps, const float* __restrict__ freq, float magnitude, int n_rot,
                                      const int* __restrict__ tok_pos, const int* __restrict__ tok_slot,
                                      const int* __restrict__ block_table, T* __restrict__ pool,
                                      T* __restrict__ q_out, int H, int d, int dr, int rank, int row_w,
                                      int page_size, int max_pages, int n_pool_pages, int append,
                                      int* __restrict__ status) {
    gi_pdl_start();
    __shared__ float red[33];
    __shared__ float cs_s[128], sn_s[128];             // cosine and sine of the token's angles, pairs 0 .. n_rot/2 - 1
    const int t = blockIdx.x, part = blockIdx.y;       // part < H: that head's query row; part == H: the cache row
    const int pos = tok_pos[t], slot = tok_slot[t];
    const float p = (float)pos;
    for (int i = threadIdx.x; i < n_rot / 2; i += blockDim.x) {
        float sn, cs;
        sincosf(p * freq[i], &sn, &cs);
        cs_s[i] = cs * magnitude; sn_s[i] = sn * magnitude;
    }
    __syncthreads();

    if (part < H) {                                    // queries: [ q' (rank) | rotated part (dr) | zeros ]
        const int h = part;
        const T* qr = q_src + (size_t)t * ldq + q_off + (size_t)h * (d + dr) + d;
        const T* ql = q_lat + ((size_t)t * H + h) * rank;
        T* dst = q_out + ((size_t)t * H + h) * row_w;
#pragma unroll 4
        for (int c = threadIdx.x; c < row_w; c += blockDim.x) {
            float v = 0.f;
            if (c < rank) {
                v = to_f32(ql[c]);
            } else if (c < rank + dr) {
                const int j = c - rank;
                v = j < n_rot ? turned(qr, j, n_rot, half, cs_s, sn_s) : to_f32(qr[j]);
            }
            dst[c] = from_f32<T>(v);
        }
        return;
    }
    if (!append || slot < 0 || !kv_src) return;
    const int lp = pos / page_size;
    if (pos < 0 || lp >= max_pages) { if (threadIdx.x == 0) atomicExch(status, 1); return; }
    const int page = block_table[(size_t)slot * max_pages + lp];
    if (page < 0 || page >= n_pool_pages) { if (threadIdx.x == 0) atomicExch(status, 2); return; }
    T* dst = pool + ((size_t)page * page_size + (pos - lp * page_size)) * row_w;

    const T* cr = kv_src + (size_t)t * ld + c_off;
    float ss = 0.f;
#pragma unroll 4
    for (int c = threadIdx.x; c < rank; c += blockDim.x) { const float x = to_f32(cr[c]); ss += x * x; }
    ss = block_sum(ss, red);
    const float inv = 1.f / sqrtf(ss / (float)rank + eps);
#pragma unroll 4
    for (int c = threadIdx.x; c < row_w; c += blockDim.x) {
        float v = 0.f;
        if (c < rank) {
            v = to_f32(cr[c]) * inv * load_w(norm_w, w_dtype, c);
        } else if (c < rank + dr) {
            const int j = c - rank;
            const T* kr = cr + rank;
            v = j < n_rot ? turned(kr, j, n_rot, half, cs_s, sn_s) : to_f32(kr[j]);
        }
        dst[c] = from_f32<T>(v);
    }
}

extern "C" int gi_latent_prepare(const void* q_src, long long ldq, int q_off, const void* kv_src, long long ld, int c_off,
                                 int half, const void* q_lat,
                                 int act_dtype, const void* norm_w, int w_dtype, float eps, const float* freq,
                                 float magnitude, int n_rot, const int* tok_pos, const int* tok_slot,
                                 const int* block_table, void* pool, void* q_out, int n_tokens, int H, int d, int dr,
                                 int rank, int row_w, int page_size, int max_pages, int n_pool_pages, int append,
                                 int* status, void* stream) {
    GI_REQUIRE(n_tokens >= 0 && H > 0 && d > 0 && dr >= 0 && rank > 0, "gi_latent_prepare: sizes must be positive");
    GI_REQUIRE(row_w >= rank + dr, "gi_latent_prepare: cache rows of %d hold no latent of %d and key part of %d",
               row_w, rank, dr);
    GI_REQUIRE(n_rot % 2 == 0 && n_rot <= dr && n_rot <= 256, "gi_latent_prepare: %d rotated dimensions of %d (at most 256)", n_rot, dr);
    GI_REQUIRE(H < 65535, "gi_latent_prepare: %d heads", H);
    GI_REQUIRE(kv_src || !append, "gi_latent_prepare: nothing to append without a latent of the layer's own");
    if (n_tokens == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (act_dtype == GI_DTYPE_F32)
        gi_launch(latent_prepare_kernel<float>, dim3(n_tokens, H + 1), dim3(128), 0, s, (const float*)q_src, ldq, q_off,
                  (const float*)kv_src, ld, c_off, half, (const float*)q_lat, norm_w, w_dtype, eps, freq, magnitude, n_rot, tok_pos, tok_slot, block_table,
                  (float*)pool, (float*)q_out, H, d, dr, rank, row_w, page_size, max_pages, n_pool_pages, append, status);
    else if (act_dtype == GI_DTYPE_BF16)
        gi_launch(latent_prepare_kernel<bf16>, dim3(n_tokens, H + 1), dim3(128), 0, s, (const bf16*)q_src, ldq, q_off,
                  (const bf16*)kv_src, ld, c_off, half, (const bf16*)q_lat, norm_w, w_dtype, eps, freq, magnitude, n_rot, tok_pos, tok_slot, block_table,
                  (bf16*)pool, (bf16*)q_out, H, d, dr, rank, row_w, page_size, max_pages, n_pool_pages, append, status);
    else
        GI_REQUIRE(false, "gi_latent_prepare: activation dtype %d", act_dtype);
    return gi_check_launch("gi_latent_prepare");
}

// ------------------------------------------------------------------ attention of single tokens over the latent rows
// Decode steps in bfloat16: one new token per sequence, all heads of a sequence read the same cached rows.  A
// block takes one token, up to 8 * HPW heads and one slice of the keys; it stages 32 rows at a time in shared
// memory, where every head's scores and weighted sums read them (the exact-order kernel fetches them once per
// head).  Warp w owns heads w HPW .. w HPW + HPW - 1 of the block's group for all keys of the slice, so the
// running maximum and sum stay inside the warp; lane j scores key j of the 32, then the lanes turn to pairs of
// value columns.  Scores, softmax and sums are float32.  The slices' (max, sum, weighted rows) go to `part`
// [tokens, slices, heads, 2 + rank] and gi_latent_decode_combine merges them with the sink.
#define LD_WARPS 8
#define LD_KEYS 32

__device__ __forceinline__ float2 bf2_to_f2(uint32_t w) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w));
}

template <int HPW, int DPL2>
__global__ void __launch_bounds__(LD_WARPS * 32)
latent_decode_kernel(const bf16* __restrict__ q, const bf16* __restrict__ pool, const int* __restrict__ block_table,
                     const int* __restrict__ tok_pos, const int* __restrict__ tok_slot, float* __restrict__ part,
                     int H, int dk, int rank, int page_size, int max_pages, int n_pool_pages, int n_splits,
                     float scale, int* __restrict__ status) {
    gi_pdl_start();
    extern __shared__ __align__(16) unsigned char ld_smem[];
    constexpr int HG = HPW * LD_WARPS;
    float* q_s = reinterpret_cast<float*>(ld_smem);                  // HG rows of dk
    uint32_t* k_s = reinterpret_cast<uint32_t*>(q_s + HG * dk);      // 32 rows of kw words (kw odd: no bank conflicts)
    const int kw = dk / 2 + 1;
    const int t = blockIdx.x, split = blockIdx.y, h0 = blockIdx.z * HG;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int slot = tok_slot[t], pos = tok_pos[t];
    const size_t stride = (size_t)rank + 2;
    float* my = part + ((size_t)t * n_splits + split) * H * stride;
    const bool dead = slot < 0 || pos < 0 || pos / page_size >= max_pages;
    const int n_chunks = dead ? 0 : pos / LD_KEYS + 1;
    const int per = (n_chunks + n_splits - 1) / n_splits;
    const int c0 = split * per, c1 = min(n_chunks, c0 + per);
    if (dead && slot >= 0 && threadIdx.x == 0) atomicExch(status, 4);

    if (c0 < c1)
        for (int i = threadIdx.x; i < HG * dk; i += blockDim.x) {
            const int hh = i / dk, c = i - hh * dk;
            q_s[i] = h0 + hh < H ? to_f32(q[((size_t)t * H + h0 + hh) * dk + c]) * scale : 0.f;
        }
    float m[HPW], l[HPW], p[HPW], acc[HPW][2 * DPL2];
#pragma unroll
    for (int hh = 0; hh < HPW; ++hh) {
        m[hh] = -INFINITY; l[hh] = 0.f;
#pragma unroll
        for (int r = 0; r < 2 * DPL2; ++r) acc[hh][r] = 0.f;
    }
    const int* bt = block_table + (size_t)(dead ? 0 : slot) * max_pages;
    const int vec_per_row = dk / 8;
    for (int c = c0; c < c1; ++c) {
        __syncthreads();
        for (int idx = threadIdx.x; idx < LD_KEYS * vec_per_row; idx += blockDim.x) {
            const int j = idx / vec_per_row, v = idx - j * vec_per_row;
            const int key = c * LD_KEYS + j;
            uint4 val = make_uint4(0u, 0u, 0u, 0u);
            if (key <= pos) {
                const int page = bt[key / page_size];
                if (page < 0 || page >= n_pool_pages) atomicExch(status, 5);
                else val = *reinterpret_cast<const uint4*>(pool + ((size_t)page * page_size + key % page_size) * dk + v * 8);
            }
            uint32_t* dst = k_s + j * kw + v * 4;
            dst[0] = val.x; dst[1] = val.y; dst[2] = val.z; dst[3] = val.w;
        }
        __syncthreads();
        const bool valid = c * LD_KEYS + lane <= pos;
        float s[HPW];
#pragma unroll
        for (int hh = 0; hh < HPW; ++hh) s[hh] = 0.f;
        const uint32_t* kr = k_s + lane * kw;
        const float* qw = q_s + (size_t)warp * HPW * dk;
        for (int i2 = 0; i2 < dk / 2; ++i2) {
            const float2 kf = bf2_to_f2(kr[i2]);
#pragma unroll
            for (int hh = 0; hh < HPW; ++hh) {
                const float2 qf = *reinterpret_cast<const float2*>(qw + hh * dk + 2 * i2);
                s[hh] = fmaf(kf.x, qf.x, s[hh]);
                s[hh] = fmaf(kf.y, qf.y, s[hh]);
            }
        }
#pragma unroll
        for (int hh = 0; hh < HPW; ++hh) {
            const float sv = valid ? s[hh] : -INFINITY;
            const float m_new = fmaxf(m[hh], warp_max(sv));          // the chunk's first key is always seen
            const float corr = expf(m[hh] - m_new);
            p[hh] = valid ? expf(sv - m_new) : 0.f;
            l[hh] = l[hh] * corr + warp_sum(p[hh]);
            m[hh] = m_new;
#pragma unroll
            for (int r = 0; r < 2 * DPL2; ++r) acc[hh][r] *= corr;
        }
        for (int j = 0; j < LD_KEYS; ++j) {
            float pj[HPW];
#pragma unroll
            for (int hh = 0; hh < HPW; ++hh) pj[hh] = __shfl_sync(0xffffffffu, p[hh], j);
#pragma unroll
            for (int r = 0; r < DPL2; ++r) {
                const int col2 = lane + 32 * r;
                if (2 * col2 < rank) {
                    const float2 vf = bf2_to_f2(k_s[j * kw + col2]);
#pragma unroll
                    for (int hh = 0; hh < HPW; ++hh) {
                        acc[hh][2 * r] = fmaf(pj[hh], vf.x, acc[hh][2 * r]);
                        acc[hh][2 * r + 1] = fmaf(pj[hh], vf.y, acc[hh][2 * r + 1]);
                    }
                }
            }
        }
    }
#pragma unroll
    for (int hh = 0; hh < HPW; ++hh) {
        const int h = h0 + warp * HPW + hh;
        if (h >= H) continue;
        float* o = my + (size_t)h * stride;
        if (lane == 0) { o[0] = m[hh]; o[1] = l[hh]; }
#pragma unroll
        for (int r = 0; r < DPL2; ++r) {
            const int col = 2 * (lane + 32 * r);
            if (col < rank) o[2 + col] = acc[hh][2 * r];
            if (col + 1 < rank) o[2 + col + 1] = acc[hh][2 * r + 1];
        }
    }
}

// The same block on tensor cores (mma.sync m16n8k16, bfloat16 operands, float32 accumulation).  A block takes
// 32 heads: the scores of a chunk, 32 heads x 32 keys, are 2 x 4 tiles, one per warp, summed over the row's
// width in steps of 16; they go through shared memory as float32 to the softmax (warp w owns heads 4w .. 4w+3,
// as above: maximum, sum and weights float32); the weights, rounded to bfloat16 as the second product's
// operand, times the staged rows' first `rank` columns are 2 x ceil(rank / 8) tiles, NTW column tiles per
// warp, with the rows read as the product's second operand by ldmatrix.trans.  Shared-memory rows are padded
// to 4 words past a multiple of 32 so that the fragments' loads meet no bank twice.
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int NTW>
__global__ void __launch_bounds__(LD_WARPS * 32)
latent_decode_mma_kernel(const bf16* __restrict__ q, const bf16* __restrict__ pool, const int* __restrict__ block_table,
                         const int* __restrict__ tok_pos, const int* __restrict__ tok_slot, float* __restrict__ part,
                         int H, int dk, int rank, int row_words, int page_size, int max_pages, int n_pool_pages,
                         int n_splits, float scale, int* __restrict__ status) {
    gi_pdl_start();
    extern __shared__ __align__(16) unsigned char ld_smem[];
    constexpr int HG = 32, PW = 20;                                  // heads per block; words per row of weights
    const int kw = row_words;                                        // words per staged row, kw % 32 == 4
    uint32_t* q_b = reinterpret_cast<uint32_t*>(ld_smem);            // HG rows of kw words (bfloat16 pairs)
    uint32_t* k_bufs = q_b + HG * kw;                                // twice 32 rows of kw words: one chunk is walked
                                                                     // while the next one's copies are in flight
    float* s_s = reinterpret_cast<float*>(k_bufs + 2 * LD_KEYS * kw);   // HG x 33 scores
    uint32_t* p_s = reinterpret_cast<uint32_t*>(s_s + HG * 33);      // HG rows of PW words: the weights
    float* corr_s = reinterpret_cast<float*>(p_s + HG * PW);         // HG
    const int t = blockIdx.x, split = blockIdx.y, h0 = blockIdx.z * HG;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, tq = lane & 3;                          // the fragments' row group and column pair
    const int slot = tok_slot[t], pos = tok_pos[t];
    const size_t stride = (size_t)rank + 2;
    float* my = part + ((size_t)t * n_splits + split) * H * stride;
    const bool dead = slot < 0 || pos < 0 || pos / page_size >= max_pages;
    const int n_chunks = dead ? 0 : pos / LD_KEYS + 1;
    const int per = (n_chunks + n_splits - 1) / n_splits;
    const int c0 = split * per, c1 = min(n_chunks, c0 + per);
    if (dead && slot >= 0 && threadIdx.x == 0) atomicExch(status, 4);
    const int vec_per_row = dk / 8, words = dk / 2;

    if (c0 < c1)
        for (int idx = threadIdx.x; idx < HG * (kw / 4); idx += blockDim.x) {
            const int hh = idx / (kw / 4), v = idx - hh * (kw / 4);
            uint4 val = make_uint4(0u, 0u, 0u, 0u);
            if (h0 + hh < H && v < vec_per_row)
                val = *reinterpret_cast<const uint4*>(q + ((size_t)t * H + h0 + hh) * dk + v * 8);
            *reinterpret_cast<uint4*>(q_b + hh * kw + v * 4) = val;
        }
    float m[4], l[4];
#pragma unroll
    for (int hh = 0; hh < 4; ++hh) { m[hh] = -INFINITY; l[hh] = 0.f; }
    float acc[2][NTW][4];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int j = 0; j < NTW; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[mt][j][e] = 0.f;
    const int* bt = block_table + (size_t)(dead ? 0 : slot) * max_pages;
    const int k_steps = (words + 7) / 8;                              // steps of 16 values; the rows' padding is zero
    const int mt_s = warp & 1, nt_s = warp >> 1;                      // this warp's tile of the scores
    const int n_tiles = (rank + 7) / 8;
    const uint32_t k_bufs_addr = (uint32_t)__cvta_generic_to_shared(k_bufs);
    // Asynchronous 16-byte copies of a chunk's rows into buffer `buf`; keys beyond the position, unmapped pages and
    // the rows' padding are filled with zeros (a copy of 0 source bytes).
    auto stage = [&](int c, int buf) {
        for (int idx = threadIdx.x; idx < LD_KEYS * (kw / 4); idx += blockDim.x) {
            const int j = idx / (kw / 4), v = idx - j * (kw / 4);
            const int key = c * LD_KEYS + j;
            const bf16* src = pool;
            int bytes = 0;
            if (key <= pos && v < vec_per_row) {
                const int page = bt[key / page_size];
                if (page < 0 || page >= n_pool_pages) atomicExch(status, 5);
                else { src = pool + ((size_t)page * page_size + key % page_size) * dk + v * 8; bytes = 16; }
            }
            const uint32_t dst = k_bufs_addr + ((buf * LD_KEYS + j) * kw + v * 4) * 4;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"(dst), "l"(src), "r"(bytes) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (c0 < c1) stage(c0, 0);

    for (int c = c0; c < c1; ++c) {
        const int buf = (c - c0) & 1;
        const uint32_t* k_s = k_bufs + buf * LD_KEYS * kw;
        const uint32_t k_s_addr = k_bufs_addr + buf * LD_KEYS * kw * 4;
        __syncthreads();                                              // the last chunk's rows and weights are done with
        if (c + 1 < c1) {
            stage(c + 1, buf ^ 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        // scores: tile (mt_s, nt_s) = heads 16 mt_s .. +15 x keys 8 nt_s .. +7
        {
            float sc[4] = {0.f, 0.f, 0.f, 0.f};
            const uint32_t* qa = q_b + (16 * mt_s + g) * kw + tq;
            const uint32_t* kb = k_s + (8 * nt_s + g) * kw + tq;
            for (int ks = 0; ks < k_steps; ++ks) {
                const uint32_t a[4] = {qa[8 * ks], qa[8 * kw + 8 * ks], qa[8 * ks + 4], qa[8 * kw + 8 * ks + 4]};
                mma_bf16_16816(sc, a, kb[8 * ks], kb[8 * ks + 4]);
            }
            float* srow = s_s + (16 * mt_s + g) * 33 + 8 * nt_s + 2 * tq;
            srow[0] = sc[0] * scale; srow[1] = sc[1] * scale;
            srow[8 * 33] = sc[2] * scale; srow[8 * 33 + 1] = sc[3] * scale;
        }
        __syncthreads();
        // softmax of the chunk: warp w owns heads 4 w .. 4 w + 3, lane j is key j
        {
            const bool valid = c * LD_KEYS + lane <= pos;
#pragma unroll
            for (int hh = 0; hh < 4; ++hh) {
                const int h = 4 * warp + hh;
                const float sv = valid ? s_s[h * 33 + lane] : -INFINITY;
                const float m_new = fmaxf(m[hh], warp_max(sv));       // the chunk's first key is always seen
                const float corr = expf(m[hh] - m_new);
                const bf16 pr = __float2bfloat16_rn(valid ? expf(sv - m_new) : 0.f);
                l[hh] = l[hh] * corr + warp_sum(__bfloat162float(pr));
                m[hh] = m_new;
                reinterpret_cast<bf16*>(p_s + h * PW)[lane] = pr;
                if (lane == 0) corr_s[h] = corr;
            }
        }
        __syncthreads();
        // weighted rows: this warp's NTW column tiles for both halves of the heads
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
            const float ca = corr_s[16 * mt + g], cb = corr_s[16 * mt + g + 8];
#pragma unroll
            for (int j = 0; j < NTW; ++j) { acc[mt][j][0] *= ca; acc[mt][j][1] *= ca; acc[mt][j][2] *= cb; acc[mt][j][3] *= cb; }
        }
#pragma unroll
        for (int ks = 0; ks < 2; ++ks) {
            uint32_t a[2][4];
#pragma unroll
            for (int mt = 0; mt < 2; ++mt) {
                const uint32_t* pa = p_s + (16 * mt + g) * PW + 8 * ks + tq;
                a[mt][0] = pa[0]; a[mt][1] = pa[8 * PW]; a[mt][2] = pa[4]; a[mt][3] = pa[8 * PW + 4];
            }
#pragma unroll
            for (int j = 0; j < NTW; ++j) {
                const int nt = warp * NTW + j;
                if (nt >= n_tiles) continue;                          // uniform over the warp
                uint32_t b0, b1;
                const uint32_t addr = k_s_addr + ((16 * ks + (lane & 15)) * kw + 4 * nt) * 4;
                asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(b0), "=r"(b1) : "r"(addr));
                mma_bf16_16816(acc[0][j], a[0], b0, b1);
                mma_bf16_16816(acc[1][j], a[1], b0, b1);
            }
        }
    }
    // this slice's (max, sum) of the heads this warp owned in the softmax, and its columns of every head
#pragma unroll
    for (int hh = 0; hh < 4; ++hh) {
        const int h = h0 + 4 * warp + hh;
        if (h < H && lane == 0) { my[(size_t)h * stride] = m[hh]; my[(size_t)h * stride + 1] = l[hh]; }
    }
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int j = 0; j < NTW; ++j) {
            const int col = 8 * (warp * NTW + j) + 2 * tq;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int h = h0 + 16 * mt + g + (e >> 1) * 8, cc = col + (e & 1);
                if (h < H && cc < rank) my[(size_t)h * stride + 2 + cc] = acc[mt][j][e];
            }
        }
}

__global__ void latent_decode_combine_kernel(const float* __restrict__ part, bf16* __restrict__ out, int H, int rank,
                                             int n_splits, const void* __restrict__ sinks, int sink_dtype) {
    gi_pdl_start();
    const int t = blockIdx.x, h = blockIdx.y;
    const size_t stride = (size_t)rank + 2;
    const float* base = part + ((size_t)t * n_splits * H + h) * stride;
    const size_t step = (size_t)H * stride;
    const float sink = sinks ? load_w(sinks, sink_dtype, h) : -INFINITY;
    float M = sink;
    for (int s = 0; s < n_splits; ++s) M = fmaxf(M, base[s * step]);
    float L = sinks ? expf(sink - M) : 0.f;
    for (int s = 0; s < n_splits; ++s) {
        const float ms = base[s * step];
        if (ms != -INFINITY) L += expf(ms - M) * base[s * step + 1];
    }
    for (int c = threadIdx.x; c < rank; c += blockDim.x) {
        float v = 0.f;
        for (int s = 0; s < n_splits; ++s) {
            const float ms = base[s * step];
            if (ms != -INFINITY) v += expf(ms - M) * base[s * step + 2 + c];
        }
        out[((size_t)t * H + h) * rank + c] = __float2bfloat16_rn(L > 0.f ? v / L : 0.f);
    }
}

extern "C" int gi_latent_decode(const void* q, const void* pool, const int* block_table, const int* tok_pos,
                                const int* tok_slot, float* part, void* out, int n_tokens, int H, int dk, int rank,
                                int page_size, int max_pages, int n_pool_pages, int n_splits, float scale,
                                const void* sinks, int sink_dtype, int* status, void* stream) {
    GI_REQUIRE(n_tokens >= 0 && H > 0 && dk > 0 && dk % 8 == 0 && rank > 0 && rank <= dk && rank <= 512,
               "gi_latent_decode: rows of %d (a multiple of 8) with %d value columns (at most 512)", dk, rank);
    GI_REQUIRE(n_splits >= 1 && n_splits <= 64 && H <= 65535 && n_tokens <= 65535, "gi_latent_decode: slices, heads, tokens");
    if (n_tokens == 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    {   // tensor cores: rows staged with 4 words of padding past a multiple of 32 words
        const int words16 = ((dk + 15) / 16) * 8;
        const int kw = words16 + ((4 - words16 % 32) + 32) % 32;
        const size_t smem_mma = ((size_t)(32 + 2 * LD_KEYS) * kw + 32 * 33 + 32 * 20 + 32) * 4;
        const int n_tiles = (rank + 7) / 8;
        const int NTW = n_tiles > 32 ? 8 : (n_tiles > 16 ? 4 : (n_tiles > 8 ? 2 : 1));
        if (smem_mma <= 200 * 1024) {
            dim3 grid_mma(n_tokens, n_splits, (H + 31) / 32);
#define LDM_CASE(N)                                                                                                    \
            if (NTW == N) {                                                                                            \
                int rc = gi_reserve_smem((const void*)latent_decode_mma_kernel<N>, smem_mma, "gi_latent_decode");      \
                if (rc) return rc;                                                                                     \
                gi_launch(latent_decode_mma_kernel<N>, grid_mma, dim3(LD_WARPS * 32), smem_mma, s, (const bf16*)q,     \
                          (const bf16*)pool, block_table, tok_pos, tok_slot, part, H, dk, rank, kw, page_size, max_pages, \
                          n_pool_pages, n_splits, scale, status);                                                      \
            }
            LDM_CASE(1) LDM_CASE(2) LDM_CASE(4) LDM_CASE(8)
#undef LDM_CASE
            int rc = gi_check_launch("gi_latent_decode");
            if (rc) return rc;
            gi_launch(latent_decode_combine_kernel, dim3(n_tokens, H), dim3(128), 0, s, (const float*)part, (bf16*)out, H, rank,
                      n_splits, sinks, sink_dtype);
            return gi_check_launch("gi_latent_decode_combine");
        }
    }
    const int HPW = H > 16 ? 4 : (H > 8 ? 2 : 1);
    const int HG = HPW * LD_WARPS;
    const int DPL2 = rank > 256 ? 8 : (rank > 128 ? 4 : (rank > 64 ? 2 : 1));
    const size_t smem = (size_t)HG * dk * 4 + (size_t)LD_KEYS * (dk / 2 + 1) * 4;
    GI_REQUIRE(smem <= 220 * 1024, "gi_latent_decode: rows of %d need %zu bytes of shared memory", dk, smem);
    dim3 grid(n_tokens, n_splits, (H + HG - 1) / HG);
#define LD_CASE(A, B)                                                                                             \
    if (HPW == A && DPL2 == B) {                                                                                  \
        int rc = gi_reserve_smem((const void*)latent_decode_kernel<A, B>, smem, "gi_latent_decode");              \
        if (rc) return rc;                                                                                        \
        gi_launch(latent_decode_kernel<A, B>, grid, dim3(LD_WARPS * 32), smem, s, (const bf16*)q, (const bf16*)pool, \
                  block_table, tok_pos, tok_slot, part, H, dk, rank, page_size, max_pages, n_pool_pages, n_splits, \
                  scale, status);                                                                                 \
    }
    LD_CASE(1, 1) LD_CASE(1, 2) LD_CASE(1, 4) LD_CASE(1, 8)
    LD_CASE(2, 1) LD_CASE(2, 2) LD_CASE(2, 4) LD_CASE(2, 8)
    LD_CASE(4, 1) LD_CASE(4, 2) LD_CASE(4, 4) LD_CASE(4, 8)
#undef LD_CASE
    int rc = gi_check_launch("gi_latent_decode");
    if (rc) return rc;
    gi_launch(latent_decode_combine_kernel, dim3(n_tokens, H), dim3(128), 0, s, (const float*)part, (bf16*)out, H, rank,
              n_splits, sinks, sink_dtype);
    return gi_check_launch("gi_latent_decode_combine");
}
