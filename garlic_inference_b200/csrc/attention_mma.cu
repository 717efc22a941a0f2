// bfloat16 attention over the paged cache on the tensor cores: a flash-style
// kernel for steps that bring several tokens per sequence (prompts) and a
// split-KV kernel for decode steps, with its combine kernel.
//
// Both compute, per query,  o = softmax_j(q . k_j * scale) v_j  over the keys
// j <= pos of the query's own sequence (and j > pos - window when window > 0),
// query head h reading key/value head h / (n_q / n_kv); scores, softmax and
// the accumulation are float32, the probabilities are rounded to bfloat16 for
// the second product.  Upstream hands all of this to a library
// (src/src-cuda/attention/fattn.cu:74-140).
//
// Tiles: 64 keys at a time, read through the block table row by row (a tile
// may span pages of any size), staged in shared memory with cp.async in two
// stages, rows padded by 16 bytes so that ldmatrix is free of bank conflicts
// for every head size.  Products are mma.sync m16n8k16.
//   prefill: one CTA = 64 consecutive queries of one sequence and one query
//            head; 4 warps of 16 queries; every warp visits all keys.
//   decode:  one CTA = one sequence, one key/value head, one slice of the
//            keys; the rows of the product are the n_q / n_kv query heads of
//            the group (at most 16); the 4 warps take 16 keys each of every
//            tile, each streaming them through a queue of its own, and are
//            merged at the end.  Each slice writes a partial
//            (max, sum, unnormalised output) to scratch memory; the combine
//            kernel merges the slices.  The number of slices is a launch
//            parameter; which keys a slice covers follows from the sequence's
//            length on the device, so a recorded launch stays valid as the
//            sequence grows.
// Head sizes: multiples of 16 up to 128; keys and values of one size, or one twice the other.
// Both kernels also take a chunk mask, a key pool with heads of its own and strided queries and outputs (AttnLayout
// below): what a mixer with several softmax maps per head over shared values needs.
#include "common.cuh"
#include <math.h>

#define AT_THREADS 128
#define AT_BN 64            // keys per tile
#define AT_BM 64            // queries per prefill CTA
#define AT_DEC_DEPTH 2      // stages of a warp's queue in the decode kernel

// ------------------------------------------------------------------------------ PTX helpers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem, bool valid) {
    const int bytes = valid ? 16 : 0;                     // 0 source bytes: the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(smem)), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(smem)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(smem)));
}
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Where the prompt kernel finds its operands when they are not the plain [rows, heads, D] and [pages, n_kv, page, D]:
// a query row's elements start at row * q_ts + head * q_hs + q_o (the output's likewise), the key pool has n_kh
// heads per page and query head h reads key head (h / group) * k_mul + k_add (the value pool keeps n_kv heads
// and head h / group).  That is what a mixer with several softmax maps per head over the same values needs: map
// m of a head lies at q_o = m D, reads key head kvh * maps + m, and writes beside the other maps.  chunk > 0: a
// query sees only the keys of its own chunk of positions (chunks counted from position 0).
// maps > 1: one launch serves all maps; the grid's head axis is then maps times as long and block y belongs to map
// y / heads, which adds map * D to q_o, map to k_add and map * DV to o_o.
// sinks: float32 [n_q], a score per query head that takes part in the softmax's denominator and has no value.
// dist_bias: float32 [n_dist, n_q], added to the scaled score of key j for the query at position i at row
// min(i - j, n_dist - 1), column the query head.  Both are null for mixers without them.
struct AttnLayout {
    long long q_ts, q_hs, q_o, o_ts, o_hs, o_o;
    int n_kh, k_mul, k_add, chunk, maps;
    const float* sinks;
    const float* dist_bias;
    int n_dist;
    int bias_smem;          // the prompt kernel keeps its head's column of dist_bias in shared memory (set by the launcher)
};
#define AT_BIAS_SMEM_MAX 8192      // distances up to which a head's biases are staged in shared memory
#define AT_LOG2E 1.4426950408889634f

// Element offset of row j of a sequence inside a pool (for key/value head kvh), or -1 when j is not below
// key_end or its page is not mapped.  No branch around the table read, so that a thread's reads for
// several rows are issued together instead of one after the other.
__device__ __forceinline__ long long kv_row_offset(const int* __restrict__ bt_row, int j, int key_end, int n_kv, int kvh,
                                                   int page_size, int max_pages, int n_pool_pages, int D) {
    const int lp = j / page_size;
    const bool in = j >= 0 && j < key_end && lp < max_pages;
    const int page = __ldg(bt_row + (in ? lp : 0));
    const bool ok = in && page >= 0 && page < n_pool_pages;
    return ok ? (((long long)page * n_kv + kvh) * page_size + (j - lp * page_size)) * D : -1;
}

// Stage one tile of 64 keys (rows key0 .. key0+63 of the sequence) of keys and values into shared memory.
// Rows at or beyond key_end, and rows whose page is not mapped, are zero-filled.
// Keys are rows of DK elements in a pool with n_kh heads per page (head kh), values rows of DV elements in a pool
// with n_kv heads per page (head kvh).
template <int DK, int DV>
__device__ __forceinline__ void load_kv_tile(bf16* sK, bf16* sV, const bf16* __restrict__ k_pool,
                                             const bf16* __restrict__ v_pool, const int* __restrict__ bt_row,
                                             int key0, int key_end, int n_kv, int kvh, int page_size,
                                             int max_pages, int n_pool_pages, int n_kh, int kh) {
    {
        constexpr int LD = DK + 8, CH = DK / 8, PASSES = AT_BN * CH / AT_THREADS;
        long long off[PASSES];
#pragma unroll
        for (int p = 0; p < PASSES; ++p)
            off[p] = kv_row_offset(bt_row, key0 + (threadIdx.x + p * AT_THREADS) / CH, key_end, n_kh, kh, page_size,
                                   max_pages, n_pool_pages, DK);
#pragma unroll
        for (int p = 0; p < PASSES; ++p) {
            const int i = threadIdx.x + p * AT_THREADS;
            const int r = i / CH, c = i % CH;
            const bool valid = off[p] >= 0;
            cp_async_16(sK + r * LD + c * 8, k_pool + (valid ? (size_t)off[p] + c * 8 : 0), valid);
        }
    }
    {
        constexpr int LD = DV + 8, CH = DV / 8, PASSES = AT_BN * CH / AT_THREADS;
        long long off[PASSES];
#pragma unroll
        for (int p = 0; p < PASSES; ++p)
            off[p] = kv_row_offset(bt_row, key0 + (threadIdx.x + p * AT_THREADS) / CH, key_end, n_kv, kvh, page_size,
                                   max_pages, n_pool_pages, DV);
#pragma unroll
        for (int p = 0; p < PASSES; ++p) {
            const int i = threadIdx.x + p * AT_THREADS;
            const int r = i / CH, c = i % CH;
            const bool valid = off[p] >= 0;
            cp_async_16(sV + r * LD + c * 8, v_pool + (valid ? (size_t)off[p] + c * 8 : 0), valid);
        }
    }
}

// A fragments (16 rows x D) of a row-major tile in shared memory, kept in registers.
template <int D>
__device__ __forceinline__ void load_a_frags(uint32_t (&a)[D / 16][4], const bf16* tile /* 16 rows, stride D+8 */) {
    constexpr int LD = D + 8;
    const int lane = threadIdx.x & 31, mat = lane >> 3, r = lane & 7;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk)
        ldmatrix_x4(a[kk], tile + ((mat & 1) * 8 + r) * LD + kk * 16 + (mat >> 1) * 8);
}

// S[16 x 8*NT] += Q[16 x D] . K[keys x D]^T for NT key n-tiles starting at row `krow0` of the staged keys.
template <int D, int NT>
__device__ __forceinline__ void qk_product(float (&s)[NT][4], const uint32_t (&a)[D / 16][4], const bf16* sK, int krow0) {
    constexpr int LD = D + 8;
    const int lane = threadIdx.x & 31, mat = lane >> 3, r = lane & 7;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[nt][e] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
        for (int np = 0; np < NT / 2; ++np) {
            uint32_t b[4];
            ldmatrix_x4(b, sK + (krow0 + np * 16 + (mat >> 1) * 8 + r) * LD + kk * 16 + (mat & 1) * 8);
            mma_16816(s[2 * np], a[kk], b[0], b[1]);
            mma_16816(s[2 * np + 1], a[kk], b[2], b[3]);
        }
    }
}

// O[16 x D] += P[16 x 16*KS] . V[keys x D] for KS key k-steps starting at row `vrow0` of the staged values.
template <int D, int KS>
__device__ __forceinline__ void pv_product(float (&o)[D / 8][4], const uint32_t (&p)[KS][4], const bf16* sV, int vrow0) {
    constexpr int LD = D + 8;
    const int lane = threadIdx.x & 31, mat = lane >> 3, r = lane & 7;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
        for (int dp = 0; dp < D / 16; ++dp) {
            uint32_t b[4];
            ldmatrix_x4_trans(b, sV + (vrow0 + ks * 16 + (mat & 1) * 8 + r) * LD + dp * 16 + (mat >> 1) * 8);
            mma_16816(o[2 * dp], p[ks], b[0], b[1]);
            mma_16816(o[2 * dp + 1], p[ks], b[2], b[3]);
        }
    }
}

// One online-softmax update of a warp's 16 rows over NT*8 scores (already scaled to the log2 domain and
// masked with -inf): rescales o, updates (m, l) and leaves bfloat16 probabilities in p.
template <int D, int NT>
__device__ __forceinline__ void softmax_update(float (&s)[NT][4], float (&m)[2], float (&l)[2], float (&o)[D / 8][4],
                                               uint32_t (&p)[NT / 2][4]) {
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        mx[0] = fmaxf(mx[0], fmaxf(s[nt][0], s[nt][1]));
        mx[1] = fmaxf(mx[1], fmaxf(s[nt][2], s[nt][3]));
    }
    float corr[2], use[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
        const float m_new = fmaxf(m[h], mx[h]);
        use[h] = m_new == -INFINITY ? 0.f : m_new;        // a row with no key yet: everything stays 0
        corr[h] = exp2f(m[h] - use[h]);
        m[h] = m_new;
    }
    float sum[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        const float p0 = exp2f(s[nt][0] - use[0]), p1 = exp2f(s[nt][1] - use[0]);
        const float p2 = exp2f(s[nt][2] - use[1]), p3 = exp2f(s[nt][3] - use[1]);
        sum[0] += p0 + p1;
        sum[1] += p2 + p3;
        p[nt / 2][(nt & 1) * 2 + 0] = pack_bf16(p0, p1);
        p[nt / 2][(nt & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
    l[0] = l[0] * corr[0] + sum[0];                        // per-thread partial sums; the quad is added up at the end
    l[1] = l[1] * corr[1] + sum[1];
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt) {
        o[dt][0] *= corr[0]; o[dt][1] *= corr[0];
        o[dt][2] *= corr[1]; o[dt][3] *= corr[1];
    }
}

// ------------------------------------------------------------------------------ prefill
// tiles[t] = {slot, first row of q, rows in the tile (<= 64), position of the first row}
template <int D, int DV>
__global__ void __launch_bounds__(AT_THREADS)
flash_prefill_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_pool, const bf16* __restrict__ v_pool,
                     const int* __restrict__ block_table, const int4* __restrict__ tiles, bf16* __restrict__ out,
                     int n_q, int n_kv, int page_size, int max_pages, int n_pool_pages, int window, float scale_log2,
                     AttnLayout lay) {
    gi_pdl_start();
    constexpr int LD = D + 8, LDV = DV + 8;
    extern __shared__ __align__(16) unsigned char at_smem[];
    bf16* sQ = reinterpret_cast<bf16*>(at_smem);
    bf16* sK = sQ + AT_BM * LD;
    bf16* sV = sK + 2 * AT_BN * LD;
    float* sB = reinterpret_cast<float*>(sV + 2 * AT_BN * LDV);       // [n_dist] when lay.bias_smem: this head's biases, in powers of two

    const int4 ti = tiles[blockIdx.x];
    const int slot = ti.x, row0 = ti.y, n_rows = ti.z, pos0 = ti.w;
    const int h = blockIdx.y % n_q, map = blockIdx.y / n_q, kvh = h / (n_q / n_kv);
    lay.q_o += (long long)map * D; lay.o_o += (long long)map * DV; lay.k_add += map;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    if (slot < 0 || n_rows <= 0) return;
    const int* bt_row = block_table + (size_t)slot * max_pages;

    const int hi = pos0 + n_rows - 1;                                   // last position of the tile
    int lo = window > 0 ? max(0, pos0 - window + 1) : 0;                // first key any row of the tile sees
    const int chunk = lay.chunk;
    if (chunk > 0) lo = max(lo, pos0 / chunk * chunk);
    const int kt_lo = lo / AT_BN, n_tiles = hi / AT_BN - kt_lo + 1;
    const int n_kh = lay.n_kh > 0 ? lay.n_kh : n_kv, kh = kvh * lay.k_mul + lay.k_add;
    if (lay.bias_smem)                           // read after the first barrier of the loop below
        for (int i = threadIdx.x; i < lay.n_dist; i += AT_THREADS) sB[i] = __ldg(lay.dist_bias + (size_t)i * n_q + h) * AT_LOG2E;

    {   // the queries of the tile, rows beyond n_rows zero-filled
        constexpr int CH = D / 8;
#pragma unroll
        for (int p = 0; p < AT_BM * CH / AT_THREADS; ++p) {
            const int i = threadIdx.x + p * AT_THREADS;
            const int r = i / CH, c = i % CH;
            const bool valid = r < n_rows;
            const bf16* src = q + (size_t)(row0 + (valid ? r : 0)) * lay.q_ts + (size_t)h * lay.q_hs + lay.q_o + c * 8;
            cp_async_16(sQ + r * LD + c * 8, src, valid);
        }
    }
    load_kv_tile<D, DV>(sK, sV, k_pool, v_pool, bt_row, kt_lo * AT_BN, hi + 1, n_kv, kvh, page_size, max_pages,
                        n_pool_pages, n_kh, kh);
    cp_async_commit();

    uint32_t a[D / 16][4];
    float o[DV / 8][4];
#pragma unroll
    for (int dt = 0; dt < DV / 8; ++dt)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[dt][e] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    const int p_row[2] = {pos0 + warp * 16 + g, pos0 + warp * 16 + g + 8};      // positions of this thread's rows
    const int p_warp_max = pos0 + warp * 16 + 15;
    // first key each of this thread's rows sees in its chunk, and the first any row of the warp sees
    const int c_row[2] = {chunk > 0 ? p_row[0] / chunk * chunk : 0, chunk > 0 ? p_row[1] / chunk * chunk : 0};
    const int c_warp = chunk > 0 ? (pos0 + warp * 16) / chunk * chunk : 0;

    for (int it = 0; it < n_tiles; ++it) {
        const int st = it & 1;
        if (it + 1 < n_tiles) {
            load_kv_tile<D, DV>(sK + (st ^ 1) * AT_BN * LD, sV + (st ^ 1) * AT_BN * LDV, k_pool, v_pool, bt_row,
                                (kt_lo + it + 1) * AT_BN, hi + 1, n_kv, kvh, page_size, max_pages, n_pool_pages, n_kh, kh);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (it == 0) load_a_frags<D>(a, sQ + warp * 16 * LD);
        const int key0 = (kt_lo + it) * AT_BN;
        const bool warp_sees = key0 <= p_warp_max && (window <= 0 || key0 + AT_BN - 1 > pos0 + warp * 16 - window) &&
                               key0 + AT_BN - 1 >= c_warp;
        if (warp_sees) {
            float s[AT_BN / 8][4];
            qk_product<D, AT_BN / 8>(s, a, sK + st * AT_BN * LD, 0);
#pragma unroll
            for (int nt = 0; nt < AT_BN / 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int j = key0 + nt * 8 + 2 * t + (e & 1);
                    const int p = p_row[e >> 1];
                    const bool ok = j <= p && (window <= 0 || j > p - window) && j >= c_row[e >> 1];
                    float sc = s[nt][e] * scale_log2;
                    if (lay.dist_bias && ok)
                        sc = lay.bias_smem ? sc + sB[min(p - j, lay.n_dist - 1)]
                                           : fmaf(__ldg(lay.dist_bias + (size_t)min(p - j, lay.n_dist - 1) * n_q + h), AT_LOG2E, sc);
                    s[nt][e] = ok ? sc : -INFINITY;
                }
            }
            uint32_t pf[AT_BN / 16][4];
            softmax_update<DV, AT_BN / 8>(s, m, l, o, pf);
            pv_product<DV, AT_BN / 16>(o, pf, sV + st * AT_BN * LDV, 0);
        }
        __syncthreads();
    }
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        l[hh] += __shfl_xor_sync(0xffffffffu, l[hh], 1);
        l[hh] += __shfl_xor_sync(0xffffffffu, l[hh], 2);
    }
    if (lay.sinks) {                                        // the sink joins the denominator: a key without a value
        const float s0 = __ldg(lay.sinks + h) * AT_LOG2E;
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            const float M = fmaxf(m[hh], s0), f = exp2f(m[hh] - M);      // f = 0 for a row that saw no key
            l[hh] = l[hh] * f + exp2f(s0 - M);
#pragma unroll
            for (int dt = 0; dt < DV / 8; ++dt) { o[dt][hh * 2] *= f; o[dt][hh * 2 + 1] *= f; }
        }
    }
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        const int r = warp * 16 + g + hh * 8;
        if (r >= n_rows) continue;
        const float inv = l[hh] > 0.f ? 1.f / l[hh] : 0.f;
        bf16* dst = out + (size_t)(row0 + r) * lay.o_ts + (size_t)h * lay.o_hs + lay.o_o;
#pragma unroll
        for (int dt = 0; dt < DV / 8; ++dt)
            *reinterpret_cast<uint32_t*>(dst + dt * 8 + 2 * t) = pack_bf16(o[dt][hh * 2] * inv, o[dt][hh * 2 + 1] * inv);
    }
}

// ------------------------------------------------------------------------------ decode (split-KV)
// part_o  [n_seqs, n_q, n_splits, D]  float32 unnormalised outputs
// part_ml [n_seqs, n_q, n_splits, 2]  float32 (max in the log2 domain, sum)
template <int D, int DV>
__global__ void __launch_bounds__(AT_THREADS)
decode_splitkv_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_pool, const bf16* __restrict__ v_pool,
                      const int* __restrict__ block_table, const int* __restrict__ tok_pos,
                      const int* __restrict__ tok_slot, float* __restrict__ part_o, float* __restrict__ part_ml,
                      int n_q, int n_kv, int page_size, int max_pages, int n_pool_pages, int window,
                      float scale_log2, int n_splits, AttnLayout lay) {
    gi_pdl_launch_dependents();
    constexpr int LD = D + 8, CH = D / 8, LDV = DV + 8, CHV = DV / 8;
    constexpr int STAGE = 16 * LD + 16 * LDV;                    // elements of one warp's stage: 16 keys, 16 values
    extern __shared__ __align__(16) unsigned char at_smem[];
    bf16* sQ = reinterpret_cast<bf16*>(at_smem);                // 16 rows
    bf16* sKV = sQ + 16 * LD;                                    // [4 warps][AT_DEC_DEPTH][keys | values][16][LD]

    const int split = blockIdx.x, kvh = blockIdx.y % n_kv, map = blockIdx.y / n_kv, b = blockIdx.z;
    const int grp = n_q / n_kv, maps = lay.maps > 1 ? lay.maps : 1;
    lay.q_o += (long long)map * D; lay.k_add += map;
    const size_t prow = ((size_t)b * maps + map) * n_q + (size_t)kvh * grp;      // first row of this block's partials
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int slot = tok_slot[b], pos = tok_pos[b];
    const int kv_len = pos + 1;
    int lo = window > 0 ? max(0, kv_len - window) : 0;
    if (lay.chunk > 0) lo = max(lo, max(pos, 0) / lay.chunk * lay.chunk);
    const int lo_al = lo / AT_BN * AT_BN;
    const int n_kh = lay.n_kh > 0 ? lay.n_kh : n_kv, kh = kvh * lay.k_mul + lay.k_add;
    const int nt_all = slot < 0 ? 0 : (kv_len - lo_al + AT_BN - 1) / AT_BN;
    const int per = (nt_all + n_splits - 1) / n_splits;
    const int t0 = split * per, t1 = min(nt_all, t0 + per);
    float* my_ml = part_ml + (prow * n_splits + split) * 2;
    gi_pdl_wait();                               // positions and slots above are set before the step's first kernel
    if (t0 >= t1) {                                              // nothing for this slice: an empty partial
        if (threadIdx.x < grp) {
            my_ml[(size_t)threadIdx.x * n_splits * 2] = -INFINITY;
            my_ml[(size_t)threadIdx.x * n_splits * 2 + 1] = 0.f;
        }
        return;
    }
    const int* bt_row = block_table + (size_t)slot * max_pages;

    for (int i = threadIdx.x; i < 16 * (D / 8); i += AT_THREADS) {
        const int r = i / (D / 8), c = i % (D / 8);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < grp) v = *reinterpret_cast<const uint4*>(q + (size_t)b * lay.q_ts + (size_t)(kvh * grp + r) * lay.q_hs + lay.q_o + c * 8);
        *reinterpret_cast<uint4*>(sQ + r * LD + c * 8) = v;
    }

    // Each warp streams its own 16 keys (and values) of every 64-key tile through a queue of its own,
    // AT_DEC_DEPTH stages deep: the warps never wait for each other while the cache is read.
    bf16* ring = sKV + warp * AT_DEC_DEPTH * STAGE;
    const int n_it = t1 - t0;
    auto issue = [&](int i) {
        if (i < n_it) {
            bf16* st = ring + (i % AT_DEC_DEPTH) * STAGE;
            const int key0 = lo_al + (t0 + i) * AT_BN + warp * 16;
            long long off[16 * CH / 32];
#pragma unroll
            for (int p = 0; p < 16 * CH / 32; ++p)
                off[p] = kv_row_offset(bt_row, key0 + (lane + p * 32) / CH, kv_len, n_kh, kh, page_size, max_pages,
                                       n_pool_pages, D);
#pragma unroll
            for (int p = 0; p < 16 * CH / 32; ++p) {
                const int idx = lane + p * 32;
                const int r = idx / CH, c = idx % CH;
                const bool valid = off[p] >= 0;
                cp_async_16(st + r * LD + c * 8, k_pool + (valid ? (size_t)off[p] + c * 8 : 0), valid);
            }
            long long offv[16 * CHV / 32];
#pragma unroll
            for (int p = 0; p < 16 * CHV / 32; ++p)
                offv[p] = kv_row_offset(bt_row, key0 + (lane + p * 32) / CHV, kv_len, n_kv, kvh, page_size, max_pages,
                                        n_pool_pages, DV);
#pragma unroll
            for (int p = 0; p < 16 * CHV / 32; ++p) {
                const int idx = lane + p * 32;
                const int r = idx / CHV, c = idx % CHV;
                const bool valid = offv[p] >= 0;
                cp_async_16(st + 16 * LD + r * LDV + c * 8, v_pool + (valid ? (size_t)offv[p] + c * 8 : 0), valid);
            }
        }
        cp_async_commit();                                       // an empty group when nothing is left: the count stays uniform
    };
#pragma unroll
    for (int i = 0; i < AT_DEC_DEPTH - 1; ++i) issue(i);

    uint32_t a[D / 16][4];
    float o[DV / 8][4];
#pragma unroll
    for (int dt = 0; dt < DV / 8; ++dt)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[dt][e] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    __syncthreads();                                             // the queries are in shared memory
    load_a_frags<D>(a, sQ);

    for (int i = 0; i < n_it; ++i) {
        issue(i + AT_DEC_DEPTH - 1);
        cp_async_wait<AT_DEC_DEPTH - 1>();
        __syncwarp();                                            // every lane's copies of stage i have landed
        const bf16* st = ring + (i % AT_DEC_DEPTH) * STAGE;
        const int key0 = lo_al + (t0 + i) * AT_BN + warp * 16;  // this warp's 16 keys of the tile
        if (key0 <= pos && key0 + 15 >= lo) {
            float s[2][4];
            qk_product<D, 2>(s, a, st, 0);
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int j = key0 + nt * 8 + 2 * t + (e & 1);
                    const bool ok = j <= pos && j >= lo;
                    float sc = s[nt][e] * scale_log2;
                    if (lay.dist_bias && ok && g + (e >> 1) * 8 < grp)
                        sc = fmaf(__ldg(lay.dist_bias + (size_t)min(pos - j, lay.n_dist - 1) * n_q + kvh * grp + g + (e >> 1) * 8),
                                  AT_LOG2E, sc);
                    s[nt][e] = ok ? sc : -INFINITY;
                }
            uint32_t pf[1][4];
            softmax_update<DV, 2>(s, m, l, o, pf);
            pv_product<DV, 1>(o, pf, st + 16 * LD, 0);
        }
        __syncwarp();                                            // the stage may be overwritten by the next issue
    }
    cp_async_wait<0>();
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        l[hh] += __shfl_xor_sync(0xffffffffu, l[hh], 1);
        l[hh] += __shfl_xor_sync(0xffffffffu, l[hh], 2);
    }
    __syncthreads();                                             // all warps are done with their queues
    // merge the four warps (each saw other keys) through shared memory, reusing the tile buffers
    float* mO = reinterpret_cast<float*>(sKV);                   // [4][16][DV]
    float* mM = mO + 4 * 16 * DV;                                // [4][16]
    float* mL = mM + 4 * 16;                                     // [4][16]
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        const int r = g + hh * 8;
#pragma unroll
        for (int dt = 0; dt < DV / 8; ++dt) {
            mO[(warp * 16 + r) * DV + dt * 8 + 2 * t] = o[dt][hh * 2];
            mO[(warp * 16 + r) * DV + dt * 8 + 2 * t + 1] = o[dt][hh * 2 + 1];
        }
        if (t == 0) { mM[warp * 16 + r] = m[hh]; mL[warp * 16 + r] = l[hh]; }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < grp * DV; i += AT_THREADS) {
        const int r = i / DV, dim = i % DV;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, mM[w * 16 + r]);
        float acc = 0.f, L = 0.f;
        if (M != -INFINITY) {
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float f = exp2f(mM[w * 16 + r] - M);       // 0 for a warp that saw no key
                acc += f * mO[(w * 16 + r) * DV + dim];
                L += f * mL[w * 16 + r];
            }
        }
        part_o[((prow + r) * n_splits + split) * DV + dim] = acc;
        if (dim == 0) {
            my_ml[(size_t)r * n_splits * 2] = M;
            my_ml[(size_t)r * n_splits * 2 + 1] = L;
        }
    }
}

template <int D>
__global__ void __launch_bounds__(128)
decode_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, bf16* __restrict__ out,
                      int n_splits, int n_q, long long o_ts, long long o_hs, long long o_o, int maps,
                      const float* __restrict__ sinks) {
    gi_pdl_start();
    const size_t row = blockIdx.x;                               // (sequence * maps + map) * n_q + head
    // where the row's result goes: dense rows, or (n_q > 0) sequence * o_ts + head * o_hs + o_o + map * D
    bf16* dst = n_q > 0 ? out + (row / ((size_t)n_q * maps)) * o_ts + (row % n_q) * o_hs + o_o + ((row / n_q) % maps) * D
                        : out + row * D;
    const float* ml = part_ml + row * n_splits * 2;
    float M = -INFINITY;
    for (int s = 0; s < n_splits; ++s) M = fmaxf(M, ml[2 * s]);
    // a sink (n_q > 0 only): one more slice with sum 1 and no output
    const float s0 = sinks ? __ldg(sinks + row % n_q) * AT_LOG2E : -INFINITY;
    M = fmaxf(M, s0);
    for (int dim = threadIdx.x; dim < D; dim += blockDim.x) {
        float acc = 0.f, L = sinks ? exp2f(s0 - M) : 0.f;
        if (M != -INFINITY) {
            for (int s = 0; s < n_splits; ++s) {
                const float ms = ml[2 * s];
                if (ms == -INFINITY) continue;                   // an empty slice: its output was never written
                const float f = exp2f(ms - M);
                acc += f * part_o[(row * n_splits + s) * D + dim];
                L += f * ml[2 * s + 1];
            }
        }
        dst[dim] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
    }
}

// ------------------------------------------------------------------------------ entry points
#define AT_DISPATCH_D(d, CALL)                                                                                 \
    switch (d) {                                                                                               \
        case 16: { CALL(16); break; }                                                                          \
        case 32: { CALL(32); break; }                                                                          \
        case 48: { CALL(48); break; }                                                                          \
        case 64: { CALL(64); break; }                                                                          \
        case 80: { CALL(80); break; }                                                                          \
        case 96: { CALL(96); break; }                                                                          \
        case 112: { CALL(112); break; }                                                                        \
        case 128: { CALL(128); break; }                                                                        \
        default: GI_REQUIRE(false, "attention (tensor cores): head_dim %d must be a multiple of 16 up to 128", d); \
    }

// Pairs (key size, value size) the kernels are built for: equal sizes, values twice the keys, keys twice the values;
// multiples of 16 up to 128.
#define AT_DISPATCH_DD(dk, dv, CALL)                                                                           \
    if ((dk) == (dv)) {                                                                                        \
        switch (dk) {                                                                                          \
            case 16: { CALL(16, 16); break; }   case 32: { CALL(32, 32); break; }                              \
            case 48: { CALL(48, 48); break; }   case 64: { CALL(64, 64); break; }                              \
            case 80: { CALL(80, 80); break; }   case 96: { CALL(96, 96); break; }                              \
            case 112: { CALL(112, 112); break; } case 128: { CALL(128, 128); break; }                          \
            default: GI_REQUIRE(false, "attention (tensor cores): head_dim %d must be a multiple of 16 up to 128", dk); \
        }                                                                                                      \
    } else if ((dv) == 2 * (dk)) {                                                                             \
        switch (dk) {                                                                                          \
            case 16: { CALL(16, 32); break; }   case 32: { CALL(32, 64); break; }                              \
            case 48: { CALL(48, 96); break; }   case 64: { CALL(64, 128); break; }                             \
            default: GI_REQUIRE(false, "attention (tensor cores): keys of %d with values of %d", dk, dv);      \
        }                                                                                                      \
    } else if ((dk) == 2 * (dv)) {                                                                             \
        switch (dv) {                                                                                          \
            case 16: { CALL(32, 16); break; }   case 32: { CALL(64, 32); break; }                              \
            case 48: { CALL(96, 48); break; }   case 64: { CALL(128, 64); break; }                             \
            default: GI_REQUIRE(false, "attention (tensor cores): keys of %d with values of %d", dk, dv);      \
        }                                                                                                      \
    } else {                                                                                                   \
        GI_REQUIRE(false, "attention (tensor cores): keys of %d with values of %d", dk, dv);                   \
    }

extern "C" int gi_attention_mma_takes(int dk, int dv) {
    const bool ok16 = dk > 0 && dv > 0 && dk % 16 == 0 && dv % 16 == 0 && dk <= 128 && dv <= 128;
    return ok16 && (dk == dv || dv == 2 * dk || dk == 2 * dv);
}

static int check_common(const char* who, int n_q, int n_kv, int d, int page_size, int max_pages, int window) {
    GI_REQUIRE(n_q > 0 && n_kv > 0 && n_q % n_kv == 0, "%s: %d query heads are no multiple of %d key/value heads", who, n_q, n_kv);
    GI_REQUIRE(d > 0 && d % 16 == 0 && d <= 128, "%s: head_dim %d must be a multiple of 16 up to 128", who, d);
    GI_REQUIRE(page_size > 0 && max_pages > 0 && window >= 0, "%s: page size, table width and window", who);
    return 0;
}

// Raises a kernel's dynamic shared memory limit, once per kernel and device.
static int set_smem(const void* kernel, size_t bytes) { return gi_reserve_smem(kernel, bytes, "attention"); }

static AttnLayout plain_layout(int n_q, int d, int dv) {
    AttnLayout lay;
    lay.q_ts = (long long)n_q * d; lay.q_hs = d; lay.q_o = 0;
    lay.o_ts = (long long)n_q * dv; lay.o_hs = dv; lay.o_o = 0;
    lay.n_kh = 0; lay.k_mul = 1; lay.k_add = 0; lay.chunk = 0; lay.maps = 1;
    lay.sinks = lay.dist_bias = nullptr; lay.n_dist = 0; lay.bias_smem = 0;
    return lay;
}

// `maps` maps per head: q [rows, n_q, maps, d], out [rows, n_q, maps, dv], key pool [pages, n_kv * maps, page, d].
static AttnLayout map_layout(int n_q, int n_kv, int d, int dv, int maps, int chunk) {
    AttnLayout lay;
    lay.q_ts = (long long)n_q * maps * d; lay.q_hs = (long long)maps * d; lay.q_o = 0;
    lay.o_ts = (long long)n_q * maps * dv; lay.o_hs = (long long)maps * dv; lay.o_o = 0;
    lay.n_kh = n_kv * maps; lay.k_mul = maps; lay.k_add = 0; lay.chunk = chunk; lay.maps = maps;
    lay.sinks = lay.dist_bias = nullptr; lay.n_dist = 0; lay.bias_smem = 0;
    return lay;
}

static int prefill_bf16_layout(const void* q, const void* k_pool, const void* v_pool, const int* block_table,
                               const int* tiles, int n_tiles, void* out, int n_q, int n_kv, int d, int dv,
                               int page_size, int max_pages, int n_pool_pages, int window, float scale,
                               AttnLayout lay, void* stream) {
    if (int rc = check_common("gi_attention_prefill_bf16", n_q, n_kv, d, page_size, max_pages, window)) return rc;
    GI_REQUIRE(n_tiles >= 0 && (long long)n_q * lay.maps <= 65535, "gi_attention_prefill_bf16: tile or head count");
    if (n_tiles == 0) return 0;
    const float scale_log2 = scale * 1.4426950408889634f;
    dim3 grid(n_tiles, n_q * lay.maps);
    lay.bias_smem = lay.dist_bias && lay.n_dist <= AT_BIAS_SMEM_MAX;
#define CALL(DK, DV)                                                                                           \
    {                                                                                                          \
        const size_t smem = ((size_t)(AT_BM + 2 * AT_BN) * (DK + 8) + (size_t)2 * AT_BN * (DV + 8)) * sizeof(bf16) + \
                            (lay.bias_smem ? (size_t)lay.n_dist * sizeof(float) : 0);                          \
        if (int rc = set_smem((const void*)flash_prefill_kernel<DK, DV>, smem)) return rc;                     \
        gi_launch(flash_prefill_kernel<DK, DV>, grid, dim3(AT_THREADS), smem, (cudaStream_t)stream,            \
            (const bf16*)q, (const bf16*)k_pool, (const bf16*)v_pool, block_table, (const int4*)tiles,         \
            (bf16*)out, n_q, n_kv, page_size, max_pages, n_pool_pages, window, scale_log2, lay);               \
    }
    AT_DISPATCH_DD(d, dv, CALL)
#undef CALL
    return gi_check_launch("gi_attention_prefill_bf16");
}

// tiles: int32 [n_tiles, 4] = {slot, first q row, rows (<= 64), position of the first row}
extern "C" int gi_attention_prefill_bf16(const void* q, const void* k_pool, const void* v_pool, const int* block_table,
                                         const int* tiles, int n_tiles, void* out, int n_q, int n_kv, int d,
                                         int page_size, int max_pages, int n_pool_pages, int window, float scale,
                                         void* stream) {
    return prefill_bf16_layout(q, k_pool, v_pool, block_table, tiles, n_tiles, out, n_q, n_kv, d, d, page_size, max_pages,
                               n_pool_pages, window, scale, plain_layout(n_q, d, d), stream);
}

// The general prompt kernel: keys of d and values of dv, `maps` softmax maps per head over the same values (q
// [rows, n_q, maps, d], out [rows, n_q, maps, dv], the key pool [pages, n_kv * maps, page, d]; one launch),
// and `chunk` (0: none).
extern "C" int gi_attention_prefill_masked_bf16(const void* q, const void* k_pool, const void* v_pool,
                                                const int* block_table, const int* tiles, int n_tiles, void* out, int n_q,
                                                int n_kv, int d, int dv, int page_size, int max_pages, int n_pool_pages,
                                                int window, int chunk, int maps, float scale, const float* sinks,
                                                const float* dist_bias, int n_dist, void* stream) {
    GI_REQUIRE(maps >= 1 && chunk >= 0, "gi_attention_prefill_masked_bf16: %d maps, chunk %d", maps, chunk);
    GI_REQUIRE((!sinks && !dist_bias) || maps == 1, "gi_attention_prefill_masked_bf16: sinks and distance biases come with one map per head");
    GI_REQUIRE(!dist_bias || n_dist > 0, "gi_attention_prefill_masked_bf16: a distance bias of %d rows", n_dist);
    AttnLayout lay = map_layout(n_q, n_kv, d, dv, maps, chunk);
    lay.sinks = sinks; lay.dist_bias = dist_bias; lay.n_dist = n_dist;
    return prefill_bf16_layout(q, k_pool, v_pool, block_table, tiles, n_tiles, out, n_q, n_kv, d, dv, page_size,
                               max_pages, n_pool_pages, window, scale, lay, stream);
}

static int decode_bf16_layout(const void* q, const void* k_pool, const void* v_pool, const int* block_table,
                              const int* tok_pos, const int* tok_slot, void* out, float* part_o, float* part_ml,
                              int n_seqs, int n_q, int n_kv, int d, int dv, int page_size, int max_pages,
                              int n_pool_pages, int window, float scale, int n_splits, AttnLayout lay, bool strided_out,
                              void* stream) {
    if (int rc = check_common("gi_attention_decode_bf16", n_q, n_kv, d, page_size, max_pages, window)) return rc;
    GI_REQUIRE(n_q / n_kv <= 16, "gi_attention_decode_bf16: %d query heads per key/value head; this kernel takes up to 16", n_q / n_kv);
    GI_REQUIRE(n_splits >= 1 && n_splits <= 65535 && (long long)n_kv * lay.maps <= 65535 && n_seqs >= 0 && n_seqs <= 65535,
               "gi_attention_decode_bf16: %d slices, %d key/value heads, %d sequences", n_splits, n_kv, n_seqs);
    if (n_seqs == 0) return 0;
    const float scale_log2 = scale * 1.4426950408889634f;
    dim3 grid(n_splits, n_kv * lay.maps, n_seqs);
    const int cq = strided_out ? n_q : 0;
#define CALL(DK, DV)                                                                                           \
    {                                                                                                          \
        size_t smem = ((size_t)16 * (DK + 8) + (size_t)4 * AT_DEC_DEPTH * 16 * (DK + 8 + DV + 8)) * sizeof(bf16); \
        const size_t merge = (size_t)16 * (DK + 8) * sizeof(bf16) + (size_t)(4 * 16 * DV + 128) * sizeof(float); \
        if (merge > smem) smem = merge;                                                                        \
        if (int rc = set_smem((const void*)decode_splitkv_kernel<DK, DV>, smem)) return rc;                    \
        gi_launch(decode_splitkv_kernel<DK, DV>, grid, dim3(AT_THREADS), smem, (cudaStream_t)stream,           \
            (const bf16*)q, (const bf16*)k_pool, (const bf16*)v_pool, block_table, tok_pos, tok_slot, part_o,  \
            part_ml, n_q, n_kv, page_size, max_pages, n_pool_pages, window, scale_log2, n_splits, lay);        \
        gi_launch(decode_combine_kernel<DV>, dim3(n_seqs * n_q * lay.maps), dim3(DV < 128 ? (DV < 32 ? 32 : DV) : 128), 0, (cudaStream_t)stream,  \
            part_o, part_ml, (bf16*)out, n_splits, cq, lay.o_ts, lay.o_hs, lay.o_o, lay.maps, cq ? lay.sinks : nullptr); \
    }
    AT_DISPATCH_DD(d, dv, CALL)
#undef CALL
    return gi_check_launch("gi_attention_decode_bf16");
}

// Scratch: part_o float32 [n_seqs * n_q * n_splits * d], part_ml float32 [n_seqs * n_q * n_splits * 2].
extern "C" int gi_attention_decode_bf16(const void* q, const void* k_pool, const void* v_pool, const int* block_table,
                                        const int* tok_pos, const int* tok_slot, void* out, float* part_o,
                                        float* part_ml, int n_seqs, int n_q, int n_kv, int d, int page_size,
                                        int max_pages, int n_pool_pages, int window, float scale, int n_splits,
                                        void* stream) {
    return decode_bf16_layout(q, k_pool, v_pool, block_table, tok_pos, tok_slot, out, part_o, part_ml, n_seqs, n_q, n_kv,
                              d, d, page_size, max_pages, n_pool_pages, window, scale, n_splits, plain_layout(n_q, d, d),
                              false, stream);
}

// The general decode kernel: as gi_attention_prefill_masked_bf16, for one token per sequence.  Scratch as above with
// dv for d and maps * n_q for n_q.
extern "C" int gi_attention_decode_masked_bf16(const void* q, const void* k_pool, const void* v_pool,
                                               const int* block_table, const int* tok_pos, const int* tok_slot, void* out,
                                               float* part_o, float* part_ml, int n_seqs, int n_q, int n_kv, int d, int dv,
                                               int page_size, int max_pages, int n_pool_pages, int window, int chunk,
                                               int maps, float scale, int n_splits, const float* sinks,
                                               const float* dist_bias, int n_dist, void* stream) {
    GI_REQUIRE(maps >= 1 && chunk >= 0, "gi_attention_decode_masked_bf16: %d maps, chunk %d", maps, chunk);
    GI_REQUIRE((!sinks && !dist_bias) || maps == 1, "gi_attention_decode_masked_bf16: sinks and distance biases come with one map per head");
    GI_REQUIRE(!dist_bias || n_dist > 0, "gi_attention_decode_masked_bf16: a distance bias of %d rows", n_dist);
    AttnLayout lay = map_layout(n_q, n_kv, d, dv, maps, chunk);
    lay.sinks = sinks; lay.dist_bias = dist_bias; lay.n_dist = n_dist;
    return decode_bf16_layout(q, k_pool, v_pool, block_table, tok_pos, tok_slot, out, part_o, part_ml, n_seqs,
                              n_q, n_kv, d, dv, page_size, max_pages, n_pool_pages, window, scale, n_splits,
                              lay, true, stream);
}

// Merges the slices' partial results of a split-KV decode kernel (this file's or the tcgen05 one):
// part_o float32 [rows * n_splits * d] unnormalised, part_ml float32 [rows * n_splits * 2] = (maximum in
// powers of two, sum); out bfloat16 [rows, d] for rows = sequences * query heads.
extern "C" int gi_attention_decode_combine(const float* part_o, const float* part_ml, void* out, int rows, int d,
                                           int n_splits, void* stream) {
    GI_REQUIRE(rows >= 0 && n_splits >= 1, "gi_attention_decode_combine: sizes");
    GI_REQUIRE(d >= 16 && d <= 128 && d % 16 == 0, "gi_attention_decode_combine: head_dim %d", d);
    if (rows == 0) return 0;
#define CALL(DD)                                                                                                 \
    gi_launch(decode_combine_kernel<DD>, dim3(rows), dim3(DD < 128 ? (DD < 32 ? 32 : DD) : 128), 0, (cudaStream_t)stream, \
              part_o, part_ml, (bf16*)out, n_splits, 0, 0LL, 0LL, 0LL, 1, (const float*)nullptr);
    AT_DISPATCH_D(d, CALL)
#undef CALL
    return gi_check_launch("gi_attention_decode_combine");
}
