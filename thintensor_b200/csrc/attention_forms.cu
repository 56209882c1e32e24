// Two further forms of causal grouped-query attention over the block cache, in float32 or bfloat16 storage with
// float32 arithmetic, for any head size up to 256, for prompts and decoding alike:
//
// * differential attention: a head's query row and a key head's cached row hold two maps of `dim` numbers each; each
//   map is a softmax attention of its own over the same values, and the head's output is
//       o = a1 - lambda * a2,   o <- o * rsqrt(mean(o^2) + eps) * gain          (over the head's value_dim numbers)
//   One warp owns a (token, query head, slice of keys), keeps both running softmaxes and reads every value once for
//   both; the subtraction and the norm are the kernel's epilogue (the merge kernel's, with several slices).
//
// * window attention with pooled blocks: position i sees the keys j with 0 <= i - j < window and, before them, one
//   entry of a second, coarser cache for each whole block of `every` tokens that ends at or before i - window (entry n
//   is the mean key and mean value of tokens n * every .. n * every + every - 1); scores may be capped,
//   s <- cap * tanh(s / cap); tokens and blocks share one softmax.  pool_blocks_kernel forms the means of the blocks
//   that a step completes, from the token cache, right after the step's keys were appended.
//
// The slices' partial (max, sum, accumulator) triples are merged in slice order, so a result does not depend on the grid.
//
// bfloat16 at the sizes listed near the end of this file runs both forms on tensor cores instead (form_kernel); the
// kernels below are the float32 path and take every other size.
#include "attention_kernels.cuh"

namespace {

constexpr int AF_ACC = ATTN_MAX_HEAD_DIM / 32;

// One running softmax of a warp; lane l owns value dimensions l, l + 32, ...
struct Running {
    float m, l;
    float acc[AF_ACC];
    __device__ __forceinline__ void clear() {
        m = -INFINITY;
        l = 0.0f;
#pragma unroll
        for (int i = 0; i < AF_ACC; ++i) acc[i] = 0.0f;
    }
    // Takes a tile's scores (one per lane, -inf for none), rescales what was gathered so far and returns this lane's weight.
    __device__ __forceinline__ float take(float score) {
        const float m_tile = tt_warp_max(score);
        if (m_tile == -INFINITY) return 0.0f;
        const float m_new = fmaxf(m, m_tile);
        const float corr = expf(m - m_new);     // 0 on the first tile
        const float p = (score == -INFINITY) ? 0.0f : expf(score - m_new);
        l = l * corr + tt_warp_sum(p);
        m = m_new;
#pragma unroll
        for (int i = 0; i < AF_ACC; ++i) acc[i] *= corr;
        return p;
    }
};

// The slices of one row and one softmax merged: acc[] (unnormalised) and the denominator.  Slice s has its accumulator
// at acc_base + s * acc_stride and its (max, sum) at ml_base + s * ml_stride.
__device__ __forceinline__ float merge_slices(const float* __restrict__ acc_base, size_t acc_stride, const float* __restrict__ ml_base,
                                              size_t ml_stride, int splits, int value_dim, int lane, float* acc) {
    float m = -INFINITY;
    for (int s = lane; s < splits; s += 32) m = fmaxf(m, __ldg(ml_base + s * ml_stride));
    m = tt_warp_max(m);
    float l = 0.0f;
#pragma unroll
    for (int i = 0; i < AF_ACC; ++i) acc[i] = 0.0f;
    for (int s = 0; s < splits; ++s) {
        const float ms = __ldg(ml_base + s * ml_stride);
        if (ms == -INFINITY) continue;
        const float w = expf(ms - m);
        l += __ldg(ml_base + s * ml_stride + 1) * w;
        const float* a = acc_base + s * acc_stride;
#pragma unroll
        for (int i = 0; i < AF_ACC; ++i) {
            const int d = lane + 32 * i;
            if (d < value_dim) acc[i] = fmaf(__ldg(a + d), w, acc[i]);
        }
    }
    return l;
}

// o = a1 / l1 - lambda * a2 / l2, normalised over the head and scaled; written in the activation type.
template <typename T>
__device__ __forceinline__ void differential_write(const float* a1, float l1, const float* a2, float l2, float lambda, float gain,
                                                   float eps, int value_dim, int lane, T* __restrict__ dst) {
    const float inv1 = l1 > 0.0f ? 1.0f / l1 : 0.0f, inv2 = l2 > 0.0f ? 1.0f / l2 : 0.0f;
    float o[AF_ACC];
    float sumsq = 0.0f;
#pragma unroll
    for (int i = 0; i < AF_ACC; ++i) {
        const int d = lane + 32 * i;
        o[i] = (d < value_dim) ? a1[i] * inv1 - lambda * (a2[i] * inv2) : 0.0f;
        sumsq += o[i] * o[i];
    }
    const float r = rsqrtf(tt_warp_sum(sumsq) / (float)value_dim + eps) * gain;
#pragma unroll
    for (int i = 0; i < AF_ACC; ++i) {
        const int d = lane + 32 * i;
        if (d < value_dim) dst[d] = tt_from_float<T>(o[i] * r);
    }
}

// q: [tokens][heads][2 * dim] (map 1, map 2); k_pool rows of 2 * dim numbers laid out the same way; v_pool transposed.
// part_acc: float32 [rows][splits][2][value_dim], part_ml: float32 [rows][splits][2][2]; both unused when splits == 1.
template <typename T>
__global__ void differential_rows_kernel(const T* __restrict__ q, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                                         const int* __restrict__ table, int table_width, int pool_blocks,
                                         const int* __restrict__ cu, const int* __restrict__ len_before, int sequences,
                                         int n_tokens, int heads, int kv_heads, int dim, int value_dim, float scale,
                                         float lambda, float gain, float eps, int splits, T* __restrict__ out,
                                         float* __restrict__ part_acc, float* __restrict__ part_ml, unsigned* status) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    extern __shared__ float q_shared[];         // ATTN_WARPS * 2 * dim
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * ATTN_WARPS + warp;
    if (row >= (long long)n_tokens * heads) return;
    const int t = (int)(row / heads), h = (int)(row - (long long)t * heads);
    const int split = blockIdx.y;
    const int b = tt_find_sequence(cu, sequences, t);
    const int pos = len_before[b] + (t - cu[b]);
    const int kh = h / (heads / kv_heads);
    const int* table_row = table + (size_t)b * table_width;
    const int row_dim = 2 * dim;

    float* qs = q_shared + warp * row_dim;
    for (int d = lane; d < row_dim; d += 32) qs[d] = tt_to_float(q[((size_t)t * heads + h) * row_dim + d]) * scale;
    __syncwarp();

    const int n_keys = pos + 1;
    int per = (n_keys + splits - 1) / splits;
    per = (per + 31) & ~31;
    const int begin = split * per;
    const int end = min(begin + per, pos + 1);

    Running one, two;
    one.clear();
    two.clear();
    for (int base = begin; base < end; base += 32) {
        const int key = base + lane;
        long long voff = -1;
        float s1 = -INFINITY, s2 = -INFINITY;
        if (key < end) {
            const long long off = tt_cache_offset(table_row, key, kh, kv_heads, row_dim, pool_blocks, status);
            if (off >= 0) {
                s1 = dot16<T>(k_pool + off, qs, dim);
                s2 = dot16<T>(k_pool + off + dim, qs + dim, dim);
                voff = tt_value_offset(table_row, key, kh, kv_heads, value_dim, pool_blocks, nullptr);
            }
        }
        const float p1 = one.take(s1), p2 = two.take(s2);
        const int count = min(32, end - base);
        for (int j = 0; j < count; ++j) {
            const float pj1 = __shfl_sync(0xffffffffu, p1, j), pj2 = __shfl_sync(0xffffffffu, p2, j);
            const long long oj = __shfl_sync(0xffffffffu, voff, j);
            if (oj < 0) continue;
            const T* vcol = v_pool + oj;
#pragma unroll
            for (int i = 0; i < AF_ACC; ++i) {
                const int d = lane + 32 * i;
                if (d < value_dim) {
                    const float v = tt_to_float(vcol[(size_t)d * TT_BLOCK_TOKENS]);
                    one.acc[i] = fmaf(pj1, v, one.acc[i]);
                    two.acc[i] = fmaf(pj2, v, two.acc[i]);
                }
            }
        }
    }

    if (splits == 1) {
        differential_write<T>(one.acc, one.l, two.acc, two.l, lambda, gain, eps, value_dim, lane, out + ((size_t)t * heads + h) * value_dim);
        return;
    }
    const size_t slot = ((size_t)row * splits + split) * 2;
#pragma unroll
    for (int i = 0; i < AF_ACC; ++i) {
        const int d = lane + 32 * i;
        if (d < value_dim) {
            part_acc[slot * value_dim + d] = one.acc[i];
            part_acc[(slot + 1) * value_dim + d] = two.acc[i];
        }
    }
    if (lane == 0) {
        part_ml[slot * 2] = one.m;
        part_ml[slot * 2 + 1] = one.l;
        part_ml[slot * 2 + 2] = two.m;
        part_ml[slot * 2 + 3] = two.l;
    }
}

template <typename T>
__global__ void differential_merge_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml, int splits,
                                          int value_dim, long long rows, float lambda, float gain, float eps, T* __restrict__ out) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * ATTN_WARPS + warp;
    if (row >= rows) return;
    const float* acc_base = part_acc + (size_t)row * splits * 2 * value_dim;
    const float* ml_base = part_ml + (size_t)row * splits * 4;
    float a1[AF_ACC], a2[AF_ACC];
    const float l1 = merge_slices(acc_base, (size_t)2 * value_dim, ml_base, 4, splits, value_dim, lane, a1);
    const float l2 = merge_slices(acc_base + value_dim, (size_t)2 * value_dim, ml_base + 2, 4, splits, value_dim, lane, a2);
    differential_write<T>(a1, l1, a2, l2, lambda, gain, eps, value_dim, lane, out + (size_t)row * value_dim);
}

constexpr int POOL_RUN = 256;       // tokens whose places in the cache pool_blocks_kernel looks up together

// Means of the blocks that this step completes: block n of sequence b (tokens n * every .. n * every + every - 1) for
// floor(before / every) <= n < floor(after / every).  grid (blocks a sequence may complete, kv heads, sequences).
template <typename T>
__global__ void pool_blocks_kernel(const T* __restrict__ k_pool, const T* __restrict__ v_pool, const int* __restrict__ table,
                                   int table_width, int pool_blocks, T* __restrict__ mean_k, T* __restrict__ mean_v,
                                   const int* __restrict__ mean_table, int mean_width, int mean_blocks, const int* __restrict__ cu,
                                   const int* __restrict__ len_before, int kv_heads, int head_dim, int value_dim, int every,
                                   unsigned* status) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    const int b = blockIdx.z, kh = blockIdx.y;
    const int before = len_before[b], after = before + (cu[b + 1] - cu[b]);
    const int n = before / every + blockIdx.x;
    if (n >= after / every) return;
    const int* table_row = table + (size_t)b * table_width;
    const int* mean_row = mean_table + (size_t)b * mean_width;
    const long long k_dst = tt_cache_offset(mean_row, n, kh, kv_heads, head_dim, mean_blocks, status);
    const long long v_dst = tt_value_offset(mean_row, n, kh, kv_heads, value_dim, mean_blocks, status);
    if (k_dst < 0 || v_dst < 0) return;
    const float share = 1.0f / (float)every;
    // the block's tokens in runs of POOL_RUN: their places in the cache are found once a run, side by side, and every
    // thread then adds its dimension over the run in token order with independent loads
    __shared__ long long k_at[POOL_RUN], v_at[POOL_RUN];
    constexpr int MOST = (2 * ATTN_MAX_HEAD_DIM + 127) / 128;      // dimensions a thread may own (blocks of at least 128 threads)
    float sum[MOST];
#pragma unroll
    for (int i = 0; i < MOST; ++i) sum[i] = 0.0f;
    for (int j0 = 0; j0 < every; j0 += POOL_RUN) {
        const int count = min(POOL_RUN, every - j0);
        __syncthreads();
        for (int j = threadIdx.x; j < count; j += blockDim.x) {
            const int position = n * every + j0 + j;
            k_at[j] = tt_cache_offset(table_row, position, kh, kv_heads, head_dim, pool_blocks, status);
            v_at[j] = tt_value_offset(table_row, position, kh, kv_heads, value_dim, pool_blocks, status);
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < MOST; ++i) {
            const int d = threadIdx.x + i * blockDim.x;
            if (d >= head_dim + value_dim) break;
            float acc = sum[i];
            if (d < head_dim) {
#pragma unroll 8
                for (int j = 0; j < count; ++j)
                    if (k_at[j] >= 0) acc += tt_to_float(k_pool[k_at[j] + d]);
            } else {
                const long long step = (long long)(d - head_dim) * TT_BLOCK_TOKENS;
#pragma unroll 8
                for (int j = 0; j < count; ++j)
                    if (v_at[j] >= 0) acc += tt_to_float(v_pool[v_at[j] + step]);
            }
            sum[i] = acc;
        }
    }
#pragma unroll
    for (int i = 0; i < MOST; ++i) {
        const int d = threadIdx.x + i * blockDim.x;
        if (d >= head_dim + value_dim) break;
        if (d < head_dim) mean_k[k_dst + d] = tt_from_float<T>(sum[i] * share);
        else mean_v[v_dst + (long long)(d - head_dim) * TT_BLOCK_TOKENS] = tt_from_float<T>(sum[i] * share);
    }
}

// The walk of attention_rows_kernel over a list of keys that starts with the visible entries of the coarser cache and
// goes on with the window's tokens; cap > 0 caps the scores.  part_acc / part_ml as in attention_rows_kernel.
template <typename T>
__global__ void pooled_window_rows_kernel(const T* __restrict__ q, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                                          const int* __restrict__ table, int table_width, int pool_blocks,
                                          const T* __restrict__ mean_k, const T* __restrict__ mean_v,
                                          const int* __restrict__ mean_table, int mean_width, int mean_blocks, int every,
                                          const int* __restrict__ cu, const int* __restrict__ len_before, int sequences,
                                          int n_tokens, int heads, int kv_heads, int head_dim, float scale, float cap, int window,
                                          int splits, T* __restrict__ out, float* __restrict__ part_acc,
                                          float* __restrict__ part_ml, unsigned* status) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    extern __shared__ float q_shared[];         // ATTN_WARPS * head_dim
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * ATTN_WARPS + warp;
    if (row >= (long long)n_tokens * heads) return;
    const int t = (int)(row / heads), h = (int)(row - (long long)t * heads);
    const int split = blockIdx.y;
    const int b = tt_find_sequence(cu, sequences, t);
    const int pos = len_before[b] + (t - cu[b]);
    const int kh = h / (heads / kv_heads);
    const int* table_row = table + (size_t)b * table_width;
    const int* mean_row = mean_table + (size_t)b * mean_width;

    float* qs = q_shared + warp * head_dim;
    for (int d = lane; d < head_dim; d += 32) qs[d] = tt_to_float(q[((size_t)t * heads + h) * head_dim + d]) * scale;
    __syncwarp();

    const int first = pos - window + 1 > 0 ? pos - window + 1 : 0;
    const int lead = pos - window + 1 > 0 ? (pos - window + 1) / every : 0;    // whole blocks that end at or before pos - window
    const int n_keys = lead + pos - first + 1;
    int per = (n_keys + splits - 1) / splits;
    per = (per + 31) & ~31;
    const int begin = split * per;
    const int end = min(begin + per, n_keys);
    const float inv_cap = cap > 0.0f ? 1.0f / cap : 0.0f;

    Running run;
    run.clear();
    for (int base = begin; base < end; base += 32) {
        const int n = base + lane;
        const T* vsrc = nullptr;
        float score = -INFINITY;
        if (n < end) {
            const bool coarse = n < lead;
            const int* trow = coarse ? mean_row : table_row;
            const int blocks = coarse ? mean_blocks : pool_blocks;
            const int at = coarse ? n : first + (n - lead);
            const long long off = tt_cache_offset(trow, at, kh, kv_heads, head_dim, blocks, status);
            if (off >= 0) {
                score = dot16<T>((coarse ? mean_k : k_pool) + off, qs, head_dim);
                if (cap > 0.0f) score = cap * tanhf(score * inv_cap);
                vsrc = (coarse ? mean_v : v_pool) + tt_value_offset(trow, at, kh, kv_heads, head_dim, blocks, nullptr);
            }
        }
        const float p = run.take(score);
        const int count = min(32, end - base);
        for (int j = 0; j < count; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            const T* vcol = reinterpret_cast<const T*>(__shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(vsrc), j));
            if (!vcol) continue;
#pragma unroll
            for (int i = 0; i < AF_ACC; ++i) {
                const int d = lane + 32 * i;
                if (d < head_dim) run.acc[i] = fmaf(pj, tt_to_float(vcol[(size_t)d * TT_BLOCK_TOKENS]), run.acc[i]);
            }
        }
    }

    if (splits == 1) {
        const float inv = run.l > 0.0f ? 1.0f / run.l : 0.0f;
#pragma unroll
        for (int i = 0; i < AF_ACC; ++i) {
            const int d = lane + 32 * i;
            if (d < head_dim) out[((size_t)t * heads + h) * head_dim + d] = tt_from_float<T>(run.acc[i] * inv);
        }
        return;
    }
    const size_t slot = (size_t)row * splits + split;
#pragma unroll
    for (int i = 0; i < AF_ACC; ++i) {
        const int d = lane + 32 * i;
        if (d < head_dim) part_acc[slot * head_dim + d] = run.acc[i];
    }
    if (lane == 0) {
        part_ml[slot * 2] = run.m;
        part_ml[slot * 2 + 1] = run.l;
    }
}


// ------------------------------------------------------------------------------------------------ tensor cores
// Both forms for bfloat16 on tensor cores (mma.sync m16n8k16, float32 accumulators and softmax), prompts and decoding.
//
// A CTA owns 64 query rows of one sequence and one key/value head, four tiles of 16 rows ((token, head of the group)
// pairs; one tile in a step of one token a sequence), and a slice of the blocks of 64 keys that those rows see.  Every block's K and V tiles are copied once per CTA
// into shared memory with cp.async, one or two blocks ahead.  With two maps a second set of four warps owns the same rows
// for map 2: it reads the other half of the query and key rows and the same value tile, so that a warp's arithmetic is that
// of an ordinary head with KD score dimensions and VD value dimensions, and the two sets meet in shared memory at the end
// (o = a1 - lambda a2, the division by the root mean square over the head, the gain).  With pooled blocks the list of
// blocks starts with those of the coarser cache, whose entry n a row at position i sees if n < floor((i - window + 1) / every).
//
// The B operands are 16-byte (for a last half chunk of the score dimensions 8-byte) pieces of cache rows: the k index of
// Q K^T is permuted alike in Q and K, the key index of P V alike in P's columns and V's rows (score column n of score
// tile j stands for key fm_key_of(j, n)), and values lie transposed inside a cache block.
// Slices of the keys (grid.z) leave (max, sum, accumulator) per row and map in the scratch of the exact kernels, in natural
// logarithm units, for the same merge kernels.

__device__ __forceinline__ void fm_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t fm_pack(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ float fm_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// cap * tanh(s / cap) through one exponential: tanh(x) = 1 - 2 / (e^(2x) + 1); absolute error about 1e-7 * cap.
__device__ __forceinline__ float fm_cap(float s, float cap, float two_log2e_over_cap) {
    const float e = fm_exp2(s * two_log2e_over_cap);
    return cap - __fdividef(2.0f * cap, e + 1.0f);
}
__device__ __forceinline__ int fm_key_of(int j, int n) { return 32 * (j >> 2) + 8 * (n >> 1) + 2 * (j & 3) + (n & 1); }
__device__ __forceinline__ void fm_cp16(void* smem_dst, const void* src) {
    const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void fm_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void fm_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// TILES: 16-row tiles of a CTA; 4 for prompts, 1 for steps of one token a sequence (more CTAs fit an SM, each with a slice of the keys)
template <int KD, int VD, int MAPS, int TILES> struct FormShape {
    static_assert(KD % 16 == 0 && VD % 8 == 0, "score dimensions in halves of a 32-wide chunk, value dimensions in 8-wide tiles");
    static constexpr int KC = KD / 32;                          // whole 32-wide chunks of a map's score dimensions
    static constexpr bool HALF = (KD % 32) != 0;                // and a last chunk of 16
    static constexpr int NT = VD / 8;
    static constexpr int K_ROW = MAPS * KD * 2;                 // bytes of one cached key row
    static constexpr bool K_SWIZZLE = (K_ROW % 128) == 0;       // rows that would start on the same bank
    static constexpr int K_TILE = 64 * K_ROW;
    static constexpr int V_TILE = VD * 128;
    static constexpr int STAGE = K_TILE + V_TILE;
    static constexpr int STAGES = STAGE <= 16384 ? 3 : 2;
    static constexpr int THREADS = TILES * MAPS * 32;
    static constexpr int EXCHANGE = MAPS == 2 ? TILES * 16 * VD * 4 : 0;    // map 2's output on its way to map 1's warps
    static constexpr int SHARED = STAGES * STAGE > EXCHANGE ? STAGES * STAGE : EXCHANGE;
};

template <int KD, int VD> struct FormState {
    static constexpr int KC = KD / 32, NT = VD / 8;
    uint32_t qa[KC + 1][4], qb[KC + 1][4];      // Q fragments of rows g and g + 8, score dimensions permuted
    float o[NT][4];
    float m_run[2], l_run[2];
};

// One block of 64 keys or entries: S = Q K^T, scale, cap, mask (row i sees index n if lo[i] <= n <= hi[i]), running softmax
// in base 2, O += P V.  load_k(j, c) returns the 16 bytes of key fm_key_of(j, g) at dimensions 32c + 8t .. + 7, load_k_half(j)
// its 8 bytes at 32 KC + 4t .. + 3; load_v(n, half) the 16 bytes of value dimension 8n + g at keys 32 half + 8t .. + 7.
template <int KD, int VD, typename LoadK, typename LoadKHalf, typename LoadV>
__device__ __forceinline__ void form_block_math(FormState<KD, VD>& st, int index_base, const int (&lo)[2], const int (&hi)[2], int t,
                                                float scale, float cap, LoadK load_k, LoadKHalf load_k_half, LoadV load_v) {
    constexpr int KC = KD / 32, NT = VD / 8;
    constexpr bool HALF = (KD % 32) != 0;
    constexpr float LOG2E = 1.4426950408889634f;
    // the eight score tiles take turns, so that consecutive products do not wait for one another's accumulator
    float s[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
#pragma unroll
    for (int c = 0; c < KC; ++c) {
        uint4 kr[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) kr[j] = load_k(j, c);
#pragma unroll
        for (int j = 0; j < 8; ++j) fm_mma(s[j], st.qa[c][0], st.qb[c][0], st.qa[c][1], st.qb[c][1], kr[j].x, kr[j].y);
#pragma unroll
        for (int j = 0; j < 8; ++j) fm_mma(s[j], st.qa[c][2], st.qb[c][2], st.qa[c][3], st.qb[c][3], kr[j].z, kr[j].w);
    }
    if constexpr (HALF) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint2 kr = load_k_half(j);
            fm_mma(s[j], st.qa[KC][0], st.qb[KC][0], st.qa[KC][1], st.qb[KC][1], kr.x, kr.y);
        }
    }
    const bool all_visible = index_base >= max(lo[0], lo[1]) && index_base + TT_BLOCK_TOKENS - 1 <= min(hi[0], hi[1]);
    const float to_log2 = cap > 0.0f ? LOG2E : scale * LOG2E;
    const float cap_factor = cap > 0.0f ? 2.0f * LOG2E / cap : 0.0f;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        float mx = -INFINITY;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                float v = s[j][2 * i + e];
                if (cap > 0.0f) v = fm_cap(v * scale, cap, cap_factor);
                v *= to_log2;
                if (!all_visible) {
                    const int index = index_base + fm_key_of(j, 2 * t + e);
                    if (index < lo[i] || index > hi[i]) v = -INFINITY;
                }
                s[j][2 * i + e] = v;
                mx = fmaxf(mx, v);
            }
        }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(st.m_run[i], mx);
        const float corr = (m_new == -INFINITY) ? 1.0f : fm_exp2(st.m_run[i] - m_new);
        const float base = (m_new == -INFINITY) ? 0.0f : m_new;
        float sum = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const float p = fm_exp2(s[j][2 * i + e] - base);
                s[j][2 * i + e] = p;
                sum += p;
            }
        }
        st.l_run[i] = st.l_run[i] * corr + sum;
        st.m_run[i] = m_new;
#pragma unroll
        for (int n = 0; n < NT; ++n) { st.o[n][2 * i] *= corr; st.o[n][2 * i + 1] *= corr; }
    }
    uint32_t pa[4][4];
#pragma unroll
    for (int mm = 0; mm < 4; ++mm) {
        pa[mm][0] = fm_pack(s[2 * mm][0], s[2 * mm][1]);
        pa[mm][1] = fm_pack(s[2 * mm][2], s[2 * mm][3]);
        pa[mm][2] = fm_pack(s[2 * mm + 1][0], s[2 * mm + 1][1]);
        pa[mm][3] = fm_pack(s[2 * mm + 1][2], s[2 * mm + 1][3]);
    }
    // likewise the output tiles, four at a time
#pragma unroll
    for (int half = 0; half < 2; ++half) {
#pragma unroll
        for (int n0 = 0; n0 < NT; n0 += 4) {
            uint4 vr[4];
#pragma unroll
            for (int n = 0; n < 4; ++n)
                if (n0 + n < NT) vr[n] = load_v(n0 + n, half);
#pragma unroll
            for (int n = 0; n < 4; ++n)
                if (n0 + n < NT) fm_mma(st.o[n0 + n], pa[2 * half][0], pa[2 * half][1], pa[2 * half][2], pa[2 * half][3], vr[n].x, vr[n].y);
#pragma unroll
            for (int n = 0; n < 4; ++n)
                if (n0 + n < NT) fm_mma(st.o[n0 + n], pa[2 * half + 1][0], pa[2 * half + 1][1], pa[2 * half + 1][2], pa[2 * half + 1][3], vr[n].z, vr[n].w);
        }
    }
}

struct FormArgs {
    const __nv_bfloat16 *q, *k_pool, *v_pool;
    const int* table;
    int table_width, pool_blocks;
    const __nv_bfloat16 *mean_k, *mean_v;       // the coarser cache (pooled blocks only)
    const int* mean_table;
    int mean_width, mean_blocks, every;
    const int *cu, *len_before;
    int sequences, heads, kv_heads, tokens_per_tile, cta_tiles, window, splits;
    float scale, cap, lambda, gain, eps;
    __nv_bfloat16* out;
    float *part_acc, *part_ml;
    unsigned* status;
};

template <int KD, int VD, int MAPS, bool POOLED, int TILES>
__global__ void __launch_bounds__(FormShape<KD, VD, MAPS, TILES>::THREADS)
form_kernel(const FormArgs a) {
    using S = FormShape<KD, VD, MAPS, TILES>;
    constexpr int KC = S::KC, NT = S::NT, STAGES = S::STAGES, ROW = MAPS * KD;
    extern __shared__ uint4 form_stage_mem[];                  // [STAGES][K tile, V tile]; at the end map 2's output
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int my_tile = warp & (TILES - 1), map = warp / TILES;
    const int kh = blockIdx.x;
    const int group = a.heads / a.kv_heads;
    const int tokens_per_cta = a.tokens_per_tile * TILES;

    // which sequence and which of its CTA tiles; late tiles of a sequence come first
    int tile = a.cta_tiles - 1 - (int)blockIdx.y;
    int b = -1;
    for (int base = 0; base < a.sequences && b < 0; base += 32) {
        const int mine = base + lane;
        const int count = mine < a.sequences ? (a.cu[mine + 1] - a.cu[mine] + tokens_per_cta - 1) / tokens_per_cta : 0;
        int prefix = count;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int up = __shfl_up_sync(0xffffffffu, prefix, o);
            if (lane >= o) prefix += up;
        }
        const unsigned owner = __ballot_sync(0xffffffffu, tile < prefix);
        if (owner) {
            const int first = __ffs(owner) - 1;
            b = base + first;
            tile -= __shfl_sync(0xffffffffu, prefix - count, first);
        } else {
            tile -= __shfl_sync(0xffffffffu, prefix, 31);
        }
    }
    if (b < 0) return;                 // a spare CTA (the grid is an upper bound): all its warps leave together
    const int seq_begin = a.cu[b], seq_new = a.cu[b + 1] - seq_begin, before = a.len_before[b];
    const int cta_tok0 = tile * tokens_per_cta;
    const int cta_tokens = min(tokens_per_cta, seq_new - cta_tok0);
    const int tok0 = cta_tok0 + my_tile * a.tokens_per_tile;
    const int tile_tokens = max(0, min(a.tokens_per_tile, seq_new - tok0));      // 0: the warp only helps copying

    // what a position sees: tokens first_of(p) .. p, and the entries 0 .. lead_of(p) - 1 of the coarser cache
    auto first_of = [&](int p) { return (POOLED && p - a.window + 1 > 0) ? p - a.window + 1 : 0; };
    auto lead_of = [&](int p) { return (POOLED && p - a.window + 1 > 0) ? (p - a.window + 1) / a.every : 0; };

    FormState<KD, VD> st;
    size_t row_at[2];                  // token * heads + head
    bool row_ok[2];
    int tok_lo[2], tok_hi[2], lead_hi[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = g + 8 * i;
        const int local = r / group;
        row_ok[i] = local < tile_tokens;
        row_at[i] = (size_t)(seq_begin + tok0 + local) * a.heads + kh * group + (r - local * group);
        const int pos = row_ok[i] ? before + tok0 + local : -1;
        tok_hi[i] = pos;
        tok_lo[i] = first_of(pos);
        lead_hi[i] = lead_of(pos) - 1;
    }
    {
        const uint4 zero4 = make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int c = 0; c < KC; ++c) {
            const uint4 va = row_ok[0] ? *reinterpret_cast<const uint4*>(a.q + row_at[0] * ROW + map * KD + 32 * c + 8 * t) : zero4;
            const uint4 vb = row_ok[1] ? *reinterpret_cast<const uint4*>(a.q + row_at[1] * ROW + map * KD + 32 * c + 8 * t) : zero4;
            st.qa[c][0] = va.x; st.qa[c][1] = va.y; st.qa[c][2] = va.z; st.qa[c][3] = va.w;
            st.qb[c][0] = vb.x; st.qb[c][1] = vb.y; st.qb[c][2] = vb.z; st.qb[c][3] = vb.w;
        }
        if constexpr (S::HALF) {
            const uint2 zero2 = make_uint2(0, 0);
            const uint2 va = row_ok[0] ? *reinterpret_cast<const uint2*>(a.q + row_at[0] * ROW + map * KD + 32 * KC + 4 * t) : zero2;
            const uint2 vb = row_ok[1] ? *reinterpret_cast<const uint2*>(a.q + row_at[1] * ROW + map * KD + 32 * KC + 4 * t) : zero2;
            st.qa[KC][0] = va.x; st.qa[KC][1] = va.y; st.qa[KC][2] = st.qa[KC][3] = 0;
            st.qb[KC][0] = vb.x; st.qb[KC][1] = vb.y; st.qb[KC][2] = st.qb[KC][3] = 0;
        }
#pragma unroll
        for (int n = 0; n < NT; ++n) { st.o[n][0] = st.o[n][1] = st.o[n][2] = st.o[n][3] = 0.0f; }
        st.m_run[0] = st.m_run[1] = -INFINITY;
        st.l_run[0] = st.l_run[1] = 0.0f;
    }

    // the CTA's list of blocks: those of the coarser cache that its last row sees, then the token blocks from the first one
    // any of its rows sees to its last row's; this CTA takes slice blockIdx.z of the list
    const int cta_lo = before + cta_tok0, cta_hi = before + cta_tok0 + cta_tokens - 1;
    const int n_coarse = (lead_of(cta_hi) + TT_BLOCK_TOKENS - 1) / TT_BLOCK_TOKENS;
    const int block0 = first_of(cta_lo) / TT_BLOCK_TOKENS, block1 = cta_hi / TT_BLOCK_TOKENS;
    const int n_items = n_coarse + block1 - block0 + 1;
    const int per = (n_items + a.splits - 1) / a.splits;
    const int item0 = min(n_items, (int)blockIdx.z * per), item1 = min(n_items, item0 + per);
    const int my_hi = tile_tokens > 0 ? before + tok0 + tile_tokens - 1 : -1;
    const int my_first = first_of(before + tok0), my_lead = tile_tokens > 0 ? lead_of(my_hi) : 0;
    const int* table_row = a.table + (size_t)b * a.table_width;
    const int* mean_row = POOLED ? a.mean_table + (size_t)b * a.mean_width : nullptr;
    uint8_t* stages = reinterpret_cast<uint8_t*>(form_stage_mem);
    unsigned bad = 0;                                            // bit i % 32: item i has no usable data

    auto issue = [&](int i) {                                    // all threads: copy item item0 + i into its stage
        const int item = item0 + i;
        if (item < item1) {
            const bool coarse = POOLED && item < n_coarse;
            const int block = coarse ? mean_row[item] : table_row[block0 + item - n_coarse];
            if (block >= 0 && block < (coarse ? a.mean_blocks : a.pool_blocks)) {
                const size_t at = (size_t)block * a.kv_heads + kh;
                const uint8_t* ksrc = reinterpret_cast<const uint8_t*>((coarse ? a.mean_k : a.k_pool) + at * TT_BLOCK_TOKENS * ROW);
                const uint8_t* vsrc = reinterpret_cast<const uint8_t*>((coarse ? a.mean_v : a.v_pool) + at * VD * TT_BLOCK_TOKENS);
                uint8_t* kdst = stages + (size_t)(i % STAGES) * S::STAGE;
                uint8_t* vdst = kdst + S::K_TILE;
                constexpr int K_CHUNKS = S::K_ROW / 16;          // 16-byte chunks per key row
                for (int c = threadIdx.x; c < S::K_TILE / 16; c += S::THREADS) {
                    const int row = c / K_CHUNKS, ch = c - row * K_CHUNKS;
                    const int to = S::K_SWIZZLE ? (ch ^ ((row & 1) << 2)) : ch;
                    fm_cp16(kdst + row * S::K_ROW + to * 16, ksrc + (size_t)c * 16);
                }
                for (int c = threadIdx.x; c < S::V_TILE / 16; c += S::THREADS) {
                    const int row = c >> 3, ch = c & 7;          // a value row is 64 tokens = 8 chunks
                    fm_cp16(vdst + row * 128 + ((ch ^ ((row & 1) << 2)) * 16), vsrc + (size_t)c * 16);
                }
                bad &= ~(1u << (i & 31));
            } else {
                bad |= 1u << (i & 31);
                if (threadIdx.x == 0) atomicOr(a.status, TT_STATUS_BAD_BLOCK);
            }
        }
        fm_commit();
    };

#pragma unroll
    for (int i = 0; i < STAGES - 1; ++i) issue(i);
    for (int i = 0; i < item1 - item0; ++i) {
        fm_wait<STAGES - 2>();                // this thread's copies of item i are done ...
        __syncthreads();                      // ... and so are everybody's; the stage of item i - 1 is free again
        issue(i + STAGES - 1);
        if ((bad >> (i & 31)) & 1u) continue;
        const int item = item0 + i;
        const bool coarse = POOLED && item < n_coarse;
        const int index_base = (coarse ? item : block0 + item - n_coarse) * TT_BLOCK_TOKENS;
        if (coarse) {
            if (index_base >= my_lead) continue;                                                  // nothing for this warp here
        } else if (index_base > my_hi || index_base + TT_BLOCK_TOKENS <= my_first) {
            continue;
        }
        const uint8_t* ktile = stages + (size_t)(i % STAGES) * S::STAGE;
        const uint8_t* vtile = ktile + S::K_TILE;
        const int lo[2] = {coarse ? 0 : tok_lo[0], coarse ? 0 : tok_lo[1]};
        const int hi[2] = {coarse ? lead_hi[0] : tok_hi[0], coarse ? lead_hi[1] : tok_hi[1]};
        form_block_math<KD, VD>(st, index_base, lo, hi, t, a.scale, a.cap,
                       [&](int j, int c) {
                           const int row = fm_key_of(j, g), ch = map * (KD / 8) + 4 * c + t;
                           const int at = S::K_SWIZZLE ? (ch ^ ((row & 1) << 2)) : ch;
                           return *reinterpret_cast<const uint4*>(ktile + row * S::K_ROW + at * 16);
                       },
                       [&](int j) {
                           const int row = fm_key_of(j, g), ch = map * (KD / 8) + 4 * KC + (t >> 1);
                           const int at = S::K_SWIZZLE ? (ch ^ ((row & 1) << 2)) : ch;
                           return *reinterpret_cast<const uint2*>(ktile + row * S::K_ROW + at * 16 + 8 * (t & 1));
                       },
                       [&](int n, int half) {
                           const int row = 8 * n + g, ch = 4 * half + t;
                           return *reinterpret_cast<const uint4*>(vtile + row * 128 + ((ch ^ ((row & 1) << 2)) * 16));
                       });
    }
    fm_wait<0>();

    // row sums live spread over the four threads of a quad
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        st.l_run[i] += __shfl_xor_sync(0xffffffffu, st.l_run[i], 1);
        st.l_run[i] += __shfl_xor_sync(0xffffffffu, st.l_run[i], 2);
    }

    if (a.splits > 1) {                 // this slice's (max, sum, accumulator) per row and map, for the merge kernel
        constexpr float LN2 = 0.6931471805599453f;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            if (!row_ok[i]) continue;
            const size_t slot = (row_at[i] * a.splits + blockIdx.z) * MAPS + map;
            float* acc = a.part_acc + slot * VD + 2 * t;
#pragma unroll
            for (int n = 0; n < NT; ++n) *reinterpret_cast<float2*>(acc + 8 * n) = make_float2(st.o[n][2 * i], st.o[n][2 * i + 1]);
            if (t == 0) *reinterpret_cast<float2*>(a.part_ml + slot * 2) = make_float2(st.m_run[i] * LN2, st.l_run[i]);
        }
        return;
    }

    float inv[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) inv[i] = st.l_run[i] > 0.0f ? 1.0f / st.l_run[i] : 0.0f;
    if constexpr (MAPS == 2) {
        __syncthreads();                // every warp is through with the stages
        float* exchange = reinterpret_cast<float*>(form_stage_mem) + (size_t)my_tile * 16 * VD;
        if (map == 1) {
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int n = 0; n < NT; ++n)
                    *reinterpret_cast<float2*>(exchange + (g + 8 * i) * VD + 8 * n + 2 * t) = make_float2(st.o[n][2 * i] * inv[i], st.o[n][2 * i + 1] * inv[i]);
        }
        __syncthreads();
        if (map == 1) return;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            float sumsq = 0.0f;
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                const float2 other = *reinterpret_cast<const float2*>(exchange + (g + 8 * i) * VD + 8 * n + 2 * t);
                st.o[n][2 * i] = st.o[n][2 * i] * inv[i] - a.lambda * other.x;
                st.o[n][2 * i + 1] = st.o[n][2 * i + 1] * inv[i] - a.lambda * other.y;
                sumsq += st.o[n][2 * i] * st.o[n][2 * i] + st.o[n][2 * i + 1] * st.o[n][2 * i + 1];
            }
            sumsq += __shfl_xor_sync(0xffffffffu, sumsq, 1);
            sumsq += __shfl_xor_sync(0xffffffffu, sumsq, 2);
            inv[i] = rsqrtf(sumsq / (float)VD + a.eps) * a.gain;
        }
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        if (!row_ok[i]) continue;
        __nv_bfloat16* dst = a.out + row_at[i] * VD + 2 * t;
#pragma unroll
        for (int n = 0; n < NT; ++n) *reinterpret_cast<uint32_t*>(dst + 8 * n) = fm_pack(st.o[n][2 * i] * inv[i], st.o[n][2 * i + 1] * inv[i]);
    }
}

// Whether the tensor-core kernel takes these sizes; the launcher below instantiates exactly these.
#define FM_DIFFERENTIAL_SHAPES(X) X(32, 64) X(48, 96) X(64, 128) X(64, 64) X(128, 128)
#define FM_POOLED_SHAPES(X) X(32) X(64) X(96) X(128)

template <int KD, int VD, int MAPS, bool POOLED, int TILES>
int form_launch_tiles(FormArgs a, int n_tokens, cudaStream_t stream) {
    using S = FormShape<KD, VD, MAPS, TILES>;
    auto kernel = form_kernel<KD, VD, MAPS, POOLED, TILES>;
    static bool configured = false;
    if (!configured) {
        const cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::SHARED);
        if (err != cudaSuccess) return (int)err;
        configured = true;
    }
    a.tokens_per_tile = 16 / (a.heads / a.kv_heads);
    const int tokens_per_cta = a.tokens_per_tile * TILES;
    a.cta_tiles = (n_tokens + tokens_per_cta - 1) / tokens_per_cta + a.sequences;       // upper bound; spare CTAs leave at once
    if (a.cta_tiles > 65535 || a.kv_heads > 65535 || a.splits > 65535) return (int)cudaErrorInvalidValue;
    return (int)tt_launch_pdl(kernel, dim3(a.kv_heads, a.cta_tiles, a.splits), dim3(S::THREADS), S::SHARED, stream, a);
}

template <int KD, int VD, int MAPS, bool POOLED>
int form_launch(const FormArgs& a, int n_tokens, cudaStream_t stream) {
    if (n_tokens == a.sequences) return form_launch_tiles<KD, VD, MAPS, POOLED, 1>(a, n_tokens, stream);     // one token a sequence
    return form_launch_tiles<KD, VD, MAPS, POOLED, 4>(a, n_tokens, stream);
}

// 0: done (or an error code); -1: sizes that the tensor-core kernel does not take
int form_differential(const FormArgs& a, int dim, int value_dim, int n_tokens, cudaStream_t stream) {
#define X(KD_, VD_) if (dim == KD_ && value_dim == VD_) return form_launch<KD_, VD_, 2, false>(a, n_tokens, stream);
    FM_DIFFERENTIAL_SHAPES(X)
#undef X
    return -1;
}
int form_pooled(const FormArgs& a, int head_dim, int n_tokens, cudaStream_t stream) {
#define X(HD_) if (head_dim == HD_) return form_launch<HD_, HD_, 1, true>(a, n_tokens, stream);
    FM_POOLED_SHAPES(X)
#undef X
    return -1;
}
}  // namespace

// Whether the tensor-core kernels take these sizes in bfloat16: maps != 0 asks about differential attention (dim numbers a
// map), maps == 0 about window attention with pooled blocks (value_dim == dim).
extern "C" int tt_attention_forms_on_tensor_cores(int maps, int heads, int kv_heads, int dim, int value_dim) {
    if (kv_heads <= 0 || heads % kv_heads || heads / kv_heads > 16) return 0;
#define X(KD_, VD_) if (maps && dim == KD_ && value_dim == VD_) return 1;
    FM_DIFFERENTIAL_SHAPES(X)
#undef X
#define X(HD_) if (!maps && dim == HD_ && value_dim == HD_) return 1;
    FM_POOLED_SHAPES(X)
#undef X
    return 0;
}

extern "C" int tt_differential_attention(const void* q, const void* k_pool, const void* v_pool, int dtype, const int* table,
                                         int table_width, int pool_blocks, const int* cu, const int* len_before, int sequences,
                                         int n_tokens, int heads, int kv_heads, int dim, int value_dim, float scale, float lambda,
                                         float gain, float eps, int splits, void* out, float* part_acc, float* part_ml,
                                         unsigned* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (dim <= 0 || 2 * dim > ATTN_MAX_HEAD_DIM || value_dim <= 0 || value_dim > ATTN_MAX_HEAD_DIM || kv_heads <= 0 || heads % kv_heads ||
        splits < 1 || splits > 65535)
        return (int)cudaErrorInvalidValue;
    if (splits > 1 && (!part_acc || !part_ml)) return (int)cudaErrorInvalidValue;
    const long long rows = (long long)n_tokens * heads;
    const dim3 grid((unsigned)((rows + ATTN_WARPS - 1) / ATTN_WARPS), (unsigned)splits);
    if (dtype == TT_BF16 && heads / kv_heads <= 16) {          // tensor cores, for the sizes they are built for
        FormArgs a = {};
        a.q = (const __nv_bfloat16*)q; a.k_pool = (const __nv_bfloat16*)k_pool; a.v_pool = (const __nv_bfloat16*)v_pool;
        a.table = table; a.table_width = table_width; a.pool_blocks = pool_blocks;
        a.cu = cu; a.len_before = len_before; a.sequences = sequences; a.heads = heads; a.kv_heads = kv_heads; a.splits = splits;
        a.scale = scale; a.lambda = lambda; a.gain = gain; a.eps = eps;
        a.out = (__nv_bfloat16*)out; a.part_acc = part_acc; a.part_ml = part_ml; a.status = status;
        const int code = form_differential(a, dim, value_dim, n_tokens, stream);
        if (code > 0) return code;
        if (code == 0) {
            if (splits > 1)
                tt_launch_pdl(differential_merge_kernel<__nv_bfloat16>, dim3(grid.x), dim3(ATTN_WARPS * 32), 0, stream, (const float*)part_acc, (const float*)part_ml, splits, value_dim, rows, lambda, gain, eps, (__nv_bfloat16*)out);
            TT_LAUNCH_CHECK();
        }
    }
    const size_t shared = (size_t)ATTN_WARPS * 2 * dim * sizeof(float);
    if (dtype == TT_F32) {
        tt_launch_pdl(differential_rows_kernel<float>, grid, dim3(ATTN_WARPS * 32), shared, stream, (const float*)q, (const float*)k_pool, (const float*)v_pool, table, table_width, pool_blocks, cu, len_before, sequences, n_tokens, heads, kv_heads, dim, value_dim, scale, lambda, gain, eps, splits, (float*)out, part_acc, part_ml, status);
        if (splits > 1)
            tt_launch_pdl(differential_merge_kernel<float>, dim3(grid.x), dim3(ATTN_WARPS * 32), 0, stream, (const float*)part_acc, (const float*)part_ml, splits, value_dim, rows, lambda, gain, eps, (float*)out);
    } else {
        tt_launch_pdl(differential_rows_kernel<__nv_bfloat16>, grid, dim3(ATTN_WARPS * 32), shared, stream, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, table, table_width, pool_blocks, cu, len_before, sequences, n_tokens, heads, kv_heads, dim, value_dim, scale, lambda, gain, eps, splits, (__nv_bfloat16*)out, part_acc, part_ml, status);
        if (splits > 1)
            tt_launch_pdl(differential_merge_kernel<__nv_bfloat16>, dim3(grid.x), dim3(ATTN_WARPS * 32), 0, stream, (const float*)part_acc, (const float*)part_ml, splits, value_dim, rows, lambda, gain, eps, (__nv_bfloat16*)out);
    }
    TT_LAUNCH_CHECK();
}

extern "C" int tt_pool_blocks(const void* k_pool, const void* v_pool, int dtype, const int* table, int table_width, int pool_blocks,
                              void* mean_k, void* mean_v, const int* mean_table, int mean_width, int mean_blocks, const int* cu,
                              const int* len_before, int sequences, int most_blocks, int kv_heads, int head_dim, int value_dim,
                              int every, unsigned* status, cudaStream_t stream) {
    if (sequences <= 0 || most_blocks <= 0) return 0;
    if (every <= 0 || head_dim <= 0 || value_dim <= 0 || kv_heads <= 0 || kv_heads > 65535 || sequences > 65535) return (int)cudaErrorInvalidValue;
    const dim3 grid((unsigned)most_blocks, (unsigned)kv_heads, (unsigned)sequences);
    const int threads = head_dim + value_dim > 128 ? 256 : 128;
    if (dtype == TT_F32)
        tt_launch_pdl(pool_blocks_kernel<float>, grid, dim3(threads), 0, stream, (const float*)k_pool, (const float*)v_pool, table, table_width, pool_blocks, (float*)mean_k, (float*)mean_v, mean_table, mean_width, mean_blocks, cu, len_before, kv_heads, head_dim, value_dim, every, status);
    else
        tt_launch_pdl(pool_blocks_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, table, table_width, pool_blocks, (__nv_bfloat16*)mean_k, (__nv_bfloat16*)mean_v, mean_table, mean_width, mean_blocks, cu, len_before, kv_heads, head_dim, value_dim, every, status);
    TT_LAUNCH_CHECK();
}

extern "C" int tt_pooled_window_attention(const void* q, const void* k_pool, const void* v_pool, int dtype, const int* table,
                                          int table_width, int pool_blocks, const void* mean_k, const void* mean_v,
                                          const int* mean_table, int mean_width, int mean_blocks, int every, const int* cu,
                                          const int* len_before, int sequences, int n_tokens, int heads, int kv_heads, int head_dim,
                                          float scale, float cap, int window, int splits, void* out, float* part_acc, float* part_ml,
                                          unsigned* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (head_dim <= 0 || head_dim > ATTN_MAX_HEAD_DIM || kv_heads <= 0 || heads % kv_heads || splits < 1 || splits > 65535 || window <= 0 || every <= 0)
        return (int)cudaErrorInvalidValue;
    if (splits > 1 && (!part_acc || !part_ml)) return (int)cudaErrorInvalidValue;
    const long long rows = (long long)n_tokens * heads;
    const dim3 grid((unsigned)((rows + ATTN_WARPS - 1) / ATTN_WARPS), (unsigned)splits);
    if (dtype == TT_BF16 && heads / kv_heads <= 16) {          // tensor cores, for the sizes they are built for
        FormArgs a = {};
        a.q = (const __nv_bfloat16*)q; a.k_pool = (const __nv_bfloat16*)k_pool; a.v_pool = (const __nv_bfloat16*)v_pool;
        a.table = table; a.table_width = table_width; a.pool_blocks = pool_blocks;
        a.mean_k = (const __nv_bfloat16*)mean_k; a.mean_v = (const __nv_bfloat16*)mean_v; a.mean_table = mean_table;
        a.mean_width = mean_width; a.mean_blocks = mean_blocks; a.every = every; a.window = window;
        a.cu = cu; a.len_before = len_before; a.sequences = sequences; a.heads = heads; a.kv_heads = kv_heads; a.splits = splits;
        a.scale = scale; a.cap = cap;
        a.out = (__nv_bfloat16*)out; a.part_acc = part_acc; a.part_ml = part_ml; a.status = status;
        const int code = form_pooled(a, head_dim, n_tokens, stream);
        if (code > 0) return code;
        if (code == 0) {
            if (splits > 1)
                tt_launch_pdl(attention_merge_kernel<__nv_bfloat16>, dim3(grid.x), dim3(ATTN_WARPS * 32), 0, stream, (const float*)part_acc, (const float*)part_ml, splits, head_dim, rows, (__nv_bfloat16*)out, AttnExtra{}, heads);
            TT_LAUNCH_CHECK();
        }
    }
    const size_t shared = (size_t)ATTN_WARPS * head_dim * sizeof(float);
    if (dtype == TT_F32) {
        tt_launch_pdl(pooled_window_rows_kernel<float>, grid, dim3(ATTN_WARPS * 32), shared, stream, (const float*)q, (const float*)k_pool, (const float*)v_pool, table, table_width, pool_blocks, (const float*)mean_k, (const float*)mean_v, mean_table, mean_width, mean_blocks, every, cu, len_before, sequences, n_tokens, heads, kv_heads, head_dim, scale, cap, window, splits, (float*)out, part_acc, part_ml, status);
        if (splits > 1)
            tt_launch_pdl(attention_merge_kernel<float>, dim3(grid.x), dim3(ATTN_WARPS * 32), 0, stream, (const float*)part_acc, (const float*)part_ml, splits, head_dim, rows, (float*)out, AttnExtra{}, heads);
    } else {
        tt_launch_pdl(pooled_window_rows_kernel<__nv_bfloat16>, grid, dim3(ATTN_WARPS * 32), shared, stream, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, table, table_width, pool_blocks, (const __nv_bfloat16*)mean_k, (const __nv_bfloat16*)mean_v, mean_table, mean_width, mean_blocks, every, cu, len_before, sequences, n_tokens, heads, kv_heads, head_dim, scale, cap, window, splits, (__nv_bfloat16*)out, part_acc, part_ml, status);
        if (splits > 1)
            tt_launch_pdl(attention_merge_kernel<__nv_bfloat16>, dim3(grid.x), dim3(ATTN_WARPS * 32), 0, stream, (const float*)part_acc, (const float*)part_ml, splits, head_dim, rows, (__nv_bfloat16*)out, AttnExtra{}, heads);
    }
    TT_LAUNCH_CHECK();
}
