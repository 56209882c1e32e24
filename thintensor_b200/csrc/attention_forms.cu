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
    for (int d = threadIdx.x; d < head_dim + value_dim; d += blockDim.x) {
        float sum = 0.0f;
        for (int j = 0; j < every; ++j) {
            const int position = n * every + j;
            if (d < head_dim) {
                const long long off = tt_cache_offset(table_row, position, kh, kv_heads, head_dim, pool_blocks, status);
                if (off >= 0) sum += tt_to_float(k_pool[off + d]);
            } else {
                const long long off = tt_value_offset(table_row, position, kh, kv_heads, value_dim, pool_blocks, status);
                if (off >= 0) sum += tt_to_float(v_pool[off + (long long)(d - head_dim) * TT_BLOCK_TOKENS]);
            }
        }
        if (d < head_dim) mean_k[k_dst + d] = tt_from_float<T>(sum * share);
        else mean_v[v_dst + (long long)(d - head_dim) * TT_BLOCK_TOKENS] = tt_from_float<T>(sum * share);
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

}  // namespace

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
    const size_t shared = (size_t)ATTN_WARPS * head_dim * sizeof(float);
    if (dtype == TT_F32) {
        tt_launch_pdl(pooled_window_rows_kernel<float>, grid, dim3(ATTN_WARPS * 32), shared, stream, (const float*)q, (const float*)k_pool, (const float*)v_pool, table, table_width, pool_blocks, (const float*)mean_k, (const float*)mean_v, mean_table, mean_width, mean_blocks, every, cu, len_before, sequences, n_tokens, heads, kv_heads, head_dim, scale, cap, window, splits, (float*)out, part_acc, part_ml, status);
        if (splits > 1)
            tt_launch_pdl(attention_merge_kernel<float>, dim3(grid.x), dim3(ATTN_WARPS * 32), 0, stream, (const float*)part_acc, (const float*)part_ml, splits, head_dim, rows, (float*)out);
    } else {
        tt_launch_pdl(pooled_window_rows_kernel<__nv_bfloat16>, grid, dim3(ATTN_WARPS * 32), shared, stream, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, table, table_width, pool_blocks, (const __nv_bfloat16*)mean_k, (const __nv_bfloat16*)mean_v, mean_table, mean_width, mean_blocks, every, cu, len_before, sequences, n_tokens, heads, kv_heads, head_dim, scale, cap, window, splits, (__nv_bfloat16*)out, part_acc, part_ml, status);
        if (splits > 1)
            tt_launch_pdl(attention_merge_kernel<__nv_bfloat16>, dim3(grid.x), dim3(ATTN_WARPS * 32), 0, stream, (const float*)part_acc, (const float*)part_ml, splits, head_dim, rows, (__nv_bfloat16*)out);
    }
    TT_LAUNCH_CHECK();
}
