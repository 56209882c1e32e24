// Softmax attention over a compressed latent: the cache holds, per token, ONE row of `rank` latent numbers
// followed by `rot` rotated key numbers that all heads share ([block][1][TT_BLOCK_TOKENS][rank + rot], no value
// pool).  A head's keys and values are linear maps of the latent (k_h = Wk_h c, v_h = Wv_h c), so neither is ever
// formed: with a_h = Wk_h^T q_h the score is (a_h . c + q_rot_h . k_rot) * scale, and the head's output is
// Wv_h (sum_j p_j c_j).  Scores, softmax weights, norms, positions and angles are float32 in both dtypes.
//
// tt_latent_prepare: one block per token.  Sums the k-slices of the down projection [q latent | kv latent | k_rot],
// divides the two latents by their root mean square (times their weights), writes the query latent for the
// up projection, rotates k_rot by the token's position and appends [c | k_rot] to the token's cache row.  A layer whose
// queries are projected directly has no query latent (q_rank 0); a token's row of the projection may hold more columns
// behind these (row_stride).  The rotation pairs halves or, interleaved, neighbours; rot_scale multiplies cosine and sine.
//
// tt_latent_attention: three kernels.  (1) A block per (token, head) sums the slices of the head's query, rotates its
// rotated part and forms a_h, threads across the latent.  (2) A warp per (token, head) and slice of the keys: a lane per
// key of a tile of 32 (16-byte loads along the row), online softmax, the weighted latents accumulated with every lane
// taking 16 bytes of a latent at a time; the slice leaves (sum, maximum, denominator) in scratch memory.  (3) A block per
// (token, head) combines the slices in order and applies Wv_h, a warp per output number, and multiplies the head by the
// sigmoid of its gate number where the layer has one.
//
// Prompts may instead EXPAND the latents they can see into per-head keys and values for the step, laid out like blocks
// of the ordinary cache (keys [block][head][64][dim + rot], values transposed [block][head][vdim][64]) with a table of
// their own, so that the tensor-core attention kernels for ordinary heads run on them:
// tt_latent_expand_plan (which blocks of which sequence the step can see, and where they go), tt_latent_gather (their
// latents into one matrix for the product with [Wk; Wv], their shared rotated parts into every head's keys),
// tt_latent_scatter (the product's rows into keys and transposed values) and tt_latent_queries (rotated queries).
#include <mma.h>

#include "attention_kernels.cuh"

constexpr int LAT_WARPS = 4;
constexpr int LAT_MAX_RANK = 512;       // numbers of the latent (a lane accumulates LAT_MAX_RANK / 32 of them)
constexpr int LAT_MAX_ROW = 1024;       // rank + rot
constexpr int LAT_MAX_DIM = 256;        // unrotated numbers of a head's query

// Number j of a rotated part `part` (rotary_dim numbers rotate, the rest pass): its pair is j + half / j - half, or with
// `interleaved` its neighbour j ^ 1 (pair index j / 2); cosine and sine are multiplied by rot_scale.
__device__ __forceinline__ float lat_rotate(const float* __restrict__ part, int j, int rotary_dim, int interleaved, int pos,
                                            const float* __restrict__ inv_freq, float rot_scale) {
    if (j >= rotary_dim) return part[j];
    const int half = rotary_dim >> 1;
    const bool first = interleaved ? !(j & 1) : j < half;
    const int pair = interleaved ? (j ^ 1) : (first ? j + half : j - half);
    const int i = interleaved ? (j >> 1) : (first ? j : j - half);
    float sn, cs;
    sincosf((float)pos * __ldg(inv_freq + i), &sn, &cs);
    sn *= rot_scale; cs *= rot_scale;
    return first ? part[j] * cs - part[pair] * sn : part[j] * cs + part[pair] * sn;
}

template <typename TOut, typename TC>
__global__ void latent_prepare_kernel(const float* __restrict__ down, int splits, size_t split_stride, int row_stride, int q_rank, int rank,
                                      int rot, const float* __restrict__ q_weight, const float* __restrict__ kv_weight, float eps,
                                      const float* __restrict__ inv_freq, int rotary_dim, int interleaved, float rot_scale,
                                      TOut* __restrict__ q_latent,
                                      TC* __restrict__ pool, const int* __restrict__ table, int table_width, int pool_blocks,
                                      const int* __restrict__ cu, const int* __restrict__ len_before, int sequences,
                                      unsigned* status) {
    tt_pdl_launch_dependents();
    const int t = blockIdx.x;
    const int b = tt_find_sequence(cu, sequences, t);           // the step's integers are written by no kernel of the step
    const int pos = len_before[b] + (t - cu[b]);
    tt_pdl_wait();
    extern __shared__ float lat_row[];                          // q_rank + rank + rot numbers, then 32 for the reductions
    const int cols = q_rank + rank + rot;
    float* reduce = lat_row + cols;
    const float* src = down + (size_t)t * row_stride;
    float sq_q = 0.0f, sq_c = 0.0f;
    for (int j = threadIdx.x; j < cols; j += blockDim.x) {
        float x = 0.0f;
        for (int s = 0; s < splits; ++s) x += src[(size_t)s * split_stride + j];
        lat_row[j] = x;
        if (j < q_rank) sq_q = fmaf(x, x, sq_q);
        else if (j < q_rank + rank) sq_c = fmaf(x, x, sq_c);
    }
    const float r_q = q_rank > 0 ? rsqrtf(tt_block_sum(sq_q, reduce) / (float)q_rank + eps) : 0.0f;
    const float r_c = rsqrtf(tt_block_sum(sq_c, reduce) / (float)rank + eps);
    for (int j = threadIdx.x; j < q_rank; j += blockDim.x)
        q_latent[(size_t)t * q_rank + j] = tt_from_float<TOut>(lat_row[j] * r_q * __ldg(q_weight + j));
    if (!pool) return;
    const long long off = tt_cache_offset(table + (size_t)b * table_width, pos, 0, 1, rank + rot, pool_blocks, status);
    if (off < 0) return;
    TC* row = pool + off;
    const float* c = lat_row + q_rank;
    for (int j = threadIdx.x; j < rank; j += blockDim.x) row[j] = tt_from_float<TC>(c[j] * r_c * __ldg(kv_weight + j));
    const float* kr = c + rank;
    for (int j = threadIdx.x; j < rot; j += blockDim.x)
        row[rank + j] = tt_from_float<TC>(lat_rotate(kr, j, rotary_dim, interleaved, pos, inv_freq, rot_scale));
}

template <typename T> __device__ __forceinline__ float lat_weight(const T* p) { return tt_to_float(*p); }

// 16 bytes of a cache row as floats: N numbers
template <typename T> struct LatVec;
template <> struct LatVec<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
        const float4 x = *reinterpret_cast<const float4*>(p);
        v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
    }
};
template <> struct LatVec<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
        const uint4 raw = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(h[i]);
            v[2 * i] = f.x; v[2 * i + 1] = f.y;
        }
    }
};

// The query a head's scores are taken with, one block per (token, head): [Wk_h^T q_plain | rotated q_rot] * scale, float32
// [tokens][heads][rank + rot].  Threads run across the latent, so that a row of Wk_h is read side by side.
template <typename TW>
__global__ void latent_absorb_kernel(const float* __restrict__ q, int q_splits, size_t q_stride, int q_row, const TW* __restrict__ w_key,
                                     const int* __restrict__ cu, const int* __restrict__ len_before, int sequences, int heads, int dim,
                                     int rot, int rank, const float* __restrict__ inv_freq, int rotary_dim, int interleaved,
                                     float rot_scale, float scale, float* __restrict__ absorbed) {
    tt_pdl_launch_dependents();
    const int t = blockIdx.x / heads, h = blockIdx.x - t * heads;
    int pos = 0;
    if (rotary_dim > 0) {
        const int b = tt_find_sequence(cu, sequences, t);
        pos = len_before[b] + (t - cu[b]);
    }
    tt_pdl_wait();
    extern __shared__ float lat_shared[];                       // dim + rot
    const float* qsrc = q + (size_t)t * q_row + (size_t)h * (dim + rot);
    for (int d = threadIdx.x; d < dim + rot; d += blockDim.x) {
        float x = 0.0f;
        for (int s = 0; s < q_splits; ++s) x += qsrc[(size_t)s * q_stride + d];
        lat_shared[d] = x;
    }
    __syncthreads();
    float* out = absorbed + ((size_t)t * heads + h) * (rank + rot);
    const float* qr = lat_shared + dim;
    for (int i = threadIdx.x; i < rot; i += blockDim.x)
        out[rank + i] = lat_rotate(qr, i, rotary_dim, interleaved, pos, inv_freq, rot_scale) * scale;
    for (int r = threadIdx.x; r < rank; r += blockDim.x) {
        const TW* col = w_key + (size_t)h * dim * rank + r;
        float a[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) a[i] = 0.0f;
        int d = 0;
        for (; d + 8 <= dim; d += 8) {                          // eight loads in flight, eight sums that do not wait for each other
            float w[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) w[i] = lat_weight(col + (size_t)(d + i) * rank);
#pragma unroll
            for (int i = 0; i < 8; ++i) a[i] = fmaf(w[i], lat_shared[d + i], a[i]);
        }
        for (; d < dim; ++d) a[0] = fmaf(lat_weight(col + (size_t)d * rank), lat_shared[d], a[0]);
        out[r] = (((a[0] + a[1]) + (a[2] + a[3])) + ((a[4] + a[5]) + (a[6] + a[7]))) * scale;
    }
}

// a cache row times the folded query: 16 bytes a load, four loads asked for before their products
template <typename TC>
__device__ __forceinline__ float lat_dot(const TC* __restrict__ row, const float* __restrict__ q, int n) {
    constexpr int VEC = LatVec<TC>::N;
    if (n % VEC) return dot16<TC>(row, q, n);
    float s0 = 0.0f, s1 = 0.0f;
    int d = 0;
    for (; d + 4 * VEC <= n; d += 4 * VEC) {
        float v[4][VEC];
#pragma unroll
        for (int i = 0; i < 4; ++i) LatVec<TC>::load(row + d + i * VEC, v[i]);
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
                if (i & 1) s1 = fmaf(v[i][e], q[d + i * VEC + e], s1); else s0 = fmaf(v[i][e], q[d + i * VEC + e], s0);
            }
    }
    for (; d < n; d += VEC) {
        float v[VEC];
        LatVec<TC>::load(row + d, v);
#pragma unroll
        for (int e = 0; e < VEC; ++e) s0 = fmaf(v[e], q[d + e], s0);
    }
    return s0 + s1;
}

// One warp per (token, head) and key slice.  window <= 0: all keys 0..pos.  window > 0: keys pos - window + 1 .. pos.
// Leaves the slice's weighted sum of latents, maximum and denominator in part_acc / part_ml.
template <typename TC>
__global__ void latent_attention_kernel(const float* __restrict__ absorbed, const TC* __restrict__ pool, const int* __restrict__ table,
                                        int table_width, int pool_blocks, const int* __restrict__ cu,
                                        const int* __restrict__ len_before, int sequences, int n_tokens, int heads, int rot, int rank,
                                        int window, int splits, float* __restrict__ part_acc, float* __restrict__ part_ml,
                                        unsigned* status) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    extern __shared__ float lat_shared[];                       // per warp: rank + rot (the absorbed query)
    constexpr int VEC = LatVec<TC>::N, CHUNKS = LAT_MAX_RANK / VEC / 32;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * LAT_WARPS + warp;   // (token, head)
    if (item >= (long long)n_tokens * heads) return;
    const int t = (int)(item / heads);
    const int split = blockIdx.y;
    const int b = tt_find_sequence(cu, sequences, t);
    const int pos = len_before[b] + (t - cu[b]);
    const int* table_row = table + (size_t)b * table_width;
    const int row_len = rank + rot;
    float* qa = lat_shared + (size_t)warp * row_len;
    const float* src = absorbed + (size_t)item * row_len;
    for (int d = lane; d < row_len; d += 32) qa[d] = src[d];
    __syncwarp();

    const int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int n_keys = pos - first + 1;
    int per = (n_keys + splits - 1) / splits;
    per = (per + 31) & ~31;
    const int begin = first + split * per;
    const int end = min(begin + per, pos + 1);
    const bool vec = (rank % VEC) == 0 && (row_len % VEC) == 0;  // a lane takes 16 bytes of a latent at a time

    float acc[CHUNKS][VEC];                                     // vec: numbers (lane + 32 c) * VEC + e; else lane + 32 (c * VEC + e)
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c)
#pragma unroll
        for (int e = 0; e < VEC; ++e) acc[c][e] = 0.0f;
    float m_run = -INFINITY, l_run = 0.0f;
    for (int base = begin; base < end; base += 32) {
        const int key = base + lane;
        long long off = -1;
        float score = -INFINITY;
        if (key < end) {
            off = tt_cache_offset(table_row, key, 0, 1, row_len, pool_blocks, status);
            if (off >= 0) score = lat_dot<TC>(pool + off, qa, row_len);
        }
        const float m_tile = tt_warp_max(score);
        if (m_tile == -INFINITY) continue;
        const float m_new = fmaxf(m_run, m_tile);
        const float corr = expf(m_run - m_new);
        const float p = (score == -INFINITY) ? 0.0f : expf(score - m_new);
        l_run = l_run * corr + tt_warp_sum(p);
        m_run = m_new;
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c)
#pragma unroll
            for (int e = 0; e < VEC; ++e) acc[c][e] *= corr;
        const int count = min(32, end - base);
        for (int j = 0; j < count; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            const long long oj = __shfl_sync(0xffffffffu, off, j);
            if (oj < 0) continue;
            const TC* crow = pool + oj;                         // the key's latent is also its value
            if (vec) {
#pragma unroll
                for (int c = 0; c < CHUNKS; ++c) {
                    const int r = (lane + 32 * c) * VEC;
                    if (r < rank) {
                        float v[VEC];
                        LatVec<TC>::load(crow + r, v);
#pragma unroll
                        for (int e = 0; e < VEC; ++e) acc[c][e] = fmaf(pj, v[e], acc[c][e]);
                    }
                }
            } else {
#pragma unroll
                for (int c = 0; c < CHUNKS; ++c)
#pragma unroll
                    for (int e = 0; e < VEC; ++e) {
                        const int r = lane + 32 * (c * VEC + e);
                        if (r < rank) acc[c][e] = fmaf(pj, tt_to_float(crow[r]), acc[c][e]);
                    }
            }
        }
    }
    const size_t slot = (size_t)item * splits + split;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c)
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
            const int r = vec ? (lane + 32 * c) * VEC + e : lane + 32 * (c * VEC + e);
            if (r < rank) part_acc[slot * rank + r] = acc[c][e];
        }
    if (lane == 0) {
        part_ml[slot * 2] = m_run;
        part_ml[slot * 2 + 1] = l_run;
    }
}

// The same for rows of whole 16-byte pieces (rank and rank + rot multiples of LatVec<TC>::N): the lanes of a warp lie ACROSS
// a cache row, lane l holding pieces l, l + 32, ... of it, so a key is three or four loads of 512 contiguous bytes for the
// warp (a lane per key read 32 different lines with every load), and the pieces that make the score are the pieces that
// are accumulated as the value.  Four keys are taken together: their loads are in flight at once, their scores are summed
// over the lanes side by side, and the running maximum moves once for the four.
template <typename TC>
__global__ void latent_attention_rows_kernel(const float* __restrict__ absorbed, const TC* __restrict__ pool,
                                             const int* __restrict__ table, int table_width, int pool_blocks,
                                             const int* __restrict__ cu, const int* __restrict__ len_before, int sequences,
                                             int n_tokens, int heads, int rot, int rank, int window, int splits,
                                             float* __restrict__ part_acc, float* __restrict__ part_ml, unsigned* status) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    constexpr int VEC = LatVec<TC>::N, ROW_PIECES = LAT_MAX_ROW / VEC / 32, VAL_PIECES = LAT_MAX_RANK / VEC / 32, KEYS = 4;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * LAT_WARPS + warp;   // (token, head)
    if (item >= (long long)n_tokens * heads) return;
    const int t = (int)(item / heads);
    const int split = blockIdx.y;
    const int b = tt_find_sequence(cu, sequences, t);
    const int pos = len_before[b] + (t - cu[b]);
    const int* table_row = table + (size_t)b * table_width;
    const int row_len = rank + rot;
    float qa[ROW_PIECES][VEC];                                  // this lane's pieces of the folded query
    const float* src = absorbed + (size_t)item * row_len;
#pragma unroll
    for (int c = 0; c < ROW_PIECES; ++c) {
        const int r = (lane + 32 * c) * VEC;
#pragma unroll
        for (int e = 0; e < VEC; ++e) qa[c][e] = r < row_len ? src[r + e] : 0.0f;
    }
    const int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int n_keys = pos - first + 1;
    int per = (n_keys + splits - 1) / splits;
    per = (per + 31) & ~31;
    const int begin = first + split * per;
    const int end = min(begin + per, pos + 1);

    float acc[VAL_PIECES][VEC];
#pragma unroll
    for (int c = 0; c < VAL_PIECES; ++c)
#pragma unroll
        for (int e = 0; e < VEC; ++e) acc[c][e] = 0.0f;
    float m_run = -INFINITY, l_run = 0.0f;
    for (int base = begin; base < end; base += KEYS) {
        float v[KEYS][VAL_PIECES][VEC];                         // the latent pieces stay for the value sum
        float score[KEYS];
        bool live[KEYS];
#pragma unroll
        for (int k = 0; k < KEYS; ++k) {
            const int key = base + k;
            long long off = -1;
            if (key < end) off = tt_cache_offset(table_row, key, 0, 1, row_len, pool_blocks, status);
            live[k] = off >= 0;
            float s = 0.0f;
#pragma unroll
            for (int c = 0; c < ROW_PIECES; ++c) {
                const int r = (lane + 32 * c) * VEC;
                float piece[VEC];
#pragma unroll
                for (int e = 0; e < VEC; ++e) piece[e] = 0.0f;
                if (live[k] && r < row_len) LatVec<TC>::load(pool + off + r, piece);
#pragma unroll
                for (int e = 0; e < VEC; ++e) s = fmaf(piece[e], qa[c][e], s);
                if (c < VAL_PIECES) {
#pragma unroll
                    for (int e = 0; e < VEC; ++e) v[k][c][e] = r < rank ? piece[e] : 0.0f;
                }
            }
            score[k] = s;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int k = 0; k < KEYS; ++k) score[k] += __shfl_xor_sync(0xffffffffu, score[k], o);
        float m_new = m_run;
#pragma unroll
        for (int k = 0; k < KEYS; ++k)
            if (live[k]) m_new = fmaxf(m_new, score[k]);
        if (m_new == -INFINITY) continue;
        const float corr = expf(m_run - m_new);                 // 0 before the first key
        float p[KEYS];
        float sum = 0.0f;
#pragma unroll
        for (int k = 0; k < KEYS; ++k) {
            p[k] = live[k] ? expf(score[k] - m_new) : 0.0f;
            sum += p[k];
        }
        l_run = l_run * corr + sum;
        m_run = m_new;
#pragma unroll
        for (int c = 0; c < VAL_PIECES; ++c)
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
                float a = acc[c][e] * corr;
#pragma unroll
                for (int k = 0; k < KEYS; ++k) a = fmaf(p[k], v[k][c][e], a);
                acc[c][e] = a;
            }
    }
    const size_t slot = (size_t)item * splits + split;
#pragma unroll
    for (int c = 0; c < VAL_PIECES; ++c)
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
            const int r = (lane + 32 * c) * VEC + e;
            if (r < rank) part_acc[slot * rank + r] = acc[c][e];
        }
    if (lane == 0) {
        part_ml[slot * 2] = m_run;
        part_ml[slot * 2 + 1] = l_run;
    }
}

// Decoding on the tensor cores (bfloat16 caches whose rows are whole pieces of 16 numbers): one CTA per (sequence, slice
// of LT_KEYS keys, group of 16 heads).  All heads of a token read the same cache rows, so the heads are the 16 rows of the
// products: S [heads x keys] = A [heads x (rank + rot)] K^T with A the folded queries, then O [heads x rank] = P C with C
// the latent part of the same rows.  The slice's rows and the folded queries are staged in shared memory once and serve
// both products; the slice's maximum is known before the second product, so nothing is rescaled.  Every warp takes 16 of
// the keys in the first product and every fourth 16-column piece of the latent in the second (warp-level
// mma.sync through the wmma interface).  Slices are combined by latent_merge_expand_kernel.
constexpr int LT_KEYS = 64, LT_HEADS = 16, LT_S_LD = LT_KEYS + 4, LT_P_LD = LT_KEYS + 8, LT_O_LD = 20;

static size_t latent_decode_shared(int row_len) {
    return (size_t)(LT_HEADS + LT_KEYS) * (row_len + 8) * sizeof(__nv_bfloat16) + (size_t)LT_HEADS * LT_S_LD * sizeof(float) +
           (size_t)LT_HEADS * LT_P_LD * sizeof(__nv_bfloat16) + (size_t)4 * LT_HEADS * LT_O_LD * sizeof(float);
}

__global__ void __launch_bounds__(128)
latent_decode_mma_kernel(const float* __restrict__ absorbed, const __nv_bfloat16* __restrict__ pool, const int* __restrict__ table,
                         int table_width, int pool_blocks, const int* __restrict__ len_before, int heads, int rot, int rank,
                         int window, int splits, float* __restrict__ part_acc, float* __restrict__ part_ml, unsigned* status) {
    using namespace nvcuda;
    tt_pdl_launch_dependents();
    extern __shared__ __align__(128) unsigned char lat_bytes[];
    const int row_len = rank + rot, ld = row_len + 8;           // rows 16 bytes apart modulo 128: no bank is met twice
    __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(lat_bytes);               // [16][ld]
    __nv_bfloat16* k_s = q_s + LT_HEADS * ld;                                       // [64][ld]
    float* s_s = reinterpret_cast<float*>(k_s + LT_KEYS * ld);                      // [16][LT_S_LD]
    __nv_bfloat16* p_s = reinterpret_cast<__nv_bfloat16*>(s_s + LT_HEADS * LT_S_LD);  // [16][LT_P_LD]
    float* o_s = reinterpret_cast<float*>(p_s + LT_HEADS * LT_P_LD);                // [4][16][LT_O_LD]
    const int t = blockIdx.x, split = blockIdx.y, h0 = blockIdx.z * LT_HEADS;       // one token per sequence: token t is sequence t
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pos = len_before[t];
    const int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int begin = first + split * LT_KEYS;
    const int end = min(begin + LT_KEYS, pos + 1);
    const int* table_row = table + (size_t)t * table_width;
    const int pieces = row_len >> 3;                            // 16-byte pieces of a row
    tt_pdl_wait();
    // the slice's rows: asynchronous 16-byte copies, all of a thread's in flight together (one after the other they cost a
    // round trip to the L2 each: 36 of them for a row of 576 numbers)
    for (int e = threadIdx.x; e < LT_KEYS * pieces; e += blockDim.x) {
        const int r = e / pieces, c = e - r * pieces;
        long long off = -1;
        if (begin + r < end) off = tt_cache_offset(table_row, begin + r, 0, 1, row_len, pool_blocks, status);
        __nv_bfloat16* dst = k_s + r * ld + 8 * c;
        if (off >= 0) {
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(pool + off + 8 * c) : "memory");
        } else {
            *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
        }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    // the folded queries: eight 16-byte loads asked for before the first is narrowed
    const int quads = row_len >> 2;
    for (int e0 = threadIdx.x; e0 < LT_HEADS * quads; e0 += 8 * blockDim.x) {
        float4 v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int e = e0 + i * blockDim.x, r = e / quads, c = e - r * quads;
            v[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (e < LT_HEADS * quads && h0 + r < heads)
                v[i] = *reinterpret_cast<const float4*>(absorbed + ((size_t)t * heads + h0 + r) * row_len + 4 * c);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int e = e0 + i * blockDim.x, r = e / quads, c = e - r * quads;
            if (e < LT_HEADS * quads) {
                __nv_bfloat162* dst = reinterpret_cast<__nv_bfloat162*>(q_s + r * ld + 4 * c);
                dst[0] = __floats2bfloat162_rn(v[i].x, v[i].y);
                dst[1] = __floats2bfloat162_rn(v[i].z, v[i].w);
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    {   // S = A K^T: this warp's 16 keys
        wmma::fragment<wmma::accumulator, 16, 16, 16, float> acc;
        wmma::fill_fragment(acc, 0.0f);
        for (int k = 0; k < row_len; k += 16) {
            wmma::fragment<wmma::matrix_a, 16, 16, 16, __nv_bfloat16, wmma::row_major> a;
            wmma::fragment<wmma::matrix_b, 16, 16, 16, __nv_bfloat16, wmma::col_major> b;
            wmma::load_matrix_sync(a, q_s + k, ld);
            wmma::load_matrix_sync(b, k_s + (16 * warp) * ld + k, ld);
            wmma::mma_sync(acc, a, b, acc);
        }
        wmma::store_matrix_sync(s_s + 16 * warp, acc, LT_S_LD, wmma::mem_row_major);
    }
    __syncthreads();
    for (int r = 4 * warp; r < 4 * warp + 4; ++r) {            // softmax of a head's row over the slice, float32
        const float s0 = begin + lane < end ? s_s[r * LT_S_LD + lane] : -INFINITY;
        const float s1 = begin + lane + 32 < end ? s_s[r * LT_S_LD + lane + 32] : -INFINITY;
        const float m = tt_warp_max(fmaxf(s0, s1));
        const float p0 = s0 == -INFINITY ? 0.0f : expf(s0 - m), p1 = s1 == -INFINITY ? 0.0f : expf(s1 - m);
        const float l = tt_warp_sum(p0 + p1);
        p_s[r * LT_P_LD + lane] = __float2bfloat16_rn(p0);
        p_s[r * LT_P_LD + lane + 32] = __float2bfloat16_rn(p1);
        if (lane == 0 && h0 + r < heads) {
            const size_t slot = ((size_t)t * heads + h0 + r) * splits + split;
            part_ml[slot * 2] = m;
            part_ml[slot * 2 + 1] = l;
        }
    }
    __syncthreads();
    float* mine = o_s + warp * LT_HEADS * LT_O_LD;
    for (int f = warp; f < (rank >> 4); f += 4) {               // O = P C: 16 columns of the latent at a time
        wmma::fragment<wmma::accumulator, 16, 16, 16, float> acc;
        wmma::fill_fragment(acc, 0.0f);
#pragma unroll
        for (int kk = 0; kk < LT_KEYS; kk += 16) {
            wmma::fragment<wmma::matrix_a, 16, 16, 16, __nv_bfloat16, wmma::row_major> a;
            wmma::fragment<wmma::matrix_b, 16, 16, 16, __nv_bfloat16, wmma::row_major> b;
            wmma::load_matrix_sync(a, p_s + kk, LT_P_LD);
            wmma::load_matrix_sync(b, k_s + kk * ld + 16 * f, ld);
            wmma::mma_sync(acc, a, b, acc);
        }
        wmma::store_matrix_sync(mine, acc, LT_O_LD, wmma::mem_row_major);
        __syncwarp();
        for (int e = lane; e < LT_HEADS * 16; e += 32) {
            const int r = e >> 4, c = e & 15;
            if (h0 + r < heads) part_acc[(((size_t)t * heads + h0 + r) * splits + split) * rank + 16 * f + c] = mine[r * LT_O_LD + c];
        }
        __syncwarp();
    }
}

// One block per (token, head): combines the key slices in slice order into the normalised sum of latents, then a warp per
// output number takes Wv_h's row times it, lanes across the latent.
template <typename TOut, typename TW>
__global__ void latent_merge_expand_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml, int splits, int rank,
                                           int vdim, int heads, const TW* __restrict__ w_value, TOut* __restrict__ out,
                                           const float* __restrict__ gate, int gate_splits, size_t gate_stride, int gate_row) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    extern __shared__ float lat_shared[];                       // rank, then splits
    const size_t row = blockIdx.x;
    const int h = (int)(row % heads);
    float head_gate = 1.0f;                                     // sigmoid of the head's gate number, where the layer has one
    if (gate) {
        float z = 0.0f;
        for (int s = 0; s < gate_splits; ++s) z += __ldg(gate + s * gate_stride + (row / heads) * (size_t)gate_row + h);
        head_gate = 1.0f / (1.0f + expf(-z));
    }
    const float* ml = part_ml + row * splits * 2;
    float m = -INFINITY;
    for (int s = 0; s < splits; ++s) m = fmaxf(m, ml[2 * s]);
    float l = 0.0f;
    for (int s = 0; s < splits; ++s)
        if (ml[2 * s] != -INFINITY) l += ml[2 * s + 1] * expf(ml[2 * s] - m);
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
    float* weight = lat_shared + rank;                          // a slice's share: exp(m_s - m) / l
    for (int s = threadIdx.x; s < splits; s += blockDim.x) weight[s] = ml[2 * s] != -INFINITY ? expf(ml[2 * s] - m) * inv : 0.0f;
    __syncthreads();
    for (int r = threadIdx.x; r < rank; r += blockDim.x) {
        float acc = 0.0f;
#pragma unroll 8
        for (int s = 0; s < splits; ++s) acc = fmaf(part_acc[(row * splits + s) * rank + r], weight[s], acc);
        lat_shared[r] = acc;
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    constexpr int VEC = LatVec<TW>::N;
    if (rank % VEC == 0) {                                      // 16 bytes of a row a load; four rows' loads in flight together
        for (int v0 = 4 * warp; v0 < vdim; v0 += 4 * warps) {
            float o[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            for (int r = lane * VEC; r < rank; r += 32 * VEC) {
                float w[4][VEC];
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    if (v0 + i < vdim) LatVec<TW>::load(w_value + ((size_t)h * vdim + v0 + i) * rank + r, w[i]);
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    if (v0 + i < vdim) {
#pragma unroll
                        for (int e = 0; e < VEC; ++e) o[i] = fmaf(w[i][e], lat_shared[r + e], o[i]);
                    }
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float total = tt_warp_sum(o[i]);
                if (lane == 0 && v0 + i < vdim) out[row * vdim + v0 + i] = tt_from_float<TOut>(total * head_gate);
            }
        }
        return;
    }
    for (int v = warp; v < vdim; v += warps) {
        const TW* wrow = w_value + ((size_t)h * vdim + v) * rank;
        float o = 0.0f;
        for (int r = lane; r < rank; r += 32) o = fmaf(lat_weight(wrow + r), lat_shared[r], o);
        o = tt_warp_sum(o);
        if (lane == 0) out[row * vdim + v] = tt_from_float<TOut>(o * head_gate);
    }
}

extern "C" int tt_latent_prepare(const float* down, int splits, long long split_stride, int row_stride, int q_rank, int rank, int rot,
                                 const float* q_weight, const float* kv_weight, float eps, const float* inv_freq, int rotary_dim,
                                 int interleaved, float rot_scale, void* q_latent, int act_dtype, void* pool, int cache_dtype, const int* table, int table_width,
                                 int pool_blocks, const int* cu, const int* len_before, int sequences, int n_tokens, unsigned* status,
                                 cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    const int cols = q_rank + rank + rot;
    if (rank <= 0 || q_rank < 0 || rot < 0 || rotary_dim < 0 || rotary_dim > rot || (rotary_dim & 1) || act_dtype != cache_dtype ||
        row_stride < cols)
        return (int)cudaErrorInvalidValue;
    const size_t shared = (size_t)(cols + 32) * sizeof(float);
    if (shared > 48 * 1024) return (int)cudaErrorInvalidValue;
    const int threads = cols >= 1024 ? 256 : 128;
#define TT_PREP(T) tt_launch_pdl(latent_prepare_kernel<T, T>, dim3(n_tokens), dim3(threads), shared, stream, down, splits, (size_t)split_stride, row_stride, q_rank, rank, rot, q_weight, kv_weight, eps, inv_freq, rotary_dim, interleaved, rot_scale, (T*)q_latent, (T*)pool, table, table_width, pool_blocks, cu, len_before, sequences, status)
    if (act_dtype == TT_F32) TT_PREP(float); else TT_PREP(__nv_bfloat16);
#undef TT_PREP
    TT_LAUNCH_CHECK();
}

extern "C" int tt_latent_attention(const float* q, int q_splits, long long q_stride, int q_row, const void* w_key, const void* w_value,
                                   int weight_dtype, const void* pool, int act_dtype, const int* table, int table_width, int pool_blocks,
                                   const int* cu, const int* len_before, int sequences, int n_tokens, int heads, int dim, int rot,
                                   int vdim, int rank, const float* inv_freq, int rotary_dim, int interleaved, float rot_scale, float scale,
                                   int window, int splits, void* out, float* absorbed, float* part_acc, float* part_ml,
                                   int one_token_each, const float* gate, int gate_splits, long long gate_stride, int gate_row,
                                   unsigned* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (rank <= 0 || rank > LAT_MAX_RANK || rank + rot > LAT_MAX_ROW || dim <= 0 || dim > LAT_MAX_DIM || vdim <= 0 || splits < 1 ||
        splits > 65535 || rotary_dim > rot || (rotary_dim & 1) || !absorbed || !part_acc || !part_ml || q_row < heads * (dim + rot))
        return (int)cudaErrorInvalidValue;
    const long long rows = (long long)n_tokens * heads;
    const long long blocks = (rows + LAT_WARPS - 1) / LAT_WARPS;
    if (rows > 2147483647LL) return (int)cudaErrorInvalidValue;
    const size_t shared = (size_t)LAT_WARPS * (rank + rot) * sizeof(float);
    const dim3 grid((unsigned)blocks, splits), block(LAT_WARPS * 32);
#define TT_ABSORB(TW) tt_launch_pdl(latent_absorb_kernel<TW>, dim3((unsigned)rows), dim3(rank >= 512 ? 512 : rank >= 256 ? 256 : 128), (size_t)(dim + rot) * sizeof(float), stream, q, q_splits, (size_t)q_stride, q_row, (const TW*)w_key, cu, len_before, sequences, heads, dim, rot, rank, inv_freq, rotary_dim, interleaved, rot_scale, scale, absorbed)
#define TT_ATT(TA) tt_launch_pdl(latent_attention_kernel<TA>, grid, block, shared, stream, (const float*)absorbed, (const TA*)pool, table, table_width, pool_blocks, cu, len_before, sequences, n_tokens, heads, rot, rank, window, splits, part_acc, part_ml, status)
#define TT_MERGE(TA, TW) tt_launch_pdl(latent_merge_expand_kernel<TA, TW>, dim3((unsigned)rows), dim3(256), (size_t)(rank + splits) * sizeof(float), stream, (const float*)part_acc, (const float*)part_ml, splits, rank, vdim, heads, (const TW*)w_value, (TA*)out, gate, gate_splits, (size_t)gate_stride, gate_row)
    if (weight_dtype == TT_F32) TT_ABSORB(float); else TT_ABSORB(__nv_bfloat16);
#define TT_ATT_ROWS(TA) tt_launch_pdl(latent_attention_rows_kernel<TA>, grid, block, 0, stream, (const float*)absorbed, (const TA*)pool, table, table_width, pool_blocks, cu, len_before, sequences, n_tokens, heads, rot, rank, window, splits, part_acc, part_ml, status)
    const int piece = act_dtype == TT_F32 ? 4 : 8;              // numbers in 16 bytes of a cache row
    if (one_token_each == 2) {                                  // the caller has checked tt_latent_decode_mma_takes and set splits for slices of LT_KEYS
        static size_t allowed = 0;
        const size_t need = latent_decode_shared(rank + rot);
        if (need > allowed) {
            const cudaError_t e = cudaFuncSetAttribute(latent_decode_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)need);
            if (e != cudaSuccess) return (int)e;
            allowed = need;
        }
        tt_launch_pdl(latent_decode_mma_kernel, dim3(n_tokens, splits, (heads + LT_HEADS - 1) / LT_HEADS), dim3(128), need, stream,
                      (const float*)absorbed, (const __nv_bfloat16*)pool, table, table_width, pool_blocks, len_before, heads, rot, rank, window,
                      splits, part_acc, part_ml, status);
    } else if (rank % piece == 0 && rot % piece == 0) {
        if (act_dtype == TT_F32) TT_ATT_ROWS(float); else TT_ATT_ROWS(__nv_bfloat16);
    } else {
        if (act_dtype == TT_F32) TT_ATT(float); else TT_ATT(__nv_bfloat16);
    }
#undef TT_ATT_ROWS
    if (act_dtype == TT_F32 && weight_dtype == TT_F32) TT_MERGE(float, float);
    else if (act_dtype == TT_F32) TT_MERGE(float, __nv_bfloat16);
    else if (weight_dtype == TT_F32) TT_MERGE(__nv_bfloat16, float);
    else TT_MERGE(__nv_bfloat16, __nv_bfloat16);
#undef TT_ABSORB
#undef TT_ATT
#undef TT_MERGE
    TT_LAUNCH_CHECK();
}


// ------------------------------------------------------------------------------------
// Expansion of the visible latents of a step of prompts (see the top of the file).
// plan: int32 [sequences + 1] first temporary block of every sequence (and their total), then [sequences] the first
// cache block (position / 64) each sequence's temporary blocks stand for.
// ------------------------------------------------------------------------------------
__global__ void latent_expand_plan_kernel(const int* __restrict__ cu, const int* __restrict__ len_before, int sequences, int window,
                                          int table_width, int bound_blocks, int* __restrict__ plan, int* __restrict__ table_tmp,
                                          unsigned* status) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int b = 0; b < sequences; ++b) {
            const int before = len_before[b], after = before + cu[b + 1] - cu[b];
            const int first_pos = (window > 0 && before - window + 1 > 0) ? before - window + 1 : 0;   // oldest key the step's first token sees
            const int first_block = first_pos / TT_BLOCK_TOKENS;
            int blocks = (after + TT_BLOCK_TOKENS - 1) / TT_BLOCK_TOKENS - first_block;
            if (at + blocks > bound_blocks) {                  // cannot happen with the bound the host computes
                atomicOr(status, TT_STATUS_BAD_SHAPE);
                blocks = bound_blocks - at;
            }
            plan[b] = at;
            plan[sequences + 1 + b] = first_block;
            at += blocks;
        }
        plan[sequences] = at;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < sequences * table_width; e += blockDim.x) {
        const int b = e / table_width, i = e - b * table_width;
        const int first_block = plan[sequences + 1 + b], blocks = plan[b + 1] - plan[b];
        table_tmp[e] = (i >= first_block && i < first_block + blocks) ? plan[b] + (i - first_block) : -1;
    }
}

// One block per row of the temporary blocks (block * 64 + token).  x: [rows][rank]; keys: [block][heads][64][dim + rot].
template <typename T>
__global__ void latent_gather_kernel(const T* __restrict__ pool, const int* __restrict__ table, int table_width, int pool_blocks,
                                     const int* __restrict__ cu, const int* __restrict__ len_before, int sequences,
                                     const int* __restrict__ plan, int heads, int dim, int rot, int rank, T* __restrict__ x,
                                     T* __restrict__ keys) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    const int row = blockIdx.x, tb = row / TT_BLOCK_TOKENS, r = row - tb * TT_BLOCK_TOKENS;
    long long off = -1;
    if (tb < plan[sequences]) {
        const int b = tt_find_sequence(plan, sequences, tb);   // plan[b] <= tb < plan[b + 1]; sequences without blocks are skipped by the search
        const int pos = (plan[sequences + 1 + b] + tb - plan[b]) * TT_BLOCK_TOKENS + r;
        if (pos < len_before[b] + cu[b + 1] - cu[b])
            off = tt_cache_offset(table + (size_t)b * table_width, pos, 0, 1, rank + rot, pool_blocks, nullptr);   // a block the window gave back: zeros
    }
    const T zero = tt_from_float<T>(0.0f);
    for (int j = threadIdx.x; j < rank; j += blockDim.x) x[(size_t)row * rank + j] = off >= 0 ? pool[off + j] : zero;
    const int hd = dim + rot;
    for (int e = threadIdx.x; e < heads * rot; e += blockDim.x) {
        const int h = e / rot, j = e - h * rot;
        keys[(((size_t)tb * heads + h) * TT_BLOCK_TOKENS + r) * hd + dim + j] = off >= 0 ? pool[off + rank + j] : zero;
    }
}

// y: float32 partial sums [splits][rows][heads * dim + heads * vdim] of x [Wk; Wv]^T.  One block per temporary block and
// head: the unrotated key parts go out row by row, the values through shared memory so that a value number's 64 tokens
// are written side by side.
template <typename T>
__global__ void latent_scatter_kernel(const float* __restrict__ y, int splits, size_t split_stride, int heads, int dim, int rot,
                                      int vdim, T* __restrict__ keys, T* __restrict__ values) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    extern __shared__ float lat_shared[];                       // [64][vdim + 1]
    const int tb = blockIdx.x / heads, h = blockIdx.x - tb * heads;
    const int cols = heads * (dim + vdim), hd = dim + rot;
    const float* base = y + (size_t)tb * TT_BLOCK_TOKENS * cols;
    for (int e = threadIdx.x; e < TT_BLOCK_TOKENS * dim; e += blockDim.x) {
        const int r = e / dim, d = e - r * dim;
        float v = 0.0f;
        for (int s = 0; s < splits; ++s) v += base[(size_t)s * split_stride + (size_t)r * cols + h * dim + d];
        keys[(((size_t)tb * heads + h) * TT_BLOCK_TOKENS + r) * hd + d] = tt_from_float<T>(v);
    }
    for (int e = threadIdx.x; e < TT_BLOCK_TOKENS * vdim; e += blockDim.x) {
        const int r = e / vdim, d = e - r * vdim;
        float v = 0.0f;
        for (int s = 0; s < splits; ++s) v += base[(size_t)s * split_stride + (size_t)r * cols + heads * dim + h * vdim + d];
        lat_shared[r * (vdim + 1) + d] = v;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < TT_BLOCK_TOKENS * vdim; e += blockDim.x) {
        const int d = e / TT_BLOCK_TOKENS, r = e - d * TT_BLOCK_TOKENS;
        values[(((size_t)tb * heads + h) * vdim + d) * TT_BLOCK_TOKENS + r] = tt_from_float<T>(lat_shared[r * (vdim + 1) + d]);
    }
}

// q: float32 partial sums [splits][tokens][heads * (dim + rot)]; out: the same numbers in T with each head's last rot
// numbers rotated by the token's position (the first rotary_dim of them, halves or neighbours paired); a token's row of q
// is q_row numbers long.
template <typename T>
__global__ void latent_queries_kernel(const float* __restrict__ q, int splits, size_t split_stride, int q_row, int heads, int dim, int rot,
                                      const float* __restrict__ inv_freq, int rotary_dim, int interleaved, float rot_scale,
                                      const int* __restrict__ cu,
                                      const int* __restrict__ len_before, int sequences, T* __restrict__ out) {
    tt_pdl_launch_dependents();
    const int t = blockIdx.x;
    const int b = tt_find_sequence(cu, sequences, t);
    const int pos = len_before[b] + (t - cu[b]);
    tt_pdl_wait();
    const int hd = dim + rot, half = rotary_dim >> 1;
    const float* row = q + (size_t)t * q_row;
    for (int e = threadIdx.x; e < heads * hd; e += blockDim.x) {
        const int i = e % hd - dim;                             // index inside the rotated part, negative in front of it
        float x = 0.0f;
        for (int s = 0; s < splits; ++s) x += row[(size_t)s * split_stride + e];
        if (i >= 0 && i < rotary_dim) {
            const bool first = interleaved ? !(i & 1) : i < half;
            const int pair = interleaved ? (first ? e + 1 : e - 1) : (first ? e + half : e - half);
            float other = 0.0f;
            for (int s = 0; s < splits; ++s) other += row[(size_t)s * split_stride + pair];
            float sn, cs;
            sincosf((float)pos * __ldg(inv_freq + (interleaved ? (i >> 1) : (first ? i : i - half))), &sn, &cs);
            sn *= rot_scale; cs *= rot_scale;
            x = first ? x * cs - other * sn : x * cs + other * sn;
        }
        out[(size_t)t * heads * hd + e] = tt_from_float<T>(x);
    }
}

extern "C" int tt_latent_expand_plan(const int* cu, const int* len_before, int sequences, int window, int table_width, int bound_blocks,
                                     int* plan, int* table_tmp, unsigned* status, cudaStream_t stream) {
    if (sequences <= 0) return 0;
    tt_launch_pdl(latent_expand_plan_kernel, dim3(1), dim3(256), 0, stream, cu, len_before, sequences, window, table_width, bound_blocks, plan,
                  table_tmp, status);
    TT_LAUNCH_CHECK();
}

extern "C" int tt_latent_gather(const void* pool, int dtype, const int* table, int table_width, int pool_blocks, const int* cu,
                                const int* len_before, int sequences, const int* plan, int bound_blocks, int heads, int dim, int rot,
                                int rank, void* x, void* keys, cudaStream_t stream) {
    if (bound_blocks <= 0) return 0;
    const dim3 grid((unsigned)bound_blocks * TT_BLOCK_TOKENS), block(128);
    if (dtype == TT_F32)
        tt_launch_pdl(latent_gather_kernel<float>, grid, block, 0, stream, (const float*)pool, table, table_width, pool_blocks, cu, len_before, sequences, plan, heads, dim, rot, rank, (float*)x, (float*)keys);
    else
        tt_launch_pdl(latent_gather_kernel<__nv_bfloat16>, grid, block, 0, stream, (const __nv_bfloat16*)pool, table, table_width, pool_blocks, cu, len_before, sequences, plan, heads, dim, rot, rank, (__nv_bfloat16*)x, (__nv_bfloat16*)keys);
    TT_LAUNCH_CHECK();
}

extern "C" int tt_latent_scatter(const float* y, int splits, long long split_stride, int bound_blocks, int heads, int dim, int rot, int vdim,
                                 void* keys, void* values, int dtype, cudaStream_t stream) {
    if (bound_blocks <= 0) return 0;
    const size_t shared = (size_t)TT_BLOCK_TOKENS * (vdim + 1) * sizeof(float);
    if (shared > 48 * 1024) return (int)cudaErrorInvalidValue;
    const dim3 grid((unsigned)bound_blocks * heads), block(256);
    if (dtype == TT_F32)
        tt_launch_pdl(latent_scatter_kernel<float>, grid, block, shared, stream, y, splits, (size_t)split_stride, heads, dim, rot, vdim, (float*)keys, (float*)values);
    else
        tt_launch_pdl(latent_scatter_kernel<__nv_bfloat16>, grid, block, shared, stream, y, splits, (size_t)split_stride, heads, dim, rot, vdim, (__nv_bfloat16*)keys, (__nv_bfloat16*)values);
    TT_LAUNCH_CHECK();
}

extern "C" int tt_latent_queries(const float* q, int splits, long long split_stride, int q_row, int heads, int dim, int rot,
                                 const float* inv_freq, int rotary_dim, int interleaved, float rot_scale, const int* cu, const int* len_before, int sequences, int n_tokens, void* out, int dtype,
                                 cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (rotary_dim > rot || (rotary_dim & 1)) return (int)cudaErrorInvalidValue;
    if (dtype == TT_F32)
        tt_launch_pdl(latent_queries_kernel<float>, dim3(n_tokens), dim3(256), 0, stream, q, splits, (size_t)split_stride, q_row, heads, dim, rot, inv_freq, rotary_dim, interleaved, rot_scale, cu, len_before, sequences, (float*)out);
    else
        tt_launch_pdl(latent_queries_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(256), 0, stream, q, splits, (size_t)split_stride, q_row, heads, dim, rot, inv_freq, rotary_dim, interleaved, rot_scale, cu, len_before, sequences, (__nv_bfloat16*)out);
    TT_LAUNCH_CHECK();
}

// Whether the tensor-core decode kernel takes these sizes (bfloat16 cache, latent and rotated part multiples of 16, shared memory), and
// the keys of one of its slices.
extern "C" int tt_latent_decode_mma_takes(int act_dtype, int rank, int rot) {
    return act_dtype == TT_BF16 && rank % 16 == 0 && rot % 16 == 0 && rank + rot <= LAT_MAX_ROW && latent_decode_shared(rank + rot) <= 200 * 1024;
}
extern "C" int tt_latent_decode_slice_keys() { return LT_KEYS; }
