// Memory-bound kernels between the matrix products: embedding gather (also with a hashed
// row for the pair of the previous token and this one), residual add fused with RMSNorm,
// the token shift of a mixer's input, rotary encoding fused with the cache append, SwiGLU,
// and the length bookkeeping of a step.  All statistics, angles and sums are float32.
//
// Counterparts in random-unknown-username/Thintensor (Triton, one token per launch):
// _copy_embed_token thinruntime/gpu_runtime.py:11396-11427; _rms_norm_kernel and
// _add_rms_norm_kernel thinruntime/triton_kernels.py:2561-2614; _rope_qk_inplace_kernel
// thinruntime/triton_kernels.py:2637-2687 with PagedKVCache._store_token
// thinruntime/gpu_runtime.py:4530-4556; _silu_mul_kernel thinruntime/triton_kernels.py:2760-2774.
#include "common.cuh"

// ------------------------------------------------------------------------------------
// embedding gather: residual[t, :] = table[token[t], :] * scale   (float32 out)
// ------------------------------------------------------------------------------------
template <typename TW>
__global__ void embed_gather_kernel(const TW* __restrict__ table, const int* __restrict__ tokens,
                                    float* __restrict__ residual, int hidden, int vocab, float scale,
                                    unsigned* status) {
    // The first kernel of every step waits before it lets its dependents start: whatever a
    // later kernel of this step reads ahead of its own wait (lengths, tables, cache blocks of
    // earlier steps) is then complete, because no kernel of this step starts before the
    // previous step's last kernel has finished.
    tt_pdl_wait();
    tt_pdl_launch_dependents();
    const int t = blockIdx.x;
    int id = tokens[t];
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) atomicOr(status, TT_STATUS_BAD_TOKEN);
        for (int j = threadIdx.x; j < hidden; j += blockDim.x) residual[(size_t)t * hidden + j] = 0.0f;
        return;
    }
    const TW* row = table + (size_t)id * hidden;
    float* out = residual + (size_t)t * hidden;
    if constexpr (sizeof(TW) == 2) {
        // rows of whole 16-byte pieces: eight numbers a load, two 16-byte stores
        if ((hidden & 7) == 0 && (((uintptr_t)table | (uintptr_t)residual) & 15) == 0) {
            for (int j = 8 * threadIdx.x; j < hidden; j += 8 * blockDim.x) {
                const uint4 raw = __ldg(reinterpret_cast<const uint4*>(row + j));
                const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
                const float2 a = __bfloat1622float2(pairs[0]), b = __bfloat1622float2(pairs[1]);
                const float2 c = __bfloat1622float2(pairs[2]), d = __bfloat1622float2(pairs[3]);
                *reinterpret_cast<float4*>(out + j) = make_float4(a.x * scale, a.y * scale, b.x * scale, b.y * scale);
                *reinterpret_cast<float4*>(out + j + 4) = make_float4(c.x * scale, c.y * scale, d.x * scale, d.y * scale);
            }
            return;
        }
    }
    for (int j = threadIdx.x; j < hidden; j += blockDim.x)
        out[j] = tt_to_float(row[j]) * scale;
}

extern "C" int tt_embed_gather(const void* table, int table_dtype, const int* tokens, float* residual, int n_tokens,
                               int hidden, int vocab, float scale, unsigned* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (table_dtype == TT_F32)
        tt_launch_pdl(embed_gather_kernel<float>, dim3(n_tokens), dim3(threads), 0, stream, (const float*)table, tokens, residual, hidden, vocab, scale, status);
    else
        tt_launch_pdl(embed_gather_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0, stream, (const __nv_bfloat16*)table, tokens, residual, hidden, vocab, scale, status);
    TT_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------
// residual add + RMSNorm, or + weight-only layer norm (centered != 0).
//   x = residual[r] + delta[0][r] + delta[1][r] + ...      (fixed order)
//   residual[r] = x                                        (only when rows == nullptr)
//   out[i] = x * rsqrt(mean(x^2) + eps) * (weight + weight_offset)
//   centered: out[i] = (x - mean(x)) * rsqrt(mean((x - mean(x))^2) + eps) * (weight + weight_offset) [+ bias]
// One block per output row; the row is kept in shared memory between the two passes.
// With `rows`, output row i is taken from residual row rows[i] and nothing is written
// back (the final norm at the wanted positions).
// ------------------------------------------------------------------------------------
template <typename TOut>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const float* __restrict__ delta, int splits,
                                   size_t split_stride, const float* __restrict__ weight, float weight_offset,
                                   float eps, TOut* __restrict__ out, const int* __restrict__ rows, int hidden,
                                   int row_cache, int centered, const float* __restrict__ bias) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    extern __shared__ float row_shared[];  // row_cache floats, then 32 for the reduction
    float* reduce = row_shared + row_cache;
    const int i = blockIdx.x;
    const int r = rows ? rows[i] : i;
    float* res = residual + (size_t)r * hidden;
    const float* del = delta ? delta + (size_t)r * hidden : nullptr;
    float sumsq = 0.0f, sum = 0.0f;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
        float x = res[j];
        for (int s = 0; s < splits; ++s) x += del[(size_t)s * split_stride + j];
        if (j < row_cache) row_shared[j] = x;
        if (!rows && splits > 0) res[j] = x;
        sumsq += x * x;
        sum += x;
    }
    // the value of element j again: from shared memory, from the stream this thread has just written, or summed anew
    auto again = [&](int j) {
        if (j < row_cache) return row_shared[j];
        float x = res[j];
        if (rows) for (int s = 0; s < splits; ++s) x += del[(size_t)s * split_stride + j];
        return x;
    };
    float mean = 0.0f, total;
    if (centered) {
        mean = tt_block_sum(sum, reduce) / (float)hidden;
        float dev = 0.0f;
        for (int j = threadIdx.x; j < hidden; j += blockDim.x) { const float d = again(j) - mean; dev += d * d; }
        total = tt_block_sum(dev, reduce);
    } else {
        total = tt_block_sum(sumsq, reduce);
    }
    const float rstd = rsqrtf(total / (float)hidden + eps);
    TOut* o = out + (size_t)i * hidden;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x)
        o[j] = tt_from_float<TOut>((again(j) - mean) * rstd * (weight[j] + weight_offset) + (bias ? bias[j] : 0.0f));
}

// four consecutive outputs as one store (the row start is 16-byte aligned and j counts groups of four)
__device__ __forceinline__ void tt_store4(float* p, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void tt_store4(__nv_bfloat16* p, float a, float b, float c, float d) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 v;
    v.x = *reinterpret_cast<const uint32_t*>(&lo);
    v.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = v;
}

// The same for hidden sizes that are multiples of 4 up to 16384: every thread keeps its
// (up to four) float4 pieces of the row in registers, all loads of the k-slices are
// independent, and the order of additions is the one of the kernel above.
#define NORM_VEC_MAX 4
// PIECES: float4 pieces of a row per thread: 1 when the block is as wide as the row (few rows: decoding), else up to
// NORM_VEC_MAX (prompts).  BATCH: how many k-slices' loads are in flight together.
template <typename TOut, int PIECES, int BATCH>
__global__ void __launch_bounds__(1024)
add_rmsnorm_vec_kernel(float* __restrict__ residual, const float* __restrict__ delta, int splits, size_t split_stride,
                       const float* __restrict__ weight, float weight_offset, float eps, TOut* __restrict__ out,
                       const int* __restrict__ rows, int hidden, int centered, const float* __restrict__ bias) {
    tt_pdl_launch_dependents();
    __shared__ float reduce[32];
    const int i = blockIdx.x;
    const int quads = hidden >> 2;
    // the norm's weight is written by no kernel: it is fetched while the previous kernel still runs
    const float4* w4 = reinterpret_cast<const float4*>(weight);
    float4 w[PIECES];
#pragma unroll
    for (int v = 0; v < PIECES; ++v) {
        const int j = threadIdx.x + v * blockDim.x;
        if (j < quads) w[v] = __ldg(w4 + j);
    }
    tt_pdl_wait();
    const int r = rows ? rows[i] : i;
    float4* res = reinterpret_cast<float4*>(residual + (size_t)r * hidden);
    const float4* del = delta ? reinterpret_cast<const float4*>(delta + (size_t)r * hidden) : nullptr;
    const size_t stride4 = split_stride >> 2;
    float4 x[PIECES];
    float sumsq = 0.0f, sum = 0.0f;
#pragma unroll
    for (int v = 0; v < PIECES; ++v) {
        const int j = threadIdx.x + v * blockDim.x;
        if (j < quads) {
            float4 a = res[j];
            // BATCH slices' loads are in flight together (one after the other they cost a round trip to the L2
            // each: a decode step's norm after a product of 16 k-slices); the additions keep the slices' order
            for (int s0 = 0; s0 < splits; s0 += BATCH) {
                float4 d[BATCH];
#pragma unroll
                for (int i = 0; i < BATCH; ++i)
                    if (s0 + i < splits) d[i] = __ldg(del + (size_t)(s0 + i) * stride4 + j);
#pragma unroll
                for (int i = 0; i < BATCH; ++i)
                    if (s0 + i < splits) { a.x += d[i].x; a.y += d[i].y; a.z += d[i].z; a.w += d[i].w; }
            }
            if (!rows && splits > 0) res[j] = a;
            x[v] = a;
            sumsq += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
            sum += (a.x + a.y) + (a.z + a.w);
        }
    }
    float total;
    if (centered) {                                           // the deviations from the mean, squared, in a pass of their own
        const float mean = tt_block_sum(sum, reduce) / (float)hidden;
        float dev = 0.0f;
#pragma unroll
        for (int v = 0; v < PIECES; ++v) {
            const int j = threadIdx.x + v * blockDim.x;
            if (j < quads) {
                x[v].x -= mean; x[v].y -= mean; x[v].z -= mean; x[v].w -= mean;
                dev += x[v].x * x[v].x + x[v].y * x[v].y + x[v].z * x[v].z + x[v].w * x[v].w;
            }
        }
        total = tt_block_sum(dev, reduce);
    } else {
        total = tt_block_sum(sumsq, reduce);
    }
    const float rstd = rsqrtf(total / (float)hidden + eps);
    TOut* o = out + (size_t)i * hidden;
#pragma unroll
    for (int v = 0; v < PIECES; ++v) {
        const int j = threadIdx.x + v * blockDim.x;
        if (j < quads) {
            float y0 = x[v].x * rstd * (w[v].x + weight_offset), y1 = x[v].y * rstd * (w[v].y + weight_offset);
            float y2 = x[v].z * rstd * (w[v].z + weight_offset), y3 = x[v].w * rstd * (w[v].w + weight_offset);
            if (bias) {
                const float4 b = __ldg(reinterpret_cast<const float4*>(bias) + j);
                y0 += b.x; y1 += b.y; y2 += b.z; y3 += b.w;
            }
            tt_store4(o + 4 * j, y0, y1, y2, y3);
        }
    }
}

static int add_norm(float* residual, const float* delta, int splits, long long split_stride,
                    const float* weight, float weight_offset, float eps, void* out, int out_dtype,
                    const int* rows, int n_rows, int hidden, int centered, const float* bias, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (!delta) splits = 0;
    if (hidden % 4 == 0 && hidden <= 4096 * NORM_VEC_MAX && split_stride % 4 == 0 && ((uintptr_t)residual & 15) == 0 &&
        ((uintptr_t)delta & 15) == 0 && ((uintptr_t)weight & 15) == 0 && ((uintptr_t)out & 15) == 0 && ((uintptr_t)bias & 15) == 0) {
        int threads = ((hidden / 4 + 31) / 32) * 32;
        if (threads > 1024) threads = 1024;
        if (n_rows >= 1024) {
            // prompts: up to four pieces of the row per thread (fewer, fatter blocks: measured 5.33 -> 5.20 ms for a
            // 2,048-token prefill of the 1B shape)
            const int fewest = (((hidden / 4 + NORM_VEC_MAX - 1) / NORM_VEC_MAX + 31) / 32) * 32;
            threads = fewest < 128 ? 128 : fewest;
            if (threads > 1024) threads = 1024;
        }
        const bool one_piece = threads * 4 >= hidden;         // the block covers the row: one piece per thread, eight slices at a time
#define TT_NORM(T, P, B) tt_launch_pdl(add_rmsnorm_vec_kernel<T, P, B>, dim3(n_rows), dim3(threads), 0, stream, residual, delta, splits, (size_t)split_stride, weight, weight_offset, eps, (T*)out, rows, hidden, centered, bias)
        if (out_dtype == TT_F32) { if (one_piece) TT_NORM(float, 1, 8); else TT_NORM(float, NORM_VEC_MAX, 2); }
        else { if (one_piece) TT_NORM(__nv_bfloat16, 1, 8); else TT_NORM(__nv_bfloat16, NORM_VEC_MAX, 2); }
#undef TT_NORM
        TT_LAUNCH_CHECK();
    }
    const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    const int row_cache = hidden <= 11264 ? hidden : 11264;  // 44 KB of the default 48 KB
    const size_t shared = (size_t)(row_cache + 32) * sizeof(float);
    if (out_dtype == TT_F32)
        tt_launch_pdl(add_rmsnorm_kernel<float>, dim3(n_rows), dim3(threads), shared, stream, residual, delta, splits, (size_t)split_stride, weight, weight_offset, eps, (float*)out, rows, hidden, row_cache, centered, bias);
    else
        tt_launch_pdl(add_rmsnorm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), shared, stream, residual, delta, splits, (size_t)split_stride, weight, weight_offset, eps, (__nv_bfloat16*)out, rows, hidden, row_cache, centered, bias);
    TT_LAUNCH_CHECK();
}

extern "C" int tt_add_rmsnorm(float* residual, const float* delta, int splits, long long split_stride,
                              const float* weight, float weight_offset, float eps, void* out, int out_dtype,
                              const int* rows, int n_rows, int hidden, cudaStream_t stream) {
    return add_norm(residual, delta, splits, split_stride, weight, weight_offset, eps, out, out_dtype, rows, n_rows, hidden, 0, nullptr, stream);
}

// the same with the mean taken off first (layer norm); bias (float32, or null) is added at the end
extern "C" int tt_add_layernorm(float* residual, const float* delta, int splits, long long split_stride,
                                const float* weight, const float* bias, float eps, void* out, int out_dtype,
                                const int* rows, int n_rows, int hidden, cudaStream_t stream) {
    return add_norm(residual, delta, splits, split_stride, weight, 0.0f, eps, out, out_dtype, rows, n_rows, hidden, 1, bias, stream);
}

// ------------------------------------------------------------------------------------
// rotary encoding + cache append.
// qkv: float32 [splits][tokens][q_cols + 2 * kv_cols] partial sums of the projection.
// For token t of sequence b at position p = len_before[b] + (t - cu[b]):
//   q' -> q_out[t] (activation dtype), k' -> key pool at p, v -> value pool at p
//   (values are stored transposed inside a block, see common.cuh).
// Rotation on the first rotary_dim numbers of each head, halves convention:
//   a' = a cos - b sin, b' = b cos + a sin, angle = inv_freq[i] * float(p) in float32.
// kv_cols == 0: the projection holds queries only and nothing is appended (a layer that
// reads another layer's cache).
// ------------------------------------------------------------------------------------
// sum of one element over the k-slices of a projection: independent loads, fixed order of additions
__device__ __forceinline__ float sum_slices(const float* __restrict__ p, int splits, size_t split_stride) {
    float total = 0.0f;
    int s = 0;
    for (; s + 4 <= splits; s += 4) {
        const float a = __ldg(p + (size_t)s * split_stride), b = __ldg(p + (size_t)(s + 1) * split_stride);
        const float c = __ldg(p + (size_t)(s + 2) * split_stride), d = __ldg(p + (size_t)(s + 3) * split_stride);
        total = (((total + a) + b) + c) + d;
    }
    for (; s < splits; ++s) total += __ldg(p + (size_t)s * split_stride);
    return total;
}

// One thread per item of a token: a rotated pair of q or k, a number beyond the rotary
// part, or a value.  grid = (tokens, ceil(items / blockDim.x)).
template <typename TAct>
__global__ void rope_append_kernel(const float* __restrict__ qkv, int splits, size_t split_stride,
                                   const float* __restrict__ inv_freq,
                                   int rotary_dim, float attention_scaling, TAct* __restrict__ q_out,
                                   TAct* __restrict__ k_pool, TAct* __restrict__ v_pool,
                                   const int* __restrict__ table, int table_width, int pool_blocks,
                                   const int* __restrict__ cu, const int* __restrict__ len_before, int sequences,
                                   int heads, int kv_heads, int head_dim, int write_cache, unsigned* status) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    const int t = blockIdx.x;
    const int b = tt_find_sequence(cu, sequences, t);
    const int pos = len_before[b] + (t - cu[b]);
    const int half = rotary_dim >> 1;
    const int q_cols = heads * head_dim;
    const int kv_cols = write_cache ? kv_heads * head_dim : 0;
    const int cols = q_cols + 2 * kv_cols;
    const float* row = qkv + (size_t)t * cols;
    const int* table_row = table + (size_t)b * table_width;
    const int rot_heads = heads + (write_cache ? kv_heads : 0);
    const int pass = head_dim - rotary_dim;  // numbers of a head that are not rotated
    const int n_rot = rot_heads * half, n_pass = rot_heads * pass;
    int w = blockIdx.y * blockDim.x + threadIdx.x;
    if (w < n_rot) {
        const int head = w / half, i = w - head * half;
        const int col = head * head_dim + i;  // k heads follow q heads in the row
        const float a = sum_slices(row + col, splits, split_stride);
        const float c2 = sum_slices(row + col + half, splits, split_stride);
        float si, co;
        sincosf(inv_freq[i] * (float)pos, &si, &co);
        co *= attention_scaling;
        si *= attention_scaling;
        const float ra = a * co - c2 * si, rb = c2 * co + a * si;
        if (head < heads) {
            q_out[(size_t)t * q_cols + col] = tt_from_float<TAct>(ra);
            q_out[(size_t)t * q_cols + col + half] = tt_from_float<TAct>(rb);
        } else {
            const long long off = tt_cache_offset(table_row, pos, head - heads, kv_heads, head_dim, pool_blocks, status);
            if (off >= 0) {
                k_pool[off + i] = tt_from_float<TAct>(ra);
                k_pool[off + i + half] = tt_from_float<TAct>(rb);
            }
        }
        return;
    }
    w -= n_rot;
    if (w < n_pass) {
        const int head = w / pass, i = rotary_dim + (w - head * pass);
        const int col = head * head_dim + i;
        const float a = sum_slices(row + col, splits, split_stride);
        if (head < heads) {
            q_out[(size_t)t * q_cols + col] = tt_from_float<TAct>(a);
        } else {
            const long long off = tt_cache_offset(table_row, pos, head - heads, kv_heads, head_dim, pool_blocks, status);
            if (off >= 0) k_pool[off + i] = tt_from_float<TAct>(a);
        }
        return;
    }
    w -= n_pass;
    if (w < kv_cols) {
        const int kh = w / head_dim, i = w - kh * head_dim;
        const float a = sum_slices(row + q_cols + kv_cols + w, splits, split_stride);
        const long long off = tt_value_offset(table_row, pos, kh, kv_heads, head_dim, pool_blocks, status);
        if (off >= 0) v_pool[off + (long long)i * TT_BLOCK_TOKENS] = tt_from_float<TAct>(a);
    }
}

// The same with four neighbouring items per thread (float4 loads, 8-byte stores of q and k): used
// when the rotary part and the rest of a head are multiples of 8 and 4 numbers.
__device__ __forceinline__ float4 sum_slices4(const float* __restrict__ p, int splits, size_t split_stride) {
    float4 total = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (int s = 0; s < splits; ++s) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(p + (size_t)s * split_stride));
        total.x += v.x; total.y += v.y; total.z += v.z; total.w += v.w;
    }
    return total;
}

constexpr int ROPE_MAX_HALF = 128;          // half of the largest rotary part (head sizes go up to 256)

template <typename TAct>
__global__ void rope_append_vec_kernel(const float* __restrict__ qkv, int splits, size_t split_stride,
                                       const float* __restrict__ inv_freq, int rotary_dim, float attention_scaling,
                                       TAct* __restrict__ q_out, TAct* __restrict__ k_pool, TAct* __restrict__ v_pool,
                                       const int* __restrict__ table, int table_width, int pool_blocks,
                                       const int* __restrict__ cu, const int* __restrict__ len_before, int sequences,
                                       int heads, int kv_heads, int head_dim, int write_cache, unsigned* status) {
    tt_pdl_launch_dependents();
    // Lengths, offsets and tables were written before the step's first kernel started: the token's sequence, position,
    // cache block and angles are found ahead of the wait for the qkv product (five dependent round trips to the L2 that
    // would otherwise follow it); only the product's slices are read after it.
    const int t = blockIdx.x;
    // one token per sequence (a decode step): token t is sequence t, which two independent loads confirm
    const int b = (sequences == (int)gridDim.x && cu[t] == t && cu[t + 1] == t + 1) ? t : tt_find_sequence(cu, sequences, t);
    const int pos = len_before[b] + (t - cu[b]);
    const int half = rotary_dim >> 1, half4 = half >> 2;
    const int q_cols = heads * head_dim;
    const int kv_cols = write_cache ? kv_heads * head_dim : 0;
    const int cols = q_cols + 2 * kv_cols;
    const float* row = qkv + (size_t)t * cols;
    const int* table_row = table + (size_t)b * table_width;
    const int rot_heads = heads + (write_cache ? kv_heads : 0);
    const int pass4 = (head_dim - rotary_dim) >> 2;
    const int n_rot = rot_heads * half4, n_pass = rot_heads * pass4;
    // the angles depend on the position only: one table per block instead of one sincosf per head and pair
    __shared__ float cos_sh[ROPE_MAX_HALF], sin_sh[ROPE_MAX_HALF];
    for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf(__ldg(inv_freq + i) * (float)pos, &sin_sh[i], &cos_sh[i]);
    // the token's cache block, looked up once: -1 where the table entry lies outside the pool (reported when a write needs it)
    int block = -1;
    if (write_cache) {
        block = table_row[pos / TT_BLOCK_TOKENS];
        if (block < 0 || block >= pool_blocks) block = -1;
    }
    const int slot = pos % TT_BLOCK_TOKENS;
    auto key_offset = [&](int kv_head) -> long long {
        if (block < 0) { atomicOr(status, TT_STATUS_BAD_BLOCK); return -1; }
        return (((long long)block * kv_heads + kv_head) * TT_BLOCK_TOKENS + slot) * head_dim;
    };
    auto value_offset = [&](int kv_head) -> long long {
        if (block < 0) { atomicOr(status, TT_STATUS_BAD_BLOCK); return -1; }
        return ((long long)block * kv_heads + kv_head) * head_dim * TT_BLOCK_TOKENS + slot;
    };
    __syncthreads();
    tt_pdl_wait();
    const int n_val = kv_cols >> 2;
    // the token's blocks (one when there are many tokens, several when there are few) walk over its items
    for (int item = blockIdx.y * blockDim.x + threadIdx.x; item < n_rot + n_pass + n_val; item += gridDim.y * blockDim.x) {
        int w = item;
        if (w < n_rot) {
            const int head = w / half4, i = (w - head * half4) * 4;
            const int col = head * head_dim + i;
            const float4 a = sum_slices4(row + col, splits, split_stride);
            const float4 c = sum_slices4(row + col + half, splits, split_stride);
            const float s0 = sin_sh[i], c0 = cos_sh[i], s1 = sin_sh[i + 1], c1 = cos_sh[i + 1];
            const float s2 = sin_sh[i + 2], c2 = cos_sh[i + 2], s3 = sin_sh[i + 3], c3 = cos_sh[i + 3];
            const float k = attention_scaling;
            const float ra0 = (a.x * c0 - c.x * s0) * k, rb0 = (c.x * c0 + a.x * s0) * k;
            const float ra1 = (a.y * c1 - c.y * s1) * k, rb1 = (c.y * c1 + a.y * s1) * k;
            const float ra2 = (a.z * c2 - c.z * s2) * k, rb2 = (c.z * c2 + a.z * s2) * k;
            const float ra3 = (a.w * c3 - c.w * s3) * k, rb3 = (c.w * c3 + a.w * s3) * k;
            TAct* dst;
            if (head < heads) {
                dst = q_out + (size_t)t * q_cols + col;
            } else {
                const long long off = key_offset(head - heads);
                if (off < 0) continue;
                dst = k_pool + off + i;
            }
            tt_store4(dst, ra0, ra1, ra2, ra3);
            tt_store4(dst + half, rb0, rb1, rb2, rb3);
            continue;
        }
        w -= n_rot;
        if (w < n_pass) {
            const int head = w / pass4, i = rotary_dim + (w - head * pass4) * 4;
            const int col = head * head_dim + i;
            const float4 a = sum_slices4(row + col, splits, split_stride);
            if (head < heads) {
                tt_store4(q_out + (size_t)t * q_cols + col, a.x, a.y, a.z, a.w);
            } else {
                const long long off = key_offset(head - heads);
                if (off >= 0) tt_store4(k_pool + off + i, a.x, a.y, a.z, a.w);
            }
            continue;
        }
        w -= n_pass;
        const int e = w * 4, kh = e / head_dim, i = e - kh * head_dim;
        const float4 a = sum_slices4(row + q_cols + kv_cols + e, splits, split_stride);
        const long long off = value_offset(kh);
        if (off >= 0) {
            TAct* dst = v_pool + off + (long long)i * TT_BLOCK_TOKENS;      // values lie transposed: one number per 64-token row
            dst[0] = tt_from_float<TAct>(a.x);
            dst[TT_BLOCK_TOKENS] = tt_from_float<TAct>(a.y);
            dst[2 * TT_BLOCK_TOKENS] = tt_from_float<TAct>(a.z);
            dst[3 * TT_BLOCK_TOKENS] = tt_from_float<TAct>(a.w);
        }
    }
}

extern "C" int tt_rope_append(const float* qkv, int splits, long long split_stride,
                              const float* inv_freq, int rotary_dim, float attention_scaling, void* q_out,
                              void* k_pool, void* v_pool, int act_dtype, const int* table, int table_width,
                              int pool_blocks, const int* cu, const int* len_before, int sequences, int n_tokens,
                              int heads, int kv_heads, int head_dim, int write_cache, unsigned* status,
                              cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (rotary_dim < 0 || rotary_dim > head_dim || (rotary_dim & 1)) return (int)cudaErrorInvalidValue;
    const int rot_heads = heads + (write_cache ? kv_heads : 0);
    if (rotary_dim % 8 == 0 && rotary_dim / 2 <= ROPE_MAX_HALF && (head_dim - rotary_dim) % 4 == 0 && split_stride % 4 == 0 && ((uintptr_t)qkv & 15) == 0 &&
        ((uintptr_t)inv_freq & 15) == 0 && ((uintptr_t)q_out & 15) == 0 && ((uintptr_t)k_pool & 15) == 0) {
        const int items4 = rot_heads * (rotary_dim / 8) + rot_heads * ((head_dim - rotary_dim) / 4) + (write_cache ? kv_heads * head_dim / 4 : 0);
        // prompts: one block per token (fewer blocks, each with more loads in flight); few tokens: a block per 128 items
        const int threads4 = n_tokens >= 1024 ? (items4 >= 256 ? 256 : (items4 >= 128 ? 128 : 64)) : 128;
        const dim3 grid4(n_tokens, n_tokens >= 1024 ? 1 : (items4 + threads4 - 1) / threads4);
        if (act_dtype == TT_F32)
            tt_launch_pdl(rope_append_vec_kernel<float>, grid4, dim3(threads4), 0, stream, qkv, splits, (size_t)split_stride, inv_freq, rotary_dim, attention_scaling, (float*)q_out, (float*)k_pool, (float*)v_pool, table, table_width, pool_blocks, cu, len_before, sequences, heads, kv_heads, head_dim, write_cache, status);
        else
            tt_launch_pdl(rope_append_vec_kernel<__nv_bfloat16>, grid4, dim3(threads4), 0, stream, qkv, splits, (size_t)split_stride, inv_freq, rotary_dim, attention_scaling, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, table, table_width, pool_blocks, cu, len_before, sequences, heads, kv_heads, head_dim, write_cache, status);
        TT_LAUNCH_CHECK();
    }
    const int items = rot_heads * (rotary_dim / 2) + rot_heads * (head_dim - rotary_dim) + (write_cache ? kv_heads * head_dim : 0);
    const int threads = 128;
    const dim3 grid(n_tokens, (items + threads - 1) / threads);
    if (grid.y > 65535) return (int)cudaErrorInvalidValue;
    if (act_dtype == TT_F32)
        tt_launch_pdl(rope_append_kernel<float>, dim3(grid), dim3(threads), 0, stream, qkv, splits, (size_t)split_stride, inv_freq, rotary_dim, attention_scaling, (float*)q_out, (float*)k_pool, (float*)v_pool, table, table_width, pool_blocks, cu, len_before, sequences, heads, kv_heads, head_dim, write_cache, status);
    else
        tt_launch_pdl(rope_append_kernel<__nv_bfloat16>, dim3(grid), dim3(threads), 0, stream, qkv, splits, (size_t)split_stride, inv_freq, rotary_dim, attention_scaling, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, table, table_width, pool_blocks, cu, len_before, sequences, heads, kv_heads, head_dim, write_cache, status);
    TT_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------
// The general form of the kernel above, for attention whose queries and keys are normalised per head,
// whose rotation pairs neighbouring numbers, or whose values have another size than its keys.
//   proj: float32 [splits][tokens][cols]; q heads start at column 0, k heads at q_cols, v heads behind them
//         (head_dim numbers per q and k head, value_dim per v head).
//   norm: q_norm / k_norm (float32 [head_dim], or null for none) multiply x / sqrt(mean(x^2) + norm_eps) per head,
//         before the rotation.
//         unit_norm != 0: both are normalised without a weight.
//   query gain: with q_gain_every > 0 the queries at position p are multiplied, after their norm, by
//         1 + q_gain_coef * ln(floor((p + 1) / q_gain_every) + 1)   (float32).
//   rotation of the first rotary_dim numbers of a head by angle inv_freq[i] * float(position):
//         interleaved != 0 pairs (2i, 2i + 1), else (i, i + rotary_dim / 2).
//   value_from_keys != 0: the projection has no value columns; a value head is its key head before the norm
//         (value_dim == head_dim).
// One warp per (token, head); the head's numbers pass through the warp's piece of shared memory.
// ------------------------------------------------------------------------------------
constexpr int QK_WARPS = 4;

template <typename TAct>
__global__ void qk_norm_rope_append_kernel(const float* __restrict__ proj, int splits, size_t split_stride, int cols,
                                           const float* __restrict__ q_norm, const float* __restrict__ k_norm, float norm_eps,
                                           const float* __restrict__ inv_freq, int rotary_dim, int interleaved,
                                           float attention_scaling, TAct* __restrict__ q_out, TAct* __restrict__ k_pool,
                                           TAct* __restrict__ v_pool, const int* __restrict__ table, int table_width,
                                           int pool_blocks, const int* __restrict__ cu, const int* __restrict__ len_before,
                                           int sequences, int n_tokens, int heads, int kv_heads, int head_dim, int value_dim,
                                           int write_cache, const float2* __restrict__ cos_sin, const int2* __restrict__ where,
                                           int unit_norm, float q_gain_coef, int q_gain_every, int value_from_keys,
                                           unsigned* status) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    extern __shared__ float head_shared[];          // QK_WARPS * max(head_dim, value_dim)
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int items = heads + (write_cache ? 2 * kv_heads : 0);
    const long long w = (long long)blockIdx.x * QK_WARPS + warp;
    if (w >= (long long)n_tokens * items) return;
    const int t = (int)(w / items), item = (int)(w - (long long)t * items);
    // with the step's table (see rope_table_kernel) the token's position, sequence, cosines and sines are looked up
    int b, pos;
    if (where) { const int2 at = where[t]; pos = at.x; b = at.y; }
    else { b = tt_find_sequence(cu, sequences, t); pos = len_before[b] + (t - cu[b]); }
    const int* table_row = table + (size_t)b * table_width;
    const float* row = proj + (size_t)t * cols;
    const int q_cols = heads * head_dim, k_cols = kv_heads * head_dim;
    if (item >= heads + kv_heads) {                 // a value head: to the transposed pool as it is
        const int kh = item - heads - kv_heads;
        const long long off = tt_value_offset(table_row, pos, kh, kv_heads, value_dim, pool_blocks, status);
        if (off < 0) return;
        const float* from = value_from_keys ? row + q_cols + kh * head_dim : row + q_cols + k_cols + kh * value_dim;
        for (int d = lane; d < value_dim; d += 32)
            v_pool[off + (long long)d * TT_BLOCK_TOKENS] = tt_from_float<TAct>(sum_slices(from + d, splits, split_stride));
        return;
    }
    const bool is_q = item < heads;
    const int head = is_q ? item : item - heads;
    const float* src = row + (is_q ? head * head_dim : q_cols + head * head_dim);
    const float* norm = is_q ? q_norm : k_norm;
    float* x = head_shared + warp * max(head_dim, value_dim);
    float sumsq = 0.0f;
    for (int d = lane; d < head_dim; d += 32) {
        const float v = sum_slices(src + d, splits, split_stride);
        x[d] = v;
        sumsq += v * v;
    }
    if (norm || unit_norm || (is_q && q_gain_every > 0)) {
        float r = 1.0f;
        if (norm || unit_norm) r = rsqrtf(tt_warp_sum(sumsq) / (float)head_dim + norm_eps);
        if (is_q && q_gain_every > 0) r *= 1.0f + q_gain_coef * logf((float)((pos + 1) / q_gain_every + 1));
        __syncwarp();
        for (int d = lane; d < head_dim; d += 32) x[d] = x[d] * r * (norm ? __ldg(norm + d) : 1.0f);
    }
    __syncwarp();
    TAct* dst;
    if (is_q) {
        dst = q_out + (size_t)t * q_cols + (size_t)head * head_dim;
    } else {
        const long long off = tt_cache_offset(table_row, pos, head, kv_heads, head_dim, pool_blocks, status);
        if (off < 0) return;
        dst = k_pool + off;
    }
    const int half = rotary_dim >> 1;
    for (int i = lane; i < half; i += 32) {
        const int ia = interleaved ? 2 * i : i, ib = interleaved ? 2 * i + 1 : i + half;
        float si, co;
        if (cos_sin) { const float2 cs = cos_sin[(size_t)t * half + i]; co = cs.x; si = cs.y; }
        else sincosf(__ldg(inv_freq + i) * (float)pos, &si, &co);
        co *= attention_scaling;
        si *= attention_scaling;
        const float a = x[ia], c = x[ib];
        dst[ia] = tt_from_float<TAct>(a * co - c * si);
        dst[ib] = tt_from_float<TAct>(c * co + a * si);
    }
    for (int d = rotary_dim + lane; d < head_dim; d += 32) dst[d] = tt_from_float<TAct>(x[d]);
}

extern "C" int tt_qk_norm_rope_append(const float* proj, int splits, long long split_stride, int cols, const float* q_norm,
                                      const float* k_norm, float norm_eps, const float* inv_freq, int rotary_dim, int interleaved,
                                      float attention_scaling, void* q_out, void* k_pool, void* v_pool, int act_dtype,
                                      const int* table, int table_width, int pool_blocks, const int* cu, const int* len_before,
                                      int sequences, int n_tokens, int heads, int kv_heads, int head_dim, int value_dim,
                                      int write_cache, const void* cos_sin_table, const void* where_table, int unit_norm,
                                      float q_gain_coef, int q_gain_every, int value_from_keys, unsigned* status,
                                      cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    const float2* cos_sin = (const float2*)cos_sin_table;        // both or neither: the step's rope table
    const int2* where = (const int2*)where_table;
    if ((cos_sin == nullptr) != (where == nullptr)) return (int)cudaErrorInvalidValue;
    if (rotary_dim < 0 || rotary_dim % 2 || rotary_dim > head_dim || head_dim <= 0 || value_dim <= 0) return (int)cudaErrorInvalidValue;
    if (value_from_keys && value_dim != head_dim) return (int)cudaErrorInvalidValue;
    const long long warps = (long long)n_tokens * (heads + (write_cache ? 2 * kv_heads : 0));
    const unsigned blocks = (unsigned)((warps + QK_WARPS - 1) / QK_WARPS);
    const size_t shared = (size_t)QK_WARPS * (head_dim > value_dim ? head_dim : value_dim) * sizeof(float);
    if (act_dtype == TT_F32)
        tt_launch_pdl(qk_norm_rope_append_kernel<float>, dim3(blocks), dim3(QK_WARPS * 32), shared, stream, proj, splits, (size_t)split_stride, cols, q_norm, k_norm, norm_eps, inv_freq, rotary_dim, interleaved, attention_scaling, (float*)q_out, (float*)k_pool, (float*)v_pool, table, table_width, pool_blocks, cu, len_before, sequences, n_tokens, heads, kv_heads, head_dim, value_dim, write_cache, cos_sin, where, unit_norm, q_gain_coef, q_gain_every, value_from_keys, status);
    else
        tt_launch_pdl(qk_norm_rope_append_kernel<__nv_bfloat16>, dim3(blocks), dim3(QK_WARPS * 32), shared, stream, proj, splits, (size_t)split_stride, cols, q_norm, k_norm, norm_eps, inv_freq, rotary_dim, interleaved, attention_scaling, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, table, table_width, pool_blocks, cu, len_before, sequences, n_tokens, heads, kv_heads, head_dim, value_dim, write_cache, cos_sin, where, unit_norm, q_gain_coef, q_gain_every, value_from_keys, status);
    TT_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------
// What every layer's rotation of a step has in common, computed once per step: for packed token t
// its position p = len_before[b] + (t - cu[b]), its sequence b, and cos and sin of inv_freq[i] * p
// (float32 angle, as in the kernels above).  The tensor-core qkv product's epilogue reads these
// instead of finding the sequence and calling sincosf again in each of the model's layers.
//   cos_sin: float2 [tokens][half]; where: int2 [tokens] = (position, sequence)
// ------------------------------------------------------------------------------------
__global__ void rope_table_kernel(const float* __restrict__ inv_freq, int half, const int* __restrict__ cu,
                                  const int* __restrict__ len_before, int sequences, float2* __restrict__ cos_sin,
                                  int2* __restrict__ where) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    const int t = blockIdx.x;
    const int b = tt_find_sequence(cu, sequences, t);
    const int pos = len_before[b] + (t - cu[b]);
    if (threadIdx.x == 0) where[t] = make_int2(pos, b);
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float si, co;
        sincosf(__ldg(inv_freq + i) * (float)pos, &si, &co);
        cos_sin[(size_t)t * half + i] = make_float2(co, si);
    }
}

extern "C" int tt_rope_table(const float* inv_freq, int half, const int* cu, const int* len_before, int sequences, int n_tokens,
                             void* cos_sin, void* where, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (half <= 0) return (int)cudaErrorInvalidValue;
    const int threads = half >= 64 ? 64 : 32;
    tt_launch_pdl(rope_table_kernel, dim3(n_tokens), dim3(threads), 0, stream, inv_freq, half, cu, len_before, sequences, (float2*)cos_sin, (int2*)where);
    TT_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------
// Gated unit: act[t, j] = f(gate[t, j]) * up[t, j].  f by `activation`: 0 silu(g) = g / (1 + exp(-g)),
// 1 relu, 2 the tanh form of gelu, 0.5 g (1 + tanh(sqrt(2 / pi) (g + 0.044715 g^3))).
// gate_up: float32 [splits][tokens][2 * inter], gate columns first.
// ------------------------------------------------------------------------------------
__device__ __forceinline__ float tt_gate_activation(float g, int activation) {
    if (activation == 1) return fmaxf(g, 0.0f);
    if (activation == 2) return 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
    return g / (1.0f + expf(-g));
}

template <typename TAct>
__global__ void swiglu_kernel(const float* __restrict__ gate_up, int splits, size_t split_stride,
                              TAct* __restrict__ act, int inter, size_t total, int activation) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t t = idx / inter;
    const int j = (int)(idx - t * inter);
    const float* row = gate_up + t * (size_t)(2 * inter);
    float g = 0.0f, u = 0.0f;
#pragma unroll 4
    for (int s = 0; s < splits; ++s) {                  // gate and up of up to four slices in flight together
        g += __ldg(row + s * split_stride + j);
        u += __ldg(row + s * split_stride + inter + j);
    }
    act[idx] = tt_from_float<TAct>(tt_gate_activation(g, activation) * u);
}

extern "C" int tt_swiglu(const float* gate_up, int splits, long long split_stride, void* act,
                         int act_dtype, int n_tokens, int inter, int activation, cudaStream_t stream) {
    const size_t total = (size_t)n_tokens * inter;
    if (total == 0) return 0;
    const int threads = 256;
    const unsigned blocks = (unsigned)((total + threads - 1) / threads);
    if (act_dtype == TT_F32)
        tt_launch_pdl(swiglu_kernel<float>, dim3(blocks), dim3(threads), 0, stream, gate_up, splits, (size_t)split_stride, (float*)act, inter, total, activation);
    else
        tt_launch_pdl(swiglu_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream, gate_up, splits, (size_t)split_stride, (__nv_bfloat16*)act, inter, total, activation);
    TT_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------
// after a step: len[b] += cu[b + 1] - cu[b]; counters[b] += 1 where the caller keeps a count of
// the steps each sequence has taken (the sampler's random numbers are indexed by it)
// ------------------------------------------------------------------------------------
__global__ void advance_lengths_kernel(int* __restrict__ len, const int* __restrict__ cu, int* __restrict__ counters, int sequences) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b < sequences) {
        len[b] += cu[b + 1] - cu[b];
        if (counters) counters[b] += 1;
    }
}

extern "C" int tt_advance_lengths(int* len, const int* cu, int* counters, int sequences, cudaStream_t stream) {
    if (sequences <= 0) return 0;
    tt_launch_pdl(advance_lengths_kernel, dim3((sequences + 127) / 128), dim3(128), 0, stream, len, cu, counters, sequences);
    TT_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------
// A few int32 numbers between device memory and pinned host memory that the device can
// address (token ids in, sampled ids out): as a kernel in the chain of a step this costs
// a fraction of a copy node in a CUDA graph.  Host memory is read and written uncached.
// ------------------------------------------------------------------------------------
__global__ void copy_int32_kernel(int* __restrict__ dst, const int* __restrict__ src, int n, const int* __restrict__ extra) {
    tt_pdl_wait();
    tt_pdl_launch_dependents();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) __stcg(dst + i, __ldcv(src + i));
    if (extra && i == n) __stcg(dst + n, __ldcv(extra));
}

// extra: one more int32 (the device status word, say) that is copied to dst[n]; may be null.
extern "C" int tt_copy_int32(int* dst, const int* src, int n, const int* extra, cudaStream_t stream) {
    if (n <= 0) return 0;
    tt_launch_pdl(copy_int32_kernel, dim3((n + 1 + 127) / 128), dim3(128), 0, stream, dst, src, n, extra);
    TT_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------
// Embedding with a hashed row for the pair (previous token, token):
//   residual[t] = table[token] * scale + pair_table[(prev * mul_prev + token * mul_cur) mod buckets]
// and row `buckets` (the last) of pair_table for a sequence's first token.  The previous token of a
// step's first token comes from the sequence's state, one int32 per slot that holds the last token
// plus one (zero: the sequence has no token yet); the block of a sequence's first token of the step
// reads it and then moves it on to the step's last token, so nobody else touches it.
// ------------------------------------------------------------------------------------
template <typename TW>
__global__ void embed_pair_gather_kernel(const TW* __restrict__ table, const TW* __restrict__ pair_table,
                                         const int* __restrict__ tokens, const int* __restrict__ cu,
                                         const int* __restrict__ slots, int sequences, int* __restrict__ last_token,
                                         float* __restrict__ residual, int hidden, int vocab, int buckets, long long mul_prev,
                                         long long mul_cur, float scale, unsigned* status) {
    tt_pdl_wait();                      // the first kernel of a step: see embed_gather_kernel
    tt_pdl_launch_dependents();
    const int t = blockIdx.x;
    const int b = tt_find_sequence(cu, sequences, t);
    const int id = tokens[t];
    int prev_plus_one;
    if (t == cu[b]) {
        int* st = last_token + slots[b];
        prev_plus_one = *st;
        __syncthreads();                // every thread has read the state before one of them moves it on
        if (threadIdx.x == 0) *st = tokens[cu[b + 1] - 1] + 1;
    } else {
        prev_plus_one = tokens[t - 1] + 1;
    }
    float* out = residual + (size_t)t * hidden;
    if (id < 0 || id >= vocab || prev_plus_one < 0 || prev_plus_one > vocab) {
        if (threadIdx.x == 0) atomicOr(status, TT_STATUS_BAD_TOKEN);
        for (int j = threadIdx.x; j < hidden; j += blockDim.x) out[j] = 0.0f;
        return;
    }
    const long long pair = prev_plus_one == 0 ? (long long)buckets
                                              : ((long long)(prev_plus_one - 1) * mul_prev + (long long)id * mul_cur) % buckets;
    const TW* row = table + (size_t)id * hidden;
    const TW* extra = pair_table + (size_t)pair * hidden;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) out[j] = tt_to_float(row[j]) * scale + tt_to_float(extra[j]);
}

extern "C" int tt_embed_pair_gather(const void* table, const void* pair_table, int table_dtype, const int* tokens, const int* cu,
                                    const int* slots, int sequences, int* last_token, float* residual, int n_tokens, int hidden,
                                    int vocab, int buckets, long long mul_prev, long long mul_cur, float scale, unsigned* status,
                                    cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (buckets <= 0 || mul_prev < 0 || mul_cur < 0) return (int)cudaErrorInvalidValue;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (table_dtype == TT_F32)
        tt_launch_pdl(embed_pair_gather_kernel<float>, dim3(n_tokens), dim3(threads), 0, stream, (const float*)table, (const float*)pair_table, tokens, cu, slots, sequences, last_token, residual, hidden, vocab, buckets, mul_prev, mul_cur, scale, status);
    else
        tt_launch_pdl(embed_pair_gather_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0, stream, (const __nv_bfloat16*)table, (const __nv_bfloat16*)pair_table, tokens, cu, slots, sequences, last_token, residual, hidden, vocab, buckets, mul_prev, mul_cur, scale, status);
    TT_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------
// Token shift: out[t] = x[t] + (x[t - 1] - x[t]) * mix, element by element, where x[t - 1] of a step's
// first token is the sequence's state (float32 [slots][hidden], zero for a new sequence).  The block of a
// sequence's first token of the step reads the state and moves it on to the step's last x, element by
// element in the same thread.
// ------------------------------------------------------------------------------------
template <typename T>
__global__ void token_shift_kernel(const T* __restrict__ x, const float* __restrict__ mix, float* __restrict__ state,
                                   T* __restrict__ out, const int* __restrict__ cu, const int* __restrict__ slots, int sequences,
                                   int hidden) {
    tt_pdl_launch_dependents();
    const int t = blockIdx.x;
    const int b = tt_find_sequence(cu, sequences, t);
    const int first = cu[b], last = cu[b + 1] - 1;
    tt_pdl_wait();
    const T* cur = x + (size_t)t * hidden;
    T* o = out + (size_t)t * hidden;
    if (t == first) {
        float* st = state + (size_t)slots[b] * hidden;
        const T* tail = x + (size_t)last * hidden;
        for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
            const float before = st[j], now = tt_to_float(cur[j]);
            st[j] = tt_to_float(tail[j]);
            o[j] = tt_from_float<T>(fmaf(before - now, __ldg(mix + j), now));
        }
    } else {
        const T* prev = cur - hidden;
        for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
            const float before = tt_to_float(prev[j]), now = tt_to_float(cur[j]);
            o[j] = tt_from_float<T>(fmaf(before - now, __ldg(mix + j), now));
        }
    }
}

extern "C" int tt_token_shift(const void* x, int dtype, const float* mix, float* state, void* out, const int* cu, const int* slots,
                              int sequences, int n_tokens, int hidden, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (dtype == TT_F32)
        tt_launch_pdl(token_shift_kernel<float>, dim3(n_tokens), dim3(threads), 0, stream, (const float*)x, mix, state, (float*)out, cu, slots, sequences, hidden);
    else
        tt_launch_pdl(token_shift_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0, stream, (const __nv_bfloat16*)x, mix, state, (__nv_bfloat16*)out, cu, slots, sequences, hidden);
    TT_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------
// embedding with a learned position vector:
//   residual[t, :] = table[token[t], :] * scale + positions[p, :],  p = len_before[b] + (t - cu[b])   (float32 out)
// A token outside the table, or a position beyond the position table's rows, raises the bad-token bit and leaves zeros.
// ------------------------------------------------------------------------------------
template <typename TW>
__global__ void embed_position_gather_kernel(const TW* __restrict__ table, const TW* __restrict__ positions,
                                             const int* __restrict__ tokens, const int* __restrict__ cu,
                                             const int* __restrict__ len_before, int sequences, float* __restrict__ residual,
                                             int hidden, int vocab, int max_positions, float scale, unsigned* status) {
    tt_pdl_wait();                      // the first kernel of a step: see embed_gather_kernel
    tt_pdl_launch_dependents();
    const int t = blockIdx.x;
    const int id = tokens[t];
    const int b = tt_find_sequence(cu, sequences, t);
    const int pos = len_before[b] + (t - cu[b]);
    float* out = residual + (size_t)t * hidden;
    if (id < 0 || id >= vocab || pos < 0 || pos >= max_positions) {
        if (threadIdx.x == 0) atomicOr(status, TT_STATUS_BAD_TOKEN);
        for (int j = threadIdx.x; j < hidden; j += blockDim.x) out[j] = 0.0f;
        return;
    }
    const TW* row = table + (size_t)id * hidden;
    const TW* prow = positions + (size_t)pos * hidden;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x)
        out[j] = tt_to_float(row[j]) * scale + tt_to_float(prow[j]);
}

extern "C" int tt_embed_position_gather(const void* table, const void* positions, int table_dtype, const int* tokens, const int* cu,
                                        const int* len_before, int sequences, float* residual, int n_tokens, int hidden, int vocab,
                                        int max_positions, float scale, unsigned* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (table_dtype == TT_F32)
        tt_launch_pdl(embed_position_gather_kernel<float>, dim3(n_tokens), dim3(threads), 0, stream, (const float*)table, (const float*)positions, tokens, cu, len_before, sequences, residual, hidden, vocab, max_positions, scale, status);
    else
        tt_launch_pdl(embed_position_gather_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0, stream, (const __nv_bfloat16*)table, (const __nv_bfloat16*)positions, tokens, cu, len_before, sequences, residual, hidden, vocab, max_positions, scale, status);
    TT_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------
// Ungated activation: act[t, j] = f(sum over slices of x[s][t, j]).  f by `activation`: 0 silu, 1 relu, 2 tanh-gelu (as
// in tt_gate_activation), 4 the exact gelu 0.5 z (1 + erf(z / sqrt 2)), 3 xielu with two numbers a = softplus(p) and c = 1/2 + softplus(q) that the caller has formed:
//   z > 0: a z^2 + z / 2;   z <= 0: c (exp(z) - 1 - z) + z / 2     (expm1f keeps small z exact)
// ------------------------------------------------------------------------------------
__device__ __forceinline__ float tt_unary_activation(float z, int activation, float a, float c) {
    if (activation == 4) return 0.5f * z * (1.0f + erff(z * 0.70710678118654752f));        // the exact gelu
    if (activation == 3) return z > 0.0f ? fmaf(a * z, z, 0.5f * z) : fmaf(c, expm1f(z) - z, 0.5f * z);
    return tt_gate_activation(z, activation);
}

template <typename TAct>
__global__ void activation_kernel(const float* __restrict__ x, int splits, size_t split_stride, TAct* __restrict__ act,
                                  size_t total, int activation, float a, float c) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    const size_t idx = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (idx >= total) return;
    if (idx + 4 <= total && (split_stride & 3) == 0) {
        float4 z = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (int s = 0; s < splits; ++s) {
            const float4 v = __ldg(reinterpret_cast<const float4*>(x + s * split_stride + idx));
            z.x += v.x; z.y += v.y; z.z += v.z; z.w += v.w;
        }
        tt_store4(act + idx, tt_unary_activation(z.x, activation, a, c), tt_unary_activation(z.y, activation, a, c),
                  tt_unary_activation(z.z, activation, a, c), tt_unary_activation(z.w, activation, a, c));
        return;
    }
    for (size_t i = idx; i < total && i < idx + 4; ++i) {
        float z = 0.0f;
        for (int s = 0; s < splits; ++s) z += __ldg(x + s * split_stride + i);
        act[i] = tt_from_float<TAct>(tt_unary_activation(z, activation, a, c));
    }
}

extern "C" int tt_activation(const float* x, int splits, long long split_stride, void* act, int act_dtype, long long total,
                             int activation, float a, float c, cudaStream_t stream) {
    if (total <= 0) return 0;
    if (activation < 0 || activation > 4) return (int)cudaErrorInvalidValue;
    const int threads = 256;
    const unsigned blocks = (unsigned)(((total + 3) / 4 + threads - 1) / threads);      // a thread takes four numbers; the last one what is left
    if (act_dtype == TT_F32)
        tt_launch_pdl(activation_kernel<float>, dim3(blocks), dim3(threads), 0, stream, x, splits, (size_t)split_stride, (float*)act, (size_t)total, activation, a, c);
    else
        tt_launch_pdl(activation_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream, x, splits, (size_t)split_stride, (__nv_bfloat16*)act, (size_t)total, activation, a, c);
    TT_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------
// The residual addition and RMSNorm of add_rmsnorm_kernel with two more steps on the way, all float32:
//   v = delta[0][r] + delta[1][r] + ...                                        (fixed order; no delta: v = 0)
//   post_weight:  v = v * rsqrt(mean(v^2) + post_eps) * (post_weight + post_offset)     (the norm after a sublayer)
//   x = residual[r] + v
//   results:      results[index][r] = x;  with depth_weights: x = sum_{j <= index} depth_weights[j] * results[j][r]
//                 (result `index` is taken from the registers; the sum runs from j = 0 upwards)
//   residual[r] = x                                                            (only when rows == nullptr)
//   out[i] = x * rsqrt(mean(x^2) + eps) * (weight + weight_offset)
// With `rows`, output row i comes from row rows[i] and neither the stream nor the results are written.
// One block per output row; the row passes through shared memory between the reductions, and a thread only ever
// revisits its own numbers of it, four at a time when the width and the strides allow 16-byte accesses.
// ------------------------------------------------------------------------------------
// VEC numbers of a row at a time: 4 (16-byte loads and stores) when the width and every stride are multiples of four.
template <int VEC> struct ChainPack { float v[VEC]; };
template <int VEC> __device__ __forceinline__ ChainPack<VEC> chain_load(const float* p) {
    ChainPack<VEC> r;
    if constexpr (VEC == 4) {
        const float4 x = *reinterpret_cast<const float4*>(p);
        r.v[0] = x.x; r.v[1] = x.y; r.v[2] = x.z; r.v[3] = x.w;
    } else {
        r.v[0] = *p;
    }
    return r;
}
template <int VEC> __device__ __forceinline__ void chain_store(float* p, const ChainPack<VEC>& r) {
    if constexpr (VEC == 4) *reinterpret_cast<float4*>(p) = make_float4(r.v[0], r.v[1], r.v[2], r.v[3]);
    else *p = r.v[0];
}
template <int VEC, typename TOut> __device__ __forceinline__ void chain_store_out(TOut* p, const ChainPack<VEC>& r) {
    if constexpr (VEC == 4) tt_store4(p, r.v[0], r.v[1], r.v[2], r.v[3]);
    else *p = tt_from_float<TOut>(r.v[0]);
}

template <typename TOut, int VEC>
__global__ void __launch_bounds__(1024)
add_rmsnorm_chain_kernel(float* __restrict__ residual, const float* __restrict__ delta, int splits, size_t split_stride,
                         const float* __restrict__ post_weight, float post_offset, float post_eps,
                         float* __restrict__ results, size_t result_stride, int index, const float* __restrict__ depth_weights,
                         const float* __restrict__ weight, float weight_offset, float eps, TOut* __restrict__ out,
                         const int* __restrict__ rows, int hidden) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    extern __shared__ __align__(16) float chain_shared[];     // hidden floats (the row), then 32 for the reductions
    float* rowbuf = chain_shared;
    float* reduce = chain_shared + hidden;
    const int i = blockIdx.x;
    const int r = rows ? rows[i] : i;
    float* res = residual + (size_t)r * hidden;
    const int first = threadIdx.x * VEC, step = blockDim.x * VEC;
    using Pack = ChainPack<VEC>;
    // 1. the delta's slices, summed, and their mean square
    float sumsq = 0.0f;
    if (delta) {
        const float* del = delta + (size_t)r * hidden;
        for (int j = first; j < hidden; j += step) {
            Pack v = chain_load<VEC>(del + j);
            for (int s = 1; s < splits; ++s) {
                const Pack more = chain_load<VEC>(del + (size_t)s * split_stride + j);
#pragma unroll
                for (int e = 0; e < VEC; ++e) v.v[e] += more.v[e];
            }
            chain_store<VEC>(rowbuf + j, v);
#pragma unroll
            for (int e = 0; e < VEC; ++e) sumsq += v.v[e] * v.v[e];
        }
    } else {
        for (int j = threadIdx.x; j < hidden; j += blockDim.x) rowbuf[j] = 0.0f;
    }
    float gain = 1.0f;
    if (post_weight) gain = rsqrtf(tt_block_sum(sumsq, reduce) / (float)hidden + post_eps);
    // 2. into the stream, kept as a result, mixed with the earlier results; every thread revisits its own numbers only
    sumsq = 0.0f;
    for (int j = first; j < hidden; j += step) {
        Pack v = chain_load<VEC>(rowbuf + j);
        if (post_weight) {
            const Pack w = chain_load<VEC>(post_weight + j);
#pragma unroll
            for (int e = 0; e < VEC; ++e) v.v[e] = v.v[e] * gain * (w.v[e] + post_offset);
        }
        Pack x = chain_load<VEC>(res + j);
#pragma unroll
        for (int e = 0; e < VEC; ++e) x.v[e] += v.v[e];
        if (results) {
            const float* mine = results + (size_t)r * hidden + j;
            if (!rows) chain_store<VEC>(results + (size_t)index * result_stride + (size_t)r * hidden + j, x);
            if (depth_weights) {
                Pack mixed;
#pragma unroll
                for (int e = 0; e < VEC; ++e) mixed.v[e] = 0.0f;
                for (int k = 0; k < index; ++k) {
                    const float wk = __ldg(depth_weights + k);
                    const Pack earlier = chain_load<VEC>(mine + (size_t)k * result_stride);
#pragma unroll
                    for (int e = 0; e < VEC; ++e) mixed.v[e] = fmaf(wk, earlier.v[e], mixed.v[e]);
                }
                const float wi = __ldg(depth_weights + index);
#pragma unroll
                for (int e = 0; e < VEC; ++e) x.v[e] = fmaf(wi, x.v[e], mixed.v[e]);
            }
        }
        if (!rows) chain_store<VEC>(res + j, x);
        chain_store<VEC>(rowbuf + j, x);
#pragma unroll
        for (int e = 0; e < VEC; ++e) sumsq += x.v[e] * x.v[e];
    }
    const float rstd = rsqrtf(tt_block_sum(sumsq, reduce) / (float)hidden + eps);
    TOut* o = out + (size_t)i * hidden;
    for (int j = first; j < hidden; j += step) {
        Pack x = chain_load<VEC>(rowbuf + j);
        const Pack w = chain_load<VEC>(weight + j);
#pragma unroll
        for (int e = 0; e < VEC; ++e) x.v[e] = x.v[e] * rstd * (w.v[e] + weight_offset);
        chain_store_out<VEC>(o + j, x);
    }
}

extern "C" int tt_add_rmsnorm_chain(float* residual, const float* delta, int splits, long long split_stride, const float* post_weight,
                                    float post_offset, float post_eps, float* results, long long result_stride, int index,
                                    const float* depth_weights, const float* weight, float weight_offset, float eps, void* out,
                                    int out_dtype, const int* rows, int n_rows, int hidden, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (hidden <= 0 || index < 0 || (depth_weights && !results)) return (int)cudaErrorInvalidValue;
    const size_t shared = ((size_t)hidden + 32) * sizeof(float);
    if (shared > 200 * 1024) return (int)cudaErrorInvalidValue;
    const bool wide = (hidden & 3) == 0 && (split_stride & 3) == 0 && (result_stride & 3) == 0 &&
                      ((((uintptr_t)residual | (uintptr_t)delta | (uintptr_t)post_weight | (uintptr_t)results | (uintptr_t)weight | (uintptr_t)out) & 15) == 0);
    const int per_thread = wide ? 4 : 1;
    int threads = hidden / per_thread >= 1024 ? 1024 : hidden / per_thread >= 512 ? 512 : hidden / per_thread >= 256 ? 256 : 128;
#define TT_CHAIN_LAUNCH(TOUT, VEC)                                                                                                              \
    do {                                                                                                                                        \
        if (shared > 48 * 1024) cudaFuncSetAttribute(add_rmsnorm_chain_kernel<TOUT, VEC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared); \
        tt_launch_pdl(add_rmsnorm_chain_kernel<TOUT, VEC>, dim3(n_rows), dim3(threads), shared, stream, residual, delta, splits, (size_t)split_stride, post_weight, post_offset, post_eps, results, (size_t)result_stride, index, depth_weights, weight, weight_offset, eps, (TOUT*)out, rows, hidden); \
    } while (0)
    if (out_dtype == TT_F32) {
        if (wide) TT_CHAIN_LAUNCH(float, 4); else TT_CHAIN_LAUNCH(float, 1);
    } else {
        if (wide) TT_CHAIN_LAUNCH(__nv_bfloat16, 4); else TT_CHAIN_LAUNCH(__nv_bfloat16, 1);
    }
#undef TT_CHAIN_LAUNCH
    TT_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------
// The stream takes a delta and is handed on narrowed: residual[r] += delta[0][r] + delta[1][r] + ... (fixed order; no delta:
// nothing is added), out[r] = residual[r] in the activation dtype.  For a part that reads the stream itself, not a norm of it.
// ------------------------------------------------------------------------------------
template <typename TOut>
__global__ void add_narrow_kernel(float* __restrict__ residual, const float* __restrict__ delta, int splits, size_t split_stride,
                                  TOut* __restrict__ out, size_t total) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    float x = residual[i];
    if (splits > 0) {
        for (int s = 0; s < splits; ++s) x += __ldg(delta + s * split_stride + i);
        residual[i] = x;
    }
    out[i] = tt_from_float<TOut>(x);
}

extern "C" int tt_add_narrow(float* residual, const float* delta, int splits, long long split_stride, void* out, int out_dtype,
                             long long total, cudaStream_t stream) {
    if (total <= 0) return 0;
    const int threads = 256;
    const unsigned blocks = (unsigned)((total + threads - 1) / threads);
    if (!delta) splits = 0;
    if (out_dtype == TT_F32)
        tt_launch_pdl(add_narrow_kernel<float>, dim3(blocks), dim3(threads), 0, stream, residual, delta, splits, (size_t)split_stride, (float*)out, (size_t)total);
    else
        tt_launch_pdl(add_narrow_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream, residual, delta, splits, (size_t)split_stride, (__nv_bfloat16*)out, (size_t)total);
    TT_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------
// A gate times a slice of a second embedding of the token: out[t][j] = gelu_tanh(sum over slices of x[s][t][j]) *
// table[tokens[t]][col_off + j], j < dim; the table has `table_cols` numbers a row.  A token outside the table raises the
// status word's bad-token bit and gets zeros.
// ------------------------------------------------------------------------------------
template <typename TOut, typename TW>
__global__ void token_side_gate_kernel(const float* __restrict__ x, int splits, size_t split_stride, const TW* __restrict__ table,
                                       int vocab, int table_cols, int col_off, const int* __restrict__ tokens, int dim,
                                       TOut* __restrict__ out, size_t total, unsigned* status) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t t = i / dim;
    const int j = (int)(i - t * dim);
    const int id = tokens[t];
    if (id < 0 || id >= vocab) {
        atomicOr(status, TT_STATUS_BAD_TOKEN);
        out[i] = tt_from_float<TOut>(0.0f);
        return;
    }
    float z = 0.0f;
    for (int s = 0; s < splits; ++s) z += __ldg(x + s * split_stride + i);
    out[i] = tt_from_float<TOut>(tt_gate_activation(z, 2) * tt_to_float(table[(size_t)id * table_cols + col_off + j]));
}

extern "C" int tt_token_side_gate(const float* x, int splits, long long split_stride, const void* table, int table_dtype, int vocab,
                                  int table_cols, int col_off, const int* tokens, int n_tokens, int dim, void* out, int out_dtype,
                                  unsigned* status, cudaStream_t stream) {
    const size_t total = (size_t)n_tokens * dim;
    if (total == 0) return 0;
    if (col_off < 0 || col_off + dim > table_cols) return (int)cudaErrorInvalidValue;
    const int threads = 256;
    const unsigned blocks = (unsigned)((total + threads - 1) / threads);
#define TT_SIDE(TO, TW) tt_launch_pdl(token_side_gate_kernel<TO, TW>, dim3(blocks), dim3(threads), 0, stream, x, splits, (size_t)split_stride, (const TW*)table, vocab, table_cols, col_off, tokens, dim, (TO*)out, total, status)
    if (out_dtype == TT_F32 && table_dtype == TT_F32) TT_SIDE(float, float);
    else if (out_dtype == TT_F32) TT_SIDE(float, __nv_bfloat16);
    else if (table_dtype == TT_F32) TT_SIDE(__nv_bfloat16, float);
    else TT_SIDE(__nv_bfloat16, __nv_bfloat16);
#undef TT_SIDE
    TT_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------
// A sigmoid gate on a mixer's read-out, in place: y[t][c] *= sigmoid(sum over slices of gate[s][t][...]) with one gate
// number per output number (column c) or per head (column c / head_width).  gate stands at the gate's first column; its
// rows are gate_row numbers apart.
// ------------------------------------------------------------------------------------
template <typename T>
__global__ void sigmoid_gate_kernel(T* __restrict__ y, int cols, const float* __restrict__ gate, int splits, size_t split_stride,
                                    int gate_row, int head_width, size_t total) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t t = i / cols;
    const int c = (int)(i - t * cols);
    const float* g = gate + t * (size_t)gate_row + (head_width > 0 ? c / head_width : c);
    float z = 0.0f;
    for (int s = 0; s < splits; ++s) z += __ldg(g + s * split_stride);
    y[i] = tt_from_float<T>(tt_to_float(y[i]) / (1.0f + expf(-z)));
}

// the same for bfloat16 rows of whole 16-byte pieces: eight numbers a thread, with a gate number each (head_width 0) or one
// for the head they all lie in (head_width a multiple of eight)
__global__ void sigmoid_gate_vec_kernel(__nv_bfloat16* __restrict__ y, int cols, const float* __restrict__ gate, int splits,
                                        size_t split_stride, int gate_row, int head_width, size_t total) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (i >= total) return;
    const size_t t = i / cols;
    const int c = (int)(i - t * cols);
    float z[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) z[e] = 0.0f;
    if (head_width > 0) {
        const float* g = gate + t * (size_t)gate_row + c / head_width;
        float one = 0.0f;
        for (int s = 0; s < splits; ++s) one += __ldg(g + s * split_stride);
#pragma unroll
        for (int e = 0; e < 8; ++e) z[e] = one;
    } else {
        const float* g = gate + t * (size_t)gate_row + c;
        for (int s = 0; s < splits; ++s) {
            const float4 a = __ldg(reinterpret_cast<const float4*>(g + s * split_stride)), b = __ldg(reinterpret_cast<const float4*>(g + s * split_stride + 4));
            z[0] += a.x; z[1] += a.y; z[2] += a.z; z[3] += a.w; z[4] += b.x; z[5] += b.y; z[6] += b.z; z[7] += b.w;
        }
    }
    uint4 raw = *reinterpret_cast<uint4*>(y + i);
    __nv_bfloat16* v = reinterpret_cast<__nv_bfloat16*>(&raw);
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = __float2bfloat16_rn(__bfloat162float(v[e]) / (1.0f + expf(-z[e])));
    *reinterpret_cast<uint4*>(y + i) = raw;
}

extern "C" int tt_sigmoid_gate(void* y, int dtype, int n_tokens, int cols, const float* gate, int splits, long long split_stride,
                               int gate_row, int head_width, cudaStream_t stream) {
    const size_t total = (size_t)n_tokens * cols;
    if (total == 0) return 0;
    const int threads = 256;
    const bool each = head_width <= 0 && gate_row % 4 == 0 && split_stride % 4 == 0 && ((uintptr_t)gate & 15) == 0;
    if (dtype == TT_BF16 && cols % 8 == 0 && ((uintptr_t)y & 15) == 0 && (each || (head_width > 0 && head_width % 8 == 0))) {
        tt_launch_pdl(sigmoid_gate_vec_kernel, dim3((unsigned)((total / 8 + threads - 1) / threads)), dim3(threads), 0, stream, (__nv_bfloat16*)y, cols,
                      gate, splits, (size_t)split_stride, gate_row, head_width > 0 ? head_width : 0, total);
        TT_LAUNCH_CHECK();
    }
    const unsigned blocks = (unsigned)((total + threads - 1) / threads);
    if (dtype == TT_F32)
        tt_launch_pdl(sigmoid_gate_kernel<float>, dim3(blocks), dim3(threads), 0, stream, (float*)y, cols, gate, splits, (size_t)split_stride, gate_row, head_width, total);
    else
        tt_launch_pdl(sigmoid_gate_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream, (__nv_bfloat16*)y, cols, gate, splits, (size_t)split_stride, gate_row, head_width, total);
    TT_LAUNCH_CHECK();
}
