// Routing of a mixture of experts.
//
// tt_route_topk: one warp per token.  Scores are the softmax of the router's logits over all experts (float32).
// Experts form `groups` equal groups of neighbours; a group's score is its largest expert score, and only experts of
// the `keep` groups with the largest scores can be chosen.  Of those the `top` largest are chosen (ties: the lower
// index), and their weights are their scores divided by the sum of the chosen scores (+ 1e-20).  The kernel writes
// the chosen experts and weights ([tokens][top]) and the same as a dense table ([tokens][experts], zero where an
// expert is not chosen).
//
// Options (RouteOptions): sigmoid scores instead of the softmax, a correction added for the choice only, groups scored by
// their two best, weights left as the scores, and gates of always-on experts from further rows of the router's matrix.
//
// tt_route_rows: the same with the router's product in front, from the token's row and the router's matrix.
//
// tt_expert_activation: the clamped gated unit of every expert's columns times the token's gate for that expert.
//
// tt_scale_expert_columns: act[t][e * width + j] *= gates[t][e] for the first experts * width columns of act; the next
// shared_width columns (an always-on expert's) are multiplied by gates[t][experts], and columns behind those stay as they are.
#include "common.cuh"

constexpr int ROUTE_MAX_EXPERTS = 512;      // a lane holds ROUTE_MAX_EXPERTS / 32 scores
constexpr int ROUTE_WARPS = 4;

// the largest value among the lanes' candidates and the lowest index that has it
__device__ __forceinline__ void route_argmax(float& value, int& index) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float v = __shfl_xor_sync(0xffffffffu, value, o);
        const int i = __shfl_xor_sync(0xffffffffu, index, o);
        if (v > value || (v == value && i < index)) { value = v; index = i; }
    }
}

// How the scores are made and used (all zero: softmax scores, a group scored by its best expert, weights renormalised).
//   sigmoid: scores are sigmoid(logit) instead of the softmax over all experts.
//   correction (float32 [experts] or null): added to the scores for the CHOICE only (groups and top); weights use the scores.
//   group_top2: a group's score is the sum of its two largest choice scores (its only one, for groups of one expert).
//   plain_weights: the weights are the chosen scores themselves instead of score / (sum of the chosen + 1e-20).
//   extra: so many more logits follow the experts'; gates[t][experts + k] = sigmoid(logit) for each (the gate of an
//   expert that every token uses).  A row of `gates` has experts + extra numbers.
struct RouteOptions {
    int sigmoid;
    const float* correction;
    int group_top2;
    int plain_weights;
    int extra;
};

// One warp routes token t from its logits (`splits` partial sums `split_stride` apart); group_best: 32 floats of the warp's own.
__device__ __forceinline__ void route_token(const float* __restrict__ logits, int splits, size_t split_stride, int t, int experts,
                                            int top, int groups, int keep, float* __restrict__ gates, int* __restrict__ chosen,
                                            float* __restrict__ weights, float* group_best_row, const RouteOptions opt) {
    const int lane = threadIdx.x & 31;
    constexpr int PER = ROUTE_MAX_EXPERTS / 32;
    float s[PER];                                               // score of expert lane + 32 * i
    float c[PER];                                               // its choice score; -inf: cannot be chosen (any more)
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int e = lane + 32 * i;
        s[i] = -INFINITY;
        if (e < experts) {
            float z = 0.0f;
            for (int k = 0; k < splits; ++k) z += logits[(size_t)k * split_stride + e];
            s[i] = z;
            m = fmaxf(m, z);
        }
    }
    if (opt.sigmoid) {
#pragma unroll
        for (int i = 0; i < PER; ++i)
            if (lane + 32 * i < experts) s[i] = 1.0f / (1.0f + expf(-s[i]));
    } else {
        m = tt_warp_max(m);
        float total = 0.0f;
#pragma unroll
        for (int i = 0; i < PER; ++i)
            if (lane + 32 * i < experts) { s[i] = expf(s[i] - m); total += s[i]; }
        total = tt_warp_sum(total);
        const float inv = 1.0f / total;
#pragma unroll
        for (int i = 0; i < PER; ++i)
            if (lane + 32 * i < experts) s[i] *= inv;
    }
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int e = lane + 32 * i;
        c[i] = e < experts ? s[i] + (opt.correction ? __ldg(opt.correction + e) : 0.0f) : -INFINITY;
    }
    const int row = experts + opt.extra;
    if (lane < opt.extra) {                                     // gates of the always-on experts
        float z = 0.0f;
        for (int k = 0; k < splits; ++k) z += logits[(size_t)k * split_stride + experts + lane];
        gates[(size_t)t * row + experts + lane] = 1.0f / (1.0f + expf(-z));
    }

    // groups: a bit per group that stays (groups <= 32)
    const int size = experts / groups;
    unsigned kept = 0xffffffffu;
    if (groups > 1 && keep < groups) {
        for (int g = 0; g < groups; ++g) {
            float best = -INFINITY;
            int where = 0x7fffffff;
#pragma unroll
            for (int i = 0; i < PER; ++i) {
                const int e = lane + 32 * i;
                if (e < experts && e / size == g && c[i] > best) { best = c[i]; where = e; }
            }
            route_argmax(best, where);
            if (opt.group_top2 && size > 1) {
                float second = -INFINITY;
#pragma unroll
                for (int i = 0; i < PER; ++i) {
                    const int e = lane + 32 * i;
                    if (e < experts && e / size == g && e != where) second = fmaxf(second, c[i]);
                }
                best += tt_warp_max(second);
            }
            if (lane == 0) group_best_row[g] = best;
        }
        __syncwarp();
        kept = 0u;
        for (int round = 0; round < keep; ++round) {
            float v = (lane < groups && !((kept >> lane) & 1u)) ? group_best_row[lane] : -INFINITY;
            int g = (lane < groups && !((kept >> lane) & 1u)) ? lane : 0x7fffffff;
            route_argmax(v, g);
            if (g < groups) kept |= 1u << g;
        }
    }
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int e = lane + 32 * i;
        if (e < experts) gates[(size_t)t * row + e] = 0.0f;
        if (e < experts && !((kept >> (e / size)) & 1u)) c[i] = -INFINITY;
    }
    __syncwarp();

    float sum = 0.0f;
    int mine = -1;                                              // lane r keeps the r-th choice (top <= 32)
    float mine_score = 0.0f;
    for (int round = 0; round < top; ++round) {
        float v = -INFINITY;
        int e = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < PER; ++i)
            if (c[i] > v) { v = c[i]; e = lane + 32 * i; }      // a lane's experts rise with i: the first largest is the lowest
        route_argmax(v, e);
        if (e == 0x7fffffff) break;                             // fewer allowed experts than top
        float score = 0.0f;
#pragma unroll
        for (int i = 0; i < PER; ++i)
            if (lane + 32 * i == e) { score = s[i]; c[i] = -INFINITY; }
        score = __shfl_sync(0xffffffffu, score, e & 31);
        sum += score;
        if (lane == round) { mine = e; mine_score = score; }
    }
    const float scale = opt.plain_weights ? 1.0f : 1.0f / (sum + 1e-20f);
    if (lane < top) {
        chosen[(size_t)t * top + lane] = mine;
        weights[(size_t)t * top + lane] = mine >= 0 ? mine_score * scale : 0.0f;
        if (mine >= 0) gates[(size_t)t * row + mine] = mine_score * scale;
    }
}

__global__ void route_topk_kernel(const float* __restrict__ logits, int splits, size_t split_stride, int n_tokens, int experts,
                                  int top, int groups, int keep, float* __restrict__ gates, int* __restrict__ chosen,
                                  float* __restrict__ weights, RouteOptions opt) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    __shared__ float group_best[ROUTE_WARPS][32];
    const int warp = threadIdx.x >> 5;
    const int t = blockIdx.x * ROUTE_WARPS + warp;
    if (t >= n_tokens) return;
    route_token(logits + (size_t)t * (experts + opt.extra), splits, split_stride, t, experts, top, groups, keep, gates, chosen, weights,
                group_best[warp], opt);
}

// The router's product and the routing in one kernel, one block per token: the token's row goes to shared memory as
// float32, every warp takes experts in turn (lanes across the row, float32 sums), and the first warp then routes the token
// from the logits in shared memory.
template <typename TX, typename TW>
__global__ void route_rows_kernel(const TX* __restrict__ x, const TW* __restrict__ w, int hidden, int n_tokens, int experts, int top,
                                  int groups, int keep, float* __restrict__ gates, int* __restrict__ chosen,
                                  float* __restrict__ weights, RouteOptions opt) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    extern __shared__ float route_shared[];                     // hidden, then experts + extra, then 32
    float* logits = route_shared + hidden;
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) route_shared[j] = tt_to_float(x[(size_t)t * hidden + j]);
    __syncthreads();
    for (int e = warp; e < experts + opt.extra; e += warps) {
        const TW* row = w + (size_t)e * hidden;
        float a[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        int j = lane;
        for (; j + 96 < hidden; j += 128) {                     // four loads in flight, four sums
            float v[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) v[i] = tt_to_float(row[j + 32 * i]);
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = fmaf(v[i], route_shared[j + 32 * i], a[i]);
        }
        for (; j < hidden; j += 32) a[0] = fmaf(tt_to_float(row[j]), route_shared[j], a[0]);
        const float z = tt_warp_sum((a[0] + a[1]) + (a[2] + a[3]));
        if (lane == 0) logits[e] = z;
    }
    __syncthreads();
    if (warp == 0) route_token(logits, 1, 0, t, experts, top, groups, keep, gates, chosen, weights, logits + experts + opt.extra, opt);
}

template <typename T>
__global__ void scale_expert_columns_kernel(T* __restrict__ act, int row_stride, int width, int experts,
                                            const float* __restrict__ gates, int gate_row, int shared_width, long long total) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int per_row = experts * width + shared_width;
    const long long t = i / per_row;
    const int c = (int)(i - t * per_row);
    const float g = gates[t * gate_row + (c < experts * width ? c / width : experts)];
    T* p = act + t * row_stride + c;
    *p = tt_from_float<T>(tt_to_float(*p) * g);
}

extern "C" int tt_route_topk(const float* logits, int splits, long long split_stride, int n_tokens, int experts, int top, int groups,
                             int keep, float* gates, int* chosen, float* weights, int sigmoid, const float* correction,
                             int group_top2, int plain_weights, int extra, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (experts <= 0 || experts > ROUTE_MAX_EXPERTS || top < 1 || top > 32 || top > experts || groups < 1 || groups > 32 ||
        experts % groups || keep < 1 || keep > groups || extra < 0 || extra > 32)
        return (int)cudaErrorInvalidValue;
    const RouteOptions opt{sigmoid, correction, group_top2, plain_weights, extra};
    tt_launch_pdl(route_topk_kernel, dim3((n_tokens + ROUTE_WARPS - 1) / ROUTE_WARPS), dim3(ROUTE_WARPS * 32), 0, stream, logits, splits,
                  (size_t)split_stride, n_tokens, experts, top, groups, keep, gates, chosen, weights, opt);
    TT_LAUNCH_CHECK();
}

// the same, 16 bytes a thread (width and row_stride are multiples of N numbers)
template <typename T, int N>
__global__ void scale_expert_columns_vec_kernel(T* __restrict__ act, int row_stride, int width, int experts,
                                                const float* __restrict__ gates, int gate_row, int shared_width, long long total) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * N;
    if (i >= total) return;
    const int per_row = experts * width + shared_width;
    const long long t = i / per_row;
    const int c = (int)(i - t * per_row);
    const float g = gates[t * gate_row + (c < experts * width ? c / width : experts)];
    uint4* p = reinterpret_cast<uint4*>(act + t * row_stride + c);
    uint4 raw = *p;
    T* v = reinterpret_cast<T*>(&raw);
#pragma unroll
    for (int e = 0; e < N; ++e) v[e] = tt_from_float<T>(tt_to_float(v[e]) * g);
    *p = raw;
}

extern "C" int tt_route_rows(const void* x, int x_dtype, const void* w, int w_dtype, int hidden, int n_tokens, int experts, int top,
                             int groups, int keep, float* gates, int* chosen, float* weights, int sigmoid, const float* correction,
                             int group_top2, int plain_weights, int extra, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (experts <= 0 || experts > ROUTE_MAX_EXPERTS || top < 1 || top > 32 || top > experts || groups < 1 || groups > 32 ||
        experts % groups || keep < 1 || keep > groups || extra < 0 || extra > 32)
        return (int)cudaErrorInvalidValue;
    const RouteOptions opt{sigmoid, correction, group_top2, plain_weights, extra};
    const size_t shared = (size_t)(hidden + experts + extra + 32) * sizeof(float);
    if (shared > 48 * 1024) return (int)cudaErrorInvalidValue;
#define TT_ROUTE(TX, TW) tt_launch_pdl(route_rows_kernel<TX, TW>, dim3(n_tokens), dim3(n_tokens <= 256 ? 512 : 128), shared, stream, (const TX*)x, (const TW*)w, hidden, n_tokens, experts, top, groups, keep, gates, chosen, weights, opt)
    if (x_dtype == TT_F32 && w_dtype == TT_F32) TT_ROUTE(float, float);
    else if (x_dtype == TT_F32) TT_ROUTE(float, __nv_bfloat16);
    else if (w_dtype == TT_F32) TT_ROUTE(__nv_bfloat16, float);
    else TT_ROUTE(__nv_bfloat16, __nv_bfloat16);
#undef TT_ROUTE
    TT_LAUNCH_CHECK();
}

extern "C" int tt_scale_expert_columns(void* act, int dtype, int n_tokens, int row_stride, int width, int experts, const float* gates,
                                       int gate_row, int shared_width, cudaStream_t stream) {
    const long long total = (long long)n_tokens * ((long long)experts * width + shared_width);
    if (total <= 0) return 0;
    const int threads = 256;
    const int n = dtype == TT_F32 ? 4 : 8;
    if (width % n == 0 && shared_width % n == 0 && row_stride % n == 0 && ((uintptr_t)act & 15) == 0) {
        const long long blocks = (total / n + threads - 1) / threads;
        if (blocks > 2147483647LL) return (int)cudaErrorInvalidValue;
        if (dtype == TT_F32)
            tt_launch_pdl(scale_expert_columns_vec_kernel<float, 4>, dim3((unsigned)blocks), dim3(threads), 0, stream, (float*)act, row_stride, width, experts, gates, gate_row, shared_width, total);
        else
            tt_launch_pdl(scale_expert_columns_vec_kernel<__nv_bfloat16, 8>, dim3((unsigned)blocks), dim3(threads), 0, stream, (__nv_bfloat16*)act, row_stride, width, experts, gates, gate_row, shared_width, total);
        TT_LAUNCH_CHECK();
    }
    const long long blocks = (total + threads - 1) / threads;
    if (blocks > 2147483647LL) return (int)cudaErrorInvalidValue;
    if (dtype == TT_F32)
        tt_launch_pdl(scale_expert_columns_kernel<float>, dim3((unsigned)blocks), dim3(threads), 0, stream, (float*)act, row_stride, width, experts, gates, gate_row, shared_width, total);
    else
        tt_launch_pdl(scale_expert_columns_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(threads), 0, stream, (__nv_bfloat16*)act, row_stride, width, experts, gates, gate_row, shared_width, total);
    TT_LAUNCH_CHECK();
}

// ------------------------------------------------------------------------------------
// The clamped gated unit of a mixture's experts, with the routing weights applied on the way.
// gate_up: float32 [splits][tokens][2 * cols], gate columns first; cols = experts * width + shared_width (the routed
// experts side by side, an always-on expert behind them).  With g' = min(g, limit) and u' = clamp(u, -limit, limit)
//   act[t][c] = g' * sigmoid(alpha * g') * (u' + 1) * gates[t][c / width]            (routed columns, limit)
//   act[t][c] = the same with shared_limit, times gates[t][experts] if shared_gated  (the always-on expert's columns)
// limit <= 0: no clamp.  Everything is float32 until the one narrowing at the end.
// ------------------------------------------------------------------------------------
template <typename TAct>
__global__ void expert_activation_kernel(const float* __restrict__ gate_up, int splits, size_t split_stride, TAct* __restrict__ act,
                                         int experts, int width, int shared_width, float limit, float shared_limit, float alpha,
                                         const float* __restrict__ gates, int gate_row, int shared_gated, long long total) {
    tt_pdl_launch_dependents();
    tt_pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int cols = experts * width + shared_width;
    const long long t = i / cols;
    const int c = (int)(i - t * cols);
    const bool routed = c < experts * width;
    const float weight = routed ? gates[t * gate_row + c / width] : (shared_gated ? gates[t * gate_row + experts] : 1.0f);
    if (weight == 0.0f) { act[i] = tt_from_float<TAct>(0.0f); return; }          // an expert the token did not choose
    const float* row = gate_up + (size_t)t * (2 * (size_t)cols) + c;
    float g = 0.0f, u = 0.0f;
#pragma unroll 4
    for (int s = 0; s < splits; ++s) {
        g += __ldg(row + s * split_stride);
        u += __ldg(row + s * split_stride + cols);
    }
    const float lim = routed ? limit : shared_limit;
    if (lim > 0.0f) { g = fminf(g, lim); u = fminf(fmaxf(u, -lim), lim); }
    act[i] = tt_from_float<TAct>(g / (1.0f + expf(-alpha * g)) * (u + 1.0f) * weight);
}

extern "C" int tt_expert_activation(const float* gate_up, int splits, long long split_stride, void* act, int act_dtype, int n_tokens,
                                    int experts, int width, int shared_width, float limit, float shared_limit, float alpha,
                                    const float* gates, int gate_row, int shared_gated, cudaStream_t stream) {
    const long long total = (long long)n_tokens * ((long long)experts * width + shared_width);
    if (total <= 0) return 0;
    const int threads = 256;
    const long long blocks = (total + threads - 1) / threads;
    if (blocks > 2147483647LL || experts < 0 || width < 0 || shared_width < 0 || (shared_gated && gate_row <= experts))
        return (int)cudaErrorInvalidValue;
    if (act_dtype == TT_F32)
        tt_launch_pdl(expert_activation_kernel<float>, dim3((unsigned)blocks), dim3(threads), 0, stream, gate_up, splits, (size_t)split_stride, (float*)act, experts, width, shared_width, limit, shared_limit, alpha, gates, gate_row, shared_gated, total);
    else
        tt_launch_pdl(expert_activation_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(threads), 0, stream, gate_up, splits, (size_t)split_stride, (__nv_bfloat16*)act, experts, width, shared_width, limit, shared_limit, alpha, gates, gate_row, shared_gated, total);
    TT_LAUNCH_CHECK();
}
