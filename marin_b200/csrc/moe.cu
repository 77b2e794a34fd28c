// A routed feed-forward (mixture of experts): a router scores every expert for every token, the `top` best are chosen,
// and the token goes through those experts only.  Expert: down( silu(gate x) * (up x) ), no biases.
//   * router: z = W_r h in float32, score = sigmoid(z) or the softmax of z over the experts; the chosen experts' scores are
//     the weights, renormalised to sum 1 over the chosen ones if asked;
//   * the weight multiplies the expert's input (x = w h, the activation sees it) or its output (x = h, result times w).
// Kernels: the router with its top-k (a warp per token), the grouping of (token, choice) pairs by expert (offsets and an
// order), and the plain expert products for any size in both dtypes (a pair per block).  A pair's result never depends on
// which other pairs the step holds or on the order they were grouped in; a token's pairs are added in choice order.
// Weights: gate|up as [experts][2 ff][h] (gate rows first), down as [experts][h][ff].
#define MB_LIB "moe"
#define MB_LIB_ID 14
#include "common.cuh"
#include "launch.cuh"

#define MR_WARPS 4

// ---- router and top-k: a warp per token -------------------------------------------------------------------------------
// expert_out int32 [tokens][top], weight_out float32 [tokens][top], choices in order of decreasing score (the lower expert
// among equals).  score_mode 0: sigmoid, 1: softmax over all experts.
template <typename T>
__global__ void __launch_bounds__(MR_WARPS * 32) moe_route_kernel(const T* __restrict__ h_rows, const float* __restrict__ router,
                                                                  int* __restrict__ expert_out, float* __restrict__ weight_out,
                                                                  int tokens, int h, int E, int top, int score_mode, int renorm) {
    PDL_ENTER();
    h_rows = pdl_fresh(h_rows);
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* z = smem + (size_t)warp * E;
    const int t = blockIdx.x * MR_WARPS + warp;
    if (t >= tokens) return;
    const T* x = h_rows + (size_t)t * h;
    for (int e = 0; e < E; ++e) {
        const float* w = router + (size_t)e * h;
        float dot = 0.0f;
        for (int i = lane; i < h; i += 32) dot = fmaf(to_f32(x[i]), w[i], dot);
        dot = warp_sum(dot);
        if (lane == 0) z[e] = dot;
    }
    __syncwarp();
    float denom = 1.0f, zmax = 0.0f;
    if (score_mode == 1) {
        float mx = -INFINITY;
        for (int e = lane; e < E; e += 32) mx = fmaxf(mx, z[e]);
        zmax = warp_max(mx);
        float sum = 0.0f;
        for (int e = lane; e < E; e += 32) sum += expf(z[e] - zmax);
        denom = warp_sum(sum);
    }
    float chosen_sum = 0.0f;
    for (int c = 0; c < top; ++c) {
        float best = -INFINITY;
        int at = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = z[e];
            if (v > best || (v == best && e < at)) { best = v; at = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
        }
        const float score = score_mode == 1 ? expf(best - zmax) / denom : 1.0f / (1.0f + expf(-best));
        chosen_sum += score;
        if (lane == 0) {
            expert_out[(size_t)t * top + c] = at;
            weight_out[(size_t)t * top + c] = score;
            z[at] = -INFINITY;
        }
        __syncwarp();
    }
    if (renorm && lane == 0)
        for (int c = 0; c < top; ++c) weight_out[(size_t)t * top + c] /= chosen_sum;
}

MB_API int mb_moe_route(const void* h_rows, int dtype, const float* router, int* expert_out, float* weight_out, int tokens, int h,
                        int E, int top, int score_mode, int renorm, cudaStream_t s) {
    if (tokens <= 0) return 0;
    if (E <= 0 || top <= 0 || top > E || h <= 0 || score_mode < 0 || score_mode > 1) return MB_ERR_BAD_SIZE;
    const size_t smem = (size_t)MR_WARPS * E * sizeof(float);
    if (smem > 48 * 1024) return MB_ERR_BAD_SIZE;
    const int blocks = (tokens + MR_WARPS - 1) / MR_WARPS;
    if (dtype == MB_F32)
        return launch_kernel(moe_route_kernel<float>, blocks, MR_WARPS * 32, smem, s, 0, (const float*)h_rows, router, expert_out,
                             weight_out, tokens, h, E, top, score_mode, renorm);
    if (dtype == MB_BF16)
        return launch_kernel(moe_route_kernel<bf16>, blocks, MR_WARPS * 32, smem, s, 0, (const bf16*)h_rows, router, expert_out,
                             weight_out, tokens, h, E, top, score_mode, renorm);
    return MB_ERR_BAD_DTYPE;
}

// ---- pairs grouped by expert: offsets[E + 1] and order[pairs] (the pairs of expert e are order[offsets[e] .. offsets[e+1])) ----
// One block.  Within an expert the pairs come in no fixed order: no result depends on it.
__global__ void __launch_bounds__(1024) moe_group_kernel(const int* __restrict__ expert_of, int pairs, int E, int* __restrict__ offsets,
                                                         int* __restrict__ order) {
    PDL_ENTER();
    expert_of = pdl_fresh(expert_of);
    extern __shared__ int counts[];            // [E] counts, then [E] cursors
    int* cursor = counts + E;
    for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) atomicAdd(&counts[expert_of[p]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < E; ++e) { offsets[e] = run; cursor[e] = run; run += counts[e]; }
        offsets[E] = run;
    }
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) order[atomicAdd(&cursor[expert_of[p]], 1)] = p;
}

MB_API int mb_moe_group(const int* expert_of, int pairs, int E, int* offsets, int* order, cudaStream_t s) {
    if (pairs <= 0) return 0;
    if (E <= 0 || (size_t)E * 8 > 48 * 1024) return MB_ERR_BAD_SIZE;
    return launch_kernel(moe_group_kernel, 1, 1024, (size_t)E * 8, s, 0, expert_of, pairs, E, offsets, order);
}

// ---- plain expert products ---------------------------------------------------------------------------------------------
#define ME_THREADS 256

// act[p][c] = silu(gate_c . x) * (up_c . x) for pair p = token * top + choice, x = h[token] (times the pair's weight where the
// weight goes on the input), rounded to the activation dtype as the tensor-core path's operand would be.
template <typename T>
__global__ void __launch_bounds__(ME_THREADS) moe_gate_up_kernel(const T* __restrict__ h_rows, const T* __restrict__ w_gate_up,
                                                                 const int* __restrict__ expert_of, const float* __restrict__ weight_of,
                                                                 T* __restrict__ act, int h, int ff, int top, int weight_on_input) {
    PDL_ENTER();
    h_rows = pdl_fresh(h_rows); expert_of = pdl_fresh(expert_of); weight_of = pdl_fresh(weight_of);
    extern __shared__ float x[];               // [h]
    const int p = blockIdx.x;
    const int token = p / top;
    const int e = expert_of[p];
    const float wgt = weight_on_input ? weight_of[p] : 1.0f;
    for (int i = threadIdx.x; i < h; i += ME_THREADS) x[i] = to_f32(from_f32<T>(to_f32(h_rows[(size_t)token * h + i]) * wgt));
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const T* base = w_gate_up + (size_t)e * 2 * ff * h;
    for (int c = warp; c < ff; c += ME_THREADS / 32) {
        const T* g = base + (size_t)c * h;
        const T* u = base + (size_t)(ff + c) * h;
        float dg = 0.0f, du = 0.0f;
        for (int i = lane; i < h; i += 32) { dg = fmaf(x[i], to_f32(g[i]), dg); du = fmaf(x[i], to_f32(u[i]), du); }
        dg = warp_sum(dg);
        du = warp_sum(du);
        if (lane == 0) act[(size_t)p * ff + c] = from_f32<T>(dg / (1.0f + expf(-dg)) * du);
    }
}

// y[token][c] += sum over the token's choices, in choice order, of (down_c . act[pair]) (times the pair's weight where the
// weight goes on the output).  A token per block.
template <typename T>
__global__ void __launch_bounds__(ME_THREADS) moe_down_kernel(const T* __restrict__ act, const T* __restrict__ w_down,
                                                              const int* __restrict__ expert_of, const float* __restrict__ weight_of,
                                                              float* __restrict__ y, int h, int ff, int top, int weight_on_input) {
    PDL_ENTER();
    act = pdl_fresh(act); expert_of = pdl_fresh(expert_of); weight_of = pdl_fresh(weight_of); y = pdl_fresh(y);
    extern __shared__ float a[];               // [ff]
    const int token = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int c = 0; c < top; ++c) {
        const int p = token * top + c;
        const int e = expert_of[p];
        const float wgt = weight_on_input ? 1.0f : weight_of[p];
        __syncthreads();
        for (int i = threadIdx.x; i < ff; i += ME_THREADS) a[i] = to_f32(act[(size_t)p * ff + i]);
        __syncthreads();
        const T* base = w_down + (size_t)e * h * ff;
        for (int col = warp; col < h; col += ME_THREADS / 32) {
            const T* w = base + (size_t)col * ff;
            float dot = 0.0f;
            for (int i = lane; i < ff; i += 32) dot = fmaf(a[i], to_f32(w[i]), dot);
            dot = warp_sum(dot);
            if (lane == 0) y[(size_t)token * h + col] += dot * wgt;
        }
    }
}

MB_API int mb_moe_experts_plain(const void* h_rows, int dtype, const void* w_gate_up, const void* w_down, const int* expert_of,
                                const float* weight_of, void* act, float* y, int tokens, int h, int ff, int top, int weight_on_input,
                                cudaStream_t s) {
    if (tokens <= 0) return 0;
    if (h <= 0 || ff <= 0 || top <= 0 || (size_t)h * 4 > 48 * 1024 || (size_t)ff * 4 > 48 * 1024) return MB_ERR_BAD_SIZE;
    int rc;
    if (dtype == MB_F32) {
        rc = launch_kernel(moe_gate_up_kernel<float>, tokens * top, ME_THREADS, (size_t)h * 4, s, 0, (const float*)h_rows,
                           (const float*)w_gate_up, expert_of, weight_of, (float*)act, h, ff, top, weight_on_input);
        if (rc != 0) return rc;
        return launch_kernel(moe_down_kernel<float>, tokens, ME_THREADS, (size_t)ff * 4, s, 0, (const float*)act, (const float*)w_down,
                             expert_of, weight_of, y, h, ff, top, weight_on_input);
    }
    if (dtype == MB_BF16) {
        rc = launch_kernel(moe_gate_up_kernel<bf16>, tokens * top, ME_THREADS, (size_t)h * 4, s, 0, (const bf16*)h_rows,
                           (const bf16*)w_gate_up, expert_of, weight_of, (bf16*)act, h, ff, top, weight_on_input);
        if (rc != 0) return rc;
        return launch_kernel(moe_down_kernel<bf16>, tokens, ME_THREADS, (size_t)ff * 4, s, 0, (const bf16*)act, (const bf16*)w_down,
                             expert_of, weight_of, y, h, ff, top, weight_on_input);
    }
    return MB_ERR_BAD_DTYPE;
}
