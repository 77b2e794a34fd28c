// Causal grouped-query attention whose weights are sigmoids instead of a softmax, over the paged cache:
//   weight(i, j) = sigmoid(q_i . k_j * scale + bias[head][min(i - j, span - 1)]),   out_i = sum_{j <= i} weight(i, j) v_j
// The weights are not normalised over the keys, so partial sums over any split of the keys simply add.  `bias` is a
// table per head over the distance i - j (whatever is added to a score as a function of head and distance: a bucketed
// distance table, a constant per head), float32 [heads][span]; distances beyond the table take its last entry.
// Keys have `d` elements, values `dv` (they may differ): K pages [page][kv_head][offset][d], V pages [..][dv].
// This file holds the head preparation (per-head RMS norm of q and k, a factor on q that depends on the position, keys
// and values into their pages) and the plain kernel that serves any size in both dtypes.
#define MB_LIB "attention_sigmoid"
#define MB_LIB_ID 10
#include "common.cuh"
#include "launch.cuh"

// ---- heads of the fused q|k|v projection: norm, query factor, cache write -----------------------------------------------
// One warp per (token, head).  Heads 0..H-1 are queries (d each), then K key heads (d), then K value heads (dv).
// q and k: RMS norm over d with q_w / k_w (null: no norm).  Queries are multiplied by
// 1 + temp_coef * ln(floor((p + 1) / temp_every) + 1) at position p (temp_coef 0: no factor).
template <typename T>
__global__ void qkv_heads_sigmoid_kernel(const T* __restrict__ qkv, int row_stride, T* __restrict__ q_out,
                                         const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
                                         const int* __restrict__ positions, float temp_coef, int temp_every,
                                         const int* __restrict__ slot_mapping, T* __restrict__ k_cache, T* __restrict__ v_cache,
                                         int H, int K, int d, int dv, int page_size, int heads_total) {
    PDL_ENTER();
    qkv = pdl_fresh(qkv);
    extern __shared__ float smem[];
    const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int widest = d > dv ? d : dv;
    float* buf = smem + (size_t)warp * widest;
    const int t = blockIdx.x;
    const int head = blockIdx.y * warps + warp;
    if (head >= heads_total) return;
    const bool is_q = head < H, is_k = !is_q && head < H + K;
    const int n = (is_q || is_k) ? d : dv;
    const size_t col = is_q ? (size_t)head * d : is_k ? (size_t)H * d + (size_t)(head - H) * d
                                                      : (size_t)(H + K) * d + (size_t)(head - H - K) * dv;
    const T* src = qkv + (size_t)t * row_stride + col;
    float ss = 0.0f;
    for (int i = lane; i < n; i += 32) { const float v = to_f32(src[i]); buf[i] = v; ss += v * v; }
    const float* w = is_q ? q_w : (is_k ? k_w : nullptr);
    float factor = 1.0f;
    if (w != nullptr) {
        ss = warp_sum(ss);
        factor = 1.0f / sqrtf(ss / (float)n + eps);
    }
    if (is_q && temp_coef != 0.0f) factor *= 1.0f + temp_coef * logf((float)((positions[t] + 1) / temp_every + 1));
    T* dst = nullptr;
    if (is_q) {
        dst = q_out + ((size_t)t * H + head) * d;
    } else {
        const int slot = slot_mapping[t];
        if (slot >= 0) {
            const int kh = is_k ? head - H : head - H - K;
            const size_t page = (size_t)(slot / page_size), off = (size_t)(slot % page_size);
            dst = (is_k ? k_cache : v_cache) + ((page * K + kh) * page_size + off) * n;
        }
    }
    if (dst != nullptr)
        for (int i = lane; i < n; i += 32) dst[i] = from_f32<T>(w != nullptr ? buf[i] * factor * w[i] : buf[i] * factor);
}

MB_API int mb_qkv_heads_sigmoid(const void* qkv, int dtype, void* q_out, const float* q_w, const float* k_w, float eps,
                                const int* positions, float temp_coef, int temp_every, const int* slot_mapping, void* k_cache,
                                void* v_cache, int tokens, int H, int K, int d, int dv, int page_size, int write_kv, cudaStream_t s) {
    if (tokens <= 0) return 0;
    if (d <= 0 || dv <= 0 || temp_every <= 0) return MB_ERR_BAD_SIZE;
    const int heads_total = write_kv ? H + 2 * K : H;
    const int row_stride = write_kv ? (H + K) * d + K * dv : H * d;
    const int warps = 4;
    dim3 grid(tokens, (heads_total + warps - 1) / warps);
    const size_t smem = (size_t)warps * (d > dv ? d : dv) * sizeof(float);
    if (smem > 48 * 1024) return MB_ERR_BAD_SIZE;
    if (dtype == MB_F32)
        return launch_kernel(qkv_heads_sigmoid_kernel<float>, grid, warps * 32, smem, s, 0, (const float*)qkv, row_stride, (float*)q_out,
                             q_w, k_w, eps, positions, temp_coef, temp_every, slot_mapping, (float*)k_cache, (float*)v_cache, H, K, d, dv,
                             page_size, heads_total);
    if (dtype == MB_BF16)
        return launch_kernel(qkv_heads_sigmoid_kernel<bf16>, grid, warps * 32, smem, s, 0, (const bf16*)qkv, row_stride, (bf16*)q_out,
                             q_w, k_w, eps, positions, temp_coef, temp_every, slot_mapping, (bf16*)k_cache, (bf16*)v_cache, H, K, d, dv,
                             page_size, heads_total);
    return MB_ERR_BAD_DTYPE;
}

// ---- the plain kernel: one block per (token, query head), keys in chunks of 128 in increasing order ------------------------
#define SG_THREADS 128
#define SG_MAX_PER_THREAD 4

template <typename T>
__global__ void __launch_bounds__(SG_THREADS) attention_sigmoid_kernel(
    const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache, T* __restrict__ out,
    const int* __restrict__ block_table, int max_pages, const int* __restrict__ req_index, const int* __restrict__ positions,
    const float* __restrict__ bias, int span, int H, int K, int d, int dv, int page_size, float scale) {
    PDL_ENTER();
    q = pdl_fresh(q); k_cache = pdl_fresh(k_cache); v_cache = pdl_fresh(v_cache);
    extern __shared__ float smem[];
    float* qs = smem;            // [d]
    float* ps = smem + d;        // [SG_THREADS]
    const int t = blockIdx.x, head = blockIdx.y;
    const int kh = head / (H / K);
    const int req = req_index[t];
    const int pos = positions[t];
    const int* table = block_table + (size_t)req * max_pages;
    const float* brow = bias + (size_t)head * span;
    const T* qrow = q + ((size_t)t * H + head) * d;
    for (int i = threadIdx.x; i < d; i += SG_THREADS) qs[i] = to_f32(qrow[i]);
    __syncthreads();
    float acc[SG_MAX_PER_THREAD];
#pragma unroll
    for (int r = 0; r < SG_MAX_PER_THREAD; ++r) acc[r] = 0.0f;
    for (int base = 0; base <= pos; base += SG_THREADS) {
        const int key = base + threadIdx.x;
        float p = 0.0f;
        if (key <= pos) {
            const size_t page = (size_t)table[key / page_size];
            const T* krow = k_cache + ((page * K + kh) * page_size + (size_t)(key % page_size)) * d;
            float dot = 0.0f;
            for (int i = 0; i < d; ++i) dot = fmaf(qs[i], to_f32(krow[i]), dot);
            const int dist = pos - key;
            const float s = fmaf(dot, scale, brow[dist < span ? dist : span - 1]);
            p = 1.0f / (1.0f + expf(-s));
        }
        __syncthreads();           // the chunk before is summed
        ps[threadIdx.x] = p;
        __syncthreads();
        const int count = min(SG_THREADS, pos - base + 1);
#pragma unroll
        for (int r = 0; r < SG_MAX_PER_THREAD; ++r) {
            const int dd = threadIdx.x + r * SG_THREADS;
            if (dd < dv) {
                float a = acc[r];
                for (int j = 0; j < count; ++j) {
                    const int kj = base + j;
                    const size_t page = (size_t)table[kj / page_size];
                    const T* vrow = v_cache + ((page * K + kh) * page_size + (size_t)(kj % page_size)) * dv;
                    a = fmaf(ps[j], to_f32(vrow[dd]), a);
                }
                acc[r] = a;
            }
        }
    }
    T* orow = out + ((size_t)t * H + head) * dv;
#pragma unroll
    for (int r = 0; r < SG_MAX_PER_THREAD; ++r) {
        const int dd = threadIdx.x + r * SG_THREADS;
        if (dd < dv) orow[dd] = from_f32<T>(acc[r]);
    }
}

MB_API int mb_attention_sigmoid(const void* q, const void* k_cache, const void* v_cache, void* out, int dtype, const int* block_table,
                                int max_pages, const int* req_index, const int* positions, const float* bias, int span, int tokens,
                                int H, int K, int d, int dv, int page_size, float scale, cudaStream_t s) {
    if (tokens <= 0) return 0;
    if (d <= 0 || dv <= 0 || dv > SG_THREADS * SG_MAX_PER_THREAD || K <= 0 || H % K != 0 || span <= 0) return MB_ERR_BAD_SIZE;
    dim3 grid(tokens, H);
    const size_t smem = (size_t)(d + SG_THREADS) * sizeof(float);
    if (smem > 48 * 1024) return MB_ERR_BAD_SIZE;
    if (dtype == MB_F32)
        return launch_kernel(attention_sigmoid_kernel<float>, grid, SG_THREADS, smem, s, 0, (const float*)q, (const float*)k_cache,
                             (const float*)v_cache, (float*)out, block_table, max_pages, req_index, positions, bias, span, H, K, d, dv,
                             page_size, scale);
    if (dtype == MB_BF16)
        return launch_kernel(attention_sigmoid_kernel<bf16>, grid, SG_THREADS, smem, s, 0, (const bf16*)q, (const bf16*)k_cache,
                             (const bf16*)v_cache, (bf16*)out, block_table, max_pages, req_index, positions, bias, span, H, K, d, dv,
                             page_size, scale);
    return MB_ERR_BAD_DTYPE;
}
