// Causal grouped-query softmax attention over the paged cache with the options several designs combine:
//   * keys of `d` elements, values of `dv` (they may differ): K pages [page][kv_head][offset][d], V pages [..][dv];
//   * which keys a position sees: all before it, the last `window`, or those of its own chunk of `chunk` positions
//     (chunks counted from position 0 of the sequence, wherever a prompt was cut);
//   * a sink: one more term in the softmax's denominator, a key of score 0 without a value,
//         p_j = exp(s_j) / (1 + sum_j exp(s_j));
//   * an output gate: the result is multiplied element by element with sigmoid(g), g a column block of the fused
//     projection.
// This file holds the head preparation (biases, RMS norm of q and k per head or over the whole projection, partial
// rotation with scaled sines and cosines, value mixing with the values an earlier layer left for the same tokens, cache
// write) and the plain attention kernel that serves any size in both dtypes.  Sums, norms, angles, scores and weights
// are float32.
#define MB_LIB "attention_sink"
#define MB_LIB_ID 13
#include "common.cuh"
#include "launch.cuh"

#define QF_THREADS 256            // at least; 1024 where a token's q and k have 4,096 elements and more

// ---- heads of the fused q|k|v(|g) projection, a token per block ---------------------------------------------------------
// A row of `row` holds q (H heads of d), k (K heads of d), v (K heads of dv), then whatever follows (the gate's columns).
// norm_mode 0: none; 1: per head over d, weight [d] shared by the heads; 2: over all of q (and all of k) at once, before
// the split into heads, weight [H d] (and [K d]).  The first rot_dim elements of a head are rotated in pairs
// (i, i + rot_dim/2) by the angle pos * inv_freq[i]; sines and cosines are multiplied by rot_mag.
// v_mode 0: values as they are; 1: they are also left in v_shared (activation dtype [tokens][K dv]) for later layers;
// 2: v <- (1 - lam) v + lam v_shared, lam = *v_lambda, and the mixed values go to the cache.
template <typename T>
__global__ void __launch_bounds__(1024) qkv_finish_kernel(
    const T* __restrict__ row, int row_stride, T* __restrict__ q_out, const float* __restrict__ q_b, const float* __restrict__ k_b,
    const float* __restrict__ v_b, int norm_mode, const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
    const int* __restrict__ positions, const float* __restrict__ inv_freq, int rot_dim, float rot_mag,
    const int* __restrict__ slot_mapping, T* __restrict__ k_cache, T* __restrict__ v_cache, int v_mode, T* __restrict__ v_shared,
    const float* __restrict__ v_lambda, int H, int K, int d, int dv, int page_size, int write_kv) {
    PDL_ENTER();
    row = pdl_fresh(row); v_shared = pdl_fresh(v_shared);
    extern __shared__ float smem[];
    const int heads = write_kv ? H + K : H;
    const int half = rot_dim >> 1;
    float* vals = smem;                        // [heads * d]: q then k, float32
    float* cs_tab = vals + (size_t)heads * d;  // [half] cosines, [half] sines
    float* head_ss = cs_tab + 2 * half;        // [heads]
    __shared__ float s_factor[2];
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x / 32, threads = blockDim.x;
    const T* src = row + (size_t)t * row_stride;
    if (inv_freq != nullptr) {
        const float pos = (float)positions[t];
        for (int i = threadIdx.x; i < half; i += threads) {
            float sn, cs;
            sincosf(pos * inv_freq[i], &sn, &cs);
            cs_tab[i] = cs * rot_mag;
            cs_tab[half + i] = sn * rot_mag;
        }
    }
    // every element of q and k (+ bias) into shared memory as float32, all threads side by side
    const int qk = heads * d, q_len = H * d;
    for (int idx = threadIdx.x; idx < qk; idx += threads) {
        float v = to_f32(src[idx]);
        if (idx < q_len) { if (q_b != nullptr) v += q_b[idx]; }
        else if (k_b != nullptr) v += k_b[idx - q_len];
        vals[idx] = v;
    }
    __syncthreads();
    // sums of squares per head: a warp per head, lanes in a fixed order
    for (int head = warp; head < heads; head += warps) {
        float ss = 0.0f;
        for (int i = lane; i < d; i += 32) { const float v = vals[head * d + i]; ss += v * v; }
        ss = warp_sum(ss);
        if (lane == 0) head_ss[head] = ss;
    }
    __syncthreads();
    if (norm_mode == 2 && threadIdx.x < 2) {
        const int first = threadIdx.x == 0 ? 0 : H, count = threadIdx.x == 0 ? H : heads - H;
        float total = 0.0f;
        for (int j = 0; j < count; ++j) total += head_ss[first + j];
        s_factor[threadIdx.x] = count > 0 ? 1.0f / sqrtf(total / (float)(count * d) + eps) : 0.0f;
    }
    __syncthreads();
    const int slot = write_kv ? slot_mapping[t] : -1;
    T* k_dst = slot >= 0 ? k_cache + (((size_t)(slot / page_size)) * K * page_size + (size_t)(slot % page_size)) * d : nullptr;
    for (int idx = threadIdx.x; idx < qk; idx += threads) {
        const int head = idx / d, i = idx - head * d;
        const bool is_q = head < H;
        const int kh = head - H;
        if (!is_q && k_dst == nullptr) continue;
        float factor = 1.0f;
        const float* w = nullptr;
        if (norm_mode == 1) {
            factor = 1.0f / sqrtf(head_ss[head] / (float)d + eps);
            w = is_q ? q_w : k_w;
        } else if (norm_mode == 2) {
            factor = s_factor[is_q ? 0 : 1];
            w = is_q ? q_w + (size_t)head * d : k_w + (size_t)kh * d;
        }
        float a = vals[idx] * factor * (w != nullptr ? w[i] : 1.0f);
        if (inv_freq != nullptr && i < rot_dim) {
            const bool low = i < half;
            const int j = low ? i : i - half, other = low ? i + half : i - half;
            const float b = vals[head * d + other] * factor * (w != nullptr ? w[other] : 1.0f);
            const float cs = cs_tab[j], sn = cs_tab[half + j];
            a = low ? a * cs - b * sn : a * cs + b * sn;
        }
        if (is_q) q_out[(size_t)t * q_len + idx] = from_f32<T>(a);
        else k_dst[(size_t)kh * page_size * d + i] = from_f32<T>(a);
    }
    if (!write_kv) return;
    const float lam = v_mode == 2 ? *v_lambda : 0.0f;
    const int vcol0 = (H + K) * d;
    for (int i = threadIdx.x; i < K * dv; i += threads) {
        float v = to_f32(src[vcol0 + i]);
        if (v_b != nullptr) v += v_b[i];
        if (v_mode == 1) v_shared[(size_t)t * K * dv + i] = from_f32<T>(v);
        else if (v_mode == 2) v = (1.0f - lam) * v + lam * to_f32(v_shared[(size_t)t * K * dv + i]);
        if (slot >= 0) {
            const int kh = i / dv, e = i % dv;
            v_cache[((((size_t)(slot / page_size)) * K + kh) * page_size + (size_t)(slot % page_size)) * dv + e] = from_f32<T>(v);
        }
    }
}

MB_API int mb_qkv_finish(const void* row, int row_stride, int dtype, void* q_out, const float* q_b, const float* k_b, const float* v_b,
                         int norm_mode, const float* q_w, const float* k_w, float eps, const int* positions, const float* inv_freq,
                         int rot_dim, float rot_mag, const int* slot_mapping, void* k_cache, void* v_cache, int v_mode, void* v_shared,
                         const float* v_lambda, int tokens, int H, int K, int d, int dv, int page_size, int write_kv, cudaStream_t s) {
    if (tokens <= 0) return 0;
    if (d <= 0 || dv <= 0 || H <= 0 || K <= 0 || rot_dim > d || (rot_dim & 1) || norm_mode < 0 || norm_mode > 2) return MB_ERR_BAD_SIZE;
    if ((v_mode == 1 || v_mode == 2) && v_shared == nullptr) return MB_ERR_BAD_SIZE;
    if (v_mode == 2 && v_lambda == nullptr) return MB_ERR_BAD_SIZE;
    if (inv_freq == nullptr) rot_dim = 0;
    const size_t smem = ((size_t)(H + K) * d + rot_dim + H + K) * sizeof(float);
    if (smem > 160 * 1024) return MB_ERR_BAD_SIZE;
#define QF_LAUNCH(TT)                                                                                                                \
    do {                                                                                                                             \
        if (smem > 48 * 1024) {                                                                                                      \
            const int rc = (int)cudaFuncSetAttribute(qkv_finish_kernel<TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (rc != 0) return rc;                                                                                                  \
        }                                                                                                                            \
        return launch_kernel(qkv_finish_kernel<TT>, tokens, (H + K) * d < 4096 ? QF_THREADS : tokens <= 64 ? 1024 : 512, smem, s, 0, (const TT*)row, row_stride, (TT*)q_out, q_b, k_b, \
                             v_b, norm_mode, q_w, k_w, eps, positions, inv_freq, rot_dim, rot_mag, slot_mapping, (TT*)k_cache,      \
                             (TT*)v_cache, v_mode, (TT*)v_shared, v_lambda, H, K, d, dv, page_size, write_kv);                       \
    } while (0)
    if (dtype == MB_F32) QF_LAUNCH(float);
    if (dtype == MB_BF16) QF_LAUNCH(bf16);
#undef QF_LAUNCH
    return MB_ERR_BAD_DTYPE;
}

// ---- the plain kernel: one block per (token, query head), keys in blocks of 128 in increasing order ----------------------
#define SK_THREADS 128
#define SK_MAX_PER_THREAD 4

template <typename T>
__global__ void __launch_bounds__(SK_THREADS) attention_sink_kernel(
    const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache, T* __restrict__ out,
    const int* __restrict__ block_table, int max_pages, const int* __restrict__ req_index, const int* __restrict__ positions,
    int H, int K, int d, int dv, int page_size, float scale, int window, int chunk, int sink, const T* __restrict__ gate,
    int gate_stride) {
    PDL_ENTER();
    q = pdl_fresh(q); k_cache = pdl_fresh(k_cache); v_cache = pdl_fresh(v_cache); gate = pdl_fresh(gate);
    extern __shared__ float smem[];
    float* qs = smem;                 // [d]
    float* ps = smem + d;             // [SK_THREADS]
    float* scratch = ps + SK_THREADS; // [32]
    const int t = blockIdx.x, head = blockIdx.y;
    const int kh = head / (H / K);
    const int req = req_index[t];
    const int pos = positions[t];
    int lo = window > 0 ? max(0, pos - window + 1) : 0;
    if (chunk > 0) lo = max(lo, (pos / chunk) * chunk);
    const int* table = block_table + (size_t)req * max_pages;
    const T* qrow = q + ((size_t)t * H + head) * d;
    for (int i = threadIdx.x; i < d; i += SK_THREADS) qs[i] = to_f32(qrow[i]);
    __syncthreads();

    // the sink is a key of score 0 whose value is zero: the running maximum starts at 0 and the sum at 1
    float m = sink ? 0.0f : -INFINITY, l = sink ? 1.0f : 0.0f;
    float acc[SK_MAX_PER_THREAD];
#pragma unroll
    for (int r = 0; r < SK_MAX_PER_THREAD; ++r) acc[r] = 0.0f;

    for (int base = lo; base <= pos; base += SK_THREADS) {
        const int key = base + threadIdx.x;
        float s = -INFINITY;
        if (key <= pos) {
            const size_t page = (size_t)table[key / page_size];
            const T* krow = k_cache + ((page * K + kh) * page_size + (size_t)(key % page_size)) * d;
            float dot = 0.0f;
            for (int i = 0; i < d; ++i) dot = fmaf(qs[i], to_f32(krow[i]), dot);
            s = dot * scale;
        }
        const float block_top = block_max(s, scratch);
        const float m_new = fmaxf(m, block_top);
        const float corr = expf(m - m_new);   // exp(-inf) = 0 on the first block without a sink
        const float p = key <= pos ? expf(s - m_new) : 0.0f;
        __syncthreads();
        ps[threadIdx.x] = p;
        const float block_total = block_sum(p, scratch);  // has the barriers that publish ps
        l = l * corr + block_total;
        m = m_new;
        const int count = min(SK_THREADS, pos - base + 1);
#pragma unroll
        for (int r = 0; r < SK_MAX_PER_THREAD; ++r) {
            const int dd = threadIdx.x + r * SK_THREADS;
            if (dd < dv) {
                float a = acc[r] * corr;
                for (int j = 0; j < count; ++j) {
                    const int kj = base + j;
                    const size_t page = (size_t)table[kj / page_size];
                    const T* vrow = v_cache + ((page * K + kh) * page_size + (size_t)(kj % page_size)) * dv;
                    a = fmaf(ps[j], to_f32(vrow[dd]), a);
                }
                acc[r] = a;
            }
        }
        __syncthreads();
    }
    T* orow = out + ((size_t)t * H + head) * dv;
    const T* grow = gate != nullptr ? gate + (size_t)t * gate_stride + (size_t)head * dv : nullptr;
#pragma unroll
    for (int r = 0; r < SK_MAX_PER_THREAD; ++r) {
        const int dd = threadIdx.x + r * SK_THREADS;
        if (dd < dv) {
            float o = acc[r] / l;
            if (grow != nullptr) o *= 1.0f / (1.0f + expf(-to_f32(grow[dd])));
            orow[dd] = from_f32<T>(o);
        }
    }
}

// gate: null, or the first gate column of token 0 (rows `gate_stride` elements apart, H heads of dv side by side).
MB_API int mb_attention_sink(const void* q, const void* k_cache, const void* v_cache, void* out, int dtype, const int* block_table,
                             int max_pages, const int* req_index, const int* positions, int tokens, int H, int K, int d, int dv,
                             int page_size, float scale, int window, int chunk, int sink, const void* gate, int gate_stride,
                             cudaStream_t s) {
    if (tokens <= 0) return 0;
    if (d <= 0 || dv <= 0 || dv > SK_THREADS * SK_MAX_PER_THREAD || K <= 0 || H % K != 0 || window < 0 || chunk < 0) return MB_ERR_BAD_SIZE;
    dim3 grid(tokens, H);
    const size_t smem = (size_t)(d + SK_THREADS + 32) * sizeof(float);
    if (smem > 48 * 1024) return MB_ERR_BAD_SIZE;
    if (dtype == MB_F32)
        return launch_kernel(attention_sink_kernel<float>, grid, SK_THREADS, smem, s, 0, (const float*)q, (const float*)k_cache,
                             (const float*)v_cache, (float*)out, block_table, max_pages, req_index, positions, H, K, d, dv, page_size,
                             scale, window, chunk, sink, (const float*)gate, gate_stride);
    if (dtype == MB_BF16)
        return launch_kernel(attention_sink_kernel<bf16>, grid, SK_THREADS, smem, s, 0, (const bf16*)q, (const bf16*)k_cache,
                             (const bf16*)v_cache, (bf16*)out, block_table, max_pages, req_index, positions, H, K, d, dv, page_size,
                             scale, window, chunk, sink, (const bf16*)gate, gate_stride);
    return MB_ERR_BAD_DTYPE;
}
