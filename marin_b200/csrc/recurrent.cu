// Recurrences over a request's tokens with a matrix-valued state per head, kept in float32 in a state slot per request:
//   * linear attention with a fixed decay per head:   S_t = decay_h S_(t-1) + k_t v_t^T,            o_t = S_t^T q_t
//   * time mixing with a decay per token and channel: o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t,   S_t = diag(w_t) S_(t-1) + k_t v_t^T
// One block walks the tokens a request brings to the step in order (a prompt portion or a single decoded token alike),
// starting from the state the steps before left and leaving the new one; the step's requests and the heads are the grid.
// Which tokens belong to a request, and its slot, are read from device arrays, so a captured graph replays the same
// launch for other requests.  A thread owns one column of the state (all key channels of one value channel), so the
// sums over key channels run in a fixed order inside one thread: a result does not depend on how the tokens were cut
// into steps or on what else the batch holds.
#define MB_LIB "recurrent"
#define MB_LIB_ID 9
#include "common.cuh"
#include "launch.cuh"

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }

// ---- linear attention with a fixed decay per head ---------------------------------------------------------------------
// q, k: [T, heads * dim], v: [T, heads * vdim] with a common row stride (slices of one projection), before their
// activation: silu is applied here.  o: float32 [T, heads * vdim].  state: [slot][head][dim][vdim].
// grid (requests, heads, ceil(vdim / blockDim.x)); shared memory: the block's columns of the state and two buffers of q|k.
template <typename T>
__global__ void linear_attention_scan_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, int row_stride,
                                             const float* __restrict__ decay, float* __restrict__ state,
                                             const int* __restrict__ cu_tokens, const int* __restrict__ state_slots,
                                             float* __restrict__ o, int heads, int dim, int vdim) {
    PDL_ENTER();
    q = pdl_fresh(q); k = pdl_fresh(k); v = pdl_fresh(v);
    extern __shared__ float smem[];
    const int cols = blockDim.x;
    float* S = smem;                       // [dim][cols]
    float* qk = smem + (size_t)dim * cols; // [2][2 * dim]
    const int r = blockIdx.x, head = blockIdx.y;
    const int j = blockIdx.z * cols + threadIdx.x;
    const bool live = j < vdim;
    const int first = cu_tokens[r], count = cu_tokens[r + 1] - first;
    if (count <= 0) return;
    float* st = state + (((size_t)state_slots[r] * heads + head) * dim) * vdim;
    if (live)
        for (int i = 0; i < dim; ++i) S[i * cols + threadIdx.x] = st[(size_t)i * vdim + j];
    const float lam = decay[head];
    for (int n = 0; n < count; ++n) {
        const size_t t = (size_t)(first + n);
        float* buf = qk + (n & 1) * 2 * dim;
        for (int i = threadIdx.x; i < dim; i += cols) {
            buf[i] = silu_f(to_f32(q[t * row_stride + (size_t)head * dim + i]));
            buf[dim + i] = silu_f(to_f32(k[t * row_stride + (size_t)head * dim + i]));
        }
        const float vj = live ? silu_f(to_f32(v[t * row_stride + (size_t)head * vdim + j])) : 0.0f;
        __syncthreads();
        if (live) {
            float acc = 0.0f;
            for (int i = 0; i < dim; ++i) {
                const float s = fmaf(lam, S[i * cols + threadIdx.x], buf[dim + i] * vj);
                S[i * cols + threadIdx.x] = s;
                acc = fmaf(s, buf[i], acc);
            }
            o[t * ((size_t)heads * vdim) + (size_t)head * vdim + j] = acc;
        }
    }
    if (live)
        for (int i = 0; i < dim; ++i) st[(size_t)i * vdim + j] = S[i * cols + threadIdx.x];
}

MB_API int mb_linear_attention_scan(const void* q, const void* k, const void* v, int dtype, int row_stride, const float* decay,
                                    float* state, const int* cu_tokens, const int* state_slots, float* o, int requests, int heads,
                                    int dim, int vdim, cudaStream_t s) {
    if (requests <= 0) return 0;
    if (heads <= 0 || dim <= 0 || vdim <= 0) return MB_ERR_BAD_SIZE;
    const int cols = vdim >= 64 ? 64 : 32;
    const size_t smem = ((size_t)dim * cols + 4 * (size_t)dim) * sizeof(float);
    if (smem > 200 * 1024) return MB_ERR_BAD_SIZE;
    dim3 grid(requests, heads, (vdim + cols - 1) / cols);
    if (dtype == MB_F32) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(linear_attention_scan_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return launch_kernel(linear_attention_scan_kernel<float>, grid, cols, smem, s, 0, (const float*)q, (const float*)k, (const float*)v,
                             row_stride, decay, state, cu_tokens, state_slots, o, heads, dim, vdim);
    }
    if (dtype == MB_BF16) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(linear_attention_scan_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return launch_kernel(linear_attention_scan_kernel<bf16>, grid, cols, smem, s, 0, (const bf16*)q, (const bf16*)k, (const bf16*)v,
                             row_stride, decay, state, cu_tokens, state_slots, o, heads, dim, vdim);
    }
    return MB_ERR_BAD_DTYPE;
}

// ---- time mixing with a decay per token and channel --------------------------------------------------------------------
// r, k, v, g: [T, heads * dim] in the activation dtype (g before its silu); wraw: float32 [T, heads * dim], the decay
// before its double exponential: w = exp(-exp(wraw + w0)).  u, w0, norm_w: float32 [heads * dim].  Each head's o is
// divided by its root mean square, times norm_w, times silu(g), and written in the activation dtype.  state: one row of
// state_stride floats per slot, [head][dim][dim] at `state`; the last row of h (the mixer's input, [T, width]) goes to
// `carry` in the same row for the next step's token shift.  grid (requests, heads), one thread per value channel.
template <typename T>
__global__ void wkv_scan_kernel(const T* __restrict__ rr, const T* __restrict__ kk, const T* __restrict__ vv, const T* __restrict__ gg,
                                const float* __restrict__ wraw, const float* __restrict__ w0, const float* __restrict__ u,
                                const float* __restrict__ norm_w, float eps, float* __restrict__ state, float* __restrict__ carry,
                                long long state_stride, const T* __restrict__ h, int width, const int* __restrict__ cu_tokens,
                                const int* __restrict__ state_slots, T* __restrict__ out, int heads, int dim) {
    PDL_ENTER();
    rr = pdl_fresh(rr); kk = pdl_fresh(kk); vv = pdl_fresh(vv); gg = pdl_fresh(gg); wraw = pdl_fresh(wraw); h = pdl_fresh(h);
    extern __shared__ float smem[];
    __shared__ float scratch[32];
    const int cols = blockDim.x;
    float* S = smem;                          // [dim][cols]
    float* us = smem + (size_t)dim * cols;    // [dim]
    float* rkw = us + dim;                    // [3 * dim]
    const int r = blockIdx.x, head = blockIdx.y, j = threadIdx.x;
    const bool live = j < dim;
    const int first = cu_tokens[r], count = cu_tokens[r + 1] - first;
    if (count <= 0) return;
    const size_t slot = (size_t)state_slots[r];
    float* st = state + slot * state_stride + (size_t)head * dim * dim;
    if (live)
        for (int i = 0; i < dim; ++i) S[i * cols + j] = st[(size_t)i * dim + j];
    for (int i = j; i < dim; i += cols) us[i] = u[(size_t)head * dim + i];
    const size_t n_all = (size_t)heads * dim;
    for (int n = 0; n < count; ++n) {
        const size_t t = (size_t)(first + n), at = t * n_all + (size_t)head * dim;
        __syncthreads();                      // the sums of the token before are done with rkw
        for (int i = j; i < dim; i += cols) {
            rkw[i] = to_f32(rr[at + i]);
            rkw[dim + i] = to_f32(kk[at + i]);
            rkw[2 * dim + i] = expf(-expf(wraw[at + i] + w0[(size_t)head * dim + i]));
        }
        const float vj = live ? to_f32(vv[at + j]) : 0.0f;
        __syncthreads();
        float acc = 0.0f;
        if (live) {
            for (int i = 0; i < dim; ++i) {
                const float s = S[i * cols + j];
                const float kv = rkw[dim + i] * vj;
                acc = fmaf(fmaf(us[i], kv, s), rkw[i], acc);
                S[i * cols + j] = fmaf(rkw[2 * dim + i], s, kv);
            }
        }
        const float ss = block_sum(acc * acc, scratch);
        if (live) {
            const float scale = 1.0f / sqrtf(ss / (float)dim + eps);
            const float z = to_f32(gg[at + j]);
            out[at + j] = from_f32<T>(acc * scale * norm_w[(size_t)head * dim + j] * silu_f(z));
        }
    }
    if (live)
        for (int i = 0; i < dim; ++i) st[(size_t)i * dim + j] = S[i * cols + j];
    if (head == 0) {
        const T* last = h + (size_t)(first + count - 1) * width;
        float* dst = carry + slot * state_stride;
        for (int i = j; i < width; i += cols) dst[i] = to_f32(last[i]);
    }
}

MB_API int mb_wkv_scan(const void* r, const void* k, const void* v, const void* g, int dtype, const float* wraw, const float* w0,
                       const float* u, const float* norm_w, float eps, float* state, float* carry, long long state_stride,
                       const void* h, int width, const int* cu_tokens, const int* state_slots, void* out, int requests, int heads,
                       int dim, cudaStream_t s) {
    if (requests <= 0) return 0;
    if (heads <= 0 || dim <= 0 || dim > 1024) return MB_ERR_BAD_SIZE;
    const int cols = (dim + 31) / 32 * 32;
    const size_t smem = ((size_t)dim * cols + 4 * (size_t)dim) * sizeof(float);
    if (smem > 200 * 1024) return MB_ERR_BAD_SIZE;
    dim3 grid(requests, heads);
    if (dtype == MB_F32) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(wkv_scan_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return launch_kernel(wkv_scan_kernel<float>, grid, cols, smem, s, 0, (const float*)r, (const float*)k, (const float*)v, (const float*)g,
                             wraw, w0, u, norm_w, eps, state, carry, state_stride, (const float*)h, width, cu_tokens, state_slots,
                             (float*)out, heads, dim);
    }
    if (dtype == MB_BF16) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(wkv_scan_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return launch_kernel(wkv_scan_kernel<bf16>, grid, cols, smem, s, 0, (const bf16*)r, (const bf16*)k, (const bf16*)v, (const bf16*)g,
                             wraw, w0, u, norm_w, eps, state, carry, state_stride, (const bf16*)h, width, cu_tokens, state_slots,
                             (bf16*)out, heads, dim);
    }
    return MB_ERR_BAD_DTYPE;
}
