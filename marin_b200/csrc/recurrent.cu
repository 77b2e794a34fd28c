// Recurrences over a request's tokens with a matrix-valued state per head, kept in float32 in a state slot per request:
//   * linear attention with a fixed decay per head:   S_t = decay_h S_(t-1) + k_t v_t^T,            o_t = S_t^T q_t
//   * time mixing with a decay per token and channel: o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t,   S_t = diag(w_t) S_(t-1) + k_t v_t^T
// One block walks the tokens a request brings to the step in order (a prompt portion or a single decoded token alike),
// starting from the state the steps before left and leaving the new one; the step's requests and the heads are the grid.
// Which tokens belong to a request, and its slot, are read from device arrays, so a captured graph replays the same
// launch for other requests.
//
// Threads: a block owns `cols` value channels (columns of the state); several threads (parts) share a column, each taking a
// contiguous run of the key channels (rows): 4 here (the kernels that keep their rows in registers, for key sizes 16, 32,
// 64 and 128, take the number as a template parameter).  The partial sums of a column are added in part order, and a
// thread's own sum runs over its rows in increasing order: a result does not depend on how the tokens were cut into
// steps or on what else the batch holds.  Per token there is one block-wide barrier: a token's inputs are fetched into
// registers while the token before is computed, and a token's partial sums are added after the next token's barrier.
// A request that brings a single token reads and writes its state in place (no copy in shared memory).
#define MB_LIB "recurrent"
#define MB_LIB_ID 9
#include "common.cuh"
#include "launch.cuh"

#define PARTS 4
#define MAX_FETCH 4                   // inputs a thread fetches ahead per token, at most
#define DEPTH 8                       // tokens whose inputs are in flight ahead of the one being computed (register-resident kernels)

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }

// ---- linear attention with a fixed decay per head ---------------------------------------------------------------------
// q, k: [T, heads * dim], v: [T, heads * vdim] with a common row stride (slices of one projection), before their
// activation: silu is applied here.  o: float32 [T, heads * vdim].  state: [slot][head][dim][vdim].
// grid (requests, heads, ceil(vdim / cols)), PARTS * cols threads (thread = part * cols + column).
template <typename T>
__global__ void linear_attention_scan_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, int row_stride,
                                             const float* __restrict__ decay, float* __restrict__ state,
                                             const int* __restrict__ cu_tokens, const int* __restrict__ state_slots,
                                             float* __restrict__ o, int heads, int dim, int vdim, int cols) {
    PDL_ENTER_WALK();
    q = pdl_fresh(q); k = pdl_fresh(k); v = pdl_fresh(v);
    extern __shared__ float smem[];
    float* qk = smem;                              // [2][2 * dim]: q then k of a token
    float* red = qk + 4 * dim;                     // [2][PARTS][cols]
    float* vs = red + 2 * PARTS * cols;            // [2][cols]
    float* S = vs + 2 * cols;                      // [dim][cols], only for requests with more than one token
    const int r = blockIdx.x, head = blockIdx.y;
    const int col = threadIdx.x % cols, part = threadIdx.x / cols;
    const int j = blockIdx.z * cols + col;
    const bool live = j < vdim;
    const int first = cu_tokens[r], count = cu_tokens[r + 1] - first;
    if (count <= 0) return;
    const int per = (dim + PARTS - 1) / PARTS;
    const int i_lo = min(dim, part * per), i_hi = min(dim, i_lo + per);
    float* st = state + (((size_t)state_slots[r] * heads + head) * dim) * vdim;
    const bool in_place = count == 1;
    if (!in_place && live)
        for (int i = i_lo; i < i_hi; ++i) S[i * cols + col] = st[(size_t)i * vdim + j];
    const float lam = decay[head];
    const int nthreads = blockDim.x;
    const size_t o_stride = (size_t)heads * vdim;
    // a token's inputs: element e < 2 dim of q|k (thread e, e + nthreads, ...) and this column's v
    float fetched[MAX_FETCH], v_next = 0.0f;
    auto fetch = [&](int n) {
        const size_t t = (size_t)(first + n);
#pragma unroll
        for (int f = 0; f < MAX_FETCH; ++f) {
            const int e = threadIdx.x + f * nthreads;
            if (e < 2 * dim) fetched[f] = to_f32((e < dim ? q : k)[t * row_stride + (size_t)head * dim + (e < dim ? e : e - dim)]);
        }
        if (live && part == 0) v_next = to_f32(v[t * row_stride + (size_t)head * vdim + j]);
    };
    fetch(0);
    for (int n = 0; n < count; ++n) {
        float* buf = qk + (n & 1) * 2 * dim;
#pragma unroll
        for (int f = 0; f < MAX_FETCH; ++f) {
            const int e = threadIdx.x + f * nthreads;
            if (e < 2 * dim) buf[e] = silu_f(fetched[f]);
        }
        if (part == 0) vs[(n & 1) * cols + col] = live ? silu_f(v_next) : 0.0f;
        if (n + 1 < count) fetch(n + 1);
        __syncthreads();
        if (n > 0 && part == 0 && live) {               // the token before: its four partial sums in part order
            const float* p = red + ((n - 1) & 1) * PARTS * cols + col;
            o[(size_t)(first + n - 1) * o_stride + (size_t)head * vdim + j] = ((p[0] + p[cols]) + p[2 * cols]) + p[3 * cols];
        }
        const float vj = vs[(n & 1) * cols + col];
        float acc = 0.0f;
        if (live) {
            if (in_place) {
#pragma unroll 4
                for (int i = i_lo; i < i_hi; ++i) {
                    const float s = fmaf(lam, st[(size_t)i * vdim + j], buf[dim + i] * vj);
                    st[(size_t)i * vdim + j] = s;
                    acc = fmaf(s, buf[i], acc);
                }
            } else {
                for (int i = i_lo; i < i_hi; ++i) {
                    const float s = fmaf(lam, S[i * cols + col], buf[dim + i] * vj);
                    S[i * cols + col] = s;
                    acc = fmaf(s, buf[i], acc);
                }
            }
        }
        red[(n & 1) * PARTS * cols + part * cols + col] = acc;
    }
    __syncthreads();
    if (part == 0 && live) {
        const float* p = red + ((count - 1) & 1) * PARTS * cols + col;
        o[(size_t)(first + count - 1) * o_stride + (size_t)head * vdim + j] = ((p[0] + p[cols]) + p[2 * cols]) + p[3 * cols];
    }
    if (!in_place && live)
        for (int i = i_lo; i < i_hi; ++i) st[(size_t)i * vdim + j] = S[i * cols + col];
}

// The same with the thread's rows of the state in registers (dim = PARTS * PER, PER a multiple of 4): no copy of the state in
// shared memory, q and k read four rows at a time.  The sums run in the same order as in the kernel above.
template <typename T, int NP, int PER>
__global__ void __launch_bounds__(NP * 64) linear_attention_scan_reg_kernel(
    const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, int row_stride, const float* __restrict__ decay,
    float* __restrict__ state, const int* __restrict__ cu_tokens, const int* __restrict__ state_slots, float* __restrict__ o,
    int heads, int vdim, int cols) {
    PDL_ENTER_WALK();
    q = pdl_fresh(q); k = pdl_fresh(k); v = pdl_fresh(v);
    constexpr int dim = NP * PER;
    constexpr int NF = (2 * dim + 127) / 128;      // q|k elements a thread fetches per token (the block has at least 128 threads)
    extern __shared__ __align__(16) float smem[];
    float* qk = smem;                              // [2][2 * dim]
    float* red = qk + 4 * dim;                     // [2][NP][cols]
    float* vs = red + 2 * NP * cols;               // [2][cols]
    const int r = blockIdx.x, head = blockIdx.y;
    const int col = threadIdx.x % cols, part = threadIdx.x / cols;
    const int j = blockIdx.z * cols + col;
    const bool live = j < vdim;
    const int first = cu_tokens[r], count = cu_tokens[r + 1] - first;
    if (count <= 0) return;
    const int i_lo = part * PER;
    float* st = state + (((size_t)state_slots[r] * heads + head) * dim + i_lo) * vdim + (live ? j : 0);
    float S[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) S[i] = live ? st[(size_t)i * vdim] : 0.0f;
    const float lam = decay[head];
    const int nthreads = blockDim.x;
    const size_t o_stride = (size_t)heads * vdim;
    // a token's inputs are asked for DEPTH tokens ahead and wait in registers: the walk never stands on a load
    float ring[DEPTH][NF], vring[DEPTH];
#define LIN_FETCH(slot, n)                                                                                             \
    do {                                                                                                               \
        const size_t t_ = (size_t)(first + (n));                                                                       \
        _Pragma("unroll") for (int f = 0; f < NF; ++f) {                                                               \
            const int e_ = threadIdx.x + f * nthreads;                                                                 \
            ring[slot][f] = e_ < 2 * dim ? to_f32((e_ < dim ? q : k)[t_ * row_stride + (size_t)head * dim + (e_ < dim ? e_ : e_ - dim)]) : 0.0f; \
        }                                                                                                              \
        vring[slot] = (live && part == 0) ? to_f32(v[t_ * row_stride + (size_t)head * vdim + j]) : 0.0f;               \
    } while (0)
#pragma unroll
    for (int u = 0; u < DEPTH; ++u) {
        if (u < count) LIN_FETCH(u, u);
    }
    for (int base = 0; base < count; base += DEPTH) {
#pragma unroll
        for (int u = 0; u < DEPTH; ++u) {
            const int n = base + u;
            if (n >= count) break;
            float* buf = qk + (n & 1) * 2 * dim;
#pragma unroll
            for (int f = 0; f < NF; ++f) {
                const int e = threadIdx.x + f * nthreads;
                if (e < 2 * dim) buf[e] = silu_f(ring[u][f]);
            }
            if (part == 0) vs[(n & 1) * cols + col] = live ? silu_f(vring[u]) : 0.0f;
            if (n + DEPTH < count) LIN_FETCH(u, n + DEPTH);
            __syncthreads();
            if (n > 0 && part == 0 && live) {
                const float* p = red + ((n - 1) & 1) * NP * cols + col;
                float sum = p[0];
#pragma unroll
                for (int w = 1; w < NP; ++w) sum += p[w * cols];       // the parts of a column in part order
                o[(size_t)(first + n - 1) * o_stride + (size_t)head * vdim + j] = sum;
            }
            const float vj = vs[(n & 1) * cols + col];
            const float4* q4 = reinterpret_cast<const float4*>(buf + i_lo);
            const float4* k4 = reinterpret_cast<const float4*>(buf + dim + i_lo);
            float acc = 0.0f;
#pragma unroll
            for (int i = 0; i < PER / 4; ++i) {
                const float4 kk = k4[i], qq = q4[i];
                S[4 * i] = fmaf(lam, S[4 * i], kk.x * vj);         acc = fmaf(S[4 * i], qq.x, acc);
                S[4 * i + 1] = fmaf(lam, S[4 * i + 1], kk.y * vj); acc = fmaf(S[4 * i + 1], qq.y, acc);
                S[4 * i + 2] = fmaf(lam, S[4 * i + 2], kk.z * vj); acc = fmaf(S[4 * i + 2], qq.z, acc);
                S[4 * i + 3] = fmaf(lam, S[4 * i + 3], kk.w * vj); acc = fmaf(S[4 * i + 3], qq.w, acc);
            }
            red[(n & 1) * NP * cols + part * cols + col] = acc;
        }
    }
#undef LIN_FETCH
    __syncthreads();
    if (part == 0 && live) {
        const float* p = red + ((count - 1) & 1) * NP * cols + col;
        float sum = p[0];
#pragma unroll
        for (int w = 1; w < NP; ++w) sum += p[w * cols];
        o[(size_t)(first + count - 1) * o_stride + (size_t)head * vdim + j] = sum;
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < PER; ++i) st[(size_t)i * vdim] = S[i];
    }
}

// dim -> (parts per column, rows per thread).  Measured on B200 (time mixing, 40 heads of 64, one prompt of 2,048 tokens):
// 4 parts of 16 rows and 16 parts of 4 rows take the same 1.3 us a token: the walk is bound by the instructions every warp
// spends per token around its few multiply-adds (staging, addresses, the barrier), 2,400 warp instructions a token with
// 32 warps and 1,200 with 8, issued at well under one a cycle; single tokens are faster with 4 parts (fewer, longer loads).
template <typename T>
static int linear_scan_reg(int dim, dim3 grid, int cols, cudaStream_t s, const void* q, const void* k, const void* v,
                           int row_stride, const float* decay, float* state, const int* cu_tokens, const int* state_slots, float* o,
                           int heads, int vdim) {
#define LIN_REG(NP, P)                                                                                                          \
    return launch_kernel(linear_attention_scan_reg_kernel<T, NP, P>, grid, NP * cols,                                            \
                         (4 * (size_t)dim + 2 * NP * cols + 2 * cols) * sizeof(float), s, 0, (const T*)q, (const T*)k, (const T*)v, \
                         row_stride, decay, state, cu_tokens, state_slots, o, heads, vdim, cols)
    switch (dim) {
        case 16: LIN_REG(4, 4);
        case 32: LIN_REG(4, 8);
        case 64: LIN_REG(4, 16);
        case 128: LIN_REG(4, 32);
    }
#undef LIN_REG
    return MB_ERR_BAD_SIZE;
}

MB_API int mb_linear_attention_scan(const void* q, const void* k, const void* v, int dtype, int row_stride, const float* decay,
                                    float* state, const int* cu_tokens, const int* state_slots, float* o, int requests, int heads,
                                    int dim, int vdim, cudaStream_t s) {
    if (requests <= 0) return 0;
    if (heads <= 0 || dim <= 0 || vdim <= 0) return MB_ERR_BAD_SIZE;
    const int cols = vdim >= 64 ? 64 : 32;
    const int threads = PARTS * cols;
    if (2 * dim > MAX_FETCH * threads) return MB_ERR_BAD_SIZE;
    const size_t smem = ((size_t)dim * cols + 4 * (size_t)dim + 2 * PARTS * cols + 2 * cols) * sizeof(float);
    if (smem > 200 * 1024) return MB_ERR_BAD_SIZE;
    dim3 grid(requests, heads, (vdim + cols - 1) / cols);
    if (dim == 16 || dim == 32 || dim == 64 || dim == 128) {       // the thread's rows of the state in registers
        if (dtype == MB_F32) return linear_scan_reg<float>(dim, grid, cols, s, q, k, v, row_stride, decay, state, cu_tokens, state_slots, o, heads, vdim);
        if (dtype == MB_BF16) return linear_scan_reg<bf16>(dim, grid, cols, s, q, k, v, row_stride, decay, state, cu_tokens, state_slots, o, heads, vdim);
        return MB_ERR_BAD_DTYPE;
    }
    if (dtype == MB_F32) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(linear_attention_scan_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return launch_kernel(linear_attention_scan_kernel<float>, grid, threads, smem, s, 0, (const float*)q, (const float*)k, (const float*)v,
                             row_stride, decay, state, cu_tokens, state_slots, o, heads, dim, vdim, cols);
    }
    if (dtype == MB_BF16) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(linear_attention_scan_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return launch_kernel(linear_attention_scan_kernel<bf16>, grid, threads, smem, s, 0, (const bf16*)q, (const bf16*)k, (const bf16*)v,
                             row_stride, decay, state, cu_tokens, state_slots, o, heads, dim, vdim, cols);
    }
    return MB_ERR_BAD_DTYPE;
}

// ---- time mixing with a decay per token and channel --------------------------------------------------------------------
// r, k, v: [T, heads * dim] in the activation dtype; wraw: float32 [T, heads * dim], the decay before its double
// exponential: w = exp(-exp(wraw + w0)).  u, w0: float32 [heads * dim].  o: float32 [T, heads * dim], before its norm
// (mb_head_norm_gate finishes it).  state: one row of state_stride floats per slot, [head][dim][dim] at `state`; the last
// row of h (the mixer's input, [T, width]) goes to `carry` in the same row for the next step's token shift.
// grid (requests, heads), PARTS * cols threads with cols = dim rounded up to a warp.
template <typename T>
__global__ void wkv_scan_kernel(const T* __restrict__ rr, const T* __restrict__ kk, const T* __restrict__ vv,
                                const float* __restrict__ wraw, const float* __restrict__ w0, const float* __restrict__ u,
                                float* __restrict__ state, float* __restrict__ carry, long long state_stride,
                                const T* __restrict__ h, int width, const int* __restrict__ cu_tokens,
                                const int* __restrict__ state_slots, float* __restrict__ o, int heads, int dim, int cols) {
    PDL_ENTER_WALK();
    rr = pdl_fresh(rr); kk = pdl_fresh(kk); vv = pdl_fresh(vv); wraw = pdl_fresh(wraw); h = pdl_fresh(h);
    extern __shared__ float smem[];
    float* rkw = smem;                             // [2][3 * dim]: r, k, decay of a token
    float* us = rkw + 6 * dim;                     // [dim]
    float* red = us + dim;                         // [2][PARTS][cols]
    float* vs = red + 2 * PARTS * cols;            // [2][cols]
    float* S = vs + 2 * cols;                      // [dim][cols], only for requests with more than one token
    const int r = blockIdx.x, head = blockIdx.y;
    const int col = threadIdx.x % cols, part = threadIdx.x / cols, j = col;
    const bool live = j < dim;
    const int first = cu_tokens[r], count = cu_tokens[r + 1] - first;
    if (count <= 0) return;
    const int per = (dim + PARTS - 1) / PARTS;
    const int i_lo = min(dim, part * per), i_hi = min(dim, i_lo + per);
    const size_t slot = (size_t)state_slots[r];
    float* st = state + slot * state_stride + (size_t)head * dim * dim;
    const bool in_place = count == 1;
    if (!in_place && live)
        for (int i = i_lo; i < i_hi; ++i) S[i * cols + col] = st[(size_t)i * dim + j];
    const int nthreads = blockDim.x;
    for (int i = threadIdx.x; i < dim; i += nthreads) us[i] = u[(size_t)head * dim + i];
    const size_t n_all = (size_t)heads * dim;
    // a token's inputs: element e < 3 dim of r|k|wraw (thread e; 3 dim <= 4 cols <= the block) and this column's v
    float fetched = 0.0f, w_off = 0.0f, v_next = 0.0f;
    const int e = threadIdx.x, which = e / dim, ei = e % dim;
    if (e < 3 * dim && which == 2) w_off = w0[(size_t)head * dim + ei];
    auto fetch = [&](int n) {
        const size_t at = (size_t)(first + n) * n_all + (size_t)head * dim;
        if (e < 3 * dim) fetched = which == 0 ? to_f32(rr[at + ei]) : which == 1 ? to_f32(kk[at + ei]) : wraw[at + ei];
        if (live && part == 0) v_next = to_f32(vv[at + j]);
    };
    fetch(0);
    for (int n = 0; n < count; ++n) {
        float* buf = rkw + (n & 1) * 3 * dim;
        if (e < 3 * dim) buf[e] = which == 2 ? expf(-expf(fetched + w_off)) : fetched;
        if (part == 0) vs[(n & 1) * cols + col] = live ? v_next : 0.0f;
        if (n + 1 < count) fetch(n + 1);
        __syncthreads();
        if (n > 0 && part == 0 && live) {               // the token before: its four partial sums in part order
            const float* p = red + ((n - 1) & 1) * PARTS * cols + col;
            o[(size_t)(first + n - 1) * n_all + (size_t)head * dim + j] = ((p[0] + p[cols]) + p[2 * cols]) + p[3 * cols];
        }
        const float vj = vs[(n & 1) * cols + col];
        float acc = 0.0f;
        if (live) {
            if (in_place) {
#pragma unroll 4
                for (int i = i_lo; i < i_hi; ++i) {
                    const float s = st[(size_t)i * dim + j];
                    const float kv = buf[dim + i] * vj;
                    acc = fmaf(fmaf(us[i], kv, s), buf[i], acc);
                    st[(size_t)i * dim + j] = fmaf(buf[2 * dim + i], s, kv);
                }
            } else {
                for (int i = i_lo; i < i_hi; ++i) {
                    const float s = S[i * cols + col];
                    const float kv = buf[dim + i] * vj;
                    acc = fmaf(fmaf(us[i], kv, s), buf[i], acc);
                    S[i * cols + col] = fmaf(buf[2 * dim + i], s, kv);
                }
            }
        }
        red[(n & 1) * PARTS * cols + part * cols + col] = acc;
    }
    __syncthreads();
    if (part == 0 && live) {
        const float* p = red + ((count - 1) & 1) * PARTS * cols + col;
        o[(size_t)(first + count - 1) * n_all + (size_t)head * dim + j] = ((p[0] + p[cols]) + p[2 * cols]) + p[3 * cols];
    }
    if (!in_place && live)
        for (int i = i_lo; i < i_hi; ++i) st[(size_t)i * dim + j] = S[i * cols + col];
    if (head == 0) {
        const T* last = h + (size_t)(first + count - 1) * width;
        float* dst = carry + slot * state_stride;
        for (int i = threadIdx.x; i < width; i += nthreads) dst[i] = to_f32(last[i]);
    }
}

// The same with the thread's rows of the state (and of u) in registers (dim = PARTS * PER, PER a multiple of 4).
// MODE 0: a request's tokens of the step in one walk, from its state slot and back into it.
// A long portion is cut into blocks of `block_len` tokens that are walked side by side (the recurrence is linear in the state):
// MODE 1: each block from a zero state, no outputs; it leaves its end state and the product of its decays per key channel in
//         `block_state` [request * nblocks + block][head][dim][dim] and `block_decay` [..][head][dim];
// (wkv_combine_kernel then turns the end states into the states the blocks start from: S <- W_b S + S_b, block after block)
// MODE 2: each block again, now from its true start state in `block_state`, writing the outputs.
template <typename T, int NP, int PER, int MODE>
__global__ void __launch_bounds__(NP * ((NP * PER) < 64 ? 32 : 64)) wkv_scan_reg_kernel(
    const T* __restrict__ rr, const T* __restrict__ kk, const T* __restrict__ vv, const float* __restrict__ wraw,
    const float* __restrict__ w0, const float* __restrict__ u, float* __restrict__ state, float* __restrict__ carry,
    long long state_stride, const T* __restrict__ h, int width, const int* __restrict__ cu_tokens,
    const int* __restrict__ state_slots, float* __restrict__ o, int heads, float* __restrict__ block_state,
    float* __restrict__ block_decay, int nblocks, int block_len) {
    PDL_ENTER_WALK();
    block_state = pdl_fresh(block_state);
    rr = pdl_fresh(rr); kk = pdl_fresh(kk); vv = pdl_fresh(vv); wraw = pdl_fresh(wraw); h = pdl_fresh(h);
    constexpr int dim = NP * PER, cols = dim < 64 ? 32 : 64;      // a head's columns are split over CTAs beyond 64
    __shared__ __align__(16) float rkw[2][3 * dim];
    __shared__ float red[2][NP][cols], vs[2][cols], outs[2 * DEPTH][cols];
    const int r = MODE == 0 ? blockIdx.x : blockIdx.x / nblocks, blk = MODE == 0 ? 0 : blockIdx.x % nblocks, head = blockIdx.y;
    const int col = threadIdx.x % cols, part = threadIdx.x / cols, j = blockIdx.z * cols + col;
    const bool live = j < dim;
    const int all_first = cu_tokens[r], all_count = cu_tokens[r + 1] - all_first;
    const int skip = MODE == 0 ? 0 : blk * block_len;
    if (all_count - skip <= 0) return;
    const int first = all_first + skip, count = MODE == 0 ? all_count : min(block_len, all_count - skip);
    const int i_lo = part * PER;
    const size_t slot = (size_t)state_slots[r];
    float* st = MODE == 0 ? state + slot * state_stride + ((size_t)head * dim + i_lo) * dim + (live ? j : 0)
                          : block_state + ((((size_t)r * nblocks + blk) * heads + head) * dim + i_lo) * dim + (live ? j : 0);
    float S[PER], U[PER], W[MODE == 1 ? PER : 1];
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        S[i] = (live && MODE != 1) ? st[(size_t)i * dim] : 0.0f;
        U[i] = u[(size_t)head * dim + i_lo + i];
        if (MODE == 1) W[i] = 1.0f;
    }
    const int nthreads = blockDim.x;
    const size_t n_all = (size_t)heads * dim;
    // this thread's elements of a token's r|k|wraw: e = thread, thread + block, ... < 3 dim
    constexpr int NF = (3 * dim + NP * cols - 1) / (NP * cols);
    float w_off[NF];
#pragma unroll
    for (int f = 0; f < NF; ++f) {
        const int e = threadIdx.x + f * NP * cols;
        w_off[f] = (e >= 2 * dim && e < 3 * dim) ? w0[(size_t)head * dim + e - 2 * dim] : 0.0f;
    }
    // a token's inputs are asked for DEPTH tokens ahead and wait in registers: the walk never stands on a load
    float ring[DEPTH][NF], vring[DEPTH];
#define WKV_FETCH(slot_, n)                                                                                            \
    do {                                                                                                               \
        const size_t at_ = (size_t)(first + (n)) * n_all + (size_t)head * dim;                                         \
        _Pragma("unroll") for (int f = 0; f < NF; ++f) {                                                               \
            const int e_ = threadIdx.x + f * NP * cols;                                                                \
            ring[slot_][f] = e_ < dim ? to_f32(rr[at_ + e_]) : e_ < 2 * dim ? to_f32(kk[at_ + e_ - dim])               \
                                      : e_ < 3 * dim ? wraw[at_ + e_ - 2 * dim] : 0.0f;                                \
        }                                                                                                              \
        vring[slot_] = (live && part == 0) ? to_f32(vv[at_ + j]) : 0.0f;                                               \
    } while (0)
#pragma unroll
    for (int d = 0; d < DEPTH; ++d) {
        if (d < count) WKV_FETCH(d, d);
    }
    for (int base = 0; base < count; base += DEPTH) {
#pragma unroll
        for (int d = 0; d < DEPTH; ++d) {
            const int n = base + d;
            if (n >= count) break;
            float* buf = rkw[n & 1];
#pragma unroll
            for (int f = 0; f < NF; ++f) {
                const int e = threadIdx.x + f * NP * cols;
                if (e < 3 * dim) buf[e] = e >= 2 * dim ? expf(-expf(ring[d][f] + w_off[f])) : ring[d][f];
            }
            if (part == 0) vs[n & 1][col] = vring[d];
            if (n + DEPTH < count) WKV_FETCH(d, n + DEPTH);
            __syncthreads();
            if (MODE != 1 && n > 0 && part == 0) {             // the token before: the parts of its column in part order
                const float (*p)[cols] = red[(n - 1) & 1];
                float sum = p[0][col];
#pragma unroll
                for (int w = 1; w < NP; ++w) sum += p[w][col];
                outs[(n - 1) % (2 * DEPTH)][col] = sum;
            }
            // Outputs leave in runs of DEPTH tokens, all threads storing, instead of one store per token from a quarter of them.
            // The run written here was gathered before this token's barrier; the other half of the ring is being filled.
            if (MODE != 1 && n > DEPTH && (n - 1) % DEPTH == 0) {
                for (int i = threadIdx.x; i < DEPTH * cols; i += nthreads) {
                    const int tt = n - 1 - DEPTH + i / cols, cc = i % cols;
                    if (blockIdx.z * cols + cc < dim)
                        o[(size_t)(first + tt) * n_all + (size_t)head * dim + blockIdx.z * cols + cc] = outs[tt % (2 * DEPTH)][cc];
                }
            }
            const float vj = vs[n & 1][col];
            const float4* r4 = reinterpret_cast<const float4*>(buf + i_lo);
            const float4* k4 = reinterpret_cast<const float4*>(buf + dim + i_lo);
            const float4* w4 = reinterpret_cast<const float4*>(buf + 2 * dim + i_lo);
            if (MODE == 1) {                                   // the state and the product of the decays only
#pragma unroll
                for (int i = 0; i < PER / 4; ++i) {
                    const float4 ki = k4[i], wi = w4[i];
                    S[4 * i] = fmaf(wi.x, S[4 * i], ki.x * vj);         W[4 * i] *= wi.x;
                    S[4 * i + 1] = fmaf(wi.y, S[4 * i + 1], ki.y * vj); W[4 * i + 1] *= wi.y;
                    S[4 * i + 2] = fmaf(wi.z, S[4 * i + 2], ki.z * vj); W[4 * i + 2] *= wi.z;
                    S[4 * i + 3] = fmaf(wi.w, S[4 * i + 3], ki.w * vj); W[4 * i + 3] *= wi.w;
                }
            } else {
                float acc = 0.0f;
#pragma unroll
                for (int i = 0; i < PER / 4; ++i) {
                    const float4 ri = r4[i], ki = k4[i], wi = w4[i];
                    float kv;
                    kv = ki.x * vj; acc = fmaf(fmaf(U[4 * i], kv, S[4 * i]), ri.x, acc);         S[4 * i] = fmaf(wi.x, S[4 * i], kv);
                    kv = ki.y * vj; acc = fmaf(fmaf(U[4 * i + 1], kv, S[4 * i + 1]), ri.y, acc); S[4 * i + 1] = fmaf(wi.y, S[4 * i + 1], kv);
                    kv = ki.z * vj; acc = fmaf(fmaf(U[4 * i + 2], kv, S[4 * i + 2]), ri.z, acc); S[4 * i + 2] = fmaf(wi.z, S[4 * i + 2], kv);
                    kv = ki.w * vj; acc = fmaf(fmaf(U[4 * i + 3], kv, S[4 * i + 3]), ri.w, acc); S[4 * i + 3] = fmaf(wi.w, S[4 * i + 3], kv);
                }
                red[n & 1][part][col] = acc;
            }
        }
    }
#undef WKV_FETCH
    if (MODE == 1) {
        if (live) {
#pragma unroll
            for (int i = 0; i < PER; ++i) st[(size_t)i * dim] = S[i];
        }
        if (col == 0 && blockIdx.z == 0) {
            float* wd = block_decay + (((size_t)r * nblocks + blk) * heads + head) * dim + i_lo;
#pragma unroll
            for (int i = 0; i < PER; ++i) wd[i] = W[i];
        }
        return;
    }
    __syncthreads();
    if (part == 0) {
        const float (*p)[cols] = red[(count - 1) & 1];
        float sum = p[0][col];
#pragma unroll
        for (int w = 1; w < NP; ++w) sum += p[w][col];
        outs[(count - 1) % (2 * DEPTH)][col] = sum;
    }
    __syncthreads();
    {   // the tokens not yet stored: from the last run's end (a run is stored when the token DEPTH + 1 after its first arrives)
        const int done = count > DEPTH + 1 ? ((count - 2) / DEPTH) * DEPTH : 0;
        for (int i = threadIdx.x; i < (count - done) * cols; i += nthreads) {
            const int tt = done + i / cols, cc = i % cols;
            if (blockIdx.z * cols + cc < dim)
                o[(size_t)(first + tt) * n_all + (size_t)head * dim + blockIdx.z * cols + cc] = outs[tt % (2 * DEPTH)][cc];
        }
    }
    if (MODE != 0) return;                                 // the combine kernel has left the state and the carried row
    if (live) {
#pragma unroll
        for (int i = 0; i < PER; ++i) st[(size_t)i * dim] = S[i];
    }
    if (head == 0 && blockIdx.z == 0) {
        const T* last = h + (size_t)(first + count - 1) * width;
        float* dst = carry + slot * state_stride;
        for (int i = threadIdx.x; i < width; i += nthreads) dst[i] = to_f32(last[i]);
    }
}

// Between the two walks over blocks: per request, head and state element, block after block, the end state of a block walked
// from zero becomes the state the block starts from, S_start(b + 1) = W_b S_start(b) + S_end(b), beginning with the request's
// state slot and ending in it; the request's last input row goes to the carried row.  grid (requests, heads, runs of 256 elements).
template <typename T>
__global__ void wkv_combine_kernel(float* __restrict__ state, float* __restrict__ carry, long long state_stride, const T* __restrict__ h,
                                   int width, const int* __restrict__ cu_tokens, const int* __restrict__ state_slots,
                                   float* __restrict__ block_state, const float* __restrict__ block_decay, int heads, int dim,
                                   int nblocks, int block_len) {
    PDL_ENTER();
    block_state = pdl_fresh(block_state); block_decay = pdl_fresh(block_decay); h = pdl_fresh(h);
    const int r = blockIdx.x, head = blockIdx.y;
    const int first = cu_tokens[r], count = cu_tokens[r + 1] - first;
    if (count <= 0) return;
    const int blocks = (count + block_len - 1) / block_len;
    const size_t slot = (size_t)state_slots[r];
    float* st = state + slot * state_stride + (size_t)head * dim * dim;
    for (int idx = blockIdx.z * blockDim.x + threadIdx.x; idx < dim * dim; idx += gridDim.z * blockDim.x) {
        const int i = idx / dim;
        float S = st[idx];
        for (int b = 0; b < blocks; ++b) {
            const size_t at = ((size_t)r * nblocks + b) * heads + head;
            const float end = block_state[at * dim * dim + idx];
            block_state[at * dim * dim + idx] = S;
            S = fmaf(block_decay[at * dim + i], S, end);
        }
        st[idx] = S;
    }
    if (head == 0 && blockIdx.z == 0) {
        const T* last = h + (size_t)(first + count - 1) * width;
        float* dst = carry + slot * state_stride;
        for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = to_f32(last[i]);
    }
}

template <typename T>
static int wkv_scan_reg(int dim, int requests, cudaStream_t s, const void* r, const void* k, const void* v, const float* wraw, const float* w0,
                        const float* u, float* state, float* carry, long long state_stride, const void* h, int width,
                        const int* cu_tokens, const int* state_slots, float* o, int heads, float* block_state, float* block_decay,
                        int nblocks, int block_len) {
    const int cols = dim < 64 ? 32 : 64;
    const int zs = (dim + cols - 1) / cols;
#define WKV_ARGS (const T*)r, (const T*)k, (const T*)v, wraw, w0, u, state, carry, state_stride, (const T*)h, width, cu_tokens, state_slots, o, \
                 heads, block_state, block_decay, nblocks, block_len
#define WKV_REG(NP, P)                                                                                                             \
    do {                                                                                                                           \
        if (nblocks <= 1) return launch_kernel(wkv_scan_reg_kernel<T, NP, P, 0>, dim3(requests, heads, zs), NP * cols, 0, s, 0, WKV_ARGS); \
        int rc = launch_kernel(wkv_scan_reg_kernel<T, NP, P, 1>, dim3(requests * nblocks, heads, zs), NP * cols, 0, s, 0, WKV_ARGS);    \
        if (rc != 0) return rc;                                                                                                    \
        rc = launch_kernel(wkv_combine_kernel<T>, dim3(requests, heads, (dim * dim + 255) / 256), 256, 0, s, 0, state, carry, state_stride, (const T*)h, width, \
                           cu_tokens, state_slots, block_state, (const float*)block_decay, heads, dim, nblocks, block_len);           \
        if (rc != 0) return rc;                                                                                                    \
        return launch_kernel(wkv_scan_reg_kernel<T, NP, P, 2>, dim3(requests * nblocks, heads, zs), NP * cols, 0, s, 0, WKV_ARGS);     \
    } while (0)
    switch (dim) {
        case 16: WKV_REG(4, 4);
        case 32: WKV_REG(4, 8);
        case 64: WKV_REG(4, 16);
        case 128: WKV_REG(4, 32);
    }
#undef WKV_REG
#undef WKV_ARGS
    return MB_ERR_BAD_SIZE;
}

// nblocks > 1 (key sizes 16, 32, 64, 128 only): every request's tokens are cut into blocks of block_len tokens that are walked
// side by side, in three launches; block_state: float32 [requests * nblocks][heads][dim][dim], block_decay: [..][heads][dim].
MB_API int mb_wkv_scan(const void* r, const void* k, const void* v, int dtype, const float* wraw, const float* w0, const float* u,
                       float* state, float* carry, long long state_stride, const void* h, int width, const int* cu_tokens,
                       const int* state_slots, float* o, int requests, int heads, int dim, float* block_state, float* block_decay,
                       int nblocks, int block_len, cudaStream_t s) {
    if (requests <= 0) return 0;
    if (nblocks > 1 && (block_state == nullptr || block_decay == nullptr || block_len <= 0 || !(dim == 16 || dim == 32 || dim == 64 || dim == 128)))
        return MB_ERR_BAD_SIZE;
    if (heads <= 0 || dim <= 0 || dim > 256) return MB_ERR_BAD_SIZE;
    const int cols = (dim + 31) / 32 * 32;
    const int threads = PARTS * cols;
    const size_t smem = ((size_t)dim * cols + 7 * (size_t)dim + 2 * PARTS * cols + 2 * cols) * sizeof(float);
    if (smem > 200 * 1024) return MB_ERR_BAD_SIZE;
    dim3 grid(requests, heads);
    if (dim == 16 || dim == 32 || dim == 64 || dim == 128) {       // the thread's rows of the state in registers
        if (dtype == MB_F32) return wkv_scan_reg<float>(dim, requests, s, r, k, v, wraw, w0, u, state, carry, state_stride, h, width, cu_tokens, state_slots, o, heads, block_state, block_decay, nblocks, block_len);
        if (dtype == MB_BF16) return wkv_scan_reg<bf16>(dim, requests, s, r, k, v, wraw, w0, u, state, carry, state_stride, h, width, cu_tokens, state_slots, o, heads, block_state, block_decay, nblocks, block_len);
        return MB_ERR_BAD_DTYPE;
    }
    if (dtype == MB_F32) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(wkv_scan_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return launch_kernel(wkv_scan_kernel<float>, grid, threads, smem, s, 0, (const float*)r, (const float*)k, (const float*)v, wraw, w0, u,
                             state, carry, state_stride, (const float*)h, width, cu_tokens, state_slots, o, heads, dim, cols);
    }
    if (dtype == MB_BF16) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(wkv_scan_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return launch_kernel(wkv_scan_kernel<bf16>, grid, threads, smem, s, 0, (const bf16*)r, (const bf16*)k, (const bf16*)v, wraw, w0, u,
                             state, carry, state_stride, (const bf16*)h, width, cu_tokens, state_slots, o, heads, dim, cols);
    }
    return MB_ERR_BAD_DTYPE;
}

// ---- per-head RMS norm, weight and gate: out[t, head, :] = o / sqrt(mean_head(o^2) + eps) * w[head, :] * silu(g) -------------
// One warp per (token, head); o float32 [T, heads * dim], g and out in the activation dtype, w float32 [heads * dim].
template <typename T>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ w, const T* __restrict__ g, float eps,
                                      T* __restrict__ out, int rows, int heads, int dim) {
    PDL_ENTER();
    o = pdl_fresh(o); g = pdl_fresh(g);
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= rows) return;
    const float* src = o + (size_t)row * dim;
    const float* wrow = w + (size_t)(row % heads) * dim;
    float ss = 0.0f;
    for (int i = lane; i < dim; i += 32) { const float x = src[i]; ss += x * x; }
    ss = warp_sum(ss);
    const float scale = 1.0f / sqrtf(ss / (float)dim + eps);
    for (int i = lane; i < dim; i += 32) {
        const size_t at = (size_t)row * dim + i;
        out[at] = from_f32<T>(src[i] * scale * wrow[i] * silu_f(to_f32(g[at])));
    }
}

MB_API int mb_head_norm_gate(const float* o, const float* w, const void* g, int dtype, float eps, void* out, int tokens, int heads, int dim,
                             cudaStream_t s) {
    const int rows = tokens * heads;
    if (rows <= 0) return 0;
    if (dim <= 0) return MB_ERR_BAD_SIZE;
    const int warps = 8;
    const int blocks = (rows + warps - 1) / warps;
    if (dtype == MB_F32)
        return launch_kernel(head_norm_gate_kernel<float>, blocks, warps * 32, 0, s, 0, o, w, (const float*)g, eps, (float*)out, rows, heads, dim);
    if (dtype == MB_BF16)
        return launch_kernel(head_norm_gate_kernel<bf16>, blocks, warps * 32, 0, s, 0, o, w, (const bf16*)g, eps, (bf16*)out, rows, heads, dim);
    return MB_ERR_BAD_DTYPE;
}
