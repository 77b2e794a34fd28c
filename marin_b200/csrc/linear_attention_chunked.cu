// Linear attention with a fixed decay per head over prompt portions, in chunks of 64 tokens on the tensor cores (mma.sync),
// compiled for one head layout: -DQK_DIM (query/key channels, a multiple of 16 up to 128), -DV_SLICE (value channels a
// CTA takes: 64 or 32; the value channels of a head are split over CTAs, the state's columns being independent).
//
// With S the state before a chunk of n <= 64 tokens, lam the head's decay, i, j positions inside the chunk:
//   o_i   = lam^(i+1) S^T q_i + sum_{j <= i} lam^(i-j) (q_i . k_j) v_j
//   S_new = lam^n S + sum_j lam^(n-1-j) k_j v_j^T
// which is the recurrence S_t = lam S_(t-1) + k_t v_t^T, o_t = S_t^T q_t written for 64 tokens at a time.  q, k, v arrive
// before their activation (silu is applied on the way into shared memory) and are bf16 operands; the state stays float32:
// it lives in the accumulator registers of the state update across the chunks of a request, and where it or another
// float32 factor has to be an operand of a product (S in q S, the decayed weights in P V, the decayed values in K^T V)
// it is split into two bf16 numbers (value = hi + lo) and multiplied twice, so that no more than the operands' own
// rounding enters.  One CTA walks one request's tokens of the step in order, from the state the steps before left.
#define MB_LIB "linear_attention_chunked"
#define MB_LIB_ID 12
#include "common.cuh"
#include "launch.cuh"
#include "mma_helpers.cuh"

#ifndef QK_DIM
#define QK_DIM 128
#endif
#ifndef V_SLICE
#define V_SLICE 64
#endif
static_assert(QK_DIM % 16 == 0 && QK_DIM >= 16 && QK_DIM <= 128, "query/key channels: a multiple of 16 up to 128");
static_assert(V_SLICE == 32 || V_SLICE == 64, "a CTA takes 32 or 64 value channels");

#define DQ QK_DIM
#define VS V_SLICE
#define CH 64
#define LDQ (DQ + 8)
#define LDS (VS + 8)
#define MT (DQ / 16)                  // 16-row tiles of the state
#define MT_W ((MT + 3) / 4)           // of which a warp owns at most this many: tiles warp, warp + 4, ...
#define NT (VS / 8)
#define LC_SMEM ((2 * CH * LDQ + 3 * CH * LDS + 2 * DQ * LDS) * 2 + 80 * 4)

// z / (1 + e^-z) with the fast exponential and division: the result is rounded to bf16, which hides their last bits, and
// the accurate ones were most of this kernel's instructions (144 activations a thread and chunk)
__device__ __forceinline__ float silu_f(float z) { return __fdividef(z, 1.0f + __expf(-z)); }

__device__ __forceinline__ void split_bf16(float x, float y, uint32_t& hi, uint32_t& lo) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
    const float2 back = __bfloat1622float2(h);
    hi = *reinterpret_cast<const uint32_t*>(&h);
    lo = pack_bf16(x - back.x, y - back.y);
}

__global__ void __launch_bounds__(128) linear_attention_chunked_kernel(
    const bf16* __restrict__ q, const bf16* __restrict__ k, const bf16* __restrict__ v, int row_stride,
    const float* __restrict__ decay, float* __restrict__ state, const int* __restrict__ cu_tokens,
    const int* __restrict__ state_slots, float* __restrict__ o, int heads, int vdim) {
    PDL_ENTER_WALK();
    q = pdl_fresh(q); k = pdl_fresh(k); v = pdl_fresh(v);
    extern __shared__ __align__(16) uint8_t smem_raw[];
    bf16* sQ = reinterpret_cast<bf16*>(smem_raw);     // [CH][LDQ]
    bf16* sK = sQ + CH * LDQ;                         // [CH][LDQ]
    bf16* sV = sK + CH * LDQ;                         // [CH][LDS]
    bf16* sVh = sV + CH * LDS;                        // decayed values, high and low parts
    bf16* sVl = sVh + CH * LDS;
    bf16* sSh = sVl + CH * LDS;                       // [DQ][LDS] the state, high and low parts
    bf16* sSl = sSh + DQ * LDS;
    float* pw = reinterpret_cast<float*>(sSl + DQ * LDS);   // lam^n, n = 0 .. 64
    const int r = blockIdx.x, head = blockIdx.y, vs0 = blockIdx.z * VS;
    const int first = cu_tokens[r], count = cu_tokens[r + 1] - first;
    if (count <= 0) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t2 = 2 * (lane & 3);
    const float lam = decay[head];
    if (threadIdx.x <= CH) pw[threadIdx.x] = threadIdx.x == 0 ? 1.0f : (lam > 0.0f ? exp2f((float)threadIdx.x * log2f(lam)) : 0.0f);
    float* st = state + (((size_t)state_slots[r] * heads + head) * DQ) * vdim + vs0;
    float S[MT_W][NT][4];
#pragma unroll
    for (int mi = 0; mi < MT_W; ++mi) {
        const int m0 = (warp + 4 * mi) * 16;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            if (m0 < DQ) {
                const float2 a = *reinterpret_cast<const float2*>(st + (size_t)(m0 + g) * vdim + nt * 8 + t2);
                const float2 b = *reinterpret_cast<const float2*>(st + (size_t)(m0 + g + 8) * vdim + nt * 8 + t2);
                S[mi][nt][0] = a.x; S[mi][nt][1] = a.y; S[mi][nt][2] = b.x; S[mi][nt][3] = b.y;
            } else {
                S[mi][nt][0] = S[mi][nt][1] = S[mi][nt][2] = S[mi][nt][3] = 0.0f;
            }
        }
    }
    const size_t o_stride = (size_t)heads * vdim;
    for (int c0 = 0; c0 < count; c0 += CH) {
        const int rows = min(CH, count - c0);
        __syncthreads();                                   // the chunk before is done with every buffer (and pw is written)
        // the state as two bf16 operands
#pragma unroll
        for (int mi = 0; mi < MT_W; ++mi) {
            const int m0 = (warp + 4 * mi) * 16;
            if (m0 < DQ) {
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    uint32_t hi, lo;
                    split_bf16(S[mi][nt][0], S[mi][nt][1], hi, lo);
                    *reinterpret_cast<uint32_t*>(sSh + (m0 + g) * LDS + nt * 8 + t2) = hi;
                    *reinterpret_cast<uint32_t*>(sSl + (m0 + g) * LDS + nt * 8 + t2) = lo;
                    split_bf16(S[mi][nt][2], S[mi][nt][3], hi, lo);
                    *reinterpret_cast<uint32_t*>(sSh + (m0 + g + 8) * LDS + nt * 8 + t2) = hi;
                    *reinterpret_cast<uint32_t*>(sSl + (m0 + g + 8) * LDS + nt * 8 + t2) = lo;
                }
            }
        }
        // the chunk's q and k (activated), rows past the request's tokens zero; eight loads of a thread in flight at a time
        constexpr int QK_ITERS = CH * (DQ / 8) * 2 / 128, QK_BATCH = QK_ITERS % 8 == 0 ? 8 : (QK_ITERS % 4 == 0 ? 4 : 2);
        static_assert(CH * (DQ / 8) * 2 % 128 == 0 && QK_ITERS % QK_BATCH == 0, "q and k vectors divide evenly over the threads");
#pragma unroll
        for (int b0 = 0; b0 < QK_ITERS; b0 += QK_BATCH) {
            uint4 raw[QK_BATCH];
#pragma unroll
            for (int u = 0; u < QK_BATCH; ++u) {
                const int idx = threadIdx.x + (b0 + u) * 128;
                const int which = idx / (CH * (DQ / 8)), rest = idx % (CH * (DQ / 8));
                const int row = rest / (DQ / 8), c = rest % (DQ / 8);
                raw[u] = make_uint4(0, 0, 0, 0);
                if (row < rows) raw[u] = *reinterpret_cast<const uint4*>((which ? k : q) + (size_t)(first + c0 + row) * row_stride + (size_t)head * DQ + c * 8);
            }
#pragma unroll
            for (int u = 0; u < QK_BATCH; ++u) {
                const int idx = threadIdx.x + (b0 + u) * 128;
                const int which = idx / (CH * (DQ / 8)), rest = idx % (CH * (DQ / 8));
                const int row = rest / (DQ / 8), c = rest % (DQ / 8);
                const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw[u]);
                uint4 packed;
                uint32_t* p = reinterpret_cast<uint32_t*>(&packed);
#pragma unroll
                for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h2[i]); p[i] = pack_bf16(silu_f(f.x), silu_f(f.y)); }
                *reinterpret_cast<uint4*>((which ? sK : sQ) + row * LDQ + c * 8) = packed;       // silu(0) = 0: padded rows stay zero
            }
        }
        // v (activated) and v times lam^(rows - 1 - row) as two bf16 operands
        constexpr int V_ITERS = CH * (VS / 8) / 128;
        uint4 vraw[V_ITERS];
#pragma unroll
        for (int u = 0; u < V_ITERS; ++u) {
            const int idx = threadIdx.x + u * 128;
            const int row = idx / (VS / 8), c = idx % (VS / 8);
            vraw[u] = make_uint4(0, 0, 0, 0);
            if (row < rows) vraw[u] = *reinterpret_cast<const uint4*>(v + (size_t)(first + c0 + row) * row_stride + (size_t)head * vdim + vs0 + c * 8);
        }
#pragma unroll
        for (int u = 0; u < V_ITERS; ++u) {
            const int idx = threadIdx.x + u * 128;
            const int row = idx / (VS / 8), c = idx % (VS / 8);
            uint4 pv, ph, pl;
            const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&vraw[u]);
            const float f = row < rows ? pw[rows - 1 - row] : 0.0f;
            uint32_t *a = reinterpret_cast<uint32_t*>(&pv), *b = reinterpret_cast<uint32_t*>(&ph), *cc = reinterpret_cast<uint32_t*>(&pl);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 z = __bfloat1622float2(h2[i]);
                const __nv_bfloat162 act = __floats2bfloat162_rn(silu_f(z.x), silu_f(z.y));
                a[i] = *reinterpret_cast<const uint32_t*>(&act);
                const float2 back = __bfloat1622float2(act);     // the decayed value of the operand the other products see
                split_bf16(back.x * f, back.y * f, b[i], cc[i]);
            }
            *reinterpret_cast<uint4*>(sV + row * LDS + c * 8) = pv;
            *reinterpret_cast<uint4*>(sVh + row * LDS + c * 8) = ph;
            *reinterpret_cast<uint4*>(sVl + row * LDS + c * 8) = pl;
        }
        __syncthreads();
        if (warp * 16 < rows) {
            const uint32_t q_addr = (uint32_t)__cvta_generic_to_shared(sQ + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDQ + (lane >> 4) * 8);
            const uint32_t k_addr = (uint32_t)__cvta_generic_to_shared(sK + ((lane & 7) + (lane >> 4) * 8) * LDQ + ((lane >> 3) & 1) * 8);
            const uint32_t b_off = (uint32_t)((((lane & 7) + ((lane >> 3) & 1) * 8) * LDS + (lane >> 4) * 8) * 2);
            const uint32_t sh_addr = (uint32_t)__cvta_generic_to_shared(sSh) + b_off, sl_addr = (uint32_t)__cvta_generic_to_shared(sSl) + b_off;
            const uint32_t v_addr = (uint32_t)__cvta_generic_to_shared(sV) + b_off;
            float s[CH / 8][4], acc[NT][4];
#pragma unroll
            for (int j = 0; j < CH / 8; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f; }
#pragma unroll
            for (int i = 0; i < NT; ++i) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.0f; }
#pragma unroll
            for (int kk = 0; kk < DQ / 16; ++kk) {
                uint32_t qa[4];
                ldsm_x4(q_addr + kk * 32, qa[0], qa[1], qa[2], qa[3]);
#pragma unroll
                for (int j = 0; j < CH / 8; j += 2) {              // q k^T
                    uint32_t b0, b1, b2, b3;
                    ldsm_x4(k_addr + (uint32_t)(j * 8 * LDQ * 2 + kk * 32), b0, b1, b2, b3);
                    mma_bf16_16816(s[j], qa, b0, b1);
                    mma_bf16_16816(s[j + 1], qa, b2, b3);
                }
#pragma unroll
                for (int dt = 0; dt < NT; dt += 2) {               // q S, S = high + low
                    uint32_t b0, b1, b2, b3;
                    ldsm_x4_trans(sh_addr + (uint32_t)(kk * 16 * LDS * 2 + dt * 16), b0, b1, b2, b3);
                    mma_bf16_16816(acc[dt], qa, b0, b1);
                    mma_bf16_16816(acc[dt + 1], qa, b2, b3);
                    ldsm_x4_trans(sl_addr + (uint32_t)(kk * 16 * LDS * 2 + dt * 16), b0, b1, b2, b3);
                    mma_bf16_16816(acc[dt], qa, b0, b1);
                    mma_bf16_16816(acc[dt + 1], qa, b2, b3);
                }
            }
            const int i0 = warp * 16 + g, i1 = i0 + 8;             // this thread's rows of the chunk
            const float f0 = pw[i0 + 1], f1 = pw[i1 + 1];
#pragma unroll
            for (int i = 0; i < NT; ++i) { acc[i][0] *= f0; acc[i][1] *= f0; acc[i][2] *= f1; acc[i][3] *= f1; }
#pragma unroll
            for (int ks = 0; ks < CH / 16; ++ks) {                 // (q k^T with decay and mask) v, the weights as high + low
                uint32_t ph[4], pl[4];
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const int j = ks * 16 + half * 8 + t2;
                    const float* sc = s[2 * ks + half];
                    const float w00 = j <= i0 ? sc[0] * pw[i0 - j] : 0.0f, w01 = j + 1 <= i0 ? sc[1] * pw[i0 - j - 1] : 0.0f;
                    const float w10 = j <= i1 ? sc[2] * pw[i1 - j] : 0.0f, w11 = j + 1 <= i1 ? sc[3] * pw[i1 - j - 1] : 0.0f;
                    split_bf16(w00, w01, ph[2 * half], pl[2 * half]);
                    split_bf16(w10, w11, ph[2 * half + 1], pl[2 * half + 1]);
                }
#pragma unroll
                for (int dt = 0; dt < NT; dt += 2) {
                    uint32_t b0, b1, b2, b3;
                    ldsm_x4_trans(v_addr + (uint32_t)(ks * 16 * LDS * 2 + dt * 16), b0, b1, b2, b3);
                    mma_bf16_16816(acc[dt], ph, b0, b1);
                    mma_bf16_16816(acc[dt + 1], ph, b2, b3);
                    mma_bf16_16816(acc[dt], pl, b0, b1);
                    mma_bf16_16816(acc[dt + 1], pl, b2, b3);
                }
            }
            float* dst = o + (size_t)(first + c0) * o_stride + (size_t)head * vdim + vs0;
#pragma unroll
            for (int i = 0; i < NT; ++i) {
                if (i0 < rows) *reinterpret_cast<float2*>(dst + (size_t)i0 * o_stride + i * 8 + t2) = make_float2(acc[i][0], acc[i][1]);
                if (i1 < rows) *reinterpret_cast<float2*>(dst + (size_t)i1 * o_stride + i * 8 + t2) = make_float2(acc[i][2], acc[i][3]);
            }
        }
        // the state: S <- lam^rows S + k^T (decayed v)
        const float fs = pw[rows];
        const uint32_t vh_addr = (uint32_t)__cvta_generic_to_shared(sVh + ((lane & 7) + ((lane >> 3) & 1) * 8) * LDS + (lane >> 4) * 8);
        const uint32_t vl_addr = (uint32_t)__cvta_generic_to_shared(sVl + ((lane & 7) + ((lane >> 3) & 1) * 8) * LDS + (lane >> 4) * 8);
#pragma unroll
        for (int mi = 0; mi < MT_W; ++mi) {
            const int m0 = (warp + 4 * mi) * 16;
            if (m0 < DQ) {
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) { S[mi][nt][0] *= fs; S[mi][nt][1] *= fs; S[mi][nt][2] *= fs; S[mi][nt][3] *= fs; }
                // k^T as the row operand: tokens are its columns, read transposed from the [token][channel] tile
                const uint32_t a_addr = (uint32_t)__cvta_generic_to_shared(sK + ((lane & 7) + (lane >> 4) * 8) * LDQ + m0 + ((lane >> 3) & 1) * 8);
#pragma unroll
                for (int ks = 0; ks < CH / 16; ++ks) {
                    uint32_t ka[4];
                    ldsm_x4_trans(a_addr + (uint32_t)(ks * 16 * LDQ * 2), ka[0], ka[1], ka[2], ka[3]);
#pragma unroll
                    for (int dt = 0; dt < NT; dt += 2) {
                        uint32_t b0, b1, b2, b3;
                        ldsm_x4_trans(vh_addr + (uint32_t)(ks * 16 * LDS * 2 + dt * 16), b0, b1, b2, b3);
                        mma_bf16_16816(S[mi][dt], ka, b0, b1);
                        mma_bf16_16816(S[mi][dt + 1], ka, b2, b3);
                        ldsm_x4_trans(vl_addr + (uint32_t)(ks * 16 * LDS * 2 + dt * 16), b0, b1, b2, b3);
                        mma_bf16_16816(S[mi][dt], ka, b0, b1);
                        mma_bf16_16816(S[mi][dt + 1], ka, b2, b3);
                    }
                }
            }
        }
    }
#pragma unroll
    for (int mi = 0; mi < MT_W; ++mi) {
        const int m0 = (warp + 4 * mi) * 16;
        if (m0 < DQ) {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                *reinterpret_cast<float2*>(st + (size_t)(m0 + g) * vdim + nt * 8 + t2) = make_float2(S[mi][nt][0], S[mi][nt][1]);
                *reinterpret_cast<float2*>(st + (size_t)(m0 + g + 8) * vdim + nt * 8 + t2) = make_float2(S[mi][nt][2], S[mi][nt][3]);
            }
        }
    }
}

MB_API int mb_linear_attention_chunked_layout(int* dq, int* vs) { *dq = DQ; *vs = VS; return 0; }

// q, k: bf16 [T, heads * QK_DIM], v: bf16 [T, heads * vdim], slices of one projection (common row stride, 16-byte
// aligned rows); vdim a multiple of V_SLICE; o: float32 [T, heads * vdim]; state: float32 [slot][head][QK_DIM][vdim].
MB_API int mb_linear_attention_chunked(const void* q, const void* k, const void* v, int row_stride, const float* decay, float* state,
                                       const int* cu_tokens, const int* state_slots, float* o, int requests, int heads, int vdim,
                                       cudaStream_t s) {
    if (requests <= 0) return 0;
    if (heads <= 0 || vdim <= 0 || vdim % VS != 0 || row_stride % 8 != 0) return MB_ERR_BAD_SIZE;
    if ((((uintptr_t)q | (uintptr_t)k | (uintptr_t)v) & 15) != 0) return MB_ERR_BAD_SIZE;
    cudaFuncSetAttribute(linear_attention_chunked_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, LC_SMEM);
    return launch_kernel(linear_attention_chunked_kernel, dim3(requests, heads, vdim / VS), 128, LC_SMEM, s, 0, (const bf16*)q, (const bf16*)k,
                         (const bf16*)v, row_stride, decay, state, cu_tokens, state_slots, o, heads, vdim);
}
