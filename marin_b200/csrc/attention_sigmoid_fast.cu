// bf16 attention with sigmoid weights on the tensor cores (mma.sync), compiled for one head layout:
//   -DHEAD_DIM (keys and queries), -DV_DIM (values), -DGROUP (query heads per kv head); both sizes multiples of 16 up to 128.
//   weight(i, j) = sigmoid(q_i . k_j * scale + bias[head][min(i - j, span - 1)]),   out_i = sum_{j <= i} weight(i, j) v_j
// There is no softmax, so nothing is rescaled and nothing is divided at the end, and partial sums over any split of the
// keys simply add: single tokens split their keys over CTAs and a second kernel adds the parts in a fixed order.
// Scores and weights are float32; the weights are rounded to bf16 for the product with V, like a softmax's.
// Prompt portions: 64 queries x 64-key blocks per CTA (the layout of attn_prefill_kernel in attention_fast.cu).
// K pages [page][kv_head][offset][HEAD_DIM], V pages [page][kv_head][offset][V_DIM].
#define MB_LIB "attention_sigmoid_fast"
#define MB_LIB_ID 11
#include "common.cuh"
#include "launch.cuh"
#include "mma_helpers.cuh"

#ifndef HEAD_DIM
#define HEAD_DIM 128
#endif
#ifndef V_DIM
#define V_DIM HEAD_DIM
#endif
#ifndef GROUP
#define GROUP 4
#endif
static_assert(HEAD_DIM % 16 == 0 && HEAD_DIM >= 16 && HEAD_DIM <= 128, "key heads: a multiple of 16 up to 128");
static_assert(V_DIM % 16 == 0 && V_DIM >= 16 && V_DIM <= 128, "value heads: a multiple of 16 up to 128");
static_assert(GROUP >= 1 && GROUP <= 8, "1 to 8 query heads per kv head");

#define D HEAD_DIM
#define DV V_DIM
#define LDK (D + 8)                   // padded rows in shared memory (elements): ldmatrix without bank conflicts
#define LDV (DV + 8)
#define BM 64
#define BN 64

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// 1 / (1 + 2^(-s log2 e)): two special-function operations per score; a score far below zero gives 1 / inf = 0.
__device__ __forceinline__ float sigmoid_fast(float s) { return __fdividef(1.0f, 1.0f + ex2_approx(s * -1.4426950408889634f)); }

// The rows of one 64-key block of K and V (cp.async); keys past `k_last` are zero (their pages may not exist).
__device__ __forceinline__ void load_kv_block(bf16* dst_k, bf16* dst_v, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                                              const int* __restrict__ table, int K, int kh, int page_shift, int key0, int k_last) {
    constexpr int CK = D / 8, CV = DV / 8;
    const int page_mask = (1 << page_shift) - 1;
    for (int idx = threadIdx.x; idx < BN * (CK + CV); idx += 128) {
        const int row = idx / (CK + CV), c = idx % (CK + CV);
        const int key = key0 + row;
        const bool is_k = c < CK;
        bf16* dst = is_k ? dst_k + row * LDK + c * 8 : dst_v + row * LDV + (c - CK) * 8;
        if (key <= k_last) {
            const size_t slot = (((size_t)table[key >> page_shift] * K + kh) << page_shift) + (size_t)(key & page_mask);
            cp_async16(dst, is_k ? k_cache + slot * D + c * 8 : v_cache + slot * DV + (c - CK) * 8);
        } else {
            *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
        }
    }
}

#define PF_SMEM ((BM * LDK + BN * LDK + BN * LDV) * 2)

__global__ void __launch_bounds__(128, 2) attn_sigmoid_prefill_kernel(
    const bf16* __restrict__ q, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache, bf16* __restrict__ out,
    const int* __restrict__ block_table, int max_pages, const int* __restrict__ cu_tokens, const int* __restrict__ seq_lens,
    int first_req, int K, int page_shift, float scale, const float* __restrict__ bias, int span) {
    PDL_ENTER_EARLY();
    q = pdl_fresh(q); k_cache = pdl_fresh(k_cache); v_cache = pdl_fresh(v_cache);
    extern __shared__ __align__(16) uint8_t smem_raw[];
    bf16* sQ = reinterpret_cast<bf16*>(smem_raw);
    bf16* sK = sQ + BM * LDK;
    bf16* sV = sK + BN * LDK;
    const int H = K * GROUP;
    const int r = first_req + blockIdx.z, h = blockIdx.y, qt = gridDim.x - 1 - blockIdx.x;   // long tiles first
    const int tok0 = cu_tokens[r], n = cu_tokens[r + 1] - tok0;
    if (qt * BM >= n) return;
    const int len = seq_lens[r], pos0 = len - n;
    const int rows = min(BM, n - qt * BM);
    const int q_first = pos0 + qt * BM, q_last = q_first + rows - 1;
    const int kh = h / GROUP;
    const int* table = block_table + (size_t)r * max_pages;
    const float* brow = bias + (size_t)h * span;
    const float b_far = brow[span - 1];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kb_last = q_last / BN;
    {
        constexpr int CHUNKS = D / 8;
        for (int idx = threadIdx.x; idx < BM * CHUNKS; idx += 128) {
            const int row = idx / CHUNKS, c = idx % CHUNKS;
            bf16* d = sQ + row * LDK + c * 8;
            if (row < rows) cp_async16(d, q + ((size_t)(tok0 + qt * BM + row) * H + h) * D + c * 8);
            else *reinterpret_cast<uint4*>(d) = make_uint4(0, 0, 0, 0);
        }
        load_kv_block(sK, sV, k_cache, v_cache, table, K, kh, page_shift, 0, q_last);
        cp_async_commit();
    }
    cp_async_wait<0>();
    __syncthreads();
    const uint32_t q_addr = (uint32_t)__cvta_generic_to_shared(sQ + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDK + (lane >> 4) * 8);
    float o[DV / 8][4];
#pragma unroll
    for (int i = 0; i < DV / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
    const int row0 = warp * 16 + (lane >> 2);                 // this thread's rows: row0 and row0 + 8
    const int qp0 = q_first + row0, qp1 = qp0 + 8;

    for (int kb = 0; kb <= kb_last; ++kb) {
        const int key0 = kb * BN;
        if (kb > 0) {                                          // the barrier at the end of the last block freed the buffers
            load_kv_block(sK, sV, k_cache, v_cache, table, K, kh, page_shift, key0, q_last);
            cp_async_commit();
            cp_async_wait<0>();
            __syncthreads();
        }
        float s[BN / 8][4];
#pragma unroll
        for (int j = 0; j < BN / 8; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f; }
        const uint32_t k_addr = (uint32_t)__cvta_generic_to_shared(sK + ((lane & 7) + (lane >> 4) * 8) * LDK + ((lane >> 3) & 1) * 8);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
            uint32_t qa[4];
            ldsm_x4(q_addr + kk * 32, qa[0], qa[1], qa[2], qa[3]);
#pragma unroll
            for (int j = 0; j < BN / 8; j += 2) {
                uint32_t b0, b1, b2, b3;
                ldsm_x4(k_addr + (uint32_t)(j * 8 * LDK * 2 + kk * 32), b0, b1, b2, b3);
                mma_bf16_16816(s[j], qa, b0, b1);
                mma_bf16_16816(s[j + 1], qa, b2, b3);
            }
        }
        // weights.  A block all of whose distances lie at or beyond the table's end takes the table's last entry; a block
        // that ends at or before the tile's first query needs no mask.
        const bool far = q_first - (key0 + BN - 1) >= span - 1;
        const bool interior = key0 + BN - 1 <= q_first;
        if (far) {
#pragma unroll
            for (int j = 0; j < BN / 8; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) s[j][e] = sigmoid_fast(fmaf(s[j][e], scale, b_far));
            }
        } else {
#pragma unroll
            for (int j = 0; j < BN / 8; ++j) {
                const int key = key0 + j * 8 + 2 * (lane & 3);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int dist = ((e & 2) ? qp1 : qp0) - (key + (e & 1));
                    const float w = sigmoid_fast(fmaf(s[j][e], scale, brow[min(max(dist, 0), span - 1)]));
                    s[j][e] = (interior || dist >= 0) ? w : 0.0f;
                }
            }
        }
        // O += P V
        const uint32_t v_addr = (uint32_t)__cvta_generic_to_shared(sV + ((lane & 7) + ((lane >> 3) & 1) * 8) * LDV + (lane >> 4) * 8);
#pragma unroll
        for (int ks = 0; ks < BN / 16; ++ks) {
            uint32_t pa[4];
            pa[0] = pack_bf16(s[2 * ks][0], s[2 * ks][1]);
            pa[1] = pack_bf16(s[2 * ks][2], s[2 * ks][3]);
            pa[2] = pack_bf16(s[2 * ks + 1][0], s[2 * ks + 1][1]);
            pa[3] = pack_bf16(s[2 * ks + 1][2], s[2 * ks + 1][3]);
#pragma unroll
            for (int dt = 0; dt < DV / 8; dt += 2) {
                uint32_t b0, b1, b2, b3;
                ldsm_x4_trans(v_addr + (uint32_t)(ks * 16 * LDV * 2 + dt * 16), b0, b1, b2, b3);
                mma_bf16_16816(o[dt], pa, b0, b1);
                mma_bf16_16816(o[dt + 1], pa, b2, b3);
            }
        }
        __syncthreads();                                       // everyone is done with this block's buffers
    }
    const int col = 2 * (lane & 3);
    if (row0 < rows) {
        bf16* dst = out + ((size_t)(tok0 + qt * BM + row0) * H + h) * DV;
#pragma unroll
        for (int i = 0; i < DV / 8; ++i) *reinterpret_cast<uint32_t*>(dst + i * 8 + col) = pack_bf16(o[i][0], o[i][1]);
    }
    if (row0 + 8 < rows) {
        bf16* dst = out + ((size_t)(tok0 + qt * BM + row0 + 8) * H + h) * DV;
#pragma unroll
        for (int i = 0; i < DV / 8; ++i) *reinterpret_cast<uint32_t*>(dst + i * 8 + col) = pack_bf16(o[i][2], o[i][3]);
    }
}

// ---- single tokens: the keys of a sequence split over CTAs --------------------------------------------------------------
// CTA (chunk, kv head, request): keys [chunk * split, +split) of the request, in 64-key blocks; the GROUP query heads of the kv
// head are rows 0..GROUP-1 of a 16-row tile; warp w takes keys 16 w .. 16 w + 15 of every block.  The four warps' sums
// are added in shared memory in warp order and written as the chunk's part: part[chunk][request][head][DV], float32.
#define DEC_SMEM ((16 * LDK + BN * LDK + BN * LDV) * 2)
static_assert(4 * GROUP * DV * 4 <= BN * LDK * 2 + BN * LDV * 2, "the warps' sums are written over the key and value block");

__global__ void __launch_bounds__(128) attn_sigmoid_decode_kernel(
    const bf16* __restrict__ q, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache, float* __restrict__ part,
    const int* __restrict__ block_table, int max_pages, const int* __restrict__ seq_lens, int K, int page_shift, float scale,
    const float* __restrict__ bias, int span, int split) {
    PDL_ENTER();
    q = pdl_fresh(q); k_cache = pdl_fresh(k_cache); v_cache = pdl_fresh(v_cache);
    extern __shared__ __align__(16) uint8_t smem_raw[];
    bf16* sQ = reinterpret_cast<bf16*>(smem_raw);
    bf16* sK = sQ + 16 * LDK;
    bf16* sV = sK + BN * LDK;
    const int chunk = blockIdx.x, kh = blockIdx.y, r = blockIdx.z, R = gridDim.z;
    const int H = K * GROUP;
    const int len = seq_lens[r], pos = len - 1;
    const int c_begin = chunk * split, c_end = min(len, c_begin + split);
    if (c_begin >= len) return;
    const int* table = block_table + (size_t)r * max_pages;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    {
        constexpr int CHUNKS = D / 8;
        for (int idx = threadIdx.x; idx < 16 * CHUNKS; idx += 128) {
            const int row = idx / CHUNKS, c = idx % CHUNKS;
            bf16* d = sQ + row * LDK + c * 8;
            if (row < GROUP) cp_async16(d, q + ((size_t)r * H + kh * GROUP + row) * D + c * 8);
            else *reinterpret_cast<uint4*>(d) = make_uint4(0, 0, 0, 0);
        }
    }
    const uint32_t q_addr = (uint32_t)__cvta_generic_to_shared(sQ + ((lane & 7) + ((lane >> 3) & 1) * 8) * LDK + (lane >> 4) * 8);
    float o[DV / 8][4];
#pragma unroll
    for (int i = 0; i < DV / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
    const int g = lane >> 2;                                   // this thread's row of the tile: a query head if g < GROUP
    const float* brow = bias + (size_t)(kh * GROUP + (g < GROUP ? g : 0)) * span;
    for (int key0 = c_begin; key0 < c_end; key0 += BN) {
        load_kv_block(sK, sV, k_cache, v_cache, table, K, kh, page_shift, key0, pos);
        cp_async_commit();
        cp_async_wait<0>();
        __syncthreads();
        float s[2][4];
        s[0][0] = s[0][1] = s[0][2] = s[0][3] = s[1][0] = s[1][1] = s[1][2] = s[1][3] = 0.0f;
        const uint32_t k_addr = (uint32_t)__cvta_generic_to_shared(sK + (warp * 16 + (lane & 7) + (lane >> 4) * 8) * LDK + ((lane >> 3) & 1) * 8);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
            uint32_t qa[4], b0, b1, b2, b3;
            ldsm_x4(q_addr + kk * 32, qa[0], qa[1], qa[2], qa[3]);
            ldsm_x4(k_addr + (uint32_t)(kk * 32), b0, b1, b2, b3);
            mma_bf16_16816(s[0], qa, b0, b1);
            mma_bf16_16816(s[1], qa, b2, b3);
        }
#pragma unroll
        for (int j = 0; j < 2; ++j) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {                      // elements 2 and 3 belong to rows 8..15: no query head
                const int key = key0 + warp * 16 + j * 8 + 2 * (lane & 3) + e;
                const int dist = pos - key;
                const float w = sigmoid_fast(fmaf(s[j][e], scale, brow[min(max(dist, 0), span - 1)]));
                s[j][e] = (g < GROUP && dist >= 0) ? w : 0.0f;
            }
            s[j][2] = s[j][3] = 0.0f;
        }
        uint32_t pa[4];
        pa[0] = pack_bf16(s[0][0], s[0][1]);
        pa[1] = pack_bf16(s[0][2], s[0][3]);
        pa[2] = pack_bf16(s[1][0], s[1][1]);
        pa[3] = pack_bf16(s[1][2], s[1][3]);
        const uint32_t v_addr = (uint32_t)__cvta_generic_to_shared(sV + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDV + (lane >> 4) * 8);
#pragma unroll
        for (int dt = 0; dt < DV / 8; dt += 2) {
            uint32_t b0, b1, b2, b3;
            ldsm_x4_trans(v_addr + (uint32_t)(dt * 16), b0, b1, b2, b3);
            mma_bf16_16816(o[dt], pa, b0, b1);
            mma_bf16_16816(o[dt + 1], pa, b2, b3);
        }
        __syncthreads();
    }
    float* sums = reinterpret_cast<float*>(sK);               // [4 warps][GROUP][DV]
    if (g < GROUP) {
        const int col = 2 * (lane & 3);
#pragma unroll
        for (int i = 0; i < DV / 8; ++i) {
            sums[(warp * GROUP + g) * DV + i * 8 + col] = o[i][0];
            sums[(warp * GROUP + g) * DV + i * 8 + col + 1] = o[i][1];
        }
    }
    __syncthreads();
    float* dst = part + (((size_t)chunk * R + r) * H + (size_t)kh * GROUP) * DV;
    for (int idx = threadIdx.x; idx < GROUP * DV; idx += 128)
        dst[idx] = ((sums[idx] + sums[GROUP * DV + idx]) + sums[2 * GROUP * DV + idx]) + sums[3 * GROUP * DV + idx];
}

// out[r][h][:] = sum over the request's chunks, in chunk order, of part[chunk][r][h][:]
__global__ void attn_sigmoid_merge_kernel(const float* __restrict__ part, const int* __restrict__ seq_lens, int split, int R, int H,
                                          bf16* __restrict__ out) {
    PDL_ENTER();
    part = pdl_fresh(part);
    const int r = blockIdx.x / H, h = blockIdx.x % H;
    const int chunks = (seq_lens[r] + split - 1) / split;
    for (int i = threadIdx.x; i < DV; i += blockDim.x) {
        float a = 0.0f;
        int c = 0;
        for (; c + 8 <= chunks; c += 8) {                      // eight loads in flight, added in chunk order
            float x[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) x[u] = part[(((size_t)(c + u) * R + r) * H + h) * DV + i];
#pragma unroll
            for (int u = 0; u < 8; ++u) a += x[u];
        }
        for (; c < chunks; ++c) a += part[(((size_t)c * R + r) * H + h) * DV + i];
        out[((size_t)r * H + h) * DV + i] = __float2bfloat16_rn(a);
    }
}

static int page_shift_of(int page_size) {
    int s = 0;
    while ((1 << s) < page_size) ++s;
    return (1 << s) == page_size ? s : -1;
}

MB_API int mb_attn_sigmoid_layout(int* d, int* dv, int* group) { *d = D; *dv = DV; *group = GROUP; return 0; }

// Single tokens: requests 0 .. requests - 1 bring one token each (token t belongs to request t).  part: float32
// [chunks][requests][K * GROUP][V_DIM]; split: keys per chunk, a multiple of 64; chunks * split covers the longest sequence.
MB_API int mb_attn_sigmoid_decode(const void* q, const void* k_cache, const void* v_cache, float* part, const int* block_table,
                                  int max_pages, const int* seq_lens, int requests, int K, int page_size, float scale,
                                  const float* bias, int span, int split, int chunks, cudaStream_t s) {
    if (requests <= 0) return 0;
    const int shift = page_shift_of(page_size);
    if (shift < 0 || split <= 0 || split % BN != 0 || chunks <= 0 || span <= 0) return MB_ERR_BAD_SIZE;
    cudaFuncSetAttribute(attn_sigmoid_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DEC_SMEM);
    return launch_kernel(attn_sigmoid_decode_kernel, dim3(chunks, K, requests), 128, DEC_SMEM, s, 0, (const bf16*)q, (const bf16*)k_cache,
                         (const bf16*)v_cache, part, block_table, max_pages, seq_lens, K, shift, scale, bias, span, split);
}

// The parts of every request added in chunk order: out bf16 [requests][K * GROUP][V_DIM].
MB_API int mb_attn_sigmoid_merge(const float* part, void* out, const int* seq_lens, int requests, int K, int split, cudaStream_t s) {
    if (requests <= 0) return 0;
    if (split <= 0) return MB_ERR_BAD_SIZE;
    return launch_kernel(attn_sigmoid_merge_kernel, requests * K * GROUP, DV >= 64 ? 64 : 32, 0, s, 0, part, seq_lens, split, requests,
                         K * GROUP, (bf16*)out);
}

// Prompt portions: requests first_req .. first_req + count - 1 of the step.
MB_API int mb_attn_sigmoid_prefill(const void* q, const void* k_cache, const void* v_cache, void* out, const int* block_table,
                                   int max_pages, const int* cu_tokens, const int* seq_lens, int first_req, int count,
                                   int max_query_len, int K, int page_size, float scale, const float* bias, int span, cudaStream_t s) {
    if (count <= 0 || max_query_len <= 0) return 0;
    const int shift = page_shift_of(page_size);
    if (shift < 0 || span <= 0) return MB_ERR_BAD_SIZE;
    cudaFuncSetAttribute(attn_sigmoid_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PF_SMEM);
    dim3 grid((max_query_len + BM - 1) / BM, K * GROUP, count);
    return launch_kernel(attn_sigmoid_prefill_kernel, grid, 128, PF_SMEM, s, 0, (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache,
                         (bf16*)out, block_table, max_pages, cu_tokens, seq_lens, first_req, K, shift, scale, bias, span);
}
