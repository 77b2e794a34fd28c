// Hyper-connections: the residual is kept as S streams x_1 .. x_S (float32 [S][tokens][h]) instead of one.  Around a
// sublayer with learned numbers in[S], out[S] and mix[S][S] (indexed [from][to]):
//     u = sum_s in[s] x_s                  what the sublayer's norm reads
//     x_t <- sum_s mix[s][t] x_s + out[t] y     all streams at once from the old ones, y the sublayer's output
// One kernel does the write of one sublayer and the read (with its RMS norm) of the next, a token per block: the streams
// are read once and written once per sublayer.  Either half may be absent (the first read of a model, the last write).
// Every sum runs in float32 in a fixed order (streams in increasing order), whatever else the batch holds.
#define MB_LIB "hyper"
#define MB_LIB_ID 12
#include "common.cuh"
#include "launch.cuh"

#define HC_MAX_STREAMS 8
#define HC_THREADS 256
#define HC_MAX_THREADS 1024        // few tokens: a row is spread over more threads, the loads of a row are all in flight at once

// mix, w_out, y null: no write.  w_in null: no read (norm_w, out unused).  y (float32 [tokens][h]) is zeroed after it
// was read, so that the next sublayer can add its output into it.
template <typename TO, int S>
__global__ void __launch_bounds__(HC_MAX_THREADS) hc_step_kernel(float* __restrict__ streams, int tokens, int h,
                                                             const float* __restrict__ mix, const float* __restrict__ w_out,
                                                             float* __restrict__ y, const float* __restrict__ w_in,
                                                             const float* __restrict__ norm_w, float eps, int unit_offset,
                                                             TO* __restrict__ out) {
    PDL_ENTER();
    streams = pdl_fresh(streams); y = pdl_fresh(y);
    extern __shared__ float u_row[];                  // [h], only with a read
    __shared__ float scratch[32];
    __shared__ float c_mix[S * S], c_out[S], c_in[S];
    if (threadIdx.x < S * S && mix != nullptr) c_mix[threadIdx.x] = mix[threadIdx.x];
    if (threadIdx.x < S) {
        if (w_out != nullptr) c_out[threadIdx.x] = w_out[threadIdx.x];
        if (w_in != nullptr) c_in[threadIdx.x] = w_in[threadIdx.x];
    }
    __syncthreads();
    const size_t t = blockIdx.x;
    const size_t plane = (size_t)tokens * h;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < h; i += blockDim.x) {
        float x[S];
#pragma unroll
        for (int s = 0; s < S; ++s) x[s] = streams[s * plane + t * h + i];
        if (mix != nullptr) {
            const float yy = y[t * h + i];
            float nx[S];
#pragma unroll
            for (int to = 0; to < S; ++to) {
                float a = 0.0f;
#pragma unroll
                for (int s = 0; s < S; ++s) a = fmaf(c_mix[s * S + to], x[s], a);
                nx[to] = fmaf(c_out[to], yy, a);
            }
#pragma unroll
            for (int s = 0; s < S; ++s) { x[s] = nx[s]; streams[s * plane + t * h + i] = nx[s]; }
        }
        if (y != nullptr) y[t * h + i] = 0.0f;
        if (w_in != nullptr) {
            float u = 0.0f;
#pragma unroll
            for (int s = 0; s < S; ++s) u = fmaf(c_in[s], x[s], u);
            u_row[i] = u;
            ss += u * u;
        }
    }
    if (w_in == nullptr) return;
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)h + eps);
    for (int i = threadIdx.x; i < h; i += blockDim.x) {
        const float wi = unit_offset ? 1.0f + norm_w[i] : norm_w[i];
        out[t * h + i] = from_f32<TO>(u_row[i] * scale * wi);
    }
}

template <typename TO, int S>
static int hc_launch(float* streams, int tokens, int h, const float* mix, const float* w_out, float* y, const float* w_in,
                     const float* norm_w, float eps, int unit_offset, void* out, cudaStream_t s) {
    const size_t smem = w_in != nullptr ? (size_t)h * sizeof(float) : 0;
    if (smem > 48 * 1024) {
        const int rc = (int)cudaFuncSetAttribute(hc_step_kernel<TO, S>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (rc != 0) return rc;
    }
    int threads = HC_THREADS;
    // (only where rows leave as bf16: in true float32 a row's sum of squares is added in the same order whatever the batch holds)
    if (tokens <= 64 && sizeof(TO) == 2) while (threads < HC_MAX_THREADS && threads * 2 <= h) threads *= 2;
    return launch_kernel(hc_step_kernel<TO, S>, tokens, threads, smem, s, 0, streams, tokens, h, mix, w_out, y, w_in, norm_w, eps,
                         unit_offset, (TO*)out);
}

template <typename TO>
static int hc_by_streams(int S, float* streams, int tokens, int h, const float* mix, const float* w_out, float* y, const float* w_in,
                         const float* norm_w, float eps, int unit_offset, void* out, cudaStream_t s) {
    switch (S) {
#define HC_CASE(n) case n: return hc_launch<TO, n>(streams, tokens, h, mix, w_out, y, w_in, norm_w, eps, unit_offset, out, s);
        HC_CASE(1) HC_CASE(2) HC_CASE(3) HC_CASE(4) HC_CASE(5) HC_CASE(6) HC_CASE(7) HC_CASE(8)
#undef HC_CASE
    }
    return MB_ERR_BAD_SIZE;
}

MB_API int mb_hc_step(float* streams, int S, int tokens, int h, const float* mix, const float* w_out, float* y, const float* w_in,
                      const float* norm_w, float eps, int unit_offset, void* out, int out_dtype, cudaStream_t s) {
    if (tokens <= 0) return 0;
    if (S < 1 || S > HC_MAX_STREAMS || h <= 0 || (size_t)h * sizeof(float) > 200 * 1024) return MB_ERR_BAD_SIZE;
    if ((mix == nullptr) != (w_out == nullptr) || (mix != nullptr && y == nullptr)) return MB_ERR_BAD_SIZE;
    if (w_in == nullptr || out_dtype == MB_F32)
        return hc_by_streams<float>(S, streams, tokens, h, mix, w_out, y, w_in, norm_w, eps, unit_offset, out, s);
    if (out_dtype == MB_BF16)
        return hc_by_streams<bf16>(S, streams, tokens, h, mix, w_out, y, w_in, norm_w, eps, unit_offset, out, s);
    return MB_ERR_BAD_DTYPE;
}

// ---- stream 0 copied to the others (all streams start as the embedding's output) -----------------------------------
__global__ void hc_spread_kernel(float* __restrict__ streams, int S, size_t plane) {
    PDL_ENTER();
    streams = pdl_fresh(streams);
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; idx < plane; idx += stride) {
        const float v = streams[idx];
        for (int s = 1; s < S; ++s) streams[s * plane + idx] = v;
    }
}

MB_API int mb_hc_spread(float* streams, int S, int tokens, int h, cudaStream_t s) {
    const size_t plane = (size_t)tokens * h;
    if (plane == 0 || S <= 1) return 0;
    const size_t want = (plane + 255) / 256;
    return launch_kernel(hc_spread_kernel, (int)(want < 148 * 16 ? want : 148 * 16), 256, 0, s, 0, streams, S, plane);
}

// ---- out[r] = sum_s streams[s][rows[r]] (rows null: every token in order): the one residual stream the head reads ----
__global__ void hc_sum_kernel(const float* __restrict__ streams, int S, size_t plane, const int* __restrict__ rows,
                              float* __restrict__ out, int h) {
    PDL_ENTER();
    streams = pdl_fresh(streams);
    const size_t row = rows != nullptr ? (size_t)rows[blockIdx.x] : (size_t)blockIdx.x;
    for (int i = threadIdx.x; i < h; i += blockDim.x) {
        float a = streams[row * h + i];
        for (int s = 1; s < S; ++s) a += streams[s * plane + row * h + i];
        out[(size_t)blockIdx.x * h + i] = a;
    }
}

MB_API int mb_hc_sum(const float* streams, int S, int tokens, int h, const int* rows, float* out, int count, cudaStream_t s) {
    if (count <= 0) return 0;
    if (S < 1 || h <= 0) return MB_ERR_BAD_SIZE;
    return launch_kernel(hc_sum_kernel, count, 256, 0, s, 0, streams, S, (size_t)tokens * h, rows, out, h);
}
