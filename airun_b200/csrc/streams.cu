// A residual made of several streams (hyper-connections): instead of one x a token carries S copies x_1..x_S, all
// equal to the embedding at the start.  A sub-layer f with the numbers a[S] (read), M[S][S] (carry, indexed
// [from][to]) and b[S] (write) and the model's factor m does
//
//     u = sum_s a[s] x_s,    y = f(norm(u)),    x_t <- sum_s M[s][t] x_s + m * b[t] * (y + y_bias)    all t at once.
//
// One kernel does the write of the sub-layer before and the read (with its root-mean-square norm) of the sub-layer
// after: a block per token reads the token's S*H numbers once, forms the new streams, stores them, and norms their
// weighted sum.  Either half can be left out: without y it only reads (the first sub-layer of a model), without a norm
// weight the weighted sum itself is stored in float32 (the end of the model: a = 1 gives the sum of the streams).
// Everything is float32; only the normed output takes the type of the products that read it.
//
// xs is [T][S][H].  Rows of request -1 are padding and are skipped.
#include "common.cuh"

#define STREAMS_MAX 8

template <typename TOut>
__global__ __launch_bounds__(256) void stream_step_kernel(
    float* __restrict__ xs, int S, int H, const float* __restrict__ y, long long y_stride, const float* __restrict__ y_bias,
    const float* __restrict__ carry, const float* __restrict__ write, float mult, const float* __restrict__ read,
    const float* __restrict__ norm_w, float eps, TOut* __restrict__ out, long long out_stride,
    const int32_t* __restrict__ req_of_token) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float s_u[];                 // [H]: the weighted sum, kept between the two passes of the norm
    __shared__ float s_m[STREAMS_MAX * STREAMS_MAX], s_b[STREAMS_MAX], s_a[STREAMS_MAX], red[33];
    const int t = blockIdx.x;
    if (req_of_token && req_of_token[t] < 0) return;
    if (threadIdx.x < S * S) s_m[threadIdx.x] = y ? carry[threadIdx.x] : 0.0f;
    if (threadIdx.x < S) {
        s_b[threadIdx.x] = y ? write[threadIdx.x] * mult : 0.0f;
        s_a[threadIdx.x] = read ? read[threadIdx.x] : 0.0f;
    }
    __syncthreads();
    float* row = xs + (size_t)t * S * H;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float x[STREAMS_MAX];
#pragma unroll
        for (int s = 0; s < STREAMS_MAX; ++s) x[s] = s < S ? row[(size_t)s * H + c] : 0.0f;
        if (y) {
            const float yv = y[(size_t)t * y_stride + c] + (y_bias ? y_bias[c] : 0.0f);
            float nx[STREAMS_MAX];
#pragma unroll
            for (int to = 0; to < STREAMS_MAX; ++to) {
                float acc = 0.0f;
#pragma unroll
                for (int from = 0; from < STREAMS_MAX; ++from)
                    if (from < S && to < S) acc = fmaf(s_m[from * S + to], x[from], acc);
                nx[to] = to < S ? fmaf(s_b[to], yv, acc) : 0.0f;
            }
#pragma unroll
            for (int s = 0; s < STREAMS_MAX; ++s) {
                x[s] = nx[s];
                if (s < S) row[(size_t)s * H + c] = nx[s];
            }
        }
        if (read) {
            float u = 0.0f;
#pragma unroll
            for (int s = 0; s < STREAMS_MAX; ++s)
                if (s < S) u = fmaf(s_a[s], x[s], u);
            s_u[c] = u;
            ss = fmaf(u, u, ss);
        }
    }
    if (!read) return;
    if (!norm_w) {
        for (int c = threadIdx.x; c < H; c += blockDim.x) out[(size_t)t * out_stride + c] = from_f32<TOut>(s_u[c]);
        return;
    }
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
    for (int c = threadIdx.x; c < H; c += blockDim.x) out[(size_t)t * out_stride + c] = from_f32<TOut>(s_u[c] * inv * norm_w[c]);
}

// xs[t][s] = x[t] for every stream s.
__global__ void stream_fill_kernel(const float* __restrict__ x, float* __restrict__ xs, long long total, int S, int H) {
    pdl_trigger();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long t = i / H;
    const int c = (int)(i - t * H);
    const float v = x[i];
    for (int s = 0; s < S; ++s) xs[((size_t)t * S + s) * H + c] = v;
}

AIRUN_EXPORT int airun_stream_fill(const float* x, float* xs, int T, int S, int H, cudaStream_t stream) {
    if (T < 0 || S <= 0 || H <= 0 || !x || !xs) return AIRUN_ERR_ARG;
    const long long total = (long long)T * H;
    if (total == 0) return AIRUN_OK;
    airun_launch(stream_fill_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, x, xs, total, S, H);
    return airun_launch_status();
}

AIRUN_EXPORT int airun_stream_step(float* xs, int T, int S, int H, const float* y, long long y_stride, const float* y_bias,
                                   const float* carry, const float* write, float mult, const float* read,
                                   const float* norm_w, float eps, void* out, int out_dtype, long long out_stride,
                                   const int32_t* req_of_token, cudaStream_t stream) {
    if (T < 0 || S <= 0 || S > STREAMS_MAX || H <= 0 || !xs || (y && (!carry || !write || y_stride < H)) ||
        (read && (!out || out_stride < H)) || (!y && !read))
        return AIRUN_ERR_ARG;
    if (T == 0) return AIRUN_OK;
    const size_t smem = (size_t)H * sizeof(float);
    if (smem > 200 * 1024) return AIRUN_ERR_ARG;
    static unsigned long long cfg_f = 0, cfg_b = 0;
    if (out_dtype == AIRUN_DT_BF16 && read && norm_w) {
        if (smem > 48 * 1024 && first_on_device(cfg_b))
            cudaFuncSetAttribute(stream_step_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        airun_launch(stream_step_kernel<__nv_bfloat16>, dim3(T), dim3(256), smem, stream, xs, S, H, y, y_stride, y_bias, carry, write,
                     mult, read, norm_w, eps, (__nv_bfloat16*)out, out_stride, req_of_token);
    } else if (out_dtype == AIRUN_DT_F32 || !read) {
        if (smem > 48 * 1024 && first_on_device(cfg_f))
            cudaFuncSetAttribute(stream_step_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        airun_launch(stream_step_kernel<float>, dim3(T), dim3(256), smem, stream, xs, S, H, y, y_stride, y_bias, carry, write, mult,
                     read, norm_w, eps, (float*)out, out_stride, req_of_token);
    } else {
        return AIRUN_ERR_UNSUPPORTED;
    }
    return airun_launch_status();
}
