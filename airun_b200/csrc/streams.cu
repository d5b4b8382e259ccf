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

// SMAX: the most streams this instance takes (4 or SMAX); the loops over streams are unrolled to it.
template <typename TOut, int SMAX>
__global__ __launch_bounds__(256) void stream_step_kernel(
    float* __restrict__ xs, int S, int H, const float* __restrict__ y, long long y_stride, const float* __restrict__ y_bias,
    const float* __restrict__ carry, const float* __restrict__ write, float mult, const float* __restrict__ read,
    const float* __restrict__ norm_w, float eps, TOut* __restrict__ out, long long out_stride,
    const int32_t* __restrict__ req_of_token) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) float s_u[];   // [H]: the weighted sum, kept between the two passes of the norm
    __shared__ float s_m[SMAX * SMAX], s_b[SMAX], s_a[SMAX], red[33];
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
    // Widths in multiples of four on 16-byte boundaries: a thread takes four neighbouring columns of every stream with
    // one load each.
    const bool vec4 = (H & 3) == 0 && ((uintptr_t)xs & 15) == 0 && (!y || (((uintptr_t)y & 15) == 0 && (y_stride & 3) == 0)) &&
                      (!y_bias || ((uintptr_t)y_bias & 15) == 0);
    if (vec4) {
        for (int c = 4 * threadIdx.x; c < H; c += 4 * blockDim.x) {
            float4 x[SMAX];
#pragma unroll
            for (int s = 0; s < SMAX; ++s)
                x[s] = s < S ? *reinterpret_cast<const float4*>(row + (size_t)s * H + c) : make_float4(0.f, 0.f, 0.f, 0.f);
            if (y) {
                float4 yv = *reinterpret_cast<const float4*>(y + (size_t)t * y_stride + c);
                if (y_bias) {
                    const float4 b4 = *reinterpret_cast<const float4*>(y_bias + c);
                    yv.x += b4.x; yv.y += b4.y; yv.z += b4.z; yv.w += b4.w;
                }
                float4 nx[SMAX];
#pragma unroll
                for (int to = 0; to < SMAX; ++to) {
                    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int from = 0; from < SMAX; ++from)
                        if (from < S && to < S) {
                            const float m = s_m[from * S + to];
                            acc.x = fmaf(m, x[from].x, acc.x); acc.y = fmaf(m, x[from].y, acc.y);
                            acc.z = fmaf(m, x[from].z, acc.z); acc.w = fmaf(m, x[from].w, acc.w);
                        }
                    const float b = to < S ? s_b[to] : 0.0f;
                    nx[to] = make_float4(fmaf(b, yv.x, acc.x), fmaf(b, yv.y, acc.y), fmaf(b, yv.z, acc.z), fmaf(b, yv.w, acc.w));
                }
#pragma unroll
                for (int s = 0; s < SMAX; ++s) {
                    x[s] = nx[s];
                    if (s < S) *reinterpret_cast<float4*>(row + (size_t)s * H + c) = nx[s];
                }
            }
            if (read) {
                float4 u = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int s = 0; s < SMAX; ++s)
                    if (s < S) {
                        const float a = s_a[s];
                        u.x = fmaf(a, x[s].x, u.x); u.y = fmaf(a, x[s].y, u.y); u.z = fmaf(a, x[s].z, u.z); u.w = fmaf(a, x[s].w, u.w);
                    }
                *reinterpret_cast<float4*>(s_u + c) = u;
                ss = fmaf(u.x, u.x, ss); ss = fmaf(u.y, u.y, ss); ss = fmaf(u.z, u.z, ss); ss = fmaf(u.w, u.w, ss);
            }
        }
    } else
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float x[SMAX];
#pragma unroll
        for (int s = 0; s < SMAX; ++s) x[s] = s < S ? row[(size_t)s * H + c] : 0.0f;
        if (y) {
            const float yv = y[(size_t)t * y_stride + c] + (y_bias ? y_bias[c] : 0.0f);
            float nx[SMAX];
#pragma unroll
            for (int to = 0; to < SMAX; ++to) {
                float acc = 0.0f;
#pragma unroll
                for (int from = 0; from < SMAX; ++from)
                    if (from < S && to < S) acc = fmaf(s_m[from * S + to], x[from], acc);
                nx[to] = to < S ? fmaf(s_b[to], yv, acc) : 0.0f;
            }
#pragma unroll
            for (int s = 0; s < SMAX; ++s) {
                x[s] = nx[s];
                if (s < S) row[(size_t)s * H + c] = nx[s];
            }
        }
        if (read) {
            float u = 0.0f;
#pragma unroll
            for (int s = 0; s < SMAX; ++s)
                if (s < S) u = fmaf(s_a[s], x[s], u);
            s_u[c] = u;
            ss = fmaf(u, u, ss);
        }
    }
    if (!read) return;
    if (!norm_w) {
        __syncthreads();                           // columns are read back by other threads than wrote them
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
#define STREAM_LAUNCH(TT, SM) do {                                                                                          \
        static unsigned long long cfg = 0;                                                                                  \
        if (smem > 48 * 1024 && first_on_device(cfg))                                                                       \
            cudaFuncSetAttribute(stream_step_kernel<TT, SM>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);      \
        airun_launch(stream_step_kernel<TT, SM>, dim3(T), dim3(256), smem, stream, xs, S, H, y, y_stride, y_bias, carry, write, \
                     mult, read, norm_w, eps, (TT*)out, out_stride, req_of_token);                                          \
    } while (0)
    if (out_dtype == AIRUN_DT_BF16 && read && norm_w) {
        if (S <= 4) STREAM_LAUNCH(__nv_bfloat16, 4);
        else STREAM_LAUNCH(__nv_bfloat16, STREAMS_MAX);
    } else if (out_dtype == AIRUN_DT_F32 || !read) {
        if (S <= 4) STREAM_LAUNCH(float, 4);
        else STREAM_LAUNCH(float, STREAMS_MAX);
    } else {
        return AIRUN_ERR_UNSUPPORTED;
    }
#undef STREAM_LAUNCH
    return airun_launch_status();
}
