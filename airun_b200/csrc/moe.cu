// A routed feed-forward: every token goes to the `top` experts with the largest scores.
//
//   z = Wr h (+ a bias per expert, when the router has one) (float32),  s = sigmoid(z) or softmax(z);  the `top` largest s (equal scores: the lower id first),
//   found as the `top` largest z: the order is the same, and float32 scores that saturate at 1 are not told apart
//   weight = s of the chosen expert, divided by the sum of the chosen ones when `renorm`
// The rows of a step are then sorted by expert so that every expert's rows are one segment of a buffer and a
// grouped product (gemm_simt.cu) runs each segment against its expert's matrices:
//   route    from the logits: ids, weights, and each row's rank among its expert's rows (a counter per expert)
//   offsets  seg[e] = rows of the experts before e
//   scatter  xs[seg[e] + rank] = h[t] (times the weight, when the weight scales the expert's INPUT)
//   ...      the experts' products on xs ...
//   combine  out[t] = sum over the token's experts, in the order they were chosen, of ys[row] (times the weight,
//            when it scales the output)
// A row's result depends on the row alone, so the order in which rows reach a segment (the counters are atomic)
// does not show in the result.  Rows of request -1 are padding: they are routed nowhere.
#include "common.cuh"

#define MOE_MAX_EXPERTS 1024

// One warp per token; z [T][z_stride >= E] are the router's logits (a product like any other, accumulated in float32).
__global__ __launch_bounds__(128) void moe_route_kernel(
    const float* __restrict__ z, long long z_stride, const float* __restrict__ bias, int T, int E, int top, int softmax_scores, int renorm,
    const int32_t* __restrict__ req_of_token, int32_t* __restrict__ ids, float* __restrict__ wts, int32_t* __restrict__ rank,
    int32_t* __restrict__ counts) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float s_all[];                     // [4][E]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * 4 + warp;
    if (t >= T) return;
    float* s_score = s_all + (size_t)warp * E;
    if (req_of_token[t] < 0) {
        for (int k = lane; k < top; k += 32) ids[(size_t)t * top + k] = -1;
        return;
    }
    for (int e = lane; e < E; e += 32) s_score[e] = z[(size_t)t * z_stride + e] + (bias ? bias[e] : 0.0f);
    __syncwarp();
    // The choice is made on the logits: sigmoid and softmax rise with them, so the order is the same, and two large
    // logits whose scores both round to 1 are still told apart.  The score of a chosen expert is worked out afterwards.
    float smax = -INFINITY, ssum = 1.0f;
    if (softmax_scores) {
        for (int e = lane; e < E; e += 32) smax = fmaxf(smax, s_score[e]);
        smax = warp_max(smax);
        ssum = 0.0f;
        for (int e = lane; e < E; e += 32) ssum += expf(s_score[e] - smax);
        ssum = warp_sum(ssum);
    }
    float total = 0.0f;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int arg = E;
        for (int e = lane; e < E; e += 32) {
            const float v = s_score[e];
            if (v > best) { best = v; arg = e; }          // within a lane ids rise, so the first of equals stays
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
        }
        if (arg >= E) arg = 0;                              // a row of NaN logits: still a valid expert
        const float score = softmax_scores ? expf(best - smax) / ssum : 1.0f / (1.0f + expf(-best));
        total += score;
        if (lane == 0) {
            ids[(size_t)t * top + k] = arg;
            wts[(size_t)t * top + k] = score;
            rank[(size_t)t * top + k] = atomicAdd(&counts[arg], 1);
            s_score[arg] = -INFINITY;
        }
        __syncwarp();
    }
    if (renorm && lane == 0)
        for (int k = 0; k < top; ++k) wts[(size_t)t * top + k] /= total;
}

__global__ void moe_offsets_kernel(const int32_t* __restrict__ counts, int32_t* __restrict__ seg, int E) {
    pdl_trigger();
    pdl_wait();
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        int at = 0;
        seg[0] = 0;
        for (int e = 0; e < E; ++e) { at += counts[e]; seg[e + 1] = at; }
    }
}

template <typename TH>
__global__ __launch_bounds__(256) void moe_scatter_kernel(
    const TH* __restrict__ h, int W, int top, const int32_t* __restrict__ ids, const float* __restrict__ wts,
    const int32_t* __restrict__ rank, const int32_t* __restrict__ seg, int scale_input, TH* __restrict__ xs,
    int32_t* __restrict__ row_of) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    for (int k = 0; k < top; ++k) {
        const int e = ids[(size_t)t * top + k];
        if (e < 0) return;
        const int row = seg[e] + rank[(size_t)t * top + k];
        if (threadIdx.x == 0) row_of[(size_t)t * top + k] = row;
        const float w = scale_input ? wts[(size_t)t * top + k] : 1.0f;
        for (int c = threadIdx.x; c < W; c += blockDim.x)
            xs[(size_t)row * W + c] = from_f32<TH>(w * to_f32<TH>(h[(size_t)t * W + c]));
    }
}

__global__ __launch_bounds__(256) void moe_combine_kernel(
    const float* __restrict__ ys, int W, int top, const int32_t* __restrict__ ids, const float* __restrict__ wts,
    const int32_t* __restrict__ row_of, int scale_output, float* __restrict__ out) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const bool pad = ids[(size_t)t * top] < 0;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float acc = 0.0f;
        if (!pad)
            for (int k = 0; k < top; ++k) {
                const float y = ys[(size_t)row_of[(size_t)t * top + k] * W + c];
                acc = scale_output ? fmaf(wts[(size_t)t * top + k], y, acc) : acc + y;
            }
        out[(size_t)t * W + c] = acc;
    }
}

AIRUN_EXPORT int airun_moe_route(const float* z, long long z_stride, const float* bias, int T, int E, int top, int softmax_scores, int renorm,
                                 const int32_t* req_of_token, int32_t* ids, float* wts, int32_t* rank, int32_t* counts,
                                 int32_t* seg, cudaStream_t stream) {
    if (T < 0 || E <= 0 || z_stride < E || E > MOE_MAX_EXPERTS || top <= 0 || top > E || !z || !req_of_token || !ids || !wts || !rank ||
        !counts || !seg)
        return AIRUN_ERR_ARG;
    if (T == 0) return AIRUN_OK;
    airun_launch(moe_route_kernel, dim3(ceil_div_i(T, 4)), dim3(128), (size_t)4 * E * sizeof(float), stream, z, z_stride, bias, T, E, top,
                 softmax_scores, renorm, req_of_token, ids, wts, rank, counts);
    airun_launch(moe_offsets_kernel, dim3(1), dim3(32), 0, stream, (const int32_t*)counts, seg, E);
    return airun_launch_status();
}

AIRUN_EXPORT int airun_moe_scatter(const void* h, int dtype, int T, int W, int top, const int32_t* ids, const float* wts,
                                   const int32_t* rank, const int32_t* seg, int scale_input, void* xs, int32_t* row_of,
                                   cudaStream_t stream) {
    if (T < 0 || W <= 0 || top <= 0 || !ids || !wts || !rank || !seg || !xs || !row_of) return AIRUN_ERR_ARG;
    if (T == 0) return AIRUN_OK;
    if (dtype == AIRUN_DT_F32)
        airun_launch(moe_scatter_kernel<float>, dim3(T), dim3(256), 0, stream, (const float*)h, W, top, ids, wts, rank, seg,
                     scale_input, (float*)xs, row_of);
    else if (dtype == AIRUN_DT_BF16)
        airun_launch(moe_scatter_kernel<__nv_bfloat16>, dim3(T), dim3(256), 0, stream, (const __nv_bfloat16*)h, W, top, ids, wts,
                     rank, seg, scale_input, (__nv_bfloat16*)xs, row_of);
    else
        return AIRUN_ERR_UNSUPPORTED;
    return airun_launch_status();
}

AIRUN_EXPORT int airun_moe_combine(const float* ys, int T, int W, int top, const int32_t* ids, const float* wts,
                                   const int32_t* row_of, int scale_output, float* out, cudaStream_t stream) {
    if (T < 0 || W <= 0 || top <= 0 || !ys || !ids || !wts || !row_of || !out) return AIRUN_ERR_ARG;
    if (T == 0) return AIRUN_OK;
    airun_launch(moe_combine_kernel, dim3(T), dim3(256), 0, stream, ys, W, top, ids, wts, row_of, scale_output, out);
    return airun_launch_status();
}
