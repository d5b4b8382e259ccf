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

// Routing by softmax scores with a correction and groups.  z [T][n_out] are the router's outputs, of which the first
// `num_real` stand for experts with matrices and the rest for experts that return their input; all of them take part in
// the softmax, the groups and the choice alike.
//   s = softmax(z) over all outputs;   c = s + correction  (the choice score; the weights use s)
//   the outputs form `groups` equal runs of neighbours; a run's score is its largest c, and only outputs of the `keep`
//   best runs can be chosen (the others count as minus infinity: c may be negative)
//   the `top` largest c are chosen (equal: the lower id);  weight = s / (sum of the chosen s + 1e-20) * weight_scale
// One warp per token.  Only experts with matrices are counted into segments.
__global__ __launch_bounds__(128) void moe_route_grouped_kernel(
    const float* __restrict__ z, long long z_stride, const float* __restrict__ correction, int T, int n_out, int num_real, int top,
    int groups, int keep, float weight_scale, const int32_t* __restrict__ req_of_token, int32_t* __restrict__ ids,
    float* __restrict__ wts, int32_t* __restrict__ rank, int32_t* __restrict__ counts) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float s_all[];                     // [4][2 * n_out + groups]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * 4 + warp;
    if (t >= T) return;
    float* s_score = s_all + (size_t)warp * (2 * n_out + groups);
    float* s_choice = s_score + n_out;
    float* s_group = s_choice + n_out;
    if (req_of_token[t] < 0) {
        for (int k = lane; k < top; k += 32) ids[(size_t)t * top + k] = -1;
        return;
    }
    float zmax = -INFINITY;
    for (int e = lane; e < n_out; e += 32) {
        const float v = z[(size_t)t * z_stride + e];
        s_score[e] = v;
        zmax = fmaxf(zmax, v);
    }
    zmax = warp_max(zmax);
    float zsum = 0.0f;
    for (int e = lane; e < n_out; e += 32) {
        const float v = expf(s_score[e] - zmax);
        s_score[e] = v;
        zsum += v;
    }
    zsum = warp_sum(zsum);
    for (int e = lane; e < n_out; e += 32) {
        const float sc = s_score[e] / zsum;
        s_score[e] = sc;
        s_choice[e] = sc + (correction ? correction[e] : 0.0f);
    }
    __syncwarp();
    if (groups > 1) {
        const int per = n_out / groups;
        for (int g = lane; g < groups; g += 32) {
            float best = -INFINITY;
            for (int e = g * per; e < (g + 1) * per; ++e) best = fmaxf(best, s_choice[e]);
            s_group[g] = best;
        }
        __syncwarp();
        // a run is kept when fewer than `keep` runs beat it (a run beats another with a larger score, or an equal one and a lower id)
        for (int g = lane; g < groups; g += 32) {
            int ahead = 0;
            const float mine = s_group[g];
            for (int o = 0; o < groups; ++o) ahead += (s_group[o] > mine || (s_group[o] == mine && o < g)) ? 1 : 0;
            if (ahead >= keep)
                for (int e = g * per; e < (g + 1) * per; ++e) s_choice[e] = -INFINITY;
        }
        __syncwarp();
    }
    float total = 0.0f;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int arg = n_out;
        for (int e = lane; e < n_out; e += 32) {
            const float v = s_choice[e];
            if (v > best) { best = v; arg = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
        }
        if (arg >= n_out) arg = 0;                          // nothing left to choose from (NaN outputs): still a valid expert
        const float score = s_score[arg];
        total += score;
        if (lane == 0) {
            ids[(size_t)t * top + k] = arg;
            wts[(size_t)t * top + k] = score;
            rank[(size_t)t * top + k] = arg < num_real ? atomicAdd(&counts[arg], 1) : 0;
            s_choice[arg] = -INFINITY;
        }
        __syncwarp();
    }
    if (lane == 0)
        for (int k = 0; k < top; ++k) wts[(size_t)t * top + k] = wts[(size_t)t * top + k] / (total + 1e-20f) * weight_scale;
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
    int32_t* __restrict__ row_of, int num_real) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    for (int k = 0; k < top; ++k) {
        const int e = ids[(size_t)t * top + k];
        if (e < 0) return;
        if (e >= num_real) {                  // an expert that hands its input on: it has no row in any segment
            if (threadIdx.x == 0) row_of[(size_t)t * top + k] = -1;
            continue;
        }
        const int row = seg[e] + rank[(size_t)t * top + k];
        if (threadIdx.x == 0) row_of[(size_t)t * top + k] = row;
        const float w = scale_input ? wts[(size_t)t * top + k] : 1.0f;
        for (int c = threadIdx.x; c < W; c += blockDim.x)
            xs[(size_t)row * W + c] = from_f32<TH>(w * to_f32<TH>(h[(size_t)t * W + c]));
    }
}

template <typename TH>
__global__ __launch_bounds__(256) void moe_combine_kernel(
    const float* __restrict__ ys, int W, int top, const int32_t* __restrict__ ids, const float* __restrict__ wts,
    const int32_t* __restrict__ row_of, int scale_output, float* __restrict__ out, const TH* __restrict__ h) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const bool pad = ids[(size_t)t * top] < 0;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float acc = 0.0f;
        if (!pad)
            for (int k = 0; k < top; ++k) {
                const int r = row_of[(size_t)t * top + k];
                const float y = r >= 0 ? ys[(size_t)r * W + c] : (h ? to_f32<TH>(h[(size_t)t * W + c]) : 0.0f);
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

AIRUN_EXPORT int airun_moe_route_grouped(const float* z, long long z_stride, const float* correction, int T, int n_out, int num_real,
                                         int top, int groups, int keep, float weight_scale, const int32_t* req_of_token, int32_t* ids,
                                         float* wts, int32_t* rank, int32_t* counts, int32_t* seg, cudaStream_t stream) {
    if (T < 0 || n_out <= 0 || z_stride < n_out || n_out > MOE_MAX_EXPERTS || num_real <= 0 || num_real > n_out || top <= 0 || groups <= 0 ||
        n_out % groups != 0 || keep <= 0 || keep > groups || top > (n_out / groups) * keep || !z || !req_of_token || !ids || !wts || !rank ||
        !counts || !seg)
        return AIRUN_ERR_ARG;
    if (T == 0) return AIRUN_OK;
    airun_launch(moe_route_grouped_kernel, dim3(ceil_div_i(T, 4)), dim3(128), (size_t)4 * (2 * n_out + groups) * sizeof(float), stream, z,
                 z_stride, correction, T, n_out, num_real, top, groups, keep, weight_scale, req_of_token, ids, wts, rank, counts);
    airun_launch(moe_offsets_kernel, dim3(1), dim3(32), 0, stream, (const int32_t*)counts, seg, num_real);
    return airun_launch_status();
}

AIRUN_EXPORT int airun_moe_scatter(const void* h, int dtype, int T, int W, int top, const int32_t* ids, const float* wts,
                                   const int32_t* rank, const int32_t* seg, int scale_input, void* xs, int32_t* row_of,
                                   int num_real, cudaStream_t stream) {
    if (T < 0 || W <= 0 || top <= 0 || !ids || !wts || !rank || !seg || !xs || !row_of || num_real <= 0) return AIRUN_ERR_ARG;
    if (T == 0) return AIRUN_OK;
    if (dtype == AIRUN_DT_F32)
        airun_launch(moe_scatter_kernel<float>, dim3(T), dim3(256), 0, stream, (const float*)h, W, top, ids, wts, rank, seg,
                     scale_input, (float*)xs, row_of, num_real);
    else if (dtype == AIRUN_DT_BF16)
        airun_launch(moe_scatter_kernel<__nv_bfloat16>, dim3(T), dim3(256), 0, stream, (const __nv_bfloat16*)h, W, top, ids, wts,
                     rank, seg, scale_input, (__nv_bfloat16*)xs, row_of, num_real);
    else
        return AIRUN_ERR_UNSUPPORTED;
    return airun_launch_status();
}

// `h` (the feed-forward's input, [T][W] of type `h_dtype`; may be null): what a chosen expert without matrices returns.
AIRUN_EXPORT int airun_moe_combine(const float* ys, int T, int W, int top, const int32_t* ids, const float* wts,
                                   const int32_t* row_of, int scale_output, float* out, const void* h, int h_dtype,
                                   cudaStream_t stream) {
    if (T < 0 || W <= 0 || top <= 0 || !ys || !ids || !wts || !row_of || !out) return AIRUN_ERR_ARG;
    if (T == 0) return AIRUN_OK;
    if (h && h_dtype == AIRUN_DT_BF16)
        airun_launch(moe_combine_kernel<__nv_bfloat16>, dim3(T), dim3(256), 0, stream, ys, W, top, ids, wts, row_of, scale_output, out,
                     (const __nv_bfloat16*)h);
    else if (!h || h_dtype == AIRUN_DT_F32)
        airun_launch(moe_combine_kernel<float>, dim3(T), dim3(256), 0, stream, ys, W, top, ids, wts, row_of, scale_output, out,
                     (const float*)h);
    else
        return AIRUN_ERR_UNSUPPORTED;
    return airun_launch_status();
}
