// Softmax attention over cache pages with the options several designs combine differently:
//
//   q = Wq h (+ bq),  k = Wk h (+ bk),  v = Wv h (+ bv)                  the products are the caller's, biases are added here
//   q, k <- x / rms(x) * w            per head, one weight vector for all heads        (`q_w`, `k_w`: before the rotation)
//   q, k <- rotation by the position  (none, pairs (i, i + r/2), or pairs (2i, 2i + 1)) over the first r dimensions
//   q, k <- x / rms(x)                per head, no weight                              (`unit_norm`: after the rotation)
//   q <- q * (1 + coef * ln(floor((p + 1) / every) + 1))                               (`temp_every` > 0)
//   s_ij = scale * q_i . k_j + table[h][min(i - j, table_len - 1)]                     (`table`: a learnt number per head and distance)
//   p_ij = exp(s_ij) / (sum over visible j' of exp(s_ij') + exp(sink_h))               (`sink`: one more term of the denominator
//                                                                                       that has no key and no value)
//   o_i = out_scale * sum_j p_ij v_j,     j visible iff j <= i and (window == 0 or i - j < window)
//
// Query head h reads KV head h / (heads / kv_heads); key rows have D elements, value rows Dv.  Norms, angles, the
// temperature, scores, the softmax and the sum over keys are float32; q, keys and values are stored in the type of
// the cache.  A page holds, for `page_size` tokens, the keys of all KV heads ([kv_heads][page_size][D]) followed by
// the values ([kv_heads][page_size][Dv]).
#include "common.cuh"

#define XA_MAX_PER_LANE 8     // D <= 256 and Dv <= 256
#define XA_PREP_WARPS 8
#define XA_WARPS 4

#define XA_ROPE_NONE 0
#define XA_ROPE_NEOX 1
#define XA_ROPE_INTERLEAVED 2

__device__ __forceinline__ void xa_store4(float* dst, float4 v) { *reinterpret_cast<float4*>(dst) = v; }
__device__ __forceinline__ void xa_store4(__nv_bfloat16* dst, float4 v) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    *reinterpret_cast<uint2*>(dst) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
}

// One block per token; a warp takes a head at a time (the query heads, then the key heads); then all threads copy
// the values.  proj is float32 [T][nh*D (+ nkv*D + nkv*Dv when store)], bias the same columns (or null).
template <typename T>
__global__ __launch_bounds__(32 * XA_PREP_WARPS) void qkv_prepare_kernel(
    const float* __restrict__ proj, long long proj_stride, const float* __restrict__ bias, const float* __restrict__ q_w,
    const float* __restrict__ k_w, int unit_norm, float eps, int rope_kind, int rdim, const float* __restrict__ inv_freq,
    const int32_t* __restrict__ rope_positions, float temp_coef, int temp_every, T* __restrict__ q_out, T* __restrict__ pool,
    const int32_t* __restrict__ block_table, int max_blocks, const int32_t* __restrict__ positions,
    const int32_t* __restrict__ req_of_token, int num_reqs, int num_pages, int page_size, int nh, int nkv, int D, int Dv,
    int store, int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    __shared__ float s_x[XA_PREP_WARPS][32 * XA_MAX_PER_LANE];
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int req = req_of_token[t], pos = positions[t];
    if (req < 0 || pos < 0) return;
    if (req >= num_reqs) {
        if (threadIdx.x == 0) atomicOr(err, AIRUN_DEV_BAD_REQ);
        return;
    }
    T* pk = nullptr;
    T* pv = nullptr;
    int slot = 0;
    if (store) {
        const int blk = pos / page_size;
        slot = pos - blk * page_size;
        const int page = blk < max_blocks ? block_table[(size_t)req * max_blocks + blk] : -1;
        if (page < 0 || page >= num_pages) {
            if (threadIdx.x == 0) atomicOr(err, AIRUN_DEV_BAD_PAGE);
            store = 0;
        } else {
            pk = pool + (size_t)page * nkv * page_size * (D + Dv);
            pv = pk + (size_t)nkv * page_size * D;
        }
    }
    const float* row = proj + (size_t)t * proj_stride;
    const float rpos = (float)(rope_positions ? rope_positions[t] : pos);
    // the angles are the same for every head of the token: one sine and cosine per rotated pair, worked out once
    __shared__ float s_cos[16 * XA_MAX_PER_LANE], s_sin[16 * XA_MAX_PER_LANE];
    if (rope_kind != XA_ROPE_NONE)
        for (int i = threadIdx.x; i < (rdim >> 1); i += blockDim.x) sincosf(rpos * inv_freq[i], &s_sin[i], &s_cos[i]);
    __syncthreads();
    const float temp = temp_every > 0 ? 1.0f + temp_coef * logf((float)((pos + 1) / temp_every) + 1.0f) : 1.0f;
    const int units = nh + (store ? nkv : 0);
    float* sx = s_x[warp];
    // Head sizes in multiples of four on 16-byte boundaries: a lane takes four neighbouring dimensions (eight for heads
    // above 128) with one load each, so both dimensions of a rotated pair (2i, 2i + 1) lie in the lane that turns them.
    const bool vec4 = (D & 3) == 0 && (proj_stride & 3) == 0 && ((uintptr_t)proj & 15) == 0 && (!bias || ((uintptr_t)bias & 15) == 0) &&
                      ((uintptr_t)q_out & 15) == 0 && (!store || ((uintptr_t)pool & 15) == 0) && rope_kind != XA_ROPE_NEOX &&
                      (!q_w || ((uintptr_t)q_w & 15) == 0) && (!k_w || ((uintptr_t)k_w & 15) == 0);
    if (vec4) {
        for (int u = warp; u < units; u += XA_PREP_WARPS) {
            const bool is_q = u < nh;
            const int col0 = u * D;
            const float* w = is_q ? q_w : k_w;
            float4 x[2];
            float ss = 0.0f;
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int d = 4 * lane + 128 * i;
                x[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (d < D) {
                    x[i] = *reinterpret_cast<const float4*>(row + col0 + d);
                    if (bias) {
                        const float4 b4 = *reinterpret_cast<const float4*>(bias + col0 + d);
                        x[i].x += b4.x; x[i].y += b4.y; x[i].z += b4.z; x[i].w += b4.w;
                    }
                }
                ss = fmaf(x[i].x, x[i].x, ss); ss = fmaf(x[i].y, x[i].y, ss); ss = fmaf(x[i].z, x[i].z, ss); ss = fmaf(x[i].w, x[i].w, ss);
            }
            if (w) {
                const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)D + eps);
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const int d = 4 * lane + 128 * i;
                    if (d < D) {
                        const float4 w4 = *reinterpret_cast<const float4*>(w + d);
                        x[i].x *= inv * w4.x; x[i].y *= inv * w4.y; x[i].z *= inv * w4.z; x[i].w *= inv * w4.w;
                    }
                }
            }
            if (rope_kind == XA_ROPE_INTERLEAVED) {
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const int d = 4 * lane + 128 * i;
                    if (d < rdim && d < D) {
                        const float c0 = s_cos[d >> 1], s0 = s_sin[d >> 1];
                        const float a = x[i].x, b = x[i].y;
                        x[i].x = a * c0 - b * s0; x[i].y = b * c0 + a * s0;
                    }
                    if (d + 2 < rdim && d < D) {
                        const float c1 = s_cos[(d >> 1) + 1], s1 = s_sin[(d >> 1) + 1];
                        const float a = x[i].z, b = x[i].w;
                        x[i].z = a * c1 - b * s1; x[i].w = b * c1 + a * s1;
                    }
                }
            }
            float mulv = is_q ? temp : 1.0f;
            if (unit_norm) {
                float s2 = 0.0f;
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    s2 = fmaf(x[i].x, x[i].x, s2); s2 = fmaf(x[i].y, x[i].y, s2); s2 = fmaf(x[i].z, x[i].z, s2); s2 = fmaf(x[i].w, x[i].w, s2);
                }
                const float inv = 1.0f / sqrtf(warp_sum(s2) / (float)D + eps);
#pragma unroll
                for (int i = 0; i < 2; ++i) { x[i].x *= inv; x[i].y *= inv; x[i].z *= inv; x[i].w *= inv; }
            }
            T* dst = is_q ? q_out + ((size_t)t * nh + u) * D : pk + ((size_t)(u - nh) * page_size + slot) * D;
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int d = 4 * lane + 128 * i;
                if (d < D) xa_store4(dst + d, make_float4(x[i].x * mulv, x[i].y * mulv, x[i].z * mulv, x[i].w * mulv));
            }
        }
        if (!store) return;
        const int vcol = (nh + nkv) * D;
        if ((Dv & 3) == 0) {
            for (int c = threadIdx.x; c < (nkv * Dv) >> 2; c += blockDim.x) {
                const int g = (4 * c) / Dv, e = 4 * c - g * Dv;
                float4 v4 = *reinterpret_cast<const float4*>(row + vcol + 4 * c);
                if (bias) {
                    const float4 b4 = *reinterpret_cast<const float4*>(bias + vcol + 4 * c);
                    v4.x += b4.x; v4.y += b4.y; v4.z += b4.z; v4.w += b4.w;
                }
                xa_store4(pv + ((size_t)g * page_size + slot) * Dv + e, v4);
            }
            return;
        }
        for (int c = threadIdx.x; c < nkv * Dv; c += blockDim.x) {
            const int g = c / Dv, e = c - g * Dv;
            pv[((size_t)g * page_size + slot) * Dv + e] = from_f32<T>(row[vcol + c] + (bias ? bias[vcol + c] : 0.0f));
        }
        return;
    }
    for (int u = warp; u < units; u += XA_PREP_WARPS) {
        const bool is_q = u < nh;
        const int col0 = u * D;                      // q heads and k heads follow each other in the row
        const float* w = is_q ? q_w : k_w;
        float x[XA_MAX_PER_LANE];
        float ss = 0.0f;
#pragma unroll
        for (int i = 0; i < XA_MAX_PER_LANE; ++i) {
            const int d = lane + 32 * i;
            x[i] = d < D ? row[col0 + d] + (bias ? bias[col0 + d] : 0.0f) : 0.0f;
            ss = fmaf(x[i], x[i], ss);
        }
        if (w) {
            const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)D + eps);
#pragma unroll
            for (int i = 0; i < XA_MAX_PER_LANE; ++i) {
                const int d = lane + 32 * i;
                if (d < D) x[i] = x[i] * inv * w[d];
            }
        }
        if (rope_kind != XA_ROPE_NONE && rdim > 0) {
            __syncwarp();
#pragma unroll
            for (int i = 0; i < XA_MAX_PER_LANE; ++i) sx[lane + 32 * i] = x[i];
            __syncwarp();
            const int half = rdim >> 1;
#pragma unroll
            for (int i = 0; i < XA_MAX_PER_LANE; ++i) {
                const int d = lane + 32 * i;
                if (d >= rdim || d >= D) continue;
                int pair, other;
                bool first;
                if (rope_kind == XA_ROPE_INTERLEAVED) { pair = d >> 1; first = (d & 1) == 0; other = d ^ 1; }
                else { first = d < half; pair = first ? d : d - half; other = first ? d + half : d - half; }
                const float sn = s_sin[pair], cs = s_cos[pair];
                const float o = sx[other];
                x[i] = first ? x[i] * cs - o * sn : x[i] * cs + o * sn;
            }
        }
        if (unit_norm) {
            float s2 = 0.0f;
#pragma unroll
            for (int i = 0; i < XA_MAX_PER_LANE; ++i) s2 = fmaf(x[i], x[i], s2);
            const float inv = 1.0f / sqrtf(warp_sum(s2) / (float)D + eps);
#pragma unroll
            for (int i = 0; i < XA_MAX_PER_LANE; ++i) x[i] *= inv;
        }
        if (is_q) {
            T* dst = q_out + ((size_t)t * nh + u) * D;
#pragma unroll
            for (int i = 0; i < XA_MAX_PER_LANE; ++i) {
                const int d = lane + 32 * i;
                if (d < D) dst[d] = from_f32<T>(x[i] * temp);
            }
        } else {
            T* dst = pk + ((size_t)(u - nh) * page_size + slot) * D;
#pragma unroll
            for (int i = 0; i < XA_MAX_PER_LANE; ++i) {
                const int d = lane + 32 * i;
                if (d < D) dst[d] = from_f32<T>(x[i]);
            }
        }
    }
    if (!store) return;
    const int vcol0 = (nh + nkv) * D;
    for (int c = threadIdx.x; c < nkv * Dv; c += blockDim.x) {
        const int g = c / Dv, e = c - g * Dv;
        pv[((size_t)g * page_size + slot) * Dv + e] = from_f32<T>(row[vcol0 + c] + (bias ? bias[vcol0 + c] : 0.0f));
    }
}

AIRUN_EXPORT int airun_qkv_prepare(const float* proj, long long proj_stride, const float* bias, const float* q_w, const float* k_w,
                                   int unit_norm, float eps, int rope_kind, int rdim, const float* inv_freq,
                                   const int32_t* rope_positions, float temp_coef, int temp_every, void* q_out, void* pool,
                                   int dtype, const int32_t* block_table, int max_blocks, const int32_t* positions,
                                   const int32_t* req_of_token, int T, int num_reqs, int num_pages, int page_size, int nh,
                                   int nkv, int D, int Dv, int store, int* err, cudaStream_t stream) {
    if (T < 0 || nh <= 0 || nkv <= 0 || D <= 0 || D > 32 * XA_MAX_PER_LANE || Dv <= 0 || temp_every < 0 || !err || !positions ||
        !req_of_token || !proj || !q_out || rdim < 0 || rdim > D || (rdim & 1) ||
        (rope_kind != XA_ROPE_NONE && rdim > 0 && !inv_freq) || rope_kind < 0 || rope_kind > 2 ||
        (store && (!pool || !block_table || page_size <= 0 || num_pages <= 0 || max_blocks <= 0)))
        return AIRUN_ERR_ARG;
    if (T == 0) return AIRUN_OK;
#define XP_LAUNCH(TT) airun_launch(qkv_prepare_kernel<TT>, dim3(T), dim3(32 * XA_PREP_WARPS), 0, stream, proj, proj_stride, bias, q_w, \
        k_w, unit_norm, eps, rope_kind, rdim, inv_freq, rope_positions, temp_coef, temp_every, (TT*)q_out, (TT*)pool, block_table, \
        max_blocks, positions, req_of_token, num_reqs, num_pages, page_size, nh, nkv, D, Dv, store, err)
    if (dtype == AIRUN_DT_F32) XP_LAUNCH(float);
    else if (dtype == AIRUN_DT_BF16) XP_LAUNCH(__nv_bfloat16);
    else return AIRUN_ERR_UNSUPPORTED;
#undef XP_LAUNCH
    return airun_launch_status();
}

// One block per (token, query head).  Each warp walks every XA_WARPS-th visible key with a running maximum, sum and
// weighted value sum of its own; the warps' partial results are merged in warp order at the end, and the sink joins
// the denominator there.  A token's result depends only on its own q, its position and the keys it sees.
template <typename T>
__global__ __launch_bounds__(32 * XA_WARPS) void softmax_attention_kernel(
    const T* __restrict__ q, T* __restrict__ out, long long out_stride, const T* __restrict__ pool,
    const int32_t* __restrict__ block_table, int max_blocks, const int32_t* __restrict__ positions,
    const int32_t* __restrict__ req_of_token, int num_reqs, int num_pages, int page_size, int nh, int nkv, int D, int Dv,
    float scale, const float* __restrict__ table, int table_len, const float* __restrict__ sink, int window, float out_scale,
    int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float s_acc[];           // [XA_WARPS][Dv], then [XA_WARPS] maxima and [XA_WARPS] sums
    float* s_m = s_acc + (size_t)XA_WARPS * Dv;
    float* s_l = s_m + XA_WARPS;
    const int t = blockIdx.x, head = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pos = positions[t], req = req_of_token[t];
    T* dst = out + (size_t)t * out_stride + (size_t)head * Dv;
    if (req < 0 || pos < 0 || req >= num_reqs) {      // a padding row
        if (req >= num_reqs && threadIdx.x == 0) atomicOr(err, AIRUN_DEV_BAD_REQ);
        for (int d = threadIdx.x; d < Dv; d += blockDim.x) dst[d] = from_f32<T>(0.0f);
        return;
    }
    const int kvh = head / (nh / nkv);
    const T* qv = q + ((size_t)t * nh + head) * D;
    float qr[XA_MAX_PER_LANE], acc[XA_MAX_PER_LANE];
#pragma unroll
    for (int i = 0; i < XA_MAX_PER_LANE; ++i) {
        const int d = lane + i * 32;
        qr[i] = d < D ? to_f32<T>(qv[d]) : 0.0f;
        acc[i] = 0.0f;
    }
    const float* tab = table ? table + (size_t)head * table_len : nullptr;
    const int32_t* bt = block_table + (size_t)req * max_blocks;
    const int begin = window > 0 ? max(0, pos - window + 1) : 0;
    bool bad = false;
    const size_t page_elems = (size_t)nkv * page_size * (D + Dv);
    float m = -INFINITY, l = 0.0f;
    for (int j = begin + warp; j <= pos; j += XA_WARPS) {
        const int blk = j / page_size;
        const int page = blk < max_blocks ? bt[blk] : -1;
        if (page < 0 || page >= num_pages) { bad = true; continue; }
        const T* pk = pool + (size_t)page * page_elems;
        const T* kj = pk + ((size_t)kvh * page_size + (j - blk * page_size)) * D;
        const T* vj = pk + (size_t)nkv * page_size * D + ((size_t)kvh * page_size + (j - blk * page_size)) * Dv;
        float dot = 0.0f;
#pragma unroll
        for (int i = 0; i < XA_MAX_PER_LANE; ++i) {
            const int d = lane + i * 32;
            if (d < D) dot = fmaf(qr[i], to_f32<T>(kj[d]), dot);
        }
        float s = warp_sum(dot) * scale;
        if (tab) s += tab[min(pos - j, table_len - 1)];
        const float mn = fmaxf(m, s);
        const float corr = expf(m - mn), w = expf(s - mn);       // m = -inf the first time: corr = 0
        l = l * corr + w;
#pragma unroll
        for (int i = 0; i < XA_MAX_PER_LANE; ++i) {
            const int d = lane + i * 32;
            if (d < Dv) acc[i] = fmaf(w, to_f32<T>(vj[d]), acc[i] * corr);
        }
        m = mn;
    }
    if (bad && lane == 0) atomicOr(err, AIRUN_DEV_BAD_PAGE);
#pragma unroll
    for (int i = 0; i < XA_MAX_PER_LANE; ++i) {
        const int d = lane + i * 32;
        if (d < Dv) s_acc[(size_t)warp * Dv + d] = acc[i];
    }
    if (lane == 0) { s_m[warp] = m; s_l[warp] = l; }
    __syncthreads();
    float top = sink ? sink[head] : -INFINITY;
#pragma unroll
    for (int w = 0; w < XA_WARPS; ++w) top = fmaxf(top, s_m[w]);
    float den = sink ? expf(sink[head] - top) : 0.0f;
    float f[XA_WARPS];
#pragma unroll
    for (int w = 0; w < XA_WARPS; ++w) {
        f[w] = s_m[w] == -INFINITY ? 0.0f : expf(s_m[w] - top);
        den = fmaf(s_l[w], f[w], den);
    }
    const float inv = den > 0.0f ? out_scale / den : 0.0f;
    for (int d = threadIdx.x; d < Dv; d += blockDim.x) {
        float o = 0.0f;
#pragma unroll
        for (int w = 0; w < XA_WARPS; ++w) o = fmaf(s_acc[(size_t)w * Dv + d], f[w], o);
        dst[d] = from_f32<T>(o * inv);
    }
}

AIRUN_EXPORT int airun_softmax_attention(const void* q, void* out, long long out_stride, const void* pool, int dtype,
                                         const int32_t* block_table, int max_blocks, const int32_t* positions,
                                         const int32_t* req_of_token, int T, int num_reqs, int num_pages, int page_size,
                                         int nh, int nkv, int D, int Dv, float scale, const float* table, int table_len,
                                         const float* sink, int window, float out_scale, int* err, cudaStream_t stream) {
    if (T < 0 || nh <= 0 || nkv <= 0 || nh % nkv != 0 || D <= 0 || D > 32 * XA_MAX_PER_LANE || Dv <= 0 ||
        Dv > 32 * XA_MAX_PER_LANE || page_size <= 0 || num_pages <= 0 || max_blocks <= 0 || window < 0 || !err || nh > 65535 ||
        out_stride < (long long)nh * Dv || (table && table_len <= 0))
        return AIRUN_ERR_ARG;
    if (T == 0) return AIRUN_OK;
    dim3 grid(T, nh);
    const size_t smem = ((size_t)XA_WARPS * Dv + 2 * XA_WARPS) * sizeof(float);
#define XA_LAUNCH(TT) airun_launch(softmax_attention_kernel<TT>, grid, dim3(32 * XA_WARPS), smem, stream, (const TT*)q, (TT*)out, \
        out_stride, (const TT*)pool, block_table, max_blocks, positions, req_of_token, num_reqs, num_pages, page_size, nh, nkv, D, Dv, \
        scale, table, table_len, sink, window, out_scale, err)
    if (dtype == AIRUN_DT_F32) XA_LAUNCH(float);
    else if (dtype == AIRUN_DT_BF16) XA_LAUNCH(__nv_bfloat16);
    else return AIRUN_ERR_UNSUPPORTED;
#undef XA_LAUNCH
    return airun_launch_status();
}
