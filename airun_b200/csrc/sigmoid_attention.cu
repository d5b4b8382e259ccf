// Attention without softmax over cache pages: every visible key weighs sigmoid(score), nothing is normalised
// over the keys.
//
//   q = Wq h, k = Wk h, v = Wv h
//   q <- q / rms(q) * wq * temp(p),  k <- k / rms(k) * wk        the root mean square runs over the WHOLE projection
//                                                                (all heads of the token at once), eps inside the root
//   temp(p) = 1 + coef * ln(floor((p + 1) / every) + 1)          (every == 0: no temperature)
//   s_ij = scale * q_i . k_j - a_h * ln(1 + b_h * (i - j)) + c_h     a, b, c: numbers per query head (a: no distance term when null)
//   o_i = sum over j <= i (and i - j < window, when window > 0) of sigmoid(s_ij) v_j
//
// Query head h reads KV head h / (heads / kv_heads).  Norms, temperature, scores, the logarithm, the sigmoid and the
// sum over keys are float32; q, keys and values are read in their storage type.  There is no rotation: positions
// enter through temp and the distance term only.
//
// A page of the cache holds, for `page_size` tokens, the keys of all KV heads ([kv_heads][page_size][D]) followed by
// the values ([kv_heads][page_size][Dv]).
#include "common.cuh"

#define SA_WARPS 4
#define SA_MAX_PER_LANE 8     // D <= 256 and Dv <= 256

__device__ __forceinline__ void sa_store4(float* dst, float4 v) { *reinterpret_cast<float4*>(dst) = v; }
__device__ __forceinline__ void sa_store4(__nv_bfloat16* dst, float4 v) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    *reinterpret_cast<uint2*>(dst) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
}
#define SA_ROW_VECS 8         // float4 a thread keeps of a projection: rows of up to 8,192 numbers are read once

// One block per token: the two norms over whole projections, the temperature, q out, keys and values into the
// token's page.  proj is float32 [T][q_width (+ nkv*kd + nkv*vd when store)].  When every width is a multiple of 4
// (and the rows are aligned) a thread reads its part of the token's q and k once, sixteen bytes at a time, keeps it in
// registers across the two sums and writes four results at a time; otherwise it goes number by number.
template <typename T>
__global__ __launch_bounds__(256) void qk_rownorm_store_kernel(
    const float* __restrict__ proj, long long proj_stride, const float* __restrict__ q_w, const float* __restrict__ k_w,
    float eps, float temp_coef, int temp_every, T* __restrict__ q_out, T* __restrict__ pool,
    const int32_t* __restrict__ block_table, int max_blocks, const int32_t* __restrict__ positions,
    const int32_t* __restrict__ req_of_token, int num_reqs, int num_pages, int page_size, int q_width, int nkv, int kd, int vd,
    int store, int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    __shared__ float red[33];
    const int t = blockIdx.x;
    const int req = req_of_token[t], pos = positions[t];
    if (req < 0 || pos < 0) return;
    if (req >= num_reqs) {
        if (threadIdx.x == 0) atomicOr(err, AIRUN_DEV_BAD_REQ);
        return;
    }
    const float* row = proj + (size_t)t * proj_stride;
    const int kw_all = nkv * kd;
    if (((q_width | kd | vd) & 3) == 0 && (proj_stride & 3) == 0 && ((uintptr_t)proj & 15) == 0 && ((uintptr_t)q_out & 15) == 0 &&
        (!store || ((uintptr_t)pool & 15) == 0) && q_width <= SA_ROW_VECS * 4 * 256 && kw_all <= SA_ROW_VECS * 4 * 256 &&
        (!q_w || ((uintptr_t)q_w & 15) == 0) && (!k_w || ((uintptr_t)k_w & 15) == 0)) {
        const int tid = threadIdx.x, qn = q_width >> 2, kn = kw_all >> 2;
        const float4* row4 = reinterpret_cast<const float4*>(row);
        int page = -1;
        if (store) {
            const int blk = pos / page_size;
            page = blk < max_blocks ? block_table[(size_t)req * max_blocks + blk] : -1;
        }
        const bool keys = store && page >= 0 && page < num_pages;
        float4 qv[SA_ROW_VECS], kv[SA_ROW_VECS];
        float ss = 0.0f, ks = 0.0f;
#pragma unroll
        for (int i = 0; i < SA_ROW_VECS; ++i) {
            const int c = tid + i * 256;
            qv[i] = c < qn ? row4[c] : make_float4(0.f, 0.f, 0.f, 0.f);
            kv[i] = (keys && c < kn) ? row4[qn + c] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int i = 0; i < SA_ROW_VECS; ++i) {
            ss = fmaf(qv[i].x, qv[i].x, ss); ss = fmaf(qv[i].y, qv[i].y, ss); ss = fmaf(qv[i].z, qv[i].z, ss); ss = fmaf(qv[i].w, qv[i].w, ss);
            ks = fmaf(kv[i].x, kv[i].x, ks); ks = fmaf(kv[i].y, kv[i].y, ks); ks = fmaf(kv[i].z, kv[i].z, ks); ks = fmaf(kv[i].w, kv[i].w, ks);
        }
        ss = block_sum(ss, red);
        ks = block_sum(ks, red);
        float inv = q_w ? rsqrtf(ss / (float)q_width + eps) : 1.0f;
        if (temp_every > 0) inv *= 1.0f + temp_coef * logf((float)((pos + 1) / temp_every) + 1.0f);
#pragma unroll
        for (int i = 0; i < SA_ROW_VECS; ++i) {
            const int c = tid + i * 256;
            if (c >= qn) break;
            const float4 w = q_w ? reinterpret_cast<const float4*>(q_w)[c] : make_float4(1.f, 1.f, 1.f, 1.f);
            sa_store4(q_out + (size_t)t * q_width + 4 * c, make_float4(qv[i].x * w.x * inv, qv[i].y * w.y * inv, qv[i].z * w.z * inv, qv[i].w * w.w * inv));
        }
        if (!store) return;
        if (!keys) {
            if (tid == 0) atomicOr(err, AIRUN_DEV_BAD_PAGE);
            return;
        }
        const int slot = pos - (pos / page_size) * page_size;
        const float kinv = k_w ? rsqrtf(ks / (float)kw_all + eps) : 1.0f;
        T* pk = pool + (size_t)page * nkv * page_size * (kd + vd);
        T* pv = pk + (size_t)nkv * page_size * kd;
#pragma unroll
        for (int i = 0; i < SA_ROW_VECS; ++i) {
            const int c = tid + i * 256;
            if (c >= kn) break;
            const int g = (4 * c) / kd, e = 4 * c - g * kd;
            const float4 w = k_w ? reinterpret_cast<const float4*>(k_w)[c] : make_float4(1.f, 1.f, 1.f, 1.f);
            sa_store4(pk + ((size_t)g * page_size + slot) * kd + e, make_float4(kv[i].x * w.x * kinv, kv[i].y * w.y * kinv, kv[i].z * w.z * kinv, kv[i].w * w.w * kinv));
        }
        const float4* v4 = row4 + qn + kn;
        for (int c = tid; c < (nkv * vd) >> 2; c += 256) {
            const int g = (4 * c) / vd, e = 4 * c - g * vd;
            sa_store4(pv + ((size_t)g * page_size + slot) * vd + e, v4[c]);
        }
        return;
    }
    float ss = 0.0f;
    for (int c = threadIdx.x; c < q_width; c += blockDim.x) ss = fmaf(row[c], row[c], ss);
    ss = block_sum(ss, red);
    float inv = q_w ? rsqrtf(ss / (float)q_width + eps) : 1.0f;
    if (temp_every > 0) inv *= 1.0f + temp_coef * logf((float)((pos + 1) / temp_every) + 1.0f);
    for (int c = threadIdx.x; c < q_width; c += blockDim.x)
        q_out[(size_t)t * q_width + c] = from_f32<T>(row[c] * (q_w ? q_w[c] : 1.0f) * inv);
    if (!store) return;
    const int blk = pos / page_size, slot = pos - blk * page_size;
    const int page = blk < max_blocks ? block_table[(size_t)req * max_blocks + blk] : -1;
    if (page < 0 || page >= num_pages) {
        if (threadIdx.x == 0) atomicOr(err, AIRUN_DEV_BAD_PAGE);
        return;
    }
    const int kw = nkv * kd;
    const float* krow = row + q_width;
    const float* vrow = krow + kw;
    float ks = 0.0f;
    for (int c = threadIdx.x; c < kw; c += blockDim.x) ks = fmaf(krow[c], krow[c], ks);
    ks = block_sum(ks, red);
    const float kinv = k_w ? rsqrtf(ks / (float)kw + eps) : 1.0f;
    T* pk = pool + (size_t)page * nkv * page_size * (kd + vd);
    T* pv = pk + (size_t)nkv * page_size * kd;
    for (int c = threadIdx.x; c < kw; c += blockDim.x) {
        const int g = c / kd, e = c - g * kd;
        pk[((size_t)g * page_size + slot) * kd + e] = from_f32<T>(krow[c] * (k_w ? k_w[c] : 1.0f) * kinv);
    }
    for (int c = threadIdx.x; c < nkv * vd; c += blockDim.x) {
        const int g = c / vd, e = c - g * vd;
        pv[((size_t)g * page_size + slot) * vd + e] = from_f32<T>(vrow[c]);
    }
}

AIRUN_EXPORT int airun_qk_rownorm_store(const float* proj, long long proj_stride, const float* q_w, const float* k_w, float eps,
                                        float temp_coef, int temp_every, void* q_out, void* pool, int dtype,
                                        const int32_t* block_table, int max_blocks, const int32_t* positions,
                                        const int32_t* req_of_token, int T, int num_reqs, int num_pages, int page_size,
                                        int q_width, int nkv, int kd, int vd, int store, int* err, cudaStream_t stream) {
    if (T < 0 || q_width <= 0 || nkv <= 0 || kd <= 0 || vd <= 0 || temp_every < 0 || !err || !positions || !req_of_token ||
        (store && (!pool || !block_table || page_size <= 0 || num_pages <= 0 || max_blocks <= 0)))
        return AIRUN_ERR_ARG;
    if (T == 0) return AIRUN_OK;
#define QS_LAUNCH(TT) airun_launch(qk_rownorm_store_kernel<TT>, dim3(T), dim3(256), 0, stream, proj, proj_stride, q_w, k_w, eps, \
        temp_coef, temp_every, (TT*)q_out, (TT*)pool, block_table, max_blocks, positions, req_of_token, num_reqs, num_pages, \
        page_size, q_width, nkv, kd, vd, store, err)
    if (dtype == AIRUN_DT_F32) QS_LAUNCH(float);
    else if (dtype == AIRUN_DT_BF16) QS_LAUNCH(__nv_bfloat16);
    else return AIRUN_ERR_UNSUPPORTED;
#undef QS_LAUNCH
    return airun_launch_status();
}

// One block per (token, query head).  Each warp walks every SA_WARPS-th visible key and adds sigmoid(s) v to its
// accumulator; the warps' sums are added in warp order at the end.  A token's result depends only on its own q,
// its position and the keys it sees.
template <typename T>
__global__ __launch_bounds__(32 * SA_WARPS) void sigmoid_attention_kernel(
    const T* __restrict__ q, T* __restrict__ out, long long out_stride, const T* __restrict__ pool,
    const int32_t* __restrict__ block_table, int max_blocks, const int32_t* __restrict__ positions,
    const int32_t* __restrict__ req_of_token, int num_reqs, int num_pages, int page_size, int nh, int nkv, int D, int Dv,
    float scale, const float* __restrict__ dist_a, const float* __restrict__ dist_b, const float* __restrict__ head_c,
    int window, int* __restrict__ err) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float s_acc[];           // [SA_WARPS][Dv]
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
    float qr[SA_MAX_PER_LANE], acc[SA_MAX_PER_LANE];
#pragma unroll
    for (int i = 0; i < SA_MAX_PER_LANE; ++i) {
        const int d = lane + i * 32;
        qr[i] = d < D ? to_f32<T>(qv[d]) : 0.0f;
        acc[i] = 0.0f;
    }
    const float a = dist_a ? dist_a[head] : 0.0f, b = dist_a ? dist_b[head] : 0.0f, c = head_c ? head_c[head] : 0.0f;
    const int32_t* bt = block_table + (size_t)req * max_blocks;
    const int begin = window > 0 ? max(0, pos - window + 1) : 0;
    bool bad = false;
    const size_t page_elems = (size_t)nkv * page_size * (D + Dv);
    for (int j = begin + warp; j <= pos; j += SA_WARPS) {
        const int blk = j / page_size;
        const int page = blk < max_blocks ? bt[blk] : -1;
        if (page < 0 || page >= num_pages) { bad = true; continue; }
        const T* pk = pool + (size_t)page * page_elems;
        const T* kj = pk + ((size_t)kvh * page_size + (j - blk * page_size)) * D;
        const T* vj = pk + (size_t)nkv * page_size * D + ((size_t)kvh * page_size + (j - blk * page_size)) * Dv;
        float dot = 0.0f;
#pragma unroll
        for (int i = 0; i < SA_MAX_PER_LANE; ++i) {
            const int d = lane + i * 32;
            if (d < D) dot = fmaf(qr[i], to_f32<T>(kj[d]), dot);
        }
        float s = warp_sum(dot) * scale + c;
        if (dist_a) s -= a * logf(1.0f + b * (float)(pos - j));
        const float w = 1.0f / (1.0f + expf(-s));
#pragma unroll
        for (int i = 0; i < SA_MAX_PER_LANE; ++i) {
            const int d = lane + i * 32;
            if (d < Dv) acc[i] = fmaf(w, to_f32<T>(vj[d]), acc[i]);
        }
    }
    if (bad && lane == 0) atomicOr(err, AIRUN_DEV_BAD_PAGE);
#pragma unroll
    for (int i = 0; i < SA_MAX_PER_LANE; ++i) {
        const int d = lane + i * 32;
        if (d < Dv) s_acc[(size_t)warp * Dv + d] = acc[i];
    }
    __syncthreads();
    for (int d = threadIdx.x; d < Dv; d += blockDim.x) {
        float o = 0.0f;
#pragma unroll
        for (int w = 0; w < SA_WARPS; ++w) o += s_acc[(size_t)w * Dv + d];
        dst[d] = from_f32<T>(o);
    }
}

AIRUN_EXPORT int airun_sigmoid_attention(const void* q, void* out, long long out_stride, const void* pool, int dtype,
                                         const int32_t* block_table, int max_blocks, const int32_t* positions,
                                         const int32_t* req_of_token, int T, int num_reqs, int num_pages, int page_size,
                                         int nh, int nkv, int D, int Dv, float scale, const float* dist_a, const float* dist_b,
                                         const float* head_c, int window, int* err, cudaStream_t stream) {
    if (T < 0 || nh <= 0 || nkv <= 0 || nh % nkv != 0 || D <= 0 || D > 32 * SA_MAX_PER_LANE || Dv <= 0 ||
        Dv > 32 * SA_MAX_PER_LANE || page_size <= 0 || num_pages <= 0 || max_blocks <= 0 || window < 0 || !err || nh > 65535 ||
        out_stride < (long long)nh * Dv || (dist_a && !dist_b))
        return AIRUN_ERR_ARG;
    if (T == 0) return AIRUN_OK;
    dim3 grid(T, nh);
    const size_t smem = (size_t)SA_WARPS * Dv * sizeof(float);
#define SA_LAUNCH(TT) airun_launch(sigmoid_attention_kernel<TT>, grid, dim3(32 * SA_WARPS), smem, stream, (const TT*)q, (TT*)out, \
        out_stride, (const TT*)pool, block_table, max_blocks, positions, req_of_token, num_reqs, num_pages, page_size, nh, nkv, D, Dv, \
        scale, dist_a, dist_b, head_c, window, err)
    if (dtype == AIRUN_DT_F32) SA_LAUNCH(float);
    else if (dtype == AIRUN_DT_BF16) SA_LAUNCH(__nv_bfloat16);
    else return AIRUN_ERR_UNSUPPORTED;
#undef SA_LAUNCH
    return airun_launch_status();
}
