// Gated linear attention: a matrix-valued state per head that decays channel by channel.
//
// Per head, with key channels d < D and value channels j < Dv, for the tokens of a request in order:
//     S[d][j] <- a_t[d] * S[d][j] + k_t[d] * v_t[j]          o_t[j] = sum_d S[d][j] * q_t[d] * q_scale
// (the output uses the state AFTER the token's own update).  The decay a_t[d] lies in (0, 1):
//     a_t = sigmoid(z_t)^(1/tau),  z_t = W2 (low_t) + bias,   low_t = the low-rank projection of the input,
// computed as  a = exp(logsigmoid(z) / tau)  (decay_kernel).
// Then, per head, o_t is divided by its root mean square over Dv (eps inside the root), multiplied by a
// weight vector shared by the heads and by silu of a gate projection (out_gate_kernel).
//
// State, decays, the recurrence and the norm are float32 whatever the storage of the activations.  The
// state of a request lives in its slot of the state tensor between steps, stored per head as [D][Dv]
// (a row per key channel, the value columns side by side), and is zero when the request starts.  The result
// at a token depends only on the request's tokens up to it, not on how they were cut into steps or on
// what else is in the batch: the recurrence runs token by token in every case.
#include "common.cuh"

// a[t][c] = exp(logsigmoid(bias[c] + sum_j low[t][j] * w2[c][j]) / tau) for c < n (= heads * D).
// The same kernel serves every second half of a low-rank pair that ends in a function of its own, in float32:
// with z = bias[c] + sum_j f(low[t][j]) * w2[c][j] (f the identity, or tanh when `in_tanh`),
//   LOWRANK_POW_SIGMOID   sigmoid(z)^(1/tau)
//   LOWRANK_EXP_SOFTPLUS  exp(-exp(p[c / group]) * softplus(z))     (p: one number per group of channels)
//   LOWRANK_SIGMOID       sigmoid(z)
//   LOWRANK_EXP_NEG_EXP   exp(-exp(z))
#define LOWRANK_POW_SIGMOID 0
#define LOWRANK_EXP_SOFTPLUS 1
#define LOWRANK_SIGMOID 2
#define LOWRANK_EXP_NEG_EXP 3
#define DECAY_TOKENS 8        // tokens of one block: a row of w2 is read once for all of them
template <typename TW>
__global__ __launch_bounds__(128) void decay_kernel(const float* __restrict__ low, long long low_stride, const TW* __restrict__ w2,
                                                    const float* __restrict__ bias, float* __restrict__ out, int T, int n, int rank,
                                                    float inv_tau, const int32_t* __restrict__ req_of_token,
                                                    int mode, int in_tanh, const float* __restrict__ group_param, int group) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float s_low[];                       // [DECAY_TOKENS][rank]
    const int t0 = blockIdx.x * DECAY_TOKENS, nt = min(DECAY_TOKENS, T - t0);
    for (int e = threadIdx.x; e < nt * rank; e += blockDim.x) {
        const int tk = e / rank, j = e - tk * rank;
        const float lv = low[(size_t)(t0 + tk) * low_stride + j];
        s_low[e] = in_tanh ? tanhf(lv) : lv;
    }
    __syncthreads();
    const int c = blockIdx.y * blockDim.x + threadIdx.x;       // a channel a thread
    if (c < n) {
        float z[DECAY_TOKENS];
        const float b = bias ? bias[c] : 0.0f;
#pragma unroll
        for (int tk = 0; tk < DECAY_TOKENS; ++tk) z[tk] = b;
        const TW* wr = w2 + (size_t)c * rank;
        for (int j = 0; j < rank; ++j) {
            const float w = to_f32<TW>(wr[j]);
#pragma unroll
            for (int tk = 0; tk < DECAY_TOKENS; ++tk)
                if (tk < nt) z[tk] = fmaf(s_low[tk * rank + j], w, z[tk]);
        }
#pragma unroll
        for (int tk = 0; tk < DECAY_TOKENS; ++tk) {
            if (tk >= nt || req_of_token[t0 + tk] < 0) continue;
            const float zz = z[tk], l1p = log1pf(expf(-fabsf(zz)));
            float r;
            if (mode == LOWRANK_POW_SIGMOID) r = expf((fminf(zz, 0.0f) - l1p) * inv_tau);      // logsigmoid(z) = min(z, 0) - log(1 + exp(-|z|))
            else if (mode == LOWRANK_EXP_SOFTPLUS) r = expf(-expf(group_param[c / group]) * (fmaxf(zz, 0.0f) + l1p));
            else if (mode == LOWRANK_SIGMOID) r = 1.0f / (1.0f + expf(-zz));
            else r = expf(-expf(zz));
            out[(size_t)(t0 + tk) * n + c] = r;
        }
    }
}

AIRUN_EXPORT int airun_lowrank_act(const float* low, long long low_stride, const void* w2, int w_dtype, const float* bias,
                                   float* out, int T, int n, int rank, float tau, const int32_t* req_of_token,
                                   int mode, int in_tanh, const float* group_param, int group, cudaStream_t stream) {
    if (T < 0 || n <= 0 || n > 65535 * 128 || rank <= 0 || rank > 1024 || !(tau > 0.0f) || !req_of_token || mode < 0 || mode > 3)
        return AIRUN_ERR_ARG;
    if (mode == LOWRANK_EXP_SOFTPLUS && (!group_param || group <= 0)) return AIRUN_ERR_ARG;
    if (T == 0) return AIRUN_OK;
    const size_t smem = (size_t)DECAY_TOKENS * rank * sizeof(float);
    const int blocks = ceil_div_i(T, DECAY_TOKENS);
    if (w_dtype == AIRUN_DT_F32)
        airun_launch(decay_kernel<float>, dim3(blocks, ceil_div_i(n, 128)), dim3(128), smem, stream, low, low_stride, (const float*)w2, bias, out, T, n, rank, 1.0f / tau, req_of_token, mode, in_tanh, group_param, group);
    else if (w_dtype == AIRUN_DT_BF16)
        airun_launch(decay_kernel<__nv_bfloat16>, dim3(blocks, ceil_div_i(n, 128)), dim3(128), smem, stream, low, low_stride, (const __nv_bfloat16*)w2, bias, out, T, n, rank, 1.0f / tau, req_of_token, mode, in_tanh, group_param, group);
    else
        return AIRUN_ERR_UNSUPPORTED;
    return airun_launch_status();
}

AIRUN_EXPORT int airun_gla_decay(const float* low, long long low_stride, const void* w2, int w_dtype, const float* bias,
                                 float* out, int T, int n, int rank, float tau, const int32_t* req_of_token,
                                 cudaStream_t stream) {
    return airun_lowrank_act(low, low_stride, w2, w_dtype, bias, out, T, n, rank, tau, req_of_token, LOWRANK_POW_SIGMOID, 0,
                             nullptr, 0, stream);
}

// The recurrence.  One block per (request, head, 32 value columns), 256 threads: a lane owns a column
// and a warp owns NS key channels d = warp * NS + i, so a thread keeps NS elements of the state in
// registers for the whole step, and q, k and the decay of a token are the same for all lanes of a warp:
// they come from shared memory as float4 that every lane reads at one address (one access for the warp).
// The tokens of the request are staged through shared memory a few at a time by asynchronous copies
// (16 bytes each where the rows allow it) into one of two stages, so that the next tokens are on their way
// while these are used.  Each warp leaves its partial sums over its key channels in shared
// memory, and the eight partial sums of every (token, column) of the stage are added together, in warp
// order, once the stage's tokens are through: nothing but the state itself chains one token to the next.
#define GLA_COLS 32
#define GLA_WARPS 8
__device__ __forceinline__ void gla_cp4(float* smem, const float* gmem) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void gla_cp16(float* smem, const float* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
// With CONST the decay is one number per head (`head_decay`), the same for every token and key channel, and nothing is
// staged for it; `in_silu` applies z * sigmoid(z) to the staged q, k and v (projections that carry their activation).
template <int NS, bool CONST>
__global__ __launch_bounds__(256) void gla_recurrent_kernel(
    const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v, long long row_stride,
    const float* __restrict__ decay, float* __restrict__ state, long long slot_stride,
    const int32_t* __restrict__ cu_tokens, const int32_t* __restrict__ state_slots, int max_slots,
    float* __restrict__ out, int heads, int D, int Dv, float q_scale, int* __restrict__ err,
    const float* __restrict__ head_decay, int in_silu) {
    pdl_trigger();
    pdl_wait();
    constexpr int DP = NS * GLA_WARPS;
    constexpr int GLA_TT = NS >= 32 ? 4 : NS >= 16 ? 8 : 16;     // tokens of a stage (static shared memory stays under 48 KB)
    __shared__ __align__(16) float s_q[2][GLA_TT][DP], s_k[2][GLA_TT][DP], s_a[2][GLA_TT][DP], s_v[2][GLA_TT][GLA_COLS];
    __shared__ float s_p[GLA_WARPS][GLA_TT][GLA_COLS];
    const int r = blockIdx.x, head = blockIdx.y, col0 = blockIdx.z * GLA_COLS;
    const int t0 = cu_tokens[r], n = cu_tokens[r + 1] - t0;
    if (n <= 0) return;
    const int slot = state_slots[r];
    if (slot < 0 || slot >= max_slots) {
        if (threadIdx.x == 0) atomicOr(err, AIRUN_DEV_BAD_REQ);
        return;
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int col = col0 + lane, d0 = warp * NS;
    const bool col_ok = col < Dv;
    // the padding beyond D and Dv is zero in both stages and is never copied into
    for (int e = threadIdx.x; e < 2 * GLA_TT * DP; e += 256) {
        (&s_q[0][0][0])[e] = 0.0f; (&s_k[0][0][0])[e] = 0.0f; (&s_a[0][0][0])[e] = 0.0f;
    }
    for (int e = threadIdx.x; e < 2 * GLA_TT * GLA_COLS; e += 256) (&s_v[0][0][0])[e] = 0.0f;
    __syncthreads();
    // 16-byte copies when every row begins on a 16-byte boundary
    const bool vec = (D % 4 == 0) && (Dv % 4 == 0) && (row_stride % 4 == 0) &&
                     ((((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)decay) & 15) == 0);
    const float dec = CONST ? head_decay[blockIdx.y] : 0.0f;
    auto stage = [&](int base, int buf) {
        const int nt = min(GLA_TT, n - base);
        if (vec) {
            const int per = D / 4, nc4 = min(GLA_COLS, Dv - col0) / 4;
            for (int e = threadIdx.x; e < nt * per; e += 256) {
                const int tt = e / per, d = (e - tt * per) * 4;
                const size_t row = (size_t)(t0 + base + tt);
                gla_cp16(&s_q[buf][tt][d], q + row * row_stride + (size_t)head * D + d);
                gla_cp16(&s_k[buf][tt][d], k + row * row_stride + (size_t)head * D + d);
                if (!CONST) gla_cp16(&s_a[buf][tt][d], decay + row * ((size_t)heads * D) + (size_t)head * D + d);
            }
            for (int e = threadIdx.x; e < nt * nc4; e += 256) {
                const int tt = e / nc4, c = (e - tt * nc4) * 4;
                gla_cp16(&s_v[buf][tt][c], v + (size_t)(t0 + base + tt) * row_stride + (size_t)head * Dv + col0 + c);
            }
        } else {
            for (int e = threadIdx.x; e < nt * D; e += 256) {
                const int tt = e / D, d = e - tt * D;
                const size_t row = (size_t)(t0 + base + tt);
                gla_cp4(&s_q[buf][tt][d], q + row * row_stride + (size_t)head * D + d);
                gla_cp4(&s_k[buf][tt][d], k + row * row_stride + (size_t)head * D + d);
                if (!CONST) gla_cp4(&s_a[buf][tt][d], decay + row * ((size_t)heads * D) + (size_t)head * D + d);
            }
            const int nc = min(GLA_COLS, Dv - col0);
            for (int e = threadIdx.x; e < nt * nc; e += 256) {
                const int tt = e / nc, c = e - tt * nc;
                gla_cp4(&s_v[buf][tt][c], v + (size_t)(t0 + base + tt) * row_stride + (size_t)head * Dv + col0 + c);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    stage(0, 0);
    // the state of this head, [D][Dv]: the lanes of a warp read one row of it side by side
    float* sbase = state + (size_t)slot * slot_stride + (size_t)head * D * Dv + (col_ok ? col : 0);
    float S[NS];
#pragma unroll
    for (int i = 0; i < NS; ++i) S[i] = (col_ok && d0 + i < D) ? sbase[(size_t)(d0 + i) * Dv] : 0.0f;
    int it = 0;
    for (int base = 0; base < n; base += GLA_TT, ++it) {
        const int buf = it & 1, nt = min(GLA_TT, n - base);
        if (base + GLA_TT < n) {
            stage(base + GLA_TT, buf ^ 1);          // that stage was last read before the barrier that ended the round before
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        if (in_silu) {
            for (int e = threadIdx.x; e < nt * DP; e += 256) {
                const float a = (&s_q[buf][0][0])[e], b = (&s_k[buf][0][0])[e];
                (&s_q[buf][0][0])[e] = a / (1.0f + expf(-a));
                (&s_k[buf][0][0])[e] = b / (1.0f + expf(-b));
            }
            for (int e = threadIdx.x; e < nt * GLA_COLS; e += 256) {
                const float a = (&s_v[buf][0][0])[e];
                (&s_v[buf][0][0])[e] = a / (1.0f + expf(-a));
            }
            __syncthreads();
        }
#pragma unroll 4
        for (int tt = 0; tt < nt; ++tt) {
            const float vj = s_v[buf][tt][lane];
            float acc0 = 0.0f, acc1 = 0.0f;
#pragma unroll
            for (int i4 = 0; i4 < NS / 4; ++i4) {
                const float4 a4 = CONST ? make_float4(dec, dec, dec, dec) : *reinterpret_cast<const float4*>(&s_a[buf][tt][d0 + 4 * i4]);
                const float4 k4 = *reinterpret_cast<const float4*>(&s_k[buf][tt][d0 + 4 * i4]);
                const float4 q4 = *reinterpret_cast<const float4*>(&s_q[buf][tt][d0 + 4 * i4]);
                S[4 * i4 + 0] = fmaf(a4.x, S[4 * i4 + 0], k4.x * vj); acc0 = fmaf(S[4 * i4 + 0], q4.x, acc0);
                S[4 * i4 + 1] = fmaf(a4.y, S[4 * i4 + 1], k4.y * vj); acc1 = fmaf(S[4 * i4 + 1], q4.y, acc1);
                S[4 * i4 + 2] = fmaf(a4.z, S[4 * i4 + 2], k4.z * vj); acc0 = fmaf(S[4 * i4 + 2], q4.z, acc0);
                S[4 * i4 + 3] = fmaf(a4.w, S[4 * i4 + 3], k4.w * vj); acc1 = fmaf(S[4 * i4 + 3], q4.w, acc1);
            }
            s_p[warp][tt][lane] = acc0 + acc1;
        }
        __syncthreads();
        for (int e = threadIdx.x; e < nt * GLA_COLS; e += 256) {
            const int tt = e / GLA_COLS, c = e - tt * GLA_COLS;
            float o = 0.0f;
#pragma unroll
            for (int w = 0; w < GLA_WARPS; ++w) o += s_p[w][tt][c];
            if (col0 + c < Dv) out[(size_t)(t0 + base + tt) * ((size_t)heads * Dv) + (size_t)head * Dv + col0 + c] = o * q_scale;
        }
        __syncthreads();
    }
    if (col_ok) {
#pragma unroll
        for (int i = 0; i < NS; ++i)
            if (d0 + i < D) sbase[(size_t)(d0 + i) * Dv] = S[i];
    }
}

static int gla_recurrent_launch(const float* q, const float* k, const float* v, long long row_stride,
                                const float* decay, const float* head_decay, int in_silu, float* state, long long slot_stride,
                                int max_slots, const int32_t* cu_tokens, const int32_t* state_slots, int num_reqs,
                                float* out, int heads, int D, int Dv, float q_scale, int* err, cudaStream_t stream) {
    if (num_reqs < 0 || heads <= 0 || D <= 0 || D > 256 || Dv <= 0 || !state || !cu_tokens || !state_slots || !err ||
        slot_stride < (long long)heads * D * Dv || heads > 65535 || (!decay && !head_decay))
        return AIRUN_ERR_ARG;
    if (num_reqs == 0) return AIRUN_OK;
    const int tiles = ceil_div_i(Dv, GLA_COLS);
    if (tiles > 65535) return AIRUN_ERR_ARG;
    dim3 grid(num_reqs, heads, tiles);
#define GLA_LAUNCH(NS, C) airun_launch(gla_recurrent_kernel<NS, C>, grid, dim3(256), 0, stream, q, k, v, row_stride, decay, state, \
        slot_stride, cu_tokens, state_slots, max_slots, out, heads, D, Dv, q_scale, err, head_decay, in_silu)
#define GLA_PICK(C) do { if (D <= 32) GLA_LAUNCH(4, C); else if (D <= 64) GLA_LAUNCH(8, C); else if (D <= 128) GLA_LAUNCH(16, C); \
        else GLA_LAUNCH(32, C); } while (0)
    if (head_decay) GLA_PICK(true);
    else GLA_PICK(false);
#undef GLA_PICK
#undef GLA_LAUNCH
    return airun_launch_status();
}

AIRUN_EXPORT int airun_gla_recurrent(const float* q, const float* k, const float* v, long long row_stride,
                                     const float* decay, float* state, long long slot_stride, int max_slots,
                                     const int32_t* cu_tokens, const int32_t* state_slots, int num_reqs,
                                     float* out, int heads, int D, int Dv, float q_scale, int* err, cudaStream_t stream) {
    if (!decay) return AIRUN_ERR_ARG;
    return gla_recurrent_launch(q, k, v, row_stride, decay, nullptr, 0, state, slot_stride, max_slots, cu_tokens, state_slots,
                                num_reqs, out, heads, D, Dv, q_scale, err, stream);
}

// The same recurrence with ONE decay per head, S <- d_h S + k v^T, o = S^T q (times q_scale); `in_silu`: q, k and v
// arrive without their activation z * sigmoid(z), which is applied as they are staged.
AIRUN_EXPORT int airun_decay_recurrent(const float* q, const float* k, const float* v, long long row_stride,
                                       const float* head_decay, int in_silu, float* state, long long slot_stride, int max_slots,
                                       const int32_t* cu_tokens, const int32_t* state_slots, int num_reqs,
                                       float* out, int heads, int D, int Dv, float q_scale, int* err, cudaStream_t stream) {
    if (!head_decay) return AIRUN_ERR_ARG;
    return gla_recurrent_launch(q, k, v, row_stride, nullptr, head_decay, in_silu, state, slot_stride, max_slots, cu_tokens,
                                state_slots, num_reqs, out, heads, D, Dv, q_scale, err, stream);
}

// out[t][c] = scale * o[t][c] / sqrt(mean_c o[t]^2 + eps) * w[c] * sigmoid(gate[t][c]) over a token's whole row of n
// numbers (all heads at once); one block per token.  o is float32 [T][n], gate float32 rows of `gate_stride`.
template <typename TOut>
__global__ __launch_bounds__(256) void rownorm_gate_kernel(const float* __restrict__ o, const float* __restrict__ gate,
                                                           long long gate_stride, const float* __restrict__ w,
                                                           TOut* __restrict__ out, long long out_stride, int n, float eps,
                                                           float scale, const int32_t* __restrict__ req_of_token) {
    pdl_trigger();
    pdl_wait();
    __shared__ float red[33];
    const int t = blockIdx.x;
    if (req_of_token[t] < 0) return;
    const float* orow = o + (size_t)t * n;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < n; c += blockDim.x) ss = fmaf(orow[c], orow[c], ss);
    ss = block_sum(ss, red);
    const float inv = scale / sqrtf(ss / (float)n + eps);
    for (int c = threadIdx.x; c < n; c += blockDim.x) {
        const float g = gate ? 1.0f / (1.0f + expf(-gate[(size_t)t * gate_stride + c])) : 1.0f;
        out[(size_t)t * out_stride + c] = from_f32<TOut>(orow[c] * inv * (w ? w[c] : 1.0f) * g);
    }
}

AIRUN_EXPORT int airun_rownorm_gate(const float* o, const float* gate, long long gate_stride, const float* w, void* out,
                                    int out_dtype, long long out_stride, int T, int n, float eps, float scale,
                                    const int32_t* req_of_token, cudaStream_t stream) {
    if (T < 0 || n <= 0 || !o || !out || !req_of_token || out_stride < n || (gate && gate_stride < n)) return AIRUN_ERR_ARG;
    if (T == 0) return AIRUN_OK;
    if (out_dtype == AIRUN_DT_F32)
        airun_launch(rownorm_gate_kernel<float>, dim3(T), dim3(256), 0, stream, o, gate, gate_stride, w, (float*)out, out_stride, n, eps, scale, req_of_token);
    else if (out_dtype == AIRUN_DT_BF16)
        airun_launch(rownorm_gate_kernel<__nv_bfloat16>, dim3(T), dim3(256), 0, stream, o, gate, gate_stride, w, (__nv_bfloat16*)out, out_stride, n, eps, scale, req_of_token);
    else
        return AIRUN_ERR_UNSUPPORTED;
    return airun_launch_status();
}

// out[t][h][j] = o[t][h][j] / sqrt(mean_j o^2 + eps) * w[j] * silu(gate[t][h][j]); one warp per (token, head).
template <typename TOut>
__global__ __launch_bounds__(128) void out_gate_kernel(const float* __restrict__ o, const float* __restrict__ gate,
                                                       long long gate_stride, const float* __restrict__ w,
                                                       TOut* __restrict__ out, long long out_stride, int T, int heads,
                                                       int Dv, float eps, const int32_t* __restrict__ req_of_token,
                                                       int gate_act, int w_per_head) {
    pdl_trigger();
    pdl_wait();
    const int unit = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (unit >= T * heads) return;
    const int t = unit / heads, h = unit - t * heads;
    if (req_of_token[t] < 0) return;
    if (w && w_per_head) w += (size_t)h * Dv;
    // the gate: silu(g) (0), sigmoid(g) (1), or g as it is (2: the caller has applied its function already)
    auto gf = [&](float g) { return gate_act == 0 ? g / (1.0f + expf(-g)) : gate_act == 1 ? 1.0f / (1.0f + expf(-g)) : g; };
    const float* orow = o + ((size_t)t * heads + h) * Dv;
    const float* grow = gate + (size_t)t * gate_stride + (size_t)h * Dv;
    TOut* dst = out + (size_t)t * out_stride + (size_t)h * Dv;
    if (Dv <= 128 && Dv % 4 == 0 && ((((uintptr_t)orow | (uintptr_t)grow) & 15) == 0)) {
        // a lane takes four values: both loads are issued before anything is used
        const bool on = lane * 4 < Dv;
        float4 ov = make_float4(0.0f, 0.0f, 0.0f, 0.0f), gv = ov, wv = make_float4(1.0f, 1.0f, 1.0f, 1.0f);
        if (on) {
            ov = *reinterpret_cast<const float4*>(orow + lane * 4);
            gv = *reinterpret_cast<const float4*>(grow + lane * 4);
            if (w) wv = make_float4(w[lane * 4], w[lane * 4 + 1], w[lane * 4 + 2], w[lane * 4 + 3]);
        }
        const float ss4 = warp_sum(ov.x * ov.x + ov.y * ov.y + ov.z * ov.z + ov.w * ov.w);
        const float inv4 = 1.0f / sqrtf(ss4 / (float)Dv + eps);
        if (on) {
            dst[lane * 4 + 0] = from_f32<TOut>(ov.x * inv4 * wv.x * gf(gv.x));
            dst[lane * 4 + 1] = from_f32<TOut>(ov.y * inv4 * wv.y * gf(gv.y));
            dst[lane * 4 + 2] = from_f32<TOut>(ov.z * inv4 * wv.z * gf(gv.z));
            dst[lane * 4 + 3] = from_f32<TOut>(ov.w * inv4 * wv.w * gf(gv.w));
        }
        return;
    }
    float ss = 0.0f;
    for (int j = lane; j < Dv; j += 32) ss = fmaf(orow[j], orow[j], ss);
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)Dv + eps);
    for (int j = lane; j < Dv; j += 32) {
        const float g = grow[j];
        dst[j] = from_f32<TOut>(orow[j] * inv * (w ? w[j] : 1.0f) * gf(g));
    }
}

AIRUN_EXPORT int airun_gla_out_gate(const float* o, const float* gate, long long gate_stride, const float* w, void* out,
                                    int out_dtype, long long out_stride, int T, int heads, int Dv, float eps,
                                    const int32_t* req_of_token, int gate_act, int w_per_head, cudaStream_t stream) {
    if (T < 0 || heads <= 0 || Dv <= 0 || !req_of_token || out_stride < (long long)heads * Dv) return AIRUN_ERR_ARG;
    if (T == 0) return AIRUN_OK;
    const int blocks = ceil_div_i((long long)T * heads, 4);
    if (out_dtype == AIRUN_DT_F32)
        airun_launch(out_gate_kernel<float>, dim3(blocks), dim3(128), 0, stream, o, gate, gate_stride, w, (float*)out, out_stride, T, heads, Dv, eps, req_of_token, gate_act, w_per_head);
    else if (out_dtype == AIRUN_DT_BF16)
        airun_launch(out_gate_kernel<__nv_bfloat16>, dim3(blocks), dim3(128), 0, stream, o, gate, gate_stride, w, (__nv_bfloat16*)out, out_stride, T, heads, Dv, eps, req_of_token, gate_act, w_per_head);
    else
        return AIRUN_ERR_UNSUPPORTED;
    return airun_launch_status();
}
