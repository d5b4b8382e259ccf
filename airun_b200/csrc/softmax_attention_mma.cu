// Softmax attention on the tensor cores (mma.sync m16n8k16, bfloat16 operands, float32 accumulation) over cache pages,
// for prompt portions (tiles of 64 tokens of one head) and for single tokens (the query heads of a KV head as the rows).  The formulas, the options and the page layout are those of
// softmax_attention.cu, its plain twin:
//
//   s_ij = scale * q_i . k_j + table[h][min(i - j, table_len - 1)]
//   o_i = out_scale * sum_j exp(s_ij) v_j / (sum_j exp(s_ij) + exp(sink_h))     over j <= i (and i - j < window)
//
// One CTA (4 warps) takes up to 64 consecutive tokens of one request and one query head; a warp owns 16 of them and
// keeps, per row, a running maximum and sum: a key tile's scores (float32, kept as log2 of the weights) lower the
// sums gathered so far to the new maximum, the weights 2^(s - max) are rounded to bfloat16 as the A operand of the
// second product, and the division by the sum, the sink and the factor come at the end.  All rows of a CTA belong to one
// head, and the distance i - j of an element depends on (row - column) alone: the 127 table entries a key tile can
// need are copied once, by one thread each, into shared memory.
//
// D and Dv are padded to the template sizes DP and DVP with zeros in shared memory, so any D, Dv up to 128 run.  A
// token's result does not depend on the other rows of its tile or on the batch: its keys are walked in tiles that
// begin at the first key its TILE can see, so the same token in another portion meets other tile borders, which moves
// the result by rounding only.
#include "common.cuh"

#define XAM_ROWS 64
#define XAM_KEYS 64
#define XAM_PAD 8
#define XAM_LOG2E 1.4426950408889634f

__device__ __forceinline__ void xam_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t xam_pack(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ void xam_cp16(void* smem, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void xam_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void xam_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
// 2^x (2^-inf = 0)
__device__ __forceinline__ float xam_exp2(float x) {
    float e;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x));
    return e;
}

// ---- bulk copies (one instruction a row, carried out by the copy engine) and the barrier that counts their bytes
__device__ __forceinline__ uint32_t xam_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void xam_mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void xam_mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void xam_mbar_arrive_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool xam_mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// false after about two seconds: the caller then gives up (all threads of the CTA together)
__device__ __forceinline__ bool xam_mbar_wait(uint32_t bar, uint32_t parity) {
    for (int i = 0; i < 64; ++i)
        if (xam_mbar_try(bar, parity)) return true;
    unsigned long long t0, t1;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
    for (;;) {
        for (int i = 0; i < 256; ++i)
            if (xam_mbar_try(bar, parity)) return true;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t1));
        if (t1 - t0 > 2000000000ull) return false;
    }
}
// bytes: a multiple of 16; both addresses on 16-byte boundaries
__device__ __forceinline__ void xam_bulk_row(void* smem, const void* gmem, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(xam_u32(smem)), "l"(gmem), "r"(bytes), "r"(bar) : "memory");
}

struct XamParams {
    const __nv_bfloat16* q;
    __nv_bfloat16* out;
    long long out_stride;
    const __nv_bfloat16* pool;
    const int32_t* block_table;
    int max_blocks;
    const int32_t* cu_tokens;
    const int32_t* context_lens;
    int num_reqs, num_pages, page_size, nh, nkv, D, Dv;
    float scale;
    const float* table;           // [nh][table_len]: added to the scaled score by distance min(i - j, table_len - 1); null: nothing
    int table_len;
    const float* sink;            // [nh]: exp(sink) joins the denominator; null: no sink
    float out_scale;
    int window;
    int skip_single;              // requests that bring ONE token are left to the kernel for single tokens
    float* partial;               // [splits][T][nh * (Dv + 2)] float32 (sums, then maximum and denominator per head), when the keys of a single token are cut over CTAs
    int splits, T;
    int* err;
};

// Copies K and V rows of key tiles from the pages into shared memory.  When D and Dv are multiples of 8 the copies
// are asynchronous 16-byte pieces; when those pieces divide the CTA's 128 threads evenly and pages are a power of
// two, a thread owns one piece (where it lies in the page and in shared memory) for every key it copies, so that a
// copy costs a page lookup and little else.  Rows beyond the last key keep what they held: their weights are zero.
template <int KS, int VS>
struct XamLoader {
    const XamParams& p;
    const int32_t* bt;
    int kvh, tid;
    bool vec, regular, is_k, bad;
    int ps_shift, key0, step, dst, stride, row;
    size_t page_elems, src;
    __device__ XamLoader(const XamParams& p_, const int32_t* bt_, int kvh_) : p(p_), bt(bt_), kvh(kvh_), tid(threadIdx.x), bad(false) {
        const int D = p.D, Dv = p.Dv;
        vec = (D % 8 == 0) && (Dv % 8 == 0);
        page_elems = (size_t)p.nkv * p.page_size * (D + Dv);
        const int lp = max(1, D / 8 + Dv / 8);
        regular = vec && lp <= 128 && 128 % lp == 0 && (p.page_size & (p.page_size - 1)) == 0;
        ps_shift = __ffs(p.page_size) - 1;
        const int u = tid % lp;
        key0 = tid / lp; step = 128 / lp;
        is_k = u < D / 8;
        dst = is_k ? u * 8 : (u - D / 8) * 8;
        stride = is_k ? KS : VS; row = is_k ? D : Dv;
        src = is_k ? (size_t)kvh * p.page_size * D + dst
                   : (size_t)p.nkv * p.page_size * D + (size_t)kvh * p.page_size * Dv + dst;
    }
    // keys kbase .. min(kbase + 63, hi) into Ks [64][KS] and Vs [64][VS]; one commit group
    __device__ __forceinline__ void load(int kbase, int hi, __nv_bfloat16* Ks, __nv_bfloat16* Vs) {
        const int nk = min(XAM_KEYS, hi - kbase + 1);
        if (regular) {
            __nv_bfloat16* d = (is_k ? Ks : Vs) + dst;
            for (int key = key0; key < nk; key += step) {
                const int j = kbase + key, blk = j >> ps_shift;
                const int page = blk < p.max_blocks ? bt[blk] : -1;
                if (page < 0 || page >= p.num_pages) { bad = true; continue; }
                xam_cp16(d + key * stride, p.pool + (size_t)page * page_elems + src + (size_t)(j & (p.page_size - 1)) * row);
            }
            xam_commit();
            return;
        }
        const int D = p.D, Dv = p.Dv;
        const int perk = vec ? D / 8 : D, perv = vec ? Dv / 8 : Dv, per = perk + perv;
        for (int e = tid; e < nk * per; e += 128) {
            const int key = e / per, u = e - key * per;
            const int j = kbase + key, blk = j / p.page_size;
            const int page = blk < p.max_blocks ? bt[blk] : -1;
            if (page < 0 || page >= p.num_pages) { bad = true; continue; }
            const __nv_bfloat16* pk = p.pool + (size_t)page * page_elems + ((size_t)kvh * p.page_size + (j - blk * p.page_size)) * D;
            const __nv_bfloat16* pv = p.pool + (size_t)page * page_elems + (size_t)p.nkv * p.page_size * D +
                                      ((size_t)kvh * p.page_size + (j - blk * p.page_size)) * Dv;
            if (vec) {
                if (u < perk) xam_cp16(Ks + key * KS + u * 8, pk + u * 8);
                else xam_cp16(Vs + key * VS + (u - perk) * 8, pv + (u - perk) * 8);
            } else if (u < perk) {
                Ks[key * KS + u] = pk[u];
            } else {
                Vs[key * VS + (u - perk)] = pv[u - perk];
            }
        }
        xam_commit();
    }
};

// ---------------------------------------------------------------------------------------------------------
// Prompt portions.  One CTA (4 warps) takes up to 64 consecutive tokens of one request and one query head; a warp
// owns 16 of them.  The CTA finds its tile by walking the requests' token counts (cu_tokens), so the launch needs
// nothing from the host but an upper bound of the tile count: ceil(T / 64) + requests.  The keys the tile can see
// are walked in tiles of 64 through two stages.  With head sizes in multiples of 8 a stage is filled by bulk copies:
// thread i asks for ONE row of the tile (key i of K, or key i - 64 of V: a page lookup and one instruction), and the
// stage's mbarrier, on which every thread arrives with the bytes it has asked for, completes when all of them have
// landed.  (Sixteen-byte cp.async pieces, sixteen a thread and tile, held all four warps up for as long as the copy
// took to be accepted: copies and products ran one after the other.)  Other head sizes are copied element by element.
template <int DP, int DVP>
__global__ __launch_bounds__(128) void softmax_attention_mma_kernel(const XamParams p) {
    pdl_trigger();
    pdl_wait();
    constexpr int QS = DP + XAM_PAD, VS = DVP + XAM_PAD;
    extern __shared__ __align__(16) unsigned char xam_smem[];
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(xam_smem);            // [64][QS]
    __nv_bfloat16* Ks0 = Qs + XAM_ROWS * QS;                                   // [2][64][QS]
    __nv_bfloat16* Vs0 = Ks0 + 2 * XAM_KEYS * QS;                              // [2][64][VS]
    float* tab = reinterpret_cast<float*>(Vs0 + 2 * XAM_KEYS * VS);            // [128]: log2(e) * table[d] by row - column + 63
    const uint32_t bar0 = xam_u32(tab + 128);                                  // two mbarriers, one a stage
    // ---- which tile (tiles later in a request see more keys: the grid is walked from its end so that they start first)
    int b = gridDim.y - 1 - blockIdx.y, req = -1, first = 0, n = 0, p0 = 0;
    for (int r = 0; r < p.num_reqs; ++r) {
        const int t0 = p.cu_tokens[r], nr = p.cu_tokens[r + 1] - t0;
        if (nr <= 0 || (p.skip_single && nr == 1)) continue;
        const int tiles = (nr + XAM_ROWS - 1) / XAM_ROWS;
        if (b < tiles) {
            req = r; first = t0 + b * XAM_ROWS; n = min(XAM_ROWS, nr - b * XAM_ROWS);
            p0 = p.context_lens[r] - nr + b * XAM_ROWS;                        // position of the tile's first token
            break;
        }
        b -= tiles;
    }
    if (req < 0) return;
    const int head = blockIdx.x, kvh = head / (p.nh / p.nkv);
    const int D = p.D, Dv = p.Dv;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    XamLoader<QS, VS> ld(p, p.block_table + (size_t)req * p.max_blocks, kvh);
    // ---- shared memory starts as zeros (the padding beyond D and Dv stays so), then the Q tile
    {
        constexpr int WORDS16 = (3 * XAM_ROWS * QS + 2 * XAM_KEYS * VS) / 8 + 128 * 4 / 16;
        uint4* z = reinterpret_cast<uint4*>(xam_smem);
        for (int e = tid; e < WORDS16; e += 128) z[e] = make_uint4(0u, 0u, 0u, 0u);
    }
    const bool bulk = ld.vec;
    if (bulk) {
        if (tid == 0) {
            xam_mbar_init(bar0, 128);
            xam_mbar_init(bar0 + 8, 128);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");       // the zeros, before the copy engine writes there
    }
    __syncthreads();
    if (ld.vec) {
        const int per = D / 8;
        for (int e = tid; e < n * per; e += 128) {
            const int row = e / per, c = (e - row * per) * 8;
            xam_cp16(Qs + row * QS + c, p.q + ((size_t)(first + row) * p.nh + head) * D + c);
        }
        xam_commit();
    } else {
        for (int e = tid; e < n * D; e += 128) {
            const int row = e / D, c = e - row * D;
            Qs[row * QS + c] = p.q[((size_t)(first + row) * p.nh + head) * D + c];
        }
    }
    const int lo = p.window > 0 ? max(0, p0 - p.window + 1) : 0;
    const int hi = p0 + n - 1;
    int pos[2], vis_lo[2];                                 // rows of this thread: warp * 16 + g and + 8
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int row = warp * 16 + g + 8 * h;
        pos[h] = row < n ? p0 + row : -1;
        vis_lo[h] = p.window > 0 ? max(0, pos[h] - p.window + 1) : 0;
    }
    float O[DVP / 8][4];
#pragma unroll
    for (int i = 0; i < DVP / 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) O[i][j] = 0.0f;
    const bool has_dist = p.table != nullptr;
    const float* table = has_dist ? p.table + (size_t)head * p.table_len : nullptr;
    const float mul = p.scale * XAM_LOG2E;                 // scores are kept as log2 of the weights
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};      // running maximum and this thread's part of the sum, per row
    // this thread's row of a tile: K of key tid (threads 0-63) or V of key tid - 64
    const bool row_k = tid < XAM_KEYS;
    const int row_key = tid & (XAM_KEYS - 1);
    const uint32_t row_bytes = (uint32_t)(row_k ? D : Dv) * 2u;
    const size_t row_off = row_k ? (size_t)kvh * p.page_size * D : (size_t)p.nkv * p.page_size * D + (size_t)kvh * p.page_size * Dv;
    const size_t page_elems = (size_t)p.nkv * p.page_size * (D + Dv);
    const int32_t* bt = p.block_table + (size_t)req * p.max_blocks;
    bool bad_page = false, gave_up = false;
    auto fill = [&](int kbase, int stage) {                // asks for the tile that begins at key kbase
        if (!bulk) {
            ld.load(kbase, hi, Ks0 + stage * XAM_KEYS * QS, Vs0 + stage * XAM_KEYS * VS);
            return;
        }
        const int j = kbase + row_key, blk = j / p.page_size;
        const int page = (j <= hi && blk < p.max_blocks) ? bt[blk] : -1;
        if (j > hi) {
            xam_mbar_arrive(bar0 + 8 * stage);
        } else if (page < 0 || page >= p.num_pages) {
            bad_page = true;
            xam_mbar_arrive(bar0 + 8 * stage);
        } else {
            xam_mbar_arrive_tx(bar0 + 8 * stage, row_bytes);
            __nv_bfloat16* dst = row_k ? Ks0 + (stage * XAM_KEYS + row_key) * QS : Vs0 + (stage * XAM_KEYS + row_key) * VS;
            xam_bulk_row(dst, p.pool + (size_t)page * page_elems + row_off + (size_t)(j - blk * p.page_size) * (row_k ? D : Dv),
                         row_bytes, bar0 + 8 * stage);
        }
    };
    fill(lo, 0);
    int it = 0;
    for (int kbase = lo; kbase <= hi; kbase += XAM_KEYS, ++it) {
        const int buf = it & 1;
        const __nv_bfloat16* Ks = Ks0 + buf * XAM_KEYS * QS;
        const __nv_bfloat16* Vs = Vs0 + buf * XAM_KEYS * VS;
        if (kbase + XAM_KEYS <= hi) fill(kbase + XAM_KEYS, buf ^ 1);
        bool landed = true;
        if (bulk) {
            if (it == 0) xam_wait<0>();                    // this thread's pieces of Q
            landed = xam_mbar_wait(bar0 + 8 * buf, (uint32_t)(it >> 1) & 1u);
        }
        // the distance terms of this tile: its last readers passed the barrier that ended the tile before
        if (has_dist && tid < 127) {
            const int d = p0 - kbase + tid - 63;
            tab[tid] = XAM_LOG2E * table[min(max(d, 0), p.table_len - 1)];
        }
        if (!__syncthreads_and(landed)) {                  // a copy that never came: every thread leaves here
            gave_up = true;
            break;
        }
        if (warp * 16 < n) {                               // a warp without rows only helps to load
            float S[XAM_KEYS / 8][4];
#pragma unroll
            for (int i = 0; i < XAM_KEYS / 8; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) S[i][j] = 0.0f;
#pragma unroll
            for (int ks = 0; ks < DP / 16; ++ks) {
                uint32_t a[4];
                const __nv_bfloat16* qa = Qs + (warp * 16 + g) * QS + ks * 16 + 2 * t;
                a[0] = *reinterpret_cast<const uint32_t*>(qa);
                a[1] = *reinterpret_cast<const uint32_t*>(qa + 8 * QS);
                a[2] = *reinterpret_cast<const uint32_t*>(qa + 8);
                a[3] = *reinterpret_cast<const uint32_t*>(qa + 8 * QS + 8);
#pragma unroll
                for (int nt = 0; nt < XAM_KEYS / 8; ++nt) {
                    const __nv_bfloat16* kb = Ks + (nt * 8 + g) * QS + ks * 16 + 2 * t;
                    xam_mma(S[nt], a, *reinterpret_cast<const uint32_t*>(kb), *reinterpret_cast<const uint32_t*>(kb + 8));
                }
            }
            // ---- weights.  The mask only where a key of the tile can be hidden from a row of this warp.
            const int row_lo = p0 + warp * 16, row_hi = min(row_lo + 15, hi);
            const int need_lo = p.window > 0 ? max(lo, row_hi - p.window + 1) : lo;
            const bool masked = kbase + XAM_KEYS - 1 > row_lo || kbase < need_lo || warp * 16 + 15 >= n;
            const float* tb = tab + warp * 16 + g + 63 - 2 * t;
            float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nt = 0; nt < XAM_KEYS / 8; ++nt)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int h = j >> 1;
                    float x = S[nt][j] * mul;
                    if (has_dist) x += tb[8 * h - nt * 8 - (j & 1)];
                    if (masked) {
                        const int key = kbase + nt * 8 + 2 * t + (j & 1);
                        x = (key <= pos[h] && key >= vis_lo[h]) ? x : -INFINITY;
                    }
                    S[nt][j] = x;
                    tmax[h] = fmaxf(tmax[h], x);
                }
            // the row's maximum so far (the four threads of a row agree on it), the old sums scaled down to it
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                tmax[h] = fmaxf(tmax[h], __shfl_xor_sync(0xffffffffu, tmax[h], 1));
                tmax[h] = fmaxf(tmax[h], __shfl_xor_sync(0xffffffffu, tmax[h], 2));
                const float m_new = fmaxf(m_run[h], tmax[h]);
                const float corr = m_new == -INFINITY ? 1.0f : xam_exp2(m_run[h] - m_new);
                m_run[h] = m_new;
                l_run[h] *= corr;
#pragma unroll
                for (int i = 0; i < DVP / 8; ++i) { O[i][2 * h] *= corr; O[i][2 * h + 1] *= corr; }
            }
#pragma unroll
            for (int nt = 0; nt < XAM_KEYS / 8; ++nt)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int h = j >> 1;
                    const float w = m_run[h] == -INFINITY ? 0.0f : xam_exp2(S[nt][j] - m_run[h]);
                    S[nt][j] = w;
                    l_run[h] += w;
                }
            // ---- O += W V
#pragma unroll
            for (int kk = 0; kk < XAM_KEYS / 16; ++kk) {
                uint32_t a[4];
                a[0] = xam_pack(S[2 * kk][0], S[2 * kk][1]);
                a[1] = xam_pack(S[2 * kk][2], S[2 * kk][3]);
                a[2] = xam_pack(S[2 * kk + 1][0], S[2 * kk + 1][1]);
                a[3] = xam_pack(S[2 * kk + 1][2], S[2 * kk + 1][3]);
#pragma unroll
                for (int nv = 0; nv < DVP / 8; ++nv) {
                    uint32_t b0, b1;                       // keys kk*16 .. +15 (rows of Vs) x columns nv*8 .. +7, transposed on the way
                    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(Vs + (kk * 16 + (lane & 15)) * VS + nv * 8);
                    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0, %1}, [%2];" : "=r"(b0), "=r"(b1) : "r"(addr));
                    xam_mma(O[nv], a, b0, b1);
                }
            }
        }
        __syncthreads();                                   // this stage and the table may be written again
    }
    if ((ld.bad || bad_page) && lane == 0) atomicOr(p.err, AIRUN_DEV_BAD_PAGE);
    if (gave_up) {
        if (tid == 0) atomicOr(p.err, AIRUN_DEV_TIMEOUT);
        return;
    }
    if (warp * 16 >= n) return;
    const float sink2 = p.sink ? p.sink[head] * XAM_LOG2E : -INFINITY;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int row = warp * 16 + g + 8 * h;
        float l = l_run[h];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        // the sink joins the denominator; if it is above every score the sums are scaled down to it
        const float top = fmaxf(m_run[h], sink2);
        const float f = top == -INFINITY ? 0.0f : xam_exp2(m_run[h] - top);
        const float den = l * f + (p.sink ? xam_exp2(sink2 - top) : 0.0f);
        const float inv = den > 0.0f ? p.out_scale * f / den : 0.0f;
        if (row >= n) continue;
        __nv_bfloat16* dst = p.out + (size_t)(first + row) * p.out_stride + (size_t)head * Dv;
#pragma unroll
        for (int i = 0; i < DVP / 8; ++i) {
            const int c = i * 8 + 2 * t;
            if (c < Dv) dst[c] = __float2bfloat16_rn(O[i][2 * h] * inv);
            if (c + 1 < Dv) dst[c + 1] = __float2bfloat16_rn(O[i][2 * h + 1] * inv);
        }
    }
}


// ---------------------------------------------------------------------------------------------------------
// Single decoded tokens.  One CTA (4 warps) per (request that brings ONE token, KV head, slice of its keys): the rows
// of the products are the G query heads of the group (up to 16), so a key or value row that is read serves all of
// them.  The slice's keys are walked in tiles of 64 through the same two stages; inside a tile warp w takes keys
// 16w .. 16w+15 with a running maximum and sum of its own per row; at the end the four warps' sums are brought to
// their common maximum and added through shared memory in warp order.  With one slice the result (with the sink, the
// division and the factor) goes to `out`; with several each slice writes its float32 sums, its maximum and its
// denominator to `partial` ([splits][T][nh * (Dv + 2)]) and xam_reduce_kernel merges them in slice order.
template <int DP, int DVP>
__global__ __launch_bounds__(128) void softmax_attention_group_kernel(const XamParams p) {
    pdl_trigger();
    pdl_wait();
    constexpr int QS = DP + XAM_PAD, VS = DVP + XAM_PAD;
    constexpr int PER = DVP / 8 * 4 + 1;                   // floats a thread hands to the merge (odd: no bank conflicts)
    extern __shared__ __align__(16) unsigned char xam_smem[];
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(xam_smem);            // [16][QS]
    __nv_bfloat16* Ks0 = Qs + 16 * QS;                                         // [2][64][QS]
    __nv_bfloat16* Vs0 = Ks0 + 2 * XAM_KEYS * QS;                              // [2][64][VS]
    const int r = blockIdx.y, kvh = blockIdx.x, slice = blockIdx.z;
    const int tok = p.cu_tokens[r];
    if (p.cu_tokens[r + 1] - tok != 1) return;
    const int pos = p.context_lens[r] - 1;                 // the token's position: the last key it sees
    const int D = p.D, Dv = p.Dv, G = p.nh / p.nkv;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    XamLoader<QS, VS> ld(p, p.block_table + (size_t)r * p.max_blocks, kvh);
    {
        constexpr int WORDS16 = ((16 + 2 * XAM_KEYS) * QS + 2 * XAM_KEYS * VS) / 8;
        uint4* z = reinterpret_cast<uint4*>(xam_smem);
        for (int e = tid; e < WORDS16; e += 128) z[e] = make_uint4(0u, 0u, 0u, 0u);
    }
    // the stages are filled by bulk copies, a row a thread, as in the tile kernel (head sizes in multiples of 8)
    const bool bulk = ld.vec;
    const uint32_t bar0 = xam_u32(Vs0 + 2 * XAM_KEYS * VS);                    // two mbarriers behind the stages
    if (bulk) {
        if (tid == 0) {
            xam_mbar_init(bar0, 128);
            xam_mbar_init(bar0 + 8, 128);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    // this slice's key tiles
    const int first_key = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    const int tiles = (pos - first_key) / XAM_KEYS + 1, per_slice = (tiles + p.splits - 1) / p.splits;
    const int lo = first_key + slice * per_slice * XAM_KEYS;
    const int hi = min(pos, first_key + (slice + 1) * per_slice * XAM_KEYS - 1);
    // a slice without keys (a short sequence cut for a long one) copies nothing: it hands on zeros, and no copy
    // may be in flight when the warps' sums go through this shared memory
    if (lo > hi) {
    } else if (ld.vec) {
        const int per = D / 8;
        for (int e = tid; e < G * per; e += 128) {
            const int row = e / per, c = (e - row * per) * 8;
            xam_cp16(Qs + row * QS + c, p.q + ((size_t)tok * p.nh + kvh * G + row) * D + c);
        }
    } else {
        for (int e = tid; e < G * D; e += 128) {
            const int row = e / D, c = e - row * D;
            Qs[row * QS + c] = p.q[((size_t)tok * p.nh + kvh * G + row) * D + c];
        }
    }
    const bool row_on[2] = {g < G, g + 8 < G};
    const bool has_dist = p.table != nullptr;
    const float* tabp[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) tabp[h] = has_dist && row_on[h] ? p.table + (size_t)(kvh * G + g + 8 * h) * p.table_len : nullptr;
    const float mul = p.scale * XAM_LOG2E;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
    float O[DVP / 8][4];
#pragma unroll
    for (int i = 0; i < DVP / 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) O[i][j] = 0.0f;
    const bool row_k = tid < XAM_KEYS;
    const int row_key = tid & (XAM_KEYS - 1);
    const uint32_t row_bytes = (uint32_t)(row_k ? D : Dv) * 2u;
    const size_t row_off = row_k ? (size_t)kvh * p.page_size * D : (size_t)p.nkv * p.page_size * D + (size_t)kvh * p.page_size * Dv;
    const size_t page_elems = (size_t)p.nkv * p.page_size * (D + Dv);
    const int32_t* bt = p.block_table + (size_t)r * p.max_blocks;
    bool bad_page = false, gave_up = false;
    auto fill = [&](int kbase, int stage) {
        if (!bulk) {
            ld.load(kbase, hi, Ks0 + stage * XAM_KEYS * QS, Vs0 + stage * XAM_KEYS * VS);
            return;
        }
        const int j = kbase + row_key, blk = j / p.page_size;
        const int page = (j <= hi && blk < p.max_blocks) ? bt[blk] : -1;
        if (j > hi) {
            xam_mbar_arrive(bar0 + 8 * stage);
        } else if (page < 0 || page >= p.num_pages) {
            bad_page = true;
            xam_mbar_arrive(bar0 + 8 * stage);
        } else {
            xam_mbar_arrive_tx(bar0 + 8 * stage, row_bytes);
            __nv_bfloat16* dst = row_k ? Ks0 + (stage * XAM_KEYS + row_key) * QS : Vs0 + (stage * XAM_KEYS + row_key) * VS;
            xam_bulk_row(dst, p.pool + (size_t)page * page_elems + row_off + (size_t)(j - blk * p.page_size) * (row_k ? D : Dv),
                         row_bytes, bar0 + 8 * stage);
        }
    };
    if (lo <= hi) {
        if (bulk) xam_commit();                            // this thread's pieces of Q
        fill(lo, 0);
    }
    int it = 0;
    for (int kbase = lo; kbase <= hi; kbase += XAM_KEYS, ++it) {
        const int buf = it & 1;
        const __nv_bfloat16* Ks = Ks0 + buf * XAM_KEYS * QS;
        const __nv_bfloat16* Vs = Vs0 + buf * XAM_KEYS * VS;
        if (kbase + XAM_KEYS <= hi) fill(kbase + XAM_KEYS, buf ^ 1);
        bool landed = true;
        if (bulk) {
            if (it == 0) xam_wait<0>();
            landed = xam_mbar_wait(bar0 + 8 * buf, (uint32_t)(it >> 1) & 1u);
        }
        if (!__syncthreads_and(landed)) {                  // a copy that never came: every thread leaves here
            gave_up = true;
            break;
        }
        const int k0 = kbase + 16 * warp;                  // this warp's sixteen keys
        if (k0 <= hi) {
            float S[2][4];
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) S[i][j] = 0.0f;
#pragma unroll
            for (int ks = 0; ks < DP / 16; ++ks) {
                uint32_t a[4];
                const __nv_bfloat16* qa = Qs + g * QS + ks * 16 + 2 * t;
                a[0] = *reinterpret_cast<const uint32_t*>(qa);
                a[1] = *reinterpret_cast<const uint32_t*>(qa + 8 * QS);
                a[2] = *reinterpret_cast<const uint32_t*>(qa + 8);
                a[3] = *reinterpret_cast<const uint32_t*>(qa + 8 * QS + 8);
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
                    const __nv_bfloat16* kb = Ks + (16 * warp + nt * 8 + g) * QS + ks * 16 + 2 * t;
                    xam_mma(S[nt], a, *reinterpret_cast<const uint32_t*>(kb), *reinterpret_cast<const uint32_t*>(kb + 8));
                }
            }
            float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int h = j >> 1, key = k0 + nt * 8 + 2 * t + (j & 1);
                    float x = S[nt][j] * mul;
                    if (row_on[h] && key <= hi) {
                        if (has_dist) x = fmaf(XAM_LOG2E, tabp[h][min(max(pos - key, 0), p.table_len - 1)], x);
                    } else {
                        x = -INFINITY;
                    }
                    S[nt][j] = x;
                    tmax[h] = fmaxf(tmax[h], x);
                }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                tmax[h] = fmaxf(tmax[h], __shfl_xor_sync(0xffffffffu, tmax[h], 1));
                tmax[h] = fmaxf(tmax[h], __shfl_xor_sync(0xffffffffu, tmax[h], 2));
                const float m_new = fmaxf(m_run[h], tmax[h]);
                const float corr = m_new == -INFINITY ? 1.0f : xam_exp2(m_run[h] - m_new);
                m_run[h] = m_new;
                l_run[h] *= corr;
#pragma unroll
                for (int i = 0; i < DVP / 8; ++i) { O[i][2 * h] *= corr; O[i][2 * h + 1] *= corr; }
            }
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int h = j >> 1;
                    const float w = m_run[h] == -INFINITY ? 0.0f : xam_exp2(S[nt][j] - m_run[h]);
                    S[nt][j] = w;
                    l_run[h] += w;
                }
            uint32_t a[4];
            a[0] = xam_pack(S[0][0], S[0][1]);
            a[1] = xam_pack(S[0][2], S[0][3]);
            a[2] = xam_pack(S[1][0], S[1][1]);
            a[3] = xam_pack(S[1][2], S[1][3]);
#pragma unroll
            for (int nv = 0; nv < DVP / 8; ++nv) {
                uint32_t b0, b1;
                const uint32_t addr = (uint32_t)__cvta_generic_to_shared(Vs + (16 * warp + (lane & 15)) * VS + nv * 8);
                asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0, %1}, [%2];" : "=r"(b0), "=r"(b1) : "r"(addr));
                xam_mma(O[nv], a, b0, b1);
            }
        }
        __syncthreads();
    }
    if ((ld.bad || bad_page) && lane == 0) atomicOr(p.err, AIRUN_DEV_BAD_PAGE);
    if (gave_up) {
        if (tid == 0) atomicOr(p.err, AIRUN_DEV_TIMEOUT);
        return;
    }
    // ---- the four warps' sums into warp 0, in warp order (the stages are free: every copy has landed)
    xam_wait<0>();
    __syncthreads();
    float* sh = reinterpret_cast<float*>(xam_smem);
    float* sh_m = sh + 128 * PER;                          // [4 warps][16 rows]: maxima, then the sums
    float* sh_l = sh_m + 64;
#pragma unroll
    for (int i = 0; i < DVP / 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) sh[(size_t)tid * PER + i * 4 + j] = O[i][j];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        float l = l_run[h];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        if (t == 0) { sh_m[warp * 16 + g + 8 * h] = m_run[h]; sh_l[warp * 16 + g + 8 * h] = l; }
    }
    __syncthreads();
    if (warp != 0) return;
    float top[2], den[2], f[2][4];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        top[h] = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) top[h] = fmaxf(top[h], sh_m[w * 16 + g + 8 * h]);
        den[h] = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float mw = sh_m[w * 16 + g + 8 * h];
            f[h][w] = mw == -INFINITY ? 0.0f : xam_exp2(mw - top[h]);
            den[h] = fmaf(sh_l[w * 16 + g + 8 * h], f[h][w], den[h]);
        }
    }
#pragma unroll
    for (int i = 0; i < DVP / 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float acc = 0.0f;
#pragma unroll
            for (int w = 0; w < 4; ++w) acc = fmaf(sh[(size_t)(w * 32 + lane) * PER + i * 4 + j], f[j >> 1][w], acc);
            O[i][j] = acc;
        }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        if (!row_on[h]) continue;
        const int head = kvh * G + g + 8 * h;
        const size_t col = (size_t)head * Dv;
        if (p.splits > 1) {
            float* base = p.partial + ((size_t)slice * p.T + tok) * ((size_t)p.nh * (Dv + 2));
            float* dst = base + col;
#pragma unroll
            for (int i = 0; i < DVP / 8; ++i) {
                const int c = i * 8 + 2 * t;
                if (c < Dv) dst[c] = O[i][2 * h];
                if (c + 1 < Dv) dst[c + 1] = O[i][2 * h + 1];
            }
            if (t == 0) {
                base[(size_t)p.nh * Dv + 2 * head] = top[h];
                base[(size_t)p.nh * Dv + 2 * head + 1] = den[h];
            }
        } else {
            const float sink2 = p.sink ? p.sink[head] * XAM_LOG2E : -INFINITY;
            const float all = fmaxf(top[h], sink2);
            const float fo = all == -INFINITY ? 0.0f : xam_exp2(top[h] - all);
            const float d = den[h] * fo + (p.sink ? xam_exp2(sink2 - all) : 0.0f);
            const float inv = d > 0.0f ? p.out_scale * fo / d : 0.0f;
            __nv_bfloat16* dst = p.out + (size_t)tok * p.out_stride + col;
#pragma unroll
            for (int i = 0; i < DVP / 8; ++i) {
                const int c = i * 8 + 2 * t;
                if (c < Dv) dst[c] = __float2bfloat16_rn(O[i][2 * h] * inv);
                if (c + 1 < Dv) dst[c + 1] = __float2bfloat16_rn(O[i][2 * h + 1] * inv);
            }
        }
    }
}

// The slices of every single token merged in slice order (each brought to the common maximum, the sink joining the
// denominator); a block per request, a head at a time per warp.
__global__ __launch_bounds__(256) void xam_reduce_kernel(const XamParams p) {
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x;
    const int tok = p.cu_tokens[r];
    if (p.cu_tokens[r + 1] - tok != 1) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, Dv = p.Dv;
    const size_t width = (size_t)p.nh * (Dv + 2);
    for (int head = warp; head < p.nh; head += 8) {
        const float sink2 = p.sink ? p.sink[head] * XAM_LOG2E : -INFINITY;
        float top = sink2;
        for (int s = 0; s < p.splits; ++s) top = fmaxf(top, p.partial[((size_t)s * p.T + tok) * width + (size_t)p.nh * Dv + 2 * head]);
        float den = p.sink ? xam_exp2(sink2 - top) : 0.0f;
        for (int s = 0; s < p.splits; ++s) {
            const float* ml = p.partial + ((size_t)s * p.T + tok) * width + (size_t)p.nh * Dv + 2 * head;
            den = fmaf(ml[1], ml[0] == -INFINITY ? 0.0f : xam_exp2(ml[0] - top), den);
        }
        const float inv = den > 0.0f ? p.out_scale / den : 0.0f;
        for (int c = lane; c < Dv; c += 32) {
            float acc = 0.0f;
            for (int s = 0; s < p.splits; ++s) {
                const float* base = p.partial + ((size_t)s * p.T + tok) * width;
                const float m = base[(size_t)p.nh * Dv + 2 * head];
                acc = fmaf(base[(size_t)head * Dv + c], m == -INFINITY ? 0.0f : xam_exp2(m - top), acc);
            }
            p.out[(size_t)tok * p.out_stride + (size_t)head * Dv + c] = __float2bfloat16_rn(acc * inv);
        }
    }
}

template <int DP, int DVP>
static int xag_launch(const XamParams& p, cudaStream_t stream) {
    const size_t tiles = (size_t)((16 + 2 * XAM_KEYS) * (DP + XAM_PAD) + 2 * XAM_KEYS * (DVP + XAM_PAD)) * sizeof(__nv_bfloat16) + 16;
    const size_t merge = (size_t)128 * (DVP / 8 * 4 + 1) * sizeof(float) + 128 * sizeof(float);
    const size_t smem = tiles > merge ? tiles : merge;
    static unsigned long long configured = 0;
    if (smem > 48 * 1024 && first_on_device(configured)) {
        cudaError_t e = cudaFuncSetAttribute(softmax_attention_group_kernel<DP, DVP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    airun_launch(softmax_attention_group_kernel<DP, DVP>, dim3(p.nkv, p.num_reqs, p.splits), dim3(128), smem, stream, p);
    int rc = airun_launch_status();
    if (rc != AIRUN_OK || p.splits <= 1) return rc;
    airun_launch(xam_reduce_kernel, dim3(p.num_reqs), dim3(256), 0, stream, p);
    return airun_launch_status();
}

template <int DP, int DVP>
static int xam_launch(const XamParams& p, int max_tiles, cudaStream_t stream) {
    const size_t smem = (size_t)(3 * XAM_ROWS * (DP + XAM_PAD) + 2 * XAM_KEYS * (DVP + XAM_PAD)) * sizeof(__nv_bfloat16) + 128 * sizeof(float) + 16;
    static unsigned long long configured = 0;
    if (smem > 48 * 1024 && first_on_device(configured)) {
        cudaError_t e = cudaFuncSetAttribute(softmax_attention_mma_kernel<DP, DVP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    if (max_tiles > 65535) return AIRUN_ERR_ARG;
    airun_launch(softmax_attention_mma_kernel<DP, DVP>, dim3(p.nh, max_tiles), dim3(128), smem, stream, p);
    return airun_launch_status();
}

static bool xam_fill(XamParams& p, const void* q, void* out, long long out_stride, const void* pool, const int32_t* block_table,
                     int max_blocks, const int32_t* cu_tokens, const int32_t* context_lens, int num_reqs, int num_pages,
                     int page_size, int nh, int nkv, int D, int Dv, float scale, const float* table, int table_len,
                     const float* sink, int window, float out_scale, int* err) {
    if (num_reqs < 0 || nh <= 0 || nkv <= 0 || nh % nkv != 0 || D <= 0 || D > 128 || Dv <= 0 || Dv > 128 || page_size <= 0 ||
        num_pages <= 0 || max_blocks <= 0 || window < 0 || !err || nh > 65535 || out_stride < (long long)nh * Dv || !cu_tokens ||
        !context_lens || (table && table_len <= 0))
        return false;
    p.q = (const __nv_bfloat16*)q; p.out = (__nv_bfloat16*)out; p.out_stride = out_stride;
    p.pool = (const __nv_bfloat16*)pool; p.block_table = block_table; p.max_blocks = max_blocks;
    p.cu_tokens = cu_tokens; p.context_lens = context_lens; p.num_reqs = num_reqs; p.num_pages = num_pages;
    p.page_size = page_size; p.nh = nh; p.nkv = nkv; p.D = D; p.Dv = Dv; p.scale = scale;
    p.table = table; p.table_len = table_len; p.sink = sink; p.out_scale = out_scale; p.window = window; p.skip_single = 0;
    p.partial = nullptr; p.splits = 1; p.T = 0; p.err = err;
    return true;
}

#define XAM_CASES(CALL)                                                              \
    const int dp = D <= 32 ? 32 : D <= 64 ? 64 : 128, dvp = Dv <= 32 ? 32 : Dv <= 64 ? 64 : 128; \
    if (dp == 32 && dvp == 32) return CALL(32, 32);                                  \
    if (dp == 32 && dvp == 64) return CALL(32, 64);                                  \
    if (dp == 32 && dvp == 128) return CALL(32, 128);                                \
    if (dp == 64 && dvp == 32) return CALL(64, 32);                                  \
    if (dp == 64 && dvp == 64) return CALL(64, 64);                                  \
    if (dp == 64 && dvp == 128) return CALL(64, 128);                                \
    if (dp == 128 && dvp == 32) return CALL(128, 32);                                \
    if (dp == 128 && dvp == 64) return CALL(128, 64);                                \
    if (dp == 128 && dvp == 128) return CALL(128, 128);                              \
    return AIRUN_ERR_UNSUPPORTED

// Prompt portions (and, with skip_single == 0, single tokens too).  max_tiles: an upper bound of the number of 64-token
// tiles of the batch, e.g. ceil(T / 64) + requests.  q [T][nh * D] and out (rows of out_stride) are bfloat16, like the pages.
AIRUN_EXPORT int airun_softmax_attention_mma(const void* q, void* out, long long out_stride, const void* pool,
                                             const int32_t* block_table, int max_blocks, const int32_t* cu_tokens,
                                             const int32_t* context_lens, int num_reqs, int max_tiles, int num_pages,
                                             int page_size, int nh, int nkv, int D, int Dv, float scale, const float* table,
                                             int table_len, const float* sink, int window, float out_scale, int skip_single,
                                             int* err, cudaStream_t stream) {
    XamParams p;
    if (max_tiles < 0 || !xam_fill(p, q, out, out_stride, pool, block_table, max_blocks, cu_tokens, context_lens, num_reqs, num_pages,
                                   page_size, nh, nkv, D, Dv, scale, table, table_len, sink, window, out_scale, err))
        return AIRUN_ERR_ARG;
    if (num_reqs == 0 || max_tiles == 0) return AIRUN_OK;
    p.skip_single = skip_single;
#define XAM_TILE(A, B) xam_launch<A, B>(p, max_tiles, stream)
    XAM_CASES(XAM_TILE);
#undef XAM_TILE
}

// The single tokens of the batch (groups of up to 16 query heads a KV head).  splits > 1: the keys of a token are cut
// into that many slices, and `partial` holds splits * T * nh * (Dv + 2) floats.
AIRUN_EXPORT int airun_softmax_attention_group(const void* q, void* out, long long out_stride, const void* pool,
                                               const int32_t* block_table, int max_blocks, const int32_t* cu_tokens,
                                               const int32_t* context_lens, int num_reqs, int num_pages, int page_size,
                                               int nh, int nkv, int D, int Dv, float scale, const float* table, int table_len,
                                               const float* sink, int window, float out_scale, int splits, float* partial,
                                               int T, int* err, cudaStream_t stream) {
    XamParams p;
    if (!xam_fill(p, q, out, out_stride, pool, block_table, max_blocks, cu_tokens, context_lens, num_reqs, num_pages, page_size,
                  nh, nkv, D, Dv, scale, table, table_len, sink, window, out_scale, err) ||
        nh / nkv > 16 || num_reqs > 65535 || splits < 1 || splits > 65535 || (splits > 1 && (!partial || T <= 0)))
        return AIRUN_ERR_ARG;
    if (num_reqs == 0) return AIRUN_OK;
    p.splits = splits; p.partial = partial; p.T = T;
#define XAM_GROUP(A, B) xag_launch<A, B>(p, stream)
    XAM_CASES(XAM_GROUP);
#undef XAM_GROUP
}
