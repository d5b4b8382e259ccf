// Attention without softmax on the tensor cores (mma.sync m16n8k16, bfloat16 operands, float32 accumulation), for
// prompt portions and for single decoded tokens.  The formulas and the page layout are those of
// sigmoid_attention.cu, its plain twin:
//
//   s_ij = scale * q_i . k_j - a_h * ln(1 + b_h * (i - j)) + c_h,   o_i = sum over visible j of sigmoid(s_ij) v_j
//
// Nothing is normalised over the keys, so there is no running maximum and no rescaling: a key tile's weights are
// formed in float32 from the float32 scores, rounded to bfloat16 as the A operand of the second product, and
// added.  The weight is 1 / (1 + 2^x) with x = -log2(e) (scale * qk + c) + a * log2(1 + b * d): one ex2 and one
// rcp per score.  In the tile kernel all rows of a CTA belong to one head, and the distance d = i - j of an
// element depends on (row - column) alone: the 127 values of a * log2(1 + b * d) of a key tile are worked out once,
// by one thread each, into shared memory.  In the kernel for single tokens the rows of a CTA are the query heads
// of a KV head, each with numbers of its own, and the logarithm is taken per score (sixteen keys a warp).
//
// D and Dv are padded to the template sizes DP and DVP with zeros in shared memory, so any D, Dv up to 128 run.
// A token's result does not depend on the other rows of its tile or on the batch; keys are added in position
// order inside a warp, and warps and key splits in their fixed order.
#include "common.cuh"

#define SAM_ROWS 64
#define SAM_KEYS 64
#define SAM_PAD 8
#define SAM_LOG2E 1.4426950408889634f

__device__ __forceinline__ void sam_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t sam_pack(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ void sam_cp16(void* smem, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void sam_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void sam_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
// 1 / (1 + 2^x): 2^x = inf gives 0, 2^x = 0 gives 1
__device__ __forceinline__ float sam_weight(float x) {
    float e, r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
    return r;
}
__device__ __forceinline__ float sam_log2(float x) {
    float r;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

// ---- bulk copies (one instruction a row, carried out by the copy engine) and the barrier that counts their bytes
__device__ __forceinline__ uint32_t sam_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void sam_mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void sam_mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void sam_mbar_arrive_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool sam_mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// false after about two seconds: the caller then gives up (all threads of the CTA together)
__device__ __forceinline__ bool sam_mbar_wait(uint32_t bar, uint32_t parity) {
    for (int i = 0; i < 64; ++i)
        if (sam_mbar_try(bar, parity)) return true;
    unsigned long long t0, t1;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
    for (;;) {
        for (int i = 0; i < 256; ++i)
            if (sam_mbar_try(bar, parity)) return true;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t1));
        if (t1 - t0 > 2000000000ull) return false;
    }
}
// bytes: a multiple of 16; both addresses on 16-byte boundaries
__device__ __forceinline__ void sam_bulk_row(void* smem, const void* gmem, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(sam_u32(smem)), "l"(gmem), "r"(bytes), "r"(bar) : "memory");
}

struct SamParams {
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
    const float* dist_a;          // null: no distance term
    const float* dist_b;
    const float* head_c;          // null: no offset
    int window;
    int skip_single;              // requests that bring ONE token are left to the kernel for single tokens
    float* partial;               // [splits][T][nh * Dv] float32, when the keys of a single token are cut over CTAs
    int splits, T;
    int* err;
};

// Copies K and V rows of key tiles from the pages into shared memory.  When D and Dv are multiples of 8 the copies
// are asynchronous 16-byte pieces; when those pieces divide the CTA's 128 threads evenly and pages are a power of
// two, a thread owns one piece (where it lies in the page and in shared memory) for every key it copies, so that a
// copy costs a page lookup and little else.  Rows beyond the last key keep what they held: their weights are zero.
template <int KS, int VS>
struct SamLoader {
    const SamParams& p;
    const int32_t* bt;
    int kvh, tid;
    bool vec, regular, is_k, bad;
    int ps_shift, key0, step, dst, stride, row;
    size_t page_elems, src;
    __device__ SamLoader(const SamParams& p_, const int32_t* bt_, int kvh_) : p(p_), bt(bt_), kvh(kvh_), tid(threadIdx.x), bad(false) {
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
        const int nk = min(SAM_KEYS, hi - kbase + 1);
        if (regular) {
            __nv_bfloat16* d = (is_k ? Ks : Vs) + dst;
            for (int key = key0; key < nk; key += step) {
                const int j = kbase + key, blk = j >> ps_shift;
                const int page = blk < p.max_blocks ? bt[blk] : -1;
                if (page < 0 || page >= p.num_pages) { bad = true; continue; }
                sam_cp16(d + key * stride, p.pool + (size_t)page * page_elems + src + (size_t)(j & (p.page_size - 1)) * row);
            }
            sam_commit();
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
                if (u < perk) sam_cp16(Ks + key * KS + u * 8, pk + u * 8);
                else sam_cp16(Vs + key * VS + (u - perk) * 8, pv + (u - perk) * 8);
            } else if (u < perk) {
                Ks[key * KS + u] = pk[u];
            } else {
                Vs[key * VS + (u - perk)] = pv[u - perk];
            }
        }
        sam_commit();
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
__global__ __launch_bounds__(128) void sigmoid_attention_mma_kernel(const SamParams p) {
    pdl_trigger();
    pdl_wait();
    constexpr int QS = DP + SAM_PAD, VS = DVP + SAM_PAD;
    extern __shared__ __align__(16) unsigned char sam_smem[];
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(sam_smem);            // [64][QS]
    __nv_bfloat16* Ks0 = Qs + SAM_ROWS * QS;                                   // [2][64][QS]
    __nv_bfloat16* Vs0 = Ks0 + 2 * SAM_KEYS * QS;                              // [2][64][VS]
    float* tab = reinterpret_cast<float*>(Vs0 + 2 * SAM_KEYS * VS);            // [128]: a * log2(1 + b * d) by row - column + 63
    const uint32_t bar0 = sam_u32(tab + 128);                                  // two mbarriers, one a stage
    // ---- which tile (tiles later in a request see more keys: the grid is walked from its end so that they start first)
    int b = gridDim.y - 1 - blockIdx.y, req = -1, first = 0, n = 0, p0 = 0;
    for (int r = 0; r < p.num_reqs; ++r) {
        const int t0 = p.cu_tokens[r], nr = p.cu_tokens[r + 1] - t0;
        if (nr <= 0 || (p.skip_single && nr == 1)) continue;
        const int tiles = (nr + SAM_ROWS - 1) / SAM_ROWS;
        if (b < tiles) {
            req = r; first = t0 + b * SAM_ROWS; n = min(SAM_ROWS, nr - b * SAM_ROWS);
            p0 = p.context_lens[r] - nr + b * SAM_ROWS;                        // position of the tile's first token
            break;
        }
        b -= tiles;
    }
    if (req < 0) return;
    const int head = blockIdx.x, kvh = head / (p.nh / p.nkv);
    const int D = p.D, Dv = p.Dv;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    SamLoader<QS, VS> ld(p, p.block_table + (size_t)req * p.max_blocks, kvh);
    // ---- shared memory starts as zeros (the padding beyond D and Dv stays so), then the Q tile
    {
        constexpr int WORDS16 = (3 * SAM_ROWS * QS + 2 * SAM_KEYS * VS) / 8 + 128 * 4 / 16;
        uint4* z = reinterpret_cast<uint4*>(sam_smem);
        for (int e = tid; e < WORDS16; e += 128) z[e] = make_uint4(0u, 0u, 0u, 0u);
    }
    const bool bulk = ld.vec;
    if (bulk) {
        if (tid == 0) {
            sam_mbar_init(bar0, 128);
            sam_mbar_init(bar0 + 8, 128);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");       // the zeros, before the copy engine writes there
    }
    __syncthreads();
    if (ld.vec) {
        const int per = D / 8;
        for (int e = tid; e < n * per; e += 128) {
            const int row = e / per, c = (e - row * per) * 8;
            sam_cp16(Qs + row * QS + c, p.q + ((size_t)(first + row) * p.nh + head) * D + c);
        }
        sam_commit();
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
    const bool has_dist = p.dist_a != nullptr;
    const float da = has_dist ? p.dist_a[head] : 0.0f, db = has_dist ? p.dist_b[head] : 0.0f;
    const float mul = -p.scale * SAM_LOG2E, add = p.head_c ? -p.head_c[head] * SAM_LOG2E : 0.0f;
    // this thread's row of a tile: K of key tid (threads 0-63) or V of key tid - 64
    const bool row_k = tid < SAM_KEYS;
    const int row_key = tid & (SAM_KEYS - 1);
    const uint32_t row_bytes = (uint32_t)(row_k ? D : Dv) * 2u;
    const size_t row_off = row_k ? (size_t)kvh * p.page_size * D : (size_t)p.nkv * p.page_size * D + (size_t)kvh * p.page_size * Dv;
    const size_t page_elems = (size_t)p.nkv * p.page_size * (D + Dv);
    const int32_t* bt = p.block_table + (size_t)req * p.max_blocks;
    bool bad_page = false, gave_up = false;
    auto fill = [&](int kbase, int stage) {                // asks for the tile that begins at key kbase
        if (!bulk) {
            ld.load(kbase, hi, Ks0 + stage * SAM_KEYS * QS, Vs0 + stage * SAM_KEYS * VS);
            return;
        }
        const int j = kbase + row_key, blk = j / p.page_size;
        const int page = (j <= hi && blk < p.max_blocks) ? bt[blk] : -1;
        if (j > hi) {
            sam_mbar_arrive(bar0 + 8 * stage);
        } else if (page < 0 || page >= p.num_pages) {
            bad_page = true;
            sam_mbar_arrive(bar0 + 8 * stage);
        } else {
            sam_mbar_arrive_tx(bar0 + 8 * stage, row_bytes);
            __nv_bfloat16* dst = row_k ? Ks0 + (stage * SAM_KEYS + row_key) * QS : Vs0 + (stage * SAM_KEYS + row_key) * VS;
            sam_bulk_row(dst, p.pool + (size_t)page * page_elems + row_off + (size_t)(j - blk * p.page_size) * (row_k ? D : Dv),
                         row_bytes, bar0 + 8 * stage);
        }
    };
    fill(lo, 0);
    int it = 0;
    for (int kbase = lo; kbase <= hi; kbase += SAM_KEYS, ++it) {
        const int buf = it & 1;
        const __nv_bfloat16* Ks = Ks0 + buf * SAM_KEYS * QS;
        const __nv_bfloat16* Vs = Vs0 + buf * SAM_KEYS * VS;
        if (kbase + SAM_KEYS <= hi) fill(kbase + SAM_KEYS, buf ^ 1);
        bool landed = true;
        if (bulk) {
            if (it == 0) sam_wait<0>();                    // this thread's pieces of Q
            landed = sam_mbar_wait(bar0 + 8 * buf, (uint32_t)(it >> 1) & 1u);
        }
        // the distance terms of this tile: its last readers passed the barrier that ended the tile before
        if (has_dist && tid < 127) {
            const int d = p0 - kbase + tid - 63;
            tab[tid] = d > 0 ? da * sam_log2(fmaf(db, (float)d, 1.0f)) : 0.0f;
        }
        if (!__syncthreads_and(landed)) {                  // a copy that never came: every thread leaves here
            gave_up = true;
            break;
        }
        if (warp * 16 < n) {                               // a warp without rows only helps to load
            float S[SAM_KEYS / 8][4];
#pragma unroll
            for (int i = 0; i < SAM_KEYS / 8; ++i)
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
                for (int nt = 0; nt < SAM_KEYS / 8; ++nt) {
                    const __nv_bfloat16* kb = Ks + (nt * 8 + g) * QS + ks * 16 + 2 * t;
                    sam_mma(S[nt], a, *reinterpret_cast<const uint32_t*>(kb), *reinterpret_cast<const uint32_t*>(kb + 8));
                }
            }
            // ---- weights.  The mask only where a key of the tile can be hidden from a row of this warp.
            const int row_lo = p0 + warp * 16, row_hi = min(row_lo + 15, hi);
            const int need_lo = p.window > 0 ? max(lo, row_hi - p.window + 1) : lo;
            const bool masked = kbase + SAM_KEYS - 1 > row_lo || kbase < need_lo || warp * 16 + 15 >= n;
            const float* tb = tab + warp * 16 + g + 63 - 2 * t;
#pragma unroll
            for (int nt = 0; nt < SAM_KEYS / 8; ++nt)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int h = j >> 1;
                    float x = fmaf(S[nt][j], mul, add);
                    if (has_dist) x += tb[8 * h - nt * 8 - (j & 1)];
                    float w = sam_weight(x);
                    if (masked) {
                        const int key = kbase + nt * 8 + 2 * t + (j & 1);
                        w = (key <= pos[h] && key >= vis_lo[h]) ? w : 0.0f;
                    }
                    S[nt][j] = w;
                }
            // ---- O += W V
#pragma unroll
            for (int kk = 0; kk < SAM_KEYS / 16; ++kk) {
                uint32_t a[4];
                a[0] = sam_pack(S[2 * kk][0], S[2 * kk][1]);
                a[1] = sam_pack(S[2 * kk][2], S[2 * kk][3]);
                a[2] = sam_pack(S[2 * kk + 1][0], S[2 * kk + 1][1]);
                a[3] = sam_pack(S[2 * kk + 1][2], S[2 * kk + 1][3]);
#pragma unroll
                for (int nv = 0; nv < DVP / 8; ++nv) {
                    uint32_t b0, b1;                       // keys kk*16 .. +15 (rows of Vs) x columns nv*8 .. +7, transposed on the way
                    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(Vs + (kk * 16 + (lane & 15)) * VS + nv * 8);
                    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0, %1}, [%2];" : "=r"(b0), "=r"(b1) : "r"(addr));
                    sam_mma(O[nv], a, b0, b1);
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
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int row = warp * 16 + g + 8 * h;
        if (row >= n) continue;
        __nv_bfloat16* dst = p.out + (size_t)(first + row) * p.out_stride + (size_t)head * Dv;
#pragma unroll
        for (int i = 0; i < DVP / 8; ++i) {
            const int c = i * 8 + 2 * t;
            if (c < Dv) dst[c] = __float2bfloat16_rn(O[i][2 * h]);
            if (c + 1 < Dv) dst[c + 1] = __float2bfloat16_rn(O[i][2 * h + 1]);
        }
    }
}

// ---------------------------------------------------------------------------------------------------------
// Single decoded tokens.  One CTA (4 warps) per (request that brings ONE token, KV head, slice of its keys): the rows
// of the products are the G query heads of the group (up to 16), so a key or value row that is read serves all of
// them.  The slice's keys are walked in tiles of 64 through the same two stages; inside a tile warp w takes keys
// 16w .. 16w+15; at the end the four warps' sums are added through shared memory in warp order.  With one slice the
// result goes to `out`; with several each slice writes float32 sums to `partial` and sam_reduce_kernel adds them
// in slice order (there is no maximum to agree on: the weights are not normalised).
template <int DP, int DVP>
__global__ __launch_bounds__(128) void sigmoid_attention_group_kernel(const SamParams p) {
    pdl_trigger();
    pdl_wait();
    constexpr int QS = DP + SAM_PAD, VS = DVP + SAM_PAD;
    constexpr int PER = DVP / 8 * 4 + 1;                   // floats a thread hands to the merge (odd: no bank conflicts)
    extern __shared__ __align__(16) unsigned char sam_smem[];
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(sam_smem);            // [16][QS]
    __nv_bfloat16* Ks0 = Qs + 16 * QS;                                         // [2][64][QS]
    __nv_bfloat16* Vs0 = Ks0 + 2 * SAM_KEYS * QS;                              // [2][64][VS]
    const int r = blockIdx.y, kvh = blockIdx.x, slice = blockIdx.z;
    const int tok = p.cu_tokens[r];
    if (p.cu_tokens[r + 1] - tok != 1) return;
    const int pos = p.context_lens[r] - 1;                 // the token's position: the last key it sees
    const int D = p.D, Dv = p.Dv, G = p.nh / p.nkv;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    SamLoader<QS, VS> ld(p, p.block_table + (size_t)r * p.max_blocks, kvh);
    {
        constexpr int WORDS16 = ((16 + 2 * SAM_KEYS) * QS + 2 * SAM_KEYS * VS) / 8;
        uint4* z = reinterpret_cast<uint4*>(sam_smem);
        for (int e = tid; e < WORDS16; e += 128) z[e] = make_uint4(0u, 0u, 0u, 0u);
    }
    // the stages are filled by bulk copies, a row a thread, as in the tile kernel (head sizes in multiples of 8)
    const bool bulk = ld.vec;
    const uint32_t bar0 = sam_u32(Vs0 + 2 * SAM_KEYS * VS);                    // two mbarriers behind the stages
    if (bulk) {
        if (tid == 0) {
            sam_mbar_init(bar0, 128);
            sam_mbar_init(bar0 + 8, 128);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    // this slice's key tiles
    const int first_key = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    const int tiles = (pos - first_key) / SAM_KEYS + 1, per_slice = (tiles + p.splits - 1) / p.splits;
    const int lo = first_key + slice * per_slice * SAM_KEYS;
    const int hi = min(pos, first_key + (slice + 1) * per_slice * SAM_KEYS - 1);
    // a slice without keys (a short sequence cut for a long one) copies nothing: it hands on zeros, and no copy
    // may be in flight when the warps' sums go through this shared memory
    if (lo > hi) {
    } else if (ld.vec) {
        const int per = D / 8;
        for (int e = tid; e < G * per; e += 128) {
            const int row = e / per, c = (e - row * per) * 8;
            sam_cp16(Qs + row * QS + c, p.q + ((size_t)tok * p.nh + kvh * G + row) * D + c);
        }
    } else {
        for (int e = tid; e < G * D; e += 128) {
            const int row = e / D, c = e - row * D;
            Qs[row * QS + c] = p.q[((size_t)tok * p.nh + kvh * G + row) * D + c];
        }
    }
    const bool row_on[2] = {g < G, g + 8 < G};
    float da[2], db[2], add[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int head = kvh * G + g + 8 * h;
        da[h] = row_on[h] && p.dist_a ? p.dist_a[head] : 0.0f;
        db[h] = row_on[h] && p.dist_a ? p.dist_b[head] : 0.0f;
        add[h] = row_on[h] && p.head_c ? -p.head_c[head] * SAM_LOG2E : 0.0f;
    }
    const bool has_dist = p.dist_a != nullptr;
    const float mul = -p.scale * SAM_LOG2E;
    float O[DVP / 8][4];
#pragma unroll
    for (int i = 0; i < DVP / 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) O[i][j] = 0.0f;
    const bool row_k = tid < SAM_KEYS;
    const int row_key = tid & (SAM_KEYS - 1);
    const uint32_t row_bytes = (uint32_t)(row_k ? D : Dv) * 2u;
    const size_t row_off = row_k ? (size_t)kvh * p.page_size * D : (size_t)p.nkv * p.page_size * D + (size_t)kvh * p.page_size * Dv;
    const size_t page_elems = (size_t)p.nkv * p.page_size * (D + Dv);
    const int32_t* bt = p.block_table + (size_t)r * p.max_blocks;
    bool bad_page = false, gave_up = false;
    auto fill = [&](int kbase, int stage) {
        if (!bulk) {
            ld.load(kbase, hi, Ks0 + stage * SAM_KEYS * QS, Vs0 + stage * SAM_KEYS * VS);
            return;
        }
        const int j = kbase + row_key, blk = j / p.page_size;
        const int page = (j <= hi && blk < p.max_blocks) ? bt[blk] : -1;
        if (j > hi) {
            sam_mbar_arrive(bar0 + 8 * stage);
        } else if (page < 0 || page >= p.num_pages) {
            bad_page = true;
            sam_mbar_arrive(bar0 + 8 * stage);
        } else {
            sam_mbar_arrive_tx(bar0 + 8 * stage, row_bytes);
            __nv_bfloat16* dst = row_k ? Ks0 + (stage * SAM_KEYS + row_key) * QS : Vs0 + (stage * SAM_KEYS + row_key) * VS;
            sam_bulk_row(dst, p.pool + (size_t)page * page_elems + row_off + (size_t)(j - blk * p.page_size) * (row_k ? D : Dv),
                         row_bytes, bar0 + 8 * stage);
        }
    };
    if (lo <= hi) {
        if (bulk) sam_commit();                            // this thread's pieces of Q
        fill(lo, 0);
    }
    int it = 0;
    for (int kbase = lo; kbase <= hi; kbase += SAM_KEYS, ++it) {
        const int buf = it & 1;
        const __nv_bfloat16* Ks = Ks0 + buf * SAM_KEYS * QS;
        const __nv_bfloat16* Vs = Vs0 + buf * SAM_KEYS * VS;
        if (kbase + SAM_KEYS <= hi) fill(kbase + SAM_KEYS, buf ^ 1);
        bool landed = true;
        if (bulk) {
            if (it == 0) sam_wait<0>();
            landed = sam_mbar_wait(bar0 + 8 * buf, (uint32_t)(it >> 1) & 1u);
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
                    sam_mma(S[nt], a, *reinterpret_cast<const uint32_t*>(kb), *reinterpret_cast<const uint32_t*>(kb + 8));
                }
            }
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int h = j >> 1, key = k0 + nt * 8 + 2 * t + (j & 1);
                    float x = fmaf(S[nt][j], mul, add[h]);
                    if (has_dist) x = fmaf(da[h], sam_log2(fmaf(db[h], (float)max(pos - key, 0), 1.0f)), x);
                    S[nt][j] = (row_on[h] && key <= hi) ? sam_weight(x) : 0.0f;
                }
            uint32_t a[4];
            a[0] = sam_pack(S[0][0], S[0][1]);
            a[1] = sam_pack(S[0][2], S[0][3]);
            a[2] = sam_pack(S[1][0], S[1][1]);
            a[3] = sam_pack(S[1][2], S[1][3]);
#pragma unroll
            for (int nv = 0; nv < DVP / 8; ++nv) {
                uint32_t b0, b1;
                const uint32_t addr = (uint32_t)__cvta_generic_to_shared(Vs + (16 * warp + (lane & 15)) * VS + nv * 8);
                asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0, %1}, [%2];" : "=r"(b0), "=r"(b1) : "r"(addr));
                sam_mma(O[nv], a, b0, b1);
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
    sam_wait<0>();
    __syncthreads();
    float* sh = reinterpret_cast<float*>(sam_smem);
#pragma unroll
    for (int i = 0; i < DVP / 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) sh[(size_t)tid * PER + i * 4 + j] = O[i][j];
    __syncthreads();
    if (warp != 0) return;
#pragma unroll
    for (int i = 0; i < DVP / 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float acc = 0.0f;
#pragma unroll
            for (int w = 0; w < 4; ++w) acc += sh[(size_t)(w * 32 + lane) * PER + i * 4 + j];
            O[i][j] = acc;
        }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        if (!row_on[h]) continue;
        const size_t col = (size_t)(kvh * G + g + 8 * h) * Dv;
        if (p.splits > 1) {
            float* dst = p.partial + ((size_t)slice * p.T + tok) * ((size_t)p.nh * Dv) + col;
#pragma unroll
            for (int i = 0; i < DVP / 8; ++i) {
                const int c = i * 8 + 2 * t;
                if (c < Dv) dst[c] = O[i][2 * h];
                if (c + 1 < Dv) dst[c + 1] = O[i][2 * h + 1];
            }
        } else {
            __nv_bfloat16* dst = p.out + (size_t)tok * p.out_stride + col;
#pragma unroll
            for (int i = 0; i < DVP / 8; ++i) {
                const int c = i * 8 + 2 * t;
                if (c < Dv) dst[c] = __float2bfloat16_rn(O[i][2 * h]);
                if (c + 1 < Dv) dst[c + 1] = __float2bfloat16_rn(O[i][2 * h + 1]);
            }
        }
    }
}

// The slices of every single token added in slice order; a block per request.
__global__ __launch_bounds__(256) void sam_reduce_kernel(const SamParams p) {
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x;
    const int tok = p.cu_tokens[r];
    if (p.cu_tokens[r + 1] - tok != 1) return;
    const size_t width = (size_t)p.nh * p.Dv;
    for (size_t c = threadIdx.x; c < width; c += blockDim.x) {
        float acc = 0.0f;
        for (int s = 0; s < p.splits; ++s) acc += p.partial[((size_t)s * p.T + tok) * width + c];
        p.out[(size_t)tok * p.out_stride + c] = __float2bfloat16_rn(acc);
    }
}

template <int DP, int DVP>
static int sag_launch(const SamParams& p, cudaStream_t stream) {
    const size_t tiles = (size_t)((16 + 2 * SAM_KEYS) * (DP + SAM_PAD) + 2 * SAM_KEYS * (DVP + SAM_PAD)) * sizeof(__nv_bfloat16) + 16;
    const size_t merge = (size_t)128 * (DVP / 8 * 4 + 1) * sizeof(float);
    const size_t smem = tiles > merge ? tiles : merge;
    static unsigned long long configured = 0;
    if (smem > 48 * 1024 && first_on_device(configured)) {
        cudaError_t e = cudaFuncSetAttribute(sigmoid_attention_group_kernel<DP, DVP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    airun_launch(sigmoid_attention_group_kernel<DP, DVP>, dim3(p.nkv, p.num_reqs, p.splits), dim3(128), smem, stream, p);
    int rc = airun_launch_status();
    if (rc != AIRUN_OK || p.splits <= 1) return rc;
    airun_launch(sam_reduce_kernel, dim3(p.num_reqs), dim3(256), 0, stream, p);
    return airun_launch_status();
}

template <int DP, int DVP>
static int sam_launch(const SamParams& p, int max_tiles, cudaStream_t stream) {
    const size_t smem = (size_t)(3 * SAM_ROWS * (DP + SAM_PAD) + 2 * SAM_KEYS * (DVP + SAM_PAD)) * sizeof(__nv_bfloat16) + 128 * sizeof(float) + 16;
    static unsigned long long configured = 0;
    if (smem > 48 * 1024 && first_on_device(configured)) {
        cudaError_t e = cudaFuncSetAttribute(sigmoid_attention_mma_kernel<DP, DVP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    if (max_tiles > 65535) return AIRUN_ERR_ARG;
    airun_launch(sigmoid_attention_mma_kernel<DP, DVP>, dim3(p.nh, max_tiles), dim3(128), smem, stream, p);
    return airun_launch_status();
}

static bool sam_fill(SamParams& p, const void* q, void* out, long long out_stride, const void* pool, const int32_t* block_table,
                     int max_blocks, const int32_t* cu_tokens, const int32_t* context_lens, int num_reqs, int num_pages,
                     int page_size, int nh, int nkv, int D, int Dv, float scale, const float* dist_a, const float* dist_b,
                     const float* head_c, int window, int* err) {
    if (num_reqs < 0 || nh <= 0 || nkv <= 0 || nh % nkv != 0 || D <= 0 || D > 128 || Dv <= 0 || Dv > 128 || page_size <= 0 ||
        num_pages <= 0 || max_blocks <= 0 || window < 0 || !err || nh > 65535 || out_stride < (long long)nh * Dv || !cu_tokens ||
        !context_lens || (dist_a && !dist_b))
        return false;
    p.q = (const __nv_bfloat16*)q; p.out = (__nv_bfloat16*)out; p.out_stride = out_stride;
    p.pool = (const __nv_bfloat16*)pool; p.block_table = block_table; p.max_blocks = max_blocks;
    p.cu_tokens = cu_tokens; p.context_lens = context_lens; p.num_reqs = num_reqs; p.num_pages = num_pages;
    p.page_size = page_size; p.nh = nh; p.nkv = nkv; p.D = D; p.Dv = Dv; p.scale = scale;
    p.dist_a = dist_a; p.dist_b = dist_b; p.head_c = head_c; p.window = window; p.skip_single = 0;
    p.partial = nullptr; p.splits = 1; p.T = 0; p.err = err;
    return true;
}

#define SAM_CASES(CALL)                                                              \
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

// Prompt portions (and, with skip_single == 0, single tokens too).  max_tiles: an upper bound of the number of
// 64-token tiles of the batch, e.g. ceil(T / 64) + requests.
AIRUN_EXPORT int airun_sigmoid_attention_mma(const void* q, void* out, long long out_stride, const void* pool,
                                             const int32_t* block_table, int max_blocks, const int32_t* cu_tokens,
                                             const int32_t* context_lens, int num_reqs, int max_tiles, int num_pages,
                                             int page_size, int nh, int nkv, int D, int Dv, float scale, const float* dist_a,
                                             const float* dist_b, const float* head_c, int window, int skip_single, int* err,
                                             cudaStream_t stream) {
    SamParams p;
    if (max_tiles < 0 || !sam_fill(p, q, out, out_stride, pool, block_table, max_blocks, cu_tokens, context_lens, num_reqs,
                                   num_pages, page_size, nh, nkv, D, Dv, scale, dist_a, dist_b, head_c, window, err))
        return AIRUN_ERR_ARG;
    if (num_reqs == 0 || max_tiles == 0) return AIRUN_OK;
    p.skip_single = skip_single;
#define SAM_TILE(A, B) sam_launch<A, B>(p, max_tiles, stream)
    SAM_CASES(SAM_TILE);
#undef SAM_TILE
}

// The single tokens of the batch (groups of up to 16 query heads a KV head).  splits > 1: the keys of a token are cut
// into that many slices, and `partial` holds splits * T * nh * Dv floats.
AIRUN_EXPORT int airun_sigmoid_attention_group(const void* q, void* out, long long out_stride, const void* pool,
                                               const int32_t* block_table, int max_blocks, const int32_t* cu_tokens,
                                               const int32_t* context_lens, int num_reqs, int num_pages, int page_size,
                                               int nh, int nkv, int D, int Dv, float scale, const float* dist_a,
                                               const float* dist_b, const float* head_c, int window, int splits,
                                               float* partial, int T, int* err, cudaStream_t stream) {
    SamParams p;
    if (!sam_fill(p, q, out, out_stride, pool, block_table, max_blocks, cu_tokens, context_lens, num_reqs, num_pages,
                  page_size, nh, nkv, D, Dv, scale, dist_a, dist_b, head_c, window, err) ||
        nh / nkv > 16 || num_reqs > 65535 || splits < 1 || splits > 65535 || (splits > 1 && (!partial || T <= 0)))
        return AIRUN_ERR_ARG;
    if (num_reqs == 0) return AIRUN_OK;
    p.splits = splits; p.partial = partial; p.T = T;
#define SAM_GROUP(A, B) sag_launch<A, B>(p, stream)
    SAM_CASES(SAM_GROUP);
#undef SAM_GROUP
}
