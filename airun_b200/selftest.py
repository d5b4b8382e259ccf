"""``airun selftest``: every kernel against a plain reference of the same operation, on the GPU.

The reference ships the same kind of check as ``airun selftest --device N --verbose``
(crates/airun-cli/src/selftest.rs:13-22): each kernel is run on random inputs and compared with a
straightforward host computation, with a bound per kind of operation (RMSNorm 1e-4 relative,
selftest.rs:886; attention 1e-3 absolute in float32, selftest.rs:2876; products by a backward-error
bound, selftest.rs:388-409).  Here the plain references are float64 torch formulas on the CPU,
written out below; none of them is used by the engine.  Exit status 0 means every line says ``ok``.
"""
from __future__ import annotations

import math
import sys
from typing import Callable, List, Tuple

import numpy as np
import torch


class _Ctx:
    """The few fields of a step context the attention wrappers read."""

    def __init__(self, dev, positions, req_of_token, num_reqs, query_lens, context_lens):
        self.positions = torch.tensor(positions, dtype=torch.int32, device=dev)
        self.req_of_token = torch.tensor(req_of_token, dtype=torch.int32, device=dev)
        self.token_ids = self.positions
        self.num_reqs, self.num_tokens = num_reqs, len(positions)
        self.query_lens, self.context_lens_host = query_lens, context_lens
        self.max_context_len = max(context_lens)
        self.decode_only = all(q == 1 for q in query_lens)
        self.err = torch.zeros(1, dtype=torch.int32, device=dev)
        self.extras = {}


class _Cache:
    def __init__(self, pool, block_table, page_size):
        self.pool, self.block_table, self.page_size, self.shared = pool, block_table, page_size, False


# ----------------------------------------------------------------------------- plain references
def ref_rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    x = x.double()
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w.double()


def ref_rope_neox(x: torch.Tensor, positions, theta: float) -> torch.Tensor:
    """x [T, heads, hd]; pairs (i, i + hd/2) turned by position * theta^(-2i/hd)."""
    hd = x.shape[-1]
    half = hd // 2
    inv = torch.tensor([theta ** (-2.0 * i / hd) for i in range(half)], dtype=torch.float64)
    ang = torch.tensor(positions, dtype=torch.float64)[:, None] * inv[None, :]
    c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
    a, b = x[..., :half].double(), x[..., half:].double()
    return torch.cat([a * c - b * s, b * c + a * s], -1)


def ref_attention(q, ks, vs, req_of_token, positions, scale, window):
    """q [T, nh, hd]; ks/vs per request [n, nkv, hd]; token t sees keys j <= its position of its
    request (and j > position - window when there is a window)."""
    T, nh, hd = q.shape
    nkv = ks[0].shape[1]
    out = torch.zeros(T, nh, hd, dtype=torch.float64)
    for t in range(T):
        r, p = req_of_token[t], positions[t]
        lo = max(0, p - window + 1) if window > 0 else 0
        k, v = ks[r][lo:p + 1].double(), vs[r][lo:p + 1].double()
        for h in range(nh):
            kv = h // (nh // nkv)
            s = (k[:, kv] @ q[t, h].double()) * scale
            out[t, h] = torch.softmax(s, 0) @ v[:, kv]
    return out


def paged(ks, vs, page_size, dtype, dev, seed=0):
    """Scatters per-request keys and values into a pool through a shuffled block table; unused
    pages hold large values that must never be read."""
    nkv, hd = ks[0].shape[1:]
    blocks = [(k.shape[0] + page_size - 1) // page_size for k in ks]
    n_pages = sum(blocks) + 3
    perm = np.random.default_rng(seed).permutation(n_pages)
    pool = torch.full((n_pages, 2, nkv, page_size, hd), 1e4, dtype=torch.float32)
    bt = torch.full((len(ks), max(blocks) + 1), -1, dtype=torch.int32)
    p = 0
    for r, (k, v) in enumerate(zip(ks, vs)):
        for b in range(blocks[r]):
            page = int(perm[p])
            p += 1
            bt[r, b] = page
            n = min(page_size, k.shape[0] - b * page_size)
            pool[page, 0, :, :n] = k[b * page_size:b * page_size + n].transpose(0, 1)
            pool[page, 1, :, :n] = v[b * page_size:b * page_size + n].transpose(0, 1)
    return pool.to(dtype).to(dev), bt.to(dev)


# ----------------------------------------------------------------------------- the checks
def _rel(got: torch.Tensor, want: torch.Tensor) -> float:
    return float((got.double().cpu() - want).abs().max() / max(float(want.abs().max()), 1e-30))


def check_rmsnorm(dev) -> Tuple[float, float]:
    from .kernels import ops
    worst = 0.0
    for T, H in ((7, 1500), (600, 1024)):
        x, d, w = torch.randn(T, H) * 3, torch.randn(T, H), 1 + 0.5 * torch.rand(H)
        xd, out = x.to(dev), torch.empty(T, H, device=dev)
        ops.rmsnorm(xd, w.to(dev), 1e-5, out, delta=d.to(dev))
        worst = max(worst, _rel(out, ref_rmsnorm(x + d, w, 1e-5)), _rel(xd, (x + d).double()))
    return worst, 1e-4


def check_embedding(dev) -> Tuple[float, float]:
    from .kernels import ops
    table = torch.randn(97, 52).to(torch.bfloat16)
    ids = [3, 96, 0, 96, 17]
    out = torch.empty(5, 52, device=dev)
    ops.embed(table.to(dev), torch.tensor(ids, dtype=torch.int32, device=dev), out)
    return _rel(out, table[ids].double()), 0.0


def check_swiglu(dev) -> Tuple[float, float]:
    from .kernels import ops
    T, inter, group = 9, 96, 16
    gate, up = torch.randn(T, inter), torch.randn(T, inter)
    mixed = torch.stack([gate.view(T, -1, group), up.view(T, -1, group)], 2).reshape(T, 2 * inter)
    out = torch.empty(T, inter, device=dev)
    ops.swiglu(mixed.to(dev), out, group)
    g = gate.double()
    return _rel(out, g / (1 + torch.exp(-g)) * up.double()), 1e-6


def check_gemm_simt(dev) -> Tuple[float, float]:
    from .kernels import ops
    M, N, K = 65, 129, 100
    a, w = torch.randn(M, K), torch.randn(N, K)
    out = torch.empty(M, N, device=dev)
    ops.gemm_simt(a.to(dev), w.to(dev), out)
    want = a.double() @ w.double().T
    bound = (a.abs().double() @ w.abs().double().T)
    return float(((out.double().cpu() - want).abs() / bound).max()), K * 2.0 ** -23


def _check_gemm_tc(dev, M, N, K, epi, swap, bn, ksplit) -> Tuple[float, float]:
    from .kernels import fast
    a = torch.randn(M, K).to(torch.bfloat16)
    w = (torch.randn(N, K) * 0.05).to(torch.bfloat16)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    full = a.double() @ w.double().T
    if epi == fast.EPI_SWIGLU:
        g, u = full.view(M, -1, 2, 16)[:, :, 0].reshape(M, -1), full.view(M, -1, 2, 16)[:, :, 1].reshape(M, -1)
        want = g / (1 + torch.exp(-g)) * u
        out = torch.empty(M, N // 2, dtype=torch.bfloat16, device=dev)
    else:
        want = full
        out = torch.empty(M, N, dtype=torch.float32, device=dev)
    fast.gemm_tcgen05(a.to(dev), w.to(dev), out, epi, swap, bn, ksplit, err)
    torch.cuda.synchronize()
    if int(err.item()):
        return float("inf"), 0.0
    tol = 2.0 ** -7 if epi == fast.EPI_SWIGLU else 1e-5          # bfloat16 output, or float32 sums of exact products
    return _rel(out, want), tol


def check_gemm_tc_portion(dev):
    from .kernels import fast
    return _check_gemm_tc(dev, 300, 520, 264, fast.EPI_F32, False, 256, 1)


def check_gemm_tc_decode(dev):
    from .kernels import fast
    return _check_gemm_tc(dev, 5, 328, 1024, fast.EPI_F32, True, 16, 4)


def check_gemm_tc_swiglu(dev):
    from .kernels import fast
    return _check_gemm_tc(dev, 40, 512, 320, fast.EPI_SWIGLU, True, 64, 2)


def _attention_case(dev, dtype, hd, nh, nkv, page, lens, qlens, window=0):
    ks = [torch.randn(n, nkv, hd) for n in lens]
    vs = [torch.randn(n, nkv, hd) for n in lens]
    rot, pos = [], []
    for r, (n, q) in enumerate(zip(lens, qlens)):
        rot += [r] * q
        pos += list(range(n - q, n))
    q = torch.randn(len(pos), nh, hd)
    if dtype == torch.bfloat16:
        q, ks, vs = q.to(dtype).float(), [k.to(dtype).float() for k in ks], [v.to(dtype).float() for v in vs]
    pool, bt = paged(ks, vs, page, dtype, dev)
    ctx = _Ctx(dev, pos, rot, len(lens), qlens, lens)
    want = ref_attention(q, ks, vs, rot, pos, 1.0 / math.sqrt(hd), window)
    return ctx, _Cache(pool, bt, page), q.to(dtype).to(dev).view(len(pos), nh * hd), want.view(len(pos), nh * hd)


def check_attention_generic(dev) -> Tuple[float, float]:
    from .kernels import ops
    ctx, cache, q, want = _attention_case(dev, torch.float32, 24, 6, 3, 8, [37, 5, 64], [37, 1, 3], window=19)
    out = torch.empty_like(q)
    ops.attention_generic(q, out, cache.pool, cache.block_table, ctx.positions, ctx.req_of_token, ctx.num_reqs,
                          6, 3, 24, 1.0 / math.sqrt(24), 19, ctx.err)
    return float((out.double().cpu() - want).abs().max()), 1e-3 if not int(ctx.err.item()) else 0.0


def check_attention_tensor_core(dev) -> Tuple[float, float]:
    """Prompt portions and decoded tokens in one batch: tcgen05 prefill and split-K decode."""
    from .kernels import fast
    hd, nh, nkv = 128, 8, 2
    ctx, cache, q, want = _attention_case(dev, torch.bfloat16, hd, nh, nkv, 16, [300, 170, 41, 999], [300, 1, 33, 1])
    out = torch.zeros_like(q)
    if not fast.attention_bf16(ctx, q, out, cache, nh, nkv, hd, 1.0 / math.sqrt(hd), 0):
        return float("inf"), 0.0
    torch.cuda.synchronize()
    return float((out.double().cpu() - want).abs().max()), 2e-2 if not int(ctx.err.item()) else 0.0


def check_attention_mma(dev) -> Tuple[float, float]:
    """A head size the tcgen05 kernel does not take: the mma.sync kernels."""
    from .kernels import fast
    hd, nh, nkv = 48, 6, 3
    ctx, cache, q, want = _attention_case(dev, torch.bfloat16, hd, nh, nkv, 8, [150, 70, 9], [150, 1, 9], window=40)
    out = torch.zeros_like(q)
    if not fast.attention_bf16(ctx, q, out, cache, nh, nkv, hd, 1.0 / math.sqrt(hd), 40):
        return float("inf"), 0.0
    torch.cuda.synchronize()
    return float((out.double().cpu() - want).abs().max()), 2e-2 if not int(ctx.err.item()) else 0.0


def check_qkv_post(dev) -> Tuple[float, float]:
    from .kernels import ops
    nh, nkv, hd, page, theta, eps = 6, 3, 48, 16, 1e6, 1e-6
    lens, qlens = [21, 7], [5, 7]
    rot, pos = [], []
    for r, (n, q) in enumerate(zip(lens, qlens)):
        rot += [r] * q
        pos += list(range(n - q, n))
    T = len(pos)
    qkv = torch.randn(T, (nh + 2 * nkv) * hd)
    qw, kw = 1 + 0.3 * torch.rand(hd), 1 + 0.3 * torch.rand(hd)
    n_pages = 6
    pool = torch.zeros(n_pages, 2, nkv, page, hd, device=dev)
    bt = torch.tensor([[4, 1, -1], [2, -1, -1]], dtype=torch.int32, device=dev)
    q_out = torch.empty(T, nh * hd, device=dev)
    inv = torch.tensor([theta ** (-2.0 * i / hd) for i in range(hd // 2)], dtype=torch.float64).float().to(dev)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    ops.qkv_post(qkv.to(dev), q_out, qw.to(dev), kw.to(dev), eps, torch.tensor(pos, dtype=torch.int32, device=dev),
                 torch.tensor(rot, dtype=torch.int32, device=dev), ops.ROPE_NEOX, hd, inv, pool, bt, 2, page,
                 nh, nkv, hd, err)
    q = qkv[:, :nh * hd].view(T, nh, hd)
    k = qkv[:, nh * hd:(nh + nkv) * hd].view(T, nkv, hd)
    v = qkv[:, (nh + nkv) * hd:].view(T, nkv, hd)
    want_q = ref_rope_neox(ref_rmsnorm(q, qw, eps), pos, theta).view(T, nh * hd)
    want_k = ref_rope_neox(ref_rmsnorm(k, kw, eps), pos, theta)
    worst = _rel(q_out, want_q)
    pool_c = pool.cpu().double()
    for t in range(T):
        page_id = int(bt[rot[t], pos[t] // page])
        worst = max(worst, float((pool_c[page_id, 0, :, pos[t] % page] - want_k[t]).abs().max()),
                    float((pool_c[page_id, 1, :, pos[t] % page] - v[t].double()).abs().max()))
    return worst, 1e-5 if not int(err.item()) else 0.0


def check_sampling(dev) -> Tuple[float, float]:
    """First maximum on ties; a draw at temperature T lands where the cumulative sum of
    exp((l - max) / T) over the rows' own order first reaches u times the total."""
    from .kernels import ops
    V = 5000
    logits = torch.randn(3, V)
    logits[0, 77] = logits[0, 4000] = 9.0                         # a tie: the first one wins
    out = torch.zeros(3, dtype=torch.int32, device=dev)
    temp = torch.tensor([0.0, 0.0, 0.7], device=dev)
    uni = torch.tensor([0.0, 0.0, 0.4321], device=dev)
    ops.sample(logits.to(dev), out, temp, uni)
    got = out.cpu().tolist()
    bad = 0.0
    if got[0] != 77 or got[1] != int(logits[1].argmax()):
        bad = 1.0
    p = torch.exp((logits[2].double() - logits[2].max().double()) / 0.7)
    cum = torch.cumsum(p, 0)
    want = int(torch.searchsorted(cum, 0.4321 * cum[-1]).item())
    # the kernel sums in float32: a draw that falls within rounding of an edge may land next door
    if abs(got[2] - want) > 1:
        bad = 1.0
    return bad, 0.5


def check_largest_logits(dev) -> Tuple[float, float]:
    """A row's largest logits with their ids, the largest first, equal values by ascending id."""
    from .kernels import ops
    V, n_cand = 151936, 105
    g = torch.Generator().manual_seed(7)
    logits = torch.round(torch.randn(2, V, generator=g) * 3.0)                   # few distinct values: ties at the cut
    ids = torch.zeros(2 * n_cand, dtype=torch.int32, device=dev)
    vals = torch.zeros(2 * n_cand, dtype=torch.float32, device=dev)
    flags = torch.zeros(2, dtype=torch.int32, device=dev)
    ops.largest_logits(logits.to(dev), torch.tensor([1, 0], dtype=torch.int32, device=dev), 2, n_cand, ids, vals, flags)
    bad = 0.0
    for j, r in enumerate((1, 0)):
        if int(flags[j].item()):
            continue                                                         # the caller would take the whole row
        row = logits[r].double()
        order = torch.argsort(-row, stable=True)[:n_cand]                   # value down; a stable sort keeps ids ascending
        if ids[j * n_cand:(j + 1) * n_cand].cpu().tolist() != order.tolist():
            bad = 1.0
    return bad, 0.5


def check_dyt_norm(dev) -> Tuple[float, float]:
    from .kernels import ops
    worst = 0.0
    for T, H in ((5, 70), (300, 1024)):
        x, d, v = torch.randn(T, H) * 2, torch.randn(T, H), torch.randn(H)
        w, b, alpha = 1 + 0.3 * torch.randn(H), torch.randn(H), torch.tensor([0.6])
        xd, out = x.to(dev), torch.empty(T, H, device=dev)
        ops.dyt_norm(xd, alpha.to(dev), w.to(dev), b.to(dev), out, delta=d.to(dev), add_vec=v.to(dev))
        sum_ = x.double() + d.double() + v.double()
        worst = max(worst, _rel(out, torch.tanh(0.6 * sum_) * w.double() + b.double()), _rel(xd, sum_))
    return worst, 1e-5


def check_clamped_unit(dev) -> Tuple[float, float]:
    """The clamped gated unit as a kernel of its own and as the epilogue of the tcgen05 gate/up product."""
    from types import SimpleNamespace
    from .kernels import fast, ops
    T, H, inter, group, limit, slope = 70, 256, 160, 16, 1.5, 1.702
    x = (torch.randn(T, H) * 0.5).to(torch.bfloat16)
    wg, wu = (torch.randn(inter, H) * 0.2).to(torch.bfloat16), (torch.randn(inter, H) * 0.2).to(torch.bfloat16)
    g = torch.clamp(x.double() @ wg.double().T, max=limit)
    u = torch.clamp(x.double() @ wu.double().T, -limit, limit)
    want = g * torch.sigmoid(slope * g) * (u + 1)
    gu = torch.stack([(x.double() @ wg.double().T).view(T, -1, group), (x.double() @ wu.double().T).view(T, -1, group)], 2).reshape(T, 2 * inter)
    out = torch.empty(T, inter, device=dev)
    ops.glu_clamped(gu.float().to(dev), out, group, limit, slope)
    worst = _rel(out, want)
    w_gu = torch.stack([wg.view(-1, group, H), wu.view(-1, group, H)], 1).reshape(2 * inter, H).contiguous().to(dev)
    buf = torch.zeros(T, inter + 8, device=dev, dtype=torch.bfloat16)
    ctx = SimpleNamespace(err=torch.zeros(1, dtype=torch.int32, device=dev))
    if not fast.linear_glu_clamped_bf16(ctx, x.to(dev), w_gu, buf[:, 8:], group, limit, slope):
        raise RuntimeError("the fused gated unit refused sizes it should take")
    return max(worst / 50, _rel(buf[:, 8:], want)), 1.5e-2          # bfloat16 output; the float32 kernel is held to 50x less


def check_linear_attention(dev) -> Tuple[float, float]:
    from .kernels import ops
    heads, D, Dv, rank, tau, eps = 3, 40, 72, 6, 5.0, 1e-5
    lens, kd, vd = [19, 1, 33], heads * D, heads * Dv
    T = sum(lens)
    proj = torch.randn(T, 2 * kd + 2 * vd + rank)
    w2, b2, wn = torch.randn(kd, rank), torch.randn(kd) + 2, 1 + 0.2 * torch.randn(Dv)
    pd = proj.to(dev)
    cu = torch.tensor([0, 19, 20, 53], dtype=torch.int32, device=dev)
    req = torch.repeat_interleave(torch.arange(3), torch.tensor(lens)).to(dev, torch.int32)
    slots = torch.tensor([2, 0, 1], dtype=torch.int32, device=dev)
    state = torch.zeros(3, heads, D, Dv, device=dev)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    decay, o, act = torch.empty(T, kd, device=dev), torch.empty(T, vd, device=dev), torch.empty(T, vd, device=dev)
    ops.gla_decay(pd[:, 2 * kd + 2 * vd:], w2.to(dev), b2.to(dev), tau, decay, req)
    ops.gla_recurrent(pd[:, :kd], pd[:, kd:2 * kd], pd[:, 2 * kd:2 * kd + vd], decay, state, cu, slots, 3, o, heads, D, Dv, D ** -0.5, err)
    ops.gla_out_gate(o, pd[:, 2 * kd + vd:2 * kd + 2 * vd], wn.to(dev), eps, act, heads, Dv, req)
    p64, worst, at = proj.double(), 0.0, 0
    for n in lens:
        rows = p64[at:at + n]
        a = torch.exp(torch.nn.functional.logsigmoid(rows[:, 2 * kd + 2 * vd:] @ w2.double().T + b2.double()) / tau).view(n, heads, D)
        q, k = rows[:, :kd].view(n, heads, D) * D ** -0.5, rows[:, kd:2 * kd].view(n, heads, D)
        v, gate = rows[:, 2 * kd:2 * kd + vd].view(n, heads, Dv), rows[:, 2 * kd + vd:2 * kd + 2 * vd]
        S, outs = torch.zeros(heads, D, Dv, dtype=torch.float64), []
        for t in range(n):
            S = a[t].unsqueeze(-1) * S + k[t].unsqueeze(-1) * v[t].unsqueeze(-2)
            outs.append((S * q[t].unsqueeze(-1)).sum(1))
        oo = torch.stack(outs)
        oo = oo / torch.sqrt((oo * oo).mean(-1, keepdim=True) + eps) * wn.double()
        worst = max(worst, _rel(act[at:at + n], oo.reshape(n, vd) * (gate * torch.sigmoid(gate))))
        at += n
    if int(err.item()):
        raise RuntimeError("the recurrence reported a device error")
    return worst, 2e-4


def check_diff_attention(dev) -> Tuple[float, float]:
    """Differential attention over scrambled pages: the float32 kernel, then the tensor-core kernels in bfloat16
    (a whole prompt in tiles, a portion, single tokens)."""
    from types import SimpleNamespace
    from .kernels import fast, ops
    heads, kvh, D, Dv, page, chunk = 4, 2, 16, 40, 8, 29
    scale, cap, lam, eps, osc = D ** -0.5, 8.0, 0.4, 1e-5, 0.6
    lens, new = [90, 12, 41], [90, 1, 7]
    qw, kd = heads * 2 * D, 2 * D
    worst = []
    for dtype in (torch.float32, torch.bfloat16):
        g = torch.Generator().manual_seed(4)
        projs = [torch.randn(n, qw + kvh * (kd + Dv), generator=g) for n in lens]
        if dtype == torch.bfloat16:
            projs = [t.to(dtype).float() for t in projs]
        nb = [(n + page - 1) // page for n in lens]
        perm = torch.randperm(sum(nb) + 2, generator=g).tolist()
        bt = torch.full((3, max(nb)), -1, dtype=torch.int32)
        for r, n in enumerate(nb):
            for b in range(n):
                bt[r, b] = perm.pop()
        pool = torch.zeros(sum(nb) + 2, page * kvh * (kd + Dv), device=dev, dtype=dtype)
        err, btd = torch.zeros(1, dtype=torch.int32, device=dev), bt.to(dev)
        for phase in (0, 1):
            spans = [(0, n - m) if phase == 0 else (n - m, n) for n, m in zip(lens, new)]
            rows = [r for r, (a, b) in enumerate(spans) if b > a]
            if not rows:
                continue
            proj = torch.cat([projs[r][spans[r][0]:spans[r][1]] for r in rows]).to(dev)
            pos = torch.cat([torch.arange(*spans[r]) for r in rows]).to(dev, torch.int32)
            req = torch.cat([torch.full((spans[r][1] - spans[r][0],), r) for r in rows]).to(dev, torch.int32)
            q = torch.empty(proj.shape[0], qw, device=dev, dtype=dtype)
            ops.qkv_bias_store(proj, None, None, None, q, pool, btd, pos, req, 3, page, qw, kvh, kd, Dv, err)
        out = torch.empty(q.shape[0], heads * Dv, device=dev, dtype=dtype)
        if dtype == torch.float32:
            ops.diff_attention(q, out, pool, btd, pos, req, 3, page, heads, kvh, D, Dv, scale, cap, chunk, 0, lam, eps, osc, err)
        else:
            counts = [spans[r][1] - spans[r][0] for r in range(3)]
            ctx = SimpleNamespace(cu_tokens=torch.tensor([0, counts[0], counts[0] + counts[1], sum(counts)], dtype=torch.int32, device=dev),
                                  context_lens=torch.tensor(lens, dtype=torch.int32, device=dev), num_reqs=3, err=err)
            part = SimpleNamespace(D=D, Dv=Dv, nh=heads, nkv=kvh, scale=scale, cap=cap, chunk=chunk, window=0, lam=lam, eps=eps,
                                   lambda_init=1.0 - osc)
            if not fast.diff_attention_bf16(ctx, q, out, SimpleNamespace(pool=pool, block_table=btd, page_size=page), part):
                raise RuntimeError("the tensor-core attention refused sizes it should take")
        if int(err.item()):
            raise RuntimeError("the attention reported a device error")
        at, w = 0, 0.0
        for r, n in enumerate(lens):
            p64 = projs[r].double()
            qq, kk = p64[:, :qw].view(n, heads, 2, D), p64[:, qw:qw + kvh * kd].view(n, kvh, 2, D)
            vv = p64[:, qw + kvh * kd:].view(n, kvh, Dv)
            i = torch.arange(n)
            vis = (i[None, :] <= i[:, None]) & (i[None, :] // chunk == i[:, None] // chunk)
            ref = torch.zeros(n, heads, Dv, dtype=torch.float64)
            for h in range(heads):
                maps = []
                for m in range(2):
                    sc = cap * torch.tanh((qq[:, h, m] @ kk[:, h // (heads // kvh), m].T) * scale / cap)
                    maps.append(torch.softmax(sc.masked_fill(~vis, -math.inf), -1) @ vv[:, h // (heads // kvh)])
                o = maps[0] - lam * maps[1]
                ref[:, h] = o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps) * osc
            k = new[r]
            w = max(w, _rel(out[at:at + k], ref.reshape(n, -1)[n - k:]))
            at += k
        worst.append(w)
    return max(worst[0], worst[1] / 200), 1e-4                     # bfloat16 storage is held to 2e-2


def check_sigmoid_attention(dev) -> Tuple[float, float]:
    """Attention without softmax over scrambled pages (norms over the whole q and k projections, a temperature that
    steps inside the portion, a distance term and an offset per head): the float32 kernel, then the tensor-core
    kernels in bfloat16 (a whole prompt, a single token whose keys are cut into slices, a portion)."""
    from types import SimpleNamespace
    from .kernels import fast, ops
    heads, kvh, D, Dv, page = 4, 2, 24, 40, 8
    scale, eps, coef, every = 0.3, 1e-5, 0.5, 11
    lens, new = [90, 700, 41], [90, 1, 7]
    qw, kw = heads * D, kvh * D
    worst = []
    for dtype in (torch.float32, torch.bfloat16):
        g = torch.Generator().manual_seed(6)
        projs = [torch.randn(n, qw + kw + kvh * Dv, generator=g) for n in lens]
        wq, wk = 1 + 0.2 * torch.randn(qw, generator=g), 1 + 0.2 * torch.randn(kw, generator=g)
        a, b, c = 0.2 + torch.rand(heads, generator=g), 0.1 + torch.rand(heads, generator=g), -3.0 + torch.randn(heads, generator=g)
        nb = [(n + page - 1) // page for n in lens]
        perm = torch.randperm(sum(nb) + 2, generator=g).tolist()
        bt = torch.full((3, max(nb)), -1, dtype=torch.int32)
        for r, n in enumerate(nb):
            for blk in range(n):
                bt[r, blk] = perm.pop()
        cache = SimpleNamespace(pool=torch.zeros(sum(nb) + 2, page * kvh * (D + Dv), device=dev, dtype=dtype),
                                block_table=bt.to(dev), page_size=page, shared=False)
        err = torch.zeros(1, dtype=torch.int32, device=dev)
        for phase in (0, 1):
            spans = [(0, n - m) if phase == 0 else (n - m, n) for n, m in zip(lens, new)]
            counts = [hi - lo for lo, hi in spans]
            if not sum(counts):
                continue
            proj = torch.cat([projs[r][lo:hi] for r, (lo, hi) in enumerate(spans)]).to(dev)
            cu = [0]
            for n in counts:
                cu.append(cu[-1] + n)
            ctx = SimpleNamespace(
                positions=torch.cat([torch.arange(lo, hi) for lo, hi in spans]).to(dev, torch.int32),
                req_of_token=torch.cat([torch.full((n,), r) for r, n in enumerate(counts)]).to(dev, torch.int32),
                cu_tokens=torch.tensor(cu, dtype=torch.int32, device=dev),
                context_lens=torch.tensor([hi for _, hi in spans], dtype=torch.int32, device=dev), num_reqs=3, err=err,
                query_lens=counts, max_context_len=max(lens), extras={}, decode_only=False,
                ws=SimpleNamespace(alloc=lambda shape, dt: torch.empty(shape, device=dev, dtype=dt)))
            q = torch.empty(proj.shape[0], qw, device=dev, dtype=dtype)
            ops.qk_rownorm_store(proj, wq.to(dev), wk.to(dev), eps, coef, every, q, cache, ctx, qw, kvh, D, Dv, store=True)
        out = torch.empty(q.shape[0], heads * Dv, device=dev, dtype=dtype)
        part = SimpleNamespace(D=D, Dv=Dv, nh=heads, nkv=kvh, scale=scale, dist_a=a.to(dev), dist_b=b.to(dev), head_c=c.to(dev), window=0)
        if dtype == torch.float32:
            ops.sigmoid_attention(q, out, cache, ctx, heads, kvh, D, Dv, scale, part.dist_a, part.dist_b, part.head_c, 0)
        elif not fast.sigmoid_attention_bf16(ctx, q, out, cache, part):
            raise RuntimeError("the tensor-core attention refused sizes it should take")
        if int(err.item()):
            raise RuntimeError("the attention reported a device error")
        at, w = 0, 0.0
        for r, n in enumerate(lens):
            p64 = projs[r].double()
            qq, kk, vv = p64[:, :qw], p64[:, qw:qw + kw], p64[:, qw + kw:].view(n, kvh, Dv)
            i = torch.arange(n)
            qq = qq / torch.sqrt((qq * qq).mean(-1, keepdim=True) + eps) * wq.double()
            qq = (qq * (1 + coef * torch.log(torch.floor((i + 1) / every) + 1)).unsqueeze(1)).view(n, heads, D)
            kk = (kk / torch.sqrt((kk * kk).mean(-1, keepdim=True) + eps) * wk.double()).view(n, kvh, D)
            dist = (i[:, None] - i[None, :]).clamp(min=0).double()
            ref = torch.zeros(n, heads, Dv, dtype=torch.float64)
            for h in range(heads):
                sc = (qq[:, h] @ kk[:, h // (heads // kvh)].T) * scale - float(a[h]) * torch.log1p(float(b[h]) * dist) + float(c[h])
                ref[:, h] = (torch.sigmoid(sc) * (i[None, :] <= i[:, None])) @ vv[:, h // (heads // kvh)]
            k = new[r]
            w = max(w, _rel(out[at:at + k], ref.reshape(n, -1)[n - k:]))
            at += k
        worst.append(w)
    return max(worst[0], worst[1] / 200), 1e-4                     # bfloat16 storage is held to 2e-2


def check_gemm_tc_activation(dev) -> Tuple[float, float]:
    """relu(x W^T)^2 and the tanh form of GELU in the tcgen05 product's epilogue, tokens and weights as the wide operand."""
    from types import SimpleNamespace
    from .kernels import fast, ops
    worst = 0.0
    ctx = SimpleNamespace(err=torch.zeros(1, dtype=torch.int32, device=dev))
    for M, N, K in ((24, 512, 256), (384, 768, 512)):
        x = torch.randn(M, K).to(torch.bfloat16)
        w = (torch.randn(N, K) * 0.06).to(torch.bfloat16)
        z = x.double() @ w.double().T
        for name, want in (("relu2", torch.relu(z) ** 2),
                           ("gelu_tanh", 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3))))):
            out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
            if not fast.linear_act_bf16(ctx, x.to(dev), w.to(dev), out, ops.ACTIVATIONS[name]):
                raise RuntimeError("the tcgen05 product refused sizes it should take")
            worst = max(worst, _rel(out, want))
    if int(ctx.err.item()):
        return float("inf"), 0.0
    return worst, 2.0 ** -7


def check_streams(dev) -> Tuple[float, float]:
    """A residual of several streams: x_t <- sum_s M[s, t] x_s + m b[t] (y + bias), then u = sum_s a[s] x_s and its norm."""
    from .kernels import ops
    worst = 0.0
    for T, S, H in ((7, 3, 100), (40, 4, 1024)):
        xs, y, yb = torch.randn(T, S, H), torch.randn(T, H), torch.randn(H)
        M, b, a, w = torch.randn(S, S), torch.randn(S), torch.randn(S), 1 + 0.3 * torch.randn(H)
        xd, out = xs.to(dev), torch.empty(T, H, device=dev)
        ops.stream_step(xd, y=y.to(dev), carry=M.to(dev), write=b.to(dev), mult=0.5, y_bias=yb.to(dev), read=a.to(dev),
                        norm_w=w.to(dev), eps=1e-5, out=out)
        new = torch.einsum("st,jsh->jth", M.double(), xs.double()) + 0.5 * b.double()[None, :, None] * (y.double() + yb.double())[:, None, :]
        u = torch.einsum("s,jsh->jh", a.double(), new)
        worst = max(worst, _rel(xd, new), _rel(out, u / torch.sqrt((u * u).mean(-1, keepdim=True) + 1e-5) * w.double()))
    return worst, 1e-5


def check_decay_attention(dev) -> Tuple[float, float]:
    """Linear attention with one decay per head over silu-activated q, k, v, two requests in a batch, then the norm over
    all heads with a sigmoid gate."""
    from .kernels import ops
    heads, D, Dv, lens = 3, 24, 40, [21, 6]
    kd, vd, T = heads * D, heads * Dv, sum(lens)
    proj, decay, w = torch.randn(T, 2 * kd + 2 * vd), torch.tensor([0.5, 0.9, 0.99]), 1 + 0.3 * torch.randn(vd)
    pd = proj.to(dev)
    state = torch.zeros(2, heads, D, Dv, device=dev)
    cu = torch.tensor([0, lens[0], T], dtype=torch.int32, device=dev)
    slots = torch.tensor([1, 0], dtype=torch.int32, device=dev)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    o, act = torch.empty(T, vd, device=dev), torch.empty(T, vd, device=dev)
    ops.decay_recurrent(pd[:, :kd], pd[:, kd:2 * kd], pd[:, 2 * kd:2 * kd + vd], decay.to(dev), True, state, cu, slots, 2, o, heads, D, Dv,
                        1.0, err)
    req = torch.cat([torch.zeros(lens[0]), torch.ones(lens[1])]).to(dev, torch.int32)
    ops.rownorm_gate(o, pd[:, 2 * kd + vd:], w.to(dev), 1e-5, act, req, scale=1.2)
    p64 = proj.double()
    f = p64 / (1 + torch.exp(-p64))
    want, at = torch.zeros(T, vd, dtype=torch.float64), 0
    for n in lens:
        S = torch.zeros(heads, D, Dv, dtype=torch.float64)
        for t in range(at, at + n):
            q, k, v = f[t, :kd].view(heads, D), f[t, kd:2 * kd].view(heads, D), f[t, 2 * kd:2 * kd + vd].view(heads, Dv)
            S = decay.double()[:, None, None] * S + k[:, :, None] * v[:, None, :]
            want[t] = torch.einsum("hdv,hd->hv", S, q).reshape(vd)
        at += n
    gated = 1.2 * want / torch.sqrt((want * want).mean(-1, keepdim=True) + 1e-5) * w.double() * torch.sigmoid(p64[:, 2 * kd + vd:])
    return max(_rel(o, want), _rel(act, gated)), 2e-5


CHECKS: List[Tuple[str, Callable]] = [
    ("embedding gather", check_embedding),
    ("rmsnorm + residual add", check_rmsnorm),
    ("swiglu", check_swiglu),
    ("q/k norm + rotary + cache write", check_qkv_post),
    ("product, float32 FFMA", check_gemm_simt),
    ("product, tcgen05 128x256 tiles", check_gemm_tc_portion),
    ("product, tcgen05 swapped + split-K", check_gemm_tc_decode),
    ("product, tcgen05 SwiGLU epilogue", check_gemm_tc_swiglu),
    ("attention, float32 generic", check_attention_generic),
    ("attention, tcgen05 prefill + split-K decode", check_attention_tensor_core),
    ("attention, mma.sync prefill + decode", check_attention_mma),
    ("dynamic tanh norm + residual add", check_dyt_norm),
    ("clamped gated unit, kernel and tcgen05 epilogue", check_clamped_unit),
    ("gated linear attention: decay, recurrence, norm and gate", check_linear_attention),
    ("differential attention, float32 and mma.sync", check_diff_attention),
    ("attention without softmax, float32 and mma.sync", check_sigmoid_attention),
    ("product, tcgen05 with an activation in the epilogue", check_gemm_tc_activation),
    ("residual of several streams: write, read and norm", check_streams),
    ("decayed linear attention: recurrence, norm over all heads and gate", check_decay_attention),
    ("sampling", check_sampling),
    ("largest logits of a row", check_largest_logits),
]


def run(device: int = 0, verbose: bool = False, out=sys.stdout) -> int:
    if not torch.cuda.is_available():
        print("airun selftest needs a CUDA GPU (sm_100a); none is visible", file=sys.stderr)
        return 2
    dev = torch.device(f"cuda:{device}")
    torch.cuda.set_device(dev)
    torch.manual_seed(0)
    failed = 0
    for name, fn in CHECKS:
        try:
            err, bound = fn(dev)
            torch.cuda.synchronize()
            ok = err <= bound
            detail = f"max error {err:.3e} (bound {bound:.1e})"
        except Exception as e:                       # noqa: BLE001 - a failing check is reported, the rest still run
            ok, detail = False, f"{type(e).__name__}: {e}"
        failed += 0 if ok else 1
        if verbose or not ok:
            print(f"{'ok  ' if ok else 'FAIL'} {name}: {detail}", file=out)
        else:
            print(f"ok   {name}", file=out)
    print(f"{len(CHECKS) - failed} of {len(CHECKS)} checks passed", file=out)
    return 0 if failed == 0 else 1
