"""The Gamanex decoder in the engine against the plain implementation (tests/plain_gamanex.py): each mechanism's
kernels alone, then whole models of several small shapes through the step function, the scheduler and the replay
tool: whole prompts, token-by-token decoding, portions down to two tokens, unequal batches, slots and pages used
again, far keys, page borders, the first tokens, the steps of the query temperature and long decoding."""
from __future__ import annotations

import math
import random
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_gamanex as P
from helpers import Replay, assert_close, bf16_noise, random_tokens

F64 = torch.float64
gpu = pytest.mark.gpu


# ----------------------------------------------------------------------------- small shapes
def shape_g1() -> dict:
    """Odd sizes everywhere (a width no tensor-core product takes): key rows unlike value rows, groups of three query
    heads, a temperature that steps every 7 positions, a layer without a feed-forward, two layers on the first
    layer's keys and values with other head counts of their own, routers that choose two and three experts."""
    return P.make_config(vocab=150, width=100, eps=3e-5, logit_scale=1.7, layers=[
        P.attention_layer(3, 1, 12, 20, scale=0.4, temp=(0.3, 7), mlp=P.dense(72)),
        P.attention_layer(2, 1, 12, 20, scale=0.3, temp=(0.9, 16), kv_from=0, mlp=P.moe(24, 5, 2)),
        P.attention_layer(4, 2, 10, 6, scale=0.5, mlp=P.moe(16, 3, 3)),
        P.attention_layer(1, 1, 12, 20, scale=0.35, kv_from=0),
        P.attention_layer(2, 2, 10, 6, temp=(0.5, 1), kv_from=2, mlp=P.dense(40))])


def shape_g2() -> dict:
    """Sizes the tensor-core kernels take in bfloat16: heads of 32 and 64, groups of four and of one, a router that
    chooses one expert, no logit scale, a reader that is not next to its owner."""
    return P.make_config(vocab=192, width=128, layers=[
        P.attention_layer(4, 1, 32, 32, temp=(0.5, 40), mlp=P.moe(32, 8, 1)),
        P.attention_layer(2, 2, 64, 32, scale=0.2, temp=(0.25, 64), mlp=P.dense(160)),
        P.attention_layer(8, 1, 32, 32, scale=0.3, kv_from=0, mlp=P.moe(48, 4, 2)),
        P.attention_layer(4, 2, 64, 32, scale=0.15, temp=(1.0, 33), kv_from=1, mlp=P.dense(96))])


SHAPES = {"g1": (shape_g1, 8), "g2": (shape_g2, 16)}     # name -> (config, page size)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name, (make, page) in SHAPES.items():
        cfg = make()
        W = P.random_weights(cfg, seed=len(name) * 7 + ord(name[-1]))
        out[name] = (P.write_folder(str(tmp_path_factory.mktemp(name)), cfg, W), cfg, W, page)
        every = P.all_experts(cfg)
        out[name + " all experts"] = (P.write_folder(str(tmp_path_factory.mktemp(name + "_all")), every, W), every, W, page)
    return out


def engine(folder, dtype, page, tokens=512, batch=256, reqs=4):
    import airun_b200
    return airun_b200.Engine.from_folder(folder, dtype=dtype, page_size=page, cache_tokens=tokens, max_batch_tokens=batch,
                                         max_requests=reqs, max_context=tokens)


def run_schedule(eng, seqs, schedule):
    """schedule: steps, each a list of (request index, tokens to take); wants every token's logits.  Returns
    {request: [T, vocab]} and frees a request when its tokens are used up."""
    from airun_b200 import StepEntry
    at = {i: 0 for i in range(len(seqs))}
    got = {i: [] for i in range(len(seqs))}
    for step in schedule:
        entries = []
        for i, n in step:
            if at[i] == 0:
                eng.manager.add_request(f"q{i}")
            entries.append(StepEntry(f"q{i}", seqs[i][at[i]:at[i] + n], tuple(range(n))))
        out = eng.runner.step(entries).cpu().numpy()
        eng.runner.raise_on_device_error()
        row = 0
        for i, n in step:
            got[i].append(out[row:row + n])
            row += n
            at[i] += n
            if at[i] == len(seqs[i]):
                eng.manager.free_request(f"q{i}")
    eng.manager.check_invariants()
    return {i: np.concatenate(v) for i, v in got.items() if v}


def compare(got, cfg, W, seq, dtype, what):
    exact = P.plain_forward(cfg, W, seq).numpy()
    if dtype == "float32":
        return assert_close(got, exact.astype(np.float32), dtype, what)
    rounded = P.plain_forward(cfg, W, seq, rnd=P.to_bf16_and_back).numpy()
    assert_close(got, rounded.astype(np.float32), dtype, what, bf16_noise(rounded, exact))


def pick(folders, name, dtype):
    """Which experts a token goes to is a comparison of logits, and now and then two are so close that bfloat16
    rounding of the router's input decides otherwise: a different, equally valid computation from there on.  So the
    bfloat16 runs use the same weights with routers that choose ALL experts (the softmax still weighs them, and
    sorting, segments and sums run as always); the choice itself is tested in float32 and on the kernel alone."""
    return folders[name if dtype == "float32" else name + " all experts"]


# ----------------------------------------------------------------------------- without a GPU
def test_config_reads_sizes_sharing_and_constants():
    from airun_b200.config import GamanexConfig, architecture_name, lookup_architecture
    d = shape_g1()
    assert architecture_name(d) == "Gamanex" and lookup_architecture("Gamanex")[0] is GamanexConfig
    c = GamanexConfig.from_dict(d)
    assert (c.vocab_size, c.hidden_size, c.norm_eps, c.logit_scale) == (150, 100, 3e-5, 1.7)
    assert [(o.layer, o.cache_from) for o in c.execution_order()] == [(0, None), (1, 0), (2, None), (3, 0), (4, 2)]
    specs = c.layer_specs()
    assert all(s.mixer == "sigmoid_attention" and s.arrangement == "gated_parallel" for s in specs)
    assert [s.feed_forward for s in specs] == ["act_mlp", "routed_experts", "routed_experts", "", "act_mlp"]
    assert [s.mixer_args["owns_cache"] for s in specs] == [True, False, True, False, False]
    assert (specs[0].mixer_args["temp_coef"], specs[0].mixer_args["temp_every"]) == (0.3, 7)
    assert (specs[2].mixer_args["temp_coef"], specs[2].mixer_args["temp_every"]) == (0.0, 0)
    assert specs[4].mixer_args["scale"] == pytest.approx(1.5 * 10 ** -0.5)
    assert (specs[1].ffn_args["top"], specs[2].ffn_args["num_experts"], specs[1].ffn_args["scores"]) == (2, 3, "softmax")
    assert specs[1].ffn_args["renormalize"] and specs[1].ffn_args["router_bias"] and specs[1].ffn_args["weight_on"] == "output"
    assert specs[0].ffn_args["activation"] == "relu2" and specs[3].arrangement_args["prefix"] == "l3"
    assert c.head() == ("lm_head", dict(scale=1.7))
    assert GamanexConfig.from_dict(c.to_dict()).to_dict() == c.to_dict()
    assert GamanexConfig.from_dict(shape_g2()).logit_scale == 1.0


def test_config_lists_every_problem():
    from airun_b200.config import ConfigError, GamanexConfig
    d = shape_g1()
    d["layers"][0]["mixer"]["kv_heads"] = 2
    d["layers"][1]["mixer"]["kv_from"] = 3
    d["layers"][2]["mlp"]["router"]["top"] = 9
    d["layers"][3]["type"] = "other"
    d["layers"][4]["mixer"]["q_temp"]["every"] = 0
    d["norm"]["eps"] = 0
    with pytest.raises(ConfigError) as e:
        GamanexConfig.from_dict(d)
    for text in ("multiple of kv_heads", "kv_from", "top exceeds", "layers[3]", "q_temp.every", "norm.eps"):
        assert text in str(e.value)
    d = shape_g2()
    d["layers"][2]["mixer"]["vdim"] = 16
    with pytest.raises(ConfigError, match="must be equal"):
        GamanexConfig.from_dict(d)


def test_declared_tensors_are_the_files_tensors():
    from airun_b200.config import GamanexConfig
    from airun_b200.engine.model import DecoderModel
    for make, _ in SHAPES.values():
        cfg = make()
        specs = {s.name: tuple(s.shape) for s in DecoderModel(GamanexConfig.from_dict(cfg), torch.float32, "cpu").weight_specs()}
        assert specs == {n: tuple(s) for n, s in P.tensor_shapes(cfg).items()}


def test_a_file_may_keep_the_second_norm_of_a_layer_without_feed_forward():
    """A layer without a feed-forward reads no second norm, scale or gate; a file that holds them all the same loads,
    any other stray tensor does not."""
    from airun_b200.config import GamanexConfig
    from airun_b200.engine.model import DecoderModel
    from airun_b200.weights import DictSource, WeightError, check_source
    cfg = shape_g1()
    bare = next(i for i, l in enumerate(cfg["layers"]) if l["mlp"] is None)
    W = dict(P.random_weights(cfg, seed=3))
    width = cfg["width"]
    W.update({f"l{bare}.norm2": torch.ones(width), f"l{bare}.ls2": torch.ones(width), f"l{bare}.rg2": torch.zeros(width, width),
              f"l{bare}.rg2.b": torch.zeros(width)})
    model = DecoderModel(GamanexConfig.from_dict(cfg), torch.float32, "cpu")
    check_source(model.weight_specs(), DictSource(W), model.ignorable_tensors())
    W[f"l{bare}.mlp.up"] = torch.zeros(4, width)
    with pytest.raises(WeightError):
        check_source(model.weight_specs(), DictSource(W), model.ignorable_tensors())


def test_readers_share_their_owners_pages():
    from airun_b200.cache.manager import CacheManager
    from airun_b200.config import GamanexConfig
    from airun_b200.engine.model import DecoderModel
    from airun_b200.parts.base import PagedKVSpec
    m = DecoderModel(GamanexConfig.from_dict(shape_g1()), torch.float32, "cpu")
    specs, src = m.cache_specs()
    assert specs[0] == specs[1] == specs[3] == PagedKVSpec(1, 12, 0, value_dim=20) and specs[0].elements_per_token() == 32
    assert specs[2] == specs[4] == PagedKVSpec(2, 10, 0, value_dim=6) and src == [None, 0, None, 0, 2]
    mgr = CacheManager(specs, src, page_size=8, num_pages=16, max_requests=4)
    assert [b.shared for b in mgr.bindings] == [False, True, False, True, True]
    assert mgr.bindings[1].gid == mgr.bindings[3].gid == mgr.bindings[0].gid != mgr.bindings[2].gid == mgr.bindings[4].gid


def test_plain_temperature_distance_and_router():
    t = P.plain_query_temperature(torch.arange(20), 0.5, 7)
    assert t[5] == 1.0 and t[6] == pytest.approx(1 + 0.5 * math.log(2)) and t[12] == t[6] and t[13] == pytest.approx(1 + 0.5 * math.log(3))
    b = P.plain_distance_bias(3, 2.0, 0.5, first=4)
    assert b.shape == (3, 7) and b[0, 4] == 0 and b[2, 0] == pytest.approx(2.0 * math.log(4.0)) and b[0, 6] == 0
    h = torch.eye(4, dtype=F64)
    wr = torch.tensor([[1.0, 0, 0, 0], [0.9, 0, 0, 0], [0, 2.0, 0, 0]], dtype=F64)
    idx, wts = P.plain_router(h[:2], wr, torch.tensor([0.0, 0.5, 0.0], dtype=F64), 2)
    assert idx.tolist() == [[1, 0], [2, 1]]                        # the bias lifts expert 1 over expert 0
    assert wts[0, 0] == pytest.approx(1 / (1 + math.exp(-0.4))) and float(wts.sum(1)[1]) == pytest.approx(1.0)
    # a key weighs sigmoid(score), whatever the other keys do: doubling the keys doubles the output
    m = dict(heads=1, kv_heads=1, dim=4, vdim=2, scale=1.0)
    q, k, v = torch.zeros(1, 4, dtype=F64), torch.zeros(1, 4, dtype=F64), torch.ones(1, 2, dtype=F64)
    zero = torch.zeros(1, dtype=F64)
    assert torch.allclose(P.plain_sigmoid_attention(q, k, v, m, zero, zero, zero), torch.full((1, 2), 0.5, dtype=F64))


# ----------------------------------------------------------------------------- kernels alone
def dev(t, dtype=torch.float32):
    return t.to("cuda", dtype).contiguous()


def batch_ctx(spans):
    """The device arrays of a step whose request r brings rows spans[r] = (first position, end)."""
    lens = [b - a for a, b in spans]
    cu = torch.tensor(np.cumsum([0] + lens), dtype=torch.int32, device="cuda")
    req = torch.cat([torch.full((n,), r) for r, n in enumerate(lens)]).to("cuda", torch.int32)
    pos = torch.cat([torch.arange(a, b) for a, b in spans]).to("cuda", torch.int32)
    ends = torch.tensor([b for _, b in spans], dtype=torch.int32, device="cuda")
    from airun_b200.engine.batch import Workspace
    return SimpleNamespace(req_of_token=req, cu_tokens=cu, positions=pos, context_lens=ends, num_reqs=len(spans),
                           num_tokens=sum(lens), decode_only=all(n == 1 for n in lens), query_lens=lens,
                           context_lens_host=[b for _, b in spans], max_query_len=max(lens), max_context_len=max(b for _, b in spans),
                           ws=Workspace(torch.device("cuda"), 8 << 20), extras={},
                           err=torch.zeros(1, dtype=torch.int32, device="cuda"))


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,n", [(5, 100), (300, 512), (3, 4100)])
def test_two_norms_in_one_pass(T, n, dtype):
    from airun_b200.kernels import ops
    g = torch.Generator().manual_seed(T)
    x, d = torch.randn(T, n, generator=g), torch.randn(T, n, generator=g)
    w1, w2 = 1 + 0.3 * torch.randn(n, generator=g), 1 + 0.3 * torch.randn(n, generator=g)
    xs, o1, o2 = dev(x), torch.empty(T, n, device="cuda", dtype=dtype), torch.empty(T, n, device="cuda", dtype=dtype)
    ops.rmsnorm_pair(xs, dev(w1), o1, dev(w2), o2, 1e-4, delta=dev(d))
    s = (x + d).double()
    assert torch.equal(xs.cpu(), x + d)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    for o, w in ((o1, w1), (o2, w2)):
        assert torch.allclose(o.cpu().double(), P.plain_rmsnorm(s, w.double(), 1e-4), atol=tol, rtol=tol)
    ops.rmsnorm_pair(xs, dev(w1), o1, dev(w2), o2, 1e-4)                 # without a delta x stays as it is
    assert torch.equal(xs.cpu(), x + d) and torch.allclose(o2.cpu().double(), P.plain_rmsnorm(s, w2.double(), 1e-4), atol=tol, rtol=tol)


@gpu
def test_activations_gates_and_the_scaled_head():
    from airun_b200.kernels import ops
    g = torch.Generator().manual_seed(2)
    z = 3 * torch.randn(7, 50, generator=g)
    want = {"relu2": torch.relu(z.double()) ** 2, "silu": z.double() * torch.sigmoid(z.double()), "relu": torch.relu(z.double()),
            "gelu_tanh": 0.5 * z.double() * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z.double() + 0.044715 * z.double() ** 3)))}
    for name, w in want.items():
        wide = torch.zeros(7, 80, device="cuda")
        ops.act(dev(z), wide[:, 10:60], ops.ACTIVATIONS[name])
        assert torch.allclose(wide[:, 10:60].cpu().double(), w, atol=1e-5, rtol=1e-5) and float(wide[:, :10].abs().max()) == 0
        out = torch.empty(7, 50, device="cuda", dtype=torch.bfloat16)
        ops.act(dev(z), out, ops.ACTIVATIONS[name])
        assert torch.allclose(out.cpu().double(), w, atol=2e-2, rtol=1e-2)
    y1, y2, g1 = torch.randn(7, 50, generator=g), torch.randn(7, 50, generator=g), torch.randn(7, 90, generator=g)
    g2, c1, c2, s1, s2 = (torch.randn(n, generator=g) for n in ((7, 50), 50, 50, 50, 50))
    out = torch.empty(7, 50, device="cuda")
    ops.gated_sum(out, dev(y1), dev(g1)[:, 40:], dev(c1), dev(s1), dev(y2), dev(g2), dev(c2), dev(s2))
    want = s1 * torch.sigmoid(g1[:, 40:] + c1).double() * y1 + s2 * torch.sigmoid(g2 + c2).double() * y2
    assert torch.allclose(out.cpu().double(), want, atol=1e-5, rtol=1e-5)
    ops.gated_sum(out, dev(y1), None, None, dev(s1))                     # a scale alone, one sub-layer
    assert torch.allclose(out.cpu(), s1 * y1, atol=1e-6)
    x = dev(z)
    ops.scale_(x, 1.7)
    assert torch.allclose(x.cpu(), 1.7 * z)


@gpu
@pytest.mark.parametrize("M,N,K", [(1, 320, 256), (9, 4096, 2048), (40, 512, 1024), (100, 768, 512), (300, 1024, 256), (1500, 4096, 512)])
def test_activation_in_the_products_epilogue(M, N, K):
    """f(x W^T) with f applied to the finished sums inside the tensor-core product, for every way the product is cut
    (weights or tokens as the wide operand, K in slices, the persistent kernel), against float64."""
    from airun_b200.kernels import fast, ops
    g = torch.Generator().manual_seed(M + N)
    x = P.to_bf16_and_back(torch.randn(M, K, generator=g))
    w = P.to_bf16_and_back(torch.randn(N, K, generator=g) / math.sqrt(K))
    z = x.double() @ w.double().T
    want = {"relu2": torch.relu(z) ** 2, "silu": z * torch.sigmoid(z), "relu": torch.relu(z),
            "gelu_tanh": 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))}
    ctx = SimpleNamespace(err=torch.zeros(1, dtype=torch.int32, device="cuda"))
    for name, ref in want.items():
        out = torch.full((M, N), 9.0, device="cuda", dtype=torch.bfloat16)
        assert fast.linear_act_bf16(ctx, dev(x).to(torch.bfloat16), dev(w).to(torch.bfloat16), out, ops.ACTIVATIONS[name])
        assert int(ctx.err.item()) == 0
        assert torch.allclose(out.cpu().double(), ref, atol=1e-2, rtol=1e-2), name


def attention_case(seq_lens, new_lens, nh, nkv, D, Dv, page, dtype, seed, temp=(0.0, 0), spike=None, norm=True):
    """Keys and values written through the prologue kernel (pages handed out in a scrambled order) for the first
    len - new tokens of every request, then the last ``new`` tokens of each as one batch.  Returns the projections,
    the norm weights, the cache, the last batch's (spans, ctx) and its q."""
    from airun_b200.kernels import ops
    g = torch.Generator().manual_seed(seed)
    width = nh * D + nkv * (D + Dv)
    reqs = []
    for n in seq_lens:
        proj = torch.randn(n, width, generator=g)
        if spike is not None:
            spike(proj, n)
        reqs.append(proj)
    qw, kw = (1 + 0.3 * torch.randn(nh * D, generator=g), 1 + 0.3 * torch.randn(nkv * D, generator=g)) if norm else (None, None)
    blocks = [(n + page - 1) // page for n in seq_lens]
    num_pages = sum(blocks) + 3
    perm = torch.randperm(num_pages, generator=g).tolist()
    bt = torch.full((len(seq_lens), max(blocks)), -1, dtype=torch.int32)
    for r, nb in enumerate(blocks):
        for b in range(nb):
            bt[r, b] = perm.pop()
    cache = SimpleNamespace(pool=torch.zeros(num_pages, nkv * page * (D + Dv), device="cuda", dtype=dtype), block_table=bt.cuda(),
                            page_size=page, shared=False)
    last = None
    for phase in (0, 1):
        spans = [(0, n - m) if phase == 0 else (n - m, n) for n, m in zip(seq_lens, new_lens)]
        if sum(b - a for a, b in spans) == 0:
            continue
        ctx = batch_ctx([s for s in spans])
        proj = dev(torch.cat([reqs[r][a:b] for r, (a, b) in enumerate(spans)]))
        q = torch.empty(proj.shape[0], nh * D, device="cuda", dtype=dtype)
        ops.qk_rownorm_store(proj, None if qw is None else dev(qw), None if kw is None else dev(kw), 1e-5, temp[0], temp[1], q,
                             cache, ctx, nh * D, nkv, D, Dv, store=True)
        assert int(ctx.err.item()) == 0
        last = (spans, ctx, q)
    return reqs, (qw, kw), cache, last


def plain_attention_rows(proj, norms, nh, nkv, D, Dv, scale, a, b, c, temp, rnd=None):
    """Every token of one request from the equations: proj [n, q | k | v] as projected."""
    rr = (lambda t: t) if rnd is None else rnd
    n, p = proj.shape[0], proj.double()
    q, k, v = p[:, :nh * D], p[:, nh * D:nh * D + nkv * D], p[:, nh * D + nkv * D:]
    if norms[0] is not None:
        q, k = P.plain_rmsnorm(q, norms[0].double(), 1e-5), P.plain_rmsnorm(k, norms[1].double(), 1e-5)
    if temp[1]:
        q = q * P.plain_query_temperature(torch.arange(n), temp[0], temp[1]).unsqueeze(1)
    m = dict(heads=nh, kv_heads=nkv, dim=D, vdim=Dv, scale=scale)
    return P.plain_sigmoid_attention(rr(q), rr(k), rr(v), m, a.double(), b.double(), c.double())


def head_numbers(nh, seed):
    g = torch.Generator().manual_seed(seed)
    return 0.2 + torch.rand(nh, generator=g), 0.1 + torch.rand(nh, generator=g), -1.5 + torch.randn(nh, generator=g)


ATTN_SHAPES = [(3, 1, 12, 20, 8), (4, 2, 64, 32, 16), (2, 2, 130, 33, 24), (8, 1, 32, 32, 16), (16, 4, 64, 64, 16), (5, 5, 16, 128, 8),
               (4, 4, 128, 128, 32), (34, 2, 16, 24, 8)]           # the last: groups of 17 query heads, more than a product tile's rows


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,D,Dv,page", ATTN_SHAPES)
def test_attention_over_scrambled_pages(nh, nkv, D, Dv, page, dtype):
    """Three unequal requests: one decodes a token, one comes whole, one brings a portion; the temperature steps
    inside the portion.  The plain kernel in both types."""
    from airun_b200.kernels import ops
    seq_lens, new_lens = [70, 9, 133], [1, 9, 67]
    temp = (0.6, 19)
    reqs, norms, cache, (spans, ctx, q) = attention_case(seq_lens, new_lens, nh, nkv, D, Dv, page, dtype, seed=nh * 7 + D, temp=temp)
    a, b, c = head_numbers(nh, D)
    out = torch.empty(q.shape[0], nh * Dv, device="cuda", dtype=dtype)
    ops.sigmoid_attention(q, out, cache, ctx, nh, nkv, D, Dv, 0.2, dev(a), dev(b), dev(c))
    assert int(ctx.err.item()) == 0
    rnd = None if dtype == torch.float32 else P.to_bf16_and_back
    want = torch.cat([plain_attention_rows(reqs[r], norms, nh, nkv, D, Dv, 0.2, a, b, c, temp, rnd)[lo:hi] for r, (lo, hi) in enumerate(spans)])
    tol = 1e-4 if dtype == torch.float32 else 3e-2
    assert torch.allclose(out.cpu().double(), want, atol=tol * float(want.abs().max()), rtol=tol)


@gpu
@pytest.mark.parametrize("single", [False, True])
@pytest.mark.parametrize("nh,nkv,D,Dv,page", ATTN_SHAPES)
def test_tensor_core_attention(nh, nkv, D, Dv, page, single):
    """The bfloat16 dispatch (tensor cores where the sizes allow) against the equations with the same rounding, for
    prompt portions beside a single token and for a batch of single tokens alone."""
    from airun_b200.kernels import fast, ops
    seq_lens = [300, 9, 133, 64]
    new_lens = [1, 1, 1, 1] if single else [1, 9, 67, 64]
    temp = (0.6, 19)
    reqs, norms, cache, (spans, ctx, q) = attention_case(seq_lens, new_lens, nh, nkv, D, Dv, page, torch.bfloat16, seed=nh + D, temp=temp)
    a, b, c = head_numbers(nh, D + 1)
    part = SimpleNamespace(nh=nh, nkv=nkv, D=D, Dv=Dv, scale=0.2, dist_a=dev(a), dist_b=dev(b), head_c=dev(c), window=0)
    out = torch.full((q.shape[0], nh * Dv), 7.0, device="cuda", dtype=torch.bfloat16)
    if not fast.sigmoid_attention_bf16(ctx, q, out, cache, part):
        pytest.skip("these sizes run on the plain kernel")
    assert int(ctx.err.item()) == 0
    want = torch.cat([plain_attention_rows(reqs[r], norms, nh, nkv, D, Dv, 0.2, a, b, c, temp, P.to_bf16_and_back)[lo:hi]
                      for r, (lo, hi) in enumerate(spans)])
    assert torch.allclose(out.cpu().double(), want, atol=3e-2 * float(want.abs().max()), rtol=3e-2)
    plain = torch.empty_like(out)
    ops.sigmoid_attention(q, plain, cache, ctx, nh, nkv, D, Dv, 0.2, part.dist_a, part.dist_b, part.head_c)
    assert torch.allclose(out.float(), plain.float(), atol=2e-2 * float(want.abs().max()), rtol=2e-2)


@gpu
@pytest.mark.parametrize("nh,nkv,D,Dv,page", [(8, 2, 64, 64, 16), (6, 3, 24, 40, 8), (2, 1, 128, 128, 32)])
def test_single_tokens_whose_keys_are_cut_into_slices(nh, nkv, D, Dv, page):
    """Three single tokens with 1,500, 700 and 3 keys behind them: few enough (request, KV head) pairs that the keys
    of each are cut over several CTAs and added up by a second kernel.  Against the equations and the plain kernel."""
    from airun_b200.kernels import fast, ops
    seq_lens, new_lens, temp = [1500, 700, 3], [1, 1, 1], (0.4, 300)
    assert fast.plan_sigmoid_slices(len(seq_lens), nkv, max(seq_lens), 2 * fast.B200_SMS) > 1
    reqs, norms, cache, (spans, ctx, q) = attention_case(seq_lens, new_lens, nh, nkv, D, Dv, page, torch.bfloat16, seed=5 + D, temp=temp)
    a, b, c = head_numbers(nh, D + 2)
    c = c - 3.0                                                         # hundreds of keys: keep the sums near the values' size
    part = SimpleNamespace(nh=nh, nkv=nkv, D=D, Dv=Dv, scale=0.2, dist_a=dev(a), dist_b=dev(b), head_c=dev(c), window=0)
    out = torch.full((3, nh * Dv), 7.0, device="cuda", dtype=torch.bfloat16)
    assert fast.sigmoid_attention_bf16(ctx, q, out, cache, part)
    assert int(ctx.err.item()) == 0
    want = torch.cat([plain_attention_rows(reqs[r], norms, nh, nkv, D, Dv, 0.2, a, b, c, temp, P.to_bf16_and_back)[lo:hi]
                      for r, (lo, hi) in enumerate(spans)])
    # every token against its own size: the short one's slices are mostly empty and must add nothing
    for row in range(3):
        assert torch.allclose(out[row].cpu().double(), want[row], atol=2e-2 * float(want[row].abs().max()), rtol=2e-2), row
    plain = torch.empty_like(out)
    ops.sigmoid_attention(q, plain, cache, ctx, nh, nkv, D, Dv, 0.2, part.dist_a, part.dist_b, part.head_c)
    for row in range(3):
        assert torch.allclose(out[row].float(), plain[row].float(), atol=2e-2 * float(want[row].abs().max()), rtol=2e-2), row


@gpu
@pytest.mark.parametrize("new", [1, 70])
@pytest.mark.parametrize("window", [1, 50, 64, 200])
def test_a_window_in_both_attention_kernels(window, new):
    """The kernels take a window for designs that have one: the key ``window`` back is out, the one before it in.
    Values are rows of ones and queries zero, so a row's result counts its visible keys' weights."""
    from airun_b200.kernels import fast, ops
    nh, D, Dv, n = 2, 16, 8, 333
    def spike(proj, n_):
        proj[:, :nh * D] = 0.0
        proj[:, nh * D + D:] = 1.0
    a, b, c = torch.tensor([0.0, 0.7]), torch.tensor([1.0, 0.5]), torch.tensor([0.3, 1.0])
    for dtype in (torch.float32, torch.bfloat16):
        reqs, norms, cache, (spans, ctx, q) = attention_case([n], [new], nh, 1, D, Dv, 8, dtype, seed=2, spike=spike, norm=False)
        out = torch.empty(new, nh * Dv, device="cuda", dtype=dtype)
        part = SimpleNamespace(nh=nh, nkv=1, D=D, Dv=Dv, scale=1.0, dist_a=dev(a), dist_b=dev(b), head_c=dev(c), window=window)
        if dtype == torch.float32:
            ops.sigmoid_attention(q, out, cache, ctx, nh, 1, D, Dv, 1.0, part.dist_a, part.dist_b, part.head_c, window)
        else:
            assert fast.sigmoid_attention_bf16(ctx, q, out, cache, part)
        for row, pos in enumerate(range(n - new, n)):
            d = torch.arange(min(window, pos + 1), dtype=F64)
            for h in range(nh):
                want = torch.sigmoid(float(c[h]) - float(a[h]) * torch.log(1 + float(b[h]) * d)).sum()
                one_more = torch.sigmoid(float(c[h]) - float(a[h]) * torch.log(torch.tensor(1 + float(b[h]) * window, dtype=F64)))
                tol = 1e-5 * float(want) if dtype == torch.float32 else max(0.3 * float(one_more), 0.004 * float(want))
                assert abs(float(out[row, h * Dv]) - float(want)) <= tol, (dtype, row, h)


@gpu
@pytest.mark.parametrize("where", ["far", "first", "page border", "itself"])
@pytest.mark.parametrize("new", [1, 12])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_one_key_that_stands_out(where, new, dtype):
    """With an offset of -150 in the sigmoid no key weighs anything, except ONE whose score is lifted by a query along
    it: the output of the last token is that key's value, 900 positions back, at position 0, on the last slot of a
    page, or the token itself.  Decoded alone and as the last row of a portion; through the dispatch of each type."""
    from airun_b200.kernels import ops, fast
    nh, nkv, D, Dv, page = 4, 2, 32, 32, 16
    n = 1000
    target = {"far": n - 1 - 900, "first": 0, "page border": 16 * 40 - 1, "itself": n - 1}[where]

    def spike(proj, n_):
        k = proj[target, nh * D:nh * D + nkv * D].view(nkv, D)
        k *= 300.0 ** 0.5 / k.norm(dim=1, keepdim=True)                # a long key: |k|^2 = 300 in every KV head
        proj[n_ - 1, :nh * D] = 0.05 * torch.randn(nh * D)
        for h in range(nh):
            proj[n_ - 1, h * D:(h + 1) * D] += k[h // (nh // nkv)]
    reqs, norms, cache, (spans, ctx, q) = attention_case([n], [new], nh, nkv, D, Dv, page, dtype, seed=11, spike=spike, norm=False)
    a, b, c = torch.zeros(nh), torch.ones(nh), torch.full((nh,), -150.0)
    out = torch.empty(new, nh * Dv, device="cuda", dtype=dtype)
    part = SimpleNamespace(nh=nh, nkv=nkv, D=D, Dv=Dv, scale=1.0, dist_a=dev(a), dist_b=dev(b), head_c=dev(c), window=0)
    if dtype == torch.float32 or not fast.sigmoid_attention_bf16(ctx, q, out, cache, part):
        ops.sigmoid_attention(q, out, cache, ctx, nh, nkv, D, Dv, 1.0, part.dist_a, part.dist_b, part.head_c)
    rnd = None if dtype == torch.float32 else P.to_bf16_and_back
    want = plain_attention_rows(reqs[0], norms, nh, nkv, D, Dv, 1.0, a, b, c, (0.0, 0), rnd)[n - new:]
    tol = 1e-4 if dtype == torch.float32 else 3e-2
    assert torch.allclose(out.cpu().double(), want, atol=tol, rtol=tol)
    v_target = reqs[0][target, nh * D + nkv * D:].view(nkv, Dv).double()
    for h in range(nh):
        got = out[-1, h * Dv:(h + 1) * Dv].cpu().double()
        assert torch.allclose(got, v_target[h // (nh // nkv)], atol=0.1), f"head {h} does not see position {target}"


@gpu
def test_distance_term_and_head_offset_per_head():
    """Two heads on the same keys with zero queries: the weight of a key is sigmoid(c_h - a_h ln(1 + b_h d)) exactly."""
    from airun_b200.kernels import ops
    nh, D, Dv, n = 2, 8, 4, 50
    def spike(proj, n_):
        proj[:, :nh * D] = 0.0
        proj[:, nh * D + D:] = 1.0                                   # every value is a row of ones
    reqs, norms, cache, (spans, ctx, q) = attention_case([n], [3], nh, 1, D, Dv, 8, torch.float32, seed=1, spike=spike, norm=False)
    a, b, c = torch.tensor([0.0, 1.5]), torch.tensor([3.0, 0.25]), torch.tensor([0.5, -0.25])
    out = torch.empty(3, nh * Dv, device="cuda")
    ops.sigmoid_attention(q, out, cache, ctx, nh, 1, D, Dv, 1.0, dev(a), dev(b), dev(c))
    for row, pos in enumerate(range(n - 3, n)):
        d = torch.arange(pos + 1, dtype=F64)
        for h in range(nh):
            want = torch.sigmoid(float(c[h]) - float(a[h]) * torch.log(1 + float(b[h]) * d)).sum()
            assert float(out[row, h * Dv]) == pytest.approx(float(want), rel=1e-5)


@gpu
@pytest.mark.parametrize("top,E", [(1, 5), (2, 12), (3, 3), (2, 7)])
def test_router_with_a_bias_weighs_by_the_softmax_over_the_chosen(top, E):
    from airun_b200.kernels import ops
    g = torch.Generator().manual_seed(E)
    T = 37
    z, bias = 2 * torch.randn(T, E + 6, generator=g), 2 * torch.randn(E, generator=g)
    req = torch.zeros(T, dtype=torch.int32)
    req[5] = -1
    ids, rank = (torch.empty(T, top, dtype=torch.int32, device="cuda") for _ in range(2))
    wts = torch.empty(T, top, device="cuda")
    counts, seg = torch.zeros(E, dtype=torch.int32, device="cuda"), torch.empty(E + 1, dtype=torch.int32, device="cuda")
    ops.moe_route(dev(z)[:, 3:3 + E], top, True, True, req.cuda(), ids, wts, rank, counts, seg, bias=dev(bias))
    val, idx = torch.topk(z[:, 3:3 + E].double() + bias.double(), top, dim=-1)
    want = torch.softmax(val, dim=-1)
    keep = req >= 0
    assert torch.equal(ids.cpu()[keep].long(), idx[keep]) and int(ids[5, 0]) == -1
    assert torch.allclose(wts.cpu().double()[keep], want[keep], atol=1e-6)
    assert (idx != torch.topk(z[:, 3:3 + E].double(), top, dim=-1)[1]).any()        # the bias changed somebody's choice
    assert int(seg[E]) == int(keep.sum()) * top


# ----------------------------------------------------------------------------- whole models
SEQ = {"g1": [83, 40, 9, 121], "g2": [150, 31, 70, 2]}


@gpu
@pytest.mark.parametrize("name", ["g1", "g2"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompts_and_residuals(folders, name, dtype):
    folder, cfg, W, page = pick(folders, name, dtype)
    eng = engine(folder, dtype, page)
    seqs = [random_tokens(n, cfg["vocab"], 40 + i) for i, n in enumerate(SEQ[name])]
    if dtype == "float32":
        seen = {}
        eng.model.layer_hook = lambda ci, x: seen.__setitem__(ci, x.cpu().double())
        got = run_schedule(eng, seqs[:1], [[(0, len(seqs[0]))]])
        eng.model.layer_hook = None
        res = []
        P.plain_forward(cfg, W, seqs[0], residuals=res)
        assert len(seen) == len(res) == len(cfg["layers"])
        for ci, want in enumerate(res):
            assert torch.allclose(seen[ci][:len(seqs[0])], want, atol=2e-4 * float(want.abs().max())), f"residual after layer {ci}"
        compare(got[0], cfg, W, seqs[0], dtype, f"{name} whole 0")
    got = run_schedule(eng, seqs, [[(i, len(s))] for i, s in enumerate(seqs)])
    for i, s in enumerate(seqs):
        compare(got[i], cfg, W, s, dtype, f"{name} whole {i}")


@gpu
@pytest.mark.parametrize("name", ["g1", "g2"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefill_then_token_by_token_and_from_the_first_token(folders, name, dtype):
    folder, cfg, W, page = pick(folders, name, dtype)
    eng = engine(folder, dtype, page)
    s = random_tokens(97, cfg["vocab"], 5)
    got = run_schedule(eng, [s], [[(0, 50)]] + [[(0, 1)]] * 47)            # temperatures step and pages fill while decoding
    compare(got[0], cfg, W, s, dtype, f"{name} prefill+decode")
    got = run_schedule(eng, [s[:45]], [[(0, 1)]] * 45)                    # every token alone, the first too
    compare(got[0], cfg, W, s[:45], dtype, f"{name} decode only")


@gpu
@pytest.mark.parametrize("name", ["g1", "g2"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_down_to_two_tokens(folders, name, dtype):
    folder, cfg, W, page = pick(folders, name, dtype)
    eng = engine(folder, dtype, page)
    s = random_tokens(140, cfg["vocab"], 6)
    for sizes in ([2, 3, 2, 5, 17, 2, 36, 11, 2, 1, 37, 22], [64, 2, 64, 10], [7] * 20):
        assert sum(sizes) == 140
        got = run_schedule(eng, [s], [[(0, n)] for n in sizes])
        compare(got[0], cfg, W, s, dtype, f"{name} portions {sizes[:4]}")


@gpu
@pytest.mark.parametrize("name", ["g1", "g2"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_batches_with_slots_and_pages_used_again(folders, name, dtype):
    """Six requests through four slots and a pool that cannot hold them all at once: portions beside single
    tokens, requests that sit a step out; every request's logits against the plain implementation AND, in
    float32, within rounding of the same request run alone."""
    folder, cfg, W, page = pick(folders, name, dtype)
    lens = [60, 33, 90, 17, 45, 71]
    seqs = [random_tokens(n, cfg["vocab"], 70 + i) for i, n in enumerate(lens)]
    rng = random.Random(3)
    eng = engine(folder, dtype, page, tokens=256 + 64, batch=128, reqs=4)
    at, live, waiting, steps = {}, [], list(range(len(seqs))), []
    while waiting or live:
        while waiting and len(live) < 4 and sum((len(seqs[i]) + 63) // 64 * 64 for i in live + [waiting[0]]) <= 320:
            live.append(waiting.pop(0)); at[live[-1]] = 0
        step = []
        for i in list(live):
            if len(live) > 1 and rng.random() < 0.25:
                continue
            left = len(seqs[i]) - at[i]
            n = 1 if left <= 6 else min(left - 6, rng.choice([2, 3, 8, 19, 30]))
            step.append((i, n)); at[i] += n
            if at[i] == len(seqs[i]):
                live.remove(i)
        if step:
            steps.append(step)
    got = run_schedule(eng, seqs, steps)
    assert max(len(s) for s in steps) >= 3
    alone = engine(folder, dtype, page) if dtype == "float32" else None
    for i, s in enumerate(seqs):
        compare(got[i], cfg, W, s, dtype, f"{name} mixed {i}")
        if alone is not None:
            one = run_schedule(alone, [s], [[(0, len(s))]])[0]
            assert np.abs(one - got[i]).max() <= 2e-4 * np.abs(one).max()


def order_cases():
    return {
        "no feed-forward anywhere": P.make_config(96, 48, [P.attention_layer(2, 1, 8, 24), P.attention_layer(3, 3, 8, 8, temp=(0.4, 3))]),
        "every layer on the first layer's keys and values": P.make_config(96, 48, [
            P.attention_layer(3, 1, 8, 12, temp=(0.2, 5), mlp=P.dense(32)), P.attention_layer(2, 1, 8, 12, kv_from=0),
            P.attention_layer(1, 1, 8, 12, kv_from=0, mlp=P.moe(8, 2, 1))], logit_scale=0.5),
        "one layer, one head, one expert of one": P.make_config(64, 40, [P.attention_layer(1, 1, 16, 8, mlp=P.moe(8, 1, 1))], eps=1e-3),
        "a reader right after its owner, then a second owner": P.make_config(96, 56, [
            P.attention_layer(2, 2, 8, 8), P.attention_layer(4, 2, 8, 8, kv_from=0, mlp=P.dense(24)),
            P.attention_layer(4, 4, 4, 12, temp=(2.0, 2), mlp=P.moe(16, 4, 4)), P.attention_layer(8, 4, 4, 12, kv_from=2, mlp=P.dense(16))]),
    }


@gpu
@pytest.mark.parametrize("name", list(order_cases()))
def test_other_orders_of_layers(name, tmp_path):
    cfg = order_cases()[name]
    W = P.random_weights(cfg, seed=3)
    folder = P.write_folder(str(tmp_path / "m"), cfg, W)
    seqs = [random_tokens(n, cfg["vocab"], 7 + n) for n in (45, 8)]
    for dtype in ("float32", "bfloat16"):
        if dtype == "bfloat16":
            cfg = P.all_experts(cfg)
            folder = P.write_folder(str(tmp_path / "all"), cfg, W)
        eng = engine(folder, dtype, 8, tokens=192, batch=64)
        got = run_schedule(eng, seqs, [[(0, 30), (1, 2)], [(0, 1), (1, 5)], [(0, 13), (1, 1)], [(0, 1)]])
        for i, sq in enumerate(seqs):
            compare(got[i], cfg, W, sq, dtype, f"{name}, request {i}")


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_over_many_steps_of_the_temperature(folders, dtype):
    folder, cfg, W, page = pick(folders, "g2", dtype)
    eng = engine(folder, dtype, page, tokens=512)
    s = random_tokens(330, cfg["vocab"], 8)
    got = run_schedule(eng, [s], [[(0, 10)]] + [[(0, 1)]] * 320)
    compare(got[0], cfg, W, s, dtype, "long decode")


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_prompt_then_single_tokens_in_an_engine_made_for_long_contexts(folders, dtype):
    """700 tokens in one step (eleven row tiles, up to eleven key tiles each), then single tokens in an engine whose
    longest context is 4,096, so the decode graph cuts every token's keys into several slices."""
    folder, cfg, W, page = pick(folders, "g2", dtype)
    eng = engine(folder, dtype, page, tokens=4096, batch=1024)
    s = random_tokens(706, cfg["vocab"], 21)
    got = run_schedule(eng, [s], [[(0, 700)]] + [[(0, 1)]] * 6)
    compare(got[0], cfg, W, s, dtype, "long prompt")


@gpu
def test_greedy_generation_through_the_entry_point(folders):
    import airun_b200
    folder, cfg, W, page = folders["g2"]
    eng = engine(folder, "float32", page, tokens=512, batch=64, reqs=4)
    prompts = [random_tokens(n, cfg["vocab"], 90 + n) for n in (70, 5, 31)]
    reqs = [eng.add_request(p, airun_b200.SamplingParams.greedy(), max_new_tokens=12) for p in prompts]
    while any(r.finished is None for r in reqs):
        eng.run_step()
    for p, r in zip(prompts, reqs):
        assert r.output == P.plain_greedy(cfg, W, p, 12)
    one = eng.generate(prompts[1], airun_b200.SamplingParams.greedy(), max_new_tokens=12)
    assert one.token_ids == P.plain_greedy(cfg, W, prompts[1], 12)


@gpu
def test_replay_tool_runs_a_gamanex_folder(folders, tmp_path):
    folder, cfg, W, page = folders["g1"]
    seqs = [random_tokens(n, cfg["vocab"], 20 + n) for n in (50, 23)]
    rp = Replay(folder, "float32", str(tmp_path), max_tokens=128, page_size=page)
    a = rp.step([dict(id="a", tokens=seqs[0][:30], want=[0, 29])])
    b = rp.step([dict(id="a", tokens=seqs[0][30:], want=[19]), dict(id="b", tokens=seqs[1], want=[22])], end=["a", "b"])
    assert rp.close() == 0
    wa, wb = P.plain_forward(cfg, W, seqs[0]).numpy(), P.plain_forward(cfg, W, seqs[1]).numpy()
    assert_close(np.concatenate([a, b]), np.stack([wa[0], wa[29], wa[49], wb[22]]).astype(np.float32), "float32", "replay")
