"""The Tagulix decoder in the engine against the plain implementation (tests/plain_tagulix.py): each mechanism's kernels
alone, then whole models of several small shapes through the step function, the scheduler and the replay tool: whole
prompts, token-by-token decoding, portions down to two tokens, unequal batches, slots and pages used again, far keys,
page borders, window edges, the first tokens, long decoding and other orders of layers."""
from __future__ import annotations

import json
import math
import os
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_tagulix as P
from helpers import Replay, assert_close, bf16_noise, random_tokens

F64 = torch.float64
gpu = pytest.mark.gpu


# ----------------------------------------------------------------------------- small shapes
def shape_t1() -> dict:
    """Odd sizes everywhere (a width no tensor-core product takes): key rows unlike value rows, groups of three query
    heads, a window of 11 over pages of 8, a full and a partial rotation, two streams, a layer without feed-forward, a
    parallel layer first, a layer that runs with the parallel layer's tensors, routers with and without groups and
    experts that return their input."""
    return P.make_config(vocab=150, width=100, eps=3e-5, mult=0.7, streams=2, layers=[
        P.parallel_layer(3, 1, 12, 20, bias_max=40, lin_heads=3, lin_dim=10, lin_vdim=12, decay=[0.5, 0.9, 0.99], temp=(0.4, 7),
                         left_scale=1.3, right_scale=0.8, mlp=P.moe(24, 5, 2, identity=1, scale=1.5, groups=(3, 2))),
        P.attention_layer(3, 1, 12, 20, window=11, rot=(12, 1000.0), mlp=P.moe(16, 3, 3, identity=0, scale=1.0, groups=(1, 1))),
        P.attention_layer(4, 2, 10, 6, window=3, rot=(4, 50.0)),
        P.parallel_layer(3, 1, 12, 20, bias_max=40, lin_heads=3, lin_dim=10, lin_vdim=12, decay=[0.5, 0.9, 0.99], temp=(0.4, 7),
                         left_scale=1.3, right_scale=0.8, mlp=P.moe(24, 5, 2, identity=1, scale=1.5, groups=(3, 2)), weights_of=0),
        P.attention_layer(3, 1, 12, 20, window=11, rot=(12, 1000.0), mlp=P.moe(16, 3, 3, identity=0, scale=1.0, groups=(1, 1)),
                          weights_of=1)])


def shape_t2() -> dict:
    """Sizes the tensor-core kernels take in bfloat16: heads of 32 and 64, groups of four and of one, four streams, a
    window of 40 over pages of 16, no rotation in one layer, a temperature that steps every 33 positions."""
    return P.make_config(vocab=192, width=128, mult=0.5, streams=4, layers=[
        P.attention_layer(4, 1, 32, 32, window=40, rot=(16, 10000.0), mlp=P.moe(32, 6, 2, identity=2, scale=1.7, groups=(2, 1))),
        P.parallel_layer(4, 2, 64, 32, bias_max=100, lin_heads=2, lin_dim=32, lin_vdim=64, decay=[0.7, 0.995], temp=(0.5, 33),
                         left_scale=1.2, right_scale=1.1, mlp=P.moe(32, 6, 2, identity=2, scale=1.7, groups=(2, 1))),
        P.attention_layer(4, 1, 32, 32, window=40, rot=(16, 10000.0), mlp=P.moe(32, 6, 2, identity=2, scale=1.7, groups=(2, 1)),
                          weights_of=0),
        P.attention_layer(2, 2, 64, 32, window=17, mlp=P.moe(48, 4, 1, identity=0, scale=1.0, groups=(2, 2)))])


def shape_t3() -> dict:
    """No streams at all (one plain residual), one query head a KV head, values that make sizes equal or 1: one stream
    of connections is shape_t4."""
    return P.make_config(vocab=64, width=48, mult=1.0, layers=[
        P.attention_layer(2, 2, 8, 8, window=200, rot=(8, 100.0), mlp=P.moe(8, 2, 1, identity=1, scale=1.0, groups=(1, 1))),
        P.parallel_layer(1, 1, 16, 16, bias_max=9, lin_heads=1, lin_dim=16, lin_vdim=16, decay=[0.8])])


def shape_t4() -> dict:
    d = shape_t3()
    d["streams"] = 1
    return d


SHAPES = {"t1": (shape_t1, 8, 8), "t2": (shape_t2, 16, 12), "t3": (shape_t3, 8, 4), "t4": (shape_t4, 8, 6)}   # config, page, rel rows


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name, (make, page, rel) in SHAPES.items():
        cfg = make()
        W = P.random_weights(cfg, seed=len(name) * 7 + ord(name[-1]), rel_rows=rel)
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
    exact = P.plain_forward(cfg, W, seq)[0].numpy()
    if dtype == "float32":
        return assert_close(got, exact.astype(np.float32), dtype, what)
    rounded = P.plain_forward(cfg, W, seq, rnd=P.to_bf16_and_back)[0].numpy()
    # the engine's rounding is another draw of the same noise (other tile borders, other orders of the sums, weights
    # rounded against a running maximum), and this design rounds in more places a layer than the others: a row is held
    # to three times its own noise, where helpers.assert_close alone would hold it to two
    assert_close(got, rounded.astype(np.float32), dtype, what, 1.5 * bf16_noise(rounded, exact))


def pick(folders, name, dtype):
    """Which experts a token goes to is a comparison of scores, and now and then two are so close that bfloat16 rounding
    of the router's input decides otherwise: a different, equally valid computation from there on.  So the bfloat16
    runs use the same weights with routers that choose ALL their outputs (the scores still weigh them, and sorting,
    segments and sums run as always); the choice itself is tested in float32 and on the kernel alone."""
    return folders[name if dtype == "float32" else name + " all experts"]


# ----------------------------------------------------------------------------- without a GPU
def test_config_reads_sizes_sharing_and_constants():
    from airun_b200.config import TagulixConfig, architecture_name, lookup_architecture
    d = shape_t1()
    assert architecture_name(d) == "Tagulix" and lookup_architecture("Tagulix")[0] is TagulixConfig
    c = TagulixConfig.from_dict(d)
    assert (c.vocab_size, c.hidden_size, c.norm_eps, c.residual_mult, c.streams) == (150, 100, 3e-5, 0.7, 2)
    assert c.owners() == [0, 1, 2] and [o.layer for o in c.execution_order()] == [0, 1, 2, 0, 1]
    assert all(o.cache_from is None for o in c.execution_order())
    c = c.with_tensor_shapes({"l0.mix.left.rel": (8, 3)})
    specs = c.layer_specs()
    assert [s.index for s in specs] == [0, 1, 2] and [s.mixer for s in specs] == ["side_by_side", "softmax_attention", "softmax_attention"]
    assert [s.feed_forward for s in specs] == ["routed_experts", "routed_experts", ""]
    assert all(s.arrangement == "hyper_connections" and s.arrangement_args["streams"] == 2 and s.arrangement_args["learned"] for s in specs)
    a = specs[0].mixer_args
    assert (a["left_scale"], a["right_scale"], a["left"], a["right"]) == (1.3, 0.8, "softmax_attention", "decay_linear_attention")
    assert (a["left_args"]["temp_coef"], a["left_args"]["temp_every"], a["left_args"]["distance_far"]) == (0.4, 7, 40)
    assert a["left_args"]["distance_rows"] == 8 and a["left_args"]["sink"] and a["left_args"]["qk_norm"] == "weight"
    assert a["right_args"]["decay"] == [0.5, 0.9, 0.99] and (a["right_args"]["key_dim"], a["right_args"]["value_dim"]) == (10, 12)
    b = specs[1].mixer_args
    assert (b["window"], b["qk_norm"], b["bias"], b["position"], b["position_args"]) == (11, "unit", True, "rotary_interleaved",
                                                                                      dict(rotary_dim=12, theta=1000.0))
    assert specs[2].mixer_args["position_args"]["rotary_dim"] == 4 and specs[2].mixer_args["scale"] == pytest.approx(3 * 10 ** -0.5)
    f = specs[0].ffn_args
    assert (f["num_experts"], f["top"], f["identity_experts"], f["weight_scale"], f["groups"], f["keep_groups"]) == (5, 2, 1, 1.5, 3, 2)
    assert f["routing"] == "grouped" and f["expert"] == "act" and f["activation"] == "gelu_erf" and f["choice_bias"]
    assert TagulixConfig.from_dict(c.to_dict()).to_dict() == TagulixConfig.from_dict(d).to_dict()
    plain = TagulixConfig.from_dict(shape_t3())
    assert plain.streams is None and plain.residual_streams() == 1 and not plain.layer_specs()[0].arrangement_args["learned"]
    assert plain.layer_specs()[0].mixer_args["window"] == 200 and "streams" not in plain.to_dict()
    assert plain.layer_specs()[1].feed_forward == "" and plain.ignorable_tensors() == ["l1.norm2", "l1.hc2.in", "l1.hc2.mix", "l1.hc2.out"]


def test_config_lists_every_problem():
    from airun_b200.config import ConfigError, TagulixConfig
    d = shape_t1()
    d["layers"][0]["mixer"]["left"]["kv_heads"] = 2
    d["layers"][0]["mixer"]["right"]["decay"] = [0.5]
    d["layers"][1]["mixer"]["rot"]["dims"] = 13
    d["layers"][1]["mlp"]["router"]["top"] = 9
    d["layers"][2]["type"] = "other"
    d["layers"][3]["weights_of"] = 4
    d["layers"][4]["mixer"]["mask"]["size"] = 12
    d["norm"]["eps"] = 0
    d["streams"] = 9
    with pytest.raises(ConfigError) as e:
        TagulixConfig.from_dict(d)
    text = str(e.value)
    for piece in ("layers[0].mixer.left.heads", "right.decay", "rot.dims", "router.top", "layers[2] needs", "layers[3].weights_of",
                  "layers[4] runs with the tensors of layer 1", "norm.eps", "streams must be at most 8"):
        assert piece in text, (piece, text)


def test_declared_tensors_are_the_files_tensors():
    from airun_b200.config import TagulixConfig
    from airun_b200.engine.model import DecoderModel
    for name, (make, _, rel) in SHAPES.items():
        shapes = P.tensor_shapes(make(), rel)
        c = TagulixConfig.from_dict(make()).with_tensor_shapes(shapes)
        m = DecoderModel(c, torch.float32, "cpu")
        declared = {s.name: tuple(s.shape) for s in m.weight_specs()}
        assert declared == shapes, (name, set(declared) ^ set(shapes))
        assert m.multi_stream and m.streams == (make().get("streams") or 1)


def test_a_mixer_of_two_keeps_two_caches():
    from airun_b200.cache.manager import CacheManager
    from airun_b200.config import TagulixConfig
    from airun_b200.engine.model import DecoderModel
    from airun_b200.parts.base import PagedKVSpec, StateSpec
    m = DecoderModel(TagulixConfig.from_dict(shape_t1()), torch.float32, "cpu")
    specs, src = m.cache_specs()
    assert src == [None] * 5
    assert specs[0] == specs[3] == (PagedKVSpec(1, 12, 0, value_dim=20), StateSpec((3, 10, 12), torch.float32))
    assert specs[1] == specs[4] == PagedKVSpec(1, 12, 11, value_dim=20) and specs[2] == PagedKVSpec(2, 10, 3, value_dim=6)
    mgr = CacheManager(specs, src, page_size=8, num_pages=16, max_requests=4)
    b = mgr.bindings
    assert [x.kind for x in b] == ["multi", "paged", "paged", "multi", "paged"]
    assert [p.kind for p in b[0].parts] == ["paged", "state"] and b[0].parts[0].gid == b[3].parts[0].gid != b[1].gid
    assert (b[0].parts[0].index, b[3].parts[0].index, b[0].parts[1].index, b[3].parts[1].index) == (0, 1, 0, 1)
    assert b[1].gid == b[4].gid and (b[1].index, b[4].index) == (0, 1) and len(mgr.paged) == 3 and len(mgr.state) == 1
    # pages come and go in every group at once; a window's pages go back as it passes
    mgr.add_request("a")
    mgr.reserve("a", 30)
    mgr.commit("a", 30)
    free = mgr.free_pages()
    assert free[b[0].parts[0].gid] == 12 and free[b[1].gid] == 14 and free[b[2].gid] == 15
    mgr.free_request("a")
    assert set(mgr.free_pages().values()) == {16}
    mgr.check_invariants()


def test_plain_buckets_router_streams_and_recurrence():
    # distances below half the rows read their own row; the rest are spread over the logarithm up to ``far``
    assert [P.plain_distance_bucket(n, 8, 40) for n in (0, 3, 4, 7, 8, 12, 13, 39, 40, 500)] == [0, 3, 4, 4, 5, 5, 6, 7, 7, 7]
    assert [P.plain_distance_bucket(n, 16, 128) for n in (7, 8, 15, 16, 31, 32, 64, 127, 128)] == [7, 8, 9, 10, 11, 12, 14, 15, 15]
    t = P.plain_query_temperature(torch.arange(20), 0.5, 7)
    assert t[5] == 1.0 and t[6] == pytest.approx(1 + 0.5 * math.log(2)) and t[12] == t[6] and t[13] == pytest.approx(1 + 0.5 * math.log(3))
    # routing: the best group by score + correction, although the correction makes every sum negative
    z = torch.tensor([[2.0, 0.5, 0.0, 1.9, 1.8, 0.0]], dtype=F64)
    corr = torch.tensor([-5.0, -5.0, -5.0, -5.1, -5.0, -5.0], dtype=F64)
    ids, w = P.plain_route(z, corr, top=2, groups=2, keep=1, scale=2.0)
    s = torch.softmax(z, -1)[0]
    assert ids.tolist() == [[0, 1]] and w[0, 0] == pytest.approx(float(2 * s[0] / (s[0] + s[1])))      # the first group holds the best sum
    ids, _ = P.plain_route(z, corr, top=2, groups=1, keep=1, scale=1.0)
    assert ids.tolist() == [[0, 4]]                                                                      # without groups: 0 and 4 (3 is corrected down)
    ids, _ = P.plain_route(z, torch.tensor([-1.0, 0, 0, 0, 0, 0], dtype=F64), top=2, groups=2, keep=1, scale=1.0)
    assert ids.tolist() == [[3, 4]]
    # an expert that returns its input: with one such expert chosen alone the feed-forward is the identity times scale
    W = {"p.router": torch.zeros(1, 4, dtype=F64), "p.correction": torch.zeros(1, dtype=F64)}
    h = torch.randn(3, 4, dtype=F64)
    out = P.plain_moe(h, W, "p", P.moe(2, 0, 1, identity=1, scale=3.0))
    assert torch.allclose(out, 3.0 * h)
    # streams: carry [from, to]
    xs = torch.tensor([[[1.0]], [[10.0]]], dtype=F64)
    new = P.plain_streams_write(xs, torch.tensor([[100.0]], dtype=F64), torch.tensor([[1.0, 2.0], [0.0, 3.0]], dtype=F64),
                                torch.tensor([1.0, -1.0], dtype=F64), 0.5)
    assert new.flatten().tolist() == [1.0 + 50.0, 2.0 + 30.0 - 50.0]
    assert float(P.plain_streams_read(xs, torch.tensor([2.0, 0.5], dtype=F64))) == 7.0
    # the recurrence: with k = v = q = 1 the output is the geometric sum of the decay
    q = torch.ones(4, 1, 1, dtype=F64)
    o, S = P.plain_decay_recurrence(q, q, q, [0.5])
    assert o.flatten().tolist() == [1.0, 1.5, 1.75, 1.875] and float(S) == 1.875
    o2, _ = P.plain_decay_recurrence(q[2:], q[2:], q[2:], [0.5], state=P.plain_decay_recurrence(q[:2], q[:2], q[:2], [0.5])[1])
    assert o2.flatten().tolist() == [1.75, 1.875]
    # the sink takes weight and gives nothing: one key, sink equal to its score, halves the output
    one = torch.ones(1, 1, 2, dtype=F64)
    assert torch.allclose(P.plain_softmax_attention(one, one, one, 1, 1, 1.0, sink=torch.tensor([2.0], dtype=F64)), torch.full((1, 2), 0.5, dtype=F64))
    # the rotation keeps lengths and turns pair i of position p by p * base^(-2i/dims); other dimensions stay
    x = torch.randn(5, 2, 6, dtype=F64)
    r = P.plain_rotate_pairs(x, torch.arange(5), 4, 100.0)
    assert torch.allclose(r.norm(dim=-1), x.norm(dim=-1)) and torch.equal(r[..., 4:], x[..., 4:]) and torch.equal(r[0], x[0])
    assert float(r[3, 0, 2]) == pytest.approx(float(x[3, 0, 2] * math.cos(0.3) - x[3, 0, 3] * math.sin(0.3)))


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
                           ws=Workspace(torch.device("cuda"), 8 << 20), extras={}, state_slots=torch.arange(len(spans), dtype=torch.int32, device="cuda"),
                           err=torch.zeros(1, dtype=torch.int32, device="cuda"))


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,S,H", [(5, 1, 100), (9, 3, 320), (3, 4, 4100), (40, 8, 64)])
def test_streams_in_one_pass(T, S, H, dtype):
    from airun_b200.kernels import ops
    g = torch.Generator().manual_seed(T + S)
    x = torch.randn(T, H, generator=g)
    xs = torch.empty(T, S, H, device="cuda")
    ops.stream_fill(dev(x), xs)
    assert torch.equal(xs.cpu(), x[:, None, :].expand(T, S, H))
    xs0 = torch.randn(T, S, H, generator=g)
    y, yb = torch.randn(T, H + 7, generator=g), torch.randn(H, generator=g)
    M, b, a, w = torch.randn(S, S, generator=g), torch.randn(S, generator=g), torch.randn(S, generator=g), 1 + 0.3 * torch.randn(H, generator=g)
    xs = dev(xs0)
    out = torch.empty(T, H, device="cuda", dtype=dtype)
    req = torch.zeros(T, dtype=torch.int32, device="cuda")
    # a read alone: the first sub-layer of a model
    ops.stream_step(xs, read=dev(a), norm_w=dev(w), eps=1e-4, out=out, req_of_token=req)
    sd = xs0.double().permute(1, 0, 2)                     # the plain functions take [S, T, H]
    tol = 1e-5 if dtype == torch.float32 else 1.5e-2
    assert torch.equal(xs.cpu(), xs0)
    assert torch.allclose(out.cpu().double(), P.plain_rmsnorm(P.plain_streams_read(sd, a.double()), w.double(), 1e-4), atol=tol, rtol=tol)
    # a write and the next read in one pass; y is a column slice, with a bias
    ops.stream_step(xs, y=dev(y)[:, 7:], carry=dev(M), write=dev(b), mult=0.6, y_bias=dev(yb), read=dev(a), norm_w=dev(w), eps=1e-4,
                    out=out, req_of_token=req)
    new = P.plain_streams_write(sd, y[:, 7:].double() + yb.double(), M.double(), b.double(), 0.6)
    assert torch.allclose(xs.cpu().double().permute(1, 0, 2), new, atol=1e-5, rtol=1e-5)
    assert torch.allclose(out.cpu().double(), P.plain_rmsnorm(P.plain_streams_read(new, a.double()), w.double(), 1e-4), atol=tol, rtol=tol)
    # the end of a model: a write, then the sum of the streams in float32
    total = torch.empty(T, H, device="cuda")
    ops.stream_step(xs, y=dev(y)[:, :H], carry=dev(M), write=dev(b), mult=1.0, read=torch.ones(S, device="cuda"), out=total, req_of_token=req)
    last = P.plain_streams_write(new, y[:, :H].double(), M.double(), b.double(), 1.0)
    assert torch.allclose(total.cpu().double(), last.sum(0), atol=2e-5, rtol=1e-5)
    # the same with everything on 16-byte boundaries (four columns a thread)
    xs2, y2 = dev(xs0), dev(y[:, :H].contiguous())
    ops.stream_step(xs2, y=y2, carry=dev(M), write=dev(b), mult=0.6, y_bias=dev(yb), read=dev(a), norm_w=dev(w), eps=1e-4, out=out,
                    req_of_token=req)
    assert torch.allclose(xs2.cpu().double().permute(1, 0, 2), P.plain_streams_write(sd, y[:, :H].double() + yb.double(), M.double(), b.double(), 0.6),
                          atol=1e-5, rtol=1e-5)
    ops.stream_step(xs2, y=y2, carry=dev(M), write=dev(b), mult=1.0, read=torch.ones(S, device="cuda"), out=total, req_of_token=req)
    twice = P.plain_streams_write(P.plain_streams_write(sd, y[:, :H].double() + yb.double(), M.double(), b.double(), 0.6), y[:, :H].double(),
                                  M.double(), b.double(), 1.0)
    assert torch.allclose(total.cpu().double(), twice.sum(0), atol=5e-5, rtol=1e-5)
    # padding rows are left alone
    req[0] = -1
    before = xs.clone()
    ops.stream_step(xs, y=dev(y)[:, :H], carry=dev(M), write=dev(b), mult=1.0, read=dev(a), norm_w=dev(w), eps=1e-4, out=out, req_of_token=req)
    assert torch.equal(xs[0], before[0]) and not torch.equal(xs[1], before[1])


def attention_case(seq_lens, new_lens, nh, nkv, D, Dv, page, dtype, seed, mode, rot=None, temp=(0.0, 0), bias=False, spike=None):
    """Keys and values written through the prologue kernel (pages handed out in a scrambled order) for the first
    len - new tokens of every request, then the last ``new`` tokens of each as one batch.  ``mode``: "weight" (a
    weighted norm before the rotation) or "unit" (an unweighted one after it).  Returns the projections, the
    prologue's constants, the cache, the last batch's (spans, ctx) and its q."""
    from airun_b200.kernels import ops
    g = torch.Generator().manual_seed(seed)
    width = nh * D + nkv * (D + Dv)
    reqs = []
    for n in seq_lens:
        proj = torch.randn(n, width, generator=g)
        if spike is not None:
            spike(proj, n)
        reqs.append(proj)
    qw, kw = (1.5 + 0.3 * torch.randn(D, generator=g), 1.5 + 0.3 * torch.randn(D, generator=g)) if mode == "weight" else (None, None)
    b = 0.5 * torch.randn(width, generator=g) if bias else None
    inv = None
    if rot:
        inv = torch.tensor([rot[1] ** (-2.0 * i / rot[0]) for i in range(rot[0] // 2)], dtype=torch.float64).float()
    blocks = [(n + page - 1) // page for n in seq_lens]
    num_pages = sum(blocks) + 3
    perm = torch.randperm(num_pages, generator=g).tolist()
    bt = torch.full((len(seq_lens), max(blocks)), -1, dtype=torch.int32)
    for r, nb in enumerate(blocks):
        for blk in range(nb):
            bt[r, blk] = perm.pop()
    cache = SimpleNamespace(pool=torch.zeros(num_pages, nkv * page * (D + Dv), device="cuda", dtype=dtype), block_table=bt.cuda(),
                            page_size=page, shared=False)
    last = None
    for phase in (0, 1):
        spans = [(0, n - m) if phase == 0 else (n - m, n) for n, m in zip(seq_lens, new_lens)]
        spans = [s for s in spans]
        if sum(e - a for a, e in spans) == 0:
            continue
        live = [(r, s) for r, s in enumerate(spans) if s[1] > s[0]]
        ctx = batch_ctx([s for _, s in live])
        table = cache.block_table
        cache.block_table = table[[r for r, _ in live]].contiguous()
        proj = dev(torch.cat([reqs[r][a:e] for r, (a, e) in live]))
        q = torch.empty(proj.shape[0], nh * D, device="cuda", dtype=dtype)
        ops.qkv_prepare(proj, None if b is None else dev(b), None if qw is None else dev(qw), None if kw is None else dev(kw),
                        mode == "unit", 1e-5, ops.ROPE_INTERLEAVED if rot else ops.ROPE_NONE, rot[0] if rot else 0,
                        None if inv is None else dev(inv), temp[0], temp[1], q, cache, ctx, nh, nkv, D, Dv, store=True)
        assert int(ctx.err.item()) == 0
        last = ([s for _, s in live], ctx, q, [r for r, _ in live])
        if phase == 0:
            cache.block_table = table
    return reqs, (qw, kw, b), cache, last


def plain_case(reqs, consts, spans, live, nh, nkv, D, Dv, scale, mode, rot, temp, window, rel, far, sink, out_scale=1.0):
    """The plain attention over the same projections: [rows of the last batch, heads * Dv]."""
    qw, kw, b = consts
    outs = []
    for r, (a, e) in zip(live, spans):
        proj = reqs[r][:e].double() + (b.double() if b is not None else 0.0)
        n = proj.shape[0]
        q, k = proj[:, :nh * D].view(n, nh, D), proj[:, nh * D:(nh + nkv) * D].view(n, nkv, D)
        v = proj[:, (nh + nkv) * D:].view(n, nkv, Dv)
        pos = torch.arange(n)
        if mode == "weight":
            q, k = P.plain_rmsnorm(q, qw.double(), 1e-5), P.plain_rmsnorm(k, kw.double(), 1e-5)
        if rot:
            q, k = P.plain_rotate_pairs(q, pos, rot[0], rot[1]), P.plain_rotate_pairs(k, pos, rot[0], rot[1])
        if mode == "unit":
            q, k = P.plain_rms(q, 1e-5), P.plain_rms(k, 1e-5)
        if temp[1]:
            q = q * P.plain_query_temperature(pos, temp[0], temp[1])[:, None, None]
        bias = None
        if rel is not None:
            bucket = torch.tensor([[P.plain_distance_bucket(i - j, rel.shape[0], far) if j <= i else 0 for j in range(n)] for i in range(n)])
            bias = rel.double()[bucket].permute(2, 0, 1)
        o = P.plain_softmax_attention(q, k, v, nh, nkv, scale, window, bias=bias, sink=None if sink is None else sink.double())
        outs.append(out_scale * o[a:e])
    return torch.cat(outs)


def run_attention(q, cache, ctx, nh, nkv, D, Dv, scale, rel, far, sink, window, out_scale=1.0):
    from airun_b200.kernels import ops
    from airun_b200.parts.softmax_attention import distance_buckets
    table = None
    if rel is not None:
        table = dev(rel)[torch.tensor(distance_buckets(rel.shape[0], far), device="cuda")].t().contiguous()
    wide = torch.zeros(q.shape[0], nh * Dv + 16, device="cuda", dtype=q.dtype)
    out = wide[:, 8:8 + nh * Dv]
    ops.softmax_attention(q, out, cache, ctx, nh, nkv, D, Dv, scale, table, None if sink is None else dev(sink), window, out_scale)
    assert int(ctx.err.item()) == 0 and float(wide[:, :8].abs().max()) == 0 and float(wide[:, 8 + nh * Dv:].abs().max()) == 0
    return out.float().cpu().double()


ATT_SHAPES = [  # heads, kv heads, D, Dv, page
    (3, 1, 12, 20, 8), (4, 2, 88, 72, 16), (8, 8, 32, 64, 16), (2, 1, 130, 6, 8), (6, 2, 64, 128, 32), (1, 1, 40, 40, 16), (16, 1, 16, 8, 8)]


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", ATT_SHAPES)
@pytest.mark.parametrize("mode", ["unit", "weight"])
def test_attention_kernels_over_scrambled_pages(shape, mode, dtype):
    """A portion beside a whole prompt beside a single token, every option at once."""
    nh, nkv, D, Dv, page = shape
    g = torch.Generator().manual_seed(D + nh)
    unit = mode == "unit"
    rot = (min(D, 8) // 2 * 2 if D % 4 else D // 2 // 2 * 2, 500.0) if unit else None
    temp = (0.0, 0) if unit else (0.6, 5)
    rel, far = (None, 0) if unit else (1.5 * torch.randn(10, nh, generator=g), 37)
    sink = None if unit else 1.0 + torch.randn(nh, generator=g)
    window = 19 if unit else 0
    seqs, new = [70, 23, 91], [13, 23, 1]
    reqs, consts, cache, (spans, ctx, q, live) = attention_case(seqs, new, nh, nkv, D, Dv, page, dtype, 5, mode, rot, temp, bias=unit)
    scale = (2.0 if unit else 0.8) * D ** -0.5
    got = run_attention(q, cache, ctx, nh, nkv, D, Dv, scale, rel, far, sink, window, out_scale=1.3)
    want = plain_case(reqs, consts, spans, live, nh, nkv, D, Dv, scale, mode, rot, temp, window, rel, far, sink, 1.3)
    tol = 2e-5 if dtype == torch.float32 else 4e-2
    assert torch.allclose(got, want, atol=tol, rtol=tol), float((got - want).abs().max())


def run_attention_tc(q, cache, ctx, nh, nkv, D, Dv, scale, rel, far, sink, window, out_scale=1.0):
    """The tensor-core kernels (tiles for portions, head groups with key slices for single tokens) on the same batch."""
    from airun_b200.kernels import fast
    from airun_b200.parts.softmax_attention import distance_buckets
    table = None
    if rel is not None:
        table = dev(rel)[torch.tensor(distance_buckets(rel.shape[0], far), device="cuda")].t().contiguous()
    part = SimpleNamespace(D=D, Dv=Dv, nh=nh, nkv=nkv, scale=scale, table=table, sink=None if sink is None else dev(sink), window=window,
                           out_scale=out_scale)
    wide = torch.zeros(q.shape[0], nh * Dv + 16, device="cuda", dtype=q.dtype)
    out = wide[:, 8:8 + nh * Dv]
    assert fast.softmax_attention_bf16(ctx, q, out, cache, part)
    assert int(ctx.err.item()) == 0 and float(wide[:, :8].abs().max()) == 0 and float(wide[:, 8 + nh * Dv:].abs().max()) == 0
    return out.float().cpu().double()


@gpu
@pytest.mark.parametrize("shape", [s_ for s_ in ATT_SHAPES if s_[2] <= 128 and s_[3] <= 128])
@pytest.mark.parametrize("mode", ["unit", "weight"])
@pytest.mark.parametrize("new", [[13, 23, 1], [1, 1, 1]])
def test_tensor_core_attention_against_the_plain_kernel_and_the_formula(shape, mode, new):
    """A portion beside a whole prompt beside a single token, and single tokens alone (700, 23 and 1500 keys: the keys
    of a single token are cut into slices, and the short request's later slices are empty)."""
    nh, nkv, D, Dv, page = shape
    g = torch.Generator().manual_seed(D + nh)
    unit = mode == "unit"
    rot = (D // 2 // 2 * 2, 500.0) if unit and D >= 4 else None
    temp = (0.0, 0) if unit else (0.6, 5)
    rel, far = (None, 0) if unit else (1.5 * torch.randn(10, nh, generator=g), 37)
    sink = None if unit else 1.0 + torch.randn(nh, generator=g)
    window = 90 if unit else 0
    seqs = [70, 23, 91] if new[0] > 1 else [700, 23, 1500]
    reqs, consts, cache, (spans, ctx, q, live) = attention_case(seqs, new, nh, nkv, D, Dv, page, torch.bfloat16, 5, mode, rot, temp, bias=unit)
    scale = (2.0 if unit else 0.8) * D ** -0.5
    want = plain_case(reqs, consts, spans, live, nh, nkv, D, Dv, scale, mode, rot, temp, window, rel, far, sink, 1.3)
    got = run_attention_tc(q, cache, ctx, nh, nkv, D, Dv, scale, rel, far, sink, window, out_scale=1.3)
    plain = run_attention(q, cache, ctx, nh, nkv, D, Dv, scale, rel, far, sink, window, out_scale=1.3)
    assert torch.allclose(got, want, atol=1e-1, rtol=3e-2), float((got - want).abs().max())       # bfloat16 q, k, v against float64
    assert torch.allclose(got, plain, atol=3e-2, rtol=3e-2), float((got - plain).abs().max())     # the same inputs: only the weights' rounding


@gpu
@pytest.mark.parametrize("window", [1, 63, 64, 65, 200])
@pytest.mark.parametrize("new", [1, 70])
def test_tensor_core_window_edges_key_by_key(window, new):
    nh = nkv = 1
    n, D, Dv, page = 300, 8, 128, 8

    def spike(proj, n_):
        proj[:, :2 * D] = 0.0
        proj[:, 2 * D:] = torch.eye(n_, n_)[:, -Dv:]           # the last 128 keys spell out their position
    reqs, consts, cache, (spans, ctx, q, live) = attention_case([n], [new], nh, nkv, D, Dv, page, torch.bfloat16, 1, "weight", spike=spike)
    got = run_attention_tc(q, cache, ctx, nh, nkv, D, Dv, 1.0, None, 0, None, window)
    for row, i in enumerate(range(n - new, n)):
        lo = max(0, i - window + 1)
        want = torch.zeros(n, dtype=F64)
        want[lo:i + 1] = 1.0 / (i + 1 - lo)
        assert torch.allclose(got[row], want[-Dv:], atol=4e-3), (i, window)


@gpu
@pytest.mark.parametrize("window", [1, 7, 8, 9, 50, 64, 200])
@pytest.mark.parametrize("new", [1, 30])
def test_window_edges_key_by_key(window, new):
    """The key just inside the window weighs, the key just outside does not: every key's value is its own position, one
    hot, so the output row of a query spells out which keys it saw."""
    from airun_b200.kernels import ops
    nh = nkv = 1
    n, D, Dv, page = 150, 8, 152, 8

    def spike(proj, n_):
        proj[:, :2 * D] = 0.0                          # equal scores: every visible key weighs 1 / visible
        proj[:, 2 * D:] = torch.eye(n_, Dv)
    reqs, consts, cache, (spans, ctx, q, live) = attention_case([n], [new], nh, nkv, D, Dv, page, torch.float32, 1, "weight", spike=spike)
    got = run_attention(q, cache, ctx, nh, nkv, D, Dv, 1.0, None, 0, None, window)
    for row, i in enumerate(range(n - new, n)):
        lo = max(0, i - window + 1)
        want = torch.zeros(Dv, dtype=F64)
        want[lo:i + 1] = 1.0 / (i + 1 - lo)
        assert torch.allclose(got[row], want, atol=1e-6), (i, window)


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("key_at", [0, 7, 8, 299, 444, 599])
@pytest.mark.parametrize("new", [1, 40])
def test_one_key_that_stands_out(key_at, new, dtype):
    """Among 600 keys ONE has a large score with the last query (its key and that query are scaled up); its value must
    be what the query returns: far back, at position 0, at a page border, and the token itself."""
    n, nh, nkv, D, Dv, page = 600, 2, 1, 16, 16, 8

    def spike(proj, n_):
        proj[:, :(nh + nkv) * D] *= 0.05
        proj[n_ - 1, :nh * D] = 0.0
        proj[n_ - 1, 0:nh * D:D] = 6.0                  # every query head of the last token points along dimension 0
        proj[key_at, nh * D:(nh + nkv) * D] = 0.0
        proj[key_at, nh * D] = 6.0                      # and so does the key at key_at
        if key_at == n_ - 1:
            proj[key_at, 0:nh * D:D] = 6.0
    reqs, consts, cache, (spans, ctx, q, live) = attention_case([n], [new], nh, nkv, D, Dv, page, dtype, 3, "weight", spike=spike)
    got = run_attention(q, cache, ctx, nh, nkv, D, Dv, 1.0, None, 0, None, 0)
    v = reqs[0][key_at, (nh + nkv) * D:].double()
    tol = 1e-3 if dtype == torch.float32 else 3e-2
    for h in range(nh):
        assert torch.allclose(got[-1, h * Dv:(h + 1) * Dv], v, atol=tol), (h, float((got[-1, h * Dv:(h + 1) * Dv] - v).abs().max()))
    want = plain_case(reqs, consts, spans, live, nh, nkv, D, Dv, 1.0, "weight", None, (0.0, 0), 0, None, 0, None)
    assert torch.allclose(got, want, atol=2e-5 if dtype == torch.float32 else 6e-2, rtol=1e-5 if dtype == torch.float32 else 3e-2)


@gpu
def test_sink_and_distance_rows_show():
    """A sink as large as the scores takes half the weight; a distance row of +30 makes its distances win."""
    nh, nkv, D, Dv, page, n = 2, 2, 8, 8, 8, 60

    def spike(proj, n_):
        proj[:, :(nh + nkv) * D] = 0.0                  # all scores 0
    reqs, consts, cache, (spans, ctx, q, live) = attention_case([n], [n], nh, nkv, D, Dv, page, torch.float32, 2, "weight", spike=spike)
    plain = run_attention(q, cache, ctx, nh, nkv, D, Dv, 1.0, None, 0, None, 0)
    sink = torch.tensor([0.0, math.log(3.0)])
    got = run_attention(q, cache, ctx, nh, nkv, D, Dv, 1.0, None, 0, sink, 0)
    i = torch.arange(1, n + 1, dtype=F64)[:, None]
    assert torch.allclose(got[:, :Dv], plain[:, :Dv] * i / (i + 1), atol=1e-6)        # exp(0) = one more key's weight
    assert torch.allclose(got[:, Dv:], plain[:, Dv:] * i / (i + 3), atol=1e-6)
    rel = torch.zeros(8, nh)
    rel[6, 0] = 30.0                                    # distances 13 .. 22 of head 0 (8 rows, far 40)
    assert [P.plain_distance_bucket(d, 8, 40) for d in (12, 13, 22, 23)] == [5, 6, 6, 7]
    got = run_attention(q, cache, ctx, nh, nkv, D, Dv, 1.0, rel, 40, None, 0)
    v = reqs[0][:, (nh + nkv) * D:(nh + nkv) * D + Dv].double()
    for t in (30, 59):
        assert torch.allclose(got[t, :Dv], v[t - 22:t - 12].mean(0), atol=1e-5)
    assert torch.allclose(got[:, Dv:], plain[:, Dv:], atol=1e-6) and torch.allclose(got[:13, :Dv], plain[:13, :Dv], atol=1e-6)


@gpu
@pytest.mark.parametrize("heads,D,Dv", [(3, 10, 12), (4, 32, 64), (1, 130, 40), (2, 64, 128)])
def test_decay_recurrence_and_gated_norm(heads, D, Dv):
    """Unequal requests in one batch, then each request's next portion and single tokens from the state the first step
    left, in other slots' company; against the recurrence run token by token."""
    from airun_b200.kernels import ops
    g = torch.Generator().manual_seed(D)
    decay = [0.5, 0.9, 0.99, 0.999][:heads]
    lens, cut = [37, 1, 20], [30, 0, 19]
    kd, vd = heads * D, heads * Dv
    projs = [torch.randn(n, 2 * kd + 2 * vd, generator=g) for n in lens]
    state = torch.zeros(5, heads, D, Dv, device="cuda")
    state[3] = 7.0                                       # a slot nobody uses stays as it is
    w = 1 + 0.3 * torch.randn(vd, generator=g)
    got = [[], [], []]
    for phase in (0, 1):
        live = [(r, (0, c) if phase == 0 else (c, n)) for r, (n, c) in enumerate(zip(lens, cut)) if (c if phase == 0 else n - c) > 0]
        ctx = batch_ctx([s for _, s in live])
        ctx.state_slots = torch.tensor([[4, 0, 2][r] for r, _ in live], dtype=torch.int32, device="cuda")
        proj = dev(torch.cat([projs[r][a:e] for r, (a, e) in live]))
        o = torch.empty(proj.shape[0], vd, device="cuda")
        ops.decay_recurrent(proj[:, :kd], proj[:, kd:2 * kd], proj[:, 2 * kd:2 * kd + vd], dev(torch.tensor(decay)), True, state,
                            ctx.cu_tokens, ctx.state_slots, ctx.num_reqs, o, heads, D, Dv, 1.0, ctx.err)
        act = torch.empty(proj.shape[0], vd, device="cuda")
        ops.rownorm_gate(o, proj[:, 2 * kd + vd:], dev(w), 1e-5, act, ctx.req_of_token, scale=1.1)
        assert int(ctx.err.item()) == 0
        row = 0
        for r, (a, e) in live:
            got[r].append((o[row:row + e - a].cpu().double(), act[row:row + e - a].cpu().double()))
            row += e - a
    assert float(state[3].min()) == 7.0 and float(state[1].abs().max()) == 0.0
    for r, n in enumerate(lens):
        p = projs[r].double()
        q, k, v = (P.plain_silu(p[:, :kd]).view(n, heads, D), P.plain_silu(p[:, kd:2 * kd]).view(n, heads, D),
                   P.plain_silu(p[:, 2 * kd:2 * kd + vd]).view(n, heads, Dv))
        o, S = P.plain_decay_recurrence(q, k, v, decay)
        want_act = 1.1 * P.plain_rmsnorm(o.reshape(n, vd), w.double(), 1e-5) * torch.sigmoid(p[:, 2 * kd + vd:])
        assert torch.allclose(torch.cat([x for x, _ in got[r]]), o.reshape(n, vd), atol=2e-4, rtol=2e-5), r
        assert torch.allclose(torch.cat([x for _, x in got[r]]), want_act, atol=2e-5, rtol=2e-5), r
        assert torch.allclose(state[[4, 0, 2][r]].cpu().double(), S, atol=2e-4, rtol=2e-5)


@gpu
@pytest.mark.parametrize("n_out,real,top,groups,keep", [(6, 4, 2, 2, 1), (20, 16, 4, 2, 1), (9, 9, 3, 3, 2), (5, 5, 5, 1, 1), (12, 7, 1, 4, 3), (40, 33, 6, 1, 1)])
def test_grouped_routing_on_the_kernel(n_out, real, top, groups, keep):
    from airun_b200.kernels import ops
    g = torch.Generator().manual_seed(n_out)
    T = 57
    z = 2 * torch.randn(T, n_out + 3, generator=g)
    corr = torch.randn(n_out, generator=g) - 3.0              # every choice score is negative
    ids, rank = (torch.empty(T, top, dtype=torch.int32, device="cuda") for _ in range(2))
    wts = torch.empty(T, top, device="cuda")
    counts, seg = torch.zeros(real, dtype=torch.int32, device="cuda"), torch.empty(real + 1, dtype=torch.int32, device="cuda")
    req = torch.zeros(T, dtype=torch.int32, device="cuda")
    req[5] = -1
    ops.moe_route_grouped(dev(z)[:, :n_out], real, top, groups, keep, 1.7, dev(corr), req, ids, wts, rank, counts, seg)
    want_ids, want_w = P.plain_route(z[:, :n_out].double(), corr.double(), top, groups, keep, 1.7)
    ids, wts, rank = ids.cpu(), wts.cpu(), rank.cpu()
    rows = [t for t in range(T) if t != 5]
    assert ids[5].tolist() == [-1] * top
    assert torch.equal(ids[rows].long(), want_ids[rows])
    assert torch.allclose(wts[rows].double(), want_w[rows], atol=1e-6, rtol=1e-5)
    for e in range(real):
        mine = sorted(int(rank[t, k]) for t in rows for k in range(top) if int(ids[t, k]) == e)
        assert mine == list(range(len(mine))) and int(counts[e]) == len(mine)
    assert seg.cpu().tolist() == np.cumsum([0] + counts.cpu().tolist()).tolist()


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,H,I,E,ident,top", [(33, 100, 24, 5, 1, 2), (200, 128, 64, 6, 2, 3), (1, 64, 16, 3, 0, 3), (700, 256, 48, 12, 3, 4)])
def test_routed_experts_part(T, H, I, E, ident, top, dtype):
    """The whole feed-forward part (routing, rows to experts, the product with the erf GELU, the sum with the experts
    that return their input) against the plain one; in bfloat16 every output is chosen, so no rounding changes a choice."""
    from airun_b200.parts.base import make_part
    g = torch.Generator().manual_seed(T)
    n_out = E + ident
    groups = 1 if n_out % 2 else 2
    if dtype == torch.bfloat16:
        top = n_out
    mlp = P.moe(I, E, top, identity=ident, scale=1.4, groups=(groups, groups))
    W = {"p.router": 2 * torch.randn(n_out, H, generator=g) / math.sqrt(H), "p.correction": 0.1 * torch.randn(n_out, generator=g)}
    for e in range(E):
        W[f"p.e{e}.up"], W[f"p.e{e}.down"] = torch.randn(I, H, generator=g) / math.sqrt(H), torch.randn(H, I, generator=g) / math.sqrt(I)
    W = {n: P.to_bf16_and_back(t) for n, t in W.items()}
    part = make_part("feed_forward", "routed_experts", prefix="p", hidden_size=H, intermediate_size=I, num_experts=E, top=top,
                     scores="softmax", weight_on="output", expert="act", activation="gelu_erf", routing="grouped", choice_bias=True,
                     groups=groups, keep_groups=groups, identity_experts=ident, weight_scale=1.4, dtype=dtype, device="cuda")
    store = {"float32": torch.float32, "compute": dtype}
    part.load_weights({s.name: dev(W[s.name], store.get(s.storage, dtype)) for s in part.weight_specs()})
    h = P.to_bf16_and_back(torch.randn(T, H, generator=g))
    ctx = batch_ctx([(0, T)])
    out = part.forward(ctx, dev(h, dtype))
    assert int(ctx.err.item()) == 0
    Wd = {n: t.double() for n, t in W.items()}
    want = P.plain_moe(h.double(), Wd, "p", mlp, rnd=P.to_bf16_and_back if dtype == torch.bfloat16 else None)
    tol = 3e-5 if dtype == torch.float32 else 3e-2
    assert torch.allclose(out.cpu().double(), want, atol=tol, rtol=tol), float((out.cpu().double() - want).abs().max())


# ----------------------------------------------------------------------------- whole models
@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(SHAPES))
def test_whole_prompts_with_the_residual_after_every_layer(folders, name, dtype):
    folder, cfg, W, page = pick(folders, name, dtype)
    eng = engine(folder, dtype, page)
    seqs = [random_tokens(n, cfg["vocab"], 10 + n) for n in (1, 2, 45, 130)]
    layers = {}
    eng.model.layer_hook = lambda ci, x: layers.__setitem__(ci, x.float().cpu().numpy().copy())
    for i, s in enumerate(seqs):
        got = run_schedule(eng, [s], [[(0, len(s))]])[0]
        compare(got, cfg, W, s, dtype, f"{name} whole prompt of {len(s)}")
        if dtype == "float32":
            _, after = P.plain_forward(cfg, W, s)
            for ci in range(len(cfg["layers"])):
                assert np.allclose(layers[ci][:len(s)], after[ci].numpy(), atol=2e-4, rtol=2e-5), (name, ci)


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["t1", "t2", "t4"])
def test_prompt_then_single_tokens_and_from_the_first_token(folders, name, dtype):
    folder, cfg, W, page = pick(folders, name, dtype)
    eng = engine(folder, dtype, page)
    s = random_tokens(97, cfg["vocab"], 3)
    got = run_schedule(eng, [s], [[(0, 40)]] + [[(0, 1)]] * 57)[0]          # the windows and several pages pass over decoded tokens
    compare(got, cfg, W, s, dtype, f"{name} prompt then single tokens")
    s = random_tokens(30, cfg["vocab"], 4)
    got = run_schedule(eng, [s], [[(0, 1)]] * 30)[0]
    compare(got, cfg, W, s, dtype, f"{name} decoded from the first token")


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["t1", "t2", "t3"])
def test_portions_of_every_size(folders, name, dtype):
    folder, cfg, W, page = pick(folders, name, dtype)
    eng = engine(folder, dtype, page)
    s = random_tokens(140, cfg["vocab"], 5)
    for cuts in ([2] * 70, [3, 5, 7, 11, 13, 17, 19, 23, 29, 13], [64, 2, 2, 1, 1, 70], [16, 17, 15, 33, 31, 8, 20]):
        assert sum(cuts) == 140
        got = run_schedule(eng, [s], [[(0, n)] for n in cuts])[0]
        compare(got, cfg, W, s, dtype, f"{name} portions {cuts[:4]}")


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["t1", "t2"])
def test_unequal_requests_through_few_slots_and_pages(folders, name, dtype):
    """Six requests through three slots and a pool that holds about two of them: pages and state slots are freed and
    used again; each request's logits equal the plain ones and those of the request run alone."""
    folder, cfg, W, page = pick(folders, name, dtype)
    lens = [61, 9, 100, 33, 2, 77]
    seqs = [random_tokens(n, cfg["vocab"], 20 + n) for n in lens]
    eng = engine(folder, dtype, page, tokens=208, batch=128, reqs=3)
    schedule = [[(0, 17), (1, 9)], [(0, 30), (2, 64)], [(0, 1), (2, 2), (3, 5)], [(0, 13), (2, 34), (3, 1)], [(3, 27), (4, 2)],
                [(5, 50)], [(5, 1)], [(5, 26)]]
    got = run_schedule(eng, seqs, schedule)
    alone = engine(folder, dtype, page, tokens=208, batch=128, reqs=3)
    for i, s in enumerate(seqs):
        compare(got[i], cfg, W, s, dtype, f"{name} request {i} in the batch")
        single = run_schedule(alone, [s], [[(0, len(s))]])[0]
        if dtype == "float32":
            assert np.allclose(got[i], single, atol=3e-4, rtol=1e-4), (name, i)


@gpu
def test_long_decoding(folders):
    folder, cfg, W, page = folders["t2"]
    eng = engine(folder, "float32", page, tokens=640)
    s = random_tokens(420, cfg["vocab"], 8)
    got = run_schedule(eng, [s], [[(0, 20)]] + [[(0, 1)]] * 400)[0]
    compare(got, cfg, W, s, "float32", "t2 four hundred single tokens")


@gpu
def test_greedy_generation_through_the_engine(folders):
    """Through the engine's own entry points and scheduler: add_request / run_step for unequal requests at once, and
    generate."""
    import airun_b200
    folder, cfg, W, page = folders["t1"]
    eng = engine(folder, "float32", page)
    prompts = [random_tokens(n, cfg["vocab"], 40 + n) for n in (5, 23, 1)]
    reqs = [eng.add_request(p, airun_b200.SamplingParams.greedy(), max_new_tokens=12) for p in prompts]
    while eng.scheduler.has_work():
        eng.run_step()
    for p, r in zip(prompts, reqs):
        assert r.output == P.plain_greedy(cfg, W, p, 12)
    one = eng.generate(prompts[1], airun_b200.SamplingParams.greedy(), max_new_tokens=12)
    assert one.token_ids == P.plain_greedy(cfg, W, prompts[1], 12)
    eng.manager.check_invariants()


@gpu
def test_replay_tool_on_a_folder(folders, tmp_path):
    folder, cfg, W, page = folders["t2"]
    a, b = random_tokens(50, cfg["vocab"], 1), random_tokens(21, cfg["vocab"], 2)
    r = Replay(folder, "float32", str(tmp_path / "out"), max_tokens=128)
    try:
        r1 = r.step([{"id": "a", "tokens": a[:30], "want": [0, 29]}])
        r2 = r.step([{"id": "a", "tokens": a[30:49], "want": []}, {"id": "b", "tokens": b, "want": [20]}], end=["b"])
        r3 = r.step([{"id": "a", "tokens": a[49:], "want": [0]}], end=["a"])
    finally:
        r.close()
    la, lb = P.plain_forward(cfg, W, a)[0].numpy(), P.plain_forward(cfg, W, b)[0].numpy()
    assert_close(np.concatenate([r1, r2, r3]), np.stack([la[0], la[29], lb[20], la[49]]).astype(np.float32), "float32", "replay")
