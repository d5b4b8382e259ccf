"""A plain, slow implementation of the Tagulix decoder for the tests: whole sequences, no cache, torch on the CPU in
float64 unless told otherwise, one function per mechanism.  It shares no code with the package.

Notation: T tokens, width W; a linear weight is [out, in] and applied as x @ w.T.  ``rnd`` (optional) rounds a tensor
where the bfloat16 engine stores one in bfloat16 (the inputs of the products, cached keys and values); it is the
identity for the exact result.

The residual is S streams x_1..x_S, all equal to the embedding at the start.  A sub-layer f with norm weight n and
the numbers a[S] (read), M[S, S] (carry, indexed [from, to]) and b[S] (write) does

    u = sum_s a[s] x_s,   y = f(rms(u) * n),   x_t <- sum_s M[s, t] x_s + m * b[t] * y     for all t at once,

with m one number of the model.  A layer is a mixer sub-layer and then a feed-forward sub-layer; the model's output
is head(rms(sum_s x_s) * n_final).  A model without streams keeps one x and adds m * y to it.

Mixers.  "attention": grouped softmax attention with biases on its four projections, neighbouring dimensions (2i,
2i + 1) of the first r dimensions of every head turned by p * base^(-2i / r), then q and k each divided by their root
mean square over the head, a window of the last w positions.  "parallel": the weighted sum of (left) a causal softmax
attention whose q and k pass a root-mean-square norm with a weight shared by all heads, whose q grows with the position
by 1 + c * ln(floor((p + 1) / e) + 1), whose scores get a learnt number per head and distance bucket, and whose
denominator holds one more term exp(sink_h); and (right) a linear attention with one decay per head,
S <- d_h S + k v^T, o = S^T q over silu-activated q, k, v, normed over all heads at once, gated by sigmoid(G h).

Feed-forward: routed experts W_down gelu(W_up h) (the erf form), chosen by softmax scores plus a correction inside
the best groups of neighbouring experts; the last few router outputs stand for experts that return their input.
"""
from __future__ import annotations

import math
from typing import Callable, Dict, List, Optional, Tuple

import torch

Rounding = Optional[Callable[[torch.Tensor], torch.Tensor]]


def _r(rnd: Rounding, t: torch.Tensor) -> torch.Tensor:
    return t if rnd is None else rnd(t)


def to_bf16_and_back(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.bfloat16).to(t.dtype)


# ----------------------------------------------------------------------------- small pieces
def plain_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def plain_rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return plain_rms(x, eps) * w


def plain_gelu_erf(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def plain_silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def plain_causal(T: int, window: int = 0) -> torch.Tensor:
    """[T, T] True where query i sees key j: j <= i, and i - j < window when there is one."""
    i = torch.arange(T).unsqueeze(1)
    j = torch.arange(T).unsqueeze(0)
    see = j <= i
    if window > 0:
        see &= (i - j) < window
    return see


# ----------------------------------------------------------------------------- rotation
def plain_rotate_pairs(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [T, heads, D]: the pairs (2i, 2i + 1), i < dims / 2, of every head turned by p * base^(-2i / dims)."""
    out = x.clone()
    for i in range(dims // 2):
        ang = positions.to(torch.float64) * (base ** (-2.0 * i / dims))
        c, s = torch.cos(ang).to(x.dtype)[:, None], torch.sin(ang).to(x.dtype)[:, None]
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = u * c - v * s
        out[..., 2 * i + 1] = v * c + u * s
    return out


# ----------------------------------------------------------------------------- softmax attention
def plain_distance_bucket(n: int, rows: int, far: int) -> int:
    """The row of a table of ``rows`` rows that distance n >= 0 reads: one row per distance below rows / 2, then rows
    spread evenly over the logarithm of the distance up to ``far``, the last row for everything beyond."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def plain_query_temperature(positions: torch.Tensor, coef: float, every: int) -> torch.Tensor:
    steps = torch.div(positions + 1, every, rounding_mode="floor")
    return 1.0 + coef * torch.log(steps.to(torch.float64) + 1.0)


def plain_softmax_attention(q, k, v, heads: int, kv_heads: int, scale: float, window: int = 0,
                            bias: Optional[torch.Tensor] = None, sink: Optional[torch.Tensor] = None,
                            rnd: Rounding = None) -> torch.Tensor:
    """q [T, heads, D], k [T, kv_heads, D], v [T, kv_heads, Dv] -> [T, heads * Dv].  ``bias`` [heads, T, T] is added
    to the scaled scores; ``sink`` [heads] adds exp(sink_h) to the denominator and nothing to the numerator.  ``rnd``
    rounds the weights where the tensor-core kernel hands them to the second product (it forms them in float32)."""
    T = q.shape[0]
    see = plain_causal(T, window)
    outs = []
    for h in range(heads):
        g = h // (heads // kv_heads)
        s = (q[:, h] @ k[:, g].T) * scale
        if bias is not None:
            s = s + bias[h]
        s = s.masked_fill(~see, -math.inf)
        top = s.max(dim=-1, keepdim=True).values
        if sink is not None:
            top = torch.maximum(top, sink[h].expand_as(top))
        e = torch.exp(s - top)
        den = e.sum(dim=-1, keepdim=True)
        if sink is not None:
            den = den + torch.exp(sink[h] - top)
        outs.append(_r(rnd, e / den) @ v[:, g])
    return torch.cat(outs, dim=-1)


def plain_window_attention(h, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float, rnd: Rounding = None):
    """The mixer "attention"."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = (h @ W[p + ".q"].T + W[p + ".q.b"]).view(T, H, D)
    k = (h @ W[p + ".k"].T + W[p + ".k.b"]).view(T, G, D)
    v = (h @ W[p + ".v"].T + W[p + ".v.b"]).view(T, G, Dv)
    rot = m.get("rot")
    if rot:
        q = plain_rotate_pairs(q, pos, rot["dims"], rot["base"])
        k = plain_rotate_pairs(k, pos, rot["dims"], rot["base"])
    q, k = plain_rms(q, eps), plain_rms(k, eps)
    window = (m.get("mask") or {}).get("size", 0)
    o = plain_softmax_attention(_r(rnd, q), _r(rnd, k), _r(rnd, v), H, G, m["scale"], window, rnd=rnd)
    return _r(rnd, o) @ W[p + ".o"].T + W[p + ".o.b"]


def plain_bias_attention(h, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float, rnd: Rounding = None, out_scale: float = 1.0):
    """The left half of the mixer "parallel", times ``out_scale`` (applied to the heads' results, where the engine
    rounds them)."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = plain_rmsnorm((h @ W[p + ".q"].T).view(T, H, D), W[p + ".q.norm"], eps)
    k = plain_rmsnorm((h @ W[p + ".k"].T).view(T, G, D), W[p + ".k.norm"], eps)
    v = (h @ W[p + ".v"].T).view(T, G, Dv)
    temp = m.get("q_temp")
    if temp:
        q = q * plain_query_temperature(pos, temp["coef"], temp["every"]).to(q.dtype)[:, None, None]
    rel = W[p + ".rel"]
    rows = rel.shape[0]
    bucket = torch.tensor([[plain_distance_bucket(i - j, rows, m["bias_max"]) if j <= i else 0 for j in range(T)]
                           for i in range(T)])
    bias = rel[bucket].permute(2, 0, 1)                       # [heads, T, T]
    o = plain_softmax_attention(_r(rnd, q), _r(rnd, k), _r(rnd, v), H, G, m["scale"], 0, bias=bias, sink=W[p + ".sink"], rnd=rnd)
    return _r(rnd, out_scale * o) @ W[p + ".o"].T


# ----------------------------------------------------------------------------- linear attention with a fixed decay
def plain_decay_recurrence(q, k, v, decay: List[float], state: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """q, k [T, heads, D], v [T, heads, Dv] -> (o [T, heads, Dv], final state [heads, D, Dv]), token by token."""
    T, H, D = q.shape
    Dv = v.shape[-1]
    S = torch.zeros(H, D, Dv, dtype=q.dtype) if state is None else state.clone()
    d = torch.tensor(decay, dtype=q.dtype)[:, None, None]
    o = torch.zeros(T, H, Dv, dtype=q.dtype)
    for t in range(T):
        S = d * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return o, S


def plain_decay_attention(h, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float, rnd: Rounding = None, out_scale: float = 1.0):
    """The right half of the mixer "parallel", times ``out_scale``.  The engine keeps q, k and v of the recurrence in
    float32, so nothing is rounded before the gated, normed heads."""
    T = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    q = plain_silu(h @ W[p + ".q"].T).view(T, H, D)
    k = plain_silu(h @ W[p + ".k"].T).view(T, H, D)
    v = plain_silu(h @ W[p + ".v"].T).view(T, H, Dv)
    o, _ = plain_decay_recurrence(q, k, v, m["decay"])
    o = plain_rmsnorm(o.reshape(T, H * Dv), W[p + ".norm"], eps) * torch.sigmoid(h @ W[p + ".g"].T)
    return _r(rnd, out_scale * o) @ W[p + ".o"].T


def plain_parallel_mixer(h, W, p: str, m: dict, eps: float, rnd: Rounding = None):
    return plain_bias_attention(h, W, p + ".left", m["left"], eps, rnd, m["left_scale"]) \
        + plain_decay_attention(h, W, p + ".right", m["right"], eps, rnd, m["right_scale"])


# ----------------------------------------------------------------------------- routed experts
def plain_route(z: torch.Tensor, correction: torch.Tensor, top: int, groups: int, keep: int, scale: float):
    """z [T, E] router outputs -> (ids [T, top], weights [T, top]).  Scores are the softmax over all outputs; the choice
    is by score + correction among the outputs of the ``keep`` groups (of ``groups`` equal runs of neighbours) whose
    best such sum is largest; the weights are the chosen scores over their sum, times ``scale``."""
    T, E = z.shape
    s = torch.softmax(z, dim=-1)
    c = s + correction
    if groups > 1:
        best = c.view(T, groups, E // groups).max(dim=-1).values
        kept = torch.topk(best, keep, dim=-1).indices
        ok = torch.zeros(T, groups, dtype=torch.bool)
        ok.scatter_(1, kept, True)
        c = c.masked_fill(~ok.repeat_interleave(E // groups, dim=1), -math.inf)
    ids = torch.topk(c, top, dim=-1).indices
    w = s.gather(1, ids)
    return ids, w / (w.sum(dim=-1, keepdim=True) + 1e-20) * scale


def plain_moe(h, W: Dict[str, torch.Tensor], p: str, mlp: dict, rnd: Rounding = None, router_in=None):
    r = mlp["router"]
    E, ident = r["experts"], r.get("identity", 0)
    g = r.get("groups") or {}
    zin = h if router_in is None else router_in
    ids, wts = plain_route(zin @ W[p + ".router"].T.to(zin.dtype), W[p + ".correction"].to(zin.dtype), r["top"], g.get("count", 1), g.get("keep", 1),
                           r.get("scale", 1.0))
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(r["top"]):
            e = int(ids[t, j])
            if e >= E:                      # one of the last ``ident`` outputs: the input itself
                out[t] += wts[t, j] * h[t]
            else:
                a = plain_gelu_erf(h[t] @ W[f"{p}.e{e}.up"].T)
                out[t] += wts[t, j] * (_r(rnd, a) @ W[f"{p}.e{e}.down"].T)
    return out


# ----------------------------------------------------------------------------- streams
def plain_streams_read(xs: torch.Tensor, a: torch.Tensor) -> torch.Tensor:
    """xs [S, T, W], a [S] -> sum_s a[s] xs[s]."""
    return torch.einsum("s,stw->tw", a, xs)


def plain_streams_write(xs: torch.Tensor, y: torch.Tensor, M: torch.Tensor, b: torch.Tensor, mult: float) -> torch.Tensor:
    """x_t <- sum_s M[s, t] x_s + mult * b[t] * y, every t from the old streams."""
    return torch.einsum("st,sjw->tjw", M, xs) + mult * b[:, None, None] * y[None]


# ----------------------------------------------------------------------------- the model
def plain_forward(config: dict, W: Dict[str, torch.Tensor], tokens: List[int], rnd: Rounding = None,
                  dtype=torch.float64) -> Tuple[torch.Tensor, torch.Tensor]:
    """(logits [T, vocab], the sum of the streams after every layer [layers, T, width])."""
    W = {n: (t.to(dtype) if t.is_floating_point() else t) for n, t in W.items()}
    eps, mult = config["norm"]["eps"], config.get("residual_mult", 1.0)
    S = config.get("streams")
    x = W["embed"][torch.tensor(tokens)]
    xs = x[None].repeat(S or 1, 1, 1)
    after = []
    for i, layer in enumerate(config["layers"]):
        src = layer.get("weights_of", i)
        p = f"l{src}"
        subs = [(1, lambda h: (plain_window_attention(h, W, p + ".mix", layer["mixer"], eps, rnd) if layer["type"] == "attention"
                               else plain_parallel_mixer(h, W, p + ".mix", layer["mixer"], eps, rnd)))]
        if layer.get("mlp"):
            subs.append((2, lambda h: plain_moe(h, W, p + ".mlp", layer["mlp"], rnd)))
        for q, f in subs:
            if S:
                u = plain_streams_read(xs, W[f"{p}.hc{q}.in"])
                y = f(_r(rnd, plain_rmsnorm(u, W[f"{p}.norm{q}"], eps)))
                xs = plain_streams_write(xs, y, W[f"{p}.hc{q}.mix"], W[f"{p}.hc{q}.out"], mult)
            else:
                xs = xs + mult * f(_r(rnd, plain_rmsnorm(xs[0], W[f"{p}.norm{q}"], eps)))[None]
        after.append(xs.sum(dim=0))
    h = _r(rnd, plain_rmsnorm(xs.sum(dim=0), W["final.norm"], eps))
    return h @ W["head"].T, torch.stack(after)


def plain_greedy(config: dict, W, prompt: List[int], n_new: int) -> List[int]:
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(torch.argmax(plain_forward(config, W, toks)[0][-1])))
    return toks[len(prompt):]


# ----------------------------------------------------------------------------- configurations and weights
def moe(ff: int, experts: int, top: int, identity: int = 0, scale: float = 1.0, groups=(1, 1)) -> dict:
    return dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top, identity=identity, scale=scale,
                                                             groups=dict(count=groups[0], keep=groups[1])))


def attention_layer(heads, kv_heads, dim, vdim, scale=None, window=None, rot=None, mlp=None, weights_of=None) -> dict:
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale if scale is not None else 3.0 * dim ** -0.5)
    if window:
        m["mask"] = dict(size=window)
    if rot:
        m["rot"] = dict(dims=rot[0], base=rot[1])
    out = dict(type="attention", mixer=m, mlp=mlp)
    if weights_of is not None:
        out["weights_of"] = weights_of
    return out


def parallel_layer(heads, kv_heads, dim, vdim, bias_max, lin_heads, lin_dim, lin_vdim, decay, scale=None, temp=None,
                   left_scale=1.0, right_scale=1.0, mlp=None, weights_of=None) -> dict:
    left = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale if scale is not None else 1.5 * dim ** -0.5,
                bias_max=bias_max)
    if temp:
        left["q_temp"] = dict(coef=temp[0], every=temp[1])
    right = dict(heads=lin_heads, dim=lin_dim, vdim=lin_vdim, decay=list(decay))
    out = dict(type="parallel", mixer=dict(left=left, right=right, left_scale=left_scale, right_scale=right_scale), mlp=mlp)
    if weights_of is not None:
        out["weights_of"] = weights_of
    return out


def make_config(vocab, width, layers, eps=1e-5, mult=1.0, streams=None) -> dict:
    import json
    d = dict(architecture="Tagulix", vocab=vocab, width=width, norm=dict(eps=eps), residual_mult=mult, layers=layers)
    if streams is not None:
        d["streams"] = streams
    return json.loads(json.dumps(d))


def all_experts(config: dict) -> dict:
    """The same model with every router choosing ALL its outputs (every group kept; the weights still come from the
    scores): a choice that no rounding can change, for comparisons in reduced precision."""
    import json
    out = json.loads(json.dumps(config))
    for l in out["layers"]:
        if l.get("mlp"):
            r = l["mlp"]["router"]
            r["top"] = r["experts"] + r.get("identity", 0)
            r["groups"]["keep"] = r["groups"]["count"]
    return out


def tensor_shapes(config: dict, rel_rows: int = 8) -> Dict[str, tuple]:
    Wd, S, shapes = config["width"], config.get("streams"), {}
    shapes["embed"] = (config["vocab"], Wd)
    shapes["head"] = (config["vocab"], Wd)
    shapes["final.norm"] = (Wd,)
    for i, l in enumerate(config["layers"]):
        if "weights_of" in l:
            continue
        p, m = f"l{i}", l["mixer"]
        x = p + ".mix."
        shapes[p + ".norm1"] = (Wd,)
        if l["type"] == "attention":
            H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            shapes.update({x + "q": (H * D, Wd), x + "q.b": (H * D,), x + "k": (G * D, Wd), x + "k.b": (G * D,),
                           x + "v": (G * Dv, Wd), x + "v.b": (G * Dv,), x + "o": (Wd, H * Dv), x + "o.b": (Wd,)})
        else:
            a, r = m["left"], m["right"]
            H, G, D, Dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            shapes.update({x + "left.q": (H * D, Wd), x + "left.k": (G * D, Wd), x + "left.v": (G * Dv, Wd), x + "left.o": (Wd, H * Dv),
                           x + "left.q.norm": (D,), x + "left.k.norm": (D,), x + "left.rel": (rel_rows, H), x + "left.sink": (H,)})
            H, D, Dv = r["heads"], r["dim"], r["vdim"]
            shapes.update({x + "right.q": (H * D, Wd), x + "right.k": (H * D, Wd), x + "right.v": (H * Dv, Wd),
                           x + "right.g": (H * Dv, Wd), x + "right.o": (Wd, H * Dv), x + "right.norm": (H * Dv,)})
        subs = [1]
        mlp = l.get("mlp")
        if mlp:
            subs.append(2)
            r, ff = mlp["router"], mlp["expert"]["ff"]
            shapes.update({p + ".norm2": (Wd,), p + ".mlp.router": (r["experts"] + r["identity"], Wd),
                           p + ".mlp.correction": (r["experts"] + r["identity"],)})
            for e in range(r["experts"]):
                shapes.update({f"{p}.mlp.e{e}.up": (ff, Wd), f"{p}.mlp.e{e}.down": (Wd, ff)})
        if S:
            for q in subs:
                shapes.update({f"{p}.hc{q}.in": (S,), f"{p}.hc{q}.out": (S,), f"{p}.hc{q}.mix": (S, S)})
    return shapes


def random_weights(config: dict, seed: int, gain: float = 1.0, rel_rows: int = 8) -> Dict[str, torch.Tensor]:
    """Weights large enough that every mechanism moves the logits: matrices N(0, gain^2 / fan_in), norm weights near 1
    (the q/k norms larger, so that the attention is peaked), distance biases and sinks of a visible size, connections
    between the streams near a rotation of them; all rounded to bfloat16, the file's type."""
    g = torch.Generator().manual_seed(seed)
    W = {}
    for name, shape in tensor_shapes(config, rel_rows).items():
        leaf = name.rsplit(".", 1)[-1]
        if leaf == "mix":
            S = shape[0]
            t = 0.6 * torch.eye(S) + 0.4 * torch.roll(torch.eye(S), 1, 1) + 0.1 * torch.randn(shape, generator=g)
        elif leaf in ("in", "out"):
            t = 1.0 / shape[0] ** 0.5 + 0.3 * torch.randn(shape, generator=g)
        elif leaf == "rel":
            t = 1.5 * torch.randn(shape, generator=g)
        elif leaf == "sink":
            t = 1.0 + torch.randn(shape, generator=g)
        elif leaf == "correction":
            t = 0.1 * torch.randn(shape, generator=g)
        elif name.endswith("q.norm") or name.endswith("k.norm"):
            t = 1.6 + 0.3 * torch.randn(shape, generator=g)
        elif len(shape) == 2:
            std = 1.0 if name == "embed" else gain / math.sqrt(shape[1])
            if leaf == "router":
                std *= 2.0
            t = torch.randn(shape, generator=g) * std
        elif leaf == "b":
            t = 0.3 * torch.randn(shape, generator=g)
        else:                                               # norm weights
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        W[name] = t.to(torch.bfloat16)
    return W


def write_folder(folder: str, config: dict, W: Dict[str, torch.Tensor]) -> str:
    import json
    import os
    from safetensors.torch import save_file
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(config, f)
    save_file({n: t.contiguous() for n, t in W.items()}, os.path.join(folder, "model.safetensors"))
    return folder
