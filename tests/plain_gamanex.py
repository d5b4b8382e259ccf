"""A plain, slow implementation of the Gamanex decoder for the tests: whole sequences, no cache, torch on the CPU
in float64 unless told otherwise, one function per mechanism.  It shares no code with the package.

Notation: T tokens, width W; a linear weight is [out, in] and applied as x @ w.T.  ``rnd`` (optional) rounds a
tensor where the bfloat16 engine stores one in bfloat16 (the inputs of the products, cached keys and values); it
is the identity for the exact result.

A layer reads the residual stream x through two norms and adds both sub-layers at once:

    h1 = rms(x) * n1,  h2 = rms(x) * n2
    x <- x + s1 * sigmoid(G1 h1 + c1) * mixer(h1) + s2 * sigmoid(G2 h2 + c2) * ff(h2)

with s1, s2 vectors of the layer (a scale per channel) and G, c a gate per sub-layer computed from that sub-layer's
own input.  The mixer is an attention without softmax and without rotation: the weight of key j for the query at
position i >= j is sigmoid(scale * q_i . k_j - a_h * ln(1 + b_h * (i - j)) + c_h), not normalised over keys; q and k
pass a root-mean-square norm over their WHOLE projection (all heads at once), and q is multiplied by a temperature
that grows with its position, 1 + coef * ln(floor((p + 1) / every) + 1).  A layer may attend over the keys and
values an earlier layer cached, with queries of its own.  The feed-forward is W_down relu(W_up h)^2, or a mixture
of SwiGLU experts whose router has a bias, takes the ``top`` largest logits and weighs them by the softmax over
those logits alone; a layer may have none.
"""
from __future__ import annotations

import json
import math
import os
from typing import Callable, Dict, List, Optional

import torch

Rounding = Optional[Callable[[torch.Tensor], torch.Tensor]]


def _r(rnd: Rounding, t: torch.Tensor) -> torch.Tensor:
    return t if rnd is None else rnd(t)


def to_bf16_and_back(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.bfloat16).to(t.dtype)


# ----------------------------------------------------------------------------- small pieces
def plain_rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w


def plain_relu2_mlp(h, w_up, w_down, rnd: Rounding = None):
    a = torch.relu(h @ w_up.T) ** 2
    return _r(rnd, a) @ w_down.T


def plain_expert(h, w_gate, w_up, w_down, rnd: Rounding = None):
    g = h @ w_gate.T
    a = g * torch.sigmoid(g) * (h @ w_up.T)
    return _r(rnd, a) @ w_down.T


def plain_router(h, w_router, b_router, top: int):
    """(ids [T, top], weights [T, top]): the ``top`` largest logits of every token and the softmax over them alone."""
    z = h @ w_router.T + b_router
    val, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(val, dim=-1)


def plain_moe(h, W: Dict[str, torch.Tensor], p: str, top: int, rnd: Rounding = None):
    idx, wts = plain_router(h, W[p + ".router"], W[p + ".router.b"], top)
    out = torch.zeros(h.shape[0], W[p + ".e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(idx[t, j])
            out[t] += wts[t, j] * plain_expert(h[t:t + 1], W[f"{p}.e{e}.gate"], W[f"{p}.e{e}.up"], W[f"{p}.e{e}.down"], rnd)[0]
    return out


# ----------------------------------------------------------------------------- attention without softmax
def plain_query_temperature(positions: torch.Tensor, coef: float, every: int) -> torch.Tensor:
    """1 + coef * ln(floor((p + 1) / every) + 1) for every position p."""
    steps = torch.div(positions + 1, every, rounding_mode="floor")
    return 1.0 + coef * torch.log(steps.to(torch.float64) + 1.0)


def plain_distance_bias(T: int, a: float, b: float, first: int = 0) -> torch.Tensor:
    """[T, first + T]: a * ln(1 + b * (i - j)) for the query at position first + i and the key at position j <= it
    (0 where the key is ahead of the query; those places are masked anyway)."""
    i = torch.arange(first, first + T).unsqueeze(1)
    j = torch.arange(first + T).unsqueeze(0)
    d = (i - j).clamp(min=0).to(torch.float64)
    return a * torch.log(1.0 + b * d)


def plain_causal(T: int, first: int = 0) -> torch.Tensor:
    i = torch.arange(first, first + T).unsqueeze(1)
    j = torch.arange(first + T).unsqueeze(0)
    return j <= i


def plain_keys_values(h, W, p: str, m: dict, eps: float, rnd: Rounding = None):
    """What a layer caches: k after its norm over the whole projection [T, G*D], and v [T, G*Dv]."""
    k = plain_rmsnorm(h @ W[p + ".k"].T, W[p + ".k.norm"], eps)
    v = h @ W[p + ".v"].T
    return _r(rnd, k), _r(rnd, v)


def plain_queries(h, W, p: str, m: dict, eps: float, positions, rnd: Rounding = None):
    q = plain_rmsnorm(h @ W[p + ".q"].T, W[p + ".q.norm"], eps)
    temp = m.get("q_temp")
    if temp:
        q = q * plain_query_temperature(positions, temp["coef"], temp["every"]).to(q.dtype).unsqueeze(1)
    return _r(rnd, q)


def plain_sigmoid_attention(q, k, v, m: dict, a, b, c, first: int = 0, rnd: Rounding = None):
    """q [T, H*D] at positions first.., k [first + T, G*D], v [first + T, G*Dv] -> [T, H*Dv].  ``rnd`` rounds the
    weights where the tensor-core kernels hand them to the second product (they are formed in float32)."""
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T, S = q.shape[0], k.shape[0]
    see = plain_causal(T, first)
    out = torch.zeros(T, H * Dv, dtype=q.dtype)
    for hh in range(H):
        g = hh // (H // G)
        s = (q[:, hh * D:(hh + 1) * D] @ k[:, g * D:(g + 1) * D].T) * m["scale"]
        s = s - plain_distance_bias(T, float(a[hh]), float(b[hh]), first).to(q.dtype)
        w = _r(rnd, torch.sigmoid(s + c[hh]) * see)
        out[:, hh * Dv:(hh + 1) * Dv] = w @ v[:, g * Dv:(g + 1) * Dv]
    return out


def plain_attention_mixer(h, W, p: str, m: dict, eps: float, k, v, positions, rnd: Rounding = None):
    q = plain_queries(h, W, p, m, eps, positions, rnd)
    o = plain_sigmoid_attention(q, k, v, m, W[p + ".r1"], W[p + ".r2"], W[p + ".pb"], rnd=rnd)
    return _r(rnd, o) @ W[p + ".o"].T


def plain_gate(h, w, b):
    return torch.sigmoid(h @ w.T + b)


# ----------------------------------------------------------------------------- the model
def plain_forward(cfg: dict, W: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64, rnd: Rounding = None,
                  residuals: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of the whole sequence.  ``residuals`` collects the stream after every layer."""
    W = {n: t.to(dtype) for n, t in W.items()}
    eps = cfg["norm"]["eps"]
    T = len(tokens)
    pos = torch.arange(T)
    x = W["embed"][torch.tensor(tokens)]
    cached = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}", layer["mixer"]
        h1 = _r(rnd, plain_rmsnorm(x, W[p + ".norm1"], eps))
        if "kv_from" in m:
            k, v = cached[m["kv_from"]]
        else:
            k, v = cached[i] = plain_keys_values(h1, W, p + ".mix", m, eps, rnd)
        y = plain_attention_mixer(h1, W, p + ".mix", m, eps, k, v, pos, rnd)
        add = W[p + ".ls1"] * plain_gate(h1, W[p + ".rg1"], W[p + ".rg1.b"]) * y
        mlp = layer.get("mlp")
        if mlp:
            h2 = _r(rnd, plain_rmsnorm(x, W[p + ".norm2"], eps))
            if mlp["kind"] == "dense":
                f = plain_relu2_mlp(h2, W[p + ".mlp.up"], W[p + ".mlp.down"], rnd)
            else:
                f = plain_moe(h2, W, p + ".mlp", mlp["router"]["top"], rnd)
            add = add + W[p + ".ls2"] * plain_gate(h2, W[p + ".rg2"], W[p + ".rg2.b"]) * f
        x = x + add
        if residuals is not None:
            residuals.append(x.clone())
    return (_r(rnd, plain_rmsnorm(x, W["final.norm"], eps)) @ W["head"].T) * cfg.get("logit_scale", 1.0)


def plain_greedy(cfg, W, prompt: List[int], n_new: int) -> List[int]:
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(torch.argmax(plain_forward(cfg, W, toks)[-1])))
    return toks[len(prompt):]


# ----------------------------------------------------------------------------- configurations and weights
def dense(ff: int) -> dict:
    return dict(kind="dense", ff=ff)


def moe(ff: int, experts: int, top: int) -> dict:
    return dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top))


def attention_layer(heads, kv_heads, dim, vdim, scale=None, temp=None, kv_from=None, mlp=None) -> dict:
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale if scale is not None else 1.5 * dim ** -0.5)
    if temp is not None:
        m["q_temp"] = dict(coef=temp[0], every=temp[1])
    if kv_from is not None:
        m["kv_from"] = kv_from
    return dict(type="attention", mixer=m, mlp=mlp)


def all_experts(cfg: dict) -> dict:
    """The same model with every router choosing ALL its experts (the weights still come from the logits): a choice
    that no rounding can change, for comparisons in reduced precision."""
    out = json.loads(json.dumps(cfg))
    for l in out["layers"]:
        if l.get("mlp") and l["mlp"]["kind"] == "moe":
            l["mlp"]["router"]["top"] = l["mlp"]["router"]["experts"]
    return out


def make_config(vocab, width, layers, eps=1e-5, logit_scale=1.0) -> dict:
    return dict(architecture="Gamanex", vocab=vocab, width=width, norm=dict(eps=eps), logit_scale=logit_scale, layers=layers)


def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    Wd, shapes = cfg["width"], {}
    shapes["embed"] = (cfg["vocab"], Wd)
    shapes["head"] = (cfg["vocab"], Wd)
    shapes["final.norm"] = (Wd,)
    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}", l["mixer"]
        x = p + ".mix."
        H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        shapes.update({p + ".norm1": (Wd,), x + "q": (H * D, Wd), x + "q.norm": (H * D,), x + "r1": (H,), x + "r2": (H,),
                       x + "pb": (H,), x + "o": (Wd, H * Dv), p + ".ls1": (Wd,), p + ".rg1": (Wd, Wd), p + ".rg1.b": (Wd,)})
        if "kv_from" not in m:
            shapes.update({x + "k": (G * D, Wd), x + "v": (G * Dv, Wd), x + "k.norm": (G * D,)})
        mlp = l.get("mlp")
        if mlp:
            shapes.update({p + ".norm2": (Wd,), p + ".ls2": (Wd,), p + ".rg2": (Wd, Wd), p + ".rg2.b": (Wd,)})
            if mlp["kind"] == "dense":
                shapes.update({p + ".mlp.up": (mlp["ff"], Wd), p + ".mlp.down": (Wd, mlp["ff"])})
            else:
                ff = mlp["expert"]["ff"]
                shapes.update({p + ".mlp.router": (mlp["router"]["experts"], Wd), p + ".mlp.router.b": (mlp["router"]["experts"],)})
                for e in range(mlp["router"]["experts"]):
                    shapes.update({f"{p}.mlp.e{e}.gate": (ff, Wd), f"{p}.mlp.e{e}.up": (ff, Wd), f"{p}.mlp.e{e}.down": (Wd, ff)})
    return shapes


def random_weights(cfg: dict, seed: int, gain: float = 1.0) -> Dict[str, torch.Tensor]:
    """Weights large enough that every mechanism moves the logits: matrices N(0, gain^2 / fan_in), norm weights and
    layer scales near 1, distance slopes and rates positive and of a visible size, a negative offset in the sigmoid so
    that most keys weigh little; all rounded to bfloat16, the file's type."""
    g = torch.Generator().manual_seed(seed)
    W = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.rsplit(".", 1)[-1]
        if len(shape) == 2:
            std = 1.0 if name == "embed" else gain / math.sqrt(shape[1])
            if leaf == "router":
                std *= 2.0
            t = torch.randn(shape, generator=g) * std
        elif leaf == "norm" or leaf in ("norm1", "norm2") or name == "final.norm":
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif leaf in ("ls1", "ls2"):
            t = 0.8 + 0.2 * torch.randn(shape, generator=g)
        elif leaf == "r1":
            t = 0.3 + 0.5 * torch.rand(shape, generator=g)
        elif leaf == "r2":
            t = 0.2 + 1.5 * torch.rand(shape, generator=g)
        elif leaf == "pb":
            t = -2.0 + 0.7 * torch.randn(shape, generator=g)
        else:                                               # the gates' and the router's biases
            t = 0.5 * torch.randn(shape, generator=g)
        W[name] = t.to(torch.bfloat16)
    return W


def write_folder(folder: str, cfg: dict, W: Dict[str, torch.Tensor]) -> str:
    from safetensors.torch import save_file
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({n: t.contiguous() for n, t in W.items()}, os.path.join(folder, "model.safetensors"))
    return folder
