"""Arrangement of a layer: norm -> mixer -> add -> norm -> feed-forward -> add.

The residual stream ``x`` is float32.  Each sub-layer returns a float32 delta;
the add is carried out by the NEXT norm (x += delta, then norm), as the
reference fuses every residual add with the norm that follows it
(crates/airun-core/src/runtime.rs:3564-3567, :3595-3599).  The block therefore
takes the delta still pending from the block before it and returns its own.

In the bfloat16 path, when the parts on both sides allow it (``fuses_norms``), a norm is not a
kernel of its own at all: the product that ends a sub-layer adds its result to x, writes
bfloat16(x * norm weight) and the sums of x^2 per token, and the product that starts the next
sub-layer scales each token's results by rsqrt(mean x^2 + eps) (parts/base.py NormedActivations).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..weights.loader import WeightSpec
from .base import CastActivations, FeedForward, Mixer, Norm, NormedActivations, Part, ResidualSink, StreamWrite, register_part


class PreNormBlock(Part):
    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Norm, ffn: FeedForward, dtype: torch.dtype):
        self.norm1, self.mixer, self.norm2, self.ffn, self.dtype = norm1, mixer, norm2, ffn, dtype

    def parts(self):
        return (self.norm1, self.mixer, self.norm2, self.ffn)

    def weight_specs(self) -> List[WeightSpec]:
        return [s for p in self.parts() for s in p.weight_specs()]

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        for p in self.parts():
            p.load_weights(tensors)

    def cache_spec(self):
        return self.mixer.cache_spec()

    def device_driven(self) -> bool:
        """Do all parts of this block read the batch's layout from the device arrays only?"""
        return all(getattr(p, "device_driven", False) for p in self.parts())

    def graph_safe(self) -> bool:
        """May steps through this block be captured into CUDA graphs at all?"""
        return all(getattr(p, "graph_safe", True) for p in self.parts())

    def accepts_normed(self) -> bool:
        """Can this block start from NormedActivations (its first norm folded into the products)?"""
        return self.dtype == torch.bfloat16 and getattr(self.mixer, "fuses_norms", False) \
            and hasattr(self.norm1, "fusable")

    def forward(self, ctx, x: torch.Tensor, pending, cache, next_norm: Optional[Norm] = None):
        """``pending``: what the block before left: None, a float32 delta still to be added to x, or
        NormedActivations (x is up to date and this block's first norm is already folded in).
        ``next_norm``: the norm that will read x next, if it may be folded into this block's last
        product; the block then returns NormedActivations instead of a delta."""
        T, H = x.shape
        bf16 = self.dtype == torch.bfloat16
        if isinstance(pending, NormedActivations):
            h = pending
        else:
            h = ctx.ws.alloc((T, H), self.dtype)
            self.norm1.forward(ctx, x, h, delta=pending)
        if bf16 and getattr(self.mixer, "fuses_norms", False) and getattr(self.ffn, "fuses_norms", False) \
                and hasattr(self.norm2, "fusable"):
            a = self.mixer.forward(ctx, h, cache, sink=ResidualSink(x, *self.norm2.fusable()))
        else:
            a = self.mixer.forward(ctx, h, cache)
        if isinstance(a, NormedActivations):
            h2 = a
        else:
            h2 = ctx.ws.alloc((T, H), self.dtype)
            self.norm2.forward(ctx, x, h2, delta=a)
        if bf16 and next_norm is not None and getattr(self.ffn, "fuses_norms", False):
            return self.ffn.forward(ctx, h2, sink=ResidualSink(x, *next_norm.fusable()))
        return self.ffn.forward(ctx, h2)


register_part("arrangement", "pre_norm", PreNormBlock)


class ParallelBlock(Part):
    """One norm, two sub-layers side by side: h = norm(x), x += mixer(h) + ffn(h).  The feed-forward may be
    absent.  As with PreNormBlock the add is left to whoever norms x next: the block returns the delta.

    When both sub-layers have the split form (parts/base.py) their output products run as ONE product:
    each writes its activation into a column slice of one buffer, and that buffer is multiplied by the
    output matrices set side by side, [Wo | Wdown], which is mixer(h) + ffn(h) with a single accumulation and
    no add kernel.  Otherwise both run whole and their deltas are added by a kernel.

    ``add_vec`` (float32 [hidden]): a row added to every token of x before the norm, on the norm's way when
    it can (``takes_add_vec``)."""
    num_norms = 1

    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Optional[Norm], ffn: Optional[FeedForward], dtype: torch.dtype):
        self.norm1, self.mixer, self.ffn, self.dtype = norm1, mixer, ffn, dtype
        self.w_out: Optional[torch.Tensor] = None
        self.split = all(hasattr(p, "forward_core") and hasattr(p, "adopt_w_out") for p in self.subs())

    def subs(self):
        return (self.mixer,) if self.ffn is None else (self.mixer, self.ffn)

    def parts(self):
        return (self.norm1,) + self.subs()

    def weight_specs(self) -> List[WeightSpec]:
        return [s for p in self.parts() for s in p.weight_specs()]

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        for p in self.parts():
            p.load_weights(tensors)
        if self.split and len(self.subs()) > 1:
            self.w_out = torch.cat([p.w_out for p in self.subs()], dim=1).contiguous()
            at = 0
            for p in self.subs():
                p.adopt_w_out(self.w_out[:, at:at + p.core_width])
                at += p.core_width

    def cache_spec(self):
        return self.mixer.cache_spec()

    def device_driven(self) -> bool:
        return all(getattr(p, "device_driven", False) for p in self.parts())

    def graph_safe(self) -> bool:
        return all(getattr(p, "graph_safe", True) for p in self.parts())

    def accepts_normed(self) -> bool:
        return False

    accepts_add_vec = True

    def forward(self, ctx, x: torch.Tensor, pending, cache, next_norm: Optional[Norm] = None, add_vec=None):
        T, H = x.shape
        h = ctx.ws.alloc((T, H), self.dtype)
        if add_vec is not None and not getattr(self.norm1, "takes_add_vec", False):
            from ..kernels import ops
            ops.add_rows(x, delta=pending, vec=add_vec)
            pending, add_vec = None, None
        if add_vec is not None:
            self.norm1.forward(ctx, x, h, delta=pending, add_vec=add_vec)
        else:
            self.norm1.forward(ctx, x, h, delta=pending)
        if self.ffn is None:
            return self.mixer.forward(ctx, h, cache)
        if self.split:
            from .linear import linear
            km = self.mixer.core_width
            act = ctx.ws.alloc((T, km + self.ffn.core_width), self.dtype)
            self.mixer.forward_core(ctx, h, act[:, :km], cache)
            self.ffn.forward_core(ctx, h, act[:, km:])
            delta = ctx.ws.alloc((T, H), torch.float32)
            linear(ctx, act, self.w_out, delta)
            return delta
        from ..kernels import ops
        a = self.mixer.forward(ctx, h, cache)
        ops.add_rows(a, delta=self.ffn.forward(ctx, h))
        return a


register_part("arrangement", "parallel", ParallelBlock)


class PostNormBlock(Part):
    """The norm sits on each sub-layer's OUTPUT: x += m * norm1(mixer(x)), then x += m * norm2(ffn(x)).  The
    sub-layers read the residual stream itself (in the compute type: a bfloat16 copy when serving in bfloat16, x as
    it is on the 32-bit path); ``residual_mult`` m scales what is added.  The feed-forward may be absent, and then
    so is norm2.  Norm and add are one kernel, which also writes the copy the next sub-layer reads; nothing is left
    pending for the next block, which gets that copy as CastActivations.  A mixer that declares
    ``input_float32 = True`` is given x in float32 whatever the compute type.  The norms must offer ``fusable()``
    (weight, eps) of a root-mean-square norm."""
    norm2_belongs_to_ffn = True

    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Optional[Norm], ffn: Optional[FeedForward], dtype: torch.dtype,
                 residual_mult: float = 1.0):
        self.norm1, self.mixer, self.norm2, self.ffn, self.dtype = norm1, mixer, norm2, ffn, dtype
        self.mult = float(residual_mult)
        for n in (norm1, norm2):
            if n is not None and not hasattr(n, "fusable"):
                raise ValueError("a post-norm block needs root-mean-square norms (parts with fusable())")

    def parts(self):
        return tuple(p for p in (self.norm1, self.mixer, self.norm2, self.ffn) if p is not None)

    def weight_specs(self) -> List[WeightSpec]:
        return [s for p in self.parts() for s in p.weight_specs()]

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        for p in self.parts():
            p.load_weights(tensors)

    def cache_spec(self):
        return self.mixer.cache_spec()

    def device_driven(self) -> bool:
        return all(getattr(p, "device_driven", False) for p in self.parts())

    def graph_safe(self) -> bool:
        return all(getattr(p, "graph_safe", True) for p in self.parts())

    def accepts_normed(self) -> bool:
        return False

    def forward(self, ctx, x: torch.Tensor, pending, cache, next_norm: Optional[Norm] = None):
        from ..kernels import ops
        T, H = x.shape
        f32 = self.dtype == torch.float32
        if isinstance(pending, torch.Tensor):           # a block of another arrangement left its delta to be added
            ops.add_rows(x, delta=pending)
            pending = None
        if f32 or getattr(self.mixer, "input_float32", False):
            h = x
        elif isinstance(pending, CastActivations):
            h = pending.h
        else:
            h = ctx.ws.alloc((T, H), self.dtype)
            ops.cast_f32(x, h)
        y = self.mixer.forward(ctx, h, cache)
        cast = None if f32 else ctx.ws.alloc((T, H), self.dtype)
        w, eps = self.norm1.fusable()
        ops.postnorm_add(x, y, w, eps, self.mult, cast=cast)
        if self.ffn is not None:
            y = self.ffn.forward(ctx, x if f32 else cast)
            cast = None if f32 else ctx.ws.alloc((T, H), self.dtype)
            w, eps = self.norm2.fusable()
            ops.postnorm_add(x, y, w, eps, self.mult, cast=cast)
        return None if f32 else CastActivations(cast)


register_part("arrangement", "post_norm", PostNormBlock)


class GatedParallelBlock(Part):
    """Two norms of the same residual stream, two sub-layers side by side, each result scaled per channel and gated by
    a sigmoid of the sub-layer's own input:

        h1 = norm1(x),  h2 = norm2(x)
        x += s1 * sigmoid(G1 h1 + c1) * mixer(h1) + s2 * sigmoid(G2 h2 + c2) * ffn(h2)

    ``layer_scale`` (the vectors s, tensors ``<prefix>.ls1`` / ``.ls2``) and ``gated`` (G and c, ``<prefix>.rg1`` /
    ``.rg1.b`` and ``.rg2`` / ``.rg2.b``) can each be left out; the feed-forward may be absent, and then so are norm2,
    s2 and the second gate.  As with the other arrangements the add is left to whoever norms x next: the block returns
    the sum of the two terms.  Both norms run as ONE pass over x when they are root-mean-square norms with the same
    eps.  A sub-layer that offers ``append_input_rows`` takes its gate's matrix into its own input product (the gate
    reads the same input) and hands the columns back (``forward(..., with_extra=True)``); otherwise the gate is a
    product of its own."""
    norm2_belongs_to_ffn = True

    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Optional[Norm], ffn: Optional[FeedForward], dtype: torch.dtype,
                 prefix: str, hidden_size: int, layer_scale: bool = True, gated: bool = True,
                 names: Optional[Dict[str, str]] = None):
        self.norm1, self.mixer, self.norm2, self.ffn, self.dtype = norm1, mixer, norm2, ffn, dtype
        self.prefix, self.H = prefix, int(hidden_size)
        self.layer_scale, self.gated = bool(layer_scale), bool(gated)
        n = dict(scale="ls{k}", gate="rg{k}", gate_bias="rg{k}.b")
        n.update(names or {})
        self.n = n
        self.scales: List[Optional[torch.Tensor]] = [None, None]
        self.gate_w: List[Optional[torch.Tensor]] = [None, None]      # None once a sub-layer has taken the matrix
        self.gate_b: List[Optional[torch.Tensor]] = [None, None]
        self.gate_in_sub = [False, False]

    def subs(self):
        return (self.mixer,) if self.ffn is None else (self.mixer, self.ffn)

    def parts(self):
        return tuple(p for p in (self.norm1, self.mixer, self.norm2, self.ffn) if p is not None)

    def _name(self, which: str, k: int) -> str:
        return f"{self.prefix}.{self.n[which].format(k=k + 1)}"

    def weight_specs(self) -> List[WeightSpec]:
        specs = [s for p in self.parts() for s in p.weight_specs()]
        for k in range(len(self.subs())):
            if self.layer_scale:
                specs.append(WeightSpec(self._name("scale", k), (self.H,), storage="float32", init="norm"))
            if self.gated:
                specs += [WeightSpec(self._name("gate", k), (self.H, self.H)),
                          WeightSpec(self._name("gate_bias", k), (self.H,), storage="float32")]
        return specs

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        for p in self.parts():
            p.load_weights(tensors)
        for k, sub in enumerate(self.subs()):
            if self.layer_scale:
                self.scales[k] = tensors[self._name("scale", k)]
            if self.gated:
                w = tensors.pop(self._name("gate", k))
                self.gate_b[k] = tensors[self._name("gate_bias", k)]
                if hasattr(sub, "append_input_rows"):
                    sub.append_input_rows(w)
                    self.gate_in_sub[k] = True
                else:
                    self.gate_w[k] = w

    def cache_spec(self):
        return self.mixer.cache_spec()

    def device_driven(self) -> bool:
        return all(getattr(p, "device_driven", False) for p in self.parts())

    def graph_safe(self) -> bool:
        return all(getattr(p, "graph_safe", True) for p in self.parts())

    def accepts_normed(self) -> bool:
        return False

    def _run(self, ctx, k: int, sub, h, *args):
        """(result, gate columns or None) of sub-layer k."""
        if self.gate_in_sub[k]:
            return sub.forward(ctx, h, *args, with_extra=True)
        y = sub.forward(ctx, h, *args)
        if not self.gated:
            return y, None
        from .linear import linear
        g = ctx.ws.alloc((h.shape[0], self.H), torch.float32)
        linear(ctx, h, self.gate_w[k], g)
        return y, g

    def forward(self, ctx, x: torch.Tensor, pending, cache, next_norm: Optional[Norm] = None):
        from ..kernels import ops
        T, H = x.shape
        if not isinstance(pending, torch.Tensor):
            pending = None
        h1 = ctx.ws.alloc((T, H), self.dtype)
        h2 = ctx.ws.alloc((T, H), self.dtype) if self.ffn is not None else None
        pair = h2 is not None and hasattr(self.norm1, "fusable") and hasattr(self.norm2, "fusable") \
            and self.norm1.fusable()[1] == self.norm2.fusable()[1]
        if pair:
            ops.rmsnorm_pair(x, self.norm1.fusable()[0], h1, self.norm2.fusable()[0], h2, self.norm1.fusable()[1], delta=pending)
        else:
            self.norm1.forward(ctx, x, h1, delta=pending)
            if h2 is not None:
                self.norm2.forward(ctx, x, h2)
        y1, g1 = self._run(ctx, 0, self.mixer, h1, cache)
        y2 = g2 = None
        if self.ffn is not None:
            y2, g2 = self._run(ctx, 1, self.ffn, h2)
        if not (self.gated or self.layer_scale or y2 is not None):
            return y1
        ops.gated_sum(y1, y1, g1, self.gate_b[0], self.scales[0], y2, g2, self.gate_b[1], self.scales[1])
        return y1


register_part("arrangement", "gated_parallel", GatedParallelBlock)


class HyperConnectionBlock(Part):
    """A residual of several streams x_1..x_S (hyper-connections).  Each sub-layer f (the mixer, then the feed-forward)
    has numbers of its own, a[S], M[S, S] (indexed [from, to]) and b[S]:

        u = sum_s a[s] x_s,    y = f(norm(u)),    x_t <- sum_s M[s, t] x_s + m * b[t] * y     (all t from the old streams)

    with m (``residual_mult``) one number of the model.  The streams are all equal to the embedding at the start and
    are summed at the end (engine/model.py).  Tensors: ``<prefix>.hc1.{in,mix,out}`` for the mixer and ``.hc2.*`` for
    the feed-forward; with ``learned`` False there are none and every a, M and b is 1 on one stream: the plain pre-norm
    residual x += m * f(norm(x)).  The write of a sub-layer's result and the read and norm for the next one are ONE
    pass over the streams (csrc/streams.cu); the last write of the block is left pending for whoever reads the streams
    next (``StreamWrite``).  A mixer with an ``output_bias`` leaves it to that pass too.  The norms must offer
    ``fusable()`` (weight, eps) of a root-mean-square norm."""
    multi_stream = True
    norm2_belongs_to_ffn = True

    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Optional[Norm], ffn: Optional[FeedForward], dtype: torch.dtype,
                 prefix: str, streams: int = 1, residual_mult: float = 1.0, learned: bool = True,
                 names: Optional[Dict[str, str]] = None):
        self.norm1, self.mixer, self.norm2, self.ffn, self.dtype = norm1, mixer, norm2, ffn, dtype
        self.prefix, self.S, self.mult, self.learned = prefix, int(streams), float(residual_mult), bool(learned)
        if self.S < 1 or (not self.learned and self.S != 1):
            raise ValueError("at least one stream; without learnt connections exactly one")
        for n_ in (norm1, norm2):
            if n_ is not None and not hasattr(n_, "fusable"):
                raise ValueError("a block over several streams needs root-mean-square norms (parts with fusable())")
        n = dict(read="hc{k}.in", carry="hc{k}.mix", write="hc{k}.out")
        n.update(names or {})
        self.n = n
        self.read: List[Optional[torch.Tensor]] = [None, None]
        self.carry: List[Optional[torch.Tensor]] = [None, None]
        self.write: List[Optional[torch.Tensor]] = [None, None]

    def subs(self):
        return (self.mixer,) if self.ffn is None else (self.mixer, self.ffn)

    def parts(self):
        return tuple(p for p in (self.norm1, self.mixer, self.norm2, self.ffn) if p is not None)

    def _name(self, which: str, k: int) -> str:
        return f"{self.prefix}.{self.n[which].format(k=k + 1)}"

    def weight_specs(self) -> List[WeightSpec]:
        specs = [s for p in self.parts() for s in p.weight_specs()]
        if self.learned:
            for k in range(len(self.subs())):
                specs += [WeightSpec(self._name("read", k), (self.S,), storage="float32", init="norm"),
                          WeightSpec(self._name("write", k), (self.S,), storage="float32", init="norm"),
                          WeightSpec(self._name("carry", k), (self.S, self.S), storage="float32", init="normal")]
        return specs

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        for p in self.parts():
            p.load_weights(tensors)
        for k in range(len(self.subs())):
            if self.learned:
                self.read[k], self.write[k] = tensors[self._name("read", k)], tensors[self._name("write", k)]
                self.carry[k] = tensors[self._name("carry", k)]
            else:
                dev = self.norm1.fusable()[0].device
                self.read[k] = torch.ones(1, dtype=torch.float32, device=dev)
                self.write[k] = torch.ones(1, dtype=torch.float32, device=dev)
                self.carry[k] = torch.ones(1, 1, dtype=torch.float32, device=dev)

    def cache_spec(self):
        return self.mixer.cache_spec()

    def device_driven(self) -> bool:
        return all(getattr(p, "device_driven", False) for p in self.parts())

    def graph_safe(self) -> bool:
        return all(getattr(p, "graph_safe", True) for p in self.parts())

    def accepts_normed(self) -> bool:
        return False

    def forward(self, ctx, xs: torch.Tensor, pending, cache, next_norm: Optional[Norm] = None):
        """``xs`` float32 [T, S, H]; ``pending``: None or the StreamWrite the block before left."""
        from ..kernels import ops
        T, S, H = xs.shape
        if pending is not None and not isinstance(pending, StreamWrite):
            raise TypeError("a block over several streams can only follow one of its kind")
        for k, (sub, norm) in enumerate(zip(self.subs(), (self.norm1, self.norm2))):
            w, eps = norm.fusable()
            h = ctx.ws.alloc((T, H), self.dtype)
            p = pending
            ops.stream_step(xs, y=p.y if p else None, carry=p.carry if p else None, write=p.write if p else None,
                            mult=p.mult if p else 1.0, y_bias=p.y_bias if p else None, read=self.read[k], norm_w=w, eps=eps,
                            out=h, req_of_token=ctx.req_of_token)
            if k == 0:
                bias = getattr(sub, "output_bias", None)
                y = sub.forward(ctx, h, cache, add_bias=False) if bias is not None else sub.forward(ctx, h, cache)
            else:
                bias, y = None, sub.forward(ctx, h)
            pending = StreamWrite(y, self.carry[k], self.write[k], self.mult, bias)
        return pending


register_part("arrangement", "hyper_connections", HyperConnectionBlock)
