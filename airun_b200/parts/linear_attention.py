"""Gated linear attention: a recurrent mixer whose state is a matrix per head.

With h the mixer's input, per head of D key channels and Dv value channels:

    q = Wq h * D^-1/2,  k = Wk h,  v = Wv h,  gate = Wg h
    a = sigmoid(W2 (W1 h) + b2)^(1/tau)          (a decay per key channel, through a low-rank pair)
    S <- diag(a) S + k v^T,   o = S^T q          (token by token; S is zero when a request starts)
    out = Wo concat_heads( o / rms(o) * w_norm * silu(gate) )

The state, the decays and the norm are float32; the state of a request lives in its slot of the cache
manager's state tensor between steps (``StateSpec``), so prompts cut into portions, single decoded
tokens and whole prompts run the same recurrence.  The five input projections run as one product over
the stacked matrix [Wq; Wk; Wv; Wg; W1].  The part has the split form (parts/base.py): ``forward_core``
leaves the gated, normed heads in a buffer and ``w_out`` is Wo.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from ..weights.loader import WeightSpec
from .base import Mixer, StateSpec, register_part
from .linear import linear


class GatedLinearAttention(Mixer):
    device_driven = True

    def __init__(self, prefix: str, hidden_size: int, num_heads: int, key_dim: int, value_dim: int, decay_rank: int,
                 tau: float, norm_eps: float, q_scale: Optional[float] = None,
                 dtype: torch.dtype = torch.bfloat16, device=None, names: Optional[Dict[str, str]] = None):
        self.prefix, self.H = prefix, int(hidden_size)
        self.nh, self.D, self.Dv, self.rank = int(num_heads), int(key_dim), int(value_dim), int(decay_rank)
        if min(self.nh, self.D, self.Dv, self.rank) <= 0:
            raise ValueError("heads, key, value and decay sizes must be positive")
        if self.D > 256:
            raise ValueError(f"{self.D} key channels a head are above the recurrence kernel's limit of 256")
        self.tau, self.eps = float(tau), float(norm_eps)
        if not self.tau > 0:
            raise ValueError(f"tau must be positive, found {tau}")
        self.q_scale = float(q_scale) if q_scale is not None else self.D ** -0.5
        self.dtype, self.device = dtype, device
        n = dict(q="q", k="k", v="v", gate="g", o="o", norm="norm", decay_in="a1", decay_out="a2", decay_bias="a2.b")
        n.update(names or {})
        self.names = {k: f"{prefix}.{v}" for k, v in n.items()}
        self.w_in = self.w_out = self.w_decay = self.decay_bias = self.norm_w = None
        self.core_width = self.nh * self.Dv

    # ---- weights ----
    def weight_specs(self) -> List[WeightSpec]:
        nm, H, kd, vd = self.names, self.H, self.nh * self.D, self.nh * self.Dv
        return [WeightSpec(nm["q"], (kd, H)), WeightSpec(nm["k"], (kd, H)), WeightSpec(nm["v"], (vd, H)),
                WeightSpec(nm["gate"], (vd, H)), WeightSpec(nm["o"], (H, vd)),
                WeightSpec(nm["norm"], (self.Dv,), storage="float32", init="norm"),
                WeightSpec(nm["decay_in"], (self.rank, H)), WeightSpec(nm["decay_out"], (kd, self.rank)),
                WeightSpec(nm["decay_bias"], (kd,), storage="float32", init="normal")]

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        nm = self.names
        self.w_in = torch.cat([tensors.pop(nm[k]) for k in ("q", "k", "v", "gate", "decay_in")], dim=0).contiguous()
        self.w_out = tensors.pop(nm["o"])
        self.w_decay = tensors.pop(nm["decay_out"])
        self.decay_bias, self.norm_w = tensors[nm["decay_bias"]], tensors[nm["norm"]]

    def adopt_w_out(self, view: torch.Tensor) -> None:
        self.w_out = view

    # ---- cache ----
    def cache_spec(self):
        return StateSpec((self.nh, self.D, self.Dv), torch.float32)

    # ---- compute ----
    def forward_core(self, ctx, h: torch.Tensor, act: torch.Tensor, cache) -> None:
        T, ws = h.shape[0], ctx.ws
        kd, vd = self.nh * self.D, self.nh * self.Dv
        proj = ws.alloc((T, 2 * kd + 2 * vd + self.rank), torch.float32)
        linear(ctx, h, self.w_in, proj)
        q, k, v = proj[:, :kd], proj[:, kd:2 * kd], proj[:, 2 * kd:2 * kd + vd]
        gate, low = proj[:, 2 * kd + vd:2 * kd + 2 * vd], proj[:, 2 * kd + 2 * vd:]
        decay = ws.alloc((T, kd), torch.float32)
        ops.gla_decay(low, self.w_decay, self.decay_bias, self.tau, decay, ctx.req_of_token)
        o = ws.alloc((T, vd), torch.float32)
        ops.gla_recurrent(q, k, v, decay, cache.state, ctx.cu_tokens, ctx.state_slots, ctx.num_reqs, o,
                          self.nh, self.D, self.Dv, self.q_scale, ctx.err)
        ops.gla_out_gate(o, gate, self.norm_w, self.eps, act, self.nh, self.Dv, ctx.req_of_token)

    def forward(self, ctx, h, cache, sink=None):
        T = h.shape[0]
        act = ctx.ws.alloc((T, self.core_width), self.dtype)
        self.forward_core(ctx, h, act, cache)
        delta = ctx.ws.alloc((T, self.H), torch.float32)
        linear(ctx, act, self.w_out, delta)
        return delta


register_part("mixer", "gated_linear_attention", GatedLinearAttention)


class DecayLinearAttention(Mixer):
    """Linear attention with ONE fixed decay per head:

        q = silu(Wq h),  k = silu(Wk h),  v = silu(Wv h)          head by head, D key and Dv value channels
        S <- d_h S + k v^T,   o = S^T q                           token by token; S is zero when a request starts
        out = out_scale * Wo ( concat_heads(o) / rms(concat_heads(o)) * w_norm * sigmoid(Wg h) )

    The root mean square runs over ALL heads of a token at once.  The decays are numbers of the configuration, not
    tensors.  The state, the recurrence, the norm and the gate are float32; the state of a request lives in its slot of
    the cache manager's state tensor between steps.  The four input projections run as one product; the part has the
    split form (parts/base.py) and can be handed the columns of a product an arrangement has run (``proj``)."""
    device_driven = True

    def __init__(self, prefix: str, hidden_size: int, num_heads: int, key_dim: int, value_dim: int, decay, norm_eps: float,
                 out_scale: float = 1.0, dtype: torch.dtype = torch.bfloat16, device=None,
                 names: Optional[Dict[str, str]] = None):
        self.prefix, self.H = prefix, int(hidden_size)
        self.nh, self.D, self.Dv = int(num_heads), int(key_dim), int(value_dim)
        if min(self.nh, self.D, self.Dv) <= 0:
            raise ValueError("heads, key and value sizes must be positive")
        if self.D > 256:
            raise ValueError(f"{self.D} key channels a head are above the recurrence kernel's limit of 256")
        decay = [float(d) for d in decay]
        if len(decay) != self.nh:
            raise ValueError(f"{len(decay)} decays for {self.nh} heads")
        self.decay = torch.tensor(decay, dtype=torch.float32, device=device)
        self.eps, self.out_scale = float(norm_eps), float(out_scale)
        self.dtype, self.device = dtype, device
        n = dict(q="q", k="k", v="v", gate="g", o="o", norm="norm")
        n.update(names or {})
        self.names = {k: f"{prefix}.{v}" for k, v in n.items()}
        self.w_in = self.w_out = self.norm_w = None
        self.core_width = self.nh * self.Dv

    def weight_specs(self) -> List[WeightSpec]:
        nm, H, kd, vd = self.names, self.H, self.nh * self.D, self.nh * self.Dv
        return [WeightSpec(nm["q"], (kd, H)), WeightSpec(nm["k"], (kd, H)), WeightSpec(nm["v"], (vd, H)),
                WeightSpec(nm["gate"], (vd, H)), WeightSpec(nm["o"], (H, vd)),
                WeightSpec(nm["norm"], (vd,), storage="float32", init="norm")]

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        nm = self.names
        self.w_in = torch.cat([tensors.pop(nm[k]) for k in ("q", "k", "v", "gate")], dim=0).contiguous()
        self.w_out = tensors.pop(nm["o"])
        self.norm_w = tensors[nm["norm"]]
        self.decay = self.decay.to(self.w_in.device)

    def adopt_w_out(self, view: torch.Tensor) -> None:
        self.w_out = view

    def cache_spec(self):
        return StateSpec((self.nh, self.D, self.Dv), torch.float32)

    def forward_core(self, ctx, h, act: torch.Tensor, cache, proj: Optional[torch.Tensor] = None) -> None:
        T, ws = act.shape[0], ctx.ws
        kd, vd = self.nh * self.D, self.nh * self.Dv
        if proj is None:
            proj = ws.alloc((T, 2 * kd + 2 * vd), torch.float32)
            linear(ctx, h, self.w_in, proj)
        q, k, v, gate = proj[:, :kd], proj[:, kd:2 * kd], proj[:, 2 * kd:2 * kd + vd], proj[:, 2 * kd + vd:2 * kd + 2 * vd]
        o = ws.alloc((T, vd), torch.float32)
        ops.decay_recurrent(q, k, v, self.decay, True, cache.state, ctx.cu_tokens, ctx.state_slots, ctx.num_reqs, o,
                            self.nh, self.D, self.Dv, 1.0, ctx.err)
        ops.rownorm_gate(o, gate, self.norm_w, self.eps, act, ctx.req_of_token, scale=self.out_scale)

    def forward(self, ctx, h, cache, sink=None):
        T = h.shape[0]
        act = ctx.ws.alloc((T, self.core_width), self.dtype)
        self.forward_core(ctx, h, act, cache)
        delta = ctx.ws.alloc((T, self.H), torch.float32)
        linear(ctx, act, self.w_out, delta)
        return delta


register_part("mixer", "decay_linear_attention", DecayLinearAttention)
