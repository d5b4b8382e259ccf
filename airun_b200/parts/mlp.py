"""SwiGLU feed-forward: down( silu(gate(h)) * up(h) ).

g = Wg h, u = Wu h, a = g / (1 + exp(-g)) * u, out = Wd a
(crates/airun-core/src/runtime.rs:688-747, crates/airun-cuda/kernels/ops.cu:191-200).
Gate and up run as one product over a matrix whose rows alternate between
blocks of ``group`` gate rows and ``group`` up rows, so a kernel that holds a
tile of the result has both factors of each output at hand.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from ..weights.loader import WeightSpec
from .base import FeedForward, NormedActivations, register_part
from .linear import linear, linear_into_residual

INTERLEAVE = 16


class SwiGLU(FeedForward):
    device_driven = True

    fuses_norms = True        # takes NormedActivations as input and a ResidualSink for its output

    def __init__(self, prefix: str, hidden_size: int, intermediate_size: int,
                 dtype: torch.dtype = torch.bfloat16, device=None, names: Optional[Dict[str, str]] = None):
        self.prefix, self.H, self.I = prefix, int(hidden_size), int(intermediate_size)
        self.dtype, self.device = dtype, device
        self.group = INTERLEAVE if self.I % INTERLEAVE == 0 else self.I
        n = dict(gate="gate_proj.weight", up="up_proj.weight", down="down_proj.weight")
        n.update(names or {})
        self.names = {k: f"{prefix}.{v}" for k, v in n.items()}
        self.w_gu = self.w_down = None

    def weight_specs(self) -> List[WeightSpec]:
        nm = self.names
        return [WeightSpec(nm["gate"], (self.I, self.H)), WeightSpec(nm["up"], (self.I, self.H)),
                WeightSpec(nm["down"], (self.H, self.I))]

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        nm, g = self.names, self.group
        gate, up = tensors.pop(nm["gate"]), tensors.pop(nm["up"])
        nb = self.I // g
        self.w_gu = torch.stack([gate.view(nb, g, self.H), up.view(nb, g, self.H)], dim=1) \
            .reshape(2 * self.I, self.H).contiguous()
        self.w_down = tensors.pop(nm["down"])

    def forward(self, ctx, h, sink=None):
        normed = h if isinstance(h, NormedActivations) else None
        hx = normed.h if normed is not None else h
        T, ws = hx.shape[0], ctx.ws
        act = ws.alloc((T, self.I), self.dtype)
        done = False
        if hx.dtype == torch.bfloat16:
            from ..kernels import fast
            done = fast.linear_swiglu_bf16(ctx, hx, self.w_gu, act, self.group, normed=normed)
        if not done:
            gu = ws.alloc((T, 2 * self.I), torch.float32)
            linear(ctx, h, self.w_gu, gu)
            ops.swiglu(gu, act, self.group)
        fused = linear_into_residual(ctx, act, self.w_down, sink)
        if fused is not None:
            return fused
        delta = ws.alloc((T, self.H), torch.float32)
        linear(ctx, act, self.w_down, delta)
        return delta


register_part("feed_forward", "swiglu", SwiGLU)


class ClampedGLU(FeedForward):
    """Gated unit whose factors are clamped: g = min(Wg h, limit), u = clamp(Wu h, -limit, limit),
    a = g * sigmoid(slope * g) * (u + 1), out = Wd a.  ``slope`` 1.702 makes g * sigmoid(slope * g) the usual
    sigmoid approximation of GELU.  Gate and up run as one product over rows interleaved in blocks of
    ``group`` (as in SwiGLU above).  It has the split form (parts/base.py): ``forward_core`` writes ``a`` into
    a buffer the arrangement gives it and ``w_out`` is Wd."""
    device_driven = True

    def __init__(self, prefix: str, hidden_size: int, intermediate_size: int, limit: float, slope: float = 1.702,
                 dtype: torch.dtype = torch.bfloat16, device=None, names: Optional[Dict[str, str]] = None):
        self.prefix, self.H, self.I = prefix, int(hidden_size), int(intermediate_size)
        self.limit, self.slope = float(limit), float(slope)
        if not self.limit > 0:
            raise ValueError(f"the clamp limit must be positive, found {limit}")
        self.dtype, self.device = dtype, device
        self.group = INTERLEAVE if self.I % INTERLEAVE == 0 else self.I
        n = dict(gate="gate", up="up", down="down")
        n.update(names or {})
        self.names = {k: f"{prefix}.{v}" for k, v in n.items()}
        self.w_gu = self.w_out = None
        self.core_width = self.I

    def weight_specs(self) -> List[WeightSpec]:
        nm = self.names
        return [WeightSpec(nm["gate"], (self.I, self.H)), WeightSpec(nm["up"], (self.I, self.H)),
                WeightSpec(nm["down"], (self.H, self.I))]

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        nm, g = self.names, self.group
        gate, up = tensors.pop(nm["gate"]), tensors.pop(nm["up"])
        nb = self.I // g
        self.w_gu = torch.stack([gate.view(nb, g, self.H), up.view(nb, g, self.H)], dim=1) \
            .reshape(2 * self.I, self.H).contiguous()
        self.w_out = tensors.pop(nm["down"])

    def adopt_w_out(self, view: torch.Tensor) -> None:
        self.w_out = view

    def forward_core(self, ctx, h: torch.Tensor, act: torch.Tensor) -> None:
        T = h.shape[0]
        if h.dtype == torch.bfloat16:
            from ..kernels import fast
            if fast.linear_glu_clamped_bf16(ctx, h, self.w_gu, act, self.group, self.limit, self.slope):
                return
        gu = ctx.ws.alloc((T, 2 * self.I), torch.float32)
        linear(ctx, h, self.w_gu, gu)
        ops.glu_clamped(gu, act, self.group, self.limit, self.slope)

    def forward(self, ctx, h, sink=None):
        T = h.shape[0]
        act = ctx.ws.alloc((T, self.I), self.dtype)
        self.forward_core(ctx, h, act)
        delta = ctx.ws.alloc((T, self.H), torch.float32)
        linear(ctx, act, self.w_out, delta)
        return delta


register_part("feed_forward", "clamped_glu", ClampedGLU)


class ActMLP(FeedForward):
    """A feed-forward without a gate: out = Wd f(Wu h), f one of ``ops.ACTIVATIONS`` (``relu2``: the square of
    relu; ``silu``; ``gelu_tanh``; ``relu``).  It has the split form (parts/base.py): ``forward_core`` writes f(Wu h)
    into a buffer the arrangement gives it and ``w_out`` is Wd."""
    device_driven = True

    def __init__(self, prefix: str, hidden_size: int, intermediate_size: int, activation: str = "relu2",
                 dtype: torch.dtype = torch.bfloat16, device=None, names: Optional[Dict[str, str]] = None):
        self.prefix, self.H, self.I = prefix, int(hidden_size), int(intermediate_size)
        if activation not in ops.ACTIVATIONS:
            raise ValueError(f"activation {activation!r} is not one of {sorted(ops.ACTIVATIONS)}")
        self.activation, self.mode = activation, ops.ACTIVATIONS[activation]
        self.dtype, self.device = dtype, device
        n = dict(up="up", down="down")
        n.update(names or {})
        self.names = {k: f"{prefix}.{v}" for k, v in n.items()}
        self.w_up = self.w_out = None
        self.core_width = self.I

    def weight_specs(self) -> List[WeightSpec]:
        nm = self.names
        return [WeightSpec(nm["up"], (self.I, self.H)), WeightSpec(nm["down"], (self.H, self.I))]

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.w_up, self.w_out = tensors.pop(self.names["up"]), tensors.pop(self.names["down"])

    def adopt_w_out(self, view: torch.Tensor) -> None:
        self.w_out = view

    def forward_core(self, ctx, h: torch.Tensor, act: torch.Tensor) -> None:
        T = h.shape[0]
        if h.dtype == torch.bfloat16:
            from ..kernels import fast
            if fast.linear_act_bf16(ctx, h, self.w_up, act, self.mode):
                return
        u = ctx.ws.alloc((T, self.I), torch.float32)
        linear(ctx, h, self.w_up, u)
        ops.act(u, act, self.mode)

    def forward(self, ctx, h, sink=None):
        T = h.shape[0]
        act = ctx.ws.alloc((T, self.I), self.dtype)
        self.forward_core(ctx, h, act)
        delta = ctx.ws.alloc((T, self.H), torch.float32)
        linear(ctx, act, self.w_out, delta)
        return delta


register_part("feed_forward", "act_mlp", ActMLP)
