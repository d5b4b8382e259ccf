"""Two mixers side by side: both read the same input, and the result is a weighted sum of theirs,

    out = left_scale * left(h) + right_scale * right(h).

The halves are registered mixers with the split form (parts/base.py), named with their constructor arguments; their
tensors lie under ``<prefix>.<left_prefix>`` and ``<prefix>.<right_prefix>``.  Each half keeps a cache or state of its
own: ``cache_spec`` is the pair of theirs, and the cache the part is handed holds the two views (``cache.parts``).
The scales go to the halves (``out_scale``), which apply them in float32 where they form their activations, so the two
input products run as ONE product over the stacked input matrices and the two output products as ONE product over the
activations set side by side, [Wo_left | Wo_right]: the sum costs no kernel of its own.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..weights.loader import WeightSpec
from .base import Mixer, make_part, register_part
from .linear import linear


class SideBySideMixer(Mixer):
    def __init__(self, prefix: str, hidden_size: int, left: str, left_args: dict, right: str, right_args: dict,
                 left_scale: float = 1.0, right_scale: float = 1.0, left_prefix: str = "left", right_prefix: str = "right",
                 dtype: torch.dtype = torch.bfloat16, device=None):
        self.prefix, self.H, self.dtype, self.device = prefix, int(hidden_size), dtype, device
        self.halves = [make_part("mixer", name, prefix=f"{prefix}.{p}", hidden_size=hidden_size, out_scale=float(sc), dtype=dtype,
                                 device=device, **args)
                       for name, args, sc, p in ((left, left_args, left_scale, left_prefix), (right, right_args, right_scale, right_prefix))]
        for m in self.halves:
            if not all(hasattr(m, a) for a in ("forward_core", "adopt_w_out", "core_width")):
                raise ValueError(f"{type(m).__name__} has no split form: it cannot stand beside another mixer")
            if getattr(m, "bias", False):
                raise ValueError("a half with an output bias cannot share its output product")
        self.device_driven = all(getattr(m, "device_driven", False) for m in self.halves)
        self.graph_safe = all(getattr(m, "graph_safe", True) for m in self.halves)
        self.w_in: Optional[torch.Tensor] = None
        self.w_out: Optional[torch.Tensor] = None
        self.core_width = sum(m.core_width for m in self.halves)

    def weight_specs(self) -> List[WeightSpec]:
        return [s for m in self.halves for s in m.weight_specs()]

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        for m in self.halves:
            m.load_weights(tensors)
        self.w_out = torch.cat([m.w_out for m in self.halves], dim=1).contiguous()
        at = 0
        for m in self.halves:
            m.adopt_w_out(self.w_out[:, at:at + m.core_width])
            at += m.core_width
        if all(getattr(m, "w_in", None) is not None for m in self.halves):
            self.w_in = torch.cat([m.w_in for m in self.halves], dim=0).contiguous()
            at = 0
            for m in self.halves:
                rows = m.w_in.shape[0]
                m.w_in = self.w_in[at:at + rows]
                at += rows

    def adopt_w_out(self, view: torch.Tensor) -> None:
        self.w_out = view
        at = 0
        for m in self.halves:
            m.adopt_w_out(view[:, at:at + m.core_width])
            at += m.core_width

    def cache_spec(self):
        return tuple(m.cache_spec() for m in self.halves)

    def forward_core(self, ctx, h, act: torch.Tensor, cache) -> None:
        T = act.shape[0]
        caches = cache.parts
        projs = [None, None]
        if self.w_in is not None:
            proj = ctx.ws.alloc((T, self.w_in.shape[0]), torch.float32)
            linear(ctx, h, self.w_in, proj)
            at = 0
            for i, m in enumerate(self.halves):
                projs[i] = proj[:, at:at + m.w_in.shape[0]]
                at += m.w_in.shape[0]
        at = 0
        for m, c, pr in zip(self.halves, caches, projs):
            m.forward_core(ctx, h, act[:, at:at + m.core_width], c, **({"proj": pr} if pr is not None else {}))
            at += m.core_width

    def forward(self, ctx, h, cache, sink=None):
        T = h.shape[0]
        act = ctx.ws.alloc((T, self.core_width), self.dtype)
        self.forward_core(ctx, h, act, cache)
        delta = ctx.ws.alloc((T, self.H), torch.float32)
        linear(ctx, act, self.w_out, delta)
        return delta


register_part("mixer", "side_by_side", SideBySideMixer)
