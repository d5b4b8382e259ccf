"""Routed experts: a feed-forward made of many small gated units of which every token uses a few.

    z = Wr h  (float32; + a bias per expert with ``router_bias``),   s = sigmoid(z)  (or softmax(z) with ``scores="softmax"``;
    softmax scores divided by the sum over the chosen ones, ``renormalize``, are the softmax over the chosen logits alone)
    the ``top`` experts with the largest s are chosen (equal scores: the lower id); the kernel orders them by z,
    which orders them as s does and still tells apart two large logits whose float32 scores both round to 1
    weight_e = s_e, divided by the sum over the chosen ones when ``renormalize``
    out = sum_e expert_e(weight_e * h)          (``weight_on="input"``: the weight scales what the expert reads)
    out = sum_e weight_e * expert_e(h)          (``weight_on="output"``)
    expert_e(x) = Wdown_e ( silu(Wgate_e x) * (Wup_e x) )

Options other designs use: experts without a gate, expert_e(x) = Wdown_e f(Wup_e x) (``expert="act"`` with an
``activation`` of ops.ACTIVATIONS); routing by softmax scores with a correction and groups (``routing="grouped"``):
the choice is by s + correction (a learnt number per router output, tensor ``correction``) among the outputs of the
``keep_groups`` best of ``groups`` equal runs of neighbouring outputs (a run's score is its largest s + correction),
the weights are the chosen s over their sum (+ 1e-20) times ``weight_scale``; and ``identity_experts``: the router's
last outputs stand for experts without matrices that return their input (they take part in the softmax, the groups and
the choice like the others).

Everything is decided on the device: a step's rows are sorted by expert into segments of one buffer and every
expert's matrices meet only their own segment (csrc/moe.cu, the grouped product of csrc/gemm_simt.cu), so the part
launches the same kernels for every batch and is replayed from CUDA graphs like the dense parts.  A token's result
depends on its own row alone.  Tensors: ``<prefix>.router`` and ``<prefix>.e<i>.{gate,up,down}``.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from ..weights.loader import WeightSpec
from .base import FeedForward, register_part
from .linear import linear
from .mlp import INTERLEAVE


class RoutedExperts(FeedForward):
    device_driven = True

    def __init__(self, prefix: str, hidden_size: int, intermediate_size: int, num_experts: int, top: int,
                 scores: str = "sigmoid", renormalize: bool = False, weight_on: str = "input", router_bias: bool = False,
                 expert: str = "swiglu", activation: str = "gelu_erf", routing: str = "top", choice_bias: bool = False,
                 groups: int = 1, keep_groups: int = 1, identity_experts: int = 0, weight_scale: float = 1.0,
                 dtype: torch.dtype = torch.bfloat16, device=None, names: Optional[Dict[str, str]] = None):
        self.prefix, self.H, self.I = prefix, int(hidden_size), int(intermediate_size)
        self.E, self.top = int(num_experts), int(top)
        if not (1 <= self.E <= 1024 and 1 <= self.top <= self.E + int(identity_experts)):
            raise ValueError(f"1 to 1024 experts and 1 to all of them a token, found {num_experts} and {top}")
        if scores not in ("sigmoid", "softmax") or weight_on not in ("input", "output"):
            raise ValueError("scores is 'sigmoid' or 'softmax', weight_on is 'input' or 'output'")
        self.softmax, self.renorm, self.on_input = scores == "softmax", bool(renormalize), weight_on == "input"
        self.dtype, self.device = dtype, device
        self.group = INTERLEAVE if self.I % INTERLEAVE == 0 else self.I
        self.router_bias = bool(router_bias)
        if expert not in ("swiglu", "act") or routing not in ("top", "grouped"):
            raise ValueError("expert is 'swiglu' or 'act', routing is 'top' or 'grouped'")
        if expert == "act" and activation not in ops.ACTIVATIONS:
            raise ValueError(f"activation must be one of {sorted(ops.ACTIVATIONS)}")
        self.gated, self.act_mode = expert == "swiglu", ops.ACTIVATIONS.get(activation, 0)
        self.grouped_routing = routing == "grouped"
        self.choice_bias, self.groups, self.keep = bool(choice_bias), int(groups), int(keep_groups)
        self.identity, self.weight_scale = int(identity_experts), float(weight_scale)
        self.n_out = self.E + self.identity
        if not self.grouped_routing and (self.choice_bias or self.groups != 1 or self.identity or self.weight_scale != 1.0):
            raise ValueError("a correction, groups, identity experts and a weight scale belong to routing='grouped'")
        if self.grouped_routing:
            if not self.softmax or self.on_input or router_bias:
                raise ValueError("grouped routing weighs the experts' outputs by softmax scores and has no bias on the logits")
            if self.identity < 0 or self.groups < 1 or self.n_out % self.groups or not (1 <= self.keep <= self.groups) \
                    or self.top > self.n_out // self.groups * self.keep:
                raise ValueError(f"{self.groups} groups must divide the router's {self.n_out} outputs, and the {self.keep} kept "
                                 f"ones must hold {self.top} of them")
        n = dict(router="router", router_bias="router.b", expert="e{e}", gate="gate", up="up", down="down", correction="correction")
        n.update(names or {})
        self.n = n
        self.w_router = self.b_router = self.w_gu = self.w_up = self.w_down = self.counts = self.correction = None
        self.extra_rows = 0          # rows an arrangement appended to the router's product

    def _name(self, e: int, which: str) -> str:
        return f"{self.prefix}.{self.n['expert'].format(e=e)}.{self.n[which]}"

    def weight_specs(self) -> List[WeightSpec]:
        specs = [WeightSpec(f"{self.prefix}.{self.n['router']}", (self.n_out, self.H))]
        if self.router_bias:
            specs.append(WeightSpec(f"{self.prefix}.{self.n['router_bias']}", (self.E,), storage="float32"))
        if self.choice_bias:
            specs.append(WeightSpec(f"{self.prefix}.{self.n['correction']}", (self.n_out,), storage="float32"))
        for e in range(self.E):
            if self.gated:
                specs.append(WeightSpec(self._name(e, "gate"), (self.I, self.H)))
            specs += [WeightSpec(self._name(e, "up"), (self.I, self.H)), WeightSpec(self._name(e, "down"), (self.H, self.I))]
        return specs

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        g, nb = self.group, self.I // self.group
        self.w_router = tensors.pop(f"{self.prefix}.{self.n['router']}")
        if self.router_bias:
            self.b_router = tensors[f"{self.prefix}.{self.n['router_bias']}"]
        if self.choice_bias:
            self.correction = tensors[f"{self.prefix}.{self.n['correction']}"]
        gus, downs = [], []
        if not self.gated:
            self.w_up = torch.stack([tensors.pop(self._name(e, "up")) for e in range(self.E)], dim=0).contiguous()      # [E, I, H]
            self.w_down = torch.stack([tensors.pop(self._name(e, "down")) for e in range(self.E)], dim=0).contiguous()  # [E, H, I]
            self.counts = torch.zeros(self.E, dtype=torch.int32, device=self.w_router.device)
            return
        for e in range(self.E):
            gate, up = tensors.pop(self._name(e, "gate")), tensors.pop(self._name(e, "up"))
            # gate and up rows alternate in blocks of ``group``, as in the dense gated units
            gus.append(torch.stack([gate.view(nb, g, self.H), up.view(nb, g, self.H)], dim=1).reshape(2 * self.I, self.H))
            downs.append(tensors.pop(self._name(e, "down")))
        self.w_gu = torch.stack(gus, dim=0).contiguous()          # [E, 2I, H]
        self.w_down = torch.stack(downs, dim=0).contiguous()      # [E, H, I]
        self.counts = torch.zeros(self.E, dtype=torch.int32, device=self.w_router.device)

    def append_input_rows(self, w: torch.Tensor) -> None:
        """``w`` [rows, hidden] joins the router's product below the router; ``forward(..., with_extra=True)`` then
        returns its float32 columns beside the result."""
        self.w_router = torch.cat([self.w_router, w], dim=0).contiguous()
        self.extra_rows = int(w.shape[0])

    def forward(self, ctx, h: torch.Tensor, sink=None, with_extra: bool = False):
        T, ws, top = h.shape[0], ctx.ws, self.top
        M = T * top
        ids, rank, row_of = (ws.alloc((T, top), torch.int32) for _ in range(3))
        wts = ws.alloc((T, top), torch.float32)
        seg = ws.alloc((self.E + 1,), torch.int32)
        self.counts.zero_()
        logits = ws.alloc((T, self.n_out + self.extra_rows), torch.float32)
        linear(ctx, h, self.w_router, logits)
        if self.grouped_routing:
            ops.moe_route_grouped(logits[:, :self.n_out], self.E, top, self.groups, self.keep, self.weight_scale, self.correction,
                                  ctx.req_of_token, ids, wts, rank, self.counts, seg)
        else:
            ops.moe_route(logits[:, :self.E], top, self.softmax, self.renorm, ctx.req_of_token, ids, wts, rank, self.counts, seg,
                          bias=self.b_router)
        xs = ws.alloc((M, self.H), self.dtype)
        ops.moe_scatter(h, top, ids, wts, rank, seg, self.on_input, xs, row_of, num_real=self.E)
        act = ws.alloc((M, self.I), self.dtype)
        fused = False
        if xs.dtype == torch.bfloat16:
            from ..kernels import fast
            if self.gated:
                fused = fast.grouped_linear_bf16(ctx, xs, self.w_gu, act, seg, swiglu_group=self.group)
            else:
                fused = fast.grouped_linear_bf16(ctx, xs, self.w_up, act, seg, act=self.act_mode)
        if not fused and self.gated:
            gu = ws.alloc((M, 2 * self.I), torch.float32)
            grouped_linear(ctx, xs, self.w_gu, gu, seg)
            ops.swiglu(gu, act, self.group)
        elif not fused:
            up = ws.alloc((M, self.I), torch.float32)
            grouped_linear(ctx, xs, self.w_up, up, seg)
            ops.act(up, act, self.act_mode)
        ys = ws.alloc((M, self.H), torch.float32)
        grouped_linear(ctx, act, self.w_down, ys, seg)
        delta = ws.alloc((T, self.H), torch.float32)
        ops.moe_combine(ys, top, ids, wts, row_of, not self.on_input, delta, passthrough=h if self.identity else None)
        if with_extra:
            return delta, (logits[:, self.n_out:] if self.extra_rows else None)
        return delta


def grouped_linear(ctx, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, seg: torch.Tensor) -> None:
    """Rows seg[e] .. seg[e+1]-1 of x times w[e]^T: x [M, K], w [E, N, K], out [M, N], seg int32 [E+1] on the device.
    bfloat16 operands go to the tensor-core kernel where it takes the sizes, everything else to the plain one."""
    if x.dtype == torch.bfloat16:
        from ..kernels import fast
        if fast.grouped_linear_bf16(ctx, x, w, out, seg):
            return
    ops.gemm_simt_grouped(x, w, out, seg)


register_part("feed_forward", "routed_experts", RoutedExperts)
