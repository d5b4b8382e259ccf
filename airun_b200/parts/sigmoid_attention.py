"""Attention without softmax over paged keys and values.

Every visible key weighs sigmoid(score) and the weights are not normalised over the keys:

    q = Wq h,  k = Wk h,  v = Wv h                                   (no biases, no rotation)
    q <- q / rms(q) * wq,  k <- k / rms(k) * wk                      with ``qk_norm`` "projection": ONE root mean square
                                                                     over the whole projection, all heads at once
    q <- q * (1 + coef * ln(floor((p + 1) / every) + 1))             with ``temp_every`` > 0: a temperature that grows
                                                                     with the query's position p
    s_ij = scale * q_i . k_j - a_h * ln(1 + b_h * (i - j)) + c_h     a, b (``distance_bias``) and c (``head_bias``) are
                                                                     numbers per query head
    o_i = sum over j <= i (and i - j < window) of sigmoid(s_ij) v_j
    out = Wo concat_heads(o)

Query head h reads KV head h / (heads / kv_heads); key rows have ``key_dim`` elements and value rows ``value_dim``
(``PagedKVSpec.value_dim``).  The three input projections run as one product; the keys are cached after their norm.
An entry of the execution order that reads another entry's cache computes q only, with norm, temperature and head
numbers of its own.  The part has the split form (parts/base.py), and ``extra_in`` lets an arrangement append rows to
the input product (a gate that reads the same input) and get their columns back (``forward(..., with_extra=True)``).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from ..weights.loader import WeightSpec
from .base import Mixer, PagedKVSpec, register_part
from .linear import linear


class SigmoidAttention(Mixer):
    device_driven = True

    def __init__(self, prefix: str, hidden_size: int, num_heads: int, num_kv_heads: int, key_dim: int, value_dim: int,
                 scale: float, norm_eps: float, qk_norm: str = "projection", temp_coef: float = 0.0, temp_every: int = 0,
                 distance_bias: bool = True, head_bias: bool = True, window: int = 0, owns_cache: bool = True,
                 dtype: torch.dtype = torch.bfloat16, device=None, names: Optional[Dict[str, str]] = None):
        self.prefix, self.H = prefix, int(hidden_size)
        self.nh, self.nkv, self.D, self.Dv = int(num_heads), int(num_kv_heads), int(key_dim), int(value_dim)
        if min(self.nh, self.nkv, self.D, self.Dv) <= 0:
            raise ValueError("head counts and sizes must be positive")
        if self.nh % self.nkv:
            raise ValueError(f"heads ({num_heads}) must be a multiple of kv_heads ({num_kv_heads})")
        if self.D > 256 or self.Dv > 256:
            raise ValueError("head sizes above 256 are beyond the attention kernels")
        if qk_norm not in ("projection", "none"):
            raise ValueError("qk_norm is 'projection' (one norm over all heads) or 'none'")
        self.scale, self.eps, self.qk_norm = float(scale), float(norm_eps), qk_norm == "projection"
        self.temp_coef, self.temp_every = float(temp_coef), int(temp_every or 0)
        self.distance_bias, self.head_bias, self.window = bool(distance_bias), bool(head_bias), int(window or 0)
        self.owns_cache = bool(owns_cache)
        self.dtype, self.device = dtype, device
        n = dict(q="q", k="k", v="v", o="o", q_norm="q.norm", k_norm="k.norm", dist_a="r1", dist_b="r2", head_c="pb")
        n.update(names or {})
        self.names = {k: f"{prefix}.{v}" for k, v in n.items()}
        self.w_in = self.w_q = self.w_out = self.q_norm_w = self.k_norm_w = self.dist_a = self.dist_b = self.head_c = None
        self.core_width = self.nh * self.Dv
        self.extra_rows = 0          # rows an arrangement appended to the input product

    # ---- weights ----
    def weight_specs(self) -> List[WeightSpec]:
        nm, H, qw, kw, vw = self.names, self.H, self.nh * self.D, self.nkv * self.D, self.nkv * self.Dv
        specs = [WeightSpec(nm["q"], (qw, H)), WeightSpec(nm["o"], (H, self.nh * self.Dv))]
        if self.owns_cache:
            specs += [WeightSpec(nm["k"], (kw, H)), WeightSpec(nm["v"], (vw, H))]
        if self.qk_norm:
            specs.append(WeightSpec(nm["q_norm"], (qw,), storage="float32", init="norm"))
            if self.owns_cache:
                specs.append(WeightSpec(nm["k_norm"], (kw,), storage="float32", init="norm"))
        if self.distance_bias:
            specs += [WeightSpec(nm["dist_a"], (self.nh,), storage="float32", init="norm"),
                      WeightSpec(nm["dist_b"], (self.nh,), storage="float32", init="norm")]
        if self.head_bias:
            specs.append(WeightSpec(nm["head_c"], (self.nh,), storage="float32"))
        return specs

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        nm = self.names
        rows = [tensors.pop(nm["q"])]
        if self.owns_cache:
            rows += [tensors.pop(nm["k"]), tensors.pop(nm["v"])]
        self.w_in = torch.cat(rows, dim=0).contiguous() if len(rows) > 1 else rows[0]
        self.w_q = self.w_in[: self.nh * self.D]
        self.w_out = tensors.pop(nm["o"])
        if self.qk_norm:
            self.q_norm_w = tensors[nm["q_norm"]]
            self.k_norm_w = tensors[nm["k_norm"]] if self.owns_cache else None
        if self.distance_bias:
            self.dist_a, self.dist_b = tensors[nm["dist_a"]], tensors[nm["dist_b"]]
        if self.head_bias:
            self.head_c = tensors[nm["head_c"]]

    def adopt_w_out(self, view: torch.Tensor) -> None:
        self.w_out = view

    def append_input_rows(self, w: torch.Tensor) -> None:
        """``w`` [rows, hidden] joins the input product below q, k and v; ``forward_core`` then returns its columns."""
        self.w_in = torch.cat([self.w_in, w], dim=0).contiguous()
        self.w_q = self.w_in[: self.nh * self.D]
        self.extra_rows = int(w.shape[0])

    # ---- cache ----
    def cache_spec(self):
        return PagedKVSpec(self.nkv, self.D, self.window, value_dim=self.Dv if self.Dv != self.D else 0)

    # ---- compute ----
    def forward_core(self, ctx, h: torch.Tensor, act: torch.Tensor, cache):
        """Writes the heads' results into ``act``; returns the float32 columns of the appended rows (or None)."""
        T, ws = h.shape[0], ctx.ws
        owns = not cache.shared
        if owns != self.owns_cache:
            raise RuntimeError(f"{self.prefix}: the execution order and the part disagree on who owns the cache")
        qw = self.nh * self.D
        width = self.w_in.shape[0]
        proj = ws.alloc((T, width), torch.float32)
        linear(ctx, h, self.w_in, proj)
        q = ws.alloc((T, qw), self.dtype)
        ops.qk_rownorm_store(proj, self.q_norm_w, self.k_norm_w, self.eps, self.temp_coef, self.temp_every, q, cache, ctx,
                             qw, self.nkv, self.D, self.Dv, store=owns)
        self.attend(ctx, q, act, cache)
        return proj[:, width - self.extra_rows:] if self.extra_rows else None

    def attend(self, ctx, q: torch.Tensor, out: torch.Tensor, cache) -> None:
        if q.dtype == torch.bfloat16:
            from ..kernels import fast
            if fast.sigmoid_attention_bf16(ctx, q, out, cache, self):
                return
        ops.sigmoid_attention(q, out, cache, ctx, self.nh, self.nkv, self.D, self.Dv, self.scale, self.dist_a, self.dist_b,
                              self.head_c, self.window)

    def forward(self, ctx, h, cache, sink=None, with_extra: bool = False):
        T = h.shape[0]
        act = ctx.ws.alloc((T, self.core_width), self.dtype)
        extra = self.forward_core(ctx, h, act, cache)
        delta = ctx.ws.alloc((T, self.H), torch.float32)
        linear(ctx, act, self.w_out, delta)
        return (delta, extra) if with_extra else delta


register_part("mixer", "sigmoid_attention", SigmoidAttention)
