"""Softmax attention over paged keys and values with the options several designs combine differently.

With h the mixer's input, H query heads and G key/value heads (query head h reads KV head h / (H / G)), key rows of
``key_dim`` and value rows of ``value_dim`` elements:

    q = Wq h,  k = Wk h,  v = Wv h                      with ``bias``: + bq, bk, bv, and + bo on the output
    ``qk_norm="weight"``   q, k <- x / rms(x) * w       per head, one weight vector for all heads, before the rotation
    the position encoding (a registered ``position`` part) on q and k
    ``qk_norm="unit"``     q, k <- x / rms(x)           per head, no weight, after the rotation
    ``temp_every`` > 0     q <- q * (1 + temp_coef * ln(floor((p + 1) / temp_every) + 1))
    s_ij = scale * q_i . k_j + rel[bucket(i - j), h]     with ``distance_rows`` B > 0: a learnt table of B rows;
                                                         bucket(n) = n for n < B/2, else
                                                         min(B - 1, B/2 + floor(ln(n / (B/2)) / ln(far / (B/2)) * (B - B/2)))
    p_ij = exp(s_ij) / (sum_j' exp(s_ij') + exp(sink_h)) with ``sink``: one more term of the denominator per head, which
                                                         has no key and no value
    o_i = sum_j p_ij v_j over j <= i (and i - j < window when ``window`` > 0),   out = out_scale * Wo concat_heads(o)

The bucket of every distance is worked out once, in double precision on the host, into a table per head that the kernels
index by min(i - j, far).  The three input projections run as one product.  The part has the split form
(parts/base.py): ``forward_core`` leaves the heads' results, times ``out_scale``, in a buffer, and can be handed the
columns of a product that an arrangement has run over several parts' stacked input matrices (``proj``).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from ..kernels import ops
from ..weights.loader import WeightSpec
from .base import Mixer, PagedKVSpec, make_part, register_part
from .linear import linear


def distance_buckets(rows: int, far: int) -> List[int]:
    """bucket(n) for n = 0 .. max(far, rows // 2): every distance beyond reads the last entry."""
    half = rows // 2
    out = []
    for n in range(max(far, half) + 1):
        if n < half or half == 0:
            out.append(min(n, rows - 1))
        else:
            out.append(min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half)))))
    return out


class SoftmaxAttention(Mixer):
    device_driven = True

    def __init__(self, prefix: str, hidden_size: int, num_heads: int, num_kv_heads: int, key_dim: int, value_dim: int,
                 scale: float, norm_eps: float = 1e-6, bias: bool = False, qk_norm: str = "none",
                 position: str = "none", position_args: Optional[dict] = None, temp_coef: float = 0.0, temp_every: int = 0,
                 distance_rows: int = 0, distance_far: int = 0, sink: bool = False, window: int = 0, out_scale: float = 1.0,
                 dtype: torch.dtype = torch.bfloat16, device=None, names: Optional[Dict[str, str]] = None):
        self.prefix, self.H = prefix, int(hidden_size)
        self.nh, self.nkv, self.D, self.Dv = int(num_heads), int(num_kv_heads), int(key_dim), int(value_dim)
        if min(self.nh, self.nkv, self.D, self.Dv) <= 0:
            raise ValueError("head counts and sizes must be positive")
        if self.nh % self.nkv:
            raise ValueError(f"heads ({num_heads}) must be a multiple of kv_heads ({num_kv_heads})")
        if self.D > 256 or self.Dv > 256:
            raise ValueError("head sizes above 256 are beyond the attention kernels")
        if qk_norm not in ("none", "weight", "unit"):
            raise ValueError("qk_norm is 'none', 'weight' (before the rotation) or 'unit' (after it, without a weight)")
        self.scale, self.eps, self.qk_norm, self.bias = float(scale), float(norm_eps), qk_norm, bool(bias)
        self.temp_coef, self.temp_every = float(temp_coef), int(temp_every or 0)
        self.distance_rows, self.distance_far = int(distance_rows or 0), int(distance_far or 0)
        if self.distance_rows and self.distance_far <= self.distance_rows // 2:
            raise ValueError("the farthest distance of the table must lie beyond half its rows")
        self.has_sink, self.window, self.out_scale = bool(sink), int(window or 0), float(out_scale)
        self.dtype, self.device = dtype, device
        self.pos = make_part("position", position, prefix=prefix, dtype=dtype, device=device, **(position_args or {}))
        kind, rdim, _ = self.pos.fused()
        if rdim > self.D:
            raise ValueError(f"{rdim} rotated dimensions do not fit a head of {self.D}")
        n = dict(q="q", k="k", v="v", o="o", q_bias="q.b", k_bias="k.b", v_bias="v.b", o_bias="o.b", q_norm="q.norm",
                 k_norm="k.norm", rel="rel", sink="sink")
        n.update(names or {})
        self.names = {k: f"{prefix}.{v}" for k, v in n.items()}
        self.w_in = self.w_out = self.in_bias = self.output_bias = self.q_norm_w = self.k_norm_w = None
        self.table = self.sink = None
        self.core_width = self.nh * self.Dv

    # ---- weights ----
    def weight_specs(self) -> List[WeightSpec]:
        nm, H, qw, kw, vw = self.names, self.H, self.nh * self.D, self.nkv * self.D, self.nkv * self.Dv
        specs = [WeightSpec(nm["q"], (qw, H)), WeightSpec(nm["k"], (kw, H)), WeightSpec(nm["v"], (vw, H)),
                 WeightSpec(nm["o"], (H, self.nh * self.Dv))]
        if self.bias:
            specs += [WeightSpec(nm["q_bias"], (qw,), storage="float32"), WeightSpec(nm["k_bias"], (kw,), storage="float32"),
                      WeightSpec(nm["v_bias"], (vw,), storage="float32"), WeightSpec(nm["o_bias"], (H,), storage="float32")]
        if self.qk_norm == "weight":
            specs += [WeightSpec(nm["q_norm"], (self.D,), storage="float32", init="norm"),
                      WeightSpec(nm["k_norm"], (self.D,), storage="float32", init="norm")]
        if self.distance_rows:
            specs.append(WeightSpec(nm["rel"], (self.distance_rows, self.nh), storage="float32"))
        if self.has_sink:
            specs.append(WeightSpec(nm["sink"], (self.nh,), storage="float32"))
        return specs + self.pos.weight_specs()

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        nm = self.names
        self.w_in = torch.cat([tensors.pop(nm["q"]), tensors.pop(nm["k"]), tensors.pop(nm["v"])], dim=0).contiguous()
        self.w_out = tensors.pop(nm["o"])
        if self.bias:
            self.in_bias = torch.cat([tensors[nm["q_bias"]], tensors[nm["k_bias"]], tensors[nm["v_bias"]]]).contiguous()
            self.output_bias = tensors[nm["o_bias"]]
        if self.qk_norm == "weight":
            self.q_norm_w, self.k_norm_w = tensors[nm["q_norm"]], tensors[nm["k_norm"]]
        if self.distance_rows:
            rel = tensors[nm["rel"]]
            idx = torch.tensor(distance_buckets(self.distance_rows, self.distance_far), dtype=torch.long, device=rel.device)
            self.table = rel[idx].t().contiguous()                 # [heads, distances]
        if self.has_sink:
            self.sink = tensors[nm["sink"]]
        self.pos.load_weights(tensors)

    def adopt_w_out(self, view: torch.Tensor) -> None:
        self.w_out = view

    # ---- cache ----
    def cache_spec(self):
        return PagedKVSpec(self.nkv, self.D, self.window, value_dim=self.Dv if self.Dv != self.D else 0)

    # ---- compute ----
    def forward_core(self, ctx, h, act: torch.Tensor, cache, proj: Optional[torch.Tensor] = None) -> None:
        """Writes out_scale * the heads' results into ``act`` ([T, heads * value_dim], rows may be strided).  ``proj``:
        float32 [T, rows of w_in], the product of h with this part's stacked input matrix when the caller has run it."""
        T, ws = act.shape[0], ctx.ws
        if cache.shared:
            raise RuntimeError(f"{self.prefix}: this attention writes a cache of its own")
        if proj is None:
            proj = ws.alloc((T, self.w_in.shape[0]), torch.float32)
            linear(ctx, h, self.w_in, proj)
        q = ws.alloc((T, self.nh * self.D), self.dtype)
        kind, rdim, inv_freq = self.pos.fused()
        ops.qkv_prepare(proj, self.in_bias, self.q_norm_w, self.k_norm_w, self.qk_norm == "unit", self.eps, kind, rdim, inv_freq,
                        self.temp_coef, self.temp_every, q, cache, ctx, self.nh, self.nkv, self.D, self.Dv, store=True,
                        rope_positions=self.pos.rotation_positions(ctx))
        self.attend(ctx, q, act, cache)

    def attend(self, ctx, q: torch.Tensor, out: torch.Tensor, cache) -> None:
        if q.dtype == torch.bfloat16:
            from ..kernels import fast
            if fast.softmax_attention_bf16(ctx, q, out, cache, self):
                return
        ops.softmax_attention(q, out, cache, ctx, self.nh, self.nkv, self.D, self.Dv, self.scale, self.table, self.sink,
                              self.window, self.out_scale)

    def forward(self, ctx, h, cache, sink=None, add_bias: bool = True):
        """The residual delta.  With ``add_bias`` False the output bias (``output_bias``, times nothing) is left to the
        caller, which adds it on its next pass over the residual."""
        T = h.shape[0]
        act = ctx.ws.alloc((T, self.core_width), self.dtype)
        self.forward_core(ctx, h, act, cache)
        delta = ctx.ws.alloc((T, self.H), torch.float32)
        linear(ctx, act, self.w_out, delta)
        if add_bias and self.output_bias is not None:
            ops.add_rows(delta, vec=self.output_bias)
        return delta


register_part("mixer", "softmax_attention", SoftmaxAttention)
