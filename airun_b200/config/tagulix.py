"""Configuration of the Tagulix decoder, read from its config.json keys.

A Tagulix model carries its residual as several streams (parts/block.py: ``hyper_connections``); every sub-layer reads
a weighted sum of them through a root-mean-square norm and writes its result, times ``residual_mult``, back into all
of them.  A layer's mixer is either a windowed softmax attention with biases, a partial rotation of neighbouring
dimensions and an unweighted q/k norm after it ("attention"), or two mixers side by side ("parallel"): a causal softmax
attention with a weighted q/k norm, a query temperature, a learnt bias per distance bucket and a sink, beside a linear
attention with one fixed decay per head, gated and normed over all heads.  The feed-forward is a mixture of ungated
GELU experts routed by softmax scores with a correction, groups and experts that return their input, or absent.  A
layer may run with the tensors of another layer and a cache of its own.

``architecture``        "Tagulix"
``vocab``, ``width``    vocabulary and residual width
``norm.eps``            eps of every root mean square
``residual_mult``       factor on every sub-layer's result (absent: 1)
``streams``             copies of the residual (absent: one plain residual without learnt connections)
``layers``              one entry per layer: ``type`` ("attention" | "parallel"), ``mixer``, ``mlp`` (null for none) and
                        optionally ``weights_of``: the layer whose tensors this layer runs with

"attention" mixer keys: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``mask.size`` (the window; absent: none),
``rot`` {``dims``, ``base``} (absent: no rotation).
"parallel" mixer keys: ``left`` {``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``bias_max``, ``q_temp`` {``coef``,
``every``}}, ``right`` {``heads``, ``dim``, ``vdim``, ``decay`` (a number per head)}, ``left_scale``, ``right_scale``.
``mlp``: {``kind``: "moe", ``expert``: {``ff``}, ``router``: {``experts``, ``top``, ``identity``, ``scale``, ``groups``:
{``count``, ``keep``}}}.

Tensor names: ``embed``, ``head``, ``final.norm`` and per layer ``l<i>.norm1|norm2``, ``l<i>.hc1|hc2.{in,mix,out}``,
``l<i>.mix.{q,k,v,o}`` with ``.b`` each, or ``l<i>.mix.left.{q,k,v,o,q.norm,k.norm,rel,sink}`` and
``l<i>.mix.right.{q,k,v,g,o,norm}``; ``l<i>.mlp.router``, ``l<i>.mlp.correction`` and ``l<i>.mlp.e<j>.{up,down}``.  The
number of rows of ``rel`` (the distance buckets) is read from the tensor's shape.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Any, Dict, List, Optional, Tuple

from .base import ConfigError, LayerCall, LayerSpec, ModelConfig

MIXERS = ("attention", "parallel")
DEFAULT_DISTANCE_ROWS = 32


@dataclass(frozen=True)
class TagulixConfig(ModelConfig):
    vocab_size: int
    hidden_size: int
    norm_eps: float
    residual_mult: float
    streams: Optional[int]                       # None: one residual without learnt connections
    layers: Tuple[Dict[str, Any], ...]
    architecture: str = "Tagulix"
    tie_word_embeddings: bool = False
    max_position_embeddings: int = 1 << 20       # the cache alone bounds a request

    # ---- reading ----
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "TagulixConfig":
        problems: List[str] = []

        def integer(where, key: str, what: str, default=None, least: int = 1) -> int:
            v = where.get(key, default) if isinstance(where, dict) else default
            if isinstance(v, bool) or not isinstance(v, int):
                problems.append(f"{what} must be an integer, found {v!r}")
                return least
            if v < least:
                problems.append(f"{what} must be at least {least}, found {v}")
                return least
            return v

        def number(where, key: str, what: str, default=None, positive: bool = False) -> float:
            v = where.get(key, default) if isinstance(where, dict) else default
            if isinstance(v, bool) or not isinstance(v, (int, float)):
                problems.append(f"{what} must be a number, found {v!r}")
                return 1.0
            if positive and not v > 0:
                problems.append(f"{what} must be positive, found {v}")
                return 1.0
            return float(v)

        def attention(m, w: str, windowed: bool) -> Dict[str, Any]:
            a: Dict[str, Any] = dict(heads=integer(m, "heads", f"{w}.heads"), dim=integer(m, "dim", f"{w}.dim"))
            a["kv_heads"] = integer(m, "kv_heads", f"{w}.kv_heads", a["heads"])
            if a["heads"] % a["kv_heads"]:
                problems.append(f"{w}.heads ({a['heads']}) must be a multiple of kv_heads ({a['kv_heads']})")
            a["vdim"] = integer(m, "vdim", f"{w}.vdim", a["dim"])
            a["scale"] = number(m, "scale", f"{w}.scale", a["dim"] ** -0.5)
            if windowed:
                if m.get("mask") is not None:
                    a["mask"] = dict(size=integer(m["mask"], "size", f"{w}.mask.size"))
                if m.get("rot") is not None:
                    r = dict(dims=integer(m["rot"], "dims", f"{w}.rot.dims", least=2),
                             base=number(m["rot"], "base", f"{w}.rot.base", 10000.0, positive=True))
                    if r["dims"] % 2 or r["dims"] > a["dim"]:
                        problems.append(f"{w}.rot.dims must be even and at most dim ({a['dim']}), found {r['dims']}")
                    a["rot"] = r
            else:
                a["bias_max"] = integer(m, "bias_max", f"{w}.bias_max", least=2)
                if m.get("q_temp") is not None:
                    a["q_temp"] = dict(coef=number(m["q_temp"], "coef", f"{w}.q_temp.coef"),
                                       every=integer(m["q_temp"], "every", f"{w}.q_temp.every"))
            return a

        V = integer(d, "vocab", "vocab")
        H = integer(d, "width", "width")
        eps = number(d.get("norm") or {}, "eps", "norm.eps", positive=True)
        mult = number(d, "residual_mult", "residual_mult", 1.0)
        streams = None if d.get("streams") is None else integer(d, "streams", "streams")
        if streams is not None and streams > 8:
            problems.append(f"streams must be at most 8, found {streams}")
        raw = d.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json cannot be used: 'layers' must be a non-empty list")
        layers: List[Dict[str, Any]] = []
        for i, l in enumerate(raw):
            w = f"layers[{i}]"
            if not isinstance(l, dict) or l.get("type") not in MIXERS or not isinstance(l.get("mixer"), dict):
                problems.append(f"{w} needs a 'type' out of {list(MIXERS)} and a 'mixer' object")
                layers.append(dict(type=None, mixer={}, mlp=None))
                continue
            m = l["mixer"]
            if l["type"] == "attention":
                mixer = attention(m, f"{w}.mixer", True)
            else:
                if not isinstance(m.get("left"), dict) or not isinstance(m.get("right"), dict):
                    problems.append(f"{w}.mixer needs 'left' and 'right' objects")
                    layers.append(dict(type=None, mixer={}, mlp=None))
                    continue
                r = m["right"]
                right = dict(heads=integer(r, "heads", f"{w}.mixer.right.heads"), dim=integer(r, "dim", f"{w}.mixer.right.dim"))
                right["vdim"] = integer(r, "vdim", f"{w}.mixer.right.vdim", right["dim"])
                decay = r.get("decay")
                if not isinstance(decay, list) or len(decay) != right["heads"] or \
                        not all(isinstance(x, (int, float)) and not isinstance(x, bool) for x in decay):
                    problems.append(f"{w}.mixer.right.decay must be a list of one number per head")
                    decay = [1.0] * right["heads"]
                right["decay"] = [float(x) for x in decay]
                mixer = dict(left=attention(m["left"], f"{w}.mixer.left", False), right=right,
                             left_scale=number(m, "left_scale", f"{w}.mixer.left_scale", 1.0),
                             right_scale=number(m, "right_scale", f"{w}.mixer.right_scale", 1.0))
            mlp = l.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "moe":
                    problems.append(f"{w}.mlp must be null or an object of kind 'moe'")
                    mlp = None
                else:
                    r = mlp.get("router") or {}
                    g = r.get("groups") or {}
                    router = dict(experts=integer(r, "experts", f"{w}.mlp.router.experts"), top=integer(r, "top", f"{w}.mlp.router.top"),
                                  identity=integer(r, "identity", f"{w}.mlp.router.identity", 0, least=0),
                                  scale=number(r, "scale", f"{w}.mlp.router.scale", 1.0),
                                  groups=dict(count=integer(g, "count", f"{w}.mlp.router.groups.count", 1),
                                              keep=integer(g, "keep", f"{w}.mlp.router.groups.keep", 1)))
                    n_out, gc, gk = router["experts"] + router["identity"], router["groups"]["count"], router["groups"]["keep"]
                    if n_out % gc or gk > gc:
                        problems.append(f"{w}.mlp.router: {gc} groups must divide the {n_out} router outputs, and keep ({gk}) "
                                        f"cannot exceed them")
                    elif router["top"] > n_out // gc * gk:
                        problems.append(f"{w}.mlp.router.top exceeds the outputs of the kept groups")
                    mlp = dict(kind="moe", expert=dict(ff=integer(mlp.get("expert") or {}, "ff", f"{w}.mlp.expert.ff")), router=router)
            entry = dict(type=l["type"], mixer=mixer, mlp=mlp)
            if l.get("weights_of") is not None:
                entry["weights_of"] = integer(l, "weights_of", f"{w}.weights_of", least=0)
            layers.append(entry)
        for i, l in enumerate(layers):
            j = l.get("weights_of")
            if j is None:
                continue
            if not (0 <= j < len(layers)) or j == i or "weights_of" in layers[j]:
                problems.append(f"layers[{i}].weights_of must name another layer with tensors of its own")
            elif any(layers[j].get(k) != l.get(k) for k in ("type", "mixer", "mlp")):
                problems.append(f"layers[{i}] runs with the tensors of layer {j}: the rest of their entries must be equal")
        if problems:
            raise ConfigError("config.json cannot be used: " + "; ".join(problems))
        return cls(vocab_size=V, hidden_size=H, norm_eps=eps, residual_mult=mult, streams=streams, layers=tuple(layers),
                   architecture=str(d.get("architecture", "Tagulix")))

    def to_dict(self) -> Dict[str, Any]:
        def copy(v):
            if isinstance(v, dict):
                return {k: copy(x) for k, x in v.items() if k != "distance_rows"}
            return list(v) if isinstance(v, list) else v
        out = {"architecture": self.architecture, "layers": [copy(dict(l)) for l in self.layers],
               "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult, "vocab": self.vocab_size,
               "width": self.hidden_size}
        if self.streams is not None:
            out["streams"] = self.streams
        return out

    def with_tensor_shapes(self, shapes: Dict[str, Tuple[int, ...]]) -> "TagulixConfig":
        """The number of distance buckets of every "parallel" layer is the number of rows of its ``rel`` tensor."""
        layers = []
        for i, l in enumerate(self.layers):
            shape = shapes.get(f"l{l.get('weights_of', i)}.mix.left.rel")
            if l["type"] == "parallel" and shape:
                l = dict(l, mixer=dict(l["mixer"], left=dict(l["mixer"]["left"], distance_rows=int(shape[0]))))
            layers.append(l)
        return replace(self, layers=tuple(layers))

    # ---- what the model is made of ----
    def tensor_names(self) -> Dict[str, str]:
        return dict(embed="embed", layer="l{i}", mixer="mix", ffn="mlp", norm1="norm1", norm2="norm2",
                    final_norm="final.norm", head="head")

    def final_norm(self) -> Tuple[str, dict]:
        return "rmsnorm", dict(size=self.hidden_size, eps=self.norm_eps, weight_name="")

    def residual_streams(self) -> int:
        return self.streams or 1

    def owners(self) -> List[int]:
        """The layers that have tensors of their own, in order."""
        return [i for i, l in enumerate(self.layers) if "weights_of" not in l]

    def layer_specs(self) -> List[LayerSpec]:
        H, specs = self.hidden_size, []
        for i in self.owners():
            l = self.layers[i]
            m = l["mixer"]
            if l["type"] == "attention":
                rot = m.get("rot")
                mixer = "softmax_attention"
                args = dict(hidden_size=H, num_heads=m["heads"], num_kv_heads=m["kv_heads"], key_dim=m["dim"], value_dim=m["vdim"],
                            scale=m["scale"], norm_eps=self.norm_eps, bias=True, qk_norm="unit",
                            position="rotary_interleaved" if rot else "none",
                            position_args=dict(rotary_dim=rot["dims"], theta=rot["base"]) if rot else {},
                            window=(m.get("mask") or {}).get("size", 0))
            else:
                a, r = m["left"], m["right"]
                temp = a.get("q_temp") or {}
                mixer = "side_by_side"
                args = dict(hidden_size=H, left_scale=m["left_scale"], right_scale=m["right_scale"],
                            left="softmax_attention",
                            left_args=dict(num_heads=a["heads"], num_kv_heads=a["kv_heads"], key_dim=a["dim"], value_dim=a["vdim"],
                                           scale=a["scale"], norm_eps=self.norm_eps, qk_norm="weight",
                                           temp_coef=temp.get("coef", 0.0), temp_every=temp.get("every", 0),
                                           # without a file to read the table's rows from: as many as bias_max allows
                                           distance_rows=a.get("distance_rows", max(2, min(DEFAULT_DISTANCE_ROWS, 2 * (a["bias_max"] - 1)))),
                                           distance_far=a["bias_max"], sink=True),
                            right="decay_linear_attention",
                            right_args=dict(num_heads=r["heads"], key_dim=r["dim"], value_dim=r["vdim"], decay=r["decay"],
                                            norm_eps=self.norm_eps))
            mlp = l["mlp"]
            if not mlp:
                ffn, fargs = "", {}
            else:
                r = mlp["router"]
                ffn = "routed_experts"
                fargs = dict(hidden_size=H, intermediate_size=mlp["expert"]["ff"], num_experts=r["experts"], top=r["top"],
                             scores="softmax", weight_on="output", expert="act", activation="gelu_erf", routing="grouped",
                             choice_bias=True, groups=r["groups"]["count"], keep_groups=r["groups"]["keep"],
                             identity_experts=r["identity"], weight_scale=r["scale"])
            specs.append(LayerSpec(mixer=mixer, mixer_args=args, feed_forward=ffn, ffn_args=fargs, norm="rmsnorm",
                                   norm_args=dict(size=H, eps=self.norm_eps, weight_name=""), arrangement="hyper_connections",
                                   arrangement_args=dict(prefix=f"l{i}", streams=self.streams or 1, residual_mult=self.residual_mult,
                                                         learned=self.streams is not None),
                                   index=i))
        return specs

    def execution_order(self) -> List[LayerCall]:
        place = {i: n for n, i in enumerate(self.owners())}
        return [LayerCall(place[l.get("weights_of", i)]) for i, l in enumerate(self.layers)]

    def ignorable_tensors(self) -> List[str]:
        """Tensors a model file may hold although nothing reads them: the second norm and connections of a layer that
        has no feed-forward."""
        return [f"l{i}.{n}" for i in self.owners() if not self.layers[i]["mlp"]
                for n in ("norm2", "hc2.in", "hc2.mix", "hc2.out")]

    def summary(self) -> str:
        kinds = [l["type"] for l in self.layers]
        shared = sum(1 for l in self.layers if "weights_of" in l)
        return (f"{self.architecture}: {len(self.layers)} layers ({kinds.count('attention')} windowed attention, "
                f"{kinds.count('parallel')} attention beside decayed linear attention; {shared} with another layer's tensors), "
                f"{self.streams or 1} residual streams, width {self.hidden_size}, vocab {self.vocab_size}")
