"""Configuration of the Gamanex decoder, read from its config.json keys.

A Gamanex model is a stack of layers in which the mixer and the feed-forward read the residual stream side by side,
each through a root-mean-square norm of its own, and each result is scaled per channel and gated by a sigmoid of the
sub-layer's input before both are added (parts/block.py: ``gated_parallel``).  The mixer is an attention without
softmax and without rotation (parts/sigmoid_attention.py); the feed-forward is W_down relu(W_up h)^2, a mixture of
SwiGLU experts, or absent.

``architecture``        "Gamanex"
``vocab``, ``width``    vocabulary and residual width
``norm.eps``            eps of every root mean square
``logit_scale``         factor on the logits (absent: 1)
``layers``              one entry per layer: ``type`` ("attention"), ``mixer`` and ``mlp`` ({"kind": "dense", "ff"},
                        {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top"}}, or null for none)

Mixer keys: ``heads``, ``kv_heads``, ``dim`` (query/key size of a head), ``vdim`` (value size), ``scale``, optionally
``q_temp`` {``coef``, ``every``} (a query temperature that grows with the position) and ``kv_from``: the layer whose
cached keys and values this layer attends over instead of caching its own.

Tensor names: ``embed``, ``head``, ``final.norm`` and per layer ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.ls1|ls2``,
``l<i>.rg1|rg2`` with ``.b``, ``l<i>.mix.{q,k,v,o,q.norm,k.norm,r1,r2,pb}``, ``l<i>.mlp.{up,down}`` or
``l<i>.mlp.router`` (with ``.b``) and ``l<i>.mlp.e<j>.{gate,up,down}``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Tuple

from .base import ConfigError, LayerCall, LayerSpec, ModelConfig

MIXERS = ("attention",)


@dataclass(frozen=True)
class GamanexConfig(ModelConfig):
    vocab_size: int
    hidden_size: int
    norm_eps: float
    logit_scale: float
    layers: Tuple[Dict[str, Any], ...]
    architecture: str = "Gamanex"
    tie_word_embeddings: bool = False
    max_position_embeddings: int = 1 << 20       # the cache alone bounds a request

    # ---- reading ----
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "GamanexConfig":
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

        V = integer(d, "vocab", "vocab")
        H = integer(d, "width", "width")
        eps = number(d.get("norm") or {}, "eps", "norm.eps", positive=True)
        logit_scale = number(d, "logit_scale", "logit_scale", 1.0)
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
            mixer: Dict[str, Any] = dict(heads=integer(m, "heads", f"{w}.mixer.heads"), dim=integer(m, "dim", f"{w}.mixer.dim"))
            mixer["kv_heads"] = integer(m, "kv_heads", f"{w}.mixer.kv_heads", mixer["heads"])
            if mixer["heads"] % mixer["kv_heads"]:
                problems.append(f"{w}.mixer.heads ({mixer['heads']}) must be a multiple of kv_heads ({mixer['kv_heads']})")
            mixer["vdim"] = integer(m, "vdim", f"{w}.mixer.vdim", mixer["dim"])
            mixer["scale"] = number(m, "scale", f"{w}.mixer.scale", mixer["dim"] ** -0.5)
            if m.get("q_temp") is not None:
                t = m["q_temp"]
                mixer["q_temp"] = dict(coef=number(t, "coef", f"{w}.mixer.q_temp.coef"),
                                       every=integer(t, "every", f"{w}.mixer.q_temp.every"))
            if m.get("kv_from") is not None:
                mixer["kv_from"] = integer(m, "kv_from", f"{w}.mixer.kv_from", least=0)
            mlp = l.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
                    problems.append(f"{w}.mlp must be null or an object of kind 'dense' or 'moe'")
                    mlp = None
                elif mlp["kind"] == "dense":
                    mlp = dict(kind="dense", ff=integer(mlp, "ff", f"{w}.mlp.ff"))
                else:
                    router = mlp.get("router") or {}
                    mlp = dict(kind="moe", expert=dict(ff=integer(mlp.get("expert") or {}, "ff", f"{w}.mlp.expert.ff")),
                               router=dict(experts=integer(router, "experts", f"{w}.mlp.router.experts"),
                                           top=integer(router, "top", f"{w}.mlp.router.top")))
                    if mlp["router"]["top"] > mlp["router"]["experts"]:
                        problems.append(f"{w}.mlp.router.top exceeds the number of experts")
            layers.append(dict(type=l["type"], mixer=mixer, mlp=mlp))
        for i, l in enumerate(layers):
            j = l["mixer"].get("kv_from")
            if j is None:
                continue
            src = layers[j] if j < i else None
            if src is None or src["type"] != "attention" or "kv_from" in src["mixer"]:
                problems.append(f"layers[{i}].mixer.kv_from must name an earlier attention layer with a cache of its own")
            elif any(src["mixer"].get(k) != l["mixer"].get(k) for k in ("kv_heads", "dim", "vdim")):
                problems.append(f"layers[{i}] reads the cache of layer {j}: their kv_heads, dim and vdim must be equal")
        if problems:
            raise ConfigError("config.json cannot be used: " + "; ".join(problems))
        return cls(vocab_size=V, hidden_size=H, norm_eps=eps, logit_scale=logit_scale, layers=tuple(layers),
                   architecture=str(d.get("architecture", "Gamanex")))

    def to_dict(self) -> Dict[str, Any]:
        def copy(v):
            return {k: copy(x) for k, x in v.items()} if isinstance(v, dict) else v
        return {"architecture": self.architecture,
                "layers": [dict(type=l["type"], mixer=copy(l["mixer"]), mlp=copy(l["mlp"])) for l in self.layers],
                "logit_scale": self.logit_scale, "norm": {"eps": self.norm_eps},
                "vocab": self.vocab_size, "width": self.hidden_size}

    # ---- what the model is made of ----
    def tensor_names(self) -> Dict[str, str]:
        return dict(embed="embed", layer="l{i}", mixer="mix", ffn="mlp", norm1="norm1", norm2="norm2",
                    final_norm="final.norm", head="head")

    def final_norm(self) -> Tuple[str, dict]:
        return "rmsnorm", dict(size=self.hidden_size, eps=self.norm_eps, weight_name="")

    def head(self) -> Tuple[str, dict]:
        return "lm_head", dict(scale=self.logit_scale)

    def layer_specs(self) -> List[LayerSpec]:
        H, specs = self.hidden_size, []
        for i, l in enumerate(self.layers):
            m = l["mixer"]
            temp = m.get("q_temp") or {}
            args = dict(hidden_size=H, num_heads=m["heads"], num_kv_heads=m["kv_heads"], key_dim=m["dim"], value_dim=m["vdim"],
                        scale=m["scale"], norm_eps=self.norm_eps, qk_norm="projection", temp_coef=temp.get("coef", 0.0),
                        temp_every=temp.get("every", 0), distance_bias=True, head_bias=True, owns_cache="kv_from" not in m)
            mlp = l["mlp"]
            if not mlp:
                ffn, fargs = "", {}
            elif mlp["kind"] == "dense":
                ffn, fargs = "act_mlp", dict(hidden_size=H, intermediate_size=mlp["ff"], activation="relu2")
            else:
                ffn, fargs = "routed_experts", dict(hidden_size=H, intermediate_size=mlp["expert"]["ff"],
                                                    num_experts=mlp["router"]["experts"], top=mlp["router"]["top"],
                                                    scores="softmax", renormalize=True, weight_on="output", router_bias=True)
            specs.append(LayerSpec(mixer="sigmoid_attention", mixer_args=args, feed_forward=ffn, ffn_args=fargs, norm="rmsnorm",
                                   norm_args=dict(size=H, eps=self.norm_eps, weight_name=""), arrangement="gated_parallel",
                                   arrangement_args=dict(prefix=f"l{i}", hidden_size=H, layer_scale=True, gated=True)))
        return specs

    def execution_order(self) -> List[LayerCall]:
        return [LayerCall(i, cache_from=l["mixer"].get("kv_from")) for i, l in enumerate(self.layers)]

    def ignorable_tensors(self) -> List[str]:
        """Tensors a model file may hold although nothing reads them: the second norm, scale and gate of a layer that
        has no feed-forward."""
        return [f"l{i}.{n}" for i, l in enumerate(self.layers) if not l["mlp"] for n in ("norm2", "ls2", "rg2", "rg2.b")]

    def summary(self) -> str:
        moe = sum(1 for l in self.layers if l["mlp"] and l["mlp"]["kind"] == "moe")
        shared = sum(1 for l in self.layers if "kv_from" in l["mixer"])
        return (f"{self.architecture}: {len(self.layers)} gated parallel layers of attention without softmax ({shared} on an "
                f"earlier layer's keys and values), {moe} with routed experts, width {self.hidden_size}, vocab {self.vocab_size}")
