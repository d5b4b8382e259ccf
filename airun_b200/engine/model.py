"""A decoder put together from parts, layer by layer, from a configuration.

The model is: token embedding, a list of layers (each an arrangement of norm,
mixer, feed-forward chosen by the configuration's ``layer_specs()``), an
execution order (a list of :class:`LayerCall`, which may name a layer twice or
let an entry read an earlier entry's cache), a final norm and an output head.
Tensor names come from the configuration's ``tensor_names()``.  The reference
assembles the same pieces per layer (crates/airun-core/src/model.rs:612-628,
crates/airun-core/src/runtime.rs:3482-3602) and keeps the output norm fused with
the last residual add (runtime.rs:3745-3746).
"""
from __future__ import annotations

import os
import sys
from typing import Dict, List, Optional, Tuple

import torch

from ..config.base import LayerCall, ModelConfig
from ..parts.base import CastActivations, StreamWrite, make_part, part_factory
from ..parts import embedding as _embedding_parts      # noqa: F401  (registers the embedding and head parts)
from ..weights.loader import (DictSource, TensorSource, WeightSpec, load_tensors, random_tensors)

# AIRUN_TRACE_LAYERS=1 prints the residual stream's rms and mean after every block (the reference's
# switch of the same name, crates/airun-core/src/runtime.rs:5265-5302).  Off by default.
TRACE_LAYERS = os.environ.get("AIRUN_TRACE_LAYERS", "") not in ("", "0")

DEFAULT_NAMES = dict(embed="model.embed_tokens.weight", layer="model.layers.{i}", mixer="self_attn",
                     ffn="mlp", norm1="input_layernorm", norm2="post_attention_layernorm",
                     final_norm="model.norm", head="lm_head.weight")


class DecoderModel:
    def __init__(self, config: ModelConfig, dtype: torch.dtype, device):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"the engine computes in float32 or bfloat16, not {dtype}")
        self.config, self.dtype, self.device = config, dtype, torch.device(device)
        names = dict(DEFAULT_NAMES)
        names.update(getattr(config, "tensor_names", lambda: {})())
        self.names = names
        V, H = config.vocab_size, config.hidden_size
        self.V, self.H = V, H
        emb_name, emb_args = config.embedding() if hasattr(config, "embedding") else ("token_embedding", {})
        self.embedding = make_part("embedding", emb_name, prefix=names["embed"], vocab_size=V, hidden_size=H,
                                   dtype=dtype, device=self.device, **emb_args)
        self.layers = []
        for i, spec in enumerate(config.layer_specs()):
            p = names["layer"].format(i=i if getattr(spec, "index", None) is None else spec.index)
            common = dict(dtype=dtype, device=self.device)
            norm1 = make_part("norm", spec.norm, prefix=f"{p}.{names['norm1']}", **spec.norm_args, **common)
            # an arrangement with one norm (``num_norms = 1``) gets no second one; a layer without a
            # feed-forward names none (``feed_forward`` empty)
            factory = part_factory("arrangement", spec.arrangement)
            two_norms = getattr(factory, "num_norms", 2) >= 2 and (
                bool(spec.feed_forward) or not getattr(factory, "norm2_belongs_to_ffn", False))
            norm2 = make_part("norm", spec.norm, prefix=f"{p}.{names['norm2']}", **spec.norm_args, **common) \
                if two_norms else None
            mixer = make_part("mixer", spec.mixer, prefix=f"{p}.{names['mixer']}", **spec.mixer_args, **common)
            ffn = make_part("feed_forward", spec.feed_forward, prefix=f"{p}.{names['ffn']}", **spec.ffn_args, **common) \
                if spec.feed_forward else None
            self.layers.append(make_part("arrangement", spec.arrangement, norm1=norm1, mixer=mixer,
                                         norm2=norm2, ffn=ffn, dtype=dtype, **getattr(spec, "arrangement_args", {})))
        # a residual of several streams: every layer's arrangement must read and write all of them
        self.multi_stream = bool(self.layers) and all(getattr(l, "multi_stream", False) for l in self.layers)
        if not self.multi_stream and any(getattr(l, "multi_stream", False) for l in self.layers):
            raise ValueError("arrangements over several residual streams cannot be mixed with arrangements over one")
        self.streams = int(getattr(config, "residual_streams", lambda: 1)()) if self.multi_stream else 1
        self._stream_ones = torch.ones(self.streams, dtype=torch.float32, device=self.device)      # the read that sums the streams
        self.order: List[LayerCall] = list(config.execution_order())
        for c in self.order:
            if not (0 <= c.layer < len(self.layers)):
                raise ValueError(f"the execution order names layer {c.layer}, the model has {len(self.layers)}")
        # the table whose rows entries of the order add to the residual stream before they run (float32 [rows, H])
        table = config.order_table() if hasattr(config, "order_table") else None
        self.order_table_name, self.order_table_rows = table if table else (None, 0)
        self.order_table: Optional[torch.Tensor] = None
        for c in self.order:
            if getattr(c, "add_row", None) is not None and not (0 <= c.add_row < self.order_table_rows):
                raise ValueError(f"the execution order adds row {c.add_row} of a table of {self.order_table_rows} rows")
        self.layer_hook = None      # debugging and tests: called as hook(entry, residual [T, H]) after every entry
        fn_name, fn_args = config.final_norm() if hasattr(config, "final_norm") else \
            ("rmsnorm", dict(size=H, eps=config.rms_norm_eps))
        self.final_norm = make_part("norm", fn_name, prefix=names["final_norm"], dtype=dtype,
                                    device=self.device, **fn_args)
        tied = bool(getattr(config, "tie_word_embeddings", False))
        head_name, head_args = config.head() if hasattr(config, "head") else ("lm_head", {})
        self.head = make_part("head", head_name, prefix=names["head"], vocab_size=V, hidden_size=H,
                              tied_to=self.embedding if tied else None, dtype=dtype, device=self.device, **head_args)
        self.tied = tied

    # ---- weights ----
    def parts(self):
        return [self.embedding] + self.layers + [self.final_norm, self.head]

    def weight_specs(self) -> List[WeightSpec]:
        specs = [s for p in self.parts() for s in p.weight_specs()]
        if self.order_table_name:
            specs.append(WeightSpec(self.order_table_name, (self.order_table_rows, self.H), storage="float32"))
        return specs

    def ignorable_tensors(self) -> List[str]:
        # a tied model's file may still carry the head (it is the same matrix); a configuration may name more
        extra = list(getattr(self.config, "ignorable_tensors", lambda: [])())
        return ([self.names["head"]] if self.tied else []) + extra

    def load(self, source: TensorSource) -> None:
        tensors = load_tensors(self.weight_specs(), source, self.dtype, self.device, self.ignorable_tensors())
        for p in self.parts():
            p.load_weights(tensors)
        if self.order_table_name:
            self.order_table = tensors[self.order_table_name]
        del tensors
        if self.device.type == "cuda":
            self.pack_weights()

    ARENA_ALIGN = 256

    def pack_weights(self) -> None:
        """Moves every tensor the parts hold (weights as the parts keep them: stacked, interleaved, tables)
        into ONE allocation, each at a 256-byte boundary, and gives the memory they came from back.  The
        reference keeps a layer's weights in one arena with 256-byte aligned sub-allocations for the same
        reasons: one allocation instead of hundreds, none of the allocator's rounding per tensor, and
        addresses that suit vector and bulk loads (crates/airun-core/src/model.rs:1332-1393).  Tensors that
        share memory (a tied head and the table; the q rows of the stacked q/k/v matrix) still do afterwards.
        Parts are found by walking the attributes of the model's parts, so a part needs nothing for it."""
        slots = []                                           # (holder, key, tensor): holder[key] or holder.key
        seen = set()

        def walk(obj):
            if id(obj) in seen:
                return
            seen.add(id(obj))
            items = vars(obj).items() if hasattr(obj, "__dict__") else ()
            for key, val in list(items):
                if isinstance(val, torch.Tensor):
                    if val.device == self.device:
                        slots.append((obj, key, val))
                elif isinstance(val, (list, tuple)):
                    if isinstance(val, list):
                        for i, v in enumerate(val):
                            if isinstance(v, torch.Tensor) and v.device == self.device:
                                slots.append((val, i, v))
                            elif hasattr(v, "weight_specs"):
                                walk(v)
                    else:
                        for v in val:
                            if hasattr(v, "weight_specs"):
                                walk(v)
                elif hasattr(val, "weight_specs"):
                    walk(val)

        for p in self.parts():
            walk(p)
        if self.order_table is not None:
            slots.append((self, "order_table", self.order_table))
        if not slots:
            return
        storages = {}                                        # storage address -> (bytes, offset in the arena)
        total = 0
        for _, _, t in slots:
            st = t.untyped_storage()
            if st.data_ptr() not in storages:
                storages[st.data_ptr()] = (st, total)
                total += (st.nbytes() + self.ARENA_ALIGN - 1) // self.ARENA_ALIGN * self.ARENA_ALIGN
        arena = torch.empty(total + self.ARENA_ALIGN, dtype=torch.uint8, device=self.device)
        base = (-arena.data_ptr()) % self.ARENA_ALIGN        # torch aligns to 512 bytes already; be sure of it
        moved = {}
        for ptr, (st, off) in storages.items():
            n = st.nbytes()
            dst = arena[base + off: base + off + n]
            dst.copy_(torch.empty(0, dtype=torch.uint8, device=self.device).set_(st, 0, (n,), (1,)))
            moved[ptr] = dst
        for holder, key, t in slots:
            dst = moved[t.untyped_storage().data_ptr()]
            esz = t.element_size()
            view = dst.view(t.dtype) if dst.numel() % esz == 0 else dst[: dst.numel() // esz * esz].view(t.dtype)
            new = torch.as_strided(view, t.shape, t.stride(), view.storage_offset() + t.storage_offset())
            if isinstance(holder, list):
                holder[key] = new
            else:
                setattr(holder, key, new)
        self.weight_arena = arena
        del storages, moved, slots
        torch.cuda.empty_cache()

    def load_random(self, seed: int) -> None:
        """Seeded random weights made on the model's device, through the same loading path."""
        tensors = random_tensors(self.weight_specs(), seed, self.device,
                                 torch.bfloat16)
        self.load(DictSource(tensors))

    def device_driven(self) -> bool:
        """True if every layer reads the batch's layout from the device arrays only, so that a step
        of a given padded size always launches the same kernels (and can be replayed from a graph)."""
        return all(getattr(l, "device_driven", lambda: False)() for l in self.layers) \
            and getattr(self.final_norm, "device_driven", False)

    def graph_safe(self) -> bool:
        """False if a part has said that its forward must not be captured into a CUDA graph (it
        decides on the host what to launch from values it reads back from the device)."""
        return all(getattr(l, "graph_safe", lambda: True)() for l in self.layers)

    # ---- cache needs ----
    def cache_specs(self) -> Tuple[List[object], List[Optional[int]]]:
        return ([self.layers[c.layer].cache_spec() for c in self.order],
                [c.cache_from for c in self.order])

    # ---- one pass over the given tokens ----
    def forward(self, ctx, want_rows: Optional[torch.Tensor], n_want: int) -> Optional[torch.Tensor]:
        T = ctx.num_tokens
        ctx.ws_main.reset()
        x = ctx.ws_main.alloc((T, self.H), torch.float32)
        self.embedding.forward(ctx, ctx.token_ids[:T], x)
        if self.multi_stream:
            return self._forward_streams(ctx, x, want_rows, n_want)
        delta = None
        trace = TRACE_LAYERS and not torch.cuda.is_current_stream_capturing()
        for ci, call in enumerate(self.order):
            ctx.ws = ctx.ws_pair[ci % 2]
            ctx.ws.reset()
            nxt = self.layers[self.order[ci + 1].layer] if ci + 1 < len(self.order) else None
            next_norm = nxt.norm1 if (nxt is not None and getattr(nxt, "accepts_normed", lambda: False)()) else None
            layer, extra = self.layers[call.layer], {}
            if getattr(call, "add_row", None) is not None:
                vec = self.order_table[call.add_row]
                if getattr(layer, "accepts_add_vec", False):
                    extra["add_vec"] = vec
                else:                                   # x += what is pending + the row, by a kernel of its own
                    from ..kernels import ops
                    ops.add_rows(x[:T], delta=delta if isinstance(delta, torch.Tensor) else None, vec=vec)
                    delta = None if isinstance(delta, torch.Tensor) else delta
            if next_norm is not None:
                extra["next_norm"] = next_norm
            delta = layer.forward(ctx, x, delta, ctx.caches[ci], **extra)
            if self.layer_hook is not None and not torch.cuda.is_current_stream_capturing():
                if isinstance(delta, torch.Tensor):
                    self.layer_hook(ci, x[:T] + delta[:T])
                elif delta is None or isinstance(delta, CastActivations):       # nothing pending: x is the stream
                    self.layer_hook(ci, x[:T])
            if trace:           # synchronises after every block: a debugging aid, as the reference's AIRUN_TRACE_LAYERS
                r = x[:ctx.num_tokens] if not isinstance(delta, torch.Tensor) else (x[:ctx.num_tokens] + delta[:ctx.num_tokens])
                print(f"[airun_b200] entry {ci} layer {call.layer}: rms {float(r.pow(2).mean().sqrt()):.6f} "
                      f"mean {float(r.mean()):+.6f}", file=sys.stderr)
        if n_want == 0:
            return None
        ctx.ws = ctx.ws_pair[len(self.order) % 2]
        ctx.ws.reset()
        hsel = ctx.ws.alloc((n_want, self.H), self.dtype)
        if isinstance(delta, CastActivations):
            delta = None
        self.final_norm.forward(ctx, x, hsel, delta=delta, rows=want_rows[:n_want])
        logits = ctx.ws_main.alloc((n_want, self.V), torch.float32)
        self.head.forward(ctx, hsel, logits)
        return logits


    def _forward_streams(self, ctx, x: torch.Tensor, want_rows: Optional[torch.Tensor], n_want: int) -> Optional[torch.Tensor]:
        """The pass over the layers with a residual of ``streams`` copies, [T, S, H]: every copy starts as the embedding,
        each block leaves its last write pending for the next pass over the streams (parts/block.py:
        HyperConnectionBlock), and the last pass writes it and sums the streams into x for the final norm."""
        from ..kernels import ops
        T, S = ctx.num_tokens, self.streams
        xs = ctx.ws_main.alloc((T, S, self.H), torch.float32)
        ops.stream_fill(x, xs)
        pending = None
        for ci, call in enumerate(self.order):
            ctx.ws = ctx.ws_pair[ci % 2]
            ctx.ws.reset()
            if getattr(call, "add_row", None) is not None:
                raise ValueError("rows of an order table are not added to a residual of several streams")
            pending = self.layers[call.layer].forward(ctx, xs, pending, ctx.caches[ci])
            if self.layer_hook is not None and not torch.cuda.is_current_stream_capturing():
                now = xs[:T]
                if isinstance(pending, StreamWrite):
                    y = pending.y[:T] + (pending.y_bias if pending.y_bias is not None else 0.0)
                    now = torch.einsum("st,jsw->jtw", pending.carry, now) + pending.mult * pending.write[None, :, None] * y[:, None, :]
                self.layer_hook(ci, now.sum(dim=1))
        if n_want == 0:
            return None
        p = pending
        ops.stream_step(xs, y=p.y if p else None, carry=p.carry if p else None, write=p.write if p else None,
                        mult=p.mult if p else 1.0, y_bias=p.y_bias if p else None, read=self._stream_ones, out=x,
                        req_of_token=ctx.req_of_token)
        ctx.ws = ctx.ws_pair[len(self.order) % 2]
        ctx.ws.reset()
        hsel = ctx.ws.alloc((n_want, self.H), self.dtype)
        self.final_norm.forward(ctx, x, hsel, rows=want_rows[:n_want])
        logits = ctx.ws_main.alloc((n_want, self.V), torch.float32)
        self.head.forward(ctx, hsel, logits)
        return logits


def build_decoder(config: ModelConfig, dtype: torch.dtype, device) -> DecoderModel:
    return DecoderModel(config, dtype, device)
