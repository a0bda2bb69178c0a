"""A decoder model put together from parts: embedding, a schedule of layer runs, final norm, head.

The model knows no architecture: it is built from a ``ModelSpec`` and a dictionary of parameters.
The schedule is data: ``runs`` is a list of (layer, whose cache, writes it?) and may name a layer
twice or let a layer read the cache of another.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from ..config import ModelSpec
from ..ops import kernels
from ..ops.linear import Linear
from .registry import BLOCKS, LOGIT_TRANSFORMS, NORMS, BuildContext, build_part, sub_weights


@dataclass(frozen=True)
class LayerRun:
    layer: int          # which layer's parts and weights run
    cache_layer: int    # the layer whose pages / state this run uses
    writes_cache: bool


class DecoderModel:
    def __init__(self, spec: ModelSpec, params: Dict[str, torch.Tensor], compute_dtype: torch.dtype,
                 device: torch.device, max_position: Optional[int] = None, weight_tiles: bool = True):
        spec.validate()
        if compute_dtype not in (torch.float32, torch.bfloat16):
            raise ValueError("compute dtype must be float32 or bfloat16")
        self.spec = spec
        self.dtype = compute_dtype
        self.device = device
        self.hidden_size = spec.hidden_size
        self.vocab_size = spec.vocab_size
        self.max_position = min(spec.max_position, max_position) if max_position else spec.max_position
        build = BuildContext(device=device, compute_dtype=compute_dtype, max_position=self.max_position,
                             weight_tiles=weight_tiles)

        emb = params["embedding.weight"]
        if tuple(emb.shape) != (spec.vocab_size, spec.hidden_size):
            raise ValueError(f"embedding has shape {tuple(emb.shape)}, expected ({spec.vocab_size}, {spec.hidden_size})")
        self.embedding = emb.to(device=device, dtype=compute_dtype).contiguous()
        self.embedding_scale = spec.embedding_scale

        self.layers: List[object] = []
        for i, layer_spec in enumerate(spec.layers):
            if layer_spec.block not in BLOCKS:
                raise KeyError(f"unknown block arrangement '{layer_spec.block}'")
            self.layers.append(BLOCKS[layer_spec.block](layer_spec, sub_weights(params, f"layers.{i}."), build))
        self.runs = [LayerRun(e.layer, e.layer if e.cache_of is None else e.cache_of, e.writes_cache)
                     for e in spec.schedule]
        self.final_norm = build_part(NORMS, "norm", spec.final_norm, sub_weights(params, "final_norm."), build)
        if spec.tie_word_embeddings:
            self.head = Linear.over(self.embedding, tiles=weight_tiles)   # the table itself, not a second row-major copy
        else:
            self.head = Linear(params["head.weight"], compute_dtype, device, tiles=weight_tiles)
            if (self.head.out_features, self.head.in_features) != (spec.vocab_size, spec.hidden_size):
                raise ValueError("head.weight has the wrong shape")
        # what the architecture does to its logits after the head (``forward(ctx, logits)``, in place); Llama: nothing
        self.logit_transform = None
        if spec.logit_transform is not None:
            self.logit_transform = build_part(LOGIT_TRANSFORMS, "logit transform", spec.logit_transform,
                                              sub_weights(params, "logit_transform."), build)

    # ------------------------------------------------------------------ what the cache manager must provide
    def cache_needs(self):
        """{layer index: CacheNeed} for layers whose pages some run uses."""
        out = {}
        for run in self.runs:
            need = self.layers[run.cache_layer].mixer.cache_need()
            if need is not None:
                out[run.cache_layer] = need
        return out

    def state_needs(self):
        out = {}
        for run in self.runs:
            need = self.layers[run.cache_layer].mixer.state_need()
            if need is not None:
                out[run.cache_layer] = need
        return out

    def weight_bytes(self) -> int:
        """Bytes of distinct weight tensors on the device (a tied head counts once). Every device tensor
        that a part holds counts, except the attributes the part's class lists in ``not_weights``:
        tables computed from constants (cos/sin), and the tile-by-tile copies that few-token products
        read in place of the row-major matrices (a step reads one or the other)."""
        seen, total = set(), 0

        def visit(obj):
            nonlocal total
            if isinstance(obj, torch.Tensor):
                if obj.is_cuda and obj.data_ptr() not in seen:
                    seen.add(obj.data_ptr())
                    total += obj.numel() * obj.element_size()
            elif hasattr(obj, "__dict__"):
                skip = getattr(type(obj), "not_weights", ())
                for k, v in vars(obj).items():
                    if k not in skip:
                        visit(v)
            elif isinstance(obj, (list, tuple)):
                for v in obj:
                    visit(v)

        visit(self.embedding)
        visit(self.layers)
        visit(self.final_norm)
        visit(self.head)
        visit(self.logit_transform)
        return total

    # ------------------------------------------------------------------ the forward pass of one step
    def forward(self, ctx) -> Optional[torch.Tensor]:
        """Runs the tokens of ``ctx`` through every scheduled layer and returns 32-bit logits
        [wanted rows, vocab] (None when no row wants logits)."""
        T = ctx.n_tokens
        x = ctx.scratch("residual", (T, self.hidden_size), torch.float32)
        with ctx.range("embedding"):
            kernels.embed(self.embedding, ctx.tokens, x, self.embedding_scale, ctx.feedback)
        ctx.tap("embedding", -1, x)
        for run in self.runs:
            with ctx.range(f"layer {run.layer}"):
                self.layers[run.layer].forward(ctx, run, x)
        k = ctx.n_logit_rows
        if k == 0:
            return None
        xn = ctx.scratch("head_in", (k, self.hidden_size), self.dtype, capacity=ctx.max_logit_rows)
        logits = ctx.scratch("logits", (k, self.vocab_size), torch.float32, capacity=ctx.max_logit_rows)
        with ctx.range("final norm and head"):
            self.final_norm.forward(x, xn, rows=ctx.logit_rows)
            ctx.tap("final_norm", -1, xn)
            self.head.forward(xn, logits)
            if self.logit_transform is not None:
                self.logit_transform.forward(ctx, logits)
        return logits
