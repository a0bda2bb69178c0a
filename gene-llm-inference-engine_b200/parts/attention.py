"""The attention mixer: grouped-query causal attention over the paged cache."""
from __future__ import annotations

import torch

from ..cache import CacheNeed
from ..config import PartSpec
from ..ops import kernels
from ..ops.linear import Linear
from .registry import POSITION_ENCODINGS, build_part, register_mixer


@register_mixer("attention")
class AttentionMixer:
    """q, k, v = W_qkv xn; position encoding on q and k; k, v stored in the request's pages;
    causal softmax(q k^T * scale) v per head with query head h reading key/value head
    h // (H / Hkv); x += W_o out (src/model/transformer.cpp:389-434).

    Params: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``, ``scale`` (multiplied
    after the dot product), ``window`` (None = all keys) and ``position`` (a PartSpec).
    Weights: ``w_qkv`` [(H+2Hkv)*hd, hidden] and ``w_o`` [hidden, H*hd]."""

    graph_safe = True      # launches depend only on the step's shape: decode steps may be captured in a CUDA graph


    def __init__(self, params, weights, build):
        self.hidden_size = int(params["hidden_size"])
        self.num_heads = int(params["num_heads"])
        self.num_kv_heads = int(params["num_kv_heads"])
        self.head_dim = int(params["head_dim"])
        self.scale = float(params["scale"])
        self.window = params.get("window")
        if self.num_heads % self.num_kv_heads:
            raise ValueError("attention: num_heads must be a multiple of num_kv_heads")
        if not kernels.attention_supported(self.head_dim):
            raise ValueError(f"attention: head size {self.head_dim} is not supported by the attention kernels "
                             f"(multiples of 16 up to 256)")
        pos_spec = params.get("position") or PartSpec("none", {})
        self.position = build_part(POSITION_ENCODINGS, "position encoding", pos_spec, {}, build)
        qkv_rows = (self.num_heads + 2 * self.num_kv_heads) * self.head_dim
        if tuple(weights["w_qkv"].shape) != (qkv_rows, self.hidden_size):
            raise ValueError(f"attention: w_qkv has shape {tuple(weights['w_qkv'].shape)}, expected "
                             f"({qkv_rows}, {self.hidden_size})")
        if tuple(weights["w_o"].shape) != (self.hidden_size, self.num_heads * self.head_dim):
            raise ValueError(f"attention: w_o has shape {tuple(weights['w_o'].shape)}")
        self.w_qkv = Linear(weights["w_qkv"], build.compute_dtype, build.device, tiles=build.weight_tiles)
        self.w_o = Linear(weights["w_o"], build.compute_dtype, build.device, tiles=build.weight_tiles)
        self.dtype = build.compute_dtype
        # bfloat16 with a head size the tensor-core kernels are built for; else the general kernel
        self.fast = self.dtype is torch.bfloat16 and kernels.attention_fast_supported(
            self.head_dim, self.num_heads, self.num_kv_heads)
        self._prefill_rows = {}
        if self.fast:
            self.chunk_keys = kernels.attention_chunk_keys()
            self.max_chunks = (build.max_position + self.chunk_keys - 1) // self.chunk_keys

    def prefill_on_tcgen05(self, page_size: int) -> bool:
        """Head sizes 64 and 128 with pages TMA can tile: prompt portions run on the tcgen05 kernel."""
        key = ("tc", page_size)
        if key not in self._prefill_rows:
            self._prefill_rows[key] = kernels.attention_prefill_tc_supported(self.head_dim, self.num_heads,
                                                                             self.num_kv_heads, page_size)
        return self._prefill_rows[key]

    def prefill_rows(self, page_size: int) -> int:
        """Query rows (tokens x heads of a group) per work item of the prefill kernel in use."""
        if page_size not in self._prefill_rows:
            self._prefill_rows[page_size] = 128 if self.prefill_on_tcgen05(page_size) else \
                kernels.attention_prefill_rows(page_size, self.head_dim)
        return self._prefill_rows[page_size]

    def cache_need(self):
        return CacheNeed(self.num_kv_heads, self.head_dim, self.window)

    def state_need(self):
        return None

    def launch_key(self, ctx, run):
        """What the mixer's launches depend on besides the token count: whose cache it uses, and (tensor-core
        kernels) how many rows are single decoded tokens, how many tiles the prompt portions make and how many
        chunks the longest context of a single token has. Asking also places this step's work lists on the device."""
        if not self.fast:
            return (run.cache_layer, run.writes_cache)
        rows, work, longest = ctx.attention_work(self.prefill_rows(ctx.page_size) // (self.num_heads // self.num_kv_heads))
        return (run.cache_layer, run.writes_cache, rows.numel(), work.shape[0],
                (longest + self.chunk_keys - 1) // self.chunk_keys)

    takes_then = True      # forward accepts ``then``

    def forward(self, ctx, run, xn: torch.Tensor, x: torch.Tensor, then=None) -> None:
        """``xn``: normalised input [T, hidden] in the compute dtype; ``x``: the 32-bit residual
        stream, to which the mixer's output is added. ``run`` names whose cache to use. ``then``: the Linear
        of the large product that follows this mixer (the feed-forward's first), for the last product here to
        ask the start of its weights into L2."""
        T = xn.shape[0]
        H, Hkv, hd = self.num_heads, self.num_kv_heads, self.head_dim
        k_cache, v_cache = ctx.pages(run.cache_layer)
        tables = ctx.block_tables(run.cache_layer)
        q = ctx.scratch("q", (T, H * hd), self.dtype)
        if self.dtype is torch.bfloat16 and kernels.gemm_rope_store_supported(
                T, self.hidden_size, H, Hkv, hd, self.position.cos, self.position.interleaved):
            # rotation and page store in the epilogue of the product
            kernels.gemm_rope_store(xn, self.w_qkv.weight, ctx.positions, ctx.row_req, tables, self.position.cos,
                                    self.position.sin, self.position.interleaved, q, k_cache, v_cache, H, Hkv, hd,
                                    ctx.page_size, write_kv=run.writes_cache, w_tiles=self.w_qkv.weight_tiles)
        else:
            qkv = ctx.scratch("qkv", (T, (H + 2 * Hkv) * hd), torch.float32)
            self.w_qkv.forward(xn, qkv)
            kernels.rope_store(qkv, ctx.positions, ctx.row_req, tables, self.position.cos, self.position.sin,
                               self.position.interleaved, q, k_cache, v_cache, H, Hkv, hd, ctx.page_size,
                               write_kv=run.writes_cache)
        att = ctx.scratch("att", (T, H * hd), self.dtype)
        if self.fast:
            # tensor-core kernels: single decoded tokens split their context over many CTAs,
            # portions of prompts run tile by tile
            rows, work, longest = ctx.attention_work(self.prefill_rows(ctx.page_size) // (H // Hkv))
            if rows.numel():
                n = rows.numel()
                part_o = ctx.scratch("att_part_o", (n, H * self.max_chunks * hd), torch.float32, capacity=ctx.max_requests)
                part_ml = ctx.scratch("att_part_ml", (n, H * self.max_chunks * 2), torch.float32, capacity=ctx.max_requests)
                n_chunks = (longest + self.chunk_keys - 1) // self.chunk_keys
                kernels.attention_decode(q, k_cache, v_cache, att, rows, ctx.row_req, ctx.positions, tables, H, Hkv, hd,
                                         ctx.page_size, self.scale, self.window, part_o, part_ml, self.max_chunks, n_chunks)
            if work.shape[0]:
                prefill = kernels.attention_prefill_tc if self.prefill_on_tcgen05(ctx.page_size) else kernels.attention_prefill
                prefill(q, k_cache, v_cache, att, work, ctx.positions, tables, H, Hkv, hd, ctx.page_size, self.scale,
                        self.window)
        else:
            kernels.attention_generic(q, k_cache, v_cache, att, ctx.row_req, ctx.positions, tables, H, Hkv, hd,
                                      ctx.page_size, self.scale, self.window)
        self.w_o.forward(att, x, accumulate=True, then=then)
