"""What a checkpoint must hold for an architecture, and how it becomes parameters of parts.

A ``WeightPlan`` lists every tensor by its name in the checkpoint with the shape the configuration
implies, the name patterns that may be present but are not used, and a function that assembles the
read tensors into the parameter dictionary of the model (``layers.3.mixer.w_qkv`` and so on).
"""
from __future__ import annotations

import fnmatch
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Tuple

import torch


@dataclass(frozen=True)
class TensorRule:
    name: str
    shape: Tuple[int, ...]
    kind: str = "matrix"     # "matrix", "vector" (norm weights and the like) or "table" (integers)


@dataclass
class WeightPlan:
    rules: List[TensorRule]
    ignorable: List[str] = field(default_factory=list)      # fnmatch patterns of unused tensors
    assemble: Callable[[Dict[str, torch.Tensor]], Dict[str, torch.Tensor]] = lambda t: dict(t)

    def is_ignorable(self, name: str) -> bool:
        return any(fnmatch.fnmatchcase(name, p) for p in self.ignorable)


def llama_weight_plan(cfg) -> WeightPlan:
    """Tensor names and shapes of a Llama checkpoint (src/loader/hf_checkpoint.cpp:214-235).

    q/k/v are concatenated into one ``w_qkv`` [A+2K, D] and gate/up into one ``w_gate_up`` [2I, D]
    (gate rows first) so that each pair of projections is a single matrix product. A tied model's
    head is the embedding table itself (one copy on the device)."""
    D, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    A, K = cfg.attn_dim, cfg.kv_dim
    rules = [TensorRule("model.embed_tokens.weight", (V, D))]
    for l in range(cfg.num_hidden_layers):
        p = f"model.layers.{l}."
        rules += [
            TensorRule(p + "input_layernorm.weight", (D,), "vector"),
            TensorRule(p + "self_attn.q_proj.weight", (A, D)),
            TensorRule(p + "self_attn.k_proj.weight", (K, D)),
            TensorRule(p + "self_attn.v_proj.weight", (K, D)),
            TensorRule(p + "self_attn.o_proj.weight", (D, A)),
            TensorRule(p + "post_attention_layernorm.weight", (D,), "vector"),
            TensorRule(p + "mlp.gate_proj.weight", (I, D)),
            TensorRule(p + "mlp.up_proj.weight", (I, D)),
            TensorRule(p + "mlp.down_proj.weight", (D, I)),
        ]
    rules.append(TensorRule("model.norm.weight", (D,), "vector"))
    ignorable = ["model.layers.*.self_attn.rotary_emb.inv_freq"]
    if cfg.tie_word_embeddings:
        ignorable.append("lm_head.weight")      # a redundant copy some exporters leave in tied models
    else:
        rules.append(TensorRule("lm_head.weight", (V, D)))

    def assemble(t: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        out: Dict[str, torch.Tensor] = {"embedding.weight": t["model.embed_tokens.weight"]}
        for l in range(cfg.num_hidden_layers):
            p, q = f"model.layers.{l}.", f"layers.{l}."
            out[q + "mixer_norm.weight"] = t[p + "input_layernorm.weight"]
            out[q + "mixer.w_qkv"] = _cat([t[p + "self_attn.q_proj.weight"], t[p + "self_attn.k_proj.weight"],
                                           t[p + "self_attn.v_proj.weight"]])
            out[q + "mixer.w_o"] = t[p + "self_attn.o_proj.weight"]
            out[q + "feed_forward_norm.weight"] = t[p + "post_attention_layernorm.weight"]
            out[q + "feed_forward.w_gate_up"] = _cat([t[p + "mlp.gate_proj.weight"], t[p + "mlp.up_proj.weight"]])
            out[q + "feed_forward.w_down"] = t[p + "mlp.down_proj.weight"]
        out["final_norm.weight"] = t["model.norm.weight"]
        out["head.weight"] = out["embedding.weight"] if cfg.tie_word_embeddings else t["lm_head.weight"]
        return out

    return WeightPlan(rules, ignorable, assemble)


def _cat(parts: List[torch.Tensor]) -> torch.Tensor:
    """Concatenates rows; parts of different stored dtypes are widened to 32-bit first."""
    if len({p.dtype for p in parts}) > 1:
        parts = [p.float() for p in parts]
    return torch.cat(parts, dim=0)
