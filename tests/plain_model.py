"""A plain, slow implementation of the Llama forward pass, sampler and generation loop.

It is the oracle of the tests: whole sequences, no cache, no batching, one function per part,
32-bit arithmetic on the CPU (64-bit where the reference uses double). It is written from the
reference's formulas, each function citing where they stand, and shares no code with the engine:
it has its own safetensors reader, its own configuration defaults and its own sampler.

Anchoring: tests/golden/ holds logits that the reference's own C++ model (gi_forward, built on the
CPU) produced for a tiny random model; tests/test_plain_model.py compares this implementation
with them (see tests/golden/make_golden.py).
"""
from __future__ import annotations

import json
import math
import struct
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

F32 = torch.float32


# --------------------------------------------------------------------------------------- files
def read_safetensors_f32(path: str) -> Dict[str, torch.Tensor]:
    """All tensors of a safetensors file widened to float32 (layout: tools/hf_io.py:52-67;
    bfloat16 -> float32 is a 16-bit shift, src/loader/dtype.cpp:23-40)."""
    with open(path, "rb") as f:
        blob = f.read()
    (n,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + n].decode("utf-8"))
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        raw = blob[8 + n + b:8 + n + e]
        if info["dtype"] == "F32":
            arr = np.frombuffer(raw, dtype="<f4").astype(np.float32)
        elif info["dtype"] == "BF16":
            arr = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32)
        elif info["dtype"] == "F16":
            arr = np.frombuffer(raw, dtype="<f2").astype(np.float32)
        else:
            raise ValueError(f"dtype {info['dtype']} of '{name}'")
        out[name] = torch.from_numpy(arr.copy()).reshape(info["shape"])
    return out


def read_config(path: str) -> dict:
    """config.json with the reference's defaults applied (src/loader/hf_checkpoint.cpp:112-134)."""
    with open(path) as f:
        c = json.load(f)
    heads = c["num_attention_heads"]
    out = {
        "hidden": c["hidden_size"], "inter": c["intermediate_size"], "layers": c["num_hidden_layers"],
        "heads": heads, "kv_heads": c.get("num_key_value_heads") or heads,
        "head_dim": c.get("head_dim") or c["hidden_size"] // heads, "vocab": c["vocab_size"],
        "max_pos": c.get("max_position_embeddings") or 2048,
        "theta": c.get("rope_theta") if c.get("rope_theta") is not None else 10000.0,
        "eps": c.get("rms_norm_eps") if c.get("rms_norm_eps") is not None else 1e-6,
        "tied": c.get("tie_word_embeddings") is True, "scaling": None,
    }
    s = c.get("rope_scaling")
    if s and s.get("rope_type", s.get("type")) == "llama3":
        out["scaling"] = (float(s["factor"]), float(s["low_freq_factor"]), float(s["high_freq_factor"]),
                          float(s["original_max_position_embeddings"]))
    return out


# --------------------------------------------------------------------------------------- parts
def plain_embedding(table: torch.Tensor, tokens: Sequence[int]) -> torch.Tensor:
    """x[t] = E[token_t], no scaling (src/model/transformer.cpp:372-376)."""
    return table[torch.tensor(list(tokens), dtype=torch.long)].to(F32).clone()


def plain_rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """scale = 1/sqrt(sum(x^2)/n + eps); out = w * (scale * x) (src/kernels/kernels.cpp:72-83)."""
    n = x.shape[-1]
    ss = (x * x).sum(dim=-1, keepdim=True)
    scale = 1.0 / torch.sqrt(ss / np.float32(n) + np.float32(eps))
    return weight.to(F32) * (scale * x)


def plain_rope_table(positions: Sequence[int], head_dim: int, theta: float, scaling=None):
    """cos/sin rows [len(positions), head_dim/2]: frequencies and angles in double, rounded to float
    at the end; "llama3" scaling in its three regimes (src/kernels/kernels.cpp:142-163). theta is
    held as a float by the reference's Config (src/loader/hf_checkpoint.cpp:125)."""
    half = head_dim // 2
    theta = float(np.float32(theta))
    cos = np.zeros((len(positions), half), dtype=np.float32)
    sin = np.zeros((len(positions), half), dtype=np.float32)
    for k in range(half):
        freq = 1.0 / math.pow(theta, 2.0 * k / head_dim)
        if scaling is not None:
            factor, low, high, original = scaling
            wavelength = 6.283185307179586476925 / freq
            if wavelength > original / low:
                freq /= factor
            elif not (wavelength < original / high):
                smooth = (original / wavelength - low) / (high - low)
                freq = (1.0 - smooth) * freq / factor + smooth * freq
        for i, p in enumerate(positions):
            angle = float(p) * freq
            cos[i, k] = np.float32(math.cos(angle))
            sin[i, k] = np.float32(math.sin(angle))
    return torch.from_numpy(cos), torch.from_numpy(sin)


def plain_rope(v: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Half-split pairing: (a, b) = (v[k], v[k + hd/2]); a' = a c - b s; b' = a s + b c
    (src/kernels/kernels.cpp:164-180). v: [T, heads, hd]; cos, sin: [T, hd/2]."""
    half = v.shape[-1] // 2
    a, b = v[..., :half], v[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([a * c - b * s, a * s + b * c], dim=-1)


def plain_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                    window: Optional[int] = None, rnd=None) -> torch.Tensor:
    """Causal grouped-query attention of a whole sequence (src/model/transformer.cpp:228-255):
    for the query at position P and head h, kv head g = h // (H / Hkv), scores
    s_j = (q . k_j) * scale for j <= P only, softmax with the sum in double
    (src/kernels/kernels.cpp:87-104), out = sum_j p_j v_j. q: [T, H, hd]; k, v: [T, Hkv, hd].
    ``rnd`` (bfloat16 engines): the unnormalised weights exp(s - max) are rounded as the operand of
    the product with v, while their sum stays 32-bit: out = (rnd(e) @ v) / sum(e)."""
    T, H, hd = q.shape
    Hkv = k.shape[1]
    mul = H // Hkv
    out = torch.zeros_like(q)
    for h in range(H):
        g = h // mul
        for P in range(T):
            lo = 0 if window is None else max(0, P - window + 1)
            s = (k[lo:P + 1, g] @ q[P, h]) * np.float32(scale)
            e = torch.exp(s - s.max())
            if rnd is None:
                p = e / e.double().sum().to(F32)
                out[P, h] = p @ v[lo:P + 1, g]
            else:
                out[P, h] = (rnd(e) @ v[lo:P + 1, g]) / e.double().sum().to(F32)
    return out


def plain_swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """g * (1 / (1 + exp(-g))) * u (src/kernels/kernels.cpp:106-110, src/model/transformer.cpp:441-447)."""
    return gate * (1.0 / (1.0 + torch.exp(-gate))) * up


def no_rounding(t: torch.Tensor) -> torch.Tensor:
    return t


def bf16_rounding(t: torch.Tensor) -> torch.Tensor:
    """Rounds to bfloat16 (nearest even) and widens again."""
    return t.to(torch.bfloat16).to(F32)


def plain_layer(x: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str, cfg: dict, cos, sin,
                rnd=no_rounding) -> torch.Tensor:
    """One layer in the reference's order: norm, q/k/v, rope on q and k, attention, o, +, norm,
    gate/up, silu*up, down, + (src/model/transformer.cpp:379-451). ``rnd`` is applied where a
    bfloat16 engine stores an activation in 16 bits (the operands of matrix products and what goes
    into the cache); sums, norms, rotation and softmax stay 32-bit either way."""
    T = x.shape[0]
    H, Hkv, hd = cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
    xb = rnd(plain_rmsnorm(x, w[prefix + "input_layernorm.weight"], cfg["eps"]))
    q = (xb @ w[prefix + "self_attn.q_proj.weight"].T).reshape(T, H, hd)
    k = (xb @ w[prefix + "self_attn.k_proj.weight"].T).reshape(T, Hkv, hd)
    v = rnd((xb @ w[prefix + "self_attn.v_proj.weight"].T).reshape(T, Hkv, hd))
    q, k = rnd(plain_rope(q, cos, sin)), rnd(plain_rope(k, cos, sin))
    att = rnd(plain_attention(q, k, v, 1.0 / math.sqrt(np.float32(hd)), cfg.get("window"),
                              None if rnd is no_rounding else rnd))
    x = x + att.reshape(T, H * hd) @ w[prefix + "self_attn.o_proj.weight"].T
    xb = rnd(plain_rmsnorm(x, w[prefix + "post_attention_layernorm.weight"], cfg["eps"]))
    h = rnd(plain_swiglu(xb @ w[prefix + "mlp.gate_proj.weight"].T, xb @ w[prefix + "mlp.up_proj.weight"].T))
    return x + h @ w[prefix + "mlp.down_proj.weight"].T


def plain_forward(w: Dict[str, torch.Tensor], cfg: dict, tokens: Sequence[int], rnd=no_rounding,
                  positions: Optional[Sequence[int]] = None) -> torch.Tensor:
    """Logits [T, vocab] at every position of one whole sequence, or only at ``positions`` (in
    their order) when given (final norm and head: src/model/transformer.cpp:453-474; the head is
    the embedding table when tied)."""
    T = len(tokens)
    cos, sin = plain_rope_table(range(T), cfg["head_dim"], cfg["theta"], cfg["scaling"])
    x = plain_embedding(w["model.embed_tokens.weight"], tokens)
    for l in range(cfg["layers"]):
        x = plain_layer(x, w, f"model.layers.{l}.", cfg, cos, sin, rnd)
    if positions is not None:
        x = x[torch.tensor(list(positions), dtype=torch.long)]
    xn = rnd(plain_rmsnorm(x, w["model.norm.weight"], cfg["eps"]))
    head = w["model.embed_tokens.weight"] if cfg["tied"] else w["lm_head.weight"]
    return xn @ head.to(F32).T


def round_weights_bf16(w: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """What a bfloat16 engine makes of 32-bit stored weights: matrices rounded, norm weights kept."""
    return {k: (v if v.dim() == 1 else bf16_rounding(v)) for k, v in w.items()}


def load_plain(model_dir: str):
    return read_safetensors_f32(f"{model_dir}/model.safetensors"), read_config(f"{model_dir}/config.json")


# --------------------------------------------------------------------------------------- sampler
_MASK = (1 << 64) - 1


class PlainSampler:
    """The reference sampler (src/sampler/sampler.cpp:16-129): splitmix64-seeded xorshift64*,
    u = (u32 >> 8) / 2^24; greedy for temperature <= 0 (lowest index on ties); otherwise
    softmax(logits / temperature) with a double sum, top-k then top-p over the tokens sorted by
    probability (descending, index ascending), inverse-CDF draw in that order, or in index order
    when no filter is on."""

    def __init__(self, temperature: float = 0.8, top_k: int = 0, top_p: float = 1.0, seed: int = 1):
        x = (seed + 0x9E3779B97F4A7C15) & _MASK
        x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
        x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _MASK
        x ^= x >> 31
        self.state = x or 1
        self.temperature, self.top_k, self.top_p = np.float32(temperature), top_k, np.float32(top_p)

    def next_uniform(self) -> np.float32:
        s = self.state
        s ^= s >> 12
        s ^= (s << 25) & _MASK
        s ^= s >> 27
        self.state = s
        u32 = ((s * 0x2545F4914F6CDD1D) & _MASK) >> 32
        return np.float32(u32 >> 8) / np.float32(16777216.0)

    def sample(self, logits: np.ndarray, u: Optional[float] = None) -> int:
        logits = np.asarray(logits, dtype=np.float32)
        if self.temperature <= 0:
            return int(np.argmax(logits))            # first maximum = lowest index
        if u is None:
            u = self.next_uniform()
        probs = np.exp((logits - logits.max()) / self.temperature).astype(np.float32)
        inv = np.float32(1.0 / probs.astype(np.float64).sum())
        probs = probs * inv
        n = len(probs)
        order = np.arange(n)
        kept = n
        use_k = 0 < self.top_k < n
        use_p = self.top_p < 1.0
        if use_k or use_p:
            order = np.lexsort((np.arange(n), -probs.astype(np.float64)))
            if use_k:
                kept = self.top_k
            if use_p:
                total = probs[order[:kept]].astype(np.float64).sum()
                cum = np.cumsum(probs[order[:kept]].astype(np.float64))
                hit = np.nonzero(cum >= np.float64(self.top_p) * total)[0]
                kept = int(hit[0]) + 1 if len(hit) else kept
        p = probs[order[:kept]].astype(np.float64)
        r = np.float64(u) * p.sum()
        cum = np.cumsum(p)
        hit = np.nonzero(r < cum)[0]
        return int(order[hit[0]]) if len(hit) else int(order[kept - 1])


def plain_generate(w, cfg, prompt: Sequence[int], max_new: int, sampler: PlainSampler,
                   stop_ids: Sequence[int] = ()) -> List[int]:
    """Token loop of the reference (src/runtime/generator.cpp:42-76): the logits at the last known
    token give the next one; a sampled end token is kept and ends the loop; positions are capped
    by the context length. The whole sequence is recomputed for every token."""
    tokens = list(prompt)
    out: List[int] = []
    while len(out) < max_new and len(tokens) < cfg["max_pos"] + 1:
        logits = plain_forward(w, cfg, tokens)[-1].numpy()
        nxt = sampler.sample(logits)
        out.append(nxt)
        tokens.append(nxt)
        if nxt in stop_ids or len(tokens) > cfg["max_pos"]:
            break
    return out
