"""Each part alone against its plain counterpart; a schedule that runs a layer twice on another
layer's cache; and a toy architecture, defined here, whose mixer keeps state of its own: it is
registered, built and stepped without any change to the framework's files."""
import math
import os

import numpy as np
import pytest
import torch

import gpu_fixtures as gf
import plain_model as pm
import tiny_configs as tc
import trace_tools as tt

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def _build():
    from geneinfer_b200.parts import BuildContext
    return lambda dtype, max_position=64: BuildContext(DEV, dtype, max_position)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_part(dtype):
    from geneinfer_b200.parts import NORMS
    w = 1 + 0.1 * torch.randn(200)
    part = NORMS["rmsnorm"]({"size": 200, "eps": 0.01}, {"weight": w.to(torch.bfloat16)}, _build()(dtype))
    assert part.weight.dtype == torch.float32              # kept in 32-bit whatever the file stores
    x = torch.randn(9, 200) * 2
    out = torch.empty(9, 200, dtype=dtype, device=DEV)
    part.forward(x.to(DEV), out)
    want = pm.plain_rmsnorm(x, w.to(torch.bfloat16).float(), 0.01)
    assert tt.rel_err(out.float().cpu().numpy(), want.numpy()) < (2e-6 if dtype is torch.float32 else 1e-2)


@pytest.mark.parametrize("scaling", [None, {"factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                                             "original_max_position": 64}])
def test_position_part_table(scaling):
    from geneinfer_b200.parts import POSITION_ENCODINGS
    part = POSITION_ENCODINGS["rope"]({"head_dim": 32, "theta": 500000.0, "pairing": "half_split", "scaling": scaling},
                                      {}, _build()(torch.float32, 300))
    tup = None if scaling is None else (32.0, 1.0, 4.0, 64.0)
    cos, sin = pm.plain_rope_table(range(300), 32, 500000.0, tup)
    assert torch.equal(part.cos.cpu(), cos) and torch.equal(part.sin.cpu(), sin)     # both computed in double


class _Ctx:
    """The least a part needs of a step: row arrays, one layer's pages, scratch."""

    def __init__(self, dtype, lens, Hkv, hd, page_size=8):
        self.page_size = page_size
        self.max_requests = len(lens)
        self._lens = list(lens)
        self._starts = [sum(lens[:i]) for i in range(len(lens))]
        T = sum(lens)
        self.n_tokens = T
        self.positions = torch.cat([torch.arange(n) for n in lens]).int().to(DEV)
        self.row_req = torch.cat([torch.full((n,), r) for r, n in enumerate(lens)]).int().to(DEV)
        stride = max((n + page_size - 1) // page_size for n in lens)
        tables = torch.full((len(lens), stride), -1, dtype=torch.int32)
        nxt = 0
        for r, n in enumerate(lens):
            for i in range((n + page_size - 1) // page_size):
                tables[r, i] = nxt
                nxt += 1
        self._tables = tables.to(DEV)
        self._pages = (torch.full((nxt, Hkv, page_size, hd), float("nan"), dtype=dtype, device=DEV),
                       torch.full((nxt, Hkv, page_size, hd), float("nan"), dtype=dtype, device=DEV))

    def pages(self, layer):
        return self._pages

    def block_tables(self, layer):
        return self._tables

    def scratch(self, name, shape, dtype, capacity=None):
        return torch.full(shape, float("nan"), dtype=dtype, device=DEV)

    def attention_work(self, per_tile):
        single = [s for s, n in zip(self._starts, self._lens) if n == 1]
        tiles = [(s + t, min(per_tile, n - t), r) for r, (s, n) in enumerate(zip(self._starts, self._lens)) if n > 1
                 for t in range(0, n, per_tile)]
        assert per_tile in (128 // 3, 64 // 3)
        return (torch.tensor(single, dtype=torch.int32, device=DEV),
                torch.tensor(tiles, dtype=torch.int32, device=DEV).reshape(len(tiles), 3), 1)


def test_a_head_size_the_kernels_do_not_serve_is_refused_when_the_model_is_built(tmp_path):
    """config.json may give any even head size (the reference accepts it); the attention kernels serve
    multiples of 16 up to 256. The refusal comes when the model is built, with the size in the message,
    not at the first step after weights and pages are on the device."""
    from geneinfer_b200.engine.loading import load_model
    config = dict(tc.TINY_A, head_dim=24, hidden_size=96, num_attention_heads=4, num_key_value_heads=2)
    folder = tc.make_model_dir(config, tc.WEIGHTS_A, str(tmp_path / "hd24"))
    with pytest.raises(ValueError, match="head size 24"):
        load_model(folder, dtype="float32")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_mixer_part(dtype):
    from geneinfer_b200.config import PartSpec
    from geneinfer_b200.parts import MIXERS, LayerRun
    D, H, Hkv, hd = 72, 6, 2, 16
    g = torch.Generator().manual_seed(3)
    w_qkv = (torch.randn((H + 2 * Hkv) * hd, D, generator=g) * 0.3).to(torch.bfloat16).float()
    w_o = (torch.randn(D, H * hd, generator=g) * 0.3).to(torch.bfloat16).float()
    rope = PartSpec("rope", {"head_dim": hd, "theta": 10000.0, "pairing": "half_split", "scaling": None})
    part = MIXERS["attention"]({"hidden_size": D, "num_heads": H, "num_kv_heads": Hkv, "head_dim": hd,
                                "scale": 0.25, "window": None, "position": rope},
                               {"w_qkv": w_qkv, "w_o": w_o}, _build()(dtype))
    assert part.cache_need().num_kv_heads == Hkv and part.state_need() is None
    lens = [11, 1, 20]
    ctx = _Ctx(dtype, lens, Hkv, hd)
    xn = torch.randn(sum(lens), D, generator=g).to(dtype)
    x = torch.randn(sum(lens), D, generator=g)
    x_dev = x.clone().to(DEV)
    part.forward(ctx, LayerRun(0, 0, True), xn.to(DEV), x_dev)
    rnd = pm.no_rounding if dtype is torch.float32 else pm.bf16_rounding
    start = 0
    for n in lens:
        seg = xn[start:start + n].float()
        cos, sin = pm.plain_rope_table(range(n), hd, 10000.0)
        qkv = seg @ w_qkv.T
        q = rnd(pm.plain_rope(qkv[:, :H * hd].reshape(n, H, hd), cos, sin))
        k = rnd(pm.plain_rope(qkv[:, H * hd:(H + Hkv) * hd].reshape(n, Hkv, hd), cos, sin))
        v = rnd(qkv[:, (H + Hkv) * hd:].reshape(n, Hkv, hd))
        want = x[start:start + n] + rnd(pm.plain_attention(q, k, v, 0.25, None, None if dtype is torch.float32 else rnd)).reshape(n, H * hd) @ w_o.T
        err = tt.rel_err(x_dev[start:start + n].cpu().numpy(), want.numpy())
        assert err < (1e-5 if dtype is torch.float32 else 1.5e-2), f"segment at {start}: {err}"
        start += n


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_part(dtype):
    from geneinfer_b200.parts import FEED_FORWARDS
    D, I = 40, 112
    g = torch.Generator().manual_seed(4)
    w_gu = (torch.randn(2 * I, D, generator=g) * 0.3).to(torch.bfloat16).float()
    w_d = (torch.randn(D, I, generator=g) * 0.3).to(torch.bfloat16).float()
    part = FEED_FORWARDS["swiglu"]({"hidden_size": D, "intermediate_size": I}, {"w_gate_up": w_gu, "w_down": w_d},
                                   _build()(dtype))
    xn = torch.randn(13, D, generator=g).to(dtype)
    x = torch.randn(13, D, generator=g)
    x_dev = x.clone().to(DEV)
    part.forward(_Ctx(dtype, [13], 1, 16), xn.to(DEV), x_dev)
    rnd = pm.no_rounding if dtype is torch.float32 else pm.bf16_rounding
    gu = xn.float() @ w_gu.T
    want = x + rnd(pm.plain_swiglu(gu[:, :I], gu[:, I:])) @ w_d.T
    assert tt.rel_err(x_dev.cpu().numpy(), want.numpy()) < (1e-5 if dtype is torch.float32 else 1.5e-2)


def test_schedule_runs_a_layer_twice_on_another_layers_cache():
    """Schedule [0, 1, 1 reading layer 0's cache without writing it]: the third run applies layer
    1's weights again, its queries attend over the keys and values layer 0 stored."""
    from geneinfer_b200.config import ScheduleEntry, parse_config
    from geneinfer_b200.engine.step import StepEngine, StepEntry
    from geneinfer_b200.parts import DecoderModel
    from geneinfer_b200.weights import load_model_folder
    _, cfg, params = load_model_folder(gf.model_dir("a"))
    spec = cfg.model_spec()
    spec.schedule = [ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(1, cache_of=0, writes_cache=False)]
    model = DecoderModel(spec, params, torch.float32, DEV)
    assert sorted(model.cache_needs()) == [0, 1]
    engine = StepEngine(model, page_size=16, n_pages=8, max_requests=2, max_step_tokens=64)
    toks = tc.random_tokens(40, 256, 3)
    engine.open("r")
    a = engine.step([StepEntry("r", toks[:25], list(range(25)))]).cpu().numpy()
    b = engine.step([StepEntry("r", toks[25:], list(range(15)))]).cpu().numpy()
    got = np.concatenate([a, b])

    w, pc = pm.load_plain(gf.model_dir("a"))
    T, H, Hkv, hd = 40, pc["heads"], pc["kv_heads"], pc["head_dim"]
    cos, sin = pm.plain_rope_table(range(T), hd, pc["theta"], pc["scaling"])
    x = pm.plain_embedding(w["model.embed_tokens.weight"], toks)
    xb0 = pm.plain_rmsnorm(x, w["model.layers.0.input_layernorm.weight"], pc["eps"])
    k0 = pm.plain_rope((xb0 @ w["model.layers.0.self_attn.k_proj.weight"].T).reshape(T, Hkv, hd), cos, sin)
    v0 = (xb0 @ w["model.layers.0.self_attn.v_proj.weight"].T).reshape(T, Hkv, hd)
    x = pm.plain_layer(x, w, "model.layers.0.", pc, cos, sin)
    x = pm.plain_layer(x, w, "model.layers.1.", pc, cos, sin)
    p = "model.layers.1."
    xb = pm.plain_rmsnorm(x, w[p + "input_layernorm.weight"], pc["eps"])
    q = pm.plain_rope((xb @ w[p + "self_attn.q_proj.weight"].T).reshape(T, H, hd), cos, sin)
    x = x + pm.plain_attention(q, k0, v0, 1.0 / math.sqrt(hd)).reshape(T, H * hd) @ w[p + "self_attn.o_proj.weight"].T
    xb = pm.plain_rmsnorm(x, w[p + "post_attention_layernorm.weight"], pc["eps"])
    x = x + pm.plain_swiglu(xb @ w[p + "mlp.gate_proj.weight"].T, xb @ w[p + "mlp.up_proj.weight"].T) @ w[p + "mlp.down_proj.weight"].T
    want = (pm.plain_rmsnorm(x, w["model.norm.weight"], pc["eps"]) @ w["model.embed_tokens.weight"].T).numpy()
    assert tt.rel_err(got, want) < gf.TOL_F32


# ------------------------------------------------------------------------------------------ a toy architecture
def _register_toy():
    """A mixer with state of its own (a decaying running sum of its inputs, carried across steps
    in the request's state slot), an architecture that alternates it with attention, its config
    class and weight plan: all defined here, entered through the public registries."""
    from geneinfer_b200.cache import StateNeed
    from geneinfer_b200.config import (Architecture, LayerSpec, ModelSpec, PartSpec, ScheduleEntry, register_architecture)
    from geneinfer_b200.parts import MIXERS, register_mixer
    from geneinfer_b200.weights.plan import TensorRule, WeightPlan
    if "toy_running_sum" in MIXERS:
        return

    @register_mixer("toy_running_sum")
    class RunningSum:
        def __init__(self, params, weights, build):
            self.size, self.decay = params["hidden_size"], params["decay"]
            self.w = weights["w_mix"].to(device=build.device, dtype=torch.float32)

        def cache_need(self):
            return None

        def state_need(self):
            return StateNeed((self.size,), "float32")

        def forward(self, ctx, run, xn, x):
            state = ctx.state(run.cache_layer)
            for seg in ctx.segments:                      # s_t = decay * s_{t-1} + xn_t, carried across steps
                s = state[seg.state_slot]
                rows = xn[seg.start:seg.start + seg.length].float()
                outs = []
                for t in range(seg.length):
                    s = self.decay * s + rows[t]
                    outs.append(s)
                state[seg.state_slot] = s
                x[seg.start:seg.start + seg.length] += torch.stack(outs) @ self.w.T

    class ToyConfig:
        architecture = "ToyForCausalLM"

        def __init__(self, j):
            self.hidden, self.layers, self.vocab, self.decay = j["hidden"], j["layers"], j["vocab"], j["decay"]
            self.max_pos = j["max_pos"]

        @classmethod
        def from_json(cls, j):
            return cls(j)

        def model_spec(self):
            D = self.hidden
            norm = PartSpec("rmsnorm", {"size": D, "eps": 1e-5})
            ffn = PartSpec("swiglu", {"hidden_size": D, "intermediate_size": 2 * D})
            rope = PartSpec("rope", {"head_dim": 16, "theta": 100.0, "pairing": "interleaved", "scaling": None})
            att = PartSpec("attention", {"hidden_size": D, "num_heads": 2, "num_kv_heads": 1, "head_dim": 16,
                                         "scale": 0.25, "window": 12, "position": rope})
            toy = PartSpec("toy_running_sum", {"hidden_size": D, "decay": self.decay})
            layers = [LayerSpec(toy if i % 2 == 0 else att, ffn, norm, norm) for i in range(self.layers)]
            return ModelSpec("ToyForCausalLM", D, self.vocab, self.max_pos, layers,
                             [ScheduleEntry(i) for i in range(self.layers)], norm, True)

    def plan(cfg):
        D = cfg.hidden
        rules = [TensorRule("emb", (cfg.vocab, D)), TensorRule("norm", (D,), "vector")]
        for i in range(cfg.layers):
            rules += [TensorRule(f"l{i}.n1", (D,), "vector"), TensorRule(f"l{i}.n2", (D,), "vector"),
                      TensorRule(f"l{i}.gu", (4 * D, D)), TensorRule(f"l{i}.down", (D, 2 * D))]
            rules += [TensorRule(f"l{i}.mix", (D, D))] if i % 2 == 0 else \
                     [TensorRule(f"l{i}.qkv", (64, D)), TensorRule(f"l{i}.o", (D, 32))]

        def assemble(t):
            out = {"embedding.weight": t["emb"], "final_norm.weight": t["norm"], "head.weight": t["emb"]}
            for i in range(cfg.layers):
                q = f"layers.{i}."
                out[q + "mixer_norm.weight"], out[q + "feed_forward_norm.weight"] = t[f"l{i}.n1"], t[f"l{i}.n2"]
                out[q + "feed_forward.w_gate_up"], out[q + "feed_forward.w_down"] = t[f"l{i}.gu"], t[f"l{i}.down"]
                if i % 2 == 0:
                    out[q + "mixer.w_mix"] = t[f"l{i}.mix"]
                else:
                    out[q + "mixer.w_qkv"], out[q + "mixer.w_o"] = t[f"l{i}.qkv"], t[f"l{i}.o"]
            return out
        return WeightPlan(rules, [], assemble)

    register_architecture(Architecture("ToyForCausalLM", ("toy",), ToyConfig, plan))


def _toy_plain(w, cfg, toks):
    """The toy model on a whole sequence, from its definition."""
    D, T = cfg["hidden"], len(toks)
    x = w["emb"][torch.tensor(toks)].float()
    for i in range(cfg["layers"]):
        xn = pm.plain_rmsnorm(x, w[f"l{i}.n1"], 1e-5)
        if i % 2 == 0:
            s, outs = torch.zeros(D), []
            for t in range(T):
                s = cfg["decay"] * s + xn[t]
                outs.append(s)
            x = x + torch.stack(outs) @ w[f"l{i}.mix"].T
        else:
            qkv = xn @ w[f"l{i}.qkv"].T
            freq = 1.0 / (100.0 ** (np.arange(8, dtype=np.float64) * 2 / 16))
            ang = np.arange(T, dtype=np.float64)[:, None] * freq[None]
            c, s_ = torch.from_numpy(np.cos(ang).astype(np.float32))[:, None], torch.from_numpy(np.sin(ang).astype(np.float32))[:, None]

            def rot(v):                                     # interleaved pairs
                a, b = v[..., 0::2], v[..., 1::2]
                out = torch.empty_like(v)
                out[..., 0::2], out[..., 1::2] = a * c - b * s_, a * s_ + b * c
                return out
            q, k, v = rot(qkv[:, :32].reshape(T, 2, 16)), rot(qkv[:, 32:48].reshape(T, 1, 16)), qkv[:, 48:].reshape(T, 1, 16)
            x = x + pm.plain_attention(q, k, v, 0.25, window=12).reshape(T, 32) @ w[f"l{i}.o"].T
        xn = pm.plain_rmsnorm(x, w[f"l{i}.n2"], 1e-5)
        gu = xn @ w[f"l{i}.gu"].T
        x = x + pm.plain_swiglu(gu[:, :2 * D], gu[:, 2 * D:]) @ w[f"l{i}.down"].T
    return (pm.plain_rmsnorm(x, w["norm"], 1e-5) @ w["emb"].T).numpy()


def test_toy_architecture_with_a_stateful_mixer(tmp_path):
    _register_toy()
    from geneinfer_b200.engine.loading import load_model
    from geneinfer_b200.engine.step import StepEngine
    from geneinfer_b200.weights import write_random_model
    cfg = {"architectures": ["ToyForCausalLM"], "model_type": "toy", "hidden": 48, "layers": 4, "vocab": 90,
           "decay": 0.9, "max_pos": 96}
    d = write_random_model(cfg, 3, str(tmp_path / "toy"), "float32", std=0.15, norm_std=0.1)
    model = load_model(d, dtype="float32")
    assert sorted(model.state_needs()) == [0, 2] and sorted(model.cache_needs()) == [1, 3]
    reqs = {f"t{i}": tc.random_tokens(n, 90, 200 + i) for i, n in enumerate([50, 96, 17, 64, 33])}
    w = pm.read_safetensors_f32(os.path.join(d, "model.safetensors"))
    plain = {rid: _toy_plain(w, cfg, toks) for rid, toks in reqs.items()}
    for steps in (tt.trace_whole(reqs), tt.trace_portions(reqs), tt.trace_mixed(reqs, seed=4, tail=8)):
        # window 12 with pages of 8: a request never holds more than 3 pages between steps, but a step's
        # portion needs pages for all its tokens
        engine = StepEngine(model, page_size=8, n_pages=4 * 13, max_requests=4, max_step_tokens=128)
        got = tt.run_in_process(engine, steps)
        tt.compare(got, plain, 5e-5, "toy model")
        engine.cache.check_invariants()
        assert engine.cache.slots.free_count == 4 and all(g.pool.free_count == g.pool.n_pages for g in engine.cache.groups)


# ------------------------------------------------------------------------- a second toy architecture
def _register_toy_routed():
    """A feed-forward with routing (router logits in 32-bit, the best of three experts per token,
    each expert a small gated unit) and a position encoding of its own (angles that grow with the
    square root of the position), entered through the public registries like the first toy."""
    from geneinfer_b200.config import (Architecture, LayerSpec, ModelSpec, PartSpec, ScheduleEntry, register_architecture)
    from geneinfer_b200.parts import (FEED_FORWARDS, MIXERS, NORMS, register_block, register_feed_forward,
                                      register_logit_transform, register_position_encoding, build_part, sub_weights)
    from geneinfer_b200.parts.block import build_extra
    from geneinfer_b200.weights.plan import TensorRule, WeightPlan
    if "toy_best_of_three" in FEED_FORWARDS:
        return

    @register_logit_transform("toy_halve")
    class Halve:
        """What an architecture does to its logits after the head: here a constant factor."""
        def __init__(self, params, weights, build):
            self.factor = float(params["factor"])

        def forward(self, ctx, logits):
            logits.mul_(self.factor)

    @register_block("toy_post_norm")
    class PostNormBlock:
        """An arrangement with a fifth part, taken from the layer's ``extra``: the mixer's output goes through a
        norm of its own before it joins the residual stream; the feed-forward half is the usual pre-norm one."""
        def __init__(self, layer_spec, weights, build):
            self.mixer_norm = build_part(NORMS, "norm", layer_spec.mixer_norm, sub_weights(weights, "mixer_norm."), build)
            self.mixer = build_part(MIXERS, "mixer", layer_spec.mixer, sub_weights(weights, "mixer."), build)
            self.post_norm = build_extra(layer_spec, "post_mixer_norm", NORMS, "norm", weights, build)
            self.feed_forward_norm = build_part(NORMS, "norm", layer_spec.feed_forward_norm, sub_weights(weights, "feed_forward_norm."), build)
            self.feed_forward = build_part(FEED_FORWARDS, "feed-forward", layer_spec.feed_forward, sub_weights(weights, "feed_forward."), build)
            self.dtype = build.compute_dtype

        def forward(self, ctx, run, x):
            xn = ctx.scratch("normed", tuple(x.shape), self.dtype)
            y = ctx.scratch("toy_mixer_out", tuple(x.shape), torch.float32)
            yn = ctx.scratch("toy_mixer_out_normed", tuple(x.shape), torch.float32)
            self.mixer_norm.forward(x, xn)
            y.zero_()
            self.mixer.forward(ctx, run, xn, y)
            self.post_norm.forward(y, yn)
            x.add_(yn)
            self.feed_forward_norm.forward(x, xn)
            self.feed_forward.forward(ctx, xn, x)

    @register_position_encoding("toy_sqrt_angles")
    class SqrtAngles:
        applies = "qk_before_store"
        interleaved = False

        def __init__(self, params, weights, build):
            half = params["head_dim"] // 2
            pos = np.sqrt(np.arange(build.max_position, dtype=np.float64))[:, None]
            ang = pos * (np.arange(half, dtype=np.float64)[None] + 1.0) * params["step"]
            self.cos = torch.from_numpy(np.cos(ang).astype(np.float32)).to(build.device).contiguous()
            self.sin = torch.from_numpy(np.sin(ang).astype(np.float32)).to(build.device).contiguous()

    @register_feed_forward("toy_best_of_three")
    class BestOfThree:
        def __init__(self, params, weights, build):
            self.D, self.I, self.E = params["hidden_size"], params["intermediate_size"], 3
            dev = build.device
            self.router = weights["router"].to(device=dev, dtype=torch.float32)          # [E, D]
            self.gate_up = weights["gate_up"].to(device=dev, dtype=torch.float32)        # [E, 2I, D]
            self.down = weights["down"].to(device=dev, dtype=torch.float32)              # [E, D, I]

        def forward(self, ctx, xn, x):
            xf = xn.float()
            best = (xf @ self.router.T).argmax(dim=-1)                                   # routing in 32-bit
            for e in range(self.E):
                rows = (best == e).nonzero(as_tuple=True)[0]
                if rows.numel():
                    gu = xf[rows] @ self.gate_up[e].T
                    g, u = gu[:, :self.I], gu[:, self.I:]
                    x[rows] += (g * torch.sigmoid(g) * u) @ self.down[e].T

    class Toy2Config:
        architecture = "ToyRoutedForCausalLM"

        def __init__(self, j):
            self.hidden, self.layers, self.vocab, self.max_pos, self.step = j["hidden"], j["layers"], j["vocab"], j["max_pos"], j["step"]

        @classmethod
        def from_json(cls, j):
            return cls(j)

        def model_spec(self):
            D = self.hidden
            norm = PartSpec("rmsnorm", {"size": D, "eps": 3e-6})
            pos = PartSpec("toy_sqrt_angles", {"head_dim": 16, "step": self.step})
            att = PartSpec("attention", {"hidden_size": D, "num_heads": 3, "num_kv_heads": 3, "head_dim": 16,
                                         "scale": 0.3, "window": None, "position": pos})
            routed = PartSpec("toy_best_of_three", {"hidden_size": D, "intermediate_size": 24})
            dense = PartSpec("swiglu", {"hidden_size": D, "intermediate_size": 40})
            # odd layers: the dense feed-forward and the arrangement with a norm after the mixer
            layers = [LayerSpec(att, routed, norm, norm) if i % 2 == 0 else
                      LayerSpec(att, dense, norm, norm, block="toy_post_norm", extra={"post_mixer_norm": norm})
                      for i in range(self.layers)]
            return ModelSpec("ToyRoutedForCausalLM", D, self.vocab, self.max_pos, layers,
                             [ScheduleEntry(i) for i in range(self.layers)], norm, True,
                             logit_transform=PartSpec("toy_halve", {"factor": 0.5}))

    def plan(cfg):
        D = cfg.hidden
        rules = [TensorRule("emb", (cfg.vocab, D)), TensorRule("norm", (D,), "vector")]
        for i in range(cfg.layers):
            rules += [TensorRule(f"l{i}.n1", (D,), "vector"), TensorRule(f"l{i}.n2", (D,), "vector"),
                      TensorRule(f"l{i}.qkv", (144, D)), TensorRule(f"l{i}.o", (D, 48))]
            if i % 2 == 0:
                rules += [TensorRule(f"l{i}.router", (3, D))] + [TensorRule(f"l{i}.e{e}.gu", (48, D)) for e in range(3)] + \
                         [TensorRule(f"l{i}.e{e}.down", (D, 24)) for e in range(3)]
            else:
                rules += [TensorRule(f"l{i}.gu", (80, D)), TensorRule(f"l{i}.down", (D, 40)), TensorRule(f"l{i}.n3", (D,), "vector")]

        def assemble(t):
            out = {"embedding.weight": t["emb"], "final_norm.weight": t["norm"], "head.weight": t["emb"]}
            for i in range(cfg.layers):
                q = f"layers.{i}."
                out[q + "mixer_norm.weight"], out[q + "feed_forward_norm.weight"] = t[f"l{i}.n1"], t[f"l{i}.n2"]
                out[q + "mixer.w_qkv"], out[q + "mixer.w_o"] = t[f"l{i}.qkv"], t[f"l{i}.o"]
                if i % 2 == 0:
                    out[q + "feed_forward.router"] = t[f"l{i}.router"]
                    out[q + "feed_forward.gate_up"] = torch.stack([t[f"l{i}.e{e}.gu"] for e in range(3)])
                    out[q + "feed_forward.down"] = torch.stack([t[f"l{i}.e{e}.down"] for e in range(3)])
                else:
                    out[q + "feed_forward.w_gate_up"], out[q + "feed_forward.w_down"] = t[f"l{i}.gu"], t[f"l{i}.down"]
                    out[q + "post_mixer_norm.weight"] = t[f"l{i}.n3"]
            return out
        return WeightPlan(rules, [], assemble)

    register_architecture(Architecture("ToyRoutedForCausalLM", ("toy_routed",), Toy2Config, plan))


def _toy_routed_plain(w, cfg, toks):
    D, T = cfg["hidden"], len(toks)
    x = w["emb"][torch.tensor(toks)].float()
    ang = np.sqrt(np.arange(T, dtype=np.float64))[:, None] * (np.arange(8, dtype=np.float64)[None] + 1.0) * cfg["step"]
    c, s_ = torch.from_numpy(np.cos(ang).astype(np.float32))[:, None], torch.from_numpy(np.sin(ang).astype(np.float32))[:, None]

    def rot(v):                                             # half-split pairs (k, k + 8)
        a, b = v[..., :8], v[..., 8:]
        return torch.cat([a * c - b * s_, a * s_ + b * c], dim=-1)
    routes = []
    for i in range(cfg["layers"]):
        xn = pm.plain_rmsnorm(x, w[f"l{i}.n1"], 3e-6)
        qkv = xn @ w[f"l{i}.qkv"].T
        q, k, v = rot(qkv[:, :48].reshape(T, 3, 16)), rot(qkv[:, 48:96].reshape(T, 3, 16)), qkv[:, 96:].reshape(T, 3, 16)
        y = pm.plain_attention(q, k, v, 0.3).reshape(T, 48) @ w[f"l{i}.o"].T
        x = x + (y if i % 2 == 0 else pm.plain_rmsnorm(y, w[f"l{i}.n3"], 3e-6))
        xn = pm.plain_rmsnorm(x, w[f"l{i}.n2"], 3e-6)
        if i % 2 == 0:
            best = (xn @ w[f"l{i}.router"].T).argmax(dim=-1)
            routes.append(best)
            y = torch.zeros_like(x)
            for t in range(T):
                e = int(best[t])
                gu = xn[t] @ w[f"l{i}.e{e}.gu"].T
                y[t] = pm.plain_swiglu(gu[None, :24], gu[None, 24:])[0] @ w[f"l{i}.e{e}.down"].T
            x = x + y
        else:
            gu = xn @ w[f"l{i}.gu"].T
            x = x + pm.plain_swiglu(gu[:, :40], gu[:, 40:]) @ w[f"l{i}.down"].T
    return (0.5 * (pm.plain_rmsnorm(x, w["norm"], 3e-6) @ w["emb"].T)).numpy(), routes


def test_toy_architecture_with_a_routed_feed_forward_and_its_own_position_encoding(tmp_path):
    _register_toy_routed()
    from geneinfer_b200.engine.loading import load_model
    from geneinfer_b200.engine.step import StepEngine
    from geneinfer_b200.weights import write_random_model
    cfg = {"architectures": ["ToyRoutedForCausalLM"], "model_type": "toy_routed", "hidden": 40, "layers": 3, "vocab": 70,
           "max_pos": 80, "step": 0.37}
    d = write_random_model(cfg, 5, str(tmp_path / "toy_routed"), "float32", std=0.2, norm_std=0.1)
    model = load_model(d, dtype="float32")
    reqs = {f"t{i}": tc.random_tokens(n, 70, 300 + i) for i, n in enumerate([40, 80, 9, 55])}
    w = pm.read_safetensors_f32(os.path.join(d, "model.safetensors"))
    plain, used = {}, set()
    for rid, toks in reqs.items():
        plain[rid], routes = _toy_routed_plain(w, cfg, toks)
        used |= {int(e) for r in routes for e in r}
    assert used == {0, 1, 2}, "the test's tokens do not reach every expert"
    for steps in (tt.trace_whole(reqs), tt.trace_portions(reqs), tt.trace_mixed(reqs, seed=6, tail=8)):
        engine = StepEngine(model, page_size=8, n_pages=4 * 10, max_requests=4, max_step_tokens=128)
        got = tt.run_in_process(engine, steps)
        tt.compare(got, plain, 5e-5, "toy routed model")
        engine.cache.check_invariants()
        assert all(g.pool.free_count == g.pool.n_pages for g in engine.cache.groups)
