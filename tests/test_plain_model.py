"""The plain implementation against the reference's own C++ model (golden logits made on the CPU by
tests/golden/make_golden.py), and the plain sampler against hand-checked cases."""
import json
import os

import numpy as np
import pytest

import plain_model as pm
import tiny_configs as tc

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def rel_err(a, b):
    """The reference's own measure: max|a-b| / max(1, max|b|) (tests/verify_forward.py:72-77)."""
    return float(np.abs(a - b).max() / max(1.0, np.abs(b).max()))


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_plain_forward_matches_reference_golden(name, tmp_path):
    with open(os.path.join(GOLDEN, name + ".json")) as f:
        rec = json.load(f)
    golden = np.load(os.path.join(GOLDEN, name + ".logits.npy"))
    model_dir = tc.make_model_dir(rec["config"], rec["weights"], str(tmp_path / name))
    w, cfg = pm.load_plain(model_dir)
    logits = pm.plain_forward(w, cfg, rec["tokens"]).numpy()
    assert logits.shape == golden.shape
    assert rel_err(logits, golden) < 1e-4
    assert (logits.argmax(-1) == golden.argmax(-1)).mean() > 0.98


def test_plain_rope_table_regimes():
    # tiny B's head size 32 with original length 64 hits all three regimes of the llama3 scaling
    cos, sin = pm.plain_rope_table([0, 1, 77], 32, 500000.0, (32.0, 1.0, 4.0, 64.0))
    assert cos.shape == (3, 16)
    assert np.allclose(cos[0].numpy(), 1.0) and np.allclose(sin[0].numpy(), 0.0)
    plain, plain_sin = pm.plain_rope_table([77], 32, 500000.0, None)
    assert np.allclose(cos[2, 0], plain[0, 0])           # fastest pair: unchanged
    assert not np.isclose(float(sin[2, 15]), float(plain_sin[0, 15]), rtol=0.5), "the slowest pair must differ from the unscaled table"
    freq_last = 1.0 / 500000.0 ** (30 / 32)
    assert np.isclose(float(cos[2, 15]), np.cos(77 * freq_last / 32.0), atol=1e-7)   # slowest pair: / factor


def test_plain_attention_is_causal_and_grouped():
    import torch
    torch.manual_seed(0)
    q, k, v = torch.randn(5, 4, 16), torch.randn(5, 2, 16), torch.randn(5, 2, 16)
    out = pm.plain_attention(q, k, v, 0.25)
    k2, v2 = k.clone(), v.clone()
    k2[4], v2[4] = 9.0, -9.0                       # the future must not matter
    out2 = pm.plain_attention(q, k2, v2, 0.25)
    assert torch.equal(out[:4], out2[:4])
    assert torch.allclose(out[0, 0], v[0, 0]) and torch.allclose(out[0, 3], v[0, 1])   # heads 2,3 read kv head 1
    w = pm.plain_attention(q, k, v, 0.25, window=2)
    assert torch.allclose(w[1], out[1]) and not torch.allclose(w[4], out[4])


def test_plain_sampler_stream_and_rules():
    s = pm.PlainSampler(temperature=0.0)
    assert s.sample(np.array([1.0, 3.0, 3.0, 2.0])) == 1           # lowest index on ties
    a, b = pm.PlainSampler(seed=7), pm.PlainSampler(seed=7)
    assert [a.next_uniform() for _ in range(4)] == [b.next_uniform() for _ in range(4)]
    assert all(0.0 <= u < 1.0 for u in (a.next_uniform() for _ in range(100)))
    logits = np.log(np.array([0.5, 0.3, 0.15, 0.05], dtype=np.float32))
    t = pm.PlainSampler(temperature=1.0)
    assert [t.sample(logits, u) for u in (0.0, 0.49, 0.51, 0.79, 0.81, 0.96)] == [0, 0, 1, 1, 2, 3]
    k2 = pm.PlainSampler(temperature=1.0, top_k=2)
    assert [k2.sample(logits, u) for u in (0.0, 0.6, 0.64, 0.99)] == [0, 0, 1, 1]
    p = pm.PlainSampler(temperature=1.0, top_p=0.7)                # keeps 0.5 + 0.3
    assert [p.sample(logits, u) for u in (0.0, 0.62, 0.63, 0.99)] == [0, 0, 1, 1]
    assert pm.PlainSampler(temperature=1.0, top_k=1).sample(logits, 0.99) == 0
    assert pm.PlainSampler(temperature=1.0, top_p=1e-6).sample(logits, 0.99) == 0


def test_plain_sampler_matches_the_reference_sampler_token_for_token():
    """tests/golden/sampler.npz holds what the reference's own sampler (its gi_sampler_check tool, built
    on the CPU by tests/golden/make_sampler_golden.py) returns for fixed logits: its generator's
    uniform numbers, its picks for given uniform numbers under every kind of setting (a tie of the
    two best logits included), and whole draws from its generator."""
    g = np.load(os.path.join(GOLDEN, "sampler.npz"))
    seeds = [int(s) for s in g["seeds"]]
    for seed, want in zip(seeds, g["uniforms"]):
        s = pm.PlainSampler(0.8, 0, 1.0, seed=seed)
        got = np.array([s.next_uniform() for _ in range(len(want))], dtype=np.float32)
        assert np.array_equal(got, want), f"seed {seed}: the generator's numbers differ"
    us = g["us"]
    checked = 0
    for vocab in (50, 384):
        logits = g[f"logits_{vocab}"]
        for k, (t, top_k, top_p) in enumerate(g["settings"]):
            s = pm.PlainSampler(float(t), int(top_k), float(top_p))
            got = [s.sample(logits, u) for u in us]
            want = g[f"uniform_{vocab}_{k}"].tolist()
            assert got == want, f"vocab {vocab}, temperature {t}, top-k {int(top_k)}, top-p {top_p}: picks differ"
            checked += len(got)
            if t > 0:
                s = pm.PlainSampler(float(t), int(top_k), float(top_p), seed=seeds[k % len(seeds)])
                drawn = [s.sample(logits) for _ in range(32)]
                assert drawn == g[f"rng_{vocab}_{k}"].tolist(), f"vocab {vocab}, setting {k}: draws from the generator differ"
    assert checked == 2 * 7 * 64
