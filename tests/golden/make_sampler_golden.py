#!/usr/bin/env python3
"""Makes the sampler goldens under tests/golden/ with the reference's own C++ sampler on the CPU.

Builds the reference's ``gi_sampler_check`` with cmake (no GPU needed) and records, for fixed
logits, what its sampler returns: the uniform numbers of its random generator for several seeds
(``rngdump``), the token for given uniform numbers under greedy, temperature, top-k and top-p
settings (``uniform``), and whole draws from its internal generator (``rng``). The result is
``sampler.npz``; tests/test_plain_model.py holds the plain sampler to it token for token.

    python tests/golden/make_sampler_golden.py --reference /path/to/gene-LLM-Inference-Engine
"""
import argparse
import os
import subprocess
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

SEEDS = [0, 1, 7, 123456789, 2 ** 63 + 5]
SETTINGS = [(0.0, 0, 1.0), (0.8, 0, 1.0), (1.0, 5, 1.0), (0.7, 0, 0.9), (1.3, 20, 0.8), (0.25, 3, 0.5), (2.0, 0, 0.3)]
VOCABS = [50, 384]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project")
    args = ap.parse_args()
    work = tempfile.mkdtemp(prefix="golden_sampler_")
    build = os.path.join(work, "build")
    subprocess.run(["cmake", "-S", args.reference, "-B", build, "-G", "Ninja", "-DCMAKE_BUILD_TYPE=Release"],
                   check=True, stdout=subprocess.DEVNULL)
    subprocess.run(["cmake", "--build", build, "--target", "gi_sampler_check"], check=True, stdout=subprocess.DEVNULL)
    exe = os.path.join(build, "gi_sampler_check")

    def run(argv, stdin=b""):
        return subprocess.run([exe, *map(str, argv)], input=stdin, stdout=subprocess.PIPE, check=True).stdout

    out = {"seeds": np.array([str(s) for s in SEEDS]), "settings": np.array(SETTINGS, dtype=np.float64)}
    out["uniforms"] = np.stack([np.frombuffer(run(["rngdump", s, 24]), dtype="<f4") for s in SEEDS])
    rng = np.random.default_rng(2024)
    us = np.concatenate([np.array([0.0, 1e-7, 0.5, 0.999999, 1.0 - 2.0 ** -24], dtype=np.float32),
                         rng.random(59, dtype=np.float32)])
    out["us"] = us
    for vocab in VOCABS:
        logits = (rng.standard_normal(vocab) * 2.5).astype(np.float32)
        logits[vocab // 3] = logits[vocab // 2] = logits.max() + 0.5          # a tie of the two best: the lowest index wins
        out[f"logits_{vocab}"] = logits
        for k, (t, top_k, top_p) in enumerate(SETTINGS):
            picked = run(["uniform", vocab, t, top_k, top_p, len(us)], logits.tobytes() + us.tobytes())
            out[f"uniform_{vocab}_{k}"] = np.frombuffer(picked, dtype="<i4")
            if t > 0:
                drawn = run(["rng", vocab, t, top_k, top_p, SEEDS[k % len(SEEDS)], 32], logits.tobytes())
                out[f"rng_{vocab}_{k}"] = np.frombuffer(drawn, dtype="<i4")
    np.savez(os.path.join(HERE, "sampler.npz"), **out)
    print("wrote sampler.npz:", len(out), "arrays")


if __name__ == "__main__":
    main()
