#!/usr/bin/env python3
"""Makes the golden logits under tests/golden/ with the reference's own C++ model on the CPU.

It writes the two sharp tiny models with this repository's random-weights writer, builds the
reference's ``gi_forward`` with cmake (no GPU needed), feeds it a fixed token sequence position by
position and stores the logits of every position as ``<name>.logits.npy`` beside a ``<name>.json``
that records configuration, weight arguments and tokens. tests/test_plain_model.py rebuilds the
same model folder from that record and compares the plain implementation with these logits.

    python tests/golden/make_golden.py --reference /path/to/gene-LLM-Inference-Engine
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import tiny_configs as tc  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project")
    args = ap.parse_args()
    work = tempfile.mkdtemp(prefix="golden_")
    build = os.path.join(work, "build")
    subprocess.run(["cmake", "-S", args.reference, "-B", build, "-G", "Ninja", "-DCMAKE_BUILD_TYPE=Release"],
                   check=True, stdout=subprocess.DEVNULL)
    subprocess.run(["cmake", "--build", build, "--target", "gi_forward"], check=True, stdout=subprocess.DEVNULL)
    cases = [("tiny_a", tc.TINY_A, tc.SHARP_A, 48, 5), ("tiny_b", tc.TINY_B, tc.SHARP_B, 100, 6)]
    for name, config, weights, n_tokens, seed in cases:
        model_dir = tc.make_model_dir(config, weights, os.path.join(work, name))
        tokens = tc.random_tokens(n_tokens, config["vocab_size"], seed)
        out = os.path.join(work, name + "_out")
        env = dict(os.environ, GI_ISA="scalar", GI_DEVICE="cpu")
        subprocess.run([os.path.join(build, "gi_forward"), model_dir, out, *map(str, tokens)], check=True, env=env)
        logits = np.fromfile(os.path.join(out, "logits.f32"), dtype="<f4").reshape(n_tokens, config["vocab_size"])
        np.save(os.path.join(HERE, name + ".logits.npy"), logits)
        with open(os.path.join(HERE, name + ".json"), "w") as f:
            json.dump({"config": config, "weights": weights, "tokens": tokens,
                       "made_by": "reference gi_forward, GI_ISA=scalar, CPU"}, f, indent=1)
        print(name, logits.shape, float(np.abs(logits).max()))


if __name__ == "__main__":
    main()
