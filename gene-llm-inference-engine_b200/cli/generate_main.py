"""gi_generate: generation from the command line, in the manner of the reference's tool of the same
name (tools/generate_main.cpp:9-25): the same option names with the same meanings where they
apply, statistics on stderr, exit code 2 for usage errors and 1 for runtime errors.

Tokenizers are out of scope here, so the prompt is given as token ids (``--prompt-ids`` or
``--prompt-ids-file``) and the generated ids are printed instead of text; ``--prompt TEXT`` is
refused with a message that says so.
"""
from __future__ import annotations

import sys
import time
from typing import List, Optional

USAGE = (
    "usage: gi_generate --model DIR (--prompt-ids \"1 2 3\" | --prompt-ids-file FILE) [--steps N] [--max-seq-len N]\n"
    "                   [--weights native|f32 | --dtype bf16|fp32] [--device cuda] [--profile] [--temperature F]\n"
    "                   [--top-k N] [--top-p F] [--seed N] [--stop-ids \"2 7\"] [--page-size N] [--kv-pages N]\n"
    "                   [--no-echo] [--quiet] [--dump-tokens FILE] [--random-weights SEED --config FILE]\n"
    "  DIR holds config.json and model.safetensors. --steps is the maximum number of positions including the\n"
    "  prompt (default: the context length). --weights f32 (= --dtype fp32) runs the whole model in true 32-bit.\n"
    "  --random-weights SEED --config FILE first writes such a folder (random bfloat16 weights from the seed, for the\n"
    "  configuration in FILE, a config.json) to DIR, or to a temporary folder when no --model is given.\n")


class UsageError(Exception):
    pass


def _int(flag: str, v: str) -> int:
    try:
        return int(v, 10)
    except ValueError:
        raise UsageError(f"invalid integer for {flag}: {v}") from None


def _float(flag: str, v: str) -> float:
    try:
        return float(v)
    except ValueError:
        raise UsageError(f"invalid number for {flag}: {v}") from None


def _ids(flag: str, text: str) -> List[int]:
    try:
        return [int(t, 10) for t in text.replace(",", " ").split()]
    except ValueError:
        raise UsageError(f"invalid token ids for {flag}") from None


def parse(argv: List[str]) -> dict:
    o = {"model": "", "prompt_ids": None, "steps": 0, "max_seq_len": 0, "weights": "native", "device": "cuda",
         "profile": False, "temperature": 0.8, "top_k": 0, "top_p": 0.9, "seed": None, "stop_ids": [],
         "page_size": 16, "kv_pages": None, "echo": True, "quiet": False, "dump_tokens": "", "random_weights": None,
         "config": "", "help": False}
    i = 0
    while i < len(argv):
        flag = argv[i]

        def value() -> str:
            nonlocal i
            if i + 1 >= len(argv):
                raise UsageError(f"missing value for {flag}")
            i += 1
            return argv[i]

        if flag == "--model": o["model"] = value()
        elif flag == "--prompt-ids": o["prompt_ids"] = _ids(flag, value())
        elif flag == "--prompt-ids-file":
            path = value()
            try:
                with open(path) as f:
                    o["prompt_ids"] = _ids(flag, f.read())
            except OSError as e:
                raise UsageError(f"cannot read {path}: {e}") from None
        elif flag == "--prompt":
            value()
            raise UsageError("--prompt TEXT needs a tokenizer, which this engine does not have: give --prompt-ids")
        elif flag in ("--tokenizer", "--threads"):
            value()          # accepted for compatibility; there is no tokenizer and no CPU thread pool here
        elif flag == "--bos": pass
        elif flag == "--steps": o["steps"] = _int(flag, value())
        elif flag == "--max-seq-len": o["max_seq_len"] = _int(flag, value())
        elif flag == "--weights": o["weights"] = value()
        elif flag == "--dtype":
            name = value().lower()
            if name not in ("bf16", "bfloat16", "fp32", "f32", "float32"):
                raise UsageError("--dtype must be bf16 or fp32")
            o["weights"] = "native" if name in ("bf16", "bfloat16") else "f32"
        elif flag == "--random-weights": o["random_weights"] = _int(flag, value())
        elif flag == "--config": o["config"] = value()
        elif flag in ("--help", "-h"): o["help"] = True
        elif flag == "--device": o["device"] = value()
        elif flag == "--profile": o["profile"] = True
        elif flag == "--temperature": o["temperature"] = _float(flag, value())
        elif flag == "--top-k": o["top_k"] = _int(flag, value())
        elif flag == "--top-p": o["top_p"] = _float(flag, value())
        elif flag == "--seed": o["seed"] = _int(flag, value())
        elif flag == "--stop-ids": o["stop_ids"] = _ids(flag, value())
        elif flag == "--page-size": o["page_size"] = _int(flag, value())
        elif flag == "--kv-pages": o["kv_pages"] = _int(flag, value())
        elif flag == "--no-echo": o["echo"] = False
        elif flag == "--quiet": o["quiet"] = True
        elif flag == "--dump-tokens": o["dump_tokens"] = value()
        else:
            raise UsageError(f"unknown option {flag}")
        i += 1
    if o["help"]:
        return o
    if (o["random_weights"] is None) != (not o["config"]):
        raise UsageError("--random-weights SEED and --config FILE go together")
    if not o["model"] and o["random_weights"] is None:
        raise UsageError("--model is required")
    if not o["prompt_ids"]:
        raise UsageError("--prompt-ids or --prompt-ids-file is required (at least one token id)")
    if o["weights"] not in ("native", "f32"):
        raise UsageError("--weights must be native or f32 (int8 is not built)")
    if not o["device"].startswith("cuda"):
        raise UsageError("--device must be cuda: this engine has no CPU or emulated device")
    if o["seed"] is None:
        o["seed"] = time.time_ns() & ((1 << 63) - 1)
    return o


def main(argv: Optional[List[str]] = None) -> int:
    try:
        o = parse(list(sys.argv[1:] if argv is None else argv))
    except UsageError as e:
        sys.stderr.write(f"error: {e}\n{USAGE}")
        return 2
    if o["help"]:
        sys.stdout.write(USAGE)
        return 0
    scratch_folder = None
    try:
        import torch
        from ..engine.generate import Engine
        from ..sampling.params import SamplingParams
        if o["random_weights"] is not None:
            # the random-weights mode: a model folder from a configuration and a seed, then everything as usual
            import json
            import tempfile
            from ..weights import write_random_model
            try:
                with open(o["config"]) as f:
                    config_json = json.load(f)
            except (OSError, ValueError) as e:
                sys.stderr.write(f"error: cannot read the configuration {o['config']}: {e}\n")
                return 2
            if not o["model"]:
                scratch_folder = tempfile.TemporaryDirectory(prefix="gi_generate_random_")
                o["model"] = scratch_folder.name
            write_random_model(config_json, o["random_weights"], o["model"], "bfloat16")
            if not o["quiet"]:
                sys.stderr.write(f"[random weights] seed {o['random_weights']}, folder {o['model']}\n")
        try:
            params = SamplingParams(o["temperature"], o["top_k"], o["top_p"], o["seed"])
        except ValueError as e:
            sys.stderr.write(f"error: {e}\n")
            return 2
        device = o["device"] if ":" in o["device"] else "cuda:0"
        t0 = time.perf_counter()
        engine = Engine(o["model"], dtype="float32" if o["weights"] == "f32" else "bfloat16", device=device,
                        max_seq_len=o["max_seq_len"] or None, page_size=o["page_size"], kv_pages=o["kv_pages"],
                        max_running=1, prefix_cache=False)
        load_s = time.perf_counter() - t0
        prompt = o["prompt_ids"]
        if o["echo"]:
            sys.stdout.write(" ".join(map(str, prompt)) + " |")
            sys.stdout.flush()

        def on_token(t: int) -> None:
            sys.stdout.write(f" {t}")
            sys.stdout.flush()

        times = {}
        rid = engine.submit(prompt, o["steps"], params, o["stop_ids"], on_token)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        while engine.step():
            if "first" not in times and engine.result(rid).generated_tokens:
                torch.cuda.synchronize()
                times["first"] = time.perf_counter()
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        sys.stdout.write("\n")
        res = engine.result(rid)
        if res.error:
            sys.stderr.write(f"error: {res.error}\n")
            return 1
        if o["dump_tokens"]:
            with open(o["dump_tokens"], "w") as f:
                f.write(" ".join(map(str, prompt)) + "\n" + " ".join(map(str, res.generated_tokens)) + "\n")
        if not o["quiet"]:
            first = times.get("first", t1)
            n_gen = len(res.generated_tokens)
            prefill_s, decode_s = first - t0, t1 - first
            cache_bytes = sum(t.numel() * t.element_size() for t in engine.steps.group_pages)
            sys.stderr.write(
                f"[stats] load {load_s:.2f} s | weights {engine.model.weight_bytes() / 2 ** 20:.0f} MiB, "
                f"cache {cache_bytes / 2 ** 20:.0f} MiB on the device | prompt {len(prompt)} tokens in {prefill_s * 1e3:.1f} ms "
                f"({len(prompt) / max(prefill_s, 1e-9):.1f} tok/s) | generated {n_gen} tokens, "
                f"{max(n_gen - 1, 0)} decode steps in {decode_s * 1e3:.1f} ms "
                f"({max(n_gen - 1, 0) / max(decode_s, 1e-9):.1f} tok/s) | seed {o['seed']} | "
                f"end token: {'yes' if res.stopped_by_end_token else 'no'}\n")
        if o["profile"]:
            from ..engine.profile import profile_report
            sys.stderr.write(profile_report(engine, prompt))
        return 0
    except Exception as e:   # runtime errors: bad model folder, kernels cannot be built, no GPU ...
        sys.stderr.write(f"error: {e}\n")
        return 1
    finally:
        if scratch_folder is not None:
            scratch_folder.cleanup()


if __name__ == "__main__":
    sys.exit(main())
