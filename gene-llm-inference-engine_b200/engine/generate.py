"""The Python entry point: an engine that takes token ids in and gives token ids out.

The interface follows the reference's C++ ``Engine`` (src/runtime/engine.h:73-94): ``submit``,
``step``, ``run_until_idle``, ``idle``, ``running``, ``waiting``, ``result``, ``stats``,
``cached_blocks`` and ``clear_prefix_cache``, plus ``generate`` for the common case of a list of
prompts. Tokenizers are out of scope: prompts and results are lists of token ids, and the end of a
text is a set of stop ids.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from ..sampling.device import DeviceSampler
from ..sampling.params import SamplingParams
from .loading import load_model
from .scheduler import GenerationRequest, RequestResult, Scheduler, SchedulerConfig, SchedulerStats
from .step import StepEngine


class Engine:
    def __init__(self, model_dir: str, dtype: str = "bfloat16", device: str = "cuda:0",
                 max_seq_len: Optional[int] = None, page_size: int = 16, kv_pages: Optional[int] = None,
                 max_running: int = 8, step_tokens: int = 2048, prefill_chunk: int = 0, prefix_cache: bool = True,
                 decode_weight_copy: bool = True, nvtx: bool = False, debug_checks: bool = False):
        """``model_dir``: folder with config.json and model.safetensors. ``dtype``: "bfloat16"
        (serving kernels) or "float32" (everything in true 32-bit). ``max_seq_len`` lowers the
        context length. ``kv_pages``: pages of ``page_size`` positions in the pool (default: room
        for ``max_running`` full contexts, within 80 % of the free device memory).
        ``decode_weight_copy`` (bfloat16): a second copy of the matrices laid out for decode steps, which
        then stream the weights faster; False saves that memory. ``nvtx`` wraps steps, layers and the head in NVTX
        ranges; ``debug_checks`` validates every step's descriptor (positions, page ids) on the host before launch."""
        self.model = load_model(model_dir, dtype=dtype, device=device, max_position=max_seq_len,
                                weight_tiles=decode_weight_copy)
        context = self.model.max_position
        if kv_pages is None:
            per_request = (context + page_size - 1) // page_size
            kv_pages = max_running * per_request
            elt = 4 if self.model.dtype is torch.float32 else 2
            page_bytes = 0
            by_key = {}
            for layer, need in self.model.cache_needs().items():
                by_key.setdefault(need.group_key, []).append(need)
            for needs in by_key.values():
                page_bytes = max(page_bytes, len(needs) * 2 * needs[0].num_kv_heads * page_size * needs[0].head_dim * elt)
            free, _ = torch.cuda.mem_get_info(torch.device(device))
            if page_bytes:
                kv_pages = max(per_request, min(kv_pages, int(0.8 * free) // max(1, page_bytes * len(by_key))))
        step_tokens = max(1, min(step_tokens, max_running * context))
        self.steps = StepEngine(self.model, page_size=page_size, n_pages=kv_pages, max_requests=max_running,
                                max_step_tokens=step_tokens, max_logit_rows=max_running, nvtx=nvtx,
                                debug_checks=debug_checks)
        self.sampler = DeviceSampler(self.model.vocab_size, self.model.device, ids=self.steps.feedback)
        self.scheduler = Scheduler(self.steps, self.sampler.sample,
                                   SchedulerConfig(max_running, step_tokens, prefill_chunk, prefix_cache),
                                   sample_async=self.sampler.sample_async)

    # ------------------------------------------------------------------ the reference's Engine interface
    def submit(self, prompt: Sequence[int], max_positions: int = 0, sampling: Optional[SamplingParams] = None,
               stop_ids: Sequence[int] = (), on_token=None) -> int:
        return self.scheduler.submit(GenerationRequest(list(prompt), max_positions, sampling or SamplingParams(),
                                                       tuple(stop_ids), on_token))

    def step(self) -> bool:
        return self.scheduler.step()

    def run_until_idle(self) -> None:
        self.scheduler.run_until_idle()

    def idle(self) -> bool:
        return self.scheduler.idle()

    def running(self) -> int:
        return len(self.scheduler.running)

    def waiting(self) -> int:
        return len(self.scheduler.waiting)

    def result(self, request_id: int) -> RequestResult:
        return self.scheduler.result(request_id)

    def forget(self, request_id: int) -> None:
        """Drops the kept tokens and result of a finished request (``generate`` does so for its own)."""
        self.scheduler.forget(request_id)

    @property
    def stats(self) -> SchedulerStats:
        return self.scheduler.stats

    def cached_blocks(self) -> int:
        return self.scheduler.prefix.entries if self.scheduler.prefix else 0

    def clear_prefix_cache(self) -> None:
        if self.scheduler.prefix:
            self.scheduler.prefix.clear()

    # ------------------------------------------------------------------ convenience
    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int = 16, temperature: float = 0.0,
                 top_k: int = 0, top_p: float = 1.0, seed: int = 1, stop_ids: Sequence[int] = ()) -> List[List[int]]:
        """Generates up to ``max_new_tokens`` for every prompt (all requests run together) and
        returns the generated token ids. Request i samples with seed ``seed + i``."""
        if max_new_tokens <= 0:
            return [[] for _ in prompts]
        ids = []
        for i, p in enumerate(prompts):
            params = SamplingParams(temperature, top_k, top_p, seed + i)
            # the token sampled at the last fed position is kept but not fed: positions = prompt + new - 1
            ids.append(self.submit(p, len(p) + max_new_tokens - 1, params, stop_ids))
        self.run_until_idle()
        out = []
        for i in ids:
            r = self.result(i)
            if r.error:
                raise RuntimeError(f"request {i}: {r.error}")
            out.append(list(r.generated_tokens))
            self.forget(i)
        return out
