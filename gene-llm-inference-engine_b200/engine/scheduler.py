"""The scheduler: admits requests, cuts prompts into portions under a token budget, decodes,
finishes and frees; and decides what happens when pages run out.

Policy of the reference engine (src/runtime/engine.cpp:64-208):
  * requests wait in a FIFO queue and are admitted at the start of a step while fewer than
    ``max_running`` are running; memory is not checked at admission but when the step is built;
  * a step takes decoding requests first (one token each), then prompt portions, oldest request
    first; each portion is limited by the step's token budget, by ``prefill_chunk``, by the
    request's position limit and by the pages that are free (or can be freed from the prefix
    cache), shrinking token by token until it fits;
  * only the row that feeds a request's last known token asks for logits; the sampled token is
    appended and fed in a later step;
  * when nothing fits: the youngest running request is preempted (its pages are given back, it goes
    to the front of the queue and is recomputed later, prompt and generated tokens, with its random
    stream kept so that the result is the same); a request that cannot fit even alone ends with an
    error;
  * a request ends on a sampled stop token (kept as its last generated token) or when its position
    limit is reached; its pages return to the pool at once.

The scheduler drives any backend with ``cache`` (a CacheManager), ``open``, ``close``, ``step`` and
``model`` (``max_position``, ``vocab_size``); tests run it on the CPU with a counting backend.

One step ahead. With a backend whose steps can take a token from the device (``token_feedback``)
and a sampler that answers later (``sample_async``), a step of plain decoding is launched before
the ids of the step before it have reached the host: each request's next token is named by its
place in the sampler's output. The host then reads the earlier step's ids while the device already
runs the next one. What a step computes is the same; only a request that ends on a stop token has
taken part in one step too many, whose row is dropped (its pages go back with the rest). A step is
launched ahead only when the set of running requests cannot change in between: nothing waits for
a free place, every running request has just fed its last known token, none reaches its position
limit, and the pages are free without eviction.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Deque, Dict, List, Optional, Sequence

from ..cache import PrefixCache
from ..sampling.params import RandomStream, SamplingParams
from .step import StepEntry


@dataclass
class SchedulerConfig:
    max_running: int = 8         # requests that hold cache memory and take part in a step at a time
    step_tokens: int = 2048      # token budget of a step
    prefill_chunk: int = 0       # most prompt tokens one request adds to a step; 0 = the step's budget
    prefix_cache: bool = True    # reuse the pages of earlier requests that start with the same tokens


@dataclass
class GenerationRequest:
    prompt: Sequence[int]
    max_positions: int = 0       # prompt + generated tokens at most; 0 or too large = the context length
    sampling: SamplingParams = field(default_factory=SamplingParams)
    stop_ids: Sequence[int] = ()
    on_token: Optional[Callable[[int], None]] = None


@dataclass
class RequestResult:
    id: int
    prompt_tokens: List[int]
    generated_tokens: List[int] = field(default_factory=list)
    finished: bool = False
    stopped_by_end_token: bool = False
    error: str = ""
    preemptions: int = 0
    cached_tokens: int = 0       # positions taken from the prefix cache instead of being computed
    first_step: int = -1
    first_token_step: int = -1
    last_step: int = -1


@dataclass
class SchedulerStats:
    steps: int = 0
    tokens: int = 0
    logits_rows: int = 0
    preemptions: int = 0
    prefix_tokens: int = 0
    prefix_hits: int = 0
    evicted_pages: int = 0
    max_tokens_in_step: int = 0
    max_chunk: int = 0
    max_running_seen: int = 0


class _Job:
    def __init__(self, jid: int, request: GenerationRequest, context: int):
        self.id = jid
        self.request = request
        self.tokens: List[int] = list(request.prompt)
        self.fed = 0                 # tokens[:fed] are in the cache
        self.cached_upto = 0         # tokens[:cached_upto] are indexed in the prefix cache
        self.limit = context if request.max_positions <= 0 else min(request.max_positions, context)
        self.stream = RandomStream(request.sampling.seed)
        self.cache = None            # RequestCache while running
        self.result = RequestResult(jid, list(request.prompt))


class _InFlight:
    """A step that has been launched: who took part, and the ids on their way to the host."""

    def __init__(self, number: int, jobs: List[_Job], takes: List[int], owners: List[_Job], pending):
        self.number = number         # the step's count (stats.steps when it was launched)
        self.jobs = jobs             # requests that fed tokens, in step order
        self.takes = takes           # tokens each fed
        self.owners = owners         # the requests whose last row asked for logits, in row order
        self.pending = pending       # None, a list of ids, or an object with result()


class Scheduler:
    def __init__(self, backend, sample_rows: Callable, config: Optional[SchedulerConfig] = None,
                 sample_async: Optional[Callable] = None):
        """``sample_rows(logits, params, uniforms) -> token ids`` turns the wanted logits rows of a
        step into one token each; ``sample_async`` does the same but returns an object whose
        ``result()`` gives the ids later (it lets a step be launched ahead)."""
        self.backend = backend
        self.sample_rows = sample_rows
        self.sample_async = sample_async
        self.lookahead = sample_async is not None and getattr(backend, "token_feedback", False)
        self._ahead: Optional[_InFlight] = None
        self.cfg = config or SchedulerConfig()
        if self.cfg.max_running < 1:
            raise ValueError("Scheduler: max_running must be >= 1")
        if self.cfg.step_tokens < 1 or self.cfg.prefill_chunk < 0:
            raise ValueError("Scheduler: step_tokens must be >= 1 and prefill_chunk >= 0")
        self.chunk = self.cfg.prefill_chunk or self.cfg.step_tokens
        self.context = backend.model.max_position
        self.vocab = backend.model.vocab_size
        self.jobs: List[_Job] = []
        self.waiting: Deque[_Job] = deque()
        self.running: List[_Job] = []
        self.stats = SchedulerStats()
        cache = backend.cache
        shareable = len(cache.groups) == 1 and not cache.groups[0].need.window and not cache.state_layers
        self.prefix: Optional[PrefixCache] = None
        if self.cfg.prefix_cache and shareable:
            self.prefix = PrefixCache(cache.groups[0].pool, cache.page_size)

    # ------------------------------------------------------------------ requests
    def submit(self, request: GenerationRequest) -> int:
        if len(request.prompt) == 0:
            raise ValueError("submit: prompt has no tokens")
        if len(request.prompt) > self.context:
            raise ValueError(f"submit: prompt of {len(request.prompt)} tokens does not fit in the context length "
                             f"{self.context}")
        for t in request.prompt:
            if not (0 <= int(t) < self.vocab):
                raise ValueError("submit: token id out of range")
        job = _Job(len(self.jobs), request, self.context)
        self.jobs.append(job)
        self.waiting.append(job)
        return job.id

    def result(self, jid: int) -> RequestResult:
        if not (0 <= jid < len(self.jobs)) or self.jobs[jid] is None:
            raise KeyError(f"request {jid} is unknown or was forgotten")
        return self.jobs[jid].result

    def forget(self, jid: int) -> None:
        """Drops what is kept of a finished request (its tokens and result), so that a long-running
        engine does not grow with every request it has served; ids are not handed out again."""
        job = self.jobs[jid] if 0 <= jid < len(self.jobs) else None
        if job is None:
            raise KeyError(f"request {jid} is unknown or was forgotten")
        if not job.result.finished:
            raise RuntimeError(f"request {jid} has not finished")
        self.jobs[jid] = None

    def idle(self) -> bool:
        return not self.waiting and not self.running and self._ahead is None

    # ------------------------------------------------------------------ life of a request
    def _admit(self) -> None:
        while self.waiting and len(self.running) < self.cfg.max_running:
            job = self.waiting.popleft()
            job.cache = self.backend.open(("job", job.id))
            job.fed = job.cached_upto = 0
            if self.prefix is not None:
                # at least one token must still be fed (it gives the logits) and the limit must leave a row
                usable = min(len(job.tokens) - 1, job.limit - 1)
                pages = self.prefix.match(job.tokens, usable) if usable > 0 else []
                if pages:
                    self.backend.cache.adopt(job.cache, 0, pages)
                    job.fed = job.cached_upto = len(pages) * self.backend.cache.page_size
                    job.result.cached_tokens += job.fed
                    self.stats.prefix_tokens += job.fed
                    self.stats.prefix_hits += 1
            self.running.append(job)
        self.stats.max_running_seen = max(self.stats.max_running_seen, len(self.running))

    def _index_new_pages(self, job: _Job) -> None:
        if self.prefix is None:
            return
        ps = self.backend.cache.page_size
        if job.fed // ps <= job.cached_upto // ps:
            return
        self.prefix.insert(job.tokens, job.fed, job.cache.tables[0][:job.cache.n_pages[0]])
        job.cached_upto = job.fed

    def _finish(self, job: _Job, error: str = "", step: int = -1) -> None:
        job.result.finished = True
        job.result.error = error
        job.result.last_step = self.stats.steps if step < 0 else step
        self.backend.close(("job", job.id))
        job.cache = None
        self.running.remove(job)

    def _preempt_youngest(self) -> None:
        job = self.running.pop()
        self.backend.close(("job", job.id))
        job.cache = None
        job.fed = 0
        job.result.preemptions += 1
        self.stats.preemptions += 1
        self.waiting.appendleft(job)

    # ------------------------------------------------------------------ one step
    def plan(self):
        """Decides the next step: returns (takes per running job, pages needed). Pure bookkeeping."""
        cache = self.backend.cache
        free = cache.free_pages() + (self.prefix.evictable() if self.prefix else 0)
        needed = 0
        budget = self.cfg.step_tokens
        takes = [0] * len(self.running)
        for phase in (0, 1):
            for k, job in enumerate(self.running):
                pending = len(job.tokens) - job.fed
                decoding = pending == 1
                if (phase == 0) != decoding:
                    continue
                take = min(pending, job.limit - job.fed, budget, 1 if phase == 0 else self.chunk)
                while take > 0 and cache.pages_needed(job.cache, take) > free:
                    take -= 1
                if take <= 0:
                    continue
                n = cache.pages_needed(job.cache, take)
                free -= n
                needed += n
                budget -= take
                takes[k] = take
        return takes, needed

    def step(self) -> bool:
        """Completes one step of the model. False (and nothing done) when no request waits or runs."""
        cur = self._ahead
        self._ahead = None
        if cur is None:
            cur = self._launch()
            if cur is None:
                return False
        if cur.jobs and self.lookahead:
            self._ahead = self._launch_ahead(cur)
        self._complete(cur)
        return True

    def _launch(self) -> Optional[_InFlight]:
        """Plans and launches a step from what the host knows. None when nothing waits or runs."""
        self._admit()
        if not self.running:
            return None
        cache = self.backend.cache
        while True:
            takes, needed = self.plan()
            if any(takes):
                break
            if len(self.running) == 1:
                self._finish(self.running[0], "the KV pool is too small for this request")
                return _InFlight(self.stats.steps, [], [], [], None)
            self._preempt_youngest()
        if self.prefix is not None and needed > cache.free_pages():
            self.stats.evicted_pages += self.prefix.evict(needed - cache.free_pages())

        entries, owners, jobs, fed_takes = [], [], [], []
        for job, take in zip(self.running, takes):
            if take == 0:
                continue
            last = job.fed + take == len(job.tokens)
            entries.append(StepEntry(("job", job.id), job.tokens[job.fed:job.fed + take], [take - 1] if last else []))
            jobs.append(job)
            fed_takes.append(take)
            if last:
                owners.append(job)
        return self._run(entries, jobs, fed_takes, owners)

    def _run(self, entries, jobs, takes, owners) -> _InFlight:
        logits = self.backend.step(entries)
        self.stats.steps += 1
        n_tokens = sum(takes)
        self.stats.tokens += n_tokens
        self.stats.max_tokens_in_step = max(self.stats.max_tokens_in_step, n_tokens)
        self.stats.max_chunk = max(self.stats.max_chunk, max(takes))
        pending = None
        if owners:
            params = [j.request.sampling for j in owners]
            uniforms = [0.0 if p.greedy else j.stream.next_uniform() for j, p in zip(owners, params)]
            pending = (self.sample_async or self.sample_rows)(logits, params, uniforms)
            self.stats.logits_rows += len(owners)
        return _InFlight(self.stats.steps, jobs, takes, owners, pending)

    def _launch_ahead(self, cur: _InFlight) -> Optional[_InFlight]:
        """Launches the step after ``cur`` from the ids ``cur`` leaves on the device, if nothing the
        host does not know yet can change who runs in it."""
        if self.waiting or len(cur.owners) != len(self.running) or len(cur.owners) != len(cur.jobs):
            return None                                   # a request could be admitted, or some still feed their prompt
        cache = self.backend.cache
        needed = 0
        for job, take in zip(cur.jobs, cur.takes):
            if job.fed + take + 1 > job.limit:
                return None                               # it ends with this step: the set of requests changes
            needed += cache.pages_needed(job.cache, 1)
        if needed > cache.free_pages():
            return None                                   # eviction or preemption: decided with all ids known
        entries = [StepEntry(("job", job.id), [-(k + 1)], [0]) for k, job in enumerate(cur.owners)]
        return self._run(entries, list(cur.owners), [1] * len(entries), list(cur.owners))

    def _complete(self, cur: _InFlight) -> None:
        """Takes a launched step's ids and does the bookkeeping that follows them."""
        sampled: Dict[int, int] = {}
        if cur.owners:
            ids = cur.pending.result() if hasattr(cur.pending, "result") else cur.pending
            sampled = {j.id: int(t) for j, t in zip(cur.owners, ids)}
        done = []
        for job, take in zip(cur.jobs, cur.takes):
            if job.result.finished:
                continue                                  # it ended on a stop token one step earlier: this row is dropped
            if job.result.first_step < 0:
                job.result.first_step = cur.number
            job.fed += take
            self._index_new_pages(job)
            if job.id in sampled:
                nxt = sampled[job.id]
                job.result.generated_tokens.append(nxt)
                job.tokens.append(nxt)
                if job.result.first_token_step < 0:
                    job.result.first_token_step = cur.number
                if job.request.on_token:
                    job.request.on_token(nxt)
                if nxt in job.request.stop_ids:
                    job.result.stopped_by_end_token = True
                    done.append(job)
                    continue
            if job.fed >= job.limit:
                done.append(job)
        for job in done:
            self._finish(job, step=cur.number)

    def run_until_idle(self) -> None:
        while self.step():
            pass
