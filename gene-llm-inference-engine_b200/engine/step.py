"""The step function: one batch of (request, its next tokens) through the model, from the cache.

A step takes any mix of prompt portions and single decoded tokens, cut anywhere. It runs only the
tokens it is given, as one batch, against what earlier steps left in the cache, and returns the
logits at the wanted places. Position of a token = the request's cached length + its index among
the request's tokens of this step (src/model/transformer.cpp:483-518). A step is all or nothing:
pages for every entry are reserved first, and if they run out everything is given back and
``OutOfPages`` is raised with no state changed.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache import CacheManager, OutOfPages, RequestCache
from ..ops import kernels
from ..parts import DecoderModel

_STATE_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "int32": torch.int32}


@dataclass
class StepEntry:
    """The next tokens of one request and the places among them whose logits are wanted. A token
    given as -(k + 1) is taken on the device from place k of the engine's ``feedback`` buffer, where
    a sampler left the id it drew from the step before (the host need not know it yet)."""
    key: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=list)


@dataclass
class Segment:
    """Where one request's tokens lie in the step's rows (host copy, for parts that need it)."""
    key: Hashable
    start: int          # first row
    length: int         # number of rows
    first_position: int
    state_slot: int
    fresh_state: bool


class StepContext:
    """What the parts see of a step: row arrays on the device, caches, state and scratch."""

    def __init__(self, engine: "StepEngine", n_tokens: int, n_requests: int, n_logit_rows: int,
                 segments: List[Segment], views: Dict[str, torch.Tensor]):
        self._engine = engine
        self.n_tokens = n_tokens
        self.n_requests = n_requests
        self.n_logit_rows = n_logit_rows
        self.segments = segments
        self.page_size = engine.page_size
        self.max_requests = engine.max_requests
        self.max_logit_rows = engine.max_logit_rows
        self.compute_dtype = engine.model.dtype
        self.tokens = views["tokens"]
        self.feedback = engine.feedback          # sampled ids of the step before, for tokens given as -(k + 1)
        self.positions = views["positions"]
        self.row_req = views["row_req"]
        self.logit_rows = views["logit_rows"]
        self.state_slots = views["state_slots"]
        self.seg_start = views["seg_start"]
        self.seg_len = views["seg_len"]
        self._tables = views["tables"]
        self._cache: Dict = {}
        self.all_single = all(s.length == 1 for s in segments)
        self.max_context = max((s.first_position + s.length for s in segments), default=0)
        # longest context among requests that bring a single token, rounded up to 1024 positions
        # (to 256 below that: one chunk of the decode attention, which then needs no merge kernel):
        # the grid of the decode attention depends on it, and a coarse value keeps the set of
        # distinct step shapes (and of captured graphs) small; chunks beyond a row's own
        # position exit at once
        longest = max((s.first_position + 1 for s in segments if s.length == 1), default=0)
        rounded = 256 if longest <= 256 else (longest + 1023) // 1024 * 1024
        self.longest_single = min(engine.model.max_position, rounded)

    def pages(self, layer: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """(keys, values) of a layer, each [pages, Hkv, page_size, head_dim]."""
        return self._engine.layer_pages[layer]

    def block_tables(self, layer: int) -> torch.Tensor:
        """Block tables [requests of this step, stride] of the group the layer belongs to."""
        return self._tables[self._engine.cache.group_of_layer[layer]]

    def state(self, layer: int) -> torch.Tensor:
        """State of a layer for every slot: [slots, *shape]; row ``state_slot`` is a request's."""
        return self._engine.layer_state[layer]

    def scratch(self, name: str, shape: Tuple[int, ...], dtype: torch.dtype, capacity: Optional[int] = None) -> torch.Tensor:
        return self._engine.scratch(name, shape, dtype, capacity)

    def recorded(self, owner, key: Tuple, launch) -> None:
        """Runs ``launch()``, a part's kernel calls for this step, through a launch program: the
        first step with this ``key`` runs it as it is and records its launches, later steps repeat the
        recording with one call into the library. ``key`` must name everything the calls depend on
        besides the contents of device buffers: the token count, how the rows split between kernels,
        whose cache is used. Addresses are covered by the engine: its buffers keep their places, and
        when one has to be replaced every recording is dropped."""
        eng = self._engine
        if not eng.use_programs or eng.tap is not None:
            launch()
            return
        full = (id(owner), key)
        program = eng._programs.get(full)
        if program is None:
            with kernels.record() as rec:
                launch()
            if len(eng._programs) >= eng.max_programs:          # a long-running server meets many shapes: the oldest goes
                eng._programs.pop(next(iter(eng._programs)))
            eng._programs[full] = rec.program
        else:
            program.run()
            eng.program_runs += 1

    def range(self, name: str):
        """A named range around some launches for profilers that show NVTX ranges (``StepEngine.nvtx``); free when off."""
        return _NvtxRange(name) if self._engine.nvtx else _NO_RANGE

    def tap(self, tag: str, layer: int, tensor: torch.Tensor) -> None:
        """Shows an intermediate activation to whoever listens (``StepEngine.tap``); the tags follow
        the reference's trace callback (src/model/model.h:16-22): "embedding", "attn_out" and
        "ffn_out" (the residual stream [tokens, hidden] after a layer's mixer / feed-forward; layer
        -1 for tensors outside the layers) and "final_norm" ([wanted rows, hidden])."""
        if self._engine.tap is not None:
            self._engine.tap(tag, layer, tensor, self)

    def attention_work(self, tokens_per_tile: int):
        """How this step's rows are shared between the two attention kernels: (rows of requests
        that bring a single token [n] on the device, tiles of longer portions [m, 3] = (first
        row, tokens, request), longest context among the single tokens). Built once per step."""
        key = ("attention_work", tokens_per_tile)
        if key not in self._cache and self.all_single:
            # decode-only step: rows 0..R-1 in order, no tiles, nothing to upload (and so nothing
            # that a captured graph would have to re-read from the host)
            self._cache[key] = (self._engine.row_index[:self.n_tokens], self._engine.no_work, self.longest_single)
        if key not in self._cache:
            single = [s.start for s in self.segments if s.length == 1]
            tiles = []
            for r, s in enumerate(self.segments):
                if s.length > 1:
                    for t in range(0, s.length, tokens_per_tile):
                        tiles.append((s.first_position + t, s.start + t, min(tokens_per_tile, s.length - t), r))
            # the causal triangle makes late tiles of a prompt the longest ones: they start first
            tiles.sort(key=lambda tile: -tile[0])
            tiles = [tile[1:] for tile in tiles]
            longest = self.longest_single
            flat = single + [v for tile in tiles for v in tile]
            dev = self._engine.upload_ints(flat)
            rows = dev[:len(single)]
            work = dev[len(single):].view(len(tiles), 3)
            self._cache[key] = (rows, work, longest)
        return self._cache[key]


class _NvtxRange:
    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        torch.cuda.nvtx.range_push(self.name)

    def __exit__(self, *exc):
        torch.cuda.nvtx.range_pop()
        return False


class _NoRange:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_NO_RANGE = _NoRange()


class StepEngine:
    token_feedback = True        # entries may name tokens by their place in ``feedback``

    def __init__(self, model: DecoderModel, page_size: int = 16, n_pages: int = 256, max_requests: int = 8,
                 max_step_tokens: int = 2048, max_logit_rows: Optional[int] = None, use_graphs: bool = True,
                 nvtx: bool = False, debug_checks: bool = False):
        """``nvtx``: every step, layer half and the head are wrapped in NVTX ranges (for profilers that show them).
        ``debug_checks``: before a step is launched its descriptor is checked on the host: every page a row reads or
        writes lies inside the pool and belongs to the row's request, positions are consecutive and inside the context."""
        if not torch.cuda.is_available():
            raise RuntimeError("StepEngine needs a CUDA device: this engine has no CPU path")
        self.model = model
        self.device = model.device
        self.page_size = page_size
        self.n_pages = n_pages
        self.max_requests = max_requests
        self.max_step_tokens = max_step_tokens
        self.max_logit_rows = max_logit_rows or max_step_tokens
        # sampled token ids stay here on the device, so that the next step can start from them
        self.feedback = torch.zeros(self.max_logit_rows, dtype=torch.int32, device=model.device)
        needs = model.cache_needs()
        state_needs = model.state_needs()
        self.cache = CacheManager(needs, page_size, n_pages, model.max_position, max_requests,
                                  state_layers=sorted(state_needs))
        # device memory of the pages: per group [layers of the group, 2 (keys, values), pages, Hkv, page, hd]
        self.group_pages: List[torch.Tensor] = []
        self.layer_pages: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}
        for group in self.cache.groups:
            need = group.need
            t = torch.empty((len(group.layers), 2, n_pages, need.num_kv_heads, page_size, need.head_dim),
                            dtype=model.dtype, device=self.device)
            t.fill_(float("nan"))       # never read before written; NaN makes a stale read visible
            self.group_pages.append(t)
            for i, layer in enumerate(group.layers):
                self.layer_pages[layer] = (t[i, 0], t[i, 1])
        self.layer_state: Dict[int, torch.Tensor] = {}
        for layer, need in state_needs.items():
            self.layer_state[layer] = torch.zeros((max_requests, *need.shape), dtype=_STATE_DTYPES[need.dtype],
                                                  device=self.device)
        self._scratch: Dict[Tuple, torch.Tensor] = {}
        self._init_descriptor()
        self.row_index = torch.arange(max(max_step_tokens, max_requests), dtype=torch.int32, device=self.device)
        self.no_work = torch.zeros((0, 3), dtype=torch.int32, device=self.device)
        # decode-only steps are captured into CUDA graphs, one per (requests, wanted rows, context bucket)
        # (only when every part says that its launches depend on nothing but the step's shape)
        self.use_graphs = use_graphs and all(
            getattr(layer.mixer, "graph_safe", False) and getattr(layer.feed_forward, "graph_safe", False)
            for layer in model.layers)
        self._graphs: Dict[Tuple, Tuple] = {}
        self.graph_replays = 0
        # launch programs of the parts, by (part, shape key): see StepContext.recorded
        self.nvtx = nvtx
        self.debug_checks = debug_checks
        self.use_programs = True
        self._programs: Dict[Tuple, object] = {}
        self.program_runs = 0
        # both caches are bounded: a server that runs for days meets ever new shapes (the oldest entry is dropped)
        self.max_programs = 4096
        self.max_graphs = 512
        # a listener for intermediate activations: tap(tag, layer, tensor, ctx); steps run outside graphs while it is set
        self.tap = None
        # the kernels' status word (a bounded wait that gave up) follows every step to pinned memory
        self._status_host = [torch.zeros(1, dtype=torch.int32).pin_memory() for _ in range(4)]
        self._status_events: List[Optional[torch.cuda.Event]] = [None] * 4
        self._status_next = 0
        self.scratch_generation = 0     # counts replaced scratch buffers: what was recorded before is stale

    # ------------------------------------------------------------------ memory
    # a buffer is given its full capacity at once while that stays below this many bytes; a larger one
    # (logits of thousands of wanted rows at a large vocabulary) grows as steps ask for more rows
    _SCRATCH_AT_ONCE = 64 << 20

    def scratch(self, name: str, shape: Tuple[int, ...], dtype: torch.dtype, capacity: Optional[int] = None) -> torch.Tensor:
        """A reusable buffer; the same name, trailing shape and dtype give the same memory each step.
        ``capacity`` is the most rows the buffer will ever need (default: the step's token limit).
        When a buffer has to grow, every captured graph is dropped first: a graph holds the addresses
        of the buffers it was captured with, and the old buffer goes back to the allocator."""
        key = (name, tuple(shape[1:]), dtype)
        buf = self._scratch.get(key)
        if buf is None or buf.shape[0] < shape[0]:
            most = max(shape[0], capacity if capacity is not None else self.max_step_tokens)
            row_bytes = max(1, int(np.prod(shape[1:], dtype=np.int64)) * torch.empty((), dtype=dtype).element_size())
            at_once = max(8, self._SCRATCH_AT_ONCE // row_bytes)
            rows = most if most <= at_once else min(most, max(at_once, 1 << (shape[0] - 1).bit_length()))
            if buf is not None:
                self._drop_captures()
            buf = torch.empty((rows, *shape[1:]), dtype=dtype, device=self.device)
            self._scratch[key] = buf
        return buf[:shape[0]]

    def _drop_captures(self) -> None:
        """Forgets everything that holds addresses of scratch memory (called before a buffer is replaced)."""
        self._graphs.clear()
        self._programs.clear()
        self.scratch_generation += 1

    def _init_descriptor(self) -> None:
        """One int32 buffer holds everything the kernels read about a step's rows and requests; a
        ring of pinned host mirrors is filled and copied with a single transfer per step."""
        T, R = self.max_step_tokens, self.max_requests
        stride = self.cache.max_pages_per_request
        self._layout: Dict[str, Tuple[int, int]] = {}
        off = 0
        for name, n in (("tokens", T), ("positions", T), ("row_req", T), ("logit_rows", self.max_logit_rows),
                        ("state_slots", R), ("seg_start", R), ("seg_len", R)):
            self._layout[name] = (off, n)
            off += n
        self._table_stride = max(stride, 1)
        self._table_off = []
        for _ in self.cache.groups:
            self._table_off.append(off)
            off += R * self._table_stride
        self._desc_size = off
        self._desc_dev = torch.zeros(off, dtype=torch.int32, device=self.device)
        self._ring = [torch.zeros(off, dtype=torch.int32).pin_memory() for _ in range(4)]
        self._ring_np = [b.numpy() for b in self._ring]
        self._ring_events: List[Optional[torch.cuda.Event]] = [None] * 4
        self._ring_next = 0
        # small integer lists that parts derive from a step (work lists of the attention kernels): the k-th
        # list of a step always lands in the same device buffer, through a ring of pinned staging buffers
        self._aux_cap = 4 * (T + R)
        self._aux_dev: List[torch.Tensor] = []
        self._aux_host: List[List[torch.Tensor]] = []
        self._aux_events: List[List[Optional[torch.cuda.Event]]] = []
        self._aux_turn: List[int] = []
        self._aux_calls = 0

    def upload_ints(self, values) -> torch.Tensor:
        """Small integer lists that a part derives from the step (work lists): copied asynchronously
        from pinned memory; the device view is valid until the next step. The k-th call of every step
        returns the same device address (copies and kernels are ordered on the stream), which lets
        recorded launches and captured graphs name it."""
        n = len(values)
        k = self._aux_calls
        self._aux_calls += 1
        if k == len(self._aux_dev):
            self._aux_dev.append(torch.zeros(self._aux_cap, dtype=torch.int32, device=self.device))
            self._aux_host.append([torch.zeros(self._aux_cap, dtype=torch.int32).pin_memory() for _ in range(4)])
            self._aux_events.append([None] * 4)
            self._aux_turn.append(0)
        if n > self._aux_dev[k].numel():
            self._drop_captures()                  # the list's place changes
            self._aux_dev[k] = torch.zeros(2 * n, dtype=torch.int32, device=self.device)
            self._aux_host[k] = [torch.zeros(2 * n, dtype=torch.int32).pin_memory() for _ in range(4)]
            self._aux_events[k] = [None] * 4
        turn = self._aux_turn[k]
        self._aux_turn[k] = (turn + 1) % 4
        if self._aux_events[k][turn] is not None:
            self._aux_events[k][turn].synchronize()
        host, dev = self._aux_host[k][turn], self._aux_dev[k]
        if n:
            host[:n] = torch.tensor(values, dtype=torch.int32)
            dev[:n].copy_(host[:n], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._aux_events[k][turn] = ev
        return dev[:n]

    # ------------------------------------------------------------------ requests
    def open(self, key: Hashable) -> RequestCache:
        return self.cache.open(key)

    def close(self, key: Hashable) -> None:
        self.cache.close(self.cache.requests[key])

    def fork(self, key: Hashable, new_key: Hashable, length: Optional[int] = None) -> RequestCache:
        """A new request on the first ``length`` cached positions of ``key`` (all by default), sharing
        their pages; the first step that writes into a shared page copies it on the device first."""
        return self.cache.fork(self.cache.requests[key], new_key, length)

    def truncate(self, key: Hashable, length: int) -> None:
        """Rewinds a request to its first ``length`` cached positions; later steps go on from there."""
        self.cache.truncate(self.cache.requests[key], length)

    def length(self, key: Hashable) -> int:
        return self.cache.requests[key].length

    # ------------------------------------------------------------------ the step
    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Runs one batch. Returns 32-bit logits [wanted, vocab] on the device, in the order of
        the entries and of each entry's ``want`` (None when nothing is wanted). The returned
        tensor is scratch memory that the next step overwrites."""
        entries = [e for e in entries if len(e.tokens) > 0]
        if not entries:
            return None
        V = self.model.vocab_size
        seen = set()
        total = 0
        n_want = 0
        for e in entries:
            if e.key in seen:
                raise ValueError(f"request {e.key!r} appears twice in one step")
            seen.add(e.key)
            if e.key not in self.cache.requests:
                raise KeyError(f"request {e.key!r} is not open")
            n = len(e.tokens)
            for tok in e.tokens:
                if not (0 <= int(tok) < V) and not (-self.max_logit_rows <= int(tok) < 0):
                    raise IndexError(f"token id {tok} is outside the vocabulary of {V}")
            for w in e.want:
                if not (0 <= int(w) < n):
                    raise IndexError(f"wanted place {w} is outside the {n} tokens of request {e.key!r}")
            rc = self.cache.requests[e.key]
            if rc.length + n > self.model.max_position:
                raise IndexError(f"request {e.key!r}: position {rc.length + n - 1} is beyond the context length "
                                 f"{self.model.max_position}")
            total += n
            n_want += len(e.want)
        if total > self.max_step_tokens:
            raise ValueError(f"{total} tokens in one step exceed the limit {self.max_step_tokens}")
        if len(entries) > self.max_requests:
            raise ValueError(f"{len(entries)} requests in one step exceed the limit {self.max_requests}")
        if n_want > self.max_logit_rows:
            raise ValueError(f"{n_want} wanted rows exceed the limit {self.max_logit_rows}")

        self._poll_status(wait=False)      # before anything is reserved: an earlier step's failure ends this call

        # ---- reserve pages for every entry, all or nothing
        reserved: List[RequestCache] = []
        copies = []
        try:
            for e in entries:
                rc = self.cache.requests[e.key]
                copies += self.cache.reserve(rc, len(e.tokens))
                reserved.append(rc)
        except OutOfPages:
            for rc in reserved:
                self.cache.rollback(rc)
            raise
        if copies:
            self._copy_pages(copies)

        # ---- describe the step
        self._aux_calls = 0
        slot = self._ring_next
        self._ring_next = (slot + 1) % len(self._ring)
        if self._ring_events[slot] is not None:
            self._ring_events[slot].synchronize()
        host = self._ring_np[slot]
        lay = self._layout
        segments: List[Segment] = []
        row = 0
        k = 0
        t_off, p_off, r_off, l_off = lay["tokens"][0], lay["positions"][0], lay["row_req"][0], lay["logit_rows"][0]
        for r, e in enumerate(entries):
            rc = self.cache.requests[e.key]
            n = len(e.tokens)
            host[t_off + row:t_off + row + n] = np.asarray(e.tokens, dtype=np.int32)
            host[p_off + row:p_off + row + n] = np.arange(rc.length, rc.length + n, dtype=np.int32)
            host[r_off + row:r_off + row + n] = r
            for w in e.want:
                host[l_off + k] = row + int(w)
                k += 1
            host[lay["state_slots"][0] + r] = rc.state_slot
            host[lay["seg_start"][0] + r] = row
            host[lay["seg_len"][0] + r] = n
            for g in range(len(self.cache.groups)):
                base = self._table_off[g] + r * self._table_stride
                npg = rc.n_pages[g]
                host[base:base + npg] = rc.tables[g][:npg]
            segments.append(Segment(e.key, row, n, rc.length, rc.state_slot, rc.fresh_state))
            row += n
        self._desc_dev.copy_(self._ring[slot], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._ring_events[slot] = ev

        dev = self._desc_dev
        R = len(entries)
        views = {
            "tokens": dev[t_off:t_off + total], "positions": dev[p_off:p_off + total],
            "row_req": dev[r_off:r_off + total], "logit_rows": dev[l_off:l_off + k],
            "state_slots": dev[lay["state_slots"][0]:lay["state_slots"][0] + R],
            "seg_start": dev[lay["seg_start"][0]:lay["seg_start"][0] + R],
            "seg_len": dev[lay["seg_len"][0]:lay["seg_len"][0] + R],
            "tables": [dev[o:o + R * self._table_stride].view(R, self._table_stride) for o in self._table_off],
        }
        for seg in segments:                       # state of a new request starts from zero
            if seg.fresh_state:
                for st in self.layer_state.values():
                    st[seg.state_slot].zero_()
        if self.debug_checks:
            self._check_descriptor(host, segments, total)
        ctx = StepContext(self, total, R, k, segments, views)
        with ctx.range(f"step {total} tokens {R} requests"):
            logits = self._run(ctx)
        self._post_status()
        for e in entries:
            self.cache.advance(self.cache.requests[e.key], len(e.tokens))
        return logits

    def _run(self, ctx: StepContext) -> Optional[torch.Tensor]:
        """The model's forward pass for this step. A decode-only step (one token per request, no
        state to zero) has a fixed launch sequence for its shape: it is run once directly, then
        captured into a CUDA graph and replayed from then on, which removes the per-launch cost on
        the host. Everything a replay reads that changes from step to step (tokens, positions,
        block tables) lives in the descriptor buffer, refreshed before the replay."""
        fresh = any(s.fresh_state for s in ctx.segments) and self.layer_state
        if not (self.use_graphs and ctx.all_single and not fresh and self.tap is None):
            with kernels.on_current_stream():
                return self.model.forward(ctx)
        key = (ctx.n_tokens, ctx.n_logit_rows, ctx.longest_single)
        entry = self._graphs.get(key)
        if entry is None:
            with kernels.on_current_stream():
                out = self.model.forward(ctx)      # also sizes scratch and configures the kernels
            before = kernels.launch_count()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph), kernels.on_current_stream():
                captured = self.model.forward(ctx)
            n_kernels = kernels.launch_count() - before
            kernels.count_launches(-n_kernels)     # captured, not launched
            if len(self._graphs) >= self.max_graphs:           # the oldest shape's graph goes
                self._graphs.pop(next(iter(self._graphs)))
            self._graphs[key] = (graph, captured, n_kernels)
            return out
        graph, captured, n_kernels = entry
        graph.replay()
        self.graph_replays += 1
        kernels.count_launches(n_kernels)
        return captured

    def _check_descriptor(self, host: np.ndarray, segments: List[Segment], total: int) -> None:
        """The step's descriptor as the kernels will read it, checked on the host (``debug_checks``): a wrong page id
        or position would make a kernel read or write another request's memory without any error."""
        lay = self._layout
        pos = host[lay["positions"][0]:lay["positions"][0] + total]
        req = host[lay["row_req"][0]:lay["row_req"][0] + total]
        ps = self.page_size
        for r, seg in enumerate(segments):
            rows = slice(seg.start, seg.start + seg.length)
            if not (req[rows] == r).all() or not (pos[rows] == np.arange(seg.first_position, seg.first_position + seg.length)).all():
                raise AssertionError(f"step descriptor: rows of request {seg.key!r} are not its consecutive positions")
            if seg.first_position + seg.length > self.model.max_position:
                raise AssertionError(f"step descriptor: request {seg.key!r} runs beyond the context length")
            rc = self.cache.requests[seg.key]
            for g, group in enumerate(self.cache.groups):
                table = host[self._table_off[g] + r * self._table_stride:self._table_off[g] + (r + 1) * self._table_stride]
                first = rc.first_live[g] if group.need.window else 0
                used = table[first:(seg.first_position + seg.length + ps - 1) // ps]
                if ((used < 0) | (used >= self.n_pages)).any():
                    raise AssertionError(f"step descriptor: request {seg.key!r} names a page outside the pool of {self.n_pages}")
                if any(group.pool.ref_count(int(p)) < 1 for p in used):
                    raise AssertionError(f"step descriptor: request {seg.key!r} names a page that is free")
        pages = [int(p) for r, seg in enumerate(segments) for g in range(len(self.cache.groups))
                 for p in self.cache.requests[seg.key].tables[g][(seg.first_position // ps):(seg.first_position + seg.length + ps - 1) // ps]]
        written = [p for p in pages if p >= 0]
        if len(set(written)) != len(written) and len(self.cache.groups) == 1:
            raise AssertionError("step descriptor: two requests of one step write into the same page")

    # ------------------------------------------------------------------ the kernels' status word
    def _post_status(self) -> None:
        """Sends the status word after the step's kernels to pinned memory (no wait)."""
        slot = self._status_next
        self._status_next = (slot + 1) % len(self._status_host)
        if self._status_events[slot] is not None:
            self._status_events[slot].synchronize()
            self._raise_on(self._status_host[slot])
        self._status_host[slot].copy_(kernels.status_word(self.device), non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._status_events[slot] = ev

    def _poll_status(self, wait: bool) -> None:
        """Looks at the status words of steps that have finished (of all steps with ``wait``) and
        raises ``KernelError`` if a kernel recorded that one of its bounded waits gave up: what
        that step computed is not to be trusted."""
        for slot, ev in enumerate(self._status_events):
            if ev is not None and (wait or ev.query()):
                ev.synchronize()
                self._status_events[slot] = None
                self._raise_on(self._status_host[slot])

    def _raise_on(self, word: torch.Tensor) -> None:
        code = int(word[0])
        if code:
            word[0] = 0
            kernels.status_word(self.device).zero_()
            for i in range(len(self._status_events)):
                self._status_events[i] = None
            raise kernels.KernelError(f"a kernel gave up a bounded wait (status {code:#x}): the results of the "
                                      f"last steps are not valid")

    def check_status(self) -> None:
        """Waits for the steps launched so far and raises if any kernel reported a failed wait.
        Callers that read logits themselves call this before they trust them."""
        self._poll_status(wait=True)

    def _copy_pages(self, copies) -> None:
        for g, pages in enumerate(self.group_pages):
            mine = [c for c in copies if c.group == g]
            if not mine:
                continue
            src = torch.tensor([c.src for c in mine], dtype=torch.int32, device=self.device)
            dst = torch.tensor([c.dst for c in mine], dtype=torch.int32, device=self.device)
            flat = pages.view(pages.shape[0] * 2, *pages.shape[2:])
            kernels.copy_pages(flat, src, dst)
