"""A backend for scheduler tests that runs on the CPU: the real cache manager, and in place of the
model a chain of hashes kept *in the pages*.

Position p of a request stores h_p = H(h_{p-1}, token_p) in its page row, and h_{p-1} is read back
through the block table, so a wrong table, a page handed to two requests, a stale page or a wrong
position changes every later value. The "logits" of a wanted row are h_p itself, and sampling maps
(h_p, u) to a token: a request's tokens are right only if its whole history was kept right.
"""
import hashlib

from geneinfer_b200.cache import CacheManager, CacheNeed, OutOfPages


def H(prev: int, token: int) -> int:
    return int.from_bytes(hashlib.blake2b(f"{prev}:{token}".encode(), digest_size=8).digest(), "little")


def pick_token(h: int, params, u: float, vocab: int) -> int:
    if params.greedy:
        return h % vocab
    return (h + int(u * 16777216.0) * 2654435761 + params.top_k * 97 + int(params.top_p * 1000)) % vocab


class FakeModel:
    def __init__(self, max_position, vocab_size):
        self.max_position, self.vocab_size = max_position, vocab_size


class FakeBackend:
    def __init__(self, n_pages, page_size=4, max_position=64, vocab=50, max_requests=8, window=None):
        self.model = FakeModel(max_position, vocab)
        self.cache = CacheManager({0: CacheNeed(1, 16, window)}, page_size, n_pages, max_position, max_requests)
        self.store = [[None] * page_size for _ in range(n_pages)]
        self.steps = []                     # per step: list of (key, n tokens, wants logits)

    def open(self, key):
        return self.cache.open(key)

    def close(self, key):
        self.cache.close(self.cache.requests[key])

    def _row(self, rc, pos):
        ps = self.cache.page_size
        page = int(rc.tables[0][pos // ps])
        assert page >= 0, f"position {pos} lies in a page that was given back"
        return self.store[page], pos % ps

    def step(self, entries):
        reserved = []
        try:
            for e in entries:
                rc = self.cache.requests[e.key]
                copies = self.cache.reserve(rc, len(e.tokens))
                for c in copies:
                    self.store[c.dst] = list(self.store[c.src])
                reserved.append(rc)
        except OutOfPages:
            for rc in reserved:
                self.cache.rollback(rc)
            raise
        out = []
        self.steps.append([(e.key, len(e.tokens), bool(e.want)) for e in entries])
        for e in entries:
            rc = self.cache.requests[e.key]
            hs = []
            for i, tok in enumerate(e.tokens):
                pos = rc.length + i
                prev = 0
                if pos > 0:
                    page, off = self._row(rc, pos - 1)
                    assert page[off] is not None and page[off][0] == pos - 1, f"position {pos - 1} was not cached"
                    prev = page[off][1]
                h = H(prev, int(tok))
                page, off = self._row(rc, pos)
                page[off] = (pos, h)
                hs.append(h)
            out += [hs[w] for w in e.want]
            self.cache.advance(rc, len(e.tokens))
        return out


class FakeFeedbackBackend(FakeBackend):
    """The same, for steps launched ahead: a token given as -(k + 1) is place k of ``feedback``,
    where the sampler below leaves its ids at once, as a sampling kernel does on the device."""
    token_feedback = True

    def __init__(self, *args, **kw):
        super().__init__(*args, **kw)
        self.feedback = []
        self.ahead_steps = 0

    def step(self, entries):
        from geneinfer_b200.engine.step import StepEntry
        if any(int(t) < 0 for e in entries for t in e.tokens):
            self.ahead_steps += 1
        resolved = [StepEntry(e.key, [self.feedback[-int(t) - 1] if int(t) < 0 else t for t in e.tokens], e.want)
                    for e in entries]
        return super().step(resolved)


class _Later:
    def __init__(self, ids):
        self._ids = ids

    def result(self):
        return self._ids


def sample_async(backend, vocab):
    """The ids are on the "device" (backend.feedback) at once; the host gets them on result()."""
    def fn(logits, params, uniforms):
        ids = [pick_token(h, p, u, vocab) for h, p, u in zip(logits, params, uniforms)]
        backend.feedback = list(ids)
        return _Later(ids)
    return fn


def sample_rows(vocab):
    def fn(logits, params, uniforms):
        return [pick_token(h, p, u, vocab) for h, p, u in zip(logits, params, uniforms)]
    return fn


def expected_alone(prompt, max_positions, params, stop_ids, context, vocab):
    """What a request generates when it runs alone and whole (the generation loop of
    src/runtime/generator.cpp:42-76 over the same chain of hashes)."""
    from geneinfer_b200.sampling import RandomStream
    limit = context if max_positions <= 0 else min(max_positions, context)
    stream = RandomStream(params.seed)
    tokens, out, h = list(prompt), [], 0
    fed = 0
    while fed < limit:
        h = H(h, tokens[fed])
        fed += 1
        if fed == len(tokens):
            u = 0.0 if params.greedy else stream.next_uniform()
            nxt = pick_token(h, params, u, vocab)
            out.append(nxt)
            tokens.append(nxt)
            if nxt in stop_ids:
                return out, True
    return out, False
