"""The scheduler's decisions, on the CPU with the hash-chain backend: order inside a step, token
budget, portions, finishing, giving pages back, and what happens when pages run out."""
import numpy as np
import pytest

import fake_backend as fb
from geneinfer_b200.engine.scheduler import GenerationRequest, Scheduler, SchedulerConfig
from geneinfer_b200.sampling import SamplingParams


def make(n_pages, page_size=4, context=64, vocab=50, window=None, **cfg):
    backend = fb.FakeBackend(n_pages, page_size, context, vocab, max_requests=cfg.get("max_running", 8), window=window)
    return backend, Scheduler(backend, fb.sample_rows(vocab), SchedulerConfig(**cfg))


def check_against_alone(backend, sched, requests):
    for jid, req in enumerate(requests):
        res = sched.result(jid)
        assert res.finished and not res.error, res.error
        want, stopped = fb.expected_alone(req.prompt, req.max_positions, req.sampling, req.stop_ids,
                                          backend.model.max_position, backend.model.vocab_size)
        assert res.generated_tokens == want, f"request {jid}"
        assert res.stopped_by_end_token == stopped


def test_decodes_first_then_portions_oldest_first_under_the_budget():
    backend, s = make(64, step_tokens=10, prefill_chunk=6, prefix_cache=False)
    a = s.submit(GenerationRequest(list(range(1, 4)), 8, SamplingParams(0.0)))     # short: decoding from step 2 on
    b = s.submit(GenerationRequest(list(range(10, 30)), 0, SamplingParams(0.0)))   # 20 tokens: portions
    c = s.submit(GenerationRequest(list(range(30, 45)), 0, SamplingParams(0.0)))
    s.step()
    assert backend.steps[0] == [(("job", 0), 3, True), (("job", 1), 6, False), (("job", 2), 1, False)]   # 3 + 6 + 1 = budget
    s.step()
    assert backend.steps[1] == [(("job", 0), 1, True), (("job", 1), 6, False), (("job", 2), 3, False)]   # decode first
    s.run_until_idle()
    assert all(sum(n for _, n, _ in st) <= 10 for st in backend.steps)
    assert s.result(a).generated_tokens and len(s.result(a).generated_tokens) == 8 - 3 + 1
    assert s.stats.max_chunk == 6 and s.stats.max_tokens_in_step == 10
    assert backend.cache.free_pages() == 64 and not backend.cache.requests


def test_results_equal_running_alone_for_random_requests():
    rng = np.random.default_rng(0)
    for trial in range(12):
        pages = [64, 20, 9][trial % 3]                  # roomy, tight, very tight
        backend, s = make(pages, step_tokens=int(rng.integers(4, 24)), prefill_chunk=int(rng.integers(0, 9)),
                          max_running=int(rng.integers(1, 6)), prefix_cache=bool(trial % 2))
        reqs = []
        for _ in range(int(rng.integers(3, 10))):
            n = int(rng.integers(1, 28))
            shared = [7, 7, 7, 7, 3, 3, 3, 3, 9] if rng.random() < 0.4 else []      # common prefixes
            prompt = (shared + [int(t) for t in rng.integers(0, 50, n)])[:32]
            temp = [0.0, 0.8][int(rng.integers(0, 2))]
            reqs.append(GenerationRequest(prompt, int(rng.integers(1, 36)),      # a request alone always fits in 9 pages
                                           SamplingParams(temp, 0, 1.0, int(rng.integers(0, 99))),
                                          stop_ids=(5,) if rng.random() < 0.5 else ()))
        for i, r in enumerate(reqs):
            s.submit(r)
            if i % 3 == 2:
                s.step()                                # staggered arrival
        s.run_until_idle()
        check_against_alone(backend, s, reqs)
        if s.prefix:
            s.prefix.clear()
        backend.cache.check_invariants()
        assert backend.cache.free_pages() == pages and not backend.cache.requests, "pages or requests were lost"


def test_steps_launched_ahead_give_the_same_results():
    """With a backend that takes tokens from the device, decode steps are launched before the ids of
    the step before are known to the host; stop tokens, limits, arrivals and short pools in between."""
    rng = np.random.default_rng(1)
    ahead = 0
    for trial in range(12):
        pages = [64, 20, 9][trial % 3]
        backend = fb.FakeFeedbackBackend(pages, 4, 64, 50, max_requests=8)
        s = Scheduler(backend, fb.sample_rows(50),
                      SchedulerConfig(max_running=int(rng.integers(1, 6)), step_tokens=int(rng.integers(4, 24)),
                                      prefill_chunk=int(rng.integers(0, 9)), prefix_cache=bool(trial % 2)),
                      sample_async=fb.sample_async(backend, 50))
        assert s.lookahead
        reqs = []
        for _ in range(int(rng.integers(3, 10))):
            n = int(rng.integers(1, 28))
            shared = [7, 7, 7, 7, 3, 3, 3, 3, 9] if rng.random() < 0.4 else []
            prompt = (shared + [int(t) for t in rng.integers(0, 50, n)])[:32]
            temp = [0.0, 0.8][int(rng.integers(0, 2))]
            reqs.append(GenerationRequest(prompt, int(rng.integers(1, 36)),
                                          SamplingParams(temp, 0, 1.0, int(rng.integers(0, 99))),
                                          stop_ids=(5, 6, 7) if rng.random() < 0.5 else ()))
        for i, r in enumerate(reqs):
            s.submit(r)
            if i % 3 == 2:
                s.step()
        s.run_until_idle()
        assert s.idle()
        check_against_alone(backend, s, reqs)
        if s.prefix:
            s.prefix.clear()
        backend.cache.check_invariants()
        assert backend.cache.free_pages() == pages and not backend.cache.requests, "pages or requests were lost"
        ahead += backend.ahead_steps
    assert ahead > 20, "no step was launched ahead"


def test_a_stop_token_drops_the_row_of_the_step_launched_ahead():
    backend = fb.FakeFeedbackBackend(32, 4, 64, 50)
    s = Scheduler(backend, fb.sample_rows(50), SchedulerConfig(max_running=2, prefix_cache=False),
                  sample_async=fb.sample_async(backend, 50))
    want, _ = fb.expected_alone([1, 2, 3], 0, SamplingParams(0.0), (), 64, 50)
    stop = want[4]                                        # ends at its 5th generated token
    first = want.index(stop)
    a = s.submit(GenerationRequest([1, 2, 3], 0, SamplingParams(0.0), stop_ids=(stop,)))
    b = s.submit(GenerationRequest([9, 8, 7, 6], 20, SamplingParams(0.0)))
    s.run_until_idle()
    assert s.result(a).generated_tokens == want[:first + 1] and s.result(a).stopped_by_end_token
    assert s.result(b).generated_tokens == fb.expected_alone([9, 8, 7, 6], 20, SamplingParams(0.0), (), 64, 50)[0]
    assert backend.ahead_steps > 0
    assert backend.cache.free_pages() == 32 and not backend.cache.requests


def test_pages_run_out_youngest_is_preempted_and_recomputed():
    backend, s = make(10, page_size=4, step_tokens=64, max_running=3, prefix_cache=False)
    reqs = [GenerationRequest([1 + i] * 10, 30, SamplingParams(0.8, 0, 1.0, seed=i)) for i in range(3)]
    for r in reqs:
        s.submit(r)
    s.run_until_idle()
    assert s.stats.preemptions > 0, "the pool was meant to be too small for three requests at once"
    assert s.result(2).preemptions >= s.result(0).preemptions == 0        # the youngest goes, the oldest never
    check_against_alone(backend, s, reqs)                                 # same tokens, the random stream went on
    assert backend.cache.free_pages() == 10


def test_a_request_that_can_never_fit_ends_with_an_error():
    backend, s = make(3, page_size=4, step_tokens=64, prefix_cache=False)
    ok = s.submit(GenerationRequest([1, 2, 3], 6, SamplingParams(0.0)))
    big = s.submit(GenerationRequest(list(range(20)), 0, SamplingParams(0.0)))      # 20 positions need 5 pages of 3
    s.run_until_idle()
    assert s.result(ok).finished and not s.result(ok).error and len(s.result(ok).generated_tokens) == 4
    assert s.result(big).finished and "too small" in s.result(big).error
    assert backend.cache.free_pages() == 3 and not backend.cache.requests


def test_prefix_cache_skips_shared_pages_and_evicts_under_pressure():
    backend, s = make(12, page_size=4, step_tokens=64, max_running=1, prefix_cache=True)
    common = list(range(1, 14))                                         # 13 tokens = 3 full pages + 1
    reqs = [GenerationRequest(common + [20 + i], 18, SamplingParams(0.0)) for i in range(3)]
    for r in reqs:
        s.submit(r)
    s.run_until_idle()
    check_against_alone(backend, s, reqs)
    assert s.result(0).cached_tokens == 0 and s.result(1).cached_tokens == 12 and s.result(2).cached_tokens == 12
    assert s.stats.prefix_hits == 2 and s.stats.prefix_tokens == 24
    fed = sum(n for st in backend.steps for _, n, _ in st)
    assert fed + s.stats.prefix_tokens == sum(min(18, len(r.prompt) + 4) for r in reqs)      # every position counted once
    other = [GenerationRequest([40 + i] * 30, 44, SamplingParams(0.0)) for i in range(2)]     # need the cached pages' room
    for r in other:
        s.submit(r)
    s.run_until_idle()
    assert s.stats.evicted_pages > 0
    check_against_alone(backend, s, reqs + other)
    s.prefix.clear()
    assert backend.cache.free_pages() == 12


def test_position_limit_inside_the_prompt_and_stop_token():
    backend, s = make(32, prefix_cache=False)
    a = s.submit(GenerationRequest(list(range(10)), 4, SamplingParams(0.0)))          # ends inside its prompt
    s.run_until_idle()
    assert s.result(a).finished and s.result(a).generated_tokens == []
    want, _ = fb.expected_alone([3, 4], 0, SamplingParams(0.0), (), 64, 50)
    stop = want[2]
    b = s.submit(GenerationRequest([3, 4], 0, SamplingParams(0.0), stop_ids=(stop,)))
    s.run_until_idle()
    assert s.result(b).generated_tokens == want[:want.index(stop) + 1] and s.result(b).stopped_by_end_token


def test_window_model_runs_through_the_scheduler():
    backend, s = make(6, page_size=4, window=5, step_tokens=7, prefix_cache=True)     # 6 pages: far less than 40 positions
    assert s.prefix is None                                                           # pages of a window cannot be shared
    r = GenerationRequest(list(range(1, 12)), 40, SamplingParams(0.0))
    s.submit(r)
    s.run_until_idle()
    res = s.result(0)
    assert res.finished and not res.error and len(res.generated_tokens) == 40 - 11 + 1
    assert backend.cache.free_pages() == 6


def test_submit_refuses_bad_requests():
    backend, s = make(8)
    with pytest.raises(ValueError, match="no tokens"):
        s.submit(GenerationRequest([]))
    with pytest.raises(ValueError, match="does not fit"):
        s.submit(GenerationRequest([1] * 65))
    with pytest.raises(ValueError, match="out of range"):
        s.submit(GenerationRequest([50]))
    with pytest.raises(ValueError):
        SamplingParams(temperature=-1.0)
    with pytest.raises(ValueError):
        SamplingParams(top_p=0.0)
    with pytest.raises(ValueError):
        SamplingParams(top_k=-1)
    assert s.step() is False


def test_sampled_ids_are_refused_when_a_kernel_reported_a_failed_wait():
    """The kernels' status word travels to the host with the sampled ids: a value other than 0 (a
    bounded wait that gave up, so a tile of garbage) must end the call instead of returning tokens."""
    import torch
    from geneinfer_b200.ops.library import KernelError
    from geneinfer_b200.sampling.device import PendingSample

    class Done:
        def synchronize(self):
            pass

    ids = torch.tensor([4, 9, 2], dtype=torch.int32)
    assert PendingSample(ids, 2, Done(), torch.zeros(1, dtype=torch.int32)).result() == [4, 9]
    cleared = []
    status = torch.tensor([0x21], dtype=torch.int32)
    with pytest.raises(KernelError, match="0x21"):
        PendingSample(ids, 3, Done(), status, lambda: cleared.append(True)).result()
    assert cleared == [True] and int(status[0]) == 0


def test_finished_requests_can_be_forgotten():
    backend = fb.FakeBackend(16, 4, 64, 50)
    s = Scheduler(backend, lambda l, p, u: [fb.pick_token(h, q, x, 50) for h, q, x in zip(l, p, u)], SchedulerConfig(2, 16, 0, False))
    a = s.submit(GenerationRequest([1, 2, 3], 6, SamplingParams(0.0)))
    with pytest.raises(RuntimeError):
        s.forget(a)                                   # still waiting
    s.run_until_idle()
    assert len(s.result(a).generated_tokens) == 4
    s.forget(a)
    with pytest.raises(KeyError):
        s.result(a)
    with pytest.raises(KeyError):
        s.forget(a)
    b = s.submit(GenerationRequest([4], 3, SamplingParams(0.0)))
    assert b == a + 1, "ids are not handed out again"
    s.run_until_idle()
    assert s.result(b).finished
