"""Continuous-batching planner policy and the engine loop on the CPU tiny model."""
import threading
import time

import pytest
import torch

from sllm_b200.engine import scheduler as sch
from sllm_b200.engine.engine import build_engine
from sllm_b200.engine.sampling import SamplerChain, SamplerChainConfig, SamplingParams
from sllm_b200.models.config import tiny_llama


def test_planner_prefill_then_round_robin_decode():
    p = sch.BatchPlanner(max_batch=2, prefill_interval=2, max_prefill_batch=4)
    for rid in (1, 2, 3):
        p.submit(rid, "m")
    r = p.next_round()
    assert r.kind == "prefill" and r.rows == [1, 2]          # capped by max_batch
    p.complete_round({1: "continue", 2: "continue"})
    r = p.next_round()
    assert r.kind == "decode" and r.rows == [1, 2]
    p.complete_round({1: "continue", 2: "finished"})
    r = p.next_round()                                         # one decode round so far: decode again
    assert r.kind == "decode" and r.rows == [1]
    p.complete_round({1: "continue"})
    r = p.next_round()                                         # interval reached and a slot is free
    assert r.kind == "prefill" and r.rows == [3]
    p.complete_round({3: "continue"})
    r = p.next_round()
    assert r.kind == "decode" and r.rows == [1, 3]
    p.complete_round({1: "finished", 3: "finished"})
    assert p.next_round() is None and p.idle()


def test_planner_cancel_backpressure_singleton_and_errors():
    p = sch.BatchPlanner(max_batch=4, prefill_interval=1)
    p.submit(1, "m")
    p.submit(2, "m", sch.LANE_SINGLETON)
    p.submit(3, "m")
    with pytest.raises(sch.PlannerError):
        p.submit(1, "m")
    with pytest.raises(sch.PlannerError):
        p.submit(0, "m")
    assert p.cancel(3) == sch.CANCELLED                        # queued: immediate
    r = p.next_round()
    assert r.kind == "prefill" and r.rows == [1]               # singleton does not join
    assert p.cancel(1) == sch.PREFILL_IN_FLIGHT                # deferred
    with pytest.raises(sch.PlannerError):
        p.next_round()
    assert p.complete_round({1: "continue"}) == [1] and p.phase(1) == sch.CANCELLED
    r = p.next_round()
    assert r.kind == "prefill" and r.rows == [2]
    with pytest.raises(sch.PlannerError):
        p.complete_round({})
    p.complete_round({2: "backpressured"})
    assert p.next_round() is None                              # nothing runnable while back-pressured
    p.set_backpressured(2, False)
    assert p.next_round().rows == [2]
    p.complete_round({2: "failed"})
    assert p.phase(2) == sch.FAILED


def _loop(max_batch=4, **kw):
    cfg = tiny_llama()
    cfg.max_context = 96
    eng = build_engine(cfg, "cpu", seed=0, max_batch=max_batch, use_cuda_graphs=False)
    return eng, sch.EngineLoop(eng, "tiny", **kw)


def _collect(loop, prompt, n, **kw):
    toks, done = [], threading.Event()
    reason = []
    req = sch.GenRequest(prompt, n, on_token=lambda t, s: toks.append(t) or True,
                         on_done=lambda r: (reason.append(r), done.set()), **kw)
    loop.submit(req)
    return req, toks, done, reason


def test_engine_loop_matches_plain_generation_and_interleaves():
    eng, loop = _loop(prefill_interval=2)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (9, 17, 5, 12, 20)]
    try:
        jobs = [_collect(loop, p, 10) for p in prompts]
        for _, _, done, _ in jobs:
            assert done.wait(60)
        ref_eng = build_engine(eng.cfg, "cpu", seed=0, max_batch=4, use_cuda_graphs=False)
        for (req, toks, _, reason), p in zip(jobs, prompts):
            assert reason == ["length"]
            assert toks == ref_eng.generate([p], 10)[0]        # batching does not change greedy results
        assert loop.rounds["decode"] >= 9 and loop.rounds["prefill"] >= 2
        assert eng.cache.pool.stats()["sequences"] == 0        # every sequence released
    finally:
        loop.shutdown(1.0)


def test_engine_loop_queue_full_cancel_timeout_and_sampling():
    eng, loop = _loop(max_batch=2, queue_capacity=2)
    try:
        gate = threading.Event()

        def slow(t, s):
            gate.wait(5)
            return True
        blocker = sch.GenRequest([1, 2, 3], 50, on_token=slow)
        loop.submit(blocker)
        time.sleep(0.2)
        r2, t2, d2, why2 = _collect(loop, [4, 5], 5)
        r3, t3, d3, why3 = _collect(loop, [6, 7], 5)
        with pytest.raises(sch.QueueFull):
            loop.submit(sch.GenRequest([8], 2))
        assert loop.cancel(r3.rid)                              # queued: cancelled at once
        assert d3.wait(5) and why3 == ["cancelled"]
        gate.set()
        assert d2.wait(30) and why2 == ["length"] and len(t2) == 5
        loop.cancel(blocker.rid)
        # timeout and stop token
        r4, t4, d4, why4 = _collect(loop, [9, 9, 9], 10_000, deadline=time.monotonic() + 0.3)
        assert d4.wait(30) and why4 == ["timeout"]
        # seeded sampling is reproducible and differs from greedy somewhere
        outs = []
        for _ in range(2):
            chain = SamplerChain(SamplerChainConfig(SamplingParams(1.5)), seed=123)
            r, t, d, why = _collect(loop, [3, 1, 4, 1, 5], 12, chain=chain)
            assert d.wait(30)
            outs.append(t)
        assert outs[0] == outs[1] and len(outs[0]) == 12
        st = loop.stats()
        assert st["accepting"] and st["queue_capacity"] == 2
    finally:
        info = loop.shutdown(1.0)
        assert "cancelled_at_shutdown" in info
    with pytest.raises(sch.QueueFull):
        loop.submit(sch.GenRequest([1], 1))


def test_prefix_fork_reuses_pages():
    eng, loop = _loop()
    loop.shutdown(0.1)
    base = list(range(1, 41))
    s1 = eng.new_sequence(base)
    l1 = eng.prefill([s1], sample=False)
    child = eng.fork_sequence(s1, base[:37] + [99, 98, 97])
    assert child.num_computed == 37
    shared = set(eng.cache.pool.pages(s1.seq_id)[:2]) & set(eng.cache.pool.pages(child.seq_id)[:2])
    assert len(shared) == 2 and eng.cache.pool.refcount(eng.cache.pool.pages(s1.seq_id)[0]) == 2
    lc = eng.prefill([child], sample=False)
    fresh = eng.new_sequence(base[:37] + [99, 98, 97])
    lf = eng.prefill([fresh], sample=False)
    assert torch.allclose(lc, lf, atol=1e-4)
    for s in (s1, child, fresh):
        eng.free_sequence(s)
    assert eng.cache.pool.stats()["free"] == eng.cache.pool.stats()["pages"]


def test_chunked_prefill_interleaves_with_decode():
    """With a prefill chunk size a long prompt runs one chunk per prefill round, and the running request decodes
    between the chunks; the results equal unchunked generation."""
    eng, loop = _loop(prefill_interval=4, prefill_chunk_tokens=8)
    g = torch.Generator().manual_seed(1)
    short = torch.randint(0, 1024, (6,), generator=g).tolist()
    long = torch.randint(0, 1024, (50,), generator=g).tolist()
    try:
        stamps = []
        first = _collect(loop, short, 30)
        first[0].on_token = lambda t, s, _o=first[0].on_token: (stamps.append(("short", loop.rounds["prefill"])), _o(t, s))[1]
        while len(first[1]) < 2:                               # the short request is decoding
            time.sleep(0.005)
        before = loop.rounds["prefill"]
        second = _collect(loop, long, 5)
        assert first[2].wait(60) and second[2].wait(60)
        ref_eng = build_engine(eng.cfg, "cpu", seed=0, max_batch=4, use_cuda_graphs=False)
        assert first[1] == ref_eng.generate([short], 30)[0]
        assert second[1] == ref_eng.generate([long], 5)[0]
        # 50 tokens in chunks of 8 = 7 prefill rounds for the long prompt
        assert loop.rounds["prefill"] - before == 7
        # the short request produced tokens while the long prompt was still being prefilled
        during = {n for who, n in stamps if before < n < before + 7}
        assert len(during) >= 3
        assert eng.cache.pool.stats()["sequences"] == 0
    finally:
        loop.shutdown(1.0)


def test_planner_prefill_more_goes_back_to_the_head():
    p = sch.BatchPlanner(max_batch=4, prefill_interval=4)
    p.submit(1, "m")
    assert p.next_round().kind == "prefill"
    p.complete_round({1: "continue"})
    p.submit(2, "m")
    p.submit(3, "m")
    for _ in range(4):
        assert p.next_round().kind == "decode"
        p.complete_round({1: "continue"})
    r = p.next_round()
    assert r.kind == "prefill" and r.rows == [2, 3]
    p.complete_round({2: "prefill_more", 3: "continue"})
    assert p.next_round().kind == "decode"                    # one decode round, then the next chunk
    p.complete_round({1: "continue", 3: "continue"})
    r = p.next_round()
    assert r.kind == "prefill" and r.rows == [2]
    p.complete_round({2: "continue"})
