"""Speculative decoding on the CPU oracle engine: providers, verification rules, transaction, controller."""
import numpy as np
import pytest

from sllm_b200.engine import speculative as SP
from sllm_b200.engine.engine import build_engine
from sllm_b200.models import config as MC


def _engine(seed=1):
    cfg = MC.tiny_llama()
    cfg.max_context = 256
    return build_engine(cfg, "cpu", seed=seed, num_pages=128, max_batch=4, use_cuda_graphs=False)


def _plain(eng, prompt, n):
    return eng.generate([prompt], n)[0]


def test_ngram_provider():
    p = SP.NgramDraftProvider(order=3, width=4)
    assert p.propose([1, 2, 3, 4, 5, 9, 1, 2, 3]) == [4, 5, 9, 1]
    assert p.propose([7, 8, 9]) == []
    assert p.propose([5, 6, 5]) == [6, 5]          # falls back to a shorter n-gram
    assert p.propose([1, 2, 3, 4, 1, 2, 3], width=2) == [4, 1]
    with pytest.raises(SP.SpeculativeError):
        SP.NgramDraftProvider(width=9)


def test_verification_rules():
    assert SP.verify_greedy([5, 6, 7], [5, 6, 9, 4]) == (2, 9)
    assert SP.verify_greedy([5, 6, 7], [5, 6, 7, 4]) == (3, 4)
    assert SP.verify_greedy([], [8]) == (0, 8)
    assert SP.verify_greedy([5, 6], [1, 2, 3], forced_accept=[True, False]) == (1, 2)
    with pytest.raises(SP.SpeculativeError):
        SP.verify_greedy([1], [1])
    # stochastic: identical distributions always accept; disjoint ones always reject and resample from p
    V = 8
    q = np.full((2, V), 1.0 / V)
    assert SP.verify_stochastic([3, 4], q, np.full((3, V), 1.0 / V), [0.99, 0.99], 0.0)[0] == 2
    q2 = np.zeros((1, V)); q2[0, 3] = 1.0
    p2 = np.zeros((2, V)); p2[0, 5] = 1.0; p2[1, 1] = 1.0
    assert SP.verify_stochastic([3], q2, p2, [0.0], 0.5) == (0, 5)
    # the rule preserves the target distribution: empirical check on a 3-symbol alphabet
    rng = np.random.default_rng(0)
    q3 = np.array([[0.7, 0.2, 0.1]]); p3 = np.array([[0.2, 0.5, 0.3], [1 / 3, 1 / 3, 1 / 3]])
    counts = np.zeros(3)
    for _ in range(20000):
        d = int(rng.choice(3, p=q3[0]))
        n, t = SP.verify_stochastic([d], q3, p3, [rng.random()], rng.random())
        counts[d if n == 1 else t] += 1
    assert np.abs(counts / counts.sum() - p3[0]).max() < 0.015


def test_speculative_equals_plain_greedy_with_ngram():
    eng = _engine()
    prompt = [5, 6, 7, 8] * 6
    want = _plain(eng, prompt, 24)
    dec = SP.SpeculativeDecoder(eng, SP.NgramDraftProvider(3, 4), width=4)
    s = eng.new_sequence(prompt)
    first = eng.prefill([s])[0]
    s.tokens.append(first)
    got = [first]
    while len(got) < 24:
        got += dec.step([s], [24 - len(got)])[0]
    assert got[:24] == want
    assert dec.acct.steps < 23 or dec.acct.accepted == 0        # accepted drafts save target steps
    assert s.num_computed == len(s.tokens) - 1
    eng.free_sequence(s)
    assert eng.cache.pool.stats()["sequences"] == 0


def test_external_draft_same_model_accepts_everything():
    eng, draft = _engine(1), _engine(1)                  # identical weights: every draft token is right
    prov = SP.ExternalDraftProvider(draft, width=4, target_vocab=eng.cfg.vocab)
    dec = SP.SpeculativeDecoder(eng, prov, width=4)
    prompts = [[3, 9, 27, 81, 11], [100, 200, 300]]
    want = [_plain(eng, p, 13) for p in prompts]
    seqs = [eng.new_sequence(p) for p in prompts]
    firsts = eng.prefill(seqs)
    got = [[f] for f in firsts]
    for s, f in zip(seqs, firsts):
        s.tokens.append(f)
    while min(len(g) for g in got) < 13:
        outs = dec.step(seqs, [13 - len(g) for g in got])
        for g, o in zip(got, outs):
            g += o
    assert [g[:13] for g in got] == want
    assert dec.acct.acceptance_rate == 1.0 and dec.acct.tokens_per_step > 2
    for s in seqs:
        dec.release(s)
        eng.free_sequence(s)
    assert draft.cache.pool.stats()["sequences"] == 0
    with pytest.raises(SP.SpeculativeError):
        SP.ExternalDraftProvider(draft, width=4, target_vocab=eng.cfg.vocab + 1)


def test_forced_acceptance_and_abort():
    eng = _engine()
    dec = SP.SpeculativeDecoder(eng, SP.NgramDraftProvider(2, 4), width=4, forced_accept_p=0.7, seed=3)
    s = eng.new_sequence([1, 2, 3, 1, 2, 3, 1, 2])
    s.tokens.append(eng.prefill([s])[0])
    s.tokens[-1] = 3                                   # keep the n-gram going so that drafts are non-empty
    n0 = len(s.tokens)
    for _ in range(6):
        dec.step([s])
    a = dec.acct
    assert a.drafted > 0 and a.emitted == len(s.tokens) - n0 and 0 < a.accepted <= a.drafted
    # a failing verify leaves tokens and KV length as they were
    t = SP.SpeculativeTransaction(eng, s, [7, 7, 7])
    assert len(s.tokens) == t.base_len + 3
    t.abort()
    assert len(s.tokens) == t.base_len and s.num_computed == t.base_len - 1 and t.state == "aborted"
    with pytest.raises(SP.SpeculativeError):
        t.commit()
    eng.free_sequence(s)


def test_engine_loop_speculative_lane_matches_plain():
    import time
    from sllm_b200.engine.scheduler import EngineLoop, GenRequest
    eng = _engine()
    prompt = [5, 6, 7, 8] * 6
    want = _plain(eng, prompt, 20)
    loop = EngineLoop(eng)
    loop.speculative = SP.SpeculativeDecoder(eng, SP.NgramDraftProvider(3, 4), width=4)
    toks, done = [], []
    loop.submit(GenRequest(prompt=prompt, max_new_tokens=20, on_token=lambda t, s: toks.append(t) or True, on_done=done.append))
    # a request that stops early on a stop token inside a block
    toks2, done2 = [], []
    loop.submit(GenRequest(prompt=prompt, max_new_tokens=20, stop_tokens=(want[7],), on_token=lambda t, s: toks2.append(t) or True,
                           on_done=done2.append))
    for _ in range(4000):
        if done and done2:
            break
        time.sleep(0.005)
    loop.shutdown(2.0)
    assert done == ["length"] and toks == want
    assert done2 == ["stop"] and toks2 == want[:want.index(want[7]) + 1]
    assert loop.speculative.acct.steps > 0
    assert eng.cache.pool.stats()["sequences"] == 0
