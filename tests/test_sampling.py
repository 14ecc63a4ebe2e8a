"""Sampler contract on CPU: parameter ranges, RNG stream, profile sampler golden cases, chain stages,
snapshot / restore, and the host mirror of the device selector."""
import math

import numpy as np
import pytest

from sllm_b200.engine import sampling as S


class FixedUniform:
    def __init__(self, u):
        self.u = u

    def next_unit(self):
        return self.u


def _restated_profile_sampler(logits, t, top_p, pp, fp, hist, u):
    """Independent restatement: penalties on seen ids, temperature, stable order, smallest top-p prefix, inverse CDF."""
    lg = np.asarray(logits, dtype=np.float64).copy()
    for tok in set(hist):
        lg[tok] -= pp + fp * hist.count(tok)
    lg = lg / t
    p = np.exp(lg - lg.max())
    p /= p.sum()
    order = sorted(range(len(p)), key=lambda i: (-p[i], i))
    cum, keep = 0.0, []
    for i in order:
        keep.append(i)
        cum += p[i]
        if cum >= top_p:
            break
    mass = sum(p[i] for i in keep)
    acc = 0.0
    for i in keep:
        acc += p[i]
        if u * mass < acc:
            return i
    return keep[-1]


@pytest.mark.parametrize("logits,t,top_p,pp,fp,hist,u", [
    ([0.2, 1.4, -0.7, 0.9, 1.4], 0.8, 0.85, 0.0, 0.0, [], 0.41),
    ([1.0, 3.0, 2.0, 0.5], 1.3, 1.0, 0.6, 0.4, [1, 1, 2], 0.07),
    ([0.5, 0.5, 0.5], 1.0, 0.01, 0.0, 0.0, [], 0.99),
    ([-2.0, 4.0, 1.5, 1.5, 0.0, 3.5], 1.9, 0.95, -0.5, 0.2, [5, 5], 0.66),
])
def test_profile_sampler_matches_restatement(logits, t, top_p, pp, fp, hist, u):
    """(The reference's own golden cases are read from its fixture file in test_reference_fixtures.py.)"""
    s = S.ProfileSampler(S.SamplingParams(t, top_p, pp, fp), hist)
    want = _restated_profile_sampler(logits, t, top_p, pp, fp, hist, u)
    assert s.select(0, np.array(logits, dtype=np.float32), FixedUniform(u)) == want


def test_parameter_ranges():
    for bad in (dict(temperature=2.1), dict(temperature=-0.1), dict(top_p=1.5), dict(presence_penalty=3),
                dict(frequency_penalty=-2.5), dict(temperature=float("nan"))):
        with pytest.raises(S.SamplingError):
            S.SamplingParams(**bad)
    assert not S.SamplingParams().requires_logits


def test_splitmix_stream_and_positional_draw():
    r = S.SplitMix64(12345)
    first = [r.next_unit() for _ in range(5)]
    assert all(0.0 <= x < 1.0 for x in first)
    assert first == [S.SplitMix64.unit_at(12345, i) for i in range(5)]
    # published SplitMix64 vector: seed 0 -> first output 0xe220a8397b1dcdaf
    assert S.SplitMix64(0).next_u64() == 0xE220A8397B1DCDAF
    assert S.derive_choice_seed(7, 0) == 7 and S.derive_choice_seed(7, 1) != S.derive_choice_seed(7, 2)


def test_greedy_never_touches_logits_or_rng():
    s = S.ProfileSampler(S.SamplingParams())
    assert s.select(17, None, None) == 17
    with pytest.raises(S.SamplingError):
        s.select(5, np.zeros(3, dtype=np.float32), None)


def test_special_values():
    s = S.ProfileSampler(S.SamplingParams(1.0))
    with pytest.raises(S.SamplingError):
        s.select(0, np.array([0.0, np.nan], dtype=np.float32), FixedUniform(0.1))
    assert s.select(0, np.array([0.0, np.inf, 3.0, np.inf], dtype=np.float32), FixedUniform(0.6)) == 3
    with pytest.raises(S.SamplingError):
        s.select(0, np.array([-np.inf, -np.inf], dtype=np.float32), FixedUniform(0.1))


def test_chain_stages():
    lg = np.array([1.0, 3.0, 2.0, 0.5, 2.9], dtype=np.float32)
    # top-k 1 is greedy whatever the draw
    ch = S.SamplerChain(S.SamplerChainConfig(S.SamplingParams(1.0), top_k=1), seed=1)
    assert ch.select(lg).token == 1
    # logit bias and the validity mask
    ch = S.SamplerChain(S.SamplerChainConfig(S.SamplingParams(0.0), logit_bias=[(3, 50.0)]), seed=1)
    assert ch.select(lg).token == 3
    mask = np.array([1, 0, 1, 1, 0], dtype=np.uint8)
    ch = S.SamplerChain(S.SamplerChainConfig(S.SamplingParams(0.0)), seed=1)
    assert ch.select(lg, valid_mask=mask).token == 2
    # ignore-eos removes the token
    ch = S.SamplerChain(S.SamplerChainConfig(S.SamplingParams(0.0), ignore_eos_token=1), seed=1)
    assert ch.select(lg).token == 4
    # repeat penalty pushes a repeated positive logit down
    ch = S.SamplerChain(S.SamplerChainConfig(S.SamplingParams(0.0), repeat_penalty=2.0), prior_tokens=[1], seed=1)
    assert ch.select(lg).token == 4
    # min-p keeps only tokens within a factor of the best
    ch = S.SamplerChain(S.SamplerChainConfig(S.SamplingParams(1.0), min_p=0.5), seed=3)
    assert {ch.select(lg).token for _ in range(50)} <= {1, 4}
    # logprobs
    ch = S.SamplerChain(S.SamplerChainConfig(S.SamplingParams(0.0), return_logprobs=True, top_logprobs=2), seed=1)
    sel = ch.select(lg)
    z = lg.astype(np.float64)
    want = z - math.log(np.exp(z).sum())
    assert sel.token == 1 and abs(sel.logprob - want[1]) < 1e-6
    assert [t for t, _ in sel.top_logprobs] == [1, 4]
    with pytest.raises(S.SamplingError):
        S.SamplerChain(S.SamplerChainConfig(S.SamplingParams(1.0), logit_bias=[(1, 200.0)]))


def test_chain_distribution_and_snapshot():
    lg = np.log(np.array([0.1, 0.2, 0.3, 0.4], dtype=np.float64)).astype(np.float32)
    ch = S.SamplerChain(S.SamplerChainConfig(S.SamplingParams(1.0)), seed=99)
    draws = [ch.select(lg).token for _ in range(4000)]
    freq = np.bincount(draws, minlength=4) / 4000
    assert np.abs(freq - [0.1, 0.2, 0.3, 0.4]).max() < 0.03
    ch.accept(2)
    blob = ch.snapshot()
    nxt = [ch.select(lg).token for _ in range(10)]
    ch2 = S.SamplerChain(S.SamplerChainConfig(S.SamplingParams(1.0)), seed=5)
    ch2.restore(blob)
    assert [ch2.select(lg).token for _ in range(10)] == nxt
    with pytest.raises(S.SamplingError):
        ch2.restore(b"\x00\x00")


def test_dry_and_mirostat_run():
    lg = np.zeros(16, dtype=np.float32)
    lg[5] = 4.0
    hist = [1, 2, 3, 5, 9, 1, 2, 3]   # "1 2 3" was followed by 5 before: DRY penalises 5
    ch = S.SamplerChain(S.SamplerChainConfig(S.SamplingParams(0.0), dry=S.DryConfig(5.0, 1.75, 2)), prior_tokens=hist)
    assert ch.select(lg).token != 5
    ch = S.SamplerChain(S.SamplerChainConfig(S.SamplingParams(1.0), mirostat=S.MirostatConfig(2)), seed=4)
    mu0 = ch.mu
    toks = [ch.select(np.random.default_rng(0).normal(size=64).astype(np.float32)).token for _ in range(5)]
    assert all(0 <= t < 64 for t in toks) and ch.mu != mu0


def test_reference_selector_matches_profile_sampler_order():
    rng = np.random.default_rng(7)
    for trial in range(50):
        lg = rng.normal(0, 2, 300).astype(np.float32)
        row = (0.8, 0.9, 0.0, 0, 1000 + trial, 3)
        tok, status, lp = S.reference_select(lg, row)
        assert status == 0
        s = S.ProfileSampler(S.SamplingParams(0.8, 0.9))
        want = s.select(0, lg, FixedUniform(S.SplitMix64.unit_at(1000 + trial, 3)))
        assert tok == want
    assert S.reference_select(np.array([np.nan, 1.0], dtype=np.float32), (1.0, 1.0, 0.0, 0, 1, 0))[1] == 1
    assert S.reference_select(np.zeros(4, dtype=np.float32), (1.0, 1.0, 0.0, 0, 1, 0), mask=np.zeros(4))[1] == 2


# ---------------------------------------------------------------------------------------------- native host sampler
def _random_chain_config(rng):
    from sllm_b200.engine import sampling as S
    pick = lambda p: rng.random() < p
    params = S.SamplingParams(temperature=float(rng.choice([0.0, 0.3, 0.8, 1.5])), top_p=float(rng.choice([1.0, 0.95, 0.7])),
                              presence_penalty=float(rng.choice([0.0, 0.5])), frequency_penalty=float(rng.choice([0.0, 0.3])))
    cfg = S.SamplerChainConfig(params=params)
    if pick(0.4):
        cfg.top_k = int(rng.integers(1, 60))
    if pick(0.4):
        cfg.min_p = float(rng.choice([0.01, 0.1]))
    if pick(0.3):
        cfg.typical_p = float(rng.choice([0.5, 0.9]))
    if pick(0.4):
        cfg.repeat_penalty, cfg.repeat_last_n = float(rng.choice([0.8, 1.2])), int(rng.integers(1, 40))
    if pick(0.3) and params.temperature > 0:
        cfg.dynamic_temperature = (0.3, 1.5)
    if pick(0.3):
        cfg.ignore_eos_token = 7
    if pick(0.4):
        toks = rng.choice(400, size=5, replace=False)
        cfg.logit_bias = [(int(t), float(b)) for t, b in zip(toks, rng.uniform(-5, 5, 5))]
    if pick(0.3):
        cfg.dry = S.DryConfig(multiplier=0.8, base=1.75, allowed_length=2, sequence_breakers=[[3], [4, 5]], penalty_last_n=int(rng.choice([0, 30])))
    if pick(0.3) and params.temperature > 0:
        cfg.xtc = S.XtcConfig(probability=0.6, threshold=0.05, min_keep=1)
    if pick(0.25):
        cfg.mirostat = S.MirostatConfig(mode=int(rng.choice([1, 2])), tau=4.0, eta=0.2, mu=8.0)
    if pick(0.5):
        cfg.return_logprobs, cfg.top_logprobs = True, int(rng.integers(0, 5))
    return cfg


@pytest.mark.parametrize("seed", range(40))
def test_native_host_sampler_matches_the_python_chain(seed):
    """The C++ chain (csrc/host/sampler.cpp) against the NumPy chain it restates: same tokens, same random-stream and
    Mirostat state after every step, log-probabilities to rounding, for random stage combinations, histories with
    repetitions (DRY / repeat penalty), grammar masks and +inf / -inf logits."""
    from sllm_b200.engine import sampling as S
    rng = np.random.default_rng(seed)
    cfg = _random_chain_config(rng)
    vocab = int(rng.integers(400, 3000))
    prior = [int(t) for t in rng.integers(0, 40, size=int(rng.integers(0, 60)))]
    chains = []
    for native in (True, False):
        S.use_native_sampler(native)
        chains.append(S.SamplerChain(cfg, prior_tokens=prior, seed=1234 + seed))
    try:
        for step in range(6):
            lg = (rng.standard_normal(vocab) * 3).astype(np.float32)
            if step == 2:
                lg[rng.integers(0, vocab, 3)] = -np.inf
            if step == 4 and cfg.params.temperature > 0 and cfg.mirostat is None:
                lg[[11, 12]] = np.inf
            mask = (rng.random(vocab) < 0.7) if step % 3 == 1 else None
            if mask is not None:
                mask[int(np.argmax(lg))] = True
            out = []
            for native, ch in zip((True, False), chains):
                S.use_native_sampler(native)
                out.append(ch.select(lg, valid_mask=mask))
            a, b = out
            assert a.token == b.token, (seed, step)
            assert (chains[0].rng.state, chains[0].draws) == (chains[1].rng.state, chains[1].draws)
            assert chains[0].mu == pytest.approx(chains[1].mu, rel=1e-12, abs=1e-12)
            if cfg.return_logprobs or cfg.top_logprobs:
                # (+inf logits make the log-probabilities NaN in both forms)
                assert np.allclose(a.logprob, b.logprob, rtol=1e-9, atol=1e-9, equal_nan=True)
                if not np.isnan(b.logprob):
                    assert [t for t, _ in a.top_logprobs] == [t for t, _ in b.top_logprobs]
                    assert np.allclose([v for _, v in a.top_logprobs], [v for _, v in b.top_logprobs], rtol=1e-9, atol=1e-9)
            for ch in chains:
                ch.accept(a.token)
    finally:
        S.use_native_sampler(True)


def test_native_host_sampler_errors_and_snapshot():
    from sllm_b200.engine import sampling as S
    S.use_native_sampler(True)
    cfg = S.SamplerChainConfig(params=S.SamplingParams(temperature=0.7, top_p=0.9), typical_p=0.8)
    ch = S.SamplerChain(cfg, seed=5)
    lg = np.zeros(64, dtype=np.float32)
    lg[9] = np.nan
    with pytest.raises(S.SamplingError, match="NaN logit at token 9"):
        ch.select(lg)
    with pytest.raises(S.SamplingError, match="empty distribution"):
        ch.select(np.zeros(64, dtype=np.float32), valid_mask=np.zeros(64, dtype=bool))
    # a restored snapshot continues the same stream through the native path
    lg = np.random.default_rng(0).standard_normal(64).astype(np.float32)
    first = [ch.select(lg).token for _ in range(3)]
    blob = ch.snapshot()
    nxt = [ch.select(lg).token for _ in range(4)]
    ch2 = S.SamplerChain(cfg, seed=99)
    ch2.restore(blob)
    assert [ch2.select(lg).token for _ in range(4)] == nxt and len(first) == 3
