"""Multi-token-prediction head: exact equivalence with target-only greedy decoding, KV reuse of the head, hidden log."""
import pytest
import torch

from sllm_b200.engine.engine import build_engine
from sllm_b200.engine.speculative import SpeculativeDecoder
from sllm_b200.models import config as mc
from sllm_b200.models.mtp import MtpDraftProvider, MtpHead, init_random_mtp_weights


def _engine(dev="cpu", seed=0, max_batch=4):
    cfg = mc.tiny_llama()
    cfg.max_context = 256
    return build_engine(cfg, dev, seed=seed, max_batch=max_batch, use_cuda_graphs=False)


def _target_only(prompts, steps, dev="cpu"):
    eng = _engine(dev)
    return eng.generate(prompts, steps)


def _spec(prompts, steps, width, dev="cpu", forced=None):
    eng = _engine(dev)
    head = MtpHead(eng, init_random_mtp_weights(eng.cfg, dev, seed=3))
    prov = MtpDraftProvider(head, width=width)
    dec = SpeculativeDecoder(eng, prov, width=width, forced_accept_p=forced)
    seqs = [eng.new_sequence(p) for p in prompts]
    first = eng.prefill(seqs)
    outs = [[t] for t in first]
    for s, t in zip(seqs, first):
        s.tokens.append(t)
    while min(len(o) for o in outs) < steps:
        live = [i for i, o in enumerate(outs) if len(o) < steps]
        new = dec.step([seqs[i] for i in live], [steps - len(outs[i]) for i in live])
        for i, toks in zip(live, new):
            outs[i].extend(toks)
    for s in seqs:
        dec.release(s)
    return [o[:steps] for o in outs], dec, head


def _prompts():
    g = torch.Generator().manual_seed(5)
    return [torch.randint(0, 1024, (n,), generator=g).tolist() for n in (9, 23, 16)]


@pytest.mark.parametrize("width", [1, 2, 4])
def test_mtp_speculation_is_exact(width):
    prompts = _prompts()
    want = _target_only(prompts, 20)
    got, dec, head = _spec(prompts, 20, width)
    assert got == want
    assert dec.acct.drafted > 0 and dec.acct.steps > 0
    # every head sequence was released
    assert head.engine.cache.pool.stats()["sequences"] == 0


def test_mtp_head_kv_reuse_matches_recompute():
    """Drafts from the incrementally maintained head equal drafts of a fresh head that replays the whole history."""
    prompts = _prompts()[:2]
    eng = _engine()
    w = init_random_mtp_weights(eng.cfg, "cpu", seed=3)
    prov = MtpDraftProvider(MtpHead(eng, w), width=3)
    seqs = [eng.new_sequence(p) for p in prompts]
    for s, t in zip(seqs, eng.prefill(seqs)):
        s.tokens.append(t)
    # keep full copies of the hidden rows: take_hidden consumes the log
    full = {id(s): eng.take_hidden(s, 0, s.num_computed).clone() for s in seqs}
    for s in seqs:
        eng._hidden_log[s.seq_id] = [(0, full[id(s)])]
    d1 = prov.propose_seqs(seqs, 3)
    # two plain target steps, then draft again: the head catches up on two positions only
    for _ in range(2):
        rows = eng.extend(seqs)
        for s, r in zip(seqs, rows):
            s.tokens.append(r[-1])
    for s in seqs:
        full[id(s)] = torch.cat([full[id(s)], eng.take_hidden(s, full[id(s)].shape[0], s.num_computed)], 0)
        eng._hidden_log[s.seq_id] = [(full[id(s)].shape[0] - 2, full[id(s)][-2:])]
    d2 = prov.propose_seqs(seqs, 3)
    fresh = MtpDraftProvider(MtpHead(eng, w), width=3)
    for s in seqs:
        eng._hidden_log[s.seq_id] = [(0, full[id(s)])]
    d3 = fresh.propose_seqs(seqs, 3)
    assert d2 == d3
    assert all(len(d) == 3 for d in d1 + d2)


def test_hidden_log_rollback_and_take():
    eng = _engine()
    eng.keep_hidden = True
    s = eng.new_sequence(list(range(1, 12)))
    s.tokens.append(eng.prefill([s])[0])
    s.tokens.extend([5, 6, 7])
    eng.extend([s])
    assert s.num_computed == 15
    eng.rollback(s, 13)
    h = eng.take_hidden(s, 3, 13)
    assert h.shape == (10, eng.cfg.d_model)
    with pytest.raises(ValueError):
        eng.take_hidden(s, 13, 14)


@pytest.mark.gpu
def test_mtp_speculation_is_exact_gpu():
    cfg = mc.tiny_llama()
    cfg.weight_format, cfg.kv_format, cfg.max_context = "bf16", "bf16", 256
    prompts = _prompts()

    def run(spec):
        eng = build_engine(cfg, "cuda", seed=0, max_batch=4)
        if not spec:
            return eng.generate(prompts, 16)
        head = MtpHead(eng, init_random_mtp_weights(cfg, "cuda", seed=3))
        dec = SpeculativeDecoder(eng, MtpDraftProvider(head, width=2), width=2)
        seqs = [eng.new_sequence(p) for p in prompts]
        outs = [[t] for t in eng.prefill(seqs)]
        for s, o in zip(seqs, outs):
            s.tokens.append(o[0])
        while min(len(o) for o in outs) < 16:
            live = [i for i, o in enumerate(outs) if len(o) < 16]
            for i, toks in zip(live, dec.step([seqs[i] for i in live], [16 - len(outs[i]) for i in live])):
                outs[i].extend(toks)
        return [o[:16] for o in outs]

    assert run(True) == run(False)


def test_mtp_component_through_gguf_and_cli(capsys, tmp_path):
    """`--with-mtp` writes the component, the loader reads it back bit-exactly, and `sllm generate
    --mtp-draft-width` yields the tokens of plain greedy generation."""
    import json
    from sllm_b200.cli import convert, main as sllm
    from sllm_b200.formats import gguf as G
    from sllm_b200.models import loader
    g, l = str(tmp_path / "m.gguf"), str(tmp_path / "m.lock.json")
    assert convert.main(["--kind", "random-llama", "--artifact", "tiny-llama", "--weight-format", "fp32", "--output", g,
                         "--derived-lock", l, "--with-mtp", "--seed", "4"]) == 0
    f = G.verify_gguf(g, G.read_derived_lock(l))
    cfg = loader.config_from_gguf(f)
    w = loader.load_mtp_gguf(f, cfg, "cpu")
    want = init_random_mtp_weights(cfg, "cpu", seed=5)
    assert torch.equal(w.fc.w, want.fc.w) and torch.equal(w.layer.qkv.w, want.layer.qkv.w)
    assert torch.equal(w.norm, want.norm) and torch.equal(w.norm_hidden, want.norm_hidden)

    def run(argv):
        capsys.readouterr()
        rc = sllm.main(argv)
        return rc, [json.loads(x) for x in capsys.readouterr().out.strip().splitlines() if x.strip()]

    src = ["--gguf", g, "--derived-lock", l, "--cpu"]
    rc, plain = run(["generate", *src, "--prompt", "hello there", "--max-new-tokens", "12"])
    rc2, spec = run(["generate", *src, "--prompt", "hello there", "--max-new-tokens", "12", "--mtp-draft-width", "2"])
    assert rc == 0 and rc2 == 0 and spec[0]["tokens"] == plain[0]["tokens"]
    # a file without the component refuses the flag
    g2, l2 = str(tmp_path / "n.gguf"), str(tmp_path / "n.lock.json")
    assert convert.main(["--kind", "random-llama", "--artifact", "tiny-llama", "--weight-format", "fp32", "--output", g2,
                         "--derived-lock", l2]) == 0
    rc3, _ = run(["generate", "--gguf", g2, "--derived-lock", l2, "--cpu", "--prompt", "x", "--mtp-draft-width", "2"])
    assert rc3 != 0


def test_mtp_after_prefix_fork_is_exact():
    """A sequence forked from a cached prefix logs hidden rows only for the tokens it computed itself: the head
    starts there, and the output still equals target-only decoding."""
    prompts = _prompts()
    want = _target_only([prompts[1]], 12)[0]
    eng = _engine()
    head = MtpHead(eng, init_random_mtp_weights(eng.cfg, "cpu", seed=3))
    dec = SpeculativeDecoder(eng, MtpDraftProvider(head, width=2), width=2)
    donor = eng.new_sequence(prompts[1][:17])
    eng.prefill([donor])
    s = eng.fork_sequence(donor, prompts[1])
    assert s.num_computed >= 16
    out = [eng.prefill([s])[0]]
    s.tokens.append(out[0])
    while len(out) < 12:
        out.extend(dec.step([s], [12 - len(out)])[0])
    assert out[:12] == want
