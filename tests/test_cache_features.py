"""Prefix cache, context shift and session checkpoints on the CPU oracle engine."""
import os

import pytest
import torch

from sllm_b200.cache import checkpoint as CK
from sllm_b200.cache.context_shift import ContextPolicy, ContextShiftError, WindowState, apply_shift
from sllm_b200.cache.prefix import PrefixCache, PrefixIdentity
from sllm_b200.engine.engine import build_engine
from sllm_b200.engine.scheduler import EngineLoop, GenRequest
from sllm_b200.models import config as MC


def _engine(max_context=256, pages=256):
    cfg = MC.tiny_llama()
    cfg.max_context = max_context
    return build_engine(cfg, "cpu", seed=1, num_pages=pages, max_batch=4, use_cuda_graphs=False)


def _greedy(eng, prompt, n, src=None):
    s = eng.fork_sequence(src, prompt) if src is not None else eng.new_sequence(prompt)
    out = []
    t = eng.prefill([s])[0]
    for _ in range(n):
        out.append(t)
        s.tokens.append(t)
        t = eng.decode([s])[0]
    eng.free_sequence(s)
    return out


def test_prefix_cache_hit_is_exact_and_bounded():
    eng = _engine()
    pc = PrefixCache(eng, PrefixIdentity(model="m"), max_entries=2, min_tokens=8)
    base = list(range(3, 45))                               # 42 tokens: 2 full pages + 10
    want = _greedy(eng, base + [7, 8, 9], 6)
    s = eng.new_sequence(base)
    eng.prefill([s])
    assert pc.publish(s, len(base))
    assert not pc.publish(s, len(base))                     # redundant
    eng.free_sequence(s)
    free0 = eng.cache.pool.stats()["free"]
    lease = pc.lookup(base + [7, 8, 9])
    assert lease is not None and lease.matched == len(base)
    got = _greedy(eng, base + [7, 8, 9], 6, src=lease)
    lease.release()
    assert got == want
    assert eng.cache.pool.stats()["free"] == free0
    # a differing identity, or too short a match, misses
    assert pc.lookup(base, PrefixIdentity(model="other")) is None
    assert pc.lookup(base[:5] + [999] * 20) is None
    part = pc.lookup(base[:20] + [999] * 20)
    assert part.matched == 20
    part.release()
    # LRU eviction under the entry bound; a leased entry is never evicted
    held = pc.lookup(base)
    for k in range(3):
        p = [100 + k] * 20
        s = eng.new_sequence(p)
        eng.prefill([s])
        pc.publish(s, 20)
        eng.free_sequence(s)
    st = pc.stats()
    assert st["entries"] <= 2 and st["evicted"] >= 1
    again = pc.lookup(base)
    assert again is not None
    again.release()
    held.release()
    pc.clear()
    assert pc.stats()["entries"] == 0
    assert eng.cache.pool.stats()["sequences"] == 0


def test_prefix_cache_through_engine_loop():
    eng = _engine()
    pc = PrefixCache(eng, min_tokens=8)
    loop = EngineLoop(eng, prefix_cache=pc)
    prompt = list(range(5, 40))
    outs = []
    for _ in range(2):
        toks, done = [], []
        req = GenRequest(prompt=prompt + [1, 2], max_new_tokens=5, on_token=lambda t, s: toks.append(t) or True,
                         on_done=done.append, prefix_seq=pc.lookup(prompt + [1, 2]))
        loop.submit(req)
        for _ in range(2000):
            if done:
                break
            import time; time.sleep(0.005)
        assert done == ["length"]
        outs.append((toks, req.prefix_hit_tokens))
    loop.shutdown(2.0)
    assert outs[0][0] == outs[1][0]
    assert outs[0][1] == 0 and outs[1][1] >= 32
    assert pc.stats()["hits"] == 1


def test_context_policy_decisions():
    kp = ContextPolicy.keep_prefix_recent(4, 8)
    st = WindowState(30, 30, 0)
    assert not kp.plan(st, 32, 1).shift
    d = kp.plan(WindowState(31, 31, 0), 32, 1)
    assert d.shift and d.prefix == (0, 4) and d.recent == (23, 31) and d.new_state == WindowState(12, 31, 1)
    assert d.retained_token_ids(list(range(31))) == [0, 1, 2, 3] + list(range(23, 31))
    assert d.retained_absolute_positions() == [0, 1, 2, 3] + list(range(23, 31))
    dis = ContextPolicy.disabled()
    assert not dis.plan(WindowState(31, 31, 0), 32, 1).shift          # exact fill is allowed
    with pytest.raises(ContextShiftError):
        dis.plan(WindowState(32, 32, 0), 32, 1)
    with pytest.raises(ContextShiftError):
        ContextPolicy.keep_prefix_recent(20, 20).plan(WindowState(31, 31, 0), 32, 1)     # overlap
    with pytest.raises(ContextShiftError):
        ContextPolicy.keep_prefix_recent(0, 0)
    i = kp.plan_initial(100, 32)
    assert i.shift and i.new_state == WindowState(12, 100, 1) and i.recent == (92, 100)
    assert not kp.plan_initial(20, 32).shift
    with pytest.raises(ContextShiftError):
        dis.plan_initial(100, 32)


def test_context_shift_generation_continues():
    eng = _engine(max_context=48)
    loop = EngineLoop(eng, context_policy=ContextPolicy.keep_prefix_recent(4, 12))
    toks, done = [], []
    req = GenRequest(prompt=list(range(3, 33)), max_new_tokens=40, on_token=lambda t, s: toks.append(t) or True,
                     on_done=done.append)
    loop.submit(req)
    import time
    for _ in range(4000):
        if done:
            break
        time.sleep(0.005)
    loop.shutdown(2.0)
    assert done == ["length"] and len(toks) == 40 and req.shift_count >= 1
    # the shifted state equals a fresh prefill of the retained tokens: replay the last shift by hand
    s = eng.new_sequence(list(range(3, 50)))
    eng.prefill([s])
    d = ContextPolicy.keep_prefix_recent(4, 12).plan(WindowState(47, 47, 0), 48, 1)
    kept = d.retained_token_ids(s.tokens)
    s2 = apply_shift(eng, s, d)
    assert s2.tokens == kept and s2.num_computed == len(kept) - 1
    a = eng.decode([s2])[0]
    f = eng.new_sequence(kept)
    b = eng.prefill([f])[0]
    assert a == b
    eng.free_sequence(s2); eng.free_sequence(f)


def test_checkpoint_roundtrip_and_tamper(tmp_path):
    eng = _engine()
    prompt = list(range(9, 60))
    s = eng.new_sequence(prompt)
    t = eng.prefill([s])[0]
    s.tokens.append(t)
    nxt = eng.decode([s])[0]
    ident = CK.CheckpointIdentity(model="sha256:abc", plan="p1", tokenizer="byte")
    # checkpoint after the prefill state: tokens include the sampled one, KV covers the first 52
    ck = CK.capture(eng, s, ident, conversation='[{"role":"user","content":"hi"}]', sampler_state={"seed": 5})
    store = CK.CheckpointStore(str(tmp_path / "ck"), max_bytes=64 << 20)
    n = store.save("sess-1", ck)
    assert store.usage_bytes() == n and store.list() == ["sess-1"]
    eng.free_sequence(s)
    back = store.load("sess-1", CK.CheckpointIdentity(model="sha256:abc", plan="p1", kv_layout=CK.kv_layout_id(eng.cache),
                                                     tokenizer="byte"))
    assert back.tokens == prompt + [t] and back.sampler_state == {"seed": 5}
    r = CK.restore(eng, back)
    r.tokens.append(nxt)
    r.num_computed = min(r.num_computed, len(r.tokens) - 1)
    eng.rollback(r, len(r.tokens))          # no-op truncate keeps the pool and the sequence consistent
    s3 = eng.new_sequence(prompt + [t, nxt])
    want = eng.prefill([s3])[0]
    got = eng.decode([r])[0]
    assert got == want
    eng.free_sequence(r); eng.free_sequence(s3)
    with pytest.raises(CK.CheckpointError, match="identity mismatch"):
        store.load("sess-1", CK.CheckpointIdentity(model="other", plan="p1", kv_layout=CK.kv_layout_id(eng.cache),
                                                    tokenizer="byte"))
    raw = bytearray(ck.encode())
    for pos in (9, 100, len(raw) - 5):
        bad = bytearray(raw); bad[pos] ^= 0x40
        with pytest.raises(CK.CheckpointError):
            CK.SessionCheckpoint.decode(bytes(bad))
    with pytest.raises(CK.CheckpointError):
        CK.SessionCheckpoint.decode(bytes(raw[:-32]))
    for bad_id in ("../x", "", "a/b", ".hidden"):
        with pytest.raises(CK.CheckpointError):
            store.save(bad_id, ck)
    small = CK.CheckpointStore(str(tmp_path / "small"), max_bytes=1024)
    with pytest.raises(CK.CheckpointError, match="quota"):
        small.save("a", ck)
    assert store.delete("sess-1") and not store.delete("sess-1")


def test_paged_kv_offset_matches_tensor_layout():
    from sllm_b200.cache.paged import paged_kv_offset
    eng = _engine()
    c = eng.cache
    L, two, pages, hkv, page, hd = c.values.shape
    assert (hkv, page, hd) == (c.spec.kv_heads, c.spec.page_size, c.spec.head_dim)
    plane = c.values[0, 0]
    flat = plane.reshape(-1)
    page_list = [5, 2, 9]
    for tok, head, ch in [(0, 0, 0), (17, 1, 3), (40, 1, 63), (33, 0, 7)]:
        off = paged_kv_offset(page_list, tok, head, ch, page, hkv, hd, elem_bytes=1)
        want = plane[page_list[tok // page], head, tok % page, ch].data_ptr() - plane.data_ptr()
        assert off * plane.element_size() == want


def test_rollback_into_a_shared_page_copies_the_tail_before_the_next_append():
    """A fork at a page boundary shares whole pages by reference count; rolling the child back into such a page and
    appending again must leave the parent's page bytes and reference counts untouched (copy-on-write of the tail)."""
    cfg = MC.tiny_llama()
    eng = build_engine(cfg, "cpu", seed=0, max_batch=4, use_cuda_graphs=False)
    page = cfg.page_size
    g = torch.Generator().manual_seed(5)
    prompt = torch.randint(0, cfg.vocab, (2 * page + 1,), generator=g).tolist()
    parent = eng.new_sequence(prompt)
    eng.prefill([parent])                                   # 2 * page + 1 tokens computed
    child = eng.fork_sequence(parent, prompt[:2 * page] + [7])      # shares the two full pages
    assert child.num_computed == 2 * page
    pool = eng.cache.pool
    shared = pool.pages(parent.seq_id)[1]
    assert pool.pages(child.seq_id)[1] == shared and pool.refcount(shared) == 2
    before = eng.cache.values[:, :, shared].clone()
    eng.rollback(child, 2 * page - 4)                       # the child's tail now lies inside the shared page
    assert pool.refcount(shared) == 1                       # the child got a private copy
    private = pool.pages(child.seq_id)[1]
    assert private != shared
    assert torch.equal(eng.cache.values[:, :, private], before)
    child.tokens += [3, 9, 11, 2]
    eng.prefill([child])                                    # appends into the private page
    assert torch.equal(eng.cache.values[:, :, shared], before)
    assert not torch.equal(eng.cache.values[:, :, private], before)
    # the parent still decodes as if nothing happened
    ref = build_engine(cfg, "cpu", seed=0, max_batch=4, use_cuda_graphs=False)
    rs = ref.new_sequence(prompt)
    first = ref.prefill([rs])
    parent.tokens.append(first[0]); rs.tokens.append(first[0])
    assert eng.decode([parent]) == ref.decode([rs])


def test_nvfp4_kv_cache_rows_and_generation():
    """NVFP4 KV pages: the row codec round trip, a generation whose decode steps agree with a prefill of the same
    tokens, and logits that stay close to the bf16-cache logits."""
    import numpy as np
    import torch
    from sllm_b200.engine.engine import build_engine
    from sllm_b200.formats import codecs
    from sllm_b200.models import config as MC
    from sllm_b200.ops import reference as ref
    torch.manual_seed(0)
    x = torch.randn(5, 3, 64) * 2
    x[0, 0, 3] = float("nan")
    x[1, 1] = 0.0
    rows, outer = ref.quant_kv_nvfp4_rows(x)
    assert rows.shape == (5, 3, 36) and rows.dtype == torch.uint8 and outer.shape == (5, 3)
    back = ref.dequant_kv_nvfp4_rows(rows, outer, 64)
    xn = torch.nan_to_num(x, nan=0.0)
    assert float(outer[1, 1]) == 1.0 and torch.equal(back[1, 1], torch.zeros(64))
    assert (back - xn).abs().max() <= 0.26 * xn.abs().amax()          # E2M1 steps are at most a quarter of the block maximum
    want = codecs.dequantize_nvfp4(*[a.reshape(15, -1) for a in codecs.quantize_kv_nvfp4(xn.numpy())[:2]], 1.0, 64)
    assert np.allclose(back.numpy().reshape(15, 64), want * outer.numpy().reshape(15, 1))
    cfg = MC.tiny_llama()
    cfg.kv_format = "nvfp4"
    eng = build_engine(cfg, "cpu", seed=3, num_pages=32, max_batch=2, use_cuda_graphs=False)
    assert eng.cache.values.shape[-1] == 36 and eng.cache.layer(0).mode == 2 and eng.cache.scales is not None
    prompt = list(range(9, 45))
    out = eng.generate([prompt], 6)[0]
    assert eng.generate([prompt + out[:3]], 3)[0] == out[3:]
    s = eng.new_sequence(prompt)
    lq = eng.prefill([s], sample=False)
    d1 = eng.decode([s], sample=False) if False else None
    eng.free_sequence(s)
    cfg_b = MC.tiny_llama()
    cfg_b.kv_format = "bf16"
    e2 = build_engine(cfg_b, "cpu", seed=3, num_pages=32, max_batch=2, use_cuda_graphs=False)
    # prefill logits do not read the cache; one decode step does
    a, b = eng.new_sequence(prompt), e2.new_sequence(prompt)
    ta, tb = eng.prefill([a])[0], e2.prefill([b])[0]
    a.tokens.append(ta); b.tokens.append(tb)
    assert ta == tb
    la, lb = eng.decode([a], sample=False).float(), e2.decode([b], sample=False).float()
    assert ((la - lb).norm() / lb.norm()).item() < 0.25 and not torch.equal(la, lb)
    assert eng.cache.bytes_per_token() < 0.35 * e2.cache.bytes_per_token()
    assert lq is not None and d1 is None
