"""Bounded longest-prefix KV cache over the paged pool.

An entry is a pool sequence owned by the cache whose pages hold the KV of a published token prefix; a new
request forks it (full pages shared by reference count, the partial last page copied), so a hit costs no
recomputation and no copy beyond one page.  The index maps a rolling hash of every page-aligned token block
chain to the entries that contain it, which makes lookup O(prompt / page) regardless of the entry count; the
unaligned tail is matched token by token.  Entries are keyed by an identity (model fingerprint, execution
plan, adapter, renderer, tokenizer, KV layout, sampling target, context policy): a differing field is a miss.
Leases pin an entry between lookup and fork; eviction is LRU over unleased entries under three bounds:
entries, tokens and bytes (defaults 256 / 1 Mi / 1 GiB as in the reference,
crates/sllm-core/src/prefix_cache.rs:21-28; publish/install counterpart crates/sllm-core/src/qwen_execution.rs:3887-4090).
"""
from __future__ import annotations

import hashlib
import struct
import threading
from dataclasses import dataclass, field
from typing import Optional

DEFAULT_MAX_ENTRIES = 256
DEFAULT_MAX_TOKENS = 1 << 20
DEFAULT_MAX_BYTES = 1 << 30


@dataclass(frozen=True)
class PrefixIdentity:
    model: str = ""
    plan: str = ""
    adapter: str = ""
    renderer: str = ""
    tokenizer: str = ""
    kv_layout: str = ""
    target: str = ""
    context_policy: str = ""

    def digest(self) -> bytes:
        h = hashlib.blake2b(digest_size=16)
        for f in (self.model, self.plan, self.adapter, self.renderer, self.tokenizer, self.kv_layout, self.target,
                  self.context_policy):
            b = f.encode("utf-8")
            h.update(struct.pack("<I", len(b)))
            h.update(b)
        return h.digest()


@dataclass
class _Entry:
    eid: int
    ident: bytes
    tokens: list
    seq_id: int
    chain: list                 # block-chain hashes this entry is indexed under
    leases: int = 0
    tick: int = 0
    hits: int = 0


class PrefixLease:
    """What `lookup` returns: quacks like an engine Sequence for `Engine.fork_sequence` and must be released."""

    def __init__(self, cache: "PrefixCache", entry: _Entry, matched: int):
        self._cache, self._entry = cache, entry
        self.tokens = entry.tokens
        self.num_computed = len(entry.tokens)
        self.seq_id = entry.seq_id
        self.matched = matched
        self._released = False

    def release(self) -> None:
        if not self._released:
            self._released = True
            self._cache._release(self._entry)


class PrefixCache:
    def __init__(self, engine, identity: Optional[PrefixIdentity] = None, max_entries: int = DEFAULT_MAX_ENTRIES,
                 max_tokens: int = DEFAULT_MAX_TOKENS, max_bytes: int = DEFAULT_MAX_BYTES, min_tokens: int = 16):
        self.engine = engine
        self.identity = identity or PrefixIdentity()
        self.max_entries, self.max_tokens, self.max_bytes = max_entries, max_tokens, max_bytes
        self.min_tokens = max(1, min_tokens)
        self.page = engine.cfg.page_size
        self.bytes_per_token = engine.cache.bytes_per_token()
        self._entries: dict = {}
        self._index: dict = {}          # chain hash -> set(entry id)
        self._lock = threading.Lock()
        self._tick = 0
        self._next = 1
        self.counters = {"lookups": 0, "hits": 0, "hit_tokens": 0, "published": 0, "evicted": 0, "rejected": 0}

    # ---------------------------------------------------------------- hashing
    def _chain(self, ident: bytes, tokens: list, limit_blocks: Optional[int] = None):
        """Yields the rolling hash after each full page of `tokens`."""
        h = ident
        n = len(tokens) // self.page
        if limit_blocks is not None:
            n = min(n, limit_blocks)
        for b in range(n):
            blk = tokens[b * self.page:(b + 1) * self.page]
            h = hashlib.blake2b(h + struct.pack(f"<{self.page}q", *blk), digest_size=16).digest()
            yield h

    # ---------------------------------------------------------------- lookup
    def lookup(self, prompt: list, identity: Optional[PrefixIdentity] = None) -> Optional[PrefixLease]:
        """Entry sharing the longest token prefix with `prompt` (at least `min_tokens`), leased; else None."""
        ident = (identity or self.identity).digest()
        with self._lock:
            self.counters["lookups"] += 1
            cands, depth = None, 0
            for i, h in enumerate(self._chain(ident, prompt)):
                ids = self._index.get(h)
                if not ids:
                    break
                cands, depth = ids, i + 1
            best, best_len = None, 0
            pool = list(cands) if cands else [e.eid for e in self._entries.values()
                                               if e.ident == ident and len(e.tokens) < self.page]
            for eid in pool:
                e = self._entries[eid]
                n = depth * self.page
                lim = min(len(e.tokens), len(prompt))
                while n < lim and e.tokens[n] == prompt[n]:
                    n += 1
                if n > best_len:
                    best, best_len = e, n
            if best is None or best_len < self.min_tokens:
                return None
            self._tick += 1
            best.tick = self._tick
            best.leases += 1
            best.hits += 1
            self.counters["hits"] += 1
            self.counters["hit_tokens"] += best_len
            return PrefixLease(self, best, best_len)

    def _release(self, e: _Entry) -> None:
        with self._lock:
            e.leases = max(0, e.leases - 1)

    # ---------------------------------------------------------------- publish
    def publish(self, seq, n_tokens: int, identity: Optional[PrefixIdentity] = None) -> bool:
        """Keeps the first `n_tokens` computed tokens of engine sequence `seq`.  Call from the thread that owns
        the engine, after the step that computed them has been committed."""
        n_tokens = min(n_tokens, seq.num_computed)
        if n_tokens < self.min_tokens or n_tokens > self.max_tokens or n_tokens * self.bytes_per_token > self.max_bytes:
            self.counters["rejected"] += 1
            return False
        ident = (identity or self.identity).digest()
        tokens = list(seq.tokens[:n_tokens])
        chain = list(self._chain(ident, tokens))
        with self._lock:
            # an entry that already covers these tokens makes the publication redundant
            if chain:
                for eid in self._index.get(chain[-1], ()):
                    e = self._entries[eid]
                    if len(e.tokens) >= n_tokens and e.tokens[:n_tokens] == tokens:
                        self._tick += 1
                        e.tick = self._tick
                        return False
            if not self._make_room(n_tokens):
                self.counters["rejected"] += 1
                return False
        try:
            child = self.engine.fork_kv(seq, n_tokens)
        except Exception:
            self.counters["rejected"] += 1
            return False
        with self._lock:
            self._tick += 1
            e = _Entry(self._next, ident, tokens, child, chain, tick=self._tick)
            self._next += 1
            self._entries[e.eid] = e
            for h in chain:
                self._index.setdefault(h, set()).add(e.eid)
            self.counters["published"] += 1
            # a shorter entry that is a strict prefix of the new one is now redundant
            for old in [o for o in self._entries.values() if o.eid != e.eid and o.ident == ident and o.leases == 0
                        and len(o.tokens) <= n_tokens and tokens[:len(o.tokens)] == o.tokens]:
                self._drop(old)
        return True

    def _usage(self):
        toks = sum(len(e.tokens) for e in self._entries.values())
        return len(self._entries), toks, toks * self.bytes_per_token

    def _make_room(self, incoming: int) -> bool:
        while True:
            n, toks, by = self._usage()
            if n + 1 <= self.max_entries and toks + incoming <= self.max_tokens \
                    and by + incoming * self.bytes_per_token <= self.max_bytes:
                return True
            victims = [e for e in self._entries.values() if e.leases == 0]
            if not victims:
                return False
            self._drop(min(victims, key=lambda e: e.tick))
            self.counters["evicted"] += 1

    def _drop(self, e: _Entry) -> None:
        for h in e.chain:
            s = self._index.get(h)
            if s is not None:
                s.discard(e.eid)
                if not s:
                    del self._index[h]
        self._entries.pop(e.eid, None)
        try:
            self.engine.free_kv(e.seq_id)
        except Exception:
            pass

    def evict_pages(self, want_tokens: int) -> int:
        """Frees least-recently-used unleased entries until about `want_tokens` tokens of pages are released
        (called when the pool runs out of pages).  Returns the number of entries dropped."""
        dropped, freed = 0, 0
        with self._lock:
            for e in sorted((e for e in self._entries.values() if e.leases == 0), key=lambda e: e.tick):
                if freed >= want_tokens:
                    break
                freed += len(e.tokens)
                self._drop(e)
                dropped += 1
                self.counters["evicted"] += 1
        return dropped

    def clear(self) -> None:
        with self._lock:
            for e in list(self._entries.values()):
                if e.leases == 0:
                    self._drop(e)

    def stats(self) -> dict:
        with self._lock:
            n, toks, by = self._usage()
            return {"entries": n, "tokens": toks, "bytes": by, **self.counters}
