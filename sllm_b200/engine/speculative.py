"""Speculative decoding: draft providers, verification rules, the transaction and the batch controller.

A step drafts up to `width` (<= 8) tokens per sequence, runs the target once over the block
[last committed token, d1 .. dk] (k + 1 rows of the same sequence in one launch - per-row positions are part of
the kernel ABI), accepts the longest verified prefix plus one target token, and rolls the KV state back to the
accepted length.  Greedy verification accepts draft i while it equals the target's argmax at row i; stochastic
verification accepts with probability min(1, p/q) and resamples the first rejection from the residual
max(0, p - q), which preserves the target distribution.  The transaction object makes the append
all-or-nothing: Staging -> Verified -> Committed, or Aborted with the KV state restored
(reference: crates/sllm-core/src/speculative.rs:10 max width, :76-260 providers, :441-524 transaction,
:526-633 verification rules; controller counterpart crates/sllm-frontend/src/generation.rs:762-1043).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import numpy as np

MAX_DRAFT_WIDTH = 8


class SpeculativeError(RuntimeError):
    pass


# ------------------------------------------------------------------------------------------ providers
class NgramDraftProvider:
    """Prompt-lookup drafting: find the most recent earlier occurrence of the last `order` tokens and propose
    what followed it."""

    def __init__(self, order: int = 3, width: int = 4, min_order: int = 1):
        if not 1 <= width <= MAX_DRAFT_WIDTH or not 1 <= order <= 16:
            raise SpeculativeError("draft width must be in 1..8 and n-gram order in 1..16")
        self.order, self.width, self.min_order = order, width, max(1, min_order)
        self.identity = f"ngram:{order}:{width}"

    def propose(self, tokens: list, width: Optional[int] = None) -> list:
        w = min(width or self.width, self.width)
        n = len(tokens)
        for order in range(min(self.order, n - 1), self.min_order - 1, -1):
            key = tokens[n - order:]
            for start in range(n - order - 1, -1, -1):
                if tokens[start:start + order] == key:
                    out = tokens[start + order:start + order + w]
                    if out:
                        return list(out)
        return []

    def observe(self, tokens: list) -> None:
        pass

    def release(self, seq_key) -> None:
        pass


class ExternalDraftProvider:
    """A smaller model on its own engine drafts greedily.  The draft model must share the target's vocabulary
    and tokenizer identity; the check runs at construction, before any request."""

    def __init__(self, draft_engine, width: int = 4, target_vocab: Optional[int] = None,
                 target_tokenizer_identity: Optional[str] = None, draft_tokenizer_identity: Optional[str] = None,
                 model_identity: str = "external"):
        if not 1 <= width <= MAX_DRAFT_WIDTH:
            raise SpeculativeError("draft width must be in 1..8")
        if target_vocab is not None and draft_engine.cfg.vocab != target_vocab:
            raise SpeculativeError(f"draft vocabulary {draft_engine.cfg.vocab} differs from the target's {target_vocab}")
        if target_tokenizer_identity is not None and draft_tokenizer_identity is not None \
                and target_tokenizer_identity != draft_tokenizer_identity:
            raise SpeculativeError("draft and target tokenizers differ")
        self.engine, self.width = draft_engine, width
        self.identity = f"external:{model_identity}:{width}"
        self._seqs: dict = {}

    def propose_batch(self, keys: list, token_lists: list, width: Optional[int] = None) -> list:
        """Greedy drafts for a batch; the draft engine keeps one sequence per key and reuses its KV prefix."""
        w = min(width or self.width, self.width)
        eng = self.engine
        seqs = []
        for key, toks in zip(keys, token_lists):
            s = self._seqs.get(key)
            if s is None:
                s = eng.new_sequence(toks)
                self._seqs[key] = s
            else:
                # keep the KV of the longest prefix the draft already computed (its own accepted drafts included)
                limit = min(s.num_computed, len(toks) - 1)
                if s.tokens[:limit] == toks[:limit]:      # the usual case, compared at C speed
                    c = limit
                else:
                    c = 0
                    while c < limit and s.tokens[c] == toks[c]:
                        c += 1
                # recompute exactly two rows whenever possible: every sequence then appends the same number of
                # rows and the catch-up replays one captured graph instead of an eager ragged prefill
                if c >= len(toks) - 2 >= 1:
                    c = len(toks) - 2
                eng.rollback(s, c)
                s.tokens = list(toks)
                s.prompt = list(toks)
            seqs.append(s)
        drafts = [[] for _ in seqs]
        # computes whatever suffix is new and samples greedily; equal suffix lengths replay a captured graph
        if len({len(s.tokens) - s.num_computed for s in seqs}) == 1 and seqs[0].num_computed > 0:
            first = [r[-1] for r in eng.extend(seqs)]
        else:
            first = eng.prefill(seqs)
        for i, s in enumerate(seqs):
            s.tokens.append(first[i])
            drafts[i].append(first[i])
        for _ in range(w - 1):
            nxt = eng.decode(seqs)
            for i, s in enumerate(seqs):
                s.tokens.append(nxt[i])
                drafts[i].append(nxt[i])
        return drafts

    def propose(self, tokens: list, width: Optional[int] = None) -> list:
        return self.propose_batch([id(tokens)], [tokens], width)[0]

    def release(self, key) -> None:
        s = self._seqs.pop(key, None)
        if s is not None:
            self.engine.free_sequence(s)


# ------------------------------------------------------------------------------------------ verification
def verify_greedy(draft: list, target_argmax: list, forced_accept: Optional[list] = None):
    """target_argmax has len(draft) + 1 entries (row i predicts the token after draft[:i]).  Returns
    (accepted_count, next_token).  `forced_accept` (benchmark only) overrides the equality test per draft."""
    if len(target_argmax) != len(draft) + 1:
        raise SpeculativeError("verification needs one target row per draft token plus one")
    n = 0
    for i, d in enumerate(draft):
        ok = forced_accept[i] if forced_accept is not None else (d == target_argmax[i])
        if not ok:
            break
        n += 1
    return n, int(target_argmax[n])


def verify_target_selected(draft: list, target_tokens: list):
    """The target already selected a token per row with its own sampler: accept while they agree."""
    return verify_greedy(draft, target_tokens)


def verify_stochastic(draft: list, q_probs: np.ndarray, p_probs: np.ndarray, uniforms, residual_uniform: float):
    """Rejection sampling.  q_probs [k, V] draft distributions, p_probs [k + 1, V] target distributions,
    uniforms: k numbers in [0, 1).  Returns (accepted_count, next_token)."""
    k = len(draft)
    if q_probs.shape[0] != k or p_probs.shape[0] != k + 1:
        raise SpeculativeError("distribution rows do not match the draft length")
    for i, d in enumerate(draft):
        q, p = float(q_probs[i, d]), float(p_probs[i, d])
        if q <= 0.0:
            raise SpeculativeError("draft token has zero draft probability")
        if uniforms[i] < min(1.0, p / q):
            continue
        resid = np.maximum(p_probs[i].astype(np.float64) - q_probs[i].astype(np.float64), 0.0)
        z = resid.sum()
        if z <= 0.0:
            resid, z = p_probs[i].astype(np.float64), float(p_probs[i].sum())
        cdf = np.cumsum(resid / z)
        return i, int(min(np.searchsorted(cdf, residual_uniform, side="right"), len(cdf) - 1))
    cdf = np.cumsum(p_probs[k].astype(np.float64) / float(p_probs[k].sum()))
    return k, int(min(np.searchsorted(cdf, residual_uniform, side="right"), len(cdf) - 1))


# ------------------------------------------------------------------------------------------ accounting / transaction
@dataclass
class SpeculativeAccounting:
    steps: int = 0
    drafted: int = 0
    accepted: int = 0
    emitted: int = 0
    empty_drafts: int = 0
    aborted: int = 0

    @property
    def acceptance_rate(self) -> float:
        return self.accepted / self.drafted if self.drafted else 0.0

    @property
    def tokens_per_step(self) -> float:
        return self.emitted / self.steps if self.steps else 0.0

    def to_dict(self) -> dict:
        return {"steps": self.steps, "drafted": self.drafted, "accepted": self.accepted, "emitted": self.emitted,
                "empty_drafts": self.empty_drafts, "aborted": self.aborted,
                "acceptance_rate": round(self.acceptance_rate, 4), "tokens_per_step": round(self.tokens_per_step, 4)}


class SpeculativeTransaction:
    """Staging -> Verified -> Committed | Aborted for one sequence and one draft block."""

    def __init__(self, engine, seq, draft: list):
        if len(draft) > MAX_DRAFT_WIDTH:
            raise SpeculativeError("draft wider than 8")
        self.engine, self.seq, self.draft = engine, seq, list(draft)
        self.base_len = len(seq.tokens)            # tokens before staging; the last one has no KV yet
        self.base_computed = seq.num_computed
        self.state = "staging"
        self.accepted = 0
        self.next_token: Optional[int] = None
        seq.tokens.extend(self.draft)

    def verified(self, accepted: int, next_token: int) -> None:
        if self.state != "staging" or not 0 <= accepted <= len(self.draft):
            raise SpeculativeError("verification out of order")
        self.accepted, self.next_token, self.state = accepted, next_token, "verified"

    def commit(self) -> list:
        """Keeps the accepted drafts, appends the target's token, truncates the KV state.  Returns new tokens."""
        if self.state != "verified":
            raise SpeculativeError("commit before verification")
        keep = self.base_len + self.accepted
        self.engine.rollback(self.seq, keep)
        self.seq.tokens.append(self.next_token)
        self.state = "committed"
        return self.draft[:self.accepted] + [self.next_token]

    def abort(self) -> None:
        if self.state in ("committed", "aborted"):
            return
        del self.seq.tokens[self.base_len:]
        self.seq.num_computed = min(self.seq.num_computed, self.base_computed)
        self.engine.cache.pool.truncate(self.seq.seq_id, self.seq.num_computed)
        self.state = "aborted"


# ------------------------------------------------------------------------------------------ controller
class SpeculativeDecoder:
    """Greedy speculative decoding for a batch of engine sequences."""

    def __init__(self, engine, provider, width: int = 4, forced_accept_p: Optional[float] = None, seed: int = 0):
        if not 1 <= width <= MAX_DRAFT_WIDTH:
            raise SpeculativeError("draft width must be in 1..8")
        self.engine, self.provider, self.width = engine, provider, width
        self.acct = SpeculativeAccounting()
        self.forced_p = forced_accept_p
        self._rng = np.random.default_rng(seed)

    def step(self, seqs: list, budgets: Optional[list] = None) -> list:
        """One speculative step; returns the tokens appended to each sequence (>= 1 each).  `budgets` caps the
        tokens a sequence may still receive."""
        eng = self.engine
        widths = [min(self.width, (b - 1) if b is not None else self.width,
                      eng.cfg.max_context - len(s.tokens) - 1) for s, b in zip(seqs, budgets or [None] * len(seqs))]
        if hasattr(self.provider, "propose_seqs"):       # providers that read engine state (the MTP head)
            drafts = self.provider.propose_seqs(seqs, max(1, max(widths)))
        elif hasattr(self.provider, "propose_batch"):
            drafts = self.provider.propose_batch([id(s) for s in seqs], [s.tokens for s in seqs], max(1, max(widths)))
        else:
            drafts = [self.provider.propose(s.tokens, max(1, w)) for s, w in zip(seqs, widths)]
        drafts = [d[:max(0, w)] for d, w in zip(drafts, widths)]
        txs = [SpeculativeTransaction(eng, s, d) for s, d in zip(seqs, drafts)]
        try:
            rows = eng.extend(seqs)                 # per sequence: argmax for every new row
        except Exception:
            for t in txs:
                t.abort()
            self.acct.aborted += len(txs)
            raise
        out = []
        for t, r in zip(txs, rows):
            forced = None
            if self.forced_p is not None:
                forced = (self._rng.random(len(t.draft)) < self.forced_p).tolist()
            n, nxt = verify_greedy(t.draft, r, forced)
            t.verified(n, nxt)
            out.append(t.commit())
            self.acct.steps += 1
            self.acct.drafted += len(t.draft)
            self.acct.accepted += n
            self.acct.emitted += n + 1
            if not t.draft:
                self.acct.empty_drafts += 1
        return out

    def release(self, seq) -> None:
        rel = getattr(self.provider, "release", None)
        if rel is not None:
            rel(id(seq))


def configure_draft(backend, args) -> None:
    """Attaches a speculative decoder to a serving backend according to the `--draft*` flags."""
    eng = backend.engine
    if args.draft == "ngram":
        provider = NgramDraftProvider(args.draft_ngram_order, args.draft_width)
    elif args.draft == "external":
        if not (args.draft_gguf and args.draft_derived_lock):
            raise SpeculativeError("--draft external needs --draft-gguf and --draft-derived-lock")
        import argparse
        from ..cli.common import open_model
        src = argparse.Namespace(gguf=args.draft_gguf, derived_lock=args.draft_derived_lock, device_index=args.device_index,
                                 target=args.target, kv_cache_encoding=None, context_length=eng.cfg.max_context,
                                 cpu=getattr(args, "cpu", False))
        d_eng, d_tok, _, d_lock = open_model(src, max_batch=eng.max_batch)
        if args.draft_vocabulary_size is not None and args.draft_vocabulary_size != d_eng.cfg.vocab:
            raise SpeculativeError("--draft-vocabulary-size does not match the draft model")
        if args.draft_model_identity and args.draft_model_identity != d_lock["semantic_model_id"]:
            raise SpeculativeError("--draft-model-identity does not match the draft model's lock")
        provider = ExternalDraftProvider(d_eng, args.draft_width, eng.cfg.vocab,
                                         getattr(backend.tokenizer, "identity", "byte"),
                                         args.draft_tokenizer_identity or getattr(d_tok, "identity", "byte"),
                                         d_lock["semantic_model_id"])
    elif args.draft == "mtp":
        from ..models.mtp import MtpDraftProvider, MtpHead
        if getattr(eng, "mtp_weights", None) is None:
            raise SpeculativeError("--draft mtp needs a model file with an MTP component (mtp.* tensors)")
        provider = MtpDraftProvider(MtpHead(eng, eng.mtp_weights), args.draft_width)
    else:
        return
    backend.loop.speculative = SpeculativeDecoder(eng, provider, args.draft_width)


def device_verify_greedy(draft, draft_len, target, base_len=None, forced=None):
    """Device-side greedy verification (no host round trip).  draft: int32 [B, W], draft_len: int32 [B],
    target: int32 [B, W + 1], base_len: optional int32 [B], forced: optional uint8 [B, W].
    Returns (accept, next, new_len) int32 [B] CUDA tensors."""
    import ctypes as C

    import torch

    from ..ops import _lib
    from ..ops.core import _p, _stream
    P, I = C.c_void_p, C.c_int
    _lib.EXTRA_KERNEL_SIGNATURES.setdefault("sllm_spec_verify_greedy", (I, [P, P, P, P, P, I, I, P, P, P, P]))
    b, w = draft.shape
    if target.shape != (b, w + 1):
        raise SpeculativeError("target must have one more column than draft")
    acc = torch.empty(b, dtype=torch.int32, device=draft.device)
    nxt = torch.empty_like(acc)
    new_len = torch.empty_like(acc)
    rc = _lib.kernels().sllm_spec_verify_greedy(_p(draft.contiguous()), _p(draft_len), _p(target.contiguous()),
                                                _p(forced), _p(base_len), w, b, _p(acc), _p(nxt), _p(new_len), _stream())
    _lib.check(rc, "spec_verify_greedy")
    return acc, nxt, new_len
