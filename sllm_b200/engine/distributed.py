"""One scheduler, many ranks: the leader/follower protocol for serving a tensor- or expert-parallel engine.

Rank 0 owns the HTTP server, the scheduler and the sequences; every call it makes on its engine that launches
device work (`prefill`, `decode`, `extend`) or changes KV ownership (`new_sequence`, `fork_sequence`,
`free_sequence`, `rollback`) is first broadcast as a small command record, and the other ranks replay it on their
own shard inside `follow()`.  All ranks therefore issue the same kernels and collectives in the same order, which
is what the fused peer-memory kernels and NCCL both require.  Commands travel over a gloo group (host side), so
the device streams stay free of control traffic.  (The reference has no multi-GPU path; this is the glue that lets
its single-process server design drive N GPUs.)

Failure detection stays on the host.  A follower whose replay raises posts the error under its rank in the
rendezvous store and leaves; the leader looks at those keys before every command and raises ``FollowerFailed``
instead of launching work that would wait for a dead rank.  A follower whose command channel fails (the leader
exited or stopped answering within the control group's timeout) raises ``LeaderLost`` and leaves.  Ranks only
leave between steps, with none of their kernels or collectives in flight.
"""
from __future__ import annotations

import pickle
from typing import Optional

import torch
import torch.distributed as dist

from .engine import Engine, Sequence

_STOP = "__stop__"
_FAIL_KEY = "sllm/follower_failed/"


class FollowerFailed(RuntimeError):
    """A follower rank reported an error; the engine group must be torn down."""


class LeaderLost(RuntimeError):
    """The command channel to the leader failed."""


def _store():
    try:
        return dist.distributed_c10d._get_default_store()
    except Exception:
        return None


class _Channel:
    def __init__(self, group=None, src: int = 0):
        self.group, self.src = group, src
        self.store = _store()
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0

    def check_followers(self) -> None:
        if self.store is None:
            return
        for r in range(self.world):
            if r != self.src and self.store.check([_FAIL_KEY + str(r)]):
                raise FollowerFailed(f"rank {r}: {self.store.get(_FAIL_KEY + str(r)).decode('utf-8', 'replace')}")

    def report_failure(self, exc: BaseException) -> None:
        if self.store is not None:
            self.store.set(_FAIL_KEY + str(self.rank), f"{type(exc).__name__}: {exc}"[:500])

    def send(self, obj) -> None:
        self.check_followers()
        try:
            dist.broadcast_object_list([obj], src=self.src, group=self.group)
        except RuntimeError as exc:        # a follower left without reporting, or the channel timed out
            self.check_followers()
            raise FollowerFailed(f"command channel failed: {exc}") from None

    def recv(self):
        box = [None]
        try:
            dist.broadcast_object_list(box, src=self.src, group=self.group)
        except RuntimeError as exc:
            raise LeaderLost(f"command channel failed: {exc}") from None
        return box[0]


class LeaderEngine:
    """Wraps the rank-0 engine; same public surface, every state-changing call is mirrored to the followers."""

    def __init__(self, engine: Engine, control_group=None):
        self._e = engine
        self._ch = _Channel(control_group)
        self._ids = {}            # id(Sequence) -> handle shared with the followers
        self._next = 1

    def __getattr__(self, name):
        return getattr(self._e, name)

    def _h(self, s: Sequence) -> int:
        return self._ids[id(s)]

    def new_sequence(self, prompt, user=None):
        s = self._e.new_sequence(prompt, user)
        h = self._next
        self._next += 1
        self._ids[id(s)] = h
        self._ch.send(("new", h, list(prompt)))
        return s

    def fork_sequence(self, src, prompt, user=None):
        s = self._e.fork_sequence(src, prompt, user)
        h = self._next
        self._next += 1
        self._ids[id(s)] = h
        src_h = self._ids.get(id(src))
        if src_h is None:         # e.g. a prefix-cache lease: followers hold the same entry under its pool sequence id
            self._ch.send(("fork_pool", h, src.seq_id, list(src.tokens[:src.num_computed]), list(prompt)))
        else:
            self._ch.send(("fork", h, src_h, list(prompt)))
        return s

    def free_sequence(self, s):
        h = self._ids.pop(id(s), None)
        self._e.free_sequence(s)
        if h is not None:
            self._ch.send(("free", h))

    def fork_kv(self, s, n_tokens):
        self._ch.send(("kvfork", self._h(s), n_tokens))
        return self._e.fork_kv(s, n_tokens)

    def free_kv(self, pool_seq_id):
        self._ch.send(("kvfree", pool_seq_id))
        self._e.free_kv(pool_seq_id)

    def rollback(self, s, length):
        self._ch.send(("rollback", self._h(s), length))
        self._e.rollback(s, length)

    def _sync_tokens(self, seqs):
        return [(self._h(s), list(s.tokens[s.num_computed:])) for s in seqs]

    def prefill(self, seqs, chunk_tokens: int = 0, sample: bool = True, embeds=None, rope_pos3=None, one_chunk: bool = False):
        if embeds is not None or rope_pos3 is not None:
            # a multimodal prompt: the spliced input rows (text embeddings with the visual rows in place) and the 3-axis
            # rotary positions travel with the command; every rank then runs the same one-chunk prefill on its shard
            e_cpu = None if embeds is None else embeds.detach().to("cpu").contiguous()
            p_cpu = None if rope_pos3 is None else rope_pos3.detach().to("cpu", torch.int32).contiguous()
            self._ch.send(("prefill_mm", self._sync_tokens(seqs), sample, e_cpu, p_cpu))
            return self._e.prefill(seqs, chunk_tokens, sample, embeds=embeds, rope_pos3=rope_pos3, one_chunk=one_chunk)
        self._ch.send(("prefill", self._sync_tokens(seqs), chunk_tokens, sample, one_chunk))
        return self._e.prefill(seqs, chunk_tokens, sample, one_chunk=one_chunk)

    def decode(self, seqs, sample: bool = True):
        self._ch.send(("decode", [(self._h(s), s.tokens[-1]) for s in seqs], sample))
        return self._e.decode(seqs, sample)

    def extend(self, seqs, sample: bool = True):
        self._ch.send(("extend", self._sync_tokens(seqs), sample))
        return self._e.extend(seqs, sample)

    def embed_hidden(self, ids):
        self._ch.send(("embed", list(ids)))
        return self._e.embed_hidden(ids)

    def generate(self, prompts, max_new_tokens, eos=None, on_token=None):
        return Engine.generate(self, prompts, max_new_tokens, eos, on_token)

    def stop_followers(self) -> None:
        self._ch.send((_STOP,))


def follow(engine: Engine, control_group=None) -> int:
    """Follower loop: replays the leader's calls until it says stop.  Returns the number of commands handled."""
    ch = _Channel(control_group)
    seqs: dict = {}
    n = 0
    while True:
        cmd = ch.recv()
        op = cmd[0]
        n += 1
        if op == _STOP:
            return n
        try:
            _replay(engine, seqs, cmd)
        except BaseException as exc:       # tell the leader on the host, then leave between steps
            ch.report_failure(exc)
            raise


def _replay(engine: Engine, seqs: dict, cmd) -> None:
    """Applies one mirrored command to this rank's engine."""
    op = cmd[0]
    if op == "new":
        seqs[cmd[1]] = engine.new_sequence(cmd[2])
    elif op == "fork":
        seqs[cmd[1]] = engine.fork_sequence(seqs[cmd[2]], cmd[3])
    elif op == "fork_pool":
        src = Sequence(prompt=list(cmd[3]))
        src.seq_id, src.num_computed = cmd[2], len(cmd[3])
        seqs[cmd[1]] = engine.fork_sequence(src, cmd[4])
    elif op == "free":
        s = seqs.pop(cmd[1], None)
        if s is not None:
            engine.free_sequence(s)
    elif op == "rollback":
        engine.rollback(seqs[cmd[1]], cmd[2])
    elif op == "kvfork":
        engine.fork_kv(seqs[cmd[1]], cmd[2])          # pool ids advance identically on every rank
    elif op == "kvfree":
        engine.free_kv(cmd[1])
    elif op == "embed":
        engine.embed_hidden(cmd[1])
    elif op == "prefill_mm":
        batch = []
        for h, new_tokens in cmd[1]:
            s = seqs[h]
            del s.tokens[s.num_computed:]
            s.tokens.extend(new_tokens)
            batch.append(s)
        dev = engine.device
        embeds = None if cmd[3] is None else cmd[3].to(dev)
        engine.prefill(batch, 0, cmd[2], embeds=embeds, rope_pos3=cmd[4], one_chunk=True)
    elif op in ("prefill", "extend"):
        batch = []
        for h, new_tokens in cmd[1]:
            s = seqs[h]
            del s.tokens[s.num_computed:]
            s.tokens.extend(new_tokens)
            batch.append(s)
        if op == "prefill":
            engine.prefill(batch, cmd[2], cmd[3], one_chunk=cmd[4])
        else:
            engine.extend(batch, cmd[2])
    elif op == "decode":
        batch = []
        for h, last in cmd[1]:
            s = seqs[h]
            if len(s.tokens) == s.num_computed:
                s.tokens.append(last)
            else:
                s.tokens[-1] = last
            batch.append(s)
        engine.decode(batch, cmd[2])
    else:
        raise RuntimeError(f"unknown engine command {op!r}")
