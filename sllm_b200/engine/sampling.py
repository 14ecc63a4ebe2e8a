"""Sampling: request parameters, the SplitMix64 stream, the profile sampler, the ordered sampler chain
and the device token selector front end.

Behavioural contract (reference: crates/sllm-core/src/sampling.rs):
  * parameter ranges: temperature [0, 2], top_p [0, 1], presence / frequency penalty [-2, 2] (:25-52);
  * RNG: SplitMix64, seeded from the request or /dev/urandom, 53-bit unit doubles (:228-319);
  * profile sampler: penalties -> temperature -> sort by scaled logit descending (ties: lower id) ->
    softmax in float64 -> shortest prefix reaching top_p -> draw over the retained mass (:364-468);
    +inf logits win uniformly, NaN is an error, temperature 0 returns the device argmax untouched;
  * chain stage order LogitBias, LegacyPenalty, RepeatPenalty, DryPenalty, GrammarMask, IgnoreEos,
    Temperature, TopK, MinP, Typical, TopP, Xtc, Mirostat, Logprobs (:646-661);
  * snapshot / restore of the mutable state (counts, history, RNG, mirostat mu);
  * device selector: additive fp32 logits + u8 validity mask prepared on the host, draw keyed by
    (seed, counter) so host and device streams are interchangeable (:1278, token_selector kernel).
"""
from __future__ import annotations

import ctypes as C
import json
import math
import os
import struct
from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np

MASK64 = (1 << 64) - 1
GAMMA = 0x9E3779B97F4A7C15
MAX_SAMPLING_HISTORY = 16384
MAX_SEQUENCE_BREAKERS = 256
MAX_SEQUENCE_BREAKER_TOKENS = 4096
MAX_LOGIT_BIAS = 4096
STAGE_ORDER = ("LogitBias", "LegacyPenalty", "RepeatPenalty", "DryPenalty", "GrammarMask", "IgnoreEos",
               "Temperature", "TopK", "MinP", "Typical", "TopP", "Xtc", "Mirostat", "Logprobs")


class SamplingError(ValueError):
    pass


def _finite_in(v, lo, hi) -> bool:
    return isinstance(v, (int, float)) and math.isfinite(v) and lo <= v <= hi


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    top_p: float = 1.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0

    def __post_init__(self):
        if not _finite_in(self.temperature, 0.0, 2.0):
            raise SamplingError("temperature must be in [0, 2]")
        if not _finite_in(self.top_p, 0.0, 1.0):
            raise SamplingError("top_p must be in [0, 1]")
        if not _finite_in(self.presence_penalty, -2.0, 2.0):
            raise SamplingError("presence_penalty must be in [-2, 2]")
        if not _finite_in(self.frequency_penalty, -2.0, 2.0):
            raise SamplingError("frequency_penalty must be in [-2, 2]")

    @property
    def requires_logits(self) -> bool:
        return self.temperature > 0.0


class SplitMix64:
    """Request-local stream; the state after k draws is seed + k * gamma."""

    def __init__(self, seed: Optional[int] = None):
        if seed is None:
            seed = int.from_bytes(os.urandom(8), "little")
        self.state = seed & MASK64

    @staticmethod
    def mix(v: int) -> int:
        v &= MASK64
        v = ((v ^ (v >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
        v = ((v ^ (v >> 27)) * 0x94D049BB133111EB) & MASK64
        return v ^ (v >> 31)

    def next_u64(self) -> int:
        self.state = (self.state + GAMMA) & MASK64
        return self.mix(self.state)

    def next_unit(self) -> float:
        return (self.next_u64() >> 11) * (1.0 / (1 << 53))

    @staticmethod
    def unit_at(seed: int, counter: int) -> float:
        """The (counter + 1)-th draw of a stream seeded with `seed` (what the device selector computes)."""
        return (SplitMix64.mix((seed + (counter + 1) * GAMMA) & MASK64) >> 11) * (1.0 / (1 << 53))


def derive_choice_seed(seed: int, choice: int) -> int:
    """Independent stream per choice of an n > 1 request (choice 0 keeps the request seed)."""
    if choice == 0:
        return seed & MASK64
    return SplitMix64.mix((seed ^ (choice * 0xD1B54A32D192ED03)) & MASK64)


def _draw_sorted(ids: np.ndarray, scaled: np.ndarray, top_p: float, rng) -> int:
    """ids / scaled: candidates (finite scaled logits).  Sort, softmax (f64), top-p prefix, draw."""
    order = np.lexsort((ids, -scaled.astype(np.float64)))
    ids, sc = ids[order], scaled[order].astype(np.float64)
    prob = np.exp(sc - sc[0])
    total = prob.sum()
    if not math.isfinite(total) or total <= 0:
        raise SamplingError("empty distribution")
    prob /= total
    cum = np.cumsum(prob)
    keep = int(np.searchsorted(cum, float(top_p), side="left")) + 1
    keep = max(1, min(keep, len(ids)))
    ids, prob = ids[:keep], prob[:keep]
    retained = prob.sum()
    u = rng.next_unit()
    thr = u * retained
    c = np.cumsum(prob)
    i = int(np.searchsorted(c, thr, side="right"))
    return int(ids[min(i, keep - 1)])


class ProfileSampler:
    """The profile-v1 sampler: penalties, temperature, top-p."""

    def __init__(self, params: SamplingParams, prior_tokens: Sequence[int] = ()):
        self.params = params
        self.counts: dict = {}
        for t in prior_tokens:
            self.accept(t)

    def accept(self, token: int) -> None:
        self.counts[token] = self.counts.get(token, 0) + 1

    def select(self, device_argmax: int, logits: Optional[np.ndarray], rng: SplitMix64) -> int:
        p = self.params
        if not p.requires_logits:
            if logits is not None and not (0 <= device_argmax < len(logits)):
                raise SamplingError("greedy token outside the vocabulary")
            return int(device_argmax)
        if logits is None:
            raise SamplingError("logits are required when temperature > 0")
        lg = np.asarray(logits, dtype=np.float32)
        if lg.size == 0:
            raise SamplingError("empty logits")
        if np.isnan(lg).any():
            raise SamplingError(f"NaN logit at token {int(np.argmax(np.isnan(lg)))}")
        pen = lg.copy()
        if self.counts:
            idx = np.fromiter(self.counts.keys(), dtype=np.int64)
            cnt = np.fromiter(self.counts.values(), dtype=np.float32)
            ok = idx < lg.size
            pen[idx[ok]] = pen[idx[ok]] - cnt[ok] * np.float32(p.frequency_penalty) - np.float32(p.presence_penalty)
        scaled = pen / np.float32(p.temperature)
        pos_inf = np.nonzero(scaled == np.inf)[0]
        if pos_inf.size:
            return int(pos_inf[min(int(rng.next_unit() * pos_inf.size), pos_inf.size - 1)])
        valid = np.nonzero(scaled != -np.inf)[0]
        if valid.size == 0:
            raise SamplingError("empty distribution")
        return _draw_sorted(valid, scaled[valid], p.top_p, rng)


@dataclass
class DryConfig:
    multiplier: float
    base: float
    allowed_length: int
    sequence_breakers: list = field(default_factory=list)
    penalty_last_n: int = MAX_SAMPLING_HISTORY

    def __post_init__(self):
        if (not _finite_in(self.multiplier, 0.0, 100.0) or not _finite_in(self.base, 1.0, 4.0)
                or not 0 <= self.allowed_length <= MAX_SAMPLING_HISTORY
                or len(self.sequence_breakers) > MAX_SEQUENCE_BREAKERS or any(len(b) == 0 for b in self.sequence_breakers)
                or sum(len(b) for b in self.sequence_breakers) > MAX_SEQUENCE_BREAKER_TOKENS
                or not 0 <= self.penalty_last_n <= MAX_SAMPLING_HISTORY):
            raise SamplingError("invalid DRY configuration")


@dataclass
class XtcConfig:
    probability: float
    threshold: float
    min_keep: int = 1

    def __post_init__(self):
        if not _finite_in(self.probability, 0.0, 1.0) or not _finite_in(self.threshold, 0.0, 1.0) or self.min_keep < 1:
            raise SamplingError("invalid XTC configuration")


@dataclass
class MirostatConfig:
    mode: int          # 1 or 2
    tau: float = 5.0
    eta: float = 0.1
    mu: float = 10.0

    def __post_init__(self):
        if self.mode not in (1, 2) or not (math.isfinite(self.tau) and self.tau > 0) or not _finite_in(self.eta, 0.0, 1.0) \
                or not (math.isfinite(self.mu) and self.mu > 0):
            raise SamplingError("invalid mirostat configuration")


@dataclass
class SamplerChainConfig:
    params: SamplingParams = field(default_factory=SamplingParams)
    top_k: Optional[int] = None
    min_p: float = 0.0
    typical_p: float = 1.0
    repeat_penalty: float = 1.0
    repeat_last_n: int = 64
    dynamic_temperature: Optional[tuple] = None   # (range, exponent)
    ignore_eos_token: Optional[int] = None
    logit_bias: list = field(default_factory=list)  # [(token, bias)]
    dry: Optional[DryConfig] = None
    xtc: Optional[XtcConfig] = None
    mirostat: Optional[MirostatConfig] = None
    return_logprobs: bool = False
    top_logprobs: int = 0

    def validate(self) -> None:
        if self.top_k is not None and not 1 <= self.top_k <= 1_048_576:
            raise SamplingError("top_k out of range")
        if not _finite_in(self.min_p, 0.0, 1.0) or not _finite_in(self.typical_p, 0.0, 1.0):
            raise SamplingError("min_p / typical_p must be in [0, 1]")
        if not _finite_in(self.repeat_penalty, 0.0, 10.0) or self.repeat_penalty == 0.0:
            raise SamplingError("repeat_penalty must be in (0, 10]")
        if not 0 <= self.repeat_last_n <= MAX_SAMPLING_HISTORY:
            raise SamplingError("repeat_last_n out of range")
        if len(self.logit_bias) > MAX_LOGIT_BIAS or any(not _finite_in(b, -100.0, 100.0) for _, b in self.logit_bias):
            raise SamplingError("logit_bias: at most 4096 entries in [-100, 100]")
        if len({t for t, _ in self.logit_bias}) != len(self.logit_bias):
            raise SamplingError("logit_bias: duplicate token")
        if not 0 <= self.top_logprobs <= 20:
            raise SamplingError("top_logprobs must be in [0, 20]")
        if self.dynamic_temperature is not None:
            rng_, exp_ = self.dynamic_temperature
            if not _finite_in(rng_, 0.0, 2.0) or not _finite_in(exp_, 0.0, 10.0):
                raise SamplingError("invalid dynamic temperature")

    @property
    def extended(self) -> bool:
        return (self.top_k is not None or self.min_p > 0 or self.typical_p < 1 or self.repeat_penalty != 1.0
                or self.dynamic_temperature is not None or bool(self.logit_bias) or self.dry is not None
                or self.xtc is not None or self.mirostat is not None)

    @property
    def requires_logits(self) -> bool:
        return self.params.requires_logits or self.mirostat is not None or self.return_logprobs or self.top_logprobs > 0

    @property
    def requires_randomness(self) -> bool:
        return self.params.requires_logits or self.mirostat is not None


@dataclass
class Selection:
    token: int
    logprob: Optional[float] = None
    top_logprobs: list = field(default_factory=list)  # [(token, logprob)]


class _NativeConfig(C.Structure):
    """struct SllmSamplerConfig of csrc/host/host_api.h."""
    _fields_ = ([(n, C.c_double) for n in ("temperature", "top_p", "min_p", "typical_p", "presence_penalty", "frequency_penalty",
                                           "repeat_penalty", "dyn_range", "dyn_exponent", "dry_multiplier", "dry_base",
                                           "xtc_probability", "xtc_threshold", "mirostat_tau", "mirostat_eta")]
                + [("bias_tokens", C.POINTER(C.c_int)), ("bias_values", C.POINTER(C.c_float)), ("dry_breakers", C.POINTER(C.c_int))]
                + [(n, C.c_int) for n in ("n_bias", "n_dry_breakers", "top_k", "repeat_last_n", "dynamic_temperature",
                                          "ignore_eos_token", "dry", "dry_allowed_length", "dry_last_n", "xtc", "xtc_min_keep",
                                          "mirostat", "return_logprobs", "top_logprobs")])


class _NativeState(C.Structure):
    _fields_ = [("rng_state", C.c_uint64), ("draws", C.c_longlong), ("mu", C.c_double)]


_native = {"lib": None, "on": None}


def _native_lib():
    if _native["lib"] is None:
        from ..ops import _lib
        lib = _lib.host()
        lib.sllm_host_sample.restype = C.c_int
        lib.sllm_host_sample.argtypes = [C.POINTER(C.c_float), C.c_int, C.POINTER(C.c_ubyte), C.POINTER(_NativeConfig),
                                         C.POINTER(_NativeState), C.POINTER(C.c_int), C.c_int, C.POINTER(C.c_int),
                                         C.POINTER(C.c_int), C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_double),
                                         C.POINTER(C.c_int), C.POINTER(C.c_double), C.POINTER(C.c_int)]
        # the hand-written mirrors above must have the layout the library was compiled with
        lib.sllm_host_sampler_abi.restype = C.c_int
        lib.sllm_host_sampler_abi.argtypes = [C.POINTER(C.c_int), C.c_int]
        buf = (C.c_int * 16)()
        n = lib.sllm_host_sampler_abi(buf, 16)
        k, s_ = _NativeConfig, _NativeState
        mine = [C.sizeof(k), k.repeat_penalty.offset, k.mirostat_eta.offset, k.bias_tokens.offset, k.dry_breakers.offset,
                k.n_bias.offset, k.ignore_eos_token.offset, k.mirostat.offset, k.top_logprobs.offset, C.sizeof(s_),
                s_.draws.offset, s_.mu.offset]
        if n != len(mine) or list(buf[:n]) != mine:
            raise SamplingError(f"host sampler struct layout mismatch: library {list(buf[:max(n, 0)])}, bindings {mine}")
        _native["lib"] = lib
    return _native["lib"]


def native_sampler_enabled() -> bool:
    if _native["on"] is None:
        _native["on"] = os.environ.get("SLLM_HOST_SAMPLER", "native") != "python"
    return _native["on"]


def use_native_sampler(on: bool) -> None:
    _native["on"] = bool(on)


class SamplerChain:
    """The ordered chain.  `select` consumes one row of logits (float32) and an optional validity mask."""

    def __init__(self, config: SamplerChainConfig, prior_tokens: Sequence[int] = (), seed: Optional[int] = None):
        config.validate()
        self.cfg = config
        self.history: list = []
        self.counts: dict = {}
        self.rng = SplitMix64(seed) if config.requires_randomness else SplitMix64(0)
        self.seed = self.rng.state
        self.draws = 0
        self.mu = config.mirostat.mu if config.mirostat else 0.0
        for t in prior_tokens:
            self.accept(t)

    # -------------------------------------------------------------- state
    def accept(self, token: int) -> None:
        self.counts[token] = self.counts.get(token, 0) + 1
        self.history.append(int(token))
        if len(self.history) > MAX_SAMPLING_HISTORY:
            del self.history[:len(self.history) - MAX_SAMPLING_HISTORY]

    def snapshot(self) -> bytes:
        body = json.dumps({"schema": "sllm-sampling-runtime-state-v1", "history": self.history,
                           "counts": sorted(self.counts.items()), "rng": self.rng.state, "draws": self.draws,
                           "mu": self.mu}).encode()
        return struct.pack("<I", len(body)) + body

    def restore(self, blob: bytes) -> None:
        if len(blob) < 4 or len(blob) > 16 * 1024 * 1024:
            raise SamplingError("invalid sampler snapshot")
        (n,) = struct.unpack("<I", blob[:4])
        if n != len(blob) - 4:
            raise SamplingError("invalid sampler snapshot length")
        d = json.loads(blob[4:])
        if d.get("schema") != "sllm-sampling-runtime-state-v1":
            raise SamplingError("unknown sampler snapshot schema")
        self.history = [int(t) for t in d["history"]]
        self.counts = {int(k): int(v) for k, v in d["counts"]}
        self.rng.state = int(d["rng"]) & MASK64
        self.draws = int(d["draws"])
        self.mu = float(d["mu"])

    # -------------------------------------------------------------- stages on logits
    def _penalised(self, logits: np.ndarray) -> np.ndarray:
        c, p = self.cfg, self.cfg.params
        lg = logits.astype(np.float32).copy()
        n = lg.size
        for tok, bias in c.logit_bias:                                   # LogitBias
            if 0 <= tok < n:
                lg[tok] += np.float32(bias)
        if self.counts and (p.frequency_penalty or p.presence_penalty):  # LegacyPenalty
            idx = np.fromiter(self.counts.keys(), dtype=np.int64)
            cnt = np.fromiter(self.counts.values(), dtype=np.float32)
            ok = idx < n
            lg[idx[ok]] -= cnt[ok] * np.float32(p.frequency_penalty) + np.float32(p.presence_penalty)
        if c.repeat_penalty != 1.0 and c.repeat_last_n and self.history:  # RepeatPenalty
            recent = np.unique(np.asarray(self.history[-c.repeat_last_n:], dtype=np.int64))
            recent = recent[recent < n]
            v = lg[recent]
            lg[recent] = np.where(v > 0, v / np.float32(c.repeat_penalty), v * np.float32(c.repeat_penalty))
        if c.dry is not None and c.dry.multiplier > 0 and self.history:   # DryPenalty
            self._apply_dry(lg)
        return lg

    def _apply_dry(self, lg: np.ndarray) -> None:
        d = self.cfg.dry
        hist = self.history[-d.penalty_last_n:] if d.penalty_last_n else self.history
        n = len(hist)
        if n < 2:
            return
        breakers = {b[0] for b in d.sequence_breakers if len(b) == 1}
        # longest match ending at each earlier position with the current suffix; the token following
        # that earlier match would extend the repetition
        best: dict = {}
        last = hist[-1]
        for i in range(n - 1):
            if hist[i] != last or last in breakers:
                continue
            length = 1
            while i - length >= 0 and length < n - 1 and hist[i - length] == hist[n - 1 - length] \
                    and hist[i - length] not in breakers:
                length += 1
            nxt = hist[i + 1]
            if length > best.get(nxt, 0):
                best[nxt] = length
        for tok, length in best.items():
            if length >= d.allowed_length and 0 <= tok < lg.size:
                lg[tok] -= np.float32(d.multiplier * d.base ** (length - d.allowed_length))

    def additive_and_mask(self, vocab: int, valid_mask: Optional[np.ndarray] = None):
        """Device selector inputs: additive fp32 logits (bias + penalties as a delta) and a u8 mask."""
        zero = np.zeros(vocab, dtype=np.float32)
        add = self._penalised(zero) if (self.cfg.logit_bias or self.counts) and not self._needs_value_dependent() else zero
        mask = np.ones(vocab, dtype=np.uint8) if valid_mask is None else np.asarray(valid_mask, dtype=np.uint8).copy()
        if self.cfg.ignore_eos_token is not None and 0 <= self.cfg.ignore_eos_token < vocab:
            mask[self.cfg.ignore_eos_token] = 0
        return add, mask

    def _needs_value_dependent(self) -> bool:
        c = self.cfg
        return c.repeat_penalty != 1.0 or c.dry is not None

    def supports_device_selector(self) -> bool:
        """True when every enabled stage is one the device kernel implements and a seed is fixed."""
        c = self.cfg
        return (c.params.requires_logits and c.typical_p >= 1.0 and c.dynamic_temperature is None and c.dry is None
                and c.xtc is None and c.mirostat is None and c.repeat_penalty == 1.0 and c.top_logprobs == 0)

    def counts_matter(self) -> bool:
        """True when token counts change the logits (legacy penalties configured)."""
        p = self.cfg.params
        return p.frequency_penalty != 0.0 or p.presence_penalty != 0.0

    def device_row(self) -> tuple:
        """(temperature, top_p, min_p, top_k, seed, counter) for the next draw; advances the counter."""
        c = self.cfg
        row = (float(c.params.temperature), float(c.params.top_p), float(c.min_p), int(c.top_k or 0), self.seed,
               self.draws)
        self.draws += 1
        self.rng.state = (self.seed + self.draws * GAMMA) & MASK64
        return row

    # -------------------------------------------------------------- host selection
    def select(self, logits: Optional[np.ndarray], device_argmax: Optional[int] = None,
               valid_mask: Optional[np.ndarray] = None) -> Selection:
        """One token from one row of logits.  The chain runs in the native host library (csrc/host/sampler.cpp);
        `SLLM_HOST_SAMPLER=python` (or `use_native_sampler(False)`) selects the NumPy form of the same chain, which is
        the oracle of the native one."""
        c = self.cfg
        if not c.requires_logits and not c.extended and valid_mask is None and c.ignore_eos_token is None:
            if device_argmax is None:
                if logits is None:
                    raise SamplingError("greedy selection needs the device argmax or logits")
                device_argmax = int(np.argmax(logits))
            return Selection(int(device_argmax))
        if logits is None:
            raise SamplingError("logits are required by the configured sampler chain")
        if native_sampler_enabled():
            return self._select_native(logits, valid_mask)
        return self._select_python(logits, valid_mask)

    def _native_config(self):
        if getattr(self, "_ncfg", None) is not None:
            return self._ncfg
        c, p = self.cfg, self.cfg.params
        keep = []
        k = _NativeConfig()
        k.temperature, k.top_p, k.min_p, k.typical_p = float(p.temperature), float(p.top_p), float(c.min_p), float(c.typical_p)
        k.presence_penalty, k.frequency_penalty = float(p.presence_penalty), float(p.frequency_penalty)
        k.repeat_penalty = float(c.repeat_penalty)
        if c.dynamic_temperature is not None:
            k.dynamic_temperature, k.dyn_range, k.dyn_exponent = 1, float(c.dynamic_temperature[0]), float(c.dynamic_temperature[1])
        if c.logit_bias:
            bt = (C.c_int * len(c.logit_bias))(*[int(t) for t, _ in c.logit_bias])
            bv = (C.c_float * len(c.logit_bias))(*[float(np.float32(b)) for _, b in c.logit_bias])
            keep += [bt, bv]
            k.bias_tokens, k.bias_values, k.n_bias = C.cast(bt, C.POINTER(C.c_int)), C.cast(bv, C.POINTER(C.c_float)), len(c.logit_bias)
        if c.dry is not None:
            single = [int(b[0]) for b in c.dry.sequence_breakers if len(b) == 1]
            br = (C.c_int * max(1, len(single)))(*single)
            keep.append(br)
            k.dry, k.dry_multiplier, k.dry_base = 1, float(c.dry.multiplier), float(c.dry.base)
            k.dry_allowed_length, k.dry_last_n = int(c.dry.allowed_length), int(c.dry.penalty_last_n)
            k.dry_breakers, k.n_dry_breakers = C.cast(br, C.POINTER(C.c_int)), len(single)
        k.top_k = int(c.top_k or 0)
        k.repeat_last_n = int(c.repeat_last_n)
        k.ignore_eos_token = -1 if c.ignore_eos_token is None else int(c.ignore_eos_token)
        if c.xtc is not None:
            k.xtc, k.xtc_probability, k.xtc_threshold, k.xtc_min_keep = 1, float(c.xtc.probability), float(c.xtc.threshold), int(c.xtc.min_keep)
        if c.mirostat is not None:
            k.mirostat, k.mirostat_tau, k.mirostat_eta = int(c.mirostat.mode), float(c.mirostat.tau), float(c.mirostat.eta)
        k.return_logprobs, k.top_logprobs = int(bool(c.return_logprobs)), int(c.top_logprobs)
        self._ncfg, self._ncfg_keep = k, keep
        return k

    def _select_native(self, logits, valid_mask) -> Selection:
        lib = _native_lib()
        raw = np.ascontiguousarray(np.asarray(logits, dtype=np.float32).reshape(-1))
        cfg = self._native_config()
        st = _NativeState(self.rng.state, self.draws, float(self.mu))
        hist = np.asarray(self.history, dtype=np.int32)
        ct = np.fromiter(self.counts.keys(), dtype=np.int32, count=len(self.counts))
        cv = np.fromiter(self.counts.values(), dtype=np.int32, count=len(self.counts))
        mask = None
        if valid_mask is not None:
            mask = np.ascontiguousarray(np.asarray(valid_mask).reshape(-1) != 0).view(np.uint8)
            if mask.size != raw.size:
                raise SamplingError("validity mask and logits differ in length")
        tok, lp, ntop = C.c_int(0), C.c_double(0.0), C.c_int(0)
        nt = max(1, self.cfg.top_logprobs)
        top_ids, top_lp = (C.c_int * nt)(), (C.c_double * nt)()
        ptr = lambda a, t: a.ctypes.data_as(C.POINTER(t)) if a is not None and a.size else None
        rc = lib.sllm_host_sample(ptr(raw, C.c_float), raw.size, ptr(mask, C.c_ubyte), C.byref(cfg), C.byref(st),
                                  ptr(hist, C.c_int), hist.size, ptr(ct, C.c_int), ptr(cv, C.c_int), ct.size, C.byref(tok),
                                  C.byref(lp), top_ids, top_lp, C.byref(ntop))
        if rc == 7:
            raise SamplingError(f"NaN logit at token {tok.value}")
        if rc == 8:
            raise SamplingError("empty distribution")
        if rc != 0:
            raise SamplingError(f"host sampler failed with status {rc}")
        self.rng.state, self.draws, self.mu = int(st.rng_state), int(st.draws), float(st.mu)
        sel = Selection(int(tok.value))
        if self.cfg.return_logprobs or self.cfg.top_logprobs:
            sel.logprob = float(lp.value)
            sel.top_logprobs = [(int(top_ids[i]), float(top_lp[i])) for i in range(ntop.value)]
        return sel

    def _select_python(self, logits, valid_mask=None) -> Selection:
        c, p = self.cfg, self.cfg.params
        raw = np.asarray(logits, dtype=np.float32)
        if np.isnan(raw).any():
            raise SamplingError(f"NaN logit at token {int(np.argmax(np.isnan(raw)))}")
        lg = self._penalised(raw)
        if valid_mask is not None:                                        # GrammarMask
            lg = np.where(np.asarray(valid_mask, dtype=bool), lg, -np.inf).astype(np.float32)
        if c.ignore_eos_token is not None and 0 <= c.ignore_eos_token < lg.size:  # IgnoreEos
            lg[c.ignore_eos_token] = -np.inf
        ids = np.nonzero(lg != -np.inf)[0]
        if ids.size == 0:
            raise SamplingError("empty distribution")
        base_logp = None
        if c.return_logprobs or c.top_logprobs:
            z = lg[ids].astype(np.float64)
            base_logp = z - (z.max() + math.log(np.exp(z - z.max()).sum()))
        if not p.requires_logits and c.mirostat is None:                  # greedy over the processed logits
            order = np.lexsort((ids, -lg[ids].astype(np.float64)))
            tok = int(ids[order[0]])
            return self._finish(tok, ids, base_logp)
        temp = p.temperature if p.temperature > 0 else 1.0
        if c.dynamic_temperature is not None and p.temperature > 0:       # Temperature (dynamic)
            rng_, exp_ = c.dynamic_temperature
            z = lg[ids].astype(np.float64)
            pr = np.exp(z - z.max())
            pr /= pr.sum()
            ent = -(pr[pr > 0] * np.log(pr[pr > 0])).sum()
            max_ent = math.log(len(ids)) if len(ids) > 1 else 1.0
            lo, hi = max(0.0, p.temperature - rng_), p.temperature + rng_
            temp = lo + (hi - lo) * (ent / max_ent) ** exp_ if max_ent > 0 else p.temperature
            temp = max(temp, 1e-6)
        scaled = (lg[ids] / np.float32(temp)).astype(np.float64)
        order = np.lexsort((ids, -scaled))
        ids, scaled = ids[order], scaled[order]
        pos_inf = np.nonzero(scaled == np.inf)[0]
        if pos_inf.size:
            u = self._unit()
            return self._finish(int(ids[pos_inf[min(int(u * pos_inf.size), pos_inf.size - 1)]]), ids, base_logp)
        if c.top_k is not None:                                           # TopK
            ids, scaled = ids[:c.top_k], scaled[:c.top_k]
        prob = np.exp(scaled - scaled[0])
        prob /= prob.sum()
        if c.min_p > 0:                                                   # MinP
            keep = prob >= c.min_p * prob[0]
            ids, prob = ids[keep], prob[keep] / prob[keep].sum()
        if c.typical_p < 1.0 and len(ids) > 1:                            # Typical
            logp = np.log(np.maximum(prob, 1e-300))
            ent = -(prob * logp).sum()
            dev = np.abs(-logp - ent)
            o2 = np.lexsort((np.arange(len(ids)), dev))
            cum = np.cumsum(prob[o2])
            k = int(np.searchsorted(cum, c.typical_p, side="left")) + 1
            sel = np.sort(o2[:max(1, k)])
            ids, prob = ids[sel], prob[sel] / prob[sel].sum()
        if p.top_p < 1.0:                                                 # TopP
            cum = np.cumsum(prob)
            k = max(1, min(int(np.searchsorted(cum, p.top_p, side="left")) + 1, len(ids)))
            ids, prob = ids[:k], prob[:k]
        if c.xtc is not None and len(ids) > 1:                            # Xtc
            if self._unit() < c.xtc.probability:
                norm = prob / prob.sum()
                above = np.nonzero(norm >= c.xtc.threshold)[0]
                if above.size >= 2:
                    drop = above[:-1]                                      # all but the least likely of them
                    if len(ids) - drop.size >= c.xtc.min_keep:
                        keepm = np.ones(len(ids), dtype=bool)
                        keepm[drop] = False
                        ids, prob = ids[keepm], prob[keepm]
        if c.mirostat is not None:                                        # Mirostat
            tok = self._mirostat(ids, prob)
            return self._finish(tok, None, base_logp, lg)
        retained = prob.sum()
        thr = self._unit() * retained
        i = int(np.searchsorted(np.cumsum(prob), thr, side="right"))
        tok = int(ids[min(i, len(ids) - 1)])
        return self._finish(tok, None, base_logp, lg)

    def _unit(self) -> float:
        self.draws += 1
        return self.rng.next_unit()

    def _mirostat(self, ids: np.ndarray, prob: np.ndarray) -> int:
        m = self.cfg.mirostat
        prob = prob / prob.sum()
        if m.mode == 1:
            # estimate the Zipf exponent from the head of the distribution, then the cut size k
            mtop = min(100, len(prob) - 1)
            if mtop >= 1:
                t = np.log(np.arange(2, mtop + 2) / np.arange(1, mtop + 1))
                b = np.log(np.maximum(prob[:mtop], 1e-300) / np.maximum(prob[1:mtop + 1], 1e-300))
                s_hat = float((t * b).sum() / (t * t).sum()) if (t * t).sum() > 0 else 1.0
            else:
                s_hat = 1.0
            eps = s_hat - 1.0
            n = len(prob)
            k = ((eps * 2 ** self.mu) / (1 - n ** (-eps))) ** (1 / s_hat) if abs(eps) > 1e-9 else float(n)
            k = int(min(max(round(k), 1), n))
            ids, prob = ids[:k], prob[:k] / prob[:k].sum()
        else:
            surprise = -np.log2(np.maximum(prob, 1e-300))
            keep = surprise <= self.mu
            if not keep.any():
                keep[0] = True
            ids, prob = ids[keep], prob[keep] / prob[keep].sum()
        thr = self._unit()
        i = int(np.searchsorted(np.cumsum(prob), thr, side="right"))
        i = min(i, len(ids) - 1)
        observed = -math.log2(max(float(prob[i]), 1e-300))
        self.mu -= m.eta * (observed - m.tau)
        return int(ids[i])

    def _finish(self, tok: int, ids_sorted, base_logp, lg=None) -> Selection:
        c = self.cfg
        sel = Selection(tok)
        if base_logp is not None:
            valid_ids = np.nonzero((lg if lg is not None else None) != -np.inf)[0] if lg is not None else None
            if valid_ids is None:
                valid_ids = np.sort(ids_sorted)
                # base_logp was computed in ascending-id order of the valid set
            pos = int(np.searchsorted(valid_ids, tok))
            sel.logprob = float(base_logp[pos])
            if c.top_logprobs:
                o = np.lexsort((valid_ids, -base_logp))[:c.top_logprobs]
                sel.top_logprobs = [(int(valid_ids[i]), float(base_logp[i])) for i in o]
        return sel


# ------------------------------------------------------------------------------------------------
# device token selector
# ------------------------------------------------------------------------------------------------
SELECTOR_ROW_DTYPE = np.dtype([("temperature", "<f4"), ("top_p", "<f4"), ("min_p", "<f4"), ("top_k", "<i4"),
                               ("seed", "<u8"), ("counter", "<u8")])
SELECTOR_RECORD_DTYPE = np.dtype([("token", "<i4"), ("status", "<i4"), ("logprob", "<f4"), ("reserved", "<f4")])


def device_select(logits, rows: Sequence[tuple], additive=None, mask=None):
    """Runs the token selector kernel. logits: CUDA bf16 [R, V]; rows: (T, top_p, min_p, top_k, seed, counter)
    per row; additive: CUDA fp32 [R, V] or None; mask: CUDA uint8 [R, V] or None.
    Returns a CUDA uint8 tensor [R, 16] of records (view with SELECTOR_RECORD_DTYPE on the host)."""
    import ctypes as C

    import torch

    from ..ops import _lib
    from ..ops.core import _p, _stream, workspace
    _lib.EXTRA_KERNEL_SIGNATURES.setdefault(
        "sllm_token_select", (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                         C.c_void_p, C.c_longlong, C.c_void_p, C.c_void_p]))
    r, v = logits.shape
    cfg = np.zeros(r, dtype=SELECTOR_ROW_DTYPE)
    for i, row in enumerate(rows):
        cfg[i] = row
    d_cfg = torch.from_numpy(cfg.view(np.uint8).reshape(r, 32)).to(logits.device, non_blocking=True)
    out = torch.empty((r, 16), dtype=torch.uint8, device=logits.device)
    wsp = workspace(logits.device)
    rc = _lib.kernels().sllm_token_select(_p(logits), logits.stride(0), _p(additive), _p(mask), _p(d_cfg), r, v,
                                          _p(wsp.ws), wsp.ws.numel(), _p(out), _stream())
    _lib.check(rc, "token_select")
    return out


def reference_select(logits: np.ndarray, row: tuple, additive=None, mask=None):
    """Host mirror of the device selector for one row (same order of stages and the same draw).
    Returns (token, status, logprob)."""
    temperature, top_p, min_p, top_k, seed, counter = row
    z = np.asarray(logits, dtype=np.float32).copy()
    if additive is not None:
        z = z + np.asarray(additive, dtype=np.float32)
    if np.isnan(z).any():
        return -1, 1, 0.0
    s = (z * np.float32(1.0 / temperature)).astype(np.float32)
    if mask is not None:
        s = np.where(np.asarray(mask, dtype=bool), s, -np.inf).astype(np.float32)
    ids = np.nonzero(s != -np.inf)[0]
    if ids.size == 0:
        return -1, 2, 0.0
    mx = s[ids].max()
    prob_all = np.exp((s[ids] - mx).astype(np.float32)).astype(np.float64)
    total = prob_all.sum()
    order = np.lexsort((ids, -s[ids].astype(np.float64)))
    ids, sc, prob = ids[order], s[ids][order], prob_all[order]
    keep = np.ones(len(ids), dtype=bool)
    if min_p > 0:
        keep &= sc >= np.float32(mx + np.float32(math.log(min_p)))
    if top_k > 0 and len(ids) > top_k:
        kth = sc[top_k - 1]
        keep &= sc >= kth          # ties at the boundary are kept
    if top_p < 1.0:
        cum = np.cumsum(prob)
        k = int(np.searchsorted(cum, top_p * total, side="left"))
        kth = sc[min(k, len(sc) - 1)]
        keep &= sc >= kth
    ids, sc, prob = ids[keep], sc[keep], prob[keep]
    kept = prob.sum()
    if not kept > 0:
        return -1, 2, 0.0
    thr = SplitMix64.unit_at(seed, counter) * kept
    i = int(np.searchsorted(np.cumsum(prob), thr, side="right"))
    i = min(i, len(ids) - 1)
    return int(ids[i]), 0, float((sc[i] - mx) - math.log(total))
