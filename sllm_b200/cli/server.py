"""`sllm-server`: the HTTP serving binary.

One resident model (`--gguf --derived-lock --model ALIAS`) or a manifest of dynamically loaded models
(`--models manifest.json`).  Emits a JSON `ready` event on stdout once the listener is bound and a JSON
`shutdown_audit` event after draining (reference: crates/sllm-server/src/bin/sllm-server.rs:81-324 flags,
:573-589 ready event, :634-637 shutdown audit).  SIGINT / SIGTERM start a graceful drain: stop accepting,
let running requests finish up to `--shutdown-timeout-seconds`, cancel the rest.
"""
from __future__ import annotations

import asyncio
import os
import signal
import sys
import threading
import time

from .common import ACT_ENCODINGS, KV_ENCODINGS, TARGET, CliError, StrictParser, emit, open_model, run_main


def build_parser() -> StrictParser:
    p = StrictParser(prog="sllm-server")
    # model source
    p.add_argument("--gguf")
    p.add_argument("--derived-lock")
    p.add_argument("--device-index", type=int, default=0)
    p.add_argument("--target", default=TARGET)
    p.add_argument("--model", default=None, help="alias of the single resident model")
    p.add_argument("--models", default=None, help="model manifest for dynamic multi-model serving")
    p.add_argument("--max-resident-models", type=int, default=4)
    p.add_argument("--cpu", action="store_true")
    p.add_argument("--allow-cpu-fallback", action="store_true",
                   help="GPU serving only: let an op that is handed a CPU tensor compute its PyTorch oracle (recorded as a "
                        "fallback) instead of failing the request")
    # listener / security
    p.add_argument("--listen", default="127.0.0.1:8080")
    p.add_argument("--api-key-env")
    p.add_argument("--api-key-file")
    p.add_argument("--cors-origins", default="")
    p.add_argument("--metrics", action="store_true")
    p.add_argument("--resumable-sse", action="store_true")
    p.add_argument("--replay-sessions", type=int, default=64)
    p.add_argument("--replay-events", type=int, default=256)
    p.add_argument("--tls-cert")
    p.add_argument("--tls-key")
    p.add_argument("--compatibility-profile", choices=("strict", "openwebui"), default="strict")
    # scheduler
    p.add_argument("--queue-capacity", type=int, default=64)
    p.add_argument("--event-capacity", type=int, default=256)
    p.add_argument("--max-batch", type=int, default=64)
    p.add_argument("--request-timeout-seconds", type=float, default=600.0)
    p.add_argument("--completion-timeout-seconds", type=float, default=None)
    p.add_argument("--shutdown-timeout-seconds", type=float, default=30.0)
    p.add_argument("--prefill-chunk-tokens", type=int, default=0)
    # context / KV
    p.add_argument("--context-length", type=int, default=None)
    p.add_argument("--kv-cache-encoding", choices=KV_ENCODINGS, default=None)
    p.add_argument("--activation-encoding", choices=ACT_ENCODINGS, default=None,
                   help="4-bit-weight models: bf16 (W4A16, default) or fp4 (W4A4 on the block-scaled tensor-core kernel)")
    p.add_argument("--prefix-cache", action="store_true")
    p.add_argument("--prefix-cache-max-entries", type=int, default=256)
    p.add_argument("--prefix-cache-max-tokens", type=int, default=1 << 20)
    p.add_argument("--prefix-cache-max-resident-bytes", type=int, default=1 << 30)
    p.add_argument("--context-policy", choices=("disabled", "keep-prefix-recent"), default="disabled")
    p.add_argument("--context-keep-recent", type=int, default=0)
    p.add_argument("--context-keep-prefix", type=int, default=0)
    # checkpoints
    p.add_argument("--checkpoint", action="store_true")
    p.add_argument("--checkpoint-directory")
    p.add_argument("--checkpoint-quota-bytes", type=int, default=8 << 30)
    p.add_argument("--checkpoint-load")
    p.add_argument("--checkpoint-save")
    # speculative decoding
    p.add_argument("--draft", choices=("none", "ngram", "external", "mtp"), default="none")
    p.add_argument("--draft-ngram-order", type=int, default=3)
    p.add_argument("--draft-width", type=int, default=4)
    p.add_argument("--draft-model-identity")
    p.add_argument("--draft-tokenizer-identity")
    p.add_argument("--draft-vocabulary-size", type=int, default=None)
    p.add_argument("--draft-gguf")
    p.add_argument("--draft-derived-lock")
    return p


def _validate(a) -> None:
    if bool(a.models) == bool(a.gguf):
        raise CliError("give either --gguf/--derived-lock (one model) or --models (manifest)")
    if a.gguf and not a.derived_lock:
        raise CliError("--gguf needs --derived-lock")
    if a.api_key_env and a.api_key_file:
        raise CliError("give at most one of --api-key-env and --api-key-file")
    if bool(a.tls_cert) != bool(a.tls_key):
        raise CliError("--tls-cert and --tls-key go together")
    if not 1 <= a.queue_capacity <= 4096 or not 1 <= a.event_capacity <= 65536:
        raise CliError("--queue-capacity must be in 1..4096 and --event-capacity in 1..65536")
    if not 1 <= a.draft_width <= 8:
        raise CliError("--draft-width must be in 1..8")
    if a.context_policy == "keep-prefix-recent" and a.context_keep_recent + a.context_keep_prefix <= 0:
        raise CliError("--context-policy keep-prefix-recent needs --context-keep-recent/--context-keep-prefix")
    if (a.checkpoint or a.checkpoint_load or a.checkpoint_save) and not a.checkpoint_directory:
        raise CliError("checkpoint flags need --checkpoint-directory")
    host, _, port = a.listen.rpartition(":")
    if not host or not port.isdigit() or not 0 <= int(port) <= 65535:
        raise CliError("--listen must be HOST:PORT")


def _credentials(a):
    from ..server.security import CredentialError, CredentialStore
    try:
        if a.api_key_env:
            tok = os.environ.get(a.api_key_env)
            if not tok:
                raise CliError(f"environment variable {a.api_key_env} is not set")
            return CredentialStore.from_user_key(tok)
        if a.api_key_file:
            return CredentialStore.from_key_file(a.api_key_file)
    except (CredentialError, OSError) as exc:
        raise CliError(f"cannot load API keys: {exc}") from None
    return CredentialStore.open()


def make_backend(a, gguf: str, derived_lock: str, alias: str, overrides=None):
    """Opens one model and wraps it in an EngineBackend according to the serving flags."""
    import argparse
    from ..cache.checkpoint import CheckpointStore
    from ..cache.context_shift import ContextPolicy
    from ..cache.prefix import PrefixCache, PrefixIdentity
    from ..server.backend import EngineBackend
    o = overrides or {}
    src = argparse.Namespace(gguf=gguf, derived_lock=derived_lock, device_index=o.get("device_index", a.device_index),
                             target=a.target, kv_cache_encoding=o.get("kv_cache_encoding") or a.kv_cache_encoding,
                             context_length=o.get("context_length") or a.context_length, cpu=a.cpu,
                             _ep=getattr(a, "_ep", None))
    tp, ctrl = getattr(a, "_tp", None), getattr(a, "_ctrl", None)
    eng, tok, g, lock = open_model(src, max_batch=o.get("max_batch") or a.max_batch, tp=tp)
    if not a.cpu and not a.allow_cpu_fallback:
        from ..ops import _lib
        _lib.set_fail_closed(True)             # serving from a GPU: a tensor that strays to the CPU is an error
    if tp is None and not a.cpu:
        eng.warm_up(greedy_modes=(False,))     # capture the decode graphs before the first request, not during it
    if tp is not None:
        from ..engine.distributed import LeaderEngine, follow
        if tp.rank != 0:
            follow(eng, ctrl)          # returns when the leader shuts down
            return None
        eng = LeaderEngine(eng, ctrl)
    policy = None
    if a.context_policy == "keep-prefix-recent":
        policy = ContextPolicy.keep_prefix_recent(a.context_keep_prefix, a.context_keep_recent)
    pc = None
    if a.prefix_cache or o.get("prefix_cache"):
        pc = PrefixCache(eng, PrefixIdentity(model=lock["fingerprint"], tokenizer=getattr(tok, "identity", "byte"),
                                             kv_layout=eng.cfg.kv_format, context_policy=policy.identity() if policy else ""),
                         a.prefix_cache_max_entries, a.prefix_cache_max_tokens, a.prefix_cache_max_resident_bytes)
    store = CheckpointStore(a.checkpoint_directory, a.checkpoint_quota_bytes) if a.checkpoint_directory else None
    backend = EngineBackend(eng, tok, aliases=(alias,), queue_capacity=a.queue_capacity, event_capacity=a.event_capacity,
                            prefill_chunk_tokens=a.prefill_chunk_tokens, prefix_cache=pc, kv_cache_encoding=eng.cfg.kv_format,
                            context_policy=policy, checkpoint_store=store)
    backend.fingerprint = lock["fingerprint"]
    if a.draft != "none":
        from ..engine.speculative import configure_draft
        configure_draft(backend, a)
    return backend


def serve(a) -> int:
    import uvicorn
    from ..server.app import ModelRegistry, ServerConfig, build_app
    from ..server.lifecycle import ServerLifecycle
    from ..server.model_lifecycle import ManifestError, ModelLifecycleRegistry, read_manifest
    life = ServerLifecycle()
    t0 = time.time()
    # The engine thread releases the interpreter lock while the GPU works and needs it back the moment a step ends; with
    # the default 5 ms switch interval a busy HTTP thread keeps it that long, which is longer than a whole decode step.
    sys.setswitchinterval(float(os.environ.get("SLLM_SWITCH_INTERVAL", "2e-4")))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        # one process per GPU: rank 0 serves HTTP and drives the others through the leader/follower protocol
        import datetime
        import torch
        import torch.distributed as dist
        from ..parallel.tp import make_tp
        if a.models:
            raise CliError("multi-rank serving takes one model (--gguf), not a manifest")
        local = int(os.environ.get("LOCAL_RANK", "0"))
        rank = int(os.environ.get("RANK", "0"))
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if a.cpu:
            raise CliError("multi-rank serving needs GPUs")
        torch.cuda.set_device(local)
        a.device_index = local
        dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=600))
        a._ctrl = dist.new_group(backend="gloo")
        from ..formats import gguf as G
        from ..models import loader
        gfile = G.GgufFile(a.gguf)
        file_cfg = loader.config_from_gguf(gfile)
        d_model = file_cfg.d_model
        gfile.close()
        a._tp = make_tp(world, rank, torch.device("cuda", local), impl="fused", max_tokens=max(a.max_batch, 128), d_model=d_model)
        a._ep = None
        if file_cfg.family == "moe":
            # the ranks that shard the attention also hold the experts: n_experts / world each
            from ..parallel.ep import FusedEP
            a._ep = FusedEP(world, rank, torch.device("cuda", local), max_tokens=max(a.max_batch, 128), d_model=d_model)
        if rank != 0:
            make_backend(a, a.gguf, a.derived_lock, a.model or "model")     # follows until the leader stops
            a._tp.close()
            dist.destroy_process_group()
            os._exit(0)
    dyn = None
    backends, fps = {}, {}
    try:
        if a.models:
            try:
                entries = read_manifest(a.models)
            except (OSError, ManifestError) as exc:
                raise CliError(f"cannot read the model manifest: {exc}") from None

            def load(entry):
                return make_backend(a, entry.gguf, entry.derived_lock, entry.alias,
                                    {"context_length": entry.context_length, "kv_cache_encoding": entry.kv_cache_encoding,
                                     "prefix_cache": entry.prefix_cache, "max_batch": entry.max_batch,
                                     "device_index": entry.device_index})

            dyn = ModelLifecycleRegistry(entries, load, lambda b: b.shutdown(a.shutdown_timeout_seconds),
                                         max_resident=a.max_resident_models)
            dyn.preload_marked()
        else:
            alias = a.model or os.path.splitext(os.path.basename(a.gguf))[0]
            b = make_backend(a, a.gguf, a.derived_lock, alias)
            backends[alias] = b
            fps[alias] = b.fingerprint
    except CliError:
        life.to("failed")
        raise
    cfg = ServerConfig(metrics=a.metrics, resumable_sse=a.resumable_sse, replay_sessions=a.replay_sessions,
                       replay_events=a.replay_events, cors_origins=tuple(o for o in a.cors_origins.split(",") if o),
                       compatibility_profile=a.compatibility_profile, request_timeout_s=a.request_timeout_seconds,
                       completion_timeout_s=a.completion_timeout_seconds, credentials=_credentials(a))
    registry = ModelRegistry(backends, dyn, fps)
    app = build_app(registry, cfg, life)
    host, _, port = a.listen.rpartition(":")
    ucfg = uvicorn.Config(app, host=host.strip("[]"), port=int(port), log_level="warning", access_log=False,
                          ssl_certfile=a.tls_cert, ssl_keyfile=a.tls_key, timeout_graceful_shutdown=int(a.shutdown_timeout_seconds))
    server = uvicorn.Server(ucfg)
    server.install_signal_handlers = lambda: None

    def announce():
        while not server.started and not server.should_exit:
            time.sleep(0.01)
        if server.started:
            life.to("ready")
            bound = [s.getsockname() for srv in server.servers for s in srv.sockets]
            emit({"event": "ready", "listen": a.listen, "bound": [f"{h[0]}:{h[1]}" for h in bound],
                  "models": registry.aliases(), "tls": bool(a.tls_cert), "authenticated": cfg.credentials.protected,
                  "dynamic_models": dyn is not None, "startup_seconds": round(time.time() - t0, 3), "pid": os.getpid()})

    def stop(signum, frame):
        life.to("draining")
        server.should_exit = True

    signal.signal(signal.SIGINT, stop)
    signal.signal(signal.SIGTERM, stop)
    threading.Thread(target=announce, daemon=True).start()
    asyncio.run(server.serve())
    life.to("draining")
    audit = {"event": "shutdown_audit", "cancelled_at_shutdown": 0, "models": {}}
    for alias, b in backends.items():
        r = b.shutdown(a.shutdown_timeout_seconds)
        eng = getattr(b, "engine", None)
        if eng is not None and hasattr(eng, "shutdown_report"):
            r["engine"] = eng.shutdown_report()       # memory by category, high-water mark, launches, fallbacks, quarantine
        audit["models"][alias] = r
        audit["cancelled_at_shutdown"] += r.get("cancelled_at_shutdown", 0)
    if dyn is not None:
        audit["dynamic"] = dyn.states()
        dyn.shutdown()
    life.to("shutdown")
    audit["uptime_seconds"] = round(time.time() - t0, 3)
    emit(audit)
    if world > 1:
        import torch.distributed as dist
        for b in backends.values():
            b.engine.stop_followers()
        a._tp.close()
        dist.destroy_process_group()
        os._exit(0)
    return 0


def main(argv=None) -> int:
    def go():
        a = build_parser().parse_args(sys.argv[1:] if argv is None else argv)
        _validate(a)
        return serve(a)
    return run_main(go)


if __name__ == "__main__":
    sys.exit(main())
