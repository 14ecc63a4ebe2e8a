"""Dependency-free Prometheus text exposition with the reference's 13 metric families
(crates/sllm-server/src/metrics.rs:20-36): fixed label enums, at most 16 model aliases, no prompt,
token, key or error text anywhere."""
from __future__ import annotations

import threading

TTFT_BUCKETS = (0.01, 0.025, 0.05, 0.1, 0.25, 0.5, 1.0, 2.5, 5.0, 10.0, 30.0)
MAX_MODELS = 16
OUTCOMES = ("completed", "cancelled", "failed", "rejected", "timeout")
TOKEN_KINDS = ("prompt", "completion")
CANCEL_REASONS = ("client_disconnect", "admin", "timeout", "shutdown")


class ServerMetrics:
    def __init__(self, model_aliases):
        self.models = list(model_aliases)[:MAX_MODELS]
        self._lock = threading.Lock()
        self.requests = {(m, o): 0 for m in self.models for o in OUTCOMES}
        self.tokens = {(m, k): 0 for m in self.models for k in TOKEN_KINDS}
        self.cancellations = {r: 0 for r in CANCEL_REASONS}
        self.http = {}
        self.ttft_sum = {m: 0.0 for m in self.models}
        self.ttft_count = {m: 0 for m in self.models}
        self.ttft_buckets = {m: [0] * (len(TTFT_BUCKETS) + 1) for m in self.models}

    def request(self, model, outcome):
        with self._lock:
            if (model, outcome) in self.requests:
                self.requests[(model, outcome)] += 1

    def add_tokens(self, model, kind, n):
        with self._lock:
            if (model, kind) in self.tokens:
                self.tokens[(model, kind)] += int(n)

    def ttft(self, model, seconds):
        with self._lock:
            if model not in self.ttft_sum:
                return
            self.ttft_sum[model] += seconds
            self.ttft_count[model] += 1
            for i, b in enumerate(TTFT_BUCKETS):
                if seconds <= b:
                    self.ttft_buckets[model][i] += 1
            self.ttft_buckets[model][-1] += 1

    def cancellation(self, reason):
        with self._lock:
            if reason in self.cancellations:
                self.cancellations[reason] += 1

    def http_response(self, status):
        klass = f"{status // 100}xx"
        with self._lock:
            self.http[klass] = self.http.get(klass, 0) + 1

    def render(self, scheduler_stats: dict, ready: bool, memory: dict) -> str:
        out = []

        def fam(name, typ, help_):
            out.append(f"# HELP {name} {help_}")
            out.append(f"# TYPE {name} {typ}")
        with self._lock:
            fam("sllm_requests_total", "counter", "Requests by terminal outcome.")
            for (m, o), v in sorted(self.requests.items()):
                out.append(f'sllm_requests_total{{model="{m}",outcome="{o}"}} {v}')
            fam("sllm_tokens_total", "counter", "Tokens processed.")
            for (m, k), v in sorted(self.tokens.items()):
                out.append(f'sllm_tokens_total{{model="{m}",kind="{k}"}} {v}')
            fam("sllm_request_ttft_seconds", "histogram", "Time to first token.")
            for m in self.models:
                for i, b in enumerate(TTFT_BUCKETS):
                    out.append(f'sllm_request_ttft_seconds_bucket{{model="{m}",le="{b}"}} {self.ttft_buckets[m][i]}')
                out.append(f'sllm_request_ttft_seconds_bucket{{model="{m}",le="+Inf"}} {self.ttft_buckets[m][-1]}')
                out.append(f'sllm_request_ttft_seconds_sum{{model="{m}"}} {self.ttft_sum[m]:.6f}')
                out.append(f'sllm_request_ttft_seconds_count{{model="{m}"}} {self.ttft_count[m]}')
            fam("sllm_cancellations_total", "counter", "Cancellations by reason.")
            for r, v in sorted(self.cancellations.items()):
                out.append(f'sllm_cancellations_total{{reason="{r}"}} {v}')
            fam("sllm_http_responses_total", "counter", "HTTP responses by status class.")
            for k, v in sorted(self.http.items()):
                out.append(f'sllm_http_responses_total{{class="{k}"}} {v}')
        for name, key, help_ in (("sllm_scheduler_accepting", "accepting", "1 while the scheduler accepts work."),
                                 ("sllm_scheduler_active_requests", "active_requests", "Requests being generated."),
                                 ("sllm_scheduler_queue_capacity", "queue_capacity", "Configured queue capacity."),
                                 ("sllm_scheduler_queue_depth", "queue_depth", "Requests waiting."),
                                 ("sllm_scheduler_slots", "slots", "Concurrent decode rows.")):
            fam(name, "gauge", help_)
            out.append(f"{name} {int(scheduler_stats.get(key, 0))}")
        fam("sllm_model_ready", "gauge", "1 when the model lifecycle is ready.")
        for m in self.models:
            out.append(f'sllm_model_ready{{model="{m}"}} {1 if ready else 0}')
        fam("sllm_backend_memory_bytes", "gauge", "Tracked device allocations by category.")
        for cat, v in sorted(memory.items()):
            out.append(f'sllm_backend_memory_bytes{{category="{cat}"}} {int(v)}')
        return "\n".join(out) + "\n"
