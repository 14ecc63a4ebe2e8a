"""Per-op evidence runners: one correctness check against the fp32 restatement of the op plus one timing with roofline
fractions, written as a schema'd JSON report (`python -m sllm_b200.evidence --help`)."""
from .runner import OPS, SCHEMA, run_op, unavailable_report, validate_report  # noqa: F401
