"""Bounded read of a client chat-template file (regular file, <= 64 KiB, UTF-8)
(reference: crates/sllm-cli/src/template_file.rs)."""
from __future__ import annotations

import os
import stat

from .common import CliError

MAX_TEMPLATE_BYTES = 64 * 1024


def read_template_file(path: str) -> str:
    try:
        st = os.lstat(path)
    except OSError as exc:
        raise CliError(f"cannot read the template file: {exc}") from None
    if not stat.S_ISREG(st.st_mode):
        raise CliError("the template file must be a regular, non-symlink file")
    if st.st_size > MAX_TEMPLATE_BYTES:
        raise CliError("the template file exceeds 64 KiB")
    with open(path, "rb") as f:
        raw = f.read(MAX_TEMPLATE_BYTES + 1)
    try:
        return raw.decode("utf-8")
    except UnicodeDecodeError:
        raise CliError("the template file is not UTF-8") from None
