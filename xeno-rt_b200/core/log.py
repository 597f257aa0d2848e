"""Stderr logging behind one environment variable.

The reference logs through ``tracing`` with an env filter and default "info"
(crates/xrt-cli/src/main.rs:67-71); its README names ``XRT_LOG``.  Here ``XRT_LOG``
is one of error, warn, info, debug (default info).
"""
from __future__ import annotations

import os
import sys

_LEVELS = {"error": 0, "warn": 1, "info": 2, "debug": 3}


def log_level() -> int:
    return _LEVELS.get(os.environ.get("XRT_LOG", "info").lower(), 2)


def log(level: str, message: str) -> None:
    if _LEVELS[level] <= log_level():
        print(f"[xrt {level}] {message}", file=sys.stderr, flush=True)
