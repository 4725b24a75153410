"""Leveled diagnostics on stderr; answers go to stdout.

Same split as the reference CLI (src/apps/ninfer.cpp:2, src/common/log.h:11-32):
one global level, four severities, `--log-level debug|info|warn|error`.
"""

from __future__ import annotations

import sys
import time

LEVELS = {"debug": 0, "info": 1, "warn": 2, "error": 3}
_level = LEVELS["warn"]
_t0 = time.time()


def set_level(name: str) -> None:
    global _level
    if name not in LEVELS:
        raise ValueError(f"unknown log level {name!r}; choose from {sorted(LEVELS)}")
    _level = LEVELS[name]


def _emit(tag: str, lvl: int, msg: str) -> None:
    if lvl >= _level:
        sys.stderr.write(f"[{tag} {time.time() - _t0:8.2f}s] {msg}\n")
        sys.stderr.flush()


def debug(msg: str) -> None:
    _emit("D", 0, msg)


def info(msg: str) -> None:
    _emit("I", 1, msg)


def warn(msg: str) -> None:
    _emit("W", 2, msg)


def error(msg: str) -> None:
    _emit("E", 3, msg)
