"""Compact structured logging: ``MM-dd HH:MM:SS.us LEVEL module file:line msg k=v``.

The level filter comes from ``PEGAINFER_LOG`` (e.g. ``info``, ``debug``,
``warning,pegainfer_b200.sched=debug``); noisy HTTP libraries are clamped to warning.

Reference parity: pegainfer-core/src/logging.rs:36-233.
"""
from __future__ import annotations

import logging
import os
import time

_NOISY = ("uvicorn.access", "uvicorn.error", "httpx", "httpcore", "asyncio", "urllib3")


class _Fmt(logging.Formatter):
    def format(self, r: logging.LogRecord) -> str:
        t = time.localtime(r.created)
        ts = f"{t.tm_mon:02d}-{t.tm_mday:02d} {t.tm_hour:02d}:{t.tm_min:02d}:{t.tm_sec:02d}.{int((r.created % 1) * 1e6):06d}"
        msg = r.getMessage()
        kv = getattr(r, "kv", None)
        if kv:
            msg += " " + " ".join(f"{k}={v}" for k, v in kv.items())
        return f"{ts} {r.levelname:<5} {r.name} {r.filename}:{r.lineno} {msg}"


def init_default(spec: str = None) -> None:
    spec = spec if spec is not None else os.environ.get("PEGAINFER_LOG", "info")
    root_level = logging.INFO
    per_module = {}
    for part in filter(None, (p.strip() for p in spec.split(","))):
        if "=" in part:
            mod, lvl = part.split("=", 1)
            per_module[mod] = getattr(logging, lvl.upper(), logging.INFO)
        else:
            root_level = getattr(logging, part.upper(), logging.INFO)
    h = logging.StreamHandler()
    h.setFormatter(_Fmt())
    root = logging.getLogger()
    root.handlers[:] = [h]
    root.setLevel(root_level)
    for n in _NOISY:
        logging.getLogger(n).setLevel(max(root_level, logging.WARNING))
    for mod, lvl in per_module.items():
        logging.getLogger(mod).setLevel(lvl)


def kv(logger: logging.Logger, level: int, msg: str, **fields) -> None:
    logger.log(level, msg, extra={"kv": fields}, stacklevel=2)
