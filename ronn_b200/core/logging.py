"""Structured logging (crates/ronn-core/src/logging.rs:16-196).

``LoggingConfig{level, timestamps, thread_ids, source_location, span_events, json_format}`` with
development / production presets; ``RONN_LOG`` (or ``RUST_LOG``, honoured for parity) overrides
the level.
"""
from __future__ import annotations

import json
import logging
import os
import sys
from dataclasses import dataclass

_LEVELS = {"trace": 5, "debug": logging.DEBUG, "info": logging.INFO, "warn": logging.WARNING,
           "warning": logging.WARNING, "error": logging.ERROR}


@dataclass
class LoggingConfig:
    level: str = "info"
    timestamps: bool = True
    thread_ids: bool = False
    source_location: bool = False
    span_events: bool = False
    json_format: bool = False

    @staticmethod
    def development() -> "LoggingConfig":
        return LoggingConfig("debug", True, True, True, True, False)

    @staticmethod
    def production() -> "LoggingConfig":
        return LoggingConfig("info", True, False, False, False, True)


class _JsonFormatter(logging.Formatter):
    def __init__(self, cfg: LoggingConfig):
        super().__init__()
        self.cfg = cfg

    def format(self, record: logging.LogRecord) -> str:
        d = {"level": record.levelname, "target": record.name, "message": record.getMessage()}
        if self.cfg.timestamps:
            d["timestamp"] = self.formatTime(record, "%Y-%m-%dT%H:%M:%S")
        if self.cfg.thread_ids:
            d["thread_id"] = record.thread
        if self.cfg.source_location:
            d["file"], d["line"] = record.pathname, record.lineno
        extra = getattr(record, "fields", None)
        if extra:
            d["fields"] = extra
        return json.dumps(d)


def init_logging(config: LoggingConfig = None, stream=None) -> logging.Logger:
    cfg = config or LoggingConfig()
    level = os.environ.get("RONN_LOG") or os.environ.get("RUST_LOG") or cfg.level
    logger = logging.getLogger("ronn_b200")
    logger.setLevel(_LEVELS.get(level.lower(), logging.INFO))
    for h in list(logger.handlers):
        logger.removeHandler(h)
    handler = logging.StreamHandler(stream or sys.stderr)
    if cfg.json_format:
        handler.setFormatter(_JsonFormatter(cfg))
    else:
        parts = []
        if cfg.timestamps:
            parts.append("%(asctime)s")
        parts.append("%(levelname)s")
        if cfg.thread_ids:
            parts.append("[%(thread)d]")
        parts.append("%(name)s")
        if cfg.source_location:
            parts.append("%(filename)s:%(lineno)d")
        parts.append("%(message)s")
        handler.setFormatter(logging.Formatter(" ".join(parts)))
    logger.addHandler(handler)
    logger.propagate = False
    return logger
