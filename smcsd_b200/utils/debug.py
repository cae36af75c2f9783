"""JSONL diagnostics: append-only records for offline inspection of an SMC run.

Each record carries the process id and a nanosecond timestamp; the files are named by
``SMC_DIAG_PATH`` and ``SMC_PROBE_RECORD_PATH`` (the reference's recorder:
smcsd/common/debug.py:1-30, which reads SGLANG_SMC_DIAG_PATH / SGLANG_SMC_PROBE_RECORD_PATH;
those names are honoured too).
"""
from __future__ import annotations

import json
import os
import time
from typing import Any, Dict, Optional


def _path(*names: str) -> Optional[str]:
    for n in names:
        p = os.environ.get(n)
        if p:
            return p
    return None


def _append(path: Optional[str], record: Dict[str, Any]) -> None:
    if not path:
        return
    rec = {"pid": os.getpid(), "timestamp_ns": time.time_ns()}
    rec.update(record)
    with open(path, "a") as f:
        f.write(json.dumps(rec, default=str) + "\n")


def append_diag_record(record: Dict[str, Any]) -> None:
    _append(_path("SMC_DIAG_PATH", "SGLANG_SMC_DIAG_PATH"), record)


def append_probe_record(record: Dict[str, Any]) -> None:
    _append(_path("SMC_PROBE_RECORD_PATH", "SGLANG_SMC_PROBE_RECORD_PATH"), record)
