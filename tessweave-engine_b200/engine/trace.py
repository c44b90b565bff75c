"""Bounded JSONL audit of scheduler events.

One JSON object per line: ``{"time", "monotonic", "event", ...}`` with the events
``launch, loaded, submit, admit, first_token, step, finish, fatal``.  Prompts, text
and token ids are never written.  The file is rotated at 20 MiB and four older
files are kept, as in the reference (flow_engine/trace.py:9-28).
"""
from __future__ import annotations

import json
import os
import threading
import time
from pathlib import Path

MAX_BYTES = 20 * 1024 * 1024
KEEP = 4


class Trace:
    def __init__(self, path=None):
        self.lock = threading.Lock()
        self.path = Path(path) if path else None
        self.file = None
        if self.path:
            self.path.parent.mkdir(parents=True, exist_ok=True)
            self.file = open(self.path, "a", encoding="utf-8")

    def _rotate(self) -> None:
        self.file.close()
        for i in range(KEEP, 0, -1):
            older = self.path.with_name(f"{self.path.name}.{i}")
            newer = self.path if i == 1 else self.path.with_name(f"{self.path.name}.{i - 1}")
            if newer.exists():
                os.replace(newer, older)
        self.file = open(self.path, "a", encoding="utf-8")

    def emit(self, kind: str, **data) -> None:
        if self.file is None:
            return
        row = json.dumps({"time": time.time(), "monotonic": time.monotonic(), "event": kind, **data}, allow_nan=False)
        with self.lock:
            if self.file.tell() + len(row) + 1 > MAX_BYTES:
                self._rotate()
            self.file.write(row + "\n")
            self.file.flush()

    def close(self) -> None:
        with self.lock:
            if self.file is not None:
                self.file.close()
                self.file = None
