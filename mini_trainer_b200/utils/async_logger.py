"""Append-only JSONL metrics logger that never blocks the training loop.

Behaviour of the reference ``AsyncStructuredLogger`` (async_structured_logger.py:13-61): an
existing file is read back into ``logs`` on start, ``log_sync(dict)`` returns immediately, each
record gets an ISO ``timestamp``, is appended as one JSON line and echoed to stdout in green.
Here the writer is a plain daemon thread draining a queue (no asyncio/aiofiles dependency);
``flush()`` waits until everything queued so far is on disk.
"""
from __future__ import annotations

import json
import queue
import threading
from datetime import datetime


class AsyncStructuredLogger:
    def __init__(self, file_name: str = "training_log.jsonl", echo: bool = True):
        self.file_name = file_name
        self.echo = echo
        self.logs = []
        try:
            with open(file_name, "r") as f:
                for line in f:
                    if line.strip():
                        self.logs.append(json.loads(line))
        except FileNotFoundError:
            pass
        self._q: queue.Queue = queue.Queue()
        self._t = threading.Thread(target=self._drain, daemon=True, name="mtb200-jsonl")
        self._t.start()

    def _drain(self) -> None:
        while True:
            data = self._q.get()
            try:
                if data is None:
                    return
                if not isinstance(data, dict):
                    raise ValueError("Logged data must be a dictionary")
                data["timestamp"] = datetime.now().isoformat()
                self.logs.append(data)
                with open(self.file_name, "a") as f:
                    f.write(json.dumps(data, indent=None) + "\n")
                if self.echo:
                    print(f"\033[92m{json.dumps(data, indent=4)}\033[0m")
            except Exception as e:  # a logging failure must not kill training
                print(f"\033[1;38;2;0;255;255mError logging data: {e}\033[0m")
            finally:
                self._q.task_done()

    def log_sync(self, data: dict) -> None:
        self._q.put(data)

    def flush(self) -> None:
        self._q.join()

    def close(self) -> None:
        self.flush()
        self._q.put(None)

    def __repr__(self) -> str:
        return f"<AsyncStructuredLogger(file_name={self.file_name})>"
