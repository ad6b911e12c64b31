"""Structured run log: one JSON object per line.

The reference only prints (args, per-epoch mean loss and loss scale, the evaluation table; dl_base.py:386-389,
853-855).  ``JsonlLogger`` keeps those prints and additionally appends machine-readable records —
per epoch: mean sampled loss, loss scale, skipped optimizer steps, device-timed step milliseconds and
samples/s; per evaluation: the metric table — to ``{out_dir}/{name}_log.jsonl`` on rank 0.
"""
from __future__ import annotations

import json
import os
import time


class JsonlLogger:
    def __init__(self, path: str | None, enabled: bool = True, echo=print):
        self.path = path if enabled else None
        self.echo = echo
        if self.path:
            os.makedirs(os.path.dirname(os.path.abspath(self.path)), exist_ok=True)

    def log(self, kind: str, **fields) -> dict:
        rec = {"t": round(time.time(), 3), "kind": kind, **fields}
        if self.path:
            with open(self.path, "a") as f:
                f.write(json.dumps(rec, default=float) + "\n")
        return rec

    def __call__(self, message: str) -> None:     # drop-in for print
        if self.echo is not None:
            self.echo(message)
        self.log("message", text=str(message))


def read_jsonl(path: str) -> list[dict]:
    with open(path) as f:
        return [json.loads(line) for line in f if line.strip()]
