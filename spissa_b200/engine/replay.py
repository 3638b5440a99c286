"""Trace replay over the engine's own step function (the body of ``bin/trace_run``).

A trace is a stream of steps; a step names requests by id, brings each one's next
tokens and says where logits are wanted. A request takes a slot at its first step and
gives it back when a step lists it under ``end``. Nothing is sampled.
"""
from __future__ import annotations

import json
import os

import numpy as np
import torch

from .engine import Engine


def replay(model_dir, dtype: str, out_dir, max_tokens: int, lines, done_out, device="cuda:0") -> int:
    page = Engine.PAGE_SIZE
    n_pages = (max_tokens + page - 1) // page
    engine = Engine.from_folder(model_dir, dtype=dtype, max_tokens=n_pages * page, max_seqs=max(1, n_pages),
                                device=device)
    slots: dict = {}
    for line in lines:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step_no = rec["step"]
        entries = []
        for e in rec.get("entries", []):
            rid = e["id"]
            if rid not in slots:
                slots[rid] = engine.acquire()
            entries.append((slots[rid], e["tokens"], e.get("want", [])))
        if entries:
            logits = engine.step(entries)
            if logits.shape[0] > 0:
                arr = logits.to(torch.float32).cpu().numpy().astype("<f4", copy=False)
                tmp = os.path.join(out_dir, f".{step_no}.f32.tmp")
                arr.tofile(tmp)
                os.replace(tmp, os.path.join(out_dir, f"{step_no}.f32"))
            # ``step`` waited for the device's status word: a kernel that gave up a bounded wait has raised by now
        for rid in rec.get("end", []):
            if rid in slots:
                engine.release(slots.pop(rid))
        done_out.write(f"done {step_no}\n")
        done_out.flush()
    return 0
