"""Builders of replay traces: the same requests cut into steps in different ways."""
import io
import json
import os

import numpy as np
import torch


def whole(requests: dict) -> list:
    """Each request alone, all its tokens in one step, logits everywhere."""
    steps = []
    for rid, toks in requests.items():
        steps.append(dict(step=len(steps), entries=[dict(id=rid, tokens=toks, want=list(range(len(toks))))],
                          end=[rid]))
    return steps


def tail_one_by_one(requests: dict, tail: int = 32) -> list:
    """Each request alone: all but the last ``tail`` tokens in one step, the rest one by one."""
    steps = []
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        steps.append(dict(step=len(steps), entries=[dict(id=rid, tokens=toks[:head], want=list(range(head)))],
                          end=[rid] if head == len(toks) else []))
        for i in range(head, len(toks)):
            steps.append(dict(step=len(steps), entries=[dict(id=rid, tokens=[toks[i]], want=[0])],
                              end=[rid] if i == len(toks) - 1 else []))
    return steps


def ragged_batches(requests: dict, batch_size: int, decode_counts: dict) -> list:
    """Batches of unequal lengths, one after another; shorter requests end earlier.

    A batch's first step carries each request's tokens but its last ``decode_counts[id]``
    (at least one token stays in the first step); then every live request brings one token
    per step until it has none left, and ends.
    """
    ids = list(requests)
    steps = []
    for b0 in range(0, len(ids), batch_size):
        group = ids[b0:b0 + batch_size]
        fed = {}
        entries, end = [], []
        for rid in group:
            toks = requests[rid]
            head = max(1, len(toks) - decode_counts.get(rid, 0))
            entries.append(dict(id=rid, tokens=toks[:head], want=list(range(head))))
            fed[rid] = head
            if head == len(toks):
                end.append(rid)
        steps.append(dict(step=len(steps), entries=entries, end=end))
        live = [r for r in group if fed[r] < len(requests[r])]
        while live:
            entries, end = [], []
            for rid in live:
                entries.append(dict(id=rid, tokens=[requests[rid][fed[rid]]], want=[0]))
                fed[rid] += 1
                if fed[rid] == len(requests[rid]):
                    end.append(rid)
            steps.append(dict(step=len(steps), entries=entries, end=end))
            live = [r for r in live if fed[r] < len(requests[r])]
    return steps


def tokens_needed(steps: list, page: int = 64) -> int:
    """The most tokens live requests hold at any time, each rounded up to a multiple of ``page``."""
    held, peak = {}, 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum((n + page - 1) // page * page for n in held.values()))
        for rid in s["end"]:
            held.pop(rid, None)
    return peak


def collect(steps: list, out_dir, vocab: int) -> dict:
    """(request id, position) -> logits row, read back from the files a replay wrote."""
    pos = {}
    got = {}
    for s in steps:
        rows = []
        for e in s["entries"]:
            base = pos.get(e["id"], 0)
            rows.extend((e["id"], base + w) for w in e["want"])
            pos[e["id"]] = base + len(e["tokens"])
        if not rows:
            continue
        arr = np.fromfile(os.path.join(out_dir, f"{s['step']}.f32"), dtype="<f4").reshape(len(rows), vocab)
        for key, row in zip(rows, arr):
            got[key] = torch.from_numpy(row.copy())
    return got


def run_in_process(folder, dtype, steps, out_dir, max_tokens=None):
    """Replay through the library's replay function (the body of bin/trace_run)."""
    from spissa_b200.engine.replay import replay
    os.makedirs(out_dir, exist_ok=True)
    lines = io.StringIO("".join(json.dumps(s) + "\n" for s in steps))
    done = io.StringIO()
    rc = replay(folder, dtype, out_dir, max_tokens or tokens_needed(steps), lines, done)
    assert rc == 0
    assert done.getvalue().split() == [x for s in steps for x in ("done", str(s["step"]))]
