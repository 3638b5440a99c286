"""The generation loop above the step function.

Requests are token lists of unequal lengths. They are served in batches: the prompts
of a batch run in ONE step, then every live sequence gets one token per step. A
sequence ends on a stop token or at its token limit; it leaves the batch and its slot
is returned at once, so later batches use it again. The shape of a turn follows the
reference (crates/spissa-runtime/src/session.rs:290-472: prefill gives the first
token, then one ``append`` per token; the token that ends a turn is returned but not
fed, :376,:432; the projected length is checked before anything runs, :307-320; the
stop test lives in the caller's callback, crates/spissa-cli/src/commands/chat.rs:617-625).

The loop needs from its engine only ``acquire()``, ``release(slot)``, ``step(entries)``
and the numbers ``free_tokens()`` / ``page_size`` for planning, and from its sampler
``sample(logits, params, requests, step)``; tests drive it with scripted fakes.

When the engine also offers ``step_device`` (tokens taken from a device tensor) and nobody
listens token by token, decoding runs one step ahead of the host: the sampler's output feeds
the next step on the device, and the host reads a step's tokens while the next step runs. A
stop token is then seen one step late; the sequence's extra token is dropped and its slot is
returned as before, so results are the same as in the step-by-step loop.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, Optional

from ..sampling import SamplingParams


@dataclass
class GenerationResult:
    request: int
    prompt_tokens: int
    tokens: list = field(default_factory=list)
    finish_reason: str = ""            # "stop" or "length"
    logits: Optional[list] = None      # per generated token, when asked for


@dataclass
class GenerationMetrics:
    batches: int = 0
    steps: int = 0
    prompt_tokens: int = 0
    generated_tokens: int = 0
    prefill_ms: float = 0.0
    decode_ms: float = 0.0
    ttft_ms: float = 0.0
    batches_first_tokens: int = 0      # tokens that came out of prefill steps

    @property
    def decode_tok_s(self) -> float:
        n = self.generated_tokens - self.batches_first_tokens
        return n / (self.decode_ms / 1000.0) if self.decode_ms > 0 and n > 0 else 0.0


def _rounded(n: int, page: int) -> int:
    return (n + page - 1) // page * page


def plan_batches(prompt_lens: list, max_new_tokens: int, token_budget: int, max_seqs: int,
                 page_size: int, max_batch: Optional[int] = None) -> list:
    """Cut the requests, in order, into batches that fit the cache.

    A request needs room for its prompt and all tokens it may generate but the last,
    rounded up to whole pages. Raises if a single request cannot fit.
    """
    cap = min(max_seqs, max_batch) if max_batch else max_seqs
    if cap <= 0:
        raise ValueError("a batch needs room for at least one sequence")
    batches, cur, used = [], [], 0
    for i, n in enumerate(prompt_lens):
        need = _rounded(n + max(max_new_tokens - 1, 0), page_size)
        if need > token_budget:
            raise ValueError(f"request {i} needs room for {need} tokens, the cache holds {token_budget}")
        if cur and (len(cur) >= cap or used + need > token_budget):
            batches.append(cur)
            cur, used = [], 0
        cur.append(i)
        used += need
    if cur:
        batches.append(cur)
    return batches


def _decode_ahead(engine, sampler, params, live, results, stop, max_new_tokens, metrics, greedy=False) -> int:
    """Decode ``live`` = [(request, slot)] to the end, one step ahead of the host. Returns the steps run.

    Every live request has its last token in ``results`` and on the host. A launch takes its tokens from the
    device tensor that the launch before sampled into; the host reads that tensor, through pinned memory, only
    after the next launch is queued. Limits by length are known when a step is launched; a stop token shows one
    step late, so a request that stopped may have run one step too many: that step's token is dropped.
    """
    import torch
    device = torch.device(engine.device)
    on_gpu = device.type == "cuda"                 # a scripted engine on the CPU drives the same decisions in tests
    done = set()                                   # requests that ended (their slots are released)
    emitted = {req: len(results[req].tokens) for req, _ in live}       # tokens out, counting those still in flight
    token_source = torch.tensor([results[req].tokens[-1] for req, _ in live], dtype=torch.int32).to(device)
    order = list(live)                             # row i of token_source belongs to order[i]
    in_flight = []                                 # [(order, pinned tokens, event)] oldest first
    steps = 0
    # the tokens come back through three pinned buffers used in turn (two steps are in flight at most): asking the
    # pinned allocator for a new one every step costs more than the copy
    landing = [torch.empty(len(live), dtype=torch.int32, pin_memory=on_gpu) for _ in range(3)]
    engine_settles = hasattr(engine, "settle")
    # an engine with per-slot headers on the device: the sampler notes its tokens there and a step takes them from
    # there by slot; otherwise a step takes them from the tensor that the sampler returned, by row
    headers = hasattr(engine, "step_note") and engine.step_note() is not None

    def settle(entry):
        rows, pinned, event = entry
        if event is not None:
            event.synchronize()
        if engine_settles:
            engine.settle()                        # the step's status word arrived before its tokens: confirm it, or
                                                   # roll it and the one in flight back and raise
        for (req, slot), tok in zip(rows, pinned.tolist()):
            if req in done:
                continue                           # it stopped a step earlier: this token was never asked for
            res = results[req]
            res.tokens.append(int(tok))
            metrics.generated_tokens += 1
            if int(tok) in stop:
                res.finish_reason = "stop"
            elif len(res.tokens) >= max_new_tokens:
                res.finish_reason = "length"
            if res.finish_reason:
                done.add(req)
                engine.release(slot)

    while True:
        nxt = [(i, rs) for i, rs in enumerate(order) if rs[0] not in done and emitted[rs[0]] < max_new_tokens]
        if not nxt:
            break
        rows = [i for i, _ in nxt]
        order = [rs for _, rs in nxt]
        step_no = emitted[order[0][0]]             # every request of a batch has the same count: they started together
        if greedy:
            # the head keeps only the best candidate of each row: no logits exist, the step returns the tokens
            token_source = engine.step_device([slot for _, slot in order], greedy=True)
        elif headers:
            logits = engine.step_device([slot for _, slot in order])
            token_source = sampler.sample(logits, params, [req for req, _ in order], step_no, note=engine.step_note())
        else:
            logits = engine.step_device([slot for _, slot in order], token_source, rows)
            token_source = sampler.sample(logits, params, [req for req, _ in order], step_no)
        pinned = landing[steps % 3][:len(order)]
        pinned.copy_(token_source, non_blocking=True)
        event = None
        if on_gpu:
            event = torch.cuda.Event()
            event.record()
        for req, _ in order:
            emitted[req] += 1
        in_flight.append((order, pinned, event))
        steps += 1
        if len(in_flight) > 1:
            settle(in_flight.pop(0))               # the step before the one just queued
    while in_flight:
        settle(in_flight.pop(0))
    return steps


def generate(engine, sampler, prompts: list, max_new_tokens: int, params: SamplingParams = SamplingParams(),
             stop_ids=(), max_batch: Optional[int] = None, on_token: Optional[Callable] = None,
             return_logits: bool = False, token_budget: Optional[int] = None):
    """Generate for every prompt; returns (results in request order, metrics).

    ``on_token(request, token) -> bool`` is called for every new token; returning False ends that
    request (reason "stop"), like the reference's callback.
    """
    if max_new_tokens <= 0:
        raise ValueError("max_new_tokens must be greater than zero")
    for i, p in enumerate(prompts):
        if len(p) == 0:
            raise ValueError(f"request {i} has an empty prompt")
    limit = getattr(engine, "max_position", None)
    if limit:
        # the last token is returned but not fed: a request stands at prompt + max_new_tokens - 1 positions at most
        for i, p in enumerate(prompts):
            if len(p) + max_new_tokens - 1 > limit:
                raise ValueError(f"request {i}: {len(p)} prompt tokens and {max_new_tokens} new ones pass the "
                                 f"model's {limit} positions")
    stop = set(int(s) for s in stop_ids)
    page = getattr(engine, "page_size", 64)
    budget = token_budget if token_budget is not None else engine.free_tokens()
    max_seqs = getattr(engine, "max_seqs", len(prompts))
    batches = plan_batches([len(p) for p in prompts], max_new_tokens, budget, max_seqs, page, max_batch)
    results = [GenerationResult(i, len(p)) for i, p in enumerate(prompts)]
    if return_logits:
        for r in results:
            r.logits = []
    metrics = GenerationMetrics()
    t_start = time.perf_counter()
    # greedy and nobody wants the logits: the engine's head returns the tokens and never writes a row of logits
    # (the reference's greedy head does the same, crates/spissa-runtime/src/models/llama/session/mod.rs:662-669)
    greedy = params.greedy and not return_logits and getattr(engine, "greedy_steps", False)

    def take(live, tokens, logits):
        """Record one new token per live request; return those that go on."""
        go_on = []
        for row, (req, slot) in enumerate(live):
            tok = int(tokens[row])
            res = results[req]
            res.tokens.append(tok)
            if return_logits:
                res.logits.append(logits[row].float().cpu())
            metrics.generated_tokens += 1
            keep = on_token(req, tok) if on_token else True
            if tok in stop or keep is False:
                res.finish_reason = "stop"
            elif len(res.tokens) >= max_new_tokens:
                res.finish_reason = "length"
            if res.finish_reason:
                engine.release(slot)
            else:
                go_on.append((req, slot))
        return go_on

    for batch in batches:
        metrics.batches += 1
        live = [(req, engine.acquire()) for req in batch]
        try:
            t0 = time.perf_counter()
            entries = [(slot, prompts[req], [len(prompts[req]) - 1]) for req, slot in live]
            if greedy:
                logits, first = None, engine.step(entries, greedy=True)
            else:
                logits = engine.step(entries)
                note = engine.step_note() if hasattr(engine, "step_note") else None
                first = sampler.sample(logits, params, [r for r, _ in live], 0, **({"note": note} if note is not None else {}))
            tokens = first.tolist()
            t1 = time.perf_counter()
            metrics.steps += 1
            metrics.prompt_tokens += sum(len(prompts[r]) for r, _ in live)
            metrics.prefill_ms += (t1 - t0) * 1000.0
            metrics.batches_first_tokens += len(live)
            if metrics.ttft_ms == 0.0:
                metrics.ttft_ms = (t1 - t_start) * 1000.0
            live = take(live, tokens, logits)
            step_no = 1
            if live and on_token is None and not return_logits and hasattr(engine, "step_device"):
                t0 = time.perf_counter()
                metrics.steps += _decode_ahead(engine, sampler, params, live, results, stop, max_new_tokens, metrics,
                                               greedy)
                metrics.decode_ms += (time.perf_counter() - t0) * 1000.0
                live = []
            while live:
                t0 = time.perf_counter()
                entries = [(slot, [results[req].tokens[-1]], [0]) for req, slot in live]
                if greedy:
                    logits, tokens = None, engine.step(entries, greedy=True).tolist()
                else:
                    logits = engine.step(entries)
                    tokens = sampler.sample(logits, params, [r for r, _ in live], step_no).tolist()
                metrics.decode_ms += (time.perf_counter() - t0) * 1000.0
                metrics.steps += 1
                live = take(live, tokens, logits)
                step_no += 1
        except BaseException:
            for _, slot in live:
                try:
                    engine.release(slot)
                except Exception:
                    pass
            raise
    return results, metrics
