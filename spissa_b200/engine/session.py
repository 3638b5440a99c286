"""A persistent chat session: one sequence that keeps its cache across turns.

Shape of a turn as in the reference (crates/spissa-runtime/src/session.rs:290-472): the
last generated token of the previous turn is not in the cache yet (:376, :432), so it is
fed first (:330-348) together with the new user tokens; the prefill gives the first token,
then one step per token until ``max_new_tokens`` or until ``on_token`` returns False. The
projected length is checked before anything runs (:307-320).
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field

from ..sampling import Sampler, SamplingParams


@dataclass
class TurnResult:
    tokens: list
    finish_reason: str
    ttft_ms: float
    prefill_ms: float
    decode_ms: float
    decode_tok_s: float
    context_len: int
    first_step_logits: object = None


class ChatSession:
    def __init__(self, engine, params: SamplingParams = SamplingParams(), max_seq_len: int | None = None):
        self.engine = engine
        self.params = params
        self.sampler = Sampler(engine.device)
        self.slot = engine.acquire()
        self.history: list = []
        self.pending = None                  # the last generated token, not yet in the cache
        self.turn = 0
        room = engine.free_tokens() + engine.length(self.slot)
        model_limit = getattr(engine, "max_position", None)
        if model_limit:
            room = min(room, model_limit)            # the reference caps a session by max_seq_len (session.rs:307-320)
        self.max_seq_len = min(max_seq_len, room) if max_seq_len else room

    def close(self):
        if self.slot is not None:
            self.engine.release(self.slot)
            self.slot = None

    def generate_turn(self, user_tokens, max_new_tokens: int, on_token=None, stop_ids=(),
                      keep_logits: bool = False) -> TurnResult:
        if not user_tokens:
            raise ValueError("a chat turn needs at least one user token")
        if max_new_tokens <= 0:
            raise ValueError("max_new_tokens must be greater than zero")
        projected = len(self.history) + len(user_tokens) + max_new_tokens
        if projected > self.max_seq_len:
            raise ValueError(f"the context would reach {projected} tokens, the limit is {self.max_seq_len}")
        stop = set(int(s) for s in stop_ids)
        t0 = time.perf_counter()
        feed = ([self.pending] if self.pending is not None else []) + list(user_tokens)
        # greedy and nobody wants the logits: the head returns the token and writes no logits, as the reference's does
        # (crates/spissa-runtime/src/models/llama/session/mod.rs:662-669)
        greedy = self.params.greedy and not keep_logits and getattr(self.engine, "greedy_steps", False)

        def next_token(tokens, want, draw):
            if greedy:
                return int(self.engine.step([(self.slot, tokens, want)], greedy=True).tolist()[0]), None
            logits = self.engine.step([(self.slot, tokens, want)])
            return int(self.sampler.sample(logits, self.params, [0], draw).tolist()[0]), logits

        tok, logits = next_token(feed, [len(feed) - 1], self.turn * 1_000_003)
        t1 = time.perf_counter()
        first_logits = logits[0].float().cpu() if keep_logits else None
        self.history.extend(user_tokens)
        out = []
        reason = "length"
        step = 1
        while True:
            out.append(tok)
            self.history.append(tok)
            self.pending = tok
            keep = on_token(tok) if on_token else True
            if tok in stop or keep is False:
                reason = "stop"
                break
            if len(out) >= max_new_tokens:
                break
            tok, _ = next_token([tok], [0], self.turn * 1_000_003 + step)
            step += 1
        t2 = time.perf_counter()
        self.turn += 1
        n_dec = len(out) - 1
        dec_ms = (t2 - t1) * 1000.0
        return TurnResult(out, reason, (t1 - t0) * 1000.0, (t1 - t0) * 1000.0, dec_ms,
                          n_dec / (dec_ms / 1000.0) if n_dec and dec_ms > 0 else 0.0,
                          self.engine.length(self.slot), first_logits)
