"""Decisions of the generation loop, driven with a scripted engine and sampler (no GPU).

The reference tests its loop the same way, with a recording fake adapter
(crates/spissa-runtime/src/session.rs:495-663).
"""
import pytest

from spissa_b200.engine.generate import generate, plan_batches
from spissa_b200.sampling import SamplingParams, draw_seed, seeded_unit, uniforms


class FakeEngine:
    """Records steps; 'logits' are just (slot, last token fed, length so far) per wanted row."""
    page_size = 64

    def __init__(self, max_seqs=4, tokens=4096, fail_at_step=None):
        self.max_seqs, self.tokens = max_seqs, tokens
        self.free = list(range(max_seqs - 1, -1, -1))
        self.length = {}
        self.steps = []
        self.acquired = []
        self.released = []
        self.fail_at_step = fail_at_step

    def free_tokens(self):
        return self.tokens

    def acquire(self):
        s = self.free.pop()
        self.length[s] = 0
        self.acquired.append(s)
        return s

    def release(self, slot):
        assert slot in self.length, "released twice"
        del self.length[slot]
        self.free.append(slot)
        self.released.append(slot)

    def step(self, entries):
        if self.fail_at_step is not None and len(self.steps) == self.fail_at_step:
            raise RuntimeError("injected")
        self.steps.append([(s, list(t), list(w)) for s, t, w in entries])
        rows = []
        for s, toks, want in entries:
            assert s in self.length
            self.length[s] += len(toks)
            rows.extend((s, toks[w], self.length[s]) for w in want)
        return rows


class ScriptSampler:
    """Next token = f(request, step): scripted per request."""

    def __init__(self, script):
        self.script = script
        self.calls = []

    def sample(self, logits, params, requests, step):
        self.calls.append((list(requests), step))

        class Out(list):
            def tolist(self):
                return list(self)
        return Out(self.script[r][step] for r in requests)


def test_plan_batches_respects_slots_and_tokens():
    assert plan_batches([10, 10, 10, 10, 10], 5, 10_000, 2, 64) == [[0, 1], [2, 3], [4]]
    assert plan_batches([10, 10, 10], 5, 10_000, 8, 64, max_batch=1) == [[0], [1], [2]]
    # 60 + 5 - 1 = 64 tokens -> one page; 61 + 5 - 1 -> two pages
    assert plan_batches([60, 61, 60], 5, 192, 8, 64) == [[0, 1], [2]]
    with pytest.raises(ValueError, match="request 1"):
        plan_batches([10, 500], 5, 256, 8, 64)


def test_unequal_prompts_stop_tokens_and_early_ends():
    eng = FakeEngine(max_seqs=4)
    script = {0: [5, 6, 99, 0, 0], 1: [99, 0, 0, 0, 0], 2: [7, 8, 9, 10, 11]}
    smp = ScriptSampler(script)
    seen = []
    res, met = generate(eng, smp, [[1, 2, 3], [4], [5, 6]], 4, SamplingParams(), stop_ids=[99],
                        on_token=lambda r, t: seen.append((r, t)) or True)
    assert [r.tokens for r in res] == [[5, 6, 99], [99], [7, 8, 9, 10]]
    assert [r.finish_reason for r in res] == ["stop", "stop", "length"]
    # one prefill step with all prompts and the last position wanted; then one token each
    assert eng.steps[0] == [(0, [1, 2, 3], [2]), (1, [4], [0]), (2, [5, 6], [1])]
    assert eng.steps[1] == [(0, [5], [0]), (2, [7], [0])]          # request 1 ended at its first token
    assert eng.steps[2] == [(0, [6], [0]), (2, [8], [0])]
    assert eng.steps[3] == [(2, [9], [0])]                         # the stop token 99 is never fed
    assert len(eng.steps) == 4                                     # the last token is returned, not fed
    assert sorted(eng.released) == [0, 1, 2] and not eng.length
    assert met.generated_tokens == 8 and met.batches == 1 and met.prompt_tokens == 6
    assert (0, 99) in seen and len(seen) == 8
    assert smp.calls[0] == ([0, 1, 2], 0) and smp.calls[1] == ([0, 2], 1)


def test_batches_follow_one_another_and_reuse_slots():
    eng = FakeEngine(max_seqs=2)
    script = {i: [i + 10] * 3 for i in range(5)}
    res, met = generate(eng, ScriptSampler(script), [[1]] * 5, 3, SamplingParams(), stop_ids=[])
    assert met.batches == 3 and all(r.tokens == [r.request + 10] * 3 for r in res)
    assert set(eng.acquired) == {0, 1} and len(eng.acquired) == 5
    assert not eng.length


def test_callback_false_ends_a_request():
    eng = FakeEngine()
    res, _ = generate(eng, ScriptSampler({0: [1, 2, 3, 4]}), [[9]], 4, SamplingParams(),
                      on_token=lambda r, t: t != 2)
    assert res[0].tokens == [1, 2] and res[0].finish_reason == "stop"


def test_max_new_tokens_one_needs_no_decode_step():
    eng = FakeEngine()
    res, _ = generate(eng, ScriptSampler({0: [1], 1: [2]}), [[9], [8, 7]], 1, SamplingParams())
    assert [r.tokens for r in res] == [[1], [2]] and len(eng.steps) == 1
    assert all(r.finish_reason == "length" for r in res)


def test_refusals_before_anything_runs():
    eng = FakeEngine()
    with pytest.raises(ValueError, match="greater than zero"):
        generate(eng, ScriptSampler({}), [[1]], 0)
    with pytest.raises(ValueError, match="empty prompt"):
        generate(eng, ScriptSampler({}), [[1], []], 2)
    with pytest.raises(ValueError, match="request 0 needs room"):
        generate(FakeEngine(tokens=64), ScriptSampler({}), [[1] * 100], 2)
    assert eng.steps == [] and eng.acquired == []


def test_failure_returns_every_slot():
    eng = FakeEngine(fail_at_step=2)
    with pytest.raises(RuntimeError, match="injected"):
        generate(eng, ScriptSampler({0: [1] * 9, 1: [2] * 9}), [[1], [2]], 8, SamplingParams())
    assert not eng.length and sorted(eng.free) == [0, 1, 2, 3]


def test_logits_are_returned_when_asked():
    class Row:
        def __init__(self, v):
            self.v = v

        def float(self):
            return self

        def cpu(self):
            return self.v

    class Eng(FakeEngine):
        def step(self, entries):
            return [Row(x) for x in super().step(entries)]

    res, _ = generate(Eng(), ScriptSampler({0: [4, 5]}), [[1, 2]], 2, SamplingParams(), return_logits=True)
    assert res[0].logits == [(0, 2, 2), (0, 4, 3)]


def test_draw_numbers_depend_on_request_and_step_only():
    p = SamplingParams(temperature=0.8, top_p=0.9, seed=17)
    alone = [uniforms(p, [3], s)[0] for s in range(4)]
    in_batch = [uniforms(p, [0, 3, 5], s)[1] for s in range(4)]
    assert alone == in_batch and len(set(alone)) == 4
    assert all(0.0 <= u < 1.0 for u in alone)
    assert seeded_unit(0) == seeded_unit(0x9E3779B97F4A7C15)
    assert draw_seed(1, 0, 0) != draw_seed(1, 1, 0) != draw_seed(1, 0, 1)


def test_sampling_params_are_checked():
    with pytest.raises(ValueError):
        SamplingParams(temperature=1.0, top_p=0.0)
    with pytest.raises(ValueError):
        SamplingParams(top_k=-1)
    assert SamplingParams().greedy and not SamplingParams(temperature=0.5).greedy


# ------------------------------------------------------------------ decoding one step ahead of the host
class DeviceFakeEngine(FakeEngine):
    """A scripted engine that also offers ``step_device``: the step's tokens come from a tensor, as on the GPU."""
    device = "cpu"

    def step_device(self, slots, token_source, rows):
        toks = [int(token_source[r]) for r in rows]
        self.steps.append([(s, [t], [0]) for s, t in zip(slots, toks)])
        for s in slots:
            assert s in self.length, "a released slot was stepped"
            self.length[s] += 1
        return [(s, t, self.length[s]) for s, t in zip(slots, toks)]


class TensorScriptSampler(ScriptSampler):
    def sample(self, logits, params, requests, step):
        import torch
        self.calls.append((list(requests), step))
        return torch.tensor([self.script[r][step] for r in requests], dtype=torch.int32)


def test_one_step_ahead_sees_a_stop_token_late_and_drops_the_extra_token():
    eng = DeviceFakeEngine(max_seqs=4)
    # request 0 stops at its third token (99), request 1 runs to the length limit, request 2 stops at once
    script = {0: [5, 6, 99, 41, 42, 43], 1: [7, 8, 9, 10, 11, 12], 2: [99, 1, 2, 3, 4, 5]}
    smp = TensorScriptSampler(script)
    results, metrics = generate(eng, smp, [[1, 2, 3], [4], [5, 6]], 5, SamplingParams(), stop_ids=[99])
    assert [r.tokens for r in results] == [[5, 6, 99], [7, 8, 9, 10, 11], [99]]
    assert [r.finish_reason for r in results] == ["stop", "length", "stop"]
    assert sorted(eng.released) == sorted(eng.acquired) and len(set(eng.released)) == 3 and not eng.length
    # the prompt step, then decode steps: request 0's stop shows one step late, so it is fed once more (its token 41
    # is never kept); the length limit is known when a step is queued, so request 1 runs no extra step
    fed = [[t[0] for _, t, _ in step] for step in eng.steps[1:]]
    assert fed == [[5, 7], [6, 8], [99, 9], [10]]
    assert metrics.generated_tokens == 3 + 5 + 1 and metrics.steps == 1 + 4
    # every draw was asked for with the request's own step number
    assert smp.calls[0] == ([0, 1, 2], 0) and smp.calls[1] == ([0, 1], 1) and smp.calls[-1] == ([1], 4)


def test_one_step_ahead_runs_batches_one_after_another_on_reused_slots():
    eng = DeviceFakeEngine(max_seqs=2)
    script = {r: [10 + r, 20 + r, 30 + r] for r in range(5)}
    results, metrics = generate(eng, TensorScriptSampler(script), [[1]] * 5, 3, SamplingParams(), stop_ids=[])
    assert [r.tokens for r in results] == [[10 + r, 20 + r, 30 + r] for r in range(5)]
    assert metrics.batches == 3 and len(eng.acquired) == 5 and sorted(eng.released) == sorted(eng.acquired)
    assert not eng.length
