"""A step is a transaction against faults that show only on the device.

The reference rolls every layer's cache back when a step fails (crates/spissa-runtime/src/models/llama/session/mod.rs:745-771)
and tests its loop with injected faults (crates/spissa-runtime/src/session.rs:495-663, session/tests_core.rs:647-661).
Here a kernel that gives up a bounded wait records a code in the device's status word; the engine confirms a step's new
lengths only when the word read zero behind the step's kernels. The faults below are made on the host (the word is
written, a forward pass raises) or by a kernel whose only wait is meant to run out after a few dozen microseconds and
then returns: nothing here faults, traps or hangs the GPU.
"""
import pytest
import torch

import tiny
from plain import llama_plain as P
from spissa_b200 import Engine, SamplingParams
from spissa_b200.csrc import lib as K
from spissa_b200.csrc.lib import KernelError
from spissa_b200.engine.engine import StepError
from spissa_b200.engine.session import ChatSession

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def model(tmp_path_factory):
    f = tmp_path_factory.mktemp("faults_A")
    tiny.make_folder(tiny.TINY_A, tiny.TINY_A_INIT, f, std=0.06)
    return (str(f),) + P.read_model_folder(f)


def books(engine):
    g = engine.cache.kv_groups
    return ({s: (q.length, {n: list(p) for n, p in q.pages.items()}) for s, q in engine.cache.seqs.items()},
            {n: grp.pages.free_count for n, grp in g.items()}, engine.cache.slots.free_count)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_forced_status_word_rolls_the_step_back_and_the_next_step_is_right(model, dtype):
    folder, pcfg, w = model
    toks = tiny.random_prompt(256, 70, 5)
    ref = P.model_logits(pcfg, w, toks, torch.float64)
    engine = Engine.from_folder(folder, dtype=dtype, max_tokens=64 * 4)
    slot = engine.acquire()
    engine.step([(slot, toks[:60], [])])
    before = books(engine)
    K.status_word(DEV).fill_(102)                               # as if a kernel had given up a wait
    with pytest.raises(KernelError, match="code 102"):
        engine.step([(slot, toks[60:66], [5])])                 # crosses into a second page
    assert books(engine) == before and engine.length(slot) == 60
    engine.cache.check()
    assert int(K.status_word(DEV).item()) == 0                  # the word is cleared: the engine goes on
    got = engine.step([(slot, toks[60:70], [0, 9])]).cpu()
    scale = float(ref.abs().max())
    assert float((got[0].double() - ref[60]).abs().max()) / scale <= tiny.TOL[dtype]
    assert float((got[1].double() - ref[69]).abs().max()) / scale <= tiny.TOL[dtype]
    engine.release(slot)
    engine.cache.check()


def test_a_wait_that_runs_out_is_reported_and_only_later_steps_are_undone(model):
    folder, pcfg, w = model
    toks = tiny.random_prompt(256, 40, 9)
    ref = P.model_logits(pcfg, w, toks, torch.float64)
    engine = Engine.from_folder(folder, dtype="float32", max_tokens=64 * 4)
    slot = engine.acquire()
    engine.step([(slot, toks[:30], [])], check=False)           # confirmed later: its status was copied before the fault
    waited = torch.zeros(1, dtype=torch.int64, device=DEV)
    K.wait_runs_out(DEV, 900, 40, waited)                       # nobody arrives on its barrier: it gives up after 40 us
    engine.step([(slot, toks[30:35], [])], check=False)         # launched after the fault: undone
    assert engine.length(slot) == 35                            # lengths count the steps in flight
    with pytest.raises(KernelError, match="code 900"):
        engine.step([(slot, toks[35:36], [0])], check=False)    # a later step may already see the fault as it begins
        engine.check()
    assert 40_000 <= int(waited.item()) < 10_000_000            # it waited its limit and no longer
    assert engine.length(slot) == 30
    engine.cache.check()
    got = engine.step([(slot, toks[30:40], [9])]).cpu()
    assert float((got[0].double() - ref[39]).abs().max()) / float(ref.abs().max()) <= tiny.TOL["float32"]
    engine.check()


def test_a_forward_pass_that_raises_gives_the_pages_back(model, monkeypatch):
    folder, _, _ = model
    engine = Engine.from_folder(folder, dtype="float32", max_tokens=64 * 4)
    slot = engine.acquire()
    engine.step([(slot, [1, 2, 3], [])])
    before = books(engine)

    def boom(*args, **kwargs):
        raise KernelError("injected")
    monkeypatch.setattr(engine.model, "forward", boom)
    with pytest.raises(KernelError, match="injected"):
        engine.step([(slot, list(range(100)), [])])             # had reserved a second page
    assert books(engine) == before
    engine.cache.check()


def test_a_chat_turn_raises_when_the_status_word_is_set(model):
    folder, _, _ = model
    engine = Engine.from_folder(folder, dtype="float32", max_tokens=64 * 4)
    chat = ChatSession(engine, SamplingParams())
    first = chat.generate_turn([5, 6, 7], 3)
    length = engine.length(chat.slot)
    K.status_word(DEV).fill_(203)
    with pytest.raises(KernelError, match="code 203"):
        chat.generate_turn([8, 9], 3)
    assert engine.length(chat.slot) == length
    again = chat.generate_turn([8, 9], 3)                       # the same turn goes through afterwards
    assert len(first.tokens) == 3 and len(again.tokens) == 3
    chat.close()
    engine.cache.check()


def test_generation_returns_every_slot_after_a_fault_and_goes_on(model):
    folder, pcfg, w = model
    engine = Engine.from_folder(folder, dtype="float32", max_tokens=64 * 6)
    prompts = [tiny.random_prompt(256, n, n) for n in (5, 20)]
    want = [P.generate_greedy(pcfg, w, p, 6) for p in prompts]
    K.status_word(DEV).fill_(101)
    with pytest.raises(KernelError):
        engine.generate(prompts, 6, SamplingParams(), stop_ids=[])
    assert engine.cache.slots.held_count == 0 and engine.free_tokens() == 64 * 6
    engine.cache.check()
    results, _ = engine.generate(prompts, 6, SamplingParams(), stop_ids=[])
    assert [r.tokens for r in results] == want


def test_a_token_from_the_device_outside_the_vocabulary_is_a_fault_not_a_wrong_row(model):
    folder, _, _ = model
    engine = Engine.from_folder(folder, dtype="float32", max_tokens=64 * 4)
    slot = engine.acquire()
    engine.step([(slot, [1, 2, 3], [])])
    source = torch.tensor([100000], dtype=torch.int32, device=DEV)
    engine.step_device([slot], source, [0])
    with pytest.raises(KernelError, match="code 301"):
        engine.check()
    assert engine.length(slot) == 3
    engine.step([(slot, [4], [0])])
    engine.cache.check()


def test_positions_beyond_the_model_are_refused_before_anything_runs(model):
    folder, _, _ = model
    engine = Engine.from_folder(folder, dtype="float32", max_tokens=64 * 4)          # the model has 128 positions
    slot = engine.acquire()
    engine.step([(slot, list(range(120)), [])])
    with pytest.raises(StepError, match="128 positions"):
        engine.step([(slot, list(range(9)), [])])
    assert engine.length(slot) == 120
    engine.step([(slot, list(range(8)), [7])])
    with pytest.raises(StepError, match="128 positions"):
        engine.step_device([slot], torch.zeros(1, dtype=torch.int32, device=DEV), [0])
    with pytest.raises(ValueError, match="128 positions"):
        engine.generate([[1] * 100], 30, SamplingParams(), stop_ids=[])
    chat = ChatSession(engine, SamplingParams(), max_seq_len=4096)
    assert chat.max_seq_len <= 128
    chat.close()


def test_the_header_follows_generation(model):
    """position, draws and last token of every slot, written by the sampler on the device."""
    folder, pcfg, w = model
    engine = Engine.from_folder(folder, dtype="float32", max_tokens=64 * 6, max_seqs=3)
    prompts = [tiny.random_prompt(256, n, n) for n in (9, 4)]
    seen = {}
    release = engine.release

    def spy(slot):                                              # read a slot's header as it is handed back
        seen[slot] = (engine.cache.header[slot].tolist(), engine.cache.draws(slot))
        release(slot)
    engine.release = spy
    results, _ = engine.generate(prompts, 5, SamplingParams(), stop_ids=[])
    engine.release = release
    assert [r.tokens for r in results] == [P.generate_greedy(pcfg, w, p, 5) for p in prompts]
    assert len(seen) == 2
    for (slot, (row, draws)), p, r in zip(sorted(seen.items()), prompts, results):
        # the last token is returned but never fed: the sequence holds the prompt and four of the five tokens
        assert row[:3] == [len(p) + 4, 5, r.tokens[-1]] and draws == 5
    s = engine.acquire()
    assert engine.cache.header[s].tolist() == [0, 0, -1, 0]     # a slot starts with a fresh header
    engine.release(s)
