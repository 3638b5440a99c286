"""The one-kernel decode path against the plain implementation and against the same engine run part by part.

Configurations E (head 64) and F (head 128) are built so that every layer qualifies; the tests check that the
kernel really ran (its run counter), that 16 sequences use the two-token-block form and 17 fall back, that
sequences of very different lengths, page crossings and a far key come out right, and that what cannot be
fused (32-bit, a head size the kernel is not built for) quietly runs part by part.
"""
import pytest
import torch

import tiny
from plain import llama_plain as P
from spissa_b200 import Engine

pytestmark = pytest.mark.gpu

TOL = tiny.TOL["bfloat16"]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name in ("A", "E", "F"):
        cfg, init = tiny.TINIES[name]
        f = tmp_path_factory.mktemp(f"fused_{name}")
        tiny.make_folder(cfg, init, f)                     # the weights' usual width: the bfloat16 budget is set for it
        out[name] = (str(f),) + P.read_model_folder(f)
    return out


def decode_rows(engine, seqs, prompt_lens, n_steps):
    """Prompts in one step, then one token each per step; returns the logits rows of the decode steps."""
    slots = [engine.acquire() for _ in seqs]
    engine.step([(s, q[:n], []) for s, q, n in zip(slots, seqs, prompt_lens)])
    rows = []
    for i in range(n_steps):
        rows.append(engine.step([(s, [q[n + i]], [0]) for s, q, n in zip(slots, seqs, prompt_lens)]).float().cpu())
    for s in slots:
        engine.release(s)
    engine.cache.check()
    return torch.stack(rows)                    # [steps, sequences, vocab]


@pytest.mark.parametrize("name", ["E", "F"])
def test_kernel_runs_and_agrees_with_plain_and_with_the_parts(folders, name):
    folder, pcfg, w = folders[name]
    V = pcfg["vocab_size"]
    lens = [130, 1, 63]                                    # a page boundary is crossed while decoding
    steps = 70
    seqs = [tiny.random_prompt(V, n + steps, 31 * n + 1) for n in lens]
    got = {}
    for fuse in (True, False):
        engine = Engine.from_folder(folder, dtype="bfloat16", max_tokens=64 * 16, use_graphs=False, fuse_decode=fuse)
        got[fuse] = decode_rows(engine, seqs, lens, steps)
        fused = engine.model._fused
        if fuse:
            assert fused is not None and fused.runs == steps, "the decode steps did not go through the kernel"
        else:
            assert not fused
    # both ways are within the bfloat16 budget of the plain implementation, at every step (so at most two budgets apart)
    for b, (q, n) in enumerate(zip(seqs, lens)):
        ref = P.model_logits(pcfg, w, q, torch.float64)
        scale = float(ref.abs().max())
        for fuse in (True, False):
            err = float((got[fuse][:, b].double() - ref[n:n + steps]).abs().max()) / scale
            assert err <= TOL, f"{name}: sequence {b}, {'one kernel' if fuse else 'part by part'}: {err:.3e}"


@pytest.mark.parametrize("name,vocab", [("E", 784), ("F", 528), ("E", 16)])
def test_the_kernel_takes_the_final_norm_and_the_head(tmp_path, name, vocab):
    """With a vocabulary that is a multiple of 16 the final norm and the head are the kernel's last product: the logits
    agree with the plain implementation and with the same kernel followed by the norm and head kernels; the greedy
    tokens are the argmax of those logits (the lowest index among equal values), also noted in the headers."""
    cfg, init = tiny.TINIES[name]
    cfg = dict(cfg, vocab_size=vocab)
    tiny.make_folder(cfg, init, tmp_path)
    pcfg, w = P.read_model_folder(tmp_path)
    lens = [70, 1, 63, 5, 33]
    steps = 6
    seqs = [tiny.random_prompt(vocab, n + steps, 13 * n + 1) for n in lens]
    got = {}
    for with_head in (True, False):
        engine = Engine.from_folder(str(tmp_path), dtype="bfloat16", max_tokens=64 * 16, use_graphs=False)
        engine.step([(engine.acquire(), [1, 2], [])])                      # plans the runners
        engine.model._fused.with_head = with_head
        got[with_head] = decode_rows(engine, seqs, lens, steps)
        fused = engine.model._fused
        assert fused.head is not None and fused.head_runs == (steps if with_head else 0)
    for b, (q, n) in enumerate(zip(seqs, lens)):
        ref = P.model_logits(pcfg, w, q, torch.float64)
        scale = float(ref.abs().max())
        for with_head in (True, False):
            err = float((got[with_head][:, b].double() - ref[n:n + steps]).abs().max()) / scale
            assert err <= TOL, f"{name}: sequence {b}, head in the kernel {with_head}: {err:.3e}"
    # greedy: the tokens without logits, teacher-forced along the same sequences
    engine = Engine.from_folder(str(tmp_path), dtype="bfloat16", max_tokens=64 * 16, use_graphs=False)
    slots = [engine.acquire() for _ in seqs]
    engine.step([(s, q[:n], []) for s, q, n in zip(slots, seqs, lens)])
    for i in range(steps):
        toks = engine.step([(s, [q[n + i]], [0]) for s, q, n in zip(slots, seqs, lens)], greedy=True).cpu()
        want = got[True][i].argmax(dim=1).int()
        assert torch.equal(toks, want), (i, toks.tolist(), want.tolist())
        header = engine.cache.header.cpu()
        for b, s in enumerate(slots):
            assert int(header[s, 2]) == int(toks[b])
    assert engine.model._fused.head_runs == steps


def test_sixteen_sequences_in_one_step_and_seventeen_part_by_part(folders):
    folder, pcfg, w = folders["E"]
    V = pcfg["vocab_size"]
    for B, expect_runs in ((16, 5), (17, 0), (9, 5)):
        lens = [3 + 11 * b for b in range(B)]
        seqs = [tiny.random_prompt(V, n + 5, 7 * n + B) for n in lens]
        engine = Engine.from_folder(folder, dtype="bfloat16", max_tokens=64 * 4 * B, max_seqs=B, use_graphs=False)
        rows = decode_rows(engine, seqs, lens, 5)
        assert engine.model._fused.runs == expect_runs
        for b in (0, B // 2, B - 1):
            ref = P.model_logits(pcfg, w, seqs[b], torch.float64)
            err = float((rows[4, b].double() - ref[lens[b] + 4]).abs().max()) / float(ref.abs().max())
            assert err <= TOL, f"{B} sequences, sequence {b}: {err:.3e}"


def test_a_token_does_not_depend_on_its_company(folders):
    """The same sequence decoded alone and among others gives the same logits bit for bit: every sum in the
    kernel has an order that depends on neither timing nor the other tokens."""
    folder, pcfg, w = folders["E"]
    V = pcfg["vocab_size"]
    lens = [40, 100, 7, 64, 129]
    seqs = [tiny.random_prompt(V, n + 6, n) for n in lens]
    engine = Engine.from_folder(folder, dtype="bfloat16", max_tokens=64 * 24, use_graphs=False)
    together = decode_rows(engine, seqs, lens, 6)
    again = decode_rows(engine, seqs, lens, 6)                                  # other slots and pages
    assert torch.equal(together, again)
    alone = decode_rows(engine, seqs[1:2], lens[1:2], 6)
    scale = float(together.abs().max())
    # the prompt ran in other company (another tile shape may round differently), the decode steps must agree closely
    assert float((alone[:, 0] - together[:, 1]).abs().max()) <= TOL * scale


def test_what_cannot_be_fused_runs_part_by_part(folders):
    folder, pcfg, w = folders["E"]
    e32 = Engine.from_folder(folder, dtype="float32", max_tokens=256, use_graphs=False)
    s = e32.acquire()
    e32.step([(s, [1, 2, 3], [])])
    e32.step([(s, [4], [0])])
    assert e32.model._fused is None                                              # 32-bit: planned and refused
    folder_a = folders["A"][0]
    ea = Engine.from_folder(folder_a, dtype="bfloat16", max_tokens=256, use_graphs=False)
    s = ea.acquire()
    ea.step([(s, [1, 2, 3], [])])
    ea.step([(s, [4], [0])])
    assert ea.model._fused is None                                               # head size 16: the kernel is not built for it


def test_long_context_far_key(folders, tmp_path):
    """One key far back, made to stand out by scaling the query and key projections: the chunked attention inside
    the kernel has to find it in whichever chunk it lies."""
    cfg, init = tiny.TINIES["E"]
    folder = tmp_path / "peaky_e"
    tiny.make_folder(cfg, init, folder, std=0.05)
    pcfg, w = P.read_model_folder(folder)
    from spissa_b200.weights import write_safetensors
    for k in list(w):
        if "q_proj" in k or "k_proj" in k:
            w[k] = (w[k].float() * 4).bfloat16()
    write_safetensors(folder / "model.safetensors", w)
    V = cfg["vocab_size"]
    lens = [900, 515]
    steps = 8
    seqs = [tiny.random_prompt(V, n + steps, n) for n in lens]
    engine = Engine.from_folder(str(folder), dtype="bfloat16", max_tokens=64 * 32, use_graphs=False)
    rows = decode_rows(engine, seqs, lens, steps)
    assert engine.model._fused.runs == steps
    for b, (q, n) in enumerate(zip(seqs, lens)):
        ref = P.model_logits(pcfg, w, q, torch.float64)
        noise = float((P.model_logits(pcfg, w, q, torch.float32).double() - ref).abs().max()) / float(ref.abs().max())
        allowed = TOL * max(1.0, noise / 5e-7)
        for i in range(steps):
            err = float((rows[i, b].double() - ref[n + i]).abs().max()) / float(ref.abs().max())
            assert err <= allowed, f"sequence {b} step {i}: {err:.3e} (allowed {allowed:.3e})"


def test_one_captured_step_serves_growing_lengths(folders):
    """With CUDA graphs the kernel reads its split of the keys from the device, so one graph per batch size and
    power-of-two length is replayed while the sequences grow page by page and the split changes under it."""
    folder, pcfg, w = folders["E"]
    V = pcfg["vocab_size"]
    lens = [262, 40]
    steps = 200                                                      # 262 -> 462 tokens: 5 to 8 pages, one wide bucket
    seqs = [tiny.random_prompt(V, n + steps, 3 * n + 1) for n in lens]
    engine = Engine.from_folder(folder, dtype="bfloat16", max_tokens=64 * 16, use_graphs=True)
    rows = decode_rows(engine, seqs, lens, steps)
    fused = engine.model._fused
    assert fused is not None and fused.runs >= 1
    assert len({split for (n, pages), split in fused._splits.items() if n == 2}) >= 3, "the split never changed"
    wide = [k for k in engine._graphs if k[2]]
    assert len(wide) == 1 and len(engine._graphs) == 1, f"graphs captured: {list(engine._graphs)}"
    for b, (q, n) in enumerate(zip(seqs, lens)):
        ref = P.model_logits(pcfg, w, q, torch.float64)
        scale = float(ref.abs().max())
        err = float((rows[:, b].double() - ref[n:n + steps]).abs().max()) / scale
        assert err <= TOL, f"sequence {b}: {err:.3e}"


@pytest.mark.parametrize("heads, kv_heads", [(10, 1), (16, 2), (5, 5)])
def test_head_groups_of_other_sizes(tmp_path, heads, kv_heads):
    """The kernel's attention holds the query heads of a kv head as columns of 8: ten heads per kv head need a
    second, partly empty column tile, eight fill one exactly, one head per kv head leaves seven of eight idle."""
    cfg = dict(tiny.TINY_E, num_attention_heads=heads, num_key_value_heads=kv_heads, num_hidden_layers=2)
    folder = tiny.make_folder(cfg, tiny.TINY_E_INIT, tmp_path / "groups")
    pcfg, w = P.read_model_folder(folder)
    V = cfg["vocab_size"]
    lens = [125, 40, 200]
    steps = 6
    seqs = [tiny.random_prompt(V, n + steps, 5 * n + heads) for n in lens]
    engine = Engine.from_folder(str(folder), dtype="bfloat16", max_tokens=64 * 16, use_graphs=False)
    rows = decode_rows(engine, seqs, lens, steps)
    assert engine.model._fused.runs == steps
    for b, (q, n) in enumerate(zip(seqs, lens)):
        ref = P.model_logits(pcfg, w, q, torch.float64)
        err = float((rows[:, b].double() - ref[n:n + steps]).abs().max()) / float(ref.abs().max())
        assert err <= TOL, f"{heads} heads, {kv_heads} kv heads, sequence {b}: {err:.3e}"


def test_real_layer_sizes_repeat_bit_for_bit():
    """Two layers of the 1B shape, eight sequences of a few hundred tokens, sixty decode steps, twice: every kernel
    on the way (tensor-core products and attention for the prompts, the one-kernel decode path, the head) has fixed
    orders of summation, so the two runs agree bit for bit whatever the timing of their CTAs and warps."""
    from spissa_b200 import LlamaConfig
    from test_big_shapes_gpu import LLAMA_1B_2L
    cfg = LlamaConfig.from_dict(LLAMA_1B_2L)
    engine = Engine.from_config(cfg, seed=5, dtype="bfloat16", max_tokens=8 * 1024, max_seqs=8, use_graphs=False)
    V = cfg.vocab_size
    lens = [300 + 37 * b for b in range(8)]
    seqs = [tiny.random_prompt(V, n + 60, 3 * n) for n in lens]
    first = decode_rows(engine, seqs, lens, 60)
    assert engine.model._fused.runs == 60
    again = decode_rows(engine, seqs, lens, 60)
    assert torch.isfinite(first).all()
    assert torch.equal(first, again)
