"""The real layer sizes, with few layers: the kernels that only large shapes reach (256-wide tensor-core
tiles, the streaming head over a 128k vocabulary, flash attention with 32 heads, K split over clusters)
inside the whole engine, against the plain implementation."""
import pytest
import torch

import tiny
import traces
from plain import llama_plain as P

pytestmark = pytest.mark.gpu

LLAMA_1B_2L = dict(
    architectures=["LlamaForCausalLM"], model_type="llama", num_hidden_layers=2, hidden_size=2048,
    num_attention_heads=32, num_key_value_heads=8, head_dim=64, intermediate_size=8192, vocab_size=128256,
    rope_theta=500000.0,
    rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                      original_max_position_embeddings=8192),
    tie_word_embeddings=True, rms_norm_eps=1e-5, max_position_embeddings=131072)

# the 8B layer (head size 128, K = 14336) with a smaller vocabulary and an untied head
LLAMA_8B_1L = dict(
    architectures=["LlamaForCausalLM"], model_type="llama", num_hidden_layers=1, hidden_size=4096,
    num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=14336, vocab_size=20000,
    rope_theta=500000.0,
    rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                      original_max_position_embeddings=8192),
    tie_word_embeddings=False, rms_norm_eps=1e-5, max_position_embeddings=131072)


# the 3B layer (width 3072, 24 heads of 128)
LLAMA_3B_1L = dict(LLAMA_8B_1L, hidden_size=3072, num_attention_heads=24, intermediate_size=8192, vocab_size=20000)


@pytest.mark.parametrize("name,cfg", [("1b", LLAMA_1B_2L), ("8b", LLAMA_8B_1L)])
def test_real_layer_sizes_against_plain(tmp_path, name, cfg):
    folder = tmp_path / name
    tiny.make_folder(cfg, dict(seed=3, norm_std=0.05), folder)
    pcfg, w = P.read_model_folder(folder)
    V = cfg["vocab_size"]
    # 300 tokens in one step (tensor-core tiles, flash prefill), 20 in one (split K), then one by one (decode kernels)
    reqs = {"long": tiny.random_prompt(V, 300, 1), "mid": tiny.random_prompt(V, 40, 2)}
    want_pos = {"long": [0, 127, 128, 255, 299], "mid": [0, 19, 39]}
    ref = {}
    for rid, toks in reqs.items():
        logits = P.model_logits(pcfg, w, toks, torch.float32)
        for p in range(len(toks)):
            ref[(rid, p)] = logits[p].double()
    scale = max(float(v.abs().max()) for v in ref.values())
    steps = [
        dict(step=0, entries=[dict(id="long", tokens=reqs["long"][:296], want=[0, 127, 128, 255]),
                              dict(id="mid", tokens=reqs["mid"][:20], want=[0, 19])], end=[]),
        dict(step=1, entries=[dict(id="mid", tokens=reqs["mid"][20:36], want=[15])], end=[]),
    ]
    for i in range(4):
        steps.append(dict(step=2 + i, entries=[dict(id="long", tokens=[reqs["long"][296 + i]], want=[0]),
                                               dict(id="mid", tokens=[reqs["mid"][36 + i]], want=[0])],
                          end=["long", "mid"] if i == 3 else []))
    for dtype in ("bfloat16", "float32"):
        out = tmp_path / f"{name}_{dtype}"
        traces.run_in_process(str(folder), dtype, steps, str(out))
        got = traces.collect(steps, str(out), V)
        # the plain run is float32 itself here (float64 would take minutes at these sizes): allow its own noise
        tol = tiny.TOL[dtype] if dtype == "bfloat16" else 2e-5
        worst = max(float((row.double() - ref[key]).abs().max()) for key, row in got.items()) / scale
        assert len(got) == 4 + 2 + 1 + 8 and worst <= tol, f"{name}/{dtype}: {worst:.3e} of the largest logit"


def _engine_and_plain_weights(cfg_dict, seed, dtype, max_tokens, max_seqs, **engine_options):
    """An engine on random weights drawn on the device, and the same tensors for the plain implementation."""
    from spissa_b200 import Engine
    from spissa_b200.config import config_from_dict
    from spissa_b200.engine.model import Model
    from spissa_b200.weights import random_tensors
    cfg = config_from_dict(cfg_dict)
    tensors = random_tensors(Model(cfg.to_spec()).weight_specs(), seed, 0.02, 0.05, torch.bfloat16, device="cuda:0")
    plain_w = {k: v.cpu() for k, v in tensors.items()}
    if dtype == "float32":
        tensors = {k: v.float() for k, v in tensors.items()}
    return Engine(cfg, tensors, dtype, max_tokens, max_seqs, **engine_options), plain_w


def test_the_whole_1b_model_on_a_short_prompt():
    """All 16 layers of the Llama-3.2-1B shape: a 40-token prompt in one step and four tokens one by one, in
    bfloat16 (split-K products, then the one-kernel decode path and the greedy head) against the plain float32 run."""
    cfg = {**LLAMA_1B_2L, "num_hidden_layers": 16}
    engine, w = _engine_and_plain_weights(cfg, 9, "bfloat16", 64 * 4, 2)
    toks = tiny.random_prompt(cfg["vocab_size"], 44, 77)
    ref = P.model_logits(cfg, w, toks, torch.float32).double()
    scale = float(ref.abs().max())
    slot = engine.acquire()
    got = [engine.step([(slot, toks[:40], [0, 39])]).cpu()]
    for i in range(40, 44):
        got.append(engine.step([(slot, [toks[i]], [0])]).cpu())
    got = torch.cat(got).double()
    want = ref[[0, 39, 40, 41, 42, 43]]
    worst = float((got - want).abs().max()) / scale
    # bfloat16 rounds the activations between the kernels of every layer; the layers' rounding errors add up like
    # independent errors, so the distance from the plain run grows with the square root of the depth (measured at these
    # sizes: 7e-3 at 2 layers, 8e-3 at 4, 1.2e-2 at 8, 1.5e-2 at 16, the same part by part and through the one-kernel
    # decode path; float32 stays at 7e-6). The tolerance of the tiny models holds for up to 3 layers.
    allowed = tiny.TOL["bfloat16"] * (16 / 3) ** 0.5
    assert worst <= allowed, f"worst error {worst:.3e} of the largest logit (allowed {allowed:.2e})"
    assert engine.model._fused is not None and engine.model._fused.runs >= 1        # later steps replay a captured launch
    # the greedy head on the same state: the token it returns is a maximum of the plain logits up to that tolerance
    other = engine.acquire()
    tok = int(engine.step([(other, toks[:40], [39])], greedy=True).tolist()[0])
    assert float(ref[39].max() - ref[39][tok]) <= allowed * scale


@pytest.mark.parametrize("n_seqs,base", [(33, "1b"), (64, "1b"), (9, "8b"), (3, "3b")])
def test_decode_batches_beyond_the_one_kernel_path_at_real_layer_sizes(n_seqs, base):
    """33 and 64 sequences decode with five launches a layer: the tensor-core weight-streaming products with the
    norms, the rotation and the cache write in their epilogues, the split-key attention, and a CUDA graph per length
    bucket, at the 1B layer sizes (two layers, a smaller vocabulary) against the plain run; the same steps launched
    directly, without graphs, give the same bits. With large layers (the 8B and 3B widths) smaller batches take this way
    too, because it is the faster one there (``engine/fused_decode.py: five_launch_from``)."""
    cfg = {"1b": {**LLAMA_1B_2L, "vocab_size": 20000}, "8b": LLAMA_8B_1L, "3b": LLAMA_3B_1L}[base]
    engine, w = _engine_and_plain_weights(cfg, 4, "bfloat16", 64 * n_seqs, n_seqs)
    V = cfg["vocab_size"]
    lens = [1 + (7 * i) % 23 for i in range(n_seqs)]
    seqs = [tiny.random_prompt(V, n + 3, 31 * i + n) for i, n in enumerate(lens)]
    refs = [P.model_logits(cfg, w, s, torch.float32).double() for s in seqs]
    scale = max(float(r.abs().max()) for r in refs)
    slots = [engine.acquire() for _ in seqs]
    engine.step([(sl, s[:n], []) for sl, s, n in zip(slots, seqs, lens)])
    worst = 0.0
    kept = []
    for i in range(3):                                          # the third step of a kind is replayed from its graph
        rows = engine.step([(sl, [s[n + i]], [0]) for sl, s, n in zip(slots, seqs, lens)]).cpu()
        kept.append(rows)
        rows = rows.double()
        for b, (r, n) in enumerate(zip(refs, lens)):
            worst = max(worst, float((rows[b] - r[n + i]).abs().max()) / scale)
    assert worst <= tiny.TOL["bfloat16"], f"worst error {worst:.3e} of the largest logit"
    assert len(engine._graphs) >= 1 and not any(k[2] for k in engine._graphs)      # captured, and not the one-kernel path
    assert engine.model._fused_prefill.runs >= 2                 # the five-launch sequence took the decode steps (run once, captured once, then replayed)
    direct, _ = _engine_and_plain_weights(cfg, 4, "bfloat16", 64 * n_seqs, n_seqs, use_graphs=False)
    slots = [direct.acquire() for _ in seqs]
    direct.step([(sl, s[:n], []) for sl, s, n in zip(slots, seqs, lens)])
    for i in range(3):
        rows = direct.step([(sl, [s[n + i]], [0]) for sl, s, n in zip(slots, seqs, lens)]).cpu()
        assert torch.equal(rows, kept[i]), f"step {i}: launched directly and replayed from a graph differ"
    del direct
    # greedy over the same step: the tensor-core head keeps candidates per tile
    engine2, _ = _engine_and_plain_weights(cfg, 4, "bfloat16", 64 * n_seqs, n_seqs)
    slots = [engine2.acquire() for _ in seqs]
    engine2.step([(sl, s[:n], []) for sl, s, n in zip(slots, seqs, lens)])
    toks = engine2.step([(sl, [s[n]], [0]) for sl, s, n in zip(slots, seqs, lens)], greedy=True).tolist()
    for b, (r, n) in enumerate(zip(refs, lens)):
        assert float(r[n].max() - r[n][toks[b]]) <= tiny.TOL["bfloat16"] * scale
