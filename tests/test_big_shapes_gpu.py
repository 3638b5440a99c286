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
