"""Layers with different cache needs in one model: a toy architecture, defined HERE, whose odd layers
attend through a sliding window while its even layers see every key.

The windowed layers get a cache group of their own whose pages are returned once no later query can
see them; the test runs prompts longer than the window whole, cut into steps and decoded one by one,
and compares with the plain implementation's windowed attention.
"""
import pytest
import torch

import tiny
from plain import llama_plain as P
from spissa_b200 import Engine
from spissa_b200.config import (LayerSpec, ModelSpec, config_from_dict, register_architecture,
                                unregister_architecture)
from spissa_b200.weights import write_random_model

pytestmark = pytest.mark.gpu
WINDOW = 70
BASE = dict(tiny.TINY_B, num_hidden_layers=4, num_key_value_heads=3, head_dim=64, hidden_size=128,
            intermediate_size=192, vocab_size=300)


class ToyWindowConfig:
    def __init__(self, d):
        self.d = d
        self.base = config_from_dict({**BASE, "architectures": ["LlamaForCausalLM"]})

    @classmethod
    def from_dict(cls, d):
        return cls(d)

    def to_dict(self):
        return dict(self.d)

    def to_spec(self):
        llama = self.base.to_spec()
        layers = []
        for i, layer in enumerate(llama.layers):
            if i % 2 == 1:
                layer = LayerSpec(layer.block, layer.mixer.with_params(window=WINDOW), layer.ffn, layer.norms)
            layers.append(layer)
        return ModelSpec(**{**llama.__dict__, "architecture": "ToyWindowForCausalLM", "layers": tuple(layers)})


@pytest.fixture()
def toy():
    register_architecture("ToyWindowForCausalLM", ToyWindowConfig)
    yield
    unregister_architecture("ToyWindowForCausalLM")


def plain_logits(w, ids):
    n = P.config_numbers(BASE)
    w = {k: v.double() for k, v in w.items()}
    inv = P.rope_inv_freq(n["theta"], n["hd"], n["scaling"])
    h = P.embedding(w["model.embed_tokens.weight"], ids)
    for i in range(n["L"]):
        p = f"model.layers.{i}."
        a = P.rms_norm(h, w[p + "input_layernorm.weight"], n["eps"])
        r = h + P.attention_block(a, w, p + "self_attn.", n, inv, window=WINDOW if i % 2 else None)
        m = P.rms_norm(r, w[p + "post_attention_layernorm.weight"], n["eps"])
        h = r + P.swiglu(m, w, p + "mlp.")
    h = P.rms_norm(h, w["model.norm.weight"], n["eps"])
    return P.linear(h, w["lm_head.weight"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_windowed_and_full_layers_share_a_model(toy, tmp_path, dtype):
    cfg = config_from_dict(dict(architectures=["ToyWindowForCausalLM"]))
    write_random_model(cfg, tmp_path, seed=9, std=0.05, norm_std=0.1)
    _, w = P.read_model_folder(tmp_path)
    engine = Engine.from_folder(tmp_path, dtype=dtype, max_tokens=64 * 9, max_seqs=2)
    assert sorted(g.request.window or 0 for g in engine.cache.kv_groups.values()) == [0, WINDOW]
    win_group = next(g for g in engine.cache.kv_groups.values() if g.request.window)
    full_group = next(g for g in engine.cache.kv_groups.values() if not g.request.window)
    reqs = [tiny.random_prompt(300, n, n) for n in (260, 90)]
    refs = [plain_logits(w, r) for r in reqs]
    scale = max(float(r.abs().max()) for r in refs)
    tol = tiny.TOL[dtype]

    # whole prompts in one ragged step
    slots = [engine.acquire() for _ in reqs]
    got = engine.step([(s, r, list(range(len(r)))) for s, r in zip(slots, reqs)]).cpu()
    assert float((got.double() - torch.cat(refs)).abs().max()) / scale <= tol
    # the windowed group has handed back what lies before the window, the full group nothing
    assert win_group.pages.held_count < full_group.pages.held_count
    engine.cache.check()
    for s in slots:
        engine.release(s)

    # a slice of the prompt, then the rest in another step, then tokens one by one (graphs included)
    slots = [engine.acquire() for _ in reqs]
    cuts = [(0, 100), (100, 200)]
    for lo, hi in cuts:
        ents = [(s, r[lo:min(hi, len(r) - 40)], []) for s, r in zip(slots, reqs) if lo < len(r) - 40]
        if ents:
            engine.step(ents)
    fed = [engine.length(s) for s in slots]
    for i in range(40):
        ents = [(s, [r[f + i]], [0]) for s, r, f in zip(slots, reqs, fed) if f + i < len(r)]
        rows = engine.step(ents).cpu()
        k = 0
        for b, (r, f) in enumerate(zip(reqs, fed)):
            if f + i < len(r):
                err = float((rows[k].double() - refs[b][f + i]).abs().max()) / scale
                assert err <= tol, f"request {b} position {f + i}: {err:.3e}"
                k += 1
    engine.cache.check()
    for s in slots:
        engine.release(s)
    assert all(g.pages.free_count == g.n_pages for g in engine.cache.kv_groups.values())


# ------------------------------------------------------------------ a layer that reads another layer's cache
class ToySharedKVConfig(ToyWindowConfig):
    """Two layers; the second has no k/v projections and attends over the keys the first one stored."""

    def to_spec(self):
        from spissa_b200.config import ScheduleEntry
        llama = config_from_dict({**BASE, "num_hidden_layers": 2, "architectures": ["LlamaForCausalLM"]}).to_spec()
        second = llama.layers[1]
        second = LayerSpec(second.block, second.mixer.with_params(shares_kv=True), second.ffn, second.norms)
        return ModelSpec(**{**llama.__dict__, "architecture": "ToySharedKVForCausalLM",
                            "layers": (llama.layers[0], second),
                            "schedule": (ScheduleEntry(0, 0, True), ScheduleEntry(1, 0, False))})


def plain_shared_logits(w, ids):
    n = P.config_numbers(BASE)
    w = {k: v.double() for k, v in w.items()}
    inv = P.rope_inv_freq(n["theta"], n["hd"], n["scaling"])
    T = len(ids)
    pos = torch.arange(T)
    h = P.embedding(w["model.embed_tokens.weight"], ids)
    # layer 0 as usual, but keep its rotated keys and its values
    p = "model.layers.0."
    a = P.rms_norm(h, w[p + "input_layernorm.weight"], n["eps"])
    k0 = P.apply_rope(P.linear(a, w[p + "self_attn.k_proj.weight"]).reshape(T, n["nkv"], n["hd"]), pos, inv)
    v0 = P.linear(a, w[p + "self_attn.v_proj.weight"]).reshape(T, n["nkv"], n["hd"])
    h = P.decoder_layer(h, w, 0, n, inv)
    # layer 1: its own queries over layer 0's keys and values
    p = "model.layers.1."
    a = P.rms_norm(h, w[p + "input_layernorm.weight"], n["eps"])
    q = P.apply_rope(P.linear(a, w[p + "self_attn.q_proj.weight"]).reshape(T, n["nh"], n["hd"]), pos, inv)
    r = h + P.linear(P.causal_attention(q, k0, v0), w[p + "self_attn.o_proj.weight"])
    m = P.rms_norm(r, w[p + "post_attention_layernorm.weight"], n["eps"])
    h = r + P.swiglu(m, w, p + "mlp.")
    h = P.rms_norm(h, w["model.norm.weight"], n["eps"])
    return P.linear(h, w["lm_head.weight"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_layer_reads_another_layers_cache(tmp_path, dtype):
    register_architecture("ToySharedKVForCausalLM", ToySharedKVConfig)
    try:
        cfg = config_from_dict(dict(architectures=["ToySharedKVForCausalLM"]))
        write_random_model(cfg, tmp_path, seed=4, std=0.05)
        _, w = P.read_model_folder(tmp_path)
        assert "model.layers.1.self_attn.k_proj.weight" not in w and "model.layers.1.self_attn.q_proj.weight" in w
        engine = Engine.from_folder(tmp_path, dtype=dtype, max_tokens=64 * 4, max_seqs=2)
        assert len(engine.cache.kv_groups) == 1 and next(iter(engine.cache.kv_groups.values())).k.shape[0] == 1
        reqs = [tiny.random_prompt(300, n, n + 1) for n in (100, 37)]
        refs = [plain_shared_logits(w, r) for r in reqs]
        scale = max(float(r.abs().max()) for r in refs)
        slots = [engine.acquire() for _ in reqs]
        head = engine.step([(s, r[:-5], list(range(len(r) - 5))) for s, r in zip(slots, reqs)]).cpu()
        want = torch.cat([ref[:-5] for ref in refs])
        assert float((head.double() - want).abs().max()) / scale <= tiny.TOL[dtype]
        for i in range(5, 0, -1):
            rows = engine.step([(s, [r[-i]], [0]) for s, r in zip(slots, reqs)]).cpu()
            for b, ref in enumerate(refs):
                assert float((rows[b].double() - ref[len(reqs[b]) - i]).abs().max()) / scale <= tiny.TOL[dtype]
    finally:
        unregister_architecture("ToySharedKVForCausalLM")
