"""Another norm and another arrangement of a layer, defined HERE, registered, built and stepped without touching
the library.

* ``CenteredNorm`` subtracts the row's mean, divides by its standard deviation and applies a weight and a bias
  (the library's norm has neither a mean nor a bias). It is also the model's final norm.
* ``ParallelBlock`` has ONE norm; the mixer and the feed-forward both read that norm's output and both add into
  the residual: h += mixer(norm(h)) + ffn(norm(h)) (the library's block norms twice and runs them one after the other).

The mixer and the feed-forward inside are the library's own attention and SwiGLU: the arrangement and the norm
are chosen by the configuration, layer by layer (layer 0 is the parallel block, layer 1 the library's pre-norm
block with the toy norm in one of its two places). Plain tensor arithmetic on the device: these parts show the
interfaces, they are no model of anyone's.
"""
import pytest
import torch

import tiny
from plain import llama_plain as P
from spissa_b200 import Engine
from spissa_b200.config import (LayerSpec, ModelSpec, PartSpec, config_from_dict, register_architecture,
                                unregister_architecture)
from spissa_b200.parts import Block, Norm, WeightSpec, register_part, unregister_part
from spissa_b200.parts.registry import build_part
from spissa_b200.weights import write_random_model

pytestmark = pytest.mark.gpu
BASE = dict(tiny.TINY_B, num_hidden_layers=2, hidden_size=80, num_attention_heads=5, num_key_value_heads=1,
            head_dim=16, intermediate_size=136, vocab_size=210, rope_scaling=None)
EPS = 3e-4


def centered_norm(h, weight, bias, eps):
    mean = h.mean(dim=-1, keepdim=True)
    var = ((h - mean) ** 2).mean(dim=-1, keepdim=True)
    return (h - mean) / torch.sqrt(var + eps) * weight + bias


class CenteredNorm(Norm):
    graph_safe = True

    def __init__(self, size, eps, prefix=""):
        super().__init__(prefix)
        self.size, self.eps = int(size), float(eps)

    def weight_specs(self):
        return [WeightSpec(self.prefix + "weight", (self.size,), init="ones"), WeightSpec(self.prefix + "bias", (self.size,))]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.weight, self.bias = tensors[self.prefix + "weight"].float(), tensors[self.prefix + "bias"].float()

    def forward(self, h, rows=None):
        if rows is not None:
            h = h[rows.long()]
        return centered_norm(h, self.weight, self.bias, self.eps).to(self.rt.act_dtype)


class ParallelBlock(Block):
    graph_safe = True

    def __init__(self, mixer, ffn, norms, prefix=""):
        super().__init__(prefix)
        self.mixer = build_part("mixer", mixer)
        self.ffn = build_part("ffn", ffn)
        self.norm = build_part("norm", norms["shared"])

    def children(self):
        return [self.norm, self.mixer, self.ffn]

    def cache_request(self):
        return self.mixer.cache_request()

    def forward(self, h, step, cache):
        x = self.norm.forward(h)                     # both branches read the same normed rows
        self.mixer.forward(x, step, cache, h)
        self.ffn.forward(x, step, h)


class ToyArrangementConfig:
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
        H = BASE["hidden_size"]
        toy_norm = lambda prefix: PartSpec("toy_centered", dict(size=H, eps=EPS), prefix=prefix)
        l0, l1 = llama.layers
        l0 = LayerSpec("toy_parallel", l0.mixer, l0.ffn, {"shared": toy_norm("model.layers.0.shared_norm.")})
        l1 = LayerSpec(l1.block, l1.mixer, l1.ffn, {"mixer": l1.norms["mixer"], "ffn": toy_norm("model.layers.1.centered.")})
        return ModelSpec(**{**llama.__dict__, "architecture": "ToyArrangementForCausalLM", "layers": (l0, l1),
                            "final_norm": toy_norm("model.final_centered.")})


@pytest.fixture()
def toy():
    register_part("norm", "toy_centered", CenteredNorm)
    register_part("block", "toy_parallel", ParallelBlock)
    register_architecture("ToyArrangementForCausalLM", ToyArrangementConfig)
    yield
    unregister_architecture("ToyArrangementForCausalLM")
    unregister_part("block", "toy_parallel")
    unregister_part("norm", "toy_centered")


def plain_logits(w, ids):
    n = P.config_numbers(BASE)
    w = {k: v.double() for k, v in w.items()}
    T = len(ids)
    pos = torch.arange(T)
    inv = P.rope_inv_freq(n["theta"], n["hd"]).double()

    def attention(a, p):
        q = P.linear(a, w[p + "self_attn.q_proj.weight"]).view(T, n["nh"], n["hd"])
        k = P.linear(a, w[p + "self_attn.k_proj.weight"]).view(T, n["nkv"], n["hd"])
        v = P.linear(a, w[p + "self_attn.v_proj.weight"]).view(T, n["nkv"], n["hd"])
        q, k = P.apply_rope(q, pos, inv), P.apply_rope(k, pos, inv)
        return P.linear(P.causal_attention(q, k, v).reshape(T, -1), w[p + "self_attn.o_proj.weight"])

    h = P.embedding(w["model.embed_tokens.weight"], ids)
    # layer 0: one norm, two branches
    x = centered_norm(h, w["model.layers.0.shared_norm.weight"], w["model.layers.0.shared_norm.bias"], EPS)
    h = h + attention(x, "model.layers.0.") + P.swiglu(x, w, "model.layers.0.mlp.")
    # layer 1: the usual arrangement, the toy norm before the feed-forward
    h = h + attention(P.rms_norm(h, w["model.layers.1.input_layernorm.weight"], n["eps"]), "model.layers.1.")
    m = centered_norm(h, w["model.layers.1.centered.weight"], w["model.layers.1.centered.bias"], EPS)
    h = h + P.swiglu(m, w, "model.layers.1.mlp.")
    h = centered_norm(h, w["model.final_centered.weight"], w["model.final_centered.bias"], EPS)
    return P.linear(h, w["lm_head.weight"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_another_norm_and_another_arrangement_run_through_the_engine(toy, tmp_path, dtype):
    cfg = config_from_dict(dict(architectures=["ToyArrangementForCausalLM"]))
    write_random_model(cfg, tmp_path, seed=4, std=0.05)
    pcfg, w = P.read_model_folder(tmp_path)
    assert "model.layers.0.shared_norm.bias" in w and "model.layers.0.input_layernorm.weight" not in w
    assert "model.final_centered.weight" in w and "model.norm.weight" not in w
    engine = Engine.from_folder(tmp_path, dtype=dtype, max_tokens=64 * 8, max_seqs=3)
    reqs = [tiny.random_prompt(210, n, 3 * n) for n in (70, 9, 130)]
    refs = [plain_logits(w, r) for r in reqs]
    scale = max(float(r.abs().max()) for r in refs)
    tol = tiny.TOL[dtype]
    slots = [engine.acquire() for _ in reqs]
    got = engine.step([(s, r, list(range(len(r)))) for s, r in zip(slots, reqs)]).cpu()
    worst = float((got.double() - torch.cat(refs)).abs().max()) / scale
    assert worst <= tol, f"whole prompts: {worst:.3e} of the largest logit (allowed {tol:.1e})"
    for s in slots:
        engine.release(s)
    # cut into steps: all but the last four tokens, then one by one; then greedy generation through the entry point
    slots = [engine.acquire() for _ in reqs]
    engine.step([(s, r[:-4], []) for s, r in zip(slots, reqs)])
    for i in (4, 3, 2, 1):
        rows = engine.step([(s, [r[-i]], [0]) for s, r in zip(slots, reqs)]).cpu()
        for b, ref in enumerate(refs):
            e = float((rows[b].double() - ref[len(reqs[b]) - i]).abs().max()) / scale
            assert e <= tol, f"sequence {b}, token -{i}: {e:.3e}"
    for s in slots:
        engine.release(s)
    engine.cache.check()
    assert engine.model._fused is None           # a block that offers no description of itself runs part by part
    results, _ = engine.generate([reqs[1]], max_new_tokens=3, stop_ids=[])
    seq = list(reqs[1])
    for tok in results[0].tokens:
        ref = plain_logits(w, seq)[-1]
        top2 = torch.topk(ref, 2).values
        if float(top2[0] - top2[1]) > 4 * tol * scale:            # a clear winner: the engine must have found it
            assert tok == int(ref.argmax())
        seq.append(tok)
