"""A mixer with state of its own, defined HERE, registered, built and stepped without touching the library.

The toy mixer keeps a running, decaying sum of its inputs per sequence (state [H]) and
projects it: s_t = a·s_{t-1} + x_t, y_t = s_t·Wᵀ. The toy architecture puts it in every
second layer, between ordinary attention layers, so one model has different mixers in
different layers, and its last layer runs twice in the schedule.
"""
import json

import pytest
import torch

import tiny
from plain import llama_plain as P
from spissa_b200 import Engine
from spissa_b200.config import (LayerSpec, ModelSpec, PartSpec, ScheduleEntry, config_from_dict,
                                register_architecture, unregister_architecture)
from spissa_b200.parts import Mixer, StateRequest, WeightSpec, register_part, unregister_part
from spissa_b200.weights import write_random_model

pytestmark = pytest.mark.gpu
DECAY = 0.75


class DecayMixer(Mixer):
    def __init__(self, hidden_size, decay, prefix=""):
        super().__init__(prefix)
        self.hidden_size, self.decay = hidden_size, decay
        self.name = prefix + "mix.weight"

    def weight_specs(self):
        return [WeightSpec(self.name, (self.hidden_size, self.hidden_size))]

    def cache_request(self):
        return StateRequest((self.hidden_size,), torch.float32)

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.w = tensors[self.name].float()

    def forward(self, x, step, cache, residual):
        starts, slots = step.host["seq_start"], step.host["seq_slot"]
        for b, slot in enumerate(slots):
            s = cache.state[slot]
            for t in range(starts[b], starts[b + 1]):
                s = self.decay * s + x[t].float()
                residual[t] += s @ self.w.t()
            cache.state[slot] = s


class ToyConfig:
    def __init__(self, d):
        self.d = d
        self.base = config_from_dict({**tiny.TINY_A, "architectures": ["LlamaForCausalLM"]})

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
                layer = LayerSpec(layer.block, PartSpec("toy_decay", dict(hidden_size=64, decay=DECAY),
                                                        prefix=f"model.layers.{i}.toy."), layer.ffn, layer.norms)
            layers.append(layer)
        schedule = (ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(0, 2))     # layer 0 runs twice
        return ModelSpec(**{**llama.__dict__, "architecture": "ToyDecayForCausalLM", "layers": tuple(layers),
                            "schedule": schedule})


@pytest.fixture()
def toy():
    register_part("mixer", "toy_decay", DecayMixer)
    register_architecture("ToyDecayForCausalLM", ToyConfig)
    yield
    unregister_architecture("ToyDecayForCausalLM")
    unregister_part("mixer", "toy_decay")


def plain_toy(pcfg, w, ids):
    n = P.config_numbers(pcfg)
    w = {k: v.double() for k, v in w.items()}
    inv = P.rope_inv_freq(n["theta"], n["hd"], n["scaling"])
    h = P.embedding(w["model.embed_tokens.weight"], ids)

    def toy_layer(x):
        p = "model.layers.1."
        a = P.rms_norm(x, w[p + "input_layernorm.weight"], n["eps"])
        s = torch.zeros(64, dtype=torch.float64)
        out = []
        for t in range(a.shape[0]):
            s = DECAY * s + a[t]
            out.append(s @ w[p + "toy.mix.weight"].t())
        r = x + torch.stack(out)
        m = P.rms_norm(r, w[p + "post_attention_layernorm.weight"], n["eps"])
        return r + P.swiglu(m, w, p + "mlp.")

    h = P.decoder_layer(h, w, 0, n, inv)
    h = toy_layer(h)
    h = P.decoder_layer(h, w, 0, n, inv)
    h = P.rms_norm(h, w["model.norm.weight"], n["eps"])
    return P.linear(h, w["model.embed_tokens.weight"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_mixer_with_state_runs_through_the_engine(toy, tmp_path, dtype):
    cfg_json = dict(architectures=["ToyDecayForCausalLM"])
    cfg = config_from_dict(cfg_json)
    write_random_model(cfg, tmp_path, seed=3, std=0.05)
    pcfg, w = P.read_model_folder(tmp_path)
    assert "model.layers.1.toy.mix.weight" in w and "model.layers.1.self_attn.q_proj.weight" not in w
    pcfg = {**tiny.TINY_A}
    engine = Engine.from_folder(tmp_path, dtype=dtype, max_tokens=64 * 6, max_seqs=3)
    assert len(engine.cache.state_groups) == 1 and len(engine.cache.kv_groups) == 1
    reqs = [tiny.random_prompt(256, n, n) for n in (20, 7, 70)]
    refs = [plain_toy(pcfg, w, r) for r in reqs]
    scale = max(float(r.abs().max()) for r in refs)
    tol = tiny.TOL[dtype]
    # whole, in one ragged step
    slots = [engine.acquire() for _ in reqs]
    got = engine.step([(s, r, list(range(len(r)))) for s, r in zip(slots, reqs)]).cpu()
    assert float((got.double() - torch.cat(refs)).abs().max()) / scale <= tol
    for s in slots:
        engine.release(s)
    # cut into steps: the state is carried in the slot; a reused slot starts from zero
    slots = [engine.acquire() for _ in reqs]
    head = engine.step([(s, r[:-3], [len(r) - 4]) for s, r in zip(slots, reqs)]).cpu()
    for b, ref in enumerate(refs):
        assert float((head[b].double() - ref[len(reqs[b]) - 4]).abs().max()) / scale <= tol
    for i in (3, 2, 1):
        rows = engine.step([(s, [r[-i]], [0]) for s, r in zip(slots, reqs)]).cpu()
        for b, ref in enumerate(refs):
            assert float((rows[b].double() - ref[len(reqs[b]) - i]).abs().max()) / scale <= tol
    for s in slots:
        engine.release(s)
    engine.cache.check()
    # a layer that offers no description of itself keeps the whole model out of the one-kernel decode path
    assert engine.model._fused is None


def test_state_is_what_it_was_after_a_refused_step_and_after_a_step_that_failed_on_the_device(toy, tmp_path):
    """Fixed-size state cannot be truncated the way a length can: the cache copies the rows of a step's sequences
    aside before the step runs and puts them back when the step is rolled back."""
    from spissa_b200.csrc import lib as K
    from spissa_b200.csrc.lib import KernelError
    from spissa_b200.engine.engine import StepError
    cfg = config_from_dict(dict(architectures=["ToyDecayForCausalLM"]))
    write_random_model(cfg, tmp_path, seed=3, std=0.05)
    pcfg, w = P.read_model_folder(tmp_path)
    engine = Engine.from_folder(tmp_path, dtype="float32", max_tokens=64 * 6, max_seqs=3)
    (group,) = engine.cache.state_groups.values()
    reqs = [tiny.random_prompt(256, n, n) for n in (20, 33)]
    refs = [plain_toy({**tiny.TINY_A}, w, r) for r in reqs]
    slots = [engine.acquire() for _ in reqs]
    engine.step([(s, r[:-2], []) for s, r in zip(slots, reqs)])
    before = group.state.clone()
    assert float(before.abs().sum()) > 0
    with pytest.raises(StepError):
        engine.step([(slots[0], [5], [0]), (slots[1], [100000], [0])])          # refused on the host
    assert torch.equal(group.state, before)
    K.status_word("cuda:0").fill_(123)
    with pytest.raises(KernelError, match="code 123"):
        engine.step([(s, [r[-2]], [0]) for s, r in zip(slots, reqs)])            # ran, then rolled back
    assert torch.equal(group.state, before)
    assert [engine.length(s) for s in slots] == [len(r) - 2 for r in reqs]
    scale = max(float(r.abs().max()) for r in refs)
    for i in (2, 1):
        rows = engine.step([(s, [r[-i]], [0]) for s, r in zip(slots, reqs)]).cpu()
        for b, ref in enumerate(refs):
            assert float((rows[b].double() - ref[len(reqs[b]) - i]).abs().max()) / scale <= tiny.TOL["float32"]
    # through the generation loop a model with state keeps one step in flight, and the result is the plain one
    for s in slots:
        engine.release(s)
    engine.cache.check()
