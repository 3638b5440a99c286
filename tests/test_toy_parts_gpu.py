"""A feed-forward with routing and another position encoding, defined HERE, registered, built and stepped
without touching the library.

* ``PairRotary`` turns neighbouring pairs (2i, 2i+1) of every head by position·θ_i instead of the halves (i, i + d/2)
  that the library's rotary part turns; it offers ``apply`` (change q and k in place), not ``rotary()``, so the
  attention mixer projects, lets it work on the 32-bit products, and only then writes the cache.
* ``RoutedFFN`` has a router and two small experts; each token goes to the expert with the larger router logit,
  weighted by the softmax of the two logits.

The toy architecture uses the pair rotation in layer 0, no position encoding at all in layer 1, and the routed
feed-forward in layer 1. These parts are plain tensor arithmetic on the device: they show the interfaces, they
are no model of anyone's.
"""
import pytest
import torch

import tiny
from plain import llama_plain as P
from spissa_b200 import Engine
from spissa_b200.config import (LayerSpec, ModelSpec, PartSpec, config_from_dict, register_architecture,
                                unregister_architecture)
from spissa_b200.parts import FeedForward, PositionEncoding, WeightSpec, register_part, unregister_part
from spissa_b200.weights import write_random_model

pytestmark = pytest.mark.gpu
BASE = dict(tiny.TINY_B, num_hidden_layers=2, hidden_size=96, num_attention_heads=3, num_key_value_heads=1,
            head_dim=32, intermediate_size=256, vocab_size=300, rope_scaling=None)
THETA = 777.0
EXPERT_WIDTH = 40


def pair_angles(positions, hd):
    inv = 1.0 / (THETA ** (torch.arange(0, hd, 2, dtype=torch.float64, device=positions.device) / hd))
    return positions.double()[:, None] * inv[None, :]                       # [T, hd / 2]


def pair_rotate(x, positions):
    """x [T, heads, hd]: (x_{2i}, x_{2i+1}) turned by position·θ_i."""
    ang = pair_angles(positions, x.shape[-1]).to(x.device)
    c, s = torch.cos(ang)[:, None, :].to(x.dtype), torch.sin(ang)[:, None, :].to(x.dtype)
    even, odd = x[..., 0::2], x[..., 1::2]
    out = torch.empty_like(x)
    out[..., 0::2] = even * c - odd * s
    out[..., 1::2] = odd * c + even * s
    return out


class PairRotary(PositionEncoding):
    graph_safe = True

    def __init__(self, prefix=""):
        super().__init__(prefix)

    def apply(self, qkv, step, nh, nkv, hd):
        T = qkv.shape[0]
        qk = qkv[:, :(nh + nkv) * hd].view(T, nh + nkv, hd)
        qk.copy_(pair_rotate(qk, step.positions))


class RoutedFFN(FeedForward):
    graph_safe = True

    def __init__(self, hidden_size, width, prefix=""):
        super().__init__(prefix)
        self.hidden_size, self.width = hidden_size, width
        self.names = dict(router=prefix + "router.weight", up=[prefix + f"experts.{e}.up.weight" for e in range(2)],
                          down=[prefix + f"experts.{e}.down.weight" for e in range(2)])

    def weight_specs(self):
        H, W = self.hidden_size, self.width
        return ([WeightSpec(self.names["router"], (2, H))] + [WeightSpec(n, (W, H)) for n in self.names["up"]] +
                [WeightSpec(n, (H, W)) for n in self.names["down"]])

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.router = tensors[self.names["router"]].float()
        self.up = [tensors[n].float() for n in self.names["up"]]
        self.down = [tensors[n].float() for n in self.names["down"]]

    def forward(self, x, step, residual):
        residual += routed_ffn(x.float(), self.router, self.up, self.down)


def routed_ffn(x, router, up, down):
    logits = x @ router.t()                                                 # [T, 2]
    weight = torch.softmax(logits, dim=-1)
    choice = logits.argmax(dim=-1)
    out = torch.zeros_like(x)
    for e in range(2):
        y = torch.relu(x @ up[e].t()) @ down[e].t()
        out += torch.where((choice == e)[:, None], weight[:, e:e + 1] * y, torch.zeros_like(y))
    return out


class ToyPartsConfig:
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
        l0, l1 = llama.layers
        l0 = LayerSpec(l0.block, l0.mixer.with_params(position=PartSpec("toy_pair_rotary", {})), l0.ffn, l0.norms)
        l1 = LayerSpec(l1.block, l1.mixer.with_params(position=None),
                       PartSpec("toy_routed", dict(hidden_size=BASE["hidden_size"], width=EXPERT_WIDTH),
                                prefix="model.layers.1.moe."), l1.norms)
        return ModelSpec(**{**llama.__dict__, "architecture": "ToyPartsForCausalLM", "layers": (l0, l1)})


@pytest.fixture()
def toy():
    register_part("position", "toy_pair_rotary", PairRotary)
    register_part("ffn", "toy_routed", RoutedFFN)
    register_architecture("ToyPartsForCausalLM", ToyPartsConfig)
    yield
    unregister_architecture("ToyPartsForCausalLM")
    unregister_part("ffn", "toy_routed")
    unregister_part("position", "toy_pair_rotary")


def plain_logits(w, ids):
    """Logits of the whole sequence and, per token, how far apart the router's two logits are."""
    n = P.config_numbers(BASE)
    w = {k: v.double() for k, v in w.items()}
    T = len(ids)
    pos = torch.arange(T)
    h = P.embedding(w["model.embed_tokens.weight"], ids)
    for i in range(2):
        p = f"model.layers.{i}."
        a = P.rms_norm(h, w[p + "input_layernorm.weight"], n["eps"])
        q = P.linear(a, w[p + "self_attn.q_proj.weight"]).view(T, n["nh"], n["hd"])
        k = P.linear(a, w[p + "self_attn.k_proj.weight"]).view(T, n["nkv"], n["hd"])
        v = P.linear(a, w[p + "self_attn.v_proj.weight"]).view(T, n["nkv"], n["hd"])
        if i == 0:
            q, k = pair_rotate(q, pos), pair_rotate(k, pos)
        ctx = P.causal_attention(q, k, v).reshape(T, -1)
        h = h + P.linear(ctx, w[p + "self_attn.o_proj.weight"])
        m = P.rms_norm(h, w[p + "post_attention_layernorm.weight"], n["eps"])
        if i == 0:
            h = h + P.swiglu(m, w, p + "mlp.")
        else:
            logits = m @ w[p + "moe.router.weight"].t()
            margin = (logits[:, 0] - logits[:, 1]).abs()
            h = h + routed_ffn(m, w[p + "moe.router.weight"], [w[p + f"moe.experts.{e}.up.weight"] for e in range(2)],
                               [w[p + f"moe.experts.{e}.down.weight"] for e in range(2)])
    h = P.rms_norm(h, w["model.norm.weight"], n["eps"])
    return P.linear(h, w["lm_head.weight"]), margin


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_routed_feed_forward_and_pair_rotation_run_through_the_engine(toy, tmp_path, dtype):
    cfg = config_from_dict(dict(architectures=["ToyPartsForCausalLM"]))
    write_random_model(cfg, tmp_path, seed=9, std=0.05)
    pcfg, w = P.read_model_folder(tmp_path)
    assert "model.layers.1.moe.router.weight" in w and "model.layers.1.mlp.gate_proj.weight" not in w
    engine = Engine.from_folder(tmp_path, dtype=dtype, max_tokens=64 * 8, max_seqs=3)
    reqs = [tiny.random_prompt(300, n, n) for n in (70, 9, 130)]
    plain = [plain_logits(w, r) for r in reqs]
    refs = [p[0] for p in plain]
    scale = max(float(r.abs().max()) for r in refs)
    tol = tiny.TOL[dtype]
    # The routed layer is the last one, so a token's choice of expert touches that token's logits only. A token
    # whose two router logits are nearly equal may go to the other expert once activations are rounded to
    # bfloat16: that is the formula's own discontinuity, not a fault, and such tokens are left out (there are few).
    near_tie = 0.0 if dtype == "float32" else 0.02
    clear = [p[1] > near_tie for p in plain]
    assert sum(int(c.sum()) for c in clear) >= 0.9 * sum(len(r) for r in reqs)
    slots = [engine.acquire() for _ in reqs]
    got = engine.step([(s, r, list(range(len(r)))) for s, r in zip(slots, reqs)]).cpu()
    err = (got.double() - torch.cat(refs)).abs().amax(dim=1) / scale
    worst = float(err[torch.cat(clear)].max())
    assert worst <= tol, f"whole prompts: {worst:.3e} of the largest logit (allowed {tol:.1e})"
    for s in slots:
        engine.release(s)
    # cut into steps: whole prompt but the last three tokens, then one by one (decode steps)
    slots = [engine.acquire() for _ in reqs]
    engine.step([(s, r[:-3], []) for s, r in zip(slots, reqs)])
    for i in (3, 2, 1):
        rows = engine.step([(s, [r[-i]], [0]) for s, r in zip(slots, reqs)]).cpu()
        for b, ref in enumerate(refs):
            if not bool(clear[b][len(reqs[b]) - i]):
                continue
            e = float((rows[b].double() - ref[len(reqs[b]) - i]).abs().max()) / scale
            assert e <= tol, f"sequence {b}, token -{i}: {e:.3e}"
    for s in slots:
        engine.release(s)
    engine.cache.check()
    assert engine.model._fused is None           # parts that offer no description of themselves run part by part


# ------------------------------------------------------------------ an embedding that needs the tokens' positions
class LearnedPositionEmbedding:
    """h[t] = E[id_t] + Ppos[position_t]: absolute, learned positions live in the embedding, which therefore needs
    more of the step than the token ids. Registered HERE under role ``embedding``."""
    graph_safe = True

    def __init__(self, vocab_size, hidden_size, max_positions, prefix="", **_):
        self.prefix = prefix
        self.vocab_size, self.hidden_size, self.max_positions = vocab_size, hidden_size, max_positions
        self.rt = None

    def children(self):
        return []

    def weight_specs(self):
        return [WeightSpec(self.prefix + "weight", (self.vocab_size, self.hidden_size)),
                WeightSpec("model.embed_positions.weight", (self.max_positions, self.hidden_size))]

    def all_weight_specs(self):
        return self.weight_specs()

    def bind(self, tensors, rt):
        self.rt = rt
        self.table = tensors[self.prefix + "weight"].float()
        self.pos = tensors["model.embed_positions.weight"].float()

    def bind_all(self, tensors, rt):
        self.bind(tensors, rt)

    def forward(self, step):
        return (self.table[step.tokens.long()] + self.pos[step.positions.long()]).contiguous()


class ToyLearnedConfig(ToyPartsConfig):
    def to_spec(self):
        llama = self.base.to_spec()
        emb = PartSpec("toy_learned_positions", dict(llama.embedding.params, max_positions=512), prefix=llama.embedding.prefix)
        layers = tuple(LayerSpec(l.block, l.mixer.with_params(position=None), l.ffn, l.norms) for l in llama.layers)
        return ModelSpec(**{**llama.__dict__, "architecture": "ToyLearnedForCausalLM", "embedding": emb, "layers": layers})


def test_an_embedding_with_learned_positions_gets_the_step(tmp_path):
    """The model hands the embedding the whole step, so positions can enter there; the layers then use no position
    encoding at all. Whole prompts, a prompt that continues, and decode steps against the same arithmetic in float64."""
    register_part("embedding", "toy_learned_positions", LearnedPositionEmbedding)
    register_architecture("ToyLearnedForCausalLM", ToyLearnedConfig)
    try:
        cfg = config_from_dict(dict(architectures=["ToyLearnedForCausalLM"]))
        write_random_model(cfg, tmp_path, seed=13, std=0.05)
        pcfg, w = P.read_model_folder(tmp_path)
        assert tuple(w["model.embed_positions.weight"].shape) == (512, BASE["hidden_size"])
        engine = Engine.from_folder(tmp_path, dtype="float32", max_tokens=64 * 8, max_seqs=2)
        n = P.config_numbers(BASE)

        def plain(ids):
            wd = {k: v.double() for k, v in w.items()}
            T = len(ids)
            h = P.embedding(wd["model.embed_tokens.weight"], ids) + wd["model.embed_positions.weight"][:T]
            for i in range(2):
                p = f"model.layers.{i}."
                a = P.rms_norm(h, wd[p + "input_layernorm.weight"], n["eps"])
                q = P.linear(a, wd[p + "self_attn.q_proj.weight"]).view(T, n["nh"], n["hd"])
                k = P.linear(a, wd[p + "self_attn.k_proj.weight"]).view(T, n["nkv"], n["hd"])
                v = P.linear(a, wd[p + "self_attn.v_proj.weight"]).view(T, n["nkv"], n["hd"])
                h = h + P.linear(P.causal_attention(q, k, v).reshape(T, -1), wd[p + "self_attn.o_proj.weight"])
                m = P.rms_norm(h, wd[p + "post_attention_layernorm.weight"], n["eps"])
                h = h + P.swiglu(m, wd, p + "mlp.")
            return P.linear(P.rms_norm(h, wd["model.norm.weight"], n["eps"]), wd["lm_head.weight"])

        reqs = [tiny.random_prompt(300, m, 3 * m) for m in (40, 75)]
        refs = [plain(r) for r in reqs]
        scale = max(float(r.abs().max()) for r in refs)
        slots = [engine.acquire() for _ in reqs]
        got = engine.step([(s, r[:-5], [0, len(r) - 6]) for s, r in zip(slots, reqs)]).cpu().double()
        want = torch.stack([refs[0][0], refs[0][34], refs[1][0], refs[1][69]])
        assert float((got - want).abs().max()) / scale <= tiny.TOL["float32"]
        for i in range(5, 0, -1):                                    # positions keep counting across steps
            rows = engine.step([(s, [r[-i]], [0]) for s, r in zip(slots, reqs)]).cpu().double()
            for b, ref in enumerate(refs):
                assert float((rows[b] - ref[len(reqs[b]) - i]).abs().max()) / scale <= tiny.TOL["float32"]
        engine.cache.check()
    finally:
        unregister_architecture("ToyLearnedForCausalLM")
        unregister_part("embedding", "toy_learned_positions")
