"""Plain, slow implementation of the Llama decoder that spissa runs.

Whole sequences, no cache, one function per part, plain tensor arithmetic on the
CPU. It shares no code with ``spissa_b200``: it reads config.json keys and
safetensors files itself. Every function cites the place in the reference
project (paths within Erik-cpu-create/spissa) whose formula it restates.

The reference is a Rust project and no Rust toolchain exists where this was
written, so this file rests on the reference's formulas (and on the reference's
own unit-test vectors, replayed in tests/test_plain.py), not on a compiled run.

The llama3 frequency scaling and the optional window are not in the reference
(crates/spissa-import/src/safetensors.rs:163-175 drops ``rope_type: llama3``);
they follow the published Llama 3.1 rule and are marked "ours" below.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import torch


# ----------------------------------------------------------------------------
# model folder
# ----------------------------------------------------------------------------

_ST_DTYPES = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16,
              "I32": torch.int32, "I64": torch.int64, "F64": torch.float64}


def read_safetensors(path) -> dict:
    """8-byte little-endian header length, JSON header, raw data.

    crates/spissa-import/src/safetensors.rs:261-289 (open), :307-323 (read by name).
    """
    raw = Path(path).read_bytes()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen])
    base = 8 + hlen
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        dt = _ST_DTYPES[meta["dtype"]]
        buf = bytearray(raw[base + lo:base + hi])
        if len(buf) == 0:
            out[name] = torch.empty(meta["shape"], dtype=dt)
        else:
            out[name] = torch.frombuffer(buf, dtype=dt).reshape(meta["shape"]).clone()
    return out


def read_model_folder(folder):
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    weights = read_safetensors(folder / "model.safetensors")
    return cfg, weights


def config_numbers(cfg: dict) -> dict:
    """The numbers the Llama path takes from config.json, with the reference's defaults.

    crates/spissa-runtime/src/models/llama/api.rs:131-171: heads, kv heads default to
    heads, hidden, eps default 1e-5, theta default 10000, head_dim default H / heads.
    """
    nh = cfg["num_attention_heads"]
    H = cfg["hidden_size"]
    return dict(
        H=H,
        I=cfg["intermediate_size"],
        L=cfg["num_hidden_layers"],
        nh=nh,
        nkv=cfg.get("num_key_value_heads") or nh,
        hd=cfg.get("head_dim") or H // nh,
        eps=cfg.get("rms_norm_eps", 1e-5),
        theta=cfg.get("rope_theta", 10000.0),
        scaling=cfg.get("rope_scaling"),
        V=cfg["vocab_size"],
    )


# ----------------------------------------------------------------------------
# parts
# ----------------------------------------------------------------------------

def embedding(table: torch.Tensor, ids) -> torch.Tensor:
    """h[t,:] = E[id_t,:], no scale; an id beyond the table is an error.

    crates/spissa-runtime/src/ops.rs:6-30.
    """
    ids = torch.as_tensor(ids, dtype=torch.long)
    if ids.numel() and (int(ids.max()) >= table.shape[0] or int(ids.min()) < 0):
        raise ValueError("token id out of range")
    return table[ids]


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """y = x · Wᵀ with W stored [out, in], no bias.

    crates/spissa-runtime/src/ops.rs:62-105.
    """
    return x @ w.t()


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """Per row: ms = Σx²/H; inv = 1/√(ms+eps); y = x·inv·w (weight multiplies directly).

    crates/spissa-runtime/src/ops.rs:159-179.
    """
    ms = (x * x).sum(dim=-1, keepdim=True) / x.shape[-1]
    inv = 1.0 / torch.sqrt(ms + eps)
    return x * inv * w


def silu(x: torch.Tensor) -> torch.Tensor:
    """silu(z) = z / (1 + e^{-z}).  crates/spissa-runtime/src/ops.rs:192-194."""
    return x / (1.0 + torch.exp(-x))


def rope_inv_freq(theta: float, rotary_dim: int, scaling=None, dtype=torch.float32) -> torch.Tensor:
    """inv_freq_i = 1 / θ^(2i/rd), computed in 32-bit like the reference.

    crates/spissa-runtime/src/rotary.rs:454-465 (exponent = 2·pair / rotary_dim,
    ``base.powf(exponent)``, all f32).

    Ours (not in the reference): ``rope_type: llama3`` rescales the table once.
    With λ = 2π/inv_freq: λ > n0/lo ⇒ inv_freq/f; λ < n0/hi ⇒ unchanged; else the
    blend (1−s)·inv_freq/f + s·inv_freq with s = (n0/λ − lo)/(hi − lo).
    """
    pair = torch.arange(0, rotary_dim, 2, dtype=dtype)
    inv = 1.0 / (torch.tensor(theta, dtype=dtype) ** (pair / rotary_dim))
    if scaling:
        kind = scaling.get("rope_type", scaling.get("type"))
        if kind == "llama3":
            f = scaling["factor"]
            lo = scaling["low_freq_factor"]
            hi = scaling["high_freq_factor"]
            n0 = scaling["original_max_position_embeddings"]
            wavelen = 2 * math.pi / inv
            out = inv.clone()
            for i in range(inv.numel()):
                lam = float(wavelen[i])
                if lam > n0 / lo:
                    out[i] = inv[i] / f
                elif lam < n0 / hi:
                    out[i] = inv[i]
                else:
                    s = (n0 / wavelen[i] - lo) / (hi - lo)
                    out[i] = (1 - s) * inv[i] / f + s * inv[i]
            inv = out
        elif kind == "linear":
            # positions divided by the factor (crates/spissa-runtime/src/rotary.rs:127-193,
            # the linear rule of the Gemma path); the same as dividing every frequency
            inv = inv / scaling["factor"]
        elif kind in (None, "default"):
            pass
        else:
            raise ValueError(f"plain implementation has no rope scaling {kind!r}")
    return inv


def apply_rope(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """Rotate-half on ``x`` [T, heads, hd]: dim i pairs with i + rd/2.

    x'_i = x_i·cos − x_{i+rd/2}·sin;  x'_{i+rd/2} = x_{i+rd/2}·cos + x_i·sin;
    angle = position · inv_freq_i.
    crates/spissa-runtime/src/rotary.rs:98-123 (loop), :467-481 (pair rotation).
    """
    half = inv_freq.numel()
    ang = positions.to(inv_freq.dtype)[:, None] * inv_freq[None, :]          # [T, rd/2]
    cos = torch.cos(ang).to(x.dtype)[:, None, :]
    sin = torch.sin(ang).to(x.dtype)[:, None, :]
    out = x.clone()
    a = x[..., :half]
    b = x[..., half:2 * half]
    out[..., :half] = a * cos - b * sin
    out[..., half:2 * half] = b * cos + a * sin
    return out


def causal_attention(q, k, v, window=None) -> torch.Tensor:
    """Causal GQA attention of one whole sequence.

    q [T, nh, hd], k and v [T, nkv, hd]; head h reads kv head h // (nh/nkv);
    scores scaled by 1/√hd; keys after the query are masked to −∞; softmax with the
    max subtracted; output [T, nh·hd].
    crates/spissa-runtime/src/rotary.rs:335-415 (scores, mask, context),
    :549-569 (softmax).
    ``window`` (ours): a query at position p sees keys p−window+1 … p only.
    """
    T, nh, hd = q.shape
    nkv = k.shape[1]
    rep = nh // nkv
    scale = 1.0 / math.sqrt(hd)
    out = torch.zeros(T, nh, hd, dtype=q.dtype)
    for h in range(nh):
        g = h // rep
        s = (q[:, h, :] @ k[:, g, :].t()) * scale                 # [T, T]
        idx = torch.arange(T)
        mask = idx[None, :] > idx[:, None]
        if window is not None:
            mask = mask | (idx[None, :] <= idx[:, None] - window)
        s = s.masked_fill(mask, float("-inf"))
        m = s.max(dim=-1, keepdim=True).values
        e = torch.exp(s - m)
        p = e / e.sum(dim=-1, keepdim=True)
        out[:, h, :] = p @ v[:, g, :]
    return out.reshape(T, nh * hd)


def attention_block(x, w, prefix, n, inv_freq, positions=None, window=None):
    """q/k/v projections, rope on q and k, attention, output projection.

    crates/spissa-runtime/src/models/llama/generate.rs:274-358 (projections),
    :373-390 (rope), :395-405 (attention), :418-450 (output projection).
    """
    T = x.shape[0]
    if positions is None:
        positions = torch.arange(T)
    q = linear(x, w[prefix + "q_proj.weight"]).reshape(T, n["nh"], n["hd"])
    k = linear(x, w[prefix + "k_proj.weight"]).reshape(T, n["nkv"], n["hd"])
    v = linear(x, w[prefix + "v_proj.weight"]).reshape(T, n["nkv"], n["hd"])
    q = apply_rope(q, positions, inv_freq)
    k = apply_rope(k, positions, inv_freq)
    a = causal_attention(q, k, v, window=window)
    return linear(a, w[prefix + "o_proj.weight"])


def swiglu(x, w, prefix):
    """act = silu(x·Wgᵀ) ⊙ (x·Wuᵀ); out = act·Wdᵀ.

    crates/spissa-runtime/src/models/llama/generate.rs:590-637 and :642-763;
    crates/spissa-runtime/src/streaming/argmax.rs:314 (silu(gate)·up).
    """
    g = linear(x, w[prefix + "gate_proj.weight"])
    u = linear(x, w[prefix + "up_proj.weight"])
    return linear(silu(g) * u, w[prefix + "down_proj.weight"])


def decoder_layer(x, w, i, n, inv_freq):
    """Pre-norm block with two residual sums.

    crates/spissa-runtime/src/models/llama/generate.rs:190-199 (input norm),
    :459 (first residual), :465-471 (post-attention norm), :773 (second residual).
    """
    p = f"model.layers.{i}."
    a = rms_norm(x, w[p + "input_layernorm.weight"], n["eps"])
    r = x + attention_block(a, w, p + "self_attn.", n, inv_freq)
    m = rms_norm(r, w[p + "post_attention_layernorm.weight"], n["eps"])
    return r + swiglu(m, w, p + "mlp.")


def model_logits(cfg: dict, weights: dict, ids, dtype=torch.float64) -> torch.Tensor:
    """Logits at every position of one whole sequence, [T, V].

    Embedding, L layers, final norm, head; the head is ``lm_head.weight`` when that
    tensor exists, else the embedding table.
    crates/spissa-runtime/src/models/llama/api.rs:292-346 (stateless generate),
    :176-181 (tied head by tensor presence).
    The reference keeps activations in f32 and widens 16-bit weights exactly
    (crates/spissa-runtime/src/tensor.rs:217-221); ``dtype`` float64 gives the
    same arithmetic with less rounding and serves as ground truth.
    """
    n = config_numbers(cfg)
    w = {k: v.to(dtype) for k, v in weights.items()}
    # the angle table stays in 32-bit, as in the reference
    inv_freq = rope_inv_freq(n["theta"], n["hd"], n["scaling"], dtype=torch.float32)
    h = embedding(w["model.embed_tokens.weight"], ids)
    for i in range(n["L"]):
        h = decoder_layer(h, w, i, n, inv_freq)
    h = rms_norm(h, w["model.norm.weight"], n["eps"])
    head = w["lm_head.weight"] if "lm_head.weight" in w else w["model.embed_tokens.weight"]
    return linear(h, head)


# ----------------------------------------------------------------------------
# sampling
# ----------------------------------------------------------------------------

def sample_argmax(logits) -> int:
    """First maximum wins (strict ``>``).  crates/spissa-runtime/src/ops.rs:309-324."""
    best, best_v = 0, float(logits[0])
    for i in range(1, len(logits)):
        v = float(logits[i])
        if v > best_v:
            best, best_v = i, v
    return best


def seeded_unit_f32(seed: int) -> float:
    """One xorshift64* step; top 24 bits / 2^24.  crates/spissa-runtime/src/ops.rs:446-457."""
    mask = (1 << 64) - 1
    x = 0x9E3779B97F4A7C15 if seed == 0 else seed & mask
    x ^= x >> 12
    x ^= (x << 25) & mask
    x ^= x >> 27
    x = (x * 0x2545F4914F6CDD1D) & mask
    return float(x >> 40) / float(1 << 24)


def sample_top_k_top_p(logits, temperature: float, top_k: int, top_p: float, seed: int) -> int:
    """Temperature, then top-k, then top-p, then one draw.

    crates/spissa-runtime/src/ops.rs:377-430: greedy when temperature ≤ 0; softmax
    of logits/T; stable descending sort; keep k; keep the shortest prefix with
    cumulative ≥ p; walk the kept list with u·total.
    """
    if temperature <= 0.0:
        return sample_argmax(logits)
    if not (0.0 < top_p <= 1.0):
        raise ValueError("top_p must be in (0, 1]")
    x = torch.as_tensor(logits, dtype=torch.float32) / temperature
    e = torch.exp(x - x.max())
    probs = e / e.sum()
    order = sorted(range(len(probs)), key=lambda i: -float(probs[i]))   # stable
    if 0 < top_k < len(order):
        order = order[:top_k]
    kept, cum = [], torch.tensor(0.0)
    for i in order:
        cum = cum + probs[i]
        kept.append(i)
        if float(cum) >= top_p:
            break
    total = torch.stack([probs[i] for i in kept]).sum()
    thr = torch.tensor(seeded_unit_f32(seed), dtype=torch.float32) * total
    for i in kept:
        if float(thr) <= float(probs[i]):
            return i
        thr = thr - probs[i]
    return sample_argmax(logits)


def generate_greedy(cfg, weights, prompt, max_new_tokens, stop_ids=(), dtype=torch.float64):
    """Whole-sequence recompute for every new token; the stop token is returned, not fed.

    crates/spissa-runtime/src/models/llama/api.rs:281-367 (stateless loop).
    """
    ids = list(prompt)
    out = []
    for _ in range(max_new_tokens):
        tok = sample_argmax(model_logits(cfg, weights, ids, dtype)[-1])
        out.append(tok)
        if tok in stop_ids:
            break
        ids.append(tok)
    return out
