"""A step's layers with the norms, the rotation and the cache write folded into the matrix products.

Part by part a layer is eight launches: norm, QKV, rotate-and-store, attention, output projection, norm, gate/up,
down. When every layer's parts describe themselves through ``fused_fields()`` (the same pre-norm / RMS norm / rotary
grouped-query attention / SwiGLU, bfloat16 description that the one-kernel decode path reads) a step of 17 tokens
to 64 (a prompt, or a decode step of that many sequences: the kernel that streams the weights, ``tc_stream``) or of
more than 128 (the tile kernel, ``tc_gemm``) runs each layer as five. Between them the tile kernel splits K over a
cluster, which has no such epilogues, and is faster than either fused form (a 100-token step: 2.1 ms against 2.6):

* QKV product on ``xw`` = residual ⊙ norm weight, its result multiplied by each row's 1/rms, rotated, q stored and
  k, v written into the paged cache in the product's epilogue;
* attention (the mixer's own ``attend``);
* output projection that adds into the 32-bit residual and, in the same epilogue, writes the residual ⊙ next norm
  weight in bfloat16 and the rows' sums of squares per tile;
* gate/up product on that, scaled by 1/rms, with silu(gate)·up;
* down projection, again preparing the next layer's first norm.

The reference's block does the same work phase by phase (crates/spissa-runtime/src/models/llama/generate.rs:193-199
norm, :274-358 projections, :373-390 rotation, :410-416 cache append, :459-471 residual and second norm). Both ways
give the same logits up to rounding and are compared with each other and with the plain implementation in the tests.
"""
from __future__ import annotations

import torch

from ..csrc import lib as K
from ..parts.linear import STREAM_TOKENS, sm_count, tile_width
from .fused_decode import collect_fused_fields, five_launch_from
from ..phases import phase

MIN_TOKENS = 17          # up to 16 tokens the weight-streaming kernels (or the one-kernel decode path) run instead
TILE_TOKENS = 129        # from here on the tile kernel's epilogues


def fuses(n_tokens: int) -> bool:
    return MIN_TOKENS <= n_tokens <= STREAM_TOKENS or n_tokens >= TILE_TOKENS


class FusedPrefill:
    def __init__(self, model, fields: list):
        self.model = model
        self.fields = fields
        self.H = fields[0]["mixer"]["hidden_size"]
        self.hd = fields[0]["mixer"]["head_dim"]
        self.runs = 0
        self.layer_bytes = max(sum(w.numel() * w.element_size() for w in (f["mixer"]["qkv"], f["mixer"]["o"], f["ffn"]["gate_up"],
                                                                     f["ffn"]["down"])) for f in fields)
        # layers whose frequency tables are equal share one table of angles per step
        tables, self.rope_id = [], []
        for f in fields:
            t = f["mixer"]["inv_freq"].detach().float().cpu()
            for i, have in enumerate(tables):
                if have.shape == t.shape and torch.equal(have, t):
                    self.rope_id.append(i)
                    break
            else:
                self.rope_id.append(len(tables))
                tables.append(t)

    @classmethod
    def plan(cls, model):
        """A runner for ``model`` or None when some layer has to run part by part."""
        fields = collect_fused_fields(model)
        if fields is None:
            return None
        hd = fields[0]["mixer"]["head_dim"]
        if hd not in (64, 128):
            return None
        for f in fields:
            if f["ffn"]["pair"] not in (64, 128):          # a tile of the gate/up product holds both halves
                return None
        return cls(model, fields)

    def takes(self, step, cache) -> bool:
        # (a decode step of up to 16 sequences comes here too where large layers make this the faster way)
        if not (fuses(step.n_tokens) or (step.all_single and step.n_tokens >= five_launch_from(self.layer_bytes))):
            return False
        for e in self.model.spec.schedule:
            g = cache.kv_groups.get(cache.cache_group.get(e.cache))
            if g is None or g.k.dtype != torch.bfloat16:
                return False
        return True

    def _tables(self, step, view, inv_freq, rope_id):
        """The step's (cos, sin) table and the tokens' cache pages, made once per step, cache group and frequency table."""
        key = ("rope", id(view.page_table), rope_id)
        got = step.scratch.get(key)
        if got is None:
            T = step.n_tokens
            cs = torch.empty(T, self.hd // 2, 2, dtype=torch.float32, device=inv_freq.device)
            tok_page = torch.empty(T, dtype=torch.int32, device=inv_freq.device)
            K.rope_table(view, inv_freq, self.hd // 2, cs, tok_page)
            got = step.scratch[key] = (cs, tok_page)
        return got

    def run(self, h: torch.Tensor, step, cache) -> None:
        """All layers on the residual stream ``h`` [T, H] (float32), in place."""
        self.runs += 1
        T, H, hd = step.n_tokens, self.H, self.hd
        dev, bf = h.device, torch.bfloat16
        sms = sm_count(dev)
        stream = T <= STREAM_TOKENS                    # the kernel that streams the weights takes these few tokens
        schedule = self.model.spec.schedule

        def product(a, w, out, mode, bn, pair=0, **kw):
            if stream:
                K.tc_stream_fused(a, w, out, mode, pair, **kw)
            else:
                K.tc_gemm_fused(a, w, out, mode, bn, **kw)

        def res_tiles(bn):
            return K.tc_stream_n_tiles(H) if stream else K.tc_gemm_n_tiles(H, bn)

        def into_residual(a, w, next_w):
            """h += a·wᵀ, and the next norm's input: (residual ⊙ next_w in bfloat16, the rows' sums of squares)."""
            bn = tile_width(T, H, sms)
            xw = torch.empty(T, H, dtype=bf, device=dev)
            if not stream and K.tc_gemm_splits(T, H, a.shape[1], bn) > 1:
                # few tiles and a long K (the down projection of a few hundred tokens): the kernel that splits K over a
                # cluster has the plain epilogues only, so the norm's input is a small kernel of its own behind it
                ssq = torch.empty(T, 1, dtype=torch.float32, device=dev)
                K.tc_gemm(a, w, h, K.TC_ACCUMULATE, bn)
                K.norm_prepare(h, next_w, xw, ssq)
            else:
                ssq = torch.empty(T, res_tiles(bn), dtype=torch.float32, device=dev)
                product(a, w, h, K.TC_ACCUMULATE, bn, xw=xw, next_w=next_w, ssq_out=ssq)
            return xw, ssq

        xw = torch.empty(T, H, dtype=bf, device=dev)
        ssq = torch.empty(T, 1, dtype=torch.float32, device=dev)
        with phase("attention_norm_ms"):
            K.norm_prepare(h, self.fields[0]["mixer_norm"]["weight"], xw, ssq)
        for i, (e, f) in enumerate(zip(schedule, self.fields)):
            m, ff = f["mixer"], f["ffn"]
            mixer = self.model.layers[e.layer].mixer
            view = cache.view(e.cache, step, True)
            nh, nkv = m["num_heads"], m["num_kv_heads"]
            # ---- QKV, rotation, cache write
            with phase("rotary_table_ms"):
                cs, tok_page = self._tables(step, view, m["inv_freq"], self.rope_id[i])
            q = torch.empty(T, nh * hd, dtype=bf, device=dev)
            n_qkv = m["qkv"].shape[0]
            bn = tile_width(T, n_qkv, sms)
            if bn % hd:
                bn = 256
            with phase("attention_norm+qkv_projection+rotary+kv_append_ms"):
                product(xw, m["qkv"], None, K.TC_QKV_ROPE, bn, row_ssq=ssq, norm_width=H, eps=f["mixer_norm"]["eps"],
                        rope=dict(cs=cs, tok_page=tok_page, positions=step.positions, q_out=q, k_pool=view.k_pool,
                                  v_pool=view.v_pool, nh=nh, nkv=nkv, hd=hd, page_size=view.page_size))
            # ---- attention, then the output projection into the residual, preparing the second norm
            with phase("attention_ms"):
                ctx = mixer.attend(q, step, view)
            with phase("o_projection+attention_residual_ms"):
                xw, ssq = into_residual(ctx, m["o"], f["ffn_norm"]["weight"])
            # ---- gate/up with silu(gate)·up on the normed residual
            act = torch.empty(T, ff["intermediate_size"], dtype=bf, device=dev)
            with phase("mlp_norm+gate_projection+up_projection+activation_multiply_ms"):
                product(xw, ff["gate_up"], act, K.TC_SILU_MUL, 2 * ff["pair"], ff["pair"], row_ssq=ssq, norm_width=H,
                        eps=f["ffn_norm"]["eps"])
            # ---- down projection into the residual, preparing the next layer's first norm
            with phase("down_projection+mlp_residual_ms"):
                if i + 1 < len(self.fields):
                    xw, ssq = into_residual(act, ff["down"], self.fields[i + 1]["mixer_norm"]["weight"])
                elif stream:
                    K.tc_stream(act, ff["down"], h, K.TC_ACCUMULATE)
                else:
                    K.tc_gemm(act, ff["down"], h, K.TC_ACCUMULATE, tile_width(T, H, sms))
